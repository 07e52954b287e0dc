/*
 * driver_api.h: the CUDA driver entry points the backend uses, resolved from libcuda.so.1 at first use so that the
 * library itself links against nothing but libc, libm, libdl and libpthread. Private to csrc/host.
 */
#ifndef AB_DRIVER_API_H
#define AB_DRIVER_API_H

#include <cuda.h>

/* X(name): name is the cuda.h identifier, which cuda.h may map to a versioned symbol (cuMemAlloc -> cuMemAlloc_v2);
 * the table member keeps the plain identifier's type, the lookup uses the mapped symbol's spelling. */
#define AB_DRIVER_ENTRIES(X)      \
	X(cuInit)                 \
	X(cuGetErrorString)       \
	X(cuDeviceGetCount)       \
	X(cuDeviceGet)            \
	X(cuDeviceGetName)        \
	X(cuDeviceGetAttribute)   \
	X(cuDeviceTotalMem)       \
	X(cuDeviceGetPCIBusId)    \
	X(cuDevicePrimaryCtxRetain) \
	X(cuDevicePrimaryCtxRelease) \
	X(cuCtxPushCurrent)       \
	X(cuCtxPopCurrent)        \
	X(cuMemGetInfo)           \
	X(cuMemAlloc)             \
	X(cuMemFree)              \
	X(cuMemHostAlloc)         \
	X(cuMemFreeHost)          \
	X(cuMemcpyHtoDAsync)      \
	X(cuMemcpyDtoHAsync)      \
	X(cuMemcpyHtoD)           \
	X(cuMemsetD8Async)        \
	X(cuStreamCreate)         \
	X(cuStreamDestroy)        \
	X(cuStreamSynchronize)    \
	X(cuStreamQuery)          \
	X(cuStreamWaitEvent)      \
	X(cuEventCreate)          \
	X(cuEventDestroy)         \
	X(cuEventRecord)          \
	X(cuEventQuery)           \
	X(cuEventElapsedTime)     \
	X(cuModuleLoadData)       \
	X(cuModuleUnload)         \
	X(cuModuleGetFunction)    \
	X(cuModuleGetGlobal)      \
	X(cuMemcpyDtoH)           \
	X(cuFuncGetParamInfo)     \
	X(cuFuncGetAttribute)     \
	X(cuFuncSetAttribute)     \
	X(cuLaunchKernel)         \
	X(cuLaunchKernelEx)       \
	X(cuStreamBeginCapture)   \
	X(cuStreamEndCapture)     \
	X(cuGraphInstantiateWithFlags) \
	X(cuGraphLaunch)          \
	X(cuGraphDestroy)         \
	X(cuGraphExecDestroy)     \
	X(cuGraphGetNodes)        \
	X(cuGraphCreate)          \
	X(cuGraphAddKernelNode)   \
	X(cuGraphAddMemcpyNode)   \
	X(cuMemcpyDtoDAsync)      \
	X(cuMemGetAddressRange)   \
	X(cuDeviceCanAccessPeer)  \
	X(cuCtxEnablePeerAccess)  \
	X(cuIpcGetMemHandle)      \
	X(cuIpcOpenMemHandle)     \
	X(cuIpcCloseMemHandle)

struct ab_driver {
#define AB_MEMBER(name) __typeof__(&name) name;
	AB_DRIVER_ENTRIES(AB_MEMBER)
#undef AB_MEMBER
};

/* The table, or NULL where libcuda.so.1 or one of the entries is missing or cuInit fails (one error line, once). */
const struct ab_driver *ab_driver(void);

#endif
