/* driver_api.c: resolves the CUDA driver interface at first use. */
#include "driver_api.h"

#include <dlfcn.h>
#include <pthread.h>
#include <stdio.h>

static struct ab_driver table;
static const struct ab_driver *resolved;
static pthread_once_t once = PTHREAD_ONCE_INIT;

#define AB_STRING_OF(x) #x
#define AB_SYMBOL_OF(x) AB_STRING_OF(x) /* expands cuda.h's versioning macro before making the string */

static void resolve(void)
{
	void *const library = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
	if (library == NULL) {
		(void)fprintf(stderr, "anemone_b200: no CUDA driver (libcuda.so.1): %s\n", dlerror());
		return;
	}
#define AB_LOOKUP(name)                                                                              \
	*(void **)(&table.name) = dlsym(library, AB_SYMBOL_OF(name));                                \
	if (table.name == NULL) {                                                                    \
		(void)fprintf(stderr, "anemone_b200: the CUDA driver lacks %s\n", AB_SYMBOL_OF(name)); \
		return;                                                                              \
	}
	AB_DRIVER_ENTRIES(AB_LOOKUP)
#undef AB_LOOKUP
	const CUresult result = table.cuInit(0);
	if (result != CUDA_SUCCESS) {
		(void)fprintf(stderr, "anemone_b200: cuInit failed (%d)\n", (int)result);
		return;
	}
	resolved = &table;
}

const struct ab_driver *ab_driver(void)
{
	(void)pthread_once(&once, resolve);
	return resolved;
}
