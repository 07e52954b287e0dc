"""anemone_b200: B200-native (sm_100a) implementation of Anemone's quantized MoE expert-layer hot path.

The product is the C-ABI library anemone_b200/lib/libanemone_b200.so (C11 host code over the CUDA driver API plus
hand-written sm_100a kernels embedded as cubins). This package holds its sources (csrc/), the build step (build.py)
and a thin ctypes binding used by the tests and the benchmark. There is no CPU fallback: loading fails loudly when the
library is missing, and every compute call fails loudly without a CUDA device.
"""
