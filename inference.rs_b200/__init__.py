"""B200-native GGUF quantized-weight matmul (Q8_0 / Q4_K / Q6_K): hand-written sm_100a CUDA kernels behind
the reference's kernel-library C ABI, with a thin Python harness for tests and benchmarks.

The compute path is the shared library ``lib/sm100a/libinferencequant_b200.so``; there is no CPU fallback:
every operation raises if the library is missing.
"""
from . import kernel_library  # noqa: F401
from .kernel_library import KernelLibraryError, library  # noqa: F401
from .dtypes import GgmlDType  # noqa: F401
from .qmatmul import GgufMatMul, QMatMul, QTensor  # noqa: F401
from . import gguf_file  # noqa: F401
