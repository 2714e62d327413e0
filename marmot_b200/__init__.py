"""marmot_b200: sm_100a kernels for marmot's quantized GGUF matmul path behind a C ABI.

The product is the shared library ``libmarmot_cuda.so`` (sources in ``csrc/``, interface in
``include/marmot_cuda.h``).  ``marmot_b200.runtime`` is a thin ctypes binding used by the tests
and the benchmark; it carries no compute of its own and raises if the library is missing.
"""
from .runtime import Context, KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, MarmotCudaError, load_library, row_bytes  # noqa: F401

__all__ = ["Context", "KIND_Q4_K", "KIND_Q6_K", "KIND_Q8_0", "MarmotCudaError", "load_library", "row_bytes"]
