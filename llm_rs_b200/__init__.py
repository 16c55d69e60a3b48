"""B200-native (sm_100a) backend for llm-rs's Q4_K / Q6_K dequantize-matmul.

`CudaBackend` mirrors the reference's `Backend` trait for the matmul path and calls the
hand-written CUDA kernels through the C ABI in include/llmrs_cuda.h.
"""
from .backend import BackendError, CudaBackend, CudaBuffer, DType, TensorView, load_library  # noqa: F401
