// Internal launchers shared between the kernel translation units and the C ABI.
// Everything here is host-callable C++; kernels live in the .cu files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace llmrs {

constexpr int QK_K = 256;            // weights per K-quant block (src/tensor/mod.rs:43)
constexpr int Q4K_BLOCK_BYTES = 144; // src/tensor/mod.rs:71
constexpr int Q6K_BLOCK_BYTES = 210; // src/tensor/mod.rs:73

// GGUF dtype ids (src/tensor/mod.rs:3-33); same values as enum llmrs_dtype.
constexpr int DT_F32 = 0, DT_Q4K = 12, DT_Q6K = 14, DT_BF16 = 30;

// Byte distance between consecutive rows of a Q6_K weight in the plane layout.
inline size_t q6k_plane_row_stride(int K) {
    size_t nb = (size_t)K / QK_K;
    return (nb * Q6K_BLOCK_BYTES + 15) / 16 * 16;
}

// Device bytes a [K, N] weight occupies in the layout the kernels read.
inline size_t weight_device_bytes(int dtype, int K, int N) {
    if (dtype == DT_Q4K) return (size_t)N * (K / QK_K) * Q4K_BLOCK_BYTES;
    if (dtype == DT_Q6K) return (size_t)N * q6k_plane_row_stride(K);
    return 0;
}

// Raw GGUF Q6_K rows -> plane layout (one-off, at upload).
cudaError_t launch_q6k_repack(const uint8_t *raw, uint8_t *planes, int K, int N, cudaStream_t s);

// Weight -> float32 [N, K], bit-exact with the reference's CPU dequantisation.
cudaError_t launch_dequant(int wdtype, const uint8_t *w, int K, int N, float *out, cudaStream_t s);

// Decode matmul on CUDA cores, float32 accumulate; any M (tokens are processed in tiles of <= 4).
// x_dtype / out_dtype are DT_F32 or DT_BF16.  *launches is incremented per kernel launched.
cudaError_t launch_gemv(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                        int K, int N, int M, cudaStream_t s, uint64_t *launches);

}  // namespace llmrs
