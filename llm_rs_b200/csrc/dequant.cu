// Dequantisation of Q4_K / Q6_K weights to float32 and the Q6_K upload re-layout.
//
// The float32 values are the ones the reference's CPU code forms
// (Q4_K: tests/ops.rs:41-59, `d*sc*q - dmin*m`; Q6_K: shaders/ops.metal:322-334,
// `d*sc*(q-32)`).  d*sc, d*sc*q and dmin*m are exact in binary32 (11+6+4 and 11+6
// significant bits), so the single rounding of the final subtraction is the same
// whether or not the compiler contracts it into an fma; d*sc*(q-32) is exact.
#include "kernels.h"
#include "llmrs_common.cuh"

namespace llmrs {

// One thread per output element; a warp covers one 32-weight sub-block, so the
// block header and the 32 quant bytes are read once per warp from L1.
__global__ void dequant_q4k_kernel(const uint8_t *__restrict__ w, float *__restrict__ out, size_t n_elems) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    size_t blk = i / QK_K;
    int e = (int)(i % QK_K);
    int sb = e / 32, j = e % 32;
    const uint8_t *b = w + blk * Q4K_BLOCK_BYTES;
    float d = f16_bits_to_f32(*(const uint16_t *)(b));
    float dmin = f16_bits_to_f32(*(const uint16_t *)(b + 2));
    const uint8_t *sc8 = b + 4;
    uint32_t sc, m;
    if (sb < 4) {
        sc = sc8[sb] & 63u;
        m = sc8[sb + 4] & 63u;
    } else {
        sc = (sc8[sb + 4] & 0x0Fu) | ((uint32_t)(sc8[sb - 4] >> 6) << 4);
        m = (sc8[sb + 4] >> 4) | ((uint32_t)(sc8[sb] >> 6) << 4);
    }
    uint8_t packed = b[16 + (sb / 2) * 32 + j];
    float q = (float)((sb & 1) ? (packed >> 4) : (packed & 0x0F));
    out[i] = d * (float)sc * q - dmin * (float)m;
}

// Position of source byte `o` (0..209) of block `b` inside a chunk of `nbc` blocks in the
// slice-major layout described in kernels.h.
__device__ __forceinline__ size_t q6k_chunk_offset(int nbc, int b, int o) {
    if (o < 128) {                      // ql[o]: half h, 32-byte run u (0 = low groups, 1 = +32), column c
        const int h = o >> 6, u = (o >> 5) & 1, c = (o >> 4) & 1, i = o & 15;
        return (size_t)48 * (4 * b + 2 * h + c) + 16 * u + i;
    }
    if (o < 192) {                      // qh[o-128]
        const int q = o - 128, h = q >> 5, c = (q >> 4) & 1, i = q & 15;
        return (size_t)48 * (4 * b + 2 * h + c) + 32 + i;
    }
    if (o < 208) return (size_t)192 * nbc + 16 * b + (o - 192);
    return (size_t)208 * nbc + 2 * b + (o - 208);
}

__device__ __forceinline__ uint8_t q6k_dev_byte(const uint8_t *row, int nb, int blk, int o) {
    const int ci = blk / 16, b = blk % 16;
    const int nbc = min(16, nb - 16 * ci);
    return row[(size_t)3360 * ci + q6k_chunk_offset(nbc, b, o)];
}

// Reads the slice-major device layout.
__global__ void dequant_q6k_dev_kernel(const uint8_t *__restrict__ w, float *__restrict__ out,
                                       int K, size_t row_stride, size_t n_elems) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    size_t row = i / (size_t)K;
    int k = (int)(i % (size_t)K);
    int nb = K / QK_K;
    int blk = k / QK_K, e = k % QK_K;
    const uint8_t *r = w + row * row_stride;
    const uint16_t dbits = (uint16_t)(q6k_dev_byte(r, nb, blk, 208) | (q6k_dev_byte(r, nb, blk, 209) << 8));
    const float d = f16_bits_to_f32(dbits);
    const int sc = (int)(int8_t)q6k_dev_byte(r, nb, blk, 192 + e / 16);
    int h = e / 128, j = e % 128;
    uint32_t lo = (j < 64) ? (q6k_dev_byte(r, nb, blk, h * 64 + j) & 0x0Fu)
                           : (uint32_t)(q6k_dev_byte(r, nb, blk, h * 64 + j - 64) >> 4);
    uint32_t hi = (q6k_dev_byte(r, nb, blk, 128 + h * 32 + (j % 32)) >> (2 * (j / 32))) & 3u;
    float q = (float)(int)(lo | (hi << 4));
    out[i] = d * (float)sc * (q - 32.0f);
}

// One thread per source byte of the raw GGUF Q6_K stream.
__global__ void q6k_repack_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ dev,
                                  int nb, size_t row_stride, size_t n_bytes) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_bytes) return;
    size_t blk = i / Q6K_BLOCK_BYTES;
    int o = (int)(i % Q6K_BLOCK_BYTES);
    size_t row = blk / (size_t)nb;
    int b_in_row = (int)(blk % (size_t)nb);
    const int ci = b_in_row / 16, b = b_in_row % 16;
    const int nbc = min(16, nb - 16 * ci);
    dev[row * row_stride + (size_t)3360 * ci + q6k_chunk_offset(nbc, b, o)] = raw[i];
}

cudaError_t launch_q6k_repack(const uint8_t *raw, uint8_t *dev, int K, int N, cudaStream_t s) {
    int nb = K / QK_K;
    size_t n_bytes = (size_t)N * nb * Q6K_BLOCK_BYTES;
    if (n_bytes == 0) return cudaSuccess;
    size_t stride = q6k_row_stride(K);
    if (stride != (size_t)nb * Q6K_BLOCK_BYTES) {
        cudaError_t e = cudaMemsetAsync(dev, 0, weight_device_bytes(DT_Q6K, K, N), s);   // padding bytes
        if (e != cudaSuccess) return e;
    }
    unsigned grid = (unsigned)((n_bytes + 255) / 256);
    q6k_repack_kernel<<<grid, 256, 0, s>>>(raw, dev, nb, stride, n_bytes);
    return cudaGetLastError();
}

cudaError_t launch_dequant(int wdtype, const uint8_t *w, int K, int N, float *out, cudaStream_t s) {
    size_t n = (size_t)K * N;
    if (n == 0) return cudaSuccess;
    unsigned grid = (unsigned)((n + 255) / 256);
    if (wdtype == DT_Q4K) dequant_q4k_kernel<<<grid, 256, 0, s>>>(w, out, n);
    else if (wdtype == DT_Q6K) dequant_q6k_dev_kernel<<<grid, 256, 0, s>>>(w, out, K, q6k_row_stride(K), n);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace llmrs
