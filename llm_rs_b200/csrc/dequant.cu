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

// Reads the plane layout described at LLMRS_LAYOUT_Q6K_PLANES.
__global__ void dequant_q6k_planes_kernel(const uint8_t *__restrict__ w, float *__restrict__ out,
                                          int K, size_t row_stride, size_t n_elems) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    size_t row = i / (size_t)K;
    int k = (int)(i % (size_t)K);
    int nb = K / QK_K;
    int b = k / QK_K, e = k % QK_K;
    const uint8_t *r = w + row * row_stride;
    const uint8_t *ql = r + (size_t)b * 128;
    const uint8_t *qh = r + (size_t)nb * 128 + (size_t)b * 64;
    const int8_t *sc = (const int8_t *)(r + (size_t)nb * 192 + (size_t)b * 16);
    float d = f16_bits_to_f32(*(const uint16_t *)(r + (size_t)nb * 208 + (size_t)b * 2));
    int h = e / 128, j = e % 128;
    uint32_t lo = (j < 64) ? (ql[h * 64 + j] & 0x0Fu) : (uint32_t)(ql[h * 64 + j - 64] >> 4);
    uint32_t hi = (qh[h * 32 + (j % 32)] >> (2 * (j / 32))) & 3u;
    float q = (float)(int)(lo | (hi << 4));
    out[i] = d * (float)sc[e / 16] * (q - 32.0f);
}

// One thread per source byte of the raw GGUF Q6_K stream.
__global__ void q6k_repack_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ planes,
                                  int nb, size_t row_stride, size_t n_bytes) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_bytes) return;
    size_t blk = i / Q6K_BLOCK_BYTES;
    int o = (int)(i % Q6K_BLOCK_BYTES);
    size_t row = blk / (size_t)nb;
    size_t b = blk % (size_t)nb;
    size_t dst;
    if (o < 128)      dst = b * 128 + o;
    else if (o < 192) dst = (size_t)nb * 128 + b * 64 + (o - 128);
    else if (o < 208) dst = (size_t)nb * 192 + b * 16 + (o - 192);
    else              dst = (size_t)nb * 208 + b * 2 + (o - 208);
    planes[row * row_stride + dst] = raw[i];
}

cudaError_t launch_q6k_repack(const uint8_t *raw, uint8_t *planes, int K, int N, cudaStream_t s) {
    int nb = K / QK_K;
    size_t n_bytes = (size_t)N * nb * Q6K_BLOCK_BYTES;
    if (n_bytes == 0) return cudaSuccess;
    size_t stride = q6k_plane_row_stride(K);
    if (stride != (size_t)nb * Q6K_BLOCK_BYTES) {
        cudaError_t e = cudaMemsetAsync(planes, 0, (size_t)N * stride, s);   // padding bytes
        if (e != cudaSuccess) return e;
    }
    unsigned grid = (unsigned)((n_bytes + 255) / 256);
    q6k_repack_kernel<<<grid, 256, 0, s>>>(raw, planes, nb, stride, n_bytes);
    return cudaGetLastError();
}

cudaError_t launch_dequant(int wdtype, const uint8_t *w, int K, int N, float *out, cudaStream_t s) {
    size_t n = (size_t)K * N;
    if (n == 0) return cudaSuccess;
    unsigned grid = (unsigned)((n + 255) / 256);
    if (wdtype == DT_Q4K) dequant_q4k_kernel<<<grid, 256, 0, s>>>(w, out, n);
    else if (wdtype == DT_Q6K) dequant_q6k_planes_kernel<<<grid, 256, 0, s>>>(w, out, K, q6k_plane_row_stride(K), n);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace llmrs
