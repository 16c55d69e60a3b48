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

// Weight e (0..255) of the raw Q4_K block at b.
__device__ __forceinline__ float q4k_block_elem(const uint8_t *b, int e) {
    int sb = e / 32, j = e % 32;
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
    return d * (float)sc * q - dmin * (float)m;
}

// One thread per output element; a warp covers one 32-weight sub-block, so the
// block header and the 32 quant bytes are read once per warp from L1.
__global__ void dequant_q4k_kernel(const uint8_t *__restrict__ w, float *__restrict__ out, size_t n_elems) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    out[i] = q4k_block_elem(w + (i / QK_K) * Q4K_BLOCK_BYTES, (int)(i % QK_K));
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

// Weight k of the row at r (nb blocks) in the slice-major device layout.
__device__ __forceinline__ float q6k_dev_row_elem(const uint8_t *r, int nb, int k) {
    int blk = k / QK_K, e = k % QK_K;
    const uint16_t dbits = (uint16_t)(q6k_dev_byte(r, nb, blk, 208) | (q6k_dev_byte(r, nb, blk, 209) << 8));
    const float d = f16_bits_to_f32(dbits);
    const int sc = (int)(int8_t)q6k_dev_byte(r, nb, blk, 192 + e / 16);
    int h = e / 128, j = e % 128;
    uint32_t lo = (j < 64) ? (q6k_dev_byte(r, nb, blk, h * 64 + j) & 0x0Fu)
                           : (uint32_t)(q6k_dev_byte(r, nb, blk, h * 64 + j - 64) >> 4);
    uint32_t hi = (q6k_dev_byte(r, nb, blk, 128 + h * 32 + (j % 32)) >> (2 * (j / 32))) & 3u;
    float q = (float)(int)(lo | (hi << 4));
    return d * (float)sc * (q - 32.0f);
}

// Reads the slice-major device layout.
__global__ void dequant_q6k_dev_kernel(const uint8_t *__restrict__ w, float *__restrict__ out,
                                       int K, size_t row_stride, size_t n_elems) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    out[i] = q6k_dev_row_elem(w + (i / (size_t)K) * row_stride, K / QK_K, (int)(i % (size_t)K));
}

// Embedding lookup (src/backend/mod.rs:25-27; shaders/ops.metal:917-965): row tokens[s] of the
// table, dequantised, becomes column s of `out` ([dim, seq_len]: element (s, k) at s*dim + k).
// The value is the float32 dequantisation above, rounded once if the output is bf16.  A token id
// outside the table is reported through err_word and reads row 0.
// A thread produces eight consecutive values (one 16-byte bf16 store): a warp covers one
// 256-weight block of one token's row with 8-byte loads of the quants.
template <int QT>
__global__ void __launch_bounds__(256)
embed_kernel(const uint8_t *__restrict__ table, size_t row_stride, int K, uint32_t vocab,
             const uint32_t *__restrict__ tokens, void *__restrict__ out, int out_bf16, uint32_t *err_word) {
    const int s = blockIdx.y;
    const int k0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;          // first of this thread's eight values
    if (k0 >= K) return;
    uint32_t tok = tokens[s];
    if (tok >= vocab) {
        if (err_word && threadIdx.x == 0) atomicCAS(err_word, 0u, (uint32_t)7);     // KERR_TOKEN_RANGE
        tok = 0;
    }
    const uint8_t *row = table + (size_t)tok * row_stride;
    const int blk = k0 / QK_K, e0 = k0 % QK_K;
    float v[8];
    if (QT == 0) {
        // tests/ops.rs:29-59: sub-block sb, quant bytes (sb/2)*32 + j, low nibble for even sb
        const uint8_t *b = row + (size_t)blk * Q4K_BLOCK_BYTES;
        const int sb = e0 / 32, j0 = e0 % 32;
        const float d = f16_bits_to_f32(*(const uint16_t *)(b));
        const float dmin = f16_bits_to_f32(*(const uint16_t *)(b + 2));
        const uint8_t *sc8 = b + 4;
        uint32_t sc, m;
        if (sb < 4) {
            sc = sc8[sb] & 63u;
            m = sc8[sb + 4] & 63u;
        } else {
            sc = (sc8[sb + 4] & 0x0Fu) | ((uint32_t)(sc8[sb - 4] >> 6) << 4);
            m = (sc8[sb + 4] >> 4) | ((uint32_t)(sc8[sb] >> 6) << 4);
        }
        const uint2 q8 = *reinterpret_cast<const uint2 *>(b + 16 + (sb / 2) * 32 + j0);
        const uint32_t w[2] = {q8.x, q8.y};
        const float ds = d * (float)sc, dm = dmin * (float)m;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t byte = (w[i / 4] >> (8 * (i % 4))) & 0xFFu;
            v[i] = ds * (float)((sb & 1) ? (byte >> 4) : (byte & 0x0Fu)) - dm;
        }
    } else {
        // slice-major device layout (kernels.h): element 128h + 32g + 16c + i of the block lives in slice
        // 4b + 2h + c: low nibbles in ql run (g & 1), low half for g < 2; bits 2g, 2g+1 of qh byte i
        const int nb = K / QK_K, ci = blk / 16, bl = blk % 16;
        const int nbc = min(16, nb - 16 * ci);
        const uint8_t *chunk = row + (size_t)3360 * ci;
        const int h = e0 / 128, g = (e0 % 128) / 32, c = (e0 % 32) / 16, i0 = e0 % 16;      // i0 is 0 or 8
        const uint8_t *sl = chunk + 48 * (4 * bl + 2 * h + c);
        const uint2 l8 = *reinterpret_cast<const uint2 *>(sl + 16 * (g & 1) + i0);
        const uint2 h8 = *reinterpret_cast<const uint2 *>(sl + 32 + i0);
        const int sc = (int)(int8_t)chunk[192 * nbc + 16 * bl + 8 * h + 2 * g + c];
        const float d = f16_bits_to_f32(*(const uint16_t *)(chunk + 208 * nbc + 2 * bl));
        const uint32_t lw[2] = {l8.x, l8.y}, hw[2] = {h8.x, h8.y};
        const float dsc = d * (float)sc;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t lb = (lw[i / 4] >> (8 * (i % 4))) & 0xFFu, hb = (hw[i / 4] >> (8 * (i % 4))) & 0xFFu;
            const uint32_t lo = g < 2 ? (lb & 0x0Fu) : (lb >> 4);
            const int q = (int)(lo | (((hb >> (2 * g)) & 3u) << 4));
            v[i] = dsc * (float)(q - 32);
        }
    }
    const size_t o = (size_t)s * K + k0;
    if (out_bf16) {
        uint4 pk;
        uint32_t *pw = reinterpret_cast<uint32_t *>(&pk);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            pw[i] = *reinterpret_cast<const uint32_t *>(&two);
        }
        *reinterpret_cast<uint4 *>((__nv_bfloat16 *)out + o) = pk;
    } else {
        float4 *dst = reinterpret_cast<float4 *>((float *)out + o);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
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

// silu(g) * u, the element-wise tail of the feed-forward front where it is not fused into the
// matmul (shaders/ops.metal:762-793, there two kernels with a bf16 rounding between them).
__global__ void silu_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, void *__restrict__ out,
                                int out_bf16, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float a = g[i];
    const float v = a / (1.0f + expf(-a)) * u[i];
    if (out_bf16) ((__nv_bfloat16 *)out)[i] = __float2bfloat16_rn(v);
    else ((float *)out)[i] = v;
}

cudaError_t launch_silu_mul(const float *gate, const float *up, void *out, int out_dtype, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate, up, out, out_dtype == DT_BF16, n);
    return cudaGetLastError();
}

cudaError_t launch_embed(int wdtype, const uint8_t *table, int K, uint32_t vocab, const uint32_t *dev_tokens,
                         int n_tokens, void *out, int out_dtype, uint32_t *err_word, cudaStream_t s) {
    if (n_tokens <= 0 || K <= 0) return cudaSuccess;
    const dim3 grid((unsigned)((K / 8 + 255) / 256), (unsigned)n_tokens);      // eight values per thread
    const int bf = out_dtype == DT_BF16;
    if (wdtype == DT_Q4K)
        embed_kernel<0><<<grid, 256, 0, s>>>(table, (size_t)(K / QK_K) * Q4K_BLOCK_BYTES, K, vocab, dev_tokens, out, bf, err_word);
    else if (wdtype == DT_Q6K)
        embed_kernel<1><<<grid, 256, 0, s>>>(table, q6k_row_stride(K), K, vocab, dev_tokens, out, bf, err_word);
    else
        return cudaErrorInvalidValue;
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
