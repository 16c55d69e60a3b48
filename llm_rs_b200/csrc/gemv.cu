// Decode matmul (GEMV, a few tokens) for Q4_K and Q6_K weights on the CUDA cores of sm_100a.
//
//   out[s*N + r] = sum_k W[r,k] * x[s*K + k]        (src/backend/mod.rs:29-34)
//
// The kernels replace matvec_q4k_simd / matvec_q6k_simd / gemm_q4k / gemm_q6k of
// the reference (shaders/ops.metal:239-289, 295-344, 357-424, 560-621) and are
// HBM-bound by design: every weight byte is read once with 128-bit loads, and
// the per-weight arithmetic is cut to about two instructions so the fp32 lanes
// keep up with the memory system:
//
//  * A lane owns a 64-weight slice of a row (Q4_K: the 32 quant bytes of one
//    sub-block pair; Q6_K: 16 qh bytes and the two 16-byte ql runs they pair
//    with) and walks R rows over that slice, so the activations it needs are
//    fetched once from shared memory per R rows.
//  * Quant fields are never shifted down or converted: `w & mask` is used as a
//    subnormal float operand (value q * 2^(shift-149)) and the activation copy
//    in shared memory is pre-multiplied by 2^(96-shift) for the position it
//    pairs with.  The accumulators therefore hold sum(q*x) * 2^-53, exactly
//    rounded like an ordinary float dot product.
//  * Block scales are applied once per sub-block, not per weight:
//      Q4_K: sum_sb [ d*sc_sb * sum_j q_j x_j  -  dmin*m_sb * sum_j x_j ]
//      Q6_K: sum_g  [ d*sc_g  * (sum_j q_j x_j - 32 * sum_j x_j) ]
//    with the per-sub-block activation sums computed once per CTA.
//
// Accumulation is float32 throughout; results agree with a float64 evaluation
// of the reference formula to ~1e-6 relative L2.
#include "kernels.h"
#include "llmrs_common.cuh"

namespace llmrs {

constexpr int SLICE = 64;          // weights per lane task
constexpr int SLICE_STRIDE = 68;   // floats per slice in shared memory: 64 activations + 4 sums;
                                   // 68 keeps 128-bit reads of consecutive lanes on distinct banks
constexpr int X_EXP = 96;          // activations are staged as x * 2^(X_EXP - shift)
constexpr float ACC_UNSCALE = 9007199254740992.0f;   // 2^53 = 2^(149 - X_EXP)

__device__ __forceinline__ float load_x(const void *x, size_t idx, int is_bf16) {
    return is_bf16 ? bf16_bits_to_f32(__ldg((const uint16_t *)x + idx)) : __ldg((const float *)x + idx);
}

__device__ __forceinline__ void store_out(void *out, size_t idx, float v, int is_bf16) {
    if (is_bf16) ((__nv_bfloat16 *)out)[idx] = __float2bfloat16_rn(v);
    else ((float *)out)[idx] = v;
}

// Left shift (in bits) of byte k of a 32-bit word when its fields are taken by masking:
// bytes 0..2 stay in place, byte 3 is brought down with one shift.
__device__ __forceinline__ int byte_shift(int k) { return k < 3 ? 8 * k : 0; }

// (small unsigned integer < 2^23) -> float without an I2F: or into 2^23, subtract.
__device__ __forceinline__ float small_uint_to_float(uint32_t v) {
    return __uint_as_float(0x4B000000u | v) - 8388608.0f;
}

// ---------------------------------------------------------------------------------------------
// Q4_K.  Raw GGUF blocks (144 B: f16 d, f16 dmin, 12 B packed 6-bit scales/mins, 128 B nibbles;
// tests/ops.rs:41-59).  Slice tau = 4*b + p is sub-block pair p of block b: quant bytes
// 32p..32p+31, low nibbles = sub-block 2p, high nibbles = sub-block 2p+1.
// Shared memory per token and slice: [0,32) x of sub-block 2p, [32,64) x of sub-block 2p+1 (both
// pre-scaled), [64] sum of the true x over sub-block 2p, [65] over sub-block 2p+1.
// ---------------------------------------------------------------------------------------------
template <int MT, int R, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
gemv_q4k_kernel(const uint8_t *__restrict__ W, const void *__restrict__ X, void *__restrict__ Out,
                int K, int N, int M, int x_bf16, int out_bf16, int kc) {
    extern __shared__ __align__(16) float xs[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.y * MT;
    const int row0 = (blockIdx.x * WARPS + warp) * R;
    const int nb = K / QK_K;
    const size_t row_bytes = (size_t)nb * Q4K_BLOCK_BYTES;
    const int tok_stride = (kc / SLICE) * SLICE_STRIDE;
    const int p = lane & 3;                 // pair index of every slice this lane visits
    const int sel = (p & 1) * 16;           // which 16-bit half of the scale words holds this pair
    const bool upper = p >= 2;              // sub-blocks 4..7 use the split 4+2 bit encoding

    float total[R][MT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) total[r][t] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += kc) {
        const int nsl = min(kc, K - k0) / SLICE;
        if (k0) __syncthreads();
        // ---- stage activations of this K-chunk ----
        for (int s = warp; s < nsl; s += WARPS) {
            const int k = lane & 3;
            const float f_lo = exp2i(X_EXP - byte_shift(k));
            const float f_hi = exp2i(X_EXP - byte_shift(k) - 4);
#pragma unroll
            for (int t = 0; t < MT; t++) {
                const int tok = min(t0 + t, M - 1);
                const size_t base = (size_t)tok * K + k0 + (size_t)s * SLICE;
                float a = load_x(X, base + lane, x_bf16);
                float b = load_x(X, base + 32 + lane, x_bf16);
                float *dst = xs + t * tok_stride + s * SLICE_STRIDE;
                dst[lane] = a * f_lo;
                dst[32 + lane] = b * f_hi;
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    a += __shfl_xor_sync(0xffffffffu, a, o);
                    b += __shfl_xor_sync(0xffffffffu, b, o);
                }
                if (lane == 0) { dst[64] = a; dst[65] = b; }
            }
        }
        __syncthreads();

        // ---- stream the weights ----
        for (int sl = lane; sl < nsl; sl += 32) {
            const int blk = (k0 / SLICE + sl) >> 2;
            uint4 hdr[R], qa[R], qb[R];
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int row = min(row0 + r, N - 1);
                const uint8_t *b = W + (size_t)row * row_bytes + (size_t)blk * Q4K_BLOCK_BYTES;
                hdr[r] = ldg128(b);
                qa[r] = ldg128(b + 16 + 32 * p);
                qb[r] = ldg128(b + 32 + 32 * p);
            }
            float acc_lo[R][MT], acc_hi[R][MT];
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int t = 0; t < MT; t++) { acc_lo[r][t] = 0.0f; acc_hi[r][t] = 0.0f; }

            const float *xsl = xs + sl * SLICE_STRIDE;
#pragma unroll
            for (int wi = 0; wi < 8; wi++) {
                float4 xl[MT], xh[MT];
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    xl[t] = *reinterpret_cast<const float4 *>(xsl + t * tok_stride + 4 * wi);
                    xh[t] = *reinterpret_cast<const float4 *>(xsl + t * tok_stride + 32 + 4 * wi);
                }
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const uint4 &q = wi < 4 ? qa[r] : qb[r];
                    const uint32_t w = (wi & 3) == 0 ? q.x : (wi & 3) == 1 ? q.y : (wi & 3) == 2 ? q.z : q.w;
                    const uint32_t top = w >> 24;
                    const float a0 = field_as_float(w & 0x0000000Fu), b0 = field_as_float(w & 0x000000F0u);
                    const float a1 = field_as_float(w & 0x00000F00u), b1 = field_as_float(w & 0x0000F000u);
                    const float a2 = field_as_float(w & 0x000F0000u), b2 = field_as_float(w & 0x00F00000u);
                    const float a3 = field_as_float(top & 0x0Fu),     b3 = field_as_float(top & 0xF0u);
#pragma unroll
                    for (int t = 0; t < MT; t++) {
                        float lo = acc_lo[r][t], hi = acc_hi[r][t];
                        lo = fmaf(a0, xl[t].x, lo); hi = fmaf(b0, xh[t].x, hi);
                        lo = fmaf(a1, xl[t].y, lo); hi = fmaf(b1, xh[t].y, hi);
                        lo = fmaf(a2, xl[t].z, lo); hi = fmaf(b2, xh[t].z, hi);
                        lo = fmaf(a3, xl[t].w, lo); hi = fmaf(b3, xh[t].w, hi);
                        acc_lo[r][t] = lo; acc_hi[r][t] = hi;
                    }
                }
            }
            // ---- block scales: tests/ops.rs:29-39, two sub-blocks at a time ----
            float2 xsum[MT];
#pragma unroll
            for (int t = 0; t < MT; t++) xsum[t] = *reinterpret_cast<const float2 *>(xsl + t * tok_stride + 64);
#pragma unroll
            for (int r = 0; r < R; r++) {
                const float d = f16_bits_to_f32((uint16_t)(hdr[r].x & 0xFFFFu));
                const float dmin = f16_bits_to_f32((uint16_t)(hdr[r].x >> 16));
                const uint32_t A = (hdr[r].y >> sel) & 0xFFFFu;    // scales[2p'], scales[2p'+1]
                const uint32_t B = (hdr[r].z >> sel) & 0xFFFFu;    // scales[4+2p'], ...
                const uint32_t C = (hdr[r].w >> sel) & 0xFFFFu;    // scales[8+2p'], ...
                const uint32_t scp = upper ? ((C & 0x0F0Fu) | ((A >> 2) & 0x3030u)) : (A & 0x3F3Fu);
                const uint32_t mnp = upper ? (((C >> 4) & 0x0F0Fu) | ((B >> 2) & 0x3030u)) : (B & 0x3F3Fu);
                const float d2 = d * ACC_UNSCALE;
                const float s_lo = d2 * small_uint_to_float(scp & 0xFFu);
                const float s_hi = d2 * small_uint_to_float(scp >> 8);
                const float m_lo = dmin * small_uint_to_float(mnp & 0xFFu);
                const float m_hi = dmin * small_uint_to_float(mnp >> 8);
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    float v = total[r][t];
                    v = fmaf(s_lo, acc_lo[r][t], v);
                    v = fmaf(s_hi, acc_hi[r][t], v);
                    v = fmaf(-m_lo, xsum[t].x, v);
                    v = fmaf(-m_hi, xsum[t].y, v);
                    total[r][t] = v;
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) {
            float v = total[r][t];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && row0 + r < N && t0 + t < M)
                store_out(Out, (size_t)(t0 + t) * N + row0 + r, v, out_bf16);
        }
}

// ---------------------------------------------------------------------------------------------
// Q6_K in the plane layout (LLMRS_LAYOUT_Q6K_PLANES).  Slice tau = 4*b + 2*h + c covers the
// weights 256b + 128h + 32g + 16c + i  (g = 0..3, i = 0..15) of the row: qh bytes 32h+16c+i,
// ql bytes 64h+16c+i (low nibble: g=0, high: g=2) and 64h+32+16c+i (low: g=1, high: g=3);
// each g is one 16-weight scale group (shaders/ops.metal:28-42, 322-334).
// Shared memory per token and slice: [16g+i] pre-scaled x, [64+g] sum of the true x over group g.
// ---------------------------------------------------------------------------------------------
template <int MT, int R, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
gemv_q6k_kernel(const uint8_t *__restrict__ W, const void *__restrict__ X, void *__restrict__ Out,
                int K, int N, int M, int x_bf16, int out_bf16, int kc, size_t row_stride) {
    extern __shared__ __align__(16) float xs[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.y * MT;
    const int row0 = (blockIdx.x * WARPS + warp) * R;
    const int nb = K / QK_K;
    const int tok_stride = (kc / SLICE) * SLICE_STRIDE;
    const int c = lane & 1, h = (lane >> 1) & 1;
    const size_t off_qh = (size_t)nb * 128, off_sc = (size_t)nb * 192, off_d = (size_t)nb * 208;

    float total[R][MT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) total[r][t] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += kc) {
        const int nsl = min(kc, K - k0) / SLICE;
        if (k0) __syncthreads();
        // ---- stage activations: lane holds positions `lane` (g = lane/16) and `lane+32` (g+2) ----
        for (int s = warp; s < nsl; s += WARPS) {
            const int sb = s >> 2, sh = (s >> 1) & 1, sc = s & 1;
            const int i = lane & 15, g = lane >> 4;
            const float f = exp2i(X_EXP - byte_shift(i & 3));
            const size_t e0 = (size_t)k0 + 256 * sb + 128 * sh + 16 * sc + i;
#pragma unroll
            for (int t = 0; t < MT; t++) {
                const int tok = min(t0 + t, M - 1);
                float a = load_x(X, (size_t)tok * K + e0 + 32 * g, x_bf16);
                float b = load_x(X, (size_t)tok * K + e0 + 32 * (g + 2), x_bf16);
                float *dst = xs + t * tok_stride + s * SLICE_STRIDE;
                dst[lane] = a * f;
                dst[32 + lane] = b * f;
#pragma unroll
                for (int o = 8; o; o >>= 1) {
                    a += __shfl_xor_sync(0xffffffffu, a, o);
                    b += __shfl_xor_sync(0xffffffffu, b, o);
                }
                if (i == 0) { dst[64 + g] = a; dst[66 + g] = b; }
            }
        }
        __syncthreads();

        for (int sl = lane; sl < nsl; sl += 32) {
            const int blk = (k0 / SLICE + sl) >> 2;
            uint4 l0[R], l1[R], qh[R];
            uint2 scw[R];
            uint16_t dh[R];
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int row = min(row0 + r, N - 1);
                const uint8_t *b = W + (size_t)row * row_stride;
                const uint8_t *ql = b + (size_t)blk * 128 + 64 * h + 16 * c;
                l0[r] = ldg128(ql);
                l1[r] = ldg128(ql + 32);
                qh[r] = ldg128(b + off_qh + (size_t)blk * 64 + 32 * h + 16 * c);
                scw[r] = __ldg(reinterpret_cast<const uint2 *>(b + off_sc + (size_t)blk * 16 + 8 * h));
                dh[r] = __ldg(reinterpret_cast<const uint16_t *>(b + off_d + (size_t)blk * 2));
            }
            const float *xsl = xs + sl * SLICE_STRIDE;
            float4 xsum[MT];
#pragma unroll
            for (int t = 0; t < MT; t++) xsum[t] = *reinterpret_cast<const float4 *>(xsl + t * tok_stride + 64);

#pragma unroll
            for (int g = 0; g < 4; g++) {
                float acc[R][MT];
#pragma unroll
                for (int r = 0; r < R; r++)
#pragma unroll
                    for (int t = 0; t < MT; t++) acc[r][t] = 0.0f;
#pragma unroll
                for (int wi = 0; wi < 4; wi++) {
                    float4 xv[MT];
#pragma unroll
                    for (int t = 0; t < MT; t++)
                        xv[t] = *reinterpret_cast<const float4 *>(xsl + t * tok_stride + 16 * g + 4 * wi);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        const uint4 &ql4 = (g & 1) ? l1[r] : l0[r];
                        const uint32_t lw = wi == 0 ? ql4.x : wi == 1 ? ql4.y : wi == 2 ? ql4.z : ql4.w;
                        const uint32_t hw = wi == 0 ? qh[r].x : wi == 1 ? qh[r].y : wi == 2 ? qh[r].z : qh[r].w;
                        const uint32_t lo = (g < 2 ? lw : (lw >> 4)) & 0x0F0F0F0Fu;
                        const uint32_t hs = g == 0 ? (hw << 4) : g == 1 ? (hw << 2) : g == 2 ? hw : (hw >> 2);
                        const uint32_t v = lo | (hs & 0x30303030u);          // four 6-bit quants, one per byte
                        const float q0 = field_as_float(v & 0x000000FFu);
                        const float q1 = field_as_float(v & 0x0000FF00u);
                        const float q2 = field_as_float(v & 0x00FF0000u);
                        const float q3 = field_as_float(v >> 24);
#pragma unroll
                        for (int t = 0; t < MT; t++) {
                            float a = acc[r][t];
                            a = fmaf(q0, xv[t].x, a);
                            a = fmaf(q1, xv[t].y, a);
                            a = fmaf(q2, xv[t].z, a);
                            a = fmaf(q3, xv[t].w, a);
                            acc[r][t] = a;
                        }
                    }
                }
                // scale of group g: int8 at scales[8h + 2g + c]
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const uint32_t sw = (g < 2 ? scw[r].x : scw[r].y) ^ 0x80808080u;   // sc + 128 per byte
                    const uint32_t sbyte = (sw >> (8 * (2 * (g & 1) + c))) & 0xFFu;
                    const float scf = small_uint_to_float(sbyte) - 128.0f;
                    const float ds = f16_bits_to_f32(dh[r]) * scf;
                    const float ds2 = ds * ACC_UNSCALE;
                    const float ds32 = ds * -32.0f;
#pragma unroll
                    for (int t = 0; t < MT; t++) {
                        const float xg = g == 0 ? xsum[t].x : g == 1 ? xsum[t].y : g == 2 ? xsum[t].z : xsum[t].w;
                        float v = total[r][t];
                        v = fmaf(ds2, acc[r][t], v);
                        v = fmaf(ds32, xg, v);
                        total[r][t] = v;
                    }
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) {
            float v = total[r][t];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && row0 + r < N && t0 + t < M)
                store_out(Out, (size_t)(t0 + t) * N + row0 + r, v, out_bf16);
        }
}

// ---------------------------------------------------------------------------------------------
// Launch
// ---------------------------------------------------------------------------------------------
namespace {

// Largest K-chunk whose staged activations fit the shared-memory budget for MT tokens.
int chunk_elems(int K, int MT) {
    int cap = MT == 1 ? 16384 : MT == 2 ? 8192 : 4096;
    return K < cap ? K : cap;
}

template <int MT, int R, int WARPS>
cudaError_t launch_one(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                       int K, int N, int M, cudaStream_t s) {
    const int kc = chunk_elems(K, MT);
    const size_t smem = (size_t)MT * (kc / SLICE) * SLICE_STRIDE * sizeof(float);
    dim3 grid((unsigned)((N + R * WARPS - 1) / (R * WARPS)), (unsigned)((M + MT - 1) / MT));
    dim3 block(WARPS * 32);
    cudaError_t e;
    if (wdtype == DT_Q4K) {
        auto kern = gemv_q4k_kernel<MT, R, WARPS>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        kern<<<grid, block, smem, s>>>(w, x, out, K, N, M, x_dtype == DT_BF16, out_dtype == DT_BF16, kc);
    } else {
        auto kern = gemv_q6k_kernel<MT, R, WARPS>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        kern<<<grid, block, smem, s>>>(w, x, out, K, N, M, x_dtype == DT_BF16, out_dtype == DT_BF16, kc,
                                       q6k_plane_row_stride(K));
    }
    return cudaGetLastError();
}

template <int MT>
cudaError_t launch_mt(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                      int K, int N, int M, cudaStream_t s) {
    // Rows per warp trade activation re-reads against CTAs in flight; small N wants more CTAs.
    if (N >= 16384) return launch_one<MT, 4, 8>(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, s);
    if (N >= 2048) return launch_one<MT, 2, 8>(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, s);
    return launch_one<MT, 1, 4>(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, s);
}

}  // namespace

cudaError_t launch_gemv(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                        int K, int N, int M, cudaStream_t s, uint64_t *launches) {
    if (K <= 0 || N <= 0 || M <= 0) return cudaSuccess;
    if (launches) (*launches)++;
    const int mt = M >= 4 ? 4 : M;
    switch (mt) {
        case 1: return launch_mt<1>(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, s);
        case 2: return launch_mt<2>(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, s);
        case 3: return launch_mt<3>(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, s);
        default: return launch_mt<4>(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, s);
    }
}

}  // namespace llmrs
