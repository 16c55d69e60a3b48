// Prefill matmul (GEMM) for Q4_K / Q6_K weights on the 5th-generation tensor cores of sm_100a.
//
//   Out[M, N] = X[M, K] . W[N, K]^T        (src/backend/mod.rs:29-34; M = seq_len >= 5 here)
//
// Replaces gemm_q4k_pipe / gemm_q6k of the reference (shaders/ops.metal:456-558, 560-621), which
// re-dequantise the weights for every 16 (or 4) tokens.  Here a CTA owns 128 weight rows and up
// to 256 tokens and walks K in stages of 128:
//
//   (persistent: one CTA per SM walks the tiles; 14 warps)
//   warps 0-7  dequantise the step's 128 x 64 weight tile straight from global memory (L2) to
//              f16 and store it into TENSOR MEMORY (tcgen05.st; thread = weight row = TMEM lane),
//              where the MMA reads it as its A operand.  Keeping the weights out of shared
//              memory matters: with both operands in shared memory the operand reads plus the
//              tile writes need ~180 B/clk of a 128 B/clk shared memory and the tensor pipe
//              measured 42 % busy.
//   warp  8    one lane issues the TMA tensor copy of the step's tokens x 64 f16 activation tile
//              (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill past the last token).
//   warp  9    allocates TMEM; one lane issues tcgen05.mma (kind::f16, f16 x f16 -> fp32,
//              M=128, N=tokens, K=16, four per step) with the accumulator in TMEM, and
//              tcgen05.commit to hand shared-memory stages back and to publish the accumulator.
//   warps 10-13 epilogue: tcgen05.ld -> token scale -> global, overlapping the next tile's K loop
//              (the accumulator is double-buffered up to 128 tokens per tile).
//
// Weights are the UMMA "A" operand (rows = TMEM lanes), tokens the "B" operand (columns), so one
// dequantised tile feeds up to 256 tokens.  Both operands are f16, not bf16: with bf16 x bf16 the
// two 8-bit roundings alone measure 2.3e-3 relative L2 on N(0,1) data, above the 2e-3 this path
// is held to; f16's 11-bit significand gives 2.8e-4 at the same tensor-core rate.  Weight values
// are RN_f16 of the exact float32 dequantisation (tests/ops.rs:41-59; shaders/ops.metal:322-334;
// clamped at +-65504, K-quant weights of real models are < 1e2), activations are scaled per
// token by a power of two before RN_f16 (activations_to_f16_kernel), products are exact and
// accumulation is fp32 in the tensor core.
// Up to 64 tokens a two-term variant (GemmCfg<TN, true>) carries weights and activations as hi + lo
// f16 pairs and reaches the decode kernel's tolerance class (1e-4) at about twice the time.
// Every wait is bounded; a wait that gives up reports a KernelError and the CTA still releases
// its TMEM before it exits.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "kernels.h"
#include "llmrs_common.cuh"
#include "pipeline.cuh"
#include "tensor_map.h"
#include "umma.cuh"

namespace llmrs {

namespace {


// Work split of the eight dequantising warps: warp w owns TMEM lanes 32*(w%4).. (a hardware rule:
// a warp reaches only its own lane quarter), thread = weight row; group g = w/4 produces the
// stages of parity g, i.e. half g (128 weights) of every 256-weight block of its row.  The two
// groups run a stage apart, so the store/barrier latency of one hides behind the arithmetic of
// the other.

// Q4_K half-block g: pairs 2g and 2g+1, each 32 quant bytes = sub-blocks 2p (low nibbles) and
// 2p+1 (high nibbles) (tests/ops.rs:29-59).
struct RawQ4 {
    uint4 hdr;      // f16 d, f16 dmin, 12 packed scale bytes
    uint4 q[4];     // quant bytes of pair 2g (q[0], q[1]) and pair 2g+1 (q[2], q[3])
};
__device__ __forceinline__ RawQ4 load_raw_q4k(const uint8_t *row_ptr, int b, int g) {
    const uint8_t *blk = row_ptr + (size_t)b * Q4K_BLOCK_BYTES;
    RawQ4 r;
    r.hdr = ldg128_pinned(blk);
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = ldg128_pinned(blk + 16 + 64 * g + 16 * i);
    return r;
}
// The block's eight 6-bit scales and mins as bytes: sc[0..3], sc[4..7], mn[0..3], mn[4..7]
// (tests/ops.rs:29-39, four sub-blocks per logic op), and (d, d/16), (-dmin, -dmin) as f16x2.
struct ScalesQ4 {
    uint32_t sc[2], mn[2];
    uint32_t d_pair, dmin_pair;
};
__device__ __forceinline__ ScalesQ4 unpack_scales_q4k(const uint4 &hdr) {
    ScalesQ4 s;
    s.sc[0] = hdr.y & 0x3F3F3F3Fu;
    s.mn[0] = hdr.z & 0x3F3F3F3Fu;
    s.sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    s.mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    const uint32_t d = hdr.x & 0xFFFFu, dmin = hdr.x >> 16;
    // high nibbles are used in place (16*q), so their scale carries 1/16 (exact unless d is subnormal)
    s.d_pair = d | (h2_mul(d, 0x2C00u) << 16);                    // (d, d * 2^-4)
    s.dmin_pair = (dmin ^ 0x8000u) * 0x00010001u;                 // (-dmin, -dmin)
    return s;
}
// One pair (64 weights) -> 32 TMEM columns at a_taddr: sub-block 2p in columns 0..15, 2p+1 in 16..31.
// scw / mnw hold the pair's two scale bytes and two min bytes in their low 16 bits.
__device__ __forceinline__ void dequant_q4k_pair(const uint4 &qa, const uint4 &qb, uint32_t scw, uint32_t mnw,
                                                 const ScalesQ4 &sq, uint32_t a_taddr) {
    const uint32_t sc2 = h2_sub(magic_lo(scw), H2_1024);          // (sc_lo, sc_hi) exact
    const uint32_t mn2 = h2_sub(magic_lo(mnw), H2_1024);
    const uint32_t ds2 = h2_mul(sc2, sq.d_pair);                  // (d*sc_lo, d*sc_hi/16), rounded to f16
    const uint32_t dm2 = h2_mul(mn2, sq.dmin_pair);               // (-dmin*m_lo, -dmin*m_hi)
    const uint32_t s_lo = h2_bcast_lo(ds2), s_hi = h2_bcast_hi(ds2);
    const uint32_t m_lo = h2_bcast_lo(dm2), m_hi = h2_bcast_hi(dm2);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    uint32_t lo[16], hi[16];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint32_t l4 = w[j] & 0x0F0F0F0Fu, h4 = w[j] & 0xF0F0F0F0u;
        lo[2 * j] = h2_fma(h2_sub(magic_lo(l4), H2_1024), s_lo, m_lo);
        lo[2 * j + 1] = h2_fma(h2_sub(magic_hi(l4), H2_1024), s_lo, m_lo);
        hi[2 * j] = h2_fma(h2_sub(magic_lo(h4), H2_1024), s_hi, m_hi);
        hi[2 * j + 1] = h2_fma(h2_sub(magic_hi(h4), H2_1024), s_hi, m_hi);
    }
    tmem_st16(a_taddr, lo);
    tmem_st16(a_taddr + 16, hi);
}
// Half-block G (template: the scale bytes are picked at compile time) -> 64 TMEM columns.
template <int G>
__device__ __forceinline__ void dequant_q4k_half(const RawQ4 &raw, const ScalesQ4 &sq, uint32_t a_taddr) {
    // sub-blocks 4G..4G+3 are bytes 0..3 of word G of the unpacked scales
    const uint32_t scw = sq.sc[G], mnw = sq.mn[G];
    dequant_q4k_pair(raw.q[0], raw.q[1], scw, mnw, sq, a_taddr);
    dequant_q4k_pair(raw.q[2], raw.q[3], scw >> 16, mnw >> 16, sq, a_taddr + 32);
}

// Q6_K half h of a block in the slice-major device layout (kernels.h): slices (h, c = 0, 1), each
// ql[64h+16c..+16) | ql[64h+32+16c..+16) | qh[32h+16c..+16).  Weight 128h + 32g + 16c + i has its
// low nibble in ql run (g & 1), low half for g < 2 and high half for g >= 2, and bits 2g..2g+1 of
// qh; group scale scales[8h + 2g + c] (shaders/ops.metal:28-42, 322-334).
struct RawQ6 {
    uint4 ql[2][2];   // [c][run]
    uint4 qh[2];      // [c]
    uint2 sc;         // int8 scales[8h .. 8h+8)
    uint32_t d;       // f16 bits
};
__device__ __forceinline__ RawQ6 load_raw_q6k(const uint8_t *row_ptr, int nb, int b, int h) {
    const int ci = b >> 4, bl = b & 15;
    const int nbc = min(16, nb - 16 * ci);
    const uint8_t *chunk = row_ptr + (size_t)3360 * ci;
    RawQ6 r;
    // slices (h, 0) and (h, 1) are 96 contiguous bytes at a multiple of 32: three whole sectors
    const uint8_t *sp = chunk + 48 * (4 * bl + 2 * h);
    ldg256_stream(sp, r.ql[0][0], r.ql[0][1]);
    ldg256_stream(sp + 32, r.qh[0], r.ql[1][0]);
    ldg256_stream(sp + 64, r.ql[1][1], r.qh[1]);
    r.sc = ldg64_pinned(chunk + 192 * nbc + 16 * bl + 8 * h);
    r.d = ldg16_pinned(chunk + 208 * nbc + 2 * bl);
    return r;
}
// Half-block -> 64 TMEM columns: K-local position 32g + 16c + i -> column 16g + 8c + i/2.
__device__ __forceinline__ void dequant_q6k_half(const RawQ6 &raw, uint32_t a_taddr) {
    const uint32_t d2 = raw.d * 0x00010001u;
    // (sc + 128) as bytes -> f16 pairs -> minus 128 -> times d: scale pairs (g, c=0), (g, c=1)
    const uint32_t s01 = raw.sc.x ^ 0x80808080u, s23 = raw.sc.y ^ 0x80808080u;
    const uint32_t ds[4] = {h2_mul(h2_sub(magic_lo(s01), 0x64806480u), d2), h2_mul(h2_sub(magic_hi(s01), 0x64806480u), d2),
                            h2_mul(h2_sub(magic_lo(s23), 0x64806480u), d2), h2_mul(h2_sub(magic_hi(s23), 0x64806480u), d2)};
    uint32_t o[4][16];                            // [g][8c + 2i + {0,1}]
#pragma unroll
    for (int c = 0; c < 2; c++) {
        const uint4 q0 = raw.ql[c][0], q1 = raw.ql[c][1], qh = raw.qh[c];
        const uint32_t l0[4] = {q0.x, q0.y, q0.z, q0.w}, l1[4] = {q1.x, q1.y, q1.z, q1.w};
        const uint32_t hw[4] = {qh.x, qh.y, qh.z, qh.w};
        uint32_t dsc[4];
#pragma unroll
        for (int g = 0; g < 4; g++) dsc[g] = c ? h2_bcast_hi(ds[g]) : h2_bcast_lo(ds[g]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // four bytes of 6-bit quants for each of the four groups, 11 logic ops for 16 weights:
            // qA keeps the g=0 bits at 0-1 and the g=2 bits at 4-5 of every qh byte, qB likewise g=1 / g=3
            const uint32_t qA = hw[i] & 0x33333333u;
            const uint32_t qB = (hw[i] >> 2) & 0x33333333u;
            const uint32_t v[4] = {(l0[i] & 0x0F0F0F0Fu) | ((qA << 4) & 0xF0F0F0F0u),
                                   (l1[i] & 0x0F0F0F0Fu) | ((qB << 4) & 0xF0F0F0F0u),
                                   ((l0[i] >> 4) & 0x0F0F0F0Fu) | (qA & 0xF0F0F0F0u),
                                   ((l1[i] >> 4) & 0x0F0F0F0Fu) | (qB & 0xF0F0F0F0u)};
#pragma unroll
            for (int g = 0; g < 4; g++) {
                o[g][8 * c + 2 * i] = h2_mul(h2_sub(magic_lo(v[g]), H2_1056), dsc[g]);      // (q - 32) * d*sc
                o[g][8 * c + 2 * i + 1] = h2_mul(h2_sub(magic_hi(v[g]), H2_1056), dsc[g]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < 4; g++) tmem_st16(a_taddr + 16 * g, o[g]);
}

// ---- two-term dequantisation: exact float32 weight -> (hi, lo) f16 pair ---------------------------
// The float32 value is the one llmrs_cuda_dequantize writes (d*sc*q - dmin*m and d*sc*(q-32): exact
// products, one rounding); hi = RN_f16(w), lo = RN_f16(w - hi) (the difference is exact in float32).
__device__ __forceinline__ void split_pair(float w0, float w1, uint32_t &hi, uint32_t &lo) {
    hi = pack_w(w0, w1);
    const float2 back = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
    lo = pack_w(w0 - back.x, w1 - back.y);
}
__device__ __forceinline__ float f16_bits_to_f32(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }
// (small unsigned integer < 2^23) -> float without a conversion instruction.
__device__ __forceinline__ float u_to_f(uint32_t v) { return __uint_as_float(0x4B000000u | v) - 8388608.0f; }

// Q4_K half-block G of a row -> 64 hi columns at a_taddr and 64 lo columns at a_taddr + 64.
template <int G>
__device__ __forceinline__ void dequant_q4k_half_split(const RawQ4 &raw, uint32_t a_taddr) {
    const uint4 &hdr = raw.hdr;
    const float d = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu)), dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
    // the eight 6-bit scales and mins as bytes (tests/ops.rs:29-39)
    const uint32_t sc_w = G == 0 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u));
    const uint32_t mn_w = G == 0 ? (hdr.z & 0x3F3F3F3Fu) : (((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u));
#pragma unroll
    for (int sl = 0; sl < 4; sl++) {                     // sub-block 4G + sl: pair sl / 2, low nibbles for even sl
        const float ds = d * u_to_f((sc_w >> (8 * sl)) & 0xFFu), dm = dmin * u_to_f((mn_w >> (8 * sl)) & 0xFFu);
        const uint4 qa = raw.q[2 * (sl >> 1)], qb = raw.q[2 * (sl >> 1) + 1];
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t nib = (sl & 1) ? ((w[j] >> 4) & 0x0F0F0F0Fu) : (w[j] & 0x0F0F0F0Fu);
            float f[4];
#pragma unroll
            for (int e = 0; e < 4; e++) f[e] = fmaf(ds, byte_to_float(nib, e), -dm);
            split_pair(f[0], f[1], hi[2 * j], lo[2 * j]);
            split_pair(f[2], f[3], hi[2 * j + 1], lo[2 * j + 1]);
        }
        tmem_st16(a_taddr + 16 * sl, hi);
        tmem_st16(a_taddr + 64 + 16 * sl, lo);
    }
}

// Q6_K half-block (slice-major layout, see dequant_q6k_half) -> 64 hi columns and 64 lo columns,
// in packed f16 arithmetic.  w = s * q with s = d * sc (float32, exact, <= 18 bits) and q = quant - 32.
// Per scale group: s_h = RN_f16(s), s_l = (s - s_h) * 2^11 (<= 8 bits: exact in f16, and scaled so that it
// is no subnormal).  Per pair of weights:
//   hi = RN_f16(q * s_h)                      one multiply
//   e  = q * s_h - hi                         one fma: the rounding error of a product is exact
//   lo = RN_f16((q * s_l) * 2^-11 + e)        one multiply, one fma
// so hi + lo = w to 2^-22 of w (w's low part below 2^-24 in magnitude excepted, as with the float32 route),
// at half the instructions of converting every weight to float32 and back (measured 154 M -> see the
// profile of the two-term kernel).
__device__ __forceinline__ uint32_t h2_neg(uint32_t a) {
    uint32_t r;
    asm("neg.f16x2 %0, %1;" : "=r"(r) : "r"(a));
    return r;
}
__device__ __forceinline__ void dequant_q6k_half_split(const RawQ6 &raw, uint32_t a_taddr) {
    const float d = f16_bits_to_f32((uint16_t)raw.d);
    constexpr uint32_t H2_2M11 = 0x10001000u;            // (2^-11, 2^-11)
#pragma unroll
    for (int g = 0; g < 4; g++) {                        // K-local 32g + 16c + i -> column 16g + 8c + i/2
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const uint32_t sw = g < 2 ? raw.sc.x : raw.sc.y;
            const int sc = (int)(int8_t)((sw >> (8 * (2 * (g & 1) + c))) & 0xFFu);     // scales[8h + 2g + c]
            const float s = d * (float)sc;
            const uint32_t s_h = pack_w(s, s);
            const float rest = s - __half2float(__ushort_as_half((uint16_t)(s_h & 0xFFFFu)));
            const uint32_t s_l = pack_w(rest * 2048.0f, rest * 2048.0f);
            const uint4 q0 = raw.ql[c][0], q1 = raw.ql[c][1], qh = raw.qh[c];
            const uint32_t l0[4] = {q0.x, q0.y, q0.z, q0.w}, l1[4] = {q1.x, q1.y, q1.z, q1.w};
            const uint32_t hw[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t lw = (g & 1) ? l1[i] : l0[i];
                const uint32_t low = g < 2 ? (lw & 0x0F0F0F0Fu) : ((lw >> 4) & 0x0F0F0F0Fu);
                const uint32_t v = low | (((hw[i] >> (2 * g)) & 0x03030303u) << 4);      // four 6-bit quants
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const uint32_t q2 = h2_sub(e ? magic_hi(v) : magic_lo(v), H2_1056);  // (q - 32) pair, exact
                    const uint32_t h = h2_mul(q2, s_h);
                    const uint32_t err = h2_fma(q2, s_h, h2_neg(h));
                    hi[8 * c + 2 * i + e] = h;
                    lo[8 * c + 2 * i + e] = h2_fma(h2_mul(q2, s_l), H2_2M11, err);
                }
            }
        }
        tmem_st16(a_taddr + 16 * g, hi);
        tmem_st16(a_taddr + 64 + 16 * g, lo);
    }
}

template <int QT> struct RawOf;
template <> struct RawOf<0> { using type = RawQ4; };
template <> struct RawOf<1> { using type = RawQ6; };

template <int QT>
__device__ __forceinline__ typename RawOf<QT>::type load_raw(const uint8_t *row_ptr, int nb, int b, int sel) {
    if constexpr (QT == 0) return load_raw_q4k(row_ptr, b, sel);
    else return load_raw_q6k(row_ptr, nb, b, sel);
}
// ---- the kernel --------------------------------------------------------------------------------

// SPLIT: the two-term variant for small token counts that must meet the decode tolerance (1e-4).
// Weights and activations are each kept as hi + lo f16 pairs (w = w_hi + w_lo to 2^-22, likewise x)
// and a stage issues three products, w_hi x_hi + w_lo x_hi + w_hi x_lo, into the same fp32
// accumulators; w_lo x_lo (2^-22 of the result) is dropped.  A weight stage is then 128 TMEM
// columns (hi in the first 64, lo behind them) and an activation stage holds the hi sub-tiles
// followed by the lo sub-tiles.  The two small products go to an accumulator of their own, which the
// epilogue adds: the tensor core's fp32 accumulation does not round to nearest, every product added
// to the large sum costs about 2^-25 of it (measured: 1.4e-5 relative after the 768 additions of
// K=4096 with one accumulator), so the large sum takes only the one product per K step it must.
template <int TN, bool SPLIT = false> struct GemmCfg {
    // A stage is 128 K elements: two 64-wide swizzled activation sub-tiles in shared memory and
    // 64 TMEM columns of weights.  One barrier round per stage keeps the single MMA-issuing
    // thread (which runs at a few cycles per instruction) ahead of the tensor core.
    static constexpr int KSUB = 2;
    static constexpr int STAGE_K = BK * KSUB;
    static constexpr int SUBTILE_BYTES = TN * BK * 2;
    static constexpr int HALF_STAGE_BYTES = SUBTILE_BYTES * KSUB;      // the hi (or only) sub-tiles of a stage
    static constexpr int STAGE_BYTES = HALF_STAGE_BYTES * (SPLIT ? 2 : 1);
    static constexpr uint32_t A_HALF_COLS = STAGE_K / 2;             // 64 TMEM columns per weight stage and term
    static constexpr uint32_t A_STAGE_COLS = A_HALF_COLS * (SPLIT ? 2 : 1);
    static_assert(!SPLIT || TN <= 64, "the two-term variant serves up to 64 tokens");
    // Tensor memory (512 columns): accumulators first, weight stages behind them.  Up to 128
    // tokens the accumulator is double-buffered, so the epilogue of one tile overlaps the K loop
    // of the next; a 256-token accumulator leaves room for one.
    // (the two-term variant has one buffer of two accumulators: main and small products)
    static constexpr int ACC_BUFS = SPLIT ? 1 : (TN <= 128 ? 2 : 1);
    static constexpr uint32_t ACC_COLS = SPLIT ? 2 * TN : TN;
    static constexpr uint32_t A_BASE_COL = ACC_BUFS * ACC_COLS;
    static constexpr int TMEM_STAGES = (512 - (int)A_BASE_COL) / (int)A_STAGE_COLS;
    static constexpr int SMEM_STAGES = (227 * 1024 - 1280 - (EPI_WARPS * (EPI_TOK * 32 * 4) + EPI_WARPS * TN_PAD * 4)) / STAGE_BYTES;
    static constexpr int STAGES = TMEM_STAGES < SMEM_STAGES ? (TMEM_STAGES < 4 ? TMEM_STAGES : 4)
                                                            : (SMEM_STAGES < 4 ? SMEM_STAGES : 4);
    static_assert(STAGES >= 2, "at least a double buffer");
    static constexpr uint32_t TMEM_USED = A_BASE_COL + STAGES * A_STAGE_COLS;
    static constexpr uint32_t TMEM_COLS = TMEM_USED <= 256 ? 256 : 512;
    static_assert(TMEM_USED <= 512, "accumulators and weight stages must fit the 512 TMEM columns");
    // epilogue staging: per epilogue warp [EPI_TOK tokens][32 rows] of up to 4 bytes, plus TN token factors
    static constexpr size_t EPI_BYTES = (size_t)EPI_WARPS * (EPI_TOK * 32 * 4) + (size_t)EPI_WARPS * TN_PAD * 4;
    static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256 + EPI_BYTES;
    static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

// Persistent: one CTA per SM walks tiles (weight tile fastest, so the CTAs of a wave share one
// activation tile through L2).  14 warps: 0-7 dequantise, 8 TMA, 9 MMA + TMEM owner, 10-13 epilogue.
template <int QT, int TN, bool SPLIT = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    using C = GemmCfg<TN, SPLIT>;
    constexpr int S = C::STAGES;
    constexpr int AB = C::ACC_BUFS;
    constexpr uint32_t IDESC = umma_idesc_f16(TN);

    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t *tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles + S * C::STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + S, *acc_full = bars + 2 * S, *acc_empty = bars + 2 * S + AB;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 2 * AB);
    uint64_t *duty_bar = bars + 16;                             // the bulk copies that fetch deposits (see the duties)
    static_assert((2 * S + 2 * AB) * 8 + 16 <= 128, "barrier area");
    uint8_t *epi_stage = tiles + S * C::STAGE_BYTES + 256;       // 256 bytes of barriers in front, 16-byte aligned

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Sched sc = make_sched(p, TN);
    const int w_tiles = sc.w_tiles;

    // Programmatic dependent launch: this kernel may start while the kernel that converts its activations
    // is still running.  Only the warps that touch what earlier kernels wrote (the activation producer and
    // the epilogue) wait for them; the dequantising warps read weights only and start at once, so the first
    // operand stages are in tensor memory when the activations arrive.
    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], DEQ_WARPS / 2 + 1); // the 4 warps of one dequant group + the TMA thread (with its bytes)
            mbar_init(&empty[s], 1);                // tcgen05.commit
        }
        for (int a = 0; a < AB; a++) {
            mbar_init(&acc_full[a], 1);             // tcgen05.commit after the tile's last MMA
            mbar_init(&acc_empty[a], EPI_WARPS);    // epilogue warps, once they have read it out
        }
        mbar_init(duty_bar, 1);
        mbar_init_fence();
    }
    if (warp == DEQ_WARPS + 1) {                    // the MMA warp owns TMEM
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DEQ_WARPS) {
        // ---------------- dequantise weight tiles: group g produces the stages of parity g ----------------
        const int r = threadIdx.x & 127, g = threadIdx.x >> 7;
        const int nb = p.K / QK_K;
        // TMEM address of this warp's lane quarter, first weight column
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + C::A_BASE_COL;
        bool ok = true;
        uint32_t unit_it = 0;                       // stages of the units before this one
        UnitIter ui;
        Unit u;
        typename RawOf<QT>::type cur;
        bool have_cur = false;                      // `cur` already holds this unit's first block
        while (ok && ui.next(sc, u)) {
            const int n0 = (u.tile % w_tiles) * TILE_ROWS;
            const int row = min(n0 + r, p.N - 1);
            const uint8_t *row_ptr = p.W + (size_t)row * p.row_stride;
            if (!have_cur) cur = load_raw<QT>(row_ptr, nb, u.b0, g);
            // the next unit's row, so that the register prefetch runs across the unit boundary
            UnitIter peek = ui;
            Unit un = u;
            const bool has_next = peek.next(sc, un);
            const uint8_t *next_row_ptr =
                p.W + (size_t)min((un.tile % w_tiles) * TILE_ROWS + r, p.N - 1) * p.row_stride;
            // (prefetch.global.L2 of the blocks further ahead was measured: 5-10 % slower on every
            // shape -- each of these row-per-lane accesses costs 32 L1 wavefronts, prefetch or not)
            for (int b = u.b0; b < u.b1; b++) {
                typename RawOf<QT>::type nxt = cur;
                if (b + 1 < u.b1) nxt = load_raw<QT>(row_ptr, nb, b + 1, g);   // in flight during this block
                else if (has_next) nxt = load_raw<QT>(next_row_ptr, nb, un.b0, g);
                const uint32_t it = unit_it + 2u * (uint32_t)(b - u.b0) + (uint32_t)g;   // stage number over all units
                const uint32_t s = it % S;
                if (it >= (uint32_t)S && !mbar_wait(&empty[s], ((it / S) - 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_EMPTY_WAIT);
                    ok = false;
                    break;
                }
                const uint32_t a_taddr = lane_base + s * C::A_STAGE_COLS;
                if constexpr (SPLIT) {
                    if constexpr (QT == 0) {
                        if (g == 0) dequant_q4k_half_split<0>(cur, a_taddr);
                        else dequant_q4k_half_split<1>(cur, a_taddr);
                    } else {
                        dequant_q6k_half_split(cur, a_taddr);
                    }
                } else if constexpr (QT == 0) {
                    const ScalesQ4 sq = unpack_scales_q4k(cur.hdr);
                    if (g == 0) dequant_q4k_half<0>(cur, sq, a_taddr);
                    else dequant_q4k_half<1>(cur, sq, a_taddr);
                } else {
                    dequant_q6k_half(cur, a_taddr);
                }
                tmem_st_wait();                      // this warp's tensor-memory stores have landed
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
                cur = nxt;
            }
            unit_it += 2u * (uint32_t)(u.b1 - u.b0);
            have_cur = has_next;
        }
    } else if (warp == DEQ_WARPS) {
        // ---------------- TMA producer of the activation tiles ----------------
        // (the whole warp walks the loop, the elected lane issues: see the MMA warp)
        const bool leader = elect_one();
        uint32_t it = 0;
        bool ok = true;
        UnitIter ui;
        Unit u;
        pdl_wait();                                   // the converted activations are complete and visible
        while (ok && ui.next(sc, u)) {
            const int t0 = (u.tile / w_tiles) * TN;
            for (int st = 2 * u.b0; st < 2 * u.b1; st++, it++) {
                const uint32_t s = it % S;
                if (it >= (uint32_t)S && !mbar_wait(&empty[s], ((it / S) - 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_EMPTY_WAIT);
                    ok = false;
                    break;
                }
                if (leader) {
                    mbar_arrive_expect_tx(&full[s], C::STAGE_BYTES);
#pragma unroll
                    for (int us = 0; us < C::KSUB; us++)
                        tma_load_2d(tiles + s * C::STAGE_BYTES + us * C::SUBTILE_BYTES, &tmap_x,
                                    st * C::STAGE_K + us * BK, t0, &full[s]);
                    if constexpr (SPLIT) {               // the lo terms are rows M .. 2M-1 of the same tensor
#pragma unroll
                        for (int us = 0; us < C::KSUB; us++)
                            tma_load_2d(tiles + s * C::STAGE_BYTES + C::HALF_STAGE_BYTES + us * C::SUBTILE_BYTES, &tmap_x,
                                        st * C::STAGE_K + us * BK, p.M + t0, &full[s]);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == DEQ_WARPS + 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp walks the schedule and waits on the barriers, so that descriptors and
        // tensor-memory addresses are formed in warp-uniform code; the elected lane issues.  (With the
        // loop under `if (lane == 0)` the issuing thread needed ~55 clocks per instruction.)
        // Shared-memory descriptors differ only in their start-address field, so the loop adds to
        // the low word of one prebuilt descriptor instead of rebuilding 64-bit values.
        const bool leader = elect_one();
        const uint64_t desc0 = umma_desc_sw128(smem_u32(tiles));
        const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
        const uint32_t desc_lo0 = (uint32_t)desc0;
        const uint32_t a_col0 = tmem_base + C::A_BASE_COL;
        bool ok = true;
        uint32_t it = 0, tcount = 0;
        UnitIter ui;
        Unit u;
        for (; ok && ui.next(sc, u); tcount++) {
            const uint32_t ab = tcount % AB;
            // the epilogue must have read this accumulator out (unit tcount - AB) before it is overwritten
            if (tcount >= (uint32_t)AB && !mbar_wait(&acc_empty[ab], ((tcount / AB) - 1) & 1, p.wait_limit)) {
                report_error(p.err, KERR_MMA_WAIT);
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + ab * C::ACC_COLS;
            for (int st = 2 * u.b0; st < 2 * u.b1; st++, it++) {
                const uint32_t s = it % S;
                if (!mbar_wait(&full[s], (it / S) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_FULL_WAIT);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t lo_s = desc_lo0 + ((s * C::STAGE_BYTES) >> 4);
                const uint32_t a_s = a_col0 + s * C::A_STAGE_COLS;
                const uint32_t first = st == 2 * u.b0 ? 0u : 1u;
                if (leader) {
#pragma unroll
                    for (int us = 0; us < C::KSUB; us++)
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; kk++) {
                            // 16 K elements further: 8 TMEM columns of A, 32 bytes inside B's swizzled row
                            const uint32_t lo = lo_s + (uint32_t)((us * C::SUBTILE_BYTES + kk * 32) >> 4);
                            const uint64_t b_desc = ((uint64_t)desc_hi << 32) | lo;
                            const uint32_t acc_flag = (us | kk) ? 1u : first;
                            umma_f16_ts(d_tmem, a_s + (uint32_t)(us * 32 + kk * 8), b_desc, IDESC, acc_flag);
                            if constexpr (SPLIT) {       // w_lo x_hi + w_hi x_lo, into the accumulator behind the main one
                                const uint64_t b_lo = ((uint64_t)desc_hi << 32) | (lo + (uint32_t)(C::HALF_STAGE_BYTES >> 4));
                                umma_f16_ts(d_tmem + TN, a_s + C::A_HALF_COLS + (uint32_t)(us * 32 + kk * 8), b_desc, IDESC, acc_flag);
                                umma_f16_ts(d_tmem + TN, a_s + (uint32_t)(us * 32 + kk * 8), b_lo, IDESC, 1u);
                            }
                        }
                    umma_commit(&empty[s]);        // stage free once these MMAs have read it
                }
                __syncwarp();
            }
            if (ok && leader) umma_commit(&acc_full[ab]);   // accumulator of this unit complete
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> shared staging -> global ----------------
        // A thread owns one weight row (its TMEM lane) and sees that row's tokens, but the output is
        // token-major: element (token, row) at token*N + row.  Each warp therefore transposes its
        // 32 rows x 16 tokens at a time through a private staging block in shared memory and writes
        // 16-byte vectors (8 bf16 / 4 fp32 consecutive rows of one token); only __syncwarp is needed.
        // A partial unit (split of the last wave) either deposits its raw fp32 accumulator in a
        // workspace slot, laid out like a tile-sized output, or adds the others' deposits to its own.
        const int quarter = warp & 3;                           // TMEM lanes this warp may read
        const int ew = warp - (DEQ_WARPS + 2);
        uint8_t *stg = epi_stage + (size_t)ew * (EPI_TOK * 32 * 4);       // [EPI_TOK tokens][32 rows]
        float *scale_s = reinterpret_cast<float *>(epi_stage + EPI_WARPS * (EPI_TOK * 32 * 4)) + ew * TN_PAD;
        constexpr int EPI_THREADS = EPI_WARPS * 32;
        struct Duty { int tt, c_first, pieces, n0, t0; } duty[2];      // the cut tiles this CTA holds a piece of
        int n_duty = 0;
        uint32_t tcount = 0;
        bool dead = false;                                      // a wait gave up: no more memory traffic, barriers only
        const bool gather = p.world > 1;
        pdl_wait();                                   // token factors, exchange counters, mailbox step: all from earlier kernels
        const uint32_t gather_step = gather ? *reinterpret_cast<volatile uint32_t *>(p.step_word) + 1u : 0u;
        UnitIter ui;
        Unit u;
        for (; !dead && ui.next(sc, u); tcount++) {
            const uint32_t ab = tcount % AB;
            const int n0 = (u.tile % w_tiles) * TILE_ROWS, t0 = (u.tile / w_tiles) * TN;
            const bool partial = u.b1 - u.b0 < sc.nb;
            // this tile's token factors (per warp copy, so no cross-warp barrier)
            for (int c = lane; c < TN; c += 32) scale_s[c] = (t0 + c < p.M) ? __ldg(p.tok_scale + t0 + c) : 0.0f;
            __syncwarp();
            if (!mbar_wait(&acc_full[ab], (tcount / AB) & 1, p.wait_limit)) {
                report_error(p.err, KERR_MMA_WAIT);
                dead = true;
            }
            tc_fence_after();

            // ---- partial unit: a tile cut along K ----
            // Every piece is deposited straight from the registers and published with one release per CTA;
            // once its own units are done, each of the P CTAs that hold a piece adds up one P-th of the tile
            // over all deposits and writes that part of the output (the duties below).  With tiles of up to
            // 128 KB this beats one CTA reading all the pieces: no CTA reads more than one tile's worth.
            const bool deposit = partial;
            int tt = 0;
            if (partial) {
                tt = u.tile - sc.n_full;
                const int tb = tt * sc.nb, te = tb + sc.nb;
                int c = (int)blockIdx.x;
                if (u.b0 != 0) {                                 // the CTA that holds the tile's first block
                    c = min(sc.gt - 1, (int)(((unsigned)tb * (unsigned)sc.gt) / (unsigned)sc.T));
                    while (c + 1 < sc.gt && tail_start(sc, c + 1) <= tb) c++;
                    while (c > 0 && tail_start(sc, c) > tb) c--;
                }
                const int c_first = c;
                c = (int)blockIdx.x;
                while (c + 1 < sc.gt && tail_start(sc, c + 1) < te) c++;
                duty[n_duty].tt = tt; duty[n_duty].c_first = c_first; duty[n_duty].pieces = c - c_first + 1;
                duty[n_duty].n0 = n0; duty[n_duty].t0 = t0;
                n_duty++;
            }

            // ---- where this unit's values go ----
            const bool o_bf16 = p.out_bf16 != 0;
            const int esz = o_bf16 ? 2 : 4;
            uint8_t *o_ptr = (uint8_t *)p.Out;
            const size_t o_stride = (size_t)p.n_total;          // elements between tokens (n_total = N unless sharded)
            const int tok_base = t0, row_base = p.row_offset + n0 + 32 * quarter, tok_lim = p.M, row_lim = p.row_offset + p.N;
            // a deposit goes token-major into this CTA's slot: slot 1 for the piece that ends its range, else 0
            float *dep = p.ws_slots + (size_t)(2 * blockIdx.x + (u.b0 != 0 ? 0 : 1)) * (TILE_ROWS * TN) + 32 * quarter + lane;
            const bool vec_ok = (o_stride % (size_t)(16 / esz)) == 0;     // 16-byte stores need whole vectors per token
            const uint32_t acc = tmem_base + ab * C::ACC_COLS + ((uint32_t)(32 * quarter) << 16);
#pragma unroll 1
            for (int g0 = 0; g0 < TN && !dead; g0 += EPI_TOK) {
                constexpr int GT = TN < EPI_TOK ? TN : EPI_TOK;  // tokens in this group
                // ---- TMEM -> registers (all loads of the group, one wait) -> scaled -> staging ----
                uint32_t v[GT / 16][16];
#pragma unroll
                for (int c = 0; c < GT / 16; c++) tmem_ld16(acc + (uint32_t)(g0 + 16 * c), v[c]);
                if constexpr (SPLIT) {                           // plus the accumulator of the small products
                    uint32_t sm[GT / 16][16];
#pragma unroll
                    for (int c = 0; c < GT / 16; c++) tmem_ld16(acc + (uint32_t)(TN + g0 + 16 * c), sm[c]);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < GT / 16; c++)
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            v[c][j] = __float_as_uint(__uint_as_float(v[c][j]) + __uint_as_float(sm[c][j]));
                }
                tmem_ld_wait();
                if (g0 + GT >= TN) {                             // last read of this accumulator: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[ab]);
                }
                if (deposit) {                                   // straight from the registers, the rows of a warp side by side
#pragma unroll
                    for (int j = 0; j < GT; j++) __stcg(dep + (size_t)(g0 + j) * TILE_ROWS, __uint_as_float(v[j / 16][j % 16]));
                    continue;
                }
#pragma unroll
                for (int c = 0; c < GT / 16; c++) {
#pragma unroll
                    for (int j4 = 0; j4 < 4; j4++) {
                        const float4 sc4 = *reinterpret_cast<const float4 *>(scale_s + g0 + 16 * c + 4 * j4);
                        const float f[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const int tl = 16 * c + 4 * j4 + j;                  // token within the group
                            const float val = __uint_as_float(v[c][4 * j4 + j]) * f[j];
                            if (o_bf16) reinterpret_cast<__nv_bfloat16 *>(stg)[tl * 32 + lane] = __float2bfloat16_rn(val);
                            else reinterpret_cast<float *>(stg)[tl * 32 + lane] = val;
                        }
                    }
                }
                __syncwarp();
                // ---- staging -> global ----
                if (vec_ok) {
                    const int vec_per_tok = 32 * esz / 16;       // 4 (bf16) or 8 (fp32) vectors per token
                    const int rows_per_vec = 16 / esz;
                    for (int i = lane; i < GT * vec_per_tok; i += 32) {
                        const int tl = i / vec_per_tok, vv = i % vec_per_tok;
                        const int tok = tok_base + g0 + tl, row = row_base + vv * rows_per_vec;
                        if (tok < tok_lim && row < row_lim) {
                            const uint4 d = *reinterpret_cast<const uint4 *>(stg + (size_t)tl * 32 * esz + vv * 16);
                            *reinterpret_cast<uint4 *>(o_ptr + ((size_t)tok * o_stride + row) * esz) = d;
                        }
                    }
                } else {
                    for (int tl = 0; tl < GT; tl++) {
                        const int tok = tok_base + g0 + tl, row = row_base + lane;
                        if (tok < tok_lim && row < row_lim) {
                            if (o_bf16) {
                                ((uint16_t *)o_ptr)[(size_t)tok * o_stride + row] =
                                    reinterpret_cast<const uint16_t *>(stg)[tl * 32 + lane];
                            } else {
                                ((float *)o_ptr)[(size_t)tok * o_stride + row] =
                                    reinterpret_cast<const float *>(stg)[tl * 32 + lane];
                            }
                        }
                    }
                }
                if (gather) {
                    // The same values, as {value, call number} words, to every peer's mailbox: a lane per row,
                    // so that a token's 32 rows cross NVLink as one 256-byte run per peer.
                    const int row = row_base + lane;
                    for (int tl = 0; tl < GT; tl++) {
                        const int tok = tok_base + g0 + tl;
                        if (tok >= tok_lim || row >= row_lim) continue;
                        const uint32_t bits = o_bf16 ? (uint32_t)reinterpret_cast<const uint16_t *>(stg)[tl * 32 + lane] << 16
                                                     : reinterpret_cast<const uint32_t *>(stg)[tl * 32 + lane];
                        const size_t word = (gather_step & 1u) * p.half_words +
                                            ((size_t)p.rank * p.M + tok) * p.N + (row - p.row_offset);
                        for (int dd = 0; dd < p.world; dd++)
                            if (dd != p.rank) mailbox_store(p.peer_box[dd] + word, bits, gather_step);
                    }
                }
                __syncwarp();                                    // staging is reused by the next group
            }
            if (deposit) {
                named_barrier_sync(2, EPI_THREADS);
                if (ew == 0 && lane == 0) {
                    __threadfence();                             // the deposits of all four warps, device-wide
                    atomicAdd(p.ws_counters + 2 * tt, 1u);
                }
            }
        }
        // ---- duties: this CTA's share of the sums of the cut tiles it holds a piece of ----
        for (int di = 0; di < n_duty && !dead; di++) {
            const Duty dy = duty[di];
            uint32_t *cnt = p.ws_counters + 2 * dy.tt;
            // the tile as TN * 32 groups of four rows; piece q of P takes groups [q * tot / P, (q + 1) * tot / P)
            constexpr int TOT = TN * (TILE_ROWS / 4);
            const int q = (int)blockIdx.x - dy.c_first;
            const int e_lo = (int)(((long long)q * TOT) / dy.pieces), e_hi = (int)(((long long)(q + 1) * TOT) / dy.pieces);
            const int n_e = e_hi - e_lo;
            const uint32_t slice_bytes = (uint32_t)n_e * 16u;
            // This CTA's share of every deposit comes into the (now idle) stage area by bulk copies: up to 128 KB
            // behind one barrier instead of a trip to L2 per few values.  Every tensor-core instruction and
            // tiled copy that used the stage area has completed: the last accumulator has been read.
            if (ew == 0 && lane == 0) {
                bool seen = false;
                for (uint32_t i = 0; i < p.wait_limit && !seen; i++) {
                    uint32_t n;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(n) : "l"(cnt) : "memory");
                    seen = n >= (uint32_t)dy.pieces;
                    if (!seen) __nanosleep(32);
                }
                if (!seen) report_error(p.err, KERR_SPLIT_WAIT);
                asm volatile("fence.proxy.async;" ::: "memory");     // the copies below read what generic stores wrote
                mbar_arrive_expect_tx(duty_bar, (uint32_t)dy.pieces * slice_bytes);
                for (int ci = 0; ci < dy.pieces; ci++) {
                    const int c = dy.c_first + ci;
                    const int k = ci == 0 ? 1 : 0;               // the first piece is the end of its CTA's range
                    const float4 *sl = reinterpret_cast<const float4 *>(p.ws_slots + (size_t)(2 * c + k) * (TILE_ROWS * TN)) + e_lo;
                    bulk_copy_g2s(tiles + (size_t)ci * slice_bytes, sl, slice_bytes, duty_bar);
                }
            }
            if (!mbar_wait(duty_bar, (uint32_t)di & 1u, p.wait_limit)) {
                report_error(p.err, KERR_FULL_WAIT);
                dead = true;
                break;
            }
            const bool o_bf16 = p.out_bf16 != 0;
            const bool vec_ok = (p.n_total & 3) == 0 && (p.row_offset & 3) == 0;
            // EU groups per thread at a time, so that the shared-memory reads, the token factors and the stores
            // of eight groups overlap (one group at a time, each step waited for the one before: 19 us per tile)
            constexpr int EU = 8;
            for (int el0 = ew * 32 + lane; el0 < n_e; el0 += EU * EPI_THREADS) {
                float4 acc4[EU];
                float ts[EU];
#pragma unroll
                for (int j = 0; j < EU; j++) {
                    acc4[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    const int e = e_lo + min(el0 + j * EPI_THREADS, n_e - 1);
                    ts[j] = __ldg(p.tok_scale + min(dy.t0 + e / (TILE_ROWS / 4), p.M - 1));
                }
                for (int ci = 0; ci < dy.pieces; ci++) {
                    const uint8_t *sl = tiles + (size_t)ci * slice_bytes;
#pragma unroll
                    for (int j = 0; j < EU; j++) {
                        const float4 v4 = *reinterpret_cast<const float4 *>(sl + (size_t)min(el0 + j * EPI_THREADS, n_e - 1) * 16);
                        acc4[j].x += v4.x; acc4[j].y += v4.y; acc4[j].z += v4.z; acc4[j].w += v4.w;
                    }
                }
#pragma unroll
                for (int j = 0; j < EU; j++) {
                    const int el = el0 + j * EPI_THREADS;
                    if (el >= n_e) continue;
                    const int e = e_lo + el;
                    const int tok = dy.t0 + e / (TILE_ROWS / 4), row = p.row_offset + dy.n0 + 4 * (e % (TILE_ROWS / 4));
                    if (tok >= p.M || row >= p.row_offset + p.N) continue;
                    float f[4] = {acc4[j].x * ts[j], acc4[j].y * ts[j], acc4[j].z * ts[j], acc4[j].w * ts[j]};
                    const int nv = min(4, p.row_offset + p.N - row);
                    const size_t o = (size_t)tok * p.n_total + row;
                    if (o_bf16) {
                        __nv_bfloat16 hb[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            hb[i] = __float2bfloat16_rn(f[i]);
                            f[i] = __bfloat162float(hb[i]);      // what the peers get is what this rank stores
                        }
                        if (vec_ok && nv == 4) {
                            *reinterpret_cast<uint2 *>((__nv_bfloat16 *)p.Out + o) = *reinterpret_cast<const uint2 *>(hb);
                        } else {
                            for (int i = 0; i < nv; i++) ((__nv_bfloat16 *)p.Out)[o + i] = hb[i];
                        }
                    } else {
                        if (vec_ok && nv == 4) {
                            *reinterpret_cast<float4 *>((float *)p.Out + o) = make_float4(f[0], f[1], f[2], f[3]);
                        } else {
                            for (int i = 0; i < nv; i++) ((float *)p.Out)[o + i] = f[i];
                        }
                    }
                    if (gather) {                                // the same values, as words, to every peer's mailbox
                        const size_t word = (gather_step & 1u) * p.half_words + ((size_t)p.rank * p.M + tok) * p.N + (row - p.row_offset);
                        for (int dd = 0; dd < p.world; dd++) {
                            if (dd == p.rank) continue;
                            uint2 *box = p.peer_box[dd] + word;
                            if (nv == 4 && (word & 1) == 0) {             // the lane's four words as two 16-byte stores
                                mailbox_store2(box, __float_as_uint(f[0]), __float_as_uint(f[1]), gather_step);
                                mailbox_store2(box + 2, __float_as_uint(f[2]), __float_as_uint(f[3]), gather_step);
                            } else {
                                for (int i = 0; i < nv; i++) mailbox_store(box + i, __float_as_uint(f[i]), gather_step);
                            }
                        }
                    }
                }
            }
            named_barrier_sync(2, EPI_THREADS);                  // every thread has read what it needs
            if (ew == 0 && lane == 0) {
                // the last of the P CTAs to finish leaves both counters at zero for the next launch
                if (atomicAdd(cnt + 1, 1u) + 1u == (uint32_t)dy.pieces) {
                    cnt[0] = 0;
                    cnt[1] = 0;
                }
            }
        }
        if (gather) {
            // ---- collect the other ranks' slices from this rank's mailbox ----
            const uint2 *box = p.peer_box[p.rank] + (gather_step & 1u) * p.half_words;
            const size_t per_src = (size_t)p.M * p.N;                    // words one sender posts
            const size_t remote = (size_t)(p.world - 1) * per_src;
            const int et = ew * 32 + lane;
            // UNPACK words in flight per thread: a batch costs one trip to L2; only words that had not
            // landed yet are polled again.
            constexpr int UNPACK = 8;
            const size_t stride = (size_t)gridDim.x * EPI_THREADS;
            bool late = dead;
            for (size_t i0 = (size_t)blockIdx.x * EPI_THREADS + et; i0 < remote && !late; i0 += UNPACK * stride) {
                uint2 got[UNPACK];
#pragma unroll
                for (int b = 0; b < UNPACK; b++) {
                    const size_t i = i0 + b * stride;
                    if (i < remote) {
                        const int q = (int)(i / per_src);
                        got[b] = mailbox_load(box + (size_t)(q < p.rank ? q : q + 1) * per_src + (i - (size_t)q * per_src));
                    }
                }
#pragma unroll
                for (int b = 0; b < UNPACK; b++) {
                    const size_t i = i0 + b * stride;
                    if (i >= remote || late) continue;
                    const int q = (int)(i / per_src);
                    const size_t rem = i - (size_t)q * per_src;
                    const int src = q < p.rank ? q : q + 1;
                    const int tok = (int)(rem / p.N), row = (int)(rem - (size_t)tok * p.N);
                    if (got[b].y != gather_step &&
                        !mailbox_wait(box + (size_t)src * per_src + rem, gather_step, p.gather_limit, got[b])) {
                        report_error(p.err, KERR_GATHER_WAIT);
                        late = true;
                        continue;
                    }
                    const size_t o = (size_t)tok * p.n_total + (size_t)src * p.N + row;
                    if (p.out_bf16) ((__nv_bfloat16 *)p.Out)[o] = __float2bfloat16_rn(__uint_as_float(got[b].x));
                    else ((float *)p.Out)[o] = __uint_as_float(got[b].x);
                }
            }
            // the last CTA to get here advances the call number for the next launch
            named_barrier_sync(2, EPI_THREADS);
            if (ew == 0 && lane == 0) {
                const uint32_t ticket = atomicAdd(p.done_counter, 1u);
                if (ticket == gridDim.x - 1) {
                    *p.done_counter = 0;
                    *p.step_word = gather_step;
                }
            }
        }
    }

    // teardown: everyone meets here, also after an abandoned wait, so TMEM is always released
    tc_fence_before();
    __syncthreads();
    if (warp == DEQ_WARPS + 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// Activations -> f16 for the tensor cores, one CTA per token.  Each token row is multiplied by a
// power of two that brings its largest magnitude to [2^13, 2^14), so no finite input overflows or
// sinks into f16's subnormals relative to its row; the inverse factor goes to tok_scale[token]
// and is applied to the token's outputs in the GEMM epilogue (exact: powers of two).
__global__ void __launch_bounds__(256)
activations_to_f16_kernel(const void *__restrict__ x, int x_is_bf16, int K, __half *__restrict__ out,
                          __half *__restrict__ out_lo, float *__restrict__ tok_scale) {
    __shared__ float red[8];
    pdl_prologue();                                   // the input is complete; the scratch's last reader has finished
    const int tok = blockIdx.x;
    const size_t base = (size_t)tok * K;
    // 8 consecutive values per thread and iteration (K is a multiple of 256)
    auto load8 = [&](int k, float (&v)[8]) {
        if (x_is_bf16) {
            const uint4 u = __ldg(reinterpret_cast<const uint4 *>((const uint16_t *)x + base + k));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
        } else {
            const float4 a = __ldg(reinterpret_cast<const float4 *>((const float *)x + base + k));
            const float4 b = __ldg(reinterpret_cast<const float4 *>((const float *)x + base + k + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
    };
    float amax = 0.0f;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        float v[8];
        load8(k, v);
#pragma unroll
        for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
    // amax < 2^(eb-126); scale 2^e with e = 14 + 126 - eb puts it below 2^14
    const int eb = (int)((__float_as_uint(amax) >> 23) & 0xFFu);
    int e = 140 - eb;
    e = max(-126, min(126, e));
    if (amax == 0.0f || eb == 255) e = 0;                // all-zero row, or inf/nan: leave as is
    const float sc = exp2i(e);
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {   // second read comes from L1/L2
        float v[8];
        load8(k, v);
        uint4 o;
        o.x = pack_w(v[0] * sc, v[1] * sc);
        o.y = pack_w(v[2] * sc, v[3] * sc);
        o.z = pack_w(v[4] * sc, v[5] * sc);
        o.w = pack_w(v[6] * sc, v[7] * sc);
        *reinterpret_cast<uint4 *>(out + base + k) = o;
        if (out_lo) {                                    // two-term variant: what the f16 value left behind
            const uint32_t h[4] = {o.x, o.y, o.z, o.w};
            uint32_t l[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 back = __half22float2(*reinterpret_cast<const __half2 *>(&h[i]));
                l[i] = pack_w(v[2 * i] * sc - back.x, v[2 * i + 1] * sc - back.y);
            }
            *reinterpret_cast<uint4 *>(out_lo + base + k) = make_uint4(l[0], l[1], l[2], l[3]);
        }
    }
    if (threadIdx.x == 0) tok_scale[tok] = exp2i(-e);
}

// ---- host side ---------------------------------------------------------------------------------

// Does cutting the last, partial wave of tiles along K pay?  The exchange is not free: every piece is a
// tile-sized fp32 store from the registers, and the sum reads one tile's worth per CTA (a tile in two pieces
// is summed by the CTA that holds its first block, more pieces share the sum out).  The two-term kernel
// keeps the rule it was measured with (up to half a wave of tiles, K >= 4096).
// `forced` = 0 / 1 overrides the rule (measurements and tests), -1 leaves it alone.
bool split_pays(int n_tiles, int nb, int sms, int forced, bool two_term) {
    const int rest = n_tiles % sms;
    if (rest == 0 || nb < 2) return false;
    if (forced >= 0) return forced != 0;
    if (two_term) return n_tiles <= sms / 2 && nb >= 16;
    // The last, partial wave runs `rest` tiles for nb block times; cut over all SMs it takes nb * rest / sms of
    // them, but the exchange and the shorter units cost the equivalent of 15-20 block times at 128- and
    // 256-token tiles (measured on a B200, split / unsplit: K=14336 -> 4096 0.55 at 128 tokens, 0.73 at 512,
    // 1.03 at 2048; K=4096 -> 14336 1.36, 1.15, 0.97).  So: where at least 20 block times are saved, or at
    // least 8 when the tail is so short that every CTA gets one block (one deposit, a small share of the sum).
    const long long saved_x_sms = (long long)nb * (sms - rest);
    return nb >= 4 && (saved_x_sms >= 20LL * sms || (saved_x_sms >= 8LL * sms && (long long)rest * nb <= sms));
}

template <int QT, int TN, bool SPLIT = false>
cudaError_t launch_tn(const GemmParams &p, const void *x_f16, cudaStream_t s, bool pdl) {
    CUtensorMap tmap;
    // two-term variant: rows M .. 2M-1 of the converted activations hold the lo terms
    cudaError_t e = encode_2d(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x_f16, (uint64_t)p.K,
                              (uint64_t)p.M * (SPLIT ? 2 : 1), (uint64_t)p.K * 2, BK, TN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (e != cudaSuccess) return e;
    constexpr size_t smem = GemmCfg<TN, SPLIT>::SMEM;
    auto kern = gemm_kernel<QT, TN, SPLIT>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int n_tiles = ((p.N + TILE_ROWS - 1) / TILE_ROWS) * ((p.M + TN - 1) / TN);
    int grid = n_tiles < p.sm_count ? n_tiles : p.sm_count;
    GemmParams q = p;
    q.split = 0;
    if (p.ws_slots && split_pays(n_tiles, p.K / QK_K, p.sm_count, p.split, SPLIT)) {
        q.split = 1;
        const int tail_blocks = (n_tiles % p.sm_count) * (p.K / QK_K);
        if (n_tiles < p.sm_count) grid = tail_blocks < p.sm_count ? tail_blocks : p.sm_count;
    }
    if (q.world > 1) grid = p.sm_count;      // CTAs without a tile still take their share of the mailbox
    return launch_dependent(kern, dim3((unsigned)grid), dim3(GEMM_THREADS), smem, s, pdl, tmap, q);
}

// Above 128 tokens: 256 or 128 tokens per tile?  A 256-token tile dequantises every weight half as often, a
// 128-token tile costs 0.62 of its time (measured) and there are twice as many, which fills the last wave
// better at some shapes: with 148 SMs, K=4096 -> 14336 at 384 tokens is 224 tiles of 256 (two waves, the
// second half empty) or 336 of 128 (three waves of 0.62): 61 against 55 us; K=14336 -> 4096 at 512 tokens
// 81 against 75 us.  The estimate counts block times of a 256-token tile: whole waves, the last one either cut
// along K (where split_pays says so; the exchange costs about 17 block times of the tile, 8 when every CTA
// gets one block) or run as a whole wave.
int tokens_per_tile_above_128(const GemmParams &p) {
    const int nb = p.K / QK_K, sms = p.sm_count > 0 ? p.sm_count : 148;
    const int w_tiles = (p.N + TILE_ROWS - 1) / TILE_ROWS;
    auto estimate = [&](int tn, double c) {
        const int tiles = w_tiles * ((p.M + tn - 1) / tn);
        const int full = tiles / sms, rest = tiles % sms;
        if (rest == 0) return (double)full * nb * c;
        if (p.ws_slots && split_pays(tiles, nb, sms, p.split, false)) {
            const double exchange = (long long)nb * (sms - rest) >= 20LL * sms ? 17.0 : 8.0;
            return ((double)full * nb + (double)rest * nb / sms + exchange) * c;
        }
        return (double)(full + 1) * nb * c;
    };
    return estimate(128, 0.62) < estimate(256, 1.0) ? 128 : 256;
}

template <int QT>
cudaError_t launch_qt(const GemmParams &p, const void *x_f16, bool two_term, cudaStream_t s, bool pdl) {
    if (two_term) return p.M <= 32 ? launch_tn<QT, 32, true>(p, x_f16, s, pdl) : launch_tn<QT, 64, true>(p, x_f16, s, pdl);
    if (p.M <= 32) return launch_tn<QT, 32>(p, x_f16, s, pdl);
    if (p.M <= 64) return launch_tn<QT, 64>(p, x_f16, s, pdl);
    if (p.M <= 128 || tokens_per_tile_above_128(p) == 128) return launch_tn<QT, 128>(p, x_f16, s, pdl);
    return launch_tn<QT, 256>(p, x_f16, s, pdl);
}

}  // namespace

// Scratch layout: [M*K f16 activations (and M*K lo terms behind them where the two-term variant
// can run), rounded up to 256 bytes][M float token scales].
static size_t scratch_x_bytes(int K, int M) {
    const size_t rows = M <= GEMM_TWO_TERM_MAX_TOKENS ? 2 * (size_t)M : (size_t)M;
    return (rows * K * 2 + 255) / 256 * 256;
}

size_t gemm_scratch_bytes(int K, int M) { return scratch_x_bytes(K, M) + (size_t)M * sizeof(float); }

cudaError_t launch_activations_to_f16(const void *x, int x_dtype, int K, int M, void *out_f16, float *tok_scale,
                                      cudaStream_t s) {
    if (K <= 0 || M <= 0 || K % 8) return cudaErrorInvalidValue;
    activations_to_f16_kernel<<<(unsigned)M, 256, 0, s>>>(x, x_dtype == DT_BF16, K, (__half *)out_f16, nullptr, tok_scale);
    return cudaGetLastError();
}

// Split workspace: [2 * sms counters in 4 KiB][2 * sms slots of 128 x 256 floats].
size_t gemm_split_counter_bytes() { return 4096; }
size_t gemm_split_workspace_bytes(int sms) {
    return gemm_split_counter_bytes() + (size_t)2 * sms * TILE_ROWS * 256 * sizeof(float);
}

cudaError_t launch_gemm(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                        int K, int N, int M, void *scratch, void *split_ws, int split_mode, ErrSink err_word,
                        cudaStream_t s, uint64_t *launches, const GemmGather *gather, bool two_term, bool pdl) {
    if (K <= 0 || N <= 0 || M <= 0) return cudaSuccess;
    if (!scratch) return cudaErrorInvalidValue;
    two_term = two_term && M <= GEMM_TWO_TERM_MAX_TOKENS;
    __half *x_f16 = (__half *)scratch;
    float *tok_scale = (float *)((uint8_t *)scratch + scratch_x_bytes(K, M));
    cudaError_t e = launch_dependent(activations_to_f16_kernel, dim3((unsigned)M), dim3(256), 0, s, pdl, x,
                                     (int)(x_dtype == DT_BF16), K, x_f16,
                                     two_term ? x_f16 + (size_t)M * K : (__half *)nullptr, tok_scale);
    if (e != cudaSuccess) return e;
    if (launches) (*launches)++;
    GemmParams p{};
    p.W = w; p.Out = out; p.err = err_word.word; p.wait_limit = err_word.mbar_polls; p.gather_limit = err_word.gather_polls; p.K = K; p.N = N; p.M = M; p.out_bf16 = out_dtype == DT_BF16;
    p.tok_scale = tok_scale;
    p.split = split_mode;          // launch_tn turns the mode into the decision
    p.n_total = N;
    if (gather && gather->world > 1) {
        p.world = gather->world; p.rank = gather->rank; p.n_total = N * gather->world; p.row_offset = gather->rank * N;
        p.done_counter = gather->done_counter; p.step_word = gather->step_word;
        p.half_words = (size_t)gather->world * M * N;
        for (int d = 0; d < gather->world; d++) p.peer_box[d] = (uint2 *)gather->peer_mailbox[d];
    }
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&p.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    if (split_ws && 2 * p.sm_count * sizeof(uint32_t) <= gemm_split_counter_bytes()) {
        p.ws_counters = (uint32_t *)split_ws;
        p.ws_slots = (float *)((uint8_t *)split_ws + gemm_split_counter_bytes());
    }
    if (wdtype == DT_Q4K) {
        p.row_stride = (size_t)(K / QK_K) * Q4K_BLOCK_BYTES;
        e = launch_qt<0>(p, x_f16, two_term, s, pdl);
    } else if (wdtype == DT_Q6K) {
        p.row_stride = q6k_row_stride(K);
        e = launch_qt<1>(p, x_f16, two_term, s, pdl);
    } else {
        return cudaErrorInvalidValue;
    }
    if (e == cudaSuccess && launches) (*launches)++;
    return e;
}

// ---- the same GEMM with its scratch in a fixed device array (nothing is allocated) -------------
// The converted activations normally live in a buffer the context grows with cudaMalloc.  Some
// callers cannot do that: a process that has handed all device memory to its own pool, or a
// latency-critical loop in which the device-wide synchronisation of cudaMalloc/cudaFree is not
// acceptable.  For them the scratch below is part of the library image: every GPU that loads the
// library carries these 8 MiB until the process exits, and no call on this path allocates.
constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

size_t gemm_static_scratch_capacity() { return STATIC_SCRATCH_BYTES; }

// Device address of g_static_scratch on `device`, which must be the current device.  In host
// code the array's name is only a handle for the runtime, not a device address, so the address
// is looked up with cudaGetSymbolAddress, once per device, and cached.
static cudaError_t static_scratch_address(int device, void **out) {
    constexpr int MAX_DEVICES = 64;
    static std::mutex lock;
    static void *addr[MAX_DEVICES] = {};
    if (device < 0 || device >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> guard(lock);
    if (!addr[device]) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_static_scratch);
        if (e != cudaSuccess) return e;
        addr[device] = ptr;
    }
    *out = addr[device];
    return cudaSuccess;
}

cudaError_t launch_gemm_static_scratch(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out,
                                       int out_dtype, int K, int N, int M, int device, ErrSink err_word,
                                       cudaStream_t s, uint64_t *launches, bool two_term, bool exact) {
    exact = exact && M <= GEMM_EXACT_MAX_TOKENS;
    if ((exact ? gemm_exact_scratch_bytes(K, M) : gemm_scratch_bytes(K, M)) > STATIC_SCRATCH_BYTES) return cudaErrorInvalidValue;
    void *scratch = nullptr;
    cudaError_t e = static_scratch_address(device, &scratch);
    if (e != cudaSuccess) return e;
    // Nothing in the scratch has to start at zero: the conversion kernel rewrites every f16
    // activation and every token scale the GEMM of this call reads.
    if (exact)
        return launch_gemm_exact(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, scratch, nullptr, 0, err_word, s, launches, nullptr);
    return launch_gemm(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, scratch, nullptr, 0, err_word, s, launches, nullptr, two_term);
}

}  // namespace llmrs
