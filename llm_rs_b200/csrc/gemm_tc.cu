// Prefill matmul (GEMM) for Q4_K / Q6_K weights on the 5th-generation tensor cores of sm_100a.
//
//   Out[M, N] = X[M, K] . W[N, K]^T        (src/backend/mod.rs:29-34; M = seq_len >= 5 here)
//
// Replaces gemm_q4k_pipe / gemm_q6k of the reference (shaders/ops.metal:456-558, 560-621), which
// re-dequantise the weights for every 16 (or 4) tokens.  Here a CTA owns 128 weight rows and up
// to 256 tokens and walks K in stages of 128:
//
//   warps 0-7  dequantise the step's 128 x 64 weight tile straight from global memory (L2) to
//              f16 and store it into TENSOR MEMORY (tcgen05.st; thread = weight row = TMEM lane),
//              where the MMA reads it as its A operand.  Keeping the weights out of shared
//              memory matters: with both operands in shared memory the operand reads plus the
//              tile writes need ~180 B/clk of a 128 B/clk shared memory and the tensor pipe
//              measured 42 % busy.  After the K loop the same warps are the epilogue
//              (TMEM -> registers -> global).
//   warp  8    one lane issues the TMA tensor copy of the step's tokens x 64 f16 activation tile
//              (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill past the last token).
//   warp  9    allocates TMEM; one lane issues tcgen05.mma (kind::f16, f16 x bf16 -> fp32,
//              M=128, N=tokens, K=16, four per step) with the accumulator in TMEM, and
//              tcgen05.commit to hand shared-memory stages back and to publish the accumulator.
//
// Weights are the UMMA "A" operand (rows = TMEM lanes), tokens the "B" operand (columns), so one
// dequantised tile feeds up to 256 tokens.  Both operands are f16, not bf16: with bf16 x bf16 the
// two 8-bit roundings alone measure 2.3e-3 relative L2 on N(0,1) data, above the 2e-3 this path
// is held to; f16's 11-bit significand gives 2.8e-4 at the same tensor-core rate.  Weight values
// are RN_f16 of the exact float32 dequantisation (tests/ops.rs:41-59; shaders/ops.metal:322-334;
// clamped at +-65504, K-quant weights of real models are < 1e2), activations are scaled per
// token by a power of two before RN_f16 (activations_to_f16_kernel), products are exact and
// accumulation is fp32 in the tensor core.
// Every wait is bounded; a wait that gives up reports a KernelError and the CTA still releases
// its TMEM before it exits.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "kernels.h"
#include "llmrs_common.cuh"
#include "pipeline.cuh"

namespace llmrs {

namespace {

constexpr int TILE_ROWS = 128;        // weight rows per CTA = UMMA M
constexpr int BK = 64;                // K elements per stage: 64 f16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int DEQ_WARPS = 8;
constexpr int GEMM_THREADS = (DEQ_WARPS + 2) * 32;

struct GemmParams {
    const uint8_t *W;
    void *Out;
    uint32_t *err;
    int K, N, M;
    int out_bf16;
    size_t row_stride;
    const float *tok_scale;   // per token: factor that undoes the power-of-two scaling of its f16 activations
};

// ---- tcgen05 / TMA wrappers ------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate = 0 overwrites D.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the A operand in tensor memory (lane = row, each 32-bit column = two K-consecutive f16).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// registers -> 32 lanes x 8 (16) consecutive 32-bit TMEM columns
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Arrives on `bar` when all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 16 consecutive fp32 columns of TMEM -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *tmap, int c0, int c1, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled 16-bit tile whose rows are 128
// bytes: start address, leading byte offset 1 (unused with swizzle), stride byte offset 1024
// (8 rows), descriptor version 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// kind::f16 instruction descriptor: D fp32 (bits 4-5 = 1), A and B format f16 (bits 7-9 and 10-12
// = 0; the two must name the same format: f16 x bf16 in one instruction is rejected by the
// hardware as an illegal instruction), both K-major (bits 15, 16 = 0), N >> 3 at bit 17,
// M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Two floats -> packed f16x2 (round to nearest even, clamped to +-65504), first value in the low half.
__device__ __forceinline__ uint32_t pack_w(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Byte q (0..255) of `word` selected by `sel` (0x4440 + byte index pattern) -> float, no I2F.
__device__ __forceinline__ float byte_to_float(uint32_t word, int byte) {
    const uint32_t bits = __byte_perm(word, 0x4B000000u, 0x7440u + (uint32_t)byte);   // 0x4B0000qq
    return __uint_as_float(bits) - 8388608.0f;
}

// 16-byte chunk `c` (0..7) of row `r` inside a 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t swz_off(int r, int c) { return (uint32_t)r * 128u + (uint32_t)((c ^ (r & 7)) << 4); }

// ---- dequantisation of one thread's 32 weights of a K step ---------------------------------------
// The raw bytes of a whole 256-weight block are fetched one block ahead into registers, so the
// global-memory latency of block b+1 hides behind the arithmetic of block b.
// The arithmetic is packed f16x2: a quant byte is dropped into the mantissa of 1024.0 by one
// byte permute (1024 + q, exact), 1024 is subtracted (exact), and one fma applies the scale and
// the minimum.  d*sc and dmin*m are rounded to f16 first, so a weight is RN_f16(q*f16(d*sc) -
// f16(dmin*m)): within 2^-11 relative of the float32 dequantisation.

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
// float -> f16 bits duplicated in both halves (clamped to the finite range).
__device__ __forceinline__ uint32_t h2_dup(float v) { return pack_w(v, v); }

// bytes (b0, b1) resp. (b2, b3) of `bytes4` -> f16x2 (1024 + b, 1024 + b'); bytes must be < 1024.
__device__ __forceinline__ uint32_t magic_lo(uint32_t bytes4) { return __byte_perm(bytes4, 0x64646464u, 0x5140u); }
__device__ __forceinline__ uint32_t magic_hi(uint32_t bytes4) { return __byte_perm(bytes4, 0x64646464u, 0x7362u); }
constexpr uint32_t H2_1024 = 0x64006400u;     // (1024.0, 1024.0)
constexpr uint32_t H2_1056 = 0x64206420u;     // (1056.0, 1056.0) = 1024 + 32

// (lo, hi) f16 halves of `v` broadcast to both halves.
__device__ __forceinline__ uint32_t h2_bcast_lo(uint32_t v) { return __byte_perm(v, 0, 0x1010u); }
__device__ __forceinline__ uint32_t h2_bcast_hi(uint32_t v) { return __byte_perm(v, 0, 0x3232u); }

// Q4_K: thread (row, h16) takes quant bytes 16*h16..16*h16+15 of every pair p: elements
// 16*h16..+15 of sub-block 2p (low nibbles) and of sub-block 2p+1 (high nibbles) (tests/ops.rs:29-59).
struct RawQ4 {
    uint4 hdr;      // f16 d, f16 dmin, 12 packed scale bytes
    uint4 q[4];     // this thread's 16 quant bytes of each pair
};
__device__ __forceinline__ RawQ4 load_raw_q4k(const uint8_t *row_ptr, int b, int h16) {
    const uint8_t *blk = row_ptr + (size_t)b * Q4K_BLOCK_BYTES;
    RawQ4 r;
    r.hdr = ldg128(blk);
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = ldg128(blk + 16 + 32 * i + 16 * h16);
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
// a_taddr: TMEM address (this warp's lane quarter, first column of the stage's weight tile).
template <int P>
__device__ __forceinline__ void dequant_q4k_step(const RawQ4 &raw, const ScalesQ4 &sq, int h16, uint32_t a_taddr) {
    // sub-blocks 2P (low nibbles) and 2P+1 (high nibbles): bytes 2P&3, (2P+1)&3 of word P>>1
    const uint32_t scw = sq.sc[P >> 1], mnw = sq.mn[P >> 1];
    const uint32_t sc2 = h2_sub((P & 1) ? magic_hi(scw) : magic_lo(scw), H2_1024);    // (sc_lo, sc_hi) exact
    const uint32_t mn2 = h2_sub((P & 1) ? magic_hi(mnw) : magic_lo(mnw), H2_1024);
    const uint32_t ds2 = h2_mul(sc2, sq.d_pair);                  // (d*sc_lo, d*sc_hi/16), rounded to f16
    const uint32_t dm2 = h2_mul(mn2, sq.dmin_pair);               // (-dmin*m_lo, -dmin*m_hi)
    const uint32_t s_lo = h2_bcast_lo(ds2), s_hi = h2_bcast_hi(ds2);
    const uint32_t m_lo = h2_bcast_lo(dm2), m_hi = h2_bcast_hi(dm2);
    const uint4 q = raw.q[P];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t l4 = w[j] & 0x0F0F0F0Fu, h4 = w[j] & 0xF0F0F0F0u;
        lo[2 * j] = h2_fma(h2_sub(magic_lo(l4), H2_1024), s_lo, m_lo);
        lo[2 * j + 1] = h2_fma(h2_sub(magic_hi(l4), H2_1024), s_lo, m_lo);
        hi[2 * j] = h2_fma(h2_sub(magic_lo(h4), H2_1024), s_hi, m_hi);
        hi[2 * j + 1] = h2_fma(h2_sub(magic_hi(h4), H2_1024), s_hi, m_hi);
    }
    // k-local positions: low sub-block 16*h16 + i -> columns 8*h16 + i/2; high: 32 + 16*h16 + i
    tmem_st8(a_taddr + 8 * h16, lo);
    tmem_st8(a_taddr + 16 + 8 * h16, hi);
}

// Q6_K (slice-major device layout, kernels.h): in K step 2h+s2 of a block, thread (row, gsel)
// takes scale groups c = 0,1 of g = 2*s2 + gsel in half h (shaders/ops.metal:28-42, 322-334).
// Both steps of a half read the same ql bytes (low nibbles for s2 = 0, high for s2 = 1).
struct RawQ6 {
    uint4 ql[2][2];   // [h][c]: ql run `gsel` of slice (h, c)
    uint4 qh[2][2];   // [h][c]
    uint4 sc;         // 16 int8 scales of the block
    uint32_t d;       // f16 bits
};
__device__ __forceinline__ RawQ6 load_raw_q6k(const uint8_t *row_ptr, int nb, int b, int gsel) {
    const int ci = b >> 4, bl = b & 15;
    const int nbc = min(16, nb - 16 * ci);
    const uint8_t *chunk = row_ptr + (size_t)3360 * ci;
    RawQ6 r;
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const uint8_t *sp = chunk + 48 * (4 * bl + 2 * h + c);
            r.ql[h][c] = ldg128(sp + 16 * gsel);
            r.qh[h][c] = ldg128(sp + 32);
        }
    r.sc = ldg128(chunk + 192 * nbc + 16 * bl);
    r.d = __ldg(reinterpret_cast<const uint16_t *>(chunk + 208 * nbc + 2 * bl));
    return r;
}
template <int P>
__device__ __forceinline__ void dequant_q6k_step(const RawQ6 &raw, int gsel, uint32_t a_taddr) {
    constexpr int h = P >> 1, s2 = P & 1;
    const int g = 2 * s2 + gsel;
    // int8 scales[8h + 4s2 + 2*gsel + c], c = 0,1: (sc + 128) as bytes -> f16 pair -> minus 128 -> times d
    const uint32_t scw = (h ? (s2 ? raw.sc.w : raw.sc.z) : (s2 ? raw.sc.y : raw.sc.x)) ^ 0x80808080u;
    const uint32_t sc2 = h2_sub(gsel ? magic_hi(scw) : magic_lo(scw), 0x64806480u);   // 1024 + 128
    const uint32_t ds2 = h2_mul(sc2, raw.d * 0x00010001u);                            // (d*sc_c0, d*sc_c1)
    uint32_t o[16];
#pragma unroll
    for (int c = 0; c < 2; c++) {
        const uint4 ql = raw.ql[h][c], qh = raw.qh[h][c];
        const uint32_t ds = c ? h2_bcast_hi(ds2) : h2_bcast_lo(ds2);
        const uint32_t lw[4] = {ql.x, ql.y, ql.z, ql.w}, hw[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t lo = (s2 ? (lw[i] >> 4) : lw[i]) & 0x0F0F0F0Fu;
            const uint32_t hi = ((hw[i] >> (2 * g)) & 0x03030303u) << 4;
            const uint32_t q = lo | hi;                                   // four 6-bit quants
            o[8 * c + 2 * i] = h2_mul(h2_sub(magic_lo(q), H2_1056), ds);   // (q - 32) * d*sc
            o[8 * c + 2 * i + 1] = h2_mul(h2_sub(magic_hi(q), H2_1056), ds);
        }
    }
    // k-local positions 32*gsel + 16c + i -> columns 16*gsel + 8c + i/2
    tmem_st16(a_taddr + 16 * gsel, o);
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

template <int TN> struct GemmCfg {
    // A stage is 128 K elements: two 64-wide swizzled activation sub-tiles in shared memory and
    // 64 TMEM columns of weights.  One barrier round per stage keeps the single MMA-issuing
    // thread (which runs at a few cycles per instruction) ahead of the tensor core.
    static constexpr int KSUB = 2;
    static constexpr int STAGE_K = BK * KSUB;
    static constexpr int SUBTILE_BYTES = TN * BK * 2;
    static constexpr int STAGE_BYTES = SUBTILE_BYTES * KSUB;
    static constexpr int STAGES = TN >= 256 ? 3 : 4;
    static constexpr uint32_t A_STAGE_COLS = STAGE_K / 2;            // 64 TMEM columns
    static constexpr uint32_t A_BASE_COL = TN;                       // accumulator in columns [0, TN)
    static constexpr uint32_t TMEM_USED = A_BASE_COL + STAGES * A_STAGE_COLS;
    static constexpr uint32_t TMEM_COLS = TMEM_USED <= 256 ? 256 : 512;
    static_assert(TMEM_USED <= 512, "accumulator and weight stages must fit the 512 TMEM columns");
    static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256;
};

template <int QT, int TN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    using C = GemmCfg<TN>;
    constexpr int S = C::STAGES;
    constexpr uint32_t IDESC = umma_idesc_f16(TN);

    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t *tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles + S * C::STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + S, *acc_full = bars + 2 * S;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TILE_ROWS;          // first weight row of the tile
    const int t0 = blockIdx.y * TN;                 // first token of the tile
    const int nstages = p.K / C::STAGE_K;           // K is a multiple of 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], DEQ_WARPS + 1);     // 8 dequant warps + the TMA thread (with its bytes)
            mbar_init(&empty[s], 1);                // tcgen05.commit
        }
        mbar_init(acc_full, 1);
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
        // ---------------- dequantise the weight tile, stage by stage ----------------
        const int r = threadIdx.x & 127, sel = threadIdx.x >> 7;
        const int row = min(n0 + r, p.N - 1);
        const uint8_t *row_ptr = p.W + (size_t)row * p.row_stride;
        const int nb = p.K / QK_K;
        bool ok = true;
        // TMEM address of this warp's lane quarter, first weight column
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + C::A_BASE_COL;
        // one stage = K steps 2*hb and 2*hb+1 of the block: wait, store 64 f16 weights, hand over
        auto stage = [&](auto hbc, const typename RawOf<QT>::type &raw, const ScalesQ4 &sq, int st) {
            constexpr int HB = decltype(hbc)::value;
            const int s = st % S;
            if (st >= S && !mbar_wait(&empty[s], ((st / S) - 1) & 1)) {
                report_error(p.err, KERR_EMPTY_WAIT);
                ok = false;
                return;
            }
            const uint32_t a_taddr = lane_base + (uint32_t)s * C::A_STAGE_COLS;
            if constexpr (QT == 0) {
                dequant_q4k_step<2 * HB>(raw, sq, sel, a_taddr);
                dequant_q4k_step<2 * HB + 1>(raw, sq, sel, a_taddr + 32);
            } else {
                dequant_q6k_step<2 * HB>(raw, sel, a_taddr);
                dequant_q6k_step<2 * HB + 1>(raw, sel, a_taddr + 32);
            }
            tmem_st_wait();                      // this warp's tensor-memory stores have landed
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        };
        typename RawOf<QT>::type cur = load_raw<QT>(row_ptr, nb, 0, sel);
        for (int b = 0; b < nb && ok; b++) {
            typename RawOf<QT>::type nxt = cur;
            if (b + 1 < nb) nxt = load_raw<QT>(row_ptr, nb, b + 1, sel);     // in flight during this block
            ScalesQ4 sq{};
            if constexpr (QT == 0) sq = unpack_scales_q4k(cur.hdr);
            stage(std::integral_constant<int, 0>{}, cur, sq, 2 * b);
            if (ok) stage(std::integral_constant<int, 1>{}, cur, sq, 2 * b + 1);
            cur = nxt;
        }
        // ---------------- epilogue: TMEM -> registers -> global ----------------
        if (ok && !mbar_wait(acc_full, 0)) {
            report_error(p.err, KERR_MMA_WAIT);
            ok = false;
        }
        if (ok) {
            tc_fence_after();
            const int quarter = warp & 3;                       // TMEM lanes this warp may read
            const int out_row = n0 + 32 * quarter + lane;
            constexpr int COLS_PER_GROUP = TN / 2;              // warps 0-3: first half, 4-7: second half
            const int col_base = (warp >> 2) * COLS_PER_GROUP;
#pragma unroll 1
            for (int c0 = 0; c0 < COLS_PER_GROUP; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(col_base + c0), v);
                tmem_ld_wait();
                if (out_row < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int tok = t0 + col_base + c0 + j;
                        if (tok < p.M) {
                            const size_t idx = (size_t)tok * p.N + out_row;
                            const float val = __uint_as_float(v[j]) * __ldg(p.tok_scale + tok);
                            if (p.out_bf16) ((__nv_bfloat16 *)p.Out)[idx] = __float2bfloat16_rn(val);
                            else ((float *)p.Out)[idx] = val;
                        }
                    }
                }
            }
        }
    } else if (warp == DEQ_WARPS) {
        // ---------------- TMA producer of the activation tiles ----------------
        if (lane == 0) {
            for (int st = 0; st < nstages; st++) {
                const int s = st % S;
                if (st >= S && !mbar_wait(&empty[s], ((st / S) - 1) & 1)) {
                    report_error(p.err, KERR_EMPTY_WAIT);
                    break;
                }
                mbar_arrive_expect_tx(&full[s], C::STAGE_BYTES);
#pragma unroll
                for (int u = 0; u < C::KSUB; u++)
                    tma_load_2d(tiles + s * C::STAGE_BYTES + u * C::SUBTILE_BYTES, &tmap_x,
                                st * C::STAGE_K + u * BK, t0, &full[s]);
            }
        }
    } else {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // Shared-memory descriptors differ only in their start-address field, so the loop adds to
            // the low word of one prebuilt descriptor instead of rebuilding 64-bit values.
            const uint64_t desc0 = umma_desc_sw128(smem_u32(tiles));
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
            const uint32_t desc_lo0 = (uint32_t)desc0;
            const uint32_t a_col0 = tmem_base + C::A_BASE_COL;
            bool ok = true;
            for (int st = 0; st < nstages && ok; st++) {
                const int s = st % S;
                if (!mbar_wait(&full[s], (st / S) & 1)) {
                    report_error(p.err, KERR_FULL_WAIT);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t lo_s = desc_lo0 + (uint32_t)((s * C::STAGE_BYTES) >> 4);
                const uint32_t a_s = a_col0 + (uint32_t)s * C::A_STAGE_COLS;
#pragma unroll
                for (int u = 0; u < C::KSUB; u++)
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; kk++) {
                        // 16 K elements further: 8 TMEM columns of A, 32 bytes inside B's swizzled row
                        const uint32_t lo = lo_s + (uint32_t)((u * C::SUBTILE_BYTES + kk * 32) >> 4);
                        const uint64_t b_desc = ((uint64_t)desc_hi << 32) | lo;
                        umma_f16_ts(tmem_base, a_s + (uint32_t)(u * 32 + kk * 8), b_desc, IDESC,
                                    (st | u | kk) ? 1u : 0u);
                    }
                umma_commit(&empty[s]);            // stage free once these MMAs have read it
            }
            if (ok) umma_commit(acc_full);         // accumulator complete
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
                          float *__restrict__ tok_scale) {
    __shared__ float red[8];
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
    }
    if (threadIdx.x == 0) tok_scale[tok] = exp2i(-e);
}

// ---- host side ---------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

template <int QT, int TN>
cudaError_t launch_tn(const GemmParams &p, const void *x_f16, cudaStream_t s) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
    const cuuint64_t strides[1] = {(cuuint64_t)p.K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)TN};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x_f16), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    constexpr size_t smem = GemmCfg<TN>::SMEM;
    auto kern = gemm_kernel<QT, TN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((p.N + TILE_ROWS - 1) / TILE_ROWS), (unsigned)((p.M + TN - 1) / TN));
    kern<<<grid, GEMM_THREADS, smem, s>>>(tmap, p);
    return cudaGetLastError();
}

template <int QT>
cudaError_t launch_qt(const GemmParams &p, const void *x_f16, cudaStream_t s) {
    if (p.M <= 32) return launch_tn<QT, 32>(p, x_f16, s);
    if (p.M <= 64) return launch_tn<QT, 64>(p, x_f16, s);
    if (p.M <= 128) return launch_tn<QT, 128>(p, x_f16, s);
    return launch_tn<QT, 256>(p, x_f16, s);
}

}  // namespace

// Scratch layout: [M*K f16 activations, rounded up to 256 bytes][M float token scales].
static size_t scratch_x_bytes(int K, int M) { return ((size_t)K * M * 2 + 255) / 256 * 256; }

size_t gemm_scratch_bytes(int K, int M) { return scratch_x_bytes(K, M) + (size_t)M * sizeof(float); }

cudaError_t launch_gemm(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                        int K, int N, int M, void *scratch, uint32_t *err_word, cudaStream_t s, uint64_t *launches) {
    if (K <= 0 || N <= 0 || M <= 0) return cudaSuccess;
    if (!scratch) return cudaErrorInvalidValue;
    __half *x_f16 = (__half *)scratch;
    float *tok_scale = (float *)((uint8_t *)scratch + scratch_x_bytes(K, M));
    activations_to_f16_kernel<<<(unsigned)M, 256, 0, s>>>(x, x_dtype == DT_BF16, K, x_f16, tok_scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) (*launches)++;
    GemmParams p{};
    p.W = w; p.Out = out; p.err = err_word; p.K = K; p.N = N; p.M = M; p.out_bf16 = out_dtype == DT_BF16;
    p.tok_scale = tok_scale;
    if (wdtype == DT_Q4K) {
        p.row_stride = (size_t)(K / QK_K) * Q4K_BLOCK_BYTES;
        e = launch_qt<0>(p, x_f16, s);
    } else if (wdtype == DT_Q6K) {
        p.row_stride = q6k_row_stride(K);
        e = launch_qt<1>(p, x_f16, s);
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
                                       int out_dtype, int K, int N, int M, int device, uint32_t *err_word,
                                       cudaStream_t s, uint64_t *launches) {
    if (gemm_scratch_bytes(K, M) > STATIC_SCRATCH_BYTES) return cudaErrorInvalidValue;
    void *scratch = nullptr;
    cudaError_t e = static_scratch_address(device, &scratch);
    if (e != cudaSuccess) return e;
    // Nothing in the scratch has to start at zero: the conversion kernel rewrites every f16
    // activation and every token scale the GEMM of this call reads.
    return launch_gemm(wdtype, w, x, x_dtype, out, out_dtype, K, N, M, scratch, err_word, s, launches);
}

}  // namespace llmrs
