// Small-batch matmul (5 .. 64 tokens) for Q4_K / Q6_K weights on the 5th-generation tensor cores of
// sm_100a, to the tolerance of the decode kernel (1e-4 relative L2; measured ~1e-6).
//
//   Out[M, N] = X[M, K] . W[N, K]^T        (src/backend/mod.rs:29-34)
//
// Replaces gemm_q4k / gemm_q4k_pipe / gemm_q6k of the reference at these token counts
// (shaders/ops.metal:357-424, 456-558, 560-621).  The idea: keep every factor that the block format
// makes an INTEGER exact in f16, let the tensor core multiply and add those, and apply the one
// factor that is a real number, the block's d, in float32 outside it.
//
//   Q4_K (tests/ops.rs:41-59):  w = d * (sc * q) - dmin * m         sc, m < 64, q < 16
//        A operand = sc * q          (<= 945: exact in f16's 11-bit significand)
//        per 256-weight block b:  acc_b[r, t] = sum_k (sc q)[r, k] * x[t, k]     (tensor core, fp32)
//        out[r, t] = sum_b d[r, b] * acc_b[r, t]  -  sum_{b, sb} (dmin * m)[r, b, sb] * xsum[t, b, sb]
//        The second sum is a small matmul of its own (K / 32 columns): dmin * m is split exactly into
//        two f16 values and rides through the tensor core into a second accumulator.
//   Q6_K (shaders/ops.metal:28-42, 322-334):  w = d * (sc * (q - 32))     sc int8, q < 64
//        sc * (q - 32) has up to 13 bits: A_hi = RN_f16(sc (q - 32)), A_lo = the rounding error
//        (-1, 0 or 1, exact); both go through the tensor core.
//
// Activations are x = x_hi + x_lo, two f16 values (to 2^-22 of the token's largest magnitude), so a
// K step is two (Q4_K) or three (Q6_K: A_lo x_lo is below 2^-22) products.  Nothing is rounded to
// f16 that is not exact there, except x itself at 2^-22.
//
// Pipeline of one CTA (persistent, one per SM, 24 warps in six warpgroups):
//   warp 18     one lane copies the raw blocks of 128 weight rows into a shared-memory ring with tiled
//               TMA copies (cp.async.bulk.tensor.2d on the weight matrix seen as a 2-D byte tensor; no
//               multicast): one 144-byte box per row for Q4_K (rows 144 bytes apart in shared memory,
//               so the 16-byte reads of consecutive rows fall into distinct banks), boxes of 48 / 16
//               bytes per row for the slices, scales and d of Q6_K's slice-major layout.
//   warps 0-15  read their row's bytes from the ring (thread = weight row), build the f16 operand and
//               store it into TENSOR MEMORY (tcgen05.st); up to four groups of four warps take the
//               operand stages (one 128-weight half of a block each) in turn.
//   warp 16     one lane issues the TMA copies of the stage's activation tiles (x_hi, x_lo and, for
//               Q4_K, the per-sub-block sums), 128-byte swizzle.
//   warp 17     allocates TMEM; one lane issues tcgen05.mma (kind::f16, A from TMEM, B from shared
//               memory, fp32 accumulators in TMEM) and the commits.
//   warps 20-23 read the block accumulator out of TMEM after every block (tcgen05.ld), multiply by
//               d[r, b] and add into float32 registers; at the end of a unit they subtract the
//               minimum term, scale by the token factor and write the results (transposed through
//               shared memory: the output is token-major).
// The kernel is launched with programmatic stream serialization: the weight side (warps 0-15, 18) starts
// while the kernel that converts the activations still runs; warps 16 and 20-23 wait for it.
// Work is cut as in the prefill kernel (umma.cuh: Sched): tiles of 128 rows x TN tokens; matrices with
// fewer tiles than SMs are cut along K over all SMs, partial sums meeting in a workspace.
// Every wait is bounded; a wait that gives up reports a KernelError and the CTA still releases its
// TMEM before it exits.
#include <cuda.h>

#include "kernels.h"
#include "llmrs_common.cuh"
#include "pipeline.cuh"
#include "tensor_map.h"
#include "umma.cuh"

namespace llmrs {

namespace {

// Six warpgroups.  Four dequantise: group grp = warp / 4 takes every G-th operand stage (half a block), so up
// to four stages are in work at once and the latencies of one (barrier round trips, shared-memory loads,
// tensor-memory stores) hide behind the arithmetic of the others.  The fifth holds the three single-warp
// roles, the sixth is the epilogue.  Registers move from the fifth group to the sixth at the start.
constexpr int XD_WARPS = 16;                                  // dequantising warps
constexpr int ACT_WARP = XD_WARPS;                            // TMA producer of the activation tiles
constexpr int MMA_WARP = XD_WARPS + 1;
constexpr int RAW_WARP = XD_WARPS + 2;                        // TMA producer of the raw weight blocks
constexpr int EPI_WARP0 = XD_WARPS + 4;                       // warp 19 has no role
constexpr int XQ_WARPS = EPI_WARP0 + EPI_WARPS;               // 24
constexpr int XQ_THREADS = XQ_WARPS * 32;
// The launch bound gives every thread 80 registers; the fifth group drops to 40 and the epilogue takes the
// 4 * 32 * 40 it frees, to 120.  (The pool is the CTA's own allocation: the launcher checks the 80.)
constexpr int REGS_LAUNCH = 80, REGS_SMALL = 40, REGS_EPI = 120;
static_assert(4 * (REGS_SMALL + REGS_EPI) <= 8 * REGS_LAUNCH, "register pool of the CTA");
constexpr int D_RING = 4;                                     // blocks whose d values are kept for the epilogue
constexpr int X_BLOCK_SUBTILES = 10;                          // activation sub-tiles per 256-weight block in the converted layout
constexpr int SHARE_MIN_PIECES = 8;                           // a cut tile in this many pieces or more is summed by all of them

template <int QT, int TN> struct ExactCfg {
    static constexpr bool MIN = QT == 0;                      // Q4_K carries a minimum term
    // Activation tiles of a stage (128 K elements), each TN tokens x 64 f16 with 128-byte swizzled rows.  The
    // x_hi tile of a 64-wide K slice is followed directly by its x_lo tile, so that ONE tensor-core
    // instruction with N = 2 TN columns forms both products of a K step: columns 0..TN-1 of the
    // accumulator take A x_hi, columns TN..2TN-1 take A x_lo.  Q4_K: the sub-block sums (hi tile, lo tile)
    // of the block come with its first stage.
    static constexpr int SUBTILE_BYTES = TN * BK * 2;
    static constexpr int STAGE_SUBTILES = MIN ? 6 : 4;
    static constexpr int STAGE_BYTES = SUBTILE_BYTES * STAGE_SUBTILES;
    static constexpr uint32_t A_TERM_COLS = 64;               // 128 K elements of one term (Q6_K: hi, then lo)
    static constexpr uint32_t A_MAIN_COLS = QT == 0 ? 64 : 128;
    static constexpr uint32_t A_MIN_COLS = MIN ? 8 : 0;       // 16 K slots of the minimum term
    static constexpr uint32_t A_STAGE_COLS = A_MAIN_COLS + A_MIN_COLS;
    // Up to 32 tokens the two products land side by side (one instruction per K step); at 64 tokens both
    // are added into the same TN columns by two instructions, which leaves tensor memory for a third
    // operand stage (the instructions are long enough there for their count not to matter).
    static constexpr bool FUSE = TN <= 32;
    static constexpr uint32_t ACC_BUF_COLS = FUSE ? 2 * TN : TN;   // one block accumulator: A x_hi | A x_lo, or their sum
    static constexpr uint32_t ACC_COLS = 2 * ACC_BUF_COLS;    // two buffers
    static constexpr uint32_t MACC_COLS = MIN ? TN : 0;       // minimum-term accumulator of the unit (one buffer)
    static constexpr uint32_t A_BASE_COL = ACC_COLS + MACC_COLS;
    static constexpr int TMEM_STAGES = (512 - (int)A_BASE_COL) / (int)A_STAGE_COLS;
    // raw ring: one slot = the bytes of one 256-weight block of 128 rows
    static constexpr int Q6_SLICE_BOX = TILE_ROWS * 48;       // one of the four 48-byte slices of a block, all rows
    static constexpr int Q6_SMALL_BOX = TILE_ROWS * 16;       // scales of the block / the 16-byte window holding its d
    static constexpr int RAW_SLOT_BYTES = QT == 0 ? TILE_ROWS * Q4K_BLOCK_BYTES : 4 * Q6_SLICE_BOX + 2 * Q6_SMALL_BOX;
    static_assert(RAW_SLOT_BYTES % 128 == 0, "tiled copies land on 128-byte boundaries");
    static constexpr size_t EPI_BYTES = (size_t)EPI_WARPS * (EPI_TOK * 32 * 4) + (size_t)EPI_WARPS * TN_PAD * 4;
    static constexpr size_t OTHER = 1024 /* alignment slack */ + 512 /* barriers */ + (size_t)D_RING * TILE_ROWS * 4 + EPI_BYTES;
    // stages: what tensor memory holds, what shared memory holds beside two raw slots, four at most
    static constexpr int SMEM_STAGES = (int)((227 * 1024 - OTHER - 2 * (size_t)RAW_SLOT_BYTES) / STAGE_BYTES);
    static constexpr int STAGES = TMEM_STAGES < SMEM_STAGES ? (TMEM_STAGES < 4 ? TMEM_STAGES : 4) : (SMEM_STAGES < 4 ? SMEM_STAGES : 4);
    static_assert(STAGES >= 2, "at least a double buffer");
    static constexpr size_t FIXED = OTHER + (size_t)STAGES * STAGE_BYTES;
    static constexpr int RAW_FIT = (int)((227 * 1024 - FIXED) / RAW_SLOT_BYTES);
    // Slots of the raw ring: as many as fit, up to six (a slot is busy from the issue of its copy, about 1.5 us
    // under load, until both groups have taken its bytes into registers).  GROUPS dequantising groups take
    // the operand stages in turn and each fetches the block of its next stage ahead of time; a group does not
    // visit every fill of a slot, so its parity wait is only right if the fill BEFORE the one it waits for
    // has certainly landed.  That fill belongs to a stage the tensor core has already consumed as long as
    // 2 * slots >= GROUPS + STAGES.
    static constexpr int GROUPS = STAGES < 4 ? STAGES : 4;
    static constexpr int RAW_SLOTS = RAW_FIT < 6 ? RAW_FIT : 6;
    static_assert(RAW_SLOTS >= 2 && 2 * RAW_SLOTS >= GROUPS + STAGES, "raw ring against the groups' look-ahead");
    // every stage belongs to one group (its warps track what they left in the stage's lo columns), and the d
    // values of a block stay in their ring until the epilogue has used them: the dequantisation runs at most
    // STAGES / 2 blocks ahead of the tensor core, which runs at most two blocks ahead of the epilogue
    static_assert(GROUPS == STAGES, "one dequantising group per operand stage");
    static_assert(D_RING >= 2 + (STAGES + 1) / 2, "ring of per-block d values");
    static constexpr size_t SMEM = FIXED + (size_t)RAW_SLOTS * RAW_SLOT_BYTES;
    static constexpr uint32_t TMEM_COLS = 512;
    static_assert(A_BASE_COL + STAGES * A_STAGE_COLS <= 512, "tensor memory budget");
};

struct ExactMaps {
    CUtensorMap w_a[3];  // per weight of the launch: bytes [N rows][row stride], box 144 x 128 (Q4_K) / 48 x 128 (Q6_K)
    CUtensorMap w_b[3];  // Q6_K: box 16 x 128
};

__device__ __forceinline__ uint4 lds128(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }

// registers -> 32 lanes x 8 consecutive 32-bit TMEM columns
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

constexpr uint32_t H2_M1024 = 0xE400E400u;    // (-1024.0, -1024.0)
constexpr uint32_t H2_2M4 = 0x2C002C00u;      // (2^-4, 2^-4)
constexpr uint32_t IDESC_NEG_A = 1u << 13;    // instruction descriptor: negate the A operand

// ---- Q4_K: half-block G of one row -> 64 TMEM columns of sc * q (exact integers) ------------------
// Pair 2G + pr holds sub-block 4G + 2 pr in its low nibbles and 4G + 2 pr + 1 in its high nibbles
// (tests/ops.rs:41-59).  A quant byte is dropped into the mantissa of 1024.0 (1024 + q, exact) and one
// fma takes it to sc * q: (1024 + q) * sc - 1024 * sc.  High nibbles stay in place (16 q) and their
// scale carries the 1/16.  All operands and results are integers below 2048 (or multiples of powers
// of two): nothing is rounded.
template <int G>
__device__ __forceinline__ void dequant_q4k_half_exact(const uint4 &hdr, const uint4 (&q)[4], uint32_t a_taddr) {
    // the six-bit scales of sub-blocks 4G .. 4G+3 as bytes (tests/ops.rs:29-39)
    const uint32_t sc_w = G == 0 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u));
#pragma unroll
    for (int pr = 0; pr < 2; pr++) {
        const uint32_t sc2 = h2_sub(magic_lo(sc_w >> (16 * pr)), H2_1024);       // (sc_even, sc_odd), exact
        const uint32_t s_lo = h2_bcast_lo(sc2);
        const uint32_t s_hi = h2_mul(h2_bcast_hi(sc2), H2_2M4);                  // sc / 16, exact
        const uint32_t c_lo = h2_mul(s_lo, H2_M1024), c_hi = h2_mul(s_hi, H2_M1024);
        const uint4 qa = q[2 * pr], qb = q[2 * pr + 1];
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            // K order inside every four weights is (0, 2, 1, 3) (the conversion kernel lays the activations
            // out the same way): bytes 0 and 2 of a word are already one f16 pair apart, so a nibble becomes
            // the mantissa of 1024.0 by ONE logic operation, and bytes 1 and 3 after one shift
            const uint32_t w8 = w[j] >> 8;
            lo[2 * j] = h2_fma((w[j] & 0x000F000Fu) | H2_1024, s_lo, c_lo);
            lo[2 * j + 1] = h2_fma((w8 & 0x000F000Fu) | H2_1024, s_lo, c_lo);
            hi[2 * j] = h2_fma((w[j] & 0x00F000F0u) | H2_1024, s_hi, c_hi);
            hi[2 * j + 1] = h2_fma((w8 & 0x00F000F0u) | H2_1024, s_hi, c_hi);
        }
        tmem_st16(a_taddr + 32 * pr, lo);
        tmem_st16(a_taddr + 32 * pr + 16, hi);
    }
}

// The minimum term's operand of one block and row: 16 K slots = 8 TMEM columns.  p = dmin * m has 17
// significant bits at most; p_hi = RN_f16(p) and p_lo = p - p_hi (the rounding error of a product, which
// one fma yields exactly) are both f16 values.  Slots 0-7: p_hi of sub-blocks 0-7, slots 8-15: p_lo; the
// sums' tile holds each sub-block's sum in slot sb and again in slot 8 + sb, so one K step of the tensor
// core forms (p_hi + p_lo) * sum.
// Range: |dmin| * 63 must stay below 65504, i.e. |dmin| < 1039 (weights of real models are below 1).
__device__ __forceinline__ void min_operand_q4k(const uint4 &hdr, uint32_t a_taddr) {
    const uint32_t mn[2] = {hdr.z & 0x3F3F3F3Fu, ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u)};
    const uint32_t dmin2 = (hdr.x >> 16) * 0x00010001u;
    uint32_t r[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t m2 = h2_sub(magic_lo(mn[i >> 1] >> (16 * (i & 1))), H2_1024);   // (m[2i], m[2i+1]), exact
        const uint32_t hi = h2_mul(m2, dmin2);
        r[i] = hi;
        r[4 + i] = h2_fma(m2, dmin2, hi ^ 0x80008000u);
    }
    tmem_st8(a_taddr, r);
}

// ---- Q6_K: half h of a block of one row -> 64 hi columns and 64 lo columns -------------------------
// Staged bytes (slice-major layout, kernels.h): slices (h, c = 0, 1), each ql[64h+16c..+16) |
// ql[64h+32+16c..+16) | qh[32h+16c..+16); weight 128h + 32g + 16c + i has its low nibble in ql run
// (g & 1), low half for g < 2 and high half for g >= 2, and bits 2g..2g+1 of qh; its group scale is
// scales[8h + 2g + c] (shaders/ops.metal:28-42, 322-334).  K-local 32g + 16c + i -> column 16g + 8c + i/2
// (with i taken in the order 0, 2, 1, 3 inside every four).
// Per pair of weights: q' = q - 32 (exact), hi = RN_f16(q' sc) (one multiply), and with -sc one fma gives
// hi - q' sc = -lo exactly; the MMA that consumes the lo columns negates its A operand.  The lo terms are
// formed, stored and multiplied only for stages in which some row has a scale above 64 in magnitude.
struct RawQ6Half {
    uint4 ql0[2], ql1[2], qh[2];   // [c]: the two ql runs and the qh run of slice (h, c)
    uint2 sc;                      // int8 scales[8h .. 8h+8)
};
// bytes (0, 2) resp. (1, 3) of a word as the mantissas of (1024.0, 1024.0): the K order (0, 2, 1, 3) inside every
// four weights that the Q4_K operand gets for free (see there) and the conversion kernel gives the activations
__device__ __forceinline__ uint32_t magic_02(uint32_t bytes4) { return __byte_perm(bytes4, 0x64646464u, 0x5240u); }
__device__ __forceinline__ uint32_t magic_13(uint32_t bytes4) { return __byte_perm(bytes4, 0x64646464u, 0x5341u); }
// WITH_LO = false forms and stores the hi columns only: valid when every |sc| of the rows a warp handles is
// at most 64, because then |sc (q - 32)| <= 2048 is exact in f16 and the lo terms are all zero.
template <bool WITH_LO>
__device__ __forceinline__ void dequant_q6k_half_exact(const RawQ6Half &raw, uint32_t a_taddr) {
    const uint2 scw = raw.sc;
    // the eight int8 scales of this half as f16 pairs: (sc + 128) as a byte in the mantissa of 1024, minus 1152
    const uint32_t s01 = scw.x ^ 0x80808080u, s23 = scw.y ^ 0x80808080u;
    constexpr uint32_t H2_1152 = 0x64806480u;
    const uint32_t sp[4] = {h2_sub(magic_lo(s01), H2_1152), h2_sub(magic_hi(s01), H2_1152),
                            h2_sub(magic_lo(s23), H2_1152), h2_sub(magic_hi(s23), H2_1152)};   // (sc[2g], sc[2g+1])
#pragma unroll
    for (int c = 0; c < 2; c++) {
        const uint4 q0 = raw.ql0[c], q1 = raw.ql1[c], qh = raw.qh[c];
        const uint32_t l0[4] = {q0.x, q0.y, q0.z, q0.w}, l1[4] = {q1.x, q1.y, q1.z, q1.w};
        const uint32_t hw[4] = {qh.x, qh.y, qh.z, qh.w};
        uint32_t s2[4], ns2[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            s2[g] = c ? h2_bcast_hi(sp[g]) : h2_bcast_lo(sp[g]);
            ns2[g] = s2[g] ^ 0x80008000u;
        }
        uint32_t hi[4][8], lo[WITH_LO ? 4 : 1][8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // four bytes of 6-bit quants for each of the four groups, 11 logic ops for 16 weights
            const uint32_t qA = hw[i] & 0x33333333u;
            const uint32_t qB = (hw[i] >> 2) & 0x33333333u;
            const uint32_t v[4] = {(l0[i] & 0x0F0F0F0Fu) | ((qA << 4) & 0xF0F0F0F0u),
                                   (l1[i] & 0x0F0F0F0Fu) | ((qB << 4) & 0xF0F0F0F0u),
                                   ((l0[i] >> 4) & 0x0F0F0F0Fu) | (qA & 0xF0F0F0F0u),
                                   ((l1[i] >> 4) & 0x0F0F0F0Fu) | (qB & 0xF0F0F0F0u)};
#pragma unroll
            for (int g = 0; g < 4; g++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const uint32_t q2 = h2_sub(e ? magic_13(v[g]) : magic_02(v[g]), H2_1056);   // (q - 32) pair, K order (0, 2, 1, 3)
                    const uint32_t h = h2_mul(q2, s2[g]);
                    hi[g][2 * i + e] = h;
                    if constexpr (WITH_LO) lo[g][2 * i + e] = h2_fma(q2, ns2[g], h);        // hi - q' sc = -lo
                }
            }
        }
#pragma unroll
        for (int g = 0; g < 4; g++) {
            tmem_st8(a_taddr + 16 * g + 8 * c, hi[g]);
            if constexpr (WITH_LO) tmem_st8(a_taddr + 64 + 16 * g + 8 * c, lo[g]);
        }
    }
}
// Does any of the eight int8 scales exceed 64 in magnitude?  (sc + 64) as an unsigned byte is above 128
// exactly then.
__device__ __forceinline__ bool q6k_scales_need_lo(uint2 sc) {
    return (__vcmpgtu4(__vadd4(sc.x, 0x40404040u), 0x80808080u) | __vcmpgtu4(__vadd4(sc.y, 0x40404040u), 0x80808080u)) != 0u;
}

// ---- the kernel --------------------------------------------------------------------------------
template <int QT, int TN>
__global__ void __launch_bounds__(XQ_THREADS, 1)
gemm_exact_kernel(const __grid_constant__ ExactMaps maps, const GemmParams p) {
    using C = ExactCfg<QT, TN>;
    constexpr int S = C::STAGES;
    constexpr int R = C::RAW_SLOTS;
    constexpr bool MIN = C::MIN;
    constexpr uint32_t IDESC = umma_idesc_f16(TN);

    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t *tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *raw_ring = tiles + S * C::STAGE_BYTES;                              // 1024-byte aligned: the stage sizes are multiples
    uint64_t *bars = reinterpret_cast<uint64_t *>(raw_ring + R * C::RAW_SLOT_BYTES);
    uint64_t *full = bars, *empty = full + S, *raw_full = empty + S, *raw_empty = raw_full + R;
    uint64_t *acc_full = raw_empty + R, *acc_empty = acc_full + 2, *macc_full = acc_empty + 2, *macc_empty = macc_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(macc_empty + 1);          // [0] TMEM base, [2] split ticket
    uint32_t *lo_flag = tmem_slot + 4;                                           // Q6_K: [stage][warp of the group]: any nonzero lo term
    static_assert((2 * S + 2 * R + 6) * 8 + 16 + 4 * 4 * 4 <= 512, "barrier area");
    float *d_ring = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(bars) + 512);   // [D_RING][128]
    uint8_t *epi_stage = reinterpret_cast<uint8_t *>(d_ring + D_RING * TILE_ROWS);
    static_assert(C::STAGE_BYTES % 1024 == 0, "stage images keep the swizzle alignment");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Sched sc = make_sched(p, TN);
    const int w_tiles = sc.w_tiles;

    // Programmatic dependent launch: this kernel may start while the kernel that converts its activations
    // is still running.  Only the warps that touch what earlier kernels wrote (the activation producer
    // and the epilogue) wait for them; the weight producer and the dequantising warps start at once,
    // so the first operand stages are ready when the activations arrive.
    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 4 + 1);               // the 4 warps of one dequantising group + the TMA thread (with its bytes)
            mbar_init(&empty[s], 1);                  // tcgen05.commit
        }
        for (int s = 0; s < R; s++) {
            mbar_init(&raw_full[s], 1);               // the weight TMA thread (with its bytes)
            mbar_init(&raw_empty[s], 8);              // the 8 warps that read a block (one group per half), once its bytes are in registers
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], 1);               // tcgen05.commit after a block's last MMA
            mbar_init(&acc_empty[a], EPI_WARPS);
        }
        mbar_init(macc_full, 1);                      // tcgen05.commit after a unit's last MMA
        mbar_init(macc_empty, EPI_WARPS);
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {                           // the MMA warp owns TMEM
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int nb = p.K / QK_K;

    if (warp < XD_WARPS) {
        // ---------------- raw bytes (shared memory) -> f16 operand (tensor memory) ----------------
        // A thread keeps the raw bytes of its half-block in registers.  The bytes of the group's NEXT stage
        // are fetched from the ring right after the stores of this one have been issued, so that their
        // shared-memory latency, the completion of the stores and the barrier round trip overlap.
        // Group grp takes the stages it = grp, grp + G, grp + 2G, ... (stage it = half (it & 1) of block
        // it / 2).  G is at most the number of stages: a group that skipped more stages than there are
        // could meet a barrier two phases behind it, where a parity wait answers for the wrong phase.
        constexpr int G = C::GROUPS;
        static_assert(G <= XD_WARPS / 4, "one warpgroup per group");
        const int r = threadIdx.x & 127, grp = threadIdx.x >> 7;
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + C::A_BASE_COL;
        bool ok = grp < G;                            // with three stages the fourth group has nothing to do
        // raw bytes of the current block
        uint4 hdr, q[4];                              // Q4_K: header, 64 quant bytes of this half
        RawQ6Half raw6;                               // Q6_K
        uint16_t dbits = 0;
        auto fetch = [&](uint32_t bk, int b_in_row, int g) -> bool {   // half g of block number bk: ring slot -> registers
            const uint32_t rs = bk % R;
            if (!mbar_wait(&raw_full[rs], (bk / R) & 1, p.wait_limit)) {
                report_error(p.err, KERR_FULL_WAIT);
                return false;
            }
            const uint8_t *slot = raw_ring + (size_t)rs * C::RAW_SLOT_BYTES;
            if constexpr (QT == 0) {
                const uint8_t *rowp = slot + (size_t)r * Q4K_BLOCK_BYTES;
                hdr = lds128(rowp);
#pragma unroll
                for (int i = 0; i < 4; i++) q[i] = lds128(rowp + 16 + 64 * g + 16 * i);
            } else {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const uint8_t *sl = slot + (size_t)(2 * g + c) * C::Q6_SLICE_BOX + (size_t)r * 48;
                    raw6.ql0[c] = lds128(sl);
                    raw6.ql1[c] = lds128(sl + 16);
                    raw6.qh[c] = lds128(sl + 32);
                }
                raw6.sc = *reinterpret_cast<const uint2 *>(slot + 4 * C::Q6_SLICE_BOX + (size_t)r * 16 + 8 * g);
                dbits = *reinterpret_cast<const uint16_t *>(slot + 4 * C::Q6_SLICE_BOX + C::Q6_SMALL_BOX + (size_t)r * 16 +
                                                            ((2 * (b_in_row & 15)) & 15));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[rs]);          // the slot may be refilled
            return true;
        };
        // the blocks of this CTA in order (across its units)
        UnitIter ui;
        Unit u;
        bool valid = ui.next(sc, u);
        int b = valid ? u.b0 : 0;
        uint32_t blk = 0;
        auto advance_to = [&](uint32_t target) {      // move to block number target (at most two on)
            while (valid && blk < target) {
                b++;
                blk++;
                if (b >= u.b1) {
                    valid = ui.next(sc, u);
                    b = valid ? u.b0 : 0;
                }
            }
        };
        uint32_t it = (uint32_t)grp;
        uint32_t lo_dirty = (1u << S) - 1u;            // Q6_K: stages whose lo columns this warp has not cleared
        if (ok) {
            advance_to(it >> 1);
            if (valid) ok = fetch(blk, b, (int)(it & 1u));
        }
        while (ok && valid) {
            const uint32_t cur = blk;
            const int g = (int)(it & 1u);
            const uint32_t s = it % S;
            const uint32_t a_taddr = lane_base + s * C::A_STAGE_COLS;
            if (it >= (uint32_t)S && !mbar_wait(&empty[s], ((it / S) - 1) & 1, p.wait_limit)) {
                report_error(p.err, KERR_EMPTY_WAIT);
                break;
            }
            tc_fence_after();
            if constexpr (QT == 0) {
                if (g == 0) {
                    dequant_q4k_half_exact<0>(hdr, q, a_taddr);
                    min_operand_q4k(hdr, a_taddr + C::A_MAIN_COLS);
                    d_ring[(cur % D_RING) * TILE_ROWS + r] = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu));
                } else {
                    dequant_q4k_half_exact<1>(hdr, q, a_taddr);
                }
            } else {
                // The tensor core takes the lo columns of a stage when ANY of its four warps needs them, so a
                // warp that does not must leave zeros there: it clears the columns once after it (or the
                // start of the kernel) left something else in them, and remembers per stage that they are clear.
                const bool any_lo = __any_sync(0xffffffffu, q6k_scales_need_lo(raw6.sc));   // warp-uniform
                if (any_lo) {
                    dequant_q6k_half_exact<true>(raw6, a_taddr);
                    lo_dirty |= 1u << s;
                } else {
                    dequant_q6k_half_exact<false>(raw6, a_taddr);
                    if ((lo_dirty >> s) & 1u) {
                        const uint32_t zeros[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
                        for (int i = 0; i < 8; i++) tmem_st8(a_taddr + C::A_TERM_COLS + 8 * i, zeros);
                        lo_dirty &= ~(1u << s);
                    }
                }
                if (lane == 0) lo_flag[s * 4 + (warp & 3)] = any_lo ? 1u : 0u;
                if (g == 0) d_ring[(cur % D_RING) * TILE_ROWS + r] = f16_bits_to_f32(dbits);
            }
            // the group's next stage, while this one's stores complete
            it += (uint32_t)G;
            advance_to(it >> 1);
            if (valid) ok = fetch(blk, b, (int)(it & 1u));
            tmem_st_wait();                          // this warp's tensor-memory stores have landed
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
    } else if (warp < EPI_WARP0) {
      // registers: this warpgroup gives up what the epilogue's per-token totals need
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SMALL));
      if (warp == ACT_WARP) {
        // ---------------- TMA producer of the activation tiles ----------------
        // (the whole warp walks the loop, the elected lane issues: see the MMA warp)
        const bool leader = elect_one();
        uint32_t it = 0;
        bool ok = true;
        UnitIter ui;
        Unit u;
        pdl_wait();                                   // the converted activations are complete and visible
        while (ok && ui.next(sc, u)) {
            const uint8_t *x_tile = p.x_tiles + (size_t)(u.tile / w_tiles) * nb * X_BLOCK_SUBTILES * C::SUBTILE_BYTES;
            for (int st = 2 * u.b0; st < 2 * u.b1; st++, it++) {
                const uint32_t s = it % S;
                if (it >= (uint32_t)S && !mbar_wait(&empty[s], ((it / S) - 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_EMPTY_WAIT);
                    ok = false;
                    break;
                }
                // The conversion kernel has written the stage as it must lie in shared memory (x_hi and x_lo
                // tiles of both 64-wide K slices, 128-byte swizzled, then the sums of the block with its first
                // half), so one untiled bulk copy brings it: the tiled copies it replaces cost one request per
                // 128-byte row, which at 64 tokens was more than the weights' own.
                const bool with_sums = MIN && (st & 1) == 0;
                const uint32_t bytes = (with_sums ? 6 : 4) * C::SUBTILE_BYTES;
                const uint8_t *src = x_tile + ((size_t)(st >> 1) * X_BLOCK_SUBTILES + (size_t)(st & 1) * 6) * C::SUBTILE_BYTES;
                if (leader) {
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_copy_g2s(tiles + s * C::STAGE_BYTES, src, bytes, &full[s]);
                }
                __syncwarp();
            }
        }
    } else if (warp == RAW_WARP) {
        // ---------------- TMA producer of the raw weight blocks ----------------
        const bool leader = elect_one();
        uint32_t blk = 0;
        bool ok = true;
        UnitIter ui;
        Unit u;
        while (ok && ui.next(sc, u)) {
            const int wt = u.tile % w_tiles;
            const int sg = (wt >= p.seg_tile[1]) + (wt >= p.seg_tile[2]);      // which weight of the launch
            const int n0 = (wt - p.seg_tile[sg]) * TILE_ROWS;
            const CUtensorMap *map_a = &maps.w_a[sg], *map_b = &maps.w_b[sg];
            for (int b = u.b0; b < u.b1; b++, blk++) {
                const uint32_t rs = blk % R;
                if (blk >= (uint32_t)R && !mbar_wait(&raw_empty[rs], ((blk / R) - 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_EMPTY_WAIT);
                    ok = false;
                    break;
                }
                uint8_t *slot = raw_ring + (size_t)rs * C::RAW_SLOT_BYTES;
                if (leader) {
                    mbar_arrive_expect_tx(&raw_full[rs], C::RAW_SLOT_BYTES);
                    if constexpr (QT == 0) {
                        tma_load_2d(slot, map_a, b * Q4K_BLOCK_BYTES, n0, &raw_full[rs]);
                    } else {
                        const int ci = b >> 4, bl = b & 15;
                        const int nbc = min(16, nb - 16 * ci);
                        const int base = 3360 * ci;
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            tma_load_2d(slot + j * C::Q6_SLICE_BOX, map_a, base + 192 * bl + 48 * j, n0, &raw_full[rs]);
                        tma_load_2d(slot + 4 * C::Q6_SLICE_BOX, map_b, base + 192 * nbc + 16 * bl, n0, &raw_full[rs]);
                        tma_load_2d(slot + 4 * C::Q6_SLICE_BOX + C::Q6_SMALL_BOX, map_b,
                                    base + 208 * nbc + ((2 * bl) & ~15), n0, &raw_full[rs]);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == MMA_WARP) {
        // ---------------- MMA issuer ----------------
        // The whole warp walks the schedule and waits on the barriers (warp-uniform control flow, so the
        // descriptors and tensor-memory addresses are formed once per warp); the elected lane issues.
        const bool leader = elect_one();
        const uint64_t desc0 = umma_desc_sw128(smem_u32(tiles));
        const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
        const uint32_t desc_lo0 = (uint32_t)desc0;
        const uint32_t a_col0 = tmem_base + C::A_BASE_COL;
        constexpr uint32_t IDESC2 = umma_idesc_f16(2 * TN);       // A x [x_hi | x_lo]
        bool ok = true;
        uint32_t it = 0, blk = 0, ucount = 0;
        UnitIter ui;
        Unit u;
        for (; ok && ui.next(sc, u); ucount++) {
            // the one minimum-term accumulator: the epilogue must have read the previous unit's out
            if (MIN && ucount >= 1u && !mbar_wait(macc_empty, (ucount - 1) & 1, p.wait_limit)) {
                report_error(p.err, KERR_MMA_WAIT);
                break;
            }
            const uint32_t m_tmem = tmem_base + C::ACC_COLS;
            for (int b = u.b0; b < u.b1 && ok; b++, blk++) {
                const uint32_t ab = blk & 1u;
                // the epilogue must have read this accumulator out (block blk - 2) before it is overwritten
                if (blk >= 2u && !mbar_wait(&acc_empty[ab], ((blk >> 1) - 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_MMA_WAIT);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + ab * C::ACC_BUF_COLS;
#pragma unroll
                for (int half = 0; half < 2; half++, it++) {
                    const uint32_t s = it % S;
                    if (!mbar_wait(&full[s], (it / S) & 1, p.wait_limit)) {
                        report_error(p.err, KERR_FULL_WAIT);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t lo_s = desc_lo0 + ((s * C::STAGE_BYTES) >> 4);
                    const uint32_t a_s = a_col0 + s * C::A_STAGE_COLS;
                    bool need_lo = false;
                    if constexpr (QT == 1)
                        need_lo = (lo_flag[s * 4] | lo_flag[s * 4 + 1] | lo_flag[s * 4 + 2] | lo_flag[s * 4 + 3]) != 0u;
                    if (leader) {
#pragma unroll
                        for (int us = 0; us < 2; us++)
#pragma unroll
                            for (int kk = 0; kk < BK / UMMA_K; kk++) {
                                // 16 K elements further: 8 TMEM columns of A, 32 bytes inside B's swizzled rows
                                const uint32_t lo = lo_s + (uint32_t)((2 * us * C::SUBTILE_BYTES + kk * 32) >> 4);
                                const uint64_t b_desc = ((uint64_t)desc_hi << 32) | lo;
                                const uint32_t a = a_s + (uint32_t)(us * 32 + kk * 8);
                                if constexpr (C::FUSE) {
                                    umma_f16_ts(d_tmem, a, b_desc, IDESC2, (half | us | kk) ? 1u : 0u);
                                } else {                     // x_hi rows, then the x_lo rows one sub-tile further, same columns
                                    umma_f16_ts(d_tmem, a, b_desc, IDESC, (half | us | kk) ? 1u : 0u);
                                    umma_f16_ts(d_tmem, a, b_desc + (uint64_t)(C::SUBTILE_BYTES >> 4), IDESC, 1u);
                                }
                                if constexpr (QT == 1) {     // the lo columns hold -lo: negate A; x_hi rows only
                                    if (need_lo) umma_f16_ts(d_tmem, a + C::A_TERM_COLS, b_desc, IDESC | IDESC_NEG_A, 1u);
                                }
                            }
                        if (MIN && half == 0) {              // (p_hi + p_lo) x sums: hi rows, then lo rows
                            const uint32_t lo = lo_s + (uint32_t)((4 * C::SUBTILE_BYTES) >> 4);
                            umma_f16_ts(m_tmem, a_s + C::A_MAIN_COLS, ((uint64_t)desc_hi << 32) | lo, IDESC, b != u.b0 ? 1u : 0u);
                            umma_f16_ts(m_tmem, a_s + C::A_MAIN_COLS,
                                        ((uint64_t)desc_hi << 32) | (lo + (uint32_t)(C::SUBTILE_BYTES >> 4)), IDESC, 1u);
                        }
                        umma_commit(&empty[s]);            // stage free once these MMAs have read it
                    }
                    __syncwarp();
                }
                if (ok && leader) umma_commit(&acc_full[ab]);   // this block's accumulator is complete
                __syncwarp();
            }
            if (MIN && ok && leader) umma_commit(macc_full);
            __syncwarp();
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_EPI));
        // ---------------- epilogue warps ----------------
        // A thread owns one weight row (its TMEM lane).  After every block it reads the block's
        // accumulator, multiplies by the row's d of that block and adds into its float32 totals; at
        // the end of the unit the minimum term comes off and the totals go out like the prefill
        // kernel's: scaled by the token factor, transposed through a per-warp staging block, written
        // as 16-byte vectors (or deposited / combined when the unit is part of a tile cut along K).
        const int quarter = warp & 3;                           // TMEM lanes this warp may read
        const int ew = warp - EPI_WARP0;
        const int row_in_tile = 32 * quarter + lane;
        uint8_t *stg = epi_stage + (size_t)ew * (EPI_TOK * 32 * 4);       // [EPI_TOK tokens][32 rows]
        float *scale_s = reinterpret_cast<float *>(epi_stage + EPI_WARPS * (EPI_TOK * 32 * 4)) + ew * TN_PAD;
        constexpr int EPI_THREADS = EPI_WARPS * 32;
        uint32_t blk = 0, ucount = 0;
        bool dead = false;
        const bool gather = p.world > 1;
        pdl_wait();                                   // token factors, exchange counters, mailbox step: all from earlier kernels
        const uint32_t gather_step = gather ? *reinterpret_cast<volatile uint32_t *>(p.step_word) + 1u : 0u;
        const uint32_t lane_off = (uint32_t)(32 * quarter) << 16;
        struct Duty { int tt, c_first, pieces, n0, t0, sg; } duty[2];  // the cut tiles this CTA holds a piece of
        int n_duty = 0;
        UnitIter ui;
        Unit u;
        for (; !dead && ui.next(sc, u); ucount++) {
            const int wt = u.tile % w_tiles, t0 = (u.tile / w_tiles) * TN;
            const int sg = (wt >= p.seg_tile[1]) + (wt >= p.seg_tile[2]);      // which weight of the launch
            const int n0 = (wt - p.seg_tile[sg]) * TILE_ROWS;
            const bool partial = u.b1 - u.b0 < sc.nb;
            for (int c = lane; c < TN; c += 32) scale_s[c] = (t0 + c < p.M) ? __ldg(p.tok_scale + t0 + c) : 0.0f;
            __syncwarp();
            float total[TN];
#pragma unroll
            for (int j = 0; j < TN; j++) total[j] = 0.0f;
            for (int b = u.b0; b < u.b1 && !dead; b++, blk++) {
                const uint32_t ab = blk & 1u;
                if (!mbar_wait(&acc_full[ab], (blk >> 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_MMA_WAIT);
                    dead = true;
                    break;
                }
                tc_fence_after();
                const float d = d_ring[(blk % D_RING) * TILE_ROWS + row_in_tile];
                const uint32_t acc = tmem_base + ab * C::ACC_BUF_COLS + lane_off;
#pragma unroll
                for (int c = 0; c < TN / 16; c++) {
                    if constexpr (C::FUSE) {
                        uint32_t vh[16], vl[16];
                        tmem_ld16(acc + 16 * c, vh);              // A x_hi
                        tmem_ld16(acc + TN + 16 * c, vl);         // A x_lo
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            total[16 * c + j] = fmaf(d, __uint_as_float(vh[j]) + __uint_as_float(vl[j]), total[16 * c + j]);
                    } else {
                        uint32_t v[16];
                        tmem_ld16(acc + 16 * c, v);               // A (x_hi + x_lo), summed by the tensor core
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) total[16 * c + j] = fmaf(d, __uint_as_float(v[j]), total[16 * c + j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ab]);
            }
            if (MIN && !dead) {
                if (!mbar_wait(macc_full, ucount & 1, p.wait_limit)) {
                    report_error(p.err, KERR_MMA_WAIT);
                    dead = true;
                } else {
                    tc_fence_after();
                    const uint32_t macc = tmem_base + C::ACC_COLS + lane_off;
#pragma unroll
                    for (int c = 0; c < TN / 16; c++) {
                        uint32_t v[16];
                        tmem_ld16(macc + 16 * c, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) total[16 * c + j] = fmaf(-32.0f, __uint_as_float(v[j]), total[16 * c + j]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(macc_empty);
                }
            }
            if (dead) break;

            // ---- partial unit: a tile cut along K ----
            // Pieces are deposited straight from the registers (token-major, the rows of a warp side by
            // side) and published with one release per CTA.  A tile in few pieces is summed by the CTA
            // that holds its first block: the tile is the last unit of that CTA's range, while the CTAs
            // after it meet the tile first (or have nothing else), so nobody waits long.  From
            // SHARE_MIN_PIECES pieces on the sum is shared out instead: every piece is deposited and, once
            // its own units are done, each of the P CTAs adds up one P-th of the tile over all deposits
            // and writes that part of the output (the duties below), so that no CTA reads P tiles.
            if (partial) {
                const int tt = u.tile - sc.n_full, tb = tt * sc.nb, te = tb + sc.nb;
                const bool is_first = u.b0 == 0;
                int c = (int)blockIdx.x;
                if (!is_first) {                                 // the CTA that holds the tile's first block
                    c = min(sc.gt - 1, (int)(((unsigned)tb * (unsigned)sc.gt) / (unsigned)sc.T));
                    while (c + 1 < sc.gt && tail_start(sc, c + 1) <= tb) c++;
                    while (c > 0 && tail_start(sc, c) > tb) c--;
                }
                const int c_first = c;
                c = (int)blockIdx.x;
                while (c + 1 < sc.gt && tail_start(sc, c + 1) < te) c++;
                const int c_last = c, pieces = c_last - c_first + 1;
                const bool shared_sum = pieces >= SHARE_MIN_PIECES;
                uint32_t *cnt = p.ws_counters + 2 * tt;
                if (!is_first || shared_sum) {
                    const int k = is_first ? 1 : 0;              // a CTA's range starts inside at most one tile and ends inside at most one
                    float *slot = p.ws_slots + (size_t)(2 * blockIdx.x + k) * (TILE_ROWS * TN) + row_in_tile;
#pragma unroll
                    for (int j = 0; j < TN; j++) __stcg(slot + j * TILE_ROWS, total[j]);
                    named_barrier_sync(2, EPI_THREADS);
                    if (ew == 0 && lane == 0) {
                        __threadfence();                         // the deposits of all four warps, device-wide
                        atomicAdd(cnt, 1u);
                    }
                    if (shared_sum) {
                        duty[n_duty].tt = tt; duty[n_duty].c_first = c_first; duty[n_duty].pieces = pieces;
                        duty[n_duty].n0 = n0; duty[n_duty].t0 = t0; duty[n_duty].sg = sg;
                        n_duty++;
                    }
                    continue;
                }
                // this CTA sums the tile: wait for the other pieces, add them, then write like a whole unit
                if (ew == 0 && lane == 0) {
                    bool seen = false;
                    for (uint32_t i = 0; i < p.wait_limit && !seen; i++) {
                        uint32_t n;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(n) : "l"(cnt) : "memory");
                        seen = n + 1u >= (uint32_t)pieces;
                        if (!seen) __nanosleep(32);
                    }
                    if (!seen) report_error(p.err, KERR_SPLIT_WAIT);
                    *cnt = 0;                                    // zero again for the next launch
                }
                named_barrier_sync(2, EPI_THREADS);
                constexpr int PU = TN <= 32 ? 4 : 2;             // pieces whose loads are in flight together
#pragma unroll
                for (int g0 = 0; g0 < TN; g0 += EPI_TOK) {
                    for (int c0 = c_first + 1; c0 <= c_last; c0 += PU) {
                        float add[PU][EPI_TOK];
#pragma unroll
                        for (int q = 0; q < PU; q++) {
                            const float *sa = p.ws_slots + (size_t)(2 * min(c0 + q, c_last)) * (TILE_ROWS * TN) +
                                              (size_t)g0 * TILE_ROWS + row_in_tile;
#pragma unroll
                            for (int j = 0; j < EPI_TOK; j++) add[q][j] = __ldcg(sa + j * TILE_ROWS);
                        }
#pragma unroll
                        for (int q = 0; q < PU; q++)
                            if (c0 + q <= c_last) {
#pragma unroll
                                for (int j = 0; j < EPI_TOK; j++) total[g0 + j] += add[q][j];
                            }
                    }
                }
            }

            // ---- where this unit's values go ----
            const bool o_bf16 = p.out_bf16 != 0;
            const int esz = o_bf16 ? 2 : 4;
            // one weight: rows [row_offset, row_offset + N) of an n_total-row output; several: each its own output
            const bool multi = p.n_seg > 1;
            uint8_t *o_ptr = (uint8_t *)(multi ? p.seg_out[sg] : p.Out);
            const int n_rows = multi ? p.seg_n[sg] : p.N, row_off = multi ? 0 : p.row_offset;
            const size_t o_stride = (size_t)(multi ? n_rows : p.n_total);    // elements between tokens
            const int tok_base = t0, row_base = row_off + n0 + 32 * quarter, tok_lim = p.M, row_lim = row_off + n_rows;
            const bool vec_ok = (o_stride % (size_t)(16 / esz)) == 0;
#pragma unroll
            for (int g0 = 0; g0 < TN; g0 += EPI_TOK) {
#pragma unroll
                for (int j = 0; j < EPI_TOK; j++) {
                    const float val = total[g0 + j] * scale_s[g0 + j];
                    if (o_bf16) reinterpret_cast<__nv_bfloat16 *>(stg)[j * 32 + lane] = __float2bfloat16_rn(val);
                    else reinterpret_cast<float *>(stg)[j * 32 + lane] = val;
                }
                __syncwarp();
                // ---- staging -> global ----
                if (vec_ok) {
                    const int vec_per_tok = 32 * esz / 16;       // 4 (bf16) or 8 (fp32) vectors per token
                    const int rows_per_vec = 16 / esz;
                    for (int i = lane; i < EPI_TOK * vec_per_tok; i += 32) {
                        const int tl = i / vec_per_tok, vv = i % vec_per_tok;
                        const int tok = tok_base + g0 + tl, row = row_base + vv * rows_per_vec;
                        if (tok < tok_lim && row < row_lim) {
                            const uint4 dv = *reinterpret_cast<const uint4 *>(stg + (size_t)tl * 32 * esz + vv * 16);
                            *reinterpret_cast<uint4 *>(o_ptr + ((size_t)tok * o_stride + row) * esz) = dv;
                        }
                    }
                } else {
                    for (int tl = 0; tl < EPI_TOK; tl++) {
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
                    for (int tl = 0; tl < EPI_TOK; tl++) {
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
        }
        // ---- duties: this CTA's share of the sums of the cut tiles it holds a piece of ----
        for (int di = 0; di < n_duty && !dead; di++) {
            const Duty dy = duty[di];
            uint32_t *cnt = p.ws_counters + 2 * dy.tt;
            if (ew == 0 && lane == 0) {
                bool seen = false;
                for (uint32_t i = 0; i < p.wait_limit && !seen; i++) {
                    uint32_t n;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(n) : "l"(cnt) : "memory");
                    seen = n >= (uint32_t)dy.pieces;
                    if (!seen) __nanosleep(32);
                }
                if (!seen) report_error(p.err, KERR_SPLIT_WAIT);
            }
            named_barrier_sync(2, EPI_THREADS);
            // the tile as TN * 32 groups of four rows; piece q of P takes groups [q * tot / P, (q + 1) * tot / P)
            constexpr int TOT = TN * (TILE_ROWS / 4);
            const int q = (int)blockIdx.x - dy.c_first;
            const int e_lo = (int)(((long long)q * TOT) / dy.pieces), e_hi = (int)(((long long)(q + 1) * TOT) / dy.pieces);
            const bool o_bf16 = p.out_bf16 != 0;
            const bool multi = p.n_seg > 1;
            void *o_base = multi ? p.seg_out[dy.sg] : p.Out;
            const int n_rows = multi ? p.seg_n[dy.sg] : p.N, row_off = multi ? 0 : p.row_offset;
            const int n_tot = multi ? n_rows : p.n_total;
            const bool vec_ok = (n_tot & 3) == 0 && (row_off & 3) == 0;
            for (int e = e_lo + ew * 32 + lane; e < e_hi; e += EPI_THREADS) {
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int c0 = 0; c0 < dy.pieces; c0 += 4) {
                    float4 v[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int c = dy.c_first + min(c0 + i, dy.pieces - 1);
                        const int k = c == dy.c_first ? 1 : 0;   // the first piece is the end of its CTA's range
                        v[i] = __ldcg(reinterpret_cast<const float4 *>(p.ws_slots + (size_t)(2 * c + k) * (TILE_ROWS * TN)) + e);
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        if (c0 + i < dy.pieces) { acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w; }
                }
                const int tok = dy.t0 + e / (TILE_ROWS / 4), row = row_off + dy.n0 + 4 * (e % (TILE_ROWS / 4));
                if (tok >= p.M || row >= row_off + n_rows) continue;
                const float ts = __ldg(p.tok_scale + tok);
                float f[4] = {acc.x * ts, acc.y * ts, acc.z * ts, acc.w * ts};
                const int nv = min(4, row_off + n_rows - row);
                const size_t o = (size_t)tok * n_tot + row;
                if (o_bf16) {
                    __nv_bfloat16 hb[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        hb[i] = __float2bfloat16_rn(f[i]);
                        f[i] = __bfloat162float(hb[i]);          // what the peers get is what this rank stores
                    }
                    if (vec_ok && nv == 4) {
                        *reinterpret_cast<uint2 *>((__nv_bfloat16 *)o_base + o) = *reinterpret_cast<const uint2 *>(hb);
                    } else {
                        for (int i = 0; i < nv; i++) ((__nv_bfloat16 *)o_base)[o + i] = hb[i];
                    }
                } else {
                    if (vec_ok && nv == 4) {
                        *reinterpret_cast<float4 *>((float *)o_base + o) = make_float4(f[0], f[1], f[2], f[3]);
                    } else {
                        for (int i = 0; i < nv; i++) ((float *)o_base)[o + i] = f[i];
                    }
                }
                if (gather) {                                    // the same values, as words, to every peer's mailbox
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
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- activations -> stage images of (x_hi, x_lo) f16 pairs, token factors and sub-block sums --------
// One CTA per token of the padded token range (whole tiles of TN tokens; the padding rows are zeros).
// The token row is multiplied by a power of two that brings its largest magnitude to [2^13, 2^14);
// x_hi = RN_f16(x * 2^e), x_lo = RN_f16(x * 2^e - x_hi); the inverse factor goes to tok_scale[token].
// The output is laid out as the matmul kernel's shared-memory stages, so that a stage is one contiguous
// piece: per token tile, per 256-weight block, X_BLOCK_SUBTILES sub-tiles of [TN rows][64 f16] with the
// 16-byte pieces of a row XOR-swizzled by (row & 7) (the 128-byte swizzle of the tensor-core descriptor):
//   0..3  x_hi, x_lo of K slice 0, x_hi, x_lo of K slice 1      (first half of the block)
//   4, 5  the sums of every 32 consecutive scaled values (what Q4_K's minimum multiplies), divided by 32 so
//         that they stay below 2^14, as hi and lo f16 parts: the sum of sub-block sb in element sb and again
//         in element 8 + sb (the order min_operand_q4k expects; the tensor core reads those 16 only)
//   6..9  x_hi, x_lo of K slice 2, x_hi, x_lo of K slice 3      (second half)
// The block size is chosen so that a thread holds at most ACT_KEEP 8-value pieces of the row, which then
// stay in registers between the maximum and the conversion (longer rows are read again, from L1/L2).
constexpr int ACT_KEEP = 2;
__global__ void __launch_bounds__(1024)
activations_exact_kernel(const void *__restrict__ x, int x_is_bf16, int K, int M, int TN, uint8_t *__restrict__ out,
                         int with_sums, float *__restrict__ tok_scale, const float *__restrict__ norm_w, float norm_eps) {
    __shared__ float red[32];
    pdl_prologue();                  // the next kernel may start its prologue; the input is complete from here on
    const int tok = blockIdx.x;
    const bool padding = tok >= M;
    const size_t base = (size_t)tok * K;
    const int nb = K / QK_K;
    const int sub_bytes = TN * 128;
    const int j = tok % TN;
    uint8_t *tile = out + (size_t)(tok / TN) * nb * X_BLOCK_SUBTILES * sub_bytes + (size_t)j * 128;
    const int sw = j & 7;
    auto load8 = [&](int k, float (&v)[8]) {
        if (padding) {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.0f;
        } else if (x_is_bf16) {
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
    const int step = (int)blockDim.x * 8;
    const int n_warps = (int)(blockDim.x >> 5);
    auto block_reduce = [&](float v, bool is_max) {   // every thread gets the block's sum or maximum
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, v, o);
            v = is_max ? fmaxf(v, other) : v + other;
        }
        __syncthreads();                              // the previous reduction's readers are done
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        v = (int)(threadIdx.x & 31) < n_warps ? red[threadIdx.x & 31] : (is_max ? 0.0f : 0.0f);
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, v, o);
            v = is_max ? fmaxf(v, other) : v + other;
        }
        return v;
    };
    // An rms_norm folded into the conversion (rms_norm_matmul* above four tokens): the row is multiplied by
    // rsqrt(mean(x^2) + eps) * w before it is split, in float32 like the reference's kernel
    // (shaders/ops.metal rms_norm), without the rounding to the activation type in between.
    auto scale8 = [&](int k, float (&v)[8], float inv_rms) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(norm_w + k)), b = __ldg(reinterpret_cast<const float4 *>(norm_w + k + 4));
        const float w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = v[i] * inv_rms * w[i];
    };
    float keep[ACT_KEEP][8];
    float inv_rms = 1.0f;
#pragma unroll
    for (int jj = 0; jj < ACT_KEEP; jj++) {
        const int k = (int)threadIdx.x * 8 + jj * step;
        if (k < K) load8(k, keep[jj]);
    }
    if (norm_w) {
        float ss = 0.0f;
#pragma unroll
        for (int jj = 0; jj < ACT_KEEP; jj++) {
            const int k = (int)threadIdx.x * 8 + jj * step;
            if (k < K) {
#pragma unroll
                for (int i = 0; i < 8; i++) ss = fmaf(keep[jj][i], keep[jj][i], ss);
            }
        }
        for (int k = (int)threadIdx.x * 8 + ACT_KEEP * step; k < K; k += step) {
            float v[8];
            load8(k, v);
#pragma unroll
            for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
        }
        inv_rms = rsqrtf(block_reduce(ss, false) / (float)K + norm_eps);
#pragma unroll
        for (int jj = 0; jj < ACT_KEEP; jj++) {
            const int k = (int)threadIdx.x * 8 + jj * step;
            if (k < K) scale8(k, keep[jj], inv_rms);
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int jj = 0; jj < ACT_KEEP; jj++) {
        const int k = (int)threadIdx.x * 8 + jj * step;
        if (k < K) {
#pragma unroll
            for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(keep[jj][i]));
        }
    }
    for (int k = (int)threadIdx.x * 8 + ACT_KEEP * step; k < K; k += step) {
        float v[8];
        load8(k, v);
        if (norm_w) scale8(k, v, inv_rms);
#pragma unroll
        for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = block_reduce(amax, true);
    const int eb = (int)((__float_as_uint(amax) >> 23) & 0xFFu);
    int e = 140 - eb;                                    // amax < 2^(eb-126): the scaled row stays below 2^14
    e = max(-126, min(126, e));
    if (amax == 0.0f || eb == 255) e = 0;                // all-zero row, or inf/nan: leave as is
    const float sc = exp2i(e);
    auto convert = [&](int k, const float (&v)[8]) {
        uint32_t h[4], l[4];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // f16 pairs in the operand's K order (0, 2, 1, 3) inside every four values
            const int ia = 4 * (i >> 1) + (i & 1), ib = ia + 2;
            const float a = v[ia] * sc, b = v[ib] * sc;
            h[i] = pack_w(a, b);
            const float2 back = __half22float2(*reinterpret_cast<const __half2 *>(&h[i]));
            l[i] = pack_w(a - back.x, b - back.y);
            const float2 lowf = __half22float2(*reinterpret_cast<const __half2 *>(&l[i]));
            sum += (back.x + lowf.x) + (back.y + lowf.y);          // what the tensor core will see
        }
        // block, half of the block, 64-wide K slice of the half, 16-byte piece of the slice's 128-byte row
        const int blk = k >> 8, half = (k >> 7) & 1, us = (k >> 6) & 1, c = (k >> 3) & 7;
        uint8_t *blockp = tile + (size_t)blk * X_BLOCK_SUBTILES * sub_bytes;
        uint8_t *dst = blockp + (size_t)(half * 6 + 2 * us) * sub_bytes + ((c ^ sw) << 4);
        *reinterpret_cast<uint4 *>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4 *>(dst + sub_bytes) = make_uint4(l[0], l[1], l[2], l[3]);
        if (with_sums) {
            // four consecutive threads hold one sub-block of 32 values (the block size is a multiple of 32)
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((threadIdx.x & 3) == 0) {
                const int sb = (k >> 5) & 7;
                const float s32 = sum * 0.03125f;
                const __half hi = __float2half_rn(s32);
                const __half lo = __float2half_rn(s32 - __half2float(hi));
                __half *row_hi = reinterpret_cast<__half *>(blockp + (size_t)4 * sub_bytes);
                __half *row_lo = reinterpret_cast<__half *>(blockp + (size_t)5 * sub_bytes);
                const int e0 = ((0 ^ sw) << 3) + sb, e1 = ((1 ^ sw) << 3) + sb;      // f16 index inside the row
                row_hi[e0] = hi;
                row_hi[e1] = hi;
                row_lo[e0] = lo;
                row_lo[e1] = lo;
            }
        }
    };
    // K is a multiple of 256 and the block a multiple of 32 threads: a warp is inside the row or outside
    // it as a whole, so the shuffles above always see full warps.
#pragma unroll
    for (int jj = 0; jj < ACT_KEEP; jj++) {
        const int k = (int)threadIdx.x * 8 + jj * step;
        if (k < K) convert(k, keep[jj]);
    }
    for (int k = (int)threadIdx.x * 8 + ACT_KEEP * step; k < K; k += step) {
        float v[8];
        load8(k, v);
        if (norm_w) scale8(k, v, inv_rms);
        convert(k, v);
    }
    if (threadIdx.x == 0 && !padding) tok_scale[tok] = exp2i(-e);
}

// ---- host side ---------------------------------------------------------------------------------

struct ExactWeights {            // the weights of one launch (one format, one K)
    int n;
    const uint8_t *w[3];
    int rows[3];
};

int exact_tn(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }
// the converted activations: whole token tiles, X_BLOCK_SUBTILES sub-tiles of TN x 128 bytes per block
size_t exact_x_bytes(int K, int M) {
    const int tn = exact_tn(M);
    const size_t m_pad = (size_t)(M + tn - 1) / tn * tn;
    return (m_pad * (size_t)(K / QK_K) * X_BLOCK_SUBTILES * 128 + 255) / 256 * 256;
}

template <int QT, int TN>
cudaError_t launch_exact_tn(const GemmParams &p, const ExactWeights &ws, int split_mode, cudaStream_t s, bool pdl) {
    using C = ExactCfg<QT, TN>;
    ExactMaps maps;
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < 3; i++) {
        const int k = i < ws.n ? i : 0;               // unused entries repeat the first weight's maps
        if (QT == 0) {
            e = encode_2d(&maps.w_a[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, ws.w[k], (uint64_t)p.row_stride, (uint64_t)ws.rows[k],
                          (uint64_t)p.row_stride, Q4K_BLOCK_BYTES, TILE_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
            if (e != cudaSuccess) return e;
            maps.w_b[i] = maps.w_a[i];
        } else {
            e = encode_2d(&maps.w_a[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, ws.w[k], (uint64_t)p.row_stride, (uint64_t)ws.rows[k],
                          (uint64_t)p.row_stride, 48, TILE_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
            if (e != cudaSuccess) return e;
            e = encode_2d(&maps.w_b[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, ws.w[k], (uint64_t)p.row_stride, (uint64_t)ws.rows[k],
                          (uint64_t)p.row_stride, 16, TILE_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
            if (e != cudaSuccess) return e;
        }
    }
    auto kern = gemm_exact_kernel<QT, TN>;
    static bool smem_set[64] = {};                    // per instantiation and device: the attribute is kept by the function
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !smem_set[dev]) {
        // the epilogue's register increase is served from the CTA's own allocation and would wait for ever
        // if the kernel had been built with fewer registers per thread than the split assumes
        cudaFuncAttributes fa;
        e = cudaFuncGetAttributes(&fa, kern);
        if (e != cudaSuccess) return e;
        if (fa.numRegs < REGS_LAUNCH) return cudaErrorInvalidConfiguration;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) smem_set[dev] = true;
    }
    const int nb = p.K / QK_K;
    const int n_tiles = ((p.N + TILE_ROWS - 1) / TILE_ROWS) * ((p.M + TN - 1) / TN);
    int grid = n_tiles < p.sm_count ? n_tiles : p.sm_count;
    GemmParams q = p;
    q.split = 0;
    // Cutting the last, partial wave of tiles along K: every SM then streams its share of the weights
    // (a whole small matrix, or the tail of a large one).  The exchange is one tile-sized float32 deposit
    // per piece, at most 32 KB at these token counts, so it is used whenever there is a partial wave and
    // there are K blocks to share out.
    const int rest = n_tiles % p.sm_count;
    const bool want = split_mode > 0 || (split_mode < 0 && rest != 0 && nb >= 4);
    if (p.ws_slots && want && rest != 0 && nb >= 2) {
        q.split = 1;
        const int tail_blocks = rest * nb;
        if (n_tiles < p.sm_count) grid = tail_blocks < p.sm_count ? tail_blocks : p.sm_count;
    }
    if (q.world > 1) grid = p.sm_count;      // CTAs without a tile still take their share of the mailbox
    return launch_dependent(kern, dim3((unsigned)grid), dim3(XQ_THREADS), (size_t)C::SMEM, s, pdl, maps, q);
}

template <int QT>
cudaError_t launch_exact_qt(const GemmParams &p, const ExactWeights &ws, int split_mode, cudaStream_t s, bool pdl) {
    if (p.M <= 16) return launch_exact_tn<QT, 16>(p, ws, split_mode, s, pdl);
    if (p.M <= 32) return launch_exact_tn<QT, 32>(p, ws, split_mode, s, pdl);
    return launch_exact_tn<QT, 64>(p, ws, split_mode, s, pdl);
}

}  // namespace

// Scratch layout: [converted activations, see activations_exact_kernel][M float token factors].
size_t gemm_exact_scratch_bytes(int K, int M) {
    return exact_x_bytes(K, M) + (size_t)M * sizeof(float);
}

static cudaError_t launch_exact_common(int wdtype, int nw, const uint8_t *const *ws, const int *ns, void *const *outs,
                                       const void *x, int x_dtype, int out_dtype, int K, int M, void *scratch,
                                       void *split_ws, int split_mode, ErrSink err_word, cudaStream_t s,
                                       uint64_t *launches, const GemmGather *gather, bool pdl, int sm_count,
                                       int acts_mode, const float *norm_w, float norm_eps) {
    if (nw < 1 || nw > 3) return cudaErrorInvalidValue;
    if (K <= 0 || M <= 0) return cudaSuccess;
    for (int i = 0; i < nw; i++)
        if (ns[i] <= 0) return nw == 1 ? cudaSuccess : cudaErrorInvalidValue;
    if (!scratch || M > GEMM_EXACT_MAX_TOKENS || K % QK_K) return cudaErrorInvalidValue;
    if (wdtype != DT_Q4K && wdtype != DT_Q6K) return cudaErrorInvalidValue;
    if (nw > 1 && gather && gather->world > 1) return cudaErrorInvalidValue;
    uint8_t *sb = (uint8_t *)scratch;
    float *tok_scale = (float *)(sb + exact_x_bytes(K, M));
    const int tn = exact_tn(M), m_pad = (M + tn - 1) / tn * tn;
    cudaError_t e = cudaSuccess;
    if (acts_mode != EXACT_ACTS_REUSE) {
        // one CTA per token, at most ACT_KEEP 8-value pieces per thread up to 16384-element rows
        int act_threads = ((K / 8 + ACT_KEEP - 1) / ACT_KEEP + 31) / 32 * 32;
        act_threads = act_threads < 64 ? 64 : act_threads > 1024 ? 1024 : act_threads;
        const bool sums = wdtype == DT_Q4K || acts_mode == EXACT_ACTS_CONVERT_ALL;
        e = launch_dependent(activations_exact_kernel, dim3((unsigned)m_pad), dim3((unsigned)act_threads), 0, s, pdl,
                             x, (int)(x_dtype == DT_BF16), K, M, tn, sb, (int)sums, tok_scale, norm_w, norm_eps);
        if (e != cudaSuccess) return e;
        if (launches) (*launches)++;
    }
    GemmParams p{};
    ExactWeights ew{};
    ew.n = nw;
    int tiles = 0;
    p.n_seg = nw;
    for (int i = 0; i < 4; i++) p.seg_tile[i] = 0x7fffffff;
    for (int i = 0; i < nw; i++) {
        ew.w[i] = ws[i];
        ew.rows[i] = ns[i];
        p.seg_tile[i] = tiles;
        p.seg_n[i] = ns[i];
        p.seg_out[i] = outs[i];
        tiles += (ns[i] + TILE_ROWS - 1) / TILE_ROWS;
    }
    const int N = nw == 1 ? ns[0] : tiles * TILE_ROWS;      // several weights: the tile space, each weight from a tile boundary
    p.W = ws[0]; p.Out = outs[0]; p.err = err_word.word; p.wait_limit = err_word.mbar_polls; p.gather_limit = err_word.gather_polls;
    p.K = K; p.N = N; p.M = M; p.out_bf16 = out_dtype == DT_BF16;
    p.tok_scale = tok_scale;
    p.x_tiles = sb;
    p.n_total = N;
    if (gather && gather->world > 1) {
        p.world = gather->world; p.rank = gather->rank; p.n_total = N * gather->world; p.row_offset = gather->rank * N;
        p.done_counter = gather->done_counter; p.step_word = gather->step_word;
        p.half_words = (size_t)gather->world * M * N;
        for (int d = 0; d < gather->world; d++) p.peer_box[d] = (uint2 *)gather->peer_mailbox[d];
    }
    p.sm_count = sm_count;
    if (p.sm_count <= 0) {
        int dev = 0;
        e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&p.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
    }
    if (split_ws && 2 * p.sm_count * sizeof(uint32_t) <= gemm_split_counter_bytes()) {
        p.ws_counters = (uint32_t *)split_ws;
        p.ws_slots = (float *)((uint8_t *)split_ws + gemm_split_counter_bytes());
    }
    if (wdtype == DT_Q4K) {
        p.row_stride = (size_t)(K / QK_K) * Q4K_BLOCK_BYTES;
        e = launch_exact_qt<0>(p, ew, split_mode, s, pdl);
    } else {
        p.row_stride = q6k_row_stride(K);
        e = launch_exact_qt<1>(p, ew, split_mode, s, pdl);
    }
    if (e == cudaSuccess && launches) (*launches)++;
    return e;
}

cudaError_t launch_gemm_exact(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                              int K, int N, int M, void *scratch, void *split_ws, int split_mode, ErrSink err_word,
                              cudaStream_t s, uint64_t *launches, const GemmGather *gather, bool pdl, int sm_count,
                              int acts_mode, const float *norm_w, float norm_eps) {
    return launch_exact_common(wdtype, 1, &w, &N, &out, x, x_dtype, out_dtype, K, M, scratch, split_ws, split_mode,
                               err_word, s, launches, gather, pdl, sm_count, acts_mode, norm_w, norm_eps);
}

cudaError_t launch_gemm_exact_multi(int wdtype, int nw, const uint8_t *const *ws, const int *ns, void *const *outs,
                                    const void *x, int x_dtype, int out_dtype, int K, int M, void *scratch,
                                    void *split_ws, int split_mode, ErrSink err_word, cudaStream_t s, uint64_t *launches,
                                    bool pdl, int sm_count, const float *norm_w, float norm_eps) {
    return launch_exact_common(wdtype, nw, ws, ns, outs, x, x_dtype, out_dtype, K, M, scratch, split_ws, split_mode,
                               err_word, s, launches, nullptr, pdl, sm_count, EXACT_ACTS_CONVERT, norm_w, norm_eps);
}

}  // namespace llmrs
