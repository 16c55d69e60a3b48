// tcgen05 / tensor-memory building blocks shared by the tensor-core matmul kernels of sm_100a: the
// work schedule (tiles, split of the last wave), thin wrappers around the PTX instructions, the
// shared-memory and instruction descriptors, and the packed-f16 helpers of the dequantisation.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "llmrs_common.cuh"
#include "pipeline.cuh"

namespace llmrs {

constexpr int TILE_ROWS = 128;        // weight rows per CTA = UMMA M
constexpr int BK = 64;                // K elements per stage: 64 f16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int DEQ_WARPS = 8;
constexpr int EPI_WARPS = 4;
constexpr int EPI_TOK = 16;           // tokens an epilogue warp transposes at a time
constexpr int TN_PAD = 256;           // floats reserved per epilogue warp for the tile's token factors
constexpr int GEMM_THREADS = (DEQ_WARPS + 2 + EPI_WARPS) * 32;

struct GemmParams {
    const uint8_t *W;
    void *Out;
    uint32_t *err;
    uint32_t wait_limit, gather_limit;   // polls before an mbarrier (or partial-sum) wait / a mailbox wait is abandoned
    int K, N, M;
    int out_bf16;
    int sm_count;
    size_t row_stride;
    const float *tok_scale;   // per token: factor that undoes the power-of-two scaling of its f16 activations
    const uint8_t *x_tiles;   // small-batch kernel: the activations as ready-made shared-memory stage images
    // Split of the last, partial wave of tiles along K (kernel: 0 = off; host: -1 = estimate decides), see Sched below.
    int split;
    uint32_t *ws_counters;    // [2 * sm_count] zero between launches: arrivals / deposits per tail tile
    float *ws_slots;          // [2 * sm_count] partial tiles of TILE_ROWS x TN floats, token-major
    // Fused all-gather of an N-sharded matmul (world > 1), the protocol of the decode kernel: this
    // rank's rows are rows [row_offset, row_offset + N) of an n_total-row output; every result is
    // stored locally and posted to each peer as one 8-byte word {value as float bits, call number}
    // in that peer's mailbox ([2 halves][world senders][M][N] words); before the kernel ends its
    // epilogue warps copy the words addressed to this rank into the local output, polling (bounded)
    // until each carries this call's number.  No fences, no flags.
    uint2 *peer_box[8];
    uint32_t *done_counter, *step_word;
    size_t half_words;
    int world, rank, n_total, row_offset;
    // Small-batch kernel, several weights of one format and K multiplied with one input in one launch
    // (n_seg > 1; no all-gather then): weight i owns the row tiles [seg_tile[i], seg_tile[i + 1]) of the
    // launch's tile space, has seg_n[i] rows and writes to seg_out[i] ([M][seg_n[i]]).  N is then
    // 128 x the number of row tiles.
    int n_seg;
    int seg_tile[4];
    int seg_n[3];
    void *seg_out[3];
};

// ---- work schedule -----------------------------------------------------------------------------
// A unit is a tile (128 weight rows x TN tokens) and a range of its 256-weight K blocks.  Without
// the split, CTA c owns the whole tiles c, c + G, ...  (G = grid size).  With it, every CTA owns
// n_tiles / G whole tiles, and the K blocks of the remaining R = n_tiles % G tiles -- the wave
// that would leave most SMs idle -- form one sequence of T = R * nb blocks that is cut into G
// equal contiguous ranges ("stream-K").  A range that covers only part of a tile yields a partial
// accumulator: every CTA but the last to arrive deposits its partial in a workspace slot, the
// last one adds the deposits to its own accumulator and writes the output.  The last arriver
// waits only for CTAs that have already taken a ticket, i.e. are running their epilogue, so the
// wait can not deadlock whatever else shares the GPU; it is bounded all the same.
struct Sched {
    int nb, w_tiles, n_tiles;
    int full_per_cta, n_full;       // whole tiles of this CTA; tiles [0, n_full) are done whole
    int T, gt;                      // tail: T blocks over the first gt CTAs
    int tail_a, tail_b;             // this CTA's range of tail blocks
};
struct Unit {
    int tile, b0, b1;
};
__device__ __forceinline__ int tail_start(const Sched &sc, int c) {      // first tail block of CTA c (c <= gt)
    return (int)(((unsigned)sc.T * (unsigned)c) / (unsigned)sc.gt);
}
__device__ __forceinline__ Sched make_sched(const GemmParams &p, int TN) {
    Sched sc;
    const int G = gridDim.x, c = blockIdx.x;
    sc.nb = p.K / QK_K;
    sc.w_tiles = (p.N + TILE_ROWS - 1) / TILE_ROWS;
    sc.n_tiles = sc.w_tiles * ((p.M + TN - 1) / TN);
    if (!p.split) {
        sc.n_full = sc.n_tiles;
        sc.full_per_cta = c < sc.n_tiles ? (sc.n_tiles - c + G - 1) / G : 0;
        sc.T = 0; sc.gt = 1; sc.tail_a = sc.tail_b = 0;
    } else {
        sc.full_per_cta = sc.n_tiles / G;
        sc.n_full = sc.full_per_cta * G;
        sc.T = (sc.n_tiles - sc.n_full) * sc.nb;
        sc.gt = max(1, min(G, sc.T));
        sc.tail_a = c < sc.gt ? tail_start(sc, c) : 0;
        sc.tail_b = c < sc.gt ? tail_start(sc, c + 1) : 0;
    }
    return sc;
}
struct UnitIter {
    int i = 0, pos = -1;
    __device__ __forceinline__ bool next(const Sched &sc, Unit &u) {
        if (i < sc.full_per_cta) {
            u.tile = blockIdx.x + i * gridDim.x;
            u.b0 = 0;
            u.b1 = sc.nb;
            i++;
            return true;
        }
        if (pos < 0) pos = sc.tail_a;
        if (pos >= sc.tail_b) return false;
        const int t = pos / sc.nb;
        u.tile = sc.n_full + t;
        u.b0 = pos - t * sc.nb;
        u.b1 = min(sc.nb, u.b0 + (sc.tail_b - pos));
        pos += u.b1 - u.b0;
        return true;
    }
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

// D[tmem] (+)= A * B; accumulate = 0 overwrites D.  The A operand lives in tensor memory
// (lane = row, each 32-bit column = two K-consecutive f16), B in shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// registers -> 32 lanes x 16 consecutive 32-bit TMEM columns
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// One lane of the (converged) warp: the lane that issues the tensor-core instructions.  The warp as a
// whole walks the loop and waits on the barriers, so that addresses and descriptors are computed in
// warp-uniform code; only the issue itself sits under the elected lane's predicate.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

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

// bytes (b0, b1) resp. (b2, b3) of `bytes4` -> f16x2 (1024 + b, 1024 + b'); bytes must be < 1024.
__device__ __forceinline__ uint32_t magic_lo(uint32_t bytes4) { return __byte_perm(bytes4, 0x64646464u, 0x5140u); }
__device__ __forceinline__ uint32_t magic_hi(uint32_t bytes4) { return __byte_perm(bytes4, 0x64646464u, 0x7362u); }
constexpr uint32_t H2_1024 = 0x64006400u;     // (1024.0, 1024.0)
constexpr uint32_t H2_1056 = 0x64206420u;     // (1056.0, 1056.0) = 1024 + 32

// (lo, hi) f16 halves of `v` broadcast to both halves.
__device__ __forceinline__ uint32_t h2_bcast_lo(uint32_t v) { return __byte_perm(v, 0, 0x1010u); }
__device__ __forceinline__ uint32_t h2_bcast_hi(uint32_t v) { return __byte_perm(v, 0, 0x3232u); }

}  // namespace llmrs
