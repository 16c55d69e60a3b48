// Decode matmul (GEMV, a few tokens) for Q4_K and Q6_K weights on sm_100a.
//
//   out[s*N + r] = sum_k W[r,k] * x[s*K + k]        (src/backend/mod.rs:29-34)
//
// Replaces matvec_q4k_simd / matvec_q6k_simd / gemm_q4k / gemm_q6k of the reference
// (shaders/ops.metal:239-289, 295-344, 357-424, 560-621).  The kernel is built to be bound by
// HBM, not by instruction issue (integer/logic instructions run at half the fp32 rate on this
// part, so a per-weight unpack + fma does not keep up with the memory system):
//
//  * Weights stream through shared memory.  One producer warp issues untiled bulk copies
//    (cp.async.bulk, completion on an mbarrier) of whole row segments into an S-stage ring; the
//    consumer warps never touch global memory for weights, so the bytes in flight are set by
//    the ring (~100 KB per SM), not by registers or occupancy.  One persistent CTA per SM.
//  * Activations are converted once per CTA to block fixed point: each group of 32 (Q4_K
//    sub-block) or 16 (Q6_K scale group) values shares a power-of-two scale and becomes 21-bit
//    integers, stored as three byte planes.  The quants stay integers too, so the inner product
//    of a group is exact integer arithmetic: dp4a on 4 quants x 4 activation bytes, three
//    planes, recombined in int32.  Unpacking costs 3 logic ops per 8 nibbles.
//  * Block scales are applied once per group, in float:
//      Q4_K: sum_sb [ d*sc_sb * sum_j q_j x_j  -  dmin*m_sb * sum_j x_j ]      (tests/ops.rs:41-59)
//      Q6_K: sum_g  [ d*sc_g  * (sum_j q_j x_j - 32 * sum_j x_j) ]              (shaders/ops.metal:322-334)
//
// The only approximation is the 21-bit rounding of the activations relative to the largest
// magnitude of their group (2^-21); sums over groups are float32.  Against a float64
// evaluation of the reference formula the result is within ~1e-6 relative L2.
#include "kernels.h"
#include "llmrs_common.cuh"
#include <cstdlib>
#include <type_traits>

#include "pipeline.cuh"

namespace llmrs {

namespace {

// A pipeline stage holds CHUNK_BLOCKS = 16 consecutive blocks of each row of the tile; a slice is
// the 64 weights one lane handles, four per block.  (Fetching a stage with two tiled TMA boxes of
// 32 rows x half a chunk instead of 32 per-row bulk copies was measured too: no earlier arrival of
// the first stage, 1.68 ms against 1.63 ms on the 225-matmul decode stack.)
// Shorter chunks were measured and are slower,
// because every bulk copy costs the copy engine about 80 clocks whatever its size: with 8-block
// chunks Q4_K 4096x128256 took 82 us against 59 us, with 4-block chunks 145 us, and even a
// one-tile matrix (4096x4096), where arithmetic could start on the first quarter of K, took
// 7.1 us against 4.6 us.
constexpr int MAX_STAGES = 8;

// Activations become integers of 8*PLANES bits (two's complement, one byte plane each; the top
// plane is signed).  |X| <= 2^XBITS keeps the integer dot product of a group inside int32.
// (Q4_K takes its high nibbles in place, as 16*q <= 240, so its integers are two bits shorter:
// 32 * 240 * 2^18 < 2^31.)
template <int PLANES, int QT = 1> struct XFmt {
    static constexpr int XBITS = PLANES == 3 ? (QT == 0 ? 18 : 20) : 15;
    static constexpr int XMAX = PLANES == 3 ? (1 << XBITS) : 32767;
};

template <int QT, int PLANES> struct Fmt;
template <int PLANES> struct Fmt<0, PLANES> {          // Q4_K, raw GGUF blocks
    static constexpr int BLOCK = Q4K_BLOCK_BYTES;
    static constexpr int CHUNK_BLOCKS = 16;
    static constexpr int CHUNK_MAX = CHUNK_BLOCKS * Q4K_BLOCK_BYTES;   // 2304
    static constexpr int GROUP_BYTES = PLANES * 32;    // one sub-block: PLANES planes of 32 bytes
    static constexpr int META = 2 * GROUP_BYTES;       // float inv_lo, inv_hi, xsum_lo, xsum_hi
    static constexpr int XSTRIDE = META + 16;          // 208 / 144: an odd number of 16-byte units,
                                                       // so consecutive lanes hit distinct banks
};
template <int PLANES> struct Fmt<1, PLANES> {          // Q6_K, slice-major chunks (see kernels.h)
    static constexpr int BLOCK = Q6K_BLOCK_BYTES;
    static constexpr int CHUNK_BLOCKS = 16;
    static constexpr int CHUNK_MAX = CHUNK_BLOCKS * Q6K_BLOCK_BYTES;   // 3360
    static constexpr int GROUP_BYTES = PLANES * 16;    // one scale group: PLANES planes of 16 bytes
    static constexpr int META = 4 * GROUP_BYTES;       // float inv[4], float xsum[4]
    static constexpr int XSTRIDE = META + 32 + 16;     // 240 / 176: odd number of 16-byte units
};

// Fused all-gather of the output slices of an N-sharded matmul (world == 0: not used).
// Rank r owns rows [row_offset, row_offset + N) of an n_total-row output.  A result travels to
// the other ranks as ONE 8-byte store {value as float bits, call number} into a mailbox in the
// peer's memory (plain peer stores over NVLink, no TMA, no multicast).  The word is written and read
// as one 64-bit relaxed system-scope access (mailbox_store / mailbox_load), which is a single access in
// the memory model, so the call number doubles as the "this value has landed" flag and no fence is
// needed anywhere: a system-scope fence was measured at 5-7 us on this machine, two of them
// per matmul in an earlier store-then-flag version of this exchange.  The results of a row tile are
// staged in shared memory and warp d posts the tile to rank d, a lane per row, so that the words cross
// NVLink as 256-byte runs rather than one 8-byte packet per row and peer.  When a CTA has finished
// its rows, its threads take a share of the mailbox words addressed to this rank, poll each until
// it carries this call's number (bounded) and write the value into the local output.  The kernel
// therefore completes on a rank only when that rank's output holds every slice, and stream order
// is all a consumer needs.
// The mailbox has two halves used in turn (call number & 1): a peer may be one call ahead, never
// two, because its next call cannot complete without this rank's values of that call.  The call
// number lives in device memory (*step_word) and the kernel advances it itself, so a captured
// CUDA graph can be replayed: nothing that changes from call to call is a launch parameter.
constexpr int MAX_GATHER_RANKS = 8;
struct GatherParams {
    uint2 *peer_box[MAX_GATHER_RANKS];        // mailbox of each rank: [2][world senders][M][N] words
    uint32_t *done_counter;                   // local word: CTAs of this launch that have finished
    uint32_t *step_word;                      // local word: calls completed so far
    size_t half_words;                        // words in one half of a mailbox: world * M * N
    int world, rank, n_total, row_offset;
};

struct GemvParams {
    GatherParams g;
    // Fused feed-forward front (W2 != nullptr; two rows per warp only): the rows of a tile alternate
    // between W (gate) and W2 (up), a warp owns gate row j and up row j, and writes
    // silu(gate . x) * (up . x) as output row j (src/arch/llama.rs:165-168; shaders/ops.metal:762-793).
    const uint8_t *W2;
    // Residual-add epilogue (Residual != nullptr): out = Residual + X . W^T, the residual read in its
    // own type (src/arch/llama.rs:163,169: matmul followed by add).
    const void *Residual;
    int res_bf16;
    // RMS norm of the activations while they are staged (NormW != nullptr): every token row is scaled by
    // rsqrt(mean(x^2) + eps) and by NormW[k] before it is rounded to its block fixed point
    // (src/arch/llama.rs:152-153,164-165: rms_norm followed by matmul; shaders/ops.metal:970-1003).
    const float *NormW;
    float norm_eps;
    // Several weights of one format and K behind one input (n_segs >= 2: the q, k and v projections,
    // src/arch/llama.rs:153-155): rows [seg_first[i], seg_first[i + 1]) of the launch are the rows of
    // seg_W[i] and go to seg_out[i], a [tokens, rows of segment i] buffer.  N is the sum of the rows.
    int n_segs;
    int seg_first[4];
    const uint8_t *seg_W[3];
    void *seg_out[3];
    const uint8_t *W;
    const void *X;
    void *Out;
    uint32_t *err;
    uint32_t wait_limit, gather_limit;   // polls before an mbarrier wait / a mailbox wait is abandoned
    int K, N, m_valid;
    int x_bf16, out_bf16;
    size_t row_stride;      // bytes between weight rows
    int n_row_tiles, n_chunks;
    int stages;             // depth of the weight ring (<= MAX_STAGES)
    int pdl;                // host: launch with programmatic stream serialization (see the kernel)
};

__device__ __forceinline__ float load_x(const void *x, size_t idx, int is_bf16) {
    return is_bf16 ? bf16_bits_to_f32(__ldg((const uint16_t *)x + idx)) : __ldg((const float *)x + idx);
}

__device__ __forceinline__ void store_out(void *out, size_t idx, float v, int is_bf16) {
    if (is_bf16) ((__nv_bfloat16 *)out)[idx] = __float2bfloat16_rn(v);
    else ((float *)out)[idx] = v;
}

__device__ __forceinline__ uint32_t dp4a_uu(uint32_t a, uint32_t b, uint32_t c) { return __dp4a(a, b, c); }

// 4 unsigned bytes (quants) x 4 signed bytes (top activation plane).
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// (small unsigned integer < 2^23) -> float without a conversion instruction.
__device__ __forceinline__ float small_uint_to_float(uint32_t v) {
    return __uint_as_float(0x4B000000u | v) - 8388608.0f;
}

// Power-of-two scale for a group whose largest magnitude is amax: returns e with
// amax * 2^e < 2^X_BITS (clamped so that 2^e and 2^-e are normal floats).
template <int PLANES, int QT>
__device__ __forceinline__ int group_exponent(float amax) {
    const int eb = (int)((__float_as_uint(amax) >> 23) & 0xFFu);      // amax < 2^(eb-126)
    int e = XFmt<PLANES, QT>::XBITS + 126 - eb;
    return max(-126, min(126, e));
}

// ---------------------------------------------------------------------------------------------
// Staging of the activations (all consumer threads, once per CTA).
// Q4_K slice (208 B): sub-block lo: plane0[32] plane1[32] plane2[32]; sub-block hi: same;
//                     then float inv_scale_lo, inv_scale_hi, xsum_lo, xsum_hi.
// Q6_K slice (240 B): group g = 0..3: plane0[16] plane1[16] plane2[16]; then float inv_scale[4],
//                     float xsum[4]; 16 B unused (keeps consecutive lanes on distinct banks).
// xsum is the sum of the rounded activations, so both terms of the formulas above see the same x.
// One thread converts one whole scale group (32 or 16 consecutive activations): maximum,
// exponent, rounding, byte planes and sum all stay in its registers, all loads of the group are
// in flight together (one trip to L2), and there are no shuffles.  Measured alternatives, on the
// 225-matmul decode stack at one token: a warp per group with five-step shuffle reductions,
// 1.88 ms per step; four activations per thread with coalesced loads and two- or three-step
// shuffles, 1.87 ms (5.07 ms at four tokens); this one 1.64 ms (3.96 ms).
// ---------------------------------------------------------------------------------------------
template <int GROUP>
__device__ __forceinline__ void load_group(const void *x, size_t idx, int is_bf16, float (&v)[GROUP]) {
    if (is_bf16) {
        const uint16_t *src = (const uint16_t *)x + idx;
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < GROUP / 8; j++) {
                const uint4 u = __ldg(reinterpret_cast<const uint4 *>(src) + j);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    v[8 * j + 2 * i] = __uint_as_float(w[i] << 16);
                    v[8 * j + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
                }
            }
        } else {                                          // a view that is not 16-byte aligned
#pragma unroll
            for (int i = 0; i < GROUP; i++) v[i] = bf16_bits_to_f32(__ldg(src + i));
        }
    } else {
        const float *src = (const float *)x + idx;
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < GROUP / 4; j++) {
                const float4 f = __ldg(reinterpret_cast<const float4 *>(src) + j);
                v[4 * j] = f.x; v[4 * j + 1] = f.y; v[4 * j + 2] = f.z; v[4 * j + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < GROUP; i++) v[i] = __ldg(src + i);
        }
    }
}

// One group -> integers of XBITS bits, their byte planes at dst + l * GROUP; returns (1/scale, sum/scale).
template <int GROUP, int PLANES, int QT>
__device__ __forceinline__ float2 quantise_group(const float (&v)[GROUP], uint8_t *dst) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < GROUP; i++) amax = fmaxf(amax, fabsf(v[i]));
    const int e = group_exponent<PLANES, QT>(amax);
    const float scale = exp2i(e);
    int X[GROUP];
    int sum = 0;
#pragma unroll
    for (int i = 0; i < GROUP; i++) {
        X[i] = min(__float2int_rn(v[i] * scale), XFmt<PLANES, QT>::XMAX);
        sum += X[i];
    }
#pragma unroll
    for (int l = 0; l < PLANES; l++) {
        uint32_t w[GROUP / 4];
#pragma unroll
        for (int j = 0; j < GROUP / 4; j++) {
            // byte l of four consecutive integers -> one word
            const uint32_t sel = (uint32_t)l | ((uint32_t)(4 + l) << 4);
            const uint32_t lo = __byte_perm((uint32_t)X[4 * j], (uint32_t)X[4 * j + 1], sel);
            const uint32_t hi = __byte_perm((uint32_t)X[4 * j + 2], (uint32_t)X[4 * j + 3], sel);
            w[j] = __byte_perm(lo, hi, 0x5410u);
        }
#pragma unroll
        for (int j = 0; j < GROUP / 16; j++)
            *reinterpret_cast<uint4 *>(dst + l * GROUP + 16 * j) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
    // an infinity or a NaN anywhere in the group makes its results NaN (fmaxf alone would drop a NaN)
    float probe = 0.0f;
#pragma unroll
    for (int i = 0; i < GROUP; i++) probe += v[i] * 0.0f;
    const float inv = probe == 0.0f ? exp2i(-e) : __uint_as_float(0x7FC00000u);
    return make_float2(inv, (float)sum * inv);
}

// RMS norm folded into the matmul: out = rsqrt(mean(x^2) + eps) * (W . (x * g)).  The row's factor is a
// scalar, so it is applied to the finished dot products and the staging needs one pass only: a group is
// loaded once, its squares are added up on the side (norm_squares), it is multiplied by the norm weight
// and rounded to its block fixed point (whose exponent follows the group's own magnitude).  The sums of
// squares meet in `red` ([warps][4] floats of shared memory) behind the barrier that ends the staging.
template <int GROUP>
__device__ __forceinline__ float norm_squares(const float (&v)[GROUP]) {
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < GROUP; i++) a = fmaf(v[i], v[i], a);
    return a;
}

template <int GROUP>
__device__ __forceinline__ void scale_group(const GemvParams &p, float (&v)[GROUP], int k0) {
#pragma unroll
    for (int j = 0; j < GROUP / 4; j++) {
        const float4 w = __ldg(reinterpret_cast<const float4 *>(p.NormW + k0) + j);
        v[4 * j] *= w.x;
        v[4 * j + 1] *= w.y;
        v[4 * j + 2] *= w.z;
        v[4 * j + 3] *= w.w;
    }
}

template <int QT, int PLANES>
__device__ void stage_activations(uint8_t *xarea, size_t xtok_bytes, const GemvParams &p, int tid, int n_threads,
                                  float (*red)[4]) {
    const int K = p.K;
    float ss[4] = {0.0f, 0.0f, 0.0f, 0.0f};              // this thread's share of every token's sum of squares
    if (QT == 0) {
        const int groups = K / 32;                       // group sb = sub-block sb of the row
        for (int gi = tid; gi < groups * p.m_valid; gi += n_threads) {
            const int t = gi / groups, sb = gi - t * groups;
            float v[32];
            load_group<32>(p.X, (size_t)t * K + 32 * (size_t)sb, p.x_bf16, v);
            if (p.NormW) {
                const float a = norm_squares<32>(v);
#pragma unroll
                for (int tt = 0; tt < 4; tt++) ss[tt] += tt == t ? a : 0.0f;
                scale_group<32>(p, v, 32 * sb);
            }
            uint8_t *sl = xarea + (size_t)t * xtok_bytes + (size_t)(sb >> 1) * Fmt<0, PLANES>::XSTRIDE;
            const float2 m = quantise_group<32, PLANES, 0>(v, sl + (sb & 1) * Fmt<0, PLANES>::GROUP_BYTES);
            float *f = reinterpret_cast<float *>(sl + Fmt<0, PLANES>::META);
            f[sb & 1] = m.x;
            f[2 + (sb & 1)] = m.y;
        }
    } else {
        // group q = 16b + 8h + 2g + c covers activations 16 q .. 16 q + 15: group g of slice 4b + 2h + c
        const int groups = K / 16;
        for (int gi = tid; gi < groups * p.m_valid; gi += n_threads) {
            const int t = gi / groups, q = gi - t * groups;
            const int g = (q >> 1) & 3, slice = ((q >> 3) << 1) | (q & 1);
            float v[16];
            load_group<16>(p.X, (size_t)t * K + 16 * (size_t)q, p.x_bf16, v);
            if (p.NormW) {
                const float a = norm_squares<16>(v);
#pragma unroll
                for (int tt = 0; tt < 4; tt++) ss[tt] += tt == t ? a : 0.0f;
                scale_group<16>(p, v, 16 * q);
            }
            uint8_t *sl = xarea + (size_t)t * xtok_bytes + (size_t)slice * Fmt<1, PLANES>::XSTRIDE;
            const float2 m = quantise_group<16, PLANES, 1>(v, sl + g * Fmt<1, PLANES>::GROUP_BYTES);
            float *f = reinterpret_cast<float *>(sl + Fmt<1, PLANES>::META);
            f[g] = m.x;
            f[4 + g] = m.y;
        }
    }
    if (p.NormW) {
#pragma unroll
        for (int tt = 0; tt < 4; tt++) {
#pragma unroll
            for (int o = 16; o; o >>= 1) ss[tt] += __shfl_xor_sync(0xffffffffu, ss[tt], o);
        }
        if ((tid & 31) == 0) {
#pragma unroll
            for (int tt = 0; tt < 4; tt++) red[tid >> 5][tt] = ss[tt];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Per-slice arithmetic.  `row` points at the staged chunk of one weight row.
// ---------------------------------------------------------------------------------------------

// Q4_K: slice sl = 4*b + p is sub-block pair p of block b: quant bytes 32p..32p+31, low nibbles
// are sub-block 2p, high nibbles sub-block 2p+1 (tests/ops.rs:41-59).
template <int MT, int R, int PLANES>
__device__ __forceinline__ void slice_q4k(const uint8_t *const (&row)[R], int sl, const uint8_t *xsl, size_t xtok_bytes,
                                          float (&total)[R][MT]) {
    const int b = sl >> 2, p = sl & 3;
    // Lane constants for the 6-bit scale unpack (tests/ops.rs:29-39).  Pair p uses scale bytes
    // (2p', 2p'+1), p' = p & 1, of the three scale words; pairs 2 and 3 use the split 4+2 bit form.
    const uint32_t pick = (p & 1) ? 0x4432u : 0x4410u;          // byte_perm selector: bytes (2p', 2p'+1), zero above
    const bool upper = p >= 2;
    const uint32_t mask_main = upper ? 0x0F0Fu : 0x3F3Fu;
    const uint32_t mask_top = upper ? 0x3030u : 0u;
    uint32_t lo[R][8], hi[R][8];
    float s_lo[R], s_hi[R], m_lo[R], m_hi[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const uint8_t *blk = row[r] + b * Q4K_BLOCK_BYTES;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * p);
        const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * p);
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            lo[r][i] = w[i] & 0x0F0F0F0Fu;
            hi[r][i] = w[i] & 0xF0F0F0F0u;        // 16*q, used in place; the 1/16 goes into the scale
        }
        const float d = f16_bits_to_f32((uint16_t)(hdr.x & 0xFFFFu));
        const float dmin = f16_bits_to_f32((uint16_t)(hdr.x >> 16));
        const uint32_t A = __byte_perm(hdr.y, 0, pick);          // scales[2p'], scales[2p'+1]
        const uint32_t B = __byte_perm(hdr.z, 0, pick);          // scales[4+2p'], ...
        const uint32_t C = __byte_perm(hdr.w, 0, pick);          // scales[8+2p'], ...
        const uint32_t scp = ((upper ? C : A) & mask_main) | ((A >> 2) & mask_top);
        const uint32_t mnp = ((upper ? (C >> 4) : B) & mask_main) | ((B >> 2) & mask_top);
        // byte -> float through the mantissa of 2^23 (one byte permute each, no conversion)
        s_lo[r] = d * (__uint_as_float(__byte_perm(scp, 0x4B000000u, 0x7440u)) - 8388608.0f);
        s_hi[r] = d * 0.0625f * (__uint_as_float(__byte_perm(scp, 0x4B000000u, 0x7441u)) - 8388608.0f);
        m_lo[r] = dmin * (__uint_as_float(__byte_perm(mnp, 0x4B000000u, 0x7440u)) - 8388608.0f);
        m_hi[r] = dmin * (__uint_as_float(__byte_perm(mnp, 0x4B000000u, 0x7441u)) - 8388608.0f);
    }
#pragma unroll
    for (int t = 0; t < MT; t++) {
        const uint8_t *xs = xsl + (size_t)t * xtok_bytes;
        using F = Fmt<0, PLANES>;
        const float4 meta = *reinterpret_cast<const float4 *>(xs + F::META);   // inv_lo, inv_hi, xsum_lo, xsum_hi
        float val[R][2];
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            uint32_t pl[PLANES][8];
#pragma unroll
            for (int l = 0; l < PLANES; l++) {
                const uint4 u0 = *reinterpret_cast<const uint4 *>(xs + hf * F::GROUP_BYTES + l * 32);
                const uint4 u1 = *reinterpret_cast<const uint4 *>(xs + hf * F::GROUP_BYTES + l * 32 + 16);
                pl[l][0] = u0.x; pl[l][1] = u0.y; pl[l][2] = u0.z; pl[l][3] = u0.w;
                pl[l][4] = u1.x; pl[l][5] = u1.y; pl[l][6] = u1.z; pl[l][7] = u1.w;
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                uint32_t s0 = 0, s1 = 0;
                int st = 0;                                               // top (signed) plane
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t q = hf ? hi[r][i] : lo[r][i];
                    s0 = dp4a_uu(q, pl[0][i], s0);
                    if (PLANES == 3) s1 = dp4a_uu(q, pl[1][i], s1);
                    st = dp4a_us(q, pl[PLANES - 1][i], st);
                }
                // exact in int32: |S| <= 32*240*2^18
                const int S = PLANES == 3 ? (st * 256 + (int)s1) * 256 + (int)s0 : st * 256 + (int)s0;
                val[r][hf] = (float)S * (hf ? meta.y : meta.x);
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            float v = total[r][t];
            v = fmaf(s_lo[r], val[r][0], v);
            v = fmaf(s_hi[r], val[r][1], v);
            v = fmaf(-m_lo[r], meta.z, v);
            v = fmaf(-m_hi[r], meta.w, v);
            total[r][t] = v;
        }
    }
}

// Q6_K: slice sl = 4*b + 2*h + c covers weights 256b + 128h + 32g + 16c + i (g = 0..3, i = 0..15).
// Staged bytes of the slice: ql[64h+16c+i] (low nibble: g=0, high: g=2), ql[64h+32+16c+i] (low: g=1,
// high: g=3), qh[32h+16c+i] (bits 2g..2g+1); each g is one scale group (shaders/ops.metal:28-42).
template <int MT, int R, int PLANES>
__device__ __forceinline__ void slice_q6k(const uint8_t *const (&row)[R], int sl, int nbc, const uint8_t *xsl,
                                          size_t xtok_bytes, float (&total)[R][MT]) {
    const int b = sl >> 2, h = (sl >> 1) & 1, c = sl & 1;
    uint32_t v[R][4][4];
    float ds[R][4];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const uint8_t *s = row[r] + 48 * sl;
        const uint4 l0 = *reinterpret_cast<const uint4 *>(s);
        const uint4 l1 = *reinterpret_cast<const uint4 *>(s + 16);
        const uint4 qh = *reinterpret_cast<const uint4 *>(s + 32);
        const uint2 scw = *reinterpret_cast<const uint2 *>(row[r] + 192 * nbc + 16 * b + 8 * h);
        const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(row[r] + 208 * nbc + 2 * b));
        const uint32_t a0[4] = {l0.x, l0.y, l0.z, l0.w}, a1[4] = {l1.x, l1.y, l1.z, l1.w};
        const uint32_t hh[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t qA = hh[i] & 0x33333333u;             // g=0 bits at 0-1, g=2 bits at 4-5
            const uint32_t qB = (hh[i] >> 2) & 0x33333333u;      // g=1 bits at 0-1, g=3 bits at 4-5
            v[r][0][i] = (a0[i] & 0x0F0F0F0Fu) | ((qA << 4) & 0xF0F0F0F0u);
            v[r][1][i] = (a1[i] & 0x0F0F0F0Fu) | ((qB << 4) & 0xF0F0F0F0u);
            v[r][2][i] = ((a0[i] >> 4) & 0x0F0F0F0Fu) | (qA & 0xF0F0F0F0u);
            v[r][3][i] = ((a1[i] >> 4) & 0x0F0F0F0Fu) | (qB & 0xF0F0F0F0u);
        }
        // int8 scale of group g sits at scales[8h + 2g + c]
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const uint32_t sw = (g < 2 ? scw.x : scw.y) ^ 0x80808080u;           // sc + 128 per byte
            const uint32_t sbyte = (sw >> (8 * (2 * (g & 1) + c))) & 0xFFu;
            ds[r][g] = d * (small_uint_to_float(sbyte) - 128.0f);
        }
    }
#pragma unroll
    for (int t = 0; t < MT; t++) {
        const uint8_t *xs = xsl + (size_t)t * xtok_bytes;
        using F = Fmt<1, PLANES>;
        const float4 inv = *reinterpret_cast<const float4 *>(xs + F::META);
        const float4 xsum = *reinterpret_cast<const float4 *>(xs + F::META + 16);
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const uint4 p0 = *reinterpret_cast<const uint4 *>(xs + g * F::GROUP_BYTES);
            const uint4 p1 = *reinterpret_cast<const uint4 *>(xs + g * F::GROUP_BYTES + 16);
            const uint4 p2 = *reinterpret_cast<const uint4 *>(xs + g * F::GROUP_BYTES + (PLANES - 1) * 16);
            const uint32_t x0[4] = {p0.x, p0.y, p0.z, p0.w}, x1[4] = {p1.x, p1.y, p1.z, p1.w};
            const uint32_t x2[4] = {p2.x, p2.y, p2.z, p2.w};                     // top (signed) plane
            const float ig = g == 0 ? inv.x : g == 1 ? inv.y : g == 2 ? inv.z : inv.w;
            const float xg = g == 0 ? xsum.x : g == 1 ? xsum.y : g == 2 ? xsum.z : xsum.w;
#pragma unroll
            for (int r = 0; r < R; r++) {
                uint32_t s0 = 0, s1 = 0;
                int st = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    s0 = dp4a_uu(v[r][g][i], x0[i], s0);
                    if (PLANES == 3) s1 = dp4a_uu(v[r][g][i], x1[i], s1);
                    st = dp4a_us(v[r][g][i], x2[i], st);
                }
                // exact in int32: |S| <= 16*63*2^20
                const int S = PLANES == 3 ? (st * 256 + (int)s1) * 256 + (int)s0 : st * 256 + (int)s0;
                const float val = fmaf((float)S, ig, -32.0f * xg);         // sum (q-32) x over the group
                total[r][t] = fmaf(ds[r][g], val, total[r][t]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel: warps 0..NCW-1 consume, warp NCW produces.  A row tile is RT = R*NCW rows; consumer
// warp w owns rows R*w..R*w+R-1 of the tile and walks the row's K chunks as they land.
// ---------------------------------------------------------------------------------------------
template <int QT, int MT, int R, int NCW, int PLANES>
__global__ void __launch_bounds__((NCW + 1) * 32, 1) gemv_kernel(const GemvParams p) {
    using F = Fmt<QT, PLANES>;
    constexpr int RT = R * NCW;
    static_assert(NCW >= MAX_GATHER_RANKS, "the fused all-gather posts with one warp per rank");
    __shared__ float norm_red[NCW][4];
    __shared__ uint64_t consumers_done;                  // every consumer warp arrives here when it has finished
    __shared__ int gave_up;                              // a bounded wait ran out somewhere in this CTA
    __shared__ float gather_out[2][MT][RT];              // fused all-gather: a row tile's results, two tiles in turn
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + MAX_STAGES;
    const int S = p.stages;
    const int n_slices = p.K / 64;
    const size_t xtok_bytes = (size_t)n_slices * F::XSTRIDE;
    uint8_t *xarea = smem + 128;   // 2 * MAX_STAGES barriers of 8 bytes in front
    uint8_t *stages = xarea + ((MT * xtok_bytes + 127) / 128) * 128;
    const size_t stage_bytes = (size_t)RT * F::CHUNK_MAX;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NCW);
        }
        mbar_init(&consumers_done, NCW);
        gave_up = 0;
        mbar_init_fence();
    }
    __syncthreads();

    // Programmatic dependent launch.  The kernel that follows this one in the stream may start
    // right away (its CTAs take SMs as ours leave them), and this kernel may have started before
    // its predecessor finished.  Weights are never written by a kernel that is still in flight
    // (upload_tensor synchronises), so the producer warp starts fetching them at once; everything
    // that reads activations or writes results comes after griddepcontrol.wait, which returns when
    // the predecessor has completed and its writes are visible.  Both are no-ops in a plain launch.
    asm volatile("griddepcontrol.launch_dependents;");
    const int nb = p.K / QK_K;
    if (warp == NCW) {
        // ---------------- producer ----------------
        uint32_t it = 0;
        bool stop = false;
        for (int rt = blockIdx.x; rt < p.n_row_tiles && !stop; rt += gridDim.x) {
            for (int c = 0; c < p.n_chunks; c++, it++) {
                const int s = it % S;
                if (*(volatile int *)&gave_up) { stop = true; break; }
                if (it >= (uint32_t)S && !mbar_wait(&empty[s], ((it / S) - 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_EMPTY_WAIT);
                    *(volatile int *)&gave_up = 1;
                    stop = true;
                    break;
                }
                const int nbc = min(F::CHUNK_BLOCKS, nb - c * F::CHUNK_BLOCKS);
                const uint32_t bytes = (uint32_t)((nbc * F::BLOCK + 15) / 16 * 16);
                if (lane == 0) mbar_arrive_expect_tx(&full[s], bytes * RT);
                __syncwarp();
                if (lane < RT) {
                    const bool pair = R == 2 && p.W2 != nullptr;
                    int row = pair ? min(rt * (RT / 2) + (lane >> 1), p.N - 1) : min(rt * RT + lane, p.N - 1);
                    const uint8_t *src = pair && (lane & 1) ? p.W2 : p.W;
                    if (p.n_segs) {                      // the weight this row belongs to
                        const int sg = (row >= p.seg_first[1]) + (row >= p.seg_first[2]);
                        src = p.seg_W[sg];
                        row -= p.seg_first[sg];
                    }
                    bulk_copy_g2s(stages + s * stage_bytes + (size_t)lane * F::CHUNK_MAX,
                                  src + (size_t)row * p.row_stride + (size_t)c * F::CHUNK_MAX, bytes, &full[s]);
                }
            }
        }
        // The producer leaves last.  In the normal course every copy has been consumed by then.  After an
        // abandoned wait, copies of up to S stages may still be in flight towards this CTA's shared
        // memory; the CTA must not end (and hand the memory to another CTA) before they have landed, so
        // the producer waits, again with a limit, for the full barrier of each stage it armed last.
        mbar_wait(&consumers_done, 0, p.wait_limit);
        if (*(volatile int *)&gave_up) {
            const uint32_t first = it > (uint32_t)S ? it - (uint32_t)S : 0u;
            for (uint32_t j = first; j < it; j++) mbar_wait(&full[j % S], (j / S) & 1, p.wait_limit);
        }
        return;
    }

    // ---------------- consumers ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // this call's step; the word is only advanced by the last CTA of a launch, after every CTA has read it
    const uint32_t gather_step = p.g.world > 0 ? *reinterpret_cast<volatile uint32_t *>(p.g.step_word) + 1u : 0u;
    stage_activations<QT, PLANES>(xarea, xtok_bytes, p, threadIdx.x, NCW * 32, norm_red);
    named_barrier_sync(1, NCW * 32);
    float inv_rms[MT];                                   // the tokens' norm factors, applied to the finished sums
#pragma unroll
    for (int t = 0; t < MT; t++) {
        inv_rms[t] = 1.0f;
        if (p.NormW) {
            float sq = 0.0f;
#pragma unroll
            for (int w = 0; w < NCW; w++) sq += norm_red[w][t];
            inv_rms[t] = rsqrtf(sq / (float)p.K + p.norm_eps);
        }
    }

    uint32_t it = 0;
    bool ok = true;
    // Every consumer warp walks every row tile of the CTA, also after a wait has run out (it then skips
    // the work), because the fused all-gather meets at a barrier once per tile.
    int tile_par = 0;
    for (int rt = blockIdx.x; rt < p.n_row_tiles; rt += gridDim.x) {
        float total[R][MT];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) total[r][t] = 0.0f;

        for (int c = 0; c < p.n_chunks && ok; c++, it++) {
            const int s = it % S;
            if (!mbar_wait(&full[s], (it / S) & 1, p.wait_limit)) {
                report_error(p.err, KERR_FULL_WAIT);
                *(volatile int *)&gave_up = 1;
                ok = false;
                break;
            }
            const int nbc = min(F::CHUNK_BLOCKS, nb - c * F::CHUNK_BLOCKS);
            const uint8_t *row[R];
#pragma unroll
            for (int r = 0; r < R; r++) row[r] = stages + s * stage_bytes + (size_t)(warp * R + r) * F::CHUNK_MAX;
            if (nbc == F::CHUNK_BLOCKS) {
                // a full chunk is two slices per lane; written out, the loads of the second overlap the
                // arithmetic of the first (measured: 7 % at two tokens, 1 % at one)
#pragma unroll
                for (int it2 = 0; it2 < 2; it2++) {
                    const int sl = lane + 32 * it2;
                    const uint8_t *xsl = xarea + (size_t)(c * F::CHUNK_BLOCKS * 4 + sl) * F::XSTRIDE;
                    if (QT == 0) slice_q4k<MT, R, PLANES>(row, sl, xsl, xtok_bytes, total);
                    else slice_q6k<MT, R, PLANES>(row, sl, nbc, xsl, xtok_bytes, total);
                }
            } else {
                for (int sl = lane; sl < 4 * nbc; sl += 32) {
                    const uint8_t *xsl = xarea + (size_t)(c * F::CHUNK_BLOCKS * 4 + sl) * F::XSTRIDE;
                    if (QT == 0) slice_q4k<MT, R, PLANES>(row, sl, xsl, xtok_bytes, total);
                    else slice_q6k<MT, R, PLANES>(row, sl, nbc, xsl, xtok_bytes, total);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }

        if (R == 2 && p.W2 != nullptr) {
            // ---- fused feed-forward front: silu(gate) * up, one output row per warp ----
#pragma unroll
            for (int t = 0; t < MT; t++) {
                float g = total[0][t], u = total[R - 1][t];
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    g += __shfl_xor_sync(0xffffffffu, g, o);
                    u += __shfl_xor_sync(0xffffffffu, u, o);
                }
                g *= inv_rms[t];
                u *= inv_rms[t];
                const int out_row = rt * (RT / 2) + warp;
                if (ok && lane == 0 && out_row < p.N && t < p.m_valid)
                    store_out(p.Out, (size_t)t * p.N + out_row, g / (1.0f + expf(-g)) * u, p.out_bf16);
            }
            continue;
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) {
                float v = total[r][t];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                v *= inv_rms[t];
                const int out_row = rt * RT + warp * R + r;
                if (ok && out_row < p.N && t < p.m_valid) {
                    if (p.n_segs) {
                        if (lane == 0) {
                            const int sg = (out_row >= p.seg_first[1]) + (out_row >= p.seg_first[2]);
                            const int n_sg = p.seg_first[sg + 1] - p.seg_first[sg];
                            store_out(p.seg_out[sg], (size_t)t * n_sg + (out_row - p.seg_first[sg]), v, p.out_bf16);
                        }
                    } else if (p.g.world == 0) {
                        if (lane == 0) {
                            const size_t o = (size_t)t * p.N + out_row;
                            if (p.Residual) v += load_x(p.Residual, o, p.res_bf16);
                            store_out(p.Out, o, v, p.out_bf16);
                        }
                    } else if (lane == 0) {               // fused all-gather: staged, posted a tile at a time
                        gather_out[tile_par][t][warp * R + r] = v;
                    }
                }
            }
        if (p.g.world > 0) {
            // Warp d takes the tile to rank d: its own rank's copy goes straight into the output, the
            // others into the peer's mailbox, a lane per row, so that a tile travels as 256-byte runs of
            // {value, call number} words instead of one 8-byte packet per row and peer.
            named_barrier_sync(1, NCW * 32);
            if (warp < p.g.world && !*(volatile int *)&gave_up) {
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    if (t >= p.m_valid) break;
                    for (int l = lane; l < RT; l += 32) {
                        const int out_row = rt * RT + l;
                        if (out_row >= p.N) break;
                        const float v = gather_out[tile_par][t][l];
                        if (warp == p.g.rank) {
                            store_out(p.Out, (size_t)t * p.g.n_total + p.g.row_offset + out_row, v, p.out_bf16);
                        } else {
                            uint2 *box = p.g.peer_box[warp] + (gather_step & 1u) * p.g.half_words +
                                         ((size_t)p.g.rank * p.m_valid + t) * p.N + out_row;
                            mailbox_store(box, __float_as_uint(v), gather_step);
                        }
                    }
                }
            }
            tile_par ^= 1;   // the next tile's barrier comes before this buffer is written again
        }
    }

    if (p.g.world > 1) {
        // ---- collect the other ranks' slices from this rank's mailbox ----
        const uint2 *box = p.g.peer_box[p.g.rank] + (gather_step & 1u) * p.g.half_words;
        const int per_src = p.m_valid * p.N;                             // words one sender posts
        const int remote = (p.g.world - 1) * per_src;
        // A thread takes words i, i + stride, ...; it has UNPACK of them in flight at a time, so a
        // batch costs one trip to L2, and polls again only the words that had not landed yet.
        constexpr int UNPACK = 8;
        const int stride = gridDim.x * (NCW * 32);
        bool late = false;
        for (int i0 = blockIdx.x * (NCW * 32) + threadIdx.x; i0 < remote && !late; i0 += UNPACK * stride) {
            uint2 got[UNPACK];
#pragma unroll
            for (int b = 0; b < UNPACK; b++) {
                const int i = i0 + b * stride;
                if (i < remote) {
                    const int q = i / per_src, rem = i - q * per_src;
                    got[b] = mailbox_load(box + (size_t)(q < p.g.rank ? q : q + 1) * per_src + rem);
                }
            }
#pragma unroll
            for (int b = 0; b < UNPACK; b++) {
                const int i = i0 + b * stride;
                if (i >= remote || late) continue;
                const int q = i / per_src, rem = i - q * per_src;
                const int src = q < p.g.rank ? q : q + 1;
                const int t = rem / p.N, row = rem - t * p.N;
                if (got[b].y != gather_step &&
                    !mailbox_wait(box + (size_t)src * per_src + rem, gather_step, p.gather_limit, got[b])) {
                    report_error(p.err, KERR_GATHER_WAIT);
                    late = true;
                    continue;
                }
                store_out(p.Out, (size_t)t * p.g.n_total + (size_t)src * p.N + row, __uint_as_float(got[b].x), p.out_bf16);
            }
        }
    }
    if (p.g.world > 0) {
        // the last CTA to get here advances the call number for the next launch; every CTA read it long ago
        named_barrier_sync(1, NCW * 32);
        if (threadIdx.x == 0) {
            const uint32_t ticket = atomicAdd(p.g.done_counter, 1u);
            if (ticket == gridDim.x - 1) {
                *p.g.done_counter = 0;
                *p.g.step_word = gather_step;
            }
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&consumers_done);         // lets the producer warp, and with it the CTA, end
}

// ---------------------------------------------------------------------------------------------
// Launch
// ---------------------------------------------------------------------------------------------
constexpr int NCW_DEFAULT = 16;
// Byte planes of the block-fixed-point activations.  Three planes (18 / 20-bit integers) put the result
// within ~1e-6 of the float64 product; two planes (15 bits) within ~3e-5, still inside the 1e-4 this path
// is held to, for a third less dot-product work and shared-memory traffic.  Q4_K, which is bound by
// instruction issue, always takes two; Q6_K takes three at one token, where it already runs at the
// speed of HBM, and two from two tokens on, where the plane reads bound it.  LLMRS_GEMV_PLANES=3 in the
// environment (read once per process) keeps three planes everywhere.
constexpr int planes_for(int QT, int MT) { return QT == 0 ? 2 : (MT == 1 ? 3 : 2); }
static bool three_planes_everywhere() {
    static const bool v = [] { const char *e = getenv("LLMRS_GEMV_PLANES"); return e && atoi(e) == 3; }();
    return v;
}
constexpr size_t SMEM_LIMIT = 226 * 1024;       // 227 KB per CTA less the kernel's static shared memory

template <int QT, int MT, int R, int NCW, int PLANES>
size_t smem_fixed(int K) {
    return 128 + ((size_t)MT * (K / 64) * Fmt<QT, PLANES>::XSTRIDE + 127) / 128 * 128;
}

// Ring depth that fits beside the staged activations (0: not even two stages fit).
template <int QT, int MT, int R, int NCW, int PLANES>
int ring_stages(int K, int want) {
    const size_t stage = (size_t)R * NCW * Fmt<QT, PLANES>::CHUNK_MAX;
    const size_t fixed = smem_fixed<QT, MT, R, NCW, PLANES>(K);
    if (fixed + 2 * stage > SMEM_LIMIT) return 0;
    int s = (int)((SMEM_LIMIT - fixed) / stage);
    if (s > want) s = want;
    return s > MAX_STAGES ? MAX_STAGES : s;
}

template <int QT, int MT, int R, int NCW, int PLANES>
cudaError_t launch_cfg(const GemvParams &p0, int sm_count, int want_stages, cudaStream_t s) {
    GemvParams p = p0;
    constexpr int RT = R * NCW;
    static_assert(RT <= 32, "one producer lane per row of the tile");
    const int out_rows_per_tile = p.W2 ? RT / 2 : RT;          // fused feed-forward front: gate and up rows alternate
    if (p.W2 && R != 2) return cudaErrorInvalidConfiguration;
    p.n_row_tiles = (p.N + out_rows_per_tile - 1) / out_rows_per_tile;
    p.n_chunks = (p.K / QK_K + Fmt<QT, PLANES>::CHUNK_BLOCKS - 1) / Fmt<QT, PLANES>::CHUNK_BLOCKS;
    p.stages = ring_stages<QT, MT, R, NCW, PLANES>(p.K, want_stages);
    if (p.stages < 2) return cudaErrorInvalidConfiguration;
    {   // no more stages than the busiest CTA has chunks to fetch (less shared memory to carve out)
        const int grid0 = p.n_row_tiles < sm_count ? p.n_row_tiles : sm_count;
        const int chunks_per_cta = (p.n_row_tiles + grid0 - 1) / grid0 * p.n_chunks;
        if (chunks_per_cta < p.stages) p.stages = chunks_per_cta;
    }
    const size_t smem = smem_fixed<QT, MT, R, NCW, PLANES>(p.K) + (size_t)p.stages * RT * Fmt<QT, PLANES>::CHUNK_MAX;
    auto kern = gemv_kernel<QT, MT, R, NCW, PLANES>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int grid = p.n_row_tiles < sm_count ? p.n_row_tiles : sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((NCW + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// Rows per warp: two rows share the staged activations in registers (measured best at every
// shape tried); one row per warp when the larger ring does not fit beside the activations.
template <int QT, int MT, int P>
cudaError_t launch_mt_planes(const GemvParams &p, int sm_count, cudaStream_t s, bool *fits) {
    constexpr int W = NCW_DEFAULT;
    *fits = true;
    if (ring_stages<QT, MT, 2, W, P>(p.K, 4) >= 2) return launch_cfg<QT, MT, 2, W, P>(p, sm_count, 4, s);
    if (!p.W2 && ring_stages<QT, MT, 1, W, P>(p.K, 4) >= 2) return launch_cfg<QT, MT, 1, W, P>(p, sm_count, 4, s);
    *fits = false;
    return cudaSuccess;
}
template <int QT, int MT>
cudaError_t launch_mt(const GemvParams &p, int sm_count, cudaStream_t s, bool *fits) {
    if (planes_for(QT, MT) == 3 || three_planes_everywhere()) return launch_mt_planes<QT, MT, 3>(p, sm_count, s, fits);
    return launch_mt_planes<QT, MT, 2>(p, sm_count, s, fits);
}

template <int QT>
cudaError_t launch_fmt(GemvParams p, int M, int x_elem, int out_elem, int sm_count, cudaStream_t s,
                       uint64_t *launches) {
    const uint8_t *X = (const uint8_t *)p.X;
    uint8_t *Out = (uint8_t *)p.Out;
    const uint8_t *Res = (const uint8_t *)p.Residual;
    int t0 = 0;
    int mt = M >= 4 ? 4 : M;
    while (t0 < M) {
        int m = M - t0 < mt ? M - t0 : mt;
        p.X = X + (size_t)t0 * p.K * x_elem;
        p.Out = Out + (size_t)t0 * p.N * out_elem;
        if (Res) p.Residual = Res + (size_t)t0 * p.N * (p.res_bf16 ? 2 : 4);
        p.m_valid = m;
        bool fits = false;
        cudaError_t e = cudaSuccess;
        switch (m) {
            case 1: e = launch_mt<QT, 1>(p, sm_count, s, &fits); break;
            case 2: e = launch_mt<QT, 2>(p, sm_count, s, &fits); break;
            case 3: e = launch_mt<QT, 3>(p, sm_count, s, &fits); break;
            default: e = launch_mt<QT, 4>(p, sm_count, s, &fits); break;
        }
        if (e != cudaSuccess) return e;
        if (!fits) {                 // staged activations of m tokens do not fit: fewer tokens per pass
            if (m == 1) return cudaErrorInvalidValue;
            mt = m - 1;
            continue;
        }
        if (launches) (*launches)++;
        t0 += m;
    }
    return cudaSuccess;
}

}  // namespace

size_t gemv_max_k() {
    // largest K whose single-token staging fits beside the smallest ring
    size_t k = 0;
    while (ring_stages<1, 1, 1, NCW_DEFAULT, 3>((int)(k + 256), 2) >= 2 && k < (1u << 20)) k += 256;
    return k;
}

cudaError_t launch_gemv(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                        int K, int N, int M, int sm_count, bool pdl, ErrSink err_word, cudaStream_t s,
                        uint64_t *launches, const void *residual, int residual_dtype, const float *norm_weight,
                        float norm_eps) {
    if (K <= 0 || N <= 0 || M <= 0) return cudaSuccess;
    GemvParams p{};
    p.pdl = pdl;
    p.NormW = norm_weight;
    p.norm_eps = norm_eps;
    p.Residual = residual;
    p.res_bf16 = residual_dtype == DT_BF16;
    p.W = w; p.X = x; p.Out = out; p.err = err_word.word; p.wait_limit = err_word.mbar_polls; p.gather_limit = err_word.gather_polls;
    p.K = K; p.N = N;
    p.x_bf16 = x_dtype == DT_BF16; p.out_bf16 = out_dtype == DT_BF16;
    const int xe = x_dtype == DT_BF16 ? 2 : 4, oe = out_dtype == DT_BF16 ? 2 : 4;
    if (wdtype == DT_Q4K) {
        p.row_stride = (size_t)(K / QK_K) * Q4K_BLOCK_BYTES;
        return launch_fmt<0>(p, M, xe, oe, sm_count, s, launches);
    }
    if (wdtype == DT_Q6K) {
        p.row_stride = q6k_row_stride(K);
        return launch_fmt<1>(p, M, xe, oe, sm_count, s, launches);
    }
    return cudaErrorInvalidValue;
}

// Two or three weights of one format and K behind the same (optionally normalised) input, one launch,
// one token pass: M <= 4 and M <= gemv_single_launch_max_tokens.  out[i] is [M, n_rows[i]].
cudaError_t launch_gemv_multi(int wdtype, int n, const uint8_t *const *ws, const int *n_rows, void *const *outs,
                              const void *x, int x_dtype, int out_dtype, int K, int M, int sm_count, bool pdl,
                              ErrSink err_word, cudaStream_t s, uint64_t *launches, const float *norm_weight,
                              float norm_eps) {
    if (n < 2 || n > 3 || K <= 0 || M <= 0 || M > 4 || M > gemv_single_launch_max_tokens(wdtype, K)) return cudaErrorInvalidValue;
    GemvParams p{};
    p.pdl = pdl;
    p.NormW = norm_weight;
    p.norm_eps = norm_eps;
    p.X = x; p.err = err_word.word; p.wait_limit = err_word.mbar_polls; p.gather_limit = err_word.gather_polls; p.K = K;
    p.x_bf16 = x_dtype == DT_BF16; p.out_bf16 = out_dtype == DT_BF16;
    p.n_segs = n;
    int first = 0;
    for (int i = 0; i < 3; i++) {
        p.seg_first[i] = first;
        if (i < n) {
            if (n_rows[i] <= 0) return cudaErrorInvalidValue;
            p.seg_W[i] = ws[i];
            p.seg_out[i] = outs[i];
            first += n_rows[i];
        }
    }
    p.seg_first[3] = first;
    for (int i = n; i < 3; i++) p.seg_first[i] = first;         // absent segments are empty
    p.N = first;
    p.W = ws[0]; p.Out = outs[0];
    if (wdtype == DT_Q4K) {
        p.row_stride = (size_t)(K / QK_K) * Q4K_BLOCK_BYTES;
        return launch_fmt<0>(p, M, 0, 0, sm_count, s, launches);
    }
    if (wdtype == DT_Q6K) {
        p.row_stride = q6k_row_stride(K);
        return launch_fmt<1>(p, M, 0, 0, sm_count, s, launches);
    }
    return cudaErrorInvalidValue;
}

// Fused feed-forward front: out[M, N] = silu(X . Wgate^T) * (X . Wup^T), both weights [K, N] of
// one type; one launch.  Returns cudaErrorInvalidConfiguration when the two-rows-per-warp
// configuration does not fit (large K with several tokens): the caller then runs two matmuls.
bool gemv_gate_up_fits(int wdtype, int K, int M) {
    if (M < 1 || M > 4 || K <= 0 || K % QK_K) return false;
    auto fits = [&](auto qt) {
        constexpr int QT = decltype(qt)::value;
        switch (M) {
            case 1: return ring_stages<QT, 1, 2, NCW_DEFAULT, 3>(K, 4) >= 2;
            case 2: return ring_stages<QT, 2, 2, NCW_DEFAULT, 3>(K, 4) >= 2;
            case 3: return ring_stages<QT, 3, 2, NCW_DEFAULT, 3>(K, 4) >= 2;
            default: return ring_stages<QT, 4, 2, NCW_DEFAULT, 3>(K, 4) >= 2;
        }
    };
    if (wdtype == DT_Q4K) return fits(std::integral_constant<int, 0>{});
    if (wdtype == DT_Q6K) return fits(std::integral_constant<int, 1>{});
    return false;
}

cudaError_t launch_gemv_gate_up(int wdtype, const uint8_t *w_gate, const uint8_t *w_up, const void *x, int x_dtype,
                                void *out, int out_dtype, int K, int N, int M, int sm_count, bool pdl,
                                ErrSink err_word, cudaStream_t s, uint64_t *launches, const float *norm_weight,
                                float norm_eps) {
    if (!gemv_gate_up_fits(wdtype, K, M)) return cudaErrorInvalidConfiguration;
    GemvParams p{};
    p.pdl = pdl;
    p.NormW = norm_weight;
    p.norm_eps = norm_eps;
    p.W = w_gate; p.W2 = w_up; p.X = x; p.Out = out; p.err = err_word.word; p.wait_limit = err_word.mbar_polls; p.gather_limit = err_word.gather_polls;
    p.K = K; p.N = N;
    p.x_bf16 = x_dtype == DT_BF16; p.out_bf16 = out_dtype == DT_BF16;
    uint64_t n = 0;
    cudaError_t e;
    if (wdtype == DT_Q4K) {
        p.row_stride = (size_t)(K / QK_K) * Q4K_BLOCK_BYTES;
        e = launch_fmt<0>(p, M, 0, 0, sm_count, s, &n);
    } else {
        p.row_stride = q6k_row_stride(K);
        e = launch_fmt<1>(p, M, 0, 0, sm_count, s, &n);
    }
    if (e == cudaSuccess && n != 1) e = cudaErrorInvalidConfiguration;
    if (launches) *launches += n;
    return e;
}

// Largest token count (<= 4) whose staged activations fit one launch of the decode kernel.
namespace {
template <int QT, int MT>
bool one_pass_fits(int K) {
    return ring_stages<QT, MT, 2, NCW_DEFAULT, 3>(K, 4) >= 2 ||
           ring_stages<QT, MT, 1, NCW_DEFAULT, 3>(K, 4) >= 2;
}
template <int QT>
int max_tokens_qt(int K) {
    if (one_pass_fits<QT, 4>(K)) return 4;
    if (one_pass_fits<QT, 3>(K)) return 3;
    if (one_pass_fits<QT, 2>(K)) return 2;
    return one_pass_fits<QT, 1>(K) ? 1 : 0;
}
}  // namespace
int gemv_single_launch_max_tokens(int wdtype, int K) {
    if (K <= 0 || K % QK_K) return 0;
    return wdtype == DT_Q4K ? max_tokens_qt<0>(K) : wdtype == DT_Q6K ? max_tokens_qt<1>(K) : 0;
}

// N-sharded decode matmul with the all-gather of the output slices fused into the kernel (see
// GatherParams).  One launch, so M <= 4 and the activations must fit the shared-memory staging.
size_t gemv_allgather_mailbox_bytes(int n_total, int M) { return (size_t)2 * M * n_total * sizeof(uint2); }

cudaError_t launch_gemv_allgather(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                                  int K, int N_local, int M, int rank, int world, void *const *peer_mailbox,
                                  uint32_t *done_counter, uint32_t *step_word, int sm_count, bool pdl,
                                  ErrSink err_word, cudaStream_t s, uint64_t *launches) {
    if (K <= 0 || N_local <= 0 || M <= 0 || M > 4 || world < 1 || world > MAX_GATHER_RANKS) return cudaErrorInvalidValue;
    if (M > gemv_single_launch_max_tokens(wdtype, K)) return cudaErrorInvalidValue;   // token passes would each post
    GemvParams p{};
    p.pdl = pdl;
    p.W = w; p.X = x; p.Out = out; p.err = err_word.word; p.wait_limit = err_word.mbar_polls; p.gather_limit = err_word.gather_polls;
    p.K = K; p.N = N_local;
    p.x_bf16 = x_dtype == DT_BF16; p.out_bf16 = out_dtype == DT_BF16;
    p.g.world = world; p.g.rank = rank; p.g.n_total = N_local * world; p.g.row_offset = rank * N_local;
    p.g.done_counter = done_counter; p.g.step_word = step_word;
    p.g.half_words = (size_t)world * M * N_local;
    for (int d = 0; d < world; d++) p.g.peer_box[d] = (uint2 *)peer_mailbox[d];
    uint64_t n = 0;
    cudaError_t e;
    // x_elem / out_elem are only used to step through token passes, of which there is one
    if (wdtype == DT_Q4K) {
        p.row_stride = (size_t)(K / QK_K) * Q4K_BLOCK_BYTES;
        e = launch_fmt<0>(p, M, 0, 0, sm_count, s, &n);
    } else if (wdtype == DT_Q6K) {
        p.row_stride = q6k_row_stride(K);
        e = launch_fmt<1>(p, M, 0, 0, sm_count, s, &n);
    } else {
        return cudaErrorInvalidValue;
    }
    if (e == cudaSuccess && n != 1) e = cudaErrorInvalidConfiguration;
    if (launches) *launches += n;
    return e;
}

}  // namespace llmrs
