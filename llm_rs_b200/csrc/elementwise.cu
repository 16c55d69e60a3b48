// The operations of a decode step other than matmul and embed: silu, mul, add
// (shaders/ops.metal:762-793), rms_norm (ops.metal:970-1003), argmax (ops.metal:803-835), rope
// (ops.metal:1011-1042), scatter_kv and gather (ops.metal:841-873) and paged attention
// (ops.metal:636-758).
// Buffers are F32 or BF16; arithmetic is float32 as in the reference's kernels, with one rounding
// to the output type.
#include "kernels.h"
#include "llmrs_common.cuh"
#include "pipeline.cuh"

namespace llmrs {

namespace {

__device__ __forceinline__ float load_f(const void *p, size_t i, int bf16) {
    return bf16 ? bf16_bits_to_f32(((const uint16_t *)p)[i]) : ((const float *)p)[i];
}
__device__ __forceinline__ void store_f(void *p, size_t i, float v, int bf16) {
    if (bf16) ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
    else ((float *)p)[i] = v;
}

// op 0: out = silu(a); 1: out = a * b; 2: out = a + b
__global__ void binary_kernel(int op, const void *a, int a_bf16, const void *b, int b_bf16, void *out, int out_bf16,
                              size_t n) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = load_f(a, i, a_bf16);
    float v;
    if (op == 0) v = x / (1.0f + expf(-x));
    else if (op == 1) v = x * load_f(b, i, b_bf16);
    else v = x + load_f(b, i, b_bf16);
    store_f(out, i, v, out_bf16);
}

// One CTA per token row: inv = rsqrt(mean(v^2) + eps); out = v * inv * weight.
__global__ void __launch_bounds__(256)
rms_norm_kernel(const void *in, int in_bf16, const float *__restrict__ weight, void *out, int out_bf16, int dim, float eps) {
    pdl_prologue();
    __shared__ float red[8];
    __shared__ float inv_s;
    const size_t off = (size_t)blockIdx.x * dim;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = load_f(in, off + i, in_bf16);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
        inv_s = rsqrtf(t / (float)dim + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        store_f(out, off + i, load_f(in, off + i, in_bf16) * inv * weight[i], out_bf16);
}

// Index of the largest value (the smallest such index on ties; NaNs never win), one CTA.
__global__ void __launch_bounds__(1024) argmax_kernel(const void *x, int bf16, uint32_t n, uint32_t *out) {
    pdl_prologue();
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    float best = -INFINITY;
    uint32_t idx = 0xFFFFFFFFu;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = load_f(x, i, bf16);
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
    auto better = [](float v, uint32_t i, float bv, uint32_t bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -INFINITY;
        idx = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : 0xFFFFFFFFu;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        if (threadIdx.x == 0) *out = idx == 0xFFFFFFFFu ? 0u : idx;      // all NaN or -inf: index 0, like the reference
    }
}

// Rotary embedding in place (shaders/ops.metal:1011-1042): x is [row_stride, seq_len] made of heads of
// head_dim; pair i of a head is (2i, 2i+1) ("interleaved") or (i, i + head_dim/2) ("split half");
// angle = position * theta^(-2i / head_dim).  One thread per pair.
// q and k go through one launch: blockIdx.z picks the buffer.
__global__ void rope_kernel(void *xq, int q_bf16, int q_stride, void *xk, int k_bf16, int k_stride,
                            const uint32_t *__restrict__ positions, int head_dim, float theta, int split_half) {
    pdl_prologue();
    void *x = blockIdx.z ? xk : xq;
    const int bf16 = blockIdx.z ? k_bf16 : q_bf16, row_stride = blockIdx.z ? k_stride : q_stride;
    const int pairs_per_row = row_stride / 2;
    const int pair = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (pair >= pairs_per_row) return;
    const int half = head_dim / 2, head = pair / half, i = pair % half;
    const size_t base = (size_t)s * row_stride + (size_t)head * head_dim;
    const size_t a = split_half ? base + i : base + 2 * i;
    const size_t b = split_half ? base + i + half : base + 2 * i + 1;
    const float freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
    const float angle = (float)positions[s] * freq;
    float sn, cs;
    sincosf(angle, &sn, &cs);
    const float x0 = load_f(x, a, bf16), x1 = load_f(x, b, bf16);
    store_f(x, a, x0 * cs - x1 * sn, bf16);
    store_f(x, b, x0 * sn + x1 * cs, bf16);
}

// rope of q and k and the two scatter_kv calls that follow it in a layer (src/arch/llama.rs:156-158) in one
// launch: blockIdx.z = 0 rotates q in place, 1 rotates k in place and writes the rotated pair into the
// key pool, 2 copies v into the value pool.  Pools and k, v share one element type.
__global__ void rope_scatter_kernel(void *q, int q_stride, void *k, const void *v, int kv_stride, int bf16,
                                    const uint32_t *__restrict__ positions, const uint32_t *__restrict__ slots,
                                    void *k_pool, void *v_pool, int head_dim, float theta, int split_half) {
    pdl_prologue();
    const int which = blockIdx.z, s = blockIdx.y;
    const int row_stride = which == 0 ? q_stride : kv_stride;
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= row_stride / 2) return;
    if (which == 2) {                                    // two values of v per thread
        const size_t src = (size_t)s * kv_stride + 2 * pair, dst = (size_t)slots[s] * kv_stride + 2 * pair;
        store_f(v_pool, dst, load_f(v, src, bf16), bf16);
        store_f(v_pool, dst + 1, load_f(v, src + 1, bf16), bf16);
        return;
    }
    void *x = which == 0 ? q : k;
    const int half = head_dim / 2, head = pair / half, i = pair % half;
    const size_t in_row = (size_t)head * head_dim + (split_half ? i : 2 * i);
    const size_t step = split_half ? half : 1;
    const size_t a = (size_t)s * row_stride + in_row, b = a + step;
    const float freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
    const float angle = (float)positions[s] * freq;
    float sn, cs;
    sincosf(angle, &sn, &cs);
    const float x0 = load_f(x, a, bf16), x1 = load_f(x, b, bf16);
    const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
    store_f(x, a, y0, bf16);
    store_f(x, b, y1, bf16);
    if (which == 1) {
        const size_t pa = (size_t)slots[s] * kv_stride + in_row;
        store_f(k_pool, pa, y0, bf16);
        store_f(k_pool, pa + step, y1, bf16);
    }
}

// pool[slot_mapping[t] * kv_dim + d] = src[t * kv_dim + d]  (ops.metal:841-853), and
// out[c * dim + d] = src[indices[c] * dim + d]              (ops.metal:859-873): rows of `width`
// elements of `esz` bytes moved by index; one of the two index sides is the identity.
__global__ void move_rows_kernel(uint8_t *dst, const uint8_t *src, const uint32_t *__restrict__ index, int scatter,
                                 size_t row_bytes, int rows) {
    pdl_prologue();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // one 2-byte unit each
    const size_t units = row_bytes / 2;
    if (i >= units * rows) return;
    const size_t r = i / units, u = i - r * units;
    const size_t from = scatter ? r : index[r], to = scatter ? index[r] : r;
    ((uint16_t *)dst)[to * units + u] = ((const uint16_t *)src)[from * units + u];
}

// Paged, variable-length, grouped-query attention with a causal mask (shaders/ops.metal:636-758).
// One CTA per (query token, head).  Keys are taken ATT_TILE positions at a time: thread j forms
// q . k_j (the key row read as 16-byte vectors, q from shared memory), the tile maximum and sum
// go through warp shuffles, and thread d accumulates sum_j p_j v_j[d] with the online-softmax
// rescaling.  A tile never crosses a page when block_size is a multiple of ATT_TILE; otherwise
// the page is looked up per position.
constexpr int ATT_TILE = 128;
constexpr int ATT_THREADS = 128;
__global__ void __launch_bounds__(ATT_THREADS)
attention_kernel(const void *q, const void *k_pool, const void *v_pool, void *out, int bf16,
                 const uint32_t *__restrict__ block_table, const uint32_t *__restrict__ query_starts,
                 const uint32_t *__restrict__ seq_lens, int n_heads, int n_kv_heads, int head_dim, int block_size,
                 int max_blocks_per_seq, int num_requests) {
    pdl_prologue();
    extern __shared__ float att_smem[];
    float *qs = att_smem;                   // [head_dim]
    float *scores = qs + head_dim;          // [ATT_TILE]
    __shared__ float red[ATT_THREADS / 32];
    __shared__ float bcast;
    const int head = blockIdx.x % n_heads, gq = blockIdx.x / n_heads;
    int req = 0;
    while (req + 1 < num_requests && (uint32_t)gq >= query_starts[req + 1]) req++;
    const int local_q = gq - (int)query_starts[req];
    const int q_count = (int)query_starts[req + 1] - (int)query_starts[req];
    const int kv_head = head / (n_heads / n_kv_heads), kv_dim = n_kv_heads * head_dim, kv_off = kv_head * head_dim;
    const float scale = rsqrtf((float)head_dim);
    const int causal_len = (int)seq_lens[req] - q_count + local_q + 1;
    const size_t q_off = (size_t)gq * n_heads * head_dim + (size_t)head * head_dim;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < head_dim; i += ATT_THREADS) qs[i] = load_f(q, q_off + i, bf16);
    __syncthreads();

    auto block_max = [&](float v) {
#pragma unroll
        for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        if (lane == 0) red[warp] = v;
        __syncthreads();
        if (tid == 0) {
            float m = red[0];
            for (int w = 1; w < ATT_THREADS / 32; w++) m = fmaxf(m, red[w]);
            bcast = m;
        }
        __syncthreads();
        return bcast;
    };
    auto block_sum = [&](float v) {
#pragma unroll
        for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        __syncthreads();                         // `red` and `bcast` of the maximum have been read
        if (lane == 0) red[warp] = v;
        __syncthreads();
        if (tid == 0) {
            float t = 0.0f;
            for (int w = 0; w < ATT_THREADS / 32; w++) t += red[w];
            bcast = t;
        }
        __syncthreads();
        return bcast;
    };
    auto kv_row = [&](int t) {                   // element offset of position t of this request in the pools
        const uint32_t page = block_table[(size_t)req * max_blocks_per_seq + t / block_size];
        return ((size_t)page * block_size + (size_t)(t % block_size)) * kv_dim + kv_off;
    };

    float acc[2] = {0.0f, 0.0f};                 // output dims tid and tid + 128 (head_dim <= 256)
    float m_i = -INFINITY, l_i = 0.0f;
    for (int t0 = 0; t0 < causal_len; t0 += ATT_TILE) {
        const int tile_len = min(ATT_TILE, causal_len - t0);
        float sc = -INFINITY;
        if (tid < tile_len) {
            const size_t row = kv_row(t0 + tid);
            float dot = 0.0f;
            if (bf16 && (head_dim % 8) == 0 && (row % 8) == 0) {
                const uint4 *kr = reinterpret_cast<const uint4 *>((const uint16_t *)k_pool + row);
                for (int i = 0; i < head_dim / 8; i++) {
                    const uint4 u = __ldg(kr + i);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        dot = fmaf(qs[8 * i + 2 * j], __uint_as_float(w[j] << 16), dot);
                        dot = fmaf(qs[8 * i + 2 * j + 1], __uint_as_float(w[j] & 0xFFFF0000u), dot);
                    }
                }
            } else {
                for (int i = 0; i < head_dim; i++) dot = fmaf(qs[i], load_f(k_pool, row + i, bf16), dot);
            }
            sc = dot * scale;
        }
        const float m_new = fmaxf(m_i, block_max(sc));
        const float rescale = __expf(m_i - m_new);       // exp(-inf) = 0 on the first tile
        const float e = tid < tile_len ? __expf(sc - m_new) : 0.0f;
        scores[tid] = e;
        const float tile_sum = block_sum(e);             // its barriers also publish scores[]
        l_i = l_i * rescale + tile_sum;
        m_i = m_new;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int d = tid + h * ATT_THREADS;
            if (d < head_dim) {
                float a = acc[h] * rescale;
                for (int j = 0; j < tile_len; j++) a = fmaf(scores[j], load_f(v_pool, kv_row(t0 + j) + d, bf16), a);
                acc[h] = a;
            }
        }
        __syncthreads();                                 // scores[] is rewritten by the next tile
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int d = tid + h * ATT_THREADS;
        if (d < head_dim) store_f(out, q_off + d, acc[h] / l_i, bf16);
    }
}

// Attention for bf16 buffers (head_dim 64 or 128, 1/2/4/8 query heads per KV head), organised around the
// memory traffic: the query heads that share a KV head are served from ONE pass over its keys and values,
// which come into shared memory 64 positions at a time by asynchronous 16-byte copies.  A long sequence
// with few query tokens (decode) is cut into `splits` ranges so that all SMs work; the ranges' partial
// (accumulator, maximum, sum) triples are merged by attention_merge_kernel.  The kernels follow further
// down (attention_decode_mma_kernel, attention_prefill_kernel); a first version that formed scores and
// weighted values on the CUDA cores took 74 us where the tensor-core one takes 40 (8 requests x 4096).
constexpr int AT2_TILE = 64;          // positions per tile: what attention_splits counts in

// 16 bytes global -> shared without a register in between (both addresses 16-byte aligned).
__device__ __forceinline__ void async_copy16(void *smem_dst, const void *gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void async_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most `Pending` of this thread's committed groups are still in flight.
template <int Pending> __device__ __forceinline__ void async_copy_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(Pending) : "memory");
}

// out = sum_s acc_s e^(m_s - m) / sum_s l_s e^(m_s - m): one CTA of HD threads per (query token, head).
// The ranges' maxima and sums are fetched by one thread each and combined with shuffles, and the
// accumulators are read eight ranges at a time: two memory round trips, where a loop over the ranges
// that used each value at once made one round trip per range (8 of the 13 us of a decode call).
__global__ void attention_merge_kernel(const float *__restrict__ partial, uint16_t *__restrict__ out, int hd, int splits,
                                       const uint32_t *__restrict__ query_starts, int n_heads, int by_request) {
    pdl_prologue();
    __shared__ float w_s[32];
    __shared__ float l_total;
    size_t th = blockIdx.x;                              // token * n_heads + head
    if (by_request) {                                    // request * n_heads + head: single-token requests only
        const int req = (int)(blockIdx.x / (unsigned)n_heads), head = (int)(blockIdx.x % (unsigned)n_heads);
        if ((int)query_starts[req + 1] - (int)query_starts[req] != 1) return;
        th = (size_t)query_starts[req] * n_heads + head;
    }
    const float *pr = partial + th * splits * (hd + 2);
    const int d = threadIdx.x;
    if (d < 32) {                                        // splits <= 32
        const float ms = d < splits ? pr[d * (hd + 2) + hd] : -INFINITY;
        const float ls = d < splits ? pr[d * (hd + 2) + hd + 1] : 0.0f;
        float m = ms;
#pragma unroll
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float w = ms == -INFINITY ? 0.0f : __expf(ms - m);
        float l = ls * w;
#pragma unroll
        for (int o = 16; o; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        w_s[d] = w;
        if (d == 0) l_total = l;
    }
    float a = 0.0f;
    int s = 0;
    for (; s + 8 <= splits; s += 8) {                    // the eight loads go out before the first is used
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = pr[(s + i) * (hd + 2) + d];
        if (s == 0) __syncthreads();                     // w_s is ready; the loads above did not need it
#pragma unroll
        for (int i = 0; i < 8; i++) a = fmaf(v[i], w_s[s + i], a);
    }
    if (s == 0) __syncthreads();
    for (; s < splits; s++) a = fmaf(pr[s * (hd + 2) + d], w_s[s], a);
    out[th * hd + d] = __bfloat16_as_ushort(__float2bfloat16_rn(a / l_total));
}

// ---- prefill attention on the tensor cores -------------------------------------------------------
// Requests with several query tokens (prefill, chunked prefill): one CTA per (request, 64 / GROUP
// consecutive query tokens, KV head).  The CTA's 64 rows are (token, head of the group) pairs, 16 per
// warp, so one key / value tile serves every head of the group and every token of the chunk.  Per tile
// of 64 positions: S = Q K^T and O += P V run as mma.sync m16n8k16 (bf16 in, fp32 out) with the
// running maximum and sum of each row in registers (the score fragments of S are the A fragments of
// P V as they stand).  Keys and values come into shared memory by asynchronous 16-byte copies; rows are
// 8 elements longer than head_dim so that fragment reads fall on distinct banks.
constexpr int FA_BN = 64;             // positions per tile
constexpr int FA_THREADS = 128;       // four warps of 16 rows

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (lo, hi) -> packed bf16x2, lo in the low half, round to nearest even
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Four 8x8 b16 matrices from shared memory: lane i gives the address of row i % 8 of matrix i / 8 and
// receives, of every matrix, elements (row lane / 4, columns 2 (lane % 4), +1); transposed: (rows
// 2 (lane % 4), +1, column lane / 4).  These are the B fragments of mma.m16n8k16 as they stand.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *row_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(row_ptr)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *row_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(row_ptr)));
}

template <int HD, int GROUP>
__global__ void __launch_bounds__(FA_THREADS)
attention_prefill_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k_pool,
                         const uint16_t *__restrict__ v_pool, uint16_t *__restrict__ out,
                         const uint32_t *__restrict__ block_table, const uint32_t *__restrict__ query_starts,
                         const uint32_t *__restrict__ seq_lens, int n_heads, int n_kv_heads, int block_size,
                         int max_blocks_per_seq, int num_requests, int skip_single) {
    pdl_prologue();
    constexpr int TOK = 64 / GROUP;                      // query tokens per CTA
    constexpr int STRIDE = HD + 8;                       // elements per shared-memory row
    constexpr int KS = HD / 16, NT = HD / 8, CH = HD / 8;
    constexpr int TILE = FA_BN * STRIDE;                 // elements of one key (or value) tile
    extern __shared__ __align__(16) uint16_t fa_s[];     // [2 buffers][key tile | value tile]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.y;
    // which request and which chunk of its query tokens: the grid holds a chunk count that no batch exceeds
    int req = 0, chunk = blockIdx.x;
    for (; req < num_requests; req++) {
        const int cnt = (int)query_starts[req + 1] - (int)query_starts[req];
        // requests of one query token are the split-sequence kernel's when it runs beside this one
        const int chunks = skip_single && cnt == 1 ? 0 : (cnt + TOK - 1) / TOK;
        if (chunk < chunks) {
            chunk = chunks - 1 - chunk;                  // late chunks see the most positions: they start first
            break;
        }
        chunk -= chunks;
    }
    if (req >= num_requests) return;
    const int q_begin = (int)query_starts[req], q_count = (int)query_starts[req + 1] - q_begin;
    const int tok0 = chunk * TOK;
    const int base_len = (int)seq_lens[req] - q_count;   // positions in front of the request's first query token
    const int kv_dim = n_kv_heads * HD, kv_off = kvh * HD;
    // this thread's two rows: r0 = 16 warp + g and r0 + 8; row -> (token tok0 + row / GROUP, head row % GROUP)
    const int r0 = 16 * warp + g, r1 = r0 + 8;
    const int tl0 = tok0 + r0 / GROUP, tl1 = tok0 + r1 / GROUP;
    const bool ok0 = tl0 < q_count, ok1 = tl1 < q_count;
    const int len0 = ok0 ? base_len + tl0 + 1 : 0, len1 = ok1 ? base_len + tl1 + 1 : 0;    // causal: visible positions
    const size_t qo0 = ((size_t)(q_begin + tl0) * n_heads + (size_t)kvh * GROUP + r0 % GROUP) * HD;
    const size_t qo1 = ((size_t)(q_begin + tl1) * n_heads + (size_t)kvh * GROUP + r1 % GROUP) * HD;
    uint32_t qa[KS][4];                                  // the rows' queries as A fragments
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const int c = 16 * ks + 2 * t;
        qa[ks][0] = ok0 ? *reinterpret_cast<const uint32_t *>(q + qo0 + c) : 0u;
        qa[ks][1] = ok1 ? *reinterpret_cast<const uint32_t *>(q + qo1 + c) : 0u;
        qa[ks][2] = ok0 ? *reinterpret_cast<const uint32_t *>(q + qo0 + c + 8) : 0u;
        qa[ks][3] = ok1 ? *reinterpret_cast<const uint32_t *>(q + qo1 + c + 8) : 0u;
    }
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    const float sc = rsqrtf((float)HD) * 1.4426950408889634f;      // scores in units of log2: exp2f below
    const int kv_len = base_len + min(tok0 + TOK, q_count);         // what the chunk's last token sees

    // the tile that starts at position p0 -> buffer `buf`, asynchronously (rows past the range: zeros, not
    // stale bits, since 0 * NaN would poison P V)
    auto fetch_tile = [&](int p0, int buf) {
        uint16_t *kb = fa_s + buf * 2 * TILE, *vb = kb + TILE;
        for (int c = tid; c < FA_BN * CH; c += FA_THREADS) {
            const int j = c / CH, ch = c % CH;
            uint16_t *kd = kb + j * STRIDE + 8 * ch, *vd = vb + j * STRIDE + 8 * ch;
            const int pos = p0 + j;
            if (pos < kv_len) {
                const uint32_t page = block_table[(size_t)req * max_blocks_per_seq + pos / block_size];
                const size_t row = ((size_t)page * block_size + (size_t)(pos % block_size)) * kv_dim + kv_off;
                async_copy16(kd, k_pool + row + 8 * ch);
                async_copy16(vd, v_pool + row + 8 * ch);
            } else {
                *reinterpret_cast<uint4 *>(kd) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(vd) = make_uint4(0, 0, 0, 0);
            }
        }
        async_copy_commit();
    };
    if (kv_len > 0) fetch_tile(0, 0);
    int buf = 0;
    for (int p0 = 0; p0 < kv_len; p0 += FA_BN, buf ^= 1) {
        const uint16_t *k_s = fa_s + buf * 2 * TILE, *v_s = k_s + TILE;
        // the other buffer was last read before the barrier that closed the previous iteration
        if (p0 + FA_BN < kv_len) {
            fetch_tile(p0 + FA_BN, buf ^ 1);             // travels while this tile is worked on
            async_copy_wait<1>();
        } else {
            async_copy_wait<0>();
        }
        __syncthreads();
        // ---- S = Q K^T: 16 rows x 64 positions per warp ----
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
        const int lm = lane >> 3, lr = lane & 7;          // ldmatrix: this lane addresses row lr of matrix lm
#pragma unroll
        for (int ks = 0; ks < KS; ks++)
#pragma unroll
            for (int nt = 0; nt < 8; nt += 2) {
                // B fragments (k = dimension, n = position) of position tiles nt and nt + 1:
                // matrices (nt, dims 0-7), (nt, dims 8-15), (nt + 1, dims 0-7), (nt + 1, dims 8-15) of the step
                uint32_t b[4];
                ldmatrix_x4(b, k_s + (8 * (nt + (lm >> 1)) + lr) * STRIDE + 16 * ks + 8 * (lm & 1));
                mma_bf16(s[nt], qa[ks], b[0], b[1]);
                mma_bf16(s[nt + 1], qa[ks], b[2], b[3]);
            }
        // ---- scale, causal mask, running maximum ----
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int pos = p0 + 8 * nt + 2 * t + e;
                s[nt][e] = pos < len0 ? s[nt][e] * sc : -INFINITY;
                s[nt][2 + e] = pos < len1 ? s[nt][2 + e] * sc : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
#pragma unroll
        for (int sh = 1; sh <= 2; sh <<= 1) {            // the four lanes of a quad hold one row
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float u0 = mn0 == -INFINITY ? 0.0f : mn0, u1 = mn1 == -INFINITY ? 0.0f : mn1;   // rows that see nothing yet
        const float f0 = exp2f(m0 - u0), f1 = exp2f(m1 - u1);
        m0 = mn0;
        m1 = mn1;
        float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                s[nt][e] = exp2f(s[nt][e] - u0);
                s[nt][2 + e] = exp2f(s[nt][2 + e] - u1);
                sum0 += s[nt][e];
                sum1 += s[nt][2 + e];
            }
        l0 = l0 * f0 + sum0;                             // this lane's columns only; the quad adds up at the end
        l1 = l1 * f1 + sum1;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            o[nt][0] *= f0; o[nt][1] *= f0;
            o[nt][2] *= f1; o[nt][3] *= f1;
        }
        // ---- O += P V: the score fragments are the A fragments of this product ----
#pragma unroll
        for (int j = 0; j < FA_BN / 16; j++) {
            const uint32_t pa[4] = {pack_bf16(s[2 * j][0], s[2 * j][1]), pack_bf16(s[2 * j][2], s[2 * j][3]),
                                    pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]), pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3])};
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                // B fragments (k = position, n = dimension) of dimension tiles nt and nt + 1, transposed on the way:
                // matrices (positions 0-7, nt), (positions 8-15, nt), (0-7, nt + 1), (8-15, nt + 1) of the step
                uint32_t b[4];
                ldmatrix_x4_trans(b, v_s + (16 * j + 8 * (lm & 1) + lr) * STRIDE + 8 * (nt + (lm >> 1)));
                mma_bf16(o[nt], pa, b[0], b[1]);
                mma_bf16(o[nt + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();                                 // every warp is done with this buffer
    }
#pragma unroll
    for (int sh = 1; sh <= 2; sh <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
        l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
    }
    const float i0 = ok0 ? 1.0f / l0 : 0.0f, i1 = ok1 ? 1.0f / l1 : 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int c = 8 * nt + 2 * t;
        if (ok0) *reinterpret_cast<uint32_t *>(out + qo0 + c) = pack_bf16(o[nt][0] * i0, o[nt][1] * i0);
        if (ok1) *reinterpret_cast<uint32_t *>(out + qo1 + c) = pack_bf16(o[nt][2] * i1, o[nt][3] * i1);
    }
}

// ---- decode attention on the tensor cores --------------------------------------------------------
// One CTA per (query token, KV head, range of the sequence); scores and weighted values are mma.sync m16n8k16: the group's heads are rows
// 0 .. GROUP-1 of the 16-row A operand (the rest are zero), and the four warps split a tile's 64 positions,
// 16 each, every warp keeping its own running maximum, sum and accumulator over the positions it sees;
// the four meet in shared memory at the end.  Per tile a warp issues 2 x HD/16 + HD/8 MMAs where the
// CUDA-core kernel spends ~1000 multiply-adds per thread.
template <int HD, int GROUP>
__global__ void __launch_bounds__(FA_THREADS)
attention_decode_mma_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k_pool,
                            const uint16_t *__restrict__ v_pool, uint16_t *__restrict__ out, float *__restrict__ partial,
                            const uint32_t *__restrict__ block_table, const uint32_t *__restrict__ query_starts,
                            const uint32_t *__restrict__ seq_lens, int n_heads, int n_kv_heads, int block_size,
                            int max_blocks_per_seq, int num_requests, int splits, int by_request) {
    pdl_prologue();
    constexpr int STRIDE = HD + 8;
    constexpr int KS = HD / 16, NT = HD / 8, CH = HD / 8;
    constexpr int TILE = FA_BN * STRIDE;
    static_assert(4 * GROUP * (HD + 2) * 4 <= 2 * TILE * 2, "the warps' results reuse the first tile buffer");
    extern __shared__ __align__(16) uint16_t fa_s[];     // [2 buffers][key tile | value tile]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.x % n_kv_heads, split = blockIdx.y;
    int gq = blockIdx.x / n_kv_heads, req = 0;
    if (by_request) {                                    // mixed batch: requests with one query token only
        req = gq;
        if ((int)query_starts[req + 1] - (int)query_starts[req] != 1) return;
        gq = (int)query_starts[req];
    } else {
        while (req + 1 < num_requests && (uint32_t)gq >= query_starts[req + 1]) req++;
    }
    const int local_q = gq - (int)query_starts[req];
    const int q_count = (int)query_starts[req + 1] - (int)query_starts[req];
    const int causal_len = (int)seq_lens[req] - q_count + local_q + 1;
    const int kv_dim = n_kv_heads * HD, kv_off = kvh * HD;
    const int tiles = (causal_len + FA_BN - 1) / FA_BN;
    const int per = (tiles + splits - 1) / splits;
    const int t_begin = min(split * per, tiles) * FA_BN, t_end = min(min((split + 1) * per, tiles) * FA_BN, causal_len);
    const size_t q_off = (size_t)gq * n_heads * HD + (size_t)kvh * GROUP * HD;
    const bool row_ok = g < GROUP;                       // row g of the A operand is head g of the group
    uint32_t qa[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const int c = 16 * ks + 2 * t;
        qa[ks][0] = row_ok ? *reinterpret_cast<const uint32_t *>(q + q_off + (size_t)g * HD + c) : 0u;
        qa[ks][2] = row_ok ? *reinterpret_cast<const uint32_t *>(q + q_off + (size_t)g * HD + c + 8) : 0u;
        qa[ks][1] = qa[ks][3] = 0u;                      // rows 8 .. 15: no heads there
    }
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;               // of row g, over this warp's positions
    const float sc = rsqrtf((float)HD);

    auto fetch_tile = [&](int p0, int buf) {
        uint16_t *kb = fa_s + buf * 2 * TILE, *vb = kb + TILE;
        for (int c = tid; c < FA_BN * CH; c += FA_THREADS) {
            const int j = c / CH, ch = c % CH;
            uint16_t *kd = kb + j * STRIDE + 8 * ch, *vd = vb + j * STRIDE + 8 * ch;
            const int pos = p0 + j;
            if (pos < t_end) {
                const uint32_t page = block_table[(size_t)req * max_blocks_per_seq + pos / block_size];
                const size_t row = ((size_t)page * block_size + (size_t)(pos % block_size)) * kv_dim + kv_off;
                async_copy16(kd, k_pool + row + 8 * ch);
                async_copy16(vd, v_pool + row + 8 * ch);
            } else {
                *reinterpret_cast<uint4 *>(kd) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(vd) = make_uint4(0, 0, 0, 0);
            }
        }
        async_copy_commit();
    };
    if (t_begin < t_end) fetch_tile(t_begin, 0);
    int buf = 0;
    const int lm = lane >> 3, lr = lane & 7;
    for (int p0 = t_begin; p0 < t_end; p0 += FA_BN, buf ^= 1) {
        const uint16_t *k_s = fa_s + buf * 2 * TILE, *v_s = k_s + TILE;
        if (p0 + FA_BN < t_end) {
            fetch_tile(p0 + FA_BN, buf ^ 1);
            async_copy_wait<1>();
        } else {
            async_copy_wait<0>();
        }
        __syncthreads();
        // ---- scores of this warp's 16 positions: two position tiles ----
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            uint32_t b[4];
            ldmatrix_x4(b, k_s + (16 * warp + 8 * (lm >> 1) + lr) * STRIDE + 16 * ks + 8 * (lm & 1));
            mma_bf16(s[0], qa[ks], b[0], b[1]);
            mma_bf16(s[1], qa[ks], b[2], b[3]);
        }
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int pos = p0 + 16 * warp + 8 * nt + 2 * t + e;
                s[nt][e] = pos < t_end ? s[nt][e] * sc : -INFINITY;
                mx = fmaxf(mx, s[nt][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;
        const float f = __expf(m_run - m_use);
        m_run = m_new;
        float sum = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                s[nt][e] = __expf(s[nt][e] - m_use);
                sum += s[nt][e];
            }
        l_run = l_run * f + sum;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { o[nt][0] *= f; o[nt][1] *= f; }
        // ---- weighted values: one step of 16 positions ----
        const uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), 0u, pack_bf16(s[1][0], s[1][1]), 0u};
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_s + (16 * warp + 8 * (lm & 1) + lr) * STRIDE + 8 * (nt + (lm >> 1)));
            mma_bf16(o[nt], pa, b[0], b[1]);
            mma_bf16(o[nt + 1], pa, b[2], b[3]);
        }
        __syncthreads();
    }
    // ---- the four warps' results meet in shared memory (the tile buffers are no longer read) ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    float *res = reinterpret_cast<float *>(fa_s);        // [warp][head][HD accumulator values, maximum, sum]
    if (row_ok) {
        float *r = res + (size_t)(warp * GROUP + g) * (HD + 2);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            r[8 * nt + 2 * t] = o[nt][0];
            r[8 * nt + 2 * t + 1] = o[nt][1];
        }
        if (t == 0) { r[HD] = m_run; r[HD + 1] = l_run; }
    }
    __syncthreads();
    for (int i = tid; i < GROUP * HD; i += FA_THREADS) {
        const int h = i / HD, d = i % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) m = fmaxf(m, res[(size_t)(w * GROUP + h) * (HD + 2) + HD]);
        float acc = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float *r = res + (size_t)(w * GROUP + h) * (HD + 2);
            const float wt = r[HD] == -INFINITY ? 0.0f : __expf(r[HD] - m);
            acc = fmaf(r[d], wt, acc);
            l = fmaf(r[HD + 1], wt, l);
        }
        const int head = kvh * GROUP + h;
        if (splits == 1) {
            out[(size_t)gq * n_heads * HD + (size_t)head * HD + d] = __bfloat16_as_ushort(__float2bfloat16_rn(acc / l));
        } else {
            float *pr = partial + (((size_t)gq * n_heads + head) * splits + split) * (HD + 2);
            pr[d] = acc;
            if (d == 0) { pr[HD] = m; pr[HD + 1] = l; }
        }
    }
}

}  // namespace

size_t attention_workspace_bytes(int total_query_tokens, int n_heads, int head_dim, int splits) {
    return splits <= 1 ? 0 : (size_t)total_query_tokens * n_heads * splits * (head_dim + 2) * sizeof(float);
}

// How many ranges to cut the sequences into: enough CTAs for two per SM, ranges of at least one tile
// (a single decode request is a chain of dependent tiles: the shorter the chain, the sooner it ends).
int attention_splits(int total_query_tokens, int n_kv_heads, int max_seq_len, int sm_count) {
    const int ctas = total_query_tokens * n_kv_heads;
    const int want = (2 * sm_count + ctas - 1) / ctas;
    const int most = (max_seq_len + AT2_TILE - 1) / AT2_TILE;
    const int s = want < most ? want : most;
    return s < 1 ? 1 : (s > 32 ? 32 : s);
}

template <int HD>
static cudaError_t launch_gqa_hd(int group, dim3 grid, cudaStream_t s, const uint16_t *q, const uint16_t *k,
                                 const uint16_t *v, uint16_t *out, float *partial, const uint32_t *bt,
                                 const uint32_t *qs, const uint32_t *sl, int n_heads, int n_kv, int block_size,
                                 int max_blocks, int n_req, int splits, int by_request, bool pdl) {
    constexpr size_t smem = (size_t)2 * 2 * FA_BN * (HD + 8) * sizeof(uint16_t);      // two buffers of a key and a value tile
#define LLMRS_GQA(G) { cudaError_t ea = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (ea != cudaSuccess) return ea; \
    return launch_dependent(attention_decode_mma_kernel<HD, G>, grid, dim3(FA_THREADS), smem, s, pdl, q, k, v, out, partial, bt, qs, sl, n_heads, n_kv, block_size, max_blocks, n_req, splits, by_request); }
    switch (group) {
        case 1: LLMRS_GQA(1)
        case 2: LLMRS_GQA(2)
        case 4: LLMRS_GQA(4)
        case 8: LLMRS_GQA(8)
        default: return cudaErrorInvalidValue;
    }
#undef LLMRS_GQA
}

// Chunks of query tokens the grid must hold: every request may end in a partial chunk.
template <int HD>
static cudaError_t launch_prefill_hd(int group, int total_q, int num_req, int n_kv, cudaStream_t s, bool pdl, const uint16_t *q,
                                     const uint16_t *k, const uint16_t *v, uint16_t *out, const uint32_t *bt,
                                     const uint32_t *qs, const uint32_t *sl, int n_heads, int block_size, int max_blocks,
                                     int skip_single) {
    constexpr size_t smem = (size_t)2 * 2 * FA_BN * (HD + 8) * sizeof(uint16_t);      // two buffers of a key and a value tile
#define LLMRS_FA(G) { const int tok = 64 / G; const dim3 grid((unsigned)((total_q + tok - 1) / tok + num_req), (unsigned)n_kv); \
    cudaError_t ea = cudaFuncSetAttribute(attention_prefill_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (ea != cudaSuccess) return ea; \
    return launch_dependent(attention_prefill_kernel<HD, G>, grid, dim3(FA_THREADS), smem, s, pdl, q, k, v, out, bt, qs, sl, n_heads, n_kv, block_size, max_blocks, num_req, skip_single); }
    switch (group) {
        case 1: LLMRS_FA(1)
        case 2: LLMRS_FA(2)
        case 4: LLMRS_FA(4)
        case 8: LLMRS_FA(8)
        default: return cudaErrorInvalidValue;
    }
#undef LLMRS_FA
}

cudaError_t launch_attention_prefill(const void *q, const void *k_pool, const void *v_pool, void *out,
                                     const uint32_t *block_table, const uint32_t *query_starts, const uint32_t *seq_lens,
                                     int total_query_tokens, int num_requests, int n_heads, int n_kv_heads, int head_dim,
                                     int block_size, int max_blocks_per_seq, bool skip_single_token_requests, cudaStream_t s,
                                     bool pdl) {
    if (total_query_tokens <= 0) return cudaSuccess;
    const int group = n_heads / n_kv_heads;
    const int skip_single = skip_single_token_requests ? 1 : 0;
    if (head_dim == 128)
        return launch_prefill_hd<128>(group, total_query_tokens, num_requests, n_kv_heads, s, pdl, (const uint16_t *)q,
                                      (const uint16_t *)k_pool, (const uint16_t *)v_pool, (uint16_t *)out, block_table,
                                      query_starts, seq_lens, n_heads, block_size, max_blocks_per_seq, skip_single);
    return launch_prefill_hd<64>(group, total_query_tokens, num_requests, n_kv_heads, s, pdl, (const uint16_t *)q,
                                 (const uint16_t *)k_pool, (const uint16_t *)v_pool, (uint16_t *)out, block_table,
                                 query_starts, seq_lens, n_heads, block_size, max_blocks_per_seq, skip_single);
}

bool attention_gqa_supported(int dtype, int n_heads, int n_kv_heads, int head_dim) {
    const int group = n_kv_heads ? n_heads / n_kv_heads : 0;
    return dtype == DT_BF16 && (head_dim == 64 || head_dim == 128) && (group == 1 || group == 2 || group == 4 || group == 8);
}

cudaError_t launch_attention_gqa(const void *q, const void *k_pool, const void *v_pool, void *out, float *workspace,
                                 const uint32_t *block_table, const uint32_t *query_starts, const uint32_t *seq_lens,
                                 int total_query_tokens, int num_requests, int n_heads, int n_kv_heads, int head_dim,
                                 int block_size, int max_blocks_per_seq, int splits, bool single_token_requests_only,
                                 cudaStream_t s, bool pdl) {
    if (total_query_tokens <= 0) return cudaSuccess;
    const int by_request = single_token_requests_only ? 1 : 0;
    const int units = by_request ? num_requests : total_query_tokens;       // what the grid runs over
    const dim3 grid((unsigned)(units * n_kv_heads), (unsigned)splits);
    const int group = n_heads / n_kv_heads;
    cudaError_t e = head_dim == 128
        ? launch_gqa_hd<128>(group, grid, s, (const uint16_t *)q, (const uint16_t *)k_pool, (const uint16_t *)v_pool,
                             (uint16_t *)out, workspace, block_table, query_starts, seq_lens, n_heads, n_kv_heads,
                             block_size, max_blocks_per_seq, num_requests, splits, by_request, pdl)
        : launch_gqa_hd<64>(group, grid, s, (const uint16_t *)q, (const uint16_t *)k_pool, (const uint16_t *)v_pool,
                            (uint16_t *)out, workspace, block_table, query_starts, seq_lens, n_heads, n_kv_heads,
                            block_size, max_blocks_per_seq, num_requests, splits, by_request, pdl);
    if (e != cudaSuccess || splits == 1) return e;
    return launch_dependent(attention_merge_kernel, dim3((unsigned)(units * n_heads)), dim3(head_dim), 0, s,
                            pdl, (const float *)workspace, (uint16_t *)out, head_dim, splits, query_starts, n_heads, by_request);
}

cudaError_t launch_rope(void *q, int q_dtype, int q_stride, void *k, int k_dtype, int k_stride, const uint32_t *positions,
                        int head_dim, float theta, int seq_len, int split_half, cudaStream_t s, bool pdl) {
    const int pairs = (q_stride > k_stride ? q_stride : k_stride) / 2;
    if (pairs <= 0 || seq_len <= 0) return cudaSuccess;
    return launch_dependent(rope_kernel, dim3((unsigned)((pairs + 255) / 256), (unsigned)seq_len, 2), dim3(256), 0, s, pdl,
                            q, (int)(q_dtype == DT_BF16), q_stride, k, (int)(k_dtype == DT_BF16), k_stride, positions,
                            head_dim, theta, split_half);
}

cudaError_t launch_rope_scatter(void *q, int q_stride, void *k, const void *v, int kv_stride, int dtype,
                                const uint32_t *positions, const uint32_t *slots, void *k_pool, void *v_pool,
                                int head_dim, float theta, int seq_len, int split_half, cudaStream_t s, bool pdl) {
    const int pairs = (q_stride > kv_stride ? q_stride : kv_stride) / 2;
    if (pairs <= 0 || seq_len <= 0) return cudaSuccess;
    return launch_dependent(rope_scatter_kernel, dim3((unsigned)((pairs + 255) / 256), (unsigned)seq_len, 3), dim3(256), 0, s,
                            pdl, q, q_stride, k, v, kv_stride, (int)(dtype == DT_BF16), positions, slots, k_pool, v_pool,
                            head_dim, theta, split_half);
}

cudaError_t launch_move_rows(void *dst, const void *src, const uint32_t *index, int scatter, size_t row_bytes,
                             int rows, cudaStream_t s, bool pdl) {
    const size_t n = row_bytes / 2 * (size_t)rows;
    if (n == 0) return cudaSuccess;
    return launch_dependent(move_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, pdl, (uint8_t *)dst,
                            (const uint8_t *)src, index, scatter, row_bytes, rows);
}

cudaError_t launch_attention(const void *q, const void *k_pool, const void *v_pool, void *out, int dtype,
                             const uint32_t *block_table, const uint32_t *query_starts, const uint32_t *seq_lens,
                             int total_query_tokens, int num_requests, int n_heads, int n_kv_heads, int head_dim,
                             int block_size, int max_blocks_per_seq, cudaStream_t s, bool pdl) {
    if (total_query_tokens <= 0) return cudaSuccess;
    const size_t smem = (size_t)(head_dim + ATT_TILE) * sizeof(float);
    return launch_dependent(attention_kernel, dim3((unsigned)(total_query_tokens * n_heads)), dim3(ATT_THREADS), smem, s,
                            pdl, q, k_pool, v_pool, out, (int)(dtype == DT_BF16), block_table, query_starts, seq_lens,
                            n_heads, n_kv_heads, head_dim, block_size, max_blocks_per_seq, num_requests);
}

cudaError_t launch_elementwise(int op, const void *a, int a_dtype, const void *b, int b_dtype, void *out,
                               int out_dtype, size_t n, cudaStream_t s, bool pdl) {
    if (n == 0) return cudaSuccess;
    return launch_dependent(binary_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, pdl, op, a,
                            (int)(a_dtype == DT_BF16), b, (int)(b_dtype == DT_BF16), out, (int)(out_dtype == DT_BF16), n);
}

cudaError_t launch_rms_norm(const void *in, int in_dtype, const float *weight, void *out, int out_dtype, int dim,
                            int rows, float eps, cudaStream_t s, bool pdl) {
    if (dim <= 0 || rows <= 0) return cudaSuccess;
    return launch_dependent(rms_norm_kernel, dim3((unsigned)rows), dim3(256), 0, s, pdl, in, (int)(in_dtype == DT_BF16),
                            weight, out, (int)(out_dtype == DT_BF16), dim, eps);
}

cudaError_t launch_argmax(const void *x, int dtype, uint32_t n, uint32_t *dev_out, cudaStream_t s) {
    argmax_kernel<<<1, 1024, 0, s>>>(x, dtype == DT_BF16, n, dev_out);
    return cudaGetLastError();
}

}  // namespace llmrs
