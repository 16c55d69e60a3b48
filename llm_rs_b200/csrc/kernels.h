// Internal launchers shared between the kernel translation units and the C ABI.
// Everything here is host-callable C++; kernels live in the .cu files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace llmrs {

constexpr int QK_K = 256;            // weights per K-quant block (src/tensor/mod.rs:43)
constexpr int Q4K_BLOCK_BYTES = 144; // src/tensor/mod.rs:71
constexpr int Q6K_BLOCK_BYTES = 210; // src/tensor/mod.rs:73

// Where a kernel reports an abandoned wait, and how long its waits may last.  Every wait inside a
// kernel (on an mbarrier, on a peer's mailbox word, on another CTA's partial sums) gives up after a
// number of polls, writes a KernelError to `word` (first error wins) and lets the kernel finish, so
// that the context stays usable and the host learns of it at its next synchronisation point.  The
// defaults are seconds; a context may shorten them (LLMRS_WAIT_POLLS), which is how the give-up path
// is tested without hanging anything.
constexpr uint32_t DEFAULT_MBAR_POLLS = 1u << 22;      // mbarrier.try_wait polls (each blocks ~1 us in hardware)
constexpr uint32_t DEFAULT_GATHER_POLLS = 1u << 25;    // mailbox polls, 32 ns apart
struct ErrSink {
    uint32_t *word;
    uint32_t mbar_polls, gather_polls;
    ErrSink(uint32_t *w = nullptr, uint32_t m = DEFAULT_MBAR_POLLS, uint32_t g = DEFAULT_GATHER_POLLS)
        : word(w), mbar_polls(m), gather_polls(g) {}
};

// GGUF dtype ids (src/tensor/mod.rs:3-33); same values as enum llmrs_dtype.
constexpr int DT_F32 = 0, DT_F16 = 1, DT_Q4_0 = 2, DT_Q8_0 = 8, DT_Q4K = 12, DT_Q6K = 14, DT_BF16 = 30;

// Device layout of Q6_K weights ("slice-major chunks", LLMRS_LAYOUT_Q6K_SLICES).  A row is cut
// into chunks of 16 blocks (the last chunk of a row may hold fewer, nbc).  A chunk holds the same
// 210*nbc bytes as the GGUF blocks it came from, regrouped so that every field a lane reads is
// 16-byte aligned and consecutive lanes hit distinct shared-memory banks:
//   [4*nbc slices of 48 B]  slice 4b+2h+c = ql[64h+16c .. +16) | ql[64h+32+16c .. +16) | qh[32h+16c .. +16)
//                           of block b (h = 0,1 half of the block, c = 0,1)
//   [nbc * 16 B]            the int8 scales of block b at 16b
//   [nbc * 2 B]             the f16 d of block b at 2b
// Chunk ci of a row starts at byte 3360*ci of the row; rows are round_up(210*nb, 32) bytes apart,
// so that the 96 bytes of a block half (slices (h,0) and (h,1)) are three aligned 32-byte sectors.
inline size_t q6k_row_stride(int K) {
    size_t nb = (size_t)K / QK_K;
    return (nb * Q6K_BLOCK_BYTES + 31) / 32 * 32;
}

// Device bytes a [K, N] weight occupies in the layout the kernels read (+16 so a bulk copy of
// the last, padded row segment stays inside the allocation).
inline size_t weight_device_bytes(int dtype, int K, int N) {
    if (dtype == DT_Q4K) return (size_t)N * (K / QK_K) * Q4K_BLOCK_BYTES;
    if (dtype == DT_Q6K) return (size_t)N * q6k_row_stride(K) + 16;
    return 0;
}

// Raw GGUF Q6_K rows -> slice-major chunks (one-off, at upload).
cudaError_t launch_q6k_repack(const uint8_t *raw, uint8_t *dev, int K, int N, cudaStream_t s);

// Weight -> float32 [N, K], bit-exact with the reference's CPU dequantisation.
cudaError_t launch_dequant(int wdtype, const uint8_t *w, int K, int N, float *out, cudaStream_t s);

// Embedding lookup: column s of out [K, n_tokens] = dequantised row dev_tokens[s] of the table
// ([K, vocab], as uploaded); out_dtype DT_F32 or DT_BF16.  grid.y = n_tokens <= 65535.
cudaError_t launch_embed(int wdtype, const uint8_t *table, int K, uint32_t vocab, const uint32_t *dev_tokens,
                         int n_tokens, void *out, int out_dtype, uint32_t *err_word, cudaStream_t s);

// (pdl, here and below: launch with programmatic stream serialization; the kernels wait for their
// predecessor before touching memory, so only the launch latency between dependent kernels goes.)
// Element-wise ops on n values (op 0: out = silu(a); 1: out = a * b; 2: out = a + b), per-row RMS norm
// ([rows] rows of dim values, float32 weight[dim]) and argmax of n values into *dev_out.
cudaError_t launch_elementwise(int op, const void *a, int a_dtype, const void *b, int b_dtype, void *out,
                               int out_dtype, size_t n, cudaStream_t s, bool pdl);
cudaError_t launch_rms_norm(const void *in, int in_dtype, const float *weight, void *out, int out_dtype, int dim,
                            int rows, float eps, cudaStream_t s, bool pdl);
cudaError_t launch_argmax(const void *x, int dtype, uint32_t n, uint32_t *dev_out, cudaStream_t s);
// Rotary embedding in place on q [q_stride, seq_len] and k [k_stride, seq_len] in one launch; scatter (dst[index[r]] = src[r]) or gather
// (dst[r] = src[index[r]]) of `rows` rows of row_bytes bytes; paged causal grouped-query attention.
cudaError_t launch_rope(void *q, int q_dtype, int q_stride, void *k, int k_dtype, int k_stride, const uint32_t *positions,
                        int head_dim, float theta, int seq_len, int split_half, cudaStream_t s, bool pdl);
// rope of q and k plus the scatter of the rotated k and of v into their pools, one launch (one element type).
cudaError_t launch_rope_scatter(void *q, int q_stride, void *k, const void *v, int kv_stride, int dtype,
                                const uint32_t *positions, const uint32_t *slots, void *k_pool, void *v_pool,
                                int head_dim, float theta, int seq_len, int split_half, cudaStream_t s, bool pdl);
cudaError_t launch_move_rows(void *dst, const void *src, const uint32_t *index, int scatter, size_t row_bytes,
                             int rows, cudaStream_t s, bool pdl);
// The bf16 attention organised around its memory traffic (head_dim 64 or 128, 1/2/4/8 query heads per
// KV head): one pass over a KV head's keys and values serves its whole group, long sequences are
// cut into `splits` ranges (attention_splits) whose partial results go through `workspace`
// (attention_workspace_bytes) and a merge kernel.
bool attention_gqa_supported(int dtype, int n_heads, int n_kv_heads, int head_dim);
int attention_splits(int total_query_tokens, int n_kv_heads, int max_seq_len, int sm_count);
size_t attention_workspace_bytes(int total_query_tokens, int n_heads, int head_dim, int splits);
cudaError_t launch_attention_gqa(const void *q, const void *k_pool, const void *v_pool, void *out, float *workspace,
                                 const uint32_t *block_table, const uint32_t *query_starts, const uint32_t *seq_lens,
                                 int total_query_tokens, int num_requests, int n_heads, int n_kv_heads, int head_dim,
                                 int block_size, int max_blocks_per_seq, int splits, bool single_token_requests_only,
                                 cudaStream_t s, bool pdl);
// The same shapes and types where requests bring several query tokens (prefill): scores and weighted
// values on the tensor cores (mma.sync, bf16), one CTA per (request, 64 / group consecutive query tokens,
// KV head); no workspace.  In a mixed batch the two kernels run side by side: this one with
// skip_single_token_requests, launch_attention_gqa with single_token_requests_only (its grid then runs over
// requests, `splits` chosen for num_requests tokens).
cudaError_t launch_attention_prefill(const void *q, const void *k_pool, const void *v_pool, void *out,
                                     const uint32_t *block_table, const uint32_t *query_starts, const uint32_t *seq_lens,
                                     int total_query_tokens, int num_requests, int n_heads, int n_kv_heads, int head_dim,
                                     int block_size, int max_blocks_per_seq, bool skip_single_token_requests, cudaStream_t s,
                                     bool pdl);
cudaError_t launch_attention(const void *q, const void *k_pool, const void *v_pool, void *out, int dtype,
                             const uint32_t *block_table, const uint32_t *query_starts, const uint32_t *seq_lens,
                             int total_query_tokens, int num_requests, int n_heads, int n_kv_heads, int head_dim,
                             int block_size, int max_blocks_per_seq, cudaStream_t s, bool pdl);

// Decode matmul: integer dot products per scale group, float32 across groups; any M (tokens are
// processed in passes of <= 4).  x_dtype / out_dtype are DT_F32 or DT_BF16.  err_word names the device
// word that receives a KernelError if a bounded wait inside the kernel gives up, and the poll limits.  *launches is
// incremented per kernel launched.  pdl: launch with programmatic stream serialization, so that
// the kernel's prologue and weight fetch overlap the tail of the kernel before it in the stream
// (requires that no kernel still in flight writes the weights).  residual (optional, [M, N] of
// residual_dtype): out = residual + matmul, added in the epilogue; with more than four tokens the
// token passes each add their part.  norm_weight (optional, float32 [K]): the activations are RMS-normalised
// (rsqrt(mean(x^2) + norm_eps) * norm_weight) as they are staged, so rms_norm + matmul is one kernel.
cudaError_t launch_gemv(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                        int K, int N, int M, int sm_count, bool pdl, ErrSink err_word, cudaStream_t s,
                        uint64_t *launches, const void *residual = nullptr, int residual_dtype = DT_F32,
                        const float *norm_weight = nullptr, float norm_eps = 0.0f);

// The decode matmul of one rank's weight rows with the all-gather fused in.  `out` is this rank's
// [M, N_local * world] result.  peer_mailbox[d] is rank d's mailbox (gemv_allgather_mailbox_bytes()
// bytes, zero before the first call) as a pointer this device can store through; each result is
// posted to the other ranks as one 8-byte {value, call number} store and the kernel copies what
// the others posted into `out` before it finishes.  step_word: a local device word, zero before
// the first call, in which the kernel counts the calls.  M <= gemv_single_launch_max_tokens().
size_t gemv_allgather_mailbox_bytes(int n_total, int M);
cudaError_t launch_gemv_allgather(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                                  int K, int N_local, int M, int rank, int world, void *const *peer_mailbox,
                                  uint32_t *done_counter, uint32_t *step_word, int sm_count, bool pdl,
                                  ErrSink err_word, cudaStream_t s, uint64_t *launches);

// Fused feed-forward front on the decode kernel: out[M, N] = silu(X . Wgate^T) * (X . Wup^T) in one
// launch (both weights [K, N], same type, as uploaded).  gemv_gate_up_fits() says whether the shape
// can run that way (M <= 4 and the two-rows-per-warp ring fits beside the staged activations).
bool gemv_gate_up_fits(int wdtype, int K, int M);
cudaError_t launch_gemv_gate_up(int wdtype, const uint8_t *w_gate, const uint8_t *w_up, const void *x, int x_dtype,
                                void *out, int out_dtype, int K, int N, int M, int sm_count, bool pdl,
                                ErrSink err_word, cudaStream_t s, uint64_t *launches,
                                const float *norm_weight = nullptr, float norm_eps = 0.0f);
// out[i] = silu(gate[i]) * up[i] over n float32 values, written as out_dtype (the unfused tail).
cudaError_t launch_silu_mul(const float *gate, const float *up, void *out, int out_dtype, size_t n, cudaStream_t s);

// Largest in_features the decode kernel can stage in shared memory.
size_t gemv_max_k();
// Largest number of tokens (0..4) the decode kernel serves in ONE launch for this weight type and
// in_features (the staged activations of all tokens must fit beside two ring stages).
int gemv_single_launch_max_tokens(int wdtype, int K);

// Two or three weights of one format and in_features behind the same input in ONE launch of the decode
// kernel (the q, k and v projections): outs[i] = X . ws[i]^T, [M, n_rows[i]].  M <= 4 and
// M <= gemv_single_launch_max_tokens; norm_weight as in launch_gemv.
cudaError_t launch_gemv_multi(int wdtype, int n, const uint8_t *const *ws, const int *n_rows, void *const *outs,
                              const void *x, int x_dtype, int out_dtype, int K, int M, int sm_count, bool pdl,
                              ErrSink err_word, cudaStream_t s, uint64_t *launches, const float *norm_weight,
                              float norm_eps);

// Prefill matmul on the tensor cores (tcgen05, f16 operands, fp32 accumulate in TMEM); M >= 1.
// The activations are first converted to per-token-scaled f16 in `scratch`
// (gemm_scratch_bytes() bytes of device memory owned by the caller).
// `split_ws` (optional): gemm_split_workspace_bytes() bytes of device memory, zeroed once by the
// caller and left zeroed by every launch; with it the kernel may cut the tiles of the last,
// partial wave along K so that every SM works until the end (split_mode: -1 = a cost estimate
// decides, 0 = never, 1 = whenever there is a partial wave).  One launch at a time per workspace.
// `gather` (optional, world > 1): this call computes one rank's rows of an N-sharded matmul; `out` is
// then the rank's full [M, N * world] result and the all-gather runs inside the kernel through the
// peers' mailboxes, exactly as in launch_gemv_allgather (same mailbox size and layout).
// `two_term` (up to GEMM_TWO_TERM_MAX_TOKENS tokens; ignored above): weights and activations are
// each carried as a hi + lo pair of f16 values and three products are accumulated per K step, which
// brings the result to the decode kernel's tolerance class (1e-4 relative L2 against float32) at
// roughly twice the time of the one-term kernel.
constexpr int GEMM_TWO_TERM_MAX_TOKENS = 64;
struct GemmGather {
    int world, rank;
    void *const *peer_mailbox;
    uint32_t *done_counter, *step_word;
};
size_t gemm_scratch_bytes(int K, int M);
size_t gemm_split_workspace_bytes(int sms);
size_t gemm_split_counter_bytes();      // the leading bytes of the workspace that must be zero
cudaError_t launch_gemm(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                        int K, int N, int M, void *scratch, void *split_ws, int split_mode, ErrSink err_word,
                        cudaStream_t s, uint64_t *launches, const GemmGather *gather = nullptr, bool two_term = false,
                        bool pdl = false);

// The small-batch matmul (up to GEMM_EXACT_MAX_TOKENS tokens) on the tensor cores at the decode
// kernel's tolerance: the integer factors of the block formats (sc * q for Q4_K, sc * (q - 32) as an
// exact hi + lo pair for Q6_K) are the f16 operand, the activations a hi + lo f16 pair, and the blocks'
// d multiplies the per-block accumulators in float32 outside the tensor core (gemm_exact.cu).
// `scratch`: gemm_exact_scratch_bytes() bytes; split_ws / split_mode / gather as for launch_gemm.
// `pdl`: both kernels are launched with programmatic stream serialization (the conversion of the
// activations overlaps the tail of the kernel before it, the weight side of the matmul overlaps the
// conversion); `sm_count` <= 0 asks the device.
// `acts_mode`: several weights multiplied with one input share its conversion: the first call converts
// with the sub-block sums whatever its format (EXACT_ACTS_CONVERT_ALL), the others reuse what the scratch
// holds (EXACT_ACTS_REUSE: same scratch, same input, K and M, and nothing else run on the scratch since).
constexpr int GEMM_EXACT_MAX_TOKENS = 64;
enum { EXACT_ACTS_CONVERT = 0, EXACT_ACTS_CONVERT_ALL = 1, EXACT_ACTS_REUSE = 2 };
size_t gemm_exact_scratch_bytes(int K, int M);
cudaError_t launch_gemm_exact(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype,
                              int K, int N, int M, void *scratch, void *split_ws, int split_mode, ErrSink err_word,
                              cudaStream_t s, uint64_t *launches, const GemmGather *gather = nullptr, bool pdl = false,
                              int sm_count = 0, int acts_mode = EXACT_ACTS_CONVERT, const float *norm_w = nullptr,
                              float norm_eps = 0.0f);      // norm_w: an rms_norm of the input folded into its conversion
// Up to three weights of one format and K against one input in ONE launch (q/k/v, gate/up): the weights' row
// tiles form one tile space, cut over the SMs like a single matrix; output i is [M][ns[i]].  No all-gather.
cudaError_t launch_gemm_exact_multi(int wdtype, int nw, const uint8_t *const *ws, const int *ns, void *const *outs,
                                    const void *x, int x_dtype, int out_dtype, int K, int M, void *scratch,
                                    void *split_ws, int split_mode, ErrSink err_word, cudaStream_t s, uint64_t *launches,
                                    bool pdl = false, int sm_count = 0, const float *norm_w = nullptr, float norm_eps = 0.0f);

// Activations -> per-token scaled f16 (one CTA per token): out_f16 [M, K], tok_scale[M] the factors that
// undo the power-of-two scaling.  The conversion kernel of launch_gemm, for the dense F16 GEMM.
cudaError_t launch_activations_to_f16(const void *x, int x_dtype, int K, int M, void *out_f16, float *tok_scale,
                                      cudaStream_t s);

// ---- the other weight types of the reference's matmul: dense F32 / F16 / BF16, Q8_0, Q4_0 (dense.cu) ----
// Q8_0 / Q4_0 device layout ("planes"): [N rows of quants, block32_quant_stride() bytes apart][N rows of f16
// scales, block32_scale_stride() bytes apart]; quant bytes in file order (Q8_0: K int8; Q4_0: K/2 bytes, byte
// j of a block holding its elements 2j (low nibble) and 2j+1 (high nibble), minus 8, as the reference reads it).
size_t block32_quant_stride(int dtype, int K);
size_t block32_scale_stride(int K);
size_t block32_device_bytes(int dtype, int K, int N);
// `rows` rows of file blocks at raw -> quants at dev_q (first row), scales at dev_s (first row).
cudaError_t launch_block32_repack(int dtype, const uint8_t *raw, uint8_t *dev_q, uint8_t *dev_s, int K, int rows,
                                  cudaStream_t s);
// Any of the five types -> float32 [N, K] (test aid; bit-exact with the CPU dequantisation).
cudaError_t launch_dense_dequant(int wdtype, const uint8_t *w, int K, int N, float *out, cudaStream_t s);
// Streaming matmul for up to 8 tokens per pass (more tokens: several passes).
bool dense_gemv_shape_ok(int wdtype, int K);
cudaError_t launch_dense_gemv(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype, int K,
                              int N, int M, int sm_count, bool pdl, cudaStream_t s, uint64_t *launches);
// Dense weights on the tensor cores (tcgen05, both operands through TMA into shared memory).
bool dense_gemm_shape_ok(int wdtype, int K);
size_t dense_gemm_scratch_bytes(int wdtype, int K, int M);
cudaError_t launch_dense_gemm(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype, int K,
                              int N, int M, void *scratch, int sm_count, ErrSink err_word, cudaStream_t s, uint64_t *launches);
// Embedding lookup from a dense table.
cudaError_t launch_dense_embed(int wdtype, const uint8_t *table, int K, uint32_t vocab, const uint32_t *dev_tokens, int n_tokens,
                               void *out, int out_dtype, uint32_t *err_word, cudaStream_t s, bool pdl);

// The same GEMM with its scratch in a fixed 8 MiB device array that is part of the library image:
// no allocation on this path.  `device` must be the current device; the first call on a device
// resolves the array's address.  Fails with cudaErrorInvalidValue when the scratch the kernel needs
// (gemm_scratch_bytes(K, M), or gemm_exact_scratch_bytes(K, M) with `exact`, which runs the kernel of
// launch_gemm_exact) exceeds gemm_static_scratch_capacity().
size_t gemm_static_scratch_capacity();
cudaError_t launch_gemm_static_scratch(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out,
                                       int out_dtype, int K, int N, int M, int device, ErrSink err_word,
                                       cudaStream_t s, uint64_t *launches, bool two_term = false, bool exact = false);

}  // namespace llmrs
