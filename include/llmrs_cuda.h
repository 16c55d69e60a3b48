/*
 * llmrs_cuda.h — C ABI of the B200 (sm_100a) backend for llm-rs's Q4_K / Q6_K
 * dequantize-matmul.
 *
 * These are the entry points a `src/backend/cuda/mod.rs` implementing the
 * reference's `Backend` trait binds with `extern "C"`.  Each declaration names
 * the reference interface it replaces (paths are inside the llm-rs project).
 * Every function returns 0 on success or a negative llmrs_status; the message
 * of the last failure on a context is available from llmrs_cuda_last_error().
 * The library never aborts the process and has no CPU fallback: without a
 * usable CUDA device llmrs_cuda_create fails.
 *
 * Conventions (src/backend/mod.rs:29-34, src/backend/metal/mod.rs:13-34,496-499):
 *   weight  shape [K = in_features, N = out_features]: N rows of K/256 blocks
 *   input   shape [K] or [K, M]: M rows of K contiguous elements
 *   output  shape [N] or [N, M]: element (token s, row r) at s*N + r
 *   1-D buffers carry dim1 = 0; M = max(input.dim1, 1).
 *
 * Every wait inside a kernel is bounded: after a number of polls it gives up, the kernel finishes,
 * and the next llmrs_cuda_sync / read_f32 returns LLMRS_ERR_KERNEL; the context stays usable.  The
 * limits are seconds by default; LLMRS_WAIT_POLLS=n at llmrs_cuda_create sets both poll counts
 * (16 .. 2^30), which is how the give-up path is tested.
 *
 * A context owns one device and one stream.  It is not thread-safe (the
 * reference backend is `Send`, never `Sync`: metal/mod.rs:1005-1009); callers
 * serialise.  Operations are enqueued on the context's stream in call order.
 */
#ifndef LLMRS_CUDA_H
#define LLMRS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF dtype ids used on this path (src/tensor/mod.rs:3-33). */
enum llmrs_dtype {
    LLMRS_F32 = 0,
    LLMRS_F16 = 1,      /* weights and embedding tables only */
    LLMRS_Q4_0 = 2,     /* weights only; read as the reference's kernel reads it, see llmrs_cuda_matmul */
    LLMRS_Q8_0 = 8,     /* weights only */
    LLMRS_Q4K = 12,
    LLMRS_Q6K = 14,
    LLMRS_I32 = 26,     /* index buffers (positions, slot mapping, page tables), as upload_u32 makes them */
    LLMRS_BF16 = 30
};

/* Device layout of a buffer's bytes. */
enum llmrs_layout {
    LLMRS_LAYOUT_RAW = 0,        /* bytes exactly as in the GGUF file / dense row-major */
    /* Q6_K regrouped for 16-byte aligned, bank-conflict-free reads; same bytes, new order.
     * A row is cut into chunks of 16 blocks (the last may hold fewer, nbc); chunk ci starts at
     * byte 3360*ci of its row and holds
     *   4*nbc slices of 48 B: slice 4b+2h+c = ql[64h+16c..+16) | ql[64h+32+16c..+16) | qh[32h+16c..+16)
     *                         of block b (h = half of the block, c = 0,1),
     *   nbc*16 B: the int8 scales of block b at 16b,   nbc*2 B: the f16 d of block b at 2b.
     * Rows are round_up(210*K/256, 32) bytes apart. */
    LLMRS_LAYOUT_Q6K_SLICES = 1,
    /* Q8_0 / Q4_0 (32-weight blocks of 34 / 18 bytes, 2-byte aligned in the file) as two planes with
     * 16-byte aligned rows: N rows of quant bytes in file order (Q8_0: K bytes, Q4_0: K/2 bytes per row,
     * rows round_up(., 16) apart), then N rows of the blocks' f16 scales (round_up(K/16, 16) apart). */
    LLMRS_LAYOUT_BLOCK32_PLANES = 2
};

enum llmrs_status {
    LLMRS_OK = 0,
    LLMRS_ERR_CUDA = -1,         /* a CUDA runtime call failed */
    LLMRS_ERR_SHAPE = -2,        /* shapes do not agree / K not a multiple of 256 */
    LLMRS_ERR_DTYPE = -3,        /* dtype not supported on this path */
    LLMRS_ERR_ARG = -4,          /* null pointer, bad size, wrong context */
    LLMRS_ERR_NO_DEVICE = -5,    /* no CUDA device / not an sm_100 device */
    LLMRS_ERR_KERNEL = -6,       /* a kernel abandoned a bounded wait; reported at the next sync/read */
    LLMRS_ERR_IO = -7,           /* a file could not be opened or read (GgufError::Io) */
    LLMRS_ERR_FORMAT = -8,       /* not a GGUF v2/v3 file, or its directory is malformed (GgufError::InvalidMagic,
                                    UnsupportedVersion, UnknownDType, UnknownMetadataType, InvalidUtf8) */
    LLMRS_ERR_NOT_FOUND = -9     /* no tensor / metadata key of that name (GgufError::TensorNotFound) */
};

typedef struct llmrs_ctx llmrs_ctx;

/* Mirrors MetalBuffer (src/backend/metal/mod.rs:13-24): device memory + dtype + dim0/dim1. */
typedef struct llmrs_buf {
    void *dptr;        /* device pointer */
    uint64_t nbytes;   /* bytes allocated at dptr */
    uint32_t dtype;    /* llmrs_dtype */
    uint32_t dim0;     /* contiguous dimension: in_features for weights, dim for activations */
    uint32_t dim1;     /* outer dimension: out_features for weights, seq_len for 2-D activations, 0 for 1-D */
    uint32_t layout;   /* llmrs_layout */
    uint32_t owned;    /* 1: llmrs_cuda_free releases dptr; 0: caller's memory (llmrs_cuda_wrap) */
    uint32_t device;   /* CUDA device ordinal the memory lives on */
} llmrs_buf;

/* Replaces MetalBackend::new (src/backend/metal/mod.rs:185).  `stream` is a
 * cudaStream_t to enqueue on, or NULL to let the context create its own. */
int llmrs_cuda_create(int device, void *stream, llmrs_ctx **out);
int llmrs_cuda_destroy(llmrs_ctx *ctx);

/* Replaces Backend::upload_tensor (src/backend/mod.rs:18; metal/mod.rs:445-484).
 * `host` holds the tensor bytes as stored in the GGUF file (TensorView.data,
 * src/tensor/mod.rs:142-147).  The bytes are copied to the device; Q6_K is
 * re-laid out there (LLMRS_LAYOUT_Q6K_SLICES), as the reference repacks Q4_K at
 * upload (metal/mod.rs:38-81).  Host memory is not retained. */
int llmrs_cuda_upload_tensor(llmrs_ctx *ctx, uint32_t dtype, const uint64_t *shape, int ndims,
                             const void *host, size_t nbytes, llmrs_buf *out);

/* Replaces Backend::alloc (src/backend/mod.rs:19; metal/mod.rs:486-494). */
int llmrs_cuda_alloc(llmrs_ctx *ctx, uint32_t dtype, const uint64_t *shape, int ndims, llmrs_buf *out);

/* Describes caller-owned device memory (for example a torch tensor used as the
 * target of an all-gather) as a buffer.  No counterpart in the reference, whose
 * buffers are always backend-allocated. */
int llmrs_cuda_wrap(llmrs_ctx *ctx, void *dptr, uint32_t dtype, const uint64_t *shape, int ndims, llmrs_buf *out);

/* Replaces Drop of MetalBuffer. */
int llmrs_cuda_free(llmrs_ctx *ctx, llmrs_buf *buf);

/* Replaces Backend::matmul (src/backend/mod.rs:29-34; metal/mod.rs:496-687):
 * out[s*N + r] = sum_k W[r,k] * in[s*K + k].  Weight dtype Q4_K or Q6_K (the path this library is built
 * around), or one of the other types the reference's dispatcher takes (metal/mod.rs:503-518, 542-562):
 * dense F32 / F16 / BF16 and Q8_0 / Q4_0, served by a streaming kernel up to 8 tokens and, for the dense
 * types, a tcgen05 GEMM above (float32 accumulation; 16-bit operands on the tensor cores, tf32 for F32
 * weights: 2e-3 class); K a multiple of 4 (F32), 8 (F16 / BF16) or 32 (Q8_0 / Q4_0).  Q4_0 is read as the
 * reference's kernel reads it (shaders/ops.metal:161-190): element e of a block is the low nibble of byte
 * e/2 for even e, the high nibble for odd e, minus 8 (ggml's Q4_0 orders the nibbles differently).  Input
 * and output each F32 or BF16 (read from the buffers).  Enqueues only.  The tensor-core path keeps
 * converted activations in a scratch buffer of the context, which grows (one cudaMalloc) the first
 * time a call needs more than any call before it: so there is no allocation once a call of the same
 * or larger M*K has been made, and a call that is to be captured in a CUDA graph must have been
 * made once outside capture (inside capture a needed growth fails with LLMRS_ERR_CUDA).  An outgrown
 * scratch buffer is kept until llmrs_cuda_destroy, so graphs captured earlier stay replayable.  The
 * same holds for the temporaries of attention, embed and the rms_norm_* calls.
 * Accuracy against the float64 product, as relative L2 error: up to 64 tokens 1e-4 or better (one token
 * the decode kernel, integer dot products; 2..64 whichever of that kernel and the small-batch tensor-core
 * kernel, which keeps the formats' integer factors exact in f16, an estimate makes cheaper for the shape);
 * from 65 tokens 2e-3 (one-term tensor-core kernel, f16 operands, measured ~4e-4).  Environment, read at
 * context creation: LLMRS_GEMV_MAX_M=m makes "decode kernel up to m tokens, tensor cores above" the rule;
 * LLMRS_TC_EXACT=0 uses the older two-term kernel from 5 to 64 tokens; LLMRS_TC_TWO_TERM=0 extends the
 * one-term kernel down to 5 tokens.
 * Kernels that cut tiles along K exchange partial sums between the CTAs of one launch, which must all be
 * resident: calls of two contexts (or streams) on one device must not overlap in time, or either may give
 * up its bounded wait (LLMRS_ERR_KERNEL at the next sync; nothing hangs). */
int llmrs_cuda_matmul(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight, const llmrs_buf *input);

/* The same product as llmrs_cuda_matmul, computed by the tensor-core kernel for any M, with that
 * kernel's scratch (the activations converted to f16 and one scale per token) held in an 8 MiB
 * device array that is built into the library instead of in memory the context allocates.  It has
 * no counterpart in the reference; it exists for hosts that must not allocate device memory once
 * they are running: a server that gave the whole GPU to its own memory pool, or a loop that cannot
 * take the device-wide synchronisation a cudaMalloc or cudaFree causes.  This call never allocates
 * or frees device memory.
 *   - Limit: the scratch must fit 8 MiB.  Up to 64 tokens (small-batch kernel, same accuracy as
 *     llmrs_cuda_matmul) it is round_up(5*K*Mp, 256) + 4*M bytes, Mp = M rounded up to 16, 32 or 64 (the
 *     converted activations are whole token tiles): 64 tokens up to K = 26112.  Above 64 tokens (one-term
 *     kernel) it is round_up(2*K*M, 256) + 4*M bytes: 1023 tokens at K=4096, 292 at K=14336.  Larger
 *     shapes fail with LLMRS_ERR_SHAPE and a message that names both sizes.
 *   - Every GPU that loads the library holds the 8 MiB until the process exits.
 *   - The first call on a device looks up the array's device address; make that first call
 *     before any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents (nothing in it
 *     needs clearing: each call rewrites what it reads).  Two calls whose kernels may overlap on
 *     the GPU (different streams or contexts on one device) race on it; serialise them. */
int llmrs_cuda_matmul_static_scratch(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight,
                                     const llmrs_buf *input);

/* Replace Backend::silu / mul / add (src/backend/mod.rs:76-78; shaders/ops.metal:762-793):
 * silu in place, out = a * b, out = a + b over buffers of equal element count (F32 or BF16 each);
 * float32 arithmetic, one rounding to the output type. */
int llmrs_cuda_silu(llmrs_ctx *ctx, llmrs_buf *x);
int llmrs_cuda_mul(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *a, const llmrs_buf *b);
int llmrs_cuda_add(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *a, const llmrs_buf *b);

/* Replaces Backend::rms_norm (src/backend/mod.rs:36-38; shaders/ops.metal:970-1003): every column
 * of input [dim] / [dim, seq_len] is scaled by rsqrt(mean(v^2) + eps) and by the float32 weight[dim]:
 * out = (v * inv_rms) * weight. */
int llmrs_cuda_rms_norm(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *input, const llmrs_buf *weight, float eps);

/* Replaces Backend::argmax (src/backend/mod.rs:21-23; shaders/ops.metal:803-835): index of the
 * largest logit, computed on the device; the call completes the stream, like the reference's
 * (metal/mod.rs:836).  On ties the smallest index wins (the reference's tree reduction leaves
 * the choice among equal maxima to its thread layout). */
int llmrs_cuda_argmax(llmrs_ctx *ctx, const llmrs_buf *logits, uint32_t *index);

/* Replaces Backend::rms_norm_heads (src/backend/mod.rs:40-43; metal/mod.rs:719-742): every
 * consecutive chunk of weight.dim0 values of x is normalised in place like a row of rms_norm. */
int llmrs_cuda_rms_norm_heads(llmrs_ctx *ctx, llmrs_buf *x, const llmrs_buf *weight, float eps);

/* Replaces Backend::rope (src/backend/mod.rs:45-47; metal/mod.rs:744-785; shaders/ops.metal:1011-1042):
 * rotary embedding of q and k in place; positions is an I32 buffer with one absolute position per
 * column; split_half = 0 rotates pairs (2i, 2i+1) of each head (RopeLayout::Interleaved), 1 rotates
 * (i, i + head_dim/2) (RopeLayout::SplitHalf). */
int llmrs_cuda_rope(llmrs_ctx *ctx, llmrs_buf *q, llmrs_buf *k, const llmrs_buf *positions, uint32_t head_dim,
                    float rope_theta, uint32_t split_half);

/* rope(q, k) and the two scatter_kv calls that follow it in a layer (src/arch/llama.rs:156-158) as one
 * call and one launch: q and k are rotated in place, the rotated k and v are written to the slots
 * slot_mapping[t] of k_pool and v_pool (kv_dim = k.dim0).  All five of one element type. */
int llmrs_cuda_rope_scatter_kv(llmrs_ctx *ctx, llmrs_buf *q, llmrs_buf *k, const llmrs_buf *v, const llmrs_buf *positions,
                               uint32_t head_dim, float rope_theta, uint32_t split_half, llmrs_buf *k_pool,
                               llmrs_buf *v_pool, const llmrs_buf *slot_mapping);

/* Replaces Backend::scatter_kv (src/backend/mod.rs:68-69; shaders/ops.metal:841-853):
 * pool[slot_mapping[t] * kv_dim + d] = src[t * kv_dim + d] for t < num_tokens. */
int llmrs_cuda_scatter_kv(llmrs_ctx *ctx, llmrs_buf *pool, const llmrs_buf *src, const llmrs_buf *slot_mapping,
                          uint32_t kv_dim, uint32_t num_tokens);

/* Replaces Backend::gather (src/backend/mod.rs:71-72; shaders/ops.metal:859-873):
 * column c of out = column indices[c] of src ([dim, seq_len]) for c < num_indices. */
int llmrs_cuda_gather(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *src, const llmrs_buf *indices,
                      uint32_t num_indices);

/* Replaces Backend::attention (src/backend/mod.rs:49-66; metal/mod.rs:880-928; shaders/ops.metal:636-758):
 * paged, variable-length, grouped-query attention with a causal mask.  q and out are
 * [n_heads * head_dim, total_query_tokens]; the pools hold pages of block_size positions of
 * n_kv_heads * head_dim values; request r owns query tokens query_starts[r] .. query_starts[r+1]
 * (query_starts has num_requests + 1 entries), has seq_lens[r] positions in total, and its page p is
 * block_table[r * max_blocks_per_seq + p].  Query token i of a request with c query tokens sees
 * positions 0 .. seq_len - c + i.  head_dim a multiple of 32, at most 256. */
int llmrs_cuda_attention(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *q, const llmrs_buf *k_pool,
                         const llmrs_buf *v_pool, const llmrs_buf *block_table, const llmrs_buf *query_starts,
                         const llmrs_buf *seq_lens, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                         uint32_t block_size, uint32_t max_blocks_per_seq);

/* out = residual + matmul(weight, input): the pairs matmul, add of src/arch/llama.rs:162-163 and
 * 168-169 as one call.  Up to LLMRS_GEMV_MAX_M tokens the decode kernel adds the residual as it
 * writes its results (no second kernel, no second pass over the output); above that the matmul is
 * followed by the add kernel.  residual has the shape of out, F32 or BF16, and may be `out` itself. */
int llmrs_cuda_matmul_add(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight, const llmrs_buf *input,
                          const llmrs_buf *residual);

/* rms_norm followed by the three projections of one input, src/arch/llama.rs:152-155, as one call:
 * out_q = matmul(wq, xn), out_k = matmul(wk, xn), out_v = matmul(wv, xn) with xn = rms_norm(input).
 * Up to LLMRS_GEMV_MAX_M tokens the weights that share a format run in ONE launch of the decode kernel
 * (a Q4_K_M file keeps wq, wk in Q4_K and wv in Q4_K or Q6_K: one or two launches instead of three, each
 * normalising the activations as it stages them); otherwise the three llmrs_cuda_rms_norm_matmul calls.
 * Same results as those calls. */
int llmrs_cuda_rms_norm_matmul_qkv(llmrs_ctx *ctx, llmrs_buf *out_q, llmrs_buf *out_k, llmrs_buf *out_v,
                                   const llmrs_buf *wq, const llmrs_buf *wk, const llmrs_buf *wv,
                                   const llmrs_buf *input, const llmrs_buf *norm_weight, float eps);

/* rms_norm followed by matmul (src/arch/llama.rs:152-155), and rms_norm followed by the feed-forward
 * front (llama.rs:164-168), as one call each: out = matmul(weight, rms_norm(input, norm_weight, eps)).
 * Up to LLMRS_GEMV_MAX_M tokens the decode kernel normalises the activations while it stages them
 * (every CTA forms the row's sum of squares itself: 4096 values), so the norm costs no launch and no
 * pass over memory, and the normalised activations are never rounded to bf16 in between.  Otherwise
 * the norm runs into a temporary first.  norm_weight is F32 [in_features]. */
int llmrs_cuda_rms_norm_matmul(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight, const llmrs_buf *input,
                               const llmrs_buf *norm_weight, float eps);
int llmrs_cuda_rms_norm_matmul_gate_up(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *w_gate, const llmrs_buf *w_up,
                                       const llmrs_buf *input, const llmrs_buf *norm_weight, float eps);

/* The front of the feed-forward block in one call: out = silu(gate) * up with gate = matmul(w_gate,
 * input) and up = matmul(w_up, input), i.e. the four calls matmul, matmul, silu, mul of
 * src/arch/llama.rs:165-168 (kernels shaders/ops.metal:762-793).  Both weights [K, N] of one type;
 * out [N] or [N, M].  Up to 4 tokens (and where the activations fit) the decode kernel forms both
 * dot products of an output row in one warp and writes silu(g) * u directly: one launch, nothing
 * intermediate in memory.  Otherwise two matmuls into float32 scratch and one element-wise kernel.
 * gate and up stay float32 until the single rounding of the output (the reference rounds each
 * to bf16 in between). */
int llmrs_cuda_matmul_gate_up(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *w_gate, const llmrs_buf *w_up,
                              const llmrs_buf *input);

/* Replaces Backend::embed (src/backend/mod.rs:25-27; metal/mod.rs:841-878, kernels
 * shaders/ops.metal:878-965) for F32 / F16 / BF16 / Q4_K / Q6_K tables (the reference's list): row tokens[s] of `table` ([dim, vocab], as
 * uploaded by upload_tensor) is dequantised into column s of `out` ([dim] for one token, else
 * [dim, n_tokens]; F32 or BF16).  `tokens` is host memory, as in the trait (tokens: &[u32]); ids
 * are checked against the table before anything is enqueued.  The values are the float32
 * dequantisation (the same numbers llmrs_cuda_dequantize writes), rounded once for a BF16 output.
 * (The reference's Metal kernel for Q4_K reads its repacked blocks, whose d*sc and dmin*m were
 * rounded to f16 at upload; this one keeps them exact.)  At most 65535 tokens per call. */
int llmrs_cuda_embed(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *table, const uint32_t *tokens,
                     uint32_t n_tokens);

/* Multi-GPU decode matmul: this rank's rows of an N-sharded weight, with the all-gather of the
 * output slices fused into the kernel.  The reference is single-GPU and has no counterpart; the
 * sharding follows from every output row reading only its own weight row (shaders/ops.metal:249-289).
 * Rank `rank` of `world` holds rows [rank*N_local, (rank+1)*N_local) (weight_shard, created by
 * upload_tensor from those rows); `out` is this rank's full result, [N_local*world] or
 * [N_local*world, M], in ordinary device memory.  peer_mailbox[d] is rank d's mailbox --
 * llmrs_cuda_allgather_mailbox_bytes() bytes, zero before the first call, 8-byte aligned -- as a
 * pointer this device can store through (peer-mapped / symmetric memory; entry `rank` is this
 * rank's own).  step_word is a word of this device's memory, zero before the first call, in
 * which the kernel counts the calls.
 * Each result is written to `out` here and posted to every other rank as one 8-byte store
 * {value, call number} into that rank's mailbox; before it finishes, the kernel copies the words
 * the other ranks posted into `out`, waiting (with a bound: a peer that never posts yields
 * LLMRS_ERR_KERNEL at the next sync) for each to carry this call's number.  When the call's
 * kernel has completed, `out` is complete: stream order is all a consumer needs.  The mailbox
 * has two halves used in turn, because a peer may be one call ahead.  All ranks must make the
 * same sequence of calls on one mailbox (same N_local and M every time).  No argument changes
 * from call to call, so a captured CUDA graph of the call can be replayed.
 * M <= llmrs_cuda_matmul_allgather_max_tokens().  Which kernel runs follows llmrs_cuda_matmul: the
 * exact decode kernel up to LLMRS_GEMV_MAX_M tokens where one launch holds their staged
 * activations, the tensor-core kernel otherwise (there N_local must be a multiple of 8). */
int llmrs_cuda_matmul_allgather(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight_shard,
                                const llmrs_buf *input, uint32_t rank, uint32_t world, void *const *peer_mailbox,
                                uint32_t *step_word);

/* Bytes of one rank's mailbox for outputs of n_total rows and `tokens` tokens. */
size_t llmrs_cuda_allgather_mailbox_bytes(uint32_t n_total, uint32_t tokens);

/* Largest number of tokens llmrs_cuda_matmul_allgather accepts for a weight of this dtype with
 * this many input features (0 if the pair is not supported).  Above it the exchange would move
 * more bytes than it saves in latency: run llmrs_cuda_matmul and a collective.  No counterpart in
 * the reference. */
#define LLMRS_ALLGATHER_MAX_TOKENS 128
int llmrs_cuda_matmul_allgather_max_tokens(uint32_t weight_dtype, uint32_t in_features);

/* Dequantises a weight (any type matmul takes) to float32 [N, K] in device memory `dev_out`
 * (N*K floats).  The reference has no such op; it exposes, for testing, the
 * values its kernels form in registers (tests/ops.rs:41-59, shaders/ops.metal:322-334). */
int llmrs_cuda_dequantize(llmrs_ctx *ctx, const llmrs_buf *weight, float *dev_out);

/* Host -> device copy into an existing buffer (same bytes as upload_tensor would
 * store for a dense dtype).  Used to refresh activations each step. */
int llmrs_cuda_write(llmrs_ctx *ctx, llmrs_buf *dst, const void *host, size_t nbytes);

/* Replaces Backend::read_to_vec_f32 (src/backend/mod.rs:80; metal/mod.rs:979-994):
 * waits for enqueued work, then copies n elements to `host`, widening BF16. */
int llmrs_cuda_read_f32(llmrs_ctx *ctx, const llmrs_buf *buf, float *host, size_t n);

/* Replaces Backend::sync (src/backend/mod.rs:88; metal/mod.rs:996-1002). */
int llmrs_cuda_sync(llmrs_ctx *ctx);

/* Replace Backend::gpu_secs_total / reset_gpu_secs (src/backend/mod.rs:84-85;
 * metal/mod.rs:264-272,442-443): device time, from events on the context's
 * stream, of the work enqueued between synchronisation points. */
int llmrs_cuda_gpu_secs_total(llmrs_ctx *ctx, double *secs);
int llmrs_cuda_reset_gpu_secs(llmrs_ctx *ctx);

/* Per-kernel timing table, the counterpart of the reference's LLM_PERF output (metal/mod.rs:150-153,
 * 323-400, 996-1002).  With LLMRS_PERF=1 in the environment at llmrs_cuda_create every operation is
 * bracketed by an event pair, and each llmrs_cuda_sync prints one line per kind of operation since the
 * previous sync to stderr: calls, device time, share, algorithmic GB/s and TFLOP/s, each also as a
 * fraction of the peaks LLMRS_PEAK_HBM_GBS / LLMRS_PEAK_TFLOPS give (defaults: the nominal 8000 GB/s and
 * 2250 TFLOP/s of a B200).  This call copies the table of the last sync into buf (NUL-terminated, at
 * most cap bytes) and returns its full length; 0 when nothing was recorded.  Operations inside a stream
 * capture are not timed. */
size_t llmrs_cuda_perf_table(llmrs_ctx *ctx, char *buf, size_t cap);

/* Number of kernels this library has launched on the context since creation. */
int llmrs_cuda_launch_count(llmrs_ctx *ctx, uint64_t *count);

/* Message of the last failure on `ctx` (or of the last failed create when ctx is NULL). */
const char *llmrs_cuda_last_error(llmrs_ctx *ctx);

/* ---- GGUF files: the on-disk step in front of upload_tensor --------------------------------------
 * Replaces GgufFile (src/gguf/mod.rs:80-86).  The reference reads the whole file into one page-aligned
 * host copy that its unified-memory GPU then addresses in place (:167-175, :307-342; metal/mod.rs:463-484).
 * Here only the directory (metadata and tensor table) stays on the host; a tensor's bytes travel
 * file -> pinned staging -> device when it is uploaded.  A handle is independent of any context and
 * may be shared by the contexts of several GPUs (each uploads its own tensors or slices). */
typedef struct llmrs_gguf llmrs_gguf;

/* One entry of the tensor table (TensorInfo, src/gguf/mod.rs:14-24; what tensor_view returns, :242-254,
 * without the bytes).  `name` stays valid until llmrs_gguf_close.  shape[0] is the contiguous
 * dimension, as stored in the file. */
typedef struct llmrs_gguf_tensor {
    const char *name;
    uint32_t dtype;      /* GGUF type id, 0..30 (src/tensor/mod.rs:96-130); not limited to llmrs_dtype */
    uint32_t n_dims;     /* at most 4 */
    uint64_t shape[4];
    uint64_t offset;     /* from the start of the data section (llmrs_gguf_data_offset) */
    uint64_t nbytes;     /* DType::storage_size of the shape (src/tensor/mod.rs:89-93) */
} llmrs_gguf_tensor;

/* Metadata value types (src/gguf/mod.rs:256-273). */
enum llmrs_gguf_type {
    LLMRS_GGUF_U8 = 0, LLMRS_GGUF_I8 = 1, LLMRS_GGUF_U16 = 2, LLMRS_GGUF_I16 = 3, LLMRS_GGUF_U32 = 4,
    LLMRS_GGUF_I32 = 5, LLMRS_GGUF_F32 = 6, LLMRS_GGUF_BOOL = 7, LLMRS_GGUF_STRING = 8, LLMRS_GGUF_ARRAY = 9,
    LLMRS_GGUF_U64 = 10, LLMRS_GGUF_I64 = 11, LLMRS_GGUF_F64 = 12
};

/* Replaces GgufFile::open (src/gguf/mod.rs:167-218): magic, version 2 or 3, key/value section, tensor
 * table, data section at the next multiple of 32.  A truncated or malformed directory is an error
 * (the reference panics on an out-of-range slice).  Failures: LLMRS_ERR_IO / LLMRS_ERR_FORMAT with
 * the text in llmrs_gguf_last_error(). */
int llmrs_gguf_open(const char *path, llmrs_gguf **out);
void llmrs_gguf_close(llmrs_gguf *g);
/* Message of the last failed llmrs_gguf_* call on this thread. */
const char *llmrs_gguf_last_error(void);

uint32_t llmrs_gguf_version(const llmrs_gguf *g);
uint64_t llmrs_gguf_file_size(const llmrs_gguf *g);        /* GgufFile::file_size (:224-226) */
uint64_t llmrs_gguf_data_offset(const llmrs_gguf *g);
uint64_t llmrs_gguf_tensor_count(const llmrs_gguf *g);
uint64_t llmrs_gguf_metadata_count(const llmrs_gguf *g);

/* Tensor table by position (GgufFile::tensors) and by name (the lookup of tensor_view, :243-244). */
int llmrs_gguf_tensor_at(const llmrs_gguf *g, uint64_t index, llmrs_gguf_tensor *out);
int llmrs_gguf_find_tensor(const llmrs_gguf *g, const char *name, llmrs_gguf_tensor *out);
/* The bytes tensor_view exposes as TensorView.data (:246-253), copied to `host` (nbytes must equal the
 * tensor's).  Eight concurrent positional reads, as read_file_fast (:307-342). */
int llmrs_gguf_read_tensor(const llmrs_gguf *g, const char *name, void *host, size_t nbytes);

/* Key/value section by position: key, type, and for arrays element type and length (any may be NULL). */
int llmrs_gguf_metadata_at(const llmrs_gguf *g, uint64_t index, const char **key, uint32_t *type,
                           uint32_t *elem_type, uint64_t *count);
/* Values by key (of two equal keys the later one, as the reference's map keeps it).
 * get_u32: MetadataValue::as_u32, U32/I32/U64/I64 truncated (src/gguf/metadata.rs:38-46);
 * get_u64: any integer or bool, sign-extended; get_f64: as_f32's F32/F64 (:48-54), not narrowed;
 * get_str: as_str (:31-36), not NUL-terminated, valid until close;
 * get_array: element type, length and, for numeric arrays, the packed little-endian elements;
 * get_array_str: element `index` of an array of strings (as_string_array, :56-61). */
int llmrs_gguf_get_u32(const llmrs_gguf *g, const char *key, uint32_t *out);
int llmrs_gguf_get_u64(const llmrs_gguf *g, const char *key, uint64_t *out);
int llmrs_gguf_get_f64(const llmrs_gguf *g, const char *key, double *out);
int llmrs_gguf_get_str(const llmrs_gguf *g, const char *key, const char **out, uint64_t *len);
int llmrs_gguf_get_array(const llmrs_gguf *g, const char *key, uint32_t *elem_type, uint64_t *count, const void **data);
int llmrs_gguf_get_array_str(const llmrs_gguf *g, const char *key, uint64_t index, const char **out, uint64_t *len);

/* Replaces Loader::opt (src/arch/mod.rs:52-57): tensor_view(name) + upload_tensor in one call, without a
 * host copy of the tensor.  The bytes are read in pieces of whole rows into two pinned staging buffers
 * (eight concurrent positional reads per piece) and copied to the device piece by piece, the read of one
 * piece overlapping the copy (and, for Q6_K, the re-layout kernel) of the one before.  Shapes: 1-D or 2-D
 * as upload_tensor takes them (trailing dimensions of 1 are dropped); dtypes as upload_tensor.
 * LLMRS_ERR_NOT_FOUND when the file has no such tensor (Loader::opt's None).  Returns when the tensor is
 * complete in device memory. */
int llmrs_cuda_upload_gguf_tensor(llmrs_ctx *ctx, const llmrs_gguf *g, const char *name, llmrs_buf *out);

/* The same for rows [first_row, first_row + n_rows) of a 2-D tensor's outer dimension (output features of
 * a weight, token rows of an embedding table): what one rank of an N-sharded matmul holds.  Only that
 * slice is read from the file.  The buffer's dim1 is n_rows.  No counterpart in the reference, which runs
 * on one GPU. */
int llmrs_cuda_upload_gguf_tensor_rows(llmrs_ctx *ctx, const llmrs_gguf *g, const char *name, uint64_t first_row,
                                       uint64_t n_rows, llmrs_buf *out);

#ifdef __cplusplus
}
#endif
#endif /* LLMRS_CUDA_H */
