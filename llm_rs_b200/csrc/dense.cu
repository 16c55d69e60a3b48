// The weight types beside Q4_K / Q6_K that the reference's matmul accepts (src/backend/metal/mod.rs:
// 503-518, 542-562, 634-686): dense F32 / F16 / BF16 and the 32-weight block formats Q8_0 / Q4_0.
//
//   out[s*N + r] = sum_k W[r,k] * x[s*K + k]        (src/backend/mod.rs:29-34)
//
//  * dense_gemv_kernel: up to 8 tokens per pass, any of the five types.  Bound by HBM: a warp owns
//    two weight rows, its lanes stride over the row in 16-byte pieces with several loads in flight,
//    float32 accumulation, warp-shuffle reduction.  Replaces matvec_f32_simd / matvec_bf16_simd /
//    matvec_f16_simd / matvec_q8_0_simd / matvec_q4_0_simd (shaders/ops.metal:52-218) and, for the
//    block formats, the reference's one-matvec-per-position loop (metal/mod.rs:634-686).
//  * dense_gemm_kernel: dense weights from 9 tokens on, tcgen05 in SS mode: weight tile (A) and
//    activation tile (B) both arrive by TMA in shared memory (128-byte swizzle), fp32 accumulators in
//    TMEM (double-buffered, so the epilogue of one tile overlaps the K loop of the next), no
//    dequantising warps.  F16 x f16 and BF16 x bf16 are kind::f16, F32 weights run as kind::tf32.
//    Replaces gemm_f32 / gemm_bf16 / gemm_f16 (shaders/ops.metal:1053-1179).
//  * Q8_0 / Q4_0 are re-laid out at upload into two planes (quants, f16 scales), both with 16-byte
//    aligned rows, because their 34- and 18-byte blocks are only 2-byte aligned in the file.
//    Q4_0 is read as the reference's kernel reads it (shaders/ops.metal:161-190): element e of a block
//    is the low nibble of byte e/2 for even e and the high nibble for odd e, minus 8.
#include <cuda.h>

#include "kernels.h"
#include "llmrs_common.cuh"
#include "pipeline.cuh"
#include "tensor_map.h"
#include "umma.cuh"

namespace llmrs {

size_t block32_quant_stride(int dtype, int K) { return (((size_t)(dtype == DT_Q8_0 ? K : K / 2)) + 15) / 16 * 16; }
size_t block32_scale_stride(int K) { return ((size_t)(K / 32) * 2 + 15) / 16 * 16; }
size_t block32_device_bytes(int dtype, int K, int N) {
    return (size_t)N * (block32_quant_stride(dtype, K) + block32_scale_stride(K));
}

namespace {

// ---- upload re-layout of Q8_0 / Q4_0: file blocks -> [N x quants][N x f16 scales] ----------------
__global__ void block32_repack_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ dev, uint8_t *__restrict__ scales,
                                      int K, int N, int block_bytes, size_t qstride, size_t sstride) {
    const int nbr = K / 32;                                   // blocks per row
    const size_t total = (size_t)N * nbr;
    const int qb = block_bytes - 2;                           // quant bytes per block: 32 or 16
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / nbr, b = i - r * nbr;
        const uint8_t *src = raw + i * block_bytes;
        scales[r * sstride + 2 * b] = src[0];
        scales[r * sstride + 2 * b + 1] = src[1];
        uint8_t *dst = dev + r * qstride + b * qb;
        for (int j = 0; j < qb; j++) dst[j] = src[2 + j];
    }
}

// ---- GEMV ---------------------------------------------------------------------------------------
struct DenseGemvParams {
    const uint8_t *W;          // dense rows, or the quant plane
    const uint8_t *S;          // Q8_0 / Q4_0: the scale plane
    const void *X;
    void *Out;
    int K, N, m_valid;
    int x_bf16, out_bf16;
    size_t row_stride, scale_stride;
};

template <int DT> struct Piece;                                          // one 16-byte piece of a weight row
template <> struct Piece<DT_F32> { static constexpr int ELEMS = 4; };
template <> struct Piece<DT_F16> { static constexpr int ELEMS = 8; };
template <> struct Piece<DT_BF16> { static constexpr int ELEMS = 8; };
template <> struct Piece<DT_Q8_0> { static constexpr int ELEMS = 16; };
template <> struct Piece<DT_Q4_0> { static constexpr int ELEMS = 32; };

// Eight consecutive weights of the piece (group g of ELEMS / 8), as floats; `scale` for the block formats.
template <int DT>
__device__ __forceinline__ void decode8(const uint4 &v, int g, float scale, float (&w)[8]) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    if constexpr (DT == DT_F16) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
            w[2 * i] = f.x; w[2 * i + 1] = f.y;
        }
    } else if constexpr (DT == DT_BF16) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            w[2 * i] = __uint_as_float(u[i] << 16);
            w[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
        }
    } else if constexpr (DT == DT_Q8_0) {                    // bytes 8g .. 8g+7, signed
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t word = u[2 * g + i] ^ 0x80808080u;                     // q + 128 as unsigned bytes
#pragma unroll
            for (int b = 0; b < 4; b++)
                w[4 * i + b] = scale * (__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7440u + b)) - 8388736.0f);
        }
    } else {                                                 // Q4_0: bytes 4g .. 4g+3 hold elements 8g .. 8g+7
        const uint32_t word = u[g];
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const uint32_t byte = (word >> (8 * b)) & 0xFFu;
            w[2 * b] = scale * (float)((int)(byte & 0xFu) - 8);
            w[2 * b + 1] = scale * (float)((int)(byte >> 4) - 8);
        }
    }
}

__device__ __forceinline__ void load_x8(const void *x, size_t idx, int is_bf16, float (&v)[8]) {
    if (is_bf16) {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>((const uint16_t *)x + idx));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4 *>((const float *)x + idx));
        const float4 b = __ldg(reinterpret_cast<const float4 *>((const float *)x + idx) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

constexpr int GEMV_ROWS = 2;      // rows per warp
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_UNROLL = 2;    // 16-byte pieces per row in flight per lane

// K a multiple of 8 (dense 16-bit), 4 (F32) or 32 (block formats); rows 16-byte aligned.
template <int DT, int MT>
__global__ void __launch_bounds__(GEMV_WARPS * 32) dense_gemv_kernel(const DenseGemvParams p) {
    pdl_prologue();
    constexpr int E = Piece<DT>::ELEMS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_pieces = p.K / E;
    const int row_step = gridDim.x * GEMV_WARPS * GEMV_ROWS;
    for (int row0 = (blockIdx.x * GEMV_WARPS + warp) * GEMV_ROWS; row0 < p.N; row0 += row_step) {
        float acc[GEMV_ROWS][MT];
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) acc[r][t] = 0.0f;
        const uint8_t *wrow[GEMV_ROWS];
        const uint8_t *srow[GEMV_ROWS];
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; r++) {
            const int row = min(row0 + r, p.N - 1);
            wrow[r] = p.W + (size_t)row * p.row_stride;
            srow[r] = p.S ? p.S + (size_t)row * p.scale_stride : nullptr;
        }
        for (int c0 = lane; c0 < n_pieces; c0 += 32 * GEMV_UNROLL) {
            uint4 v[GEMV_UNROLL][GEMV_ROWS];
            float sc[GEMV_UNROLL][GEMV_ROWS];
#pragma unroll
            for (int uu = 0; uu < GEMV_UNROLL; uu++) {
                const int c = c0 + 32 * uu;
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; r++) {
                    if (c < n_pieces) {
                        v[uu][r] = ldg128_pinned(wrow[r] + (size_t)c * 16);
                        sc[uu][r] = 1.0f;
                        if constexpr (DT == DT_Q8_0 || DT == DT_Q4_0) {
                            const int blk = DT == DT_Q8_0 ? c >> 1 : c;
                            sc[uu][r] = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(srow[r]) + blk));
                        }
                    }
                }
            }
#pragma unroll
            for (int uu = 0; uu < GEMV_UNROLL; uu++) {
                const int c = c0 + 32 * uu;
                if (c >= n_pieces) continue;
                const int k0 = c * E;
                if constexpr (DT == DT_F32) {
                    float xv[MT][4];
#pragma unroll
                    for (int t = 0; t < MT; t++) {
                        if (p.x_bf16) {
                            const uint2 u = __ldg(reinterpret_cast<const uint2 *>((const uint16_t *)p.X + (size_t)t * p.K + k0));
                            xv[t][0] = __uint_as_float(u.x << 16); xv[t][1] = __uint_as_float(u.x & 0xFFFF0000u);
                            xv[t][2] = __uint_as_float(u.y << 16); xv[t][3] = __uint_as_float(u.y & 0xFFFF0000u);
                        } else {
                            const float4 f = __ldg(reinterpret_cast<const float4 *>((const float *)p.X + (size_t)t * p.K + k0));
                            xv[t][0] = f.x; xv[t][1] = f.y; xv[t][2] = f.z; xv[t][3] = f.w;
                        }
                    }
#pragma unroll
                    for (int r = 0; r < GEMV_ROWS; r++) {
                        const float w[4] = {__uint_as_float(v[uu][r].x), __uint_as_float(v[uu][r].y),
                                            __uint_as_float(v[uu][r].z), __uint_as_float(v[uu][r].w)};
#pragma unroll
                        for (int t = 0; t < MT; t++)
#pragma unroll
                            for (int e = 0; e < 4; e++) acc[r][t] = fmaf(w[e], xv[t][e], acc[r][t]);
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < E / 8; g++) {
                        float w[GEMV_ROWS][8];
#pragma unroll
                        for (int r = 0; r < GEMV_ROWS; r++) decode8<DT>(v[uu][r], g, sc[uu][r], w[r]);
#pragma unroll
                        for (int t = 0; t < MT; t++) {
                            float xv[8];
                            load_x8(p.X, (size_t)t * p.K + k0 + 8 * g, p.x_bf16, xv);
#pragma unroll
                            for (int r = 0; r < GEMV_ROWS; r++)
#pragma unroll
                                for (int e = 0; e < 8; e++) acc[r][t] = fmaf(w[r][e], xv[e], acc[r][t]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; r++)
#pragma unroll
            for (int t = 0; t < MT; t++) {
                float s = acc[r][t];
#pragma unroll
                for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0 && row0 + r < p.N && t < p.m_valid) {
                    const size_t o = (size_t)t * p.N + row0 + r;
                    if (p.out_bf16) ((__nv_bfloat16 *)p.Out)[o] = __float2bfloat16_rn(s);
                    else ((float *)p.Out)[o] = s;
                }
            }
    }
}

template <int DT>
cudaError_t launch_gemv_dt(DenseGemvParams p, int M, int x_elem, int out_elem, int sm_count, bool pdl, cudaStream_t s,
                           uint64_t *launches) {
    const uint8_t *X = (const uint8_t *)p.X;
    uint8_t *Out = (uint8_t *)p.Out;
    const int warps_needed = (p.N + GEMV_ROWS - 1) / GEMV_ROWS;
    int grid = (warps_needed + GEMV_WARPS - 1) / GEMV_WARPS;
    if (grid > sm_count * 8) grid = sm_count * 8;
    for (int t0 = 0; t0 < M;) {
        const int m = M - t0 >= 8 ? 8 : M - t0 >= 4 ? 4 : M - t0 >= 2 ? 2 : 1;
        p.X = X + (size_t)t0 * p.K * x_elem;
        p.Out = Out + (size_t)t0 * p.N * out_elem;
        p.m_valid = m;
        cudaError_t e;
        switch (m) {
            case 8: e = launch_dependent(dense_gemv_kernel<DT, 8>, dim3(grid), dim3(GEMV_WARPS * 32), 0, s, pdl, p); break;
            case 4: e = launch_dependent(dense_gemv_kernel<DT, 4>, dim3(grid), dim3(GEMV_WARPS * 32), 0, s, pdl, p); break;
            case 2: e = launch_dependent(dense_gemv_kernel<DT, 2>, dim3(grid), dim3(GEMV_WARPS * 32), 0, s, pdl, p); break;
            default: e = launch_dependent(dense_gemv_kernel<DT, 1>, dim3(grid), dim3(GEMV_WARPS * 32), 0, s, pdl, p); break;
        }
        if (e != cudaSuccess) return e;
        if (launches) (*launches)++;
        t0 += m;
    }
    return cudaSuccess;
}

// ---- dense GEMM on the tensor cores, both operands in shared memory ---------------------------------
constexpr int DG_WARPS = 6;               // 0: TMA, 1: MMA + TMEM owner, 2-5: epilogue
constexpr int DG_THREADS = DG_WARPS * 32;
constexpr int DG_STAGE_K_BYTES = 128;     // one swizzled row: 64 16-bit or 32 float elements of K

template <int TN> struct DenseGemmCfg {
    static constexpr int A_BYTES = TILE_ROWS * DG_STAGE_K_BYTES;
    static constexpr int B_BYTES = TN * DG_STAGE_K_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr size_t EPI_BYTES = (size_t)EPI_WARPS * (EPI_TOK * 32 * 4) + (size_t)EPI_WARPS * TN_PAD * 4;
    static constexpr int FIT = (int)((227 * 1024 - 1024 - 256 - EPI_BYTES) / STAGE_BYTES);
    static constexpr int STAGES = FIT < 6 ? FIT : 6;
    static_assert(STAGES >= 3, "pipeline depth");
    static constexpr uint32_t TMEM_COLS = 2 * TN <= 32 ? 32 : 2 * TN <= 64 ? 64 : 2 * TN <= 128 ? 128 : 2 * TN <= 256 ? 256 : 512;
    static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256 + EPI_BYTES;
};

struct DenseGemmParams {
    void *Out;
    uint32_t *err;
    uint32_t wait_limit;
    int K, N, M;
    int out_bf16;
    int k_stages;               // ceil(K / elements per 128-byte row)
    int elems_per_stage;        // 64 (16-bit) or 32 (float)
    const float *tok_scale;     // per-token factor undoing the scaling of f16 activations, or nullptr
};

// D[tmem] (+)= A * B with both operands in shared memory.  KIND 0/1: kind::f16 (f16 or bf16), 2: kind::tf32.
template <int KIND>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Instruction descriptor: D fp32; A and B of format `fmt` (0 f16, 1 bf16, 2 tf32), both K-major.
__host__ __device__ constexpr uint32_t dense_idesc(int fmt, int n) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
}

template <int KIND, int TN>
__global__ void __launch_bounds__(DG_THREADS, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                  const DenseGemmParams p) {
    using C = DenseGemmCfg<TN>;
    constexpr int S = C::STAGES;
    constexpr uint32_t IDESC = dense_idesc(KIND, TN);
    extern __shared__ uint8_t smem_raw[];
    uint8_t *tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles + S * C::STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + S, *acc_full = bars + 2 * S, *acc_empty = bars + 2 * S + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 4);
    uint8_t *epi_stage = tiles + S * C::STAGE_BYTES + 256;
    static_assert((2 * 6 + 4) * 8 + 8 <= 256, "barrier area");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int w_tiles = (p.N + TILE_ROWS - 1) / TILE_ROWS;
    const int n_tiles = w_tiles * ((p.M + TN - 1) / TN);
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], EPI_WARPS);
        }
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer: weight tile and activation tile of every K stage ----------------
        const bool leader = elect_one();
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int n0 = (tile % w_tiles) * TILE_ROWS, t0 = (tile / w_tiles) * TN;
            for (int ks = 0; ks < p.k_stages; ks++, it++) {
                const uint32_t s = it % S;
                if (it >= (uint32_t)S && !mbar_wait(&empty[s], ((it / S) - 1) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_EMPTY_WAIT);
                    ok = false;
                    break;
                }
                if (leader) {
                    mbar_arrive_expect_tx(&full[s], C::STAGE_BYTES);
                    tma_load_2d(tiles + s * C::STAGE_BYTES, &tmap_w, ks * p.elems_per_stage, n0, &full[s]);
                    tma_load_2d(tiles + s * C::STAGE_BYTES + C::A_BYTES, &tmap_x, ks * p.elems_per_stage, t0, &full[s]);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        const bool leader = elect_one();
        const uint64_t desc0 = umma_desc_sw128(smem_u32(tiles));
        const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
        const uint32_t desc_lo0 = (uint32_t)desc0;
        uint32_t it = 0, tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, tcount++) {
            const uint32_t ab = tcount & 1u;
            if (tcount >= 2u && !mbar_wait(&acc_empty[ab], ((tcount >> 1) - 1) & 1, p.wait_limit)) {
                report_error(p.err, KERR_MMA_WAIT);
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + ab * TN;
            for (int ks = 0; ks < p.k_stages; ks++, it++) {
                const uint32_t s = it % S;
                if (!mbar_wait(&full[s], (it / S) & 1, p.wait_limit)) {
                    report_error(p.err, KERR_FULL_WAIT);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_lo = desc_lo0 + ((s * C::STAGE_BYTES) >> 4);
                const uint32_t b_lo = a_lo + (uint32_t)(C::A_BYTES >> 4);
                const uint32_t first = ks ? 1u : 0u;
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)                  // 32 bytes of K per instruction
                        umma_ss<KIND>(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + 2u * kk),
                                      ((uint64_t)desc_hi << 32) | (b_lo + 2u * kk), IDESC, kk ? 1u : first);
                    umma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && leader) umma_commit(&acc_full[ab]);
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> shared staging -> global ----------------
        const int quarter = warp & 3;
        const int ew = warp - 2;
        uint8_t *stg = epi_stage + (size_t)ew * (EPI_TOK * 32 * 4);
        float *scale_s = reinterpret_cast<float *>(epi_stage + EPI_WARPS * (EPI_TOK * 32 * 4)) + ew * TN_PAD;
        uint32_t tcount = 0;
        const int esz = p.out_bf16 ? 2 : 4;
        const bool vec_ok = ((size_t)p.N % (size_t)(16 / esz)) == 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, tcount++) {
            const uint32_t ab = tcount & 1u;
            const int n0 = (tile % w_tiles) * TILE_ROWS, t0 = (tile / w_tiles) * TN;
            for (int c = lane; c < TN; c += 32)
                scale_s[c] = (t0 + c < p.M) ? (p.tok_scale ? __ldg(p.tok_scale + t0 + c) : 1.0f) : 0.0f;
            __syncwarp();
            if (!mbar_wait(&acc_full[ab], (tcount >> 1) & 1, p.wait_limit)) {
                report_error(p.err, KERR_MMA_WAIT);
                break;
            }
            tc_fence_after();
            const uint32_t acc = tmem_base + ab * TN + ((uint32_t)(32 * quarter) << 16);
            const int row_base = n0 + 32 * quarter;
#pragma unroll 1
            for (int g0 = 0; g0 < TN; g0 += EPI_TOK) {
                uint32_t v[16];
                tmem_ld16(acc + (uint32_t)g0, v);
                tmem_ld_wait();
                if (g0 + EPI_TOK >= TN) {                        // last read of this accumulator: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[ab]);
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float val = __uint_as_float(v[j]) * scale_s[g0 + j];
                    if (p.out_bf16) reinterpret_cast<__nv_bfloat16 *>(stg)[j * 32 + lane] = __float2bfloat16_rn(val);
                    else reinterpret_cast<float *>(stg)[j * 32 + lane] = val;
                }
                __syncwarp();
                if (vec_ok) {
                    const int vec_per_tok = 32 * esz / 16, rows_per_vec = 16 / esz;
                    for (int i = lane; i < EPI_TOK * vec_per_tok; i += 32) {
                        const int tl = i / vec_per_tok, vv = i % vec_per_tok;
                        const int tok = t0 + g0 + tl, row = row_base + vv * rows_per_vec;
                        if (tok < p.M && row < p.N)
                            *reinterpret_cast<uint4 *>((uint8_t *)p.Out + ((size_t)tok * p.N + row) * esz) =
                                *reinterpret_cast<const uint4 *>(stg + (size_t)tl * 32 * esz + vv * 16);
                    }
                } else {
                    for (int tl = 0; tl < EPI_TOK; tl++) {
                        const int tok = t0 + g0 + tl, row = row_base + lane;
                        if (tok < p.M && row < p.N) {
                            if (p.out_bf16) ((uint16_t *)p.Out)[(size_t)tok * p.N + row] = reinterpret_cast<const uint16_t *>(stg)[tl * 32 + lane];
                            else ((float *)p.Out)[(size_t)tok * p.N + row] = reinterpret_cast<const float *>(stg)[tl * 32 + lane];
                        }
                    }
                }
                __syncwarp();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// element-wise conversions of the activations for the dense GEMM: out_kind 0: bf16, 1: f32
__global__ void __launch_bounds__(256) convert_activations_kernel(const void *__restrict__ x, int x_is_bf16, void *__restrict__ out,
                                                                  int out_f32, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x_is_bf16 ? bf16_bits_to_f32(((const uint16_t *)x)[i]) : ((const float *)x)[i];
        if (out_f32) ((float *)out)[i] = v;
        else ((__nv_bfloat16 *)out)[i] = __float2bfloat16_rn(v);
    }
}

template <int KIND, int TN>
cudaError_t launch_dense_tn(const void *w, const void *x_conv, DenseGemmParams p, int sm_count, cudaStream_t s) {
    using C = DenseGemmCfg<TN>;
    const CUtensorMapDataType ty = KIND == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : KIND == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const int esz = KIND == 2 ? 4 : 2;
    CUtensorMap tw, tx;
    cudaError_t e = encode_2d(&tw, ty, w, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)p.K * esz, (uint32_t)p.elems_per_stage,
                              TILE_ROWS, CU_TENSOR_MAP_SWIZZLE_128B);
    if (e != cudaSuccess) return e;
    e = encode_2d(&tx, ty, x_conv, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)p.K * esz, (uint32_t)p.elems_per_stage, TN,
                  CU_TENSOR_MAP_SWIZZLE_128B);
    if (e != cudaSuccess) return e;
    auto kern = dense_gemm_kernel<KIND, TN>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    if (e != cudaSuccess) return e;
    const int n_tiles = ((p.N + TILE_ROWS - 1) / TILE_ROWS) * ((p.M + TN - 1) / TN);
    const int grid = n_tiles < sm_count ? n_tiles : sm_count;
    kern<<<grid, DG_THREADS, C::SMEM, s>>>(tw, tx, p);
    return cudaGetLastError();
}

template <int KIND>
cudaError_t launch_dense_kind(const void *w, const void *x_conv, const DenseGemmParams &p, int sm_count, cudaStream_t s) {
    if (p.M <= 32) return launch_dense_tn<KIND, 32>(w, x_conv, p, sm_count, s);
    if (p.M <= 64) return launch_dense_tn<KIND, 64>(w, x_conv, p, sm_count, s);
    if (p.M <= 128) return launch_dense_tn<KIND, 128>(w, x_conv, p, sm_count, s);
    return launch_dense_tn<KIND, 256>(w, x_conv, p, sm_count, s);
}

// ---- embedding lookup from a dense table -----------------------------------------------------------
// Replaces embed_batch_f32 / embed_batch_bf16 / embed_batch_f16 (shaders/ops.metal:878-915): column s of
// out [K, n_tokens] = row tokens[s] of the table, widened to float32 and rounded once to the output type.
__global__ void __launch_bounds__(256) dense_embed_kernel(const uint8_t *__restrict__ table, int wdtype, int K, uint32_t vocab,
                                                          const uint32_t *__restrict__ tokens, void *__restrict__ out, int out_bf16,
                                                          uint32_t *err_word) {
    pdl_prologue();
    uint32_t tok = tokens[blockIdx.y];
    if (tok >= vocab) {
        if (err_word && threadIdx.x == 0) atomicCAS(err_word, 0u, (uint32_t)KERR_TOKEN_RANGE);
        tok = 0;
    }
    const size_t esz = wdtype == DT_F32 ? 4 : 2;
    const uint8_t *row = table + (size_t)tok * K * esz;
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < K; k += gridDim.x * blockDim.x) {
        float v;
        if (wdtype == DT_F32) v = ((const float *)row)[k];
        else if (wdtype == DT_F16) v = f16_bits_to_f32(((const uint16_t *)row)[k]);
        else v = bf16_bits_to_f32(((const uint16_t *)row)[k]);
        const size_t o = (size_t)blockIdx.y * K + k;
        if (out_bf16) ((__nv_bfloat16 *)out)[o] = __float2bfloat16_rn(v);
        else ((float *)out)[o] = v;
    }
}

// Test aid: any of the five types -> float32 [N, K], the values the CPU dequantisation forms (every
// widening is exact; scale * q is one float32 product).
__global__ void __launch_bounds__(256) dense_dequant_kernel(const uint8_t *__restrict__ w, int wdtype, int K, int N, float *__restrict__ out,
                                                            size_t qstride, size_t sstride) {
    const size_t n = (size_t)N * K;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / K, k = i - r * K;
        float v;
        if (wdtype == DT_F32) v = ((const float *)w)[i];
        else if (wdtype == DT_F16) v = f16_bits_to_f32(((const uint16_t *)w)[i]);
        else if (wdtype == DT_BF16) v = bf16_bits_to_f32(((const uint16_t *)w)[i]);
        else {
            const float scale = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(w + (size_t)N * qstride + r * sstride + 2 * (k / 32)));
            if (wdtype == DT_Q8_0) v = scale * (float)(int8_t)w[r * qstride + k];
            else {
                const uint8_t byte = w[r * qstride + k / 2];
                v = scale * (float)((k & 1) ? (int)(byte >> 4) - 8 : (int)(byte & 0xF) - 8);
            }
        }
        out[i] = v;
    }
}

}  // namespace

cudaError_t launch_block32_repack(int dtype, const uint8_t *raw, uint8_t *dev_q, uint8_t *dev_s, int K, int rows,
                                  cudaStream_t s) {
    if ((dtype != DT_Q8_0 && dtype != DT_Q4_0) || K % 32) return cudaErrorInvalidValue;
    const size_t total = (size_t)rows * (K / 32);
    const int grid = (int)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
    block32_repack_kernel<<<grid > 0 ? grid : 1, 256, 0, s>>>(raw, dev_q, dev_s, K, rows, dtype == DT_Q8_0 ? 34 : 18,
                                                            block32_quant_stride(dtype, K), block32_scale_stride(K));
    return cudaGetLastError();
}

cudaError_t launch_dense_dequant(int wdtype, const uint8_t *w, int K, int N, float *out, cudaStream_t s) {
    if (!dense_gemv_shape_ok(wdtype, K) && !(K > 0 && (wdtype == DT_F32 || wdtype == DT_F16 || wdtype == DT_BF16)))
        return cudaErrorInvalidValue;
    const size_t n = (size_t)N * K;
    const int grid = (int)((n + 255) / 256 < 65535 ? (n + 255) / 256 : 65535);
    dense_dequant_kernel<<<grid > 0 ? grid : 1, 256, 0, s>>>(w, wdtype, K, N, out, block32_quant_stride(wdtype == DT_Q4_0 ? DT_Q4_0 : DT_Q8_0, K),
                                                           block32_scale_stride(K));
    return cudaGetLastError();
}

bool dense_gemv_shape_ok(int wdtype, int K) {
    switch (wdtype) {
        case DT_F32: return K % 4 == 0;
        case DT_F16: case DT_BF16: return K % 8 == 0;
        case DT_Q8_0: case DT_Q4_0: return K % 32 == 0;
        default: return false;
    }
}

cudaError_t launch_dense_gemv(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype, int K,
                              int N, int M, int sm_count, bool pdl, cudaStream_t s, uint64_t *launches) {
    if (K <= 0 || N <= 0 || M <= 0) return cudaSuccess;
    if (!dense_gemv_shape_ok(wdtype, K)) return cudaErrorInvalidValue;
    DenseGemvParams p{};
    p.W = w; p.X = x; p.Out = out; p.K = K; p.N = N;
    p.x_bf16 = x_dtype == DT_BF16; p.out_bf16 = out_dtype == DT_BF16;
    const int xe = p.x_bf16 ? 2 : 4, oe = p.out_bf16 ? 2 : 4;
    switch (wdtype) {
        case DT_F32: p.row_stride = (size_t)K * 4; return launch_gemv_dt<DT_F32>(p, M, xe, oe, sm_count, pdl, s, launches);
        case DT_F16: p.row_stride = (size_t)K * 2; return launch_gemv_dt<DT_F16>(p, M, xe, oe, sm_count, pdl, s, launches);
        case DT_BF16: p.row_stride = (size_t)K * 2; return launch_gemv_dt<DT_BF16>(p, M, xe, oe, sm_count, pdl, s, launches);
        case DT_Q8_0:
        case DT_Q4_0:
            p.row_stride = block32_quant_stride(wdtype, K);
            p.scale_stride = block32_scale_stride(K);
            p.S = w + (size_t)N * p.row_stride;
            return wdtype == DT_Q8_0 ? launch_gemv_dt<DT_Q8_0>(p, M, xe, oe, sm_count, pdl, s, launches)
                                     : launch_gemv_dt<DT_Q4_0>(p, M, xe, oe, sm_count, pdl, s, launches);
        default: return cudaErrorInvalidValue;
    }
}

bool dense_gemm_shape_ok(int wdtype, int K) {
    return (wdtype == DT_F32 && K % 4 == 0) || ((wdtype == DT_F16 || wdtype == DT_BF16) && K % 8 == 0);
}

// Scratch: the activations in the weight's own element type where the caller's differ, and for F16 weights
// one float per token (their power-of-two scaling).
size_t dense_gemm_scratch_bytes(int wdtype, int K, int M) {
    const size_t esz = wdtype == DT_F32 ? 4 : 2;
    return ((size_t)M * K * esz + 255) / 256 * 256 + (size_t)M * sizeof(float);
}

cudaError_t launch_dense_gemm(int wdtype, const uint8_t *w, const void *x, int x_dtype, void *out, int out_dtype, int K,
                              int N, int M, void *scratch, int sm_count, ErrSink err_word, cudaStream_t s, uint64_t *launches) {
    if (K <= 0 || N <= 0 || M <= 0) return cudaSuccess;
    if (!dense_gemm_shape_ok(wdtype, K) || !scratch) return cudaErrorInvalidValue;
    DenseGemmParams p{};
    p.Out = out; p.err = err_word.word; p.wait_limit = err_word.mbar_polls;
    p.K = K; p.N = N; p.M = M; p.out_bf16 = out_dtype == DT_BF16;
    p.elems_per_stage = wdtype == DT_F32 ? 32 : 64;
    p.k_stages = (K + p.elems_per_stage - 1) / p.elems_per_stage;
    const void *x_conv = x;
    float *tok_scale = (float *)((uint8_t *)scratch + ((size_t)M * K * (wdtype == DT_F32 ? 4 : 2) + 255) / 256 * 256);
    cudaError_t e = cudaSuccess;
    if (wdtype == DT_F16) {                                  // per-token scaled f16 activations (gemm_tc.cu)
        e = launch_activations_to_f16(x, x_dtype, K, M, scratch, tok_scale, s);
        if (e != cudaSuccess) return e;
        if (launches) (*launches)++;
        x_conv = scratch;
        p.tok_scale = tok_scale;
    } else {
        const bool want_f32 = wdtype == DT_F32;
        const bool have = want_f32 ? x_dtype == DT_F32 : x_dtype == DT_BF16;
        if (!have || (reinterpret_cast<uintptr_t>(x) & 15)) {
            const size_t n = (size_t)M * K;
            const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
            convert_activations_kernel<<<grid, 256, 0, s>>>(x, x_dtype == DT_BF16, scratch, want_f32, n);
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
            if (launches) (*launches)++;
            x_conv = scratch;
        }
    }
    if (wdtype == DT_F16) e = launch_dense_kind<0>(w, x_conv, p, sm_count, s);
    else if (wdtype == DT_BF16) e = launch_dense_kind<1>(w, x_conv, p, sm_count, s);
    else e = launch_dense_kind<2>(w, x_conv, p, sm_count, s);
    if (e == cudaSuccess && launches) (*launches)++;
    return e;
}

cudaError_t launch_dense_embed(int wdtype, const uint8_t *table, int K, uint32_t vocab, const uint32_t *dev_tokens, int n_tokens,
                               void *out, int out_dtype, uint32_t *err_word, cudaStream_t s, bool pdl) {
    if (n_tokens <= 0) return cudaSuccess;
    if (wdtype != DT_F32 && wdtype != DT_F16 && wdtype != DT_BF16) return cudaErrorInvalidValue;
    const int gx = (K + 255) / 256 < 32 ? (K + 255) / 256 : 32;
    return launch_dependent(dense_embed_kernel, dim3(gx, n_tokens), dim3(256), 0, s, pdl, table, wdtype, K, vocab, dev_tokens, out,
                            (int)(out_dtype == DT_BF16), err_word);
}

}  // namespace llmrs
