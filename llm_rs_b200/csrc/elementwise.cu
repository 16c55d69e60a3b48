// The small operations that sit between the matmuls of a decode step: silu, mul, add
// (shaders/ops.metal:762-793), rms_norm (ops.metal:970-1003) and argmax (ops.metal:803-835).
// Buffers are F32 or BF16; arithmetic is float32 as in the reference's kernels, with one rounding
// to the output type.
#include "kernels.h"
#include "llmrs_common.cuh"

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

}  // namespace

cudaError_t launch_elementwise(int op, const void *a, int a_dtype, const void *b, int b_dtype, void *out,
                               int out_dtype, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    binary_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(op, a, a_dtype == DT_BF16, b, b_dtype == DT_BF16, out,
                                                             out_dtype == DT_BF16, n);
    return cudaGetLastError();
}

cudaError_t launch_rms_norm(const void *in, int in_dtype, const float *weight, void *out, int out_dtype, int dim,
                            int rows, float eps, cudaStream_t s) {
    if (dim <= 0 || rows <= 0) return cudaSuccess;
    rms_norm_kernel<<<(unsigned)rows, 256, 0, s>>>(in, in_dtype == DT_BF16, weight, out, out_dtype == DT_BF16, dim, eps);
    return cudaGetLastError();
}

cudaError_t launch_argmax(const void *x, int dtype, uint32_t n, uint32_t *dev_out, cudaStream_t s) {
    argmax_kernel<<<1, 1024, 0, s>>>(x, dtype == DT_BF16, n, dev_out);
    return cudaGetLastError();
}

}  // namespace llmrs
