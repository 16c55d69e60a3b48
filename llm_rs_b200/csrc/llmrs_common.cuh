// Small device helpers shared by the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace llmrs {

// IEEE binary16 bits -> float, exact (subnormals included).
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

// bf16 bits -> float, exact.
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float((uint32_t)b << 16);
}

// 128-bit read-only global load.
__device__ __forceinline__ uint4 ldg128(const void *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
}

// The float whose bit pattern is `bits`.  For bits < 2^23 this is the subnormal
// bits * 2^-149: a masked bit field of quants becomes a float operand with no
// shift and no int->float conversion.  fma handles subnormal inputs at full
// rate and the product with a normal float is rounded once, so nothing is lost.
// (Needs the default -ftz=false.)
__device__ __forceinline__ float field_as_float(uint32_t bits) { return __uint_as_float(bits); }

// 2^e as a float, -126 <= e <= 127.
__device__ __forceinline__ float exp2i(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }

}  // namespace llmrs
