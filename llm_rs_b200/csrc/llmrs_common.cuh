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

// The same load as an instruction the compiler may not move or delay: used where a load is issued
// early on purpose (register prefetch) and must stay ahead of the waits that follow it.
__device__ __forceinline__ uint4 ldg128_pinned(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
// 32 bytes (one sector) in one instruction, not allocated in L1: for bytes that are read exactly
// once.  The address must be 32-byte aligned.
__device__ __forceinline__ void ldg256_stream(const void *p, uint4 &lo, uint4 &hi) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(p));
}
__device__ __forceinline__ uint2 ldg64_pinned(const void *p) {
    uint2 r;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldg16_pinned(const void *p) {
    uint16_t r;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
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
