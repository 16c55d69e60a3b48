// mbarrier + bulk-copy (TMA, untiled) helpers for sm_100a.  Every wait is bounded: after
// WAIT_LIMIT polls it gives up, the caller records an error code and leaves the kernel, so a
// logic error can not spin a shared GPU forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace llmrs {

// Polls of mbarrier.try_wait before a wait is abandoned.  Each try_wait blocks for a
// hardware-defined slice (on the order of a microsecond), so this is seconds, not cycles.
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// Kernel error codes written to the context's device error word (first error wins).
enum KernelError : uint32_t {
    KERR_NONE = 0,
    KERR_FULL_WAIT = 1,    // a consumer gave up waiting for a bulk copy to land
    KERR_EMPTY_WAIT = 2,   // the producer gave up waiting for a stage to be released
    KERR_MMA_WAIT = 3,     // a wait on tensor-core completion gave up
    KERR_TMEM_ALLOC = 4,
    KERR_GATHER_WAIT = 5,  // the fused all-gather gave up waiting for a peer's slice
    KERR_SPLIT_WAIT = 6,   // a split-K tile gave up waiting for the other CTAs' partial sums
    KERR_TOKEN_RANGE = 7   // embed: a token id beyond the table (row 0 was read instead)
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy (bulk copies, tensor cores).
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// true when the phase with the given parity has completed; false after `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = WAIT_LIMIT) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Untiled bulk copy global -> shared, completion reported to `bar` in bytes.
// dst, src and bytes must all be multiples of 16.
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Tiled (tensor-map) copy of one 2-D box global -> shared, completion reported to `bar` in bytes.
// c0 (innermost coordinate) times the element size must be a multiple of 16 bytes; the destination
// must be 128-byte aligned.  Parts of the box outside the tensor are filled with zeros and still count.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const void *tmap, int c0, int c1, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

// Barrier over a subset of the CTA's warps (id 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void report_error(uint32_t *err_word, uint32_t code) {
    if (err_word) atomicCAS(err_word, 0u, code);
}

// Mailbox word {value, tag} of the fused all-gather, written by one GPU and polled by another.  The
// pair travels as ONE 64-bit scalar access on both sides (value in the low half, tag in the high
// half): a relaxed system-scope 64-bit store and a relaxed system-scope 64-bit load are each single
// accesses in the memory model, so a reader that sees the tag sees the value that was stored with
// it.  (A vector store of two 32-bit words would be two accesses whose order is unspecified.)
__device__ __forceinline__ void mailbox_store(uint2 *w, uint32_t value_bits, uint32_t tag) {
    const unsigned long long word = ((unsigned long long)tag << 32) | (unsigned long long)value_bits;
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(w), "l"(word) : "memory");
}
// Two neighbouring words (w 16-byte aligned) in one 16-byte store.  A vector store is performed as one
// access per element, here per 64-bit {value, tag} word, in no particular order: each word still arrives whole.
__device__ __forceinline__ void mailbox_store2(uint2 *w, uint32_t v0, uint32_t v1, uint32_t tag) {
    const unsigned long long w0 = ((unsigned long long)tag << 32) | (unsigned long long)v0;
    const unsigned long long w1 = ((unsigned long long)tag << 32) | (unsigned long long)v1;
    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(w), "l"(w0), "l"(w1) : "memory");
}
__device__ __forceinline__ uint2 mailbox_load(const uint2 *w) {
    unsigned long long word;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(word) : "l"(w) : "memory");
    return make_uint2((uint32_t)word, (uint32_t)(word >> 32));
}
// Polls until the word carries `tag`; false after `limit` polls 32 ns apart.
__device__ __forceinline__ bool mailbox_wait(const uint2 *w, uint32_t tag, uint32_t limit, uint2 &out) {
    for (uint32_t spin = 0; spin < limit; spin++) {
        out = mailbox_load(w);
        if (out.y == tag) return true;
        __nanosleep(32);
    }
    return false;
}

// Programmatic dependent launch for the short kernels of a decode step.  Launched with programmatic
// stream serialization, a kernel's CTAs may become resident while its predecessor in the stream is
// still running; pdl_prologue() at the top of the kernel first lets the NEXT kernel do the same and
// then waits until the predecessor has completed and its writes are visible.  Nothing is read or
// written before that, so the semantics are those of a plain launch; what is saved is the launch
// latency between dependent kernels (2-3 us each, several hundred kernels per decode step).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
    pdl_trigger();
    pdl_wait();
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                    bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace llmrs
