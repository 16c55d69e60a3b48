// Host side of the tiled TMA copies: cuTensorMapEncodeTiled, reached through the runtime's driver
// entry point lookup so that the library needs no link against libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace llmrs {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 2-D tensor of `rows` rows of `row_elems` elements, rows `row_stride_bytes` apart; box = box_elems x box_rows.
inline cudaError_t encode_2d(CUtensorMap *out, CUtensorMapDataType type, const void *base, uint64_t row_elems,
                             uint64_t rows, uint64_t row_stride_bytes, uint32_t box_elems, uint32_t box_rows,
                             CUtensorMapSwizzle swizzle) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {row_elems, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_elems, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, type, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace llmrs
