// Host side of TMA: tensor maps for bfloat16 tensors with the 128-byte swizzle, built with the driver's
// cuTensorMapEncodeTiled, which is found through the runtime (the library does not link libcuda).
// No reference counterpart (the reference's kernels predate TMA).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

typedef CUresult (*st_tma_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline st_tma_encode_fn st_tma_encoder() {
    static st_tma_encode_fn fn = nullptr;
    static bool looked_up = false;
    if (!looked_up) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (st_tma_encode_fn)p;
        else
            (void)cudaGetLastError();
        looked_up = true;
    }
    return fn;
}

// rank: 2 or 3; dims / box in elements, innermost first; rows of the tensor are contiguous.  The innermost
// box extent must be 64 elements (128 bytes, the swizzle's span).  Returns 0 or -1.
static inline int st_tma_encode_bf16(CUtensorMap* out, const void* base, int rank, const unsigned long long* dims,
                                     const unsigned* box) {
    st_tma_encode_fn enc = st_tma_encoder();
    if (!enc || rank < 2 || rank > 3 || box[0] != 64) return -1;
    cuuint64_t d[3], strides[2];
    cuuint32_t b[3], elem[3] = {1, 1, 1};
    unsigned long long stride = 2;
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        stride *= dims[i];
        if (i + 1 < rank) strides[i] = stride;       // bytes between consecutive indices of dimension i + 1
    }
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, strides,
                           b, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1;
}
