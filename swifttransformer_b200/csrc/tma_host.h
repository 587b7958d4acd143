// Host side of TMA: tensor maps for bfloat16 tensors with the 128-byte swizzle, built with the driver's
// cuTensorMapEncodeTiled, which is found through the runtime (the library does not link libcuda).
// No reference counterpart (the reference's kernels predate TMA).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

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

// The same with the strides given: strides[i] is the distance in bytes between consecutive indices of dimension
// i + 1 (a multiple of 16; dimensions may be listed in any order of their strides, the innermost is contiguous).
static inline int st_tma_encode_bf16_strided(CUtensorMap* out, const void* base, int rank, const unsigned long long* dims,
                                             const unsigned long long* strides, const unsigned* box) {
    st_tma_encode_fn enc = st_tma_encoder();
    if (!enc || rank < 2 || rank > 3 || box[0] != 64) return -1;
    cuuint64_t d[3], st[2];
    cuuint32_t b[3], elem[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        if (i + 1 < rank) st[i] = strides[i];
    }
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, st, b,
                           elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1;
}

// The tensor map of a paged key/value pool for the attention kernels fed by TMA: a rank-3 tensor
// [page x layer x (K|V) x kv_head][position in page][head_dim] with boxes of one page of one head and 64 of its
// elements.  Encoded once per pool and geometry and kept in a small table (per translation unit).
// rows: pages x layers x 2 x kv_heads.  Returns 0 or -4 (ST_ERR_BAD_ARG).
static inline int st_tma_pool_map(const void* pool, long long rows, int page_size, int d, CUtensorMap* out) {
    struct Entry {
        const void* pool;
        long long rows;
        int page_size, d;
        CUtensorMap map;
    };
    static std::mutex mutex;
    static Entry table[16];
    static int n = 0, next = 0;
    std::lock_guard<std::mutex> lock(mutex);
    for (int i = 0; i < n; ++i) {
        const Entry& e = table[i];
        if (e.pool == pool && e.rows == rows && e.page_size == page_size && e.d == d) {
            *out = e.map;
            return 0;
        }
    }
    const unsigned long long dims[3] = {(unsigned long long)d, (unsigned long long)page_size, (unsigned long long)rows};
    const unsigned box[3] = {64, (unsigned)page_size, 1};
    CUtensorMap m;
    if (st_tma_encode_bf16(&m, pool, 3, dims, box)) return -4;
    Entry& e = table[next];
    e.pool = pool; e.rows = rows; e.page_size = page_size; e.d = d; e.map = m;
    next = (next + 1) % 16;
    if (n < 16) ++n;
    *out = m;
    return 0;
}
