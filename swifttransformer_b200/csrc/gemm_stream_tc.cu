// Matrix product for a few dozen tokens (decode steps of 9 to 128 requests), bfloat16, on the
// 5th-generation tensor cores fed by TMA:
//   out[m, n] = act( sum_k x[m,k] * w[n,k] + bias[n] ),   m < M <= 128,  w stored [out, in]
// At these sizes the product is still weight streaming (every byte of w is read once, x stays in L2), so
// the kernel is a deep copy pipeline with the arithmetic on the side.
//
// Operands are swapped: 128 rows of w are the M side of tcgen05.mma (the lanes of tensor memory), the
// tokens its N side (16 to 128, a multiple of 16), so a block's accumulator is 128 lanes x M columns.
// One warp issues TMA copies (a [128 x 64] box of w and a [M x 64] box of x per stage, landing in the
// 128-byte swizzle the matrix descriptors expect, completion by mbarrier expect_tx); one warp issues the
// products (four K=16 steps per stage, tcgen05.commit frees the stage); four warps read the accumulator
// with tcgen05.ld and run the epilogue.  The copies of w start before the programmatic-launch dependency
// is waited for (weights do not depend on the step), those of x after it.
//
// One block per 128 output features and slice of k.  When there are too few feature tiles to occupy the
// GPU, k is cut into up to 8 slices whose blocks form a thread-block cluster: each leaves its partial
// tile in its own shared memory and, after a cluster barrier, reduces every S-th token column over all
// slices through distributed shared memory, in slice order, and runs the epilogue for it.  No global
// scratch, no atomics; the result does not depend on timing.
//
// Waits are bounded: a wait that expires marks the block dead, `status` gets 5, and the block leaves
// after freeing its tensor memory.  The reference calls cuBLAS for these products at every batch size
// (src/csrc/layer/attention.cc:102-111,255-264, src/csrc/layer/ffn.cc:71-105) and adds bias and
// activation in separate kernels.
#include <cooperative_groups.h>
#include <mutex>

#include "tcgen05.cuh"
#include "tma_host.h"
namespace cg = cooperative_groups;

#define GS_THREADS 192          // warp 0: copies, warp 1: products, warps 2-5: epilogue
#define GS_STAGES 6
#define GS_BM 128               // output features per block (tensor-memory lanes)
#define GS_BK 64                // k per stage: one 128-byte swizzle span

__device__ __forceinline__ bool gs_wait(uint32_t mbar, uint32_t parity, volatile int* dead) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.b32 %0, 1, 0, p;\n\t}\n" : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
        if (done) return true;
        if (i > 64) {
            if ((i & 63) == 0 && *dead) return false;
            __nanosleep(32);
        }
    }
    *dead = 1;
    return false;
}

// mt: tokens rounded up to a multiple of 16 (the N of the products and the rows of an x box)
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_tc_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                      const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int mt,
                      int act, int out_f32, int* status) {
    extern __shared__ unsigned char gs_raw[];
    __shared__ __align__(8) unsigned long long s_full[GS_STAGES], s_empty[GS_STAGES], s_accum;
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;
    ST_PDL_TRIGGER();
    const uint32_t base = (tc_smem(gs_raw) + 1023u) & ~1023u;
    const uint32_t W_BYTES = GS_BM * 128, X_BYTES = (uint32_t)mt * 128;       // bytes of one stage's boxes
    const uint32_t STAGE = W_BYTES + ((X_BYTES + 1023u) & ~1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tmem_cols = mt <= 32 ? 32 : (mt <= 64 ? 64 : 128);
    const int n0 = blockIdx.x * GS_BM;
    const int n_slices = gridDim.y, slice = blockIdx.y;
    const int nkb = (K + GS_BK - 1) / GS_BK;
    const int kb_per = (nkb + n_slices - 1) / n_slices;
    const int kb_begin = slice * kb_per, kb_end = min(nkb, kb_begin + kb_per);
    const int n_it = max(0, kb_end - kb_begin);
    volatile int* dead = &s_dead;

    if (tid == 0) {
        for (int s = 0; s < GS_STAGES; ++s) {
            tc_mbar_init(tc_smem(&s_full[s]), 1);
            tc_mbar_init(tc_smem(&s_empty[s]), 1);
        }
        tc_mbar_init(tc_smem(&s_accum), 1);
        tc_mbar_init_fence();
        s_dead = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem(&s_tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;

    if (warp == 0 && lane == 0) {
        // ---- copies.  The first stages' weights go out before the wait for the kernel before this one.
        const int ahead = min(n_it, GS_STAGES);
        for (int it = 0; it < ahead; ++it) {
            const uint32_t full = tc_smem(&s_full[it]);
            tc_mbar_expect_tx(full, W_BYTES + X_BYTES);
            tc_tma_load_2d(base + it * STAGE, &w_map, (kb_begin + it) * GS_BK, n0, full);
        }
        ST_PDL_WAIT();
        for (int it = 0; it < ahead; ++it)
            tc_tma_load_2d(base + it * STAGE + W_BYTES, &x_map, (kb_begin + it) * GS_BK, 0, tc_smem(&s_full[it]));
        for (int it = ahead; it < n_it; ++it) {
            const int s = it % GS_STAGES;
            if (!gs_wait(tc_smem(&s_empty[s]), ((it / GS_STAGES) - 1) & 1, dead)) break;
            const uint32_t full = tc_smem(&s_full[s]);
            tc_mbar_expect_tx(full, W_BYTES + X_BYTES);
            tc_tma_load_2d(base + s * STAGE, &w_map, (kb_begin + it) * GS_BK, n0, full);
            tc_tma_load_2d(base + s * STAGE + W_BYTES, &x_map, (kb_begin + it) * GS_BK, 0, full);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- products: D[128 features x mt tokens] += W tile (K-major) . X tile^T (K-major)
        const uint32_t idesc = tc_idesc(GS_BM, mt, 0, 0);
        for (int it = 0; it < n_it; ++it) {
            const int s = it % GS_STAGES;
            if (!gs_wait(tc_smem(&s_full[s]), (it / GS_STAGES) & 1, dead)) break;
            tc_fence_after_sync();
            const uint64_t dw = tc_desc(base + s * STAGE, 16, 1024), dx = tc_desc(base + s * STAGE + W_BYTES, 16, 1024);
#pragma unroll
            for (int kk = 0; kk < GS_BK / 16; ++kk) tc_mma(tmem, dw + ((kk * 32) >> 4), dx + ((kk * 32) >> 4), idesc, it > 0 || kk > 0);
            tc_commit(tc_smem(&s_empty[s]));
        }
        tc_commit(tc_smem(&s_accum));
    }
    // ---- epilogue warps: thread (q, lane) owns feature 32 q + lane, where q = warp % 4 names the
    // quarter of the tensor-memory lanes this warp may read
    float* part = reinterpret_cast<float*>(gs_raw + (base - tc_smem(gs_raw)));    // [mt][128], over the stages
    bool alive = true;
    if (warp >= 2) {
        const int q = warp & 3, f = q * 32 + lane;
        const int n = n0 + f;
        if (n_it > 0) alive = gs_wait(tc_smem(&s_accum), 0, dead);
        tc_fence_after_sync();
        const float b = (bias && n < N && slice == 0 && n_slices == 1) ? bias[n] : 0.f;
        const uint32_t t_row = tmem + ((uint32_t)(q * 32) << 16);
        for (int c0 = 0; c0 < mt; c0 += 32) {
            float v[32];
            if (n_it > 0) { tc_ld32(t_row + c0, v); tc_ld_wait(); }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int m = c0 + j;
                if (m >= mt) continue;
                const float a = n_it > 0 ? v[j] : 0.f;
                if (n_slices > 1) {
                    part[m * GS_BM + f] = a;
                } else if (m < M && n < N && alive) {
                    const float r = apply_act(a + b, act);
                    if (out_f32) reinterpret_cast<float*>(out)[(size_t)m * N + n] = r;
                    else reinterpret_cast<bf16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(r);
                }
            }
        }
    }
    tc_fence_before_sync();
    if (n_slices > 1) {
        // every slice's tile is in its block's shared memory (the products and copies that used the
        // space have completed: the accumulator barrier follows the last product)
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (warp >= 2) {
            const int q = warp & 3, f = q * 32 + lane;
            const int n = n0 + f;
            const float b = (bias && n < N) ? bias[n] : 0.f;
            // Four tokens per turn with all their remote loads in flight together: a load from another
            // block's shared memory takes most of a microsecond, and one token at a time made this loop
            // the longest part of the kernel.  The sum runs in slice order.
            const float* remote[8];
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) remote[sl] = cluster.map_shared_rank(part, sl < n_slices ? sl : 0);
            for (int m0 = slice; m0 < M; m0 += 4 * n_slices) {
                float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int m = m0 + u * n_slices;
#pragma unroll
                    for (int sl = 0; sl < 8; ++sl)
                        if (sl < n_slices && m < M) a[u] += remote[sl][m * GS_BM + f];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int m = m0 + u * n_slices;
                    if (m < M && n < N) {
                        const float r = apply_act(a[u] + b, act);
                        if (out_f32) reinterpret_cast<float*>(out)[(size_t)m * N + n] = r;
                        else reinterpret_cast<bf16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(r);
                    }
                }
            }
        }
        cluster.sync();           // the other blocks may still be reading this block's tile
    } else {
        __syncthreads();
    }
    if (s_dead && tid == 0) atomicExch(status, 5);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------------
struct GsMapEntry {
    const void* ptr;
    long long rows, cols;
    unsigned box_rows;
    CUtensorMap map;
};
static std::mutex gs_mutex;
static GsMapEntry gs_maps[256];
static int gs_n_maps = 0, gs_next = 0;

// map of a row-major [rows, cols] bfloat16 matrix with boxes of box_rows x 64; weights are looked up in a
// small table (their maps never change), activations are encoded per call
static int gs_map(const void* ptr, long long rows, long long cols, unsigned box_rows, bool cache, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(gs_mutex);
    if (cache) {
        for (int i = 0; i < gs_n_maps; ++i) {
            const GsMapEntry& e = gs_maps[i];
            if (e.ptr == ptr && e.rows == rows && e.cols == cols && e.box_rows == box_rows) { *out = e.map; return 0; }
        }
    }
    const unsigned long long dims[2] = {(unsigned long long)cols, (unsigned long long)rows};
    const unsigned box[2] = {GS_BK, box_rows};
    if (st_tma_encode_bf16(out, ptr, 2, dims, box)) return ST_ERR_BAD_ARG;
    if (cache) {
        GsMapEntry& e = gs_maps[gs_next];
        e.ptr = ptr; e.rows = rows; e.cols = cols; e.box_rows = box_rows; e.map = *out;
        gs_next = (gs_next + 1) % 256;
        if (gs_n_maps < 256) ++gs_n_maps;
    }
    return 0;
}

// slices of k (the cluster size): enough blocks to occupy the GPU with one block per SM, at least four
// stages of k per slice, at most 8
static int gs_slices(int N, int K) {
    const int tiles = (N + GS_BM - 1) / GS_BM, nkb = (K + GS_BK - 1) / GS_BK;
    int s = st_sm_count() / tiles;
    if (s > nkb / 4) s = nkb / 4;
    if (s > 8) s = 8;
    return s < 1 ? 1 : s;
}

ST_EXPORT int st_gemm_stream_tc_max_rows() { return 128; }

// x [M, K] bfloat16, w [N, K] bfloat16, bias [N] float or null, out [M, N] bfloat16 or float; K % 8 == 0.
// `status` (device int) is set to 5 if a wait inside the kernel expired.
ST_EXPORT int st_gemm_stream_tc(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                                int act, int out_f32, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 128) return ST_ERR_TOO_LARGE;
    if (K <= 0 || K % 8) return ST_ERR_BAD_SIZE;
    if (!aligned16(x) || !aligned16(w) || !status) return ST_ERR_BAD_ARG;
    const int mt = (M + 15) / 16 * 16;
    CUtensorMap w_map, x_map;
    int r = gs_map(w, N, K, GS_BM, true, &w_map);
    if (r) return r;
    r = gs_map(x, M, K, (unsigned)mt, false, &x_map);
    if (r) return r;
    const size_t stage = (size_t)GS_BM * 128 + (((size_t)mt * 128 + 1023) & ~(size_t)1023);
    const size_t smem = GS_STAGES * stage + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (smem > 200 * 1024) return ST_ERR_TOO_LARGE;
    const int slices = gs_slices(N, K);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + GS_BM - 1) / GS_BM, slices);
    cfg.blockDim = dim3(GS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (st_pdl_enabled("stream_tc")) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (slices > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = slices;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_tc_kernel, w_map, x_map, bias, out, M, N, K, mt, act, out_f32, status);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return st_launch_status();
}
