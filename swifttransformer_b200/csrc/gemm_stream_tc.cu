// Matrix product for a few dozen tokens (decode steps of 9 to 128 requests), bfloat16, on the
// 5th-generation tensor cores fed by TMA:
//   out[m, n] = act( sum_k x[m,k] * w[n,k] + bias[n] ),   m < M <= 128,  w stored [out, in]
// At these sizes the product is still weight streaming (every byte of w is read once, x stays in L2), and in
// a decode step it waits for the kernel before it.  So the kernel is two deep copy rings with the arithmetic
// on the side, and the ring of the weights is filled BEFORE the wait: when the activations arrive, most of
// a block's weights are already in its shared memory.
//
// Operands are swapped: BM rows of w (64 or 128) are the M side of tcgen05.mma (the lanes of tensor memory),
// the tokens its N side (16 to 128, a multiple of 16), so a block's accumulator is BM lanes x M columns.
// Tiles of 64 features give one block per SM without cutting k for the model's wide products (q|k|v 96,
// fc1 128 tiles at OPT-1.3B); where even they are too few (output projection, fc2: 32 tiles) k is cut into
// slices whose blocks do NOT meet: each leaves its float sums in `parts[slice][M][N]`, and the norm kernel
// behind adds them in slice order to the residual rows it reads anyway (no cluster, no atomics, no second
// pass; the result does not depend on timing).
//
// A stage is 32 KB of weights: G = 4 (2) blocks of 64 k for 64 (128) rows, fetched by ONE copy of a rank-3 box
// [64 k][rows][G blocks of k] (the matrix seen as [k % 64][row][k / 64]), which lands as G tiles of rows x 128
// bytes in the 128-byte swizzle the matrix descriptors expect.  What a box holds of one row is what it reads
// contiguously from memory, and that decides the rate: with one block of k per box (128 bytes of a row) all the
// blocks of the GPU together drew 1.5 TB/s whatever the depth of their rings; with 512 bytes of a row 4.2 TB/s (the
// library's products, whose tiles also hold 128 bytes of a row, reach 3.5 to 4.1; the mma.sync kernel, which
// reads whole rows, 5.5).  The engine does not use this kernel (see ops.STREAM_TC_MAX_ROWS): in a decode step it
// cannot start copying under the kernel before it, because a block that keeps 200 KB in flight never shares an
// SM with that kernel's blocks, and kernel against kernel the library is ahead.
//
// Warps: 0 issues the weight copies (completion by mbarrier expect_tx; the first ring-full before the
// programmatic-launch dependency is waited for), 1 the activation copies (a [64 k][M][G] box per stage, after
// the wait), 2 the products (4 G K=16 steps per stage; tcgen05.commit frees both stages), 4-7 read the accumulator with tcgen05.ld and run the epilogue (warp 3 idles: a warp may
// only read the quarter of tensor memory that its number modulo 4 names).  With 64 rows the accumulator lies
// in lanes 0-15 of every quarter, so half the lanes of an epilogue warp carry a feature.
//
// Waits are bounded: a wait that expires marks the block dead, `status` gets 5, and the block leaves
// after freeing its tensor memory.  The reference calls cuBLAS for these products at every batch size
// (src/csrc/layer/attention.cc:102-111,255-264, src/csrc/layer/ffn.cc:71-105) and adds bias and
// activation in separate kernels.
#include <mutex>

#include "tcgen05.cuh"
#include "tma_host.h"

#define GS_THREADS 256
#define GS_BK 64                // k per stage: one 128-byte swizzle span
#define GS_MAX_W 8              // stages of the weight ring at most
#define GS_MAX_X 4              // stages of the activation ring at most
#define GS_RING_BYTES (216 * 1024)

#ifdef GS_PROFILE
__device__ unsigned long long gs_prof[4][64];
__device__ __forceinline__ unsigned long long gs_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define GS_STAMP(i) do { if (blockIdx.y == 0 && (blockIdx.x & 31) == 0 && (blockIdx.x >> 5) < 4) gs_prof[blockIdx.x >> 5][i] = gs_now(); } while (0)
ST_EXPORT int st_gemm_stream_tc_profile(unsigned long long* host) { return (int)cudaMemcpyFromSymbol(host, gs_prof, sizeof(gs_prof)); }
#else
#define GS_STAMP(i) do {} while (0)
#endif

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
// nw, nx: stages of the two rings.  parts != null: slice blockIdx.y leaves its float sums in parts[slice][M][N]
// (no bias, no activation); else gridDim.y == 1 and out gets act(sum + bias).
template <int BM>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_tc_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                      const float* __restrict__ bias, void* __restrict__ out, float* __restrict__ parts, int M, int N,
                      int K, int mt, int nw, int nx, int act, int out_f32, int* status) {
    extern __shared__ unsigned char gs_raw[];
    __shared__ __align__(8) unsigned long long s_wfull[GS_MAX_W], s_wempty[GS_MAX_W], s_xfull[GS_MAX_X],
        s_xempty[GS_MAX_X], s_accum;
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;
    ST_PDL_TRIGGER();
    if (threadIdx.x == 0) GS_STAMP(0);
    constexpr int G = 256 / BM;                                              // blocks of 64 k per stage
    constexpr uint32_t W_TILE = BM * 128, W_BYTES = W_TILE * G;              // bytes of one weight stage
    const uint32_t X_TILE = (uint32_t)mt * 128, X_BYTES = X_TILE * G;        // bytes of one activation stage
    const uint32_t wbase = (tc_smem(gs_raw) + 1023u) & ~1023u;
    const uint32_t xbase = wbase + (uint32_t)nw * W_BYTES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tmem_cols = mt <= 32 ? 32 : (mt <= 64 ? 64 : 128);
    const int n0 = blockIdx.x * BM;
    const int n_slices = gridDim.y, slice = blockIdx.y;
    const int nkb = (K / GS_BK + G - 1) / G;                                 // stages of k in all
    const int kb_per = (nkb + n_slices - 1) / n_slices;
    const int kb_begin = slice * kb_per, kb_end = min(nkb, kb_begin + kb_per);
    const int n_it = max(0, kb_end - kb_begin);
    volatile int* dead = &s_dead;

    if (tid == 0) {
        for (int s = 0; s < nw; ++s) {
            tc_mbar_init(tc_smem(&s_wfull[s]), 1);
            tc_mbar_init(tc_smem(&s_wempty[s]), 1);
        }
        for (int s = 0; s < nx; ++s) {
            tc_mbar_init(tc_smem(&s_xfull[s]), 1);
            tc_mbar_init(tc_smem(&s_xempty[s]), 1);
        }
        tc_mbar_init(tc_smem(&s_accum), 1);
        tc_mbar_init_fence();
        s_dead = 0;
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem(&s_tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    if (threadIdx.x == 0) GS_STAMP(1);

    if (warp == 0 && lane == 0) {
        // ---- weights: they do not depend on the step, so the ring is filled at once; a stage is refilled
        // when the products that read it have completed
        for (int it = 0; it < n_it; ++it) {
            const int s = it % nw;
            if (it >= nw && !gs_wait(tc_smem(&s_wempty[s]), ((it / nw) - 1) & 1, dead)) break;
            const uint32_t full = tc_smem(&s_wfull[s]);
            tc_mbar_expect_tx(full, W_BYTES);
            tc_tma_load_3d(wbase + s * W_BYTES, &w_map, 0, n0, (kb_begin + it) * G, full);
            if (it < 8) GS_STAMP(8 + it);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- activations: written by the kernel before this one
        ST_PDL_WAIT();
        GS_STAMP(2);
        for (int it = 0; it < n_it; ++it) {
            const int s = it % nx;
            if (it >= nx && !gs_wait(tc_smem(&s_xempty[s]), ((it / nx) - 1) & 1, dead)) break;
            const uint32_t full = tc_smem(&s_xfull[s]);
            tc_mbar_expect_tx(full, X_BYTES);
            tc_tma_load_3d(xbase + s * X_BYTES, &x_map, 0, 0, (kb_begin + it) * G, full);
            if (it < 8) GS_STAMP(16 + it);
        }
    } else if (warp == 2 && lane == 0) {
        // ---- products: D[BM features x mt tokens] += W tile (K-major) . X tile^T (K-major)
        const uint32_t idesc = tc_idesc(BM, mt, 0, 0);
        for (int it = 0; it < n_it; ++it) {
            const int sw = it % nw, sx = it % nx;
            if (!gs_wait(tc_smem(&s_wfull[sw]), (it / nw) & 1, dead)) break;
            if (it < 8) GS_STAMP(24 + it);
            if (!gs_wait(tc_smem(&s_xfull[sx]), (it / nx) & 1, dead)) break;
            if (it < 8) GS_STAMP(32 + it);
            tc_fence_after_sync();
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint64_t dw = tc_desc(wbase + sw * W_BYTES + g * W_TILE, 16, 1024);
                const uint64_t dx = tc_desc(xbase + sx * X_BYTES + g * X_TILE, 16, 1024);
#pragma unroll
                for (int kk = 0; kk < GS_BK / 16; ++kk)
                    tc_mma(tmem, dw + ((kk * 32) >> 4), dx + ((kk * 32) >> 4), idesc, it > 0 || g > 0 || kk > 0);
            }
            tc_commit(tc_smem(&s_wempty[sw]));
            tc_commit(tc_smem(&s_xempty[sx]));
        }
        tc_commit(tc_smem(&s_accum));
    } else if (warp >= 4) {
        // ---- epilogue: quarter q of the tensor-memory lanes belongs to warp 4 + q; with 128 rows lane l of the
        // quarter is feature 32 q + l, with 64 rows lanes 0-15 are features 16 q + l and the others carry nothing
        constexpr int PER_Q = BM / 4;
        const int q = warp & 3, f = q * PER_Q + lane;
        const int n = n0 + f;
        const bool mine = lane < PER_Q && n < N;
        bool alive = true;
        if (n_it > 0) alive = gs_wait(tc_smem(&s_accum), 0, dead);
        if (warp == 4 && lane == 0) GS_STAMP(3);
        tc_fence_after_sync();
        const float b = (bias && mine && !parts) ? bias[n] : 0.f;
        const uint32_t t_row = tmem + ((uint32_t)(q * 32) << 16);
        for (int c0 = 0; c0 < mt; c0 += 32) {
            float v[32];
            if (n_it > 0) { tc_ld32(t_row + c0, v); tc_ld_wait(); }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int m = c0 + j;
                if (m >= M || !mine || !alive) continue;
                const float a = n_it > 0 ? v[j] : 0.f;
                if (parts) {
                    parts[((size_t)slice * M + m) * N + n] = a;
                } else {
                    const float r = apply_act(a + b, act);
                    if (out_f32) reinterpret_cast<float*>(out)[(size_t)m * N + n] = r;
                    else reinterpret_cast<bf16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(r);
                }
            }
        }
    }
    if (warp == 4 && lane == 0) GS_STAMP(4);
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) GS_STAMP(5);
    if (s_dead && tid == 0) atomicExch(status, 5);
    if (warp == 2) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------------
struct GsMapEntry {
    const void* ptr;
    long long rows, cols;
    unsigned box_rows, depth;
    CUtensorMap map;
};
static std::mutex gs_mutex;
static GsMapEntry gs_maps[256];
static int gs_n_maps = 0, gs_next = 0;

// map of a row-major [rows, cols] bfloat16 matrix (cols a multiple of 64) seen as [cols / 64][rows][64], with
// boxes of 64 x box_rows x (256 / box_rows... the caller's depth); weights are looked up in a small table (their
// maps never change), activations are encoded per call
static int gs_map(const void* ptr, long long rows, long long cols, unsigned box_rows, unsigned depth, bool cache,
                  CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(gs_mutex);
    if (cache) {
        for (int i = 0; i < gs_n_maps; ++i) {
            const GsMapEntry& e = gs_maps[i];
            if (e.ptr == ptr && e.rows == rows && e.cols == cols && e.box_rows == box_rows && e.depth == depth) { *out = e.map; return 0; }
        }
    }
    const unsigned long long dims[3] = {GS_BK, (unsigned long long)rows, (unsigned long long)(cols / GS_BK)};
    const unsigned long long strides[2] = {(unsigned long long)cols * 2, GS_BK * 2};     // bytes: a row, a block of k
    const unsigned box[3] = {GS_BK, box_rows, depth};
    if (st_tma_encode_bf16_strided(out, ptr, 3, dims, strides, box)) return ST_ERR_BAD_ARG;
    if (cache) {
        GsMapEntry& e = gs_maps[gs_next];
        e.ptr = ptr; e.rows = rows; e.cols = cols; e.box_rows = box_rows; e.depth = depth; e.map = *out;
        gs_next = (gs_next + 1) % 256;
        if (gs_n_maps < 256) ++gs_n_maps;
    }
    return 0;
}

// rows of w per block: 64 while that gives at most one block per SM, else 128
static int gs_bm(int N) { return (N + 63) / 64 <= st_sm_count() ? 64 : 128; }

// slices of k when the slices' sums are left as parts: enough blocks to occupy the GPU with one block per SM,
// at least two stages of k (64 KB of weights) per slice, at most 8
static int gs_slices(int N, int K) {
    const int bm = gs_bm(N), g = 256 / bm;
    const int tiles = (N + bm - 1) / bm, nkb = (K / GS_BK + g - 1) / g;
    int s = st_sm_count() / tiles;
    if (s > nkb / 2) s = nkb / 2;
    if (s > 8) s = 8;
    return s < 1 ? 1 : s;
}

ST_EXPORT int st_gemm_stream_tc_max_rows() { return 128; }

// Into how many slices of k st_gemm_stream_tc_parts cuts a product with w [N, K] (1: it is not cut).
ST_EXPORT int st_gemm_stream_tc_slices(int N, int K) { return (N <= 0 || K <= 0) ? 1 : gs_slices(N, K); }

// Whether the kernel runs this product in one wave of blocks (one per SM at most), which is where it is meant to be
// used: more blocks than SMs run one after the other with nothing to hide the turn-round.
ST_EXPORT int st_gemm_stream_tc_one_wave(int N) {
    const int bm = gs_bm(N);
    return N > 0 && (N + bm - 1) / bm <= st_sm_count();
}

static int gs_launch(const void* x, const void* w, const float* bias, void* out, float* parts, int slices, int M, int N,
                     int K, int act, int out_f32, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 128) return ST_ERR_TOO_LARGE;
    if (K <= 0 || K % GS_BK) return ST_ERR_BAD_SIZE;
    if (!aligned16(x) || !aligned16(w) || !status) return ST_ERR_BAD_ARG;
    const int mt = (M + 15) / 16 * 16;
    const int bm = gs_bm(N), g = 256 / bm;
    CUtensorMap w_map, x_map;
    int r = gs_map(w, N, K, (unsigned)bm, (unsigned)g, true, &w_map);
    if (r) return r;
    r = gs_map(x, M, K, (unsigned)mt, (unsigned)g, false, &x_map);
    if (r) return r;
    // the rings: two stages of activations (four when they are small), the rest weights
    const int nkb = (K / GS_BK + g - 1) / g;
    const int per_slice = (nkb + slices - 1) / slices;
    const size_t wb = (size_t)bm * 128 * g, xb = (size_t)mt * 128 * g;
    int nx = mt > 32 ? 2 : GS_MAX_X;
    if (nx > per_slice) nx = per_slice;
    int nw = (int)((GS_RING_BYTES - nx * xb) / wb);
    if (nw > GS_MAX_W) nw = GS_MAX_W;
    if (nw > per_slice) nw = per_slice;
    if (nw < 1 || nx < 1) return ST_ERR_TOO_LARGE;
    const size_t smem = nw * wb + nx * xb + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             GS_RING_BYTES + 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_stream_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     GS_RING_BYTES + 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + bm - 1) / bm, slices);
    cfg.blockDim = dim3(GS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    int n = 0;
    if (st_pdl_enabled("stream_tc")) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    const cudaError_t e =
        bm == 64 ? cudaLaunchKernelEx(&cfg, gemm_stream_tc_kernel<64>, w_map, x_map, bias, out, parts, M, N, K, mt, nw, nx,
                                      act, out_f32, status)
                 : cudaLaunchKernelEx(&cfg, gemm_stream_tc_kernel<128>, w_map, x_map, bias, out, parts, M, N, K, mt, nw,
                                      nx, act, out_f32, status);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return st_launch_status();
}

// x [M, K] bfloat16, w [N, K] bfloat16, bias [N] float or null, out [M, N] bfloat16 or float; K % 64 == 0.
// `status` (device int) is set to 5 if a wait inside the kernel expired.
ST_EXPORT int st_gemm_stream_tc(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                                int act, int out_f32, int* status, void* stream) {
    return gs_launch(x, w, bias, out, nullptr, 1, M, N, K, act, out_f32, status, stream);
}

// The slices' float sums of x . w^T, parts [st_gemm_stream_tc_slices(N, K)][M][N]: no bias, no activation.
ST_EXPORT int st_gemm_stream_tc_parts(const void* x, const void* w, float* parts, int M, int N, int K, int* status,
                                      void* stream) {
    if (!parts) return ST_ERR_BAD_ARG;
    return gs_launch(x, w, nullptr, nullptr, parts, (N <= 0 || K <= 0) ? 1 : gs_slices(N, K), M, N, K, 0, 1, status, stream);
}
