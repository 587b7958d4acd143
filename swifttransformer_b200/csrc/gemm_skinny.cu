// Matrix product for a handful of tokens (decode steps), bfloat16:
//   out[m, n] = act( sum_k x[m,k] * w[n,k] + bias[n] ),   m < M <= 32,  w stored [out, in]
// At these sizes the product is weight streaming: every byte of w is read once
// and the arithmetic is free, so the kernel is built around the loads.
//
// Operands are swapped for the tensor cores: 16 rows of w are the M side of an
// m16n8k16 product and 8 tokens its N side.  A thread loads its fragments
// straight from global memory, 16 contiguous bytes at a time: within a block of
// 32 k the lane with (group g, thread-in-group t) takes k = 8t..8t+7 of row g and
// row g+8 of w and of token g of x, and feeds elements (0,1 | 2,3) and (4,5 | 6,7)
// to two consecutive products.  (The activations are read with L2-only loads: under programmatic
// dependent launch this block may have become resident before its predecessor wrote them, and
// only loads that bypass the per-SM caches are sure to see the new values after the wait.)  The product sums over k, so any assignment of k
// to fragment slots is right as long as w and x use the same one.  No shared
// memory staging, no barriers in the main loop; each of the block's 8 warps
// takes every 8th k-block (two rounds of two blocks in flight) and the partial sums meet in
// shared memory.  One thread block per 16 output features and slice of k: when
// there are too few features to fill the GPU, k is cut into up to 8 slices
// (gridDim.y) whose blocks form a thread-block cluster; the partial sums stay
// in each block's shared memory, and after a cluster barrier the first block
// of the cluster adds them in slice order through distributed shared memory
// and runs the epilogue.  No global scratch, no fences, no atomics: a round
// trip through L2 costs more than a microsecond here, and the old scheme
// (scratch + counter + re-read) needed four of them.
//
// Epilogues: bias and activation; float or bfloat16 output; or the fused
// q|k|v form: q (+bias) to a dense buffer, k and v (+bias) straight into the
// paged cache at each token's position (what st_qkv_to_cache does after a
// library product).
//
// The reference calls cuBLAS for these products at every batch size
// (src/csrc/layer/attention.cc:102-111,255-264, src/csrc/layer/ffn.cc:71-105,
// src/csrc/model/gpt/gpt.cc:192-201) and adds bias / activation / cache
// writes in separate kernels.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)
#define SK_UNROLL 1      // k-blocks per round with up to 8 tokens; one with more (registers: four blocks per SM either way)

struct QkvTarget {
    bf16* q_out;               // [M, qw]
    bf16* pool;                // paged cache
    const int* positions;      // [M]
    const int* seq_of_token;   // [M]
    const int* slots;          // [sequences]
    const int* block_table;    // [slots, max_pages]
    int* status;
    int max_pages, num_pages, n_layers, layer, nkv, d, page_size, qw, write_kv;
};

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const bf16* p) {   // weights: read once, do not keep in L1
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// KFULL: K is a multiple of 32 (known when compiling: no test on k inside a block of 32)
template <int NT, bool QKV, bool KFULL>
__global__ void __launch_bounds__(SK_THREADS, NT <= 2 ? 4 : 2)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias,
                   void* __restrict__ out, int M, int N, int K, int act, int out_f32, QkvTarget tgt) {
    __shared__ float red[SK_WARPS][16][8 * NT + 1];
    __shared__ float part[16 * 8 * NT];      // this block's sums over its slice of k
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 16;
    const bf16* wa = w + (size_t)min(row0 + g, N - 1) * K + t * 8;
    const bf16* wb = w + (size_t)min(row0 + g + 8, N - 1) * K + t * 8;
    const bf16* xr[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = j * 8 + g < M;
        xr[j] = x + (size_t)(xok[j] ? j * 8 + g : 0) * K + t * 8;
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    // this block's slice of the k-blocks
    const int nkb_all = (K + 31) >> 5;
    const int per_slice = (nkb_all + gridDim.y - 1) / gridDim.y;
    const int kb_begin = blockIdx.y * per_slice;
    const int nkb = min(nkb_all, kb_begin + per_slice);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // Two register buffers of SK_UNROLL k-blocks each: the loads of the next round are in flight
    // while the current one is multiplied.  The successor may be scheduled from now on; this
    // kernel's own first round of weight loads is issued before it waits for its predecessor
    // (weights are written by no kernel, so the memory system stays busy across the kernel
    // boundary); the activations are read after the wait.
    constexpr int UNR = NT == 1 ? SK_UNROLL : 1;
    struct Round { uint4 ua[UNR], ub[UNR], xb[UNR][NT]; };
    auto issue_w = [&](Round& r, int kb0) {
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int kb = kb0 + u * SK_WARPS;
            const bool ok = kb < nkb && (KFULL || kb * 32 + t * 8 < K);   // K % 8 == 0: a 16-byte piece is inside or outside as a whole
            r.ua[u] = ok ? ldg_stream(wa + kb * 32) : zero;
            r.ub[u] = ok ? ldg_stream(wb + kb * 32) : zero;
        }
    };
    auto issue_x = [&](Round& r, int kb0) {
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int kb = kb0 + u * SK_WARPS;
            const bool ok = kb < nkb && (KFULL || kb * 32 + t * 8 < K);
#pragma unroll
            for (int j = 0; j < NT; ++j)
                r.xb[u][j] = (ok && xok[j]) ? __ldcg(reinterpret_cast<const uint4*>(xr[j] + kb * 32)) : zero;
        }
    };
    auto consume = [&](const Round& r) {
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                mma16816(acc[j], r.ua[u].x, r.ub[u].x, r.ua[u].y, r.ub[u].y, r.xb[u][j].x, r.xb[u][j].y);
                mma16816(acc[j], r.ua[u].z, r.ub[u].z, r.ua[u].w, r.ub[u].w, r.xb[u][j].z, r.xb[u][j].w);
            }
        }
    };
    ST_PDL_TRIGGER();
    constexpr int STEP = SK_WARPS * UNR;
    const int kb_first = kb_begin + warp;
    Round ra, rb, rc;
    issue_w(ra, kb_first);          // out-of-range blocks load nothing
    if (NT == 1) issue_w(rb, kb_first + STEP);
    // What the epilogue needs and no kernel of the step writes is fetched now, under the weight stream,
    // instead of at the end, where every dependent load is a round trip on the critical path: the bias
    // of this thread's output feature (the same in all of its epilogue turns, 256 being a multiple of
    // 16) and, for key/value features, the page of its first token (a chain of four loads).
    float bias_pre = 0.f;
    if (bias && row0 + (int)(threadIdx.x & 15) < N) bias_pre = bias[row0 + (threadIdx.x & 15)];
    int pos_pre = -1, page_pre = -1;
    if (QKV && tgt.write_kv && row0 + 15 >= tgt.qw && (int)(threadIdx.x >> 4) < M && threadIdx.x < 16 * 8 * NT) {
        const int m = threadIdx.x >> 4;
        pos_pre = tgt.positions[m];
        if (pos_pre >= 0)
            page_pre = tgt.block_table[(size_t)tgt.slots[tgt.seq_of_token[m]] * tgt.max_pages + pos_pre / tgt.page_size];
    }
    ST_PDL_WAIT();
    if (NT == 1) {
        // three rounds in flight (two of them asked for before the wait)
        issue_x(ra, kb_first);
        issue_x(rb, kb_first + STEP);
        for (int kb0 = kb_first; kb0 < nkb; kb0 += 3 * STEP) {
            if (kb0 + 2 * STEP < nkb) { issue_w(rc, kb0 + 2 * STEP); issue_x(rc, kb0 + 2 * STEP); }
            consume(ra);
            if (kb0 + 3 * STEP < nkb) { issue_w(ra, kb0 + 3 * STEP); issue_x(ra, kb0 + 3 * STEP); }
            if (kb0 + STEP < nkb) consume(rb);
            if (kb0 + 4 * STEP < nkb) { issue_w(rb, kb0 + 4 * STEP); issue_x(rb, kb0 + 4 * STEP); }
            if (kb0 + 2 * STEP < nkb) consume(rc);
        }
    } else {
        issue_x(ra, kb_first);
        for (int kb0 = kb_first; kb0 < nkb; kb0 += 2 * STEP) {
            const bool more_b = kb0 + STEP < nkb;
            if (more_b) { issue_w(rb, kb0 + STEP); issue_x(rb, kb0 + STEP); }
            consume(ra);
            if (kb0 + 2 * STEP < nkb) { issue_w(ra, kb0 + 2 * STEP); issue_x(ra, kb0 + 2 * STEP); }
            if (more_b) consume(rb);
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        red[warp][g][j * 8 + 2 * t] = acc[j][0];
        red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
        red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
        red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    const int n_slices = gridDim.y;            // == cluster size when > 1
    if (n_slices > 1) {
        for (int i = threadIdx.x; i < 16 * 8 * NT; i += SK_THREADS) {
            const int r = i & 15, m = i >> 4;
            float v = 0.f;
#pragma unroll
            for (int wi = 0; wi < SK_WARPS; ++wi) v += red[wi][r][m];
            part[i] = v;
        }
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                        // every slice's sums are in place
        if (cluster.block_rank() != 0) {
            cluster.sync();                    // stay until the first block has read this block's sums
            return;
        }
    }
    for (int i = threadIdx.x; i < 16 * 8 * NT; i += SK_THREADS) {
        const int r = i & 15, m = i >> 4;
        const int n = row0 + r;
        float v = 0.f;
        if (n_slices > 1) {
            cg::cluster_group cluster = cg::this_cluster();
            for (int sl = 0; sl < n_slices; ++sl) v += cluster.map_shared_rank(part, sl)[i];
        } else {
#pragma unroll
            for (int wi = 0; wi < SK_WARPS; ++wi) v += red[wi][r][m];
        }
        if (m >= M || n >= N) continue;
        v += bias_pre;
        if (!QKV) {
            v = apply_act(v, act);
            if (out_f32) reinterpret_cast<float*>(out)[(size_t)m * N + n] = v;
            else reinterpret_cast<bf16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(v);
        } else {
            if (n < tgt.qw) {
                tgt.q_out[(size_t)m * tgt.qw + n] = __float2bfloat16_rn(v);
            } else if (tgt.write_kv) {
                const bool pre = i == (int)threadIdx.x;     // this thread's first turn: fetched at the start
                const int pos = pre ? pos_pre : tgt.positions[m];
                if (pos < 0) continue;                      // padding token of a fixed-shape step
                const int page = pre ? page_pre
                                     : tgt.block_table[(size_t)tgt.slots[tgt.seq_of_token[m]] * tgt.max_pages + pos / tgt.page_size];
                if (page < 0 || page >= tgt.num_pages) { atomicExch(tgt.status, 1); continue; }
                const int kw = tgt.nkv * tgt.d;
                const int rr = n - tgt.qw;
                const int kv = rr / kw, rem = rr - kv * kw;
                const int head = rem / tgt.d, dim = rem - head * tgt.d;
                tgt.pool[(((((size_t)page * tgt.n_layers + tgt.layer) * 2 + kv) * tgt.nkv + head) * tgt.page_size
                          + pos % tgt.page_size) * tgt.d + dim] = __float2bfloat16_rn(v);
            }
        }
    }
    if (n_slices > 1) cg::this_cluster().sync();   // the other blocks of the cluster may leave now
}

ST_EXPORT int st_gemm_skinny_max_rows() { return 32; }

// how many slices k is cut into (the cluster size): as many blocks as fit on the GPU at once (about
// four per SM) and no more, at most 8; at least one round of loads per warp and slice
static int skinny_slices(int N, int K) {
    const int tiles = (N + 15) / 16;
    int s = (4 * st_sm_count()) / tiles;
    const int nkb = (K + 31) / 32;
    if (s > nkb / (SK_WARPS * SK_UNROLL)) s = nkb / (SK_WARPS * SK_UNROLL);
    if (s > 8) s = 8;
    return s < 1 ? 1 : s;
}

template <typename... KArgs, typename... Args>
static int launch_skinny_kernel(void (*kernel)(KArgs...), dim3 grid, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (st_pdl_enabled("skinny")) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (grid.y > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = grid.y;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return st_launch_status();
}

template <bool QKV>
static int launch_skinny(const void* x, const void* w, const float* bias, void* out, int M, int N, int K, int act,
                         int out_f32, const QkvTarget& tgt, cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 32) return ST_ERR_TOO_LARGE;
    if (K <= 0 || K % 8) return ST_ERR_BAD_SIZE;
    if (!aligned16(x) || !aligned16(w)) return ST_ERR_BAD_ARG;
    dim3 grid((N + 15) / 16, skinny_slices(N, K));
#define LAUNCH_SK(NT)                                                                                              \
    (K % 32 == 0 ? launch_skinny_kernel(gemm_skinny_kernel<NT, QKV, true>, grid, s, (const bf16*)x, (const bf16*)w, \
                                        bias, out, M, N, K, act, out_f32, tgt)                                      \
                 : launch_skinny_kernel(gemm_skinny_kernel<NT, QKV, false>, grid, s, (const bf16*)x, (const bf16*)w, \
                                        bias, out, M, N, K, act, out_f32, tgt))
    if (M <= 8) return LAUNCH_SK(1);
    if (M <= 16) return LAUNCH_SK(2);
    return LAUNCH_SK(4);
#undef LAUNCH_SK
}

ST_EXPORT int st_gemm_skinny(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                             int act, int out_f32, void* stream) {
    QkvTarget none = {};
    return launch_skinny<false>(x, w, bias, out, M, N, K, act, out_f32, none, (cudaStream_t)stream);
}

// x [M,K] . w [(nh + 2 nkv) d, K]^T + bias -> q_out [M, nh d] and the paged cache
ST_EXPORT int st_gemm_skinny_qkv(const void* x, const void* w, const float* bias, void* q_out, void* pool,
                                 const int* positions, const int* seq_of_token, const int* slots,
                                 const int* block_table, int max_pages, int num_pages, int n_layers, int layer,
                                 int M, int K, int nh, int nkv, int d, int page_size, int write_kv, int* status,
                                 void* stream) {
    if (nh <= 0 || nkv <= 0 || d <= 0 || page_size <= 0 || layer < 0 || layer >= n_layers) return ST_ERR_BAD_ARG;
    QkvTarget tgt;
    tgt.q_out = (bf16*)q_out; tgt.pool = (bf16*)pool; tgt.positions = positions; tgt.seq_of_token = seq_of_token;
    tgt.slots = slots; tgt.block_table = block_table; tgt.status = status; tgt.max_pages = max_pages;
    tgt.num_pages = num_pages; tgt.n_layers = n_layers; tgt.layer = layer; tgt.nkv = nkv; tgt.d = d;
    tgt.page_size = page_size; tgt.qw = nh * d; tgt.write_kv = write_kv;
    return launch_skinny<true>(x, w, bias, nullptr, M, (nh + 2 * nkv) * d, K, 0, 0, tgt, (cudaStream_t)stream);
}
