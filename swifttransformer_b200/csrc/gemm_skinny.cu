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
// Two fusions take a neighbour of the product into its kernel.  The residual sum behind is what decode steps
// use.  The norm in front is correct and tested but not used by the engine: in the recorded step a product
// runs fastest when all its blocks start together on an idle GPU right behind a small norm kernel (whose few
// microseconds hide the product's launch and first loads); with the norm inside, the product either starts
// early, block by block as its predecessor drains, and streams at half the rate, or starts late and shows
// its own prologue (OPT-1.3B decode step at batch 8: 1.27 to 1.68 ms against 1.12):
//   * a norm in front: the activations are norm(x) of the float residual rows x (LayerNorm or RMS norm,
//     two-pass variance in float).  The blocks form clusters of as many blocks as there are rows (1, 2, 4
//     or 8): block r of a cluster normalises row r with all its threads and stores the bfloat16 row into the
//     shared memory of every block of the cluster (distributed shared memory), so a row is read from L2 once
//     per cluster, and after one cluster barrier every block has all rows next to its tensor cores;
//   * the residual sum behind: out[m, n] += product + bias in float, in place (each element has one owner).
//
// A third variant (up to 8 tokens, K from 544 to 2048, one wave of blocks, no slices of k) brings ALL of a block's
// weights onto the SM before the wait for the kernel before it: the first two rounds in registers as ever, the
// rest (up to 48 KB per block, four blocks per SM) with 16-byte asynchronous copies into shared memory.  Behind
// a norm kernel, whose few microseconds the copies have to themselves, the product then finds its weights next
// to the tensor cores when its activations arrive, instead of streaming three quarters of them behind the wait.
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
#define SK_XPAD 32        // bfloat16 elements between the rows of the normalised activations in shared memory
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

// The float rows a norm in front of the product reads, and the norm's constants.
struct NormSource {
    const float* x;            // [M, K] residual rows
    const float* gamma;        // [K] or null
    const float* beta;         // [K] or null
    float eps;
    int kind;                  // 0 LayerNorm, 1 RMS norm, 2 none (cast only)
};

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_stream(const bf16* p) {   // weights: read once, do not keep in L1
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// KFULL: K is a multiple of 32 (known when compiling: no test on k inside a block of 32)
// XV: 0; or the float4 pieces of a row each thread normalises (K <= 1024 * XV): the norm in front; or -1: the
//     residual sum behind (out is float and the product is added to what is there); or -2: all weights brought
//     on chip before the wait (NT == 1, KFULL, no slices of k, 16 < K / 32 <= 64); -3: both of the last two;
//     -4: slices of k that do not meet: slice y leaves its sums, in float and without the bias, in out[y][M][N]
//     (blocks of their own, no cluster; the norm kernel behind adds the parts in slice order)
// out_f32: 0 bfloat16, 1 float
template <int NT, bool QKV, bool KFULL, int XV>
__global__ void __launch_bounds__(SK_THREADS, NT <= 2 ? 4 : 2)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias,
                   void* __restrict__ out, int M, int N, int K, int act, int out_f32, QkvTarget tgt, NormSource src) {
    __shared__ float red[SK_WARPS][16][8 * NT + 1];
    __shared__ float part[16 * 8 * NT];      // this block's sums over its slice of k
    extern __shared__ __align__(16) unsigned char sk_dyn[];
    bf16* xs = reinterpret_cast<bf16*>(sk_dyn);      // XV > 0: the normalised rows, [M][K + SK_XPAD]
    constexpr bool PRE = XV == -2 || XV == -3;       // the k-blocks behind the first 2 x SK_WARPS in shared memory
    constexpr bool RESID = XV == -1 || XV == -3;     // the residual sum behind
    constexpr bool PARTS = XV == -4;                 // slices of k leave their parts
    constexpr int REG_KB = 2 * SK_WARPS;
    bf16* ws = reinterpret_cast<bf16*>(sk_dyn);      // PRE: [16][K - 32 REG_KB + 32] (rows 64 bytes askew: no bank conflicts)
    const int ws_stride = K - 32 * REG_KB + 32;
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
            for (int j = 0; j < NT; ++j) {
                if (XV > 0)      // row g of the normalised rows in shared memory (rows 64 bytes askew: no bank conflicts)
                    r.xb[u][j] = (ok && xok[j]) ? *reinterpret_cast<const uint4*>(xs + (size_t)g * (K + SK_XPAD) + kb * 32 + t * 8) : zero;
                else
                    r.xb[u][j] = (ok && xok[j]) ? __ldcg(reinterpret_cast<const uint4*>(xr[j] + kb * 32)) : zero;
            }
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
    if constexpr (PRE) {
        // the rest of this block's weights, asked for now: rows row0 .. row0 + 15, k from 32 REG_KB on
        const int cpr = (K - 32 * REG_KB) >> 3;        // 16-byte pieces per row
        for (int r = warp; r < 16; r += SK_WARPS) {
            const bf16* src = w + (size_t)min(row0 + r, N - 1) * K + 32 * REG_KB;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(ws + (size_t)r * ws_stride);
            for (int c = lane; c < cpr; c += 32)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + c * 16), "l"(src + c * 8));
        }
        asm volatile("cp.async.commit_group;\n" ::);
    }
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
    // the norm's gain and shift for this thread's pieces of a row are static too
    constexpr bool NORM_PRE = XV > 0 && XV <= 2;      // wider rows: too many registers, fetched when used
    float4 gam[NORM_PRE ? XV : 1], bet[NORM_PRE ? XV : 1];
    (void)gam; (void)bet;
    if (XV > 0) cluster_arrive();                     // matched below: every block of the cluster has started
    if (NORM_PRE) {
#pragma unroll
        for (int i = 0; i < (NORM_PRE ? XV : 1); ++i) {
            const int col = (i * SK_THREADS + threadIdx.x) * 4;
            gam[i] = (src.gamma && col < K) ? *reinterpret_cast<const float4*>(src.gamma + col) : make_float4(1.f, 1.f, 1.f, 1.f);
            bet[i] = (src.beta && col < K) ? *reinterpret_cast<const float4*>(src.beta + col) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float resid_pre = 0.f;
    ST_PDL_WAIT();
    if constexpr (RESID) {
        // the residual element this thread adds to in its first epilogue turn, asked for now
        const int m = threadIdx.x >> 4, n = row0 + (threadIdx.x & 15);
        if (threadIdx.x < 16 * 8 * NT && m < M && n < N && (gridDim.y == 1 || blockIdx.y == 0))
            resid_pre = __ldcg(reinterpret_cast<const float*>(out) + (size_t)m * N + n);
    }
    if constexpr (XV > 0) {
        // Block r of the cluster normalises row r with all its threads (the pieces of the row stay in
        // registers between the two passes) and stores it, in bfloat16, into every block of the cluster.
        cg::cluster_group cluster = cg::this_cluster();
        const int cs = (int)cluster.num_blocks(), r = (int)cluster.block_rank();
        __shared__ float nscratch[32];
        bool first_row = true;
        for (int row = r; row < M; row += cs) {
            float4 v[XV > 0 ? XV : 1];
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                const int col = (i * SK_THREADS + threadIdx.x) * 4;
                v[i] = col < K ? __ldcg(reinterpret_cast<const float4*>(src.x + (size_t)row * K + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
                sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
            float mean = 0.f, rstd = 1.f;
            if (src.kind == 0) {
                mean = block_sum(sum, nscratch) / (float)K;
                float sq = 0.f;
#pragma unroll
                for (int i = 0; i < XV; ++i) {
                    const int col = (i * SK_THREADS + threadIdx.x) * 4;
                    if (col < K) {
                        const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
                        sq += (a * a + b * b) + (c * c + d * d);
                    }
                }
                rstd = rsqrtf(block_sum(sq, nscratch) / (float)K + src.eps);
            } else if (src.kind == 1) {
                float sq = 0.f;
#pragma unroll
                for (int i = 0; i < XV; ++i) sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
                rstd = rsqrtf(block_sum(sq, nscratch) / (float)K + src.eps);
            }
            if (first_row) { cluster_wait(); first_row = false; }
#pragma unroll
            for (int i = 0; i < XV; ++i) {
                const int col = (i * SK_THREADS + threadIdx.x) * 4;
                if (col < K) {
                    float4 y;
                    if (src.kind == 2) {
                        y = v[i];
                    } else {
                        float4 ga, be;
                        if (NORM_PRE) { ga = gam[NORM_PRE ? i : 0]; be = bet[NORM_PRE ? i : 0]; }
                        else {
                            ga = src.gamma ? *reinterpret_cast<const float4*>(src.gamma + col) : make_float4(1.f, 1.f, 1.f, 1.f);
                            be = src.beta ? *reinterpret_cast<const float4*>(src.beta + col) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                        y.x = (v[i].x - mean) * rstd * ga.x + be.x;
                        y.y = (v[i].y - mean) * rstd * ga.y + be.y;
                        y.z = (v[i].z - mean) * rstd * ga.z + be.z;
                        y.w = (v[i].w - mean) * rstd * ga.w + be.w;
                    }
                    uint2 packed;
                    *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(y.x, y.y);
                    *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(y.z, y.w);
                    for (int dst = 0; dst < cs; ++dst)
                        *reinterpret_cast<uint2*>(cluster.map_shared_rank(xs, dst) + (size_t)row * (K + SK_XPAD) + col) = packed;
                }
            }
        }
        if (first_row) cluster_wait();           // a block without a row of its own
        cluster.sync();                          // every row is in place in every block
        if (row0 >= N) return;                   // a block that only filled the cluster: nothing reads its memory from here on
    }
    if constexpr (PRE) {
        // the activations of all of this warp's k-blocks are asked for at once; the weights are on the SM
        issue_x(ra, kb_first);
        issue_x(rb, kb_first + STEP);
        constexpr int MAXS = (64 - REG_KB) / SK_WARPS;          // k-blocks per warp in shared memory at most
        uint4 xq[MAXS];
#pragma unroll
        for (int j = 0; j < MAXS; ++j) {
            const int kb = REG_KB + warp + j * SK_WARPS;
            xq[j] = (kb < nkb && xok[0]) ? __ldcg(reinterpret_cast<const uint4*>(xr[0] + kb * 32)) : zero;
        }
        consume(ra);
        consume(rb);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();                                        // every thread's copies have landed
#pragma unroll
        for (int j = 0; j < MAXS; ++j) {
            const int kb = REG_KB + warp + j * SK_WARPS;
            if (kb < nkb) {
                const uint4 ua = *reinterpret_cast<const uint4*>(ws + (size_t)g * ws_stride + (kb - REG_KB) * 32 + t * 8);
                const uint4 ub = *reinterpret_cast<const uint4*>(ws + (size_t)(g + 8) * ws_stride + (kb - REG_KB) * 32 + t * 8);
                mma16816(acc[0], ua.x, ub.x, ua.y, ub.y, xq[j].x, xq[j].y);
                mma16816(acc[0], ua.z, ub.z, ua.w, ub.w, xq[j].z, xq[j].w);
            }
        }
    } else if (NT == 1) {
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
    const int n_slices = PARTS ? 1 : gridDim.y;            // == cluster size when > 1
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
        if (PARTS) {
            reinterpret_cast<float*>(out)[((size_t)blockIdx.y * M + m) * N + n] = v;
            continue;
        }
        v += bias_pre;
        if (!QKV) {
            v = apply_act(v, act);
            if (RESID) {             // the residual sum, in place: this thread is the element's only owner
                float* o = reinterpret_cast<float*>(out) + (size_t)m * N + n;
                *o = (i == (int)threadIdx.x ? resid_pre : __ldcg(o)) + v;
            } else if (out_f32) reinterpret_cast<float*>(out)[(size_t)m * N + n] = v;
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

// ST_B200_SKINNY_NO_PRE=1 in the environment: no product brings its weights on chip before its wait (for measurements)
static inline bool st_skinny_pre_enabled() {
    static const char* const off = getenv("ST_B200_SKINNY_NO_PRE");
    return !(off && off[0] && off[0] != '0');
}

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

// cluster_x: blocks along x that form a cluster (the norm in front), else 1; along y the slices of k do
template <typename... KArgs, typename... Args>
static int launch_skinny_kernel(const char* tag, void (*kernel)(KArgs...), dim3 grid, size_t smem, int cluster_x,
                                cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n = 0;
    // A product whose blocks form clusters over slices of k starts after its predecessor has finished, not as
    // its blocks drain: started early, its clusters land wherever room appears and the step is 3 % slower
    // (OPT-1.3B, batch 8: 1.152 against 1.120 ms).
    if (st_pdl_enabled(tag) && grid.y == 1) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (grid.y > 1 || cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
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

template <bool QKV, int XV = 0>
static int launch_skinny(const void* x, const void* w, const float* bias, void* out, int M, int N, int K, int act,
                         int out_f32, const QkvTarget& tgt, cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 32) return ST_ERR_TOO_LARGE;
    if (K <= 0 || K % 8) return ST_ERR_BAD_SIZE;
    if (!aligned16(x) || !aligned16(w)) return ST_ERR_BAD_ARG;
    dim3 grid((N + 15) / 16, skinny_slices(N, K));
    const NormSource no_norm = {};
    if constexpr (XV == 0 || XV == -1) {
        // All weights on chip before the wait: a few tokens, K of 544 to 2048, one wave of blocks of four per SM and
        // no slices of k.  A product with the residual sum behind runs uncut this way even where it would be cut over
        // k to fill the GPU (the output projection: 128 blocks of 16 features): its blocks are started early, find
        // room beside a single-token attention of a few requests and have their 64 KB on chip when the attention
        // ends (OPT-1.3B decode step, batch 1: 0.880 -> 0.802 ms; batch 8, where the attention leaves no room: the same).
        constexpr int PV = XV == 0 ? -2 : -3;
        const bool one_slice = grid.y == 1 || XV == -1;
        const size_t pre_smem = (size_t)16 * (K - 32 * 2 * SK_WARPS + 32) * sizeof(bf16);
        if (M <= 8 && K % 32 == 0 && K > 32 * 2 * SK_WARPS && K <= 2048 && one_slice && st_skinny_pre_enabled()) {
            static int blocks_per_sm = -1;
            static size_t allowed = 0;
            if (pre_smem > allowed) {
                if (cudaFuncSetAttribute(gemm_skinny_kernel<1, QKV, true, PV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(16 * (2048 - 32 * 2 * SK_WARPS + 32) * sizeof(bf16))) == cudaSuccess)
                    allowed = 16 * (2048 - 32 * 2 * SK_WARPS + 32) * sizeof(bf16);
                else
                    (void)cudaGetLastError();
            }
            if (blocks_per_sm < 0 && allowed) {
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, gemm_skinny_kernel<1, QKV, true, PV>, SK_THREADS,
                                                                  allowed) != cudaSuccess) { (void)cudaGetLastError(); blocks_per_sm = 0; }
            }
            if (pre_smem <= allowed && (long long)grid.x <= (long long)blocks_per_sm * st_sm_count())
                return launch_skinny_kernel("skinny", gemm_skinny_kernel<1, QKV, true, PV>, dim3(grid.x, 1), pre_smem, 1, s,
                                            (const bf16*)x, (const bf16*)w, bias, out, M, N, K, act, out_f32, tgt, no_norm);
        }
    }
#define LAUNCH_SK(NT)                                                                                              \
    (K % 32 == 0 ? launch_skinny_kernel(XV == -1 ? (K > 4096 ? "gemm_add_wide" : "gemm_add") : "skinny", gemm_skinny_kernel<NT, QKV, true, XV>, grid, 0, 1, s, (const bf16*)x,      \
                                        (const bf16*)w, bias, out, M, N, K, act, out_f32, tgt, no_norm)            \
                 : launch_skinny_kernel(XV == -1 ? "gemm_add" : "skinny", gemm_skinny_kernel<NT, QKV, false, XV>, grid, 0, 1, s, (const bf16*)x,     \
                                        (const bf16*)w, bias, out, M, N, K, act, out_f32, tgt, no_norm))
    if (M <= 8) return LAUNCH_SK(1);
    if (M <= 16) return LAUNCH_SK(2);
    return LAUNCH_SK(4);
#undef LAUNCH_SK
}

// The norm in front: at most 8 rows, K a multiple of 32 up to 8192.  One block per 16 features, no slices of
// k (the blocks along x form clusters of as many blocks as rows instead).
ST_EXPORT int st_gemm_skinny_norm_applies(int M, int K) { return M >= 1 && M <= 8 && K % 32 == 0 && K >= 32 && K <= 8192; }

template <bool QKV>
static int launch_skinny_norm(const NormSource& src, const void* w, const float* bias, void* out, int M, int N, int K,
                              int act, int out_f32, const QkvTarget& tgt, cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (!st_gemm_skinny_norm_applies(M, K)) return ST_ERR_BAD_SIZE;
    if (src.kind < 0 || src.kind > 2) return ST_ERR_BAD_ARG;
    if (!aligned16(src.x) || !aligned16(w) || !aligned16(src.gamma) || !aligned16(src.beta)) return ST_ERR_BAD_ARG;
    int cs = 1;
    while (cs < M) cs *= 2;
    const int tiles = (N + 15) / 16;
    dim3 grid((tiles + cs - 1) / cs * cs, 1);
    const size_t smem = (size_t)M * (K + SK_XPAD) * sizeof(bf16);
#define LAUNCH_SKN(XV)                                                                                             \
    do {                                                                                                           \
        static size_t allowed = 48 * 1024 - 6 * 1024;      /* what a kernel may use without asking, less its static part */ \
        if (smem > allowed) {                                                                                      \
            cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<1, QKV, true, XV>,                             \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (e != cudaSuccess) return (int)e;                                                                   \
            allowed = smem;                                                                                        \
        }                                                                                                          \
        return launch_skinny_kernel(QKV ? "qkv_norm" : "gemm_norm", gemm_skinny_kernel<1, QKV, true, XV>, grid, smem, cs, s, (const bf16*)nullptr, \
                                    (const bf16*)w, bias, out, M, N, K, act, out_f32, tgt, src);                   \
    } while (0)
    if (K <= 1024) LAUNCH_SKN(1);
    if (K <= 2048) LAUNCH_SKN(2);
    if (K <= 4096) LAUNCH_SKN(4);
    LAUNCH_SKN(8);
#undef LAUNCH_SKN
}

// act( norm(x) . w^T + bias ) for at most 8 float rows x [M, K]: the norm of st_add_norm (kind 0 LayerNorm, 1 RMS
// norm, 2 none; gamma and beta may be null) fused in front of the product.
ST_EXPORT int st_gemm_skinny_norm(const float* x, const float* gamma, const float* beta, float eps, int kind,
                                  const void* w, const float* bias, void* out, int M, int N, int K, int act,
                                  int out_f32, void* stream) {
    const NormSource src = {x, gamma, beta, eps, kind};
    QkvTarget none = {};
    if (out_f32 < 0 || out_f32 > 1) return ST_ERR_BAD_ARG;
    return launch_skinny_norm<false>(src, w, bias, out, M, N, K, act, out_f32, none, (cudaStream_t)stream);
}

// The slices of k a product of up to 8 tokens is cut into (st_gemm_skinny_parts_slices(N, K); 1: it is not cut) as
// blocks of their own: parts [slices][M][N] float = the slices' sums of x . w^T, no bias.  No cluster and no early
// start: the launch of a cluster and the meeting of its blocks through distributed shared memory cost 1.3 us per
// product in a decode step, and the norm kernel that follows reads the parts in the trip to memory it makes anyway.
ST_EXPORT int st_gemm_skinny_parts_slices(int N, int K) { return (K > 0 && K % 32 == 0 && N > 0) ? skinny_slices(N, K) : 1; }

ST_EXPORT int st_gemm_skinny_parts(const void* x, const void* w, float* parts, int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 8) return ST_ERR_TOO_LARGE;
    if (K <= 0 || K % 32) return ST_ERR_BAD_SIZE;
    if (!aligned16(x) || !aligned16(w) || !parts) return ST_ERR_BAD_ARG;
    const dim3 grid((N + 15) / 16, skinny_slices(N, K));
    const QkvTarget none = {};
    const NormSource no_norm = {};
    gemm_skinny_kernel<1, false, true, -4><<<grid, SK_THREADS, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, (const bf16*)w, nullptr, parts, M, N, K, 0, 1, none, no_norm);
    return st_launch_status();
}

// out [M, N] (float) += x . w^T + bias: the residual sum fused behind the product.
ST_EXPORT int st_gemm_skinny_add(const void* x, const void* w, const float* bias, float* out, int M, int N, int K,
                                 void* stream) {
    QkvTarget none = {};
    return launch_skinny<false, -1>(x, w, bias, out, M, N, K, 0, 1, none, (cudaStream_t)stream);
}

ST_EXPORT int st_gemm_skinny(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                             int act, int out_f32, void* stream) {
    if (out_f32 < 0 || out_f32 > 1) return ST_ERR_BAD_ARG;
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

// The same with the norm of the float residual rows x fused in front (see st_gemm_skinny_norm).
ST_EXPORT int st_gemm_skinny_norm_qkv(const float* x, const float* gamma, const float* beta, float eps, int kind,
                                      const void* w, const float* bias, void* q_out, void* pool,
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
    const NormSource src = {x, gamma, beta, eps, kind};
    return launch_skinny_norm<true>(src, w, bias, nullptr, M, (nh + 2 * nkv) * d, K, 0, 0, tgt, (cudaStream_t)stream);
}
