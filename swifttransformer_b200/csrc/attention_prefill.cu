// Paged, chunked causal attention for portions of prompts, bfloat16 storage.
//
// One thread block per (tile of 128 consecutive query tokens of one request,
// head).  The queries at positions start_pos + off .. attend every key of the
// request up to their own position (or inside their window), so a portion
// that begins in the middle of a prompt reads the earlier portions' keys from
// the pages and its own keys, written just before, from the same place.  Key
// and value tiles of 64 positions, aligned to absolute positions, are gathered
// page by page into shared memory with 16-byte asynchronous copies (double
// buffered); scores and the weighted value sum run on the tensor cores
// (m16n8k16, bfloat16 in, float accumulate), softmax statistics are float and
// online.  Rows of a tile past the end of the cache are filled with zeros, not
// read: a reused page may hold anything.
//
// Reference counterparts: src/csrc/kernel/fused_context_stage_attention.cu:82-453
// (16x16 wmma tiles over this step's q/k/v buffer only, whole prompts only) and
// src/csrc/kernel/xformers_attention.cu:313-393.  Chunked prefill over the
// cache has no counterpart there.
#include "mma_sync.cuh"

#define PF_BM 128            // query rows per thread block (16 per warp)
#define PF_BN 64             // keys per tile
#define PF_THREADS 256
#define LOG2E 1.4426950408889634f

// tiles[i] = {index of the request in the step, offset of the tile in the request's new tokens}
template <int DMAX>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, bf16* __restrict__ out,
                         const int* __restrict__ tiles, const int* __restrict__ q_start,
                         const int* __restrict__ start_pos, const int* __restrict__ slots,
                         const int* __restrict__ block_table, int max_pages, int n_layers, int layer,
                         int nh, int nkv, int d, int page_size, float scale_log2, int window, int q_stride,
                         int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK = sQ + PF_BM * DMAX;            // [2][PF_BN][DMAX]
    bf16* sV = sK + 2 * PF_BN * DMAX;        // [2][PF_BN][DMAX]

    // the head is x, the fastest index in the order blocks start: all heads of the longest tile first
    const int seq = tiles[2 * blockIdx.y], off = tiles[2 * blockIdx.y + 1];
    const int h = blockIdx.x, kvh = h / (nh / nkv);
    const int tok0 = q_start[seq] + off;
    const int n_rows = min(PF_BM, q_start[seq + 1] - tok0);
    if (n_rows <= 0) return;      // a padding tile of a fixed-shape step (the whole block leaves before any barrier)
    const int pos0 = start_pos[seq] + off;           // position of the tile's first query
    const int pos_last = pos0 + n_rows - 1;
    const int* bt = block_table + (size_t)slots[seq] * max_pages;
    const int chunks = d >> 3;                       // 16-byte chunks per row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kt_begin = key_lo / PF_BN, kt_end = pos_last / PF_BN + 1;
    const int kv_hi = pos_last + 1;                  // keys at or beyond this are never needed

    const size_t head_stride = (size_t)page_size * d;
    const size_t kv_stride = (size_t)nkv * head_stride;

    // four threads share a key row of a tile: one page lookup per thread and tile
    constexpr int KV_TPR = PF_THREADS / PF_BN;
    const int kv_r = threadIdx.x / KV_TPR, kv_c0 = threadIdx.x % KV_TPR;
    auto load_kv = [&](int kt, int buf) {
        bf16* dk = sK + buf * PF_BN * DMAX;
        bf16* dv = sV + buf * PF_BN * DMAX;
        const int key = kt * PF_BN + kv_r;
        bool ok = key >= key_lo && key < kv_hi;         // outside: never read (its page may be gone)
        const bf16* src = pool;
        if (ok) {
            const int page = bt[key / page_size];
            ok = page >= 0;                             // a hole in the block table: zeros, no access before the pool
            if (!ok && status) *status = 1;             // and the host hears of it
            if (ok) src = pool + ((size_t)page * n_layers + layer) * 2 * kv_stride + kvh * head_stride
                          + (size_t)(key % page_size) * d;
        }
        for (int c = kv_c0; c < chunks; c += KV_TPR) {
            cp_async16(tile_ptr<DMAX>(dk, kv_r, c), ok ? src + c * 8 : pool, ok);
            cp_async16(tile_ptr<DMAX>(dv, kv_r, c), ok ? src + kv_stride + c * 8 : pool, ok);
        }
    };

    // queries of the tile (rows past the portion's end are zero)
    {
        constexpr int Q_TPR = PF_THREADS / PF_BM;
        const int r = threadIdx.x / Q_TPR;
        const bool ok = r < n_rows;
        const bf16* src = q + (size_t)(tok0 + (ok ? r : 0)) * q_stride + h * d;
        for (int c = threadIdx.x % Q_TPR; c < chunks; c += Q_TPR) cp_async16(tile_ptr<DMAX>(sQ, r, c), src + c * 8, ok);
    }
    load_kv(kt_begin, 0);
    cp_async_commit();

    float o_acc[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    // running maximum in the scaled (log2) domain, running sum
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // this thread's two rows of the warp's 16 and their positions (-1: no query in that row)
    const int row_a = warp * 16 + (lane >> 2), row_b = row_a + 8;
    const int pos_a = row_a < n_rows ? pos0 + row_a : -1;
    const int pos_b = row_b < n_rows ? pos0 + row_b : -1;
    const int lo_a = window > 0 ? pos_a - window + 1 : 0, lo_b = window > 0 ? pos_b - window + 1 : 0;
    // the warp's rows: a tile whose keys all lie at or before the first row's position (and inside
    // every row's window) needs no mask
    const int warp_pos_first = pos0 + warp * 16;
    const bool warp_full = warp * 16 + 16 <= n_rows;
    const bool warp_idle = warp * 16 >= n_rows;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) load_kv(kt + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* tK = sK + buf * PF_BN * DMAX;
        const bf16* tV = sV + buf * PF_BN * DMAX;
        // a warp whose rows all lie before this tile's first key (causal) has nothing to do in it
        const bool skip = warp_idle || kt * PF_BN > warp_pos_first + 15;
        if (!skip) {
            // S = Q K^T for the warp's 16 rows x 64 keys
            float s_acc[PF_BN / 8][4];
#pragma unroll
            for (int i = 0; i < PF_BN / 8; ++i) { s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < DMAX / 16; ++kk) {
                if (kk * 16 < d) {
                    uint32_t a[4];
                    ldmatrix_x4(a[0], a[1], a[2], a[3],
                                tile_ptr<DMAX>(sQ, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4)));
#pragma unroll
                    for (int np = 0; np < PF_BN / 16; ++np) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(b0, b1, b2, b3,
                                    tile_ptr<DMAX>(const_cast<bf16*>(tK), np * 16 + (lane & 7) + (lane >> 4) * 8,
                                                   2 * kk + ((lane >> 3) & 1)));
                        mma_bf16(s_acc[2 * np], a, b0, b1);
                        mma_bf16(s_acc[2 * np + 1], a, b2, b3);
                    }
                }
            }
            // mask (only on tiles that touch the diagonal, a window's edge or a ragged last warp)
            const bool need_mask = !warp_full || kt * PF_BN + PF_BN - 1 > warp_pos_first ||
                                   (window > 0 && kt * PF_BN < warp_pos_first + 15 - window + 1);
            if (need_mask) {
#pragma unroll
                for (int nt = 0; nt < PF_BN / 8; ++nt) {
                    const int key = kt * PF_BN + nt * 8 + (lane & 3) * 2;
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int k2 = key + e;
                        if (k2 > pos_a || k2 < lo_a) s_acc[nt][e] = -INFINITY;
                        if (k2 > pos_b || k2 < lo_b) s_acc[nt][2 + e] = -INFINITY;
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < PF_BN / 8; ++nt) {
                mx[0] = fmaxf(mx[0], fmaxf(s_acc[nt][0], s_acc[nt][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s_acc[nt][2], s_acc[nt][3]));
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r] * scale_log2);   // scale > 0: max commutes with it
                m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;            // a row with no key yet
                corr[r] = fast_exp2(m_run[r] - m_use[r]);                 // m_run = -inf: 0
                m_run[r] = m_new;
            }
            float rs[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < PF_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pa = fast_exp2(fmaf(s_acc[nt][e], scale_log2, -m_use[0]));
                    const float pb = fast_exp2(fmaf(s_acc[nt][2 + e], scale_log2, -m_use[1]));
                    s_acc[nt][e] = pa; s_acc[nt][2 + e] = pb;
                    rs[0] += pa; rs[1] += pb;
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
                rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
                l_run[r] = l_run[r] * corr[r] + rs[r];
            }
#pragma unroll
            for (int i = 0; i < DMAX / 8; ++i) {
                o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
                o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
            }
            // O += P V
#pragma unroll
            for (int j = 0; j < PF_BN / 16; ++j) {
                uint32_t a[4];
                a[0] = pack_bf16(s_acc[2 * j][0], s_acc[2 * j][1]);
                a[1] = pack_bf16(s_acc[2 * j][2], s_acc[2 * j][3]);
                a[2] = pack_bf16(s_acc[2 * j + 1][0], s_acc[2 * j + 1][1]);
                a[3] = pack_bf16(s_acc[2 * j + 1][2], s_acc[2 * j + 1][3]);
#pragma unroll
                for (int np = 0; np < DMAX / 16; ++np) {
                    if (np * 16 < d) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4_trans(b0, b1, b2, b3,
                                          tile_ptr<DMAX>(const_cast<bf16*>(tV), j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                         2 * np + (lane >> 4)));
                        mma_bf16(o_acc[2 * np], a, b0, b1);
                        mma_bf16(o_acc[2 * np + 1], a, b2, b3);
                    }
                }
            }
        }
        __syncthreads();   // the buffer is refilled by the next round's copies
    }
    cp_async_wait<0>();

    // normalise and store
    const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
    for (int nt = 0; nt < DMAX / 8; ++nt) {
        const int dim = nt * 8 + (lane & 3) * 2;
        if (dim < d) {
            if (row_a < n_rows)
                *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(tok0 + row_a) * nh + h) * d + dim) =
                    __floats2bfloat162_rn(o_acc[nt][0] * inv_a, o_acc[nt][1] * inv_a);
            if (row_b < n_rows)
                *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(tok0 + row_b) * nh + h) * d + dim) =
                    __floats2bfloat162_rn(o_acc[nt][2] * inv_b, o_acc[nt][3] * inv_b);
        }
    }
}

template <int DMAX>
static int launch_prefill(const void* q, const void* pool, void* out, const int* tiles, int n_tiles,
                          const int* q_start, const int* start_pos, const int* slots, const int* block_table,
                          int max_pages, int n_layers, int layer, int nh, int nkv, int d, int page_size,
                          float scale, int window, int q_stride, int* status, cudaStream_t s) {
    const size_t smem = (size_t)(PF_BM + 4 * PF_BN) * DMAX * sizeof(bf16);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DMAX>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nh, n_tiles);
    attention_prefill_kernel<DMAX><<<grid, PF_THREADS, smem, s>>>((const bf16*)q, (const bf16*)pool, (bf16*)out,
        tiles, q_start, start_pos, slots, block_table, max_pages, n_layers, layer, nh, nkv, d, page_size,
        scale * LOG2E, window, q_stride, status);
    return st_launch_status();
}

ST_EXPORT int st_attention_prefill_tile_rows() { return PF_BM; }

ST_EXPORT int st_attention_prefill(const void* q, const void* pool, void* out, const int* tiles, int n_tiles,
                                   const int* q_start, const int* start_pos, const int* slots,
                                   const int* block_table, int max_pages, int n_layers, int layer, int nh, int nkv,
                                   int d, int page_size, float scale, int window, int q_stride, int* status, void* stream) {
    if (n_tiles <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || n_tiles > 65535) return ST_ERR_BAD_ARG;
    if (d <= 0 || d % 16) return ST_ERR_BAD_SIZE;
    if (d > 256) return ST_ERR_TOO_LARGE;
    if (q_stride <= 0) q_stride = nh * d;      // a dense [tokens, nh * d] query tensor
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 64)
        return launch_prefill<64>(q, pool, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                  n_layers, layer, nh, nkv, d, page_size, scale, window, q_stride, status, s);
    if (d <= 128)
        return launch_prefill<128>(q, pool, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                   n_layers, layer, nh, nkv, d, page_size, scale, window, q_stride, status, s);
    return launch_prefill<256>(q, pool, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                               n_layers, layer, nh, nkv, d, page_size, scale, window, q_stride, status, s);
}
