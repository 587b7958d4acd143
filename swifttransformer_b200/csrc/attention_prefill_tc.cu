// Paged, chunked causal attention for portions of prompts on the 5th-generation
// tensor cores (tcgen05), bfloat16 storage, head sizes up to 128.
//
// One thread block of 128 threads per (tile of 128 consecutive query tokens of
// one request, head): thread i owns query row i, which is also lane i of the
// block's tensor memory (TMEM).  Per tile of 64 keys:
//
//   S = Q K^T     one thread issues tcgen05.mma (M 128, N 64, K 16 per instruction) with Q and the
//                 key tile read from shared memory through matrix descriptors (K-major, 128-byte
//                 swizzle); the accumulator is 64 TMEM columns;
//   softmax       every thread reads its row of S with tcgen05.ld, masks, keeps the running maximum
//                 and sum in float, and writes P = exp2(S - max) as bfloat16 into shared memory in
//                 the same swizzled K-major layout;
//   O_t = P V     tcgen05.mma again (N = head_dim, the value tile as an MN-major operand) into the
//                 next TMEM columns; the thread reads its row back and adds it, rescaled, to the
//                 output row it keeps in registers.
//
// Completion of the asynchronous products is tracked with tcgen05.commit on an mbarrier; the wait
// is bounded (on expiry the kernel records it in `status`, frees its TMEM and returns: it cannot
// hang).  Key and value tiles are gathered page by page with 16-byte asynchronous copies, double
// buffered, directly into the swizzled layout the matrix descriptors describe; rows past the end
// of the cache are zero-filled, never read.  Several blocks share an SM (each allocates 128 or
// 256 of the 512 TMEM columns), so one block's softmax overlaps another's products.
//
// Same mathematics as attention_prefill.cu (the mma.sync kernel, which stays for head sizes
// above 128) and as the plain kernel.  Reference counterparts:
// src/csrc/kernel/fused_context_stage_attention.cu:82-453 and src/csrc/kernel/xformers_attention.cu:313-393.
#include "common.cuh"

#define TC_BM 128
#define TC_BN 64
#define TC_THREADS 128
#define TC_LOG2E 1.4426950408889634f
#define TC_WAIT_LIMIT (1u << 20)

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_cp16(uint32_t dst, const void* src, bool pred) {
    const int n = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void tc_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void tc_cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
// writes made through the generic proxy (cp.async, st.shared) become visible to the tensor cores' async proxy
__device__ __forceinline__ void tc_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ float tc_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// shared-memory matrix descriptor: 128-byte swizzle, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::f16: bfloat16 operands, float accumulator
__device__ __forceinline__ uint32_t tc_idesc(int m, int n, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, int accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
// bounded wait for the given phase parity; false: gave up
__device__ __forceinline__ bool tc_wait(uint32_t mbar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.b32 %0, 1, 0, p;\n\t}\n" : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// 32 consecutive float columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// DB: 64-wide blocks of the head dimension (1: head_dim <= 64, 2: <= 128)
template <int DB>
__global__ void __launch_bounds__(TC_THREADS)
attention_prefill_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, bf16* __restrict__ out,
                            const int* __restrict__ tiles, const int* __restrict__ q_start,
                            const int* __restrict__ start_pos, const int* __restrict__ slots,
                            const int* __restrict__ block_table, int max_pages, int n_layers, int layer,
                            int nh, int nkv, int d, int page_size, float scale_log2, int window, int* status) {
    extern __shared__ unsigned char tc_raw[];
    __shared__ __align__(8) unsigned long long s_mbar;
    __shared__ uint32_t s_tmem;
    // tiles of the swizzled layouts must start on 1024-byte boundaries
    const uint32_t base = (tc_smem(tc_raw) + 1023u) & ~1023u;
    constexpr uint32_t Q_BLK = TC_BM * 128, KV_BLK = TC_BN * 128;       // bytes of one [rows][64] block
    const uint32_t sQ = base;                                            // DB blocks
    const uint32_t sK = sQ + DB * Q_BLK;                                 // 2 buffers x DB blocks
    const uint32_t sV = sK + 2 * DB * KV_BLK;                            // 2 buffers x DB blocks
    const uint32_t sP = sV + 2 * DB * KV_BLK;                            // one [128][64] block
    constexpr int TMEM_COLS = DB == 1 ? 128 : 256;                       // 64 for S + head_dim for O, a power of two

    const int tid = threadIdx.x, warp = tid >> 5;
    const int seq = tiles[2 * blockIdx.x], off = tiles[2 * blockIdx.x + 1];
    const int h = blockIdx.y, kvh = h / (nh / nkv);
    const int tok0 = q_start[seq] + off;
    const int n_rows = min(TC_BM, q_start[seq + 1] - tok0);
    const int pos0 = start_pos[seq] + off;
    const int pos_last = pos0 + n_rows - 1;
    const int* bt = block_table + (size_t)slots[seq] * max_pages;
    const int chunks = d >> 3;
    const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kt_begin = key_lo / TC_BN, kt_end = pos_last / TC_BN + 1;
    const int kv_hi = pos_last + 1;
    const size_t head_stride = (size_t)page_size * d;
    const size_t kv_stride = (size_t)nkv * head_stride;

    const uint32_t mbar = tc_smem(&s_mbar);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(mbar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }

    // element (row, 16-byte chunk c) of a tile made of [rows][64] blocks: chunk index xor-ed with the
    // row inside each group of eight rows (the 128-byte swizzle of the matrix descriptors)
    auto tile_addr = [](uint32_t tile, uint32_t blk_bytes, int row, int c) -> uint32_t {
        return tile + (c >> 3) * blk_bytes + row * 128 + (((c & 7) ^ (row & 7)) << 4);
    };
    // two threads share a key row of a tile: one page lookup per thread and tile
    const int kv_r = tid >> 1, kv_c0 = tid & 1;
    auto load_kv = [&](int kt, int buf) {
        const int key = kt * TC_BN + kv_r;
        const bool ok = key >= key_lo && key < kv_hi;       // outside: never read (its page may be gone)
        const bf16* src = pool;
        if (ok) {
            const int page = bt[key / page_size];
            src = pool + ((size_t)page * n_layers + layer) * 2 * kv_stride + kvh * head_stride + (size_t)(key % page_size) * d;
        }
        for (int c = kv_c0; c < chunks; c += 2) {
            tc_cp16(tile_addr(sK + buf * DB * KV_BLK, KV_BLK, kv_r, c), ok ? src + c * 8 : pool, ok);
            tc_cp16(tile_addr(sV + buf * DB * KV_BLK, KV_BLK, kv_r, c), ok ? src + kv_stride + c * 8 : pool, ok);
        }
    };
    {   // the tile's queries: thread i loads row i (rows past the portion's end are zero)
        const bool ok = tid < n_rows;
        const bf16* src = q + ((size_t)(tok0 + (ok ? tid : 0)) * nh + h) * d;
        for (int c = 0; c < chunks; ++c) tc_cp16(tile_addr(sQ, Q_BLK, tid, c), src + c * 8, ok);
    }
    load_kv(kt_begin, 0);
    tc_cp_commit();

    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);     // this warp's 32 lanes
    const uint32_t t_S = tmem, t_O = tmem + TC_BN;
    const uint32_t idesc_s = tc_idesc(TC_BM, TC_BN, 0, 0);
    const uint32_t idesc_o = tc_idesc(TC_BM, d, 0, 1);

    float o_acc[DB * 64];
#pragma unroll
    for (int i = 0; i < DB * 64; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int pos = tid < n_rows ? pos0 + tid : -1;
    const int lo = window > 0 ? pos - window + 1 : 0;
    uint32_t phase = 0;
    bool alive = true;

    for (int kt = kt_begin; kt < kt_end && alive; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) load_kv(kt + 1, buf ^ 1);
        tc_cp_commit();
        tc_cp_wait<1>();
        tc_fence_async_smem();
        __syncthreads();
        // ---- S = Q K^T
        if (tid == 0) {
            tc_fence_after_sync();
            const uint32_t kb = sK + buf * DB * KV_BLK;
            for (int kk = 0; kk * 16 < d; ++kk) {
                const uint32_t o = (kk >> 2) * Q_BLK + (kk & 3) * 32, ob = (kk >> 2) * KV_BLK + (kk & 3) * 32;
                tc_mma(t_S, tc_desc(sQ + o, 16, 1024), tc_desc(kb + ob, 16, 1024), idesc_s, kk > 0);
            }
            tc_commit(mbar);
        }
        if (!tc_wait(mbar, phase)) { alive = false; }
        phase ^= 1;
        tc_fence_after_sync();
        // ---- softmax of this thread's row
        const bool need_mask = kt * TC_BN + TC_BN - 1 > pos || (window > 0 && kt * TC_BN < lo);
        float s[TC_BN];
        tc_ld32(t_row, s);              // S: columns 0..63 of this thread's lane
        tc_ld32(t_row + 32, s + 32);
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < TC_BN; ++c) {
            if (need_mask) {
                const int key = kt * TC_BN + c;
                if (key > pos || key < lo) s[c] = -INFINITY;
            }
            mx = fmaxf(mx, s[c]);
        }
        const float m_new = fmaxf(m_run, mx * scale_log2);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float corr = tc_exp2(m_run - m_use);
        m_run = m_new;
        float rs = 0.f;
        const uint32_t prow = sP + tid * 128;
#pragma unroll
        for (int c8 = 0; c8 < TC_BN / 8; ++c8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p0 = tc_exp2(fmaf(s[c8 * 8 + 2 * e], scale_log2, -m_use));
                const float p1 = tc_exp2(fmaf(s[c8 * 8 + 2 * e + 1], scale_log2, -m_use));
                rs += p0 + p1;
                __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                w[e] = *reinterpret_cast<uint32_t*>(&pk);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n"
                         ::"r"(prow + ((c8 ^ (tid & 7)) << 4)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        }
        l_run = l_run * corr + rs;
        tc_fence_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        // ---- O_t = P V
        if (tid == 0) {
            tc_fence_after_sync();
            const uint32_t vb = sV + buf * DB * KV_BLK;
            for (int j = 0; j < TC_BN / 16; ++j)
                tc_mma(t_O, tc_desc(sP + j * 32, 16, 1024), tc_desc(vb + j * 2048, KV_BLK, 1024), idesc_o, j > 0);
            tc_commit(mbar);
        }
        if (!tc_wait(mbar, phase)) { alive = false; }
        phase ^= 1;
        tc_fence_after_sync();
#pragma unroll
        for (int cb = 0; cb < DB * 2; ++cb) {
            if (cb * 32 < d) {
                float ov[32];
                tc_ld32(t_row + TC_BN + cb * 32, ov);      // O_t: columns 64..64+head_dim
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[cb * 32 + i] = fmaf(o_acc[cb * 32 + i], corr, ov[i]);
            }
        }
        tc_fence_before_sync();
        // S, O_t, P and the key/value buffer are free for the next tile; a thread whose wait expired
        // takes the whole block out of the loop, so that no barrier is ever left half-attended
        alive = __syncthreads_and(alive);
    }
    tc_cp_wait<0>();
    if (!alive && tid == 0) atomicExch(status, 3);

    if (alive && tid < n_rows) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        bf16* orow = out + ((size_t)(tok0 + tid) * nh + h) * d;
#pragma unroll
        for (int c = 0; c < DB * 8; ++c) {
            if (c * 8 < d) {
                uint4 w;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(o_acc[c * 8] * inv, o_acc[c * 8 + 1] * inv);
                __nv_bfloat162 p1 = __floats2bfloat162_rn(o_acc[c * 8 + 2] * inv, o_acc[c * 8 + 3] * inv);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(o_acc[c * 8 + 4] * inv, o_acc[c * 8 + 5] * inv);
                __nv_bfloat162 p3 = __floats2bfloat162_rn(o_acc[c * 8 + 6] * inv, o_acc[c * 8 + 7] * inv);
                w.x = *reinterpret_cast<uint32_t*>(&p0); w.y = *reinterpret_cast<uint32_t*>(&p1);
                w.z = *reinterpret_cast<uint32_t*>(&p2); w.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(orow + c * 8) = w;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int DB>
static int launch_prefill_tc(const void* q, const void* pool, void* out, const int* tiles, int n_tiles,
                             const int* q_start, const int* start_pos, const int* slots, const int* block_table,
                             int max_pages, int n_layers, int layer, int nh, int nkv, int d, int page_size,
                             float scale, int window, int* status, cudaStream_t s) {
    const size_t smem = (size_t)DB * (TC_BM * 128 + 4 * TC_BN * 128) + TC_BM * 128 + 1024;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<DB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, nh);
    attention_prefill_tc_kernel<DB><<<grid, TC_THREADS, smem, s>>>((const bf16*)q, (const bf16*)pool, (bf16*)out,
        tiles, q_start, start_pos, slots, block_table, max_pages, n_layers, layer, nh, nkv, d, page_size,
        scale * TC_LOG2E, window, status);
    return st_launch_status();
}

ST_EXPORT int st_attention_prefill_tc_max_head_dim() { return 128; }

// Same arguments as st_attention_prefill plus `status` (set to 3 if a wait for the tensor cores expired).
ST_EXPORT int st_attention_prefill_tc(const void* q, const void* pool, void* out, const int* tiles, int n_tiles,
                                      const int* q_start, const int* start_pos, const int* slots,
                                      const int* block_table, int max_pages, int n_layers, int layer, int nh,
                                      int nkv, int d, int page_size, float scale, int window, int* status,
                                      void* stream) {
    if (n_tiles <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || nh > 65535 || !status) return ST_ERR_BAD_ARG;
    if (d <= 0 || d % 16) return ST_ERR_BAD_SIZE;
    if (d > 128) return ST_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 64)
        return launch_prefill_tc<1>(q, pool, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                    n_layers, layer, nh, nkv, d, page_size, scale, window, status, s);
    return launch_prefill_tc<2>(q, pool, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                n_layers, layer, nh, nkv, d, page_size, scale, window, status, s);
}
