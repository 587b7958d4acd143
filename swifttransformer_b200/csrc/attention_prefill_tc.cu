// Paged, chunked causal attention for portions of prompts on the 5th-generation
// tensor cores (tcgen05), bfloat16 storage, head sizes up to 128.
//
// Two warpgroups (256 threads) work on one (tile of 128 consecutive query tokens
// of one request, head).  In each warpgroup thread i owns query row i, which is
// also lane i of tensor memory (TMEM); the two warpgroups take alternate key
// tiles (the chain of dependent steps is what bounds a causal tile's time, and
// this halves it) and merge their results at the end.  A kernel that allocates
// tensor memory gets one thread block per SM (the occupancy query says so for
// every block size and shared-memory size); a block may hold several such
// sets (TC_SETS, neighbouring heads of the same query tile).  Measured on
// OPT-1.3B shapes, one set per block (108 us per layer) beats two (125 us).
// Per tile of 64 keys, in one warpgroup:
//
//   S = Q K^T     one thread issues tcgen05.mma (M 128, N 64, K 16 per instruction) with Q and the
//                 key tile read from shared memory through matrix descriptors (K-major, 128-byte
//                 swizzle); the accumulator is 64 TMEM columns;
//   softmax       every thread reads its row of S with tcgen05.ld, masks, keeps the running maximum
//                 and sum in float, and writes P = exp2(S - max) as bfloat16 into shared memory in
//                 the same swizzled K-major layout;
//   O += P V      tcgen05.mma again (N = head_dim, the value tile as an MN-major operand),
//                 accumulating in the next TMEM columns.  The reference maximum of a row is only
//                 moved when the true maximum has grown by more than 2^8 (then the row of O is
//                 rescaled in TMEM with tcgen05.ld / tcgen05.st); otherwise P is taken relative
//                 to the older reference, which is exact after the final division by the sum.
// O += P V of a tile and S of the warpgroup's next tile are issued together and share one
// completion barrier, so a tile costs one round trip to the tensor cores.
//
// Completion of the asynchronous products is tracked with tcgen05.commit on an mbarrier; the wait
// is bounded (on expiry the kernel records it in `status`, frees its TMEM and returns: it cannot
// hang).  Key and value tiles are gathered page by page with 16-byte asynchronous copies directly into the swizzled layout the matrix descriptors describe; rows past the end
// of the cache are zero-filled, never read.  Two blocks share an SM for head sizes up to 64 (each allocates 256
// of the 512 TMEM columns), so one warpgroup's softmax overlaps another's products.
//
// Same mathematics as attention_prefill.cu (the mma.sync kernel, which stays for head sizes
// above 128) and as the plain kernel.  Reference counterparts:
// src/csrc/kernel/fused_context_stage_attention.cu:82-453 and src/csrc/kernel/xformers_attention.cu:313-393.
#include "tcgen05.cuh"

#define TC_SET_THREADS 256  // two warpgroups work on one (query tile, head)

// DB: 64-wide blocks of the head dimension (1: head_dim <= 64, 2: <= 128).  TC_SETS (query tile, head)
// pairs per block: a set needs 2 x (64 + 64 DB) of the 512 tensor-memory columns, so 2 is possible for DB == 1.
#define TC_SETS 1
template <int DB>
__global__ void __launch_bounds__(TC_SETS * TC_SET_THREADS, 1)
attention_prefill_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, bf16* __restrict__ out,
                            const int* __restrict__ tiles, const int* __restrict__ q_start,
                            const int* __restrict__ start_pos, const int* __restrict__ slots,
                            const int* __restrict__ block_table, int max_pages, int n_layers, int layer,
                            int nh, int nkv, int d, int page_size, float scale_log2, int window, int q_stride, int* status) {
    extern __shared__ unsigned char tc_raw[];
    constexpr int SETS = TC_SETS;
    __shared__ __align__(8) unsigned long long s_mbar[2 * SETS];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead[2 * SETS];
    // tiles of the swizzled layouts must start on 1024-byte boundaries
    const uint32_t base = (tc_smem(tc_raw) + 1023u) & ~1023u;
    constexpr uint32_t Q_BLK = TC_BM * 128, KV_BLK = TC_BN * 128;       // bytes of one [rows][64] block
    constexpr uint32_t WG_BYTES = 2 * DB * KV_BLK + Q_BLK;              // K, V (DB blocks each), P
    constexpr int WG_COLS = 64 + 64 * DB;                               // S, then O
    constexpr uint32_t SET_BYTES = DB * Q_BLK + 2 * WG_BYTES;           // Q, then the two warpgroups' tiles
    constexpr int TMEM_COLS = SETS * 2 * WG_COLS <= 256 ? 256 : 512;    // SETS x 2 warpgroups x WG_COLS, a power of two

    const int tid = threadIdx.x, set = tid >> 8, wg = (tid >> 7) & 1, row = tid & 127, warp4 = (tid >> 5) & 3;
    const int wgi = set * 2 + wg;                                        // index of the warpgroup in the block
    {   // the aligned tiles must fit into what was asked for at launch
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        if (base + SETS * SET_BYTES > tc_smem(tc_raw) + dyn) {
            if (tid == 0) atomicExch(status, 4);
            return;
        }
    }
    const uint32_t sQ = base + set * SET_BYTES;                          // DB blocks, shared by the set's warpgroups
    const uint32_t sK = sQ + DB * Q_BLK + wg * WG_BYTES;                 // this warpgroup's key tile: DB blocks
    const uint32_t sV = sK + DB * KV_BLK;                                // its value tile
    const uint32_t sP = sV + DB * KV_BLK;                                // one [128][64] block

    // the head is x, the fastest index in the order blocks start: all heads of the longest tile first
    const int seq = tiles[2 * blockIdx.y], off = tiles[2 * blockIdx.y + 1];
    const int h_raw = blockIdx.x * SETS + set;
    const bool active = h_raw < nh;                  // an odd number of heads leaves the last block's second set idle
    const int h = active ? h_raw : nh - 1, kvh = h / (nh / nkv);
    const int tok0 = q_start[seq] + off;
    const int n_rows = min(TC_BM, q_start[seq + 1] - tok0);
    if (n_rows <= 0) return;      // a padding tile of a fixed-shape step (the whole block leaves before any barrier)
    const int pos0 = start_pos[seq] + off;
    const int pos_last = pos0 + n_rows - 1;
    const int* bt = block_table + (size_t)slots[seq] * max_pages;
    const int chunks = d >> 3;
    const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kt_begin = key_lo / TC_BN, kt_end = pos_last / TC_BN + 1;
    const int kv_hi = pos_last + 1;
    const size_t head_stride = (size_t)page_size * d;
    const size_t kv_stride = (size_t)nkv * head_stride;
    // this warpgroup's key tiles: kt_begin + wg, then every second one
    const int n_my = active ? (kt_end - kt_begin - wg + 1) / 2 : 0;
    auto my_kt = [&](int i) { return kt_begin + wg + 2 * i; };

    const uint32_t mbar = tc_smem(&s_mbar[wgi]);
    if (row == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(mbar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        s_dead[wgi] = 0;
    }
    if (tid < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }

    // element (row, 16-byte chunk c) of a tile made of [rows][64] blocks: chunk index xor-ed with the
    // row inside each group of eight rows (the 128-byte swizzle of the matrix descriptors)
    auto tile_addr = [](uint32_t tile, uint32_t blk_bytes, int r, int c) -> uint32_t {
        return tile + (c >> 3) * blk_bytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
    };
    // two threads of a warpgroup share a key row of a tile: one page lookup per thread and tile
    const int kv_r = row >> 1, kv_c0 = row & 1;
    auto load_kv_part = [&](int kt, int which) {               // which: 0 = keys, 1 = values
        const int key = kt * TC_BN + kv_r;
        bool ok = key >= key_lo && key < kv_hi;                 // outside: never read (its page may be gone)
        const bf16* src = pool;
        if (ok) {
            const int page = bt[key / page_size];
            ok = page >= 0;                                     // a hole in the block table: zeros, no access before the pool
            if (!ok) *status = 1;                               // and the host hears of it
            if (ok) src = pool + (((size_t)page * n_layers + layer) * 2 + which) * kv_stride + kvh * head_stride
                          + (size_t)(key % page_size) * d;
        }
        const uint32_t dst = which ? sV : sK;
        for (int c = kv_c0; c < chunks; c += 2) tc_cp16(tile_addr(dst, KV_BLK, kv_r, c), ok ? src + c * 8 : pool, ok);
    };
    if (active) {   // the tile's queries: two threads per row (rows past the portion's end are zero)
        const bool ok = row < n_rows;
        const bf16* src = q + (size_t)(tok0 + (ok ? row : 0)) * q_stride + h * d;
        for (int c = wg; c < chunks; c += 2) tc_cp16(tile_addr(sQ, Q_BLK, row, c), src + c * 8, ok);
    }
    // One key and one value buffer per warpgroup.  A buffer is refilled at the top of the round at whose
    // end it is read: K(i+1) once S(i) has completed, V(i) once O += P V of round i-1 has completed; the
    // copies land while the round's softmax runs.
    if (n_my > 0) load_kv_part(my_kt(0), 0);
    tc_cp_commit();
    tc_cp_wait<0>();                 // Q (this thread's part) and K(0) have landed
    tc_fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();                 // all of Q, both mbarriers, the TMEM address
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t t_wg = tmem + wgi * WG_COLS;                              // S at +0, O at +64
    const uint32_t t_row = t_wg + ((uint32_t)(warp4 * 32) << 16);            // this warp's 32 lanes
    const uint32_t idesc_s = tc_idesc(TC_BM, TC_BN, 0, 0);
    const uint32_t idesc_o = tc_idesc(TC_BM, d, 0, 1);
    auto issue_s = [&]() {              // S = Q K^T with the key tile in shared memory (one thread)
        const uint32_t kb = sK;
        for (int kk = 0; kk * 16 < d; ++kk) {
            const uint32_t o = (kk >> 2) * Q_BLK + (kk & 3) * 32, ob = (kk >> 2) * KV_BLK + (kk & 3) * 32;
            tc_mma(t_wg, tc_desc(sQ + o, 16, 1024), tc_desc(kb + ob, 16, 1024), idesc_s, kk > 0);
        }
    };

    float m_ref = -INFINITY, l_run = 0.f;       // reference maximum (scaled, log2 domain) and running sum
    const int pos = row < n_rows ? pos0 + row : -1;
    const int lo = window > 0 ? pos - window + 1 : 0;
    uint32_t phase = 0;
    bool alive = true;

    if (n_my > 0 && row == 0) {
        tc_fence_after_sync();
        issue_s();
        tc_commit(mbar);
    }
    // Round i of this warpgroup: wait for S(i) (and O += P V of round i-1); start the copies of K(i+1)
    // and V(i); softmax of S(i) -> P(i), moving the row's reference maximum (and rescaling its O row
    // in TMEM) only when needed; then one thread issues O += P(i) V(i) and S(i+1) together.
#ifdef TC_PROFILE
    // timing stamps of block (0,0), warpgroup 0: 5 per round, after status[16] (status must be large enough)
    unsigned long long* prof = reinterpret_cast<unsigned long long*>(status + 16);
#define TC_STAMP(k) if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0 && i < 40) { unsigned long long t_; \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); prof[i * 5 + (k)] = t_; }
#else
#define TC_STAMP(k)
#endif
    for (int i = 0; i < n_my && alive; ++i) {
        const int kt = my_kt(i);
        TC_STAMP(0)
        if (!tc_wait(mbar, phase)) { alive = false; atomicExch(&s_dead[wgi], 1); }
        TC_STAMP(1)
        phase ^= 1;
        tc_fence_after_sync();
        if (i + 1 < n_my) load_kv_part(my_kt(i + 1), 0);
        load_kv_part(kt, 1);
        tc_cp_commit();
        const bool need_mask = kt * TC_BN + TC_BN - 1 > pos || (window > 0 && kt * TC_BN < lo);
        float s[TC_BN];
        tc_ld32(t_row, s);              // S: columns 0..63 of this thread's lane
        tc_ld32(t_row + 32, s + 32);
        tc_ld_wait();
        TC_STAMP(2)
        if (need_mask) {
#pragma unroll
            for (int c = 0; c < TC_BN; ++c) {
                const int key = kt * TC_BN + c;
                if (key > pos || key < lo) s[c] = -INFINITY;
            }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one of 64
#pragma unroll
        for (int c = 0; c < TC_BN; c += 4) {
            mx4[0] = fmaxf(mx4[0], s[c]); mx4[1] = fmaxf(mx4[1], s[c + 1]);
            mx4[2] = fmaxf(mx4[2], s[c + 2]); mx4[3] = fmaxf(mx4[3], s[c + 3]);
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_new = fmaxf(m_ref, mx * scale_log2);
        // move the reference only when the maximum grew by more than 2^8 (or from "no key yet")
        const bool move = m_new > m_ref + 8.f;
        if (__any_sync(0xffffffffu, move) && i > 0) {
            // rescale this row of O in tensor memory (every lane of the warp takes part; a lane that
            // does not move multiplies by one)
            const float corr = move ? tc_exp2(m_ref - m_new) : 1.f;
#pragma unroll
            for (int cb = 0; cb < DB * 2; ++cb) {
                if (cb * 32 < d) {
                    float ov[32];
                    tc_ld32(t_row + 64 + cb * 32, ov);
                    tc_ld_wait();
#pragma unroll
                    for (int k = 0; k < 32; ++k) ov[k] *= corr;
                    tc_st32(t_row + 64 + cb * 32, ov);
                }
            }
            tc_st_wait();
            l_run *= corr;
        }
        if (move) m_ref = m_new;
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t prow = sP + row * 128;
#pragma unroll
        for (int c8 = 0; c8 < TC_BN / 8; ++c8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p0 = tc_exp2(fmaf(s[c8 * 8 + 2 * e], scale_log2, -m_use));
                const float p1 = tc_exp2(fmaf(s[c8 * 8 + 2 * e + 1], scale_log2, -m_use));
                rs4[e] += p0 + p1;
                __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                w[e] = *reinterpret_cast<uint32_t*>(&pk);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n"
                         ::"r"(prow + ((c8 ^ (row & 7)) << 4)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        }
        l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
        TC_STAMP(3)
        tc_cp_wait<0>();             // K(i+1) and V(i) are in place
        tc_fence_async_smem();
        tc_fence_before_sync();
        tc_wg_sync(wgi);
        TC_STAMP(4)
        // a thread whose wait expired takes its whole warpgroup out of the loop
        if (s_dead[wgi]) alive = false;
        if (row == 0 && alive) {
            tc_fence_after_sync();
            const uint32_t vb = sV;
            for (int jj = 0; jj < TC_BN / 16; ++jj)
                tc_mma(t_wg + 64, tc_desc(sP + jj * 32, 16, 1024), tc_desc(vb + jj * 2048, KV_BLK, 1024), idesc_o,
                       i > 0 || jj > 0);
            if (i + 1 < n_my) issue_s();
            tc_commit(mbar);
        }
    }
    if (alive && n_my > 0) {
        if (!tc_wait(mbar, phase)) { alive = false; atomicExch(&s_dead[wgi], 1); }
        tc_fence_after_sync();
    }
    tc_cp_wait<0>();
    tc_fence_before_sync();
    __syncthreads();
    {
        bool dead = false;
#pragma unroll
        for (int k = 0; k < 2 * SETS; ++k) dead |= s_dead[k] != 0;
        if (dead) {
            alive = false;
            if (tid == 0) atomicExch(status, 3);
        }
    }
    // ---- merge the two warpgroups: the second leaves (max, sum, O row) in shared memory (every product
    // has completed, so the tiles' space is free: (2 + head_dim) x 128 floats from its start)
    float* mrg = reinterpret_cast<float*>(tc_raw + (base - tc_smem(tc_raw)) + set * SET_BYTES);
    const float m_fin = n_my > 0 ? m_ref : -INFINITY;
    if (alive && active && wg == 1) {
        mrg[row] = m_fin;
        mrg[128 + row] = l_run;
#pragma unroll
        for (int cb = 0; cb < DB * 2; ++cb) {
            if (cb * 32 < d) {
                float ov[32];
                if (n_my > 0) { tc_ld32(t_row + 64 + cb * 32, ov); tc_ld_wait(); }
#pragma unroll
                for (int k = 0; k < 32; ++k) mrg[(2 + cb * 32 + k) * 128 + row] = n_my > 0 ? ov[k] : 0.f;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (alive && active && wg == 0) {   // warp-uniform: tcgen05.ld needs whole warps; only the store looks at the row
        const float m1 = mrg[row], l1 = mrg[128 + row];
        const float m = fmaxf(m_fin, m1);
        const float a0 = m_fin == -INFINITY ? 0.f : tc_exp2(m_fin - m), a1 = m1 == -INFINITY ? 0.f : tc_exp2(m1 - m);
        const float l = l_run * a0 + l1 * a1;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* orow = out + ((size_t)(tok0 + row) * nh + h) * d;
#pragma unroll
        for (int cb = 0; cb < DB * 2; ++cb) {
            if (cb * 32 < d) {
                float ov[32];
                tc_ld32(t_row + 64 + cb * 32, ov);       // warpgroup 0 always has a tile (the first one)
                tc_ld_wait();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (cb * 32 + c * 8 >= d || row >= n_rows) continue;   // head sizes that are no multiple of 32; rows past the end
                    float r[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) r[k] = (ov[c * 8 + k] * a0 + mrg[(2 + cb * 32 + c * 8 + k) * 128 + row] * a1) * inv;
                    uint4 w;
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(r[0], r[1]), p1 = __floats2bfloat162_rn(r[2], r[3]);
                    __nv_bfloat162 p2 = __floats2bfloat162_rn(r[4], r[5]), p3 = __floats2bfloat162_rn(r[6], r[7]);
                    w.x = *reinterpret_cast<uint32_t*>(&p0); w.y = *reinterpret_cast<uint32_t*>(&p1);
                    w.z = *reinterpret_cast<uint32_t*>(&p2); w.w = *reinterpret_cast<uint32_t*>(&p3);
                    *reinterpret_cast<uint4*>(orow + cb * 32 + c * 8) = w;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (tid < 32) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

static size_t tc_smem_bytes(int db) {
    // per set: Q, then per warpgroup K, V and P (reused for the merge); a kilobyte of slack to reach a
    // 1024-byte boundary
    const size_t set = (size_t)db * TC_BM * 128 + 2 * ((size_t)2 * db * TC_BN * 128 + TC_BM * 128);
    return TC_SETS * set + 1024;
}

template <int DB>
static int launch_prefill_tc(const void* q, const void* pool, void* out, const int* tiles, int n_tiles,
                             const int* q_start, const int* start_pos, const int* slots, const int* block_table,
                             int max_pages, int n_layers, int layer, int nh, int nkv, int d, int page_size,
                             float scale, int window, int q_stride, int* status, cudaStream_t s) {
    const size_t smem = tc_smem_bytes(DB);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<DB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // all of the SM's configurable memory as shared memory: otherwise the driver sizes the
        // carve-out for one block and a second block does not become resident
        e = cudaFuncSetAttribute(attention_prefill_tc_kernel<DB>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    constexpr int SETS = TC_SETS;
    dim3 grid((nh + SETS - 1) / SETS, n_tiles);
    attention_prefill_tc_kernel<DB><<<grid, SETS * TC_SET_THREADS, smem, s>>>((const bf16*)q, (const bf16*)pool, (bf16*)out,
        tiles, q_start, start_pos, slots, block_table, max_pages, n_layers, layer, nh, nkv, d, page_size,
        scale * TC_LOG2E, window, q_stride, status);
    return st_launch_status();
}

ST_EXPORT int st_attention_prefill_tc_max_head_dim() { return 128; }

// how many blocks of the kernel for head sizes <= 64 * db fit one SM (for profiles and tests)
ST_EXPORT int st_attention_prefill_tc_blocks_per_sm(int db) {
    int n = 0;
    const size_t smem = tc_smem_bytes(db);
    cudaError_t e;
    if (db == 1) {
        cudaFuncSetAttribute(attention_prefill_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(attention_prefill_tc_kernel<1>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_prefill_tc_kernel<1>, TC_SETS * TC_SET_THREADS, smem);
    } else {
        cudaFuncSetAttribute(attention_prefill_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_prefill_tc_kernel<2>, TC_SETS * TC_SET_THREADS, smem);
    }
    return e == cudaSuccess ? n : -(int)e;
}

// Same arguments as st_attention_prefill plus `status` (set to 3 if a wait for the tensor cores expired).
ST_EXPORT int st_attention_prefill_tc(const void* q, const void* pool, void* out, const int* tiles, int n_tiles,
                                      const int* q_start, const int* start_pos, const int* slots,
                                      const int* block_table, int max_pages, int n_layers, int layer, int nh,
                                      int nkv, int d, int page_size, float scale, int window, int q_stride, int* status,
                                      void* stream) {
    if (n_tiles <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || n_tiles > 65535 || !status) return ST_ERR_BAD_ARG;
    if (d <= 0 || d % 16) return ST_ERR_BAD_SIZE;
    if (d > 128) return ST_ERR_TOO_LARGE;
    if (q_stride <= 0) q_stride = nh * d;      // a dense [tokens, nh * d] query tensor
    cudaStream_t s = (cudaStream_t)stream;
    if (d <= 64)
        return launch_prefill_tc<1>(q, pool, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                    n_layers, layer, nh, nkv, d, page_size, scale, window, q_stride, status, s);
    return launch_prefill_tc<2>(q, pool, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                n_layers, layer, nh, nkv, d, page_size, scale, window, q_stride, status, s);
}
