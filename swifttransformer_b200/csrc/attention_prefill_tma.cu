// Paged, chunked causal attention for portions of prompts: tcgen05 tensor cores fed by TMA.
//
// The variant of attention_prefill_tc.cu for head sizes 64 and 128 and pages of 8, 16, 32 or 64
// positions (a tile of 64 keys is then a whole number of pages).  Same mathematics and the same
// layouts in shared and tensor memory; what differs is who does what:
//
//   * Keys and values come in by TMA: one rank-3 tensor map describes the whole cache pool as
//     [page x layer x (K|V) x kv_head][position in page][head_dim]; a box is (one page of one head,
//     64 of the head's elements) and lands in shared memory already in the 128-byte swizzle that the
//     matrix descriptors expect.  A copy announces its bytes on an mbarrier (expect_tx) and the
//     barrier completes when they have landed.  No multicast; only pages that hold a key the tile
//     may see are fetched (the others may have been given back): the rest of a tile, which is
//     masked, is filled from the tile's first live page so that it holds finite numbers.
//   * Each of the two (optionally three) warpgroups (every second or third key tile of one (query tile,
//     head), merged at the end) has two extra warps: one issues the products (its first lane), one the copies (lane j fetches
//     the number of page j of the tile after next and issues that page's copies).  Keys and values
//     are double-buffered, with a "landed" and a "free" mbarrier per buffer (the latter completed by
//     tcgen05.commit after the product that reads the buffer).  S of the next tile is issued as soon
//     as the softmax threads have read S of this one from tensor memory and runs under their
//     softmax; O += P V follows when P is written.  With one warp for both jobs that warp was the
//     bottleneck (measured: 2.3 us per tile, 1.7 with the page numbers fetched ahead).
//
// Waits are bounded; a wait that expires marks the block dead, the block's other waits end early,
// `status` gets 3, tensor memory is freed and the kernel returns.
// Reference counterparts: src/csrc/kernel/fused_context_stage_attention.cu:82-453 and
// src/csrc/kernel/xformers_attention.cu:313-393.
#include <mutex>

#include "tcgen05.cuh"
#include "tma_host.h"

// threads of a block with NWG softmax warpgroups: the softmax threads, then NWG warps that issue products and NWG
// warps that issue copies, filled up to whole warpgroups (setmaxnreg works on warpgroups)
#define TM_THREADS(NWG) (128 * (NWG) + ((NWG) == 2 ? 128 : 256))
// Registers per thread after a block of three warpgroups has redistributed them.  setmaxnreg moves registers
// inside what the block was given at launch (threads x the kernel's register count, 640 x 96), not inside the
// SM's whole file: a request beyond that waits forever.  The sum below must fit; the launcher checks it against
// the compiled kernel's register count and falls back to two warpgroups otherwise.
#define TM_REGS_SOFTMAX 136
#define TM_REGS_ISSUE 32
#define TM_REGS_AFTER(NWG) (128 * (NWG) * TM_REGS_SOFTMAX + (TM_THREADS(NWG) - 128 * (NWG)) * TM_REGS_ISSUE)
static_assert(TM_REGS_AFTER(3) <= TM_THREADS(3) * 96, "setmaxnreg asks for more registers than a block of 640 threads x 96 owns");

// bounded wait that also ends when the block has been marked dead
__device__ __forceinline__ bool tm_wait(uint32_t mbar, uint32_t parity, volatile int* dead) {
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
// named barriers of a warpgroup and the warp that issues its products (160 threads): A = "S has been read",
// B = "P has been written".  Softmax threads only arrive, the issuing warp waits.
__device__ __forceinline__ void tm_arrive(int wg, int which) {
    const int id = 2 * wg + which;
    if (id == 0) asm volatile("bar.arrive 1, 160;\n" ::: "memory");
    else if (id == 1) asm volatile("bar.arrive 2, 160;\n" ::: "memory");
    else if (id == 2) asm volatile("bar.arrive 3, 160;\n" ::: "memory");
    else if (id == 3) asm volatile("bar.arrive 4, 160;\n" ::: "memory");
    else if (id == 4) asm volatile("bar.arrive 5, 160;\n" ::: "memory");
    else asm volatile("bar.arrive 6, 160;\n" ::: "memory");
}
__device__ __forceinline__ void tm_sync(int wg, int which) {
    const int id = 2 * wg + which;
    if (id == 0) asm volatile("bar.sync 1, 160;\n" ::: "memory");
    else if (id == 1) asm volatile("bar.sync 2, 160;\n" ::: "memory");
    else if (id == 2) asm volatile("bar.sync 3, 160;\n" ::: "memory");
    else if (id == 3) asm volatile("bar.sync 4, 160;\n" ::: "memory");
    else if (id == 4) asm volatile("bar.sync 5, 160;\n" ::: "memory");
    else asm volatile("bar.sync 6, 160;\n" ::: "memory");
}

// DB: 64-wide blocks of the head dimension (head_dim == 64 DB).  NWG: softmax warpgroups (2 or 3), each with
// its own key tiles (every NWG-th one), buffers, accumulators, issuing warps and barriers.  Three of them give
// each scheduler three softmax warps to choose from instead of two; their registers come from the issuing
// warps (setmaxnreg), and tensor memory has room for three accumulators only at head size 64.
template <int DB, int NWG>
__global__ void __launch_bounds__(TM_THREADS(NWG), 1)
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q,
                             bf16* __restrict__ out, const int* __restrict__ tiles, const int* __restrict__ q_start,
                             const int* __restrict__ start_pos, const int* __restrict__ slots,
                             const int* __restrict__ block_table, int max_pages, int n_layers, int layer,
                             int nh, int nkv, int page_size, float scale_log2, int window, int q_stride, int* status) {
    extern __shared__ unsigned char tm_raw[];
    // per warpgroup: S done, O done, then "landed" for the buffers K0, K1, V0, V1, then "free" for the same four
    __shared__ __align__(8) unsigned long long s_mbar[NWG][10];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;
    constexpr int d = 64 * DB;
    constexpr uint32_t Q_BLK = TC_BM * 128, KV_BLK = TC_BN * 128;       // bytes of one [rows][64] block
    constexpr uint32_t BUF = DB * KV_BLK;                               // one key or value tile
    constexpr uint32_t WG_BYTES = 4 * BUF + Q_BLK;                      // K x2, V x2, and a [128][64] block that was P's
    constexpr int WG_COLS = 64 + 64 * DB + 32;                          // S, then O, then P (64 packed bfloat16 per row)
    constexpr uint32_t ALL_BYTES = DB * Q_BLK + NWG * WG_BYTES;
    constexpr int TMEM_COLS = NWG * WG_COLS <= 256 ? 256 : 512;
    static_assert(NWG * WG_COLS <= 512, "tensor memory has 512 columns");
    static_assert((NWG - 1) * (2 + 64 * DB) * 128 * 4 <= ALL_BYTES, "the merge reuses the tiles' space");
    constexpr int N_SOFTMAX = 128 * NWG;
    const uint32_t base = (tc_smem(tm_raw) + 1023u) & ~1023u;           // swizzled tiles start on 1024-byte boundaries

    const int tid = threadIdx.x;
    // softmax, products, copies, and (three warpgroups) two warps that only fill the last warpgroup
    const int role = tid < N_SOFTMAX ? 0 : tid < N_SOFTMAX + 32 * NWG ? 1 : tid < N_SOFTMAX + 64 * NWG ? 2 : 3;
    const bool issuer = role != 0;
    const int wg = role == 0 ? tid >> 7 : role == 1 ? (tid - N_SOFTMAX) >> 5 : role == 2 ? (tid - N_SOFTMAX - 32 * NWG) >> 5 : 0;
    const int row = tid & 127, warp4 = (tid >> 5) & 3;
    {
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        if (base + ALL_BYTES > tc_smem(tm_raw) + dyn) {
            if (tid == 0) atomicExch(status, 4);
            return;
        }
    }
    const uint32_t sQ = base;
    const uint32_t sK = sQ + DB * Q_BLK + wg * WG_BYTES;                 // two key buffers
    const uint32_t sV = sK + 2 * BUF;                                    // two value buffers

    // Blocks start in the order of their linear index, x fastest: the head is x, so that all heads of
    // the longest tile start first (the host lists the tiles longest key range first).
    const int seq = tiles[2 * blockIdx.y], off = tiles[2 * blockIdx.y + 1];
    const int h = blockIdx.x, kvh = h / (nh / nkv);
    const int tok0 = q_start[seq] + off;
    const int n_rows = min(TC_BM, q_start[seq + 1] - tok0);
    if (n_rows <= 0) return;      // a padding tile of a fixed-shape step (the whole block leaves before any barrier)
    const int pos0 = start_pos[seq] + off;
    const int pos_last = pos0 + n_rows - 1;
    const int* bt = block_table + (size_t)slots[seq] * max_pages;
    const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kt_begin = key_lo / TC_BN, kt_end = pos_last / TC_BN + 1;
    const int kv_hi = pos_last + 1;
    const int n_my = (kt_end - kt_begin - wg + NWG - 1) / NWG;           // this warpgroup's tiles: every NWG-th one
    auto my_kt = [&](int i) { return kt_begin + wg + NWG * i; };

    const uint32_t mb_s = tc_smem(&s_mbar[wg][0]), mb_o = tc_smem(&s_mbar[wg][1]);
    const uint32_t mb_full = tc_smem(&s_mbar[wg][2]), mb_free = tc_smem(&s_mbar[wg][6]);   // four each, 8 bytes apart
    if (tid == 0) {
        for (int w = 0; w < NWG; ++w)
            for (int k = 0; k < 10; ++k) tc_mbar_init(tc_smem(&s_mbar[w][k]), 1);
        tc_mbar_init_fence();
        s_dead = 0;
    }
    if (tid < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    auto tile_addr = [](uint32_t tile, uint32_t blk_bytes, int r, int c) -> uint32_t {
        return tile + (c >> 3) * blk_bytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
    };
    if (!issuer) {   // the tile's queries: NWG threads per row (rows past the portion's end are zero)
        const bool ok = row < n_rows;
        const bf16* src = q + (size_t)(tok0 + (ok ? row : 0)) * q_stride + h * d;
        for (int c = wg; c < d / 8; c += NWG) tc_cp16(tile_addr(sQ, Q_BLK, row, c), src + c * 8, ok);
        tc_cp_commit();
        tc_cp_wait<0>();
    }
    tc_fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();                 // Q, the mbarriers, the TMEM address
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t t_wg = tmem + wg * WG_COLS;                               // S at +0, O at +64
    volatile int* dead = &s_dead;
    // barrier of the whole block, by name and count so that the issuing warps and the softmax warps can meet
    // from different places in the code
    auto block_sync = [&]() { asm volatile("bar.sync 7, %0;\n" ::"n"(TM_THREADS(NWG)) : "memory"); };
    // Three warpgroups: every warp of the block is here (the only returns above are taken by the whole block).
    // The issuing warpgroups give registers back, the softmax warpgroups' request below waits until they are there.
    if (issuer && NWG == 3) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(TM_REGS_ISSUE));

    if (role == 1) {
        // ---- the warp that issues the products (its first lane; the others only keep the named barriers' count)
        const bool lead = (tid & 31) == 0;
        bool alive = true;
        const uint32_t idesc_s = tc_idesc(TC_BM, TC_BN, 0, 0);
        const uint32_t idesc_o = tc_idesc(TC_BM, d, 0, 1);
        const uint64_t dq = tc_desc(sQ, 16, 1024), dk = tc_desc(sK, 16, 1024);
        const uint64_t dv = tc_desc(sV, KV_BLK, 1024);
        // descriptors differ only in the start address (in units of 16 bytes, the low bits)
        auto issue_s = [&](int buf) {
#pragma unroll
            for (int kk = 0; kk < d / 16; ++kk)
                tc_mma(t_wg, dq + (((kk >> 2) * Q_BLK + (kk & 3) * 32) >> 4),
                       dk + ((buf * BUF + (kk >> 2) * KV_BLK + (kk & 3) * 32) >> 4), idesc_s, kk > 0);
            tc_commit(mb_s);
            tc_commit(mb_free + 8 * buf);                 // the key buffer may be refilled when S is complete
        };
        if (lead && n_my > 0) {
            if (tm_wait(mb_full, 0, dead)) {
                tc_fence_after_sync();
                issue_s(0);
            } else alive = false;
        }
        for (int i = 0; i < n_my; ++i) {
            const int b = i & 1;                              // tile i's buffers
            __syncwarp();
            tm_sync(wg, 0);          // S(i) is complete and in the softmax threads' registers
            if (lead && alive && i + 1 < n_my) {
                if (tm_wait(mb_full + 8 * (b ^ 1), ((i + 1) >> 1) & 1, dead)) {
                    tc_fence_after_sync();
                    issue_s(b ^ 1);
                } else alive = false;
            }
            __syncwarp();
            tm_sync(wg, 1);          // P(i) is written; O += P V of tile i-1 has completed
            if (lead && alive) {
                if (tm_wait(mb_full + 8 * (2 + b), (i >> 1) & 1, dead)) {
                    tc_fence_after_sync();
#pragma unroll
                    for (int jj = 0; jj < TC_BN / 16; ++jj)
                        tc_mma_ts(t_wg + 64, t_wg + 64 + 64 * DB + jj * 8, dv + ((b * BUF + jj * 2048) >> 4), idesc_o, i > 0 || jj > 0);
                    tc_commit(mb_o);
                    tc_commit(mb_free + 8 * (2 + b));     // the value buffer may be refilled
                } else alive = false;
            }
        }
        __syncwarp();
    }
    if (role == 2) {
        // ---- the warp that issues the copies.  Lane j fetches the number of page j of a key tile (one tile
        // ahead of its use, so that the load's latency is hidden) and issues that page's copies; lane 0
        // waits for the buffers to become free.
        const int lane = tid & 31;
        const bool lead = lane == 0;
        bool alive = true;                                     // kept the same in all lanes
        const int n_pg = TC_BN / page_size;                    // pages of a key tile: 1 to 8
        // This lane's page of this warpgroup's tile number i.  A page without a key this query tile may see
        // may have been given back: its part of the buffer (masked later) is filled from the tile's first
        // live page instead, so that it holds finite numbers.
        auto page_of = [&](int i) -> int {
            if (lane >= n_pg || i >= n_my) return -1;
            const int k0 = my_kt(i) * TC_BN;
            const int pg_lo = max(k0, key_lo) / page_size, pg_hi = (min(k0 + TC_BN, kv_hi) - 1) / page_size;
            return __ldg(bt + min(max(k0 / page_size + lane, pg_lo), pg_hi));
        };
        uint32_t n_fetch = 0;            // four 8-bit counters (modulo 256): copies announced on each "landed" barrier
        // keys (which = 0) or values (1) of a key tile -> buffer `buf`; `page` as page_of() gave it.  A hole in
        // the table (-1) gives a coordinate outside the tensor, for which the copy delivers zeros.
        auto fetch = [&](int page, int which, int buf) {
            const int x = which * 2 + buf;
            const uint32_t dst = sK + x * BUF, mb = mb_full + 8 * x;
            n_fetch += 1u << (8 * x);
            if (lead) tc_mbar_expect_tx(mb, BUF);
            __syncwarp();
            if (lane < n_pg) {
                const int c2 = page < 0 ? -1 : ((page * n_layers + layer) * 2 + which) * nkv + kvh;
                if (page < 0) *status = 1;       // the host hears of the hole
                const uint32_t o = (uint32_t)(lane * page_size) * 128;
#pragma unroll
                for (int b = 0; b < DB; ++b) tc_tma_load_3d(dst + b * KV_BLK + o, &kv_map, b * 64, 0, c2, mb);
            }
        };
        // lane 0 waits until the product that read the buffer last has completed; every lane gets the answer
        auto is_free = [&](int which, int buf, uint32_t parity) -> bool {
            int ok = 0;
            if (lead) ok = tm_wait(mb_free + 8 * (which * 2 + buf), parity, dead) ? 1 : 0;
            return __shfl_sync(0xffffffffu, ok, 0) != 0;
        };
        if (n_my > 0) {
            const int p0 = page_of(0), p1 = page_of(1);
            fetch(p0, 0, 0);
            if (n_my > 1) fetch(p1, 0, 1);
            fetch(p0, 1, 0);
            if (n_my > 1) fetch(p1, 1, 1);
        }
        int page_next = page_of(2);
        for (int i = 0; i + 2 < n_my && alive; ++i) {          // tile i+2 goes where tile i was
            const int b = i & 1;
            const uint32_t par = (i >> 1) & 1;
            const int page = page_next;
            page_next = page_of(i + 3);                        // used in the next round
            if (is_free(0, b, par)) fetch(page, 0, b); else alive = false;
            if (alive && is_free(1, b, par)) fetch(page, 1, b); else alive = false;
        }
        if (*dead && lead) {
            // the block is giving up: copies still in flight must land before its shared memory goes away
            for (int x = 0; x < 4; ++x) {
                const uint32_t c = (n_fetch >> (8 * x)) & 255u;
                if (c) tc_wait(mb_full + 8 * x, (c - 1) & 1);
            }
        }
        __syncwarp();
    }
    if (issuer) {
        // the issuing warps (and the warps that only fill a warpgroup) are done: they meet the softmax warps at
        // the block's three last barriers and leave
        tc_fence_before_sync();
        block_sync();
        block_sync();
        block_sync();
        return;
    }
    if (NWG == 3) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(TM_REGS_SOFTMAX));

    // ---- softmax threads: thread `row` of the warpgroup owns query row `row` = TMEM lane `row`
    const uint32_t t_row = t_wg + ((uint32_t)(warp4 * 32) << 16);
    float m_ref = -INFINITY, l_run = 0.f;       // reference maximum (scaled, log2 domain) and running sum
    bool alive = true;
    if (!issuer) {
        const int pos = row < n_rows ? pos0 + row : -1;
        const int lo = window > 0 ? pos - window + 1 : 0;
        uint32_t ph_s = 0, ph_o = 0;
#ifdef TC_PROFILE
        // timing stamps of block (0,0), thread 0: 6 per round, after status[16] (status must be large enough)
        unsigned long long* prof = reinterpret_cast<unsigned long long*>(status + 16);
#define TM_STAMP(k) if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0 && i < 40) { unsigned long long t_; \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); prof[i * 6 + (k)] = t_; }
#else
#define TM_STAMP(k)
#endif
        for (int i = 0; i < n_my; ++i) {
            const int kt = my_kt(i);
            TM_STAMP(0)
            if (alive && !tm_wait(mb_s, ph_s, dead)) alive = false;
            ph_s ^= 1;
            tc_fence_after_sync();
            TM_STAMP(1)
            float s[TC_BN];
            tc_ld32(t_row, s);              // S: columns 0..63 of this thread's lane
            tc_ld32(t_row + 32, s + 32);
            tc_ld_wait();
            tc_fence_before_sync();
            tm_arrive(wg, 0);
            TM_STAMP(2)
            const bool need_mask = kt * TC_BN + TC_BN - 1 > pos || (window > 0 && kt * TC_BN < lo);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < TC_BN; ++c) {
                    const int key = kt * TC_BN + c;
                    if (key > pos || key < lo) s[c] = -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains of three-input maxima
#pragma unroll
            for (int c = 0; c < TC_BN; c += 8) {
                mx4[0] = tc_max3(mx4[0], s[c], s[c + 1]); mx4[1] = tc_max3(mx4[1], s[c + 2], s[c + 3]);
                mx4[2] = tc_max3(mx4[2], s[c + 4], s[c + 5]); mx4[3] = tc_max3(mx4[3], s[c + 6], s[c + 7]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_new = fmaxf(m_ref, mx * scale_log2);
            // move the reference only when the maximum grew by more than 2^8 (or from "no key yet")
            const bool move = m_new > m_ref + 8.f;
            const float m_old = m_ref;
            if (move) m_ref = m_new;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // P = exp2(S - reference) as packed bfloat16, still in registers: this runs while O += P V of
            // the previous tile is still on the tensor cores
            float rs8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};      // four chains of pairwise sums
            uint32_t w[TC_BN / 2];
            const float neg_m = -m_use;
#pragma unroll
            for (int c2 = 0; c2 < TC_BN / 2; ++c2) {
                float a0, a1;
                tc_fma2(a0, a1, s[2 * c2], s[2 * c2 + 1], scale_log2, neg_m);
                const float p0 = tc_exp2(a0), p1 = tc_exp2(a1);
                tc_add2(rs8[2 * (c2 & 3)], rs8[2 * (c2 & 3) + 1], p0, p1);
                __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                w[c2] = *reinterpret_cast<uint32_t*>(&pk);
            }
            TM_STAMP(3)
            if (i > 0) {     // O += P V of tile i-1: O may be rescaled and P overwritten after it
                if (alive && !tm_wait(mb_o, ph_o, dead)) alive = false;
                ph_o ^= 1;
                tc_fence_after_sync();
            }
            if (__any_sync(0xffffffffu, move) && i > 0) {
                // rescale this row of O in tensor memory (every lane of the warp takes part; a lane that
                // does not move multiplies by one)
                const float corr = move ? tc_exp2(m_old - m_new) : 1.f;
#pragma unroll
                for (int cb = 0; cb < DB * 2; ++cb) {
                    float ov[32];
                    tc_ld32(t_row + 64 + cb * 32, ov);
                    tc_ld_wait();
#pragma unroll
                    for (int k = 0; k < 32; ++k) ov[k] *= corr;
                    tc_st32(t_row + 64 + cb * 32, ov);
                }
                tc_st_wait();
                l_run *= corr;
            }
            TM_STAMP(4)
            // P stays in tensor memory: this row's 64 packed bfloat16, the A operand of O += P V
            tc_st32(t_row + 64 + 64 * DB, reinterpret_cast<const float*>(w));
            l_run += ((rs8[0] + rs8[1]) + (rs8[2] + rs8[3])) + ((rs8[4] + rs8[5]) + (rs8[6] + rs8[7]));
            tc_st_wait();
            tc_fence_before_sync();
            tm_arrive(wg, 1);
            TM_STAMP(5)
        }
        if (n_my > 0) {
            if (alive && !tm_wait(mb_o, ph_o, dead)) alive = false;
            tc_fence_after_sync();
        }
    }
    tc_fence_before_sync();
    block_sync();
    if (s_dead) {
        alive = false;
        if (tid == 0) atomicExch(status, 3);
    }
    // ---- merge the warpgroups: all but the first leave (max, sum, O row) in shared memory (every product
    // and copy has completed, so the tiles' space is free: (2 + head_dim) x 128 floats each from its start)
    float* mrg_all = reinterpret_cast<float*>(tm_raw + (base - tc_smem(tm_raw)));
    constexpr int MRG = (2 + d) * 128;
    const float m_fin = n_my > 0 ? m_ref : -INFINITY;
    if (alive && !issuer && wg > 0) {
        float* mrg = mrg_all + (wg - 1) * MRG;
        mrg[row] = m_fin;
        mrg[128 + row] = l_run;
#pragma unroll
        for (int cb = 0; cb < DB * 2; ++cb) {
            float ov[32];
            if (n_my > 0) { tc_ld32(t_row + 64 + cb * 32, ov); tc_ld_wait(); }
#pragma unroll
            for (int k = 0; k < 32; ++k) mrg[(2 + cb * 32 + k) * 128 + row] = n_my > 0 ? ov[k] : 0.f;
        }
    }
    tc_fence_before_sync();
    block_sync();
    if (alive && !issuer && wg == 0) {   // warp-uniform: tcgen05.ld needs whole warps; only the store looks at the row
        float m = m_fin, a[NWG], l;
#pragma unroll
        for (int w = 1; w < NWG; ++w) m = fmaxf(m, mrg_all[(w - 1) * MRG + row]);
        a[0] = m_fin == -INFINITY ? 0.f : tc_exp2(m_fin - m);
        l = l_run * a[0];
#pragma unroll
        for (int w = 1; w < NWG; ++w) {
            const float mw = mrg_all[(w - 1) * MRG + row];
            a[w] = mw == -INFINITY ? 0.f : tc_exp2(mw - m);
            l += mrg_all[(w - 1) * MRG + 128 + row] * a[w];
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* orow = out + ((size_t)(tok0 + row) * nh + h) * d;
#pragma unroll
        for (int cb = 0; cb < DB * 2; ++cb) {
            float ov[32];
            tc_ld32(t_row + 64 + cb * 32, ov);       // warpgroup 0 always has a tile (the first one)
            tc_ld_wait();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (row >= n_rows) continue;
                float r[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    float v = ov[c * 8 + k] * a[0];
#pragma unroll
                    for (int w = 1; w < NWG; ++w) v += mrg_all[(w - 1) * MRG + (2 + cb * 32 + c * 8 + k) * 128 + row] * a[w];
                    r[k] = v * inv;
                }
                uint4 w;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(r[0], r[1]), p1 = __floats2bfloat162_rn(r[2], r[3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(r[4], r[5]), p3 = __floats2bfloat162_rn(r[6], r[7]);
                w.x = *reinterpret_cast<uint32_t*>(&p0); w.y = *reinterpret_cast<uint32_t*>(&p1);
                w.z = *reinterpret_cast<uint32_t*>(&p2); w.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(orow + cb * 32 + c * 8) = w;
            }
        }
    }
    tc_fence_before_sync();
    block_sync();
    if (tid < 32) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------------
static size_t tm_smem_bytes(int db, int nwg) {
    // Q, then per warpgroup two key and two value tiles and P; a kilobyte of slack to reach a 1024-byte boundary
    return (size_t)db * TC_BM * 128 + nwg * ((size_t)4 * db * TC_BN * 128 + TC_BM * 128) + 1024;
}

// Softmax warpgroups per block for head size 64: two, or three when asked for (head size 128 always runs two:
// tensor memory holds no third accumulator of that size).  Measured on 32 heads x 64, one request: three
// warpgroups take 60.9 instead of 64.2 us at 2048 tokens and 541 instead of 619 us at 8192, and a whole
// 2048-token prefill of OPT-1.3B takes 5.94 ms either way; the positions of this architecture end at 2048, so
// two stay the rule.
static int tm_wg_d64 = 2;
ST_EXPORT void st_attention_prefill_tma_warpgroups(int n) { tm_wg_d64 = n == 3 ? 3 : 2; }

template <int DB, int NWG>
static int launch_prefill_tma(const CUtensorMap& map, const void* q, void* out, const int* tiles, int n_tiles,
                              const int* q_start, const int* start_pos, const int* slots, const int* block_table,
                              int max_pages, int n_layers, int layer, int nh, int nkv, int page_size, float scale,
                              int window, int q_stride, int* status, cudaStream_t s) {
    const size_t smem = tm_smem_bytes(DB, NWG);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tma_kernel<DB, NWG>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nh, n_tiles);
    attention_prefill_tma_kernel<DB, NWG><<<grid, TM_THREADS(NWG), smem, s>>>(map, (const bf16*)q, (bf16*)out, tiles,
        q_start, start_pos, slots, block_table, max_pages, n_layers, layer, nh, nkv, page_size, scale * TC_LOG2E, window, q_stride,
        status);
    return st_launch_status();
}

// The three-warpgroup kernel may only run if the registers it asks for with setmaxnreg are within what its
// blocks own at launch (checked once against the compiled kernel).
static bool tm_three_warpgroups_fit() {
    static int fit = -1;
    if (fit < 0) {
        cudaFuncAttributes a;
        fit = cudaFuncGetAttributes(&a, attention_prefill_tma_kernel<1, 3>) == cudaSuccess &&
              (long long)a.numRegs * TM_THREADS(3) >= TM_REGS_AFTER(3) && a.numRegs >= TM_REGS_ISSUE ? 1 : 0;
    }
    return fit == 1;
}

// 1 if the TMA-fed kernel takes this head size and page size
ST_EXPORT int st_attention_prefill_tma_applies(int d, int page_size) {
    return (d == 64 || d == 128) && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

// Same arguments as st_attention_prefill_tc plus the number of pages in the pool (the tensor map covers the
// whole pool).  `status` is set to 3 if a wait expired.
ST_EXPORT int st_attention_prefill_tma(const void* q, const void* pool, long long n_pages, void* out, const int* tiles,
                                       int n_tiles, const int* q_start, const int* start_pos, const int* slots,
                                       const int* block_table, int max_pages, int n_layers, int layer, int nh,
                                       int nkv, int d, int page_size, float scale, int window, int q_stride, int* status,
                                       void* stream) {
    if (n_tiles <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || n_tiles > 65535 || n_pages <= 0 || !status) return ST_ERR_BAD_ARG;
    if (!st_attention_prefill_tma_applies(d, page_size)) return ST_ERR_BAD_SIZE;
    const long long rows = n_pages * n_layers * 2 * nkv;
    if (rows >= (1ll << 31)) return ST_ERR_TOO_LARGE;          // TMA coordinates are 32-bit
    if ((reinterpret_cast<uintptr_t>(pool) & 15) != 0) return ST_ERR_BAD_ARG;
    CUtensorMap map;
    int r = st_tma_pool_map(pool, rows, page_size, d, &map);
    if (r) return r;
    if (q_stride <= 0) q_stride = nh * d;      // a dense [tokens, nh * d] query tensor
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 64 && tm_wg_d64 == 3 && tm_three_warpgroups_fit())
        return launch_prefill_tma<1, 3>(map, q, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                        n_layers, layer, nh, nkv, page_size, scale, window, q_stride, status, s);
    if (d == 64)
        return launch_prefill_tma<1, 2>(map, q, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                        n_layers, layer, nh, nkv, page_size, scale, window, q_stride, status, s);
    return launch_prefill_tma<2, 2>(map, q, out, tiles, n_tiles, q_start, start_pos, slots, block_table, max_pages,
                                    n_layers, layer, nh, nkv, page_size, scale, window, q_stride, status, s);
}
