// Paged, chunked causal attention for portions of prompts, head size 64: the TMA-fed tcgen05 kernel of
// attention_prefill_tma.cu made persistent.
//
// attention_prefill_tma.cu runs one thread block per (tile of 128 queries, head).  A block there pays, before
// its first product and after its last, for things that overlap with nothing: a chain of dependent loads to
// find its work, the queries, the first keys, and at the end the merge of its two warpgroups and the store.
// With causal prompts most tiles are short, and at 2048 tokens x 32 heads that fixed part is 40 % of the
// kernel's time (3.5 blocks per SM, one at a time).  Here the grid is one block per SM and every block walks
// through its share of the (tile, head) pairs:
//
//   * the pairs are dealt out in rounds over the blocks, every second round backwards (the host lists the
//     tiles longest first, so every block gets a like amount of work);
//   * the warps that issue copies and products never stop at a pair's end: key and value tiles of the next
//     pair follow those of this one through the same double buffers (the barriers' phases run on), the next
//     pair's queries are already in the second query buffer, and S of its first key tile is on the tensor
//     cores while the softmax threads still merge and store this pair's result;
//   * the softmax threads of the two warpgroups (every second key tile each, as before) meet once per pair,
//     when both have read their last S: the second warpgroup then leaves (max, sum, O) in one of two merge
//     buffers and goes on, the first combines and stores;
//   * P never goes through shared memory: a softmax thread writes its row of P (64 packed bfloat16) into tensor
//     memory with tcgen05.st and O += P V takes it from there as its A operand (one instruction and a wait
//     instead of eight swizzled stores and a proxy fence: 54.0 -> 52.2 us per layer at 2048 tokens, 575 -> 537
//     at 8192; two P buffers, so that P(i) would not wait for the product of tile i - 1, were slower: 56.4).
//
// Mathematics, the layouts of Q, K and V in shared memory and of S and O in tensor memory, the bounded waits and
// their status codes are those of attention_prefill_tma.cu.  Reference counterparts: src/csrc/kernel/fused_context_stage_attention.cu:82-453
// and src/csrc/kernel/xformers_attention.cu:313-393.
#include "tcgen05.cuh"
#include "tma_host.h"

#define TP_THREADS 384                              // 256 softmax threads, 2 warps issuing products, 2 issuing copies
#define TP_D 64
#define TP_Q_BYTES (TC_BM * 128)                    // a [128][64] block of bfloat16
#define TP_KV_BYTES (TC_BN * 128)                   // a [64][64] block
#define TP_WG_BYTES (4 * TP_KV_BYTES)               // K x2, V x2
#define TP_MRG_FLOATS ((2 + TP_D) * 128)
#define TP_ALL_BYTES (2 * TP_Q_BYTES + 2 * TP_WG_BYTES + 2 * TP_MRG_FLOATS * 4)
#define TP_WG_COLS 256                              // S (64 columns), then O (64), then P (32: 64 packed bfloat16)

__device__ __forceinline__ bool tp_wait(uint32_t mbar, uint32_t parity, volatile int* dead) {
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
// Named barriers.  1-4: a warpgroup and the warp that issues its products (160 threads), A = "S has been read",
// B = "P has been written": softmax threads arrive, the issuing warp waits.  7: the whole block.  8: all softmax
// threads and both product-issuing warps, once per pair: "the next pair's queries are in place, this pair's last
// S has been read".  9 and 10 (pairs in turn): the softmax threads, "the second warpgroup's share is in the
// merge buffer".
__device__ __forceinline__ void tp_arrive(int wg, int which) {
    const int id = 2 * wg + which;
    if (id == 0) asm volatile("bar.arrive 1, 160;\n" ::: "memory");
    else if (id == 1) asm volatile("bar.arrive 2, 160;\n" ::: "memory");
    else if (id == 2) asm volatile("bar.arrive 3, 160;\n" ::: "memory");
    else asm volatile("bar.arrive 4, 160;\n" ::: "memory");
}
__device__ __forceinline__ void tp_sync(int wg, int which) {
    const int id = 2 * wg + which;
    if (id == 0) asm volatile("bar.sync 1, 160;\n" ::: "memory");
    else if (id == 1) asm volatile("bar.sync 2, 160;\n" ::: "memory");
    else if (id == 2) asm volatile("bar.sync 3, 160;\n" ::: "memory");
    else asm volatile("bar.sync 4, 160;\n" ::: "memory");
}
__device__ __forceinline__ void tp_pair_sync() { asm volatile("bar.sync 8, 320;\n" ::: "memory"); }
__device__ __forceinline__ void tp_merge_arrive(int k) {
    if (k & 1) asm volatile("bar.arrive 10, 256;\n" ::: "memory");
    else asm volatile("bar.arrive 9, 256;\n" ::: "memory");
}
__device__ __forceinline__ void tp_merge_sync(int k) {
    if (k & 1) asm volatile("bar.sync 10, 256;\n" ::: "memory");
    else asm volatile("bar.sync 9, 256;\n" ::: "memory");
}

// one (tile of queries, head) pair
struct TpPair {
    int h, kvh, tok0, n_rows, pos0, key_lo, kt_begin, kt_end, kv_hi;
    const int* bt;
};
struct TpWork {
    const int* tiles;
    const int* q_start;
    const int* start_pos;
    const int* slots;
    const int* block_table;
    int max_pages, n_tiles, nh, nkv, window, q_stride;
};
// The next pair of this block at or after round `r` (advanced past it), or false.  Round r deals pairs
// r G .. r G + G - 1 to the G blocks, forwards in even rounds, backwards in odd ones; a padding tile of a
// fixed-shape step (no rows) is passed over.  Every role of the block calls this with the same arguments and
// sees the same sequence.
__device__ __forceinline__ bool tp_next(int& r, const TpWork& w, TpPair& p) {
    const int G = gridDim.x, c = blockIdx.x;
    const long long total = (long long)w.n_tiles * w.nh;
    for (;; ++r) {
        if ((long long)r * G >= total) return false;
        const long long e = (long long)r * G + ((r & 1) ? G - 1 - c : c);
        if (e >= total) continue;
        const int ty = (int)(e / w.nh);
        const int seq = w.tiles[2 * ty], off = w.tiles[2 * ty + 1];
        const int tok0 = w.q_start[seq] + off;
        const int n_rows = min(TC_BM, w.q_start[seq + 1] - tok0);
        if (n_rows <= 0) continue;
        p.h = (int)(e - (long long)ty * w.nh);
        p.kvh = p.h / (w.nh / w.nkv);
        p.tok0 = tok0;
        p.n_rows = n_rows;
        p.pos0 = w.start_pos[seq] + off;
        const int pos_last = p.pos0 + n_rows - 1;
        p.key_lo = w.window > 0 ? max(0, p.pos0 - w.window + 1) : 0;
        p.kt_begin = p.key_lo / TC_BN;
        p.kt_end = pos_last / TC_BN + 1;
        p.kv_hi = pos_last + 1;
        p.bt = w.block_table + (size_t)w.slots[seq] * w.max_pages;
        ++r;
        return true;
    }
}
__device__ __forceinline__ int tp_tiles_of(const TpPair& p, int wg) { return (p.kt_end - p.kt_begin - wg + 1) / 2; }

__global__ void __launch_bounds__(TP_THREADS, 1)
attention_prefill_tmap_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q,
                              bf16* __restrict__ out, TpWork work, int n_layers, int layer, int page_size,
                              float scale_log2, int* status) {
    extern __shared__ unsigned char tp_raw[];
    // per warpgroup: S done, O done, then "landed" for the buffers K0, K1, V0, V1, then "free" for the same four
    __shared__ __align__(8) unsigned long long s_mbar[2][10];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;
    constexpr int d = TP_D;
    const uint32_t base = (tc_smem(tp_raw) + 1023u) & ~1023u;           // swizzled tiles start on 1024-byte boundaries
    const int tid = threadIdx.x;
    const int role = tid < 256 ? 0 : tid < 320 ? 1 : 2;                 // softmax, products, copies
    const int wg = role == 0 ? tid >> 7 : role == 1 ? (tid - 256) >> 5 : (tid - 320) >> 5;
    const int row = tid & 127, warp4 = (tid >> 5) & 3;
    {
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        if (base + TP_ALL_BYTES > tc_smem(tp_raw) + dyn) {
            if (tid == 0) atomicExch(status, 4);
            return;
        }
    }
    const uint32_t sQ = base;                                            // two query buffers
    const uint32_t sK = sQ + 2 * TP_Q_BYTES + wg * TP_WG_BYTES;          // two key buffers
    const uint32_t sV = sK + 2 * TP_KV_BYTES;                            // two value buffers
    float* mrg_all = reinterpret_cast<float*>(tp_raw + (base - tc_smem(tp_raw)) + 2 * TP_Q_BYTES + 2 * TP_WG_BYTES);
    const uint32_t mb_s = tc_smem(&s_mbar[wg][0]), mb_o = tc_smem(&s_mbar[wg][1]);
    const uint32_t mb_full = tc_smem(&s_mbar[wg][2]), mb_free = tc_smem(&s_mbar[wg][6]);   // four each, 8 bytes apart
    if (tid == 0) {
        for (int w = 0; w < 2; ++w)
            for (int k = 0; k < 10; ++k) tc_mbar_init(tc_smem(&s_mbar[w][k]), 1);
        tc_mbar_init_fence();
        s_dead = 0;
    }
    if (tid < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();                 // the mbarriers, the TMEM address
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t t_wg = tmem + wg * TP_WG_COLS;                        // S at +0, O at +64
    volatile int* dead = &s_dead;
    auto block_sync = [&]() { asm volatile("bar.sync 7, %0;\n" ::"n"(TP_THREADS) : "memory"); };
    auto tile_addr = [](uint32_t tile, int r, int c) -> uint32_t { return tile + r * 128 + (((c & 7) ^ (r & 7)) << 4); };

    int round = 0;                   // cursor into this block's pairs
    TpPair cur;
    bool have = tp_next(round, work, cur);

    if (role == 1) {
        // ---- the warp that issues the products (its first lane; the others only keep the barriers' counts)
        const bool lead = (tid & 31) == 0;
        bool alive = true;
        const uint32_t idesc_s = tc_idesc(TC_BM, TC_BN, 0, 0);
        const uint32_t idesc_o = tc_idesc(TC_BM, d, 0, 1);
        const uint64_t dk = tc_desc(sK, 16, 1024), dv = tc_desc(sV, TP_KV_BYTES, 1024);
        uint32_t g = 0;              // key tiles of this warpgroup so far, over all pairs: buffer g & 1, phase (g >> 1) & 1
        tp_pair_sync();              // the first pair's queries are in place
        for (int k = 0; have; ++k) {
            const int n_my = tp_tiles_of(cur, wg);
            const uint64_t dq = tc_desc(sQ + (k & 1) * TP_Q_BYTES, 16, 1024);
            auto issue_s = [&](int buf) {
#pragma unroll
                for (int kk = 0; kk < d / 16; ++kk)
                    tc_mma(t_wg, dq + ((kk * 32) >> 4), dk + ((buf * TP_KV_BYTES + kk * 32) >> 4), idesc_s, kk > 0);
                tc_commit(mb_s);
                tc_commit(mb_free + 8 * buf);                 // the key buffer may be refilled when S is complete
            };
            if (lead && alive && n_my > 0) {
                if (tp_wait(mb_full + 8 * (g & 1), (g >> 1) & 1, dead)) {
                    tc_fence_after_sync();
                    issue_s(g & 1);
                } else alive = false;
            }
            for (int i = 0; i < n_my; ++i) {
                const uint32_t gi = g + i;
                const int b = gi & 1;
                __syncwarp();
                tp_sync(wg, 0);          // S(i) is in the softmax threads' registers
                if (lead && alive && i + 1 < n_my) {
                    if (tp_wait(mb_full + 8 * (b ^ 1), ((gi + 1) >> 1) & 1, dead)) {
                        tc_fence_after_sync();
                        issue_s(b ^ 1);
                    } else alive = false;
                }
                __syncwarp();
                tp_sync(wg, 1);          // P(i) is written; O += P V of tile i-1 has completed
                if (lead && alive) {
                    if (tp_wait(mb_full + 8 * (2 + b), (gi >> 1) & 1, dead)) {
                        tc_fence_after_sync();
#pragma unroll
                        for (int jj = 0; jj < TC_BN / 16; ++jj)
                            tc_mma_ts(t_wg + 64, t_wg + 128 + jj * 8, dv + ((b * TP_KV_BYTES + jj * 2048) >> 4), idesc_o,
                                      i > 0 || jj > 0);
                        tc_commit(mb_o);
                        tc_commit(mb_free + 8 * (2 + b));     // the value buffer may be refilled
                    } else alive = false;
                }
            }
            g += n_my;
            have = tp_next(round, work, cur);
            __syncwarp();
            tp_pair_sync();          // the next pair's queries are in place (after the last pair: only the count)
        }
        __syncwarp();
    } else if (role == 2) {
        // ---- the warp that issues the copies.  Lane j looks up page j of a key tile and issues that page's copies;
        // lane 0 waits for the buffers to become free.  It runs ahead of everybody else, across pairs.
        const int lane = tid & 31;
        const bool lead = lane == 0;
        bool alive = true;                                     // kept the same in all lanes
        const int n_pg = TC_BN / page_size;                    // pages of a key tile: 1 to 8
        uint32_t n_fetch[4] = {0, 0, 0, 0};                    // copies announced on each "landed" barrier
        uint32_t g = 0;
        for (; have && alive; have = tp_next(round, work, cur)) {
            const int n_my = tp_tiles_of(cur, wg);
            // This lane's page of this warpgroup's tile i.  A page without a key this query tile may see may have
            // been given back: its part of the buffer (masked later) is filled from the tile's first live page
            // instead, so that it holds finite numbers.
            auto page_of = [&](int i) -> int {
                if (lane >= n_pg || i >= n_my) return -1;
                const int k0 = (cur.kt_begin + wg + 2 * i) * TC_BN;
                const int pg_lo = max(k0, cur.key_lo) / page_size, pg_hi = (min(k0 + TC_BN, cur.kv_hi) - 1) / page_size;
                return __ldg(cur.bt + min(max(k0 / page_size + lane, pg_lo), pg_hi));
            };
            int page_next = page_of(0);
            for (int i = 0; i < n_my && alive; ++i) {
                const uint32_t gi = g + i;
                const int b = gi & 1;
                const int page = page_next;
                page_next = page_of(i + 1);                    // its latency passes under this tile's waits
                for (int which = 0; which < 2 && alive; ++which) {
                    const int x = which * 2 + b;
                    if (gi >= 2) {                             // the product that read the buffer last has completed
                        int ok = 0;
                        if (lead) ok = tp_wait(mb_free + 8 * x, ((gi - 2) >> 1) & 1, dead) ? 1 : 0;
                        if (!__shfl_sync(0xffffffffu, ok, 0)) { alive = false; break; }
                    }
                    const uint32_t dst = sK + x * TP_KV_BYTES, mb = mb_full + 8 * x;
                    ++n_fetch[x];
                    if (lead) tc_mbar_expect_tx(mb, TP_KV_BYTES);
                    __syncwarp();
                    if (lane < n_pg) {
                        // a hole in the table (-1) gives a coordinate outside the tensor: the copy delivers zeros
                        const int c2 = page < 0 ? -1 : ((page * n_layers + layer) * 2 + which) * work.nkv + cur.kvh;
                        if (page < 0) *status = 1;             // and the host hears of it
                        tc_tma_load_3d(dst + (uint32_t)(lane * page_size) * 128, &kv_map, 0, 0, c2, mb);
                    }
                }
            }
            g += n_my;
        }
        if (*dead && lead) {
            // the block is giving up: copies still in flight must land before its shared memory goes away
            for (int x = 0; x < 4; ++x)
                if (n_fetch[x]) tc_wait(mb_full + 8 * x, (n_fetch[x] - 1) & 1);
        }
        __syncwarp();
    } else {
        // ---- softmax threads: thread `row` of the warpgroup owns query row `row` = TMEM lane `row`
        const uint32_t t_row = t_wg + ((uint32_t)(warp4 * 32) << 16);
        bool alive = true;
        uint32_t ph_s = 0, ph_o = 0;                   // phases of "S done" and "O done": they run on over the pairs
        // the tile's queries: two threads per row (one per warpgroup), every second 16-byte piece each; rows past
        // the portion's end are zero
        auto load_q = [&](const TpPair& p, int buf) {
            const bool ok = row < p.n_rows;
            const bf16* src = q + (size_t)(p.tok0 + (ok ? row : 0)) * work.q_stride + p.h * d;
            for (int c = wg; c < d / 8; c += 2) tc_cp16(tile_addr(sQ + buf * TP_Q_BYTES, row, c), src + c * 8, ok);
        };
        TpPair nxt;
        bool have_nxt = false;
        if (have) {
            load_q(cur, 0);
            tc_cp_commit();
            have_nxt = tp_next(round, work, nxt);
            if (have_nxt) load_q(nxt, 1);
        }
        tc_cp_commit();
        tc_cp_wait<1>();                               // this thread's pieces of the first pair's queries have landed
        tc_fence_async_smem();
        tp_pair_sync();
        for (int k = 0; have; ++k) {
            const int n_my = tp_tiles_of(cur, wg);
            const int pos = row < cur.n_rows ? cur.pos0 + row : -1;
            const int lo = work.window > 0 ? pos - work.window + 1 : 0;
            float m_ref = -INFINITY, l_run = 0.f;      // reference maximum (scaled, log2 domain) and running sum
            for (int i = 0; i < n_my; ++i) {
                const int kt = cur.kt_begin + wg + 2 * i;
                if (alive && !tp_wait(mb_s, ph_s, dead)) alive = false;
                ph_s ^= 1;
                tc_fence_after_sync();
                float s[TC_BN];
                tc_ld32(t_row, s);              // S: columns 0..63 of this thread's lane
                tc_ld32(t_row + 32, s + 32);
                tc_ld_wait();
                tc_fence_before_sync();
                tp_arrive(wg, 0);
                const bool need_mask = kt * TC_BN + TC_BN - 1 > pos || (work.window > 0 && kt * TC_BN < lo);
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
                if (i > 0) {     // O += P V of tile i-1: O may be rescaled and P overwritten after it
                    if (alive && !tp_wait(mb_o, ph_o, dead)) alive = false;
                    ph_o ^= 1;
                    tc_fence_after_sync();
                }
                if (__any_sync(0xffffffffu, move) && i > 0) {
                    // rescale this row of O in tensor memory (every lane of the warp takes part; a lane that
                    // does not move multiplies by one)
                    const float corr = move ? tc_exp2(m_old - m_new) : 1.f;
#pragma unroll
                    for (int cb = 0; cb < 2; ++cb) {
                        float ov[32];
                        tc_ld32(t_row + 64 + cb * 32, ov);
                        tc_ld_wait();
#pragma unroll
                        for (int kk = 0; kk < 32; ++kk) ov[kk] *= corr;
                        tc_st32(t_row + 64 + cb * 32, ov);
                    }
                    tc_st_wait();
                    l_run *= corr;
                }
                tc_st32(t_row + 128, reinterpret_cast<const float*>(w));     // P: this row's 64 packed bfloat16 into tensor memory
                l_run += ((rs8[0] + rs8[1]) + (rs8[2] + rs8[3])) + ((rs8[4] + rs8[5]) + (rs8[6] + rs8[7]));
                tc_st_wait();
                tc_fence_before_sync();
                tp_arrive(wg, 1);
            }
            // Both warpgroups have read their last S of this pair and the next pair's queries (asked for a pair
            // ago) have landed: the tensor cores may go on with the next pair while this one is merged and stored.
            tc_cp_wait<0>();
            tc_fence_async_smem();
            tc_fence_before_sync();
            tp_pair_sync();
            if (n_my > 0) {
                if (alive && !tp_wait(mb_o, ph_o, dead)) alive = false;
                ph_o ^= 1;
                tc_fence_after_sync();
            }
            // ---- merge: the second warpgroup leaves (max, sum, O row) in this pair's merge buffer
            const float m_fin = n_my > 0 ? m_ref : -INFINITY;
            float* mrg = mrg_all + (k & 1) * TP_MRG_FLOATS;
            if (wg == 1) {
                mrg[row] = m_fin;
                mrg[128 + row] = l_run;
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                    float ov[32];
                    if (n_my > 0) { tc_ld32(t_row + 64 + cb * 32, ov); tc_ld_wait(); }
#pragma unroll
                    for (int kk = 0; kk < 32; ++kk) mrg[(2 + cb * 32 + kk) * 128 + row] = n_my > 0 ? ov[kk] : 0.f;
                }
                tc_fence_before_sync();
                __threadfence_block();
                tp_merge_arrive(k);
            } else {
                tp_merge_sync(k);
                const float mw = mrg[row];
                const float m = fmaxf(m_fin, mw);
                const float a0 = m_fin == -INFINITY ? 0.f : tc_exp2(m_fin - m);
                const float a1 = mw == -INFINITY ? 0.f : tc_exp2(mw - m);
                const float l = l_run * a0 + mrg[128 + row] * a1;
                const float inv = l > 0.f ? 1.f / l : 0.f;
                bf16* orow = out + ((size_t)(cur.tok0 + row) * work.nh + cur.h) * d;
#pragma unroll
                for (int cb = 0; cb < 2; ++cb) {
                    float ov[32];
                    tc_ld32(t_row + 64 + cb * 32, ov);       // the first warpgroup always has a tile (the first one)
                    tc_ld_wait();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if (row >= cur.n_rows || !alive) continue;
                        float r[8];
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk)
                            r[kk] = (ov[c * 8 + kk] * a0 + mrg[(2 + cb * 32 + c * 8 + kk) * 128 + row] * a1) * inv;
                        uint4 v;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(r[0], r[1]), p1 = __floats2bfloat162_rn(r[2], r[3]);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(r[4], r[5]), p3 = __floats2bfloat162_rn(r[6], r[7]);
                        v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                        v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                        *reinterpret_cast<uint4*>(orow + cb * 32 + c * 8) = v;
                    }
                }
                tc_fence_before_sync();
            }
            // ---- on to the next pair; the queries of the pair after it go where this pair's were
            cur = nxt;
            have = have_nxt;
            have_nxt = have && tp_next(round, work, nxt);
            if (have_nxt) load_q(nxt, k & 1);
            tc_cp_commit();
        }
    }
    tc_fence_before_sync();
    block_sync();
    if (s_dead && tid == 0) atomicExch(status, 3);
    if (tid < 32) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------------------
// 1 if the persistent kernel takes this head size and page size
ST_EXPORT int st_attention_prefill_tmap_applies(int d, int page_size) {
    return d == TP_D && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

// Same arguments as st_attention_prefill_tma (q_stride: elements between the query rows of consecutive tokens;
// 0: nh * d, a dense [tokens, nh * d] tensor).  `status` is set to 3 if a wait expired, to 1 if a key range
// crosses a hole in a block table.
ST_EXPORT int st_attention_prefill_tmap(const void* q, const void* pool, long long n_pages, void* out, const int* tiles,
                                        int n_tiles, const int* q_start, const int* start_pos, const int* slots,
                                        const int* block_table, int max_pages, int n_layers, int layer, int nh,
                                        int nkv, int d, int page_size, float scale, int window, int q_stride, int* status,
                                        void* stream) {
    if (n_tiles <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || n_pages <= 0 || !status) return ST_ERR_BAD_ARG;
    if (!st_attention_prefill_tmap_applies(d, page_size)) return ST_ERR_BAD_SIZE;
    const long long rows = n_pages * n_layers * 2 * nkv;
    if (rows >= (1ll << 31)) return ST_ERR_TOO_LARGE;          // TMA coordinates are 32-bit
    if ((reinterpret_cast<uintptr_t>(pool) & 15) != 0 || (reinterpret_cast<uintptr_t>(q) & 15) != 0) return ST_ERR_BAD_ARG;
    CUtensorMap map;
    int r = st_tma_pool_map(pool, rows, page_size, d, &map);
    if (r) return r;
    const size_t smem = TP_ALL_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tmap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    TpWork work;
    work.tiles = tiles; work.q_start = q_start; work.start_pos = start_pos; work.slots = slots;
    work.block_table = block_table; work.max_pages = max_pages; work.n_tiles = n_tiles; work.nh = nh; work.nkv = nkv;
    work.window = window;
    work.q_stride = q_stride > 0 ? q_stride : nh * d;
    const long long total = (long long)n_tiles * nh;
    const int sms = st_sm_count();
    const int grid = (int)(total < sms ? total : sms);
    attention_prefill_tmap_kernel<<<grid, TP_THREADS, smem, (cudaStream_t)stream>>>(
        map, (const bf16*)q, (bf16*)out, work, n_layers, layer, page_size, scale * TC_LOG2E, status);
    return st_launch_status();
}
