// Paged attention for queries that stand alone (decode tokens and very short portions) on the
// warp-level tensor cores, bfloat16 storage, head sizes that are multiples of 16 up to 128.
//
// The lane-per-element kernel (attention_decode.cu) spends about as many issue slots as memory
// cycles: every 16 bytes of a key or value cost eight conversions and eight multiply-adds.  Here
// the arithmetic is a handful of m16n8k16 products per 16 keys and the kernel is back to being a
// copy loop:
//
//   * One thread block per (query token, kv head, split of the key range) and up to 8 query heads that
//     share the kv head (one for multi-head attention, the group for grouped-query attention).  The
//     products are taken transposed: S^T = K Q^T with the 16 KEYS of a group as the 16-row operand and
//     the heads as the 8 columns, O^T += V^T P^T with 16 head dimensions as the rows: four products per
//     16 keys for each of the two instead of eight, two exponentials per lane and head pair instead of
//     eight per lane, half the accumulator registers.  (With the heads as the 16 rows, fifteen of which
//     are empty in multi-head attention, the kernel spent as many issue slots as memory cycles.)
//   * Each of the block's warps (four, or eight when the launch has few and long blocks: the chain of
//     groups a warp works through is then half as long) runs its own pipeline, without block-wide barriers: it takes
//     every fourth (eighth) group of 16 keys, gathers their key and value rows page by page with 16-byte
//     asynchronous copies into its own ring of shared-memory stages (xor-swizzled rows), and while
//     later groups are in flight computes S = Q K^T (ldmatrix + mma.sync), the online softmax in
//     float, and O += P V (ldmatrix.trans + mma.sync) for the oldest one.
//   * The warps' (max, sum, O) are merged through shared memory; with several splits the
//     block leaves its result in `partial` and the split that arrives last merges them, in split
//     order (same protocol and layout as attention_decode.cu).
//
//   * Optionally the kernel takes the q|k|v product as the library left it (rows of q, k and v features, bias
//     included) instead of queries: it reads its queries from there, copies the keys and values of this step's own
//     tokens from those rows into its shared-memory stages (asynchronously, like rows of the cache), and once its own
//     token's rows have landed writes them from there into their page.  A decode step of more tokens than the
//     weight-streaming product serves then has no separate cache-write kernel.
//
// Rows of a group past the end of the key range are zero-filled, never read, and masked.
// Same mathematics as src/csrc/kernel/fused_decoding_stage_attention_mha.cu:159-318 in the
// reference (scalar arithmetic there, one warp per head).
#include "mma_sync.cuh"

#define DM_KEYS 16               // keys per group: the k extent of P V and two n-tiles of S
#define DM_LOG2E 1.4426950408889634f

// stages of a warp's ring.  Few: 50 / 68 KB per block of four warps, so that several blocks share an SM.  DEEP: when the
// launch has no more blocks than the GPU has SMs a block may take the SM's shared memory for itself, and a warp asks
// for up to five groups of keys before the wait for the kernel before this one: a decode step of one to four
// requests then finds nearly all of its keys in shared memory when its queries arrive, instead of fetching three
// of a warp's five groups one after the other behind them (3.5 us per layer at batch 1).
template <int DMAX, bool DEEP> struct DmStages { static constexpr int value = DEEP ? 6 : (DMAX == 64 ? 3 : 2); };

// The q|k|v form: `q` is the product [tokens, (nh + 2 nkv) d] (q features, then k, then v; bias included),
// `q_stride` the elements of one of its rows.  Keys from the request's `start_pos` on are this step's: the token at
// position p of the request is row t - (pos - p) (a request's tokens of a step are consecutive rows in the order of
// their positions).  on == 0: `q` holds queries only, [tokens, nh d], and every key is in the cache.
struct DmQkv {
    int q_stride, num_pages, write_kv, on;       // on: host side only (which variant is launched)
};

// head_dim <= DMAX, a multiple of 16; FULL: head_dim == DMAX, known when compiling (no tests on it in the loops)
// QKV: the q|k|v form (a variant of its own, so that the plain form keeps its registers)
template <int DMAX, bool FULL, int DM_WARPS, bool DEEP, bool QKV>
__global__ void __launch_bounds__(DM_WARPS * 32, QKV ? (DM_WARPS == 4 ? (DMAX == 64 ? 4 : 3) : (DMAX == 64 ? 2 : 1)) : 0)
attention_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, bf16* __restrict__ out,
                            float* __restrict__ partial, const int* __restrict__ items,
                            const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ slots, const int* __restrict__ start_pos,
                            const int* __restrict__ block_table, int max_pages,
                            int n_layers, int layer, int nh, int nkv, int d_arg, int page_size, int page_shift,
                            float scale_log2, int window, int n_splits, int* __restrict__ counters,
                            int* __restrict__ status, DmQkv qkv) {
    const int d = FULL ? DMAX : d_arg;
    // page_shift: log2(page_size) if that is a power of two, else -1
    constexpr int STAGES = DmStages<DMAX, DEEP>::value;
    constexpr int DM_THREADS = DM_WARPS * 32;
    constexpr int STAGE_ELEMS = 2 * DM_KEYS * DMAX;              // keys, then values, of one group
    extern __shared__ __align__(128) unsigned char dm_raw[];
    bf16* sKV = reinterpret_cast<bf16*>(dm_raw);                 // [DM_WARPS][STAGES][2][DM_KEYS][DMAX]
    int* s_pages = reinterpret_cast<int*>(sKV + DM_WARPS * STAGES * STAGE_ELEMS);
    __shared__ float s_m[DM_WARPS][8], s_l[DM_WARPS][8];
    __shared__ int s_last;
    ST_PDL_TRIGGER();
    // Which token, where it stands, its slot and the page numbers of its key range are inputs of the step
    // that no kernel of the step writes: this chain of dependent loads runs before the wait for the kernel
    // before this one, under that kernel's tail.  The queries and this step's keys and values come after.
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0) return;            // a padding entry of a fixed-shape step
    const int group = nh / nkv;                                   // query heads per kv head
    const int chunks_per_kv = (group + 7) / 8;
    const int kvh = blockIdx.y / chunks_per_kv;
    const int h0 = kvh * group + (blockIdx.y % chunks_per_kv) * 8;    // first query head of this block
    const int n_heads = min(8, kvh * group + group - h0);
    const int split = blockIdx.z;
    const int pos = positions[t];
    if (pos < 0) return;   // padding entry of a fixed-shape launch
    const int seq = seq_of_token[t];
    const int slot = slots[seq];
    // keys below this position were written by earlier steps: they may be read before the wait for the
    // kernel before this one (which writes this step's keys and values); null: none may
    const int old_hi = start_pos ? start_pos[seq] : 0;
    const int new_lo = QKV ? old_hi : 0x7fffffff;          // keys from here on come from the q|k|v rows of this step
    const int* bt = block_table + (size_t)slot * max_pages;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int hi = pos + 1;
    int per = (hi - lo + n_splits - 1) / n_splits;
    per = (per + 15) / 16 * 16;
    const int k_lo = lo + split * per;
    const int k_hi = min(hi, k_lo + per);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = d >> 3;

    // the page numbers of this block's key range and the queries, fetched once
    const int p_lo = k_lo / page_size;
    if (k_lo < k_hi) {
        const int n_pages = (k_hi - 1) / page_size - p_lo + 1;
        for (int i = threadIdx.x; i < n_pages; i += DM_THREADS) {
            const int page = __ldcg(bt + p_lo + i);
            s_pages[i] = page;
            if (page < 0 && status) *status = 1;     // a hole in the block table: zeros are read for it and the host hears of it
        }
    }
    __syncthreads();          // the page numbers are in place for every warp

    const size_t head_stride = (size_t)page_size * d;
    const size_t kv_stride = (size_t)nkv * head_stride;
    const size_t page_stride = (size_t)n_layers * 2 * kv_stride;
    const bf16* kbase = pool + (size_t)layer * 2 * kv_stride + kvh * head_stride;   // this layer's and head's keys in page 0

    // this warp's groups of 16 keys: warp, warp + 4, ... of the block's range
    const int n_groups = k_lo < k_hi ? (k_hi - k_lo + DM_KEYS - 1) / DM_KEYS : 0;
    const int my_n = (n_groups - warp + DM_WARPS - 1) / DM_WARPS;
    // shared-memory addresses of this warp's stages and, per lane, the offsets its ldmatrix and copy
    // instructions use inside a stage: nothing of this is recomputed per group
    const uint32_t my_stages = smem_u32(sKV + warp * STAGES * STAGE_ELEMS);
    constexpr uint32_t STAGE_BYTES = STAGE_ELEMS * sizeof(bf16), V_BYTES = DM_KEYS * DMAX * sizeof(bf16);
    // keys as the row operand of S^T (plain ldmatrix: matrices = keys 0-7 | 8-15 x dims 16 kk + 0-7 | 8-15) and
    // values as the row operand of O^T (transposing ldmatrix: matrices = keys 0-7 | 8-15 x dims 16 mt + 0-7 | 8-15,
    // in the order the fragment wants its rows = dims)
    uint32_t k_off[DMAX / 16], v_off[DMAX / 16];
#pragma unroll
    for (int kk = 0; kk < DMAX / 16; ++kk) {
        k_off[kk] = (uint32_t)(tile_ptr<DMAX>(sKV, (lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4)) - sKV) * 2;
        v_off[kk] = V_BYTES + (uint32_t)(tile_ptr<DMAX>(sKV, (lane & 7) + (lane >> 4) * 8, 2 * kk + ((lane >> 3) & 1)) - sKV) * 2;
    }
    // Consecutive lanes copy consecutive 16-byte chunks of a row (whole 128-byte lines per instruction).
    // Which (row of the group, chunk) a lane copies in its j-th turn does not depend on the group: worked
    // out once, with the shared-memory offset (-1: no such turn for this head size).
    constexpr int TURNS = DM_KEYS * (DMAX / 8) / 32;
    int ld_row[TURNS], ld_col[TURNS];
    uint32_t ld_off[TURNS];
#pragma unroll
    for (int j = 0; j < TURNS; ++j) {
        const int idx = lane + 32 * j;
        const int r = idx / chunks, c = idx - r * chunks;
        ld_row[j] = r < DM_KEYS ? r : -1;
        ld_col[j] = c * 8;
        ld_off[j] = r < DM_KEYS ? (uint32_t)(tile_ptr<DMAX>(sKV, r, c) - sKV) * 2 : 0;
    }
    // When pages hold a multiple of 16 positions and the range starts on such a multiple, the 16 keys of a
    // group lie in one page: one page lookup per group instead of one per copied row.
    const bool one_page = page_size % DM_KEYS == 0 && k_lo % DM_KEYS == 0;
    auto load_group = [&](int i, int stage) {
        const uint32_t dk = my_stages + stage * STAGE_BYTES;
        const int key0 = k_lo + (warp + i * DM_WARPS) * DM_KEYS;
        if (one_page && (!QKV || key0 + DM_KEYS <= new_lo)) {
            const int pg = page_shift >= 0 ? key0 >> page_shift : key0 / page_size;
            const int page = s_pages[pg - p_lo];
            const bool page_ok = page >= 0;      // a hole in the block table: zeros instead of an access before the pool
            const bf16* base = kbase + (size_t)(page_ok ? page : 0) * page_stride + (key0 - pg * page_size) * d;
#pragma unroll
            for (int j = 0; j < TURNS; ++j) {
                if (ld_row[j] < 0) continue;
                const bool ok = page_ok && key0 + ld_row[j] < k_hi;
                const bf16* src = base + ld_row[j] * d + ld_col[j];
                cp_async16_s(dk + ld_off[j], ok ? src : pool, ok);
                cp_async16_s(dk + V_BYTES + ld_off[j], ok ? src + kv_stride : pool, ok);
            }
            return;
        }
#pragma unroll
        for (int j = 0; j < TURNS; ++j) {
            if (ld_row[j] < 0) continue;
            const int key = key0 + ld_row[j];
            bool ok = key < k_hi;
            const bf16 *src = pool, *vsrc = pool;
            if (QKV && ok && key >= new_lo) {    // a key of this step: from its token's row of the product
                src = q + (size_t)(t - (pos - key)) * qkv.q_stride + (size_t)(nh + kvh) * d + ld_col[j];
                vsrc = src + (size_t)nkv * d;
            } else if (ok) {
                const int pg = page_shift >= 0 ? key >> page_shift : key / page_size;
                const int page = s_pages[pg - p_lo];
                ok = page >= 0;                  // a hole in the block table: zeros instead of an access before the pool
                if (ok) {
                    src = kbase + (size_t)page * page_stride + (key - pg * page_size) * d + ld_col[j];
                    vsrc = src + kv_stride;
                }
            }
            cp_async16_s(dk + ld_off[j], src, ok);
            cp_async16_s(dk + V_BYTES + ld_off[j], vsrc, ok);
        }
    };
    // The first stages: groups whose keys all lie below old_hi were written by earlier steps and are asked
    // for now, under the tail of the kernel before this one; the rest, and the queries, after the wait.
    int early = 0;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (early == s && s < my_n && k_lo + (warp + s * DM_WARPS + 1) * DM_KEYS <= old_hi) {
            load_group(s, s);
            cp_async_commit();
            ++early;
        }
    }
    ST_PDL_WAIT();
    // the queries as the column operand of S^T: lane (g, t) holds dims 2t, 2t+1 (and +8) of head g for every
    // block of 16 dims, straight from global memory (one trip, no staging)
    const int g = lane >> 2, t4 = lane & 3;
    uint32_t qb[DMAX / 16][2];
    {
        const size_t feat = (size_t)(h0 + min(g, n_heads - 1)) * d + 2 * t4;
        const bf16* qrow = q + (size_t)t * (QKV ? qkv.q_stride : nh * d) + feat;
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            qb[kk][0] = qb[kk][1] = 0u;
            if (kk * 16 < d && g < n_heads) {
                qb[kk][0] = __ldcg(reinterpret_cast<const unsigned*>(qrow + kk * 16));
                qb[kk][1] = __ldcg(reinterpret_cast<const unsigned*>(qrow + kk * 16 + 8));
            }
        }
    }
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s >= early) {
            if (s < my_n) load_group(s, s);
            cp_async_commit();
        }
    }
    // O^T: rows = dims (16 per tile), columns = heads: lane (g, t) holds dims 16 mt + g (and + 8) of heads 2t, 2t+1
    float o_acc[DMAX / 16][4];
#pragma unroll
    for (int i = 0; i < DMAX / 16; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // heads 2t and 2t+1 (the same in every g)
    // where this lane's P operand comes from: keys 2t, 2t+1 (and + 8) of head g lie in lanes (2t, g/2) and (2t+1, g/2)
    const int src_a = (2 * t4) * 4 + (g >> 1), src_b = (2 * t4 + 1) * 4 + (g >> 1);
    const bool odd_head = g & 1;

    for (int i = 0; i < my_n; ++i) {
        if (i + STAGES - 1 < my_n) load_group(i + STAGES - 1, (i + STAGES - 1) % STAGES);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();       // group i has landed (for this lane; the barrier covers the others)
        __syncwarp();
        const uint32_t st = my_stages + (i % STAGES) * STAGE_BYTES;
        // S^T = K Q^T: 16 keys x 8 heads; lane (g, t): keys g and g + 8 of heads 2t, 2t+1
        float s_acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            if (kk * 16 < d) {
                uint32_t a[4];
                ldmatrix_x4_s(a[0], a[1], a[2], a[3], st + k_off[kk]);
                mma_bf16(s_acc, a, qb[kk][0], qb[kk][1]);
            }
        }
        const int key0 = k_lo + (warp + i * DM_WARPS) * DM_KEYS;
        if constexpr (QKV) {
            // this block's own token's key and value rows have landed with this group: from the stage into their page
            if (pos >= key0 && pos < key0 + DM_KEYS && qkv.write_kv && blockIdx.y % chunks_per_kv == 0) {
                const int pg = page_shift >= 0 ? pos >> page_shift : pos / page_size;
                const int page = s_pages[pg - p_lo];
                if (page < 0 || page >= qkv.num_pages) {
                    if (status) *status = 1;
                } else if (lane < 2 * chunks) {
                    const int kv = lane >= chunks, c = lane - kv * chunks, r = pos - key0;
                    const uint4 v = *reinterpret_cast<const uint4*>(
                        tile_ptr<DMAX>(sKV + (size_t)(warp * STAGES + i % STAGES) * STAGE_ELEMS + kv * DM_KEYS * DMAX, r, c));
                    bf16* dst = const_cast<bf16*>(kbase) + (size_t)page * page_stride + kv * kv_stride + (pos - pg * page_size) * d + c * 8;
                    *reinterpret_cast<uint4*>(dst) = v;
                }
            }
        }
        if (key0 + DM_KEYS > k_hi) {       // the range's last group: keys past its end do not count
            if (key0 + g >= k_hi) s_acc[0] = s_acc[1] = -INFINITY;
            if (key0 + g + 8 >= k_hi) s_acc[2] = s_acc[3] = -INFINITY;
        }
        // The reference maximum of a head only moves when the true maximum has grown by more than 2^8 (or
        // from "no key yet"): until then P is taken relative to the older reference, which is exact after
        // the final division by the sum, and O and the sum need no rescaling.
        float mx[2] = {fmaxf(s_acc[0], s_acc[2]), fmaxf(s_acc[1], s_acc[3])};
        float corr[2] = {1.f, 1.f}, m_use[2];
        bool moved = false;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 4));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 8));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
            const float m_new = fmaxf(m_run[r], mx[r] * scale_log2);   // scale > 0: max commutes with it
            if (m_new > m_run[r] + 8.f) {
                corr[r] = fast_exp2(m_run[r] - m_new);                // m_run = -inf: 0
                m_run[r] = m_new;
                moved = true;
            }
            m_use[r] = (m_run[r] == -INFINITY) ? 0.f : m_run[r];
        }
        moved = __any_sync(0xffffffffu, moved);
        const float p0 = fast_exp2(fmaf(s_acc[0], scale_log2, -m_use[0])), p1 = fast_exp2(fmaf(s_acc[1], scale_log2, -m_use[1]));
        const float p2 = fast_exp2(fmaf(s_acc[2], scale_log2, -m_use[0])), p3 = fast_exp2(fmaf(s_acc[3], scale_log2, -m_use[1]));
        float rs[2] = {p0 + p2, p1 + p3};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 4);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 8);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 16);
            l_run[r] = l_run[r] * corr[r] + rs[r];
        }
        // P^T as the column operand of O^T: (key g | key g + 8) of each of this lane's heads packed, fetched by the
        // lane that needs keys 2t, 2t+1 of head g, and re-paired by key
        const uint32_t x_even = pack_bf16(p0, p2), x_odd = pack_bf16(p1, p3);
        const uint32_t ae = __shfl_sync(0xffffffffu, x_even, src_a), ao = __shfl_sync(0xffffffffu, x_odd, src_a);
        const uint32_t be = __shfl_sync(0xffffffffu, x_even, src_b), bo = __shfl_sync(0xffffffffu, x_odd, src_b);
        const uint32_t xa = odd_head ? ao : ae, xb = odd_head ? bo : be;
        const uint32_t pb0 = __byte_perm(xa, xb, 0x5410), pb1 = __byte_perm(xa, xb, 0x7632);
        // O^T = O^T corr + V^T P^T
#pragma unroll
        for (int mt = 0; mt < DMAX / 16; ++mt) {
            if (mt * 16 < d) {
                if (moved) {
                    o_acc[mt][0] *= corr[0]; o_acc[mt][1] *= corr[1];
                    o_acc[mt][2] *= corr[0]; o_acc[mt][3] *= corr[1];
                }
                uint32_t a[4];
                ldmatrix_x4_trans_s(a[0], a[1], a[2], a[3], st + v_off[mt]);
                mma_bf16(o_acc[mt], a, pb0, pb1);
            }
        }
        __syncwarp();                      // every lane is done with the stage before it is refilled
    }
    cp_async_wait<0>();
    __syncthreads();                       // all warps are done with their stages: the space is reused

    // ---- merge the warps: each leaves (max, sum, O) of its 8 heads in shared memory
    float* s_o = reinterpret_cast<float*>(sKV);                  // [DM_WARPS][8][d]
    {
        if (g == 0) {
            s_m[warp][2 * t4] = m_run[0]; s_l[warp][2 * t4] = l_run[0];
            s_m[warp][2 * t4 + 1] = m_run[1]; s_l[warp][2 * t4 + 1] = l_run[1];
        }
#pragma unroll
        for (int mt = 0; mt < DMAX / 16; ++mt) {
            const int dim = mt * 16 + g;
            if (dim < d) {                 // d is a multiple of 16: dim + 8 < d as well
                float* pa = s_o + ((size_t)warp * 8 + 2 * t4) * d + dim;
                pa[0] = o_acc[mt][0]; pa[d] = o_acc[mt][1];
                pa[8] = o_acc[mt][2]; pa[d + 8] = o_acc[mt][3];
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_heads * d; i += DM_THREADS) {
        const int r = i / d, e = i - r * d;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w) mm = fmaxf(mm, s_m[w][r]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w) {
            const float f = s_m[w][r] == -INFINITY ? 0.f : exp2f(s_m[w][r] - mm);
            ll += s_l[w][r] * f;
            a += s_o[((size_t)w * 8 + r) * d + e] * f;
        }
        const int h = h0 + r;
        if (n_splits == 1) {
            out[((size_t)t * nh + h) * d + e] = __float2bfloat16_rn(a / ll);
        } else {
            float* part = partial + (((size_t)blockIdx.x * nh + h) * n_splits + split) * (d + 2);
            part[2 + e] = a;
            if (e == 0) { part[0] = mm; part[1] = ll; }
        }
    }
    if (n_splits == 1 || !counters) return;
    // The split that arrives last at this (token, first head of the block) merges all of them (in split
    // order, so the result does not depend on which one that was) and resets the counter.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* c = counters + (size_t)blockIdx.x * nh + h0;
        s_last = atomicAdd(c, 1) == n_splits - 1;
        if (s_last) *c = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < n_heads * d; i += DM_THREADS) {
        const int r = i / d, e = i - r * d;
        const int h = h0 + r;
        const float* all = partial + ((size_t)blockIdx.x * nh + h) * n_splits * (d + 2);
        float gm = -INFINITY;
        for (int sp = 0; sp < n_splits; ++sp) gm = fmaxf(gm, __ldcg(all + (size_t)sp * (d + 2)));
        float gl = 0.f, a = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float ms = __ldcg(all + (size_t)sp * (d + 2));
            const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - gm);
            gl += __ldcg(all + (size_t)sp * (d + 2) + 1) * f;
            a += __ldcg(all + (size_t)sp * (d + 2) + 2 + e) * f;
        }
        out[((size_t)t * nh + h) * d + e] = __float2bfloat16_rn(a / gl);
    }
}

template <int DMAX, bool DEEP>
static size_t dm_smem_bytes(int d, int block_pages, int warps) {
    const int DM_WARPS = warps;
    const size_t stages = (size_t)DM_WARPS * DmStages<DMAX, DEEP>::value * 2 * DM_KEYS * DMAX * sizeof(bf16);
    const size_t merge = (size_t)DM_WARPS * 8 * d * sizeof(float);         // reuses the stages' space
    return (stages > merge ? stages : merge) + (size_t)block_pages * sizeof(int);
}

ST_EXPORT int st_attention_decode_mma_applies(int d) { return d > 0 && d % 16 == 0 && d <= 128; }

static int dm_launch(const void* q, const DmQkv& qkv, const void* pool, void* out, float* partial, const int* items,
                     int n_items, const int* positions, const int* seq_of_token, const int* slots,
                     const int* start_pos, const int* block_table, int max_pages, int n_layers,
                     int layer, int nh, int nkv, int d, int page_size, float scale, int window,
                     int n_splits, int* counters, int warps, int* status, void* stream) {
    if (n_items <= 0) return 0;
    if (warps != 4 && warps != 8) return ST_ERR_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || n_splits < 1 || n_splits > 65535) return ST_ERR_BAD_ARG;
    if (!st_attention_decode_mma_applies(d)) return ST_ERR_BAD_SIZE;
    if (n_splits > 1 && !partial) return ST_ERR_BAD_ARG;
    const int group = nh / nkv;
    const long long gy = (long long)nkv * ((group + 7) / 8);
    if (gy > 65535) return ST_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_items, (unsigned)gy, n_splits);
    const float sl2 = scale * DM_LOG2E;
    int page_shift = -1;
    for (int b = 0; b < 30; ++b)
        if (page_size == (1 << b)) page_shift = b;
    int rc;
    // one block per SM at most: the deep ring
    const bool deep = !qkv.on && (long long)n_items * gy * n_splits <= st_sm_count();
#define LAUNCH_DM(DMAX, FULL, WARPS, DEEP, QKV)                                                                           \
    do {                                                                                                             \
        const size_t smem = dm_smem_bytes<DMAX, DEEP>(d, st_decode_block_pages(max_pages, page_size, window, n_splits), WARPS); \
        if (smem > 200 * 1024) return ST_ERR_TOO_LARGE;                                                              \
        static bool configured = false;                                                                              \
        if (!configured) {                                                                                           \
            cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<DMAX, FULL, WARPS, DEEP, QKV>,               \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
            if (e != cudaSuccess) return (int)e;                                                                     \
            configured = true;                                                                                       \
        }                                                                                                            \
        rc = st_launch_pdl("decode_mma", attention_decode_mma_kernel<DMAX, FULL, WARPS, DEEP, QKV>, grid, dim3(WARPS * 32), \
                           smem, s, (const bf16*)q, (const bf16*)pool, (bf16*)out,                                   \
                           n_splits > 1 ? partial : (float*)nullptr, items, positions, seq_of_token, slots,          \
                           start_pos, block_table, max_pages, n_layers, layer, nh, nkv, d, page_size, page_shift, sl2, window,  \
                           n_splits, counters, status, qkv);                                                         \
    } while (0)
#define LAUNCH_DM_W(DMAX, FULL)                                                                                      \
    do {                                                                                                             \
        if (deep && dm_smem_bytes<DMAX, true>(d, st_decode_block_pages(max_pages, page_size, window, n_splits), warps) <= 200 * 1024) { \
            if (warps == 8) LAUNCH_DM(DMAX, FULL, 8, true, false); else LAUNCH_DM(DMAX, FULL, 4, true, false); }     \
        else if (qkv.on) { if (warps == 8) LAUNCH_DM(DMAX, FULL, 8, false, true); else LAUNCH_DM(DMAX, FULL, 4, false, true); } \
        else { if (warps == 8) LAUNCH_DM(DMAX, FULL, 8, false, false); else LAUNCH_DM(DMAX, FULL, 4, false, false); } \
    } while (0)
    if (d == 64) LAUNCH_DM_W(64, true);
    else if (d < 64) LAUNCH_DM_W(64, false);
    else if (d == 128) LAUNCH_DM_W(128, true);
    else LAUNCH_DM_W(128, false);
#undef LAUNCH_DM_W
#undef LAUNCH_DM
    return rc;
}

// Same arguments and scratch layout as st_attention_decode, and the number of warps per block (4 or 8);
// start_pos (per request: the tokens it had in the cache before this step, or null) tells which keys earlier
// steps wrote, so that their copies can start before the kernel before this one has finished.
ST_EXPORT int st_attention_decode_mma(const void* q, const void* pool, void* out, float* partial, const int* items,
                                      int n_items, const int* positions, const int* seq_of_token, const int* slots,
                                      const int* start_pos, const int* block_table, int max_pages, int n_layers,
                                      int layer, int nh, int nkv, int d, int page_size, float scale, int window,
                                      int n_splits, int* counters, int warps, int* status, void* stream) {
    const DmQkv none = {};
    return dm_launch(q, none, pool, out, partial, items, n_items, positions, seq_of_token, slots, start_pos, block_table,
                     max_pages, n_layers, layer, nh, nkv, d, page_size, scale, window, n_splits, counters, warps, status,
                     stream);
}

// The q|k|v form: `qkv` [tokens, (nh + 2 nkv) d] is the fused projection of ALL the step's tokens (bfloat16, bias
// included), every token of the step is one of the items, and start_pos (required) tells where each request's tokens
// of this step begin.  The kernel writes each token's key and value rows into its page (write_kv; the pool has
// num_pages pages) and attends over the cache and the step's own rows.  No other kernel may need this step's keys in
// the cache (a step with prompt tiles does).
ST_EXPORT int st_attention_decode_mma_qkv(const void* qkv, void* pool, void* out, float* partial,
                                          const int* items, int n_items, const int* positions, const int* seq_of_token,
                                          const int* slots, const int* start_pos, const int* block_table, int max_pages,
                                          int num_pages, int n_layers, int layer, int nh, int nkv, int d, int page_size,
                                          float scale, int window, int n_splits, int* counters, int warps, int write_kv,
                                          int* status, void* stream) {
    if (!start_pos || !qkv || num_pages <= 0) return ST_ERR_BAD_ARG;
    if (!aligned16(qkv) || !aligned16(pool)) return ST_ERR_BAD_ARG;
    const DmQkv form = {(nh + 2 * nkv) * d, num_pages, write_kv ? 1 : 0, 1};
    return dm_launch(qkv, form, pool, out, partial, items, n_items, positions, seq_of_token, slots, start_pos, block_table,
                     max_pages, n_layers, layer, nh, nkv, d, page_size, scale, window, n_splits, counters, warps, status,
                     stream);
}
