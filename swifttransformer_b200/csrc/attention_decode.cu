// Paged attention for queries that stand alone (decode tokens and very short
// portions), bfloat16 storage, float arithmetic: a bandwidth-bound kernel.
//
// One thread block per (query token, head, split of the key range).  Eight
// lanes share a key: each loads 16 bytes of the key row (and later of the
// value row) per 64 dims, so a warp reads four full rows per instruction and
// every byte of the cache is read once.  Each 8-lane group runs its own online
// softmax over the keys it visits; the sixteen groups of a block, and then the
// splits of a token, are merged with the usual max / sum rescaling in float.
// With one split the block writes the normalised output itself; otherwise it
// leaves (max, sum, weighted values) in `partial` and st_attention_combine
// finishes.
//
// Same mathematics as src/csrc/kernel/fused_decoding_stage_attention_mha.cu:159-318
// in the reference (which keeps the value sum in the storage type and
// handles one fixed set of head sizes); the K/V write that the reference does
// in that kernel is done beforehand by st_qkv_to_cache.
#include "common.cuh"

#define DEC_THREADS 128
#define DEC_GROUPS (DEC_THREADS / 8)
#define LOG2E 1.4426950408889634f

struct __align__(16) bf16x8 { __nv_bfloat162 v[4]; };

// 16-byte load that is served by L2, not by the per-SM caches: the newest key/value row and the
// queries were written by the kernel just before this one, which may still have been running when
// this block became resident (programmatic dependent launch).
__device__ __forceinline__ bf16x8 ldg16(const bf16* p) {
    bf16x8 r;
    *reinterpret_cast<uint4*>(&r) = __ldcg(reinterpret_cast<const uint4*>(p));
    return r;
}

// head_dim <= 64 * NCHUNK, a multiple of 8; FULL: head_dim == 64 * NCHUNK, known when compiling
template <int NCHUNK, bool FULL>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, bf16* __restrict__ out,
                        float* __restrict__ partial, const int* __restrict__ items,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages,
                        int n_layers, int layer, int nh, int nkv, int d_arg, int page_size, float scale_log2,
                        int window, int n_splits, int* __restrict__ counters, int* __restrict__ status) {
    const int d = FULL ? 64 * NCHUNK : d_arg;
    __shared__ float s_m[DEC_GROUPS], s_l[DEC_GROUPS];
    __shared__ int s_last;
    extern __shared__ float s_acc[];   // [DEC_GROUPS][d]
    ST_PDL_TRIGGER();
    // the token's position, slot and page numbers are inputs of the step that no kernel of the step writes:
    // they are fetched before the wait for the kernel before this one; queries, keys and values after it
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0) return;            // a padding entry of a fixed-shape step
    const int h = blockIdx.y, split = blockIdx.z;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    if (pos < 0) return;   // padding entry of a fixed-shape launch
    const int slot = slots[seq_of_token[t]];
    const int* bt = block_table + (size_t)slot * max_pages;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int hi = pos + 1;
    int per = (hi - lo + n_splits - 1) / n_splits;
    per = (per + 15) / 16 * 16;
    const int k_lo = lo + split * per;
    const int k_hi = min(hi, k_lo + per);
    // the page ids of this block's key range, fetched once: a round then costs one trip to memory
    // (the rows), not two (page id, then rows)
    int* s_pages = reinterpret_cast<int*>(s_acc + DEC_GROUPS * d);
    const int p_lo = k_lo / page_size;
    if (k_lo < k_hi) {
        const int n_pages = (k_hi - 1) / page_size - p_lo + 1;
        for (int i = threadIdx.x; i < n_pages; i += DEC_THREADS) {
            const int page = __ldcg(bt + p_lo + i);
            s_pages[i] = page;
            if (page < 0 && status) *status = 1;     // a hole in the block table: its keys are dropped and the host hears of it
        }
    }
    ST_PDL_WAIT();
    __syncthreads();

    const int g = threadIdx.x >> 3, l8 = threadIdx.x & 7;
    float qf[NCHUNK][8];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
        const int dim0 = (c * 8 + l8) * 8;
        if (dim0 < d) {
            const bf16x8 v = ldg16(q + ((size_t)t * nh + h) * d + dim0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(v.v[i]);
                qf[c][2 * i] = f.x * scale_log2;
                qf[c][2 * i + 1] = f.y * scale_log2;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) qf[c][i] = 0.f;
        }
    }
    float acc[NCHUNK][8];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const size_t head_stride = (size_t)page_size * d;
    const size_t kv_stride = (size_t)nkv * head_stride;

    // Every lane of the block runs the same number of rounds (the shuffles need all 32 lanes).  In a
    // round each 8-lane group takes KU keys; the loads of the next round are issued before the
    // current one is used (two register buffers), so that rows are in flight all the time.  A key
    // past the end re-reads the last key and is dropped.
    constexpr int KU = NCHUNK == 1 ? 4 : (NCHUNK == 2 ? 2 : 1);
    constexpr int STEP = DEC_GROUPS * KU;
    struct Round { bf16x8 k[KU][NCHUNK], v[KU][NCHUNK]; bool valid[KU]; };
    auto issue = [&](Round& r, int key0) {
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int kk = key0 + u * DEC_GROUPS + g;
            r.valid[u] = kk < k_hi;
            const int key = r.valid[u] ? kk : k_hi - 1;
            const int pg = key / page_size;
            int page = s_pages[pg - p_lo];
            if (page < 0) { r.valid[u] = false; page = 0; }   // a hole in the block table: the key is dropped, no access before the pool
            const bf16* krow = pool + ((size_t)page * n_layers + layer) * 2 * kv_stride + kvh * head_stride
                               + (size_t)(key - pg * page_size) * d;
#pragma unroll
            for (int c = 0; c < NCHUNK; ++c) {
                const int dim0 = (c * 8 + l8) * 8;
                if (dim0 < d) { r.k[u][c] = ldg16(krow + dim0); r.v[u][c] = ldg16(krow + kv_stride + dim0); }
            }
        }
    };
    auto consume = [&](const Round& r) {
        float s[KU];
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            float a = 0.f;
#pragma unroll
            for (int c = 0; c < NCHUNK; ++c) {
                const int dim0 = (c * 8 + l8) * 8;
                if (dim0 < d) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(r.k[u][c].v[i]);
                        a = fmaf(qf[c][2 * i], f.x, a);
                        a = fmaf(qf[c][2 * i + 1], f.y, a);
                    }
                }
            }
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            a += __shfl_xor_sync(0xffffffffu, a, 4);
            s[u] = r.valid[u] ? a : -INFINITY;
        }
        float m_new = m;
#pragma unroll
        for (int u = 0; u < KU; ++u) m_new = fmaxf(m_new, s[u]);
        if (m_new == -INFINITY) return;               // this group has had no key so far
        const float corr = exp2f(m - m_new);          // m = -inf before the first key: exp2f(-inf) = 0
        float p[KU];
        float psum = 0.f;
#pragma unroll
        for (int u = 0; u < KU; ++u) { p[u] = exp2f(s[u] - m_new); psum += p[u]; }
        l = l * corr + psum;
        m = m_new;
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
            const int dim0 = (c * 8 + l8) * 8;
            if (dim0 < d) {
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[c][i] *= corr;
#pragma unroll
                for (int u = 0; u < KU; ++u) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(r.v[u][c].v[i]);
                        acc[c][2 * i] = fmaf(p[u], f.x, acc[c][2 * i]);
                        acc[c][2 * i + 1] = fmaf(p[u], f.y, acc[c][2 * i + 1]);
                    }
                }
            }
        }
    };
    if (k_lo < k_hi) {
        Round ra, rb;
        issue(ra, k_lo);
        for (int key0 = k_lo; key0 < k_hi; key0 += 2 * STEP) {
            const bool more_b = key0 + STEP < k_hi;           // uniform over the block
            if (more_b) issue(rb, key0 + STEP);
            consume(ra);
            if (key0 + 2 * STEP < k_hi) issue(ra, key0 + 2 * STEP);
            if (more_b) consume(rb);
        }
    }
    if (l8 == 0) { s_m[g] = m; s_l[g] = l; }
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
        const int dim0 = (c * 8 + l8) * 8;
        if (dim0 < d) {
#pragma unroll
            for (int i = 0; i < 8; ++i) s_acc[g * d + dim0 + i] = acc[c][i];
        }
    }
    __syncthreads();
    float mm = -INFINITY;
#pragma unroll
    for (int i = 0; i < DEC_GROUPS; ++i) mm = fmaxf(mm, s_m[i]);
    float ll = 0.f;
#pragma unroll
    for (int i = 0; i < DEC_GROUPS; ++i) ll += (s_m[i] == -INFINITY) ? 0.f : s_l[i] * exp2f(s_m[i] - mm);
    float* part = partial ? partial + (((size_t)blockIdx.x * nh + h) * n_splits + split) * (d + 2) : nullptr;
    for (int e = threadIdx.x; e < d; e += DEC_THREADS) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < DEC_GROUPS; ++i)
            a += (s_m[i] == -INFINITY) ? 0.f : s_acc[i * d + e] * exp2f(s_m[i] - mm);
        if (n_splits == 1) out[((size_t)t * nh + h) * d + e] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
        else part[2 + e] = a;
    }
    if (n_splits > 1 && threadIdx.x == 0) { part[0] = mm; part[1] = ll; }
    if (n_splits == 1 || !counters) return;
    // The split that arrives last at this (token, head) merges all of them (in split order, so the
    // result does not depend on which one that was) and resets the counter for the next launch.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* c = counters + (size_t)blockIdx.x * nh + h;
        s_last = atomicAdd(c, 1) == n_splits - 1;
        if (s_last) *c = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* all = partial + ((size_t)blockIdx.x * nh + h) * n_splits * (d + 2);
    float gm = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) gm = fmaxf(gm, __ldcg(all + (size_t)sp * (d + 2)));
    float gl = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
        const float ms = __ldcg(all + (size_t)sp * (d + 2));
        gl += (ms == -INFINITY) ? 0.f : __ldcg(all + (size_t)sp * (d + 2) + 1) * exp2f(ms - gm);
    }
    for (int e = threadIdx.x; e < d; e += DEC_THREADS) {
        float a = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float ms = __ldcg(all + (size_t)sp * (d + 2));
            a += (ms == -INFINITY) ? 0.f : __ldcg(all + (size_t)sp * (d + 2) + 2 + e) * exp2f(ms - gm);
        }
        out[((size_t)t * nh + h) * d + e] = __float2bfloat16_rn(gl > 0.f ? a / gl : 0.f);
    }
}

// merge the splits of every (item, head)
__global__ void attention_combine_kernel(const float* __restrict__ partial, bf16* __restrict__ out,
                                         const int* __restrict__ items, const int* __restrict__ positions,
                                         int nh, int d, int n_splits) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = items ? items[blockIdx.x] : blockIdx.x;
    if (t < 0 || positions[t] < 0) return;
    const int h = blockIdx.y;
    const float* part = partial + ((size_t)blockIdx.x * nh + h) * n_splits * (d + 2);
    float mm = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, part[(size_t)s * (d + 2)]);
    float ll = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part[(size_t)s * (d + 2)];
        ll += (ms == -INFINITY) ? 0.f : part[(size_t)s * (d + 2) + 1] * exp2f(ms - mm);
    }
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part[(size_t)s * (d + 2)];
            a += (ms == -INFINITY) ? 0.f : part[(size_t)s * (d + 2) + 2 + e] * exp2f(ms - mm);
        }
        out[((size_t)t * nh + h) * d + e] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
    }
}

// Number of floats of scratch that st_attention_decode needs for n_splits > 1.
ST_EXPORT long long st_attention_decode_scratch_floats(int n_items, int nh, int d, int n_splits) {
    return n_splits > 1 ? (long long)n_items * nh * n_splits * (d + 2) : 0;
}

// counters: n_items * nh ints, zero before the first launch (the kernel leaves them zero), or null: the
// splits are then merged by a second kernel.  status: null, or a word that is set to 1 when a key range
// crosses a hole in a block table.
ST_EXPORT int st_attention_decode(const void* q, const void* pool, void* out, float* partial, const int* items,
                                  int n_items, const int* positions, const int* seq_of_token, const int* slots,
                                  const int* block_table, int max_pages, int n_layers, int layer, int nh, int nkv,
                                  int d, int page_size, float scale, int window, int n_splits, int* counters,
                                  int* status, void* stream) {
    if (n_items <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || page_size <= 0 || n_splits < 1 || n_splits > 65535) return ST_ERR_BAD_ARG;
    if (d % 8 || d <= 0) return ST_ERR_BAD_SIZE;
    if (d > 256) return ST_ERR_TOO_LARGE;
    if (n_splits > 1 && !partial) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_items, nh, n_splits);
    // merge buffers of the 16 key groups, then the page ids of the block's key range
    const size_t smem = (size_t)DEC_GROUPS * d * sizeof(float)
                        + (size_t)st_decode_block_pages(max_pages, page_size, window, n_splits) * sizeof(int);
    if (smem > 48 * 1024) return ST_ERR_TOO_LARGE;
    const float sl2 = scale * LOG2E;
#define LAUNCH_DEC(NC)                                                                                         \
    (d == 64 * NC ? LAUNCH_DEC2(NC, true) : LAUNCH_DEC2(NC, false))
#define LAUNCH_DEC2(NC, FULL)                                                                                  \
    st_launch_pdl("decode", attention_decode_kernel<NC, FULL>, grid, dim3(DEC_THREADS), smem, s, (const bf16*)q,               \
        (const bf16*)pool, (bf16*)out, n_splits > 1 ? partial : (float*)nullptr, items, positions,              \
        seq_of_token, slots, block_table, max_pages, n_layers, layer, nh, nkv, d, page_size, sl2, window,       \
        n_splits, counters, status)
    int rc;
    if (d <= 64) rc = LAUNCH_DEC(1);
    else if (d <= 128) rc = LAUNCH_DEC(2);
    else if (d <= 192) rc = LAUNCH_DEC(3);
    else rc = LAUNCH_DEC(4);
#undef LAUNCH_DEC
#undef LAUNCH_DEC2
    if (rc) return rc;
    if (n_splits > 1 && !counters) {
        dim3 g2(n_items, nh);
        rc = st_launch_pdl("combine", attention_combine_kernel, g2, dim3(64), 0, s, (const float*)partial, (bf16*)out, items,
                           positions, nh, d, n_splits);
    }
    return rc;
}

// ---------------------------------------------------------------------------
// The same operation for callers that cannot allocate: scratch inside the
// library.  See attention_decode_noalloc.h for who needs this and the rules.
// ---------------------------------------------------------------------------
#include <stdio.h>
#include "attention_decode_noalloc.h"

// counters first (as ints), then the partial results
static __device__ __align__(256) float st_noalloc_scratch[ST_NOALLOC_MAX_PAIRS + ST_NOALLOC_SCRATCH_FLOATS];

#define ST_NOALLOC_MAX_DEVICES 64
// In host code the array's name is only a handle for the runtime, not an address a kernel can use:
// the device address is asked for once per device and kept here.
static float* st_noalloc_device_ptr[ST_NOALLOC_MAX_DEVICES];

static void noalloc_say(char* err, int err_len, const char* fmt, long long a, long long b) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, fmt, a, b);
}

ST_EXPORT int st_attention_decode_noalloc(const void* q, const void* pool, void* out, const int* items, int n_items,
                                          const int* positions, const int* seq_of_token, const int* slots,
                                          const int* block_table, int max_pages, int n_layers, int layer, int nh,
                                          int nkv, int d, int page_size, float scale, int window, int n_splits,
                                          void* stream, char* err, int err_len) {
    if (err && err_len > 0) err[0] = 0;
    if (n_items <= 0) return 0;
    if (nh <= 0 || d <= 0 || n_splits < 1) {
        noalloc_say(err, err_len, "invalid sizes: %lld heads, %lld splits", nh, n_splits);
        return ST_ERR_BAD_ARG;
    }
    const long long pairs = (long long)n_items * nh;
    const long long floats = n_splits > 1 ? pairs * n_splits * (d + 2) : 0;
    if (pairs > ST_NOALLOC_MAX_PAIRS) {
        noalloc_say(err, err_len, "%lld (token, head) pairs exceed the built-in scratch's limit of %lld",
                    pairs, (long long)ST_NOALLOC_MAX_PAIRS);
        return ST_ERR_TOO_LARGE;
    }
    if (floats > ST_NOALLOC_SCRATCH_FLOATS) {
        noalloc_say(err, err_len, "the call needs %lld floats of scratch; the built-in scratch holds %lld",
                    floats, (long long)ST_NOALLOC_SCRATCH_FLOATS);
        return ST_ERR_TOO_LARGE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= ST_NOALLOC_MAX_DEVICES) {
        noalloc_say(err, err_len, "device index %lld is beyond the %lld devices this entry point keeps track of",
                    dev, (long long)ST_NOALLOC_MAX_DEVICES);
        return ST_ERR_BAD_ARG;
    }
    if (!st_noalloc_device_ptr[dev]) {   // first call on this device: set-up (not inside a stream capture)
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, st_noalloc_scratch);
        if (e != cudaSuccess) {
            noalloc_say(err, err_len, "cudaGetSymbolAddress failed with error %lld on device %lld", (long long)e, dev);
            return (int)e;
        }
        st_noalloc_device_ptr[dev] = p;
    }
    float* base = st_noalloc_device_ptr[dev];
    int* counters = reinterpret_cast<int*>(base);
    float* partial = base + ST_NOALLOC_MAX_PAIRS;
    if (n_splits > 1) {
        // the array keeps whatever the last call left: the counters must start at zero
        e = cudaMemsetAsync(counters, 0, (size_t)pairs * sizeof(int), (cudaStream_t)stream);
        if (e != cudaSuccess) return (int)e;
    }
    return st_attention_decode(q, pool, out, partial, items, n_items, positions, seq_of_token, slots, block_table,
                               max_pages, n_layers, layer, nh, nkv, d, page_size, scale, window, n_splits,
                               n_splits > 1 ? counters : nullptr, nullptr, stream);
}
