// Plain paged attention: one thread block per (query token, head), for any
// head size, page size, number of heads and groups, in float or bfloat16
// storage with float arithmetic throughout.
//
// The query at position p of a request attends the keys lo..p of that
// request, lo = max(0, p - window + 1) (window <= 0: all keys), read from the
// pages its block table names; the step's own keys have been written before.
// Keys are visited in tiles of KT aligned to absolute positions and reduced in
// a fixed order, so the result for a position does not depend on how the
// request was cut into steps or on what else is in the batch.
//
// Formulas: src/csrc/kernel/fused_decoding_stage_attention_mha.cu:159-252
// (scores, softmax) and :254-318 (weighted sum of values); the prompt kernel
// src/csrc/kernel/fused_context_stage_attention.cu:226-404 computes the same
// per row.  Not taken over: the -10000 additive mask and the +1e-6 in the
// denominator; masked keys are simply not visited.
#include "common.cuh"

#define KT 128  // keys per tile == threads per block

template <typename T>
__global__ void __launch_bounds__(KT)
attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pool, T* __restrict__ out,
                       const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                       const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages,
                       int n_layers, int layer, int nh, int nkv, int d, int page_size, float scale, int window,
                       int* __restrict__ status) {
    extern __shared__ float smem[];
    float* sq = smem;        // [d] query, pre-scaled
    float* sp = smem + d;    // [KT] probabilities of the tile
    __shared__ float scratch[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (nh / nkv);
    const int pos = positions[t];
    if (pos < 0) return;   // padding token of a fixed-shape step
    const int slot = slots[seq_of_token[t]];
    const int* bt = block_table + (size_t)slot * max_pages;
    for (int e = threadIdx.x; e < d; e += blockDim.x) sq[e] = to_f32(q[((size_t)t * nh + h) * d + e]) * scale;
    __syncthreads();
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int hi = pos + 1;
    const int ndim = (d + KT - 1) / KT;   // output dims per thread (d <= 2*KT is enforced by the launcher)
    float acc[2] = {0.f, 0.f};
    float m = -INFINITY, l = 0.f;
    for (int base = (lo / KT) * KT; base < hi; base += KT) {
        const int j = base + threadIdx.x;
        float s = -INFINITY;
        if (j >= lo && j < hi) {
            const int page = bt[j / page_size];
            if (page >= 0) {     // a hole in the block table: the key is dropped, no access before the pool
                const T* krow = pool + (((((size_t)page * n_layers + layer) * 2 + 0) * nkv + kvh) * page_size + j % page_size) * d;
                float dot = 0.f;
                for (int e = 0; e < d; ++e) dot += sq[e] * to_f32(krow[e]);
                s = dot;
            } else if (status) {
                *status = 1;     // reported to the host: the step's bookkeeping is broken
            }
        }
        const float tile_max = block_max(s, scratch);
        const float m_new = fmaxf(m, tile_max);
        const float p = (j >= lo && j < hi) ? expf(s - m_new) : 0.f;
        const float tile_sum = block_sum(p, scratch);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + tile_sum;
        m = m_new;
        sp[threadIdx.x] = p;
        __syncthreads();
        const int j_end = min(KT, hi - base);
        const int j_begin = max(0, lo - base);
        for (int c = 0; c < ndim; ++c) {
            const int e = threadIdx.x + c * KT;
            if (e < d) {
                float a = acc[c] * corr;
                for (int jj = j_begin; jj < j_end; ++jj) {
                    const int key = base + jj;
                    const int page = bt[key / page_size];
                    if (page < 0) continue;      // dropped above: its weight is zero
                    const T* vrow = pool + (((((size_t)page * n_layers + layer) * 2 + 1) * nkv + kvh) * page_size + key % page_size) * d;
                    a += sp[jj] * to_f32(vrow[e]);
                }
                acc[c] = a;
            }
        }
        __syncthreads();
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;      // no key at all (every page missing): zeros, not NaN
    for (int c = 0; c < ndim; ++c) {
        const int e = threadIdx.x + c * KT;
        if (e < d) out[((size_t)t * nh + h) * d + e] = from_f32<T>(acc[c] * inv);
    }
}

ST_EXPORT int st_attention_plain(const void* q, const void* pool, void* out, const int* positions,
                                 const int* seq_of_token, const int* slots, const int* block_table, int max_pages,
                                 int n_layers, int layer, int n_tokens, int nh, int nkv, int d, int page_size,
                                 float scale, int window, int dtype, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || d <= 0 || page_size <= 0) return ST_ERR_BAD_ARG;
    if (d > 2 * KT) return ST_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, nh);
    const size_t smem = (size_t)(d + KT) * sizeof(float);
    if (dtype == 0)
        attention_plain_kernel<float><<<grid, KT, smem, s>>>((const float*)q, (const float*)pool, (float*)out,
            positions, seq_of_token, slots, block_table, max_pages, n_layers, layer, nh, nkv, d, page_size, scale, window, status);
    else if (dtype == 1)
        attention_plain_kernel<bf16><<<grid, KT, smem, s>>>((const bf16*)q, (const bf16*)pool, (bf16*)out,
            positions, seq_of_token, slots, block_table, max_pages, n_layers, layer, nh, nkv, d, page_size, scale, window, status);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}
