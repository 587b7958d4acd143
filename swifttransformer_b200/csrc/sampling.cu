// Token selection from float logits [n_rows, vocab]: greedy argmax, and
// temperature sampling with an optional top-k cut, one thread block per row.
//
// The reference selects greedily only (src/csrc/kernel/findmax.cu:15-39, called
// from src/csrc/model/gpt/gpt.cc:205-210); on equal values it keeps whichever
// thread writes last.  Here ties go to the lowest id, and sampling is added:
//   p_i = exp((z_i - max z) / T) over the kept ids, draw by inverse CDF in id
//   order with a uniform number derived from (seed, draw index) alone, so a
//   request's tokens do not depend on what else is in the batch.
#include "common.cuh"

#define SAMPLE_THREADS 1024

// lowest index among the largest values; rows whose length is a multiple of 4 are read four at a time
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    __shared__ float sv[SAMPLE_THREADS / 32];
    __shared__ int si[SAMPLE_THREADS / 32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if ((vocab & 3) == 0) {
        const int nvec = vocab >> 2;
        for (int v0 = threadIdx.x; v0 < nvec; v0 += 2 * SAMPLE_THREADS) {
            const int v1 = v0 + SAMPLE_THREADS;
            const float4 a = load4(row + 4 * v0);
            const float4 b = v1 < nvec ? load4(row + 4 * v1) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (av[k] > best || best_i == 0x7fffffff) { best = av[k]; best_i = 4 * v0 + k; }
            if (v1 < nvec) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (bv[k] > best) { best = bv[k]; best_i = 4 * v1 + k; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            if (v > best || best_i == 0x7fffffff) { best = v; best_i = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < best_i)) { best = sv[w]; best_i = si[w]; }
        out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

ST_EXPORT int st_argmax(const float* logits, int n_rows, int vocab, int* out, void* stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return ST_ERR_BAD_SIZE;
    argmax_kernel<<<n_rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, vocab, out);
    return st_launch_status();
}

// 64-bit mix (splitmix64 finaliser) -> uniform float in [0,1)
__host__ __device__ __forceinline__ float st_uniform(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed * 0x9E3779B97F4A7C15ull + (counter + 1) * 0xBF58476D1CE4E5B9ull;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// Per row r: temperature temps[r] (<= 0: greedy), top_k[r] (<= 0: all ids), seed seeds[r], draw index counters[r].
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temps,
              const int* __restrict__ top_k, const long long* __restrict__ seeds,
              const long long* __restrict__ counters, int* __restrict__ out) {
    __shared__ float scratch[32];
    __shared__ float s_part[SAMPLE_THREADS];
    __shared__ int s_pick;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const float temp = temps[r];
    // max (and, for greedy rows, its lowest index)
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > best || best_i == 0x7fffffff) { best = v; best_i = i; }
    }
    const float zmax = block_max(best, scratch);
    if (temp <= 0.f) {
        int cand = (best == zmax) ? best_i : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __shared__ int s_cand[SAMPLE_THREADS / 32];
        if ((threadIdx.x & 31) == 0) s_cand[threadIdx.x >> 5] = cand;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < SAMPLE_THREADS / 32; ++w) cand = min(cand, s_cand[w]);
            out[r] = cand;
        }
        return;
    }
    // top-k threshold: the k-th largest value, found by bisection on the value
    // range (counts of elements >= mid), 40 halvings of [min, max].
    float thr = -INFINITY;
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
        float lo_v = INFINITY;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) lo_v = fminf(lo_v, row[i]);
        float lo = -block_max(-lo_v, scratch), hi = zmax;   // count(>= lo) = vocab >= k, count(>= hi) >= 1
        for (int it = 0; it < 40; ++it) {
            const float mid = lo + 0.5f * (hi - lo);
            if (!(mid > lo && mid < hi)) break;
            float c = 0.f;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += row[i] >= mid ? 1.f : 0.f;
            const float cnt = block_sum(c, scratch);
            if (cnt >= (float)k) lo = mid; else hi = mid;
        }
        thr = lo;   // at least k values are >= lo; values tied at the cut are all kept
    }
    const float inv_t = 1.0f / temp;
    // each thread owns a contiguous chunk so that the CDF runs in id order
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int b = threadIdx.x * chunk, e = min(vocab, b + chunk);
    float part = 0.f;
    for (int i = b; i < e; ++i) {
        const float v = row[i];
        if (v >= thr) part += expf((v - zmax) * inv_t);
    }
    s_part[threadIdx.x] = part;
    if (threadIdx.x == 0) s_pick = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) total += s_part[i];
        const float target = st_uniform((unsigned long long)seeds[r], (unsigned long long)counters[r]) * total;
        float run = 0.f;
        int owner = SAMPLE_THREADS - 1;
        for (int i = 0; i < SAMPLE_THREADS; ++i) {
            if (run + s_part[i] > target) { owner = i; break; }
            run += s_part[i];
        }
        // walk the owner's chunk
        const int ob = owner * chunk, oe = min(vocab, ob + chunk);
        int pick = -1, last_kept = -1;
        for (int i = ob; i < oe; ++i) {
            const float v = row[i];
            if (v >= thr) {
                run += expf((v - zmax) * inv_t);
                last_kept = i;
                if (run > target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last_kept;
        s_pick = pick;
    }
    __syncthreads();
    if (s_pick < 0) {   // rounding left the target beyond the last kept id: take the highest kept id
        int cand = -1;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) if (row[i] >= thr) cand = max(cand, i);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = max(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __shared__ int s_c2[SAMPLE_THREADS / 32];
        if ((threadIdx.x & 31) == 0) s_c2[threadIdx.x >> 5] = cand;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < SAMPLE_THREADS / 32; ++w) cand = max(cand, s_c2[w]);
            out[r] = cand;
        }
    } else if (threadIdx.x == 0) {
        out[r] = s_pick;
    }
}

ST_EXPORT int st_sample(const float* logits, int n_rows, int vocab, const float* temps, const int* top_k,
                        const long long* seeds, const long long* counters, int* out, void* stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return ST_ERR_BAD_SIZE;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, vocab, temps, top_k, seeds, counters, out);
    return st_launch_status();
}

// the same uniform number on the host, for callers that want to reproduce a draw
ST_EXPORT float st_uniform_host(long long seed, long long counter) {
    return st_uniform((unsigned long long)seed, (unsigned long long)counter);
}
