// Split a fused q|k|v projection, add its bias, keep q and write k, v into
// the paged cache at each token's position.
//
// Page pool layout (one pool per group of cache layers that share a shape):
//   pool[page][layer][0=K,1=V][kv_head][slot_in_page][head_dim]
// so that the keys of one (page, layer, head) are one contiguous
// page_size x head_dim box.  The block table maps (request slot, position /
// page_size) to a page id.
//
// Counterparts in the reference: bias add src/csrc/kernel/addbias.cu:71-88,
// prompt K/V scatter src/csrc/kernel/kvcache_mgmt.cu:29-80, and the decode
// kernel's own K/V write src/csrc/kernel/fused_decoding_stage_attention_mha.cu:130-140;
// here one kernel serves every kind of token.
#include "common.cuh"

// 16 bytes of T as floats and back
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int W = 4;
    __device__ static void unpack(const uint4& u, float* f) {
        f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
    }
    __device__ static uint4 pack(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};
template <> struct Vec16<bf16> {
    static constexpr int W = 8;
    __device__ static void unpack(const uint4& u, float* f) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            f[2 * i] = p.x; f[2 * i + 1] = p.y;
        }
    }
    __device__ static uint4 pack(const float* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// VEC: head_dim is a multiple of the elements in 16 bytes; a thread moves up to four such pieces per turn,
// all of them loaded before the chain position -> request -> slot -> page has been followed (the loads do
// not depend on it), so that chain's latency is hidden under them.
template <typename T, bool VEC>
__global__ void qkv_to_cache_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                    T* __restrict__ q_out, T* __restrict__ pool,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ slots, const int* __restrict__ block_table,
                                    int max_pages, int num_pages, int n_layers, int layer, int nh, int nkv,
                                    int d, int page_size, int write_kv, int* __restrict__ status) {
    // the kernel after this one may start its own preparations now (it waits for this one to end before it
    // touches anything written here)
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int qw = nh * d, kw = nkv * d;
    const T* row = qkv + (size_t)t * (qw + 2 * kw);
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    constexpr int W = VEC ? Vec16<T>::W : 1;
    constexpr int TURN = 4;
    const int all = (qw + 2 * kw) / W;
    uint4 held[TURN];
    if (VEC) {
#pragma unroll
        for (int j = 0; j < TURN; ++j) {
            const int v = (q_out ? 0 : qw / W) + threadIdx.x + j * blockDim.x;
            if (v < all) held[j] = *reinterpret_cast<const uint4*>(row + (size_t)v * W);
        }
    }
    int page = -1, off = 0;
    if (write_kv && pos >= 0) {   // pos < 0: padding token of a fixed-shape step, nothing is cached
        page = block_table[(size_t)slots[seq] * max_pages + pos / page_size];
        off = pos % page_size;
        if (page < 0 || page >= num_pages) {   // a hole in the block table: record it, write nothing
            if (threadIdx.x == 0) atomicExch(status, 1);
            page = -1;
        }
    }
    // q_out null: the queries stay where they are (the attention kernels read them with the row's stride) and
    // only keys and values move
    const int first = q_out ? 0 : qw / W;
    const int total = (page >= 0 ? qw + 2 * kw : qw) / W;
    auto target = [&](int e) -> T* {
        if (e < qw) return q_out + (size_t)t * qw + e;
        const int r = e - qw;
        const int kv = r / kw, rem = r - kv * kw;
        const int head = rem / d, dim = rem - head * d;
        return pool + (((((size_t)page * n_layers + layer) * 2 + kv) * nkv + head) * page_size + off) * d + dim;
    };
    if (VEC) {
        for (int base = first; base < total; base += TURN * blockDim.x) {
#pragma unroll
            for (int j = 0; j < TURN; ++j) {
                const int v = base + threadIdx.x + j * blockDim.x;
                if (v >= total) continue;
                const int e = v * W;
                const uint4 u = base == first ? held[j] : *reinterpret_cast<const uint4*>(row + e);
                float f[W];
                Vec16<T>::unpack(u, f);
                if (bias) {
#pragma unroll
                    for (int k = 0; k < W; k += 4) {
                        const float4 b = load4(bias + e + k);
                        f[k] += b.x; f[k + 1] += b.y; f[k + 2] += b.z; f[k + 3] += b.w;
                    }
                }
                *reinterpret_cast<uint4*>(target(e)) = Vec16<T>::pack(f);
            }
        }
    } else {
        for (int e = first + threadIdx.x; e < total; e += blockDim.x) {
            float a = to_f32(row[e]);
            if (bias) a += bias[e];
            *target(e) = from_f32<T>(a);
        }
    }
}

template <typename T>
static int launch_qkv_to_cache(const void* qkv, const float* bias, void* q_out, void* pool, const int* positions,
                               const int* seq_of_token, const int* slots, const int* block_table, int max_pages,
                               int num_pages, int n_layers, int layer, int n_tokens, int nh, int nkv, int d,
                               int page_size, int write_kv, int* status, cudaStream_t s) {
    constexpr int W16 = 16 / (int)sizeof(T);      // elements in 16 bytes
    const bool vec = d % W16 == 0 && aligned16(qkv) && aligned16(bias) && aligned16(q_out) && aligned16(pool);
    const int work = (nh + 2 * nkv) * d / (vec ? W16 * 4 : 1);   // a thread moves four pieces per turn
    int block = (work + 31) / 32 * 32;
    if (block > 512) block = 512;
    if (block < 64) block = 64;
    if (vec)
        qkv_to_cache_kernel<T, true><<<n_tokens, block, 0, s>>>((const T*)qkv, bias, (T*)q_out, (T*)pool, positions,
            seq_of_token, slots, block_table, max_pages, num_pages, n_layers, layer, nh, nkv, d, page_size, write_kv, status);
    else
        qkv_to_cache_kernel<T, false><<<n_tokens, block, 0, s>>>((const T*)qkv, bias, (T*)q_out, (T*)pool, positions,
            seq_of_token, slots, block_table, max_pages, num_pages, n_layers, layer, nh, nkv, d, page_size, write_kv, status);
    return st_launch_status();
}

ST_EXPORT int st_qkv_to_cache(const void* qkv, const float* bias, void* q_out, void* pool, const int* positions,
                              const int* seq_of_token, const int* slots, const int* block_table, int max_pages,
                              int num_pages, int n_layers, int layer, int n_tokens, int nh, int nkv, int d,
                              int page_size, int write_kv, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || d <= 0 || page_size <= 0 || layer < 0 || layer >= n_layers) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return launch_qkv_to_cache<float>(qkv, bias, q_out, pool, positions, seq_of_token, slots, block_table,
            max_pages, num_pages, n_layers, layer, n_tokens, nh, nkv, d, page_size, write_kv, status, s);
    if (dtype == 1)
        return launch_qkv_to_cache<bf16>(qkv, bias, q_out, pool, positions, seq_of_token, slots, block_table,
            max_pages, num_pages, n_layers, layer, n_tokens, nh, nkv, d, page_size, write_kv, status, s);
    return ST_ERR_BAD_DTYPE;
}
