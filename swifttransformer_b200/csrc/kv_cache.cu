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

// VEC: head_dim % 4 == 0, four elements per access
template <typename T, bool VEC>
__global__ void qkv_to_cache_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                    T* __restrict__ q_out, T* __restrict__ pool,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ slots, const int* __restrict__ block_table,
                                    int max_pages, int num_pages, int n_layers, int layer, int nh, int nkv,
                                    int d, int page_size, int write_kv, int* __restrict__ status) {
    const int t = blockIdx.x;
    const int qw = nh * d, kw = nkv * d;
    const T* row = qkv + (size_t)t * (qw + 2 * kw);
    const int pos = positions[t];
    int page = -1, off = 0;
    if (write_kv && pos >= 0) {   // pos < 0: padding token of a fixed-shape step, nothing is cached
        page = block_table[(size_t)slots[seq_of_token[t]] * max_pages + pos / page_size];
        off = pos % page_size;
        if (page < 0 || page >= num_pages) {   // a hole in the block table: record it, write nothing
            if (threadIdx.x == 0) atomicExch(status, 1);
            page = -1;
        }
    }
    constexpr int W = VEC ? 4 : 1;
    const int total = (page >= 0 ? qw + 2 * kw : qw) / W;
    for (int v = threadIdx.x; v < total; v += blockDim.x) {
        const int e = v * W;
        T* dst;
        if (e < qw) {
            dst = q_out + (size_t)t * qw + e;
        } else {
            const int r = e - qw;
            const int kv = r / kw, rem = r - kv * kw;
            const int head = rem / d, dim = rem - head * d;
            dst = pool + (((((size_t)page * n_layers + layer) * 2 + kv) * nkv + head) * page_size + off) * d + dim;
        }
        if (VEC) {
            float4 a = load4(row + e);
            if (bias) a = add4(a, load4(bias + e));
            store4(dst, a);
        } else {
            float a = to_f32(row[e]);
            if (bias) a += bias[e];
            *dst = from_f32<T>(a);
        }
    }
}

template <typename T>
static int launch_qkv_to_cache(const void* qkv, const float* bias, void* q_out, void* pool, const int* positions,
                               const int* seq_of_token, const int* slots, const int* block_table, int max_pages,
                               int num_pages, int n_layers, int layer, int n_tokens, int nh, int nkv, int d,
                               int page_size, int write_kv, int* status, cudaStream_t s) {
    const bool vec = d % 4 == 0 && aligned16(qkv) && aligned16(bias) && aligned16(q_out) && aligned16(pool);
    const int work = (nh + 2 * nkv) * d / (vec ? 4 : 1);
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
