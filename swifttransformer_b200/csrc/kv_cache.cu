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

template <typename T>
__global__ void qkv_to_cache_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                    T* __restrict__ q_out, T* __restrict__ pool,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ slots, const int* __restrict__ block_table,
                                    int max_pages, int num_pages, int n_layers, int layer, int nh, int nkv,
                                    int d, int page_size, int write_kv, int* __restrict__ status) {
    const int t = blockIdx.x;
    const int qw = nh * d, kw = nkv * d;
    const T* row = qkv + (size_t)t * (qw + 2 * kw);
    for (int e = threadIdx.x; e < qw; e += blockDim.x) {
        float v = to_f32(row[e]);
        if (bias) v += bias[e];
        q_out[(size_t)t * qw + e] = from_f32<T>(v);
    }
    if (!write_kv) return;
    const int pos = positions[t];
    if (pos < 0) return;   // padding token of a fixed-shape step
    const int slot = slots[seq_of_token[t]];
    const int page = block_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {   // a hole in the block table: record it, write nothing
        if (threadIdx.x == 0) atomicExch(status, 1);
        return;
    }
    const int off = pos % page_size;
    for (int e = threadIdx.x; e < 2 * kw; e += blockDim.x) {
        const int kv = e / kw, rem = e - kv * kw;
        const int head = rem / d, dim = rem - head * d;
        float v = to_f32(row[qw + e]);
        if (bias) v += bias[qw + e];
        const size_t idx = (((((size_t)page * n_layers + layer) * 2 + kv) * nkv + head) * page_size + off) * d + dim;
        pool[idx] = from_f32<T>(v);
    }
}

ST_EXPORT int st_qkv_to_cache(const void* qkv, const float* bias, void* q_out, void* pool, const int* positions,
                              const int* seq_of_token, const int* slots, const int* block_table, int max_pages,
                              int num_pages, int n_layers, int layer, int n_tokens, int nh, int nkv, int d,
                              int page_size, int write_kv, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || d <= 0 || page_size <= 0 || layer < 0 || layer >= n_layers) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = 256;
    if (dtype == 0)
        qkv_to_cache_kernel<float><<<n_tokens, block, 0, s>>>((const float*)qkv, bias, (float*)q_out, (float*)pool,
            positions, seq_of_token, slots, block_table, max_pages, num_pages, n_layers, layer, nh, nkv, d,
            page_size, write_kv, status);
    else if (dtype == 1)
        qkv_to_cache_kernel<bf16><<<n_tokens, block, 0, s>>>((const bf16*)qkv, bias, (bf16*)q_out, (bf16*)pool,
            positions, seq_of_token, slots, block_table, max_pages, num_pages, n_layers, layer, nh, nkv, d,
            page_size, write_kv, status);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}
