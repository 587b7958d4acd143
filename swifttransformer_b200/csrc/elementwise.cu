// Embedding lookup with learned positions, residual-add + normalisation,
// bias + activation, and small index utilities.
//
// Counterparts in the reference: embedding src/csrc/kernel/embedding.cu:16-35,
// LayerNorm with the fused residual add src/csrc/kernel/layernorm.cu:16-98,
// bias+activation src/csrc/kernel/fused_addbias_activ.cu:25-45, residual add
// src/csrc/kernel/addbias.cu:22-37, last-row gather src/csrc/kernel/gather_last_tokens.cu:23-37.
// Differences by design: sums, statistics and the residual stream are float for
// every storage type; the variance is two-pass; any width is accepted.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename T, typename TO>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, int width,
                             const int* __restrict__ pos, const T* __restrict__ pos_table, int pos_offset,
                             TO* __restrict__ out) {
    const int t = blockIdx.x;
    const T* row = table + (size_t)ids[t] * width;
    const T* prow = pos_table ? pos_table + (size_t)(pos[t] + pos_offset) * width : nullptr;
    TO* o = out + (size_t)t * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float v = to_f32(row[e]);
        if (prow) v += to_f32(prow[e]);
        o[e] = from_f32<TO>(v);
    }
}

// out[t,:] = in[t,:] + pos_table[pos[t]+offset,:]   (used after a project_in product)
template <typename T, typename TO>
__global__ void add_positions_kernel(const T* __restrict__ in, int width, const int* __restrict__ pos,
                                     const T* __restrict__ pos_table, int pos_offset, TO* __restrict__ out) {
    const int t = blockIdx.x;
    const T* prow = pos_table + (size_t)(pos[t] + pos_offset) * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x)
        out[(size_t)t * width + e] = from_f32<TO>(to_f32(in[(size_t)t * width + e]) + to_f32(prow[e]));
}

// out_dtype: 0 float, 1 same as dtype
ST_EXPORT int st_embed(const int* ids, const void* table, int n_tokens, int width, const int* pos,
                       const void* pos_table, int pos_offset, void* out, int dtype, int out_f32, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = width >= 1024 ? 256 : 128;
    if (dtype == 0) {
        embed_kernel<float, float><<<n_tokens, block, 0, s>>>(ids, (const float*)table, width, pos,
                                                               (const float*)pos_table, pos_offset, (float*)out);
    } else if (dtype == 1) {
        if (out_f32)
            embed_kernel<bf16, float><<<n_tokens, block, 0, s>>>(ids, (const bf16*)table, width, pos,
                                                                  (const bf16*)pos_table, pos_offset, (float*)out);
        else
            embed_kernel<bf16, bf16><<<n_tokens, block, 0, s>>>(ids, (const bf16*)table, width, pos,
                                                                 (const bf16*)pos_table, pos_offset, (bf16*)out);
    } else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}

ST_EXPORT int st_add_positions(const void* in, int n_tokens, int width, const int* pos, const void* pos_table,
                               int pos_offset, void* out, int dtype, int out_f32, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = width >= 1024 ? 256 : 128;
    if (dtype == 0)
        add_positions_kernel<float, float><<<n_tokens, block, 0, s>>>((const float*)in, width, pos,
                                                                       (const float*)pos_table, pos_offset, (float*)out);
    else if (dtype == 1) {
        if (out_f32)
            add_positions_kernel<bf16, float><<<n_tokens, block, 0, s>>>((const bf16*)in, width, pos,
                                                                          (const bf16*)pos_table, pos_offset, (float*)out);
        else
            add_positions_kernel<bf16, bf16><<<n_tokens, block, 0, s>>>((const bf16*)in, width, pos,
                                                                         (const bf16*)pos_table, pos_offset, (bf16*)out);
    } else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}

// ------------------------------------------------------- residual add + norm
// For output row r (input row i = rows ? rows[r] : r):
//   s = x[i] + delta[i] + delta_bias        (delta, delta_bias optional)
//   resid_out[i] = s                        (optional; may alias x)
//   y = kind 0: (s - mean(s)) * rsqrt(var(s) + eps) * gamma + beta   (LayerNorm)
//       kind 1: s * rsqrt(mean(s^2) + eps) * gamma                   (RMS norm)
//       kind 2: s                                                    (no norm)
//   out_act[r] = T(y)  (optional), out_f32[r] = y  (optional; may alias x when rows is null)
// The row is staged in shared memory as float; all statistics are float.
template <typename T>
__global__ void add_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                const T* __restrict__ delta, const float* __restrict__ delta_bias,
                                float* resid_out, const float* __restrict__ gamma,
                                const float* __restrict__ beta, float eps, int kind, int width,
                                T* __restrict__ out_act, float* out_f32) {
    extern __shared__ float srow[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t i = rows ? (size_t)rows[r] : (size_t)r;
    const float* xr = x + i * width;
    float sum = 0.f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float v = xr[e];
        if (delta) v += to_f32(delta[i * width + e]);
        if (delta_bias) v += delta_bias[e];
        srow[e] = v;
        sum += v;
    }
    if (resid_out) {
        for (int e = threadIdx.x; e < width; e += blockDim.x) resid_out[i * width + e] = srow[e];
    }
    float mean = 0.f, rstd = 1.f;
    if (kind == 0) {
        mean = block_sum(sum, scratch) / (float)width;
        float sq = 0.f;
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            const float d = srow[e] - mean;
            sq += d * d;
        }
        const float var = block_sum(sq, scratch) / (float)width;
        rstd = 1.0f / sqrtf(var + eps);
    } else if (kind == 1) {
        float sq = 0.f;
        for (int e = threadIdx.x; e < width; e += blockDim.x) sq += srow[e] * srow[e];
        const float ms = block_sum(sq, scratch) / (float)width;
        rstd = 1.0f / sqrtf(ms + eps);
    }
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float y = srow[e];
        if (kind != 2) {
            y = (y - mean) * rstd;
            if (gamma) y *= gamma[e];
            if (beta) y += beta[e];
        }
        if (out_act) out_act[(size_t)r * width + e] = from_f32<T>(y);
        if (out_f32) out_f32[(size_t)r * width + e] = y;
    }
}

ST_EXPORT int st_add_norm(const float* x, const int* rows, const void* delta, const float* delta_bias,
                          float* resid_out, const float* gamma, const float* beta, float eps, int kind,
                          int n_rows, int width, void* out_act, float* out_f32, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (kind < 0 || kind > 2 || width <= 0) return ST_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return ST_ERR_TOO_LARGE;
    int block = 128;
    if (width >= 2048) block = 256;
    if (width >= 8192) block = 512;
    if (dtype == 0) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_norm_kernel<float><<<n_rows, block, smem, s>>>(x, rows, (const float*)delta, delta_bias, resid_out,
                                                           gamma, beta, eps, kind, width, (float*)out_act, out_f32);
    } else if (dtype == 1) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_norm_kernel<bf16><<<n_rows, block, smem, s>>>(x, rows, (const bf16*)delta, delta_bias, resid_out,
                                                          gamma, beta, eps, kind, width, (bf16*)out_act, out_f32);
    } else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}

// ------------------------------------------------------------ bias + activation
template <typename T>
__global__ void bias_act_kernel(T* __restrict__ y, const float* __restrict__ bias, int act, size_t total, int width) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = to_f32(y[i]);
        if (bias) v += bias[i % width];
        y[i] = from_f32<T>(apply_act(v, act));
    }
}

ST_EXPORT int st_bias_act(void* y, const float* bias, int act, int n_rows, int width, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    const size_t total = (size_t)n_rows * width;
    int grid = (int)((total + 255) / 256);
    if (grid > 148 * 16) grid = 148 * 16;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0) bias_act_kernel<float><<<grid, 256, 0, s>>>((float*)y, bias, act, total, width);
    else if (dtype == 1) bias_act_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)y, bias, act, total, width);
    else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}

// ------------------------------------------------------------- index utilities
// dst[idx[i]] = val[i] for i < *count (count read on the device so that the
// launch shape does not depend on it).
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx,
                                   const int* __restrict__ val, const int* __restrict__ count) {
    const int n = *count;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[idx[i]] = val[i];
}

ST_EXPORT int st_scatter_i32(int* dst, const int* idx, const int* val, const int* count, int max_count, void* stream) {
    if (max_count <= 0) return 0;
    int grid = (max_count + 255) / 256;
    if (grid > 64) grid = 64;
    scatter_i32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(dst, idx, val, count);
    return st_launch_status();
}
