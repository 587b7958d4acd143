// Plain matrix product with a fused epilogue, float arithmetic only:
//   out[n, m] = act( sum_k a[n,k] * w[m,k] + bias[m] )       w stored [out, in]
// Every output element is one chain of fused multiply-adds over k in ascending
// order, whatever the number of rows, so a row's result does not depend on the
// batch it is in.  This is the matrix product of the 32-bit path (no tensor
// cores, no reduced-precision mode) and the plain twin of the bfloat16 one.
//
// The reference calls cuBLAS for all five products (src/csrc/util/cublas_wrapper.cc:29-53,
// call sites src/csrc/layer/attention.cc:102,255, src/csrc/layer/ffn.cc:71,96,
// src/csrc/model/gpt/gpt.cc:192) and adds bias / activation in separate kernels.
#include "common.cuh"

#define GBM 64
#define GBN 64
#define GBK 16

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const T* __restrict__ a, const T* __restrict__ w, const float* __restrict__ bias,
                  TO* __restrict__ out, int n_rows, int n_out, int k_dim, int act) {
    __shared__ float sa[GBK][GBM + 4];
    __shared__ float sw[GBK][GBN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // tx -> out features, ty -> rows
    const int row0 = blockIdx.y * GBM, col0 = blockIdx.x * GBN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < k_dim; k0 += GBK) {
        // 64 x 16 elements of each operand, 256 threads -> 4 each
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = threadIdx.x + it * 256;
            const int r = idx / GBK, kk = idx % GBK;
            const int k = k0 + kk;
            const int ar = row0 + r, wr = col0 + r;
            sa[kk][r] = (ar < n_rows && k < k_dim) ? to_f32(a[(size_t)ar * k_dim + k]) : 0.f;
            sw[kk][r] = (wr < n_out && k < k_dim) ? to_f32(w[(size_t)wr * k_dim + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GBK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx * 4 + j;
            if (c >= n_out) continue;
            float v = acc[i][j];
            if (bias) v += bias[c];
            out[(size_t)r * n_out + c] = from_f32<TO>(apply_act(v, act));
        }
    }
}

ST_EXPORT int st_gemm_plain(const void* a, const void* w, const float* bias, void* out, int n_rows, int n_out,
                            int k_dim, int act, int dtype, int out_f32, void* stream) {
    if (n_rows <= 0 || n_out <= 0) return 0;
    if (k_dim <= 0) return ST_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((n_out + GBN - 1) / GBN, (n_rows + GBM - 1) / GBM);
    if (grid.y > 65535) return ST_ERR_TOO_LARGE;
    if (dtype == 0)
        gemm_plain_kernel<float, float><<<grid, 256, 0, s>>>((const float*)a, (const float*)w, bias, (float*)out,
                                                              n_rows, n_out, k_dim, act);
    else if (dtype == 1) {
        if (out_f32)
            gemm_plain_kernel<bf16, float><<<grid, 256, 0, s>>>((const bf16*)a, (const bf16*)w, bias, (float*)out,
                                                                 n_rows, n_out, k_dim, act);
        else
            gemm_plain_kernel<bf16, bf16><<<grid, 256, 0, s>>>((const bf16*)a, (const bf16*)w, bias, (bf16*)out,
                                                                n_rows, n_out, k_dim, act);
    } else return ST_ERR_BAD_DTYPE;
    return st_launch_status();
}
