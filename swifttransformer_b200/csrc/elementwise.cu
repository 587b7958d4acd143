// Embedding lookup with learned positions, residual-add + normalisation,
// bias + activation, and small index utilities.
//
// Counterparts in the reference: embedding src/csrc/kernel/embedding.cu:16-35,
// LayerNorm with the fused residual add src/csrc/kernel/layernorm.cu:16-98,
// bias+activation src/csrc/kernel/fused_addbias_activ.cu:25-45, residual add
// src/csrc/kernel/addbias.cu:22-37, last-row gather src/csrc/kernel/gather_last_tokens.cu:23-37.
// Differences by design: sums, statistics and the residual stream are float for
// every storage type; the variance is two-pass; any width is accepted (widths
// that are a multiple of 4 take the vector path: four elements per access and
// several independent loads in flight per thread, which is what makes the
// kernels bandwidth- rather than latency-bound at decode batch sizes).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// VEC: width % 4 == 0.  src != nullptr: rows come from src[t] instead of table[ids[t]].
template <typename T, typename TO, bool VEC>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, const T* __restrict__ src,
                             int width, const int* __restrict__ pos, const T* __restrict__ pos_table,
                             int pos_offset, TO* __restrict__ out) {
    ST_PDL_WAIT();
    ST_PDL_TRIGGER();
    const int t = blockIdx.x;
    const T* row = src ? src + (size_t)t * width : table + (size_t)ids[t] * width;
    // a padding token of a fixed-shape step stands at position -1: it gets no position row (with an offset of
    // zero the row would lie before the table), and what is computed for it is never used
    const int p = pos_table ? pos[t] : 0;
    const T* prow = (pos_table && p >= 0) ? pos_table + (size_t)(p + pos_offset) * width : nullptr;
    TO* o = out + (size_t)t * width;
    if (VEC) {
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
            float4 v = src ? load4_cg(row + e) : load4(row + e);
            if (prow) v = add4(v, load4(prow + e));
            store4(o + e, v);
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            float v = src ? load1_cg(row + e) : to_f32(row[e]);
            if (prow) v += to_f32(prow[e]);
            o[e] = from_f32<TO>(v);
        }
    }
}

template <typename T, typename TO>
static int launch_embed(const int* ids, const void* table, const void* src, int n_tokens, int width, const int* pos,
                        const void* pos_table, int pos_offset, void* out, cudaStream_t s) {
    const bool vec = width % 4 == 0 && aligned16(table) && aligned16(src) && aligned16(pos_table) && aligned16(out);
    int block = vec ? (width / 4 + 31) / 32 * 32 : 256;
    if (block > 512) block = 512;
    if (block < 32) block = 32;
    if (vec)
        return st_launch_pdl("embed", embed_kernel<T, TO, true>, dim3(n_tokens), dim3(block), 0, s, ids, (const T*)table,
                             (const T*)src, width, pos, (const T*)pos_table, pos_offset, (TO*)out);
    return st_launch_pdl("embed", embed_kernel<T, TO, false>, dim3(n_tokens), dim3(block), 0, s, ids, (const T*)table,
                         (const T*)src, width, pos, (const T*)pos_table, pos_offset, (TO*)out);
}

// out[t] = table[ids[t]] (+ pos_table[pos[t] + pos_offset]);  out is float when out_f32, else the table's type
ST_EXPORT int st_embed(const int* ids, const void* table, int n_tokens, int width, const int* pos,
                       const void* pos_table, int pos_offset, void* out, int dtype, int out_f32, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0) return launch_embed<float, float>(ids, table, nullptr, n_tokens, width, pos, pos_table, pos_offset, out, s);
    if (dtype != 1) return ST_ERR_BAD_DTYPE;
    if (out_f32) return launch_embed<bf16, float>(ids, table, nullptr, n_tokens, width, pos, pos_table, pos_offset, out, s);
    return launch_embed<bf16, bf16>(ids, table, nullptr, n_tokens, width, pos, pos_table, pos_offset, out, s);
}

// out[t] = in[t] + pos_table[pos[t] + pos_offset]   (used after a project_in product)
ST_EXPORT int st_add_positions(const void* in, int n_tokens, int width, const int* pos, const void* pos_table,
                               int pos_offset, void* out, int dtype, int out_f32, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0) return launch_embed<float, float>(nullptr, nullptr, in, n_tokens, width, pos, pos_table, pos_offset, out, s);
    if (dtype != 1) return ST_ERR_BAD_DTYPE;
    if (out_f32) return launch_embed<bf16, float>(nullptr, nullptr, in, n_tokens, width, pos, pos_table, pos_offset, out, s);
    return launch_embed<bf16, bf16>(nullptr, nullptr, in, n_tokens, width, pos, pos_table, pos_offset, out, s);
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
// Further float addends of the residual sum: `n` tensors of the shape of x, `stride` elements apart (the slices of
// k a product was cut into leave their parts for the norm kernel to add, in slice order, instead of meeting in
// the product's own kernel).
struct AddParts {
    const float* p;
    int n;
    long long stride;
};

template <typename T, bool VEC>
__global__ void add_norm_kernel(const float* x, const int* __restrict__ rows,
                                const T* __restrict__ delta, const float* __restrict__ delta_bias, AddParts parts,
                                float* resid_out, const float* __restrict__ gamma,
                                const float* __restrict__ beta, float eps, int kind, int width,
                                T* __restrict__ out_act, float* out_f32) {
    extern __shared__ __align__(16) float srow[];
    __shared__ float scratch[32];
    // gain and shift of this thread's first two vectors are fetched before the wait for the kernel
    // before this one (no kernel writes them): at the end they would be one more round trip to memory
    float4 g_pre[2], b_pre[2];
    if (VEC && kind != 2) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int e = (threadIdx.x + j * blockDim.x) * 4;
            g_pre[j] = (gamma && e < width) ? load4(gamma + e) : make_float4(1.f, 1.f, 1.f, 1.f);
            b_pre[j] = (beta && e < width) ? load4(beta + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    ST_PDL_TRIGGER();       // before the wait: see add_norm_vec_kernel
    ST_PDL_WAIT();
    const int r = blockIdx.x;
    const size_t i = rows ? (size_t)rows[r] : (size_t)r;
    const float* xr = x + i * width;
    float sum = 0.f;
    if (VEC) {
        const int nvec = width >> 2;
        for (int v0 = threadIdx.x; v0 < nvec; v0 += blockDim.x * 2) {   // two independent sets of loads in flight
            const int v1 = v0 + blockDim.x;
            const bool two = v1 < nvec;
            float4 a = load4_cg(xr + v0 * 4), b = two ? load4_cg(xr + v1 * 4) : make_float4(0, 0, 0, 0);
            if (delta || parts.n) {
                float4 da = delta ? load4_cg(delta + i * width + v0 * 4) : make_float4(0, 0, 0, 0);
                float4 db = (delta && two) ? load4_cg(delta + i * width + v1 * 4) : make_float4(0, 0, 0, 0);
                for (int sl = 0; sl < parts.n; ++sl) {
                    da = add4(da, load4_cg(parts.p + sl * parts.stride + i * width + v0 * 4));
                    if (two) db = add4(db, load4_cg(parts.p + sl * parts.stride + i * width + v1 * 4));
                }
                a = add4(a, da);
                if (two) b = add4(b, db);
            }
            if (delta_bias) {
                a = add4(a, load4(delta_bias + v0 * 4));
                if (two) b = add4(b, load4(delta_bias + v1 * 4));
            }
            store4(srow + v0 * 4, a);
            sum += (a.x + a.y) + (a.z + a.w);
            if (two) {
                store4(srow + v1 * 4, b);
                sum += (b.x + b.y) + (b.z + b.w);
            }
            if (resid_out) {
                store4(resid_out + i * width + v0 * 4, a);
                if (two) store4(resid_out + i * width + v1 * 4, b);
            }
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            float v = load1_cg(xr + e);
            if (delta || parts.n) {
                float dv = delta ? load1_cg(delta + i * width + e) : 0.f;
                for (int sl = 0; sl < parts.n; ++sl) dv += load1_cg(parts.p + sl * parts.stride + i * width + e);
                v += dv;
            }
            if (delta_bias) v += delta_bias[e];
            srow[e] = v;
            sum += v;
            if (resid_out) resid_out[i * width + e] = v;
        }
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
        __syncthreads();
        float sq = 0.f;
        for (int e = threadIdx.x; e < width; e += blockDim.x) sq += srow[e] * srow[e];
        const float ms = block_sum(sq, scratch) / (float)width;
        rstd = 1.0f / sqrtf(ms + eps);
    } else {
        __syncthreads();
    }
    if (VEC) {
        int turn = 0;
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4, ++turn) {
            float4 y = load4(srow + e);
            if (kind != 2) {
                y = make_float4((y.x - mean) * rstd, (y.y - mean) * rstd, (y.z - mean) * rstd, (y.w - mean) * rstd);
                if (turn < 2) {
                    const float4 g = turn == 0 ? g_pre[0] : g_pre[1];
                    y = add4(make_float4(y.x * g.x, y.y * g.y, y.z * g.z, y.w * g.w), turn == 0 ? b_pre[0] : b_pre[1]);
                } else {
                    if (gamma) { const float4 g = load4(gamma + e); y = make_float4(y.x * g.x, y.y * g.y, y.z * g.z, y.w * g.w); }
                    if (beta) y = add4(y, load4(beta + e));
                }
            }
            if (out_act) store4(out_act + (size_t)r * width + e, y);
            if (out_f32) store4(out_f32 + (size_t)r * width + e, y);
        }
    } else {
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
}

// The vector form (width % 4 == 0): a row lives in its block's registers, VPT vectors of four per thread, and
// a block walks rows blockIdx.x, blockIdx.x + gridDim.x, ...  With VPT == 2 the next row is loaded while
// this one is reduced and written, so memory stays busy across the two block-wide reductions.  Gain, shift
// and the bias of delta are fetched once per block, before the wait for the kernel before this one (no
// kernel writes them).  Every row is computed by the same code in the same order whatever the number of
// rows: the result of a token does not depend on the batch.
template <typename T, int VPT, bool PARTS>
__global__ void __launch_bounds__(512, (VPT == 2 && !PARTS) ? 2 : 1) add_norm_vec_kernel(const float* x, const int* __restrict__ rows,
                                    const T* __restrict__ delta, const float* __restrict__ delta_bias, AddParts parts,
                                    float* resid_out, const float* __restrict__ gamma,
                                    const float* __restrict__ beta, float eps, int kind, int width, int n_rows,
                                    T* __restrict__ out_act, float* out_f32) {
    __shared__ float scratch[32];
    constexpr bool AHEAD = VPT == 2;
    const int nvec = width >> 2;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    bool ok[VPT];
    float4 g[VPT], b[VPT], db[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        ok[j] = v < nvec;
        g[j] = (kind != 2 && gamma && ok[j]) ? load4(gamma + 4 * v) : make_float4(1.f, 1.f, 1.f, 1.f);
        b[j] = (kind != 2 && beta && ok[j]) ? load4(beta + 4 * v) : zero4;
        db[j] = (delta_bias && ok[j]) ? load4(delta_bias + 4 * v) : zero4;
    }
    // The successor (a weight-streaming product in decode steps) may become resident before this kernel's own
    // dependency is met: what it does before its wait touches only memory that no kernel of the step writes,
    // and it brings its weights on chip meanwhile (OPT-1.3B decode step at batch 8: 1.121 -> 1.046 ms).  Its wait
    // still covers this kernel, and this kernel ends only after its own wait has returned.
    ST_PDL_TRIGGER();
    ST_PDL_WAIT();
    auto fetch = [&](int r, float4* xa, float4* da) -> size_t {
        const size_t i = rows ? (size_t)rows[r] : (size_t)r;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            xa[j] = ok[j] ? load4_cg(x + i * width + 4 * v) : zero4;
            da[j] = (delta && ok[j]) ? load4_cg(delta + i * width + 4 * v) : zero4;
            if constexpr (PARTS) {
                // all of a batch of four parts asked for before the first is added (one trip to L2 per batch, not per part)
                for (int s0 = 0; s0 < parts.n; s0 += 4) {
                    float4 pv[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        pv[u] = (ok[j] && s0 + u < parts.n) ? load4_cg(parts.p + (s0 + u) * parts.stride + i * width + 4 * v) : zero4;
#pragma unroll
                    for (int u = 0; u < 4; ++u) da[j] = add4(da[j], pv[u]);
                }
            }
        }
        return i;
    };
    float4 xa[VPT], da[VPT], xn[AHEAD ? VPT : 1], dn[AHEAD ? VPT : 1];
    int r = blockIdx.x;
    size_t i = 0, i_next = 0;
    if (AHEAD && r < n_rows) i = fetch(r, xa, da);
    for (; r < n_rows; r += gridDim.x) {
        if (AHEAD) {
            if (r + (int)gridDim.x < n_rows) i_next = fetch(r + gridDim.x, xn, dn);
        } else {
            i = fetch(r, xa, da);
        }
        float4 sv[VPT];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            sv[j] = add4(add4(xa[j], da[j]), db[j]);
            if (ok[j]) {
                sum += (sv[j].x + sv[j].y) + (sv[j].z + sv[j].w);
                if (resid_out) store4(resid_out + i * width + 4 * (threadIdx.x + j * blockDim.x), sv[j]);
            }
        }
        float mean = 0.f, rstd = 1.f;
        if (kind == 0) {
            mean = block_sum(sum, scratch) / (float)width;
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (ok[j]) {
                    const float d0 = sv[j].x - mean, d1 = sv[j].y - mean, d2 = sv[j].z - mean, d3 = sv[j].w - mean;
                    sq += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
                }
            }
            rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
        } else if (kind == 1) {
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (ok[j]) sq += (sv[j].x * sv[j].x + sv[j].y * sv[j].y) + (sv[j].z * sv[j].z + sv[j].w * sv[j].w);
            rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (!ok[j]) continue;
            float4 y = sv[j];
            if (kind != 2) {
                y = make_float4((y.x - mean) * rstd * g[j].x + b[j].x, (y.y - mean) * rstd * g[j].y + b[j].y,
                                (y.z - mean) * rstd * g[j].z + b[j].z, (y.w - mean) * rstd * g[j].w + b[j].w);
            }
            const size_t o = (size_t)r * width + 4 * (threadIdx.x + j * blockDim.x);
            if (out_act) store4(out_act + o, y);
            if (out_f32) store4(out_f32 + o, y);
        }
        if (AHEAD) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) { xa[j] = xn[j]; da[j] = dn[j]; }
            i = i_next;
        }
    }
}

template <typename T>
static int launch_add_norm(const float* x, const int* rows, const void* delta, const float* delta_bias, AddParts parts,
                           float* resid_out, const float* gamma, const float* beta, float eps, int kind, int n_rows,
                           int width, void* out_act, float* out_f32, cudaStream_t s) {
    const size_t smem = (size_t)width * sizeof(float);
    const bool vec = width % 4 == 0 && aligned16(x) && aligned16(delta) && aligned16(delta_bias) && aligned16(parts.p) &&
                     parts.stride % 4 == 0 &&
                     aligned16(resid_out) && aligned16(gamma) && aligned16(beta) && aligned16(out_act) &&
                     aligned16(out_f32);
    if (vec && width <= 8192) {
        // rows in registers: two vectors of four per thread up to 4096 wide, four beyond; a block takes several rows
        const int vpt = width <= 4096 ? 2 : 4;
        int block = (width / (4 * vpt) + 31) / 32 * 32;
        if (block < 64) block = 64;
        int grid = st_sm_count() * (vpt == 2 ? 4 : 2);
        if (grid > n_rows) grid = n_rows;
#define LAUNCH_VEC_NORM(VPT, PARTS)                                                                                          \
        return st_launch_pdl("norm", add_norm_vec_kernel<T, VPT, PARTS>, dim3(grid), dim3(block), 0, s, x, rows, (const T*)delta, \
                             delta_bias, parts, resid_out, gamma, beta, eps, kind, width, n_rows, (T*)out_act, out_f32)
        if (vpt == 2) { if (parts.n) LAUNCH_VEC_NORM(2, true); LAUNCH_VEC_NORM(2, false); }
        if (parts.n) LAUNCH_VEC_NORM(4, true);
        LAUNCH_VEC_NORM(4, false);
#undef LAUNCH_VEC_NORM
    }
    int block = vec ? (width / 8 + 31) / 32 * 32 : 256;   // vector path: two vectors per thread and round
    if (block > 512) block = 512;
    if (block < 64) block = 64;
    auto kern = vec ? add_norm_kernel<T, true> : add_norm_kernel<T, false>;
    if (smem > 40 * 1024) {     // with the kernel's static part past what a kernel may use without asking
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return st_launch_pdl("norm", kern, dim3(n_rows), dim3(block), smem, s, x, rows, (const T*)delta, delta_bias, parts, resid_out,
                         gamma, beta, eps, kind, width, (T*)out_act, out_f32);
}

// parts: n_parts further float addends [n_parts][rows of x][width], part_stride elements apart, or null / 0
ST_EXPORT int st_add_norm(const float* x, const int* rows, const void* delta, const float* delta_bias,
                          const float* parts, int n_parts, long long part_stride, float* resid_out, const float* gamma, const float* beta, float eps, int kind,
                          int n_rows, int width, void* out_act, float* out_f32, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (kind < 0 || kind > 2 || width <= 0) return ST_ERR_BAD_ARG;
    if ((size_t)width * sizeof(float) > 200 * 1024) return ST_ERR_TOO_LARGE;
    if (n_parts < 0 || n_parts > 16 || (n_parts > 0 && !parts)) return ST_ERR_BAD_ARG;
    const AddParts ap = {n_parts > 0 ? parts : nullptr, n_parts > 0 ? n_parts : 0, part_stride};
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0)
        return launch_add_norm<float>(x, rows, delta, delta_bias, ap, resid_out, gamma, beta, eps, kind, n_rows, width,
                                      out_act, out_f32, s);
    if (dtype == 1)
        return launch_add_norm<bf16>(x, rows, delta, delta_bias, ap, resid_out, gamma, beta, eps, kind, n_rows, width,
                                     out_act, out_f32, s);
    return ST_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------ bias + activation
template <typename T, bool VEC>
__global__ void bias_act_kernel(T* __restrict__ y, const float* __restrict__ bias, int act, size_t total, int width) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (VEC) {
        const size_t nvec = total >> 2;
        for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
            float4 a = load4(y + v * 4);
            if (bias) a = add4(a, load4(bias + (v * 4) % width));
            store4(y + v * 4, make_float4(apply_act(a.x, act), apply_act(a.y, act), apply_act(a.z, act), apply_act(a.w, act)));
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            float v = to_f32(y[i]);
            if (bias) v += bias[i % width];
            y[i] = from_f32<T>(apply_act(v, act));
        }
    }
}

ST_EXPORT int st_bias_act(void* y, const float* bias, int act, int n_rows, int width, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    const size_t total = (size_t)n_rows * width;
    const bool vec = width % 4 == 0 && aligned16(y) && aligned16(bias);
    const size_t work = vec ? total / 4 : total;
    int grid = (int)((work + 255) / 256);
    if (grid > st_sm_count() * 8) grid = st_sm_count() * 8;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == 0) {
        if (vec) bias_act_kernel<float, true><<<grid, 256, 0, s>>>((float*)y, bias, act, total, width);
        else bias_act_kernel<float, false><<<grid, 256, 0, s>>>((float*)y, bias, act, total, width);
    } else if (dtype == 1) {
        if (vec) bias_act_kernel<bf16, true><<<grid, 256, 0, s>>>((bf16*)y, bias, act, total, width);
        else bias_act_kernel<bf16, false><<<grid, 256, 0, s>>>((bf16*)y, bias, act, total, width);
    } else return ST_ERR_BAD_DTYPE;
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

// dst[i] = src[from[i]] where from[i] >= 0: tokens that the previous step sampled become this step's
// inputs without a trip through the host.
__global__ void gather_where_i32_kernel(int* __restrict__ dst, const int* __restrict__ from,
                                        const int* __restrict__ src, int n, int n_src) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int f = from[i];
    if (f >= 0 && f < n_src) dst[i] = src[f];
}

ST_EXPORT int st_gather_where_i32(int* dst, const int* from, const int* src, int n, int n_src, void* stream) {
    if (n <= 0) return 0;
    gather_where_i32_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(dst, from, src, n, n_src);
    return st_launch_status();
}

ST_EXPORT int st_scatter_i32(int* dst, const int* idx, const int* val, const int* count, int max_count, void* stream) {
    if (max_count <= 0) return 0;
    int grid = (max_count + 255) / 256;
    if (grid > 64) grid = 64;
    scatter_i32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(dst, idx, val, count);
    return st_launch_status();
}
