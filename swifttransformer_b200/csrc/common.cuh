// Shared device helpers for the sm_100a kernels of this engine.
//
// Conventions of every exported launcher (extern "C", called through ctypes):
//   * pointers are device pointers, `stream` is a cudaStream_t passed as void*;
//   * `dtype` selects the storage type of activations / matrices: 0 = float,
//     1 = __nv_bfloat16.  Vectors (biases, norm weights) are always float;
//   * the return value is 0 on success, a positive cudaError_t from the launch,
//     or a negative ST_ERR_* code for arguments the kernel refuses.  Nothing is
//     ever computed wrongly for an unsupported size: it is refused.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ST_ERR_BAD_DTYPE (-1)
#define ST_ERR_BAD_SIZE (-2)
#define ST_ERR_TOO_LARGE (-3)
#define ST_ERR_BAD_ARG (-4)

#define ST_EXPORT extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// four consecutive elements as float, for either storage type (16- resp. 8-byte accesses)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
// the same through L2 only (see the note on programmatic dependent launch below): for data that the
// kernel just before may have written while this block was already resident
__device__ __forceinline__ float4 load4_cg(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4_cg(const bf16* p) {
    const uint2 u = __ldcg(reinterpret_cast<const uint2*>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float load1_cg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float load1_cg(const bf16* p) {
    return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    uint2 u;
    *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide reductions with a fixed order (xor butterflies inside a warp, then
// the warp partials combined in warp-index order by every thread), so the
// result is the same bit pattern in every thread and on every launch.
// `scratch` holds at least 32 floats; the call ends with the scratch free for reuse.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < nwarp; ++i) r += scratch[i];
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
    for (int i = 1; i < nwarp; ++i) r = fmaxf(r, scratch[i]);
    return r;
}

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == 1) return v > 0.f ? v : 0.f;                                // relu
    if (act == 2) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));  // gelu (erf form)
    return v;
}

static inline int st_launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch ---------------------------------------
// Kernels of a decode step are short and depend on one another; launched this
// way, a kernel's blocks may become resident while its predecessor in the
// stream is still running.  A kernel launched so must execute ST_PDL_WAIT()
// before it reads anything its predecessors write and before it writes
// anything at all; what comes before the wait may only touch memory that no
// kernel writes (weights).  After the wait every predecessor has finished and
// its writes are visible.  ST_PDL_TRIGGER() lets the successor's blocks be
// scheduled as soon as there is room.  In a kernel that is launched the plain
// way both are no-ops.  ST_B200_NO_PDL=1 in the environment turns the launch
// attribute off.
#include <stdlib.h>
#include <utility>
#define ST_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
#define ST_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")

#include <string.h>
// ST_B200_NO_PDL=1 turns the attribute off for every kernel; ST_B200_PDL_ONLY=a,b limits it to the
// kernels whose tag is listed (for finding a kernel that breaks the rules above).
// The environment is read once, at the first launch.
static inline bool st_pdl_enabled(const char* tag) {
    static const char* const off = getenv("ST_B200_NO_PDL");
    static const char* const only = getenv("ST_B200_PDL_ONLY");
    if (off && off[0] && off[0] != '0') return false;
    if (only && only[0]) return strstr(only, tag) != nullptr;
    return true;
}

// Streaming multiprocessors of the current device (asked once per device).
static inline int st_sm_count() {
    static int count[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!count[dev]) {
        int n = 0;
        count[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    return count[dev];
}

// Page numbers one block of the single-token attention kernels keeps in shared memory: those of its own
// part of the key range (the whole range, or a window of it, cut into n_splits parts rounded up to 16 keys),
// not of the longest request the block table has room for.
static inline int st_decode_block_pages(int max_pages, int page_size, int window, int n_splits) {
    long long span = (long long)max_pages * page_size;
    if (window > 0 && window < span) span = window;
    long long per = (span + n_splits - 1) / n_splits;
    per = (per + 15) / 16 * 16;
    const long long pages = per / page_size + 2;
    return (int)(pages < max_pages ? pages : max_pages);
}

template <typename... KArgs, typename... Args>
static inline int st_launch_pdl(const char* tag, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = st_pdl_enabled(tag) ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return st_launch_status();
}
