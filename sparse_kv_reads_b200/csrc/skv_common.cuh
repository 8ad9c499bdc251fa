// Shared device helpers for the sm_100a kernels of the clustered sparse KV-cache attention library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "skv.h"

namespace skv {

constexpr float NEG_BIG = -1.0e30f;      // finite stand-in for -inf in running maxima (no NaN from inf - inf)
constexpr int HEAD_DIM = 128;            // the only head dimension the kernels are built for
constexpr float LOG2E = 1.4426950408889634f;

// last CUDA error seen by an entry point (host side)
extern thread_local cudaError_t g_last_cuda_error;

#define SKV_CUDA_OK(expr)                         \
    do {                                          \
        cudaError_t e__ = (expr);                 \
        if (e__ != cudaSuccess) {                 \
            skv::g_last_cuda_error = e__;         \
            return SKV_E_CUDA;                    \
        }                                         \
    } while (0)

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int device_sm_count();
int device_max_smem_optin();
bool pdl_enabled();

// Programmatic dependent launch.  A kernel launched through launch_pdl may start while the kernel before it
// on the stream is still running; everything it reads from that kernel (and every write it makes) must come
// after pdl_wait(), which returns once the earlier kernel has completed and its writes are visible.  What it
// does before the wait - loading data no kernel of the same step writes - overlaps the earlier kernel's tail.
// pdl_trigger() in the earlier kernel allows the later one to be scheduled; without it the later kernel
// starts when the earlier one ends, as in a plain launch.  Every kernel launched this way executes
// pdl_wait() before it finishes, so that completion stays transitive along the stream.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Cached positions of head `head`: runs of `n_group` consecutive heads share one entry of n_dev (a batch whose
// sequences differ in length: n_group = KV heads per sequence); n_group 0 = every head reads n_dev[0].
__device__ __forceinline__ int positions_of(const int32_t *n_dev, int n_group, int head) {
    return n_dev[n_group > 0 ? head / n_group : 0];
}

// ---------------------------------------------------------------------------------------------
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
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide sum; `red` is shared scratch of >= 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float *red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Exclusive block scan of one int per thread; returns this thread's offset, `total` to all threads.
// `red` is shared scratch of >= 33 ints.
__device__ __forceinline__ int block_excl_scan(int v, int *red, int &total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) red[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int w = (lane < nw) ? red[lane] : 0;
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        red[lane] = winc - w;                 // exclusive offset of each warp
        if (lane == 31) red[32] = winc;       // grand total
    }
    __syncthreads();
    total = red[32];
    return red[wid] + inc - v;
}

// 16-byte asynchronous global->shared copy; src_bytes = 0 writes zeros instead of reading.
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, int src_bytes) {
    unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gsrc), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ float load_as_float(const float *p) { return *p; }
__device__ __forceinline__ float load_as_float(const __nv_bfloat16 *p) { return __bfloat162float(*p); }

// Eight consecutive elements starting at p (16-byte aligned for bf16, 32-byte for float) as floats.
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4 *>(p);
    float4 b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Four consecutive elements (one lane's share of a 128-wide row spread over a warp) as floats.
__device__ __forceinline__ float4 load4(const __nv_bfloat16 *p) {
    uint2 u = *reinterpret_cast<const uint2 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
    float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 load4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

__device__ __forceinline__ void store_out(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_out(__nv_bfloat16 *p, float v) { *p = __float2bfloat16(v); }

// 8-bit copy of one component of a unit vector: floor(u * 127 + 0.5).
__device__ __forceinline__ int8_t quant8(float u) { return static_cast<int8_t>(floorf(u * 127.0f + 0.5f)); }

// Order-preserving map float -> uint32 (larger float <=> larger key).
__device__ __forceinline__ uint32_t float_key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

}  // namespace skv
