// Matrix-vector products of the single-token (decode) forward: y[B, N] = x[B, K] . W[N, K]^T for a handful of
// sequences (B <= 8), bf16 in and out, float32 accumulation.  The weights are read exactly once, so the
// product is bound by HBM; what decides its speed at this size is how early the bytes are requested.
//
// A CTA owns a run of consecutive rows of W - one contiguous slab of memory, at most 96 KB - and asks for all
// of it with 16-byte asynchronous copies into shared memory as its very first action.  Under programmatic
// dependent launch that happens while the kernel ahead on the stream is still finishing: weights are written by
// no kernel, so they may be fetched before the wait, and only the input vector has to wait for the producer.
// The input is then built in shared memory in one of three ways, each CTA for itself (it is a few KB, read
// from L2), which folds the element-wise kernels between the products into them:
//   mode 0  x as given;
//   mode 1  residual add and RMSNorm: h_out = bf16(h_in + delta), x = bf16(h_out * rsqrt(mean(h_out^2) + eps) * g)
//           (CTA 0 also stores h_out, out of place because the other CTAs still read h_in);
//   mode 2  x = bf16(bf16(silu(gate)) * up) from gate_up[B, 2K].
// The roundings are those of the separate kernels (skv_dense.cu) and of the unfused module forward.
// Warp w of the CTA then takes rows w, w + 8, ... of the slab: a lane multiplies 16-byte pieces of the row with
// the matching pieces of every sequence's input, and the warp reduces the B sums.
#include "skv_common.cuh"

namespace skv {

constexpr int GEMV_THREADS = 256, GEMV_WARPS = 8;
constexpr int GEMV_SLAB_MAX = 96 * 1024;

struct GemvParams {
    const __nv_bfloat16 *W;
    __nv_bfloat16 *y;
    int N, K, B, mode, rows_per_cta;
    const __nv_bfloat16 *x;        // mode 0: [B, K]; mode 2: gate_up [B, 2K]
    const __nv_bfloat16 *h_in, *delta, *g;
    __nv_bfloat16 *h_out;
    float eps;
};

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16(x)); }

template <int BP>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float s_part[8][GEMV_WARPS];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int K = p.K, kv = K >> 3;                         // 16-byte pieces per row
    const int r0 = blockIdx.x * p.rows_per_cta;
    const int R = min(p.rows_per_cta, p.N - r0);
    __nv_bfloat16 *ws = reinterpret_cast<__nv_bfloat16 *>(smem);                      // [rows_per_cta][K]
    __nv_bfloat16 *xs = ws + (size_t)p.rows_per_cta * K;                              // [BP][K]
    __nv_bfloat16 *gs = xs + (size_t)BP * K;                                          // [K] (mode 1)

    // 1. the slab (and the norm weights): requested before anything else, also before the producer ends
    {
        if (p.mode == 1)
            for (int c = tid; c < kv; c += GEMV_THREADS) cp_async16(gs + c * 8, p.g + c * 8, 16);
        cp_async_commit();                                  // group 0: norm weights (empty otherwise)
        const __nv_bfloat16 *src = p.W + (size_t)r0 * K;
        const int pieces = R * kv;
        for (int c = tid; c < pieces; c += GEMV_THREADS) cp_async16(ws + (size_t)c * 8, src + (size_t)c * 8, 16);
        cp_async_commit();                                  // group 1: the slab
    }
    pdl_wait();
    pdl_trigger();

    // 2. the input of every sequence, in shared memory as bf16
    if (p.mode == 0) {
        for (int c = tid; c < BP * kv; c += GEMV_THREADS) {
            const int b = c / kv, v = c - b * kv;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (b < p.B) val = __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)b * K + v * 8));
            *reinterpret_cast<uint4 *>(xs + (size_t)b * K + v * 8) = val;
        }
    } else if (p.mode == 2) {
        for (int c = tid; c < BP * kv; c += GEMV_THREADS) {
            const int b = c / kv, v = c - b * kv;
            __align__(16) __nv_bfloat16 o[8];
            if (b < p.B) {
                float g[8], u[8];
                load8(p.x + (size_t)b * 2 * K + v * 8, g);
                load8(p.x + (size_t)b * 2 * K + K + v * 8, u);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(bf16r(g[k] / (1.f + __expf(-g[k]))) * u[k]);
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(0.f);
            }
            *reinterpret_cast<uint4 *>(xs + (size_t)b * K + v * 8) = *reinterpret_cast<const uint4 *>(o);
        }
    } else {
        // BP sequences share the 8 warps: wpr warps per sequence, each a contiguous range of the row
        constexpr int wpr = GEMV_WARPS / BP;
        const int b = wid / wpr, sub = wid % wpr;
        const int per = (kv + wpr - 1) / wpr;
        const int v0 = min(sub * per, kv), v1 = min(v0 + per, kv);
        float ss = 0.f;
        if (b < p.B) {
            const __nv_bfloat16 *hr = p.h_in + (size_t)b * K;
            const __nv_bfloat16 *dr = p.delta ? p.delta + (size_t)b * K : nullptr;
            for (int v = v0 + lane; v < v1; v += 32) {
                float a[8];
                load8(hr + v * 8, a);
                __align__(16) __nv_bfloat16 o[8];
                if (dr) {
                    float d[8];
                    load8(dr + v * 8, d);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        o[i] = __float2bfloat16(a[i] + d[i]);
                        a[i] = __bfloat162float(o[i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16(a[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(a[i], a[i], ss);
                *reinterpret_cast<uint4 *>(xs + (size_t)b * K + v * 8) = *reinterpret_cast<const uint4 *>(o);
                if (blockIdx.x == 0 && p.h_out)
                    *reinterpret_cast<uint4 *>(p.h_out + (size_t)b * K + v * 8) = *reinterpret_cast<const uint4 *>(o);
            }
        } else if (b < BP) {
            for (int v = v0 + lane; v < v1; v += 32) *reinterpret_cast<uint4 *>(xs + (size_t)b * K + v * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        ss = warp_sum(ss);
        if (lane == 0) s_part[wid / wpr][sub] = ss;
        cp_async_wait<1>();                                 // the norm weights have landed
        __syncthreads();
        if (b < p.B) {
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < wpr; ++i) tot += s_part[b][i];
            const float inv = rsqrtf(tot / (float)K + p.eps);
            for (int v = v0 + lane; v < v1; v += 32) {
                float a[8], g[8];
                load8(xs + (size_t)b * K + v * 8, a);
                load8(gs + v * 8, g);
                __align__(16) __nv_bfloat16 o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16(a[i] * inv * g[i]);
                *reinterpret_cast<uint4 *>(xs + (size_t)b * K + v * 8) = *reinterpret_cast<const uint4 *>(o);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // 3. rows of the slab
    for (int r = wid; r < R; r += GEMV_WARPS) {
        float acc[BP];
#pragma unroll
        for (int b = 0; b < BP; ++b) acc[b] = 0.f;
        const __nv_bfloat16 *wr = ws + (size_t)r * K;
#pragma unroll 2
        for (int v = lane; v < kv; v += 32) {
            float w[8];
            load8(wr + v * 8, w);
#pragma unroll
            for (int b = 0; b < BP; ++b) {
                float xv[8];
                load8(xs + (size_t)b * K + v * 8, xv);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[b] = fmaf(w[i], xv[i], acc[b]);
            }
        }
#pragma unroll
        for (int b = 0; b < BP; ++b) {
            const float s = warp_sum(acc[b]);
            if (lane == 0 && b < p.B) p.y[(size_t)b * p.N + r0 + r] = __float2bfloat16(s);
        }
    }
}

}  // namespace skv

using namespace skv;

extern "C" int skv_gemv(const void *W, int N, int K, void *y, int B, int mode, const void *x, const void *h_in,
                        const void *delta, const void *norm_w, void *h_out, float eps, void *stream) {
    if (!W || !y) return SKV_E_NULL;
    if (mode < 0 || mode > 2) return SKV_E_RANGE;
    if (mode == 1 ? (!h_in || !norm_w) : !x) return SKV_E_NULL;
    if (B < 1 || B > 8 || N < 1 || K < 8 || K % 8) return SKV_E_RANGE;
    if (!aligned16(W) || !aligned16(y) || (x && !aligned16(x)) || (h_in && !aligned16(h_in)) ||
        (delta && !aligned16(delta)) || (norm_w && !aligned16(norm_w)) || (h_out && !aligned16(h_out)))
        return SKV_E_ALIGN;
    const int BP = B <= 1 ? 1 : (B <= 2 ? 2 : (B <= 4 ? 4 : 8));
    const size_t row = (size_t)K * 2;
    if (row > (size_t)GEMV_SLAB_MAX) return SKV_E_TOO_LARGE;
    // one wave of CTAs where the slab allows it, else slabs of the largest size (two of them share an SM)
    int rows = (N + device_sm_count() - 1) / device_sm_count();
    const int fit = (int)(GEMV_SLAB_MAX / row);
    if (rows > fit) rows = fit;
    const size_t smem = (size_t)rows * row + (size_t)BP * row + (mode == 1 ? row : 0);
    if (smem > (size_t)device_max_smem_optin()) return SKV_E_TOO_LARGE;
    GemvParams p;
    p.W = static_cast<const __nv_bfloat16 *>(W); p.y = static_cast<__nv_bfloat16 *>(y);
    p.N = N; p.K = K; p.B = B; p.mode = mode; p.rows_per_cta = rows;
    p.x = static_cast<const __nv_bfloat16 *>(x); p.h_in = static_cast<const __nv_bfloat16 *>(h_in);
    p.delta = static_cast<const __nv_bfloat16 *>(delta); p.g = static_cast<const __nv_bfloat16 *>(norm_w);
    p.h_out = static_cast<__nv_bfloat16 *>(h_out); p.eps = eps;
    typedef void (*Kern)(const GemvParams);
    const int bi = BP == 1 ? 0 : (BP == 2 ? 1 : (BP == 4 ? 2 : 3));
    const Kern table[4] = {gemv_kernel<1>, gemv_kernel<2>, gemv_kernel<4>, gemv_kernel<8>};
    static size_t configured[64][4] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (configured[dev][bi] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(table[bi], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][bi] = smem;
    }
    const int ctas = (N + rows - 1) / rows;
    SKV_CUDA_OK(launch_pdl(table[bi], dim3(ctas), dim3(GEMV_THREADS), smem, static_cast<cudaStream_t>(stream), p));
    return SKV_OK;
}
