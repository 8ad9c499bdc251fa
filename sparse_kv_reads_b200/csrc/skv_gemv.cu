// Matrix-vector products of the single-token (decode) forward, bf16 weights [N, K] row-major, up to eight
// sequences at once, fp32 accumulation.  A decode GEMV is pure weight streaming (2 flop per weight byte
// pair), so the kernel is built for HBM bandwidth: 16-byte loads, several rows per warp in flight, the
// activation vector staged once per CTA in shared memory.  Two fusions remove launches around it:
//   NORM  - the activation is RMSNorm(h + delta) * w computed in the prologue (every CTA redoes this tiny
//           reduction; CTA 0 also stores the new residual stream), replacing a separate add + norm launch;
//   GATED - rows n and n + N are a gate/up pair and the output is silu(gate) * up, replacing a launch.
#include "skv_common.cuh"

namespace skv {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = GV_THREADS / 32;
constexpr int GV_ROWS = 2;               // output rows (or gate/up pairs) per warp per step
constexpr int GV_BMAX = 8;

struct GemvParams {
    const __nv_bfloat16 *W;      // [N or 2N, K]
    const __nv_bfloat16 *x;      // [B, K] (plain) or residual stream h [B, K] (NORM)
    const __nv_bfloat16 *delta;  // [B, K] or null (NORM)
    const __nv_bfloat16 *norm_w; // [K] (NORM)
    __nv_bfloat16 *h_out;        // [B, K] new residual stream (NORM; may alias nothing that is read)
    __nv_bfloat16 *y;            // [B, N]
    int B, N, K;
    float eps;
};

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16(v)); }

template <bool NORM, bool GATED>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) float xs[];          // [B][K]
    __shared__ float red[32];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int K = p.K, B = p.B, vecs = K >> 3;
    // ---- activation vector into shared memory ------------------------------------------------------------
    for (int b = 0; b < B; ++b) {
        float ss = 0.f;
        for (int v = tid; v < vecs; v += GV_THREADS) {
            float a[8];
            load8(p.x + (int64_t)b * K + v * 8, a);
            if (NORM) {
                if (p.delta) {
                    float dl[8];
                    load8(p.delta + (int64_t)b * K + v * 8, dl);
#pragma unroll
                    for (int i = 0; i < 8; ++i) a[i] = bf16r(a[i] + dl[i]);
                }
                if (blockIdx.x == 0) {
                    __align__(16) __nv_bfloat16 o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16(a[i]);
                    *reinterpret_cast<uint4 *>(p.h_out + (int64_t)b * K + v * 8) = *reinterpret_cast<const uint4 *>(o);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(a[i], a[i], ss);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) xs[b * K + v * 8 + i] = a[i];
        }
        if (NORM) {
            const float inv = rsqrtf(block_sum(ss, red) / (float)K + p.eps);
            for (int v = tid; v < vecs; v += GV_THREADS) {
                float g[8];
                load8(p.norm_w + v * 8, g);
#pragma unroll
                for (int i = 0; i < 8; ++i) xs[b * K + v * 8 + i] = bf16r(xs[b * K + v * 8 + i] * inv * g[i]);
            }
        }
    }
    __syncthreads();
    // ---- rows ----------------------------------------------------------------------------------------
    const int N = p.N;
    constexpr int NW = GATED ? 2 * GV_ROWS : GV_ROWS;    // weight rows streamed together by a warp
    for (int r0 = (blockIdx.x * GV_WARPS + wid) * GV_ROWS; r0 < N; r0 += gridDim.x * GV_WARPS * GV_ROWS) {
        float acc[NW][GV_BMAX];
#pragma unroll
        for (int j = 0; j < NW; ++j)
#pragma unroll
            for (int b = 0; b < GV_BMAX; ++b) acc[j][b] = 0.f;
        const __nv_bfloat16 *rows[NW];
#pragma unroll
        for (int j = 0; j < NW; ++j) {
            const int r = r0 + (j % GV_ROWS) + (GATED && j >= GV_ROWS ? N : 0);
            rows[j] = p.W + (int64_t)min(r, (GATED ? 2 * N : N) - 1) * K;
        }
#pragma unroll 2
        for (int v = lane; v < vecs; v += 32) {
            uint4 w[NW];
#pragma unroll
            for (int j = 0; j < NW; ++j) w[j] = __ldg(reinterpret_cast<const uint4 *>(rows[j] + v * 8));
#pragma unroll
            for (int b = 0; b < GV_BMAX; ++b) {
                if (b < B) {
                    const float4 x0 = *reinterpret_cast<const float4 *>(xs + b * K + v * 8);
                    const float4 x1 = *reinterpret_cast<const float4 *>(xs + b * K + v * 8 + 4);
#pragma unroll
                    for (int j = 0; j < NW; ++j) {
                        const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&w[j]);
                        const float2 a = __bfloat1622float2(h2[0]), bq = __bfloat1622float2(h2[1]);
                        const float2 c = __bfloat1622float2(h2[2]), dq = __bfloat1622float2(h2[3]);
                        float s = acc[j][b];
                        s = fmaf(a.x, x0.x, s); s = fmaf(a.y, x0.y, s); s = fmaf(bq.x, x0.z, s); s = fmaf(bq.y, x0.w, s);
                        s = fmaf(c.x, x1.x, s); s = fmaf(c.y, x1.y, s); s = fmaf(dq.x, x1.z, s); s = fmaf(dq.y, x1.w, s);
                        acc[j][b] = s;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NW; ++j)
#pragma unroll
            for (int b = 0; b < GV_BMAX; ++b)
                if (b < B) acc[j][b] = warp_sum(acc[j][b]);
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < GV_ROWS; ++j) {
                const int r = r0 + j;
                if (r < N)
#pragma unroll
                    for (int b = 0; b < GV_BMAX; ++b)
                        if (b < B) {
                            float out = acc[j][b];
                            if (GATED) {
                                const float g = bf16r(out), u = bf16r(acc[j + GV_ROWS][b]);   // both are bf16 tensors unfused
                                out = bf16r(g / (1.f + __expf(-g))) * u;
                            }
                            p.y[(int64_t)b * N + r] = __float2bfloat16(out);
                        }
            }
        }
    }
}

template <bool NORM, bool GATED>
static int launch_gemv(const GemvParams &p, cudaStream_t st) {
    auto kern = gemv_kernel<NORM, GATED>;
    const size_t smem = (size_t)p.B * p.K * 4;
    static size_t configured[64] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (smem > 48 * 1024 && configured[dev] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = smem;
    }
    const int per_cta = GV_WARPS * GV_ROWS;
    int ctas = (p.N + per_cta - 1) / per_cta;
    const int cap = 8 * device_sm_count();                 // longer rows-per-CTA loops beyond eight CTAs per SM
    if (ctas > cap) ctas = cap;
    kern<<<ctas, GV_THREADS, smem, st>>>(p);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

}  // namespace skv

using namespace skv;

extern "C" int skv_gemv(const void *W, const void *x, void *y, int B, int N, int K, void *stream) {
    if (!W || !x || !y) return SKV_E_NULL;
    if (B < 1 || B > GV_BMAX || N < 1 || K < 8 || K % 8) return SKV_E_RANGE;
    if ((size_t)B * K * 4 > (size_t)device_max_smem_optin() - 1024) return SKV_E_RANGE;
    if (!aligned16(W) || !aligned16(x)) return SKV_E_ALIGN;
    GemvParams p{static_cast<const __nv_bfloat16 *>(W), static_cast<const __nv_bfloat16 *>(x), nullptr, nullptr, nullptr,
                 static_cast<__nv_bfloat16 *>(y), B, N, K, 0.f};
    return launch_gemv<false, false>(p, static_cast<cudaStream_t>(stream));
}

extern "C" int skv_norm_gemv(const void *W, const void *h, const void *delta, const void *norm_w, void *h_out, void *y,
                             int B, int N, int K, float eps, int gated, void *stream) {
    if (!W || !h || !norm_w || !h_out || !y) return SKV_E_NULL;
    if (B < 1 || B > GV_BMAX || N < 1 || K < 8 || K % 8) return SKV_E_RANGE;
    if ((size_t)B * K * 4 > (size_t)device_max_smem_optin() - 1024) return SKV_E_RANGE;
    if (!aligned16(W) || !aligned16(h) || !aligned16(norm_w) || !aligned16(h_out) || (delta && !aligned16(delta)))
        return SKV_E_ALIGN;
    if (h_out == h || h_out == delta) return SKV_E_RANGE;        // other CTAs still read the old stream
    GemvParams p{static_cast<const __nv_bfloat16 *>(W), static_cast<const __nv_bfloat16 *>(h),
                 static_cast<const __nv_bfloat16 *>(delta), static_cast<const __nv_bfloat16 *>(norm_w),
                 static_cast<__nv_bfloat16 *>(h_out), static_cast<__nv_bfloat16 *>(y), B, N, K, eps};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return gated ? launch_gemv<true, true>(p, st) : launch_gemv<true, false>(p, st);
}
