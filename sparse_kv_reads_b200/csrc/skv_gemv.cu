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

// A CTA owns GV_R weight rows (GATED: GV_R / 2 gate rows and their up rows) and all its threads split the
// K dimension of those rows: item i = (row, 8-element chunk), thread t takes items t, t + 256, ...  The
// 16-byte weight loads of the first items are requested before the activation prologue, so the prologue's
// latency chain (load, reduce, normalise) hides behind the weight stream.  Each warp's 32 items lie in one
// row (K is a multiple of 256), so an item step ends in one warp reduction; the per-warp partial sums are
// combined per row in a fixed order.
constexpr int GV_R = 4;
constexpr int GV_IT = 8;                 // items a thread holds in flight

template <bool NORM, bool GATED>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) float xs[];          // [B][K], then partial sums [B][items / 32]
    __shared__ float red[32];
    const int tid = threadIdx.x, lane = tid & 31;
    const int K = p.K, B = p.B, vecs = K >> 3, N = p.N;
    const int items = GV_R * vecs;
    float *part = xs + (size_t)B * K;
    constexpr int OUT_R = GATED ? GV_R / 2 : GV_R;       // output rows per CTA
    const int r_base = blockIdx.x * OUT_R;
    auto row_ptr = [&](int lr) {                         // weight row of local row lr
        int r = GATED ? r_base + (lr % OUT_R) + (lr >= OUT_R ? N : 0) : r_base + lr;
        r = min(r, (GATED ? 2 * N : N) - 1);
        return p.W + (int64_t)r * K;
    };
    uint4 w[GV_IT];
#pragma unroll
    for (int j = 0; j < GV_IT; ++j) {
        const int i = tid + j * GV_THREADS;
        w[j] = make_uint4(0u, 0u, 0u, 0u);
        if (i < items) w[j] = __ldg(reinterpret_cast<const uint4 *>(row_ptr(i / vecs) + (i % vecs) * 8));
    }
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
                float g[8];
                load8(p.norm_w + v * 8, g);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    ss = fmaf(a[i], a[i], ss);
                    a[i] *= g[i];                        // the 1/rms factor is applied after the reduction
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) xs[b * K + v * 8 + i] = a[i];
        }
        if (NORM) {
            const float inv = rsqrtf(block_sum(ss, red) / (float)K + p.eps);
            if (tid == 0) part[(size_t)B * (items >> 5) + b] = inv;
        }
    }
    __syncthreads();
    // ---- items ---------------------------------------------------------------------------------------
    for (int i0 = 0; i0 < items; i0 += GV_IT * GV_THREADS) {
        if (i0) {
#pragma unroll
            for (int j = 0; j < GV_IT; ++j) {
                const int i = i0 + tid + j * GV_THREADS;
                w[j] = make_uint4(0u, 0u, 0u, 0u);
                if (i < items) w[j] = __ldg(reinterpret_cast<const uint4 *>(row_ptr(i / vecs) + (i % vecs) * 8));
            }
        }
#pragma unroll
        for (int j = 0; j < GV_IT; ++j) {
            const int i = i0 + tid + j * GV_THREADS;
            if (i - lane >= items) continue;             // warp-uniform
            const int chunk = i % vecs;
            const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&w[j]);
            const float2 a = __bfloat1622float2(h2[0]), bq = __bfloat1622float2(h2[1]);
            const float2 c = __bfloat1622float2(h2[2]), dq = __bfloat1622float2(h2[3]);
            for (int b = 0; b < B; ++b) {
                const float4 x0 = *reinterpret_cast<const float4 *>(xs + b * K + chunk * 8);
                const float4 x1 = *reinterpret_cast<const float4 *>(xs + b * K + chunk * 8 + 4);
                float s = a.x * x0.x;
                s = fmaf(a.y, x0.y, s); s = fmaf(bq.x, x0.z, s); s = fmaf(bq.y, x0.w, s);
                s = fmaf(c.x, x1.x, s); s = fmaf(c.y, x1.y, s); s = fmaf(dq.x, x1.z, s); s = fmaf(dq.y, x1.w, s);
                s = warp_sum(s);
                if (lane == 0) part[b * (items >> 5) + (i >> 5)] = s;
            }
        }
    }
    __syncthreads();
    // ---- rows: partial sums in order, 1/rms, bf16 rounding as the unfused forward, activation ---------------
    const int ppr = vecs >> 5;                           // partials per weight row
    for (int t = tid; t < B * OUT_R; t += GV_THREADS) {
        const int b = t / OUT_R, lr = t % OUT_R, r = r_base + lr;
        if (r >= N) continue;
        float s0 = 0.f, s1 = 0.f;
        for (int k = 0; k < ppr; ++k) s0 += part[b * (items >> 5) + lr * ppr + k];
        if (GATED)
            for (int k = 0; k < ppr; ++k) s1 += part[b * (items >> 5) + (lr + OUT_R) * ppr + k];
        const float inv = NORM ? part[(size_t)B * (items >> 5) + b] : 1.f;     // 1/rms of sequence b
        float out = s0 * inv;
        if (GATED) {
            const float g = bf16r(out), u = bf16r(s1 * inv);
            out = bf16r(g / (1.f + __expf(-g))) * u;
        }
        p.y[(int64_t)b * N + r] = __float2bfloat16(out);
    }
}

template <bool NORM, bool GATED>
static int launch_gemv(const GemvParams &p, cudaStream_t st) {
    auto kern = gemv_kernel<NORM, GATED>;
    const int items = GV_R * (p.K >> 3);
    const size_t smem = ((size_t)p.B * p.K + (size_t)p.B * (items >> 5) + GV_BMAX) * 4;
    static size_t configured[64] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (smem > 48 * 1024 && configured[dev] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = smem;
    }
    const int out_r = GATED ? GV_R / 2 : GV_R;
    kern<<<(p.N + out_r - 1) / out_r, GV_THREADS, smem, st>>>(p);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

}  // namespace skv

using namespace skv;

extern "C" int skv_gemv(const void *W, const void *x, void *y, int B, int N, int K, void *stream) {
    if (!W || !x || !y) return SKV_E_NULL;
    if (B < 1 || B > GV_BMAX || N < 1 || K < 256 || K % 256) return SKV_E_RANGE;
    if ((size_t)B * (K + K / 64 + 8) * 4 > (size_t)device_max_smem_optin() - 1024) return SKV_E_RANGE;
    if (!aligned16(W) || !aligned16(x)) return SKV_E_ALIGN;
    GemvParams p{static_cast<const __nv_bfloat16 *>(W), static_cast<const __nv_bfloat16 *>(x), nullptr, nullptr, nullptr,
                 static_cast<__nv_bfloat16 *>(y), B, N, K, 0.f};
    return launch_gemv<false, false>(p, static_cast<cudaStream_t>(stream));
}

extern "C" int skv_norm_gemv(const void *W, const void *h, const void *delta, const void *norm_w, void *h_out, void *y,
                             int B, int N, int K, float eps, int gated, void *stream) {
    if (!W || !h || !norm_w || !h_out || !y) return SKV_E_NULL;
    if (B < 1 || B > GV_BMAX || N < 1 || K < 256 || K % 256) return SKV_E_RANGE;
    if ((size_t)B * (K + K / 64 + 8) * 4 > (size_t)device_max_smem_optin() - 1024) return SKV_E_RANGE;
    if (!aligned16(W) || !aligned16(h) || !aligned16(norm_w) || !aligned16(h_out) || (delta && !aligned16(delta)))
        return SKV_E_ALIGN;
    if (h_out == h || h_out == delta) return SKV_E_RANGE;        // other CTAs still read the old stream
    GemvParams p{static_cast<const __nv_bfloat16 *>(W), static_cast<const __nv_bfloat16 *>(h),
                 static_cast<const __nv_bfloat16 *>(delta), static_cast<const __nv_bfloat16 *>(norm_w),
                 static_cast<__nv_bfloat16 *>(h_out), static_cast<__nv_bfloat16 *>(y), B, N, K, eps};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return gated ? launch_gemv<true, true>(p, st) : launch_gemv<true, false>(p, st);
}
