// Small fused kernels for the single-token (decode) forward of a Qwen3 layer around the attention:
// residual add + RMSNorm, per-head QK-RMSNorm + rotary embedding + KV-cache write, SiLU(gate) * up.
// Each replaces five to twenty element-wise launches of a framework-level forward; they are
// latency-bound (a few KB per sequence), so the point is one launch instead of many.
#include "skv_rope.cuh"

namespace skv {

// h += delta (when given), rounded to bf16 as the residual stream is stored; out = RMSNorm(h) * w.
// One CTA per sequence; hidden a multiple of 8.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16 *h, const __nv_bfloat16 *delta,
                                                          const __nv_bfloat16 *w, __nv_bfloat16 *out, int hidden,
                                                          float eps) {
    __shared__ float red[32];
    const int b = blockIdx.x, tid = threadIdx.x;
    __nv_bfloat16 *hr = h + (int64_t)b * hidden;
    const __nv_bfloat16 *dr = delta ? delta + (int64_t)b * hidden : nullptr;
    const int vecs = hidden >> 3;
    float ss = 0.f;
    for (int v = tid; v < vecs; v += 256) {
        float x[8];
        load8(hr + v * 8, x);
        if (dr) {
            float y[8];
            load8(dr + v * 8, y);
            __align__(16) __nv_bfloat16 o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                o[i] = __float2bfloat16(x[i] + y[i]);
                x[i] = __bfloat162float(o[i]);
            }
            *reinterpret_cast<uint4 *>(hr + v * 8) = *reinterpret_cast<const uint4 *>(o);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)hidden + eps);
    __nv_bfloat16 *orow = out + (int64_t)b * hidden;
    for (int v = tid; v < vecs; v += 256) {
        float x[8], g[8];
        load8(hr + v * 8, x);
        load8(w + v * 8, g);
        __align__(16) __nv_bfloat16 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16(x[i] * inv * g[i]);
        *reinterpret_cast<uint4 *>(orow + v * 8) = *reinterpret_cast<const uint4 *>(o);
    }
}

// qkv [B, (H + 2*H_kv) * 128] -> q_out [B*H, 128] (normed, rotated), K/V cache rows at the new token's position (pos[0], or pos[sequence]).
// One warp per (sequence, head); lane l owns components 4l..4l+3; the rotation pairs i with i+64.
__global__ void __launch_bounds__(128) qk_rope_cache_kernel(const __nv_bfloat16 *qkv, const __nv_bfloat16 *qw,
                                                            const __nv_bfloat16 *kw, const __nv_bfloat16 *cos_t,
                                                            const __nv_bfloat16 *sin_t, const int64_t *pos_dev,
                                                            int pos_per_seq, __nv_bfloat16 *q_out, __nv_bfloat16 *k_cache,
                                                            __nv_bfloat16 *v_cache, int B, int H, int H_kv,
                                                            int64_t cache_b_stride, int64_t cache_h_stride,
                                                            int64_t cache_row_stride, float eps) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int per = H + 2 * H_kv;
    if (item >= B * per) return;
    const int b = item / per, j = item % per;
    const int64_t pos = pos_dev[pos_per_seq ? b : 0];
    const __nv_bfloat16 *src = qkv + ((int64_t)b * per + j) * HEAD_DIM + lane * 4;
    if (j >= H + H_kv) {                                              // value head: straight into the cache
        __nv_bfloat16 *dst = v_cache + b * cache_b_stride + (j - H - H_kv) * cache_h_stride + pos * cache_row_stride;
        *reinterpret_cast<uint2 *>(dst + lane * 4) = *reinterpret_cast<const uint2 *>(src);
        return;
    }
    const bool is_q = j < H;
    const float4 r = norm_rope_head(src - lane * 4, is_q ? qw : kw, cos_t + pos * HEAD_DIM, sin_t + pos * HEAD_DIM, eps,
                                    lane);
    __nv_bfloat16 *dst = is_q ? q_out + ((int64_t)b * H + j) * HEAD_DIM
                              : k_cache + b * cache_b_stride + (j - H) * cache_h_stride + pos * cache_row_stride;
    store_bf16x4(dst + lane * 4, r);
}

// gate_up [B, 2*inter] (gate first) -> out [B, inter] = silu(gate) * up, rounded as the unfused forward does
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16 *gate_up, __nv_bfloat16 *out, int B,
                                                       int inter) {
    const int vecs = inter >> 3;
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (int64_t)B * vecs) return;
    const int b = (int)(i / vecs), v = (int)(i % vecs);
    float g[8], u[8];
    load8(gate_up + (int64_t)b * 2 * inter + v * 8, g);
    load8(gate_up + (int64_t)b * 2 * inter + inter + v * 8, u);
    __align__(16) __nv_bfloat16 o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(bf16_round(g[k] / (1.f + __expf(-g[k]))) * u[k]);
    *reinterpret_cast<uint4 *>(out + (int64_t)b * inter + v * 8) = *reinterpret_cast<const uint4 *>(o);
}

}  // namespace skv

using namespace skv;

extern "C" int skv_add_rmsnorm(void *h, const void *delta, const void *w, void *out, int B, int hidden, float eps,
                               void *stream) {
    if (!h || !w || !out) return SKV_E_NULL;
    if (B <= 0 || hidden <= 0 || hidden % 8) return SKV_E_RANGE;
    if (!aligned16(h) || !aligned16(w) || !aligned16(out) || (delta && !aligned16(delta))) return SKV_E_ALIGN;
    add_rmsnorm_kernel<<<B, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16 *>(h), static_cast<const __nv_bfloat16 *>(delta),
        static_cast<const __nv_bfloat16 *>(w), static_cast<__nv_bfloat16 *>(out), hidden, eps);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

extern "C" int skv_qk_rope_cache(const void *qkv, const void *q_norm_w, const void *k_norm_w, const void *cos_table,
                                 const void *sin_table, const int64_t *pos_dev, int pos_per_seq, void *q_out, void *k_cache,
                                 void *v_cache, int B, int H, int H_kv, int d, int64_t cache_batch_stride,
                                 int64_t cache_head_stride, int64_t cache_row_stride, float eps, void *stream) {
    if (!qkv || !q_norm_w || !k_norm_w || !cos_table || !sin_table || !pos_dev || !q_out || !k_cache || !v_cache)
        return SKV_E_NULL;
    if (d != HEAD_DIM) return SKV_E_DIM;
    if (B <= 0 || H <= 0 || H_kv <= 0) return SKV_E_RANGE;
    if (!aligned16(qkv) || !aligned16(q_out) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(cos_table) ||
        !aligned16(sin_table) || cache_row_stride % 8 || cache_head_stride % 8 || cache_batch_stride % 8)
        return SKV_E_ALIGN;
    const int items = B * (H + 2 * H_kv);
    SKV_CUDA_OK(launch_pdl(qk_rope_cache_kernel, dim3((items + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream),
        static_cast<const __nv_bfloat16 *>(qkv), static_cast<const __nv_bfloat16 *>(q_norm_w),
        static_cast<const __nv_bfloat16 *>(k_norm_w), static_cast<const __nv_bfloat16 *>(cos_table),
        static_cast<const __nv_bfloat16 *>(sin_table), pos_dev, pos_per_seq, static_cast<__nv_bfloat16 *>(q_out),
        static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache), B, H, H_kv, cache_batch_stride,
        cache_head_stride, cache_row_stride, eps));
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

extern "C" int skv_silu_mul(const void *gate_up, void *out, int B, int inter, void *stream) {
    if (!gate_up || !out) return SKV_E_NULL;
    if (B <= 0 || inter <= 0 || inter % 8) return SKV_E_RANGE;
    if (!aligned16(gate_up) || !aligned16(out)) return SKV_E_ALIGN;
    const int64_t items = (int64_t)B * (inter / 8);
    silu_mul_kernel<<<(unsigned)((items + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16 *>(gate_up), static_cast<__nv_bfloat16 *>(out), B, inter);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}
