// Per-head QK-RMSNorm + rotary embedding of one 128-component head by one warp (lane l owns components
// 4l..4l+3; the rotation pairs component i with i +- 64, 16 lanes away), with the roundings of the unfused
// module forward: the normed head is a bf16 tensor, each product of the rotation is rounded, then their sum.
#pragma once

#include "skv_common.cuh"

namespace skv {

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// src: the head's 128 raw values; w: norm weights; cs, sn: the position's rows of the cos / sin tables.
// Returns the lane's four rotated components, already rounded to bf16 values.
__device__ __forceinline__ float4 norm_rope_head(const __nv_bfloat16 *src, const __nv_bfloat16 *w,
                                                 const __nv_bfloat16 *cs, const __nv_bfloat16 *sn, float eps, int lane) {
    float4 x = load4(src + lane * 4);
    const float ms = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w) / (float)HEAD_DIM;
    const float inv = rsqrtf(ms + eps);
    const float4 g = load4(w + lane * 4);
    x.x = bf16_round(x.x * inv * g.x); x.y = bf16_round(x.y * inv * g.y);
    x.z = bf16_round(x.z * inv * g.z); x.w = bf16_round(x.w * inv * g.w);
    const float4 c = load4(cs + lane * 4), s = load4(sn + lane * 4);
    float4 o;
    o.x = __shfl_xor_sync(0xffffffffu, x.x, 16); o.y = __shfl_xor_sync(0xffffffffu, x.y, 16);
    o.z = __shfl_xor_sync(0xffffffffu, x.z, 16); o.w = __shfl_xor_sync(0xffffffffu, x.w, 16);
    const float sg = lane < 16 ? -1.f : 1.f;                          // rot(x) = cat(-x2, x1)
    float4 r;
    r.x = bf16_round(bf16_round(x.x * c.x) + bf16_round(sg * o.x * s.x));
    r.y = bf16_round(bf16_round(x.y * c.y) + bf16_round(sg * o.y * s.y));
    r.z = bf16_round(bf16_round(x.z * c.z) + bf16_round(sg * o.z * s.z));
    r.w = bf16_round(bf16_round(x.w * c.w) + bf16_round(sg * o.w * s.w));
    return r;
}

__device__ __forceinline__ void store_bf16x4(__nv_bfloat16 *dst, const float4 &r) {
    __align__(8) __nv_bfloat16 ob[4] = {__float2bfloat16(r.x), __float2bfloat16(r.y), __float2bfloat16(r.z),
                                        __float2bfloat16(r.w)};
    *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(ob);
}

}  // namespace skv
