// Cluster scoring from summaries, shared (per KV head) score, top-budget selection by a weighted
// select over order-preserving keys, and the ordered list of positions to read - one launch.
//
// Bytes per head: n_c summaries (128 B int8 or 512 B float32 direction + 12 B) and one int16 label
// per cached position; everything else lives in shared memory.  The selection never sorts: it finds
// the threshold key t with  sum(count | key > t) < need  by binning order-preserving integer keys
// over the range still in question (256 bins a pass, usually one pass) and ranking the last <= 32
// candidates in a warp, then settles exact ties in slot order, which reproduces "take
// clusters in decreasing score, lower slot first among equals, until the counts reach need".
#include <cuda_fp16.h>

#include "skv_pick.cuh"
#include "skv_rope.cuh"

namespace skv {

constexpr int SEL_THREADS = 256;
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int SEL_MAX_CTAS = 64;          // CTAs that score one head's clusters in parallel

struct SelectParams {
    skv_state st;
    const void *q;
    int G;
    const int32_t *n_dev;
    int n_group;
    float *w;
    uint32_t *selbits;        // [heads, C/32 + 1]
    int32_t *idx;             // null: no row list is built
    int64_t idx_stride;
    int32_t *cnt;
    const float *shared_in;
    float *shared_out;
    float *e_out;
    float *zbuf;              // [heads, G, C] scaled scores handed from the scoring CTAs to the picking CTA
    int32_t *ticket;          // [heads]
    float *pstat;             // [heads, SEL_MAX_CTAS, 16, 2] slice (max, sum of exp) per query head
    float scale;
    int group;                // how a group's query heads share one ranking: SKV_GROUP_*
    skv_rope rope;            // rope.qkv != null: the queries are computed here from the raw projection
    unsigned long long *probe;  // optional [16] phase time stamps (ns) of head 0's picking CTA, for tuning
};

static unsigned long long *g_probe = nullptr;

__device__ __forceinline__ void stamp(const SelectParams &p, int h, int slot) {
    if (p.probe && h == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.probe[slot] = t;
    }
}

// Reduce `nv` (<= 16) per-thread values at once over the block: op = max (IS_MAX) or sum.
template <bool IS_MAX, int NV>
__device__ __forceinline__ void block_reduce_vec(float (&v)[NV], float *red /* [16][SEL_WARPS] */) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int g = 0; g < NV; ++g) {                 // the NV butterflies are independent: they overlap
            const float y = __shfl_xor_sync(0xffffffffu, v[g], o);
            v[g] = IS_MAX ? fmaxf(v[g], y) : v[g] + y;
        }
    if (lane == 0)
#pragma unroll
        for (int g = 0; g < NV; ++g) red[g * SEL_WARPS + wid] = v[g];
    __syncthreads();
#pragma unroll
    for (int g = 0; g < NV; ++g) v[g] = (lane < SEL_WARPS) ? red[g * SEL_WARPS + lane] : (IS_MAX ? -INFINITY : 0.f);
#pragma unroll
    for (int o = SEL_WARPS / 2; o > 0; o >>= 1)
#pragma unroll
        for (int g = 0; g < NV; ++g) {
            const float y = __shfl_xor_sync(0xffffffffu, v[g], o);
            v[g] = IS_MAX ? fmaxf(v[g], y) : v[g] + y;
        }
#pragma unroll
    for (int g = 0; g < NV; ++g) v[g] = __shfl_sync(0xffffffffu, v[g], 0);
    __syncthreads();
}

// ---- tensor-core scoring of 8-bit summaries against a bf16 query -------------------------------------
// scores[g][c] = q_g . dir8_c for 8 clusters per warp as one m16n8k16 chain (k = 128): the query heads sit
// on the M side (zero rows beyond G), the int8 directions are widened to fp16 in registers (exact), the
// bf16 query is exact in fp16 too, accumulation is fp32.  The k index is permuted the same way on both
// operands so that lane (n, j) reads bytes [32j, 32j+32) of cluster n with two 16-byte loads.
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two int8 (bytes `lo`, `lo`+1 of w, already biased by +128) -> packed fp16 pair holding their signed values
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t biased, uint32_t selector) {
    uint32_t h;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(biased), "r"(0x64646464u), "r"(selector));   // 1024 + u
    const __half2 v = __hsub2(*reinterpret_cast<__half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x6480)));
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// QK-norm + rotary of KV head h's G query heads, a warp per head, into sq (when given); with `first` (the head's
// first CTA) they are also stored for the attention launch and the token's K and V rows are written.
__device__ __forceinline__ void rope_heads(const skv_rope &r, int h, bool first, int G, float *sq) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int seq = h / r.H_kv, hk = h % r.H_kv, per_seq = r.H + 2 * r.H_kv;
    const int64_t pos = r.pos[r.pos_per_seq ? seq : 0];
    const __nv_bfloat16 *row = static_cast<const __nv_bfloat16 *>(r.qkv) + (int64_t)seq * per_seq * HEAD_DIM;
    const __nv_bfloat16 *cs = static_cast<const __nv_bfloat16 *>(r.cos_table) + pos * HEAD_DIM;
    const __nv_bfloat16 *sn = static_cast<const __nv_bfloat16 *>(r.sin_table) + pos * HEAD_DIM;
    const int jobs = G + (first ? 2 : 0);
    for (int j = wid; j < jobs; j += SEL_WARPS) {
        if (j < G) {
            const int qh = hk * G + j;
            const float4 v = norm_rope_head(row + (int64_t)qh * HEAD_DIM, static_cast<const __nv_bfloat16 *>(r.q_norm_w),
                                            cs, sn, r.eps, lane);
            if (sq) *reinterpret_cast<float4 *>(sq + j * HEAD_DIM + lane * 4) = v;
            if (first)
                store_bf16x4(static_cast<__nv_bfloat16 *>(r.q_out) + ((int64_t)seq * r.H + qh) * HEAD_DIM + lane * 4, v);
        } else {
            const int64_t at = seq * r.cache_batch_stride + hk * r.cache_head_stride + pos * r.cache_row_stride;
            if (j == G) {
                const float4 v = norm_rope_head(row + (int64_t)(r.H + hk) * HEAD_DIM,
                                                static_cast<const __nv_bfloat16 *>(r.k_norm_w), cs, sn, r.eps, lane);
                store_bf16x4(static_cast<__nv_bfloat16 *>(r.k_cache) + at + lane * 4, v);
            } else {
                const __nv_bfloat16 *src = row + (int64_t)(r.H + r.H_kv + hk) * HEAD_DIM + lane * 4;
                *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(r.v_cache) + at + lane * 4) =
                    *reinterpret_cast<const uint2 *>(src);
            }
        }
    }
}

// Grid (ctas, heads).  Every CTA scores a slice of the head's clusters: e = (longest or shortest key) x
// projection of the query on the cluster's mean direction, scaled by 1/sqrt(d); it then leaves
// exp(z - slice max) in zbuf and its (max, sum) per query head in pstat.  The last CTA of the head to
// finish (atomic ticket, no waiting) combines the slices' statistics into the shared score
// sum_g softmax_g(z)[c] without another exponential, finds the threshold key by an adaptive-range weighted select
// and writes the weights and the selection bits.
template <typename TQ, int GP>
__global__ void __launch_bounds__(SEL_THREADS) score_pick_kernel(const SelectParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_last;
    __shared__ float s_stat[32];                                    // a lone CTA's own statistics: [G][2]
    const int C = p.st.C, G = p.G, d = HEAD_DIM;
    const int h = blockIdx.y, b = blockIdx.x, nb = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    float *z = reinterpret_cast<float *>(smem_raw);                 // [G][C]: slice scores, later exp values
    const int zfloats = p.shared_in ? 0 : G * C;
    uint32_t *key = reinterpret_cast<uint32_t *>(z + zfloats);      // [C]
    int *ci = reinterpret_cast<int *>(key + C);                     // [C]
    float *sq = reinterpret_cast<float *>(ci + C);                  // [G][128]
    float *red = sq + G * d;                                        // [16][SEL_WARPS]
    int *hist = reinterpret_cast<int *>(red + 16 * SEL_WARPS);      // [4][256]
    int *ired = hist + 4 * 256;                                     // [40]
    float *fb = reinterpret_cast<float *>(ired + 40);               // [SEL_MAX_CTAS][16] slice factors
    uint8_t *sel = reinterpret_cast<uint8_t *>(fb + SEL_MAX_CTAS * 16);   // [C + 1]
    // while a slice is scored, key and ci hold its longest and shortest key lengths (the pick fills them later);
    // an empty cluster is marked by a longest length of -inf, so that no third array of counts is needed
    // (8,192 slots x 4 query heads would not fit the shared memory of an SM with one)
    float *smx = reinterpret_cast<float *>(key), *smn = reinterpret_cast<float *>(ci);

    const int n_c = min(max(p.st.n_c[h], 0), C);
    const int end = p.st.end[h];
    const int need = p.st.need[h];
    const bool active = end > 1 && need > 0;
    const bool scoring = active && !p.shared_in;
    if (!scoring && b != 0) return;
    const float *count = p.st.count + (int64_t)h * C;
    float *zg = p.zbuf + (int64_t)h * G * C;
    float *ps = p.pstat + (int64_t)h * SEL_MAX_CTAS * 32;          // [ctas][G][2]
    const int per = (((n_c + nb - 1) / nb) + 3) & ~3;              // clusters per scoring CTA
    const float inv_per = 1.0f / (float)max(per, 1);
    if (b == 0) stamp(p, h, 0);
    if (!scoring) {
        pdl_wait();
        pdl_trigger();
        if (p.rope.qkv) rope_heads(p.rope, h, true, G, nullptr);   // nothing to score: the token's rows are still due
    }

    if (scoring) {
        const int c_lo = min(b * per, n_c), c_hi = min(c_lo + per, n_c), mine = c_hi - c_lo;
        const float *mmax = p.st.mmax + (int64_t)h * C, *mmin = p.st.mmin + (int64_t)h * C;
        const TQ *q = static_cast<const TQ *>(p.q) + (int64_t)h * G * d;
        const bool q8 = p.st.summary_bits == 8;
        const int part = lane & 7, grp = lane >> 3;
        // The CTA takes 128 clusters per iteration, a warp 16 of them (8 lanes, one 16-byte load each, per
        // cluster): all loads of an iteration are requested before the query is staged, so the two latencies overlap and enough
        // bytes are in flight to stream the summaries at memory speed.
        int4 raw[4];
        float rawc[4], rawx[4], rawn[4];
        float4 rawf = make_float4(0.f, 0.f, 0.f, 0.f);
        auto fetch8 = [&](int c0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int c = c0 + (k * SEL_WARPS + wid) * 4 + grp;
                raw[k] = make_int4(0, 0, 0, 0);
                rawc[k] = rawx[k] = rawn[k] = 0.f;
                if (c < c_hi) {
                    raw[k] = __ldg(reinterpret_cast<const int4 *>(p.st.dir8 + ((int64_t)h * C + c) * d + part * 16));
                    rawc[k] = count[c]; rawx[k] = mmax[c]; rawn[k] = mmin[c];
                }
            }
        };
        constexpr bool TC = sizeof(TQ) == 2;               // bf16 query: tensor-core scoring of 8-bit summaries
        int4 rawa[4], rawb[4];                            // TC path: bytes [32j, 32j+32) of this lane's clusters
        int4 nxta[4], nxtb[4];                            // the next iteration's, requested one iteration ahead
        const int nrow = lane >> 2, jq = lane & 3;
        auto fetch_tc = [&](int c0, int4 (&da)[4], int4 (&db)[4]) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int c = c0 + (k * SEL_WARPS + wid) * 8 + nrow;
                da[k] = db[k] = make_int4(0, 0, 0, 0);
                if (c < c_hi) {
                    const int4 *src = reinterpret_cast<const int4 *>(p.st.dir8 + ((int64_t)h * C + c) * d + jq * 32);
                    da[k] = __ldg(src);
                    db[k] = __ldg(src + 1);
                }
            }
        };
        if (q8 && TC) {
            fetch_tc(c_lo, rawa, rawb);
        } else if (q8) {
            fetch8(c_lo);
        } else {
            const int c = c_lo + wid;
            if (c < c_hi) rawf = __ldg(reinterpret_cast<const float4 *>(p.st.sum_dir + ((int64_t)h * C + c) * d + lane * 4));
        }
        // the slice's lengths and counts go to shared memory up front: read in the scoring loop from global memory
        // they cost a dependent round trip per eight clusters (30 us of a 38 us launch with one CTA per head)
        for (int i = tid; i < mine; i += SEL_THREADS) {
            smx[i] = count[c_lo + i] == 0.f ? -INFINITY : mmax[c_lo + i];
            smn[i] = mmin[c_lo + i];
        }
        pdl_wait();                                        // the query comes from the kernel before this one
        pdl_trigger();
        if (p.rope.qkv) {
            rope_heads(p.rope, h, b == 0, G, sq);
        } else {
            for (int i = tid; i < G * d; i += SEL_THREADS) sq[i] = load_as_float(q + i);
        }
        __syncthreads();
        if (q8 && TC) {
            // query fragments (A): rows = query heads, k permuted as described above
            uint32_t qa[8][4];
            const int g0 = nrow, g1 = nrow + 8;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const float *q0 = sq + g0 * d + 32 * jq + 4 * ks, *q1 = sq + g1 * d + 32 * jq + 4 * ks;
                qa[ks][0] = g0 < G ? pack_half2(q0[0], q0[1]) : 0u;
                qa[ks][2] = g0 < G ? pack_half2(q0[2], q0[3]) : 0u;
                qa[ks][1] = (GP > 8 && g1 < G) ? pack_half2(q1[0], q1[1]) : 0u;
                qa[ks][3] = (GP > 8 && g1 < G) ? pack_half2(q1[2], q1[3]) : 0u;
            }
            for (int c0 = c_lo; c0 < c_hi; c0 += SEL_WARPS * 32) {
                if (c0 != c_lo) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) { rawa[k] = nxta[k]; rawb[k] = nxtb[k]; }
                }
                if (c0 + SEL_WARPS * 32 < c_hi) fetch_tc(c0 + SEL_WARPS * 32, nxta, nxtb);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int cbase = c0 + (k * SEL_WARPS + wid) * 8;
                    if (cbase >= c_hi) continue;                        // warp-uniform
                    const uint32_t w[8] = {(uint32_t)rawa[k].x, (uint32_t)rawa[k].y, (uint32_t)rawa[k].z,
                                           (uint32_t)rawa[k].w, (uint32_t)rawb[k].x, (uint32_t)rawb[k].y,
                                           (uint32_t)rawb[k].z, (uint32_t)rawb[k].w};
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    int n2i = 0;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        n2i = __dp4a((int)w[ks], (int)w[ks], n2i);
                        const uint32_t biased = w[ks] ^ 0x80808080u;
                        mma_f16_16816(acc, qa[ks], bytes_to_half2(biased, 0x4140u), bytes_to_half2(biased, 0x4342u));
                    }
                    n2i += __shfl_xor_sync(0xffffffffu, n2i, 1);
                    n2i += __shfl_xor_sync(0xffffffffu, n2i, 2);            // |dir8|^2 of cluster cbase + nrow
                    // lane (g, j) holds the dots of clusters cbase + 2j, 2j + 1: fetch their norms
                    const int na = __shfl_sync(0xffffffffu, n2i, (2 * jq) * 4);
                    const int nb2 = __shfl_sync(0xffffffffu, n2i, (2 * jq + 1) * 4);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int c = cbase + 2 * jq + i;
                        if (c < c_hi) {
                            const float inv = 1.0f / fmaxf(sqrtf((float)(i ? nb2 : na)), 1e-12f);
                            const float mx = smx[c - c_lo], mn = smn[c - c_lo];
#pragma unroll
                            for (int r = 0; r < (GP > 8 ? 2 : 1); ++r) {
                                const int g = nrow + 8 * r;
                                if (g < G) {
                                    const float pr = acc[2 * r + i] * inv;
                                    float e = pr >= 0.f ? mx * pr : mn * pr;
                                    if (mx == -INFINITY) e = -INFINITY;       // empty cluster
                                    z[g * C + (c - c_lo)] = e * p.scale;
                                    if (p.e_out) p.e_out[((int64_t)h * G + g) * C + c] = e;
                                }
                            }
                        }
                    }
                }
            }
        } else if (q8) {
            for (int c0 = c_lo; c0 < c_hi; c0 += SEL_WARPS * 16) {
                if (c0 != c_lo) fetch8(c0);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int c = c0 + (k * SEL_WARPS + wid) * 4 + grp;
                    const bool live = c < c_hi;
                    const float cn = rawc[k], mx = rawx[k], mn = rawn[k];
                    float v[16];
                    const int8_t *bb = reinterpret_cast<const int8_t *>(&raw[k]);
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = (float)bb[i];
                    float n2 = 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) n2 = fmaf(v[i], v[i], n2);
                    n2 += __shfl_xor_sync(0xffffffffu, n2, 1);
                    n2 += __shfl_xor_sync(0xffffffffu, n2, 2);
                    n2 += __shfl_xor_sync(0xffffffffu, n2, 4);
                    const float inv = 1.0f / fmaxf(sqrtf(n2), 1e-12f);
                    for (int g = 0; g < G; ++g) {
                        const float4 *qs = reinterpret_cast<const float4 *>(sq + g * d + part * 16);
                        float dot = 0.f;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float4 t = qs[i];
                            dot = fmaf(v[4 * i], t.x, dot);
                            dot = fmaf(v[4 * i + 1], t.y, dot);
                            dot = fmaf(v[4 * i + 2], t.z, dot);
                            dot = fmaf(v[4 * i + 3], t.w, dot);
                        }
                        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
                        if (part == 0 && live) {
                            const float pr = dot * inv;
                            float e = pr >= 0.f ? mx * pr : mn * pr;
                            if (cn == 0.f) e = -INFINITY;
                            z[g * C + (c - c_lo)] = e * p.scale;
                            if (p.e_out) p.e_out[((int64_t)h * G + g) * C + c] = e;
                        }
                    }
                }
            }
        } else {
            const float *sd = p.st.sum_dir + (int64_t)h * C * d;
            for (int c = c_lo + wid; c < c_hi; c += SEL_WARPS) {
                const float4 v = rawf;
                if (c + SEL_WARPS < c_hi)
                    rawf = __ldg(reinterpret_cast<const float4 *>(sd + (int64_t)(c + SEL_WARPS) * d + lane * 4));
                const float n2 = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
                const float inv = 1.0f / fmaxf(sqrtf(n2), 1e-12f);
                for (int g = 0; g < G; ++g) {
                    const float4 t = *reinterpret_cast<const float4 *>(sq + g * d + lane * 4);
                    const float dot = warp_sum(v.x * t.x + v.y * t.y + v.z * t.z + v.w * t.w);
                    if (lane == 0) {
                        const float pr = dot * inv;
                        float e = pr >= 0.f ? mmax[c] * pr : mmin[c] * pr;
                        if (count[c] == 0.f) e = -INFINITY;
                        z[g * C + (c - c_lo)] = e * p.scale;
                        if (p.e_out) p.e_out[((int64_t)h * G + g) * C + c] = e;
                    }
                }
            }
        }
        __syncthreads();
        // slice statistics: max and sum of exp(z - max) per query head; zbuf <- exp(z - max)
        float zm[GP], tot[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            float m = -INFINITY;
            if (g < G)
                for (int c = tid; c < mine; c += SEL_THREADS) m = fmaxf(m, z[g * C + c]);
            zm[g] = m;
        }
        block_reduce_vec<true, GP>(zm, red);
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            float s = 0.f;
            if (g < G)
                for (int c = tid; c < mine; c += SEL_THREADS) {
                    const float zz = z[g * C + c];
                    // the max modes rank the scaled scores themselves; sum_share hands on exp(z - slice max)
                    const float ex = p.group != SKV_GROUP_SUM_SHARE ? zz : (zz > -INFINITY ? expf(zz - zm[g]) : 0.f);
                    if (nb > 1) __stcg(zg + g * C + c_lo + c, ex);
                    else z[g * C + c] = ex;                 // a lone CTA keeps the values where the pick reads them
                    s += ex;
                }
            tot[g] = s;
        }
        block_reduce_vec<false, GP>(tot, red);
        if (tid == 0)
#pragma unroll
            for (int g = 0; g < GP; ++g)
                if (g < G) {
                    if (nb > 1) {
                        __stcg(ps + (b * 16 + g) * 2, zm[g]);
                        __stcg(ps + (b * 16 + g) * 2 + 1, tot[g]);
                    } else {                               // one CTA per head: nothing goes through global memory
                        s_stat[2 * g] = zm[g];
                        s_stat[2 * g + 1] = tot[g];
                    }
                }
        if (b == 0) stamp(p, h, 1);
        if (nb > 1) {
            __threadfence();
            __syncthreads();
            if (tid == 0) s_last = atomicAdd(p.ticket + h, 1) == nb - 1;
            __syncthreads();
            if (!s_last) return;
            __threadfence();
            if (tid == 0) p.ticket[h] = 0;
        } else {
            __syncthreads();                               // thread 0's statistics are read by other warps below
        }
    }
    stamp(p, h, 2);
    // ---- the head's picking CTA from here on ---------------------------------------------------------
    // Everything this CTA needs from global memory - the slices' statistics, their exp values, the clusters'
    // counts - is requested before any of it is used (four loads per thread at a time), so the prologue of
    // the pick costs about one round trip to L2 instead of one per loop iteration.
    float2 s0 = make_float2(-INFINITY, 0.f), s1 = s0;
    const bool stat_warp = scoring && wid < G;               // one warp per query head; G <= 16 > SEL_WARPS loops below
    if (stat_warp) {
        if (nb == 1) {
            if (lane == 0) s0 = make_float2(s_stat[2 * wid], s_stat[2 * wid + 1]);
        } else {
            if (lane < nb) s0 = __ldcg(reinterpret_cast<const float2 *>(ps + (lane * 16 + wid) * 2));
            if (lane + 32 < nb) s1 = __ldcg(reinterpret_cast<const float2 *>(ps + ((lane + 32) * 16 + wid) * 2));
        }
    }
    if (scoring && nb > 1)
        for (int g = 0; g < G; ++g)
            for (int c = tid; c < n_c; c += 4 * SEL_THREADS) {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int cc = c + j * SEL_THREADS;
                    v[j] = cc < n_c ? __ldcg(zg + g * C + cc) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int cc = c + j * SEL_THREADS;
                    if (cc < n_c) z[g * C + cc] = v[j];
                }
            }
    for (int c = tid; c < n_c; c += 4 * SEL_THREADS) {    // (only the slots in use are looked at below)
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cc = c + j * SEL_THREADS;
            v[j] = cc < n_c ? count[cc] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cc = c + j * SEL_THREADS;
            if (cc < n_c) ci[cc] = (int)v[j];
        }
    }
    // the selection as bits: the pick writes the words that hold slots in use (nothing selected: cleared here), the
    // rest are zero; bit C (the always-read rows) is added on the way out (C need not be a multiple of 32 here)
    uint32_t *sbits = reinterpret_cast<uint32_t *>(sel);
    const int words = C / 32 + 1;
    for (int wd = (active ? (n_c + 31) >> 5 : 0) + tid; wd < words; wd += SEL_THREADS) sbits[wd] = 0u;
    if (tid == 0 && !p.idx) p.cnt[h] = 0;             // the attention kernel adds the rows it reads
    if (scoring) {
        // slice factors exp(max_b - max) / total per query head
        for (int g = wid; g < G; g += SEL_WARPS) {     // a lane holds up to two slices
            if (g != wid) {                            // more query heads than warps: the later ones load here
                s0 = s1 = make_float2(-INFINITY, 0.f);
                if (nb == 1) {
                    if (lane == 0) s0 = make_float2(s_stat[2 * g], s_stat[2 * g + 1]);
                } else {
                    if (lane < nb) s0 = __ldcg(reinterpret_cast<const float2 *>(ps + (lane * 16 + g) * 2));
                    if (lane + 32 < nb) s1 = __ldcg(reinterpret_cast<const float2 *>(ps + ((lane + 32) * 16 + g) * 2));
                }
            }
            const float m = warp_max(fmaxf(s0.x, s1.x));
            if (p.group != SKV_GROUP_SUM_SHARE) {          // only the head's best score is needed (max_rel)
                if (lane == 0) fb[g] = m;
                continue;
            }
            const float e0 = s0.x > -INFINITY ? expf(s0.x - m) : 0.f, e1 = s1.x > -INFINITY ? expf(s1.x - m) : 0.f;
            const float t = warp_sum(e0 * s0.y + e1 * s1.y);
            if (lane < nb) fb[lane * 16 + g] = e0 / t;
            if (lane + 32 < nb) fb[(lane + 32) * 16 + g] = e1 / t;
        }
    }
    __syncthreads();
    stamp(p, h, 3);
    uint32_t kmin = 0xffffffffu, kmax = 0u;        // range of the keys of clusters with members, and their number
    int nvalid = 0;
    const int kend = p.shared_out ? C : n_c;       // keys of spare slots matter only to a caller who asked for the scores
    if (scoring) {
#pragma unroll 2
        for (int c = tid; c < kend; c += SEL_THREADS) {
            float s = -INFINITY;
            if (c < n_c && ci[c] > 0 && p.group != SKV_GROUP_SUM_SHARE) {
                for (int g = 0; g < G; ++g)
                    s = fmaxf(s, z[g * C + c] - (p.group == SKV_GROUP_MAX_REL ? fb[g] : 0.f));
            } else if (c < n_c && ci[c] > 0) {
                int sl = (int)((float)c * inv_per);            // slice of cluster c, without an integer division
                sl += ((sl + 1) * per <= c) - (sl * per > c);
                const float *f = fb + sl * 16;
                s = 0.f;
                for (int g = 0; g < G; ++g) s += z[g * C + c] * f[g];
            }
            const uint32_t k = float_key(s);
            key[c] = k;
            if (c < n_c && ci[c] > 0) { kmin = min(kmin, k); kmax = max(kmax, k); ++nvalid; }
            if (p.shared_out) p.shared_out[(int64_t)h * C + c] = s;
        }
    } else if (active) {
        const float *sin = p.shared_in + (int64_t)h * C;
        for (int c = tid; c < kend; c += SEL_THREADS) {
            const float s = c < n_c ? sin[c] : -INFINITY;
            const uint32_t k = float_key(s);
            key[c] = k;
            if (c < n_c && ci[c] > 0) { kmin = min(kmin, k); kmax = max(kmax, k); ++nvalid; }
            if (p.shared_out) p.shared_out[(int64_t)h * C + c] = s;
        }
    }
    stamp(p, h, 4);
    pick_by_threshold<SEL_THREADS, int, true>(key, ci, nullptr, hist, ired, n_c, need, active, kmin, kmax, nvalid, sbits);
    stamp(p, h, 6);
    // ---- weights and selection bits out ---------------------------------------------------------
    float *w = p.w + (int64_t)h * (C + 1);
    for (int c = tid; c <= C; c += SEL_THREADS) w[c] = c == C ? 1.f : (float)((sbits[c >> 5] >> (c & 31)) & 1u);
    uint32_t *bits = p.selbits + (int64_t)h * words;
    for (int wd = tid; wd < words; wd += SEL_THREADS) bits[wd] = sbits[wd] | (wd == (C >> 5) ? 1u << (C & 31) : 0u);
    stamp(p, h, 7);
}

// Ordered list of the positions to read, one CTA per head (only when a caller asks for the list).
__global__ void __launch_bounds__(512) list_kernel(const SelectParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int ired[40];
    const int C = p.st.C, h = blockIdx.x, tid = threadIdx.x;
    const int words = C / 32 + 1;
    uint32_t *bits = reinterpret_cast<uint32_t *>(smem_raw);
    for (int i = tid; i < words; i += 512) bits[i] = p.selbits[(int64_t)h * words + i];
    __syncthreads();
    const int16_t *lab = p.st.labels + (int64_t)h * p.st.capacity;
    const int nn = min(max(positions_of(p.n_dev, p.n_group, h), 0), p.st.capacity);
    const int vecs = (nn + 7) >> 3;
    const int per = (vecs + 511) / 512;
    const int v0 = min(tid * per, vecs), v1 = min(v0 + per, vecs);
    int mine = 0;
    bool bad = false;
    for (int v = v0; v < v1; ++v) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(lab + v * 8);
        const int16_t *l8 = reinterpret_cast<const int16_t *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int pos = v * 8 + i;
            const unsigned l = (unsigned)(int)l8[i];
            if (pos < nn) {
                if (l <= (unsigned)C) mine += (bits[l >> 5] >> (l & 31)) & 1u;
                else bad = true;
            }
        }
    }
    int total;
    int off = block_excl_scan(mine, ired, total);
    int32_t *out = p.idx + (int64_t)h * p.idx_stride;
    for (int v = v0; v < v1; ++v) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(lab + v * 8);
        const int16_t *l8 = reinterpret_cast<const int16_t *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int pos = v * 8 + i;
            const unsigned l = (unsigned)(int)l8[i];
            if (pos < nn && l <= (unsigned)C && ((bits[l >> 5] >> (l & 31)) & 1u)) out[off++] = pos;
        }
    }
    if (tid == 0) p.cnt[h] = total;
    if (bad && p.st.status) atomicOr(p.st.status + h, SKV_ST_BAD_INDEX);
}

static size_t select_smem(int G, int C, bool scored) {
    size_t b = 0;
    if (scored) b += (size_t)G * C * 4;
    b += (size_t)C * 4 * 2;                 // key, ci
    b += (size_t)G * HEAD_DIM * 4;          // sq
    b += 16 * SEL_WARPS * 4 + 4 * 256 * 4 + 40 * 4 + SEL_MAX_CTAS * 16 * 4;
    b += C + 1 + 16;
    return (b + 15) & ~size_t(15);
}

static int64_t select_ws_bytes(int heads, int G, int C) {
    int64_t z = ((int64_t)heads * G * C * 4 + 255) / 256 * 256;
    int64_t t = ((int64_t)heads * 4 + 255) / 256 * 256;
    int64_t bits = ((int64_t)heads * (C / 32 + 1) * 4 + 255) / 256 * 256;
    int64_t ps = (int64_t)heads * SEL_MAX_CTAS * 32 * 4;
    return z + t + bits + ps;
}

}  // namespace skv

using namespace skv;

// Tuning aid: a device array of 16 uint64 that receives phase time stamps of the selection kernel (null: off).
extern "C" void skv_debug_select_probe(void *dev_ptr) { skv::g_probe = static_cast<unsigned long long *>(dev_ptr); }

extern "C" int64_t skv_select_workspace_bytes(int heads, int G, int C) {
    if (heads <= 0 || G < 1 || G > 16 || C < 16 || (C & (C - 1)) || C > 16384) return SKV_E_RANGE;
    return select_ws_bytes(heads, G, C);
}

extern "C" int skv_select(const skv_state *st, const void *q, int dtype, int G, const int32_t *n_dev, int n_group, float *w,
                          uint32_t *selbits, int32_t *idx, int64_t idx_stride, int32_t *cnt, const float *shared_in,
                          float *shared_out, float *e_out, void *workspace, float scale, int group,
                          const skv_rope *rope, void *stream) {
    if (!st || !n_dev || !w || !cnt || !workspace) return SKV_E_NULL;
    if (!shared_in && !q && !rope) return SKV_E_NULL;
    if (rope) {
        if (shared_in) return SKV_E_RANGE;               // nothing to score, so nothing to rotate
        if (!rope->qkv || !rope->q_norm_w || !rope->k_norm_w || !rope->cos_table || !rope->sin_table || !rope->pos ||
            !rope->q_out || !rope->k_cache || !rope->v_cache)
            return SKV_E_NULL;
        if (dtype != SKV_BF16) return SKV_E_DTYPE;
        if (rope->H_kv < 1 || rope->H < rope->H_kv || rope->H % rope->H_kv || rope->H / rope->H_kv != G ||
            st->heads % rope->H_kv)
            return SKV_E_RANGE;
        if (!aligned16(rope->qkv) || !aligned16(rope->q_out) || !aligned16(rope->k_cache) || !aligned16(rope->v_cache) ||
            rope->cache_row_stride % 8 || rope->cache_head_stride % 8 || rope->cache_batch_stride % 8)
            return SKV_E_ALIGN;
    }
    if (!st->count || !st->n_c || !st->end || !st->need || !st->labels || !st->mmax || !st->mmin) return SKV_E_NULL;
    if (st->d != HEAD_DIM) return SKV_E_DIM;
    if (st->C < 16 || (st->C & (st->C - 1)) || st->C > 16384) return SKV_E_DIM;
    if (G < 1 || G > 16) return SKV_E_DIM;
    if (dtype != SKV_BF16 && dtype != SKV_F32) return SKV_E_DTYPE;
    if (st->summary_bits != 8 && st->summary_bits != 32) return SKV_E_RANGE;
    if (group < SKV_GROUP_SUM_SHARE || group > SKV_GROUP_MAX_REL || n_group < 0) return SKV_E_RANGE;
    if (st->summary_bits == 8 ? !st->dir8 : !st->sum_dir) return SKV_E_NULL;
    if (st->heads <= 0 || st->heads > 65535 || st->capacity <= 0 || (idx && idx_stride < st->capacity)) return SKV_E_RANGE;
    if (st->capacity % 8 || !aligned16(st->labels) || !aligned16(workspace)) return SKV_E_ALIGN;
    if (st->summary_bits == 8 ? !aligned16(st->dir8) : !aligned16(st->sum_dir)) return SKV_E_ALIGN;
    const size_t smem = select_smem(G, st->C, shared_in == nullptr);
    if ((int)smem > device_max_smem_optin()) return SKV_E_DIM;
    SelectParams p;
    p.st = *st; p.q = q; p.G = G; p.n_dev = n_dev; p.n_group = n_group; p.w = w; p.idx = idx; p.idx_stride = idx_stride; p.cnt = cnt;
    p.shared_in = shared_in; p.shared_out = shared_out; p.e_out = e_out; p.scale = scale; p.group = group;
    p.rope = rope ? *rope : skv_rope{};
    p.probe = g_probe;
    char *ws = static_cast<char *>(workspace);
    p.zbuf = reinterpret_cast<float *>(ws);
    ws += ((int64_t)st->heads * G * st->C * 4 + 255) / 256 * 256;
    p.ticket = reinterpret_cast<int32_t *>(ws);
    ws += ((int64_t)st->heads * 4 + 255) / 256 * 256;
    p.selbits = selbits ? selbits : reinterpret_cast<uint32_t *>(ws);
    ws += ((int64_t)st->heads * (st->C / 32 + 1) * 4 + 255) / 256 * 256;
    p.pstat = reinterpret_cast<float *>(ws);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    using Kern = void (*)(const SelectParams);
    const int gsel = G <= 1 ? 0 : G <= 2 ? 1 : G <= 4 ? 2 : G <= 8 ? 3 : 4;
    static const Kern table[2][5] = {
        {score_pick_kernel<__nv_bfloat16, 1>, score_pick_kernel<__nv_bfloat16, 2>, score_pick_kernel<__nv_bfloat16, 4>,
         score_pick_kernel<__nv_bfloat16, 8>, score_pick_kernel<__nv_bfloat16, 16>},
        {score_pick_kernel<float, 1>, score_pick_kernel<float, 2>, score_pick_kernel<float, 4>,
         score_pick_kernel<float, 8>, score_pick_kernel<float, 16>}};
    Kern kern = table[dtype][gsel];
    static size_t configured[64][2][5] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (smem > 48 * 1024 && configured[dev][dtype][gsel] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][dtype][gsel] = smem;
    }
    // As many CTAs per head as fit ONE wave of two CTAs per SM, and at most 16: a CTA's cost is mostly a fixed
    // chain of latencies, so a second wave costs more than longer slices do, and every slice adds statistics
    // for the picking CTA to combine (8 heads on B200: 16 slices 17.9 us, 37 slices 20.6 us, 8 slices 19.2 us).
    // Many heads: one CTA per head.
    int ctas = 2 * device_sm_count() / st->heads;
    ctas = ctas < 1 ? 1 : (ctas > 16 ? 16 : ctas);
    if (shared_in) ctas = 1;
    SKV_CUDA_OK(launch_pdl(kern, dim3(ctas, st->heads), dim3(SEL_THREADS), smem, s, p));
    if (idx) list_kernel<<<st->heads, 512, (st->C / 32 + 1) * 4, s>>>(p);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}
