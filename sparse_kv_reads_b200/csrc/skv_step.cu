// Selection and attention of one decode step in ONE launch, for launches with few (sequence, KV head) pairs.
//
// With 8 to about 36 heads a step is a chain of latencies, not a stream: two launches, each with a hand-off
// through global memory to the head's last CTA (the pick; the merge of the split partials).  Here a head is
// served by thread-block clusters of 8 CTAs that talk through distributed shared memory instead:
//   1. every CTA stages its eighth of the head's 8-bit cluster summaries (requested before the wait for the
//      launch ahead) and scores it on mma.sync f16 tiles; each warp keeps the maximum and the sum of
//      exp(score - maximum) of the clusters it scored, per query head, and stores that pair into the shared
//      memory of all 8 CTAs of its cluster;
//   2. after a cluster barrier every warp combines the 32 pairs into the softmax's maximum and total, every
//      CTA turns the scores of ITS clusters into shared scores (sum over the query heads of each head's
//      softmax share) and order-preserving keys, and stores those into all 8 CTAs; after a second barrier
//      every CTA holds all keys and runs the same threshold pick as the selection kernel for itself, so no
//      CTA waits for another one's pick;
//   3. every CTA attends over its range of positions, rows taken straight from the labels;
//   4. the 8 partials of a cluster meet in the shared memory of its first CTA, which merges them; only one
//      partial per cluster (4 per head at 8 heads, none at 32 heads) goes through global memory, where the
//      output product or the head's last cluster (a ticket) merges them.
// Remote shared memory is written with plain st.shared::cluster stores (this GPU's memory only, no multicast).
// Every CTA of a cluster executes all four cluster barriers unconditionally; nothing spins.
#include <cuda_fp16.h>

#include "skv_attend_core.cuh"
#include "skv_pick.cuh"
#include "skv_rope.cuh"

namespace skv {

// CTAs of NW = 4 warps, two per SM.  (8 warps with a ring of one tile each - the same shared memory, 16 warps per
// SM - were measured at batch 1, 32k: 690 against 697 tok/s, no gain; the kernel stays generic in NW.)
constexpr int STEP_CS = 8, STEP_LPT = 8, STEP_STAGES = 2;
constexpr int STEP_GROUPS = 2;                            // label groups of STEP_LPT per thread and pass
__host__ __device__ constexpr int step_pass(int nw) { return nw * 32 * STEP_LPT * STEP_GROUPS; }   // positions per pass
__host__ __device__ constexpr int step_slices(int nw) { return STEP_CS * nw; }   // (CTA, warp) pairs that score a head
constexpr int STEP_PART_LD = 132;                         // floats per partial row: 128 sums, max, sum, rows, unused

struct StepParams {
    skv_state st;
    const void *q;             // [heads*G, 128] bf16 (unused with rope)
    const void *K, *V;
    const int32_t *n_dev;
    int n_group;
    void *out;
    float *w;                  // [heads, C+1] or null
    uint32_t *selbits;         // [heads, C/32+1] or null
    int32_t *cnt;              // [heads] rows read
    float *part;               // [heads, ncl, G, 132]
    int32_t *ticket;           // [heads]
    int G, ncl;
    int64_t ksh, ksr, vsh, vsr;
    float scale, scale_log2;
    skv_rope rope;
    unsigned long long *probe; // optional [CTAs][16] phase time stamps (probe builds only)
};

static unsigned long long *g_step_probe = nullptr;

__device__ __forceinline__ void step_stamp(const StepParams &p, int slot) {
#ifdef SKV_STEP_PROBE
    if (p.probe && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.probe[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 + slot] = t;
    }
#else
    (void)p; (void)slot;
#endif
}

// ---- thread-block cluster primitives ---------------------------------------------------------------------
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// shared::cluster address of `ptr` (a shared-memory pointer of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t remote_addr(const void *ptr, unsigned rank) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(a), "r"(rank));
    return out;
}
__device__ __forceinline__ void remote_store(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void remote_store4(uint32_t addr, const float4 &v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

__device__ __forceinline__ void step_mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two int8 (already biased by +128) -> packed fp16 pair of their signed values (exact)
__device__ __forceinline__ uint32_t step_bytes_to_half2(uint32_t biased, uint32_t selector) {
    uint32_t hh;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(hh) : "r"(biased), "r"(0x64646464u), "r"(selector));   // 1024 + u
    const __half2 v = __hsub2(*reinterpret_cast<__half2 *>(&hh), __half2half2(__ushort_as_half((unsigned short)0x6480)));
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t step_pack_half2(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// Exclusive scan of one int per thread over the CTA's NW warps with a single barrier; every thread gets `total`.
// `buf` (NW ints) must not have been read since the last barrier but one, which two passes of the row list satisfy.
template <int NW>
__device__ __forceinline__ int step_excl_scan(int v, int *buf, int &total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) buf[wid] = inc;
    __syncthreads();
    int base = 0;
    total = 0;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        const int t = buf[w];
        base += w < wid ? t : 0;
        total += t;
    }
    return base + inc - v;
}

// QK-norm + rotary of KV head h's G query heads into sq (float values of the bf16 results) and sqb (bf16);
// `store_q`: also to the caller's q buffer; `store_kv`: this CTA reads the new token's position, so it
// writes the token's K and V rows itself before it gathers them.
__device__ __forceinline__ void step_rope(const skv_rope &r, int h, bool store_q, bool store_kv, int G, float *sq,
                                          __nv_bfloat16 *sqb, int nw) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int seq = h / r.H_kv, hk = h % r.H_kv, per_seq = r.H + 2 * r.H_kv;
    const int64_t pos = r.pos[r.pos_per_seq ? seq : 0];
    const __nv_bfloat16 *row = static_cast<const __nv_bfloat16 *>(r.qkv) + (int64_t)seq * per_seq * HEAD_DIM;
    const __nv_bfloat16 *cs = static_cast<const __nv_bfloat16 *>(r.cos_table) + pos * HEAD_DIM;
    const __nv_bfloat16 *sn = static_cast<const __nv_bfloat16 *>(r.sin_table) + pos * HEAD_DIM;
    const int jobs = G + (store_kv ? 2 : 0);
    for (int j = wid; j < jobs; j += nw) {
        if (j < G) {
            const int qh = hk * G + j;
            const float4 v = norm_rope_head(row + (int64_t)qh * HEAD_DIM, static_cast<const __nv_bfloat16 *>(r.q_norm_w),
                                            cs, sn, r.eps, lane);
            *reinterpret_cast<float4 *>(sq + j * HEAD_DIM + lane * 4) = v;
            store_bf16x4(sqb + j * HEAD_DIM + lane * 4, v);
            if (store_q)
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

// Bytes of the selection's scratch, which shares the front of the dynamic shared memory with the gather rings.
__host__ __device__ inline int step_per_max(int C) { return ((C / STEP_CS) + 7) & ~7; }
__host__ __device__ inline size_t step_sel_bytes(int G, int C, int nw) {
    return (size_t)step_per_max(C) * 128 + (size_t)G * step_per_max(C) * 4 + (size_t)C * 4 + (size_t)step_per_max(C) * 8 +
           (size_t)step_slices(nw) * (8 * 2 + 4) * 4;       // + the slices' statistics (scores, keys)
}
__host__ __device__ inline size_t step_front_bytes(int G, int C, int stages, int nw) {
    const size_t ring = (size_t)nw * stages * 8192, sel = (step_sel_bytes(G, C, nw) + 127) & ~size_t(127);
    return ring > sel ? ring : sel;
}
__host__ __device__ inline size_t step_smem_bytes(int G, int C, int stages, int nw) {
    size_t b = step_front_bytes(G, C, stages, nw);
    b += ((size_t)(C / 32 + 1) * 4 + 15) & ~size_t(15);       // selection bits
    b += (size_t)G * HEAD_DIM * 4 + (size_t)G * HEAD_DIM * 2;  // query, float and bf16
    b += (size_t)STEP_CS * G * STEP_PART_LD * 4;               // partials received by the cluster's first CTA
    b += 608 * 4;                                              // histogram and candidates of the pick
    return (b + 127) & ~size_t(127);
}

// Grid (8 * ncl, heads), clusters of 8 CTAs along x, NW warps.
template <int STAGES, int GP, int NW>
__global__ void __launch_bounds__(NW * 32, 2) step_kernel(const StepParams p) {
    constexpr int STEP_THREADS = NW * 32, STEP_WARPS = NW, STEP_SUB = STEP_THREADS * STEP_LPT;
    constexpr int STEP_SLICES = step_slices(NW), SPL = STEP_SLICES / 32;    // slices per lane when they are combined
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint32_t s_vmask[STEP_WARPS][STAGES];
    __shared__ int s_flag;
    __shared__ int s_scan[40];
    __shared__ int ired[40];
    __shared__ uint16_t s_rows[step_pass(NW)];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.y, split = blockIdx.x, S = gridDim.x;
    const unsigned rank = cluster_rank();
    const int C = p.st.C, G = p.G;
    cluster_arrive();                                      // barrier 0: "my shared memory exists"; waited for ahead of the first remote store
    step_stamp(p, 0);

    // ---- shared memory map ------------------------------------------------------------------------------
    const int per_max = step_per_max(C);
    unsigned char *sumst = smem;                                              // [per_max][128] this CTA's summaries
    uint32_t *key = reinterpret_cast<uint32_t *>(smem);                       // [C] keys of all clusters, over sumst once it is scored
    float *zown = reinterpret_cast<float *>(smem + (size_t)per_max * 128);    // [G][per_max] scaled scores of this CTA's clusters
    float *cntf = zown + (size_t)G * per_max;                                 // [C] member counts
    float *smx = cntf + C, *smn = smx + per_max;                              // [per_max] key lengths of this CTA's clusters
    float *stat = smn + per_max;                                              // [slices][GP][2] (max, sum of exp) per query head
    int *stat2 = reinterpret_cast<int *>(stat + STEP_SLICES * GP * 2);        // [slices][4] smallest / largest key, clusters with members
    unsigned char *tail = smem + step_front_bytes(G, C, STAGES, NW);
    uint32_t *s_bits = reinterpret_cast<uint32_t *>(tail);
    tail += ((size_t)(C / 32 + 1) * 4 + 15) & ~size_t(15);
    float *sq = reinterpret_cast<float *>(tail);
    tail += (size_t)G * HEAD_DIM * 4;
    __nv_bfloat16 *sqb = reinterpret_cast<__nv_bfloat16 *>(tail);
    tail += (size_t)G * HEAD_DIM * 2;
    float *recv = reinterpret_cast<float *>(tail);                            // [8][G][132]
    tail += (size_t)STEP_CS * G * STEP_PART_LD * 4;
    int *hist = reinterpret_cast<int *>(tail);

    // ---- every load that depends on nothing goes out first, the ones sized by the cluster count right after ----
    const int n_c = min(max(p.st.n_c[h], 0), C);
    const int end = p.st.end[h], need = p.st.need[h];
    const int n = min(max(positions_of(p.n_dev, p.n_group, h), 0), p.st.capacity);
    uint2 qraw[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};                 // four query components per piece
    if (!p.rope.qkv) {
        const uint2 *qsrc = reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(p.q) + (int64_t)h * G * HEAD_DIM);
#pragma unroll
        for (int j = 0; j < 2; ++j)
            if (tid + j * STEP_THREADS < G * 32) qraw[j] = __ldg(qsrc + tid + j * STEP_THREADS);
    }
    const int chunk = max(16, (((n + S - 1) / S + 15) >> 4) << 4);            // multiples of 16: aligned label loads
    const int p0 = min(split * chunk, n), p1 = min(p0 + chunk, n);
    const int16_t *lab = p.st.labels + (int64_t)h * p.st.capacity;
    // a pass lists STEP_GROUPS groups of 8 labels per thread, so that the few positions by which a range exceeds
    // 8 labels per thread (n is rarely a multiple of the grid) do not cost a pass of their own
    uint4 raw[STEP_GROUPS];
#pragma unroll
    for (int j = 0; j < STEP_GROUPS; ++j) {
        raw[j] = make_uint4(0u, 0u, 0u, 0u);
        const int at = p0 + j * STEP_SUB + tid * STEP_LPT;
        if (at < p1) raw[j] = __ldg(reinterpret_cast<const uint4 *>(lab + at));
    }
    const bool active = end > 1 && need > 0 && n_c > 0;
    const int per = (((n_c + STEP_CS - 1) / STEP_CS) + 7) & ~7;              // clusters scored per CTA
    const int c_lo = min((int)rank * per, n_c), c_hi = min(c_lo + per, n_c), mine = active ? c_hi - c_lo : 0;
    {
        const int8_t *src = p.st.dir8 + ((int64_t)h * C + c_lo) * HEAD_DIM;
        for (int i = tid; i < mine * 8; i += STEP_THREADS) {
            const int c = i >> 3, k = i & 7;
            cp_async16(sumst + c * 128 + ((k ^ (c & 7)) << 4), src + (int64_t)c * HEAD_DIM + k * 16, 16);
        }
        // counts of all the head's clusters, key lengths of this CTA's (both 16-byte aligned: c_lo is a multiple of 8)
        const float *count = p.st.count + (int64_t)h * C;
        if (active)
            for (int i = tid; i < (n_c + 3) >> 2; i += STEP_THREADS) cp_async16(cntf + 4 * i, count + 4 * i, 16);
        const float *mmax = p.st.mmax + (int64_t)h * C + c_lo, *mmin = p.st.mmin + (int64_t)h * C + c_lo;
        for (int i = tid; i < (mine + 3) >> 2; i += STEP_THREADS) {
            cp_async16(smx + 4 * i, mmax + 4 * i, 16);
            cp_async16(smn + 4 * i, mmin + 4 * i, 16);
        }
        cp_async_commit();
    }
    pdl_wait();                                            // the query comes from the launch ahead
    pdl_trigger();
    step_stamp(p, 1);
    if (p.rope.qkv) {
        const int64_t pos = p.rope.pos[p.rope.pos_per_seq ? h / p.rope.H_kv : 0];
        const int s_kv = (int)min((int64_t)(S - 1), max((int64_t)0, pos / chunk));
        step_rope(p.rope, h, split == 0, split == s_kv, G, sq, sqb, STEP_WARPS);
    } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = tid + j * STEP_THREADS;
            if (i < G * 32) {
                *reinterpret_cast<uint2 *>(sqb + i * 4) = qraw[j];
                const __nv_bfloat162 *hh = reinterpret_cast<const __nv_bfloat162 *>(&qraw[j]);
                const float2 a = __bfloat1622float2(hh[0]), b = __bfloat1622float2(hh[1]);
                *reinterpret_cast<float4 *>(sq + i * 4) = make_float4(a.x, a.y, b.x, b.y);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    step_stamp(p, 9);

    // ---- scores of this CTA's clusters: q . dir8 on f16 tiles, 8 clusters per warp and chain.  A warp keeps the
    // scores of the clusters it scored in registers, takes their maximum and the sum of exp(score - maximum) per
    // query head with shuffles, and leaves exp(score - maximum): its clusters are one of the head's 32 "slices"
    // (8 CTAs x 4 warps), whose statistics every CTA later combines into the softmax over all clusters.
    const int nrow = lane >> 2, jq = lane & 3;
    float w_max = -INFINITY, w_sum = 0.f;
    {
        uint32_t qa[8][4];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const float *q0 = sq + nrow * HEAD_DIM + 32 * jq + 4 * ks;
            qa[ks][0] = nrow < G ? step_pack_half2(q0[0], q0[1]) : 0u;
            qa[ks][2] = nrow < G ? step_pack_half2(q0[2], q0[3]) : 0u;
            qa[ks][1] = qa[ks][3] = 0u;                                       // at most 8 query heads: rows 8..15 unused
        }
        // (rolled on purpose: the kernel runs every phase once, so its speed follows its code size)
#pragma unroll 1
        for (int cb = warp * 8; cb < mine; cb += STEP_WARPS * 8) {
            const int c = cb + nrow;
            int4 ra = make_int4(0, 0, 0, 0), rb = ra;
            if (c < mine) {
                ra = *reinterpret_cast<const int4 *>(sumst + c * 128 + (((2 * jq) ^ (c & 7)) << 4));
                rb = *reinterpret_cast<const int4 *>(sumst + c * 128 + (((2 * jq + 1) ^ (c & 7)) << 4));
            }
            const uint32_t wv[8] = {(uint32_t)ra.x, (uint32_t)ra.y, (uint32_t)ra.z, (uint32_t)ra.w,
                                    (uint32_t)rb.x, (uint32_t)rb.y, (uint32_t)rb.z, (uint32_t)rb.w};
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, acd[4] = {0.f, 0.f, 0.f, 0.f};   // two chains of four: half the latency
            int n2i = 0;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                n2i = __dp4a((int)wv[ks], (int)wv[ks], n2i);
                const uint32_t biased = wv[ks] ^ 0x80808080u;
                if (ks & 1) step_mma_f16(acd, qa[ks], step_bytes_to_half2(biased, 0x4140u), step_bytes_to_half2(biased, 0x4342u));
                else step_mma_f16(acc, qa[ks], step_bytes_to_half2(biased, 0x4140u), step_bytes_to_half2(biased, 0x4342u));
            }
            n2i += __shfl_xor_sync(0xffffffffu, n2i, 1);
            n2i += __shfl_xor_sync(0xffffffffu, n2i, 2);                      // |dir8|^2 of cluster cb + nrow
            const int na = __shfl_sync(0xffffffffu, n2i, (2 * jq) * 4);
            const int nb2 = __shfl_sync(0xffffffffu, n2i, (2 * jq + 1) * 4);
            float zz[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int cl = cb + 2 * jq + i;
                if (cl < mine && nrow < G) {
                    const float inv = 1.0f / fmaxf(sqrtf((float)(i ? nb2 : na)), 1e-12f);
                    const float pr = (acc[i] + acd[i]) * inv;
                    float e = pr >= 0.f ? smx[cl] * pr : smn[cl] * pr;
                    if (cntf[c_lo + cl] == 0.f) e = -INFINITY;
                    zz[i] = e * p.scale;
                    zown[nrow * per_max + cl] = zz[i];
                }
            }
            // running maximum and sum of exp(score - maximum) of the clusters this lane has seen
            const float mt = fmaxf(w_max, fmaxf(zz[0], zz[1]));
            if (mt > -INFINITY) {
                w_sum = w_sum * expf(w_max - mt) + expf(zz[0] - mt) + expf(zz[1] - mt);   // exp(-inf) = 0
                w_max = mt;
            }
        }
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {                                    // over the four lanes of a query head
            const float om = __shfl_xor_sync(0xffffffffu, w_max, o), os = __shfl_xor_sync(0xffffffffu, w_sum, o);
            const float mt = fmaxf(w_max, om);
            if (mt > -INFINITY) {
                w_sum = w_sum * expf(w_max - mt) + os * expf(om - mt);
                w_max = mt;
            }
        }
    }
    step_stamp(p, 2);
    cluster_wait();                                        // barrier 0: every CTA of the cluster is running
    {
        // this warp's statistics go to all 8 CTAs of the cluster (its own included): lane r < 8 stores to CTA r
        const int slice = (int)rank * STEP_WARPS + warp;
        const int g_src = lane >> 3;                                          // lanes 8 j .. 8 j + 7 carry query heads 4 k + j
#pragma unroll
        for (int g0 = 0; g0 < GP; g0 += 4) {
            const int g = g0 + g_src;
            const float vm = __shfl_sync(0xffffffffu, w_max, (g & 7) * 4), vs = __shfl_sync(0xffffffffu, w_sum, (g & 7) * 4);
            if (g < G) {
                const uint32_t a = remote_addr(stat + ((size_t)slice * GP + g) * 2, lane & 7);
                remote_store(a, vm);
                remote_store(a + 4, vs);
            }
        }
    }
    for (int i = tid; i < 512; i += STEP_THREADS) hist[i] = 0;               // for the pick's first pass
    cluster_arrive();                                      // barrier 1: the statistics of all slices are everywhere
    cluster_wait();
    step_stamp(p, 3);

    // ---- shared scores of this CTA's clusters -> keys, to all 8 CTAs --------------------------------------
    {
        // softmax over ALL the head's clusters per query head: maximum M and total T from the slices' statistics
        // (lane = slice); every warp derives them for itself
        float Mg[GP], iT[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            Mg[g] = 0.f; iT[g] = 0.f;
            if (g < G) {
                float2 st[SPL];
                float M = -INFINITY;
#pragma unroll
                for (int k = 0; k < SPL; ++k) {
                    st[k] = *reinterpret_cast<const float2 *>(stat + ((size_t)(lane + 32 * k) * GP + g) * 2);
                    M = fmaxf(M, st[k].x);
                }
                M = warp_max(M);
                float T = 0.f;
#pragma unroll
                for (int k = 0; k < SPL; ++k) T = fmaf(st[k].x > -INFINITY ? expf(st[k].x - M) : 0.f, st[k].y, T);
                T = warp_sum(T);
                Mg[g] = M > -INFINITY ? M : 0.f;
                iT[g] = T > 0.f ? 1.0f / T : 0.f;
            }
        }
        // four consecutive clusters per thread: sum over the query heads of each head's softmax share
        uint32_t kmin = 0xffffffffu, kmax = 0u;
        int nvalid = 0;
        const int c4 = tid * 4;
        if (c4 < mine) {
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int g = 0; g < GP; ++g)
                if (g < G) {
                    const float4 z = *reinterpret_cast<const float4 *>(zown + g * per_max + c4);
                    sc[0] = fmaf(expf(z.x - Mg[g]), iT[g], sc[0]);
                    sc[1] = fmaf(expf(z.y - Mg[g]), iT[g], sc[1]);
                    sc[2] = fmaf(expf(z.z - Mg[g]), iT[g], sc[2]);
                    sc[3] = fmaf(expf(z.w - Mg[g]), iT[g], sc[3]);
                }
            const float4 cn = *reinterpret_cast<const float4 *>(cntf + c_lo + c4);
            const float cnv[4] = {cn.x, cn.y, cn.z, cn.w};
            uint32_t kk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bool live = c4 + i < mine && cnv[i] > 0.f;
                kk[i] = float_key(live ? sc[i] : -INFINITY);
                if (live) { kmin = min(kmin, kk[i]); kmax = max(kmax, kk[i]); ++nvalid; }
            }
            const float4 kv = make_float4(__uint_as_float(kk[0]), __uint_as_float(kk[1]), __uint_as_float(kk[2]),
                                          __uint_as_float(kk[3]));
#pragma unroll
            for (unsigned dst = 0; dst < STEP_CS; ++dst) remote_store4(remote_addr(key + c_lo + c4, dst), kv);
        }
        kmin = __reduce_min_sync(0xffffffffu, kmin);
        kmax = __reduce_max_sync(0xffffffffu, kmax);
        nvalid = __reduce_add_sync(0xffffffffu, nvalid);
        if (lane < STEP_CS) {
            const uint32_t a = remote_addr(stat2 + ((int)rank * STEP_WARPS + warp) * 4, lane);
            asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(kmin), "r"(kmax), "r"((uint32_t)nvalid), "r"(0u)
                         : "memory");
        }
    }
    // selection bits: the pick writes the words that hold slots in use (nothing selected: cleared here), the rest are
    // zero, bit C (the always-read rows; C is a multiple of 32: bit 0 of the last word) is set
    {
        const int words = C / 32 + 1, used = (n_c + 31) >> 5;
        for (int wd = (active ? used : 0) + tid; wd < words; wd += STEP_THREADS) s_bits[wd] = wd == words - 1 ? 1u : 0u;
    }
    cluster_arrive();                                      // barrier 2: the keys of all clusters are everywhere
    cluster_wait();
    step_stamp(p, 10);

    // ---- every CTA derives the selection for itself ---------------------------------------------------------
    {
        uint32_t kmin = 0xffffffffu, kmax = 0u;
        int nvalid = 0;
#pragma unroll
        for (int k = 0; k < SPL; ++k) {
            const int4 v = *reinterpret_cast<const int4 *>(stat2 + (lane + 32 * k) * 4);
            kmin = min(kmin, (uint32_t)v.x); kmax = max(kmax, (uint32_t)v.y); nvalid += v.z;
        }
        kmin = __reduce_min_sync(0xffffffffu, kmin);
        kmax = __reduce_max_sync(0xffffffffu, kmax);
        nvalid = __reduce_add_sync(0xffffffffu, nvalid);
        pick_by_threshold<STEP_THREADS, float, true, true>(key, cntf, nullptr, hist, ired, n_c, need, active, kmin, kmax,
                                                           nvalid, s_bits);
        step_stamp(p, 11);
    }
    __syncthreads();                                       // the selection's scratch is free: the rings take its place
    step_stamp(p, 4);

    // ---- attention over this CTA's range of positions, rows taken straight from the labels ------------------
    WarpAttendT<STAGES> wa;
    wa.init(sqb, G, smem + warp * (STAGES * 8192), s_vmask[warp],
            static_cast<const char *>(p.K) + (int64_t)h * p.ksh * 2, static_cast<const char *>(p.V) + (int64_t)h * p.vsh * 2,
            p.ksr * 2, p.vsr * 2, p.scale_log2);
    int read_rows = 0;
    bool bad = false;
    for (int sub0 = p0; sub0 < p1; sub0 += step_pass(NW)) {
        uint32_t take = 0;
#pragma unroll
        for (int j = 0; j < STEP_GROUPS; ++j) {
            const int base = sub0 + j * STEP_SUB + tid * STEP_LPT;
            if (base < p1) {
                const int16_t *l16 = reinterpret_cast<const int16_t *>(&raw[j]);
#pragma unroll
                for (int i = 0; i < STEP_LPT; ++i) {
                    const unsigned l = (unsigned)(int)l16[i];
                    if (base + i < p1) {
                        if (l <= (unsigned)C) take |= ((s_bits[l >> 5] >> (l & 31)) & 1u) << (j * STEP_LPT + i);
                        else bad = true;
                    }
                }
            }
            if (base + step_pass(NW) < p1) raw[j] = __ldg(reinterpret_cast<const uint4 *>(lab + base + step_pass(NW)));
        }
        int total;
        int off = step_excl_scan<STEP_WARPS>(__popc(take), s_scan, total);
        while (take) {
            const int i = __ffs(take) - 1;
            take &= take - 1;
            s_rows[off++] = (uint16_t)((i >> 3) * STEP_SUB + tid * STEP_LPT + (i & 7));
        }
        __syncthreads();
        if (sub0 == p0) step_stamp(p, 12);
        read_rows += total;
        const int tiles = (total + TILE_ROWS - 1) / TILE_ROWS;
        const int tper = (tiles + STEP_WARPS - 1) / STEP_WARPS;
        const int t0 = min(warp * tper, tiles), t1 = min(t0 + tper, tiles);
        wa.run(t0, t1, [&](int row) { return row < total ? sub0 + (int)s_rows[row] : -1; });
        if (sub0 == p0) step_stamp(p, 13);
        __syncthreads();                                   // the list is rewritten by the next pass
    }
    step_stamp(p, 5);
    if (bad && p.st.status) atomicOr(p.st.status + h, SKV_ST_BAD_INDEX);
    float *red = reinterpret_cast<float *>(smem);          // [warp][g][132] over the rings, which are drained
    wa.store_partial(red, warp, G);
    __syncthreads();
    // this CTA's partial goes to the cluster's first CTA: thread t owns column t
    const bool col = tid < HEAD_DIM;                       // thread t < 128 owns column t of the partials
    const int tc = col ? tid : 0;
    for (int g = 0; g < G; ++g) {
        float M = NEG_BIG;
#pragma unroll
        for (int w = 0; w < STEP_WARPS; ++w) M = fmaxf(M, red[(w * G + g) * 132 + 128]);
        float dn = 0.f, nm = 0.f;
#pragma unroll
        for (int w = 0; w < STEP_WARPS; ++w) {
            const float *r = red + (w * G + g) * 132;
            const float f = fast_exp2(r[128] - M);
            dn += f * r[129];
            nm += f * r[tc];
        }
        float *dst = recv + ((size_t)rank * G + g) * STEP_PART_LD;
        if (col) remote_store(remote_addr(dst + tid, 0), nm);
        if (tid == 0) {
            remote_store(remote_addr(dst + 128, 0), M);
            remote_store(remote_addr(dst + 129, 0), dn);
            remote_store(remote_addr(dst + 130, 0), (float)read_rows);
        }
    }
    cluster_arrive();                                      // barrier 3: the cluster's partials are in its first CTA
    if (split == STEP_CS - 1) {
        // the selection for callers who look at it, written by a CTA that has nothing to merge, while it waits
        const int words = C / 32 + 1;
        if (p.selbits)
            for (int wd = tid; wd < words; wd += STEP_THREADS) p.selbits[(int64_t)h * words + wd] = s_bits[wd];
        if (p.w)
            for (int c = tid; c <= C; c += STEP_THREADS)
                p.w[(int64_t)h * (C + 1) + c] = (float)((s_bits[c >> 5] >> (c & 31)) & 1u);
    }
    cluster_wait();
    step_stamp(p, 6);
    if (rank != 0) return;

    // ---- the cluster's first CTA folds the 8 partials; with several clusters per head the last one merges ---
    __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);
    const int kcl = split / STEP_CS;                        // this cluster among the head's
    float rows_f = 0.f;
#pragma unroll
    for (int r = 0; r < STEP_CS; ++r) rows_f += recv[(size_t)r * G * STEP_PART_LD + 130];
    for (int g = 0; g < G; ++g) {
        float M = NEG_BIG;
#pragma unroll
        for (int r = 0; r < STEP_CS; ++r) M = fmaxf(M, recv[((size_t)r * G + g) * STEP_PART_LD + 128]);
        float dn = 0.f, nm = 0.f;
#pragma unroll
        for (int r = 0; r < STEP_CS; ++r) {
            const float *row = recv + ((size_t)r * G + g) * STEP_PART_LD;
            const float f = fast_exp2(row[128] - M);
            dn = fmaf(f, row[129], dn);
            nm = fmaf(f, row[tc], nm);
        }
        if (p.ncl == 1 && out) {
            if (col) store_out(out + ((int64_t)h * G + g) * HEAD_DIM + tid, dn > 0.f ? nm / dn : 0.f);
        } else {
            float *pa = p.part + (((int64_t)h * p.ncl + kcl) * G + g) * STEP_PART_LD;
            if (col) __stcg(pa + tid, nm);
            if (tid == 0) {
                __stcg(pa + 128, M);
                __stcg(pa + 129, dn);
                __stcg(pa + 130, rows_f);
            }
        }
    }
    if (p.ncl == 1 && out) {
        if (tid == 0 && p.cnt) p.cnt[h] = (int)rows_f;
        step_stamp(p, 7);
        return;
    }
    if (!out) {                                            // the output product merges the clusters' partials itself
        step_stamp(p, 7);
        return;
    }
    __syncthreads();                                       // every thread's partial stores are ordered before thread 0's fence
    if (tid == 0) {
        __threadfence();                                   // cumulative: the CTA's stores are visible before the ticket moves
        s_flag = atomicAdd(p.ticket + h, 1) == p.ncl - 1;
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();
    // the last of the head's clusters merges them all: every value is requested before any is used
    const float *src = p.part + (int64_t)h * p.ncl * G * STEP_PART_LD;
    float total_rows = 0.f;
    for (int g = 0; g < G; ++g) {
        float pm[STEP_CS], pd[STEP_CS], pn[STEP_CS], pr[STEP_CS];
#pragma unroll
        for (int k = 0; k < STEP_CS; ++k) {
            pm[k] = NEG_BIG; pd[k] = pn[k] = pr[k] = 0.f;
            if (k < p.ncl) {
                const float *row = src + ((size_t)k * G + g) * STEP_PART_LD;
                pm[k] = __ldcg(row + 128);
                pd[k] = __ldcg(row + 129);
                pn[k] = __ldcg(row + tc);
                if (g == 0) pr[k] = __ldcg(row + 130);
            }
        }
        float M = NEG_BIG;
#pragma unroll
        for (int k = 0; k < STEP_CS; ++k) M = fmaxf(M, pm[k]);
        float dn = 0.f, nm = 0.f;
#pragma unroll
        for (int k = 0; k < STEP_CS; ++k) {
            const float f = fast_exp2(pm[k] - M);
            dn = fmaf(f, pd[k], dn);
            nm = fmaf(f, pn[k], nm);
            total_rows += pr[k];
        }
        if (col) store_out(out + ((int64_t)h * G + g) * HEAD_DIM + tid, dn > 0.f ? nm / dn : 0.f);
    }
    if (tid == 0) {
        if (p.cnt) p.cnt[h] = (int)total_rows;
        p.ticket[h] = 0;                                   // ready for the next launch on this stream
    }
    step_stamp(p, 7);
}

using StepKern = void (*)(const StepParams);

// (a ring of three tiles per warp was measured: 35.0 against 35.2 us per layer at 8 heads, not worth 32 KB per CTA)
static int step_stages(int) { return STEP_STAGES; }
static StepKern step_kernel_for(int G, int) {
    return G <= 2 ? step_kernel<STEP_STAGES, 2, 4> : (G <= 4 ? step_kernel<STEP_STAGES, 4, 4> : step_kernel<STEP_STAGES, 8, 4>);
}

// The kernel's dynamic shared memory limit only ever grows: one record per device and kernel variant, shared by
// the occupancy query and the launch (a smaller request must not lower what a larger shape configured).
static int step_configure(StepKern kern, int G, int nw, size_t smem) {
    static size_t configured[64][3][2] = {};
    const int gsel = G <= 2 ? 0 : (G <= 4 ? 1 : 2), wsel = nw == 8;
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (configured[dev][gsel][wsel] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][gsel][wsel] = smem;
    }
    return SKV_OK;
}

// Clusters of 8 CTAs of `nw` warps that one launch can keep resident on this device for (G, C); cached per device
// and shape.
static int step_resident_clusters(int G, int C, int nw) {
    struct Entry { int dev, G, C, nw, n; };
    static Entry cache[32];
    static int used = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    for (int i = 0; i < used; ++i)
        if (cache[i].dev == dev && cache[i].G == G && cache[i].C == C && cache[i].nw == nw) return cache[i].n;
    const size_t smem = step_smem_bytes(G, C, step_stages(nw), nw);
    if ((int)smem > device_max_smem_optin()) return 0;
    StepKern kern = step_kernel_for(G, nw);
    if (step_configure(kern, G, nw, smem) != SKV_OK) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(STEP_CS * 64, 1, 1);
    cfg.blockDim = dim3(nw * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = STEP_CS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    if (used < 32) cache[used++] = Entry{dev, G, C, nw, n};
    return n;
}

static int step_warps_for(int, int, int) { return 4; }

}  // namespace skv

using namespace skv;

extern "C" void skv_debug_step_probe(void *dev_ptr) { skv::g_step_probe = static_cast<unsigned long long *>(dev_ptr); }

extern "C" int skv_step_clusters(int heads, int G, int C, int summary_bits) {
    if (heads <= 0 || G < 1 || G > 8 || C < 64 || (C & (C - 1)) || C > 2048 || summary_bits != 8) return 0;
    const int resident = step_resident_clusters(G, C, step_warps_for(heads, G, C));
    // More than one wave of clusters: the two launches serve better.  Measured at 64 heads (two waves): the one
    // launch is 4 us faster alone (32.8 against 36.9 us at 8k / 5 %) but, launched without programmatic
    // serialization, loses in the decode step (batch 8 x 8k: 3,800 against 4,448 tok/s); at 256 heads it loses alone.
    if (resident < heads) return 0;                         // more than one wave of clusters: the two-launch path streams better
    int ncl = resident / heads;
    return ncl > 8 ? 8 : ncl;
}

extern "C" int64_t skv_step_workspace_bytes(int heads, int G, int clusters) {
    if (heads <= 0 || G < 1 || G > 8 || clusters < 1 || clusters > 64) return SKV_E_RANGE;
    const int64_t part = (((int64_t)heads * clusters * G * STEP_PART_LD * 4) + 255) / 256 * 256;
    return part + (((int64_t)heads * 4) + 255) / 256 * 256;
}

extern "C" int skv_step(const skv_state *st, const void *q, int G, const int32_t *n_dev, int n_group, const void *K,
                        const void *V,
                        int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride, int64_t v_row_stride,
                        float *w, uint32_t *selbits, int32_t *cnt, void *out, void *workspace, int clusters,
                        float scale, const skv_rope *rope, void *stream) {
    if (!st || !n_dev || !K || !V || !workspace) return SKV_E_NULL;
    if (!q && !rope) return SKV_E_NULL;
    if (rope) {
        if (!rope->qkv || !rope->q_norm_w || !rope->k_norm_w || !rope->cos_table || !rope->sin_table || !rope->pos ||
            !rope->q_out || !rope->k_cache || !rope->v_cache)
            return SKV_E_NULL;
        if (rope->H_kv < 1 || rope->H < rope->H_kv || rope->H % rope->H_kv || rope->H / rope->H_kv != G ||
            st->heads % rope->H_kv)
            return SKV_E_RANGE;
        if (!aligned16(rope->qkv) || !aligned16(rope->q_out) || !aligned16(rope->k_cache) || !aligned16(rope->v_cache) ||
            rope->cache_row_stride % 8 || rope->cache_head_stride % 8 || rope->cache_batch_stride % 8)
            return SKV_E_ALIGN;
    }
    if (!st->count || !st->n_c || !st->end || !st->need || !st->labels || !st->mmax || !st->mmin || !st->dir8)
        return SKV_E_NULL;
    if (st->d != HEAD_DIM || G < 1 || G > 8) return SKV_E_DIM;
    if (st->C < 64 || (st->C & (st->C - 1)) || st->C > 2048 || clusters > STEP_CS) return SKV_E_DIM;
    if (st->summary_bits != 8) return SKV_E_RANGE;
    if (st->heads <= 0 || st->heads > 65535 || st->capacity <= 0 || clusters < 1 || clusters > 64 || n_group < 0)
        return SKV_E_RANGE;
    if (st->capacity % 8 || !aligned16(st->labels) || !aligned16(st->dir8) || !aligned16(workspace) || !aligned16(K) ||
        !aligned16(V) || (out && !aligned16(out)) || (q && !aligned16(q)))
        return SKV_E_ALIGN;
    if ((k_row_stride * 2) % 16 || (v_row_stride * 2) % 16 || (k_head_stride * 2) % 16 || (v_head_stride * 2) % 16 ||
        k_row_stride < HEAD_DIM || v_row_stride < HEAD_DIM)
        return SKV_E_ALIGN;
    const int nw = step_warps_for(st->heads, G, st->C);
    const size_t smem = step_smem_bytes(G, st->C, step_stages(nw), nw);
    if ((int)smem > device_max_smem_optin()) return SKV_E_DIM;
    StepParams p;
    p.st = *st; p.q = q; p.K = K; p.V = V; p.n_dev = n_dev; p.n_group = n_group; p.out = out; p.w = w; p.selbits = selbits; p.cnt = cnt;
    p.part = static_cast<float *>(workspace);
    p.ticket = reinterpret_cast<int32_t *>(static_cast<char *>(workspace) +
                                           (((int64_t)st->heads * clusters * G * STEP_PART_LD * 4) + 255) / 256 * 256);
    p.G = G; p.ncl = clusters;
    p.ksh = k_head_stride; p.ksr = k_row_stride; p.vsh = v_head_stride; p.vsr = v_row_stride;
    p.scale = scale; p.scale_log2 = scale * LOG2E;
    p.rope = rope ? *rope : skv_rope{};
    p.probe = g_step_probe;
    StepKern kern = step_kernel_for(G, nw);
    {
        const int rc = step_configure(kern, G, nw, smem);
        if (rc) return rc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(STEP_CS * clusters, st->heads, 1);
    cfg.blockDim = dim3(nw * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = STEP_CS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // The launch does not ask for programmatic serialization itself: measured on B200, a cluster launch scheduled
    // while the kernel ahead still runs costs the decode step 10 us per layer (its clusters start late), far more
    // than the early loads save.  It still triggers its dependents early (SKV_STEP_PDL=1 restores the attribute).
    static const bool step_pdl = [] { const char *e = getenv("SKV_STEP_PDL"); return e && e[0] == '1'; }();
    cfg.numAttrs = pdl_enabled() && step_pdl ? 2 : 1;
    SKV_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}
