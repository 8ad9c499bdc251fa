// Insertion of the keys that leave the recent window into their nearest clusters, with the two-way
// split of a cluster that passes its head's cap done inside the same kernel: one CTA per
// (layer, sequence, KV head), every layer of the model in one launch.
//
// Per inserted key a CTA reads the key row, the n_c centroids (128 B int8 or 512 B float32 each) and
// one direction-sum row (read + write).  A split additionally scans the head's int16 labels for the
// members (2 B per clustered position), stages the members' unit directions in shared memory once and
// runs every pass of the 2-means / median cut from there.
#include "skv_common.cuh"

namespace skv {

constexpr int INS_THREADS = 512;
constexpr int INS_WARPS = INS_THREADS / 32;

struct InsertParams {
    skv_state st;
    const void *const *k_layers;
    int hpl;
    int64_t ksh, ksr;
    const int32_t *n_dev;
    int n_group;
    int window;
    double budget;
    float delta;
    int reset_at;
    int max_members;
    float capk;
    int var_min;
};

// shared-memory views used by the split
struct SplitSmem {
    float *U;        // [max_members][128] unit directions of the members
    float *mag;      // [max_members]
    float *proj;     // [max_members]
    int *mem;        // [max_members] positions
    uint8_t *side;   // [max_members]
};

struct ArgBest {
    float v;
    int i;
};
// larger value wins; equal values: the lower index (first maximum)
__device__ __forceinline__ ArgBest better_max(ArgBest a, ArgBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ArgBest warp_argmax(ArgBest x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better_max(x, y);
    }
    return x;
}

// Split cluster `c` of entry `e` in two; the second half takes slot `slot_new`.  Returns (to every
// thread) whether the split was done.  The rule: 2-means on the members' unit directions seeded with
// the first member and the member least similar to it, four updates; if a half would hold under a
// quarter of the members, cut at the median projection on the line between the two centroids.
template <typename T>
__device__ bool split_cluster(const InsertParams &p, int e, const T *Kh, const float *s_mu, int c, int slot_new,
                              int stop, const SplitSmem &sm, float *sa, float *sb, float *sdiff, float *fred,
                              int *ired) {
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int C = p.st.C;
    int16_t *lab = p.st.labels + (int64_t)e * p.st.capacity;

    // 1. members in position order
    const int vecs = (stop + 7) >> 3;
    const int per = (vecs + INS_THREADS - 1) / INS_THREADS;
    const int v0 = min(tid * per, vecs), v1 = min(v0 + per, vecs);
    int mine = 0;
    for (int v = v0; v < v1; ++v) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(lab + v * 8);
        const int16_t *l8 = reinterpret_cast<const int16_t *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int pos = v * 8 + i;
            mine += (pos >= 1 && pos < stop && l8[i] == c);
        }
    }
    int m;
    int off = block_excl_scan(mine, ired, m);
    if (m > p.max_members || m < 2) {
        if (tid == 0 && m > p.max_members && p.st.status) atomicOr(p.st.status + e, SKV_ST_SPLIT_TOO_BIG);
        return false;
    }
    for (int v = v0; v < v1; ++v) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(lab + v * 8);
        const int16_t *l8 = reinterpret_cast<const int16_t *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int pos = v * 8 + i;
            if (pos >= 1 && pos < stop && l8[i] == c) sm.mem[off++] = pos;
        }
    }
    __syncthreads();
    // 2. stage unit directions and lengths
    const float4 mu4 = *reinterpret_cast<const float4 *>(s_mu + lane * 4);
    for (int j = wid; j < m; j += INS_WARPS) {
        float4 k = load4(Kh + (int64_t)sm.mem[j] * p.ksr + lane * 4);
        k.x -= mu4.x; k.y -= mu4.y; k.z -= mu4.z; k.w -= mu4.w;
        const float mg = sqrtf(warp_sum(k.x * k.x + k.y * k.y + k.z * k.z + k.w * k.w));
        const float inv = 1.0f / fmaxf(mg, 1e-12f);
        *reinterpret_cast<float4 *>(sm.U + j * HEAD_DIM + lane * 4) = make_float4(k.x * inv, k.y * inv, k.z * inv, k.w * inv);
        if (lane == 0) sm.mag[j] = mg;
    }
    __syncthreads();
    // 3. seeds: first member, and the member least similar to it (first minimum)
    if (tid < HEAD_DIM) sa[tid] = sm.U[tid];
    __syncthreads();
    {
        const float4 a4 = *reinterpret_cast<const float4 *>(sa + lane * 4);
        for (int j = wid; j < m; j += INS_WARPS) {
            const float4 u = *reinterpret_cast<const float4 *>(sm.U + j * HEAD_DIM + lane * 4);
            const float s = warp_sum(u.x * a4.x + u.y * a4.y + u.z * a4.z + u.w * a4.w);
            if (lane == 0) sm.proj[j] = s;
        }
    }
    __syncthreads();
    if (wid == 0) {
        ArgBest b{-INFINITY, 0x7fffffff};
        for (int j = lane; j < m; j += 32) b = better_max(b, ArgBest{-sm.proj[j], j});
        b = warp_argmax(b);
        if (lane == 0) ired[0] = b.i;
    }
    __syncthreads();
    const int far = ired[0];
    if ((unsigned)far >= (unsigned)m) {                   // NaN similarities (a non-finite member): leave the cluster whole
        if (tid == 0 && p.st.status) atomicOr(p.st.status + e, SKV_ST_BAD_INDEX);
        return false;
    }
    if (tid < HEAD_DIM) sb[tid] = sm.U[far * HEAD_DIM + tid];
    __syncthreads();
    // 4. 2-means: four updates, then the final sides with the projections
    for (int it = 0; it <= 4; ++it) {
        if (it == 4 && tid < HEAD_DIM) sdiff[tid] = sb[tid] - sa[tid];
        if (it == 4) __syncthreads();
        {
            const float4 a4 = *reinterpret_cast<const float4 *>(sa + lane * 4);
            const float4 b4 = *reinterpret_cast<const float4 *>(sb + lane * 4);
            const float4 d4 = *reinterpret_cast<const float4 *>(sdiff + lane * 4);
            for (int j = wid; j < m; j += INS_WARPS) {
                const float4 u = *reinterpret_cast<const float4 *>(sm.U + j * HEAD_DIM + lane * 4);
                const float da = warp_sum(u.x * a4.x + u.y * a4.y + u.z * a4.z + u.w * a4.w);
                const float db = warp_sum(u.x * b4.x + u.y * b4.y + u.z * b4.z + u.w * b4.w);
                if (it == 4) {
                    const float pj = warp_sum(u.x * d4.x + u.y * d4.y + u.z * d4.z + u.w * d4.w);
                    if (lane == 0) sm.proj[j] = pj;
                }
                if (lane == 0) sm.side[j] = db > da;
            }
        }
        __syncthreads();
        if (it == 4) break;
        float s0 = 0.f, s1 = 0.f;
        int n1 = 0;
        if (tid < HEAD_DIM)
            for (int j = 0; j < m; ++j) {
                const float u = sm.U[j * HEAD_DIM + tid];
                if (sm.side[j]) { s1 += u; ++n1; } else s0 += u;
            }
        const float q0 = block_sum(tid < HEAD_DIM ? s0 * s0 : 0.f, fred);
        const float q1 = block_sum(tid < HEAD_DIM ? s1 * s1 : 0.f, fred);
        if (tid == 0) ired[1] = n1;
        __syncthreads();
        n1 = ired[1];
        if (tid < HEAD_DIM) {
            if (m - n1 > 0) sa[tid] = s0 / fmaxf(sqrtf(q0), 1e-12f);
            if (n1 > 0) sb[tid] = s1 / fmaxf(sqrtf(q1), 1e-12f);
        }
        __syncthreads();
    }
    // 5. lopsided -> median cut on the projections (ties by member order)
    int n1 = 0;
    for (int j = tid; j < m; j += INS_THREADS) n1 += sm.side[j];
    n1 = warp_sum_int(n1);
    if (lane == 0) ired[2 + wid] = n1;
    __syncthreads();
    n1 = 0;
    for (int w = 0; w < INS_WARPS; ++w) n1 += ired[2 + w];
    __syncthreads();
    if ((float)n1 < 0.25f * (float)m || (float)n1 > 0.75f * (float)m) {
        const int halfm = m / 2;
        for (int j = tid; j < m; j += INS_THREADS) {
            const float pj = sm.proj[j];
            int rank = 0;
            for (int i = 0; i < m; ++i) {
                const float pi = sm.proj[i];
                rank += (pi < pj) || (pi == pj && i < j);
            }
            sm.side[j] = rank >= halfm;
        }
        __syncthreads();
    }
    // 6. both halves' summaries (member order), centroids, 8-bit copies, labels
    float s0 = 0.f, s1 = 0.f;
    if (tid < HEAD_DIM)
        for (int j = 0; j < m; ++j) {
            const float u = sm.U[j * HEAD_DIM + tid];
            if (sm.side[j]) s1 += u; else s0 += u;
        }
    const float q0 = block_sum(tid < HEAD_DIM ? s0 * s0 : 0.f, fred);
    const float q1 = block_sum(tid < HEAD_DIM ? s1 * s1 : 0.f, fred);
    const int64_t r0 = (int64_t)e * C + c, r1 = (int64_t)e * C + slot_new;
    if (tid < HEAD_DIM) {
        p.st.sum_dir[r0 * HEAD_DIM + tid] = s0;
        p.st.sum_dir[r1 * HEAD_DIM + tid] = s1;
        const float u0 = s0 / fmaxf(sqrtf(q0), 1e-12f), u1 = s1 / fmaxf(sqrtf(q1), 1e-12f);
        p.st.cent[r0 * HEAD_DIM + tid] = u0;
        p.st.cent[r1 * HEAD_DIM + tid] = u1;
        if (p.st.summary_bits == 8) {
            const int8_t b0 = quant8(u0), b1 = quant8(u1);
            p.st.cent8[r0 * HEAD_DIM + tid] = b0;
            p.st.cent8[r1 * HEAD_DIM + tid] = b1;
            p.st.dir8[r0 * HEAD_DIM + tid] = b0;
            p.st.dir8[r1 * HEAD_DIM + tid] = b1;
        }
    }
    for (int j = tid; j < m; j += INS_THREADS)
        if (sm.side[j]) lab[sm.mem[j]] = (int16_t)slot_new;
    if (wid == 0) {
        float x0 = 0.f, x1 = 0.f, y0 = INFINITY, y1 = INFINITY;
        int c1 = 0;
        for (int j = lane; j < m; j += 32) {
            const float mg = sm.mag[j];
            if (sm.side[j]) { x1 = fmaxf(x1, mg); y1 = fminf(y1, mg); ++c1; }
            else { x0 = fmaxf(x0, mg); y0 = fminf(y0, mg); }
        }
        x0 = warp_max(x0); x1 = warp_max(x1);
        y0 = -warp_max(-y0); y1 = -warp_max(-y1);
        c1 = warp_sum_int(c1);
        if (lane == 0) {
            p.st.mmax[r0] = x0; p.st.mmax[r1] = x1;
            p.st.mmin[r0] = y0; p.st.mmin[r1] = y1;
            p.st.count[r0] = (float)(m - c1);
            p.st.count[r1] = (float)c1;
            p.st.n_c[e] = slot_new + 1;
            p.st.nsplit[e] += 1;
        }
    }
    __syncthreads();
    return true;
}

template <typename T>
__global__ void __launch_bounds__(INS_THREADS) insert_kernel(const InsertParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(16) float s_kn[HEAD_DIM], s_mu[HEAD_DIM], sa[HEAD_DIM], sb[HEAD_DIM], sdiff[HEAD_DIM];
    __shared__ float fred[32];
    __shared__ int ired[40];
    __shared__ float s_bv[INS_WARPS];
    __shared__ int s_bi[INS_WARPS];
    __shared__ int s_dec[2];

    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int C = p.st.C;
    const int layer = e / p.hpl, hh = e % p.hpl;
    const T *Kh = static_cast<const T *>(p.k_layers[layer]) + (int64_t)hh * p.ksh;

    SplitSmem sm;
    sm.U = reinterpret_cast<float *>(smem_raw);
    sm.mag = sm.U + (size_t)p.max_members * HEAD_DIM;
    sm.proj = sm.mag + p.max_members;
    sm.mem = reinterpret_cast<int *>(sm.proj + p.max_members);
    sm.side = reinterpret_cast<uint8_t *>(sm.mem + p.max_members);

    const int n = positions_of(p.n_dev, p.n_group, hh);
    const int old_end = p.st.end[e];
    int n_act = min(p.st.n_c[e], C);                      // a corrupt count must not index past the slots
    int new_end = max(max(n - p.window, 1), old_end);
    new_end = min(new_end, p.st.capacity);
    if (n_act <= 0) new_end = old_end;                    // nothing fitted yet: the host builds first
    const float cap = p.st.cap[e];
    const float vthr = p.st.vthr ? p.st.vthr[e] : INFINITY;
    const bool by_spread = vthr < INFINITY;
    float mu = 0.f, ks = 0.f;
    if (tid < HEAD_DIM) {
        mu = p.st.mu_ref[(int64_t)e * HEAD_DIM + tid];
        ks = p.st.ksum[(int64_t)e * HEAD_DIM + tid];
        s_mu[tid] = mu;
    }
    int16_t *lab = p.st.labels + (int64_t)e * p.st.capacity;
    const bool q8 = p.st.summary_bits == 8;

    for (int pos = old_end; pos < new_end; ++pos) {
        float kr = 0.f;
        if (tid < HEAD_DIM) {
            const float k = load_as_float(Kh + (int64_t)pos * p.ksr + tid);
            ks += k;
            kr = k - mu;
        }
        const float mag = sqrtf(block_sum(kr * kr, fred));
        if (tid < HEAD_DIM) s_kn[tid] = kr / fmaxf(mag, 1e-12f);
        __syncthreads();
        // nearest centroid among the n_act slots in use; first maximum wins
        ArgBest best{-INFINITY, 0x7fffffff};
        if (q8) {
            const int8_t *c8 = p.st.cent8 + (int64_t)e * C * HEAD_DIM;
            const int part = lane & 7, grp = lane >> 3;
            float kn[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) kn[i] = s_kn[part * 16 + i];
#pragma unroll 4
            for (int c0 = wid * 4; c0 < n_act; c0 += INS_WARPS * 4) {
                const int c = c0 + grp;
                float dot = 0.f;
                if (c < n_act) {
                    const int4 raw = *reinterpret_cast<const int4 *>(c8 + (int64_t)c * HEAD_DIM + part * 16);
                    const int8_t *b = reinterpret_cast<const int8_t *>(&raw);
#pragma unroll
                    for (int i = 0; i < 16; ++i) dot = fmaf((float)b[i], kn[i], dot);
                }
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                dot += __shfl_xor_sync(0xffffffffu, dot, 4);
                if (c < n_act) best = better_max(best, ArgBest{dot, c});
            }
        } else {
            const float *cf = p.st.cent + (int64_t)e * C * HEAD_DIM;
            const float4 k4 = *reinterpret_cast<const float4 *>(s_kn + lane * 4);
#pragma unroll 4
            for (int c = wid; c < n_act; c += INS_WARPS) {
                const float4 v = *reinterpret_cast<const float4 *>(cf + (int64_t)c * HEAD_DIM + lane * 4);
                const float dot = warp_sum(v.x * k4.x + v.y * k4.y + v.z * k4.z + v.w * k4.w);
                best = better_max(best, ArgBest{dot, c});
            }
        }
        best = warp_argmax(best);
        if (lane == 0) { s_bv[wid] = best.v; s_bi[wid] = best.i; }
        __syncthreads();
        if (wid == 0) {
            ArgBest b = lane < INS_WARPS ? ArgBest{s_bv[lane], s_bi[lane]} : ArgBest{-INFINITY, 0x7fffffff};
            b = warp_argmax(b);
            if (lane == 0) s_dec[0] = b.i;
        }
        __syncthreads();
        const int bi = s_dec[0];
        if ((unsigned)bi >= (unsigned)n_act) {
            // A key with an Inf or NaN component makes every dot product NaN, no slot beats the sentinel, and
            // there is no nearest cluster: the position joins the always-read rows instead, and the head is flagged.
            if (tid == 0) {
                lab[pos] = (int16_t)C;
                if (p.st.status) atomicOr(p.st.status + e, SKV_ST_BAD_INDEX);
            }
            __syncthreads();
            continue;
        }
        const int64_t row = (int64_t)e * C + bi;
        // fold the key into its cluster's summary
        float sd = 0.f;
        if (tid < HEAD_DIM) {
            sd = p.st.sum_dir[row * HEAD_DIM + tid] + s_kn[tid];
            p.st.sum_dir[row * HEAD_DIM + tid] = sd;
        }
        float n2 = 0.f;
        if (q8 || by_spread) n2 = block_sum(sd * sd, fred);
        if (q8 && tid < HEAD_DIM) p.st.dir8[row * HEAD_DIM + tid] = quant8(sd / fmaxf(sqrtf(n2), 1e-12f));
        if (tid == 0) {
            p.st.mmax[row] = fmaxf(p.st.mmax[row], mag);
            p.st.mmin[row] = fminf(p.st.mmin[row], mag);
            const float cn = p.st.count[row] + 1.0f;
            p.st.count[row] = cn;
            lab[pos] = (int16_t)bi;
            int dec = 0;
            // over the size cap (which may grow with the clustered keys), or its directions spread too widely
            const bool wide = by_spread && (1.0f - n2 / (cn * cn) > vthr) && cn >= (float)p.var_min;
            if ((cn > fmaxf(cap, p.capk * (float)pos) || wide) && cn >= 2.0f) {
                if (n_act < C) dec = 1;
                else if (p.st.status) atomicOr(p.st.status + e, SKV_ST_NO_SLOT);
            }
            s_dec[1] = dec;
        }
        __syncthreads();                                  // label and count visible to the whole CTA
        if (s_dec[1]) {
            if (split_cluster<T>(p, e, Kh, s_mu, bi, n_act, pos + 1, sm, sa, sb, sdiff, fred, ired)) ++n_act;
        }
        __syncthreads();
    }
    // lengths, budget in keys, drift and reset flags
    if (new_end > old_end && tid < HEAD_DIM) p.st.ksum[(int64_t)e * HEAD_DIM + tid] = ks;
    const int nb = new_end - 1;
    float dv = 0.f;
    if (tid < HEAD_DIM) {
        const float mu_t = ks / (float)max(nb, 1);
        dv = (mu_t - mu) * (mu_t - mu);
    }
    const float dist = sqrtf(block_sum(dv, fred));
    if (tid == 0) {
        p.st.end[e] = new_end;
        p.st.need[e] = nb > 0 ? (int)ceil(p.budget * (double)nb) : 0;
        int f = 0;
        if (nb > 0 && dist > p.delta * p.st.rbar[e]) f |= SKV_FLAG_DRIFT;
        if (p.reset_at > 0 && n_act >= p.reset_at) f |= SKV_FLAG_RESET;
        if (f) p.st.flags[e] |= f;
    }
}

static size_t insert_smem(int max_members) { return ((size_t)max_members * (HEAD_DIM * 4 + 4 + 4 + 4 + 1) + 15) & ~size_t(15); }

}  // namespace skv

using namespace skv;

extern "C" int skv_insert_max_members(void) {
    const int room = device_max_smem_optin() - 8 * 1024;     // static shared memory and slack
    return room / (HEAD_DIM * 4 + 13);
}

extern "C" int skv_insert(const skv_state *st, const void *const *k_layers, int heads_per_layer, int dtype,
                          int64_t k_head_stride, int64_t k_row_stride, const int32_t *n_dev, int n_group, int window,
                          double budget,
                          float delta, int reset_at, int max_members, float capk, int var_min, void *stream) {
    if (!st || !k_layers || !n_dev) return SKV_E_NULL;
    if (!st->sum_dir || !st->cent || !st->mmax || !st->mmin || !st->count || !st->n_c || !st->cap || !st->rbar ||
        !st->ksum || !st->mu_ref || !st->flags || !st->nsplit || !st->end || !st->need || !st->labels)
        return SKV_E_NULL;
    if (st->d != HEAD_DIM) return SKV_E_DIM;
    if (st->C < 16 || (st->C & (st->C - 1)) || st->C > 16384) return SKV_E_DIM;
    if (dtype != SKV_BF16 && dtype != SKV_F32) return SKV_E_DTYPE;
    if (st->summary_bits != 8 && st->summary_bits != 32) return SKV_E_RANGE;
    if (st->summary_bits == 8 && (!st->dir8 || !st->cent8)) return SKV_E_NULL;
    if (st->heads <= 0 || heads_per_layer <= 0 || st->heads % heads_per_layer || window < 0 || budget < 0.0 ||
        st->capacity <= 0 || reset_at < 0 || capk < 0.f || var_min < 0 || n_group < 0)
        return SKV_E_RANGE;
    if (max_members < 2 || max_members > skv_insert_max_members()) return SKV_E_RANGE;
    const int esz = dtype == SKV_BF16 ? 2 : 4;
    if (st->capacity % 8 || !aligned16(st->labels) || !aligned16(st->sum_dir) || !aligned16(st->cent)) return SKV_E_ALIGN;
    if ((k_row_stride * esz) % 16 || (k_head_stride * esz) % 16 || k_row_stride < HEAD_DIM) return SKV_E_ALIGN;
    if (st->summary_bits == 8 && !aligned16(st->cent8)) return SKV_E_ALIGN;
    InsertParams p;
    p.st = *st; p.k_layers = k_layers; p.hpl = heads_per_layer; p.ksh = k_head_stride; p.ksr = k_row_stride;
    p.n_dev = n_dev; p.n_group = n_group; p.window = window; p.budget = budget; p.delta = delta; p.reset_at = reset_at;
    p.max_members = max_members; p.capk = capk; p.var_min = var_min;
    const size_t smem = insert_smem(max_members);
    auto kern = dtype == SKV_BF16 ? insert_kernel<__nv_bfloat16> : insert_kernel<float>;
    static size_t configured[64][2] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (smem > 32 * 1024 && configured[dev][dtype] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][dtype] = smem;
    }
    kern<<<st->heads, INS_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}
