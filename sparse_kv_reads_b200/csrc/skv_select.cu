// Cluster scoring from summaries, shared (per KV head) softmax-sum score, top-budget selection by a
// weighted radix select, and the ordered list of positions to read - one CTA per KV head, one launch.
//
// Bytes per head: n_c summaries (128 B int8 or 512 B float32 direction + 12 B) and one int16 label
// per cached position; everything else lives in shared memory.  The selection never sorts: it finds
// the threshold key t with  sum(count | key > t) < need  by four 8-bit radix passes over
// order-preserving integer keys, then settles exact ties in slot order, which reproduces "take
// clusters in decreasing score, lower slot first among equals, until the counts reach need".
#include "skv_common.cuh"

namespace skv {

constexpr int SEL_THREADS = 256;
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int SEL_MAX_CTAS = 64;          // CTAs that score one head's clusters in parallel

struct SelectParams {
    skv_state st;
    const void *q;
    int G;
    const int32_t *n_dev;
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
    float scale;
};

// Reduce `nv` (<= 16) per-thread values at once over the block: op = max (IS_MAX) or sum.
template <bool IS_MAX>
__device__ __forceinline__ void block_reduce_vec(float *v, int nv, float *red /* [16][SEL_WARPS] */) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int g = 0; g < nv; ++g) {
        float x = IS_MAX ? warp_max(v[g]) : warp_sum(v[g]);
        if (lane == 0) red[g * SEL_WARPS + wid] = x;
    }
    __syncthreads();
    for (int g = 0; g < nv; ++g) {
        float x = (lane < SEL_WARPS) ? red[g * SEL_WARPS + lane] : (IS_MAX ? -INFINITY : 0.f);
        v[g] = IS_MAX ? warp_max(x) : warp_sum(x);
    }
    __syncthreads();
}

// Grid (ctas, heads).  Every CTA scores a slice of the head's clusters and leaves the scaled scores in
// zbuf; the last CTA of the head to finish (atomic ticket, no waiting) forms the shared score, finds
// the threshold and writes the weights and the selection bits.
template <typename TQ>
__global__ void __launch_bounds__(SEL_THREADS) score_pick_kernel(const SelectParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_last;
    const int C = p.st.C, G = p.G, d = HEAD_DIM;
    const int h = blockIdx.y, b = blockIdx.x, nb = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    float *z = reinterpret_cast<float *>(smem_raw);                 // [G][C] (picking CTA)
    const int zfloats = p.shared_in ? 0 : G * C;
    uint32_t *key = reinterpret_cast<uint32_t *>(z + zfloats);      // [C]
    int *ci = reinterpret_cast<int *>(key + C);                     // [C]
    float *sq = reinterpret_cast<float *>(ci + C);                  // [G][128]
    float *red = sq + G * d;                                        // [16][SEL_WARPS]
    int *hist = reinterpret_cast<int *>(red + 16 * SEL_WARPS);      // [256]
    int *ired = hist + 256;                                         // [40]
    uint8_t *sel = reinterpret_cast<uint8_t *>(ired + 40);          // [C + 1]

    const int n_c = min(max(p.st.n_c[h], 0), C);
    const int end = p.st.end[h];
    const int need = p.st.need[h];
    const bool active = end > 1 && need > 0;
    const bool scoring = active && !p.shared_in;
    if (!scoring && b != 0) return;
    const float *count = p.st.count + (int64_t)h * C;
    float *zg = p.zbuf + (int64_t)h * G * C;

    if (scoring) {
        // ---- scores of this CTA's slice of clusters ------------------------------------------
        const TQ *q = static_cast<const TQ *>(p.q) + (int64_t)h * G * d;
        for (int i = tid; i < G * d; i += SEL_THREADS) sq[i] = load_as_float(q + i);
        __syncthreads();
        const int per = (((n_c + nb - 1) / nb) + 3) & ~3;
        const int c_lo = min(b * per, n_c), c_hi = min(c_lo + per, n_c);
        const float *mmax = p.st.mmax + (int64_t)h * C, *mmin = p.st.mmin + (int64_t)h * C;
        if (p.st.summary_bits == 8) {
            const int8_t *dir8 = p.st.dir8 + (int64_t)h * C * d;
            const int part = lane & 7, grp = lane >> 3;
#pragma unroll 2
            for (int c0 = c_lo + wid * 4; c0 < c_hi; c0 += SEL_WARPS * 4) {
                const int c = c0 + grp;
                const bool live = c < c_hi;
                float v[16];
                float cn = 0.f, mx = 0.f, mn = 0.f;
                if (live) {
                    const int4 raw = __ldg(reinterpret_cast<const int4 *>(dir8 + (int64_t)c * d + part * 16));
                    cn = count[c]; mx = mmax[c]; mn = mmin[c];
                    const int8_t *bb = reinterpret_cast<const int8_t *>(&raw);
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = (float)bb[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
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
                        __stcg(zg + g * C + c, e * p.scale);
                        if (p.e_out) p.e_out[((int64_t)h * G + g) * C + c] = e;
                    }
                }
            }
        } else {
            const float *sd = p.st.sum_dir + (int64_t)h * C * d;
#pragma unroll 2
            for (int c = c_lo + wid; c < c_hi; c += SEL_WARPS) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(sd + (int64_t)c * d + lane * 4));
                const float n2 = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
                const float inv = 1.0f / fmaxf(sqrtf(n2), 1e-12f);
                for (int g = 0; g < G; ++g) {
                    const float4 t = *reinterpret_cast<const float4 *>(sq + g * d + lane * 4);
                    const float dot = warp_sum(v.x * t.x + v.y * t.y + v.z * t.z + v.w * t.w);
                    if (lane == 0) {
                        const float pr = dot * inv;
                        float e = pr >= 0.f ? mmax[c] * pr : mmin[c] * pr;
                        if (count[c] == 0.f) e = -INFINITY;
                        __stcg(zg + g * C + c, e * p.scale);
                        if (p.e_out) p.e_out[((int64_t)h * G + g) * C + c] = e;
                    }
                }
            }
        }
        if (nb > 1) {
            __threadfence();
            __syncthreads();
            if (tid == 0) s_last = atomicAdd(p.ticket + h, 1) == nb - 1;
            __syncthreads();
            if (!s_last) return;
            __threadfence();
            if (tid == 0) p.ticket[h] = 0;
        } else {
            __syncthreads();
        }
    }
    // ---- the head's picking CTA from here on ---------------------------------------------------------
    for (int c = tid; c < C; c += SEL_THREADS) {
        ci[c] = c < n_c ? (int)count[c] : 0;
        sel[c] = 0;
    }
    if (tid == 0) {
        sel[C] = 1;
        if (!p.idx) p.cnt[h] = 0;                     // the attention kernel adds the rows it reads
    }
    if (scoring) {
        for (int i = tid; i < G * n_c; i += SEL_THREADS) {
            const int g = i / n_c, c = i - g * n_c;
            z[g * C + c] = __ldcg(zg + g * C + c);
        }
    }
    __syncthreads();
    if (scoring) {
        // ---- shared score: sum over the group of each query head's softmax over clusters ----
        float zm[16], tot[16];
        for (int g = 0; g < G; ++g) {
            float m = -INFINITY;
            for (int c = tid; c < n_c; c += SEL_THREADS) m = fmaxf(m, z[g * C + c]);
            zm[g] = m;
        }
        block_reduce_vec<true>(zm, G, red);
        for (int g = 0; g < G; ++g) {                     // z becomes exp(z - max): one exponential per score
            float s = 0.f;
            for (int c = tid; c < n_c; c += SEL_THREADS) {
                const float ex = (ci[c] > 0 && zm[g] > -INFINITY) ? expf(z[g * C + c] - zm[g]) : 0.f;
                z[g * C + c] = ex;
                s += ex;
            }
            tot[g] = s;
        }
        block_reduce_vec<false>(tot, G, red);
        for (int c = tid; c < C; c += SEL_THREADS) {
            float s = -INFINITY;
            if (c < n_c && ci[c] > 0) {
                s = 0.f;
                for (int g = 0; g < G; ++g) s += z[g * C + c] / tot[g];
            }
            key[c] = float_key(s);
            if (p.shared_out) p.shared_out[(int64_t)h * C + c] = s;
        }
    } else if (active) {
        const float *sin = p.shared_in + (int64_t)h * C;
        for (int c = tid; c < C; c += SEL_THREADS) {
            const float s = c < n_c ? sin[c] : -INFINITY;
            key[c] = float_key(s);
            if (p.shared_out) p.shared_out[(int64_t)h * C + c] = s;
        }
    }
    __syncthreads();

    if (active) {
        // ---- threshold: smallest key t with sum(count | key > t) < need ----------------------
        uint32_t prefix = 0;
        int above = 0;
        for (int level = 3; level >= 0; --level) {
            const int shift = level * 8;
            for (int i = tid; i < 256; i += SEL_THREADS) hist[i] = 0;
            __syncthreads();
            for (int c0 = wid * 32; c0 < n_c; c0 += SEL_THREADS) {
                // keys of one warp mostly share a digit: lanes with equal digits add up first, one atomic per digit
                const int c = c0 + lane;
                const uint32_t k = c < n_c ? key[c] : 0u;
                const bool match = c < n_c && ci[c] > 0 &&
                                   (level == 3 || (k >> (shift + 8)) == (prefix >> (shift + 8)));
                const unsigned live = __ballot_sync(0xffffffffu, match);
                if (match) {
                    const uint32_t dg = (k >> shift) & 255u;
                    const unsigned peers = __match_any_sync(live, dg);
                    const int sum = __reduce_add_sync(peers, ci[c]);
                    if (lane == __ffs(peers) - 1) atomicAdd(&hist[dg], sum);
                }
            }
            __syncthreads();
            if (wid == 0) {
                // lane owns digits [8*lane, 8*lane+8); suffix sums from the top digit down
                int loc[8], mine = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) { loc[i] = hist[lane * 8 + i]; mine += loc[i]; }
                int suf = mine;                               // inclusive suffix over lanes >= lane
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int t = __shfl_down_sync(0xffffffffu, suf, o);
                    if (lane + o < 32) suf += t;
                }
                int higher = suf - mine;                      // counts in digits above this lane's range
                // A(dg) = above + counts of digits > dg; smallest dg with A(dg) < need
                int best = 256;
                int run = higher;
#pragma unroll
                for (int i = 7; i >= 0; --i) {
                    if (above + run < need) best = lane * 8 + i;
                    run += loc[i];
                }
                // digits scanned top-down inside the lane, so `best` is the lowest passing digit of the lane
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
                // counts strictly above digit `best`
                int gt = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) gt += (lane * 8 + i > best) ? loc[i] : 0;
                gt = warp_sum_int(gt);
                if (lane == 0) { ired[0] = best; ired[1] = gt; }
            }
            __syncthreads();
            prefix |= (uint32_t)ired[0] << shift;
            above += ired[1];
            __syncthreads();
        }
        const uint32_t tau = prefix;
        int ties = 0;
        for (int c = tid; c < n_c; c += SEL_THREADS) {
            const uint32_t k = key[c];
            sel[c] = k > tau;
            ties += (k == tau);
        }
        ties = warp_sum_int(ties);
        if (lane == 0) ired[2 + wid] = ties;
        __syncthreads();
        if (wid == 0) {
            int t = lane < SEL_WARPS ? ired[2 + lane] : 0;
            t = warp_sum_int(t);
            // equal keys: slot order, each taken while the keys ranked before it stay under need
            int running = above;
            if (t > 0)
                for (int base = 0; base < n_c; base += 32) {
                    const int c = base + lane;
                    const bool tie = c < n_c && key[c] == tau;
                    const int mine = tie ? ci[c] : 0;
                    int inc = mine;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        int u = __shfl_up_sync(0xffffffffu, inc, o);
                        if (lane >= o) inc += u;
                    }
                    if (tie) sel[c] = (running + inc - mine) < need;
                    running += __shfl_sync(0xffffffffu, inc, 31);
                }
        }
        __syncthreads();
    }
    // ---- weights and selection bits out ---------------------------------------------------------
    float *w = p.w + (int64_t)h * (C + 1);
    for (int c = tid; c <= C; c += SEL_THREADS) w[c] = sel[c] ? 1.f : 0.f;
    const int words = C / 32 + 1;
    uint32_t *bits = p.selbits + (int64_t)h * words;
    for (int wd = tid; wd < words; wd += SEL_THREADS) {
        uint32_t v = 0;
        for (int i = 0; i < 32; ++i) {
            const int c = wd * 32 + i;
            if (c <= C && sel[c]) v |= 1u << i;
        }
        bits[wd] = v;
    }
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
    const int nn = min(max(p.n_dev[0], 0), p.st.capacity);
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
    b += 16 * SEL_WARPS * 4 + 256 * 4 + 40 * 4;
    b += C + 1 + 16;
    return (b + 15) & ~size_t(15);
}

static int64_t select_ws_bytes(int heads, int G, int C) {
    int64_t z = ((int64_t)heads * G * C * 4 + 255) / 256 * 256;
    int64_t t = ((int64_t)heads * 4 + 255) / 256 * 256;
    int64_t bits = ((int64_t)heads * (C / 32 + 1) * 4 + 255) / 256 * 256;
    return z + t + bits;
}

}  // namespace skv

using namespace skv;

extern "C" int64_t skv_select_workspace_bytes(int heads, int G, int C) {
    if (heads <= 0 || G < 1 || G > 16 || C < 16 || (C & (C - 1)) || C > 16384) return SKV_E_RANGE;
    return select_ws_bytes(heads, G, C);
}

extern "C" int skv_select(const skv_state *st, const void *q, int dtype, int G, const int32_t *n_dev, float *w,
                          uint32_t *selbits, int32_t *idx, int64_t idx_stride, int32_t *cnt, const float *shared_in,
                          float *shared_out, float *e_out, void *workspace, float scale, void *stream) {
    if (!st || !n_dev || !w || !cnt || !workspace) return SKV_E_NULL;
    if (!shared_in && !q) return SKV_E_NULL;
    if (!st->count || !st->n_c || !st->end || !st->need || !st->labels || !st->mmax || !st->mmin) return SKV_E_NULL;
    if (st->d != HEAD_DIM) return SKV_E_DIM;
    if (st->C < 16 || (st->C & (st->C - 1)) || st->C > 16384) return SKV_E_DIM;
    if (G < 1 || G > 16) return SKV_E_DIM;
    if (dtype != SKV_BF16 && dtype != SKV_F32) return SKV_E_DTYPE;
    if (st->summary_bits != 8 && st->summary_bits != 32) return SKV_E_RANGE;
    if (st->summary_bits == 8 ? !st->dir8 : !st->sum_dir) return SKV_E_NULL;
    if (st->heads <= 0 || st->heads > 65535 || st->capacity <= 0 || (idx && idx_stride < st->capacity)) return SKV_E_RANGE;
    if (st->capacity % 8 || !aligned16(st->labels) || !aligned16(workspace)) return SKV_E_ALIGN;
    if (st->summary_bits == 8 ? !aligned16(st->dir8) : !aligned16(st->sum_dir)) return SKV_E_ALIGN;
    const size_t smem = select_smem(G, st->C, shared_in == nullptr);
    if ((int)smem > device_max_smem_optin()) return SKV_E_DIM;
    SelectParams p;
    p.st = *st; p.q = q; p.G = G; p.n_dev = n_dev; p.w = w; p.idx = idx; p.idx_stride = idx_stride; p.cnt = cnt;
    p.shared_in = shared_in; p.shared_out = shared_out; p.e_out = e_out; p.scale = scale;
    char *ws = static_cast<char *>(workspace);
    p.zbuf = reinterpret_cast<float *>(ws);
    ws += ((int64_t)st->heads * G * st->C * 4 + 255) / 256 * 256;
    p.ticket = reinterpret_cast<int32_t *>(ws);
    ws += ((int64_t)st->heads * 4 + 255) / 256 * 256;
    p.selbits = selbits ? selbits : reinterpret_cast<uint32_t *>(ws);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto kern = dtype == SKV_BF16 ? score_pick_kernel<__nv_bfloat16> : score_pick_kernel<float>;
    static size_t configured[64][2] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (smem > 48 * 1024 && configured[dev][dtype] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][dtype] = smem;
    }
    int ctas = (2 * device_sm_count() + st->heads - 1) / st->heads;
    ctas = ctas < 1 ? 1 : (ctas > SEL_MAX_CTAS ? SEL_MAX_CTAS : ctas);
    if (shared_in) ctas = 1;
    kern<<<dim3(ctas, st->heads), SEL_THREADS, smem, s>>>(p);
    if (idx) list_kernel<<<st->heads, 512, (st->C / 32 + 1) * 4, s>>>(p);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}
