// Prompt fit of the cluster state: mean and centring, cosine k-means (float32 FFMA GEMM with a fused
// arg-max), position-ordered accumulation of the summaries, division of the clusters over the cap, the
// 8-bit copies; and the recentring rebuild that keeps the centroids.  Host-orchestrated (several
// launches, one device->host read per split round), used at the end of the prompt, never inside
// the decode graph.
//
// Numerics: the assignment needs float32-grade dot products (a 1e-5 relative error already moves
// percents of the labels after ten Lloyd steps), so the [keys x 128] . [128 x centroids] product
// runs on the CUDA cores in float32 with sequential-k accumulation, not on reduced-precision tensor
// tiles.  Every per-cluster sum is taken in position order by one warp, so reruns are bit-identical.
#include "skv_common.cuh"

namespace skv {

constexpr int MEAN_CHUNKS = 64;          // row chunks of the two-level column sums
constexpr int KWAY_MAX = 128;            // most parts one cluster is divided into at the fit

struct FitView {
    skv_state st;
    const int32_t *list;      // entry -> head of st (null: identity)
    int entries;
    int end;                  // clustered positions are [1, end)
    int m;                    // end - 1
    int64_t ksh, ksr;
    const void *K;
    const void *const *k_layers;   // optional device table: cache of layer head / hpl (then K is unused)
    int hpl;                       // heads per layer of that table
    // workspace
    float *Xn;                // [entries, m, 128]
    float *mag;               // [entries, m]
    float *colpart;           // [entries, MEAN_CHUNKS, 128]
    float *sqpart;            // [entries, MEAN_CHUNKS]
    int32_t *members;         // [entries, m]
    int16_t *part;            // [entries, m]
    int32_t *cand;            // [entries, C]
    int32_t *moff;            // [entries, C + 1]
    int32_t *extra;           // [entries, C]
    int32_t *base;            // [entries, C]
    int32_t *ncand;           // [entries]
    int32_t *counters;        // [4]: candidates this round, clusters split this round
};

__device__ __forceinline__ int head_of(const FitView &v, int e) { return v.list ? v.list[e] : e; }

// First cached row of head h: in the one cache given, or in its layer's cache when a table of layers is given.
template <typename T>
__device__ __forceinline__ const T *keys_of(const FitView &v, int h) {
    if (v.k_layers) return static_cast<const T *>(v.k_layers[h / v.hpl]) + (int64_t)(h % v.hpl) * v.ksh;
    return static_cast<const T *>(v.K) + (int64_t)h * v.ksh;
}

// ---- column sums of the clustered keys (two levels, fixed order) -----------------------------------
template <typename T>
__global__ void __launch_bounds__(128) colsum_kernel(const FitView v) {
    const int e = blockIdx.y, chunk = blockIdx.x, t = threadIdx.x;
    const int h = head_of(v, e);
    const T *Kh = keys_of<T>(v, h);
    const int per = (v.m + MEAN_CHUNKS - 1) / MEAN_CHUNKS;
    const int i0 = chunk * per, i1 = min(i0 + per, v.m);
    float s = 0.f;
    for (int i = i0; i < i1; ++i) s += load_as_float(Kh + (int64_t)(i + 1) * v.ksr + t);
    v.colpart[((int64_t)e * MEAN_CHUNKS + chunk) * HEAD_DIM + t] = s;
}

// mu = mean (or ksum / m of the running sum when recentring), ksum = column sum; stats zeroed.
__global__ void __launch_bounds__(128) mean_kernel(const FitView v, int recentre) {
    const int e = blockIdx.x, t = threadIdx.x;
    const int h = head_of(v, e);
    float s = 0.f;
    for (int c = 0; c < MEAN_CHUNKS; ++c) s += v.colpart[((int64_t)e * MEAN_CHUNKS + c) * HEAD_DIM + t];
    const float old = v.st.ksum[(int64_t)h * HEAD_DIM + t];
    const float mu = v.m > 0 ? (recentre ? old : s) / (float)v.m : 0.f;
    v.st.mu_ref[(int64_t)h * HEAD_DIM + t] = mu;
    v.st.ksum[(int64_t)h * HEAD_DIM + t] = s;
}

// unit directions and lengths about mu; per-chunk sums of squared lengths
template <typename T>
__global__ void __launch_bounds__(256) centre_kernel(const FitView v) {
    __shared__ float s_sq[8];
    const int e = blockIdx.y, chunk = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int h = head_of(v, e);
    const T *Kh = keys_of<T>(v, h);
    const float4 mu = *reinterpret_cast<const float4 *>(v.st.mu_ref + (int64_t)h * HEAD_DIM + lane * 4);
    const int per = (v.m + MEAN_CHUNKS - 1) / MEAN_CHUNKS;
    const int i0 = chunk * per, i1 = min(i0 + per, v.m);
    float sq = 0.f;
    for (int i = i0 + wid; i < i1; i += 8) {
        float4 k = load4(Kh + (int64_t)(i + 1) * v.ksr + lane * 4);
        k.x -= mu.x; k.y -= mu.y; k.z -= mu.z; k.w -= mu.w;
        const float n2 = warp_sum(k.x * k.x + k.y * k.y + k.z * k.z + k.w * k.w);
        const float mg = sqrtf(n2);
        const float inv = 1.0f / fmaxf(mg, 1e-12f);
        *reinterpret_cast<float4 *>(v.Xn + ((int64_t)e * v.m + i) * HEAD_DIM + lane * 4) =
            make_float4(k.x * inv, k.y * inv, k.z * inv, k.w * inv);
        if (lane == 0) v.mag[(int64_t)e * v.m + i] = mg;
        sq += n2;
    }
    if (lane == 0) s_sq[wid] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int w = 0; w < 8; ++w) s += s_sq[w];
        v.sqpart[(int64_t)e * MEAN_CHUNKS + chunk] = s;
    }
}

__global__ void rbar_kernel(const FitView v) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= v.entries) return;
    float s = 0.f;
    for (int c = 0; c < MEAN_CHUNKS; ++c) s += v.sqpart[(int64_t)e * MEAN_CHUNKS + c];
    v.st.rbar[head_of(v, e)] = v.m > 0 ? sqrtf(s / (float)v.m) : 0.f;
}

// starting centroids: the unit directions at the given clustered-key indices
__global__ void __launch_bounds__(128) seed_kernel(const FitView v, const int32_t *init_pos, int C_init) {
    const int e = blockIdx.y, j = blockIdx.x, t = threadIdx.x;
    const int h = head_of(v, e);
    if (j >= C_init) {                                   // slots beyond the fitted ones start empty
        v.st.cent[((int64_t)h * v.st.C + j) * HEAD_DIM + t] = 0.f;
        return;
    }
    if (init_pos) {                                      // null: the caller's centroids stay as they are
        const int i = min(max(init_pos[j], 0), v.m - 1);
        v.st.cent[((int64_t)h * v.st.C + j) * HEAD_DIM + t] = v.Xn[((int64_t)e * v.m + i) * HEAD_DIM + t];
    }
    if (j == 0 && t == 0) v.st.n_c[h] = C_init;
}

// ---- nearest centroid of every clustered key: float32 GEMM tile with a fused arg-max ---------------
// CTA = 128 keys x all n_c centroids in chunks of 64; 256 threads, each 8 keys x 4 centroids: per four steps of k
// a thread issues 12 128-bit shared loads for 128 FFMA, which keeps the shared-memory pipe (the limit of the
// 4 x 4 tiling this replaces: 8 loads per 64 FFMA) behind the FMA pipe.  Both tiles sit in shared memory
// k-contiguous (row stride 132 floats); a thread's centroids are tx, tx+16, tx+32, tx+48 so that a quarter-warp's
// 128-bit loads cover all banks; its keys are rows 8 ty .. 8 ty + 7 (a warp reads two rows at a time: broadcasts).
// Every dot product is a sequential-k chain of float32 FMAs, as before: the arithmetic is unchanged.
constexpr int AS_ROWS = 128, AS_COLS = 64, AS_LD = 132, AS_RPT = 8;
constexpr int AS_SMEM = (AS_ROWS + AS_COLS) * AS_LD * 4;

struct Arg {
    float v;
    int i;
};
__device__ __forceinline__ void arg_take(Arg &a, float v, int i) {
    if (v > a.v || (v == a.v && i < a.i)) { a.v = v; a.i = i; }
}

__global__ void __launch_bounds__(256, 2) assign_kernel(const FitView v) {
    extern __shared__ __align__(16) float smem_f[];
    float *Xs = smem_f, *Cs = smem_f + AS_ROWS * AS_LD;
    const int e = blockIdx.y, tile = blockIdx.x, tid = threadIdx.x;
    const int h = head_of(v, e);
    const int tx = tid & 15, ty = tid >> 4;
    const int n_c = min(max(v.st.n_c[h], 0), v.st.C);
    const int r0 = tile * AS_ROWS;
    const float *X = v.Xn + ((int64_t)e * v.m + r0) * HEAD_DIM;
    const int rows = min(AS_ROWS, v.m - r0);
    for (int i = tid; i < AS_ROWS * 32; i += 256) {
        const int r = i >> 5, k4 = i & 31;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows) x = *reinterpret_cast<const float4 *>(X + (int64_t)r * HEAD_DIM + k4 * 4);
        *reinterpret_cast<float4 *>(Xs + r * AS_LD + k4 * 4) = x;
    }
    Arg best[AS_RPT];
#pragma unroll
    for (int i = 0; i < AS_RPT; ++i) best[i] = Arg{-INFINITY, 0x7fffffff};
    const float *cent = v.st.cent + (int64_t)h * v.st.C * HEAD_DIM;
    for (int c0 = 0; c0 < n_c; c0 += AS_COLS) {
        __syncthreads();
        for (int i = tid; i < AS_COLS * 32; i += 256) {
            const int c = i >> 5, k4 = i & 31;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c0 + c < n_c) x = *reinterpret_cast<const float4 *>(cent + (int64_t)(c0 + c) * HEAD_DIM + k4 * 4);
            *reinterpret_cast<float4 *>(Cs + c * AS_LD + k4 * 4) = x;
        }
        __syncthreads();
        float acc[AS_RPT][4];
#pragma unroll
        for (int i = 0; i < AS_RPT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 2
        for (int k = 0; k < HEAD_DIM; k += 4) {
            float4 xr[AS_RPT], cr[4];
#pragma unroll
            for (int i = 0; i < AS_RPT; ++i) xr[i] = *reinterpret_cast<const float4 *>(Xs + (ty * AS_RPT + i) * AS_LD + k);
#pragma unroll
            for (int j = 0; j < 4; ++j) cr[j] = *reinterpret_cast<const float4 *>(Cs + (tx + 16 * j) * AS_LD + k);
#pragma unroll
            for (int i = 0; i < AS_RPT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(xr[i].x, cr[j].x, acc[i][j]);
                    acc[i][j] = fmaf(xr[i].y, cr[j].y, acc[i][j]);
                    acc[i][j] = fmaf(xr[i].z, cr[j].z, acc[i][j]);
                    acc[i][j] = fmaf(xr[i].w, cr[j].w, acc[i][j]);
                }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + tx + 16 * j;
            if (c < n_c)
#pragma unroll
                for (int i = 0; i < AS_RPT; ++i) arg_take(best[i], acc[i][j], c);
        }
    }
    int16_t *lab = v.st.labels + (int64_t)h * v.st.capacity + 1;
#pragma unroll
    for (int i = 0; i < AS_RPT; ++i) {
        Arg b = best[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
            arg_take(b, ov, oi);
        }
        const int r = ty * AS_RPT + i;
        if (tx == 0 && r < rows) lab[r0 + r] = (int16_t)(b.i == 0x7fffffff ? 0 : b.i);
    }
}

// ---- the same assignment on the tensor cores ---------------------------------------------------------------
// x . c as three TF32 products of a two-term split (x = xh + xl, c = ch + cl with xh = tf32(x), xl = tf32(x - xh)):
// xl ch + xh cl + xh ch, accumulated in float32 by mma.sync m16n8k8.  For unit vectors the split loses at most
// 3 x 2^-22 and the accumulation a few 2^-23 per step - small, but not below the 1e-7 at which Lloyd steps start
// to diverge, so the tensor-core value only DECIDES rows whose two best centroids
// are further apart than ASSIGN_MARGIN (twice a generous bound on |tensor-core value - FFMA chain value|); the few
// rows inside the margin (about one in 10^4) are recomputed by their warp with the sequential float32 chain of
// assign_kernel, centroid by centroid, first maximum wins.  The labels are therefore those of assign_kernel, bit
// for bit (tests compare the two).  CTA = 128 keys x chunks of 64 centroids, warp w owns rows 16 w .. 16 w + 15.
constexpr float ASSIGN_MARGIN = 4.0e-5f;

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32_1688(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// best and second-best value of a row (with the best's index; equal values: the lower index is "better")
struct Top2 {
    float v1, v2;
    int i1;
};
__device__ __forceinline__ void top2_take(Top2 &t, float v, int i) {
    if (v > t.v1 || (v == t.v1 && i < t.i1)) { t.v2 = t.v1; t.v1 = v; t.i1 = i; }
    else if (v > t.v2) t.v2 = v;
}
__device__ __forceinline__ void top2_merge(Top2 &t, float v1, float v2, int i1) {
    top2_take(t, v1, i1);
    if (v2 > t.v2) t.v2 = v2;
}

__global__ void __launch_bounds__(256, 2) assign_tc_kernel(const FitView v) {
    extern __shared__ __align__(16) float smem_f[];
    float *Xs = smem_f, *Cs = smem_f + AS_ROWS * AS_LD;
    const int e = blockIdx.y, tile = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = head_of(v, e);
    const int g = lane >> 2, t = lane & 3;
    const int n_c = min(max(v.st.n_c[h], 0), v.st.C);
    const int r0 = tile * AS_ROWS;
    const float *X = v.Xn + ((int64_t)e * v.m + r0) * HEAD_DIM;
    const int rows = min(AS_ROWS, v.m - r0);
    for (int i = tid; i < AS_ROWS * 32; i += 256) {
        const int r = i >> 5, k4 = i & 31;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows) x = *reinterpret_cast<const float4 *>(X + (int64_t)r * HEAD_DIM + k4 * 4);
        *reinterpret_cast<float4 *>(Xs + r * AS_LD + k4 * 4) = x;
    }
    Top2 best[2] = {{-INFINITY, -INFINITY, 0x7fffffff}, {-INFINITY, -INFINITY, 0x7fffffff}};   // rows 16 w + g, + 8
    const float *cent = v.st.cent + (int64_t)h * v.st.C * HEAD_DIM;
    const float *xa = Xs + (warp * 16 + g) * AS_LD + t, *xb = xa + 8 * AS_LD;
    for (int c0 = 0; c0 < n_c; c0 += AS_COLS) {
        __syncthreads();
        for (int i = tid; i < AS_COLS * 32; i += 256) {
            const int c = i >> 5, k4 = i & 31;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c0 + c < n_c) x = *reinterpret_cast<const float4 *>(cent + (int64_t)(c0 + c) * HEAD_DIM + k4 * 4);
            *reinterpret_cast<float4 *>(Cs + c * AS_LD + k4 * 4) = x;
        }
        __syncthreads();
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll 2
        for (int k0 = 0; k0 < HEAD_DIM; k0 += 8) {
            const float af[4] = {xa[k0], xb[k0], xa[k0 + 4], xb[k0 + 4]};
            uint32_t ah[4], al[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ah[i] = to_tf32(af[i]);
                al[i] = to_tf32(af[i] - __uint_as_float(ah[i]));
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float *cb = Cs + (nt * 8 + g) * AS_LD + k0 + t;
                const float b0 = cb[0], b1 = cb[4];
                const uint32_t bh0 = to_tf32(b0), bh1 = to_tf32(b1);
                const uint32_t bl0 = to_tf32(b0 - __uint_as_float(bh0)), bl1 = to_tf32(b1 - __uint_as_float(bh1));
                mma_tf32_1688(acc[nt], al, bh0, bh1);                        // the small terms first
                mma_tf32_1688(acc[nt], ah, bl0, bl1);
                mma_tf32_1688(acc[nt], ah, bh0, bh1);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = c0 + nt * 8 + 2 * t + j;
                if (c < n_c) {
                    top2_take(best[0], acc[nt][j], c);
                    top2_take(best[1], acc[nt][2 + j], c);
                }
            }
    }
    // the four lanes of a row hold the top two of their own columns: merge them
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int o = 1; o < 4; o <<= 1) {
            const float v1 = __shfl_xor_sync(0xffffffffu, best[r].v1, o);
            const float v2 = __shfl_xor_sync(0xffffffffu, best[r].v2, o);
            const int i1 = __shfl_xor_sync(0xffffffffu, best[r].i1, o);
            top2_merge(best[r], v1, v2, i1);
        }
    int16_t *lab = v.st.labels + (int64_t)h * v.st.capacity + 1;
    unsigned redo = 0u;                                    // rows of this warp (bit = row within its 16) to recompute
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + 8 * r;
        const bool decided = best[r].v1 - best[r].v2 > ASSIGN_MARGIN;     // false for NaN and for a single centroid's -inf rival? (inf - -inf = inf: decided)
        const unsigned bal = __ballot_sync(0xffffffffu, t == 0 && row < rows && !decided);
        if (t == 0 && row < rows && decided) lab[r0 + row] = (int16_t)best[r].i1;
        // ballot bit 4 g marks row g (+ 8 r)
#pragma unroll
        for (int gg = 0; gg < 8; ++gg) redo |= ((bal >> (4 * gg)) & 1u) << (gg + 8 * r);
    }
    while (redo) {                                         // warp-uniform: every lane built the same mask
        const int rr = __ffs(redo) - 1;
        redo &= redo - 1;
        const float *xr = Xs + (warp * 16 + rr) * AS_LD;
        Arg b{-INFINITY, 0x7fffffff};
        for (int c = lane; c < n_c; c += 32) {
            const float *cr = cent + (int64_t)c * HEAD_DIM;
            float a = 0.f;
#pragma unroll 8
            for (int k = 0; k < HEAD_DIM; k += 4) {        // the sequential chain of assign_kernel, same order
                const float4 x = *reinterpret_cast<const float4 *>(xr + k);
                const float4 cc = *reinterpret_cast<const float4 *>(cr + k);
                a = fmaf(x.x, cc.x, a);
                a = fmaf(x.y, cc.y, a);
                a = fmaf(x.z, cc.z, a);
                a = fmaf(x.w, cc.w, a);
            }
            arg_take(b, a, c);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
            arg_take(b, ov, oi);
        }
        if (lane == 0) lab[r0 + warp * 16 + rr] = (int16_t)(b.i == 0x7fffffff ? 0 : b.i);
    }
}

// ---- summaries of every slot from the labels, members taken in position order by one warp --------------
// lloyd != 0: write cent = unit(sum) where the slot has members (a Lloyd update) instead of the summaries.
__global__ void __launch_bounds__(256) accumulate_kernel(const FitView v, int lloyd, int slots) {
    const int e = blockIdx.y, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int h = head_of(v, e);
    if (c >= slots) return;
    const int16_t *lab = v.st.labels + (int64_t)h * v.st.capacity + 1;
    const float *X = v.Xn + (int64_t)e * v.m * HEAD_DIM;
    const float *mg = v.mag + (int64_t)e * v.m;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    float mx = 0.f, mn = INFINITY;
    int cnt = 0;
    const bool live = c < v.st.n_c[h];
    if (live) {
        // A lane tests eight labels per step (one 16-byte load where the labels are aligned; clustered position i
        // is element i + 1 of the head's labels, so the aligned groups start at i = 7, 15, ...), the members are
        // then taken lane by lane and label by label, i.e. in position order, as the sums require.
        const int16_t *lab0 = lab - 1;                       // element p = position p; lab0 is 16-byte aligned
        const int last = v.m + 1;                            // positions [1, last)
        for (int p0 = 0; p0 < last; p0 += 256) {
            const int pb = p0 + lane * 8;
            unsigned mask = 0u;
            if (pb < last) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(lab0 + pb);
                const int16_t *l8 = reinterpret_cast<const int16_t *>(&raw);
#pragma unroll
                for (int j = 0; j < 8; ++j) mask |= (unsigned)(pb + j >= 1 && pb + j < last && l8[j] == c) << j;
            }
            unsigned lanes = __ballot_sync(0xffffffffu, mask != 0u);
            while (lanes) {
                const int l = __ffs(lanes) - 1;
                lanes &= lanes - 1;
                unsigned m8 = __shfl_sync(0xffffffffu, mask, l);
                cnt += __popc(m8);
                while (m8) {
                    const int j = p0 + l * 8 + (__ffs(m8) - 1) - 1;      // clustered-key index of the member
                    m8 &= m8 - 1;
                    const float4 x = *reinterpret_cast<const float4 *>(X + (int64_t)j * HEAD_DIM + lane * 4);
                    s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
                    const float g = mg[j];
                    mx = fmaxf(mx, g);
                    mn = fminf(mn, g);
                }
            }
        }
    }
    const int64_t row = (int64_t)h * v.st.C + c;
    if (lloyd) {
        if (cnt > 0) {
            const float n2 = warp_sum(s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w);
            const float inv = 1.0f / fmaxf(sqrtf(n2), 1e-12f);
            *reinterpret_cast<float4 *>(v.st.cent + row * HEAD_DIM + lane * 4) =
                make_float4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
        }
        return;
    }
    *reinterpret_cast<float4 *>(v.st.sum_dir + row * HEAD_DIM + lane * 4) = s;
    if (lane == 0) {
        v.st.mmax[row] = mx;
        v.st.mmin[row] = mn;
        v.st.count[row] = (float)cnt;
    }
}

// cap of each head after a fit, flags cleared, slots beyond n_c wiped
__global__ void finish_fit_kernel(const FitView v, float cap_keys, float split_factor, int C_init, int fitted,
                                  float var_factor) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= v.entries) return;
    const int h = head_of(v, e);
    if (fitted) {
        float cap = INFINITY;
        if (split_factor > 0.f) cap = cap_keys > 0.f ? cap_keys : split_factor * (float)v.m / (float)C_init;
        v.st.cap[h] = cap;
        v.st.nsplit[h] = 0;
        v.st.status[h] = 0;
        if (v.st.vthr) {
            // spread threshold: var_factor x the mean over the fitted clusters in use of 1 - |sum_dir|^2 / count^2
            float thr = INFINITY;
            if (var_factor > 0.f) {
                float sum = 0.f, used = 0.f;
                for (int c = 0; c < C_init; ++c) {
                    const float cn = v.st.count[(int64_t)h * v.st.C + c];
                    if (cn > 0.f) {
                        const float *sd = v.st.sum_dir + ((int64_t)h * v.st.C + c) * HEAD_DIM;
                        float n2 = 0.f;
                        for (int i = 0; i < HEAD_DIM; ++i) n2 = fmaf(sd[i], sd[i], n2);
                        sum += fmaxf(1.0f - n2 / (cn * cn), 0.f);
                        used += 1.f;
                    }
                }
                thr = var_factor * sum / fmaxf(used, 1.f);
            }
            v.st.vthr[h] = thr;
        }
    }
    v.st.flags[h] = 0;
    v.st.end[h] = v.end;
}

// 8-bit copies of the direction sums and centroids of every slot
__global__ void __launch_bounds__(256) refresh8_kernel(const FitView v) {
    const int e = blockIdx.y, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int h = head_of(v, e);
    if (c >= v.st.C) return;
    const int64_t row = ((int64_t)h * v.st.C + c) * HEAD_DIM + lane * 4;
    const float4 a = *reinterpret_cast<const float4 *>(v.st.sum_dir + row);
    const float4 b = *reinterpret_cast<const float4 *>(v.st.cent + row);
    const float ia = 1.0f / fmaxf(sqrtf(warp_sum(a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w)), 1e-12f);
    const float ib = 1.0f / fmaxf(sqrtf(warp_sum(b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w)), 1e-12f);
    char4 qa, qb;
    qa.x = quant8(a.x * ia); qa.y = quant8(a.y * ia); qa.z = quant8(a.z * ia); qa.w = quant8(a.w * ia);
    qb.x = quant8(b.x * ib); qb.y = quant8(b.y * ib); qb.z = quant8(b.z * ib); qb.w = quant8(b.w * ib);
    *reinterpret_cast<char4 *>(v.st.dir8 + row) = qa;
    *reinterpret_cast<char4 *>(v.st.cent8 + row) = qb;
}

// ---- division of the clusters over the cap, one round ----------------------------------------------
// counters: [0] candidates over all entries, [1] clusters split, [2] most candidates in one entry,
//           [3] most parts asked for one cluster
__global__ void __launch_bounds__(256) find_over_kernel(const FitView v, int kway, float split_factor, float capk) {
    __shared__ int ired[40];
    const int e = blockIdx.x, tid = threadIdx.x;
    const int h = head_of(v, e);
    const int C = v.st.C;
    const int n_c = min(max(v.st.n_c[h], 0), C);
    const float cap = fmaxf(v.st.cap[h], capk * (float)v.m);
    const float *count = v.st.count + (int64_t)h * C;
    const int per = (C + 255) / 256;
    const int c0 = min(tid * per, n_c), c1 = min(c0 + per, n_c);
    int mine = 0;
    for (int c = c0; c < c1; ++c) mine += (count[c] > cap && count[c] >= 2.0f);
    int total;
    int off = block_excl_scan(mine, ired, total);
    int32_t *cand = v.cand + (int64_t)e * C;
    for (int c = c0; c < c1; ++c)
        if (count[c] > cap && count[c] >= 2.0f) cand[off++] = c;
    __syncthreads();
    if (tid == 0) {
        int32_t *moff = v.moff + (int64_t)e * (C + 1);
        int run = 0, kmax = 2;
        for (int j = 0; j < total; ++j) {
            moff[j] = run;
            const float cn = count[cand[j]];
            run += (int)cn;
            if (kway) kmax = max(kmax, (int)ceilf(cn * split_factor / cap));
        }
        moff[total] = run;
        v.ncand[e] = total;
        if (total) {
            atomicAdd(v.counters + 0, total);
            atomicMax(v.counters + 2, total);
            atomicMax(v.counters + 3, kmax);
        }
    }
}

// member lists of the candidates, in position order: one warp per candidate
__global__ void __launch_bounds__(256) members_kernel(const FitView v) {
    const int e = blockIdx.y, lane = threadIdx.x & 31;
    const int j = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (j >= v.ncand[e]) return;
    const int h = head_of(v, e);
    const int c = v.cand[(int64_t)e * v.st.C + j];
    const int16_t *lab = v.st.labels + (int64_t)h * v.st.capacity + 1;
    int32_t *mem = v.members + (int64_t)e * v.m + v.moff[(int64_t)e * (v.st.C + 1) + j];
    int run = 0;
    for (int i0 = 0; i0 < v.m; i0 += 32) {
        const int i = i0 + lane;
        const bool hit = i < v.m && lab[i] == c;
        const unsigned b = __ballot_sync(0xffffffffu, hit);
        if (hit) mem[run + __popc(b & ((1u << lane) - 1u))] = i;
        run += __popc(b);
    }
}

constexpr int PART_CH = 32;                 // members staged per chunk in partition_kernel (a multiple of 8)

struct PartSmem {
    float *cents;   // [k][128]
    float *sums;    // [k][128]
    int *sizes;     // [k]
    int *newid;     // [k]
};

// Partition the members of one candidate cluster: k-way cosine k-means from evenly spaced members
// (kway) or the two-way split with the median-cut fallback.  One CTA per candidate.
__global__ void __launch_bounds__(256) partition_kernel(const FitView v, int kway, float split_factor, int iters,
                                                        int kcap, float *projbuf, float capk) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float fred[32];
    __shared__ int ired[40];
    const int e = blockIdx.y, j = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (j >= v.ncand[e]) return;
    const int h = head_of(v, e);
    const int C = v.st.C;
    const int c = v.cand[(int64_t)e * C + j];
    const int o0 = v.moff[(int64_t)e * (C + 1) + j];
    const int cnt = v.moff[(int64_t)e * (C + 1) + j + 1] - o0;
    const int32_t *mem = v.members + (int64_t)e * v.m + o0;
    int16_t *prt = v.part + (int64_t)e * v.m + o0;
    float *proj = projbuf + (int64_t)e * v.m + o0;
    const float *X = v.Xn + (int64_t)e * v.m * HEAD_DIM;
    (void)c;
    if (kway) {
        const float cap = fmaxf(v.st.cap[h], capk * (float)v.m);
        int k = (int)ceilf((float)cnt * split_factor / cap);
        k = min(max(k, 2), kcap);
        float *stage = reinterpret_cast<float *>(smem_raw);          // [PART_CH][128]: a chunk of members' directions
        float *cents = stage + PART_CH * HEAD_DIM;
        float *sums = cents + (size_t)kcap * HEAD_DIM;
        int *sizes = reinterpret_cast<int *>(sums + (size_t)kcap * HEAD_DIM);
        int *newid = sizes + kcap;
        for (int i = tid; i < k * HEAD_DIM; i += 256) {
            const int jj = i >> 7, t = i & 127;
            const int seed = min((int)(((int64_t)jj * cnt) / k), cnt - 1);
            cents[i] = X[(int64_t)mem[seed] * HEAD_DIM + t];
        }
        __syncthreads();
        for (int it = 0; it <= iters; ++it) {
            const bool last = it == iters;
            if (!last) {
                for (int i = tid; i < k * HEAD_DIM; i += 256) sums[i] = 0.f;
                for (int i = tid; i < k; i += 256) sizes[i] = 0;
            }
            // The members go by in chunks of PART_CH: a warp fetches its rows of the chunk (all requested at once),
            // assigns them, and leaves them in shared memory, from where thread t adds component t of the chunk's
            // members to their parts' sums in member order - the order of the additions is that of a single pass over
            // all members, so the sums are the same bits, without one dependent global load per member.
            for (int c0 = 0; c0 < cnt; c0 += PART_CH) {
                float4 x[PART_CH / 8];
#pragma unroll
                for (int q = 0; q < PART_CH / 8; ++q) {
                    const int r = c0 + wid + 8 * q;
                    x[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (r < cnt) x[q] = *reinterpret_cast<const float4 *>(X + (int64_t)mem[r] * HEAD_DIM + lane * 4);
                }
#pragma unroll
                for (int q = 0; q < PART_CH / 8; ++q) {
                    const int r = c0 + wid + 8 * q;
                    if (r >= cnt) continue;                      // warp-uniform
                    float bv = -INFINITY;
                    int bi = 0;
                    for (int jj = 0; jj < k; ++jj) {
                        const float4 cc = *reinterpret_cast<const float4 *>(cents + jj * HEAD_DIM + lane * 4);
                        const float dot = warp_sum(x[q].x * cc.x + x[q].y * cc.y + x[q].z * cc.z + x[q].w * cc.w);
                        if (dot > bv) { bv = dot; bi = jj; }
                    }
                    if (lane == 0) prt[r] = (int16_t)bi;
                    if (!last) *reinterpret_cast<float4 *>(stage + (wid + 8 * q) * HEAD_DIM + lane * 4) = x[q];
                }
                if (last) continue;
                __syncthreads();
                const int rows = min(PART_CH, cnt - c0);
                if (tid < HEAD_DIM) {
                    for (int r = 0; r < rows; ++r) sums[prt[c0 + r] * HEAD_DIM + tid] += stage[r * HEAD_DIM + tid];
                } else if (tid == HEAD_DIM) {
                    for (int r = 0; r < rows; ++r) sizes[prt[c0 + r]] += 1;
                }
                __syncthreads();
            }
            __syncthreads();
            if (last) break;
            for (int jj = wid; jj < k; jj += 8) {
                const float4 s = *reinterpret_cast<const float4 *>(sums + jj * HEAD_DIM + lane * 4);
                const float n2 = warp_sum(s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w);
                if (sizes[jj] > 0) {
                    const float inv = 1.0f / fmaxf(sqrtf(n2), 1e-12f);
                    *reinterpret_cast<float4 *>(cents + jj * HEAD_DIM + lane * 4) =
                        make_float4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
                }
            }
            __syncthreads();
        }
        // number the non-empty parts 0, 1, ... in part order
        for (int i = tid; i < k; i += 256) sizes[i] = 0;
        __syncthreads();
        if (tid == 0) {
            for (int r = 0; r < cnt; ++r) sizes[prt[r]] += 1;
            int run = 0;
            for (int jj = 0; jj < k; ++jj) { newid[jj] = run; run += sizes[jj] > 0; }
            v.extra[(int64_t)e * C + j] = run - 1;
        }
        __syncthreads();
        for (int r = tid; r < cnt; r += 256) prt[r] = (int16_t)newid[prt[r]];
        return;
    }
    // ---- two-way split -------------------------------------------------------------------------
    float *stage = reinterpret_cast<float *>(smem_raw);              // [PART_CH][128]
    float *sa = stage + PART_CH * HEAD_DIM, *sb = sa + HEAD_DIM, *sdiff = sb + HEAD_DIM;
    if (tid < HEAD_DIM) sa[tid] = X[(int64_t)mem[0] * HEAD_DIM + tid];
    __syncthreads();
    {
        const float4 a4 = *reinterpret_cast<const float4 *>(sa + lane * 4);
        for (int r = wid; r < cnt; r += 8) {
            const float4 x = *reinterpret_cast<const float4 *>(X + (int64_t)mem[r] * HEAD_DIM + lane * 4);
            const float s = warp_sum(x.x * a4.x + x.y * a4.y + x.z * a4.z + x.w * a4.w);
            if (lane == 0) proj[r] = s;
        }
    }
    __syncthreads();
    if (wid == 0) {
        float bv = INFINITY;
        int bi = 0x7fffffff;
        for (int r = lane; r < cnt; r += 32) {
            const float s = proj[r];
            if (s < bv || (s == bv && r < bi)) { bv = s; bi = r; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov < bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) ired[0] = bi;
    }
    __syncthreads();
    if ((unsigned)ired[0] >= (unsigned)cnt) {
        // every similarity is NaN (a member with an Inf or NaN component): no farthest member, no split
        if (tid == 0) {
            v.extra[(int64_t)e * C + j] = 0;
            if (v.st.status) atomicOr(v.st.status + h, SKV_ST_BAD_INDEX);
        }
        return;
    }
    if (tid < HEAD_DIM) sb[tid] = X[(int64_t)mem[ired[0]] * HEAD_DIM + tid];
    __syncthreads();
    for (int it = 0; it <= 4; ++it) {
        if (it == 4 && tid < HEAD_DIM) sdiff[tid] = sb[tid] - sa[tid];
        if (it == 4) __syncthreads();
        float s0 = 0.f, s1 = 0.f;
        int n1 = 0;
        {
            // members in chunks, as in the k-way path: fetched by the warp that assigns them, then added up per
            // component in member order from shared memory
            const float4 a4 = *reinterpret_cast<const float4 *>(sa + lane * 4);
            const float4 b4 = *reinterpret_cast<const float4 *>(sb + lane * 4);
            const float4 d4 = *reinterpret_cast<const float4 *>(sdiff + lane * 4);
            for (int c0 = 0; c0 < cnt; c0 += PART_CH) {
                float4 x[PART_CH / 8];
#pragma unroll
                for (int q = 0; q < PART_CH / 8; ++q) {
                    const int r = c0 + wid + 8 * q;
                    x[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (r < cnt) x[q] = *reinterpret_cast<const float4 *>(X + (int64_t)mem[r] * HEAD_DIM + lane * 4);
                }
#pragma unroll
                for (int q = 0; q < PART_CH / 8; ++q) {
                    const int r = c0 + wid + 8 * q;
                    if (r >= cnt) continue;                      // warp-uniform
                    const float da = warp_sum(x[q].x * a4.x + x[q].y * a4.y + x[q].z * a4.z + x[q].w * a4.w);
                    const float db = warp_sum(x[q].x * b4.x + x[q].y * b4.y + x[q].z * b4.z + x[q].w * b4.w);
                    if (it == 4) {
                        const float pj = warp_sum(x[q].x * d4.x + x[q].y * d4.y + x[q].z * d4.z + x[q].w * d4.w);
                        if (lane == 0) proj[r] = pj;
                    }
                    if (lane == 0) prt[r] = db > da;
                    if (it < 4) *reinterpret_cast<float4 *>(stage + (wid + 8 * q) * HEAD_DIM + lane * 4) = x[q];
                }
                if (it == 4) continue;
                __syncthreads();
                const int rows = min(PART_CH, cnt - c0);
                if (tid < HEAD_DIM) {
                    for (int r = 0; r < rows; ++r) {
                        const float u = stage[r * HEAD_DIM + tid];
                        if (prt[c0 + r]) { s1 += u; ++n1; } else s0 += u;
                    }
                }
                __syncthreads();
            }
        }
        __syncthreads();
        if (it == 4) break;
        const float q0 = block_sum(tid < HEAD_DIM ? s0 * s0 : 0.f, fred);
        const float q1 = block_sum(tid < HEAD_DIM ? s1 * s1 : 0.f, fred);
        if (tid == 0) ired[1] = n1;
        __syncthreads();
        n1 = ired[1];
        if (tid < HEAD_DIM) {
            if (cnt - n1 > 0) sa[tid] = s0 / fmaxf(sqrtf(q0), 1e-12f);
            if (n1 > 0) sb[tid] = s1 / fmaxf(sqrtf(q1), 1e-12f);
        }
        __syncthreads();
    }
    int n1 = 0;
    for (int r = tid; r < cnt; r += 256) n1 += prt[r];
    n1 = warp_sum_int(n1);
    if (lane == 0) ired[2 + wid] = n1;
    __syncthreads();
    n1 = 0;
    for (int w = 0; w < 8; ++w) n1 += ired[2 + w];
    __syncthreads();
    if ((float)n1 < 0.25f * (float)cnt || (float)n1 > 0.75f * (float)cnt) {
        const int halfm = cnt / 2;
        for (int r = tid; r < cnt; r += 256) {
            const float pj = proj[r];
            int rank = 0;
            for (int i = 0; i < cnt; ++i) {
                const float pi = proj[i];
                rank += (pi < pj) || (pi == pj && i < r);
            }
            prt[r] = rank >= halfm;
        }
        n1 = cnt - halfm;
    }
    if (tid == 0) v.extra[(int64_t)e * C + j] = (n1 > 0 && n1 < cnt) ? 1 : 0;
}

// spare slots in candidate order; a cluster whose run of new slots would pass C waits for a later round
__global__ void slots_kernel(const FitView v) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= v.entries) return;
    const int h = head_of(v, e);
    const int C = v.st.C, nc = v.ncand[e];
    int run = v.st.n_c[h], taken = 0, kept = 0;
    for (int j = 0; j < nc; ++j) {
        const int ex = v.extra[(int64_t)e * C + j];
        const bool keep = ex > 0 && run + ex <= C;
        v.base[(int64_t)e * C + j] = keep ? run : -1;
        if (keep) { taken += ex; ++kept; }
        run += ex;
    }
    if (kept) {
        v.st.n_c[h] += taken;
        v.st.nsplit[h] += taken;
        atomicAdd(v.counters + 1, kept);
    } else if (nc > 0 && v.st.status) {
        atomicOr(v.st.status + h, SKV_ST_NO_SLOT);
    }
}

// rewrite the summaries, centroids and labels of a split cluster: one warp per part, members in order
__global__ void __launch_bounds__(256) apply_kernel(const FitView v) {
    const int e = blockIdx.y, j = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (j >= v.ncand[e]) return;
    const int C = v.st.C;
    const int base = v.base[(int64_t)e * C + j];
    if (base < 0) return;
    const int h = head_of(v, e);
    const int c = v.cand[(int64_t)e * C + j];
    const int parts = v.extra[(int64_t)e * C + j] + 1;
    const int o0 = v.moff[(int64_t)e * (C + 1) + j];
    const int cnt = v.moff[(int64_t)e * (C + 1) + j + 1] - o0;
    const int32_t *mem = v.members + (int64_t)e * v.m + o0;
    const int16_t *prt = v.part + (int64_t)e * v.m + o0;
    const float *X = v.Xn + (int64_t)e * v.m * HEAD_DIM;
    const float *mg = v.mag + (int64_t)e * v.m;
    int16_t *lab = v.st.labels + (int64_t)h * v.st.capacity + 1;
    for (int pn = wid; pn < parts; pn += 8) {
        const int slot = pn == 0 ? c : base + pn - 1;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        float mx = 0.f, mn = INFINITY;
        int n = 0;
        for (int r0 = 0; r0 < cnt; r0 += 32) {
            const int r = r0 + lane;
            const bool hit = r < cnt && prt[r] == pn;
            if (hit) lab[mem[r]] = (int16_t)slot;
            unsigned b = __ballot_sync(0xffffffffu, hit);
            n += __popc(b);
            while (b) {
                const int rr = r0 + __ffs(b) - 1;
                b &= b - 1;
                const int i = mem[rr];
                const float4 x = *reinterpret_cast<const float4 *>(X + (int64_t)i * HEAD_DIM + lane * 4);
                s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
                const float g = mg[i];
                mx = fmaxf(mx, g);
                mn = fminf(mn, g);
            }
        }
        const int64_t row = (int64_t)h * C + slot;
        *reinterpret_cast<float4 *>(v.st.sum_dir + row * HEAD_DIM + lane * 4) = s;
        const float inv = 1.0f / fmaxf(sqrtf(warp_sum(s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w)), 1e-12f);
        *reinterpret_cast<float4 *>(v.st.cent + row * HEAD_DIM + lane * 4) =
            make_float4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
        if (lane == 0) {
            v.st.mmax[row] = mx;
            v.st.mmin[row] = mn;
            v.st.count[row] = (float)n;
        }
    }
}

// ---- host orchestration ---------------------------------------------------------------------------
static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

static int64_t carve(FitView &v, char *base, int entries, int m, int C) {
    int64_t o = 0;
    auto take = [&](int64_t bytes) { char *p = base ? base + o : nullptr; o += align256(bytes); return p; };
    v.Xn = reinterpret_cast<float *>(take((int64_t)entries * m * HEAD_DIM * 4));
    v.mag = reinterpret_cast<float *>(take((int64_t)entries * m * 4));
    v.colpart = reinterpret_cast<float *>(take((int64_t)entries * MEAN_CHUNKS * HEAD_DIM * 4));
    v.sqpart = reinterpret_cast<float *>(take((int64_t)entries * MEAN_CHUNKS * 4));
    v.members = reinterpret_cast<int32_t *>(take((int64_t)entries * m * 4));
    v.part = reinterpret_cast<int16_t *>(take((int64_t)entries * m * 2));
    v.cand = reinterpret_cast<int32_t *>(take((int64_t)entries * C * 4));
    v.moff = reinterpret_cast<int32_t *>(take((int64_t)entries * (C + 1) * 4));
    v.extra = reinterpret_cast<int32_t *>(take((int64_t)entries * C * 4));
    v.base = reinterpret_cast<int32_t *>(take((int64_t)entries * C * 4));
    v.ncand = reinterpret_cast<int32_t *>(take((int64_t)entries * 4));
    v.counters = reinterpret_cast<int32_t *>(take(64));
    return o;
}

static int64_t fit_bytes(int entries, int m, int C) {
    FitView v;
    int64_t o = carve(v, nullptr, entries, m, C);
    return o + align256((int64_t)entries * m * 4);      // + projections of the two-way split
}

static int check_state(const skv_state *st) {
    if (!st) return SKV_E_NULL;
    if (!st->sum_dir || !st->cent || !st->mmax || !st->mmin || !st->count || !st->n_c || !st->cap || !st->rbar ||
        !st->ksum || !st->mu_ref || !st->flags || !st->status || !st->nsplit || !st->end || !st->need || !st->labels)
        return SKV_E_NULL;
    if (st->d != HEAD_DIM) return SKV_E_DIM;
    if (st->C < 16 || (st->C & (st->C - 1)) || st->C > 16384) return SKV_E_DIM;
    if (st->summary_bits != 8 && st->summary_bits != 32) return SKV_E_RANGE;
    if (st->summary_bits == 8 && (!st->dir8 || !st->cent8)) return SKV_E_NULL;
    if (st->heads <= 0 || st->capacity <= 0) return SKV_E_RANGE;
    if (st->capacity % 8 || !aligned16(st->labels) || !aligned16(st->sum_dir) || !aligned16(st->cent) ||
        !aligned16(st->mu_ref))
        return SKV_E_ALIGN;
    return SKV_OK;
}

template <typename T>
static int centre_and_assign(FitView &v, int recentre, cudaStream_t s) {
    colsum_kernel<T><<<dim3(MEAN_CHUNKS, v.entries), 128, 0, s>>>(v);
    mean_kernel<<<v.entries, 128, 0, s>>>(v, recentre);
    centre_kernel<T><<<dim3(MEAN_CHUNKS, v.entries), 256, 0, s>>>(v);
    rbar_kernel<<<(v.entries + 127) / 128, 128, 0, s>>>(v);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

// process-wide switch (skv_fit_tensor_cores); SKV_FIT_TC=1 in the environment starts with the tensor-core kernel.
// Off by default: measured on B200 the two are equally fast (the float32 kernel reaches 42 TFLOP/s) and give the same
// labels, so the simpler one runs.
static bool g_fit_tensor_cores = [] { const char *e = getenv("SKV_FIT_TC"); return e && e[0] == '1'; }();

static int launch_assign(const FitView &v, cudaStream_t s) {
    static bool configured[64] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (!configured[dev]) {
        SKV_CUDA_OK(cudaFuncSetAttribute(assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AS_SMEM));
        SKV_CUDA_OK(cudaFuncSetAttribute(assign_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AS_SMEM));
        configured[dev] = true;
    }
    const dim3 grid((v.m + AS_ROWS - 1) / AS_ROWS, v.entries);
    if (!g_fit_tensor_cores) assign_kernel<<<grid, 256, AS_SMEM, s>>>(v);
    else assign_tc_kernel<<<grid, 256, AS_SMEM, s>>>(v);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

static int split_rounds(FitView &v, float *projbuf, float split_factor, int iters, float capk, bool kway,
                        cudaStream_t s) {
    for (int round = 0; round < 256; ++round) {
        int32_t host[4] = {0, 0, 0, 0};
        SKV_CUDA_OK(cudaMemsetAsync(v.counters, 0, 16, s));
        find_over_kernel<<<v.entries, 256, 0, s>>>(v, kway ? 1 : 0, split_factor, capk);
        SKV_CUDA_OK(cudaMemcpyAsync(host, v.counters, 16, cudaMemcpyDeviceToHost, s));
        SKV_CUDA_OK(cudaStreamSynchronize(s));
        if (host[0] == 0) break;
        const int maxc = host[2];
        const int kcap = kway ? (host[3] < 2 ? 2 : (host[3] > KWAY_MAX ? KWAY_MAX : host[3])) : 2;
        members_kernel<<<dim3((maxc + 7) / 8, v.entries), 256, 0, s>>>(v);
        const size_t smem = (size_t)PART_CH * HEAD_DIM * 4 + (kway ? (size_t)kcap * (2 * HEAD_DIM * 4 + 8) + 64 : 3 * HEAD_DIM * 4);
        if (smem > 48 * 1024)
            SKV_CUDA_OK(cudaFuncSetAttribute(partition_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        partition_kernel<<<dim3(maxc, v.entries), 256, smem, s>>>(v, kway ? 1 : 0, split_factor, iters, kcap, projbuf,
                                                                  capk);
        slots_kernel<<<(v.entries + 127) / 128, 128, 0, s>>>(v);
        apply_kernel<<<dim3(maxc, v.entries), 256, 0, s>>>(v);
        SKV_CUDA_OK(cudaMemcpyAsync(host, v.counters, 16, cudaMemcpyDeviceToHost, s));
        SKV_CUDA_OK(cudaStreamSynchronize(s));
        if (host[1] == 0 && !kway) break;
        kway = false;
    }
    return SKV_OK;
}

}  // namespace skv

using namespace skv;

extern "C" void skv_fit_tensor_cores(int on) { skv::g_fit_tensor_cores = on != 0; }

extern "C" int64_t skv_fit_workspace_bytes(int heads, int m, int C, int d) {
    if (heads <= 0 || m < 0 || C < 16 || d != HEAD_DIM) return SKV_E_RANGE;
    return fit_bytes(heads, m < 1 ? 1 : m, C);
}

extern "C" int skv_fit(const skv_state *st, const void *K, int dtype, int64_t k_head_stride, int64_t k_row_stride,
                       int n, int window, int C_init, int iters, const int32_t *init_pos, float cap_keys,
                       float split_factor, float capk, float var_factor, const int32_t *head_list, int n_list,
                       const void *const *k_layers, int heads_per_layer, void *workspace, int64_t workspace_bytes,
                       void *stream) {
    int rc = check_state(st);
    if (rc) return rc;
    if ((!K && !k_layers) || !workspace) return SKV_E_NULL;
    if (k_layers && (heads_per_layer < 1 || st->heads % heads_per_layer)) return SKV_E_RANGE;
    if (!init_pos) iters = 0;                            // given centroids are kept: no Lloyd step
    if (dtype != SKV_BF16 && dtype != SKV_F32) return SKV_E_DTYPE;
    if (n < 0 || n > st->capacity || window < 0 || iters < 0 || C_init < 1 || C_init > st->C || cap_keys < 0.f ||
        split_factor < 0.f || capk < 0.f || var_factor < 0.f)
        return SKV_E_RANGE;
    if (head_list && (n_list < 1 || n_list > st->heads)) return SKV_E_RANGE;
    const int esz = dtype == SKV_BF16 ? 2 : 4;
    if ((K && !aligned16(K)) || !aligned16(workspace) || (k_row_stride * esz) % 16 || (k_head_stride * esz) % 16 ||
        k_row_stride < HEAD_DIM)
        return SKV_E_ALIGN;
    const int end = n - window > 1 ? n - window : 1;
    const int m = end - 1;
    if (m < 1) return SKV_E_RANGE;                      // nothing to cluster yet
    const int entries = head_list ? n_list : st->heads;
    if (workspace_bytes < fit_bytes(entries, m, st->C)) return SKV_E_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    FitView v;
    v.st = *st; v.list = head_list; v.entries = entries; v.end = end; v.m = m;
    v.ksh = k_head_stride; v.ksr = k_row_stride; v.K = K; v.k_layers = k_layers; v.hpl = heads_per_layer;
    const int64_t used = carve(v, static_cast<char *>(workspace), entries, m, st->C);
    float *projbuf = reinterpret_cast<float *>(static_cast<char *>(workspace) + used);
    rc = dtype == SKV_BF16 ? centre_and_assign<__nv_bfloat16>(v, 0, s) : centre_and_assign<float>(v, 0, s);
    if (rc) return rc;
    seed_kernel<<<dim3(st->C, entries), 128, 0, s>>>(v, init_pos, C_init);
    for (int it = 0; it < iters; ++it) {
        if ((rc = launch_assign(v, s))) return rc;
        accumulate_kernel<<<dim3((C_init + 7) / 8, entries), 256, 0, s>>>(v, 1, C_init);
    }
    if ((rc = launch_assign(v, s))) return rc;
    accumulate_kernel<<<dim3((st->C + 7) / 8, entries), 256, 0, s>>>(v, 0, st->C);
    finish_fit_kernel<<<(entries + 127) / 128, 128, 0, s>>>(v, cap_keys, split_factor, C_init, 1, var_factor);
    SKV_CUDA_OK(cudaGetLastError());
    if (split_factor > 0.f && (rc = split_rounds(v, projbuf, split_factor, iters, capk, true, s))) return rc;
    if (st->summary_bits == 8) refresh8_kernel<<<dim3((st->C + 7) / 8, entries), 256, 0, s>>>(v);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

extern "C" int skv_rebin(const skv_state *st, const int32_t *head_list, int n_list, int end, const void *K, int dtype,
                         int64_t k_head_stride, int64_t k_row_stride, float split_factor, int iters, float capk,
                         void *workspace, int64_t workspace_bytes, void *stream) {
    int rc = check_state(st);
    if (rc) return rc;
    if (!K || !workspace || !head_list) return SKV_E_NULL;
    if (dtype != SKV_BF16 && dtype != SKV_F32) return SKV_E_DTYPE;
    if (n_list < 1 || n_list > st->heads || end < 2 || end > st->capacity || split_factor < 0.f || iters < 0 ||
        capk < 0.f)
        return SKV_E_RANGE;
    const int esz = dtype == SKV_BF16 ? 2 : 4;
    if (!aligned16(K) || !aligned16(workspace) || (k_row_stride * esz) % 16 || (k_head_stride * esz) % 16 ||
        k_row_stride < HEAD_DIM)
        return SKV_E_ALIGN;
    const int m = end - 1;
    if (workspace_bytes < fit_bytes(n_list, m, st->C)) return SKV_E_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    FitView v;
    v.st = *st; v.list = head_list; v.entries = n_list; v.end = end; v.m = m;
    v.ksh = k_head_stride; v.ksr = k_row_stride; v.K = K; v.k_layers = nullptr; v.hpl = 1;
    const int64_t used = carve(v, static_cast<char *>(workspace), n_list, m, st->C);
    float *projbuf = reinterpret_cast<float *>(static_cast<char *>(workspace) + used);
    rc = dtype == SKV_BF16 ? centre_and_assign<__nv_bfloat16>(v, 1, s) : centre_and_assign<float>(v, 1, s);
    if (rc) return rc;
    if ((rc = launch_assign(v, s))) return rc;
    accumulate_kernel<<<dim3((st->C + 7) / 8, n_list), 256, 0, s>>>(v, 0, st->C);
    finish_fit_kernel<<<(n_list + 127) / 128, 128, 0, s>>>(v, 0.f, 0.f, 1, 0, 0.f);
    SKV_CUDA_OK(cudaGetLastError());
    // Rebinning about a new mean can leave clusters over their cap, larger than the insert's in-kernel split
    // stages; they are divided here, two ways at a time, as the reference's PyTorch path divides a cluster
    // over the cap when it next receives a key (ssa/attn/sphere_gpu.py:247-249, :307-338).
    if (split_factor > 0.f && (rc = split_rounds(v, projbuf, split_factor, iters, capk, false, s))) return rc;
    if (st->summary_bits == 8) refresh8_kernel<<<dim3((st->C + 7) / 8, n_list), 256, 0, s>>>(v);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}
