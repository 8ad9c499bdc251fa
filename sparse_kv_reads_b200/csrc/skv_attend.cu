// Indexed-gather split-K flash-decode over a list of cached rows, with the log-sum-exp merge done
// by the last CTA of each head (no second launch).
//
// Work layout: grid (splits, heads).  A head's row list is cut into tiles of 16 rows; the tiles are
// dealt in contiguous runs to the head's (splits x WARPS) warps.  Every warp runs its own
// cp.async pipeline (STAGES tiles of 16 K rows + 16 V rows, 256 B each for bf16) into a private
// XOR-swizzled shared-memory ring, so the main loop has no block-wide barrier.  For bf16 the
// scores S = Q K^T and the update O += P V are mma.sync m16n8k16 tiles with the (<= 16) query
// heads of the group on the M side, fp32 accumulation and a per-warp online softmax in base 2.
// The work is HBM-bound (G flop per byte); the tensor-core tiles only keep the issue slots free
// for the gathers.  float32 caches take a plain CUDA-core path with float32 arithmetic throughout.
#include <type_traits>

#include "skv_attend_core.cuh"
#include "skv_common.cuh"

namespace skv {

constexpr int PART_LD = 132;               // floats per partial row: 128 sums, max, sum, 2 unused

struct AttendParams {
    const void *q, *K, *V;
    const int32_t *idx, *cnt, *n_dev;
    void *out;
    float *part;       // [heads, splits, G, 132]: 128 sums, max (base-2 units), sum of weights, 2 unused
    int32_t *ticket;   // [heads]
    int32_t *status;   // [heads] or null
    int heads, G, n_group;
    int64_t ksh, ksr, vsh, vsr, idx_stride;
    int rows_limit, splits;
    float scale_log2;  // softmax scale * log2(e)
    // rows taken straight from the labels (no list): position p < n is read iff its label's bit is set
    const int16_t *labels;     // [heads, lab_stride]
    const uint32_t *selbits;   // [heads, sel_words], bit C = always-read rows
    int32_t *cnt_out;          // [heads] rows read, accumulated (zeroed by the selection kernel)
    int64_t lab_stride;
    int sel_words, C;
    unsigned long long *probe;  // optional [CTAs][8] phase time stamps (ns), for tuning
    // fractional cluster weights (rows of sampled clusters): a row of label l enters the softmax with weight wl[l],
    // i.e. log2(wl[l]) is added to its score; rows of weight 0 are not read.  Needs labels, lab_stride and C.
    const float *wl;           // [heads, C + 1] or null
};

static unsigned long long *g_attend_probe = nullptr;

// Phase time stamps exist only in builds with -DSKV_ATTEND_PROBE: the tests on a pointer inside the tile loop
// cost the label-driven kernel 3.5 % at 256 heads (176 us against 170 us), so the library proper has none.
__device__ __forceinline__ void stamp(const AttendParams &p, int slot) {
#ifdef SKV_ATTEND_PROBE
    if (p.probe && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.probe[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 8 + slot] = t;
    }
#else
    (void)p; (void)slot;
#endif
}

// Which tiles a warp owns: contiguous runs, identical arithmetic in every CTA of the head.
struct Share {
    int count, s_eff, t0, t1;
};
__device__ __forceinline__ Share my_share(const AttendParams &p, int head, int split, int warp, int warps) {
    Share s;
    s.count = p.idx ? p.cnt[head] : positions_of(p.n_dev, p.n_group, head);
    if (s.count < 0) s.count = 0;
    const int tiles = (s.count + TILE_ROWS - 1) / TILE_ROWS;
    s.s_eff = min(p.splits, max(1, (tiles + warps - 1) / warps));
    const int slots = s.s_eff * warps;
    const int per = (tiles + slots - 1) / slots;
    const int ws = split * warps + warp;
    s.t0 = min(ws * per, tiles);
    s.t1 = min(s.t0 + per, tiles);
    return s;
}

// Position of list entry `row` of this head, or -1 when past the end / out of range.
__device__ __forceinline__ int fetch_pos(const AttendParams &p, int head, int row, int count) {
    if (row >= count) return -1;
    if (!p.idx) return row;
    int pos = __ldg(p.idx + (int64_t)head * p.idx_stride + row);
    if (pos < 0 || pos >= p.rows_limit) {
        if (p.status) atomicOr(p.status + head, SKV_ST_BAD_INDEX);
        return -1;
    }
    return pos;
}

// Combine the partial (max, sum, acc) sets that the warps of this CTA left in shared memory
// (red[set][g][132]: 128 acc, then max, sum), publish the CTA's partial, and let the last CTA of the
// head merge all partials into `out`.  blockDim.x must be 128 (one thread per output column).
template <typename T>
__device__ __forceinline__ void finish_head(const AttendParams &p, const float *red, int sets, int head, int split,
                                            int s_eff, int *sh_flag, float *stage, int stage_rows) {
    const int G = p.G, tid = threadIdx.x;
    T *out = static_cast<T *>(p.out);
    float *pa = p.part + ((int64_t)head * p.splits + split) * G * PART_LD;
#pragma unroll 1
    for (int g = 0; g < G; ++g) {
        float M = NEG_BIG;
        for (int w = 0; w < sets; ++w) M = fmaxf(M, red[(w * G + g) * 132 + 128]);
        float dn = 0.f, nm = 0.f;
        for (int w = 0; w < sets; ++w) {
            const float *r = red + (w * G + g) * 132;
            float f = fast_exp2(r[128] - M);
            dn += f * r[129];
            nm += f * r[tid];
        }
        if (s_eff == 1) {
            store_out(out + ((int64_t)head * G + g) * HEAD_DIM + tid, dn > 0.f ? nm / dn : 0.f);
        } else {
            __stcg(pa + g * PART_LD + tid, nm);
            if (tid == 0) __stcg(reinterpret_cast<float2 *>(pa + g * PART_LD + HEAD_DIM), make_float2(M, dn));
        }
    }
    if (s_eff == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int t = atomicAdd(p.ticket + head, 1);
        *sh_flag = (t == s_eff - 1);
    }
    __syncthreads();
    stamp(p, 5);
    if (!*sh_flag) return;
    __threadfence();
    // Merge of the head's partials by this (last) CTA.  The partial rows are copied into the shared memory
    // the CTA no longer needs with asynchronous 16-byte copies, all requested before any is used: one round
    // trip to L2 where they fit (stage_rows rows), chunks of one query head's splits with a running maximum
    // otherwise.  Up to four query heads are then folded at once, each by 4 / (their number) warps that share
    // its rows; a lane owns four columns.
    float *stg = stage;
    __shared__ __align__(16) float s_sum[4][PART_LD];
    const int lane = tid & 31, wid = tid >> 5;
    const float *src = p.part + (int64_t)head * p.splits * G * PART_LD;
    const int gc = max(1, min(G, stage_rows / s_eff));        // query heads staged together
    const int cs = gc > 1 ? s_eff : min(s_eff, stage_rows);   // splits per chunk
    for (int g0 = 0; g0 < G; g0 += gc) {
        const int ng = min(gc, G - g0);
        float M = NEG_BIG, dn = 0.f;                           // carried over chunks only when ng == 1
        float4 nm = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < s_eff; s0 += cs) {
            const int ns = min(cs, s_eff - s0);
            if (ng == G) {                                     // every row of the head: one contiguous block
                const int chunks = ns * G * (PART_LD / 4);
                const float *blk = src + (int64_t)s0 * G * PART_LD;
                for (int c = tid; c < chunks; c += 128) cp_async16(stg + c * 4, blk + c * 4, 16);
            } else {                                           // rows of query heads [g0, g0 + ng) only
                for (int gi = 0; gi < ng; ++gi)
                    for (int i = wid; i < ns; i += 4) {
                        const float *row = src + ((int64_t)(s0 + i) * G + g0 + gi) * PART_LD;
                        float *dst = stg + (i * ng + gi) * PART_LD;
                        cp_async16(dst + lane * 4, row + lane * 4, 16);
                        if (lane == 0) cp_async16(dst + HEAD_DIM, row + HEAD_DIM, 16);
                    }
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
            stamp(p, 7);
            // staged row of (split i, query head gi): stg + (i * ng + gi) * PART_LD
            const bool last_chunk = s0 + cs >= s_eff;
            for (int gb = 0; gb < ng; gb += 4) {
                const int nq = min(4, ng - gb), wpg = 4 / nq;
                const int gi = gb + wid / wpg, sub = wid % wpg;
                if (wid < nq * wpg) {
                    if (ng > 1) { M = NEG_BIG; dn = 0.f; nm = make_float4(0.f, 0.f, 0.f, 0.f); }
                    const float *rows = stg + gi * PART_LD;
                    const int ld = ng * PART_LD;
                    float mb = NEG_BIG;
                    for (int i = lane; i < ns; i += 32) mb = fmaxf(mb, rows[i * ld + HEAD_DIM]);
                    mb = fmaxf(M, warp_max(mb));
                    const float al = fast_exp2(M - mb);
                    M = mb;
                    dn *= al; nm.x *= al; nm.y *= al; nm.z *= al; nm.w *= al;
#pragma unroll 4
                    for (int i = sub; i < ns; i += wpg) {
                        const float2 ml = *reinterpret_cast<const float2 *>(rows + i * ld + HEAD_DIM);
                        const float4 a = *reinterpret_cast<const float4 *>(rows + i * ld + lane * 4);
                        const float f = fast_exp2(ml.x - M);
                        dn = fmaf(f, ml.y, dn);
                        nm.x = fmaf(f, a.x, nm.x); nm.y = fmaf(f, a.y, nm.y);
                        nm.z = fmaf(f, a.z, nm.z); nm.w = fmaf(f, a.w, nm.w);
                    }
                    *reinterpret_cast<float4 *>(&s_sum[wid][lane * 4]) = nm;
                    if (lane == 0) s_sum[wid][HEAD_DIM] = dn;
                }
                __syncthreads();
                if (ng > 1 || last_chunk)
                    for (int qi = 0; qi < nq; ++qi) {
                        float num = 0.f, den = 0.f;
                        for (int w = 0; w < wpg; ++w) {
                            num += s_sum[qi * wpg + w][tid];
                            den += s_sum[qi * wpg + w][HEAD_DIM];
                        }
                        store_out(out + ((int64_t)head * G + g0 + gb + qi) * HEAD_DIM + tid, den > 0.f ? num / den : 0.f);
                    }
                __syncthreads();
            }
        }
    }
    if (tid == 0) p.ticket[head] = 0;     // ready for the next call on this stream
    stamp(p, 6);
}

// ---------------------------------------------------------------------------------------------
// bf16 tensor-core path over a list of rows
// ---------------------------------------------------------------------------------------------
template <int WARPS, int STAGES, bool HI>
__global__ void __launch_bounds__(WARPS * 32, 3) attend_mma_kernel(const AttendParams p) {
    static_assert(WARPS == 4, "finish_head expects 128 threads");
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint32_t s_vmask[WARPS][STAGES];
    __shared__ int s_flag;
    const int warp = threadIdx.x >> 5;
    const int head = blockIdx.y, split = blockIdx.x;
    const int G = p.G;
    const Share sh = my_share(p, head, split, warp, WARPS);
    if (split >= sh.s_eff) return;
    typename std::conditional<HI, WarpAttend<STAGES, true>, WarpAttendT<STAGES>>::type wa;
    wa.init(static_cast<const __nv_bfloat16 *>(p.q) + (int64_t)head * G * HEAD_DIM, G, smem + warp * (STAGES * 8192),
            s_vmask[warp], static_cast<const char *>(p.K) + (int64_t)head * p.ksh * 2,
            static_cast<const char *>(p.V) + (int64_t)head * p.vsh * 2, p.ksr * 2, p.vsr * 2, p.scale_log2);
    wa.run(sh.t0, sh.t1, [&](int row) { return fetch_pos(p, head, row, sh.count); });
    __syncthreads();                       // every warp is done with its ring: reuse it
    float *red = reinterpret_cast<float *>(smem);
    wa.store_partial(red, warp, G);
    __syncthreads();
    finish_head<__nv_bfloat16>(p, red, WARPS, head, split, sh.s_eff, &s_flag, red, WARPS * STAGES * 8192 / (PART_LD * 4));
}

// ---------------------------------------------------------------------------------------------
// bf16 tensor-core path straight from the labels: every CTA owns a contiguous range of positions,
// lists the selected ones of 2,048 positions at a time in shared memory (ascending), and attends over
// them.  No global row list is written or read; cnt_out receives the number of rows read.
// ---------------------------------------------------------------------------------------------
// LPT = labels a thread tests per pass (8 or 16): short ranges (many CTAs per head) use 8 so that every thread
// of the CTA takes part in listing; a pass covers LAB_SUB = 128 x LPT positions.
template <int WARPS, int STAGES, bool HI, int LPT>
__global__ void __launch_bounds__(WARPS * 32, 3) attend_labels_kernel(const AttendParams p) {
    static_assert(WARPS == 4, "finish_head expects 128 threads");
    static_assert(LPT == 8 || LPT == 16, "a thread's labels are one or two 16-byte loads");
    constexpr int LAB_SUB = WARPS * 32 * LPT, LV = LPT / 8;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint32_t s_vmask[WARPS][STAGES];
    __shared__ int s_flag;
    __shared__ int s_scan[40];
    __shared__ uint16_t s_rows[LAB_SUB];   // offsets from the pass start, ascending
    const int warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int head = blockIdx.y, split = blockIdx.x;
    const int G = p.G, C = p.C;
    const int n = min(max(positions_of(p.n_dev, p.n_group, head), 0), (int)p.lab_stride);
    // position ranges: multiples of 16 so that a thread's 16 labels are two aligned 16-byte loads
    const int chunk = max(16, (((n + p.splits - 1) / p.splits + 15) >> 4) << 4);
    const int s_eff = max(1, (n + chunk - 1) / chunk);
    if (split >= s_eff) return;
    const int p0 = split * chunk, p1 = min(p0 + chunk, n);
    uint32_t *s_bits = reinterpret_cast<uint32_t *>(smem + WARPS * STAGES * 8192);
    const int16_t *lab = p.labels + (int64_t)head * p.lab_stride;
    stamp(p, 0);
    // the first pass's labels are requested before anything else so that their latency overlaps the
    // loads of the selection bits and of the query
    uint4 raw[LV];
#pragma unroll
    for (int v = 0; v < LV; ++v) {
        raw[v] = make_uint4(0u, 0u, 0u, 0u);
        if (p0 + tid * LPT + v * 8 < p1) raw[v] = __ldg(reinterpret_cast<const uint4 *>(lab + p0 + tid * LPT + v * 8));
    }
    pdl_wait();                            // selection bits and query come from the kernels before this one
    pdl_trigger();
    for (int i = tid; i < p.sel_words; i += WARPS * 32) s_bits[i] = p.selbits[(int64_t)head * p.sel_words + i];
    typename std::conditional<HI, WarpAttend<STAGES, true>, WarpAttendT<STAGES>>::type wa;
    wa.init(static_cast<const __nv_bfloat16 *>(p.q) + (int64_t)head * G * HEAD_DIM, G, smem + warp * (STAGES * 8192),
            s_vmask[warp], static_cast<const char *>(p.K) + (int64_t)head * p.ksh * 2,
            static_cast<const char *>(p.V) + (int64_t)head * p.vsh * 2, p.ksr * 2, p.vsr * 2, p.scale_log2);
    int read_rows = 0;
    bool bad = false;
    __syncthreads();
    stamp(p, 1);
    for (int sub0 = p0; sub0 < p1; sub0 += LAB_SUB) {
        const int base = sub0 + tid * LPT;
        uint32_t take = 0;
        if (base < p1) {
            const int16_t *l16 = reinterpret_cast<const int16_t *>(raw);
#pragma unroll
            for (int i = 0; i < LPT; ++i) {
                const unsigned l = (unsigned)(int)l16[i];
                if (base + i < p1) {
                    if (l <= (unsigned)C) take |= ((s_bits[l >> 5] >> (l & 31)) & 1u) << i;
                    else bad = true;
                }
            }
        }
#pragma unroll
        for (int v = 0; v < LV; ++v)                     // next pass's labels, in flight during this pass's attention
            if (base + LAB_SUB + v * 8 < p1)
                raw[v] = __ldg(reinterpret_cast<const uint4 *>(lab + base + LAB_SUB + v * 8));
        int total;
        int off = block_excl_scan(__popc(take), s_scan, total);
        while (take) {
            const int i = __ffs(take) - 1;
            take &= take - 1;
            s_rows[off++] = (uint16_t)(tid * LPT + i);
        }
        __syncthreads();
        stamp(p, 2);
        read_rows += total;
        const int tiles = (total + TILE_ROWS - 1) / TILE_ROWS;
        const int per = (tiles + WARPS - 1) / WARPS;
        const int t0 = min(warp * per, tiles), t1 = min(t0 + per, tiles);
        wa.run(t0, t1, [&](int row) { return row < total ? sub0 + (int)s_rows[row] : -1; });
        __syncthreads();                   // the list is rewritten by the next pass
        stamp(p, 3);
    }
    if (tid == 0 && p.cnt_out) atomicAdd(p.cnt_out + head, read_rows);
    if (bad && p.status) atomicOr(p.status + head, SKV_ST_BAD_INDEX);
    float *red = reinterpret_cast<float *>(smem);
    wa.store_partial(red, warp, G);
    __syncthreads();
    stamp(p, 4);
    finish_head<__nv_bfloat16>(p, red, WARPS, head, split, s_eff, &s_flag, red, WARPS * STAGES * 8192 / (PART_LD * 4));
}

// ---------------------------------------------------------------------------------------------
// CUDA-core path (float32 caches; also a second implementation of the bf16 case for cross-checks)
// Half a warp per row: lane (sub) owns 8 consecutive components.
// ---------------------------------------------------------------------------------------------
template <typename T, int GP>
__global__ void __launch_bounds__(128) attend_simple_kernel(const AttendParams p) {
    constexpr int WARPS = 4;
    __shared__ __align__(16) float red[2 * WARPS * GP * 132];
    __shared__ int s_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y, split = blockIdx.x;
    const int G = p.G;
    const Share sh = my_share(p, head, split, warp, WARPS);
    if (split >= sh.s_eff) return;
    const int sub = lane & 15, half = lane >> 4;
    const unsigned hmask = half ? 0xffff0000u : 0x0000ffffu;    // the two halves of a warp diverge on skipped rows
    const T *q = static_cast<const T *>(p.q) + (int64_t)head * G * HEAD_DIM;
    const T *Kb = static_cast<const T *>(p.K) + (int64_t)head * p.ksh;
    const T *Vb = static_cast<const T *>(p.V) + (int64_t)head * p.vsh;

    float qr[GP][8], acc[GP][8], m[GP], l[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        m[g] = NEG_BIG;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
        if (g < G) load8(q + g * HEAD_DIM + sub * 8, qr[g]);
        else
#pragma unroll
            for (int i = 0; i < 8; ++i) qr[g][i] = 0.f;
    }
    for (int t = sh.t0; t < sh.t1; ++t) {
        int mypos = fetch_pos(p, head, t * TILE_ROWS + sub, sh.count);
        float mylw = 0.f;
        if (p.wl && mypos >= 0) {                           // the row's weight, by its label
            const unsigned l = (unsigned)(int)p.labels[(int64_t)head * p.lab_stride + mypos];
            const float wgt = l <= (unsigned)p.C ? p.wl[(int64_t)head * (p.C + 1) + l] : 0.f;
            if (wgt > 0.f) mylw = log2f(wgt);
            else mypos = -1;
        }
#pragma unroll 2
        for (int i = 0; i < 8; ++i) {
            const int pos = __shfl_sync(0xffffffffu, mypos, half + 2 * i);
            const float lw = __shfl_sync(0xffffffffu, mylw, half + 2 * i);
            if (pos < 0) continue;                          // uniform within the half warp
            float kv[8], vv[8];
            load8(Kb + (int64_t)pos * p.ksr + sub * 8, kv);
            load8(Vb + (int64_t)pos * p.vsr + sub * 8, vv);
#pragma unroll
            for (int g = 0; g < GP; ++g) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) s = fmaf(qr[g][e], kv[e], s);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(hmask, s, o, 16);
                const float z = fmaf(s, p.scale_log2, lw);
                const float mn = fmaxf(m[g], z);
                const float al = exp2f(m[g] - mn), pr = exp2f(z - mn);
                m[g] = mn;
                l[g] = l[g] * al + pr;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pr, vv[e], acc[g][e] * al);
            }
        }
    }
    const int set = warp * 2 + half;
    for (int g = 0; g < G; ++g) {
        float *r = red + (set * G + g) * 132;
#pragma unroll
        for (int e = 0; e < 8; ++e) r[sub * 8 + e] = acc[g][e];
        if (sub == 0) { r[128] = m[g]; r[129] = l[g]; }
    }
    __syncthreads();
    finish_head<T>(p, red, 2 * WARPS, head, split, sh.s_eff, &s_flag, red, 2 * WARPS * GP);
}

// natural-log merge of caller-provided partials
__global__ void merge_kernel(const float *m, const float *l, const float *a, float *out, int S, int G) {
    const int head = blockIdx.x, tid = threadIdx.x;
    for (int g = 0; g < G; ++g) {
        float M = NEG_BIG;
        for (int s = 0; s < S; ++s) M = fmaxf(M, m[((int64_t)head * S + s) * G + g]);
        float dn = 0.f, nm = 0.f;
        for (int s = 0; s < S; ++s) {
            const int64_t o = ((int64_t)head * S + s) * G + g;
            const float f = expf(m[o] - M);
            dn += f * l[o];
            nm += f * a[o * HEAD_DIM + tid];
        }
        out[((int64_t)head * G + g) * HEAD_DIM + tid] = nm / dn;
    }
}

constexpr int MMA_WARPS = 4, MMA_STAGES = 2;   // 64 KB of rings per CTA: three CTAs (12 warps) per SM
constexpr int MMA_SMEM = MMA_WARPS * MMA_STAGES * 8192;

template <bool HI>
static int launch_mma(const AttendParams &p, dim3 grid, cudaStream_t st) {
    auto kern = attend_mma_kernel<MMA_WARPS, MMA_STAGES, HI>;
    static bool configured[64] = {};       // the attribute is kept per device
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (!configured[dev]) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM));
        configured[dev] = true;
    }
    kern<<<grid, MMA_WARPS * 32, MMA_SMEM, st>>>(p);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

template <bool HI, int STAGES, int LPT>
static int launch_labels_as(const AttendParams &p, dim3 grid, cudaStream_t st) {
    auto kern = attend_labels_kernel<MMA_WARPS, STAGES, HI, LPT>;
    static size_t configured[64] = {};
    const size_t smem = (size_t)MMA_WARPS * STAGES * 8192 + (size_t)p.sel_words * 4;
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (configured[dev] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = smem;
    }
    SKV_CUDA_OK(launch_pdl(kern, grid, dim3(MMA_WARPS * 32), smem, st, p));
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

// Short position ranges (many CTAs per head) list 8 labels per thread, long ones 16.
template <bool HI>
static int launch_labels(const AttendParams &p, dim3 grid, cudaStream_t st) {
    const bool lpt8 = (p.lab_stride + p.splits - 1) / p.splits <= MMA_WARPS * 32 * 8;
    return lpt8 ? launch_labels_as<HI, MMA_STAGES, 8>(p, grid, st) : launch_labels_as<HI, MMA_STAGES, 16>(p, grid, st);
}

template <typename T>
static int launch_simple(const AttendParams &p, dim3 grid, cudaStream_t st) {
    if (p.G <= 1) attend_simple_kernel<T, 1><<<grid, 128, 0, st>>>(p);
    else if (p.G <= 2) attend_simple_kernel<T, 2><<<grid, 128, 0, st>>>(p);
    else if (p.G <= 4) attend_simple_kernel<T, 4><<<grid, 128, 0, st>>>(p);
    else attend_simple_kernel<T, 8><<<grid, 128, 0, st>>>(p);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

}  // namespace skv

using namespace skv;

extern "C" void skv_debug_attend_probe(void *dev_ptr) { skv::g_attend_probe = static_cast<unsigned long long *>(dev_ptr); }

extern "C" int skv_attend_splits(int heads) {
    if (heads <= 0) return SKV_E_RANGE;
    // One wave of CTAs, never more: a CTA's cost has a large fixed part (prologue, partial merge), so a
    // second, nearly empty wave costs more than it spreads.  Three CTAs fit an SM; with few heads the
    // partials to merge are what costs, so two per SM are enough there.  Measured on B200 at 32k / 20 %:
    // 8 heads 37 splits, 64 heads 6, 256 heads 1 were the fastest of the values tried.
    const int sms = device_sm_count();
    int s = 3 * sms / heads;
    if (s > 8) s = 2 * sms / heads;
    // (256 heads at 32k / 20 %: three CTAs per head even out SMs holding one and two CTAs, 168 us against 172 us, but
    // cost 7 to 20 % at 8k, where a CTA has little to do: one CTA per head stays)
    return s < 1 ? 1 : s;
}

extern "C" int64_t skv_attend_workspace_bytes(int heads, int G, int d, int splits) {
    if (heads <= 0 || G <= 0 || d != HEAD_DIM || splits <= 0) return SKV_E_RANGE;
    int64_t part = (int64_t)heads * splits * G * PART_LD * 4;
    int64_t tk = (((int64_t)heads * 4) + 255) / 256 * 256;
    return part + tk;
}

// Host-side checks of skv_attend's arguments (no CUDA call): shared with skv_attend_static so that both
// reject the same calls with the same codes before anything is enqueued.
static int attend_check(const void *q, const void *K, const void *V, const int32_t *idx, const int32_t *cnt,
                        const int32_t *n_dev, int n_group, const void *out, const void *workspace, int heads, int G, int d,
                        int dtype,
                        int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride, int64_t v_row_stride,
                        int rows_limit, int splits) {
    const int base = dtype & 0xff;
    const bool force_simple = (dtype >> 8) & 1;
    if (!q || !K || !V || !out || !workspace) return SKV_E_NULL;
    if (idx ? !cnt : !n_dev) return SKV_E_NULL;
    if (d != HEAD_DIM) return SKV_E_DIM;
    if (base != SKV_BF16 && base != SKV_F32) return SKV_E_DTYPE;
    if (heads <= 0 || heads > 65535 || splits <= 0 || splits > 65535 || rows_limit < 0 || n_group < 0) return SKV_E_RANGE;
    if (G < 1 || G > 16 || ((base == SKV_F32 || force_simple) && G > 8)) return SKV_E_DIM;
    const int esz = base == SKV_BF16 ? 2 : 4;
    if (!aligned16(q) || !aligned16(K) || !aligned16(V) || !aligned16(out) || !aligned16(workspace)) return SKV_E_ALIGN;
    if ((k_row_stride * esz) % 16 || (v_row_stride * esz) % 16 || (k_head_stride * esz) % 16 ||
        (v_head_stride * esz) % 16 || k_row_stride < d || v_row_stride < d)
        return SKV_E_ALIGN;
    return SKV_OK;
}

// mode bit 0 of `dtype >> 8` forces the CUDA-core path for bf16 (cross-checks)
extern "C" int skv_attend(const void *q, const void *K, const void *V, const int32_t *idx, const int32_t *cnt,
                          const int32_t *n_dev, int n_group, void *out, void *workspace, int32_t *status, int heads,
                          int G, int d, int dtype, int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride,
                          int64_t v_row_stride, int64_t idx_stride, int rows_limit, int splits, float scale,
                          void *stream) {
    const int base = dtype & 0xff;
    const bool force_simple = (dtype >> 8) & 1;
    const int rc = attend_check(q, K, V, idx, cnt, n_dev, n_group, out, workspace, heads, G, d, dtype, k_head_stride,
                                k_row_stride, v_head_stride, v_row_stride, rows_limit, splits);
    if (rc) return rc;
    AttendParams p;
    p.q = q; p.K = K; p.V = V; p.idx = idx; p.cnt = cnt; p.n_dev = n_dev; p.out = out; p.status = status;
    p.part = static_cast<float *>(workspace);
    p.ticket = reinterpret_cast<int32_t *>(p.part + (int64_t)heads * splits * G * PART_LD);
    p.heads = heads; p.G = G; p.n_group = n_group;
    p.ksh = k_head_stride; p.ksr = k_row_stride; p.vsh = v_head_stride; p.vsr = v_row_stride;
    p.idx_stride = idx_stride; p.rows_limit = rows_limit; p.splits = splits;
    p.scale_log2 = scale * LOG2E;
    p.labels = nullptr; p.selbits = nullptr; p.cnt_out = nullptr; p.lab_stride = 0; p.sel_words = 0; p.C = 0;
    p.probe = nullptr; p.wl = nullptr;
    dim3 grid(splits, heads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (base == SKV_F32) return launch_simple<float>(p, grid, st);
    if (force_simple) return launch_simple<__nv_bfloat16>(p, grid, st);
    return G > 8 ? launch_mma<true>(p, grid, st) : launch_mma<false>(p, grid, st);
}

extern "C" int skv_attend_labels(const void *q, const void *K, const void *V, const int16_t *labels,
                                 int64_t label_stride, const uint32_t *selbits, int C, const int32_t *n_dev, int n_group,
                                 void *out,
                                 void *workspace, int32_t *cnt, int32_t *status, int heads, int G, int d, int dtype,
                                 int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride,
                                 int64_t v_row_stride, int splits, float scale, void *stream) {
    if (!q || !K || !V || !labels || !selbits || !n_dev || !out || !workspace) return SKV_E_NULL;
    if (d != HEAD_DIM) return SKV_E_DIM;
    if (dtype != SKV_BF16) return SKV_E_DTYPE;                   // float32 caches take the list path
    if (G < 1 || G > 16 || C < 16 || (C & (C - 1)) || C > 16384) return SKV_E_DIM;
    if (heads <= 0 || heads > 65535 || splits <= 0 || splits > 65535 || label_stride <= 0 || n_group < 0) return SKV_E_RANGE;
    if (!aligned16(q) || !aligned16(K) || !aligned16(V) || !aligned16(out) || !aligned16(workspace) ||
        !aligned16(labels) || label_stride % 8)
        return SKV_E_ALIGN;
    if ((k_row_stride * 2) % 16 || (v_row_stride * 2) % 16 || (k_head_stride * 2) % 16 || (v_head_stride * 2) % 16 ||
        k_row_stride < d || v_row_stride < d)
        return SKV_E_ALIGN;
    AttendParams p;
    p.q = q; p.K = K; p.V = V; p.idx = nullptr; p.cnt = nullptr; p.n_dev = n_dev; p.out = out; p.status = status;
    p.part = static_cast<float *>(workspace);
    p.ticket = reinterpret_cast<int32_t *>(p.part + (int64_t)heads * splits * G * PART_LD);
    p.heads = heads; p.G = G; p.n_group = n_group;
    p.ksh = k_head_stride; p.ksr = k_row_stride; p.vsh = v_head_stride; p.vsr = v_row_stride;
    p.idx_stride = 0; p.rows_limit = 0; p.splits = splits;
    p.scale_log2 = scale * LOG2E;
    p.probe = g_attend_probe; p.wl = nullptr;
    p.labels = labels; p.selbits = selbits; p.cnt_out = cnt; p.lab_stride = label_stride;
    p.sel_words = C / 32 + 1; p.C = C;
    dim3 grid(splits, heads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return G > 8 ? launch_labels<true>(p, grid, st) : launch_labels<false>(p, grid, st);
}

extern "C" int skv_attend_weighted(const void *q, const void *K, const void *V, const int16_t *labels,
                                   int64_t label_stride, const float *w, int C, const int32_t *n_dev, int n_group,
                                   void *out,
                                   void *workspace, int32_t *status, int heads, int G, int d, int dtype,
                                   int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride,
                                   int64_t v_row_stride, int splits, float scale, void *stream) {
    const int rc = attend_check(q, K, V, nullptr, nullptr, n_dev, n_group, out, workspace, heads, G, d, dtype, k_head_stride,
                                k_row_stride, v_head_stride, v_row_stride, 0, splits);
    if (rc) return rc;
    if (!labels || !w) return SKV_E_NULL;
    if (G > 8 || C < 16 || (C & (C - 1)) || C > 16384) return SKV_E_DIM;
    if (label_stride <= 0) return SKV_E_RANGE;
    AttendParams p;
    p.q = q; p.K = K; p.V = V; p.idx = nullptr; p.cnt = nullptr; p.n_dev = n_dev; p.out = out; p.status = status;
    p.part = static_cast<float *>(workspace);
    p.ticket = reinterpret_cast<int32_t *>(p.part + (int64_t)heads * splits * G * PART_LD);
    p.heads = heads; p.G = G; p.n_group = n_group;
    p.ksh = k_head_stride; p.ksr = k_row_stride; p.vsh = v_head_stride; p.vsr = v_row_stride;
    p.idx_stride = 0; p.rows_limit = 0; p.splits = splits;
    p.scale_log2 = scale * LOG2E;
    p.labels = labels; p.selbits = nullptr; p.cnt_out = nullptr; p.lab_stride = label_stride; p.sel_words = 0; p.C = C;
    p.probe = nullptr; p.wl = w;
    dim3 grid(splits, heads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return (dtype & 0xff) == SKV_F32 ? launch_simple<float>(p, grid, st) : launch_simple<__nv_bfloat16>(p, grid, st);
}

extern "C" int skv_merge(const float *m, const float *l, const float *a, float *out, int heads, int S, int G, int d,
                         void *stream) {
    if (!m || !l || !a || !out) return SKV_E_NULL;
    if (d != HEAD_DIM) return SKV_E_DIM;
    if (heads <= 0 || S <= 0 || G <= 0) return SKV_E_RANGE;
    merge_kernel<<<heads, HEAD_DIM, 0, static_cast<cudaStream_t>(stream)>>>(m, l, a, out, S, G);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

// ---------------------------------------------------------------------------------------------
// Attention with library-owned scratch: for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
// The split partials and ticket words of this variant live in a fixed array that is part of the
// library image, so every GPU that loads the library carries these 8 MiB until the process exits.
static __device__ __align__(256) unsigned char g_attend_scratch[SKV_STATIC_SCRATCH_BYTES];

// Device address of g_attend_scratch on the current device.  In host code the array's name is only a
// stand-in for the symbol, not something a kernel can dereference; the address has to be asked for,
// once per device, with that device current.
static int static_scratch(void **out) {
    static void *cached[64] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (!cached[dev]) {
        void *p = nullptr;
        SKV_CUDA_OK(cudaGetSymbolAddress(&p, g_attend_scratch));
        cached[dev] = p;
    }
    *out = cached[dev];
    return SKV_OK;
}

extern "C" int skv_attend_static(const void *q, const void *K, const void *V, const int32_t *idx, const int32_t *cnt,
                                 const int32_t *n_dev, int n_group, void *out, int32_t *status, int heads, int G, int d,
                                 int dtype,
                                 int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride,
                                 int64_t v_row_stride, int64_t idx_stride, int rows_limit, int splits, float scale,
                                 void *stream) {
    // the same argument checks as skv_attend, ahead of every CUDA call (any aligned non-null pointer stands in for
    // the workspace, which is the library's own array here)
    int rc = attend_check(q, K, V, idx, cnt, n_dev, n_group, out, q, heads, G, d, dtype, k_head_stride, k_row_stride,
                          v_head_stride, v_row_stride, rows_limit, splits);
    if (rc) return rc;
    const int64_t need = skv_attend_workspace_bytes(heads, G, d, splits);
    if (need < 0) return (int)need;
    if (need > (int64_t)SKV_STATIC_SCRATCH_BYTES) return SKV_E_TOO_LARGE;
    void *scratch = nullptr;
    rc = static_scratch(&scratch);
    if (rc) return rc;
    // Earlier calls with other shapes left their partials here.  Only the ticket words have to start at
    // zero (partials are always written before they are read); they sit at the end of the layout.
    unsigned char *tickets = static_cast<unsigned char *>(scratch) + (int64_t)heads * splits * G * PART_LD * 4;
    SKV_CUDA_OK(cudaMemsetAsync(tickets, 0, (size_t)heads * 4, static_cast<cudaStream_t>(stream)));
    return skv_attend(q, K, V, idx, cnt, n_dev, n_group, out, scratch, status, heads, G, d, dtype, k_head_stride, k_row_stride,
                      v_head_stride, v_row_stride, idx_stride, rows_limit, splits, scale, stream);
}
