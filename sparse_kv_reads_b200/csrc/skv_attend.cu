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
#include "skv_common.cuh"

namespace skv {

struct AttendParams {
    const void *q, *K, *V;
    const int32_t *idx, *cnt, *n_dev;
    void *out;
    float *part_acc;   // [heads, splits, G, 128]
    float *part_ml;    // [heads, splits, G, 2]   (max in base-2 units, sum)
    int32_t *ticket;   // [heads]
    int32_t *status;   // [heads] or null
    int heads, G;
    int64_t ksh, ksr, vsh, vsr, idx_stride;
    int rows_limit, splits;
    float scale_log2;  // softmax scale * log2(e)
};

constexpr int TILE_ROWS = 16;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem) {
    unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem) {
    unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

// Which tiles a warp owns: contiguous runs, identical arithmetic in every CTA of the head.
struct Share {
    int count, s_eff, t0, t1;
};
__device__ __forceinline__ Share my_share(const AttendParams &p, int head, int split, int warp, int warps) {
    Share s;
    s.count = p.idx ? p.cnt[head] : p.n_dev[0];
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
                                            int s_eff, int *sh_flag) {
    const int G = p.G, tid = threadIdx.x;
    T *out = static_cast<T *>(p.out);
    float *pa = p.part_acc + ((int64_t)head * p.splits + split) * G * HEAD_DIM;
    float *pm = p.part_ml + ((int64_t)head * p.splits + split) * G * 2;
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
            __stcg(pa + g * HEAD_DIM + tid, nm);
            if (tid == 0) {
                __stcg(pm + 2 * g, M);
                __stcg(pm + 2 * g + 1, dn);
            }
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
    if (!*sh_flag) return;
    __threadfence();
    const float *qa = p.part_acc + (int64_t)head * p.splits * G * HEAD_DIM;
    const float *qm = p.part_ml + (int64_t)head * p.splits * G * 2;
#pragma unroll 1
    for (int g = 0; g < G; ++g) {
        float M = NEG_BIG;
        for (int s = 0; s < s_eff; ++s) M = fmaxf(M, __ldcg(qm + (s * G + g) * 2));
        float dn = 0.f, nm = 0.f;
#pragma unroll 4
        for (int s = 0; s < s_eff; ++s) {
            float f = fast_exp2(__ldcg(qm + (s * G + g) * 2) - M);
            dn += f * __ldcg(qm + (s * G + g) * 2 + 1);
            nm += f * __ldcg(qa + (s * G + g) * HEAD_DIM + tid);
        }
        store_out(out + ((int64_t)head * G + g) * HEAD_DIM + tid, dn > 0.f ? nm / dn : 0.f);
    }
    if (tid == 0) p.ticket[head] = 0;     // ready for the next call on this stream
}

// ---------------------------------------------------------------------------------------------
// bf16 tensor-core path
// ---------------------------------------------------------------------------------------------
template <int WARPS, int STAGES, bool HI>
__global__ void __launch_bounds__(WARPS * 32) attend_mma_kernel(const AttendParams p) {
    static_assert(WARPS == 4, "finish_head expects 128 threads");
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint32_t s_vmask[WARPS][STAGES];
    __shared__ int s_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y, split = blockIdx.x;
    const int G = p.G;
    const Share sh = my_share(p, head, split, warp, WARPS);
    if (split >= sh.s_eff) return;

    unsigned char *ring = smem + warp * (STAGES * 8192);
    const __nv_bfloat16 *q = static_cast<const __nv_bfloat16 *>(p.q) + (int64_t)head * G * HEAD_DIM;
    const char *Kb = static_cast<const char *>(p.K) + (int64_t)head * p.ksh * 2;
    const char *Vb = static_cast<const char *>(p.V) + (int64_t)head * p.vsh * 2;
    const int64_t krow = p.ksr * 2, vrow = p.vsr * 2;

    // query fragments (A operand), rows = query heads of the group, zero beyond G
    uint32_t qa[8][4];
    {
        const int r0 = lane >> 2, r1 = r0 + 8, c = 2 * (lane & 3);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int col = 16 * ks + c;
            qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t *>(q + r0 * HEAD_DIM + col) : 0u;
            qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t *>(q + r0 * HEAD_DIM + col + 8) : 0u;
            qa[ks][1] = (HI && r1 < G) ? *reinterpret_cast<const uint32_t *>(q + r1 * HEAD_DIM + col) : 0u;
            qa[ks][3] = (HI && r1 < G) ? *reinterpret_cast<const uint32_t *>(q + r1 * HEAD_DIM + col + 8) : 0u;
        }
    }

    float acc[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    float m0 = NEG_BIG, m1 = NEG_BIG, l0 = 0.f, l1 = 0.f;

    const int sub = lane & 15, half = lane >> 4;
    auto issue = [&](int tile, int stage, int mypos) {
        unsigned char *kb = ring + stage * 8192, *vb = kb + 4096;
        const uint32_t vm = __ballot_sync(0xffffffffu, mypos >= 0) & 0xffffu;
        if (lane == 0) s_vmask[warp][stage] = vm;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = half + 2 * i;
            const int pos = __shfl_sync(0xffffffffu, mypos, r);
            const int off = r * 256 + ((sub ^ (r & 7)) << 4);
            const bool ok = pos >= 0;
            cp_async16(kb + off, ok ? Kb + (int64_t)pos * krow + sub * 16 : Kb, ok ? 16 : 0);
            cp_async16(vb + off, ok ? Vb + (int64_t)pos * vrow + sub * 16 : Vb, ok ? 16 : 0);
        }
    };

    int it = sh.t0;
    int pos_next = (it < sh.t1) ? fetch_pos(p, head, it * TILE_ROWS + sub, sh.count) : -1;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (it < sh.t1) {
            const int mypos = pos_next;
            ++it;
            pos_next = (it < sh.t1) ? fetch_pos(p, head, it * TILE_ROWS + sub, sh.count) : -1;
            issue(it - 1, s, mypos);
        }
        cp_async_commit();
    }

    for (int t = sh.t0; t < sh.t1; ++t) {
        const int stage = (t - sh.t0) % STAGES;
        if (it < sh.t1) {
            const int mypos = pos_next;
            ++it;
            pos_next = (it < sh.t1) ? fetch_pos(p, head, it * TILE_ROWS + sub, sh.count) : -1;
            issue(it - 1, (t - sh.t0 + STAGES - 1) % STAGES, mypos);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();

        const unsigned char *kb = ring + stage * 8192, *vb = kb + 4096;
        const uint32_t vmask = s_vmask[warp][stage];
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const int row = (lane & 7) + ((lane >> 4) << 3);
            const int csel = (lane >> 3) & 1;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, kb + row * 256 + (((2 * ks + csel) ^ (row & 7)) << 4));
                mma_bf16_16816(s[0], qa[ks], b[0], b[1]);
                mma_bf16_16816(s[1], qa[ks], b[2], b[3]);
            }
        }
        // online softmax in base 2; columns of s are the tile's rows (keys)
        const int kc = 2 * (lane & 3);
        bool ok[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 2; ++i) ok[nt][i] = (vmask >> (nt * 8 + kc + i)) & 1u;
        float z0[2][2], z1[2][2];
        float mt0 = NEG_BIG, mt1 = NEG_BIG;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                z0[nt][i] = ok[nt][i] ? s[nt][i] * p.scale_log2 : NEG_BIG;
                mt0 = fmaxf(mt0, z0[nt][i]);
                if (HI) {
                    z1[nt][i] = ok[nt][i] ? s[nt][2 + i] * p.scale_log2 : NEG_BIG;
                    mt1 = fmaxf(mt1, z1[nt][i]);
                }
            }
        mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 1));
        mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 2));
        const float mn0 = fmaxf(m0, mt0);
        const float al0 = fast_exp2(m0 - mn0);
        m0 = mn0;
        float al1 = 1.f;
        if (HI) {
            mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 1));
            mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 2));
            const float mn1 = fmaxf(m1, mt1);
            al1 = fast_exp2(m1 - mn1);
            m1 = mn1;
        }
        float p0[2][2], p1[2][2];
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                p0[nt][i] = ok[nt][i] ? fast_exp2(z0[nt][i] - m0) : 0.f;
                rs0 += p0[nt][i];
                if (HI) {
                    p1[nt][i] = ok[nt][i] ? fast_exp2(z1[nt][i] - m1) : 0.f;
                    rs1 += p1[nt][i];
                }
            }
        l0 = l0 * al0 + rs0;
        if (HI) l1 = l1 * al1 + rs1;
        uint32_t pa[4];
        pa[0] = pack_bf16(p0[0][0], p0[0][1]);
        pa[2] = pack_bf16(p0[1][0], p0[1][1]);
        pa[1] = HI ? pack_bf16(p1[0][0], p1[0][1]) : 0u;
        pa[3] = HI ? pack_bf16(p1[1][0], p1[1][1]) : 0u;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            acc[j][0] *= al0;
            acc[j][1] *= al0;
            if (HI) {
                acc[j][2] *= al1;
                acc[j][3] *= al1;
            }
        }
        {
            const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
            const int csel = lane >> 4;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vb + row * 256 + (((2 * jj + csel) ^ (row & 7)) << 4));
                mma_bf16_16816(acc[2 * jj], pa, b[0], b[1]);
                mma_bf16_16816(acc[2 * jj + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    if (HI) {
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }
    __syncthreads();                       // every warp is done with its ring: reuse it
    float *red = reinterpret_cast<float *>(smem);
    {
        const int r0 = lane >> 2, r1 = r0 + 8, c = 2 * (lane & 3);
        if (r0 < G) {
            float *r = red + (warp * G + r0) * 132;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                r[8 * j + c] = acc[j][0];
                r[8 * j + c + 1] = acc[j][1];
            }
            if ((lane & 3) == 0) { r[128] = m0; r[129] = l0; }
        }
        if (HI && r1 < G) {
            float *r = red + (warp * G + r1) * 132;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                r[8 * j + c] = acc[j][2];
                r[8 * j + c + 1] = acc[j][3];
            }
            if ((lane & 3) == 0) { r[128] = m1; r[129] = l1; }
        }
    }
    __syncthreads();
    finish_head<__nv_bfloat16>(p, red, WARPS, head, split, sh.s_eff, &s_flag);
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
        const int mypos = fetch_pos(p, head, t * TILE_ROWS + sub, sh.count);
#pragma unroll 2
        for (int i = 0; i < 8; ++i) {
            const int pos = __shfl_sync(0xffffffffu, mypos, half + 2 * i);
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
                const float z = s * p.scale_log2;
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
    finish_head<T>(p, red, 2 * WARPS, head, split, sh.s_eff, &s_flag);
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

constexpr int MMA_WARPS = 4, MMA_STAGES = 3;
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

extern "C" int skv_attend_splits(int heads) {
    if (heads <= 0) return SKV_E_RANGE;
    const int sms = device_sm_count();
    int s = (2 * sms + heads - 1) / heads;
    return s < 1 ? 1 : s;
}

extern "C" int64_t skv_attend_workspace_bytes(int heads, int G, int d, int splits) {
    if (heads <= 0 || G <= 0 || d != HEAD_DIM || splits <= 0) return SKV_E_RANGE;
    int64_t acc = (int64_t)heads * splits * G * d * 4;
    int64_t ml = (int64_t)heads * splits * G * 2 * 4;
    int64_t tk = (((int64_t)heads * 4) + 255) / 256 * 256;
    return acc + ml + tk;
}

// mode bit 0 of `dtype >> 8` forces the CUDA-core path for bf16 (cross-checks)
extern "C" int skv_attend(const void *q, const void *K, const void *V, const int32_t *idx, const int32_t *cnt,
                          const int32_t *n_dev, void *out, void *workspace, int32_t *status, int heads, int G, int d,
                          int dtype, int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride,
                          int64_t v_row_stride, int64_t idx_stride, int rows_limit, int splits, float scale,
                          void *stream) {
    const int base = dtype & 0xff;
    const bool force_simple = (dtype >> 8) & 1;
    if (!q || !K || !V || !out || !workspace) return SKV_E_NULL;
    if (idx ? !cnt : !n_dev) return SKV_E_NULL;
    if (d != HEAD_DIM) return SKV_E_DIM;
    if (base != SKV_BF16 && base != SKV_F32) return SKV_E_DTYPE;
    if (heads <= 0 || heads > 65535 || splits <= 0 || splits > 65535 || rows_limit < 0) return SKV_E_RANGE;
    if (G < 1 || G > 16 || ((base == SKV_F32 || force_simple) && G > 8)) return SKV_E_DIM;
    const int esz = base == SKV_BF16 ? 2 : 4;
    if (!aligned16(q) || !aligned16(K) || !aligned16(V) || !aligned16(out) || !aligned16(workspace)) return SKV_E_ALIGN;
    if ((k_row_stride * esz) % 16 || (v_row_stride * esz) % 16 || (k_head_stride * esz) % 16 ||
        (v_head_stride * esz) % 16 || k_row_stride < d || v_row_stride < d)
        return SKV_E_ALIGN;
    AttendParams p;
    p.q = q; p.K = K; p.V = V; p.idx = idx; p.cnt = cnt; p.n_dev = n_dev; p.out = out; p.status = status;
    p.part_acc = static_cast<float *>(workspace);
    p.part_ml = p.part_acc + (int64_t)heads * splits * G * d;
    p.ticket = reinterpret_cast<int32_t *>(p.part_ml + (int64_t)heads * splits * G * 2);
    p.heads = heads; p.G = G;
    p.ksh = k_head_stride; p.ksr = k_row_stride; p.vsh = v_head_stride; p.vsr = v_row_stride;
    p.idx_stride = idx_stride; p.rows_limit = rows_limit; p.splits = splits;
    p.scale_log2 = scale * LOG2E;
    dim3 grid(splits, heads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (base == SKV_F32) return launch_simple<float>(p, grid, st);
    if (force_simple) return launch_simple<__nv_bfloat16>(p, grid, st);
    return G > 8 ? launch_mma<true>(p, grid, st) : launch_mma<false>(p, grid, st);
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
                                 const int32_t *n_dev, void *out, int32_t *status, int heads, int G, int d, int dtype,
                                 int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride,
                                 int64_t v_row_stride, int64_t idx_stride, int rows_limit, int splits, float scale,
                                 void *stream) {
    const int64_t need = skv_attend_workspace_bytes(heads, G, d, splits);
    if (need < 0) return (int)need;
    if (need > (int64_t)SKV_STATIC_SCRATCH_BYTES) return SKV_E_TOO_LARGE;
    void *scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc) return rc;
    // Earlier calls with other shapes left their partials here.  Only the ticket words have to start at
    // zero (partials are always written before they are read); they sit at the end of the layout.
    unsigned char *tickets = static_cast<unsigned char *>(scratch) + (int64_t)heads * splits * G * (d + 2) * 4;
    SKV_CUDA_OK(cudaMemsetAsync(tickets, 0, (size_t)heads * 4, static_cast<cudaStream_t>(stream)));
    return skv_attend(q, K, V, idx, cnt, n_dev, out, scratch, status, heads, G, d, dtype, k_head_stride, k_row_stride,
                      v_head_stride, v_row_stride, idx_stride, rows_limit, splits, scale, stream);
}
