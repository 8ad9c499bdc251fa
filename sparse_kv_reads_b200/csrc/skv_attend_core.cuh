// One warp's share of the gather attention: a private cp.async ring of 16-row K/V tiles in shared
// memory, mma.sync m16n8k16 bf16 tiles for Q K^T and P V, online softmax in base 2.
#pragma once

#include "skv_common.cuh"

namespace skv {

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

// Register state and pipeline of one warp.  HI: the group has more than 8 query heads (rows 8..15 of
// the M side are live).  The ring holds STAGES tiles of 16 K rows + 16 V rows (8 KB per stage).
template <int STAGES, bool HI>
struct WarpAttend {
    uint32_t qa[8][4];
    float acc[16][4];
    float m0, m1, l0, l1;
    unsigned char *ring;
    volatile uint32_t *vmask;            // [STAGES] validity bits of the rows of each staged tile
    const char *Kb, *Vb;
    int64_t krow, vrow;
    float scale_log2;
    int lane;

    __device__ __forceinline__ void init(const __nv_bfloat16 *q, int G, unsigned char *ring_, uint32_t *vmask_,
                                         const char *Kb_, const char *Vb_, int64_t krow_, int64_t vrow_,
                                         float scale_log2_) {
        lane = threadIdx.x & 31;
        ring = ring_; vmask = vmask_; Kb = Kb_; Vb = Vb_; krow = krow_; vrow = vrow_; scale_log2 = scale_log2_;
        const int r0 = lane >> 2, r1 = r0 + 8, c = 2 * (lane & 3);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int col = 16 * ks + c;
            qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t *>(q + r0 * HEAD_DIM + col) : 0u;
            qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t *>(q + r0 * HEAD_DIM + col + 8) : 0u;
            qa[ks][1] = (HI && r1 < G) ? *reinterpret_cast<const uint32_t *>(q + r1 * HEAD_DIM + col) : 0u;
            qa[ks][3] = (HI && r1 < G) ? *reinterpret_cast<const uint32_t *>(q + r1 * HEAD_DIM + col + 8) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        m0 = m1 = NEG_BIG;
        l0 = l1 = 0.f;
    }

    // start the copies of one tile; `mypos` (lanes 0..15 and again 16..31) = position of row lane%16, -1 = none
    __device__ __forceinline__ void issue(int stage, int mypos) {
        unsigned char *kb = ring + stage * 8192, *vb = kb + 4096;
        const int sub = lane & 15, half = lane >> 4;
        const uint32_t vm = __ballot_sync(0xffffffffu, mypos >= 0) & 0xffffu;
        if (lane == 0) vmask[stage] = vm;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = half + 2 * i;
            const int pos = __shfl_sync(0xffffffffu, mypos, r);
            const int off = r * 256 + ((sub ^ (r & 7)) << 4);
            const bool ok = pos >= 0;
            cp_async16(kb + off, ok ? Kb + (int64_t)pos * krow + sub * 16 : Kb, ok ? 16 : 0);
            cp_async16(vb + off, ok ? Vb + (int64_t)pos * vrow + sub * 16 : Vb, ok ? 16 : 0);
        }
    }

    // scores, online softmax and the P V update for the tile staged in `stage`
    __device__ __forceinline__ void consume(int stage) {
        const unsigned char *kb = ring + stage * 8192, *vb = kb + 4096;
        const uint32_t vm = vmask[stage];
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
        const int kc = 2 * (lane & 3);
        bool ok[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 2; ++i) ok[nt][i] = (vm >> (nt * 8 + kc + i)) & 1u;
        float z0[2][2], z1[2][2];
        float mt0 = NEG_BIG, mt1 = NEG_BIG;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                z0[nt][i] = ok[nt][i] ? s[nt][i] * scale_log2 : NEG_BIG;
                mt0 = fmaxf(mt0, z0[nt][i]);
                if (HI) {
                    z1[nt][i] = ok[nt][i] ? s[nt][2 + i] * scale_log2 : NEG_BIG;
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
    }

    // Tiles [t0, t1) of a row list; pos_of(row) gives the cached position of list entry `row` or -1.
    // All copies have landed and been consumed on return, so the call can be repeated.
    template <typename PosFn>
    __device__ __forceinline__ void run(int t0, int t1, PosFn pos_of) {
        const int sub = lane & 15;
        int it = t0;
        int pos_next = (it < t1) ? pos_of(it * TILE_ROWS + sub) : -1;
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (it < t1) {
                const int mypos = pos_next;
                ++it;
                pos_next = (it < t1) ? pos_of(it * TILE_ROWS + sub) : -1;
                issue(s, mypos);
            }
            cp_async_commit();
        }
        for (int t = t0; t < t1; ++t) {
            const int stage = (t - t0) % STAGES;
            if (it < t1) {
                const int mypos = pos_next;
                ++it;
                pos_next = (it < t1) ? pos_of(it * TILE_ROWS + sub) : -1;
                issue((t - t0 + STAGES - 1) % STAGES, mypos);
            }
            cp_async_commit();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            consume(stage);
            __syncwarp();
        }
        cp_async_wait<0>();
    }

    // leave this warp's (acc, max, sum) for rows < G in red[(warp*G + g)*132 ...]
    __device__ __forceinline__ void store_partial(float *red, int warp, int G) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        if (HI) {
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        }
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
};

// The same warp worker for groups of at most 8 query heads, with the operand roles swapped: the 16 keys of
// a tile sit on the M side of S^T = K Q^T and the (<= 8) heads on N, so no accumulator row is padding; P is
// turned into the B operand of O^T = V^T P with two movmatrix transposes.  Half the MMAs and 32 fewer
// registers than the heads-on-M layout.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

template <int STAGES>
struct WarpAttendT {
    uint32_t qb[8][2];                   // Q^T fragments: [k-step][d, d + 8], column = head
    float acc[8][4];                     // O^T: [16-row d tile]: (d, hA), (d, hB), (d + 8, hA), (d + 8, hB)
    float mA, mB, lA, lB;                // running max / partial sum of heads hA = 2 (lane % 4), hB = hA + 1
    unsigned char *ring;
    volatile uint32_t *vmask;
    const char *Kb, *Vb;
    int64_t krow, vrow;
    float scale_log2;
    int lane;

    __device__ __forceinline__ void init(const __nv_bfloat16 *q, int G, unsigned char *ring_, uint32_t *vmask_,
                                         const char *Kb_, const char *Vb_, int64_t krow_, int64_t vrow_,
                                         float scale_log2_) {
        lane = threadIdx.x & 31;
        ring = ring_; vmask = vmask_; Kb = Kb_; Vb = Vb_; krow = krow_; vrow = vrow_; scale_log2 = scale_log2_;
        const int head = lane >> 2, c = 2 * (lane & 3);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int col = 16 * ks + c;
            qb[ks][0] = head < G ? *reinterpret_cast<const uint32_t *>(q + head * HEAD_DIM + col) : 0u;
            qb[ks][1] = head < G ? *reinterpret_cast<const uint32_t *>(q + head * HEAD_DIM + col + 8) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        mA = mB = NEG_BIG;
        lA = lB = 0.f;
    }

    __device__ __forceinline__ void issue(int stage, int mypos) {
        unsigned char *kb = ring + stage * 8192, *vb = kb + 4096;
        const int sub = lane & 15, half = lane >> 4;
        const uint32_t vm = __ballot_sync(0xffffffffu, mypos >= 0) & 0xffffu;
        if (lane == 0) vmask[stage] = vm;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = half + 2 * i;
            const int pos = __shfl_sync(0xffffffffu, mypos, r);
            const int off = r * 256 + ((sub ^ (r & 7)) << 4);
            const bool ok = pos >= 0;
            cp_async16(kb + off, ok ? Kb + (int64_t)pos * krow + sub * 16 : Kb, ok ? 16 : 0);
            cp_async16(vb + off, ok ? Vb + (int64_t)pos * vrow + sub * 16 : Vb, ok ? 16 : 0);
        }
    }

    __device__ __forceinline__ void consume(int stage) {
        const unsigned char *kb = ring + stage * 8192, *vb = kb + 4096;
        const uint32_t vm = vmask[stage];
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            float s2[4] = {0.f, 0.f, 0.f, 0.f};          // two chains of four products: half the dependent latency
            const int mi = lane >> 3;
            const int row = (lane & 7) + ((mi & 1) << 3), csel = mi >> 1;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, kb + row * 256 + (((2 * ks + csel) ^ (row & 7)) << 4));
                if (ks & 1) mma_bf16_16816(s2, a, qb[ks][0], qb[ks][1]);
                else mma_bf16_16816(s, a, qb[ks][0], qb[ks][1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += s2[i];
        }
        const int k0 = lane >> 2;                        // this lane's keys: k0 and k0 + 8
        const bool ok0 = (vm >> k0) & 1u, ok1 = (vm >> (k0 + 8)) & 1u;
        const float zA0 = ok0 ? s[0] * scale_log2 : NEG_BIG, zB0 = ok0 ? s[1] * scale_log2 : NEG_BIG;
        const float zA1 = ok1 ? s[2] * scale_log2 : NEG_BIG, zB1 = ok1 ? s[3] * scale_log2 : NEG_BIG;
        float tA = fmaxf(zA0, zA1), tB = fmaxf(zB0, zB1);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {               // over the 8 lanes that share lane % 4
            tA = fmaxf(tA, __shfl_xor_sync(0xffffffffu, tA, o));
            tB = fmaxf(tB, __shfl_xor_sync(0xffffffffu, tB, o));
        }
        const float nA = fmaxf(mA, tA), nB = fmaxf(mB, tB);
        const float alA = fast_exp2(mA - nA), alB = fast_exp2(mB - nB);
        mA = nA; mB = nB;
        const float pA0 = ok0 ? fast_exp2(zA0 - nA) : 0.f, pB0 = ok0 ? fast_exp2(zB0 - nB) : 0.f;
        const float pA1 = ok1 ? fast_exp2(zA1 - nA) : 0.f, pB1 = ok1 ? fast_exp2(zB1 - nB) : 0.f;
        lA = lA * alA + pA0 + pA1;
        lB = lB * alB + pB0 + pB1;
        const uint32_t b0 = movmatrix_trans(pack_bf16(pA0, pB0));      // keys 0-7   -> k = 2 (lane % 4) + {0, 1}
        const uint32_t b1 = movmatrix_trans(pack_bf16(pA1, pB1));      // keys 8-15
        if (__any_sync(0xffffffffu, alA != 1.f || alB != 1.f)) {       // the maxima settle after a few tiles
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[j][0] *= alA; acc[j][1] *= alB;
                acc[j][2] *= alA; acc[j][3] *= alB;
            }
        }
        {
            const int mi = lane >> 3;
            const int row = (lane & 7) + ((mi >> 1) << 3), csel = mi & 1;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, vb + row * 256 + (((2 * mt + csel) ^ (row & 7)) << 4));
                mma_bf16_16816(acc[mt], a, b0, b1);
            }
        }
    }

    template <typename PosFn>
    __device__ __forceinline__ void run(int t0, int t1, PosFn pos_of) {
        const int sub = lane & 15;
        int it = t0;
        int pos_next = (it < t1) ? pos_of(it * TILE_ROWS + sub) : -1;
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (it < t1) {
                const int mypos = pos_next;
                ++it;
                pos_next = (it < t1) ? pos_of(it * TILE_ROWS + sub) : -1;
                issue(s, mypos);
            }
            cp_async_commit();
        }
        for (int t = t0; t < t1; ++t) {
            const int stage = (t - t0) % STAGES;
            if (it < t1) {
                const int mypos = pos_next;
                ++it;
                pos_next = (it < t1) ? pos_of(it * TILE_ROWS + sub) : -1;
                issue((t - t0 + STAGES - 1) % STAGES, mypos);
            }
            cp_async_commit();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            consume(stage);
            __syncwarp();
        }
        cp_async_wait<0>();
    }

    __device__ __forceinline__ void store_partial(float *red, int warp, int G) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            lA += __shfl_xor_sync(0xffffffffu, lA, o);
            lB += __shfl_xor_sync(0xffffffffu, lB, o);
        }
        const int hA = 2 * (lane & 3), hB = hA + 1, d0 = lane >> 2;
        if (hA < G) {
            float *r = red + (warp * G + hA) * 132;
#pragma unroll
            for (int j = 0; j < 8; ++j) { r[16 * j + d0] = acc[j][0]; r[16 * j + d0 + 8] = acc[j][2]; }
            if (d0 == 0) { r[128] = mA; r[129] = lA; }
        }
        if (hB < G) {
            float *r = red + (warp * G + hB) * 132;
#pragma unroll
            for (int j = 0; j < 8; ++j) { r[16 * j + d0] = acc[j][1]; r[16 * j + d0 + 8] = acc[j][3]; }
            if (d0 == 0) { r[128] = mB; r[129] = lB; }
        }
    }
};

}  // namespace skv
