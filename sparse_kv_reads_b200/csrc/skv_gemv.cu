// Matrix-vector products of the single-token (decode) forward: y[B, N] = x[B, K] . W[N, K]^T for a handful of
// sequences (B <= 8), bf16 in and out, float32 accumulation.  The weights are read exactly once, so the
// product is bound by HBM; what decides its speed at this size is how early the bytes are requested.
//
// A CTA owns a run of consecutive rows of W - one contiguous slab of memory, at most 96 KB - and asks for all
// of it with 16-byte asynchronous copies into shared memory as its very first action.  Under programmatic
// dependent launch that happens while the kernel ahead on the stream is still finishing: weights are written by
// no kernel, so they may be fetched before the wait, and only the input vector has to wait for the producer.
// The input is then built in shared memory in one of three ways, each CTA for itself (it is a few KB, read
// from L2), which folds the element-wise kernels between the products into them:
//   mode 0  x as given;
//   mode 1  residual add and RMSNorm: h_out = bf16(h_in + delta), x = bf16(h_out * rsqrt(mean(h_out^2) + eps) * g)
//           (CTA 0 also stores h_out, out of place because the other CTAs still read h_in);
//   mode 2  x = bf16(bf16(silu(gate)) * up) from gate_up[B, 2K];
//   mode 4  x = the attention output, merged here from the split partials the one-launch decode step left
//           (skv_gemv_attended): the output product does the last log-sum-exp merge while it builds its input.
// The roundings are those of the separate kernels (skv_dense.cu) and of the unfused module forward.
// The products themselves run on the tensor cores where K is a multiple of 64: 16 rows of the slab x 16 inputs
// are one mma.sync m16n8k16 A tile (ldmatrix from the slab, stored with its 16-byte pieces XOR-swizzled by the
// row so that the eight rows of a matrix fall into different banks), the B tile holds up to 8 sequences, so 1
// and 8 sequences cost the same.  The 8 warps share the slab's 16-row tiles and, when there are fewer than 8
// tiles, ranges of K; partial sums meet in shared memory.  Other K take a plain float path: warp w multiplies
// rows w, w + 8, ... piece by piece with every sequence's input and reduces the sums over its lanes.
#include "skv_attend_core.cuh"

#include <cstring>

namespace skv {

constexpr int GEMV_THREADS = 256, GEMV_WARPS = 8;
constexpr int GEMV_SLAB_MAX = 96 * 1024;

struct GemvParams {
    const __nv_bfloat16 *W;
    __nv_bfloat16 *y;
    int N, K, B, mode, rows_per_cta;
    int row_group;                 // float path: rows a warp takes at a time (1 or 2)
    int nslabs, stages;            // slabs of rows_per_cta rows over the matrix; 1 or 2 slab buffers per CTA
    const __nv_bfloat16 *x;        // mode 0: [B, K]; mode 2: gate_up [B, 2K]
    const __nv_bfloat16 *h_in, *delta, *g;
    __nv_bfloat16 *h_out;
    float eps;
    // exchange through peer memory (row-parallel products of a tensor-parallel group); world 0 = unused
    uint2 *out_data[8];            // every rank's buffer: [2 slots][world][cap] of {value bits, epoch}
    const uint32_t *out_tick;
    int out_world, out_rank, out_seq, out_cap;
    const uint2 *in_data;          // the local buffer
    const uint32_t *in_tick;
    int in_world, in_seq, in_cap, wait_limit;
    int32_t *status;
    // mode 4: the input is the attention output, still in the split partials skv_step left ([heads, ncl, G, 132]
    // floats: 128 sums, running maximum in base-2 units, sum of weights, rows read): every CTA merges them itself
    const float *att_part;
    int att_ncl, att_G;
    int32_t *att_cnt;              // [heads] rows read per head, written by CTA 0 (may be null)
};

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16(x)); }

constexpr int WAIT_KPOLLS_DEFAULT = 8192;   // x 1024 polls of a little under a microsecond each: about five seconds

// Every exchanged value travels as ONE 64-bit word {float bits, epoch}, stored and loaded as a single 64-bit
// access: the memory model makes each such access single-copy atomic, so value and epoch cannot be seen apart (a
// vector access of two 32-bit halves would formally be two accesses in no given order).  The epoch names the
// decode step (the buffer's tick) and the exchange within it, so a reader that finds the epoch it expects has the
// value too - no fence, no separate flag, one NVLink flight.
__device__ __forceinline__ uint32_t epoch_of(const uint32_t *tick, int seq) { return tick[0] * 256u + (uint32_t)seq + 1u; }

__device__ __forceinline__ void store_pair(uint2 *dst, float v, uint32_t epoch) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)epoch << 32);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
}

// Eight consecutive partial sums of one rank (64 bytes = four 16-byte loads of two 64-bit words each), polled
// until all eight carry `epoch`; bounded: on expiry *status gets SKV_ST_WAIT_TIMEOUT and whatever is there is
// used.  A wait that does not succeed at once looks at the status word first: once any wait of this GPU has
// given up (the word is sticky until the host clears it), later waits give up after a single look instead of
// each spending the full limit, so a lost peer costs one limit per step and not one per polled element.
__device__ __forceinline__ void load_pairs8(const uint2 *src, uint32_t epoch, int32_t *status, int limit,
                                            float (&out)[8]) {
    unsigned long long q[8];
    int it = 0;
    for (;;) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];"
                         : "=l"(q[2 * i]), "=l"(q[2 * i + 1])
                         : "l"(reinterpret_cast<const uint4 *>(src) + i) : "memory");
        bool ok = true;
#pragma unroll
        for (int i = 0; i < 8; ++i) ok = ok && (uint32_t)(q[i] >> 32) == epoch;
        if (ok) break;
        if (it == 0 && status && (*reinterpret_cast<volatile int32_t *>(status) & SKV_ST_WAIT_TIMEOUT)) break;
        if (++it >= limit) {
            if (status) atomicOr(status, SKV_ST_WAIT_TIMEOUT);
            break;
        }
        __nanosleep(40);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __uint_as_float((uint32_t)q[i]);
}

// One output value: to y, or as a float partial into slot/rank of every GPU's buffer.
__device__ __forceinline__ void emit(const GemvParams &p, int b, int row, float v, uint32_t epoch) {
    if (p.out_world == 0) {
        p.y[(size_t)b * p.N + row] = __float2bfloat16(v);
        return;
    }
    const size_t off = (size_t)((p.out_seq & 1) * p.out_world + p.out_rank) * p.out_cap + (size_t)b * p.N + row;
#pragma unroll
    for (int r = 0; r < 8; ++r)
        if (r < p.out_world) store_pair(p.out_data[r] + off, v, epoch);
}

// The float path of a slab: a warp takes NR rows at a time, so that the input is read and unpacked once for all of
// them and their sums are independent chains (each row's sum is added up in the same order as it would be alone).
template <int BP, int NR>
__device__ __forceinline__ void rows_dot(const GemvParams &p, const __nv_bfloat16 *ws, const __nv_bfloat16 *xs, int R,
                                         int r0, int K, int kv, uint32_t out_epoch) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int r = wid * NR; r < R; r += GEMV_WARPS * NR) {
        float acc[NR][BP];
        const __nv_bfloat16 *wr[NR];
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            wr[j] = ws + (size_t)min(r + j, R - 1) * K;   // rows past the slab repeat its last row; their sums are dropped
#pragma unroll
            for (int b = 0; b < BP; ++b) acc[j][b] = 0.f;
        }
#pragma unroll 2
        for (int v = lane; v < kv; v += 32) {
            float w[NR][8];
#pragma unroll
            for (int j = 0; j < NR; ++j) load8(wr[j] + v * 8, w[j]);
#pragma unroll
            for (int b = 0; b < BP; ++b) {
                float xv[8];
                load8(xs + (size_t)b * K + v * 8, xv);
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < NR; ++j) acc[j][b] = fmaf(w[j][i], xv[i], acc[j][b]);
            }
        }
#pragma unroll
        for (int j = 0; j < NR; ++j)
#pragma unroll
            for (int b = 0; b < BP; ++b) {
                const float sum = warp_sum(acc[j][b]);
                if (lane == 0 && b < p.B && r + j < R) emit(p, b, r0 + r + j, sum, out_epoch);
            }
    }
}

// MULTI: the CTA walks over several slabs with two buffers (else exactly one slab, and no loop to pay for)
template <int BP, bool TC, bool MULTI>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float s_part[8][GEMV_WARPS];
    __shared__ __align__(16) float s_red[GEMV_WARPS][16 * 8];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int K = p.K, kv = K >> 3;                         // 16-byte pieces per row
    const int xld = TC ? K + 8 : K;                         // input row stride: 16 bytes of padding spread the banks
    __nv_bfloat16 *ws0 = reinterpret_cast<__nv_bfloat16 *>(smem);                     // [stages][rows_per_cta][K]
    __nv_bfloat16 *xs = ws0 + (size_t)(MULTI ? 2 : 1) * p.rows_per_cta * K;           // [BP][xld]
    __nv_bfloat16 *gs = xs + (size_t)BP * xld;                                        // [K] (mode 1)
    // A CTA takes slabs blockIdx.x, blockIdx.x + gridDim.x, ...: one when a wave of CTAs covers the matrix, else
    // several, the next one streaming into the other buffer while this one is multiplied.
    auto request_slab = [&](int slab, __nv_bfloat16 *ws) {
        const int r0 = slab * p.rows_per_cta;
        const int R = min(p.rows_per_cta, p.N - r0);
        const __nv_bfloat16 *src = p.W + (size_t)r0 * K;
        const int pieces = R * kv;
        if (TC) {                                           // pieces swizzled by their row
            const unsigned inv = (unsigned)((0x100000000ull + kv - 1) / kv);   // c / kv by multiplication: exact for c < 2^16
            for (int c = tid; c < pieces; c += GEMV_THREADS) {
                const int r = (int)__umulhi((unsigned)c, inv), col = c - r * kv;
                cp_async16(ws + (size_t)r * K + ((col ^ (r & 7)) << 3), src + (size_t)c * 8, 16);
            }
        } else {
            for (int c = tid; c < pieces; c += GEMV_THREADS) cp_async16(ws + (size_t)c * 8, src + (size_t)c * 8, 16);
        }
    };

    // 1. the slab (and the norm weights): requested before anything else, also before the producer ends
    {
        if (p.mode == 1 || p.mode == 3)
            for (int c = tid; c < kv; c += GEMV_THREADS) cp_async16(gs + c * 8, p.g + c * 8, 16);
        cp_async_commit();                                  // group 0: norm weights (empty otherwise)
        request_slab(blockIdx.x, ws0);
        cp_async_commit();                                  // group 1: the first slab
    }
    pdl_wait();
    pdl_trigger();
    const uint32_t out_epoch = p.out_world ? epoch_of(p.out_tick, p.out_seq) : 0u;
    const uint32_t in_epoch = p.mode == 3 ? epoch_of(p.in_tick, p.in_seq) : 0u;

    // 2. the input of every sequence, in shared memory as bf16
    if (p.mode == 4) {
        // log-sum-exp merge of the attention partials, eight output components at a time; element e of the input
        // row-major over (sequence, query head, component) belongs to query head e / 128 of the partials
        const int ncl = p.att_ncl, G = p.att_G;
        for (int c = tid; c < BP * kv; c += GEMV_THREADS) {
            const int b = c / kv, v = c - b * kv;
            __align__(16) __nv_bfloat16 o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(0.f);
            if (b < p.B) {
                const size_t e0 = (size_t)b * K + (size_t)v * 8;
                const size_t qh = e0 >> 7;                   // flat query head: (sequence, KV head, head of the group)
                const int t0 = (int)(e0 & 127);
                const size_t head = qh / G;
                const int g = (int)(qh - head * G);
                float4 a0[8], a1[8];
                float pm[8], pd[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {                // every load goes out before any value is used
                    pm[k] = NEG_BIG; pd[k] = 0.f;
                    a0[k] = a1[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (k < ncl) {
                        const float *row = p.att_part + ((head * ncl + k) * G + g) * 132;
                        pm[k] = __ldcg(row + 128);
                        pd[k] = __ldcg(row + 129);
                        a0[k] = __ldcg(reinterpret_cast<const float4 *>(row + t0));
                        a1[k] = __ldcg(reinterpret_cast<const float4 *>(row + t0 + 4));
                    }
                }
                float M = NEG_BIG;
#pragma unroll
                for (int k = 0; k < 8; ++k) M = fmaxf(M, pm[k]);
                float dn = 0.f, nm[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float f = fast_exp2(pm[k] - M);
                    dn = fmaf(f, pd[k], dn);
                    nm[0] = fmaf(f, a0[k].x, nm[0]); nm[1] = fmaf(f, a0[k].y, nm[1]);
                    nm[2] = fmaf(f, a0[k].z, nm[2]); nm[3] = fmaf(f, a0[k].w, nm[3]);
                    nm[4] = fmaf(f, a1[k].x, nm[4]); nm[5] = fmaf(f, a1[k].y, nm[5]);
                    nm[6] = fmaf(f, a1[k].z, nm[6]); nm[7] = fmaf(f, a1[k].w, nm[7]);
                }
                const float inv = dn > 0.f ? 1.0f / dn : 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(nm[k] * inv);
            }
            *reinterpret_cast<uint4 *>(xs + (size_t)b * xld + v * 8) = *reinterpret_cast<const uint4 *>(o);
        }
        if (blockIdx.x == 0 && p.att_cnt) {
            const int heads = (int)(((size_t)p.B * K) >> 7) / G;
            for (int hd = tid; hd < heads; hd += GEMV_THREADS) {
                float rows = 0.f;
                for (int k = 0; k < ncl; ++k) rows += __ldcg(p.att_part + (((size_t)hd * ncl + k) * G) * 132 + 130);
                p.att_cnt[hd] = (int)rows;
            }
        }
    } else if (p.mode == 0) {
        for (int c = tid; c < BP * kv; c += GEMV_THREADS) {
            const int b = c / kv, v = c - b * kv;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (b < p.B) val = __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)b * K + v * 8));
            *reinterpret_cast<uint4 *>(xs + (size_t)b * xld + v * 8) = val;
        }
    } else if (p.mode == 2) {
        for (int c = tid; c < BP * kv; c += GEMV_THREADS) {
            const int b = c / kv, v = c - b * kv;
            __align__(16) __nv_bfloat16 o[8];
            if (b < p.B) {
                float g[8], u[8];
                load8(p.x + (size_t)b * 2 * K + v * 8, g);
                load8(p.x + (size_t)b * 2 * K + K + v * 8, u);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(bf16r(g[k] / (1.f + __expf(-g[k]))) * u[k]);
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(0.f);
            }
            *reinterpret_cast<uint4 *>(xs + (size_t)b * xld + v * 8) = *reinterpret_cast<const uint4 *>(o);
        }
    } else {
        // BP sequences share the 8 warps: wpr warps per sequence, each a contiguous range of the row
        constexpr int wpr = GEMV_WARPS / BP;
        const int b = wid / wpr, sub = wid % wpr;
        const int per = (kv + wpr - 1) / wpr;
        const int v0 = min(sub * per, kv), v1 = min(v0 + per, kv);
        float ss = 0.f;
        if (b < p.B) {
            const __nv_bfloat16 *hr = p.h_in + (size_t)b * K;
            const __nv_bfloat16 *dr = p.delta ? p.delta + (size_t)b * K : nullptr;
            const bool summed = p.mode == 3;                 // delta = sum of the ranks' partials, in rank order
            for (int v = v0 + lane; v < v1; v += 32) {
                float a[8];
                load8(hr + v * 8, a);
                __align__(16) __nv_bfloat16 o[8];
                if (dr || summed) {
                    float d[8];
                    if (summed) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) d[i] = 0.f;
                        for (int r = 0; r < p.in_world; ++r) {
                            float part[8];
                            load_pairs8(p.in_data + (size_t)((p.in_seq & 1) * p.in_world + r) * p.in_cap + (size_t)b * K + v * 8,
                                        in_epoch, p.status, p.wait_limit, part);
#pragma unroll
                            for (int i = 0; i < 8; ++i) d[i] += part[i];
                        }
                    } else {
                        load8(dr + v * 8, d);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        o[i] = __float2bfloat16(a[i] + d[i]);
                        a[i] = __bfloat162float(o[i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16(a[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(a[i], a[i], ss);
                *reinterpret_cast<uint4 *>(xs + (size_t)b * xld + v * 8) = *reinterpret_cast<const uint4 *>(o);
                if (blockIdx.x == 0 && p.h_out)
                    *reinterpret_cast<uint4 *>(p.h_out + (size_t)b * K + v * 8) = *reinterpret_cast<const uint4 *>(o);
            }
        } else if (b < BP) {
            for (int v = v0 + lane; v < v1; v += 32) *reinterpret_cast<uint4 *>(xs + (size_t)b * xld + v * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        ss = warp_sum(ss);
        if (lane == 0) s_part[wid / wpr][sub] = ss;
        cp_async_wait<1>();                                 // the norm weights have landed
        __syncthreads();
        if (b < p.B) {
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < wpr; ++i) tot += s_part[b][i];
            const float inv = rsqrtf(tot / (float)K + p.eps);
            for (int v = v0 + lane; v < v1; v += 32) {
                float a[8], g[8];
                load8(xs + (size_t)b * xld + v * 8, a);
                load8(gs + v * 8, g);
                __align__(16) __nv_bfloat16 o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16(a[i] * inv * g[i]);
                *reinterpret_cast<uint4 *>(xs + (size_t)b * xld + v * 8) = *reinterpret_cast<const uint4 *>(o);
            }
        }
    }
    // 3. the slabs
    int it = 0;
    for (int slab = blockIdx.x; slab < (MULTI ? p.nslabs : (int)blockIdx.x + 1); slab += gridDim.x, ++it) {
    const __nv_bfloat16 *ws = MULTI ? ws0 + (size_t)(it & 1) * p.rows_per_cta * K : ws0;
    const int r0 = slab * p.rows_per_cta;
    const int R = min(p.rows_per_cta, p.N - r0);
    if (MULTI && slab + (int)gridDim.x < p.nslabs) {
        request_slab(slab + gridDim.x, ws0 + (size_t)((it + 1) & 1) * p.rows_per_cta * K);
        cp_async_commit();
        cp_async_wait<1>();                                 // all but the slab just requested have landed
    } else {
        cp_async_wait<0>();
    }
    __syncthreads();
    if (TC) {
        const int ntiles = (R + 15) >> 4;
        const int ks = ntiles >= GEMV_WARPS ? 1 : GEMV_WARPS / ntiles;      // ranges of K per tile
        const int steps = K >> 4, per = (steps + ks - 1) / ks;
        const int n = lane >> 2, kq = 2 * (lane & 3);                        // B fragment: sequence n, inputs kq, kq + 1
        const __nv_bfloat16 *xrow = xs + (size_t)n * xld + kq;
        const int arow = (lane & 7) + ((lane >> 3) & 1) * 8, apiece = lane >> 4;
        for (int item = wid; item < ntiles * ks; item += GEMV_WARPS) {
            const int t = item % ntiles, sp = item / ntiles;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const int row = min(t * 16 + arow, R - 1);      // rows past the slab repeat its last row; their sums are dropped
            const __nv_bfloat16 *abase = ws + (size_t)row * K;
            const int s1 = min((sp + 1) * per, steps);
#pragma unroll 4
            for (int st = sp * per; st < s1; ++st) {
                uint32_t a[4];
                ldmatrix_x4(a, abase + (((2 * st + apiece) ^ (row & 7)) << 3));
                uint32_t b0 = 0u, b1 = 0u;
                if (n < BP) {
                    b0 = *reinterpret_cast<const uint32_t *>(xrow + st * 16);
                    b1 = *reinterpret_cast<const uint32_t *>(xrow + st * 16 + 8);
                }
                mma_bf16_16816(acc, a, b0, b1);
            }
            // D fragment: rows lane / 4 and + 8 of the tile, sequences kq and kq + 1
            if (ks == 1) {
                const int ra = r0 + t * 16 + (lane >> 2), rb = ra + 8;
                if (kq < p.B) {
                    if (ra < r0 + R) emit(p, kq, ra, acc[0], out_epoch);
                    if (rb < r0 + R) emit(p, kq, rb, acc[2], out_epoch);
                }
                if (kq + 1 < p.B) {
                    if (ra < r0 + R) emit(p, kq + 1, ra, acc[1], out_epoch);
                    if (rb < r0 + R) emit(p, kq + 1, rb, acc[3], out_epoch);
                }
            } else {
                float *d = s_red[item];                    // [row in tile][sequence]
                d[(lane >> 2) * 8 + kq] = acc[0];
                d[(lane >> 2) * 8 + kq + 1] = acc[1];
                d[((lane >> 2) + 8) * 8 + kq] = acc[2];
                d[((lane >> 2) + 8) * 8 + kq + 1] = acc[3];
            }
        }
        if (ks > 1) {                                       // fewer than 8 tiles: one pass, sum the K ranges
            __syncthreads();
            for (int o = tid; o < ntiles * 128; o += GEMV_THREADS) {
                const int t = o >> 7, e = o & 127, rr = e >> 3, b = e & 7;
                float sum = 0.f;
                for (int sp = 0; sp < ks; ++sp) sum += s_red[sp * ntiles + t][e];
                const int rg = t * 16 + rr;
                if (rg < R && b < p.B) emit(p, b, r0 + rg, sum, out_epoch);
            }
        }
    } else
    if (p.row_group == 2) rows_dot<BP, 2>(p, ws, xs, R, r0, K, kv, out_epoch);
    else rows_dot<BP, 1>(p, ws, xs, R, r0, K, kv, out_epoch);
    if (MULTI) __syncthreads();                             // this buffer and s_red are free for the slab after next
    }
}

// The write side of an exchange for producers that are not a product of this file (a library GEMM at batches beyond
// 8): this rank's partial sums y[total] (bf16) go, as float values paired with the epoch, into its place in every
// GPU's buffer - two pairs per 16-byte store, each 64-bit pair single-copy atomic.
struct PushTargets {
    uint2 *data[8];
};
__global__ void __launch_bounds__(256) comm_push_kernel(const __nv_bfloat16 *y, int total, PushTargets out,
                                                        const uint32_t *tick, int world, int rank, int seq, int cap) {
    pdl_wait();
    pdl_trigger();
    const uint32_t epoch = epoch_of(tick, seq);
    const size_t base = (size_t)((seq & 1) * world + rank) * cap;
    for (int v = blockIdx.x * 256 + threadIdx.x; v < total / 8; v += gridDim.x * 256) {
        float f[8];
        load8(y + (size_t)v * 8, f);
        unsigned long long w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = (unsigned long long)__float_as_uint(f[i]) | ((unsigned long long)epoch << 32);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= world) break;
            uint2 *dst = out.data[r] + base + (size_t)v * 8;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(dst + 2 * i), "l"(w[2 * i]), "l"(w[2 * i + 1])
                             : "memory");
        }
    }
}

// delta[B, N] = sum over ranks of an exchange's partials, for consumers that are not a product of this file and
// for groups whose partials are too many for every CTA of the consuming product to add up for itself.  Eight
// lanes share a run of eight elements, one rank each, so that all ranks are polled at once; their values meet
// in a fixed tree of shuffles (the same on every GPU, so all GPUs obtain the same bits).
__global__ void __launch_bounds__(256) comm_reduce_kernel(const uint2 *data, const uint32_t *tick, int world, int seq,
                                                          int cap, int32_t *status, int limit, __nv_bfloat16 *delta,
                                                          int total) {
    pdl_wait();
    pdl_trigger();
    const uint32_t epoch = epoch_of(tick, seq);
    const int r = threadIdx.x & 7;
    const int vecs = total / 8;
    for (int v0 = (blockIdx.x * 256 + threadIdx.x) >> 3; v0 < ((vecs + 31) & ~31); v0 += (gridDim.x * 256) >> 3) {
        float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const bool live = v0 < vecs;
        if (live && r < world)
            load_pairs8(data + (size_t)((seq & 1) * world + r) * cap + (size_t)v0 * 8, epoch, status, limit, d);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1)
#pragma unroll
            for (int i = 0; i < 8; ++i) d[i] += __shfl_xor_sync(0xffffffffu, d[i], o);
        if (live && r == 0) {
            __align__(16) __nv_bfloat16 o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16(d[i]);
            *reinterpret_cast<uint4 *>(delta + (size_t)v0 * 8) = *reinterpret_cast<const uint4 *>(o);
        }
    }
}

__global__ void comm_tick_kernel(uint32_t *tick) { tick[0] += 1u; }

struct GemvPlan {
    int BP, rows, nslabs, stages, ctas;
    bool tc, worthwhile;
    size_t smem;
};

// Rows per slab, slabs per CTA and shared memory.  Where one CTA per SM covers the matrix with slabs of at most
// 96 KB, every CTA takes one slab (all of it requested at once).  Larger matrices run two CTAs per SM that
// each walk over several smaller slabs with two buffers, the next slab streaming in while this one is
// multiplied; the inputs are then built once per CTA, not once per slab.  `worthwhile` is false when the inputs
// every CTA rebuilds outweigh what it multiplies them with (many sequences of a long row, one slab per CTA):
// a library GEMM serves those shapes better.
static int plan_gemv(int N, int K, int B, int mode, GemvPlan &pl) {
    if (B < 1 || B > 8 || N < 1 || K < 8 || K % 8 || mode < 0 || mode > 3) return SKV_E_RANGE;
    pl.BP = B <= 1 ? 1 : (B <= 2 ? 2 : (B <= 4 ? 4 : 8));
    // one sequence: the float path needs no reduction, and the tensor-core path gains nothing there (measured in the
    // decode step at batch 1: 704 against 707 tok/s)
    pl.tc = K % 64 == 0 && pl.BP > 1;
    const size_t row = (size_t)K * 2;
    const size_t fixed = (size_t)pl.BP * (row + (pl.tc ? 16 : 0)) + (mode == 1 || mode == 3 ? row : 0);   // inputs (+ norm weights)
    const size_t optin = (size_t)device_max_smem_optin();
    const size_t per_cta = optin / 2 - 2048;
    const int sms = device_sm_count();
    size_t slab = per_cta > fixed ? per_cta - fixed : 0;
    if (slab > (size_t)GEMV_SLAB_MAX) slab = GEMV_SLAB_MAX;
    int rows = (N + sms - 1) / sms;
    if (slab >= row && (size_t)rows * row <= slab) {                      // one slab per CTA, one CTA per SM
        pl.stages = 1;
        pl.rows = rows;
        pl.nslabs = (N + rows - 1) / rows;
        pl.ctas = pl.nslabs;
        pl.smem = (size_t)rows * row + fixed;
        pl.worthwhile = slab >= 2 * fixed;
        return SKV_OK;
    }
    if (pl.BP > 1 && slab >= row && (int64_t)N <= 2LL * sms * (int64_t)(slab / row)) {
        // several sequences, up to two such waves: still one (large) slab per CTA, two CTAs per SM - the tensor-core
        // path pays per slab for its barriers and reduction, so few large slabs beat many small ones
        pl.stages = 1;
        pl.rows = (N + 2 * sms - 1) / (2 * sms);
        pl.nslabs = (N + pl.rows - 1) / pl.rows;
        pl.ctas = pl.nslabs;
        pl.smem = (size_t)pl.rows * row + fixed;
        pl.worthwhile = slab >= 2 * fixed;
        return SKV_OK;
    }
    pl.stages = 2;
    size_t half = per_cta > fixed ? (per_cta - fixed) / 2 : 0;            // two CTAs per SM, two buffers each
    if (half > 48 * 1024) half = 48 * 1024;
    if (half < row) {                                                     // long rows: one CTA per SM
        half = optin > fixed + 2 * row + 2048 ? (optin - fixed - 2048) / 2 : 0;
        if (half > 48 * 1024) half = 48 * 1024;
    }
    if (half < row) return SKV_E_TOO_LARGE;
    pl.rows = (int)(half / row);
    pl.nslabs = (N + pl.rows - 1) / pl.rows;
    pl.ctas = pl.nslabs < 2 * sms ? pl.nslabs : 2 * sms;
    pl.smem = 2 * (size_t)pl.rows * row + fixed;
    // several sequences walk the slabs on the tensor-core path, whose per-slab barriers and reduction cost more than
    // a library GEMM's tiles do (measured on B200: 31.5 MB x 4 sequences 12.4 us against 8.3 us); one sequence wins
    pl.worthwhile = pl.BP == 1 && (size_t)pl.rows * row * (pl.nslabs / pl.ctas) >= fixed;
    return pl.smem > optin ? SKV_E_TOO_LARGE : SKV_OK;
}

}  // namespace skv

using namespace skv;

extern "C" int skv_gemv_supported(int N, int K, int B, int mode) {
    GemvPlan pl;
    return plan_gemv(N, K, B, mode, pl) == SKV_OK && pl.worthwhile ? 1 : 0;
}

// Layout of an exchange buffer: data [2 slots][world][cap] of 8-byte {value, epoch} pairs, then the tick and the
// status word of the owning rank
static int64_t comm_data_bytes(int world, int cap) { return ((int64_t)2 * world * cap * 8 + 255) / 256 * 256; }

static int wait_polls(const skv_comm *c) {
    const int64_t k = c->wait_kpolls > 0 ? c->wait_kpolls : WAIT_KPOLLS_DEFAULT;
    return (int)(k * 1024 > 0x7fffffff ? 0x7fffffff : k * 1024);
}

static int check_comm(const skv_comm *c) {
    if (c->world < 1 || c->world > 8 || c->rank < 0 || c->rank >= c->world || c->cap_elems < 8 || c->cap_elems % 8)
        return SKV_E_RANGE;
    if (!c->tick || !c->status) return SKV_E_NULL;
    for (int r = 0; r < c->world; ++r)
        if (!c->data[r]) return SKV_E_NULL;
    return SKV_OK;
}

struct AttentionPartials {
    const float *part;
    int ncl, G;
    int32_t *cnt;
};

static int gemv_launch(const void *W, int N, int K, void *y, int B, int mode, const void *x, const void *h_in,
                       const void *delta, const void *norm_w, void *h_out, float eps, const skv_comm *in, int in_seq,
                       const skv_comm *out, int out_seq, void *stream, const AttentionPartials *att = nullptr) {
    if (!W || (!y && !out)) return SKV_E_NULL;
    if (mode < 0 || mode > 4 || (mode == 3) != (in != nullptr) || (mode == 4) != (att != nullptr)) return SKV_E_RANGE;
    if (mode == 4) {
        if (!att->part) return SKV_E_NULL;
        if (att->ncl < 1 || att->ncl > 8 || att->G < 1 || att->G > 16 || K % (128 * att->G)) return SKV_E_RANGE;
        if (!aligned16(att->part)) return SKV_E_ALIGN;
    } else if (mode == 1 || mode == 3 ? (!h_in || !norm_w) : !x) return SKV_E_NULL;
    if (B < 1 || B > 8 || N < 1 || K < 8 || K % 8) return SKV_E_RANGE;
    if (!aligned16(W) || (y && !aligned16(y)) || (x && !aligned16(x)) || (h_in && !aligned16(h_in)) ||
        (delta && !aligned16(delta)) || (norm_w && !aligned16(norm_w)) || (h_out && !aligned16(h_out)))
        return SKV_E_ALIGN;
    for (const skv_comm *c : {in, out}) {
        if (!c) continue;
        const int rc = check_comm(c);
        if (rc) return rc;
    }
    if ((in && (in_seq < 0 || in_seq > 254 || (int64_t)B * K > in->cap_elems)) ||
        (out && (out_seq < 0 || out_seq > 254 || (int64_t)B * N > out->cap_elems)))
        return SKV_E_RANGE;
    GemvPlan pl;
    const int rc = plan_gemv(N, K, B, mode == 4 ? 0 : mode, pl);
    if (rc) return rc;
    const int BP = pl.BP, rows = pl.rows;
    const bool tc = pl.tc;
    const size_t smem = pl.smem;
    GemvParams p = {};
    p.W = static_cast<const __nv_bfloat16 *>(W); p.y = static_cast<__nv_bfloat16 *>(y);
    p.N = N; p.K = K; p.B = B; p.mode = mode; p.rows_per_cta = rows; p.nslabs = pl.nslabs; p.stages = pl.stages;
    {
        // rows per warp and pass: two where that leaves the busiest warp no more rows than one at a time does (a single
        // sequence only).  Measured in the decode step at batch 1: pairs 727-731 tok/s, one row 714, groups of up to
        // four 720.
        int best = 1, best_rows = (rows + GEMV_WARPS - 1) / GEMV_WARPS;
        for (int g = 2; g <= 2 && BP == 1; ++g) {
            const int groups = (rows + g - 1) / g, most = (groups + GEMV_WARPS - 1) / GEMV_WARPS * g;
            if (most <= best_rows) { best = g; best_rows = most; }
        }
        p.row_group = best;
    }
    p.x = static_cast<const __nv_bfloat16 *>(x); p.h_in = static_cast<const __nv_bfloat16 *>(h_in);
    p.delta = static_cast<const __nv_bfloat16 *>(delta); p.g = static_cast<const __nv_bfloat16 *>(norm_w);
    p.h_out = static_cast<__nv_bfloat16 *>(h_out); p.eps = eps;
    if (att) { p.att_part = att->part; p.att_ncl = att->ncl; p.att_G = att->G; p.att_cnt = att->cnt; }
    if (out) {
        for (int r = 0; r < out->world; ++r) p.out_data[r] = static_cast<uint2 *>(out->data[r]);
        p.out_tick = out->tick;
        p.out_world = out->world; p.out_rank = out->rank; p.out_seq = out_seq; p.out_cap = out->cap_elems;
    }
    if (in) {
        p.in_data = static_cast<const uint2 *>(in->data[in->rank]); p.in_tick = in->tick;
        p.in_world = in->world; p.in_seq = in_seq; p.in_cap = in->cap_elems; p.status = in->status;
        p.wait_limit = wait_polls(in);
    }
    typedef void (*Kern)(const GemvParams);
    const int bi = (BP == 1 ? 0 : (BP == 2 ? 1 : (BP == 4 ? 2 : 3))) + (tc ? 4 : 0) + (pl.stages > 1 ? 8 : 0);
    const Kern table[16] = {
        gemv_kernel<1, false, false>, gemv_kernel<2, false, false>, gemv_kernel<4, false, false>, gemv_kernel<8, false, false>,
        gemv_kernel<1, true, false>,  gemv_kernel<2, true, false>,  gemv_kernel<4, true, false>,  gemv_kernel<8, true, false>,
        gemv_kernel<1, false, true>,  gemv_kernel<2, false, true>,  gemv_kernel<4, false, true>,  gemv_kernel<8, false, true>,
        gemv_kernel<1, true, true>,   gemv_kernel<2, true, true>,   gemv_kernel<4, true, true>,   gemv_kernel<8, true, true>};
    static size_t configured[64][16] = {};
    int dev = 0;
    SKV_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SKV_E_RANGE;
    if (configured[dev][bi] < smem) {
        SKV_CUDA_OK(cudaFuncSetAttribute(table[bi], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev][bi] = smem;
    }
    SKV_CUDA_OK(launch_pdl(table[bi], dim3(pl.ctas), dim3(GEMV_THREADS), smem, static_cast<cudaStream_t>(stream), p));
    return SKV_OK;
}

extern "C" int skv_gemv(const void *W, int N, int K, void *y, int B, int mode, const void *x, const void *h_in,
                        const void *delta, const void *norm_w, void *h_out, float eps, void *stream) {
    if (mode == 3 || mode == 4) return SKV_E_RANGE;
    return gemv_launch(W, N, K, y, B, mode, x, h_in, delta, norm_w, h_out, eps, nullptr, 0, nullptr, 0, stream);
}

extern "C" int skv_gemv_tp(const void *W, int N, int K, void *y, int B, int mode, const void *x, const void *h_in,
                           const void *norm_w, void *h_out, float eps, const skv_comm *in, int in_seq,
                           const skv_comm *out, int out_seq, void *stream) {
    if (mode == 4) return SKV_E_RANGE;
    return gemv_launch(W, N, K, y, B, mode, x, h_in, nullptr, norm_w, h_out, eps, in, in_seq, out, out_seq, stream);
}

extern "C" int skv_gemv_attended(const void *W, int N, int K, void *y, int B, const float *partials, int clusters, int G,
                                 int32_t *cnt, const skv_comm *out, int out_seq, void *stream) {
    const AttentionPartials att = {partials, clusters, G, cnt};
    return gemv_launch(W, N, K, y, B, 4, nullptr, nullptr, nullptr, nullptr, nullptr, 0.f, nullptr, 0, out, out_seq,
                       stream, &att);
}

extern "C" int64_t skv_comm_bytes(int world, int cap_elems) {
    if (world < 1 || world > 8 || cap_elems < 8 || cap_elems % 8) return SKV_E_RANGE;
    return comm_data_bytes(world, cap_elems) + 256;       // tick, status
}

extern "C" int skv_comm_view(skv_comm *c, void *const *bases, int world, int rank, int cap_elems) {
    if (!c || !bases) return SKV_E_NULL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || cap_elems < 8 || cap_elems % 8) return SKV_E_RANGE;
    const int64_t db = comm_data_bytes(world, cap_elems);
    *c = skv_comm{};
    c->world = world; c->rank = rank; c->cap_elems = cap_elems;
    for (int r = 0; r < world; ++r) {
        if (!bases[r]) return SKV_E_NULL;
        c->data[r] = bases[r];
    }
    char *own = static_cast<char *>(bases[rank]) + db;
    c->tick = reinterpret_cast<uint32_t *>(own);
    c->status = reinterpret_cast<int32_t *>(own + 64);
    return SKV_OK;
}

extern "C" int skv_comm_alloc(int64_t bytes, void **ptr) {
    if (!ptr) return SKV_E_NULL;
    if (bytes <= 0) return SKV_E_RANGE;
    SKV_CUDA_OK(cudaMalloc(ptr, (size_t)bytes));
    SKV_CUDA_OK(cudaMemset(*ptr, 0, (size_t)bytes));
    SKV_CUDA_OK(cudaDeviceSynchronize());
    return SKV_OK;
}
extern "C" int skv_comm_export(const void *ptr, void *handle64) {
    if (!ptr || !handle64) return SKV_E_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    SKV_CUDA_OK(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle64), const_cast<void *>(ptr)));
    return SKV_OK;
}
extern "C" int skv_comm_open(const void *handle64, void **ptr) {
    if (!ptr || !handle64) return SKV_E_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    SKV_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return SKV_OK;
}
extern "C" int skv_comm_close(void *ptr) {
    if (!ptr) return SKV_E_NULL;
    SKV_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return SKV_OK;
}
extern "C" int skv_comm_free(void *ptr) {
    if (!ptr) return SKV_E_NULL;
    SKV_CUDA_OK(cudaFree(ptr));
    return SKV_OK;
}

extern "C" int skv_comm_tick(const skv_comm *c, void *stream) {
    if (!c || !c->tick) return SKV_E_NULL;
    comm_tick_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(c->tick);
    SKV_CUDA_OK(cudaGetLastError());
    return SKV_OK;
}

extern "C" int skv_comm_reduce(const skv_comm *c, int seq, void *delta, int B, int N, void *stream) {
    if (!c || !delta) return SKV_E_NULL;
    const int rc = check_comm(c);
    if (rc) return rc;
    if (seq < 0 || seq > 254 || B < 1 || N < 8 || N % 8 || (int64_t)B * N > c->cap_elems) return SKV_E_RANGE;
    if (!aligned16(delta)) return SKV_E_ALIGN;
    const int total = B * N, blocks = (total + 255) / 256;          // eight lanes per run of eight elements
    const int cap_blocks = 2 * device_sm_count();
    SKV_CUDA_OK(launch_pdl(comm_reduce_kernel, dim3(blocks > cap_blocks ? cap_blocks : blocks), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), static_cast<const uint2 *>(c->data[c->rank]),
                           (const uint32_t *)c->tick, c->world, seq, c->cap_elems, c->status, wait_polls(c),
                           static_cast<__nv_bfloat16 *>(delta), total));
    return SKV_OK;
}

extern "C" int skv_comm_push(const skv_comm *c, int seq, const void *y, int B, int N, void *stream) {
    if (!c || !y) return SKV_E_NULL;
    const int rc = check_comm(c);
    if (rc) return rc;
    if (seq < 0 || seq > 254 || B < 1 || N < 8 || N % 8 || (int64_t)B * N > c->cap_elems) return SKV_E_RANGE;
    if (!aligned16(y)) return SKV_E_ALIGN;
    PushTargets out = {};
    for (int r = 0; r < c->world; ++r) out.data[r] = static_cast<uint2 *>(c->data[r]);
    const int total = B * N, blocks = (total / 8 + 255) / 256, cap_blocks = 2 * device_sm_count();
    SKV_CUDA_OK(launch_pdl(comm_push_kernel, dim3(blocks > cap_blocks ? cap_blocks : blocks), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16 *>(y), total, out,
                           (const uint32_t *)c->tick, c->world, c->rank, seq, c->cap_elems));
    return SKV_OK;
}

extern "C" int skv_comm_status(const skv_comm *c) {
    if (!c || !c->status) return SKV_E_NULL;
    int32_t word = 0;
    SKV_CUDA_OK(cudaMemcpy(&word, c->status, 4, cudaMemcpyDeviceToHost));
    return word & 0x7fffffff;
}
