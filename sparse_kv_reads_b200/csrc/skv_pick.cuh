// Top-budget selection over order-preserving keys, shared by the selection kernel and the one-launch decode step.
#pragma once

#include "skv_common.cuh"

namespace skv {

// Marks in sel[c] (c < n_c) the clusters taken in decreasing key (equal keys: lower slot first) until the member
// counts ci[] of the taken ones reach `need`; the cluster that crosses `need` is taken.  Never sorts: it finds the
// threshold key tau with  sum(count | key > tau) < need  and settles exact ties at tau in slot order.
//   key[c]   order-preserving integer keys of the shared scores (float_key), c < n_c
//   ci[c]    member counts (int, or float holding whole numbers); clusters with ci[c] <= 0 are never taken
//   sel      BITS false: one byte per cluster, zeroed by the caller for c < n_c
//   bits     BITS true: the selection as bit c % 32 of word c / 32 instead; every word that holds a slot < n_c is
//            written (the caller zeroes them when `active` is false)
//   hist     608 ints of shared scratch, 16-byte aligned; ired 40 ints
//   kmin, kmax, nvalid   this THREAD's partial range and count of the keys of clusters with members (the block
//            reduction happens here); `active` false: nothing is taken (the reductions and barriers still run).
//            READY true: they are the whole block's values already, and hist is zero on entry (no reduction, and
//            the first pass does not clear)
// Block-wide: every thread of the NT-thread CTA calls it; sel is complete (and synchronised) on return.
template <int NT, typename CT, bool BITS = false, bool READY = false>
__device__ __forceinline__ void pick_by_threshold(const uint32_t *key, const CT *ci, uint8_t *sel, int *hist,
                                                  int *ired, int n_c, int need, bool active, uint32_t kmin,
                                                  uint32_t kmax, int nvalid, uint32_t *bits = nullptr) {
    constexpr int NW = NT / 32;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid == 0) ired[1] = 0;                        // the candidates' counter (a barrier lies before its first use)
    if (!READY) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
            kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
            nvalid += __shfl_xor_sync(0xffffffffu, nvalid, o);
        }
        if (lane == 0) { ired[8 + wid] = (int)kmin; ired[16 + wid] = (int)kmax; ired[24 + wid] = nvalid; }
        __syncthreads();
    }
    if (active) {
        // ---- threshold: the smallest key t with sum(count | key > t) < need.  The keys still in question are
        // binned linearly over their range (256 bins, weighted by the clusters' counts); the bin in which the
        // running count passes `need` becomes the new range, until at most 32 candidates are left, which a
        // warp ranks against each other directly.  Scores crowd into a few octaves, so binning the range they
        // span (instead of the keys' top bytes) usually needs a single pass.  Every warp scans the histogram
        // for itself, and the candidates have words of their own, so the usual course costs three barriers and
        // two passes over the keys.
        if (!READY) {
            kmin = 0xffffffffu; kmax = 0u; nvalid = 0;
            for (int w = 0; w < NW; ++w) {
                kmin = min(kmin, (uint32_t)ired[8 + w]);
                kmax = max(kmax, (uint32_t)ired[16 + w]);
                nvalid += ired[24 + w];
            }
        }
        uint32_t lo = kmin, hi = kmax, tau = 0u;
        int above = 0, cand = nvalid;
        int *hw = hist, *hn = hist + 256, *cw = hist + 512, *cn = hist + 544, *cs = hist + 576;
        int pass = 0;
        for (; pass < 8 && cand > 32 && lo < hi; ++pass) {
            if (!READY || pass > 0) {
                if (pass > 0) __syncthreads();        // every warp has read the histogram before it is cleared
                for (int i = tid; i < 512; i += NT) hist[i] = 0;
                __syncthreads();
            }
            const int shift = max(0, 24 - __clz(hi - lo));            // (hi - lo) >> shift <= 255
            for (int c = tid; c < n_c; c += NT) {
                const uint32_t k = key[c];
                if (ci[c] > 0 && k >= lo && k <= hi) {
                    const int bin = (int)((k - lo) >> shift);
                    atomicAdd(&hw[bin], (int)ci[c]);
                    atomicAdd(&hn[bin], 1);
                }
            }
            __syncthreads();
            int loc[8], mine = 0;                     // lane owns bins [8*lane, 8*lane+8)
            {
                const int4 a = reinterpret_cast<const int4 *>(hw)[lane * 2], b = reinterpret_cast<const int4 *>(hw)[lane * 2 + 1];
                loc[0] = a.x; loc[1] = a.y; loc[2] = a.z; loc[3] = a.w; loc[4] = b.x; loc[5] = b.y; loc[6] = b.z; loc[7] = b.w;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) mine += loc[i];
            int suf = mine;                           // inclusive suffix over lanes >= lane
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_down_sync(0xffffffffu, suf, o);
                if (lane + o < 32) suf += t;
            }
            int run = suf - mine;                     // counts in bins above this lane's range
            int best = 256;                           // smallest bin b with above + count(bins > b) < need
#pragma unroll
            for (int i = 7; i >= 0; --i) {
                if (above + run < need) best = lane * 8 + i;
                run += loc[i];
            }
            best = min(__reduce_min_sync(0xffffffffu, best), 255);
            int gt = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) gt += (lane * 8 + i > best) ? loc[i] : 0;
            above += __reduce_add_sync(0xffffffffu, gt);
            cand = hn[best];
            const uint32_t nlo = lo + ((uint32_t)best << shift);
            const uint32_t span = (1u << shift) - 1u;
            hi = (hi - nlo > span) ? nlo + span : hi;
            lo = nlo;
        }
        if (nvalid > 0 && lo < hi) {
            // At most 32 candidates are left in [lo, hi].  Every cluster above that range is taken, none below it
            // is, and a candidate is taken while the members ranked before it - larger key, or the same key in a
            // lower slot - stay under `need` (the one that crosses it is taken).  One pass over the keys marks the
            // clusters above the range and lists the candidates; every warp ranks them for itself.
            if (READY && pass == 0) __syncthreads();  // the counter's reset, when no pass put a barrier after it
            if (BITS) {
                for (int base = wid * 32; base < n_c; base += NT) {   // a warp's 32 slots are one word
                    const int c = base + lane;
                    const uint32_t k = c < n_c ? key[c] : 0u;
                    const unsigned v = __ballot_sync(0xffffffffu, c < n_c && k > hi);
                    if (lane == 0) bits[base >> 5] = v;
                    if (c < n_c && k >= lo && k <= hi && ci[c] > 0) {
                        const int j = atomicAdd(&ired[1], 1);
                        if (j < 32) { cw[j] = (int)k; cn[j] = (int)ci[c]; cs[j] = c; }
                    }
                }
            } else {
                for (int c = tid; c < n_c; c += NT) {
                    const uint32_t k = key[c];
                    sel[c] = k > hi;
                    if (k >= lo && k <= hi && ci[c] > 0) {
                        const int j = atomicAdd(&ired[1], 1);
                        if (j < 32) { cw[j] = (int)k; cn[j] = (int)ci[c]; cs[j] = c; }
                    }
                }
            }
            __syncthreads();
            if (wid == 0) {
                const int m = min(ired[1], 32);
                const uint32_t kl = lane < m ? (uint32_t)cw[lane] : 0u;
                const int nl = lane < m ? cn[lane] : 0, sl = lane < m ? cs[lane] : 0;
                int before = 0;                       // members of the candidates ranked ahead of this lane's
                for (int j = 0; j < m; ++j) {
                    const uint32_t kj = __shfl_sync(0xffffffffu, kl, j);
                    const int nj = __shfl_sync(0xffffffffu, nl, j), sj = __shfl_sync(0xffffffffu, sl, j);
                    before += (kj > kl || (kj == kl && sj < sl)) ? nj : 0;
                }
                if (lane < m && above + before < need) {
                    if (BITS) atomicOr(&bits[sl >> 5], 1u << (sl & 31));
                    else sel[sl] = 1;
                }
            }
        } else {
            // one key value left, possibly shared by many clusters (or no cluster has members: everything is marked)
            if (nvalid > 0) tau = lo;
            int ties = 0;
            if (BITS) {
                for (int base = wid * 32; base < n_c; base += NT) {
                    const int c = base + lane;
                    const uint32_t k = c < n_c ? key[c] : 0u;
                    const unsigned v = __ballot_sync(0xffffffffu, c < n_c && k >= tau);
                    if (lane == 0) bits[base >> 5] = v;
                    ties += (c < n_c && k == tau);
                }
            } else {
                for (int c = tid; c < n_c; c += NT) {
                    const uint32_t k = key[c];
                    sel[c] = k >= tau;                // a lone cluster at the threshold is taken: above < need
                    ties += (k == tau);
                }
            }
            ties = __reduce_add_sync(0xffffffffu, ties);
            if (lane == 0) ired[32 + wid] = ties;
            __syncthreads();
            int t = 0;
            for (int w = 0; w < NW; ++w) t += ired[32 + w];
            if (t > 1 && wid == 0) {
                // several clusters share the threshold key: slot order, each taken while the keys ranked before
                // it stay under need
                int running = above;
                for (int base = 0; base < n_c; base += 32) {
                    const int c = base + lane;
                    const bool tie = c < n_c && key[c] == tau;
                    if (!__any_sync(0xffffffffu, tie)) continue;
                    const int mine = tie ? (int)ci[c] : 0;
                    int inc = mine;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int u = __shfl_up_sync(0xffffffffu, inc, o);
                        if (lane >= o) inc += u;
                    }
                    const bool keep = (running + inc - mine) < need;
                    if (BITS) {
                        const unsigned drop = __ballot_sync(0xffffffffu, tie && !keep);
                        if (lane == 0 && drop) bits[base >> 5] &= ~drop;
                    } else if (tie) {
                        sel[c] = keep;
                    }
                    running += __shfl_sync(0xffffffffu, inc, 31);
                }
            }
        }
        __syncthreads();
    }
}

}  // namespace skv
