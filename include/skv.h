/* skv.h - C ABI of the B200 (sm_100a) clustered sparse KV-cache decode-attention library.
 *
 * Every entry point takes raw device pointers, element strides and sizes; none takes a framework
 * type.  Unless stated otherwise a call allocates nothing, never synchronises and reads nothing back
 * to the host, so it can be recorded into a CUDA graph; all work is ordered on the `stream` argument
 * (a cudaStream_t passed as void*).
 * Lengths live in device memory.  `n_dev` holds the number of cached positions; `n_group` says how heads map to its
 * entries: head h reads n_dev[h / n_group], so a batch whose sequences differ in length passes one entry per sequence
 * and n_group = KV heads per sequence; n_group = 0 means every head reads n_dev[0] (all sequences equally long, the
 * reference's own limit: README.md:62).
 * Return value: 0 on success, a negative SKV_E_* code when an
 * argument is rejected on the host (nothing is launched then).  Problems met on the device (no spare
 * slot, a cluster too large to split, an index out of range) are recorded per head in the
 * caller-owned `status` words of skv_state and never fault.
 *
 * Each declaration names the interface of the reference project (aaholmes/sparse-kv-reads, package
 * `ssa`) that it replaces, as file:line within that project.
 */
#ifndef SKV_H
#define SKV_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKV_VERSION 101

/* host-side argument errors */
#define SKV_OK            0
#define SKV_E_NULL       -1   /* a required pointer is null */
#define SKV_E_DIM        -2   /* head_dim, group size or slot count not supported */
#define SKV_E_DTYPE      -3   /* unknown element type */
#define SKV_E_ALIGN      -4   /* pointer or stride not 16-byte aligned */
#define SKV_E_RANGE      -5   /* size or option out of range */
#define SKV_E_WORKSPACE  -6   /* workspace too small */
#define SKV_E_CUDA       -7   /* a CUDA runtime call failed (see skv_last_cuda_error) */
#define SKV_E_TOO_LARGE  -8   /* beyond the fixed capacity of a no-allocation entry point */

/* element types of q / K / V / out */
#define SKV_BF16 0
#define SKV_F32  1

/* bits of skv_state.flags (the reference's: ssa/kernels/sphere_fused.py:226-227) */
#define SKV_FLAG_DRIFT 1      /* the running key mean moved more than delta * rbar from mu_ref */
#define SKV_FLAG_RESET 2      /* the cluster count reached reset_at */
/* bits of skv_state.status (device-side problems; sticky until the host clears them) */
#define SKV_ST_NO_SLOT      1 /* a cluster passed its cap but every slot is in use */
#define SKV_ST_SPLIT_TOO_BIG 2 /* a cluster over the cap has more members than the split can stage */
#define SKV_ST_BAD_INDEX    4 /* a listed position or a label was out of range and was skipped */
#define SKV_ST_WAIT_TIMEOUT 8 /* a bounded wait for another GPU's partial sums gave up (skv_comm.status) */

/* Cluster state of `heads` independent (layer, sequence, KV head) entries, structure of arrays.
 * Arrays are contiguous over heads: x[head][...].  Mirrors the tensors of
 * ssa/attn/sphere_gpu.py:145-164 plus ssa/kernels/sphere_fused.py:363-378 and
 * ssa/kernels/graph_kernels.py:204-216 (end_dev, need_dev). */
typedef struct skv_state {
    int32_t heads;        /* entries in this view */
    int32_t C;            /* slots per head (power of two >= 16) */
    int32_t d;            /* head dimension (128) */
    int32_t capacity;     /* positions per head in `labels` */
    int32_t summary_bits; /* 8: score/search the int8 copies; 32: the float32 vectors */
    int32_t reserved;
    float   *sum_dir;     /* [heads, C, d]  sum of member unit directions */
    float   *cent;        /* [heads, C, d]  unit centroids searched by the insert */
    int8_t  *dir8;        /* [heads, C, d]  round(unit(sum_dir) * 127); null when summary_bits == 32 */
    int8_t  *cent8;       /* [heads, C, d]  round(cent * 127);          null when summary_bits == 32 */
    float   *mmax;        /* [heads, C]     longest member key (about mu_ref) */
    float   *mmin;        /* [heads, C]     shortest member key, +inf when empty */
    float   *count;       /* [heads, C]     member count */
    int32_t *n_c;         /* [heads]        slots in use */
    float   *cap;         /* [heads]        split a cluster holding more keys than this (+inf: never) */
    float   *vthr;        /* [heads]        ... or whose directions spread more than this (+inf: never) */
    float   *rbar;        /* [heads]        rms key length at the last (re)build */
    float   *ksum;        /* [heads, d]     running sum of clustered keys */
    float   *mu_ref;      /* [heads, d]     reference mean the keys are centred with */
    int32_t *flags;       /* [heads]        SKV_FLAG_* */
    int32_t *status;      /* [heads]        SKV_ST_* */
    int32_t *nsplit;      /* [heads]        splits done on the device */
    int32_t *end;         /* [heads]        clustered positions are [1, end) */
    int32_t *need;        /* [heads]        keys the selection must cover: ceil(budget * (end - 1)) */
    int16_t *labels;      /* [heads, capacity]  slot of each position; C = always read */
} skv_state;

int skv_version(void);
const char *skv_error_string(int code);
/* last cudaError_t seen by a call that returned SKV_E_CUDA, as text */
const char *skv_last_cuda_error(void);

/* Number of split partials skv_attend uses for `heads` KV heads on the current device
 * (replaces the split count of ssa/kernels/graph_kernels.py:218). */
int skv_attend_splits(int heads);

/* Bytes of the float workspace skv_attend needs for (heads, G, d, splits):
 * partial outputs, partial (max, sum) pairs and one ticket word per head. */
int64_t skv_attend_workspace_bytes(int heads, int G, int d, int splits);

/* Exact softmax attention of one query per query head over a LIST of cached rows, split over
 * CTAs, merged by log-sum-exp by the last CTA of each head.
 * Replaces _list_kernel + _merge_kernel (ssa/kernels/labeled_attn.py:202-245, :123-140); with
 * idx == NULL it attends over rows [0, n_dev[0]) and replaces _dense_dev_kernel
 * (ssa/kernels/graph_kernels.py:27-59).
 *   q    [heads*G, d]            one query per query head, contiguous, dtype
 *   K, V [heads, rows, d]        read in place: element strides *_head_stride, *_row_stride, unit last stride
 *   idx  [heads, idx_stride]     int32 row positions (any order); cnt [heads] rows listed per head
 *   out  [heads*G, d]            dtype
 *   workspace                    skv_attend_workspace_bytes(...) bytes, zero-initialised ONCE by the
 *                                caller (the ticket words return to zero after every call)
 *   rows_limit                   positions >= rows_limit are skipped and flagged in status (may be null)
 */
int skv_attend(const void *q, const void *K, const void *V, const int32_t *idx, const int32_t *cnt,
               const int32_t *n_dev, int n_group, void *out, void *workspace, int32_t *status,
               int heads, int G, int d, int dtype,
               int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride, int64_t v_row_stride,
               int64_t idx_stride, int rows_limit, int splits, float scale, void *stream);

/* Attention over the cached rows [0, n_dev[0]) with a WEIGHT per cluster: a row whose label is l enters the
 * softmax with weight w[l] (log w[l] is added to its score); rows of weight 0 are not read.  With 0/1 weights this
 * is skv_attend over the selected rows; fractional weights carry the clusters drawn among the ones the selection
 * left out (ssa/attn/tail_sample.py:35-63), each weighted draws / (S x probability).  Replaces the label-weighted
 * attention of attend_sampled (ssa/kernels/sphere_fused.py:503-518; spec ssa/attn/labeled.py:24-44).
 *   labels [heads, label_stride] int16, w [heads, C+1] float32 (column C = the always-read rows); G <= 8;
 *   q, K, V, out, workspace, splits as in skv_attend (float32 arithmetic on the CUDA cores: an eager-API call). */
int skv_attend_weighted(const void *q, const void *K, const void *V, const int16_t *labels, int64_t label_stride,
                        const float *w, int C, const int32_t *n_dev, int n_group, void *out, void *workspace,
                        int32_t *status,
                        int heads, int G, int d, int dtype,
                        int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride, int64_t v_row_stride,
                        int splits, float scale, void *stream);

/* Fixed capacity, in bytes, of the scratch array behind skv_attend_static. */
#define SKV_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)

/* skv_attend for callers that cannot allocate device memory.  No counterpart in the reference (its
 * Python side always allocates through the framework); it exists for hosts that hand the library
 * only the buffers they were given: a serving process that reserved all of HBM for its KV-cache
 * pool at start-up and has no headroom left for a workspace, a latency-critical decode loop that
 * must not pay the device-wide stall of a cudaMalloc, or a foreign-function caller (cgo, JNI) with
 * no CUDA allocator of its own.
 * Same arguments and result as skv_attend, minus the workspace: the split partials and ticket words
 * live in a SKV_STATIC_SCRATCH_BYTES array inside the library (held by every GPU that loads the
 * library, until exit).  Returns SKV_E_TOO_LARGE when skv_attend_workspace_bytes(heads, G, d, splits)
 * exceeds that; lower `splits` or use skv_attend.  The call itself allocates nothing.
 * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with that
 * device current); make that first call before any stream capture.
 * All calls share the one array: two calls whose kernels overlap on the GPU (different streams, or
 * several host threads) race on it and give wrong results - serialise them. */
int skv_attend_static(const void *q, const void *K, const void *V, const int32_t *idx, const int32_t *cnt,
                      const int32_t *n_dev, int n_group, void *out, int32_t *status,
                      int heads, int G, int d, int dtype,
                      int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride, int64_t v_row_stride,
                      int64_t idx_stride, int rows_limit, int splits, float scale, void *stream);

/* Log-sum-exp merge of caller-provided partials (natural-log maxima), float32 output.
 * Replaces merge_splits (ssa/kernels/labeled_attn.py:143-151).
 *   m, l [heads, S, G], a [heads, S, G, d] -> out [heads*G, d] */
int skv_merge(const float *m, const float *l, const float *a, float *out, int heads, int S, int G, int d,
              void *stream);

/* QK-RMSNorm + rotary embedding + KV-cache write of the new token, folded into skv_select (optional): the selection
 * needs the rotated queries first of all, so its CTAs compute them from the raw q/k/v product themselves instead of
 * waiting for a separate launch (skv_qk_rope_cache, which this replaces on that path; same arithmetic and
 * roundings).  Every scoring CTA rotates the G query heads of its KV head for its own use; the first CTA of each
 * (sequence, KV head) also stores them to q_out (for the attention launch) and writes the new K and V rows. */
typedef struct skv_rope {
    const void *qkv;                 /* [B, (H + 2 H_kv) * 128] bf16: q heads, then k heads, then v heads */
    const void *q_norm_w, *k_norm_w; /* [128] bf16 */
    const void *cos_table, *sin_table; /* [positions, 128] bf16 */
    const int64_t *pos;              /* device: position of the new token, [1] or one per sequence (pos_per_seq) */
    void *q_out;                     /* [B * H, 128] bf16 */
    void *k_cache, *v_cache;         /* bf16 caches of this layer */
    int32_t H, H_kv;                 /* query and KV heads per sequence (state.heads = B * H_kv) */
    int64_t cache_batch_stride, cache_head_stride, cache_row_stride;   /* elements */
    float eps;
    int32_t pos_per_seq;             /* 0: every sequence writes at pos[0]; 1: sequence s at pos[s] */
} skv_rope;

/* How the G query heads of a KV head share one ranking of its clusters (ssa/attn/sphere_gpu.py:431-439) */
#define SKV_GROUP_SUM_SHARE 0   /* sum over the heads of each head's softmax over clusters */
#define SKV_GROUP_MAX       1   /* largest scaled score of any head */
#define SKV_GROUP_MAX_REL   2   /* largest score relative to that head's best cluster */

/* Score clusters from their summaries once per KV head for its G query heads, form the shared score
 * (`group`: SKV_GROUP_*) and take clusters in decreasing shared
 * score (equal scores: lower slot first) until their key counts reach state.need.  Several CTAs score
 * a head's clusters in parallel; the last one to finish picks.  Outputs the 0/1 weights, the same
 * selection as a bit set (bit C = always-read rows: position 0 and the recent window carry label C),
 * and - only when `idx` is given - the list of positions to read in ascending order.
 * Replaces _score_kernel, _shared_pick/_pick_dev_kernel (ssa/kernels/sphere_fused.py:230-289,
 * ssa/kernels/graph_kernels.py:133-141) and _compact_dev_kernel (graph_kernels.py:144-155);
 * selection rule of SphereIndexGPU._rank_mask (ssa/attn/sphere_gpu.py:402-410).
 *   q          [heads*G, d] dtype
 *   n_dev      cached positions, n_group as described at the top of this file
 *   w          [heads, C+1] float32 0/1 weights out (column C = 1)
 *   selbits    [heads, C/32+1] uint32 out, or null (kept in the workspace then)
 *   idx, cnt   idx [heads, idx_stride] int32 or null; cnt [heads]: rows listed, or 0 when idx is null
 *              (skv_attend_labels then adds the rows it reads)
 *   shared_in  optional [heads, C] float32: use these shared scores instead of scoring (tests)
 *   shared_out optional [heads, C] float32: the shared scores used
 *   e_out      optional [heads, G, C] float32: per-query-head cluster scores (before the 1/sqrt(d) scale)
 *   workspace  skv_select_workspace_bytes(heads, G, C) bytes, zero-initialised once by the caller
 *   group      SKV_GROUP_* (shared_in, when given, is ranked as it is)
 *   rope       optional: compute the queries from the raw projection first (see skv_rope); q is then unused,
 *              bf16 only, G = rope->H / rope->H_kv
 */
int64_t skv_select_workspace_bytes(int heads, int G, int C);
int skv_select(const skv_state *st, const void *q, int dtype, int G, const int32_t *n_dev, int n_group,
               float *w, uint32_t *selbits, int32_t *idx, int64_t idx_stride, int32_t *cnt,
               const float *shared_in, float *shared_out, float *e_out, void *workspace, float scale, int group,
               const skv_rope *rope, void *stream);

/* Tuning aid without a counterpart in the reference: `dev_ptr` is a device array of 16 uint64 that receives
 * nanosecond time stamps of the phases of skv_select's kernel for head 0 (null switches it off). */
void skv_debug_select_probe(void *dev_ptr);
/* Overlap of consecutive launches (programmatic dependent launch).  When on, skv_qk_rope_cache, skv_select and
 * skv_attend_labels may be scheduled before the kernel ahead of them on the stream has ended; they load what no
 * kernel of the same decode step writes (cluster summaries, labels) and then wait for that kernel.  The caller
 * turns it on only where this holds: the cluster state (skv_insert, skv_fit, skv_rebin) must not be written by
 * the launch directly ahead of skv_select or skv_attend_labels.  Off by default; SKV_PDL=0 in the environment
 * keeps it off.  Process-wide switch, read at launch time. */
void skv_set_overlap(int on);
/* Same for skv_attend_labels: device uint64 [CTAs][8] phase stamps of every CTA (null = off).  Takes effect only
 * in a library built with -DSKV_ATTEND_PROBE (the stamps cost that kernel 3.5 % at large batch). */
void skv_debug_attend_probe(void *dev_ptr);

/* skv_attend without a row list: every CTA owns a range of positions, reads their int16 labels, keeps
 * the positions whose label's bit is set in `selbits` (from skv_select) and attends over them; `cnt`
 * (zeroed by skv_select) receives the rows read per head.  bf16 caches only.  Replaces
 * _compact_dev_kernel + _list_kernel + _merge_kernel (ssa/kernels/graph_kernels.py:144-155,
 * ssa/kernels/labeled_attn.py:202-245, :123-140) in one launch.  label_stride a multiple of 8. */
int skv_attend_labels(const void *q, const void *K, const void *V, const int16_t *labels, int64_t label_stride,
                      const uint32_t *selbits, int C, const int32_t *n_dev, int n_group, void *out, void *workspace,
                      int32_t *cnt, int32_t *status, int heads, int G, int d, int dtype,
                      int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride, int64_t v_row_stride,
                      int splits, float scale, void *stream);

/* Selection and attention of one decode step in ONE launch, for launches with few heads (8 to about 36 on a
 * B200), where two launches and their hand-offs through global memory cost more than the bytes they move.
 * A head is served by `clusters` thread-block clusters of 8 CTAs: each CTA scores an eighth of the head's
 * clusters and shares the scores with its cluster through distributed shared memory, every CTA then derives
 * the selection for itself (the shared score and threshold rule of skv_select, group SKV_GROUP_SUM_SHARE),
 * attends over its range of positions (rows straight from the labels, as skv_attend_labels) and the cluster's
 * first CTA merges its 8 partials; only one partial per cluster passes through the workspace.
 * Replaces SphereIndexGraph.step's launches after the insert - _score_kernel, _pick_dev_kernel,
 * _compact_dev_kernel, _list_kernel, _merge_kernel (ssa/kernels/graph_kernels.py:229-244) - for bf16 caches,
 * 8-bit summaries, G <= 8, 64 <= C <= 2048.
 *   skv_step_clusters        clusters per head to launch with on the current device (1..8), or 0 when this
 *                            shape is better served by skv_select + skv_attend_labels (many heads, other modes)
 *   skv_step_workspace_bytes bytes of `workspace` (zero-initialised once by the caller)
 *   q          [heads*G, d] bf16, or null with `rope` (the queries are then computed from the raw projection
 *              as in skv_select; the CTA that reads the new token's position writes its K and V rows)
 *   w, selbits optional outputs as in skv_select;  cnt [heads] receives the rows read per head
 *   out        [heads*G, d] bf16; or null: the last merge is left to the consumer - the workspace then holds, per
 *              head, `clusters` partials [heads, clusters, G, 132] of float32 (128 weighted sums, their running
 *              maximum in base-2 units, the sum of weights, the rows read) and cnt is not written; skv_gemv_attended
 *              (the output product) merges them while it builds its input, which saves a hand-off through a ticket */
int skv_step_clusters(int heads, int G, int C, int summary_bits);
int64_t skv_step_workspace_bytes(int heads, int G, int clusters);
int skv_step(const skv_state *st, const void *q, int G, const int32_t *n_dev, int n_group, const void *K, const void *V,
             int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride, int64_t v_row_stride,
             float *w, uint32_t *selbits, int32_t *cnt, void *out, void *workspace, int clusters,
             float scale, const skv_rope *rope, void *stream);
/* Tuning aid: device uint64 [CTAs][8] phase stamps of skv_step's kernel (builds with -DSKV_STEP_PROBE only). */
void skv_debug_step_probe(void *dev_ptr);

/* Insert the keys that left the recent window since the last call (positions [end, max(1, n-window)))
 * into their nearest clusters, one CTA per entry of `st` (all layers of a model in one launch),
 * splitting a cluster in two inside the kernel when it passes its head's cap; then update end, need,
 * the drift flag and the status word.
 * Replaces _bin_kernel/_bin_dev_kernel + _split_cluster (ssa/kernels/sphere_fused.py:48-227,
 * ssa/kernels/graph_kernels.py:62-130) and AllLayerInsert (graph_kernels.py:286-325); split rule of
 * _bisect_padded (ssa/attn/sphere_gpu.py:76-102).
 *   k_layers        device array [heads / heads_per_layer] of K base addresses (one cache tensor per layer)
 *   heads_per_layer entries of st per cache tensor; entry e reads head (e % heads_per_layer) of layer (e / heads_per_layer)
 *   budget          fraction of the clustered keys to cover (need = ceil(budget * (end-1)), in double)
 *   delta           drift threshold in units of rbar;  reset_at: 0 = never
 *   max_members     largest cluster the in-kernel split stages (<= skv_insert_max_members())
 *   capk            cap per clustered key when the cap grows with the context (a cluster splits above
 *                   max(cap, capk * clustered keys)); 0 = fixed cap
 *   var_min         fewest keys a cluster must hold to split on the spread threshold state.vthr
 */
int skv_insert(const skv_state *st, const void *const *k_layers, int heads_per_layer, int dtype,
               int64_t k_head_stride, int64_t k_row_stride, const int32_t *n_dev, int n_group, int window,
               double budget, float delta, int reset_at, int max_members, float capk, int var_min, void *stream);
int skv_insert_max_members(void);

/* The nearest-centroid passes of skv_fit / skv_rebin are float32 FMA chains on the CUDA cores (42 TFLOP/s on B200).
 * skv_fit_tensor_cores(1) runs them on the tensor cores instead: three TF32 products of a two-term split with
 * float32 accumulation, and every key whose two best centroids are closer than that value can tell apart is
 * recomputed with the float32 chain, so the labels are the same bit for bit (tests compare the two).  Measured equal
 * in speed (0.188 s against 0.184 s for a 32k prompt x 28 layers), hence off by default; process-wide switch. */
void skv_fit_tensor_cores(int on);

/* Workspace bytes of skv_fit / skv_rebin for `heads` heads of `m` clustered keys. */
int64_t skv_fit_workspace_bytes(int heads, int m, int C, int d);

/* Prompt fit of `st` from positions [1, end) of K, end = max(1, n - window): mean, centring, cosine
 * k-means with C_init centroids started from rows init_pos (device int32 [C_init], positions within
 * the clustered keys) and `iters` Lloyd steps, summaries, cap, then division of every cluster over
 * the cap (k-means over its members into ceil(count*split_factor/cap) parts, then two-way splits
 * until none is over the cap or the slots run out), and the 8-bit copies.
 * Synchronises the stream between split rounds; not for graph capture.
 * Replaces spherical_kmeans (ssa/attn/clusterkv.py:27-46), SphereIndexGPU._build/_bin
 * (ssa/attn/sphere_gpu.py:166-219), _split_after_fit/_split_overflow/_split_batch (:302-391) and
 * _refresh8 (ssa/kernels/sphere_fused.py:398-406).
 *   init_pos    device int32 [C_init]: clustered-key indices whose directions start the k-means; null: keep the
 *               centroids the caller put into state.cent[:, :C_init] and fit nothing (`partition="random"`:
 *               fixed directions shared by all heads, ssa/attn/sphere_gpu.py:13-14,:147)
 *   cap_keys > 0: absolute cap; else cap = split_factor * m / C_init when split_factor > 0; else no cap
 *   capk        growing cap (see skv_insert); var_factor > 0: state.vthr = var_factor x the mean spread of the
 *               fitted clusters (ssa/attn/sphere_gpu.py:214-217), else +inf
 *   k_layers    optional device table of cache base pointers, one per heads_per_layer consecutive heads of st (K is
 *               unused then): the states of several layers, stacked, are fitted in one call - one set of launches
 *               and one host round trip per split round for the whole model instead of one per layer
 *   head_list   optional device int32 [n_list]: fit only these entries of st (a head that reached reset_at,
 *               SphereIndexGPU._reset_heads, sphere_gpu.py:283-293); null = all heads.  Workspace for n_list heads.
 */
int skv_fit(const skv_state *st, const void *K, int dtype, int64_t k_head_stride, int64_t k_row_stride,
            int n, int window, int C_init, int iters, const int32_t *init_pos, float cap_keys,
            float split_factor, float capk, float var_factor, const int32_t *head_list, int n_list,
            const void *const *k_layers, int heads_per_layer, void *workspace, int64_t workspace_bytes,
            void *stream);

/* Recentre and rebin selected heads with their centroids kept (new mean = ksum / (end-1)):
 * replaces the recentring branch of SphereIndexGPU._build (ssa/attn/sphere_gpu.py:187-219 with mu given;
 * callers ssa/kernels/sphere_fused.py:453-464).  `head_list` device int32 [n_list] entries of st;
 * `end`: clustered positions are [1, end) (the host's copy of state.end).  Workspace as for a fit of n_list heads.
 * split_factor > 0: clusters the rebinning left over their cap are then divided two ways at a time (iters, capk as
 * in skv_fit) - what the reference's PyTorch path does when such a cluster next receives a key; its kernels, and
 * skv_insert, cannot stage a cluster much larger than the cap, so without this it would stay oversized.
 * split_factor = 0: rebin only. */
int skv_rebin(const skv_state *st, const int32_t *head_list, int n_list, int end, const void *K, int dtype,
              int64_t k_head_stride, int64_t k_row_stride, float split_factor, int iters, float capk,
              void *workspace, int64_t workspace_bytes, void *stream);

/* ---- single-token forward around the attention (bf16) ------------------------------------------------
 * The decode graph of the reference runs the engine's modules one framework op at a time
 * (ssa/models/graph_decode.py:98-117: norm1, q/k/v, q_norm, k_norm, apply_rope, index_copy_, o, norm2, ffn).
 * These three launches replace the element-wise ops among them; the matrix products stay library GEMVs. */

/* h [B, hidden] += delta (delta may be null), stored in bf16; out = RMSNorm(h) * w.  Replaces the residual
 * add and layer.norm1 / layer.norm2 / final_norm (graph_decode.py:100,116-118). */
int skv_add_rmsnorm(void *h, const void *delta, const void *w, void *out, int B, int hidden, float eps, void *stream);

/* qkv [B, (H + 2*H_kv) * d] (query heads, then key heads, then value heads) -> q_out [B*H, d] with the per-head
 * RMSNorm and the rotary embedding applied, and the new key (normed, rotated) and value written into the caches
 * [B, H_kv, L, d] at row pos_dev[0] (pos_per_seq = 0) or pos_dev[sequence] (1).  cos/sin tables [positions, d] bf16.  Replaces q_norm, k_norm, apply_rope
 * and the two index_copy_ calls (graph_decode.py:101-108). */
int skv_qk_rope_cache(const void *qkv, const void *q_norm_w, const void *k_norm_w, const void *cos_table,
                      const void *sin_table, const int64_t *pos_dev, int pos_per_seq, void *q_out, void *k_cache,
                      void *v_cache,
                      int B, int H, int H_kv, int d, int64_t cache_batch_stride, int64_t cache_head_stride,
                      int64_t cache_row_stride, float eps, void *stream);

/* gate_up [B, 2*inter] (gate columns first) -> out [B, inter] = silu(gate) * up: the element-wise middle of
 * layer.ffn (graph_decode.py:117). */
int skv_silu_mul(const void *gate_up, void *out, int B, int inter, void *stream);

/* y[B, N] = x[B, K] . W[N, K]^T for B <= 8 sequences (bf16, float32 accumulation): the projections of a decode
 * step (the reference runs them as the engine's nn.Linear modules, models/graph_decode.py:100-121).  The input
 * is built inside the kernel:
 *   mode 0  x [B, K] as given;
 *   mode 1  h_out = h_in + delta (delta may be null), x = RMSNorm(h_out) * norm_w: the residual add and norm of
 *           skv_add_rmsnorm, out of place (h_out must not alias h_in; h_out may be null);
 *   mode 2  x = silu(gate) * up from x = gate_up [B, 2K], as skv_silu_mul.
 * W row-major [N, K], K a multiple of 8 and at most 49,152; all pointers 16-byte aligned.  Takes part in
 * skv_set_overlap: the weights are requested before the wait for the launch ahead. */
int skv_gemv(const void *W, int N, int K, void *y, int B, int mode, const void *x, const void *h_in,
             const void *delta, const void *norm_w, void *h_out, float eps, void *stream);
/* ---- sum of row-parallel products over the GPUs of a tensor-parallel group, through peer memory ----------------
 * Replaces the all-reduce after the row-parallel `o` and `down` products of a tensor-parallel decode step (the
 * reference decodes on one GPU; its host model's layers are models/graph_decode.py:100-121).  Every GPU of the
 * group owns one exchange buffer, mapped into the other processes (skv_comm_alloc / export / open):
 *   data   [2 slots][world][cap_elems] of 8-byte pairs {float32 bits, epoch}
 *   tick   uint32, advanced once per decode step on every GPU (skv_comm_tick)
 * The producing product (skv_gemv_tp with `out` set) stores each of its float32 sums, paired with the epoch
 * tick x 256 + seq + 1, into slot seq % 2 / row `rank` of EVERY GPU's buffer with one aligned 8-byte store over
 * NVLink: no fence and no flag, a reader that finds the epoch has the value.  The consuming product (mode 3)
 * polls the `world` partials of each input element until they carry the epoch - a bounded wait (wait_kpolls, about
 * five seconds by default), after which it sets SKV_ST_WAIT_TIMEOUT in *status and carries on - and adds them in rank order, so
 * every GPU obtains the same bits.  `seq` numbers the exchanges of a step (0..254), the same on every GPU; two
 * slots are enough for a decoder layer (`o`, `down` alternate): a slot's next producer cannot start anywhere
 * before every GPU has consumed the other slot, which each does after its use of this one. */
typedef struct skv_comm {
    int32_t world, rank;
    int32_t cap_elems;        /* pairs per (slot, source rank); a multiple of 8 */
    int32_t wait_kpolls;      /* polls (x 1024, a little under a microsecond each) before a wait gives up; 0 = 8192 */
    void     *data[8];        /* every rank's buffer, as mapped in this process */
    uint32_t *tick;           /* local */
    int32_t  *status;         /* local, one word */
} skv_comm;
/* Bytes of one exchange buffer (data, then tick and status of the owner). */
int64_t skv_comm_bytes(int world, int cap_elems);
/* cudaMalloc + zero fill of an exchange buffer on the current device; 64-byte handle for the other processes
 * (cudaIpcGetMemHandle); mapping of another process's buffer (cudaIpcOpenMemHandle); unmapping; release. */
int skv_comm_alloc(int64_t bytes, void **ptr);
int skv_comm_export(const void *ptr, void *handle64);
int skv_comm_open(const void *handle64, void **ptr);
int skv_comm_close(void *ptr);
int skv_comm_free(void *ptr);
/* Fills `c` for buffers `bases[0..world)` (bases[rank] is the local one). */
int skv_comm_view(skv_comm *c, void *const *bases, int world, int rank, int cap_elems);
/* Advances the local tick (one tiny launch): once per decode step, on every GPU, ahead of the step's exchanges. */
int skv_comm_tick(const skv_comm *c, void *stream);
/* skv_gemv with the exchange: `out` non-null -> the sums go to every GPU's buffer as exchange `out_seq` instead of
 * y; mode 3 -> as mode 1 with delta = the sum over ranks of exchange `in_seq` of `in` (no delta argument). */
int skv_gemv_tp(const void *W, int N, int K, void *y, int B, int mode, const void *x, const void *h_in,
                const void *norm_w, void *h_out, float eps, const skv_comm *in, int in_seq,
                const skv_comm *out, int out_seq, void *stream);
/* The write side for producers other than skv_gemv (a library GEMM at batches beyond 8): this rank's partial sums
 * y[B, N] (bf16) go into its place in every GPU's buffer as exchange `seq`; skv_comm_reduce on every GPU then gives
 * the sum, the same bits everywhere.  The pair stands where a tensor-parallel host would call an all-reduce (the
 * reference decodes on one GPU). */
int skv_comm_push(const skv_comm *c, int seq, const void *y, int B, int N, void *stream);
/* delta[B, N] (bf16) = sum over ranks of exchange `seq`, after the same wait: for consumers other than skv_gemv. */
int skv_comm_reduce(const skv_comm *c, int seq, void *delta, int B, int N, void *stream);
/* The buffer's status word (SKV_ST_WAIT_TIMEOUT), read back with a synchronising copy; negative on error. */
int skv_comm_status(const skv_comm *c);

/* y[B, N] = attention output . W^T straight from the partials skv_step left with out == null: every CTA of the product
 * merges the `clusters` partials of each query head (log-sum-exp) into its input row; CTA 0 also writes the rows read
 * per head to `cnt` (may be null).  K = query heads per sequence x 128; partials [B * K / (128 G), clusters, G, 132].
 * `out`/`out_seq` as in skv_gemv_tp (null: plain output to y).  Replaces _merge_kernel + the engine's o projection
 * (ssa/kernels/labeled_attn.py:123-140, ssa/models/graph_decode.py:113-115). */
int skv_gemv_attended(const void *W, int N, int K, void *y, int B, const float *partials, int clusters, int G,
                      int32_t *cnt, const skv_comm *out, int out_seq, void *stream);

/* 1 when skv_gemv serves this shape well; 0 when it cannot run it or when the inputs every CTA rebuilds would
 * outweigh the weights it multiplies them with (many sequences of a long row: use a library GEMM there). */
int skv_gemv_supported(int N, int K, int B, int mode);

#ifdef __cplusplus
}
#endif
#endif /* SKV_H */
