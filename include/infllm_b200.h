/*
 * infllm_b200 — C ABI of the B200 (sm_100a) context-memory attention library.
 *
 * The reference (thunlp/InfLLM) is pure Python and has no FFI.  This header is the native
 * boundary that the Python drop-in classes (infllm_b200.attention.ContextManager,
 * CudaMultiStageDotProductionAttention, RotaryEmbeddingESM) bind with ctypes.  Each entry
 * point names the reference code it replaces, as file:line inside the reference repository.
 *
 * Conventions
 *   - every function returns 0 on success or a negative INFLLM_E_* code; nothing throws,
 *     aborts or traps.  infllm_last_error() gives the message of the calling thread's last error.
 *   - pointers named d_* are device pointers, h_* host pointers.  `stream` is a cudaStream_t
 *     passed as void*; work is enqueued on it and the call returns without synchronising unless
 *     stated otherwise.  The caller owns every buffer it passes in.
 *   - activations are bf16 (INFLLM_BF16) or fp16 (INFLLM_FP16); accumulators are fp32.
 *   - tensor layouts are given as (dims) with explicit element strides where the caller may
 *     pass a view; head_dim is always contiguous.
 */
#ifndef INFLLM_B200_H
#define INFLLM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define INFLLM_OK 0
#define INFLLM_E_BADARG (-1)    /* a size, stride or pointer is not acceptable */
#define INFLLM_E_CAPACITY (-2)  /* e.g. max_cached_block < topk: the reference asserts in CudaCache.alloc
                                   (inf_llm/attention/context_manager.py:19) */
#define INFLLM_E_CUDA (-3)      /* a CUDA runtime call failed; message holds cudaGetErrorString */
#define INFLLM_E_TIMEOUT (-4)   /* a bounded wait ran out */
#define INFLLM_E_UNSUPPORTED (-5)
#define INFLLM_E_NOMEM (-6)

#define INFLLM_BF16 0
#define INFLLM_FP16 1
#define INFLLM_F32 2 /* accepted only as the output type of infllm_lse_merge */

#define INFLLM_CACHE_LRU 0   /* cache_strategy "lru"   (context_manager.py:504-508) */
#define INFLLM_CACHE_LRU_S 1 /* cache_strategy "lru-s" (context_manager.py:454-470, 510-513): a cached unit's stamp is a
                              * decayed sum of the attention mass its keys received; every exec block then waits for
                              * the device, so look-ahead retrieval and attend-ahead decode are off */

/* mask modes of one attention stage (torch_impl.py:60-78) */
#define INFLLM_MASK_NONE 0
#define INFLLM_MASK_WINDOW 1     /* keep 0 <= i - j + offset < size */
#define INFLLM_MASK_COMPLEMENT 2 /* keep i - j + offset >= size */

const char* infllm_last_error(void);
/* Library build information: "infllm_b200 <version> sm_100a". */
const char* infllm_version(void);

/* ------------------------------------------------------------------ RoPE
 * Replaces RotaryEmbeddingESM (inf_llm/attention/rope.py:4-112).
 * infllm_rope_table: fp32 cos/sin of angle = (t * scale) * inv_freq[f], t in [0, length), f in
 *   [0, head_dim/2); d_cos/d_sin are (length, head_dim/2) (rope.py:49-65; the reference stores the
 *   halves duplicated).  h_inv_freq holds head_dim/2 fp32 values (rope.py:22-24).
 * infllm_rope_apply: out[h, t, :] = x[h, t, :] rotated to position pos0 + t * pos_step (pos_step 0
 *   gives the "one angle" form of rope.py:89-104; pos_step 1 the window-relative form of
 *   rope.py:35-47, 107-112).  Math in fp32, result rounded to `dtype` like the reference.
 *   x is (n_heads, len, head_dim) with element strides x_hs (head) and x_ts (token); out likewise. */
int infllm_rope_table(const float* h_inv_freq, float scale, int head_dim, int64_t length,
                      float* d_cos, float* d_sin, void* stream);
int infllm_rope_apply(const void* d_x, int64_t x_hs, int64_t x_ts, void* d_out, int64_t o_hs, int64_t o_ts,
                      int n_heads, int64_t len, int head_dim, const float* d_cos, const float* d_sin,
                      int64_t table_len, int64_t pos0, int pos_step, int dtype, void* stream);

/* ------------------------------------------------- multi-stage attention
 * Replaces MultiStageDotProductionAttention.append / get_result
 * (inf_llm/attention/dot_production_attention/base.py:3-30, torch_impl.py:15-96,
 * triton_impl.py:403-556): attention that is normalised jointly over several append()ed stages.
 *
 * State carried between stages, owned by the caller: d_acc (n_heads, lq, head_dim) fp32 un-normalised
 * output, d_m (n_heads, lq) fp32 running row maximum in the log2 domain, d_l (n_heads, lq) fp32
 * running denominator.
 *
 * infllm_attn_stage: fold one stage into the state.  first != 0 starts from an empty state (the
 *   buffers need not be initialised).  q (n_heads, lq, head_dim), k/v (n_kv_heads, lk, head_dim)
 *   with head/token element strides; lk may be 0.  mask_mode/mask_offset/mask_size as above, with
 *   i the query row and j the key row of this stage.
 * infllm_attn_finalize: out = acc / l in `dtype`, d_lse (n_heads, lq) fp32 = log-sum-exp of every row
 *   in the log2 domain (row with no visible key: out 0, lse -inf).
 * infllm_attn_colsum: per-key score of one stage = sum over queries of the jointly normalised
 *   probability (torch_impl.py:27-30; triton_impl.py:231-401), computed from the final d_lse.
 *   d_score is (n_heads, lk) fp32 with head stride score_hs; accumulate != 0 adds into it. */
int infllm_attn_stage(const void* d_q, int64_t q_hs, int64_t q_ts,
                      const void* d_k, int64_t k_hs, int64_t k_ts,
                      const void* d_v, int64_t v_hs, int64_t v_ts,
                      int n_heads, int n_kv_heads, int64_t lq, int64_t lk, int head_dim,
                      int mask_mode, int64_t mask_offset, int64_t mask_size,
                      float* d_acc, float* d_m, float* d_l, int first, int dtype, void* stream);
int infllm_attn_finalize(const float* d_acc, const float* d_m, const float* d_l,
                         void* d_out, int64_t o_hs, int64_t o_ts, float* d_lse,
                         int n_heads, int64_t lq, int head_dim, int dtype, void* stream);
int infllm_attn_colsum(const void* d_q, int64_t q_hs, int64_t q_ts,
                       const void* d_k, int64_t k_hs, int64_t k_ts,
                       int n_heads, int n_kv_heads, int64_t lq, int64_t lk, int head_dim,
                       int mask_mode, int64_t mask_offset, int64_t mask_size,
                       const float* d_lse, float* d_score, int64_t score_hs, int accumulate,
                       int dtype, void* stream);

/* ------------------------------------------------------ retrieval kernels
 * infllm_block_topk replaces calc_block_topk / VectorTensor.get_topk
 *   (context_manager.py:366-383, 159-163): scores[b] = <block_k[b, :], qbar> for b < n_blocks
 *   (fp32 accumulation), then the k highest in descending order, ties to the lower id.
 *   d_block_k (n_blocks, width) in `dtype`, row stride `width`; d_qbar (width) fp32.
 *   d_scores (n_blocks) fp32 scratch/out; d_out_ids (k) int32; d_out_scores (k) fp32 (may be NULL).
 *   id_base is added to every id written (unit-range sharding).  k <= 1024.
 * infllm_repr_select replaces get_block_k + mean (context_manager.py:268-277, 664-670): for each of
 *   n_new consecutive blocks of block_size tokens starting at row tok0 of d_k, and each query
 *   head h, the repr_topk tokens with the largest d_score[h, tok] (ties to the lower token) are
 *   gathered from K head h / (n_heads / n_kv_heads) and averaged; rows written to
 *   d_block_k_out (n_new, n_heads * head_dim) in `dtype`. */
int infllm_block_topk(const void* d_block_k, int64_t n_blocks, int width, const float* d_qbar,
                      float* d_scores, int k, int id_base, int32_t* d_out_ids, float* d_out_scores,
                      int dtype, void* stream);
/* infllm_block_score_rows: the same scores for a short HOST list of n unit ids only (d_scores[i] = score of unit
 * h_rows[i]); used to re-rank the look-ahead candidates of the next exec block after new units were sealed. */
int infllm_block_score_rows(const void* d_block_k, const int32_t* h_rows, int n, int width, const float* d_qbar,
                            float* d_scores, int dtype, void* stream);
int infllm_repr_select(const void* d_k, int64_t k_hs, int64_t k_ts, const float* d_score, int64_t score_hs,
                       int64_t tok0, int n_new, int block_size, int repr_topk,
                       int n_heads, int n_kv_heads, int head_dim, void* d_block_k_out, int dtype,
                       void* stream);

/* One new token (decode), as one launch: K and V rows (n_kv_heads, head_dim; heads k_hs / v_hs elements apart)
 * are copied to d_k_raw / d_v_out (heads kv_hs apart), K is also rotated to position pos_local into d_k_rot, Q
 * (n_heads rows, q_hs apart) is rotated to pos_local into d_q_loc and to pos_global into d_q_glb (heads qs_hs
 * apart), d_qbar (n_heads*head_dim fp32) receives d_q_glb — the query mean of a one-token exec block
 * (context_manager.py:373-375) — and d_score[h * score_hs] = 0 opens the token's score column.  Replaces the
 * per-token torch.cat / RoPE calls of ContextManager.append (context_manager.py:700-747) and _append (:480). */
int infllm_ingest_token(const void* d_q, int64_t q_hs, const void* d_k, int64_t k_hs, const void* d_v, int64_t v_hs,
                        void* d_q_loc, void* d_q_glb, int64_t qs_hs, float* d_qbar, void* d_k_raw, void* d_k_rot,
                        void* d_v_out, int64_t kv_hs, float* d_score, int64_t score_hs, int n_heads, int n_kv_heads,
                        int head_dim, const float* d_cos, const float* d_sin, int64_t table_len, int64_t pos_local,
                        int64_t pos_global, int dtype, void* stream);

/* ---------------------------------------------------------- decode attention
 * Split-K attention of ONE query token per head over a list of key/value segments, followed by a
 * log-sum-exp merge; replaces the two attn.append calls of ContextManager._append
 * (context_manager.py:486-489, 526-531) when the exec block is a single token.
 * Segment s: keys/values (n_kv_heads, seg_len[s], head_dim), tokens contiguous, at h_seg_k[s] / h_seg_v[s]
 * (device pointers) with head stride h_seg_hs[s] elements; h_seg_q[s] selects the query variant
 * (0: d_q0, 1: d_q1) — the local stage uses the window-relative rotation, the global stage the
 * one-angle rotation.  The h_seg_* arrays are HOST arrays of n_seg <= INFLLM_MAX_SEGMENTS entries.
 * The key list of every KV head is cut into at most max_parts runs (two CTAs per SM over all KV heads, fewer
 * for short lists); every run yields one partial per head: normalised output d_part_o (max_parts, n_heads,
 * head_dim) fp32 and log2-domain log-sum-exp d_part_lse (max_parts, n_heads); *n_parts receives how many were
 * written (infllm_attn_decode_max_parts bounds it; any max_parts >= 1 works).
 * logit_seg >= 0 also exports that segment's scaled log2-domain logits to d_logits (n_heads, seg_len).
 * infllm_lse_merge combines n_part partials into out (n_heads, head_dim) in `dtype` (head stride o_hs;
 * INFLLM_F32 keeps a rank's partial in fp32 for a second merge)
 * and d_lse (n_heads, may be NULL): the same merge serves the chunks of one GPU and the per-rank
 * partials gathered from several GPUs (unit-range sharding). */
#define INFLLM_MAX_SEGMENTS 80
int64_t infllm_attn_decode_max_parts(int n_seg, int64_t total_keys);
int infllm_attn_decode(const void* d_q0, const void* d_q1, int n_heads, int n_kv_heads, int head_dim,
                       int n_seg, const void* const* h_seg_k, const void* const* h_seg_v,
                       const int64_t* h_seg_hs, const int32_t* h_seg_len, const int32_t* h_seg_q,
                       float* d_part_o, float* d_part_lse, int max_parts, int* n_parts,
                       int logit_seg, float* d_logits, int dtype, void* stream);
int infllm_lse_merge(const float* d_part_o, const float* d_part_lse, int n_part, int n_heads, int head_dim,
                     void* d_out, int64_t o_hs, float* d_lse, int dtype, void* stream);
/* The same merge over partials that lie part_o_stride / part_lse_stride floats apart (e.g. rows [o | lse] as the
 * ranks' all-gather delivers them).  With d_logits (n_heads, logit_len), the scaled log2-domain logits that
 * infllm_attn_decode exported for a window segment, it also adds the token's attention row into the accumulated
 * local scores: d_score[h * score_hs + j] += exp2(d_logits[h, j] - lse[h]) (context_manager.py:488, 623-625). */
int infllm_lse_merge_ex(const float* d_part_o, int64_t part_o_stride, const float* d_part_lse,
                        int64_t part_lse_stride, int n_part, int n_heads, int head_dim, void* d_out, int64_t o_hs,
                        float* d_lse, int dtype, const float* d_logits, int64_t logit_len, float* d_score,
                        int64_t score_hs, const int32_t* d_skip, void* stream);
/* (d_skip, may be NULL: a device word; when it is non-zero at run time the call does nothing — the partials
 * were declared invalid by whoever produced them.) */

/* infllm_attn_decode whose segments [first_unit_seg, first_unit_seg + n_units) are memory units named on the
 * DEVICE: unit i is d_unit_ids[i]; this GPU owns the ids [id_lo, id_lo + n_owned) and finds them in cache slot
 * d_slot_table[id - id_lo] (K then V, unit_bytes, at d_cache + slot * unit_bytes; -1: not cached).  Units of other
 * owners and ids < 0 get weight zero; an owned unit that is not cached gets weight zero and sets *d_miss = 1.
 * h_seg_k / h_seg_v of those segments are ignored.  Lets the attention follow a device-side retrieval without a
 * host round trip.  With d_cache == NULL, d_slot_table is read as a table of 64-bit unit ADDRESSES instead (id - id_lo
 * -> where the unit's K block lives, V at + unit_bytes / 2; 0 = nowhere): the unit is then attended wherever it is,
 * for instance in place in pinned host memory.  infllm_slot_table_update writes d_table[h_ids[i]] = h_slots[i] (ids must not repeat). */
int infllm_attn_decode_units(const void* d_q0, const void* d_q1, int n_heads, int n_kv_heads, int head_dim, int n_seg,
                             const void* const* h_seg_k, const void* const* h_seg_v, const int64_t* h_seg_hs,
                             const int32_t* h_seg_len, const int32_t* h_seg_q, int first_unit_seg, int n_units,
                             const int32_t* d_unit_ids, const int32_t* d_slot_table, int id_lo, int n_owned,
                             const void* d_cache, int64_t unit_bytes, int32_t* d_miss, float* d_part_o,
                             float* d_part_lse, int max_parts, int* n_parts, int logit_seg, float* d_logits,
                             int dtype, void* stream);
int infllm_slot_table_update(int32_t* d_table, const int32_t* h_ids, const int32_t* h_slots, int n, void* stream);
/* The same for a table of unit ADDRESSES (unit id -> where its K block lives right now; V follows at unit_bytes / 2):
 * d_table[h_ids[i]] = h_addrs[i].  infllm_shard_token_run reads such a table when its d_unit_ptrs is set: a
 * retrieved unit is then found wherever it lives — in a cache slot, or in place in the pinned host store, which the
 * GPU reads over PCIe — so that no token ever has to wait for a refill. */
int infllm_ptr_table_update(uint64_t* d_table, const int32_t* h_ids, const uint64_t* h_addrs, int n, void* stream);

/* infllm_attn_decode_noalloc has no counterpart in the reference.  It is infllm_attn_decode followed by
 * infllm_lse_merge in one call that allocates nothing: the split-K partials go to a scratch array that is
 * part of the library image (about 5.3 MB of every GPU that loads the library, until the process exits)
 * instead of a buffer from the caller.  It is meant for callers that hold raw device pointers but cannot
 * obtain device memory themselves at the point of the call: a serving engine whose own pool has already
 * claimed the whole GPU, so that cudaMalloc fails or stalls every stream; a plugin running inside such
 * an engine's step function, where allocation is forbidden by contract; a latency-critical decode loop
 * that must not touch an allocator at all.  The caller still passes the queries, the key/value segments
 * and the output: d_out (n_heads, head_dim) in `dtype` with head stride o_hs, d_lse (n_heads) or NULL.
 * Limits: head_dim 128, n_heads <= 64, and at most 160 chunks of 128 keys summed over the segments (a
 * segment of L keys takes ceil(L/128) chunks); beyond that the call returns INFLLM_E_CAPACITY and
 * nothing is launched.  The first call made on a device looks up the scratch address for that device
 * (a cudaGetSymbolAddress call with that device current); make that first call before any stream
 * capture begins.  All calls on a device share the one scratch array, which keeps what the last call
 * wrote: two calls that may overlap on the GPU (different streams, or concurrent host threads) race
 * and must be serialised by the caller.  Nothing in the array needs clearing between calls. */
int infllm_attn_decode_noalloc(const void* d_q0, const void* d_q1, int n_heads, int n_kv_heads, int head_dim,
                               int n_seg, const void* const* h_seg_k, const void* const* h_seg_v,
                               const int64_t* h_seg_hs, const int32_t* h_seg_len, const int32_t* h_seg_q,
                               void* d_out, int64_t o_hs, float* d_lse, int dtype, void* stream);

/* ------------------------------------------------------------ context memory
 * One infllm_ctx is the native state of one batch element ("unit") of the reference's
 * ContextManager (context_manager.py:196-816): token buffers for the local window and the
 * un-sealed remainder, the init sink, representative keys, the pinned host store of sealed
 * memory units, the GPU cache of max_cached_block units with LRU replacement, and the
 * exec-block loop of append() (context_manager.py:682-813, _append :474-545, append_global
 * :614-679). */
typedef struct infllm_ctx infllm_ctx;

typedef struct infllm_config {
  int32_t n_heads, n_kv_heads, head_dim;
  int32_t n_init, n_local, block_size, max_cached_block, topk, exc_block_size, repr_topk;
  int32_t cache_strategy; /* INFLLM_CACHE_* */
  int32_t dtype;          /* INFLLM_BF16 / INFLLM_FP16 */
  double score_decay;     /* lru-s only; a double because the reference multiplies Python floats by it */
  float rope_base, rope_scale;
  int32_t device;         /* CUDA device ordinal */
  int32_t shard_rank, shard_world; /* unit-range sharding of the store; 0,1 = not sharded */
  int32_t debug_flags;    /* 0 in production; test switches, one per bit —
                           *  1: exec blocks on the shape-generic mma.sync kernels, no tcgen05 kernels
                           *  2: no look-ahead retrieval: every exec block waits for its ids from the device
                           *  4: refills from a device copy of the store by one cudaMemcpyAsync per unit as well
                           *     (refills from the pinned host store always are, like MemoryUnit.load,
                           *     context_manager.py:57-71), not by the copy kernel
                           *  8: the two-heads-per-CTA tcgen05 attention kernel whatever the head count
                           * 16: one-token appends wait for the retrieved ids before launching the attention */
  int32_t look_depth;     /* exec blocks ranked and staged ahead of the running one; 0 = default (2), at most 8; the
                           * cache gets that many times topk spare slots */
  int32_t chunk_topk_calc; /* chunk_topk_calc of the reference (context_manager.py:749-770, 548-610), in tokens; 0 = off:
                           * a call of more than one token is cut into chunks of this size rounded down to whole exec
                           * blocks, and every exec block of a chunk retrieves among the units sealed when it started */
  int32_t device_store_mb; /* 0 (default): sealed units live in the pinned host store only and every cache refill is a
                           * host-to-device copy, as in the reference (MemoryUnit.load, context_manager.py:57-71).
                           * > 0: up to this many MiB of the store's first units are ALSO kept in device memory taken
                           * from the pool of infllm_device_store_reserve, and a refill of such a unit is a
                           * device-to-device copy.  The cache, its LRU order and the host store are unchanged. */
  int32_t reserved[2];    /* zero */
} infllm_config;

/* Device copy of the store: one pool per device, shared by every context of the process whose configuration asks
 * for a device copy (device_store_mb > 0).  infllm_device_store_reserve allocates `bytes` of device memory on
 * `device` (rounded down to whole 128 MiB slabs) — the only allocation the device copy ever makes, done here and
 * not inside append; contexts take slabs from it as their stores grow and hand them back when they are reset or
 * destroyed, and a context that finds the pool empty simply keeps refilling from the host.  Calling it again
 * grows the pool.  infllm_device_store_release frees the slabs no context holds; infllm_device_store_info reports
 * the pool's size and what is handed out.  No counterpart in the reference, whose sealed units live on the host only. */
int infllm_device_store_reserve(int device, int64_t bytes);
int infllm_device_store_release(int device);
int infllm_device_store_info(int device, int64_t* total_bytes, int64_t* used_bytes);

/* Validates the configuration (exc_block_size <= n_local, context_manager.py:219;
 * max_cached_block >= topk, context_manager.py:19 -> INFLLM_E_CAPACITY) and allocates nothing
 * large: buffers are created on the first append (context_manager.py:292-363). */
int infllm_ctx_create(const infllm_config* cfg, infllm_ctx** out);
int infllm_ctx_destroy(infllm_ctx* ctx);
/* Forget every token but keep the allocations (device buffers, pinned host store). */
int infllm_ctx_reset(infllm_ctx* ctx);

/* ContextManager.append (context_manager.py:682-813) for one unit: q (n_heads, len, head_dim) and
 * k, v (n_kv_heads, len, head_dim), un-rotated, element strides given; out (n_heads, len, head_dim).
 * Runs every exec block of the call; synchronises with the host once per exec block that has more
 * sealed units than topk (the retrieved ids are needed to plan the cache), otherwise asynchronous. */
int infllm_ctx_append(infllm_ctx* ctx, const void* d_q, int64_t q_hs, int64_t q_ts,
                      const void* d_k, int64_t k_hs, int64_t k_ts,
                      const void* d_v, int64_t v_hs, int64_t v_ts,
                      void* d_out, int64_t o_hs, int64_t o_ts, int64_t len, void* stream);

/* Introspection (what the reference keeps as Python attributes). */
typedef struct infllm_ctx_info {
  int64_t length;        /* ContextManager.length (context_manager.py:211, 793, 815) */
  int64_t frontier;      /* first token not yet in the init sink or a sealed unit */
  int64_t num_blocks;    /* num_global_block (:319, 673) */
  int64_t init_len;      /* init_k.size(-2) (:341, 628-646) */
  int64_t num_cached;    /* len(cached_blocks[u]) */
  int64_t load_count;    /* LRU clock (:226, 505) */
  int64_t exec_blocks;   /* exec blocks run by the last append */
  int64_t h2d_bytes, d2h_bytes; /* store traffic since create/reset */
  int64_t cache_hits, cache_misses, evictions;
  int64_t h2d_late_bytes; /* the part of h2d_bytes that an exec block had to wait for (not staged ahead of it) */
  int64_t inplace_units;  /* one-token appends: retrieved units whose keys the attention read in place from the store
                           * (over PCIe from the pinned host store, or from its device copy) because their refill had
                           * not landed in a cache slot yet */
} infllm_ctx_info;
int infllm_ctx_get_info(infllm_ctx* ctx, infllm_ctx_info* info);
/* Per-kernel timing, off by default.  When enabled, the context records a CUDA event pair around each
 * launch of its hot kernels on the stream they run on.  infllm_ctx_get_profile synchronises, adds up
 * and clears the records: for each slot the device milliseconds, the algorithmic work (FLOPs of visible
 * query-key pairs for the attention slots, bytes for the HBM-bound slots) and the number of launches. */
#define INFLLM_PROF_ATTN 0   /* exec-block attention: 4*D*H*(visible pairs) FLOPs */
#define INFLLM_PROF_COLSUM 1 /* local-score pass: 2*D*H*(visible local pairs) FLOPs */
#define INFLLM_PROF_DECODE 2 /* one-token attention: K and V bytes of every attended key */
#define INFLLM_PROF_TOPK 3   /* unit scoring + top-k: bytes of the representative keys */
#define INFLLM_PROF_SLOTS 4
int infllm_ctx_profile(infllm_ctx* ctx, int enable);
int infllm_ctx_get_profile(infllm_ctx* ctx, double* ms, double* work, int64_t* launches);
/* Event trace of the exec-block loop, off by default: when enabled the context records a CUDA event at fixed
 * points of every stream it uses (labels: 0 attention begin, 1 attention end, 2 urgent score tiles end,
 * 3 sealing + candidate scoring end, 4 rest of the score pass end, 5/6 look-ahead ranking begin/end,
 * 7/8 begin/end of the refill copies staged ahead for a later exec block (copy stream), 9 representative keys end,
 * 10 packing of sealed units end, 11/12 begin/end of the refill copies an exec block waits for (urgent stream)).
 * infllm_ctx_get_trace synchronises, returns (label, exec block, ms since the first mark) in record order and
 * clears the trace. */
int infllm_ctx_trace(infllm_ctx* ctx, int enable);
int infllm_ctx_get_trace(infllm_ctx* ctx, int32_t* labels, int64_t* exec_blocks, float* ms, int cap, int* n);
/* Host time (microseconds, summed since the last call) the exec-block loop spent in each of its phases:
 * 0 device ranking + sync, 1 cache plan + late fetches, 2 look-ahead launch, 3 attention launch,
 * 4 look-ahead wait + staging copies, 5 sealing, 6 candidate wait + ranking, 7 unused.  Diagnostics. */
#define INFLLM_HOST_TIMERS 8
int infllm_ctx_get_host_timers(infllm_ctx* ctx, double* us);
/* The tensor-core kernels bound every wait on a barrier; a wait that runs out makes the kernel record
 * an error and return instead of hanging.  infllm_device_error synchronises the device, reads the
 * record (code 0 = none, 1 = wait ran out; `where` identifies the wait) and clears it. */
int infllm_device_error(int* code, int* where);
/* Writes the record from the host (code 0 clears it): lets a host-side test check that the product path reports a
 * recorded error — infllm_ctx_append returns INFLLM_E_TIMEOUT at the latest on the call after the one whose kernel
 * recorded it — without making a wait run out on the GPU. */
int infllm_device_error_set(int code, int where);
/* Number of kernels this library has launched in the process so far. */
long long infllm_launch_count(void);

/* cached_blocks[u] in dict order: ids and stamps (LRU clock, or lru-s score). Returns count in *n. */
int infllm_ctx_get_cached(infllm_ctx* ctx, int32_t* h_ids, double* h_stamps, int cap, int* n);
/* Retrieval of exec block `eb` of the last append, in the order the scorer returned it. */
int infllm_ctx_get_topk(infllm_ctx* ctx, int64_t eb, int32_t* h_ids, int cap, int* n);
/* Copies representative-key rows [b0, b0+n) (n_heads*head_dim each, `dtype`) to a host buffer; synchronises. */
int infllm_ctx_get_block_k(infllm_ctx* ctx, int64_t b0, int64_t n, void* h_dst);
/* Test/bench hook: install a synthetic store without running a prefill (decode-only workloads):
 * n_units sealed units whose K/V the library reads from h_units (n_units, 2, n_kv_heads, block_size,
 * head_dim) — copied into the pinned store — representative keys from h_block_k (n_units, n_heads*head_dim),
 * an init sink (n_kv_heads, n_init, head_dim) x2 and a local window (n_kv_heads, n_local, head_dim) x2,
 * all in `dtype` on the host.  length becomes n_init + n_units*block_size + n_local. */
int infllm_ctx_load_synthetic(infllm_ctx* ctx, int64_t n_units, const void* h_units, const void* h_block_k,
                              const void* h_init_k, const void* h_init_v, const void* h_win_k,
                              const void* h_win_v, void* stream);

/* ------------------------------------------------ KV-head-group sharding (no counterpart in the reference)
 * Every rank runs a context on its own slice of the heads (n_heads / n_kv_heads of the config are the LOCAL
 * counts); the one exchange is the sum over ranks of the retrieval scores, which the reference forms over all
 * heads at once (context_manager.py:373-378).  After it every rank takes the same top-k and keeps the same LRU
 * order.  The sums are NCCL all-reduces; NCCL is looked up at run time in the process (PyTorch has loaded it).
 * infllm_comm_unique_id fills infllm_comm_id_bytes() bytes on one rank; the caller sends them to the others
 * (any channel), every rank calls infllm_comm_create with them (a collective call), then infllm_ctx_set_comm on
 * each fresh context.  One communicator serves any number of contexts of the process. */
typedef struct infllm_comm infllm_comm;
int infllm_comm_id_bytes(void);
int infllm_comm_unique_id(void* h_out);
int infllm_comm_create(const void* h_id, int rank, int world, infllm_comm** out);
int infllm_comm_destroy(infllm_comm* comm);
int infllm_ctx_set_comm(infllm_ctx* ctx, infllm_comm* comm);

/* ------------------------------------------- exchange through peer memory (no counterpart in the reference)
 * For the unit-range sharded decode: every rank owns a mailbox buffer that every rank of the node can write (CUDA
 * IPC).  infllm_mailbox_create allocates it and returns its handle (infllm_mailbox_handle_bytes() bytes); the
 * caller gathers the handles of all ranks and passes them, in rank order, to infllm_mailbox_open.
 * infllm_mailbox_put copies a message into slot [this rank] of every rank's mailbox (at slot_off + rank *
 * slot_bytes) with a kernel and then sets the flag word [this rank] at flag_off of every mailbox to `seq`;
 * infllm_mailbox_wait makes `stream` wait — at most limit_us microseconds — until all ranks' flag words of the
 * local mailbox show `seq`; a sender that does not arrive leaves 1 + its rank in *d_err, and kernels behind the
 * wait that are given d_err write nothing.  With miss_off >= 0 the word at that offset of every received message
 * is OR-ed into *d_any_miss; d_clear (may be NULL) is a device word the same kernel sets to zero.
 * infllm_topk_pairs ranks the gathered retrieval candidates, world messages
 * [k score bit patterns | k ids] (sender_stride_words apart), into the k best ids: descending score, ties to the
 * lower id, ids < 0 are padding.  The exchanges of one token alternate (candidates, partials), which is the
 * flow control: a mailbox slot is rewritten only after every rank has consumed it. */
typedef struct infllm_mailbox infllm_mailbox;
int infllm_mailbox_handle_bytes(void);
int infllm_mailbox_create(int64_t bytes, int rank, int world, void* h_handle, infllm_mailbox** out);
int infllm_mailbox_open(infllm_mailbox* m, const void* h_handles);
/* Instead of opening rank `rank`'s handle: that rank's buffer is `d_buffer`, device memory of this process (several
 * ranks emulated in one process, or a stand-in for a rank that will never post, in a test of the bounded waits). */
int infllm_mailbox_alias(infllm_mailbox* m, int rank, void* d_buffer);
void* infllm_mailbox_local(infllm_mailbox* m);
int infllm_mailbox_destroy(infllm_mailbox* m);
int infllm_mailbox_put(infllm_mailbox* m, const void* d_src, int64_t bytes, int64_t slot_off, int64_t slot_bytes,
                       int64_t flag_off, uint32_t seq, void* stream);
int infllm_mailbox_wait(infllm_mailbox* m, int64_t flag_off, uint32_t seq, int limit_us, int* d_err, int64_t slot_off,
                        int64_t slot_bytes, int64_t miss_off, int32_t* d_any_miss, int32_t* d_clear, void* stream);
int infllm_topk_pairs(const int32_t* d_cand, int64_t sender_stride_words, int world, int k, int32_t* d_out_ids,
                      const int* d_err, void* stream);

/* One decode token of a unit-range shard, every launch of it in one call (no counterpart in the reference): ingest,
 * local scoring + top-k, candidate exchange, global top-k, attention over the owned retrieved units and this
 * rank's share of the window, local merge, partial exchange, final merge with the accumulation of the local
 * scores, and the copy of [retrieved ids (topk) | exchange error | any miss | pad] to h_status.  All pointers are
 * device pointers except h_status (pinned host).  Token buffers are (n_kv_heads, cap, head_dim), token slot `at`
 * holds position `at` of the rotary table (cap rows); the accumulated scores are (n_heads, cap) fp32. */
typedef struct infllm_shard_token {
  const void *d_q, *d_k, *d_vin;           /* the token: q (n_heads rows, q_hs apart), k / v (n_kv_heads rows) */
  int64_t q_hs, k_hs, v_hs;
  void *d_q_loc, *d_q_glb;                 /* (n_heads, head_dim) rotated queries */
  float* d_qbar;                           /* (n_heads * head_dim) */
  void *d_k_raw, *d_k_rot, *d_v;           /* token buffers */
  float* d_score;
  const float *d_cos, *d_sin;
  int64_t cap, at;                         /* slots of the token buffers; the new token's slot */
  int32_t n_heads, n_kv_heads, head_dim, dtype, n_local, block_size, topk, pad0;
  const void* d_block_k;                   /* this rank's representative keys (n_owned rows) */
  float* d_scores;                         /* (n_owned) scratch */
  int32_t n_owned, id_lo;                  /* this rank owns the ids [id_lo, id_lo + n_owned) */
  int32_t* d_cand;                         /* (2 * topk) message: score bits, ids */
  int32_t* d_status;                       /* (topk + 4) */
  int32_t* h_status;
  const int32_t* d_slot_table;             /* (n_owned) id - id_lo -> cache slot or -1 */
  const void* d_cache;
  int64_t unit_bytes;
  int64_t share_at, share_len;             /* this rank's share of the window: slots [share_at, share_at + share_len) */
  const void *d_init_k, *d_init_v;         /* sink (n_kv_heads, init_len, head_dim); init_len 0 on ranks without it */
  int64_t ovf_at, ovf_len;                 /* tokens between the last sealed unit and the window; len 0 without */
  int32_t init_len, max_parts;
  float *d_part_o, *d_part_lse, *d_logits; /* split-K scratch; logits (n_heads, share_len) */
  float* d_pack;                           /* (n_heads * (head_dim + 1) + 4) message: o, lse, miss word */
  void* d_out;                             /* (n_heads, head_dim) result */
  float* d_lse;                            /* (n_heads) */
  int64_t cand_off, cand_slot, cand_bytes, part_off, part_slot, part_bytes, flag1_off, flag2_off; /* mailbox layout */
  uint32_t seq;
  int32_t wait_us;
  const uint64_t* d_unit_ptrs;             /* (n_owned) id - id_lo -> address of the unit's K block; NULL: the slot table */
  uint32_t* d_ticket;                      /* one zeroed word: scoring and top-k as ONE launch; NULL: two launches */
  int64_t ll_part_off, ll_part_slot;       /* the same for the partials: slots of part_bytes / 4 8-byte words */
  int64_t ll_cand_off, ll_cand_slot;       /* 0, or a second candidate region of the mailbox, slots of 2 * topk 8-byte
                                              words: the candidates travel as {value, seq} pairs that carry their own
                                              arrival flag (no system-wide fence, no flag word) */
  uint64_t* d_stamps;                      /* NULL, or 8 words: the device's nanosecond timer before the token and behind
                                              each of its 7 launches (a one-thread kernel per stamp: for a profiling pass) */
} infllm_shard_token;
int infllm_shard_token_run(const infllm_shard_token* args, infllm_mailbox* mailbox, void* stream);

/* One memory unit from the pinned host store into a cache slot, asynchronously on `stream`: MemoryUnit.load's
 * host-to-device copy (context_manager.py:57-71) for callers that keep their own cache. */
int infllm_unit_fetch(void* d_slot, const void* h_unit, int64_t bytes, void* stream);

/* The cache of a caller that keeps its own units (the unit-range shard of the sharded decode), in one call per
 * retrieval: of `ids` (n <= 256; negative entries and ids outside [id_lo, id_lo + n_owned) are skipped) the LRU
 * table plans the evictions and takes the stamp load_count (context_manager.py:246-265, 495-515), units that are
 * not cached go from the pinned store into free slots on `stream` (MemoryUnit.load, context_manager.py:57-71), and
 * the device tables learn the changes (slot, or -1; address of the slot, or of the unit in the pinned store).
 * All fields are the caller's; the library keeps nothing between calls. */
typedef struct infllm_shard_cache {
  struct infllm_lru* lru;
  int32_t* slot_of;        /* (n_owned) cache slot of unit id_lo + i, -1: not cached */
  int32_t* free_slots;     /* stack of free slots; n_free of them are valid */
  int32_t n_free, id_lo, n_owned, pad;
  int64_t load_count, hits, misses;
  void* d_cache;           /* slots of unit_bytes */
  const void* h_units;     /* pinned store: unit id_lo + i at i * unit_bytes */
  int64_t unit_bytes;
  int32_t* d_slot_table;   /* may be NULL */
  uint64_t* d_ptr_table;   /* may be NULL */
} infllm_shard_cache;
int infllm_shard_refill(infllm_shard_cache* cache, const int32_t* ids, int n, void* stream);

/* Persistence (the reference keeps a layer's memory only live, in past_key_values, greedy_search.py:99):
 * infllm_ctx_save writes the whole memory of a context — sink, sealed units, representative keys, un-sealed tokens
 * with their accumulated scores, LRU table and counters — to a file; infllm_ctx_load brings it back into a
 * context created with the same configuration, refills the cache as the LRU table lists it, and the next append
 * continues as if nothing had happened.  Both synchronise `stream`. */
int infllm_ctx_save(infllm_ctx* ctx, const char* path, void* stream);
int infllm_ctx_load(infllm_ctx* ctx, const char* path, void* stream);

/* ----------------------------------------------------- host logic, GPU-free
 * The LRU table alone (context_manager.py:246-265, 495-515): dict-ordered ids with stamps.
 * Exposed so that the eviction order can be tested without a device. */
typedef struct infllm_lru infllm_lru;
int infllm_lru_create(int capacity, infllm_lru** out);
int infllm_lru_destroy(infllm_lru* t);
/* Evicts for `wanted` (n ids), writes evicted ids (in eviction order) to h_evicted (cap n_cached), count to *n_evicted. */
int infllm_lru_plan(infllm_lru* t, const int32_t* wanted, int n, int32_t* h_evicted, int* n_evicted);
int infllm_lru_stamp(infllm_lru* t, const int32_t* wanted, int n, double value);
int infllm_lru_scale(infllm_lru* t, double factor);             /* lru-s decay */
int infllm_lru_add(infllm_lru* t, int32_t id, double value);    /* lru-s score add */
int infllm_lru_items(infllm_lru* t, int32_t* h_ids, double* h_stamps, int cap, int* n);

#ifdef __cplusplus
}
#endif
#endif /* INFLLM_B200_H */
