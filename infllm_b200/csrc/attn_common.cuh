// Parameter blocks shared by the attention kernels and the context-memory runtime.
#pragma once
#include "common.cuh"

namespace infllm {

// One contiguous run of keys/values of a stage.  Tokens are `ts` elements apart, heads `hs`.
struct KvSeg {
  const void* k;
  const void* v;
  int64_t hs;
  int32_t ts;
  int32_t len;
};

constexpr int kMaxSeg = 80;    // segments per launch (retrieved units + init sink + overflow + window)
constexpr int kMaxStage = 2;   // stages fused in one launch

// One stage = one append() of the reference's multi-stage attention: its own queries, mask and keys.
struct StageDesc {
  const void* q;  // (H, lq, D)
  int64_t q_hs, q_ts;
  int32_t mask_mode;
  int32_t seg_begin, seg_end;  // range in AttnParams::seg
  int64_t mask_offset, mask_size;
  int64_t lk;  // total keys of the stage
};

struct AttnParams {
  StageDesc stage[kMaxStage];
  KvSeg seg[kMaxSeg];
  int32_t n_stage;
  int32_t n_heads, n_kv_heads;
  int32_t first, last;  // first: start from an empty state; last: write out/lse instead of the state
  int64_t lq;
  float* acc;  // (H, lq, D) fp32 state
  float* m;    // (H, lq)
  float* l;    // (H, lq)
  void* out;   // (H, lq, D) in dtype, when last
  int64_t o_hs, o_ts;
  float* lse;  // (H, lq) log2-domain LSE, when last (may be null)
  float scale_log2;  // log2(e) / sqrt(D)
};

// [lo, hi] inclusive range of key indices of a stage that a block of query rows [i0, i1] can see
__host__ __device__ inline void visible_key_range(int mode, int64_t off, int64_t size, int64_t i0, int64_t i1,
                                                  int64_t lk, int64_t* lo, int64_t* hi) {
  int64_t a = 0, b = lk - 1;
  if (mode == INFLLM_MASK_WINDOW) {
    a = i0 + off - size + 1;
    b = i1 + off;
  } else if (mode == INFLLM_MASK_COMPLEMENT) {
    b = i1 + off - size;
  }
  *lo = a < 0 ? 0 : a;
  *hi = b > lk - 1 ? lk - 1 : b;
}

__device__ __forceinline__ bool mask_keep(int mode, int64_t off, int64_t size, int64_t i, int64_t j) {
  int64_t dist = i - j + off;
  if (mode == INFLLM_MASK_WINDOW) return dist >= 0 && dist < size;
  if (mode == INFLLM_MASK_COMPLEMENT) return dist >= size;
  return true;
}

// Decode attention whose unit segments are resolved on the device: segment first_seg + i of the launch holds
// the unit ids[i].  This lets the attention follow the top-k kernel on the stream before the host has seen the ids.
// Two ways to find a unit: `ptrs`, a table of addresses (unit id -> where its K block lives right now: a cache
// slot, a device copy of the store, or the pinned host store, which the GPU reads in place; 0 = nowhere), or
// `table`, unit id -> cache slot (-1 when not cached) with the cache's base address.  A unit that cannot be found
// contributes nothing and sets *miss.
struct DecodeIndirect {
  const int32_t* ids = nullptr;    // n_units unit ids (device memory)
  const int32_t* table = nullptr;  // unit id -> cache slot, -1 when the unit is not cached (device memory)
  const unsigned long long* ptrs = nullptr;  // unit id -> address of its K block (V follows at unit_bytes / 2)
  const char* cache = nullptr;     // slot 0
  const unsigned long long* landing = nullptr;  // with ptrs: n_units addresses of landing slots (0 = none); a unit whose
                                   // address has bit 0 set (it lives in the store) is also written to the slot of
                                   // its place in ids
  int64_t unit_bytes = 0;          // K then V of one unit
  int32_t n_units = 0, first_seg = 0;
  int32_t* miss = nullptr;
  // unit-range sharding: this GPU owns the ids [id_lo, id_lo + n_owned) and the tables start at id_lo; a retrieved
  // unit of another rank, or a padding id < 0, gets weight zero here and is not a miss
  int32_t id_lo = 0, n_owned = 0x7fffffff;
  // the launch directly before this one on the stream is a chain kernel (common.cuh) that writes nothing the other
  // segments need: their keys are attended to before the kernel waits for it, the units' after
  int32_t early_rest = 0;
};

int attn_general_launch(const AttnParams& p, int head_dim, int dtype, cudaStream_t s);
int attn_decode_launch(const void* q0, const void* q1, int64_t q_hs, int n_heads, int n_kv_heads, int head_dim, int n_seg,
                       const KvSeg* segs, const int32_t* seg_q, float* part_o, float* part_lse, int max_parts,
                       int* n_parts_out, int logit_seg, float* logits, int dtype, cudaStream_t s,
                       const DecodeIndirect* ind);
// Optional first step of the merge: wait (bounded) until `world` senders' flag words show `seq` — the partials being
// merged were put into this GPU's mailbox by peers.  A flag that does not arrive within `limit` polls leaves
// 1 + its rank in *err and the kernel writes nothing.
struct MergeWait {
  // flag-in-data partials: when set, partial p's o row and lse are 8-byte words {value, seq} at
  // ll[p * o_ps + h * head_dim + d] and ll[p * lse_ps + n_heads * head_dim + h] (strides in words); every thread polls
  // the words it needs until they carry `seq` (bounded by `limit`), part_o / part_lse / flags are not used
  const volatile unsigned long long* ll = nullptr;
  const volatile uint32_t* flags = nullptr;
  uint32_t seq = 0, limit = 0;
  int32_t world = 0;
  int* err = nullptr;
};
int lse_merge_launch(const float* part_o, const float* part_lse, int n_part, int n_heads, int head_dim, void* out,
                     int64_t o_hs, float* lse, int dtype, cudaStream_t s, const float* logits, int64_t logit_len,
                     float* score, int64_t score_hs, const int32_t* skip, int64_t o_ps = 0, int64_t lse_ps = 0,
                     const MergeWait* wait = nullptr);
int attn_colsum_launch(const void* q, int64_t q_hs, int64_t q_ts, const void* k, int64_t k_hs, int64_t k_ts,
                       int n_heads, int n_kv_heads, int64_t lq, int64_t lk, int head_dim, int mask_mode,
                       int64_t mask_offset, int64_t mask_size, const float* lse, float* score, int64_t score_hs,
                       int accumulate, int dtype, cudaStream_t s);

}  // namespace infllm
