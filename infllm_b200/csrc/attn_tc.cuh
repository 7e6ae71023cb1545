// Parameter blocks and host entry points of the tensor-core attention kernels (attn_tc.cu).
#pragma once
#include "attn_common.cuh"
#include "tc_common.cuh"

namespace infllm {

constexpr int kTcMaxMaps = 12;
constexpr int kTile = 128;

struct TcSeg {
  int16_t map_k, map_v;  // indices into AttnTcParams::maps
  int32_t tok0;          // token coordinate of the segment's first key
  int32_t c3_k, c3_v;    // 4th coordinate for rank-4 maps (cache slots), -1 for rank-3 maps
  int32_t len;
};

struct TcStage {
  int32_t map_q, q_row0;
  int32_t mask_mode, seg_begin, seg_end, pad;
  int64_t mask_offset, mask_size, lk;
};

struct AttnTcParams {
  alignas(64) CUtensorMap maps[kTcMaxMaps];
  TcStage stage[kMaxStage];
  TcSeg seg[kMaxSeg];
  int32_t n_stage, n_heads, n_kv_heads, pad;
  int64_t lq;
  void* out;
  int64_t o_hs, o_ts;
  float* lse;
  float scale_log2;
  int* err;
  // two-head kernel only: the key tiles of a work item are cut into n_split runs; with n_split > 1 every run
  // writes an un-normalised partial (acc, m, l) and attn_tc_combine merges them
  int32_t n_split, pad2;
  float* part_acc;  // (n_split, H, lq, 128)
  float* part_m;    // (n_split, H, lq)
  float* part_l;    // (n_split, H, lq)
};

struct ColsumTcParams {
  alignas(64) CUtensorMap map_q, map_k;
  int32_t q_row0, k_tok0, n_heads, group;
  int64_t lq, lk;
  int32_t mask_mode, accumulate;
  int32_t tiles_per_cta, pad;
  int64_t mask_offset, mask_size;
  const float* lse;
  float* score;
  int64_t score_hs;
  float scale_log2;
  int* err;
};


int encode_rows_map(CUtensorMap* map, int dtype, const void* base, int64_t rows, int64_t heads, int64_t hs, int64_t ts);
bool tc_rows_ok(const void* base, int64_t hs, int64_t ts);
int tc_get_error_ptr(int** p);
// one CTA per (128-query tile, head)
int attn_tc3_launch(const AttnTcParams& P, int dtype, cudaStream_t s);
// two query heads of one KV head per CTA (needs an even number of query heads per KV head)
int attn_tc2_launch(const AttnTcParams& P, int dtype, cudaStream_t s);
size_t attn_tc2_scratch_floats(int n_split, int n_heads, int64_t lq);
int colsum_tc_launch_maps(const CUtensorMap& map_q, const CUtensorMap& map_k, int q_row0, int k_tok0, int n_heads,
                          int n_kv_heads, int64_t lq, int64_t lk, int mask_mode, int64_t mask_offset,
                          int64_t mask_size, const float* lse, float* score, int64_t score_hs, int accumulate,
                          int dtype, cudaStream_t s);
int colsum_tc_launch(const void* q, int64_t q_hs, int64_t q_ts, const void* k, int64_t k_hs, int64_t k_ts, int n_heads,
                     int n_kv_heads, int64_t lq, int64_t lk, int mask_mode, int64_t mask_offset, int64_t mask_size,
                     const float* lse, float* score, int64_t score_hs, int accumulate, int dtype, cudaStream_t s);

}  // namespace infllm
