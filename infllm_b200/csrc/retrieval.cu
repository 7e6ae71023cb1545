// Retrieval kernels: memory-unit scoring + top-k, and representative-key selection at sealing.
//
// block_score_topk_kernel  k <= 64 over <= 16384 units, the usual case: HBM-streaming GEMV (one warp per
//                     representative-key row, 16-byte loads, query mean staged in shared memory, fp32
//                     accumulation) whose last CTA ranks the scores (threshold from the maxima of small
//                     groups, rank sort of the few candidates).
// block_score_kernel + topk_select_kernel  any size: the same GEMV, then a 4-pass 8-bit radix select of the
//                     k-th largest score, an index-ordered gather of the winners and a rank sort.
//                     Both: descending score, ties to the lower id.
// repr_select_kernel  per (new unit, query head): repr_topk arg-max rounds over the accumulated
//                     local scores, gather + mean of the chosen un-rotated keys.
#include <algorithm>

#include "common.cuh"

namespace infllm {

constexpr int kScoreWarps = 8;
constexpr int kMaxScoreRows = 512;  // candidate rows per launch of block_score_rows_kernel

template <typename T>
__global__ void __launch_bounds__(kScoreWarps * 32)
block_score_kernel(const T* __restrict__ bk, int64_t n, int width, const float* __restrict__ qbar,
                   float* __restrict__ scores) {
  extern __shared__ float sq[];
  for (int i = threadIdx.x; i < width; i += blockDim.x) sq[i] = qbar[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * kScoreWarps + warp;
  if (row >= n) return;
  const T* p = bk + row * (int64_t)width;
  float acc = 0.f;
#pragma unroll 4
  for (int c = lane * 8; c < width; c += 32 * 8) {
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(p + c));
    const typename Act<T>::T2* v2 = reinterpret_cast<const typename Act<T>::T2*>(&raw);
    const float4 qa = *reinterpret_cast<const float4*>(sq + c);
    const float4 qb = *reinterpret_cast<const float4*>(sq + c + 4);
    float2 f0 = Act<T>::to_f2(v2[0]), f1 = Act<T>::to_f2(v2[1]), f2 = Act<T>::to_f2(v2[2]),
           f3 = Act<T>::to_f2(v2[3]);
    acc = fmaf(f0.x, qa.x, acc);
    acc = fmaf(f0.y, qa.y, acc);
    acc = fmaf(f1.x, qa.z, acc);
    acc = fmaf(f1.y, qa.w, acc);
    acc = fmaf(f2.x, qb.x, acc);
    acc = fmaf(f2.y, qb.y, acc);
    acc = fmaf(f3.x, qb.z, acc);
    acc = fmaf(f3.y, qb.w, acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) scores[row] = acc;
}

// the same dot product for a short list of rows: scores[i] = <bk[rows[i], :], qbar>.  The list travels in the
// kernel parameters; `scores` may live in pinned host memory (the host reads it after an event).
struct RowList {
  int32_t rows[kMaxScoreRows];
};
template <typename T>
__global__ void __launch_bounds__(kScoreWarps * 32)
block_score_rows_kernel(const T* __restrict__ bk, const __grid_constant__ RowList list, int n, int width,
                        const float* __restrict__ qbar, float* __restrict__ scores) {
  const int32_t* rows = list.rows;
  extern __shared__ float sq[];
  for (int i = threadIdx.x; i < width; i += blockDim.x) sq[i] = qbar[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int i = blockIdx.x * kScoreWarps + warp;
  if (i >= n) return;
  const T* p = bk + (int64_t)rows[i] * width;
  float acc = 0.f;
#pragma unroll 4
  for (int c = lane * 8; c < width; c += 32 * 8) {
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(p + c));
    const typename Act<T>::T2* v2 = reinterpret_cast<const typename Act<T>::T2*>(&raw);
    const float4 qa = *reinterpret_cast<const float4*>(sq + c);
    const float4 qb = *reinterpret_cast<const float4*>(sq + c + 4);
    float2 f0 = Act<T>::to_f2(v2[0]), f1 = Act<T>::to_f2(v2[1]), f2 = Act<T>::to_f2(v2[2]),
           f3 = Act<T>::to_f2(v2[3]);
    acc = fmaf(f0.x, qa.x, acc);
    acc = fmaf(f0.y, qa.y, acc);
    acc = fmaf(f1.x, qa.z, acc);
    acc = fmaf(f1.y, qa.w, acc);
    acc = fmaf(f2.x, qb.x, acc);
    acc = fmaf(f2.y, qb.y, acc);
    acc = fmaf(f3.x, qb.z, acc);
    acc = fmaf(f3.y, qb.w, acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) scores[i] = acc;
}

__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float <-> larger key
}

constexpr int kTopkThreads = 1024;

// exclusive scan of one int per thread over the CTA; returns the thread's offset, *total = sum
__device__ int block_exclusive_scan(int v, int* warp_tot /*32*/, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    warp_tot[lane] = winc - w;  // exclusive warp offsets
    if (lane == 31) *total = winc;
  }
  __syncthreads();
  int off = warp_tot[warp] + inc - v;
  __syncthreads();
  return off;
}

__global__ void __launch_bounds__(kTopkThreads)
topk_select_kernel(const float* __restrict__ scores, int64_t n, int k, int id_base, int32_t* __restrict__ out_ids,
                   float* __restrict__ out_scores) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_krem;
  __shared__ int warp_tot[32];
  __shared__ int s_total;
  extern __shared__ unsigned char dyn[];
  uint32_t* ckey = reinterpret_cast<uint32_t*>(dyn);   // k candidate keys
  int32_t* cidx = reinterpret_cast<int32_t*>(ckey + k);  // k candidate ids
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_prefix = 0;
    s_krem = k;
  }
  __syncthreads();
  // radix select, most significant byte first
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < 256; i += kTopkThreads) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    for (int64_t i = tid; i < n; i += kTopkThreads) {
      uint32_t key = float_key(scores[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int krem = s_krem, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= krem) break;
        krem -= hist[b];
      }
      s_krem = krem;
      s_prefix = prefix | ((uint32_t)b << shift);
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;  // key of the k-th largest score
  const int need_eq = s_krem;     // how many keys equal to it belong to the top k
  const int n_gt = k - need_eq;
  // contiguous index chunk per thread keeps "equal" winners in ascending id order
  const int64_t per = (n + kTopkThreads - 1) / kTopkThreads;
  const int64_t lo = per * tid, hi = (lo + per < n) ? lo + per : n;
  int cgt = 0, ceq = 0;
  for (int64_t i = lo; i < hi; ++i) {
    uint32_t key = float_key(scores[i]);
    cgt += key > thr;
    ceq += key == thr;
  }
  int ogt = block_exclusive_scan(cgt, warp_tot, &s_total);
  int oeq = block_exclusive_scan(ceq, warp_tot, &s_total);
  for (int64_t i = lo; i < hi; ++i) {
    uint32_t key = float_key(scores[i]);
    if (key > thr) {
      ckey[ogt] = key;
      cidx[ogt++] = (int32_t)i;
    } else if (key == thr) {
      if (oeq < need_eq) {
        ckey[n_gt + oeq] = key;
        cidx[n_gt + oeq] = (int32_t)i;
      }
      ++oeq;
    }
  }
  __syncthreads();
  // rank sort of the k winners: descending key, ascending id
  for (int i = tid; i < k; i += kTopkThreads) {
    uint32_t ki = ckey[i];
    int32_t ii = cidx[i];
    int rank = 0;
    for (int j = 0; j < k; ++j) {
      uint32_t kj = ckey[j];
      rank += (kj > ki) || (kj == ki && cidx[j] < ii);
    }
    out_ids[rank] = ii + id_base;
    if (out_scores) out_scores[rank] = scores[ii];
  }
}

// ---------------------------------------------------------------------------------------------------------
// Fast path for the usual sizes (k <= 64 over at most 16384 scores), one CTA of 1024 threads.
//
// Every score becomes a 64-bit key: (order-preserving bits of the score) << 32 | ~id, so that a larger key
// means "ranks earlier" (higher score, then lower id) and no two keys are equal.  Thread t keeps the keys of
// scores t, t + 1024, ... in registers; four neighbouring threads form a group of 64 scores.
//   1. tau = the k-th largest of the 256 group maxima, found by counting for every group how many maxima are
//      larger.  tau is a lower bound of the k-th largest key overall, and exactly k groups hold a maximum
//      >= tau.
//   2. every key >= tau is a candidate: at most 64k of them (a few more than k unless the scores are laid out
//      adversarially), appended to a shared list.
//   3. rank sort of the candidates; the first k leave in order.
// No loop waits on data of another CTA.
constexpr int kFastItems = 16;                   // scores per thread: up to 16384 units (2M tokens of 128-token units)
constexpr int kFastMaxK = 64;
constexpr int kFastMaxN = kFastItems * kTopkThreads;
constexpr int kFastGroups = kTopkThreads / 4;
constexpr int kFastCand = 4 * kFastItems * kFastMaxK;  // k groups of 4 threads x kFastItems scores

__device__ __forceinline__ unsigned long long topk_key(float v, int id) {
  if (!(v == v)) v = -INFINITY;  // NaN ranks with -inf
  return ((unsigned long long)float_key(v) << 32) | (uint32_t)(~(uint32_t)id);
}
__device__ __forceinline__ unsigned long long max64(unsigned long long a, unsigned long long b) { return a > b ? a : b; }

// `gm` holds kFastGroups keys, `cand` kFastCand keys, `s_cnt` one int, `s_tau` one key.  All 1024 threads call.
__device__ void cta_topk_fast(const float* scores, int n, int k, int id_base, int32_t* __restrict__ out_ids,
                              float* __restrict__ out_scores, unsigned long long* gm, unsigned long long* cand,
                              int* s_cnt, unsigned long long* s_tau, int32_t* __restrict__ out_ids_copy = nullptr) {
  const int tid = threadIdx.x;
  unsigned long long key[kFastItems];
#pragma unroll
  for (int e = 0; e < kFastItems; ++e) {
    const int i = tid + e * kTopkThreads;
    key[e] = i < n ? topk_key(__ldcg(scores + i), i) : 0ull;  // 0: below every real key
  }
  unsigned long long x = key[0];
#pragma unroll
  for (int e = 1; e < kFastItems; ++e) x = max64(x, key[e]);
  x = max64(x, __shfl_xor_sync(0xffffffffu, x, 1));
  x = max64(x, __shfl_xor_sync(0xffffffffu, x, 2));
  if ((tid & 3) == 0) gm[tid >> 2] = x;
  if (tid == 0) *s_cnt = 0;
  __syncthreads();
  // ---- 1. tau = the k-th largest group maximum: the four threads of a group count, a quarter each, how many
  //         group maxima are larger than their own; the group that counts k - 1 holds tau
  {
    const int q0 = tid & 3;  // interleaved quarters: the four threads read neighbouring words
    int larger = 0;
#pragma unroll 8
    for (int j = 0; j < kFastGroups / 4; ++j) larger += gm[4 * j + q0] > x;
    larger += __shfl_xor_sync(0xffffffffu, larger, 1);
    larger += __shfl_xor_sync(0xffffffffu, larger, 2);
    if ((tid & 3) == 0 && larger == k - 1) *s_tau = x;  // keys are unique (0 only among padding groups, see below)
  }
  __syncthreads();
  const unsigned long long tau = *s_tau;
  // ---- 2. candidates
#pragma unroll
  for (int e = 0; e < kFastItems; ++e)
    if (key[e] >= tau && key[e] != 0ull) {
      int p = atomicAdd(s_cnt, 1);
      if (p < kFastCand) cand[p] = key[e];
    }
  __syncthreads();
  const int nc = *s_cnt < kFastCand ? *s_cnt : kFastCand;  // k <= nc <= 64k
  // ---- 3. rank of every candidate = how many candidates rank before it
  for (int c = tid; c < nc; c += kTopkThreads) {
    const unsigned long long mine = cand[c];
    int rank = 0;
    for (int j = 0; j < nc; ++j) rank += cand[j] > mine;
    if (rank < k) {
      const int id = (int)(~(uint32_t)(mine & 0xffffffffu));
      out_ids[rank] = id + id_base;
      if (out_ids_copy) out_ids_copy[rank] = id + id_base;  // e.g. pinned host memory: no copy behind the kernel
      if (out_scores) out_scores[rank] = __ldcg(scores + id);
    }
  }
}

__global__ void __launch_bounds__(kTopkThreads)
topk_fast_kernel(const float* __restrict__ scores, int n, int k, int id_base, int32_t* __restrict__ out_ids,
                 float* __restrict__ out_scores) {
  __shared__ unsigned long long sm[kFastGroups];
  __shared__ unsigned long long cand[kFastCand];
  __shared__ int s_cnt;
  __shared__ unsigned long long s_tau;
  if (threadIdx.x == 0) s_tau = 0ull;
  cta_topk_fast(scores, n, k, id_base, out_ids, out_scores, sm, cand, &s_cnt, &s_tau);
}

// Scoring and top-k in one launch: CTAs of 32 warps stream the representative keys (one warp per row, the whole
// row's 16-byte loads in flight at once); the CTA that finishes last — known from a ticket counter, nobody
// waits — ranks the scores.  `ticket` must be zero at launch and is zero again when the kernel ends.
template <typename T>
__global__ void __launch_bounds__(kTopkThreads)
block_score_topk_kernel(const T* __restrict__ bk, int n, int width, const float* __restrict__ qbar,
                        float* __restrict__ scores, int k, int id_base, int32_t* __restrict__ out_ids,
                        float* __restrict__ out_scores, unsigned int* __restrict__ ticket,
                        int32_t* __restrict__ out_ids_copy) {
  extern __shared__ __align__(16) unsigned char dyn_raw[];
  float* sq = reinterpret_cast<float*>(dyn_raw);
  __shared__ unsigned long long sm[kFastGroups];
  __shared__ unsigned long long cand[kFastCand];
  __shared__ int s_cnt;
  __shared__ unsigned long long s_tau;
  __shared__ bool s_last;
  chain_enter();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Rows of up to 2048 elements (the usual 4096 needs two rounds of it) live in a rolling buffer of eight 16-byte
  // loads per lane: a piece is consumed and at once replaced by the matching piece of the warp's next row, so that
  // the loads never drain between rows.  The first row's loads go out before the query vector is staged.
  // Consecutive rows go to different SMs, so that a short list still draws on every SM's path to memory.
  const int stride_rows = gridDim.x * 32;
  const int pieces = (width + 2047) / 2048;  // pieces of 32 lanes x 8 loads x 8 elements per row
  int row = warp * gridDim.x + blockIdx.x, piece = 0;
  uint4 raw[8];
  auto issue = [&](int r, int pc) {
    const T* p = bk + (int64_t)r * width + pc * 2048;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = pc * 2048 + (u * 32 + lane) * 8;
      raw[u] = (r < n && c < width) ? __ldcs(reinterpret_cast<const uint4*>(p + (u * 32 + lane) * 8)) : make_uint4(0, 0, 0, 0);
    }
  };
  issue(row, 0);
  for (int i = threadIdx.x; i < width; i += kTopkThreads) sq[i] = qbar[i];
  __syncthreads();
  float acc = 0.f;
  while (row < n) {
    int nrow = row, npiece = piece + 1;
    if (npiece == pieces) {
      npiece = 0;
      nrow = row + stride_rows;
    }
    const bool more = nrow < n;
    const T* np = bk + (int64_t)(more ? nrow : 0) * width + npiece * 2048 + lane * 8;
    const int c0 = piece * 2048 + lane * 8, cn0 = npiece * 2048 + lane * 8;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + u * 256;
      const typename Act<T>::T2* v2 = reinterpret_cast<const typename Act<T>::T2*>(&raw[u]);
      const float2 f0 = Act<T>::to_f2(v2[0]), f1 = Act<T>::to_f2(v2[1]), f2 = Act<T>::to_f2(v2[2]),
                   f3 = Act<T>::to_f2(v2[3]);
      // the slot is free: the matching piece of what comes next is requested before this one is summed
      raw[u] = (more && cn0 + u * 256 < width) ? __ldcs(reinterpret_cast<const uint4*>(np + u * 256)) : make_uint4(0, 0, 0, 0);
      if (c < width) {
        const float4 qa = *reinterpret_cast<const float4*>(sq + c);
        const float4 qb = *reinterpret_cast<const float4*>(sq + c + 4);
        acc = fmaf(f0.x, qa.x, acc);
        acc = fmaf(f0.y, qa.y, acc);
        acc = fmaf(f1.x, qa.z, acc);
        acc = fmaf(f1.y, qa.w, acc);
        acc = fmaf(f2.x, qb.x, acc);
        acc = fmaf(f2.y, qb.y, acc);
        acc = fmaf(f3.x, qb.z, acc);
        acc = fmaf(f3.y, qb.w, acc);
      }
    }
    if (npiece == 0) {  // the row is complete
      acc = warp_sum(acc);
      if (lane == 0) scores[row] = acc;
      acc = 0.f;
    }
    row = nrow;
    piece = npiece;
  }
  __threadfence();  // this warp's scores are visible device-wide before the CTA takes its ticket
  if (!ticket) return;
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) *ticket = 0;
  if (threadIdx.x == 0) s_tau = 0ull;
  cta_topk_fast(scores, n, k, id_base, out_ids, out_scores, sm, cand, &s_cnt, &s_tau, out_ids_copy);
}

template <typename T>
__global__ void repr_select_kernel(const T* __restrict__ k, int64_t k_hs, int64_t k_ts,
                                   const float* __restrict__ score, int64_t score_hs, int64_t tok0,
                                   int block_size, int repr_topk, int group, int head_dim,
                                   T* __restrict__ out, int64_t out_stride) {
  extern __shared__ float sm[];
  float* sc = sm;                                      // block_size scores
  int* sel = reinterpret_cast<int*>(sm + block_size);  // repr_topk winners
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  const int64_t t0 = tok0 + (int64_t)b * block_size;
  for (int i = tid; i < block_size; i += blockDim.x) sc[i] = score[h * score_hs + t0 + i];
  __syncthreads();
  for (int r = 0; r < repr_topk; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < block_size; i += blockDim.x) {
      float v = sc[i];
      if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      red_v[warp] = bv;
      red_i[warp] = bi;
    }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < nwarp; ++w)
        if (red_v[w] > bv || (red_v[w] == bv && red_i[w] < bi)) {
          bv = red_v[w];
          bi = red_i[w];
        }
      if (bi == 0x7fffffff) bi = 0;  // every remaining score is -inf or NaN
      sel[r] = bi;
      sc[bi] = -INFINITY;
    }
    __syncthreads();
  }
  const T* kh = k + (int64_t)(h / group) * k_hs;
  for (int d = tid; d < head_dim; d += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < repr_topk; ++r) acc += Act<T>::to_f(kh[(t0 + sel[r]) * k_ts + d]);
    out[(int64_t)b * out_stride + (int64_t)h * head_dim + d] = Act<T>::from_f(acc / (float)repr_topk);
  }
}

// Device copy of the cache's unit -> slot table (-1: not cached), read by the decode attention when it resolves
// the retrieved units itself.  The host sends the entries that changed as kernel parameters.
constexpr int kMaxTableUpdates = 128;
struct TableUpdates {
  int32_t id[kMaxTableUpdates];
  int32_t slot[kMaxTableUpdates];
};
__global__ void slot_table_update_kernel(int32_t* __restrict__ table, const __grid_constant__ TableUpdates u, int n) {
  const int i = threadIdx.x;
  if (i < n) table[u.id[i]] = u.slot[i];
}

// ids must not repeat within one call
int slot_table_update_launch(int32_t* table, const int32_t* ids, const int32_t* slots, int n, cudaStream_t s) {
  for (int done = 0; done < n; done += kMaxTableUpdates) {
    const int m = n - done < kMaxTableUpdates ? n - done : kMaxTableUpdates;
    TableUpdates u;
    for (int i = 0; i < m; ++i) {
      u.id[i] = ids[done + i];
      u.slot[i] = slots[done + i];
    }
    slot_table_update_kernel<<<1, kMaxTableUpdates, 0, s>>>(table, u, m);
    INFLLM_LAUNCH_OK("slot_table_update_kernel");
  }
  return INFLLM_OK;
}

// the same for the table of unit addresses (unit id -> where its K block lives)
struct PtrUpdates {
  int32_t id[kMaxTableUpdates];
  unsigned long long val[kMaxTableUpdates];
};
__global__ void ptr_table_update_kernel(unsigned long long* __restrict__ table, const __grid_constant__ PtrUpdates u, int n) {
  // scheduled once the kernel before it has passed its own wait: everything older is complete, and what follows this
  // kernel may be scheduled at once (the attention starts on the keys that need no table)
  chain_trigger();
  chain_wait();
  const int i = threadIdx.x;
  if (i < n) table[u.id[i]] = u.val[i];
}

int ptr_table_update_launch(unsigned long long* table, const int32_t* ids, const unsigned long long* vals, int n,
                            cudaStream_t s) {
  for (int done = 0; done < n; done += kMaxTableUpdates) {
    const int m = n - done < kMaxTableUpdates ? n - done : kMaxTableUpdates;
    PtrUpdates u;
    for (int i = 0; i < m; ++i) {
      u.id[i] = ids[done + i];
      u.val[i] = vals[done + i];
    }
    launch_chained(ptr_table_update_kernel, dim3(1), dim3(kMaxTableUpdates), 0, s, table, u, m);
    INFLLM_LAUNCH_OK("ptr_table_update_kernel");
  }
  return INFLLM_OK;
}

// out_ids_copy (may be null; honoured only by the one-launch form, i.e. with a ticket, k <= 64, n <= 16384): a second
// place for the ids, written by the same threads - pinned host memory saves the copy behind the kernel
int block_topk_launch(const void* bk, int64_t n, int width, const float* qbar, float* scores, int k, int id_base,
                      int32_t* out_ids, float* out_scores, int dtype, cudaStream_t s, unsigned int* ticket,
                      int32_t* out_ids_copy) {
  if (out_ids_copy && !(ticket && k <= kFastMaxK && n <= kFastMaxN))
    return fail(INFLLM_E_UNSUPPORTED, "block_topk: a second id destination needs the one-launch form");
  if (n <= 0 || k <= 0 || k > n) return fail(INFLLM_E_BADARG, "block_topk: need 0 < k <= n_blocks (k=%d n=%lld)", k, (long long)n);
  if (k > 1024) return fail(INFLLM_E_UNSUPPORTED, "block_topk: k=%d > 1024", k);
  if (width % 8 != 0 || width > 12 * 1024 || ((uintptr_t)bk % 16) != 0)
    return fail(INFLLM_E_BADARG, "block_topk: width %d must be a multiple of 8, at most 12288, rows 16-byte aligned", width);
  if (k <= kFastMaxK && n <= kFastMaxN) {
    // one launch when the caller lends a ticket counter, else scoring and ranking back to back
    const unsigned grid = (unsigned)std::min<int64_t>(n, 148);
    const size_t smem = width * sizeof(float);
    INFLLM_DISPATCH_DTYPE(dtype, T, {
      auto kern = block_score_topk_kernel<T>;
      // the kernel's static shared memory (ranking scratch) plus the query vector passes the 48 KiB a launch gets
      // without asking
      // (asked for at every launch: the opt-in holds for the current device only)
      INFLLM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      launch_chained(kern, dim3(grid), dim3(kTopkThreads), smem, s, (const T*)bk, (int)n, width, qbar, scores, k, id_base,
                     out_ids, out_scores, ticket, out_ids_copy);
    });
    INFLLM_LAUNCH_OK("block_score_topk_kernel");
    if (!ticket) {
      topk_fast_kernel<<<1, kTopkThreads, 0, s>>>(scores, (int)n, k, id_base, out_ids, out_scores);
      INFLLM_LAUNCH_OK("topk_fast_kernel");
    }
    return INFLLM_OK;
  }
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    block_score_kernel<T><<<(unsigned)ceil_div(n, kScoreWarps), kScoreWarps * 32, width * sizeof(float), s>>>(
        (const T*)bk, n, width, qbar, scores);
  });
  INFLLM_LAUNCH_OK("block_score_kernel");
  topk_select_kernel<<<1, kTopkThreads, k * 8, s>>>(scores, n, k, id_base, out_ids, out_scores);
  INFLLM_LAUNCH_OK("topk_select_kernel");
  return INFLLM_OK;
}

// the two halves of block_topk_launch on their own, for callers that put an exchange between them (the sum of the
// scores over the ranks of a KV-head-group sharding)
int block_score_launch(const void* bk, int64_t n, int width, const float* qbar, float* scores, int dtype,
                       cudaStream_t s) {
  if (n <= 0) return INFLLM_OK;
  if (width % 8 != 0 || width > 12 * 1024 || ((uintptr_t)bk % 16) != 0)
    return fail(INFLLM_E_BADARG, "block_score: width %d must be a multiple of 8, at most 12288, rows 16-byte aligned", width);
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    block_score_kernel<T><<<(unsigned)ceil_div(n, kScoreWarps), kScoreWarps * 32, width * sizeof(float), s>>>(
        (const T*)bk, n, width, qbar, scores);
  });
  INFLLM_LAUNCH_OK("block_score_kernel");
  return INFLLM_OK;
}

int topk_launch(const float* scores, int64_t n, int k, int id_base, int32_t* out_ids, float* out_scores,
                cudaStream_t s) {
  if (n <= 0 || k <= 0 || k > n) return fail(INFLLM_E_BADARG, "topk: need 0 < k <= n (k=%d n=%lld)", k, (long long)n);
  if (k > 1024) return fail(INFLLM_E_UNSUPPORTED, "topk: k=%d > 1024", k);
  if (k <= kFastMaxK && n <= kFastMaxN) {
    topk_fast_kernel<<<1, kTopkThreads, 0, s>>>(scores, (int)n, k, id_base, out_ids, out_scores);
    INFLLM_LAUNCH_OK("topk_fast_kernel");
  } else {
    topk_select_kernel<<<1, kTopkThreads, k * 8, s>>>(scores, n, k, id_base, out_ids, out_scores);
    INFLLM_LAUNCH_OK("topk_select_kernel");
  }
  return INFLLM_OK;
}

int block_score_rows_launch(const void* bk, const int32_t* rows, int n, int width, const float* qbar, float* scores,
                            int dtype, cudaStream_t s) {
  for (int done = 0; done < n; done += kMaxScoreRows) {  // `rows` is a host array
    const int m = n - done < kMaxScoreRows ? n - done : kMaxScoreRows;
    RowList list;
    for (int i = 0; i < m; ++i) list.rows[i] = rows[done + i];
    INFLLM_DISPATCH_DTYPE(dtype, T, {
      block_score_rows_kernel<T><<<(unsigned)ceil_div(m, kScoreWarps), kScoreWarps * 32, width * sizeof(float), s>>>(
          (const T*)bk, list, m, width, qbar, scores + done);
    });
    INFLLM_LAUNCH_OK("block_score_rows_kernel");
  }
  return INFLLM_OK;
}

int repr_select_launch(const void* k, int64_t k_hs, int64_t k_ts, const float* score, int64_t score_hs,
                       int64_t tok0, int n_new, int block_size, int repr_topk, int n_heads, int n_kv_heads,
                       int head_dim, void* out, int dtype, cudaStream_t s) {
  if (n_new <= 0) return INFLLM_OK;
  if (repr_topk <= 0 || repr_topk > block_size) return fail(INFLLM_E_BADARG, "repr_select: repr_topk %d vs block_size %d", repr_topk, block_size);
  if (n_heads % n_kv_heads) return fail(INFLLM_E_BADARG, "repr_select: heads %d / kv heads %d", n_heads, n_kv_heads);
  dim3 grid(n_new, n_heads);
  size_t smem = block_size * sizeof(float) + repr_topk * sizeof(int);
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    repr_select_kernel<T><<<grid, 128, smem, s>>>((const T*)k, k_hs, k_ts, score, score_hs, tok0, block_size,
                                                  repr_topk, n_heads / n_kv_heads, head_dim, (T*)out,
                                                  (int64_t)n_heads * head_dim);
  });
  INFLLM_LAUNCH_OK("repr_select_kernel");
  return INFLLM_OK;
}

}  // namespace infllm

extern "C" int infllm_block_topk(const void* d_block_k, int64_t n_blocks, int width, const float* d_qbar,
                                 float* d_scores, int k, int id_base, int32_t* d_out_ids, float* d_out_scores,
                                 int dtype, void* stream) {
  using namespace infllm;
  if (!d_block_k || !d_qbar || !d_scores || !d_out_ids) return fail(INFLLM_E_BADARG, "block_topk: null pointer");
  return block_topk_launch(d_block_k, n_blocks, width, d_qbar, d_scores, k, id_base, d_out_ids, d_out_scores, dtype,
                           (cudaStream_t)stream, nullptr, nullptr);
}

extern "C" int infllm_repr_select(const void* d_k, int64_t k_hs, int64_t k_ts, const float* d_score,
                                  int64_t score_hs, int64_t tok0, int n_new, int block_size, int repr_topk,
                                  int n_heads, int n_kv_heads, int head_dim, void* d_block_k_out, int dtype,
                                  void* stream) {
  using namespace infllm;
  if (!d_k || !d_score || !d_block_k_out) return fail(INFLLM_E_BADARG, "repr_select: null pointer");
  return repr_select_launch(d_k, k_hs, k_ts, d_score, score_hs, tok0, n_new, block_size, repr_topk, n_heads,
                            n_kv_heads, head_dim, d_block_k_out, dtype, (cudaStream_t)stream);
}

extern "C" int infllm_block_score_rows(const void* d_block_k, const int32_t* h_rows, int n, int width,
                                       const float* d_qbar, float* d_scores, int dtype, void* stream) {
  using namespace infllm;
  if (!d_block_k || !h_rows || !d_qbar || !d_scores || n < 0) return fail(INFLLM_E_BADARG, "block_score_rows: bad argument");
  if (width % 8 != 0 || width > 12 * 1024) return fail(INFLLM_E_BADARG, "block_score_rows: width %d", width);
  return block_score_rows_launch(d_block_k, h_rows, n, width, d_qbar, d_scores, dtype, (cudaStream_t)stream);
}

extern "C" int infllm_ptr_table_update(uint64_t* d_table, const int32_t* h_ids, const uint64_t* h_addrs, int n, void* stream) {
  using namespace infllm;
  if (!d_table || (n > 0 && (!h_ids || !h_addrs)) || n < 0) return fail(INFLLM_E_BADARG, "ptr_table_update: bad argument");
  static_assert(sizeof(uint64_t) == sizeof(unsigned long long), "64-bit table entries");
  return ptr_table_update_launch(reinterpret_cast<unsigned long long*>(d_table), h_ids,
                                 reinterpret_cast<const unsigned long long*>(h_addrs), n, (cudaStream_t)stream);
}

// d_table[h_ids[i]] = h_slots[i] for i < n on `stream` (ids must not repeat); -1 marks "not cached"
extern "C" int infllm_slot_table_update(int32_t* d_table, const int32_t* h_ids, const int32_t* h_slots, int n,
                                        void* stream) {
  using namespace infllm;
  if (!d_table || (n > 0 && (!h_ids || !h_slots)) || n < 0) return fail(INFLLM_E_BADARG, "slot_table_update: bad argument");
  return slot_table_update_launch(d_table, h_ids, h_slots, n, (cudaStream_t)stream);
}
