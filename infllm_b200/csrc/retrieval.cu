// Retrieval kernels: memory-unit scoring + top-k, and representative-key selection at sealing.
//
// block_score_kernel  HBM-streaming GEMV (one warp per representative-key row, 16-byte loads,
//                     query mean staged in shared memory, fp32 accumulation).
// topk_argmax_kernel  k <= 64 over <= 8192 scores: per-thread register sort, per-warp pops, one final warp merge.
// topk_select_kernel  any size: 4-pass 8-bit radix select of the k-th largest score, then an
//                     index-ordered gather of the winners and a rank sort.  Both: descending score,
//                     ties to the lower id.
// repr_select_kernel  per (new unit, query head): repr_topk arg-max rounds over the accumulated
//                     local scores, gather + mean of the chosen un-rotated keys.
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

// Small k (the usual topk of 16-64) over at most 8192 scores, one CTA of 32 warps.  Every thread sorts its 8
// strided scores in registers; every warp then pops its k best by repeatedly taking the best of the 32 lane
// heads (warp shuffles only); finally warp 0 pops the k best of the 32 sorted warp lists.  No CTA-wide
// barrier inside the loops.  Order: descending score, ties to the lower id (NaN scores rank last).
constexpr int kArgmaxItems = 8;
struct ScoreId {
  float v;
  int i;
};
__device__ __forceinline__ bool before(float av, int ai, float bv, int bi) {
  return av > bv || (av == bv && ai < bi);
}
__global__ void __launch_bounds__(kTopkThreads)
topk_argmax_kernel(const float* __restrict__ scores, int n, int k, int id_base, int32_t* __restrict__ out_ids,
                   float* __restrict__ out_scores) {
  extern __shared__ unsigned char dyn[];
  float* cv = reinterpret_cast<float*>(dyn);           // [32 warps][k] values
  int* ci = reinterpret_cast<int*>(cv + 32 * k);        // [32 warps][k] ids
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float v[kArgmaxItems];
  int id[kArgmaxItems];
#pragma unroll
  for (int e = 0; e < kArgmaxItems; ++e) {
    int i = tid + e * kTopkThreads;
    float x = i < n ? scores[i] : -INFINITY;
    v[e] = (x == x) ? x : -INFINITY;
    id[e] = i < n ? i : 0x7fffffff;
  }
  // odd-even transposition sort of the 8 register pairs, best first
#pragma unroll
  for (int pass = 0; pass < kArgmaxItems; ++pass) {
#pragma unroll
    for (int e = pass & 1; e + 1 < kArgmaxItems; e += 2) {
      if (before(v[e + 1], id[e + 1], v[e], id[e])) {
        float tv = v[e]; v[e] = v[e + 1]; v[e + 1] = tv;
        int ti = id[e]; id[e] = id[e + 1]; id[e + 1] = ti;
      }
    }
  }
  // the warp's k best: pop the best lane head k times
  for (int r = 0; r < k; ++r) {
    float bv = v[0];
    int bi = id[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (before(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      cv[warp * k + r] = bv;
      ci[warp * k + r] = bi;
    }
    if (id[0] == bi && bi != 0x7fffffff) {  // this lane owned the winner: shift its list up
#pragma unroll
      for (int e = 0; e + 1 < kArgmaxItems; ++e) {
        v[e] = v[e + 1];
        id[e] = id[e + 1];
      }
      v[kArgmaxItems - 1] = -INFINITY;
      id[kArgmaxItems - 1] = 0x7fffffff;
    }
  }
  __syncthreads();
  if (warp == 0) {
    int head = 0;  // lane l walks warp l's sorted list
    for (int r = 0; r < k; ++r) {
      float hv = head < k ? cv[lane * k + head] : -INFINITY;
      int hi = head < k ? ci[lane * k + head] : 0x7fffffff;
      float bv = hv;
      int bi = hi;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (before(ov, oi, bv, bi)) {
          bv = ov;
          bi = oi;
        }
      }
      if (hi == bi && bi != 0x7fffffff) ++head;
      if (lane == 0) {
        out_ids[r] = (bi == 0x7fffffff ? 0 : bi) + id_base;
        if (out_scores) out_scores[r] = bv;
      }
    }
  }
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

int block_topk_launch(const void* bk, int64_t n, int width, const float* qbar, float* scores, int k, int id_base,
                      int32_t* out_ids, float* out_scores, int dtype, cudaStream_t s) {
  if (n <= 0 || k <= 0 || k > n) return fail(INFLLM_E_BADARG, "block_topk: need 0 < k <= n_blocks (k=%d n=%lld)", k, (long long)n);
  if (k > 1024) return fail(INFLLM_E_UNSUPPORTED, "block_topk: k=%d > 1024", k);
  if (width % 8 != 0 || width > 12 * 1024 || ((uintptr_t)bk % 16) != 0)
    return fail(INFLLM_E_BADARG, "block_topk: width %d must be a multiple of 8, at most 12288, rows 16-byte aligned", width);
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    block_score_kernel<T><<<(unsigned)ceil_div(n, kScoreWarps), kScoreWarps * 32, width * sizeof(float), s>>>(
        (const T*)bk, n, width, qbar, scores);
  });
  INFLLM_LAUNCH_OK("block_score_kernel");
  if (k <= 64 && n <= (int64_t)kArgmaxItems * kTopkThreads) {
    topk_argmax_kernel<<<1, kTopkThreads, 32 * k * 8, s>>>(scores, (int)n, k, id_base, out_ids, out_scores);
    INFLLM_LAUNCH_OK("topk_argmax_kernel");
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
                           (cudaStream_t)stream);
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
