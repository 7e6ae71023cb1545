// Rotary position embedding kernels.
// Follows RotaryEmbeddingESM of the reference (inf_llm/attention/rope.py): half-rotation layout,
// fp32 tables of angle = (t * scale) * inv_freq, fp32 products added and rounded once to the
// activation type.  HBM-bound elementwise work: 16-byte loads/stores, one thread per 8+8 elements.
#include <algorithm>

#include "common.cuh"

namespace infllm {

__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float scale, int half, int64_t length,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= length * half) return;
  int64_t t = idx / half;
  int f = (int)(idx - t * half);
  float ang = __fmul_rn(__fmul_rn((float)t, scale), inv_freq[f]);  // rope.py:53-55
  cos_t[idx] = cosf(ang);
  sin_t[idx] = sinf(ang);
}

// x (H, L, D) strided -> out (H, L, D) strided, row t rotated to position pos0 + t*pos_step.
template <typename T>
__global__ void rope_apply_kernel(const T* __restrict__ x, int64_t x_hs, int64_t x_ts, T* __restrict__ out,
                                  int64_t o_hs, int64_t o_ts, int n_heads, int64_t len, int head_dim,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  int64_t pos0, int pos_step) {
  const int half = head_dim / 2;
  const int chunks = half / 8;  // 16-byte chunks per half row
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)n_heads * len * chunks;
  if (idx >= total) return;
  int c = (int)(idx % chunks);
  int64_t t = (idx / chunks) % len;
  int h = (int)(idx / ((int64_t)chunks * len));
  const T* src = x + h * x_hs + t * x_ts + c * 8;
  T* dst = out + h * o_hs + t * o_ts + c * 8;
  int64_t pos = pos0 + t * pos_step;
  const float* cs = cos_t + pos * half + c * 8;
  const float* sn = sin_t + pos * half + c * 8;
  uint4 lo = *reinterpret_cast<const uint4*>(src);
  uint4 hi = *reinterpret_cast<const uint4*>(src + half);
  const T* a = reinterpret_cast<const T*>(&lo);
  const T* b = reinterpret_cast<const T*>(&hi);
  uint4 olo, ohi;
  T* oa = reinterpret_cast<T*>(&olo);
  T* ob = reinterpret_cast<T*>(&ohi);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float x1 = Act<T>::to_f(a[i]), x2 = Act<T>::to_f(b[i]);
    float cv = cs[i], sv = sn[i];
    // (x * cos) + (rotate_half(x) * sin), each product rounded to fp32 first (rope.py:47)
    oa[i] = Act<T>::from_f(__fadd_rn(__fmul_rn(x1, cv), __fmul_rn(-x2, sv)));
    ob[i] = Act<T>::from_f(__fadd_rn(__fmul_rn(x2, cv), __fmul_rn(x1, sv)));
  }
  *reinterpret_cast<uint4*>(dst) = olo;
  *reinterpret_cast<uint4*>(dst + half) = ohi;
}

// plain strided row copy (H, L, D) -> (H, L, D), 16 bytes per thread
template <typename T>
__global__ void copy_rows_kernel(const T* __restrict__ x, int64_t x_hs, int64_t x_ts, T* __restrict__ out,
                                 int64_t o_hs, int64_t o_ts, int n_heads, int64_t len, int head_dim) {
  const int chunks = head_dim / 8;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)n_heads * len * chunks;
  if (idx >= total) return;
  int c = (int)(idx % chunks);
  int64_t t = (idx / chunks) % len;
  int h = (int)(idx / ((int64_t)chunks * len));
  *reinterpret_cast<uint4*>(out + h * o_hs + t * o_ts + c * 8) =
      *reinterpret_cast<const uint4*>(x + h * x_hs + t * x_ts + c * 8);
}

// mean over the rows of each exec block of the one-angle-rotated queries:
// qbar[e, h*D + d] = mean_t q[h, e*exc + t, d]  (context_manager.py:373-375), fp32.
template <typename T>
__global__ void qbar_kernel(const T* __restrict__ q, int64_t q_hs, int64_t q_ts, int64_t len, int exc,
                            int head_dim, float* __restrict__ qbar, int64_t qbar_stride) {
  int e = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  int64_t st = (int64_t)e * exc;
  int64_t ed = st + exc < len ? st + exc : len;
  float acc = 0.f;
  const T* p = q + h * q_hs + d;
  for (int64_t t = st; t < ed; ++t) acc += Act<T>::to_f(p[t * q_ts]);
  qbar[e * qbar_stride + (int64_t)h * head_dim + d] = acc / (float)(ed - st);
}

// K and V of n_new consecutive units -> the host store's unit layout [unit][K|V][head][token][d], contiguous,
// so that one device-to-host copy moves all of them
__global__ void pack_units_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, int64_t hs16, int64_t tok0,
                                  int n_new, int block_size, int n_kv_heads, int d16, uint4* __restrict__ out) {
  const int64_t per_head = (int64_t)block_size * d16;  // 16-byte chunks of one head of one unit
  const int64_t per_half = per_head * n_kv_heads;
  const int64_t total = 2 * per_half * n_new;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t u = i / (2 * per_half), r = i % (2 * per_half);
    int is_v = r >= per_half;
    r -= is_v ? per_half : 0;
    int64_t hh = r / per_head, w = r % per_head;
    const uint4* src = (is_v ? v : k) + hh * hs16 + (tok0 + u * block_size) * d16 + w;
    out[i] = *src;
  }
}

int pack_units_launch(const void* k, const void* v, int64_t hs, int64_t tok0, int n_new, int block_size, int n_kv_heads,
                      int head_dim, void* out, cudaStream_t s) {
  if (n_new <= 0) return INFLLM_OK;
  const int64_t total = 2ll * n_new * n_kv_heads * block_size * (head_dim / 8);
  int blocks = (int)std::min<int64_t>(ceil_div(total, 256), 1184);
  pack_units_kernel<<<blocks, 256, 0, s>>>((const uint4*)k, (const uint4*)v, hs / 8, tok0, n_new, block_size,
                                           n_kv_heads, head_dim / 8, (uint4*)out);
  INFLLM_LAUNCH_OK("pack_units_kernel");
  return INFLLM_OK;
}

// Refill copy of whole units into cache slots by the SMs: one CTA of 256 threads per unit, four 16-byte loads in
// flight per thread, one launch per batch.  The context uses it for units that have a copy in device memory.  It
// also works on the pinned host store (the host pointers are device-visible under unified addressing) and gets
// 49 GB/s out of the link where one 512 KiB cudaMemcpyAsync per unit gets 38 GB/s, but its CTAs then hold SM
// resources for the length of the transfer, which cost a concurrent exec-block attention more than the faster
// copies gained; host-resident units therefore go through the copy engine.
constexpr int kMaxStageUnits = 64;
struct StageList {
  const uint4* src[kMaxStageUnits];
  uint4* dst[kMaxStageUnits];
};
constexpr int kStageThreads = 256;
__global__ void __launch_bounds__(kStageThreads) stage_units_kernel(const __grid_constant__ StageList list, int n16) {
  const uint4* __restrict__ src = list.src[blockIdx.x];
  uint4* __restrict__ dst = list.dst[blockIdx.x];
  int i = threadIdx.x;
  for (; i + 3 * kStageThreads < n16; i += 4 * kStageThreads) {
    const uint4 a = __ldcs(src + i), b = __ldcs(src + i + kStageThreads), c = __ldcs(src + i + 2 * kStageThreads),
                d = __ldcs(src + i + 3 * kStageThreads);
    dst[i] = a;
    dst[i + kStageThreads] = b;
    dst[i + 2 * kStageThreads] = c;
    dst[i + 3 * kStageThreads] = d;
  }
  for (; i < n16; i += kStageThreads) dst[i] = __ldcs(src + i);
}

int stage_units_launch(const void* const* h_src, void* const* d_dst, int n, int64_t unit_bytes, cudaStream_t s) {
  for (int done = 0; done < n; done += kMaxStageUnits) {
    const int m = n - done < kMaxStageUnits ? n - done : kMaxStageUnits;
    StageList list;
    for (int i = 0; i < m; ++i) {
      list.src[i] = (const uint4*)h_src[done + i];
      list.dst[i] = (uint4*)d_dst[done + i];
    }
    stage_units_kernel<<<m, kStageThreads, 0, s>>>(list, (int)(unit_bytes / 16));
    INFLLM_LAUNCH_OK("stage_units_kernel");
  }
  return INFLLM_OK;
}

// One new token (decode): what the per-token launches of an append do — copy K and V into the token buffers,
// rotate K to its window position, rotate Q both ways, take the query "mean" of the one-token exec block and
// clear the token's score column — as one launch.  CTA b < n_heads handles query head b, the others one KV
// head each; thread i owns the element pair (i, i + head_dim/2).  Same arithmetic as rope_apply_kernel.
template <typename T>
__global__ void ingest_token_kernel(const T* __restrict__ q, int64_t q_hs, const T* __restrict__ k, int64_t k_hs,
                                    const T* __restrict__ v, int64_t v_hs, T* __restrict__ q_loc,
                                    T* __restrict__ q_glb, int64_t qs_hs, float* __restrict__ qbar,
                                    T* __restrict__ k_raw, T* __restrict__ k_rot, T* __restrict__ v_out,
                                    int64_t kv_hs, float* __restrict__ score, int64_t score_hs, int n_heads,
                                    int head_dim, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                    int64_t pos_loc, int64_t pos_glb, int32_t* __restrict__ clear) {
  chain_enter();
  const int half = head_dim / 2, i = threadIdx.x, b = blockIdx.x;
  if (clear && b == 0 && i == 0) *clear = 0;  // the "retrieved unit not cached" flag of this token's attention
  if (i >= half) return;
  const float cl = cos_t[pos_loc * half + i], sl = sin_t[pos_loc * half + i];
  if (b < n_heads) {
    const float x1 = Act<T>::to_f(q[b * q_hs + i]), x2 = Act<T>::to_f(q[b * q_hs + i + half]);
    const float cg = cos_t[pos_glb * half + i], sg = sin_t[pos_glb * half + i];
    q_loc[b * qs_hs + i] = Act<T>::from_f(__fadd_rn(__fmul_rn(x1, cl), __fmul_rn(-x2, sl)));
    q_loc[b * qs_hs + i + half] = Act<T>::from_f(__fadd_rn(__fmul_rn(x2, cl), __fmul_rn(x1, sl)));
    const T g1 = Act<T>::from_f(__fadd_rn(__fmul_rn(x1, cg), __fmul_rn(-x2, sg)));
    const T g2 = Act<T>::from_f(__fadd_rn(__fmul_rn(x2, cg), __fmul_rn(x1, sg)));
    q_glb[b * qs_hs + i] = g1;
    q_glb[b * qs_hs + i + half] = g2;
    qbar[(int64_t)b * head_dim + i] = Act<T>::to_f(g1);
    qbar[(int64_t)b * head_dim + i + half] = Act<T>::to_f(g2);
    if (i == 0) score[b * score_hs] = 0.f;
  } else {
    const int hk = b - n_heads;
    const T r1 = k[hk * k_hs + i], r2 = k[hk * k_hs + i + half];
    k_raw[hk * kv_hs + i] = r1;
    k_raw[hk * kv_hs + i + half] = r2;
    v_out[hk * kv_hs + i] = v[hk * v_hs + i];
    v_out[hk * kv_hs + i + half] = v[hk * v_hs + i + half];
    const float x1 = Act<T>::to_f(r1), x2 = Act<T>::to_f(r2);
    k_rot[hk * kv_hs + i] = Act<T>::from_f(__fadd_rn(__fmul_rn(x1, cl), __fmul_rn(-x2, sl)));
    k_rot[hk * kv_hs + i + half] = Act<T>::from_f(__fadd_rn(__fmul_rn(x2, cl), __fmul_rn(x1, sl)));
  }
}

int ingest_token_launch(const void* q, int64_t q_hs, const void* k, int64_t k_hs, const void* v, int64_t v_hs,
                        void* q_loc, void* q_glb, int64_t qs_hs, float* qbar, void* k_raw, void* k_rot, void* v_out,
                        int64_t kv_hs, float* score, int64_t score_hs, int n_heads, int n_kv_heads, int head_dim,
                        const float* cos_t, const float* sin_t, int64_t table_len, int64_t pos_loc, int64_t pos_glb,
                        int dtype, cudaStream_t s, int32_t* clear) {
  if (head_dim % 2 || head_dim > 2048) return fail(INFLLM_E_BADARG, "ingest: head_dim %d", head_dim);
  if (pos_loc < 0 || pos_loc >= table_len || pos_glb < 0 || pos_glb >= table_len)
    return fail(INFLLM_E_BADARG, "ingest: positions %lld / %lld outside the table of %lld rows", (long long)pos_loc,
                (long long)pos_glb, (long long)table_len);
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    launch_chained(ingest_token_kernel<T>, dim3(n_heads + n_kv_heads), dim3(head_dim / 2), 0, s,
        (const T*)q, q_hs, (const T*)k, k_hs, (const T*)v, v_hs, (T*)q_loc, (T*)q_glb, qs_hs, qbar, (T*)k_raw, (T*)k_rot,
        (T*)v_out, kv_hs, score, score_hs, n_heads, head_dim, cos_t, sin_t, pos_loc, pos_glb, clear);
  });
  INFLLM_LAUNCH_OK("ingest_token_kernel");
  return INFLLM_OK;
}

int rope_apply_launch(const void* x, int64_t x_hs, int64_t x_ts, void* out, int64_t o_hs, int64_t o_ts,
                      int n_heads, int64_t len, int head_dim, const float* cos_t, const float* sin_t,
                      int64_t table_len, int64_t pos0, int pos_step, int dtype, cudaStream_t s) {
  if (len == 0) return INFLLM_OK;
  if (head_dim % 16 != 0) return fail(INFLLM_E_BADARG, "rope: head_dim %d is not a multiple of 16", head_dim);
  if (pos0 < 0 || pos0 + (len - 1) * pos_step >= table_len)
    return fail(INFLLM_E_BADARG, "rope: positions [%lld, %lld] outside the table of %lld rows", (long long)pos0,
                (long long)(pos0 + (len - 1) * pos_step), (long long)table_len);
  if ((x_hs | x_ts | o_hs | o_ts) % 8 != 0 || ((uintptr_t)x | (uintptr_t)out) % 16 != 0)
    return fail(INFLLM_E_BADARG, "rope: rows must be 16-byte aligned");
  int64_t total = (int64_t)n_heads * len * (head_dim / 16);
  int threads = 256;
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    rope_apply_kernel<T><<<(unsigned)ceil_div(total, threads), threads, 0, s>>>(
        (const T*)x, x_hs, x_ts, (T*)out, o_hs, o_ts, n_heads, len, head_dim, cos_t, sin_t, pos0, pos_step);
  });
  INFLLM_LAUNCH_OK("rope_apply_kernel");
  return INFLLM_OK;
}

int copy_rows_launch(const void* x, int64_t x_hs, int64_t x_ts, void* out, int64_t o_hs, int64_t o_ts,
                     int n_heads, int64_t len, int head_dim, cudaStream_t s) {
  if (len == 0) return INFLLM_OK;
  if ((x_hs | x_ts | o_hs | o_ts) % 8 != 0 || ((uintptr_t)x | (uintptr_t)out) % 16 != 0 || head_dim % 8)
    return fail(INFLLM_E_BADARG, "copy_rows: rows must be 16-byte aligned");
  int64_t total = (int64_t)n_heads * len * (head_dim / 8);
  copy_rows_kernel<__half><<<(unsigned)ceil_div(total, 256), 256, 0, s>>>(
      (const __half*)x, x_hs, x_ts, (__half*)out, o_hs, o_ts, n_heads, len, head_dim);
  INFLLM_LAUNCH_OK("copy_rows_kernel");
  return INFLLM_OK;
}

int qbar_launch(const void* q, int64_t q_hs, int64_t q_ts, int n_heads, int64_t len, int exc, int head_dim,
                float* qbar, int64_t qbar_stride, int dtype, cudaStream_t s) {
  if (len == 0) return INFLLM_OK;
  dim3 grid((unsigned)ceil_div(len, exc), n_heads);
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    qbar_kernel<T><<<grid, head_dim, 0, s>>>((const T*)q, q_hs, q_ts, len, exc, head_dim, qbar, qbar_stride);
  });
  INFLLM_LAUNCH_OK("qbar_kernel");
  return INFLLM_OK;
}

}  // namespace infllm

extern "C" int infllm_rope_table(const float* h_inv_freq, float scale, int head_dim, int64_t length,
                                 float* d_cos, float* d_sin, void* stream) {
  using namespace infllm;
  if (!h_inv_freq || !d_cos || !d_sin || head_dim <= 0 || head_dim % 2 || length <= 0)
    return fail(INFLLM_E_BADARG, "rope_table: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  int half = head_dim / 2;
  float* d_inv = nullptr;
  INFLLM_CUDA_OK(cudaMallocAsync(&d_inv, half * sizeof(float), s));
  INFLLM_CUDA_OK(cudaMemcpyAsync(d_inv, h_inv_freq, half * sizeof(float), cudaMemcpyHostToDevice, s));
  int64_t total = length * half;
  rope_table_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, s>>>(d_inv, scale, half, length, d_cos, d_sin);
  INFLLM_LAUNCH_OK("rope_table_kernel");
  INFLLM_CUDA_OK(cudaFreeAsync(d_inv, s));
  return INFLLM_OK;
}

extern "C" int infllm_rope_apply(const void* d_x, int64_t x_hs, int64_t x_ts, void* d_out, int64_t o_hs,
                                 int64_t o_ts, int n_heads, int64_t len, int head_dim, const float* d_cos,
                                 const float* d_sin, int64_t table_len, int64_t pos0, int pos_step, int dtype,
                                 void* stream) {
  using namespace infllm;
  if (!d_x || !d_out || !d_cos || !d_sin) return fail(INFLLM_E_BADARG, "rope_apply: null pointer");
  return rope_apply_launch(d_x, x_hs, x_ts, d_out, o_hs, o_ts, n_heads, len, head_dim, d_cos, d_sin, table_len,
                           pos0, pos_step, dtype, (cudaStream_t)stream);
}

extern "C" int infllm_ingest_token(const void* d_q, int64_t q_hs, const void* d_k, int64_t k_hs, const void* d_v,
                                   int64_t v_hs, void* d_q_loc, void* d_q_glb, int64_t qs_hs, float* d_qbar,
                                   void* d_k_raw, void* d_k_rot, void* d_v_out, int64_t kv_hs, float* d_score,
                                   int64_t score_hs, int n_heads, int n_kv_heads, int head_dim, const float* d_cos,
                                   const float* d_sin, int64_t table_len, int64_t pos_local, int64_t pos_global,
                                   int dtype, void* stream) {
  using namespace infllm;
  if (!d_q || !d_k || !d_v || !d_q_loc || !d_q_glb || !d_qbar || !d_k_raw || !d_k_rot || !d_v_out || !d_score || !d_cos ||
      !d_sin)
    return fail(INFLLM_E_BADARG, "ingest_token: null pointer");
  if (n_heads <= 0 || n_kv_heads <= 0) return fail(INFLLM_E_BADARG, "ingest_token: %d / %d heads", n_heads, n_kv_heads);
  return ingest_token_launch(d_q, q_hs, d_k, k_hs, d_v, v_hs, d_q_loc, d_q_glb, qs_hs, d_qbar, d_k_raw, d_k_rot, d_v_out,
                             kv_hs, d_score, score_hs, n_heads, n_kv_heads, head_dim, d_cos, d_sin, table_len, pos_local,
                             pos_global, dtype, (cudaStream_t)stream, nullptr);
}
