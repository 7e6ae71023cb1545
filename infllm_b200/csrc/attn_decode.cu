// Decode attention: one query token per head over a list of key/value segments.
//
// HBM-streaming split-K: the keys of all segments are cut into chunks of kDecodeChunk tokens; one CTA
// handles one chunk of one KV head for all the query heads of its group, reading each K and V row
// exactly once with 16-byte loads (a half-warp covers one 256-byte row).  Each CTA writes a
// normalised partial output and its log-sum-exp; infllm_lse_merge combines partials — the chunks of one
// GPU and, for unit-range sharding, the partials gathered from other GPUs.
// Replaces the two attn.append calls of ContextManager._append (context_manager.py:486-489, 526-531)
// for single-token exec blocks.
#include "attn_common.cuh"

namespace infllm {

constexpr int kDecodeChunk = 128;
constexpr int kDecodeThreads = 128;
constexpr int kMaxGroup = 8;  // query heads per KV head

struct DecodeSeg {
  const void* k;
  const void* v;
  int64_t hs;
  int32_t ts;
  int32_t len;
};

struct DecodeParams {
  DecodeSeg seg[kMaxSeg];
  int32_t part_begin[kMaxSeg + 1];  // first partial index of each segment
  uint8_t qsel[kMaxSeg];            // query variant per segment
  int32_t n_seg, n_heads, n_kv_heads;
  int32_t logit_seg;  // segment whose raw logits are exported, or -1
  const void* q[2];   // (H, D) each, heads q_hs elements apart
  int64_t q_hs;
  float* part_o;      // (n_part, H, D)
  float* part_lse;    // (n_part, H)
  float* logits;      // (H, seg_len[logit_seg])
  float scale_log2;
};

template <int HD, typename T>
__global__ void __launch_bounds__(kDecodeThreads)
attn_decode_kernel(const __grid_constant__ DecodeParams P) {
  static_assert(HD == 128, "one half-warp covers a 128-element row");
  __shared__ float s_q[kMaxGroup][HD];
  __shared__ float s_p[kMaxGroup][kDecodeChunk];
  __shared__ float s_o[kDecodeThreads / 16][kMaxGroup][HD / 8][8 + 1];  // [half-warp][head][16-byte chunk][element]
  __shared__ float s_m[kMaxGroup], s_l[kMaxGroup];

  const int part = blockIdx.x, hkv = blockIdx.y;
  const int group = P.n_heads / P.n_kv_heads;
  int sg = 0;
  while (sg + 1 < P.n_seg && P.part_begin[sg + 1] <= part) ++sg;
  const DecodeSeg& S = P.seg[sg];
  const int j0 = (part - P.part_begin[sg]) * kDecodeChunk;
  const int nk = (S.len - j0) < kDecodeChunk ? (S.len - j0) : kDecodeChunk;
  const T* qsrc = (const T*)P.q[P.qsel[sg]];
  for (int i = threadIdx.x; i < group * HD; i += kDecodeThreads) {
    int gi = i / HD, d = i % HD;
    s_q[gi][d] = Act<T>::to_f(qsrc[(int64_t)(hkv * group + gi) * P.q_hs + d]);
  }
  __syncthreads();

  const int hw = threadIdx.x >> 4;  // half-warp index 0..7
  const int l16 = threadIdx.x & 15; // lane within the half-warp: owns elements [l16*8, l16*8+8)
  const T* kbase = (const T*)S.k + (int64_t)hkv * S.hs + (int64_t)j0 * S.ts + l16 * 8;
  const T* vbase = (const T*)S.v + (int64_t)hkv * S.hs + (int64_t)j0 * S.ts + l16 * 8;

  // ---- logits: s[g][j] = <q_g, k_j> * scale
  for (int j = hw; j < kDecodeChunk; j += kDecodeThreads / 16) {
    float part_dot[kMaxGroup];
#pragma unroll
    for (int gi = 0; gi < kMaxGroup; ++gi) part_dot[gi] = 0.f;
    if (j < nk) {
      uint4 raw = __ldg(reinterpret_cast<const uint4*>(kbase + (int64_t)j * S.ts));
      const typename Act<T>::T2* k2 = reinterpret_cast<const typename Act<T>::T2*>(&raw);
      float kf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = Act<T>::to_f2(k2[e]);
        kf[2 * e] = f.x;
        kf[2 * e + 1] = f.y;
      }
#pragma unroll
      for (int gi = 0; gi < kMaxGroup; ++gi) {
        if (gi < group) {
          float a = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) a = fmaf(kf[e], s_q[gi][l16 * 8 + e], a);
          part_dot[gi] = a;
        }
      }
    }
#pragma unroll
    for (int gi = 0; gi < kMaxGroup; ++gi) {
      if (gi < group) {
        float a = part_dot[gi];
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        a += __shfl_xor_sync(0xffffffffu, a, 4);
        a += __shfl_xor_sync(0xffffffffu, a, 8);
        if (l16 == 0) s_p[gi][j] = j < nk ? a * P.scale_log2 : -INFINITY;
      }
    }
  }
  __syncthreads();
  if (sg == P.logit_seg) {
    for (int i = threadIdx.x; i < group * nk; i += kDecodeThreads) {
      int gi = i / nk, j = i % nk;
      P.logits[(int64_t)(hkv * group + gi) * S.len + j0 + j] = s_p[gi][j];
    }
  }
  // ---- softmax over the chunk: one warp per query head (looping if the group is larger than 4)
  {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int gi = warp; gi < group; gi += kDecodeThreads / 32) {
      float mx = -INFINITY;
      for (int j = lane; j < kDecodeChunk; j += 32) mx = fmaxf(mx, s_p[gi][j]);
      mx = warp_max(mx);
      float sum = 0.f;
      for (int j = lane; j < kDecodeChunk; j += 32) {
        float pv = exp2f(s_p[gi][j] - mx);
        s_p[gi][j] = pv;
        sum += pv;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        s_m[gi] = mx;
        s_l[gi] = sum;
      }
    }
  }
  __syncthreads();
  // ---- o[g][d] = sum_j p[g][j] v[j][d]
  float acc[kMaxGroup][8];
#pragma unroll
  for (int gi = 0; gi < kMaxGroup; ++gi)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[gi][e] = 0.f;
  for (int j = hw; j < nk; j += kDecodeThreads / 16) {
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(vbase + (int64_t)j * S.ts));
    const typename Act<T>::T2* v2 = reinterpret_cast<const typename Act<T>::T2*>(&raw);
    float vf[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = Act<T>::to_f2(v2[e]);
      vf[2 * e] = f.x;
      vf[2 * e + 1] = f.y;
    }
#pragma unroll
    for (int gi = 0; gi < kMaxGroup; ++gi) {
      if (gi < group) {
        float pv = s_p[gi][j];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[gi][e] = fmaf(pv, vf[e], acc[gi][e]);
      }
    }
  }
#pragma unroll
  for (int gi = 0; gi < kMaxGroup; ++gi)
    if (gi < group)
#pragma unroll
      for (int e = 0; e < 8; ++e) s_o[hw][gi][l16][e] = acc[gi][e];
  __syncthreads();
  for (int i = threadIdx.x; i < group * HD; i += kDecodeThreads) {
    int gi = i / HD, d = i % HD;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeThreads / 16; ++w) v += s_o[w][gi][d >> 3][d & 7];
    int h = hkv * group + gi;
    P.part_o[((int64_t)part * P.n_heads + h) * HD + d] = v / s_l[gi];
    if (d == 0) P.part_lse[(int64_t)part * P.n_heads + h] = s_m[gi] + log2f(s_l[gi]);
  }
}

// out[h, :] = sum_p w_p o_p / sum_p w_p with w_p = exp2(lse_p - max lse); lse = max + log2(sum w)
template <typename T>
__global__ void lse_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, int n_part,
                                 int n_heads, int head_dim, T* __restrict__ out, int64_t o_hs,
                                 float* __restrict__ lse) {
  const int h = blockIdx.x;
  float mx = -INFINITY;
  for (int p = 0; p < n_part; ++p) mx = fmaxf(mx, part_lse[(int64_t)p * n_heads + h]);
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float num = 0.f, den = 0.f;
    if (mx != -INFINITY) {
      for (int p = 0; p < n_part; ++p) {
        float w = exp2f(part_lse[(int64_t)p * n_heads + h] - mx);
        den += w;
        num = fmaf(w, part_o[((int64_t)p * n_heads + h) * head_dim + d], num);
      }
    }
    out[(int64_t)h * o_hs + d] = Act<T>::from_f(den > 0.f ? num / den : 0.f);
    if (d == 0 && lse) lse[h] = den > 0.f ? mx + log2f(den) : -INFINITY;
  }
}

// score[h, j] += exp2(logit[h, j] - lse[h]): the local-stage column sums of a one-token exec block
__global__ void decode_score_kernel(const float* __restrict__ logits, int64_t len, const float* __restrict__ lse,
                                    float* __restrict__ score, int64_t score_hs) {
  int h = blockIdx.y;
  int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= len) return;
  score[h * score_hs + j] += exp2f(logits[h * len + j] - lse[h]);
}

int decode_score_launch(const float* logits, int64_t len, const float* lse, float* score, int64_t score_hs,
                        int n_heads, cudaStream_t s) {
  if (len <= 0) return INFLLM_OK;
  dim3 grid((unsigned)ceil_div(len, 256), n_heads);
  decode_score_kernel<<<grid, 256, 0, s>>>(logits, len, lse, score, score_hs);
  INFLLM_LAUNCH_OK("decode_score_kernel");
  return INFLLM_OK;
}

int attn_decode_launch(const void* q0, const void* q1, int64_t q_hs, int n_heads, int n_kv_heads, int head_dim, int n_seg,
                       const KvSeg* segs, const int32_t* seg_q, float* part_o, float* part_lse, int max_parts,
                       int* n_parts_out, int logit_seg, float* logits, int dtype, cudaStream_t s) {
  if (head_dim != 128) return fail(INFLLM_E_UNSUPPORTED, "decode attention: head_dim %d (128 is built)", head_dim);
  if (n_heads % n_kv_heads || n_heads / n_kv_heads > kMaxGroup)
    return fail(INFLLM_E_UNSUPPORTED, "decode attention: %d query heads per kv head (at most %d)",
                n_kv_heads ? n_heads / n_kv_heads : 0, kMaxGroup);
  if (n_seg <= 0 || n_seg > kMaxSeg) return fail(INFLLM_E_BADARG, "decode attention: %d segments (1..%d)", n_seg, kMaxSeg);
  DecodeParams P{};
  int parts = 0, ns = 0;
  int logit_seg_packed = -1;
  for (int i = 0; i < n_seg; ++i) {
    if (segs[i].len <= 0) continue;  // empty segments contribute nothing
    if (((uintptr_t)segs[i].k | (uintptr_t)segs[i].v) % 16 || segs[i].hs % 8 || segs[i].ts % 8)
      return fail(INFLLM_E_BADARG, "decode attention: segment %d rows are not 16-byte aligned", i);
    P.seg[ns] = {segs[i].k, segs[i].v, segs[i].hs, segs[i].ts, segs[i].len};
    P.qsel[ns] = (uint8_t)(seg_q[i] ? 1 : 0);
    P.part_begin[ns] = parts;
    if (i == logit_seg) logit_seg_packed = ns;
    parts += (int)ceil_div(segs[i].len, kDecodeChunk);
    ++ns;
  }
  P.part_begin[ns] = parts;
  if (n_parts_out) *n_parts_out = parts;
  if (parts == 0) return INFLLM_OK;
  if (parts > max_parts) return fail(INFLLM_E_CAPACITY, "decode attention: %d partials exceed the scratch for %d", parts, max_parts);
  P.n_seg = ns; P.n_heads = n_heads; P.n_kv_heads = n_kv_heads; P.logit_seg = logit_seg_packed;
  P.q[0] = q0; P.q[1] = q1 ? q1 : q0; P.q_hs = q_hs;
  P.part_o = part_o; P.part_lse = part_lse; P.logits = logits;
  P.scale_log2 = kLog2e / sqrtf((float)head_dim);
  dim3 grid(parts, n_kv_heads);
  INFLLM_DISPATCH_DTYPE(dtype, T, { attn_decode_kernel<128, T><<<grid, kDecodeThreads, 0, s>>>(P); });
  INFLLM_LAUNCH_OK("attn_decode_kernel");
  return INFLLM_OK;
}

int lse_merge_launch(const float* part_o, const float* part_lse, int n_part, int n_heads, int head_dim, void* out,
                     int64_t o_hs, float* lse, int dtype, cudaStream_t s) {
  if (n_part <= 0) return fail(INFLLM_E_BADARG, "lse_merge: no partials");
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    lse_merge_kernel<T><<<n_heads, 128, 0, s>>>(part_o, part_lse, n_part, n_heads, head_dim, (T*)out, o_hs, lse);
  });
  INFLLM_LAUNCH_OK("lse_merge_kernel");
  return INFLLM_OK;
}

}  // namespace infllm

extern "C" int64_t infllm_attn_decode_max_parts(int n_seg, int64_t total_keys) {
  return total_keys / infllm::kDecodeChunk + n_seg + 1;
}

extern "C" int infllm_attn_decode(const void* d_q0, const void* d_q1, int n_heads, int n_kv_heads, int head_dim,
                                  int n_seg, const void* const* h_seg_k, const void* const* h_seg_v,
                                  const int64_t* h_seg_hs, const int32_t* h_seg_len, const int32_t* h_seg_q,
                                  float* d_part_o, float* d_part_lse, int max_parts, int* n_parts,
                                  int logit_seg, float* d_logits, int dtype, void* stream) {
  using namespace infllm;
  if (!d_q0 || !h_seg_k || !h_seg_v || !h_seg_hs || !h_seg_len || !h_seg_q || !d_part_o || !d_part_lse)
    return fail(INFLLM_E_BADARG, "attn_decode: null pointer");
  if (n_seg <= 0 || n_seg > kMaxSeg) return fail(INFLLM_E_BADARG, "attn_decode: %d segments (1..%d)", n_seg, kMaxSeg);
  if (logit_seg >= 0 && !d_logits) return fail(INFLLM_E_BADARG, "attn_decode: logits requested without a buffer");
  KvSeg segs[kMaxSeg];
  for (int i = 0; i < n_seg; ++i) segs[i] = {h_seg_k[i], h_seg_v[i], h_seg_hs[i], head_dim, h_seg_len[i]};
  return attn_decode_launch(d_q0, d_q1, head_dim, n_heads, n_kv_heads, head_dim, n_seg, segs, h_seg_q, d_part_o, d_part_lse,
                            max_parts, n_parts, logit_seg, d_logits, dtype, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------ allocation-free variant
// Scratch for infllm_attn_decode_noalloc: the split-K partials live in this file-scope array instead of
// a caller-provided buffer.  Every GPU that loads the library holds these bytes until the process exits.
constexpr int kStaticMaxParts = 160;  // 160 chunks of 128 keys
constexpr int kStaticMaxHeads = 64;
constexpr size_t kStaticFloats = (size_t)kStaticMaxParts * kStaticMaxHeads * (128 + 1);  // outputs + log-sum-exps
static __device__ __align__(256) float g_decode_scratch[kStaticFloats];
// device addresses of the array, one per device ordinal, looked up on the first call made on that device
static float* g_decode_scratch_ptr[64] = {nullptr};

extern "C" int infllm_attn_decode_noalloc(const void* d_q0, const void* d_q1, int n_heads, int n_kv_heads,
                                          int head_dim, int n_seg, const void* const* h_seg_k,
                                          const void* const* h_seg_v, const int64_t* h_seg_hs,
                                          const int32_t* h_seg_len, const int32_t* h_seg_q, void* d_out, int64_t o_hs,
                                          float* d_lse, int dtype, void* stream) {
  using namespace infllm;
  if (!d_q0 || !h_seg_k || !h_seg_v || !h_seg_hs || !h_seg_len || !h_seg_q || !d_out)
    return fail(INFLLM_E_BADARG, "attn_decode_noalloc: null pointer");
  if (n_seg <= 0 || n_seg > kMaxSeg)
    return fail(INFLLM_E_BADARG, "attn_decode_noalloc: %d segments (1..%d)", n_seg, kMaxSeg);
  if (head_dim != 128) return fail(INFLLM_E_UNSUPPORTED, "attn_decode_noalloc: head_dim %d (128 is built)", head_dim);
  if (n_heads <= 0 || n_heads > kStaticMaxHeads)
    return fail(INFLLM_E_CAPACITY, "attn_decode_noalloc: %d heads exceed the built-in scratch for %d", n_heads,
                kStaticMaxHeads);
  long parts = 0;
  for (int i = 0; i < n_seg; ++i)
    if (h_seg_len[i] > 0) parts += (h_seg_len[i] + kDecodeChunk - 1) / kDecodeChunk;
  if (parts > kStaticMaxParts)
    return fail(INFLLM_E_CAPACITY,
                "attn_decode_noalloc: %ld chunks of %d keys exceed the built-in scratch for %d chunks; use "
                "infllm_attn_decode with a caller-provided buffer", parts, kDecodeChunk, kStaticMaxParts);
  if (parts == 0) return fail(INFLLM_E_BADARG, "attn_decode_noalloc: no keys");
  int dev = 0;
  INFLLM_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(INFLLM_E_UNSUPPORTED, "attn_decode_noalloc: device ordinal %d", dev);
  if (!g_decode_scratch_ptr[dev]) {
    // In host code the array's name is only a handle; the kernels need its address on the current device.
    float* p = nullptr;
    INFLLM_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_decode_scratch));
    g_decode_scratch_ptr[dev] = p;
  }
  float* part_o = g_decode_scratch_ptr[dev];
  float* part_lse = part_o + (size_t)kStaticMaxParts * kStaticMaxHeads * 128;
  KvSeg segs[kMaxSeg];
  for (int i = 0; i < n_seg; ++i) segs[i] = {h_seg_k[i], h_seg_v[i], h_seg_hs[i], head_dim, h_seg_len[i]};
  int n_parts = 0;
  cudaStream_t s = (cudaStream_t)stream;
  // Nothing in the scratch has to start at zero: every partial the merge reads is written by the
  // split-K kernel of this same call, whatever an earlier call left behind.
  INFLLM_TRY(attn_decode_launch(d_q0, d_q1, head_dim, n_heads, n_kv_heads, head_dim, n_seg, segs, h_seg_q, part_o,
                                part_lse, kStaticMaxParts, &n_parts, -1, nullptr, dtype, s));
  return lse_merge_launch(part_o, part_lse, n_parts, n_heads, head_dim, d_out, o_hs, d_lse, dtype, s);
}

extern "C" int infllm_lse_merge(const float* d_part_o, const float* d_part_lse, int n_part, int n_heads,
                                int head_dim, void* d_out, int64_t o_hs, float* d_lse, int dtype, void* stream) {
  using namespace infllm;
  if (!d_part_o || !d_part_lse || !d_out) return fail(INFLLM_E_BADARG, "lse_merge: null pointer");
  return lse_merge_launch(d_part_o, d_part_lse, n_part, n_heads, head_dim, d_out, o_hs, d_lse, dtype,
                          (cudaStream_t)stream);
}
