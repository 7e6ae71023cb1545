// Decode attention: one query token per head over a list of key/value segments.
//
// HBM-streaming split-K: the keys of all segments are cut into chunks (128 tokens through the C entry points,
// 64 inside the context, which wants more CTAs in flight); one single-warp CTA handles one chunk of one KV
// head for all the query heads of its group, reading each K and V row exactly once with 16-byte cp.async
// copies that are all issued before the first is used.  Each CTA writes a
// normalised partial output and its log-sum-exp; infllm_lse_merge combines partials — the chunks of one
// GPU and, for unit-range sharding, the partials gathered from other GPUs.
// Replaces the two attn.append calls of ContextManager._append (context_manager.py:486-489, 526-531)
// for single-token exec blocks.
#include "attn_common.cuh"
#include "mma_common.cuh"

namespace infllm {

constexpr int kDecodeChunk = 128;
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
  DecodeIndirect ind; // n_units == 0: every segment carries its own pointers
};

// wait until at most n of this thread's cp.async groups are pending (n is a constant after unrolling)
__device__ __forceinline__ void cp_wait_upto(int n) {
  if (n <= 0) mma::cp_async_wait<0>();
  else if (n == 1) mma::cp_async_wait<1>();
  else if (n == 2) mma::cp_async_wait<2>();
  else mma::cp_async_wait<3>();
  __syncwarp();  // the other lanes' copies are visible too
}

// One warp per CTA and per chunk of 64 * ROUNDS keys of one KV head.  The warp first issues every 16-byte
// cp.async of its K and V rows (32 KiB per round, XOR-swizzled tiles in shared memory), so that a full SM holds
// about 200 KiB of loads in flight, then runs S = Q K^T and O = P V on the tensor cores (mma.sync m16n8k16: the
// query heads of the group are the first rows of the 16-row operand, the rest is zero) with the softmax of the
// chunk in registers in between.
template <int HD, int ROUNDS, typename T>
__global__ void __launch_bounds__(32) attn_decode_kernel(const __grid_constant__ DecodeParams P) {
  static_assert(HD == 128, "tiles of 64 keys x 128 elements");
  using namespace mma;
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int kTileBytes = 64 * HD * 2;
  constexpr int kChunk = 64 * ROUNDS;
  const uint32_t s0 = smem_u32(smem);
  const int lane = threadIdx.x, g = lane >> 2, t4 = lane & 3;
  const int part = blockIdx.x, hkv = blockIdx.y;
  const int group = P.n_heads / P.n_kv_heads;
  int sg = 0;
  while (sg + 1 < P.n_seg && P.part_begin[sg + 1] <= part) ++sg;
  const DecodeSeg& S = P.seg[sg];
  const int j0 = (part - P.part_begin[sg]) * kChunk;
  const int nk = (S.len - j0) < kChunk ? (S.len - j0) : kChunk;
  const void* seg_k = S.k;
  const void* seg_v = S.v;
  if (P.ind.n_units > 0) {
    const int u = sg - P.ind.first_seg;
    if (u >= 0 && u < P.ind.n_units) {
      const int id = __ldg(P.ind.ids + u) - P.ind.id_lo;
      const bool mine = id >= 0 && id < P.ind.n_owned;
      const int slot = mine ? __ldg(P.ind.table + id) : -1;
      if (slot < 0) {
        // not cached: this chunk's partials get weight zero here; the host launches the unit again after the
        // refill.  A unit that another rank owns is that rank's business.
        if (lane == 0 && mine) *P.ind.miss = 1;
        const int grp = P.n_heads / P.n_kv_heads;
        for (int i = lane; i < grp * HD; i += 32)
          P.part_o[((int64_t)part * P.n_heads + hkv * grp + i / HD) * HD + i % HD] = 0.f;
        if (lane < grp) P.part_lse[(int64_t)part * P.n_heads + hkv * grp + lane] = -INFINITY;
        return;
      }
      seg_k = P.ind.cache + (int64_t)slot * P.ind.unit_bytes;
      seg_v = (const char*)seg_k + P.ind.unit_bytes / 2;
    }
  }
  const T* kbase = (const T*)seg_k + (int64_t)hkv * S.hs + (int64_t)j0 * S.ts;
  const T* vbase = (const T*)seg_v + (int64_t)hkv * S.hs + (int64_t)j0 * S.ts;
  // ---- all loads of the chunk: groups K0, V0, K1, V1 ...; rows past the end are zero-filled
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
#pragma unroll
    for (int kv = 0; kv < 2; ++kv) {
      const T* base = kv ? vbase : kbase;
      const uint32_t dst = s0 + (uint32_t)((2 * r + kv) * kTileBytes);
#pragma unroll 8
      for (int i = 0; i < 64 * (HD / 8) / 32; ++i) {
        const int idx = lane + 32 * i, row = idx / (HD / 8), c = idx % (HD / 8);
        const int jr = r * 64 + row;
        const bool ok = jr < nk;
        cp_async16(dst + tile_off<HD>(row, c), base + (ok ? (int64_t)jr * S.ts : 0) + c * 8, ok);
      }
      cp_async_commit();
    }
  }
  // ---- the group's queries as A fragments: row g of the operand is head hkv * group + g, rows >= group are zero
  const bool qrow = g < group;
  const int h = hkv * group + (qrow ? g : 0);
  const T* qp = (const T*)P.q[P.qsel[sg]] + (int64_t)h * P.q_hs;
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    qf[ks][0] = qrow ? __ldg(reinterpret_cast<const uint32_t*>(qp + ks * 16 + t4 * 2)) : 0u;
    qf[ks][2] = qrow ? __ldg(reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + t4 * 2)) : 0u;
    qf[ks][1] = qf[ks][3] = 0u;
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m = -INFINITY, l = 0.f;  // l: this thread's share of the row sum, reduced over the quad at the end
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const uint32_t kt = s0 + (uint32_t)(2 * r * kTileBytes), vt = kt + kTileBytes;
    cp_wait_upto(2 * ROUNDS - 1 - 2 * r);
    float sacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        const int mid = lane >> 3;
        const int rr = np * 16 + (mid >> 1) * 8 + (lane & 7), c = ks * 2 + (mid & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kt + tile_off<HD>(rr, c), b0, b1, b2, b3);
        mma16816<T>(sacc[np * 2], qf[ks], b0, b1);
        mma16816<T>(sacc[np * 2 + 1], qf[ks], b2, b3);
      }
    }
    // scale, cut at the end of the segment, softmax of this round against the running maximum
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = r * 64 + i * 8 + t4 * 2 + e;
        const float v = j < nk ? sacc[i][e] * P.scale_log2 : -INFINITY;
        sacc[i][e] = v;
        mx = fmaxf(mx, v);
        if (sg == P.logit_seg && qrow && j < nk) P.logits[(int64_t)h * S.len + j0 + j] = v;
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m, mx);
    const float ms = mn == -INFINITY ? 0.f : mn;
    const float al = exp2f(m - ms);
    m = mn;
    float rs = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sacc[i][0] = exp2f(sacc[i][0] - ms);
      sacc[i][1] = exp2f(sacc[i][1] - ms);
      rs += sacc[i][0] + sacc[i][1];
    }
    l = l * al + rs;
    if (r > 0) {
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= al;
        o[i][1] *= al;
      }
    }
    cp_wait_upto(2 * ROUNDS - 2 - 2 * r);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t pa[4];
      pa[0] = pack2<T>(sacc[2 * ks][0], sacc[2 * ks][1]);
      pa[2] = pack2<T>(sacc[2 * ks + 1][0], sacc[2 * ks + 1][1]);
      pa[1] = pa[3] = 0u;
#pragma unroll
      for (int dn = 0; dn < HD / 16; ++dn) {
        const int mid = lane >> 3;
        const int rr = ks * 16 + (mid & 1) * 8 + (lane & 7), c = dn * 2 + (mid >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vt + tile_off<HD>(rr, c), b0, b1, b2, b3);
        mma16816<T>(o[dn * 2], pa, b0, b1);
        mma16816<T>(o[dn * 2 + 1], pa, b2, b3);
      }
    }
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (qrow) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float* po = P.part_o + ((int64_t)part * P.n_heads + h) * HD + t4 * 2;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) *reinterpret_cast<float2*>(po + i * 8) = make_float2(o[i][0] * inv, o[i][1] * inv);
    if (t4 == 0) P.part_lse[(int64_t)part * P.n_heads + h] = l > 0.f ? m + log2f(l) : -INFINITY;
  }
}

// out[h, :] = sum_p w_p o_p / sum_p w_p with w_p = exp2(lse_p - max lse); lse = max + log2(sum w).
// One CTA per head: kMergeGroups groups of head_dim threads share the partials, eight loads in flight each.
// With `logits` the CTA then adds this token's local attention row into the accumulated scores:
// score[h, j] += exp2(logit[h, j] - lse[h]) — the column sums of a one-token exec block.
constexpr int kMergeGroups = 8;
constexpr int kMergeUnroll = 20;  // partials a thread keeps in flight: 8 groups x 20 cover 160 partials
constexpr int kMergeCols = 4;     // score columns a thread keeps in flight: 4 x 1024 cover a 4096-token window
template <typename T>
__global__ void __launch_bounds__(1024)
lse_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, int n_part, int n_heads,
                 int head_dim, T* __restrict__ out, int64_t o_hs, float* __restrict__ lse,
                 const float* __restrict__ logits, int64_t logit_len, float* __restrict__ score, int64_t score_hs,
                 const int32_t* __restrict__ skip, int64_t o_ps, int64_t lse_ps) {
  extern __shared__ float s_w[];  // n_part weights
  if (skip && *skip) return;  // the partials were not written: a retrieved unit was not cached
  __shared__ float s_red[32];
  __shared__ float s_num[kMergeGroups][128];
  __shared__ float s_mx, s_den;
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  const int grp = tid / head_dim, d = tid % head_dim, ngrp = blockDim.x / head_dim;
  // every global load of the common case is issued before the first one is needed
  const float* po = part_o + (int64_t)h * head_dim + d;
  const int64_t ps = o_ps;  // floats from one partial to the next
  float pv[kMergeUnroll];
#pragma unroll
  for (int u = 0; u < kMergeUnroll; ++u) {
    const int p = grp + u * ngrp;
    pv[u] = p < n_part ? __ldcs(po + (int64_t)p * ps) : 0.f;
  }
  float lg[kMergeCols], sc[kMergeCols];
#pragma unroll
  for (int i = 0; i < kMergeCols; ++i) {
    const int64_t j = tid + (int64_t)i * blockDim.x;
    const bool ok = logits != nullptr && j < logit_len;
    lg[i] = ok ? __ldcs(logits + h * logit_len + j) : 0.f;
    sc[i] = ok ? score[h * score_hs + j] : 0.f;
  }
  float mx = -INFINITY;
  for (int p = tid; p < n_part; p += blockDim.x) {
    const float v = part_lse[(int64_t)p * lse_ps + h];
    s_w[p] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    float v = lane < nwarp ? s_red[lane] : -INFINITY;
    v = warp_max(v);
    if (lane == 0) s_mx = v;
  }
  __syncthreads();
  mx = s_mx;
  float den = 0.f;
  if (mx != -INFINITY)
    for (int p = tid; p < n_part; p += blockDim.x) {
      const float w = exp2f(s_w[p] - mx);
      s_w[p] = w;
      den += w;
    }
  den = warp_sum(den);
  __syncthreads();
  if (lane == 0) s_red[warp] = den;
  __syncthreads();
  if (warp == 0) {
    float v = lane < nwarp ? s_red[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) s_den = v;
  }
  __syncthreads();
  den = s_den;
  float num = 0.f;
  if (mx != -INFINITY) {
#pragma unroll
    for (int u = 0; u < kMergeUnroll; ++u) {
      const int p = grp + u * ngrp;
      if (p < n_part) num = fmaf(s_w[p], pv[u], num);
    }
    for (int p = grp + kMergeUnroll * ngrp; p < n_part; p += ngrp) num = fmaf(s_w[p], __ldcs(po + (int64_t)p * ps), num);
  }
  s_num[grp][d] = num;
  __syncthreads();
  if (tid < head_dim) {
    float tot = 0.f;
    for (int g2 = 0; g2 < ngrp; ++g2) tot += s_num[g2][tid];
    out[(int64_t)h * o_hs + tid] = Act<T>::from_f(den > 0.f ? tot / den : 0.f);
  }
  const float l = den > 0.f ? mx + log2f(den) : -INFINITY;
  if (tid == 0 && lse) lse[h] = l;
  if (logits) {
#pragma unroll
    for (int i = 0; i < kMergeCols; ++i) {
      const int64_t j = tid + (int64_t)i * blockDim.x;
      if (j < logit_len) score[h * score_hs + j] = sc[i] + exp2f(lg[i] - l);
    }
    for (int64_t j = tid + (int64_t)kMergeCols * blockDim.x; j < logit_len; j += blockDim.x)
      score[h * score_hs + j] += exp2f(logits[h * logit_len + j] - l);
  }
}

int attn_decode_launch(const void* q0, const void* q1, int64_t q_hs, int n_heads, int n_kv_heads, int head_dim, int n_seg,
                       const KvSeg* segs, const int32_t* seg_q, float* part_o, float* part_lse, int max_parts,
                       int* n_parts_out, int logit_seg, float* logits, int dtype, cudaStream_t s, int chunk,
                       const DecodeIndirect* ind, int part_base) {
  if (chunk != 64 && chunk != 128) return fail(INFLLM_E_BADARG, "decode attention: chunk %d (64 or 128)", chunk);
  if (head_dim != 128) return fail(INFLLM_E_UNSUPPORTED, "decode attention: head_dim %d (128 is built)", head_dim);
  if (n_heads <= 0 || n_kv_heads <= 0)
    return fail(INFLLM_E_BADARG, "decode attention: %d query heads / %d kv heads", n_heads, n_kv_heads);
  if (n_heads % n_kv_heads || n_heads / n_kv_heads > kMaxGroup)
    return fail(INFLLM_E_UNSUPPORTED, "decode attention: %d query heads per kv head (at most %d)",
                n_heads / n_kv_heads, kMaxGroup);
  if (n_seg <= 0 || n_seg > kMaxSeg) return fail(INFLLM_E_BADARG, "decode attention: %d segments (1..%d)", n_seg, kMaxSeg);
  DecodeParams P{};
  if (ind && ind->n_units > 0) {
    if (!ind->ids || !ind->table || !ind->cache || !ind->miss || ind->first_seg < 0 ||
        ind->first_seg + ind->n_units > n_seg)
      return fail(INFLLM_E_BADARG, "decode attention: bad device-resolved unit list");
    for (int i = 0; i < ind->n_units; ++i)
      if (segs[ind->first_seg + i].len <= 0) return fail(INFLLM_E_BADARG, "decode attention: empty unit segment");
    P.ind = *ind;
  }
  int parts = 0, ns = 0;
  int logit_seg_packed = -1;
  for (int i = 0; i < n_seg; ++i) {
    if (segs[i].len <= 0) continue;  // empty segments contribute nothing
    if (ind && ind->n_units > 0 && i == ind->first_seg) P.ind.first_seg = ns;
    if (((uintptr_t)segs[i].k | (uintptr_t)segs[i].v) % 16 || segs[i].hs % 8 || segs[i].ts % 8)
      return fail(INFLLM_E_BADARG, "decode attention: segment %d rows are not 16-byte aligned", i);
    P.seg[ns] = {segs[i].k, segs[i].v, segs[i].hs, segs[i].ts, segs[i].len};
    P.qsel[ns] = (uint8_t)(seg_q[i] ? 1 : 0);
    P.part_begin[ns] = parts;
    if (i == logit_seg) logit_seg_packed = ns;
    parts += (int)ceil_div(segs[i].len, chunk);
    ++ns;
  }
  P.part_begin[ns] = parts;
  if (n_parts_out) *n_parts_out = parts;
  if (parts == 0) return INFLLM_OK;
  if (part_base < 0 || part_base + parts > max_parts)
    return fail(INFLLM_E_CAPACITY, "decode attention: %d partials exceed the scratch for %d", part_base + parts, max_parts);
  P.n_seg = ns; P.n_heads = n_heads; P.n_kv_heads = n_kv_heads; P.logit_seg = logit_seg_packed;
  P.q[0] = q0; P.q[1] = q1 ? q1 : q0; P.q_hs = q_hs;
  P.part_o = part_o + (int64_t)part_base * n_heads * head_dim;
  P.part_lse = part_lse + (int64_t)part_base * n_heads;
  P.logits = logits;
  P.scale_log2 = kLog2e / sqrtf((float)head_dim);
  dim3 grid(parts, n_kv_heads);
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    if (chunk == 64) {
      attn_decode_kernel<128, 1, T><<<grid, 32, 32 * 1024, s>>>(P);
    } else {
      auto kern = attn_decode_kernel<128, 2, T>;
      INFLLM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
      kern<<<grid, 32, 64 * 1024, s>>>(P);
    }
  });
  INFLLM_LAUNCH_OK("attn_decode_kernel");
  return INFLLM_OK;
}

int lse_merge_launch(const float* part_o, const float* part_lse, int n_part, int n_heads, int head_dim, void* out,
                     int64_t o_hs, float* lse, int dtype, cudaStream_t s, const float* logits, int64_t logit_len,
                     float* score, int64_t score_hs, const int32_t* skip, int64_t o_ps, int64_t lse_ps) {
  if (o_ps <= 0) o_ps = (int64_t)n_heads * head_dim;
  if (lse_ps <= 0) lse_ps = n_heads;
  if (n_part <= 0) return fail(INFLLM_E_BADARG, "lse_merge: no partials");
  if (n_part > 8192) return fail(INFLLM_E_CAPACITY, "lse_merge: %d partials (at most 8192)", n_part);
  if (head_dim <= 0 || head_dim > 128 || head_dim % 32)
    return fail(INFLLM_E_UNSUPPORTED, "lse_merge: head_dim %d (a multiple of 32, at most 128)", head_dim);
  if (dtype == INFLLM_F32) {
    lse_merge_kernel<float><<<n_heads, kMergeGroups * head_dim, n_part * sizeof(float), s>>>(
        part_o, part_lse, n_part, n_heads, head_dim, (float*)out, o_hs, lse, logits, logit_len, score, score_hs, skip,
        o_ps, lse_ps);
  } else {
    INFLLM_DISPATCH_DTYPE(dtype, T, {
      lse_merge_kernel<T><<<n_heads, kMergeGroups * head_dim, n_part * sizeof(float), s>>>(
          part_o, part_lse, n_part, n_heads, head_dim, (T*)out, o_hs, lse, logits, logit_len, score, score_hs, skip,
          o_ps, lse_ps);
    });
  }
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
                            max_parts, n_parts, logit_seg, d_logits, dtype, (cudaStream_t)stream, kDecodeChunk, nullptr, 0);
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
                                part_lse, kStaticMaxParts, &n_parts, -1, nullptr, dtype, s, kDecodeChunk, nullptr, 0));
  return lse_merge_launch(part_o, part_lse, n_parts, n_heads, head_dim, d_out, o_hs, d_lse, dtype, s, nullptr, 0, nullptr, 0, nullptr, 0, 0);
}

extern "C" int infllm_lse_merge(const float* d_part_o, const float* d_part_lse, int n_part, int n_heads,
                                int head_dim, void* d_out, int64_t o_hs, float* d_lse, int dtype, void* stream) {
  using namespace infllm;
  if (!d_part_o || !d_part_lse || !d_out) return fail(INFLLM_E_BADARG, "lse_merge: null pointer");
  return lse_merge_launch(d_part_o, d_part_lse, n_part, n_heads, head_dim, d_out, o_hs, d_lse, dtype,
                          (cudaStream_t)stream, nullptr, 0, nullptr, 0, nullptr, 0, 0);
}

extern "C" int infllm_lse_merge_ex(const float* d_part_o, int64_t part_o_stride, const float* d_part_lse,
                                   int64_t part_lse_stride, int n_part, int n_heads, int head_dim, void* d_out,
                                   int64_t o_hs, float* d_lse, int dtype, const float* d_logits, int64_t logit_len,
                                   float* d_score, int64_t score_hs, const int32_t* d_skip, void* stream) {
  using namespace infllm;
  if (!d_part_o || !d_part_lse || !d_out) return fail(INFLLM_E_BADARG, "lse_merge_ex: null pointer");
  if (part_o_stride < (int64_t)n_heads * head_dim || part_lse_stride < n_heads)
    return fail(INFLLM_E_BADARG, "lse_merge_ex: partial strides %lld / %lld are shorter than a partial",
                (long long)part_o_stride, (long long)part_lse_stride);
  if (d_logits && (!d_score || !d_lse || logit_len < 0))
    return fail(INFLLM_E_BADARG, "lse_merge_ex: logits without a score buffer");
  return lse_merge_launch(d_part_o, d_part_lse, n_part, n_heads, head_dim, d_out, o_hs, d_lse, dtype,
                          (cudaStream_t)stream, d_logits, d_logits ? logit_len : 0, d_score, score_hs, d_skip,
                          part_o_stride, part_lse_stride);
}

// infllm_attn_decode whose segments [first_unit_seg, first_unit_seg + n_units) are memory units named on the
// DEVICE: unit i is d_unit_ids[i]; this GPU owns the ids [id_lo, id_lo + n_owned) and finds them in cache slot
// d_slot_table[id - id_lo] (K then V of unit_bytes at d_cache + slot * unit_bytes; -1: not cached).  Units of
// other owners and ids < 0 get weight zero; an owned unit that is not cached gets weight zero and sets *d_miss.
// The h_seg_k / h_seg_v entries of those segments are ignored.
extern "C" int infllm_attn_decode_units(const void* d_q0, const void* d_q1, int n_heads, int n_kv_heads, int head_dim,
                                        int n_seg, const void* const* h_seg_k, const void* const* h_seg_v,
                                        const int64_t* h_seg_hs, const int32_t* h_seg_len, const int32_t* h_seg_q,
                                        int first_unit_seg, int n_units, const int32_t* d_unit_ids,
                                        const int32_t* d_slot_table, int id_lo, int n_owned, const void* d_cache,
                                        int64_t unit_bytes, int32_t* d_miss, float* d_part_o, float* d_part_lse,
                                        int max_parts, int* n_parts, int logit_seg, float* d_logits, int dtype,
                                        void* stream) {
  using namespace infllm;
  if (!d_q0 || !h_seg_k || !h_seg_v || !h_seg_hs || !h_seg_len || !h_seg_q || !d_part_o || !d_part_lse)
    return fail(INFLLM_E_BADARG, "attn_decode_units: null pointer");
  if (n_seg <= 0 || n_seg > kMaxSeg) return fail(INFLLM_E_BADARG, "attn_decode_units: %d segments (1..%d)", n_seg, kMaxSeg);
  if (logit_seg >= 0 && !d_logits) return fail(INFLLM_E_BADARG, "attn_decode_units: logits requested without a buffer");
  KvSeg segs[kMaxSeg];
  for (int i = 0; i < n_seg; ++i) {
    const bool unit = i >= first_unit_seg && i < first_unit_seg + n_units;
    segs[i] = {unit ? nullptr : h_seg_k[i], unit ? nullptr : h_seg_v[i], h_seg_hs[i], head_dim, h_seg_len[i]};
  }
  DecodeIndirect ind;
  ind.ids = d_unit_ids; ind.table = d_slot_table; ind.cache = (const char*)d_cache; ind.unit_bytes = unit_bytes;
  ind.n_units = n_units; ind.first_seg = first_unit_seg; ind.miss = d_miss; ind.id_lo = id_lo; ind.n_owned = n_owned;
  return attn_decode_launch(d_q0, d_q1, head_dim, n_heads, n_kv_heads, head_dim, n_seg, segs, h_seg_q, d_part_o,
                            d_part_lse, max_parts, n_parts, logit_seg, d_logits, dtype, (cudaStream_t)stream,
                            kDecodeChunk, n_units > 0 ? &ind : nullptr, 0);
}
