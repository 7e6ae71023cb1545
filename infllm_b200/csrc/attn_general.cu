// General multi-stage attention for arbitrary shapes (any lq, lk, masks, several key segments).
//
// This is the shape-generic kernel behind the multi-stage attention class: 64-query x 64-key tiles,
// mma.sync m16n8k16 with fp32 accumulation, cp.async double buffering, online softmax in the log2
// domain with the running state (acc, m, l) carried in HBM between stages, exactly the contract of
// the reference's append()/get_result() (dot_production_attention/base.py:18-30).  The 512-query
// exec-block fast path of the context memory uses the tcgen05 kernel in attn_tc.cu instead; this
// one serves ragged shapes, short query blocks and the column-sum (per-key score) pass.
#include "attn_common.cuh"
#include "attn_tc.cuh"
#include "mma_common.cuh"

namespace infllm {

namespace {

using namespace mma;

constexpr int BM = 64;  // query rows per CTA (4 warps x 16)
constexpr int BN = 64;  // keys per tile
constexpr int NTHREADS = 128;

// load `rows` rows (token stride ts elements) x HD elements into a swizzled tile; rows >= valid are zero-filled
template <int HD, typename T>
__device__ __forceinline__ void load_tile(uint32_t dst, const T* src, int64_t ts, int valid, int rows) {
  constexpr int CH = HD / 8;
  for (int idx = threadIdx.x; idx < rows * CH; idx += NTHREADS) {
    int r = idx / CH, c = idx % CH;
    bool ok = r < valid;
    const T* p = src + (ok ? (int64_t)r * ts : 0) + c * 8;
    cp_async16(dst + tile_off<HD>(r, c), p, ok);
  }
}

template <int HD, typename T>
__global__ void __launch_bounds__(NTHREADS)
attn_general_kernel(const __grid_constant__ AttnParams P) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int TILE_BYTES = BN * HD * 2;
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + BM * HD * 2;
  const uint32_t sV = sK + 2 * TILE_BYTES;

  const int h = blockIdx.y;
  const int hkv = h / (P.n_heads / P.n_kv_heads);
  const int64_t i0 = (int64_t)blockIdx.x * BM;
  const int rows_q = (int)((P.lq - i0) < BM ? (P.lq - i0) : BM);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int64_t row_a = i0 + warp * 16 + g;  // the two query rows this thread owns
  const int64_t row_b = row_a + 8;

  float o[HD / 8][4];
  float m_a, m_b, l_a, l_b;
  if (P.first) {
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m_a = m_b = -INFINITY;
    l_a = l_b = 0.f;
  } else {
    const float* accp = P.acc + ((int64_t)h * P.lq) * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      int col = i * 8 + t4 * 2;
      float2 va = row_a < P.lq ? *reinterpret_cast<const float2*>(accp + row_a * HD + col) : make_float2(0.f, 0.f);
      float2 vb = row_b < P.lq ? *reinterpret_cast<const float2*>(accp + row_b * HD + col) : make_float2(0.f, 0.f);
      o[i][0] = va.x; o[i][1] = va.y; o[i][2] = vb.x; o[i][3] = vb.y;
    }
    m_a = row_a < P.lq ? P.m[(int64_t)h * P.lq + row_a] : -INFINITY;
    m_b = row_b < P.lq ? P.m[(int64_t)h * P.lq + row_b] : -INFINITY;
    // the denominators are kept as per-thread partials of the quad: lane t4 == 0 carries the stored value
    l_a = (row_a < P.lq && t4 == 0) ? P.l[(int64_t)h * P.lq + row_a] : 0.f;
    l_b = (row_b < P.lq && t4 == 0) ? P.l[(int64_t)h * P.lq + row_b] : 0.f;
  }

  for (int st = 0; st < P.n_stage; ++st) {
    const StageDesc& S = P.stage[st];
    int64_t vis_lo, vis_hi;
    visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
    if (vis_lo > vis_hi) continue;
    // queries of this stage -> smem -> A fragments
    __syncthreads();  // previous stage's tiles are no longer read
    load_tile<HD, T>(sQ, (const T*)S.q + (int64_t)h * S.q_hs + i0 * S.q_ts, S.q_ts, rows_q, BM);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      int r = warp * 16 + (lane & 15), c = ks * 2 + (lane >> 4);
      ldmatrix_x4(sQ + tile_off<HD>(r, c), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    int64_t seg_j0 = 0;  // stage key index of the segment's first key
    for (int sg = S.seg_begin; sg < S.seg_end; ++sg) {
      const KvSeg& G = P.seg[sg];
      const int64_t seg_len = G.len;
      // tiles of this segment that intersect the visible range
      int64_t a = vis_lo - seg_j0, b = vis_hi - seg_j0;
      if (a < 0) a = 0;
      if (b > seg_len - 1) b = seg_len - 1;
      if (a <= b) {
        const int t_first = (int)(a / BN), t_last = (int)(b / BN);
        const T* kbase = (const T*)G.k + (int64_t)hkv * G.hs;
        const T* vbase = (const T*)G.v + (int64_t)hkv * G.hs;
        __syncthreads();
        {
          int64_t r0 = (int64_t)t_first * BN;
          int valid = (int)((seg_len - r0) < BN ? (seg_len - r0) : BN);
          load_tile<HD, T>(sK, kbase + r0 * G.ts, G.ts, valid, BN);
          load_tile<HD, T>(sV, vbase + r0 * G.ts, G.ts, valid, BN);
          cp_async_commit();
        }
        for (int t = t_first; t <= t_last; ++t) {
          const int buf = (t - t_first) & 1;
          if (t < t_last) {
            int64_t r0 = (int64_t)(t + 1) * BN;
            int valid = (int)((seg_len - r0) < BN ? (seg_len - r0) : BN);
            load_tile<HD, T>(sK + (buf ^ 1) * TILE_BYTES, kbase + r0 * G.ts, G.ts, valid, BN);
            load_tile<HD, T>(sV + (buf ^ 1) * TILE_BYTES, vbase + r0 * G.ts, G.ts, valid, BN);
            cp_async_commit();
            cp_async_wait<1>();
          } else {
            cp_async_wait<0>();
          }
          __syncthreads();
          const uint32_t kt = sK + buf * TILE_BYTES, vt = sV + buf * TILE_BYTES;
          // S = Q K^T  (16 rows x 64 keys per warp)
          float sacc[BN / 8][4];
#pragma unroll
          for (int i = 0; i < BN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
              int mid = lane >> 3;
              int r = np * 16 + (mid >> 1) * 8 + (lane & 7), c = ks * 2 + (mid & 1);
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4(kt + tile_off<HD>(r, c), b0, b1, b2, b3);
              mma16816<T>(sacc[np * 2], qf[ks], b0, b1);
              mma16816<T>(sacc[np * 2 + 1], qf[ks], b2, b3);
            }
          }
          // scale, mask, online softmax
          const int64_t jt = seg_j0 + (int64_t)t * BN;  // stage key index of the tile's first key
          const int64_t jlim = seg_j0 + seg_len;
          float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
          for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              int64_t j = jt + i * 8 + t4 * 2 + (e & 1);
              int64_t row = (e < 2) ? row_a : row_b;
              bool keep = j < jlim && row < P.lq && mask_keep(S.mask_mode, S.mask_offset, S.mask_size, row, j);
              float v = keep ? sacc[i][e] * P.scale_log2 : -INFINITY;
              sacc[i][e] = v;
              if (e < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
            }
          }
          mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
          mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
          mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
          mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
          const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
          const float ms_a = mn_a == -INFINITY ? 0.f : mn_a, ms_b = mn_b == -INFINITY ? 0.f : mn_b;
          const float al_a = exp2f(m_a - ms_a), al_b = exp2f(m_b - ms_b);
          m_a = mn_a; m_b = mn_b;
          float rs_a = 0.f, rs_b = 0.f;
#pragma unroll
          for (int i = 0; i < BN / 8; ++i) {
            sacc[i][0] = exp2f(sacc[i][0] - ms_a);
            sacc[i][1] = exp2f(sacc[i][1] - ms_a);
            sacc[i][2] = exp2f(sacc[i][2] - ms_b);
            sacc[i][3] = exp2f(sacc[i][3] - ms_b);
            rs_a += sacc[i][0] + sacc[i][1];
            rs_b += sacc[i][2] + sacc[i][3];
          }
          l_a = l_a * al_a + rs_a;  // per-thread partial sums; reduced over the quad at the end
          l_b = l_b * al_b + rs_b;
#pragma unroll
          for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b;
          }
          // O += P V
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            uint32_t pa[4];
            pa[0] = pack2<T>(sacc[2 * ks][0], sacc[2 * ks][1]);
            pa[1] = pack2<T>(sacc[2 * ks][2], sacc[2 * ks][3]);
            pa[2] = pack2<T>(sacc[2 * ks + 1][0], sacc[2 * ks + 1][1]);
            pa[3] = pack2<T>(sacc[2 * ks + 1][2], sacc[2 * ks + 1][3]);
#pragma unroll
            for (int dn = 0; dn < HD / 16; ++dn) {
              int mid = lane >> 3;
              int r = ks * 16 + (mid & 1) * 8 + (lane & 7), c = dn * 2 + (mid >> 1);
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4_trans(vt + tile_off<HD>(r, c), b0, b1, b2, b3);
              mma16816<T>(o[dn * 2], pa, b0, b1);
              mma16816<T>(o[dn * 2 + 1], pa, b2, b3);
            }
          }
          __syncthreads();  // all warps done with this buffer before it is refilled
        }
      }
      seg_j0 += seg_len;
    }
  }

  // The running denominators are per-thread partials over the quad's columns: they were all scaled
  // by the same per-row factors, so one reduction at the end gives the row sums.
  float la = l_a, lb = l_b;
  la += __shfl_xor_sync(0xffffffffu, la, 1);
  la += __shfl_xor_sync(0xffffffffu, la, 2);
  lb += __shfl_xor_sync(0xffffffffu, lb, 1);
  lb += __shfl_xor_sync(0xffffffffu, lb, 2);

  if (P.last) {
    T* outp = (T*)P.out + (int64_t)h * P.o_hs;
    const float inv_a = la > 0.f ? 1.f / la : 0.f, inv_b = lb > 0.f ? 1.f / lb : 0.f;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      int col = i * 8 + t4 * 2;
      if (row_a < P.lq)
        *reinterpret_cast<uint32_t*>(outp + row_a * P.o_ts + col) = pack2<T>(o[i][0] * inv_a, o[i][1] * inv_a);
      if (row_b < P.lq)
        *reinterpret_cast<uint32_t*>(outp + row_b * P.o_ts + col) = pack2<T>(o[i][2] * inv_b, o[i][3] * inv_b);
    }
    if (P.lse && t4 == 0) {
      if (row_a < P.lq) P.lse[(int64_t)h * P.lq + row_a] = la > 0.f ? m_a + log2f(la) : -INFINITY;
      if (row_b < P.lq) P.lse[(int64_t)h * P.lq + row_b] = lb > 0.f ? m_b + log2f(lb) : -INFINITY;
    }
  } else {
    float* accp = P.acc + ((int64_t)h * P.lq) * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      int col = i * 8 + t4 * 2;
      if (row_a < P.lq) *reinterpret_cast<float2*>(accp + row_a * HD + col) = make_float2(o[i][0], o[i][1]);
      if (row_b < P.lq) *reinterpret_cast<float2*>(accp + row_b * HD + col) = make_float2(o[i][2], o[i][3]);
    }
    if (t4 == 0) {
      if (row_a < P.lq) { P.m[(int64_t)h * P.lq + row_a] = m_a; P.l[(int64_t)h * P.lq + row_a] = la; }
      if (row_b < P.lq) { P.m[(int64_t)h * P.lq + row_b] = m_b; P.l[(int64_t)h * P.lq + row_b] = lb; }
    }
  }
}

// ---------------------------------------------------------------------------------- column sums
// score[h, j] (+)= sum_i exp2(s2[i, j] - lse2[i]) over the visible queries of key j.
// One CTA owns 64 keys of one head (K tile resident in shared memory) and streams the query tiles.
template <int HD, typename T>
__global__ void __launch_bounds__(NTHREADS)
attn_colsum_kernel(const T* __restrict__ q, int64_t q_hs, int64_t q_ts, const T* __restrict__ k, int64_t k_hs,
                   int64_t k_ts, int group, int64_t lq, int64_t lk, int mask_mode, int64_t mask_offset,
                   int64_t mask_size, const float* __restrict__ lse, float* __restrict__ score, int64_t score_hs,
                   int accumulate, float scale_log2) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int TILE_BYTES = BN * HD * 2;
  const uint32_t sK = smem_u32(smem);
  const uint32_t sQ = sK + TILE_BYTES;  // two query tiles
  float* red = reinterpret_cast<float*>(smem + 3 * TILE_BYTES);  // 4 warps x 64 columns

  const int h = blockIdx.y, hkv = h / group;
  const int64_t j0 = (int64_t)blockIdx.x * BN;
  const int keys = (int)((lk - j0) < BN ? (lk - j0) : BN);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  // query rows that can see any key of this tile
  int64_t qi_lo = 0, qi_hi = lq - 1;
  if (mask_mode == INFLLM_MASK_WINDOW) {
    qi_lo = j0 - mask_offset;
    qi_hi = j0 + keys - 1 - mask_offset + mask_size - 1;
  } else if (mask_mode == INFLLM_MASK_COMPLEMENT) {
    qi_lo = j0 - mask_offset + mask_size;
  }
  if (qi_lo < 0) qi_lo = 0;
  if (qi_hi > lq - 1) qi_hi = lq - 1;

  float cs[BN / 8][2];
#pragma unroll
  for (int i = 0; i < BN / 8; ++i) cs[i][0] = cs[i][1] = 0.f;

  if (qi_lo <= qi_hi) {
    const int t_first = (int)(qi_lo / BM), t_last = (int)(qi_hi / BM);
    const T* qh = q + (int64_t)h * q_hs;
    load_tile<HD, T>(sK, k + (int64_t)hkv * k_hs + j0 * k_ts, k_ts, keys, BN);
    {
      int64_t r0 = (int64_t)t_first * BM;
      int valid = (int)((lq - r0) < BM ? (lq - r0) : BM);
      load_tile<HD, T>(sQ, qh + r0 * q_ts, q_ts, valid, BM);
    }
    cp_async_commit();
    for (int t = t_first; t <= t_last; ++t) {
      const int buf = (t - t_first) & 1;
      if (t < t_last) {
        int64_t r0 = (int64_t)(t + 1) * BM;
        int valid = (int)((lq - r0) < BM ? (lq - r0) : BM);
        load_tile<HD, T>(sQ + (buf ^ 1) * TILE_BYTES, qh + r0 * q_ts, q_ts, valid, BM);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const uint32_t qt = sQ + buf * TILE_BYTES;
      float sacc[BN / 8][4];
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t qf[4];
        {
          int r = warp * 16 + (lane & 15), c = ks * 2 + (lane >> 4);
          ldmatrix_x4(qt + tile_off<HD>(r, c), qf[0], qf[1], qf[2], qf[3]);
        }
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          int mid = lane >> 3;
          int r = np * 16 + (mid >> 1) * 8 + (lane & 7), c = ks * 2 + (mid & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(sK + tile_off<HD>(r, c), b0, b1, b2, b3);
          mma16816<T>(sacc[np * 2], qf, b0, b1);
          mma16816<T>(sacc[np * 2 + 1], qf, b2, b3);
        }
      }
      const int64_t row_a = (int64_t)t * BM + warp * 16 + g, row_b = row_a + 8;
      const float lse_a = row_a < lq ? lse[(int64_t)h * lq + row_a] : INFINITY;
      const float lse_b = row_b < lq ? lse[(int64_t)h * lq + row_b] : INFINITY;
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int64_t j = j0 + i * 8 + t4 * 2 + (e & 1);
          int64_t row = (e < 2) ? row_a : row_b;
          float ls = (e < 2) ? lse_a : lse_b;
          bool keep = j < lk && row < lq && ls != -INFINITY && mask_keep(mask_mode, mask_offset, mask_size, row, j);
          float p = keep ? exp2f(sacc[i][e] * scale_log2 - ls) : 0.f;
          cs[i][e & 1] += p;
        }
      }
      __syncthreads();
    }
  }
  // reduce over the 8 row groups of the warp, then over the 4 warps
#pragma unroll
  for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float v = cs[i][e];
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      if (g == 0) red[warp * BN + i * 8 + t4 * 2 + e] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < keys) {
    int c = threadIdx.x;
    float v = red[c] + red[BN + c] + red[2 * BN + c] + red[3 * BN + c];
    float* dst = score + (int64_t)h * score_hs + j0 + c;
    *dst = accumulate ? *dst + v : v;
  }
}

template <int HD>
int launch_general(const AttnParams& p, int dtype, cudaStream_t s) {
  dim3 grid((unsigned)ceil_div(p.lq, BM), p.n_heads);
  size_t smem = (size_t)BM * HD * 2 + 4 * (size_t)BN * HD * 2;
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    auto kern = attn_general_kernel<HD, T>;
    INFLLM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, NTHREADS, smem, s>>>(p);
  });
  INFLLM_LAUNCH_OK("attn_general_kernel");
  return INFLLM_OK;
}

template <int HD>
int launch_colsum(const void* q, int64_t q_hs, int64_t q_ts, const void* k, int64_t k_hs, int64_t k_ts, int n_heads,
                  int n_kv_heads, int64_t lq, int64_t lk, int mask_mode, int64_t mask_offset, int64_t mask_size,
                  const float* lse, float* score, int64_t score_hs, int accumulate, int dtype, cudaStream_t s) {
  dim3 grid((unsigned)ceil_div(lk, BN), n_heads);
  size_t smem = 3 * (size_t)BN * HD * 2 + 4 * BN * sizeof(float);
  float scale_log2 = kLog2e / sqrtf((float)HD);
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    auto kern = attn_colsum_kernel<HD, T>;
    INFLLM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, NTHREADS, smem, s>>>((const T*)q, q_hs, q_ts, (const T*)k, k_hs, k_ts, n_heads / n_kv_heads, lq, lk,
                                      mask_mode, mask_offset, mask_size, lse, score, score_hs, accumulate,
                                      scale_log2);
  });
  INFLLM_LAUNCH_OK("attn_colsum_kernel");
  return INFLLM_OK;
}

template <typename T>
__global__ void attn_finalize_kernel(const float* __restrict__ acc, const float* __restrict__ m,
                                     const float* __restrict__ l, T* __restrict__ out, int64_t o_hs, int64_t o_ts,
                                     float* __restrict__ lse, int64_t lq, int head_dim) {
  int64_t row = blockIdx.x;  // h * lq + i
  int64_t h = row / lq, i = row - h * lq;
  float lv = l[row];
  float inv = lv > 0.f ? 1.f / lv : 0.f;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x)
    out[h * o_hs + i * o_ts + d] = Act<T>::from_f(acc[row * head_dim + d] * inv);
  if (lse && threadIdx.x == 0) lse[row] = lv > 0.f ? m[row] + log2f(lv) : -INFINITY;
}

}  // namespace

int attn_general_launch(const AttnParams& p, int head_dim, int dtype, cudaStream_t s) {
  if (p.lq <= 0) return INFLLM_OK;
  if (p.n_heads % p.n_kv_heads) return fail(INFLLM_E_BADARG, "attention: %d heads / %d kv heads", p.n_heads, p.n_kv_heads);
  if (head_dim == 128) return launch_general<128>(p, dtype, s);
  if (head_dim == 64) return launch_general<64>(p, dtype, s);
  return fail(INFLLM_E_UNSUPPORTED, "attention: head_dim %d (64 and 128 are built)", head_dim);
}

int attn_colsum_launch(const void* q, int64_t q_hs, int64_t q_ts, const void* k, int64_t k_hs, int64_t k_ts,
                       int n_heads, int n_kv_heads, int64_t lq, int64_t lk, int head_dim, int mask_mode,
                       int64_t mask_offset, int64_t mask_size, const float* lse, float* score, int64_t score_hs,
                       int accumulate, int dtype, cudaStream_t s) {
  if (lk <= 0) return INFLLM_OK;
  if (n_heads % n_kv_heads) return fail(INFLLM_E_BADARG, "colsum: %d heads / %d kv heads", n_heads, n_kv_heads);
  if (head_dim == 128)
    return launch_colsum<128>(q, q_hs, q_ts, k, k_hs, k_ts, n_heads, n_kv_heads, lq, lk, mask_mode, mask_offset,
                              mask_size, lse, score, score_hs, accumulate, dtype, s);
  if (head_dim == 64)
    return launch_colsum<64>(q, q_hs, q_ts, k, k_hs, k_ts, n_heads, n_kv_heads, lq, lk, mask_mode, mask_offset,
                             mask_size, lse, score, score_hs, accumulate, dtype, s);
  return fail(INFLLM_E_UNSUPPORTED, "colsum: head_dim %d (64 and 128 are built)", head_dim);
}

}  // namespace infllm

static int check_rows(const void* p, int64_t hs, int64_t ts, const char* what) {
  if (((uintptr_t)p % 16) || (hs % 8) || (ts % 8))
    return infllm::fail(INFLLM_E_BADARG, "%s: base and strides must keep rows 16-byte aligned", what);
  return INFLLM_OK;
}

extern "C" int infllm_attn_stage(const void* d_q, int64_t q_hs, int64_t q_ts, const void* d_k, int64_t k_hs,
                                 int64_t k_ts, const void* d_v, int64_t v_hs, int64_t v_ts, int n_heads,
                                 int n_kv_heads, int64_t lq, int64_t lk, int head_dim, int mask_mode,
                                 int64_t mask_offset, int64_t mask_size, float* d_acc, float* d_m, float* d_l,
                                 int first, int dtype, void* stream) {
  using namespace infllm;
  if (!d_q || !d_acc || !d_m || !d_l || lq < 0 || lk < 0 || n_heads <= 0 || n_kv_heads <= 0)
    return fail(INFLLM_E_BADARG, "attn_stage: bad argument");
  if (lk > 0 && (!d_k || !d_v)) return fail(INFLLM_E_BADARG, "attn_stage: null keys/values");
  if (k_hs != v_hs || k_ts != v_ts) return fail(INFLLM_E_BADARG, "attn_stage: k and v must share strides");
  if (k_ts > INT32_MAX) return fail(INFLLM_E_BADARG, "attn_stage: token stride too large");
  INFLLM_TRY(check_rows(d_q, q_hs, q_ts, "attn_stage q"));
  if (lk > 0) {
    INFLLM_TRY(check_rows(d_k, k_hs, k_ts, "attn_stage k"));
    INFLLM_TRY(check_rows(d_v, v_hs, v_ts, "attn_stage v"));
  }
  if (mask_mode < INFLLM_MASK_NONE || mask_mode > INFLLM_MASK_COMPLEMENT)
    return fail(INFLLM_E_BADARG, "attn_stage: mask mode %d", mask_mode);
  AttnParams p{};
  p.n_stage = 1;
  p.stage[0].q = d_q; p.stage[0].q_hs = q_hs; p.stage[0].q_ts = q_ts;
  p.stage[0].mask_mode = mask_mode; p.stage[0].mask_offset = mask_offset; p.stage[0].mask_size = mask_size;
  p.stage[0].lk = lk;
  // a stage longer than one segment's 31-bit length is split
  int nseg = 0;
  for (int64_t pos = 0; pos < lk && nseg < kMaxSeg; ++nseg) {
    int64_t n = lk - pos < (1 << 30) ? lk - pos : (1 << 30);
    p.seg[nseg].k = (const char*)d_k + pos * k_ts * 2; p.seg[nseg].v = (const char*)d_v + pos * v_ts * 2;
    p.seg[nseg].hs = k_hs; p.seg[nseg].ts = (int32_t)k_ts; p.seg[nseg].len = (int32_t)n;
    pos += n;
  }
  p.stage[0].seg_begin = 0; p.stage[0].seg_end = nseg;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.first = first; p.last = 0; p.lq = lq;
  p.acc = d_acc; p.m = d_m; p.l = d_l; p.out = nullptr; p.lse = nullptr;
  p.scale_log2 = kLog2e / sqrtf((float)head_dim);
  return attn_general_launch(p, head_dim, dtype, (cudaStream_t)stream);
}

extern "C" int infllm_attn_finalize(const float* d_acc, const float* d_m, const float* d_l, void* d_out, int64_t o_hs,
                                    int64_t o_ts, float* d_lse, int n_heads, int64_t lq, int head_dim, int dtype,
                                    void* stream) {
  using namespace infllm;
  if (!d_acc || !d_m || !d_l || !d_out) return fail(INFLLM_E_BADARG, "attn_finalize: null pointer");
  if (lq <= 0) return INFLLM_OK;
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    attn_finalize_kernel<T><<<(unsigned)(n_heads * lq), 128, 0, (cudaStream_t)stream>>>(
        d_acc, d_m, d_l, (T*)d_out, o_hs, o_ts, d_lse, lq, head_dim);
  });
  INFLLM_LAUNCH_OK("attn_finalize_kernel");
  return INFLLM_OK;
}

extern "C" int infllm_attn_colsum(const void* d_q, int64_t q_hs, int64_t q_ts, const void* d_k, int64_t k_hs,
                                  int64_t k_ts, int n_heads, int n_kv_heads, int64_t lq, int64_t lk, int head_dim,
                                  int mask_mode, int64_t mask_offset, int64_t mask_size, const float* d_lse,
                                  float* d_score, int64_t score_hs, int accumulate, int dtype, void* stream) {
  using namespace infllm;
  if (!d_q || !d_lse || !d_score || lq < 0 || lk < 0) return fail(INFLLM_E_BADARG, "attn_colsum: bad argument");
  if (lk == 0 || lq == 0) return INFLLM_OK;
  if (!d_k) return fail(INFLLM_E_BADARG, "attn_colsum: null keys");
  INFLLM_TRY(check_rows(d_q, q_hs, q_ts, "attn_colsum q"));
  INFLLM_TRY(check_rows(d_k, k_hs, k_ts, "attn_colsum k"));
  // full 128-row tiles on both sides: the tcgen05 kernel; ragged small shapes: the mma.sync kernel
  if (head_dim == 128 && lq >= 128 && lq <= 512 && lk >= 128 && n_heads % n_kv_heads == 0 && lk < (1ll << 31))
    return colsum_tc_launch(d_q, q_hs, q_ts, d_k, k_hs, k_ts, n_heads, n_kv_heads, lq, lk, mask_mode, mask_offset,
                            mask_size, d_lse, d_score, score_hs, accumulate, dtype, (cudaStream_t)stream);
  return attn_colsum_launch(d_q, q_hs, q_ts, d_k, k_hs, k_ts, n_heads, n_kv_heads, lq, lk, head_dim, mask_mode,
                            mask_offset, mask_size, d_lse, d_score, score_hs, accumulate, dtype,
                            (cudaStream_t)stream);
}
