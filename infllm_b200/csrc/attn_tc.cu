// Tensor-core (tcgen05 + TMEM + TMA) attention kernels for head_dim 128.
//
// attn_tc3_kernel   one 128-query tile of one head per CTA, all stages of an exec block fused:
//                   local window stage (window-relative rotated q/k, causal window mask) and global
//                   stage (one-angle q; retrieved units in their cache slots, init sink, overflow),
//                   jointly normalised.  Warp-specialised: 8 softmax warps (two threads per query row, each
//                   owning half of the tile's key columns; row = TMEM lane), 1 TMA producer warp, two issuing
//                   threads (S = Q K^T and O += P V).  S accumulates in TMEM (three buffers), P is written back
//                   over its S columns and feeds the P V product from TMEM, O stays in TMEM for the whole tile
//                   with lazy rescaling; K/V tiles are double buffered.
// attn_tc2_kernel   the same for two query heads of one KV head per CTA, key tiles cut into runs (few heads per GPU).
// colsum_tc_kernel  per-key score pass: S^T = K Q^T with keys as TMEM lanes; a CTA keeps one head's query tiles
//                   resident and streams a run of key tiles through a TMA ring and four TMEM buffers; four
//                   threads per key sum exp2(s - lse) over the queries that see it.
// Every mbarrier wait is bounded; a wait that runs out records an error code and the CTA unwinds.
#include <algorithm>
#include <type_traits>

#include "attn_common.cuh"
#include "tc_common.cuh"
#include "attn_tc.cuh"

namespace infllm {

using namespace tc;

__device__ int g_tc_error[4];  // [0] code, [1] where, [2] blockIdx.x, [3] blockIdx.y

__device__ __forceinline__ void record_error(int* err, int code, int where) {
  if (atomicCAS(&err[0], 0, code) == 0) {
    err[1] = where;
    err[2] = blockIdx.x;
    err[3] = blockIdx.y;
  }
}

// wait that also gives up when another role of the CTA has already failed
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err,
                                              int where) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
  }
  *abort_flag = 1;
  record_error(err, kErrWaitTimeout, where);
  return false;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Blackwell's packed fp32 pairs and three-input maximum: half the instructions of the scalar forms
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 ffma2(float a0, float a1, float2 b, float2 c) {
  float2 d;
  asm("{ .reg .b64 ra, rb, rc, rd; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; mov.b64 rc, {%6,%7}; "
      "fma.rn.f32x2 rd, ra, rb, rc; mov.b64 {%0,%1}, rd; }"
      : "=f"(d.x), "=f"(d.y) : "f"(a0), "f"(a1), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{ .reg .b64 ra, rb, rd; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; add.rn.f32x2 rd, ra, rb; mov.b64 {%0,%1}, rd; }"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// exp2 of a pair on the FMA and integer pipes (the special-function unit does 16 per clock per SM, which bounds the
// softmax when every exponential goes there): x = n + f with n the nearest integer (magic-number rounding) and f in
// [-0.5, 0.5], 2^f by a cubic (relative error 7e-4, below the rounding of a 16-bit P), n added into the exponent
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 magic = make_float2(12582912.f, 12582912.f), neg_magic = make_float2(-12582912.f, -12582912.f);
  const float2 t = fadd2(x, magic);
  const float2 n = fadd2(t, neg_magic);
  const float2 f = fadd2(x, make_float2(-n.x, -n.y));
  float2 p = ffma2(f.x, f.y, make_float2(0.0555041f, 0.0555041f), make_float2(0.2402265f, 0.2402265f));
  p = ffma2(p.x, p.y, f, make_float2(0.6931472f, 0.6931472f));
  p = ffma2(p.x, p.y, f, make_float2(1.f, 1.f));
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                     __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
}

// two exponentials per special-function instruction: exp2 of a pair of fp32 arguments evaluated in fp16
// (relative error about 5e-4, arguments below -25 give 0), returned as fp32
__device__ __forceinline__ float2 ex2_pair(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  uint32_t u = *reinterpret_cast<uint32_t*>(&h), r;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(r) : "r"(u));
  return __half22float2(*reinterpret_cast<__half2*>(&r));
}

// The two threads that share a query row publish a progress counter in shared memory; bounded like every wait.
constexpr int kPairDone = 0x40000000;
__device__ __forceinline__ bool pair_wait(volatile int* flag, int want, volatile int* abort_flag, int* err, int where) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (*flag >= want) return true;
    if (*abort_flag) return false;
    if (i > 256) __nanosleep(32);
  }
  *abort_flag = 1;
  record_error(err, kErrWaitTimeout, where);
  return false;
}

// tiles [first, last] of a segment that intersect the visible key range [vis_lo, vis_hi] of the stage
__device__ __forceinline__ bool seg_tiles(int64_t vis_lo, int64_t vis_hi, int64_t seg_j0, int seg_len, int* first,
                                          int* last) {
  int64_t a = vis_lo - seg_j0, b = vis_hi - seg_j0;
  if (a < 0) a = 0;
  if (b > seg_len - 1) b = seg_len - 1;
  if (a > b) return false;
  *first = (int)(a / kTile);
  *last = (int)(b / kTile);
  return true;
}

// ------------------------------------------------------------------------------------------------
// attn_tc2_kernel: two query heads of the same KV head per CTA.
// The exec-block kernel above is bound by the L2 -> shared-memory traffic of its K/V tiles (64 KB per
// 8.4 MFLOP).  Here every K/V tile feeds two 128-query tiles (heads 2p and 2p+1 of one KV head, same
// query rows, hence the same masks and tile list), which halves that traffic; the key tiles of a work
// item are cut into n_split runs so that the grid still covers the SMs, and the runs' partial results
// are merged by attn_tc_combine_kernel.  P = exp2(S - m) goes back into the TMEM columns of S as packed
// 16-bit pairs and is the A operand of the P V product straight from TMEM; exponentials are evaluated
// two per instruction in fp16.  16 softmax warps (2 heads x 128 rows x 2 column halves), 1 TMA warp,
// 1 MMA warp.
namespace tc2 {
constexpr int kQ = 0;                            // Q of head A, then head B
constexpr int kK = kQ + 4 * kSubTileBytes;       // two stages
constexpr int kV = kK + 4 * kSubTileBytes;       // two stages
constexpr int kBar = kV + 4 * kSubTileBytes;
constexpr int kXmax = kBar + 256;                // row maxima: 2 heads x 2 tile parities x 2 halves x 128 rows
constexpr int kXsum = kXmax + 4096;              // row sums: 2 heads x 2 halves x 128 rows
constexpr int kXflag = kXsum + 2048;             // progress counters: 2 heads x 2 halves x 128 rows
constexpr int kTotal = kXflag + 2048;
enum { T2_Q_FULL = 0, T2_Q_EMPTY, T2_K_FULL0, T2_K_FULL1, T2_K_EMPTY0, T2_K_EMPTY1, T2_V_FULL0, T2_V_FULL1, T2_V_EMPTY0, T2_V_EMPTY1, T2_S_FULLA, T2_S_FULLB,
       T2_P_FULLA, T2_P_FULLB, T2_O_FULL, T2_N_BARS };
}  // namespace tc2

// number of key tiles of stage S that the 128-row query block starting at i0 visits
__device__ __forceinline__ int stage_tiles(const AttnTcParams& P, const TcStage& S, int64_t vis_lo, int64_t vis_hi) {
  int n = 0;
  int64_t j0s = 0;
  for (int sg = S.seg_begin; sg < S.seg_end; ++sg) {
    int tf, tl;
    if (seg_tiles(vis_lo, vis_hi, j0s, P.seg[sg].len, &tf, &tl)) n += tl - tf + 1;
    j0s += P.seg[sg].len;
  }
  return n;
}

template <typename T>
__global__ void __launch_bounds__(576, 1) attn_tc2_kernel(const __grid_constant__ AttnTcParams P) {
  using namespace tc2;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t sQ = s_base + kQ, sK = s_base + kK, sV = s_base + kV;
  const uint32_t bars = s_base + kBar;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kBar + T2_N_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kBar + T2_N_BARS * 8 + 8);
  float* xmax = reinterpret_cast<float*>(smem + kXmax);
  float* xsum = reinterpret_cast<float*>(smem + kXsum);
  volatile int* xflag = reinterpret_cast<volatile int*>(smem + kXflag);
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hA = 2 * blockIdx.y, hkv = hA / (P.n_heads / P.n_kv_heads);
  const int64_t i0 = (int64_t)blockIdx.x * kTile;
  const int rows_q = (int)((P.lq - i0) < kTile ? (P.lq - i0) : kTile);
  const int split = blockIdx.z;

  // this CTA's run [g0, g1) of the work item's key tiles, numbered over all stages
  int n_total = 0;
  for (int st = 0; st < P.n_stage; ++st) {
    const TcStage& S = P.stage[st];
    int64_t vis_lo, vis_hi;
    visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
    if (vis_lo <= vis_hi) n_total += stage_tiles(P, S, vis_lo, vis_hi);
  }
  const int g0 = (int)((int64_t)n_total * split / P.n_split), g1 = (int)((int64_t)n_total * (split + 1) / P.n_split);

  if (threadIdx.x == 0) {
    for (int i = 0; i < T2_N_BARS; ++i) mbar_init(bar(i), (i == T2_P_FULLA || i == T2_P_FULLB) ? 256u : 1u);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 512) xflag[threadIdx.x] = 0;
  if (warp == 17) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S/P of head A [0,128), of head B [128,256), O of head A [256,384), of head B [384,512)
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  constexpr uint32_t idesc_qk = make_idesc(kBf16, 128, 128, false);
  constexpr uint32_t idesc_pv = make_idesc(kBf16, 128, 128, true);

  if (warp == 16) {
    // ======================================================================== TMA producer
    if (lane == 0) {
      int g = 0, it = 0, sidx = 0;
      bool ok = true;
      for (int st = 0; st < P.n_stage && ok; ++st) {
        const TcStage& S = P.stage[st];
        int64_t vis_lo, vis_hi;
        visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
        if (vis_lo > vis_hi) continue;
        const int n_st = stage_tiles(P, S, vis_lo, vis_hi);
        const bool active = (g > g0 ? g : g0) < (g + n_st < g1 ? g + n_st : g1);
        if (active) {
          if (sidx >= 1) ok = wait_or_abort(bar(T2_Q_EMPTY), (sidx - 1) & 1, abort_flag, P.err, 500);
          if (!ok) break;
          mbar_expect_tx(bar(T2_Q_FULL), 4 * kSubTileBytes);
          for (int x = 0; x < 2; ++x) {
            tma_load_3d(sQ + x * 2 * kSubTileBytes, &P.maps[S.map_q], bar(T2_Q_FULL), 0, S.q_row0 + (int)i0, hA + x);
            tma_load_3d(sQ + x * 2 * kSubTileBytes + kSubTileBytes, &P.maps[S.map_q], bar(T2_Q_FULL), 64,
                        S.q_row0 + (int)i0, hA + x);
          }
          ++sidx;
        }
        int64_t seg_j0 = 0;
        for (int sg = S.seg_begin; sg < S.seg_end && ok; ++sg) {
          const TcSeg& G = P.seg[sg];
          int tf, tl;
          if (seg_tiles(vis_lo, vis_hi, seg_j0, G.len, &tf, &tl)) {
            for (int t = tf; t <= tl && ok; ++t, ++g) {
              if (g < g0 || g >= g1) continue;
              const int b = it & 1, tok = G.tok0 + t * kTile;
              if (it >= 2) ok = wait_or_abort(bar(T2_K_EMPTY0 + b), ((it >> 1) - 1) & 1, abort_flag, P.err, 501);
              if (!ok) break;
              const uint32_t dk = sK + b * 2 * kSubTileBytes, dv = sV + b * 2 * kSubTileBytes;
              mbar_expect_tx(bar(T2_K_FULL0 + b), 2 * kSubTileBytes);
              if (G.c3_k < 0) {
                tma_load_3d(dk, &P.maps[G.map_k], bar(T2_K_FULL0 + b), 0, tok, hkv);
                tma_load_3d(dk + kSubTileBytes, &P.maps[G.map_k], bar(T2_K_FULL0 + b), 64, tok, hkv);
              } else {
                tma_load_4d(dk, &P.maps[G.map_k], bar(T2_K_FULL0 + b), 0, tok, hkv, G.c3_k);
                tma_load_4d(dk + kSubTileBytes, &P.maps[G.map_k], bar(T2_K_FULL0 + b), 64, tok, hkv, G.c3_k);
              }
              if (it >= 2) ok = wait_or_abort(bar(T2_V_EMPTY0 + b), ((it >> 1) - 1) & 1, abort_flag, P.err, 502);
              if (!ok) break;
              mbar_expect_tx(bar(T2_V_FULL0 + b), 2 * kSubTileBytes);
              if (G.c3_v < 0) {
                tma_load_3d(dv, &P.maps[G.map_v], bar(T2_V_FULL0 + b), 0, tok, hkv);
                tma_load_3d(dv + kSubTileBytes, &P.maps[G.map_v], bar(T2_V_FULL0 + b), 64, tok, hkv);
              } else {
                tma_load_4d(dv, &P.maps[G.map_v], bar(T2_V_FULL0 + b), 0, tok, hkv, G.c3_v);
                tma_load_4d(dv + kSubTileBytes, &P.maps[G.map_v], bar(T2_V_FULL0 + b), 64, tok, hkv, G.c3_v);
              }
              ++it;
            }
          }
          seg_j0 += G.len;
        }
      }
      if (!ok) {
        // give loads that are still in flight a bounded chance to land before the CTA's memory goes away
        for (int b = 0; b < 2; ++b) {
          for (uint32_t i = 0; i < 4096 && !mbar_try_wait(bar(T2_K_FULL0 + b), 0) && !mbar_try_wait(bar(T2_K_FULL0 + b), 1); ++i) __nanosleep(64);
          for (uint32_t i = 0; i < 4096 && !mbar_try_wait(bar(T2_V_FULL0 + b), 0) && !mbar_try_wait(bar(T2_V_FULL0 + b), 1); ++i) __nanosleep(64);
        }
      }
    }
  } else if (warp == 17) {
    // ========================================================================== MMA issuer
    if (lane == 0) {
      int g = 0, it = 0, sidx = 0;
      bool ok = true;
      // S(x) = Q(x) K(tile j)^T into head x's S columns
      auto issue_qk = [&](int x, int j) {
        const uint32_t kt = sK + (j & 1) * 2 * kSubTileBytes, qt = sQ + x * 2 * kSubTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint64_t ad = make_sdesc(qt + (ks >> 2) * kSubTileBytes + (ks & 3) * 32, 16, 1024);
          uint64_t bd = make_sdesc(kt + (ks >> 2) * kSubTileBytes + (ks & 3) * 32, 16, 1024);
          mma_ss(tmem + x * 128, ad, bd, idesc_qk, ks > 0);
        }
        tc_commit(bar(T2_S_FULLA + x));
      };
      // O(x) += P(x) V(tile j): P from TMEM (keys 0-63 in S columns [0,32), keys 64-127 in [64,96)), V d-contiguous
      auto issue_pv = [&](int x, int j) -> bool {
        if (!wait_or_abort(bar(T2_P_FULLA + x), j & 1, abort_flag, P.err, 510)) return false;
        if (x == 0 && !wait_or_abort(bar(T2_V_FULL0 + (j & 1)), (j >> 1) & 1, abort_flag, P.err, 511)) return false;
        tc_fence_after();
        const uint32_t vt = sV + (j & 1) * 2 * kSubTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t a_t = tmem + x * 128 + (ks < 4 ? 8 * ks : 64 + 8 * (ks - 4));
          uint64_t bd = make_sdesc(vt + ks * 2048, kSubTileBytes, 1024);
          mma_ts(tmem + 256 + x * 128, a_t, bd, idesc_pv, (j > 0) || (ks > 0));
        }
        return true;
      };
      for (int st = 0; st < P.n_stage && ok; ++st) {
        const TcStage& S = P.stage[st];
        int64_t vis_lo, vis_hi;
        visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
        if (vis_lo > vis_hi) continue;
        const int n_st = stage_tiles(P, S, vis_lo, vis_hi);
        const int lo = g > g0 ? g : g0, hi = g + n_st < g1 ? g + n_st : g1;
        g += n_st;
        if (lo >= hi) continue;
        const int n_loc = hi - lo;  // this CTA's tiles of this stage: local indices it .. it + n_loc - 1
        ok = wait_or_abort(bar(T2_Q_FULL), sidx & 1, abort_flag, P.err, 512);
        ++sidx;
        if (!ok) break;
        // prologue: both heads' S for the first tile
        ok = wait_or_abort(bar(T2_K_FULL0 + (it & 1)), (it >> 1) & 1, abort_flag, P.err, 513);
        if (!ok) break;
        tc_fence_after();
        issue_qk(0, it);
        issue_qk(1, it);
        tc_commit(bar(T2_K_EMPTY0 + (it & 1)));
        for (int j = it; j < it + n_loc && ok; ++j) {
          const bool more = j + 1 < it + n_loc;
          ok = issue_pv(0, j);
          if (!ok) break;
          if (more) {
            ok = wait_or_abort(bar(T2_K_FULL0 + ((j + 1) & 1)), ((j + 1) >> 1) & 1, abort_flag, P.err, 514);
            if (!ok) break;
            tc_fence_after();
            issue_qk(0, j + 1);  // head A's next S while head B's softmax is still at work
          }
          ok = issue_pv(1, j);
          if (!ok) break;
          tc_commit(bar(T2_V_EMPTY0 + (j & 1)));
          if (more) {
            issue_qk(1, j + 1);
            tc_commit(bar(T2_K_EMPTY0 + ((j + 1) & 1)));
          }
        }
        tc_commit(bar(T2_Q_EMPTY));  // every product that reads this stage's Q tiles has been issued
        it += n_loc;
      }
      if (ok) tc_commit(bar(T2_O_FULL));
    }
  } else {
    // ===================================================================== softmax / epilogue
    // warps 0-7 serve head A, 8-15 head B; in each group warp w and w+4 own the same 32 query rows (TMEM lanes)
    // and split the tile's 128 key columns in halves
    const int x = warp >> 3, wq = warp & 7;
    const int quad = wq & 3, half = wq >> 2;
    const int row = quad * 32 + lane;
    const int64_t qi = i0 + row;
    const bool row_valid = qi < P.lq;
    const uint32_t lane_base = ((uint32_t)(quad * 32)) << 16;
    const int col0 = half * 64;
    const uint32_t tS = tmem + x * 128 + lane_base, tO = tmem + 256 + x * 128 + lane_base;
    float* gmax = xmax + x * 512;
    float* gsum = xsum + x * 256;
    volatile int* gflag = xflag + x * 256;
    float m_ref = -INFINITY, l_part = 0.f;  // m_ref in the scaled log2 domain; l over this thread's columns
    int g = 0, it = 0;
    bool ok = true;
    for (int st = 0; st < P.n_stage && ok; ++st) {
      const TcStage& S = P.stage[st];
      int64_t vis_lo, vis_hi;
      visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
      if (vis_lo > vis_hi) continue;
      // keys [jlo, jhi] of this stage are visible to this thread's query row
      int64_t jlo = 0, jhi = S.lk - 1;
      if (S.mask_mode == INFLLM_MASK_WINDOW) {
        jlo = qi + S.mask_offset - S.mask_size + 1;
        jhi = qi + S.mask_offset;
      } else if (S.mask_mode == INFLLM_MASK_COMPLEMENT) {
        jhi = qi + S.mask_offset - S.mask_size;
      }
      if (!row_valid) jhi = -1, jlo = 0;
      int64_t seg_j0 = 0;
      for (int sg = S.seg_begin; sg < S.seg_end && ok; ++sg) {
        const TcSeg& G = P.seg[sg];
        int tf, tl;
        if (seg_tiles(vis_lo, vis_hi, seg_j0, G.len, &tf, &tl)) {
          for (int t = tf; t <= tl && ok; ++t, ++g) {
            if (g < g0 || g >= g1) continue;
            ok = __all_sync(0xffffffffu, wait_or_abort(bar(T2_S_FULLA + x), it & 1, abort_flag, P.err, 520));
            if (!ok) break;
            tc_fence_after();
            // visible columns of this tile for this row, relative to this thread's 64 columns
            const int64_t jt = seg_j0 + (int64_t)t * kTile;
            const int64_t lim = seg_j0 + G.len - 1;
            const int64_t a = jlo > jt ? jlo : jt, e = jhi < lim ? jhi : lim;
            const int c_lo = (int)(a - jt) - col0;
            const int c_hi = (int)((e - jt) > (kTile - 1) ? (kTile - 1) : (e - jt)) - col0;
            const bool full = c_lo <= 0 && c_hi >= 63;
            // ---- pass 1: row maximum of the raw scores
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              float s[32];
              tmem_ld32(tS + col0 + cc * 32, reinterpret_cast<uint32_t*>(s));
              tmem_wait_ld();
              if (full) {
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                  mx4[0] = fmaxf(mx4[0], s[c]);
                  mx4[1] = fmaxf(mx4[1], s[c + 1]);
                  mx4[2] = fmaxf(mx4[2], s[c + 2]);
                  mx4[3] = fmaxf(mx4[3], s[c + 3]);
                }
              } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                  const int cg = cc * 32 + c;
                  mx4[c & 3] = fmaxf(mx4[c & 3], (cg >= c_lo && cg <= c_hi) ? s[c] : -INFINITY);
                }
              }
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the other half's maximum of the same row
            gmax[(it & 1) * 256 + half * 128 + row] = mx;
            __threadfence_block();
            gflag[half * 128 + row] = it + 1;
            ok = __all_sync(0xffffffffu, pair_wait(&gflag[(half ^ 1) * 128 + row], it + 1, abort_flag, P.err, 521));
            if (!ok) break;
            mx = fmaxf(mx, gmax[(it & 1) * 256 + (half ^ 1) * 128 + row]) * P.scale_log2;
            // lazy rescaling: the reference maximum only moves when the row maximum grew by more than 2^8
            float alpha = 1.f;
            bool resc = false;
            if (mx > m_ref) {
              if (m_ref == -INFINITY) {
                m_ref = mx;  // nothing accumulated for this row yet
              } else if (mx - m_ref > 8.f) {
                alpha = ex2_approx(m_ref - mx);
                l_part *= alpha;
                m_ref = mx;
                resc = true;
              }
            }
            // O of this head is quiet here: S of this tile being complete implies that the previous P V is too
            if (__any_sync(0xffffffffu, resc) && it >= 1) {
#pragma unroll
              for (int cc = 0; cc < 2; ++cc) {
                uint32_t o[32];
                tmem_ld32(tO + col0 + cc * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
                tmem_st32(tO + col0 + cc * 32, o);
              }
              tmem_wait_st();
            }
            // ---- pass 2: P = exp2(S * scale - m), two exponentials per instruction, packed 16-bit pairs
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              float s[32];
              uint32_t pk[16];
              tmem_ld32(tS + col0 + cc * 32, reinterpret_cast<uint32_t*>(s));
              tmem_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; c += 4) {
                float a0 = fmaf(s[c], P.scale_log2, neg_m), a1 = fmaf(s[c + 1], P.scale_log2, neg_m);
                float a2 = fmaf(s[c + 2], P.scale_log2, neg_m), a3 = fmaf(s[c + 3], P.scale_log2, neg_m);
                if (!full) {
                  const int cg = cc * 32 + c;
                  a0 = (cg >= c_lo && cg <= c_hi) ? a0 : -INFINITY;
                  a1 = (cg + 1 >= c_lo && cg + 1 <= c_hi) ? a1 : -INFINITY;
                  a2 = (cg + 2 >= c_lo && cg + 2 <= c_hi) ? a2 : -INFINITY;
                  a3 = (cg + 3 >= c_lo && cg + 3 <= c_hi) ? a3 : -INFINITY;
                }
                const float2 p01 = ex2_pair(a0, a1), p23 = ex2_pair(a2, a3);
                rs4[0] += p01.x; rs4[1] += p01.y; rs4[2] += p23.x; rs4[3] += p23.y;
                typename Act<T>::T2 v01 = Act<T>::from_f2(p01.x, p01.y), v23 = Act<T>::from_f2(p23.x, p23.y);
                pk[c >> 1] = *reinterpret_cast<uint32_t*>(&v01);
                pk[(c >> 1) + 1] = *reinterpret_cast<uint32_t*>(&v23);
              }
              // 32 keys of P, packed, over S columns this thread has already consumed
              tmem_st16(tS + col0 + cc * 16, pk);
            }
            l_part += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(T2_P_FULLA + x));
            ++it;
          }
        }
        seg_j0 += G.len;
      }
    }
    // ---- epilogue (each half handles its 64 output columns)
    gsum[half * 128 + row] = l_part;
    __threadfence_block();
    gflag[half * 128 + row] = kPairDone;
    if (ok) ok = __all_sync(0xffffffffu, pair_wait(&gflag[(half ^ 1) * 128 + row], kPairDone, abort_flag, P.err, 522));
    const float l_sum = l_part + gsum[(half ^ 1) * 128 + row];
    if (ok && it >= 1) ok = __all_sync(0xffffffffu, wait_or_abort(bar(T2_O_FULL), 0, abort_flag, P.err, 523));
    if (ok) {
      tc_fence_after();
      const int h = hA + x;
      if (P.n_split == 1) {
        const float inv = (it >= 1 && l_sum > 0.f) ? 1.f / l_sum : 0.f;
        T* orow = (T*)P.out + (int64_t)h * P.o_hs + qi * P.o_ts + col0;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t o[32];
          if (it >= 1) {
            tmem_ld32(tO + col0 + cc * 32, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = 0;
          }
          if (row_valid) {
#pragma unroll
            for (int k = 0; k < 32; k += 8) {
              uint4 v;
              uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                typename Act<T>::T2 v2 = Act<T>::from_f2(__uint_as_float(o[k + 2 * e]) * inv,
                                                         __uint_as_float(o[k + 2 * e + 1]) * inv);
                pv[e] = *reinterpret_cast<uint32_t*>(&v2);
              }
              *reinterpret_cast<uint4*>(orow + cc * 32 + k) = v;
            }
          }
        }
        if (half == 0 && row_valid && P.lse) P.lse[(int64_t)h * P.lq + qi] = l_sum > 0.f ? m_ref + log2f(l_sum) : -INFINITY;
      } else {
        // un-normalised partial of this run of key tiles
        const int64_t prow = ((int64_t)split * P.n_heads + h) * P.lq + qi;
        float* arow = P.part_acc + prow * 128 + col0;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t o[32];
          if (it >= 1) {
            tmem_ld32(tO + col0 + cc * 32, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = 0;
          }
          if (row_valid) {
#pragma unroll
            for (int k = 0; k < 32; k += 4)
              *reinterpret_cast<uint4*>(arow + cc * 32 + k) = make_uint4(o[k], o[k + 1], o[k + 2], o[k + 3]);
          }
        }
        if (half == 0 && row_valid) {
          P.part_m[prow] = m_ref;
          P.part_l[prow] = l_sum;
        }
      }
    }
  }
  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------
// attn_tc3_kernel: one 128-query tile of one head per CTA; P never touches shared memory.  P = exp2(S - m) goes back
// into the TMEM columns of its S buffer as packed 16-bit pairs and is the A operand of the P V product from there
// (a key tile moves 160 KB through shared memory: Q, K, V operand reads and the TMA fill of K and V), and there are
// three S/P buffers in TMEM, so that S runs a tile ahead of the softmax.  Eleven warps: eight softmax warps, the TMA
// producer, and one issuing thread per product (one thread for both was the longest serial chain of a tile).
// The softmax warps read S in the 16-lane shape: warps w and w+4 share a TMEM lane quarter and take 16 of its rows
// each with all 128 key columns, a row is spread over the four threads of a quad, so a row maximum is two shuffles
// and no thread waits for another warp.  Every fourth pair of exponentials is a cubic on the FMA pipe.  The producer
// asks for K one tile ahead of V (the V buffer frees late in a tile's cycle and K(t+1) queued behind that wait).
// What the clock stamps of one CTA say (cycles per 128-key tile, 131072-token prefill): the period is 2100-2200 and
// it is the softmax warps' (1700 of work, 400 of waits and loop); S is ready 2000 cycles before they come for it; a
// K or V tile takes 900-1000 cycles from request to arrival, which is also what the loads alone allow (a CTA whose
// softmax does nothing and whose P V products are left out still needs 1600 per tile: four 16 KB boxes at about 40
// bytes per clock and SM from L2).  Tried and not kept: a second softmax team on alternate tiles with its own S
// buffer and accumulator (the chain S -> softmax -> P V -> next S of one team is as long as two tiles; 94 us),
// asking TMEM for the next tile's scores before this tile's exponentials (111 us), an L2 prefetch of the key tiles
// four to eight tiles ahead (no change), all exponentials or half of them on the special-function unit (87, 86 us).
// 83 us per exec block of the 128K prefill.
namespace tc3 {
constexpr int kQ = 0;
constexpr int kK = kQ + 2 * kSubTileBytes;       // two stages
constexpr int kV = kK + 4 * kSubTileBytes;       // two stages
constexpr int kBar = kV + 4 * kSubTileBytes;
constexpr int kXmax = kBar + 256;                // reference maxima of the 128 rows, for the epilogue's layout
constexpr int kXsum = kXmax + 512;               // row sums of the 128 rows
constexpr int kTotal = kXsum + 512;
constexpr int kPolyEvery = 4;
enum { T3_Q_FULL = 0, T3_Q_EMPTY, T3_K_FULL0, T3_K_FULL1, T3_K_EMPTY0, T3_K_EMPTY1, T3_V_FULL0, T3_V_FULL1, T3_V_EMPTY0,
       T3_V_EMPTY1, T3_S_FULL0, T3_S_FULL1, T3_S_FULL2, T3_P_FULL0, T3_P_FULL1, T3_P_FULL2, T3_PV_DONE0, T3_PV_DONE1, T3_PV_DONE2,
       T3_O_FULL, T3_N_BARS };
}  // namespace tc3

template <typename T>
__global__ void __launch_bounds__(352, 1) attn_tc3_kernel(const __grid_constant__ AttnTcParams P) {
  using namespace tc3;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t sQ = s_base + kQ, sK = s_base + kK, sV = s_base + kV;
  const uint32_t bars = s_base + kBar;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kBar + T3_N_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kBar + T3_N_BARS * 8 + 8);
  float* xmax = reinterpret_cast<float*>(smem + kXmax);
  float* xsum = reinterpret_cast<float*>(smem + kXsum);
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, hkv = h / (P.n_heads / P.n_kv_heads);
  const int64_t i0 = (int64_t)blockIdx.x * kTile;
  const int rows_q = (int)((P.lq - i0) < kTile ? (P.lq - i0) : kTile);

  if (threadIdx.x == 0) {
    for (int i = 0; i < T3_N_BARS; ++i) mbar_init(bar(i), (i >= T3_P_FULL0 && i <= T3_P_FULL2) ? 256u : 1u);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tO = tmem + 384;  // three S/P buffers at columns [0,128), [128,256), [256,384)
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  constexpr uint32_t idesc_qk = make_idesc(kBf16, 128, 128, false);
  constexpr uint32_t idesc_pv = make_idesc(kBf16, 128, 128, true);

  if (warp == 8) {
    // ======================================================================== TMA producer
    // K runs one tile ahead of V: the buffer of K(t+1) is free as soon as S(t-1) has been formed, that of V(t) only
    // when the P V product of tile t-2 has run, late in the tile's cycle; asked for in tile order, K(t+1) queued
    // behind that wait and S(t+1) was not ready when the softmax warps came for it.
    if (lane == 0) {
      int it = 0, sidx = 0;
      bool ok = true;
      struct { int it, tok, c3, map; } pend = {-1, 0, 0, 0};  // the V tile that has not been asked for yet
      auto load_v = [&]() {
        const int b = pend.it & 1;
        if (pend.it >= 2) ok = wait_or_abort(bar(T3_V_EMPTY0 + b), ((pend.it >> 1) - 1) & 1, abort_flag, P.err, 602);
        if (!ok) return;
        const uint32_t dv = sV + b * 2 * kSubTileBytes;
        mbar_expect_tx(bar(T3_V_FULL0 + b), 2 * kSubTileBytes);
        if (pend.c3 < 0) {
          tma_load_3d(dv, &P.maps[pend.map], bar(T3_V_FULL0 + b), 0, pend.tok, hkv);
          tma_load_3d(dv + kSubTileBytes, &P.maps[pend.map], bar(T3_V_FULL0 + b), 64, pend.tok, hkv);
        } else {
          tma_load_4d(dv, &P.maps[pend.map], bar(T3_V_FULL0 + b), 0, pend.tok, hkv, pend.c3);
          tma_load_4d(dv + kSubTileBytes, &P.maps[pend.map], bar(T3_V_FULL0 + b), 64, pend.tok, hkv, pend.c3);
        }
        pend.it = -1;
      };
      for (int st = 0; st < P.n_stage && ok; ++st) {
        const TcStage& S = P.stage[st];
        int64_t vis_lo, vis_hi;
        visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
        if (vis_lo > vis_hi) continue;
        if (stage_tiles(P, S, vis_lo, vis_hi) == 0) continue;
        if (sidx >= 1) ok = wait_or_abort(bar(T3_Q_EMPTY), (sidx - 1) & 1, abort_flag, P.err, 600);
        if (!ok) break;
        mbar_expect_tx(bar(T3_Q_FULL), 2 * kSubTileBytes);
        tma_load_3d(sQ, &P.maps[S.map_q], bar(T3_Q_FULL), 0, S.q_row0 + (int)i0, h);
        tma_load_3d(sQ + kSubTileBytes, &P.maps[S.map_q], bar(T3_Q_FULL), 64, S.q_row0 + (int)i0, h);
        ++sidx;
        int64_t seg_j0 = 0;
        for (int sg = S.seg_begin; sg < S.seg_end && ok; ++sg) {
          const TcSeg& G = P.seg[sg];
          int tf, tl;
          if (seg_tiles(vis_lo, vis_hi, seg_j0, G.len, &tf, &tl)) {
            for (int t = tf; t <= tl && ok; ++t, ++it) {
              const int b = it & 1, tok = G.tok0 + t * kTile;
              if (it >= 2) ok = wait_or_abort(bar(T3_K_EMPTY0 + b), ((it >> 1) - 1) & 1, abort_flag, P.err, 601);
              if (!ok) break;
              const uint32_t dk = sK + b * 2 * kSubTileBytes;
              mbar_expect_tx(bar(T3_K_FULL0 + b), 2 * kSubTileBytes);
              if (G.c3_k < 0) {
                tma_load_3d(dk, &P.maps[G.map_k], bar(T3_K_FULL0 + b), 0, tok, hkv);
                tma_load_3d(dk + kSubTileBytes, &P.maps[G.map_k], bar(T3_K_FULL0 + b), 64, tok, hkv);
              } else {
                tma_load_4d(dk, &P.maps[G.map_k], bar(T3_K_FULL0 + b), 0, tok, hkv, G.c3_k);
                tma_load_4d(dk + kSubTileBytes, &P.maps[G.map_k], bar(T3_K_FULL0 + b), 64, tok, hkv, G.c3_k);
              }
              if (pend.it >= 0) load_v();
              if (!ok) break;
              pend.it = it, pend.tok = tok, pend.c3 = G.c3_v, pend.map = G.map_v;
            }
          }
          seg_j0 += G.len;
        }
      }
      if (ok && pend.it >= 0) load_v();
      if (!ok) {
        // give loads that are still in flight a bounded chance to land before the CTA's memory goes away
        for (int b = 0; b < 2; ++b) {
          for (uint32_t i = 0; i < 4096 && !mbar_try_wait(bar(T3_K_FULL0 + b), 0) && !mbar_try_wait(bar(T3_K_FULL0 + b), 1); ++i) __nanosleep(64);
          for (uint32_t i = 0; i < 4096 && !mbar_try_wait(bar(T3_V_FULL0 + b), 0) && !mbar_try_wait(bar(T3_V_FULL0 + b), 1); ++i) __nanosleep(64);
        }
      }
    }
  } else if (warp == 9 || warp == 10) {
    // ========================================================================== MMA issuers
    // Two threads: warp 10 issues S = Q K^T, warp 9 issues O += P V.  One thread doing both was the longest serial
    // chain of a key tile (waits, 16 products that each hold the thread while the pipe is busy, commits: about
    // 2500 cycles); apart they take about 1100 each and the softmax sets the pace.  What the tensor pipe ordered
    // before - S of tile t+2 may overwrite its buffer only when P V of tile t has read P from it - is now the
    // wait for that product's commit.
    if (lane == 0) {
      int nt[kMaxStage], n_act = 0, n = 0;  // tiles per stage that has any, in order
      for (int st = 0; st < P.n_stage; ++st) {
        const TcStage& S = P.stage[st];
        int64_t vis_lo, vis_hi;
        visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
        if (vis_lo > vis_hi) continue;
        const int c = stage_tiles(P, S, vis_lo, vis_hi);
        if (c > 0) nt[n_act++] = c, n += c;
      }
      bool ok = true;
      if (warp == 10) {
        const uint64_t qd0 = make_sdesc(sQ, 16, 1024);
        const uint64_t kd0[2] = {make_sdesc(sK, 16, 1024), make_sdesc(sK + 2 * kSubTileBytes, 16, 1024)};
        int sq = 0, tq = 0;
        for (int iq = 0; iq < n && ok; ++iq) {
          const int b = iq & 1;
          if (tq == 0) ok = wait_or_abort(bar(T3_Q_FULL), sq & 1, abort_flag, P.err, 610);
          if (ok) ok = wait_or_abort(bar(T3_K_FULL0 + b), (iq >> 1) & 1, abort_flag, P.err, 611);
          const int b3 = iq % 3;  // S/P buffer: free once the P V product of tile iq-3 has read P from it
          if (ok && iq >= 3) ok = wait_or_abort(bar(T3_PV_DONE0 + b3), ((iq / 3) - 1) & 1, abort_flag, P.err, 614);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t off = (uint64_t)(((ks >> 2) * kSubTileBytes + (ks & 3) * 32) >> 4);
            mma_ss(tmem + b3 * 128, qd0 + off, kd0[b] + off, idesc_qk, ks > 0);
          }
          tc_commit(bar(T3_S_FULL0 + b3));
          tc_commit(bar(T3_K_EMPTY0 + b));
          if (++tq == nt[sq]) {
            tc_commit(bar(T3_Q_EMPTY));  // the last product that reads this stage's Q tile
            ++sq;
            tq = 0;
          }
        }
      } else {
        const uint64_t vd0[2] = {make_sdesc(sV, kSubTileBytes, 1024), make_sdesc(sV + 2 * kSubTileBytes, kSubTileBytes, 1024)};
        for (int ip = 0; ip < n && ok; ++ip) {
          const int b = ip & 1;
          const int b3 = ip % 3;
          ok = wait_or_abort(bar(T3_P_FULL0 + b3), (ip / 3) & 1, abort_flag, P.err, 612);
          ok = ok && wait_or_abort(bar(T3_V_FULL0 + b), (ip >> 1) & 1, abort_flag, P.err, 613);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            // A = P from TMEM: keys 0-63 in the buffer's columns [0,32), keys 64-127 in [64,96)
            const uint32_t a_t = tmem + b3 * 128 + 8 * ks;
            mma_ts(tO, a_t, vd0[b] + (uint64_t)((ks * 2048) >> 4), idesc_pv, (ip > 0) || (ks > 0));
          }
          tc_commit(bar(T3_V_EMPTY0 + b));
          tc_commit(bar(T3_PV_DONE0 + b3));
        }
        if (ok) tc_commit(bar(T3_O_FULL));
      }
    }
  } else if (warp < 8) {
    // ===================================================================== softmax / epilogue
    // Eight warps: warps w and w+4 share a TMEM lane quarter and take 16 of its query rows each, with all 128 key
    // columns of those rows: the 16x256b load spreads a row over the four threads of a quad, so a row maximum is two
    // shuffles and no thread waits for another warp.  A thread holds rows r and r+8, two columns of every block of 8.
    const int quad = warp & 3, rh = warp >> 2;
    const int rbase = quad * 32 + rh * 16 + (lane >> 2);
    const int cq = 2 * (lane & 3);
    const uint32_t lane_base = ((uint32_t)(quad * 32 + rh * 16)) << 16;
    const int64_t qrow[2] = {i0 + rbase, i0 + rbase + 8};
    const bool valid[2] = {qrow[0] < P.lq, qrow[1] < P.lq};
    float m_ref[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};
    int it = 0;
    bool ok = true;
    for (int st = 0; st < P.n_stage && ok; ++st) {
      const TcStage& S = P.stage[st];
      int64_t vis_lo, vis_hi;
      visible_key_range(S.mask_mode, S.mask_offset, S.mask_size, i0, i0 + rows_q - 1, S.lk, &vis_lo, &vis_hi);
      if (vis_lo > vis_hi) continue;
      int64_t jlo[2], jhi[2];  // keys of this stage visible to this thread's two query rows
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        jlo[r] = 0, jhi[r] = S.lk - 1;
        if (S.mask_mode == INFLLM_MASK_WINDOW) {
          jlo[r] = qrow[r] + S.mask_offset - S.mask_size + 1;
          jhi[r] = qrow[r] + S.mask_offset;
        } else if (S.mask_mode == INFLLM_MASK_COMPLEMENT) {
          jhi[r] = qrow[r] + S.mask_offset - S.mask_size;
        }
        if (!valid[r]) jhi[r] = -1, jlo[r] = 0;
      }
      int64_t seg_j0 = 0;
      for (int sg = S.seg_begin; sg < S.seg_end && ok; ++sg) {
        const TcSeg& G = P.seg[sg];
        int tf, tl;
        if (seg_tiles(vis_lo, vis_hi, seg_j0, G.len, &tf, &tl)) {
          for (int t = tf; t <= tl && ok; ++t, ++it) {
            const int b3 = it % 3;
            const uint32_t tS = tmem + b3 * 128 + lane_base;
            ok = __all_sync(0xffffffffu, wait_or_abort(bar(T3_S_FULL0 + b3), (it / 3) & 1, abort_flag, P.err, 620));
            if (!ok) break;
            tc_fence_after();
            float s[64];
            tmem_ld_16x256b_x16(tS, reinterpret_cast<uint32_t*>(s));
            tmem_wait_ld();
            const int64_t jt = seg_j0 + (int64_t)t * kTile;
            const int64_t lim = seg_j0 + G.len - 1;  // last key of the segment
            int c_lo[2], c_hi[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const int64_t a = jlo[r] > jt ? jlo[r] : jt, e = jhi[r] < lim ? jhi[r] : lim;
              c_lo[r] = (int)(a - jt);
              c_hi[r] = (int)((e - jt) > (kTile - 1) ? (kTile - 1) : (e - jt));
            }
            if (!(c_lo[0] <= 0 && c_hi[0] >= kTile - 1 && c_lo[1] <= 0 && c_hi[1] >= kTile - 1)) {
#pragma unroll
              for (int i = 0; i < 64; ++i) {
                const int col = 8 * (i >> 2) + cq + (i & 1), r = (i >> 1) & 1;
                s[i] = (col >= c_lo[r] && col <= c_hi[r]) ? s[i] : -INFINITY;
              }
            }
            float mxa[2] = {-INFINITY, -INFINITY}, mxb[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              mxa[0] = fmax3(mxa[0], s[4 * j], s[4 * j + 1]);
              mxa[1] = fmax3(mxa[1], s[4 * j + 2], s[4 * j + 3]);
              mxb[0] = fmax3(mxb[0], s[4 * j + 4], s[4 * j + 5]);
              mxb[1] = fmax3(mxb[1], s[4 * j + 6], s[4 * j + 7]);
            }
            float alpha[2] = {1.f, 1.f}, neg_m[2];
            bool resc = false;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              float mx = fmaxf(mxa[r], mxb[r]);
              mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
              mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2)) * P.scale_log2;
              // lazy rescaling: the reference maximum only moves when the row maximum grew by more than 2^8
              if (mx > m_ref[r]) {
                if (m_ref[r] == -INFINITY) {
                  m_ref[r] = mx;  // nothing accumulated for this row yet
                } else if (mx - m_ref[r] > 8.f) {
                  alpha[r] = ex2_approx(m_ref[r] - mx);
                  l_part[r] *= alpha[r];
                  m_ref[r] = mx;
                  resc = true;
                }
              }
              neg_m[r] = m_ref[r] == -INFINITY ? 0.f : -m_ref[r];
            }
            uint32_t pk[32];
            float2 rs[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            const float2 sc2 = make_float2(P.scale_log2, P.scale_log2);
            const float2 nm2[2] = {make_float2(neg_m[0], neg_m[0]), make_float2(neg_m[1], neg_m[1])};
#pragma unroll
            for (int k = 0; k < 32; ++k) {  // pair k: block k/2, row k%2 - which is where the 16x128b store wants it
              const int r = k & 1;
              const float2 a = ffma2(s[2 * k], s[2 * k + 1], sc2, nm2[r]);
              float2 p;
              if ((k % kPolyEvery) == kPolyEvery - 1) {
                p = ex2_poly2(a);  // one pair in kPolyEvery off the special-function unit
              } else {
                p = make_float2(ex2_approx(a.x), ex2_approx(a.y));
              }
              rs[r] = fadd2(rs[r], p);
              typename Act<T>::T2 v = Act<T>::from_f2(p.x, p.y);
              pk[k] = *reinterpret_cast<uint32_t*>(&v);
            }
            l_part[0] += rs[0].x + rs[0].y;
            l_part[1] += rs[1].x + rs[1].y;
            if (__any_sync(0xffffffffu, resc) && it >= 1) {
              // O holds the products up to tile it-1: wait for the last of them, then scale this warp's 16 rows
              ok = __all_sync(0xffffffffu, wait_or_abort(bar(T3_PV_DONE0 + ((it - 1) % 3)), ((it - 1) / 3) & 1, abort_flag,
                                                         P.err, 622));
              if (!ok) break;
              tc_fence_after();
              uint32_t o[64];
              tmem_ld_16x256b_x16(tO + lane_base, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 64; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha[(i >> 1) & 1]);
              tmem_st_16x256b_x16(tO + lane_base, o);
            }
            // P, packed, over the first 64 columns of the S buffer: column c holds keys 2c, 2c+1
            tmem_st_16x128b_x16(tS, pk);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(T3_P_FULL0 + b3));
          }
        }
        seg_j0 += G.len;
      }
    }
    // ---- epilogue: row sums and reference maxima go through shared memory to the thread-per-row layout, in which
    // each warp writes 64 output columns of 32 rows
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_part[r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if ((lane & 3) == 0) {
        xsum[rbase + 8 * r] = l;
        xmax[rbase + 8 * r] = m_ref[r];
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const int half = warp >> 2, row = quad * 32 + lane, col0 = half * 64;
    const int64_t qi = i0 + row;
    const bool row_valid = qi < P.lq;
    const uint32_t row_base = ((uint32_t)(quad * 32)) << 16;
    const float l_sum = xsum[row], m_row = xmax[row];
    if (ok && it >= 1) ok = __all_sync(0xffffffffu, wait_or_abort(bar(T3_O_FULL), 0, abort_flag, P.err, 624));
    if (ok) {
      tc_fence_after();
      const float inv = (it >= 1 && l_sum > 0.f) ? 1.f / l_sum : 0.f;
      T* orow = (T*)P.out + (int64_t)h * P.o_hs + qi * P.o_ts + col0;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        if (it >= 1) {
          tmem_ld32(tO + row_base + col0 + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) o[k] = 0;
        }
        if (row_valid) {
#pragma unroll
          for (int k = 0; k < 32; k += 8) {
            uint4 v;
            uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              typename Act<T>::T2 v2 = Act<T>::from_f2(__uint_as_float(o[k + 2 * e]) * inv,
                                                       __uint_as_float(o[k + 2 * e + 1]) * inv);
              pv[e] = *reinterpret_cast<uint32_t*>(&v2);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + k) = v;
          }
        }
      }
      if (half == 0 && row_valid && P.lse) P.lse[(int64_t)h * P.lq + qi] = l_sum > 0.f ? m_row + log2f(l_sum) : -INFINITY;
    }
  }
  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

// out = sum_s acc_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), lse = m + log2(denominator); one warp per row
template <typename T>
__global__ void attn_tc_combine_kernel(const float* __restrict__ acc, const float* __restrict__ m,
                                       const float* __restrict__ l, int n_split, int n_heads, int64_t lq,
                                       T* __restrict__ out, int64_t o_hs, int64_t o_ts, float* __restrict__ lse) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // h * lq + i
  if (row >= (int64_t)n_heads * lq) return;
  const int lane = threadIdx.x & 31;
  const int64_t h = row / lq, i = row - h * lq;
  const int64_t stride = (int64_t)n_heads * lq;
  float mx = -INFINITY;
  for (int s = 0; s < n_split; ++s) mx = fmaxf(mx, m[s * stride + row]);
  float den = 0.f;
  float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
  if (mx != -INFINITY) {
    for (int s = 0; s < n_split; ++s) {
      const float ms = m[s * stride + row];
      if (ms == -INFINITY) continue;
      const float w = exp2f(ms - mx);
      den = fmaf(w, l[s * stride + row], den);
      const float4 a = *reinterpret_cast<const float4*>(acc + (s * stride + row) * 128 + lane * 4);
      num.x = fmaf(w, a.x, num.x);
      num.y = fmaf(w, a.y, num.y);
      num.z = fmaf(w, a.z, num.z);
      num.w = fmaf(w, a.w, num.w);
    }
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  typename Act<T>::T2 v01 = Act<T>::from_f2(num.x * inv, num.y * inv), v23 = Act<T>::from_f2(num.z * inv, num.w * inv);
  uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&v01), *reinterpret_cast<uint32_t*>(&v23));
  *reinterpret_cast<uint2*>(out + h * o_hs + i * o_ts + lane * 4) = v;
  if (lane == 0 && lse) lse[row] = den > 0.f ? mx + log2f(den) : -INFINITY;
}

// ------------------------------------------------------------------------------------ column sums
// One CTA owns one query head and a run of 128-key tiles.  The head's query tiles (at most four, 512 queries)
// and their log-sum-exps stay in shared memory for the whole CTA; the key tiles stream through a two-stage TMA
// ring; every (key tile, visible query tile) pair is one S^T = K Q^T into one of four TMEM buffers, which 16
// compute warps (four threads per key row, 32 query columns each) turn into sum_q exp2(s - lse_q).  A key
// tile is loaded once per head and a query tile once per CTA, which keeps the L2 traffic an order of magnitude
// below one load per pair.
namespace colsum_smem {
constexpr int kQTiles = 4;                     // resident query tiles
constexpr int kMaxKeyTiles = 10;               // key tiles per CTA
constexpr int kBufs = 4;                       // TMEM accumulators in flight
constexpr int kQ = 0;
constexpr int kK = kQ + kQTiles * 2 * kSubTileBytes;   // two stages
constexpr int kLse = kK + 2 * 2 * kSubTileBytes;       // kQTiles x 128 fp32
constexpr int kBar = kLse + kQTiles * 512;
constexpr int kAcc = kBar + 128;               // [key tile][column quarter][key] partial sums
constexpr int kTotal = kAcc + kMaxKeyTiles * 4 * 128 * 4;
}  // namespace colsum_smem

// query tiles [tf, tl] that can see a key of the tile starting at j0 (tl < tf: none)
__device__ __forceinline__ void colsum_q_tiles(const ColsumTcParams& P, int64_t j0, int keys, int* tf, int* tl) {
  int64_t lo = 0, hi = P.lq - 1;
  if (P.mask_mode == INFLLM_MASK_WINDOW) {
    lo = j0 - P.mask_offset;
    hi = j0 + keys - 1 - P.mask_offset + P.mask_size - 1;
  } else if (P.mask_mode == INFLLM_MASK_COMPLEMENT) {
    lo = j0 - P.mask_offset + P.mask_size;
  }
  if (lo < 0) lo = 0;
  if (hi > P.lq - 1) hi = P.lq - 1;
  if (lo > hi) {
    *tf = 0;
    *tl = -1;
  } else {
    *tf = (int)(lo / kTile);
    *tl = (int)(hi / kTile);
  }
}

template <typename T>
__global__ void __launch_bounds__(576, 1) colsum_tc_kernel(const __grid_constant__ ColsumTcParams P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t sQ = s_base + colsum_smem::kQ, sK = s_base + colsum_smem::kK;
  float* s_lse = reinterpret_cast<float*>(smem + colsum_smem::kLse);
  float* s_acc = reinterpret_cast<float*>(smem + colsum_smem::kAcc);
  const uint32_t bars = s_base + colsum_smem::kBar;
  constexpr int NB = colsum_smem::kBufs;
  // barriers: 0 q_full, 1-2 k_full, 3-4 k_free, then s_full[NB], free[NB]
  constexpr int KF = 1, KE = 3, SF = 5, FR = 5 + NB;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + colsum_smem::kBar + 112);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + colsum_smem::kBar + 120);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, hkv = h / P.group;
  const int n_key_tiles = (int)((P.lk + kTile - 1) / kTile);
  const int kt0 = blockIdx.x * P.tiles_per_cta;
  const int kt1 = kt0 + P.tiles_per_cta < n_key_tiles ? kt0 + P.tiles_per_cta : n_key_tiles;
  if (threadIdx.x == 0) {
    mbar_init(bar(0), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(KF + i), 1);
      mbar_init(bar(KE + i), 1);
    }
    for (int i = 0; i < NB; ++i) {
      mbar_init(bar(SF + i), 1);
      mbar_init(bar(FR + i), 512);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < colsum_smem::kMaxKeyTiles * 4 * 128; i += blockDim.x) s_acc[i] = 0.f;
  for (int i = threadIdx.x; i < colsum_smem::kQTiles * 128; i += blockDim.x)
    s_lse[i] = i < P.lq ? P.lse[(int64_t)h * P.lq + i] : INFINITY;
  if (warp == 17) {
    tmem_alloc(smem_u32(tmem_slot), 128 * NB);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  constexpr uint32_t idesc = make_idesc(kBf16, 128, 128, false);

  // the query tiles any key tile of this CTA needs
  int q_first = 1 << 30, q_last = -1;
  for (int kt = kt0; kt < kt1; ++kt) {
    const int64_t j0 = (int64_t)kt * kTile;
    const int keys = (int)((P.lk - j0) < kTile ? (P.lk - j0) : kTile);
    int tf, tl;
    colsum_q_tiles(P, j0, keys, &tf, &tl);
    if (tl >= tf) {
      q_first = tf < q_first ? tf : q_first;
      q_last = tl > q_last ? tl : q_last;
    }
  }
  const bool any = q_last >= q_first;

  if (warp == 16) {
    // ============================================================== producer: query tiles once, then key tiles
    if (lane == 0 && any) {
      mbar_expect_tx(bar(0), (uint32_t)(q_last - q_first + 1) * 2 * kSubTileBytes);
      for (int t = q_first; t <= q_last; ++t) {
        tma_load_3d(sQ + t * 2 * kSubTileBytes, &P.map_q, bar(0), 0, P.q_row0 + t * kTile, h);
        tma_load_3d(sQ + t * 2 * kSubTileBytes + kSubTileBytes, &P.map_q, bar(0), 64, P.q_row0 + t * kTile, h);
      }
      bool ok = true;
      int n = 0;  // key tiles with work, in order
      for (int kt = kt0; kt < kt1 && ok; ++kt) {
        const int64_t j0 = (int64_t)kt * kTile;
        const int keys = (int)((P.lk - j0) < kTile ? (P.lk - j0) : kTile);
        int tf, tl;
        colsum_q_tiles(P, j0, keys, &tf, &tl);
        if (tl < tf) continue;
        const int b = n & 1;
        if (n >= 2) ok = wait_or_abort(bar(KE + b), ((n >> 1) - 1) & 1, abort_flag, P.err, 410);
        if (!ok) break;
        mbar_expect_tx(bar(KF + b), 2 * kSubTileBytes);
        tma_load_3d(sK + b * 2 * kSubTileBytes, &P.map_k, bar(KF + b), 0, P.k_tok0 + (int)j0, hkv);
        tma_load_3d(sK + b * 2 * kSubTileBytes + kSubTileBytes, &P.map_k, bar(KF + b), 64, P.k_tok0 + (int)j0, hkv);
        ++n;
      }
    }
  } else if (warp == 17) {
    // ======================================================================================= MMA issuer
    if (lane == 0 && any) {
      bool ok = wait_or_abort(bar(0), 0, abort_flag, P.err, 411);
      int n = 0, step = 0;
      for (int kt = kt0; kt < kt1 && ok; ++kt) {
        const int64_t j0 = (int64_t)kt * kTile;
        const int keys = (int)((P.lk - j0) < kTile ? (P.lk - j0) : kTile);
        int tf, tl;
        colsum_q_tiles(P, j0, keys, &tf, &tl);
        if (tl < tf) continue;
        const int kb = n & 1;
        ok = wait_or_abort(bar(KF + kb), (n >> 1) & 1, abort_flag, P.err, 412);
        const uint32_t kt_s = sK + kb * 2 * kSubTileBytes;
        for (int t = tf; t <= tl && ok; ++t, ++step) {
          const int b = step % NB;
          if (step >= NB) ok = wait_or_abort(bar(FR + b), ((step / NB) - 1) & 1, abort_flag, P.err, 413);
          if (!ok) break;
          tc_fence_after();
          const uint32_t qt = sQ + t * 2 * kSubTileBytes;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            // S^T = K Q^T: keys are the M rows (TMEM lanes), queries the N columns
            uint64_t ad = make_sdesc(kt_s + (ks >> 2) * kSubTileBytes + (ks & 3) * 32, 16, 1024);
            uint64_t bd = make_sdesc(qt + (ks >> 2) * kSubTileBytes + (ks & 3) * 32, 16, 1024);
            mma_ss(tmem + b * 128, ad, bd, idesc, ks > 0);
          }
          tc_commit(bar(SF + b));
        }
        if (ok) tc_commit(bar(KE + kb));  // every product that reads this key tile has been issued
        ++n;
      }
    }
  } else {
    // ========================================================================================== compute
    const int quad = warp & 3, part = warp >> 2;
    const int krow = quad * 32 + lane;
    const int col0 = part * 32;
    const uint32_t lane_base = ((uint32_t)(quad * 32)) << 16;
    bool ok = true;
    int step = 0, n = 0;
    for (int kt = kt0; kt < kt1 && ok; ++kt) {
      const int64_t j0 = (int64_t)kt * kTile;
      const int keys = (int)((P.lk - j0) < kTile ? (P.lk - j0) : kTile);
      int tf, tl;
      colsum_q_tiles(P, j0, keys, &tf, &tl);
      if (tl < tf) continue;
      // queries that see this thread's key
      const int64_t kj = j0 + krow;
      int64_t vi_lo = 0, vi_hi = P.lq - 1;
      if (P.mask_mode == INFLLM_MASK_WINDOW) {
        vi_lo = kj - P.mask_offset;
        vi_hi = kj - P.mask_offset + P.mask_size - 1;
      } else if (P.mask_mode == INFLLM_MASK_COMPLEMENT) {
        vi_lo = kj - P.mask_offset + P.mask_size;
      }
      if (vi_lo < 0) vi_lo = 0;
      if (vi_hi > P.lq - 1) vi_hi = P.lq - 1;
      if (kj >= P.lk) vi_hi = -1;
      float total = 0.f;
      for (int t = tf; t <= tl && ok; ++t, ++step) {
        const int b = step % NB;
        ok = __all_sync(0xffffffffu, wait_or_abort(bar(SF + b), (step / NB) & 1, abort_flag, P.err, 414));
        if (!ok) break;
        tc_fence_after();
        float sv[32];
        tmem_ld32(tmem + b * 128 + lane_base + col0, reinterpret_cast<uint32_t*>(sv));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(bar(FR + b));  // the accumulator is in registers: the buffer can be overwritten
        const int64_t q0 = (int64_t)t * kTile + col0;
        const int64_t a = vi_lo > q0 ? vi_lo : q0, e = vi_hi < q0 + 31 ? vi_hi : q0 + 31;
        const int c_lo = (int)(a - q0), c_hi = (int)(e - q0);
        const float* ls = s_lse + t * kTile + col0;
        float acc4[4] = {0.f, 0.f, 0.f, 0.f};
        if (c_lo == 0 && c_hi == 31) {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(ls + c);
            const float2 p01 = ex2_pair(fmaf(sv[c], P.scale_log2, -l4.x), fmaf(sv[c + 1], P.scale_log2, -l4.y));
            const float2 p23 = ex2_pair(fmaf(sv[c + 2], P.scale_log2, -l4.z), fmaf(sv[c + 3], P.scale_log2, -l4.w));
            acc4[0] += p01.x;
            acc4[1] += p01.y;
            acc4[2] += p23.x;
            acc4[3] += p23.y;
          }
        } else if (c_lo <= c_hi) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float pv = ex2_approx(fmaf(sv[c], P.scale_log2, -ls[c]));
            acc4[c & 3] += (c >= c_lo && c <= c_hi) ? pv : 0.f;
          }
        }
        // a query row without any visible key has lse = -inf; it cannot see this key either, so it is masked above
        total += (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
      }
      // every thread owns one slot per key tile: no atomics, and the final sum below has a fixed order
      s_acc[((kt - kt0) * 4 + part) * 128 + krow] = total;
      ++n;
    }
    (void)n;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 128 && !(*abort_flag)) {
    for (int kt = kt0; kt < kt1; ++kt) {
      const int64_t kj = (int64_t)kt * kTile + threadIdx.x;
      if (kj >= P.lk) break;
      const float* sa = s_acc + ((kt - kt0) * 4) * 128 + threadIdx.x;
      const float v = (sa[0] + sa[128]) + (sa[256] + sa[384]);
      float* dst = P.score + (int64_t)h * P.score_hs + kj;
      *dst = P.accumulate ? *dst + v : v;
    }
  }
  if (warp == 17) tmem_dealloc(tmem, 128 * NB);
}

// ---------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encoder() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int encode_tensor_map(CUtensorMap* map, int dtype, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn enc = get_encoder();
  if (!enc) return fail(INFLLM_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i < rank - 1; ++i) gs[i] = strides_bytes[i];
  CUresult r = enc(map, dtype == INFLLM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(INFLLM_E_BADARG, "cuTensorMapEncodeTiled failed with code %d (rank %d, inner dim %llu)", (int)r, rank,
                (unsigned long long)dims[0]);
  return INFLLM_OK;
}

// rows of `D`=128 elements: (D, rows, heads) view of a (heads, rows, D) tensor with element strides hs / ts
int encode_rows_map(CUtensorMap* map, int dtype, const void* base, int64_t rows, int64_t heads, int64_t hs, int64_t ts) {
  uint64_t dims[3] = {128, (uint64_t)rows, (uint64_t)heads};
  uint64_t strides[2] = {(uint64_t)ts * 2, (uint64_t)hs * 2};
  uint32_t box[3] = {64, 128, 1};
  return encode_tensor_map(map, dtype, base, 3, dims, strides, box);
}

bool tc_rows_ok(const void* base, int64_t hs, int64_t ts) {
  return ((uintptr_t)base % 16) == 0 && (hs * 2) % 16 == 0 && (ts * 2) % 16 == 0 && hs > 0 && ts > 0;
}

int tc_get_error_ptr(int** p) {
  static int* cached[64] = {nullptr};  // per device ordinal
  int dev = 0;
  INFLLM_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(INFLLM_E_UNSUPPORTED, "device ordinal %d", dev);
  if (!cached[dev]) {
    void* d = nullptr;
    INFLLM_CUDA_OK(cudaGetSymbolAddress(&d, g_tc_error));
    cached[dev] = (int*)d;
  }
  *p = cached[dev];
  return INFLLM_OK;
}

int attn_tc3_launch(const AttnTcParams& P, int dtype, cudaStream_t s) {
  if (P.lq <= 0) return INFLLM_OK;
  dim3 grid((unsigned)ceil_div(P.lq, kTile), P.n_heads);
  const size_t smem = tc3::kTotal + 1024;
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    auto kern = attn_tc3_kernel<T>;
    // the opt-in holds for the current device only, and a process may drive several: asked for at every launch
    INFLLM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 352, smem, s>>>(P);
  });
  INFLLM_LAUNCH_OK("attn_tc3_kernel");
  return INFLLM_OK;
}

size_t attn_tc2_scratch_floats(int n_split, int n_heads, int64_t lq) {
  return n_split > 1 ? (size_t)n_split * n_heads * lq * (128 + 2) : 0;
}

int attn_tc2_launch(const AttnTcParams& P, int dtype, cudaStream_t s) {
  if (P.lq <= 0) return INFLLM_OK;
  const int group = P.n_heads / P.n_kv_heads;
  if (group % 2) return fail(INFLLM_E_UNSUPPORTED, "two-head attention kernel: %d query heads per kv head", group);
  if (P.n_split < 1 || (P.n_split > 1 && (!P.part_acc || !P.part_m || !P.part_l)))
    return fail(INFLLM_E_BADARG, "two-head attention kernel: split %d without partial buffers", P.n_split);
  dim3 grid((unsigned)ceil_div(P.lq, kTile), P.n_heads / 2, P.n_split);
  const size_t smem = tc2::kTotal + 1024;
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    auto kern = attn_tc2_kernel<T>;
    // the opt-in holds for the current device only, and a process may drive several: asked for at every launch
    INFLLM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 576, smem, s>>>(P);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) {
      cudaFuncAttributes fa{};
      cudaFuncGetAttributes(&fa, kern);
      return fail(INFLLM_E_CUDA, "launch of attn_tc2_kernel failed: %s (grid %u x %u x %u, 576 threads, %zu bytes dynamic + "
                  "%zu static shared memory; the kernel uses %d registers, at most %d threads per CTA)",
                  cudaGetErrorString(le), grid.x, grid.y, grid.z, smem, fa.sharedSizeBytes, fa.numRegs,
                  fa.maxThreadsPerBlock);
    }
  });
  if (P.n_split > 1) {
    const int64_t rows = (int64_t)P.n_heads * P.lq;
    INFLLM_DISPATCH_DTYPE(dtype, T, {
      attn_tc_combine_kernel<T><<<(unsigned)ceil_div(rows, 8), 256, 0, s>>>(
          P.part_acc, P.part_m, P.part_l, P.n_split, P.n_heads, P.lq, (T*)P.out, P.o_hs, P.o_ts, P.lse);
    });
    INFLLM_LAUNCH_OK("attn_tc_combine_kernel");
  }
  return INFLLM_OK;
}

int colsum_tc_launch_maps(const CUtensorMap& map_q, const CUtensorMap& map_k, int q_row0, int k_tok0, int n_heads,
                          int n_kv_heads, int64_t lq, int64_t lk, int mask_mode, int64_t mask_offset,
                          int64_t mask_size, const float* lse, float* score, int64_t score_hs, int accumulate,
                          int dtype, cudaStream_t s) {
  if (lq > colsum_smem::kQTiles * kTile)
    return fail(INFLLM_E_UNSUPPORTED, "colsum (tensor-core kernel): %lld queries, at most %d", (long long)lq,
                colsum_smem::kQTiles * kTile);
  ColsumTcParams P{};
  P.map_q = map_q; P.map_k = map_k;
  P.q_row0 = q_row0; P.k_tok0 = k_tok0; P.n_heads = n_heads; P.group = n_heads / n_kv_heads;
  P.lq = lq; P.lk = lk; P.mask_mode = mask_mode; P.accumulate = accumulate;
  P.mask_offset = mask_offset; P.mask_size = mask_size; P.lse = lse; P.score = score; P.score_hs = score_hs;
  P.scale_log2 = kLog2e / sqrtf(128.f);
  INFLLM_TRY(tc_get_error_ptr(&P.err));
  // one CTA per (head, run of key tiles): about one CTA per SM, never more than kMaxKeyTiles tiles each
  const int n_tiles = (int)ceil_div(lk, kTile);
  int chunks = std::max(1, 148 / n_heads);
  chunks = std::min(chunks, n_tiles);
  int per = (int)ceil_div(n_tiles, chunks);
  per = std::min(per, colsum_smem::kMaxKeyTiles);
  P.tiles_per_cta = per;
  dim3 grid((unsigned)ceil_div(n_tiles, per), n_heads);
  const size_t smem = colsum_smem::kTotal + 1024;
  INFLLM_DISPATCH_DTYPE(dtype, T, {
    auto kern = colsum_tc_kernel<T>;
    // the opt-in holds for the current device only, and a process may drive several: asked for at every launch
    INFLLM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 576, smem, s>>>(P);
  });
  INFLLM_LAUNCH_OK("colsum_tc_kernel");
  return INFLLM_OK;
}

int colsum_tc_launch(const void* q, int64_t q_hs, int64_t q_ts, const void* k, int64_t k_hs, int64_t k_ts, int n_heads,
                     int n_kv_heads, int64_t lq, int64_t lk, int mask_mode, int64_t mask_offset, int64_t mask_size,
                     const float* lse, float* score, int64_t score_hs, int accumulate, int dtype, cudaStream_t s) {
  CUtensorMap mq, mk;
  INFLLM_TRY(encode_rows_map(&mq, dtype, q, lq, n_heads, q_hs, q_ts));
  INFLLM_TRY(encode_rows_map(&mk, dtype, k, lk, n_kv_heads, k_hs, k_ts));
  return colsum_tc_launch_maps(mq, mk, 0, 0, n_heads, n_kv_heads, lq, lk, mask_mode, mask_offset, mask_size, lse, score,
                               score_hs, accumulate, dtype, s);
}

}  // namespace infllm

// Reads and clears the error record of the tensor-core kernels: code 0 = none, 1 = a bounded wait ran out.
// Synchronises the device.
extern "C" int infllm_device_error(int* code, int* where) {
  using namespace infllm;
  int h[4] = {0, 0, 0, 0};
  INFLLM_CUDA_OK(cudaDeviceSynchronize());
  INFLLM_CUDA_OK(cudaMemcpyFromSymbol(h, g_tc_error, sizeof(h)));
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    INFLLM_CUDA_OK(cudaMemcpyToSymbol(g_tc_error, z, sizeof(z)));
  }
  if (code) *code = h[0];
  if (where) *where = h[1];
  return INFLLM_OK;
}

extern "C" int infllm_device_error_set(int code, int where) {
  using namespace infllm;
  const int h[4] = {code, where, 0, 0};
  INFLLM_CUDA_OK(cudaDeviceSynchronize());
  INFLLM_CUDA_OK(cudaMemcpyToSymbol(g_tc_error, h, sizeof(h)));
  return INFLLM_OK;
}

