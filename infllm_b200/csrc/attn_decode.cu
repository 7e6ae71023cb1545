// Decode attention: one query token per head over a list of key/value segments.
//
// HBM-streaming split-K without shared-memory staging.  The keys of one KV head — all segments laid end to end —
// are cut into groups of 16; a CTA of 6 warps takes a contiguous run of groups (the grid is two CTAs per SM: every
// SM streams from the first cycle, nobody waits for a second wave), and a warp handles one group at a time, all the
// query heads of the KV head at once:
//   * every K and V byte goes from global memory straight into the registers of the thread that needs it as an
//     mma.sync operand — sixteen 16-byte loads per thread and group, all issued before the first is used, each warp
//     instruction covering whole 64- or 128-byte runs of a row.  The tensor-core fragments do not care in which
//     order the head dimension is summed, nor which output column stands for which dimension, so the loads can be
//     laid out for the memory system and the fragments follow (the permutation is the same for Q and K, and undone
//     when O is written);
//   * S = Q K^T as m16n8k16 products with the group's query heads as rows (rows past the group size are zero), the
//     softmax of the group in registers, then O^T += V^T P^T with the head dimension as rows and the query heads as
//     columns, whose A operand pairs the same dimension of two consecutive keys with one byte permute each.
// The warps of a CTA merge their (m, l, O) through shared memory into one normalised partial per CTA and head plus
// its log-sum-exp; infllm_lse_merge combines the partials — the runs of one GPU and, for unit-range sharding, the
// partials gathered from other GPUs.  (Folding that merge into the CTA that finishes last for a KV head was tried:
// its serial tail — 37 partials and 4 x 4096 score columns behind 192 threads — cost 50 us; a second launch of one
// wide CTA per head with every load issued up front costs 4.)
// A unit that the table of unit addresses places in the store (not in a cache slot) is read in place — over PCIe
// when the store is pinned host memory — and the rows are also written to a landing slot on the device, from where
// the host later refills the cache without a second trip over the link.
// Replaces the two attn.append calls of ContextManager._append (context_manager.py:486-489, 526-531) for
// single-token exec blocks.
#include <algorithm>

#include "attn_common.cuh"
#include "mma_common.cuh"

namespace infllm {

constexpr int kDecodeChunk = 128;  // keys per unit of the capacity rule of the allocation-free entry point
constexpr int kMaxGroup = 8;       // query heads per KV head
constexpr int kDecWarps = 6;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecMaxRuns = 2 * 148;  // CTAs of one launch over all KV heads: two per SM

struct DecodeSeg {
  const void* k;
  const void* v;
  int64_t hs;
  int32_t ts;
  int32_t len;
};

struct DecodeParams {
  DecodeSeg seg[kMaxSeg];
  int32_t item_begin[kMaxSeg + 1];  // first 16-key group of each segment within one KV head's list
  uint8_t qsel[kMaxSeg];            // query variant per segment
  int32_t n_seg, n_heads, n_kv_heads, n_items, n_runs;
  int32_t logit_seg;  // segment whose scaled logits are exported, or -1
  const void* q[2];   // (H, D) each, heads q_hs elements apart
  int64_t q_hs;
  float* part_o;      // (n_runs, H, D)
  float* part_lse;    // (n_runs, H)
  float* logits;      // (H, seg_len[logit_seg])
  float scale_log2;
  DecodeIndirect ind; // n_units == 0: every segment carries its own pointers
};

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

template <typename T>
__global__ void __launch_bounds__(kDecThreads, 2) attn_decode_kernel(const __grid_constant__ DecodeParams P) {
  using namespace mma;
  constexpr int HD = 128;
  __shared__ __align__(16) float sm_o[kDecWarps][kMaxGroup][HD];
  __shared__ float sm_m[kDecWarps][kMaxGroup], sm_l[kDecWarps][kMaxGroup];
  const bool early = P.ind.early_rest != 0 && P.ind.n_units > 0;
  if (early) chain_trigger(); else chain_enter();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int run = blockIdx.x, hkv = blockIdx.y;
  const int group = P.n_heads / P.n_kv_heads;
  const bool qrow = g < group;          // this thread's S row is a real query head
  const int hq = hkv * group + (qrow ? g : 0);

  uint4 qf[4];  // Q of head hq: elements j*32 + t*8 .. +7 for j = 0..3 (zero for rows past the group)
  int cur_q = -1;
  float ot[8][4];  // O^T tile i: [0],[1] = dim g*8+i of heads 2t, 2t+1; [2],[3] = dim 64+g*8+i
#pragma unroll
  for (int i = 0; i < 8; ++i) ot[i][0] = ot[i][1] = ot[i][2] = ot[i][3] = 0.f;
  float m = -INFINITY, l = 0.f;  // running maximum of head g; this thread's share of its row sum

  // A run is a contiguous share of the groups outside the device-resolved units plus a contiguous share of the
  // units' groups; the CTA's warps divide into two teams in proportion, one per kind, so that both kinds proceed side
  // by side.  The first kind needs no retrieval: with early_rest its team has not waited for the kernel's
  // predecessor, only the units' team does.
  const char *kbase = nullptr, *vbase = nullptr;
  char* deposit = nullptr;  // != nullptr: the segment is a unit read in place; its K block's copy in the landing slot
  bool seg_ok = true;
  const int u_beg = P.ind.n_units > 0 ? P.item_begin[P.ind.first_seg] : 0;
  const int u_end = P.ind.n_units > 0 ? P.item_begin[P.ind.first_seg + P.ind.n_units] : 0;
  const int n_unit = u_end - u_beg, n_rest = P.n_items - n_unit;
  int w_rest = n_unit == 0 ? kDecWarps : (kDecWarps * n_rest + P.n_items / 2) / P.n_items;
  if (n_unit > 0 && n_rest > 0) w_rest = w_rest < 1 ? 1 : (w_rest > kDecWarps - 1 ? kDecWarps - 1 : w_rest);
  const bool unit_team = warp >= w_rest;
  if (unit_team && early) chain_wait();
  const int n_kind = unit_team ? n_unit : n_rest, team = unit_team ? kDecWarps - w_rest : w_rest;
  const int lo = (int)((int64_t)run * n_kind / P.n_runs), hi = (int)((int64_t)(run + 1) * n_kind / P.n_runs);
  int sg = 0, sg_resolved = -1;
#pragma unroll 1
  for (int j = lo + (unit_team ? warp - w_rest : warp); j < hi; j += team) {
    const int it = unit_team ? u_beg + j : (j < u_beg ? j : j + n_unit);
    while (it >= P.item_begin[sg + 1]) ++sg;
    const DecodeSeg& S = P.seg[sg];
    if (sg != sg_resolved) {  // pointers of the segment; a memory unit named on the device is looked up here
      sg_resolved = sg;
      seg_ok = true;
      deposit = nullptr;
      const void* sk = S.k;
      const void* sv = S.v;
      const int u = sg - P.ind.first_seg;
      if (P.ind.n_units > 0 && u >= 0 && u < P.ind.n_units) {
        const int id = __ldg(P.ind.ids + u) - P.ind.id_lo;
        const bool mine = id >= 0 && id < P.ind.n_owned;
        if (P.ind.ptrs) {  // table of addresses: wherever the unit lives (cache slot, device copy, pinned host store)
          const unsigned long long a = mine ? __ldg(P.ind.ptrs + id) : 0ull;
          seg_ok = a != 0ull;
          sk = reinterpret_cast<const void*>(a & ~1ull);
          // bit 0: the address is the unit's place in the store, not a cache slot
          if ((a & 1ull) && P.ind.landing) {
            const unsigned long long la = __ldg(P.ind.landing + u);
            if (la) deposit = reinterpret_cast<char*>(la) + (int64_t)hkv * S.hs * 2;
          }
          sv = reinterpret_cast<const char*>(sk) + P.ind.unit_bytes / 2;
        } else {
          const int slot = mine ? __ldg(P.ind.table + id) : -1;
          seg_ok = slot >= 0;
          sk = P.ind.cache + (int64_t)(slot < 0 ? 0 : slot) * P.ind.unit_bytes;
          sv = reinterpret_cast<const char*>(sk) + P.ind.unit_bytes / 2;
        }
        // not cached: the unit contributes nothing here and the host, which learns the same from its own tables,
        // attends to it after the refill.  A unit that another rank owns is that rank's business.
        if (!seg_ok && mine && P.ind.miss && lane == 0) *P.ind.miss = 1;
      }
      kbase = reinterpret_cast<const char*>(sk) + (int64_t)hkv * S.hs * 2;
      vbase = reinterpret_cast<const char*>(sv) + (int64_t)hkv * S.hs * 2;
      if ((int)P.qsel[sg] != cur_q) {
        cur_q = P.qsel[sg];
        const char* qp = reinterpret_cast<const char*>(P.q[cur_q]) + (int64_t)hq * P.q_hs * 2;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          qf[j] = qrow ? __ldg(reinterpret_cast<const uint4*>(qp + j * 64 + t * 16)) : make_uint4(0, 0, 0, 0);
      }
    }
    if (!seg_ok) continue;
    const int j0 = (it - P.item_begin[sg]) * 16;
    const int nk = S.len - j0 < 16 ? S.len - j0 : 16;
    const int64_t row_bytes = (int64_t)S.ts * 2;
    // ---- every load of the group.  K: keys j0 + nt*8 + g (this thread's B-fragment column), 64 bytes of the row in
    //      four pieces j*64 + t*16; V: keys j0 + {2t, 2t+1, 2t+8, 2t+9}, 32 bytes in two pieces p*128 + g*16.
    //      Rows past the end of the segment are read from its last row and masked below.
    uint4 kr[2][4], vr[4][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int r = nt * 8 + g;
      const char* rp = kbase + (int64_t)(j0 + (r < nk ? r : nk - 1)) * row_bytes + t * 16;
#pragma unroll
      for (int j = 0; j < 4; ++j) kr[nt][j] = ld_stream16(rp + j * 64);
    }
#pragma unroll
    for (int ki = 0; ki < 4; ++ki) {
      const int r = 2 * t + (ki & 1) + (ki >> 1) * 8;
      const char* rp = vbase + (int64_t)(j0 + (r < nk ? r : nk - 1)) * row_bytes + g * 16;
      vr[ki][0] = ld_stream16(rp);
      vr[ki][1] = ld_stream16(rp + 128);
    }
    if (deposit) {  // what was just read, to the same place of the landing slot (K block, then V block)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int r = nt * 8 + g;
        if (r < nk) {
          char* wp = deposit + (int64_t)(j0 + r) * row_bytes + t * 16;
#pragma unroll
          for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(wp + j * 64) = kr[nt][j];
        }
      }
#pragma unroll
      for (int ki = 0; ki < 4; ++ki) {
        const int r = 2 * t + (ki & 1) + (ki >> 1) * 8;
        if (r < nk) {
          char* wp = deposit + P.ind.unit_bytes / 2 + (int64_t)(j0 + r) * row_bytes + g * 16;
          *reinterpret_cast<uint4*>(wp) = vr[ki][0];
          *reinterpret_cast<uint4*>(wp + 128) = vr[ki][1];
        }
      }
    }
    // ---- S = Q K^T: rows = query heads, columns = the 16 keys (two n-tiles), 8 k-steps of 16 elements
    float sacc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t a0[4] = {qf[j].x, 0u, qf[j].y, 0u};
        mma16816<T>(sacc[nt], a0, kr[nt][j].x, kr[nt][j].y);
        const uint32_t a1[4] = {qf[j].z, 0u, qf[j].w, 0u};
        mma16816<T>(sacc[nt], a1, kr[nt][j].z, kr[nt][j].w);
      }
    }
    // ---- softmax of the group against the running maximum: this thread holds keys nt*8 + 2t + e of head g
    float sv[4];
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = nt * 8 + 2 * t + e;
        const float v = (qrow && key < nk) ? sacc[nt][e] * P.scale_log2 : -INFINITY;
        sv[nt * 2 + e] = v;
        mx = fmaxf(mx, v);
        if (sg == P.logit_seg && qrow && key < nk) P.logits[(int64_t)hq * S.len + j0 + key] = v;
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m, mx);
    const float ms = mn == -INFINITY ? 0.f : mn;
    const float al = exp2f(m - ms);  // 0 for the first group of a row
    m = mn;
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = exp2f(sv[i] - ms);
    l = l * al + (p[0] + p[1]) + (p[2] + p[3]);
    // the O^T columns of this thread are heads 2t and 2t+1: their factors come from the lanes that own those rows
    const float a0 = __shfl_sync(0xffffffffu, al, (2 * t) * 4), a1 = __shfl_sync(0xffffffffu, al, (2 * t + 1) * 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ot[i][0] *= a0;
      ot[i][1] *= a1;
      ot[i][2] *= a0;
      ot[i][3] *= a1;
    }
    // ---- O^T += V^T P^T: B = P^T (this thread: head g, keys 2t, 2t+1 | 2t+8, 2t+9), A = V^T built by byte permutes
    const uint32_t b0 = pack2<T>(p[0], p[1]), b1 = pack2<T>(p[2], p[3]);
    const uint32_t* v00 = reinterpret_cast<const uint32_t*>(&vr[0][0]);
    const uint32_t* v10 = reinterpret_cast<const uint32_t*>(&vr[1][0]);
    const uint32_t* v20 = reinterpret_cast<const uint32_t*>(&vr[2][0]);
    const uint32_t* v30 = reinterpret_cast<const uint32_t*>(&vr[3][0]);
    const uint32_t* v01 = reinterpret_cast<const uint32_t*>(&vr[0][1]);
    const uint32_t* v11 = reinterpret_cast<const uint32_t*>(&vr[1][1]);
    const uint32_t* v21 = reinterpret_cast<const uint32_t*>(&vr[2][1]);
    const uint32_t* v31 = reinterpret_cast<const uint32_t*>(&vr[3][1]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = i >> 1;
      const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;  // the high or the low 16 bits of both words
      uint32_t a[4];
      a[0] = __byte_perm(v00[r], v10[r], sel);  // dim g*8+i of keys 2t, 2t+1
      a[1] = __byte_perm(v01[r], v11[r], sel);  // dim 64+g*8+i
      a[2] = __byte_perm(v20[r], v30[r], sel);  // keys 2t+8, 2t+9
      a[3] = __byte_perm(v21[r], v31[r], sel);
      mma16816<T>(ot[i], a, b0, b1);
    }
  }
  // ---- the warps' results meet in shared memory
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (qrow && t == 0) {
    sm_m[warp][g] = m;
    sm_l[warp][g] = l;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int head = 2 * t + e;
      if (head < group) {
        sm_o[warp][head][g * 8 + i] = ot[i][e];
        sm_o[warp][head][64 + g * 8 + i] = ot[i][2 + e];
      }
    }
  }
  __syncthreads();
  const int64_t prow = (int64_t)run * P.n_heads + hkv * group;  // first head row of this CTA's partial
  for (int idx = tid; idx < group * HD; idx += kDecThreads) {
    const int h = idx / HD, d = idx % HD;
    float mxw = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mxw = fmaxf(mxw, sm_m[w][h]);
    float den = 0.f, num = 0.f;
    if (mxw != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        const float wt = exp2f(sm_m[w][h] - mxw);
        den = fmaf(wt, sm_l[w][h], den);
        num = fmaf(wt, sm_o[w][h][d], num);
      }
    }
    P.part_o[(prow + h) * HD + d] = den > 0.f ? num / den : 0.f;
    if (d == 0) P.part_lse[prow + h] = den > 0.f ? mxw + log2f(den) : -INFINITY;
  }
}

// out[h, :] = sum_p w_p o_p / sum_p w_p with w_p = exp2(lse_p - max lse); lse = max + log2(sum w).
// One CTA per head.  Every global load of the common case is issued before anything waits: eight groups of
// head_dim threads share the partials (group g takes partials g, g + 8, ...: 40 of them in a single round of
// loads), and every thread also owns four score columns of the window; meanwhile warp 0 turns the partials'
// log-sum-exps into weights.  Two barriers in all.
// With `logits` the CTA adds this token's local attention row into the accumulated scores:
// score[h, j] += exp2(logit[h, j] - lse[h]) — the column sums of a one-token exec block.
constexpr int kMergeGroups = 8;
constexpr int kMergeUnroll = 5;  // partials a thread has in flight: 8 groups x 5 cover 40 partials in one round
constexpr int kMergeCols = 4;    // score columns a thread keeps in flight: 4 x 1024 cover a 4096-token window
template <typename T>
__global__ void __launch_bounds__(1024)
lse_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, int n_part, int n_heads,
                 int head_dim, T* __restrict__ out, int64_t o_hs, float* __restrict__ lse,
                 const float* __restrict__ logits, int64_t logit_len, float* __restrict__ score, int64_t score_hs,
                 const int32_t* __restrict__ skip, int64_t o_ps, int64_t lse_ps, const MergeWait wait) {
  extern __shared__ float s_w[];  // n_part weights
  __shared__ float s_num[kMergeGroups][128];
  __shared__ float s_mx, s_den;
  chain_enter();
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (wait.flags) {  // the partials come from peers: every CTA waits for every sender's flag, with a bound
    bool ok = true;
    if (tid < wait.world) {
      uint32_t i = 0;
      while (wait.flags[tid] != wait.seq) {
        if (++i > wait.limit) {
          ok = false;
          break;
        }
        __nanosleep(200);
      }
      if (!ok) atomicExch(wait.err, 1 + tid);
      __threadfence_system();
    }
    if (__syncthreads_or(!ok)) return;  // a sender did not arrive: nothing is written
  }
  if (skip && *skip) return;  // the partials were declared invalid by whoever produced them
  const int grp = tid / head_dim, d = tid % head_dim, ngrp = blockDim.x / head_dim;
  const float* po = part_o + (int64_t)h * head_dim + d;
  bool ll_ok = true;
  auto ll_get = [&](int64_t idx, int sender) -> float {  // a word that carries its own arrival flag
    const volatile unsigned long long* p = wait.ll + idx;
    unsigned long long v = *p;
    for (uint32_t it = 0; (uint32_t)(v >> 32) != wait.seq; v = *p) {
      if (++it > wait.limit) {
        ll_ok = false;
        atomicExch(wait.err, 1 + sender);
        break;
      }
      __nanosleep(100);
    }
    return __uint_as_float((uint32_t)v);
  };
  float pv[kMergeUnroll];
#pragma unroll
  for (int u = 0; u < kMergeUnroll; ++u) {
    const int p = grp + u * ngrp;
    pv[u] = p >= n_part ? 0.f : wait.ll ? ll_get((int64_t)p * o_ps + (int64_t)h * head_dim + d, p) : __ldcs(po + (int64_t)p * o_ps);
  }
  float lg[kMergeCols], sc[kMergeCols];
#pragma unroll
  for (int i = 0; i < kMergeCols; ++i) {
    const int64_t j = tid + (int64_t)i * blockDim.x;
    const bool ok = logits != nullptr && j < logit_len;
    lg[i] = ok ? __ldcs(logits + h * logit_len + j) : 0.f;
    sc[i] = ok ? score[h * score_hs + j] : 0.f;
  }
  if (warp == 0) {
    float mx = -INFINITY;
    for (int p = lane; p < n_part; p += 32) {
      const float v = wait.ll ? ll_get((int64_t)p * lse_ps + (int64_t)n_heads * head_dim + h, p) : part_lse[(int64_t)p * lse_ps + h];
      s_w[p] = v;
      mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    float den = 0.f;
    for (int p = lane; p < n_part; p += 32) {
      const float w = mx == -INFINITY ? 0.f : exp2f(s_w[p] - mx);
      s_w[p] = w;
      den += w;
    }
    den = warp_sum(den);
    if (lane == 0) {
      s_mx = mx;
      s_den = den;
    }
  }
  if (__syncthreads_or(!ll_ok)) return;  // a sender's words did not arrive: nothing is written
  const float den = s_den;
  const float l = den > 0.f ? s_mx + log2f(den) : -INFINITY;
  float num = 0.f;
#pragma unroll
  for (int u = 0; u < kMergeUnroll; ++u) {
    const int p = grp + u * ngrp;
    if (p < n_part) num = fmaf(s_w[p], pv[u], num);
  }
  for (int p = grp + kMergeUnroll * ngrp; p < n_part; p += ngrp) num = fmaf(s_w[p], __ldcs(po + (int64_t)p * o_ps), num);
  s_num[grp][d] = num;
  if (logits) {  // the score columns need no one else's result
#pragma unroll
    for (int i = 0; i < kMergeCols; ++i) {
      const int64_t j = tid + (int64_t)i * blockDim.x;
      if (j < logit_len) score[h * score_hs + j] = sc[i] + exp2f(lg[i] - l);
    }
    for (int64_t j = tid + (int64_t)kMergeCols * blockDim.x; j < logit_len; j += blockDim.x)
      score[h * score_hs + j] += exp2f(logits[h * logit_len + j] - l);
  }
  if (tid == 0 && lse) lse[h] = l;
  __syncthreads();
  if (tid < head_dim) {
    float tot = 0.f;
    for (int g2 = 0; g2 < ngrp; ++g2) tot += s_num[g2][tid];
    out[(int64_t)h * o_hs + tid] = Act<T>::from_f(den > 0.f ? tot / den : 0.f);
  }
}

int attn_decode_launch(const void* q0, const void* q1, int64_t q_hs, int n_heads, int n_kv_heads, int head_dim, int n_seg,
                       const KvSeg* segs, const int32_t* seg_q, float* part_o, float* part_lse, int max_parts,
                       int* n_parts_out, int logit_seg, float* logits, int dtype, cudaStream_t s,
                       const DecodeIndirect* ind) {
  if (head_dim != 128) return fail(INFLLM_E_UNSUPPORTED, "decode attention: head_dim %d (128 is built)", head_dim);
  if (n_heads <= 0 || n_kv_heads <= 0)
    return fail(INFLLM_E_BADARG, "decode attention: %d query heads / %d kv heads", n_heads, n_kv_heads);
  if (n_heads % n_kv_heads || n_heads / n_kv_heads > kMaxGroup)
    return fail(INFLLM_E_UNSUPPORTED, "decode attention: %d query heads per kv head (at most %d)",
                n_heads / n_kv_heads, kMaxGroup);
  if (n_seg <= 0 || n_seg > kMaxSeg) return fail(INFLLM_E_BADARG, "decode attention: %d segments (1..%d)", n_seg, kMaxSeg);
  if (q_hs % 8 || ((uintptr_t)q0 | (uintptr_t)(q1 ? q1 : q0)) % 16)
    return fail(INFLLM_E_BADARG, "decode attention: query rows are not 16-byte aligned");
  DecodeParams P{};
  if (ind && ind->n_units > 0) {
    if (!ind->ids || (!ind->table && !ind->ptrs) || (ind->table && !ind->cache) || ind->first_seg < 0 ||
        ind->first_seg + ind->n_units > n_seg)
      return fail(INFLLM_E_BADARG, "decode attention: bad device-resolved unit list");
    for (int i = 0; i < ind->n_units; ++i)
      if (segs[ind->first_seg + i].len <= 0) return fail(INFLLM_E_BADARG, "decode attention: empty unit segment");
    P.ind = *ind;
  }
  int items = 0, ns = 0;
  int logit_seg_packed = -1;
  for (int i = 0; i < n_seg; ++i) {
    if (segs[i].len <= 0) continue;  // empty segments contribute nothing
    if (ind && ind->n_units > 0 && i == ind->first_seg) P.ind.first_seg = ns;
    if (((uintptr_t)segs[i].k | (uintptr_t)segs[i].v) % 16 || segs[i].hs % 8 || segs[i].ts % 8)
      return fail(INFLLM_E_BADARG, "decode attention: segment %d rows are not 16-byte aligned", i);
    P.seg[ns] = {segs[i].k, segs[i].v, segs[i].hs, segs[i].ts, segs[i].len};
    P.qsel[ns] = (uint8_t)(seg_q[i] ? 1 : 0);
    P.item_begin[ns] = items;
    if (i == logit_seg) logit_seg_packed = ns;
    items += (int)ceil_div(segs[i].len, 16);
    ++ns;
  }
  P.item_begin[ns] = items;
  // one run of 16-key groups per CTA, two CTAs per SM over all KV heads
  int runs = std::max(1, kDecMaxRuns / n_kv_heads);
  runs = std::min(runs, std::max(items, 1));
  runs = std::min(runs, max_parts);
  if (n_parts_out) *n_parts_out = items > 0 ? runs : 0;
  if (items == 0) return INFLLM_OK;
  if (runs <= 0) return fail(INFLLM_E_CAPACITY, "decode attention: no room for partials (max_parts %d)", max_parts);
  P.n_seg = ns; P.n_heads = n_heads; P.n_kv_heads = n_kv_heads; P.logit_seg = logit_seg_packed;
  P.n_items = items; P.n_runs = runs;
  P.q[0] = q0; P.q[1] = q1 ? q1 : q0; P.q_hs = q_hs;
  P.part_o = part_o;
  P.part_lse = part_lse;
  P.logits = logits;
  P.scale_log2 = kLog2e / sqrtf((float)head_dim);
  dim3 grid(runs, n_kv_heads);
  INFLLM_DISPATCH_DTYPE(dtype, T, { launch_chained(attn_decode_kernel<T>, grid, dim3(kDecThreads), 0, s, P); });
  INFLLM_LAUNCH_OK("attn_decode_kernel");
  return INFLLM_OK;
}

int lse_merge_launch(const float* part_o, const float* part_lse, int n_part, int n_heads, int head_dim, void* out,
                     int64_t o_hs, float* lse, int dtype, cudaStream_t s, const float* logits, int64_t logit_len,
                     float* score, int64_t score_hs, const int32_t* skip, int64_t o_ps, int64_t lse_ps,
                     const MergeWait* wait) {
  const MergeWait w = wait ? *wait : MergeWait{};
  if (o_ps <= 0) o_ps = (int64_t)n_heads * head_dim;
  if (lse_ps <= 0) lse_ps = n_heads;
  if (n_part <= 0) return fail(INFLLM_E_BADARG, "lse_merge: no partials");
  if (n_part > 8192) return fail(INFLLM_E_CAPACITY, "lse_merge: %d partials (at most 8192)", n_part);
  if (w.ll && (n_part > kMergeUnroll * kMergeGroups || !w.err))
    return fail(INFLLM_E_BADARG, "lse_merge: %d flag-in-data partials (at most %d)", n_part, kMergeUnroll * kMergeGroups);
  if (head_dim <= 0 || head_dim > 128 || head_dim % 32)
    return fail(INFLLM_E_UNSUPPORTED, "lse_merge: head_dim %d (a multiple of 32, at most 128)", head_dim);
  if (dtype == INFLLM_F32) {
    launch_chained(lse_merge_kernel<float>, dim3(n_heads), dim3(kMergeGroups * head_dim), n_part * sizeof(float), s,
        part_o, part_lse, n_part, n_heads, head_dim, (float*)out, o_hs, lse, logits, logit_len, score, score_hs, skip,
        o_ps, lse_ps, w);
  } else {
    INFLLM_DISPATCH_DTYPE(dtype, T, {
      launch_chained(lse_merge_kernel<T>, dim3(n_heads), dim3(kMergeGroups * head_dim), n_part * sizeof(float), s,
          part_o, part_lse, n_part, n_heads, head_dim, (T*)out, o_hs, lse, logits, logit_len, score, score_hs, skip,
          o_ps, lse_ps, w);
    });
  }
  INFLLM_LAUNCH_OK("lse_merge_kernel");
  return INFLLM_OK;
}

}  // namespace infllm

extern "C" int64_t infllm_attn_decode_max_parts(int n_seg, int64_t total_keys) {
  const int64_t groups = total_keys / 16 + n_seg + 1;
  return groups < infllm::kDecMaxRuns ? groups : infllm::kDecMaxRuns;
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
                            max_parts, n_parts, logit_seg, d_logits, dtype, (cudaStream_t)stream, nullptr);
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
                                part_lse, kStaticMaxParts, &n_parts, -1, nullptr, dtype, s, nullptr));
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
  ind.ids = d_unit_ids; ind.cache = (const char*)d_cache; ind.unit_bytes = unit_bytes;
  if (d_cache) ind.table = d_slot_table;
  else ind.ptrs = reinterpret_cast<const unsigned long long*>(d_slot_table);  // a table of unit addresses
  ind.n_units = n_units; ind.first_seg = first_unit_seg; ind.miss = d_miss; ind.id_lo = id_lo; ind.n_owned = n_owned;
  return attn_decode_launch(d_q0, d_q1, head_dim, n_heads, n_kv_heads, head_dim, n_seg, segs, h_seg_q, d_part_o,
                            d_part_lse, max_parts, n_parts, logit_seg, d_logits, dtype, (cudaStream_t)stream,
                            n_units > 0 ? &ind : nullptr);
}
