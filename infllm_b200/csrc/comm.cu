// Communicator for KV-head-group sharding: every rank runs the context memory on its own slice of the heads, and
// the only exchange is the sum over ranks of the retrieval scores (the reference scores a unit with the mean query
// of ALL heads, context_manager.py:373-378), after which every rank takes the same top-k and keeps the same LRU
// order.  The sums are NCCL all-reduces on the caller's stream.  NCCL is looked up at run time in the library the
// process has already loaded (PyTorch's), so that this library neither links against nor requires it elsewhere.
#include <dlfcn.h>

#include <new>
#include <nccl.h>

#include "common.cuh"

namespace infllm {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

static NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.ok ? &api : nullptr;
  tried = true;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return nullptr;
  api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
  api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
  api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
  api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
  api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
  api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy && api.GetErrorString;
  return api.ok ? &api : nullptr;
}

}  // namespace infllm

// two communicators: one for the main stream, one for the look-ahead stream, so that collectives issued on the two
// streams never share a communicator
struct infllm_comm {
  ncclComm_t comm[2] = {nullptr, nullptr};
  int rank = 0, world = 1;
};

using namespace infllm;

namespace infllm {
int comm_allreduce_sum(infllm_comm* c, int which, float* d_buf, size_t n, cudaStream_t s) {
  NcclApi* api = nccl_api();
  if (!api || !c || !c->comm[which & 1]) return fail(INFLLM_E_BADARG, "all-reduce without a communicator");
  ncclResult_t r = api->AllReduce(d_buf, d_buf, n, ncclFloat32, ncclSum, c->comm[which & 1], s);
  if (r != ncclSuccess) return fail(INFLLM_E_CUDA, "ncclAllReduce failed: %s", api->GetErrorString(r));
  return INFLLM_OK;
}
int comm_world(const infllm_comm* c) { return c ? c->world : 1; }
}  // namespace infllm

extern "C" int infllm_comm_id_bytes(void) { return 2 * (int)sizeof(ncclUniqueId); }

extern "C" int infllm_comm_unique_id(void* h_out) {
  NcclApi* api = nccl_api();
  if (!api) return fail(INFLLM_E_UNSUPPORTED, "NCCL (libnccl.so.2) is not available in this process");
  if (!h_out) return fail(INFLLM_E_BADARG, "comm_unique_id: null pointer");
  for (int i = 0; i < 2; ++i) {
    ncclResult_t r = api->GetUniqueId(reinterpret_cast<ncclUniqueId*>(h_out) + i);
    if (r != ncclSuccess) return fail(INFLLM_E_CUDA, "ncclGetUniqueId failed: %s", api->GetErrorString(r));
  }
  return INFLLM_OK;
}

extern "C" int infllm_comm_create(const void* h_id, int rank, int world, infllm_comm** out) {
  NcclApi* api = nccl_api();
  if (!api) return fail(INFLLM_E_UNSUPPORTED, "NCCL (libnccl.so.2) is not available in this process");
  if (!h_id || !out || world < 1 || rank < 0 || rank >= world) return fail(INFLLM_E_BADARG, "comm_create: bad argument");
  infllm_comm* c = new (std::nothrow) infllm_comm();
  if (!c) return fail(INFLLM_E_NOMEM, "comm_create: out of host memory");
  c->rank = rank;
  c->world = world;
  for (int i = 0; i < 2; ++i) {
    ncclResult_t r = api->CommInitRank(&c->comm[i], world, reinterpret_cast<const ncclUniqueId*>(h_id)[i], rank);
    if (r != ncclSuccess) {
      delete c;
      return fail(INFLLM_E_CUDA, "ncclCommInitRank failed: %s", api->GetErrorString(r));
    }
  }
  *out = c;
  return INFLLM_OK;
}

extern "C" int infllm_comm_destroy(infllm_comm* c) {
  if (!c) return INFLLM_OK;
  NcclApi* api = nccl_api();
  for (int i = 0; i < 2; ++i)
    if (api && c->comm[i]) api->CommDestroy(c->comm[i]);
  delete c;
  return INFLLM_OK;
}

// ------------------------------------------------------------------------------------------------------------
// Exchange through peer memory for the unit-range sharded decode: every rank owns one mailbox buffer that all
// ranks can write (CUDA IPC mappings); a message is put straight into slot [sender] of every peer's mailbox by a
// kernel, followed by a flag word holding the sequence number of the exchange; the receiver's next kernels start
// behind a kernel that waits — with a bound — until every sender's flag shows that number.  No host round trip,
// no collective library call on the token's path.
//
// The waits are bounded: when a flag does not arrive within the limit (a peer died or fell far behind) the wait
// kernel records an error word and returns, the kernels behind it see the word and write nothing, and the host
// reads it with the token's result.

struct infllm_mailbox {
  void* local = nullptr;        // this rank's buffer
  void* peer[16] = {nullptr};   // the same buffer of every rank as mapped here (peer[rank] == local)
  bool aliased[16] = {false};   // peer[r] is a pointer of this process (infllm_mailbox_alias): not ours to unmap
  size_t bytes = 0;
  int rank = 0, world = 1;
};

namespace infllm {

constexpr int kMaxPeers = 16;
struct PeerList {
  void* dst[kMaxPeers];
  uint32_t* flag[kMaxPeers];
};

// one CTA per destination: copy n16 16-byte words, make them visible system-wide, then raise the flag
__global__ void __launch_bounds__(256)
peer_put_kernel(const uint4* __restrict__ src, int n16, const __grid_constant__ PeerList peers, uint32_t seq) {
  chain_enter();
  uint4* dst = reinterpret_cast<uint4*>(peers.dst[blockIdx.x]);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    volatile uint32_t* f = peers.flag[blockIdx.x];
    *f = seq;
  }
}

// lane q waits for flags[q] == seq, at most `limit` polls of ~200 ns; *err = 1 + q when one ran out.
// With miss_words != nullptr (one word per sender, inside the messages just received) their OR goes to *any_miss.
__global__ void peer_wait_kernel(const volatile uint32_t* flags, uint32_t seq, int world, uint32_t limit, int* err,
                                 const volatile int32_t* miss_words, int64_t miss_stride, int32_t* any_miss,
                                 int32_t* clear_word) {
  const int q = threadIdx.x;
  if (clear_word && q == 0) *clear_word = 0;
  bool ok = true;
  if (q < world) {
    uint32_t i = 0;
    while (flags[q] != seq) {
      if (++i > limit) {
        ok = false;
        break;
      }
      __nanosleep(200);
    }
    if (!ok) atomicExch(err, 1 + q);
  }
  __threadfence_system();
  const unsigned all_ok = __all_sync(0xffffffffu, ok);
  if (any_miss) {
    int m = (q < world && miss_words && all_ok) ? miss_words[q * miss_stride] : 0;
    m = __any_sync(0xffffffffu, m != 0);
    if (q == 0) *any_miss = (m || !all_ok) ? 1 : 0;
  }
}

// The candidate exchange of a sharded token as ONE kernel of one CTA: put this rank's message into every peer's
// mailbox and raise the flags, wait (bounded) for every sender's flag here, rank the gathered candidates.  Nobody
// waits before it has put, so the ranks cannot block one another.
__device__ void rank_candidates(const int32_t* __restrict__ cand, int64_t sender_stride, int world, int k,
                                int32_t* __restrict__ out_ids, float* s_score, int32_t* s_id);

__global__ void __launch_bounds__(256)
exchange_rank_kernel(const uint4* __restrict__ src, int n16, const __grid_constant__ PeerList peers, int world, uint32_t seq,
                     const volatile uint32_t* flags, uint32_t limit, int* err, int32_t* clear_word,
                     const int32_t* __restrict__ cand, int64_t sender_stride, int k, int32_t* __restrict__ out_ids) {
  __shared__ float s_score[1024];
  __shared__ int32_t s_id[1024];
  chain_enter();
  const int tid = threadIdx.x;
  for (int i = tid; i < world * n16; i += blockDim.x) reinterpret_cast<uint4*>(peers.dst[i / n16])[i % n16] = src[i % n16];
  __threadfence_system();
  __syncthreads();
  if (tid < world) {
    volatile uint32_t* f = peers.flag[tid];
    *f = seq;
  }
  if (clear_word && tid == 0) *clear_word = 0;
  bool ok = true;
  if (tid < world) {
    uint32_t i = 0;
    while (flags[tid] != seq) {
      if (++i > limit) {
        ok = false;
        break;
      }
      __nanosleep(200);
    }
    if (!ok) atomicExch(err, 1 + tid);
    __threadfence_system();
  }
  if (__syncthreads_or(!ok)) {  // the exchange failed: no retrieval
    for (int i = tid; i < k; i += blockDim.x) out_ids[i] = -1;
    return;
  }
  rank_candidates(cand, sender_stride, world, k, out_ids, s_score, s_id);
}

// The same exchange with the arrival flag inside the data: every 32-bit word of the message travels as an 8-byte
// store {word, seq} into the peer's slot and the receiver polls each word until it carries this token's sequence
// number.  An aligned 8-byte store arrives whole, so there is no system-wide fence and no separate flag store behind
// the data: one link latency instead of three.  Slots of 2k 8-byte words per sender; sequence numbers start at 1
// and the region starts zeroed.
struct PeerWords {
  unsigned long long* dst[kMaxPeers];
};
__global__ void __launch_bounds__(256)
exchange_rank_ll_kernel(const int32_t* __restrict__ src, const __grid_constant__ PeerWords peers, int world, uint32_t seq,
                        const volatile unsigned long long* local, int64_t sender_stride, uint32_t limit, int* err,
                        int32_t* clear_word, int k, int32_t* __restrict__ out_ids) {
  __shared__ float s_score[1024];
  __shared__ int32_t s_id[1024];
  chain_enter();
  const int tid = threadIdx.x, m = 2 * k, n = world * k;
  for (int i = tid; i < world * m; i += blockDim.x) {
    const unsigned long long w = ((unsigned long long)seq << 32) | (uint32_t)src[i % m];
    *reinterpret_cast<volatile unsigned long long*>(peers.dst[i / m] + i % m) = w;
  }
  if (clear_word && tid == 0) *clear_word = 0;
  bool ok = true;
  for (int i = tid; i < world * m && ok; i += blockDim.x) {
    const int r = i / m, w = i % m;
    const volatile unsigned long long* p = local + (int64_t)r * sender_stride + w;
    unsigned long long v = *p;
    for (uint32_t it = 0; (uint32_t)(v >> 32) != seq; v = *p) {
      if (++it > limit) {
        ok = false;
        atomicExch(err, 1 + r);
        break;
      }
      __nanosleep(100);
    }
    if (w < k) s_score[r * k + w] = __int_as_float((int32_t)(uint32_t)v);
    else s_id[r * k + w - k] = (int32_t)(uint32_t)v;
  }
  if (__syncthreads_or(!ok)) {  // the exchange failed: no retrieval
    for (int i = tid; i < k; i += blockDim.x) out_ids[i] = -1;
    return;
  }
  for (int i = tid; i < k; i += blockDim.x) out_ids[i] = -1;  // fewer than k real candidates: padding
  __syncthreads();
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = s_score[i];
    const int32_t id = s_id[i];
    if (id < 0) continue;
    int rank = 0;
    for (int j = 0; j < n; ++j) {
      const int32_t oj = s_id[j];
      rank += oj >= 0 && (s_score[j] > v || (s_score[j] == v && oj < id));
    }
    if (rank < k) out_ids[rank] = id;
  }
}

// one CTA per destination: the message's n 32-bit words as {word, seq} pairs into this rank's slot there
__global__ void __launch_bounds__(256)
peer_put_ll_kernel(const uint32_t* __restrict__ src, int n, const __grid_constant__ PeerWords peers, uint32_t seq) {
  chain_enter();
  volatile unsigned long long* dst = peers.dst[blockIdx.x];
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = ((unsigned long long)seq << 32) | src[i];
}

__device__ void rank_candidates(const int32_t* __restrict__ cand, int64_t sender_stride, int world, int k,
                                int32_t* __restrict__ out_ids, float* s_score, int32_t* s_id) {
  const int n = world * k;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int32_t* c = cand + (int64_t)(i / k) * sender_stride;
    s_score[i] = __int_as_float(__ldcv(c + i % k));  // written by peers a moment ago: not through a stale cache line
    s_id[i] = __ldcv(c + k + i % k);
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) out_ids[i] = -1;  // fewer than k real candidates: padding
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = s_score[i];
    const int32_t id = s_id[i];
    if (id < 0) continue;
    int rank = 0;
    for (int j = 0; j < n; ++j) {
      const int32_t oj = s_id[j];
      rank += oj >= 0 && (s_score[j] > v || (s_score[j] == v && oj < id));
    }
    if (rank < k) out_ids[rank] = id;
  }
}

// the k best of world * k gathered candidates [sender][score bits (k) | ids (k)]: descending score, ties to the
// lower id, ids < 0 are padding; one CTA
__global__ void __launch_bounds__(256)
topk_pairs_kernel(const int32_t* __restrict__ cand, int64_t sender_stride, int world, int k, int32_t* __restrict__ out_ids,
                  const int* __restrict__ err) {
  __shared__ float s_score[1024];
  __shared__ int32_t s_id[1024];
  const int n = world * k;
  if (err && *err) {  // the exchange failed: no retrieval
    for (int i = threadIdx.x; i < k; i += blockDim.x) out_ids[i] = -1;
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int32_t* c = cand + (int64_t)(i / k) * sender_stride;
    s_score[i] = __int_as_float(c[i % k]);
    s_id[i] = c[k + i % k];
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) out_ids[i] = -1;  // fewer than k real candidates: padding
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = s_score[i];
    const int32_t id = s_id[i];
    if (id < 0) continue;
    int rank = 0;
    for (int j = 0; j < n; ++j) {
      const int32_t oj = s_id[j];
      rank += oj >= 0 && (s_score[j] > v || (s_score[j] == v && oj < id));
    }
    if (rank < k) out_ids[rank] = id;
  }
}

}  // namespace infllm

extern "C" int infllm_mailbox_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

// allocates this rank's mailbox (zeroed) and writes its IPC handle to h_handle
extern "C" int infllm_mailbox_create(int64_t bytes, int rank, int world, void* h_handle, infllm_mailbox** out) {
  if (bytes <= 0 || !h_handle || !out || world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(INFLLM_E_BADARG, "mailbox_create: bad argument (at most %d ranks)", kMaxPeers);
  infllm_mailbox* m = new (std::nothrow) infllm_mailbox();
  if (!m) return fail(INFLLM_E_NOMEM, "mailbox_create: out of host memory");
  m->bytes = (size_t)bytes;
  m->rank = rank;
  m->world = world;
  cudaError_t e = cudaMalloc(&m->local, m->bytes);
  if (e == cudaSuccess) e = cudaMemset(m->local, 0, m->bytes);
  if (e == cudaSuccess && world > 1) e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(h_handle), m->local);
  if (e != cudaSuccess) {
    if (m->local) cudaFree(m->local);
    delete m;
    return fail(INFLLM_E_CUDA, "mailbox_create: %s", cudaGetErrorString(e));
  }
  m->peer[rank] = m->local;
  *out = m;
  return INFLLM_OK;
}

// h_handles: world handles in rank order (as gathered by the caller); maps every peer's mailbox
extern "C" int infllm_mailbox_open(infllm_mailbox* m, const void* h_handles) {
  if (!m || !h_handles) return fail(INFLLM_E_BADARG, "mailbox_open: null pointer");
  const cudaIpcMemHandle_t* hs = reinterpret_cast<const cudaIpcMemHandle_t*>(h_handles);
  for (int r = 0; r < m->world; ++r) {
    if (r == m->rank) continue;
    cudaError_t e = cudaIpcOpenMemHandle(&m->peer[r], hs[r], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(INFLLM_E_CUDA, "mailbox_open: rank %d: %s", r, cudaGetErrorString(e));
  }
  return INFLLM_OK;
}

extern "C" void* infllm_mailbox_local(infllm_mailbox* m) { return m ? m->local : nullptr; }

extern "C" int infllm_mailbox_alias(infllm_mailbox* m, int rank, void* d_buffer) {
  if (!m || !d_buffer || rank < 0 || rank >= m->world || rank == m->rank || m->peer[rank])
    return fail(INFLLM_E_BADARG, "mailbox_alias: bad argument");
  m->peer[rank] = d_buffer;
  m->aliased[rank] = true;
  return INFLLM_OK;
}
extern "C" int infllm_mailbox_destroy(infllm_mailbox* m) {
  if (!m) return INFLLM_OK;
  for (int r = 0; r < m->world; ++r)
    if (r != m->rank && m->peer[r] && !m->aliased[r]) cudaIpcCloseMemHandle(m->peer[r]);
  if (m->local) cudaFree(m->local);
  delete m;
  return INFLLM_OK;
}

// d_src (bytes, a multiple of 16) -> offset slot_off + rank * slot_bytes of every rank's mailbox, then the flag word
// at flag_off + 4 * rank of every mailbox is set to seq
extern "C" int infllm_mailbox_put(infllm_mailbox* m, const void* d_src, int64_t bytes, int64_t slot_off,
                                  int64_t slot_bytes, int64_t flag_off, uint32_t seq, void* stream) {
  if (!m || !d_src || bytes <= 0 || bytes % 16 || bytes > slot_bytes || slot_off % 16 || slot_bytes % 16 ||
      slot_off + (int64_t)m->world * slot_bytes > (int64_t)m->bytes || flag_off + 4 * m->world > (int64_t)m->bytes)
    return fail(INFLLM_E_BADARG, "mailbox_put: bad argument");
  PeerList pl{};
  for (int r = 0; r < m->world; ++r) {
    if (!m->peer[r]) return fail(INFLLM_E_BADARG, "mailbox_put: rank %d is not mapped (infllm_mailbox_open)", r);
    pl.dst[r] = (char*)m->peer[r] + slot_off + (int64_t)m->rank * slot_bytes;
    pl.flag[r] = reinterpret_cast<uint32_t*>((char*)m->peer[r] + flag_off) + m->rank;
  }
  launch_chained(peer_put_kernel, dim3(m->world), dim3(256), 0, (cudaStream_t)stream, (const uint4*)d_src, (int)(bytes / 16), pl, seq);
  INFLLM_LAUNCH_OK("peer_put_kernel");
  return INFLLM_OK;
}

// waits on `stream` until the flag words of all ranks at flag_off show seq (bounded: limit_us microseconds);
// d_err receives 1 + rank of a sender that did not arrive.  With miss_off >= 0 the word at
// slot_off + r * slot_bytes + miss_off of every received message is OR-ed into *d_any_miss.  d_clear (may be
// null): a device word set to zero by the same kernel (the miss word of the message about to be built).
extern "C" int infllm_mailbox_wait(infllm_mailbox* m, int64_t flag_off, uint32_t seq, int limit_us, int* d_err,
                                   int64_t slot_off, int64_t slot_bytes, int64_t miss_off, int32_t* d_any_miss,
                                   int32_t* d_clear, void* stream) {
  if (!m || !d_err || flag_off < 0 || flag_off + 4 * m->world > (int64_t)m->bytes)
    return fail(INFLLM_E_BADARG, "mailbox_wait: bad argument");
  const uint32_t limit = (uint32_t)((limit_us > 0 ? limit_us : 100000) * 5ll);  // polls of ~200 ns
  const volatile int32_t* mw = miss_off >= 0 ? reinterpret_cast<const volatile int32_t*>((char*)m->local + slot_off + miss_off) : nullptr;
  peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const volatile uint32_t*>((char*)m->local + flag_off), seq, m->world, limit, d_err, mw,
      slot_bytes / 4, d_any_miss, d_clear);
  INFLLM_LAUNCH_OK("peer_wait_kernel");
  return INFLLM_OK;
}

// global top-k of the candidates gathered in the local mailbox: world messages [score bits (k) | ids (k)] int32
extern "C" int infllm_topk_pairs(const int32_t* d_cand, int64_t sender_stride_words, int world, int k,
                                 int32_t* d_out_ids, const int* d_err, void* stream) {
  if (!d_cand || !d_out_ids || world < 1 || k < 1 || world * k > 1024)
    return fail(INFLLM_E_BADARG, "topk_pairs: bad argument (world * k <= 1024)");
  topk_pairs_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(d_cand, sender_stride_words, world, k, d_out_ids, d_err);
  INFLLM_LAUNCH_OK("topk_pairs_kernel");
  return INFLLM_OK;
}

// ------------------------------------------------------------------------------------------------------------
// One decode token of a unit-range shard as ONE call: every launch of the token — ingest, local scoring and top-k,
// candidate exchange, global top-k, attention over the owned retrieved units and this rank's share of the window,
// local merge, partial exchange, final merge with the score accumulation, and the copy of the status words to the
// host — goes onto `stream` without returning to the caller in between.  The caller fills the argument block once
// and updates the few fields that move with the token.
#include "attn_common.cuh"

namespace infllm {
int ingest_token_launch(const void* q, int64_t q_hs, const void* k, int64_t k_hs, const void* v, int64_t v_hs,
                        void* q_loc, void* q_glb, int64_t qs_hs, float* qbar, void* k_raw, void* k_rot, void* v_out,
                        int64_t kv_hs, float* score, int64_t score_hs, int n_heads, int n_kv_heads, int head_dim,
                        const float* cos_t, const float* sin_t, int64_t table_len, int64_t pos_loc, int64_t pos_glb,
                        int dtype, cudaStream_t s, int32_t* clear);
int block_topk_launch(const void* bk, int64_t n, int width, const float* qbar, float* scores, int k, int id_base,
                      int32_t* out_ids, float* out_scores, int dtype, cudaStream_t s, unsigned int* ticket,
                      int32_t* out_ids_copy = nullptr);
}  // namespace infllm

__global__ void stamp_kernel(unsigned long long* p) {
  chain_enter();
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *p = t;
}
#define INFLLM_STAMP(i)                                                                                   \
  if (a->d_stamps) {                                                                                      \
    launch_chained(stamp_kernel, dim3(1), dim3(1), 0, s, reinterpret_cast<unsigned long long*>(a->d_stamps) + (i)); \
    INFLLM_LAUNCH_OK("stamp_kernel");                                                                     \
  }

extern "C" int infllm_shard_token_run(const infllm_shard_token* a, infllm_mailbox* mb, void* stream) {
  if (!a || !mb) return fail(INFLLM_E_BADARG, "shard_token_run: null pointer");
  if (a->topk <= 0 || a->topk > kMaxSeg - 3 || a->n_owned < a->topk)
    return fail(INFLLM_E_BADARG, "shard_token_run: needs topk <= n_owned (topk %d, owned %d)", a->topk, a->n_owned);
  cudaStream_t s = (cudaStream_t)stream;
  const int H = a->n_heads, HKV = a->n_kv_heads, D = a->head_dim, esz = 2;
  const int64_t row = a->at * D * esz;
  char *k_raw = (char*)a->d_k_raw, *k_rot = (char*)a->d_k_rot, *vbuf = (char*)a->d_v;
  INFLLM_STAMP(0);
  // 1. the token: copies, rotations, query mean, score column
  INFLLM_TRY(ingest_token_launch(a->d_q, a->q_hs, a->d_k, a->k_hs, a->d_vin, a->v_hs, a->d_q_loc, a->d_q_glb, D, a->d_qbar,
                                 k_raw + row, k_rot + row, vbuf + row, a->cap * D, a->d_score + a->at, a->cap, H, HKV, D,
                                 a->d_cos, a->d_sin, a->cap, a->at, a->n_local - 1, a->dtype, s, nullptr));
  INFLLM_STAMP(1);
  // 2. this rank's candidates: [score bits (topk) | ids (topk)]
  INFLLM_TRY(block_topk_launch(a->d_block_k, a->n_owned, H * D, a->d_qbar, a->d_scores, a->topk, a->id_lo,
                               a->d_cand + a->topk, reinterpret_cast<float*>(a->d_cand), a->dtype, s, a->d_ticket));
  INFLLM_STAMP(2);
  // 3. exchange 1, global top-k
  int* err = a->d_status + a->topk;
  int32_t* any_miss = a->d_status + a->topk + 1;
  int32_t* miss_word = reinterpret_cast<int32_t*>(a->d_pack + (int64_t)H * (D + 1));
  const uint32_t limit = (uint32_t)((a->wait_us > 0 ? a->wait_us : 100000) * 5ll);  // polls of ~200 ns
  {
    if (a->cand_bytes % 16 || a->cand_bytes > a->cand_slot || mb->world * a->topk > 1024)
      return fail(INFLLM_E_BADARG, "shard_token_run: candidate message of %lld bytes", (long long)a->cand_bytes);
    PeerList pl{};
    for (int r = 0; r < mb->world; ++r) {
      if (!mb->peer[r]) return fail(INFLLM_E_BADARG, "shard_token_run: rank %d is not mapped (infllm_mailbox_open)", r);
      pl.dst[r] = (char*)mb->peer[r] + a->cand_off + (int64_t)mb->rank * a->cand_slot;
      pl.flag[r] = reinterpret_cast<uint32_t*>((char*)mb->peer[r] + a->flag1_off) + mb->rank;
    }
    if (a->ll_cand_slot > 0) {
      if (a->ll_cand_off % 8 || a->ll_cand_slot % 8 || a->ll_cand_slot < 16ll * a->topk ||
          a->ll_cand_off + (int64_t)mb->world * a->ll_cand_slot > (int64_t)mb->bytes)
        return fail(INFLLM_E_BADARG, "shard_token_run: flag-in-data candidate region at %lld, slots of %lld bytes",
                    (long long)a->ll_cand_off, (long long)a->ll_cand_slot);
      PeerWords pw{};
      for (int r = 0; r < mb->world; ++r)
        pw.dst[r] = reinterpret_cast<unsigned long long*>((char*)mb->peer[r] + a->ll_cand_off + (int64_t)mb->rank * a->ll_cand_slot);
      launch_chained(exchange_rank_ll_kernel, dim3(1), dim3(256), 0, s, reinterpret_cast<const int32_t*>(a->d_cand), pw,
                     mb->world, a->seq,
                     reinterpret_cast<const volatile unsigned long long*>((char*)mb->local + a->ll_cand_off),
                     a->ll_cand_slot / 8, limit, err, miss_word, a->topk, a->d_status);
      INFLLM_LAUNCH_OK("exchange_rank_ll_kernel");
    } else {
    launch_chained(exchange_rank_kernel, dim3(1), dim3(256), 0, s,
        reinterpret_cast<const uint4*>(a->d_cand), (int)(a->cand_bytes / 16), pl, mb->world, a->seq,
        reinterpret_cast<const volatile uint32_t*>((char*)mb->local + a->flag1_off), limit, err, miss_word,
        reinterpret_cast<const int32_t*>((char*)mb->local + a->cand_off), a->cand_slot / 4, a->topk, a->d_status);
    INFLLM_LAUNCH_OK("exchange_rank_kernel");
    }
  }
  INFLLM_STAMP(3);
  // 4. attention: [retrieved units, resolved on the device | window share | sink | overflow]
  KvSeg segs[kMaxSeg];
  int32_t qsel[kMaxSeg];
  int n = 0;
  for (; n < a->topk; ++n) {
    segs[n] = {nullptr, nullptr, (int64_t)a->block_size * D, D, a->block_size};
    qsel[n] = 1;
  }
  int logit_seg = -1;
  if (a->share_len > 0) {
    logit_seg = n;
    segs[n] = {k_rot + a->share_at * D * esz, vbuf + a->share_at * D * esz, a->cap * D, D, (int32_t)a->share_len};
    qsel[n++] = 0;
  }
  if (a->init_len > 0) {
    segs[n] = {a->d_init_k, a->d_init_v, (int64_t)a->init_len * D, D, a->init_len};
    qsel[n++] = 1;
  }
  if (a->ovf_len > 0) {
    segs[n] = {k_raw + a->ovf_at * D * esz, vbuf + a->ovf_at * D * esz, a->cap * D, D, (int32_t)a->ovf_len};
    qsel[n++] = 1;
  }
  DecodeIndirect ind;
  ind.ids = a->d_status; ind.table = a->d_slot_table; ind.cache = (const char*)a->d_cache; ind.unit_bytes = a->unit_bytes;
  ind.ptrs = reinterpret_cast<const unsigned long long*>(a->d_unit_ptrs);  // set: found wherever the unit lives
  ind.n_units = a->topk; ind.first_seg = 0; ind.miss = miss_word; ind.id_lo = a->id_lo; ind.n_owned = a->n_owned;
  ind.early_rest = a->d_stamps ? 0 : 1;  // behind the candidate exchange: the window share and the sink do not wait for it
  int parts = 0;
  INFLLM_TRY(attn_decode_launch(a->d_q_loc, a->d_q_glb, D, H, HKV, D, n, segs, qsel, a->d_part_o, a->d_part_lse,
                                a->max_parts, &parts, logit_seg, a->d_logits, a->dtype, s, &ind));
  INFLLM_STAMP(4);
  INFLLM_TRY(lse_merge_launch(a->d_part_o, a->d_part_lse, parts, H, D, a->d_pack, D, a->d_pack + (int64_t)H * D,
                              INFLLM_F32, s, nullptr, 0, nullptr, 0, nullptr));
  INFLLM_STAMP(5);
  // 5. exchange 2, merge of the ranks' partials + this rank's share of the local scores.  (Putting the merged rows
  //    into the peers' slots from the merge kernel's 32 CTAs, flags raised by the last of them, took 18.7 us against
  //    4.7 + 8.1 for the two kernels: 32 system-wide fences behind small remote stores.)
  const bool ll_part = a->ll_part_slot > 0;
  if (ll_part) {
    const int words = (int)(a->part_bytes / 4);
    if (a->ll_part_off % 8 || a->ll_part_slot < 8ll * words || a->ll_part_slot % 8 ||
        a->ll_part_off + (int64_t)mb->world * a->ll_part_slot > (int64_t)mb->bytes)
      return fail(INFLLM_E_BADARG, "shard_token_run: flag-in-data partial region at %lld, slots of %lld bytes",
                  (long long)a->ll_part_off, (long long)a->ll_part_slot);
    PeerWords pw{};
    for (int r = 0; r < mb->world; ++r)
      pw.dst[r] = reinterpret_cast<unsigned long long*>((char*)mb->peer[r] + a->ll_part_off + (int64_t)mb->rank * a->ll_part_slot);
    launch_chained(peer_put_ll_kernel, dim3(mb->world), dim3(256), 0, s, reinterpret_cast<const uint32_t*>(a->d_pack), words, pw,
                   a->seq);
    INFLLM_LAUNCH_OK("peer_put_ll_kernel");
  } else {
    INFLLM_TRY(infllm_mailbox_put(mb, a->d_pack, a->part_bytes, a->part_off, a->part_slot, a->flag2_off, a->seq, stream));
  }
  INFLLM_STAMP(6);
  // the final merge waits for the peers' partials itself (every CTA polls, with the bound: the flag words, or the
  // data words that carry their flag)
  (void)any_miss;
  MergeWait mw;
  mw.flags = ll_part ? nullptr : reinterpret_cast<const volatile uint32_t*>((char*)mb->local + a->flag2_off);
  mw.ll = ll_part ? reinterpret_cast<const volatile unsigned long long*>((char*)mb->local + a->ll_part_off) : nullptr;
  mw.seq = a->seq; mw.limit = limit; mw.world = mb->world; mw.err = err;
  const float* parts_g = reinterpret_cast<const float*>((char*)mb->local + a->part_off);
  const int64_t ps = ll_part ? a->ll_part_slot / 8 : a->part_slot / 4;
  INFLLM_TRY(lse_merge_launch(parts_g, parts_g + (int64_t)H * D, mb->world, H, D, a->d_out, D, a->d_lse, a->dtype, s,
                              a->share_len > 0 ? a->d_logits : nullptr, a->share_len, a->d_score + a->share_at, a->cap,
                              nullptr, ps, ps, &mw));
  INFLLM_STAMP(7);
  // 6. retrieval and status words for the host
  INFLLM_CUDA_OK(cudaMemcpyAsync(a->h_status, a->d_status, (a->topk + 4) * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  return INFLLM_OK;
}
