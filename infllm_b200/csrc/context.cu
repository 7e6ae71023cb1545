// Native state and exec-block loop of one unit of the context memory.
//
// Follows ContextManager of the reference (inf_llm/attention/context_manager.py:196-816) in
// behaviour, not in structure.  Tokens are addressed by their absolute index in the sequence:
//   [0, init_len)                          the init sink            (reference: init_k / init_v)
//   [n_init + b*bs, n_init + (b+1)*bs)     sealed memory unit b     (reference: global_blocks[u][b])
//   [frontier, length)                     the un-sealed remainder  (reference: global_remainder),
//                                          whose tail of n_local tokens is the local window (local_k/v)
// The remainder lives in ONE device buffer per tensor (raw keys, rotated keys, values, accumulated
// local score); there is no gather buffer: the attention kernels read retrieved units in place
// from their cache slots, the sink from its own buffer and the overflow from the remainder buffer.
// Sealed units are copied to a pinned host store on a side stream and come back into one of
// max_cached_block cache slots with cudaMemcpyAsync when retrieval asks for them.
#include <algorithm>
#include <chrono>
#include <cstring>
#include <future>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "attn_common.cuh"
#include "attn_tc.cuh"

struct infllm_comm;  // comm.cu

namespace infllm {

// kernels of the other translation units
int rope_apply_launch(const void* x, int64_t x_hs, int64_t x_ts, void* out, int64_t o_hs, int64_t o_ts,
                      int n_heads, int64_t len, int head_dim, const float* cos_t, const float* sin_t,
                      int64_t table_len, int64_t pos0, int pos_step, int dtype, cudaStream_t s);
int copy_rows_launch(const void* x, int64_t x_hs, int64_t x_ts, void* out, int64_t o_hs, int64_t o_ts,
                     int n_heads, int64_t len, int head_dim, cudaStream_t s);
int pack_units_launch(const void* k, const void* v, int64_t hs, int64_t tok0, int n_new, int block_size, int n_kv_heads,
                      int head_dim, void* out, cudaStream_t s);
int stage_units_launch(const void* const* h_src, void* const* d_dst, int n, int64_t unit_bytes, cudaStream_t s);
int qbar_launch(const void* q, int64_t q_hs, int64_t q_ts, int n_heads, int64_t len, int exc, int head_dim,
                float* qbar, int64_t qbar_stride, int dtype, cudaStream_t s);
int block_topk_launch(const void* bk, int64_t n, int width, const float* qbar, float* scores, int k, int id_base,
                      int32_t* out_ids, float* out_scores, int dtype, cudaStream_t s, unsigned int* ticket,
                      int32_t* out_ids_copy = nullptr);
int block_score_rows_launch(const void* bk, const int32_t* rows, int n, int width, const float* qbar, float* scores,
                            int dtype, cudaStream_t s);
int repr_select_launch(const void* k, int64_t k_hs, int64_t k_ts, const float* score, int64_t score_hs,
                       int64_t tok0, int n_new, int block_size, int repr_topk, int n_heads, int n_kv_heads,
                       int head_dim, void* out, int dtype, cudaStream_t s);
int ingest_token_launch(const void* q, int64_t q_hs, const void* k, int64_t k_hs, const void* v, int64_t v_hs,
                        void* q_loc, void* q_glb, int64_t qs_hs, float* qbar, void* k_raw, void* k_rot, void* v_out,
                        int64_t kv_hs, float* score, int64_t score_hs, int n_heads, int n_kv_heads, int head_dim,
                        const float* cos_t, const float* sin_t, int64_t table_len, int64_t pos_loc, int64_t pos_glb,
                        int dtype, cudaStream_t s, int32_t* clear);
int block_score_launch(const void* bk, int64_t n, int width, const float* qbar, float* scores, int dtype,
                       cudaStream_t s);
int topk_launch(const float* scores, int64_t n, int k, int id_base, int32_t* out_ids, float* out_scores,
                cudaStream_t s);
int comm_allreduce_sum(infllm_comm* c, int which, float* d_buf, size_t n, cudaStream_t s);
int slot_table_update_launch(int32_t* table, const int32_t* ids, const int32_t* slots, int n, cudaStream_t s);
int ptr_table_update_launch(unsigned long long* table, const int32_t* ids, const unsigned long long* vals, int n,
                            cudaStream_t s);

// ------------------------------------------------------------------------------------- LRU table
// cached_blocks[u] of the reference: a dict id -> stamp whose iteration (insertion) order breaks
// ties at eviction (context_manager.py:246-265: stable sort of dict items by stamp).
struct LruTable {
  int capacity;
  std::list<std::pair<int32_t, double>> items;  // dict order
  std::unordered_map<int32_t, std::list<std::pair<int32_t, double>>::iterator> index;

  explicit LruTable(int cap) : capacity(cap) {}
  bool has(int32_t id) const { return index.count(id) != 0; }
  size_t size() const { return items.size(); }
  void clear() {
    items.clear();
    index.clear();
  }
  // context_manager.py:496-502 + 246-265
  void plan(const int32_t* wanted, int n, std::vector<int32_t>* evicted) {
    evicted->clear();
    long num_remove = (long)items.size() - capacity;
    for (int i = 0; i < n; ++i)
      if (!has(wanted[i])) ++num_remove;
    if (num_remove <= 0) return;
    std::vector<std::pair<int32_t, double>> order(items.begin(), items.end());
    std::stable_sort(order.begin(), order.end(),
                     [](const std::pair<int32_t, double>& a, const std::pair<int32_t, double>& b) {
                       return a.second < b.second;
                     });
    std::vector<int32_t> keep(wanted, wanted + n);
    std::sort(keep.begin(), keep.end());
    long removed = 0;
    for (auto& kv : order) {
      if (!std::binary_search(keep.begin(), keep.end(), kv.first)) {
        auto it = index.find(kv.first);
        items.erase(it->second);
        index.erase(it);
        evicted->push_back(kv.first);
        ++removed;
      }
      if (removed >= num_remove) return;
    }
  }
  // context_manager.py:504-513: assignment keeps an existing key in place, a new key goes last
  void stamp(const int32_t* wanted, int n, double value) {
    for (int i = 0; i < n; ++i) set(wanted[i], value);
  }
  void set(int32_t id, double value) {
    auto it = index.find(id);
    if (it != index.end()) {
      it->second->second = value;
    } else {
      items.emplace_back(id, value);
      index[id] = std::prev(items.end());
    }
  }
  void scale(double f) {
    for (auto& kv : items) kv.second *= f;
  }
  bool add(int32_t id, double v) {
    auto it = index.find(id);
    if (it == index.end()) return false;
    it->second->second += v;
    return true;
  }
};

// --------------------------------------------------------------------------------------- context
struct TokenBuffers {
  void* k_raw = nullptr;  // (H_kv, cap, D) un-rotated keys
  void* k_rot = nullptr;  // (H_kv, cap, D) keys rotated to position (token - rope_origin)
  void* v = nullptr;      // (H_kv, cap, D)
  float* score = nullptr; // (H, cap) accumulated local attention mass
  int64_t cap = 0;        // tokens
  int64_t t0 = 0;         // absolute token index of slot 0
  int64_t zero_upto = 0;  // K and V rows in [end of data, zero_upto) are known to hold zeros
};

}  // namespace infllm

using namespace infllm;

struct infllm_ctx {
  infllm_config cfg;
  int esz = 2;                 // bytes per activation element
  int64_t width = 0;           // n_heads * head_dim
  int64_t unit_elems = 0;      // n_kv_heads * block_size * head_dim (K or V of one unit)
  int64_t unit_bytes = 0;      // K and V of one unit
  bool initialized = false;

  int64_t length = 0, frontier = 0, num_blocks = 0, init_len = 0, load_count = 0;
  bool init_full = false;

  TokenBuffers tb;
  void* init_k = nullptr;  // (H_kv, n_init, D)
  void* init_v = nullptr;
  void* block_k = nullptr;  // (block_k_cap, width)
  int64_t block_k_cap = 0;

  // RoPE
  float *cos_t = nullptr, *sin_t = nullptr;
  int64_t tab_len = 0;
  int64_t rope_origin = -1;  // absolute token index that has position 0 in k_rot

  // per-call scratch
  int64_t sub_max = 0;       // tokens per internal sub-append
  void *q_loc = nullptr, *q_glb = nullptr;  // (H, sub_max, D)
  float* qbar = nullptr;     // (sub_max/exc + 1, width)
  float* lse = nullptr;      // (H, exc)
  float *st_acc = nullptr, *st_m = nullptr, *st_l = nullptr;  // carried attention state (H, exc, D) / (H, exc)
  float* scores = nullptr;   // (scores_cap) unit scores
  // chunk_topk_calc (context_manager.py:749-770): in a call of more than one token every exec block of a chunk is
  // ranked over the units that were sealed when the chunk started
  bool chunk_mode = false;
  int64_t call_off = 0;   // where the running internal call starts within the caller's tokens
  int64_t chunk_n0 = 0;   // units sealed at the start of the running chunk
  float* unit_prob = nullptr;    // lru-s: (H, topk * block_size) attention mass of the retrieved units' keys
  float* h_unit_prob = nullptr;  // its pinned host copy
  int64_t scores_cap = 0;
  int32_t* d_topk = nullptr; // (topk)
  infllm_comm* comm = nullptr;  // KV-head-group sharding: the retrieval scores are summed over the ranks
  unsigned int* tickets = nullptr;  // "last CTA" counters of the fused scoring kernel: [0] main stream, [1] look-ahead stream
  int32_t* h_topk = nullptr; // pinned
  float *part_o = nullptr, *part_lse = nullptr, *dec_logits = nullptr;
  int max_parts = 0;

  // unit store
  void* cache = nullptr;  // (max_cached, 2, H_kv, bs, D)
  std::vector<int> free_slots;
  std::vector<cudaEvent_t> slot_ev;   // per slot: behind the last look-ahead copy into it
  std::vector<char> slot_ev_used;
  std::unordered_map<int32_t, int> slot_of;
  // Device table "where unit b lives right now" for the decode attention that resolves the retrieved units
  // itself: the address of the unit's K block — its cache slot once a refill is known to have landed, else its place
  // in the device copy of the store or in the pinned host store (which the GPU reads in place over PCIe).  Every
  // sealed unit has an address, so a one-token attention never has to wait for the host.
  unsigned long long* d_unit_ptrs = nullptr;
  int64_t tab_cap = 0;
  bool table_valid = false;                          // false: rebuild before the next use
  std::unordered_map<int32_t, int32_t> tab_updates;  // entries changed since the last flush: slot, or -1 = the store
  std::unordered_map<int32_t, int32_t> dev_table;    // units whose entry points to a cache slot since the last flush
  int32_t* d_miss = nullptr;                         // cleared with every token (kept for the ingest kernel)
  // One-token appends run ahead of the host: the retrieval of token t is launched, its ids travel to the host on the
  // mail stream, and the host applies them to the LRU order (evictions, refills) only when token t+1 or t+2 is
  // appended — or when somebody asks for the tables.  Ring of the tokens whose ids have not been applied yet.
  struct PendingToken {
    int32_t* h_ids = nullptr;  // pinned: topk ids
    cudaEvent_t ev = nullptr;  // on the mail stream, behind the copy of the ids
    int64_t serial = 0;        // the append call it belongs to
    std::vector<int32_t> listed;  // units the device table showed in a cache slot when the token was launched
    std::vector<int> landing;     // the landing slot of every retrieval position at that time (-1: none)
  };
  static constexpr int kPendSlots = 4, kMaxOutstanding = 1;
  // A retrieved unit that is not in a cache slot is read in place from the store by the one-token attention, which
  // also writes what it read to a landing slot: a free cache slot set aside for retrieval position i.  When the
  // retrieval is applied, that slot simply becomes the unit's cache slot — the refill costs no copy and the unit
  // crosses PCIe once — and another free slot is set aside for position i.
  std::vector<int> landing_slots;   // per retrieval position: the slot set aside, -1 = none
  std::vector<int> landing_listed;  // what the device table (entries tab_cap + i) shows
  std::vector<int> settle_landing;  // per id of the retrieval being applied: the slot it was deposited in, or -1
  PendingToken pend[kPendSlots];
  int pend_head = 0, pend_count = 0;
  int32_t* d_topk_ring = nullptr;  // kPendSlots x topk
  int64_t call_serial = 0;
  cudaStream_t last_stream = nullptr;  // stream of the last append (for calls that take none)
  std::vector<void*> slabs;  // pinned host memory
  std::future<void*> slab_future;  // the next slab, being pinned by a helper thread
  bool slab_pending = false;
  int64_t slab_units = 0;
  LruTable lru{0};

  // tensor-core path: tensor maps of the buffers the kernels read through TMA
  bool use_tc = false;
  int64_t init_cap = 0;  // rows allocated for the sink buffers (at least one 128-row tile)
  CUtensorMap m_qloc, m_qglb, m_krot, m_kraw, m_v, m_cache, m_initk, m_initv;
  int* tc_err = nullptr;
  // The tensor-core kernels record a bounded wait that ran out in a device-side record; a copy of it travels to
  // h_tc_err with the candidate scores of every exec block and at the end of every call, and the host reads it
  // behind a wait it performs anyway: infllm_ctx_append then returns INFLLM_E_TIMEOUT.
  int32_t* h_tc_err = nullptr;   // pinned, 4 words
  cudaEvent_t ev_err = nullptr;  // behind the last copy of the record
  bool err_pending = false;
  float* tc_part = nullptr;  // partial results of the two-head attention kernel's key-tile runs
  size_t tc_part_floats = 0;

  // look-ahead retrieval inside one append: while exec block t runs, the top-k of t+1 over the units known
  // so far is computed on a second stream and its misses are staged into spare slots; after t's sealing
  // only the candidates (that top-k plus the newly sealed units) are re-scored and ranked on the host
  float* scores_aux = nullptr;
  int64_t scores_aux_cap = 0;
  struct LookAhead {
    int64_t target = -1;   // exec block (index inside the current call) this look-ahead is for
    int64_t n_spec = 0;    // units that existed when it was launched
    bool launched = false, staged = false;
    std::vector<int32_t> ids;
    int32_t* h_ids = nullptr;  // pinned: ids written by the device
    cudaEvent_t ev = nullptr;
    cudaEvent_t ev_staged = nullptr;  // on the copy stream, behind the copies staged for this exec block
    bool staged_recorded = false;
  };
  static constexpr int kMaxLookDepth = 8;
  int look_depth = 2;                             // exec blocks ranked ahead (cfg.look_depth overrides)
  LookAhead la[kMaxLookDepth + 1];
  std::unordered_map<int32_t, int64_t> staged_for;  // staged unit -> latest exec block that wants it
  int32_t* h_spec = nullptr;        // pinned: look-ahead ids
  int32_t* h_cand_rows = nullptr;   // pinned: candidate unit ids
  float* h_cand_scores = nullptr;   // pinned: their scores
  float* d_cand_scores = nullptr;   // device side of the same mailbox
  int32_t* d_spec = nullptr;        // device side of the look-ahead id mailboxes, (look_depth + 1) x topk
  cudaStream_t mail_stream = nullptr;  // carries the small result copies to the host, off the main stream
  int cand_cap = 0;
  std::unordered_map<int32_t, int> staged;  // unit -> slot holding a prefetched copy
  bool staged_pending = false;              // staged copies issued since the last wait on them

  // sealed units leave through a packing buffer (two in rotation) and one copy per run of units
  void* pack_buf[2] = {nullptr, nullptr};
  cudaEvent_t ev_pack[2] = {nullptr, nullptr};
  bool pack_used[2] = {false, false};
  int pack_idx = 0, pack_units = 0;
  cudaStream_t d2h_stream = nullptr;
  cudaEvent_t ev_d2h = nullptr, ev_ingest = nullptr;
  bool ingest_event_due = false;  // a one-token append left ev_ingest unrecorded
  bool d2h_recorded = false;
  int64_t d2h_synced_upto_urgent = 0;  // the same bookkeeping for the urgent stream
  int64_t d2h_synced_upto = 0;  // units below this id are known to be in the host store as far as copy_stream is concerned

  cudaStream_t copy_stream = nullptr, aux_stream = nullptr;
  cudaEvent_t ev_main = nullptr, ev_copy = nullptr, ev_sync = nullptr, ev_attn = nullptr, ev_attn_prev = nullptr, ev_spec = nullptr,
              ev_cand = nullptr, ev_seal = nullptr, ev_stage = nullptr;
  bool attn_recorded = false, attn_prev_recorded = false, spec_recorded = false;
  cudaStream_t urgent_stream = nullptr;  // copies an exec block is waiting for, past the queue of staged copies

  // optional per-kernel timing (infllm_ctx_profile): CUDA events around the launches on their stream
  bool prof = false;
  std::vector<cudaEvent_t> ev_pool;
  size_t ev_used = 0;
  struct Pending { int slot; cudaEvent_t a, b; };
  std::vector<Pending> pending;
  double prof_ms[INFLLM_PROF_SLOTS] = {0}, prof_work[INFLLM_PROF_SLOTS] = {0};
  int64_t prof_launches[INFLLM_PROF_SLOTS] = {0};

  // optional event trace of the exec-block loop (infllm_ctx_trace): (label, exec block, event) in record order
  bool trace_on = false;
  struct Mark { int label; int64_t eb; cudaEvent_t ev; };
  std::vector<Mark> marks;

  // host-side time spent in each phase of the exec-block loop, microseconds (diagnostics)
  double host_us[INFLLM_HOST_TIMERS] = {0};

  // trace of the last append
  std::vector<std::vector<int32_t>> trace_topk;
  infllm_ctx_info counters{};

  char* host_unit(int64_t b) { return (char*)slabs[b / slab_units] + (b % slab_units) * unit_bytes; }
  // Device copy of the store.  The reference keeps sealed units on the host because its GPUs have tens of GB; with
  // 180 GB of HBM a copy of the first dev_cap units stays on the device as well, and a cache refill of such a unit is
  // a device-to-device copy instead of a trip over PCIe.  Nothing else changes: the cache, its LRU order and the host
  // store are what they were.  Units [0, dev_units) have a device copy.
  std::vector<void*> dev_slabs;
  int64_t dev_cap = 0, dev_units = 0;
  bool dev_resident(int64_t b) const { return b < dev_units; }
  char* dev_unit(int64_t b) { return (char*)dev_slabs[b / slab_units] + (b % slab_units) * unit_bytes; }
  const char* unit_src(int64_t b) { return dev_resident(b) ? dev_unit(b) : host_unit(b); }
};

namespace {

int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// trace labels
enum { TR_ATTN_BEGIN = 0, TR_ATTN_END, TR_URGENT_END, TR_SEAL_END, TR_REST_END, TR_SPEC_BEGIN, TR_SPEC_END,
       TR_STAGE_BEGIN, TR_STAGE_END, TR_REPR_END, TR_PACK_END, TR_LATE_BEGIN, TR_LATE_END };
void trace_mark(infllm_ctx* c, cudaStream_t s, int label, int64_t eb);
void trace_mark(infllm_ctx* c, cudaStream_t s, int label, int64_t eb) {
  if (!c->trace_on || c->marks.size() > 20000) return;
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, s);
  c->marks.push_back({label, eb, e});
}

struct HostTimer {
  double* acc;
  std::chrono::steady_clock::time_point t0;
  explicit HostTimer(double* a) : acc(a), t0(std::chrono::steady_clock::now()) {}
  ~HostTimer() { *acc += std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count(); }
};

// timing scope: records an event pair around the launches issued while it lives
struct ProfScope {
  infllm_ctx* c;
  cudaStream_t s;
  int slot;
  cudaEvent_t a = nullptr, b = nullptr;
  ProfScope(infllm_ctx* c_, cudaStream_t s_, int slot_, double work) : c(c_), s(s_), slot(slot_) {
    if (!c->prof) return;
    while (c->ev_pool.size() < c->ev_used + 2) {
      cudaEvent_t e;
      if (cudaEventCreate(&e) != cudaSuccess) return;
      c->ev_pool.push_back(e);
    }
    a = c->ev_pool[c->ev_used++];
    b = c->ev_pool[c->ev_used++];
    c->prof_work[slot] += work;
    c->prof_launches[slot] += 1;
    cudaEventRecord(a, s);
  }
  ~ProfScope() {
    if (!a) return;
    cudaEventRecord(b, s);
    c->pending.push_back({slot, a, b});
  }
};

int free_buffers(TokenBuffers& tb, cudaStream_t s) {
  if (tb.k_raw) INFLLM_CUDA_OK(cudaFreeAsync(tb.k_raw, s));
  if (tb.k_rot) INFLLM_CUDA_OK(cudaFreeAsync(tb.k_rot, s));
  if (tb.v) INFLLM_CUDA_OK(cudaFreeAsync(tb.v, s));
  if (tb.score) INFLLM_CUDA_OK(cudaFreeAsync(tb.score, s));
  tb = TokenBuffers{};
  return INFLLM_OK;
}

int lazy_init(infllm_ctx* c, cudaStream_t s) {
  const infllm_config& g = c->cfg;
  // keep freed device memory in the pool: the token buffers are re-created at every compaction
  cudaMemPool_t pool;
  INFLLM_CUDA_OK(cudaDeviceGetDefaultMemPool(&pool, g.device));
  uint64_t keep = UINT64_MAX;
  INFLLM_CUDA_OK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));

  {
    // refills from a device copy of the store are kernels of a few small CTAs: on high-priority streams they are
    // placed ahead of the CTAs of the main stream's grids that have not started yet
    int lo = 0, hi = 0;
    INFLLM_CUDA_OK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    INFLLM_CUDA_OK(cudaStreamCreateWithPriority(&c->copy_stream, cudaStreamNonBlocking, hi));
    INFLLM_CUDA_OK(cudaStreamCreateWithPriority(&c->urgent_stream, cudaStreamNonBlocking, hi));
  }
  INFLLM_CUDA_OK(cudaStreamCreateWithFlags(&c->d2h_stream, cudaStreamNonBlocking));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_d2h, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_ingest, cudaEventDisableTiming));
  c->pack_units = g.exc_block_size / g.block_size + 2;
  for (int i = 0; i < 2; ++i) {
    INFLLM_CUDA_OK(cudaMalloc(&c->pack_buf[i], (int64_t)c->pack_units * c->unit_bytes));
    INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_pack[i], cudaEventDisableTiming));
  }
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_main, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_copy, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_sync, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_attn, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_attn_prev, cudaEventDisableTiming));
  {
    int lo = 0, hi = 0;  // the look-ahead kernels are short and latency matters: highest priority
    INFLLM_CUDA_OK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    INFLLM_CUDA_OK(cudaStreamCreateWithPriority(&c->aux_stream, cudaStreamNonBlocking, hi));
  }
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_spec, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_cand, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_seal, cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_stage, cudaEventDisableTiming));

  const int64_t D = g.head_dim, H = g.n_heads, HKV = g.n_kv_heads;
  c->sub_max = round_up(std::max<int64_t>(16384, 2 * g.exc_block_size), g.exc_block_size);
  // RoPE table: positions of a call stay below n_local + sub_max; twice that so that the origin
  // moves (and the window is re-rotated) only every sub_max tokens
  c->tab_len = g.n_local + 2 * c->sub_max + 1;
  INFLLM_CUDA_OK(cudaMalloc(&c->cos_t, c->tab_len * (D / 2) * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->sin_t, c->tab_len * (D / 2) * sizeof(float)));
  {
    std::vector<float> inv(D / 2);
    // rope.py:22-24: 1 / base ** (arange(0, D, 2) / D) in fp32
    for (int i = 0; i < D / 2; ++i) inv[i] = 1.0f / powf(g.rope_base, (float)(2 * i) / (float)D);
    INFLLM_TRY(infllm_rope_table(inv.data(), g.rope_scale, (int)D, c->tab_len, c->cos_t, c->sin_t, s));
  }
  // buffers that TMA tiles may over-read are zero-filled once: a tile row past the valid data must not
  // hold NaN bit patterns (0 * NaN would poison P V)
  c->init_cap = std::max<int64_t>(g.n_init, 128);
  INFLLM_CUDA_OK(cudaMalloc(&c->init_k, HKV * c->init_cap * D * c->esz));
  INFLLM_CUDA_OK(cudaMalloc(&c->init_v, HKV * c->init_cap * D * c->esz));
  INFLLM_CUDA_OK(cudaMemsetAsync(c->init_k, 0, HKV * c->init_cap * D * c->esz, s));
  INFLLM_CUDA_OK(cudaMemsetAsync(c->init_v, 0, HKV * c->init_cap * D * c->esz, s));
  INFLLM_CUDA_OK(cudaMalloc(&c->q_loc, H * c->sub_max * D * c->esz));
  INFLLM_CUDA_OK(cudaMalloc(&c->q_glb, H * c->sub_max * D * c->esz));
  INFLLM_CUDA_OK(cudaMemsetAsync(c->q_loc, 0, H * c->sub_max * D * c->esz, s));
  INFLLM_CUDA_OK(cudaMemsetAsync(c->q_glb, 0, H * c->sub_max * D * c->esz, s));
  INFLLM_CUDA_OK(cudaMalloc(&c->qbar, (c->sub_max / g.exc_block_size + 1) * c->width * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->lse, H * g.exc_block_size * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->st_acc, H * g.exc_block_size * D * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->st_m, H * g.exc_block_size * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->st_l, H * g.exc_block_size * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->d_topk, std::max(1, g.topk) * sizeof(int32_t)));
  INFLLM_CUDA_OK(cudaMalloc((void**)&c->d_miss, sizeof(int32_t)));
  INFLLM_CUDA_OK(cudaMemsetAsync(c->d_miss, 0, sizeof(int32_t), s));
  {
    const int per = std::max(1, g.topk);
    INFLLM_CUDA_OK(cudaMalloc((void**)&c->d_topk_ring, (size_t)infllm_ctx::kPendSlots * per * sizeof(int32_t)));
    for (auto& pt : c->pend) {
      INFLLM_CUDA_OK(cudaHostAlloc((void**)&pt.h_ids, per * sizeof(int32_t), cudaHostAllocDefault));
      INFLLM_CUDA_OK(cudaEventCreateWithFlags(&pt.ev, cudaEventDisableTiming));
    }
  }
  INFLLM_CUDA_OK(cudaMalloc((void**)&c->tickets, 2 * sizeof(unsigned int)));
  INFLLM_CUDA_OK(cudaMemsetAsync(c->tickets, 0, 2 * sizeof(unsigned int), s));
  INFLLM_CUDA_OK(cudaHostAlloc((void**)&c->h_topk, std::max(1, g.topk) * sizeof(int32_t),
                               cudaHostAllocDefault));
  INFLLM_CUDA_OK(cudaHostAlloc((void**)&c->h_spec, std::max(1, g.topk) * sizeof(int32_t), cudaHostAllocDefault));
  c->cand_cap = g.topk + (c->look_depth + 1) * (g.exc_block_size / g.block_size + 2) + 4;
  for (auto& l : c->la) {
    INFLLM_CUDA_OK(cudaHostAlloc((void**)&l.h_ids, std::max(1, g.topk) * sizeof(int32_t), cudaHostAllocDefault));
    INFLLM_CUDA_OK(cudaEventCreateWithFlags(&l.ev, cudaEventDisableTiming));
    INFLLM_CUDA_OK(cudaEventCreateWithFlags(&l.ev_staged, cudaEventDisableTiming));
  }
  INFLLM_CUDA_OK(cudaHostAlloc((void**)&c->h_cand_rows, c->cand_cap * sizeof(int32_t), cudaHostAllocDefault));
  INFLLM_CUDA_OK(cudaHostAlloc((void**)&c->h_cand_scores, c->cand_cap * sizeof(float), cudaHostAllocDefault));
  INFLLM_CUDA_OK(cudaMalloc((void**)&c->d_cand_scores, c->cand_cap * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc((void**)&c->d_spec, (c->look_depth + 1) * std::max(1, g.topk) * sizeof(int32_t)));
  INFLLM_CUDA_OK(cudaStreamCreateWithFlags(&c->mail_stream, cudaStreamNonBlocking));
  // decode partials: window + units + sink + overflow, each segment may add one ragged chunk
  int64_t dec_keys = (int64_t)g.n_local + (int64_t)g.topk * g.block_size + g.n_init + g.block_size + g.exc_block_size;
  (void)dec_keys;
  c->max_parts = 2 * 148;  // the decode attention launches at most two CTAs per SM, one partial each
  INFLLM_CUDA_OK(cudaMalloc(&c->part_o, (int64_t)c->max_parts * H * D * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->part_lse, (int64_t)c->max_parts * H * sizeof(float)));
  INFLLM_CUDA_OK(cudaMalloc(&c->dec_logits, H * ((int64_t)g.n_local + 1) * sizeof(float)));
  // max_cached_block slots hold the cache proper; topk more per look-ahead step hold the copies staged ahead
  const int64_t n_slots = (int64_t)g.max_cached_block + (int64_t)c->look_depth * g.topk;
  INFLLM_CUDA_OK(cudaMalloc(&c->cache, n_slots * c->unit_bytes));
  INFLLM_CUDA_OK(cudaMemsetAsync(c->cache, 0, n_slots * c->unit_bytes, s));
  c->use_tc = D == 128 && g.block_size % 128 == 0 && !(g.debug_flags & 1);
  if (c->use_tc) {
    INFLLM_TRY(encode_rows_map(&c->m_qloc, g.dtype, c->q_loc, c->sub_max, H, c->sub_max * D, D));
    INFLLM_TRY(encode_rows_map(&c->m_qglb, g.dtype, c->q_glb, c->sub_max, H, c->sub_max * D, D));
    INFLLM_TRY(encode_rows_map(&c->m_initk, g.dtype, c->init_k, c->init_cap, HKV, c->init_cap * D, D));
    INFLLM_TRY(encode_rows_map(&c->m_initv, g.dtype, c->init_v, c->init_cap, HKV, c->init_cap * D, D));
    // cache slots as (D, block_size, H_kv, 2 * slots): the last index is slot * 2 + (0 keys | 1 values)
    uint64_t dims[4] = {128, (uint64_t)g.block_size, (uint64_t)HKV, 2ull * (uint64_t)n_slots};
    uint64_t strides[3] = {(uint64_t)(D * c->esz), (uint64_t)(g.block_size * D * c->esz),
                           (uint64_t)(c->unit_bytes / 2)};
    uint32_t box[4] = {64, 128, 1, 1};
    INFLLM_TRY(encode_tensor_map(&c->m_cache, g.dtype, c->cache, 4, dims, strides, box));
    INFLLM_TRY(tc_get_error_ptr(&c->tc_err));
    INFLLM_CUDA_OK(cudaHostAlloc((void**)&c->h_tc_err, 4 * sizeof(int32_t), cudaHostAllocDefault));
    c->h_tc_err[0] = c->h_tc_err[1] = c->h_tc_err[2] = c->h_tc_err[3] = 0;
    INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->ev_err, cudaEventDisableTiming));
  }
  c->free_slots.clear();
  for (int i = (int)n_slots - 1; i >= 0; --i) c->free_slots.push_back(i);
  c->slot_ev.assign(n_slots, nullptr);
  c->slot_ev_used.assign(n_slots, 0);
  c->slab_units = std::max<int64_t>(16, (128ll << 20) / c->unit_bytes);
  c->dev_cap = (int64_t)g.device_store_mb * (1ll << 20) / c->unit_bytes;  // device copy of the store, in units
  c->initialized = true;
  return INFLLM_OK;
}

// Sends a copy of the tensor-core kernels' error record to the host on `copy_on`, ordered behind what stream s has
// enqueued so far (copy_on == s: no extra ordering needed).
int send_device_error(infllm_ctx* c, cudaStream_t s, cudaStream_t copy_on) {
  if (!c->tc_err || !c->h_tc_err) return INFLLM_OK;
  if (copy_on != s) {
    INFLLM_CUDA_OK(cudaEventRecord(c->ev_main, s));
    INFLLM_CUDA_OK(cudaStreamWaitEvent(copy_on, c->ev_main, 0));
  }
  INFLLM_CUDA_OK(cudaMemcpyAsync(c->h_tc_err, c->tc_err, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, copy_on));
  INFLLM_CUDA_OK(cudaEventRecord(c->ev_err, copy_on));
  c->err_pending = true;
  return INFLLM_OK;
}

// Reads the last copy of the record if it has landed (never waits): a recorded error becomes INFLLM_E_TIMEOUT,
// and the device-side record is cleared on s so that the next report names a new event.
int poll_device_error(infllm_ctx* c, cudaStream_t s) {
  if (!c->err_pending || cudaEventQuery(c->ev_err) != cudaSuccess) {
    cudaGetLastError();  // cudaErrorNotReady is not an error of ours
    return INFLLM_OK;
  }
  c->err_pending = false;
  if (c->h_tc_err[0] == 0) return INFLLM_OK;
  const int code = c->h_tc_err[0], where = c->h_tc_err[1], bx = c->h_tc_err[2], by = c->h_tc_err[3];
  c->h_tc_err[0] = 0;
  INFLLM_CUDA_OK(cudaMemsetAsync(c->tc_err, 0, 4 * sizeof(int32_t), s));
  return fail(INFLLM_E_TIMEOUT, "a bounded wait of a tensor-core kernel ran out (code %d, wait %d, CTA %d,%d): the rows "
              "that CTA was to write are not valid", code, where, bx, by);
}

// make room for tokens [frontier, length + add) in the token buffers
int ensure_tokens(infllm_ctx* c, int64_t add, cudaStream_t s) {
  const infllm_config& g = c->cfg;
  TokenBuffers& tb = c->tb;
  const int64_t D = g.head_dim, H = g.n_heads, HKV = g.n_kv_heads;
  if (tb.cap > 0 && c->length + add - tb.t0 <= tb.cap) return INFLLM_OK;
  const int64_t live0 = c->frontier, live = c->length - c->frontier;
  const int64_t need = live + add;
  TokenBuffers nb;
  nb.cap = round_up(need + std::max<int64_t>(4096, g.n_local), 256);
  nb.t0 = live0;
  INFLLM_CUDA_OK(cudaMallocAsync(&nb.k_raw, HKV * nb.cap * D * c->esz, s));
  INFLLM_CUDA_OK(cudaMallocAsync(&nb.k_rot, HKV * nb.cap * D * c->esz, s));
  INFLLM_CUDA_OK(cudaMallocAsync(&nb.v, HKV * nb.cap * D * c->esz, s));
  INFLLM_CUDA_OK(cudaMallocAsync((void**)&nb.score, H * nb.cap * sizeof(float), s));
  if (live > 0) {
    const int64_t off = (live0 - tb.t0) * D * c->esz;
    const size_t w = live * D * c->esz;
    INFLLM_CUDA_OK(cudaMemcpy2DAsync(nb.k_raw, nb.cap * D * c->esz, (char*)tb.k_raw + off, tb.cap * D * c->esz, w, HKV,
                                     cudaMemcpyDeviceToDevice, s));
    INFLLM_CUDA_OK(cudaMemcpy2DAsync(nb.k_rot, nb.cap * D * c->esz, (char*)tb.k_rot + off, tb.cap * D * c->esz, w, HKV,
                                     cudaMemcpyDeviceToDevice, s));
    INFLLM_CUDA_OK(cudaMemcpy2DAsync(nb.v, nb.cap * D * c->esz, (char*)tb.v + off, tb.cap * D * c->esz, w, HKV,
                                     cudaMemcpyDeviceToDevice, s));
    INFLLM_CUDA_OK(cudaMemcpy2DAsync(nb.score, nb.cap * sizeof(float), tb.score + (live0 - tb.t0),
                                     tb.cap * sizeof(float), live * sizeof(float), H, cudaMemcpyDeviceToDevice, s));
  }
  if (tb.cap > 0) {
    // the packing kernels of sealed units read the old buffers on the device-to-host stream
    if (c->d2h_recorded) INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->ev_d2h, 0));
    INFLLM_TRY(free_buffers(tb, s));
  }
  c->tb = nb;
  if (c->use_tc) {
    INFLLM_TRY(encode_rows_map(&c->m_krot, g.dtype, nb.k_rot, nb.cap, HKV, nb.cap * D, D));
    INFLLM_TRY(encode_rows_map(&c->m_kraw, g.dtype, nb.k_raw, nb.cap, HKV, nb.cap * D, D));
    INFLLM_TRY(encode_rows_map(&c->m_v, g.dtype, nb.v, nb.cap, HKV, nb.cap * D, D));
  }
  return INFLLM_OK;
}

int ensure_block_k(infllm_ctx* c, int64_t n, cudaStream_t s) {
  if (n <= c->block_k_cap) return INFLLM_OK;
  int64_t cap = std::max<int64_t>(16, c->block_k_cap);
  while (cap < n) cap *= 2;  // VectorTensor.append_cache doubles (context_manager.py:128-138)
  void* nb = nullptr;
  INFLLM_CUDA_OK(cudaMallocAsync(&nb, cap * c->width * c->esz, s));
  if (c->num_blocks > 0)
    INFLLM_CUDA_OK(cudaMemcpyAsync(nb, c->block_k, c->num_blocks * c->width * c->esz, cudaMemcpyDeviceToDevice, s));
  if (c->block_k) {
    if (c->spec_recorded) INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->ev_spec, 0));  // look-ahead scoring reads the old rows
    INFLLM_CUDA_OK(cudaFreeAsync(c->block_k, s));
  }
  c->block_k = nb;
  c->block_k_cap = cap;
  return INFLLM_OK;
}

// Pinning a slab takes tens of milliseconds; a helper thread does it ahead of need
void* alloc_slab(int device, size_t bytes) {
  void* p = nullptr;
  if (cudaSetDevice(device) != cudaSuccess || cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

int ensure_host_units(infllm_ctx* c, int64_t n) {
  const size_t bytes = (size_t)(c->slab_units * c->unit_bytes);
  while ((int64_t)c->slabs.size() * c->slab_units < n) {
    void* p = nullptr;
    if (c->slab_pending) {
      p = c->slab_future.get();
      c->slab_pending = false;
    }
    if (!p) {
      cudaError_t e = cudaHostAlloc(&p, bytes, cudaHostAllocDefault);
      if (e != cudaSuccess) return fail(INFLLM_E_NOMEM, "pinned host store: cudaHostAlloc of %lld bytes failed: %s",
                                        (long long)bytes, cudaGetErrorString(e));
    }
    c->slabs.push_back(p);
  }
  // once the last slab is half full, the next one is pinned in the background
  if (!c->slab_pending && n + c->slab_units / 2 > (int64_t)c->slabs.size() * c->slab_units) {
    c->slab_future = std::async(std::launch::async, alloc_slab, c->cfg.device, bytes);
    c->slab_pending = true;
  }
  return INFLLM_OK;
}

int ensure_scores(infllm_ctx* c, int64_t n, cudaStream_t s) {
  if (n <= c->scores_cap) return INFLLM_OK;
  int64_t cap = std::max<int64_t>(1024, c->scores_cap);
  while (cap < n) cap *= 2;
  if (c->scores) INFLLM_CUDA_OK(cudaFreeAsync(c->scores, s));
  INFLLM_CUDA_OK(cudaMallocAsync((void**)&c->scores, cap * sizeof(float), s));
  c->scores_cap = cap;
  return INFLLM_OK;
}

// scoring and top-k of n units on stream s.  Alone, one fused launch; with a communicator (KV-head-group sharding:
// this context holds a slice of the heads) the scores are summed over the ranks between the two halves, so that
// every rank ranks the same numbers.  `which` picks the communicator of the stream (0 main, 1 look-ahead).
int score_topk(infllm_ctx* c, int64_t n, const float* qbar, float* scores, int32_t* d_ids, cudaStream_t s, int which,
               int k = 0, int32_t* ids_copy = nullptr) {
  const infllm_config& g = c->cfg;
  if (k <= 0) k = g.topk;
  if (!c->comm)
    return block_topk_launch(c->block_k, n, (int)c->width, qbar, scores, k, 0, d_ids, nullptr, g.dtype, s,
                             c->tickets + which, ids_copy);
  INFLLM_TRY(block_score_launch(c->block_k, n, (int)c->width, qbar, scores, g.dtype, s));
  INFLLM_TRY(comm_allreduce_sum(c->comm, which, scores, (size_t)n, s));
  return topk_launch(scores, n, k, 0, d_ids, nullptr, s);
}

// ids of one exec block straight from the device scorer: scoring + top-k, then a host sync on the result
int retrieve_now(infllm_ctx* c, int eb_in_call, std::vector<int32_t>* ids, cudaStream_t s) {
  const infllm_config& g = c->cfg;
  ids->clear();
  const int64_t n = c->chunk_mode ? c->chunk_n0 : c->num_blocks;
  if (n <= g.topk) {  // context_manager.py:370-371, :553-559
    for (int64_t b = 0; b < n; ++b) ids->push_back((int32_t)b);
    return INFLLM_OK;
  }
  INFLLM_TRY(ensure_scores(c, n, s));
  {
    ProfScope ps(c, s, INFLLM_PROF_TOPK, (double)n * c->width * c->esz);
    INFLLM_TRY(score_topk(c, n, c->qbar + (int64_t)eb_in_call * c->width, c->scores, c->d_topk, s, 0));
  }
  INFLLM_CUDA_OK(cudaMemcpyAsync(c->h_topk, c->d_topk, g.topk * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  INFLLM_CUDA_OK(cudaEventRecord(c->ev_sync, s));
  INFLLM_CUDA_OK(cudaEventSynchronize(c->ev_sync));  // the ids decide the cache plan (context_manager.py:163)
  ids->assign(c->h_topk, c->h_topk + g.topk);
  return INFLLM_OK;
}

// look-ahead for a LATER exec block of the call, on the second stream: top-k over the units sealed so far
int lookahead_launch(infllm_ctx* c, int64_t target, cudaStream_t s) {
  const infllm_config& g = c->cfg;
  infllm_ctx::LookAhead& la = c->la[target % (c->look_depth + 1)];
  la.target = target;
  la.launched = true;
  la.staged = false;
  la.staged_recorded = false;
  la.n_spec = c->num_blocks;
  la.ids.clear();
  if (la.n_spec <= g.topk) return INFLLM_OK;  // every known unit is a candidate; nothing to rank
  // ev_seal was recorded on s right after the last sealing (or after the query means at the start of the
  // call): the look-ahead needs nothing that s enqueued later, in particular not the rest of the score pass
  INFLLM_CUDA_OK(cudaStreamWaitEvent(c->aux_stream, c->ev_seal, 0));
  if (la.n_spec > c->scores_aux_cap) {
    int64_t cap = std::max<int64_t>(1024, c->scores_aux_cap);
    while (cap < la.n_spec) cap *= 2;
    if (c->scores_aux) INFLLM_CUDA_OK(cudaFreeAsync(c->scores_aux, c->aux_stream));
    INFLLM_CUDA_OK(cudaMallocAsync((void**)&c->scores_aux, cap * sizeof(float), c->aux_stream));
    c->scores_aux_cap = cap;
  }
  trace_mark(c, c->aux_stream, TR_SPEC_BEGIN, target);
  ProfScope ps(c, c->aux_stream, INFLLM_PROF_TOPK, (double)la.n_spec * c->width * c->esz);
  int32_t* d_ids = c->d_spec + (target % (c->look_depth + 1)) * std::max(1, g.topk);
  INFLLM_TRY(score_topk(c, la.n_spec, c->qbar + target * c->width, c->scores_aux, d_ids, c->aux_stream, 1));
  INFLLM_CUDA_OK(cudaMemcpyAsync(la.h_ids, d_ids, g.topk * sizeof(int32_t), cudaMemcpyDeviceToHost, c->aux_stream));
  trace_mark(c, c->aux_stream, TR_SPEC_END, target);
  INFLLM_CUDA_OK(cudaEventRecord(la.ev, c->aux_stream));
  INFLLM_CUDA_OK(cudaEventRecord(c->ev_spec, c->aux_stream));
  c->spec_recorded = true;
  return INFLLM_OK;
}

// an event behind the copy just issued into a cache slot on the copy stream: whoever later writes the slot from
// another stream waits for it (the copy may have been abandoned, never awaited, and still be in flight)
int mark_slot_copy(infllm_ctx* c, void* slot_ptr) {
  const int slot = (int)(((char*)slot_ptr - (char*)c->cache) / c->unit_bytes);
  if (!c->slot_ev[slot]) INFLLM_CUDA_OK(cudaEventCreateWithFlags(&c->slot_ev[slot], cudaEventDisableTiming));
  INFLLM_CUDA_OK(cudaEventRecord(c->slot_ev[slot], c->copy_stream));
  c->slot_ev_used[slot] = 1;
  return INFLLM_OK;
}

// after the look-ahead ids arrived: copy the ones that are not resident into spare slots (side stream)
int lookahead_stage(infllm_ctx* c, int64_t target) {
  const infllm_config& g = c->cfg;
  infllm_ctx::LookAhead& la = c->la[target % (c->look_depth + 1)];
  if (la.n_spec <= g.topk) {
    for (int64_t b = 0; b < la.n_spec; ++b) la.ids.push_back((int32_t)b);
  } else {
    INFLLM_CUDA_OK(cudaEventSynchronize(la.ev));
    la.ids.assign(la.h_ids, la.h_ids + g.topk);
  }
  la.staged = true;
  std::vector<const void*> src;
  std::vector<void*> dst;
  std::vector<char> on_device;
  for (int32_t b : la.ids) {
    if (c->slot_of.count(b)) continue;
    auto sf = c->staged_for.find(b);
    if (sf != c->staged_for.end()) {  // already on its way for an earlier exec block: keep it until this one
      sf->second = std::max(sf->second, target);
      continue;
    }
    if (c->free_slots.empty()) break;  // no spare slot: the unit is fetched at plan time instead
    int slot = c->free_slots.back();
    c->free_slots.pop_back();
    c->staged[b] = slot;
    c->staged_for[b] = target;
    if (b >= c->d2h_synced_upto) {  // sealed recently: its copy-out must land in the store first
      INFLLM_CUDA_OK(cudaStreamWaitEvent(c->copy_stream, c->ev_d2h, 0));
      c->d2h_synced_upto = c->num_blocks;
    }
    src.push_back(c->unit_src(b));
    dst.push_back((char*)c->cache + (int64_t)slot * c->unit_bytes);
    on_device.push_back(c->dev_resident(b));
    if (!c->dev_resident(b)) c->counters.h2d_bytes += c->unit_bytes;
    c->staged_pending = true;
  }
  if (!src.empty()) {
    // the spare slots taken above may have held units that the previous exec block's attention read
    if (c->attn_prev_recorded) INFLLM_CUDA_OK(cudaStreamWaitEvent(c->copy_stream, c->ev_attn_prev, 0));
    trace_mark(c, c->copy_stream, TR_STAGE_BEGIN, target);  // behind the waits: the interval is copy time only
    // Units that have a device copy are gathered by the copy kernel (one launch for the batch); units that only the
    // pinned host store holds travel by one cudaMemcpyAsync each on the copy engine: a kernel that reads host memory
    // gets more out of the link (49 against 38 GB/s) but its CTAs sit on SMs for the whole transfer and slowed the
    // exec-block attention by a tenth when measured, so that the prompt took longer - also when only 4 of a batch's
    // 13 units went through the kernel on a stream of its own beside the copy engine (attention 88 -> 92 us, prompt
    // unchanged; 6 and more units: slower).  Flag bit 2: no copy kernel.
    std::vector<const void*> ksrc;
    std::vector<void*> kdst;
    for (size_t i = 0; i < src.size(); ++i) {
      if (!on_device[i] || (g.debug_flags & 4)) {
        INFLLM_CUDA_OK(cudaMemcpyAsync(dst[i], src[i], c->unit_bytes, cudaMemcpyDefault, c->copy_stream));
      } else {
        ksrc.push_back(src[i]);
        kdst.push_back(dst[i]);
      }
    }
    if (!ksrc.empty()) INFLLM_TRY(stage_units_launch(ksrc.data(), kdst.data(), (int)ksrc.size(), c->unit_bytes, c->copy_stream));
    for (size_t i = 0; i < src.size(); ++i) INFLLM_TRY(mark_slot_copy(c, dst[i]));
  }
  if (c->staged_pending) {
    INFLLM_CUDA_OK(cudaEventRecord(c->ev_stage, c->copy_stream));
    // the exec block this batch is for waits for this event only, not for batches staged later for later blocks
    INFLLM_CUDA_OK(cudaEventRecord(la.ev_staged, c->copy_stream));
    la.staged_recorded = true;
  }
  if (!src.empty()) trace_mark(c, c->copy_stream, TR_STAGE_END, target);
  return INFLLM_OK;
}

// score the candidates of the next exec block (look-ahead ids + units sealed since) on s; results to pinned memory
int candidates_launch(infllm_ctx* c, int64_t eb_next, int* n_cand, cudaStream_t s) {
  const infllm_config& g = c->cfg;
  const infllm_ctx::LookAhead& la = c->la[eb_next % (c->look_depth + 1)];
  const int64_t n_spec = la.n_spec;
  const std::vector<int32_t>& spec_ids = la.ids;
  const int64_t n_now = c->num_blocks;
  *n_cand = 0;
  if (n_now <= g.topk) return INFLLM_OK;  // all units, in id order, no scoring (context_manager.py:370-371)
  int n = 0;
  for (int32_t b : spec_ids) c->h_cand_rows[n++] = b;
  for (int64_t b = n_spec; b < n_now && n < c->cand_cap; ++b) c->h_cand_rows[n++] = (int32_t)b;
  if ((int64_t)spec_ids.size() + (n_now - n_spec) > c->cand_cap)
    return fail(INFLLM_E_CAPACITY, "look-ahead: %lld candidates exceed %d", (long long)(spec_ids.size() + n_now - n_spec), c->cand_cap);
  INFLLM_TRY(block_score_rows_launch(c->block_k, c->h_cand_rows, n, (int)c->width,
                                     c->qbar + eb_next * c->width, c->d_cand_scores, g.dtype, s));
  if (c->comm) INFLLM_TRY(comm_allreduce_sum(c->comm, 0, c->d_cand_scores, (size_t)n, s));
  // the scores travel to the host on their own stream so that the main stream goes straight on
  INFLLM_CUDA_OK(cudaEventRecord(c->ev_main, s));
  INFLLM_CUDA_OK(cudaStreamWaitEvent(c->mail_stream, c->ev_main, 0));
  INFLLM_CUDA_OK(cudaMemcpyAsync(c->h_cand_scores, c->d_cand_scores, n * sizeof(float), cudaMemcpyDeviceToHost,
                                 c->mail_stream));
  INFLLM_TRY(send_device_error(c, c->mail_stream, c->mail_stream));  // this exec block's attention is behind ev_main
  INFLLM_CUDA_OK(cudaEventRecord(c->ev_cand, c->mail_stream));
  *n_cand = n;
  return INFLLM_OK;
}

// rank the candidates on the host: descending score, ties to the lower id — the device scorer's order
int candidates_finish(infllm_ctx* c, int n_cand, std::vector<int32_t>* ids) {
  const infllm_config& g = c->cfg;
  ids->clear();
  if (n_cand == 0) {
    for (int64_t b = 0; b < c->num_blocks; ++b) ids->push_back((int32_t)b);
    return INFLLM_OK;
  }
  INFLLM_CUDA_OK(cudaEventSynchronize(c->ev_cand));
  INFLLM_TRY(poll_device_error(c, c->mail_stream));
  std::vector<int> order(n_cand);
  for (int i = 0; i < n_cand; ++i) order[i] = i;
  const int32_t* rows = c->h_cand_rows;
  const float* sc = c->h_cand_scores;
  std::sort(order.begin(), order.end(), [&](int a, int b) {
    if (sc[a] != sc[b]) return sc[a] > sc[b];
    return rows[a] < rows[b];
  });
  for (int i = 0; i < g.topk && i < n_cand; ++i) ids->push_back(rows[order[i]]);
  return INFLLM_OK;
}

// cache plan for `ids` (LRU eviction, stamps), adoption of staged copies, late fetches; s waits for the copies
enum PlanMode {
  PLAN_PREFILL = 0,       // the device table is not kept up to date (rebuilt when decode next needs it)
  PLAN_DECODE_SYNC = 1,   // one-token append that waited for its ids: s waits for the refills
  PLAN_DECODE_ASYNC = 2,  // ids of an earlier token applied late: refills go to the copy stream and nobody waits;
                          // a unit is listed in the device table once its copy is known to have landed
};
int mark_slot_copy(infllm_ctx* c, void* slot_ptr);

int plan_and_refill(infllm_ctx* c, const std::vector<int32_t>& ids, int64_t eb, cudaStream_t s, int mode) {
  const infllm_config& g = c->cfg;
  const bool track = mode != PLAN_PREFILL;
  if (!track) c->table_valid = false;
  std::vector<int32_t> evicted;
  c->lru.plan(ids.data(), (int)ids.size(), &evicted);
  for (int32_t b : evicted) {  // MemoryUnit.offload -> CudaCache.delete (context_manager.py:104-109)
    auto it = c->slot_of.find(b);
    if (it != c->slot_of.end()) {
      // a look-ahead that found this unit cached did not stage it: if a later exec block wants it, the slot keeps
      // its data as a staged copy instead of going back to the pool
      int64_t wanted_by = -1;
      for (int i = 0; i <= c->look_depth; ++i) {
        const infllm_ctx::LookAhead& l = c->la[i];
        if (l.launched && l.staged && l.target > eb && std::find(l.ids.begin(), l.ids.end(), b) != l.ids.end())
          wanted_by = std::max(wanted_by, l.target);
      }
      if (wanted_by >= 0) {
        c->staged[b] = it->second;
        c->staged_for[b] = wanted_by;
      } else {
        c->free_slots.push_back(it->second);
      }
      c->slot_of.erase(it);
      if (track) c->tab_updates[b] = -1;
    }
  }
  c->counters.evictions += (int64_t)evicted.size();
  if (g.cache_strategy == INFLLM_CACHE_LRU) {
    c->load_count += 1;
    c->lru.stamp(ids.data(), (int)ids.size(), (double)c->load_count);
  } else {
    c->lru.stamp(ids.data(), (int)ids.size(), 0.0);
  }
  bool late = false;
  std::vector<const void*> late_src;
  std::vector<void*> late_dst;
  for (int32_t b : ids) {
    if (c->slot_of.count(b)) {
      c->counters.cache_hits += 1;
      continue;
    }
    c->counters.cache_misses += 1;
    auto st = c->staged.find(b);
    if (st != c->staged.end()) {  // the look-ahead already brought it in
      c->slot_of[b] = st->second;
      if (track) c->tab_updates[b] = st->second;
      // s waits for THIS unit's copy: a unit sealed a moment ago can be staged for a later exec block and still be
      // retrieved by this one, so the event of "this exec block's batch" would not cover it
      if (c->slot_ev_used[st->second]) INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->slot_ev[st->second], 0));
      c->staged.erase(st);
      c->staged_for.erase(b);
      continue;
    }
    if (mode == PLAN_DECODE_ASYNC) {
      int ls = -1;
      for (size_t i = 0; i < ids.size() && i < c->settle_landing.size(); ++i)
        if (ids[i] == b) ls = c->settle_landing[i];
      if (ls >= 0) {
        // the token's attention read this unit in place and left it in a landing slot: that slot is its cache slot now
        c->slot_of[b] = ls;
        c->tab_updates[b] = ls;
        if (!c->dev_resident(b)) c->counters.h2d_bytes += c->unit_bytes;  // crossed PCIe inside the attention
        continue;
      }
    }
    if (c->free_slots.empty()) {
      // spare slots are all holding look-ahead copies that were not wanted after all: reclaim one
      if (c->staged.empty())
        return fail(INFLLM_E_CAPACITY, "no free cache slot for unit %d (max_cached_block %d)", b, g.max_cached_block);
      auto victim = c->staged.begin();
      for (auto it2 = c->staged.begin(); it2 != c->staged.end(); ++it2)
        if (std::find(ids.begin(), ids.end(), it2->first) == ids.end()) { victim = it2; break; }
      c->free_slots.push_back(victim->second);
      if (track) c->tab_updates[victim->first] = -1;
      c->staged_for.erase(victim->first);
      c->staged.erase(victim);
    }
    int slot = c->free_slots.back();
    c->free_slots.pop_back();
    c->slot_of[b] = slot;
    if (mode == PLAN_DECODE_SYNC) c->tab_updates[b] = slot;
    const int64_t tok0 = (int64_t)g.n_init + (int64_t)b * g.block_size;  // the unit's first token
    if (tok0 >= c->tb.t0 && tok0 + g.block_size <= c->length) {
      // sealed so recently that its tokens are still in the token buffers: copy on the device, on the main stream
      // (behind the sealing), instead of waiting for the copy-out to land and coming back over PCIe
      const int64_t D = g.head_dim, row = (int64_t)g.block_size * D * c->esz;
      char* dst = (char*)c->cache + (int64_t)slot * c->unit_bytes;
      const int64_t src = (tok0 - c->tb.t0) * D * c->esz, pitch = c->tb.cap * D * c->esz;
      // a look-ahead copy into this slot that was abandoned may still be in flight on the copy stream
      if (c->slot_ev_used[slot]) INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->slot_ev[slot], 0));
      INFLLM_CUDA_OK(cudaMemcpy2DAsync(dst, row, (char*)c->tb.k_raw + src, pitch, row, g.n_kv_heads,
                                       cudaMemcpyDeviceToDevice, s));
      INFLLM_CUDA_OK(cudaMemcpy2DAsync(dst + c->unit_bytes / 2, row, (char*)c->tb.v + src, pitch, row, g.n_kv_heads,
                                       cudaMemcpyDeviceToDevice, s));
      if (mode == PLAN_DECODE_ASYNC) c->tab_updates[b] = slot;  // ordered on s ahead of the next attention
      continue;
    }
    if (mode == PLAN_DECODE_ASYNC) c->tab_updates[b] = slot;  // no landing slot was free: fetched like a waited-for refill
    if (!late) {
      // slots freed above may still be read by the previous exec block's attention
      if (c->attn_recorded) INFLLM_CUDA_OK(cudaStreamWaitEvent(c->urgent_stream, c->ev_attn, 0));
      late = true;
      trace_mark(c, c->urgent_stream, TR_LATE_BEGIN, eb);
    }
    // an abandoned look-ahead copy into this slot may still be in flight on the copy stream
    if (c->slot_ev_used[slot]) INFLLM_CUDA_OK(cudaStreamWaitEvent(c->urgent_stream, c->slot_ev[slot], 0));
    if (b >= c->d2h_synced_upto_urgent) {
      if (c->d2h_recorded) INFLLM_CUDA_OK(cudaStreamWaitEvent(c->urgent_stream, c->ev_d2h, 0));
      c->d2h_synced_upto_urgent = c->num_blocks;
    }
    // on a stream of its own: the exec block must not wait behind the copies staged for later blocks
    if ((g.debug_flags & 4) || !c->dev_resident(b)) {
      INFLLM_CUDA_OK(cudaMemcpyAsync((char*)c->cache + (int64_t)slot * c->unit_bytes, c->unit_src(b), c->unit_bytes,
                                     cudaMemcpyDefault, c->urgent_stream));
    } else {
      late_src.push_back(c->unit_src(b));
      late_dst.push_back((char*)c->cache + (int64_t)slot * c->unit_bytes);
    }
    if (!c->dev_resident(b)) {
      c->counters.h2d_bytes += c->unit_bytes;
      c->counters.h2d_late_bytes += c->unit_bytes;
    }
  }
  // look-ahead copies that were not wanted: their slots go back to the pool (later copies into them are
  // ordered behind the unfinished ones on the side stream; no kernel reads them)
  for (auto it = c->staged.begin(); it != c->staged.end();) {
    if (c->staged_for[it->first] <= eb) {  // staged for this exec block (or an earlier one) and not taken
      c->free_slots.push_back(it->second);
      c->staged_for.erase(it->first);
      it = c->staged.erase(it);
    } else {
      ++it;
    }
  }
  if (!late_src.empty())
    INFLLM_TRY(stage_units_launch(late_src.data(), late_dst.data(), (int)late_src.size(), c->unit_bytes, c->urgent_stream));
  if (late) {
    trace_mark(c, c->urgent_stream, TR_LATE_END, eb);
    INFLLM_CUDA_OK(cudaEventRecord(c->ev_copy, c->urgent_stream));
    INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->ev_copy, 0));
  }
  if (c->staged.empty()) c->staged_pending = false;
  return INFLLM_OK;
}

// bring the device table of unit addresses up to date on stream s
int flush_table(infllm_ctx* c, cudaStream_t s) {
  const int topk = c->cfg.topk;
  if (c->tab_cap < c->block_k_cap || !c->d_unit_ptrs) {
    if (c->d_unit_ptrs) INFLLM_CUDA_OK(cudaFreeAsync(c->d_unit_ptrs, s));
    c->tab_cap = std::max<int64_t>(c->block_k_cap, 1024);
    // entries [tab_cap, tab_cap + topk): the landing slot of every retrieval position
    INFLLM_CUDA_OK(cudaMallocAsync((void**)&c->d_unit_ptrs, (c->tab_cap + topk) * sizeof(unsigned long long), s));
    c->table_valid = false;
  }
  // a free slot set aside for every retrieval position (fewer when the pool runs dry: those positions deposit nothing)
  c->landing_slots.resize(topk, -1);
  for (int i = 0; i < topk; ++i) {
    if (c->landing_slots[i] >= 0 || c->free_slots.empty()) continue;
    const int slot = c->free_slots.back();
    c->free_slots.pop_back();
    // an abandoned look-ahead copy of an earlier prefill may still be on its way into this slot
    if (c->slot_ev_used[slot]) INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->slot_ev[slot], 0));
    c->landing_slots[i] = slot;
  }
  auto slot_addr = [&](int slot) { return (unsigned long long)(uintptr_t)((char*)c->cache + (int64_t)slot * c->unit_bytes); };
  if (!c->table_valid) {
    // every sealed unit at its place in the store; the cached ones whose copies are known to have landed at their
    // slots.  The upload is ordered on s (the runtime stages a pageable source before it returns).
    std::vector<unsigned long long> all((size_t)(c->tab_cap + topk), 0ull);
    for (int i = 0; i < topk; ++i)
      if (c->landing_slots[i] >= 0) all[(size_t)(c->tab_cap + i)] = slot_addr(c->landing_slots[i]);
    c->landing_listed = c->landing_slots;
    // (bit 0 of an address in the store says "read in place and deposit in the landing slot")
    for (int64_t b = 0; b < c->num_blocks; ++b) all[(size_t)b] = (unsigned long long)(uintptr_t)c->unit_src(b) | 1ull;
    c->tab_updates.clear();
    c->dev_table.clear();
    // every cached unit got there by a copy that s waited for (a prefill exec block's plan) or that ran on s
    for (auto& kv : c->slot_of) {
      all[(size_t)kv.first] = slot_addr(kv.second);
      c->dev_table[kv.first] = kv.second;
    }
    if (c->d2h_recorded) INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->ev_d2h, 0));   // the store holds every sealed unit
    INFLLM_CUDA_OK(cudaMemcpyAsync(c->d_unit_ptrs, all.data(), all.size() * sizeof(unsigned long long),
                                   cudaMemcpyHostToDevice, s));
    c->table_valid = true;
    return INFLLM_OK;
  }
  std::vector<int32_t> ids;
  std::vector<unsigned long long> vals;
  c->landing_listed.resize(topk, -1);
  for (int i = 0; i < topk; ++i)
    if (c->landing_listed[i] != c->landing_slots[i]) {
      ids.push_back((int32_t)(c->tab_cap + i));
      vals.push_back(c->landing_slots[i] >= 0 ? slot_addr(c->landing_slots[i]) : 0ull);
      c->landing_listed[i] = c->landing_slots[i];
    }
  for (auto& kv : c->tab_updates) {
    if (kv.first < 0 || kv.first >= c->num_blocks) continue;
    ids.push_back(kv.first);
    if (kv.second >= 0) {
      vals.push_back(slot_addr(kv.second));
      c->dev_table[kv.first] = kv.second;
    } else {
      vals.push_back((unsigned long long)(uintptr_t)c->unit_src(kv.first) | 1ull);
      c->dev_table.erase(kv.first);
    }
  }
  c->tab_updates.clear();
  if (ids.empty()) return INFLLM_OK;
  return ptr_table_update_launch(c->d_unit_ptrs, ids.data(), vals.data(), (int)ids.size(), s);
}

// Apply the oldest pending retrieval of a one-token append to the cache: wait for its ids (they left the device
// right behind the scorer, long ago as a rule) and evict and refill as the reference does at that token.
int settle_one(infllm_ctx* c, cudaStream_t s) {
  if (c->pend_count <= 0) return INFLLM_OK;
  const infllm_config& g = c->cfg;
  infllm_ctx::PendingToken& p = c->pend[c->pend_head];
  {
    HostTimer ht(&c->host_us[0]);
    INFLLM_CUDA_OK(cudaEventSynchronize(p.ev));
  }
  std::vector<int32_t> ids(p.h_ids, p.h_ids + g.topk);
  // the units that token's attention did not find in a cache slot were read in place and sit in the landing slots
  c->settle_landing.assign(ids.size(), -1);
  for (size_t i = 0; i < ids.size(); ++i)
    if (std::find(p.listed.begin(), p.listed.end(), ids[i]) == p.listed.end()) {
      c->counters.inplace_units += 1;
      if (i < p.landing.size() && p.landing[i] >= 0 && c->landing_slots[i] == p.landing[i]) {
        c->settle_landing[i] = p.landing[i];
        c->landing_slots[i] = -1;  // handed to the unit; flush_table sets another slot aside
      }
    }
  c->pend_head = (c->pend_head + 1) % infllm_ctx::kPendSlots;
  c->pend_count -= 1;
  {
    HostTimer ht(&c->host_us[1]);
    INFLLM_TRY(plan_and_refill(c, ids, 0, s, PLAN_DECODE_ASYNC));
  }
  c->settle_landing.clear();
  if (p.serial == c->call_serial) c->trace_topk.push_back(ids);
  return INFLLM_OK;
}

int settle_all(infllm_ctx* c, cudaStream_t s) {
  while (c->pend_count > 0) INFLLM_TRY(settle_one(c, s));
  return INFLLM_OK;
}

// what sealing does after an exec block that ended at absolute token `end` (context_manager.py:614-679):
// `take` tokens go to the init sink, then `n_new` units are sealed; a pure function of the lengths
struct SealPlan {
  int64_t take = 0;
  int n_new = 0;
  int64_t new_frontier = 0;
};

SealPlan plan_seal(const infllm_ctx* c, int64_t end) {
  const infllm_config& g = c->cfg;
  SealPlan p;
  int64_t rem = end - c->frontier;
  if (!c->init_full && rem > g.n_local) {  // :628-646
    p.take = std::min<int64_t>(g.n_init - c->init_len, rem - g.n_local);
    rem -= p.take;
  }
  while (rem - g.block_size >= g.n_local) {  // :649
    rem -= g.block_size;
    ++p.n_new;
  }
  p.new_frontier = c->frontier + p.take + (int64_t)p.n_new * g.block_size;
  return p;
}

int seal_apply(infllm_ctx* c, const SealPlan& sp, cudaStream_t s) {
  const infllm_config& g = c->cfg;
  TokenBuffers& tb = c->tb;
  const int64_t D = g.head_dim, HKV = g.n_kv_heads, bs = g.block_size;
  if (sp.take > 0) {
    const size_t w = sp.take * D * c->esz;
    const int64_t src = (c->frontier - tb.t0) * D * c->esz, dst = c->init_len * D * c->esz;
    INFLLM_CUDA_OK(cudaMemcpy2DAsync((char*)c->init_k + dst, c->init_cap * D * c->esz, (char*)tb.k_raw + src,
                                     tb.cap * D * c->esz, w, HKV, cudaMemcpyDeviceToDevice, s));
    INFLLM_CUDA_OK(cudaMemcpy2DAsync((char*)c->init_v + dst, c->init_cap * D * c->esz, (char*)tb.v + src,
                                     tb.cap * D * c->esz, w, HKV, cudaMemcpyDeviceToDevice, s));
    c->init_len += sp.take;
    c->frontier += sp.take;
  }
  if (c->init_len == g.n_init) c->init_full = true;
  const int n_new = sp.n_new;
  if (n_new == 0) return INFLLM_OK;
  INFLLM_TRY(ensure_block_k(c, c->num_blocks + n_new, s));
  INFLLM_TRY(ensure_host_units(c, c->num_blocks + n_new));
  INFLLM_TRY(repr_select_launch(tb.k_raw, tb.cap * D, D, tb.score, tb.cap, c->frontier - tb.t0, n_new, (int)bs,
                                g.repr_topk, g.n_heads, g.n_kv_heads, (int)D,
                                (char*)c->block_k + c->num_blocks * c->width * c->esz, g.dtype, s));
  trace_mark(c, s, TR_REPR_END, c->num_blocks);
  c->num_blocks += n_new;
  c->frontier += n_new * bs;
  return INFLLM_OK;
}

// Pool of device memory for the device copies of the stores, one per device ordinal: filled by
// infllm_device_store_reserve (the only place that allocates), handed out in slabs of kPoolSlabBytes.
constexpr size_t kPoolSlabBytes = 128ull << 20;
struct DevicePool {
  std::mutex mu;
  std::vector<void*> free_slabs;
  int64_t total = 0, used = 0;  // slabs
};
DevicePool g_pool[64];

void* pool_take(int dev) {
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_pool[dev].mu);
  if (g_pool[dev].free_slabs.empty()) return nullptr;
  void* p = g_pool[dev].free_slabs.back();
  g_pool[dev].free_slabs.pop_back();
  g_pool[dev].used += 1;
  return p;
}

void pool_give(int dev, void* p) {
  if (dev < 0 || dev >= 64 || !p) return;
  std::lock_guard<std::mutex> lk(g_pool[dev].mu);
  g_pool[dev].free_slabs.push_back(p);
  g_pool[dev].used -= 1;
}

void release_dev_slabs(infllm_ctx* c) {
  for (void* p : c->dev_slabs) pool_give(c->cfg.device, p);
  c->dev_slabs.clear();
  c->dev_units = 0;
}

// device slabs for units [0, n): taken from the pool as the store grows; when the pool is empty the copy stops growing
int ensure_dev_units(infllm_ctx* c, int64_t n) {
  if ((size_t)(c->slab_units * c->unit_bytes) > kPoolSlabBytes) {
    c->dev_cap = c->dev_units;
    return INFLLM_E_NOMEM;
  }
  while ((int64_t)c->dev_slabs.size() * c->slab_units < n) {
    void* p = pool_take(c->cfg.device);
    if (!p) {
      c->dev_cap = c->dev_units;
      return INFLLM_E_NOMEM;
    }
    c->dev_slabs.push_back(p);
  }
  return INFLLM_OK;
}

// after the host store was filled by the host (synthetic load, restore from a file): the device copy of its head
int fill_dev_store(infllm_ctx* c, int64_t n_units) {
  const int64_t n = std::min(n_units, c->dev_cap);
  c->dev_units = 0;
  if (n <= 0 || ensure_dev_units(c, n) != INFLLM_OK) return INFLLM_OK;
  for (int64_t b0 = 0; b0 < n;) {
    const int64_t run = std::min(n - b0, c->slab_units - b0 % c->slab_units);
    INFLLM_CUDA_OK(cudaMemcpy(c->dev_unit(b0), c->host_unit(b0), (size_t)(run * c->unit_bytes), cudaMemcpyHostToDevice));
    b0 += run;
  }
  c->dev_units = n;
  return INFLLM_OK;
}

// second half of sealing: the new units' K/V go to the host store.  `first` is the id of the first new unit,
// `tok0` its first token (absolute); called after the units were counted in.
int seal_offload(infllm_ctx* c, int64_t first, int n_new, int64_t tok0, cudaStream_t s) {
  if (n_new <= 0) return INFLLM_OK;
  const infllm_config& g = c->cfg;
  TokenBuffers& tb = c->tb;
  const int64_t D = g.head_dim, HKV = g.n_kv_heads, bs = g.block_size;
  // offload to the host store (MemoryUnit.__init__, context_manager.py:39-45), entirely on the device-to-host
  // stream: pack the new units into the store's layout, then one copy per run of units.  The tokens were
  // final when they were ingested; ev_ingest orders the packing behind that.
  if (c->ingest_event_due) {
    INFLLM_CUDA_OK(cudaEventRecord(c->ev_ingest, s));
    c->ingest_event_due = false;
  }
  INFLLM_CUDA_OK(cudaStreamWaitEvent(c->d2h_stream, c->ev_ingest, 0));
  for (int done = 0; done < n_new;) {
    const int n = std::min(n_new - done, c->pack_units);
    const int r = c->pack_idx;
    c->pack_idx ^= 1;
    INFLLM_TRY(pack_units_launch(tb.k_raw, tb.v, tb.cap * D, tok0 + (int64_t)done * bs - tb.t0, n, (int)bs, (int)HKV,
                                 (int)D, c->pack_buf[r], c->d2h_stream));
    for (int i = 0; i < n;) {  // runs that stay inside one slab of the store are contiguous on the host
      const int64_t b0 = first + done + i;
      const int run = (int)std::min<int64_t>(n - i, c->slab_units - b0 % c->slab_units);
      INFLLM_CUDA_OK(cudaMemcpyAsync(c->host_unit(b0), (char*)c->pack_buf[r] + (int64_t)i * c->unit_bytes,
                                     (int64_t)run * c->unit_bytes, cudaMemcpyDeviceToHost, c->d2h_stream));
      // the device copy of the store grows with the same runs while it has room (readers order themselves behind
      // ev_d2h exactly as they do for the host copy)
      if (b0 == c->dev_units && b0 + run <= c->dev_cap && ensure_dev_units(c, b0 + run) == INFLLM_OK) {
        INFLLM_CUDA_OK(cudaMemcpyAsync(c->dev_unit(b0), (char*)c->pack_buf[r] + (int64_t)i * c->unit_bytes,
                                       (int64_t)run * c->unit_bytes, cudaMemcpyDeviceToDevice, c->d2h_stream));
        c->dev_units = b0 + run;
      }
      i += run;
    }
    c->counters.d2h_bytes += (int64_t)n * c->unit_bytes;
    done += n;
  }
  INFLLM_CUDA_OK(cudaEventRecord(c->ev_d2h, c->d2h_stream));
  c->d2h_recorded = true;
  trace_mark(c, c->d2h_stream, TR_PACK_END, first);
  (void)s;
  return INFLLM_OK;
}

// column sums of the local stage for the window keys [j_begin, j_end) (indices relative to the window start ks),
// added into the score buffer; `work` is the FLOP count attributed to this launch
int local_scores(infllm_ctx* c, cudaStream_t s, int64_t st, int64_t ks, int64_t lq, int64_t lk, int64_t j_begin,
                 int64_t j_end, double work) {
  if (j_end <= j_begin) return INFLLM_OK;
  const infllm_config& g = c->cfg;
  TokenBuffers& tb = c->tb;
  const int64_t D = g.head_dim, H = g.n_heads, HKV = g.n_kv_heads;
  const int64_t n = j_end - j_begin, tok = ks - tb.t0 + j_begin, off = (lk - lq) - j_begin;
  ProfScope ps(c, s, INFLLM_PROF_COLSUM, work);
  if (c->use_tc && lq > 64 && lq <= 512)
    return colsum_tc_launch_maps(c->m_qloc, c->m_krot, (int)st, (int)tok, (int)H, (int)HKV, lq, n, INFLLM_MASK_WINDOW,
                                 off, g.n_local, c->lse, tb.score + tok, tb.cap, 1, g.dtype, s);
  return attn_colsum_launch((const char*)c->q_loc + st * D * c->esz, c->sub_max * D, D,
                            (char*)tb.k_rot + tok * D * c->esz, tb.cap * D, D, (int)H, (int)HKV, lq, n, (int)D,
                            INFLLM_MASK_WINDOW, off, g.n_local, c->lse, tb.score + tok, tb.cap, 1, g.dtype, s);
}

// lru-s (context_manager.py:454-470): every cached unit's score decays, and each retrieved unit gains the attention
// mass its keys received from this exec block's queries, summed over heads.  The host needs the sums before it plans
// the next exec block, as in the reference (a blocking copy there too).
int unit_score_update(infllm_ctx* c, const std::vector<int32_t>& ids, const char* qglb, int64_t lq, cudaStream_t s) {
  const infllm_config& g = c->cfg;
  const int64_t D = g.head_dim, H = g.n_heads, HKV = g.n_kv_heads, bs = g.block_size;
  const int64_t cols = (int64_t)g.topk * bs, n = (int64_t)ids.size();
  if (!c->unit_prob) {
    INFLLM_CUDA_OK(cudaMalloc((void**)&c->unit_prob, H * cols * sizeof(float)));
    INFLLM_CUDA_OK(cudaHostAlloc((void**)&c->h_unit_prob, H * cols * sizeof(float), cudaHostAllocDefault));
  }
  for (int64_t i = 0; i < n; ++i) {
    const char* base = (const char*)c->cache + (int64_t)c->slot_of[ids[i]] * c->unit_bytes;
    INFLLM_TRY(attn_colsum_launch(qglb, c->sub_max * D, D, base, bs * D, D, (int)H, (int)HKV, lq, bs, (int)D,
                                  INFLLM_MASK_NONE, 0, 0, c->lse, c->unit_prob + i * bs, cols, 0, g.dtype, s));
  }
  INFLLM_CUDA_OK(cudaMemcpy2DAsync(c->h_unit_prob, n * bs * sizeof(float), c->unit_prob, cols * sizeof(float),
                                   n * bs * sizeof(float), H, cudaMemcpyDeviceToHost, s));
  INFLLM_CUDA_OK(cudaStreamSynchronize(s));
  c->lru.scale(g.score_decay);
  for (int64_t i = 0; i < n; ++i) {
    float sum = 0.f;  // the reference sums in fp32: over a unit's keys, then over the heads
    for (int64_t h = 0; h < H; ++h) {
      float row = 0.f;
      for (int64_t j = 0; j < bs; ++j) row += c->h_unit_prob[(h * n + i) * bs + j];
      sum += row;
    }
    c->lru.add(ids[i], (double)sum);
  }
  return INFLLM_OK;
}

// one internal call of at most sub_max tokens whose exec-block boundaries coincide with the caller's
int append_sub(infllm_ctx* c, const char* q, int64_t q_hs, int64_t q_ts, const char* k, int64_t k_hs, int64_t k_ts,
               const char* v, int64_t v_hs, int64_t v_ts, char* out, int64_t o_hs, int64_t o_ts, int64_t L,
               cudaStream_t s) {
  const infllm_config& g = c->cfg;
  const int64_t D = g.head_dim, H = g.n_heads, HKV = g.n_kv_heads, bs = g.block_size;
  const int esz = c->esz;
  const int64_t T = c->length;
  INFLLM_TRY(ensure_tokens(c, L, s));
  TokenBuffers& tb = c->tb;
  const int64_t kv_hs = tb.cap * D;  // head stride of the token buffers, elements
  // ---- ingest the new tokens
  const int64_t at = T - tb.t0;
  const int64_t q_hs_s = c->sub_max * D;
  if (c->use_tc) {
    // a 128-row tile that ends the window may reach past the last ingested token: keep those rows finite.
    // Rows are zeroed well ahead of the data so that token-by-token appends rarely pay for it.
    if (tb.zero_upto < std::min<int64_t>(tb.cap, at + L + 128)) {
      const int64_t upto = std::min<int64_t>(tb.cap, at + L + 128 + 4096), pad = upto - (at + L);
      INFLLM_CUDA_OK(cudaMemset2DAsync((char*)tb.v + (at + L) * D * esz, kv_hs * esz, 0, pad * D * esz, HKV, s));
      INFLLM_CUDA_OK(cudaMemset2DAsync((char*)tb.k_rot + (at + L) * D * esz, kv_hs * esz, 0, pad * D * esz, HKV, s));
      INFLLM_CUDA_OK(cudaMemset2DAsync((char*)tb.k_raw + (at + L) * D * esz, kv_hs * esz, 0, pad * D * esz, HKV, s));
      tb.zero_upto = upto;
    }
  }
  // RoPE: keys keep the position (token - rope_origin) until the table would run out
  const int64_t win0 = std::max<int64_t>(T - g.n_local, 0);  // oldest key any query of this call can see locally
  if (c->rope_origin < 0 || T + L - c->rope_origin > c->tab_len || win0 < c->rope_origin) {
    c->rope_origin = win0;
    if (T > win0)
      INFLLM_TRY(rope_apply_launch((char*)tb.k_raw + (win0 - tb.t0) * D * esz, kv_hs, D,
                                   (char*)tb.k_rot + (win0 - tb.t0) * D * esz, kv_hs, D, (int)HKV, T - win0, (int)D,
                                   c->cos_t, c->sin_t, c->tab_len, 0, 1, g.dtype, s));
  }
  if (L == 1) {
    // one token: copies, the three rotations, the query mean and the cleared score column in one launch
    INFLLM_TRY(ingest_token_launch(q, q_hs, k, k_hs, v, v_hs, c->q_loc, c->q_glb, q_hs_s, c->qbar,
                                   (char*)tb.k_raw + at * D * esz, (char*)tb.k_rot + at * D * esz,
                                   (char*)tb.v + at * D * esz, kv_hs, tb.score + at, tb.cap, (int)H, (int)HKV, (int)D,
                                   c->cos_t, c->sin_t, c->tab_len, T - c->rope_origin, g.n_local - 1, g.dtype, s,
                                   c->d_miss));
    c->ingest_event_due = true;  // recorded when a sealing asks for it (seal_offload): one call less per token
  } else {
    INFLLM_TRY(copy_rows_launch(k, k_hs, k_ts, (char*)tb.k_raw + at * D * esz, kv_hs, D, (int)HKV, L, (int)D, s));
    INFLLM_TRY(copy_rows_launch(v, v_hs, v_ts, (char*)tb.v + at * D * esz, kv_hs, D, (int)HKV, L, (int)D, s));
    INFLLM_CUDA_OK(cudaEventRecord(c->ev_ingest, s));
    c->ingest_event_due = false;
    INFLLM_CUDA_OK(cudaMemset2DAsync(tb.score + at, tb.cap * sizeof(float), 0, L * sizeof(float), H, s));
    INFLLM_TRY(rope_apply_launch((char*)tb.k_raw + at * D * esz, kv_hs, D, (char*)tb.k_rot + at * D * esz, kv_hs, D,
                                 (int)HKV, L, (int)D, c->cos_t, c->sin_t, c->tab_len, T - c->rope_origin, 1, g.dtype,
                                 s));
    // queries: window-relative rotation for the local stage, the single position n_local-1 for the
    // global stage (context_manager.py:480 and :744-747)
    INFLLM_TRY(rope_apply_launch(q, q_hs, q_ts, c->q_loc, q_hs_s, D, (int)H, L, (int)D, c->cos_t, c->sin_t, c->tab_len,
                                 T - c->rope_origin, 1, g.dtype, s));
    INFLLM_TRY(rope_apply_launch(q, q_hs, q_ts, c->q_glb, q_hs_s, D, (int)H, L, (int)D, c->cos_t, c->sin_t, c->tab_len,
                                 g.n_local - 1, 0, g.dtype, s));
    INFLLM_TRY(qbar_launch(c->q_glb, q_hs_s, D, (int)H, L, g.exc_block_size, (int)D, c->qbar, c->width, g.dtype, s));
  }

  // one-token appends whose retrieval has not been applied to the cache yet: a call that is not itself such a token
  // needs the cache as the reference would have it
  const bool run_ahead = L == 1 && D == 128 && c->num_blocks > g.topk && g.topk <= kMaxSeg - 4 && !(g.debug_flags & 16) &&
                         g.chunk_topk_calc == 0 && g.cache_strategy == INFLLM_CACHE_LRU;
  if (!run_ahead) INFLLM_TRY(settle_all(c, s));
  if (L > 1) {  // units a previous one-token append fetched ahead are not wanted by a prefill's look-ahead
    for (auto it = c->staged.begin(); it != c->staged.end();) {
      if (c->staged_for[it->first] == INT64_MAX) {
        c->free_slots.push_back(it->second);
        c->staged_for.erase(it->first);
        it = c->staged.erase(it);
      } else {
        ++it;
      }
    }
    // the slots set aside for one-token attentions to deposit in go back to the pool
    for (int slot : c->landing_slots)
      if (slot >= 0) c->free_slots.push_back(slot);
    c->landing_slots.clear();
    c->landing_listed.clear();
    c->table_valid = false;
  }
  std::vector<int32_t> ids;
  for (auto& l : c->la) l.target = -1, l.launched = l.staged = false;
  if (L > 1) INFLLM_CUDA_OK(cudaEventRecord(c->ev_seal, s));  // the look-ahead's starting point; one token has none
  std::vector<KvSeg> gsegs;
  int eb = 0, n_cand = 0;
  bool have_ids = false;  // the ids of this exec block were already ranked at the end of the previous one
  for (int64_t st = 0; st < L; st += g.exc_block_size, ++eb) {  // context_manager.py:762
    const int64_t ed = std::min<int64_t>(st + g.exc_block_size, L);
    const int64_t S = T + st, E = T + ed, lq = ed - st;
    const int64_t ks = std::max<int64_t>(S - g.n_local, 0), lk = E - ks;  // local keys [ks, E) (:772-773)
    // One-token exec blocks over more units than a retrieval takes run ahead of the host: the attention is launched
    // right behind the top-k kernel and finds the retrieved units through the device table of unit addresses —
    // in their cache slots, or in place in the store when they are not (yet) cached — so neither the GPU nor the
    // host waits for the other.  The ids reach the host on the mail stream and are applied to the LRU order when
    // one of the next tokens arrives (settle_one): same evictions and refills as the reference, one or two tokens
    // later in wall-clock time.
    if (c->chunk_mode) {
      const int64_t chunk = (int64_t)(g.chunk_topk_calc / g.exc_block_size) * g.exc_block_size;
      if ((c->call_off + st) % chunk == 0) c->chunk_n0 = c->num_blocks;
    }
    const bool spec = run_ahead;
    const bool ids_direct = !c->comm && g.topk <= 64 && c->num_blocks <= 16384;  // the scorer's one-launch form
    cudaEvent_t token_ev = nullptr;
    int32_t* d_ids_tok = nullptr;  // the device-side ids of a run-ahead token
    if (!spec) {
      if (!have_ids) {
        HostTimer ht(&c->host_us[0]);
        INFLLM_TRY(retrieve_now(c, eb, &ids, s));
      }
      {
        HostTimer ht(&c->host_us[1]);
        INFLLM_TRY(plan_and_refill(c, ids, eb, s, L == 1 ? PLAN_DECODE_SYNC : PLAN_PREFILL));
      }
      c->trace_topk.push_back(ids);
    } else {
      ids.clear();
      // at most kMaxOutstanding tokens ahead of the cache: apply the older retrievals first
      while (c->pend_count >= infllm_ctx::kMaxOutstanding) INFLLM_TRY(settle_one(c, s));
      INFLLM_TRY(ensure_scores(c, c->num_blocks, s));
      const int slot = (c->pend_head + c->pend_count) % infllm_ctx::kPendSlots;
      infllm_ctx::PendingToken& pt = c->pend[slot];
      d_ids_tok = c->d_topk_ring + (int64_t)slot * std::max(1, g.topk);
      {
        ProfScope ps(c, s, INFLLM_PROF_TOPK, (double)c->num_blocks * c->width * c->esz);
        INFLLM_TRY(score_topk(c, c->num_blocks, c->qbar, c->scores, d_ids_tok, s, 0, g.topk, ids_direct ? pt.h_ids : nullptr));
      }
      if (ids_direct) {
        // the ranking threads wrote the ids into the pinned words themselves; the event that tells the host so is
        // recorded behind the token's last kernel, so that nothing stands between the kernels of the chain
        token_ev = pt.ev;
      } else {
        INFLLM_CUDA_OK(cudaEventRecord(c->ev_main, s));
        INFLLM_CUDA_OK(cudaStreamWaitEvent(c->mail_stream, c->ev_main, 0));
        INFLLM_CUDA_OK(cudaMemcpyAsync(pt.h_ids, d_ids_tok, g.topk * sizeof(int32_t), cudaMemcpyDeviceToHost, c->mail_stream));
        INFLLM_CUDA_OK(cudaEventRecord(pt.ev, c->mail_stream));
      }
      pt.serial = c->call_serial;
      c->pend_count += 1;
      INFLLM_TRY(flush_table(c, s));
      pt.listed.clear();
      for (auto& kv : c->dev_table) pt.listed.push_back(kv.first);
      pt.landing = c->landing_slots;
    }
    // bit 1 of the flags turns the look-ahead off; a chunk's retrievals are fixed when it starts, so they need none
    const bool more = ed < L && !(g.debug_flags & 2) && !c->chunk_mode;
    const int64_t n_eb = (L + g.exc_block_size - 1) / g.exc_block_size;
    HostTimer* ht_attn = new HostTimer(&c->host_us[3]);
    trace_mark(c, s, TR_ATTN_BEGIN, eb);
    const int64_t ovf = std::max<int64_t>(E - c->frontier - g.n_local, 0);  // :391
    // global key segments: retrieved units (in place in their cache slots), sink, overflow
    gsegs.clear();
    if (spec)  // resolved on the device
      for (int i = 0; i < g.topk; ++i) gsegs.push_back({nullptr, nullptr, bs * D, (int32_t)D, (int32_t)bs});
    for (int32_t b : ids) {
      const char* base = (const char*)c->cache + (int64_t)c->slot_of[b] * c->unit_bytes;
      gsegs.push_back({base, base + c->unit_bytes / 2, bs * D, (int32_t)D, (int32_t)bs});
    }
    if (c->init_len > 0) gsegs.push_back({c->init_k, c->init_v, c->init_cap * D, (int32_t)D, (int32_t)c->init_len});
    if (ovf > 0)
      gsegs.push_back({(char*)tb.k_raw + (c->frontier - tb.t0) * D * esz, (char*)tb.v + (c->frontier - tb.t0) * D * esz,
                       kv_hs, (int32_t)D, (int32_t)ovf});
    char* out_eb = out + st * o_ts * esz;
    const char* qloc_eb = (const char*)c->q_loc + st * D * esz;
    const char* qglb_eb = (const char*)c->q_glb + st * D * esz;
    const bool decode_path = lq == 1 && D == 128;
    double local_pairs_eb = 0;
    if (decode_path) {
      // ---- one-token exec block: split-K decode over [visible window | global segments]
      const int64_t wlo = std::max<int64_t>(E - g.n_local, ks);  // window mask of the single query
      std::vector<KvSeg> segs;
      std::vector<int32_t> qsel;
      segs.push_back({(char*)tb.k_rot + (wlo - tb.t0) * D * esz, (char*)tb.v + (wlo - tb.t0) * D * esz, kv_hs,
                      (int32_t)D, (int32_t)(E - wlo)});
      qsel.push_back(0);
      for (auto& sgm : gsegs) {
        segs.push_back(sgm);
        qsel.push_back(1);
      }
      int parts = 0;
      double dec_keys = 0;
      for (auto& sgm : segs) dec_keys += sgm.len;
      if (segs.size() > (size_t)kMaxSeg)
        return fail(INFLLM_E_UNSUPPORTED, "decode: %zu key segments exceed %d", segs.size(), kMaxSeg);
      DecodeIndirect ind;
      if (spec) {  // the retrieved units are named on the device and found through the table of unit addresses
        ind.ids = d_ids_tok;
        ind.ptrs = c->d_unit_ptrs;
        ind.unit_bytes = c->unit_bytes;
        ind.n_units = g.topk;
        ind.first_seg = 1;
        ind.landing = c->d_unit_ptrs + c->tab_cap;
        ind.early_rest = 1;  // behind the scorer or the table update: neither writes what the window and the sink need
      }
      {
        // the merge also adds this token's local attention row into the accumulated scores
        ProfScope ps(c, s, INFLLM_PROF_DECODE, dec_keys * HKV * D * 2 * esz);
        INFLLM_TRY(attn_decode_launch(qloc_eb, qglb_eb, q_hs_s, (int)H, (int)HKV, (int)D, (int)segs.size(), segs.data(),
                                      qsel.data(), c->part_o, c->part_lse, c->max_parts, &parts, 0, c->dec_logits,
                                      g.dtype, s, spec ? &ind : nullptr));
        INFLLM_TRY(lse_merge_launch(c->part_o, c->part_lse, parts, (int)H, (int)D, out_eb, o_hs, c->lse, g.dtype, s,
                                    c->dec_logits, E - wlo, tb.score + (wlo - tb.t0), tb.cap, nullptr));
      }
    } else {
      // ---- local stage + global stage, jointly normalised (context_manager.py:486-489, 526-533)
      double local_pairs = 0, all_glk = 0;
      for (int64_t i = 0; i < lq; ++i) local_pairs += (double)std::min<int64_t>(S + i + 1, g.n_local);
      for (auto& sgm : gsegs) all_glk += sgm.len;
      local_pairs_eb = local_pairs;
      const bool tc_now = c->use_tc && lq > 64 && gsegs.size() + 1 <= (size_t)kMaxSeg;
      if (tc_now) {
        AttnTcParams TP{};
        TP.maps[0] = c->m_qloc; TP.maps[1] = c->m_qglb; TP.maps[2] = c->m_krot; TP.maps[3] = c->m_kraw;
        TP.maps[4] = c->m_v; TP.maps[5] = c->m_cache; TP.maps[6] = c->m_initk; TP.maps[7] = c->m_initv;
        TP.n_stage = 2; TP.n_heads = (int)H; TP.n_kv_heads = (int)HKV; TP.lq = lq;
        TP.out = out_eb; TP.o_hs = o_hs; TP.o_ts = o_ts; TP.lse = c->lse;
        TP.scale_log2 = kLog2e / sqrtf((float)D); TP.err = c->tc_err;
        TP.stage[0].map_q = 0; TP.stage[0].q_row0 = (int)st; TP.stage[0].mask_mode = INFLLM_MASK_WINDOW;
        TP.stage[0].mask_offset = lk - lq; TP.stage[0].mask_size = g.n_local; TP.stage[0].lk = lk;
        TP.stage[0].seg_begin = 0; TP.stage[0].seg_end = 1;
        TP.seg[0] = {2, 4, (int32_t)(ks - tb.t0), -1, -1, (int32_t)lk};
        int ns = 1;
        // The reference passes a complement window for the global stage whose offset makes every
        // (query, key) pair visible (context_manager.py:437); the stage is therefore unmasked.
        for (int32_t b : ids) {
          const int slot = c->slot_of[b];
          TP.seg[ns++] = {5, 5, 0, slot * 2, slot * 2 + 1, (int32_t)bs};
        }
        if (c->init_len > 0) TP.seg[ns++] = {6, 7, 0, -1, -1, (int32_t)c->init_len};
        if (ovf > 0) TP.seg[ns++] = {3, 4, (int32_t)(c->frontier - tb.t0), -1, -1, (int32_t)ovf};
        TP.stage[1].map_q = 1; TP.stage[1].q_row0 = (int)st; TP.stage[1].mask_mode = INFLLM_MASK_NONE;
        TP.stage[1].lk = (int64_t)all_glk; TP.stage[1].seg_begin = 1; TP.stage[1].seg_end = ns;
        ProfScope ps(c, s, INFLLM_PROF_ATTN, 4.0 * D * H * (local_pairs + (double)lq * all_glk));
        // The one-head kernel runs one CTA per (128-query tile, head): with few heads on this GPU (a KV-head-group
        // shard) its grid leaves most SMs idle, and the two-head kernel, which also cuts the key tiles into runs,
        // fills them.  Flag bit 3 forces the two-head kernel.
        const bool few_ctas = lq >= 256 && ((lq + 127) / 128) * H <= 74;
        if ((H / HKV) % 2 == 0 && ((g.debug_flags & 8) || few_ctas)) {
          // two heads of a KV head per CTA; cut the key tiles into runs until the grid covers the SMs
          const int items = (int)((lq + 127) / 128) * (int)(H / 2);
          TP.n_split = std::max(1, std::min(8, 148 / items));
          const size_t need = attn_tc2_scratch_floats(TP.n_split, (int)H, lq);
          if (need > c->tc_part_floats) {
            if (c->tc_part) INFLLM_CUDA_OK(cudaFreeAsync(c->tc_part, s));
            INFLLM_CUDA_OK(cudaMallocAsync((void**)&c->tc_part, need * sizeof(float), s));
            c->tc_part_floats = need;
          }
          if (TP.n_split > 1) {
            TP.part_acc = c->tc_part;
            TP.part_m = c->tc_part + (size_t)TP.n_split * H * lq * 128;
            TP.part_l = TP.part_m + (size_t)TP.n_split * H * lq;
          }
          INFLLM_TRY(attn_tc2_launch(TP, g.dtype, s));
        } else {
          TP.n_split = 1;
          INFLLM_TRY(attn_tc3_launch(TP, g.dtype, s));
        }
      } else {
      AttnParams P{};
      P.n_heads = (int)H; P.n_kv_heads = (int)HKV; P.lq = lq; P.first = 1;
      P.acc = c->st_acc; P.m = c->st_m; P.l = c->st_l;
      P.out = out_eb; P.o_hs = o_hs; P.o_ts = o_ts; P.lse = c->lse;
      P.scale_log2 = kLog2e / sqrtf((float)D);
      P.stage[0].q = qloc_eb; P.stage[0].q_hs = q_hs_s; P.stage[0].q_ts = D;
      P.stage[0].mask_mode = INFLLM_MASK_WINDOW; P.stage[0].mask_offset = lk - lq; P.stage[0].mask_size = g.n_local;
      P.stage[0].lk = lk; P.stage[0].seg_begin = 0; P.stage[0].seg_end = 1;
      P.seg[0] = {(char*)tb.k_rot + (ks - tb.t0) * D * esz, (char*)tb.v + (ks - tb.t0) * D * esz, kv_hs, (int32_t)D,
                  (int32_t)lk};
      size_t done = 0;
      int nseg = 1;
      int64_t glk = 0;
      while (done < gsegs.size() && nseg < kMaxSeg) {
        P.seg[nseg++] = gsegs[done];
        glk += gsegs[done].len;
        ++done;
      }
      P.n_stage = 2;
      P.stage[1].q = qglb_eb; P.stage[1].q_hs = q_hs_s; P.stage[1].q_ts = D;
      P.stage[1].mask_mode = INFLLM_MASK_NONE; P.stage[1].lk = glk; P.stage[1].seg_begin = 1; P.stage[1].seg_end = nseg;
      P.last = done == gsegs.size();
      {
        ProfScope ps(c, s, INFLLM_PROF_ATTN, 4.0 * D * H * (local_pairs + (double)lq * all_glk));
        INFLLM_TRY(attn_general_launch(P, (int)D, g.dtype, s));
      }
      while (done < gsegs.size()) {  // more segments than one launch holds: carry the state
        AttnParams R{};
        R.n_heads = (int)H; R.n_kv_heads = (int)HKV; R.lq = lq; R.first = 0;
        R.acc = c->st_acc; R.m = c->st_m; R.l = c->st_l;
        R.out = out_eb; R.o_hs = o_hs; R.o_ts = o_ts; R.lse = c->lse; R.scale_log2 = P.scale_log2;
        R.n_stage = 1;
        R.stage[0].q = qglb_eb; R.stage[0].q_hs = q_hs_s; R.stage[0].q_ts = D; R.stage[0].mask_mode = INFLLM_MASK_NONE;
        int ns = 0;
        int64_t rl = 0;
        while (done < gsegs.size() && ns < kMaxSeg) {
          R.seg[ns++] = gsegs[done];
          rl += gsegs[done].len;
          ++done;
        }
        R.stage[0].lk = rl; R.stage[0].seg_begin = 0; R.stage[0].seg_end = ns;
        R.last = done == gsegs.size();
        ProfScope ps(c, s, INFLLM_PROF_ATTN, 0.0);
        INFLLM_TRY(attn_general_launch(R, (int)D, g.dtype, s));
      }
      }
    }
    if (g.cache_strategy == INFLLM_CACHE_LRU_S && !ids.empty()) INFLLM_TRY(unit_score_update(c, ids, qglb_eb, lq, s));
    // ev_attn: behind this exec block's attention; ev_attn_prev: behind the previous one's
    std::swap(c->ev_attn, c->ev_attn_prev);
    c->attn_prev_recorded = c->attn_recorded;
    INFLLM_CUDA_OK(cudaEventRecord(c->ev_attn, s));
    c->attn_recorded = true;
    if (token_ev) INFLLM_CUDA_OK(cudaEventRecord(token_ev, s));
    delete ht_attn;
    trace_mark(c, s, TR_ATTN_END, eb);
    // the look-ahead of the next exec blocks goes out behind the attention launch: it runs on its own stream and
    // the attention is what the main stream waits for
    if (more) {
      HostTimer ht(&c->host_us[2]);
      for (int d = 1; d <= c->look_depth; ++d) {
        const int64_t tgt = eb + d;
        infllm_ctx::LookAhead& la = c->la[tgt % (c->look_depth + 1)];
        if (tgt < n_eb && !(la.launched && la.target == tgt)) INFLLM_TRY(lookahead_launch(c, tgt, s));
      }
    }

    const SealPlan sp = plan_seal(c, E);
    // accumulated local score of every window key (context_manager.py:488, 623-625).  Sealing only needs
    // the scores of the tokens it is about to seal, so their 128-key tiles go first; the rest of the
    // window follows behind the sealing and overlaps the host's cache planning for the next exec block.
    int64_t j_u = 0;
    if (!decode_path) {
      j_u = std::min<int64_t>(lk, std::max<int64_t>(sp.new_frontier - ks, 0));
      j_u = std::min<int64_t>(lk, (j_u + 127) / 128 * 128);
      if (!more) j_u = lk;  // nothing to overlap with: one launch
      INFLLM_TRY(local_scores(c, s, st, ks, lq, lk, 0, j_u, local_pairs_eb));
    }
    trace_mark(c, s, TR_URGENT_END, eb);
    if (more) {
      HostTimer ht(&c->host_us[4]);
      for (int d = 1; d <= c->look_depth; ++d) {
        const int64_t tgt = eb + d;
        infllm_ctx::LookAhead& la = c->la[tgt % (c->look_depth + 1)];
        if (tgt < n_eb && la.launched && la.target == tgt && !la.staged) INFLLM_TRY(lookahead_stage(c, tgt));
      }
    }
    const int64_t first_new = c->num_blocks, tok_new = c->frontier + sp.take;
    {
      HostTimer ht(&c->host_us[5]);
      INFLLM_TRY(seal_apply(c, sp, s));
      if (more) INFLLM_CUDA_OK(cudaEventRecord(c->ev_seal, s));
    }
    if (more) INFLLM_TRY(candidates_launch(c, eb + 1, &n_cand, s));
    trace_mark(c, s, TR_SEAL_END, eb);
    INFLLM_TRY(seal_offload(c, first_new, sp.n_new, tok_new, s));  // off the ranking's critical path
    if (L == 1 && sp.n_new > 0) {
      // a one-token attention finds a unit through the table of unit addresses: the new units are listed at their
      // place in the store, which the copy-out must have reached first (once per block_size tokens)
      INFLLM_CUDA_OK(cudaStreamWaitEvent(s, c->ev_d2h, 0));
      c->d2h_synced_upto = c->d2h_synced_upto_urgent = c->num_blocks;
      for (int64_t b = first_new; b < c->num_blocks; ++b) c->tab_updates[(int32_t)b] = -1;
    }
    if (!decode_path) INFLLM_TRY(local_scores(c, s, st, ks, lq, lk, j_u, lk, 0.0));
    trace_mark(c, s, TR_REST_END, eb);
    have_ids = false;
    if (more) {
      HostTimer ht(&c->host_us[6]);
      INFLLM_TRY(candidates_finish(c, n_cand, &ids));
      have_ids = true;
    }
  }
  c->length += L;
  c->counters.exec_blocks += eb;
  return INFLLM_OK;
}

}  // namespace

extern "C" int infllm_ctx_create(const infllm_config* cfg, infllm_ctx** out) {
  if (!cfg || !out) return fail(INFLLM_E_BADARG, "ctx_create: null pointer");
  const infllm_config& g = *cfg;
  if (g.n_heads <= 0 || g.n_kv_heads <= 0 || g.n_heads % g.n_kv_heads)
    return fail(INFLLM_E_BADARG, "ctx_create: %d heads / %d kv heads", g.n_heads, g.n_kv_heads);
  if (g.head_dim != 128 && g.head_dim != 64)
    return fail(INFLLM_E_UNSUPPORTED, "ctx_create: head_dim %d (64 and 128 are built)", g.head_dim);
  if (g.n_init < 0 || g.n_local <= 0 || g.block_size <= 0 || g.topk <= 0 || g.exc_block_size <= 0 || g.repr_topk <= 0)
    return fail(INFLLM_E_BADARG, "ctx_create: sizes must be positive");
  if (g.exc_block_size > g.n_local)  // context_manager.py:219
    return fail(INFLLM_E_BADARG, "ctx_create: exc_block_size %d > n_local %d", g.exc_block_size, g.n_local);
  if (g.max_cached_block < g.topk)  // CudaCache.alloc would assert (context_manager.py:19)
    return fail(INFLLM_E_CAPACITY, "ctx_create: max_cached_block %d < topk %d: a retrieval could not be held in the cache",
                g.max_cached_block, g.topk);
  if (g.repr_topk > g.block_size) return fail(INFLLM_E_BADARG, "ctx_create: repr_topk %d > block_size %d", g.repr_topk, g.block_size);
  if (g.block_size % 8) return fail(INFLLM_E_BADARG, "ctx_create: block_size %d must be a multiple of 8", g.block_size);
  if (g.dtype != INFLLM_BF16 && g.dtype != INFLLM_FP16) return fail(INFLLM_E_UNSUPPORTED, "ctx_create: dtype code %d", g.dtype);
  if (g.cache_strategy != INFLLM_CACHE_LRU && g.cache_strategy != INFLLM_CACHE_LRU_S)
    return fail(INFLLM_E_UNSUPPORTED, "ctx_create: cache strategy code %d", g.cache_strategy);
  if (g.topk > 1024) return fail(INFLLM_E_UNSUPPORTED, "ctx_create: topk %d > 1024", g.topk);
  if (g.chunk_topk_calc != 0 && g.chunk_topk_calc < g.exc_block_size)
    return fail(INFLLM_E_BADARG, "ctx_create: chunk_topk_calc %d < exc_block_size %d", g.chunk_topk_calc, g.exc_block_size);
  infllm_ctx* c = new (std::nothrow) infllm_ctx();
  if (!c) return fail(INFLLM_E_NOMEM, "ctx_create: out of host memory");
  c->cfg = g;
  // lru-s: the cache plan of an exec block depends on the attention of the one before it (context_manager.py:
  // 454-470), so nothing is ranked, staged or attended ahead of the host
  if (g.cache_strategy == INFLLM_CACHE_LRU_S) c->cfg.debug_flags |= 2 | 16 | 32;
  c->esz = 2;
  c->width = (int64_t)g.n_heads * g.head_dim;
  c->unit_elems = (int64_t)g.n_kv_heads * g.block_size * g.head_dim;
  c->unit_bytes = 2 * c->unit_elems * c->esz;
  c->lru = LruTable(g.max_cached_block);
  if (g.look_depth > 0) c->look_depth = std::min<int>(g.look_depth, infllm_ctx::kMaxLookDepth);
  *out = c;
  return INFLLM_OK;
}

extern "C" int infllm_ctx_reset(infllm_ctx* c) {
  if (!c) return fail(INFLLM_E_BADARG, "ctx_reset: null context");
  if (c->initialized) {
    INFLLM_CUDA_OK(cudaSetDevice(c->cfg.device));
    INFLLM_CUDA_OK(cudaStreamSynchronize(c->copy_stream));
    INFLLM_CUDA_OK(cudaStreamSynchronize(c->urgent_stream));
    INFLLM_CUDA_OK(cudaStreamSynchronize(c->aux_stream));
    INFLLM_CUDA_OK(cudaStreamSynchronize(c->d2h_stream));
    INFLLM_CUDA_OK(cudaStreamSynchronize(c->mail_stream));
  }
  c->pend_head = c->pend_count = 0;  // retrievals not yet applied belong to the tokens that are forgotten
  c->landing_slots.clear();
  c->landing_listed.clear();
  c->d2h_synced_upto = 0;
  c->d2h_synced_upto_urgent = 0;
  release_dev_slabs(c);
  c->dev_cap = (int64_t)c->cfg.device_store_mb * (1ll << 20) / std::max<int64_t>(c->unit_bytes, 1);
  c->d2h_recorded = false;
  c->pack_used[0] = c->pack_used[1] = false;
  c->length = c->frontier = c->num_blocks = c->init_len = c->load_count = 0;
  c->init_full = false;
  c->rope_origin = -1;
  c->tb.t0 = 0;
  c->lru.clear();
  c->slot_of.clear();
  c->table_valid = false;
  c->tab_updates.clear();
  c->dev_table.clear();
  c->free_slots.clear();
  for (int i = c->cfg.max_cached_block + c->look_depth * c->cfg.topk - 1; i >= 0; --i) c->free_slots.push_back(i);
  c->staged.clear();
  c->staged_for.clear();
  for (auto& l : c->la) l.target = -1, l.launched = l.staged = false;
  c->staged_pending = false;
  c->trace_topk.clear();
  c->attn_recorded = false;
  c->attn_prev_recorded = false;
  c->spec_recorded = false;
  c->counters = infllm_ctx_info{};
  return INFLLM_OK;
}

extern "C" int infllm_ctx_destroy(infllm_ctx* c) {
  if (!c) return INFLLM_OK;
  if (c->initialized) {
    cudaSetDevice(c->cfg.device);
    cudaDeviceSynchronize();
    free_buffers(c->tb, nullptr);
    void* dev[] = {c->init_k, c->init_v, c->cos_t, c->sin_t, c->q_loc, c->q_glb, c->qbar, c->lse, c->st_acc, c->st_m,
                   c->st_l, c->d_topk, c->tickets, c->d_miss, c->part_o, c->part_lse, c->dec_logits, c->cache};
    for (void* p : dev)
      if (p) cudaFree(p);
    if (c->block_k) cudaFreeAsync(c->block_k, nullptr);
    if (c->scores) cudaFreeAsync(c->scores, nullptr);
    if (c->d_unit_ptrs) cudaFreeAsync(c->d_unit_ptrs, nullptr);

    if (c->d_topk_ring) cudaFree(c->d_topk_ring);
    for (auto& pt : c->pend) {
      if (pt.h_ids) cudaFreeHost(pt.h_ids);
      if (pt.ev) cudaEventDestroy(pt.ev);
    }
    if (c->unit_prob) cudaFree(c->unit_prob);
    if (c->h_unit_prob) cudaFreeHost(c->h_unit_prob);
    if (c->h_topk) cudaFreeHost(c->h_topk);
    if (c->h_tc_err) cudaFreeHost(c->h_tc_err);
    if (c->ev_err) cudaEventDestroy(c->ev_err);
    if (c->h_spec) cudaFreeHost(c->h_spec);
    for (auto& l : c->la) {
      if (l.h_ids) cudaFreeHost(l.h_ids);
      if (l.ev) cudaEventDestroy(l.ev);
      if (l.ev_staged) cudaEventDestroy(l.ev_staged);
    }
    if (c->h_cand_rows) cudaFreeHost(c->h_cand_rows);
    if (c->h_cand_scores) cudaFreeHost(c->h_cand_scores);
    if (c->scores_aux) cudaFreeAsync(c->scores_aux, nullptr);
    if (c->tc_part) cudaFreeAsync(c->tc_part, nullptr);
    cudaStreamDestroy(c->aux_stream);
    cudaStreamDestroy(c->mail_stream);
    if (c->d_cand_scores) cudaFree(c->d_cand_scores);
    if (c->d_spec) cudaFree(c->d_spec);
    cudaStreamDestroy(c->d2h_stream);
    cudaEventDestroy(c->ev_d2h);
    cudaEventDestroy(c->ev_ingest);
    for (int i = 0; i < 2; ++i) {
      if (c->pack_buf[i]) cudaFree(c->pack_buf[i]);
      if (c->ev_pack[i]) cudaEventDestroy(c->ev_pack[i]);
    }
    cudaEventDestroy(c->ev_spec);
    cudaEventDestroy(c->ev_cand);
    cudaEventDestroy(c->ev_seal);
    cudaEventDestroy(c->ev_stage);
    if (c->slab_pending) {
      void* p = c->slab_future.get();
      if (p) cudaFreeHost(p);
    }
    for (cudaEvent_t e : c->slot_ev)
      if (e) cudaEventDestroy(e);
    for (void* p : c->slabs) cudaFreeHost(p);
    release_dev_slabs(c);
    cudaStreamDestroy(c->copy_stream);
    cudaEventDestroy(c->ev_main);
    cudaEventDestroy(c->ev_copy);
    cudaEventDestroy(c->ev_sync);
    cudaEventDestroy(c->ev_attn);
    cudaEventDestroy(c->ev_attn_prev);
    cudaStreamDestroy(c->urgent_stream);
    for (cudaEvent_t e : c->ev_pool) cudaEventDestroy(e);
    cudaDeviceSynchronize();
  }
  delete c;
  return INFLLM_OK;
}

extern "C" int infllm_ctx_append(infllm_ctx* c, const void* d_q, int64_t q_hs, int64_t q_ts, const void* d_k,
                                 int64_t k_hs, int64_t k_ts, const void* d_v, int64_t v_hs, int64_t v_ts, void* d_out,
                                 int64_t o_hs, int64_t o_ts, int64_t len, void* stream) {
  if (!c) return fail(INFLLM_E_BADARG, "ctx_append: null context");
  if (len < 0 || (len > 0 && (!d_q || !d_k || !d_v || !d_out))) return fail(INFLLM_E_BADARG, "ctx_append: bad argument");
  if (len == 0) return INFLLM_OK;
  if ((o_hs % 2) || (o_ts % 2) || ((uintptr_t)d_out % 4))
    return fail(INFLLM_E_BADARG, "ctx_append: output rows must be 4-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  INFLLM_CUDA_OK(cudaSetDevice(c->cfg.device));
  if (!c->initialized) INFLLM_TRY(lazy_init(c, s));
  INFLLM_TRY(poll_device_error(c, s));
  c->call_serial += 1;
  c->last_stream = s;
  c->trace_topk.clear();
  c->counters.exec_blocks = 0;
  const int esz = c->esz;
  c->chunk_mode = c->cfg.chunk_topk_calc > 0 && len > 1;  // context_manager.py:749
  for (int64_t off = 0; off < len; off += c->sub_max) {
    const int64_t n = std::min<int64_t>(c->sub_max, len - off);
    c->call_off = off;
    INFLLM_TRY(append_sub(c, (const char*)d_q + off * q_ts * esz, q_hs, q_ts, (const char*)d_k + off * k_ts * esz, k_hs,
                          k_ts, (const char*)d_v + off * v_ts * esz, v_hs, v_ts, (char*)d_out + off * o_ts * esz, o_hs,
                          o_ts, n, s));
  }
  if (c->use_tc && len > 64) INFLLM_TRY(send_device_error(c, s, s));  // read by the next call (or by get_info)
  return INFLLM_OK;
}

// the tables the host keeps lag behind one-token appends by design: anyone who asks for them gets them up to date
static int settle_for_caller(infllm_ctx* c) {
  if (!c->initialized || c->pend_count == 0) return INFLLM_OK;
  INFLLM_CUDA_OK(cudaSetDevice(c->cfg.device));
  return settle_all(c, c->last_stream);
}

extern "C" int infllm_ctx_get_info(infllm_ctx* c, infllm_ctx_info* info) {
  if (!c || !info) return fail(INFLLM_E_BADARG, "ctx_get_info: null pointer");
  INFLLM_TRY(settle_for_caller(c));
  *info = c->counters;
  info->length = c->length;
  info->frontier = c->frontier;
  info->num_blocks = c->num_blocks;
  info->init_len = c->init_len;
  info->num_cached = (int64_t)c->lru.size();
  info->load_count = c->load_count;
  return INFLLM_OK;
}

extern "C" int infllm_ctx_profile(infllm_ctx* c, int enable) {
  if (!c) return fail(INFLLM_E_BADARG, "ctx_profile: null context");
  c->prof = enable != 0;
  return INFLLM_OK;
}

extern "C" int infllm_ctx_get_profile(infllm_ctx* c, double* ms, double* work, int64_t* launches) {
  if (!c || !ms || !work || !launches) return fail(INFLLM_E_BADARG, "ctx_get_profile: null pointer");
  if (c->initialized) {
    INFLLM_CUDA_OK(cudaSetDevice(c->cfg.device));
    for (auto& p : c->pending) {
      INFLLM_CUDA_OK(cudaEventSynchronize(p.b));
      float t = 0.f;
      INFLLM_CUDA_OK(cudaEventElapsedTime(&t, p.a, p.b));
      c->prof_ms[p.slot] += t;
    }
  }
  c->pending.clear();
  c->ev_used = 0;
  for (int i = 0; i < INFLLM_PROF_SLOTS; ++i) {
    ms[i] = c->prof_ms[i];
    work[i] = c->prof_work[i];
    launches[i] = c->prof_launches[i];
    c->prof_ms[i] = c->prof_work[i] = 0;
    c->prof_launches[i] = 0;
  }
  return INFLLM_OK;
}

extern "C" int infllm_ctx_trace(infllm_ctx* c, int enable) {
  if (!c) return fail(INFLLM_E_BADARG, "ctx_trace: null context");
  c->trace_on = enable != 0;
  return INFLLM_OK;
}

extern "C" int infllm_ctx_get_trace(infllm_ctx* c, int32_t* labels, int64_t* ebs, float* ms, int cap, int* n) {
  if (!c || !n) return fail(INFLLM_E_BADARG, "ctx_get_trace: null pointer");
  int k = 0;
  if (!c->marks.empty()) {
    INFLLM_CUDA_OK(cudaSetDevice(c->cfg.device));
    INFLLM_CUDA_OK(cudaDeviceSynchronize());
    for (auto& m : c->marks) {
      if (k < cap && labels && ebs && ms) {
        float t = 0.f;
        cudaEventElapsedTime(&t, c->marks[0].ev, m.ev);
        labels[k] = m.label;
        ebs[k] = m.eb;
        ms[k] = t;
        ++k;
      }
    }
    for (auto& m : c->marks) cudaEventDestroy(m.ev);
    c->marks.clear();
  }
  *n = k;
  return INFLLM_OK;
}

extern "C" int infllm_ctx_get_host_timers(infllm_ctx* c, double* us) {
  if (!c || !us) return fail(INFLLM_E_BADARG, "ctx_get_host_timers: null pointer");
  for (int i = 0; i < INFLLM_HOST_TIMERS; ++i) {
    us[i] = c->host_us[i];
    c->host_us[i] = 0;
  }
  return INFLLM_OK;
}

extern "C" int infllm_ctx_get_cached(infllm_ctx* c, int32_t* h_ids, double* h_stamps, int cap, int* n) {
  if (!c || !n) return fail(INFLLM_E_BADARG, "ctx_get_cached: null pointer");
  INFLLM_TRY(settle_for_caller(c));
  int i = 0;
  for (auto& kv : c->lru.items) {
    if (i < cap) {
      if (h_ids) h_ids[i] = kv.first;
      if (h_stamps) h_stamps[i] = kv.second;
    }
    ++i;
  }
  *n = i;
  return INFLLM_OK;
}

extern "C" int infllm_ctx_get_topk(infllm_ctx* c, int64_t eb, int32_t* h_ids, int cap, int* n) {
  if (!c || !n) return fail(INFLLM_E_BADARG, "ctx_get_topk: null pointer");
  INFLLM_TRY(settle_for_caller(c));
  if (eb < 0 || eb >= (int64_t)c->trace_topk.size())
    return fail(INFLLM_E_BADARG, "ctx_get_topk: exec block %lld of %zu", (long long)eb, c->trace_topk.size());
  const auto& t = c->trace_topk[eb];
  for (int i = 0; i < (int)t.size() && i < cap; ++i) h_ids[i] = t[i];
  *n = (int)t.size();
  return INFLLM_OK;
}

extern "C" int infllm_ctx_get_block_k(infllm_ctx* c, int64_t b0, int64_t n, void* h_dst) {
  if (!c || !h_dst) return fail(INFLLM_E_BADARG, "ctx_get_block_k: null pointer");
  if (b0 < 0 || n < 0 || b0 + n > c->num_blocks) return fail(INFLLM_E_BADARG, "ctx_get_block_k: range outside the %lld sealed units", (long long)c->num_blocks);
  if (n == 0) return INFLLM_OK;
  INFLLM_CUDA_OK(cudaSetDevice(c->cfg.device));
  INFLLM_CUDA_OK(cudaDeviceSynchronize());
  INFLLM_CUDA_OK(cudaMemcpy(h_dst, (char*)c->block_k + b0 * c->width * c->esz, n * c->width * c->esz, cudaMemcpyDeviceToHost));
  return INFLLM_OK;
}

extern "C" int infllm_ctx_load_synthetic(infllm_ctx* c, int64_t n_units, const void* h_units, const void* h_block_k,
                                         const void* h_init_k, const void* h_init_v, const void* h_win_k,
                                         const void* h_win_v, void* stream) {
  if (!c || !h_units || !h_block_k || !h_win_k || !h_win_v) return fail(INFLLM_E_BADARG, "ctx_load_synthetic: null pointer");
  const infllm_config& g = c->cfg;
  if (g.n_init > 0 && (!h_init_k || !h_init_v)) return fail(INFLLM_E_BADARG, "ctx_load_synthetic: null init sink");
  cudaStream_t s = (cudaStream_t)stream;
  INFLLM_CUDA_OK(cudaSetDevice(g.device));
  if (!c->initialized) INFLLM_TRY(lazy_init(c, s));
  INFLLM_TRY(infllm_ctx_reset(c));
  const int64_t D = g.head_dim, HKV = g.n_kv_heads;
  INFLLM_TRY(ensure_host_units(c, n_units));
  for (int64_t b = 0; b < n_units; ++b) memcpy(c->host_unit(b), (const char*)h_units + b * c->unit_bytes, c->unit_bytes);
  INFLLM_TRY(fill_dev_store(c, n_units));
  INFLLM_TRY(ensure_block_k(c, n_units, s));
  INFLLM_CUDA_OK(cudaMemcpyAsync(c->block_k, h_block_k, n_units * c->width * c->esz, cudaMemcpyHostToDevice, s));
  if (g.n_init > 0) {
    INFLLM_CUDA_OK(cudaMemcpy2DAsync(c->init_k, c->init_cap * D * c->esz, h_init_k, g.n_init * D * c->esz,
                                     g.n_init * D * c->esz, HKV, cudaMemcpyHostToDevice, s));
    INFLLM_CUDA_OK(cudaMemcpy2DAsync(c->init_v, c->init_cap * D * c->esz, h_init_v, g.n_init * D * c->esz,
                                     g.n_init * D * c->esz, HKV, cudaMemcpyHostToDevice, s));
  }
  c->init_len = g.n_init;
  c->init_full = true;
  c->num_blocks = n_units;
  c->d2h_synced_upto = n_units;  // written into the store by the host just above
  c->frontier = g.n_init + n_units * (int64_t)g.block_size;
  c->length = c->frontier;
  // the local window enters through the ordinary ingest path, without queries: tokens only
  INFLLM_TRY(ensure_tokens(c, g.n_local, s));
  TokenBuffers& tb = c->tb;
  const int64_t kv_hs = tb.cap * D;
  void* tmp = nullptr;
  const size_t wbytes = HKV * (int64_t)g.n_local * D * c->esz;
  INFLLM_CUDA_OK(cudaMallocAsync(&tmp, 2 * wbytes, s));
  INFLLM_CUDA_OK(cudaMemcpyAsync(tmp, h_win_k, wbytes, cudaMemcpyHostToDevice, s));
  INFLLM_CUDA_OK(cudaMemcpyAsync((char*)tmp + wbytes, h_win_v, wbytes, cudaMemcpyHostToDevice, s));
  const int64_t at = c->length - tb.t0;
  INFLLM_TRY(copy_rows_launch(tmp, (int64_t)g.n_local * D, D, (char*)tb.k_raw + at * D * c->esz, kv_hs, D, (int)HKV,
                              g.n_local, (int)D, s));
  INFLLM_TRY(copy_rows_launch((char*)tmp + wbytes, (int64_t)g.n_local * D, D, (char*)tb.v + at * D * c->esz, kv_hs, D,
                              (int)HKV, g.n_local, (int)D, s));
  INFLLM_CUDA_OK(cudaMemset2DAsync(tb.score + at, tb.cap * sizeof(float), 0, g.n_local * sizeof(float), g.n_heads, s));
  c->rope_origin = c->length;
  INFLLM_TRY(rope_apply_launch((char*)tb.k_raw + at * D * c->esz, kv_hs, D, (char*)tb.k_rot + at * D * c->esz, kv_hs, D,
                               (int)HKV, g.n_local, (int)D, c->cos_t, c->sin_t, c->tab_len, 0, 1, g.dtype, s));
  INFLLM_CUDA_OK(cudaFreeAsync(tmp, s));
  c->length += g.n_local;
  INFLLM_CUDA_OK(cudaStreamSynchronize(s));
  return INFLLM_OK;
}

// ------------------------------------------------------------------ LRU table alone (host, GPU-free)
struct infllm_lru {
  LruTable t;
  explicit infllm_lru(int cap) : t(cap) {}
};

extern "C" int infllm_lru_create(int capacity, infllm_lru** out) {
  if (!out || capacity <= 0) return fail(INFLLM_E_BADARG, "lru_create: bad argument");
  *out = new (std::nothrow) infllm_lru(capacity);
  return *out ? INFLLM_OK : fail(INFLLM_E_NOMEM, "lru_create: out of host memory");
}
extern "C" int infllm_lru_destroy(infllm_lru* t) {
  delete t;
  return INFLLM_OK;
}
extern "C" int infllm_lru_plan(infllm_lru* t, const int32_t* wanted, int n, int32_t* h_evicted, int* n_evicted) {
  if (!t || (n > 0 && !wanted) || !n_evicted) return fail(INFLLM_E_BADARG, "lru_plan: null pointer");
  std::vector<int32_t> ev;
  t->t.plan(wanted, n, &ev);
  for (size_t i = 0; i < ev.size(); ++i)
    if (h_evicted) h_evicted[i] = ev[i];
  *n_evicted = (int)ev.size();
  return INFLLM_OK;
}
extern "C" int infllm_lru_stamp(infllm_lru* t, const int32_t* wanted, int n, double value) {
  if (!t || (n > 0 && !wanted)) return fail(INFLLM_E_BADARG, "lru_stamp: null pointer");
  t->t.stamp(wanted, n, value);
  return INFLLM_OK;
}
extern "C" int infllm_lru_scale(infllm_lru* t, double factor) {
  if (!t) return fail(INFLLM_E_BADARG, "lru_scale: null pointer");
  t->t.scale(factor);
  return INFLLM_OK;
}
extern "C" int infllm_lru_add(infllm_lru* t, int32_t id, double value) {
  if (!t) return fail(INFLLM_E_BADARG, "lru_add: null pointer");
  return t->t.add(id, value) ? INFLLM_OK : fail(INFLLM_E_BADARG, "lru_add: id %d is not in the table", id);
}
extern "C" int infllm_lru_items(infllm_lru* t, int32_t* h_ids, double* h_stamps, int cap, int* n) {
  if (!t || !n) return fail(INFLLM_E_BADARG, "lru_items: null pointer");
  int i = 0;
  for (auto& kv : t->t.items) {
    if (i < cap) {
      if (h_ids) h_ids[i] = kv.first;
      if (h_stamps) h_stamps[i] = kv.second;
    }
    ++i;
  }
  *n = i;
  return INFLLM_OK;
}

extern "C" int infllm_unit_fetch(void* d_slot, const void* h_unit, int64_t bytes, void* stream) {
  if (!d_slot || !h_unit || bytes <= 0) return fail(INFLLM_E_BADARG, "unit_fetch: bad argument");
  INFLLM_CUDA_OK(cudaMemcpyAsync(d_slot, h_unit, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return INFLLM_OK;
}

constexpr int kShardMaxIds = 256;
// The cache of a caller that keeps its own (the unit-range shard of the sharded decode): LRU plan for the owned
// part of a retrieval, eviction, refills from the pinned store on `stream`, and the two device tables, in one call.
extern "C" int infllm_shard_refill(infllm_shard_cache* c, const int32_t* ids, int n, void* stream) {
  if (!c || !c->lru || !c->slot_of || !c->free_slots || (n > 0 && !ids)) return fail(INFLLM_E_BADARG, "shard_refill: null pointer");
  if (n > kShardMaxIds) return fail(INFLLM_E_BADARG, "shard_refill: %d ids, at most %d", n, kShardMaxIds);
  c->load_count += 1;
  int32_t owned[kShardMaxIds];
  int m = 0;
  for (int i = 0; i < n; ++i)
    if (ids[i] >= c->id_lo && ids[i] < c->id_lo + c->n_owned) owned[m++] = ids[i];
  if (m == 0) return INFLLM_OK;
  int32_t ch_ids[2 * kShardMaxIds], ch_slots[2 * kShardMaxIds];
  uint64_t ch_addrs[2 * kShardMaxIds];
  int n_ch = 0;
  std::vector<int32_t> ev;
  c->lru->t.plan(owned, m, &ev);
  for (int32_t b : ev) {
    const int i = b - c->id_lo;
    if (i < 0 || i >= c->n_owned || c->slot_of[i] < 0 || n_ch >= 2 * kShardMaxIds)
      return fail(INFLLM_E_CAPACITY, "shard_refill: evicted unit %d is not in the cache", b);
    c->free_slots[c->n_free++] = c->slot_of[i];
    c->slot_of[i] = -1;
    ch_ids[n_ch] = i, ch_slots[n_ch] = -1;
    ch_addrs[n_ch++] = (uint64_t)(uintptr_t)c->h_units + (uint64_t)i * (uint64_t)c->unit_bytes;
  }
  c->lru->t.stamp(owned, m, (double)c->load_count);
  for (int j = 0; j < m; ++j) {
    const int i = owned[j] - c->id_lo;
    if (c->slot_of[i] >= 0) {
      c->hits += 1;
      continue;
    }
    c->misses += 1;
    if (c->n_free <= 0 || n_ch >= 2 * kShardMaxIds) return fail(INFLLM_E_CAPACITY, "shard_refill: no free cache slot");
    const int slot = c->free_slots[--c->n_free];
    c->slot_of[i] = slot;
    char* dst = (char*)c->d_cache + (size_t)slot * (size_t)c->unit_bytes;
    INFLLM_CUDA_OK(cudaMemcpyAsync(dst, (const char*)c->h_units + (size_t)i * (size_t)c->unit_bytes, (size_t)c->unit_bytes,
                                   cudaMemcpyHostToDevice, (cudaStream_t)stream));
    ch_ids[n_ch] = i, ch_slots[n_ch] = slot;
    ch_addrs[n_ch++] = (uint64_t)(uintptr_t)dst;
  }
  if (n_ch > 0) {
    if (c->d_slot_table) INFLLM_TRY(infllm_slot_table_update(c->d_slot_table, ch_ids, ch_slots, n_ch, stream));
    if (c->d_ptr_table) INFLLM_TRY(infllm_ptr_table_update(c->d_ptr_table, ch_ids, ch_addrs, n_ch, stream));
  }
  return INFLLM_OK;
}

extern "C" int infllm_ctx_set_comm(infllm_ctx* c, infllm_comm* comm) {
  if (!c) return fail(INFLLM_E_BADARG, "ctx_set_comm: null context");
  if (c->length != 0) return fail(INFLLM_E_BADARG, "ctx_set_comm: the context already holds tokens");
  c->comm = comm;
  return INFLLM_OK;
}

// ------------------------------------------------------------------------------------------- persistence
// The reference keeps a layer's memory only live, inside past_key_values (inf_llm/utils/greedy_search.py:99);
// these two calls write it to a file and bring it back, so that a session can be resumed in another process.
// File: a header of int64 words, then the LRU table (id, stamp) in dict order, the sink, the representative keys,
// the un-sealed tokens (raw keys, values, accumulated scores) and the sealed units as the host store holds them.
// The rotated keys are not stored: they are rotated anew on the next append.
namespace {
constexpr int64_t kStateMagic = 0x324d454d4c464e49ll;  // "INFLMEM2"
constexpr int kStateHdrWords = 24;

bool put(FILE* f, const void* p, size_t n) { return n == 0 || fwrite(p, 1, n, f) == n; }
bool get(FILE* f, void* p, size_t n) { return n == 0 || fread(p, 1, n, f) == n; }

int64_t decay_bits(double d) {
  int64_t b;
  memcpy(&b, &d, sizeof(b));
  return b;
}

struct FileCloser {
  FILE* f;
  ~FileCloser() {
    if (f) fclose(f);
  }
};
}  // namespace

extern "C" int infllm_ctx_save(infllm_ctx* c, const char* path, void* stream) {
  if (!c || !path) return fail(INFLLM_E_BADARG, "ctx_save: null pointer");
  if (!c->initialized) return fail(INFLLM_E_BADARG, "ctx_save: the context holds nothing yet");
  INFLLM_TRY(settle_for_caller(c));
  const infllm_config& g = c->cfg;
  cudaStream_t s = (cudaStream_t)stream;
  INFLLM_CUDA_OK(cudaSetDevice(g.device));
  // every copy-out of a sealed unit must have landed in the host store
  INFLLM_CUDA_OK(cudaStreamSynchronize(s));
  INFLLM_CUDA_OK(cudaStreamSynchronize(c->d2h_stream));
  const int64_t D = g.head_dim, H = g.n_heads, HKV = g.n_kv_heads;
  const int64_t live = c->length - c->frontier, n_lru = (int64_t)c->lru.items.size();
  FILE* f = fopen(path, "wb");
  if (!f) return fail(INFLLM_E_BADARG, "ctx_save: cannot open %s", path);
  const int64_t hdr[kStateHdrWords] = {
      kStateMagic, H, HKV, D, g.n_init, g.n_local, g.block_size, g.dtype, c->length, c->frontier,
      c->num_blocks, c->init_len, c->init_full ? 1 : 0, c->load_count, n_lru, g.cache_strategy,
      g.max_cached_block, g.topk, g.exc_block_size, g.repr_topk, g.chunk_topk_calc, decay_bits(g.score_decay), 0, 0};
  bool ok = put(f, hdr, sizeof(hdr));
  for (auto& kv : c->lru.items) {
    const int64_t id = kv.first;
    ok = ok && put(f, &id, sizeof(id)) && put(f, &kv.second, sizeof(double));
  }
  std::vector<char> buf;
  auto dump2d = [&](const void* dev, int64_t pitch, int64_t width, int64_t rows) -> bool {  // strided device rows
    if (width * rows == 0) return true;
    buf.resize((size_t)(width * rows));
    if (cudaMemcpy2D(buf.data(), width, dev, pitch, width, rows, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
    return put(f, buf.data(), buf.size());
  };
  ok = ok && dump2d(c->init_k, c->init_cap * D * c->esz, c->init_len * D * c->esz, HKV);
  ok = ok && dump2d(c->init_v, c->init_cap * D * c->esz, c->init_len * D * c->esz, HKV);
  ok = ok && dump2d(c->block_k, c->width * c->esz, c->width * c->esz, c->num_blocks);
  const TokenBuffers& tb = c->tb;
  const int64_t off = (c->frontier - tb.t0) * D * c->esz, pitch = tb.cap * D * c->esz;
  ok = ok && dump2d((char*)tb.k_raw + off, pitch, live * D * c->esz, HKV);
  ok = ok && dump2d((char*)tb.v + off, pitch, live * D * c->esz, HKV);
  ok = ok && dump2d(tb.score + (c->frontier - tb.t0), tb.cap * sizeof(float), live * sizeof(float), H);
  for (int64_t b = 0; ok && b < c->num_blocks; ++b) ok = put(f, c->host_unit(b), (size_t)c->unit_bytes);
  ok = (fclose(f) == 0) && ok;
  if (!ok) return fail(INFLLM_E_CUDA, "ctx_save: writing %s failed", path);
  return INFLLM_OK;
}

// Everything the file says is checked before any state of the context (or the GPU) is touched: the header
// against the configuration, the lengths against each other, the LRU entries against the unit count and the cache
// size, and the file's size against what those lengths imply.
extern "C" int infllm_ctx_load(infllm_ctx* c, const char* path, void* stream) {
  if (!c || !path) return fail(INFLLM_E_BADARG, "ctx_load: null pointer");
  const infllm_config& g = c->cfg;
  cudaStream_t s = (cudaStream_t)stream;
  FileCloser fc{fopen(path, "rb")};
  FILE* f = fc.f;
  if (!f) return fail(INFLLM_E_BADARG, "ctx_load: cannot open %s", path);
  int64_t hdr[kStateHdrWords];
  if (!get(f, hdr, sizeof(hdr)) || hdr[0] != kStateMagic)
    return fail(INFLLM_E_BADARG, "ctx_load: %s is not a saved context memory", path);
  if (hdr[1] != g.n_heads || hdr[2] != g.n_kv_heads || hdr[3] != g.head_dim || hdr[4] != g.n_init || hdr[5] != g.n_local ||
      hdr[6] != g.block_size || hdr[7] != g.dtype || hdr[15] != g.cache_strategy || hdr[16] != g.max_cached_block ||
      hdr[17] != g.topk || hdr[18] != g.exc_block_size || hdr[19] != g.repr_topk || hdr[20] != g.chunk_topk_calc ||
      hdr[21] != decay_bits(g.score_decay))
    return fail(INFLLM_E_BADARG, "ctx_load: %s was saved with another configuration", path);
  const int64_t D = g.head_dim, H = g.n_heads, HKV = g.n_kv_heads;
  const int64_t length = hdr[8], frontier = hdr[9], n_units = hdr[10], init_len = hdr[11], n_lru = hdr[14];
  const int64_t live = length - frontier;
  if (length < 0 || frontier < 0 || n_units < 0 || n_units > INT32_MAX || init_len < 0 || init_len > g.n_init ||
      live < 0 || frontier != init_len + n_units * (int64_t)g.block_size || (hdr[12] != 0) != (init_len == g.n_init) ||
      (n_units > 0 && init_len != g.n_init) || hdr[13] < 0)
    return fail(INFLLM_E_BADARG, "ctx_load: %s holds inconsistent lengths (length %lld, frontier %lld, %lld units, sink %lld)",
                path, (long long)length, (long long)frontier, (long long)n_units, (long long)init_len);
  if (n_lru < 0 || n_lru > g.max_cached_block)
    return fail(INFLLM_E_BADARG, "ctx_load: %s lists %lld cached units, the cache holds %d", path, (long long)n_lru,
                g.max_cached_block);
  const int64_t esz = 2, unit_bytes = 2 * (int64_t)HKV * g.block_size * D * esz;
  const int64_t expect = (int64_t)sizeof(hdr) + n_lru * 16 + 2 * HKV * init_len * D * esz + n_units * H * D * esz +
                         2 * HKV * live * D * esz + H * live * (int64_t)sizeof(float) + n_units * unit_bytes;
  if (fseek(f, 0, SEEK_END) != 0 || (int64_t)ftell(f) != expect || fseek(f, (long)sizeof(hdr), SEEK_SET) != 0)
    return fail(INFLLM_E_BADARG, "ctx_load: %s has not the %lld bytes its header implies", path, (long long)expect);
  std::vector<std::pair<int32_t, double>> lru;
  {
    std::vector<char> seen((size_t)n_units, 0);
    for (int64_t i = 0; i < n_lru; ++i) {
      int64_t id;
      double stamp;
      if (!get(f, &id, sizeof(id)) || !get(f, &stamp, sizeof(stamp)))
        return fail(INFLLM_E_BADARG, "ctx_load: %s ends inside the cache table", path);
      if (id < 0 || id >= n_units || seen[(size_t)id] || !(stamp == stamp))
        return fail(INFLLM_E_BADARG, "ctx_load: %s lists cached unit %lld (of %lld units) wrongly", path, (long long)id,
                    (long long)n_units);
      seen[(size_t)id] = 1;
      lru.push_back({(int32_t)id, stamp});
    }
  }
  INFLLM_CUDA_OK(cudaSetDevice(g.device));
  if (!c->initialized) INFLLM_TRY(lazy_init(c, s));
  INFLLM_TRY(infllm_ctx_reset(c));
  bool ok = true;
  std::vector<char> buf;
  auto fill2d = [&](void* dev, int64_t pitch, int64_t width, int64_t rows) -> bool {
    if (width * rows == 0) return true;
    buf.resize((size_t)(width * rows));
    if (!get(f, buf.data(), buf.size())) return false;
    return cudaMemcpy2D(dev, pitch, buf.data(), width, width, rows, cudaMemcpyHostToDevice) == cudaSuccess;
  };
  ok = ok && fill2d(c->init_k, c->init_cap * D * c->esz, init_len * D * c->esz, HKV);
  ok = ok && fill2d(c->init_v, c->init_cap * D * c->esz, init_len * D * c->esz, HKV);
  if (ok && ensure_block_k(c, std::max<int64_t>(n_units, 1), s) != INFLLM_OK) ok = false;
  if (ok && cudaStreamSynchronize(s) != cudaSuccess) ok = false;
  ok = ok && fill2d(c->block_k, c->width * c->esz, c->width * c->esz, n_units);
  // the un-sealed tokens go to the start of fresh token buffers
  c->length = c->frontier = frontier;
  if (ok && ensure_tokens(c, live, s) != INFLLM_OK) ok = false;
  if (ok && cudaStreamSynchronize(s) != cudaSuccess) ok = false;
  if (ok) {
    TokenBuffers& tb = c->tb;
    const int64_t pitch = tb.cap * D * c->esz, off = (frontier - tb.t0) * D * c->esz;
    ok = fill2d((char*)tb.k_raw + off, pitch, live * D * c->esz, HKV) &&
         fill2d((char*)tb.v + off, pitch, live * D * c->esz, HKV) &&
         fill2d(tb.score + (frontier - tb.t0), tb.cap * sizeof(float), live * sizeof(float), H);
  }
  if (ok && ensure_host_units(c, n_units) != INFLLM_OK) ok = false;
  for (int64_t b = 0; ok && b < n_units; ++b) ok = get(f, c->host_unit(b), (size_t)c->unit_bytes);
  if (ok && fill_dev_store(c, n_units) != INFLLM_OK) ok = false;
  if (!ok) {
    infllm_ctx_reset(c);
    return fail(INFLLM_E_CUDA, "ctx_load: reading %s failed", path);
  }
  c->length = length;
  c->num_blocks = n_units;
  c->init_len = init_len;
  c->init_full = hdr[12] != 0;
  c->load_count = hdr[13];
  c->d2h_synced_upto = n_units;
  c->d2h_synced_upto_urgent = n_units;
  c->rope_origin = -1;  // the window is rotated anew by the next append
  // the cache comes back as the LRU table lists it (n_lru <= max_cached_block slots were checked above)
  for (auto& kv : lru) {
    const int slot = c->free_slots.back();
    c->free_slots.pop_back();
    c->slot_of[kv.first] = slot;
    c->lru.set(kv.first, kv.second);
    INFLLM_CUDA_OK(cudaMemcpyAsync((char*)c->cache + (int64_t)slot * c->unit_bytes, c->host_unit(kv.first), c->unit_bytes,
                                   cudaMemcpyHostToDevice, s));
  }
  INFLLM_CUDA_OK(cudaStreamSynchronize(s));
  return INFLLM_OK;
}

// ------------------------------------------------------------------------------- device-store pool
extern "C" int infllm_device_store_reserve(int device, int64_t bytes) {
  if (device < 0 || device >= 64 || bytes < 0) return fail(INFLLM_E_BADARG, "device_store_reserve: bad argument");
  INFLLM_CUDA_OK(cudaSetDevice(device));
  const int64_t n = bytes / (int64_t)kPoolSlabBytes;
  for (int64_t i = 0; i < n; ++i) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, kPoolSlabBytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(INFLLM_E_NOMEM, "device_store_reserve: cudaMalloc failed after %lld of %lld slabs of 128 MiB: %s",
                  (long long)i, (long long)n, cudaGetErrorString(e));
    }
    std::lock_guard<std::mutex> lk(g_pool[device].mu);
    g_pool[device].free_slabs.push_back(p);
    g_pool[device].total += 1;
  }
  return INFLLM_OK;
}

extern "C" int infllm_device_store_release(int device) {
  if (device < 0 || device >= 64) return fail(INFLLM_E_BADARG, "device_store_release: bad device");
  INFLLM_CUDA_OK(cudaSetDevice(device));
  INFLLM_CUDA_OK(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lk(g_pool[device].mu);
  for (void* p : g_pool[device].free_slabs) cudaFree(p);
  g_pool[device].total -= (int64_t)g_pool[device].free_slabs.size();
  g_pool[device].free_slabs.clear();
  return INFLLM_OK;
}

extern "C" int infllm_device_store_info(int device, int64_t* total_bytes, int64_t* used_bytes) {
  if (device < 0 || device >= 64) return fail(INFLLM_E_BADARG, "device_store_info: bad device");
  std::lock_guard<std::mutex> lk(g_pool[device].mu);
  if (total_bytes) *total_bytes = g_pool[device].total * (int64_t)kPoolSlabBytes;
  if (used_bytes) *used_bytes = g_pool[device].used * (int64_t)kPoolSlabBytes;
  return INFLLM_OK;
}
