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
