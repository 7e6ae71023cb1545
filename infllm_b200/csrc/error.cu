// Error reporting of the C ABI: one message per host thread.
#include <atomic>

#include "common.cuh"

namespace infllm {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace infllm

extern "C" const char* infllm_last_error(void) { return infllm::g_err; }
extern "C" const char* infllm_version(void) { return "infllm_b200 0.1 sm_100a"; }
extern "C" long long infllm_launch_count(void) { return infllm::g_launches.load(); }
