// Error reporting of the C ABI: one message per host thread.
#include "common.cuh"

namespace infllm {

static thread_local char g_err[512] = "";

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
