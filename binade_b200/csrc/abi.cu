// Status plumbing of the C ABI: thread-local last error, version.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace bn {

static thread_local char g_error[512] = "";

int fail(int code, const char *msg) {
  snprintf(g_error, sizeof g_error, "%s", msg);
  return code;
}

int fail_cuda(cudaError_t e, const char *where) {
  snprintf(g_error, sizeof g_error, "%s: %s (%s)", where, cudaGetErrorString(e), cudaGetErrorName(e));
  return BN_ERR_CUDA;
}

}  // namespace bn

extern "C" const char *bn_last_error(void) { return bn::g_error; }
extern "C" int bn_abi_version(void) { return 201; }
