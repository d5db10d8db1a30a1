// Error state and version of the C-ABI library (see include/triattention_b200.h).
#include "abi_internal.h"
#include <cstdio>
#include <cstring>

namespace {
thread_local char g_error[512] = "";
}

void tri_set_error(const char* what) {
  std::snprintf(g_error, sizeof(g_error), "%s", what ? what : "unknown error");
}

int tri_launch_status(const char* where) {
  const cudaError_t e = cudaGetLastError();   // launch-configuration errors; execution errors surface at the next sync
  if (e == cudaSuccess) return TRI_OK;
  std::snprintf(g_error, sizeof(g_error), "%s: %s", where, cudaGetErrorString(e));
  return TRI_ERR_CUDA;
}

extern "C" const char* tri_last_error(void) { return g_error; }
extern "C" int tri_abi_version(void) { return 5; }   // 4: tri_write_kv, tri_attention_sweep; 5: tri_decode_tail_hint
