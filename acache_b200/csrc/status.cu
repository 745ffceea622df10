// Status strings and the per-thread CUDA error record.
#include <stdlib.h>

#include "common.cuh"

namespace acache {
static thread_local cudaError_t g_last_error = cudaSuccess;
void set_last_cuda_error(cudaError_t e) { g_last_error = e; }

bool chained_launches() {
  static const bool on = [] {
    const char* v = getenv("ACACHE_CHAINED_LAUNCHES");
    return !(v && v[0] == '0');
  }();
  return on;
}
}  // namespace acache

extern "C" const char* acache_status_string(int status) {
  switch (status) {
    case ACACHE_OK: return "ok";
    case ACACHE_EINVAL: return "invalid argument";
    case ACACHE_EUNSUPPORTED: return "unsupported configuration";
    case ACACHE_ECUDA: return "CUDA error";
    case ACACHE_ELIMIT: return "size beyond a fixed limit";
    case ACACHE_ETIMEOUT: return "bounded device wait gave up";
    default: return "unknown status";
  }
}

extern "C" const char* acache_last_cuda_error(void) { return cudaGetErrorString(acache::g_last_error); }

extern "C" int acache_abi_version(void) { return 1; }
