// Error reporting and version of libinquant_b200.so.
#include <stdio.h>

#include "common.cuh"

namespace inq {
char* last_error_buffer() {
  static thread_local char buffer[256] = "";
  return buffer;
}
int fail_cuda(cudaError_t err, const char* where) {
  snprintf(last_error_buffer(), 256, "%s: %s", where, cudaGetErrorString(err));
  return INQ_ERR_CUDA;
}
}  // namespace inq

extern "C" const char* inq_last_error(void) { return inq::last_error_buffer(); }
extern "C" int inq_version(void) { return 1; }
