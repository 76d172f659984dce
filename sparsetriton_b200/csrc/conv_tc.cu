#include "conv_tc.cuh"
#include "common.cuh"
namespace st {
bool tc_supported(int, int, int) { return false; }
int tc_conv_gather(int, const void*, const void*, const int32_t*, void*, int64_t, int64_t, int, int, int, bool,
                   cudaStream_t) {
  set_error("tensor-core kernels not built");
  return ST_ERR_UNSUPPORTED;
}
}  // namespace st
