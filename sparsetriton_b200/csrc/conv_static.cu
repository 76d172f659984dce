// Weight gradient for callers that must not allocate: the fp32 partials that the regular
// st_conv_wgrad() takes from a caller-provided workspace live here in a fixed device array.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "conv_maps.cuh"
#include "conv_tc.cuh"

namespace st {

int wgrad_chunks(int64_t n_out);
int reduce_partials(int dtype, const float* partial, int chunks, int64_t n, void* out, cudaStream_t s);
template <typename T, typename Map>
int simt_wgrad(const T* x, const T* dy, const Map& map, T* dw, float* partial, int64_t n_rows, int64_t n_src, int K,
               int cin, int cout, cudaStream_t s);

// 64 MiB per GPU, resident from the moment the library is loaded on that GPU until the process ends.
constexpr int64_t kStaticScratchBytes = 64ll << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// The array's name is only a host-side handle; kernels need its device address, which differs per
// GPU.  It is looked up once per device (with that device current) and remembered.
constexpr int kMaxDevices = 64;
static void* g_scratch_ptr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

static int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("st_conv_wgrad_static: cannot identify the current device (%s)",
              e != cudaSuccess ? cudaGetErrorString(e) : "index out of range");
    return ST_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) {
      set_error("st_conv_wgrad_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return ST_ERR_CUDA;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = static_cast<float*>(g_scratch_ptr[dev]);
  return ST_OK;
}

}  // namespace st

using namespace st;

extern "C" {

int64_t st_conv_wgrad_static_max_bytes(void) { return kStaticScratchBytes; }

int st_conv_wgrad_static(int dtype, const void* X, const void* dY, const int32_t* nbr, void* dW, int64_t n_in,
                         int64_t n_out, int K, int cin, int cout, void* stream) {
  if (dtype != ST_F32 && dtype != ST_F16 && dtype != ST_BF16) {
    set_error("st_conv_wgrad_static: unknown feature dtype %d", dtype);
    return ST_ERR_DTYPE;
  }
  if (n_in < 0 || n_out < 0 || K < 1 || K > ST_MAX_KVOL || cin < 1 || cout < 1 || n_in > 0x7FFFFFFFll ||
      n_out > 0x7FFFFFFFll || !dW || (n_out > 0 && (!X || !dY || !nbr))) {
    set_error("st_conv_wgrad_static: bad arguments");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t n_w = (int64_t)K * cin * cout;
  if (n_out == 0) {
    const cudaError_t e = cudaMemsetAsync(dW, 0, (size_t)n_w * (dtype == ST_F32 ? 4 : 2), s);
    if (e != cudaSuccess) {
      set_error("st_conv_wgrad_static(empty): %s", cudaGetErrorString(e));
      return ST_ERR_CUDA;
    }
    return check_launch("st_conv_wgrad_static(empty)");
  }
  // Which kernel would run, and how many partial bytes it writes.
  const bool use_tc = tc_wgrad_supported(dtype, n_out, K, cin, cout);
  const int64_t need = use_tc ? tc_wgrad_partial_bytes(dtype, n_out, K, cin, cout)
                              : (int64_t)wgrad_chunks(n_out) * n_w * 4;
  if (need > kStaticScratchBytes) {
    set_error("st_conv_wgrad_static: this layer needs %lld bytes of partial sums, the built-in scratch holds %lld; "
              "use st_conv_wgrad with a caller-provided workspace",
              (long long)need, (long long)kStaticScratchBytes);
    return ST_ERR_WORKSPACE;
  }
  float* partial = nullptr;
  int rc = static_scratch(&partial);
  if (rc != ST_OK) return rc;
  // Every partial that is read below is written first by the kernel of this call (both kernels
  // store their whole (chunk, K, cin, cout) block, zeros included), so nothing has to be cleared.
  if (use_tc) {
    int chunks = 0;
    rc = tc_conv_wgrad(dtype, X, dY, nbr, MapPlan{}, partial, &chunks, n_out, n_in, K, cin, cout, s);
    if (rc != ST_OK) return rc;
    return reduce_partials(dtype, partial, chunks, n_w, dW, s);
  }
  StoredMap map{nbr, K};
  switch (dtype) {
    case ST_F32:
      return simt_wgrad<float, StoredMap>(static_cast<const float*>(X), static_cast<const float*>(dY), map,
                                          static_cast<float*>(dW), partial, n_out, n_in, K, cin, cout, s);
    case ST_F16:
      return simt_wgrad<__half, StoredMap>(static_cast<const __half*>(X), static_cast<const __half*>(dY), map,
                                           static_cast<__half*>(dW), partial, n_out, n_in, K, cin, cout, s);
    default:
      return simt_wgrad<__nv_bfloat16, StoredMap>(static_cast<const __nv_bfloat16*>(X),
                                                  static_cast<const __nv_bfloat16*>(dY), map,
                                                  static_cast<__nv_bfloat16*>(dW), partial, n_out, n_in, K, cin, cout,
                                                  s);
  }
}

}  // extern "C"
