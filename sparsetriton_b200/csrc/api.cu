// Library-wide plumbing: version, error text, offset packing and a block-hierarchical prefix sum.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace st {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

void note_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return ST_ERR_CUDA;
  }
  return ST_OK;
}

bool pack_offsets(const int32_t* host, int K, Offsets* out) {
  for (int i = 0; i < K * 3; ++i) {
    if (host[i] < -32768 || host[i] > 32767) return false;
    out->v[i] = (int16_t)host[i];
  }
  return true;
}

// ---------------------------------------------------------------------------------------------
// Exclusive scan: 1024 values per block, block sums scanned recursively (three levels cover 2^30).
// ---------------------------------------------------------------------------------------------
constexpr int kScanBlock = 1024;

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* block_total) {
  __shared__ uint32_t warp_sums[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, d);
    if (lane >= d) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = warp_sums[lane];
    uint32_t wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xFFFFFFFFu, wi, d);
      if (lane >= d) wi += t;
    }
    warp_sums[lane] = wi - w;  // exclusive offset of each warp
    if (lane == 31) *block_total = wi;
  }
  __syncthreads();
  return incl - v + warp_sums[warp];
}

__global__ void __launch_bounds__(kScanBlock)
scan_blocks_kernel(const uint32_t* in, uint32_t* out, int64_t n, uint32_t* block_sums) {
  __shared__ uint32_t total;
  int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  uint32_t v = i < n ? in[i] : 0u;
  uint32_t ex = block_exclusive_scan(v, &total);
  if (i < n) out[i] = ex;
  if (threadIdx.x == 0 && block_sums) block_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanBlock)
scan_add_kernel(uint32_t* out, int64_t n, const uint32_t* block_offsets) {
  int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  if (i < n) out[i] += block_offsets[blockIdx.x];
}

__global__ void scan_total_kernel(const uint32_t* last_in, const uint32_t* last_out, int64_t* total) {
  *total = (int64_t)(*last_in) + (int64_t)(*last_out);
}

__global__ void scan_zero_total_kernel(int64_t* total) { *total = 0; }

int64_t scan_tmp_bytes(int64_t n) {
  // copy of the last input value + level-1 and level-2 block sums
  int64_t b1 = (n + kScanBlock - 1) / kScanBlock;
  int64_t b2 = (b1 + kScanBlock - 1) / kScanBlock;
  return align_up(4, 256) + align_up(b1 * 4, 256) + align_up(b2 * 4, 256) + 256;
}

int exclusive_scan_u32(const uint32_t* in, uint32_t* out, int64_t n, void* tmp, int64_t* total,
                       cudaStream_t stream) {
  if (n <= 0) {
    if (total) { scan_zero_total_kernel<<<1, 1, 0, stream>>>(total); note_launches(1); }
    return check_launch("scan(empty)");
  }
  const int64_t b1 = (n + kScanBlock - 1) / kScanBlock;
  const int64_t b2 = (b1 + kScanBlock - 1) / kScanBlock;
  if (b2 > kScanBlock) {
    set_error("scan: %lld values exceed the three-level limit", (long long)n);
    return ST_ERR_UNSUPPORTED;
  }
  char* p = static_cast<char*>(tmp);
  uint32_t* last_in = reinterpret_cast<uint32_t*>(p);
  p += align_up(4, 256);
  uint32_t* sums1 = reinterpret_cast<uint32_t*>(p);
  p += align_up(b1 * 4, 256);
  uint32_t* sums2 = reinterpret_cast<uint32_t*>(p);

  // in may alias out: keep the last input value for the total
  if (total) cudaMemcpyAsync(last_in, in + (n - 1), 4, cudaMemcpyDeviceToDevice, stream);
  { scan_blocks_kernel<<<(unsigned)b1, kScanBlock, 0, stream>>>(in, out, n, sums1); note_launches(1); }
  if (b1 > 1) {
    { scan_blocks_kernel<<<(unsigned)b2, kScanBlock, 0, stream>>>(sums1, sums1, b1, sums2); note_launches(1); }
    if (b2 > 1) {
      { scan_blocks_kernel<<<1, kScanBlock, 0, stream>>>(sums2, sums2, b2, nullptr); note_launches(1); }
      { scan_add_kernel<<<(unsigned)b2, kScanBlock, 0, stream>>>(sums1, b1, sums2); note_launches(1); }
    }
    { scan_add_kernel<<<(unsigned)b1, kScanBlock, 0, stream>>>(out, n, sums1); note_launches(1); }
  }
  if (total) { scan_total_kernel<<<1, 1, 0, stream>>>(last_in, out + (n - 1), total); note_launches(1); }
  return check_launch("scan");
}

}  // namespace st

extern "C" {

int st_version(void) { return 1; }

const char* st_last_error_string(void) { return st::g_error; }

long long st_launch_count(void) { return st::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
