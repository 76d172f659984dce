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
// Exclusive scan.  Up to 16.7 M values take two launches: the sum of every span of 4096 values, then
// each block adds up the sums of the spans before its own (at most 4096 of them, L2-resident) and
// scans its span; the last block also writes the grand total.  Longer inputs go through 1024 values
// per block with the block sums scanned recursively (three levels cover 2^30).
// ---------------------------------------------------------------------------------------------
constexpr int kScanBlock = 1024;
constexpr int kScanPer = 4;                              // consecutive values per thread in the two-launch form
constexpr int kScanSpan = kScanBlock * kScanPer;
constexpr int64_t kScanDirectSpans = 4096;

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

__device__ __forceinline__ uint32_t block_sum(uint32_t v) {
  __shared__ uint32_t warp_part[32];
  __shared__ uint32_t result;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = __reduce_add_sync(0xFFFFFFFFu, v);
  if (lane == 0) warp_part[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const uint32_t w = __reduce_add_sync(0xFFFFFFFFu, warp_part[lane]);
    if (lane == 0) result = w;
  }
  __syncthreads();
  return result;
}

__global__ void __launch_bounds__(kScanBlock) scan_span_sums_kernel(const uint32_t* in, int64_t n, uint32_t* sums) {
  const int64_t first = (int64_t)blockIdx.x * kScanSpan + (int64_t)threadIdx.x * kScanPer;
  uint32_t mine = 0;
#pragma unroll
  for (int j = 0; j < kScanPer; ++j)
    if (first + j < n) mine += in[first + j];
  const uint32_t all = block_sum(mine);
  if (threadIdx.x == 0) sums[blockIdx.x] = all;
}

// `in` may alias `out`: a block reads only its own span before it writes it
__global__ void __launch_bounds__(kScanBlock)
scan_spans_kernel(const uint32_t* in, uint32_t* out, int64_t n, const uint32_t* sums, int64_t* total) {
  __shared__ uint32_t span_total;
  uint32_t before = 0;
  for (int i = threadIdx.x; i < (int)blockIdx.x; i += kScanBlock) before += sums[i];
  const uint32_t base = blockIdx.x > 0 ? block_sum(before) : 0u;
  const int64_t first = (int64_t)blockIdx.x * kScanSpan + (int64_t)threadIdx.x * kScanPer;
  uint32_t v[kScanPer];
  uint32_t mine = 0;
#pragma unroll
  for (int j = 0; j < kScanPer; ++j) {
    v[j] = first + j < n ? in[first + j] : 0u;
    mine += v[j];
  }
  uint32_t run = base + block_exclusive_scan(mine, &span_total);
#pragma unroll
  for (int j = 0; j < kScanPer; ++j) {
    if (first + j < n) out[first + j] = run;
    run += v[j];
  }
  if (total && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) *total = (int64_t)base + (int64_t)span_total;
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
  const int64_t spans = (n + kScanSpan - 1) / kScanSpan;
  if (spans <= kScanDirectSpans) {
    // the span sums live where the recursive form keeps its level-1 block sums (that array is four times as long)
    uint32_t* sums = reinterpret_cast<uint32_t*>(static_cast<char*>(tmp) + align_up(4, 256));
    if (spans > 1) { scan_span_sums_kernel<<<(unsigned)spans, kScanBlock, 0, stream>>>(in, n, sums); note_launches(1); }
    scan_spans_kernel<<<(unsigned)spans, kScanBlock, 0, stream>>>(in, out, n, sums, total);
    note_launches(1);
    return check_launch("scan");
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
