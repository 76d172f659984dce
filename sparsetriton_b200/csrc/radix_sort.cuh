// Stable LSD radix sort of (key, int32 value) pairs, 9-bit digits, keys of 32 or 64 bits.
//
// A block owns a contiguous tile of the sequence, each of its warps a contiguous chunk of the tile.
// A warp ranks its elements 32 at a time with match.any, which keeps equal digits in their original
// order; the warps of a block and the blocks of the grid are ordered by exclusive prefixes per digit
// value, so the result is deterministic (no atomics decide a position).  Per pass: a per-tile
// histogram, one exclusive prefix per digit value over the tiles, and the scatter.  The histogram
// matrix has one column per tile, not per warp: with 2048 elements per tile it is a quarter of the
// sequence's length.  Included by the translation units that sort (file-local kernels).
#pragma once

#include "common.cuh"

namespace st {
namespace {

constexpr int kSortPerLane = 8;                      // elements per lane
constexpr int kSortChunk = 32 * kSortPerLane;        // elements per warp
constexpr int kSortWarps = 8;                        // warps per block
constexpr int kSortTile = kSortWarps * kSortChunk;   // elements per block
constexpr int kDigitBitsMax = 9;
constexpr int kBucketsMax = 1 << kDigitBitsMax;

// hist[d * n_tiles + tile] = number of elements of the tile whose digit is d
template <typename KeyT>
__global__ void __launch_bounds__(kSortWarps * 32) sort_hist_kernel(const KeyT* __restrict__ keys, int64_t n,
                                                                   int shift, int bits, int64_t n_tiles,
                                                                   uint32_t* __restrict__ hist) {
  __shared__ uint32_t count[kBucketsMax];
  constexpr int T = kSortWarps * 32;
  const int buckets = 1 << bits;
  for (int d = threadIdx.x; d < buckets; d += T) count[d] = 0;
  __syncthreads();
  const int64_t begin = (int64_t)blockIdx.x * kSortTile, end = min(n, begin + kSortTile);
  for (int64_t i = begin + threadIdx.x; i < end; i += T)
    atomicAdd(&count[(uint32_t)(keys[i] >> shift) & (uint32_t)(buckets - 1)], 1u);
  __syncthreads();
  for (int d = threadIdx.x; d < buckets; d += T) hist[(int64_t)d * n_tiles + blockIdx.x] = count[d];
}

// One block per digit value d: hist[d * n_tiles + *] <- its exclusive prefix over the tiles,
// totals[d] <- the number of elements with that digit.
__global__ void __launch_bounds__(256) sort_bucket_scan_kernel(uint32_t* __restrict__ hist, int64_t n_tiles,
                                                              uint32_t* __restrict__ totals) {
  __shared__ uint32_t warp_sum[8];
  __shared__ uint32_t carry_s;
  uint32_t* row = hist + (int64_t)blockIdx.x * n_tiles;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < n_tiles; base += 256) {
    const int64_t i = base + threadIdx.x;
    const uint32_t v = i < n_tiles ? row[i] : 0u;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t u = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += u;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    uint32_t before = carry_s;
    for (int w = 0; w < warp; ++w) before += warp_sum[w];
    if (i < n_tiles) row[i] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == 255) carry_s = before + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = carry_s;
}

// Stable scatter of one digit pass: `prefix` is hist after sort_bucket_scan_kernel; the first output
// position of digit d is the sum of totals[0..d), which every block works out for itself.  The block
// keeps its elements in registers: it counts them per warp and digit, turns the counts into each
// warp's first output position per digit, and ranks.
template <typename KeyT>
__global__ void __launch_bounds__(kSortWarps * 32)
    sort_scatter_kernel(const KeyT* __restrict__ keys, const int32_t* __restrict__ vals, int64_t n, int shift,
                        int bits, int64_t n_tiles, const uint32_t* __restrict__ prefix,
                        const uint32_t* __restrict__ totals, KeyT* __restrict__ keys_out,
                        int32_t* __restrict__ vals_out) {
  constexpr int T = kSortWarps * 32;
  __shared__ uint32_t next[kSortWarps][kBucketsMax];
  __shared__ uint32_t base[kBucketsMax];
  __shared__ uint32_t part[kSortWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int buckets = 1 << bits;
  const uint32_t digit_mask = (uint32_t)(buckets - 1);
  for (int e = threadIdx.x; e < kSortWarps * kBucketsMax; e += T) (&next[0][0])[e] = 0;
  {
    // exclusive scan of totals[0..buckets) by the whole block: each thread owns a run of `per` digits
    constexpr int kPer = (kBucketsMax + T - 1) / T;
    const int per = (buckets + T - 1) / T;
    uint32_t mine[kPer];
    uint32_t sum = 0;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int d = threadIdx.x * per + i;
      mine[i] = (i < per && d < buckets) ? totals[d] : 0u;
      sum += mine[i];
    }
    uint32_t inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t u = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += u;
    }
    if (lane == 31) part[warp] = inc;
    __syncthreads();
    uint32_t before = inc - sum;
    for (int w = 0; w < warp; ++w) before += part[w];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int d = threadIdx.x * per + i;
      if (i < per && d < buckets) base[d] = before;
      before += mine[i];
    }
  }
  // this warp's elements, 32 consecutive ones per step, and their count per digit
  const int64_t begin = (int64_t)blockIdx.x * kSortTile + warp * kSortChunk;
  KeyT key[kSortPerLane];
  int32_t val[kSortPerLane];
  uint32_t digit[kSortPerLane];
#pragma unroll
  for (int j = 0; j < kSortPerLane; ++j) {
    const int64_t i = begin + j * 32 + lane;
    const bool live = i < n;
    key[j] = live ? keys[i] : (KeyT)0;
    val[j] = live ? vals[i] : 0;
    // lanes past the end get a digit of their own so that they never share a bucket with live ones
    digit[j] = live ? ((uint32_t)(key[j] >> shift) & digit_mask) : 0xFFFFFFFFu;
  }
  __syncthreads();                                       // next[][] cleared, base[] written
#pragma unroll
  for (int j = 0; j < kSortPerLane; ++j)
    if (digit[j] != 0xFFFFFFFFu) atomicAdd(&next[warp][digit[j]], 1u);
  __syncthreads();
  // next[w][d] <- first output position of warp w's elements of digit d
  for (int d = threadIdx.x; d < buckets; d += T) {
    uint32_t run = base[d] + prefix[(int64_t)d * n_tiles + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) {
      const uint32_t c = next[w][d];
      next[w][d] = run;
      run += c;
    }
  }
  __syncthreads();
  const uint32_t lower = (1u << lane) - 1u;
#pragma unroll
  for (int j = 0; j < kSortPerLane; ++j) {
    const uint32_t d = digit[j];
    const bool live = d != 0xFFFFFFFFu;
    const uint32_t peers = __match_any_sync(0xFFFFFFFFu, d);
    uint32_t first = 0;
    if (live) first = next[warp][d];
    __syncwarp();
    if (live && (peers & lower) == 0) next[warp][d] = first + (uint32_t)__popc(peers);
    __syncwarp();
    if (live) {
      const uint32_t dst = first + (uint32_t)__popc(peers & lower);
      keys_out[dst] = key[j];
      vals_out[dst] = val[j];
    }
  }
}

inline int64_t sort_tiles(int64_t n) { return n > 0 ? (n + kSortTile - 1) / kSortTile : 1; }
inline int sort_passes_for_bits(int key_bits) { return (key_bits + kDigitBitsMax - 1) / kDigitBitsMax; }
inline int64_t sort_hist_bytes(int64_t n) { return sort_tiles(n) * kBucketsMax * 4; }

// The digit passes over `key_bits` low bits of (keys_in, vals_in), ping-ponging with (keys_alt, vals_alt).
// After an odd number of passes the result is in the alt buffers, after an even number in the in buffers;
// the pointers to the sorted arrays are returned through *keys_sorted / *vals_sorted (either may be null).
template <typename KeyT>
void radix_sort_pairs(KeyT* keys_in, int32_t* vals_in, KeyT* keys_alt, int32_t* vals_alt, int64_t n, int key_bits,
                      uint32_t* hist, uint32_t* totals, KeyT** keys_sorted, int32_t** vals_sorted, cudaStream_t st) {
  const int passes = sort_passes_for_bits(key_bits);
  const int bits = (key_bits + passes - 1) / passes;
  const int64_t n_tiles = sort_tiles(n);
  const unsigned blocks = (unsigned)n_tiles;
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = pass * bits;
    sort_hist_kernel<KeyT><<<blocks, kSortWarps * 32, 0, st>>>(keys_in, n, shift, bits, n_tiles, hist);
    sort_bucket_scan_kernel<<<1u << bits, 256, 0, st>>>(hist, n_tiles, totals);
    sort_scatter_kernel<KeyT><<<blocks, kSortWarps * 32, 0, st>>>(keys_in, vals_in, n, shift, bits, n_tiles, hist, totals,
                                                                 keys_alt, vals_alt);
    note_launches(3);
    KeyT* tk = keys_in; keys_in = keys_alt; keys_alt = tk;
    int32_t* tv = vals_in; vals_in = vals_alt; vals_alt = tv;
  }
  if (keys_sorted) *keys_sorted = keys_in;
  if (vals_sorted) *vals_sorted = vals_in;
}

}  // namespace
}  // namespace st
