// Shared device helpers: coordinate loads, key packing, slot hashing, table probing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sparsetriton_b200.h"

namespace st {

constexpr unsigned long long kEmptyKey = 0xFFFFFFFFFFFFFFFFull;

// Sets the thread-local error text returned by st_last_error_string().
void set_error(const char* fmt, ...);
// Returns ST_OK or records the pending launch error and returns ST_ERR_CUDA.
int check_launch(const char* what);
// Adds n to the process-wide count of kernels this library has enqueued (st_launch_count()).
void note_launches(int n);

// Kernel offsets travel inside the launch parameters.
struct Offsets {
  int16_t v[ST_MAX_KVOL * 3];
};

// Fills an Offsets from a host (K,3) int32 array; returns false if a value does not fit int16.
bool pack_offsets(const int32_t* host, int K, Offsets* out);

struct Int3 {
  int x, y, z;
};

template <typename CT>
__device__ __forceinline__ int4 load_coord(const CT* base, int64_t row);

template <>
__device__ __forceinline__ int4 load_coord<int32_t>(const int32_t* base, int64_t row) {
  return __ldg(reinterpret_cast<const int4*>(base) + row);
}
template <>
__device__ __forceinline__ int4 load_coord<int16_t>(const int16_t* base, int64_t row) {
  short4 s = __ldg(reinterpret_cast<const short4*>(base) + row);
  return make_int4(s.x, s.y, s.z, s.w);
}

template <typename CT>
__device__ __forceinline__ void store_coord(CT* base, int64_t row, int b, int x, int y, int z);
template <>
__device__ __forceinline__ void store_coord<int32_t>(int32_t* base, int64_t row, int b, int x, int y, int z) {
  reinterpret_cast<int4*>(base)[row] = make_int4(b, x, y, z);
}
template <>
__device__ __forceinline__ void store_coord<int16_t>(int16_t* base, int64_t row, int b, int x, int y, int z) {
  reinterpret_cast<short4*>(base)[row] = make_short4((short)b, (short)x, (short)y, (short)z);
}

// batch<<48 | x<<32 | y<<16 | z, each field truncated to 16 bits.
__host__ __device__ __forceinline__ unsigned long long pack_key(int b, int x, int y, int z) {
  return ((unsigned long long)(uint16_t)b << 48) | ((unsigned long long)(uint16_t)x << 32) |
         ((unsigned long long)(uint16_t)y << 16) | (unsigned long long)(uint16_t)z;
}

__host__ __device__ __forceinline__ bool key_representable(int b, int x, int y, int z) {
  return ((unsigned)b | (unsigned)x | (unsigned)y | (unsigned)z) <= 0xFFFFu;
}

// 64 -> 32 bit mixer (two multiply/xor-shift rounds).
__host__ __device__ __forceinline__ uint32_t mix_key(unsigned long long k) {
  k *= 0x9E3779B97F4A7C15ull;
  k ^= k >> 32;
  k *= 0xD6E8FEB86659FD93ull;
  k ^= k >> 32;
  return (uint32_t)k;
}

// View of an open-addressing table.  mask = capacity-1 when capacity is a power of two, else 0.
struct Table {
  const unsigned long long* keys;
  const int32_t* vals;
  uint32_t capacity;
  uint32_t mask;
};

__host__ __device__ __forceinline__ uint32_t home_slot(unsigned long long key, uint32_t capacity, uint32_t mask) {
  uint32_t h = mix_key(key);
  return mask ? (h & mask) : (h % capacity);
}

__host__ __device__ __forceinline__ uint32_t next_slot(uint32_t slot, uint32_t capacity) {
  ++slot;
  return slot == capacity ? 0u : slot;
}

// Row index stored for key, or -1.  Linear probing; stops at the first empty slot.
__device__ __forceinline__ int32_t table_find(const Table& t, unsigned long long key) {
  uint32_t slot = home_slot(key, t.capacity, t.mask);
  for (uint32_t step = 0; step < t.capacity; ++step) {
    unsigned long long k = __ldg(t.keys + slot);
    if (k == key) return __ldg(t.vals + slot);
    if (k == kEmptyKey) return -1;
    slot = next_slot(slot, t.capacity);
  }
  return -1;
}

inline Table make_table(const int64_t* keys, const int32_t* vals, int64_t capacity) {
  Table t;
  t.keys = reinterpret_cast<const unsigned long long*>(keys);
  t.vals = vals;
  t.capacity = (uint32_t)capacity;
  t.mask = (capacity > 0 && (capacity & (capacity - 1)) == 0) ? (uint32_t)(capacity - 1) : 0u;
  return t;
}

// q (n,4) int32 <- coordinates stored in the table, by row; absent rows get batch -1.
int unpack_table_coords(const int64_t* keys, const int32_t* vals, int64_t capacity, int32_t* q, int64_t n,
                        cudaStream_t stream);

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Exclusive prefix sum of n uint32 values (in != out allowed, in == out allowed); *total (device
// or pinned host, may be null) receives the sum as int64.  tmp must hold scan_tmp_bytes(n).
int64_t scan_tmp_bytes(int64_t n);
int exclusive_scan_u32(const uint32_t* in, uint32_t* out, int64_t n, void* tmp, int64_t* total, cudaStream_t stream);

}  // namespace st
