// Coordinate hash table: clear, build (insert) and query.
//
// Open addressing with linear probing over two arrays (keys int64, vals int32).  The key is the
// exact packed coordinate, so two different coordinates never alias.  One thread serves one
// coordinate; its probe sequence walks consecutive slots, i.e. stays inside one or two 32-byte
// sectors of the key array for the load factors used (<= 0.67).
#include "common.cuh"

namespace st {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
hash_clear_kernel(unsigned long long* keys, int32_t* vals, int64_t capacity) {
  // two slots per thread so that key stores are 16 bytes wide
  int64_t i = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * 2;
  if (i + 1 < capacity && (reinterpret_cast<uintptr_t>(keys) & 15) == 0) {
    reinterpret_cast<ulonglong2*>(keys)[i >> 1] = make_ulonglong2(kEmptyKey, kEmptyKey);
    vals[i] = -1;
    vals[i + 1] = -1;
  } else {
    for (int64_t j = i; j < capacity && j < i + 2; ++j) {
      keys[j] = kEmptyKey;
      vals[j] = -1;
    }
  }
}

// Two coordinates per thread, their probes interleaved: an insert is a chain of dependent round trips to L2 (the
// claim, then on a collision the next slot), and the kernel is bound by that latency, not by bytes.  The first probe
// of a key is the compare-and-swap itself -- at the load factors used most home slots are still empty, and a plain
// load first would only add a round trip.
template <typename CT>
__global__ void __launch_bounds__(kThreads)
hash_build_kernel(const CT* __restrict__ coords, int64_t n, unsigned long long* keys, int32_t* vals,
                  uint32_t capacity, uint32_t mask, int32_t* status) {
  constexpr int kPer = 2;
  const int64_t i0 = (int64_t)blockIdx.x * (kThreads * kPer) + threadIdx.x;
  unsigned long long key[kPer];
  uint32_t slot[kPer];
  bool live[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int64_t i = i0 + (int64_t)j * kThreads;
    live[j] = i < n;
    key[j] = 0;
    slot[j] = 0;
    if (!live[j]) continue;
    const int4 c = load_coord<CT>(coords, i);
    if (!key_representable(c.x, c.y, c.z, c.w)) {
      // a negative value or one above 65535 has no key of its own (it would alias another cell's): the
      // row is left out of the table, where st_hash_query could never return it anyway
      atomicOr(status, ST_DEV_BAD_INDEX);
      live[j] = false;
      continue;
    }
    key[j] = pack_key(c.x, c.y, c.z, c.w);
    slot[j] = home_slot(key[j], capacity, mask);
  }
  for (uint32_t step = 0; step < capacity && (live[0] || live[1]); ++step) {
    unsigned long long seen[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j)
      if (live[j]) seen[j] = atomicCAS(keys + slot[j], kEmptyKey, key[j]);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      if (!live[j]) continue;
      if (seen[j] == kEmptyKey || seen[j] == key[j]) {
        atomicMax(vals + slot[j], (int32_t)(i0 + (int64_t)j * kThreads));  // repeated coordinate: largest row stays
        live[j] = false;
      } else {
        slot[j] = next_slot(slot[j], capacity);
      }
    }
  }
  if (live[0] || live[1]) atomicOr(status, ST_DEV_TABLE_FULL);
}

template <typename CT>
__global__ void __launch_bounds__(kThreads)
hash_query_kernel(const CT* __restrict__ coords, int64_t m, Table table, int32_t* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= m) return;
  int4 c = load_coord<CT>(coords, i);
  int32_t r = -1;
  if (table.capacity != 0 && key_representable(c.x, c.y, c.z, c.w))
    r = table_find(table, pack_key(c.x, c.y, c.z, c.w));
  out[i] = r;
}

// q[row] = coordinate stored in the table for that row (int32 x 4); rows absent from the table keep
// batch = -1.  Recovers per-row coordinates from a table when only the table is at hand.
__global__ void __launch_bounds__(kThreads)
table_rows_init_kernel(int4* q, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < n) q[i] = make_int4(-1, 0, 0, 0);
}

__global__ void __launch_bounds__(kThreads)
table_unpack_kernel(const unsigned long long* __restrict__ keys, const int32_t* __restrict__ vals, int64_t capacity,
                    int4* q, int64_t n) {
  int64_t s = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (s >= capacity) return;
  const unsigned long long k = keys[s];
  const int32_t v = vals[s];
  if (k == kEmptyKey || v < 0 || v >= n) return;
  q[v] = make_int4((int)(k >> 48), (int)((k >> 32) & 0xFFFF), (int)((k >> 16) & 0xFFFF), (int)(k & 0xFFFF));
}

int unpack_table_coords(const int64_t* keys, const int32_t* vals, int64_t capacity, int32_t* q, int64_t n,
                        cudaStream_t stream) {
  if (n > 0) {
    table_rows_init_kernel<<<(unsigned)((n + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
        reinterpret_cast<int4*>(q), n);
    note_launches(1);
  }
  if (n > 0 && capacity > 0) {
    table_unpack_kernel<<<(unsigned)((capacity + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
        reinterpret_cast<const unsigned long long*>(keys), vals, capacity, reinterpret_cast<int4*>(q), n);
    note_launches(1);
  }
  return check_launch("unpack_table_coords");
}

}  // namespace st

using namespace st;

extern "C" {

int st_hash_clear(int64_t* keys, int32_t* vals, int64_t capacity, void* stream) {
  if (capacity < 0 || (capacity > 0 && (!keys || !vals))) {
    set_error("st_hash_clear: bad arguments");
    return ST_ERR_ARG;
  }
  if (capacity == 0) return ST_OK;
  int64_t threads = (capacity + 1) / 2;
  { hash_clear_kernel<<<(unsigned)((threads + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<unsigned long long*>(keys), vals, capacity); note_launches(1); }
  return check_launch("st_hash_clear");
}

int st_hash_build(const void* coords, int64_t n, int coord_dtype, int64_t* keys, int32_t* vals, int64_t capacity,
                  int32_t* status, void* stream) {
  if (n < 0 || capacity < 0 || capacity > 0x7FFFFFFFll || n > 0x7FFFFFFFll || !status ||
      (n > 0 && (!coords || !keys || !vals))) {
    set_error("st_hash_build: bad arguments");
    return ST_ERR_ARG;
  }
  if (n == 0) return ST_OK;
  if (capacity < n) {
    set_error("st_hash_build: capacity %lld < number of keys %lld", (long long)capacity, (long long)n);
    return ST_ERR_ARG;
  }
  Table t = make_table(keys, vals, capacity);
  unsigned grid = (unsigned)((n + 2 * kThreads - 1) / (2 * kThreads));          // two coordinates per thread
  auto* k = reinterpret_cast<unsigned long long*>(keys);
  if (coord_dtype == ST_I32)
    { hash_build_kernel<int32_t><<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const int32_t*>(coords), n, k, vals, t.capacity, t.mask, status); note_launches(1); }
  else if (coord_dtype == ST_I16)
    { hash_build_kernel<int16_t><<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const int16_t*>(coords), n, k, vals, t.capacity, t.mask, status); note_launches(1); }
  else {
    set_error("st_hash_build: unknown coordinate dtype %d", coord_dtype);
    return ST_ERR_DTYPE;
  }
  return check_launch("st_hash_build");
}

int st_hash_query(const void* coords, int64_t m, int coord_dtype, const int64_t* keys, const int32_t* vals,
                  int64_t capacity, int32_t* out, void* stream) {
  if (m < 0 || capacity < 0 || capacity > 0x7FFFFFFFll || (m > 0 && (!coords || !out)) ||
      (capacity > 0 && (!keys || !vals))) {
    set_error("st_hash_query: bad arguments");
    return ST_ERR_ARG;
  }
  if (m == 0) return ST_OK;
  Table t = make_table(keys, vals, capacity);
  unsigned grid = (unsigned)((m + kThreads - 1) / kThreads);
  if (coord_dtype == ST_I32)
    { hash_query_kernel<int32_t><<<grid, kThreads, 0, (cudaStream_t)stream>>>(static_cast<const int32_t*>(coords), m,
                                                                           t, out); note_launches(1); }
  else if (coord_dtype == ST_I16)
    { hash_query_kernel<int16_t><<<grid, kThreads, 0, (cudaStream_t)stream>>>(static_cast<const int16_t*>(coords), m,
                                                                           t, out); note_launches(1); }
  else {
    set_error("st_hash_query: unknown coordinate dtype %d", coord_dtype);
    return ST_ERR_DTYPE;
  }
  return check_launch("st_hash_query");
}

}  // extern "C"
