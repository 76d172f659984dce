// Kernel-map construction: output coordinates of strided / transposed convolutions, the dense
// output-stationary neighbour map, its inverse, and its compaction into (in, out, offset) triples.
//
// All kernels enumerate the flat index t = row * K + k with one thread per t, so a warp sweeps the
// offsets of one or two voxels, coordinate loads are warp-wide broadcasts and every write of the
// (rows, K) tables is coalesced.  Order-defining steps (which duplicate survives, where a row
// lands) are functions of t only, so results do not depend on scheduling.
#include "common.cuh"

namespace st {

constexpr int kBlock = 1024;  // = scan block, 32 warps

// Candidate output coordinate of input c under offset k; false if filtered out.
__device__ __forceinline__ bool candidate(const int4& c, const Offsets& off, int k, int stride, bool transposed,
                                          const Int3& new_shape, Int3* v) {
  int o[3] = {off.v[k * 3 + 0], off.v[k * 3 + 1], off.v[k * 3 + 2]};
  int in[3] = {c.y, c.z, c.w};
  int out[3];
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    if (transposed) {
      out[a] = in[a] * stride + o[a];
    } else {
      int t = in[a] + o[a];
      if (stride > 1) {
        // floor division / non-negative remainder, as Python's // and % on integers
        int q = t / stride;
        int r = t - q * stride;
        if (r != 0) return false;
        out[a] = q;
      } else {
        out[a] = t;
      }
    }
  }
  if (out[0] < 0 || out[0] >= new_shape.x || out[1] < 0 || out[1] >= new_shape.y || out[2] < 0 ||
      out[2] >= new_shape.z)
    return false;
  v->x = out[0];
  v->y = out[1];
  v->z = out[2];
  return true;
}

struct OutCoordsWorkspace {
  unsigned long long* keys;  // scratch table keys
  uint32_t* min_flat;        // smallest flat candidate index per key
  uint32_t* win_bits;        // one ballot word per warp of candidates
  uint32_t* block_counts;    // winners per block, then exclusive offsets
  void* scan_tmp;
  uint32_t capacity;         // power of two
  int64_t n_flat;
  int64_t n_blocks;
};

static int64_t scratch_capacity(int64_t n, int K, int stride, int transposed) {
  // candidates that can pass the stride filter per input: ceil(ks/stride)^3 <= K; use K when unknown
  int64_t per_input = K;
  if (!transposed && stride > 1) {
    int ks = 1;
    while (ks * ks * ks < K) ++ks;
    int64_t c = (ks + stride - 1) / stride;
    per_input = c * c * c;
  }
  int64_t want = 2 * n * per_input;
  int64_t cap = 1024;
  while (cap < want) cap <<= 1;
  return cap;
}

static bool carve(void* workspace, int64_t bytes, int64_t n, int K, int stride, int transposed,
                  OutCoordsWorkspace* w) {
  int64_t cap = scratch_capacity(n, K, stride, transposed);
  int64_t n_flat = n * K;
  int64_t n_blocks = (n_flat + kBlock - 1) / kBlock;
  char* p = static_cast<char*>(workspace);
  char* end = p + bytes;
  w->keys = reinterpret_cast<unsigned long long*>(p);
  p += align_up(cap * 8, 256);
  w->min_flat = reinterpret_cast<uint32_t*>(p);
  p += align_up(cap * 4, 256);
  w->win_bits = reinterpret_cast<uint32_t*>(p);
  p += align_up(n_blocks * (kBlock / 32) * 4, 256);
  w->block_counts = reinterpret_cast<uint32_t*>(p);
  p += align_up(n_blocks * 4, 256);
  w->scan_tmp = p;
  p += scan_tmp_bytes(n_blocks);
  w->capacity = (uint32_t)cap;
  w->n_flat = n_flat;
  w->n_blocks = n_blocks;
  return p <= end && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0;
}

__global__ void __launch_bounds__(256)
scratch_clear_kernel(unsigned long long* keys, uint32_t* min_flat, uint32_t capacity) {
  uint32_t i = blockIdx.x * 256u + threadIdx.x;
  if (i < capacity) {
    keys[i] = kEmptyKey;
    min_flat[i] = 0xFFFFFFFFu;
  }
}

// Pass A: insert every surviving candidate, keep the smallest flat index per coordinate.
template <typename CT>
__global__ void __launch_bounds__(kBlock)
outcoords_insert_kernel(const CT* __restrict__ coords, int64_t n_flat, int K, Offsets off, int stride,
                        bool transposed, Int3 new_shape, unsigned long long* keys, uint32_t* min_flat,
                        uint32_t capacity, int32_t* status) {
  int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  if (t >= n_flat) return;
  uint32_t row = (uint32_t)(t / K);
  int k = (int)(t - (int64_t)row * K);
  int4 c = load_coord<CT>(coords, row);
  Int3 v;
  if (!candidate(c, off, k, stride, transposed, new_shape, &v)) return;
  unsigned long long key = pack_key(c.x, v.x, v.y, v.z);
  uint32_t mask = capacity - 1;
  uint32_t slot = mix_key(key) & mask;
  for (uint32_t step = 0; step < capacity; ++step) {
    unsigned long long seen = keys[slot];
    if (seen == kEmptyKey) seen = atomicCAS(keys + slot, kEmptyKey, key);
    if (seen == kEmptyKey || seen == key) {
      atomicMin(min_flat + slot, (uint32_t)t);
      return;
    }
    slot = (slot + 1) & mask;
  }
  atomicOr(status, ST_DEV_TABLE_FULL);
}

// Pass B: a candidate wins if it holds the smallest flat index of its coordinate.
template <typename CT>
__global__ void __launch_bounds__(kBlock)
outcoords_mark_kernel(const CT* __restrict__ coords, int64_t n_flat, int K, Offsets off, int stride,
                      bool transposed, Int3 new_shape, const unsigned long long* __restrict__ keys,
                      const uint32_t* __restrict__ min_flat, uint32_t capacity, uint32_t* win_bits,
                      uint32_t* block_counts) {
  int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  bool win = false;
  if (t < n_flat) {
    uint32_t row = (uint32_t)(t / K);
    int k = (int)(t - (int64_t)row * K);
    int4 c = load_coord<CT>(coords, row);
    Int3 v;
    if (candidate(c, off, k, stride, transposed, new_shape, &v)) {
      unsigned long long key = pack_key(c.x, v.x, v.y, v.z);
      uint32_t mask = capacity - 1;
      uint32_t slot = mix_key(key) & mask;
      for (uint32_t step = 0; step < capacity; ++step) {
        unsigned long long seen = keys[slot];
        if (seen == key) {
          win = (min_flat[slot] == (uint32_t)t);
          break;
        }
        if (seen == kEmptyKey) break;  // cannot happen after pass A unless the table overflowed
        slot = (slot + 1) & mask;
      }
    }
  }
  uint32_t bits = __ballot_sync(0xFFFFFFFFu, win);
  if ((threadIdx.x & 31) == 0) win_bits[(int64_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5)] = bits;
  int total = __syncthreads_count(win);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = (uint32_t)total;
}

// Pass C: winners write their coordinate at (block offset + rank inside the block).
template <typename CT>
__global__ void __launch_bounds__(kBlock)
outcoords_write_kernel(const CT* __restrict__ coords, int64_t n_flat, int K, Offsets off, int stride,
                       bool transposed, Int3 new_shape, const uint32_t* __restrict__ win_bits,
                       const uint32_t* __restrict__ block_offsets, CT* out, int64_t out_capacity,
                       int32_t* status) {
  __shared__ uint32_t warp_offset[kBlock / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t bits = win_bits[(int64_t)blockIdx.x * (kBlock / 32) + warp];
  if (warp == 0) {
    uint32_t cnt = __popc(win_bits[(int64_t)blockIdx.x * (kBlock / 32) + lane]);
    uint32_t incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t x = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += x;
    }
    warp_offset[lane] = incl - cnt;
  }
  __syncthreads();
  if (!((bits >> lane) & 1u)) return;
  int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  int64_t dst = (int64_t)block_offsets[blockIdx.x] + warp_offset[warp] + __popc(bits & ((1u << lane) - 1u));
  if (dst >= out_capacity) {
    atomicOr(status, ST_DEV_OUT_OVERFLOW);
    return;
  }
  uint32_t row = (uint32_t)(t / K);
  int k = (int)(t - (int64_t)row * K);
  int4 c = load_coord<CT>(coords, row);
  Int3 v;
  candidate(c, off, k, stride, transposed, new_shape, &v);
  store_coord<CT>(out, dst, c.x, v.x, v.y, v.z);
}

// nbr[o,k] = row of (b, out*stride - off[k]) or -1.
template <typename CT>
__global__ void __launch_bounds__(256)
map_build_kernel(const CT* __restrict__ out_coords, int64_t n_flat, int K, Offsets off, int stride, Int3 shape,
                 Table table, int32_t* __restrict__ nbr) {
  int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= n_flat) return;
  int64_t row = t / K;
  int k = (int)(t - row * K);
  int4 c = load_coord<CT>(out_coords, row);
  int x = c.y * stride - off.v[k * 3 + 0];
  int y = c.z * stride - off.v[k * 3 + 1];
  int z = c.w * stride - off.v[k * 3 + 2];
  int32_t r = -1;
  if (x >= 0 && x < shape.x && y >= 0 && y < shape.y && z >= 0 && z < shape.z && table.capacity != 0 &&
      key_representable(c.x, x, y, z))
    r = table_find(table, pack_key(c.x, x, y, z));
  nbr[t] = r;
}

__global__ void __launch_bounds__(256) fill_i32_kernel(int32_t* p, int64_t n, int32_t v) {
  int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i < n) p[i] = v;
}

__global__ void __launch_bounds__(256)
map_invert_kernel(const int32_t* __restrict__ nbr, int64_t n_flat, int K, int64_t n_in, int32_t* inv) {
  int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= n_flat) return;
  int32_t i = nbr[t];
  if (i < 0 || i >= n_in) return;
  int64_t o = t / K;
  int k = (int)(t - o * K);
  inv[(int64_t)i * K + k] = (int32_t)o;
}

__global__ void __launch_bounds__(kBlock)
pairs_count_kernel(const int32_t* __restrict__ nbr, int64_t n_flat, uint32_t* block_counts) {
  int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  bool valid = t < n_flat && nbr[t] >= 0;
  int total = __syncthreads_count(valid);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = (uint32_t)total;
}

__global__ void __launch_bounds__(kBlock)
pairs_write_kernel(const int32_t* __restrict__ nbr, int64_t n_flat, int K, const uint32_t* __restrict__ block_offsets,
                   int32_t* triples, int64_t capacity, int32_t* status) {
  __shared__ uint32_t warp_offset[kBlock / 32];
  __shared__ uint32_t warp_count[kBlock / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  int32_t i = t < n_flat ? nbr[t] : -1;
  uint32_t bits = __ballot_sync(0xFFFFFFFFu, i >= 0);
  if (lane == 0) warp_count[warp] = __popc(bits);
  __syncthreads();
  if (warp == 0) {
    uint32_t cnt = warp_count[lane];
    uint32_t incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t x = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += x;
    }
    warp_offset[lane] = incl - cnt;
  }
  __syncthreads();
  if (i < 0) return;
  int64_t dst = (int64_t)block_offsets[blockIdx.x] + warp_offset[warp] + __popc(bits & ((1u << lane) - 1u));
  if (dst >= capacity) {
    atomicOr(status, ST_DEV_OUT_OVERFLOW);
    return;
  }
  int64_t o = t / K;
  triples[dst * 3 + 0] = i;
  triples[dst * 3 + 1] = (int32_t)o;
  triples[dst * 3 + 2] = (int32_t)(t - o * K);
}

template <typename CT>
static int outcoords_count_impl(const CT* coords, int64_t n, const Offsets& off, int K, int stride, bool transposed,
                                Int3 ns, OutCoordsWorkspace& w, int64_t* n_out, int32_t* status, cudaStream_t s) {
  { scratch_clear_kernel<<<(w.capacity + 255) / 256, 256, 0, s>>>(w.keys, w.min_flat, w.capacity); note_launches(1); }
  { outcoords_insert_kernel<CT><<<(unsigned)w.n_blocks, kBlock, 0, s>>>(coords, w.n_flat, K, off, stride, transposed,
                                                                      ns, w.keys, w.min_flat, w.capacity, status); note_launches(1); }
  { outcoords_mark_kernel<CT><<<(unsigned)w.n_blocks, kBlock, 0, s>>>(coords, w.n_flat, K, off, stride, transposed, ns,
                                                                    w.keys, w.min_flat, w.capacity, w.win_bits,
                                                                    w.block_counts); note_launches(1); }
  int rc = check_launch("st_outcoords_count");
  if (rc != ST_OK) return rc;
  return exclusive_scan_u32(w.block_counts, w.block_counts, w.n_blocks, w.scan_tmp, n_out, s);
}

}  // namespace st

using namespace st;

static int outcoords_args(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K,
                          int stride, const int32_t* new_shape_host, void* workspace, int64_t workspace_bytes,
                          int transposed, Offsets* off, Int3* ns, OutCoordsWorkspace* w, const char* who) {
  if (n < 0 || K < 1 || K > ST_MAX_KVOL || stride < 1 || !offsets_host || !new_shape_host ||
      (n > 0 && (!coords || !workspace))) {
    set_error("%s: bad arguments", who);
    return ST_ERR_ARG;
  }
  if (coord_dtype != ST_I16 && coord_dtype != ST_I32) {
    set_error("%s: unknown coordinate dtype %d", who, coord_dtype);
    return ST_ERR_DTYPE;
  }
  if (n * (int64_t)K >= 0xFFFFFFFFll) {
    set_error("%s: n*K = %lld does not fit the 32-bit candidate index", who, (long long)(n * (int64_t)K));
    return ST_ERR_UNSUPPORTED;
  }
  if (!pack_offsets(offsets_host, K, off)) {
    set_error("%s: offset outside int16", who);
    return ST_ERR_UNSUPPORTED;
  }
  ns->x = new_shape_host[0];
  ns->y = new_shape_host[1];
  ns->z = new_shape_host[2];
  if (n > 0 && !carve(workspace, workspace_bytes, n, K, stride, transposed, w)) {
    set_error("%s: workspace too small or not 256-byte aligned", who);
    return ST_ERR_WORKSPACE;
  }
  return ST_OK;
}

extern "C" {

int64_t st_outcoords_workspace_bytes(int64_t n, int K, int stride, int transposed) {
  if (n <= 0 || K < 1) return 256;
  int64_t cap = scratch_capacity(n, K, stride, transposed);
  int64_t n_blocks = (n * K + kBlock - 1) / kBlock;
  return align_up(cap * 8, 256) + align_up(cap * 4, 256) + align_up(n_blocks * (kBlock / 32) * 4, 256) +
         align_up(n_blocks * 4, 256) + scan_tmp_bytes(n_blocks) + 256;
}

int st_outcoords_count(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K, int stride,
                       int transposed, const int32_t* new_shape_host, void* workspace, int64_t workspace_bytes,
                       int64_t* n_out, int32_t* status, void* stream) {
  Offsets off;
  Int3 ns;
  OutCoordsWorkspace w;
  if (!n_out || !status) {
    set_error("st_outcoords_count: null n_out/status");
    return ST_ERR_ARG;
  }
  int rc = outcoords_args(coords, n, coord_dtype, offsets_host, K, stride, new_shape_host, workspace,
                          workspace_bytes, transposed, &off, &ns, &w, "st_outcoords_count");
  if (rc != ST_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) return exclusive_scan_u32(nullptr, nullptr, 0, nullptr, n_out, s);
  if (coord_dtype == ST_I32)
    return outcoords_count_impl<int32_t>(static_cast<const int32_t*>(coords), n, off, K, stride, transposed != 0, ns,
                                         w, n_out, status, s);
  return outcoords_count_impl<int16_t>(static_cast<const int16_t*>(coords), n, off, K, stride, transposed != 0, ns, w,
                                       n_out, status, s);
}

int st_outcoords_write(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K, int stride,
                       int transposed, const int32_t* new_shape_host, void* workspace, int64_t workspace_bytes,
                       void* out_coords, int64_t out_capacity, int32_t* status, void* stream) {
  Offsets off;
  Int3 ns;
  OutCoordsWorkspace w;
  if (!status || out_capacity < 0 || (out_capacity > 0 && !out_coords)) {
    set_error("st_outcoords_write: bad output arguments");
    return ST_ERR_ARG;
  }
  int rc = outcoords_args(coords, n, coord_dtype, offsets_host, K, stride, new_shape_host, workspace,
                          workspace_bytes, transposed, &off, &ns, &w, "st_outcoords_write");
  if (rc != ST_OK) return rc;
  if (n == 0) return ST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (coord_dtype == ST_I32)
    { outcoords_write_kernel<int32_t><<<(unsigned)w.n_blocks, kBlock, 0, s>>>(
        static_cast<const int32_t*>(coords), w.n_flat, K, off, stride, transposed != 0, ns, w.win_bits,
        w.block_counts, static_cast<int32_t*>(out_coords), out_capacity, status); note_launches(1); }
  else
    { outcoords_write_kernel<int16_t><<<(unsigned)w.n_blocks, kBlock, 0, s>>>(
        static_cast<const int16_t*>(coords), w.n_flat, K, off, stride, transposed != 0, ns, w.win_bits,
        w.block_counts, static_cast<int16_t*>(out_coords), out_capacity, status); note_launches(1); }
  return check_launch("st_outcoords_write");
}

int st_map_build(const void* out_coords, int64_t n_out, int coord_dtype, const int32_t* offsets_host, int K,
                 int lookup_stride, const int32_t* lookup_shape_host, const int64_t* keys, const int32_t* vals,
                 int64_t capacity, int32_t* nbr, void* stream) {
  if (n_out < 0 || K < 1 || K > ST_MAX_KVOL || lookup_stride < 1 || !offsets_host || !lookup_shape_host ||
      capacity < 0 || capacity > 0x7FFFFFFFll || (n_out > 0 && (!out_coords || !nbr)) ||
      (capacity > 0 && (!keys || !vals))) {
    set_error("st_map_build: bad arguments");
    return ST_ERR_ARG;
  }
  Offsets off;
  if (!pack_offsets(offsets_host, K, &off)) {
    set_error("st_map_build: offset outside int16");
    return ST_ERR_UNSUPPORTED;
  }
  if (n_out == 0) return ST_OK;
  Int3 shape = {lookup_shape_host[0], lookup_shape_host[1], lookup_shape_host[2]};
  Table t = make_table(keys, vals, capacity);
  int64_t n_flat = n_out * K;
  unsigned grid = (unsigned)((n_flat + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (coord_dtype == ST_I32)
    { map_build_kernel<int32_t><<<grid, 256, 0, s>>>(static_cast<const int32_t*>(out_coords), n_flat, K, off,
                                                   lookup_stride, shape, t, nbr); note_launches(1); }
  else if (coord_dtype == ST_I16)
    { map_build_kernel<int16_t><<<grid, 256, 0, s>>>(static_cast<const int16_t*>(out_coords), n_flat, K, off,
                                                   lookup_stride, shape, t, nbr); note_launches(1); }
  else {
    set_error("st_map_build: unknown coordinate dtype %d", coord_dtype);
    return ST_ERR_DTYPE;
  }
  return check_launch("st_map_build");
}

int st_map_invert(const int32_t* nbr, int64_t n_out, int K, int64_t n_in, int32_t* inv, void* stream) {
  if (n_out < 0 || n_in < 0 || K < 1 || (n_out > 0 && !nbr) || (n_in > 0 && !inv)) {
    set_error("st_map_invert: bad arguments");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int64_t n_inv = n_in * K;
  if (n_inv > 0) { fill_i32_kernel<<<(unsigned)((n_inv + 255) / 256), 256, 0, s>>>(inv, n_inv, -1); note_launches(1); }
  int64_t n_flat = n_out * K;
  if (n_flat > 0 && n_in > 0)
    { map_invert_kernel<<<(unsigned)((n_flat + 255) / 256), 256, 0, s>>>(nbr, n_flat, K, n_in, inv); note_launches(1); }
  return check_launch("st_map_invert");
}

int64_t st_map_pairs_workspace_bytes(int64_t n_out, int K) {
  int64_t n_blocks = (n_out * K + kBlock - 1) / kBlock;
  if (n_blocks < 1) n_blocks = 1;
  return align_up(n_blocks * 4, 256) + scan_tmp_bytes(n_blocks) + 256;
}

int st_map_pairs_count(const int32_t* nbr, int64_t n_out, int K, void* workspace, int64_t workspace_bytes,
                       int64_t* n_pairs, void* stream) {
  if (n_out < 0 || K < 1 || !n_pairs || (n_out > 0 && (!nbr || !workspace))) {
    set_error("st_map_pairs_count: bad arguments");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int64_t n_flat = n_out * K;
  if (n_flat == 0) return exclusive_scan_u32(nullptr, nullptr, 0, nullptr, n_pairs, s);
  if (workspace_bytes < st_map_pairs_workspace_bytes(n_out, K) || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("st_map_pairs_count: workspace too small or misaligned");
    return ST_ERR_WORKSPACE;
  }
  int64_t n_blocks = (n_flat + kBlock - 1) / kBlock;
  uint32_t* counts = static_cast<uint32_t*>(workspace);
  void* tmp = static_cast<char*>(workspace) + align_up(n_blocks * 4, 256);
  { pairs_count_kernel<<<(unsigned)n_blocks, kBlock, 0, s>>>(nbr, n_flat, counts); note_launches(1); }
  int rc = check_launch("st_map_pairs_count");
  if (rc != ST_OK) return rc;
  return exclusive_scan_u32(counts, counts, n_blocks, tmp, n_pairs, s);
}

int st_map_pairs_write(const int32_t* nbr, int64_t n_out, int K, void* workspace, int64_t workspace_bytes,
                       int32_t* triples, int64_t capacity, int32_t* status, void* stream) {
  if (n_out < 0 || K < 1 || !status || capacity < 0 || (capacity > 0 && !triples) ||
      (n_out > 0 && (!nbr || !workspace))) {
    set_error("st_map_pairs_write: bad arguments");
    return ST_ERR_ARG;
  }
  int64_t n_flat = n_out * K;
  if (n_flat == 0) return ST_OK;
  if (workspace_bytes < st_map_pairs_workspace_bytes(n_out, K)) {
    set_error("st_map_pairs_write: workspace too small");
    return ST_ERR_WORKSPACE;
  }
  int64_t n_blocks = (n_flat + kBlock - 1) / kBlock;
  { pairs_write_kernel<<<(unsigned)n_blocks, kBlock, 0, (cudaStream_t)stream>>>(
      nbr, n_flat, K, static_cast<const uint32_t*>(workspace), triples, capacity, status); note_launches(1); }
  return check_launch("st_map_pairs_write");
}

}  // extern "C"
