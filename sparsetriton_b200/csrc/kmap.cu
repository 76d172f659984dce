// Kernel-map construction: output coordinates of strided / transposed convolutions, the dense
// output-stationary neighbour map, its inverse, and its compaction into (in, out, offset) triples.
//
// The map kernels enumerate the flat index t = row * K + k with one thread per t, so a warp sweeps
// the offsets of one or two voxels, coordinate loads are warp-wide broadcasts and every write of the
// (rows, K) tables is coalesced; the output-coordinate kernels give each input row one thread that
// loops over its K offsets.  Order-defining steps (which duplicate survives, where a row lands) are
// functions of t only, so results do not depend on scheduling.
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

// One axis of candidate(): output coordinate of input coordinate `in` under axis offset `o`.
__device__ __forceinline__ bool axis_candidate(int in, int o, int stride, bool transposed, int extent, int* out) {
  int v;
  if (transposed) {
    v = in * stride + o;
  } else {
    const int t = in + o;
    if (stride == 2) {                                      // the usual stride: no division
      if (t & 1) return false;
      v = t >> 1;
    } else if (stride > 1) {
      const int q = t / stride;
      if (t - q * stride != 0) return false;
      v = q;
    } else {
      v = t;
    }
  }
  *out = v;
  return v >= 0 && v < extent;
}

// f(k, v) for every offset k of input c that passes candidate(), in ascending k.  KS = 0 walks all K
// offsets.  KS > 0 requires the offsets to be the product grid k = (ix * KS + iy) * KS + iz (what every
// cubic kernel gives): the filters are then separable, so each axis is evaluated KS times instead of
// KS^3 times and only the surviving combinations are visited (8 of 27 at most for a stride-2 k3 layer).
// These sweeps were bound by instruction issue (ncu: SM throughput 62-71 %, DRAM 3-25 %).
// Per axis of a product grid of offsets: the offsets that pass axis_candidate(), compacted to the front (output
// coordinate and offset index), and how many there are.
template <int KS>
struct AxisLists {
  int vx[KS], vy[KS], vz[KS], jx[KS], jy[KS], jz[KS];
  int nx, ny, nz;
};

template <int KS>
__device__ __forceinline__ void axis_lists(const int4& c, const Offsets& off, int stride, bool transposed,
                                           const Int3& new_shape, AxisLists<KS>& a) {
  a.nx = a.ny = a.nz = 0;
#pragma unroll
  for (int j = 0; j < KS; ++j) {
    int v;
    if (axis_candidate(c.y, off.v[(j * KS * KS) * 3 + 0], stride, transposed, new_shape.x, &v)) {
#pragma unroll
      for (int q = 0; q < KS; ++q)
        if (q == a.nx) {
          a.vx[q] = v;
          a.jx[q] = j;
        }
      ++a.nx;
    }
    if (axis_candidate(c.z, off.v[(j * KS) * 3 + 1], stride, transposed, new_shape.y, &v)) {
#pragma unroll
      for (int q = 0; q < KS; ++q)
        if (q == a.ny) {
          a.vy[q] = v;
          a.jy[q] = j;
        }
      ++a.ny;
    }
    if (axis_candidate(c.w, off.v[j * 3 + 2], stride, transposed, new_shape.z, &v)) {
#pragma unroll
      for (int q = 0; q < KS; ++q)
        if (q == a.nz) {
          a.vz[q] = v;
          a.jz[q] = j;
        }
      ++a.nz;
    }
  }
}

template <int KS>
__device__ __forceinline__ int pick(const int (&a)[KS], int i) {
  int r = a[0];
#pragma unroll
  for (int q = 1; q < KS; ++q) r = (i == q) ? a[q] : r;
  return r;
}

template <int KS, typename F>
__device__ __forceinline__ void for_each_candidate(const int4& c, const Offsets& off, int K, int stride, bool transposed,
                                                   const Int3& new_shape, F&& f) {
  if constexpr (KS == 0) {
    for (int k = 0; k < K; ++k) {
      Int3 v;
      if (candidate(c, off, k, stride, transposed, new_shape, &v)) f(k, v);
    }
  } else {
    // The three loops below run over this thread's own candidates only -- at most ceil(KS / stride) per axis --
    // where a sweep over all KS^3 combinations makes a warp walk every combination that any of its lanes needs
    // (all 27 of a stride-2 k3 layer, of which a lane uses 3.4 on average).
    AxisLists<KS> a;
    axis_lists<KS>(c, off, stride, transposed, new_shape, a);
#pragma unroll 1
    for (int ax = 0; ax < a.nx; ++ax) {
      const int x = pick<KS>(a.vx, ax), ix = pick<KS>(a.jx, ax);
#pragma unroll 1
      for (int ay = 0; ay < a.ny; ++ay) {
        const int y = pick<KS>(a.vy, ay), iy = pick<KS>(a.jy, ay);
#pragma unroll 1
        for (int az = 0; az < a.nz; ++az) f((ix * KS + iy) * KS + pick<KS>(a.jz, az), Int3{x, y, pick<KS>(a.vz, az)});
      }
    }
  }
}

// The rows of a warp have 1 to 8 candidates each on a stride-2 k3 layer, 3.4 on average: with one row per lane a
// warp runs the body eight times at 42 % of its lanes.  Here every lane first lists its candidates (cell number,
// owner lane, offset) in a shared line of the warp, at the positions a prefix sum of the counts gives, and the warp
// then takes the listed candidates 32 at a time, one per lane: f(owner lane, k, cell).  For layers whose rows have at
// most kDensePerRow candidates (see dense_sweep_ok) and whose cell numbers fit 32 bits (kDirectMaxCells).  Every
// lane of the warp must call it; `live` says whether the lane has a row.
constexpr int kDensePerRow = 8;

template <typename F>
__device__ __forceinline__ void warp_dense_candidates(bool live, const int4& c, const Offsets& off, int stride,
                                                      const Int3& new_shape, uint2* line, F&& f) {
  const int lane = threadIdx.x & 31;
  AxisLists<3> a;
  a.nx = a.ny = a.nz = 0;
  if (live) axis_lists<3>(c, off, stride, false, new_shape, a);
  const int mine = a.nx * a.ny * a.nz;
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += u;
  }
  const int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
  int q = incl - mine;
#pragma unroll 1
  for (int ax = 0; ax < a.nx; ++ax) {
    const int x = pick<3>(a.vx, ax), ix = pick<3>(a.jx, ax);
#pragma unroll 1
    for (int ay = 0; ay < a.ny; ++ay) {
      const int y = pick<3>(a.vy, ay), iy = pick<3>(a.jy, ay);
      const int plane = ((c.x * new_shape.x + x) * new_shape.y + y) * new_shape.z;
#pragma unroll 1
      for (int az = 0; az < a.nz; ++az)
        line[q++] = make_uint2((uint32_t)(plane + pick<3>(a.vz, az)),
                               ((uint32_t)lane << 8) | (uint32_t)((ix * 3 + iy) * 3 + pick<3>(a.jz, az)));
    }
  }
  __syncwarp();
  for (int i = lane; i < total; i += 32) {
    const uint2 e = line[i];
    f((int)(e.y >> 8), (int)(e.y & 255u), e.x);
  }
  __syncwarp();
}

// Whether warp_dense_candidates() serves the layer: a cubic k3 product grid at stride 2, not transposed, whose
// offsets along an axis do not all share a parity (then at most two of the three pass the stride filter).
static bool dense_sweep_ok(const Offsets& off, int ks, int stride, bool transposed) {
  if (ks != 3 || stride != 2 || transposed) return false;
  for (int axis = 0; axis < 3; ++axis) {
    const int step = axis == 0 ? 9 : (axis == 1 ? 3 : 1);
    int odd = 0;
    for (int j = 0; j < 3; ++j) odd += off.v[(j * step) * 3 + axis] & 1;
    if (odd == 0 || odd == 3) return false;
  }
  return true;
}

// KS such that the K offsets are the product grid for_each_candidate<KS> expects (2 or 3), else 0.
static int product_kernel_size(const Offsets& off, int K) {
  for (int ks = 2; ks <= 3; ++ks) {
    if (ks * ks * ks != K) continue;
    bool ok = true;
    for (int k = 0; k < K && ok; ++k) {
      const int ix = k / (ks * ks), iy = (k / ks) % ks, iz = k % ks;
      ok = off.v[k * 3 + 0] == off.v[(ix * ks * ks) * 3 + 0] && off.v[k * 3 + 1] == off.v[(iy * ks) * 3 + 1] &&
           off.v[k * 3 + 2] == off.v[iz * 3 + 2];
    }
    if (ok) return ks;
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Output coordinates.  One thread per input row sweeps the K offsets of its row.
//
//   count   candidates that survive the stride / range filters -> scratch-table capacity, chosen ON
//           THE DEVICE as the power of two >= 1.5 x candidates (the host only reserves the worst case)
//   clear   that many 16-byte slots {key, smallest candidate index, output row} to all ones
//   insert  exact-key open addressing; atomicMin keeps the smallest flat index n*K+k per coordinate
//   mark    a candidate wins if it holds that smallest index; K win bits and a win count per row
//   scan    exclusive prefix sum of the per-row counts = first output row of each input row
//   write   winners store their coordinate (ordered by flat index) and leave their output row in the
//           table slot, so that the neighbour map can be produced by a scatter over the same
//           candidates instead of N_out*K probes of the input table (st_outcoords_map)
// ---------------------------------------------------------------------------------------------
constexpr int kRowThreads = 256;

struct OutCoordsHeader {                 // first 256 bytes of the workspace
  unsigned long long n_candidates;
  uint32_t capacity;                     // power of two
  uint32_t pad;
};

// One slot of the dedupe table: 16 bytes, so that a probe, the minimum of the candidate indices and the output
// row of the coordinate all live in one 32-byte sector (three separate arrays cost three sectors per candidate).
struct __align__(16) Slot {
  unsigned long long key;                // exact packed coordinate, all ones = empty
  uint32_t flat;                         // smallest flat candidate index n*K+k seen for the key
  uint32_t out_row;                      // output row of the coordinate (written by the `write` pass)
};

struct OutCoordsWorkspace {
  OutCoordsHeader* header;
  Slot* slots;                           // scratch table
  uint32_t* win_words;                   // (n, words) win bits of each input row
  uint32_t* row_counts;                  // wins per input row, then their exclusive prefix sum
  void* scan_tmp;
  int64_t capacity_max;                  // slots reserved (worst case)
  int words;                             // ceil(K / 32)
};

static int64_t scratch_capacity(int64_t n, int K, int stride, int transposed) {
  // candidates that can pass the stride filter per input: ceil(ks/stride)^3 <= K
  int64_t per_input = K;
  if (!transposed && stride > 1) {
    int ks = 1;
    while (ks * ks * ks < K) ++ks;
    int64_t c = (ks + stride - 1) / stride;
    per_input = c * c * c;
  }
  int64_t want = (3 * n * per_input + 1) / 2;
  int64_t cap = 1024;
  while (cap < want) cap <<= 1;
  return cap;
}

static int64_t outcoords_bytes(int64_t n, int K, int stride, int transposed) {
  const int64_t cap = scratch_capacity(n, K, stride, transposed);
  const int words = (K + 31) / 32;
  return 256 + align_up(cap * (int64_t)sizeof(Slot), 256) + align_up(n * words * 4, 256) + align_up(n * 4, 256) +
         scan_tmp_bytes(n) + 256;
}

static bool carve(void* workspace, int64_t bytes, int64_t n, int K, int stride, int transposed,
                  OutCoordsWorkspace* w) {
  const int64_t cap = scratch_capacity(n, K, stride, transposed);
  w->words = (K + 31) / 32;
  char* p = static_cast<char*>(workspace);
  char* end = p + bytes;
  w->header = reinterpret_cast<OutCoordsHeader*>(p);
  p += 256;
  w->slots = reinterpret_cast<Slot*>(p);
  p += align_up(cap * (int64_t)sizeof(Slot), 256);
  w->win_words = reinterpret_cast<uint32_t*>(p);
  p += align_up(n * w->words * 4, 256);
  w->row_counts = reinterpret_cast<uint32_t*>(p);
  p += align_up(n * 4, 256);
  w->scan_tmp = p;
  p += scan_tmp_bytes(n);
  w->capacity_max = cap;
  return p <= end && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0;
}

template <typename CT, int KS>
__global__ void __launch_bounds__(kRowThreads)
outcoords_count_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed,
                       Int3 new_shape, OutCoordsHeader* header) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  int cnt = 0;
  if (row < n) {
    const int4 c = load_coord<CT>(coords, row);
    for_each_candidate<KS>(c, off, K, stride, transposed, new_shape, [&](int, const Int3&) { ++cnt; });
  }
  // block sum -> one atomic per block
  __shared__ int warp_sum[kRowThreads / 32];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) cnt += __shfl_down_sync(0xFFFFFFFFu, cnt, d);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
    for (int i = 0; i < kRowThreads / 32; ++i) total += warp_sum[i];
    if (total) atomicAdd(&header->n_candidates, (unsigned long long)total);
  }
}

// Table capacity for the counted candidates: the power of two >= 1.5 x candidates, at most what was reserved.
__device__ __forceinline__ uint32_t capacity_for(unsigned long long n_candidates, unsigned long long capacity_max) {
  const unsigned long long want = (3 * n_candidates + 1) / 2;
  unsigned long long cap = 1024;
  while (cap < want && cap < capacity_max) cap <<= 1;
  return (uint32_t)cap;
}

// Chooses the capacity (every thread works it out from the candidate count; one thread records it for the
// kernels that follow) and clears that many slots: 16-byte stores of all ones.
__global__ void __launch_bounds__(256)
scratch_clear_kernel(OutCoordsHeader* header, unsigned long long capacity_max, Slot* slots) {
  const uint32_t capacity = capacity_for(header->n_candidates, capacity_max);
  if (blockIdx.x == 0 && threadIdx.x == 0) header->capacity = capacity;
  const uint4 empty = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
  for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < capacity; i += gridDim.x * 256u)
    reinterpret_cast<uint4*>(slots)[i] = empty;
}

// Records candidate index `flat` for `key`: finds or claims the key's slot and lowers the slot's index to `flat`.
// Capacity is a power of two.  Returns false when the table is full.
//
// Four out of five candidates of a strided layer are repeats of a coordinate another input has already
// produced, and they arrive roughly in ascending order of `flat`, so a repeat usually finds its key in place
// with a smaller index already stored: one 16-byte read (past L1, which may hold an old copy) and no atomic.
// A stale read can only show an empty slot that is taken by now (the compare-and-swap then returns the owner)
// or an index larger than the current one (the minimum is then applied needlessly): both are harmless.
__device__ __forceinline__ bool scratch_record(Slot* slots, uint32_t capacity, unsigned long long key, uint32_t flat) {
  const uint32_t mask = capacity - 1;
  uint32_t slot = mix_key(key) & mask;
  for (uint32_t step = 0; step < capacity; ++step) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(slots + slot));
    unsigned long long seen = (unsigned long long)v.x | ((unsigned long long)v.y << 32);
    if (seen == kEmptyKey) seen = atomicCAS(&slots[slot].key, kEmptyKey, key);
    else if (seen == key) {
      if (v.z > flat) atomicMin(&slots[slot].flat, flat);
      return true;
    }
    if (seen == kEmptyKey || seen == key) {
      atomicMin(&slots[slot].flat, flat);
      return true;
    }
    slot = (slot + 1) & mask;
  }
  return false;
}

// The slot holding `key` with its contents (one 16-byte load per probe), or index 0xFFFFFFFF.
struct Found {
  uint32_t slot, flat, out_row;
};
__device__ __forceinline__ Found scratch_find(const Slot* slots, uint32_t capacity, unsigned long long key) {
  const uint32_t mask = capacity - 1;
  uint32_t slot = mix_key(key) & mask;
  for (uint32_t step = 0; step < capacity; ++step) {
    const uint4 v = *reinterpret_cast<const uint4*>(slots + slot);
    const unsigned long long seen = (unsigned long long)v.x | ((unsigned long long)v.y << 32);
    if (seen == key) return Found{slot, v.z, v.w};
    if (seen == kEmptyKey) break;
    slot = (slot + 1) & mask;
  }
  return Found{0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
}

template <typename CT, int KS>
__global__ void __launch_bounds__(kRowThreads)
outcoords_insert_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed,
                        Int3 new_shape, const OutCoordsHeader* header, Slot* slots, int32_t* status) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  if (row >= n) return;
  const uint32_t capacity = header->capacity;
  const int4 c = load_coord<CT>(coords, row);
  const uint32_t flat0 = (uint32_t)row * (uint32_t)K;
  bool full = false;
  for_each_candidate<KS>(c, off, K, stride, transposed, new_shape, [&](int k, const Int3& v) {
    if (full) return;
    if (!scratch_record(slots, capacity, pack_key(c.x, v.x, v.y, v.z), flat0 + (uint32_t)k)) {
      atomicOr(status, ST_DEV_TABLE_FULL);
      full = true;
    }
  });
}

template <typename CT, int KS>
__global__ void __launch_bounds__(kRowThreads)
outcoords_mark_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed,
                      Int3 new_shape, const OutCoordsHeader* header, const Slot* slots, uint32_t* win_words, int words,
                      uint32_t* row_counts) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  if (row >= n) return;
  const uint32_t capacity = header->capacity;
  const int4 c = load_coord<CT>(coords, row);
  const uint32_t flat0 = (uint32_t)row * (uint32_t)K;
  uint32_t count = 0;
  if constexpr (KS == 0) {
    for (int w = 0; w < words; ++w) {
      uint32_t bits = 0;
      const int k_end = min(K, (w + 1) * 32);
      for (int k = w * 32; k < k_end; ++k) {
        Int3 v;
        if (!candidate(c, off, k, stride, transposed, new_shape, &v)) continue;
        const Found f = scratch_find(slots, capacity, pack_key(c.x, v.x, v.y, v.z));
        if (f.slot != 0xFFFFFFFFu && f.flat == flat0 + (uint32_t)k) bits |= 1u << (k & 31);
      }
      win_words[row * words + w] = bits;
      count += __popc(bits);
    }
  } else {
    uint32_t bits = 0;                                       // KS <= 3: a single word of win bits
    for_each_candidate<KS>(c, off, K, stride, transposed, new_shape, [&](int k, const Int3& v) {
      const Found f = scratch_find(slots, capacity, pack_key(c.x, v.x, v.y, v.z));
      if (f.slot != 0xFFFFFFFFu && f.flat == flat0 + (uint32_t)k) bits |= 1u << k;
    });
    win_words[row * words] = bits;
    count = __popc(bits);
  }
  row_counts[row] = count;
}

template <typename CT>
__global__ void __launch_bounds__(kRowThreads)
outcoords_write_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed,
                       Int3 new_shape, const OutCoordsHeader* header, Slot* slots,
                       const uint32_t* __restrict__ win_words, int words,
                       const uint32_t* __restrict__ row_offsets, CT* out, int64_t out_capacity, int32_t* status) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  if (row >= n) return;
  const uint32_t capacity = header->capacity;
  const int4 c = load_coord<CT>(coords, row);
  int64_t dst = row_offsets[row];
  for (int w = 0; w < words; ++w) {
    uint32_t bits = win_words[row * words + w];
    while (bits) {
      const int k = w * 32 + __ffs(bits) - 1;
      bits &= bits - 1;
      Int3 v;
      candidate(c, off, k, stride, transposed, new_shape, &v);
      if (dst >= out_capacity) {
        atomicOr(status, ST_DEV_OUT_OVERFLOW);
        return;
      }
      store_coord<CT>(out, dst, c.x, v.x, v.y, v.z);
      const Found f = scratch_find(slots, capacity, pack_key(c.x, v.x, v.y, v.z));
      if (f.slot != 0xFFFFFFFFu) slots[f.slot].out_row = (uint32_t)dst;      // the coordinate's output row
      ++dst;
    }
  }
}

// nbr[out_row(candidate), k] = max(input row): the neighbour map by scatter.  nbr must hold -1.
template <typename CT, int KS>
__global__ void __launch_bounds__(kRowThreads)
outcoords_map_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed,
                     Int3 new_shape, Int3 in_shape, const OutCoordsHeader* header, const Slot* slots, int32_t* nbr,
                     int64_t n_out) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  if (row >= n) return;
  const uint32_t capacity = header->capacity;
  const int4 c = load_coord<CT>(coords, row);
  // an input outside its own grid is never found by the bounds-checked lookup of the probing form
  if (c.y < 0 || c.y >= in_shape.x || c.z < 0 || c.z >= in_shape.y || c.w < 0 || c.w >= in_shape.z) return;
  for_each_candidate<KS>(c, off, K, stride, transposed, new_shape, [&](int k, const Int3& v) {
    const Found f = scratch_find(slots, capacity, pack_key(c.x, v.x, v.y, v.z));
    if (f.slot == 0xFFFFFFFFu) return;
    const uint32_t o = f.out_row;
    if (o < (uint32_t)n_out) atomicMax(nbr + (int64_t)o * K + k, (int32_t)row);   // duplicate coordinates: largest row
  });
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

// Submanifold map over the table's own coordinates, probing only half of the offsets.  With offsets that
// come in opposite pairs (off[K-1-k] = -off[k]) and queries that are the table's rows, "i is the
// neighbour of o at k" means "o is the neighbour of i at K-1-k": a thread probes offset k <= K/2 of its
// row, stores the hit, and mirrors it with atomicMax (the table's own rule for duplicate coordinates:
// the largest row wins).  nbr must hold -1 in its upper half.
template <typename CT>
__global__ void __launch_bounds__(256)
map_build_half_kernel(const CT* __restrict__ coords, int64_t n_half, int K, Offsets off, Int3 shape, Table table,
                      int32_t* __restrict__ nbr) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= n_half) return;
  const int half = K / 2 + 1;
  const int64_t row = t / half;
  const int k = (int)(t - row * half);
  const int4 c = load_coord<CT>(coords, row);
  const int x = c.y - off.v[k * 3 + 0], y = c.z - off.v[k * 3 + 1], z = c.w - off.v[k * 3 + 2];
  int32_t r = -1;
  if (x >= 0 && x < shape.x && y >= 0 && y < shape.y && z >= 0 && z < shape.z && table.capacity != 0 &&
      key_representable(c.x, x, y, z))
    r = table_find(table, pack_key(c.x, x, y, z));
  nbr[row * K + k] = r;
  if (k == K / 2 || r < 0) return;
  // the mirrored entry looks this row's own coordinate up, which the probing form bounds-checks
  if (c.y < 0 || c.y >= shape.x || c.z < 0 || c.z >= shape.y || c.w < 0 || c.w >= shape.z) return;
  atomicMax(nbr + (int64_t)r * K + (K - 1 - k), (int32_t)row);
}

// Rows that the table does not return for their own coordinate (smaller duplicates, coordinates outside
// the grid) are nobody's mirror image: their upper half is probed directly.
template <typename CT>
__global__ void __launch_bounds__(256)
map_build_rest_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, Int3 shape, Table table,
                      int32_t* __restrict__ nbr, int32_t* __restrict__ asymmetric_rows) {
  const int64_t row = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (row >= n) return;
  if (nbr[row * K + K / 2] == (int32_t)row) return;
  if (asymmetric_rows) atomicAdd(asymmetric_rows, 1);
  const int4 c = load_coord<CT>(coords, row);
  for (int k = K / 2 + 1; k < K; ++k) {
    const int x = c.y - off.v[k * 3 + 0], y = c.z - off.v[k * 3 + 1], z = c.w - off.v[k * 3 + 2];
    int32_t r = -1;
    if (x >= 0 && x < shape.x && y >= 0 && y < shape.y && z >= 0 && z < shape.z && table.capacity != 0 &&
        key_representable(c.x, x, y, z))
      r = table_find(table, pack_key(c.x, x, y, z));
    nbr[row * K + k] = r;
  }
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

// ---------------------------------------------------------------------------------------------
// Output coordinates by direct addressing.  When the caller knows how many samples the batch holds and the
// output grid of all samples has few enough cells, a coordinate needs no hash table: its cell number
// ((b * X + x) * Y + y) * Z + z addresses one bit of a bitmap (C3: 67 M cells = 8 MB; a 1440 x 1440 x 41 lidar
// batch of 16 at stride 2: 22 MB), which stays in L2 together with everything derived from it, where the
// 16-byte slots of the dedupe table (128 MB on C3) are DRAM round trips.
//
//   bits      every candidate sets the bit of its cell                         -> set bits = output coordinates
//   ranks     popcount per block of 256 cells + exclusive scan                 -> rank of a cell = its dense index
//   minflat   every candidate lowers min_flat[rank(cell)] to its flat index n*K+k (the first discoverer)
//   order     the winners' flat indices set bits of a second bitmap over n*K; its ranks are the output rows:
//             coordinates come out ordered by first occurrence (n-major, k-minor), exactly as from the table
//   write     winner r stores its coordinate at row rank(min_flat[r]) and leaves that row in out_row[r]
//   map       candidate (n, k) looks up out_row[rank(cell)] and scatters n into nbr[row, k]
// ---------------------------------------------------------------------------------------------
struct DirectLayout {
  int64_t cells, n_cell_blocks, n_flat_blocks, n_out_max;
  uint32_t* cell_bits;      // n_cell_blocks * 8 words
  uint32_t* cell_prefix;    // n_cell_blocks
  uint32_t* flat_bits;      // n_flat_blocks * 8 words
  uint32_t* flat_prefix;    // n_flat_blocks
  uint32_t* min_flat;       // n_out_max
  uint32_t* out_row;        // n_out_max
  void* scan_tmp;
};

constexpr int64_t kDirectMaxCells = 1ll << 29;          // a bitmap of 64 MB at most: it has to live in L2

// Lays the direct-addressing arrays out in `workspace` (after its 256-byte header); false when the batch size is
// unknown, the grid is too large or the workspace (sized for the dedupe table) does not hold them.
static bool direct_layout(void* workspace, int64_t bytes, int64_t n, int K, int stride, int transposed, const Int3& ns,
                          int batch_bound, DirectLayout* d) {
  if (batch_bound < 1 || ns.x < 1 || ns.y < 1 || ns.z < 1) return false;
  const int64_t per_sample = (int64_t)ns.x * ns.y * ns.z;
  if (per_sample > kDirectMaxCells || (int64_t)batch_bound * per_sample > kDirectMaxCells) return false;
  d->cells = (int64_t)batch_bound * per_sample;
  d->n_cell_blocks = (d->cells + 255) / 256;
  d->n_flat_blocks = (n * K + 255) / 256;
  int64_t per_input = K;
  if (!transposed && stride > 1) {
    int ks = 1;
    while (ks * ks * ks < K) ++ks;
    const int64_t c = (ks + stride - 1) / stride;
    per_input = c * c * c;
  }
  d->n_out_max = n * per_input < d->cells ? n * per_input : d->cells;
  char* p = static_cast<char*>(workspace) + 256;
  char* end = static_cast<char*>(workspace) + bytes;
  auto take = [&](int64_t nbytes) {
    char* q = p;
    p += align_up(nbytes, 256);
    return q;
  };
  d->cell_bits = reinterpret_cast<uint32_t*>(take(d->n_cell_blocks * 32));
  d->cell_prefix = reinterpret_cast<uint32_t*>(take(d->n_cell_blocks * 4));
  d->flat_bits = reinterpret_cast<uint32_t*>(take(d->n_flat_blocks * 32));
  d->flat_prefix = reinterpret_cast<uint32_t*>(take(d->n_flat_blocks * 4));
  d->min_flat = reinterpret_cast<uint32_t*>(take(d->n_out_max * 4));
  d->out_row = reinterpret_cast<uint32_t*>(take(d->n_out_max * 4));
  const int64_t scan_n = d->n_cell_blocks > d->n_flat_blocks ? d->n_cell_blocks : d->n_flat_blocks;
  d->scan_tmp = take(scan_tmp_bytes(scan_n));
  return p <= end;
}

__device__ __forceinline__ int64_t cell_index(int b, const Int3& v, const Int3& shape) {
  return (((int64_t)b * shape.x + v.x) * shape.y + v.y) * shape.z + v.z;
}

// Number of set bits below bit i: the block's prefix plus the popcounts inside its 256-bit block (one 32-byte
// sector).
template <typename IndexT>
__device__ __forceinline__ uint32_t bit_rank(const uint32_t* __restrict__ bits, const uint32_t* __restrict__ prefix,
                                             IndexT i) {
  const IndexT blk = i >> 8;
  const uint4* p = reinterpret_cast<const uint4*>(bits + blk * 8);
  const uint4 lo = p[0], hi = p[1];
  const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  const int wi = (int)((i >> 5) & 7);
  const uint32_t below = (1u << (i & 31)) - 1u;
  uint32_t r = prefix[blk];
#pragma unroll
  for (int j = 0; j < 8; ++j) r += __popc(w[j] & (j < wi ? 0xFFFFFFFFu : (j == wi ? below : 0u)));
  return r;
}

template <typename CT, int KS, bool DENSE = false>
__global__ void __launch_bounds__(kRowThreads)
direct_bits_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed,
                   Int3 new_shape, int batch_bound, uint32_t* bits, int32_t* status) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  if constexpr (DENSE) {
    __shared__ uint2 lines[kRowThreads / 32][32 * kDensePerRow];
    bool live = row < n;
    const int4 c = live ? load_coord<CT>(coords, row) : make_int4(0, 0, 0, 0);
    if (live && (unsigned)c.x >= (unsigned)batch_bound) {
      atomicOr(status, ST_DEV_BAD_INDEX);
      live = false;
    }
    warp_dense_candidates(live, c, off, stride, new_shape, lines[threadIdx.x >> 5], [&](int, int, uint32_t cell) {
      const uint32_t m = 1u << (cell & 31);
      if (!(__ldcg(bits + (cell >> 5)) & m)) atomicOr(bits + (cell >> 5), m);
    });
    return;
  }
  if (row >= n) return;
  const int4 c = load_coord<CT>(coords, row);
  if ((unsigned)c.x >= (unsigned)batch_bound) {           // a sample the caller did not announce: no cell for it
    atomicOr(status, ST_DEV_BAD_INDEX);
    return;
  }
  for_each_candidate<KS>(c, off, K, stride, transposed, new_shape, [&](int, const Int3& v) {
    const int64_t i = cell_index(c.x, v, new_shape);
    const uint32_t m = 1u << (i & 31);
    if (!(__ldcg(bits + (i >> 5)) & m)) atomicOr(bits + (i >> 5), m);
  });
}

// counts[b] = set bits of block b (8 words)
__global__ void __launch_bounds__(256)
bit_block_count_kernel(const uint32_t* __restrict__ bits, int64_t n_blocks, uint32_t* __restrict__ counts) {
  const int64_t b = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (b >= n_blocks) return;
  const uint4* p = reinterpret_cast<const uint4*>(bits + b * 8);
  const uint4 lo = p[0], hi = p[1];
  counts[b] = __popc(lo.x) + __popc(lo.y) + __popc(lo.z) + __popc(lo.w) + __popc(hi.x) + __popc(hi.y) + __popc(hi.z) +
              __popc(hi.w);
}

template <typename CT, int KS, bool DENSE = false>
__global__ void __launch_bounds__(kRowThreads)
direct_minflat_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed,
                      Int3 new_shape, int batch_bound, const uint32_t* __restrict__ bits,
                      const uint32_t* __restrict__ prefix, uint32_t* min_flat) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  if constexpr (DENSE) {
    __shared__ uint2 lines[kRowThreads / 32][32 * kDensePerRow];
    bool live = row < n;
    const int4 c = live ? load_coord<CT>(coords, row) : make_int4(0, 0, 0, 0);
    if ((unsigned)c.x >= (unsigned)batch_bound) live = false;
    const uint32_t warp_row = (uint32_t)(row - (threadIdx.x & 31));
    warp_dense_candidates(live, c, off, stride, new_shape, lines[threadIdx.x >> 5], [&](int owner, int k, uint32_t cell) {
      const uint32_t r = bit_rank<uint32_t>(bits, prefix, cell);
      const uint32_t flat = (warp_row + (uint32_t)owner) * (uint32_t)K + (uint32_t)k;
      if (__ldcg(min_flat + r) > flat) atomicMin(min_flat + r, flat);
    });
    return;
  }
  if (row >= n) return;
  const int4 c = load_coord<CT>(coords, row);
  if ((unsigned)c.x >= (unsigned)batch_bound) return;
  const uint32_t flat0 = (uint32_t)row * (uint32_t)K;
  for_each_candidate<KS>(c, off, K, stride, transposed, new_shape, [&](int k, const Int3& v) {
    const uint32_t r = bit_rank(bits, prefix, cell_index(c.x, v, new_shape));
    const uint32_t flat = flat0 + (uint32_t)k;
    if (__ldcg(min_flat + r) > flat) atomicMin(min_flat + r, flat);
  });
}

__global__ void __launch_bounds__(256)
direct_flatbits_kernel(const uint32_t* __restrict__ min_flat, int64_t n_out, uint32_t n_flat, uint32_t* flat_bits,
                       int32_t* status) {
  const int64_t r = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (r >= n_out) return;
  const uint32_t f = min_flat[r];
  if (f >= n_flat) {                          // no candidate has this rank: the caller asked for more rows than exist
    atomicOr(status, ST_DEV_OUT_OVERFLOW);
    return;
  }
  atomicOr(flat_bits + (f >> 5), 1u << (f & 31));
}

template <typename CT>
__global__ void __launch_bounds__(256)
direct_write_kernel(const CT* __restrict__ coords, int K, Offsets off, int stride, bool transposed, Int3 new_shape,
                    const uint32_t* __restrict__ min_flat, int64_t n_out, uint32_t n_flat,
                    const uint32_t* __restrict__ flat_bits, const uint32_t* __restrict__ flat_prefix, CT* out,
                    int64_t out_capacity, uint32_t* out_row, int32_t* status) {
  const int64_t r = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (r >= n_out) return;
  const uint32_t f = min_flat[r];
  if (f >= n_flat) {
    out_row[r] = 0xFFFFFFFFu;
    return;
  }
  const uint32_t dst = bit_rank(flat_bits, flat_prefix, f);
  out_row[r] = dst;
  if ((int64_t)dst >= out_capacity) {
    atomicOr(status, ST_DEV_OUT_OVERFLOW);
    return;
  }
  const uint32_t row = f / (uint32_t)K;
  const int k = (int)(f - row * (uint32_t)K);
  const int4 c = load_coord<CT>(coords, row);
  Int3 v;
  candidate(c, off, k, stride, transposed, new_shape, &v);
  store_coord<CT>(out, dst, c.x, v.x, v.y, v.z);
}

// nbr[out_row(candidate), k] = max(input row), as outcoords_map_kernel.  nbr must hold -1.
template <typename CT, int KS, bool DENSE = false>
__global__ void __launch_bounds__(kRowThreads)
direct_map_kernel(const CT* __restrict__ coords, int64_t n, int K, Offsets off, int stride, bool transposed, Int3 new_shape,
                  Int3 in_shape, int batch_bound, const uint32_t* __restrict__ bits, const uint32_t* __restrict__ prefix,
                  const uint32_t* __restrict__ out_row, int32_t* nbr, int64_t n_out) {
  const int64_t row = (int64_t)blockIdx.x * kRowThreads + threadIdx.x;
  if constexpr (DENSE) {
    __shared__ uint2 lines[kRowThreads / 32][32 * kDensePerRow];
    bool live = row < n;
    const int4 c = live ? load_coord<CT>(coords, row) : make_int4(0, 0, 0, 0);
    if ((unsigned)c.x >= (unsigned)batch_bound) live = false;
    if (c.y < 0 || c.y >= in_shape.x || c.z < 0 || c.z >= in_shape.y || c.w < 0 || c.w >= in_shape.z) live = false;
    const int32_t warp_row = (int32_t)(row - (threadIdx.x & 31));
    warp_dense_candidates(live, c, off, stride, new_shape, lines[threadIdx.x >> 5], [&](int owner, int k, uint32_t cell) {
      const uint32_t o = out_row[bit_rank<uint32_t>(bits, prefix, cell)];
      if (o < (uint32_t)n_out) atomicMax(nbr + (int64_t)o * K + k, warp_row + owner);
    });
    return;
  }
  if (row >= n) return;
  const int4 c = load_coord<CT>(coords, row);
  if ((unsigned)c.x >= (unsigned)batch_bound) return;
  if (c.y < 0 || c.y >= in_shape.x || c.z < 0 || c.z >= in_shape.y || c.w < 0 || c.w >= in_shape.z) return;
  for_each_candidate<KS>(c, off, K, stride, transposed, new_shape, [&](int k, const Int3& v) {
    const uint32_t o = out_row[bit_rank(bits, prefix, cell_index(c.x, v, new_shape))];
    if (o < (uint32_t)n_out) atomicMax(nbr + (int64_t)o * K + k, (int32_t)row);
  });
}

template <typename CT>
static int direct_count_impl(const CT* coords, int64_t n, const Offsets& off, int K, int stride, bool transposed, Int3 ns,
                             int batch_bound, const DirectLayout& d, int64_t* n_out, int32_t* status, cudaStream_t s) {
  const unsigned grid = (unsigned)((n + kRowThreads - 1) / kRowThreads);
  cudaMemsetAsync(d.cell_bits, 0, (size_t)d.n_cell_blocks * 32, s);
  const int ks = product_kernel_size(off, K);
  if (dense_sweep_ok(off, ks, stride, transposed))
    direct_bits_kernel<CT, 3, true><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, status);
  else if (ks == 3)
    direct_bits_kernel<CT, 3><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, status);
  else if (ks == 2)
    direct_bits_kernel<CT, 2><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, status);
  else
    direct_bits_kernel<CT, 0><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, status);
  bit_block_count_kernel<<<(unsigned)((d.n_cell_blocks + 255) / 256), 256, 0, s>>>(d.cell_bits, d.n_cell_blocks, d.cell_prefix);
  note_launches(2);
  int rc = check_launch("st_outcoords_count");
  if (rc != ST_OK) return rc;
  return exclusive_scan_u32(d.cell_prefix, d.cell_prefix, d.n_cell_blocks, d.scan_tmp, n_out, s);
}

template <typename CT>
static int direct_write_impl(const CT* coords, int64_t n, const Offsets& off, int K, int stride, bool transposed, Int3 ns,
                             int batch_bound, const DirectLayout& d, CT* out, int64_t n_out, int32_t* status,
                             cudaStream_t s) {
  if (n_out > d.n_out_max) {
    set_error("st_outcoords_write: %lld output rows asked for, at most %lld can exist", (long long)n_out,
              (long long)d.n_out_max);
    return ST_ERR_ARG;
  }
  if (n_out == 0) return ST_OK;
  const unsigned grid = (unsigned)((n + kRowThreads - 1) / kRowThreads);
  const unsigned out_grid = (unsigned)((n_out + 255) / 256);
  cudaMemsetAsync(d.min_flat, 0xFF, (size_t)n_out * 4, s);
  cudaMemsetAsync(d.flat_bits, 0, (size_t)d.n_flat_blocks * 32, s);
  const int ks = product_kernel_size(off, K);
  if (dense_sweep_ok(off, ks, stride, transposed))
    direct_minflat_kernel<CT, 3, true><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, d.cell_prefix, d.min_flat);
  else if (ks == 3)
    direct_minflat_kernel<CT, 3><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, d.cell_prefix, d.min_flat);
  else if (ks == 2)
    direct_minflat_kernel<CT, 2><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, d.cell_prefix, d.min_flat);
  else
    direct_minflat_kernel<CT, 0><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, batch_bound, d.cell_bits, d.cell_prefix, d.min_flat);
  direct_flatbits_kernel<<<out_grid, 256, 0, s>>>(d.min_flat, n_out, (uint32_t)(n * K), d.flat_bits, status);
  bit_block_count_kernel<<<(unsigned)((d.n_flat_blocks + 255) / 256), 256, 0, s>>>(d.flat_bits, d.n_flat_blocks, d.flat_prefix);
  note_launches(3);
  int rc = exclusive_scan_u32(d.flat_prefix, d.flat_prefix, d.n_flat_blocks, d.scan_tmp, nullptr, s);
  if (rc != ST_OK) return rc;
  direct_write_kernel<CT><<<out_grid, 256, 0, s>>>(coords, K, off, stride, transposed, ns, d.min_flat, n_out, (uint32_t)(n * K),
                                                   d.flat_bits, d.flat_prefix, out, n_out, d.out_row, status);
  note_launches(1);
  return check_launch("st_outcoords_write");
}

template <typename CT>
static int outcoords_count_impl(const CT* coords, int64_t n, const Offsets& off, int K, int stride, bool transposed,
                                Int3 ns, OutCoordsWorkspace& w, int64_t* n_out, int32_t* status, cudaStream_t s) {
  const unsigned grid = (unsigned)((n + kRowThreads - 1) / kRowThreads);
  cudaMemsetAsync(w.header, 0, sizeof(OutCoordsHeader), s);
  const int ks = product_kernel_size(off, K);
#define ST_SWEEP(KS)                                                                                                  \
  {                                                                                                                   \
    outcoords_count_kernel<CT, KS><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, w.header); \
    scratch_clear_kernel<<<1184, 256, 0, s>>>(w.header, (unsigned long long)w.capacity_max, w.slots);                \
    outcoords_insert_kernel<CT, KS><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, w.header, \
                                                                 w.slots, status);                                   \
    outcoords_mark_kernel<CT, KS><<<grid, kRowThreads, 0, s>>>(coords, n, K, off, stride, transposed, ns, w.header,   \
                                                               w.slots, w.win_words, w.words, w.row_counts);         \
    note_launches(4);                                                                                                 \
  }
  if (ks == 3) ST_SWEEP(3) else if (ks == 2) ST_SWEEP(2) else ST_SWEEP(0)
#undef ST_SWEEP
  int rc = check_launch("st_outcoords_count");
  if (rc != ST_OK) return rc;
  return exclusive_scan_u32(w.row_counts, w.row_counts, n, w.scan_tmp, n_out, s);
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
  return outcoords_bytes(n, K, stride, transposed);
}

int st_outcoords_count(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K, int stride,
                       int transposed, const int32_t* new_shape_host, int batch_bound, void* workspace,
                       int64_t workspace_bytes, int64_t* n_out, int32_t* status, void* stream) {
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
  DirectLayout d;
  if (direct_layout(workspace, workspace_bytes, n, K, stride, transposed, ns, batch_bound, &d)) {
    if (coord_dtype == ST_I32)
      return direct_count_impl<int32_t>(static_cast<const int32_t*>(coords), n, off, K, stride, transposed != 0, ns,
                                        batch_bound, d, n_out, status, s);
    return direct_count_impl<int16_t>(static_cast<const int16_t*>(coords), n, off, K, stride, transposed != 0, ns,
                                      batch_bound, d, n_out, status, s);
  }
  if (coord_dtype == ST_I32)
    return outcoords_count_impl<int32_t>(static_cast<const int32_t*>(coords), n, off, K, stride, transposed != 0, ns,
                                         w, n_out, status, s);
  return outcoords_count_impl<int16_t>(static_cast<const int16_t*>(coords), n, off, K, stride, transposed != 0, ns, w,
                                       n_out, status, s);
}

int st_outcoords_write(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K, int stride,
                       int transposed, const int32_t* new_shape_host, int batch_bound, void* workspace,
                       int64_t workspace_bytes, void* out_coords, int64_t out_capacity, int32_t* status, void* stream) {
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
  DirectLayout d;
  if (direct_layout(workspace, workspace_bytes, n, K, stride, transposed, ns, batch_bound, &d)) {
    if (coord_dtype == ST_I32)
      return direct_write_impl<int32_t>(static_cast<const int32_t*>(coords), n, off, K, stride, transposed != 0, ns,
                                        batch_bound, d, static_cast<int32_t*>(out_coords), out_capacity, status, s);
    return direct_write_impl<int16_t>(static_cast<const int16_t*>(coords), n, off, K, stride, transposed != 0, ns,
                                      batch_bound, d, static_cast<int16_t*>(out_coords), out_capacity, status, s);
  }
  const unsigned grid = (unsigned)((n + kRowThreads - 1) / kRowThreads);
  if (coord_dtype == ST_I32) {
    outcoords_write_kernel<int32_t><<<grid, kRowThreads, 0, s>>>(
        static_cast<const int32_t*>(coords), n, K, off, stride, transposed != 0, ns, w.header, w.slots,
        w.win_words, w.words, w.row_counts, static_cast<int32_t*>(out_coords), out_capacity, status);
  } else {
    outcoords_write_kernel<int16_t><<<grid, kRowThreads, 0, s>>>(
        static_cast<const int16_t*>(coords), n, K, off, stride, transposed != 0, ns, w.header, w.slots,
        w.win_words, w.words, w.row_counts, static_cast<int16_t*>(out_coords), out_capacity, status);
  }
  note_launches(1);
  return check_launch("st_outcoords_write");
}

int st_outcoords_map(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K, int stride,
                     int transposed, const int32_t* new_shape_host, const int32_t* in_shape_host, int batch_bound,
                     void* workspace, int64_t workspace_bytes, int32_t* nbr, int64_t n_out, void* stream) {
  Offsets off;
  Int3 ns;
  OutCoordsWorkspace w;
  if (n_out < 0 || (n_out > 0 && !nbr) || !in_shape_host) {
    set_error("st_outcoords_map: bad output arguments");
    return ST_ERR_ARG;
  }
  int rc = outcoords_args(coords, n, coord_dtype, offsets_host, K, stride, new_shape_host, workspace,
                          workspace_bytes, transposed, &off, &ns, &w, "st_outcoords_map");
  if (rc != ST_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t n_map = n_out * K;
  if (n_map > 0) cudaMemsetAsync(nbr, 0xFF, (size_t)n_map * sizeof(int32_t), s);            // every entry -1
  if (n == 0 || n_out == 0) return check_launch("st_outcoords_map");
  const unsigned grid = (unsigned)((n + kRowThreads - 1) / kRowThreads);
  const Int3 in_shape = {in_shape_host[0], in_shape_host[1], in_shape_host[2]};
  const int ks = product_kernel_size(off, K);
  DirectLayout d;
  if (direct_layout(workspace, workspace_bytes, n, K, stride, transposed, ns, batch_bound, &d)) {
    const bool dense = dense_sweep_ok(off, ks, stride, transposed != 0);
#define ST_DMAP(CT, KS, DENSE)                                                                                        \
  direct_map_kernel<CT, KS, DENSE><<<grid, kRowThreads, 0, s>>>(static_cast<const CT*>(coords), n, K, off, stride,   \
                                                                transposed != 0, ns, in_shape, batch_bound,          \
                                                                d.cell_bits, d.cell_prefix, d.out_row, nbr, n_out)
    if (coord_dtype == ST_I32) {
      if (dense) ST_DMAP(int32_t, 3, true); else if (ks == 3) ST_DMAP(int32_t, 3, false);
      else if (ks == 2) ST_DMAP(int32_t, 2, false); else ST_DMAP(int32_t, 0, false);
    } else {
      if (dense) ST_DMAP(int16_t, 3, true); else if (ks == 3) ST_DMAP(int16_t, 3, false);
      else if (ks == 2) ST_DMAP(int16_t, 2, false); else ST_DMAP(int16_t, 0, false);
    }
#undef ST_DMAP
    note_launches(1);
    return check_launch("st_outcoords_map");
  }
#define ST_MAP(CT, KS)                                                                                              \
  outcoords_map_kernel<CT, KS><<<grid, kRowThreads, 0, s>>>(static_cast<const CT*>(coords), n, K, off, stride,     \
                                                            transposed != 0, ns, in_shape, w.header, w.slots, nbr, \
                                                            n_out)
  if (coord_dtype == ST_I32) {
    if (ks == 3) ST_MAP(int32_t, 3); else if (ks == 2) ST_MAP(int32_t, 2); else ST_MAP(int32_t, 0);
  } else {
    if (ks == 3) ST_MAP(int16_t, 3); else if (ks == 2) ST_MAP(int16_t, 2); else ST_MAP(int16_t, 0);
  }
#undef ST_MAP
  note_launches(1);
  return check_launch("st_outcoords_map");
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

int st_map_build_symmetric(const void* coords, int64_t n, int coord_dtype, const int32_t* offsets_host, int K,
                           const int32_t* lookup_shape_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                           int32_t* nbr, int32_t* asymmetric_rows, void* stream) {
  if (n < 0 || K < 1 || K > ST_MAX_KVOL || (K & 1) == 0 || !offsets_host || !lookup_shape_host || capacity < 0 ||
      capacity > 0x7FFFFFFFll || (n > 0 && (!coords || !nbr)) || (capacity > 0 && (!keys || !vals))) {
    set_error("st_map_build_symmetric: bad arguments (K must be odd)");
    return ST_ERR_ARG;
  }
  for (int k = 0; k < K; ++k)
    for (int a = 0; a < 3; ++a)
      if (offsets_host[k * 3 + a] != -offsets_host[(K - 1 - k) * 3 + a]) {
        set_error("st_map_build_symmetric: offsets %d and %d are not opposite", k, K - 1 - k);
        return ST_ERR_ARG;
      }
  Offsets off;
  if (!pack_offsets(offsets_host, K, &off)) {
    set_error("st_map_build_symmetric: offset outside int16");
    return ST_ERR_UNSUPPORTED;
  }
  if (coord_dtype != ST_I32 && coord_dtype != ST_I16) {
    set_error("st_map_build_symmetric: unknown coordinate dtype %d", coord_dtype);
    return ST_ERR_DTYPE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (asymmetric_rows) cudaMemsetAsync(asymmetric_rows, 0, sizeof(int32_t), s);
  if (n == 0) return ST_OK;
  const Int3 shape = {lookup_shape_host[0], lookup_shape_host[1], lookup_shape_host[2]};
  const Table t = make_table(keys, vals, capacity);
  const int64_t n_flat = n * K, n_half = n * (K / 2 + 1);
  cudaMemsetAsync(nbr, 0xFF, (size_t)n_flat * sizeof(int32_t), s);                             // every entry -1
  if (coord_dtype == ST_I32) {
    map_build_half_kernel<int32_t><<<(unsigned)((n_half + 255) / 256), 256, 0, s>>>(static_cast<const int32_t*>(coords),
                                                                                   n_half, K, off, shape, t, nbr);
    map_build_rest_kernel<int32_t><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<const int32_t*>(coords), n, K,
                                                                              off, shape, t, nbr, asymmetric_rows);
  } else {
    map_build_half_kernel<int16_t><<<(unsigned)((n_half + 255) / 256), 256, 0, s>>>(static_cast<const int16_t*>(coords),
                                                                                   n_half, K, off, shape, t, nbr);
    map_build_rest_kernel<int16_t><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<const int16_t*>(coords), n, K,
                                                                              off, shape, t, nbr, asymmetric_rows);
  }
  note_launches(2);
  return check_launch("st_map_build_symmetric");
}

int st_map_invert(const int32_t* nbr, int64_t n_out, int K, int64_t n_in, int32_t* inv, void* stream) {
  if (n_out < 0 || n_in < 0 || K < 1 || (n_out > 0 && !nbr) || (n_in > 0 && !inv)) {
    set_error("st_map_invert: bad arguments");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int64_t n_inv = n_in * K;
  if (n_inv > 0) cudaMemsetAsync(inv, 0xFF, (size_t)n_inv * sizeof(int32_t), s);           // every entry -1
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
