// Row order of a neighbour map for the tensor-core kernels.
//
// The implicit-GEMM kernels work on tiles of 128 rows and skip a kernel offset for a tile only when
// none of its 128 rows has a neighbour there.  In the natural row order nearly every tile touches
// nearly every offset, and 70-80 % of what the tensor cores multiply is zero fill.  Rows with the
// same set of occupied offsets behave alike, so the kernels may walk the rows in the order of their
// K-bit occupancy mask instead: tiles then share masks, far fewer (tile, offset) stages remain and
// those are denser.  The order only decides which rows share a tile; every row's own sum still
// runs over the offsets in ascending k, so forward and feature-gradient results do not depend on it.
//
// order = stable LSD radix sort of the rows by mask (9-bit digits); equal masks keep their original
// order and no atomic decides a position, so the result is deterministic.
#include "common.cuh"
#include "radix_sort.cuh"

namespace st {

namespace {

// key[r] = occupancy mask of row r (bit k: nbr[r,k] >= 0) for K <= 32, a 32-bit hash of the whole
// pattern beyond (equal patterns still get equal keys); val[r] = r.
__global__ void __launch_bounds__(128) row_keys_kernel(const int32_t* __restrict__ nbr, int64_t n, int K,
                                                      uint32_t* __restrict__ keys, int32_t* __restrict__ vals) {
  extern __shared__ int32_t stage[];                     // 128 rows x K entries when K <= 64
  const int64_t row0 = (int64_t)blockIdx.x * 128;
  const int rows = (int)min((int64_t)128, n - row0);
  const int64_t row = row0 + threadIdx.x;
  uint32_t key = 0;
  if (K <= 64) {
    const int32_t* src = nbr + row0 * K;
    for (int e = threadIdx.x; e < rows * K; e += 128) stage[e] = __ldg(src + e);
    __syncthreads();
    if (threadIdx.x < rows) {
      const int32_t* mine = stage + threadIdx.x * K;
      if (K <= 32) {
        for (int k = 0; k < K; ++k) key |= (mine[k] >= 0 ? 1u : 0u) << k;
      } else {
        for (int k = 0; k < K; ++k) key = key * 0x9E3779B1u + (mine[k] >= 0 ? (uint32_t)(k + 1) : 0u);
      }
    }
  } else if (threadIdx.x < rows) {
    for (int k = 0; k < K; ++k) key = key * 0x9E3779B1u + (__ldg(nbr + row * K + k) >= 0 ? (uint32_t)(k + 1) : 0u);
  }
  if (threadIdx.x < rows) {
    keys[row] = key;
    vals[row] = (int32_t)row;
  }
}

// Tile plan: the map re-laid so that the 128 source rows of one (tile, offset) step are one
// contiguous 512-byte line, in the row order the kernels walk, plus a per-tile bit mask of the
// offsets that have a neighbour anywhere in the tile.
//   tmap [(tile * K + k) * 128 + r] = nbr[order[tile * 128 + r], k]      (-1 past the last row)
//   tmask[tile * MW + k / 32] bit (k % 32)                                 MW = ceil(K / 32)
// One block per tile.  A warp reads one row at a time as a run of consecutive entries (a warp-wide
// load touches one or two lines, not 32) into shared memory, `kPlanChunk` offsets at a time, with the
// loads of eight rows in flight together; the block writes them back transposed.
constexpr int kPlanChunk = 64;

__global__ void __launch_bounds__(128) plan_tiles_kernel(const int32_t* __restrict__ nbr,
                                                        const int32_t* __restrict__ order, int64_t n_rows, int K,
                                                        int MW, int32_t* __restrict__ tmap,
                                                        uint32_t* __restrict__ tmask) {
  extern __shared__ int32_t stage[];                      // 128 x (min(K, kPlanChunk) | 1) entries
  __shared__ int64_t src_row[128];
  __shared__ uint32_t mask_word[2];                       // the (at most two) mask words of a chunk
  const int64_t tile = blockIdx.x;
  const int r = threadIdx.x, warp = r >> 5, lane = r & 31;
  const int64_t pos = tile * 128 + r;
  src_row[r] = pos < n_rows ? (order ? (int64_t)__ldg(order + pos) : pos) : -1;
  for (int k0 = 0; k0 < K; k0 += kPlanChunk) {
    const int kc = min(kPlanChunk, K - k0);
    const int pitch = kc | 1;                              // odd: conflict-free column reads
    if (r < 2) mask_word[r] = 0;
    __syncthreads();
    // a warp per row: lane l fetches entries l and l + 32 of the chunk, eight rows' loads issued together
#pragma unroll 8
    for (int row = warp; row < 128; row += 4) {
      const int64_t src = src_row[row];
      const int32_t* from = nbr + src * K + k0;
      const int32_t lo = (src >= 0 && lane < kc) ? __ldg(from + lane) : -1;
      const int32_t hi = (src >= 0 && lane + 32 < kc) ? __ldg(from + lane + 32) : -1;
      if (lane < kc) stage[row * pitch + lane] = lo;
      if (lane + 32 < kc) stage[row * pitch + lane + 32] = hi;
    }
    __syncthreads();
    for (int k = 0; k < kc; ++k) {
      const int32_t v = stage[r * pitch + k];
      tmap[(tile * K + k0 + k) * 128 + r] = v;
      const uint32_t any = __ballot_sync(0xFFFFFFFFu, v >= 0);
      if (any && lane == 0) atomicOr(&mask_word[k >> 5], 1u << (k & 31));
    }
    __syncthreads();
    if (r < (kc + 31) / 32) tmask[tile * MW + (k0 >> 5) + r] = mask_word[r];
    __syncthreads();
  }
}

struct OrderScratch {
  uint32_t *keys_a, *keys_b, *hist, *totals;
  int32_t* vals_b;
};

int64_t carve(OrderScratch* s, void* ws, int64_t n, int K) {
  (void)K;
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    char* p = ws ? static_cast<char*>(ws) + off : nullptr;
    off += align_up(bytes > 0 ? bytes : 1, 256);
    return p;
  };
  const int64_t nn = n > 0 ? n : 1;
  s->keys_a = reinterpret_cast<uint32_t*>(take(nn * 4));
  s->keys_b = reinterpret_cast<uint32_t*>(take(nn * 4));
  s->vals_b = reinterpret_cast<int32_t*>(take(nn * 4));
  s->hist = reinterpret_cast<uint32_t*>(take(sort_hist_bytes(nn)));
  s->totals = reinterpret_cast<uint32_t*>(take(kBucketsMax * 4));
  return off;
}

// The radix passes over (keys, row ids) already placed in (s.keys_a, start of the value ping-pong);
// the sorted row ids land in `order`, the sorted keys in *sorted_keys.
int passes_for(int K) { return ((K < 32 ? K : 32) + kDigitBitsMax - 1) / kDigitBitsMax; }
int32_t* first_vals(const OrderScratch& s, int K, int32_t* order) { return passes_for(K) % 2 == 0 ? order : s.vals_b; }

void sort_passes(const OrderScratch& s, int64_t n_rows, int K, int32_t* order, uint32_t** sorted_keys, cudaStream_t st) {
  const int key_bits = K < 32 ? K : 32;
  // ping-pong so that the last pass lands in `order`
  int32_t* vals_in = first_vals(s, K, order);
  int32_t* vals_alt = vals_in == order ? s.vals_b : order;
  radix_sort_pairs<uint32_t>(s.keys_a, vals_in, s.keys_b, vals_alt, n_rows, key_bits, s.hist, s.totals, sorted_keys,
                             nullptr, st);
}

// ---- plan of the INVERSE map straight from the forward map (K <= 32), without writing the inverse ----
__global__ void __launch_bounds__(256) iota_clear_kernel(uint32_t* keys, int32_t* vals, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i < n) {
    keys[i] = 0u;
    vals[i] = (int32_t)i;
  }
}

// keys[i] |= 1 << k for every nbr[o,k] = i: the occupancy mask of row i of the inverse map.
// kFlatQuads runs of four consecutive entries per thread (16-byte loads, all issued before they are used).
constexpr int kFlatQuads = 4;
constexpr int kFlatPerBlock = 256 * 4 * kFlatQuads;

__device__ __forceinline__ void load_quads(const int32_t* __restrict__ nbr, int64_t n_flat, int64_t block_first,
                                           int32_t (&v)[kFlatQuads][4]) {
  const bool aligned = (reinterpret_cast<uintptr_t>(nbr) & 15) == 0;
#pragma unroll
  for (int q = 0; q < kFlatQuads; ++q) {
    const int64_t t0 = block_first + ((int64_t)q * 256 + threadIdx.x) * 4;
    v[q][0] = v[q][1] = v[q][2] = v[q][3] = -1;
    if (t0 + 3 < n_flat && aligned) {
      const int4 w = __ldg(reinterpret_cast<const int4*>(nbr + t0));
      v[q][0] = w.x; v[q][1] = w.y; v[q][2] = w.z; v[q][3] = w.w;
    } else {
      for (int j = 0; j < 4 && t0 + j < n_flat; ++j) v[q][j] = __ldg(nbr + t0 + j);
    }
  }
}

// IndexT: the type the flat index is divided in (32 bits when the map has fewer than 2^31 entries: a 64-bit division
// per run made these kernels instruction-bound).
template <typename IndexT>
__global__ void __launch_bounds__(256)
inverse_keys_kernel(const int32_t* __restrict__ nbr, int64_t n_flat, int K, int64_t n_in, uint32_t* keys) {
  const int64_t block_first = (int64_t)blockIdx.x * kFlatPerBlock;
  int32_t v[kFlatQuads][4];
  load_quads(nbr, n_flat, block_first, v);
#pragma unroll
  for (int q = 0; q < kFlatQuads; ++q) {
    const int64_t t0 = block_first + ((int64_t)q * 256 + threadIdx.x) * 4;
    int k = (int)((IndexT)t0 % (IndexT)K);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (v[q][j] >= 0 && v[q][j] < n_in) atomicOr(keys + v[q][j], 1u << k);
      if (++k == K) k = 0;
    }
  }
}

__global__ void __launch_bounds__(256) rank_kernel(const int32_t* __restrict__ order, int64_t n, int32_t* rank) {
  const int64_t p = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (p < n) rank[order[p]] = (int32_t)p;
}

// tmask[tile] = OR of the tile's 128 sorted keys (K <= 32: one word per tile)
__global__ void __launch_bounds__(128) tile_mask_kernel(const uint32_t* __restrict__ sorted_keys, int64_t n,
                                                       uint32_t* __restrict__ tmask) {
  __shared__ uint32_t part[4];
  const int64_t p = (int64_t)blockIdx.x * 128 + threadIdx.x;
  const uint32_t m = __reduce_or_sync(0xFFFFFFFFu, p < n ? sorted_keys[p] : 0u);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) tmask[blockIdx.x] = part[0] | part[1] | part[2] | part[3];
}

// tmap_inv[(tile(pos) * K + k) * 128 + pos % 128] = o for nbr[o,k] = i, pos = rank[i]; tmap_inv holds -1
template <typename IndexT>
__global__ void __launch_bounds__(256)
inverse_plan_scatter_kernel(const int32_t* __restrict__ nbr, int64_t n_flat, int K, int64_t n_in,
                            const int32_t* __restrict__ rank, int32_t* __restrict__ tmap) {
  const int64_t block_first = (int64_t)blockIdx.x * kFlatPerBlock;
  int32_t v[kFlatQuads][4];
  load_quads(nbr, n_flat, block_first, v);
  int32_t pos[kFlatQuads][4];
#pragma unroll
  for (int q = 0; q < kFlatQuads; ++q)
#pragma unroll
    for (int j = 0; j < 4; ++j) pos[q][j] = (v[q][j] >= 0 && v[q][j] < n_in) ? __ldg(rank + v[q][j]) : -1;
#pragma unroll
  for (int q = 0; q < kFlatQuads; ++q) {
    const int64_t t0 = block_first + ((int64_t)q * 256 + threadIdx.x) * 4;
    int64_t o = (int64_t)((IndexT)t0 / (IndexT)K);
    int k = (int)(t0 - o * K);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (pos[q][j] >= 0) tmap[((int64_t)(pos[q][j] >> 7) * K + k) * 128 + (pos[q][j] & 127)] = (int32_t)o;
      if (++k == K) {
        k = 0;
        ++o;
      }
    }
  }
}

}  // namespace

}  // namespace st

using namespace st;

extern "C" {

int64_t st_map_row_order_workspace_bytes(int64_t n_rows, int K) {
  OrderScratch s;
  return carve(&s, nullptr, n_rows, K);
}

int st_map_row_order(const int32_t* nbr, int64_t n_rows, int K, int32_t* order, void* workspace,
                     int64_t workspace_bytes, void* stream) {
  if (n_rows < 0 || K < 1 || n_rows > 0x7FFFFFFFll || (n_rows > 0 && (!nbr || !order || !workspace))) {
    set_error("st_map_row_order: bad arguments");
    return ST_ERR_ARG;
  }
  if (n_rows == 0) return ST_OK;
  OrderScratch s;
  if (workspace_bytes < carve(&s, workspace, n_rows, K)) {
    set_error("st_map_row_order: workspace of %lld bytes is too small", (long long)workspace_bytes);
    return ST_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t stage_bytes = K <= 64 ? (size_t)128 * K * 4 : 0;
  {
    row_keys_kernel<<<(unsigned)((n_rows + 127) / 128), 128, stage_bytes, st>>>(nbr, n_rows, K, s.keys_a,
                                                                                first_vals(s, K, order));
    note_launches(1);
  }
  sort_passes(s, n_rows, K, order, nullptr, st);
  return check_launch("st_map_row_order");
}

int64_t st_map_plan_workspace_bytes(int64_t n_rows, int K) { return st_map_row_order_workspace_bytes(n_rows, K); }

int64_t st_map_plan_inverse_workspace_bytes(int64_t n_in, int K) {
  return st_map_row_order_workspace_bytes(n_in, K) + align_up((n_in > 0 ? n_in : 1) * 4, 256);
}

int st_map_plan_inverse(const int32_t* nbr, int64_t n_out, int K, int64_t n_in, int32_t* order, int32_t* tmap,
                        uint32_t* tmask, void* workspace, int64_t workspace_bytes, void* stream) {
  if (n_out < 0 || n_in < 0 || K < 1 || K > 32 || n_in > 0x7FFFFFFFll || (n_out > 0 && !nbr) ||
      (n_in > 0 && (!order || !tmap || !tmask || !workspace))) {
    set_error("st_map_plan_inverse: bad arguments (K must be <= 32)");
    return ST_ERR_ARG;
  }
  if (n_in == 0) return ST_OK;
  OrderScratch s;
  const int64_t sort_bytes = carve(&s, workspace, n_in, K);
  if (workspace_bytes < st_map_plan_inverse_workspace_bytes(n_in, K)) {
    set_error("st_map_plan_inverse: workspace of %lld bytes is too small", (long long)workspace_bytes);
    return ST_ERR_WORKSPACE;
  }
  int32_t* rank = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + sort_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t n_flat = n_out * K, n_tiles = (n_in + 127) / 128, n_tmap = n_tiles * K * 128;
  const unsigned rows_grid = (unsigned)((n_in + 255) / 256);
  iota_clear_kernel<<<rows_grid, 256, 0, st>>>(s.keys_a, first_vals(s, K, order), n_in);
  const unsigned flat_grid = (unsigned)((n_flat + kFlatPerBlock - 1) / kFlatPerBlock);
  const bool narrow = n_flat + kFlatPerBlock < 0x7FFFFFFFll;           // every flat index a thread forms fits 32 bits
  if (n_flat > 0) {
    if (narrow) inverse_keys_kernel<uint32_t><<<flat_grid, 256, 0, st>>>(nbr, n_flat, K, n_in, s.keys_a);
    else inverse_keys_kernel<int64_t><<<flat_grid, 256, 0, st>>>(nbr, n_flat, K, n_in, s.keys_a);
  }
  note_launches(2);
  uint32_t* sorted_keys = nullptr;
  sort_passes(s, n_in, K, order, &sorted_keys, st);
  rank_kernel<<<rows_grid, 256, 0, st>>>(order, n_in, rank);
  tile_mask_kernel<<<(unsigned)n_tiles, 128, 0, st>>>(sorted_keys, n_in, tmask);
  cudaMemsetAsync(tmap, 0xFF, (size_t)n_tmap * sizeof(int32_t), st);                  // every entry -1
  if (n_flat > 0) {
    if (narrow) inverse_plan_scatter_kernel<uint32_t><<<flat_grid, 256, 0, st>>>(nbr, n_flat, K, n_in, rank, tmap);
    else inverse_plan_scatter_kernel<int64_t><<<flat_grid, 256, 0, st>>>(nbr, n_flat, K, n_in, rank, tmap);
  }
  note_launches(3);
  return check_launch("st_map_plan_inverse");
}

int st_map_plan(const int32_t* nbr, int64_t n_rows, int K, int sort_rows, int32_t* order, int32_t* tmap,
                uint32_t* tmask, void* workspace, int64_t workspace_bytes, void* stream) {
  if (n_rows < 0 || K < 1 || n_rows > 0x7FFFFFFFll ||
      (n_rows > 0 && (!nbr || !tmap || !tmask || (sort_rows && (!order || !workspace))))) {
    set_error("st_map_plan: bad arguments");
    return ST_ERR_ARG;
  }
  if (n_rows == 0) return ST_OK;
  if (sort_rows) {
    int rc = st_map_row_order(nbr, n_rows, K, order, workspace, workspace_bytes, stream);
    if (rc != ST_OK) return rc;
  }
  const int64_t n_tiles = (n_rows + 127) / 128;
  {
    const size_t stage_bytes = (size_t)128 * ((K < kPlanChunk ? K : kPlanChunk) | 1) * 4;
    plan_tiles_kernel<<<(unsigned)n_tiles, 128, stage_bytes, (cudaStream_t)stream>>>(
        nbr, sort_rows ? order : nullptr, n_rows, K, (K + 31) / 32, tmap, tmask);
    note_launches(1);
  }
  return check_launch("st_map_plan");
}

}  // extern "C"
