// Where a convolution kernel gets "which input row feeds output row r under offset k" from:
// a stored dense map, or the coordinate hash table probed on the fly.
#pragma once

#include "common.cuh"

namespace st {

// Dense (rows, K) table, -1 = none.
struct StoredMap {
  const int32_t* nbr;
  int K;
  // No per-tile state.
  template <int BM>
  __device__ __forceinline__ void prepare(int4* /*smem_coords*/, int64_t /*row0*/, int64_t /*n_rows*/) const {}
  __device__ __forceinline__ int32_t get(const int4* /*smem_coords*/, int /*m*/, int64_t row, int k) const {
    return __ldg(nbr + row * K + k);
  }
};

// curr = out*stride - off[k]; bounds check; table probe.
template <typename CT>
struct HashFlyMap {
  const CT* coords;
  Offsets off;
  Table table;
  Int3 shape;
  int stride;
  template <int BM>
  __device__ __forceinline__ void prepare(int4* smem_coords, int64_t row0, int64_t n_rows) const {
    for (int m = threadIdx.x; m < BM; m += blockDim.x) {
      int64_t r = row0 + m;
      smem_coords[m] = r < n_rows ? load_coord<CT>(coords, r) : make_int4(0, -1, -1, -1);
    }
  }
  __device__ __forceinline__ int32_t get(const int4* smem_coords, int m, int64_t /*row*/, int k) const {
    int4 c = smem_coords[m];
    int x = c.y * stride - off.v[k * 3 + 0];
    int y = c.z * stride - off.v[k * 3 + 1];
    int z = c.w * stride - off.v[k * 3 + 2];
    if (c.y < 0 || x < 0 || x >= shape.x || y < 0 || y >= shape.y || z < 0 || z >= shape.z ||
        table.capacity == 0 || !key_representable(c.x, x, y, z))
      return -1;
    return table_find(table, pack_key(c.x, x, y, z));
  }
};

}  // namespace st
