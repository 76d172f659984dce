// Sparse <-> dense conversion: scatter the rows of a sparse tensor into a (B, X, Y, Z, C) volume and
// gather them back (the backward of the scatter).
//
// Both directions are pure copies, bound by HBM: one thread moves one 16-byte piece of a feature row
// (consecutive threads = consecutive pieces of one row, so loads and stores are full sectors); rows
// whose width or base address does not allow 16-byte pieces are moved element by element.  The four
// coordinates of a row are one 8- or 16-byte load that the threads of the row share through L1.
#include "common.cuh"

namespace st {

namespace {

struct DenseShape {
  int B, X, Y, Z;
};

// Dense row (voxel index) of coordinate c, or -1 when it lies outside the volume.
__device__ __forceinline__ int64_t dense_row(const int4& c, const DenseShape& s) {
  if ((unsigned)c.x >= (unsigned)s.B || (unsigned)c.y >= (unsigned)s.X || (unsigned)c.z >= (unsigned)s.Y ||
      (unsigned)c.w >= (unsigned)s.Z)
    return -1;
  return (((int64_t)c.x * s.X + c.y) * s.Y + c.z) * s.Z + c.w;
}

// PIECE = uint4 (16 bytes) or a 2- / 4-byte element.  pieces = pieces per row.
// GATHER = false: dense[row(c)] <- sparse[i];  true: sparse[i] <- dense[row(c)] (zeros outside).
template <typename CT, typename PIECE, bool GATHER>
__global__ void __launch_bounds__(256)
dense_move_kernel(const CT* __restrict__ coords, int64_t n, int pieces, DenseShape shape, const PIECE* __restrict__ src,
                  PIECE* __restrict__ dst, int32_t* status) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t row = t / pieces;
  if (row >= n) return;
  const int piece = (int)(t - row * pieces);
  const int64_t d = dense_row(load_coord<CT>(coords, row), shape);
  if (d < 0) {
    if (status && piece == 0) atomicOr(status, ST_DEV_BAD_INDEX);
    if (GATHER) {
      PIECE zero;
      memset(&zero, 0, sizeof(PIECE));
      dst[row * pieces + piece] = zero;
    }
    return;
  }
  if (GATHER)
    dst[row * pieces + piece] = __ldg(src + d * pieces + piece);
  else
    dst[d * pieces + piece] = __ldg(src + row * pieces + piece);
}

template <typename CT, bool GATHER>
int launch_move(const void* coords, int64_t n, int row_bytes, int esize, DenseShape shape, const void* src, void* dst,
                int32_t* status, cudaStream_t s) {
  const bool wide = row_bytes % 16 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  const int pieces = wide ? row_bytes / 16 : row_bytes / esize;
  const int64_t threads = n * pieces;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  const CT* c = static_cast<const CT*>(coords);
  if (wide)
    dense_move_kernel<CT, uint4, GATHER><<<grid, 256, 0, s>>>(c, n, pieces, shape, static_cast<const uint4*>(src),
                                                               static_cast<uint4*>(dst), status);
  else if (esize == 4)
    dense_move_kernel<CT, uint32_t, GATHER><<<grid, 256, 0, s>>>(c, n, pieces, shape, static_cast<const uint32_t*>(src),
                                                                  static_cast<uint32_t*>(dst), status);
  else
    dense_move_kernel<CT, uint16_t, GATHER><<<grid, 256, 0, s>>>(c, n, pieces, shape, static_cast<const uint16_t*>(src),
                                                                  static_cast<uint16_t*>(dst), status);
  note_launches(1);
  return check_launch(GATHER ? "st_to_dense_bwd" : "st_to_dense_fwd");
}

int dense_args(const char* who, int dtype, const void* a, const void* coords, int coord_dtype, int64_t n, int C,
               int batch, const int32_t* shape_host, const void* b, DenseShape* shape, int* esize) {
  if (n < 0 || C < 1 || batch < 0 || !shape_host || (n > 0 && (!a || !coords || !b))) {
    set_error("%s: bad arguments", who);
    return ST_ERR_ARG;
  }
  if (dtype != ST_F32 && dtype != ST_F16 && dtype != ST_BF16) {
    set_error("%s: unknown feature dtype %d", who, dtype);
    return ST_ERR_DTYPE;
  }
  if (coord_dtype != ST_I16 && coord_dtype != ST_I32) {
    set_error("%s: unknown coordinate dtype %d", who, coord_dtype);
    return ST_ERR_DTYPE;
  }
  if (shape_host[0] < 0 || shape_host[1] < 0 || shape_host[2] < 0) {
    set_error("%s: negative spatial extent", who);
    return ST_ERR_ARG;
  }
  *shape = DenseShape{batch, shape_host[0], shape_host[1], shape_host[2]};
  *esize = dtype == ST_F32 ? 4 : 2;
  return ST_OK;
}

// Channel-wise concatenation of two feature matrices and its inverse, in 16-byte pieces: whole[r] = left[r] | right[r].
// The split hands an autograd graph two CONTIGUOUS gradients where slicing a concatenated gradient gives two strided
// views that every consumer then has to copy.
template <bool SPLIT>
__global__ void __launch_bounds__(256)
cols_kernel(uint4* __restrict__ whole, int64_t n, int pieces, int left_pieces, uint4* __restrict__ left,
            uint4* __restrict__ right) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= n * pieces) return;
  const int64_t row = t / pieces;
  const int p = (int)(t - row * pieces);
  uint4* part = p < left_pieces ? left + row * left_pieces + p : right + row * (pieces - left_pieces) + (p - left_pieces);
  if (SPLIT)
    *part = whole[t];
  else
    whole[t] = *part;
}

}  // namespace
}  // namespace st

using namespace st;

extern "C" {

int st_to_dense_fwd(int dtype, const void* feats, const void* coords, int coord_dtype, int64_t n, int C, int batch,
                    const int32_t* shape_host, void* dense, int32_t* status, void* stream) {
  DenseShape shape;
  int esize;
  int rc = dense_args("st_to_dense_fwd", dtype, feats, coords, coord_dtype, n, C, batch, shape_host, dense, &shape, &esize);
  if (rc != ST_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t cells = (int64_t)batch * shape.X * shape.Y * shape.Z;
  if (cells > 0) {
    if (!dense) {
      set_error("st_to_dense_fwd: null output");
      return ST_ERR_ARG;
    }
    cudaMemsetAsync(dense, 0, (size_t)cells * C * esize, s);
  }
  if (n == 0 || cells == 0) return check_launch("st_to_dense_fwd");
  if (coord_dtype == ST_I32)
    return launch_move<int32_t, false>(coords, n, C * esize, esize, shape, feats, dense, status, s);
  return launch_move<int16_t, false>(coords, n, C * esize, esize, shape, feats, dense, status, s);
}

int st_to_dense_bwd(int dtype, const void* grad_dense, const void* coords, int coord_dtype, int64_t n, int C, int batch,
                    const int32_t* shape_host, void* grad_feats, void* stream) {
  DenseShape shape;
  int esize;
  int rc = dense_args("st_to_dense_bwd", dtype, grad_dense, coords, coord_dtype, n, C, batch, shape_host, grad_feats,
                      &shape, &esize);
  if (rc != ST_OK) return rc;
  if (n == 0) return ST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (coord_dtype == ST_I32)
    return launch_move<int32_t, true>(coords, n, C * esize, esize, shape, grad_dense, grad_feats, nullptr, s);
  return launch_move<int16_t, true>(coords, n, C * esize, esize, shape, grad_dense, grad_feats, nullptr, s);
}

static int cols_args(const char* who, const void* whole, int64_t n, int left_bytes, int right_bytes, const void* left,
                     const void* right) {
  if (n < 0 || left_bytes < 0 || right_bytes < 0 || (n > 0 && left_bytes + right_bytes > 0 && !whole) ||
      (n > 0 && left_bytes > 0 && !left) || (n > 0 && right_bytes > 0 && !right)) {
    set_error("%s: bad arguments", who);
    return ST_ERR_ARG;
  }
  const uintptr_t bits = reinterpret_cast<uintptr_t>(whole) | reinterpret_cast<uintptr_t>(left) | reinterpret_cast<uintptr_t>(right);
  if (left_bytes % 16 || right_bytes % 16 || (bits & 15)) {
    set_error("%s: rows and pointers must be multiples of 16 bytes", who);
    return ST_ERR_UNSUPPORTED;
  }
  return ST_OK;
}

int st_concat_cols(const void* left, const void* right, int64_t n, int left_bytes, int right_bytes, void* out, void* stream) {
  int rc = cols_args("st_concat_cols", out, n, left_bytes, right_bytes, left, right);
  if (rc != ST_OK) return rc;
  const int pieces = (left_bytes + right_bytes) / 16;
  if (n == 0 || pieces == 0) return ST_OK;
  cols_kernel<false><<<(unsigned)((n * pieces + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      static_cast<uint4*>(out), n, pieces, left_bytes / 16, const_cast<uint4*>(static_cast<const uint4*>(left)),
      const_cast<uint4*>(static_cast<const uint4*>(right)));
  note_launches(1);
  return check_launch("st_concat_cols");
}

int st_split_cols(const void* whole, int64_t n, int left_bytes, int right_bytes, void* left, void* right, void* stream) {
  int rc = cols_args("st_split_cols", whole, n, left_bytes, right_bytes, left, right);
  if (rc != ST_OK) return rc;
  const int pieces = (left_bytes + right_bytes) / 16;
  if (n == 0 || pieces == 0) return ST_OK;
  cols_kernel<true><<<(unsigned)((n * pieces + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      const_cast<uint4*>(static_cast<const uint4*>(whole)), n, pieces, left_bytes / 16, static_cast<uint4*>(left),
      static_cast<uint4*>(right));
  note_launches(1);
  return check_launch("st_split_cols");
}

}  // extern "C"
