// Tensor-core (tcgen05 / TMEM) implicit-GEMM convolution kernels: host-side interface.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace st {

// True if the tcgen05 gather kernel handles a product with c_red reduction channels and c_acc
// accumulator (output) channels in this dtype.
bool tc_supported(int dtype, int c_red, int c_acc);
// Process-wide switch: when off, tc_supported() answers false and the CUDA-core kernels run.
void tc_set_enabled(bool on);
// Process-wide switch: when off, products over a tile plan run their cp.async forms instead of the TMA-fed ones.
void tc_set_tma(bool on);
void tc_set_dense_tiles(bool on);

// OUT[r,:] = sum_k IN[map[r,k],:] . B_k over a stored (n_rows, K) map.
//   w_transposed = false: B_k = W[k]   with W (K, c_red, c_acc)   (forward)
//   w_transposed = true : B_k = W[k]^T with W (K, c_acc, c_red)   (dgrad over the inverse map)
// `plan` (all members may be null) describes how the rows are walked:
//   order : a permutation of the rows; tiles are formed from rows order[0..127], order[128..255], ...
//           (the result does not depend on it)
//   tmap, tmask : the map in tile-plan form for that order (see row_order.cu); when given, `map`
//           itself is not read.
struct MapPlan {
  const int32_t* order = nullptr;
  const int32_t* tmap = nullptr;
  const uint32_t* tmask = nullptr;
};
int tc_conv_gather(int dtype, const void* in, const void* w, const int32_t* map, const MapPlan& plan, void* out,
                   int64_t n_rows, int64_t n_src, int K, int c_red, int c_acc, bool w_transposed, cudaStream_t stream,
                   bool w_flip = false);   // w_flip: offset k multiplies with slice K-1-k

// Arguments of the hash-on-the-fly forms.
struct HashFlyArgs {
  const void* coords;      // (n_rows, 4) output coordinates
  int coord_dtype;         // ST_I16 / ST_I32
  const Offsets* offsets;
  const int64_t* keys;     // table over the (possibly scaled) input coordinates
  const int32_t* vals;
  int64_t capacity;
  const int32_t* shape;    // host, 3 values
  int stride;
};

// Forward over the table probed on the fly.
int tc_conv_gather_hashfly(int dtype, const void* in, const void* w, const HashFlyArgs& h, void* out, int64_t n_rows,
                           int64_t n_src, int K, int c_red, int c_acc, cudaStream_t stream);
// Feature gradient without a stored map, gather form over a table of the OUTPUT coordinates.
int tc_conv_dgrad_inverse(int dtype, const void* dy, const void* w, const int32_t* q_coords, const Offsets& off,
                          const int64_t* out_keys, const int32_t* out_vals, int64_t out_capacity, int stride, void* dx,
                          int64_t n_in, int64_t n_out, int K, int cin, int cout, cudaStream_t stream);
int tc_conv_wgrad_hashfly(int dtype, const void* x, const void* dy, const HashFlyArgs& h, float* partial,
                          int* n_chunks_out, int64_t n_rows, int64_t n_src, int K, int cin, int cout,
                          cudaStream_t stream);

// Tensor-core weight gradient: fills fp32 partials (n_chunks, K, cin, cout) that the caller reduces.
bool tc_wgrad_supported(int dtype, int64_t n_rows, int K, int cin, int cout);
int64_t tc_wgrad_partial_bytes(int dtype, int64_t n_rows, int K, int cin, int cout);
// inverse_plan: `plan` is the tile plan of the INVERSE map; then n_rows counts the rows of x (the plan's rows) and
// n_src the rows of dy (the rows the plan's entries name).
int tc_conv_wgrad(int dtype, const void* x, const void* dy, const int32_t* map, const MapPlan& plan, float* partial,
                  int* n_chunks_out, int64_t n_rows, int64_t n_src, int K, int cin, int cout, cudaStream_t stream,
                  bool inverse_plan = false, void* sorted_rows = nullptr, bool presorted = false);
// Whether tc_conv_wgrad over a tile plan with a row order would copy dY into tile order (into `sorted_rows`), and that
// copy alone; with it made beforehand, tc_conv_wgrad takes presorted = true.
bool tc_wgrad_sorts_rows(int dtype, int64_t n_rows, int K, int cin, int cout);
int tc_wgrad_sort_rows(int dtype, const void* dy, const int32_t* order, int64_t n_rows, int cout, void* sorted,
                       cudaStream_t stream);

// Cycle counters of timing experiments (see Params2::dbg).
int tc_read_prof(long long* host_out, int n);

// Copies the sticky device status words of the tensor-core kernels (flags, wait site, block, extra)
// to host memory and synchronises the stream.
int tc_read_status(int32_t* host_out4, cudaStream_t stream, bool wait = true);
int tc_clear_status(cudaStream_t stream);

}  // namespace st
