// C entry points of the convolution products: argument checks, dtype dispatch, choice between the
// tensor-core (tcgen05) kernels and the general CUDA-core kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "conv_maps.cuh"
#include "conv_tc.cuh"

namespace st {

int wgrad_chunks(int64_t n_out);
int reduce_partials(int dtype, const float* partial, int chunks, int64_t n, void* out, cudaStream_t s);

template <typename T, typename Map>
int simt_gather(const T* in, const T* w, const Map& map, T* out, int64_t n_rows, int64_t n_src, int K, int c_red,
                int c_acc, bool w_transposed, cudaStream_t s);
template <typename T, typename Map>
int simt_scatter(const T* in, const T* w, const Map& map, T* out, float* out32, int64_t n_rows, int64_t n_dst, int K,
                 int c_red, int c_acc, cudaStream_t s);
template <typename T, typename Map>
int simt_wgrad(const T* x, const T* dy, const Map& map, T* dw, float* partial, int64_t n_rows, int64_t n_src, int K,
               int cin, int cout, cudaStream_t s);

static int64_t elem_size(int dtype) { return dtype == ST_F32 ? 4 : 2; }

static int check_conv_args(const char* who, int dtype, int64_t n_in, int64_t n_out, int K, int cin, int cout) {
  if (dtype != ST_F32 && dtype != ST_F16 && dtype != ST_BF16) {
    set_error("%s: unknown feature dtype %d", who, dtype);
    return ST_ERR_DTYPE;
  }
  if (n_in < 0 || n_out < 0 || K < 1 || K > ST_MAX_KVOL || cin < 1 || cout < 1 || n_in > 0x7FFFFFFFll ||
      n_out > 0x7FFFFFFFll) {
    set_error("%s: bad sizes n_in=%lld n_out=%lld K=%d cin=%d cout=%d", who, (long long)n_in, (long long)n_out, K,
              cin, cout);
    return ST_ERR_ARG;
  }
  return ST_OK;
}

static int64_t wgrad_partial_bytes(int64_t n_out, int K, int cin, int cout) {
  return align_up((int64_t)wgrad_chunks(n_out) * K * cin * cout * 4, 256);
}

// Partials of whichever weight-gradient kernel would run, so one workspace serves both.
// The tensor-core form also keeps a copy of dY in tile order behind its partials (see tc_conv_wgrad).
static int64_t wgrad_sorted_offset(int dtype, int64_t n_out, int K, int cin, int cout) {
  return align_up(tc_wgrad_partial_bytes(dtype, n_out, K, cin, cout), 256);
}
static int64_t wgrad_workspace_bytes(int dtype, int64_t n_out, int K, int cin, int cout) {
  int64_t simt = wgrad_partial_bytes(n_out, K, cin, cout);
  int64_t tcb = wgrad_sorted_offset(dtype, n_out, K, cin, cout);
  if (tcb > 0) tcb += align_up(n_out * (int64_t)cout * (dtype == ST_F32 ? 4 : 2), 256);
  return simt > tcb ? simt : tcb;
}

// Scratch of the gather-form feature gradient of the hash-on-the-fly algorithm: a status word, a
// table over the output coordinates (power-of-two capacity >= 2 n_out) and one int32x4 coordinate
// per input row.
static int64_t out_table_capacity(int64_t n_out) {
  int64_t cap = 1024;
  while (cap < 2 * n_out) cap <<= 1;
  return cap;
}
static int64_t inverse_dgrad_bytes(int64_t n_in, int64_t n_out) {
  const int64_t cap = out_table_capacity(n_out);
  return 256 + align_up(cap * 8, 256) + align_up(cap * 4, 256) + align_up(n_in * 16, 256);
}

// Dispatch a callable over the feature dtype.
template <typename F>
static int by_dtype(int dtype, F&& f) {
  switch (dtype) {
    case ST_F32: return f(static_cast<float*>(nullptr));
    case ST_F16: return f(static_cast<__half*>(nullptr));
    default: return f(static_cast<__nv_bfloat16*>(nullptr));
  }
}

template <typename CT>
static HashFlyMap<CT> make_hashfly(const void* coords, const Offsets& off, const int64_t* keys, const int32_t* vals,
                                   int64_t capacity, const int32_t* shape, int stride) {
  HashFlyMap<CT> m;
  m.coords = static_cast<const CT*>(coords);
  m.off = off;
  m.table = make_table(keys, vals, capacity);
  m.shape = Int3{shape[0], shape[1], shape[2]};
  m.stride = stride;
  return m;
}

static int check_hashfly_args(const char* who, const void* coords, int coord_dtype, const int32_t* offsets_host,
                              const int64_t* keys, const int32_t* vals, int64_t capacity, const int32_t* shape,
                              int stride, int K, int64_t n_out, Offsets* off) {
  if (coord_dtype != ST_I16 && coord_dtype != ST_I32) {
    set_error("%s: unknown coordinate dtype %d", who, coord_dtype);
    return ST_ERR_DTYPE;
  }
  if (!offsets_host || !shape || stride < 1 || capacity < 0 || capacity > 0x7FFFFFFFll ||
      (capacity > 0 && (!keys || !vals)) || (n_out > 0 && !coords)) {
    set_error("%s: bad map arguments", who);
    return ST_ERR_ARG;
  }
  if (!pack_offsets(offsets_host, K, off)) {
    set_error("%s: offset outside int16", who);
    return ST_ERR_UNSUPPORTED;
  }
  return ST_OK;
}

}  // namespace st

using namespace st;

extern "C" {

int st_conv_uses_tensor_cores(int dtype, int cin, int cout) { return tc_supported(dtype, cin, cout) ? 1 : 0; }

int st_debug_prof(long long* out, int n) { return st::tc_read_prof(out, n); }

int st_set_tensor_cores(int enable) {
  tc_set_enabled(enable != 0);
  return ST_OK;
}

int st_set_tma(int enable) {
  tc_set_tma(enable != 0);
  return ST_OK;
}

int st_set_dense_tiles(int enable) {
  tc_set_dense_tiles(enable != 0);
  return ST_OK;
}

int st_device_status(int32_t* out4, void* stream) {
  if (!out4) {
    set_error("st_device_status: null output");
    return ST_ERR_ARG;
  }
  return tc_read_status(out4, (cudaStream_t)stream);
}

int st_device_status_enqueue(int32_t* pinned_out4, void* stream) {
  if (!pinned_out4) {
    set_error("st_device_status_enqueue: null output");
    return ST_ERR_ARG;
  }
  return tc_read_status(pinned_out4, (cudaStream_t)stream, /*wait=*/false);
}

int st_device_status_clear(void* stream) { return tc_clear_status((cudaStream_t)stream); }

int64_t st_conv_workspace_bytes(int dtype, int64_t n_in, int64_t n_out, int K, int cin, int cout) {
  (void)n_in;
  if (n_out < 0 || K < 1 || cin < 1 || cout < 1) return 256;
  return wgrad_workspace_bytes(dtype, n_out, K, cin, cout) + 256;
}

int64_t st_conv_hashfly_workspace_bytes(int dtype, int64_t n_in, int64_t n_out, int K, int cin, int cout) {
  if (n_in < 0 || n_out < 0 || K < 1 || cin < 1 || cout < 1) return 256;
  int64_t scatter = dtype == ST_F32 ? 0 : align_up(n_in * cin * 4, 256);
  int64_t wg = wgrad_workspace_bytes(dtype, n_out, K, cin, cout);
  int64_t inv = inverse_dgrad_bytes(n_in, n_out);
  int64_t m = scatter > wg ? scatter : wg;
  return (m > inv ? m : inv) + 256;
}

int st_conv_fwd_planned(int dtype, const void* X, const void* W, const int32_t* nbr, const int32_t* row_order,
                        const int32_t* tmap, const uint32_t* tmask, void* Y,
                        int64_t n_in, int64_t n_out, int K, int cin, int cout, void* workspace,
                        int64_t workspace_bytes, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  int rc = check_conv_args("st_conv_fwd", dtype, n_in, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  if (n_out == 0) return ST_OK;
  if (!X && n_in > 0 || !W || !nbr || !Y) {
    set_error("st_conv_fwd: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (tc_supported(dtype, cin, cout))
    return tc_conv_gather(dtype, X, W, nbr, MapPlan{row_order, tmap, tmask}, Y, n_out, n_in, K, cin, cout, /*w_transposed=*/false, s);
  StoredMap map{nbr, K};
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    return simt_gather<T, StoredMap>(static_cast<const T*>(X), static_cast<const T*>(W), map, static_cast<T*>(Y),
                                     n_out, n_in, K, cin, cout, false, s);
  });
}

int st_conv_fwd(int dtype, const void* X, const void* W, const int32_t* nbr, void* Y, int64_t n_in, int64_t n_out,
                int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  return st_conv_fwd_planned(dtype, X, W, nbr, nullptr, nullptr, nullptr, Y, n_in, n_out, K, cin, cout, workspace, workspace_bytes, stream);
}

int st_conv_dgrad_planned(int dtype, const void* dY, const void* W, const int32_t* inv, const int32_t* row_order,
                          const int32_t* tmap, const uint32_t* tmask, void* dX, int64_t n_in, int64_t n_out, int K, int cin, int cout, void* workspace,
                          int64_t workspace_bytes, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  int rc = check_conv_args("st_conv_dgrad", dtype, n_in, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  if (n_in == 0) return ST_OK;
  // the inverse map itself may be absent when its plan is given (st_map_plan_inverse) and the tensor-core
  // kernels take the shape: they read the map only through the plan
  const bool planned = tmap && tmask;
  const bool tc = tc_supported(dtype, cout, cin);
  if (!dY && n_out > 0 || !W || !dX || (!inv && !(planned && tc))) {
    set_error("st_conv_dgrad: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (tc)
    return tc_conv_gather(dtype, dY, W, inv, MapPlan{row_order, tmap, tmask}, dX, n_in, n_out, K, cout, cin, /*w_transposed=*/true, s);
  StoredMap map{inv, K};
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    return simt_gather<T, StoredMap>(static_cast<const T*>(dY), static_cast<const T*>(W), map, static_cast<T*>(dX),
                                     n_in, n_out, K, cout, cin, true, s);
  });
}

int st_conv_dgrad(int dtype, const void* dY, const void* W, const int32_t* inv, void* dX, int64_t n_in, int64_t n_out,
                  int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  return st_conv_dgrad_planned(dtype, dY, W, inv, nullptr, nullptr, nullptr, dX, n_in, n_out, K, cin, cout, workspace, workspace_bytes,
                               stream);
}

int st_conv_dgrad_mirrored(int dtype, const void* dY, const void* W, const int32_t* nbr, const int32_t* row_order,
                           const int32_t* tmap, const uint32_t* tmask, void* dX, int64_t n, int K, int cin, int cout,
                           void* workspace, int64_t workspace_bytes, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  int rc = check_conv_args("st_conv_dgrad_mirrored", dtype, n, n, K, cin, cout);
  if (rc != ST_OK) return rc;
  if (n == 0) return ST_OK;
  if (!dY || !W || !nbr || !dX) {
    set_error("st_conv_dgrad_mirrored: null pointer");
    return ST_ERR_ARG;
  }
  if (!tc_supported(dtype, cout, cin)) {
    set_error("st_conv_dgrad_mirrored: shape outside the tensor-core kernels; use st_conv_dgrad over the inverse map");
    return ST_ERR_UNSUPPORTED;
  }
  return tc_conv_gather(dtype, dY, W, nbr, MapPlan{row_order, tmap, tmask}, dX, n, n, K, cout, cin, /*w_transposed=*/true,
                        (cudaStream_t)stream, /*w_flip=*/true);
}

static int wgrad_planned(int dtype, const void* X, const void* dY, const int32_t* nbr, const int32_t* row_order,
                         const int32_t* tmap, const uint32_t* tmask, void* dW, int64_t n_in, int64_t n_out, int K, int cin,
                         int cout, void* workspace, int64_t workspace_bytes, void* stream, bool presorted) {
  int rc = check_conv_args("st_conv_wgrad", dtype, n_in, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  if (!dW || (n_out > 0 && (!X || !dY || !nbr))) {
    set_error("st_conv_wgrad: null pointer");
    return ST_ERR_ARG;
  }
  if (n_out > 0 && (!workspace || workspace_bytes < wgrad_workspace_bytes(dtype, n_out, K, cin, cout) ||
                    (reinterpret_cast<uintptr_t>(workspace) & 255))) {
    set_error("st_conv_wgrad: workspace too small or misaligned");
    return ST_ERR_WORKSPACE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (n_out > 0 && tc_wgrad_supported(dtype, n_out, K, cin, cout)) {
    int chunks = 0;
    void* sorted_rows = static_cast<char*>(workspace) + wgrad_sorted_offset(dtype, n_out, K, cin, cout);
    rc = tc_conv_wgrad(dtype, X, dY, nbr, MapPlan{row_order, tmap, tmask}, static_cast<float*>(workspace), &chunks, n_out, n_in, K, cin, cout, s,
                       /*inverse_plan=*/false, sorted_rows, presorted);
    if (rc != ST_OK) return rc;
    return reduce_partials(dtype, static_cast<const float*>(workspace), chunks, (int64_t)K * cin * cout, dW, s);
  }
  StoredMap map{nbr, K};
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    return simt_wgrad<T, StoredMap>(static_cast<const T*>(X), static_cast<const T*>(dY), map, static_cast<T*>(dW),
                                    static_cast<float*>(workspace), n_out, n_in, K, cin, cout, s);
  });
}

int st_conv_wgrad_planned(int dtype, const void* X, const void* dY, const int32_t* nbr, const int32_t* row_order,
                          const int32_t* tmap, const uint32_t* tmask, void* dW, int64_t n_in, int64_t n_out, int K, int cin,
                          int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  return wgrad_planned(dtype, X, dY, nbr, row_order, tmap, tmask, dW, n_in, n_out, K, cin, cout, workspace, workspace_bytes,
                       stream, /*presorted=*/false);
}

int st_conv_wgrad_presort(int dtype, const void* dY, const int32_t* row_order, int64_t n_out, int K, int cin, int cout,
                          void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = check_conv_args("st_conv_wgrad_presort", dtype, n_out, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  if (n_out == 0 || !row_order || !tc_wgrad_supported(dtype, n_out, K, cin, cout) ||
      !tc_wgrad_sorts_rows(dtype, n_out, K, cin, cout))
    return ST_ERR_UNSUPPORTED;                              // st_conv_wgrad_planned makes no copy for this layer
  if (!dY || !workspace || workspace_bytes < wgrad_workspace_bytes(dtype, n_out, K, cin, cout) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("st_conv_wgrad_presort: null dY, or workspace too small or misaligned");
    return ST_ERR_WORKSPACE;
  }
  void* sorted_rows = static_cast<char*>(workspace) + wgrad_sorted_offset(dtype, n_out, K, cin, cout);
  return tc_wgrad_sort_rows(dtype, dY, row_order, n_out, cout, sorted_rows, (cudaStream_t)stream);
}

int st_conv_wgrad_planned_presorted(int dtype, const void* X, const void* dY, const int32_t* nbr, const int32_t* row_order,
                                    const int32_t* tmap, const uint32_t* tmask, void* dW, int64_t n_in, int64_t n_out,
                                    int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  return wgrad_planned(dtype, X, dY, nbr, row_order, tmap, tmask, dW, n_in, n_out, K, cin, cout, workspace, workspace_bytes,
                       stream, /*presorted=*/true);
}

int64_t st_conv_wgrad_inverse_workspace_bytes(int dtype, int64_t n_in, int K, int cin, int cout) {
  if (n_in < 0 || K < 1 || cin < 1 || cout < 1) return 256;
  return align_up(tc_wgrad_partial_bytes(dtype, n_in, K, cin, cout), 256) + 256;
}

int st_conv_wgrad_inverse_planned(int dtype, const void* X, const void* dY, const int32_t* row_order, const int32_t* tmap,
                                  const uint32_t* tmask, void* dW, int64_t n_in, int64_t n_out, int K, int cin, int cout,
                                  void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = check_conv_args("st_conv_wgrad_inverse_planned", dtype, n_in, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  if (!dW || !tmap || !tmask || n_in < 1 || n_out < 1 || !X || !dY) {
    set_error("st_conv_wgrad_inverse_planned: null pointer or empty tensor");
    return ST_ERR_ARG;
  }
  if (!tc_wgrad_supported(dtype, n_in, K, cin, cout)) {
    set_error("st_conv_wgrad_inverse_planned: shape not served by the tensor-core kernels");
    return ST_ERR_UNSUPPORTED;
  }
  if (!workspace || workspace_bytes < st_conv_wgrad_inverse_workspace_bytes(dtype, n_in, K, cin, cout) - 256 ||
      (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("st_conv_wgrad_inverse_planned: workspace too small or misaligned");
    return ST_ERR_WORKSPACE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int chunks = 0;
  rc = tc_conv_wgrad(dtype, X, dY, nullptr, MapPlan{row_order, tmap, tmask}, static_cast<float*>(workspace), &chunks, n_in,
                     n_out, K, cin, cout, s, true);
  if (rc != ST_OK) return rc;
  return reduce_partials(dtype, static_cast<const float*>(workspace), chunks, (int64_t)K * cin * cout, dW, s);
}

int st_conv_wgrad(int dtype, const void* X, const void* dY, const int32_t* nbr, void* dW, int64_t n_in, int64_t n_out,
                  int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  return st_conv_wgrad_planned(dtype, X, dY, nbr, nullptr, nullptr, nullptr, dW, n_in, n_out, K, cin, cout, workspace, workspace_bytes,
                               stream);
}

int st_conv_fwd_hashfly(int dtype, const void* X, const void* W, const void* out_coords, int coord_dtype,
                        const int32_t* offsets_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                        const int32_t* lookup_shape_host, int lookup_stride, void* Y, int64_t n_in, int64_t n_out,
                        int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  int rc = check_conv_args("st_conv_fwd_hashfly", dtype, n_in, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  Offsets off;
  rc = check_hashfly_args("st_conv_fwd_hashfly", out_coords, coord_dtype, offsets_host, keys, vals, capacity,
                          lookup_shape_host, lookup_stride, K, n_out, &off);
  if (rc != ST_OK) return rc;
  if (n_out == 0) return ST_OK;
  if (!X && n_in > 0 || !W || !Y) {
    set_error("st_conv_fwd_hashfly: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (tc_supported(dtype, cin, cout)) {
    HashFlyArgs h{out_coords, coord_dtype, &off, keys, vals, capacity, lookup_shape_host, lookup_stride};
    return tc_conv_gather_hashfly(dtype, X, W, h, Y, n_out, n_in, K, cin, cout, s);
  }
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if (coord_dtype == ST_I32) {
      auto map = make_hashfly<int32_t>(out_coords, off, keys, vals, capacity, lookup_shape_host, lookup_stride);
      return simt_gather<T, HashFlyMap<int32_t>>(static_cast<const T*>(X), static_cast<const T*>(W), map,
                                                 static_cast<T*>(Y), n_out, n_in, K, cin, cout, false, s);
    }
    auto map = make_hashfly<int16_t>(out_coords, off, keys, vals, capacity, lookup_shape_host, lookup_stride);
    return simt_gather<T, HashFlyMap<int16_t>>(static_cast<const T*>(X), static_cast<const T*>(W), map,
                                               static_cast<T*>(Y), n_out, n_in, K, cin, cout, false, s);
  });
}

int st_conv_dgrad_hashfly(int dtype, const void* dY, const void* W, const void* out_coords, int coord_dtype,
                          const int32_t* offsets_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                          const int32_t* lookup_shape_host, int lookup_stride, void* dX, int64_t n_in, int64_t n_out,
                          int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = check_conv_args("st_conv_dgrad_hashfly", dtype, n_in, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  Offsets off;
  rc = check_hashfly_args("st_conv_dgrad_hashfly", out_coords, coord_dtype, offsets_host, keys, vals, capacity,
                          lookup_shape_host, lookup_stride, K, n_out, &off);
  if (rc != ST_OK) return rc;
  if (n_in == 0) return ST_OK;
  if (!dY && n_out > 0 || !W || !dX) {
    set_error("st_conv_dgrad_hashfly: null pointer");
    return ST_ERR_ARG;
  }
  if (tc_supported(dtype, cout, cin) && n_out > 0 && capacity > 0) {
    // Gather form: dX[i] = sum_k dY[o(i,k)] . W[k]^T with o found in a table over the output coordinates.
    if (!workspace || workspace_bytes < inverse_dgrad_bytes(n_in, n_out) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255)) {
      set_error("st_conv_dgrad_hashfly: workspace too small or misaligned");
      return ST_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t cap = out_table_capacity(n_out);
    char* p = static_cast<char*>(workspace);
    int32_t* status = reinterpret_cast<int32_t*>(p);
    p += 256;
    int64_t* okeys = reinterpret_cast<int64_t*>(p);
    p += align_up(cap * 8, 256);
    int32_t* ovals = reinterpret_cast<int32_t*>(p);
    p += align_up(cap * 4, 256);
    int32_t* q = reinterpret_cast<int32_t*>(p);
    cudaMemsetAsync(status, 0, 4, s);
    rc = st_hash_clear(okeys, ovals, cap, stream);
    if (rc != ST_OK) return rc;
    rc = st_hash_build(out_coords, n_out, coord_dtype, okeys, ovals, cap, status, stream);
    if (rc != ST_OK) return rc;
    rc = unpack_table_coords(keys, vals, capacity, q, n_in, s);
    if (rc != ST_OK) return rc;
    return tc_conv_dgrad_inverse(dtype, dY, W, q, off, okeys, ovals, cap, lookup_stride, dX, n_in, n_out, K, cin,
                                 cout, s);
  }
  float* out32 = static_cast<float*>(dX);
  if (dtype != ST_F32) {
    if (!workspace || workspace_bytes < align_up(n_in * cin * 4, 256) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255)) {
      set_error("st_conv_dgrad_hashfly: workspace too small or misaligned");
      return ST_ERR_WORKSPACE;
    }
    out32 = static_cast<float*>(workspace);
  }
  cudaStream_t s = (cudaStream_t)stream;
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if (coord_dtype == ST_I32) {
      auto map = make_hashfly<int32_t>(out_coords, off, keys, vals, capacity, lookup_shape_host, lookup_stride);
      return simt_scatter<T, HashFlyMap<int32_t>>(static_cast<const T*>(dY), static_cast<const T*>(W), map,
                                                  static_cast<T*>(dX), out32, n_out, n_in, K, cout, cin, s);
    }
    auto map = make_hashfly<int16_t>(out_coords, off, keys, vals, capacity, lookup_shape_host, lookup_stride);
    return simt_scatter<T, HashFlyMap<int16_t>>(static_cast<const T*>(dY), static_cast<const T*>(W), map,
                                                static_cast<T*>(dX), out32, n_out, n_in, K, cout, cin, s);
  });
}

int st_conv_wgrad_hashfly(int dtype, const void* X, const void* dY, const void* out_coords, int coord_dtype,
                          const int32_t* offsets_host, const int64_t* keys, const int32_t* vals, int64_t capacity,
                          const int32_t* lookup_shape_host, int lookup_stride, void* dW, int64_t n_in, int64_t n_out,
                          int K, int cin, int cout, void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = check_conv_args("st_conv_wgrad_hashfly", dtype, n_in, n_out, K, cin, cout);
  if (rc != ST_OK) return rc;
  Offsets off;
  rc = check_hashfly_args("st_conv_wgrad_hashfly", out_coords, coord_dtype, offsets_host, keys, vals, capacity,
                          lookup_shape_host, lookup_stride, K, n_out, &off);
  if (rc != ST_OK) return rc;
  if (!dW || (n_out > 0 && (!X || !dY))) {
    set_error("st_conv_wgrad_hashfly: null pointer");
    return ST_ERR_ARG;
  }
  if (n_out > 0 && (!workspace || workspace_bytes < wgrad_workspace_bytes(dtype, n_out, K, cin, cout) ||
                    (reinterpret_cast<uintptr_t>(workspace) & 255))) {
    set_error("st_conv_wgrad_hashfly: workspace too small or misaligned");
    return ST_ERR_WORKSPACE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (n_out > 0 && tc_wgrad_supported(dtype, n_out, K, cin, cout)) {
    HashFlyArgs h{out_coords, coord_dtype, &off, keys, vals, capacity, lookup_shape_host, lookup_stride};
    int chunks = 0;
    rc = tc_conv_wgrad_hashfly(dtype, X, dY, h, static_cast<float*>(workspace), &chunks, n_out, n_in, K, cin, cout, s);
    if (rc != ST_OK) return rc;
    return reduce_partials(dtype, static_cast<const float*>(workspace), chunks, (int64_t)K * cin * cout, dW, s);
  }
  return by_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if (coord_dtype == ST_I32) {
      auto map = make_hashfly<int32_t>(out_coords, off, keys, vals, capacity, lookup_shape_host, lookup_stride);
      return simt_wgrad<T, HashFlyMap<int32_t>>(static_cast<const T*>(X), static_cast<const T*>(dY), map,
                                                static_cast<T*>(dW), static_cast<float*>(workspace), n_out, n_in, K,
                                                cin, cout, s);
    }
    auto map = make_hashfly<int16_t>(out_coords, off, keys, vals, capacity, lookup_shape_host, lookup_stride);
    return simt_wgrad<T, HashFlyMap<int16_t>>(static_cast<const T*>(X), static_cast<const T*>(dY), map,
                                              static_cast<T*>(dW), static_cast<float*>(workspace), n_out, n_in, K, cin,
                                              cout, s);
  });
}

}  // extern "C"
