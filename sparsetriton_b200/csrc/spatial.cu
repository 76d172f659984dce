// Pooling and nearest-neighbour upsampling of sparse tensors.
//
// Pooling: every input voxel belongs to exactly one output cell, out = floor((in + padding - ks/2) / stride)
// per axis.  Output rows are the distinct cells in ascending (batch, x, y, z) order.  The cell of every
// input becomes an integer key, the (key, row) pairs are radix-sorted, segment heads are marked and
// scanned, and the features of each output row are reduced over its own contiguous segment of the
// sorted list: no atomics, no -inf / zero prefill, fp32 accumulation in a fixed order.  The backward
// pass is a gather per input row (mean: grad / count; max: grad where the input equals the maximum).
//
// Upsampling: input row i becomes the scale^3 output rows i*scale^3 + (dx*scale + dy)*scale + dz at
// coordinates in*scale + (dx, dy, dz) with the same features; backward sums those rows in fp32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "radix_sort.cuh"

namespace st {

namespace {

struct PoolGeom {
  int shift;            // padding - kernel_size / 2
  int stride;
  int lo[3];            // smallest cell index per axis (may be negative)
  int ext[3];           // cells per axis
  int batch;
};

__host__ __device__ __forceinline__ int floor_div(int a, int b) {
  int q = a / b;
  return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q;
}

struct PoolScratch {
  unsigned long long *keys_a, *keys_b;
  int32_t *vals_a, *vals_b;
  uint32_t *hist, *totals;
  uint32_t* heads;      // per sorted position: 1 at the first element of a segment, then its exclusive scan
  void* scan_tmp;
};

int64_t pool_carve(PoolScratch* s, void* ws, int64_t n) {
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    char* p = ws ? static_cast<char*>(ws) + off : nullptr;
    off += align_up(bytes > 0 ? bytes : 1, 256);
    return p;
  };
  const int64_t nn = n > 0 ? n : 1;
  s->keys_a = reinterpret_cast<unsigned long long*>(take(nn * 8));
  s->keys_b = reinterpret_cast<unsigned long long*>(take(nn * 8));
  s->vals_a = reinterpret_cast<int32_t*>(take(nn * 4));
  s->vals_b = reinterpret_cast<int32_t*>(take(nn * 4));
  s->hist = reinterpret_cast<uint32_t*>(take(sort_hist_bytes(nn)));
  s->totals = reinterpret_cast<uint32_t*>(take(kBucketsMax * 4));
  s->heads = reinterpret_cast<uint32_t*>(take(nn * 4));
  s->scan_tmp = take(scan_tmp_bytes(nn));
  return off;
}

int key_bits_of(const PoolGeom& g) {
  unsigned long long cells = (unsigned long long)(g.batch > 0 ? g.batch : 1);
  for (int a = 0; a < 3; ++a) cells *= (unsigned long long)(g.ext[a] > 0 ? g.ext[a] : 1);
  int bits = 1;
  while (bits < 64 && (cells >> bits) != 0) ++bits;
  return bits;
}

// key = linear index of the cell in the (batch, ext0, ext1, ext2) box: ascending keys = ascending
// (batch, x, y, z).  Inputs outside the stated grid or batch get the key past every cell (sorted last,
// no output row) and raise ST_DEV_BAD_INDEX.
template <typename CT>
__global__ void __launch_bounds__(256)
pool_keys_kernel(const CT* __restrict__ coords, int64_t n, PoolGeom g, Int3 in_shape, unsigned long long invalid_key,
                 unsigned long long* __restrict__ keys, int32_t* __restrict__ vals, int32_t* status) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const int4 c = load_coord<CT>(coords, i);
  unsigned long long key = invalid_key;
  if ((unsigned)c.x < (unsigned)g.batch && (unsigned)c.y < (unsigned)in_shape.x && (unsigned)c.z < (unsigned)in_shape.y &&
      (unsigned)c.w < (unsigned)in_shape.z) {
    const int x = floor_div(c.y + g.shift, g.stride) - g.lo[0];
    const int y = floor_div(c.z + g.shift, g.stride) - g.lo[1];
    const int z = floor_div(c.w + g.shift, g.stride) - g.lo[2];
    key = (((unsigned long long)c.x * g.ext[0] + x) * g.ext[1] + y) * g.ext[2] + z;
  } else {
    atomicOr(status, ST_DEV_BAD_INDEX);
  }
  keys[i] = key;
  vals[i] = (int32_t)i;
}

__global__ void __launch_bounds__(256)
pool_heads_kernel(const unsigned long long* __restrict__ sorted_keys, int64_t n, unsigned long long invalid_key,
                  uint32_t* __restrict__ heads) {
  const int64_t p = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (p >= n) return;
  const unsigned long long k = sorted_keys[p];
  heads[p] = (k != invalid_key && (p == 0 || sorted_keys[p - 1] != k)) ? 1u : 0u;
}

// After the scan heads[p] = number of segment heads before p.  A head at p opens output row heads[p].
template <typename CT>
__global__ void __launch_bounds__(256)
pool_write_kernel(const unsigned long long* __restrict__ sorted_keys, const int32_t* __restrict__ sorted_rows,
                  const uint32_t* __restrict__ heads, int64_t n, int64_t n_out, PoolGeom g, unsigned long long invalid_key,
                  CT* __restrict__ out_coords, int32_t* __restrict__ in_to_out, int32_t* __restrict__ members,
                  int32_t* __restrict__ seg_start) {
  const int64_t p = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (p > n) return;
  if (p == n) {
    // close the last segment: positions holding the invalid key are not members of any row
    int64_t live = n;
    // (binary search for the first invalid key; sorted last)
    int64_t lo = 0, hi = n;
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (sorted_keys[mid] == invalid_key) hi = mid; else lo = mid + 1;
    }
    live = lo;
    seg_start[n_out] = (int32_t)live;
    return;
  }
  const unsigned long long k = sorted_keys[p];
  const int32_t row = sorted_rows[p];
  members[p] = row;
  if (k == invalid_key) {
    in_to_out[row] = -1;
    return;
  }
  const bool head = p == 0 || sorted_keys[p - 1] != k;
  const uint32_t o = head ? heads[p] : heads[p] - 1u;      // exclusive count of heads before p
  in_to_out[row] = (int32_t)o;
  if (head) {
    seg_start[o] = (int32_t)p;
    unsigned long long r = k;
    const int z = (int)(r % g.ext[2]); r /= g.ext[2];
    const int y = (int)(r % g.ext[1]); r /= g.ext[1];
    const int x = (int)(r % g.ext[0]); r /= g.ext[0];
    store_coord<CT>(out_coords, o, (int)r, x + g.lo[0], y + g.lo[1], z + g.lo[2]);
  }
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One thread per (output row, channel): consecutive threads read consecutive channels of the same
// member rows.  MAX = false: mean over the segment; true: maximum.
template <typename T, bool MAX>
__global__ void __launch_bounds__(256)
pool_fwd_kernel(const T* __restrict__ feats, int C, const int32_t* __restrict__ members,
                const int32_t* __restrict__ seg_start, int64_t n_out, T* __restrict__ out) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t o = t / C;
  if (o >= n_out) return;
  const int c = (int)(t - o * C);
  const int begin = __ldg(seg_start + o), end = __ldg(seg_start + o + 1);
  float acc = MAX ? -INFINITY : 0.f;
  for (int p = begin; p < end; ++p) {
    const float v = to_f32<T>(feats[(int64_t)__ldg(members + p) * C + c]);
    acc = MAX ? fmaxf(acc, v) : acc + v;
  }
  if (!MAX) acc /= (float)(end - begin);
  out[t] = from_f32<T>(acc);
}

template <typename T, bool MAX>
__global__ void __launch_bounds__(256)
pool_bwd_kernel(const T* __restrict__ grad_out, const T* __restrict__ feats, const T* __restrict__ out, int C,
                const int32_t* __restrict__ in_to_out, const int32_t* __restrict__ seg_start, int64_t n,
                T* __restrict__ grad_in) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t i = t / C;
  if (i >= n) return;
  const int c = (int)(t - i * C);
  const int32_t o = __ldg(in_to_out + i);
  float g = 0.f;
  if (o >= 0) {
    const float go = to_f32<T>(grad_out[(int64_t)o * C + c]);
    if (MAX) {
      // every input that equals the maximum receives the gradient, as the reference's `in == out` test does
      g = (to_f32<T>(feats[t]) == to_f32<T>(out[(int64_t)o * C + c])) ? go : 0.f;
    } else {
      g = go / (float)(__ldg(seg_start + o + 1) - __ldg(seg_start + o));
    }
  }
  grad_in[t] = from_f32<T>(g);
}

template <typename CT, typename T>
__global__ void __launch_bounds__(256)
upsample_fwd_kernel(const T* __restrict__ feats, const CT* __restrict__ coords, int64_t n, int C, int scale,
                    T* __restrict__ out_feats, CT* __restrict__ out_coords) {
  // thread = (output row, channel); channel 0 also writes the coordinate
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int s3 = scale * scale * scale;
  const int64_t o = t / C;
  if (o >= n * s3) return;
  const int c = (int)(t - o * C);
  const int64_t i = o / s3;
  const int step = (int)(o - i * s3);
  out_feats[t] = feats[i * C + c];
  if (c == 0) {
    const int4 q = load_coord<CT>(coords, i);
    const int dz = step % scale, dy = (step / scale) % scale, dx = step / (scale * scale);
    store_coord<CT>(out_coords, o, q.x, q.y * scale + dx, q.z * scale + dy, q.w * scale + dz);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
upsample_bwd_kernel(const T* __restrict__ grad_out, int64_t n, int C, int s3, T* __restrict__ grad_in) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t i = t / C;
  if (i >= n) return;
  const int c = (int)(t - i * C);
  float acc = 0.f;
  for (int step = 0; step < s3; ++step) acc += to_f32<T>(grad_out[(i * s3 + step) * C + c]);
  grad_in[t] = from_f32<T>(acc);
}

bool pool_geom(int ks, int pad, int stride, const int32_t* shape_host, int batch, PoolGeom* g) {
  if (ks < 1 || stride < 1 || !shape_host || batch < 0) return false;
  g->shift = pad - ks / 2;
  g->stride = stride;
  g->batch = batch;
  for (int a = 0; a < 3; ++a) {
    if (shape_host[a] < 0) return false;
    g->lo[a] = floor_div(g->shift, stride);
    const int hi = floor_div((shape_host[a] > 0 ? shape_host[a] - 1 : 0) + g->shift, stride);
    g->ext[a] = hi - g->lo[a] + 1;
  }
  return true;
}

}  // namespace
}  // namespace st

using namespace st;

#define ST_FEAT_DISPATCH(dtype, ...)                                  \
  switch (dtype) {                                                      \
    case ST_F32: { using T = float; __VA_ARGS__; break; }                      \
    case ST_F16: { using T = __half; __VA_ARGS__; break; }                     \
    case ST_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    default: set_error("unknown feature dtype %d", dtype); return ST_ERR_DTYPE; \
  }

extern "C" {

int64_t st_pool_workspace_bytes(int64_t n) {
  PoolScratch s;
  return pool_carve(&s, nullptr, n);
}

int st_pool_count(const void* coords, int64_t n, int coord_dtype, int kernel_size, int padding, int stride,
                  const int32_t* shape_host, int batch, void* workspace, int64_t workspace_bytes, int64_t* n_out,
                  int32_t* status, void* stream) {
  PoolGeom g;
  if (n < 0 || n > 0x7FFFFFFFll || !n_out || !status || !pool_geom(kernel_size, padding, stride, shape_host, batch, &g) ||
      (n > 0 && (!coords || !workspace))) {
    set_error("st_pool_count: bad arguments");
    return ST_ERR_ARG;
  }
  if (coord_dtype != ST_I16 && coord_dtype != ST_I32) {
    set_error("st_pool_count: unknown coordinate dtype %d", coord_dtype);
    return ST_ERR_DTYPE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) return exclusive_scan_u32(nullptr, nullptr, 0, nullptr, n_out, s);
  PoolScratch w;
  if (workspace_bytes < pool_carve(&w, workspace, n) || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("st_pool_count: workspace too small or not 256-byte aligned");
    return ST_ERR_WORKSPACE;
  }
  const int bits = key_bits_of(g);           // keys 0 .. cells-1 are real cells, `cells` itself marks invalid rows
  if (bits > 62) {
    set_error("st_pool_count: grid of more than 2^62 cells");
    return ST_ERR_UNSUPPORTED;
  }
  unsigned long long cells = (unsigned long long)(g.batch > 0 ? g.batch : 1);
  for (int a = 0; a < 3; ++a) cells *= (unsigned long long)(g.ext[a] > 0 ? g.ext[a] : 1);
  const Int3 in_shape = {shape_host[0], shape_host[1], shape_host[2]};
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (coord_dtype == ST_I32)
    pool_keys_kernel<int32_t><<<grid, 256, 0, s>>>(static_cast<const int32_t*>(coords), n, g, in_shape, cells, w.keys_a,
                                                   w.vals_a, status);
  else
    pool_keys_kernel<int16_t><<<grid, 256, 0, s>>>(static_cast<const int16_t*>(coords), n, g, in_shape, cells, w.keys_a,
                                                   w.vals_a, status);
  note_launches(1);
  unsigned long long* sorted_keys = nullptr;
  radix_sort_pairs<unsigned long long>(w.keys_a, w.vals_a, w.keys_b, w.vals_b, n, bits, w.hist, w.totals, &sorted_keys,
                                       nullptr, s);
  pool_heads_kernel<<<grid, 256, 0, s>>>(sorted_keys, n, cells, w.heads);
  note_launches(1);
  int rc = check_launch("st_pool_count");
  if (rc != ST_OK) return rc;
  return exclusive_scan_u32(w.heads, w.heads, n, w.scan_tmp, n_out, s);
}

int st_pool_write(const void* coords, int64_t n, int coord_dtype, int kernel_size, int padding, int stride,
                  const int32_t* shape_host, int batch, void* workspace, int64_t workspace_bytes, void* out_coords,
                  int64_t n_out, int32_t* in_to_out, int32_t* members, int32_t* seg_start, void* stream) {
  PoolGeom g;
  if (n < 0 || n_out < 0 || !pool_geom(kernel_size, padding, stride, shape_host, batch, &g) || !seg_start ||
      (n > 0 && (!coords || !workspace || !in_to_out || !members)) || (n_out > 0 && !out_coords)) {
    set_error("st_pool_write: bad arguments");
    return ST_ERR_ARG;
  }
  if (coord_dtype != ST_I16 && coord_dtype != ST_I32) {
    set_error("st_pool_write: unknown coordinate dtype %d", coord_dtype);
    return ST_ERR_DTYPE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) {
    cudaMemsetAsync(seg_start, 0, sizeof(int32_t), s);
    return check_launch("st_pool_write");
  }
  PoolScratch w;
  if (workspace_bytes < pool_carve(&w, workspace, n)) {
    set_error("st_pool_write: workspace too small");
    return ST_ERR_WORKSPACE;
  }
  unsigned long long cells = (unsigned long long)(g.batch > 0 ? g.batch : 1);
  for (int a = 0; a < 3; ++a) cells *= (unsigned long long)(g.ext[a] > 0 ? g.ext[a] : 1);
  // the same pass count as st_pool_count decides which ping-pong buffer holds the sorted pairs
  const bool in_b = sort_passes_for_bits(key_bits_of(g)) % 2 == 1;
  const unsigned long long* sorted_keys = in_b ? w.keys_b : w.keys_a;
  const int32_t* sorted_rows = in_b ? w.vals_b : w.vals_a;
  const unsigned grid = (unsigned)((n + 1 + 255) / 256);
  if (coord_dtype == ST_I32)
    pool_write_kernel<int32_t><<<grid, 256, 0, s>>>(sorted_keys, sorted_rows, w.heads, n, n_out, g, cells,
                                                    static_cast<int32_t*>(out_coords), in_to_out, members, seg_start);
  else
    pool_write_kernel<int16_t><<<grid, 256, 0, s>>>(sorted_keys, sorted_rows, w.heads, n, n_out, g, cells,
                                                    static_cast<int16_t*>(out_coords), in_to_out, members, seg_start);
  note_launches(1);
  return check_launch("st_pool_write");
}

int st_pool_fwd(int dtype, const void* feats, int C, const int32_t* members, const int32_t* seg_start, int64_t n_out,
                int mode_max, void* out, void* stream) {
  if (C < 1 || n_out < 0 || (n_out > 0 && (!feats || !members || !seg_start || !out))) {
    set_error("st_pool_fwd: bad arguments");
    return ST_ERR_ARG;
  }
  if (n_out == 0) return ST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((n_out * C + 255) / 256);
  ST_FEAT_DISPATCH(dtype, {
    if (mode_max)
      pool_fwd_kernel<T, true><<<grid, 256, 0, s>>>(static_cast<const T*>(feats), C, members, seg_start, n_out,
                                                    static_cast<T*>(out));
    else
      pool_fwd_kernel<T, false><<<grid, 256, 0, s>>>(static_cast<const T*>(feats), C, members, seg_start, n_out,
                                                     static_cast<T*>(out));
  });
  note_launches(1);
  return check_launch("st_pool_fwd");
}

int st_pool_bwd(int dtype, const void* grad_out, const void* feats, const void* out, int C, const int32_t* in_to_out,
                const int32_t* seg_start, int64_t n, int mode_max, void* grad_in, void* stream) {
  if (C < 1 || n < 0 || (n > 0 && (!grad_out || !in_to_out || !seg_start || !grad_in || (mode_max && (!feats || !out))))) {
    set_error("st_pool_bwd: bad arguments");
    return ST_ERR_ARG;
  }
  if (n == 0) return ST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((n * C + 255) / 256);
  ST_FEAT_DISPATCH(dtype, {
    if (mode_max)
      pool_bwd_kernel<T, true><<<grid, 256, 0, s>>>(static_cast<const T*>(grad_out), static_cast<const T*>(feats),
                                                    static_cast<const T*>(out), C, in_to_out, seg_start, n,
                                                    static_cast<T*>(grad_in));
    else
      pool_bwd_kernel<T, false><<<grid, 256, 0, s>>>(static_cast<const T*>(grad_out), nullptr, nullptr, C, in_to_out,
                                                     seg_start, n, static_cast<T*>(grad_in));
  });
  note_launches(1);
  return check_launch("st_pool_bwd");
}

int st_upsample_fwd(int dtype, const void* feats, const void* coords, int coord_dtype, int64_t n, int C, int scale,
                    void* out_feats, void* out_coords, void* stream) {
  if (n < 0 || C < 1 || scale < 1 || (n > 0 && (!feats || !coords || !out_feats || !out_coords))) {
    set_error("st_upsample_fwd: bad arguments");
    return ST_ERR_ARG;
  }
  if (coord_dtype != ST_I16 && coord_dtype != ST_I32) {
    set_error("st_upsample_fwd: unknown coordinate dtype %d", coord_dtype);
    return ST_ERR_DTYPE;
  }
  if (n == 0) return ST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t threads = n * scale * scale * scale * C;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  ST_FEAT_DISPATCH(dtype, {
    if (coord_dtype == ST_I32)
      upsample_fwd_kernel<int32_t, T><<<grid, 256, 0, s>>>(static_cast<const T*>(feats), static_cast<const int32_t*>(coords),
                                                           n, C, scale, static_cast<T*>(out_feats),
                                                           static_cast<int32_t*>(out_coords));
    else
      upsample_fwd_kernel<int16_t, T><<<grid, 256, 0, s>>>(static_cast<const T*>(feats), static_cast<const int16_t*>(coords),
                                                           n, C, scale, static_cast<T*>(out_feats),
                                                           static_cast<int16_t*>(out_coords));
  });
  note_launches(1);
  return check_launch("st_upsample_fwd");
}

int st_upsample_bwd(int dtype, const void* grad_out, int64_t n, int C, int scale, void* grad_in, void* stream) {
  if (n < 0 || C < 1 || scale < 1 || (n > 0 && (!grad_out || !grad_in))) {
    set_error("st_upsample_bwd: bad arguments");
    return ST_ERR_ARG;
  }
  if (n == 0) return ST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((n * C + 255) / 256);
  ST_FEAT_DISPATCH(dtype, {
    upsample_bwd_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(grad_out), n, C, scale * scale * scale,
                                                static_cast<T*>(grad_in));
  });
  note_launches(1);
  return check_launch("st_upsample_bwd");
}

}  // extern "C"
