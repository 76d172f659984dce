// General-shape convolution kernels on the CUDA cores (fp32 FMA, fp32 accumulation).
//
// They serve every channel count and dtype, are the exact-fp32 path, and back the tensor-core
// kernels for shapes those do not cover.  Three products share one 64x64x16 register-tiled
// micro-kernel (256 threads, 4x4 accumulators each):
//   gather : OUT[r,:]  = sum_k IN[map(r,k),:] . B_k          forward, and dgrad over the inverse map
//   scatter: OUT32[map(r,k),:] += IN[r,:] . B_k               dgrad of the hash-on-the-fly form
//   wgrad  : P[chunk,k] = sum_{r in chunk} X[map(r,k),:]^T . dY[r,:]   then a fixed-order reduce
// (tile, offset) pairs without a single valid neighbour are skipped.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "conv_maps.cuh"

namespace st {

constexpr int BM = 64, BN = 64, BK = 16, kConvThreads = 256;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct Tiles {
  float a[BK][BM + 4];
  float b[BK][BN + 4];
};

__device__ __forceinline__ void micro_kernel(const Tiles& s, float (&acc)[4][4]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int kk = 0; kk < BK; ++kk) {
    float4 av = *reinterpret_cast<const float4*>(&s.a[kk][ty * 4]);
    float4 bv = *reinterpret_cast<const float4*>(&s.b[kk][tx * 4]);
    float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// B_k[r][a] = W[k*c_red*c_acc_total... ] addressed through two strides so that the same code reads
// W[k] (forward) or W[k]^T (dgrad): element (red, acc) sits at  wk + red*stride_red + acc*stride_acc.
template <typename T>
__device__ __forceinline__ void load_b_tile(Tiles& s, const T* wk, int red0, int c_red, int acc0, int c_acc,
                                            int64_t stride_red, int64_t stride_acc) {
  for (int e = threadIdx.x; e < BK * BN; e += kConvThreads) {
    int kk, n;
    if (stride_acc == 1) { kk = e / BN; n = e % BN; } else { n = e / BK; kk = e % BK; }
    int r = red0 + kk, a = acc0 + n;
    s.b[kk][n] = (r < c_red && a < c_acc) ? to_f<T>(wk[r * stride_red + a * stride_acc]) : 0.f;
  }
}

// ------------------------------------------------------------------------------------------ gather
template <typename T, typename Map>
__global__ void __launch_bounds__(kConvThreads)
conv_gather_kernel(const T* __restrict__ in, const T* __restrict__ w, Map map, T* __restrict__ out, int64_t n_rows,
                   int64_t n_src, int K, int c_red, int c_acc, int64_t stride_red, int64_t stride_acc) {
  __shared__ Tiles s;
  __shared__ int4 s_coord[BM];
  __shared__ int32_t s_idx[BM];
  const int64_t row0 = (int64_t)blockIdx.x * BM;
  const int acc0 = blockIdx.y * BN;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  float acc[4][4] = {};
  map.template prepare<BM>(s_coord, row0, n_rows);
  __syncthreads();
  for (int k = 0; k < K; ++k) {
    int any = 0;
    if (threadIdx.x < BM) {
      int64_t r = row0 + threadIdx.x;
      int32_t i = r < n_rows ? map.get(s_coord, threadIdx.x, r, k) : -1;
      if (i >= n_src) i = -1;
      s_idx[threadIdx.x] = i;
      any = i >= 0;
    }
    if (!__syncthreads_or(any)) continue;
    const T* wk = w + (int64_t)k * c_red * c_acc;
    for (int red0 = 0; red0 < c_red; red0 += BK) {
      for (int e = threadIdx.x; e < BM * BK; e += kConvThreads) {
        int m = e / BK, kk = e % BK;
        int32_t i = s_idx[m];
        int c = red0 + kk;
        s.a[kk][m] = (i >= 0 && c < c_red) ? to_f<T>(in[(int64_t)i * c_red + c]) : 0.f;
      }
      load_b_tile<T>(s, wk, red0, c_red, acc0, c_acc, stride_red, stride_acc);
      __syncthreads();
      micro_kernel(s, acc);
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t r = row0 + ty * 4 + i;
    if (r >= n_rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int a = acc0 + tx * 4 + j;
      if (a < c_acc) out[r * c_acc + a] = from_f<T>(acc[i][j]);
    }
  }
}

// ----------------------------------------------------------------------------------------- scatter
template <typename T, typename Map>
__global__ void __launch_bounds__(kConvThreads)
conv_scatter_kernel(const T* __restrict__ in, const T* __restrict__ w, Map map, float* out32, int64_t n_rows,
                    int64_t n_dst, int K, int c_red, int c_acc, int64_t stride_red, int64_t stride_acc) {
  __shared__ Tiles s;
  __shared__ int4 s_coord[BM];
  __shared__ int32_t s_idx[BM];
  const int64_t row0 = (int64_t)blockIdx.x * BM;
  const int acc0 = blockIdx.y * BN;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  map.template prepare<BM>(s_coord, row0, n_rows);
  __syncthreads();
  for (int k = 0; k < K; ++k) {
    int any = 0;
    if (threadIdx.x < BM) {
      int64_t r = row0 + threadIdx.x;
      int32_t i = r < n_rows ? map.get(s_coord, threadIdx.x, r, k) : -1;
      if (i >= n_dst) i = -1;
      s_idx[threadIdx.x] = i;
      any = i >= 0;
    }
    if (!__syncthreads_or(any)) continue;
    float acc[4][4] = {};
    const T* wk = w + (int64_t)k * c_red * c_acc;
    for (int red0 = 0; red0 < c_red; red0 += BK) {
      for (int e = threadIdx.x; e < BM * BK; e += kConvThreads) {
        int m = e / BK, kk = e % BK;
        int64_t r = row0 + m;
        int c = red0 + kk;
        s.a[kk][m] = (r < n_rows && c < c_red) ? to_f<T>(in[r * c_red + c]) : 0.f;
      }
      load_b_tile<T>(s, wk, red0, c_red, acc0, c_acc, stride_red, stride_acc);
      __syncthreads();
      micro_kernel(s, acc);
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int32_t dst = s_idx[ty * 4 + i];
      if (dst < 0) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int a = acc0 + tx * 4 + j;
        if (a < c_acc) atomicAdd(out32 + (int64_t)dst * c_acc + a, acc[i][j]);
      }
    }
    __syncthreads();  // s_idx is rewritten by the next offset
  }
}

// ------------------------------------------------------------------------------------------- wgrad
// grid = (chunks, K, ci_tiles * co_tiles); partial[chunk][k][ci][co] in fp32.
template <typename T, typename Map>
__global__ void __launch_bounds__(kConvThreads)
conv_wgrad_kernel(const T* __restrict__ x, const T* __restrict__ dy, Map map, float* __restrict__ partial,
                  int64_t n_rows, int64_t n_src, int K, int cin, int cout, int64_t rows_per_chunk) {
  __shared__ Tiles s;
  __shared__ int4 s_coord[BK];
  __shared__ int32_t s_idx[BK];
  const int k = blockIdx.y;
  const int co_tiles = (cout + BN - 1) / BN;
  const int ci0 = (blockIdx.z / co_tiles) * BM, co0 = (blockIdx.z % co_tiles) * BN;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int64_t chunk0 = (int64_t)blockIdx.x * rows_per_chunk;
  const int64_t chunk1 = min(chunk0 + rows_per_chunk, n_rows);
  float acc[4][4] = {};
  for (int64_t r0 = chunk0; r0 < chunk1; r0 += BK) {
    map.template prepare<BK>(s_coord, r0, chunk1);
    __syncthreads();
    int any = 0;
    if (threadIdx.x < BK) {
      int64_t r = r0 + threadIdx.x;
      int32_t i = r < chunk1 ? map.get(s_coord, threadIdx.x, r, k) : -1;
      if (i >= n_src) i = -1;
      s_idx[threadIdx.x] = i;
      any = i >= 0;
    }
    if (!__syncthreads_or(any)) continue;
    for (int e = threadIdx.x; e < BK * BM; e += kConvThreads) {
      int kk = e / BM, m = e % BM;
      int32_t i = s_idx[kk];
      int c = ci0 + m;
      s.a[kk][m] = (i >= 0 && c < cin) ? to_f<T>(x[(int64_t)i * cin + c]) : 0.f;
    }
    for (int e = threadIdx.x; e < BK * BN; e += kConvThreads) {
      int kk = e / BN, n = e % BN;
      int c = co0 + n;
      s.b[kk][n] = (s_idx[kk] >= 0 && c < cout) ? to_f<T>(dy[(r0 + kk) * cout + c]) : 0.f;
    }
    __syncthreads();
    micro_kernel(s, acc);
    __syncthreads();
  }
  float* p = partial + ((int64_t)blockIdx.x * K + k) * cin * cout;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int ci = ci0 + ty * 4 + i;
    if (ci >= cin) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int co = co0 + tx * 4 + j;
      if (co < cout) p[(int64_t)ci * cout + co] = acc[i][j];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partial, int chunks, int64_t n, T* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  float sum = 0.f;
  for (int c = 0; c < chunks; ++c) sum += partial[(int64_t)c * n + i];
  out[i] = from_f<T>(sum);
}

template <typename T>
__global__ void __launch_bounds__(256) cast_from_f32_kernel(const float* __restrict__ in, int64_t n, T* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i < n) out[i] = from_f<T>(in[i]);
}

// ------------------------------------------------------------------------------------ host drivers
int wgrad_chunks(int64_t n_out) {
  int64_t c = (n_out + 4095) / 4096;
  if (c < 1) c = 1;
  if (c > 32) c = 32;
  return (int)c;
}

template <typename T, typename Map>
int simt_gather(const T* in, const T* w, const Map& map, T* out, int64_t n_rows, int64_t n_src, int K, int c_red,
                int c_acc, bool w_transposed, cudaStream_t s) {
  if (n_rows == 0) return ST_OK;
  dim3 grid((unsigned)((n_rows + BM - 1) / BM), (unsigned)((c_acc + BN - 1) / BN));
  // forward: B_k = W[k] (c_red=cin rows, c_acc=cout cols).  dgrad: B_k = W[k]^T, W[k] is (c_acc, c_red).
  int64_t sr = w_transposed ? 1 : c_acc, sa = w_transposed ? c_red : 1;
  { conv_gather_kernel<T, Map><<<grid, kConvThreads, 0, s>>>(in, w, map, out, n_rows, n_src, K, c_red, c_acc, sr, sa); note_launches(1); }
  return check_launch("conv_gather_kernel");
}

template <typename T, typename Map>
int simt_scatter(const T* in, const T* w, const Map& map, T* out, float* out32, int64_t n_rows, int64_t n_dst, int K,
                 int c_red, int c_acc, cudaStream_t s) {
  int64_t n = n_dst * c_acc;
  if (n == 0) return ST_OK;
  cudaMemsetAsync(out32, 0, n * sizeof(float), s);
  if (n_rows > 0) {
    dim3 grid((unsigned)((n_rows + BM - 1) / BM), (unsigned)((c_acc + BN - 1) / BN));
    { conv_scatter_kernel<T, Map><<<grid, kConvThreads, 0, s>>>(in, w, map, out32, n_rows, n_dst, K, c_red, c_acc, 1,
                                                              c_red); note_launches(1); }
  }
  if (reinterpret_cast<void*>(out) != reinterpret_cast<void*>(out32))
    { cast_from_f32_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out32, n, out); note_launches(1); }
  return check_launch("conv_scatter_kernel");
}

template <typename T, typename Map>
int simt_wgrad(const T* x, const T* dy, const Map& map, T* dw, float* partial, int64_t n_rows, int64_t n_src, int K,
               int cin, int cout, cudaStream_t s) {
  int64_t n = (int64_t)K * cin * cout;
  if (n == 0) return ST_OK;
  if (n_rows == 0) {
    cudaMemsetAsync(dw, 0, n * sizeof(T), s);
    return check_launch("wgrad(empty)");
  }
  int chunks = wgrad_chunks(n_rows);
  int64_t rows_per_chunk = (n_rows + chunks - 1) / chunks;
  rows_per_chunk = (rows_per_chunk + BK - 1) / BK * BK;
  dim3 grid((unsigned)chunks, (unsigned)K, (unsigned)(((cin + BM - 1) / BM) * ((cout + BN - 1) / BN)));
  { conv_wgrad_kernel<T, Map><<<grid, kConvThreads, 0, s>>>(x, dy, map, partial, n_rows, n_src, K, cin, cout,
                                                          rows_per_chunk); note_launches(1); }
  { reduce_partials_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(partial, chunks, n, dw); note_launches(1); }
  return check_launch("conv_wgrad_kernel");
}

// out[i] = sum over chunks of partial[chunk][i], cast to the feature dtype (fixed summation order).
int reduce_partials(int dtype, const float* partial, int chunks, int64_t n, void* out, cudaStream_t s) {
  if (n <= 0) return ST_OK;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == ST_F32) {
    reduce_partials_kernel<float><<<grid, 256, 0, s>>>(partial, chunks, n, static_cast<float*>(out));
  } else if (dtype == ST_F16) {
    reduce_partials_kernel<__half><<<grid, 256, 0, s>>>(partial, chunks, n, static_cast<__half*>(out));
  } else {
    reduce_partials_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(partial, chunks, n, static_cast<__nv_bfloat16*>(out));
  }
  note_launches(1);
  return check_launch("reduce_partials");
}

#define ST_INSTANTIATE(T, MAP)                                                                                     \
  template int simt_gather<T, MAP>(const T*, const T*, const MAP&, T*, int64_t, int64_t, int, int, int, bool,     \
                                   cudaStream_t);                                                                  \
  template int simt_scatter<T, MAP>(const T*, const T*, const MAP&, T*, float*, int64_t, int64_t, int, int, int,  \
                                    cudaStream_t);                                                                 \
  template int simt_wgrad<T, MAP>(const T*, const T*, const MAP&, T*, float*, int64_t, int64_t, int, int, int,    \
                                  cudaStream_t);

ST_INSTANTIATE(float, StoredMap)
ST_INSTANTIATE(__half, StoredMap)
ST_INSTANTIATE(__nv_bfloat16, StoredMap)
ST_INSTANTIATE(float, HashFlyMap<int16_t>)
ST_INSTANTIATE(__half, HashFlyMap<int16_t>)
ST_INSTANTIATE(__nv_bfloat16, HashFlyMap<int16_t>)
ST_INSTANTIATE(float, HashFlyMap<int32_t>)
ST_INSTANTIATE(__half, HashFlyMap<int32_t>)
ST_INSTANTIATE(__nv_bfloat16, HashFlyMap<int32_t>)

}  // namespace st
