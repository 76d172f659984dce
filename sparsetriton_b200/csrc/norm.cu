// Per-sample batch normalisation of sparse features, with the ReLU that follows it folded in.
//
// Reference: nn/functional/norm.py:20-112 (statistics per (batch index, channel) over the rows of that
// sample, biased variance, eps inside the square root) and the ReLU module applied to its output.
// The layer is pure streaming work over an (N, C) matrix, so it is written as four passes that each
// read the features once:
//   forward   sums (twice: mean, then centred second moment) -> normalise + scale + shift (+ ReLU)
//   backward  the two per-(sample, channel) sums of the gradient -> dX
// instead of the dozen elementwise launches and one-hot matrix products an op-by-op formulation
// costs.  Per-(sample, channel) sums are reduced per thread over a strip of rows and then added with
// one fp32 atomic per strip, sample and channel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace st {

namespace {

constexpr int kBnThreads = 256;
constexpr int kBnRowsPerBlock = 512;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Thread layout of the two reduction kernels: the block's threads form (row lanes) x (channel lanes);
// a thread walks its channel down a strip of rows and flushes its two sums whenever the sample
// changes (rows of a sample are contiguous in every tensor the convolutions produce, so normally
// once or twice per strip).
struct Lanes {
  int c_lanes, r_lanes;
};
__host__ __device__ inline Lanes lanes_for(int C) {
  int c = 1;
  while (c * 2 <= C && c * 2 <= kBnThreads) c *= 2;
  return Lanes{c, kBnThreads / c};
}

// Sample of row r, or -1 (and ST_DEV_BAD_INDEX in *status) when the stored index is not in [0, B): such a
// row takes part in no sum and its output is zero, so a bad index never reaches the (B, C) arrays.
__device__ __forceinline__ int sample_of(const int32_t* __restrict__ batch, int64_t r, int B, int32_t* status) {
  const int b = batch ? __ldg(batch + r) : 0;
  if ((unsigned)b < (unsigned)B) return b;
  if (status) atomicOr(status, ST_DEV_BAD_INDEX);
  return -1;
}

// The shift of sample b taken from the data: the value of the sample's first row (0 when there is none).  Sums
// of (x - shift) and (x - shift)^2 around a value of the distribution keep the one-pass variance accurate.
template <typename T>
__device__ __forceinline__ float shift_from_row(const T* __restrict__ x, const int32_t* __restrict__ first_row, int b, int C,
                                                int c) {
  if (!first_row) return 0.f;
  const int32_t r = __ldg(first_row + b);
  return r >= 0 ? to_f(x[(int64_t)r * C + c]) : 0.f;
}

// sums[(b*C + c)*2 + 0] += sum (x - shift),  [.. + 1] += sum (x - shift)^2      shift (B, C) or null
template <typename T>
__global__ void __launch_bounds__(kBnThreads) bn_sums_kernel(const T* __restrict__ x, const int32_t* __restrict__ batch,
                                                            int64_t n, int C, int B, const float* __restrict__ shift,
                                                            const int32_t* __restrict__ first_row,
                                                            float* __restrict__ sums, int32_t* status) {
  const Lanes L = lanes_for(C);
  const int cl = threadIdx.x % L.c_lanes, rl = threadIdx.x / L.c_lanes;
  const int64_t row0 = (int64_t)blockIdx.x * kBnRowsPerBlock;
  const int64_t row_end = min(n, row0 + kBnRowsPerBlock);
  for (int c = cl; c < C; c += L.c_lanes) {
    float s0 = 0.f, s1 = 0.f, sh = 0.f;
    int cur = -1;
    for (int64_t r = row0 + rl; r < row_end; r += L.r_lanes) {
      const int b = sample_of(batch, r, B, status);
      if (b != cur) {
        if (cur >= 0) {
          atomicAdd(sums + ((int64_t)cur * C + c) * 2, s0);
          atomicAdd(sums + ((int64_t)cur * C + c) * 2 + 1, s1);
        }
        cur = b;
        s0 = s1 = 0.f;
        if (b >= 0) sh = shift ? __ldg(shift + (int64_t)b * C + c) : shift_from_row(x, first_row, b, C, c);
      }
      if (b < 0) continue;
      const float v = to_f(x[r * C + c]) - sh;
      s0 += v;
      s1 += v * v;
    }
    if (cur >= 0) {
      atomicAdd(sums + ((int64_t)cur * C + c) * 2, s0);
      atomicAdd(sums + ((int64_t)cur * C + c) * 2 + 1, s1);
    }
  }
}

// y = relu?((x - mean) * rstd * w + bias)
template <typename T>
__global__ void __launch_bounds__(kBnThreads) bn_apply_kernel(const T* __restrict__ x, const int32_t* __restrict__ batch,
                                                             int64_t n, int C, int B, const float* __restrict__ mean,
                                                             const float* __restrict__ rstd, const float* __restrict__ w,
                                                             const float* __restrict__ bias, int relu, T* __restrict__ y,
                                                             int32_t* status) {
  const int64_t total = n * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / C;
    const int c = (int)(i - r * C);
    const int b = sample_of(batch, r, B, status);
    if (b < 0) {
      y[i] = from_f<T>(0.f);
      continue;
    }
    const int64_t s = (int64_t)b * C + c;
    float v = (to_f(x[i]) - __ldg(mean + s)) * __ldg(rstd + s);
    if (w) v *= __ldg(w + c);
    if (bias) v += __ldg(bias + c);
    if (relu) v = fmaxf(v, 0.f);
    y[i] = from_f<T>(v);
  }
}

// dz = dy * [z > 0 if relu];  sums[..0] += sum dz,  sums[..1] += sum dz * xhat
template <typename T>
__global__ void __launch_bounds__(kBnThreads)
    bn_bwd_sums_kernel(const T* __restrict__ x, const T* __restrict__ dy, const int32_t* __restrict__ batch, int64_t n, int C,
                       int B, const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ w,
                       const float* __restrict__ bias, int relu, float* __restrict__ sums, int32_t* status) {
  const Lanes L = lanes_for(C);
  const int cl = threadIdx.x % L.c_lanes, rl = threadIdx.x / L.c_lanes;
  const int64_t row0 = (int64_t)blockIdx.x * kBnRowsPerBlock;
  const int64_t row_end = min(n, row0 + kBnRowsPerBlock);
  for (int c = cl; c < C; c += L.c_lanes) {
    const float wc = w ? __ldg(w + c) : 1.f, bc = bias ? __ldg(bias + c) : 0.f;
    float s0 = 0.f, s1 = 0.f, m = 0.f, rs = 0.f;
    int cur = -1;
    for (int64_t r = row0 + rl; r < row_end; r += L.r_lanes) {
      const int b = sample_of(batch, r, B, status);
      if (b != cur) {
        if (cur >= 0) {
          atomicAdd(sums + ((int64_t)cur * C + c) * 2, s0);
          atomicAdd(sums + ((int64_t)cur * C + c) * 2 + 1, s1);
        }
        cur = b;
        s0 = s1 = 0.f;
        if (b >= 0) {
          m = __ldg(mean + (int64_t)b * C + c);
          rs = __ldg(rstd + (int64_t)b * C + c);
        }
      }
      if (b < 0) continue;
      const float xhat = (to_f(x[r * C + c]) - m) * rs;
      float dz = to_f(dy[r * C + c]);
      if (relu && !(xhat * wc + bc > 0.f)) dz = 0.f;
      s0 += dz;
      s1 += dz * xhat;
    }
    if (cur >= 0) {
      atomicAdd(sums + ((int64_t)cur * C + c) * 2, s0);
      atomicAdd(sums + ((int64_t)cur * C + c) * 2 + 1, s1);
    }
  }
}

// dx = rstd * w / n_b * (n_b * dz - sum dz - xhat * sum dz*xhat)
template <typename T>
__global__ void __launch_bounds__(kBnThreads)
    bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, const int32_t* __restrict__ batch, int64_t n, int C,
                        int B, const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ w,
                        const float* __restrict__ bias, int relu, const float* __restrict__ sums,
                        const float* __restrict__ inv_count, T* __restrict__ dx, int32_t* status) {
  const int64_t total = n * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / C;
    const int c = (int)(i - r * C);
    const int b = sample_of(batch, r, B, status);
    if (b < 0) {
      dx[i] = from_f<T>(0.f);
      continue;
    }
    const int64_t s = (int64_t)b * C + c;
    const float wc = w ? __ldg(w + c) : 1.f, bc = bias ? __ldg(bias + c) : 0.f;
    const float rs = __ldg(rstd + s);
    const float xhat = (to_f(x[i]) - __ldg(mean + s)) * rs;
    float dz = to_f(dy[i]);
    if (relu && !(xhat * wc + bc > 0.f)) dz = 0.f;
    const float ic = __ldg(inv_count + b);
    const float v = rs * wc * (dz - ic * (__ldg(sums + s * 2) + xhat * __ldg(sums + s * 2 + 1)));
    dx[i] = from_f<T>(v);
  }
}

// ---- 16-byte vector forms (C a multiple of 16 / sizeof(T)): a thread owns V consecutive channels, a
// warp reads whole 128-byte lines.
template <typename T> struct Vec { static constexpr int V = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ uint4 load_raw(const T* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4& raw, float (&out)[Vec<T>::V]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::V; ++i) out[i] = to_f(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&in)[Vec<T>::V]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec<T>::V; ++i) e[i] = from_f<T>(in[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Both vector kernels give a block a strip of rows and lay its threads out as (row lanes) x (C / V
// channel lanes), so a thread keeps its V channels for the whole strip and holds the per-(sample,
// channel) coefficients in registers, reloading them only when the sample changes (rows of a sample
// are contiguous in every tensor the convolutions produce).  Each pass of the row loop issues the loads
// of kBnUnroll rows before it uses any of them, which is what keeps enough bytes in flight per SM.
constexpr int kBnUnroll = 4;

// Reduction kernels.  MODE 0: sums of (x - shift) and its square; MODE 1: sums of dz and dz * xhat.
template <typename T, int MODE>
__global__ void __launch_bounds__(kBnThreads)
    bn_sums_vec_kernel(const T* __restrict__ x, const T* __restrict__ dy, const int32_t* __restrict__ batch, int64_t n, int C,
                       int B, const float* __restrict__ p0 /* shift | mean */, const float* __restrict__ rstd,
                       const float* __restrict__ w, const float* __restrict__ bias, int relu, float* __restrict__ sums,
                       int rows_per_block, int32_t* status, const int32_t* __restrict__ first_row /* MODE 0: shift rows */) {
  constexpr int V = Vec<T>::V;
  constexpr int U = kBnUnroll;
  const int c_lanes = C / V;                      // <= kBnThreads is checked by the caller
  const int r_lanes = kBnThreads / c_lanes;
  const int cl = threadIdx.x % c_lanes, rl = threadIdx.x / c_lanes;
  const int c0 = cl * V;
  const int64_t row0 = (int64_t)blockIdx.x * rows_per_block;
  const int64_t row_end = min(n, row0 + rows_per_block);
  float s0[V], s1[V], a[V], b[V], wc[V], bc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    s0[i] = s1[i] = a[i] = 0.f;
    b[i] = 1.f;
    wc[i] = (MODE == 1 && w) ? __ldg(w + c0 + i) : 1.f;
    bc[i] = (MODE == 1 && bias) ? __ldg(bias + c0 + i) : 0.f;
  }
  int cur = -1;
  auto flush = [&]() {
    if (cur < 0) return;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      atomicAdd(sums + ((int64_t)cur * C + c0 + i) * 2, s0[i]);
      atomicAdd(sums + ((int64_t)cur * C + c0 + i) * 2 + 1, s1[i]);
      s0[i] = s1[i] = 0.f;
    }
  };
  // Sums that belong to the sample of the block's first row (normally all of them) are added up across
  // the row lanes in shared memory first, so that the block issues one atomic per channel and component
  // instead of one per thread.
  __shared__ float red[kBnThreads * 2 * V];
  const int b_common = row0 < n ? sample_of(batch, row0, B, nullptr) : 0;
  for (int64_t r = row0 + rl; r < row_end; r += (int64_t)U * r_lanes) {
    uint4 xr[U], dr[U];
    int bt[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int64_t rr = r + (int64_t)j * r_lanes;
      bt[j] = -1;
      if (rr < row_end) {
        bt[j] = sample_of(batch, rr, B, status);
        xr[j] = load_raw(x + rr * C + c0);
        if (MODE == 1) dr[j] = load_raw(dy + rr * C + c0);
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      if (r + (int64_t)j * r_lanes >= row_end) break;
      if (bt[j] < 0) {                             // index outside [0, B): the row joins no sum
        flush();
        cur = -1;
        continue;
      }
      if (bt[j] != cur) {
        flush();
        cur = bt[j];
#pragma unroll
        for (int i = 0; i < V; ++i) {
          a[i] = p0 ? __ldg(p0 + (int64_t)cur * C + c0 + i) : (MODE == 0 ? shift_from_row(x, first_row, cur, C, c0 + i) : 0.f);
          if (MODE == 1) b[i] = __ldg(rstd + (int64_t)cur * C + c0 + i);
        }
      }
      float xv[V];
      unpack_vec<T>(xr[j], xv);
      if (MODE == 0) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float v = xv[i] - a[i];
          s0[i] += v;
          s1[i] += v * v;
        }
      } else {
        float dv[V];
        unpack_vec<T>(dr[j], dv);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float xhat = (xv[i] - a[i]) * b[i];
          float dz = dv[i];
          if (relu && !(xhat * wc[i] + bc[i] > 0.f)) dz = 0.f;
          s0[i] += dz;
          s1[i] += dz * xhat;
        }
      }
    }
  }
  if (cur != b_common) flush();              // leftovers of another sample: added directly (flush zeroes the sums)
  // Row lanes that share a warp (fewer than 32 channel lanes) are added up by shuffles; what is left
  // is one partial per warp, or per row lane when a warp spans a single row.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int d = c_lanes; d < 32; d <<= 1) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      s0[i] += __shfl_xor_sync(0xFFFFFFFFu, s0[i], d);
      s1[i] += __shfl_xor_sync(0xFFFFFFFFu, s1[i], d);
    }
  }
  const bool warp_shared = c_lanes < 32;
  const int groups = warp_shared ? kBnThreads / 32 : r_lanes;
  if (!warp_shared || lane < c_lanes) {
    float* mine = red + ((size_t)(warp_shared ? warp : rl) * c_lanes + cl) * 2 * V;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      mine[2 * i] = s0[i];
      mine[2 * i + 1] = s1[i];
    }
  }
  __syncthreads();
  if (b_common < 0) return;                      // everything was added directly (the partials are zero)
  // thread t < 2*C adds up entry e = t of every group:  red[(g * c_lanes + cl) * 2V + j],  e = cl * 2V + j
  for (int e = threadIdx.x; e < 2 * C; e += kBnThreads) {
    float acc = 0.f;
    for (int q = 0; q < groups; ++q) acc += red[(size_t)q * c_lanes * 2 * V + e];
    const int c = (e / (2 * V)) * V + (e % (2 * V)) / 2;
    atomicAdd(sums + ((int64_t)b_common * C + c) * 2 + (e & 1), acc);
  }
}

// Elementwise kernels: MODE 0 forward, MODE 1 backward.  A block covers rows_per_block rows.
template <typename T, int MODE>
__global__ void __launch_bounds__(kBnThreads)
    bn_apply_vec_kernel(const T* __restrict__ x, const T* __restrict__ dy, const int32_t* __restrict__ batch, int64_t n, int C,
                        int B, const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ w,
                        const float* __restrict__ bias, int relu, const float* __restrict__ sums,
                        const float* __restrict__ inv_count, T* __restrict__ out, int rows_per_block, int32_t* status) {
  constexpr int V = Vec<T>::V;
  constexpr int U = kBnUnroll;
  const int c_lanes = C / V;
  const int r_lanes = kBnThreads / c_lanes;
  const int cl = threadIdx.x % c_lanes, rl = threadIdx.x / c_lanes;
  const int c0 = cl * V;
  const int64_t row0 = (int64_t)blockIdx.x * rows_per_block;
  const int64_t row_end = min(n, row0 + rows_per_block);
  float m[V], rs[V], wc[V], bc[V], q0[V], q1[V];
  float ic = 0.f;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    m[i] = q0[i] = q1[i] = 0.f;
    rs[i] = 1.f;
    wc[i] = w ? __ldg(w + c0 + i) : 1.f;
    bc[i] = bias ? __ldg(bias + c0 + i) : 0.f;
  }
  int cur = -1;
  for (int64_t r = row0 + rl; r < row_end; r += (int64_t)U * r_lanes) {
    uint4 xr[U], dr[U];
    int bt[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int64_t rr = r + (int64_t)j * r_lanes;
      bt[j] = -1;
      if (rr < row_end) {
        bt[j] = sample_of(batch, rr, B, status);
        xr[j] = load_raw(x + rr * C + c0);
        if (MODE == 1) dr[j] = load_raw(dy + rr * C + c0);
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int64_t rr = r + (int64_t)j * r_lanes;
      if (rr >= row_end) break;
      if (bt[j] < 0) {                             // index outside [0, B): the row's output is zero
        float zero[V];
#pragma unroll
        for (int i = 0; i < V; ++i) zero[i] = 0.f;
        store_vec(out + rr * C + c0, zero);
        continue;
      }
      if (bt[j] != cur) {
        cur = bt[j];
        const int64_t s = (int64_t)cur * C + c0;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          m[i] = __ldg(mean + s + i);
          rs[i] = __ldg(rstd + s + i);
          if (MODE == 1) {
            q0[i] = __ldg(sums + (s + i) * 2);
            q1[i] = __ldg(sums + (s + i) * 2 + 1);
          }
        }
        if (MODE == 1) ic = __ldg(inv_count + cur);
      }
      float xv[V], res[V];
      unpack_vec<T>(xr[j], xv);
      if (MODE == 0) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float v = (xv[i] - m[i]) * rs[i];
          if (w) v *= wc[i];
          if (bias) v += bc[i];
          if (relu) v = fmaxf(v, 0.f);
          res[i] = v;
        }
      } else {
        float dv[V];
        unpack_vec<T>(dr[j], dv);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float xhat = (xv[i] - m[i]) * rs[i];
          float dz = dv[i];
          if (relu && !(xhat * wc[i] + bc[i] > 0.f)) dz = 0.f;
          res[i] = rs[i] * wc[i] * (dz - ic * (q0[i] + xhat * q1[i]));
        }
      }
      store_vec(out + rr * C + c0, res);
    }
  }
}

// One thread per channel: mean / rstd of every sample from the shifted one-pass sums, and the running buffers
// (averages of the per-sample statistics over all B samples, empty ones counting as zero).
template <typename T>
__global__ void __launch_bounds__(128)
bn_finalize_kernel(const float* __restrict__ sums, const T* __restrict__ x, const int32_t* __restrict__ first_row,
                   const float* __restrict__ inv_count, int B, int C, float eps, float momentum, float* __restrict__ mean,
                   float* __restrict__ rstd, float* running_mean, float* running_var) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= C) return;
  float mean_sum = 0.f, var_sum = 0.f;
  for (int b = 0; b < B; ++b) {
    const float ic = __ldg(inv_count + b);
    const float shift = shift_from_row(x, first_row, b, C, c);
    const float m1 = sums[((int64_t)b * C + c) * 2] * ic;
    const float var = fmaxf(sums[((int64_t)b * C + c) * 2 + 1] * ic - m1 * m1, 0.f);
    const float m = shift + m1;
    mean[(int64_t)b * C + c] = m;
    rstd[(int64_t)b * C + c] = rsqrtf(var + eps);
    mean_sum += m;
    var_sum += var;
  }
  if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean_sum / (float)B;
  if (running_var) running_var[c] = (1.f - momentum) * running_var[c] + momentum * var_sum / (float)B;
}

// first[b] = smallest row whose batch index is b, as an unsigned minimum over the rows that open a run of equal
// indices (first holds 0xFFFFFFFF = -1 "no row" on entry)
__global__ void __launch_bounds__(256)
bn_first_rows_kernel(const int32_t* __restrict__ batch, int64_t n, int B, uint32_t* first) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const int b = __ldg(batch + i);
  if ((unsigned)b >= (unsigned)B) return;
  if (i == 0 || __ldg(batch + i - 1) != b) atomicMin(first + b, (uint32_t)i);
}

// dW[c] = sum_b sums[b,c,1], dB[c] = sum_b sums[b,c,0]
__global__ void __launch_bounds__(128)
bn_param_grads_kernel(const float* __restrict__ sums, int B, int C, float* dW, float* dB) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= C) return;
  float w = 0.f, b0 = 0.f;
  for (int b = 0; b < B; ++b) {
    b0 += sums[((int64_t)b * C + c) * 2];
    w += sums[((int64_t)b * C + c) * 2 + 1];
  }
  if (dW) dW[c] = w;
  if (dB) dB[c] = b0;
}

// The vector forms need whole 16-byte vectors per row, aligned rows, and at most kBnThreads channel lanes.
template <typename T>
bool vec_ok(int C, const void* a, const void* b, const void* c) {
  constexpr int V = Vec<T>::V;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return C % V == 0 && C / V <= kBnThreads && kBnThreads % (C / V) == 0 && al(a) && al(b) && al(c);
}

int check_bn(const char* who, int dtype, int64_t n, int C, int B) {
  if (dtype != ST_F32 && dtype != ST_F16 && dtype != ST_BF16) {
    set_error("%s: unsupported feature dtype %d", who, dtype);
    return ST_ERR_DTYPE;
  }
  if (n < 0 || C < 1 || B < 1) {
    set_error("%s: bad sizes (n=%lld, C=%d, B=%d)", who, (long long)n, C, B);
    return ST_ERR_ARG;
  }
  return ST_OK;
}

unsigned strip_blocks(int64_t n) { return (unsigned)((n + kBnRowsPerBlock - 1) / kBnRowsPerBlock); }
// Rows per block of the vector kernels: four passes of the unrolled row loop per thread.
int apply_rows(int C, int V) { return 4 * kBnUnroll * (kBnThreads / (C / V)); }
unsigned apply_blocks(int64_t n, int rows) { return (unsigned)((n + rows - 1) / rows); }
unsigned flat_blocks(int64_t total) {
  int64_t b = (total + kBnThreads * 4 - 1) / (kBnThreads * 4);
  return (unsigned)(b < 1 ? 1 : (b > 148 * 32 ? 148 * 32 : b));
}

}  // namespace

}  // namespace st

using namespace st;

#define ST_BN_DISPATCH(dtype, ...)                                   \
  do {                                                               \
    if ((dtype) == ST_F32) { using T = float; __VA_ARGS__; }         \
    else if ((dtype) == ST_F16) { using T = __half; __VA_ARGS__; }   \
    else { using T = __nv_bfloat16; __VA_ARGS__; }                   \
  } while (0)

extern "C" {

int st_bn_sums(int dtype, const void* X, const int32_t* batch, int64_t n, int C, int B, const float* shift, float* sums,
               int32_t* status, void* stream) {
  int rc = check_bn("st_bn_sums", dtype, n, C, B);
  if (rc != ST_OK) return rc;
  if (!sums || (n > 0 && !X)) {
    set_error("st_bn_sums: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)B * C, s) != cudaSuccess) return check_launch("st_bn_sums");
  if (n > 0) {
    ST_BN_DISPATCH(dtype, {
      if (vec_ok<T>(C, X, nullptr, nullptr))
      {
        const int rows = apply_rows(C, Vec<T>::V);
        bn_sums_vec_kernel<T, 0><<<apply_blocks(n, rows), kBnThreads, 0, s>>>(static_cast<const T*>(X), nullptr, batch, n, C, B,
                                                                              shift, nullptr, nullptr, nullptr, 0, sums, rows,
                                                                              status, nullptr);
      }
      else
        bn_sums_kernel<T><<<strip_blocks(n), kBnThreads, 0, s>>>(static_cast<const T*>(X), batch, n, C, B, shift, nullptr, sums,
                                                                status);
    });
    note_launches(1);
  }
  return check_launch("st_bn_sums");
}

int st_bn_apply(int dtype, const void* X, const int32_t* batch, int64_t n, int C, int B, const float* mean,
                const float* rstd, const float* weight, const float* bias, int relu, void* Y, int32_t* status, void* stream) {
  int rc = check_bn("st_bn_apply", dtype, n, C, B);
  if (rc != ST_OK) return rc;
  if (n == 0) return ST_OK;
  if (!X || !Y || !mean || !rstd) {
    set_error("st_bn_apply: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  ST_BN_DISPATCH(dtype, {
    if (vec_ok<T>(C, X, Y, nullptr))
    {
      const int rows = apply_rows(C, Vec<T>::V);
      bn_apply_vec_kernel<T, 0><<<apply_blocks(n, rows), kBnThreads, 0, s>>>(static_cast<const T*>(X), nullptr, batch, n, C, B,
                                                                             mean, rstd, weight, bias, relu, nullptr,
                                                                             nullptr, static_cast<T*>(Y), rows, status);
    }
    else
      bn_apply_kernel<T><<<flat_blocks(n * C), kBnThreads, 0, s>>>(static_cast<const T*>(X), batch, n, C, B, mean, rstd, weight,
                                                                   bias, relu, static_cast<T*>(Y), status);
  });
  note_launches(1);
  return check_launch("st_bn_apply");
}

int st_bn_backward_sums(int dtype, const void* X, const void* dY, const int32_t* batch, int64_t n, int C, int B,
                        const float* mean, const float* rstd, const float* weight, const float* bias, int relu,
                        float* sums, int32_t* status, void* stream) {
  int rc = check_bn("st_bn_backward_sums", dtype, n, C, B);
  if (rc != ST_OK) return rc;
  if (!sums || !mean || !rstd || (n > 0 && (!X || !dY))) {
    set_error("st_bn_backward_sums: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)B * C, s) != cudaSuccess)
    return check_launch("st_bn_backward_sums");
  if (n > 0) {
    ST_BN_DISPATCH(dtype, {
      if (vec_ok<T>(C, X, dY, nullptr))
      {
        const int rows = apply_rows(C, Vec<T>::V);
        bn_sums_vec_kernel<T, 1><<<apply_blocks(n, rows), kBnThreads, 0, s>>>(static_cast<const T*>(X),
                                                                              static_cast<const T*>(dY), batch, n, C, B, mean, rstd,
                                                                              weight, bias, relu, sums, rows, status, nullptr);
      }
      else
        bn_bwd_sums_kernel<T><<<strip_blocks(n), kBnThreads, 0, s>>>(static_cast<const T*>(X), static_cast<const T*>(dY), batch,
                                                                     n, C, B, mean, rstd, weight, bias, relu, sums, status);
    });
    note_launches(1);
  }
  return check_launch("st_bn_backward_sums");
}

int st_bn_backward_apply(int dtype, const void* X, const void* dY, const int32_t* batch, int64_t n, int C, int B,
                         const float* mean, const float* rstd, const float* weight, const float* bias, int relu,
                         const float* sums, const float* inv_count, void* dX, int32_t* status, void* stream) {
  int rc = check_bn("st_bn_backward_apply", dtype, n, C, B);
  if (rc != ST_OK) return rc;
  if (n == 0) return ST_OK;
  if (!X || !dY || !dX || !mean || !rstd || !sums || !inv_count) {
    set_error("st_bn_backward_apply: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  ST_BN_DISPATCH(dtype, {
    if (vec_ok<T>(C, X, dY, dX))
    {
      const int rows = apply_rows(C, Vec<T>::V);
      bn_apply_vec_kernel<T, 1><<<apply_blocks(n, rows), kBnThreads, 0, s>>>(
          static_cast<const T*>(X), static_cast<const T*>(dY), batch, n, C, B, mean, rstd, weight, bias, relu, sums, inv_count,
          static_cast<T*>(dX), rows, status);
    }
    else
      bn_bwd_apply_kernel<T><<<flat_blocks(n * C), kBnThreads, 0, s>>>(static_cast<const T*>(X), static_cast<const T*>(dY), batch,
                                                                       n, C, B, mean, rstd, weight, bias, relu, sums, inv_count,
                                                                       static_cast<T*>(dX), status);
  });
  note_launches(1);
  return check_launch("st_bn_backward_apply");
}

int st_bn_first_rows(const int32_t* batch, int64_t n, int B, int32_t* first_row, void* stream) {
  if (n < 0 || B < 1 || !first_row || (n > 0 && !batch) || n > 0x7FFFFFFFll) {
    set_error("st_bn_first_rows: bad arguments");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(first_row, 0xFF, sizeof(int32_t) * (size_t)B, s) != cudaSuccess) return check_launch("st_bn_first_rows");
  if (n > 0) {
    bn_first_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(batch, n, B, reinterpret_cast<uint32_t*>(first_row));
    note_launches(1);
  }
  return check_launch("st_bn_first_rows");
}

int st_bn_forward_stats(int dtype, const void* X, const int32_t* batch, const int32_t* first_row, int64_t n, int C, int B,
                        const float* inv_count, float eps, float momentum, float* sums, float* mean, float* rstd,
                        float* running_mean, float* running_var, int32_t* status, void* stream) {
  int rc = check_bn("st_bn_forward_stats", dtype, n, C, B);
  if (rc != ST_OK) return rc;
  if (!sums || !mean || !rstd || !inv_count || (n > 0 && !X)) {
    set_error("st_bn_forward_stats: null pointer");
    return ST_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)B * C, s) != cudaSuccess) return check_launch("st_bn_forward_stats");
  ST_BN_DISPATCH(dtype, {
    if (n > 0) {
      if (vec_ok<T>(C, X, nullptr, nullptr)) {
        const int rows = apply_rows(C, Vec<T>::V);
        bn_sums_vec_kernel<T, 0><<<apply_blocks(n, rows), kBnThreads, 0, s>>>(static_cast<const T*>(X), nullptr, batch, n, C, B,
                                                                              nullptr, nullptr, nullptr, nullptr, 0, sums, rows,
                                                                              status, first_row);
      } else {
        bn_sums_kernel<T><<<strip_blocks(n), kBnThreads, 0, s>>>(static_cast<const T*>(X), batch, n, C, B, nullptr, first_row,
                                                                  sums, status);
      }
      note_launches(1);
    }
    bn_finalize_kernel<T><<<(unsigned)((C + 127) / 128), 128, 0, s>>>(sums, static_cast<const T*>(X), n > 0 ? first_row : nullptr,
                                                                      inv_count, B, C, eps, momentum, mean, rstd, running_mean,
                                                                      running_var);
    note_launches(1);
  });
  return check_launch("st_bn_forward_stats");
}

int st_bn_backward(int dtype, const void* X, const void* dY, const int32_t* batch, int64_t n, int C, int B, const float* mean,
                   const float* rstd, const float* weight, const float* bias, int relu, int batch_stats,
                   const float* inv_count, float* sums, void* dX, float* dW, float* dB, int32_t* status, void* stream) {
  int rc = st_bn_backward_sums(dtype, X, dY, batch, n, C, B, mean, rstd, weight, bias, relu, sums, status, stream);
  if (rc != ST_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (dW || dB) {
    bn_param_grads_kernel<<<(unsigned)((C + 127) / 128), 128, 0, s>>>(sums, B, C, dW, dB);
    note_launches(1);
  }
  if (!dX) return check_launch("st_bn_backward");
  if (!batch_stats) {
    // fixed (running) statistics: the two correction terms vanish
    if (cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)B * C, s) != cudaSuccess) return check_launch("st_bn_backward");
  }
  return st_bn_backward_apply(dtype, X, dY, batch, n, C, B, mean, rstd, weight, bias, relu, sums, inv_count, dX, status, stream);
}

}  // extern "C"
