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

// ---- Streaming forms: rows whose 16-byte vectors number a power of two (every width the networks use).
// A block owns a contiguous range of rows, which is one contiguous range of bytes of every (N, C) operand, and
// walks it in chunks of 16 KB.  A producer warp brings the chunks into a ring of shared-memory stages with bulk
// asynchronous copies (one instruction per chunk and operand, completion counted in bytes on the stage's
// mbarrier), so the bytes in flight per SM are set by the ring (128-192 KB with two blocks per SM) and cost
// no registers; the 256 consumer threads read their vectors from shared memory, keep the coefficients of their
// V channels in registers and, in the elementwise modes, store the result straight to global memory.
// MODE 0: sums of (x - shift), (x - shift)^2   1: sums of dz, dz * xhat   2: forward output   3: dX.
namespace stream {

constexpr int kChunkBytes = 16384;
constexpr int kConsumers = kBnThreads;                  // 8 warps
constexpr int kThreads = kConsumers + 32;               // + the producer warp
constexpr long long kWaitCycles = 4000000000ll;          // ~2 s: a wait that long means a copy never arrived

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.shared::cta.b64 t, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out or another warp of the block has given up already.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      if (status) atomicOr(status, ST_DEV_TIMEOUT);
      return false;
    }
  }
}
// `bytes` (a multiple of 16) from global `src` (16-byte aligned) to shared `dst` (16-byte aligned).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <int MODE> struct Ring {
  static constexpr int kOperands = (MODE == 1 || MODE == 3) ? 2 : 1;
  static constexpr int kStages = kOperands == 2 ? 3 : 4;
  static constexpr int kIdBytes = 4096;                   // batch indices of a chunk's rows (at most 1024 rows)
  static constexpr int kStageBytes = kOperands * kChunkBytes + kIdBytes;
  static constexpr int kBytes = kStages * kStageBytes + 128;
};

}  // namespace stream

template <typename T, int MODE>
__global__ void __launch_bounds__(stream::kThreads, 2)
    bn_stream_kernel(const T* __restrict__ x, const T* __restrict__ dy, const int32_t* __restrict__ batch, int64_t n, int C,
                     int B, const float* __restrict__ p0 /* MODE 0: unused, else mean */, const float* __restrict__ rstd,
                     const float* __restrict__ w, const float* __restrict__ bias, int relu,
                     const float* __restrict__ sums_in, const float* __restrict__ inv_count, float* __restrict__ sums_out,
                     T* __restrict__ out, const int32_t* __restrict__ first_row, int64_t chunks_per_block, int32_t* status) {
  using namespace stream;
  constexpr int V = Vec<T>::V;
  constexpr int A = Ring<MODE>::kOperands, S = Ring<MODE>::kStages;
  constexpr bool kSums = MODE < 2, kBackward = (MODE & 1) != 0;
  extern __shared__ unsigned char bn_smem_raw[];
  __shared__ unsigned long long full[S], empty[S];
  __shared__ int abort_word, last_lap[S];
  volatile int* abort_flag = &abort_word;
  const uint32_t raw = smem_u32(bn_smem_raw);
  const uint32_t ring = (raw + 127u) & ~127u;
  const unsigned char* ring_ptr = bn_smem_raw + (ring - raw);

  const int row_bytes = C * (int)sizeof(T);
  const int R = kChunkBytes / row_bytes;                 // rows per chunk (a power of two >= 4)
  const int c_lanes = C / V;
  const int64_t n_chunks = (n + R - 1) / R;
  const int64_t k_begin = (int64_t)blockIdx.x * chunks_per_block;
  const int64_t k_end = min(n_chunks, k_begin + chunks_per_block);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), kConsumers / 32);
      last_lap[s] = -1;
    }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  float s0[V], s1[V];
#pragma unroll
  for (int i = 0; i < V; ++i) s0[i] = s1[i] = 0.f;
  int cur = -1;
  const int cl = threadIdx.x % c_lanes, c0 = cl * V;
  const int b_common = (kSums && k_begin < k_end) ? sample_of(batch, k_begin * R, B, nullptr) : -1;

  if (warp == kConsumers / 32) {
    // ---- producer: lane 0 keeps the ring full
    if (lane == 0) {
      for (int64_t k = k_begin; k < k_end; ++k) {
        const int64_t i = k - k_begin;
        const int s = (int)(i % S);
        const int lap = (int)(i / S);
        if (lap > 0 && !mbar_wait(smem_u32(&empty[s]), (uint32_t)(lap - 1) & 1u, abort_flag, status)) break;
        const int64_t row_start = k * R;
        const int rows = (int)min((int64_t)R, n - row_start);
        const uint32_t bytes = (uint32_t)rows * (uint32_t)row_bytes;
        // batch indices travel with the chunk, in whole 16-byte pieces (the last rows of the last chunk, at most
        // three, are read directly by their consumers)
        const uint32_t id_bytes = batch ? ((uint32_t)rows * 4u) & ~15u : 0u;
        const uint32_t bar = smem_u32(&full[s]);
        const uint32_t stage = ring + (uint32_t)s * Ring<MODE>::kStageBytes;
        mbar_arrive_expect_tx(bar, A * bytes + id_bytes);
        last_lap[s] = lap;
        bulk_load(stage, x + row_start * C, bytes, bar);
        if (A == 2) bulk_load(stage + kChunkBytes, dy + row_start * C, bytes, bar);
        if (id_bytes) bulk_load(stage + A * kChunkBytes, batch + row_start, id_bytes, bar);
      }
    }
  } else {
    // ---- consumers: thread t owns vectors t, t + 256, t + 512, t + 768 of every chunk (always the same V channels)
    const int rl = threadIdx.x / c_lanes, r_step = kConsumers / c_lanes;
    float a[V], b[V], wc[V], bc[V], q0[V], q1[V];
    float ic = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      a[i] = q0[i] = q1[i] = 0.f;
      b[i] = 1.f;
      wc[i] = (MODE != 0 && w) ? __ldg(w + c0 + i) : 1.f;
      bc[i] = (MODE != 0 && bias) ? __ldg(bias + c0 + i) : 0.f;
    }
    auto flush = [&]() {                       // sums of a sample other than the block's first: added directly
      if (!kSums || cur < 0) return;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        atomicAdd(sums_out + ((int64_t)cur * C + c0 + i) * 2, s0[i]);
        atomicAdd(sums_out + ((int64_t)cur * C + c0 + i) * 2 + 1, s1[i]);
        s0[i] = s1[i] = 0.f;
      }
    };
    for (int64_t k = k_begin; k < k_end; ++k) {
      const int64_t i = k - k_begin;
      const int s = (int)(i % S);
      const uint32_t parity = (uint32_t)(i / S) & 1u;
      const int64_t row_start = k * R;
      const int rows = (int)min((int64_t)R, n - row_start);
      int ok = 1;
      if (lane == 0) ok = mbar_wait(smem_u32(&full[s]), parity, abort_flag, status) ? 1 : 0;
      if (!__shfl_sync(0xFFFFFFFFu, ok, 0)) break;
      const unsigned char* stage = ring_ptr + (size_t)s * Ring<MODE>::kStageBytes;
      const uint4* sx = reinterpret_cast<const uint4*>(stage);
      const uint4* sd = reinterpret_cast<const uint4*>(stage + (A - 1) * kChunkBytes);
      const int32_t* sid = reinterpret_cast<const int32_t*>(stage + A * kChunkBytes);
      const int rows_copied = rows & ~3;           // rows whose batch index came with the chunk
      int bt[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row_local = rl + j * r_step;
        int bj = -2;
        if (row_local < rows) {
          bj = !batch ? 0 : (row_local < rows_copied ? sid[row_local] : __ldg(batch + row_start + row_local));
          if ((unsigned)bj >= (unsigned)B) {
            if (status) atomicOr(status, ST_DEV_BAD_INDEX);
            bj = -1;
          }
        }
        bt[j] = bj;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (bt[j] == -2) continue;
        const uint4 xr = sx[j * kConsumers + threadIdx.x];
        uint4 dr = xr;
        if (A == 2) dr = sd[j * kConsumers + threadIdx.x];
        T* dst = kSums ? nullptr : out + row_start * C + (int64_t)(j * kConsumers + threadIdx.x) * V;
        if (bt[j] < 0) {                         // index outside [0, B): joins no sum, comes out as zeros
          if (kSums) {
            flush();
            cur = -1;
          } else {
            float zero[V];
#pragma unroll
            for (int i = 0; i < V; ++i) zero[i] = 0.f;
            store_vec(dst, zero);
          }
          continue;
        }
        if (bt[j] != cur) {
          flush();                               // the sums of the sample being left go out directly
          cur = bt[j];
          const int64_t sc = (int64_t)cur * C + c0;
#pragma unroll
          for (int i = 0; i < V; ++i) {
            if (MODE == 0) {
              a[i] = shift_from_row(x, first_row, cur, C, c0 + i);
            } else {
              a[i] = __ldg(p0 + sc + i);
              b[i] = __ldg(rstd + sc + i);
            }
            if (MODE == 3) {
              q0[i] = __ldg(sums_in + (sc + i) * 2);
              q1[i] = __ldg(sums_in + (sc + i) * 2 + 1);
            }
          }
          if (MODE == 3) ic = __ldg(inv_count + cur);
        }
        float xv[V], res[V];
        unpack_vec<T>(xr, xv);
        if (MODE == 0) {
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float v = xv[i] - a[i];
            s0[i] += v;
            s1[i] += v * v;
          }
        } else if (MODE == 2) {
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float v = (xv[i] - a[i]) * b[i];
            if (w) v *= wc[i];
            if (bias) v += bc[i];
            if (relu) v = fmaxf(v, 0.f);
            res[i] = v;
          }
          store_vec(dst, res);
        } else {
          float dv[V];
          unpack_vec<T>(dr, dv);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float xhat = (xv[i] - a[i]) * b[i];
            float dz = dv[i];
            if (relu && !(xhat * wc[i] + bc[i] > 0.f)) dz = 0.f;
            if (MODE == 1) {
              s0[i] += dz;
              s1[i] += dz * xhat;
            } else {
              res[i] = b[i] * wc[i] * (dz - ic * (q0[i] + xhat * q1[i]));
            }
          }
          if (MODE == 3) store_vec(dst, res);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[s]));          // this warp has read its part of the stage
    }
    if (kSums && cur != b_common) flush();       // what is left belongs to another sample than the block's first
  }

  if (kSums) {
    // Partial sums of the block's first sample: row lanes that share a warp are added by shuffles, the rest
    // through shared memory, then one atomic per channel and component.
    const bool consumer = warp < kConsumers / 32;
    if (consumer) {
      for (int d = c_lanes; d < 32; d <<= 1) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          s0[i] += __shfl_xor_sync(0xFFFFFFFFu, s0[i], d);
          s1[i] += __shfl_xor_sync(0xFFFFFFFFu, s1[i], d);
        }
      }
    }
    const bool warp_shared = c_lanes < 32;
    const int groups = warp_shared ? kConsumers / 32 : kConsumers / c_lanes;
    __syncthreads();                             // every stage has been read (or a wait gave up): the ring is free
    float* red = reinterpret_cast<float*>(bn_smem_raw + (ring - raw));
    if (consumer && (!warp_shared || lane < c_lanes)) {
      float* mine = red + ((size_t)(warp_shared ? warp : threadIdx.x / c_lanes) * c_lanes + cl) * 2 * V;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        mine[2 * i] = s0[i];
        mine[2 * i + 1] = s1[i];
      }
    }
    __syncthreads();
    if (b_common >= 0 && !*abort_flag) {
      for (int e = threadIdx.x; e < 2 * C; e += kThreads) {
        float acc = 0.f;
        for (int q = 0; q < groups; ++q) acc += red[(size_t)q * c_lanes * 2 * V + e];
        const int c = (e / (2 * V)) * V + (e % (2 * V)) / 2;
        atomicAdd(sums_out + ((int64_t)b_common * C + c) * 2 + (e & 1), acc);
      }
    }
  } else {
    __syncthreads();
  }
  // A wait gave up: before the block's shared memory is released, give every copy that was issued a (bounded)
  // chance to land.
  if (*abort_flag && threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      if (last_lap[s] < 0) continue;
      const long long t0 = clock64();
      while (!mbar_try(smem_u32(&full[s]), (uint32_t)last_lap[s] & 1u) && clock64() - t0 < kWaitCycles) {
      }
    }
  }
}

// mean / rstd of every (sample, channel) from the shifted one-pass sums, and the running buffers (averages of the
// per-sample statistics over all B samples, empty ones counting as zero).  A block covers 32 channels with 16
// sample lanes, so the loads of a sample's shift row (one DRAM round trip each) overlap instead of queueing up
// behind one another; the per-channel totals are added in a fixed order (lane by lane), so the running buffers
// come out the same on every run.
constexpr int kFinChannels = 32, kFinLanes = 16;
template <typename T>
__global__ void __launch_bounds__(kFinChannels * kFinLanes)
bn_finalize_kernel(const float* __restrict__ sums, const T* __restrict__ x, const int32_t* __restrict__ first_row,
                   const float* __restrict__ inv_count, int B, int C, float eps, float momentum, float* __restrict__ mean,
                   float* __restrict__ rstd, float* running_mean, float* running_var) {
  __shared__ float part_mean[kFinLanes][kFinChannels], part_var[kFinLanes][kFinChannels];
  const int tx = threadIdx.x % kFinChannels, ty = threadIdx.x / kFinChannels;
  const int c = blockIdx.x * kFinChannels + tx;
  float mean_sum = 0.f, var_sum = 0.f;
  if (c < C) {
    for (int b = ty; b < B; b += kFinLanes) {
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
  }
  part_mean[ty][tx] = mean_sum;
  part_var[ty][tx] = var_sum;
  __syncthreads();
  if (ty != 0 || c >= C) return;
  mean_sum = var_sum = 0.f;
  for (int l = 0; l < kFinLanes; ++l) {
    mean_sum += part_mean[l][tx];
    var_sum += part_var[l][tx];
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

// The streaming kernels need whole 16-byte vectors per row, a power-of-two number of them (<= 256: every block
// thread keeps its channels from chunk to chunk and a chunk holds at least four rows) and 16-byte aligned operands.
template <typename T>
bool stream_ok(int C, const void* a, const void* b, const void* c) {
  constexpr int V = Vec<T>::V;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (C % V != 0) return false;
  const int lanes = C / V;
  return lanes >= 1 && lanes <= kBnThreads && (lanes & (lanes - 1)) == 0 && al(a) && al(b) && al(c);
}
bool ids_ok(const int32_t* batch) { return (reinterpret_cast<uintptr_t>(batch) & 15) == 0; }

constexpr int kBnMaxDevices = 64;
int bn_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kBnMaxDevices) ? dev : 0;
}
int bn_sm_count() {
  static int count[kBnMaxDevices] = {0};
  const int dev = bn_device();
  if (count[dev] == 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    count[dev] = v > 0 ? v : 148;
  }
  return count[dev];
}

// Launches bn_stream_kernel<T, MODE> over all n rows: two blocks per SM, each a contiguous range of chunks.
template <typename T, int MODE>
bool launch_stream(const T* x, const T* dy, const int32_t* batch, int64_t n, int C, int B, const float* p0, const float* rstd,
                   const float* w, const float* bias, int relu, const float* sums_in, const float* inv_count, float* sums_out,
                   T* out, const int32_t* first_row, int32_t* status, cudaStream_t s) {
  auto kernel = bn_stream_kernel<T, MODE>;
  constexpr int smem = stream::Ring<MODE>::kBytes;
  static bool configured[kBnMaxDevices] = {};
  const int dev = bn_device();
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    configured[dev] = true;
  }
  const int rows = stream::kChunkBytes / (C * (int)sizeof(T));
  const int64_t n_chunks = (n + rows - 1) / rows;
  int64_t grid = 2 * (int64_t)bn_sm_count();
  if (grid > n_chunks) grid = n_chunks;
  const int64_t per_block = (n_chunks + grid - 1) / grid;
  grid = (n_chunks + per_block - 1) / per_block;
  kernel<<<(unsigned)grid, stream::kThreads, smem, s>>>(x, dy, batch, n, C, B, p0, rstd, w, bias, relu, sums_in, inv_count,
                                                         sums_out, out, first_row, per_block, status);
  return true;
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
    if (stream_ok<T>(C, X, Y, nullptr) && ids_ok(batch) &&
        launch_stream<T, 2>(static_cast<const T*>(X), nullptr, batch, n, C, B, mean, rstd, weight, bias, relu, nullptr, nullptr,
                            nullptr, static_cast<T*>(Y), nullptr, status, s)) {
    } else if (vec_ok<T>(C, X, Y, nullptr))
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
      if (stream_ok<T>(C, X, dY, nullptr) && ids_ok(batch) &&
          launch_stream<T, 1>(static_cast<const T*>(X), static_cast<const T*>(dY), batch, n, C, B, mean, rstd, weight, bias, relu,
                              nullptr, nullptr, sums, nullptr, nullptr, status, s)) {
      } else if (vec_ok<T>(C, X, dY, nullptr))
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
    if (stream_ok<T>(C, X, dY, dX) && ids_ok(batch) &&
        launch_stream<T, 3>(static_cast<const T*>(X), static_cast<const T*>(dY), batch, n, C, B, mean, rstd, weight, bias, relu,
                            sums, inv_count, nullptr, static_cast<T*>(dX), nullptr, status, s)) {
    } else if (vec_ok<T>(C, X, dY, dX))
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
      if (stream_ok<T>(C, X, nullptr, nullptr) && ids_ok(batch) &&
          launch_stream<T, 0>(static_cast<const T*>(X), nullptr, batch, n, C, B, nullptr, nullptr, nullptr, nullptr, 0, nullptr,
                              nullptr, sums, nullptr, first_row, status, s)) {
      } else if (vec_ok<T>(C, X, nullptr, nullptr)) {
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
    bn_finalize_kernel<T><<<(unsigned)((C + kFinChannels - 1) / kFinChannels), kFinChannels * kFinLanes, 0, s>>>(sums, static_cast<const T*>(X), n > 0 ? first_row : nullptr,
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
