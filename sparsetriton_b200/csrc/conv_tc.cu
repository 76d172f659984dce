// Implicit-GEMM sparse convolution on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   OUT[r, :] = sum_k  IN[map(r,k), :] . B_k            r = output row, k = kernel offset
//
// One persistent CTA per SM walks 128-row output tiles.  The fp32 accumulator of a tile lives in
// TMEM for all of its kernel offsets (two buffers, so the epilogue of tile i overlaps the MMAs of
// tile i+1).  Warp roles:
//   warps 0-3  epilogue : tcgen05.ld the accumulator, convert, store rows of OUT
//   warp  4    MMA      : one elected lane issues tcgen05.mma / tcgen05.commit
//   warps 5-8  producer : per non-empty (tile, offset) and per 128-byte slice of the reduction
//                         dimension, gather the 128 input rows (cp.async, 16 B, zero-fill for "no
//                         neighbour") and the matching slice of W[k] into a ring of shared-memory
//                         stages laid out in the 128-byte-swizzled canonical operand format
// Stages are handed over with mbarriers: cp.async completion arrives on `full`, tcgen05.commit on
// `empty`.  (tile, offset) pairs in which no row has a neighbour are skipped altogether.
// Every wait is bounded: on expiry the kernel records ST_DEV_TIMEOUT and unwinds.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "conv_maps.cuh"
#include "conv_tc.cuh"

namespace st {

namespace tc {

constexpr int kTileM = 128;
constexpr int kEpilogueWarps = 4, kProducerWarps = 4;
constexpr int kMmaWarp = kEpilogueWarps;                       // warp 4
constexpr int kFirstProducerWarp = kMmaWarp + 1;               // warps 5..8
constexpr int kThreads = (kEpilogueWarps + 1 + kProducerWarps) * 32;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kABlockBytes = kTileM * 128;                     // 128 rows x 128 B
constexpr int kMaxStages = 8;
constexpr long long kWaitCycles = 4000000000ll;                // ~2 s at 2 GHz

__device__ int32_t g_status[4];                                // [0] flags, [1] where, [2] block, [3] extra

struct Params {
  const void* in;          // (n_src, c_red)
  const void* w;           // (K, rows_w, cols_w)
  void* out;               // (n_rows, c_acc)
  int64_t n_rows, n_src;
  int K, c_red, c_acc;
  int esize;               // bytes per element (2 or 4)
  int w_rows, w_cols;      // W[k] is (w_rows, w_cols) row-major in memory
  int b_mn_major;          // 1: B_k = W[k] (rows = reduction), 0: B_k = W[k]^T (cols = reduction)
  int k_blocks;            // 128-byte slices of the reduction dimension
  int a_stage_bytes;       // kABlockBytes
  int w_stage_bytes;       // bytes of one W slice
  int stage_bytes;
  int stages;
  int tmem_cols;           // power of two >= 2 * c_acc
  uint32_t idesc;
  int out_kind;            // ST_F32 / ST_F16 / ST_BF16
  int64_t n_tiles;
};

// ------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.shared::cta.b64 t, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false if the limit expired or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      if (atomicOr(&g_status[0], ST_DEV_TIMEOUT) == 0) {
        g_status[1] = where;
        g_status[2] = blockIdx.x;
      }
      return false;
    }
  }
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void producer_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kProducerThreads) : "memory");
}

// Shared-memory operand descriptor for rows of 128 bytes.
//   lbo_bytes  distance between 128-byte column blocks (MN-major operands); ignored for K-major
//   sbo_bytes  distance between row groups: 1024 (8 rows) for the 128-byte swizzle, 512 (4 rows) for
//              the 128-byte swizzle with 32-byte atoms
//   layout     2 = SWIZZLE_128B (16-byte chunk index ^= row % 8)
//              1 = SWIZZLE_128B_BASE32B (32-byte chunk index ^= row % 4): the only swizzled layout
//                  the tensor core accepts for an MN-major operand of 32-bit elements (tf32)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;   // descriptor version of sm_100
  d |= (uint64_t)layout << 61;
  return d;
}

// Position (in 16-byte units) at which logical chunk c of row r is stored inside its 128-byte row.
__device__ __forceinline__ int swz16(int c, int r) { return c ^ (r & 7); }
__device__ __forceinline__ int swz32(int c, int r) { return c ^ ((r & 3) << 1); }

struct __align__(8) Control {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long acc_full[2];
  unsigned long long acc_empty[2];
  uint32_t stage_info[kMaxStages];     // bit0 first stage of its tile, bit1 last stage, bits 8.. MMA K-steps
  uint32_t group_mask[kProducerWarps]; // per-warp "some row has a neighbour" bits of the current offset group
  uint32_t tmem_base;
  int abort_flag;
};

// Store 32 fp32 accumulator columns of one row.
template <int N>
__device__ __forceinline__ void store_cols(void* out_row, int col0, int out_kind, const uint32_t* v) {
  if (out_kind == ST_F32) {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out_row) + col0);
#pragma unroll
    for (int i = 0; i < N / 4; ++i)
      dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]),
                           __uint_as_float(v[4 * i + 3]));
  } else {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(out_row) + (size_t)col0 * 2);
#pragma unroll
    for (int i = 0; i < N / 8; ++i) {
      uint32_t p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float lo = __uint_as_float(v[8 * i + 2 * j]), hi = __uint_as_float(v[8 * i + 2 * j + 1]);
        if (out_kind == ST_BF16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
          p[j] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(lo, hi);
          p[j] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      dst[i] = make_uint4(p[0], p[1], p[2], p[3]);
    }
  }
}

template <typename Map>
__global__ void __launch_bounds__(kThreads, 1) gather_kernel(const Params p, const Map map) {
  extern __shared__ unsigned char smem_raw[];
  // stage ring first (1024-byte aligned for the swizzle pattern), control block after it
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  unsigned char* ring_ptr = smem_raw + (ring - raw);
  Control* ctl = reinterpret_cast<Control*>(ring_ptr + (size_t)p.stages * p.stage_bytes);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), kProducerThreads + 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[b]), kEpilogueWarps * 32);
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&ctl->tmem_base), (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  const int red_bytes = p.c_red * p.esize;

  if (warp >= kFirstProducerWarp) {
    // =============================================================== producers
    const int t = threadIdx.x - kFirstProducerWarp * 32;    // 0..127 = row inside the tile
    const int pwarp = t >> 5;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const int kr = 128 / p.esize;                            // reduction elements per 128-byte slice
    const int w_col_bytes = p.w_cols * p.esize;

    // Fill one stage: slice kb of the gathered rows and of W[k]; kb < 0 sends the end-of-tile marker.
    auto emit = [&](int k, int kb, bool has, int32_t src_row, bool first) {
      ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag, 1);
      if (!ok) return;
      int valid_bytes = 0;
      if (kb >= 0) {
        const uint32_t a_base = ring + (uint32_t)stage * p.stage_bytes;
        const uint32_t w_base = a_base + p.a_stage_bytes;
        // ---- A: this thread's row, up to 8 chunks of 16 B; chunk c is stored at position c ^ (row % 8)
        valid_bytes = min(128, red_bytes - kb * 128);
        const int chunks = valid_bytes >> 4;
        const char* src = has ? static_cast<const char*>(p.in) + (size_t)src_row * red_bytes + kb * 128
                              : static_cast<const char*>(p.w);
        const uint32_t a_row = a_base + (uint32_t)t * 128u;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (c < chunks) cp_async16(a_row + (uint32_t)((c ^ (t & 7)) << 4), src + (has ? c * 16 : 0), has ? 16u : 0u);
        // ---- slice of W[k]
        const char* wk = static_cast<const char*>(p.w) + (size_t)k * p.w_rows * w_col_bytes;
        if (p.b_mn_major) {
          // rows [kb*kr, kb*kr + R) of W[k], all 128-byte column blocks; block cb sits kr*128 B after block cb-1
          const int R = min(kr, p.w_rows - kb * kr);
          const int n_cb = (w_col_bytes + 127) >> 7;
          const char* wrow0 = wk + (size_t)kb * kr * w_col_bytes;
          for (int cb = 0; cb < n_cb; ++cb) {
            const int cb_chunks = min(128, w_col_bytes - cb * 128) >> 4;
            const uint32_t blk = w_base + (uint32_t)(cb * kr * 128);
            for (int e = t; e < R * 8; e += kProducerThreads) {
              const int c = e & 7, r = e >> 3;
              if (c < cb_chunks)
                cp_async16(blk + (uint32_t)(r * 128 + ((p.esize == 4 ? swz32(c, r) : swz16(c, r)) << 4)),
                           wrow0 + (size_t)r * w_col_bytes + cb * 128 + c * 16, 16u);
            }
          }
        } else {
          // column block kb of W[k] (columns = reduction), all w_rows rows
          const int wchunks = min(128, w_col_bytes - kb * 128) >> 4;
          for (int e = t; e < p.w_rows * 8; e += kProducerThreads) {
            const int c = e & 7, r = e >> 3;
            if (c < wchunks)
              cp_async16(w_base + (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)),
                         wk + (size_t)r * w_col_bytes + kb * 128 + c * 16, 16u);
          }
        }
      }
      cp_async_arrive_noinc(smem_u32(&ctl->full[stage]));
      if (t == 0) {
        ctl->stage_info[stage] = (first ? 1u : 0u) | (kb < 0 ? 2u : 0u) | ((uint32_t)(valid_bytes >> 5) << 8);
        mbar_arrive(smem_u32(&ctl->full[stage]));
      }
      if (++stage == p.stages) {
        stage = 0;
        phase ^= 1u;
      }
    };

    for (int64_t tile = blockIdx.x; tile < p.n_tiles && ok; tile += gridDim.x) {
      const int64_t row = tile * kTileM + t;
      const bool row_ok = row < p.n_rows;
      typename Map::RowState rs = map.row_state(row, row_ok);
      int done = 0;                                          // offsets of this tile sent so far
      for (int k0 = 0; k0 < p.K && ok; k0 += 32) {
        // which of the offsets k0..k0+31 have a neighbour in this row / in any row of the tile
        uint32_t mine = 0;
        const int kn = min(32, p.K - k0);
        for (int j = 0; j < kn; ++j) {
          const int32_t i = row_ok ? map.get(rs, row, k0 + j) : -1;
          if (i >= 0 && i < p.n_src) mine |= 1u << j;
        }
        const uint32_t warp_mask = __reduce_or_sync(0xFFFFFFFFu, mine);
        producer_bar_sync();                                 // the previous group's masks have been read
        if (lane == 0) ctl->group_mask[pwarp] = warp_mask;
        producer_bar_sync();
        uint32_t m = ctl->group_mask[0] | ctl->group_mask[1] | ctl->group_mask[2] | ctl->group_mask[3];
        while (m && ok) {
          const int j = __ffs(m) - 1;
          m &= m - 1;
          const bool has = (mine >> j) & 1u;
          const int32_t src_row = has ? map.get(rs, row, k0 + j) : 0;
          for (int kb = 0; kb < p.k_blocks && ok; ++kb) emit(k0 + j, kb, has, src_row, done == 0 && kb == 0);
          ++done;
        }
      }
      // a tile without any neighbour still has to produce zeros: one all-zero slice against W[0]
      if (ok && done == 0) emit(0, 0, false, 0, true);
      if (ok) emit(0, -1, false, 0, false);                  // end-of-tile marker
    }
    cp_async_wait_all();
  } else if (warp == kMmaWarp) {
    // =============================================================== MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      const int a_kstep_bytes = 32;
      // MN-major B: one K-step covers 32 B of reduction = (32/esize) rows of 128 B
      const int b_kstep_bytes = p.b_mn_major ? (32 / p.esize) * 128 : 32;
      const uint32_t b_lbo = p.b_mn_major ? (uint32_t)(128 / p.esize) * 128u : 16u;
      const bool b_base32 = p.b_mn_major && p.esize == 4;
      const uint32_t b_sbo = b_base32 ? 512u : 1024u, b_layout = b_base32 ? 1u : 2u;
      for (int64_t tile = blockIdx.x; tile < p.n_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[buf]), acc_phase[buf] ^ 1u, abort_flag, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_addr = tmem_base + (uint32_t)(buf * p.c_acc);
        for (;;) {
          ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_flag, 3);
          if (!ok) break;
          fence_proxy_async();
          tc_fence_after();
          const uint32_t info = ctl->stage_info[stage];
          const int ksteps = (int)(info >> 8);
          const uint32_t a_base = ring + (uint32_t)stage * p.stage_bytes;
          const uint32_t w_base = a_base + p.a_stage_bytes;
          for (int ks = 0; ks < ksteps; ++ks) {
            const uint64_t da = smem_desc(a_base + ks * a_kstep_bytes, 16u, 1024u, 2u);
            const uint64_t db = smem_desc(w_base + ks * b_kstep_bytes, b_lbo, b_sbo, b_layout);
            const uint32_t accumulate = ((info & 1u) && ks == 0) ? 0u : 1u;
            if (p.esize == 2)
              mma_f16(d_addr, da, db, p.idesc, accumulate);
            else
              mma_tf32(d_addr, da, db, p.idesc, accumulate);
          }
          mma_commit(smem_u32(&ctl->empty[stage]));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
          if (info & 2u) break;                             // end-of-tile marker (carries no MMA)
        }
        if (!ok) break;
        mma_commit(smem_u32(&ctl->acc_full[buf]));
        acc_phase[buf] ^= 1u;
        buf ^= 1;
      }
    }
    __syncwarp();
  } else {
    // =============================================================== epilogue (warps 0..3)
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    bool ok = true;
    const int out_es = p.out_kind == ST_F32 ? 4 : 2;
    for (int64_t tile = blockIdx.x; tile < p.n_tiles && ok; tile += gridDim.x) {
      ok = mbar_wait(smem_u32(&ctl->acc_full[buf]), acc_phase[buf], abort_flag, 4);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int64_t row = tile * kTileM + warp * 32 + lane;
      char* out_row = static_cast<char*>(p.out) + (size_t)row * p.c_acc * out_es;
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * p.c_acc);
      for (int c0 = 0; c0 < p.c_acc; c0 += 32) {
        uint32_t v[32];
        if (p.c_acc - c0 >= 32) {
          tmem_ld32(t_row + c0, v);
          tmem_ld_wait();
          if (row < p.n_rows) store_cols<32>(out_row, c0, p.out_kind, v);
        } else {
          tmem_ld16(t_row + c0, v);
          tmem_ld_wait();
          if (row < p.n_rows) store_cols<16>(out_row, c0, p.out_kind, v);
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->acc_empty[buf]));
      acc_phase[buf] ^= 1u;
      buf ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// Map adapters: what a producer thread keeps per row.
struct StoredRows {
  const int32_t* nbr;
  int K;
  struct RowState {};
  __device__ __forceinline__ RowState row_state(int64_t, bool) const { return RowState{}; }
  __device__ __forceinline__ int32_t get(const RowState&, int64_t row, int k) const {
    return __ldg(nbr + row * K + k);
  }
};

}  // namespace tc

static int g_sm_count = 0;

static int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count = n > 0 ? n : 148;
  }
  return g_sm_count;
}

static bool g_tc_enabled = true;

void tc_set_enabled(bool on) { g_tc_enabled = on; }

bool tc_supported(int dtype, int c_red, int c_acc) {
  if (!g_tc_enabled) return false;
  if (dtype != ST_F32 && dtype != ST_F16 && dtype != ST_BF16) return false;
  const int es = dtype == ST_F32 ? 4 : 2;
  const int kstep = 32 / es;                       // reduction elements per MMA
  if (c_red < kstep || c_red % kstep != 0 || c_red > 512) return false;
  if (c_acc < 16 || c_acc % 16 != 0 || c_acc > 256) return false;
  return true;
}

static bool fill_params(tc::Params* p, int dtype, const void* in, const void* w, void* out, int64_t n_rows,
                        int64_t n_src, int K, int c_red, int c_acc, bool w_transposed) {
  const int es = dtype == ST_F32 ? 4 : 2;
  p->in = in;
  p->w = w;
  p->out = out;
  p->n_rows = n_rows;
  p->n_src = n_src;
  p->K = K;
  p->c_red = c_red;
  p->c_acc = c_acc;
  p->esize = es;
  p->b_mn_major = w_transposed ? 0 : 1;
  p->w_rows = w_transposed ? c_acc : c_red;
  p->w_cols = w_transposed ? c_red : c_acc;
  p->k_blocks = (c_red * es + 127) / 128;
  p->a_stage_bytes = tc::kABlockBytes;
  if (p->b_mn_major) {
    const int n_cb = (c_acc * es + 127) / 128;
    p->w_stage_bytes = n_cb * (128 / es) * 128;
  } else {
    p->w_stage_bytes = c_acc * 128;
  }
  p->w_stage_bytes = (p->w_stage_bytes + 1023) / 1024 * 1024;
  p->stage_bytes = p->a_stage_bytes + p->w_stage_bytes;
  const int budget = 200 * 1024;
  int stages = budget / p->stage_bytes;
  if (stages > tc::kMaxStages) stages = tc::kMaxStages;
  if (stages < 2) return false;
  p->stages = stages;
  int cols = 32;
  while (cols < 2 * c_acc) cols <<= 1;
  p->tmem_cols = cols;
  const uint32_t fmt = dtype == ST_F16 ? 0u : (dtype == ST_BF16 ? 1u : 2u);
  p->idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)p->b_mn_major << 16) | ((uint32_t)(c_acc >> 3) << 17) |
             ((uint32_t)(tc::kTileM >> 4) << 24);
  p->out_kind = dtype;
  p->n_tiles = (n_rows + tc::kTileM - 1) / tc::kTileM;
  return true;
}

int tc_conv_gather(int dtype, const void* in, const void* w, const int32_t* map, void* out, int64_t n_rows,
                   int64_t n_src, int K, int c_red, int c_acc, bool w_transposed, cudaStream_t stream) {
  tc::Params p;
  if (!fill_params(&p, dtype, in, w, out, n_rows, n_src, K, c_red, c_acc, w_transposed)) {
    set_error("tc_conv_gather: shape does not fit the shared-memory ring");
    return ST_ERR_UNSUPPORTED;
  }
  if (n_rows == 0) return ST_OK;
  const size_t smem = (size_t)p.stages * p.stage_bytes + sizeof(tc::Control) + 1024;
  auto kernel = tc::gather_kernel<tc::StoredRows>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      set_error("tc_conv_gather: cannot raise the dynamic shared memory limit: %s", cudaGetErrorString(e));
      return ST_ERR_CUDA;
    }
    configured = true;
  }
  int64_t grid = p.n_tiles < sm_count() ? p.n_tiles : sm_count();
  tc::StoredRows rows{map, K};
  kernel<<<(unsigned)grid, tc::kThreads, smem, stream>>>(p, rows);
  note_launches(1);
  return check_launch("tc_conv_gather");
}

int tc_read_status(int32_t* host_out4, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyFromSymbolAsync(host_out4, tc::g_status, sizeof(int32_t) * 4, 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    set_error("tc_read_status: %s", cudaGetErrorString(e));
    return ST_ERR_CUDA;
  }
  return ST_OK;
}

}  // namespace st
