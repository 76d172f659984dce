// Implicit-GEMM sparse convolution on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   OUT[r, :] = sum_k  IN[map(r,k), :] . B_k            r = output row, k = kernel offset
//
// Persistent CTAs (one per SM) of 288 threads with fixed warp roles:
//   warps 0-3  epilogue : tcgen05.ld the accumulators, convert, store rows of OUT
//   warp  4    MMA      : one elected lane issues tcgen05.mma / tcgen05.commit
//   warps 5-8  producer : gather the input rows (cp.async, 16 B, zero-fill for "no neighbour") and
//                         the slices of W[k] into shared-memory rings laid out in the
//                         128-byte-swizzled canonical operand format
// Rings are handed over with mbarriers; every wait is bounded: on expiry the kernel records
// ST_DEV_TIMEOUT in a sticky device word and unwinds.  The same producer code serves a stored
// neighbour map or the coordinate hash table probed on the fly (the Map template argument).
// Stored maps that come with a tile plan run on the TMA-fed kernels of conv_tc_plan.cuh; the kernels in
// this file are their cp.async counterparts (hash on the fly, maps without a plan, unaligned tensors).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "conv_maps.cuh"
#include "conv_tc.cuh"
#include "tc_ptx.cuh"

namespace st {

namespace tc {

constexpr int kTileM = 128;
constexpr int kEpilogueWarps = 4, kProducerWarps = 4;
constexpr int kMmaWarp = kEpilogueWarps;                       // warp 4
constexpr int kFirstProducerWarp = kMmaWarp + 1;               // warps 5..8
constexpr int kThreads = (kEpilogueWarps + 1 + kProducerWarps) * 32;
constexpr int kProducerThreads = kProducerWarps * 32;
// The gather kernel runs several producer groups of kProducerWarps warps each (see gather2_kernel).
constexpr int kGatherGroups = 1;
constexpr int kPlannedLag = 1;          // stages a planned producer group keeps in flight behind the newest
constexpr int kGatherThreads = (kEpilogueWarps + 1 + kGatherGroups * kProducerWarps) * 32;
constexpr int kABlockBytes = kTileM * 128;                     // 128 rows x 128 B


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

// Map adapters: what a producer thread keeps per row, and how it finds the source row of offset k.
struct StoredRows {
  static constexpr bool kPlanned = false;
  const int32_t* nbr;
  int K;
  struct RowState {};
  __device__ __forceinline__ RowState row_state(int64_t, bool) const { return RowState{}; }
  __device__ __forceinline__ int32_t get(const RowState&, int64_t row, int k) const {
    return __ldg(nbr + row * K + k);
  }
};

// A stored map in tile-plan form: tmap[(tile * K + k) * 128 + r] is the source row of tile row r for
// offset k, tmask[tile * MW + k / 32] bit (k % 32) says whether the tile has any neighbour at k.
// The producers then need no staging of map entries at all: a step's 128 indices are one line.
struct PlannedRows {
  static constexpr bool kPlanned = true;
  const int32_t* tmap;
  const uint32_t* tmask;
  int K, MW;
  struct RowState {};
  __device__ __forceinline__ RowState row_state(int64_t, bool) const { return RowState{}; }
  __device__ __forceinline__ int32_t get(const RowState&, int64_t, int) const { return -1; }
};

// Forward rule of the hash-on-the-fly form: source = table[(b, out * stride - off_k)] if inside the shape.
template <typename CT>
struct HashRows {
  const CT* coords;
  Offsets off;
  Table table;
  Int3 shape;
  int stride;
  static constexpr bool kPlanned = false;
  using RowState = int4;
  __device__ __forceinline__ RowState row_state(int64_t row, bool valid) const {
    return valid ? load_coord<CT>(coords, row) : make_int4(0, 0, 0, 0);
  }
  __device__ __forceinline__ int32_t get(const RowState& c, int64_t, int k) const {
    const int x = c.y * stride - off.v[k * 3 + 0];
    const int y = c.z * stride - off.v[k * 3 + 1];
    const int z = c.w * stride - off.v[k * 3 + 2];
    if (x < 0 || x >= shape.x || y < 0 || y >= shape.y || z < 0 || z >= shape.z || table.capacity == 0 ||
        !key_representable(c.x, x, y, z))
      return -1;
    return table_find(table, pack_key(c.x, x, y, z));
  }
};

// Inverse rule (feature gradient): rows are inputs with table-space coordinate q; the source is the
// output row at (q + off_k) / stride when the division is exact on every axis and that output exists.
struct InverseRows {
  const int32_t* q;        // (n_in, 4) int32, batch = -1 for rows that are not in the input table
  Offsets off;
  Table table;             // over the OUTPUT coordinates
  int stride;
  static constexpr bool kPlanned = false;
  using RowState = int4;
  __device__ __forceinline__ RowState row_state(int64_t row, bool valid) const {
    return valid ? __ldg(reinterpret_cast<const int4*>(q) + row) : make_int4(-1, 0, 0, 0);
  }
  __device__ __forceinline__ int32_t get(const RowState& c, int64_t, int k) const {
    if (c.x < 0 || table.capacity == 0) return -1;
    int v[3] = {c.y + off.v[k * 3 + 0], c.z + off.v[k * 3 + 1], c.w + off.v[k * 3 + 2]};
#pragma unroll
    for (int a = 0; a < 3; ++a) {
      if (v[a] < 0) return -1;
      if (stride > 1) {
        const int qt = v[a] / stride;
        if (qt * stride != v[a]) return -1;
        v[a] = qt;
      }
    }
    if (!key_representable(c.x, v[0], v[1], v[2])) return -1;
    return table_find(table, pack_key(c.x, v[0], v[1], v[2]));
  }
};


// =================================================================================================
// Gather kernel, second form: one copy of a W[k] slice serves several row tiles.
//
// A CTA works on a "super tile" of S consecutive 128-row tiles whose S accumulators sit side by side
// in TMEM (S * C_out columns; two such sets when they fit, so that the epilogue overlaps the next
// super tile).  The loop order is offset-major: for each kernel offset that has a neighbour anywhere
// in the super tile the W[k] slice is copied once into its own ring, then one gathered-row stage per
// sub tile that needs it goes through the row ring.  With the 20 %-filled maps of surface data the
// W copies were 5/6 of the shared-memory fill traffic of the first form; here they are divided by S.
// Each producer thread first fetches the map entries of its S rows for 32 offsets at a time
// (independent loads into a local array), so no stage waits for an index load.
// =================================================================================================
// Cycle counters for timing experiments: compiled in only with -DST_TC_PROFILE (and read when dbg bit
// 256 is set); otherwise PROF_CLOCK() is a constant and the bookkeeping disappears.
__device__ long long g_prof[160 * 16];
#ifdef ST_TC_PROFILE
#define PROF_CLOCK() clock64()
#define ST_DBG(p, bit) ((p).dbg & (bit))
#else
#define PROF_CLOCK() 0ll
#define ST_DBG(p, bit) 0          // the experiment switches of Params2::dbg exist in instrumented builds only
#endif


constexpr int kMaxSub = 4;
constexpr int kMaxWSlots = 4;
constexpr int kMaxAStages = 12;
constexpr int kGroup = 16;                                   // kernel offsets whose map entries are staged at a time
constexpr int kIdxTileBytes = kGroup * kMaxSub * kTileM * 4;  // 32 KB

struct Params2 {
  const void* in;
  const void* w;
  void* out;
  const int32_t* order;    // optional: tile row r stands for row order[r] of the map and of OUT
  int64_t n_rows, n_src, n_super;
  int K, c_red, c_acc, esize;
  int w_rows, w_cols, b_mn_major, k_blocks;
  int w_slot_bytes, w_slots, a_stages;
  int sub;                 // row tiles per super tile (S)
  int acc_bufs;            // 1 or 2 accumulator sets
  int tmem_cols;
  uint32_t idesc;
  int out_kind;
  int idx_bytes;           // shared memory for staged map entries (0 with a tile plan)
  int n_slots, slot_bytes; // planned_gather_kernel: ring of slots
  int part;                // planned_gather_kernel: sub tiles per slot
  int w_flip;              // 1: offset k multiplies with W[K-1-k] (feature gradient of a submanifold layer over its own map)
  int dbg;                 // timing experiments only (wrong results): 1 no proxy fence, 2 no MMA, 4 no row copies, 8 no zero-fill copies
};

struct __align__(8) Control2 {
  unsigned long long a_full[kMaxAStages], a_empty[kMaxAStages];
  unsigned long long w_full[kMaxWSlots], w_empty[kMaxWSlots];
  unsigned long long acc_full[2], acc_empty[2];
  // bits 0-1 sub tile, bit 2 first MMA into that accumulator, bit 3 takes the next W slot,
  // bit 4 frees the W slot afterwards, bit 5 end of super tile (no data), bits 8.. K-steps
  uint32_t a_info[kMaxAStages];
  uint32_t group_mask[kProducerWarps][kMaxSub];
  unsigned long long group_bar;        // barrier among the producer warps
  uint32_t tmem_base;
  int abort_flag;
};

template <typename Map, int ESIZE>
__global__ void __launch_bounds__(kGatherThreads, 1) gather2_kernel(const Params2 p, const Map map) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - raw);
  const uint32_t w_ring = base;
  const uint32_t a_ring = base + (uint32_t)(p.w_slots * p.w_slot_bytes);
  // map entries of the current offset group: idx_tile[(j * kMaxSub + s) * 128 + row]
  int32_t* idx_tile = reinterpret_cast<int32_t*>(base_ptr + (size_t)p.w_slots * p.w_slot_bytes +
                                                 (size_t)p.a_stages * kABlockBytes);
  Control2* ctl = reinterpret_cast<Control2*>(reinterpret_cast<unsigned char*>(idx_tile) + p.idx_bytes);
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.a_stages; ++s) {
      mbar_init(smem_u32(&ctl->a_full[s]), kProducerWarps);
      mbar_init(smem_u32(&ctl->a_empty[s]), 1);
    }
    for (int s = 0; s < p.w_slots; ++s) {
      mbar_init(smem_u32(&ctl->w_full[s]), kProducerWarps);
      mbar_init(smem_u32(&ctl->w_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[b]), kEpilogueWarps * 32);
    }
    mbar_init(smem_u32(&ctl->group_bar), kProducerWarps);
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
  const int red_bytes = p.c_red * ESIZE;
  const int set_cols = p.sub * p.c_acc;                      // TMEM columns of one accumulator set

  if (warp >= kFirstProducerWarp) {
    // =============================================================== producers
    // Producer groups: a single warp runs its (mostly dependent) instruction stream at a fraction of
    // the issue rate, so with one producer warp per scheduler the copies were bound by instruction
    // latency.  With a stored tile plan the steps are dealt round-robin to kGatherGroups groups of four
    // warps, each of which copies whole steps on its own; the forms that stage map entries in shared
    // memory (hash on the fly, plain stored map) run on group 0 alone.
    const int group = (threadIdx.x - kFirstProducerWarp * 32) / kProducerThreads;
    const int t = (threadIdx.x - kFirstProducerWarp * 32) % kProducerThreads;
    const int pwarp = t >> 5;
    int a_stage = 0, w_slot = 0;
    uint32_t a_phase = 0, w_phase = 0;
    bool ok = true;
    const int kr = 128 / ESIZE;
    const int w_col_bytes = p.w_cols * ESIZE;
    StageQueue<Map::kPlanned ? kPlannedLag : 3> queue;
    queue.clear();
    // Barrier among the four producer warps with a bounded wait (a plain bar.sync could hang if one warp
    // had given up after an expired wait).
    uint32_t group_phase = 0;
    auto producer_sync = [&]() {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->group_bar));
      ok = mbar_wait_warp(smem_u32(&ctl->group_bar), group_phase, abort_flag, 28, lane) && ok;
      group_phase ^= 1u;
    };
    long long t_pref = 0, t_acq_a = 0, t_acq_w = 0, t_total0 = PROF_CLOCK(), t_push = 0, t_copy = 0;
    long long n_flush = 0, t_w = 0, t_idx = 0;
    // Wait until the consumer has released a slot.  If it has not yet, first hand over every stage
    // still held back in the queue, so that the consumer can never be waiting for this warp.
    auto acquire = [&](uint32_t bar, uint32_t parity, int where) {
      int ready = 0;
      if (lane == 0) ready = mbar_try(bar, parity) ? 1 : 0;
      ready = __shfl_sync(0xFFFFFFFFu, ready, 0);
      if (ready) return true;
      const long long c0 = PROF_CLOCK();
      queue.flush(lane);
      ++n_flush;
      const bool r = mbar_wait_warp(bar, parity, abort_flag, where, lane);
      if (where == 21) t_acq_w += PROF_CLOCK() - c0; else t_acq_a += PROF_CLOCK() - c0;
      return r;
    };

    auto send_w_at = [&](int k, int kb, int slot, uint32_t parity) {
      ok = acquire(smem_u32(&ctl->w_empty[slot]), parity ^ 1u, 21);
      if (!ok) return;
      const uint32_t w_base = w_ring + (uint32_t)slot * p.w_slot_bytes;
      const char* wk = static_cast<const char*>(p.w) + (size_t)(p.w_flip ? p.K - 1 - k : k) * p.w_rows * w_col_bytes;
      if (ST_DBG(p, 16)) {
      } else if (p.b_mn_major) {
        const int R = min(kr, p.w_rows - kb * kr);
        const int n_cb = (w_col_bytes + 127) >> 7;
        const char* wrow0 = wk + (size_t)kb * kr * w_col_bytes;
        for (int cb = 0; cb < n_cb; ++cb) {
          const int cb_chunks = min(128, w_col_bytes - cb * 128) >> 4;
          const uint32_t blk = w_base + (uint32_t)(cb * kr * 128);
          for (int e = t; e < R * 8; e += kProducerThreads) {
            const int c = e & 7, r = e >> 3;
            if (c < cb_chunks)
              cp_async16(blk + (uint32_t)(r * 128 + ((ESIZE == 4 ? swz32(c, r) : swz16(c, r)) << 4)),
                         wrow0 + (size_t)r * w_col_bytes + cb * 128 + c * 16, 16u);
          }
        }
      } else {
        const int wchunks = min(128, w_col_bytes - kb * 128) >> 4;
        for (int e = t; e < p.w_rows * 8; e += kProducerThreads) {
          const int c = e & 7, r = e >> 3;
          if (c < wchunks)
            cp_async16(w_base + (uint32_t)(r * 128 + (swz16(c, r) << 4)), wk + (size_t)r * w_col_bytes + kb * 128 + c * 16,
                       16u);
        }
      }
      cp_async_commit();
      queue.push(smem_u32(&ctl->w_full[slot]), lane);
    };
    auto next_w = [&]() {
      if (++w_slot == p.w_slots) {
        w_slot = 0;
        w_phase ^= 1u;
      }
    };
    auto next_a = [&]() {
      if (++a_stage == p.a_stages) {
        a_stage = 0;
        a_phase ^= 1u;
      }
    };
    auto send_w = [&](int k, int kb) {
      send_w_at(k, kb, w_slot, w_phase);
      if (ok) next_w();
    };
    // flags: see Control2::a_info.  `idx_line` holds the 128 source rows of the stage (shared memory;
    // null: a stage of zeros).  Eight consecutive lanes fetch the eight 16-byte pieces of one row, so a
    // warp-wide cp.async touches 4 whole 128-byte lines (a lane-per-row split touches 32 lines per
    // instruction and is bound by L1 wavefronts); thread t serves rows 8*(t/8) .. 8*(t/8)+7.
    auto send_a = [&](int kb, const int32_t* idx_line, uint32_t flags) {
      ok = acquire(smem_u32(&ctl->a_empty[a_stage]), a_phase ^ 1u, 22);
      if (!ok) return;
      const long long cc = PROF_CLOCK();
      int valid_bytes = 0;
      if (!(flags & 32u)) {
        valid_bytes = min(128, red_bytes - kb * 128);
        const int c = t & 7, g = t >> 3;
        if (c < (valid_bytes >> 4) && !ST_DBG(p, 4)) {
          int32_t r[8];
          if (idx_line) {
            const int4 lo = *reinterpret_cast<const int4*>(idx_line + g * 8);
            const int4 hi = *reinterpret_cast<const int4*>(idx_line + g * 8 + 4);
            r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
            r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = -1;
          }
          const char* src0 = static_cast<const char*>(p.in) + kb * 128 + c * 16;
          const uint32_t dst0 = a_ring + (uint32_t)a_stage * kABlockBytes + (uint32_t)(g * 8 * 128);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const bool has = r[i] >= 0;
            cp_async16(dst0 + (uint32_t)(i * 128 + ((c ^ i) << 4)),
                       has ? src0 + (size_t)r[i] * red_bytes : static_cast<const char*>(p.w), has ? 16u : 0u);
          }
        }
      }
      if (t == 0) ctl->a_info[a_stage] = flags | ((uint32_t)(valid_bytes >> 5) << 8);
      cp_async_commit();
      const long long cq = PROF_CLOCK();
      t_copy += cq - cc;
      queue.push(smem_u32(&ctl->a_full[a_stage]), lane);
      t_push += PROF_CLOCK() - cq;
      if (++a_stage == p.a_stages) {
        a_stage = 0;
        a_phase ^= 1u;
      }
    };

    if constexpr (Map::kPlanned) {
      // ----- stored map in tile-plan form: no staging, no barrier among the producer warps -----
      const int64_t n_tiles = (p.n_rows + kTileM - 1) / kTileM;
      const int piece = t & 7, line8 = (t >> 3) * 8;
      // A ring slot always belongs to the same group (slot index modulo the groups; the row ring has a
      // multiple of kGatherGroups slots), so the group that waits for a slot to be released has itself
      // filled it on every earlier lap.  This matters: an mbarrier wait names a phase only by its
      // parity, and a group that did not take part in a slot's previous lap could be two laps ahead
      // of the consumer and mistake an old phase for the one it needs.
      struct Step {
        const int32_t* line;     // row step: its 128 source rows (null: zeros / no data)
        int k, kb;
        uint32_t flags;          // row step: see Control2::a_info
        int slot;
        uint32_t parity;
        bool is_w, valid;
      };
      Step cur{nullptr, 0, 0, 0u, 0, 0u, false, false};
      int4 cur_lo = make_int4(-1, -1, -1, -1), cur_hi = cur_lo;
      auto run = [&](const Step& d, const int4& lo, const int4& hi) {
        if (d.is_w) {
          const long long cw = PROF_CLOCK();
          send_w_at(d.k, d.kb, d.slot, d.parity);
          t_w += PROF_CLOCK() - cw;
          return;
        }
        ok = acquire(smem_u32(&ctl->a_empty[d.slot]), d.parity ^ 1u, 22);
        if (!ok) return;
        const long long cc = PROF_CLOCK();
        int valid_bytes = 0;
        if (!(d.flags & 32u)) {
          valid_bytes = min(128, red_bytes - d.kb * 128);
          if (piece < (valid_bytes >> 4) && !ST_DBG(p, 4)) {
            const int32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const char* src0 = static_cast<const char*>(p.in) + d.kb * 128 + piece * 16;
            const uint32_t dst0 = a_ring + (uint32_t)d.slot * kABlockBytes + (uint32_t)(line8 * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const bool has = (uint32_t)r[i] < (uint32_t)p.n_src;
              cp_async16(dst0 + (uint32_t)(i * 128 + ((piece ^ i) << 4)),
                         has ? src0 + (size_t)r[i] * red_bytes : static_cast<const char*>(p.w), has ? 16u : 0u);
            }
          }
        }
        if (t == 0) ctl->a_info[d.slot] = d.flags | ((uint32_t)(valid_bytes >> 5) << 8);
        cp_async_commit();
        const long long cq = PROF_CLOCK();
        t_copy += cq - cc;
        queue.push(smem_u32(&ctl->a_full[d.slot]), lane);
        t_push += PROF_CLOCK() - cq;
      };
      // Deal one step.  Every group keeps count of the ring slots; the owner of the step's slot loads
      // the step's indices now and issues the step it had pending (one step of distance hides the load).
      auto deal = [&](const Step& d) {
        if (d.slot % kGatherGroups != group) return;
        int4 lo = make_int4(-1, -1, -1, -1), hi = lo;
        if (d.line) {
          lo = __ldg(reinterpret_cast<const int4*>(d.line + line8));
          hi = __ldg(reinterpret_cast<const int4*>(d.line + line8 + 4));
        }
        if (cur.valid && ok) run(cur, cur_lo, cur_hi);
        cur = d;
        cur_lo = lo;
        cur_hi = hi;
      };
      auto cp_emit = [&](const int32_t* line, int k, int kb, uint32_t flags, bool w_first) {
        if (w_first) {
          deal(Step{nullptr, k, kb, 0u, w_slot, w_phase, true, true});
          next_w();
        }
        deal(Step{line, k, kb, flags, a_stage, a_phase, false, true});
        next_a();
      };

      auto emit = [&](const int32_t* line, int k, int kb, uint32_t flags, bool w_first) {
        cp_emit(line, k, kb, flags, w_first);
      };
      auto load_masks = [&](int64_t tile0, int word, uint32_t* m) {
#pragma unroll
        for (int s = 0; s < kMaxSub; ++s)
          m[s] = (s < p.sub && tile0 + s < n_tiles) ? __ldg(map.tmask + (tile0 + s) * map.MW + word) : 0u;
      };
      uint32_t next_m[kMaxSub];
      load_masks((int64_t)blockIdx.x * p.sub, 0, next_m);
      for (int64_t st_i = blockIdx.x; st_i < p.n_super && ok; st_i += gridDim.x) {
        const long long cpf = PROF_CLOCK();
        const int64_t tile0 = st_i * p.sub;
        uint32_t m0[kMaxSub];
#pragma unroll
        for (int s = 0; s < kMaxSub; ++s) m0[s] = next_m[s];
        if (st_i + gridDim.x < p.n_super) {
          const int64_t next_tile0 = (st_i + gridDim.x) * p.sub;
          load_masks(next_tile0, 0, next_m);
          // The index lines of a super tile are one contiguous block of the plan.  A step's indices are
          // loaded only one step ahead, so a miss to DRAM there would cost a full memory latency per
          // step and warp: bring the next super tile's block into L2 now.
          const int64_t tiles = min((int64_t)p.sub, n_tiles - next_tile0);
          const char* block = reinterpret_cast<const char*>(map.tmap + next_tile0 * map.K * (int64_t)kTileM);
          const int64_t lines = min(tiles * map.K * 4, (int64_t)1024);           // 128-byte lines
          for (int64_t l = t; l < lines; l += kProducerThreads) prefetch_l2(block + l * 128);
        }
        t_pref += PROF_CLOCK() - cpf;
        uint32_t touched = 0;
        for (int word = 0; word < map.MW && ok; ++word) {
          uint32_t m[kMaxSub], m_any = 0;
          if (word == 0) {
#pragma unroll
            for (int s = 0; s < kMaxSub; ++s) m[s] = m0[s];
          } else {
            load_masks(tile0, word, m);
          }
#pragma unroll
          for (int s = 0; s < kMaxSub; ++s) m_any |= m[s];
          while (m_any && ok) {
            const int j = __ffs(m_any) - 1;
            m_any &= m_any - 1;
            const int k = word * 32 + j;
            uint32_t users = 0;
#pragma unroll
            for (int s = 0; s < kMaxSub; ++s) users |= ((m[s] >> j) & 1u) << s;
            const int last_user = 31 - __clz(users);
            for (int kb = 0; kb < p.k_blocks && ok; ++kb) {
              bool first_of_w = true;
#pragma unroll
              for (int s = 0; s < kMaxSub; ++s) {
                if (!((users >> s) & 1u) || !ok) continue;
                uint32_t flags = (uint32_t)s;
                if (kb == 0 && !((touched >> s) & 1u)) flags |= 4u;
                if (first_of_w) flags |= 8u;
                if (s == last_user) flags |= 16u;
                emit(map.tmap + ((tile0 + s) * map.K + k) * (int64_t)kTileM, k, kb, flags, first_of_w);
                first_of_w = false;
              }
            }
            touched |= users;
          }
        }
        // sub tiles that exist but never got a neighbour still have to write zeros
        for (int s = 0; s < p.sub && ok; ++s) {
          if (tile0 + s < n_tiles && !((touched >> s) & 1u)) emit(nullptr, 0, 0, (uint32_t)s | 4u | 8u | 16u, true);
        }
        if (ok) emit(nullptr, 0, 0, 32u, false);                       // end of super tile
      }
      if (cur.valid && ok) run(cur, cur_lo, cur_hi);
    } else if (group == 0) {
      for (int64_t st_i = blockIdx.x; st_i < p.n_super && ok; st_i += gridDim.x) {
        const int64_t row0 = st_i * p.sub * kTileM + t;          // this thread's position in sub tile 0
        typename Map::RowState rs[kMaxSub];
        int64_t arow[kMaxSub];                                    // the rows these positions stand for
        bool row_ok[kMaxSub];
  #pragma unroll
        for (int s = 0; s < kMaxSub; ++s) {
          const int64_t pos = row0 + (int64_t)s * kTileM;
          row_ok[s] = s < p.sub && pos < p.n_rows;
          arow[s] = (row_ok[s] && p.order) ? (int64_t)__ldg(p.order + pos) : pos;
          rs[s] = map.row_state(arow[s], row_ok[s]);
        }
        uint32_t touched = 0;                                     // sub tiles whose accumulator has been started
        for (int k0 = 0; k0 < p.K && ok; k0 += kGroup) {
          const long long cpf = PROF_CLOCK();
          const int kn = min(kGroup, p.K - k0);
          uint32_t mine[kMaxSub];
          int32_t got[kMaxSub][kGroup];
  #pragma unroll
          for (int s = 0; s < kMaxSub; ++s) {
  #pragma unroll
            for (int j = 0; j < kGroup; ++j)
              got[s][j] = (row_ok[s] && j < kn && !ST_DBG(p, 32)) ? map.get(rs[s], arow[s], k0 + j) : -1;
          }
          // every stage of the previous group has been issued by every producer thread: the tile can be rewritten
          producer_sync();
  #pragma unroll
          for (int s = 0; s < kMaxSub; ++s) {
            mine[s] = 0;
  #pragma unroll
            for (int j = 0; j < kGroup; ++j) {
              int32_t i = got[s][j];
              if (i >= p.n_src) i = -1;
              idx_tile[(j * kMaxSub + s) * kTileM + t] = i;
              if (i >= 0) mine[s] |= 1u << j;
            }
          }
  #pragma unroll
          for (int s = 0; s < kMaxSub; ++s) {
            const uint32_t wm = __reduce_or_sync(0xFFFFFFFFu, mine[s]);
            if (lane == 0) ctl->group_mask[pwarp][s] = wm;
          }
          producer_sync();
          uint32_t m[kMaxSub], m_any = 0;
  #pragma unroll
          for (int s = 0; s < kMaxSub; ++s) {
            m[s] = ctl->group_mask[0][s] | ctl->group_mask[1][s] | ctl->group_mask[2][s] | ctl->group_mask[3][s];
            m_any |= m[s];
          }
          t_pref += PROF_CLOCK() - cpf;
          while (m_any && ok) {
            const int j = __ffs(m_any) - 1;
            m_any &= m_any - 1;
            uint32_t users = 0;                                   // sub tiles that need this offset
  #pragma unroll
            for (int s = 0; s < kMaxSub; ++s) users |= ((m[s] >> j) & 1u) << s;
            const int last_user = 31 - __clz(users);
            for (int kb = 0; kb < p.k_blocks && ok; ++kb) {
              send_w(k0 + j, kb);
              bool first_of_w = true;
  #pragma unroll
              for (int s = 0; s < kMaxSub; ++s) {
                if (!((users >> s) & 1u) || !ok) continue;
                uint32_t flags = (uint32_t)s;
                if (kb == 0 && !((touched >> s) & 1u)) flags |= 4u;
                if (first_of_w) flags |= 8u;
                if (s == last_user) flags |= 16u;
                send_a(kb, idx_tile + (j * kMaxSub + s) * kTileM, flags);
                first_of_w = false;
              }
            }
            touched |= users;
          }
        }
        // sub tiles that exist but never got a neighbour still have to write zeros
        for (int s = 0; s < p.sub && ok; ++s) {
          const bool exists = (st_i * p.sub + s) * (int64_t)kTileM < p.n_rows;
          if (exists && !((touched >> s) & 1u)) {
            send_w(0, 0);
            if (ok) send_a(0, nullptr, (uint32_t)s | 4u | 8u | 16u);
          }
        }
        if (ok) {                                                   // end of super tile
          send_a(0, nullptr, 32u);
        }
        queue.flush(lane);                                          // let the epilogue of this super tile start
      }
    }
    queue.flush(lane);
    if (ST_DBG(p, 256) && t == 0 && group == 0) {
      long long* o = g_prof + (size_t)blockIdx.x * 16;
      o[0] = PROF_CLOCK() - t_total0; o[1] = t_pref; o[2] = t_acq_a; o[3] = t_acq_w; o[4] = n_flush; o[5] = t_push; o[6] = t_copy; o[7] = t_w; o[15] = t_idx;
    }
  } else if (warp == kMmaWarp) {
    // =============================================================== MMA issuer
    if (lane == 0) {
      int a_stage = 0, w_slot = 0;
      uint32_t a_phase = 0, w_phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      const uint32_t b_kstep16 = (p.b_mn_major ? (32 / ESIZE) * 128 : 32) >> 4;   // K-step advance, 16-byte units
      const uint32_t b_lbo = p.b_mn_major ? (uint32_t)(128 / ESIZE) * 128u : 16u;
      const bool b_base32 = p.b_mn_major && ESIZE == 4;
      // descriptors without their 14-bit start address (the address stays below 2^18, so a plain OR works)
      const uint64_t a_desc_hi = smem_desc(0u, 16u, 1024u, 2u);
      const uint64_t b_desc_hi = smem_desc(0u, b_lbo, b_base32 ? 512u : 1024u, b_base32 ? 1u : 2u);
      const uint32_t idesc = p.idesc;
      uint32_t w_lo = 0;
      long long m_acc = 0, m_a = 0, m_w = 0, m_t0 = PROF_CLOCK(), m_n = 0, m_issue = 0, m_commit = 0;
      for (int64_t st_i = blockIdx.x; st_i < p.n_super && ok; st_i += gridDim.x) {
        long long c0 = PROF_CLOCK();
        ok = mbar_wait(smem_u32(&ctl->acc_empty[buf]), acc_phase[buf] ^ 1u, abort_flag, 23);
        m_acc += PROF_CLOCK() - c0;
        if (!ok) break;
        tc_fence_after();
        for (;;) {
          c0 = PROF_CLOCK();
          ok = mbar_wait(smem_u32(&ctl->a_full[a_stage]), a_phase, abort_flag, 24);
          m_a += PROF_CLOCK() - c0;
          ++m_n;
          if (!ok) break;
          const uint32_t info = ctl->a_info[a_stage];
          if (info & 8u) {                                      // this stage starts a new W slice
            c0 = PROF_CLOCK();
            ok = mbar_wait(smem_u32(&ctl->w_full[w_slot]), w_phase, abort_flag, 25);
            m_w += PROF_CLOCK() - c0;
            if (!ok) break;
            w_lo = (w_ring + (uint32_t)w_slot * p.w_slot_bytes) >> 4;
          }
          tc_fence_after();
          const long long ci0 = PROF_CLOCK();
          const int ksteps = ST_DBG(p, 2) ? 0 : (int)(info >> 8);
          const uint32_t a_lo = (a_ring + (uint32_t)a_stage * kABlockBytes) >> 4;
          const uint32_t d_addr = tmem_base + (uint32_t)(buf * set_cols + (int)(info & 3u) * p.c_acc);
          const uint32_t fresh = (info & 4u) ? 0u : 1u;          // 0: the first MMA overwrites the accumulator
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            if (ks < ksteps) {
              const uint64_t da = a_desc_hi | (uint64_t)(a_lo + ks * 2);
              const uint64_t db = b_desc_hi | (uint64_t)(w_lo + ks * b_kstep16);
              if (ESIZE == 2)
                mma_f16(d_addr, da, db, idesc, ks == 0 ? fresh : 1u);
              else
                mma_tf32(d_addr, da, db, idesc, ks == 0 ? fresh : 1u);
            }
          }
          const long long ci1 = PROF_CLOCK();
          if (ST_DBG(p, 512)) mbar_arrive(smem_u32(&ctl->a_empty[a_stage])); else
          mma_commit(smem_u32(&ctl->a_empty[a_stage]));
          if (++a_stage == p.a_stages) {
            a_stage = 0;
            a_phase ^= 1u;
          }
          if (info & 16u) {                                     // last user of the W slice
            if (ST_DBG(p, 512)) mbar_arrive(smem_u32(&ctl->w_empty[w_slot])); else
            mma_commit(smem_u32(&ctl->w_empty[w_slot]));
            if (++w_slot == p.w_slots) {
              w_slot = 0;
              w_phase ^= 1u;
            }
          }
          m_issue += ci1 - ci0;
          m_commit += PROF_CLOCK() - ci1;
          if (info & 32u) break;
        }
        if (!ok) break;
        mma_commit(smem_u32(&ctl->acc_full[buf]));
        acc_phase[buf] ^= 1u;
        if (p.acc_bufs == 2) buf ^= 1;
      }
      if (ST_DBG(p, 256)) {
        long long* o = g_prof + (size_t)blockIdx.x * 16;
        o[8] = PROF_CLOCK() - m_t0; o[9] = m_acc; o[10] = m_a; o[11] = m_w; o[12] = m_n; o[13] = m_issue; o[14] = m_commit;
      }
    }
    __syncwarp();
  } else {
    // =============================================================== epilogue (warps 0..3)
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    bool ok = true;
    const int out_es = p.out_kind == ST_F32 ? 4 : 2;
    for (int64_t st_i = blockIdx.x; st_i < p.n_super && ok; st_i += gridDim.x) {
      // where this lane's rows go: known before the accumulators are ready, so fetched before the wait
      int64_t dst_rows[kMaxSub];
#pragma unroll
      for (int s = 0; s < kMaxSub; ++s) {
        const int64_t row = (st_i * p.sub + s) * (int64_t)kTileM + warp * 32 + lane;
        dst_rows[s] = (s < p.sub && p.order && row < p.n_rows) ? (int64_t)__ldg(p.order + row) : row;
      }
      ok = mbar_wait(smem_u32(&ctl->acc_full[buf]), acc_phase[buf], abort_flag, 26, 256);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int s = 0; s < kMaxSub; ++s) {
        if (s >= p.sub) break;
        const int64_t row = (st_i * p.sub + s) * (int64_t)kTileM + warp * 32 + lane;
        if ((st_i * p.sub + s) * (int64_t)kTileM >= p.n_rows) break;         // whole sub tile past the end
        const int64_t dst_row = dst_rows[s];
        char* out_row = static_cast<char*>(p.out) + (size_t)dst_row * p.c_acc * out_es;
        const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * set_cols + s * p.c_acc);
        for (int c0 = 0; c0 < p.c_acc && !ST_DBG(p, 128); c0 += 32) {
          uint32_t v[32];
          if (p.c_acc - c0 >= 32) {
            tmem_ld32(t_row + c0, v);
            tmem_ld_wait();
            if (row < p.n_rows && !ST_DBG(p, 64)) store_cols<32>(out_row, c0, p.out_kind, v);
          } else {
            tmem_ld16(t_row + c0, v);
            tmem_ld_wait();
            if (row < p.n_rows) store_cols<16>(out_row, c0, p.out_kind, v);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->acc_empty[buf]));
      acc_phase[buf] ^= 1u;
      if (p.acc_bufs == 2) buf ^= 1;
    }
  }

  // After an expired wait, bulk copies of this CTA may still be in flight: give them time to land
  // before the CTA's shared memory and mbarriers go away (they complete within microseconds).
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// =================================================================================================
// Weight gradient on the tensor cores.
//
//   dW[k][ci][co] = sum_r  X[map(r,k)][ci] * dY[r][co]
//
// The reduction runs over rows, so both operands enter the MMA "MN-major" (channels contiguous,
// one 128-byte line per row): A = dY tile (M = 128 output channels), B = gathered X rows
// (N = up to 128 input channels), K = the 128 rows of a tile.  A CTA owns a chunk of row tiles, a
// group of G kernel offsets (G accumulators of N columns fill TMEM), one 128-wide block of output
// channels and one block of input channels; it keeps its G accumulators in TMEM across all of its
// tiles and finally writes them as fp32 partials  partial[chunk][k][ci][co]  that a second kernel
// sums in chunk order ("split by offset", deterministic).  The dY tile is loaded once per tile and
// reused by every offset of the group.
// =================================================================================================
constexpr int kWgradBSlotsMax = 6;

struct WgradParams {
  const void* x;         // (n_src, cin)
  const void* dy;        // (n_rows, cout)
  const int32_t* order;  // optional: tile row r stands for row order[r] of the map and of dY
  float* partial;        // (n_chunks, K, cin, cout)
  int64_t n_rows, n_src, n_tiles, tiles_per_chunk;
  int K, cin, cout, esize;
  int group;             // offsets per CTA (accumulators in TMEM)
  int n_kgroups;
  int ci_blk;            // input channels per CTA (MMA N)
  int n_ciblk, n_coblk;
  int a_slot_bytes, b_slot_bytes, b_slots;
  int quad;              // planned_wgrad_kernel: offsets per shared-memory slot (b_slots counts such slots)
  int a_slots;           // planned_wgrad_kernel: depth of the tile-operand ring
  int swap;              // planned_wgrad_kernel: 1 = the plan is the INVERSE map's (tile operand X, gathered operand dY)
  int dense_tiles;       // planned_wgrad_kernel: 1 = the tile operand's rows lie in tile order (a copy permuted by `order`,
                         // or no `order` at all): a tile is one 2-D box per column block instead of 32 row gathers
  int tmem_cols;
  uint32_t idesc_base;   // everything but N
};

struct __align__(8) WgradControl {
  unsigned long long a_full[2], a_empty[2];
  unsigned long long b_full[kWgradBSlotsMax], b_empty[kWgradBSlotsMax];
  unsigned long long acc_full;
  uint32_t b_info[kWgradBSlotsMax];    // bits 0-7 accumulator index, bit 8 end-of-tile marker
  uint32_t group_mask[kProducerWarps];
  uint32_t touched;                    // accumulators that received at least one MMA
  uint32_t tmem_base;
  int abort_flag;
};

template <typename Map>
__global__ void __launch_bounds__(kThreads, 1) wgrad_kernel(const WgradParams p, const Map map) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - raw);
  const uint32_t a_ring = base;
  const uint32_t b_ring = base + 2u * (uint32_t)p.a_slot_bytes;
  WgradControl* ctl =
      reinterpret_cast<WgradControl*>(base_ptr + 2 * (size_t)p.a_slot_bytes + (size_t)p.b_slots * p.b_slot_bytes);
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work item of this CTA
  const int chunk = blockIdx.x;
  const int kgroup = blockIdx.y;
  const int coblk = blockIdx.z / p.n_ciblk, ciblk = blockIdx.z % p.n_ciblk;
  const int k_first = kgroup * p.group;
  const int g_count = min(p.group, p.K - k_first);
  const int co0 = coblk * 128, co_cnt = min(128, p.cout - co0);
  const int ci0 = ciblk * p.ci_blk, ci_cnt = min(p.ci_blk, p.cin - ci0);
  const int64_t tile_begin = (int64_t)chunk * p.tiles_per_chunk;
  const int64_t tile_end = min(p.n_tiles, tile_begin + p.tiles_per_chunk);

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctl->a_full[s]), kProducerThreads);
      mbar_init(smem_u32(&ctl->a_empty[s]), 1);
    }
    for (int s = 0; s < p.b_slots; ++s) {
      mbar_init(smem_u32(&ctl->b_full[s]), kProducerThreads + 1);
      mbar_init(smem_u32(&ctl->b_empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->acc_full), 2);
    ctl->abort_flag = 0;
    ctl->touched = 0;
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
  const bool base32 = p.esize == 4;                 // 32-bit elements: 128-byte swizzle with 32-byte atoms

  if (warp >= kFirstProducerWarp) {
    // =============================================================== producers
    const int t = threadIdx.x - kFirstProducerWarp * 32;
    const int pwarp = t >> 5;
    int a_slot = 0, b_slot = 0;
    uint32_t a_phase = 0, b_phase = 0;
    bool ok = true;
    const int x_row_bytes = p.cin * p.esize, dy_row_bytes = p.cout * p.esize;
    const int a_bytes = co_cnt * p.esize, b_bytes = ci_cnt * p.esize;      // bytes of this CTA's channel blocks

    // Copy `bytes` of one row into the 128-byte-line blocks of a slot (line t of every block).
    // (Letting eight lanes share a row, so that a warp-wide cp.async touches whole lines, was measured
    // slower here: the producers are bound by instruction issue and the row exchange costs shuffles.)
    auto copy_row = [&](uint32_t slot_base, const char* src, int bytes, bool valid) {
      const int n_chunks = bytes >> 4;
      for (int c = 0; c < n_chunks; ++c) {
        const int blk = c >> 3, cc = c & 7;
        const uint32_t dst = slot_base + (uint32_t)(blk * kABlockBytes + t * 128 + ((base32 ? swz32(cc, t) : swz16(cc, t)) << 4));
        cp_async16(dst, valid ? src + c * 16 : static_cast<const char*>(p.dy), valid ? 16u : 0u);
      }
    };
    auto send_b = [&](int acc, bool marker, bool has, int32_t src_row) {
      ok = mbar_wait(smem_u32(&ctl->b_empty[b_slot]), b_phase ^ 1u, abort_flag, 11);
      if (!ok) return;
      if (!marker)
        copy_row(b_ring + (uint32_t)b_slot * p.b_slot_bytes,
                 static_cast<const char*>(p.x) + (size_t)(has ? src_row : 0) * x_row_bytes + (size_t)ci0 * p.esize,
                 b_bytes, has);
      cp_async_arrive_noinc(smem_u32(&ctl->b_full[b_slot]));
      if (t == 0) {
        ctl->b_info[b_slot] = (uint32_t)acc | (marker ? 0x100u : 0u);
        mbar_arrive(smem_u32(&ctl->b_full[b_slot]));
      }
      if (++b_slot == p.b_slots) {
        b_slot = 0;
        b_phase ^= 1u;
      }
    };

    if constexpr (Map::kPlanned) {
      // stored map in tile-plan form: the tile's mask says which offsets to visit, a step's source rows
      // are one coalesced line; no barrier among the producer warps
      const int word = k_first >> 5, shift = k_first & 31;
      const uint32_t group_bits = g_count >= 32 ? 0xFFFFFFFFu : ((1u << g_count) - 1u);
      for (int64_t tile = tile_begin; tile < tile_end && ok; ++tile) {
        uint32_t m = (__ldg(map.tmask + tile * map.MW + word) >> shift) & group_bits;
        if (!m) continue;
        const int64_t pos = tile * kTileM + t;
        const bool row_ok = pos < p.n_rows;
        const int64_t row = (row_ok && p.order) ? (int64_t)__ldg(p.order + pos) : pos;
        int32_t idx[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          idx[j] = ((m >> j) & 1u) ? __ldg(map.tmap + ((tile * map.K + k_first + j) * (int64_t)kTileM + t)) : -1;
        ok = mbar_wait(smem_u32(&ctl->a_empty[a_slot]), a_phase ^ 1u, abort_flag, 10);
        if (!ok) break;
        copy_row(a_ring + (uint32_t)a_slot * p.a_slot_bytes,
                 static_cast<const char*>(p.dy) + (size_t)(row_ok ? row : 0) * dy_row_bytes + (size_t)co0 * p.esize,
                 a_bytes, row_ok);
        cp_async_arrive_noinc(smem_u32(&ctl->a_full[a_slot]));
        if (++a_slot == 2) {
          a_slot = 0;
          a_phase ^= 1u;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (((m >> j) & 1u) && ok) send_b(j, false, (uint32_t)idx[j] < (uint32_t)p.n_src, idx[j]);
        }
        if (ok) send_b(0, true, false, 0);                     // end of tile: lets the MMA warp free the dY slot
      }
    } else {
      for (int64_t tile = tile_begin; tile < tile_end && ok; ++tile) {
        const int64_t pos = tile * kTileM + t;
        const bool row_ok = pos < p.n_rows;
        const int64_t row = (row_ok && p.order) ? (int64_t)__ldg(p.order + pos) : pos;
        typename Map::RowState rs = map.row_state(row, row_ok);
        // neighbours of this row for the offsets of the group (independent loads, then a bit mask)
        int32_t idx[32];
        uint32_t mine = 0;
  #pragma unroll
        for (int j = 0; j < 32; ++j) {
          int32_t i = (j < g_count && row_ok) ? map.get(rs, row, k_first + j) : -1;
          if (i >= p.n_src) i = -1;
          idx[j] = i;
          if (i >= 0) mine |= 1u << j;
        }
        const uint32_t warp_mask = __reduce_or_sync(0xFFFFFFFFu, mine);
        producer_bar_sync<kProducerThreads>();
        if (lane == 0) ctl->group_mask[pwarp] = warp_mask;
        producer_bar_sync<kProducerThreads>();
        uint32_t m = ctl->group_mask[0] | ctl->group_mask[1] | ctl->group_mask[2] | ctl->group_mask[3];
        if (m) {
          // dY tile: once per tile, shared by all offsets of the group
          ok = mbar_wait(smem_u32(&ctl->a_empty[a_slot]), a_phase ^ 1u, abort_flag, 10);
          if (!ok) break;
          copy_row(a_ring + (uint32_t)a_slot * p.a_slot_bytes,
                   static_cast<const char*>(p.dy) + (size_t)(row_ok ? row : 0) * dy_row_bytes + (size_t)co0 * p.esize,
                   a_bytes, row_ok);
          cp_async_arrive_noinc(smem_u32(&ctl->a_full[a_slot]));
          if (++a_slot == 2) {
            a_slot = 0;
            a_phase ^= 1u;
          }
          while (m && ok) {
            const int j = __ffs(m) - 1;
            m &= m - 1;
            send_b(j, false, (mine >> j) & 1u, idx[j]);
          }
          if (ok) send_b(0, true, false, 0);                   // end of tile: lets the MMA warp free the dY slot
        }
      }
    }
    if (ok) send_b(0xFF, true, false, 0);                     // end of work
    cp_async_wait_all();
  } else if (warp == kMmaWarp) {
    // =============================================================== MMA issuer
    if (lane == 0) {
      int a_slot = 0, b_slot = 0;
      uint32_t a_phase = 0, b_phase = 0;
      uint32_t touched = 0;
      bool ok = true, have_a = false;
      const int rows_per_step = 32 / p.esize;                  // reduction rows per MMA (16 or 8)
      const int ksteps = kTileM / rows_per_step;
      const uint32_t step_bytes = (uint32_t)rows_per_step * 128u;
      const uint32_t sbo = base32 ? 512u : 1024u, layout = base32 ? 1u : 2u;
      const uint32_t idesc = p.idesc_base | ((uint32_t)(p.ci_blk >> 3) << 17);
      for (;;) {
        ok = mbar_wait(smem_u32(&ctl->b_full[b_slot]), b_phase, abort_flag, 12);
        if (!ok) break;
        const uint32_t info = ctl->b_info[b_slot];
        const bool marker = (info & 0x100u) != 0;
        const int acc = (int)(info & 0xFFu);
        if (!marker) {
          if (!have_a) {
            ok = mbar_wait(smem_u32(&ctl->a_full[a_slot]), a_phase, abort_flag, 13);
            if (!ok) break;
            have_a = true;
          }
          fence_proxy_async();
          tc_fence_after();
          const uint32_t a_base = a_ring + (uint32_t)a_slot * p.a_slot_bytes;
          const uint32_t b_base = b_ring + (uint32_t)b_slot * p.b_slot_bytes;
          const uint32_t d_addr = tmem_base + (uint32_t)(acc * p.ci_blk);
          for (int ks = 0; ks < ksteps; ++ks) {
            const uint64_t da = smem_desc(a_base + ks * step_bytes, kABlockBytes, sbo, layout);
            const uint64_t db = smem_desc(b_base + ks * step_bytes, kABlockBytes, sbo, layout);
            const uint32_t accumulate = (((touched >> acc) & 1u) || ks > 0) ? 1u : 0u;
            if (p.esize == 2)
              mma_f16(d_addr, da, db, idesc, accumulate);
            else
              mma_tf32(d_addr, da, db, idesc, accumulate);
          }
          touched |= 1u << acc;
        }
        mma_commit(smem_u32(&ctl->b_empty[b_slot]));
        if (++b_slot == p.b_slots) {
          b_slot = 0;
          b_phase ^= 1u;
        }
        if (marker) {
          if (acc == 0xFF) break;                               // end of work
          if (have_a) {                                         // end of tile: the dY slot may be refilled
            mma_commit(smem_u32(&ctl->a_empty[a_slot]));
            if (++a_slot == 2) {
              a_slot = 0;
              a_phase ^= 1u;
            }
            have_a = false;
          }
        }
      }
      if (ok) {
        ctl->touched = touched;
        mma_commit(smem_u32(&ctl->acc_full));
        mbar_arrive(smem_u32(&ctl->acc_full));
      }
    }
    __syncwarp();
  } else {
    // =============================================================== epilogue (warps 0..3)
    bool ok = mbar_wait(smem_u32(&ctl->acc_full), 0u, abort_flag, 14, 512);
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (ok) {
      tc_fence_after();
      const uint32_t touched = ctl->touched;
      const int co = warp * 32 + lane;                           // accumulator row = output channel
      for (int j = 0; j < g_count; ++j) {
        float* dst = p.partial + (((size_t)chunk * p.K + (k_first + j)) * p.cin + ci0) * p.cout + co0 + co;
        const bool live = (touched >> j) & 1u;
        for (int c0 = 0; c0 < ci_cnt; c0 += 16) {
          uint32_t v[32];
          tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(j * p.ci_blk + c0), v);
          tmem_ld_wait();
          if (co < co_cnt) {
#pragma unroll
            for (int c = 0; c < 16; ++c) dst[(size_t)(c0 + c) * p.cout] = live ? __uint_as_float(v[c]) : 0.f;
          }
        }
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

}  // namespace tc

}  // namespace st

#include "conv_tc_plan.cuh"

namespace st {

// Per-device state: the SM count and whether a kernel's dynamic shared memory limit has been raised are
// properties of the device the launch goes to, so both are remembered by device ordinal.
constexpr int kMaxDevices = 64;

static int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

static int sm_count() {
  static int count[kMaxDevices] = {0};
  const int dev = current_device();
  if (count[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    count[dev] = n > 0 ? n : 148;
  }
  return count[dev];
}

static bool g_tc_enabled = true;

void tc_set_enabled(bool on) { g_tc_enabled = on; }

// Whether the planned products may use the TMA-fed kernels (else their cp.async forms over the same plan).
static bool g_tma_enabled = true;

void tc_set_tma(bool on) { g_tma_enabled = on; }

static bool g_dense_tiles = true;
void tc_set_dense_tiles(bool on) { g_dense_tiles = on; }

bool tc_supported(int dtype, int c_red, int c_acc) {
  if (!g_tc_enabled) return false;
  if (dtype != ST_F32 && dtype != ST_F16 && dtype != ST_BF16) return false;
  const int es = dtype == ST_F32 ? 4 : 2;
  const int kstep = 32 / es;                       // reduction elements per MMA
  if (c_red < kstep || c_red % kstep != 0 || c_red > 512) return false;
  if (c_acc < 16 || c_acc % 16 != 0 || c_acc > 256) return false;
  return true;
}

static bool fill_params2(tc::Params2* p, int dtype, const void* in, const void* w, void* out, int64_t n_rows,
                         int64_t n_src, int K, int c_red, int c_acc, bool w_transposed, bool planned = false) {
  const int es = dtype == ST_F32 ? 4 : 2;
  p->in = in;
  p->w = w;
  p->out = out;
  p->order = nullptr;
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
  int w_bytes = p->b_mn_major ? ((c_acc * es + 127) / 128) * (128 / es) * 128 : c_acc * 128;
  p->w_slot_bytes = (w_bytes + 1023) / 1024 * 1024;
  // accumulators: as many row tiles per W copy as TMEM allows (<= 4); a second set only when it is free
  int sub = 512 / c_acc;
  if (sub > tc::kMaxSub) sub = tc::kMaxSub;
#ifdef ST_TC_PROFILE
  {
    // experiment: prefer two accumulator sets (epilogue overlaps the next super tile) over sharing W
    const char* e = getenv("ST_TC_ACC2");
    if (e && atoi(e) && sub >= 2 && 2 * sub * c_acc > 512) sub /= 2;
  }
#endif
  p->acc_bufs = (2 * sub * c_acc <= 512) ? 2 : 1;
  const int64_t n_tiles = (n_rows + tc::kTileM - 1) / tc::kTileM;
  // small problems: do not leave SMs idle for the sake of sharing
  while (sub > 1 && (n_tiles + sub - 1) / sub < sm_count()) --sub;
  p->sub = sub;
  p->n_super = (n_tiles + sub - 1) / sub;
  int cols = 32;
  while (cols < p->acc_bufs * sub * c_acc) cols <<= 1;
  p->tmem_cols = cols;
  p->w_slots = 3;
  p->idx_bytes = planned ? 0 : tc::kIdxTileBytes;
  p->n_slots = 0;
  p->slot_bytes = 0;
  p->part = 1;
  p->w_flip = 0;
  const int budget = 222 * 1024 - p->idx_bytes;
  int a_stages = (budget - p->w_slots * p->w_slot_bytes) / tc::kABlockBytes;
  if (a_stages > tc::kMaxAStages) a_stages = tc::kMaxAStages;
  if (a_stages < 4) {
    p->w_slots = 2;
    a_stages = (budget - p->w_slots * p->w_slot_bytes) / tc::kABlockBytes;
    if (a_stages > tc::kMaxAStages) a_stages = tc::kMaxAStages;
  }
  if (a_stages < (planned ? tc::kProducerWarps : 2)) return false;
  // slot ownership by index needs whole rounds: of the four TMA-issuing warps or of the cp.async groups
  a_stages -= a_stages % (planned ? tc::kProducerWarps : tc::kGatherGroups);
  p->a_stages = a_stages;
  const uint32_t fmt = dtype == ST_F16 ? 0u : (dtype == ST_BF16 ? 1u : 2u);
  p->idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)p->b_mn_major << 16) | ((uint32_t)(c_acc >> 3) << 17) |
             ((uint32_t)(tc::kTileM >> 4) << 24);
  p->out_kind = dtype;
  p->dbg = 0;
#ifdef ST_TC_PROFILE
  {
    // timing experiments of instrumented builds only (see Params2::dbg)
    const char* e = getenv("ST_TC_DEBUG");
    p->dbg = e ? atoi(e) : 0;
    const char* g = getenv("ST_TC_ASTAGES");
    if (g && atoi(g) >= 4 && atoi(g) <= p->a_stages) p->a_stages = atoi(g) / 4 * 4;
    const char* f = getenv("ST_TC_SUB");
    if (f && atoi(f) >= 1 && atoi(f) <= sub) {
      p->sub = atoi(f);
      p->n_super = (n_tiles + p->sub - 1) / p->sub;
    }
  }
#endif
  return true;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  // The encoder is a driver call and wants the device's context current on the calling thread.  A thread that has
  // made no runtime call that binds it yet (an autograd worker on its first backward node) would get an error from
  // the encoder and the caller would quietly take the cp.async kernels for that one call: bind it here.
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    cudaGetLastError();
  }
  return fn;
}

// Descriptor of a row-major (rows, cols) matrix for tile::gather4: box = one 128-byte line, 128-byte swizzle.
static bool make_gather_desc(CUtensorMap* desc, const void* base, int64_t rows, int cols, int esize, int dtype,
                             bool atom32 = false) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || !base || rows < 1 || (reinterpret_cast<uintptr_t>(base) & 15) || (cols * esize) % 16) return false;
  const CUtensorMapDataType dt = dtype == ST_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == ST_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                   : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * esize};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / esize), 1};
  const cuuint32_t estride[2] = {1, 1};
  return fn(desc, dt, 2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
            atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Descriptor of the weights seen as a (K * w_rows, w_cols) matrix; the box is one 128-byte column block
// of a W[k] slice: `box_rows` rows.  `atom32` selects the 128-byte swizzle with 32-byte atoms (MN-major
// operands of 32-bit elements), else the plain 128-byte swizzle.
static bool make_weight_desc(CUtensorMap* desc, const void* base, int64_t rows, int cols, int esize, int dtype,
                             int box_rows, bool atom32) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || !base || rows < 1 || box_rows < 1 || box_rows > 256 || (reinterpret_cast<uintptr_t>(base) & 15) ||
      (cols * esize) % 16)
    return false;
  const CUtensorMapDataType dt = dtype == ST_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == ST_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                   : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * esize};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)box_rows};
  const cuuint32_t estride[2] = {1, 1};
  return fn(desc, dt, 2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
            atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename Map>
static int launch_gather(tc::Params2 p, const Map& map, cudaStream_t stream) {
  const size_t smem = (size_t)p.w_slots * p.w_slot_bytes + (size_t)p.a_stages * tc::kABlockBytes +
                      p.idx_bytes + sizeof(tc::Control2) + 1024;
  auto kernel = p.esize == 2 ? tc::gather2_kernel<Map, 2> : tc::gather2_kernel<Map, 4>;
  static bool configured[2][kMaxDevices] = {};             // per element size and device (one set per Map instantiation)
  if (!configured[p.esize == 4][current_device()]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      set_error("tc gather: cannot raise the dynamic shared memory limit: %s", cudaGetErrorString(e));
      return ST_ERR_CUDA;
    }
    configured[p.esize == 4][current_device()] = true;
  }
  int64_t grid = p.n_super < sm_count() ? p.n_super : sm_count();
  kernel<<<(unsigned)grid, tc::kGatherThreads, smem, stream>>>(p, map);
  note_launches(1);
  return check_launch("tc gather");
}

// A stored map in tile-plan form: the TMA-fed kernel when the tensors can be described to the copy
// engine (16-byte aligned bases and row pitches) and two whole-offset slots fit in shared memory,
// else the cp.async producers of gather2_kernel over the same plan.
static int launch_planned(tc::Params2 p, const tc::PlannedRows& map, cudaStream_t stream) {
  CUtensorMap in_desc, w_desc;
  memset(&in_desc, 0, sizeof(in_desc));
  memset(&w_desc, 0, sizeof(w_desc));
  // Two CTAs per SM (experiment switch of instrumented builds): super tiles of at most two row tiles whose
  // accumulators take at most half of TMEM, rings cut to half of the shared memory, twice the CTAs.  Measured
  // slower on every layer tried (64 -> 128 k3 s2 forward 0.33 -> 0.47 ms, dgrad 0.25 -> 0.44 ms; submanifold
  // 32..256 channels 1.5-1.8x slower): what bounds these kernels is the copy engine's rate of row gathers per SM,
  // which two half-size pipelines share, while each W slice is then fetched for two row tiles instead of four.
  int smem_budget = 222 * 1024;
  int ctas_per_sm = 1;
#ifdef ST_TC_PROFILE
  {
    const char* e = getenv("ST_TC_HALF");
    if (e && atoi(e)) {
      const int64_t n_tiles = (p.n_rows + tc::kTileM - 1) / tc::kTileM;
      int sub = p.sub < 2 ? p.sub : 2;
      while (sub > 1 && sub * p.c_acc > 256) --sub;
      if (sub * p.c_acc <= 256) {
        p.sub = sub;
        p.n_super = (n_tiles + sub - 1) / sub;
        p.acc_bufs = (2 * sub * p.c_acc <= 256) ? 2 : 1;
        int cols = 32;
        while (cols < p.acc_bufs * sub * p.c_acc) cols <<= 1;
        p.tmem_cols = cols;
        smem_budget = 110 * 1024;
        ctas_per_sm = 2;
      }
    }
  }
#endif
  p.part = p.sub;                        // smaller parts (more slots in flight) were measured slower
#ifdef ST_TC_PROFILE
  {
    const char* e = getenv("ST_TC_PART");
    if (e && atoi(e) >= 1 && atoi(e) <= p.sub) p.part = atoi(e);
  }
#endif
  int n_slots = 0;
  for (;;) {
    p.slot_bytes = p.w_slot_bytes + p.part * tc::kABlockBytes;
    n_slots = (int)((smem_budget - (int)sizeof(tc::Control3)) / p.slot_bytes);
    if (n_slots > tc::kMaxSlots3) n_slots = tc::kMaxSlots3;
    // the slot that carries an offset's W slice is held until the offset's last item: the ring must
    // have room for all of an offset's items
    if (n_slots >= (p.sub + p.part - 1) / p.part || p.part >= p.sub) break;
    ++p.part;
  }
  p.n_slots = n_slots;
  const bool tma = g_tma_enabled && n_slots >= 2 && p.n_src > 0 &&
                   make_gather_desc(&in_desc, p.in, p.n_src, p.c_red, p.esize, p.out_kind) &&
                   make_weight_desc(&w_desc, p.w, (int64_t)p.K * p.w_rows, p.w_cols, p.esize, p.out_kind,
                                    p.b_mn_major ? 128 / p.esize : p.w_rows, p.b_mn_major && p.esize == 4);
  if (!tma) return launch_gather(p, map, stream);
  const size_t smem = (size_t)p.n_slots * p.slot_bytes + sizeof(tc::Control3) + 1024;
  auto kernel = p.esize == 2 ? tc::planned_gather_kernel<2> : tc::planned_gather_kernel<4>;
  static bool configured[2][kMaxDevices] = {};
  if (!configured[p.esize == 4][current_device()]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      set_error("tc planned gather: cannot raise the dynamic shared memory limit: %s", cudaGetErrorString(e));
      return ST_ERR_CUDA;
    }
    configured[p.esize == 4][current_device()] = true;
  }
  const int64_t max_ctas = (int64_t)ctas_per_sm * sm_count();
  int64_t grid = p.n_super < max_ctas ? p.n_super : max_ctas;
  kernel<<<(unsigned)grid, tc::kThreads, smem, stream>>>(p, map, in_desc, w_desc);
  note_launches(1);
  return check_launch("tc planned gather");
}

int tc_conv_gather(int dtype, const void* in, const void* w, const int32_t* map, const MapPlan& plan, void* out,
                   int64_t n_rows, int64_t n_src, int K, int c_red, int c_acc, bool w_transposed, cudaStream_t stream,
                   bool w_flip) {
  tc::Params2 p;
  const bool planned = plan.tmap && plan.tmask;
  if (!fill_params2(&p, dtype, in, w, out, n_rows, n_src, K, c_red, c_acc, w_transposed, planned)) {
    set_error("tc_conv_gather: shape does not fit shared memory");
    return ST_ERR_UNSUPPORTED;
  }
  if (n_rows == 0) return ST_OK;
  p.order = plan.order;
  p.w_flip = w_flip ? 1 : 0;
  if (planned) return launch_planned(p, tc::PlannedRows{plan.tmap, plan.tmask, K, (K + 31) / 32}, stream);
  return launch_gather(p, tc::StoredRows{map, K}, stream);
}

template <typename CT>
static tc::HashRows<CT> make_hash_rows(const HashFlyArgs& h) {
  tc::HashRows<CT> m;
  m.coords = static_cast<const CT*>(h.coords);
  m.off = *h.offsets;
  m.table = make_table(h.keys, h.vals, h.capacity);
  m.shape = Int3{h.shape[0], h.shape[1], h.shape[2]};
  m.stride = h.stride;
  return m;
}

int tc_conv_gather_hashfly(int dtype, const void* in, const void* w, const HashFlyArgs& h, void* out, int64_t n_rows,
                           int64_t n_src, int K, int c_red, int c_acc, cudaStream_t stream) {
  tc::Params2 p;
  if (!fill_params2(&p, dtype, in, w, out, n_rows, n_src, K, c_red, c_acc, /*w_transposed=*/false)) {
    set_error("tc_conv_gather_hashfly: shape does not fit shared memory");
    return ST_ERR_UNSUPPORTED;
  }
  if (n_rows == 0) return ST_OK;
  if (h.coord_dtype == ST_I32) return launch_gather(p, make_hash_rows<int32_t>(h), stream);
  return launch_gather(p, make_hash_rows<int16_t>(h), stream);
}

// Inverse rule for the feature gradient without a stored map: input row i (table-space coordinate
// q_i) receives from output o = (q_i + off_k) / stride when that division is exact and o exists.
int tc_conv_dgrad_inverse(int dtype, const void* dy, const void* w, const int32_t* q_coords, const Offsets& off,
                          const int64_t* out_keys, const int32_t* out_vals, int64_t out_capacity, int stride, void* dx,
                          int64_t n_in, int64_t n_out, int K, int cin, int cout, cudaStream_t stream) {
  tc::Params2 p;
  if (!fill_params2(&p, dtype, dy, w, dx, n_in, n_out, K, cout, cin, /*w_transposed=*/true)) {
    set_error("tc_conv_dgrad_inverse: shape does not fit shared memory");
    return ST_ERR_UNSUPPORTED;
  }
  if (n_in == 0) return ST_OK;
  tc::InverseRows m;
  m.q = q_coords;
  m.off = off;
  m.table = make_table(out_keys, out_vals, out_capacity);
  m.stride = stride;
  return launch_gather(p, m, stream);
}

// ------------------------------------------------------------------------------------------- wgrad
struct WgradPlan {
  tc::WgradParams p;
  int n_chunks;
  size_t smem;
};

static bool plan_wgrad(WgradPlan* plan, int dtype, int64_t n_rows, int K, int cin, int cout) {
  if (!g_tc_enabled) return false;
  if (dtype != ST_F32 && dtype != ST_F16 && dtype != ST_BF16) return false;
  const int es = dtype == ST_F32 ? 4 : 2;
  if (cin % 16 != 0 || cin < 16 || cout % 8 != 0 || cout < 8 || n_rows <= 0) return false;
  tc::WgradParams& p = plan->p;
  p.esize = es;
  p.K = K;
  p.cin = cin;
  p.cout = cout;
  p.n_rows = n_rows;
  p.n_tiles = (n_rows + tc::kTileM - 1) / tc::kTileM;
  // input-channel block: at most 256 bytes per row (two 128-byte lines), i.e. 128 (16-bit) or 64 (32-bit) channels
  const int ci_max = 256 / es;
  p.n_ciblk = (cin + ci_max - 1) / ci_max;
  p.ci_blk = ((cin + p.n_ciblk - 1) / p.n_ciblk + 15) / 16 * 16;
  p.n_ciblk = (cin + p.ci_blk - 1) / p.ci_blk;
  p.n_coblk = (cout + 127) / 128;
  p.group = 512 / p.ci_blk;
  if (p.group > 32) p.group = 32;
  if (p.group > K) p.group = K;
  p.n_kgroups = (K + p.group - 1) / p.group;
  // (Equal shares, 7 + 7 + 7 + 6 offsets instead of 8 + 8 + 8 + 3, measured slower: every group then loads the
  // dY tile of nearly every row tile, and the kernel is bound by what the copy engine moves, not by the longest CTA.)
  int cols = 32;
  while (cols < p.group * p.ci_blk) cols <<= 1;
  p.tmem_cols = cols;
  p.a_slot_bytes = (128 * es / 128) * tc::kABlockBytes;                 // 128 output channels
  p.b_slot_bytes = ((p.ci_blk * es + 127) / 128) * tc::kABlockBytes;
  int b_slots = (200 * 1024 - 2 * p.a_slot_bytes) / p.b_slot_bytes;
  if (b_slots > tc::kWgradBSlotsMax) b_slots = tc::kWgradBSlotsMax;
  if (b_slots < 2) return false;
  p.b_slots = b_slots;
  const uint32_t fmt = dtype == ST_F16 ? 0u : (dtype == ST_BF16 ? 1u : 2u);
  p.idesc_base = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(tc::kTileM >> 4) << 24);
  const int64_t ctas_per_chunk = (int64_t)p.n_kgroups * p.n_coblk * p.n_ciblk;
  // CTAs per launch.  Two per SM by default; one per SM when a chunk is a single CTA (a second wave would
  // only add partial sums to write and reduce); four per SM when the offsets are split over more than
  // four groups (wide input blocks, four offsets per group): with an odd kernel the group that holds the
  // centre offset then carries about half of all pairs on a small share of the CTAs, and smaller CTAs
  // are what lets the other SMs share that load.  (With four groups or fewer, two per SM measured best.)
  int64_t target = 2 * (int64_t)sm_count();
  if (ctas_per_chunk == 1) target = sm_count();
  else if (p.n_kgroups > 4) target = 4 * (int64_t)sm_count();
  int64_t chunks = (target + ctas_per_chunk - 1) / ctas_per_chunk;
  if (chunks > sm_count()) chunks = sm_count();
#ifdef ST_TC_PROFILE
  {
    const char* e = getenv("ST_TC_WCHUNKS");
    if (e && atoi(e) >= 1) chunks = atoi(e);
  }
#endif
  if (chunks > p.n_tiles) chunks = p.n_tiles;
  if (chunks > 256) chunks = 256;
  if (chunks < 1) chunks = 1;
  p.tiles_per_chunk = (p.n_tiles + chunks - 1) / chunks;
  plan->n_chunks = (int)((p.n_tiles + p.tiles_per_chunk - 1) / p.tiles_per_chunk);
  plan->smem = 2 * (size_t)p.a_slot_bytes + (size_t)p.b_slots * p.b_slot_bytes + sizeof(tc::WgradControl) + 1024;
  return true;
}

bool tc_wgrad_supported(int dtype, int64_t n_rows, int K, int cin, int cout) {
  WgradPlan plan;
  return plan_wgrad(&plan, dtype, n_rows, K, cin, cout);
}

int64_t tc_wgrad_partial_bytes(int dtype, int64_t n_rows, int K, int cin, int cout) {
  WgradPlan plan;
  if (!plan_wgrad(&plan, dtype, n_rows, K, cin, cout)) return 0;
  return (int64_t)plan.n_chunks * K * cin * cout * 4;
}

template <typename Map>
static int launch_wgrad(WgradPlan& plan, const Map& map, cudaStream_t stream) {
  auto kernel = tc::wgrad_kernel<Map>;
  static bool configured[kMaxDevices] = {};               // per device (one set per Map instantiation)
  if (!configured[current_device()]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      set_error("tc wgrad: cannot raise the dynamic shared memory limit: %s", cudaGetErrorString(e));
      return ST_ERR_CUDA;
    }
    configured[current_device()] = true;
  }
  dim3 grid((unsigned)plan.n_chunks, (unsigned)plan.p.n_kgroups, (unsigned)(plan.p.n_coblk * plan.p.n_ciblk));
  kernel<<<grid, tc::kThreads, plan.smem, stream>>>(plan.p, map);
  note_launches(1);
  return check_launch("tc wgrad");
}

// dst[r] = src[order[r]] for rows of `vecs` 16-byte pieces: the tile operand of the weight gradient in the order
// the kernel walks it, so that a tile of 128 rows is a dense box.  Eight pieces per thread, the eight row
// numbers loaded before the eight pieces, so that a thread keeps 128 bytes in flight.
constexpr int kPermutePer = 8;

template <typename IndexT>
__global__ void __launch_bounds__(256)
permute_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ order, int64_t n_rows, int vecs,
                    uint4* __restrict__ dst) {
  const IndexT total = (IndexT)(n_rows * vecs);
  const IndexT first = (IndexT)blockIdx.x * (256 * kPermutePer) + threadIdx.x;
  int64_t from[kPermutePer];
#pragma unroll
  for (int j = 0; j < kPermutePer; ++j) {
    const IndexT i = first + (IndexT)j * 256;
    from[j] = -1;
    if (i < total) {
      const IndexT r = i / (IndexT)vecs;
      from[j] = (int64_t)__ldg(order + r) * vecs + (int64_t)(i - r * (IndexT)vecs);
    }
  }
  uint4 piece[kPermutePer];
#pragma unroll
  for (int j = 0; j < kPermutePer; ++j)
    if (from[j] >= 0) piece[j] = __ldg(src + from[j]);
#pragma unroll
  for (int j = 0; j < kPermutePer; ++j)
    if (from[j] >= 0) dst[first + (IndexT)j * 256] = piece[j];
}

static void launch_permute_rows(const void* src, const int32_t* order, int64_t n_rows, int vecs, void* dst,
                                cudaStream_t stream) {
  const int64_t total = n_rows * vecs;
  const unsigned blocks = (unsigned)((total + 256 * kPermutePer - 1) / (256 * kPermutePer));
  if (total + 256 * kPermutePer < 0xFFFFFFFFll)
    permute_rows_kernel<uint32_t><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(src), order, n_rows, vecs,
                                                              static_cast<uint4*>(dst));
  else
    permute_rows_kernel<int64_t><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(src), order, n_rows, vecs,
                                                             static_cast<uint4*>(dst));
  note_launches(1);
}

// The copy pass pays for itself when a tile is fetched by four CTAs or more (offset groups x channel blocks); with two
// groups (32 input channels: 16 offsets per group) it only adds its own cost.
static bool wgrad_copy_pays(const tc::WgradParams& p) { return p.n_kgroups * p.n_ciblk * p.n_coblk >= 4; }

// Tile-plan form: the TMA-fed kernel when both tensors can be described to the copy engine and two
// slots fit, else the cp.async producers of wgrad_kernel over the same plan.  `sorted_rows`: scratch for a copy of
// the tile operand in tile order (n_rows x cout elements), or null.
static int launch_wgrad_planned(WgradPlan& plan, const tc::PlannedRows& map, cudaStream_t stream, void* sorted_rows,
                                bool presorted) {
  tc::WgradParams& p = plan.p;
  if (p.swap) {
    // ring 1 holds X tiles (ci_blk wide), ring 2 the gathered dY rows (128 output channels wide)
    const int t = p.a_slot_bytes;
    p.a_slot_bytes = p.b_slot_bytes;
    p.b_slot_bytes = t;
  }
  // Shared memory: a ring of dY tiles and a ring of X-row slots of `quad` offsets each.  Two shapes, chosen by
  // measurement: rows of one 128-byte line travel four offsets to a slot, two slots, indices loaded as the
  // task comes up; wider rows (two lines, 128 or more 16-bit channels) travel one offset to a slot with three
  // dY tiles in flight and the indices loaded ahead.
  const bool wide = p.b_slot_bytes >= 2 * tc::kABlockBytes;
  int a_slots = wide ? 3 : 2, quad = wide ? 1 : tc::kProducerWarps, ahead = wide ? 2 : 0, b_cap = wide ? tc::kWgradBSlots3 : 4;
#ifdef ST_TC_PROFILE
  {
    const char* e = getenv("ST_TC_QUAD");
    if (e && atoi(e) >= 1 && atoi(e) <= tc::kProducerWarps) quad = atoi(e);
    const char* f = getenv("ST_TC_ASLOTS");
    if (f && atoi(f) >= 2 && atoi(f) <= tc::kWgradASlots3) a_slots = atoi(f);
    const char* g = getenv("ST_TC_AHEAD");
    if (g) ahead = atoi(g);
    const char* h = getenv("ST_TC_BCAP");
    if (h && atoi(h) >= 2 && atoi(h) <= tc::kWgradBSlots3) b_cap = atoi(h);
  }
#endif
  if (quad > p.group) quad = p.group;
  int budget = 222 * 1024 - a_slots * p.a_slot_bytes - (int)sizeof(tc::WgradControl3);
  while (a_slots > 2 && budget < 2 * quad * p.b_slot_bytes) {
    --a_slots;
    budget += p.a_slot_bytes;
  }
  while (quad > 1 && budget < 2 * quad * p.b_slot_bytes) --quad;
  CUtensorMap x_desc, dy_desc, tile_box_desc;
  memset(&x_desc, 0, sizeof(x_desc));
  memset(&dy_desc, 0, sizeof(dy_desc));
  memset(&tile_box_desc, 0, sizeof(tile_box_desc));
  const int dtype = p.esize == 4 ? ST_F32 : ST_BF16;      // element size is all the copy engine needs to know
  const bool tma = g_tma_enabled && budget >= 2 * quad * p.b_slot_bytes && p.n_src > 0 &&
                   make_gather_desc(&x_desc, p.x, p.swap ? p.n_rows : p.n_src, p.cin, p.esize, dtype, p.esize == 4) &&
                   make_gather_desc(&dy_desc, p.dy, p.swap ? p.n_src : p.n_rows, p.cout, p.esize, dtype, p.esize == 4);
  // The dY tile of a step is 128 rows picked through `order`: 32 row gathers per 128-byte column block, and every
  // offset group (and input-channel block) of a row chunk fetches it again.  With the rows copied into tile order once
  // (one streaming pass) a tile is a dense box, which the copy engine moves 2.3x faster.
  // `presorted`: the caller made that copy already (tc_wgrad_sort_rows, typically on another stream beside the
  // feature gradient).
  p.dense_tiles = 0;
  if (tma && !p.swap && g_dense_tiles &&
      (p.order == nullptr || (sorted_rows != nullptr && (presorted || wgrad_copy_pays(p)))) &&
      (p.cout * p.esize) % 16 == 0) {
    const void* tiles = p.dy;
    if (p.order) {
      if (!presorted) launch_permute_rows(p.dy, p.order, p.n_rows, p.cout * p.esize / 16, sorted_rows, stream);
      tiles = sorted_rows;
    }
    if (make_weight_desc(&tile_box_desc, tiles, p.n_rows, p.cout, p.esize, dtype, tc::kTileM, p.esize == 4)) p.dense_tiles = 1;
  }
  if (!tma) {
    if (p.swap) {
      set_error("tc wgrad over the inverse plan needs the TMA kernels (16-byte aligned tensors, st_set_tma(1))");
      return ST_ERR_UNSUPPORTED;
    }
    return launch_wgrad(plan, map, stream);
  }
  p.quad = quad;
  p.a_slots = a_slots;
  int slots = budget / (quad * p.b_slot_bytes);
#ifdef ST_TC_PROFILE
  {
    const char* e = getenv("ST_TC_BSLOTS");
    if (e && atoi(e) >= 2 && atoi(e) <= slots) slots = atoi(e);
  }
#endif
  p.b_slots = slots > b_cap ? b_cap : slots;
  const size_t smem = (size_t)a_slots * p.a_slot_bytes + (size_t)p.b_slots * quad * p.b_slot_bytes + sizeof(tc::WgradControl3) + 1024;
  auto kernel = ahead == 0 ? tc::planned_wgrad_kernel<0> : (ahead == 2 ? tc::planned_wgrad_kernel<2> : tc::planned_wgrad_kernel<4>);
  static bool configured[kMaxDevices] = {};
  if (!configured[current_device()]) {
    for (auto k : {tc::planned_wgrad_kernel<0>, tc::planned_wgrad_kernel<2>, tc::planned_wgrad_kernel<4>}) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) {
        set_error("tc planned wgrad: cannot raise the dynamic shared memory limit: %s", cudaGetErrorString(e));
        return ST_ERR_CUDA;
      }
    }
    configured[current_device()] = true;
  }
  dim3 grid((unsigned)plan.n_chunks, (unsigned)p.n_kgroups, (unsigned)(p.n_coblk * p.n_ciblk));
  kernel<<<grid, tc::kThreads, smem, stream>>>(p, map, x_desc, dy_desc, tile_box_desc);
  note_launches(1);
  return check_launch("tc planned wgrad");
}

static bool prepare_wgrad(WgradPlan* plan, int dtype, const void* x, const void* dy, float* partial, int64_t n_rows,
                          int64_t n_src, int K, int cin, int cout) {
  if (!plan_wgrad(plan, dtype, n_rows, K, cin, cout)) {
    set_error("tc wgrad: unsupported shape");
    return false;
  }
  plan->p.x = x;
  plan->p.dy = dy;
  plan->p.order = nullptr;
  plan->p.quad = 1;
  plan->p.a_slots = 2;
  plan->p.swap = 0;
  plan->p.dense_tiles = 0;
  plan->p.partial = partial;
  plan->p.n_src = n_src;
  return true;
}

int tc_conv_wgrad(int dtype, const void* x, const void* dy, const int32_t* map, const MapPlan& rows, float* partial,
                  int* n_chunks_out, int64_t n_rows, int64_t n_src, int K, int cin, int cout, cudaStream_t stream,
                  bool inverse_plan, void* sorted_rows, bool presorted) {
  WgradPlan plan;
  if (!prepare_wgrad(&plan, dtype, x, dy, partial, n_rows, n_src, K, cin, cout)) return ST_ERR_UNSUPPORTED;
  plan.p.order = rows.order;
  plan.p.swap = inverse_plan ? 1 : 0;
  if (inverse_plan && !(rows.tmap && rows.tmask)) {
    set_error("tc wgrad: the inverse form needs a tile plan");
    return ST_ERR_ARG;
  }
  int rc;
  if (rows.tmap && rows.tmask)
    rc = launch_wgrad_planned(plan, tc::PlannedRows{rows.tmap, rows.tmask, K, (K + 31) / 32}, stream, sorted_rows,
                              presorted);
  else
    rc = launch_wgrad(plan, tc::StoredRows{map, K}, stream);
  *n_chunks_out = plan.n_chunks;
  return rc;
}

bool tc_wgrad_sorts_rows(int dtype, int64_t n_rows, int K, int cin, int cout) {
  WgradPlan plan;
  if (!g_tma_enabled || !g_dense_tiles || !plan_wgrad(&plan, dtype, n_rows, K, cin, cout)) return false;
  return wgrad_copy_pays(plan.p) && (plan.p.cout * plan.p.esize) % 16 == 0;
}

int tc_wgrad_sort_rows(int dtype, const void* dy, const int32_t* order, int64_t n_rows, int cout, void* sorted,
                       cudaStream_t stream) {
  const int esize = dtype == ST_F32 ? 4 : 2;
  if ((cout * esize) % 16 != 0 || ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(sorted)) & 15)) {
    set_error("tc wgrad: rows to sort must be whole 16-byte pieces at 16-byte aligned addresses");
    return ST_ERR_UNSUPPORTED;
  }
  launch_permute_rows(dy, order, n_rows, cout * esize / 16, sorted, stream);
  return check_launch("tc wgrad row sort");
}

int tc_conv_wgrad_hashfly(int dtype, const void* x, const void* dy, const HashFlyArgs& h, float* partial,
                          int* n_chunks_out, int64_t n_rows, int64_t n_src, int K, int cin, int cout,
                          cudaStream_t stream) {
  WgradPlan plan;
  if (!prepare_wgrad(&plan, dtype, x, dy, partial, n_rows, n_src, K, cin, cout)) return ST_ERR_UNSUPPORTED;
  *n_chunks_out = plan.n_chunks;
  if (h.coord_dtype == ST_I32) return launch_wgrad(plan, make_hash_rows<int32_t>(h), stream);
  return launch_wgrad(plan, make_hash_rows<int16_t>(h), stream);
}

int tc_read_prof(long long* host_out, int n) {
  cudaDeviceSynchronize();
  return cudaMemcpyFromSymbol(host_out, tc::g_prof, sizeof(long long) * n) == cudaSuccess ? ST_OK : ST_ERR_CUDA;
}

int tc_read_status(int32_t* host_out4, cudaStream_t stream, bool wait) {
  cudaError_t e = cudaMemcpyFromSymbolAsync(host_out4, tc::g_status, sizeof(int32_t) * 4, 0, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess && wait) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    set_error("tc_read_status: %s", cudaGetErrorString(e));
    return ST_ERR_CUDA;
  }
  return ST_OK;
}

int tc_clear_status(cudaStream_t stream) {
  void* addr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&addr, tc::g_status);
  if (e == cudaSuccess) e = cudaMemsetAsync(addr, 0, sizeof(int32_t) * 4, stream);
  if (e != cudaSuccess) {
    set_error("tc_clear_status: %s", cudaGetErrorString(e));
    return ST_ERR_CUDA;
  }
  return ST_OK;
}

}  // namespace st
