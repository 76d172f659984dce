// Gather kernel for a stored map in tile-plan form, fed by TMA.  Included by conv_tc.cu (one
// translation unit: the device status word and the PTX wrappers are file-local there).
//
//   OUT[order[r], :] = sum_k  IN[tmap(r, k), :] . B_k
//
// Same roles as gather2_kernel (warps 0-3 epilogue, warp 4 MMA issuer, warps 5-8 producers) and the
// same super tiles of S row tiles that share the copies of W, but the unit that travels through
// shared memory is a whole kernel offset of the super tile:
//
//   slot = [ W slice of (k, kb) | rows of sub tile 0 | ... | rows of sub tile S-1 ]      one mbarrier
//
// or, to have more and smaller slots in flight, a part of it: the super tile's S sub tiles are dealt
// in parts of P; the offset's first item carries the W slice and its slot is held back until the
// offset's last item has been multiplied.
//
// Producer warp w fetches the rows of sub tile w with 32 tile::gather4 copies (lane l: rows 4l..4l+3;
// "-1" and rows past the end of the source are out of bounds and arrive as zeros); warp 0 also
// fetches the W slice with one or two tiled copies; each warp announces its own bytes on the slot's
// mbarrier.  The MMA
// thread then waits once, issues up to 4 x S tcgen05.mma and commits once per offset.  With one wait
// / commit per 16-KB row stage (gather2_kernel) the MMA thread's own instruction stream was the
// bottleneck (about 600 cycles of bookkeeping for 256 cycles of tensor work).
//
// Every producer warp waits for every slot's release, whether or not its sub tile takes part in the
// offset: an mbarrier wait names a phase only by its parity, so a warp that skipped laps of a slot
// could be two laps ahead of the consumer and mistake an old phase for the one it needs.
#pragma once

namespace st {
namespace tc {

constexpr int kMaxSlots3 = 6;

struct __align__(8) Control3 {
  unsigned long long full[kMaxSlots3], empty[kMaxSlots3];
  unsigned long long acc_full[2], acc_empty[2];
  // bits 0-3 sub tiles that take part, bits 4-7 those whose accumulator starts here, bits 8-11 K-steps,
  // bit 12 end of super tile (no data), bit 13 the slot carries the offset's W slice, bit 14 last item
  // of the offset, bits 16-17 which part of the super tile the slot's rows belong to
  uint32_t info[kMaxSlots3];
  uint32_t tmem_base;
  int abort_flag;
};

template <int ESIZE>
__global__ void __launch_bounds__(kThreads, 1) planned_gather_kernel(const Params2 p, const PlannedRows map,
                                                                     const __grid_constant__ CUtensorMap in_desc,
                                                                     const __grid_constant__ CUtensorMap w_desc) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - raw);
  Control3* ctl = reinterpret_cast<Control3*>(base_ptr + (size_t)p.n_slots * p.slot_bytes);
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.n_slots; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), kProducerWarps);
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
  const int red_bytes = p.c_red * ESIZE;
  const int set_cols = p.sub * p.c_acc;                      // TMEM columns of one accumulator set
  const int64_t n_tiles = (p.n_rows + kTileM - 1) / kTileM;

  if (warp >= kFirstProducerWarp) {
    // =============================================================== producers
    const int pw = warp - kFirstProducerWarp;                // sub tile served by this warp
    const int kr = 128 / ESIZE;
    const int w_col_bytes = p.w_cols * ESIZE;
    const uint32_t w_bytes = p.b_mn_major ? (uint32_t)(((w_col_bytes + 127) >> 7) * kr * 128) : (uint32_t)(p.w_rows * 128);
    int slot = 0;
    uint32_t phase = 0;
    bool ok = true;
    struct Item {
      int k, kb;
      uint32_t users, fresh;   // sub tiles of this item (absolute bits)
      int part;                // which group of p.part sub tiles
      bool has_w, last;        // carries the W slice / is the offset's last item
      int slot;
      uint32_t parity;
      bool marker, valid;
    };
    Item pend{0, 0, 0u, 0u, 0, false, false, 0, 0u, false, false};
    int4 pend_idx = make_int4(-1, -1, -1, -1);

    auto run = [&](const Item& d, const int4& idx) {
      ok = mbar_wait_warp(smem_u32(&ctl->empty[d.slot]), d.parity ^ 1u, abort_flag, 31, lane);
      if (!ok) return;
      const uint32_t bar = smem_u32(&ctl->full[d.slot]);
      const uint32_t slot_base = base + (uint32_t)d.slot * (uint32_t)p.slot_bytes;
      const bool copy_rows = !d.marker && !ST_DBG(p, 4) && ((d.users >> pw) & 1u);
      if (lane == 0) {
        // Every producer warp arrives on every slot, announcing the bytes of its own copies first (a
        // copy that completed before its bytes were announced would drive the count negative).
        const bool copy_w = pw == 0 && d.has_w && !d.marker && !ST_DBG(p, 16);
        if (pw == 0) {
          const int valid_bytes = d.marker ? 0 : min(128, red_bytes - d.kb * 128);
          ctl->info[d.slot] = d.users | (d.fresh << 4) | ((uint32_t)(valid_bytes >> 5) << 8) | (d.marker ? 0x1000u : 0u) |
                              (d.has_w ? 0x2000u : 0u) | (d.last ? 0x4000u : 0u) | ((uint32_t)d.part << 16);
        }
        const uint32_t bytes = (copy_w ? w_bytes : 0u) + (copy_rows ? (uint32_t)kABlockBytes : 0u);
        if (bytes) mbar_arrive_expect_tx(bar, bytes); else mbar_arrive(bar);
        if (copy_w) {
          const int kw = p.w_flip ? p.K - 1 - d.k : d.k;     // which W slice this offset multiplies with
          if (p.b_mn_major) {
            const int n_cb = (w_col_bytes + 127) >> 7;
            for (int cb = 0; cb < n_cb; ++cb)
              tma_load_2d(slot_base + (uint32_t)(cb * kr * 128), &w_desc, bar, cb * kr, kw * p.w_rows + d.kb * kr);
          } else {
            tma_load_2d(slot_base, &w_desc, bar, d.kb * kr, kw * p.w_rows);
          }
        }
      }
      __syncwarp();
      if (copy_rows)
        tma_gather4(slot_base + (uint32_t)p.w_slot_bytes + (uint32_t)(pw - d.part * p.part) * kABlockBytes +
                        (uint32_t)lane * 512u,
                    &in_desc, bar, d.kb * kr, idx.x, idx.y, idx.z, idx.w);
    };
    // Queue one item: its indices are loaded now and it is issued when the next one is queued, so the
    // load overlaps the previous item's wait and copies.
    auto emit_item = [&](int64_t tile0, const Item& d, bool zeros) {
      int4 idx = make_int4(-1, -1, -1, -1);
      if (!d.marker && !zeros && ((d.users >> pw) & 1u))
        idx = __ldg(reinterpret_cast<const int4*>(map.tmap + ((tile0 + pw) * map.K + d.k) * (int64_t)kTileM) + lane);
      if (pend.valid && ok) run(pend, pend_idx);
      pend = d;
      pend.slot = slot;
      pend.parity = phase;
      pend.valid = true;
      pend_idx = idx;
      if (++slot == p.n_slots) {
        slot = 0;
        phase ^= 1u;
      }
    };
    // One offset of the super tile: an item per part (p.part sub tiles) that has a user; the first one
    // carries the W slice, which the later ones read from its slot.
    auto emit = [&](int64_t tile0, int k, int kb, uint32_t users, uint32_t fresh, bool marker, bool zeros) {
      if (marker) {
        emit_item(tile0, Item{0, 0, 0u, 0u, 0, false, false, 0, 0u, true, true}, false);
        return;
      }
      const uint32_t part_bits = (1u << p.part) - 1u;
      bool first = true;
      for (int q = 0; q * p.part < p.sub; ++q) {
        const uint32_t u = users & (part_bits << (q * p.part));
        if (!u) continue;
        const bool last = (users >> ((q + 1) * p.part)) == 0u;
        emit_item(tile0, Item{k, kb, u, fresh & u, q, first, last, 0, 0u, false, true}, zeros);
        first = false;
      }
    };
    auto load_masks = [&](int64_t tile0, int word, uint32_t* m) {
#pragma unroll
      for (int s = 0; s < kMaxSub; ++s)
        m[s] = (s < p.sub && tile0 + s < n_tiles) ? __ldg(map.tmask + (tile0 + s) * map.MW + word) : 0u;
    };
    uint32_t next_m[kMaxSub];
    load_masks((int64_t)blockIdx.x * p.sub, 0, next_m);
    for (int64_t st_i = blockIdx.x; st_i < p.n_super && ok; st_i += gridDim.x) {
      const int64_t tile0 = st_i * p.sub;
      uint32_t m0[kMaxSub];
#pragma unroll
      for (int s = 0; s < kMaxSub; ++s) m0[s] = next_m[s];
      if (st_i + gridDim.x < p.n_super) {
        const int64_t next_tile0 = (st_i + gridDim.x) * p.sub;
        load_masks(next_tile0, 0, next_m);
        // the index lines of a super tile are one contiguous block of the plan: have the next one in L2
        const int64_t tiles = min((int64_t)p.sub, n_tiles - next_tile0);
        const char* block = reinterpret_cast<const char*>(map.tmap + next_tile0 * map.K * (int64_t)kTileM);
        const int64_t lines = min(tiles * map.K * 4, (int64_t)1024);               // 128-byte lines
        for (int64_t l = (warp - kFirstProducerWarp) * 32 + lane; l < lines; l += kProducerThreads)
          prefetch_l2(block + l * 128);
      }
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
          uint32_t users = 0;
#pragma unroll
          for (int s = 0; s < kMaxSub; ++s) users |= ((m[s] >> j) & 1u) << s;
          for (int kb = 0; kb < p.k_blocks && ok; ++kb)
            emit(tile0, word * 32 + j, kb, users, kb == 0 ? (users & ~touched) : 0u, false, false);
          touched |= users;
        }
      }
      // sub tiles that exist but never got a neighbour still have to write zeros
      uint32_t untouched = 0;
      for (int s = 0; s < p.sub; ++s)
        if (tile0 + s < n_tiles && !((touched >> s) & 1u)) untouched |= 1u << s;
      if (untouched && ok) emit(tile0, 0, 0, untouched, untouched, false, true);
      if (ok) emit(tile0, 0, 0, 0u, 0u, true, false);                            // end of super tile
    }
    if (pend.valid && ok) run(pend, pend_idx);
  } else if (warp == kMmaWarp) {
    // =============================================================== MMA issuer
    if (lane == 0) {
      int slot = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      const uint32_t b_kstep16 = (p.b_mn_major ? (32 / ESIZE) * 128 : 32) >> 4;   // K-step advance, 16-byte units
      const uint32_t b_lbo = p.b_mn_major ? (uint32_t)(128 / ESIZE) * 128u : 16u;
      const bool b_base32 = p.b_mn_major && ESIZE == 4;
      const uint64_t a_desc_hi = smem_desc(0u, 16u, 1024u, 2u);
      const uint64_t b_desc_hi = smem_desc(0u, b_lbo, b_base32 ? 512u : 1024u, b_base32 ? 1u : 2u);
      const uint32_t idesc = p.idesc;
      uint32_t w_lo = 0;
      int held = -1;                                          // slot kept for its W slice
      for (int64_t st_i = blockIdx.x; st_i < p.n_super && ok; st_i += gridDim.x) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[buf]), acc_phase[buf] ^ 1u, abort_flag, 32);
        if (!ok) break;
        tc_fence_after();
        for (;;) {
          ok = mbar_wait(smem_u32(&ctl->full[slot]), phase, abort_flag, 33);
          if (!ok) break;
          const uint32_t info = ctl->info[slot];
          tc_fence_after();
          const uint32_t slot_base = base + (uint32_t)slot * (uint32_t)p.slot_bytes;
          if (info & 0x2000u) {                                  // the offset's W slice lives in this slot
            w_lo = slot_base >> 4;
            held = slot;
          }
          if (!(info & 0x1000u) && !ST_DBG(p, 2)) {
            const int ksteps = (int)((info >> 8) & 15u);
            const int part0 = (int)((info >> 16) & 3u) * p.part;
#pragma unroll
            for (int s = 0; s < kMaxSub; ++s) {
              if (!((info >> s) & 1u)) continue;
              const uint32_t a_lo = (slot_base + (uint32_t)p.w_slot_bytes + (uint32_t)(s - part0) * kABlockBytes) >> 4;
              const uint32_t d_addr = tmem_base + (uint32_t)(buf * set_cols + s * p.c_acc);
              const uint32_t fresh = ((info >> (4 + s)) & 1u) ? 0u : 1u;        // 0: the first MMA overwrites
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
            }
          }
          // A slot that holds the W slice stays with the consumer until the offset's last item is done.
          if (info & 0x1000u) {
            mma_commit(smem_u32(&ctl->empty[slot]));
          } else if (info & 0x4000u) {
            if (held >= 0 && held != slot) mma_commit(smem_u32(&ctl->empty[held]));
            mma_commit(smem_u32(&ctl->empty[slot]));
            held = -1;
          } else if (held != slot) {
            mma_commit(smem_u32(&ctl->empty[slot]));
          }
          if (++slot == p.n_slots) {
            slot = 0;
            phase ^= 1u;
          }
          if (info & 0x1000u) break;
        }
        if (!ok) break;
        mma_commit(smem_u32(&ctl->acc_full[buf]));
        acc_phase[buf] ^= 1u;
        if (p.acc_bufs == 2) buf ^= 1;
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
      ok = mbar_wait(smem_u32(&ctl->acc_full[buf]), acc_phase[buf], abort_flag, 34, 256);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int s = 0; s < kMaxSub; ++s) {
        if (s >= p.sub) break;
        const int64_t row = (st_i * p.sub + s) * (int64_t)kTileM + warp * 32 + lane;
        if ((st_i * p.sub + s) * (int64_t)kTileM >= p.n_rows) break;         // whole sub tile past the end
        char* out_row = static_cast<char*>(p.out) + (size_t)dst_rows[s] * p.c_acc * out_es;
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
// Weight gradient over a stored map in tile-plan form, fed by TMA.
//
//   dW[k][ci][co] = sum_r  X[tmap(r, k)][ci] * dY[order[r]][co]
//
// Same decomposition as wgrad_kernel (a CTA owns a chunk of row tiles, a group of G offsets whose G
// accumulators fill TMEM, a block of output channels and one of input channels; fp32 partials per
// chunk), but:
//   - the tile's mask says which offsets of the group have any neighbour in the tile; both the
//     producers and the MMA thread read it, so no step descriptors travel through shared memory;
//   - the dY tile and the gathered X rows arrive by tile::gather4 (rows of dY through `order`, rows
//     of X through the tile's index lines);
//   - up to Q offsets share one shared-memory slot and one mbarrier (producer warp q fetches the
//     rows of the q-th of them), so the MMA thread waits and commits once per Q x 8 (16) MMAs.
// Every producer warp arrives on every barrier (see planned_gather_kernel).
// =================================================================================================
constexpr int kWgradASlots3 = 4;
constexpr int kWgradBSlots3 = 12;

struct __align__(8) WgradControl3 {
  unsigned long long a_full[kWgradASlots3], a_empty[kWgradASlots3];
  unsigned long long b_full[kWgradBSlots3], b_empty[kWgradBSlots3];
  unsigned long long acc_full;
  uint32_t touched;
  uint32_t tmem_base;
  int abort_flag;
};

template <int kAhead>
__global__ void __launch_bounds__(kThreads, 1) planned_wgrad_kernel(const WgradParams p, const PlannedRows map,
                                                                    const __grid_constant__ CUtensorMap x_desc,
                                                                    const __grid_constant__ CUtensorMap dy_desc,
                                                                    const __grid_constant__ CUtensorMap tile_box_desc) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - raw);
  const uint32_t a_ring = base;
  const uint32_t b_ring = base + (uint32_t)p.a_slots * (uint32_t)p.a_slot_bytes;
  const uint32_t quad_bytes = (uint32_t)p.quad * (uint32_t)p.b_slot_bytes;
  WgradControl3* ctl = reinterpret_cast<WgradControl3*>(base_ptr + (size_t)p.a_slots * p.a_slot_bytes + (size_t)p.b_slots * quad_bytes);
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
  // The chunk takes every gridDim.x-th tile: in sorted row order the number of occupied offsets grows
  // along the rows, so contiguous ranges of tiles would be very unequal pieces of work.
  const int64_t tile_begin = chunk, tile_end = p.n_tiles, tile_step = gridDim.x;
  const int word = k_first >> 5, shift = k_first & 31;
  const uint32_t group_bits = g_count >= 32 ? 0xFFFFFFFFu : ((1u << g_count) - 1u);
  const int per_line = 128 / p.esize;                       // elements of one 128-byte line
  // The per-tile operand (ring 1, rows taken through `order`) and the per-offset operand (ring 2, rows taken
  // through the plan's index lines).  Over the forward map the tile operand is dY (M side of the product) and
  // the gathered one X (N side); with p.swap the kernel walks the plan of the INVERSE map instead: the tile
  // operand is X, the gathered one dY, and the MMA takes its A operand from ring 2 and its B operand from ring 1.
  const int m_blocks = (co_cnt * p.esize + 127) >> 7;       // 128-byte column blocks of dY rows
  const int n_blocks = (ci_cnt * p.esize + 127) >> 7;       // ... of X rows
  const int a_blocks = p.swap ? n_blocks : m_blocks;        // blocks of the tile operand
  const int b_blocks = p.swap ? m_blocks : n_blocks;        // blocks of the gathered operand
  const CUtensorMap* tile_desc = p.swap ? &x_desc : &dy_desc;
  const CUtensorMap* gath_desc = p.swap ? &dy_desc : &x_desc;
  const int tile_col0 = p.swap ? ci0 : co0, gath_col0 = p.swap ? co0 : ci0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.a_slots; ++s) {
      mbar_init(smem_u32(&ctl->a_full[s]), kProducerWarps);
      mbar_init(smem_u32(&ctl->a_empty[s]), 1);
    }
    for (int s = 0; s < p.b_slots; ++s) {
      mbar_init(smem_u32(&ctl->b_full[s]), kProducerWarps);
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

  auto tile_mask = [&](int64_t tile) { return (__ldg(map.tmask + tile * map.MW + word) >> shift) & group_bits; };

  if (warp >= kFirstProducerWarp) {
    // =============================================================== producers
    // The CTA's copies form one sequence of tasks: per tile with an occupied offset, the dY tile (A), then
    // one slot of X rows per `quad` occupied offsets (B).  Every producer warp walks the whole sequence (it
    // has to arrive on every barrier) with two cursors: `fetch` runs kAhead tasks in front and loads the
    // row indices a task needs (a line of `order` or of the plan) into a short register queue, `issue`
    // waits for the task's slot and starts its copies with indices that have long arrived.  Without the
    // look-ahead every slot paid one trip to DRAM for its indices before its copies could start.
    if constexpr (kAhead == 0) {
      // plain form: each task loads its row indices, waits for its slot and starts its copies
      const int pw = warp - kFirstProducerWarp;
      int a_slot = 0, b_slot = 0;
      uint32_t a_phase = 0, b_phase = 0;
      bool ok = true;
      uint32_t m_next = tile_begin < tile_end ? tile_mask(tile_begin) : 0u;
      for (int64_t tile = tile_begin; tile < tile_end && ok; tile += tile_step) {
        uint32_t m = m_next;
        if (tile + tile_step < tile_end) m_next = tile_mask(tile + tile_step);
        if (!m) continue;
        // ---- the dY tile: rows order[tile * 128 + r], or one dense box when the rows lie in tile order
        if (p.dense_tiles) {
          ok = mbar_wait_warp(smem_u32(&ctl->a_empty[a_slot]), a_phase ^ 1u, abort_flag, 35, lane);
          if (!ok) break;
          const uint32_t bar = smem_u32(&ctl->a_full[a_slot]);
          const uint32_t slot_base = a_ring + (uint32_t)a_slot * (uint32_t)p.a_slot_bytes;
          if (lane == 0) {
            int mine = 0;
            for (int b = pw; b < a_blocks; b += kProducerWarps) ++mine;
            if (mine) mbar_arrive_expect_tx(bar, (uint32_t)mine * kABlockBytes); else mbar_arrive(bar);
            for (int b = pw; b < a_blocks; b += kProducerWarps)
              tma_load_2d(slot_base + (uint32_t)b * kABlockBytes, &tile_box_desc, bar, tile_col0 + b * per_line,
                          (int)(tile * kTileM));
          }
          __syncwarp();
          if (++a_slot == p.a_slots) {
            a_slot = 0;
            a_phase ^= 1u;
          }
        } else {
          const int64_t pos = tile * kTileM + 4 * lane;
          int4 rows;
          if (p.order) {
            // the last tile's line may run past the end of `order`: read only what exists
            rows.x = pos + 0 < p.n_rows ? __ldg(p.order + pos + 0) : -1;
            rows.y = pos + 1 < p.n_rows ? __ldg(p.order + pos + 1) : -1;
            rows.z = pos + 2 < p.n_rows ? __ldg(p.order + pos + 2) : -1;
            rows.w = pos + 3 < p.n_rows ? __ldg(p.order + pos + 3) : -1;
          } else {
            rows = make_int4((int)pos, (int)pos + 1, (int)pos + 2, (int)pos + 3);
          }
          if (pos + 0 >= p.n_rows) rows.x = -1;
          if (pos + 1 >= p.n_rows) rows.y = -1;
          if (pos + 2 >= p.n_rows) rows.z = -1;
          if (pos + 3 >= p.n_rows) rows.w = -1;
          ok = mbar_wait_warp(smem_u32(&ctl->a_empty[a_slot]), a_phase ^ 1u, abort_flag, 35, lane);
          if (!ok) break;
          const uint32_t bar = smem_u32(&ctl->a_full[a_slot]);
          const uint32_t slot_base = a_ring + (uint32_t)a_slot * (uint32_t)p.a_slot_bytes;
          // column block b is fetched by warp b % 4
          int mine = 0;
          for (int b = pw; b < a_blocks; b += kProducerWarps) ++mine;
          if (lane == 0) {
            if (mine) mbar_arrive_expect_tx(bar, (uint32_t)mine * kABlockBytes); else mbar_arrive(bar);
          }
          __syncwarp();
          for (int b = pw; b < a_blocks; b += kProducerWarps)
            tma_gather4(slot_base + (uint32_t)b * kABlockBytes + (uint32_t)lane * 512u, tile_desc, bar, tile_col0 + b * per_line,
                        rows.x, rows.y, rows.z, rows.w);
          if (++a_slot == p.a_slots) {
            a_slot = 0;
            a_phase ^= 1u;
          }
        }
        // ---- the gathered X rows, `quad` offsets per slot: warp q fetches the q-th of them
        while (m && ok) {
          int my_j = -1;
          for (int q = 0; q < p.quad && m; ++q) {
            const int j = __ffs(m) - 1;
            m &= m - 1;
            if (q == pw) my_j = j;
          }
          int4 idx = make_int4(-1, -1, -1, -1);
          if (my_j >= 0)
            idx = __ldg(reinterpret_cast<const int4*>(map.tmap + (tile * map.K + k_first + my_j) * (int64_t)kTileM) + lane);
          ok = mbar_wait_warp(smem_u32(&ctl->b_empty[b_slot]), b_phase ^ 1u, abort_flag, 36, lane);
          if (!ok) break;
          const uint32_t bar = smem_u32(&ctl->b_full[b_slot]);
          const uint32_t stage = b_ring + (uint32_t)b_slot * quad_bytes + (uint32_t)pw * (uint32_t)p.b_slot_bytes;
          if (lane == 0) {
            if (my_j >= 0) mbar_arrive_expect_tx(bar, (uint32_t)b_blocks * kABlockBytes); else mbar_arrive(bar);
          }
          __syncwarp();
          if (my_j >= 0) {
            for (int b = 0; b < b_blocks; ++b)
              tma_gather4(stage + (uint32_t)b * kABlockBytes + (uint32_t)lane * 512u, gath_desc, bar, gath_col0 + b * per_line, idx.x,
                          idx.y, idx.z, idx.w);
          }
          if (++b_slot == p.b_slots) {
            b_slot = 0;
            b_phase ^= 1u;
          }
        }
      }
    } else {
    const int pw = warp - kFirstProducerWarp;
    struct Cursor {
      int64_t tile;
      uint32_t m, m_next, b_count;
      int a_slot, b_slot;
      uint32_t a_phase, b_phase;
      bool in_tile;
    };
    struct Task {
      int kind;                 // 0 none, 1 dY tile, 2 X rows
      int64_t tile;
      int slot;
      uint32_t parity;
      int my_j;                 // kind 2: offset (within the group) this warp copies, or -1
    };
    auto cursor = [&]() {
      Cursor c;
      c.tile = tile_begin;
      c.m = 0;
      c.m_next = tile_begin < tile_end ? tile_mask(tile_begin) : 0u;
      c.b_count = 0;
      c.a_slot = c.b_slot = 0;
      c.a_phase = c.b_phase = 0;
      c.in_tile = false;
      return c;
    };
    auto next = [&](Cursor& c) {
      Task t{0, 0, 0, 0u, -1};
      for (;;) {
        if (c.tile >= tile_end) return t;
        if (!c.in_tile) {
          c.m = c.m_next;
          c.m_next = c.tile + tile_step < tile_end ? tile_mask(c.tile + tile_step) : 0u;
          if (!c.m) {
            c.tile += tile_step;
            continue;
          }
          c.in_tile = true;
          t = Task{1, c.tile, c.a_slot, c.a_phase, -1};
          if (++c.a_slot == p.a_slots) {
            c.a_slot = 0;
            c.a_phase ^= 1u;
          }
          return t;
        }
        // `quad` offsets per slot: warp q copies the q-th of them; with one offset per slot the warps take turns
        int my_j = -1;
        for (int q = 0; q < p.quad && c.m; ++q) {
          const int j = __ffs(c.m) - 1;
          c.m &= c.m - 1;
          if ((p.quad == 1 ? (int)(c.b_count & (kProducerWarps - 1)) : q) == pw) my_j = j;
        }
        t = Task{2, c.tile, c.b_slot, c.b_phase, my_j};
        ++c.b_count;
        if (++c.b_slot == p.b_slots) {
          c.b_slot = 0;
          c.b_phase ^= 1u;
        }
        if (!c.m) {
          c.in_tile = false;
          c.tile += tile_step;
        }
        return t;
      }
    };
    int a_mine = 0;                                   // column blocks of the dY tile this warp copies (block b: warp b % 4)
    for (int b = pw; b < a_blocks; b += kProducerWarps) ++a_mine;
    auto load_rows = [&](const Task& t) {
      int4 rows = make_int4(-1, -1, -1, -1);
      if (t.kind == 1 && a_mine) {
        const int64_t pos = t.tile * kTileM + 4 * lane;
        if (!p.order) {
          rows = make_int4((int)pos, (int)pos + 1, (int)pos + 2, (int)pos + 3);
        } else if (pos + 3 < p.n_rows && (reinterpret_cast<uintptr_t>(p.order) & 15) == 0) {
          rows = __ldg(reinterpret_cast<const int4*>(p.order + pos));
        } else {
          // the last tile's line may run past the end of `order`: read only what exists
          rows.x = pos + 0 < p.n_rows ? __ldg(p.order + pos + 0) : -1;
          rows.y = pos + 1 < p.n_rows ? __ldg(p.order + pos + 1) : -1;
          rows.z = pos + 2 < p.n_rows ? __ldg(p.order + pos + 2) : -1;
          rows.w = pos + 3 < p.n_rows ? __ldg(p.order + pos + 3) : -1;
        }
        if (pos + 0 >= p.n_rows) rows.x = -1;
        if (pos + 1 >= p.n_rows) rows.y = -1;
        if (pos + 2 >= p.n_rows) rows.z = -1;
        if (pos + 3 >= p.n_rows) rows.w = -1;
      } else if (t.kind == 2 && t.my_j >= 0) {
        rows = __ldg(reinterpret_cast<const int4*>(map.tmap + (t.tile * map.K + k_first + t.my_j) * (int64_t)kTileM) + lane);
      }
      return rows;
    };
    bool ok = true;
    auto issue = [&](const Task& t, const int4& rows) {
      if (t.kind == 1) {
        ok = mbar_wait_warp(smem_u32(&ctl->a_empty[t.slot]), t.parity ^ 1u, abort_flag, 35, lane);
        if (!ok) return;
        const uint32_t bar = smem_u32(&ctl->a_full[t.slot]);
        const uint32_t slot_base = a_ring + (uint32_t)t.slot * (uint32_t)p.a_slot_bytes;
        if (lane == 0) {
          if (a_mine) mbar_arrive_expect_tx(bar, (uint32_t)a_mine * kABlockBytes); else mbar_arrive(bar);
          if (p.dense_tiles)
            for (int b = pw; b < a_blocks; b += kProducerWarps)
              tma_load_2d(slot_base + (uint32_t)b * kABlockBytes, &tile_box_desc, bar, tile_col0 + b * per_line,
                          (int)(t.tile * kTileM));
        }
        __syncwarp();
        if (!p.dense_tiles)
          for (int b = pw; b < a_blocks; b += kProducerWarps)
            tma_gather4(slot_base + (uint32_t)b * kABlockBytes + (uint32_t)lane * 512u, tile_desc, bar, tile_col0 + b * per_line,
                        rows.x, rows.y, rows.z, rows.w);
      } else {
        ok = mbar_wait_warp(smem_u32(&ctl->b_empty[t.slot]), t.parity ^ 1u, abort_flag, 36, lane);
        if (!ok) return;
        const uint32_t bar = smem_u32(&ctl->b_full[t.slot]);
        const uint32_t stage = b_ring + (uint32_t)t.slot * quad_bytes + (uint32_t)(p.quad == 1 ? 0 : pw) * (uint32_t)p.b_slot_bytes;
        if (lane == 0) {
          if (t.my_j >= 0) mbar_arrive_expect_tx(bar, (uint32_t)b_blocks * kABlockBytes); else mbar_arrive(bar);
        }
        __syncwarp();
        if (t.my_j >= 0) {
          for (int b = 0; b < b_blocks; ++b)
            tma_gather4(stage + (uint32_t)b * kABlockBytes + (uint32_t)lane * 512u, gath_desc, bar, gath_col0 + b * per_line, rows.x,
                        rows.y, rows.z, rows.w);
        }
      }
    };
    Cursor fetch = cursor();
    Task queued[kAhead];
    int4 queued_rows[kAhead];
#pragma unroll
    for (int d = 0; d < kAhead; ++d) {
      queued[d] = next(fetch);
      queued_rows[d] = load_rows(queued[d]);
    }
    while (queued[0].kind != 0 && ok) {
      issue(queued[0], queued_rows[0]);
#pragma unroll
      for (int d = 0; d + 1 < kAhead; ++d) {
        queued[d] = queued[d + 1];
        queued_rows[d] = queued_rows[d + 1];
      }
      queued[kAhead - 1] = next(fetch);
      queued_rows[kAhead - 1] = load_rows(queued[kAhead - 1]);
    }
    }
  } else if (warp == kMmaWarp) {
    // =============================================================== MMA issuer
    if (lane == 0) {
      int a_slot = 0, b_slot = 0;
      uint32_t a_phase = 0, b_phase = 0;
      uint32_t touched = 0;
      bool ok = true;
      const int rows_per_step = 32 / p.esize;                  // reduction rows per MMA (16 or 8)
      const int ksteps = kTileM / rows_per_step;
      const uint32_t step_bytes = (uint32_t)rows_per_step * 128u;
      const uint32_t sbo = base32 ? 512u : 1024u, layout = base32 ? 1u : 2u;
      const uint32_t idesc = p.idesc_base | ((uint32_t)(p.ci_blk >> 3) << 17);
      const uint64_t desc_hi = smem_desc(0u, kABlockBytes, sbo, layout);
      uint32_t m_next = tile_begin < tile_end ? tile_mask(tile_begin) : 0u;
      for (int64_t tile = tile_begin; tile < tile_end && ok; tile += tile_step) {
        uint32_t m = m_next;
        if (tile + tile_step < tile_end) m_next = tile_mask(tile + tile_step);
        if (!m) continue;
        ok = mbar_wait(smem_u32(&ctl->a_full[a_slot]), a_phase, abort_flag, 37);
        if (!ok) break;
        const uint32_t a_lo = (a_ring + (uint32_t)a_slot * (uint32_t)p.a_slot_bytes) >> 4;
        while (m && ok) {
          ok = mbar_wait(smem_u32(&ctl->b_full[b_slot]), b_phase, abort_flag, 38);
          if (!ok) break;
          tc_fence_after();
          for (int q = 0; q < p.quad && m; ++q) {
            const int j = __ffs(m) - 1;
            m &= m - 1;
            const uint32_t b_lo = (b_ring + (uint32_t)b_slot * quad_bytes + (uint32_t)q * (uint32_t)p.b_slot_bytes) >> 4;
            const uint32_t d_addr = tmem_base + (uint32_t)(j * p.ci_blk);
            const uint32_t first = ((touched >> j) & 1u) ? 1u : 0u;
            for (int ks = 0; ks < ksteps; ++ks) {
              const uint64_t da = desc_hi | (uint64_t)((p.swap ? b_lo : a_lo) + ks * (step_bytes >> 4));   // dY rows (M)
              const uint64_t db = desc_hi | (uint64_t)((p.swap ? a_lo : b_lo) + ks * (step_bytes >> 4));   // X rows (N)
              if (p.esize == 2)
                mma_f16(d_addr, da, db, idesc, ks == 0 ? first : 1u);
              else
                mma_tf32(d_addr, da, db, idesc, ks == 0 ? first : 1u);
            }
            touched |= 1u << j;
          }
          mma_commit(smem_u32(&ctl->b_empty[b_slot]));
          if (++b_slot == p.b_slots) {
            b_slot = 0;
            b_phase ^= 1u;
          }
        }
        mma_commit(smem_u32(&ctl->a_empty[a_slot]));
        if (++a_slot == p.a_slots) {
          a_slot = 0;
          a_phase ^= 1u;
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
    bool ok = mbar_wait(smem_u32(&ctl->acc_full), 0u, abort_flag, 39, 512);
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

}  // namespace tc
}  // namespace st
