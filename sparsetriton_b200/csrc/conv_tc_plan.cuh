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
  // bit 12 end of super tile (no data)
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
      uint32_t users, fresh;
      int slot;
      uint32_t parity;
      bool marker, valid;
    };
    Item pend{0, 0, 0u, 0u, 0, 0u, false, false};
    int4 pend_idx = make_int4(-1, -1, -1, -1);

    auto run = [&](const Item& d, const int4& idx) {
      ok = mbar_wait_warp(smem_u32(&ctl->empty[d.slot]), d.parity ^ 1u, abort_flag, 31, lane);
      if (!ok) return;
      const uint32_t bar = smem_u32(&ctl->full[d.slot]);
      const uint32_t slot_base = base + (uint32_t)d.slot * (uint32_t)p.slot_bytes;
      const bool copy_rows = !d.marker && !(p.dbg & 4) && ((d.users >> pw) & 1u);
      if (lane == 0) {
        // Every producer warp arrives on every slot, announcing the bytes of its own copies first (a
        // copy that completed before its bytes were announced would drive the count negative).
        const bool copy_w = pw == 0 && !d.marker && !(p.dbg & 16);
        if (pw == 0) {
          const int valid_bytes = d.marker ? 0 : min(128, red_bytes - d.kb * 128);
          ctl->info[d.slot] = d.users | (d.fresh << 4) | ((uint32_t)(valid_bytes >> 5) << 8) | (d.marker ? 0x1000u : 0u);
        }
        const uint32_t bytes = (copy_w ? w_bytes : 0u) + (copy_rows ? (uint32_t)kABlockBytes : 0u);
        if (bytes) mbar_arrive_expect_tx(bar, bytes); else mbar_arrive(bar);
        if (copy_w) {
          if (p.b_mn_major) {
            const int n_cb = (w_col_bytes + 127) >> 7;
            for (int cb = 0; cb < n_cb; ++cb)
              tma_load_2d(slot_base + (uint32_t)(cb * kr * 128), &w_desc, bar, cb * kr, d.k * p.w_rows + d.kb * kr);
          } else {
            tma_load_2d(slot_base, &w_desc, bar, d.kb * kr, d.k * p.w_rows);
          }
        }
      }
      __syncwarp();
      if (copy_rows)
        tma_gather4(slot_base + (uint32_t)p.w_slot_bytes + (uint32_t)pw * kABlockBytes + (uint32_t)lane * 512u, &in_desc,
                    bar, d.kb * kr, idx.x, idx.y, idx.z, idx.w);
    };
    // Queue one item: its indices are loaded now and it is issued when the next one is queued, so the
    // load overlaps the previous item's wait and copies.
    auto emit = [&](int64_t tile0, int k, int kb, uint32_t users, uint32_t fresh, bool marker, bool zeros) {
      int4 idx = make_int4(-1, -1, -1, -1);
      if (!marker && !zeros && ((users >> pw) & 1u))
        idx = __ldg(reinterpret_cast<const int4*>(map.tmap + ((tile0 + pw) * map.K + k) * (int64_t)kTileM) + lane);
      if (pend.valid && ok) run(pend, pend_idx);
      pend = Item{k, kb, users, fresh, slot, phase, marker, true};
      pend_idx = idx;
      if (++slot == p.n_slots) {
        slot = 0;
        phase ^= 1u;
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
      for (int64_t st_i = blockIdx.x; st_i < p.n_super && ok; st_i += gridDim.x) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[buf]), acc_phase[buf] ^ 1u, abort_flag, 32);
        if (!ok) break;
        tc_fence_after();
        for (;;) {
          ok = mbar_wait(smem_u32(&ctl->full[slot]), phase, abort_flag, 33);
          if (!ok) break;
          const uint32_t info = ctl->info[slot];
          tc_fence_after();
          if (!(info & 0x1000u) && !(p.dbg & 2)) {
            const uint32_t slot_base = base + (uint32_t)slot * (uint32_t)p.slot_bytes;
            const uint32_t w_lo = slot_base >> 4;
            const int ksteps = (int)((info >> 8) & 15u);
#pragma unroll
            for (int s = 0; s < kMaxSub; ++s) {
              if (!((info >> s) & 1u)) continue;
              const uint32_t a_lo = (slot_base + (uint32_t)p.w_slot_bytes + (uint32_t)s * kABlockBytes) >> 4;
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
          mma_commit(smem_u32(&ctl->empty[slot]));
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
        for (int c0 = 0; c0 < p.c_acc && !(p.dbg & 128); c0 += 32) {
          uint32_t v[32];
          if (p.c_acc - c0 >= 32) {
            tmem_ld32(t_row + c0, v);
            tmem_ld_wait();
            if (row < p.n_rows && !(p.dbg & 64)) store_cols<32>(out_row, c0, p.out_kind, v);
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

}  // namespace tc
}  // namespace st
