// Dispatch fused into the grouped GEMM that consumes the dispatched rows.
//
// The reference hands the dispatched rows to the host framework's GEMM only after the dispatch
// kernel's exit barrier (moonep/dispatch.py:687-691, README.md:45): the all-to-all is never
// overlapped with the expert math.  Here the GEMM kernel itself carries the all-to-all: every
// GEMM CTA has one extra "copy warp" that streams this rank's token rows through a small
// shared-memory ring with 1-D bulk copies (global -> shared -> peer global over NVLink), straight
// into their expert-grouped rows on the destination ranks, while the CTA's other warps run the
// tensor-core pipeline on the rows that have already ARRIVED from the peers.  No SM is given up
// to communication and no barrier separates the two.
//
// Arrival tracking.  Each rank owns one int32 counter per 128-row block of its row buffer (ARRIVE
// in the meta chunk).  A sender adds the number of row parts it has completed to the destination
// block's counter with red.release.sys after cp.async.bulk.wait_group has reported the copies
// complete; the GEMM's TMA producer polls the counter of the block it is about to load with
// ld.acquire.sys (bounded), then fences the async proxy and loads.  A block expects 128 rows x
// `nsplit` parts: real rows arrive from their source ranks, padding rows are zeroed by the
// owner's own copy warps and counted the same way.  In this mode every (token, k) entry travels
// as a real row: a duplicate of a token on one destination rank is not expanded locally, because
// nothing may sit between arrival and use (1.5x the NVLink bytes at the benchmark shape, hidden
// under the GEMM).
//
// Order.  Entries are sent in the planner's `send_order` (by local expert index, then by home
// rank rotated by the sender's rank, then by token), in windows of gridDim.x * 8 entries of which
// CTA c takes 8 consecutive ones: 8 consecutive entries are 8 consecutive rows of one
// destination block, so their completions are signalled with ONE release.  Every destination
// thus receives its group j from all sources at about the same time, and the GEMM walks its
// groups in that same order: after the first group it is never starved.
#pragma once
#include <cstdint>

#include "common/layout.h"
#include "device/sync.cuh"
#include "device/tma.cuh"

namespace mep {

constexpr int FD_PART_CAP = 7168;   // bytes of a ring stage; a row travels in nsplit equal parts
constexpr int FD_LA = 2;            // loads issued ahead of the store being issued
constexpr int FD_RUN = 8;           // consecutive entries per CTA and window

struct FusedDispatch {
  // ---- consumer side: the GEMM producer waits for the rows of a tile -----------------------
  const int32_t* arrive;   // this rank's ARRIVE counters (null: rows are already in place)
  int expect;              // 128 * nsplit
  // ---- sender side (x == null: this launch sends nothing) -----------------------------------
  const uint8_t* x;        // [S][row_bytes] this rank's token rows
  const float* w;          // [N] route weights, or null
  const int32_t* dst;      // [N] plan destinations (negative = duplicate of the same token)
  const int32_t* order;    // [N] sending order
  const int32_t* zero_fill;  // [2*epn][2] padding rows of this rank
  uint8_t* hidden;         // symmetric row buffer, chunk of rank 0
  int32_t* meta;           // symmetric meta buffer, chunk of rank 0
  long long hidden_stride_bytes;   // between consecutive ranks' chunks
  long long meta_stride;           // int32 elements
  long long weights_off, link_off, src_off, arrive_off, NvS;
  int N, K, epn, rank, R, fresh, row_bytes, nsplit;
};

// One warp.  `ring` holds NST stages of FD_PART_CAP bytes, `full` NST mbarriers (initialised with
// count 1 by the caller), `slots` 2 * NST words of scratch.  `wait_full(bar, parity)` is the
// caller's bounded mbarrier wait (returns false after a timeout or an abort).
template <int NST, class WaitFn>
__device__ __forceinline__ void fused_dispatch_copy_warp(const FusedDispatch& d, uint8_t* ring,
                                                         uint64_t* full, unsigned long long* slots,
                                                         int cta, int n_cta, WaitFn wait_full) {
  static_assert(NST > FD_LA + 1, "the ring must hold the loads in flight and at least one store");
  const int lane = threadIdx.x & 31;
  const int part_bytes = d.row_bytes / d.nsplit;
  int32_t* my_meta = d.meta + (size_t)d.rank * d.meta_stride;
  uint8_t* my_rows = d.hidden + (size_t)d.rank * d.hidden_stride_bytes;

  // ---- padding rows of MY buffer: zeroed with plain stores, counted like arrivals ------------
  for (int g0 = 0; g0 < 2 * d.epn; g0 += 32) {
    const int g = g0 + lane;
    int first_l = 0, n_l = 0;
    if (g < 2 * d.epn) { first_l = d.zero_fill[2 * g]; n_l = d.zero_fill[2 * g + 1]; }
    for (int j = 0; j < 32 && g0 + j < 2 * d.epn; ++j) {
      const int first = __shfl_sync(0xffffffffu, first_l, j);
      const int n = __shfl_sync(0xffffffffu, n_l, j);
      if (n <= 0 || first < 0 || (long long)first + n > d.NvS) continue;
      for (int r = first + cta; r < first + n; r += n_cta) {
        uint4* row = reinterpret_cast<uint4*>(my_rows + (size_t)r * d.row_bytes);
        for (int v = lane; v < d.row_bytes / 16; v += 32) row[v] = make_uint4(0, 0, 0, 0);
        if (lane == 0) {
          if (d.w != nullptr) my_meta[d.weights_off + r] = 0;
          if (d.fresh) { my_meta[d.link_off + r] = LINK_NONE; my_meta[d.src_off + r] = -1; }
        }
        __syncwarp();
        if (lane == 0) red_release_sys_add(my_meta + d.arrive_off + (r >> 7), d.nsplit);
      }
    }
  }

  // ---- my entries: windows of n_cta * FD_RUN positions of the sending order -------------------
  const long long win = (long long)n_cta * FD_RUN;
  const long long n_win = (d.N + win - 1) / win;
  long long n_ent = 0;     // entries of this CTA (a prefix of its window slots)
  if (n_win > 0) {
    const long long last0 = (n_win - 1) * win + (long long)cta * FD_RUN;
    long long tail = d.N - last0;
    tail = tail < 0 ? 0 : (tail > FD_RUN ? FD_RUN : tail);
    n_ent = (n_win - 1) * FD_RUN + tail;
  }
  const long long n_units = n_ent * d.nsplit;
  // lane 0's pipeline state
  unsigned long long pend_ctr = 0ull;
  int pend_cnt = 0;
  bool ok = true;
  auto flush = [&]() {
    if (pend_cnt > 0) {
      fence_proxy_async();
      red_release_sys_add(reinterpret_cast<int32_t*>(pend_ctr), pend_cnt);
      pend_cnt = 0;
    }
  };
  auto completed = [&](int stage) {       // the unit that used `stage` has fully landed
    const unsigned long long ctr = slots[NST + stage];
    if (ctr == 0ull) return;              // a unit that sent nothing
    if (ctr != pend_ctr) { flush(); pend_ctr = ctr; }
    ++pend_cnt;
  };
  auto store_unit = [&](long long v) {    // unit v's load has been issued: wait for it, send it on
    const int sv = (int)(v % NST);
    if (!wait_full(&full[sv], (uint32_t)(v / NST) & 1u)) { ok = false; return; }
    bulk_s2g(reinterpret_cast<void*>(slots[sv]), ring + (size_t)sv * FD_PART_CAP, (uint32_t)part_bytes);
    bulk_commit();
  };

  for (long long u0 = 0; u0 < n_units; u0 += 32) {
    // ---- all lanes: decode 32 units (entry -> source row, destination row, counter) ----------
    const long long u = u0 + lane;
    unsigned long long src = 0ull, dstp = 0ull, ctr = 0ull;
    if (u < n_units) {
      const long long ie = u / d.nsplit;
      const int part = (int)(u - ie * d.nsplit);
      const long long pos = (ie / FD_RUN) * win + (long long)cta * FD_RUN + (ie % FD_RUN);
      const int entry = d.order[pos];
      if ((unsigned)entry < (unsigned)d.N) {
        const int dv = d.dst[entry];
        const long long raw = dv >= 0 ? dv : -(long long)dv - 1;
        const long long dr = raw / d.NvS, row = raw - dr * d.NvS;
        if (dr < d.R) {
          const int tok = entry / d.K;
          src = (unsigned long long)(d.x + (size_t)tok * d.row_bytes + (size_t)part * part_bytes);
          dstp = (unsigned long long)(d.hidden + (size_t)dr * d.hidden_stride_bytes +
                                      (size_t)row * d.row_bytes + (size_t)part * part_bytes);
          int32_t* peer_meta = d.meta + (size_t)dr * d.meta_stride;
          ctr = (unsigned long long)(peer_meta + d.arrive_off + (row >> 7));
          if (part == 0 && d.w != nullptr) peer_meta[d.weights_off + row] = __float_as_int(d.w[entry]);
        }
      }
    }
    __syncwarp();     // the weight stores above are ordered before lane 0's releases below
    // ---- lane 0: feed the units through the ring ----------------------------------------------
    const int nb = (int)((n_units - u0) < 32 ? (n_units - u0) : 32);
    for (int l = 0; l < nb; ++l) {
      const unsigned long long s_src = __shfl_sync(0xffffffffu, src, l);
      const unsigned long long s_dst = __shfl_sync(0xffffffffu, dstp, l);
      const unsigned long long s_ctr = __shfl_sync(0xffffffffu, ctr, l);
      if (lane == 0 && ok) {
        const long long uu = u0 + l;
        const int s = (int)(uu % NST);
        if (uu >= NST) {
          // units 0 .. uu-FD_LA-1 have been committed; all but the most recent NST-FD_LA-1 of
          // those groups are complete after this wait, i.e. every unit up to uu-NST
          bulk_wait<NST - FD_LA - 1>();
          completed(s);
        }
        if (s_src != 0ull) {
          slots[s] = s_dst;
          slots[NST + s] = s_ctr;
          mbar_expect_tx(&full[s], (uint32_t)part_bytes);
          bulk_g2s(ring + (size_t)s * FD_PART_CAP, reinterpret_cast<const void*>(s_src),
                   (uint32_t)part_bytes, &full[s]);
        } else {
          // an entry that failed its index checks: keep the ring in phase, send nothing
          slots[s] = 0ull;
          slots[NST + s] = 0ull;
          mbar_arrive(&full[s]);
        }
        if (uu >= FD_LA) {
          const long long v = uu - FD_LA;
          if (slots[v % NST] != 0ull) store_unit(v);
          else { if (!wait_full(&full[v % NST], (uint32_t)(v / NST) & 1u)) ok = false; bulk_commit(); }
        }
      }
    }
  }
  if (lane == 0) {
    if (ok) {
      for (long long v = n_units > FD_LA ? n_units - FD_LA : 0; v < n_units && ok; ++v) {
        if (slots[v % NST] != 0ull) store_unit(v);
        else { if (!wait_full(&full[v % NST], (uint32_t)(v / NST) & 1u)) ok = false; bulk_commit(); }
      }
    }
    bulk_wait<0>();        // also on an abort: nothing of this thread stays in flight
    if (ok) {
      for (long long v = n_units > NST ? n_units - NST : 0; v < n_units; ++v) completed((int)(v % NST));
      flush();
    }
  }
  __syncwarp();
}

}  // namespace mep
