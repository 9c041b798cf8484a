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
// block's counter (a system-scope reduction) after cp.async.bulk.wait_group has reported the
// copies complete; watcher lanes of the GEMM's producer warp poll the counters of the group the
// producer is about to load with ld.acquire.sys (bounded, with back-off), the producer then
// fences the async proxy and loads.  A block expects 128 rows x
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
  int debug;   // timing experiments, compiled in only with -DMEP_GEMM_EXPERIMENTS (see fd_dbg)
};

// Timing experiments (results are wrong when set): 1 = arrival signals without the release fence,
// 4 = the copy warp issues no stores, 8 = neither loads nor stores.  A constant false in a normal build.
#ifdef MEP_GEMM_EXPERIMENTS
__device__ __forceinline__ bool fd_dbg(const FusedDispatch& d, int bit) { return (d.debug & bit) != 0; }
#else
__device__ __forceinline__ constexpr bool fd_dbg(const FusedDispatch&, int) { return false; }
#endif

// One warp.  `ring` holds NST stages of FD_PART_CAP bytes and `full` NST mbarriers (initialised
// with count 1 by the caller): lane i < NST owns stage i.  The warp works in lockstep rounds of
// NST units (a unit is one part of one row): every owning lane loads its unit into its stage,
// waits for it, stores it to the destination, waits for that store to complete, and the lanes
// whose units share a destination counter signal it with ONE release.  All per-unit scalar work
// is thereby spread over NST lanes; NST * 7 KB per round trip of (load + remote store) latency
// keeps 148 CTAs well above the NVLink rate.  `wait_full(bar, parity)` is the caller's bounded
// mbarrier wait (false after a timeout or an abort).
template <int NST, class WaitFn>
__device__ __forceinline__ void fused_dispatch_copy_warp(const FusedDispatch& d, uint8_t* ring,
                                                         uint64_t* full, int cta, int n_cta,
                                                         WaitFn wait_full) {
  static_assert(NST >= 1 && NST <= 32, "one lane per ring stage");
  const int lane = threadIdx.x & 31;
  const int part_bytes = d.row_bytes / d.nsplit;
  int32_t* my_meta = d.meta + (size_t)d.rank * d.meta_stride;
  uint8_t* my_rows = d.hidden + (size_t)d.rank * d.hidden_stride_bytes;

  // ---- padding rows of MY buffer: zeroed with plain stores, counted like arrivals ------------
  // Done in slices between the batches of entries below: the padding of local group j is needed
  // when the GEMM reaches group j, which is when the senders reach round j of the sending order,
  // and doing all of it up front would only delay the first groups.
  auto do_pads = [&](int g_from, int g_to) {
    for (int g0 = g_from; g0 < g_to; g0 += 32) {
      const int g = g0 + lane;
      int first_l = 0, n_l = 0;
      if (g < g_to) { first_l = d.zero_fill[2 * g]; n_l = d.zero_fill[2 * g + 1]; }
      for (int j = 0; j < 32 && g0 + j < g_to; ++j) {
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
  };

  // ---- my entries: windows of n_cta * FD_RUN positions of the sending order -------------------
  const int win = n_cta * FD_RUN;
  const int n_win = (d.N + win - 1) / win;
  int n_ent = 0;           // entries of this CTA (a prefix of its window slots)
  if (n_win > 0) {
    int tail = d.N - ((n_win - 1) * win + cta * FD_RUN);
    tail = tail < 0 ? 0 : (tail > FD_RUN ? FD_RUN : tail);
    n_ent = (n_win - 1) * FD_RUN + tail;
  }
  const int n_units = n_ent * d.nsplit;
  constexpr int PER_BATCH = 32 / NST * NST;        // units decoded at once, a multiple of NST
  const int NvS = (int)d.NvS;
  uint8_t* my_stage = ring + (size_t)(lane < NST ? lane : 0) * FD_PART_CAP;
  uint64_t* my_full = &full[lane < NST ? lane : 0];
  uint32_t parity = 0;     // of my_full: flips every time this lane has used its stage
  bool ok = true;
  const int n_batches = (n_units + PER_BATCH - 1) / PER_BATCH;
  int pad_g = d.epn < 2 ? d.epn : 2;       // local groups whose padding is done
  int batch = 0;
  do_pads(0, pad_g);

  for (int u0 = 0; u0 < n_units && ok; u0 += PER_BATCH, ++batch) {
    {   // keep the padding two groups ahead of the senders' position in the sending order
      int upto = (int)(((long long)(batch + 1) * d.epn) / n_batches) + 2;
      upto = upto > d.epn ? d.epn : upto;
      if (upto > pad_g) { do_pads(pad_g, upto); pad_g = upto; }
    }
    // ---- all lanes: decode up to PER_BATCH units (entry -> source, destination, counter) -----
    const int u = u0 + lane;
    unsigned long long src = 0ull, dstp = 0ull, ctr = 0ull;
    if (lane < PER_BATCH && u < n_units) {
      const int ie = u / d.nsplit;
      const int part = u - ie * d.nsplit;
      const int pos = (ie / FD_RUN) * win + cta * FD_RUN + (ie % FD_RUN);
      const int entry = d.order[pos];
      if ((unsigned)entry < (unsigned)d.N) {
        const int dv = d.dst[entry];
        const int raw = dv >= 0 ? dv : -dv - 1;
        const int dr = raw / NvS, row = raw - dr * NvS;
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
    // The route weights above are plain stores to the peers; ONE system-scope fence per batch (by
    // lane 0, made cumulative over the warp by the barriers around it) orders them before every
    // arrival signal of this batch.  The rows themselves need no fence: a signal is only issued
    // after cp.async.bulk.wait_group has reported the row's copy complete, so a relaxed reduction
    // is enough per round.  (A release per round cost a full drain of the SM's stores each time
    // and made the copy warp, not NVLink, the limit.)
    __syncwarp();
    if (lane == 0 && !fd_dbg(d, 1)) fence_sys();
    __syncwarp();
    // ---- rounds of NST units: lane i < NST moves unit u0 + r0 + i through stage i ---------------
    for (int r0 = 0; r0 < PER_BATCH && u0 + r0 < n_units; r0 += NST) {
      const int from = r0 + (lane < NST ? lane : 0);
      const unsigned long long s_src = __shfl_sync(0xffffffffu, src, from);
      const unsigned long long s_dst = __shfl_sync(0xffffffffu, dstp, from);
      const unsigned long long s_ctr = __shfl_sync(0xffffffffu, ctr, from);
      const bool act = lane < NST && u0 + from < n_units && s_src != 0ull;
      bool sent = false;
      if (act) {
        if (!fd_dbg(d, 8)) {
          mbar_expect_tx(my_full, (uint32_t)part_bytes);
          bulk_g2s(my_stage, reinterpret_cast<const void*>(s_src), (uint32_t)part_bytes, my_full);
          sent = wait_full(my_full, parity);
          parity ^= 1u;
          if (sent && !fd_dbg(d, 4)) {
            bulk_s2g(reinterpret_cast<void*>(s_dst), my_stage, (uint32_t)part_bytes);
            bulk_commit();
            bulk_wait<0>();          // complete, not just read: the rows may now be announced
          }
        } else {
          sent = true;
        }
        if (sent && !fd_dbg(d, 1)) fence_proxy_async();
      }
      // a load that never landed ends this warp's work (the status is already recorded)
      if (__any_sync(0xffffffffu, act && !sent)) ok = false;
      // lanes whose units share a destination counter announce them with one release
      const unsigned long long key = (act && sent) ? s_ctr : 0ull;
      const unsigned grp = __match_any_sync(0xffffffffu, key);
      if (key != 0ull && lane == __ffs(grp) - 1) {
        red_relaxed_sys_add(reinterpret_cast<int32_t*>(key), __popc(grp));
      }
      if (!ok) break;
    }
  }
  if (lane < NST) bulk_wait<0>();
  __syncwarp();
  do_pads(pad_g, 2 * d.epn);               // the rest, and the prefetch-slot groups (consumed last)
}

}  // namespace mep
