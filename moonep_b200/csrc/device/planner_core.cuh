// Shared device code of the planner: the parameter block, warp arg-max helpers and the
// single-CTA solver (steps 1-4 of the algorithm).  Included by the planner kernel and by the
// entry point that runs the planner without allocating memory.
#pragma once
#include <cuda_runtime.h>

#include "common/layout.h"
#include "device/sync.cuh"

namespace mep {

struct PlanParams {
  SyncCtx sync;
  int E, epn, S, K, token_padding;
  int64_t N, NvS;
  int64_t tpe_off, link_off, src_off;
  const int32_t* topk;      // [Rv][N]
  const int32_t* tpe;       // [Rv][E]
  int32_t* dst;             // [Rv][N]
  int32_t* cu_seqlens;      // [Rv][2epn]
  int32_t* zero_fill;       // [Rv][2epn][2]
  int32_t* etc;             // [Rv][R][epn]
  int32_t* remote_stats;    // [Rv][2]
  int32_t* scratch;         // [Rv][scratch_ints]
  int64_t scratch_ints;
  // Fused dispatch -> GEMM path (both optional; null / 0 when unused).
  // send_order [Rv][N]: this rank's entries in the order in which its copy warps send them:
  // by local expert index first (round j = e % epn), inside a round by home rank starting at
  // the sender's own, then by token.  Every destination therefore receives its group j from all
  // sources at about the same time, which is the order in which its GEMM consumes the groups.
  int32_t* send_order;
  int64_t arrive_off;       // ARRIVE counters in the meta chunk, cleared before the exchange
  int n_arrive;
};

// Position of expert e in the sending order of `rank` (see PlanParams::send_order).
MEP_HD int send_perm(int e, int epn, int R, int rank) {
  const int h = e / epn, j = e - h * epn;
  int rot = h - rank;
  if (rot < 0) rot += R;
  return j * R + rot;
}

constexpr int PLAN_THREADS = 512;
constexpr int PLAN_WARPS = PLAN_THREADS / 32;

// (value, index) arg-max with ties to the smaller index, across a warp.
__device__ __forceinline__ void warp_argmax(int& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    int ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}
__device__ __forceinline__ void warp_argmin(int& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    int ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov < v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// Steps 1-4 of the algorithm, executed by CTA 0 of every rank.
static __device__ void plan_solve(const PlanParams& p, int rank, const int32_t* tbl /*[R][E]*/,
                           int32_t* smem) {
  const int R = p.sync.R, E = p.E, epn = p.epn;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y;
  int32_t* scratch = p.scratch + (size_t)vr * p.scratch_ints;
  int32_t* tpe_cumsum = scratch;
  int32_t* alloc = scratch + (size_t)R * E;
  int32_t* alloc_cumsum = scratch + (size_t)2 * R * E;
  int32_t* expert_off = scratch + (size_t)3 * R * E;
  int32_t* etc = p.etc + (size_t)vr * R * epn;

  int32_t* count = smem;                 // [E]
  int32_t* remaining = smem + E;         // [E]
  int32_t* balance = smem + 2 * E;       // [R]
  int32_t* recv_from = balance + R;      // [R]
  int32_t* recv_amt = recv_from + R;     // [R]
  int32_t* stat1 = recv_amt + R;         // [R]
  int32_t* quotas = stat1 + R;           // [PLAN_WARPS][R]

  // 1. prefix over source ranks, per-expert totals
  for (int e = tid; e < E; e += PLAN_THREADS) {
    int run = 0;
    for (int r = 0; r < R; ++r) {
      run += tbl[(size_t)r * E + e];
      tpe_cumsum[(size_t)r * E + e] = run;
    }
    count[e] = run;
    remaining[e] = run;
  }
  for (int i = tid; i < R; i += PLAN_THREADS) { recv_from[i] = -1; recv_amt[i] = 0; stat1[i] = 0; }
  for (int i = tid; i < R * epn; i += PLAN_THREADS) etc[i] = -1;
  for (size_t i = tid; i < (size_t)R * E; i += PLAN_THREADS) expert_off[i] = 0;
  __syncthreads();
  const int CAP = (int)p.N;
  for (int h = warp; h < R; h += PLAN_WARPS) {
    int s = 0;
    for (int j = lane; j < epn; j += 32) s += count[h * epn + j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) balance[h] = s - CAP;
  }
  for (size_t i = tid; i < (size_t)E * R; i += PLAN_THREADS) {
    int e = (int)(i / R), d = (int)(i % R);
    alloc[i] = (d == e / epn) ? count[e] : 0;
  }
  __syncthreads();

  // 2. receiver selection (one warp; at most R-1 rounds)
  if (warp == 0) {
    for (int round = 0; round < R; ++round) {
      int mxv = INT32_MIN, mxi = INT32_MAX, mnv = INT32_MAX, mni = INT32_MAX;
      for (int r = lane; r < R; r += 32) {
        int b = balance[r];
        if (b > mxv) { mxv = b; mxi = r; }
        if (b < mnv) { mnv = b; mni = r; }
      }
      warp_argmax(mxv, mxi);
      warp_argmin(mnv, mni);
      if (mxv <= 0) break;
      if (lane == 0) {
        int move = -mnv;
        recv_from[mni] = mxi;
        recv_amt[mni] = move;
        balance[mxi] = mxv - move;
        balance[mni] = 0;
      }
      __syncwarp();
    }
  }
  __syncthreads();

  // 3. expert selection, one warp per home group
  for (int h = warp; h < R; h += PLAN_WARPS) {
    int32_t* q = quotas + warp * R;
    for (int d = lane; d < R; d += 32) q[d] = recv_from[d] == h ? recv_amt[d] : 0;
    __syncwarp();
    for (int guard = 0; guard < epn + R + 2; ++guard) {
      int qv = INT32_MIN, qi = INT32_MAX;
      for (int d = lane; d < R; d += 32)
        if (q[d] > qv) { qv = q[d]; qi = d; }
      warp_argmax(qv, qi);
      if (qv <= 0) break;
      int rv = INT32_MIN, ri = INT32_MAX;
      for (int j = lane; j < epn; j += 32) {
        int v = remaining[h * epn + j];
        if (v > rv) { rv = v; ri = j; }
      }
      warp_argmax(rv, ri);
      int take = min(rv, qv);
      if (take <= 0) break;  // cannot happen for consistent inputs
      if (lane == 0) {
        int e = h * epn + ri;
        alloc[(size_t)e * R + qi] += take;
        alloc[(size_t)e * R + h] -= take;
        remaining[e] -= take;
        q[qi] -= take;
      }
      __syncwarp();
    }
  }
  __syncthreads();

  // 4a. prefix over destination ranks
  for (int e = tid; e < E; e += PLAN_THREADS) {
    int run = 0;
    for (int d = 0; d < R; ++d) {
      run += alloc[(size_t)e * R + d];
      alloc_cumsum[(size_t)e * R + d] = run;
    }
  }
  // 4b. layout of every destination rank, one warp per rank
  const int tp = p.token_padding;
  for (int d = warp; d < R; d += PLAN_WARPS) {
    const int h = recv_from[d];
    int nremote = 0;
    if (h >= 0) {
      for (int j0 = 0; j0 < epn; j0 += 32) {
        int j = j0 + lane;
        bool has = j < epn && alloc[(size_t)(h * epn + j) * R + d] > 0;
        unsigned m = __ballot_sync(0xffffffffu, has);
        if (has) etc[d * epn + nremote + __popc(m & ((1u << lane) - 1))] = h * epn + j;
        nremote += __popc(m);
      }
    }
    __syncwarp();
    if (lane == 0) {
      if (h >= 0) atomicAdd(&stat1[h], nremote);
      if (d == rank) p.remote_stats[(size_t)vr * 2] = nremote;
    }
    int carry = 0;
    for (int g0 = 0; g0 < 2 * epn; g0 += 32) {
      int g = g0 + lane;
      int eid = -1, cnt = 0;
      if (g < epn) {
        eid = d * epn + g;
      } else if (g < 2 * epn && g - epn < nremote) {
        eid = etc[d * epn + (g - epn)];
      }
      if (eid >= 0) cnt = alloc[(size_t)eid * R + d];
      int padded = cnt > 0 ? (cnt + tp - 1) / tp * tp : 0;
      int incl = padded;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int end = carry + incl, start = end - padded;
      if (g < 2 * epn) {
        if (cnt > 0) expert_off[(size_t)d * E + eid] = start;
        if (d == rank) {
          p.cu_seqlens[(size_t)vr * 2 * epn + g] = end;
          int npad = padded - cnt;
          p.zero_fill[((size_t)vr * 2 * epn + g) * 2 + 0] = (cnt > 0 && npad > 0) ? start + cnt : 0;
          p.zero_fill[((size_t)vr * 2 * epn + g) * 2 + 1] = (cnt > 0 && npad > 0) ? npad : 0;
        }
      }
      carry = __shfl_sync(0xffffffffu, end, 31);
    }
    if (lane == 0 && (int64_t)carry > p.NvS)
      report_failure(p.sync, ST_BAD_INDEX, 40, d, carry, (int)p.NvS);
  }
  __syncthreads();
  if (tid == 0) p.remote_stats[(size_t)vr * 2 + 1] = stat1[rank];
}

}  // namespace mep
