// Online redundant-expert planner for sm_100a.
//
// What it computes is defined by the CPU oracle (ref/plan_ref.cc), which mirrors the
// reference's oracle (tests/planning_reference.py) and device planner
// (moonep/planning.py:495-1098).  How it computes it differs from the reference:
//  * the reference solves the plan on rank 0 only, parks rank 0's sort on rank 1 and
//    broadcasts three E*R tables through NVLS (planning.py:578-582, 917-934).  Here the
//    gathered tpe[R][E] table (a few KB) is all-gathered with peer stores and EVERY rank
//    solves redundantly in ONE CTA.  The solve is integer-only, hence bit-identical on all
//    ranks, so there is no broadcast, no rank-0 serialisation and ONE cross-rank barrier
//    instead of three.
//  * while CTA 0 exchanges and solves, the other CTAs histogram their slice of top-k.
//  * duplicates of a token on one destination rank are published as per-slot chain links by
//    the SOURCE (common/layout.h) instead of per-slot source records that the destination
//    turns into groups with atomics (dispatch.py:499-681).
#include <cuda_runtime.h>

#include "common/layout.h"
#include "device/planner_core.cuh"
#include "device/sync.cuh"
#include "host/ctx.h"
#include "host/errors.h"

namespace mep {

__global__ void __launch_bounds__(PLAN_THREADS, 1) ep_plan_kernel(const PlanParams p) {
  extern __shared__ int32_t smem[];
  const SyncCtx& sc = p.sync;
  const int R = sc.R, E = p.E, K = p.K;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y, rank = sc.rank_base + vr;
  const int G = gridDim.x, c = blockIdx.x;
  int32_t* st = sync_state_of(sc);
  const int parity = st[3] & 1;
  const int32_t* topk = p.topk + (size_t)vr * p.N;
  int32_t* dst = p.dst + (size_t)vr * p.N;
  int32_t* scratch = p.scratch + (size_t)vr * p.scratch_ints;
  int32_t* hist_g = scratch + (size_t)4 * R * E;
  const int64_t tbl_off = p.tpe_off + (int64_t)parity * R * E;
  pdl_launch_dependents();   // the dispatch kernel that follows may set itself up meanwhile

  // slice of entries owned by this CTA (whole tokens)
  const int tpc = (p.S + G - 1) / G;
  const int tok0 = min(p.S, c * tpc), tok1 = min(p.S, tok0 + tpc);
  const int64_t i0 = (int64_t)tok0 * K, i1 = (int64_t)tok1 * K;

  if (c == 0) {
    // all-gather of tpe by peer stores: my row into everyone's table
    const int32_t* my_tpe = p.tpe + (size_t)vr * E;
    for (int64_t i = tid; i < (int64_t)R * E; i += PLAN_THREADS) {
      int peer = (int)(i / E), e = (int)(i % E);
      sc.meta[(size_t)peer * sc.meta_stride + tbl_off + (size_t)rank * E + e] = my_tpe[e];
    }
  }
  // histogram of my slice (smem cnt[E] sits after the solver's area so both can coexist)
  int32_t* cnt = smem;
  for (int e = tid; e < E; e += PLAN_THREADS) cnt[e] = 0;
  __syncthreads();
  for (int64_t i = i0 + tid; i < i1; i += PLAN_THREADS) {
    int e = topk[i];
    if ((unsigned)e < (unsigned)E) atomicAdd(&cnt[e], 1);
    else report_failure(sc, ST_BAD_INDEX, 10, -1, e, E);
  }
  __syncthreads();
  for (int e = tid; e < E; e += PLAN_THREADS) hist_g[(size_t)c * E + e] = cnt[e];
  if (c == 0) {
    // arrival counters of the fused dispatch -> GEMM path start at zero; clearing them before
    // the exchange orders the clear before every peer's first increment of this step
    int32_t* arrive = sc.meta + (size_t)rank * sc.meta_stride + p.arrive_off;
    for (int i = tid; i < p.n_arrive; i += PLAN_THREADS) arrive[i] = 0;
    cta_cross_rank_exchange(sc, 1);
    plan_solve(p, rank, sc.meta + (size_t)rank * sc.meta_stride + tbl_off, smem);
  }
  grid_sync(sc, 2);
  if (c == 0 && tid == 0) st[3] = parity ^ 1;

  const int32_t* tpe_cumsum = scratch;
  const int32_t* alloc_cumsum = scratch + (size_t)2 * R * E;
  const int32_t* expert_off = scratch + (size_t)3 * R * E;

  // running count of each expert before my slice: earlier ranks + earlier CTAs of my rank
  for (int e = tid; e < E; e += PLAN_THREADS) {
    int base = rank > 0 ? tpe_cumsum[(size_t)(rank - 1) * E + e] : 0;
    for (int cc = 0; cc < c; ++cc) base += hist_g[(size_t)cc * E + e];
    cnt[e] = base;
  }
  // sending order: exclusive prefix of my per-expert counts in the permuted expert order
  int32_t* pperm = smem + E;
  if (p.send_order != nullptr) {
    const int32_t* my_tpe = p.tpe + (size_t)vr * E;
    for (int e = tid; e < E; e += PLAN_THREADS) pperm[send_perm(e, p.epn, R, rank)] = my_tpe[e];
  }
  __syncthreads();
  if (warp == 0 && p.send_order != nullptr) {
    int run = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int n = e < E ? pperm[e] : 0;
      int incl = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (e < E) pperm[e] = run + incl - n;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  // stable rank of every entry among the entries of its expert (one warp, in order)
  if (warp == 0) {
    for (int64_t b = i0; b < i1; b += 32) {
      int64_t i = b + lane;
      bool valid = i < i1;
      int e = valid ? topk[i] : -1 - lane;
      if (valid && (unsigned)e >= (unsigned)E) e = 0;
      unsigned m = __match_any_sync(0xffffffffu, e);
      int before = __popc(m & ((1u << lane) - 1));
      int base = valid ? cnt[e] : 0;
      __syncwarp();
      if (valid && before == 0) cnt[e] = base + __popc(m);
      __syncwarp();
      if (valid) dst[i] = base + before;  // global rank of the entry, resolved below
    }
  }
  __syncthreads();
  // destination rank and row of every entry
  for (int64_t i = i0 + tid; i < i1; i += PLAN_THREADS) {
    int e = topk[i];
    if ((unsigned)e >= (unsigned)E) e = 0;
    int g = dst[i];
    const int32_t* ac = alloc_cumsum + (size_t)e * R;
    int lo = 0, hi = R;  // first d with ac[d] > g
    while (lo < hi) {
      int mid = (lo + hi) >> 1;
      if (ac[mid] > g) hi = mid; else lo = mid + 1;
    }
    int dest = lo;
    if (dest >= R) { report_failure(sc, ST_BAD_INDEX, 20, e, g, ac[R - 1]); dest = R - 1; }
    int prev = dest > 0 ? ac[dest - 1] : 0;
    int64_t row = (int64_t)expert_off[(size_t)dest * E + e] + (g - prev);
    if (row < 0 || row >= p.NvS) { report_failure(sc, ST_BAD_INDEX, 21, dest, (int)row, (int)p.NvS); row = 0; }
    dst[i] = (int)((int64_t)dest * p.NvS + row);
    if (p.send_order != nullptr) {
      const int mine_before = rank > 0 ? tpe_cumsum[(size_t)(rank - 1) * E + e] : 0;
      const int64_t pos = (int64_t)pperm[send_perm(e, p.epn, R, rank)] + (g - mine_before);
      if (pos >= 0 && pos < p.N) p.send_order[(size_t)vr * p.N + pos] = (int32_t)i;
      else report_failure(sc, ST_BAD_INDEX, 22, e, (int)pos, (int)p.N);
    }
  }
  __syncthreads();
  // duplicate canonicalisation + chain links: K lanes per token (32 / K tokens per warp), the
  // lanes of a token that share a destination rank find one another with match.any, so nothing
  // is kept in per-thread arrays
  const int tpw = 32 / K;
  const int tl = lane / K, k = lane - tl * K;
  for (int t0 = tok0 + warp * tpw; t0 < tok1; t0 += PLAN_WARPS * tpw) {
    const int t = t0 + tl;
    const bool valid = tl < tpw && t < tok1;
    int32_t* d = dst + (size_t)t * K;
    const int raw = valid ? d[k] : 0;
    const int dr = valid ? (int)(raw / p.NvS) : 0;
    const unsigned m = __match_any_sync(0xffffffffu, valid ? ((tl << 8) | dr) : (0x40000000 | lane));
    const bool dup = (m & ((1u << lane) - 1u)) != 0u;
    const unsigned above = lane < 31 ? (m & ~((2u << lane) - 1u)) : 0u;
    const int nl = above ? __ffs(above) - 1 : lane;
    const int raw_next = __shfl_sync(0xffffffffu, raw, nl);
    if (valid) {
      const int next = above ? (int)(raw_next - (int64_t)dr * p.NvS) : LINK_NONE;
      const int64_t row = raw - (int64_t)dr * p.NvS;
      int32_t* peer = sc.meta + (size_t)dr * sc.meta_stride;
      peer[p.link_off + row] = next | (dup ? LINK_DUP_BIT : 0);
      peer[p.src_off + row] = (int32_t)((int64_t)rank * p.N + (int64_t)t * K + k);
      if (dup) d[k] = -raw - 1;
    }
  }
}

}  // namespace mep

using namespace mep;

extern "C" {

// Dynamic shared memory the planner needs for (R, E).
int64_t mep_plan_smem_bytes(int R, int E) {
  return (int64_t)sizeof(int32_t) * (2 * (int64_t)E + 4 * R + (int64_t)PLAN_WARPS * R);
}

// Fresh plan for this rank (or for all virtual ranks).  send_order [Rv][N] may be null (it is
// only needed by the fused dispatch -> GEMM path).  Leaves the chain links in the peers'
// meta chunks; they become visible with the next cross-rank barrier (the dispatch kernel's
// exit barrier, or an explicit mep_launch_sync).
int mep_launch_plan(const void* ctx_, const int32_t* topk, const int32_t* tpe, int32_t* dst,
                    int32_t* cu_seqlens, int32_t* zero_fill, int32_t* etc, int32_t* remote_stats,
                    int32_t* send_order, cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  PlanParams p;
  p.sync = c.sync(KID_PLAN);
  p.E = c.E; p.epn = c.epn; p.S = c.S; p.K = c.K; p.token_padding = c.token_padding;
  p.N = c.N; p.NvS = c.NvS;
  p.tpe_off = c.ml.tpe_off; p.link_off = c.ml.link_off; p.src_off = c.ml.src_off;
  p.topk = topk; p.tpe = tpe; p.dst = dst; p.cu_seqlens = cu_seqlens; p.zero_fill = zero_fill;
  p.etc = etc; p.remote_stats = remote_stats;
  p.scratch = c.plan_scratch; p.scratch_ints = c.plan_scratch_ints;
  p.send_order = send_order; p.arrive_off = c.ml.arrive_off; p.n_arrive = (int)(c.NvS / 128 + 1);
  size_t smem = (size_t)mep_plan_smem_bytes(c.R, c.E);
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_plan_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(c.num_sms, c.Rv());
  MEP_CUDA_OK(launch_coop((const void*)ep_plan_kernel, grid, dim3(PLAN_THREADS), smem, stream, p));
  return 0;
}

}  // extern "C"
