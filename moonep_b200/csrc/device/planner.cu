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
#include "device/sync.cuh"
#include "host/ctx.h"
#include "host/errors.h"

namespace mep {

struct PlanParams {
  SyncCtx sync;
  int E, epn, S, K, token_padding;
  int64_t N, NvS;
  int64_t tpe_off, link_off;
  const int32_t* topk;      // [Rv][N]
  const int32_t* tpe;       // [Rv][E]
  int32_t* dst;             // [Rv][N]
  int32_t* cu_seqlens;      // [Rv][2epn]
  int32_t* zero_fill;       // [Rv][2epn][2]
  int32_t* etc;             // [Rv][R][epn]
  int32_t* remote_stats;    // [Rv][2]
  int32_t* scratch;         // [Rv][scratch_ints]
  int64_t scratch_ints;
};

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
__device__ void plan_solve(const PlanParams& p, int rank, const int32_t* tbl /*[R][E]*/,
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
  __syncthreads();
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
  }
  __syncthreads();
  // duplicate canonicalisation + chain links, one thread per token
  for (int t = tok0 + tid; t < tok1; t += PLAN_THREADS) {
    int32_t* d = dst + (size_t)t * K;
    int raw[MAX_TOPK];
    int dr[MAX_TOPK];
#pragma unroll 4
    for (int k = 0; k < K; ++k) {
      raw[k] = d[k];
      dr[k] = (int)(raw[k] / p.NvS);
    }
    for (int k = 0; k < K; ++k) {
      bool dup = false;
      for (int j = 0; j < k; ++j) dup |= dr[j] == dr[k];
      int next = LINK_NONE;
      for (int j = K - 1; j > k; --j)
        if (dr[j] == dr[k]) next = (int)(raw[j] - (int64_t)dr[j] * p.NvS);
      int64_t row = raw[k] - (int64_t)dr[k] * p.NvS;
      sc.meta[(size_t)dr[k] * sc.meta_stride + p.link_off + row] = next | (dup ? LINK_DUP_BIT : 0);
      if (dup) d[k] = -raw[k] - 1;
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

// Fresh plan for this rank (or for all virtual ranks).  Leaves the chain links in the peers'
// meta chunks; they become visible with the next cross-rank barrier (the dispatch kernel's
// exit barrier, or an explicit mep_launch_sync).
int mep_launch_plan(const void* ctx_, const int32_t* topk, const int32_t* tpe, int32_t* dst,
                    int32_t* cu_seqlens, int32_t* zero_fill, int32_t* etc, int32_t* remote_stats,
                    cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  PlanParams p;
  p.sync = c.sync(KID_PLAN);
  p.E = c.E; p.epn = c.epn; p.S = c.S; p.K = c.K; p.token_padding = c.token_padding;
  p.N = c.N; p.NvS = c.NvS;
  p.tpe_off = c.ml.tpe_off; p.link_off = c.ml.link_off;
  p.topk = topk; p.tpe = tpe; p.dst = dst; p.cu_seqlens = cu_seqlens; p.zero_fill = zero_fill;
  p.etc = etc; p.remote_stats = remote_stats;
  p.scratch = c.plan_scratch; p.scratch_ints = c.plan_scratch_ints;
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
