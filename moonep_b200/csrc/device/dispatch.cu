// Dispatch: fused permute + all-to-all of bf16 token rows and fp32 route weights, written
// straight into their expert-grouped slots in the destination ranks' buffers, plus the local
// duplicate expansion that follows it.
//
// Reference counterparts: DispatchKernel (moonep/dispatch.py:268-692) and
// DispatchEpilogueKernel (moonep/dispatch_epilogue.py:167-304).  Here:
//  * each row is staged once in shared memory by a 1-D bulk copy and then bulk-stored to at
//    most one slot per destination rank; the K stores of a row are issued by K lanes in
//    parallel, each tracking its own bulk group;
//  * there is no dedup builder: the chain links were written by the planner (source side);
//    the kernel only snapshots this rank's links into the plan after its exit barrier;
//  * padding rows are zeroed with bulk stores from one zero row, and their weight and link
//    slots are reset locally.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common/layout.h"
#include "device/dup_groups.cuh"
#include "device/sync.cuh"
#include "device/tma.cuh"
#include "host/ctx.h"
#include "host/errors.h"

namespace mep {

struct DispatchParams {
  SyncCtx sync;
  int S, K, H, epn;
  int64_t N, NvS, hidden_stride, weights_off, link_off, src_off;
  const __nv_bfloat16* x;     // [Rv][S][H]
  const float* w;             // [Rv][S][K] or null
  const int32_t* dst;         // [Rv][N]
  const int32_t* zero_fill;   // [Rv][2epn][2]
  __nv_bfloat16* hidden;      // symmetric, chunk of rank 0
  int32_t* link_out;          // [Rv][NvS] or null
  int32_t* src_out;           // [Rv][NvS] or null
  int entry_barrier;
  int fresh;                  // plan made by the preceding planner launch
};

constexpr int DISPATCH_THREADS = 128;

template <int ST>
__global__ void __launch_bounds__(DISPATCH_THREADS, 1) ep_dispatch_kernel(const DispatchParams p) {
  constexpr int LA = ST / 2;  // loads kept in flight; the other half of the ring drains stores
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[ST];
  const SyncCtx& sc = p.sync;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y, rank = sc.rank_base + vr;
  const int G = gridDim.x, c = blockIdx.x;
  const uint32_t row_bytes = (uint32_t)p.H * 2u;
  uint8_t* ring = smem_raw;
  uint8_t* zero_row = smem_raw + (size_t)ST * row_bytes;

  if (tid == 0) {
    for (int s = 0; s < ST; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  for (uint32_t i = tid * 16u; i < row_bytes; i += DISPATCH_THREADS * 16u)
    *reinterpret_cast<uint4*>(zero_row + i) = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  __syncthreads();
  pdl_launch_dependents();   // the expansion kernel may be scheduled; it waits for this one to end
  pdl_wait();                // a preceding planner launch has completed: its plan is readable
  if (tid == 0) phase_stamp(sc.trace, 0, c, 0);          // set up, predecessor complete
  if (p.entry_barrier) cross_rank_barrier(sc, 1);
  if (tid == 0) phase_stamp(sc.trace, 0, c, 1);          // past the entry barrier

  const __nv_bfloat16* x = p.x + (size_t)vr * p.S * p.H;
  const int32_t* dst = p.dst + (size_t)vr * p.N;
  const int n_tok = c < p.S ? (p.S - c + G - 1) / G : 0;

  if (warp == 0) {
    // ---- rows: load once, store to every destination rank that needs the payload --------
    if (lane == 0) {
      for (int j = 0; j < LA && j < n_tok; ++j) {
        mbar_expect_tx(&full[j], row_bytes);
        bulk_g2s(ring + (size_t)j * row_bytes, x + (size_t)(c + (int64_t)j * G) * p.H, row_bytes,
                 &full[j]);
      }
    }
    __syncwarp();
    for (int j = 0; j < n_tok; ++j) {
      const int s = j % ST;
      const int t = c + j * G;
      int d = lane < p.K ? dst[(size_t)t * p.K + lane] : -1;
      mbar_wait(sc, &full[s], (uint32_t)(j / ST) & 1u, 10);
      if (d >= 0) {
        int64_t dr = d / p.NvS, row = d - dr * p.NvS;
        if (dr < sc.R) {
          bulk_s2g(p.hidden + ((size_t)dr * p.hidden_stride + row) * p.H,
                   ring + (size_t)s * row_bytes, row_bytes);
        } else {
          report_failure(sc, ST_BAD_INDEX, 11, (int)dr, d, (int)p.NvS);
        }
      }
      bulk_commit();
      if (j + LA < n_tok) {
        // the stage to refill was last read by the stores of token j + LA - ST
        bulk_wait_read<ST - LA>();
        __syncwarp();
        if (lane == 0) {
          const int s2 = (j + LA) % ST;
          mbar_expect_tx(&full[s2], row_bytes);
          bulk_g2s(ring + (size_t)s2 * row_bytes, x + (size_t)(c + (int64_t)(j + LA) * G) * p.H,
                   row_bytes, &full[s2]);
        }
      }
    }
    bulk_wait<0>();
    fence_proxy_async();
  } else if (warp == 1) {
    // ---- route weights: one 4-byte store per (token, k), duplicates included -------------
    if (p.w != nullptr) {
      const float* w = p.w + (size_t)vr * p.N;
      const int64_t n_ent = (int64_t)n_tok * p.K;
      for (int64_t i = lane; i < n_ent; i += 32) {
        int j = (int)(i / p.K), k = (int)(i - (int64_t)j * p.K);
        int64_t e = (int64_t)(c + (int64_t)j * G) * p.K + k;
        int d = dst[e];
        int64_t raw = d >= 0 ? d : -(int64_t)d - 1;
        int64_t dr = raw / p.NvS, row = raw - dr * p.NvS;
        if (dr < sc.R)
          sc.meta[(size_t)dr * sc.meta_stride + p.weights_off + row] = __float_as_int(w[e]);
      }
    }
  } else {
    // ---- padding rows of MY shard: zero payload, weight 0, link NONE ----------------------
    const int32_t* zf = p.zero_fill + (size_t)vr * 2 * p.epn * 2;
    int32_t* my_meta = sc.meta + (size_t)rank * sc.meta_stride;
    __nv_bfloat16* my_shard = p.hidden + (size_t)rank * p.hidden_stride * p.H;
    int pending = 0;
    for (int g = 0; g < 2 * p.epn; ++g) {
      const int first = zf[2 * g], n = zf[2 * g + 1];
      if (n <= 0 || first < 0 || (int64_t)first + n > p.NvS) continue;
      if (warp == 2) {
        // one elected thread issues the row stores of this CTA's share
        if (lane == 0) {
          for (int r = first + c; r < first + n; r += G) {
            bulk_s2g(my_shard + (size_t)r * p.H, zero_row, row_bytes);
            if (++pending == 16) { bulk_commit(); bulk_wait_read<4>(); pending = 0; }
          }
        }
      } else {
        for (int r = first + c * 32 + lane; r < first + n; r += G * 32) {
          if (p.w != nullptr) my_meta[p.weights_off + r] = 0;
          if (p.fresh) { my_meta[p.link_off + r] = LINK_NONE; my_meta[p.src_off + r] = -1; }
        }
      }
    }
    if (warp == 2 && lane == 0) { bulk_commit(); bulk_wait<0>(); fence_proxy_async(); }
  }
  if (tid == 0) phase_stamp(sc.trace, 0, c, 2);          // this CTA's rows, weights and padding issued
  fence_sys();
  cross_rank_barrier(sc, 2);
  if (tid == 0) phase_stamp(sc.trace, 0, c, 3);          // past the exit barrier

  if (p.link_out != nullptr) {
    const int32_t* src = sc.meta + (size_t)rank * sc.meta_stride + p.link_off;
    int32_t* out = p.link_out + (size_t)vr * p.NvS;
    for (int64_t i = (int64_t)c * DISPATCH_THREADS + tid; i < p.NvS; i += (int64_t)G * DISPATCH_THREADS)
      out[i] = src[i];
  }
  if (p.src_out != nullptr) {
    const int32_t* src = sc.meta + (size_t)rank * sc.meta_stride + p.src_off;
    int32_t* out = p.src_out + (size_t)vr * p.NvS;
    for (int64_t i = (int64_t)c * DISPATCH_THREADS + tid; i < p.NvS; i += (int64_t)G * DISPATCH_THREADS)
      out[i] = src[i];
  }
}

// ---- duplicate expansion (local) ---------------------------------------------------------
struct ExpandParams {
  SyncCtx sync;                // status block and time budget of the bounded waits
  int H, epn;
  int64_t NvS, hidden_stride;
  int rank_base;
  __nv_bfloat16* hidden;       // symmetric base
  const int32_t* link;         // [Rv][NvS] plan-owned
  const int32_t* cu_seqlens;   // [Rv][2epn]
};

constexpr int EXPAND_THREADS = 128;

// One CTA per SM.  Pass by pass a CTA collects the duplicate groups whose primary lies in its share
// of this rank's rows (blocks of rows dealt round-robin, dup_groups.cuh) and then streams them: one
// bulk load of the primary row into a ring stage, one bulk store per duplicate from that stage
// (the duplicates of a group are issued by as many lanes in parallel), loads running ST/2 stages
// ahead of the stores.  The rows never pass through registers.
template <int ST>
__global__ void __launch_bounds__(EXPAND_THREADS, 1) ep_expand_kernel(const ExpandParams p) {
  constexpr int LA = ST / 2;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[ST];
  __shared__ DupGroupList L;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y, rank = p.rank_base + vr;
  const int32_t* link = p.link + (size_t)vr * p.NvS;
  const uint32_t row_bytes = (uint32_t)p.H * 2u;
  uint8_t* ring = smem_raw;
  if (tid == 0) {
    for (int s = 0; s < ST; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();                // the dispatch kernel before this one has completed
  int64_t rows64 = p.cu_seqlens[(size_t)vr * 2 * p.epn + 2 * p.epn - 1];
  if (rows64 > p.NvS) rows64 = p.NvS;
  const int rows = (int)rows64;
  uint8_t* shard = reinterpret_cast<uint8_t*>(p.hidden + (size_t)rank * p.hidden_stride * p.H);
  const int n_pass = dup_group_passes(rows, (int)gridDim.x);
  uint32_t issued = 0;       // groups this CTA has pushed through the ring so far (all passes)
  for (int pass = 0; pass < n_pass; ++pass) {
    collect_dup_groups(L, link, pass, (int)blockIdx.x, (int)gridDim.x, rows);
    const int ng = L.n;
    if (warp == 0 && ng > 0) {
      if (lane == 0) {
        for (int j = 0; j < LA && j < ng; ++j) {
          const uint32_t q = issued + j;
          mbar_expect_tx(&full[q % ST], row_bytes);
          bulk_g2s(ring + (size_t)(q % ST) * row_bytes, shard + (size_t)L.prim[j] * row_bytes, row_bytes,
                   &full[q % ST]);
        }
      }
      __syncwarp();
      for (int j = 0; j < ng; ++j) {
        const uint32_t q = issued + j;
        const int s = (int)(q % ST);
        mbar_wait(p.sync, &full[s], (q / ST) & 1u, 10);
        const int n = L.count[j];
        if (lane < n) {
          const int dr = dup_row(L, link, j, lane);
          if (dr >= 0 && dr < rows)
            bulk_s2g(shard + (size_t)dr * row_bytes, ring + (size_t)s * row_bytes, row_bytes);
        }
        bulk_commit();
        if (j + LA < ng) {
          // the stage to refill was last read by the stores of group q + LA - ST
          bulk_wait_read<ST - LA>();
          __syncwarp();
          if (lane == 0) {
            const uint32_t q2 = q + LA;
            mbar_expect_tx(&full[q2 % ST], row_bytes);
            bulk_g2s(ring + (size_t)(q2 % ST) * row_bytes, shard + (size_t)L.prim[j + LA] * row_bytes,
                     row_bytes, &full[q2 % ST]);
          }
        }
      }
      // the next pass reuses the stages from the start: everything of this pass has left them
      bulk_wait_read<0>();
      __syncwarp();
    }
    issued += (uint32_t)ng;
    __syncthreads();         // the list is rebuilt by all threads in the next pass
  }
  if (warp == 0) bulk_wait<0>();
}

// ---- fused dispatch -> GEMM path: the two small kernels around the fused GEMM launches ----------
// (the dispatch itself runs inside the GEMM kernel, device/fused_dispatch.cuh)
struct ArriveResetParams {
  SyncCtx sync;
  int64_t arrive_off;
  int n_arrive;
};
// Dispatch with a saved plan: clear this rank's arrival counters, then meet the group.  The
// barrier does what the entry barrier of the stand-alone dispatch does (every peer has finished
// reading this rank's row buffer) and orders the clear before every peer's first increment.
// With a fresh plan the planner kernel does both.
__global__ void __launch_bounds__(128, 1) ep_arrive_reset_kernel(const ArriveResetParams p) {
  const SyncCtx& sc = p.sync;
  const int rank = sc.rank_base + (int)blockIdx.y;
  int32_t* arrive = sc.meta + (size_t)rank * sc.meta_stride + p.arrive_off;
  for (int i = threadIdx.x; i < p.n_arrive; i += blockDim.x) arrive[i] = 0;
  cta_cross_rank_exchange(sc, 1);
}

struct SnapshotParams {
  const int32_t* link_src;
  const int32_t* src_src;
  int32_t* link_out;
  int32_t* src_out;
  int64_t n;
};
// Copies this rank's chain links and source records out of the meta chunk into the plan, once
// the fused GEMM launches of a fresh plan have completed (every block of rows has then arrived,
// and a source publishes its records before it sends its first row).
__global__ void __launch_bounds__(256) ep_plan_snapshot_kernel(const SnapshotParams p) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.n; i += (int64_t)gridDim.x * blockDim.x) {
    p.link_out[i] = p.link_src[i];
    p.src_out[i] = p.src_src[i];
  }
}

template <int ST>
static int launch_dispatch_t(const BufferCtx& c, DispatchParams& p, size_t smem,
                             cudaStream_t stream) {
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_dispatch_kernel<ST>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(c.num_sms, c.Rv());
  MEP_CUDA_OK(launch_chained((const void*)ep_dispatch_kernel<ST>, grid, dim3(DISPATCH_THREADS), smem,
                             stream, p, /*coop=*/1, c.pdl && p.fresh));
  return 0;
}

}  // namespace mep

using namespace mep;

extern "C" {

// x [Rv][S][H] bf16, w [Rv][S][K] fp32 or null, dst [Rv][N], zero_fill [Rv][2epn][2],
// link_out [Rv][NvS] or null.  fresh != 0: the plan comes from the planner launch that
// precedes this one on the stream (its barrier stands in for the entry sync).  shard selects
// the row buffer the rows land in (0, or 1 once a second shard is registered).
int mep_launch_dispatch(const void* ctx_, const void* x, const float* w, const int32_t* dst,
                        const int32_t* zero_fill, int32_t* link_out, int32_t* src_out, int entry_barrier,
                        int fresh, int shard, cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  if (c.H % 8 != 0) return fail(-1, "dispatch needs H %% 8 == 0 (got %d)", c.H);
  if (c.shard_base(shard) == nullptr) return fail(-4, "dispatch: shard %d does not exist", shard);
  DispatchParams p;
  p.sync = c.sync(KID_DISPATCH);
  p.S = c.S; p.K = c.K; p.H = c.H; p.epn = c.epn;
  p.N = c.N; p.NvS = c.NvS; p.hidden_stride = c.hidden_stride;
  p.weights_off = c.ml.weights_off; p.link_off = c.ml.link_off; p.src_off = c.ml.src_off;
  p.x = (const __nv_bfloat16*)x; p.w = w; p.dst = dst; p.zero_fill = zero_fill;
  p.hidden = (__nv_bfloat16*)c.shard_base(shard); p.link_out = link_out; p.src_out = src_out;
  p.entry_barrier = entry_barrier; p.fresh = fresh;
  const size_t row = (size_t)c.H * 2;
  // virtual groups must keep gridDim.x * R CTAs co-resident: leave room for 2 CTAs per SM
  const size_t budget = c.virt ? 100 * 1024 : 200 * 1024;
  if (9 * row <= budget) return launch_dispatch_t<8>(c, p, 9 * row, stream);
  if (5 * row <= budget) return launch_dispatch_t<4>(c, p, 5 * row, stream);
  if (3 * row <= 220 * 1024) return launch_dispatch_t<2>(c, p, 3 * row, stream);
  return fail(-2, "dispatch: H=%d does not fit a 2-stage ring", c.H);
}

// Copy every primary row to its duplicates inside this rank's shard.
int mep_launch_expand(const void* ctx_, const int32_t* link, const int32_t* cu_seqlens, int shard,
                      cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  if (c.shard_base(shard) == nullptr) return fail(-4, "expand: shard %d does not exist", shard);
  ExpandParams p;
  p.sync = c.sync(KID_EXPAND);
  p.H = c.H; p.epn = c.epn; p.NvS = c.NvS; p.hidden_stride = c.hidden_stride;
  p.rank_base = c.virt ? 0 : c.rank;
  p.hidden = (__nv_bfloat16*)c.shard_base(shard); p.link = link; p.cu_seqlens = cu_seqlens;
  // one CTA per SM (a virtual group shares the SMs between its ranks); the ring takes what
  // shared memory the group lists leave
  const size_t row = (size_t)c.H * 2;
  int gx = c.num_sms_local / c.Rv();
  if (gx < 1) gx = 1;
  dim3 grid(gx, c.Rv());
  const void* kern;
  size_t smem;
  if (8 * row <= 160 * 1024) { kern = (const void*)ep_expand_kernel<8>; smem = 8 * row; }
  else if (4 * row <= 200 * 1024) { kern = (const void*)ep_expand_kernel<4>; smem = 4 * row; }
  else if (2 * row <= 200 * 1024) { kern = (const void*)ep_expand_kernel<2>; smem = 2 * row; }
  else return fail(-2, "expand: H=%d does not fit a 2-stage ring", c.H);
  static thread_local size_t configured[3] = {0, 0, 0};
  const int which = kern == (const void*)ep_expand_kernel<8> ? 0 : (kern == (const void*)ep_expand_kernel<4> ? 1 : 2);
  if (smem > 48 * 1024 && smem > configured[which]) {
    MEP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[which] = smem;
  }
  MEP_CUDA_OK(launch_chained(kern, grid, dim3(EXPAND_THREADS), smem, stream, p, /*coop=*/0, c.pdl));
  return 0;
}

// Saved-plan entry of the fused dispatch -> GEMM path (see ep_arrive_reset_kernel).
int mep_launch_arrive_reset(const void* ctx_, cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  ArriveResetParams p;
  p.sync = c.sync(KID_DISPATCH);
  p.arrive_off = c.ml.arrive_off;
  p.n_arrive = (int)(c.NvS / 128 + 1);
  dim3 grid(1, c.Rv());
  MEP_CUDA_OK(launch_coop((const void*)ep_arrive_reset_kernel, grid, dim3(128), 0, stream, p));
  return 0;
}

// Fresh-plan exit of the fused path: link_out / src_out [NvS] of the plan.
int mep_launch_plan_snapshot(const void* ctx_, int32_t* link_out, int32_t* src_out, cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  if (c.virt) return fail(-1, "plan snapshot: the fused path runs one rank per launch");
  SnapshotParams p;
  const int32_t* mine = c.meta + (size_t)c.rank * c.meta_stride;
  p.link_src = mine + c.ml.link_off; p.src_src = mine + c.ml.src_off;
  p.link_out = link_out; p.src_out = src_out; p.n = c.NvS;
  ep_plan_snapshot_kernel<<<32, 256, 0, stream>>>(p);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
