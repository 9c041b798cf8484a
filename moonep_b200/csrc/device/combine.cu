// Combine: local fp32 pre-reduction of duplicate rows, then every rank PULLS the rows of its
// own tokens from the peers' shards and sums them in fp32 in ascending k.
//
// Reference counterparts: CombinePrologueKernel (moonep/combine_prologue.py:196-484) and
// CombineKernel (moonep/combine.py:210-511).  The sum is unweighted, as in the reference:
// the route weights travel with dispatch so that the expert FFN can apply them.
// Rounding points are the same as in the CPU simulator (ref/sim_ref.cc): one bf16 rounding
// of each pre-reduced primary row, one of the final sum; additions are fp32 in chain / k
// order, so results are bitwise reproducible.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common/layout.h"
#include "device/dup_groups.cuh"
#include "device/sync.cuh"
#include "device/tma.cuh"
#include "host/ctx.h"
#include "host/errors.h"

namespace mep {

__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- row accumulation in packed fp32 pairs ---------------------------------------------------
// The kernels that sum bf16 rows in fp32 (pre-reduction, pull combine) are bound by instruction
// issue, not by memory, when they run one accumulator warp per scheduler with scalar adds
// (measured: ~220 warp instructions and 0.65 us per 14 KB row).  They therefore keep their
// accumulators as f32x2 pairs (add.rn.f32x2, one instruction per two sums, same IEEE result per
// lane as two scalar adds), take the first row of a sum by assignment, and use seven accumulator
// warps, so that every scheduler has a second warp to issue from.
constexpr int ACC_WARPS = 7;
constexpr int ACC_THREADS = ACC_WARPS * 32;      // 224: a 7168-element row is exactly 4 vectors per thread

__device__ __forceinline__ unsigned long long pack_f32x2(uint32_t lo, uint32_t hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// 8 bf16 (one 16-byte vector) as four fp32 pairs
__device__ __forceinline__ void bf16x8_to_f32x2(const uint4& v, unsigned long long* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = pack_f32x2(w[i] << 16, w[i] & 0xFFFF0000u);
}
__device__ __forceinline__ uint4 f32x2_to_bf16x8(const unsigned long long* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(f[i]));
    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(lo), __uint_as_float(hi));
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
// acc (+)= one staged row; `first` is uniform over the CTA's accumulator threads
template <int NV>
__device__ __forceinline__ void accumulate_row(unsigned long long (&acc)[NV][4], const uint4* src, int ta,
                                               int nvec, bool first) {
  if (first) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = ta + i * ACC_THREADS;
      if (v < nvec) bf16x8_to_f32x2(src[v], acc[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = ta + i * ACC_THREADS;
      if (v < nvec) {
        unsigned long long t[4];
        bf16x8_to_f32x2(src[v], t);
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[i][q] = add_f32x2(acc[i][q], t[q]);
      }
    }
  }
}

// ---- prologue: primary += duplicates (local) ---------------------------------------------
struct PrologueParams {
  SyncCtx sync;               // status block and time budget of the bounded waits
  int H, epn;
  int64_t NvS, hidden_stride;
  int rank_base;
  __nv_bfloat16* hidden;
  const int32_t* link;        // [Rv][NvS]
  const int32_t* cu_seqlens;  // [Rv][2epn]
};

constexpr int PROLOGUE_ACC_THREADS = ACC_THREADS;
constexpr int PROLOGUE_THREADS = 32 + PROLOGUE_ACC_THREADS;     // loader warp + accumulator warps

__device__ __forceinline__ void named_bar_sync(int id, int n) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}

// One CTA per SM.  Pass by pass a CTA collects the duplicate groups whose primary lies in its share
// of this rank's rows (blocks of rows dealt round-robin, dup_groups.cuh), then the loader lane streams
// every group's rows (primary first, duplicates in chain order) through a ring of bulk loads while
// the accumulator warps sum them in fp32 registers, round once to bf16 and hand the row to a bulk
// store back onto the primary.  NV: 16-byte vectors per accumulator thread.
template <int ST, int NV>
__global__ void __launch_bounds__(PROLOGUE_THREADS, 1) ep_combine_prologue_kernel(const PrologueParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[ST];
  __shared__ __align__(8) uint64_t empty[ST];
  __shared__ int last_flag[ST];
  __shared__ DupGroupList L;
  const SyncCtx& sc = p.sync;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y, rank = p.rank_base + vr;
  const int32_t* link = p.link + (size_t)vr * p.NvS;
  const uint32_t row_bytes = (uint32_t)p.H * 2u;
  const int nvec = p.H / 8;
  uint8_t* ring = smem_raw;
  uint8_t* out_stage = smem_raw + (size_t)ST * row_bytes;
  if (tid == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], PROLOGUE_ACC_THREADS / 32); }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();   // the pull kernel may set up its ring; it waits for this kernel to end
  int64_t rows64 = p.cu_seqlens[(size_t)vr * 2 * p.epn + 2 * p.epn - 1];
  if (rows64 > p.NvS) rows64 = p.NvS;
  const int rows = (int)rows64;
  uint8_t* shard = reinterpret_cast<uint8_t*>(p.hidden + (size_t)rank * p.hidden_stride * p.H);
  const int n_pass = dup_group_passes(rows, (int)gridDim.x);
  uint32_t moved = 0;        // rows through the ring so far (loader and accumulators count alike)
  uint32_t out_n = 0;        // rows stored so far (accumulators)
  const int ta = tid - 32;
  for (int pass = 0; pass < n_pass; ++pass) {
    collect_dup_groups(L, link, pass, (int)blockIdx.x, (int)gridDim.x, rows);
    const int ng = L.n;
    if (warp == 0) {
      if (lane == 0) {
        for (int j = 0; j < ng; ++j) {
          const int n = L.count[j];
          for (int e = 0; e <= n; ++e, ++moved) {
            const int s = (int)(moved % ST);
            if (moved >= ST) mbar_wait(sc, &empty[s], ((moved / ST) & 1u) ^ 1u, 20);
            int r = e == 0 ? L.prim[j] : dup_row(L, link, j, e - 1);
            if (r < 0 || r >= rows) { report_failure(sc, ST_BAD_INDEX, 21, j, r, rows); r = L.prim[j]; }
            last_flag[s] = e == n;
            mbar_expect_tx(&full[s], row_bytes);
            bulk_g2s(ring + (size_t)s * row_bytes, shard + (size_t)r * row_bytes, row_bytes, &full[s]);
          }
        }
      }
      __syncwarp();
    } else {
      for (int j = 0; j < ng; ++j) {
        unsigned long long acc[NV][4];
        bool first = true;
        for (int guard = 0; guard < MAX_TOPK; ++guard, ++moved) {
          const int s = (int)(moved % ST);
          const bool ok = mbar_wait(sc, &full[s], (moved / ST) & 1u, 30);
          const uint4* src = reinterpret_cast<const uint4*>(ring + (size_t)s * row_bytes);
          const int is_last = ok ? last_flag[s] : 1;
          accumulate_row<NV>(acc, src, ta, nvec, first);
          first = false;
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);
          if (is_last) { ++moved; break; }
        }
        // stage the bf16 row and hand it to one bulk store onto the primary
        uint8_t* os = out_stage + (size_t)(out_n & 1u) * row_bytes;
        if (out_n >= 2) {
          if (ta == 0) bulk_wait_read<1>();
          named_bar_sync(1, PROLOGUE_ACC_THREADS);
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int v = ta + i * PROLOGUE_ACC_THREADS;
          if (v < nvec) reinterpret_cast<uint4*>(os)[v] = f32x2_to_bf16x8(acc[i]);
        }
        fence_proxy_async_smem();
        named_bar_sync(1, PROLOGUE_ACC_THREADS);
        if (ta == 0) {
          bulk_s2g(shard + (size_t)L.prim[j] * row_bytes, os, row_bytes);
          bulk_commit();
        }
        ++out_n;
      }
    }
    __syncthreads();         // the list is rebuilt by all threads in the next pass
  }
  if (ta == 0) bulk_wait<0>();
}

// ---- combine: remote pull + K-way fp32 sum -----------------------------------------------
struct CombineParams {
  SyncCtx sync;
  int S, K, H;
  int64_t N, NvS, hidden_stride, weights_off;
  const int32_t* dst;            // [Rv][N]
  const __nv_bfloat16* hidden;   // symmetric base
  __nv_bfloat16* out;            // [Rv][S][H]
  float* w_out;                  // [Rv][S][K] or null
};

constexpr int COMBINE_ACC_THREADS = ACC_THREADS;
constexpr int COMBINE_THREADS = 32 + COMBINE_ACC_THREADS + 32;  // loader, accumulator warps, weights

// NV: 16-byte vectors per accumulator thread (H <= NV * 128 * 8)
template <int ST, int NV>
__global__ void __launch_bounds__(COMBINE_THREADS, 1) ep_combine_kernel(const CombineParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[ST];
  __shared__ __align__(8) uint64_t empty[ST];
  __shared__ int last_flag[ST];
  const SyncCtx& sc = p.sync;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y;
  const int G = gridDim.x, c = blockIdx.x;
  const uint32_t row_bytes = (uint32_t)p.H * 2u;
  const int nvec = p.H / 8;
  uint8_t* ring = smem_raw;

  if (tid == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], COMBINE_ACC_THREADS / 32); }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();                 // this rank's pre-reduction kernel has completed
  if (tid == 0) phase_stamp(sc.trace, 1, c, 0);
  cross_rank_barrier(sc, 1);  // every rank's shard (and its pre-reduction) is final
  if (tid == 0) phase_stamp(sc.trace, 1, c, 1);          // past the entry barrier: pulls start

  const int32_t* dst = p.dst + (size_t)vr * p.N;
  const int n_tok = c < p.S ? (p.S - c + G - 1) / G : 0;

  if (warp == 0) {
    // ---- loader: one remote bulk read per primary entry -----------------------------------
    int prod = 0;
    int d_next = (n_tok > 0 && lane < p.K) ? dst[(size_t)c * p.K + lane] : -1;
    for (int j = 0; j < n_tok; ++j) {
      const int d = d_next;   // the next token's destinations are fetched while this one is issued
      d_next = (j + 1 < n_tok && lane < p.K) ? dst[(size_t)(c + (int64_t)(j + 1) * G) * p.K + lane] : -1;
      unsigned prim = __ballot_sync(0xffffffffu, d >= 0);
      while (prim) {
        int k = __ffs(prim) - 1;
        prim &= prim - 1;
        int dk = __shfl_sync(0xffffffffu, d, k);
        if (lane == 0) {
          const int s = prod % ST;
          if (prod >= ST) mbar_wait(sc, &empty[s], ((uint32_t)(prod / ST) & 1u) ^ 1u, 20);
          int64_t dr = dk / p.NvS, row = dk - dr * p.NvS;
          if (dr >= sc.R) { report_failure(sc, ST_BAD_INDEX, 21, (int)dr, dk, (int)p.NvS); dr = 0; }
          last_flag[s] = prim == 0;
          mbar_expect_tx(&full[s], row_bytes);
          bulk_g2s(ring + (size_t)s * row_bytes,
                   p.hidden + ((size_t)dr * p.hidden_stride + row) * p.H, row_bytes, &full[s]);
        }
        ++prod;
      }
    }
  } else if (warp <= COMBINE_ACC_THREADS / 32) {
    // ---- accumulators ----------------------------------------------------------------------
    const int ta = tid - 32;
    __nv_bfloat16* out = p.out + (size_t)vr * p.S * p.H;
    int cons = 0;
    for (int j = 0; j < n_tok; ++j) {
      unsigned long long acc[NV][4];
      bool first = true;
      for (int guard = 0; guard < MAX_TOPK; ++guard) {
        const int s = cons % ST;
        bool ok = mbar_wait(sc, &full[s], (uint32_t)(cons / ST) & 1u, 30);
        const uint4* src = reinterpret_cast<const uint4*>(ring + (size_t)s * row_bytes);
        const int is_last = ok ? last_flag[s] : 1;
        accumulate_row<NV>(acc, src, ta, nvec, first);
        first = false;
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        ++cons;
        if (is_last) break;
      }
      // The summed row goes straight from the accumulators to this rank's output with 16-byte
      // stores (consecutive threads, consecutive vectors).  The output is local memory, so the
      // stores cost little, and keeping them out of shared memory leaves two more stages to the
      // ring of remote reads: the pull is bound by bytes in flight over the read latency.
      uint4* orow = reinterpret_cast<uint4*>(out + (size_t)(c + (int64_t)j * G) * p.H);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        int v = ta + i * COMBINE_ACC_THREADS;
        if (v < nvec) orow[v] = f32x2_to_bf16x8(acc[i]);
      }
    }
  } else if (p.w_out != nullptr) {
    // ---- route weights back to token-major, raw 32-bit words -------------------------------
    float* w_out = p.w_out + (size_t)vr * p.N;
    const int64_t n_ent = (int64_t)n_tok * p.K;
    for (int64_t i = lane; i < n_ent; i += 32) {
      int j = (int)(i / p.K), k = (int)(i - (int64_t)j * p.K);
      int64_t e = (int64_t)(c + (int64_t)j * G) * p.K + k;
      int d = dst[e];
      int64_t raw = d >= 0 ? d : -(int64_t)d - 1;
      int64_t dr = raw / p.NvS, row = raw - dr * p.NvS;
      int bits = dr < sc.R ? sc.meta[(size_t)dr * sc.meta_stride + p.weights_off + row] : 0;
      w_out[e] = __int_as_float(bits);
    }
  }
  if (tid == 32) phase_stamp(sc.trace, 1, c, 2);         // this CTA's tokens are summed and stored
}

// ---- pushed combine: barrier, then every rank sums the K rows its peers pushed per token -------
// Counterpart of the pull combine for the fused path: the GEMM epilogue (grouped_gemm.cu, PUSH)
// already stored every result row into staging[home rank][token*K + k], so what is left is one
// cross-rank barrier and a local, bandwidth-bound K-way fp32 sum in ascending k.  Route-weight
// grads (backward of dispatch) ride along: each rank first pushes its per-row scalars to the
// owners' fp32 staging, the owners read them back after the barrier.
struct PushReduceParams {
  SyncCtx sync;
  int S, K, H, epn;
  int64_t N, NvS, push_stride, wpush_stride;
  const __nv_bfloat16* push;       // symmetric [R][N][H]
  float* wpush;                    // symmetric [R][N]
  const int32_t* src_info;         // [Rv][NvS]
  const float* row_scalar;         // [Rv][NvS] or null
  const int32_t* cu_seqlens;       // [Rv][2epn]
  __nv_bfloat16* out;              // [Rv][S][H]
  float* w_out;                    // [Rv][S][K] or null
};

constexpr int PUSH_REDUCE_THREADS = 256;

__global__ void __launch_bounds__(PUSH_REDUCE_THREADS, 1) ep_push_reduce_kernel(const PushReduceParams p) {
  const SyncCtx& sc = p.sync;
  const int tid = threadIdx.x;
  const int vr = blockIdx.y, rank = sc.rank_base + vr;
  const int G = gridDim.x, c = blockIdx.x;
  if (p.row_scalar != nullptr) {
    const int32_t* si = p.src_info + (size_t)vr * p.NvS;
    const float* rs = p.row_scalar + (size_t)vr * p.NvS;
    int64_t rows = p.cu_seqlens[(size_t)vr * 2 * p.epn + 2 * p.epn - 1];
    if (rows > p.NvS) rows = p.NvS;
    for (int64_t r = (int64_t)c * PUSH_REDUCE_THREADS + tid; r < rows; r += (int64_t)G * PUSH_REDUCE_THREADS) {
      const int v = si[r];
      if (v < 0) continue;
      const int64_t sr = v / p.N, ent = v - sr * p.N;
      if (sr < sc.R) p.wpush[(size_t)sr * p.wpush_stride + ent] = rs[r];
    }
  }
  fence_sys();
  cross_rank_barrier(sc, 1);
  const uint4* mine = reinterpret_cast<const uint4*>(p.push + (size_t)rank * p.push_stride);
  uint4* out = reinterpret_cast<uint4*>(p.out + (size_t)vr * p.S * p.H);
  const int nvec = p.H / 8;
  for (int s = c; s < p.S; s += G) {
    const uint4* base = mine + (size_t)s * p.K * nvec;
    for (int v = tid; v < nvec; v += PUSH_REDUCE_THREADS) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int k0 = 0; k0 < p.K; k0 += 8) {
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          raw[u] = k0 + u < p.K ? base[(size_t)(k0 + u) * nvec + v] : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float t[8];
          bf16x8_to_f32(raw[u], t);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] += t[q];
        }
      }
      out[(size_t)s * nvec + v] = f32_to_bf16x8(acc);
    }
  }
  if (p.w_out != nullptr) {
    const float* wm = p.wpush + (size_t)rank * p.wpush_stride;
    float* wo = p.w_out + (size_t)vr * p.N;
    for (int64_t i = (int64_t)c * PUSH_REDUCE_THREADS + tid; i < p.N; i += (int64_t)G * PUSH_REDUCE_THREADS)
      wo[i] = wm[i];
  }
}

template <int ST, int NV>
static int launch_combine_t(const BufferCtx& c, CombineParams& p, size_t smem, cudaStream_t stream) {
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_combine_kernel<ST, NV>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(c.num_sms, c.Rv());
  MEP_CUDA_OK(launch_chained((const void*)ep_combine_kernel<ST, NV>, grid, dim3(COMBINE_THREADS), smem,
                             stream, p, /*coop=*/1, c.pdl));
  return 0;
}

template <int NV>
static int launch_combine_nv(const BufferCtx& c, CombineParams& p, cudaStream_t stream) {
  const size_t row = (size_t)c.H * 2;
  const size_t budget = c.virt ? 100 * 1024 : 210 * 1024;
  if (14 * row <= budget) return launch_combine_t<14, NV>(c, p, 14 * row, stream);
  if (10 * row <= budget) return launch_combine_t<10, NV>(c, p, 10 * row, stream);
  if (6 * row <= budget) return launch_combine_t<6, NV>(c, p, 6 * row, stream);
  if (3 * row <= 220 * 1024) return launch_combine_t<3, NV>(c, p, 3 * row, stream);
  return fail(-2, "combine: H=%d does not fit a 2-stage ring", c.H);
}

template <int ST, int NV>
static int launch_prologue_t(const BufferCtx& c, PrologueParams& p, size_t smem, cudaStream_t stream) {
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_combine_prologue_kernel<ST, NV>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  // one CTA per SM (a virtual group shares the SMs between its ranks)
  int gx = c.num_sms_local / c.Rv();
  if (gx < 1) gx = 1;
  ep_combine_prologue_kernel<ST, NV><<<dim3(gx, c.Rv()), PROLOGUE_THREADS, smem, stream>>>(p);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int NV>
static int launch_prologue_nv(const BufferCtx& c, PrologueParams& p, cudaStream_t stream) {
  const size_t row = (size_t)c.H * 2;
  const size_t budget = 200 * 1024;
  if (12 * row <= budget) return launch_prologue_t<10, NV>(c, p, 12 * row, stream);
  if (6 * row <= budget) return launch_prologue_t<4, NV>(c, p, 6 * row, stream);
  if (4 * row <= budget) return launch_prologue_t<2, NV>(c, p, 4 * row, stream);
  return fail(-2, "combine prologue: H=%d does not fit a 2-stage ring", c.H);
}

}  // namespace mep

using namespace mep;

extern "C" {

int mep_launch_combine_prologue(const void* ctx_, const int32_t* link, const int32_t* cu_seqlens,
                                cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  PrologueParams p;
  p.sync = c.sync(KID_PROLOGUE);
  p.H = c.H; p.epn = c.epn; p.NvS = c.NvS; p.hidden_stride = c.hidden_stride;
  p.rank_base = c.virt ? 0 : c.rank;
  p.hidden = (__nv_bfloat16*)c.hidden; p.link = link; p.cu_seqlens = cu_seqlens;
  const int nvec = c.H / 8;
  const int nv = (nvec + PROLOGUE_ACC_THREADS - 1) / PROLOGUE_ACC_THREADS;
  if (nv <= 1) return launch_prologue_nv<1>(c, p, stream);
  if (nv <= 2) return launch_prologue_nv<2>(c, p, stream);
  if (nv <= 4) return launch_prologue_nv<4>(c, p, stream);
  if (nv <= 10) return launch_prologue_nv<10>(c, p, stream);
  return fail(-3, "combine prologue: H=%d is larger than 16384", c.H);
}

// Finish a pushed combine: push [R][push_stride] bf16 rows / wpush [R][wpush_stride] fp32 scalars
// are the symmetric staging buffers; row_scalar (may be null) is this rank's per-row scalar to
// send home (route-weight grads); out [Rv][S][H], w_out [Rv][S][K] or null.
int mep_launch_push_reduce(const void* ctx_, const void* push, int64_t push_stride, void* wpush,
                           int64_t wpush_stride, const int32_t* src_info, const float* row_scalar,
                           const int32_t* cu_seqlens, void* out, float* w_out, int grid_x,
                           cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  PushReduceParams p;
  p.sync = c.sync(KID_COMBINE);
  p.S = c.S; p.K = c.K; p.H = c.H; p.epn = c.epn; p.N = c.N; p.NvS = c.NvS;
  p.push_stride = push_stride; p.wpush_stride = wpush_stride;
  p.push = (const __nv_bfloat16*)push; p.wpush = (float*)wpush; p.src_info = src_info;
  p.row_scalar = row_scalar; p.cu_seqlens = cu_seqlens; p.out = (__nv_bfloat16*)out; p.w_out = w_out;
  dim3 grid(grid_x > 0 ? grid_x : c.num_sms, c.Rv());
  MEP_CUDA_OK(launch_coop((const void*)ep_push_reduce_kernel, grid, dim3(PUSH_REDUCE_THREADS), 0, stream, p));
  return 0;
}

// dst [Rv][N], out [Rv][S][H] bf16, w_out [Rv][S][K] fp32 or null.
int mep_launch_combine(const void* ctx_, const int32_t* dst, void* out, float* w_out,
                       cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  if (c.H % 8 != 0) return fail(-1, "combine needs H %% 8 == 0 (got %d)", c.H);
  CombineParams p;
  p.sync = c.sync(KID_COMBINE);
  p.S = c.S; p.K = c.K; p.H = c.H; p.N = c.N; p.NvS = c.NvS;
  p.hidden_stride = c.hidden_stride; p.weights_off = c.ml.weights_off;
  p.dst = dst; p.hidden = (const __nv_bfloat16*)c.hidden;
  p.out = (__nv_bfloat16*)out; p.w_out = w_out;
  const int nvec = c.H / 8;
  const int nv = (nvec + COMBINE_ACC_THREADS - 1) / COMBINE_ACC_THREADS;
  if (nv <= 1) return launch_combine_nv<1>(c, p, stream);
  if (nv <= 2) return launch_combine_nv<2>(c, p, stream);
  if (nv <= 4) return launch_combine_nv<4>(c, p, stream);
  if (nv <= 10) return launch_combine_nv<10>(c, p, stream);
  return fail(-3, "combine: H=%d is larger than 16384", c.H);
}

}  // extern "C"
