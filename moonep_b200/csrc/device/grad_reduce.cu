// reduce_grad: every home rank pulls the fp32 gradients that other ranks accumulated for ITS
// experts in their prefetch-slot grad buffers, adds them to its local grad in ascending
// (rank, slot) order, and then every rank zeroes its own consumed slots.
//
// Reference counterpart: GradReduceKernel (moonep/grad_reduce.py:151-389), one launch per
// projection with 128x128 2-D TMA tiles.  Here gate/up/down go through ONE launch and the
// tensors are handled as contiguous fp32 strings cut into 16 KB chunks: the accumulator
// threads seed registers from the local grad, add each remote chunk as it lands in the ring
// and store back.  The accumulation order (slot id d*epn+b ascending) is fixed, so results
// are bitwise reproducible, as the reference's tests require (tests/test_grad_reduce.py:193).
#include <cuda_runtime.h>

#include <cstdlib>
#include <string>

#include "common/layout.h"
#include "device/sync.cuh"
#include "device/tma.cuh"
#include "host/ctx.h"
#include "host/errors.h"

namespace mep {

constexpr int GR_MAX_TENSORS = 3;
constexpr int GR_ACC_THREADS = 128;
constexpr int GR_THREADS = 32 + GR_ACC_THREADS;
// Chunk size (bytes) is a template parameter of the kernel: 32 KB chunks in a 6-stage ring on a
// real group (64 KB chunks need 128 accumulator registers per thread and spill), 16 KB chunks in
// the single-GPU virtual group, whose CTAs must share the SMs.

struct GradReduceParams {
  SyncCtx sync;
  int epn, n_tensors, entry_barrier, zero_consumed;
  const int32_t* etc;                     // [Rv][R*epn]
  float* local[GR_MAX_TENSORS];           // [Rv][epn][expert_elems]
  float* pool[GR_MAX_TENSORS];            // slot (d,b) at pool + d*rank_stride + b*expert_elems
  int64_t expert_elems[GR_MAX_TENSORS];
  int64_t rank_stride[GR_MAX_TENSORS];    // elements
};

template <int ST, uint32_t GR_CHUNK>
__global__ void __launch_bounds__(GR_THREADS, 1) ep_grad_reduce_kernel(const GradReduceParams p) {
  constexpr int GR_VEC_PER_THREAD = GR_CHUNK / 16 / GR_ACC_THREADS;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[ST];
  __shared__ __align__(8) uint64_t empty[ST];
  __shared__ int n_active;
  const SyncCtx& sc = p.sync;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y, rank = sc.rank_base + vr;
  const int G = gridDim.x, c = blockIdx.x;
  const int R = sc.R, epn = p.epn;
  uint8_t* ring = smem_raw;
  int32_t* cnt = reinterpret_cast<int32_t*>(smem_raw + (size_t)ST * GR_CHUNK);  // [epn]
  int32_t* start = cnt + epn;                                                   // [epn]
  int32_t* active = start + epn;                                                // [epn]
  int32_t* srcs = active + epn;                                                 // [R*epn] CSR

  if (tid == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], GR_ACC_THREADS / 32); }
    mbar_fence_init();
    n_active = 0;
  }
  for (int i = tid; i < epn; i += GR_THREADS) cnt[i] = 0;
  __syncthreads();
  const int32_t* etc = p.etc + (size_t)vr * R * epn;
  for (int i = tid; i < R * epn; i += GR_THREADS) {
    int e = etc[i];
    if (e >= 0 && e / epn == rank) atomicAdd(&cnt[e - rank * epn], 1);
  }
  __syncthreads();
  if (warp == 0) {
    int base = 0, run = 0;
    for (int j0 = 0; j0 < epn; j0 += 32) {
      int j = j0 + lane;
      int n = j < epn ? cnt[j] : 0;
      unsigned m = __ballot_sync(0xffffffffu, n > 0);
      if (n > 0) active[base + __popc(m & ((1u << lane) - 1))] = j;
      base += __popc(m);
      int incl = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (j < epn) start[j] = run + incl - n;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) n_active = base;
  }
  __syncthreads();
  // ascending slot order per expert: each active expert's list is filled by one thread that
  // walks the whole table in order (deterministic; the table is small)
  for (int a = tid; a < n_active; a += GR_THREADS) {
    int le = active[a], want = rank * epn + le, pos = start[le];
    for (int i = 0; i < R * epn; ++i)
      if (etc[i] == want) srcs[pos++] = i;
  }
  __syncthreads();
  if (p.entry_barrier) cross_rank_barrier(sc, 1);
  const int na = n_active;

  int64_t items_before[GR_MAX_TENSORS + 1];
  items_before[0] = 0;
  for (int t = 0; t < p.n_tensors; ++t) {
    int64_t nch = (p.expert_elems[t] * 4 + GR_CHUNK - 1) / GR_CHUNK;
    items_before[t + 1] = items_before[t] + nch * na;
  }
  const int64_t total = items_before[p.n_tensors];
  const int64_t n_items = c < total ? (total - c + G - 1) / G : 0;
  auto decode = [&](int64_t j, int& t, int& le, int64_t& off_elems, uint32_t& bytes) {
    int64_t idx = c + j * G;
    t = 0;
    while (t + 1 < p.n_tensors && idx >= items_before[t + 1]) ++t;
    idx -= items_before[t];
    int64_t nch = (p.expert_elems[t] * 4 + GR_CHUNK - 1) / GR_CHUNK;
    int a = (int)(idx / nch);
    int64_t ch = idx - (int64_t)a * nch;
    le = active[a];
    off_elems = ch * (GR_CHUNK / 4);
    int64_t rem = (p.expert_elems[t] - off_elems) * 4;
    bytes = (uint32_t)(rem < (int64_t)GR_CHUNK ? rem : (int64_t)GR_CHUNK);
  };

  if (warp == 0) {
    if (lane == 0) {
      int prod = 0;
      for (int64_t j = 0; j < n_items; ++j) {
        int t, le; int64_t off; uint32_t bytes;
        decode(j, t, le, off, bytes);
        const int ns = cnt[le];
        // entry -1 is the local grad chunk itself: it seeds the accumulators, so the home
        // rank's own read is pipelined with the remote ones instead of stalling each item
        for (int q = -1; q < ns; ++q, ++prod) {
          const int s = prod % ST;
          if (prod >= ST) mbar_wait(sc, &empty[s], ((uint32_t)(prod / ST) & 1u) ^ 1u, 20);
          const float* src;
          if (q < 0) {
            src = p.local[t] + ((size_t)vr * epn + le) * p.expert_elems[t] + off;
          } else {
            int slot = srcs[start[le] + q];
            int d = slot / epn, b = slot - d * epn;
            src = p.pool[t] + (size_t)d * p.rank_stride[t] + (size_t)b * p.expert_elems[t] + off;
          }
          mbar_expect_tx(&full[s], bytes);
          bulk_g2s(ring + (size_t)s * GR_CHUNK, src, bytes, &full[s]);
        }
      }
    }
  } else {
    const int ta = tid - 32;
    int cons = 0;
    for (int64_t j = 0; j < n_items; ++j) {
      int t, le; int64_t off; uint32_t bytes;
      decode(j, t, le, off, bytes);
      const int nvec = (int)(bytes / 16);
      float4* g = reinterpret_cast<float4*>(p.local[t] + ((size_t)vr * epn + le) * p.expert_elems[t] + off);
      float4 acc[GR_VEC_PER_THREAD];
      const int ns = cnt[le];
      for (int q = -1; q < ns; ++q, ++cons) {
        const int s = cons % ST;
        mbar_wait(sc, &full[s], (uint32_t)(cons / ST) & 1u, 30);
        const float4* src = reinterpret_cast<const float4*>(ring + (size_t)s * GR_CHUNK);
#pragma unroll
        for (int i = 0; i < GR_VEC_PER_THREAD; ++i) {
          int v = ta + i * GR_ACC_THREADS;
          if (v < nvec) {
            float4 x = src[v];
            if (q < 0) {
              acc[i] = x;
            } else {
              acc[i].x += x.x; acc[i].y += x.y; acc[i].z += x.z; acc[i].w += x.w;
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
#pragma unroll
      for (int i = 0; i < GR_VEC_PER_THREAD; ++i) {
        int v = ta + i * GR_ACC_THREADS;
        if (v < nvec) g[v] = acc[i];
      }
    }
  }
  // every home rank has read what it needs before anyone clears
  cross_rank_barrier(sc, 2);
  if (!p.zero_consumed) return;
  // clear my consumed slots (local memory): the first ring stage becomes a block of zeros that one
  // thread per CTA bulk-stores over this CTA's share of every consumed slot (the copy engine
  // writes full lines at a rate that per-thread 16-byte stores of 160 threads do not reach)
  for (uint32_t i = (uint32_t)tid * 16u; i < GR_CHUNK; i += GR_THREADS * 16u)
    *reinterpret_cast<uint4*>(ring + i) = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0) {
    int pending = 0;
    for (int b = 0; b < epn; ++b) {
      if (etc[rank * epn + b] < 0) continue;
      for (int t = 0; t < p.n_tensors; ++t) {
        uint8_t* z = reinterpret_cast<uint8_t*>(p.pool[t] + (size_t)rank * p.rank_stride[t] +
                                                (size_t)b * p.expert_elems[t]);
        const int64_t bytes = p.expert_elems[t] * 4;
        for (int64_t off = (int64_t)c * GR_CHUNK; off < bytes; off += (int64_t)G * GR_CHUNK) {
          const int64_t n = bytes - off < (int64_t)GR_CHUNK ? bytes - off : (int64_t)GR_CHUNK;
          bulk_s2g(z + off, ring, (uint32_t)n);
          if (++pending == 8) { bulk_commit(); pending = 0; }
        }
      }
    }
    bulk_commit();
    bulk_wait<0>();
  }
}

template <int ST, uint32_t GR_CHUNK>
static int launch_gr_t(const BufferCtx& c, GradReduceParams& p, int grid_x, cudaStream_t stream) {
  size_t smem = (size_t)ST * GR_CHUNK + sizeof(int32_t) * ((size_t)3 * c.epn + (size_t)c.epn * c.R);
  if (smem > 220 * 1024) return fail(-2, "reduce_grad: E=%d is too large for the slot lists", c.E);
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_grad_reduce_kernel<ST, GR_CHUNK>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(grid_x > 0 ? grid_x : c.num_sms_weights, c.Rv());
  MEP_CUDA_OK(launch_coop_paired((const void*)ep_grad_reduce_kernel<ST, GR_CHUNK>, grid, dim3(GR_THREADS), smem, stream, p));
  return 0;
}

// ---- standalone cross-rank barrier ---------------------------------------------------------
struct SyncParams { SyncCtx sync; };
__global__ void __launch_bounds__(128, 1) ep_sync_kernel(const SyncParams p) {
  cta_cross_rank_exchange(p.sync, 1);
}

}  // namespace mep

using namespace mep;

extern "C" {

// etc [Rv][R*epn]; per tensor: local grad [Rv][epn][elems] fp32, pool base, elements per expert
// (multiple of 4), element stride between ranks' pools.  grid_x > 0 overrides the number of CTAs
// (the Buffer's num_sms_weights): a reduce that runs next to nothing may take more SMs.
int mep_launch_grad_reduce(const void* ctx_, const int32_t* etc, int n, void* const* local,
                           void* const* pool, const int64_t* expert_elems,
                           const int64_t* rank_stride, int entry_barrier, int zero_consumed,
                           int grid_x, cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  if (n < 1 || n > GR_MAX_TENSORS) return fail(-1, "reduce_grad: %d tensors (1..%d)", n, GR_MAX_TENSORS);
  GradReduceParams p;
  p.sync = c.sync(KID_REDUCE, /*channel=*/1);
  p.epn = c.epn; p.n_tensors = n; p.etc = etc; p.entry_barrier = entry_barrier;
  p.zero_consumed = zero_consumed;
  for (int t = 0; t < n; ++t) {
    if (expert_elems[t] % 4 != 0 || rank_stride[t] % 4 != 0 ||
        ((uintptr_t)local[t] | (uintptr_t)pool[t]) % 16 != 0)
      return fail(-3, "reduce_grad: tensor %d is not 16-byte aligned / sized", t);
    p.local[t] = (float*)local[t]; p.pool[t] = (float*)pool[t];
    p.expert_elems[t] = expert_elems[t]; p.rank_stride[t] = rank_stride[t];
  }
  if (c.virt) return launch_gr_t<4, 16 * 1024>(c, p, grid_x, stream);
  // ring geometry: MOONEP_B200_GR_RING = <stages>x<KB> selects one of the built variants (tuning)
  static int cfg = -1;
  if (cfg < 0) {
    const char* e = getenv("MOONEP_B200_GR_RING");
    cfg = 0;
    if (e != nullptr) {
      const std::string v(e);
      cfg = v == "4x16" ? 1 : v == "8x16" ? 2 : v == "12x16" ? 3 : v == "16x8" ? 4 : v == "4x32" ? 5 : v == "6x32" ? 6 : 0;
    }
  }
  switch (cfg) {
    case 1: return launch_gr_t<4, 16 * 1024>(c, p, grid_x, stream);
    case 3: return launch_gr_t<12, 16 * 1024>(c, p, grid_x, stream);
    case 4: return launch_gr_t<16, 8 * 1024>(c, p, grid_x, stream);
    case 5: return launch_gr_t<4, 32 * 1024>(c, p, grid_x, stream);
    case 6: return launch_gr_t<6, 32 * 1024>(c, p, grid_x, stream);
    default: return launch_gr_t<8, 16 * 1024>(c, p, grid_x, stream);
  }
}

// Pure cross-rank barrier (one CTA per rank).
int mep_launch_sync(const void* ctx_, cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  SyncParams p;
  p.sync = c.sync(KID_SYNC);
  dim3 grid(1, c.Rv());
  MEP_CUDA_OK(launch_coop((const void*)ep_sync_kernel, grid, dim3(128), 0, stream, p));
  return 0;
}

}  // extern "C"
