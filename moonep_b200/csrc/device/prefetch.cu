// prefetch_weight: owners push the weights (and optional scale tensors) of experts that the
// plan made redundant into the prefetch slots of the ranks that will compute them.
//
// Reference counterpart: PrefetchKernel (moonep/prefetch.py:227-470), which moves 128x128 /
// 128x256 tiles with 2-D TMA and needs a retiled view for scale tensors
// (prefetch.py:524-543).  An expert matrix and a prefetch slot are both CONTIGUOUS byte
// ranges, so here every tensor is an opaque byte string per expert, cut into 16 KB chunks:
// one local bulk load per chunk fans out to one bulk store per destination slot.  Any dtype
// and any per-expert shape whose byte size is a multiple of 16 rides the same path (bf16
// weights, packed MXFP4 bytes, ue8m0 / fp32 block scales) with no retiling.
#include <cuda_runtime.h>

#include "common/layout.h"
#include "device/sync.cuh"
#include "device/tma.cuh"
#include "host/ctx.h"
#include "host/errors.h"

namespace mep {

constexpr int PF_MAX_TENSORS = 6;
constexpr int PF_THREADS = 64;
// Chunk size (bytes) is a template parameter of the kernel: 32 KB on a real group, 16 KB in the
// single-GPU virtual group, whose CTAs must share the SMs.

struct PrefetchParams {
  SyncCtx sync;
  int epn, n_tensors;
  const int32_t* etc;                       // [Rv][R*epn]
  const uint8_t* local[PF_MAX_TENSORS];     // [Rv][epn][expert_bytes]
  uint8_t* pool[PF_MAX_TENSORS];            // slot (d, b) at pool + d*rank_stride + b*expert_bytes
  int64_t expert_bytes[PF_MAX_TENSORS];
  int64_t rank_stride[PF_MAX_TENSORS];      // bytes between ranks' pools
};

template <int ST, uint32_t PF_CHUNK>
__global__ void __launch_bounds__(PF_THREADS, 1) ep_prefetch_kernel(const PrefetchParams p) {
  constexpr int LA = ST / 2;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[ST];
  const SyncCtx& sc = p.sync;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vr = blockIdx.y, rank = sc.rank_base + vr;
  const int G = gridDim.x, c = blockIdx.x;
  const int R = sc.R, epn = p.epn;
  uint8_t* ring = smem_raw;
  int32_t* cnt = reinterpret_cast<int32_t*>(smem_raw + (size_t)ST * PF_CHUNK);  // [epn]
  int32_t* start = cnt + epn;                                                   // [epn]
  int32_t* cursor = start + epn;                                                // [epn]
  int32_t* active = cursor + epn;                                               // [epn]
  int32_t* dests = active + epn;                                                // [R*epn] CSR
  __shared__ int n_active;

  if (tid == 0) {
    for (int s = 0; s < ST; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    n_active = 0;
  }
  for (int i = tid; i < epn; i += PF_THREADS) { cnt[i] = 0; cursor[i] = 0; }
  __syncthreads();
  // which of my experts go where: count, prefix, fill (slot id = d*epn + b)
  const int32_t* etc = p.etc + (size_t)vr * R * epn;
  for (int i = tid; i < R * epn; i += PF_THREADS) {
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
  for (int i = tid; i < R * epn; i += PF_THREADS) {
    int e = etc[i];
    if (e >= 0 && e / epn == rank) {
      int le = e - rank * epn;
      dests[start[le] + atomicAdd(&cursor[le], 1)] = i;
    }
  }
  __syncthreads();
  const int na = n_active;

  if (warp == 0 && na > 0) {
    // flattened work list: (tensor, active expert, chunk); this CTA takes items c, c+G, ...
    int64_t items_before[PF_MAX_TENSORS + 1];
    items_before[0] = 0;
    for (int t = 0; t < p.n_tensors; ++t) {
      int64_t nch = (p.expert_bytes[t] + PF_CHUNK - 1) / PF_CHUNK;
      items_before[t + 1] = items_before[t] + nch * na;
    }
    const int64_t total = items_before[p.n_tensors];
    const int64_t n_items = c < total ? (total - c + G - 1) / G : 0;
    auto decode = [&](int64_t j, const uint8_t*& src, uint32_t& bytes, int& t_out, int& le_out,
                      int64_t& off_out) {
      int64_t idx = c + j * G;
      int t = 0;
      while (t + 1 < p.n_tensors && idx >= items_before[t + 1]) ++t;
      idx -= items_before[t];
      int64_t nch = (p.expert_bytes[t] + PF_CHUNK - 1) / PF_CHUNK;
      int a = (int)(idx / nch);
      int64_t ch = idx - (int64_t)a * nch;
      int le = active[a];
      int64_t off = ch * PF_CHUNK;
      int64_t rem = p.expert_bytes[t] - off;
      bytes = (uint32_t)(rem < (int64_t)PF_CHUNK ? rem : (int64_t)PF_CHUNK);
      src = p.local[t] + ((size_t)vr * epn + le) * p.expert_bytes[t] + off;
      t_out = t; le_out = le; off_out = off;
    };
    if (lane == 0) {
      for (int64_t j = 0; j < LA && j < n_items; ++j) {
        const uint8_t* src; uint32_t bytes; int t, le; int64_t off;
        decode(j, src, bytes, t, le, off);
        mbar_expect_tx(&full[j], bytes);
        bulk_g2s(ring + (size_t)j * PF_CHUNK, src, bytes, &full[j]);
      }
    }
    __syncwarp();
    for (int64_t j = 0; j < n_items; ++j) {
      const int s = (int)(j % ST);
      const uint8_t* src; uint32_t bytes; int t, le; int64_t off;
      decode(j, src, bytes, t, le, off);
      mbar_wait(sc, &full[s], (uint32_t)(j / ST) & 1u, 10);
      const int nd = cnt[le];
      for (int q = lane; q < nd; q += 32) {
        int slot = dests[start[le] + q];
        int d = slot / epn, b = slot - d * epn;
        bulk_s2g(p.pool[t] + (size_t)d * p.rank_stride[t] + (size_t)b * p.expert_bytes[t] + off,
                 ring + (size_t)s * PF_CHUNK, bytes);
      }
      bulk_commit();
      if (j + LA < n_items) {
        bulk_wait_read<ST - LA>();
        __syncwarp();
        if (lane == 0) {
          const uint8_t* src2; uint32_t bytes2; int t2, le2; int64_t off2;
          decode(j + LA, src2, bytes2, t2, le2, off2);
          const int s2 = (int)((j + LA) % ST);
          mbar_expect_tx(&full[s2], bytes2);
          bulk_g2s(ring + (size_t)s2 * PF_CHUNK, src2, bytes2, &full[s2]);
        }
      }
    }
    bulk_wait<0>();
    fence_proxy_async();
  }
  fence_sys();
  cross_rank_barrier(sc, 2);  // prefetched weights are visible on every rank
}

template <int ST, uint32_t PF_CHUNK>
static int launch_prefetch_t(const BufferCtx& c, PrefetchParams& p, cudaStream_t stream) {
  size_t smem = (size_t)ST * PF_CHUNK + sizeof(int32_t) * ((size_t)4 * c.epn + (size_t)c.epn * c.R);
  if (smem > 220 * 1024) return fail(-2, "prefetch: E=%d is too large for the slot lists", c.E);
  static thread_local size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_prefetch_kernel<ST, PF_CHUNK>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(c.num_sms_weights, c.Rv());
  MEP_CUDA_OK(launch_coop_paired((const void*)ep_prefetch_kernel<ST, PF_CHUNK>, grid, dim3(PF_THREADS), smem, stream, p));
  return 0;
}

}  // namespace mep

using namespace mep;

extern "C" {

// etc [Rv][R*epn]; for each of n tensors: local [Rv][epn][expert_bytes], pool base, bytes per
// expert (multiple of 16) and the byte stride between ranks' pools.
int mep_launch_prefetch(const void* ctx_, const int32_t* etc, int n, const void* const* local,
                        void* const* pool, const int64_t* expert_bytes, const int64_t* rank_stride,
                        cudaStream_t stream) {
  const BufferCtx& c = *(const BufferCtx*)ctx_;
  if (n < 1 || n > PF_MAX_TENSORS) return fail(-1, "prefetch: %d tensors (1..%d)", n, PF_MAX_TENSORS);
  PrefetchParams p;
  p.sync = c.sync(KID_PREFETCH, /*channel=*/1);
  p.epn = c.epn; p.n_tensors = n; p.etc = etc;
  for (int t = 0; t < n; ++t) {
    if (expert_bytes[t] % 16 != 0 || rank_stride[t] % 16 != 0 ||
        ((uintptr_t)local[t] | (uintptr_t)pool[t]) % 16 != 0)
      return fail(-3, "prefetch: tensor %d is not 16-byte aligned / sized", t);
    p.local[t] = (const uint8_t*)local[t]; p.pool[t] = (uint8_t*)pool[t];
    p.expert_bytes[t] = expert_bytes[t]; p.rank_stride[t] = rank_stride[t];
  }
  if (c.virt) return launch_prefetch_t<4, 16 * 1024>(c, p, stream);
  return launch_prefetch_t<6, 32 * 1024>(c, p, stream);
}

}  // extern "C"
