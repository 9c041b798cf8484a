// Host-side description of one Buffer: sizes, the symmetric buffers and the local scratch.
// Created once (mep_ctx_create) and passed by handle to every launcher, like the `ctx` dict
// the reference threads through its launch_* functions (moonep/api.py:200-414).
//
// virt != 0 marks a single-GPU virtual group: the "symmetric" buffers hold all R chunks on
// this device, every per-rank local tensor is stacked [R, ...] contiguously, and every
// kernel is launched with gridDim.y == R so that one cooperative launch runs all ranks.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "common/layout.h"
#include "device/sync.cuh"

namespace mep {

struct BufferCtx {
  int rank, R, virt;
  int E, epn, S, K, H, token_padding, num_sms, num_sms_local, num_sms_weights;
  int64_t N, NvS;
  void* hidden;            // bf16 [R][hidden_stride_rows][H], symmetric
  void* hidden2;           // optional second row buffer of the same geometry (null until enabled)
  int64_t hidden_stride;   // rows between consecutive ranks' shards
  int32_t* meta;           // int32 [R][meta_stride], symmetric
  int64_t meta_stride;
  MetaLayout ml;
  int32_t* sync_state;     // [2 channels][Rv][SYNC_STATE_INTS]
  int32_t* status;         // host-visible [8]
  int32_t* plan_scratch;   // [Rv][plan_scratch_ints]
  int64_t plan_scratch_ints;
  unsigned long long timeout_ns;
  int sm_count;
  long long* trace;        // device buffer of phase stamps, or null
  int pdl;                 // chain plan -> dispatch -> expand and prologue -> combine programmatically

  int Rv() const { return virt ? R : 1; }
  // Row buffer that a launch with the given shard index works on (null when it does not exist).
  // The choice is a launch ARGUMENT: nothing in the context changes between launches, so
  // dispatches into different shards may be issued from different threads or streams.
  void* shard_base(int shard) const { return shard == 0 ? hidden : (shard == 1 ? hidden2 : nullptr); }
  // channel 0: dispatch / combine; channel 1: prefetch_weight / reduce_grad.  Each channel has
  // its own flag slots, epoch and grid-barrier word, so one kernel of each family may be in
  // flight at the same time (on different streams) without disturbing the other's barriers.
  SyncCtx sync(int kernel_id, int channel = 0) const {
    SyncCtx s;
    s.trace = trace;
    s.rank_base = virt ? 0 : rank;
    s.R = R;
    s.meta = meta;
    s.meta_stride = meta_stride;
    s.flags_off = ml.flags_off + (int64_t)channel * align_up64(R, 32);
    s.sync_state = sync_state + (size_t)channel * Rv() * SYNC_STATE_INTS;
    s.status = status;
    s.timeout_ns = timeout_ns;
    s.kernel_id = kernel_id;
    return s;
  }
};

// Scratch ints per rank needed by the planner: tpe_cumsum[R*E] + alloc[E*R] +
// alloc_cumsum[E*R] + expert_off[R*E] + per-CTA histograms [num_sms*E].
inline int64_t plan_scratch_ints(int R, int E, int num_sms) {
  return (int64_t)4 * R * E + (int64_t)num_sms * E;
}

// Cooperative launch helper: all CTAs of grid (gx, gy) must be co-resident.
template <class Params>
inline cudaError_t launch_coop(const void* kernel, dim3 grid, dim3 block, size_t smem,
                               cudaStream_t stream, Params& params) {
  void* args[] = {(void*)&params};
  return cudaLaunchCooperativeKernel(kernel, grid, block, args, smem, stream);
}

// Launch of a kernel that FOLLOWS another kernel of the same chain on the stream.  With pdl != 0
// (and outside stream capture) it carries the programmatic-serialisation attribute: the kernel
// may be scheduled while its predecessor still runs and must call pdl_wait() before it touches
// anything the predecessor wrote.  coop != 0 adds the cooperative attribute.
template <class Params>
inline cudaError_t launch_chained(const void* kernel, dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Params& params, int coop, int pdl) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (pdl && (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)) pdl = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (coop) { attr[n].id = cudaLaunchAttributeCooperative; attr[n].val.cooperative = 1; ++n; }
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)n;
  void* args[] = {(void*)&params};
  return cudaLaunchKernelExC(&cfg, kernel, args);
}

// Same, but the CTAs are placed as clusters of two (x-neighbours share one TPC).  The copy kernels
// that run NEXT TO a CTA-pair GEMM use it: they then occupy whole SM pairs, so every SM they leave
// free still has a free partner for a GEMM pair, whichever kernel the hardware places first.
// The kernels themselves use no cluster feature.  Odd grids fall back to the plain launch.
template <class Params>
inline cudaError_t launch_coop_paired(const void* kernel, dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, Params& params) {
  if (grid.x % 2 != 0) return launch_coop(kernel, grid, block, smem, stream, params);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  void* args[] = {(void*)&params};
  return cudaLaunchKernelExC(&cfg, kernel, args);
}

}  // namespace mep
