// Device-side synchronisation primitives: bounded waits, a per-rank software grid barrier
// and the cross-rank barrier on peer-memory flags.
//
// Counterparts in the reference: grid_sync (moonep/_common.py:249-271), cross_rank_barrier
// (_common.py:274-346).  Differences that matter:
//  * every wait is bounded.  The reference spins for up to 100 s and then traps
//    (_common.py:36,335-341), which destroys the CUDA context.  Here a wait that runs out
//    records {code, kernel, phase, rank, peer, observed, expected} in a host-visible status
//    block, raises a rank-local abort flag so that later waits of the same rank fall through,
//    and the kernel runs to its end and returns.  The host raises an exception afterwards.
//  * the cross-rank flags are monotonically increasing epochs (one slot per peer) instead of
//    a self-resetting +1/-1 counter: a slot is written by exactly one peer, a late or early
//    arrival can never be confused with another round, and no reset traffic is needed.
//  * "rank" is rank_base + blockIdx.y.  A real launch has gridDim.y == 1.  A single-GPU
//    launch with gridDim.y == R runs all R ranks of a virtual EP group as ONE cooperative
//    kernel over R chunks of the same address space, which is how the multi-rank paths are
//    tested on one device.
#pragma once
#include <cstdint>

namespace mep {

enum StatusCode : int {
  ST_OK = 0,
  ST_TIMEOUT_GRID = 1,     // rank-local grid barrier ran out
  ST_TIMEOUT_PEER = 2,     // a peer's flag never reached the expected epoch
  ST_TIMEOUT_MBAR = 3,     // an mbarrier (TMA completion) wait ran out
  ST_BAD_INDEX = 4,        // a computed row / slot index was outside its extent
  ST_TIMEOUT_ARRIVAL = 5,  // fused path: a tile's rows never arrived
};

enum KernelId : int {
  KID_SYNC = 1, KID_PLAN = 2, KID_DISPATCH = 3, KID_EXPAND = 4, KID_PROLOGUE = 5,
  KID_COMBINE = 6, KID_PREFETCH = 7, KID_REDUCE = 8, KID_GEMM = 9,
};

// Per-(virtual-)rank local synchronisation state, 8 int32:
//   [0] grid barrier word   [1] barrier epoch   [2] abort flag   [3] plan parity
constexpr int SYNC_STATE_INTS = 8;

// Device-side phase stamps (tracing): with -DMEP_PHASE_STAMPS a kernel's CTAs record
// %globaltimer at a few named points into trace[kernel][cta][phase] (int64 ns), which the host
// reads after the run (Buffer.phase_stamps(), bench.py --trace).  Without the flag phase_stamp()
// is empty and the kernels carry nothing of it.
constexpr int TRACE_KERNELS = 4;      // 0 dispatch, 1 combine, 2 fused GEMM producer, 3 fused GEMM copy warp
constexpr int TRACE_CTAS = 320;
constexpr int TRACE_PHASES = 8;
#ifdef MEP_PHASE_STAMPS
__device__ __forceinline__ void phase_stamp(long long* trace, int kernel, int cta, int phase) {
  if (trace != nullptr && cta < TRACE_CTAS && phase < TRACE_PHASES) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    trace[((size_t)kernel * TRACE_CTAS + cta) * TRACE_PHASES + phase] = (long long)t;
  }
}
#else
__device__ __forceinline__ void phase_stamp(long long*, int, int, int) {}
#endif

struct SyncCtx {
  long long* trace;        // phase stamps, or null (see phase_stamp)
  int rank_base;
  int R;
  int32_t* meta;           // symmetric meta buffer, chunk of rank 0
  int64_t meta_stride;     // int32 elements between consecutive ranks' chunks
  int64_t flags_off;       // offset of FLAGS[R] inside a chunk
  int32_t* sync_state;     // local, [gridDim.y][SYNC_STATE_INTS]
  int32_t* status;         // host-visible, [8]
  unsigned long long timeout_ns;
  int kernel_id;
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int32_t* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int32_t* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(int32_t* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(int32_t* p, int v) {
  asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(int32_t* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// Orders async-proxy (TMA / bulk copy) accesses against generic-proxy accesses.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Programmatic dependent launch (reference: moonep/_common.py:393-406).  A kernel launched with
// the programmatic-serialisation attribute may start while its predecessor on the stream still
// runs; pdl_wait() blocks until the predecessor has COMPLETED and its writes are visible, so
// everything before it (barrier set-up, shared-memory initialisation, parameter decoding) overlaps
// the predecessor's tail.  pdl_launch_dependents() in the predecessor allows that early start.
// Both are no-ops in kernels that are launched plainly.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ int32_t* sync_state_of(const SyncCtx& c) {
  return c.sync_state + (size_t)blockIdx.y * SYNC_STATE_INTS;
}
__device__ __forceinline__ bool aborted(const SyncCtx& c) {
  return ld_relaxed_gpu(sync_state_of(c) + 2) != 0;
}

// Record the first failure and raise the rank's abort flag.
static __device__ __noinline__ void report_failure(const SyncCtx& c, int code, int phase, int peer,
                                            int observed, int expected) {
  int32_t* st = sync_state_of(c);
  atomicExch(st + 2, 1);
  if (atomicCAS(c.status, 0, code) == 0) {
    c.status[1] = c.kernel_id;
    c.status[2] = phase;
    c.status[3] = c.rank_base + (int)blockIdx.y;
    c.status[4] = peer;
    c.status[5] = observed;
    c.status[6] = expected;
    __threadfence_system();
  }
}

// Spin until pred() holds or the time budget runs out.  Returns false on timeout or when the
// rank was already aborted.  pred must be cheap and side-effect free.
template <class Pred>
__device__ __forceinline__ bool bounded_wait(const SyncCtx& c, Pred pred) {
  if (pred()) return true;
  unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    if (pred()) return true;
    if ((++spins & 63u) == 0) {
      if (aborted(c)) return false;
      if (globaltimer_ns() - t0 > c.timeout_ns) return false;
    }
  }
}

// Rank-local grid barrier over the gridDim.x CTAs that share blockIdx.y.  Must be reached by
// every thread of every such CTA; the launch must be cooperative so that all of them are
// resident.  sys != 0 makes earlier writes of this CTA visible at system scope first.
__device__ __forceinline__ void grid_sync(const SyncCtx& c, int phase, bool sys = false) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (sys) fence_sys(); else fence_gpu();
    int32_t* bar = sync_state_of(c);
    const unsigned n = gridDim.x;
    if (n > 1) {
      unsigned inc = blockIdx.x == 0 ? (0x80000000u - (n - 1)) : 1u;
      unsigned old = atomicAdd((unsigned*)bar, inc);
      bool ok = bounded_wait(c, [&] {
        return ((old ^ (unsigned)ld_acquire_gpu(bar)) & 0x80000000u) != 0;
      });
      if (!ok && !aborted(c)) report_failure(c, ST_TIMEOUT_GRID, phase, -1, (int)old, (int)n);
    }
    fence_gpu();
  }
  __syncthreads();
}

// The cross-rank part of the barrier, executed by ONE CTA of the rank (all its threads):
// publish this rank's next epoch into every peer's flag slot, then wait until every peer's
// epoch has reached it.  Writes made by this CTA (and everything it has observed through
// acquire operations) before the call are visible to the peers' readers afterwards.
__device__ __forceinline__ void cta_cross_rank_exchange(const SyncCtx& c, int phase) {
  __shared__ int s_epoch;
  int32_t* st = sync_state_of(c);
  const int rank = c.rank_base + (int)blockIdx.y;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_epoch = st[1] + 1;
    st[1] = s_epoch;
  }
  __syncthreads();
  const int epoch = s_epoch;
  for (int p = threadIdx.x; p < c.R; p += blockDim.x) {
    int32_t* theirs = c.meta + (size_t)p * c.meta_stride + c.flags_off + rank;
    fence_sys();
    st_release_sys(theirs, epoch);
  }
  for (int p = threadIdx.x; p < c.R; p += blockDim.x) {
    const int32_t* mine = c.meta + (size_t)rank * c.meta_stride + c.flags_off + p;
    int seen = 0;
    bool ok = bounded_wait(c, [&] {
      seen = ld_acquire_sys(mine);
      return (int)(seen - epoch) >= 0;
    });
    if (!ok && !aborted(c)) report_failure(c, ST_TIMEOUT_PEER, phase, p, seen, epoch);
  }
  __syncthreads();
}

// Cross-rank barrier: when it returns, every write (generic or completed bulk copy) that any
// CTA of any rank issued before its own call is visible to every thread of this rank.
__device__ __forceinline__ void cross_rank_barrier(const SyncCtx& c, int phase) {
  grid_sync(c, phase, /*sys=*/true);
  if (blockIdx.x == 0) cta_cross_rank_exchange(c, phase);
  grid_sync(c, phase + 1000, /*sys=*/false);
  fence_proxy_async();
}

}  // namespace mep
