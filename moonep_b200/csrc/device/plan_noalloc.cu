// See plan_noalloc.h: the planner for one rank, with its scratch in a static device array.
#include "device/plan_noalloc.h"

#include <cuda_runtime.h>

#include "common/layout.h"
#include "device/planner_core.cuh"
#include "device/sync.cuh"
#include "host/errors.h"

namespace mep {

// Working tables of the solver (tpe_cumsum, alloc, alloc_cumsum, expert_off: R*E each), then
// 8 words of rank-local sync state (only the abort flag is used here) and 8 status words.
constexpr int NOALLOC_TABLE_INTS = 4 * MEP_NOALLOC_MAX_RE;
constexpr int NOALLOC_INTS = NOALLOC_TABLE_INTS + 16;
static __device__ __align__(256) int32_t g_plan_scratch[NOALLOC_INTS];

struct LocalPlanParams {
  PlanParams plan;
  const int32_t* tpe_all;
  int rank;
  int32_t* status_out;
};

__global__ void __launch_bounds__(PLAN_THREADS, 1) ep_plan_local_kernel(const LocalPlanParams lp) {
  extern __shared__ int32_t smem[];
  const PlanParams& p = lp.plan;
  const SyncCtx& sc = p.sync;
  const int R = sc.R, E = p.E, K = p.K, rank = lp.rank;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the array keeps the previous call's contents: the abort flag and the status block must
  // start at zero
  if (tid < 16) p.scratch[NOALLOC_TABLE_INTS + tid] = 0;
  __syncthreads();
  plan_solve(p, rank, lp.tpe_all, smem);
  __syncthreads();
  const int32_t* tpe_cumsum = p.scratch;
  const int32_t* alloc_cumsum = p.scratch + (size_t)2 * R * E;
  const int32_t* expert_off = p.scratch + (size_t)3 * R * E;
  int32_t* cnt = smem;
  for (int e = tid; e < E; e += PLAN_THREADS)
    cnt[e] = rank > 0 ? tpe_cumsum[(size_t)(rank - 1) * E + e] : 0;
  __syncthreads();
  if (warp == 0) {
    for (int64_t b = 0; b < p.N; b += 32) {
      int64_t i = b + lane;
      bool valid = i < p.N;
      int e = valid ? p.topk[i] : -1 - lane;
      if (valid && (unsigned)e >= (unsigned)E) { report_failure(sc, ST_BAD_INDEX, 10, -1, e, E); e = 0; }
      unsigned m = __match_any_sync(0xffffffffu, e);
      int before = __popc(m & ((1u << lane) - 1));
      int base = valid ? cnt[e] : 0;
      __syncwarp();
      if (valid && before == 0) cnt[e] = base + __popc(m);
      __syncwarp();
      if (valid) p.dst[i] = base + before;
    }
  }
  __syncthreads();
  for (int64_t i = tid; i < p.N; i += PLAN_THREADS) {
    int e = p.topk[i];
    if ((unsigned)e >= (unsigned)E) e = 0;
    int g = p.dst[i];
    const int32_t* ac = alloc_cumsum + (size_t)e * R;
    int lo = 0, hi = R;
    while (lo < hi) {
      int mid = (lo + hi) >> 1;
      if (ac[mid] > g) hi = mid; else lo = mid + 1;
    }
    int dest = lo;
    if (dest >= R) { report_failure(sc, ST_BAD_INDEX, 20, e, g, ac[R - 1]); dest = R - 1; }
    int prev = dest > 0 ? ac[dest - 1] : 0;
    int64_t row = (int64_t)expert_off[(size_t)dest * E + e] + (g - prev);
    if (row < 0 || row >= p.NvS) { report_failure(sc, ST_BAD_INDEX, 21, dest, (int)row, (int)p.NvS); row = 0; }
    p.dst[i] = (int)((int64_t)dest * p.NvS + row);
  }
  __syncthreads();
  for (int t = tid; t < p.S; t += PLAN_THREADS) {
    int32_t* d = p.dst + (size_t)t * K;
    int dr[MAX_TOPK];
    for (int k = 0; k < K; ++k) dr[k] = (int)(d[k] / p.NvS);
    for (int k = K - 1; k >= 1; --k) {
      bool dup = false;
      for (int j = 0; j < k; ++j) dup |= dr[j] == dr[k];
      if (dup) d[k] = -d[k] - 1;
    }
  }
  __syncthreads();
  if (lp.status_out != nullptr && tid < 8) lp.status_out[tid] = sc.status[tid];
}

}  // namespace mep

using namespace mep;

extern "C" int mep_plan_local_noalloc(const int32_t* tpe_all, const int32_t* topk, int rank, int R,
                                      int E, int S, int K, int token_padding, int32_t* dst,
                                      int32_t* cu_seqlens, int32_t* zero_fill, int32_t* etc,
                                      int32_t* remote_stats, int32_t* status, cudaStream_t stream) {
  if (R < 1 || E < 1 || E % R != 0 || rank < 0 || rank >= R || S < 1 || K < 1 || K > MAX_TOPK ||
      R > MAX_RANKS || token_padding < 1)
    return fail(-1, "plan_local_noalloc: bad sizes R=%d E=%d rank=%d S=%d K=%d", R, E, rank, S, K);
  if ((long long)R * E > MEP_NOALLOC_MAX_RE)
    return fail(-2, "plan_local_noalloc: R*E = %lld exceeds the built-in scratch (max %d); use a Buffer",
                (long long)R * E, MEP_NOALLOC_MAX_RE);
  const int64_t NvS = nvs_rows(S, K, E / R, token_padding);
  if (NvS > MAX_NVS || (int64_t)R * NvS > INT32_MAX)
    return fail(-3, "plan_local_noalloc: NvS=%lld does not fit the slot encoding", (long long)NvS);
  // Device address of the static array for the CURRENT device.  The array's name is only a
  // host-side handle here; a kernel must be given this address.  It is looked up on every call (a
  // host-side table lookup once the module is loaded) rather than cached: nothing can go stale
  // after a device reset, and host threads share no mutable state.
  void* ptr = nullptr;
  MEP_CUDA_OK(cudaGetSymbolAddress(&ptr, g_plan_scratch));
  if (ptr == nullptr) return fail(-4, "plan_local_noalloc: the scratch array has no device address");
  int32_t* scratch = (int32_t*)ptr;
  LocalPlanParams lp;
  PlanParams& p = lp.plan;
  p.sync.trace = nullptr; p.sync.rank_base = rank; p.sync.R = R; p.sync.meta = nullptr; p.sync.meta_stride = 0;
  p.sync.flags_off = 0;
  p.sync.sync_state = scratch + NOALLOC_TABLE_INTS;       // [8], abort flag at word 2
  p.sync.status = scratch + NOALLOC_TABLE_INTS + 8;       // [8]
  p.sync.timeout_ns = 0; p.sync.kernel_id = KID_PLAN;
  p.E = E; p.epn = E / R; p.S = S; p.K = K; p.token_padding = token_padding;
  p.N = (int64_t)S * K; p.NvS = NvS; p.tpe_off = 0; p.link_off = 0; p.src_off = 0;
  p.topk = topk; p.tpe = nullptr; p.dst = dst; p.cu_seqlens = cu_seqlens; p.zero_fill = zero_fill;
  p.etc = etc; p.remote_stats = remote_stats;
  p.scratch = scratch; p.scratch_ints = NOALLOC_INTS;
  p.send_order = nullptr; p.arrive_off = 0; p.n_arrive = 0;
  lp.tpe_all = tpe_all; lp.rank = rank; lp.status_out = status;
  const size_t smem = sizeof(int32_t) * (2 * (size_t)E + 4 * (size_t)R + (size_t)PLAN_WARPS * R);
  if (smem > 48 * 1024) {
    // E <= 16384 keeps this below 133 KB; raising the limit is not an allocation
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_plan_local_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  ep_plan_local_kernel<<<1, PLAN_THREADS, smem, stream>>>(lp);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}
