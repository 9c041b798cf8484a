// Grouped bf16 GEMM for sm_100a on the 5th-generation tensor cores: tcgen05.mma issued by one
// thread per CTA, operands staged in shared memory by tiled TMA loads (no cluster multicast),
// fp32 accumulators in tensor memory, read back with tcgen05.ld for fused epilogues.
//
// The reference ships no GEMM: it hands cu_seqlens and the [2*epn, H, H'] compute view to the
// host framework's "VM group GEMM" (README.md:45-68).  This kernel is that GEMM.  One
// persistent CTA per SM walks a static tile list derived on the device from cu_seqlens (no
// host synchronisation), with three warp roles:
//   warp 0      TMA producer        (4-stage ring of 128x64 A and 256x64 B tiles, 48 KB each)
//   warp 1      MMA issuer          (128x256x16 UMMAs, two 256-column TMEM accumulators)
//   warps 2..5  epilogue            (TMEM -> registers -> global, plain stores or staged TMA
//                                   stores), overlapped with the next tile's main loop through
//                                   the second accumulator
// Modes:
//   token-major (groups partition the rows of A and C):
//        C[rows of g] = A[rows of g] * B[g]     B K-major ([N][K]) or MN-major ([K][N])
//        epilogues: bf16 store, fp32 store, or SwiGLU: the tile holds 128 gate and 128 up
//        columns of the same output columns; writes gate, up and silu(gate)*up*row_scale.
//        Up to two K segments accumulate into one tile (dX = dG*Wg^T + dU*Wu^T).
//        PUSH epilogue (GEMM fused with the combine all-to-all): each finished row segment is
//        stored, over NVLink, straight into the slot of its (token, k) entry in the token's
//        HOME rank's staging buffer, so the transfer overlaps the math tile by tile; the home
//        rank then only sums K local rows per token.
//   weight-grad (groups partition the REDUCTION dimension):
//        D[g] (+)= A[rows of g]^T * B[rows of g]   both operands MN-major, fp32 output by TMA
//        store / reduce-add; or (template SGD) the optimizer step fused in: the accumulator is
//        applied straight to the bf16 weights, w = bf16(w - lr * acc), through a per-warp TMA
//        ring of weight blocks, for every local expert that has no replica this step.  Those
//        kernels run eight epilogue warps (two per quarter of the accumulator's lanes, one half
//        of the columns each) and take their split of the shared memory at launch.
// Group g < split reads/writes allocation 0 (local experts), g >= split allocation 1 (this
// rank's prefetch / reduce slots): the [2*epn] compute view never has to be contiguous.
// CTA pairs (template TWO, clusters of two CTAs, tcgen05 cta_group::2): the leader issues
// 256x256x16 MMAs over both CTAs' shared memory; each CTA stages its own 128 rows of A and half
// of the B tile (32 KB per k-block instead of 48 KB, six stages), which lifts the single-CTA
// kernel's limit of 12 KB of operand reads per MMA.  Both CTAs' loads count on the LEADER's full
// barrier, on which only the leader's producer arrives (expecting the bytes of both): a per-stage
// arrival from the peer over the cluster network measured 2x slower overall.  Token-major pairs
// cover 256 rows of one group; weight-grad pairs 256 rows of the weight matrix.
// Measured A/B (32 groups x 1024 rows, H=7168, H'=2048, interleaved runs under the power cap):
// pairs +13% gate/up, +13% down, +18% down dgrad, +7% gate/up dgrad, +24% weight grad.
// Fused dispatch (template DISP, token-major kernels whose A operand is the dispatched rows): a
// seventh warp per CTA sends this rank's token rows to their destination ranks while the other
// warps compute, and the TMA producer waits for a tile's rows to have arrived before it loads
// them (device/fused_dispatch.cuh).  That variant gives up one operand stage for the copy ring.
// Every mbarrier wait is bounded; on expiry the CTA records an error, drains and frees TMEM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "device/fused_dispatch.cuh"
#include "device/tcgen05.cuh"
#include "host/ctx.h"
#include "host/errors.h"

namespace mep {
void* driver_tensor_map_encode();

constexpr int BM = 128, BN = 256, BK = 64, GEMM_STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_TILE_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int GEMM_THREADS = 192;
// SGD kernels: eight epilogue warps, two per quarter of the accumulator's lanes, each with one
// half of the tile's columns (the read-modify-write stream of a warp is a chain of latencies:
// accumulator load, weight block landed, update, store read; twice the warps run twice the chains)
constexpr int GEMM_THREADS_SGD = 320;
constexpr int GEMM_THREADS_DISP = 224;      // + the copy warp of the fused dispatch
constexpr int MAX_GROUPS = 1024;
// CTA-pair variant: each CTA stages A (16 KB) and half of B (16 KB) per k-block, six stages.
constexpr int GEMM_STAGES2 = 6;
constexpr int STAGE_BYTES2 = A_TILE_BYTES + B_TILE_BYTES / 2;

enum { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_F32 = 2, EPI_PUSH = 3 };

struct GemmKParams {
  CUtensorMap a[2];
  CUtensorMap b[2][2];
  CUtensorMap c[2];        // weight-grad output (fp32), per allocation
  CUtensorMap b2[2][2];    // K-major B with a 128-row box (CTA-pair variant)
  CUtensorMap o;           // bf16 output of the token-major epilogue (32 x 64 store boxes)
  const int32_t* cu_seqlens;
  int ngroups, split, total_rows, N, K, nseg, rows_per_expert, Mw, accumulate, zero_empty_below;
  // Timing experiments, compiled in only with -DMEP_GEMM_EXPERIMENTS (results are wrong when
  // non-zero), a bit mask: 1 = skip the epilogue's global stores, 2 = skip its TMEM loads, 4 =
  // issue no MMAs (barriers only), 8 = issue no TMA loads (barriers only).  In a normal build
  // gemm_dbg() is a constant false and none of those branches exists.  Bit 16 (plain-store
  // epilogues, results stay correct) is a host-side choice of the epilogue and always available.
  int debug;
  int stages, wb;   // SGD kernels: operand stages and weight blocks per epilogue warp of this launch
  // SGD kernels: 1 = only the tiles whose grads are STORED (experts with replicas, slot groups),
  // 2 = only the tiles that are applied to the weights, 0 = all.  Lets the grads that have to
  // travel be computed first, so that their reduce runs beside the rest of the weight grad.
  int wg_select;
  int g_begin; // groups below this index are skipped (a launch may cover a suffix of the groups)
  int tma_out; // outputs are 16-byte aligned: whole 32-row blocks leave through TMA stores
  // weight grad fused with the SGD step: a local expert's tile is applied straight to its bf16
  // weights, w = bf16(w - lr * acc), instead of being stored as an fp32 grad.  Experts whose
  // sgd_keep flag is set (they have replicas elsewhere, whose grads must be added first) and the
  // slot groups are still written as fp32 grads.
  __nv_bfloat16* sgd_w;
  CUtensorMap wmap;        // the same weights as a [G0 * Mw][N] bf16 tensor, 32-row x 64-column boxes, 128B swizzle
  const int32_t* sgd_keep;
  float sgd_lr;
  void* out[3];
  const float* row_scale;
  long long ldc;
  int32_t* status;
  unsigned long long timeout_ns;
  // EPI_PUSH: results go straight to the token's home rank (see the epilogue)
  const int32_t* src_info;
  void* push_base;
  long long push_rank_stride;
  int push_entries, push_ranks;
  FusedDispatch disp;      // DISP kernels only
  long long* trace;        // phase stamps of the fused launches (see sync.cuh), or null
  // DISP: budget of a wait for rows from other ranks.  It is shorter than timeout_ns, which bounds
  // the waits that only follow from it (the MMA thread on the operand ring, the epilogue on the
  // accumulator), so that a missing row is reported as what it is.
  unsigned long long arrive_timeout_ns;
};

#ifdef MEP_GEMM_EXPERIMENTS
__device__ __forceinline__ bool gemm_dbg(const GemmKParams& p, int bit) { return (p.debug & bit) != 0; }
#else
__device__ __forceinline__ constexpr bool gemm_dbg(const GemmKParams&, int) { return false; }
#endif

struct Tile {
  int g, row0, rows, n0, num_kb, alloc, g_local, m0;
  bool valid;
};

// CLUSTER: the barrier also receives plain arrivals from the pair's other CTA, so the wait
// acquires at cluster scope.  Barriers completed by TMA byte counts or tcgen05.commit do not need it.
template <bool CLUSTER = false>
__device__ __forceinline__ bool gemm_wait(uint64_t* bar, uint32_t parity, volatile int* s_abort,
                                          const GemmKParams& p, int where) {
  auto ready = [&] { return CLUSTER ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
  if (ready()) return true;
  unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (!ready()) {
    if ((++spins & 255u) == 0) {
      if (*s_abort) return false;
      if (globaltimer_ns() - t0 > p.timeout_ns) {
        *s_abort = 1;
        if (p.status != nullptr && atomicCAS(p.status, 0, ST_TIMEOUT_MBAR) == 0) {
          p.status[1] = KID_GEMM;
          p.status[2] = where;
          p.status[3] = (int)blockIdx.x;
        }
        return false;
      }
    }
  }
  return true;
}

// Fused dispatch: wait until all rows of the 128-row block have arrived (counter >= expect).
__device__ __forceinline__ bool arrive_wait(const int32_t* ctr, int expect, int block, volatile int* s_abort,
                                            const GemmKParams& p) {
  int seen = ld_acquire_sys(ctr);
  if (seen >= expect) return true;
  unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while ((seen = ld_acquire_sys(ctr)) < expect) {
    // many CTAs watch the same few counters while the senders' reductions land on them: back off
    __nanosleep(500);
    if ((++spins & 63u) == 0) {
      if (*s_abort) return false;
      if (globaltimer_ns() - t0 > p.arrive_timeout_ns) {
        *s_abort = 1;
        if (p.status != nullptr && atomicCAS(p.status, 0, ST_TIMEOUT_ARRIVAL) == 0) {
          p.status[1] = KID_GEMM;
          p.status[2] = 6;
          p.status[3] = (int)blockIdx.x;
          p.status[4] = block;
          p.status[5] = seen;
          p.status[6] = expect;
        }
        return false;
      }
    }
  }
  return true;
}

// TWO: the tile list counts PAIRS of 128-row tiles (256 rows of one group); CTA `crank` of the
// pair takes the rows [256*mi + 128*crank, +128) and may end up with none in a group's last pair.
template <bool WGRAD, int EPI, bool TWO = false>
__device__ __forceinline__ Tile get_tile(const GemmKParams& p, int id, const int* s_end,
                                         const int* s_prefix, int n_tiles_n, int crank = 0) {
  Tile t;
  t.valid = true;
  if constexpr (WGRAD) {
    constexpr int TMW = TWO ? 2 * BM : BM;       // a pair owns 256 rows of the weight matrix
    const int mt = p.Mw / TMW;
    const int tpg = mt * n_tiles_n;
    t.g = id / tpg;
    int local = id - t.g * tpg;
    int ni = local / mt, mi = local - ni * mt;
    int start = t.g == 0 ? 0 : s_end[t.g - 1];
    t.row0 = start;
    t.rows = s_end[t.g] - start;
    t.m0 = mi * TMW + crank * BM;
    t.n0 = ni * BN;
    t.num_kb = (t.rows + BK - 1) / BK;
    if (t.rows <= 0 && t.g >= p.zero_empty_below) t.valid = false;
    if (t.rows <= 0 && p.sgd_w != nullptr && t.g < p.split &&
        (p.sgd_keep == nullptr || p.sgd_keep[t.g] == 0)) t.valid = false;   // zero grad: nothing to apply
    if (t.g < p.g_begin) t.valid = false;
  } else {
    // largest g with prefix[g] * n_tiles_n <= id
    int lo = 0, hi = p.ngroups - 1;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if ((long long)s_prefix[mid] * n_tiles_n <= id) lo = mid; else hi = mid - 1;
    }
    t.g = lo;
    int start = t.g == 0 ? 0 : s_end[t.g - 1];
    int len = s_end[t.g] - start;
    constexpr int TM = TWO ? 2 * BM : BM;
    int mt = max(1, (len + TM - 1) / TM);
    int local = id - s_prefix[t.g] * n_tiles_n;
    int ni = local / mt, mi = local - ni * mt;
    t.row0 = start + mi * TM + crank * BM;
    t.rows = max(0, min(BM, s_end[t.g] - t.row0));
    t.m0 = 0;
    t.n0 = ni * (EPI == EPI_SWIGLU ? BN / 2 : BN);
    t.num_kb = p.nseg * ((p.K + BK - 1) / BK);
  }
  t.alloc = t.g >= p.split ? 1 : 0;
  t.g_local = t.alloc ? t.g - p.split : t.g;
  if constexpr (WGRAD) {
    if (p.wg_select != 0 && p.sgd_w != nullptr) {
      const bool applied = t.alloc == 0 && (p.sgd_keep == nullptr || p.sgd_keep[t.g_local] == 0);
      if ((p.wg_select == 2) != applied) t.valid = false;
    }
  }
  return t;
}

// Operand stages of the kernels whose geometry is fixed at compile time; the fused dispatch gives
// one up for its copy ring.
template <bool TWO, bool DISP = false> __host__ __device__ constexpr int gemm_stages() {
  return (TWO ? GEMM_STAGES2 : GEMM_STAGES) - (DISP ? 1 : 0);
}
// The SGD kernels (weight grad with the optimizer step in the epilogue) take their geometry at
// launch instead (GemmKParams::stages / wb, sgd_geometry() below): how the shared memory is best
// split between operand stages and weight blocks depends on the group length.
constexpr int SGD_RING_MAX = 8;      // 4 KB weight blocks per epilogue warp, at most
// Fused dispatch: stages of the copy ring (the pair kernel with the staged bf16 epilogue has less
// shared memory to spare).
template <bool TWO, int EPI> __host__ __device__ constexpr int fd_stages() { return (TWO && EPI == EPI_BF16) ? 5 : 8; }
template <bool TWO, bool DISP = false, int EPI = EPI_BF16> __host__ __device__ constexpr int gemm_smem() {   // dynamic shared memory
  return gemm_stages<TWO, DISP>() * (TWO ? STAGE_BYTES2 : STAGE_BYTES) + 1024 +
         (DISP ? fd_stages<TWO, EPI>() * FD_PART_CAP : 0);
}

template <bool WGRAD, bool A_MN, bool B_MN, int EPI, bool TWO = false, bool SGD = false, bool DISP = false>
__global__ void __launch_bounds__(SGD ? GEMM_THREADS_SGD : (DISP ? GEMM_THREADS_DISP : GEMM_THREADS), 1)
ep_grouped_gemm_kernel(const __grid_constant__ GemmKParams p) {
  static_assert(!SGD || (WGRAD && EPI == EPI_F32), "the fused SGD step belongs to the weight grad");
  static_assert(!DISP || (!WGRAD && !SGD), "the fused dispatch feeds a token-major GEMM");
  // operand stages: a constant, except in the SGD kernels (upper bound; p.stages are used)
  constexpr int GEMM_STAGES = SGD ? (TWO ? GEMM_STAGES2 : mep::GEMM_STAGES) : gemm_stages<TWO, DISP>();
  const int nst = SGD ? p.stages : GEMM_STAGES;
  constexpr int FD_NST = fd_stages<TWO, EPI>();
  constexpr int STAGE_BYTES = TWO ? STAGE_BYTES2 : mep::STAGE_BYTES;
  constexpr int WB_MAX = SGD ? SGD_RING_MAX : 1;
  const int WB = SGD ? p.wb : 1;
  const int crank = TWO ? (int)cluster_cta_rank() : 0;        // 0 = leader of the pair
  const int work_id0 = TWO ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int work_stride = TWO ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t full[GEMM_STAGES];
  __shared__ __align__(8) uint64_t empty[GEMM_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_groups_ready;   // DISP: written by the arrival watchers, read by the producer
  __shared__ int s_end[MAX_GROUPS];
  __shared__ int s_prefix[WGRAD ? 1 : MAX_GROUPS + 1];
  // per-warp staging of the fp32 epilogues: 32 x 33 floats token-major, a 4 KB swizzled block for
  // the weight grad
  __shared__ __align__(1024) float s_epi[(EPI == EPI_F32) ? 4 * 32 * 33 : 1];
  // fused SGD: per epilogue warp a ring of WB 32 x 32 bf16 weight blocks (in dynamic shared
  // memory, behind the operand stages) and their "landed" barriers
  __shared__ __align__(8) uint64_t wbar[SGD ? 8 : 4][WB_MAX];
  __shared__ __align__(128) uint8_t s_push[(EPI == EPI_PUSH) ? 4 * 4096 : 16];
  // staging of the bf16 epilogue: per warp one 32 x 64 block (128-byte rows, 128B swizzle)
  __shared__ __align__(1024) uint8_t s_out[(!WGRAD && EPI == EPI_BF16) ? 4 * 4096 : 16];
  // fused dispatch: "landed" barriers of the copy ring
  __shared__ __align__(8) uint64_t fd_full[DISP ? FD_NST : 1];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  volatile int* abortp = &s_abort;

  if (tid == 0) {
    // CTA pairs: both CTAs' loads are credited to the LEADER's full barrier, which only the
    // leader's producer arrives on (expecting the bytes of both CTAs); no per-stage remote arrive
    for (int s = 0; s < GEMM_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], (TWO ? 8 : 4) * (SGD ? 2 : 1)); }
    for (int a = 0; a < (SGD ? 8 : 4) * WB_MAX; ++a) mbar_init(&wbar[a / WB_MAX][a % WB_MAX], 1);
    if constexpr (DISP) for (int a = 0; a < FD_NST; ++a) mbar_init(&fd_full[a], 1);
    mbar_fence_init();
    s_abort = 0;
    s_groups_ready = 0;
  }
  // group table
  for (int g = tid; g < p.ngroups; g += (int)blockDim.x)
    s_end[g] = p.cu_seqlens != nullptr ? p.cu_seqlens[g] : p.total_rows;
  __syncthreads();
  if (warp == 0) {
    // exclusive prefix of M tiles per group (token-major); cheap serial-by-chunks scan
    int run = 0;
    for (int g0 = 0; g0 < p.ngroups; g0 += 32) {
      int g = g0 + lane;
      int len = 0;
      if (g < p.ngroups) len = s_end[g] - (g == 0 ? 0 : s_end[g - 1]);
      constexpr int TM = TWO ? 2 * BM : BM;
      int mt = (len > 0 && g >= p.g_begin) ? (len + TM - 1) / TM : 0;
      int incl = mt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (g < p.ngroups) s_prefix[g] = run + incl - mt;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_prefix[p.ngroups] = run;
  }
  if (warp == 1) {
    if constexpr (TWO) { tmem_alloc2(&s_tmem, 512); tmem_relinquish2(); }
    else { tmem_alloc(&s_tmem, 512); tmem_relinquish(); }
  }
  tc_fence_before();
  if constexpr (TWO) cluster_sync_all();     // the peer's barriers exist before anyone arrives on them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  const int bn_eff = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  const int n_tiles_n = (p.N + bn_eff - 1) / bn_eff;
  long long total_tiles;
  if constexpr (WGRAD) total_tiles = (long long)p.ngroups * (p.Mw / (TWO ? 2 * BM : BM)) * n_tiles_n;
  else total_tiles = (long long)s_prefix[p.ngroups] * n_tiles_n;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      tma_prefetch_desc(&p.a[0]);
      tma_prefetch_desc(&p.b[0][0]);
      int it = 0;
      bool ok = true;
      int groups_ready = 0;      // DISP: groups [0, groups_ready) are known to have arrived
      if constexpr (DISP) phase_stamp(p.trace, 2, (int)blockIdx.x, 0);       // producer starts
      bool stamped_first = false;
      for (long long id = work_id0; id < total_tiles && ok; id += work_stride) {
        Tile t = get_tile<WGRAD, EPI, TWO>(p, (int)id, s_end, s_prefix, n_tiles_n, crank);
        if (!t.valid) continue;
        const int kb_per_seg = WGRAD ? t.num_kb : (p.K + BK - 1) / BK;
        if constexpr (DISP) {
          // The rows of this tile come from other ranks' copy warps.  The other lanes of this warp
          // watch the arrival counters group by group (below) and publish how many groups are
          // complete; waiting for the tile's whole GROUP rather than for its own 128 rows makes
          // every CTA enter a group at about the same time, as CTAs that start together do: the
          // tiles in flight then share one group's rows and weights in L2 instead of two groups'.
          if (p.disp.arrive != nullptr && t.rows > 0 && t.g >= groups_ready) {
#ifdef MEP_GEMM_EXPERIMENTS
            const unsigned long long t_begin = globaltimer_ns();
#endif
            unsigned long long t0 = 0ull;
            unsigned spins = 0;
            while ((groups_ready = *(volatile int*)&s_groups_ready) <= t.g) {
              if ((++spins & 63u) == 0) {
                if (t0 == 0ull) t0 = globaltimer_ns();
                if (*abortp || globaltimer_ns() - t0 > p.timeout_ns) { ok = false; break; }
              }
            }
            if (!ok) break;
            __threadfence_block();
            fence_proxy_async();   // the rows were written through the async proxy (or by plain stores)
            if (!stamped_first) { phase_stamp(p.trace, 2, (int)blockIdx.x, 1); stamped_first = true; }   // first group arrived
#ifdef MEP_GEMM_EXPERIMENTS
            if (p.status != nullptr)                   // experiments: total arrival wait of all CTAs, in microseconds
              atomicAdd(p.status + 6, (int)((globaltimer_ns() - t_begin) / 1000ull));
#endif
          }
        }
        for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
          const int s = it % nst;
          if (it >= nst &&
              !gemm_wait(&empty[s], ((uint32_t)(it / nst) & 1u) ^ 1u, abortp, p, 1)) {
            ok = false;
            break;
          }
          uint8_t* sa = tiles + (size_t)s * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          uint32_t lead_bar = 0;
          if constexpr (TWO) lead_bar = mapa_u32(&full[s], 0);
          if (gemm_dbg(p, 8)) {
            if (crank == 0) mbar_arrive(&full[s]);
            continue;
          }
          // the peer's bytes may land before this arrival: the pending count keeps the phase open
          if (crank == 0) mbar_expect_tx(&full[s], TWO ? 2 * STAGE_BYTES : STAGE_BYTES);
          const int seg = kb / kb_per_seg;
          const int k0 = (kb - seg * kb_per_seg) * BK;
          if constexpr (WGRAD && TWO) {
            // this CTA's 128 columns of A (t.m0 is already its half) and its half of the B tile
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d_pair(sa + j * 8192, &p.a[0], t.m0 + 64 * j, t.row0 + k0, lead_bar);
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d_pair(sb + j * 8192, &p.b[0][0], t.n0 + 128 * crank + 64 * j, t.row0 + k0, lead_bar);
          } else if constexpr (WGRAD) {
            // A: [token rows][Mw cols], two 64-column blocks; B: [token rows][N cols], four
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &p.a[0], t.m0 + 64 * j, t.row0 + k0, &full[s]);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &p.b[0][0], t.n0 + 64 * j, t.row0 + k0, &full[s]);
          } else {
            if constexpr (TWO) tma_load_2d_pair(sa, &p.a[seg], k0, t.row0, lead_bar);
            else tma_load_2d(sa, &p.a[seg], k0, t.row0, &full[s]);
            const int erow = t.g_local * p.rows_per_expert;
            if constexpr (TWO) {
              // this CTA's half of the B tile: N columns [128*crank, +128) of the pair's tile
              if constexpr (B_MN) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  if constexpr (EPI == EPI_SWIGLU)   // leader: 128 gate columns, peer: 128 up columns
                    tma_load_2d_pair(sb + j * 8192, &p.b[crank][t.alloc], t.n0 + 64 * j, erow + k0, lead_bar);
                  else
                    tma_load_2d_pair(sb + j * 8192, &p.b[seg][t.alloc], t.n0 + 128 * crank + 64 * j, erow + k0, lead_bar);
                }
              } else {
                tma_load_2d_pair(sb, &p.b2[seg][t.alloc], k0, erow + t.n0 + 128 * crank, lead_bar);
              }
            } else if constexpr (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) {
                if constexpr (EPI == EPI_SWIGLU) {
                  const int part = j / (BN / 128);
                  tma_load_2d(sb + j * 8192, &p.b[part][t.alloc],
                              t.n0 + 64 * (j % (BN / 128)), erow + k0, &full[s]);
                } else {
                  tma_load_2d(sb + j * 8192, &p.b[seg][t.alloc], t.n0 + 64 * j, erow + k0, &full[s]);
                }
              }
            } else {
              tma_load_2d(sb, &p.b[seg][t.alloc], k0, erow + t.n0, &full[s]);
            }
          }
        }
      }
      if constexpr (DISP) phase_stamp(p.trace, 2, (int)blockIdx.x, 2);       // last operand load issued
    } else if (DISP && p.disp.arrive != nullptr) {
      // ---- arrival watchers (lanes 1..31): group after group, wait until every 128-row block of
      // the group has all its rows, then publish the number of complete groups to lane 0 --------
      if constexpr (DISP) {
        for (int g = 0; g < p.ngroups; ++g) {
          const int b0 = (g == 0 ? 0 : s_end[g - 1]) >> 7, b1 = s_end[g] >> 7;
          bool okw = true;
          for (int b = b0 + lane - 1; b < b1 && okw; b += 31)
            okw = arrive_wait(p.disp.arrive + b, p.disp.expect, b, abortp, p);
          if (!__all_sync(0xfffffffeu, okw)) break;
          if (lane == 1) {
            __threadfence_block();
            *(volatile int*)&s_groups_ready = g + 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0 && TWO && crank != 0) {
      // peer CTA of a pair: the leader issues the MMAs for both
    } else if (lane == 0) {
      constexpr uint32_t idesc = make_instr_desc_bf16(TWO ? 2 * BM : BM, BN, A_MN, B_MN);
      int it = 0, tile_n = 0;
      bool ok = true;
      for (long long id = work_id0; id < total_tiles && ok; id += work_stride) {
        Tile t = get_tile<WGRAD, EPI, TWO>(p, (int)id, s_end, s_prefix, n_tiles_n, crank);
        if (!t.valid) continue;
        const int acc = tile_n & 1;
        if (tile_n >= 2 &&
            !gemm_wait<TWO>(&acc_empty[acc], ((uint32_t)(tile_n >> 1) & 1u) ^ 1u, abortp, p, 2)) break;
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)acc * BN;
        for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
          const int s = it % nst;
          if (!gemm_wait(&full[s], (uint32_t)(it / nst) & 1u, abortp, p, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            if (gemm_dbg(p, 4)) break;
            const uint64_t da = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sb + kk * 32, 16, 1024);
            if constexpr (TWO) umma_bf16_2cta(tacc, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            else umma_bf16(tacc, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          // stage reusable (in both CTAs of a pair) once these MMAs have read it
          if constexpr (TWO) umma_commit_2cta(&empty[s], 3);
          else umma_commit(&empty[s]);
        }
        if (!ok) break;
        if constexpr (TWO) umma_commit_2cta(&acc_full[acc], 3);   // accumulator complete, both halves
        else umma_commit(&acc_full[acc]);
        ++tile_n;
      }
    }
  } else if (DISP && warp >= 6) {
    // ================= fused dispatch: this CTA's share of the all-to-all =================
    if constexpr (DISP) {
      if (p.disp.x != nullptr) {
        uint8_t* ring = tiles + (size_t)nst * STAGE_BYTES;
#ifdef MEP_GEMM_EXPERIMENTS
        const unsigned long long t_begin = globaltimer_ns();
#endif
        if (lane == 0) phase_stamp(p.trace, 3, (int)blockIdx.x, 0);          // copy warp starts
        fused_dispatch_copy_warp<FD_NST>(
            p.disp, ring, fd_full, (int)blockIdx.x, (int)gridDim.x,
            [&](uint64_t* bar, uint32_t parity) { return gemm_wait(bar, parity, abortp, p, 7); });
        if (lane == 0) phase_stamp(p.trace, 3, (int)blockIdx.x, 1);          // all rows sent and announced
#ifdef MEP_GEMM_EXPERIMENTS
        if (lane == 0 && p.status != nullptr)      // experiments: longest copy-warp run, in microseconds
          atomicMax(p.status + 7, (int)((globaltimer_ns() - t_begin) / 1000ull));
#endif
      }
    }
  } else {
    // ================= epilogue (4 warps, one TMEM lane quarter each) =================
    const int q = warp & 3;
    const int r_in_tile = q * 32 + lane;
    // SGD: warps 2..5 take the tile's first 128 columns, warps 6..9 the other 128
    const int half = SGD ? (warp - 2) >> 2 : 0;
    const int ew = q + 4 * half;
    constexpr int CB = SGD ? BN / 64 / 2 : BN / 64;     // 64-column weight blocks per warp and tile
    const int cofs = half * CB * 64;
    int tile_n = 0;
    // ---- fused SGD: weight blocks stream through this warp's ring, ahead of the tiles ----------
    // Block k of the stream (the 32-row x 64-column blocks of this warp's rows, tile after tile,
    // fused tiles only) lives in buffer k % WB.  The load cursor runs up to WB blocks ahead of the
    // block being updated, across tile boundaries.  Blocks are as wide as the 128B swizzle
    // allows: the TMA engine moves about one box row per 5 cycles per SM whatever its length
    // (measured), so 64-byte rows cap this epilogue at half the HBM rate.
    constexpr int WBLK = 4096, WCOLS = 64;
    uint8_t* wring = tiles + (size_t)nst * STAGE_BYTES + ew * (WB * WBLK);
    int wseq = 0, lseq = 0;                // blocks consumed / loads issued (a few thousand per launch)
    long long lid = work_id0;              // cursor: tile id, block in tile, cached coordinates
    int lc = 0, l_y0 = 0, l_n0 = 0;
    bool l_have = false;
    auto sgd_tile = [&](const Tile& u) {
      return u.valid && u.alloc == 0 && (p.sgd_keep == nullptr || p.sgd_keep[u.g_local] == 0);
    };
    auto cursor_settle = [&]() {           // move to the next existing block at or after (lid, lc)
      while (lid < total_tiles) {
        if (!l_have) {
          const Tile u = get_tile<WGRAD, EPI, TWO>(p, (int)lid, s_end, s_prefix, n_tiles_n, crank);
          if (sgd_tile(u)) { l_have = true; l_y0 = u.g_local * p.Mw + u.m0 + q * 32; l_n0 = u.n0; lc = 0; }
        }
        if (l_have && lc < CB && l_n0 + cofs + lc * WCOLS < p.N) return;
        l_have = false;
        lid += work_stride;
      }
    };
    auto issue_loads = [&]() {             // lane 0 issues; every lane tracks the cursor
      while (lid < total_tiles && lseq < wseq + WB) {
        if (lane == 0) {
          uint64_t* bar = &wbar[ew][lseq % WB];
          mbar_expect_tx(bar, WBLK);
          tma_load_2d(wring + (lseq % WB) * WBLK, &p.wmap, l_n0 + cofs + lc * WCOLS, l_y0, bar);
        }
        ++lseq;
        ++lc;
        cursor_settle();
      }
    };
    if constexpr (SGD) {
      cursor_settle();
      issue_loads();
    }
    for (long long id = work_id0; id < total_tiles; id += work_stride) {
      Tile t = get_tile<WGRAD, EPI, TWO>(p, (int)id, s_end, s_prefix, n_tiles_n, crank);
      if (!t.valid) continue;
      const int acc = tile_n & 1;
      bool sgd_fuse = false;
      if constexpr (SGD) sgd_fuse = sgd_tile(t);
      if (!gemm_wait(&acc_full[acc], (uint32_t)(tile_n >> 1) & 1u, abortp, p, 4)) break;
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * BN + ((uint32_t)(q * 32) << 16);
      const bool have_acc = t.num_kb > 0;
      if constexpr (EPI == EPI_SWIGLU) {
        const bool row_ok = r_in_tile < t.rows;
        const long long row = (long long)t.row0 + r_in_tile;
        // (read past L1: with the fused dispatch the scale was written by another rank moments ago)
        const float rs = (row_ok && p.row_scale != nullptr) ? __ldcg(p.row_scale + row) : 1.f;
        __nv_bfloat16* og = (__nv_bfloat16*)p.out[0];
        __nv_bfloat16* ou = (__nv_bfloat16*)p.out[1];
        __nv_bfloat16* oa = (__nv_bfloat16*)p.out[2];
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t rg[32], ru[32];
          if (!gemm_dbg(p, 2)) {
            tmem_ld_32x32(tacc + c * 32, rg);
            tmem_ld_32x32(tacc + 128 + c * 32, ru);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) rg[i] = ru[i] = 0u;
          }
          const int col = t.n0 + c * 32;
          if (row_ok && col < p.N) {
            uint32_t pg[16], pu[16], pa[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float g0 = __uint_as_float(rg[2 * i]), g1 = __uint_as_float(rg[2 * i + 1]);
              float u0 = __uint_as_float(ru[2 * i]), u1 = __uint_as_float(ru[2 * i + 1]);
              __nv_bfloat162 hg = __floats2bfloat162_rn(g0, g1);
              __nv_bfloat162 hu = __floats2bfloat162_rn(u0, u1);
              // the saved gate/up are bf16; the activation is computed from the rounded values
              // so that backward recomputes exactly what forward used
              float2 fg = __bfloat1622float2(hg), fu = __bfloat1622float2(hu);
              float a0 = fg.x / (1.f + __expf(-fg.x)) * fu.x * rs;
              float a1 = fg.y / (1.f + __expf(-fg.y)) * fu.y * rs;
              __nv_bfloat162 ha = __floats2bfloat162_rn(a0, a1);
              pg[i] = *reinterpret_cast<uint32_t*>(&hg);
              pu[i] = *reinterpret_cast<uint32_t*>(&hu);
              pa[i] = *reinterpret_cast<uint32_t*>(&ha);
            }
            const long long off = row * p.ldc + col;
            if (gemm_dbg(p, 1)) {
            } else if (col + 32 <= p.N) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                if (og) reinterpret_cast<uint4*>(og + off)[v] = make_uint4(pg[4 * v], pg[4 * v + 1], pg[4 * v + 2], pg[4 * v + 3]);
                if (ou) reinterpret_cast<uint4*>(ou + off)[v] = make_uint4(pu[4 * v], pu[4 * v + 1], pu[4 * v + 2], pu[4 * v + 3]);
                reinterpret_cast<uint4*>(oa + off)[v] = make_uint4(pa[4 * v], pa[4 * v + 1], pa[4 * v + 2], pa[4 * v + 3]);
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) {
                const __nv_bfloat16* sg = reinterpret_cast<const __nv_bfloat16*>(pg);
                const __nv_bfloat16* su = reinterpret_cast<const __nv_bfloat16*>(pu);
                const __nv_bfloat16* sa2 = reinterpret_cast<const __nv_bfloat16*>(pa);
                if (og) og[off + i] = sg[i];
                if (ou) ou[off + i] = su[i];
                oa[off + i] = sa2[i];
              }
            }
          }
        }
      } else if constexpr (EPI == EPI_PUSH) {
        // thread = output row.  The row's owner entry (source rank, token*K+k) comes from the
        // per-slot source record; padding rows have none and are dropped.  64 columns at a time
        // are staged in a swizzled per-warp pad and leave as full 128-byte lines: every store
        // instruction covers 4 rows x 128 B, 8 lanes per row, addressed at the home rank.
        uint8_t* pad = s_push + q * 4096;
        const bool row_ok = r_in_tile < t.rows;
        const long long row = (long long)t.row0 + r_in_tile;
        const int si = row_ok ? p.src_info[row] : -1;
        unsigned long long dptr = 0ull;
        if (si >= 0) {
          const int sr = si / p.push_entries, ent = si - sr * p.push_entries;
          if (sr < p.push_ranks)
            dptr = (unsigned long long)((__nv_bfloat16*)p.push_base + (long long)sr * p.push_rank_stride +
                                        (long long)ent * p.ldc + t.n0);
        }
#pragma unroll 1
        for (int c2 = 0; c2 < BN / 64; ++c2) {
          uint32_t ra[32], rb[32];
          tmem_ld_32x32(tacc + c2 * 64, ra);
          tmem_ld_32x32(tacc + c2 * 64 + 32, rb);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t* src = j < 4 ? ra + 8 * j : rb + 8 * (j - 4);
            uint32_t pk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(src[2 * i]), __uint_as_float(src[2 * i + 1]));
              pk[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(pad + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
          __syncwarp();
          const int j = lane & 7;
          const bool col_ok = t.n0 + c2 * 64 + j * 8 < p.N;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int rr = g * 4 + (lane >> 3);
            const unsigned long long pr = __shfl_sync(0xffffffffu, dptr, rr);
            const uint4 v = *reinterpret_cast<const uint4*>(pad + rr * 128 + ((j ^ (rr & 7)) << 4));
            if (pr != 0ull && col_ok)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(pr) + c2 * 64 + j * 8) = v;
          }
          __syncwarp();
        }
      } else {
        bool row_ok;
        long long off_row;
        int col_base;
        if constexpr (WGRAD) {
          row_ok = t.m0 + r_in_tile < p.Mw;
          off_row = ((long long)t.g_local * p.Mw + t.m0 + r_in_tile) * p.ldc;
          col_base = t.n0;
        } else {
          row_ok = r_in_tile < t.rows;
          off_row = ((long long)t.row0 + r_in_tile) * p.ldc;
          col_base = t.n0;
        }
        void* outp = WGRAD ? p.out[t.alloc] : p.out[0];
        if constexpr (EPI == EPI_F32 && WGRAD) {
          // fp32 weight-grad tiles are 128 KB each and the main loop is short (one group's
          // tokens), so the epilogue must move ~30 GB/s per SM.  Four warps of plain stores
          // cannot (measured: ~14 B/clk/SM), so each warp stages 32x32 blocks in shared memory
          // (128-byte swizzle, conflict-free 16-byte stores) and hands them to the TMA engine:
          // a tiled store, or a tiled reduce-add when accumulating into existing grads.
          uint8_t* pad = reinterpret_cast<uint8_t*>(s_epi) + q * 4096;
          const int y0 = t.g_local * p.Mw + t.m0 + q * 32;
          const CUtensorMap* cmap = &p.c[t.alloc];
          if (SGD && sgd_fuse) {
            // Weights travel by TMA both ways: a block is 32 rows x 64 bf16 (128-byte rows, 128B
            // swizzle); lane i owns row i of the block, exactly the accumulator row it reads from
            // tensor memory, so no transposition is needed.  The block is updated in place,
            // stored back, and its buffer handed to the load cursor.
            const float nlr = -p.sgd_lr;
            bool wok = true;
#pragma unroll 1
            for (int c = 0; c < CB; ++c) {
              if (col_base + cofs + c * WCOLS >= p.N) break;
              const int b = wseq % WB;
              uint8_t* wbuf = wring + b * WBLK;
              uint32_t ra[32], rb[32];
              if (!gemm_dbg(p, 2)) {
                tmem_ld_32x32(tacc + cofs + c * WCOLS, ra);
                tmem_ld_32x32(tacc + cofs + c * WCOLS + 32, rb);
              }
              if (!gemm_wait(&wbar[ew][b], (uint32_t)(wseq / WB) & 1u, abortp, p, 5)) {
                if (!gemm_dbg(p, 2)) tmem_ld_wait();
                wok = false;
                break;
              }
              if (!gemm_dbg(p, 2)) {
                tmem_ld_wait();
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) ra[i] = rb[i] = 0u;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t* g = j < 4 ? ra + 8 * j : rb + 8 * (j - 4);
                uint4* slot = reinterpret_cast<uint4*>(wbuf + lane * 128 + ((j ^ (lane & 7)) << 4));
                uint4 w4 = *slot;
                __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(&w4);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 x = __bfloat1622float2(w2[i]);
                  w2[i] = __floats2bfloat162_rn(__fmaf_rn(nlr, __uint_as_float(g[2 * i]), x.x),
                                                __fmaf_rn(nlr, __uint_as_float(g[2 * i + 1]), x.y));
                }
                *slot = w4;
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (!gemm_dbg(p, 1)) {
                  tma_store_2d(&p.wmap, col_base + cofs + c * WCOLS, y0, wbuf);
                  bulk_commit();
                }
                bulk_wait_read<0>();                // the store has read the buffer: it may be refilled
              }
              ++wseq;
              issue_loads();
            }
            if (!wok) break;
          } else if (half == 0)      // (SGD kernels: a tile that is not applied is stored by warps 2..5 alone)
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            if (have_acc && !gemm_dbg(p, 2)) {
              tmem_ld_32x32(tacc + c * 32, r);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
            if (lane == 0) bulk_wait_read<0>();     // the previous block has left the pad
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(pad + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            const int x0 = col_base + c * 32;
            if (lane == 0 && x0 < p.N && !gemm_dbg(p, 1)) {
              if (p.accumulate) tma_reduce_add_2d(cmap, x0, y0, pad);
              else tma_store_2d(cmap, x0, y0, pad);
              bulk_commit();
            }
          }
        } else if constexpr (EPI == EPI_F32) {
          // token-major fp32 output (router logits): rows of a tile may belong to the next
          // group, so stores stay row-masked; each warp transposes through a padded pad so
          // that every store instruction writes one full 128-byte line.
          float* pad = s_epi + q * (32 * 33);
          const long long row_stride = p.ldc;
          const long long off_warp = WGRAD ? ((long long)t.g_local * p.Mw + t.m0 + q * 32) * p.ldc
                                           : ((long long)t.row0 + q * 32) * p.ldc;
          const int rows_ok = WGRAD ? min(32, p.Mw - (t.m0 + q * 32)) : min(32, t.rows - q * 32);
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            if (have_acc && !gemm_dbg(p, 2)) {
              tmem_ld_32x32(tacc + c * 32, r);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
            const int col = col_base + c * 32 + lane;
#pragma unroll
            for (int i = 0; i < 32; ++i) pad[lane * 33 + i] = __uint_as_float(r[i]);
            __syncwarp();
            if (col < p.N && !gemm_dbg(p, 1)) {
              float* o = (float*)outp + off_warp + col;
#pragma unroll 8
              for (int rr = 0; rr < 32; ++rr) {
                if (rr < rows_ok) {
                  float v = pad[rr * 33 + lane];
                  if (p.accumulate) v += o[rr * row_stride];
                  o[rr * row_stride] = v;
                }
              }
            }
            __syncwarp();
          }
        } else if (EPI == EPI_BF16 && !WGRAD && p.tma_out != 0 && q * 32 + 32 <= t.rows) {
          // all 32 rows of this warp belong to the group: stage 32 x 64 blocks (128-byte rows,
          // 128B swizzle, conflict-free 16-byte stores) and let the TMA engine write full lines
          uint8_t* pad = s_out + q * 4096;
          const int y0 = t.row0 + q * 32;
#pragma unroll 1
          for (int c2 = 0; c2 < BN / 64; ++c2) {
            const int col = col_base + c2 * 64;
            if (col >= p.N) break;
            uint32_t ra[32], rb[32];
            if (have_acc && !gemm_dbg(p, 2)) {
              tmem_ld_32x32(tacc + c2 * 64, ra);
              tmem_ld_32x32(tacc + c2 * 64 + 32, rb);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) ra[i] = rb[i] = 0u;
            }
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t* src = j < 4 ? ra + 8 * j : rb + 8 * (j - 4);
              uint32_t pk[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(src[2 * i]), __uint_as_float(src[2 * i + 1]));
                pk[i] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(pad + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && !gemm_dbg(p, 1)) {
              tma_store_2d(&p.o, col, y0, pad);
              bulk_commit();
            }
          }
        } else
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          if (have_acc && !gemm_dbg(p, 2)) {
            tmem_ld_32x32(tacc + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          const int col = col_base + c * 32;
          if (!row_ok || col >= p.N || gemm_dbg(p, 1)) continue;
          if constexpr (EPI == EPI_F32) {
            // unreachable: the fp32 epilogue is the transposed loop below
          } else {
            __nv_bfloat16* o = (__nv_bfloat16*)outp + off_row + col;
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
              pk[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            if (col + 32 <= p.N) {
#pragma unroll
              for (int v = 0; v < 4; ++v)
                reinterpret_cast<uint4*>(o)[v] = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
            } else {
              const __nv_bfloat16* sp = reinterpret_cast<const __nv_bfloat16*>(pk);
              for (int i = 0; i < 32 && col + i < p.N; ++i) o[i] = sp[i];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (TWO && crank != 0) mbar_arrive_remote(&acc_empty[acc], 0);   // the leader issues the MMAs
        else mbar_arrive(&acc_empty[acc]);
      }
      ++tile_n;
    }
  }
  // ---- teardown: everything joins, in-flight work is given time to land on an abort ----------
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  if (warp >= 2 && lane == 0) bulk_wait<0>();   // epilogue TMA stores have completed
  // Pushed rows: the kernel that consumes them on the home rank runs behind a cross-rank barrier
  // that this rank enters from a LATER launch of the same stream, so the end of this kernel
  // already orders the stores; one fence here (instead of one per tile, which made every epilogue
  // warp wait for an NVLink round trip per tile) keeps that independent of how the next launch arrives.
  if constexpr (EPI == EPI_PUSH) { if (warp >= 2) __threadfence_system(); }
  if constexpr (TWO) cluster_sync_all();        // neither CTA leaves while its peer may still touch it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (TWO) tmem_dealloc2(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

// ---- host side -----------------------------------------------------------------------------------
struct GemmDesc {
  int32_t mode, epi, b_mn, nseg;
  int32_t ngroups, split, total_rows, N, K, rows_per_expert, Mw, accumulate, zero_empty_below, grid;
  int32_t debug, g_begin;
  int64_t a_rows;
  int64_t lda[2];
  const void* a[2];
  const void* b[2][2];
  int64_t b_rows[2];
  int64_t ldb;
  const int32_t* cu_seqlens;
  void* out[3];
  int64_t ldc;
  const float* row_scale;
  int32_t* status;
  int64_t timeout_ns;
  const int32_t* src_info;
  void* push_base;
  int64_t push_rank_stride;
  int32_t push_entries, push_ranks;
  int32_t two_cta, wg_select;
  void* sgd_w;
  const int32_t* sgd_keep;
  float sgd_lr;
  // Fused dispatch (0 = off): 1 = only wait for the rows of each tile to arrive, 2 = also send
  // this rank's rows.  disp_ctx is the Buffer's context; the A operand must be the row buffer
  // `disp_shard` of that Buffer.
  int32_t disp_mode;
  const void* disp_ctx;
  const void* disp_x;
  const float* disp_w;
  const int32_t* disp_dst;
  const int32_t* disp_order;
  const int32_t* disp_zero_fill;
  int32_t disp_fresh, disp_shard;
};

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                             CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                             CUtensorMapFloatOOBfill);

// 2-D fp32 tensor [rows][cols], box 32 x 32 (128-byte rows), 128B swizzle: weight-grad output.
static int make_map_f32(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld) {
  EncodeFn enc = (EncodeFn)driver_tensor_map_encode();
  if (!enc) return fail(-10, "CUDA driver entry cuTensorMapEncodeTiled not available");
  if (((uintptr_t)base & 15) != 0 || (ld * 4) % 16 != 0)
    return fail(-11, "weight-grad output must be 16-byte aligned with a 16-byte multiple row stride");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-12, "cuTensorMapEncodeTiled (fp32) failed with code %d", (int)r);
  return 0;
}

// 2-D bf16 tensor [rows][cols] (row stride ld elements), box [box_rows][box_cols], 128B swizzle.
static int make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld,
                    int box_cols, int box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeFn enc = (EncodeFn)driver_tensor_map_encode();
  if (!enc) return fail(-10, "CUDA driver entry cuTensorMapEncodeTiled not available");
  if (((uintptr_t)base & 15) != 0 || (ld * 2) % 16 != 0)
    return fail(-11, "GEMM operand must be 16-byte aligned with a 16-byte multiple row stride");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-12, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

// Fused dispatch launches: CTAs of different ranks wait for one another's copy warps, so the whole
// grid must be resident at once.  The grid never exceeds what the device holds next to the weight
// ops' CTAs, and a cooperative launch makes the driver guarantee the residency; MOONEP_B200_FD_COOP=0
// launches plainly instead (the waits stay bounded either way).
static bool fused_dispatch_cooperative() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("MOONEP_B200_FD_COOP");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// SGD kernels: dynamic shared memory of a launch (operand stages, alignment slack, four rings of
// 4 KB weight blocks) and the most that the kernel may ask for next to its static part.
static int sgd_smem(const GemmKParams& kp, bool two) {
  return kp.stages * (two ? STAGE_BYTES2 : STAGE_BYTES) + 1024 + 8 * kp.wb * 4096;
}
// How an SGD launch splits its shared memory between operand stages and weight blocks (4 KB, per
// epilogue warp).  Measured on the benchmark's shapes (32 x 1024, 64 x 512, 256 x 128 rows): the
// depth of the weight ring hardly matters once eight warps run the read-modify-write chains (a
// warp needs ~1.4 us per block whatever the depth), so the operand ring gets what is left after
// two (pairs) or three (single CTA, whose stages are 48 KB) blocks per warp.
// MOONEP_B200_SGD_RING="stages,blocks" overrides the choice (tuning).
static void sgd_geometry(bool pair, GemmKParams* kp) {
  if (pair) { kp->stages = 4; kp->wb = 2; }
  else { kp->stages = 2; kp->wb = 3; }
  if (const char* e = getenv("MOONEP_B200_SGD_RING")) {
    int a = 0, b = 0;
    if (sscanf(e, "%d,%d", &a, &b) == 2 && a >= 2 && a <= (pair ? GEMM_STAGES2 : GEMM_STAGES) && b >= 2 &&
        b <= SGD_RING_MAX) {
      kp->stages = a; kp->wb = b;
    }
  }
}
static int sgd_smem_limit(const void* kern) {
  cudaFuncAttributes fa;
  int dev = 0, optin = 0;
  if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) { cudaGetLastError(); return 0; }
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  return optin - (int)fa.sharedSizeBytes;
}

// CTA-pair launch: clusters of two CTAs, one pair per two SMs.
template <bool A_MN, bool B_MN, int EPI, bool WGRAD = false, bool SGD = false, bool DISP = false>
static int launch_gemm2(const GemmKParams& kp, int grid, cudaStream_t stream) {
  auto kern = ep_grouped_gemm_kernel<WGRAD, A_MN, B_MN, EPI, true, SGD, DISP>;
  const int GEMM_SMEM2 = SGD ? sgd_smem(kp, true) : gemm_smem<true, DISP, EPI>();
  static bool configured = false;
  if (!configured) {
    const int most = SGD ? sgd_smem_limit((const void*)kern) : GEMM_SMEM2;
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    configured = true;
  }
  if (SGD && GEMM_SMEM2 > sgd_smem_limit((const void*)kern))
    return fail(-3, "gemm: %d operand stages + %d weight blocks do not fit in shared memory", kp.stages, kp.wb);
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(grid / 2 * 2));
  cfg.blockDim = dim3(SGD ? GEMM_THREADS_SGD : (DISP ? GEMM_THREADS_DISP : GEMM_THREADS));
  cfg.dynamicSmemBytes = GEMM_SMEM2;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  // the fused dispatch makes CTAs of different ranks wait for one another's copy warps: the
  // whole grid must be resident at once, which a cooperative launch guarantees
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (DISP && fused_dispatch_cooperative()) ? 2 : 1;
  // A persistent grid must not exceed what is resident at once: not every SM can be paired
  // into a cluster (GPCs with an odd SM count leave one out), and a second wave of persistent
  // CTAs would double the run time.
  static int max_clusters = -1;
  if (max_clusters < 0) {
    int n = 0;
    cudaLaunchConfig_t probe = cfg;
    probe.gridDim = dim3(2 * 148);
    if (cudaOccupancyMaxActiveClusters(&n, kern, &probe) != cudaSuccess || n < 1) { cudaGetLastError(); n = 1 << 20; }
    max_clusters = n;
  }
  int use = max_clusters;
  {
    // a launch with a CTA limit shares the GPU with a copy kernel that is placed as SM pairs too:
    // leave it its pairs out of what the device can hold, or this persistent grid would need a
    // second wave
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (grid < sms && max_clusters < (1 << 20)) use = max_clusters - (sms - grid + 1) / 2;
    if (use < 1) use = 1;
  }
  if ((int)cfg.gridDim.x / 2 > use) cfg.gridDim = dim3((unsigned)(2 * use));
  MEP_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, kp));
  return 0;
}

template <bool WGRAD, bool A_MN, bool B_MN, int EPI, bool SGD = false, bool DISP = false>
static int launch_gemm(const GemmKParams& kp, int grid, cudaStream_t stream) {
  auto kern = ep_grouped_gemm_kernel<WGRAD, A_MN, B_MN, EPI, false, SGD, DISP>;
  const int GEMM_SMEM = SGD ? sgd_smem(kp, false) : gemm_smem<false, DISP, EPI>();
  static bool configured = false;
  if (!configured) {
    const int most = SGD ? sgd_smem_limit((const void*)kern) : GEMM_SMEM;
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    configured = true;
  }
  if (SGD && GEMM_SMEM > sgd_smem_limit((const void*)kern))
    return fail(-3, "gemm: %d operand stages + %d weight blocks do not fit in shared memory", kp.stages, kp.wb);
  if constexpr (DISP) {
    // CTAs of different ranks wait for one another's copy warps: all of them must be resident
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (grid > sms) grid = sms;
    if (fused_dispatch_cooperative()) {
      GemmKParams kpc = kp;
      MEP_CUDA_OK(launch_coop((const void*)kern, dim3(grid), dim3(GEMM_THREADS_DISP), GEMM_SMEM, stream, kpc));
    } else {
      kern<<<grid, GEMM_THREADS_DISP, GEMM_SMEM, stream>>>(kp);
      MEP_CUDA_OK(cudaGetLastError());
    }
    return 0;
  }
  kern<<<grid, SGD ? GEMM_THREADS_SGD : GEMM_THREADS, GEMM_SMEM, stream>>>(kp);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace mep

using namespace mep;

extern "C" {

int mep_gemm_desc_bytes() { return (int)sizeof(GemmDesc); }

int mep_gemm_launch(const GemmDesc* d, cudaStream_t stream) {
  if (d->ngroups < 1 || d->ngroups > MAX_GROUPS) return fail(-1, "gemm: ngroups=%d out of range", d->ngroups);
  GemmKParams kp;
  std::memset(&kp, 0, sizeof(kp));
  kp.cu_seqlens = d->cu_seqlens; kp.ngroups = d->ngroups; kp.split = d->split;
  kp.total_rows = d->total_rows; kp.N = d->N; kp.K = d->K; kp.nseg = d->nseg;
  kp.rows_per_expert = d->rows_per_expert; kp.Mw = d->Mw; kp.accumulate = d->accumulate;
  kp.zero_empty_below = d->zero_empty_below;
  kp.debug = d->debug; kp.g_begin = d->g_begin;
#ifdef MEP_GEMM_EXPERIMENTS
  if (const char* e = getenv("MOONEP_B200_GEMM_EXPERIMENT")) kp.debug |= atoi(e);   // timing only: results are wrong
#endif
  kp.src_info = d->src_info; kp.push_base = d->push_base; kp.push_rank_stride = d->push_rank_stride;
  kp.push_entries = d->push_entries; kp.push_ranks = d->push_ranks;
  kp.out[0] = d->out[0]; kp.out[1] = d->out[1]; kp.out[2] = d->out[2];
  kp.row_scale = d->row_scale; kp.ldc = d->ldc; kp.status = d->status;
  kp.timeout_ns = (unsigned long long)(d->timeout_ns > 0 ? d->timeout_ns : 2000000000ll);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = d->grid > 0 ? d->grid : sms;
  int rc = 0;
  if (d->mode == 1) {
    // weight grad: A [a_rows][Mw] and B [a_rows][N], both read as MN-major 64x64 boxes
    if (d->Mw % BM != 0) return fail(-2, "wgrad: Mw=%d must be a multiple of %d", d->Mw, BM);
    if ((rc = make_map(&kp.a[0], d->a[0], d->a_rows, d->Mw, d->lda[0], 64, BK))) return rc;
    if ((rc = make_map(&kp.b[0][0], d->b[0][0], d->a_rows, d->N, d->ldb, 64, BK))) return rc;
    kp.a[1] = kp.a[0]; kp.b[0][1] = kp.b[1][0] = kp.b[1][1] = kp.b[0][0];
    if (d->epi != EPI_F32) return fail(-3, "wgrad writes fp32");
    if (d->sgd_w != nullptr) {
      if (d->accumulate) return fail(-13, "wgrad: the fused SGD step cannot accumulate into existing grads");
      if (d->N % 8 != 0 || ((uintptr_t)d->sgd_w & 15) != 0)
        return fail(-14, "wgrad: the fused SGD step needs N %% 8 == 0 and 16-byte aligned weights");
      kp.sgd_w = (__nv_bfloat16*)d->sgd_w; kp.sgd_keep = d->sgd_keep; kp.sgd_lr = d->sgd_lr;
      const int n_w = d->split < d->ngroups ? d->split : d->ngroups;
      if ((rc = make_map(&kp.wmap, d->sgd_w, (int64_t)n_w * d->Mw, d->N, d->ldc, 64, 32))) return rc;
    }
    const int n_local = d->split < d->ngroups ? d->split : d->ngroups;
    if ((rc = make_map_f32(&kp.c[0], d->out[0], (int64_t)n_local * d->Mw, d->N, d->ldc))) return rc;
    kp.c[1] = kp.c[0];
    if (d->ngroups > d->split) {
      if (d->out[1] == nullptr) return fail(-8, "wgrad: groups >= split need a slot grad tensor");
      if ((rc = make_map_f32(&kp.c[1], d->out[1], (int64_t)(d->ngroups - d->split) * d->Mw, d->N, d->ldc))) return rc;
    }
    const bool pair = d->two_cta != 0 && grid >= 2 && d->Mw % (2 * BM) == 0;
    if (kp.sgd_w != nullptr) sgd_geometry(pair, &kp);
    kp.wg_select = kp.sgd_w != nullptr ? d->wg_select : 0;
    if (kp.sgd_w != nullptr)
      return pair ? launch_gemm2<true, true, EPI_F32, true, true>(kp, grid, stream)
                  : launch_gemm<true, true, true, EPI_F32, true>(kp, grid, stream);
    return pair ? launch_gemm2<true, true, EPI_F32, true>(kp, grid, stream)
                : launch_gemm<true, true, true, EPI_F32>(kp, grid, stream);
  }
  // A reduction tail is legal: the TMA loads zero-fill A beyond K, which also cancels whatever
  // a MN-major B tile picks up from the next expert's rows.
  if (d->K % 8 != 0) return fail(-4, "gemm: K=%d must be a multiple of 8", d->K);
  if (d->nseg < 1 || d->nseg > 2) return fail(-5, "gemm: nseg=%d", d->nseg);
  for (int s = 0; s < d->nseg; ++s)
    if ((rc = make_map(&kp.a[s], d->a[s], d->a_rows, d->K, d->lda[s], BK, BM))) return rc;
  if (d->nseg == 1) kp.a[1] = kp.a[0];
  const int nsel = (d->epi == EPI_SWIGLU) ? 2 : d->nseg;
  for (int s = 0; s < 2; ++s)
    for (int al = 0; al < 2; ++al) {
      const void* base = d->b[s < nsel ? s : 0][al] ? d->b[s < nsel ? s : 0][al] : d->b[s < nsel ? s : 0][0];
      const int64_t rows = d->b[s < nsel ? s : 0][al] ? d->b_rows[al] : d->b_rows[0];
      if (d->b_mn) {   // [K rows][N cols] per expert
        if ((rc = make_map(&kp.b[s][al], base, rows, d->N, d->ldb, 64, BK))) return rc;
        kp.b2[s][al] = kp.b[s][al];
      } else {         // [N rows][K cols] per expert
        if ((rc = make_map(&kp.b[s][al], base, rows, d->K, d->ldb, BK, BN))) return rc;
        if ((rc = make_map(&kp.b2[s][al], base, rows, d->K, d->ldb, BK, BN / 2))) return rc;
      }
    }
  // output maps of the staged epilogues (plain stores remain for unaligned outputs and for the
  // warps whose 32 rows straddle the end of a group)
  // The SwiGLU epilogue keeps plain stores: staging its three outputs measured no faster.
  if (d->epi == EPI_BF16 && (d->ldc * 2) % 16 == 0 && ((uintptr_t)d->out[0] & 15) == 0) {
    if ((rc = make_map(&kp.o, d->out[0], d->a_rows, d->N, d->ldc, 64, 32))) return rc;
    kp.tma_out = (d->debug & 16) ? 0 : 1;
  }
  const bool two = d->two_cta != 0 && grid >= 2;
  if (d->disp_mode != 0) {
    // ---- fused dispatch: the A operand is a row buffer of the Buffer behind disp_ctx ----------
    if (d->disp_ctx == nullptr) return fail(-20, "gemm: the fused dispatch needs the Buffer's context");
    const BufferCtx& c = *(const BufferCtx*)d->disp_ctx;
    if (c.virt) return fail(-21, "gemm: the fused dispatch runs one rank per launch (no virtual groups)");
    if (c.token_padding % BM != 0)
      return fail(-22, "gemm: the fused dispatch needs token_padding %% %d == 0 (tiles must not straddle groups)", BM);
    if (d->nseg != 1 || !d->b_mn || (d->epi != EPI_SWIGLU && d->epi != EPI_BF16))
      return fail(-23, "gemm: the fused dispatch feeds the gate/up (SwiGLU) and the down-dgrad GEMMs only");
    uint8_t* rows = (uint8_t*)c.shard_base(d->disp_shard);
    const long long row_bytes = (long long)c.H * 2;
    if (rows == nullptr || (const uint8_t*)d->a[0] != rows + (size_t)c.rank * c.hidden_stride * row_bytes)
      return fail(-24, "gemm: with the fused dispatch the A operand must be this rank's row buffer %d", d->disp_shard);
    const int nsplit = (int)((row_bytes + FD_PART_CAP - 1) / FD_PART_CAP);
    if (row_bytes % (16 * nsplit) != 0)
      return fail(-25, "gemm: a row of %lld bytes cannot travel in %d equal 16-byte multiples", row_bytes, nsplit);
    FusedDispatch& f = kp.disp;
    f.arrive = c.meta + (size_t)c.rank * c.meta_stride + c.ml.arrive_off;
    f.expect = BM * nsplit;
    f.nsplit = nsplit; f.row_bytes = (int)row_bytes;
    f.hidden = rows; f.meta = c.meta;
    f.hidden_stride_bytes = (long long)c.hidden_stride * row_bytes; f.meta_stride = c.meta_stride;
    f.weights_off = c.ml.weights_off; f.link_off = c.ml.link_off; f.src_off = c.ml.src_off;
    f.arrive_off = c.ml.arrive_off; f.NvS = c.NvS;
    f.N = (int)c.N; f.K = c.K; f.epn = c.epn; f.rank = c.rank; f.R = c.R; f.fresh = d->disp_fresh;
    if (d->disp_mode == 2) {
      if (d->disp_x == nullptr || d->disp_dst == nullptr || d->disp_order == nullptr || d->disp_zero_fill == nullptr)
        return fail(-26, "gemm: the fused dispatch needs the token rows, the plan's dst, send order and padding ranges");
      if (((uintptr_t)d->disp_x & 15) != 0) return fail(-27, "gemm: token rows must be 16-byte aligned");
      f.x = (const uint8_t*)d->disp_x; f.w = d->disp_w; f.dst = d->disp_dst; f.order = d->disp_order;
      f.zero_fill = d->disp_zero_fill;
    }
    kp.trace = c.trace;
    kp.arrive_timeout_ns = c.timeout_ns;                       // waits on other ranks: the Buffer's budget
    kp.timeout_ns = c.timeout_ns + c.timeout_ns / 2 + 200000000ull;
#ifdef MEP_GEMM_EXPERIMENTS
    if (const char* e = getenv("MOONEP_B200_FD_EXPERIMENT")) f.debug = atoi(e);
#endif
    if (d->epi == EPI_SWIGLU) {
      if (two) return launch_gemm2<false, true, EPI_SWIGLU, false, false, true>(kp, grid, stream);
      return launch_gemm<false, false, true, EPI_SWIGLU, false, true>(kp, grid, stream);
    }
    if (two) return launch_gemm2<false, true, EPI_BF16, false, false, true>(kp, grid, stream);
    return launch_gemm<false, false, true, EPI_BF16, false, true>(kp, grid, stream);
  }
  if (d->epi == EPI_SWIGLU) {
    if (!d->b_mn) return fail(-6, "swiglu epilogue expects MN-major weights");
    if (two) return launch_gemm2<false, true, EPI_SWIGLU>(kp, grid, stream);
    return launch_gemm<false, false, true, EPI_SWIGLU>(kp, grid, stream);
  }
  if (d->epi == EPI_BF16) {
    if (two) return d->b_mn ? launch_gemm2<false, true, EPI_BF16>(kp, grid, stream)
                            : launch_gemm2<false, false, EPI_BF16>(kp, grid, stream);
    return d->b_mn ? launch_gemm<false, false, true, EPI_BF16>(kp, grid, stream)
                   : launch_gemm<false, false, false, EPI_BF16>(kp, grid, stream);
  }
  if (d->epi == EPI_F32)
    return d->b_mn ? launch_gemm<false, false, true, EPI_F32>(kp, grid, stream)
                   : launch_gemm<false, false, false, EPI_F32>(kp, grid, stream);
  if (d->epi == EPI_PUSH) {
    if (d->src_info == nullptr || d->push_base == nullptr || d->push_entries <= 0)
      return fail(-9, "gemm: the push epilogue needs src_info and a staging buffer");
    if (two) return d->b_mn ? launch_gemm2<false, true, EPI_PUSH>(kp, grid, stream)
                            : launch_gemm2<false, false, EPI_PUSH>(kp, grid, stream);
    return d->b_mn ? launch_gemm<false, false, true, EPI_PUSH>(kp, grid, stream)
                   : launch_gemm<false, false, false, EPI_PUSH>(kp, grid, stream);
  }
  return fail(-7, "gemm: unknown epilogue %d", d->epi);
}

}  // extern "C"
