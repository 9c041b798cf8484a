// Shared constants and small integer helpers used by the CPU oracle, the host launchers
// and the device kernels.  Everything here is plain C++ (no CUDA), so that the oracle and
// the kernels cannot drift apart on an encoding.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define MEP_HD __host__ __device__ __forceinline__
#else
#define MEP_HD inline
#endif

namespace mep {

// ---- duplicate chains -----------------------------------------------------------------
// A token whose top-k picks several experts that are computed on the SAME destination rank
// sends its hidden row there once (to the "primary" slot, the smallest k); the other slots
// ("duplicates") are filled on the destination from the primary.  The reference rebuilds
// this relation on the destination with atomics from a per-slot source record
// (moonep/dispatch.py:499-681).  Here the SOURCE rank, which already knows all K slots of
// its token, writes one 32-bit link per slot into the destination's meta chunk:
//   bits 23..0  : local row offset of the next duplicate of the same token, or LINK_NONE
//   bit  30     : this slot is a duplicate (not the primary of its chain)
// A slot that is alone (no duplicates) holds LINK_NONE.  Chains are in ascending k.
constexpr int32_t LINK_NONE = 0x00FFFFFF;
constexpr int32_t LINK_DUP_BIT = 0x40000000;
constexpr int32_t LINK_NEXT_MASK = 0x00FFFFFF;
// Same encoding limits as the reference (moonep/planning.py:1231-1255).
constexpr int MAX_TOPK = 32;
constexpr int MAX_RANKS = 128;
constexpr int64_t MAX_NVS = (1 << 24) - 1;

MEP_HD int64_t align_up64(int64_t x, int64_t a) { return (x + a - 1) / a * a; }
MEP_HD int align_up(int x, int a) { return (x + a - 1) / a * a; }

// Rows of the per-rank dispatch buffer: S*K real rows plus worst-case padding of the
// (at most) 2*epn non-empty groups (moonep/api.py:265-266).
MEP_HD int64_t nvs_rows(int64_t S, int64_t K, int64_t epn, int64_t token_padding) {
  return align_up64(S * K + (token_padding - 1) * 2 * epn, token_padding);
}

// ---- meta chunk layout (int32 elements, one chunk per rank in symmetric memory) ---------
//   WEIGHTS  [NvS]        fp32 route weights, slot order (bit-cast)
//   LINK     [NvS]        duplicate chain links written by the source ranks
//   TPE      [2][R][E]    gathered tokens-per-expert, double buffered by plan parity
//   FLAGS    [2][R]       barrier arrival epochs, slot p is written by rank p; channel 0 serves
//                         dispatch / combine, channel 1 the weight ops (prefetch_weight,
//                         reduce_grad), so the two families may run concurrently
//   ARRIVE   [NvS/128+1]  per-128-row tile arrival counters (fused dispatch->GEMM path)
//   SRC      [NvS]        per slot: source_rank * (S*K) + (token*K + k) of the entry that owns
//                         it, written by the source ranks' planners (-1 on padding rows); the
//                         GEMM epilogue that pushes results home reads it
struct MetaLayout {
  int64_t weights_off, link_off, tpe_off, flags_off, arrive_off, src_off, total;
};
MEP_HD MetaLayout meta_layout(int64_t NvS, int64_t R, int64_t E) {
  MetaLayout m;
  m.weights_off = 0;
  m.link_off = align_up64(NvS, 4);
  m.tpe_off = m.link_off + align_up64(NvS, 4);
  m.flags_off = m.tpe_off + align_up64(2 * R * E, 4);
  m.arrive_off = m.flags_off + 2 * align_up64(R, 32);
  m.src_off = m.arrive_off + align_up64(NvS / 128 + 1, 32);
  m.total = m.src_off + align_up64(NvS, 4);
  return m;
}

}  // namespace mep
