// Duplicate groups of a slice of this rank's rows, collected into shared memory.
//
// A duplicate group is a primary row followed (through the per-row chain links, common/layout.h)
// by the rows of the same token on this rank.  The two local kernels that work on groups -- the
// expansion after dispatch (primary copied to its duplicates) and the pre-reduction before the
// pull combine (duplicates added into the primary) -- are bandwidth kernels: each CTA first
// collects the groups whose primary lies in its slice of rows into a compact list, with every
// chain walked by its own thread (the dependent link loads of many groups overlap), and then
// streams the rows through a ring of bulk copies.  Reference counterparts build the same lists
// from their atomics-made dedup arrays (moonep/dispatch_epilogue.py:167-304,
// moonep/combine_prologue.py:196-484).
#pragma once
#include <cstdint>

#include "common/layout.h"

namespace mep {

constexpr int DG_CHUNK = 128;        // rows scanned per pass of a CTA
constexpr int DG_BLOCK = 16;         // consecutive rows that one CTA takes; blocks go round-robin over the CTAs
constexpr int DG_POOL = 1024;        // duplicate rows recorded per pass (7 per row before the slow path)

struct DupGroupList {
  int n;                              // groups found in this pass
  int pool_used;
  int prim[DG_CHUNK];                 // primary row of group i
  int start[DG_CHUNK];                // first entry of group i in pool, or -1 (walk the chain)
  int count[DG_CHUNK];                // duplicates of group i
  int pool[DG_POOL];                  // duplicate rows, chain order
};

// Rows are dealt to the CTAs in blocks of DG_BLOCK, round-robin: primaries cluster (with
// experts that sit next to one another, whole expert groups hold nothing but primaries and others
// nothing but duplicates), and contiguous slices would leave most CTAs idle.  Passes a CTA needs:
__device__ __forceinline__ int dup_group_passes(int rows, int n_cta) {
  const int blocks = (rows + DG_BLOCK - 1) / DG_BLOCK;
  const int per_pass = n_cta * (DG_CHUNK / DG_BLOCK);
  return (blocks + per_pass - 1) / per_pass;
}

// All threads of the CTA.  Collects the groups whose primary is among the rows of pass `pass` of
// CTA `cta`; rows >= `rows` do not exist.  Ends with a __syncthreads(): the list is complete and
// readable by every thread.
__device__ __forceinline__ void collect_dup_groups(DupGroupList& L, const int32_t* link, int pass, int cta,
                                                   int n_cta, int rows) {
  if (threadIdx.x == 0) { L.n = 0; L.pool_used = 0; }
  __syncthreads();
  for (int i = (int)threadIdx.x; i < DG_CHUNK; i += (int)blockDim.x) {
    const long long block = ((long long)pass * (DG_CHUNK / DG_BLOCK) + i / DG_BLOCK) * n_cta + cta;
    const long long r64 = block * DG_BLOCK + i % DG_BLOCK;
    if (r64 >= rows) continue;
    const int r = (int)r64;
    const int l = link[r];
    int next = l & LINK_NEXT_MASK;
    if ((l & LINK_DUP_BIT) != 0 || next == LINK_NONE || next >= rows) continue;
    // count the chain, reserve room, record it; the order of groups in the list is irrelevant
    int n = 0;
    for (int x = next; x != LINK_NONE && x < rows && n < MAX_TOPK - 1; x = link[x] & LINK_NEXT_MASK) ++n;
    const int at_i = atomicAdd(&L.n, 1);
    int at = atomicAdd(&L.pool_used, n);
    if (at + n > DG_POOL) at = -1;
    L.prim[at_i] = r;
    L.count[at_i] = n;
    L.start[at_i] = at;
    if (at >= 0) {
      int k = 0;
      for (int x = next; k < n; x = link[x] & LINK_NEXT_MASK) L.pool[at + k++] = x;
    }
  }
  __syncthreads();
}

// Row of duplicate k of group i (falls back to walking the chain when the pool was full).
__device__ __forceinline__ int dup_row(const DupGroupList& L, const int32_t* link, int i, int k) {
  if (L.start[i] >= 0) return L.pool[L.start[i] + k];
  int x = link[L.prim[i]] & LINK_NEXT_MASK;
  for (int j = 0; j < k; ++j) x = link[x] & LINK_NEXT_MASK;
  return x;
}

}  // namespace mep
