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

constexpr int DG_CHUNK = 256;        // rows scanned per pass of a CTA
constexpr int DG_POOL = 1024;        // duplicate rows recorded per pass

struct DupGroupList {
  int n;                              // groups found in this pass
  int pool_used;
  int prim[DG_CHUNK];                 // primary row of group i
  int start[DG_CHUNK];                // first entry of group i in pool, or -1 (walk the chain)
  int count[DG_CHUNK];                // duplicates of group i
  int pool[DG_POOL];                  // duplicate rows, chain order
};

// All threads of the CTA.  Scans rows [r0, r1) (r1 - r0 <= DG_CHUNK), rows >= `rows` do not exist.
// Ends with a __syncthreads(): the list is complete and readable by every thread.
__device__ __forceinline__ void collect_dup_groups(DupGroupList& L, const int32_t* link, int r0, int r1,
                                                   int rows) {
  if (threadIdx.x == 0) { L.n = 0; L.pool_used = 0; }
  __syncthreads();
  for (int r = r0 + (int)threadIdx.x; r < r1; r += (int)blockDim.x) {
    const int l = link[r];
    int next = l & LINK_NEXT_MASK;
    if ((l & LINK_DUP_BIT) != 0 || next == LINK_NONE || next >= rows) continue;
    // count the chain, reserve room, record it; the order of groups in the list is irrelevant
    int n = 0;
    for (int x = next; x != LINK_NONE && x < rows && n < MAX_TOPK - 1; x = link[x] & LINK_NEXT_MASK) ++n;
    const int i = atomicAdd(&L.n, 1);
    int at = atomicAdd(&L.pool_used, n);
    if (at + n > DG_POOL) at = -1;
    L.prim[i] = r;
    L.count[i] = n;
    L.start[i] = at;
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
