// Planner entry point that allocates nothing.  It has no counterpart in the reference.
//
// Who needs it: code that may not call cudaMalloc when it wants a plan -- a plug-in living
// inside another runtime's memory budget (an inference server or a framework allocator that
// owns the whole device and forbids side allocations), a caller on a stream that is being
// captured, or a process that loaded this library only for one call and has no Buffer (whose
// constructor allocates scratch and symmetric memory) to lean on.
//
// What it does: the plan of ONE rank from an already gathered tokens-per-expert table: the same
// integer solve and per-entry assignment as the Buffer's planner kernel, in one CTA, without
// touching peer memory.  The caller passes every input and output; the planner's working
// tables (4 * R * E int32 plus a few status words) live in a file-scope device array inside
// the library instead of in memory allocated per Buffer.
//
// Limits and rules:
//   * R * E <= MEP_NOALLOC_MAX_RE (16384, e.g. E = 2048 experts on 8 ranks); larger problems
//     are rejected with an error, nothing is launched.
//   * the array (about 257 KB) is resident on every GPU that loads the library until exit.
//   * every call looks the array's device address up (cudaGetSymbolAddress with the calling
//     thread's current device); the FIRST call on a device also loads the module.  Make that
//     first call outside any stream capture.  Nothing is cached on the host, so a device reset
//     between calls is harmless and host threads share no state here.
//   * all calls on a device share the array, and it keeps what the last call left there; the
//     kernel clears the words that must start at zero.  Two calls that overlap on the GPU (two
//     streams, or two host threads) race on it: serialise them.
//   * no cudaMalloc / cudaFree / allocating library routine is called, on any path.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#define MEP_NOALLOC_MAX_RE 16384

extern "C" {

// All pointers are device pointers supplied by the caller.
//   tpe_all       [R][E]      in   tokens of expert e held by source rank r (already gathered)
//   topk          [S*K]       in   this rank's expert ids, token-major
//   dst           [S*K]       out  canonical destinations (negative = duplicate on that rank)
//   cu_seqlens    [2*epn]     out  padded END row of each group of this rank
//   zero_fill     [2*epn][2]  out  (first padding row, number of padding rows)
//   etc           [R][epn]    out  experts_to_copy table of the whole group
//   remote_stats  [2]         out
//   status        [8] or null out  0 in word 0 when every index stayed in range
// Returns 0 when the kernel was launched, a negative code (see mep_last_error) otherwise.
int mep_plan_local_noalloc(const int32_t* tpe_all, const int32_t* topk, int rank, int R, int E,
                           int S, int K, int token_padding, int32_t* dst, int32_t* cu_seqlens,
                           int32_t* zero_fill, int32_t* etc, int32_t* remote_stats,
                           int32_t* status, cudaStream_t stream);
}
