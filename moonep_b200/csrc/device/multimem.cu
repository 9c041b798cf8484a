// NVSwitch multicast (NVLS) stores: one store through the multicast alias of a symmetric buffer
// lands in every rank's copy.  The reference broadcasts its plan tables this way
// (multimem.st.relaxed.sys.v4, moonep/planning.py:147-156,917-922).  This library's planner needs
// no broadcast (every rank solves redundantly), so the only user is this utility: it copies a
// local table into the same offset of every rank's chunk, for callers that keep replicated
// tables in symmetric memory.  Stores only: nothing here loads through a multicast address.
#include <cuda_runtime.h>

#include <cstdint>

#include "host/errors.h"

namespace mep {

__global__ void __launch_bounds__(256) ep_multimem_bcast_kernel(uint32_t* alias, const uint32_t* src,
                                                                int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint32_t v = src[i];
    asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(alias + i), "r"(v) : "memory");
  }
  // the stores are ordered before whatever flag or barrier the caller uses next
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

}  // namespace mep

using namespace mep;

extern "C" {

// alias_dst: address inside the multicast alias of a symmetric tensor (4-byte aligned); src: n
// 32-bit words in local memory.  After the caller's next cross-rank synchronisation every rank's
// chunk holds the words at the same offset.
int mep_launch_multimem_bcast(void* alias_dst, const void* src, int64_t n, cudaStream_t stream) {
  if (alias_dst == nullptr || src == nullptr || n < 0) return fail(-1, "multimem bcast: bad arguments");
  if (((uintptr_t)alias_dst & 3) != 0 || ((uintptr_t)src & 3) != 0)
    return fail(-2, "multimem bcast: addresses must be 4-byte aligned");
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 64) blocks = 64;
  ep_multimem_bcast_kernel<<<blocks, 256, 0, stream>>>((uint32_t*)alias_dst, (const uint32_t*)src, n);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
