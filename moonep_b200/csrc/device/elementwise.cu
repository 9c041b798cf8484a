// Memory-bound MoE ops that have no counterpart in the reference (it is a pure communication
// library): router top-k + softmax + tokens-per-expert histogram and its backward, the SwiGLU
// backward (the forward is fused into the gate/up GEMM epilogue), and the fused SGD update of
// bf16 weights from fp32 grads.  All are bandwidth kernels: 16-byte vector accesses, one pass.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "host/errors.h"

namespace mep {

// ---- router: top-k over (logits + bias), softmax over the selected unbiased logits ------------
constexpr int ROUTER_WARPS = 4;

__global__ void __launch_bounds__(ROUTER_WARPS * 32)
ep_router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int S, int E,
                      int K, int32_t* __restrict__ topk, float* __restrict__ weights,
                      int32_t* __restrict__ tpe) {
  extern __shared__ float s_vals[];   // [ROUTER_WARPS][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* v = s_vals + (size_t)warp * E;
  for (int s = blockIdx.x * ROUTER_WARPS + warp; s < S; s += gridDim.x * ROUTER_WARPS) {
    const float* row = logits + (size_t)s * E;
    for (int e = lane; e < E; e += 32) v[e] = row[e] + (bias ? bias[e] : 0.f);
    __syncwarp();
    float sel_logit = 0.f;   // lane k keeps the k-th selected raw logit
    int sel_idx = -1;
    for (int k = 0; k < K; ++k) {
      float bv = -FLT_MAX;
      int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        float x = v[e];
        if (x > bv) { bv = x; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == k) { sel_idx = bi; sel_logit = row[bi]; }
      if (lane == 0) v[bi] = -FLT_MAX;
      __syncwarp();
    }
    // softmax over the K selected logits (lanes 0..K-1)
    float m = lane < K ? sel_logit : -FLT_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float ex = lane < K ? __expf(sel_logit - m) : 0.f;
    float sum = ex;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane < K) {
      topk[(size_t)s * K + lane] = sel_idx;
      weights[(size_t)s * K + lane] = ex / sum;
      atomicAdd(&tpe[sel_idx], 1);
    }
    __syncwarp();
  }
}

// d logits = softmax backward scattered to the selected experts (zero elsewhere), bf16 so that
// it can feed the tensor-core GEMMs of the router's weight and input gradients.
__global__ void ep_router_topk_bwd_kernel(const float* __restrict__ weights, const float* __restrict__ dweights,
                                          const int32_t* __restrict__ topk, int S, int E, int K,
                                          __nv_bfloat16* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  for (int s = blockIdx.x * wpb + warp; s < S; s += gridDim.x * wpb) {
    float w = lane < K ? weights[(size_t)s * K + lane] : 0.f;
    float dw = lane < K ? dweights[(size_t)s * K + lane] : 0.f;
    float dot = w * dw;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    __nv_bfloat16* row = dlogits + (size_t)s * E;
    for (int e = lane; e < E; e += 32) row[e] = __float2bfloat16(0.f);
    __syncwarp();
    if (lane < K) row[topk[(size_t)s * K + lane]] = __float2bfloat16(w * (dw - dot));
  }
}

// ---- SwiGLU backward ----------------------------------------------------------------------------
// act = silu(g) * u * w  =>  dg = dact * u * w * silu'(g), du = dact * silu(g) * w,
//                            dw = sum_h dact * silu(g) * u
__global__ void __launch_bounds__(256)
ep_swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dact, const __nv_bfloat16* __restrict__ gate,
                     const __nv_bfloat16* __restrict__ up, const float* __restrict__ row_scale,
                     const int32_t* __restrict__ rows_ptr, int max_rows, int Hp,
                     __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dup,
                     float* __restrict__ dscale) {
  __shared__ float red[8];
  int rows = rows_ptr ? min(*rows_ptr, max_rows) : max_rows;
  const int nvec = Hp / 8;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float w = row_scale ? row_scale[r] : 1.f;
    const uint4* pd = reinterpret_cast<const uint4*>(dact + (size_t)r * Hp);
    const uint4* pg = reinterpret_cast<const uint4*>(gate + (size_t)r * Hp);
    const uint4* pu = reinterpret_cast<const uint4*>(up + (size_t)r * Hp);
    uint4* og = reinterpret_cast<uint4*>(dgate + (size_t)r * Hp);
    uint4* ou = reinterpret_cast<uint4*>(dup + (size_t)r * Hp);
    float acc = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      uint4 d4 = pd[v], g4 = pg[v], u4 = pu[v], rg, ru;
      const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d4);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
      __nv_bfloat162* og2 = reinterpret_cast<__nv_bfloat162*>(&rg);
      __nv_bfloat162* ou2 = reinterpret_cast<__nv_bfloat162*>(&ru);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 d = __bfloat1622float2(d2[i]), g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
        float s0 = 1.f / (1.f + __expf(-g.x)), s1 = 1.f / (1.f + __expf(-g.y));
        float sg0 = g.x * s0, sg1 = g.y * s1;
        acc += d.x * sg0 * u.x + d.y * sg1 * u.y;
        float dg0 = d.x * u.x * w * (s0 * (1.f + g.x * (1.f - s0)));
        float dg1 = d.y * u.y * w * (s1 * (1.f + g.y * (1.f - s1)));
        og2[i] = __floats2bfloat162_rn(dg0, dg1);
        ou2[i] = __floats2bfloat162_rn(d.x * sg0 * w, d.y * sg1 * w);
      }
      og[v] = rg;
      ou[v] = ru;
    }
    if (dscale) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) dscale[r] = t;
      }
      __syncthreads();
    }
  }
}

// ---- SGD: w(bf16) -= lr * g(fp32) ----------------------------------------------------------------
__global__ void __launch_bounds__(256)
ep_sgd_kernel(__nv_bfloat16* __restrict__ w, const float* __restrict__ g, long long n, float lr,
              const int32_t* __restrict__ only, long long vec_per_expert) {
  const long long nvec = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float nlr = -lr;
  long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x, v1 = nvec;
  if (only != nullptr) {
    // masked form: blockIdx.y is the expert; experts with a zero flag were updated elsewhere
    if (only[blockIdx.y] == 0) return;
    v0 += (long long)blockIdx.y * vec_per_expert;
    v1 = (long long)(blockIdx.y + 1) * vec_per_expert;
  }
  for (long long v = v0; v < v1; v += stride) {
    uint4 w4 = reinterpret_cast<uint4*>(w)[v];
    float4 g0 = reinterpret_cast<const float4*>(g)[2 * v], g1 = reinterpret_cast<const float4*>(g)[2 * v + 1];
    __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(&w4);
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = __bfloat1622float2(w2[i]);
      w2[i] = __floats2bfloat162_rn(__fmaf_rn(nlr, gg[2 * i], x.x), __fmaf_rn(nlr, gg[2 * i + 1], x.y));
    }
    reinterpret_cast<uint4*>(w)[v] = w4;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nvec * 8; i < n; ++i) w[i] = __float2bfloat16(__fmaf_rn(nlr, g[i], __bfloat162float(w[i])));
}

}  // namespace mep

using namespace mep;

extern "C" {

int mep_router_topk(const float* logits, const float* bias, int S, int E, int K, int32_t* topk,
                    float* weights, int32_t* tpe, cudaStream_t stream) {
  if (K > 32 || K < 1 || E < K) return fail(-1, "router: need 1 <= K <= min(32, E)");
  size_t smem = (size_t)ROUTER_WARPS * E * sizeof(float);
  if (smem > 200 * 1024) return fail(-2, "router: E=%d too large", E);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MEP_CUDA_OK(cudaFuncSetAttribute((const void*)ep_router_topk_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  MEP_CUDA_OK(cudaMemsetAsync(tpe, 0, sizeof(int32_t) * E, stream));
  int blocks = (S + ROUTER_WARPS - 1) / ROUTER_WARPS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ep_router_topk_kernel<<<blocks, ROUTER_WARPS * 32, smem, stream>>>(logits, bias, S, E, K, topk, weights, tpe);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

int mep_router_topk_bwd(const float* weights, const float* dweights, const int32_t* topk, int S, int E,
                        int K, void* dlogits, cudaStream_t stream) {
  int blocks = (S + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ep_router_topk_bwd_kernel<<<blocks, 256, 0, stream>>>(weights, dweights, topk, S, E, K,
                                                       (__nv_bfloat16*)dlogits);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

int mep_swiglu_bwd(const void* dact, const void* gate, const void* up, const float* row_scale,
                   const int32_t* rows_ptr, int max_rows, int Hp, void* dgate, void* dup,
                   float* dscale, cudaStream_t stream) {
  if (Hp % 8 != 0) return fail(-1, "swiglu_bwd: H'=%d must be a multiple of 8", Hp);
  int blocks = max_rows < 148 * 16 ? max_rows : 148 * 16;
  if (blocks < 1) return 0;
  ep_swiglu_bwd_kernel<<<blocks, 256, 0, stream>>>(
      (const __nv_bfloat16*)dact, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, row_scale,
      rows_ptr, max_rows, Hp, (__nv_bfloat16*)dgate, (__nv_bfloat16*)dup, dscale);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

int mep_sgd_update(void* w, const float* g, long long n, float lr, cudaStream_t stream) {
  if (((uintptr_t)w | (uintptr_t)g) % 16 != 0) return fail(-1, "sgd: tensors must be 16-byte aligned");
  long long nvec = n / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  ep_sgd_kernel<<<(int)blocks, 256, 0, stream>>>((__nv_bfloat16*)w, g, n, lr, nullptr, 1);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Same update, restricted to the experts whose flag is non-zero: w and g are [experts][elems].
int mep_sgd_update_masked(void* w, const float* g, long long experts, long long elems, const int32_t* only,
                          float lr, cudaStream_t stream) {
  if (((uintptr_t)w | (uintptr_t)g) % 16 != 0 || elems % 8 != 0)
    return fail(-1, "sgd: tensors must be 16-byte aligned and elems a multiple of 8");
  if (experts < 1 || experts > 65535) return fail(-2, "sgd: 1..65535 experts");
  long long nvec = elems / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  ep_sgd_kernel<<<dim3((unsigned)blocks, (unsigned)experts), 256, 0, stream>>>(
      (__nv_bfloat16*)w, g, 0, lr, only, nvec);
  MEP_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
