// Creation / destruction of the per-Buffer host context (see host/ctx.h).
#include "host/ctx.h"

#include <cuda_runtime.h>

#include "host/errors.h"

using namespace mep;

extern "C" {

int64_t mep_meta_chunk_ints(int64_t NvS, int R, int E) { return meta_layout(NvS, R, E).total; }
int64_t mep_plan_scratch_ints(int R, int E, int num_sms) { return plan_scratch_ints(R, E, num_sms); }
int mep_sync_state_ints() { return SYNC_STATE_INTS; }
// out[6]: weights_off, link_off, tpe_off, flags_off, arrive_off, src_off
void mep_meta_offsets(int64_t NvS, int R, int E, int64_t* out) {
  MetaLayout m = meta_layout(NvS, R, E);
  out[0] = m.weights_off; out[1] = m.link_off; out[2] = m.tpe_off; out[3] = m.flags_off;
  out[4] = m.arrive_off; out[5] = m.src_off;
}

// Returns an opaque handle (0 on failure, see mep_last_error).
void* mep_ctx_create(int rank, int R, int virt, int E, int S, int K, int H, int token_padding,
                     int num_sms, int num_sms_local, int num_sms_weights, void* hidden, int64_t hidden_stride_rows,
                     void* meta, int64_t meta_stride_ints, void* sync_state, void* status,
                     void* plan_scratch, int64_t timeout_ns) {
  if (R <= 0 || E <= 0 || E % R != 0 || S <= 0 || K <= 0 || K > MAX_TOPK || R > MAX_RANKS) {
    fail(-1, "ctx: bad sizes R=%d E=%d S=%d K=%d", R, E, S, K);
    return nullptr;
  }
  BufferCtx* c = new BufferCtx();
  c->rank = rank; c->R = R; c->virt = virt; c->E = E; c->epn = E / R; c->S = S; c->K = K; c->H = H;
  c->token_padding = token_padding; c->num_sms = num_sms; c->num_sms_local = num_sms_local;
  c->num_sms_weights = num_sms_weights > 0 ? num_sms_weights : num_sms;
  c->N = (int64_t)S * K;
  c->NvS = nvs_rows(S, K, c->epn, token_padding);
  if (c->NvS > MAX_NVS || (int64_t)R * c->NvS > INT32_MAX) {
    fail(-2, "ctx: NvS=%lld does not fit the 24-bit row / 31-bit slot encodings", (long long)c->NvS);
    delete c;
    return nullptr;
  }
  c->hidden = hidden; c->hidden2 = nullptr; c->hidden_stride = hidden_stride_rows;
  c->meta = (int32_t*)meta; c->meta_stride = meta_stride_ints;
  c->ml = meta_layout(c->NvS, R, E);
  c->sync_state = (int32_t*)sync_state; c->status = (int32_t*)status;
  c->plan_scratch = (int32_t*)plan_scratch;
  c->plan_scratch_ints = plan_scratch_ints(R, E, num_sms);
  c->timeout_ns = (unsigned long long)timeout_ns;
  c->pdl = 0;
  c->trace = nullptr;
  int dev = 0;
  c->sm_count = 0;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, dev);
  return c;
}

void mep_ctx_destroy(void* ctx) { delete (BufferCtx*)ctx; }

// Phase stamps: 1 when the library was built with -DMEP_PHASE_STAMPS; the buffer holds
// mep_trace_ints64() int64 words (kernels x CTAs x phases).
int mep_phase_stamps_compiled() {
#ifdef MEP_PHASE_STAMPS
  return 1;
#else
  return 0;
#endif
}
int64_t mep_trace_ints64() { return (int64_t)TRACE_KERNELS * TRACE_CTAS * TRACE_PHASES; }
void mep_trace_dims(int* out) { out[0] = TRACE_KERNELS; out[1] = TRACE_CTAS; out[2] = TRACE_PHASES; }
void mep_ctx_set_trace(void* ctx, void* trace) {
  if (ctx != nullptr) ((BufferCtx*)ctx)->trace = (long long*)trace;
}

// Programmatic dependent launch of the kernel chains (Buffer(enable_pdl=...)).
void mep_ctx_set_pdl(void* ctx, int enable) {
  if (ctx != nullptr) ((BufferCtx*)ctx)->pdl = enable ? 1 : 0;
}

// Registers the second symmetric row buffer (same geometry as the first).  Launchers select a
// buffer with their `shard` argument; nothing in the context is switched around a launch.
int mep_ctx_set_second_shard(void* ctx, void* hidden2) {
  BufferCtx* c = (BufferCtx*)ctx;
  if (c == nullptr || hidden2 == nullptr) return fail(-1, "ctx: set_second_shard needs a context and a buffer");
  c->hidden2 = hidden2;
  return 0;
}

}  // extern "C"
