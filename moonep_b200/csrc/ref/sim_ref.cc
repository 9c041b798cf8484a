// CPU multi-rank simulator of dispatch / combine semantics: all R ranks live in one process
// and plain arrays stand in for peer memory.  It is the oracle for the device kernels and
// the engine of the GPU-less configuration (R simulated ranks).
//
// Semantics follow the reference kernels: fused permute + all-to-all with one payload copy
// per destination rank (moonep/dispatch.py:387-448), zero-filled group padding
// (dispatch.py:467-497), local duplicate expansion (dispatch_epilogue.py:212-304), fp32
// pre-reduction of duplicates in chain order (combine_prologue.py:196-484) and the K-way
// fp32 pull-sum of primaries in ascending k (combine.py:308-435).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "common/layout.h"

namespace {

inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
// Round to nearest even, as cvt.rn.bf16.f32 does.
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7FFFu + lsb;
  return (uint16_t)(u >> 16);
}

struct Elem {
  int size;  // 4 = fp32, 2 = bf16
  float load(const uint8_t* p, int64_t i) const {
    if (size == 4) { float f; std::memcpy(&f, p + 4 * i, 4); return f; }
    uint16_t v; std::memcpy(&v, p + 2 * i, 2); return bf16_to_f32(v);
  }
  void store(uint8_t* p, int64_t i, float f) const {
    if (size == 4) { std::memcpy(p + 4 * i, &f, 4); return; }
    uint16_t v = f32_to_bf16(f); std::memcpy(p + 2 * i, &v, 2);
  }
};

}  // namespace

extern "C" {

// Dispatch for all ranks at once.
//   x        [R][S][H]   elem_size bytes per element (2 = bf16, 4 = fp32)
//   w        [R][S][K]   fp32 route weights, may be null
//   dst      [R][N]      canonical destinations from the planner
//   zero_fill[R][2epn][2]
//   hidden   [R][NvS][H] out (rows outside real+padding rows are left untouched)
//   w_nvs    [R][NvS]    out, may be null iff w is null
//   link     [R][NvS]    out duplicate chains (see common/layout.h)
//   expand   != 0: copy each primary row to its duplicates (the dispatch epilogue)
int mep_sim_dispatch(const void* x, const float* w, const int32_t* dst, const int32_t* zero_fill,
                     int R, int S, int K, int H, int epn, int64_t NvS, int elem_size,
                     void* hidden, float* w_nvs, int32_t* link, int expand) {
  if (elem_size != 2 && elem_size != 4) return -1;
  const int64_t N = (int64_t)S * K;
  const size_t row_bytes = (size_t)H * elem_size;
  const uint8_t* xs = (const uint8_t*)x;
  uint8_t* hs = (uint8_t*)hidden;
  for (int r = 0; r < R; ++r) {
    for (int s = 0; s < S; ++s) {
      const int32_t* d = dst + (size_t)r * N + (size_t)s * K;
      for (int k = 0; k < K; ++k) {
        int64_t raw = d[k] >= 0 ? d[k] : -(int64_t)d[k] - 1;
        int64_t dr = raw / NvS, loff = raw % NvS;
        if (dr < 0 || dr >= R) return -2;
        if (w && w_nvs) w_nvs[(size_t)dr * NvS + loff] = w[((size_t)r * S + s) * K + k];
        if (d[k] >= 0)
          std::memcpy(hs + ((size_t)dr * NvS + loff) * row_bytes,
                      xs + ((size_t)r * S + s) * row_bytes, row_bytes);
        if (link) {
          // next entry of this token on the same destination rank, if any
          int32_t next = mep::LINK_NONE;
          for (int j = k + 1; j < K; ++j) {
            int64_t rj = d[j] >= 0 ? d[j] : -(int64_t)d[j] - 1;
            if (rj / NvS == dr) { next = (int32_t)(rj % NvS); break; }
          }
          link[(size_t)dr * NvS + loff] = next | (d[k] < 0 ? mep::LINK_DUP_BIT : 0);
        }
      }
    }
  }
  for (int r = 0; r < R; ++r)
    for (int g = 0; g < 2 * epn; ++g) {
      int64_t first = zero_fill[((size_t)r * 2 * epn + g) * 2];
      int64_t n = zero_fill[((size_t)r * 2 * epn + g) * 2 + 1];
      if (n <= 0) continue;
      std::memset(hs + ((size_t)r * NvS + first) * row_bytes, 0, (size_t)n * row_bytes);
      if (w_nvs) std::memset(w_nvs + (size_t)r * NvS + first, 0, (size_t)n * 4);
      if (link)
        for (int64_t i = 0; i < n; ++i) link[(size_t)r * NvS + first + i] = mep::LINK_NONE;
    }
  if (expand && link) {
    // Real rows of rank r are [group start, first padding row) of every non-empty group.
    // Walking dst again is simpler than walking groups and touches exactly the real rows.
    for (int r = 0; r < R; ++r)
      for (int64_t i = 0; i < N; ++i) {
        int32_t dv = dst[(size_t)r * N + i];
        if (dv < 0) continue;
        int64_t dr = dv / NvS, loff = dv % NvS;
        int32_t l = link[(size_t)dr * NvS + loff];
        const uint8_t* src = hs + ((size_t)dr * NvS + loff) * row_bytes;
        int guard = 0;
        while ((l & mep::LINK_NEXT_MASK) != mep::LINK_NONE) {
          int64_t nx = l & mep::LINK_NEXT_MASK;
          std::memcpy(hs + ((size_t)dr * NvS + nx) * row_bytes, src, row_bytes);
          l = link[(size_t)dr * NvS + nx];
          if (++guard > mep::MAX_TOPK) return -3;
        }
      }
  }
  return 0;
}

// Combine for all ranks at once (unweighted sum, like the reference: the route-weight
// multiply belongs to the expert FFN).
//   hidden [R][NvS][H] in/out: with prologue != 0 each primary row is first replaced by the
//          fp32 sum of itself and its duplicates (chain order), rounded to the element type
//   out    [R][S][H]
//   w_nvs  [R][NvS] / w_out [R][S][K]: optional bit-exact gather of the route weights
int mep_sim_combine(void* hidden, const float* w_nvs, const int32_t* dst, const int32_t* link,
                    int R, int S, int K, int H, int64_t NvS, int elem_size, int prologue,
                    void* out, float* w_out) {
  if (elem_size != 2 && elem_size != 4) return -1;
  Elem el{elem_size};
  const int64_t N = (int64_t)S * K;
  const size_t row_bytes = (size_t)H * elem_size;
  uint8_t* hs = (uint8_t*)hidden;
  uint8_t* os = (uint8_t*)out;
  std::vector<float> acc(H);
  if (prologue && link) {
    for (int r = 0; r < R; ++r)
      for (int64_t i = 0; i < N; ++i) {
        int32_t dv = dst[(size_t)r * N + i];
        if (dv < 0) continue;
        int64_t dr = dv / NvS, loff = dv % NvS;
        int32_t l = link[(size_t)dr * NvS + loff];
        if ((l & mep::LINK_NEXT_MASK) == mep::LINK_NONE) continue;
        uint8_t* prim = hs + ((size_t)dr * NvS + loff) * row_bytes;
        for (int h = 0; h < H; ++h) acc[h] = el.load(prim, h);
        int guard = 0;
        while ((l & mep::LINK_NEXT_MASK) != mep::LINK_NONE) {
          int64_t nx = l & mep::LINK_NEXT_MASK;
          const uint8_t* dp = hs + ((size_t)dr * NvS + nx) * row_bytes;
          for (int h = 0; h < H; ++h) acc[h] += el.load(dp, h);
          l = link[(size_t)dr * NvS + nx];
          if (++guard > mep::MAX_TOPK) return -3;
        }
        for (int h = 0; h < H; ++h) el.store(prim, h, acc[h]);
      }
  }
  for (int r = 0; r < R; ++r)
    for (int s = 0; s < S; ++s) {
      const int32_t* d = dst + (size_t)r * N + (size_t)s * K;
      for (int h = 0; h < H; ++h) acc[h] = 0.f;
      for (int k = 0; k < K; ++k) {
        int64_t raw = d[k] >= 0 ? d[k] : -(int64_t)d[k] - 1;
        int64_t dr = raw / NvS, loff = raw % NvS;
        if (w_nvs && w_out) w_out[((size_t)r * S + s) * K + k] = w_nvs[(size_t)dr * NvS + loff];
        if (d[k] < 0) continue;
        const uint8_t* src = hs + ((size_t)dr * NvS + loff) * row_bytes;
        for (int h = 0; h < H; ++h) acc[h] += el.load(src, h);
      }
      uint8_t* o = os + ((size_t)r * S + s) * row_bytes;
      for (int h = 0; h < H; ++h) el.store(o, h, acc[h]);
    }
  return 0;
}

}  // extern "C"
