// CPU oracle of the online redundant-expert planner.
//
// Behavioural counterpart of the reference's torch oracle (tests/planning_reference.py:25-236)
// and of its device planner (moonep/planning.py:584-1098): given the per-source-rank token
// counts tpe[R][E] it decides, for every expert, how many of its tokens each rank computes so
// that every rank receives exactly S*K rows, lays the groups out in each rank's buffer, and
// maps every (token, k) entry of one source rank to its destination slot.
//
// All arithmetic is integer, so the device planner must reproduce these tables bit for bit.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#include "common/layout.h"

namespace {

// First index of the maximum (ties -> smaller index), as torch.argmax does on CPU.
template <class It>
int argmax_first(It b, It e) {
  int best = 0;
  int i = 0;
  auto bv = *b;
  for (It it = b; it != e; ++it, ++i)
    if (*it > bv) { bv = *it; best = i; }
  return best;
}
template <class It>
int argmin_first(It b, It e) {
  int best = 0;
  int i = 0;
  auto bv = *b;
  for (It it = b; it != e; ++it, ++i)
    if (*it < bv) { bv = *it; best = i; }
  return best;
}

}  // namespace

extern "C" {

// Solve the plan for ALL ranks.  Returns 0 on success, a negative code when an invariant of
// the algorithm is violated (these are the AssertionErrors of the torch oracle).
//   tpe            [R][E]        in   tokens of expert e held by source rank r
//   tpe_cumsum     [R][E]        out  inclusive prefix over source ranks
//   alloc          [E][R]        out  tokens of expert e computed on rank d
//   alloc_cumsum   [E][R]        out  inclusive prefix over destination ranks
//   expert_off     [R][E]        out  first row of expert e in rank d's buffer (0 if absent)
//   cu_seqlens     [R][2epn]     out  padded END row of each group
//   zero_fill      [R][2epn][2]  out  (first padding row, number of padding rows)
//   experts_to_copy[R][epn]      out  expert computed in prefetch slot b of rank d, or -1
//   remote_stats   [R][2]        out  (#remote experts I compute, #slots elsewhere holding mine)
int mep_ref_plan_solve(const int32_t* tpe, int R, int E, int S, int K, int token_padding,
                       int64_t NvS, int32_t* tpe_cumsum, int32_t* alloc, int32_t* alloc_cumsum,
                       int32_t* expert_off, int32_t* cu_seqlens, int32_t* zero_fill,
                       int32_t* experts_to_copy, int32_t* remote_stats) {
  if (R <= 0 || E <= 0 || E % R != 0) return -1;
  const int epn = E / R;
  const int64_t CAP = (int64_t)S * K;

  for (int e = 0; e < E; ++e) {
    int32_t run = 0;
    for (int r = 0; r < R; ++r) {
      run += tpe[(size_t)r * E + e];
      tpe_cumsum[(size_t)r * E + e] = run;
    }
  }
  const int32_t* expert_count = tpe_cumsum + (size_t)(R - 1) * E;

  std::vector<int64_t> balance(R);
  for (int h = 0; h < R; ++h) {
    int64_t s = 0;
    for (int j = 0; j < epn; ++j) s += expert_count[h * epn + j];
    balance[h] = s - CAP;
  }

  std::memset(alloc, 0, sizeof(int32_t) * (size_t)E * R);
  for (int e = 0; e < E; ++e) alloc[(size_t)e * R + e / epn] = expert_count[e];

  // Receiver selection: the most overloaded home group fills the emptiest rank completely.
  std::vector<int32_t> z((size_t)R * R, 0);
  for (int round = 0; round <= R; ++round) {
    int h = argmax_first(balance.begin(), balance.end());
    int u = argmin_first(balance.begin(), balance.end());
    if (balance[h] <= 0) break;
    if (round == R) return -2;  // cannot happen: every round zeroes one receiver
    int64_t move = -balance[u];
    z[(size_t)h * R + u] = (int32_t)move;
    balance[h] -= move;
    balance[u] = 0;
  }

  // Expert selection: which experts of home group h move to which receiver.
  std::vector<int32_t> remaining(epn), quotas(R);
  for (int h = 0; h < R; ++h) {
    for (int j = 0; j < epn; ++j) remaining[j] = expert_count[h * epn + j];
    for (int d = 0; d < R; ++d) quotas[d] = z[(size_t)h * R + d];
    for (int guard = 0; guard <= epn + R + 1; ++guard) {
      int d = argmax_first(quotas.begin(), quotas.end());
      int32_t quota = quotas[d];
      if (quota <= 0) break;
      if (guard == epn + R + 1) return -3;
      int le = argmax_first(remaining.begin(), remaining.end());
      int32_t take = std::min(remaining[le], quota);
      if (take <= 0) return -4;
      int e = h * epn + le;
      alloc[(size_t)e * R + d] += take;
      alloc[(size_t)e * R + h] -= take;
      remaining[le] -= take;
      quotas[d] -= take;
    }
  }

  for (int e = 0; e < E; ++e) {
    int64_t s = 0;
    for (int d = 0; d < R; ++d) {
      s += alloc[(size_t)e * R + d];
      alloc_cumsum[(size_t)e * R + d] = (int32_t)s;
    }
    if (s != expert_count[e]) return -5;
  }
  for (int d = 0; d < R; ++d) {
    int64_t s = 0;
    for (int e = 0; e < E; ++e) s += alloc[(size_t)e * R + d];
    if (s > CAP) return -6;
  }

  std::memset(expert_off, 0, sizeof(int32_t) * (size_t)R * E);
  std::memset(cu_seqlens, 0, sizeof(int32_t) * (size_t)R * 2 * epn);
  std::memset(zero_fill, 0, sizeof(int32_t) * (size_t)R * 2 * epn * 2);
  std::memset(remote_stats, 0, sizeof(int32_t) * (size_t)R * 2);
  for (size_t i = 0; i < (size_t)R * epn; ++i) experts_to_copy[i] = -1;

  for (int d = 0; d < R; ++d) {
    const int ls = d * epn, le = ls + epn;
    int nremote = 0;
    for (int e = 0; e < E; ++e) {
      if (alloc[(size_t)e * R + d] > 0 && !(e >= ls && e < le)) {
        if (nremote >= epn) return -7;
        experts_to_copy[(size_t)d * epn + nremote++] = e;
        remote_stats[(size_t)(e / epn) * 2 + 1] += 1;
      }
    }
    remote_stats[(size_t)d * 2 + 0] = nremote;
    int64_t start = 0;
    for (int g = 0; g < 2 * epn; ++g) {
      int expert_id = -1;
      int32_t cnt = 0;
      if (g < epn) {
        expert_id = ls + g;
        cnt = alloc[(size_t)expert_id * R + d];
      } else if (experts_to_copy[(size_t)d * epn + (g - epn)] >= 0) {
        expert_id = experts_to_copy[(size_t)d * epn + (g - epn)];
        cnt = alloc[(size_t)expert_id * R + d];
      }
      int64_t padded = cnt > 0 ? mep::align_up64(cnt, token_padding) : 0;
      int64_t aligned_end = start + padded;
      cu_seqlens[(size_t)d * 2 * epn + g] = (int32_t)aligned_end;
      if (cnt > 0) {
        expert_off[(size_t)d * E + expert_id] = (int32_t)start;
        int64_t n_pad = padded - cnt;
        if (n_pad > 0) {
          zero_fill[((size_t)d * 2 * epn + g) * 2 + 0] = (int32_t)(start + cnt);
          zero_fill[((size_t)d * 2 * epn + g) * 2 + 1] = (int32_t)n_pad;
        }
      }
      start = aligned_end;
    }
    if (start > NvS) return -8;
  }
  return 0;
}

// Map the N = S*K entries of ONE source rank to destination slots.
//   dst[i] = dest_rank*NvS + row   for the first entry of a token that lands on dest_rank,
//   dst[i] = -(dest_rank*NvS+row)-1 for later entries of the same token on the same rank
//            (payload is not sent again; the route weight still is).
// (moonep/planning.py:1016-1081, tests/planning_reference.py:146-236)
int mep_ref_plan_assign(int rank, const int32_t* topk, int R, int E, int S, int K, int64_t NvS,
                        const int32_t* tpe_cumsum, const int32_t* alloc_cumsum,
                        const int32_t* expert_off, int32_t* dst) {
  const int64_t N = (int64_t)S * K;
  std::vector<int32_t> counter(E, 0);
  for (int64_t i = 0; i < N; ++i) {
    int e = topk[i];
    if (e < 0 || e >= E) return -1;
    int64_t prev = rank == 0 ? 0 : tpe_cumsum[(size_t)(rank - 1) * E + e];
    int64_t g = prev + counter[e]++;
    const int32_t* ac = alloc_cumsum + (size_t)e * R;
    int dest = (int)(std::upper_bound(ac, ac + R, (int32_t)g) - ac);
    if (dest >= R) return -2;
    int64_t prev_alloc = dest == 0 ? 0 : ac[dest - 1];
    int64_t v = (int64_t)dest * NvS + expert_off[(size_t)dest * E + e] + (g - prev_alloc);
    if (v > INT32_MAX) return -3;
    dst[i] = (int32_t)v;
  }
  for (int s = 0; s < S; ++s) {
    int32_t* d = dst + (size_t)s * K;
    for (int k = 1; k < K; ++k) {
      int64_t rk = d[k] / NvS;
      for (int j = 0; j < k; ++j) {
        int64_t raw = d[j] >= 0 ? d[j] : -(int64_t)d[j] - 1;
        if (raw / NvS == rk) { d[k] = -d[k] - 1; break; }
      }
    }
  }
  return 0;
}

}  // extern "C"
