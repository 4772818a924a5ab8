// Activation save-level solver: which (layer, chunk) slots to offload at which tier.
//
// Native counterpart of the reference's C transmission scheduler
// (helpers/transmission_scheduler/transmission_scheduler/transmission_scheduler.c:25-533) with its own
// formulation.  Tasks are the (layer, chunk) forward computations in execution order.  Task t ends
// computing at c_t = sum(compute[0..t]).  Saving it at tier L costs an outbound transfer of
// dur[t][L] ms and is worth value[t][L] ms of avoided recompute.  Rules:
//   (a) one outbound transfer at a time, in task order;
//   (b) a transfer starts no earlier than c_t;
//   (c) with N device slots, task t's transfer must finish before task t+N-1 starts computing
//       (its slot is recycled then), i.e. by c_{t+N-2};
//   (d) pinned tasks (the tail that never leaves the GPU) transfer nothing and earn their best value.
// The per-option durations come from the caller, so the same solver serves a PCIe host link or a
// faster NVLink peer-HBM link (the planner passes bytes / link bandwidth of whichever home it chose).
//
// State s = ticks the channel stays busy after c_t (s >= 0).  Choosing L: finish = s + dur;
// feasible iff finish <= deadline_t = c_{t+N-2} - c_t; next state s' = max(0, finish - compute[t+1]).
// The window is bounded by the largest finite deadline (a backlog beyond it can never be paid off) plus what the
// deadline-free tail can queue, so the table is T x (W+1) BYTES: only the chosen tier is stored per cell.  The
// predecessor of a cell follows from the transition (s = s' - dur + gap) except for the cells that collapse to
// s' = 0, which keep their arg-max source per task.  A round of a thousand tasks with a window of ten thousand
// ticks needs ~10 MB (the reference re-centres a sliding buffer with memmove for the same purpose,
// transmission_scheduler.c:25-209).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

namespace {

constexpr float NEG = -1e30f;

// new_row[j + shift] = max(new_row[j + shift], cur[j] + v) for j in [lo, hi); records choice/prev.
// Scalar reference loop.
inline void relax_scalar(const float* cur, float* nxt, uint8_t* choice, int32_t* prev, int lo, int hi, int shift,
                         float v, uint8_t L) {
  for (int j = lo; j < hi; ++j) {
    const float cand = cur[j] + v;
    const int d = j + shift;
    if (cand > nxt[d]) {
      nxt[d] = cand;
      choice[d] = L;
      prev[d] = j;
    }
  }
}

#if defined(__x86_64__)
__attribute__((target("avx2"))) inline void relax_avx2(const float* cur, float* nxt, uint8_t* choice, int32_t* prev,
                                                       int lo, int hi, int shift, float v, uint8_t L) {
  const __m256 vv = _mm256_set1_ps(v);
  const __m256i step = _mm256_setr_epi32(0, 1, 2, 3, 4, 5, 6, 7);
  int j = lo;
  for (; j + 8 <= hi; j += 8) {
    const __m256 cand = _mm256_add_ps(_mm256_loadu_ps(cur + j), vv);
    const __m256 old = _mm256_loadu_ps(nxt + j + shift);
    const __m256 gt = _mm256_cmp_ps(cand, old, _CMP_GT_OQ);
    const int mask = _mm256_movemask_ps(gt);
    if (mask == 0) continue;
    _mm256_storeu_ps(nxt + j + shift, _mm256_blendv_ps(old, cand, gt));
    const __m256i pj = _mm256_add_epi32(_mm256_set1_epi32(j), step);
    const __m256i pold = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(prev + j + shift));
    _mm256_storeu_si256(reinterpret_cast<__m256i*>(prev + j + shift),
                        _mm256_blendv_epi8(pold, pj, _mm256_castps_si256(gt)));
    for (int b = 0; b < 8; ++b)
      if (mask & (1 << b)) choice[j + shift + b] = L;
  }
  relax_scalar(cur, nxt, choice, prev, j, hi, shift, v, L);
}
#endif

inline void relax(const float* cur, float* nxt, uint8_t* choice, int32_t* prev, int lo, int hi, int shift, float v,
                  uint8_t L, bool avx2) {
  if (hi <= lo) return;
#if defined(__x86_64__)
  if (avx2) {
    relax_avx2(cur, nxt, choice, prev, lo, hi, shift, v, L);
    return;
  }
#endif
  relax_scalar(cur, nxt, choice, prev, lo, hi, shift, v, L);
}

}  // namespace

extern "C" {

// Number of bytes of scratch the solver will allocate for (T, window) — exposed so callers can
// refuse absurd problems up front (counterpart of compute_buf_size in the reference).
int64_t ftb_dp_buf_size(int T, int window_ticks) {
  return static_cast<int64_t>(T) * (window_ticks + 1) + 2 * static_cast<int64_t>(window_ticks + 1) * 4 +
         static_cast<int64_t>(T) * 8;
}

// compute_ms[T]; dur_ms[T*k]; value[T*k]; pinned[T] (0/1); n_slots = N; tick_ms > 0.
// valid_k[T]: number of valid tiers of task t (heterogeneous layers), 1..k.
// out_choice[T] receives the tier (0..k-1) or -1 for pinned/on-device tasks.
// Returns the optimal total value, or -1 if no feasible assignment exists (even all tier 0 is too slow).
double ftb_dp_solve(int T, int k, int n_slots, const double* compute_ms, const double* dur_ms, const double* value,
                    const uint8_t* pinned, const int32_t* valid_k, double tick_ms, int32_t* out_choice,
                    int force_scalar) {
  if (T <= 0) return 0.0;
  bool avx2 = false;
#if defined(__x86_64__)
  avx2 = !force_scalar && __builtin_cpu_supports("avx2");
#endif
  std::vector<int64_t> c(T + 1, 0);      // c[t+1] = end of task t in ticks (cumulative, rounded once)
  {
    double acc = 0;
    for (int t = 0; t < T; ++t) {
      acc += compute_ms[t];
      c[t + 1] = static_cast<int64_t>(std::llround(acc / tick_ms));
    }
  }
  auto cend = [&](int t) { return c[t + 1]; };
  // deadline (relative to c_t) by which task t's transfer must be finished
  std::vector<int64_t> deadline(T);
  int64_t W = 0;
  for (int t = 0; t < T; ++t) {
    const int last = t + n_slots - 2;   // task whose END marks the recycle time
    if (n_slots >= 2 && last < T - 1) deadline[t] = cend(last) - cend(t);
    else if (n_slots < 2) deadline[t] = 0;
    else deadline[t] = std::numeric_limits<int64_t>::max() / 4;
    if (deadline[t] < std::numeric_limits<int64_t>::max() / 8) W = std::max(W, deadline[t]);
  }
  // tasks with no finite deadline (the tail of the round) can still queue behind each other: their backlog is at
  // most the sum of their longest transfers
  {
    int64_t tail = 0;
    for (int t = 0; t < T; ++t) {
      if (pinned[t] || deadline[t] < std::numeric_limits<int64_t>::max() / 8) continue;
      double dmax = 0;
      for (int L = 0; L < valid_k[t]; ++L) dmax = std::max(dmax, dur_ms[t * k + L]);
      tail += static_cast<int64_t>(std::ceil(dmax / tick_ms));
    }
    W = std::max<int64_t>(W, tail);
  }
  W = std::min<int64_t>(std::max<int64_t>(W, 1), 1 << 22);
  const int S = static_cast<int>(W) + 1;

  std::vector<float> cur(S, NEG), nxt(S, NEG);
  std::vector<uint8_t> choice(static_cast<size_t>(T) * S, 255);
  std::vector<int32_t> prev(2 * static_cast<size_t>(S), -1);   // scratch rows for the relax kernels (not kept per task)
  std::vector<int32_t> prev0(T, -1);                            // source state of the cell s' = 0, per task
  std::vector<int64_t> gaps(T, 0);
  cur[0] = 0.f;

  for (int t = 0; t < T; ++t) {
    std::fill(nxt.begin(), nxt.end(), NEG);
    uint8_t* ch = choice.data() + static_cast<size_t>(t) * S;
    int32_t* pv = prev.data();
    pv[0] = -1;
    const int64_t gap = (t + 1 < T) ? (cend(t + 1) - cend(t)) : 0;   // compute time of task t+1 in ticks
    gaps[t] = gap;
    if (pinned[t]) {
      double best = 0;
      for (int L = 0; L < valid_k[t]; ++L) best = std::max(best, value[t * k + L]);
      // backlog just drains by `gap`
      const int g = static_cast<int>(std::min<int64_t>(gap, S));
      // states j < g collapse to 0
      float m = NEG; int arg = -1;
      for (int j = 0; j < std::min(g + 1, S); ++j) if (cur[j] > m) { m = cur[j]; arg = j; }
      if (arg >= 0) { nxt[0] = m + static_cast<float>(best); ch[0] = 254; pv[0] = arg; }
      relax(cur.data(), nxt.data(), ch, pv, g + 1, S, -g, static_cast<float>(best), 254, avx2);
    } else {
      for (int L = 0; L < valid_k[t]; ++L) {
        const int64_t d = static_cast<int64_t>(std::ceil(dur_ms[t * k + L] / tick_ms - 1e-9));
        const float v = static_cast<float>(value[t * k + L]);
        // feasible source states: j + d <= deadline
        const int64_t jmax64 = std::min<int64_t>(S - 1, deadline[t] - d);
        if (jmax64 < 0) continue;
        const int jmax = static_cast<int>(jmax64);
        // destination = max(0, j + d - gap), clipped to the window
        const int64_t sh = d - gap;
        // part 1: j + sh <= 0  -> destination 0
        const int jz = static_cast<int>(std::min<int64_t>(jmax, -sh));
        if (jz >= 0) {
          float m = NEG; int arg = -1;
          for (int j = 0; j <= jz; ++j) if (cur[j] > m) { m = cur[j]; arg = j; }
          if (arg >= 0 && m + v > nxt[0]) { nxt[0] = m + v; ch[0] = static_cast<uint8_t>(L); pv[0] = arg; }
        }
        // part 2: shifted copy
        const int lo = static_cast<int>(std::max<int64_t>(0, -sh + 1));
        const int hi = static_cast<int>(std::min<int64_t>(jmax + 1, S - sh));
        relax(cur.data(), nxt.data(), ch, pv, lo, hi, static_cast<int>(sh), v, static_cast<uint8_t>(L), avx2);
      }
    }
    prev0[t] = pv[0];
    cur.swap(nxt);
  }
  // best terminal state
  float best = NEG; int arg = -1;
  for (int j = 0; j < S; ++j) if (cur[j] > best) { best = cur[j]; arg = j; }
  if (arg < 0 || best <= NEG / 2) return -1.0;
  for (int t = T - 1; t >= 0; --t) {
    const uint8_t L = choice[static_cast<size_t>(t) * S + arg];
    if (L == 255) return -1.0;
    out_choice[t] = (L == 254) ? -1 : static_cast<int32_t>(L);
    if (arg == 0) {
      arg = prev0[t];                       // several source states collapse to 0: the arg-max one was recorded
    } else {
      // s' = s + dur - gap (pinned: s' = s - gap), so the source follows from the chosen tier
      const int64_t d = (L == 254) ? 0 : static_cast<int64_t>(std::ceil(dur_ms[t * k + L] / tick_ms - 1e-9));
      const int64_t src = static_cast<int64_t>(arg) - d + gaps[t];
      arg = (src < 0 || src >= S) ? -1 : static_cast<int>(src);
    }
    if (arg < 0) return -1.0;
  }
  return static_cast<double>(best);
}

}  // extern "C"
