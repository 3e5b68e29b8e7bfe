// CPU implementation of the fused LM-head + log-probability op and of log-prob from
// materialised logits. Oracle for the CUDA kernels and the code path of the CPU device.
//
// Batch invariance: a row's result is a function of that row only. Dot products use a fixed
// 8-lane accumulation order over K, logits are folded in row chunks of `chunk_rows` (the
// chunk only bounds the temporary, it never enters the arithmetic), and the vocabulary is
// decomposed exactly like the CUDA kernel: 8 canonical slices of ceil(V/8) columns,
// 1792-column sub-slices folded left to right in groups of 32 columns, sub-slices merged
// left to right, slices merged by a balanced binary tree.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <thread>
#include <vector>

namespace {

constexpr int kSlices = 8;
constexpr int kSubCols = 1792;
constexpr int kGroup = 32;
const float kNegInf = -std::numeric_limits<float>::infinity();

inline float dot_fixed(const float* a, const float* b, int k) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= k; i += 8)
    for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
  for (int j = 0; i < k; ++i, ++j) acc[j] += a[i] * b[i];
  return ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}

struct State {
  float m = kNegInf;  // running max of the scaled logits
  float l = 0.f;      // sum of exp(x - m)
};

inline void fold_group(State& s, const float* x, int n) {
  float mx = x[0];
  for (int j = 1; j < n; ++j) mx = std::max(mx, x[j]);
  const float mn = std::max(s.m, mx);
  float acc = 0.f;
  for (int j = 0; j < n; ++j) acc += std::exp(x[j] - mn);
  const float corr = (s.m == kNegInf) ? 0.f : std::exp(s.m - mn);
  s.l = s.l * corr + acc;
  s.m = mn;
}

inline void merge(State& a, const State& b) {
  const float mn = std::max(a.m, b.m);
  const float ca = (a.m == kNegInf) ? 0.f : std::exp(a.m - mn);
  const float cb = (b.m == kNegInf) ? 0.f : std::exp(b.m - mn);
  a.l = a.l * ca + b.l * cb;
  a.m = mn;
}

// State of canonical slice `sl` of one row of scaled logits given through a column accessor:
// 1792-column sub-slices, each folded in groups of 32 columns, merged left to right.
template <typename LogitAt>
inline State slice_state(int v, int sl, LogitAt&& at) {
  const int vs = (v + kSlices - 1) / kSlices;
  const int s_begin = std::min(v, sl * vs), s_end = std::min(v, (sl + 1) * vs);
  float buf[kGroup];
  State acc;
  bool first = true;
  for (int c0 = s_begin; c0 < s_end; c0 += kSubCols) {
    State sub;
    const int c1 = std::min(c0 + kSubCols, s_end);
    for (int g = c0; g < c1; g += kGroup) {
      const int n = std::min(kGroup, c1 - g);
      for (int j = 0; j < n; ++j) buf[j] = at(g + j);
      fold_group(sub, buf, n);
    }
    if (first) {
      acc = sub;
      first = false;
    } else {
      merge(acc, sub);
    }
  }
  return acc;
}

// The eight slice states of a row -> its log-sum-exp, by the balanced tree.
inline float tree_lse(State (&slice)[kSlices]) {
  for (int w = kSlices; w > 1; w >>= 1)
    for (int i = 0; i < w / 2; ++i) {
      State a = slice[2 * i];
      merge(a, slice[2 * i + 1]);
      slice[i] = a;
    }
  return slice[0].m + std::log(slice[0].l);
}

// log-sum-exp of one row of scaled logits given through a column accessor
template <typename LogitAt>
inline float row_lse(int v, LogitAt&& at) {
  State slice[kSlices];
  for (int sl = 0; sl < kSlices; ++sl) slice[sl] = slice_state(v, sl, at);
  return tree_lse(slice);
}

// out[r][c] = scale * <h_r, w_c> for nr rows and v columns. Columns are the outer loop so that a
// weight row is read once per chunk of rows; every dot product is still dot_fixed, so the
// result does not depend on nr. Compiled once more for AVX2 hosts (the eight accumulation
// lanes become one vector; the arithmetic and its order are the same, there is no FMA).
#if defined(__GNUC__) && defined(__x86_64__)
__attribute__((target_clones("avx2", "default")))
#endif
void logits_chunk(const float* h, const float* w, float* out, int nr, int k, int v, int out_stride, float scale) {
  for (int c = 0; c < v; ++c) {
    const float* wc = w + static_cast<size_t>(c) * k;
    for (int r = 0; r < nr; ++r)
      out[static_cast<size_t>(r) * out_stride + c] = dot_fixed(h + static_cast<size_t>(r) * k, wc, k) * scale;
  }
}

template <typename F>
void parallel_rows(int rows, int threads, F&& f) {
  threads = std::max(1, std::min(threads, rows));
  if (threads == 1) {
    f(0, rows);
    return;
  }
  std::vector<std::thread> pool;
  const int per = (rows + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const int lo = t * per, hi = std::min(rows, lo + per);
    if (lo < hi) pool.emplace_back([=, &f] { f(lo, hi); });
  }
  for (auto& th : pool) th.join();
}

}  // namespace

// hidden [m, k], weight [v, k], both fp32 row-major; ids [m] int64; logp / lse [m] fp32
// (lse may be null). `chunk_rows` bounds the logits temporary to chunk_rows * v floats per
// worker thread. Ids outside [0, v) give logp = 0.
extern "C" int ka_cpu_lmhead_logp(const float* hidden, const float* weight, const long long* ids, float* logp,
                                  float* lse, int m, int k, int v, float scale, int chunk_rows, int threads) {
  if (m <= 0) return 0;
  if (k <= 0 || v <= 0 || chunk_rows <= 0 || !(scale > 0.f)) return -1;
  parallel_rows(m, threads, [&](int lo, int hi) {
    std::vector<float> logits(static_cast<size_t>(chunk_rows) * v);
    for (int r0 = lo; r0 < hi; r0 += chunk_rows) {
      const int nr = std::min(chunk_rows, hi - r0);
      logits_chunk(hidden + static_cast<size_t>(r0) * k, weight, logits.data(), nr, k, v, v, scale);
      for (int r = 0; r < nr; ++r) {
        const float* x = logits.data() + static_cast<size_t>(r) * v;
        const float row_l = row_lse(v, [&](int c) { return x[c]; });
        if (lse) lse[r0 + r] = row_l;
        const long long id = ids[r0 + r];
        logp[r0 + r] = (id >= 0 && id < v) ? x[id] - row_l : 0.f;
      }
    }
  });
  return 0;
}

// logits fp32 [rows, v] with row stride in elements.
extern "C" int ka_cpu_logits_logp(const float* logits, long long row_stride, int rows, int v, const long long* ids,
                                  float scale, float* logp, float* lse, int threads) {
  if (rows <= 0) return 0;
  if (v <= 0 || !(scale > 0.f)) return -1;
  parallel_rows(rows, threads, [&](int lo, int hi) {
    for (int r = lo; r < hi; ++r) {
      const float* x = logits + static_cast<long long>(r) * row_stride;
      const float row_l = row_lse(v, [&](int c) { return x[c] * scale; });
      if (lse) lse[r] = row_l;
      const long long id = ids[r];
      logp[r] = (id >= 0 && id < v) ? x[id] * scale - row_l : 0.f;
    }
  });
  return 0;
}

// Vocabulary-parallel form, one shard: weight_shard holds rows [v_lo, v_lo + v_local) of the
// LM head, which must be whole canonical slices of the v_global-column vocabulary (slices
// slice0 .. slice0 + n_slices - 1). Writes, per row, the (max, sum) state of each of those
// slices into states[m][n_slices][2] and the scaled logit of the row's id into target[m] when
// the id lies in this shard (0 otherwise). The arithmetic is the single-process one.
extern "C" int ka_cpu_lmhead_logp_shard(const float* hidden, const float* weight_shard, const long long* ids,
                                        float* states, float* target, int m, int k, int v_global, int v_lo,
                                        int v_local, float scale, int threads) {
  if (m <= 0) return 0;
  if (k <= 0 || v_global <= 0 || v_local < 0 || !(scale > 0.f)) return -1;
  const int vs = (v_global + kSlices - 1) / kSlices;
  if (v_lo % vs != 0) return -2;
  const int slice0 = v_lo / vs;
  const int n_slices = (v_local + vs - 1) / vs;
  if (v_lo + v_local != std::min(v_global, (slice0 + n_slices) * vs) && v_local != 0) return -2;
  parallel_rows(m, threads, [&](int lo, int hi) {
    std::vector<float> logits(static_cast<size_t>(std::max(1, v_local)));
    for (int r = lo; r < hi; ++r) {
      const float* h = hidden + static_cast<size_t>(r) * k;
      logits_chunk(h, weight_shard, logits.data(), 1, k, v_local, v_local, scale);
      for (int i = 0; i < n_slices; ++i) {
        const State st = slice_state(v_global, slice0 + i, [&](int c) { return logits[c - v_lo]; });
        states[(static_cast<size_t>(r) * n_slices + i) * 2] = st.m;
        states[(static_cast<size_t>(r) * n_slices + i) * 2 + 1] = st.l;
      }
      const long long id = ids[r];
      target[r] = (id >= v_lo && id < v_lo + v_local) ? logits[id - v_lo] : 0.f;
    }
  });
  return 0;
}

// Merge step of the vocabulary-parallel form: states[m][8][2] in slice order (every rank's
// slices, concatenated in rank order), target[m] = sum over ranks of their target logits (only
// one is non-zero) -> logp, lse. Ids outside [0, v_global) give logp = 0.
extern "C" int ka_cpu_lmhead_logp_merge(const float* states, const float* target, const long long* ids, float* logp,
                                        float* lse, int m, int v_global) {
  for (int r = 0; r < m; ++r) {
    State slice[kSlices];
    for (int i = 0; i < kSlices; ++i) {
      slice[i].m = states[(static_cast<size_t>(r) * kSlices + i) * 2];
      slice[i].l = states[(static_cast<size_t>(r) * kSlices + i) * 2 + 1];
    }
    const float row_l = tree_lse(slice);
    if (lse) lse[r] = row_l;
    const long long id = ids[r];
    logp[r] = (id >= 0 && id < v_global) ? target[r] - row_l : 0.f;
  }
  return 0;
}
