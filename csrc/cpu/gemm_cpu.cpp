// CPU oracles for the GEMM paths: a fixed-order GEMM, and an emulator of the tensor-parallel
// reduce-scatter arithmetic (8 canonical K slices, each slice partial rounded to bf16 once,
// partials added in fp32 in the order ((0+1)+(2+3))+((4+5)+(6+7)), residual added after one
// more bf16 rounding). The emulator takes the number of ranks only to show that it does not
// enter the arithmetic: any rank count gives the same bits.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline float bf16_round(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u) return f;
  u += 0x7FFFu + ((u >> 16) & 1u);
  u &= 0xFFFF0000u;
  std::memcpy(&f, &u, 4);
  return f;
}

inline float dot_range(const float* a, const float* b, int k0, int k1) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = k0;
  for (; i + 8 <= k1; i += 8)
    for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
  for (int j = 0; i < k1; ++i, ++j) acc[j] += a[i] * b[i];
  return ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}

template <typename F>
void parallel_rows(int rows, F&& f) {
  const int threads = std::max(1, std::min<int>(rows, std::min(16u, std::thread::hardware_concurrency())));
  std::vector<std::thread> pool;
  const int per = (rows + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const int lo = t * per, hi = std::min(rows, lo + per);
    if (lo < hi) pool.emplace_back([=, &f] { f(lo, hi); });
  }
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// c[m, n] = a[m, k] * b[n, k]^T, fp32, each dot product in a fixed 8-lane order.
int ka_cpu_gemm(const float* a, const float* b, float* c, int m, int n, int k) {
  parallel_rows(m, [&](int lo, int hi) {
    for (int i = lo; i < hi; ++i)
      for (int j = 0; j < n; ++j) c[static_cast<size_t>(i) * n + j] = dot_range(a + static_cast<size_t>(i) * k,
                                                                                 b + static_cast<size_t>(j) * k, 0, k);
  });
  return 0;
}

// out[m, n] = bf16( tree_s bf16(a[:, slice s] * b[:, slice s]^T) ) (+ residual after rounding),
// the arithmetic of the fused GEMM -> reduce-scatter. `world` must divide 8; it only decides
// which rank would own which slices, not the result.
int ka_cpu_gemm_sliced(const float* a, const float* b, const float* residual, float* out, int m, int n, int k,
                       int world) {
  if (k % 8 != 0 || (world != 1 && world != 2 && world != 4 && world != 8)) return -1;
  const int ks = k / 8;
  parallel_rows(m, [&](int lo, int hi) {
    for (int i = lo; i < hi; ++i)
      for (int j = 0; j < n; ++j) {
        float p[8];
        for (int r = 0; r < world; ++r)                       // every rank ...
          for (int s = r * (8 / world); s < (r + 1) * (8 / world); ++s)  // ... computes its slices
            p[s] = bf16_round(dot_range(a + static_cast<size_t>(i) * k, b + static_cast<size_t>(j) * k, s * ks,
                                        (s + 1) * ks));
        float v = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
        if (residual) v = bf16_round(v) + residual[static_cast<size_t>(i) * n + j];
        out[static_cast<size_t>(i) * n + j] = bf16_round(v);
      }
  });
  return 0;
}

}  // extern "C"
