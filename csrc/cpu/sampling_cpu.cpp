// CPU implementation of the fused sampler: the same definition as csrc/sm100/sampling.cu,
// written as straight serial code. Because every probability mass is a fixed-point integer
// and exp_det / Philox are shared through csrc/common/detmath.h, this returns the same token
// as the CUDA kernels for the same (row contents, seed, row id, step).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../common/detmath.h"

namespace {

using ka::exp_det;
using ka::float_to_key;
using ka::key_to_float;
using ka::mass_fixed;
using ka::mass_fraction;
using ka::mass_scale_u24;

constexpr int kMaxTopK = 1024;

struct KeyIdx {
  uint32_t key;
  uint32_t idx;
};

// sorted order of the sampler: larger key first, smaller token id first among equals
inline bool before(const KeyIdx& a, const KeyIdx& b) { return a.key > b.key || (a.key == b.key && a.idx < b.idx); }

int sample_row_topk(const float* x, int v, float inv_temp, int top_k, float top_p, uint32_t u24) {
  const int kk = std::min(std::min(top_k, kMaxTopK), v);
  std::vector<KeyIdx> all(v);
  for (int i = 0; i < v; ++i) all[i] = {float_to_key(x[i]), static_cast<uint32_t>(i)};
  std::partial_sort(all.begin(), all.begin() + kk, all.end(), before);
  std::vector<uint64_t> q(kk);
  const float y0 = ka::mul_rn(key_to_float(all[0].key), inv_temp);
  for (int i = 0; i < kk; ++i) {
    const float y = ka::mul_rn(key_to_float(all[i].key), inv_temp);
    q[i] = mass_fixed(exp_det(ka::sub_rn(y, y0)));
  }
  uint64_t z = 0;
  for (int i = 0; i < kk; ++i) z += q[i];
  int keep = kk;
  uint64_t zk = z;
  if (top_p < 1.0f) {
    const uint64_t limit = mass_fraction(static_cast<double>(top_p), z);
    uint64_t cum = 0;
    for (int i = 0; i < kk; ++i) {
      if (i > 0 && cum > limit) {
        keep = i;
        break;
      }
      cum += q[i];
    }
    zk = 0;
    for (int i = 0; i < keep; ++i) zk += q[i];
  }
  const uint64_t target = mass_scale_u24(u24, zk);
  uint64_t acc = 0;
  for (int i = 0; i < keep; ++i) {
    acc += q[i];
    if (acc > target) return static_cast<int>(all[i].idx);
  }
  return static_cast<int>(all[keep - 1].idx);
}

int sample_row_general(const float* x, int v, float inv_temp, int top_k, float top_p, uint32_t u24) {
  std::vector<KeyIdx> all(v);
  uint32_t max_key = 0;
  for (int i = 0; i < v; ++i) {
    all[i] = {float_to_key(x[i]), static_cast<uint32_t>(i)};
    max_key = std::max(max_key, all[i].key);
  }
  const float y_max = ka::mul_rn(key_to_float(max_key), inv_temp);
  std::vector<KeyIdx> sorted = all;
  std::sort(sorted.begin(), sorted.end(), before);
  auto mass_of = [&](uint32_t key) {
    const float y = ka::mul_rn(key_to_float(key), inv_temp);
    return mass_fixed(exp_det(ka::sub_rn(y, y_max)));
  };
  // prefix length by count
  size_t n_keep = static_cast<size_t>(v);
  if (top_k > 0 && top_k < v) n_keep = static_cast<size_t>(top_k);
  uint64_t zk = 0;
  for (size_t i = 0; i < n_keep; ++i) zk += mass_of(sorted[i].key);
  if (top_p < 1.0f) {
    const uint64_t limit = mass_fraction(static_cast<double>(top_p), zk);
    uint64_t cum = 0;
    size_t n_p = static_cast<size_t>(v);
    for (size_t i = 0; i < static_cast<size_t>(v); ++i) {
      if (i > 0 && cum > limit) {
        n_p = i;
        break;
      }
      cum += mass_of(sorted[i].key);
    }
    n_keep = std::min(n_keep, n_p);
  }
  std::vector<uint8_t> kept(v, 0);
  uint64_t kept_mass = 0;
  for (size_t i = 0; i < n_keep; ++i) {
    kept[sorted[i].idx] = 1;
    kept_mass += mass_of(sorted[i].key);
  }
  const uint64_t target = mass_scale_u24(u24, kept_mass);
  uint64_t acc = 0;
  int last = 0;
  for (int i = 0; i < v; ++i) {
    if (!kept[i]) continue;
    const uint64_t q = mass_of(all[i].key);
    acc += q;
    last = i;
    if (q != 0 && acc > target) return i;
  }
  return last;
}

}  // namespace

// logits: fp32 [rows, vocab] (callers widen 16-bit inputs, which is exact); semantics and
// argument meaning as ka_sample in csrc/sm100/sampling.h.
extern "C" int ka_cpu_sample(const float* logits, long long row_stride, int rows, int vocab, const long long* row_ids,
                             float inv_temperature, int top_k, float top_p, unsigned long long seed,
                             unsigned long long step, int* out) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || !(inv_temperature > 0.f) || !(top_p > 0.f)) return -1;
  for (int r = 0; r < rows; ++r) {
    const float* x = logits + static_cast<long long>(r) * row_stride;
    const uint64_t rid = row_ids ? static_cast<uint64_t>(row_ids[r]) : static_cast<uint64_t>(r);
    const uint32_t u24 = ka::uniform_u24(seed, rid, step);
    out[r] = (top_k >= 1 && top_k <= kMaxTopK) ? sample_row_topk(x, vocab, inv_temperature, top_k, top_p, u24)
                                               : sample_row_general(x, vocab, inv_temperature, top_k, top_p, u24);
  }
  return 0;
}

extern "C" unsigned int ka_cpu_uniform_u24(unsigned long long seed, unsigned long long row, unsigned long long step) {
  return ka::uniform_u24(seed, row, step);
}
