// CPU attention (oracle and CPU path): causal or full softmax attention with grouped KV
// heads, one query row at a time in fp32, keys visited in increasing order.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

// q: [B, L, Hq, D], k/v: [B, L, Hkv, D], out: [B, L, Hq, D], all fp32 contiguous;
// lse: [B, Hq, L] or null.
extern "C" int ka_cpu_attention(const float* q, const float* k, const float* v, float* out, float* lse, int batch,
                                int seq_len, int hq, int hkv, int d, float scale, int causal) {
  if (hq % hkv != 0) return -1;
  const int group = hq / hkv;
  std::vector<float> s(seq_len);
  for (int b = 0; b < batch; ++b)
    for (int h = 0; h < hq; ++h) {
      const int hk = h / group;
      for (int i = 0; i < seq_len; ++i) {
        const float* qi = q + ((static_cast<size_t>(b) * seq_len + i) * hq + h) * d;
        const int n = causal ? i + 1 : seq_len;
        float mx = -std::numeric_limits<float>::infinity();
        for (int j = 0; j < n; ++j) {
          const float* kj = k + ((static_cast<size_t>(b) * seq_len + j) * hkv + hk) * d;
          float acc = 0.f;
          for (int t = 0; t < d; ++t) acc += qi[t] * kj[t];
          s[j] = acc * scale;
          mx = std::max(mx, s[j]);
        }
        float l = 0.f;
        for (int j = 0; j < n; ++j) {
          s[j] = std::exp(s[j] - mx);
          l += s[j];
        }
        float* oi = out + ((static_cast<size_t>(b) * seq_len + i) * hq + h) * d;
        for (int t = 0; t < d; ++t) oi[t] = 0.f;
        for (int j = 0; j < n; ++j) {
          const float* vj = v + ((static_cast<size_t>(b) * seq_len + j) * hkv + hk) * d;
          const float w = s[j] / l;
          for (int t = 0; t < d; ++t) oi[t] += w * vj[t];
        }
        if (lse) lse[(static_cast<size_t>(b) * hq + h) * seq_len + i] = mx + std::log(l);
      }
    }
  return 0;
}
