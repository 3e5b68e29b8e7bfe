// CPU implementations of the decoder's memory-bound ops (RMSNorm with fused residual, rotary
// embedding, SwiGLU) with the rounding points of the CUDA kernels in csrc/sm100/elementwise.cu:
// inputs and outputs are bf16 values carried in fp32 arrays, intermediate math is fp32.
#include <cmath>
#include <cstdint>
#include <cstring>

namespace {

inline float bf16_round(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u) return f;  // inf / nan
  u += 0x7FFFu + ((u >> 16) & 1u);
  u &= 0xFFFF0000u;
  std::memcpy(&f, &u, 4);
  return f;
}

}  // namespace

extern "C" {

// y = bf16(bf16(x' * rsqrt(mean(x'^2) + eps)) * w), x' = bf16(x + residual) when residual is given.
// The sum of squares follows the CUDA kernel's order: 256 strided lanes of 8-element vectors,
// a butterfly inside each group of 32 lanes, then the 8 groups left to right.
int ka_cpu_rmsnorm(const float* x, const float* residual, const float* w, float* y, float* residual_out, int rows,
                   int d, float eps) {
  if (d % 8 != 0) return -1;
  const int nvec = d / 8;
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + static_cast<size_t>(r) * d;
    const float* rr = residual ? residual + static_cast<size_t>(r) * d : nullptr;
    float lane[256];
    for (int t = 0; t < 256; ++t) lane[t] = 0.f;
    float* tmp = y + static_cast<size_t>(r) * d;  // holds x' until the second pass
    for (int i = 0; i < nvec; ++i) {
      const int t = i % 256;
      for (int j = 0; j < 8; ++j) {
        const int c = i * 8 + j;
        const float v = rr ? bf16_round(xr[c] + rr[c]) : xr[c];
        tmp[c] = v;
        lane[t] = std::fmaf(v, v, lane[t]);
      }
    }
    float warp_sum[8];
    for (int wg = 0; wg < 8; ++wg) {
      float v[32];
      for (int l = 0; l < 32; ++l) v[l] = lane[wg * 32 + l];
      for (int o = 16; o > 0; o >>= 1) {
        float n[32];
        for (int l = 0; l < 32; ++l) n[l] = v[l] + v[l ^ o];
        for (int l = 0; l < 32; ++l) v[l] = n[l];
      }
      warp_sum[wg] = v[0];
    }
    float total = 0.f;
    for (int wg = 0; wg < 8; ++wg) total += warp_sum[wg];
    const float inv = 1.0f / std::sqrt(total / static_cast<float>(d) + eps);
    for (int c = 0; c < d; ++c) {
      const float v = tmp[c];
      if (residual_out) residual_out[static_cast<size_t>(r) * d + c] = v;
      tmp[c] = bf16_round(bf16_round(v * inv) * w[c]);
    }
  }
  return 0;
}

// x: [tokens, heads, hd] contiguous, in place; cos/sin: [max_pos, hd/2].
int ka_cpu_rope(float* x, const long long* positions, const float* cos_t, const float* sin_t, int tokens, int heads,
                int hd) {
  if (hd % 2 != 0) return -1;
  const int half = hd / 2;
  for (int t = 0; t < tokens; ++t)
    for (int h = 0; h < heads; ++h) {
      float* p = x + (static_cast<size_t>(t) * heads + h) * hd;
      for (int j = 0; j < half; ++j) {
        const float c = cos_t[positions[t] * half + j], s = sin_t[positions[t] * half + j];
        const float a = p[j], b = p[j + half];
        p[j] = bf16_round(a * c - b * s);
        p[j + half] = bf16_round(b * c + a * s);
      }
    }
  return 0;
}

// out = bf16(bf16(silu(gate)) * up)
int ka_cpu_swiglu(const float* gate, const float* up, float* out, long long n) {
  for (long long i = 0; i < n; ++i) {
    const float g = gate[i];
    const float s = bf16_round(g / (1.0f + std::exp(-g)));
    out[i] = bf16_round(s * up[i]);
  }
  return 0;
}

}  // extern "C"
