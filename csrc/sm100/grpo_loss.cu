// GRPO objective: group-normalised advantages and the clipped-ratio policy loss, forward and
// the gradient coefficients in one pass.
//
//   ratio_t = exp(logp_new_t - logp_old_t)
//   obj_t   = min(ratio_t * A, clip(ratio_t, 1 - eps_low, 1 + eps_high) * A)
//   kl_t    = exp(ref_t - new_t) - (ref_t - new_t) - 1                        (if beta > 0)
//   loss    = mean over valid tokens of (-obj_t + beta * kl_t)     [token mean], or the mean over
//             sequences of each sequence's token mean                         [sequence mean]
//
// One CTA per sequence reduces its tokens in a fixed order, one CTA combines the sequences in
// index order: no atomics, so the loss is bitwise reproducible run to run. The kernel also
// writes d(loss_t)/d(logp_new_t) per token (unnormalised) and a per-sequence weight; the
// backward pass is the product of the two with the upstream gradient.
//
// The reference mentions the GRPO loss only in its README feature list.
#include <cstdint>
#include <cuda_runtime.h>

#include "common/ptx.cuh"

namespace ka {
namespace {

constexpr int kThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float exp_f(float x) { return ex2_approx(__fmul_rn(x, kLog2e)); }

__device__ __forceinline__ float block_sum_fixed(float v, float* s_warp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) s_warp[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < kThreads / 32; ++w) t = __fadd_rn(t, s_warp[w]);
  return t;
}

// rewards [n_groups * group]; adv = (r - mean_group) / (std_group + eps), std unbiased.
__global__ void advantages_kernel(const float* __restrict__ rewards, float* __restrict__ adv, int n_groups, int group,
                                  float eps) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  const float* r = rewards + static_cast<long long>(g) * group;
  float sum = 0.f;
  for (int i = 0; i < group; ++i) sum = __fadd_rn(sum, r[i]);
  const float mean = __fdiv_rn(sum, static_cast<float>(group));
  float ss = 0.f;
  for (int i = 0; i < group; ++i) {
    const float d = __fsub_rn(r[i], mean);
    ss = __fmaf_rn(d, d, ss);
  }
  const float var = group > 1 ? __fdiv_rn(ss, static_cast<float>(group - 1)) : 0.f;
  const float inv = __fdiv_rn(1.f, __fadd_rn(__fsqrt_rn(var), eps));
  for (int i = 0; i < group; ++i) adv[static_cast<long long>(g) * group + i] = __fmul_rn(__fsub_rn(r[i], mean), inv);
}

__global__ void __launch_bounds__(kThreads)
grpo_tokens_kernel(const float* __restrict__ logp_new, const float* __restrict__ logp_old,
                   const float* __restrict__ logp_ref, const float* __restrict__ adv,
                   const unsigned char* __restrict__ mask, int seq_len, float eps_low, float eps_high, float beta,
                   float* __restrict__ raw_grad, float* __restrict__ seq_sum, float* __restrict__ seq_cnt,
                   float* __restrict__ seq_clip) {
  __shared__ float s_warp[kThreads / 32];
  const int seq = blockIdx.x;
  const float a = adv[seq];
  float sum = 0.f, cnt = 0.f, clipped = 0.f;
  for (int t = threadIdx.x; t < seq_len; t += kThreads) {
    const long long i = static_cast<long long>(seq) * seq_len + t;
    float g = 0.f;
    if (!mask || mask[i]) {
      const float ln = logp_new[i];
      const float ratio = exp_f(__fsub_rn(ln, logp_old[i]));
      const float s1 = __fmul_rn(ratio, a);
      const float rc = fminf(fmaxf(ratio, 1.f - eps_low), 1.f + eps_high);
      const float s2 = __fmul_rn(rc, a);
      const bool unclipped = s1 <= s2;
      float loss = -(unclipped ? s1 : s2);
      g = unclipped ? -s1 : 0.f;  // d(-ratio*A)/d logp_new = -ratio*A
      if (beta > 0.f && logp_ref) {
        const float d = __fsub_rn(logp_ref[i], ln);
        const float e = exp_f(d);
        loss = __fmaf_rn(beta, __fsub_rn(__fsub_rn(e, d), 1.f), loss);
        g = __fmaf_rn(beta, __fsub_rn(1.f, e), g);
      }
      sum = __fadd_rn(sum, loss);
      cnt = __fadd_rn(cnt, 1.f);
      clipped = __fadd_rn(clipped, unclipped ? 0.f : 1.f);
    }
    raw_grad[i] = g;
  }
  const float ts = block_sum_fixed(sum, s_warp);
  const float tc = block_sum_fixed(cnt, s_warp);
  const float tk = block_sum_fixed(clipped, s_warp);
  if (threadIdx.x == 0) {
    seq_sum[seq] = ts;
    seq_cnt[seq] = tc;
    seq_clip[seq] = tk;
  }
}

// out[0] = loss, out[1] = clip fraction, out[2] = valid tokens; seq_w[g] = weight of a token
// of sequence g in the loss.
__global__ void grpo_finish_kernel(const float* __restrict__ seq_sum, const float* __restrict__ seq_cnt,
                                   const float* __restrict__ seq_clip, int n_seq, int seq_mean,
                                   float* __restrict__ seq_w, float* __restrict__ out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float total = 0.f, count = 0.f, clip = 0.f, mean_acc = 0.f, valid_seq = 0.f;
  for (int g = 0; g < n_seq; ++g) {
    total = __fadd_rn(total, seq_sum[g]);
    count = __fadd_rn(count, seq_cnt[g]);
    clip = __fadd_rn(clip, seq_clip[g]);
    if (seq_cnt[g] > 0.f) {
      mean_acc = __fadd_rn(mean_acc, __fdiv_rn(seq_sum[g], seq_cnt[g]));
      valid_seq = __fadd_rn(valid_seq, 1.f);
    }
  }
  if (seq_mean) {
    out[0] = valid_seq > 0.f ? __fdiv_rn(mean_acc, valid_seq) : 0.f;
    for (int g = 0; g < n_seq; ++g)
      seq_w[g] = seq_cnt[g] > 0.f ? __fdiv_rn(1.f, __fmul_rn(seq_cnt[g], valid_seq)) : 0.f;
  } else {
    out[0] = count > 0.f ? __fdiv_rn(total, count) : 0.f;
    const float w = count > 0.f ? __fdiv_rn(1.f, count) : 0.f;
    for (int g = 0; g < n_seq; ++g) seq_w[g] = w;
  }
  out[1] = count > 0.f ? __fdiv_rn(clip, count) : 0.f;
  out[2] = count;
}

__global__ void grpo_backward_kernel(const float* __restrict__ raw_grad, const float* __restrict__ seq_w,
                                     const float* __restrict__ upstream, float* __restrict__ grad, int seq_len,
                                     long long n) {
  const float up = upstream[0];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    grad[i] = __fmul_rn(__fmul_rn(raw_grad[i], seq_w[i / seq_len]), up);
}

}  // namespace
}  // namespace ka

extern "C" {

int ka_grpo_advantages(const float* rewards, float* adv, int n_groups, int group, float eps, void* stream) {
  if (n_groups <= 0) return 0;
  ka::advantages_kernel<<<(n_groups + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(rewards, adv, n_groups,
                                                                                             group, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// logp_*: [n_seq, seq_len] fp32; adv: [n_seq]; mask: [n_seq, seq_len] uint8 or null.
// raw_grad: [n_seq, seq_len]; seq_ws: 4 * n_seq floats of scratch (sum, count, clipped, weight);
// out: 3 floats (loss, clip fraction, valid tokens).
int ka_grpo_loss_fwd(const float* logp_new, const float* logp_old, const float* logp_ref, const float* adv,
                     const unsigned char* mask, int n_seq, int seq_len, float eps_low, float eps_high, float beta,
                     int seq_mean, float* raw_grad, float* seq_ws, float* out, void* stream) {
  if (n_seq <= 0 || seq_len <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ka::grpo_tokens_kernel<<<n_seq, ka::kThreads, 0, st>>>(logp_new, logp_old, logp_ref, adv, mask, seq_len, eps_low,
                                                         eps_high, beta, raw_grad, seq_ws, seq_ws + n_seq,
                                                         seq_ws + 2 * n_seq);
  ka::grpo_finish_kernel<<<1, 32, 0, st>>>(seq_ws, seq_ws + n_seq, seq_ws + 2 * n_seq, n_seq, seq_mean,
                                          seq_ws + 3 * n_seq, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int ka_grpo_loss_bwd(const float* raw_grad, const float* seq_w, const float* upstream, float* grad, int n_seq,
                     int seq_len, void* stream) {
  const long long n = static_cast<long long>(n_seq) * seq_len;
  if (n <= 0) return 0;
  const int blocks = static_cast<int>((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  ka::grpo_backward_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(raw_grad, seq_w, upstream, grad,
                                                                                 seq_len, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
