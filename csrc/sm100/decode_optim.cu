// Two small kernels of the RL loop.
//
//   attention_decode: one new query token per sequence against a KV cache (rollout phase).
//       One CTA per (sequence, query head); keys are visited in increasing order and the
//       reductions run in a fixed order, so the result does not depend on the batch.
//   adamw_step: fused AdamW update over a flat parameter group: bf16 parameter, fp32 master
//       copy, fp32 moments, fp32 or bf16 gradient, bias correction and decoupled weight decay.
//
// Neither exists in the reference (its executor comments defer generation to a future vLLM
// integration, rl_engine/executors/rollout.py:33).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "common/ptx.cuh"

namespace ka {
namespace {

constexpr int kD = 128;
constexpr int kDecThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

// q: [B, Hq, D]; cache_k / cache_v: [B, max_len, Hkv, D]; lens[b]: valid keys (incl. the new
// token); out: [B, Hq, D].
__global__ void __launch_bounds__(kDecThreads)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache_k,
                        const __nv_bfloat16* __restrict__ cache_v, const int* __restrict__ lens,
                        __nv_bfloat16* __restrict__ out, int hq, int hkv, int max_len, float scale) {
  extern __shared__ float s_scores[];  // [max_len]
  __shared__ float s_q[kD];
  __shared__ float s_red[kDecThreads / 32];
  const int b = blockIdx.x / hq, h = blockIdx.x % hq;
  const int hk = h / (hq / hkv);
  const int n = lens[b];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  s_q[tid] = __bfloat162float(q[(static_cast<size_t>(b) * hq + h) * kD + tid]);
  __syncthreads();
  const float c = scale * kLog2e;
  // scores: one warp per key, lanes split the head dimension
  float wmax = -CUDART_INF_F;
  for (int j = warp; j < n; j += kDecThreads / 32) {
    const __nv_bfloat16* kp = cache_k + ((static_cast<size_t>(b) * max_len + j) * hkv + hk) * kD;
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < kD / 32; ++t) acc = __fmaf_rn(s_q[lane + 32 * t], __bfloat162float(kp[lane + 32 * t]), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
    if (lane == 0) s_scores[j] = acc;
    wmax = fmaxf(wmax, acc);
  }
  if (lane == 0) s_red[warp] = wmax;
  __syncthreads();
  float m = s_red[0];
  for (int w = 1; w < kDecThreads / 32; ++w) m = fmaxf(m, s_red[w]);
  // probabilities; the normaliser is summed by one thread in key order
  for (int j = tid; j < n; j += kDecThreads) s_scores[j] = ex2_approx(__fmul_rn(__fsub_rn(s_scores[j], m), c));
  __syncthreads();
  // output: thread d owns one element of the head dimension, keys in order
  float acc = 0.f, l = 0.f;
  for (int j = 0; j < n; ++j) {
    const float p = s_scores[j];
    l = __fadd_rn(l, p);
    acc = __fmaf_rn(p, __bfloat162float(cache_v[((static_cast<size_t>(b) * max_len + j) * hkv + hk) * kD + tid]), acc);
  }
  out[(static_cast<size_t>(b) * hq + h) * kD + tid] = __float2bfloat16_rn(__fdiv_rn(acc, l));
}

template <typename G>
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ param, float* __restrict__ master, const G* __restrict__ grad,
                             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float beta1,
                             float beta2, float eps, float weight_decay, float bc1, float bc2, float grad_scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g;
    if constexpr (sizeof(G) == 2) g = __bfloat162float(grad[i]); else g = grad[i];
    g = __fmul_rn(g, grad_scale);
    const float mi = __fmaf_rn(beta1, m[i], __fmul_rn(1.f - beta1, g));
    const float vi = __fmaf_rn(beta2, v[i], __fmul_rn(1.f - beta2, __fmul_rn(g, g)));
    m[i] = mi;
    v[i] = vi;
    const float mh = __fdiv_rn(mi, bc1);
    const float vh = __fdiv_rn(vi, bc2);
    float w = master[i];
    w = __fsub_rn(w, __fmul_rn(lr, __fmul_rn(weight_decay, w)));
    w = __fsub_rn(w, __fmul_rn(lr, __fdiv_rn(mh, __fadd_rn(__fsqrt_rn(vh), eps))));
    master[i] = w;
    param[i] = __float2bfloat16_rn(w);
  }
}

}  // namespace
}  // namespace ka

extern "C" {

int ka_attention_decode(const void* q, const void* cache_k, const void* cache_v, const int* lens, void* out, int batch,
                        int hq, int hkv, int head_dim, int max_len, float scale, void* stream) {
  using namespace ka;
  if (batch <= 0) return 0;
  if (head_dim != kD || hq % hkv != 0 || max_len * 4 > 200 * 1024) return -1;
  static int configured_bytes = 0;
  const int smem = max_len * 4;
  if (smem > 48 * 1024 && smem > configured_bytes) {
    if (cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -10;
    configured_bytes = smem;
  }
  attention_decode_kernel<<<batch * hq, kDecThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(cache_k),
      static_cast<const __nv_bfloat16*>(cache_v), lens, static_cast<__nv_bfloat16*>(out), hq, hkv, max_len, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// step >= 1; grad_is_bf16 selects the gradient type; grad_scale multiplies the gradient first.
int ka_adamw_step(void* param, float* master, const void* grad, int grad_is_bf16, float* m, float* v, long long n,
                  float lr, float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                  int num_sms, void* stream) {
  using namespace ka;
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  long long blocks = (n + 255) / 256;
  if (blocks > static_cast<long long>(num_sms) * 16) blocks = static_cast<long long>(num_sms) * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<__nv_bfloat16*>(param), master, static_cast<const __nv_bfloat16*>(grad), m, v, n, lr, beta1, beta2,
        eps, weight_decay, bc1, bc2, grad_scale);
  else
    adamw_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(static_cast<__nv_bfloat16*>(param), master,
                                                                 static_cast<const float*>(grad), m, v, n, lr, beta1,
                                                                 beta2, eps, weight_decay, bc1, bc2, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
