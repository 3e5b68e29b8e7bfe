// Small kernels of the RL loop.
//
//   attention_decode: one new query token per sequence against a KV cache (rollout phase).
//       One CTA per (sequence, KV head): the query heads of a GQA group share every K / V
//       load. Scores: a warp per key, lanes over the head dimension. Output: the keys are cut
//       into four interleaved sets, each thread owns two output dimensions of one set, and the
//       four partial sums are added in a fixed order, so the result does not depend on the
//       batch. (Groups that are not 1, 2, 4 or 8 heads wide take the older one-CTA-per-head
//       kernel.)
//   decode_qkv_rope_cache: what lies between the fused qkv projection and attention in a decode
//       step, in one launch: split q / k / v, rotate q and k, write k and v into the cache slot.
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

// q: [B, Hq, D]; caches: [B, max_len, Hkv, D]; one CTA per (sequence, KV head), GQ = Hq / Hkv.
constexpr int kGqaThreads = 256;
constexpr int kKeySplits = 4;

template <int GQ>
__global__ void __launch_bounds__(kGqaThreads)
attention_decode_gqa_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache_k,
                            const __nv_bfloat16* __restrict__ cache_v, const int* __restrict__ lens,
                            __nv_bfloat16* __restrict__ out, int hq, int hkv, int max_len, float scale) {
  extern __shared__ float s_scores[];  // [GQ][max_len]
  __shared__ float s_q[GQ][kD];
  __shared__ float s_part[kKeySplits][GQ][kD];
  __shared__ float s_l[kKeySplits][GQ];
  __shared__ float s_max[kGqaThreads / 32][GQ];
  const int b = blockIdx.x / hkv, hk = blockIdx.x % hkv;
  const int n = lens[b];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t kv_row = static_cast<size_t>(hkv) * kD;  // elements between consecutive keys
  const __nv_bfloat16* kbase = cache_k + (static_cast<size_t>(b) * max_len * hkv + hk) * kD;
  const __nv_bfloat16* vbase = cache_v + (static_cast<size_t>(b) * max_len * hkv + hk) * kD;
  for (int i = tid; i < GQ * kD; i += kGqaThreads)
    s_q[i / kD][i % kD] = __bfloat162float(q[(static_cast<size_t>(b) * hq + hk * GQ + i / kD) * kD + i % kD]);
  __syncthreads();

  // ---- scores: warp w takes keys w, w + 8, ...; lane l holds dimensions 4l .. 4l + 3
  float qr[GQ][4], wmax[GQ];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    wmax[g] = -CUDART_INF_F;
#pragma unroll
    for (int e = 0; e < 4; ++e) qr[g][e] = s_q[g][4 * lane + e];
  }
#pragma unroll 4
  for (int j = warp; j < n; j += kGqaThreads / 32) {
    const uint2 raw = *reinterpret_cast<const uint2*>(kbase + j * kv_row + 4 * lane);
    const __nv_bfloat162 k01 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 k23 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float kf[4] = {__bfloat162float(k01.x), __bfloat162float(k01.y), __bfloat162float(k23.x),
                         __bfloat162float(k23.y)};
    float acc[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      float a = __fmul_rn(qr[g][0], kf[0]);
      a = __fmaf_rn(qr[g][1], kf[1], a);
      a = __fmaf_rn(qr[g][2], kf[2], a);
      a = __fmaf_rn(qr[g][3], kf[3], a);
      acc[g] = a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int g = 0; g < GQ; ++g) acc[g] = __fadd_rn(acc[g], __shfl_xor_sync(0xffffffffu, acc[g], o));
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < GQ; ++g) s_scores[g * max_len + j] = acc[g];
    }
#pragma unroll
    for (int g = 0; g < GQ; ++g) wmax[g] = fmaxf(wmax[g], acc[g]);
  }
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < GQ; ++g) s_max[warp][g] = wmax[g];
  }
  __syncthreads();
  const float c = scale * kLog2e;
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    float m = s_max[0][g];
#pragma unroll
    for (int w = 1; w < kGqaThreads / 32; ++w) m = fmaxf(m, s_max[w][g]);
    for (int j = tid; j < n; j += kGqaThreads)
      s_scores[g * max_len + j] = ex2_approx(__fmul_rn(__fsub_rn(s_scores[g * max_len + j], m), c));
  }
  __syncthreads();

  // ---- output: thread = (key set, dimension pair); a key set is j = set, set + 4, ...
  const int d2 = tid & 63, set = tid >> 6;
  float acc[GQ][2], l[GQ];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    acc[g][0] = 0.f;
    acc[g][1] = 0.f;
    l[g] = 0.f;
  }
#pragma unroll 8
  for (int j = set; j < n; j += kKeySplits) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(vbase + j * kv_row + 2 * d2);
    const float v0 = __bfloat162float(v.x), v1 = __bfloat162float(v.y);
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      const float p = s_scores[g * max_len + j];
      l[g] = __fadd_rn(l[g], p);
      acc[g][0] = __fmaf_rn(p, v0, acc[g][0]);
      acc[g][1] = __fmaf_rn(p, v1, acc[g][1]);
    }
  }
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    s_part[set][g][2 * d2] = acc[g][0];
    s_part[set][g][2 * d2 + 1] = acc[g][1];
    if (d2 == 0) s_l[set][g] = l[g];
  }
  __syncthreads();
  for (int i = tid; i < GQ * kD; i += kGqaThreads) {
    const int g = i / kD, d = i % kD;
    const float a = __fadd_rn(__fadd_rn(s_part[0][g][d], s_part[1][g][d]), __fadd_rn(s_part[2][g][d], s_part[3][g][d]));
    const float ls = __fadd_rn(__fadd_rn(s_l[0][g], s_l[1][g]), __fadd_rn(s_l[2][g], s_l[3][g]));
    out[(static_cast<size_t>(b) * hq + hk * GQ + g) * kD + d] = __float2bfloat16_rn(__fdiv_rn(a, ls));
  }
}

// qkv: [B, (hq + 2 hkv) * 128] bf16 (row stride qkv_stride), the output of the fused projection.
// pos [B]: position of the new token; slot [1]: cache row to write (both on the device, so a
// CUDA graph can replay the launch). q_out [B, hq, 128] rotated; cache_k / cache_v
// [B, max_len, hkv, 128]: row [b, slot] receives the rotated key and the value.
// The rotation is rope_kernel's arithmetic (elementwise.cu), so the bits are the same.
__global__ void __launch_bounds__(64)
decode_qkv_rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, long long qkv_stride,
                             const long long* __restrict__ pos, const long long* __restrict__ slot,
                             const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                             __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ cache_k,
                             __nv_bfloat16* __restrict__ cache_v, int hq, int hkv, int max_len) {
  constexpr int half = kD / 2;
  const int b = blockIdx.y, head = blockIdx.x, j = threadIdx.x;  // head in [0, hq + 2 hkv)
  const __nv_bfloat16* src = qkv + b * qkv_stride + static_cast<long long>(head) * kD;
  const long long s = slot[0];
  if (head < hq + hkv) {
    const long long p = pos[b];
    const float c = cos_t[p * half + j], sn = sin_t[p * half + j];
    const float a = __bfloat162float(src[j]), bb = __bfloat162float(src[j + half]);
    const __nv_bfloat16 lo = __float2bfloat16_rn(__fsub_rn(__fmul_rn(a, c), __fmul_rn(bb, sn)));
    const __nv_bfloat16 hi = __float2bfloat16_rn(__fadd_rn(__fmul_rn(bb, c), __fmul_rn(a, sn)));
    __nv_bfloat16* dst = head < hq ? q_out + (static_cast<long long>(b) * hq + head) * kD
                                   : cache_k + ((static_cast<long long>(b) * max_len + s) * hkv + (head - hq)) * kD;
    dst[j] = lo;
    dst[j + half] = hi;
  } else {
    __nv_bfloat16* dst = cache_v + ((static_cast<long long>(b) * max_len + s) * hkv + (head - hq - hkv)) * kD;
    dst[j] = src[j];
    dst[j + half] = src[j + half];
  }
}

// One element of the update (shared by the scalar and the 4-wide kernel: same bits).
__device__ __forceinline__ float adamw_one(float g, float& m, float& v, float& w, float lr, float beta1, float beta2,
                                           float eps, float weight_decay, float bc1, float bc2, float grad_scale) {
  g = __fmul_rn(g, grad_scale);
  m = __fmaf_rn(beta1, m, __fmul_rn(1.f - beta1, g));
  v = __fmaf_rn(beta2, v, __fmul_rn(1.f - beta2, __fmul_rn(g, g)));
  const float mh = __fdiv_rn(m, bc1);
  const float vh = __fdiv_rn(v, bc2);
  w = __fsub_rn(w, __fmul_rn(lr, __fmul_rn(weight_decay, w)));
  w = __fsub_rn(w, __fmul_rn(lr, __fdiv_rn(mh, __fadd_rn(__fsqrt_rn(vh), eps))));
  return w;
}

// Four elements per thread with 16-byte (fp32) / 8-byte (bf16) accesses; elements past the last
// multiple of four are handled one by one by the first threads.
template <typename G>
__global__ void __launch_bounds__(256)
adamw_kernel(__nv_bfloat16* __restrict__ param, float* __restrict__ master, const G* __restrict__ grad,
             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float beta1, float beta2, float eps,
             float weight_decay, float bc1, float bc2, float grad_scale) {
  const long long n4 = n / 4;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = tid; i < n4; i += stride) {
    float g[4];
    if constexpr (sizeof(G) == 2) {
      const uint2 raw = reinterpret_cast<const uint2*>(grad)[i];
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      g[0] = __bfloat162float(a.x); g[1] = __bfloat162float(a.y); g[2] = __bfloat162float(b.x); g[3] = __bfloat162float(b.y);
    } else {
      const float4 t = reinterpret_cast<const float4*>(grad)[i];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    }
    float4 m4 = reinterpret_cast<float4*>(m)[i], v4 = reinterpret_cast<float4*>(v)[i];
    float4 w4 = reinterpret_cast<float4*>(master)[i];
    adamw_one(g[0], m4.x, v4.x, w4.x, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
    adamw_one(g[1], m4.y, v4.y, w4.y, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
    adamw_one(g[2], m4.z, v4.z, w4.z, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
    adamw_one(g[3], m4.w, v4.w, w4.w, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    reinterpret_cast<float4*>(master)[i] = w4;
    const __nv_bfloat162 o0 = __floats2bfloat162_rn(w4.x, w4.y), o1 = __floats2bfloat162_rn(w4.z, w4.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&o0);
    o.y = *reinterpret_cast<const uint32_t*>(&o1);
    reinterpret_cast<uint2*>(param)[i] = o;
  }
  for (long long i = n4 * 4 + tid; i < n; i += stride) {
    float g;
    if constexpr (sizeof(G) == 2) g = __bfloat162float(grad[i]); else g = grad[i];
    float mi = m[i], vi = v[i], w = master[i];
    adamw_one(g, mi, vi, w, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
    m[i] = mi;
    v[i] = vi;
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
  const int gq = hq / hkv;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((gq == 1 || gq == 2 || gq == 4 || gq == 8) && static_cast<long long>(gq) * max_len * 4 <= 160 * 1024) {
    const int smem_g = gq * max_len * 4;
    const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
    const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(cache_k);
    const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(cache_v);
    __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(out);
    // the shared-memory opt-in is per device and cheap: set it on every call that needs it
#define KA_LAUNCH_GQA(GQ)                                                                                       \
  do {                                                                                                          \
    if (smem_g > 40 * 1024 &&                                                                                   \
        cudaFuncSetAttribute(attention_decode_gqa_kernel<GQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                             smem_g) != cudaSuccess)                                                            \
      return -10;                                                                                               \
    attention_decode_gqa_kernel<GQ><<<batch * hkv, kGqaThreads, smem_g, st>>>(qb, kb, vb, lens, ob, hq, hkv,    \
                                                                               max_len, scale);                 \
  } while (0)
    if (gq == 1) KA_LAUNCH_GQA(1);
    else if (gq == 2) KA_LAUNCH_GQA(2);
    else if (gq == 4) KA_LAUNCH_GQA(4);
    else KA_LAUNCH_GQA(8);
#undef KA_LAUNCH_GQA
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
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

// See decode_qkv_rope_cache_kernel. head_dim is 128.
int ka_decode_qkv_rope_cache(const void* qkv, long long qkv_stride, const long long* pos, const long long* slot,
                             const float* cos_t, const float* sin_t, void* q_out, void* cache_k, void* cache_v,
                             int batch, int hq, int hkv, int max_len, void* stream) {
  using namespace ka;
  if (batch <= 0) return 0;
  dim3 grid(static_cast<unsigned>(hq + 2 * hkv), static_cast<unsigned>(batch));
  decode_qkv_rope_cache_kernel<<<grid, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), qkv_stride, pos, slot, cos_t, sin_t, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(cache_k), static_cast<__nv_bfloat16*>(cache_v), hq, hkv, max_len);
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
  long long blocks = (n / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
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
