// Per-token log-probability from materialised logits, one pass, no temporaries.
//
//   logp[r] = scale * logits[r, ids[r]] - logsumexp_v(scale * logits[r, v])
//
// This is the operation the reference implements as chunked `log_softmax(...).gather(...)`
// (rl_engine/kernels/sampling.py:91-112), which writes and re-reads a [chunk, V] temporary.
// Here one CTA streams a row once with 16-byte loads and keeps an online (max, sum-exp) per
// thread; the per-thread states are merged in a fixed butterfly order, so a row's result
// does not depend on how many rows are in the call.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "common/ptx.cuh"
#include "sampling.h"

namespace ka {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static constexpr int kVec = 4;
  __device__ static float f(float v) { return v; }
};
template <>
struct Cvt<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static float f(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <>
struct Cvt<__half> {
  static constexpr int kVec = 8;
  __device__ static float f(__half v) { return __half2float(v); }
};

// state: sum_j 2^(x_j*s2 - R) with R = round(m*s2)
__device__ __forceinline__ void fold_vec(const float* x, int n, float s2, float& m, float& l) {
  float mx = x[0];
#pragma unroll
  for (int j = 1; j < 8; ++j)
    if (j < n) mx = fmaxf(mx, x[j]);
  const float mn = fmaxf(m, mx);
  const float neg_old = __fmul_rn(-m, s2);
  const float neg = __fmul_rn(-mn, s2);
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (j < n) acc = __fadd_rn(acc, ex2_approx(__fmaf_rn(x[j], s2, neg)));
  l = __fmaf_rn(l, ex2_approx(__fsub_rn(neg, neg_old)), acc);
  m = mn;
}

__device__ __forceinline__ void merge_state(float& m, float& l, float m2, float l2, float s2) {
  const float mn = fmaxf(m, m2);
  const float a = (m == -CUDART_INF_F) ? 0.f : ex2_approx(__fsub_rn(__fmul_rn(-mn, s2), __fmul_rn(-m, s2)));
  const float b = (m2 == -CUDART_INF_F) ? 0.f : ex2_approx(__fsub_rn(__fmul_rn(-mn, s2), __fmul_rn(-m2, s2)));
  l = __fadd_rn(__fmul_rn(l, a), __fmul_rn(l2, b));
  m = mn;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
logits_logp_kernel(const T* __restrict__ logits, long long row_stride, int v, const long long* __restrict__ ids,
                   float scale, float* __restrict__ logp, float* __restrict__ lse, int rows) {
  __shared__ float s_m[kWarps], s_l[kWarps];
  constexpr int kVec = Cvt<T>::kVec;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float s2 = scale * kLog2e;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* rp = logits + static_cast<long long>(row) * row_stride;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(rp) & 15u) == 0;
    float m = -CUDART_INF_F, l = 0.f;
    float x[8];
    if (vec_ok) {
      const int nvec = v / kVec;
      const uint4* p = reinterpret_cast<const uint4*>(rp);
      for (int i = tid; i < nvec; i += kThreads) {
        const uint4 raw = __ldcs(p + i);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < kVec; ++j) x[j] = Cvt<T>::f(e[j]);
        fold_vec(x, kVec, s2, m, l);
      }
      for (int i = nvec * kVec + tid; i < v; i += kThreads) {
        x[0] = Cvt<T>::f(rp[i]);
        fold_vec(x, 1, s2, m, l);
      }
    } else {
      for (int i = tid; i < v; i += kThreads) {
        x[0] = Cvt<T>::f(rp[i]);
        fold_vec(x, 1, s2, m, l);
      }
    }
    // NOTE: the per-thread element assignment differs between the vector and scalar paths;
    // rows of one tensor share alignment whenever V * sizeof(T) is a multiple of 16.
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
      // both partners must compute the same value: order the pair by lane
      float ma = (lane & o) ? m2 : m, la = (lane & o) ? l2 : l;
      const float mb = (lane & o) ? m : m2, lb = (lane & o) ? l : l2;
      merge_state(ma, la, mb, lb, s2);
      m = ma;
      l = la;
    }
    if (lane == 0) {
      s_m[warp] = m;
      s_l[warp] = l;
    }
    __syncthreads();
    if (tid == 0) {
      float mm = s_m[0], ll = s_l[0];
      for (int w = 1; w < kWarps; ++w) merge_state(mm, ll, s_m[w], s_l[w], s2);
      const float out_lse = __fmaf_rn(lg2_approx(ll), kLn2, __fmul_rn(mm, scale));
      if (lse) lse[row] = out_lse;
      const long long id = ids[row];
      float r = 0.f;
      if (id >= 0 && id < v) r = __fsub_rn(__fmul_rn(Cvt<T>::f(rp[id]), scale), out_lse);
      logp[row] = r;
    }
    __syncthreads();
  }
}

template <typename T>
int launch(const void* logits, long long row_stride, int rows, int v, const long long* ids, float scale, float* logp,
           float* lse, int num_sms, cudaStream_t st) {
  int grid = rows < num_sms * 4 ? rows : num_sms * 4;
  logits_logp_kernel<T><<<grid, kThreads, 0, st>>>(static_cast<const T*>(logits), row_stride, v, ids, scale, logp, lse,
                                                   rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace
}  // namespace ka

// logits: [rows, vocab] with `row_stride` elements between rows; ids: [rows] int64 (ids
// outside [0, vocab) give 0); logp / lse: [rows] fp32 (lse may be null). scale > 0.
extern "C" int ka_logits_logp(const void* logits, int dtype, long long row_stride, int rows, int vocab,
                              const long long* ids, float scale, float* logp, float* lse, int num_sms,
                              void* stream) {
  using namespace ka;
  if (rows <= 0) return 0;
  if (vocab <= 0 || !(scale > 0.f)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case KA_DTYPE_F32:
      return launch<float>(logits, row_stride, rows, vocab, ids, scale, logp, lse, num_sms, st);
    case KA_DTYPE_BF16:
      return launch<__nv_bfloat16>(logits, row_stride, rows, vocab, ids, scale, logp, lse, num_sms, st);
    case KA_DTYPE_F16:
      return launch<__half>(logits, row_stride, rows, vocab, ids, scale, logp, lse, num_sms, st);
    default:
      return -2;
  }
}
