// Memory-bound layer ops of the decoder, each a single pass with 16-byte accesses and fp32
// math: RMSNorm (with optional fused residual add), rotary embedding, SwiGLU.
// Every reduction runs in a fixed order inside one CTA, so a row's output depends on that row
// only (batch invariance). None of these exists in the reference, which only names them
// (rl_engine/platforms/constants.py:75-80, README feature list).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common/ptx.cuh"

namespace ka {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

struct alignas(16) Bf16x8 {
  __nv_bfloat16 v[8];
};

__device__ __forceinline__ float block_sum_fixed(float v, float* s_warp, int n_warps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (lane == 0) s_warp[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < n_warps; ++w) t = __fadd_rn(t, s_warp[w]);  // same order in every thread
  __syncthreads();
  return t;
}

// y = (x [+ residual]) * rsqrt(mean(x^2) + eps) * w ; if residual_out: residual_out = x + residual
// One CTA per row, D % 8 == 0.
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
               __nv_bfloat16* __restrict__ residual_out, int rows, int d, float eps) {
  __shared__ float s_warp[8];
  const int nvec = d / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const Bf16x8* xp = reinterpret_cast<const Bf16x8*>(x + static_cast<size_t>(row) * d);
    const Bf16x8* rp = residual ? reinterpret_cast<const Bf16x8*>(residual + static_cast<size_t>(row) * d) : nullptr;
    Bf16x8* ro = residual_out ? reinterpret_cast<Bf16x8*>(residual_out + static_cast<size_t>(row) * d) : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Bf16x8 a = xp[i];
      if (rp) {
        const Bf16x8 b = rp[i];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          a.v[j] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(a.v[j]), __bfloat162float(b.v[j])));
        if (ro) ro[i] = a;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = __bfloat162float(a.v[j]);
        ss = __fmaf_rn(f, f, ss);
      }
    }
    const float total = block_sum_fixed(ss, s_warp, blockDim.x >> 5);
    const float inv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(d)), eps)));
    const Bf16x8* wp = reinterpret_cast<const Bf16x8*>(w);
    Bf16x8* yp = reinterpret_cast<Bf16x8*>(y + static_cast<size_t>(row) * d);
    const Bf16x8* src = (rp && ro) ? reinterpret_cast<const Bf16x8*>(ro) : xp;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Bf16x8 a = src[i];
      if (rp && !ro) {
        const Bf16x8 b = rp[i];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          a.v[j] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(a.v[j]), __bfloat162float(b.v[j])));
      }
      const Bf16x8 ww = wp[i];
      Bf16x8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float n = __fmul_rn(__bfloat162float(a.v[j]), inv);
        // round the normalised value to bf16 before the weight, as the usual bf16 module does
        o.v[j] = __float2bfloat16_rn(__fmul_rn(__bfloat162float(__float2bfloat16_rn(n)), __bfloat162float(ww.v[j])));
      }
      yp[i] = o;
    }
  }
}

// Rotary embedding, "rotate half" convention: for i < hd/2
//   out[i]        = x[i] * cos[pos, i] - x[i + hd/2] * sin[pos, i]
//   out[i + hd/2] = x[i + hd/2] * cos[pos, i] + x[i] * sin[pos, i]
// x: [tokens, heads, hd] (token stride given), cos/sin: [max_pos, hd/2] fp32, in place.
__global__ void __launch_bounds__(256)
rope_kernel(__nv_bfloat16* __restrict__ x, long long token_stride, const long long* __restrict__ positions,
            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int tokens, int heads, int hd) {
  const int half = hd / 2;
  const long long total = static_cast<long long>(tokens) * heads * half;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i % half);
    const long long th = i / half;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const long long pos = positions[t];
    const float c = cos_t[pos * half + j], s = sin_t[pos * half + j];
    __nv_bfloat16* p = x + t * token_stride + static_cast<long long>(h) * hd;
    const float a = __bfloat162float(p[j]), b = __bfloat162float(p[j + half]);
    p[j] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
    p[j + half] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
  }
}

// The same rotation with 16-byte accesses: a thread takes eight consecutive pairs (j .. j + 7 and
// their partners in the second half). hd / 2 must be a multiple of 8, rows 16-byte aligned.
__global__ void __launch_bounds__(256)
rope_vec8_kernel(__nv_bfloat16* __restrict__ x, long long token_stride, const long long* __restrict__ positions,
                 const float* __restrict__ cos_t, const float* __restrict__ sin_t, int tokens, int heads, int hd) {
  const int half = hd / 2, groups = half / 8;
  const long long total = static_cast<long long>(tokens) * heads * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i % groups) * 8;
    const long long th = i / groups;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const long long pos = positions[t];
    const float4* cp = reinterpret_cast<const float4*>(cos_t + pos * half + j);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + pos * half + j);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    __nv_bfloat16* p = x + t * token_stride + static_cast<long long>(h) * hd;
    Bf16x8 lo = *reinterpret_cast<const Bf16x8*>(p + j), hi = *reinterpret_cast<const Bf16x8*>(p + j + half);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = __bfloat162float(lo.v[e]), b = __bfloat162float(hi.v[e]);
      lo.v[e] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(a, c[e]), __fmul_rn(b, sn[e])));
      hi.v[e] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(b, c[e]), __fmul_rn(a, sn[e])));
    }
    *reinterpret_cast<Bf16x8*>(p + j) = lo;
    *reinterpret_cast<Bf16x8*>(p + j + half) = hi;
  }
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float silu_f(float g) {
  // g * sigmoid(g) = g * (0.5 + 0.5 * tanh(g / 2)): one special-function op per element
  // (the result is rounded to bf16, tanh.approx is accurate to about 2^-11)
  return __fmul_rn(g, __fmaf_rn(0.5f, tanh_approx(__fmul_rn(0.5f, g)), 0.5f));
}

// out[r, j] = silu(gate[r, j]) * up[r, j]; gate/up are column halves of one [rows, 2f] tensor
// when up == gate + f (row stride 2f), or separate tensors.
__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, long long in_stride,
              __nv_bfloat16* __restrict__ out, int rows, int f) {
  const int nvec = f / 8;
  const long long total = static_cast<long long>(rows) * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nvec;
    const int c = static_cast<int>(i % nvec);
    const Bf16x8 g = reinterpret_cast<const Bf16x8*>(gate + r * in_stride)[c];
    const Bf16x8 u = reinterpret_cast<const Bf16x8*>(up + r * in_stride)[c];
    Bf16x8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = __bfloat162float(__float2bfloat16_rn(silu_f(__bfloat162float(g.v[j]))));
      o.v[j] = __float2bfloat16_rn(__fmul_rn(a, __bfloat162float(u.v[j])));
    }
    reinterpret_cast<Bf16x8*>(out + r * static_cast<long long>(f))[c] = o;
  }
}

// Backward of SwiGLU: d_gate = d_out * up * (sig + g*sig*(1-sig)), d_up = d_out * silu(g).
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, long long in_stride,
                  const __nv_bfloat16* __restrict__ d_out, __nv_bfloat16* __restrict__ d_gate,
                  __nv_bfloat16* __restrict__ d_up, long long dgrad_stride, int rows, int f) {
  const int nvec = f / 8;
  const long long total = static_cast<long long>(rows) * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nvec;
    const int c = static_cast<int>(i % nvec);
    const Bf16x8 g = reinterpret_cast<const Bf16x8*>(gate + r * in_stride)[c];
    const Bf16x8 u = reinterpret_cast<const Bf16x8*>(up + r * in_stride)[c];
    const Bf16x8 d = reinterpret_cast<const Bf16x8*>(d_out + r * static_cast<long long>(f))[c];
    Bf16x8 dg, du;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gf = __bfloat162float(g.v[j]), uf = __bfloat162float(u.v[j]), df = __bfloat162float(d.v[j]);
      const float sig = __fdiv_rn(1.f, __fadd_rn(1.f, ex2_approx(__fmul_rn(-gf, kLog2e))));
      const float dsilu = __fmaf_rn(__fmul_rn(gf, sig), __fsub_rn(1.f, sig), sig);
      dg.v[j] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(df, uf), dsilu));
      du.v[j] = __float2bfloat16_rn(__fmul_rn(df, __fmul_rn(gf, sig)));
    }
    reinterpret_cast<Bf16x8*>(d_gate + r * dgrad_stride)[c] = dg;
    reinterpret_cast<Bf16x8*>(d_up + r * dgrad_stride)[c] = du;
  }
}

// Backward of y = bf16(bf16(x * inv) * w).
//   dx = inv * (dy*w - n * mean(dy*w*n)),  n = x * inv;   dw_partial[chunk] = sum_rows dy * n
// One CTA per chunk of kRmsChunk rows (fixed, so the order in which rows enter d_w does not
// depend on the grid); threads own columns. kRows rows are in flight at once: their x and dy
// vectors are loaded once into registers and serve all three steps (sum of squares, the dot
// product, dx / dw), and the block reductions of the kRows rows share their two barriers.
constexpr int kRmsChunk = 64;

// Fixed-order sums of R values per thread over the CTA (8 warps): lanes by xor-shuffle, then the
// eight warp sums left to right, the same in every thread.
template <int R>
__device__ __forceinline__ void block_sum_fixed_multi(float (&v)[R], float (*s_warp)[8]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[r] = __fadd_rn(v[r], __shfl_xor_sync(0xffffffffu, v[r], o));
    if (lane == 0) s_warp[r][warp] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t = __fadd_rn(t, s_warp[r][w]);
    v[r] = t;
  }
  __syncthreads();
}

// VPT: 16-byte vectors per thread and row (d <= 2048 * VPT); kRows: rows in flight.
template <int VPT, int kRows>
__global__ void __launch_bounds__(256, 2)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                   int rows, int d, float eps) {
  __shared__ float s_warp[kRows][8];
  const int chunk = blockIdx.x;
  const int r0 = chunk * kRmsChunk, r1 = min(rows, r0 + kRmsChunk);
  const int nvec = d / 8;
  float dw_acc[VPT][8];
#pragma unroll
  for (int a = 0; a < VPT; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[a][j] = 0.f;
  const Bf16x8* wp = reinterpret_cast<const Bf16x8*>(w);  // re-read per use: it stays in L1
  for (int row0 = r0; row0 < r1; row0 += kRows) {
    Bf16x8 xv[kRows][VPT], gv[kRows][VPT];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int row = row0 + r;
#pragma unroll
      for (int a = 0; a < VPT; ++a) {
        const int i = threadIdx.x + a * 256;
        if (row < r1 && i < nvec) {
          xv[r][a] = reinterpret_cast<const Bf16x8*>(x + static_cast<size_t>(row) * d)[i];
          gv[r][a] = reinterpret_cast<const Bf16x8*>(dy + static_cast<size_t>(row) * d)[i];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            xv[r][a].v[j] = __float2bfloat16_rn(0.f);
            gv[r][a].v[j] = __float2bfloat16_rn(0.f);
          }
        }
      }
    }
    float red[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      float ss = 0.f;
#pragma unroll
      for (int a = 0; a < VPT; ++a)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float f = __bfloat162float(xv[r][a].v[j]);
          ss = __fmaf_rn(f, f, ss);
        }
      red[r] = ss;
    }
    block_sum_fixed_multi<kRows>(red, s_warp);
    float inv[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      inv[r] = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(red[r], static_cast<float>(d)), eps)));
      float dot = 0.f;
#pragma unroll
      for (int a = 0; a < VPT; ++a) {
        const int i = threadIdx.x + a * 256;
        if (i >= nvec) continue;
        const Bf16x8 wv = wp[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = __fmul_rn(__bfloat162float(xv[r][a].v[j]), inv[r]);
          dot = __fmaf_rn(__fmul_rn(__bfloat162float(gv[r][a].v[j]), __bfloat162float(wv.v[j])), n, dot);
        }
      }
      red[r] = dot;
    }
    block_sum_fixed_multi<kRows>(red, s_warp);
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int row = row0 + r;
      if (row >= r1) break;  // uniform over the CTA
      const float mean_dot = __fdiv_rn(red[r], static_cast<float>(d));
#pragma unroll
      for (int a = 0; a < VPT; ++a) {
        const int i = threadIdx.x + a * 256;
        if (i >= nvec) continue;
        const Bf16x8 wv = wp[i];
        Bf16x8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = __fmul_rn(__bfloat162float(xv[r][a].v[j]), inv[r]);
          const float g = __bfloat162float(gv[r][a].v[j]);
          const float gw = __fmul_rn(g, __bfloat162float(wv.v[j]));
          o.v[j] = __float2bfloat16_rn(__fmul_rn(inv[r], __fsub_rn(gw, __fmul_rn(n, mean_dot))));
          dw_acc[a][j] = __fmaf_rn(g, n, dw_acc[a][j]);  // rows enter in increasing order
        }
        reinterpret_cast<Bf16x8*>(dx + static_cast<size_t>(row) * d)[i] = o;
      }
    }
  }
#pragma unroll
  for (int a = 0; a < VPT; ++a) {
    const int i = threadIdx.x + a * 256;
    if (i >= nvec) continue;
    float4* dst = reinterpret_cast<float4*>(dw_part + static_cast<size_t>(chunk) * d + i * 8);
    dst[0] = make_float4(dw_acc[a][0], dw_acc[a][1], dw_acc[a][2], dw_acc[a][3]);
    dst[1] = make_float4(dw_acc[a][4], dw_acc[a][5], dw_acc[a][6], dw_acc[a][7]);
  }
}

// d_w[c] = sum over chunks (in index order) of dw_part[chunk][c]
__global__ void rmsnorm_dw_kernel(const float* __restrict__ dw_part, __nv_bfloat16* __restrict__ dw, int chunks, int d) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float acc = 0.f;
  for (int k = 0; k < chunks; ++k) acc = __fadd_rn(acc, dw_part[static_cast<size_t>(k) * d + c]);
  dw[c] = __float2bfloat16_rn(acc);
}

int grid_for(long long work_items, int threads, int num_sms) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(num_sms) * 8;
  if (g > cap) g = cap;
  return g < 1 ? 1 : static_cast<int>(g);
}

}  // namespace
}  // namespace ka

extern "C" {

int ka_rmsnorm(const void* x, const void* residual, const void* w, void* y, void* residual_out, int rows, int d,
               float eps, int num_sms, void* stream) {
  using namespace ka;
  if (rows <= 0) return 0;
  if (d % 8 != 0) return -1;
  const int grid = rows < num_sms * 8 ? rows : num_sms * 8;
  rmsnorm_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(residual_out),
      rows, d, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int ka_rope(void* x, long long token_stride, const long long* positions, const float* cos_t, const float* sin_t,
            int tokens, int heads, int hd, int num_sms, void* stream) {
  using namespace ka;
  if (tokens <= 0) return 0;
  if (hd % 2 != 0) return -1;
  if ((hd / 2) % 8 == 0 && token_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    const long long groups = static_cast<long long>(tokens) * heads * (hd / 16);
    rope_vec8_kernel<<<grid_for(groups, 256, num_sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(x), token_stride, positions, cos_t, sin_t, tokens, heads, hd);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  const long long total = static_cast<long long>(tokens) * heads * (hd / 2);
  rope_kernel<<<grid_for(total, 256, num_sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), token_stride, positions, cos_t, sin_t, tokens, heads, hd);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int ka_swiglu(const void* gate, const void* up, long long in_stride, void* out, int rows, int f, int num_sms,
              void* stream) {
  using namespace ka;
  if (rows <= 0) return 0;
  if (f % 8 != 0 || in_stride % 8 != 0) return -1;
  const long long total = static_cast<long long>(rows) * (f / 8);
  swiglu_kernel<<<grid_for(total, 256, num_sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), in_stride,
      static_cast<__nv_bfloat16*>(out), rows, f);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int ka_swiglu_bwd(const void* gate, const void* up, long long in_stride, const void* d_out, void* d_gate, void* d_up,
                  long long dgrad_stride, int rows, int f, int num_sms, void* stream) {
  using namespace ka;
  if (rows <= 0) return 0;
  if (f % 8 != 0 || in_stride % 8 != 0 || dgrad_stride % 8 != 0) return -1;
  const long long total = static_cast<long long>(rows) * (f / 8);
  swiglu_bwd_kernel<<<grid_for(total, 256, num_sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), in_stride,
      static_cast<const __nv_bfloat16*>(d_out), static_cast<__nv_bfloat16*>(d_gate), static_cast<__nv_bfloat16*>(d_up),
      dgrad_stride, rows, f);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Rows per partial sum of the weight gradient (the size of dw_part follows from it).
int ka_rmsnorm_bwd_chunk() { return ka::kRmsChunk; }

// x, dy: [rows, d] bf16; dx: [rows, d] bf16; dw: [d] bf16; dw_part: scratch of
// ceil(rows / ka_rmsnorm_bwd_chunk()) * d floats. d % 8 == 0 and d <= 8192.
int ka_rmsnorm_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw, float* dw_part, int rows, int d,
                   float eps, void* stream) {
  using namespace ka;
  if (rows <= 0) return 0;
  if (d % 8 != 0 || d > 8192) return -1;
  const int chunks = (rows + kRmsChunk - 1) / kRmsChunk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wb = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* gb = static_cast<const __nv_bfloat16*>(dy);
  __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(dx);
  const int vpt = (d / 8 + 255) / 256;
  if (vpt <= 1)
    rmsnorm_bwd_kernel<1, 4><<<chunks, 256, 0, st>>>(xb, wb, gb, ob, dw_part, rows, d, eps);
  else if (vpt == 2)
    rmsnorm_bwd_kernel<2, 2><<<chunks, 256, 0, st>>>(xb, wb, gb, ob, dw_part, rows, d, eps);
  else
    rmsnorm_bwd_kernel<4, 1><<<chunks, 256, 0, st>>>(xb, wb, gb, ob, dw_part, rows, d, eps);
  rmsnorm_dw_kernel<<<(d + 255) / 256, 256, 0, st>>>(dw_part, static_cast<__nv_bfloat16*>(dw), chunks, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
