// Attention backward for sm_100a (causal / full, GQA, head_dim 128), deterministic: no atomics.
//
//   delta[b, h, i] = sum_d dO[i, d] * O[i, d]
//   P  = exp(scale * Q K^T - lse),   dP = dO V^T,   dS = P * (dP - delta) * scale
//   dQ = dS K            kernel attention_bwd_dq_kernel : one CTA per (sequence, q head, q tile),
//                        walks the KV tiles in increasing order, dQ accumulates in TMEM
//   dV = P^T dO, dK = dS^T Q   kernel attention_bwd_dkv_kernel: one CTA per (sequence, kv head,
//                        kv tile), walks (q head of the group, q tile) in a fixed order; it
//                        works on S^T = K Q^T so that its threads own KV rows
//
// All five products are tcgen05.mma 128 x 128 tiles; operands that are needed "transposed"
// (K and Q as [d, rows], dO as [d, rows]) are read through MN-major descriptors from the same
// TMA tiles, so nothing is transposed in memory. Every accumulation order is fixed, so the
// gradients are bitwise reproducible and independent of the batch.
//
// The reference has no attention kernel and no backward pass of any kind: it routes the op
// type "attention" to a backend name (rl_engine/kernels/registry.py:41-55).
#include <cstdint>
#include <cuda_bf16.h>
#include <math_constants.h>

#include "common/bounded_wait.cuh"
#include "common/ptx.cuh"
#include "common/tmap.cuh"
#include "attention_common.cuh"

namespace ka {
namespace {

constexpr int kD = 128;
constexpr int kT = 128;                    // tile rows (queries or keys)
constexpr int kSoftThreads = 256;          // 8 warps: two threads per TMEM lane (64 columns each)
constexpr int kThreads = kSoftThreads + 64;  // + TMA warp + MMA warp
constexpr int kWarpTma = kSoftThreads / 32, kWarpMma = kSoftThreads / 32 + 1;
constexpr int kTileBytes = 128 * 128 * 2;
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  const float* lse;     // [B, Hq, L]
  const float* delta;   // [B, Hq, L]
  __nv_bfloat16* dq;    // [B*L, Hq*128], token stride dq_stride
  __nv_bfloat16* dk;    // [B*L, Hkv*128]
  __nv_bfloat16* dv;
  long long dq_stride, dk_stride, dv_stride;
  int batch, seq_len, hq, hkv;
  float scale;
  int causal;
  int* status;
  unsigned long long timeout_ns;
};

// delta[b, h, i] = sum_d dO * O (fp32), one warp per (token, head)
__global__ void attention_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_stride,
                                       const __nv_bfloat16* __restrict__ d_o, long long do_stride,
                                       float* __restrict__ delta, int batch, int seq_len, int hq) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(batch) * seq_len * hq;
  if (w >= total) return;
  const int h = static_cast<int>(w % hq);
  const long long tok = w / hq;
  const uint2 a = *reinterpret_cast<const uint2*>(o + tok * o_stride + h * kD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(d_o + tok * do_stride + h * kD + lane * 4);
  float acc = 0.f;
  acc = __fmaf_rn(__uint_as_float(a.x << 16), __uint_as_float(b.x << 16), acc);
  acc = __fmaf_rn(__uint_as_float(a.x & 0xFFFF0000u), __uint_as_float(b.x & 0xFFFF0000u), acc);
  acc = __fmaf_rn(__uint_as_float(a.y << 16), __uint_as_float(b.y << 16), acc);
  acc = __fmaf_rn(__uint_as_float(a.y & 0xFFFF0000u), __uint_as_float(b.y & 0xFFFF0000u), acc);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
  if (lane == 0) {
    const int b_ = static_cast<int>(tok / seq_len), i = static_cast<int>(tok % seq_len);
    delta[(static_cast<long long>(b_) * hq + h) * seq_len + i] = acc;
  }
}

struct CtlDq {
  uint64_t qdo_full;      // Q and dO tiles loaded
  uint64_t kv_full, kv_empty;
  uint64_t s_full;        // S and dP ready in TMEM
  uint64_t ds_full;       // dS tile written (count: softmax warps)
  uint64_t acc_full;      // final dQ ready
  uint32_t tmem_base;
  int abort_flag;
};

// ------------------------------------------------------------------------------------------------
// dQ kernel
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1)
attention_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                        const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t q_tile = base, do_tile = base + kTileBytes, k_tile = base + 2 * kTileBytes,
                 v_tile = base + 3 * kTileBytes, ds_tile = base + 4 * kTileBytes;
  uint8_t* ds_ptr = smem + 4 * kTileBytes;
  CtlDq* ctl = reinterpret_cast<CtlDq*>(smem + 5 * kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.seq_len + kT - 1) / kT;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x % n_qt);
  const int bh = blockIdx.x / n_qt;
  const int h = bh % p.hq, b = bh / p.hq;
  const int hk = h / (p.hq / p.hkv);
  const int q_row0 = qt * kT, tok0 = b * p.seq_len;
  const int kv_end = p.causal ? min(p.seq_len, q_row0 + kT) : p.seq_len;
  const int n_kv = (kv_end + kT - 1) / kT;
  WaitCtx wctx{&ctl->abort_flag, p.status, p.timeout_ns};

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl->qdo_full), 1);
    mbar_init(smem_u32(&ctl->kv_full), 1);
    mbar_init(smem_u32(&ctl->kv_empty), 1);
    mbar_init(smem_u32(&ctl->s_full), 1);
    mbar_init(smem_u32(&ctl->ds_full), kSoftThreads / 32);
    mbar_init(smem_u32(&ctl->acc_full), 1);
    ctl->abort_flag = 0;
    fence_mbar_init_cluster();
  }
  if (warp == kWarpMma) {
    tmem_alloc<1>(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 128, tmem_dq = tmem_base + 256;

  if (warp == kWarpTma) {
    if (lane == 0) {
      const uint32_t f = smem_u32(&ctl->qdo_full);
      mbar_arrive_expect_tx(f, 2 * kTileBytes);
      tma_load_2d(q_tile, &tm_q, h * kD, tok0 + q_row0, f);
      tma_load_2d(q_tile + 16384, &tm_q, h * kD + 64, tok0 + q_row0, f);
      tma_load_2d(do_tile, &tm_do, h * kD, tok0 + q_row0, f);
      tma_load_2d(do_tile + 16384, &tm_do, h * kD + 64, tok0 + q_row0, f);
      for (int j = 0; j < n_kv; ++j) {
        if (!mbar_wait_bounded(smem_u32(&ctl->kv_empty), (j & 1) ^ 1u, wctx, 41, j)) break;
        const uint32_t full = smem_u32(&ctl->kv_full);
        mbar_arrive_expect_tx(full, 2 * kTileBytes);
        const int row = tok0 + j * kT;
        tma_load_2d(k_tile, &tm_k, hk * kD, row, full);
        tma_load_2d(k_tile + 16384, &tm_k, hk * kD + 64, row, full);
        tma_load_2d(v_tile, &tm_v, hk * kD, row, full);
        tma_load_2d(v_tile + 16384, &tm_v, hk * kD + 64, row, full);
      }
    }
  } else if (warp == kWarpMma) {
    if (lane == 0) {
      const uint32_t idesc_kk = umma_idesc_bf16_f32(kT, kT);             // both operands K-major
      const uint32_t idesc_kmn = umma_idesc_bf16_f32(kT, kD) | (1u << 16);  // B MN-major
      bool ok = mbar_wait_bounded(smem_u32(&ctl->qdo_full), 0, wctx, 42, 0);
      for (int j = 0; j < n_kv && ok; ++j) {
        ok = mbar_wait_bounded(smem_u32(&ctl->kv_full), j & 1, wctx, 43, j);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)  // S = Q K^T
          umma_bf16<1>(tmem_s, desc_kmajor(q_tile, kk), desc_kmajor(k_tile, kk), idesc_kk, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)  // dP = dO V^T
          umma_bf16<1>(tmem_dp, desc_kmajor(do_tile, kk), desc_kmajor(v_tile, kk), idesc_kk, kk > 0 ? 1u : 0u);
        umma_commit<1>(smem_u32(&ctl->s_full));
        ok = mbar_wait_bounded(smem_u32(&ctl->ds_full), j & 1, wctx, 44, j);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kT / 16; ++kk)  // dQ += dS K
          umma_bf16<1>(tmem_dq, desc_kmajor(ds_tile, kk), desc_mnmajor(k_tile, kk), idesc_kmn, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit<1>(smem_u32(&ctl->kv_empty));
        if (j + 1 == n_kv) umma_commit<1>(smem_u32(&ctl->acc_full));
      }
    }
  } else {
    const int tid = threadIdx.x;
    const int row = tid & 127, part = tid >> 7;
    const int q_pos = q_row0 + row;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float c = p.scale * kLog2e;
    const bool row_ok = q_pos < p.seq_len;
    const long long stat = (static_cast<long long>(b) * p.hq + h) * p.seq_len + q_pos;
    const float neg_lse2 = row_ok ? __fmul_rn(-p.lse[stat], kLog2e) : 0.f;
    const float dlt = row_ok ? p.delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const bool mine = mbar_wait_bounded(smem_u32(&ctl->s_full), j & 1, wctx, 45, j);
      ok = __all_sync(0xffffffffu, mine) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const int kv0 = j * kT + part * 64;
      const int limit = row_ok ? ((p.causal ? min(q_pos, p.seq_len - 1) : p.seq_len - 1) - kv0) : -1;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t sv[32], dv[32];
        __syncwarp();
        tmem_ld_32x32(tmem_s + lane_base + part * 64 + g * 32, sv);
        tmem_ld_32x32(tmem_dp + lane_base + part * 64 + g * 32, dv);
        tmem_ld_wait_dep(sv);
        tmem_ld_wait_dep(dv);
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float d0 = 0.f, d1 = 0.f;
          if (g * 32 + i <= limit) {
            const float pr = ex2_approx(__fmaf_rn(__uint_as_float(sv[i]), c, neg_lse2));
            d0 = __fmul_rn(__fmul_rn(pr, __fsub_rn(__uint_as_float(dv[i]), dlt)), p.scale);
          }
          if (g * 32 + i + 1 <= limit) {
            const float pr = ex2_approx(__fmaf_rn(__uint_as_float(sv[i + 1]), c, neg_lse2));
            d1 = __fmul_rn(__fmul_rn(pr, __fsub_rn(__uint_as_float(dv[i + 1]), dlt)), p.scale);
          }
          w[i >> 1] = pack_bf16(d0, d1);
        }
        store_tile_row32(ds_ptr, row, part * 64 + g * 32, w);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->ds_full));
    }
    if (ok && n_kv > 0) {
      const bool mine = mbar_wait_bounded(smem_u32(&ctl->acc_full), 0, wctx, 46, 0);
      ok = __all_sync(0xffffffffu, mine) != 0;
    }
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* dst = p.dq + static_cast<long long>(tok0 + q_pos) * p.dq_stride + h * kD + part * 64;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld_32x32(tmem_dq + lane_base + part * 64 + g * 32, v);
        tmem_ld_wait_dep(v);
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(dst + g * 32 + i) =
                make_uint4(pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                           pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                           pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                           pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
        }
      }
    }
  }
  if (ctl->abort_flag) drain_in_flight();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWarpMma) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// dK / dV kernel
// ------------------------------------------------------------------------------------------------
struct CtlDkv {
  uint64_t kv_full;       // K and V tiles loaded (once)
  uint64_t qdo_full, qdo_empty;
  uint64_t st_full;       // S^T and dP^T ready in TMEM
  uint64_t pds_full;      // P^T and dS^T tiles written (count: softmax warps)
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
  float lse2[2][kT];      // -lse * log2(e) of the current q tile, double-buffered by iteration
  float delta[2][kT];
};

__global__ void __launch_bounds__(kThreads, 1)
attention_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                         const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t k_tile = base, v_tile = base + kTileBytes, q_tile = base + 2 * kTileBytes,
                 do_tile = base + 3 * kTileBytes, pt_tile = base + 4 * kTileBytes, dst_tile = base + 5 * kTileBytes;
  uint8_t* pt_ptr = smem + 4 * kTileBytes;
  uint8_t* dst_ptr = smem + 5 * kTileBytes;
  CtlDkv* ctl = reinterpret_cast<CtlDkv*>(smem + 6 * kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = (p.seq_len + kT - 1) / kT;
  const int jt = static_cast<int>(blockIdx.x % n_t);           // kv tile (early tiles are the heavy ones)
  const int bh = blockIdx.x / n_t;
  const int hk = bh % p.hkv, b = bh / p.hkv;
  const int group = p.hq / p.hkv;
  const int kv_row0 = jt * kT, tok0 = b * p.seq_len;
  const int qt0 = p.causal ? jt : 0;
  const int n_q = n_t - qt0;                                   // q tiles per head
  const int n_iter = group * n_q;
  WaitCtx wctx{&ctl->abort_flag, p.status, p.timeout_ns};

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl->kv_full), 1);
    mbar_init(smem_u32(&ctl->qdo_full), 1);
    mbar_init(smem_u32(&ctl->qdo_empty), 1);
    mbar_init(smem_u32(&ctl->st_full), 1);
    mbar_init(smem_u32(&ctl->pds_full), kSoftThreads / 32);
    mbar_init(smem_u32(&ctl->acc_full), 1);
    ctl->abort_flag = 0;
    fence_mbar_init_cluster();
  }
  if (warp == kWarpMma) {
    tmem_alloc<1>(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t tmem_st = tmem_base, tmem_dpt = tmem_base + 128, tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 384;

  if (warp == kWarpTma) {
    if (lane == 0) {
      const uint32_t f = smem_u32(&ctl->kv_full);
      mbar_arrive_expect_tx(f, 2 * kTileBytes);
      tma_load_2d(k_tile, &tm_k, hk * kD, tok0 + kv_row0, f);
      tma_load_2d(k_tile + 16384, &tm_k, hk * kD + 64, tok0 + kv_row0, f);
      tma_load_2d(v_tile, &tm_v, hk * kD, tok0 + kv_row0, f);
      tma_load_2d(v_tile + 16384, &tm_v, hk * kD + 64, tok0 + kv_row0, f);
      for (int n = 0; n < n_iter; ++n) {
        const int h = hk * group + n / n_q, qt = qt0 + n % n_q;
        if (!mbar_wait_bounded(smem_u32(&ctl->qdo_empty), (n & 1) ^ 1u, wctx, 51, n)) break;
        const uint32_t full = smem_u32(&ctl->qdo_full);
        mbar_arrive_expect_tx(full, 2 * kTileBytes);
        const int row = tok0 + qt * kT;
        tma_load_2d(q_tile, &tm_q, h * kD, row, full);
        tma_load_2d(q_tile + 16384, &tm_q, h * kD + 64, row, full);
        tma_load_2d(do_tile, &tm_do, h * kD, row, full);
        tma_load_2d(do_tile + 16384, &tm_do, h * kD + 64, row, full);
      }
    }
  } else if (warp == kWarpMma) {
    if (lane == 0) {
      const uint32_t idesc_kk = umma_idesc_bf16_f32(kT, kT);
      const uint32_t idesc_kmn = umma_idesc_bf16_f32(kT, kD) | (1u << 16);
      bool ok = mbar_wait_bounded(smem_u32(&ctl->kv_full), 0, wctx, 52, 0);
      for (int n = 0; n < n_iter && ok; ++n) {
        ok = mbar_wait_bounded(smem_u32(&ctl->qdo_full), n & 1, wctx, 53, n);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)  // S^T = K Q^T
          umma_bf16<1>(tmem_st, desc_kmajor(k_tile, kk), desc_kmajor(q_tile, kk), idesc_kk, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)  // dP^T = V dO^T
          umma_bf16<1>(tmem_dpt, desc_kmajor(v_tile, kk), desc_kmajor(do_tile, kk), idesc_kk, kk > 0 ? 1u : 0u);
        umma_commit<1>(smem_u32(&ctl->st_full));
        ok = mbar_wait_bounded(smem_u32(&ctl->pds_full), n & 1, wctx, 54, n);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kT / 16; ++kk)  // dV += P^T dO
          umma_bf16<1>(tmem_dv, desc_kmajor(pt_tile, kk), desc_mnmajor(do_tile, kk), idesc_kmn, (n > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kT / 16; ++kk)  // dK += dS^T Q
          umma_bf16<1>(tmem_dk, desc_kmajor(dst_tile, kk), desc_mnmajor(q_tile, kk), idesc_kmn, (n > 0 || kk > 0) ? 1u : 0u);
        umma_commit<1>(smem_u32(&ctl->qdo_empty));
        if (n + 1 == n_iter) umma_commit<1>(smem_u32(&ctl->acc_full));
      }
    }
  } else {
    // Thread (row, part): KV row `row` of the tile, query columns [part * 64, part * 64 + 64).
    // One named barrier per iteration, reached by all 256 threads whatever happened before.
    const int tid = threadIdx.x;
    const int row = tid & 127, part = tid >> 7;
    const int kv_pos = kv_row0 + row;
    const bool row_ok = kv_pos < p.seq_len;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float c = p.scale * kLog2e;
    bool ok = true;
    for (int n = 0; n < n_iter; ++n) {
      const int h = hk * group + n / n_q, qt = qt0 + n % n_q;
      const int buf = n & 1;
      if (tid < kT) {
        const int qp = qt * kT + tid;
        const long long stat = (static_cast<long long>(b) * p.hq + h) * p.seq_len + qp;
        const bool v_ok = qp < p.seq_len;
        ctl->lse2[buf][tid] = v_ok ? __fmul_rn(-p.lse[stat], kLog2e) : 0.f;
        ctl->delta[buf][tid] = v_ok ? p.delta[stat] : 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kSoftThreads) : "memory");
      if (ctl->abort_flag) ok = false;
      if (ok) {
        const bool mine = mbar_wait_bounded(smem_u32(&ctl->st_full), n & 1, wctx, 55, n);
        ok = __all_sync(0xffffffffu, mine) != 0;
      }
      if (!ok) continue;
      tc_fence_after_sync();
      const int q0 = qt * kT + part * 64;  // first query column of this thread
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t sv[32], dv[32];
        __syncwarp();
        tmem_ld_32x32(tmem_st + lane_base + part * 64 + g * 32, sv);
        tmem_ld_32x32(tmem_dpt + lane_base + part * 64 + g * 32, dv);
        tmem_ld_wait_dep(sv);
        tmem_ld_wait_dep(dv);
        uint32_t wp[16], wd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], dsv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = part * 64 + g * 32 + i + e;   // inside the q tile
            const int qp = q0 + g * 32 + i + e;           // position in the sequence
            const bool valid = row_ok && qp < p.seq_len && (!p.causal || kv_pos <= qp);
            float pr = 0.f, ds = 0.f;
            if (valid) {
              pr = ex2_approx(__fmaf_rn(__uint_as_float(sv[i + e]), c, ctl->lse2[buf][col]));
              ds = __fmul_rn(__fmul_rn(pr, __fsub_rn(__uint_as_float(dv[i + e]), ctl->delta[buf][col])), p.scale);
            }
            pv[e] = pr;
            dsv[e] = ds;
          }
          wp[i >> 1] = pack_bf16(pv[0], pv[1]);
          wd[i >> 1] = pack_bf16(dsv[0], dsv[1]);
        }
        store_tile_row32(pt_ptr, row, part * 64 + g * 32, wp);
        store_tile_row32(dst_ptr, row, part * 64 + g * 32, wd);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->pds_full));
    }
    if (ok && n_iter > 0) {
      const bool mine = mbar_wait_bounded(smem_u32(&ctl->acc_full), 0, wctx, 56, 0);
      ok = __all_sync(0xffffffffu, mine) != 0;
    }
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* dk = p.dk + static_cast<long long>(tok0 + kv_pos) * p.dk_stride + hk * kD + part * 64;
      __nv_bfloat16* dv_out = p.dv + static_cast<long long>(tok0 + kv_pos) * p.dv_stride + hk * kD + part * 64;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t a[32], bq[32];
        __syncwarp();
        tmem_ld_32x32(tmem_dv + lane_base + part * 64 + g * 32, a);
        tmem_ld_32x32(tmem_dk + lane_base + part * 64 + g * 32, bq);
        tmem_ld_wait_dep(a);
        tmem_ld_wait_dep(bq);
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            *reinterpret_cast<uint4*>(dv_out + g * 32 + i) =
                make_uint4(pack_bf16(__uint_as_float(a[i]), __uint_as_float(a[i + 1])),
                           pack_bf16(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3])),
                           pack_bf16(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5])),
                           pack_bf16(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7])));
            *reinterpret_cast<uint4*>(dk + g * 32 + i) =
                make_uint4(pack_bf16(__uint_as_float(bq[i]), __uint_as_float(bq[i + 1])),
                           pack_bf16(__uint_as_float(bq[i + 2]), __uint_as_float(bq[i + 3])),
                           pack_bf16(__uint_as_float(bq[i + 4]), __uint_as_float(bq[i + 5])),
                           pack_bf16(__uint_as_float(bq[i + 6]), __uint_as_float(bq[i + 7])));
          }
        }
      }
    }
  }
  if (ctl->abort_flag) drain_in_flight();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWarpMma) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

}  // namespace
}  // namespace ka

// q, k, v, o, d_o: [B*L, heads*128] bf16 views (token strides in elements); lse: [B, Hq, L];
// delta: scratch [B, Hq, L] fp32; dq / dk / dv: outputs with their own token strides.
extern "C" int ka_attention_bwd(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                                long long v_stride, const void* o, long long o_stride, const void* d_o,
                                long long do_stride, const float* lse, float* delta, void* dq, long long dq_stride,
                                void* dk, long long dk_stride, void* dv, long long dv_stride, int batch, int seq_len,
                                int hq, int hkv, int head_dim, float scale, int causal, int* status,
                                unsigned long long timeout_ns, void* stream) {
  using namespace ka;
  if (batch <= 0 || seq_len <= 0) return 0;
  if (head_dim != kD || hq % hkv != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  constexpr int kSmemDq = 5 * kTileBytes + 1024 + 256;
  constexpr int kSmemDkv = 6 * kTileBytes + 1024 + 2304;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDq) != cudaSuccess ||
        cudaFuncSetAttribute(attention_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDkv) != cudaSuccess)
      return -10;
    configured = true;
  }
  const uint64_t tokens = static_cast<uint64_t>(batch) * seq_len;
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_tmap_2d_16bit_sw128(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, q, tokens, static_cast<uint64_t>(hq) * kD,
                                    q_stride, kT, 64);
  if (rc) return -20 + rc;
  rc = make_tmap_2d_16bit_sw128(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, k, tokens, static_cast<uint64_t>(hkv) * kD,
                                k_stride, kT, 64);
  if (rc) return -40 + rc;
  rc = make_tmap_2d_16bit_sw128(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, v, tokens, static_cast<uint64_t>(hkv) * kD,
                                v_stride, kT, 64);
  if (rc) return -60 + rc;
  rc = make_tmap_2d_16bit_sw128(&tdo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d_o, tokens, static_cast<uint64_t>(hq) * kD,
                                do_stride, kT, 64);
  if (rc) return -80 + rc;
  const long long n_warps = static_cast<long long>(tokens) * hq;
  attention_delta_kernel<<<static_cast<unsigned>((n_warps * 32 + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), o_stride, static_cast<const __nv_bfloat16*>(d_o), do_stride, delta, batch,
      seq_len, hq);
  BwdParams p = {};
  p.lse = lse;
  p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq);
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.dq_stride = dq_stride;
  p.dk_stride = dk_stride;
  p.dv_stride = dv_stride;
  p.batch = batch;
  p.seq_len = seq_len;
  p.hq = hq;
  p.hkv = hkv;
  p.scale = scale;
  p.causal = causal;
  p.status = status;
  p.timeout_ns = timeout_ns;
  const int n_t = (seq_len + kT - 1) / kT;
  attention_bwd_dq_kernel<<<static_cast<unsigned>(batch) * hq * n_t, kThreads, kSmemDq, st>>>(tq, tk, tv, tdo, p);
  attention_bwd_dkv_kernel<<<static_cast<unsigned>(batch) * hkv * n_t, kThreads, kSmemDkv, st>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
