// Batch-invariant causal attention forward for sm_100a (GQA, head_dim 128).
//
// One CTA per (sequence, query head, 128-row query tile). Q, K and V tiles arrive by TMA;
// S = Q K^T and O_j = P_j V_j are tcgen05.mma (M=128, N=128) with fp32 accumulators in TMEM
// (two S buffers and one O accumulator); eight softmax warps give every query row two
// threads (64 columns each, so each scheduler has two warps to interleave; four per row ran
// slower, the registers no longer fit), pull their part of the S row into registers in one go, write P as bf16 into a swizzled shared-memory tile
// that the second MMA consumes, and let the MMA accumulate O in TMEM. The running maximum is
// only moved when it grows by more than 2^8 (then O is rescaled in TMEM), so the common tile
// needs no correction pass.
// KV tiles are visited in increasing order, always 128 wide, whatever the batch size or the
// number of heads on this GPU, so a query row's output depends on that sequence only.
//
// The reference only routes the name "attention" to a backend string
// (rl_engine/kernels/registry.py:41-55); there is no attention kernel in it.
#include <cstdint>
#include <cstdio>
#include <cuda_bf16.h>
#include <math_constants.h>

#include "common/bounded_wait.cuh"
#include "common/ptx.cuh"
#include "common/tmap.cuh"
#include "attention_common.cuh"

namespace ka {
namespace {

constexpr int kD = 128;         // head dim
constexpr int kBQ = 128;        // query rows per CTA
constexpr int kBKV = 128;       // keys per tile
constexpr int kSplit = 2;        // softmax threads per query row (64 columns each)
constexpr int kSoftThreads = 128 * kSplit;
constexpr int kThreads = kSoftThreads + 64;  // softmax warps, then one TMA warp and one MMA warp
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KiB: two 64-column boxes of 128 rows
constexpr int kKvStages = 2;
constexpr int kSmemBytes = kTileBytes /*Q*/ + kKvStages * 2 * kTileBytes /*K,V*/ + kTileBytes /*P*/ + 1024 + 8192;
constexpr float kLog2e = 1.4426950408889634f;

struct Control {
  uint64_t q_full;
  uint64_t kv_full[kKvStages];
  uint64_t kv_empty[kKvStages];
  uint64_t s_full[2];
  uint64_t s_empty[2];
  uint64_t p_full;
  uint64_t p_empty;
  uint64_t o_full;
  uint32_t tmem_base;
  int abort_flag;
  float half_max[2][kSplit][128];  // [tile parity][column part][row]
  float half_sum[kSplit][128];
};

struct AttnParams {
  __nv_bfloat16* out;     // [B, L, Hq, D] with token stride out_stride
  float* lse;             // [B, Hq, L] or null (natural-log log-sum-exp of the scaled scores)
  long long out_stride;   // elements between tokens in out
  int batch, seq_len, hq, hkv;
  float scale;            // softmax scale (1/sqrt(D))
  int causal;
  int* status;
  unsigned long long timeout_ns;
};

__global__ void __launch_bounds__(kThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t q_tile = base;
  const uint32_t kv_tiles = base + kTileBytes;                       // stage s: K at +s*64K, V at +s*64K+32K
  const uint32_t p_tile = kv_tiles + kKvStages * 2 * kTileBytes;
  uint8_t* p_ptr = smem + kTileBytes + kKvStages * 2 * kTileBytes;
  Control* ctl = reinterpret_cast<Control*>(p_ptr + kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.seq_len + kBQ - 1) / kBQ;
  // heavy (late) query tiles first
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x % n_qt);
  const int bh = blockIdx.x / n_qt;
  const int h = bh % p.hq;
  const int b = bh / p.hq;
  const int hk = h / (p.hq / p.hkv);
  const int q_row0 = qt * kBQ;                       // inside the sequence
  const int tok0 = b * p.seq_len;                    // first token of the sequence
  const int kv_end = p.causal ? min(p.seq_len, q_row0 + kBQ) : p.seq_len;
  const int n_kv = (kv_end + kBKV - 1) / kBKV;

  WaitCtx wctx{&ctl->abort_flag, p.status, p.timeout_ns};

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl->q_full), 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(smem_u32(&ctl->kv_full[s]), 1);
      mbar_init(smem_u32(&ctl->kv_empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl->s_full[i]), 1);
      mbar_init(smem_u32(&ctl->s_empty[i]), 4 * kSplit);
    }
    mbar_init(smem_u32(&ctl->o_full), 1);
    mbar_init(smem_u32(&ctl->p_full), 4 * kSplit);
    mbar_init(smem_u32(&ctl->p_empty), 1);
    ctl->abort_flag = 0;
    fence_mbar_init_cluster();
  }
  if (warp == kSoftThreads / 32 + 1) {
    tmem_alloc<1>(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t tmem_s = tmem_base;          // S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 256;    // O accumulator: columns [256,384)

  if (warp == kSoftThreads / 32) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t qf = smem_u32(&ctl->q_full);
      mbar_arrive_expect_tx(qf, kTileBytes);
      tma_load_2d(q_tile, &tm_q, h * kD, tok0 + q_row0, qf);
      tma_load_2d(q_tile + 16384, &tm_q, h * kD + 64, tok0 + q_row0, qf);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % kKvStages;
        const uint32_t ph = (j / kKvStages) & 1;
        if (!mbar_wait_bounded(smem_u32(&ctl->kv_empty[s]), ph ^ 1u, wctx, 31, s)) break;
        const uint32_t full = smem_u32(&ctl->kv_full[s]);
        const uint32_t kt = kv_tiles + s * 2 * kTileBytes, vt = kt + kTileBytes;
        mbar_arrive_expect_tx(full, 2 * kTileBytes);
        const int row = tok0 + j * kBKV;
        tma_load_2d(kt, &tm_k, hk * kD, row, full);
        tma_load_2d(kt + 16384, &tm_k, hk * kD + 64, row, full);
        tma_load_2d(vt, &tm_v, hk * kD, row, full);
        tma_load_2d(vt + 16384, &tm_v, hk * kD + 64, row, full);
      }
    }
  } else if (warp == kSoftThreads / 32 + 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_bf16_f32(kBQ, kBKV);
      const uint32_t idesc_o = umma_idesc_bf16_f32(kBQ, kD) | (1u << 16);  // B (V) is MN-major
      bool ok = mbar_wait_bounded(smem_u32(&ctl->q_full), 0, wctx, 32, 0);
      auto issue_s = [&](int j) -> bool {
        const int s = j % kKvStages, sb = j & 1;
        if (!mbar_wait_bounded(smem_u32(&ctl->kv_full[s]), (j / kKvStages) & 1, wctx, 33, s)) return false;
        if (!mbar_wait_bounded(smem_u32(&ctl->s_empty[sb]), ((j >> 1) & 1) ^ 1u, wctx, 34, sb)) return false;
        tc_fence_after_sync();
        const uint32_t kt = kv_tiles + s * 2 * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          umma_bf16<1>(tmem_s + sb * 128, desc_kmajor(q_tile, kk), desc_kmajor(kt, kk), idesc_s, kk > 0 ? 1u : 0u);
        umma_commit<1>(smem_u32(&ctl->s_full[sb]));
        return true;
      };
      if (ok && n_kv > 0) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j % kKvStages;
        ok = mbar_wait_bounded(smem_u32(&ctl->p_full), j & 1, wctx, 35, j);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t vt = kv_tiles + s * 2 * kTileBytes + kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kBKV / 16; ++kk)
          umma_bf16<1>(tmem_o, desc_kmajor(p_tile, kk), desc_mnmajor(vt, kk), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit<1>(smem_u32(&ctl->p_empty));      // P tile reusable, O up to date
        umma_commit<1>(smem_u32(&ctl->kv_empty[s]));
        if (j + 1 == n_kv) umma_commit<1>(smem_u32(&ctl->o_full));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output
    // Thread (row, part) owns 32 columns of query row `row`: four threads per row, so every
    // scheduler interleaves four warps. Every iteration executes exactly one named barrier
    // whatever happened before it, and the decision to stop is taken from the shared abort
    // flag after that barrier, so no thread is left behind.
    constexpr int kCols = kBKV / kSplit;    // columns per thread
    constexpr int kLd = kCols / 32;         // tcgen05.ld groups per thread
    const int tid = threadIdx.x;
    const int row = tid & 127;              // query row inside the tile == TMEM lane
    const int part = tid >> 7;              // which kCols columns
    const int q_pos = q_row0 + row;
    const float c = p.scale * kLog2e;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float m = -CUDART_INF_F;                // reference maximum of the row (may lag the true one by < 2^8)
    float l = 0.f;                          // this thread's part of the row sum
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1;
      uint32_t sv[kLd][32];
      float mx = -CUDART_INF_F;
      const int kv0 = j * kBKV + part * kCols;
      const int limit = (p.causal ? min(q_pos, p.seq_len - 1) : p.seq_len - 1) - kv0;  // last allowed column
      const bool full_tile = limit >= kCols - 1;
      if (ok) {
        const bool mine = mbar_wait_bounded(smem_u32(&ctl->s_full[sb]), (j >> 1) & 1, wctx, 38, sb);
        ok = __all_sync(0xffffffffu, mine) != 0;
      }
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int g = 0; g < kLd; ++g) tmem_ld_32x32(tmem_s + lane_base + sb * 128 + part * kCols + g * 32, sv[g]);
#pragma unroll
        for (int g = 0; g < kLd; ++g) tmem_ld_wait_dep(sv[g]);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->s_empty[sb]));  // S buffer free for tile j + 2
        float a0 = -CUDART_INF_F, a1 = -CUDART_INF_F;
#pragma unroll
        for (int g = 0; g < kLd; ++g) {
          if (full_tile) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              a0 = fmaxf(a0, __uint_as_float(sv[g][i]));
              a1 = fmaxf(a1, __uint_as_float(sv[g][i + 1]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              a0 = fmaxf(a0, (g * 32 + i <= limit) ? __uint_as_float(sv[g][i]) : -CUDART_INF_F);
          }
        }
        mx = fmaxf(a0, a1);
      }
      ctl->half_max[sb][part][row] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(kSoftThreads) : "memory");
      if (ctl->abort_flag) ok = false;
      if (!ok) continue;
#pragma unroll
      for (int q = 0; q < kSplit; ++q) mx = fmaxf(mx, ctl->half_max[sb][q][row]);
      // move the reference maximum only on the first tile or when it would grow by more than
      // 2^8 in the exponent; otherwise probabilities are taken relative to the old reference
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m) {
        if (m == -CUDART_INF_F) {
          m = mx;
        } else if (__fmul_rn(__fsub_rn(mx, m), c) > 8.f) {
          alpha = ex2_approx(__fmul_rn(__fsub_rn(m, mx), c));
          m = mx;
          rescale = true;
        }
      }
      const float m_ref = (m == -CUDART_INF_F) ? 0.f : m;
      const float neg = __fmul_rn(-m_ref, c);

      // the P tile (and O) are ours once the previous P V product has completed
      {
        const bool mine2 = mbar_wait_bounded(smem_u32(&ctl->p_empty), (j & 1) ^ 1u, wctx, 39, j);
        ok = __all_sync(0xffffffffu, mine2) != 0;
        if (!ok) continue;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // rare: bring this thread's columns of O in TMEM to the new reference
        tc_fence_after_sync();
        uint32_t v[32];
#pragma unroll
        for (int g = 0; g < kLd; ++g) {
          __syncwarp();
          tmem_ld_32x32(tmem_o + lane_base + part * kCols + g * 32, v);
          tmem_ld_wait_dep(v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__fmul_rn(__uint_as_float(v[i]), alpha));
          tmem_st_32x32(tmem_o + lane_base + part * kCols + g * 32, v);
        }
        tmem_st_wait();
      }
      float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
#pragma unroll
      for (int g = 0; g < kLd; ++g) {
        float e[32];
        if (full_tile) {
#pragma unroll
          for (int i = 0; i < 32; ++i) e[i] = ex2_approx(__fmaf_rn(__uint_as_float(sv[g][i]), c, neg));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            e[i] = (g * 32 + i <= limit) ? ex2_approx(__fmaf_rn(__uint_as_float(sv[g][i]), c, neg)) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          ls0 = __fadd_rn(ls0, e[i]);
          ls1 = __fadd_rn(ls1, e[i + 1]);
          ls2 = __fadd_rn(ls2, e[i + 2]);
          ls3 = __fadd_rn(ls3, e[i + 3]);
        }
        // columns col .. col+31 of the row: box (col >> 6), 16-byte chunks ((col >> 5) & 1) * 4 + 0..3
        const int col = part * kCols + g * 32;
        uint8_t* rowp = p_ptr + (col >> 6) * 16384 + row * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int phys = (((col >> 5) & 1) * 4 + ch) ^ (row & 7);
          uint4 w;
          w.x = pack_bf16(e[ch * 8 + 0], e[ch * 8 + 1]);
          w.y = pack_bf16(e[ch * 8 + 2], e[ch * 8 + 3]);
          w.z = pack_bf16(e[ch * 8 + 4], e[ch * 8 + 5]);
          w.w = pack_bf16(e[ch * 8 + 6], e[ch * 8 + 7]);
          *reinterpret_cast<uint4*>(rowp + phys * 16) = w;
        }
      }
      l = __fmaf_rn(l, alpha, __fadd_rn(__fadd_rn(ls0, ls1), __fadd_rn(ls2, ls3)));
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full));
    }

    // combine the parts of the row sum (fixed order)
    ctl->half_sum[part][row] = l;
    asm volatile("bar.sync 1, %0;" ::"n"(kSoftThreads) : "memory");
    if (ctl->abort_flag) ok = false;
    float l_total = ctl->half_sum[0][row];
#pragma unroll
    for (int q = 1; q < kSplit; ++q) l_total = __fadd_rn(l_total, ctl->half_sum[q][row]);
    if (ok && n_kv > 0) {
      const bool mine = mbar_wait_bounded(smem_u32(&ctl->o_full), 0, wctx, 37, 0);
      ok = __all_sync(0xffffffffu, mine) != 0;
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = l_total > 0.f ? __fdiv_rn(1.f, l_total) : 0.f;
      __nv_bfloat16* dst = p.out + static_cast<long long>(tok0 + q_pos) * p.out_stride + h * kD + part * kCols;
      uint32_t v[32];
#pragma unroll
      for (int g = 0; g < kLd; ++g) {
        __syncwarp();
        tmem_ld_32x32(tmem_o + lane_base + part * kCols + g * 32, v);
        tmem_ld_wait_dep(v);
        if (q_pos < p.seq_len) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16(__fmul_rn(__uint_as_float(v[i]), inv), __fmul_rn(__uint_as_float(v[i + 1]), inv));
            w.y = pack_bf16(__fmul_rn(__uint_as_float(v[i + 2]), inv), __fmul_rn(__uint_as_float(v[i + 3]), inv));
            w.z = pack_bf16(__fmul_rn(__uint_as_float(v[i + 4]), inv), __fmul_rn(__uint_as_float(v[i + 5]), inv));
            w.w = pack_bf16(__fmul_rn(__uint_as_float(v[i + 6]), inv), __fmul_rn(__uint_as_float(v[i + 7]), inv));
            *reinterpret_cast<uint4*>(dst + g * 32 + i) = w;
          }
        }
      }
      if (p.lse && part == 0 && q_pos < p.seq_len)
        p.lse[(static_cast<long long>(b) * p.hq + h) * p.seq_len + q_pos] =
            __fmaf_rn(lg2_approx(l_total), 0.6931471805599453f, __fmul_rn(m, p.scale));
    }
  }

  if (ctl->abort_flag) drain_in_flight();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kSoftThreads / 32 + 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

}  // namespace
}  // namespace ka

// q: [B*L, Hq*128] view with `q_stride` elements between tokens; k, v: [B*L, Hkv*128] views
// (strides k_stride, v_stride); out: [B*L, Hq*128] with out_stride; lse: [B, Hq, L] fp32 or
// null. All bf16, 16-byte aligned, strides multiples of 8.
extern "C" int ka_attention_fwd(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                                long long v_stride, void* out, long long out_stride, float* lse, int batch,
                                int seq_len, int hq, int hkv, int head_dim, float scale, int causal, int* status,
                                unsigned long long timeout_ns, void* stream) {
  using namespace ka;
  if (batch <= 0 || seq_len <= 0) return 0;
  if (head_dim != kD || hq % hkv != 0) return -1;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return -10;
    configured = true;
  }
  const uint64_t tokens = static_cast<uint64_t>(batch) * seq_len;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d_16bit_sw128(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, q, tokens, static_cast<uint64_t>(hq) * kD,
                                    q_stride, kBQ, 64);
  if (rc) return -20 + rc;
  rc = make_tmap_2d_16bit_sw128(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, k, tokens, static_cast<uint64_t>(hkv) * kD,
                                k_stride, kBKV, 64);
  if (rc) return -40 + rc;
  rc = make_tmap_2d_16bit_sw128(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, v, tokens, static_cast<uint64_t>(hkv) * kD,
                                v_stride, kBKV, 64);
  if (rc) return -60 + rc;
  AttnParams p = {};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.out_stride = out_stride;
  p.batch = batch;
  p.seq_len = seq_len;
  p.hq = hq;
  p.hkv = hkv;
  p.scale = scale;
  p.causal = causal;
  p.status = status;
  p.timeout_ns = timeout_ns;
  const int n_qt = (seq_len + kBQ - 1) / kBQ;
  const unsigned grid = static_cast<unsigned>(batch) * hq * n_qt;
  attention_fwd_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
