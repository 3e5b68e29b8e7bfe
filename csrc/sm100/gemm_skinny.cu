// Skinny bf16 GEMM for decode-sized batches on sm_100a: C[M, N] = A[M, K] * W[N, K]^T with
// M <= 64 (one new token per sequence), bitwise equal to the tiled kernel of gemm.cu.
//
// With a handful of rows the product is a stream of the weight matrix, so the operands are
// swapped: the WEIGHTS are the 128-row A operand of tcgen05.mma and the activations the narrow
// B operand (N = the batch padded to 16 / 32 / 64), D^T[n, m] accumulating in TMEM. Every CTA
// owns 128 weight rows and walks the whole K in one accumulation chain (no split-K: the order
// of the sum over K is the one the tiled kernel uses, so a row's result does not depend on
// which of the two kernels its batch size selects). Nearly all shared memory is a TMA ring of
// weight tiles (11 stages x 16 KiB in flight per SM), which is what a memory-bound stream
// needs. Measured: a CTA streams about 80 GB/s, bounded by load latency over that ring, so
// shapes with N >= 128 x (number of SMs) run near the HBM rate and N = 4096 (32 CTAs) at about
// a quarter of it; taking fewer weight rows per CTA did not help (the K loop then becomes
// bound by the rate of MMA instructions), and splitting K would change the order of the sum.
//
// The reference has no GEMM of its own (it names backends in rl_engine/kernels/registry.py:41-55).
#include <cstdint>
#include <cuda_bf16.h>

#include "common/bounded_wait.cuh"
#include "common/ptx.cuh"
#include "common/tmap.cuh"

namespace ka {
namespace {

constexpr int kMmaRows = 128;  // M of the MMA (rows of shared memory it reads per K step)
constexpr int kBK = 64;        // K per stage: one 128-byte swizzled row
constexpr int kThreads = 192;  // four epilogue warps, one TMA warp, one MMA warp
constexpr int kMaxStages = 32;

// NB: batch rows padded (the MMA's N); R: weight rows per CTA
template <int NB, int R>
struct Cfg {
  static constexpr int kWBytes = R * kBK * 2;
  static constexpr int kXBytes = NB * kBK * 2;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStages = (196 * 1024) / kStageBytes > kMaxStages ? kMaxStages : (196 * 1024) / kStageBytes;
  // slack: the MMA of the last stage reads kMmaRows rows starting at its (shorter) weight tile
  static constexpr int kSlack = (kMmaRows - R) * kBK * 2;
  static constexpr int kSmemBytes = kStages * kStageBytes + kSlack + 1024 + 1024;
};

struct Control {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct SkinnyParams {
  __nv_bfloat16* out;   // [M, N], row stride ldc
  long long ldc;
  int m, n, k;
  int* status;
  unsigned long long timeout_ns;
};

template <int NB, int R>
__global__ void __launch_bounds__(kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const __grid_constant__ SkinnyParams p) {
  using C = Cfg<NB, R>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  Control* ctl = reinterpret_cast<Control*>(smem + C::kStages * C::kStageBytes + C::kSlack);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * R;
  const int num_kb = (p.k + kBK - 1) / kBK;
  constexpr int kTmemCols = NB < 32 ? 32 : NB;

  WaitCtx wctx{&ctl->abort_flag, p.status, p.timeout_ns};
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->acc_full), 1);
    ctl->abort_flag = 0;
    fence_mbar_init_cluster();
  }
  if (warp == 5) {
    tmem_alloc<1>(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % C::kStages;
        if (!mbar_wait_bounded(smem_u32(&ctl->empty[s]), ((kb / C::kStages) & 1) ^ 1u, wctx, 61, s)) break;
        const uint32_t full = smem_u32(&ctl->full[s]);
        const uint32_t wt = base + s * C::kStageBytes, xt = wt + C::kWBytes;
        mbar_arrive_expect_tx(full, C::kStageBytes);
        tma_load_2d(wt, &tm_w, kb * kBK, n0, full);
        tma_load_2d(xt, &tm_x, kb * kBK, 0, full);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_f32(kMmaRows, NB);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % C::kStages;
        ok = mbar_wait_bounded(smem_u32(&ctl->full[s]), (kb / C::kStages) & 1, wctx, 62, s);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t wt = base + s * C::kStageBytes, xt = wt + C::kWBytes;
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k)
          umma_bf16<1>(tmem_base, umma_desc_k_sw128(wt + k * 32), umma_desc_k_sw128(xt + k * 32), idesc,
                       (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit<1>(smem_u32(&ctl->empty[s]));
      }
      if (ok) umma_commit<1>(smem_u32(&ctl->acc_full));
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // TMEM lane = weight row (output column n), TMEM column = batch row m.
    const bool mine = mbar_wait_bounded(smem_u32(&ctl->acc_full), 0, wctx, 63, 0);
    const bool ok = __all_sync(0xffffffffu, mine) != 0;
    if (ok && warp * 32 < R) {
      tc_fence_after_sync();
      const int n = n0 + warp * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll
      for (int c0 = 0; c0 < kTmemCols; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c0, v);
        tmem_ld_wait();
        if (n < p.n) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int m = c0 + i;
            if (m < p.m) p.out[static_cast<long long>(m) * p.ldc + n] = __float2bfloat16_rn(__uint_as_float(v[i]));
          }
        }
      }
    }
  }

  if (ctl->abort_flag) drain_in_flight();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

template <int NB, int R>
int launch(const void* a, long long lda, const void* w, long long ldw, const SkinnyParams& p, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<NB, R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg<NB, R>::kSmemBytes) != cudaSuccess)
      return -10;
    configured = true;
  }
  CUtensorMap tw, tx;
  int rc = make_tmap_2d_16bit_sw128(&tw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, w, static_cast<uint64_t>(p.n),
                                    static_cast<uint64_t>(p.k), ldw, R, kBK);
  if (rc) return -20 + rc;
  rc = make_tmap_2d_16bit_sw128(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, static_cast<uint64_t>(p.m),
                                static_cast<uint64_t>(p.k), lda, NB, kBK);
  if (rc) return -40 + rc;
  const unsigned grid = static_cast<unsigned>((p.n + R - 1) / R);
  gemm_skinny_kernel<NB, R><<<grid, kThreads, Cfg<NB, R>::kSmemBytes, stream>>>(tw, tx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace
}  // namespace ka

// out[M, N] (bf16, row stride ldc) = a[M, K] (row stride lda) times w[N, K]^T (row stride ldw),
// for 1 <= M <= 64. Strides in elements, multiples of 8; pointers 16-byte aligned.
extern "C" int ka_gemm_skinny_bf16(const void* a, long long lda, const void* w, long long ldw, void* out,
                                   long long ldc, int m, int n, int k, int* status,
                                   unsigned long long timeout_ns, void* stream) {
  using namespace ka;
  if (m <= 0 || n <= 0) return 0;
  if (m > 64 || k <= 0) return -1;
  const int nb = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
  SkinnyParams p = {};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldc = ldc;
  p.m = m;
  p.n = n;
  p.k = k;
  p.status = status;
  p.timeout_ns = timeout_ns;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (nb == 16) return launch<16, 128>(a, lda, w, ldw, p, st);
  if (nb == 32) return launch<32, 128>(a, lda, w, ldw, p, st);
  return launch<64, 128>(a, lda, w, ldw, p, st);
}
