// Batch-invariant bf16 GEMM for sm_100a: persistent CTA pairs, TMA operand ring,
// tcgen05.mma (cta_group::2, M=256 N=256 K=16) into double-buffered TMEM accumulators, and an
// epilogue that either stores the tile or emits fp32 K-slice partials for the tensor-parallel
// reduce-scatter (see gemm.h). Operands may be K-major or MN-major (the latter serves the
// backward GEMMs without transposes).
//
// The reference has no GEMM of its own; its registry only names backends
// (rl_engine/kernels/registry.py:20-30).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cuda_bf16.h>

#include "common/bounded_wait.cuh"
#include "common/ptx.cuh"
#include "common/tmap.cuh"
#include "gemm.h"

namespace ka {
namespace {

constexpr int kG = 2;              // CTAs per tile
constexpr int kBM = 128;           // rows per CTA
constexpr int kBN = 256;           // columns per tile
constexpr int kBK = 64;            // K per stage
constexpr int kUmmaK = 16;
constexpr int kEpiWarps = 8;        // two per TMEM lane quarter: columns [0,128) and [128,256)
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kWarpTma = kEpiWarps, kWarpMma = kEpiWarps + 1, kWarpPub = kEpiWarps + 2;
constexpr int kThreads = kEpiThreads + 96;  // epilogue warps, TMA producer, MMA issuer, one spare warp
constexpr int kStages = 6;
constexpr int kABytes = kBM * kBK * 2;            // 16 KiB
constexpr int kBBytes = (kBN / kG) * kBK * 2;     // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTxBytes = kStageBytes * kG;
constexpr int kTileBytes = kStages * kStageBytes;
constexpr int kEpiBufWords = 32 * 33;     // per epilogue warp: 32 rows x 32 words, padded
constexpr int kSmemBytes = kTileBytes + 1024 + 512 + kEpiWarps * kEpiBufWords * 4;
constexpr int kGroupM = 8;         // row tiles that share a column tile in the schedule

struct Control {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
};

enum Where : int { kWProducer = 11, kWMmaFull = 12, kWMmaTmem = 13, kWEpi = 14, kWReduceFlag = 15, kWGatherFlag = 16 };

// MN-major operand tile written by TMA as 64-element (128 B) wide boxes of 64 K-rows each:
// 16-byte chunks along MN are contiguous (swizzled), 8 K-rows form a 1024 B group (SBO), the
// next 64 MN elements start one box (8 KiB) further (LBO).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(8192 >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

struct Unit {
  int m_blk, n_blk, slice;
};

__device__ __forceinline__ void decode_unit(const GemmParams& p, int tiles_m, int tiles_n, int u, Unit& out) {
  const int t = u / p.k_slices;
  out.slice = u - t * p.k_slices;
  const int per_group = kGroupM * tiles_n;
  const int g = t / per_group;
  const int gm = min(kGroupM, tiles_m - g * kGroupM);
  const int r = t - g * per_group;
  out.n_blk = r / gm;
  out.m_blk = g * kGroupM + (r - out.n_blk * gm);
  // all-gather mode: start with the row tiles whose source is this rank, they need no wait
  if (p.a_gather) out.m_blk = (out.m_blk + (p.rank * p.a_rows_per_rank) / (kBM * kG)) % tiles_m;
  // reduce-scatter mode: start with the row tiles this rank owns, then the next rank's, ... so
  // that at any time every rank stores to a different owner; with one order for all ranks
  // everybody would send to rank 0 first, then to rank 1, ... and each owner's link in turn
  // would carry the whole traffic while the others idle (o_proj of 32768 tokens on 8 GPUs:
  // 1.20 ms with one order, 0.70 ms rotated)
  if (p.epilogue == kEpiPartialF32 && p.world > 1)
    out.m_blk = (out.m_blk + static_cast<int>((static_cast<long long>(p.rank) * p.rows_per_rank) / (kBM * kG))) % tiles_m;
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory"); }

__device__ __forceinline__ void tmem_ld_wait_dep(uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),
        "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]),
        "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]),
        "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]),
        "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
      :
      : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

struct RowCtx {
  float neg_lse2;  // -lse * log2(e)
  float gs;        // upstream gradient * scale
  long long tgt;   // target column inside this shard (or out of range)
};

// Layout of the reduce-scatter staging buffer of one owner rank. A partial tile is not stored
// row-major: the 32 rows x 64 columns that one epilogue warp stores at a time are one contiguous
// 4 KiB fragment, [slice][row block][column tile][row quarter][column half][column pair], so
// that a warp's stores to the owner (another GPU for 7/8 of the tiles at TP = 8) cover whole
// contiguous kilobytes instead of 128-byte pieces 8 KiB apart (which reached 160 GB/s over
// NVLink). The reduce tail reads with the same function.
constexpr int kFragElems = 32 * 64;                  // bf16 elements of a fragment
constexpr int kTileElems = kBM * kBN;                // 16 fragments
__device__ __forceinline__ long long stage_offset(int slice, int rblks, int tiles_n, int lr, int col) {
  const int rblk = lr / kBM, r = lr - rblk * kBM;
  const int nb = col / kBN, c = col - nb * kBN;
  const int frag = ((r >> 5) * 2 + (c >> 7)) * 2 + ((c >> 6) & 1);
  return ((static_cast<long long>(slice) * rblks + rblk) * tiles_n + nb) * kTileElems +
         static_cast<long long>(frag) * kFragElems + (r & 31) * 64 + (c & 63);
}

// Store 32 consecutive accumulator columns of the warp's 32 rows. Each lane holds one row
// (that is how tcgen05.ld hands out TMEM lanes); the values are transposed through a padded
// shared-memory tile so that the global stores are whole 64 / 128-byte row segments: eight
// (fp32) or four (bf16) lanes cover one row segment contiguously. This matters most for the
// partial tiles that go to another GPU, where every store instruction becomes NVLink packets.
//
// bf16 outputs are staged two 32-column groups at a time (`half` 0 then 1) and stored after the
// second, so that a row segment is 128 bytes: a whole line for the peer's memory system instead
// of two half-line writes (64-byte segments reached about 140 GB/s over NVLink).
__device__ __forceinline__ void store_group_warp(const GemmParams& p, const uint32_t (&v)[32], uint32_t* wbuf,
                                                 long long row_w0, int col, int slice_global, const RowCtx& rc,
                                                 int lane, int half) {
  const bool f32 = p.epilogue == kEpiStoreF32;
  if (f32 && col >= p.n) return;  // uniform over the warp
  uint32_t* mine = wbuf + lane * 33 + (f32 ? 0 : half * 16);
  if (f32) {
#pragma unroll
    for (int j = 0; j < 32; ++j) mine[j] = v[j];
  } else if (p.epilogue == kEpiLogitsGrad) {
    const float s2 = p.scale * 1.4426950408889634f;
    float d[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float pr = ex2_approx(__fmaf_rn(__uint_as_float(v[j]), s2, rc.neg_lse2));
      const float one = (col + j == rc.tgt) ? 1.f : 0.f;
      d[j] = __fmul_rn(rc.gs, __fsub_rn(one, pr));
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) mine[j] = pack_bf16(d[2 * j], d[2 * j + 1]);
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) mine[j] = pack_bf16(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
  }
  __syncwarp();
  if (!f32) {
    if (half == 0) return;   // stored together with the next group
    col -= 32;               // first column of the staged pair of groups
    if (col >= p.n) return;  // uniform over the warp
  }
  if (f32) {
    float* base = static_cast<float*>(p.c) + row_w0 * p.ldc + col;
    const long long ld = p.ldc;
    const int c = lane & 7, r0 = lane >> 3;
    const bool col_ok = col + c * 4 + 4 <= p.n;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = r0 + 4 * it;
      if (col_ok && row_w0 + r < p.m) {
        const uint32_t* src = wbuf + r * 33 + c * 4;
        *reinterpret_cast<uint4*>(base + r * ld + c * 4) = make_uint4(src[0], src[1], src[2], src[3]);
      }
    }
  } else {
    __nv_bfloat16* base;
    long long ld;
    if (p.epilogue == kEpiPartialF32) {
      const int owner = static_cast<int>(row_w0 / p.rows_per_rank);
      const int lr = static_cast<int>(row_w0 - static_cast<long long>(owner) * p.rows_per_rank);
      base = static_cast<__nv_bfloat16*>(p.stage[owner]) +
             stage_offset(slice_global, p.rows_per_rank / kBM, (p.n + kBN - 1) / kBN, lr, col);
      ld = 64;  // rows of a fragment are 64 elements apart
    } else {
      base = static_cast<__nv_bfloat16*>(p.c) + row_w0 * p.ldc + col;
      ld = p.ldc;
    }
    const int c = lane & 7, r0 = lane >> 3;   // eight lanes cover the 128 bytes of one row
    const bool col_ok = col + c * 8 + 8 <= p.n;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = r0 + 4 * it;
      if (col_ok && row_w0 + r < p.m) {
        const uint32_t* src = wbuf + r * 33 + c * 4;
        *reinterpret_cast<uint4*>(base + r * ld + c * 8) = make_uint4(src[0], src[1], src[2], src[3]);
      }
    }
  }
  __syncwarp();
}

__device__ __forceinline__ float4 ld_f4_sys(const float* p) {
  return ld_relaxed_sys_f4(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles = smem_raw + (tiles_addr - raw_addr);
  Control* ctl = reinterpret_cast<Control*>(tiles + kTileBytes);
  uint32_t* epi_buf = reinterpret_cast<uint32_t*>(tiles + kTileBytes + 512);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair_id = blockIdx.x / kG;
  const int n_pairs = gridDim.x / kG;
  const int tiles_m = (p.m + kBM * kG - 1) / (kBM * kG);
  const int tiles_n = (p.n + kBN - 1) / kBN;
  const int n_units = tiles_m * tiles_n * p.k_slices;
  const int k_per_slice = p.k / p.k_slices;
  const int num_kb = (k_per_slice + kBK - 1) / kBK;

  WaitCtx wctx{&ctl->abort_flag, p.status, p.timeout_ns};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->tfull[b]), 1);
      mbar_init(smem_u32(&ctl->tempty[b]), kEpiWarps * kG);
    }
    ctl->abort_flag = 0;
    fence_mbar_init_cluster();
  }
  if (warp == kWarpMma) {
    tmem_alloc<kG>(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish<kG>();
  }
  if (warp == kWarpTma && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair_id; u < n_units && ok; u += n_pairs) {
        Unit un;
        decode_unit(p, tiles_m, tiles_n, u, un);
        const int row0 = un.m_blk * (kBM * kG) + static_cast<int>(cta_rank) * kBM;
        const int col0 = un.n_blk * kBN + static_cast<int>(cta_rank) * (kBN / kG);
        const int kbase = un.slice * k_per_slice;
        if (p.a_gather) {
          // rows of another rank become readable when that rank's push has been flagged
          const int src = row0 / p.a_rows_per_rank;
          const int blk = (row0 - src * p.a_rows_per_rank) / kBM;
          const int blocks = p.a_rows_per_rank / kBM;
          if (row0 < p.m)
            ok = flag_wait_bounded(p.a_flags[p.rank] + static_cast<size_t>(src) * blocks + blk, p.epoch, wctx,
                                   kWGatherFlag, src * 65536 + blk);
          if (!ok) break;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(smem_u32(&ctl->empty[stage]), phase ^ 1u, wctx, kWProducer, stage);
          if (!ok) break;
          const uint32_t a_dst = tiles_addr + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const uint32_t full = smem_u32(&ctl->full[stage]);
          if (leader) mbar_arrive_expect_tx(full, kTxBytes);
          const uint32_t full_leader = mapa_u32(full, 0);
          const int k0 = kbase + kb * kBK;
          if (p.a_major == 0) {
            tma_load_2d_pair(a_dst, &tm_a, k0, row0, full_leader);
          } else {
            tma_load_2d_pair(a_dst, &tm_a, row0, k0, full_leader);
            tma_load_2d_pair(a_dst + 8192, &tm_a, row0 + 64, k0, full_leader);
          }
          if (p.b_major == 0) {
            tma_load_2d_pair(b_dst, &tm_b, k0, col0, full_leader);
          } else {
            tma_load_2d_pair(b_dst, &tm_b, col0, k0, full_leader);
            tma_load_2d_pair(b_dst + 8192, &tm_b, col0 + 64, k0, full_leader);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && leader) {
      const uint32_t idesc = umma_idesc_bf16_f32(kBM * kG, kBN) | (static_cast<uint32_t>(p.a_major) << 15) |
                             (static_cast<uint32_t>(p.b_major) << 16);
      const uint32_t a_step = p.a_major == 0 ? 2u : 128u;  // descriptor units (16 B) per K=16
      const uint32_t b_step = p.b_major == 0 ? 2u : 128u;
      int stage = 0;
      uint32_t phase = 0;
      int abuf = 0;
      uint32_t aphase = 0;
      bool ok = true;
      for (int u = pair_id; u < n_units && ok; u += n_pairs) {
        ok = mbar_wait_bounded(smem_u32(&ctl->tempty[abuf]), aphase ^ 1u, wctx, kWMmaTmem, abuf);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(abuf * kBN);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(smem_u32(&ctl->full[stage]), phase, wctx, kWMmaFull, stage);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = tiles_addr + stage * kStageBytes;
          const uint64_t a_desc = p.a_major == 0 ? umma_desc_k_sw128(a_addr) : umma_desc_mn_sw128(a_addr);
          const uint64_t b_desc =
              p.b_major == 0 ? umma_desc_k_sw128(a_addr + kABytes) : umma_desc_mn_sw128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            umma_bf16<kG>(d_tmem, a_desc + a_step * k, b_desc + b_step * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit<kG>(smem_u32(&ctl->empty[stage]));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit<kG>(smem_u32(&ctl->tfull[abuf]));
        abuf ^= 1;
        if (abuf == 0) aphase ^= 1u;
      }
    }
  } else if (warp == kWarpPub) {
    // (spare warp: the flags of the partial tiles are raised by the epilogue warps once, after
    // the CTA's last unit; a system-scope fence and a flag per unit made every unit wait for the
    // round trip of its own peer stores: 1.47 ms against 1.20 ms for o_proj of 32768 tokens)
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-7)
    // Warp w reads TMEM lanes 32 * (w & 3) .. +31 (its rows) and columns 128 * (w >> 2) .. +127.
    // The unit loop has no CTA-wide barrier: a warp whose wait runs out simply leaves it. The
    // named barriers of the copy and reduce phases are reached by all 256 threads.
    const int tid = threadIdx.x;
    const int wq = warp & 3, wh = warp >> 2;
    bool ok = true;

    if (p.a_gather) {
      // ---- all-gather: push this rank's rows of A into every peer's gather buffer, one
      // 128-row block at a time, then raise the block's flag on that peer.
      const int blocks = p.a_rows_per_rank / kBM;
      const int vec_per_row = p.k / 8;  // 16-byte vectors
      const uint4* src = static_cast<const uint4*>(p.a_local);
      const long long nv = static_cast<long long>(kBM) * vec_per_row;
      // work item = (destination, 128-row block), destination-major starting with this rank, so
      // the local copy (which this rank's own GEMM needs first) leaves first
      for (int it = blockIdx.x; it < blocks * p.world; it += gridDim.x) {
        const int d = it / blocks, blk = it - d * blocks;
        const int dst_rank = (p.rank + d) % p.world;
        const long long v0 = static_cast<long long>(blk) * nv;
        uint4* dst = static_cast<uint4*>(p.a_bufs[dst_rank]) +
                     static_cast<long long>(p.rank) * p.a_rows_per_rank * vec_per_row + v0;
        constexpr int kS = kEpiThreads;
        for (long long i = tid; i < nv; i += 4 * kS) {
          // four independent 16-byte copies in flight per thread
          uint4 t0 = src[v0 + i], t1, t2, t3;
          const bool b1 = i + kS < nv, b2 = i + 2 * kS < nv, b3 = i + 3 * kS < nv;
          if (b1) t1 = src[v0 + i + kS];
          if (b2) t2 = src[v0 + i + 2 * kS];
          if (b3) t3 = src[v0 + i + 3 * kS];
          dst[i] = t0;
          if (b1) dst[i + kS] = t1;
          if (b2) dst[i + 2 * kS] = t2;
          if (b3) dst[i + 3 * kS] = t3;
        }
        epi_bar();
        if (tid == 0) {
          __threadfence_system();
          st_release_sys_u32(p.a_flags[dst_rank] + static_cast<size_t>(p.rank) * blocks + blk, p.epoch);
        }
      }
    }

    int abuf = 0;
    uint32_t aphase = 0;
    const uint32_t tempty_leader = mapa_u32(smem_u32(&ctl->tempty[0]), 0);
    for (int u = pair_id; u < n_units; u += n_pairs) {
      Unit un;
      decode_unit(p, tiles_m, tiles_n, u, un);
      const long long row_w0 = static_cast<long long>(un.m_blk) * (kBM * kG) + cta_rank * kBM + wq * 32;
      const long long row = row_w0 + lane;
      const bool mine = mbar_wait_bounded(smem_u32(&ctl->tfull[abuf]), aphase, wctx, kWEpi, abuf);
      ok = __all_sync(0xffffffffu, mine) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(wq * 32) << 16) +
                            static_cast<uint32_t>(abuf * kBN + wh * (kBN / 2));
      const int col0 = un.n_blk * kBN + wh * (kBN / 2);
      const int slice_global = p.slice_base + un.slice;
      RowCtx rc = {0.f, 0.f, -1};
      if (p.epilogue == kEpiLogitsGrad && row < p.m) {
        rc.neg_lse2 = __fmul_rn(-p.row_lse[row], 1.4426950408889634f);
        rc.gs = __fmul_rn(p.row_g[row], p.scale);
        rc.tgt = p.row_ids[row] - p.col_offset;
      }
      uint32_t* wbuf = epi_buf + warp * kEpiBufWords;
      uint32_t va[32], vb[32];
      tmem_ld_32x32(trow, va);
      tmem_ld_wait_dep(va);
#pragma unroll
      for (int g = 0; g < kBN / 64; g += 2) {
        __syncwarp();
        tmem_ld_32x32(trow + (g + 1) * 32, vb);
        store_group_warp(p, va, wbuf, row_w0, col0 + g * 32, slice_global, rc, lane, 0);
        __syncwarp();
        tmem_ld_wait_dep(vb);
        if (g + 2 < kBN / 64) tmem_ld_32x32(trow + (g + 2) * 32, va);
        store_group_warp(p, vb, wbuf, row_w0, col0 + (g + 1) * 32, slice_global, rc, lane, 1);
        __syncwarp();
        if (g + 2 < kBN / 64) tmem_ld_wait_dep(va);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + static_cast<uint32_t>(abuf) * 8u);
      abuf ^= 1;
      if (abuf == 0) aphase ^= 1u;
    }

    if (p.epilogue == kEpiPartialF32) {
      // Publish the partial tiles: every thread makes its own stores visible system-wide, the
      // CTA meets, then the flags of all units this CTA computed are raised (the owners read
      // them in their reduce tails, which start after their own last unit anyway).
      __threadfence_system();
      epi_bar();  // every epilogue thread gets here, whether or not its loop ran to the end
      if (ctl->abort_flag) ok = false;
      if (ok) {
        const int rblks = p.rows_per_rank / kBM;
        int k = 0;
        for (int u = pair_id; u < n_units; u += n_pairs, ++k) {
          if ((k % kEpiThreads) != tid) continue;
          Unit un;
          decode_unit(p, tiles_m, tiles_n, u, un);
          const long long row0 = static_cast<long long>(un.m_blk) * (kBM * kG) + cta_rank * kBM;
          if (row0 < p.m) {
            const int owner = static_cast<int>(row0 / p.rows_per_rank);
            const int rblk = static_cast<int>((row0 - static_cast<long long>(owner) * p.rows_per_rank) / kBM);
            st_release_sys_u32(p.flags[owner] + (static_cast<size_t>(p.slice_base + un.slice) * rblks + rblk) * tiles_n +
                                   un.n_blk,
                               p.epoch);
          }
        }
      }
    }
    if (p.epilogue == kEpiPartialF32 && ok && p.out != nullptr) {
      // ---- reduce-scatter tail (skipped when the caller only wants the partials staged): the rows this rank owns, slices combined by a balanced tree
      const int rblks = p.rows_per_rank / kBM;
      const int items = rblks * tiles_n;
      const int rows_valid = min(p.rows_per_rank, p.m - p.rank * p.rows_per_rank);
      for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int rblk = it / tiles_n, nb = it - rblk * tiles_n;
        if (rblk * kBM >= rows_valid) continue;  // block past the end of the matrix: nobody writes it
        if (tid < p.total_slices)
          flag_wait_bounded(p.flags[p.rank] + (static_cast<size_t>(tid) * rblks + rblk) * tiles_n + nb, p.epoch, wctx,
                            kWReduceFlag, it);
        epi_bar();
        if (ctl->abort_flag) break;
        const int ncols = min(kBN, p.n - nb * kBN);
        const int vec_per_row = ncols / 8;  // 8 bf16 = 16 bytes
        const size_t slice_stride = static_cast<size_t>(rblks) * tiles_n * kTileElems;
#pragma unroll 2
        for (int i = tid; i < kBM * vec_per_row; i += kEpiThreads) {
          const int r = i / vec_per_row, c8 = i - r * vec_per_row;
          const int lr = rblk * kBM + r;
          if (lr >= rows_valid) continue;
          const size_t off = static_cast<size_t>(lr) * p.n + nb * kBN + c8 * 8;  // in out / residual (row-major)
          const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(p.stage[p.rank]) +
                                      stage_offset(0, rblks, tiles_n, lr, nb * kBN + c8 * 8);
          float4 lo[8], hi[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (q < p.total_slices) {
              // weak L2 loads: the acquire on the flags (and the barrier) orders them after the peers'
              // stores, and unlike system-scope strong loads they pipeline
              const float4 raw = __ldcg(reinterpret_cast<const float4*>(base + q * slice_stride));
              const uint32_t w0 = __float_as_uint(raw.x), w1 = __float_as_uint(raw.y), w2 = __float_as_uint(raw.z),
                             w3 = __float_as_uint(raw.w);
              lo[q] = make_float4(__uint_as_float(w0 << 16), __uint_as_float(w0 & 0xFFFF0000u),
                                  __uint_as_float(w1 << 16), __uint_as_float(w1 & 0xFFFF0000u));
              hi[q] = make_float4(__uint_as_float(w2 << 16), __uint_as_float(w2 & 0xFFFF0000u),
                                  __uint_as_float(w3 << 16), __uint_as_float(w3 & 0xFFFF0000u));
            } else {
              lo[q] = make_float4(0.f, 0.f, 0.f, 0.f);
              hi[q] = lo[q];
            }
          }
          float4 a0 = add4(add4(add4(lo[0], lo[1]), add4(lo[2], lo[3])), add4(add4(lo[4], lo[5]), add4(lo[6], lo[7])));
          float4 a1 = add4(add4(add4(hi[0], hi[1]), add4(hi[2], hi[3])), add4(add4(hi[4], hi[5]), add4(hi[6], hi[7])));
          if (p.residual) {
            // residual add in bf16 arithmetic order: round the GEMM result first, as a separate
            // bf16 linear + add would
            const uint4 rr = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.residual) + off);
            auto addr = [](float g, uint32_t rbits) {
              return __fadd_rn(__bfloat162float(__float2bfloat16_rn(g)), __uint_as_float(rbits));
            };
            a0.x = addr(a0.x, rr.x << 16);
            a0.y = addr(a0.y, rr.x & 0xFFFF0000u);
            a0.z = addr(a0.z, rr.y << 16);
            a0.w = addr(a0.w, rr.y & 0xFFFF0000u);
            a1.x = addr(a1.x, rr.z << 16);
            a1.y = addr(a1.y, rr.z & 0xFFFF0000u);
            a1.z = addr(a1.z, rr.w << 16);
            a1.w = addr(a1.w, rr.w & 0xFFFF0000u);
          }
          uint4 o;
          o.x = pack_bf16(a0.x, a0.y);
          o.y = pack_bf16(a0.z, a0.w);
          o.z = pack_bf16(a1.x, a1.y);
          o.w = pack_bf16(a1.z, a1.w);
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + off) = o;
        }
      }
    }
  }

  // ------------------------------------------------------------------ common exit
  if (ctl->abort_flag) {
    st_shared_cluster_u32(mapa_u32(smem_u32(&ctl->abort_flag), cta_rank ^ 1u), 1u);
    drain_in_flight();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == kWarpMma) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<kG>(tmem_base, 512);
  }
}

int max_ctas(int num_sms) {
  static int cached = 0;
  if (cached > 0) return cached;
  if (cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(num_sms / 2 * 2));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_bf16_kernel, &cfg) != cudaSuccess || clusters <= 0) {
    cudaGetLastError();
    clusters = num_sms / 2;
  }
  int n = clusters * 2;
  if (n > num_sms / 2 * 2) n = num_sms / 2 * 2;
  cached = n;
  return n;
}

}  // namespace

// Shared by the plain entry point and the tensor-parallel ones (tp_gemm.cu): build the
// tensor maps for the operand layouts in `p` and launch.
int gemm_launch(const void* a, long long lda, const void* b, long long ldb, const GemmParams& p, int num_sms,
                bool full_grid, cudaStream_t stream) {
  if (p.m <= 0 || p.n <= 0 || p.k <= 0) return 0;
  if (p.k % 8 != 0 || p.n % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return -1;
  if (p.k_slices < 1 || p.k % p.k_slices != 0 || (p.k_slices > 1 && (p.k / p.k_slices) % kBK != 0)) return -2;
  if (p.a_major == 1 && p.m % 8 != 0) return -3;
  CUtensorMap tm_a, tm_b;
  int rc;
  if (p.a_major == 0)
    rc = make_tmap_2d_16bit_sw128(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, p.m, p.k, lda, kBM, kBK);
  else
    rc = make_tmap_2d_16bit_sw128(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, p.k, p.m, lda, kBK, 64);
  if (rc != 0) return -20 + rc;
  if (p.b_major == 0)
    rc = make_tmap_2d_16bit_sw128(&tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b, p.n, p.k, ldb, kBN / kG, kBK);
  else
    rc = make_tmap_2d_16bit_sw128(&tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b, p.k, p.n, ldb, kBK, 64);
  if (rc != 0) return -40 + rc;
  int ctas = max_ctas(num_sms);
  if (ctas <= 0) return -10;
  const int tiles_m = (p.m + kBM * kG - 1) / (kBM * kG), tiles_n = (p.n + kBN - 1) / kBN;
  const int units = tiles_m * tiles_n * p.k_slices;
  if (!full_grid && units * kG < ctas) ctas = units * kG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_kernel, tm_a, tm_b, p);
  if (e != cudaSuccess) {
    fprintf(stderr, "[kernel_align_b200] gemm launch failed: %s\n", cudaGetErrorString(e));
    return -11;
  }
  return 0;
}

}  // namespace ka

extern "C" int ka_gemm_bf16(const void* a, long long lda, int a_major, const void* b, long long ldb, int b_major,
                            void* c, long long ldc, int out_f32, int m, int n, int k, int* status, int num_sms,
                            unsigned long long timeout_ns, void* stream) {
  ka::GemmParams p = {};
  p.m = m;
  p.n = n;
  p.k = k;
  p.a_major = a_major ? 1 : 0;
  p.b_major = b_major ? 1 : 0;
  p.epilogue = out_f32 ? ka::kEpiStoreF32 : ka::kEpiStoreBf16;
  p.c = c;
  p.ldc = ldc;
  p.k_slices = 1;
  p.total_slices = 1;
  p.world = 1;
  p.status = status;
  p.timeout_ns = timeout_ns;
  return ka::gemm_launch(a, lda, b, ldb, p, num_sms, false, static_cast<cudaStream_t>(stream));
}

extern "C" int ka_lmhead_logits_grad(const void* hidden, const void* weight, const long long* ids, const float* lse,
                                     const float* g, void* d_logits, long long ldd, int m, int n, int k, float scale,
                                     int col_offset, int* status, int num_sms, unsigned long long timeout_ns,
                                     void* stream) {
  ka::GemmParams p = {};
  p.m = m;
  p.n = n;
  p.k = k;
  p.epilogue = ka::kEpiLogitsGrad;
  p.c = d_logits;
  p.ldc = ldd;
  p.k_slices = 1;
  p.total_slices = 1;
  p.world = 1;
  p.row_lse = lse;
  p.row_g = g;
  p.row_ids = ids;
  p.scale = scale;
  p.col_offset = col_offset;
  p.status = status;
  p.timeout_ns = timeout_ns;
  return ka::gemm_launch(hidden, k, weight, k, p, num_sms, false, static_cast<cudaStream_t>(stream));
}
