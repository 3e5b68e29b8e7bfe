// Fused LM-head + log-probability kernel for sm_100a.
//
//   logp[r] = scale * <H[r,:], W[ids[r],:]>  -  logsumexp_v( scale * <H[r,:], W[v,:]> )
//
// H is [M, K] bf16 (row-major), W is this rank's vocabulary shard [V_local, K] bf16
// (row-major); the [M, V] logits are never written to memory. bf16 tiles are brought in by
// TMA, multiplied by tcgen05.mma into fp32 accumulators in TMEM, and the epilogue warps keep
// a running (max, sum-exp, target-logit) per row straight out of TMEM.
//
// Reproducibility contract (per row, bitwise):
//   * the global vocabulary is cut into 8 canonical slices of ceil(V/8) columns, each slice
//     into sub-slices of 1792 columns, each sub-slice into 256-column MMA tiles;
//   * one thread owns one row of one sub-slice and folds its tiles left to right;
//   * sub-slices of a slice are merged left to right, the 8 slices by a balanced binary
//     tree. A rank that holds 8/N contiguous slices evaluates a whole subtree locally and the
//     top log2(N) levels after the exchange, so 1, 2, 4 and 8 GPUs run the same arithmetic.
//   Nothing depends on M, on which CTA processed a tile, or on arrival order.
//
// Multi-GPU: after a rank has merged its slices for a 128-row block it stores the block's
// (max, sum-exp, target) triples into every peer's exchange buffer with plain peer stores,
// then releases a per-(source rank, block) flag; each rank finishes the blocks it pushed by
// waiting (bounded) for the other ranks' flags and running the top of the tree.
//
// Row-sharded input (gather mode): a rank may hold only its 1/N of the rows. A seventh warp then
// pushes the rank's rows of the panel (and their ids) into every peer's gather arena with bulk
// copies staged through shared memory, 32 rows at a time, and raises a flag per (source rank,
// 128-row block) when a block is complete; the TMA producer waits (bounded) for the flag of a
// remote block and loads it from this GPU's own arena. Every rank walks its own rows first, so
// the transfer hides behind the first 1/N of the panel's tensor work. The arithmetic per row
// is the one above: the results equal the single-GPU ones bit for bit.
//
// Replaces the reference's `torch.matmul` + `SamplerBackend.compute_logp`
// (rl_engine/kernels/sampling.py:91-112), which materialises [G, L, V] logits twice.

#include <cfloat>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cuda_bf16.h>
#include <math_constants.h>
#include <mutex>

#include "common/bounded_wait.cuh"
#include "common/ptx.cuh"
#include "common/tmap.cuh"
#include "fused_lmhead_logp.h"

namespace ka {
namespace {

constexpr int kBM = 128;         // rows per CTA (TMEM lanes)
constexpr int kBN = 256;         // columns per MMA tile
constexpr int kBK = 64;          // bf16 elements per 128-byte swizzled row
constexpr int kUmmaK = 16;       // K per tcgen05.mma of kind::f16
constexpr int kSubCols = 1792;   // columns per canonical sub-slice (7 tiles)
constexpr int kSlices = 8;       // canonical slices of the global vocabulary
constexpr int kThreads = 224;    // warps 0-3 epilogue, 4 TMA producer, 5 MMA issuer, 6 row pusher
constexpr int kPushChunk = 8192; // bytes per staged bulk copy of the row pusher (two buffers)
constexpr int kPushRows = 32;    // rows per push unit
constexpr int kMaxDeferred = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int G>
struct Cfg {
  static constexpr int kBRows = kBN / G;                 // W rows each CTA loads per stage
  static constexpr int kABytes = kBM * kBK * 2;          // 16 KiB
  static constexpr int kBBytes = kBRows * kBK * 2;       // 32 KiB (G=1) or 16 KiB (G=2)
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (G == 1) ? 4 : 6;
  static constexpr int kTxBytes = kStageBytes * G;       // bytes counted on the leader's barrier
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kSmemBytes = kTileBytes + 1024 /*alignment*/ + 2048 /*control*/;
  static constexpr int kSmemBytesGather = kSmemBytes + 2 * kPushChunk;  // + the pusher's staging
};

struct Control {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint64_t pbar[2];
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
  int n_deferred;
  uint16_t deferred[kMaxDeferred];
};
static_assert(sizeof(Control) <= 2048, "control block too large");

enum Where : int {
  kWhereProducerEmpty = 1,
  kWhereMmaFull = 2,
  kWhereMmaTmemEmpty = 3,
  kWhereEpiTmemFull = 4,
  kWherePeerFlag = 5,
  kWhereGatherFlag = 6,
  kWherePushLoad = 7
};

struct Item {
  int m_tile;
  int chunk;
  int col_begin;
  int col_end;
  int n_tiles;
};

__device__ __forceinline__ void decode_item(const LogpParams& p, int i, Item& it) {
  // Work order. A wave of CTAs covers mg row tiles x cg sub-slices. Either the row-tile group is
  // the outer loop and its rows of H stay in L2 while all of W streams past once per group
  // (c_outer = 0), or the group of sub-slices is the outer loop and its columns of W stay in
  // L2 while all row tiles of the panel stream past once per group (c_outer = 1: less memory
  // traffic when this rank's W is small, as with a vocabulary sharded eight ways).
  int g, h, mg_sz, cg_sz, r2;
  if (p.c_outer) {
    const int full = p.n_mtiles * p.cg;          // items of a full group of sub-slices
    h = i / full;
    cg_sz = min(p.cg, p.n_chunks - h * p.cg);
    const int r = i - h * full;
    g = r / (p.mg * cg_sz);
    mg_sz = min(p.mg, p.n_mtiles - g * p.mg);
    r2 = r - g * p.mg * cg_sz;
  } else {
    const int per_group = p.mg * p.n_chunks;
    g = i / per_group;
    mg_sz = min(p.mg, p.n_mtiles - g * p.mg);
    const int r = i - g * per_group;
    h = r / (mg_sz * p.cg);
    cg_sz = min(p.cg, p.n_chunks - h * p.cg);
    r2 = r - h * mg_sz * p.cg;
  }
  // Which of the two indices runs fastest over consecutive CTAs decides which CTAs are
  // neighbours: the sub-slices of one row tile (m_fast = 0), or the row tiles of one sub-slice.
  int m_local, c_local;
  if (p.m_fast) {
    c_local = r2 / mg_sz;
    m_local = r2 - c_local * mg_sz;
  } else {
    m_local = r2 / cg_sz;
    c_local = r2 - m_local * cg_sz;
  }
  it.m_tile = g * p.mg + m_local + p.mt_rot;
  if (it.m_tile >= p.n_mtiles) it.m_tile -= p.n_mtiles;
  // Schedule position -> (slice, sub-slice): sub-slice major, so that the sub-slices that run
  // side by side have the same position inside their slices and therefore the same number of
  // tiles; CTAs that share W tiles through L2 then stay in step. The partials are stored
  // slice major (chunk = slice * sub + sub-slice), which is what the merge walks.
  const int sched = h * p.cg + c_local;
  const int q = sched / p.n_slices_local;
  const int sl = sched - q * p.n_slices_local;
  it.chunk = sl * p.sub + q;
  const int slice_begin = sl * p.vs;
  const int slice_end = min(slice_begin + p.vs, p.v_local);
  it.col_begin = slice_begin + q * kSubCols;
  it.col_end = min(it.col_begin + kSubCols, slice_end);
  it.n_tiles = it.col_end > it.col_begin ? (it.col_end - it.col_begin + kBN - 1) / kBN : 0;
}

// (m, l) describes sum_j exp(x_j) = l * exp(scale * m) with m the running maximum of the raw
// accumulator values. s2 = scale * log2(e). The arithmetic is spelled with explicit
// intrinsics so that every call site rounds identically.
__device__ __forceinline__ void merge2(float& m, float& l, float m2, float l2, float s2) {
  const float mn = fmaxf(m, m2);
  const float a = (m == -CUDART_INF_F) ? 0.f : ex2_approx(__fmul_rn(__fsub_rn(m, mn), s2));
  const float b = (m2 == -CUDART_INF_F) ? 0.f : ex2_approx(__fmul_rn(__fsub_rn(m2, mn), s2));
  l = __fadd_rn(__fmul_rn(l, a), __fmul_rn(l2, b));
  m = mn;
}

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

// Fold 32 consecutive columns of one row into the running state.
//   col0   first column of the group inside the tile
//   valid  number of real columns in the tile (the rest is masked out)
//   tcol   target column inside the tile, or a negative / large value if not in the tile
__device__ __forceinline__ void fold32(const uint32_t (&v)[32], int col0, int valid, int tcol,
                                       float s2, float& m, float& l, float& t) {
  float x[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]);
  if (col0 + 32 > valid) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j >= valid) x[j] = -CUDART_INF_F;
  }
  const int tj = tcol - col0;
  if (static_cast<unsigned>(tj) < 32u) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j == tj) t = x[j];
  }
  float c0 = fmaxf(x[0], x[1]), c1 = fmaxf(x[2], x[3]), c2 = fmaxf(x[4], x[5]),
        c3 = fmaxf(x[6], x[7]);
#pragma unroll
  for (int j = 8; j < 32; j += 8) {
    c0 = fmaxf(c0, fmaxf(x[j], x[j + 1]));
    c1 = fmaxf(c1, fmaxf(x[j + 2], x[j + 3]));
    c2 = fmaxf(c2, fmaxf(x[j + 4], x[j + 5]));
    c3 = fmaxf(c3, fmaxf(x[j + 6], x[j + 7]));
  }
  const float mn = fmaxf(m, fmaxf(fmaxf(c0, c1), fmaxf(c2, c3)));
  // Exponents are taken relative to R(m) = round(m * s2); the running sum is rescaled by
  // 2^(R(m_old) - R(m_new)), which is exactly 1 when the maximum did not move and 0 when
  // m_old is -inf.
  const float neg_old = __fmul_rn(-m, s2);
  const float neg = __fmul_rn(-mn, s2);
  const float corr = ex2_approx(__fsub_rn(neg, neg_old));
  float s0 = 0.f, s1 = 0.f, s2a = 0.f, s3 = 0.f;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    s0 = __fadd_rn(s0, ex2_approx(__fmaf_rn(x[j], s2, neg)));
    s1 = __fadd_rn(s1, ex2_approx(__fmaf_rn(x[j + 1], s2, neg)));
    s2a = __fadd_rn(s2a, ex2_approx(__fmaf_rn(x[j + 2], s2, neg)));
    s3 = __fadd_rn(s3, ex2_approx(__fmaf_rn(x[j + 3], s2, neg)));
  }
  const float gs = __fadd_rn(__fadd_rn(s0, s1), __fadd_rn(s2a, s3));
  l = __fmaf_rn(l, corr, gs);
  m = mn;
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Merge this rank's sub-slice partials of one row: chains inside each slice, then the local
// subtree. Leaves (m_out, l_out) as the rank's partial.
__device__ __forceinline__ void merge_local(const LogpParams& p, int rp, float s2, float& m_out,
                                            float& l_out) {
  float lm[kSlices], ll[kSlices];
#pragma unroll
  for (int sl = 0; sl < kSlices; ++sl) {
    lm[sl] = -CUDART_INF_F;
    ll[sl] = 0.f;
  }
#pragma unroll
  for (int sl = 0; sl < kSlices; ++sl) {
    if (sl < p.n_slices_local) {
      const size_t base = static_cast<size_t>(sl) * p.sub;
      float m = __ldcg(p.part_m + (base + 0) * p.ldp + rp);
      float l = __ldcg(p.part_l + (base + 0) * p.ldp + rp);
      for (int q = 1; q < p.sub; ++q) {
        const float m2 = __ldcg(p.part_m + (base + q) * p.ldp + rp);
        const float l2 = __ldcg(p.part_l + (base + q) * p.ldp + rp);
        merge2(m, l, m2, l2, s2);
      }
      lm[sl] = m;
      ll[sl] = l;
    }
  }
#pragma unroll
  for (int w = kSlices; w > 1; w >>= 1) {
    if (w <= p.n_slices_local) {
#pragma unroll
      for (int i = 0; i < w / 2; ++i) {
        float m = lm[2 * i], l = ll[2 * i];
        merge2(m, l, lm[2 * i + 1], ll[2 * i + 1], s2);
        lm[i] = m;
        ll[i] = l;
      }
    }
  }
  m_out = lm[0];
  l_out = ll[0];
}

__device__ __forceinline__ void write_result(const LogpParams& p, long long row, float m, float l, float t,
                                             bool has_t, bool id_ok) {
  // lse = scale*m + ln(l); logp = scale*t - lse
  const float lse = __fmaf_rn(lg2_approx(l), kLn2, __fmul_rn(m, p.scale));
  if (p.lse) p.lse[row] = lse;
  p.logp[row] = (id_ok && has_t) ? __fsub_rn(__fmul_rn(t, p.scale), lse) : 0.f;
}

// Where the rows of a 128-row block of the panel come from and go to.
struct RowRef {
  int src;            // rank that holds the row
  int j;              // row inside the source's part of the panel (gather) or inside the panel
  bool ok;            // a real row
  long long out_row;  // index into logp / lse, or -1 if this rank does not write the row
};

__device__ __forceinline__ RowRef row_ref(const LogpParams& p, int blk, int tid) {
  RowRef r;
  if (p.gather) {
    r.src = blk / p.bps;
    r.j = (blk - r.src * p.bps) * kBM + tid;
    r.ok = r.j < p.rows_local;
    const long long lr = static_cast<long long>(p.local_row_begin) + r.j;
    r.out_row = p.out_all ? static_cast<long long>(r.src) * p.m_local + lr : (r.src == p.rank ? lr : -1);
  } else {
    r.src = p.rank;
    r.j = blk * kBM + tid;
    r.ok = r.j < p.rows;
    r.out_row = static_cast<long long>(p.row_begin) + r.j;
  }
  return r;
}

// Token id of a row. A remote row's id sits in this rank's gather arena and may only be read
// once the block's flag has been seen (by this thread or by one it synchronised with).
__device__ __forceinline__ long long load_id(const LogpParams& p, const RowRef& r) {
  if (!r.ok) return -1;
  if (!p.gather) return p.ids[static_cast<long long>(p.row_begin) + r.j];
  if (r.src == p.rank) return p.ids[static_cast<long long>(p.local_row_begin) + r.j];
  return ld_relaxed_sys_s64(p.gids[p.rank] +
                            (static_cast<size_t>(p.epoch & 1u) * p.world + r.src) * p.pl + r.j);
}

// Row pusher (one warp, gather mode): copies this rank's rows of the panel, 32 rows per unit,
// into every peer's gather arena. Lane 0 stages 8 KiB pieces through shared memory with bulk
// copies (global -> shared -> peer global); all lanes forward the ids. The warp that completes
// the last piece of a 128-row block raises the block's flag on every peer.
__device__ __forceinline__ void push_rows(const LogpParams& p, Control* ctl, uint32_t stage_addr,
                                          const WaitCtx& wctx, int lane) {
  const int n_units = (p.rows_local + kPushRows - 1) / kPushRows;
  const size_t row_bytes = static_cast<size_t>(p.k) * 2;
  const size_t gen_src = static_cast<size_t>(p.epoch & 1u) * p.world + p.rank;
  const int blocks_pl = p.pl / kBM;
  uint32_t phases = 0;  // bit b: parity to wait for on pbar[b]
  uint32_t n_chunks = 0;
  bool ok = true;
  for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
    const int j0 = u * kPushRows;
    const int nrows = min(kPushRows, p.rows_local - j0);
    if (lane == 0) {
      const size_t bytes = static_cast<size_t>(nrows) * row_bytes;
      const uint8_t* src = static_cast<const uint8_t*>(p.h_local) +
                           (static_cast<size_t>(p.local_row_begin) + j0) * row_bytes;
      const size_t dst_off = (gen_src * p.pl + j0) * row_bytes;
      for (size_t off = 0; off < bytes; off += kPushChunk) {
        const uint32_t n = static_cast<uint32_t>(min(static_cast<size_t>(kPushChunk), bytes - off));
        const uint32_t b = n_chunks & 1u;
        bulk_wait_group_read<1>();  // the stores that last read this buffer are done with it
        const uint32_t bar = smem_u32(&ctl->pbar[b]);
        const uint32_t buf = stage_addr + b * kPushChunk;
        mbar_arrive_expect_tx(bar, n);
        bulk_load(buf, src + off, n, bar);
        ok = mbar_wait_bounded(bar, (phases >> b) & 1u, wctx, kWherePushLoad, static_cast<int>(b));
        if (!ok) break;
        phases ^= 1u << b;
        for (int d = 1; d < p.world; ++d) {
          const int dst = (p.rank - d + p.world) % p.world;  // the rank that needs these rows soonest first
          bulk_store(p.gbuf[dst] + dst_off + off, buf, n);
        }
        bulk_commit_group();
        ++n_chunks;
      }
      bulk_wait_group<0>();  // every piece of the unit has been written
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) break;
    if (lane < nrows) {
      const long long id = p.ids[static_cast<long long>(p.local_row_begin) + j0 + lane];
      for (int d = 1; d < p.world; ++d) {
        const int dst = (p.rank - d + p.world) % p.world;
        st_relaxed_sys_s64(p.gids[dst] + gen_src * p.pl + j0 + lane, id);
      }
    }
    __threadfence_system();
    __syncwarp();
    if (lane == 0) {
      const int blk = j0 / kBM;
      const int units_in_blk = (min(kBM, p.rows_local - blk * kBM) + kPushRows - 1) / kPushRows;
      const unsigned prev = atomicAdd(&p.pcount[blk], 1u);
      if (prev + 1u == static_cast<unsigned>(units_in_blk)) {
        p.pcount[blk] = 0u;  // self-cleaning for the next launch
        __threadfence_system();
        for (int d = 1; d < p.world; ++d) {
          const int dst = (p.rank - d + p.world) % p.world;
          st_release_sys_u32(p.gflag[dst] + static_cast<size_t>(p.rank) * blocks_pl + blk, p.epoch);
        }
      }
    }
  }
}

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
fused_lmhead_logp_kernel(const __grid_constant__ CUtensorMap tm_h,
                         const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_g,
                         const __grid_constant__ LogpParams p) {
  using C = Cfg<G>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles = smem_raw + (tiles_addr - raw_addr);
  Control* ctl = reinterpret_cast<Control*>(tiles + C::kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (G == 2) ? cluster_ctarank() : 0u;
  const bool leader = (cta_rank == 0);
  const int pair_id = blockIdx.x / G;
  const int n_pairs = gridDim.x / G;
  const int n_items = p.n_mtiles * p.n_chunks;
  const int num_kb = (p.k + kBK - 1) / kBK;
  const float s2 = p.scale * kLog2e;

  WaitCtx wctx{&ctl->abort_flag, p.status, p.timeout_ns};

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->tfull[b]), 1);
      mbar_init(smem_u32(&ctl->tempty[b]), 4 * G);
      mbar_init(smem_u32(&ctl->pbar[b]), 1);
    }
    ctl->abort_flag = 0;
    ctl->is_last = 0;
    ctl->n_deferred = 0;
    fence_mbar_init_cluster();
  }
  if (warp == 5) {
    tmem_alloc<G>(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish<G>();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_h);
    tma_prefetch_desc(&tm_w);
    if (p.gather) tma_prefetch_desc(&tm_g);
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (G == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // L2 eviction hints. The rows of H that a wave works on are read again for every tile of
      // every sub-slice, the W tiles are streamed: 1 keeps H and lets W go first, 2 keeps H
      // only, 3 keeps W only, 0 gives no preference.
      const uint64_t pol_h = (p.l2_hint == 1 || p.l2_hint == 2) ? l2_policy_evict_last() : l2_policy_evict_normal();
      const uint64_t pol_w = p.l2_hint == 1 ? l2_policy_evict_first()
                                            : (p.l2_hint == 3 ? l2_policy_evict_last() : l2_policy_evict_normal());
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = pair_id; i < n_items && ok; i += n_pairs) {
        Item it;
        decode_item(p, i, it);
        int row0 = p.row_begin + it.m_tile * (kBM * G) + static_cast<int>(cta_rank) * kBM;
        const CUtensorMap* tm_a = &tm_h;
        if (p.gather) {
          const int blk = it.m_tile * G + static_cast<int>(cta_rank);
          const int src = blk / p.bps;
          const int j0 = (blk - src * p.bps) * kBM;
          if (src == p.rank) {
            row0 = p.local_row_begin + j0;  // own rows: straight from the caller's tensor
          } else {
            // another rank's rows: from this GPU's arena, once that rank has flagged the block
            row0 = (static_cast<int>(p.epoch & 1u) * p.world + src) * p.pl + j0;
            tm_a = &tm_g;
            if (j0 < p.rows_local && it.n_tiles > 0) {
              ok = flag_wait_bounded(p.gflag[p.rank] + static_cast<size_t>(src) * (p.pl / kBM) + j0 / kBM,
                                     p.epoch, wctx, kWhereGatherFlag, blk);
              if (!ok) break;
              fence_proxy_async_global();
            }
          }
        }
        for (int nt = 0; nt < it.n_tiles && ok; ++nt) {
          const int n0 = it.col_begin + nt * kBN;
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = mbar_wait_bounded(smem_u32(&ctl->empty[stage]), phase ^ 1u, wctx,
                                   kWhereProducerEmpty, stage);
            if (!ok) break;
            const uint32_t a_dst = tiles_addr + stage * C::kStageBytes;
            const uint32_t b_dst = a_dst + C::kABytes;
            const uint32_t full = smem_u32(&ctl->full[stage]);
            if constexpr (G == 1) {
              mbar_arrive_expect_tx(full, C::kTxBytes);
              tma_load_2d_hint(a_dst, tm_a, kb * kBK, row0, full, pol_h);
              tma_load_2d_hint(b_dst, &tm_w, kb * kBK, n0, full, pol_w);
              tma_load_2d_hint(b_dst + 128 * kBK * 2, &tm_w, kb * kBK, n0 + 128, full, pol_w);
            } else {
              if (leader) mbar_arrive_expect_tx(full, C::kTxBytes);
              const uint32_t full_leader = mapa_u32(full, 0);
              tma_load_2d_pair_hint(a_dst, tm_a, kb * kBK, row0, full_leader, pol_h);
              tma_load_2d_pair_hint(b_dst, &tm_w, kb * kBK, n0 + static_cast<int>(cta_rank) * C::kBRows,
                                    full_leader, pol_w);
            }
            if (++stage == C::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(kBM * G, kBN);
      int stage = 0;
      uint32_t phase = 0;
      int abuf = 0;
      uint32_t aphase = 0;
      bool ok = true;
      for (int i = pair_id; i < n_items && ok; i += n_pairs) {
        Item it;
        decode_item(p, i, it);
        for (int nt = 0; nt < it.n_tiles && ok; ++nt) {
          ok = mbar_wait_bounded(smem_u32(&ctl->tempty[abuf]), aphase ^ 1u, wctx,
                                 kWhereMmaTmemEmpty, abuf);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(abuf * kBN);
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = mbar_wait_bounded(smem_u32(&ctl->full[stage]), phase, wctx, kWhereMmaFull, stage);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t a_addr = tiles_addr + stage * C::kStageBytes;
            const uint64_t a_desc = umma_desc_k_sw128(a_addr);
            const uint64_t b_desc = umma_desc_k_sw128(a_addr + C::kABytes);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              // advancing K by 16 bf16 = 32 bytes = 2 units of the 16-byte address field
              umma_bf16<G>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                           (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit<G>(smem_u32(&ctl->empty[stage]));
            if (++stage == C::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (!ok) break;
          umma_commit<G>(smem_u32(&ctl->tfull[abuf]));
          abuf ^= 1;
          if (abuf == 0) aphase ^= 1u;
        }
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ row pusher
    if (p.gather && p.world > 1) push_rows(p, ctl, tiles_addr + C::kTileBytes + 2048, wctx, lane);
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    // Control flow rule: every named-barrier call below is reached by all 128 threads; a
    // failed wait only skips work, and the decision to leave is taken from the shared abort
    // flag right after a barrier, so it is uniform.
    const int tid = threadIdx.x;  // 0..127 == TMEM lane == row inside the CTA's 128-row block
    int abuf = 0;
    uint32_t aphase = 0;
    bool ok = true;
    const uint32_t tempty_leader_base =
        (G == 2) ? mapa_u32(smem_u32(&ctl->tempty[0]), 0) : smem_u32(&ctl->tempty[0]);
    for (int i = pair_id; i < n_items; i += n_pairs) {
      Item it;
      decode_item(p, i, it);
      const int blk = it.m_tile * G + static_cast<int>(cta_rank);  // 128-row block in the panel
      const int rp = blk * kBM + tid;                              // row inside the panel
      const RowRef rr = row_ref(p, blk, tid);
      const bool row_ok = rr.ok;
      // A remote row's id arrives with the row: it is read after the first accumulator of the
      // item is full, which the producer's wait for the block's flag precedes.
      bool have_id = !p.gather || rr.src == p.rank;
      long long id = have_id ? load_id(p, rr) : -1;
      bool id_ok = id >= 0 && id < static_cast<long long>(p.v_global);
      long long lid = id - p.vocab_offset;  // column inside this rank's shard
      bool t_here = id_ok && lid >= it.col_begin && lid < it.col_end;
      int tcol_item = t_here ? static_cast<int>(lid) - it.col_begin : -(1 << 30);

      float m = -CUDART_INF_F, l = 0.f, t = 0.f;
      for (int nt = 0; nt < it.n_tiles; ++nt) {
        const bool mine = mbar_wait_bounded(smem_u32(&ctl->tfull[abuf]), aphase, wctx,
                                            kWhereEpiTmemFull, abuf, static_cast<unsigned>(p.epi_sleep_ns));
        ok = __all_sync(0xffffffffu, mine) != 0;  // warp-uniform: tcgen05.ld needs convergence
        if (!ok) break;
        tc_fence_after_sync();
        if (!have_id) {
          have_id = true;
          id = load_id(p, rr);
          id_ok = id >= 0 && id < static_cast<long long>(p.v_global);
          lid = id - p.vocab_offset;
          t_here = id_ok && lid >= it.col_begin && lid < it.col_end;
          tcol_item = t_here ? static_cast<int>(lid) - it.col_begin : -(1 << 30);
        }
        const int valid = min(kBN, it.col_end - (it.col_begin + nt * kBN));
        const int tcol = tcol_item - nt * kBN;
        const uint32_t trow = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                              static_cast<uint32_t>(abuf * kBN);
        uint32_t va[32], vb[32];
        tmem_ld_32x32(trow, va);
        tmem_ld_wait_dep(va);
#pragma unroll
        for (int g = 0; g < kBN / 32; g += 2) {
          __syncwarp();
          tmem_ld_32x32(trow + (g + 1) * 32, vb);
          if (g * 32 < valid) fold32(va, g * 32, valid, tcol, s2, m, l, t);
          __syncwarp();
          tmem_ld_wait_dep(vb);
          if (g + 2 < kBN / 32) tmem_ld_32x32(trow + (g + 2) * 32, va);
          if ((g + 1) * 32 < valid) fold32(vb, (g + 1) * 32, valid, tcol, s2, m, l, t);
          __syncwarp();
          if (g + 2 < kBN / 32) tmem_ld_wait_dep(va);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (G == 2)
            mbar_arrive_cluster(tempty_leader_base + static_cast<uint32_t>(abuf) * 8u);
          else
            mbar_arrive(tempty_leader_base + static_cast<uint32_t>(abuf) * 8u);
        }
        abuf ^= 1;
        if (abuf == 0) aphase ^= 1u;
      }

      // ---- publish the sub-slice partial, find out whether this block is complete locally
      if (ok && row_ok) {
        p.part_m[static_cast<size_t>(it.chunk) * p.ldp + rp] = m;
        p.part_l[static_cast<size_t>(it.chunk) * p.ldp + rp] = l;
        if (t_here) p.tgt[rp] = t;
      }
      __threadfence();
      epi_bar();
      if (ctl->abort_flag) {  // uniform: read after the barrier, set before it
        ok = false;
        break;
      }
      if (tid == 0) {
        const unsigned prev = atomicAdd(&p.counters[blk], 1u);
        const int last = (prev + 1u == static_cast<unsigned>(p.n_chunks)) ? 1 : 0;
        if (last) p.counters[blk] = 0u;  // self-cleaning for the next launch
        ctl->is_last = last;
      }
      epi_bar();
      const bool is_last = ctl->is_last != 0;
      if (is_last) {
        __threadfence();
        if (!have_id) {
          // This item had no tiles. If another sub-slice of the block had some, its producer saw
          // the block's flag and the arrival counter orders this read after it; if none had,
          // the shard is empty and has_t is false whatever is read here.
          id = load_id(p, rr);
          id_ok = id >= 0 && id < static_cast<long long>(p.v_global);
          lid = id - p.vocab_offset;
        }
        const bool has_t = id_ok && lid >= 0 && lid < static_cast<long long>(p.v_local);
        float mm = -CUDART_INF_F, ml = 0.f, mt = 0.f;
        if (row_ok) {
          merge_local(p, rp, s2, mm, ml);
          if (has_t) mt = __ldcg(p.tgt + rp);
        }
        if (p.world == 1) {
          if (row_ok) write_result(p, rr.out_row, mm, ml, mt, has_t, id_ok);
        } else {
          // Every rank that writes the block's rows gets the triple: all ranks, or only the
          // rank that holds the rows when each rank keeps its own results.
          const bool to_all = !p.gather || p.out_all;
          const size_t slot = (static_cast<size_t>(p.epoch & 1u) * p.world + p.rank) * p.ldp + rp;
          const float4 v = make_float4(mm, ml, mt, has_t ? 1.f : 0.f);
          if (row_ok) {
            if (to_all) {
              for (int d = 0; d < p.world; ++d) st_relaxed_sys_f4(p.xbuf[d] + slot, v);
            } else {
              st_relaxed_sys_f4(p.xbuf[rr.src] + slot, v);
            }
          }
          __threadfence_system();
          epi_bar();
          if (to_all ? (tid < p.world) : (tid == 0)) {
            const int d = to_all ? tid : rr.src;
            st_release_sys_u32(p.xflag[d] + static_cast<size_t>(p.rank) * p.n_blocks_max + blk, p.epoch);
          }
          if (tid == 0 && (to_all || rr.src == p.rank)) {
            const int n = ctl->n_deferred;
            if (n < kMaxDeferred) {
              ctl->deferred[n] = static_cast<uint16_t>(blk);
              ctl->n_deferred = n + 1;
            } else {
              report_failure(wctx, kBadArgument, kWherePeerFlag, blk, n, 0);
            }
          }
        }
      }
      epi_bar();  // is_last and the deferred list are reused by the next item
    }

    // ---- cross-rank finish: top of the tree for the blocks this CTA pushed
    if (p.world > 1 && ok) {
      const int n_def = ctl->n_deferred;
      for (int d = 0; d < n_def; ++d) {
        const int blk = ctl->deferred[d];
        const RowRef rr = row_ref(p, blk, tid);
        if (tid < p.world) {
          flag_wait_bounded(p.xflag[p.rank] + static_cast<size_t>(tid) * p.n_blocks_max + blk, p.epoch,
                            wctx, kWherePeerFlag, blk);
        } else if (tid == 32 && p.gather && rr.src != p.rank && (blk - rr.src * p.bps) * kBM < p.rows_local) {
          // the ids of another rank's rows are read below: make sure its push has landed even if
          // this rank never loaded the block (an empty vocabulary shard)
          flag_wait_bounded(p.gflag[p.rank] + static_cast<size_t>(rr.src) * (p.pl / kBM) + (blk - rr.src * p.bps),
                            p.epoch, wctx, kWhereGatherFlag, blk);
        }
        epi_bar();
        if (ctl->abort_flag) break;  // uniform, as above
        const int rp = blk * kBM + tid;
        if (rr.ok) {
          float lm[kSlices], ll[kSlices];
          float t = 0.f;
          bool has_t = false;
#pragma unroll
          for (int r = 0; r < kSlices; ++r) {
            lm[r] = -CUDART_INF_F;
            ll[r] = 0.f;
            if (r < p.world) {
              const size_t slot = (static_cast<size_t>(p.epoch & 1u) * p.world + r) * p.ldp + rp;
              const float4 v = ld_relaxed_sys_f4(p.xbuf[p.rank] + slot);
              lm[r] = v.x;
              ll[r] = v.y;
              if (v.w != 0.f) {
                t = v.z;
                has_t = true;
              }
            }
          }
#pragma unroll
          for (int w = kSlices; w > 1; w >>= 1) {
            if (w <= p.world) {
#pragma unroll
              for (int i = 0; i < w / 2; ++i) {
                float m = lm[2 * i], l = ll[2 * i];
                merge2(m, l, lm[2 * i + 1], ll[2 * i + 1], s2);
                lm[i] = m;
                ll[i] = l;
              }
            }
          }
          const long long id = load_id(p, rr);
          const bool id_ok = id >= 0 && id < static_cast<long long>(p.v_global);
          write_result(p, rr.out_row, lm[0], ll[0], t, has_t, id_ok);
        }
      }
    }
  }

  // ------------------------------------------------------------------ common exit
  if (ctl->abort_flag) {
    if constexpr (G == 2) {
      // make the peer CTA leave its waits too
      st_shared_cluster_u32(mapa_u32(smem_u32(&ctl->abort_flag), cta_rank ^ 1u), 1u);
    }
    drain_in_flight();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (G == 2) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 5) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<G>(tmem_base, 512);
  }
}

constexpr int kMaxDevices = 64;

// Resident CTAs of the kernel on the current device. The shared-memory opt-in is a per-device
// attribute, so both it and the occupancy answer are set up and cached per device.
template <int G>
int max_ctas(int num_sms) {
  static std::mutex mu;
  static int cached[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] > 0) return cached[dev];
  using C = Cfg<G>;
  auto* kern = fused_lmhead_logp_kernel<G>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytesGather) !=
      cudaSuccess)
    return -1;
  int n = num_sms;
  if (G == 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(num_sms / 2 * 2));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytesGather;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = num_sms / 2;
    }
    n = clusters * 2;
    if (n > num_sms / 2 * 2) n = num_sms / 2 * 2;
  }
  cached[dev] = n;
  return n;
}

template <int G>
int launch_panel(const CUtensorMap& tm_h, const CUtensorMap& tm_w, const CUtensorMap& tm_g, const LogpParams& p,
                 int num_sms, cudaStream_t stream) {
  using C = Cfg<G>;
  int ctas = max_ctas<G>(num_sms);
  if (ctas <= 0) return -10;
  const int n_items = p.n_mtiles * p.n_chunks;
  // with sharded rows every CTA also carries a pusher, so the grid is not shrunk to the items
  if (!p.gather && n_items * G < ctas) ctas = n_items * G;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = p.gather ? C::kSmemBytesGather : C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = G;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, fused_lmhead_logp_kernel<G>, tm_h, tm_w, tm_g, p);
  if (e != cudaSuccess) {
    fprintf(stderr, "[kernel_align_b200] fused_lmhead_logp launch failed: %s\n", cudaGetErrorString(e));
    return -11;
  }
  return 0;
}

size_t ws_status_offset(int v_global, int panel_rows) {
  const int vs = (v_global + kSlices - 1) / kSlices;
  const int sub = (vs + kSubCols - 1) / kSubCols;
  const size_t ldp = static_cast<size_t>(panel_rows);
  const size_t n_chunks = static_cast<size_t>(kSlices) * sub;  // upper bound (world == 1)
  const size_t n_blocks = ldp / kBM;
  size_t bytes = 2 * n_chunks * ldp * sizeof(float);  // part_m, part_l
  bytes += ldp * sizeof(float);                       // tgt
  bytes += n_blocks * sizeof(unsigned);               // counters
  return (bytes + 255) / 256 * 256;
}

// Layout of the gather arena (see ka_lmhead_logp_gather_bytes).
struct GatherLayout {
  size_t ids_off, flag_off, pcount_off, total;
};
GatherLayout gather_layout(int world, int panel_rows, int k) {
  GatherLayout g;
  const size_t rows2 = 2 * static_cast<size_t>(panel_rows);
  const size_t blocks_pl = static_cast<size_t>(panel_rows / world) / kBM;
  g.ids_off = rows2 * static_cast<size_t>(k) * 2;
  g.flag_off = g.ids_off + rows2 * sizeof(long long);
  g.pcount_off = g.flag_off + (static_cast<size_t>(world) * blocks_pl * sizeof(unsigned) + 255) / 256 * 256;
  g.total = g.pcount_off + (blocks_pl * sizeof(unsigned) + 255) / 256 * 256;
  return g;
}

struct FwdArgs {
  const void* hidden;  // all rows, or this rank's rows when `sharded`
  const void* weight;
  const long long* ids;
  float* logp;
  float* lse;
  void* workspace;
  size_t workspace_bytes;
  void* const* peer_exchange;
  void* const* peer_gather;
  int m;  // rows of `hidden`
  int k, v_global, v_local, vocab_offset, world, rank;
  unsigned epoch_base;
  float scale;
  int panel_rows, sharded, out_all, cta_group, cg_pref, m_fast, l2_hint, num_sms;
  unsigned long long timeout_ns;
  cudaStream_t stream;
};

int forward_impl(const FwdArgs& a) {
  if (a.m <= 0) return 0;
  if (a.k % 8 != 0 || a.k <= 0) return -1;
  if (!(a.world == 1 || a.world == 2 || a.world == 4 || a.world == 8) || a.rank < 0 || a.rank >= a.world) return -2;
  if (!(a.scale > 0.f)) return -3;
  if (a.cta_group != 1 && a.cta_group != 2) return -4;
  if (a.panel_rows <= 0 || a.panel_rows % 256 != 0) return -5;
  if (a.workspace_bytes < ka_lmhead_logp_workspace_bytes(a.v_global, a.panel_rows)) return -6;
  if (a.world > 1 && a.peer_exchange == nullptr) return -7;
  const bool gather = a.sharded && a.world > 1;
  if (gather) {
    if (a.peer_gather == nullptr) return -13;
    if (a.panel_rows % (256 * a.world) != 0) return -14;
    if ((reinterpret_cast<uintptr_t>(a.hidden) & 15u) != 0) return -15;
  }

  const int vs = (a.v_global + kSlices - 1) / kSlices;
  const int sub = (vs + kSubCols - 1) / kSubCols;
  const int n_slices_local = kSlices / a.world;
  if (a.vocab_offset != a.rank * n_slices_local * vs) return -8;
  {
    const long long hi = static_cast<long long>(a.rank + 1) * n_slices_local * vs;
    const long long end = hi < a.v_global ? hi : a.v_global;
    const long long expect = end - a.vocab_offset > 0 ? end - a.vocab_offset : 0;
    if (a.v_local != expect) return -9;
  }
  const size_t ldp = static_cast<size_t>(a.panel_rows);
  const size_t n_blocks_max = ldp / kBM;
  if (n_blocks_max > 65535) return -12;

  LogpParams p = {};
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  const size_t n_chunks_max = static_cast<size_t>(kSlices) * sub;
  p.part_m = reinterpret_cast<float*>(ws);
  p.part_l = p.part_m + n_chunks_max * ldp;
  p.tgt = p.part_l + n_chunks_max * ldp;
  p.counters = reinterpret_cast<unsigned*>(p.tgt + ldp);
  p.status = reinterpret_cast<int*>(ws + ws_status_offset(a.v_global, a.panel_rows));
  if (a.world > 1) {
    const size_t xbuf_bytes = 2 * static_cast<size_t>(a.world) * ldp * sizeof(float4);
    for (int d = 0; d < a.world; ++d) {
      uint8_t* base = static_cast<uint8_t*>(a.peer_exchange[d]);
      if (!base) return -7;
      p.xbuf[d] = reinterpret_cast<float4*>(base);
      p.xflag[d] = reinterpret_cast<unsigned*>(base + xbuf_bytes);
    }
  }
  p.ids = a.ids;
  p.logp = a.logp;
  p.lse = a.lse;
  p.m = a.m;
  p.k = a.k;
  p.v_global = a.v_global;
  p.v_local = a.v_local;
  p.vocab_offset = a.vocab_offset;
  p.vs = vs;
  p.sub = sub;
  p.n_slices_local = n_slices_local;
  p.n_chunks = n_slices_local * sub;
  p.ldp = static_cast<int>(ldp);
  p.n_blocks_max = static_cast<int>(n_blocks_max);
  p.world = a.world;
  p.rank = a.rank;
  p.scale = a.scale;
  p.timeout_ns = a.timeout_ns;
  // Sub-slices that run side by side (cg) x row tiles that run side by side (mg) ~ CTA pairs.
  // The caller's preference (0: the default of 8), which KA_LOGP_CG overrides for tuning.
  int cg_pref = a.cg_pref >= 1 && a.cg_pref <= 64 ? a.cg_pref : 8;
  if (const char* e = getenv("KA_LOGP_CG")) {
    const int v = atoi(e);
    if (v >= 1 && v <= 64) cg_pref = v;
  }
  p.l2_hint = a.l2_hint >= 0 && a.l2_hint <= 3 ? a.l2_hint : 0;
  p.epi_sleep_ns = 200;  // measured 111 - 113 ms against 114 - 116 ms without the sleep (G = 256, CTA pair)
  if (const char* e = getenv("KA_LOGP_EPI_SLEEP")) {
    const int v = atoi(e);
    if (v >= 0 && v <= 100000) p.epi_sleep_ns = v;
  }
  if (const char* e = getenv("KA_LOGP_L2HINT")) {
    const int v = atoi(e);
    if (v >= 0 && v <= 3) p.l2_hint = v;
  }
  p.m_fast = (a.m_fast & 1) ? 1 : 0;
  p.c_outer = (a.m_fast & 2) ? 1 : 0;
  p.cg = p.n_chunks < cg_pref ? p.n_chunks : cg_pref;
  {
    const int pairs = a.num_sms / a.cta_group;
    int mg = pairs / p.cg;
    if (mg < 1) mg = 1;
    p.mg = mg;
  }

  CUtensorMap tm_h, tm_w, tm_g;
  int rc = make_tmap_2d_16bit_sw128(&tm_h, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.hidden, static_cast<uint64_t>(a.m),
                                    static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.k), kBM, kBK);
  if (rc != 0) return -20 + rc;
  rc = make_tmap_2d_16bit_sw128(&tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.weight,
                                static_cast<uint64_t>(a.v_local > 0 ? a.v_local : 1), static_cast<uint64_t>(a.k),
                                static_cast<uint64_t>(a.k), 128, kBK);
  if (rc != 0) return -40 + rc;
  tm_g = tm_h;
  const int rows_per_mtile = kBM * a.cta_group;
  unsigned epoch = a.epoch_base;

  if (!gather) {
    for (int row_begin = 0; row_begin < a.m; row_begin += a.panel_rows) {
      const int rows = (a.m - row_begin) < a.panel_rows ? (a.m - row_begin) : a.panel_rows;
      p.row_begin = row_begin;
      p.rows = rows;
      p.n_mtiles = (rows + rows_per_mtile - 1) / rows_per_mtile;
      p.epoch = epoch++;
      rc = (a.cta_group == 1) ? launch_panel<1>(tm_h, tm_w, tm_g, p, a.num_sms, a.stream)
                              : launch_panel<2>(tm_h, tm_w, tm_g, p, a.num_sms, a.stream);
      if (rc != 0) return rc;
    }
    return 0;
  }

  // ---- rows sharded over the ranks
  const GatherLayout gl = gather_layout(a.world, a.panel_rows, a.k);
  for (int d = 0; d < a.world; ++d) {
    uint8_t* base = static_cast<uint8_t*>(a.peer_gather[d]);
    if (!base) return -13;
    p.gbuf[d] = base;
    p.gids[d] = reinterpret_cast<long long*>(base + gl.ids_off);
    p.gflag[d] = reinterpret_cast<unsigned*>(base + gl.flag_off);
  }
  p.pcount = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(a.peer_gather[a.rank]) + gl.pcount_off);
  p.gather = 1;
  p.out_all = a.out_all ? 1 : 0;
  p.m_local = a.m;
  p.pl = a.panel_rows / a.world;
  p.h_local = a.hidden;
  rc = make_tmap_2d_16bit_sw128(&tm_g, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.peer_gather[a.rank],
                                2ull * static_cast<uint64_t>(a.panel_rows), static_cast<uint64_t>(a.k),
                                static_cast<uint64_t>(a.k), kBM, kBK);
  if (rc != 0) return -60 + rc;
  for (int lrb = 0; lrb < a.m; lrb += p.pl) {
    const int rows_local = (a.m - lrb) < p.pl ? (a.m - lrb) : p.pl;
    int bps = (rows_local + kBM - 1) / kBM;
    bps += bps & 1;
    p.local_row_begin = lrb;
    p.rows_local = rows_local;
    p.bps = bps;
    p.row_begin = 0;
    p.rows = a.world * bps * kBM;
    p.n_mtiles = a.world * bps / a.cta_group;
    p.mt_rot = a.rank * bps / a.cta_group;
    p.epoch = epoch++;
    rc = (a.cta_group == 1) ? launch_panel<1>(tm_h, tm_w, tm_g, p, a.num_sms, a.stream)
                            : launch_panel<2>(tm_h, tm_w, tm_g, p, a.num_sms, a.stream);
    if (rc != 0) return rc;
  }
  return 0;
}

}  // namespace
}  // namespace ka

extern "C" {

size_t ka_lmhead_logp_workspace_bytes(int v_global, int panel_rows) {
  return ka::ws_status_offset(v_global, panel_rows) + 256;
}

size_t ka_lmhead_logp_exchange_bytes(int world, int panel_rows) {
  const size_t ldp = static_cast<size_t>(panel_rows);
  const size_t n_blocks = ldp / ka::kBM;
  const size_t xbuf = 2 * static_cast<size_t>(world) * ldp * sizeof(float4);
  const size_t xflag = static_cast<size_t>(world) * n_blocks * sizeof(unsigned);
  return xbuf + (xflag + 255) / 256 * 256;
}

size_t ka_lmhead_logp_gather_bytes(int world, int panel_rows, int k) {
  if (world < 1 || panel_rows <= 0 || panel_rows % (256 * world) != 0 || k <= 0) return 0;
  return ka::gather_layout(world, panel_rows, k).total;
}

int ka_lmhead_logp_status_offset(int v_global, int panel_rows) {
  return static_cast<int>(ka::ws_status_offset(v_global, panel_rows));
}

// See fused_lmhead_logp.h for the contracts.
int ka_lmhead_logp_forward(const void* hidden, const void* weight, const long long* ids, float* logp,
                           float* lse, void* workspace, size_t workspace_bytes, void* const* peer_exchange,
                           int m, int k, int v_global, int v_local, int vocab_offset, int world, int rank,
                           unsigned epoch_base, float scale, int panel_rows, int cta_group, int num_sms,
                           unsigned long long timeout_ns, void* stream_ptr) {
  ka::FwdArgs a = {hidden, weight, ids, logp, lse, workspace, workspace_bytes, peer_exchange, nullptr,
                   m, k, v_global, v_local, vocab_offset, world, rank, epoch_base, scale, panel_rows,
                   0, 1, cta_group, 0, 0, 0, num_sms, timeout_ns, static_cast<cudaStream_t>(stream_ptr)};
  return ka::forward_impl(a);
}

int ka_lmhead_logp_forward_sched(const void* hidden, const void* weight, const long long* ids, float* logp,
                                 float* lse, void* workspace, size_t workspace_bytes, void* const* peer_exchange,
                                 int m, int k, int v_global, int v_local, int vocab_offset, int world, int rank,
                                 unsigned epoch_base, float scale, int panel_rows, int cta_group, int cg_pref,
                                 int m_fast, int l2_hint, int num_sms, unsigned long long timeout_ns,
                                 void* stream_ptr) {
  ka::FwdArgs a = {hidden, weight, ids, logp, lse, workspace, workspace_bytes, peer_exchange, nullptr,
                   m, k, v_global, v_local, vocab_offset, world, rank, epoch_base, scale, panel_rows,
                   0, 1, cta_group, cg_pref, m_fast, l2_hint, num_sms, timeout_ns,
                   static_cast<cudaStream_t>(stream_ptr)};
  return ka::forward_impl(a);
}

int ka_lmhead_logp_forward_sharded(const void* hidden_local, const void* weight, const long long* ids_local,
                                   float* logp, float* lse, void* workspace, size_t workspace_bytes,
                                   void* const* peer_exchange, void* const* peer_gather, int m_local, int k,
                                   int v_global, int v_local, int vocab_offset, int world, int rank,
                                   unsigned epoch_base, float scale, int panel_rows, int out_all, int cta_group,
                                   int cg_pref, int m_fast, int l2_hint, int num_sms, unsigned long long timeout_ns,
                                   void* stream_ptr) {
  ka::FwdArgs a = {hidden_local, weight, ids_local, logp, lse, workspace, workspace_bytes, peer_exchange,
                   peer_gather, m_local, k, v_global, v_local, vocab_offset, world, rank, epoch_base, scale,
                   panel_rows, 1, out_all, cta_group, cg_pref, m_fast, l2_hint, num_sms, timeout_ns,
                   static_cast<cudaStream_t>(stream_ptr)};
  return ka::forward_impl(a);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Allocation-free entry point (see fused_lmhead_logp_noalloc.h for who needs it and the rules).
// ------------------------------------------------------------------------------------------
#include "fused_lmhead_logp_noalloc.h"

// The kernel's scratch for callers that cannot allocate: partials, target logits, counters
// and status for one panel of KA_NOALLOC_PANEL_ROWS rows at up to KA_NOALLOC_MAX_VOCAB
// columns. In host code this name is only a handle for cudaGetSymbolAddress, never a pointer.
static __device__ __align__(256) unsigned char ka_noalloc_scratch[KA_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;  // devices with a cached scratch address
std::mutex g_noalloc_mutex;
void* g_noalloc_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device, resolved once per device.
void* noalloc_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, ka_noalloc_scratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "[kernel_align_b200] cudaGetSymbolAddress(ka_noalloc_scratch) failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return nullptr;
    }
    g_noalloc_ptr[dev] = p;
  }
  return g_noalloc_ptr[dev];
}
}  // namespace

extern "C" int ka_lmhead_logp_forward_noalloc(const void* hidden, const void* weight, const long long* ids,
                                              float* logp, float* lse, int m, int k, int vocab, float scale,
                                              int cta_group, int num_sms, unsigned long long timeout_ns,
                                              void* stream) {
  if (vocab <= 0 || vocab > KA_NOALLOC_MAX_VOCAB ||
      ka_lmhead_logp_workspace_bytes(vocab, KA_NOALLOC_PANEL_ROWS) > static_cast<size_t>(KA_NOALLOC_SCRATCH_BYTES)) {
    fprintf(stderr,
            "[kernel_align_b200] ka_lmhead_logp_forward_noalloc: vocab %d is outside the built-in scratch "
            "(max %d); use ka_lmhead_logp_forward with a caller-provided workspace\n",
            vocab, KA_NOALLOC_MAX_VOCAB);
    return -30;
  }
  void* scratch = noalloc_scratch_for_current_device();
  if (scratch == nullptr) return -31;
  // Counters and status must start at zero; a call that was aborted may have left them dirty.
  const size_t status_off = static_cast<size_t>(ka_lmhead_logp_status_offset(vocab, KA_NOALLOC_PANEL_ROWS));
  const size_t counters_bytes = (KA_NOALLOC_PANEL_ROWS / ka::kBM) * sizeof(unsigned);
  const size_t clear_from = (status_off - counters_bytes) / 256 * 256;  // rounded down into the tgt tail, which is
                                                                        // rewritten before it is read
  if (cudaMemsetAsync(static_cast<unsigned char*>(scratch) + clear_from, 0, status_off + 256 - clear_from,
                      static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return -32;
  return ka_lmhead_logp_forward(hidden, weight, ids, logp, lse, scratch, KA_NOALLOC_SCRATCH_BYTES, nullptr, m, k,
                                vocab, vocab, 0, 1, 0, 1u, scale, KA_NOALLOC_PANEL_ROWS, cta_group, num_sms,
                                timeout_ns, stream);
}

extern "C" int ka_lmhead_logp_noalloc_status(int vocab, int* host_out) {
  if (vocab <= 0 || vocab > KA_NOALLOC_MAX_VOCAB) return -30;
  void* scratch = noalloc_scratch_for_current_device();
  if (scratch == nullptr) return -31;
  const size_t status_off = static_cast<size_t>(ka_lmhead_logp_status_offset(vocab, KA_NOALLOC_PANEL_ROWS));
  const cudaError_t e = cudaMemcpy(host_out, static_cast<unsigned char*>(scratch) + status_off,
                                   ka::kStatusWords * sizeof(int), cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? 0 : -34;
}
