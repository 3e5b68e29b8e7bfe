// Batch-invariant causal attention forward for sm_100a (GQA, head_dim 128).
//
// One CTA works on TWO 128-row query tiles that share a KV head: two query heads of one GQA
// group at the same rows (even group size) or two consecutive row tiles of one head. K and V
// tiles arrive by TMA into a five-slot ring and are used by both tiles. S_t = Q_t K^T and
// O_t += P_t V are tcgen05.mma (M=128, N=128) with fp32 accumulators in TMEM: columns
// [0,128) and [128,256) hold S_0 and S_1, [256,384) and [384,512) hold O_0 and O_1. Four
// softmax warps per tile give every query row one thread: it reads its S row from TMEM in
// 32-column chunks (a maximum pass, then an exponential pass with packed two-lane fp32
// arithmetic) and writes P as packed bf16 back into the first 64 columns of the same S region,
// from where the second MMA reads it as a TMEM A operand, so P never touches shared memory
// (whose bandwidth the Q K^T products need). The first half of P is signalled early, so half
// of the P V product overlaps the rest of the softmax; while the softmax warps of one tile
// work, the tensor core runs the other tile's MMAs. The running maximum is only moved when it
// grows by more than 2^8 (then the O row is rescaled in TMEM), so the common tile needs no
// correction pass. The kernel is persistent: one CTA per SM walks a list of work items dealt
// heaviest first, and the loads and first products of the next item overlap the output pass.
// KV tiles are visited in increasing order, always 128 wide, whatever the batch size, the
// pairing or the number of heads on this GPU, so a query row's output depends on its own
// sequence only.
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
constexpr int kBQ = 128;        // query rows per tile
constexpr int kBKV = 128;       // keys per tile
constexpr int kTiles = 2;       // query tiles per CTA
constexpr int kSoftThreads = 128 * kTiles;
constexpr int kThreads = kSoftThreads + 64;  // softmax warps, then one TMA warp and one MMA warp
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KiB: two 64-column boxes of 128 rows
constexpr int kSlots = 5;                  // ring of K / V tiles
constexpr int kSmemBytes = kTiles * kTileBytes + kSlots * kTileBytes + 1024 + 512;
constexpr float kLog2e = 1.4426950408889634f;

struct Control {
  uint64_t q_full;
  uint64_t q_empty;   // every S product of the current item has completed: the Q tiles may be replaced
  uint64_t ring_full[kSlots];
  uint64_t ring_empty[kSlots];
  uint64_t s_full[kTiles];    // S_t of the next KV tile is in TMEM
  uint64_t p_full[kTiles][2]; // P_t for keys [64 h, 64 h + 64) written (h = 1: the whole S_t row has been read)
  uint64_t pv_done[kTiles];   // O_t includes every P V product issued so far
  uint32_t tmem_base;
  int abort_flag;
};

struct AttnParams {
  __nv_bfloat16* out;     // [B, L, Hq, D] with token stride out_stride
  float* lse;             // [B, Hq, L] or null (natural-log log-sum-exp of the scaled scores)
  long long out_stride;   // elements between tokens in out
  int batch, seq_len, hq, hkv;
  int pair_heads;         // 1: the two tiles are heads h, h+1 at the same rows; 0: row tiles 2i, 2i+1
  float scale;            // softmax scale (1/sqrt(D))
  int causal;
  int* status;
  unsigned long long timeout_ns;
};

struct TileCoord {
  int h;        // query head
  int row0;     // first query row inside the sequence
  int n_kv;     // KV tiles this query tile visits (0: the tile does not exist)
};

__device__ __forceinline__ TileCoord tile_coord(const AttnParams& p, int unit, int head_unit, int t) {
  const int n_qt = (p.seq_len + kBQ - 1) / kBQ;
  TileCoord c;
  int qt;
  if (p.pair_heads) {
    c.h = head_unit * 2 + t;
    qt = unit;
  } else {
    c.h = head_unit;
    qt = unit * 2 + t;
  }
  c.row0 = qt * kBQ;
  if (qt >= n_qt) {
    c.n_kv = 0;
  } else {
    const int kv_end = p.causal ? min(p.seq_len, c.row0 + kBQ) : p.seq_len;
    c.n_kv = (kv_end + kBKV - 1) / kBKV;
  }
  return c;
}

struct Item {
  TileCoord tc[kTiles];
  int b, hk, tok0, n_max;
};

__device__ __forceinline__ Item decode_item(const AttnParams& p, int item, int n_units, int n_head_units, int per_unit,
                                            int group) {
  Item w;
  const int unit = n_units - 1 - item / per_unit;     // heavy (late) rows first
  const int bh = item % per_unit;
  const int head_unit = bh % n_head_units;
  w.b = bh / n_head_units;
  w.tc[0] = tile_coord(p, unit, head_unit, 0);
  w.tc[1] = tile_coord(p, unit, head_unit, 1);
  w.hk = w.tc[0].h / group;
  w.tok0 = w.b * p.seq_len;
  w.n_max = max(w.tc[0].n_kv, w.tc[1].n_kv);
  return w;
}

// Items are dealt to the resident CTAs in rounds, left to right in even rounds and right to
// left in odd ones: with items sorted heaviest first this keeps the CTAs' totals within about
// one item of each other without a shared counter. Each pair of CTAs walks its rounds starting
// at a different one, so the CTAs do not all reach their output pass (a burst of stores) at
// the same moment. Returns -1 for a slot of the last, partial round that holds no item.
__device__ __forceinline__ int item_of_step(int step, int n_rounds, int n_items) {
  const int g = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  const int round = (step + (c >> 1)) % n_rounds;
  const int item = round * g + ((round & 1) ? g - 1 - c : c);
  return item < n_items ? item : -1;
}

__global__ void __launch_bounds__(kThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t q_tiles = base;                               // tile t at + t * 32 KiB
  const uint32_t ring = base + kTiles * kTileBytes;            // slot s at + s * 32 KiB
  Control* ctl = reinterpret_cast<Control*>(smem + (kTiles + kSlots) * kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work items: (row unit, head unit, sequence). Items are numbered heaviest row unit first
  // and dealt in rounds to the resident CTAs, which walk their items in a loop; all
  // pipeline counters run on across items, so the loads and the first S products of the next
  // item overlap the last softmax tiles and the output pass of the current one.
  const int n_qt = (p.seq_len + kBQ - 1) / kBQ;
  const int n_units = p.pair_heads ? n_qt : (n_qt + 1) / 2;
  const int n_head_units = p.pair_heads ? p.hq / 2 : p.hq;
  const int per_unit = n_head_units * p.batch;
  const int n_items = n_units * per_unit;
  const int group = p.hq / p.hkv;
  const int n_rounds = (n_items + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

  WaitCtx wctx{&ctl->abort_flag, p.status, p.timeout_ns};

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctl->q_full), 1);
    mbar_init(smem_u32(&ctl->q_empty), 1);
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(smem_u32(&ctl->ring_full[s]), 1);
      mbar_init(smem_u32(&ctl->ring_empty[s]), 1);
    }
    for (int t = 0; t < kTiles; ++t) {
      mbar_init(smem_u32(&ctl->s_full[t]), 1);
      mbar_init(smem_u32(&ctl->p_full[t][0]), 4);
      mbar_init(smem_u32(&ctl->p_full[t][1]), 4);
      mbar_init(smem_u32(&ctl->pv_done[t]), 1);
    }
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

  if (warp == kSoftThreads / 32) {
    // ------------------------------------------------------------------ TMA producer
    // Ring order: K(0), then for every KV tile j: K(j+1) (if any), V(j). The MMA warp consumes
    // and releases the slots in this same order.
    if (lane == 0) {
      const uint32_t qf = smem_u32(&ctl->q_full);
      int it = 0, qi = 0;
      bool ok = true;
      for (int step = 0; step < n_rounds && ok; ++step) {
        const int item = item_of_step(step, n_rounds, n_items);
        if (item < 0) continue;
        const Item w = decode_item(p, item, n_units, n_head_units, per_unit, group);
        if (!mbar_wait_bounded(smem_u32(&ctl->q_empty), (qi & 1) ^ 1u, wctx, 30, item)) break;
        mbar_arrive_expect_tx(qf, (w.tc[1].n_kv > 0 ? 2 : 1) * kTileBytes);
        tma_load_2d(q_tiles, &tm_q, w.tc[0].h * kD, w.tok0 + w.tc[0].row0, qf);
        tma_load_2d(q_tiles + 16384, &tm_q, w.tc[0].h * kD + 64, w.tok0 + w.tc[0].row0, qf);
        if (w.tc[1].n_kv > 0) {
          tma_load_2d(q_tiles + kTileBytes, &tm_q, w.tc[1].h * kD, w.tok0 + w.tc[1].row0, qf);
          tma_load_2d(q_tiles + kTileBytes + 16384, &tm_q, w.tc[1].h * kD + 64, w.tok0 + w.tc[1].row0, qf);
        }
        auto load = [&](const CUtensorMap* tm, int j) {
          const int s = it % kSlots;
          if (!mbar_wait_bounded(smem_u32(&ctl->ring_empty[s]), ((it / kSlots) & 1) ^ 1u, wctx, 31, s)) {
            ok = false;
            return;
          }
          const uint32_t full = smem_u32(&ctl->ring_full[s]);
          const uint32_t dst = ring + s * kTileBytes;
          mbar_arrive_expect_tx(full, kTileBytes);
          tma_load_2d(dst, tm, w.hk * kD, w.tok0 + j * kBKV, full);
          tma_load_2d(dst + 16384, tm, w.hk * kD + 64, w.tok0 + j * kBKV, full);
          ++it;
        };
        load(&tm_k, 0);
        for (int j = 0; j < w.n_max && ok; ++j) {
          if (j + 1 < w.n_max) load(&tm_k, j + 1);
          if (ok) load(&tm_v, j);
        }
        ++qi;
      }
    }
  } else if (warp == kSoftThreads / 32 + 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Per KV tile j and query tile t: O_t += P_t(j) V(j), then S_t(j+1) = Q_t K(j+1). The P V
    // product is issued first because P_t(j) lives in the S_t columns that the next Q K product
    // overwrites; the tensor core executes the two in issue order.
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_bf16_f32(kBQ, kBKV);
      const uint32_t idesc_o = umma_idesc_bf16_f32(kBQ, kD) | (1u << 16);  // B (V) is MN-major
      int it = 0, qi = 0;
      int cnt[kTiles] = {0, 0};     // tile-iterations so far: the phase of p_full / s_full / pv_done
      bool ok = true;
      auto take = [&](uint32_t& tile_addr, int& slot) {
        slot = it % kSlots;
        if (!mbar_wait_bounded(smem_u32(&ctl->ring_full[slot]), (it / kSlots) & 1, wctx, 33, slot)) ok = false;
        tile_addr = ring + slot * kTileBytes;
        ++it;
      };
      // Operand descriptors are a base (tile 0 of Q, slot 0 of the ring) plus small constants in
      // the 16-byte address field: the whole buffer lies below 256 KiB, so the sums never carry
      // out of that field, and issuing an MMA costs an add instead of rebuilding the descriptor.
      const uint64_t dq0 = desc_kmajor(q_tiles, 0), dk0 = desc_kmajor(ring, 0), dv0 = desc_mnmajor(ring, 0);
      auto issue_s = [&](int t, uint32_t kt) {
        const uint64_t dq = dq0 + static_cast<uint64_t>((t * kTileBytes) >> 4);
        const uint64_t dk = dk0 + static_cast<uint64_t>((kt - ring) >> 4);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint64_t koff = static_cast<uint64_t>(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          umma_bf16<1>(tmem_base + t * 128, dq + koff, dk + koff, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit<1>(smem_u32(&ctl->s_full[t]));
      };
      for (int step = 0; step < n_rounds && ok; ++step) {
        const int item = item_of_step(step, n_rounds, n_items);
        if (item < 0) continue;
        const Item w = decode_item(p, item, n_units, n_head_units, per_unit, group);
        ok = mbar_wait_bounded(smem_u32(&ctl->q_full), qi & 1, wctx, 32, item);
        if (!ok) break;
        uint32_t kt = 0, vt = 0;
        int kslot = 0, vslot = 0;
        take(kt, kslot);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int t = 0; t < kTiles; ++t)
          if (w.tc[t].n_kv > 0) issue_s(t, kt);
        umma_commit<1>(smem_u32(&ctl->ring_empty[kslot]));
        if (w.n_max == 1) umma_commit<1>(smem_u32(&ctl->q_empty));
        for (int j = 0; j < w.n_max && ok; ++j) {
          const bool has_next = j + 1 < w.n_max;
          if (has_next) take(kt, kslot);
          if (ok) take(vt, vslot);
          if (!ok) break;
#pragma unroll
          for (int t = 0; t < kTiles; ++t) {
            if (!ok || j >= w.tc[t].n_kv) continue;
            // the first half of P is signalled as soon as it is written, so its part of the
            // product runs while the softmax warps are still on the second half
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              if (!ok) continue;
              ok = mbar_wait_bounded(smem_u32(&ctl->p_full[t][hf]), cnt[t] & 1, wctx, 35, t);
              if (!ok) continue;
              tc_fence_after_sync();
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4) {
                const int kk = hf * 4 + k4;
                const uint64_t dv = dv0 + static_cast<uint64_t>((vt - ring + kk * 2048) >> 4);
                umma_bf16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, dv, idesc_o,
                             (j > 0 || kk > 0) ? 1u : 0u);
              }
            }
            if (!ok) continue;
            ++cnt[t];
            umma_commit<1>(smem_u32(&ctl->pv_done[t]));
            if (j + 1 < w.tc[t].n_kv) issue_s(t, kt);
          }
          if (!ok) break;
          if (has_next) umma_commit<1>(smem_u32(&ctl->ring_empty[kslot]));
          umma_commit<1>(smem_u32(&ctl->ring_empty[vslot]));
          if (j + 2 == w.n_max) umma_commit<1>(smem_u32(&ctl->q_empty));   // the last S products are issued
        }
        ++qi;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output
    // Warps 0-3 own query tile 0, warps 4-7 tile 1; thread `row` owns one query row == one TMEM
    // lane. No thread waits for another softmax thread, so a warp that gives up just stops.
    const int t = warp >> 2;
    const int row = threadIdx.x & 127;
    const float c = p.scale * kLog2e;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + t * 128;          // S_t, and P_t in its first 64 columns
    const uint32_t tmem_o = tmem_base + lane_base + 256 + t * 128;
    int cnt = 0;                            // tile-iterations of this tile so far (barrier phases)
    bool ok = true;

    for (int step = 0; step < n_rounds && ok; ++step) {
    const int item = item_of_step(step, n_rounds, n_items);
    if (item < 0) continue;
    const Item wi = decode_item(p, item, n_units, n_head_units, per_unit, group);
    const TileCoord tc = wi.tc[t];
    const int b = wi.b, tok0 = wi.tok0;
    const int q_pos = tc.row0 + row;
    float m = -CUDART_INF_F;                // reference maximum of the row (may lag the true one by < 2^8)
    float l = 0.f;

    for (int j = 0; j < tc.n_kv && ok; ++j, ++cnt) {
      uint32_t va[32], vb[32];     // two 32-column chunks of the S row in flight
      const int kv0 = j * kBKV;
      const int limit = (p.causal ? min(q_pos, p.seq_len - 1) : p.seq_len - 1) - kv0;  // last allowed column
      // Rows grow with the lane, so lane 0 has the smallest limit of the warp and lane 31 the
      // largest: the tile is unmasked for the whole warp, or only its first n_act 32-column
      // chunks hold any allowed column (the diagonal tile of a causal row block, a ragged end).
      const int lim_lo = __shfl_sync(0xffffffffu, limit, 0), lim_hi = __shfl_sync(0xffffffffu, limit, 31);
      const bool warp_full = lim_lo >= kBKV - 1;
      const int n_act = lim_hi < 0 ? 0 : min(4, lim_hi / 32 + 1);
      {
        const bool mine = mbar_wait_bounded(smem_u32(&ctl->s_full[t]), cnt & 1, wctx, 38, t);
        ok = __all_sync(0xffffffffu, mine) != 0;
        if (!ok) break;
      }
      tc_fence_after_sync();
      auto mask_chunk = [&](uint32_t (&v)[32], int g) {
        if (g * 32 + 31 > lim_lo) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (g * 32 + i > limit) v[i] = __float_as_uint(-CUDART_INF_F);
        }
      };
      float a0 = -CUDART_INF_F, a1 = -CUDART_INF_F, a2 = -CUDART_INF_F, a3 = -CUDART_INF_F;
      auto max_chunk = [&](const uint32_t (&v)[32]) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          a0 = max3(a0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
          a1 = max3(a1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
          a2 = max3(a2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
          a3 = max3(a3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
        }
      };
      // Pass 1: the row maximum. Unmasked tile: chunks 2 and 3 first, then 0 and 1, which stay
      // in registers for the start of pass 2 (the S row is read from TMEM one and a half
      // times, never held whole: 128 live values would not fit the register budget).
      if (warp_full) {
        tmem_ld_32x32(tmem_s + 64, va);
        tmem_ld_32x32(tmem_s + 96, vb);
        tmem_ld_wait_dep(va);
        tmem_ld_wait_dep(vb);
        max_chunk(va);
        max_chunk(vb);
        tmem_ld_32x32(tmem_s, va);
        tmem_ld_32x32(tmem_s + 32, vb);
        tmem_ld_wait_dep(va);
        tmem_ld_wait_dep(vb);
        max_chunk(va);
        max_chunk(vb);
      } else {
        for (int g = 0; g < n_act; ++g) {
          tmem_ld_32x32(tmem_s + g * 32, va);
          tmem_ld_wait_dep(va);
          mask_chunk(va, g);
          max_chunk(va);
        }
      }
      const float mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
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

      if (__any_sync(0xffffffffu, rescale)) {
        // rare: bring this row of O in TMEM to the new reference, once the P V product of the
        // previous KV tile has landed
        const bool mine = mbar_wait_bounded(smem_u32(&ctl->pv_done[t]), (cnt - 1) & 1, wctx, 39, t);
        ok = __all_sync(0xffffffffu, mine) != 0;
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t v[32];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          __syncwarp();
          tmem_ld_32x32(tmem_o + g * 32, v);
          tmem_ld_wait_dep(v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__fmul_rn(__uint_as_float(v[i]), alpha));
          tmem_st_32x32(tmem_o + g * 32, v);
        }
      }
      // Pass 2: probabilities, 32 columns at a time; masked columns hold -inf and give 0.
      float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
      uint32_t w[32];
      auto exp_chunk = [&](const uint32_t (&v)[32], int half) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float x0, x1, x2, x3;
          fma2(x0, x1, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), c, c, neg, neg);
          fma2(x2, x3, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]), c, c, neg, neg);
          const float e0 = ex2_approx(x0), e1 = ex2_approx(x1), e2 = ex2_approx(x2), e3 = ex2_approx(x3);
          add2(ls0, ls1, ls0, ls1, e0, e1);
          add2(ls2, ls3, ls2, ls3, e2, e3);
          w[half * 16 + (i >> 1)] = pack_bf16(e0, e1);
          w[half * 16 + (i >> 1) + 1] = pack_bf16(e2, e3);
        }
      };
      if (warp_full) {
        exp_chunk(va, 0);
        tmem_ld_32x32(tmem_s + 64, va);        // chunk 2 on its way while chunk 1 is processed
        exp_chunk(vb, 1);
        tmem_st_32x32(tmem_s, w);              // P columns [0,64) as 32 packed words over S columns [0,32)
        tmem_ld_wait_dep(va);
        tmem_ld_32x32(tmem_s + 96, vb);
        exp_chunk(va, 0);
        tmem_st_wait();                        // first half of P is in TMEM: let its P V product start
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full[t][0]));
        tmem_ld_wait_dep(vb);
        exp_chunk(vb, 1);
        tmem_st_32x32(tmem_s + 32, w);         // P columns [64,128) over S columns [32,64)
      } else {
        // chunks past n_act are masked for every row of the warp: their P is zero, no exp
#pragma unroll
        for (int hblk = 0; hblk < 2; ++hblk) {
#pragma unroll
          for (int g2 = 0; g2 < 2; ++g2) {
            const int g = hblk * 2 + g2;
            if (g < n_act) {
              tmem_ld_32x32(tmem_s + g * 32, va);
              tmem_ld_wait_dep(va);
              mask_chunk(va, g);
              exp_chunk(va, g2);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) w[g2 * 16 + i] = 0u;
            }
          }
          // P of this half overwrites S columns [32 hblk, 32 hblk + 32): chunk hblk, already read
          tmem_st_32x32(tmem_s + hblk * 32, w);
          if (hblk == 0) {
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full[t][0]));
          }
        }
      }
      l = __fmaf_rn(l, alpha, __fadd_rn(__fadd_rn(ls0, ls1), __fadd_rn(ls2, ls3)));
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full[t][1]));
    }

    if (ok && tc.n_kv > 0) {
      const bool mine = mbar_wait_bounded(smem_u32(&ctl->pv_done[t]), (cnt - 1) & 1, wctx, 37, t);
      ok = __all_sync(0xffffffffu, mine) != 0;
    }
    if (ok && tc.n_kv > 0) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? __fdiv_rn(1.f, l) : 0.f;
      // The row goes out 32 columns at a time straight from registers (shared memory bandwidth
      // belongs to the MMAs), with the next TMEM load in flight while a chunk is stored.
      uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<long long>(tok0 + q_pos) * p.out_stride + tc.h * kD);
      uint32_t va[32], vb[32];
      auto emit = [&](const uint32_t (&v)[32], int g) {
        if (q_pos < p.seq_len) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w4;
            w4.x = pack_bf16(__fmul_rn(__uint_as_float(v[i]), inv), __fmul_rn(__uint_as_float(v[i + 1]), inv));
            w4.y = pack_bf16(__fmul_rn(__uint_as_float(v[i + 2]), inv), __fmul_rn(__uint_as_float(v[i + 3]), inv));
            w4.z = pack_bf16(__fmul_rn(__uint_as_float(v[i + 4]), inv), __fmul_rn(__uint_as_float(v[i + 5]), inv));
            w4.w = pack_bf16(__fmul_rn(__uint_as_float(v[i + 6]), inv), __fmul_rn(__uint_as_float(v[i + 7]), inv));
            dst[g * 4 + (i >> 3)] = w4;
          }
        }
      };
      tmem_ld_32x32(tmem_o, va);
      tmem_ld_32x32(tmem_o + 32, vb);
      tmem_ld_wait_dep(va);
      tmem_ld_wait_dep(vb);
      emit(va, 0);
      tmem_ld_32x32(tmem_o + 64, va);
      emit(vb, 1);
      tmem_ld_32x32(tmem_o + 96, vb);
      tmem_ld_wait_dep(va);
      tmem_ld_wait_dep(vb);
      emit(va, 2);
      emit(vb, 3);
      if (p.lse && q_pos < p.seq_len)
        p.lse[(static_cast<long long>(b) * p.hq + tc.h) * p.seq_len + q_pos] =
            __fmaf_rn(lg2_approx(l), 0.6931471805599453f, __fmul_rn(m, p.scale));
      // the O columns are read: order those reads before this warp's next arrival on p_full,
      // after which the MMA warp overwrites O
      tc_fence_before_sync();
    }
    }  // items
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
  p.pair_heads = ((hq / hkv) % 2 == 0) ? 1 : 0;
  const unsigned n_items = p.pair_heads ? static_cast<unsigned>(batch) * (hq / 2) * n_qt
                                        : static_cast<unsigned>(batch) * hq * ((n_qt + 1) / 2);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned grid = n_items < static_cast<unsigned>(sms) ? n_items : static_cast<unsigned>(sms);
  attention_fwd_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
