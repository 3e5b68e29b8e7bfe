// Fused temperature / top-k / top-p token sampling for sm_100a: one CTA per row, one launch
// per call, the logits row is read once from HBM (later passes hit L2).
//
// Semantics (the order the reference gets from FlashInfer's default "top_k_first",
// rl_engine/kernels/sampling.py:61-64, with the temperature applied once):
//   1. y = logits / temperature
//   2. keep the k largest y; ties at the k-th value are kept in increasing token-id order
//   3. softmax over the survivors, sorted by (y descending, token id ascending); keep token i
//      while the probability mass of the tokens before it is <= top_p
//   4. draw u from Philox4x32-10 keyed by (seed, row id, step) and invert the CDF
// Probability masses are 32.32 fixed-point integers (csrc/common/detmath.h), so every sum is
// exact and order-free: the token depends only on (row contents, seed, row id, step), not on
// the batch size, the launch shape or the schedule, and the C++ CPU path reproduces it bit
// for bit.
//
// Three kernels:
//   sample_topk_kernel     top_k in [1, 1024] (greedy = top_k 1), optional top_p
//   sample_topk_cluster_kernel  the same for 16-bit logits and few rows: a cluster of 2 or 4
//                          CTAs per row, candidates exchanged through distributed shared memory
//   sample_general_kernel  no top_k (or k > 1024), optional top_p: threshold search by radix
//                          descent on (count, mass) histograms; for bf16 rows in one step on a
//                          histogram of counts per key (the mass of a key is a function of the key)
#include <cstdint>
#include <cstdlib>
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../common/detmath.h"
#include "sampling.h"

namespace ka {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kCandCap = 4096;
constexpr int kMaxTopK = 1024;

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kVec = 4;
  static constexpr int kLowBit = 0;
  static constexpr bool kPacked = false;
  static constexpr uint32_t kInf2 = 0;
  __device__ static float to_float(float v) { return v; }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static constexpr int kLowBit = 16;
  static constexpr bool kPacked = true;
  static constexpr uint32_t kInf2 = 0x7F807F80u;  // +inf bit pattern, twice
  __device__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <>
struct Elem<__half> {
  static constexpr int kVec = 8;
  static constexpr int kLowBit = 13;
  static constexpr bool kPacked = true;
  static constexpr uint32_t kInf2 = 0x7C007C00u;
  __device__ static float to_float(__half v) { return __half2float(v); }
};

// Visit every element of a row once: 16-byte vector loads when the row allows it.
template <typename T, typename F>
__device__ __forceinline__ void for_each_key(const T* __restrict__ row, int v, bool vec_ok, F&& f) {
  constexpr int kVec = Elem<T>::kVec;
  const int tid = threadIdx.x;
  if (vec_ok) {
    const int nvec = v / kVec;
    const uint4* p = reinterpret_cast<const uint4*>(row);
    for (int i = tid; i < nvec; i += blockDim.x) {
      const uint4 raw = p[i];
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < kVec; ++j) f(float_to_key(Elem<T>::to_float(e[j])), i * kVec + j);
    }
    for (int i = nvec * kVec + tid; i < v; i += blockDim.x) f(float_to_key(Elem<T>::to_float(row[i])), i);
  } else {
    for (int i = tid; i < v; i += blockDim.x) f(float_to_key(Elem<T>::to_float(row[i])), i);
  }
}

// The same visit with four 16-byte loads in flight per thread (a single CTA walking a row is
// bound by the latency of its loads). The order of the visits differs, so only for callbacks
// that do not depend on it.
template <typename T, typename F>
__device__ __forceinline__ void for_each_key_x4(const T* __restrict__ row, int v, bool vec_ok, F&& f) {
  constexpr int kVec = Elem<T>::kVec;
  if (!vec_ok) {
    for_each_key<T>(row, v, false, f);
    return;
  }
  const int tid = threadIdx.x;
  const int stride = blockDim.x;
  const int nvec = v / kVec;
  const uint4* p = reinterpret_cast<const uint4*>(row);
  int i = tid;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) raw[u] = p[i + u * stride];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
      for (int j = 0; j < kVec; ++j) f(float_to_key(Elem<T>::to_float(e[j])), (i + u * stride) * kVec + j);
    }
  }
  for (; i < nvec; i += stride) {
    const uint4 raw = p[i];
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < kVec; ++j) f(float_to_key(Elem<T>::to_float(e[j])), i * kVec + j);
  }
  for (int k = nvec * kVec + tid; k < v; k += stride) f(float_to_key(Elem<T>::to_float(row[k])), k);
}

__device__ __forceinline__ int block_sum_int(int v, int* s_warp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) s_warp[warp] = v;
  __syncthreads();
  int t = (lane < static_cast<int>(blockDim.x >> 5)) ? s_warp[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// Exclusive prefix sum over the block in thread order; `total` receives the block sum.
__device__ __forceinline__ unsigned long long block_exscan_u64(unsigned long long v, unsigned long long* s_warp,
                                                             unsigned long long& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  unsigned long long w = (lane < static_cast<int>(blockDim.x >> 5)) ? s_warp[lane] : 0ull;
  unsigned long long winc = w;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long n = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += n;
  }
  total = __shfl_sync(0xffffffffu, winc, 31);
  const unsigned long long warp_off = __shfl_sync(0xffffffffu, winc - w, warp);
  return warp_off + inc - v;
}

struct TopkSmem {
  uint32_t cand_key[kCandCap];
  uint32_t cand_idx[kCandCap];
  uint32_t sorted_key[kMaxTopK];
  uint32_t sorted_idx[kMaxTopK];
  unsigned long long mass[kMaxTopK];
  unsigned long long scan[kWarps];
  int red[kWarps];
  int count;
};

// Final step of the top-k path, run by one warp: survivors sorted by (key desc, id asc) with
// masses q[0..n); apply top-p, draw, return the position picked. All sums are integers, so
// the warp-parallel prefix sums give exactly the result of a serial walk.
__device__ __forceinline__ int pick_sorted_warp(const unsigned long long* q, int n, float top_p, uint32_t u24) {
  const int lane = threadIdx.x & 31;
  // lane owns the contiguous slice [lane * per, lane * per + per)
  const int per = (n + 31) / 32;
  const int lo = min(n, lane * per), hi = min(n, lo + per);
  unsigned long long mine = 0;
  for (int i = lo; i < hi; ++i) mine += q[i];
  unsigned long long inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  const unsigned long long z = __shfl_sync(0xffffffffu, inc, 31);
  const unsigned long long before = inc - mine;  // mass of the elements before this lane's slice
  int keep = n;
  unsigned long long zk = z;
  if (top_p < 1.0f) {
    // keep = first i > 0 with (mass before i) > limit, else n
    const unsigned long long limit = mass_fraction(static_cast<double>(top_p), z);
    int first = n;
    unsigned long long cum = before;
    for (int i = lo; i < hi; ++i) {
      if (i > 0 && cum > limit) {
        first = i;
        break;
      }
      cum += q[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
    keep = first;
    // zk = mass of the first `keep` elements
    unsigned long long part = 0;
    for (int i = lo; i < min(hi, keep); ++i) part += q[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    zk = part;
  }
  const unsigned long long target = mass_scale_u24(u24, zk);
  int pick = keep - 1;
  {
    int first = n;
    unsigned long long acc = before;
    for (int i = lo; i < min(hi, keep); ++i) {
      acc += q[i];
      if (acc > target) {
        first = i;
        break;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
    if (first < keep) pick = first;
  }
  return pick;
}

constexpr int kTopkThreads = 512;

// Two 16-bit floats (bf16 or fp16 bit patterns) -> two order-preserving 16-bit keys; NaN -> 0.
template <typename T>
__device__ __forceinline__ uint32_t key16x2(uint32_t w) {
  const uint32_t nan = __vcmpgtu2(w & 0x7FFF7FFFu, Elem<T>::kInf2);
  const uint32_t sign = (w >> 15) & 0x00010001u;
  const uint32_t k = w ^ (sign * 0xFFFFu | 0x80008000u);
  return k & ~nan;
}

template <typename T>
__device__ __forceinline__ T from_bits16(uint32_t h) {
  const unsigned short us = static_cast<unsigned short>(h);
  return *reinterpret_cast<const T*>(&us);
}

// Second half of the top-k path, shared by the one-CTA and the cluster kernel: n_cand candidates
// sit in s.cand_key / s.cand_idx (in any order; if there are more than the buffer holds the row
// is searched exactly), the kk largest by (key desc, id asc) are the survivors; masses, top-p
// and the draw follow. Run by all threads of one CTA.
template <typename T>
__device__ __forceinline__ void topk_finish(TopkSmem& s, int n_cand, const T* __restrict__ rp, int v, bool vec_ok,
                                            int kk, float inv_temp, float top_p, unsigned long long seed,
                                            unsigned long long step, const long long* __restrict__ row_ids, int row,
                                            int* __restrict__ out) {
  const int tid = threadIdx.x;
  const int nt = blockDim.x;
  if (n_cand > kCandCap) {
    // ---- rare: more ties / near-ties than the candidate buffer holds. Exact radix select by
    // counting passes, then an index-ordered pick among the ties at the threshold.
    uint32_t tau = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = tau | (1u << bit);
      int local = 0;
      for_each_key<T>(rp, v, vec_ok, [&](uint32_t key, int) { local += (key >= cand) ? 1 : 0; });
      if (block_sum_int(local, s.red) >= kk) tau = cand;
    }
    int local_gt = 0;
    for_each_key<T>(rp, v, vec_ok, [&](uint32_t key, int) { local_gt += (key > tau) ? 1 : 0; });
    const int n_gt = block_sum_int(local_gt, s.red);
    const int quota = kk - n_gt;
    if (tid == 0) s.count = 0;
    __syncthreads();
    for_each_key<T>(rp, v, vec_ok, [&](uint32_t key, int i) {
      if (key > tau) {
        const int slot = atomicAdd(&s.count, 1);
        s.cand_key[slot] = key;
        s.cand_idx[slot] = static_cast<uint32_t>(i);
      }
    });
    __syncthreads();
    unsigned long long tie_base = 0;
    constexpr int kPer = 8;
    for (int base = 0; base < v && tie_base < static_cast<unsigned long long>(quota); base += nt * kPer) {
      const int i0 = base + tid * kPer;
      int mine = 0;
      for (int j = 0; j < kPer; ++j) {
        const int i = i0 + j;
        if (i < v && float_to_key(Elem<T>::to_float(rp[i])) == tau) ++mine;
      }
      unsigned long long total;
      unsigned long long off = tie_base + block_exscan_u64(static_cast<unsigned long long>(mine), s.scan, total);
      for (int j = 0; j < kPer; ++j) {
        const int i = i0 + j;
        if (i < v && float_to_key(Elem<T>::to_float(rp[i])) == tau) {
          if (off < static_cast<unsigned long long>(quota)) {
            s.cand_key[n_gt + off] = tau;
            s.cand_idx[n_gt + off] = static_cast<uint32_t>(i);
          }
          ++off;
        }
      }
      tie_base += total;
    }
    __syncthreads();
    n_cand = kk;
  }

  // ---- rank sort of the candidates by (key desc, id asc); the first kk are the survivors
  for (int i = tid; i < n_cand; i += nt) {
    const uint32_t ki = s.cand_key[i], ii = s.cand_idx[i];
    int rank = 0;
    for (int j = 0; j < n_cand; ++j) {
      const uint32_t kj = s.cand_key[j], ij = s.cand_idx[j];
      rank += (kj > ki || (kj == ki && ij < ii)) ? 1 : 0;
    }
    if (rank < kk) {
      s.sorted_key[rank] = ki;
      s.sorted_idx[rank] = ii;
    }
  }
  __syncthreads();

  // ---- masses, top-p, draw
  const float y0 = mul_rn(key_to_float(s.sorted_key[0]), inv_temp);
  for (int i = tid; i < kk; i += nt) {
    const float y = mul_rn(key_to_float(s.sorted_key[i]), inv_temp);
    s.mass[i] = mass_fixed(exp_det(sub_rn(y, y0)));
  }
  __syncthreads();
  if (tid < 32) {
    const unsigned long long rid = row_ids ? static_cast<unsigned long long>(row_ids[row])
                                           : static_cast<unsigned long long>(row);
    const int pos = pick_sorted_warp(s.mass, kk, top_p, uniform_u24(seed, rid, step));
    if (tid == 0) out[row] = static_cast<int>(s.sorted_idx[pos]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads, 2)
sample_topk_kernel(const T* __restrict__ logits, long long row_stride, int v, const long long* __restrict__ row_ids,
                   float inv_temp, int top_k, float top_p, unsigned long long seed, unsigned long long step,
                   int* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TopkSmem& s = *reinterpret_cast<TopkSmem*>(smem_raw);
  const int tid = threadIdx.x;
  const int nt = blockDim.x;
  const int row = blockIdx.x;
  const T* rp = logits + static_cast<long long>(row) * row_stride;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(rp) & 15u) == 0;
  const int kk = min(min(top_k, kMaxTopK), v);
  uint32_t lower = 0;  // 32-bit key: at least kk elements of the row are >= lower

  if (tid == 0) s.count = 0;
  if constexpr (Elem<T>::kPacked) {
    // ---- 16-bit inputs: keys stay packed two per register. Each thread keeps two running
    // maxima (even / odd elements), 1024 in all; the kk-th largest of them bounds the kk-th
    // largest element of the row from below.
    uint32_t tm2 = 0;
    const int nvec = vec_ok ? v / 8 : 0;
    const uint4* vp = reinterpret_cast<const uint4*>(rp);
    // eight independent 16-byte loads in flight per thread: the row is latency-, not
    // bandwidth-bound when a single CTA pulls it
    constexpr int kU = 8;
    int i = tid;
    for (; i + (kU - 1) * nt < nvec; i += kU * nt) {
      uint4 raw[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) raw[u] = __ldg(vp + i + u * nt);
#pragma unroll
      for (int u = 0; u < kU; ++u)
        tm2 = __vmaxu2(tm2, __vmaxu2(__vmaxu2(key16x2<T>(raw[u].x), key16x2<T>(raw[u].y)),
                                     __vmaxu2(key16x2<T>(raw[u].z), key16x2<T>(raw[u].w))));
    }
    for (; i < nvec; i += nt) {
      const uint4 raw = __ldg(vp + i);
      tm2 = __vmaxu2(tm2, __vmaxu2(__vmaxu2(key16x2<T>(raw.x), key16x2<T>(raw.y)),
                                   __vmaxu2(key16x2<T>(raw.z), key16x2<T>(raw.w))));
    }
    const unsigned short* hp = reinterpret_cast<const unsigned short*>(rp);
    for (int t = nvec * 8 + tid; t < v; t += nt) tm2 = __vmaxu2(tm2, key16x2<T>(hp[t]) & 0xFFFFu);
    const uint32_t m_lo = tm2 & 0xFFFFu, m_hi = tm2 >> 16;
    uint32_t low16 = 0;
    for (int bit = 15; bit >= 0; --bit) {
      const uint32_t cand = low16 | (1u << bit);
      const int cnt = __syncthreads_count(m_lo >= cand) + __syncthreads_count(m_hi >= cand);
      if (cnt >= kk) low16 = cand;
    }
    // ---- pass 2 (L2): collect every element whose 16-bit key is >= the bound
    const uint32_t low2 = low16 * 0x00010001u;
    auto push = [&](uint32_t bits16, int idx) {
      const int slot = atomicAdd(&s.count, 1);
      if (slot < kCandCap) {
        s.cand_key[slot] = float_to_key(Elem<T>::to_float(from_bits16<T>(bits16)));
        s.cand_idx[slot] = static_cast<uint32_t>(idx);
      }
    };
    auto scan_vec = [&](const uint4& raw, int vi) {
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      const uint32_t h0 = __vcmpgeu2(key16x2<T>(w[0]), low2), h1 = __vcmpgeu2(key16x2<T>(w[1]), low2);
      const uint32_t h2 = __vcmpgeu2(key16x2<T>(w[2]), low2), h3 = __vcmpgeu2(key16x2<T>(w[3]), low2);
      if ((h0 | h1 | h2 | h3) == 0u) return;
      const uint32_t hit[4] = {h0, h1, h2, h3};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (hit[j] & 0xFFFFu) push(w[j] & 0xFFFFu, vi * 8 + 2 * j);
        if (hit[j] >> 16) push(w[j] >> 16, vi * 8 + 2 * j + 1);
      }
    };
    i = tid;
    for (; i + (kU - 1) * nt < nvec; i += kU * nt) {
      uint4 raw[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) raw[u] = __ldg(vp + i + u * nt);
#pragma unroll
      for (int u = 0; u < kU; ++u) scan_vec(raw[u], i + u * nt);
    }
    for (; i < nvec; i += nt) scan_vec(__ldg(vp + i), i);
    for (int t = nvec * 8 + tid; t < v; t += nt)
      if ((key16x2<T>(hp[t]) & 0xFFFFu) >= low16) push(hp[t], t);
  } else {
    // ---- 32-bit inputs
    uint32_t tm[2] = {0, 0};
    for_each_key<T>(rp, v, vec_ok, [&](uint32_t key, int i) { tm[i & 1] = max(tm[i & 1], key); });
    for (int bit = 31; bit >= Elem<T>::kLowBit; --bit) {
      const uint32_t cand = lower | (1u << bit);
      const int cnt = __syncthreads_count(tm[0] >= cand) + __syncthreads_count(tm[1] >= cand);
      if (cnt >= kk) lower = cand;
    }
    for_each_key<T>(rp, v, vec_ok, [&](uint32_t key, int i) {
      if (key >= lower) {
        const int slot = atomicAdd(&s.count, 1);
        if (slot < kCandCap) {
          s.cand_key[slot] = key;
          s.cand_idx[slot] = static_cast<uint32_t>(i);
        }
      }
    });
  }
  __syncthreads();
  int n_cand = s.count;
  __syncthreads();

  topk_finish<T>(s, n_cand, rp, v, vec_ok, kk, inv_temp, top_p, seed, step, row_ids, row, out);
}

// ------------------------------------------------------------------------------------------
// Cluster variant of the top-k kernel for 16-bit logits and few rows: C CTAs of a thread-block
// cluster share one row, so that C SMs pull it instead of one (a single CTA is bound by the
// latency of its own loads; with 64 rows only 64 of the 148 SMs would work at all).
//   1. CTA r scans its 1/C of the row and finds, as above, a bound that at least kk of its own
//      elements reach. The largest of the C bounds is valid for the whole row: the part that
//      produced it alone holds kk elements at or above it.
//   2. The bounds travel through distributed shared memory (one store per peer, one cluster
//      barrier); every CTA collects the elements of its part that reach the common bound.
//   3. Counts are exchanged the same way, every CTA copies its candidates into CTA 0's list at
//      its offset (remote shared-memory stores), and CTA 0 finishes as the one-CTA kernel does.
// The survivors are the kk largest by (key desc, id asc) of a candidate set that contains them
// all, so the token is the one the one-CTA kernel and the CPU library return. No multicast.
// ------------------------------------------------------------------------------------------
constexpr int kMaxCluster = 4;

struct ClusterXchg {
  uint32_t low[kMaxCluster];   // bound found by each CTA of the cluster
  int cnt[kMaxCluster];        // candidates collected by each CTA
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p)), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_remote_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

template <typename T, int C>
__global__ void __launch_bounds__(kTopkThreads, 2)
sample_topk_cluster_kernel(const T* __restrict__ logits, long long row_stride, int v,
                           const long long* __restrict__ row_ids, float inv_temp, int top_k, float top_p,
                           unsigned long long seed, unsigned long long step, int* __restrict__ out) {
  static_assert(Elem<T>::kPacked, "the cluster kernel takes 16-bit logits");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TopkSmem& s = *reinterpret_cast<TopkSmem*>(smem_raw);
  ClusterXchg& x = *reinterpret_cast<ClusterXchg*>(smem_raw + sizeof(TopkSmem));
  const int tid = threadIdx.x;
  const int nt = blockDim.x;
  const int row = blockIdx.x / C;
  const int cr = static_cast<int>(cluster_rank());
  const T* rp = logits + static_cast<long long>(row) * row_stride;  // 16-byte aligned (checked by the host)
  const int kk = min(min(top_k, kMaxTopK), v);
  if (tid == 0) s.count = 0;

  // ---- this CTA's part: vectors [v0, v1) of the row, the scalar tail goes to the last CTA
  const int nvec = v / 8;
  const int v0 = static_cast<int>(static_cast<long long>(nvec) * cr / C);
  const int v1 = static_cast<int>(static_cast<long long>(nvec) * (cr + 1) / C);
  const uint4* vp = reinterpret_cast<const uint4*>(rp);
  const unsigned short* hp = reinterpret_cast<const unsigned short*>(rp);
  const bool has_tail = cr == C - 1;
  constexpr int kU = 8;
  uint32_t tm2 = 0;
  int i = v0 + tid;
  for (; i + (kU - 1) * nt < v1; i += kU * nt) {
    uint4 raw[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) raw[u] = __ldg(vp + i + u * nt);
#pragma unroll
    for (int u = 0; u < kU; ++u)
      tm2 = __vmaxu2(tm2, __vmaxu2(__vmaxu2(key16x2<T>(raw[u].x), key16x2<T>(raw[u].y)),
                                   __vmaxu2(key16x2<T>(raw[u].z), key16x2<T>(raw[u].w))));
  }
  for (; i < v1; i += nt) {
    const uint4 raw = __ldg(vp + i);
    tm2 = __vmaxu2(tm2, __vmaxu2(__vmaxu2(key16x2<T>(raw.x), key16x2<T>(raw.y)),
                                 __vmaxu2(key16x2<T>(raw.z), key16x2<T>(raw.w))));
  }
  if (has_tail)
    for (int t = nvec * 8 + tid; t < v; t += nt) tm2 = __vmaxu2(tm2, key16x2<T>(hp[t]) & 0xFFFFu);
  const uint32_t m_lo = tm2 & 0xFFFFu, m_hi = tm2 >> 16;
  uint32_t low16 = 0;
  for (int bit = 15; bit >= 0; --bit) {
    const uint32_t cand = low16 | (1u << bit);
    const int cnt = __syncthreads_count(m_lo >= cand) + __syncthreads_count(m_hi >= cand);
    if (cnt >= kk) low16 = cand;
  }
  // ---- the largest of the C bounds serves the whole row
  if (tid < C) st_remote_u32(map_to_cta(&x.low[cr], static_cast<uint32_t>(tid)), low16);
  cluster_sync_all();
#pragma unroll
  for (int r = 0; r < C; ++r) low16 = max(low16, x.low[r]);

  // ---- collect this part's elements at or above the bound (second pass: L2)
  const uint32_t low2 = low16 * 0x00010001u;
  auto push = [&](uint32_t bits16, int idx) {
    const int slot = atomicAdd(&s.count, 1);
    if (slot < kCandCap) {
      s.cand_key[slot] = float_to_key(Elem<T>::to_float(from_bits16<T>(bits16)));
      s.cand_idx[slot] = static_cast<uint32_t>(idx);
    }
  };
  auto scan_vec = [&](const uint4& raw, int vi) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    const uint32_t h0 = __vcmpgeu2(key16x2<T>(w[0]), low2), h1 = __vcmpgeu2(key16x2<T>(w[1]), low2);
    const uint32_t h2 = __vcmpgeu2(key16x2<T>(w[2]), low2), h3 = __vcmpgeu2(key16x2<T>(w[3]), low2);
    if ((h0 | h1 | h2 | h3) == 0u) return;
    const uint32_t hit[4] = {h0, h1, h2, h3};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (hit[j] & 0xFFFFu) push(w[j] & 0xFFFFu, vi * 8 + 2 * j);
      if (hit[j] >> 16) push(w[j] >> 16, vi * 8 + 2 * j + 1);
    }
  };
  i = v0 + tid;
  for (; i + (kU - 1) * nt < v1; i += kU * nt) {
    uint4 raw[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) raw[u] = __ldg(vp + i + u * nt);
#pragma unroll
    for (int u = 0; u < kU; ++u) scan_vec(raw[u], i + u * nt);
  }
  for (; i < v1; i += nt) scan_vec(__ldg(vp + i), i);
  if (has_tail)
    for (int t = nvec * 8 + tid; t < v; t += nt)
      if ((key16x2<T>(hp[t]) & 0xFFFFu) >= low16) push(hp[t], t);
  __syncthreads();
  const int mine = s.count;  // may exceed the buffer: then the total does too and CTA 0 searches the row exactly
  if (tid < C) st_remote_u32(map_to_cta(&x.cnt[cr], static_cast<uint32_t>(tid)), static_cast<uint32_t>(mine));
  cluster_sync_all();
  int total = 0, offset = 0;
#pragma unroll
  for (int r = 0; r < C; ++r) {
    if (r < cr) offset += x.cnt[r];
    total += x.cnt[r];
  }
  // ---- candidates of the other CTAs move into CTA 0's list
  if (cr != 0 && total <= kCandCap) {
    const uint32_t dst_key = map_to_cta(&s.cand_key[0], 0u), dst_idx = map_to_cta(&s.cand_idx[0], 0u);
    for (int j = tid; j < mine; j += nt) {
      st_remote_u32(dst_key + 4u * static_cast<uint32_t>(offset + j), s.cand_key[j]);
      st_remote_u32(dst_idx + 4u * static_cast<uint32_t>(offset + j), s.cand_idx[j]);
    }
  }
  cluster_sync_all();  // after this barrier nobody touches another CTA's shared memory
  if (cr != 0) return;
  topk_finish<T>(s, total, rp, v, true, kk, inv_temp, top_p, seed, step, row_ids, row, out);
}

// ------------------------------------------------------------------------------------------
// General kernel: no top-k bound small enough for the candidate list.
//
// The kept set is a prefix of the order (key desc, id asc): the first n* elements with
//   n* = min(k, smallest n with mass(first n) > top_p * Z_k)      (Z_k = mass of the first k)
// The prefix is located by radix descent over the key bits (11, 11, 10) with exact integer
// histograms of element counts and fixed-point masses (fp32 and fp16 rows), or at full key
// resolution from a histogram of counts per key (bf16 rows, descend16 below); ties at the
// threshold key are cut in token-id order. The draw inverts the CDF over the kept set in
// token-id order: every thread owns a contiguous piece of the row, two block scans give it the
// ties and the kept mass before its piece.
// Measured, bf16 [G, 128256] ~ N(0, 2), T = 0.7, top_p = 0.9 without top_k: 108 us at G = 64 and
// 211 us at G = 256 (two waves of one CTA per SM); with the three-level descent and a block scan
// per 8192 elements in the draw it took about 550 us.
// ------------------------------------------------------------------------------------------
constexpr int kBins = 2048;

struct GeneralSmem {
  unsigned int cnt[kBins];
  unsigned long long mass[kBins];
  unsigned long long scan[kWarps];
  int red[kWarps];
  uint32_t max_key;
  // results of a descent
  uint32_t prefix;
  unsigned long long above_cnt;
  unsigned long long above_mass;
  int sel_bin;
  int pick;
};

constexpr int kGeneralSmemBytes = (static_cast<int>(sizeof(GeneralSmem)) + 15) / 16 * 16;

// One descent: find key tau and the (count, mass) strictly above it such that the element
// that crosses `limit` lies among the keys equal to tau. `by_mass` selects the criterion:
//   by count: first key where count_above + count(key) >  limit  (limit = k - 1)
//   by mass : first key where mass_above  + mass(key)  >  limit
template <typename T>
__device__ void descend(const T* rp, int v, bool vec_ok, float inv_temp, float y_max, bool by_mass,
                        unsigned long long limit, GeneralSmem& s, uint32_t& tau, unsigned long long& above_cnt,
                        unsigned long long& above_mass) {
  const int tid = threadIdx.x;
  uint32_t prefix = 0;
  int known_bits = 0;
  above_cnt = 0;
  above_mass = 0;
  const int widths[3] = {11, 11, 10};
  for (int round = 0; round < 3; ++round) {
    const int w = widths[round];
    const int shift = 32 - known_bits - w;
    for (int b = tid; b < kBins; b += kThreads) {
      s.cnt[b] = 0;
      s.mass[b] = 0;
    }
    __syncthreads();
    for_each_key<T>(rp, v, vec_ok, [&](uint32_t key, int) {
      const bool match = known_bits == 0 || (key >> (32 - known_bits)) == (prefix >> (32 - known_bits));
      if (match) {
        const int bin = (key >> shift) & ((1 << w) - 1);
        atomicAdd(&s.cnt[bin], 1u);
        const float y = mul_rn(key_to_float(key), inv_temp);
        atomicAdd(&s.mass[bin], mass_fixed(exp_det(sub_rn(y, y_max))));
      }
    });
    __syncthreads();
    if (tid == 0) {
      unsigned long long c = above_cnt, m = above_mass;
      int sel = 0;
      for (int b = (1 << w) - 1; b >= 0; --b) {
        const unsigned long long nc = c + s.cnt[b], nm = m + s.mass[b];
        const bool crosses = by_mass ? (nm > limit) : (nc > limit);
        if (crosses || b == 0) {
          sel = b;
          break;
        }
        c = nc;
        m = nm;
      }
      s.sel_bin = sel;
      s.above_cnt = c;
      s.above_mass = m;
    }
    __syncthreads();
    prefix |= static_cast<uint32_t>(s.sel_bin) << shift;
    above_cnt = s.above_cnt;
    above_mass = s.above_mass;
    known_bits += w;
    __syncthreads();
  }
  tau = prefix;
}

// ---- bf16 rows: one descent at full key resolution ------------------------------------------
// A bf16 value has 16 significant bits, so key >> 16 names the key and the mass of a key is a
// function of the key alone: a histogram of element COUNTS per key gives every (count, mass)
// the search needs, mass(key) * count(key) being the exact integer sum the element-wise walk
// would produce. The 65536 keys are taken in two halves of 32768 counters (128 KiB of shared
// memory), upper half (non-negative values) first; the second pass over the row only happens
// when the threshold lies among the negative values. No 64-bit atomics, and the counters of a
// row spread over hundreds of keys instead of a few dozen coarse bins.
constexpr int kHalfBins = 32768;
constexpr int kHistBytes = kHalfBins * 4;

__device__ __forceinline__ uint32_t key16_to_key(uint32_t k16) {
  if (k16 == 0) return 0u;  // NaN
  return (k16 << 16) | ((k16 & 0x8000u) ? 0u : 0xFFFFu);
}

__device__ __forceinline__ unsigned long long key16_mass(uint32_t k16, float inv_temp, float y_max) {
  const float y = mul_rn(key_to_float(key16_to_key(k16)), inv_temp);
  return mass_fixed(exp_det(sub_rn(y, y_max)));
}

// Same contract as descend(); `present` additionally receives the number of elements equal to tau.
template <typename T>
__device__ void descend16(const T* rp, int v, bool vec_ok, float inv_temp, float y_max, bool by_mass,
                          unsigned long long limit, GeneralSmem& s, unsigned int* hist, uint32_t& tau,
                          unsigned long long& above_cnt, unsigned long long& above_mass,
                          unsigned long long& present) {
  const int tid = threadIdx.x;
  constexpr int kPer = kHalfBins / kThreads;  // bins per thread, walked from the top down
  unsigned long long carry_cnt = 0, carry_mass = 0;
  for (int half = 1; half >= 0; --half) {
    for (int b = tid; b < kHalfBins; b += kThreads) hist[b] = 0;
    if (tid == 0) s.sel_bin = -1;
    __syncthreads();
    for_each_key_x4<T>(rp, v, vec_ok, [&](uint32_t key, int) {
      const uint32_t k16 = key >> 16;
      if (static_cast<int>(k16 >> 15) == half) atomicAdd(&hist[k16 & 0x7FFFu], 1u);
    });
    __syncthreads();
    const int top = kHalfBins - 1 - tid * kPer;
    const uint32_t hi_bit = static_cast<uint32_t>(half) << 15;
    // totals of this thread's bins; the walk starts at a different bin in every lane, so that
    // the lanes of a warp (whose ranges are kPer words apart) read different banks
    static_assert(kPer == 32, "the rotation below assumes one bin per bank and lane");
    unsigned long long my_cnt = 0, my_mass = 0;
    for (int j = 0; j < kPer; ++j) {
      const int b = top - ((j + tid) & (kPer - 1));
      const unsigned int c = hist[b];
      if (c) {
        my_cnt += c;
        my_mass += c * key16_mass(hi_bit | static_cast<uint32_t>(b), inv_temp, y_max);
      }
    }
    unsigned long long tot_cnt, tot_mass;
    const unsigned long long pre_cnt = carry_cnt + block_exscan_u64(my_cnt, s.scan, tot_cnt);
    const unsigned long long pre_mass = carry_mass + block_exscan_u64(my_mass, s.scan, tot_mass);
    const unsigned long long crit_pre = by_mass ? pre_mass : pre_cnt;
    const unsigned long long crit_mine = by_mass ? my_mass : my_cnt;
    if (crit_pre <= limit && crit_pre + crit_mine > limit) {  // the crossing is in this thread's bins
      unsigned long long c = pre_cnt, m = pre_mass;
      for (int j = 0; j < kPer; ++j) {
        const unsigned int n = hist[top - j];
        const unsigned long long nc = c + n;
        const unsigned long long nm =
            m + (n ? n * key16_mass(hi_bit | static_cast<uint32_t>(top - j), inv_temp, y_max) : 0ull);
        if (by_mass ? (nm > limit) : (nc > limit)) {
          s.sel_bin = top - j;
          s.above_cnt = c;
          s.above_mass = m;
          break;
        }
        c = nc;
        m = nm;
      }
    }
    __syncthreads();
    if (s.sel_bin >= 0) {
      tau = key16_to_key(hi_bit | static_cast<uint32_t>(s.sel_bin));
      above_cnt = s.above_cnt;
      above_mass = s.above_mass;
      present = hist[s.sel_bin];
      __syncthreads();
      return;
    }
    carry_cnt += tot_cnt;
    carry_mass += tot_mass;
    __syncthreads();
  }
  // nothing crossed: the lowest key (NaN, mass 0), as the bitwise descent ends in bin 0 of every level
  tau = 0u;
  present = hist[0];
  above_cnt = carry_cnt - hist[0];
  above_mass = carry_mass;
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
sample_general_kernel(const T* __restrict__ logits, long long row_stride, int v, const long long* __restrict__ row_ids,
                      float inv_temp, int top_k, float top_p, unsigned long long seed, unsigned long long step,
                      int* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  GeneralSmem& s = *reinterpret_cast<GeneralSmem*>(smem_raw);
  constexpr bool kKey16 = std::is_same<T, __nv_bfloat16>::value;
  unsigned int* hist = reinterpret_cast<unsigned int*>(smem_raw + kGeneralSmemBytes);  // kKey16 only
  const int tid = threadIdx.x;
  const int row = blockIdx.x;
  const T* rp = logits + static_cast<long long>(row) * row_stride;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(rp) & 15u) == 0;

  // ---- row maximum
  uint32_t tmax = 0;
  for_each_key_x4<T>(rp, v, vec_ok, [&](uint32_t key, int) { tmax = max(tmax, key); });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tmax = max(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
  if (tid == 0) s.max_key = 0;
  __syncthreads();
  if ((tid & 31) == 0) atomicMax(&s.max_key, tmax);
  __syncthreads();
  const float y_max = mul_rn(key_to_float(s.max_key), inv_temp);

  // ---- where the kept prefix ends: (tau, number of ties at tau that are kept)
  uint32_t tau = 0;                     // threshold key
  unsigned long long tie_keep = ~0ull;  // ties at tau kept, in id order
  unsigned long long kept_mass = 0;     // mass of the kept set
  {
    // total mass and, if top_k is set, the top-k prefix
    unsigned long long k_above_cnt = 0, k_above_mass = 0;
    uint32_t k_tau = 0;
    unsigned long long k_ties = ~0ull;
    unsigned long long zk;
    const bool has_k = top_k > 0 && top_k < v;
    if (has_k) {
      if constexpr (kKey16) {
        unsigned long long unused;
        descend16<T>(rp, v, vec_ok, inv_temp, y_max, false, static_cast<unsigned long long>(top_k - 1), s, hist,
                     k_tau, k_above_cnt, k_above_mass, unused);
      } else {
        descend<T>(rp, v, vec_ok, inv_temp, y_max, false, static_cast<unsigned long long>(top_k - 1), s, k_tau,
                   k_above_cnt, k_above_mass);
      }
      k_ties = static_cast<unsigned long long>(top_k) - k_above_cnt;
      const float y = mul_rn(key_to_float(k_tau), inv_temp);
      zk = k_above_mass + k_ties * mass_fixed(exp_det(sub_rn(y, y_max)));
    } else {
      // everything is kept by the count criterion: Z = total mass
      unsigned long long local = 0;
      for_each_key_x4<T>(rp, v, vec_ok, [&](uint32_t key, int) {
        const float y = mul_rn(key_to_float(key), inv_temp);
        local += mass_fixed(exp_det(sub_rn(y, y_max)));
      });
      unsigned long long total;
      block_exscan_u64(local, s.scan, total);
      zk = total;
    }
    tau = has_k ? k_tau : 0u;
    tie_keep = k_ties;
    kept_mass = zk;
    if (top_p < 1.0f) {
      const unsigned long long limit = mass_fraction(static_cast<double>(top_p), zk);
      uint32_t p_tau;
      unsigned long long p_above_cnt, p_above_mass, p_present = 0;
      if constexpr (kKey16) {
        descend16<T>(rp, v, vec_ok, inv_temp, y_max, true, limit, s, hist, p_tau, p_above_cnt, p_above_mass,
                     p_present);
      } else {
        descend<T>(rp, v, vec_ok, inv_temp, y_max, true, limit, s, p_tau, p_above_cnt, p_above_mass);
      }
      // element i (in sorted order) is kept while the mass before it is <= limit
      const float y = mul_rn(key_to_float(p_tau), inv_temp);
      const unsigned long long q = mass_fixed(exp_det(sub_rn(y, y_max)));
      unsigned long long p_ties;
      if (p_above_mass > limit) {
        p_ties = 0;  // cannot happen: the descent stops at the first crossing key
      } else if (q == 0) {
        p_ties = ~0ull;
      } else {
        p_ties = (limit - p_above_mass) / q + 1;
      }
      // the tighter of the two prefixes wins
      bool p_tighter;
      if (!has_k) {
        p_tighter = true;
      } else if (p_tau != k_tau) {
        p_tighter = p_tau > k_tau;
      } else {
        p_tighter = p_ties < k_ties;
      }
      if (p_tighter) {
        tau = p_tau;
        tie_keep = p_ties;
        // the kept mass follows from the number of ties actually present
        unsigned long long present;
        if constexpr (kKey16) {
          present = p_present;  // the histogram had the count
        } else {
          int local = 0;
          for_each_key<T>(rp, v, vec_ok, [&](uint32_t key, int) { local += (key == p_tau) ? 1 : 0; });
          present = static_cast<unsigned long long>(block_sum_int(local, s.red));
        }
        const unsigned long long used = p_ties < present ? p_ties : present;
        tie_keep = used;
        kept_mass = p_above_mass + used * q;
      }
    }
  }

  // ---- draw: invert the CDF over the kept set in token-id order
  const unsigned long long rid = row_ids ? static_cast<unsigned long long>(row_ids[row])
                                         : static_cast<unsigned long long>(row);
  const unsigned long long target = mass_scale_u24(uniform_u24(seed, rid, step), kept_mass);
  if (tid == 0) s.pick = -1;
  // Thread t owns the elements [t * chunk, (t + 1) * chunk) and walks them in order, up to three
  // times: the ties before a thread and the kept mass before it come from two block scans.
  constexpr int kVec = Elem<T>::kVec;
  const int chunk = ((v + kThreads - 1) / kThreads + 7) & ~7;
  const int begin = min(v, tid * chunk), end = min(v, begin + chunk);
  auto walk = [&](auto&& f) {
    int i = begin;
    if (vec_ok) {
      for (; i + kVec <= end; i += kVec) {
        const uint4 raw = *reinterpret_cast<const uint4*>(rp + i);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < kVec; ++j) f(float_to_key(Elem<T>::to_float(e[j])), i + j);
      }
    }
    for (; i < end; ++i) f(float_to_key(Elem<T>::to_float(rp[i])), i);
  };
  unsigned long long my_ties = 0;
  walk([&](uint32_t key, int) { my_ties += (key == tau) ? 1u : 0u; });
  unsigned long long tie_total;
  const unsigned long long tie_first = block_exscan_u64(my_ties, s.scan, tie_total);
  // Visit the kept elements of the chunk in id order. The walk only sets a flag per element
  // (64 at a time); the masses are then computed for the flagged ones alone, so that a warp
  // runs the exponential as often as its busiest lane has kept elements, not once per element.
  auto walk_kept = [&](auto&& f) {
    unsigned long long tie_off = tie_first, bits = 0;
    int bits_base = begin;
    auto flush = [&]() {
      while (bits) {
        const int j = __ffsll(static_cast<long long>(bits)) - 1;
        bits &= bits - 1;
        const int i = bits_base + j;
        f(float_to_key(Elem<T>::to_float(rp[i])), i);
      }
    };
    walk([&](uint32_t key, int i) {
      if (i - bits_base == 64) {
        flush();
        bits_base = i;
      }
      bool kept = key > tau;
      if (key == tau) {
        kept = tie_off < tie_keep;
        ++tie_off;
      }
      bits |= static_cast<unsigned long long>(kept ? 1u : 0u) << (i - bits_base);
    });
    flush();
  };
  auto mass_of = [&](uint32_t key) {
    const float y = mul_rn(key_to_float(key), inv_temp);
    return static_cast<unsigned long long>(mass_fixed(exp_det(sub_rn(y, y_max))));
  };
  unsigned long long my_mass = 0;
  int last_kept = -1;
  walk_kept([&](uint32_t key, int i) {
    my_mass += mass_of(key);
    last_kept = i;
  });
  unsigned long long mass_total;
  const unsigned long long mass_first = block_exscan_u64(my_mass, s.scan, mass_total);
  if (mass_first <= target && mass_first + my_mass > target) {  // exactly one thread
    unsigned long long acc = mass_first;
    int found = -1;
    walk_kept([&](uint32_t key, int i) {
      const unsigned long long q = mass_of(key);
      acc += q;
      if (found < 0 && q != 0 && acc > target) found = i;
    });
    s.pick = found;
  }
  __syncthreads();
  // target == kept_mass can only happen when kept_mass is 0 (all masses underflowed):
  // fall back to the last kept element, or the row maximum position.
  if (s.pick < 0) {
    const int cand = last_kept;
    int best = cand;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    __syncthreads();
    if ((tid & 31) == 0) s.red[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
      int b = -1;
      for (int w = 0; w < kWarps; ++w) b = max(b, s.red[w]);
      s.pick = b < 0 ? 0 : b;
    }
    __syncthreads();
  }
  if (tid == 0) out[row] = s.pick;
}

template <typename T>
int launch_sampling(const void* logits, long long row_stride, int rows, int v, const long long* row_ids,
                    float inv_temp, int top_k, float top_p, unsigned long long seed, unsigned long long step,
                    int* out, cudaStream_t stream) {
  const T* lp = static_cast<const T*>(logits);
  cudaError_t e;
  if (top_k >= 1 && top_k <= kMaxTopK) {
    static bool configured = false;
    if (!configured) {
      e = cudaFuncSetAttribute(sample_topk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(sizeof(TopkSmem)));
      if (e != cudaSuccess) return -10;
      configured = true;
    }
    // few rows of 16-bit logits may be given several CTAs per row (a cluster)
    int cluster = 1;
    if constexpr (Elem<T>::kPacked) {
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      const bool aligned = (reinterpret_cast<uintptr_t>(lp) & 15u) == 0 && (row_stride * sizeof(T)) % 16 == 0 && v >= 8192;
      // Measured (bf16 [G, 128256], k = 50, L2 flushed): 28.7 / 28.7 / 30.6 us for 1 / 2 / 4 CTAs
      // per row at G = 64, 31.6 / 35.7 / 50.0 at G = 128. A row's two passes are a small part of
      // the kernel's latency chain (bound search, candidate sort, masses, draw), so more SMs per
      // row buy nothing here; the variant stays available but is not chosen by default.
      (void)sms;
      if (const char* e = getenv("KA_SAMPLE_CLUSTER")) {      // 2 / 4: CTAs per row (opt-in)
        const int c = atoi(e);
        if (c == 1 || ((c == 2 || c == 4) && aligned)) cluster = c;
      }
    }
    if (cluster > 1) {
      if constexpr (Elem<T>::kPacked) {
        const int smem = static_cast<int>(sizeof(TopkSmem) + sizeof(ClusterXchg));
        auto* k2 = sample_topk_cluster_kernel<T, 2>;
        auto* k4 = sample_topk_cluster_kernel<T, 4>;
        static bool cluster_configured = false;
        if (!cluster_configured) {
          if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
              cudaFuncSetAttribute(k4, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return -10;
          cluster_configured = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(rows * cluster));
        cfg.blockDim = dim3(kTopkThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, cluster == 2 ? k2 : k4, lp, row_stride, v, row_ids, inv_temp, top_k, top_p, seed,
                               step, out);
        return e == cudaSuccess ? 0 : -11;
      }
    }
    sample_topk_kernel<T><<<rows, kTopkThreads, sizeof(TopkSmem), stream>>>(lp, row_stride, v, row_ids, inv_temp, top_k,
                                                                         top_p, seed, step, out);
  } else {
    constexpr int smem = kGeneralSmemBytes + (std::is_same<T, __nv_bfloat16>::value ? kHistBytes : 0);
    static bool configured = false;
    if (!configured) {
      e = cudaFuncSetAttribute(sample_general_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return -10;
      configured = true;
    }
    sample_general_kernel<T><<<rows, kThreads, smem, stream>>>(lp, row_stride, v, row_ids, inv_temp, top_k, top_p,
                                                              seed, step, out);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -11;
}

}  // namespace
}  // namespace ka

extern "C" int ka_sample(const void* logits, int dtype, long long row_stride, int rows, int vocab,
                         const long long* row_ids, float inv_temperature, int top_k, float top_p,
                         unsigned long long seed, unsigned long long step, int* out, void* stream) {
  using namespace ka;
  if (rows <= 0) return 0;
  if (vocab <= 0 || !(inv_temperature > 0.f) || !(top_p > 0.f)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case KA_DTYPE_F32:
      return launch_sampling<float>(logits, row_stride, rows, vocab, row_ids, inv_temperature, top_k, top_p, seed,
                                    step, out, st);
    case KA_DTYPE_BF16:
      return launch_sampling<__nv_bfloat16>(logits, row_stride, rows, vocab, row_ids, inv_temperature, top_k, top_p,
                                            seed, step, out, st);
    case KA_DTYPE_F16:
      return launch_sampling<__half>(logits, row_stride, rows, vocab, row_ids, inv_temperature, top_k, top_p, seed,
                                     step, out, st);
    default:
      return -2;
  }
}
