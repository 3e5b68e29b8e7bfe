// Deterministic all-reduce (sum) over NVLink peer memory, in place on symmetric buffers.
//
// Two phases in one kernel. Rank r owns the r-th slice of the vector: it loads that slice from
// every rank's buffer with plain peer loads, adds the contributions in the fixed order
// ((0+1)+(2+3))+((4+5)+(6+7)) in fp32, and stores the result into every rank's buffer with peer
// stores. No atomics and no switch-side reduction, so the result is bitwise reproducible run
// to run. CTA c of every rank handshakes only with CTA c of the other ranks (start: "my input is
// final"; done: "my writes have landed"), so no CTA ever waits on another CTA of its own grid.
// Every wait is bounded and reports into the status block.
//
// The reference has no collective of any kind; this is the gradient all-reduce of the training
// step (README "deterministic collectives" bullet).
#include <cstdint>
#include <cuda_bf16.h>

#include "common/bounded_wait.cuh"
#include "common/ptx.cuh"

namespace ka {
namespace {

constexpr int kThreads = 512;

struct ArParams {
  void* buf[8];          // per rank: the vector (symmetric memory)
  unsigned* flags[8];    // per rank: [2][world][grid] start / done epochs
  long long n;           // elements, multiple of world * vector width
  int world, rank;
  int is_bf16;
  unsigned epoch;
  unsigned* epoch_dev;   // or null: [0] epoch of the last call on this vector, [1] CTAs that are done
  int* status;
  unsigned long long timeout_ns;
};

// Bulk data uses weak L2 loads / plain stores (they pipeline); ordering against the other ranks
// comes from the acquire / release on the handshake flags.
__device__ __forceinline__ float4 ld4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
__device__ __forceinline__ float4 tree8(const float4 (&s)[8], int world) {
  if (world == 1) return s[0];
  if (world == 2) return add4(s[0], s[1]);
  if (world == 4) return add4(add4(s[0], s[1]), add4(s[2], s[3]));
  return add4(add4(add4(s[0], s[1]), add4(s[2], s[3])), add4(add4(s[4], s[5]), add4(s[6], s[7])));
}

// Device-side epoch: the last CTA of the grid to get here stores the epoch this call used.
__device__ __forceinline__ void finish_epoch(const ArParams& p, unsigned epoch) {
  if (p.epoch_dev == nullptr) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(p.epoch_dev + 1, 1u);
    if (prev + 1u == gridDim.x) {
      p.epoch_dev[1] = 0u;
      __threadfence();
      p.epoch_dev[0] = epoch;
    }
  }
}

__global__ void __launch_bounds__(kThreads)
allreduce_det_kernel(const __grid_constant__ ArParams p) {
  __shared__ int abort_flag;
  const int tid = threadIdx.x;
  if (tid == 0) abort_flag = 0;
  __syncthreads();
  WaitCtx wctx{&abort_flag, p.status, p.timeout_ns};
  const int grid = gridDim.x, cta = blockIdx.x;
  // The epoch is a launch argument, or (so that a captured graph can replay the launch) one more
  // than the word the previous call left in device memory. Every CTA reads that word before it
  // counts itself done, and only the last CTA to be done advances it.
  const unsigned epoch = p.epoch_dev ? __ldcg(p.epoch_dev) + 1u : p.epoch;

  // ---- start handshake: every rank's kernel has begun, so every input is final
  if (tid < p.world) {
    st_release_sys_u32(p.flags[tid] + (0 * p.world + p.rank) * grid + cta, epoch);
    flag_wait_bounded(p.flags[p.rank] + (0 * p.world + tid) * grid + cta, epoch, wctx, 21, tid);
  }
  __syncthreads();
  if (abort_flag) {
    finish_epoch(p, epoch);
    return;
  }

  const long long slice = p.n / p.world;
  const long long begin = slice * p.rank;
  if (!p.is_bf16) {
    const long long nvec = slice / 4;
    for (long long i = static_cast<long long>(cta) * kThreads + tid; i < nvec; i += static_cast<long long>(grid) * kThreads) {
      const long long off = begin + i * 4;
      float4 s[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.world) s[r] = ld4(static_cast<const float*>(p.buf[r]) + off);
      const float4 t = tree8(s, p.world);
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.world) *reinterpret_cast<float4*>(static_cast<float*>(p.buf[r]) + off) = t;
    }
  } else {
    const long long nvec = slice / 4;  // 4 bf16 = 8 bytes per step
    for (long long i = static_cast<long long>(cta) * kThreads + tid; i < nvec; i += static_cast<long long>(grid) * kThreads) {
      const long long off = begin + i * 4;
      float4 s[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.world) {
          const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.buf[r]) + off));
          const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          s[r] = make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
        }
      const float4 t = tree8(s, p.world);
      const __nv_bfloat162 o0 = __floats2bfloat162_rn(t.x, t.y), o1 = __floats2bfloat162_rn(t.z, t.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&o0);
      o.y = *reinterpret_cast<const uint32_t*>(&o1);
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.world) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.buf[r]) + off) = o;
    }
  }

  // ---- done handshake: my stores have landed everywhere; leave when everyone's have
  __threadfence_system();
  __syncthreads();
  if (tid < p.world) {
    st_release_sys_u32(p.flags[tid] + (1 * p.world + p.rank) * grid + cta, epoch);
    flag_wait_bounded(p.flags[p.rank] + (1 * p.world + tid) * grid + cta, epoch, wctx, 22, tid);
  }
  finish_epoch(p, epoch);
}

}  // namespace
}  // namespace ka

extern "C" {

int ka_allreduce_grid(int num_sms) { return num_sms < 64 ? num_sms : 64; }

// Bytes of flags each rank keeps next to its vector (zero-initialised once).
size_t ka_allreduce_flag_bytes(int world, int num_sms) {
  return static_cast<size_t>(2) * world * ka_allreduce_grid(num_sms) * sizeof(unsigned);
}

// bufs[r] / flags[r]: rank r's vector and flag block as mapped in this process. n elements,
// a multiple of world * 4. epoch must grow by one per call on these buffers.
int ka_allreduce_det_ex(void* const* bufs, void* const* flags, long long n, int is_bf16, int world, int rank,
                        unsigned epoch, unsigned* epoch_dev, int* status, int num_sms, unsigned long long timeout_ns,
                        void* stream);

int ka_allreduce_det(void* const* bufs, void* const* flags, long long n, int is_bf16, int world, int rank,
                     unsigned epoch, int* status, int num_sms, unsigned long long timeout_ns, void* stream) {
  return ka_allreduce_det_ex(bufs, flags, n, is_bf16, world, rank, epoch, nullptr, status, num_sms, timeout_ns, stream);
}

// The same with an optional device-side epoch: `epoch_dev` points to two zero-initialised words
// of this rank's memory that belong to the vector; the kernel then uses *epoch_dev + 1 and stores
// it back when it is done, so the launch can be captured in a CUDA graph and replayed. `epoch`
// is ignored in that case. All ranks must use the same mode for a vector.
int ka_allreduce_det_ex(void* const* bufs, void* const* flags, long long n, int is_bf16, int world, int rank,
                        unsigned epoch, unsigned* epoch_dev, int* status, int num_sms, unsigned long long timeout_ns,
                        void* stream) {
  using namespace ka;
  if (!(world == 1 || world == 2 || world == 4 || world == 8) || rank < 0 || rank >= world) return -50;
  if (n % (static_cast<long long>(world) * 4) != 0) return -51;
  if (world == 1 || n == 0) return 0;
  ArParams p = {};
  for (int r = 0; r < world; ++r) {
    p.buf[r] = bufs[r];
    p.flags[r] = static_cast<unsigned*>(flags[r]);
  }
  p.n = n;
  p.world = world;
  p.rank = rank;
  p.is_bf16 = is_bf16;
  p.epoch = epoch;
  p.epoch_dev = epoch_dev;
  p.status = status;
  p.timeout_ns = timeout_ns;
  // a short vector does not need the whole grid: fewer CTAs, fewer handshakes (the flag index
  // depends on the grid size, which every rank derives from the same n)
  int grid = ka_allreduce_grid(num_sms);
  const long long vec_per_rank = n / world / 4;
  const long long want = (vec_per_rank + kThreads - 1) / kThreads;
  if (want < grid) grid = want < 1 ? 1 : static_cast<int>(want);
  allreduce_det_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
