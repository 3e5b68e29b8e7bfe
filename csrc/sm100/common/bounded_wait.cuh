// Bounded waits and the status word they report into.
//
// Every spin in this tree (on an mbarrier, on a flag another CTA or another GPU writes)
// goes through one of these helpers. A wait that exceeds its time limit records where it
// gave up, raises the CTA-wide abort flag and returns false; callers unwind to the common
// exit path, so a missing signal ends the kernel with an error code instead of a hang.
#pragma once

#include "ptx.cuh"

namespace ka {

// Layout of the int32 status buffer every kernel with waits writes into.
enum StatusSlot : int {
  kStatusCode = 0,   // 0 = ok, otherwise a StatusCode
  kStatusWhere = 1,  // kernel-specific site id of the wait that gave up
  kStatusBlock = 2,  // blockIdx.x of the reporter
  kStatusAux0 = 3,   // site-specific (barrier index, block id, ...)
  kStatusAux1 = 4,   // site-specific (expected value)
  kStatusAux2 = 5,   // site-specific (value seen)
  kStatusWords = 8
};

enum StatusCode : int {
  kOk = 0,
  kTimeoutMbarrier = 1,
  kTimeoutFlag = 2,
  kBadArgument = 3
};

struct WaitCtx {
  volatile int* abort_flag;  // shared memory, one per CTA
  int* status;               // global, kStatusWords ints
  unsigned long long timeout_ns;
};

__device__ __forceinline__ void report_failure(const WaitCtx& ctx, int code, int where, int aux0,
                                               int aux1, int aux2) {
  *ctx.abort_flag = 1;
  if (atomicCAS(&ctx.status[kStatusCode], 0, code) == 0) {
    ctx.status[kStatusWhere] = where;
    ctx.status[kStatusBlock] = static_cast<int>(blockIdx.x);
    ctx.status[kStatusAux0] = aux0;
    ctx.status[kStatusAux1] = aux1;
    ctx.status[kStatusAux2] = aux2;
  }
}

// Wait for the phase with the given parity of an mbarrier in this CTA's shared memory.
// `sleep_ns` > 0 makes the waiter sleep between polls: for warps that wait most of the time
// (an epilogue that needs a tenth of a tile's duration) a polling loop costs issue slots and
// power for nothing, and a few hundred nanoseconds of extra latency are hidden by the
// double-buffered accumulator.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                                  int where, int aux0, unsigned sleep_ns = 0u) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((++spins & 31u) == 0u) {
      if (*ctx.abort_flag) return false;
      if (globaltimer_ns() - t0 > ctx.timeout_ns) {
        report_failure(ctx, kTimeoutMbarrier, where, aux0, static_cast<int>(parity), 0);
        return false;
      }
    }
  }
}

// Wait until a 32-bit epoch flag in global memory (possibly written by another GPU) has
// reached `expected`, reading it with acquire semantics at system scope. Epochs only grow, and
// a writer may already be one call ahead, so "reached" means seen - expected >= 0 in wrapping
// arithmetic.
__device__ __forceinline__ bool flag_wait_bounded(const uint32_t* flag, uint32_t expected,
                                                  const WaitCtx& ctx, int where, int aux0) {
  uint32_t seen = ld_acquire_sys_u32(flag);
  if (static_cast<int32_t>(seen - expected) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    seen = ld_acquire_sys_u32(flag);
    if (static_cast<int32_t>(seen - expected) >= 0) return true;
    if ((++spins & 15u) == 0u) {
      if (*ctx.abort_flag) return false;
      if (globaltimer_ns() - t0 > ctx.timeout_ns) {
        report_failure(ctx, kTimeoutFlag, where, aux0, static_cast<int>(expected),
                       static_cast<int>(seen));
        return false;
      }
      __nanosleep(200);
    }
  }
}

// Give asynchronous copies and MMAs that this CTA still has in flight time to land before
// the CTA releases its shared memory and TMEM on the error path. Bounded by construction.
__device__ __forceinline__ void drain_in_flight() {
  const uint64_t t0 = globaltimer_ns();
  while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
}

}  // namespace ka
