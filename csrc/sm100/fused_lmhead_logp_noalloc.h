// Allocation-free variant of the fused LM-head + log-probability forward pass.
//
// This entry point has no counterpart in the reference (Flink-ddd/Kernel-Align): it exists
// for hosts that drive this library but are not in a position to create device memory.
// Typical cases: a rollout worker whose serving engine reserved the whole HBM for its own
// pool at start-up, so a later cudaMalloc simply fails; a control loop that must not hit the
// device-wide synchronisation cudaMalloc/cudaFree imply; a C or Rust host that has no
// allocator of its own to hand a workspace from. Such a caller still owns its inputs and
// outputs, but cannot provide the kernel's scratch (the per-sub-slice partial maxima and
// sums, the arrival counters and the status block).
//
// The scratch therefore lives inside the library image, in one fixed device array of
// KA_NOALLOC_SCRATCH_BYTES that every GPU loading the library holds until the process exits.
// Consequences the caller has to know:
//   * Limits: vocab <= KA_NOALLOC_MAX_VOCAB; any number of rows (they are processed in
//     panels of KA_NOALLOC_PANEL_ROWS). Larger vocabularies are rejected with -30 and a
//     message on stderr; nothing is launched.
//   * The first call on a device resolves the array's device address (cudaGetSymbolAddress)
//     and configures the kernel. Make that first call during start-up, before any stream
//     capture begins on that device.
//   * The array is shared by every call and keeps whatever the previous call left. The
//     entry point clears the counters and the status block on `stream` before launching;
//     the rest is overwritten before it is read. Two calls whose kernels overlap on the GPU
//     (different streams, or different host threads) race on the array: serialise them.
//   * Single GPU only (no vocabulary sharding): the exchange buffers of the multi-GPU path
//     must be peer-mapped, which a static array cannot be.
// No cudaMalloc, cudaFree, or allocating library routine is called on any path.
#pragma once

#include <cstddef>

#define KA_NOALLOC_MAX_VOCAB 262144
#define KA_NOALLOC_PANEL_ROWS 8192
#define KA_NOALLOC_SCRATCH_BYTES 9994752

extern "C" {

// hidden [m, k] bf16 row-major, weight [vocab, k] bf16 row-major, ids [m] int64,
// logp [m] fp32 (output), lse [m] fp32 (output, may be null). scale > 0, k % 8 == 0.
// `timeout_ns` bounds every wait inside the kernel (on a TMA transfer, an accumulator, a
// barrier); a wait that runs out is reported through the status block and the kernel returns.
// Pass about 2e9; with 0 every wait that is not satisfied at once gives up.
// Returns 0 on success; -30 if vocab exceeds KA_NOALLOC_MAX_VOCAB; -31 if the scratch address
// could not be resolved; -32 if clearing the counters and the status block could not be
// enqueued on `stream`; other negative codes as ka_lmhead_logp_forward.
int ka_lmhead_logp_forward_noalloc(const void* hidden, const void* weight, const long long* ids, float* logp,
                                   float* lse, int m, int k, int vocab, float scale, int cta_group, int num_sms,
                                   unsigned long long timeout_ns, void* stream);

// Copies the 8-word status block that calls with this `vocab` write on the current device to
// `host_out` (a blocking copy). All zeros when no bounded wait gave up.
int ka_lmhead_logp_noalloc_status(int vocab, int* host_out);
}
