// Fused LM-head + per-token log-probability: C entry points and the kernel parameter block.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace ka {

struct LogpParams {
  const long long* ids;  // [M] global token ids; ids outside [0, V) give logp = 0
  float* logp;           // [M]
  float* lse;            // [M] or nullptr: log-sum-exp of the scaled logits
  float* part_m;         // [n_chunks][ldp] running max of each canonical sub-slice
  float* part_l;         // [n_chunks][ldp] sum-exp relative to part_m
  float* tgt;            // [ldp] raw target logit, written by the sub-slice that holds it
  unsigned* counters;    // [n_blocks_max] arrivals per 128-row block (self-cleaning)
  int* status;           // [kStatusWords] error report, see common/bounded_wait.cuh
  float4* xbuf[8];       // per destination rank: [2][world][ldp] (m, l, t, has_t)
  unsigned* xflag[8];    // per destination rank: [world][n_blocks_max] epoch of last push
  int m, k;
  int v_global, v_local, vocab_offset;
  int row_begin, rows;   // panel processed by this launch
  int vs;                // canonical slice width = ceil(V / 8)
  int sub;               // sub-slices per slice = ceil(vs / 1792)
  int n_slices_local;    // 8 / world
  int n_chunks;          // n_slices_local * sub
  int ldp;               // panel leading dimension (rows, multiple of 256)
  int n_blocks_max;      // ldp / 128
  int n_mtiles;          // row tiles of 128 * cta_group rows in this panel
  int mg, cg;            // schedule: row tiles x sub-slices that run concurrently
  int world, rank;
  unsigned epoch;        // value the flags of this launch carry
  float scale;           // logits are scale * <h, w>; must be > 0
  unsigned long long timeout_ns;
};

}  // namespace ka

extern "C" {

// Bytes of per-rank scratch (partials, counters, status). Must be zero-initialised once.
size_t ka_lmhead_logp_workspace_bytes(int v_global, int panel_rows);
// Byte offset of the int32[8] status block inside the workspace.
int ka_lmhead_logp_status_offset(int v_global, int panel_rows);
// Bytes of the symmetric exchange buffer each rank maps for its peers (world > 1).
// Must be zero-initialised once; flags carry monotonically increasing epochs afterwards.
size_t ka_lmhead_logp_exchange_bytes(int world, int panel_rows);

// Enqueue the forward pass on `stream`. Rows are processed in panels of `panel_rows`
// (multiple of 256), each panel one kernel launch reusing the same scratch, so scratch size
// does not grow with M. `epoch_base` must be larger than every epoch used before on this
// exchange buffer; the call consumes ceil(m / panel_rows) consecutive epochs.
// `peer_exchange[d]` is rank d's exchange buffer as mapped into this process (world > 1).
// Returns 0 or a negative argument/launch error; device-side timeouts are reported through
// the status block.
int ka_lmhead_logp_forward(const void* hidden, const void* weight, const long long* ids, float* logp,
                           float* lse, void* workspace, size_t workspace_bytes, void* const* peer_exchange,
                           int m, int k, int v_global, int v_local, int vocab_offset, int world, int rank,
                           unsigned epoch_base, float scale, int panel_rows, int cta_group, int num_sms,
                           unsigned long long timeout_ns, void* stream);
}
