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
  int mt_rot;            // rotation of the row-tile order (row-sharded input: own rows first)
  int l2_hint;           // L2 eviction hints of the operand loads, see the producer
  int m_fast;            // work order inside a wave: 1 = consecutive CTAs take consecutive row tiles
  int c_outer;           // 1 = groups of sub-slices are the outer loop (W stays in L2, H streams)
  int epi_sleep_ns;      // the epilogue warps sleep this long between polls of the accumulator barrier

  // ---- row-sharded input (gather != 0): rank r holds rows [r * m_local, (r + 1) * m_local) of
  // the hidden states and the ids; the kernel pushes its rows of the panel into every peer's
  // gather buffer and reads the other ranks' rows from its own buffer once their flags are up.
  int gather;
  int out_all;           // 1: every rank writes all world * m_local results; 0: only its own m_local
  int m_local;           // rows per rank (the same on every rank)
  int pl;                // rows per rank and panel = panel_rows / world (multiple of 256)
  int local_row_begin;   // first local row of this panel
  int rows_local;        // local rows in this panel (the same on every rank)
  int bps;               // 128-row blocks per source rank in this panel (even)
  const void* h_local;   // [m_local, k] bf16
  uint8_t* gbuf[8];      // per destination rank: [2][world][pl][k] bf16 gathered rows
  long long* gids[8];    // per destination rank: [2][world][pl] gathered ids
  unsigned* gflag[8];    // per destination rank: [world][pl / 128] epoch of the last pushed block
  unsigned* pcount;      // [pl / 128] local: 32-row pieces of a block pushed so far (self-cleaning)
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

// The same with an explicit schedule: `cg_pref` sub-slices of the vocabulary run side by side
// (0: the default, 8), the CTAs that are left over them work on different row tiles; `m_fast`
// bit 0 says whether consecutive CTAs take consecutive row tiles of one sub-slice (1) or the
// sub-slices of one row tile (0), bit 1 whether the groups of sub-slices are the outer loop of
// the work order (W stays in L2 and H streams) instead of the groups of row tiles; `l2_hint` gives the operand loads an L2 eviction priority
// (0 none, 1 keep the hidden rows and let the weight tiles go first, 2 keep the hidden rows,
// 3 keep the weight tiles). The schedule changes which tiles share the L2 at a time, hence
// memory traffic and power, never a result: every combination gives the same bits.
int ka_lmhead_logp_forward_sched(const void* hidden, const void* weight, const long long* ids, float* logp,
                                 float* lse, void* workspace, size_t workspace_bytes, void* const* peer_exchange,
                                 int m, int k, int v_global, int v_local, int vocab_offset, int world, int rank,
                                 unsigned epoch_base, float scale, int panel_rows, int cta_group, int cg_pref,
                                 int m_fast, int l2_hint, int num_sms, unsigned long long timeout_ns, void* stream);

// Bytes of the symmetric gather arena each rank maps for its peers when the rows are sharded
// over the ranks: two generations of panel_rows x k bf16 rows and of panel_rows ids, the block
// flags and the push counters. Must be zero-initialised once.
size_t ka_lmhead_logp_gather_bytes(int world, int panel_rows, int k);

// Row-sharded variant: rank r passes only its rows `hidden_local` [m_local, k] and `ids_local`
// [m_local] of a batch of world * m_local rows (global row = r * m_local + local row). Inside
// the kernel every rank pushes its rows of a panel to the peers' gather arenas with bulk copies
// over NVLink and raises a flag per (source rank, 128-row block); the TMA producer waits
// (bounded) for a block's flag and then loads the block from this GPU's own arena, own rows
// first. `out_all` = 0: logp / lse are [m_local], this rank's rows. `out_all` = 1: they are
// [world * m_local] and every rank writes every row. `peer_gather[d]` is rank d's gather arena
// as mapped into this process. panel_rows must be a multiple of 256 * world. Consumes
// ceil(m_local / (panel_rows / world)) epochs of the exchange and gather arenas.
int ka_lmhead_logp_forward_sharded(const void* hidden_local, const void* weight, const long long* ids_local,
                                   float* logp, float* lse, void* workspace, size_t workspace_bytes,
                                   void* const* peer_exchange, void* const* peer_gather, int m_local, int k,
                                   int v_global, int v_local, int vocab_offset, int world, int rank,
                                   unsigned epoch_base, float scale, int panel_rows, int out_all, int cta_group,
                                   int cg_pref, int m_fast, int l2_hint, int num_sms, unsigned long long timeout_ns,
                                   void* stream);
}
