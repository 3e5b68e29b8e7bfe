// Tensor-parallel linear layers with the collective fused into the GEMM kernel
// (csrc/sm100/gemm.cu does the work; this file owns the entry points and buffer layouts).
//
//   ka_gemm_reduce_scatter   row-parallel linear (K sharded): every rank multiplies its K
//       slices; the epilogue stores each slice partial (rounded to bf16 once) into the staging buffer of
//       the rank that owns those rows (peer stores over NVLink) and raises a per-tile flag; the
//       same kernel then adds, in fp32, for the rows it owns, the 8 canonical slices in the fixed
//       order ((0+1)+(2+3))+((4+5)+(6+7)), adds the residual and writes bf16. Because K is
//       always cut into the same 8 slices, 1, 2, 4 and 8 ranks perform the same additions.
//   ka_all_gather_gemm       column-parallel linear on row-sharded input: every rank copies
//       its rows into all peers' gather buffers block by block (peer stores + flags) while the
//       GEMM already runs on the rows it has; tiles of remote rows wait for their flag.
//
// Both keep two generations of their exchange buffers, selected by the parity of `epoch`, so a
// rank that is one call ahead never overwrites data a slower rank is still reading.
#include <cstdint>
#include <cuda_bf16.h>

#include "gemm.h"

namespace {
constexpr int kBlk = 128;
constexpr int kTileN = 256;
constexpr int kSlices = 8;

inline size_t round256(size_t v) { return (v + 255) / 256 * 256; }
inline int rows_per_rank_of(int m, int world) {
  const int per = (m + world - 1) / world;
  return (per + kBlk - 1) / kBlk * kBlk;
}
}  // namespace

extern "C" {

// Bytes of the symmetric buffer a rank maps for ka_gemm_reduce_scatter: two generations of
// [8 slices][row blocks][column tiles][128 x 256] bf16 staging (whole tiles, each stored as 16
// contiguous warp fragments, see stage_offset in gemm.cu), then the flags of both generations.
size_t ka_gemm_rs_exchange_bytes(int m, int n, int world) {
  const size_t rpr = rows_per_rank_of(m, world);
  const size_t stage = round256(static_cast<size_t>(kSlices) * (rpr / kBlk) * ((n + kTileN - 1) / kTileN) * kBlk * kTileN *
                                sizeof(__nv_bfloat16));
  const size_t flags = round256(static_cast<size_t>(kSlices) * (rpr / kBlk) * ((n + kTileN - 1) / kTileN) * 4);
  return 2 * stage + 2 * flags;
}

int ka_gemm_rs_rows_per_rank(int m, int world) { return rows_per_rank_of(m, world); }

// a: [m, k_local] bf16 (this rank's K shard = 8/world canonical slices), b: [n, k_local] bf16
// (b_major = 0) or [k_local, n] (b_major = 1),
// out: [rows_per_rank, n] bf16 (this rank's rows of the reduced result), residual: same shape
// or null. exchange[r]: rank r's symmetric buffer as mapped here. Must be zero-initialised
// once; `epoch` must grow by one per call on a given buffer.
int ka_gemm_reduce_scatter(const void* a, long long lda, const void* b, long long ldb, int b_major, void* out,
                           const void* residual, void* const* exchange, int m, int n, int k_local, int world, int rank,
                           unsigned epoch,
                           int* status, int num_sms, unsigned long long timeout_ns, void* stream) {
  if (!(world == 1 || world == 2 || world == 4 || world == 8) || rank < 0 || rank >= world) return -50;
  if (n % 8 != 0) return -51;
  ka::GemmParams p = {};
  p.m = m;
  p.n = n;
  p.k = k_local;
  p.a_major = 0;
  p.b_major = b_major ? 1 : 0;
  p.epilogue = ka::kEpiPartialF32;
  p.k_slices = kSlices / world;
  p.slice_base = rank * p.k_slices;
  p.total_slices = kSlices;
  p.world = world;
  p.rank = rank;
  p.rows_per_rank = rows_per_rank_of(m, world);
  const size_t rpr = p.rows_per_rank;
  const size_t stage = round256(static_cast<size_t>(kSlices) * (rpr / kBlk) * ((n + kTileN - 1) / kTileN) * kBlk * kTileN *
                                sizeof(__nv_bfloat16));
  const size_t flags = round256(static_cast<size_t>(kSlices) * (rpr / kBlk) * ((n + kTileN - 1) / kTileN) * 4);
  const unsigned gen = epoch & 1u;
  for (int r = 0; r < world; ++r) {
    uint8_t* base = static_cast<uint8_t*>(exchange[r]);
    if (!base) return -52;
    p.stage[r] = base + gen * stage;
    p.flags[r] = reinterpret_cast<unsigned*>(base + 2 * stage + gen * flags);
  }
  p.epoch = epoch;
  p.out = out;
  p.residual = residual;
  p.status = status;
  p.timeout_ns = timeout_ns;
  return ka::gemm_launch(a, lda, b, ldb, p, num_sms, true, static_cast<cudaStream_t>(stream));
}

// Bytes of the symmetric buffer for ka_all_gather_gemm: two generations of the gathered
// activations [world * rows_per_rank, k] bf16, then the flags of both generations.
size_t ka_ag_gemm_exchange_bytes(int rows_per_rank, int k, int world) {
  const size_t buf = round256(static_cast<size_t>(world) * rows_per_rank * k * 2);
  const size_t flags = round256(static_cast<size_t>(world) * (rows_per_rank / kBlk) * 4);
  return 2 * buf + 2 * flags;
}

// a_local: [rows_per_rank, k] bf16 (rows_per_rank multiple of 128), b: [n_local, k] bf16
// (b_major = 0) or [k, n_local] (b_major = 1),
// c: [world * rows_per_rank, n_local] bf16 = all_gather(a_local) @ b^T.
int ka_all_gather_gemm(const void* a_local, const void* b, long long ldb, int b_major, void* c, long long ldc,
                       void* const* exchange, int rows_per_rank, int n_local, int k, int world, int rank,
                       unsigned epoch, int* status, int num_sms, unsigned long long timeout_ns, void* stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return -50;
  if (rows_per_rank % kBlk != 0 || k % 8 != 0) return -53;
  ka::GemmParams p = {};
  p.m = world * rows_per_rank;
  p.n = n_local;
  p.k = k;
  p.a_major = 0;
  p.b_major = b_major ? 1 : 0;
  p.epilogue = ka::kEpiStoreBf16;
  p.c = c;
  p.ldc = ldc;
  p.k_slices = 1;
  p.total_slices = 1;
  p.world = world;
  p.rank = rank;
  p.a_gather = 1;
  p.a_rows_per_rank = rows_per_rank;
  p.a_local = a_local;
  const size_t buf = round256(static_cast<size_t>(world) * rows_per_rank * k * 2);
  const size_t flags = round256(static_cast<size_t>(world) * (rows_per_rank / kBlk) * 4);
  const unsigned gen = epoch & 1u;
  for (int r = 0; r < world; ++r) {
    uint8_t* base = static_cast<uint8_t*>(exchange[r]);
    if (!base) return -52;
    p.a_bufs[r] = base + gen * buf;
    p.a_flags[r] = reinterpret_cast<unsigned*>(base + 2 * buf + gen * flags);
  }
  p.epoch = epoch;
  p.status = status;
  p.timeout_ns = timeout_ns;
  return ka::gemm_launch(p.a_bufs[rank], k, b, ldb, p, num_sms, true, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
