// Batch-invariant bf16 GEMM on tcgen05 (C entry points and parameter block).
//
//   C[M, N] = op(A) * op(B)^T   with fp32 accumulation in TMEM
//
// Operand layouts (row-major storage):
//   a_major = 0: A is [M, K] (K contiguous)        a_major = 1: A is [K, M] (M contiguous)
//   b_major = 0: B is [N, K] (K contiguous)        b_major = 1: B is [K, N] (N contiguous)
// so that y = x W^T, dx = dy W and dW = dy^T x all run without a transpose pass.
//
// Invariance: one CTA pair owns a 256 x 256 output tile and walks K in a fixed order that
// does not depend on M, N or the grid; there is no split-K chosen from the problem size.
// With k_slices > 1 the K range is cut into that many equal slices whose fp32 partial sums
// are emitted separately, each rounded to bf16 once (the tensor-parallel path adds them in fp32
// in a fixed tree order and rounds the sum once more).
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace ka {

enum GemmEpilogue : int {
  kEpiStoreBf16 = 0,    // C bf16 [M, N]
  kEpiStoreF32 = 1,     // C fp32 [M, N]
  kEpiPartialF32 = 2,   // K-slice partial (fp32 accumulated, stored as bf16), pushed to the row owner's staging buffer
  kEpiLogitsGrad = 3    // C bf16 = g[row] * scale * (onehot(ids[row]) - exp(scale * acc - lse[row]))
};

struct GemmParams {
  int m, n, k;            // k: this rank's K extent
  int a_major, b_major;
  int epilogue;
  void* c;                // kEpiStoreBf16 / kEpiStoreF32 output
  long long ldc;
  // --- K-slice partials + reduce-scatter (kEpiPartialF32)
  int k_slices;           // local slices (each k / k_slices wide, multiple of 64)
  int slice_base;         // global index of the first local slice (rank * k_slices)
  int total_slices;       // canonical slice count (8)
  int world, rank;
  int rows_per_rank;      // rows of the output each rank owns (multiple of 128)
  void* stage[8];         // per owner rank: [total_slices][row blocks][column tiles][128 x 256] bf16, fragment-major
  unsigned* flags[8];     // per owner rank: [total_slices][row blocks of 128][n tiles of 256]
  unsigned epoch;
  void* out;              // reduced bf16 [rows_per_rank, n] of this rank
  const void* residual;   // optional bf16 [rows_per_rank, n] added after the reduction
  // --- all-gather of A (a_gather != 0): A is read from `a` = this rank's gather buffer
  //     [world * rows_per_rank_a, k]; rows of rank r become valid when a_flags[r * blocks + b] == epoch
  int a_gather;
  int a_rows_per_rank;
  const void* a_local;    // this rank's rows [a_rows_per_rank, k] to push to every peer
  void* a_bufs[8];        // per destination rank: its gather buffer
  unsigned* a_flags[8];   // per destination rank: [world][row blocks of 128]
  // --- kEpiLogitsGrad: gradient of the log-prob w.r.t. the logits, from recomputed logits
  const float* row_lse;       // [m] log-sum-exp of the scaled logits (natural log)
  const float* row_g;         // [m] upstream gradient of logp
  const long long* row_ids;   // [m] global target ids
  float scale;
  int col_offset;             // global index of column 0 (vocabulary shard offset)
  int* status;
  unsigned long long timeout_ns;
};

// Build the tensor maps for the operand layouts in `p` and launch on `stream`. `full_grid`
// keeps one CTA per SM even for small problems (the tensor-parallel paths use every CTA for
// their copy and reduce phases).
int gemm_launch(const void* a, long long lda, const void* b, long long ldb, const GemmParams& p, int num_sms,
                bool full_grid, cudaStream_t stream);

}  // namespace ka

extern "C" {

// Plain GEMM: c = op(a) op(b)^T. out_f32 selects fp32 output. All leading dimensions in
// elements; m, n, k multiples of 8. Returns 0 or a negative code.
// d_logits[m, n] (bf16) for logp = scale * logits[ids] - logsumexp(scale * logits), with the
// logits recomputed as hidden[m, k] x weight[n, k]^T inside the kernel.
int ka_lmhead_logits_grad(const void* hidden, const void* weight, const long long* ids, const float* lse,
                          const float* g, void* d_logits, long long ldd, int m, int n, int k, float scale,
                          int col_offset, int* status, int num_sms, unsigned long long timeout_ns, void* stream);

int ka_gemm_bf16(const void* a, long long lda, int a_major, const void* b, long long ldb, int b_major, void* c,
                 long long ldc, int out_f32, int m, int n, int k, int* status, int num_sms,
                 unsigned long long timeout_ns, void* stream);
}
