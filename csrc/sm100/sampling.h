// Fused sampling: C entry point.
#pragma once

#include <cstdint>

enum KaDtype : int { KA_DTYPE_F32 = 0, KA_DTYPE_BF16 = 1, KA_DTYPE_F16 = 2 };

extern "C" {
// Sample one token per row of `logits` ([rows, vocab], row stride in elements).
//   row_ids          optional [rows] int64: the identity of each row for the random stream
//                    (default: the row index). A row sampled under the same
//                    (seed, row id, step) gives the same token in any batch.
//   inv_temperature  1 / temperature, > 0
//   top_k            <= 0: no top-k filter; 1: greedy
//   top_p            in (0, 1]; 1 disables the filter
//   out              [rows] int32 token ids
// Returns 0, or a negative code for bad arguments / launch failure.
int ka_sample(const void* logits, int dtype, long long row_stride, int rows, int vocab, const long long* row_ids,
              float inv_temperature, int top_k, float top_p, unsigned long long seed, unsigned long long step,
              int* out, void* stream);
}
