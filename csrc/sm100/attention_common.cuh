// Helpers shared by the attention forward and backward kernels: operand descriptors for
// 128 x 128 bf16 tiles stored as two 64-column TMA boxes, TMEM load dependency pinning,
// proxy fence, bf16 packing and the swizzled store of a bf16 row into a K-major tile.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>

#include "common/ptx.cuh"

namespace ka {
namespace {

// K-major tile: 128 rows x 128 columns as two 64-column boxes (16 KiB each), 128 B rows.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int kstep) {
  return umma_desc_k_sw128(tile + (kstep >> 2) * 16384 + (kstep & 3) * 32);
}
// MN-major tile (V): boxes of 64 d-columns x 128 kv rows; a K step of 16 rows is 2048 B.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int kstep) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>(((tile + kstep * 2048) & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(16384 >> 4) << 16;  // next 64 d-columns: one box further
  d |= static_cast<uint64_t>(1024 >> 4) << 32;   // next 8 kv rows
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ void tmem_ld_wait_dep(uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),
        "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]),
        "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]),
        "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]),
        "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
      :
      : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// max of three (one instruction on sm_100a)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two fp32 lanes per instruction: (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1), each lane rounded
// exactly like a scalar fma.rn; and the lane-wise sum.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// Write 32 consecutive bf16 values (already packed two per word, 16 words) of row `row`,
// columns [col, col + 32), into a K-major 128 x 128 tile laid out as two 64-column boxes with
// the 128-byte swizzle (the layout tcgen05.mma expects for an A operand written by hand).
__device__ __forceinline__ void store_tile_row32(uint8_t* tile, int row, int col, const uint32_t (&w)[16]) {
  uint8_t* rowp = tile + (col >> 6) * 16384 + row * 128;
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    const int phys = (((col >> 5) & 1) * 4 + ch) ^ (row & 7);
    *reinterpret_cast<uint4*>(rowp + phys * 16) = make_uint4(w[ch * 4], w[ch * 4 + 1], w[ch * 4 + 2], w[ch * 4 + 3]);
  }
}

}  // namespace
}  // namespace ka
