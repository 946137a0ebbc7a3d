// The warp-level tensor-core path (mma.sync m16n8k16, bfloat16 in, float accumulate) and what feeds it: 16-byte
// asynchronous copies into shared memory and ldmatrix loads of four 8 x 8 pieces.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  int bytes = pred ? 16 : 0;  // 0 source bytes: the 16 destination bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (lo, hi) minus what `packed` holds of them, as a bfloat16 pair: x = bf16(x) + bf16(x - bf16(x)) to 16 bits
__device__ __forceinline__ uint32_t pack_rest(float lo, float hi, uint32_t packed) {
  const float2 head = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed));
  __nv_bfloat162 v = __floats2bfloat162_rn(lo - head.x, hi - head.y);
  return *reinterpret_cast<uint32_t*>(&v);
}
