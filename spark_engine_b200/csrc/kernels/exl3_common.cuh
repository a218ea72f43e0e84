// Shared device code of the EXL3 kernels: trellis decode (4 bits/weight), codebooks, the warp-level
// 128-point Walsh-Hadamard transform and the m16n8k16 MMA wrapper.
// Format contract: engine-rs/shim/qwen_exl3.cuh:17-117, reference/qwen38/exl3.py:66-110.
#pragma once
#include "../common/ptx.cuh"

namespace spark {

constexpr uint32_t EXL3_MUL1 = 0x83DCD12Du;
constexpr uint32_t EXL3_MCG = 0xCBAC1FEDu;
constexpr float INV_SQRT_128 = 0.08838834764831845f;

// two trellis states -> two fp16 weights packed in a half2
template <int CB>
__device__ __forceinline__ uint32_t exl3_pair(uint32_t s0, uint32_t s1) {
  if (CB == 0) {   // mul1: fp16(1024 + bytesum) * k_inv + k_bias, fused (one rounding)
    const uint32_t a = __dp4a(s0 * EXL3_MUL1, 0x01010101u, 0x6400u);     // 0x6400 + sum == bits of fp16(1024+sum)
    const uint32_t b = __dp4a(s1 * EXL3_MUL1, 0x01010101u, 0x6400u);
    const uint32_t packed = __byte_perm(a, b, 0x5410);
    const __half2 inv = __halves2half2(__ushort_as_half(0x1eee), __ushort_as_half(0x1eee));
    const __half2 bias = __halves2half2(__ushort_as_half(0xc931), __ushort_as_half(0xc931));
    const __half2 v = __hfma2(*reinterpret_cast<const __half2*>(&packed), inv, bias);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {         // mcg: fp16(lo16) + fp16(hi16) of the masked product
    const uint32_t y0 = ((s0 * EXL3_MCG) & 0x8FFF8FFFu) ^ 0x3B603B60u;
    const uint32_t y1 = ((s1 * EXL3_MCG) & 0x8FFF8FFFu) ^ 0x3B603B60u;
    const uint32_t lo = (y0 & 0xFFFFu) | (y1 << 16);
    const uint32_t hi = (y0 >> 16) | (y1 & 0xFFFF0000u);
    const __half2 v = __hadd2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&hi));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// 4-bit tile: lane l holds word l of the tile (32 words) and decodes stream positions 8l..8l+7.
// State j = 16 bits of the (prev:cur) window ending 4(j+1) bits into `cur` (MSB-first stream).
// w[0],w[1] = B fragment of columns 0..7, w[2],w[3] = columns 8..15 (m16n8k16, lane = 4*col + row/2).
template <int CB>
__device__ __forceinline__ void exl3_decode8_b4(uint32_t cur, uint32_t prev, uint32_t (&w)[4]) {
  // The decode is bound by the integer ALU pipe (shift / logic / permute), so the eight 16-bit windows are
  // cut with as few of those as possible: a copy of the window shifted by 4 bits makes every state start
  // on a byte or half-word boundary of one register (byte-permute, shift or mask: one op each); only the
  // two states that straddle `prev` need shift + mask.
  const uint32_t c4 = __funnelshift_r(cur, prev, 4);
  const uint32_t s0 = __funnelshift_r(cur, prev, 28) & 0xFFFFu;
  const uint32_t s1 = __funnelshift_r(cur, prev, 24) & 0xFFFFu;
  const uint32_t s2 = c4 >> 16;                         // window bits 20..35
  const uint32_t s3 = cur >> 16;                        // 16..31
  const uint32_t s4 = __byte_perm(c4, 0u, 0x4421);      // 12..27
  const uint32_t s5 = __byte_perm(cur, 0u, 0x4421);     // 8..23
  const uint32_t s6 = c4 & 0xFFFFu;                     // 4..19
  const uint32_t s7 = cur & 0xFFFFu;                    // 0..15
  w[0] = exl3_pair<CB>(s0, s1);
  w[1] = exl3_pair<CB>(s2, s3);
  w[2] = exl3_pair<CB>(s4, s5);
  w[3] = exl3_pair<CB>(s6, s7);
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 128-point Walsh-Hadamard (unnormalised) held by one warp: lane l owns elements 4l..4l+3.
__device__ __forceinline__ void fwht128_warp(float (&v)[4], int lane) {
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[2] = a - c; v[1] = b + d; v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool hi = lane & m;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = hi ? o - v[i] : v[i] + o;
    }
  }
}

}  // namespace spark
