// Micro-scaled weight formats on the decode path and their converters.
//
//   format 0: FP8 e4m3 weights [N,K] with one fp32 scale per 128x128 block (dense projections, shared experts)
//   format 1: MXFP4: E2M1 nibbles [N,K/2] (low nibble = even k) with one E8M0 scale per 32 along K (routed experts)
//
// mx_gemv_kernel: y[R<=16, N] = x[R,K] W^T for decode / verify rows and for MoE (expert,row) pairs.  The weights
// go from global memory straight into `mma.sync.m16n8k16` B fragments: a thread loads 16 consecutive bytes of one
// weight row and feeds them to consecutive k-steps, the activation fragment is read from shared memory with the
// same k permutation (a contraction does not care in which order k is visited as long as A and B agree).  With
// <= 16 rows the kernel is bound by the weight stream, so the warp-level MMA is the right tool: it removes the
// R x FMA cost per weight that a SIMT GEMV pays.  FP8 block scales are applied to a per-iteration accumulator
// (one iteration of a warp never crosses a 128-deep block), MXFP4 scales (powers of two) to the fp16 weight
// pairs.  K is split over the 8 warps of a CTA in a fixed pattern and summed in warp order: run-to-run bitwise
// equal, and a row's result does not depend on the other rows.
// Reference kernels replaced: engine-rs/shim/ds41_mx.cu fp8_gemv_mx / up_mx / down_mx, fp8.cu, fp8ws.cu.
//
// mx_dequant_kernel: both formats -> bf16 [rows, K] for the tcgen05 GEMM of prefill-size batches.
// act_quant kernels: FP8 1x128 (fp32 or power-of-two scale) and MXFP8 1x32 (E8M0) activation quantisation
// (reference/ds41/kernel.py:59-93; engine-rs/shim/ds41_mx.cu:320-375).
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdlib>

#include "../common/ptx.cuh"

#ifndef SPARK_FP4_CVT
#define SPARK_FP4_CVT 0            // 1: E2M1 through the hardware conversion instruction, 0: integer-pipe decode
#endif

namespace spark {

constexpr int MXV_WARPS = 8;
constexpr int MXV_COLS = 16;       // output columns per CTA (two n8 tiles, every warp covers all of them)

__device__ __forceinline__ uint32_t fp8x2_to_h2(uint16_t v) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return static_cast<uint32_t>(r.x) | (static_cast<uint32_t>(r.y) << 16);
}
__device__ __forceinline__ uint32_t h2_scale(uint32_t v, __half2 scale) {
  const __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&v), scale);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t fp4x2_to_h2(uint8_t v, __half2 scale) {
  __half2_raw r = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(v), __NV_E2M1);
  __half2 h = __hmul2(*reinterpret_cast<__half2*>(&r), scale);
  return *reinterpret_cast<uint32_t*>(&h);
}
// Eight E2M1 nibbles of one 32-bit word -> four half2 on the integer pipe (the conversion instruction runs on the
// transcendental unit and caps a memory-bound decode kernel at a fraction of HBM bandwidth).  A nibble s|ee|m shifted
// so that ee|m lands on fp16 bits 11..9 reads as the E2M1 value times 2^-14, subnormal 0.5 included; the 2^14 goes
// into the block scale.  Nibbles i and i+4 sit 16 bits apart, so one shift places both halves of pair i:
// h[i] = (nibble i, nibble i+4).  The staged activations use the matching order within every 8 k.
__device__ __forceinline__ void fp4x8_to_h2x4(uint32_t w, __half2 scale14, uint32_t (&h)[4]) {
  h[0] = h2_scale(((w << 9) & 0x0E000E00u) | ((w << 12) & 0x80008000u), scale14);
  h[1] = h2_scale(((w << 5) & 0x0E000E00u) | ((w << 8) & 0x80008000u), scale14);
  h[2] = h2_scale(((w << 1) & 0x0E000E00u) | ((w << 4) & 0x80008000u), scale14);
  h[3] = h2_scale(((w >> 3) & 0x0E000E00u) | (w & 0x80008000u), scale14);
}
// 2^(e-127) as fp16 (clamped to the normal range of fp16: exponents outside [-14, 15] do not occur in weights)
__device__ __forceinline__ __half2 e8m0_h2(uint8_t e) {
  int ex = static_cast<int>(e) - 127;
  ex = max(-14, min(15, ex));
  const uint16_t bits = static_cast<uint16_t>((ex + 15) << 10);
  __half_raw hr; hr.x = bits;
  return __half2half2(*reinterpret_cast<__half*>(&hr));
}
// 2^(e-127+14) as fp16 for the shift-decoded E2M1 values: block scales from 2^-28 to 2 are exact, which covers
// weights (a scale above 2 would mean weight magnitudes above 12)
__device__ __forceinline__ __half2 e8m0_h2_x14(uint8_t e) {
  int ex = static_cast<int>(e) - 127 + 14;
  ex = max(-14, min(15, ex));
  const uint16_t bits = static_cast<uint16_t>((ex + 15) << 10);
  __half_raw hr; hr.x = bits;
  return __half2half2(*reinterpret_cast<__half*>(&hr));
}
__device__ __forceinline__ float e8m0_f32(uint8_t e) { return __uint_as_float(static_cast<uint32_t>(e ? e : 0) << 23); }

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// FMT 0: W = e4m3 [N,K], scales fp32 [N/128, K/128].  FMT 1: W = nibbles [N,K/2], scales u8 [N, K/32].
// FMT 2: W = e4m3 [N,K], scales u8 (E8M0) [N, K/32] (MXFP8).
// RB = rows held in shared memory (1, 4, 8 or 16).  act 1: x is [gate | up] (2K wide), swiglu while staging.
template <int FMT, int RB, typename TO>
__global__ void __launch_bounds__(MXV_WARPS * 32, 2)
mx_gemv_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const uint8_t* __restrict__ W, const void* __restrict__ scales,
               long long w_expert_stride, long long s_expert_stride, TO* __restrict__ y, int ldy, int rows_per_item,
               int N, int K, const int* __restrict__ pair_expert, const int* __restrict__ pair_row, int act, float limit,
               int cgroups, int xvec) {
  extern __shared__ __align__(16) uint8_t smem_mx[];
  const int XS = K + 8;                                        // row stride in halfs: 16 bytes mod 128 -> no conflicts
  __half* xs = reinterpret_cast<__half*>(smem_mx);              // [RB][XS]
  float* red = reinterpret_cast<float*>(smem_mx + static_cast<size_t>(RB) * XS * 2);   // [2][warps][16][16]
  const int item = blockIdx.y;
  if (pair_expert && pair_expert[item] < 0) return;            // pair of an expert that lives on another rank
  const int e = pair_expert ? pair_expert[item] : 0;
  const int xr0 = pair_row ? pair_row[item] : item * rows_per_item;
  const int R = rows_per_item;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * MXV_COLS * cgroups;
  constexpr int KI = FMT == 1 ? 128 : 64;                      // k per warp iteration (4 threads x 16 bytes)
  constexpr int KT = KI / 4;                                   // k per thread per iteration
  constexpr int STEPS = KT / 4;                                // mma k-steps per iteration
  const int iters = K / KI;
  const size_t row_bytes = FMT == 1 ? (K >> 1) : K;
  const uint8_t* Wb = W + static_cast<size_t>(e) * w_expert_stride;
  const uint8_t* w_lo = Wb + static_cast<size_t>(n0 + g) * row_bytes + t * 16;
  const uint8_t* w_hi = w_lo + 8 * row_bytes;
  const float* sc_f = nullptr;
  const uint8_t* sc_lo = nullptr; const uint8_t* sc_hi = nullptr;
  if (FMT == 0) sc_f = reinterpret_cast<const float*>(scales) + static_cast<size_t>(e) * s_expert_stride;
  else {
    // FMT 1: a lane's 16 bytes are one 32-k scale block; FMT 2: 16 k = half a block, lanes (0,1) and (2,3) share one
    sc_lo = reinterpret_cast<const uint8_t*>(scales) + static_cast<size_t>(e) * s_expert_stride +
            static_cast<size_t>(n0 + g) * (K >> 5) + (FMT == 1 ? t : (t >> 1));
    sc_hi = sc_lo + 8 * (K >> 5);
  }
  constexpr int SPI = FMT == 1 ? 4 : 2;                        // scale blocks per warp iteration
  const __half* xa = xs + (g < RB ? g : 0) * XS + t * KT;       // row g of A
  const __half* xb = xs + ((g + 8) < RB ? (g + 8) : 0) * XS + t * KT;
  const bool has_a = g < RB, has_b = (g + 8) < RB;

  // A CTA walks `cgroups` groups of 16 output columns with the staged rows kept in shared memory.  The weight loads
  // of batch b+1 (the next U k-slices of this warp, or the first ones of the next column group) are issued before
  // the MMAs of batch b, so the memory pipe stays full across the per-group reductions.
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  constexpr int U = 4;                                         // k-slices per batch
  const int nb = (iters + MXV_WARPS * U - 1) / (MXV_WARPS * U);      // batches per column group
  const int total = cgroups * nb;
  uint4 wl0[U], wh0[U], wl1[U], wh1[U];
  uint8_t sl0[U], sh0[U], sl1[U], sh1[U];

  auto load = [&](uint4 (&wl)[U], uint4 (&wh)[U], uint8_t (&sl)[U], uint8_t (&sh)[U], int bi) {
    if (bi >= total) return;
    const int cg = bi / nb, kb = bi - cg * nb;
    const size_t goff = static_cast<size_t>(cg) * MXV_COLS * row_bytes;
    const size_t soff = static_cast<size_t>(cg) * MXV_COLS * (K >> 5);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int it = (kb * MXV_WARPS + warp) * U + u;          // U adjacent k-slices: 64 * U contiguous bytes per row
      if (it < iters) {
        wl[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + goff + static_cast<size_t>(it) * 64));
        wh[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + goff + static_cast<size_t>(it) * 64));
        if (FMT != 0) { sl[u] = __ldg(sc_lo + soff + it * SPI); sh[u] = __ldg(sc_hi + soff + it * SPI); }
      }
    }
  };

  auto compute = [&](const uint4 (&wl)[U], const uint4 (&wh)[U], const uint8_t (&sl)[U], const uint8_t (&sh)[U], int bi) {
    const int cg = bi / nb, kb = bi - cg * nb;
    const int nc = n0 + cg * MXV_COLS;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int it = (kb * MXV_WARPS + warp) * U + u;          // U adjacent k-slices: 64 * U contiguous bytes per row
      if (it >= iters) break;
      float c[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const uint32_t* pl = reinterpret_cast<const uint32_t*>(&wl[u]);
      const uint32_t* ph = reinterpret_cast<const uint32_t*>(&wh[u]);
      __half2 hl, hh;
      if (FMT == 2) { hl = e8m0_h2(sl[u]); hh = e8m0_h2(sh[u]); }
#if SPARK_FP4_CVT
      if (FMT == 1) { hl = e8m0_h2(sl[u]); hh = e8m0_h2(sh[u]); }
#else
      if (FMT == 1) { hl = e8m0_h2_x14(sl[u]); hh = e8m0_h2_x14(sh[u]); }
#endif
      uint32_t dl[4], dh[4];
#pragma unroll
      for (int s = 0; s < STEPS; ++s) {
        // A: 4 staged k of rows g / g+8
        uint2 av = make_uint2(0u, 0u), bv = make_uint2(0u, 0u);
        if (has_a) av = *reinterpret_cast<const uint2*>(xa + it * KI + s * 4);
        if (has_b) bv = *reinterpret_cast<const uint2*>(xb + it * KI + s * 4);
        uint32_t b0l, b1l, b0h, b1h;
        if (FMT == 0) {
          const uint32_t vl = pl[s], vh = ph[s];
          b0l = fp8x2_to_h2(static_cast<uint16_t>(vl & 0xffffu)); b1l = fp8x2_to_h2(static_cast<uint16_t>(vl >> 16));
          b0h = fp8x2_to_h2(static_cast<uint16_t>(vh & 0xffffu)); b1h = fp8x2_to_h2(static_cast<uint16_t>(vh >> 16));
        } else if (FMT == 2) {
          const uint32_t vl = pl[s], vh = ph[s];
          b0l = h2_scale(fp8x2_to_h2(static_cast<uint16_t>(vl & 0xffffu)), hl); b1l = h2_scale(fp8x2_to_h2(static_cast<uint16_t>(vl >> 16)), hl);
          b0h = h2_scale(fp8x2_to_h2(static_cast<uint16_t>(vh & 0xffffu)), hh); b1h = h2_scale(fp8x2_to_h2(static_cast<uint16_t>(vh >> 16)), hh);
        } else {
#if SPARK_FP4_CVT
          const uint32_t vl = pl[s >> 1] >> ((s & 1) * 16), vh = ph[s >> 1] >> ((s & 1) * 16);
          b0l = fp4x2_to_h2(static_cast<uint8_t>(vl & 0xffu), hl); b1l = fp4x2_to_h2(static_cast<uint8_t>((vl >> 8) & 0xffu), hl);
          b0h = fp4x2_to_h2(static_cast<uint8_t>(vh & 0xffu), hh); b1h = fp4x2_to_h2(static_cast<uint8_t>((vh >> 8) & 0xffu), hh);
#else
          // one 32-bit word feeds two steps: pairs (0,4),(1,5) then (2,6),(3,7) of its 8 k
          if ((s & 1) == 0) { fp4x8_to_h2x4(pl[s >> 1], hl, dl); fp4x8_to_h2x4(ph[s >> 1], hh, dh); }
          b0l = dl[(s & 1) * 2]; b1l = dl[(s & 1) * 2 + 1];
          b0h = dh[(s & 1) * 2]; b1h = dh[(s & 1) * 2 + 1];
#endif
        }
        mma16816(c[0], av.x, bv.x, av.y, bv.y, b0l, b1l);
        mma16816(c[1], av.x, bv.x, av.y, bv.y, b0h, b1h);
      }
      float sc = 1.f;
      if (FMT == 0) sc = __ldg(sc_f + static_cast<size_t>(nc >> 7) * (K >> 7) + ((it * KI) >> 7));
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[0][j] = fmaf(c[0][j], sc, acc[0][j]); acc[1][j] = fmaf(c[1][j], sc, acc[1][j]); }
    }
    if (kb == nb - 1) {
      // fixed-order sum over the warps: red[parity][warp][row][col]; the parity buffer lets the next group's
      // partials land while slow threads still read this group's
      float* rb = red + (cg & 1) * (MXV_WARPS * 256);
      float* rw = rb + warp * 256;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        rw[g * 16 + nt * 8 + 2 * t] = acc[nt][0];
        rw[g * 16 + nt * 8 + 2 * t + 1] = acc[nt][1];
        rw[(g + 8) * 16 + nt * 8 + 2 * t] = acc[nt][2];
        rw[(g + 8) * 16 + nt * 8 + 2 * t + 1] = acc[nt][3];
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      }
      __syncthreads();
      const int row = threadIdx.x >> 4, col = threadIdx.x & 15;
      if (row < R && nc + col < N) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < MXV_WARPS; ++w) v += rb[w * 256 + row * 16 + col];
        y[static_cast<size_t>(item * rows_per_item + row) * ldy + nc + col] = static_cast<TO>(v);
      }
    }
  };

  load(wl0, wh0, sl0, sh0, 0);            // the first weights are in flight while the rows are staged
  if (xvec) {
    // 16-byte loads, four in flight per thread: the rows are staged in about one memory latency
    const int K8 = K >> 3, chunks = RB * K8;
    constexpr int SU = 4;
    for (int i0 = threadIdx.x; i0 < chunks; i0 += blockDim.x * SU) {
      uint4 gq[SU], uq[SU];
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int i = i0 + u * blockDim.x;
        gq[u] = make_uint4(0u, 0u, 0u, 0u); uq[u] = gq[u];
        if (i < chunks) {
          const int r = i / K8, k = (i - r * K8) * 8;
          if (r < R) {
            const __nv_bfloat16* xr = x + static_cast<size_t>(xr0 + r) * ldx;
            gq[u] = *reinterpret_cast<const uint4*>(xr + k);
            if (act != 0) uq[u] = *reinterpret_cast<const uint4*>(xr + K + k);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i >= chunks) break;
        const int r = i / K8, k = (i - r * K8) * 8;
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gq[u]);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uq[u]);
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = __bfloat1622float2(gp[j]);
          float v0 = g.x, v1 = g.y;
          if (act != 0) {
            const float2 uu = __bfloat1622float2(up[j]);
            float g0 = g.x, g1 = g.y, u0 = uu.x, u1 = uu.y;
            if (limit > 0.f) {
              g0 = fminf(g0, limit); g1 = fminf(g1, limit);
              u0 = fminf(fmaxf(u0, -limit), limit); u1 = fminf(fmaxf(u1, -limit), limit);
            }
            v0 = g0 / (1.f + __expf(-g0)) * u0; v1 = g1 / (1.f + __expf(-g1)) * u1;
          }
          const __half2 h = __floats2half2_rn(v0, v1);
          op[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        if (FMT == 1 && !SPARK_FP4_CVT) o = make_uint4(__byte_perm(o.x, o.z, 0x5410), __byte_perm(o.x, o.z, 0x7632),     // k order 0 4 1 5 2 6 3 7
                                     __byte_perm(o.y, o.w, 0x5410), __byte_perm(o.y, o.w, 0x7632));
        *reinterpret_cast<uint4*>(xs + r * XS + k) = o;
      }
    }
  } else {
    for (int i = threadIdx.x; i < RB * (K >> 1); i += blockDim.x) {
      const int r = i / (K >> 1), k = (i - r * (K >> 1)) * 2;
      float v0 = 0.f, v1 = 0.f;
      if (r < R) {
        const __nv_bfloat16* xr = x + static_cast<size_t>(xr0 + r) * ldx;
        const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + k));
        if (act == 0) { v0 = g.x; v1 = g.y; }
        else {
          const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + K + k));
          float g0 = g.x, g1 = g.y, u0 = u.x, u1 = u.y;
          if (limit > 0.f) {
            g0 = fminf(g0, limit); g1 = fminf(g1, limit);
            u0 = fminf(fmaxf(u0, -limit), limit); u1 = fminf(fmaxf(u1, -limit), limit);
          }
          v0 = g0 / (1.f + __expf(-g0)) * u0; v1 = g1 / (1.f + __expf(-g1)) * u1;
        }
      }
      if (FMT == 1 && !SPARK_FP4_CVT) {                   // k order 0 4 1 5 2 6 3 7 within every 8 (matches fp4x8_to_h2x4)
        __half* q = xs + r * XS + (k & ~7);
        q[(k & 3) * 2 + ((k & 7) >> 2)] = __float2half_rn(v0);
        q[((k + 1) & 3) * 2 + (((k + 1) & 7) >> 2)] = __float2half_rn(v1);
      } else {
        *reinterpret_cast<__half2*>(xs + r * XS + k) = __floats2half2_rn(v0, v1);
      }
    }
  }
  __syncthreads();

  for (int bi = 0; bi < total; bi += 2) {
    load(wl1, wh1, sl1, sh1, bi + 1);
    compute(wl0, wh0, sl0, sh0, bi);
    load(wl0, wh0, sl0, sh0, bi + 2);
    if (bi + 1 < total) compute(wl1, wh1, sl1, sh1, bi + 1);
  }
}

template <int FMT, int RB, typename TO>
static int launch_mx_gemv(const void* x, int ldx, const void* W, const void* sc, long long wes, long long ses, void* y,
                          int ldy, int items, int rows, int N, int K, const int* pe, const int* pr, int act, float limit,
                          cudaStream_t s) {
  auto kern = mx_gemv_kernel<FMT, RB, TO>;
  const int smem = RB * (K + 8) * 2 + 2 * MXV_WARPS * 256 * 4;
  if (smem > 200 * 1024) return -6;
  // column groups per CTA: as many as keep four CTAs per SM's worth of work in the grid
  const int ngroups = N / MXV_COLS;
  int cgroups = 1;
  static const bool xvec_ok = [] { const char* e = getenv("SPARK_MXV_XVEC"); return !e || atoi(e) != 0; }();
  static const int cg_max = [] { const char* e = getenv("SPARK_MXV_CG"); return e ? atoi(e) : 4; }();   // tuning knob
  for (int c = cg_max; c > 1; c >>= 1)
    if (ngroups % c == 0 && static_cast<long long>(ngroups / c) * items >= 592) { cgroups = c; break; }
  if (smem > 48 * 1024) {
    static int set_for = 0;
    if (!set_for) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); set_for = 1; }
  }
  dim3 grid(ngroups / cgroups, items);
  kern<<<grid, MXV_WARPS * 32, smem, s>>>((const __nv_bfloat16*)x, ldx, (const uint8_t*)W, sc, wes, ses, (TO*)y, ldy, rows,
                                          N, K, pe, pr, act, limit, cgroups,
                                          xvec_ok && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (ldx & 7) == 0 ? 1 : 0);
  return spark_launch_rc(__func__);
}

template <int FMT, typename TO>
static int dispatch_rows(const void* x, int ldx, const void* W, const void* sc, long long wes, long long ses, void* y,
                         int ldy, int items, int rows, int N, int K, const int* pe, const int* pr, int act, float limit,
                         cudaStream_t s) {
  if (rows <= 1) return launch_mx_gemv<FMT, 1, TO>(x, ldx, W, sc, wes, ses, y, ldy, items, rows, N, K, pe, pr, act, limit, s);
  if (rows <= 4) return launch_mx_gemv<FMT, 4, TO>(x, ldx, W, sc, wes, ses, y, ldy, items, rows, N, K, pe, pr, act, limit, s);
  if (rows <= 8) return launch_mx_gemv<FMT, 8, TO>(x, ldx, W, sc, wes, ses, y, ldy, items, rows, N, K, pe, pr, act, limit, s);
  return launch_mx_gemv<FMT, 16, TO>(x, ldx, W, sc, wes, ses, y, ldy, items, rows, N, K, pe, pr, act, limit, s);
}

// ------------------------------------------------------------------------------------------ dequant to bf16
// one thread = 16 consecutive k of one row; rows = experts x N flattened (scales follow the same flattening)
template <int FMT>
__global__ void mx_dequant_kernel(const uint8_t* __restrict__ W, const void* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                                  long long rows, int N, int K) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = K >> 4;
  if (i >= rows * per_row) return;
  const long long r = i / per_row;
  const int k0 = static_cast<int>(i - r * per_row) << 4;
  float v[16];
  if (FMT == 0) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(W + r * K + k0));
    const long long e = r / N; const int n = static_cast<int>(r - e * N);
    const float sc = __ldg(reinterpret_cast<const float*>(scales) + (e * (N >> 7) + (n >> 7)) * (K >> 7) + (k0 >> 7));
    const uint16_t* p = reinterpret_cast<const uint16_t*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t h = fp8x2_to_h2(p[j]);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
      v[2 * j] = f.x * sc; v[2 * j + 1] = f.y * sc;
    }
  } else {
    const uint2 q = __ldg(reinterpret_cast<const uint2*>(W + r * (K >> 1) + (k0 >> 1)));
    const float sc = e8m0_f32(__ldg(reinterpret_cast<const uint8_t*>(scales) + r * (K >> 5) + (k0 >> 5)));
    const uint8_t* p = reinterpret_cast<const uint8_t*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(p[j]), __NV_E2M1);
      const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
      v[2 * j] = f.x * sc; v[2 * j + 1] = f.y * sc;
    }
  }
  uint4 o[2];
  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
  for (int j = 0; j < 8; ++j) ob[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  uint4* dst = reinterpret_cast<uint4*>(out + r * K + k0);
  dst[0] = o[0]; dst[1] = o[1];
}

// ------------------------------------------------------------------------------------------ activation quant
// One warp per (row, block).  BLOCK 128 -> e4m3 + fp32 scale (amax/448, clamp 1e-4; optionally rounded up to a
// power of two); BLOCK 32 -> e4m3 + E8M0 scale byte (MXFP8: 2^ceil(log2(amax/448))).  act 1: x = [gate | up].
template <int BLOCK, typename TI>
__global__ void act_quant_kernel(const TI* __restrict__ x, int ldx, uint8_t* __restrict__ q, void* __restrict__ scales, int R,
                                 int K, int pow2, int act, float limit) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nb = K / BLOCK;
  if (warp >= R * nb) return;
  const int r = warp / nb, b = warp - r * nb;
  constexpr int PER = BLOCK / 32;
  float v[PER];
  float amax = 0.f;
  const TI* xr = x + static_cast<size_t>(r) * ldx;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int k = b * BLOCK + lane * PER + j;
    float a = static_cast<float>(xr[k]);
    if (act) {
      float u = static_cast<float>(xr[K + k]);
      if (limit > 0.f) { a = fminf(a, limit); u = fminf(fmaxf(u, -limit), limit); }
      a = a / (1.f + __expf(-a)) * u;
    }
    v[j] = a;
    amax = fmaxf(amax, fabsf(a));
  }
  amax = warp_max(amax);
  amax = fmaxf(amax, 1e-4f);
  float sc = amax / 448.f;
  if (BLOCK == 32 || pow2) sc = exp2f(ceilf(log2f(sc)));
  if (lane == 0) {
    if (BLOCK == 32) reinterpret_cast<uint8_t*>(scales)[static_cast<size_t>(r) * nb + b] =
        static_cast<uint8_t>(__float_as_uint(sc) >> 23);
    else reinterpret_cast<float*>(scales)[static_cast<size_t>(r) * nb + b] = sc;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const float s = fminf(fmaxf(v[j] / sc, -448.f), 448.f);
    q[static_cast<size_t>(r) * K + b * BLOCK + lane * PER + j] =
        static_cast<uint8_t>(__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3));
  }
}

}  // namespace spark

using namespace spark;

// fmt 0 = FP8 128x128-block scales (fp32), 1 = MXFP4, 2 = MXFP8 (E8M0 per 32).  Strides are per expert (bytes for W, elements for scales).
extern "C" int spark_mx_gemv(const void* x, int ldx, const void* W, const void* scales, int fmt, long long w_expert_stride,
                             long long s_expert_stride, void* y, int ldy, int items, int rows_per_item, int N, int K,
                             const int* pair_expert, const int* pair_row, int act, float limit, int out_f32, cudaStream_t s) {
  if (items <= 0 || rows_per_item <= 0) return 0;
  if (rows_per_item > 16 || N % 16 || K % 128) return -5;
#define SPARK_MXV(FMT, TO) dispatch_rows<FMT, TO>(x, ldx, W, scales, w_expert_stride, s_expert_stride, y, ldy, items, \
                                                  rows_per_item, N, K, pair_expert, pair_row, act, limit, s)
  if (fmt == 0) return out_f32 ? SPARK_MXV(0, float) : SPARK_MXV(0, __nv_bfloat16);
  if (fmt == 1) return out_f32 ? SPARK_MXV(1, float) : SPARK_MXV(1, __nv_bfloat16);
  if (fmt == 2) return out_f32 ? SPARK_MXV(2, float) : SPARK_MXV(2, __nv_bfloat16);
#undef SPARK_MXV
  return -5;
}

extern "C" int spark_mx_dequant(const void* W, const void* scales, int fmt, void* out, long long rows, int N, int K,
                                cudaStream_t s) {
  if (rows <= 0) return 0;
  if (K % 128 || N % 128) return -5;
  const long long n = rows * (K >> 4);
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  if (fmt == 0) mx_dequant_kernel<0><<<blocks, 256, 0, s>>>((const uint8_t*)W, scales, (__nv_bfloat16*)out, rows, N, K);
  else mx_dequant_kernel<1><<<blocks, 256, 0, s>>>((const uint8_t*)W, scales, (__nv_bfloat16*)out, rows, N, K);
  return spark_launch_rc(__func__);
}

// block 128 -> fp32 scales [R, K/128]; block 32 -> E8M0 bytes [R, K/32].  x bf16 (in_f32 0) or fp32.
extern "C" int spark_act_quant(const void* x, int ldx, int in_f32, void* q, void* scales, int R, int K, int block, int pow2,
                               int act, float limit, cudaStream_t s) {
  if (R <= 0) return 0;
  if ((block != 128 && block != 32) || K % block) return -5;
  const long long warps = static_cast<long long>(R) * (K / block);
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
#define SPARK_AQ(B, T) act_quant_kernel<B, T><<<blocks, 256, 0, s>>>((const T*)x, ldx, (uint8_t*)q, scales, R, K, pow2, act, limit)
  if (block == 128) { if (in_f32) SPARK_AQ(128, float); else SPARK_AQ(128, __nv_bfloat16); }
  else { if (in_f32) SPARK_AQ(32, float); else SPARK_AQ(32, __nv_bfloat16); }
#undef SPARK_AQ
  return spark_launch_rc(__func__);
}

// ------------------------------------------------------------------------------------------ grouped MXFP4 GEMM
// Prefill-size MoE over MXFP4 experts: rows in expert order, <= 64 rows per work item (a half of a 128-row tile of
// the MoE sort).  The packed expert weights cross HBM once (0.5 byte per weight + scales) and go straight into MMA
// fragments, exactly like the decode GEMV, but every decoded fragment now feeds up to four 16-row tiles; the
// activations of the item (bf16 -> fp16, optional SwiGLU of a [gate | up] input) are staged per 512-deep K chunk and
// shared by the 8 warps of the CTA, each of which owns 16 output columns for the whole K (no cross-warp reduction:
// one fixed summation order per output).  Grid (N/128, 2 * tiles).
namespace spark {

constexpr int MXG_KC = 512;        // K chunk staged in shared memory
constexpr int MXG_ROWS = 64;

__global__ void __launch_bounds__(256, 2)
mx_mgemm_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const uint8_t* __restrict__ W, const uint8_t* __restrict__ scales,
                long long w_expert_stride, long long s_expert_stride, const int4* __restrict__ tiles,
                const int* __restrict__ ntile, void* __restrict__ y, int ldy, int out_f32, int N, int K, int act, float limit) {
  const int tile = blockIdx.y >> 1, half = blockIdx.y & 1;
  if (tile >= *ntile) return;
  const int4 td = tiles[tile];
  const int row0 = td.x + half * MXG_ROWS;
  const int nrows = min(min(td.x + 128, td.y) - row0, MXG_ROWS);
  if (nrows <= 0) return;
  const int e = td.z;
  // Activation layout in shared memory: inside every 128-k block the four lanes' 32-k runs are interleaved in groups
  // of four elements (element k sits at ((k % 32) / 4) * 16 + (k / 32) * 4 + k % 4), so that the 8-byte fragment
  // loads of a k-step are contiguous over the lane quad; with rows 32 bytes (mod 128) apart a warp's 32 loads
  // cover 256 bytes in the minimum of two shared-memory wavefronts.
  constexpr int XS = MXG_KC + 16;
  extern __shared__ __align__(16) uint8_t smem_mg[];
  __half* xs = reinterpret_cast<__half*>(smem_mg);              // [64][XS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int mts = (nrows + 15) >> 4;
  const int n0 = blockIdx.x * 128 + warp * 16;
  const size_t row_bytes = K >> 1;
  const uint8_t* w_lo = W + static_cast<size_t>(e) * w_expert_stride + static_cast<size_t>(n0 + g) * row_bytes + t * 16;
  const uint8_t* w_hi = w_lo + 8 * row_bytes;
  const uint8_t* sc_lo = scales + static_cast<size_t>(e) * s_expert_stride + static_cast<size_t>(n0 + g) * (K >> 5) + t;
  const uint8_t* sc_hi = sc_lo + 8 * (K >> 5);
  float acc[4][2][4];
#pragma unroll
  for (int m = 0; m < 4; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[m][0][j] = 0.f; acc[m][1][j] = 0.f; }
  constexpr int IPC = MXG_KC / 128;                // warp iterations per chunk (128 k each)
  for (int k0 = 0; k0 < K; k0 += MXG_KC) {
    // this chunk's packed weights are requested before the activations are staged
    uint4 wl[IPC], wh[IPC];
    uint8_t sl[IPC], sh[IPC];
#pragma unroll
    for (int u = 0; u < IPC; ++u) {
      const int it = (k0 >> 7) + u;
      if (k0 + u * 128 < K) {
        wl[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + static_cast<size_t>(it) * 64));
        wh[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + static_cast<size_t>(it) * 64));
        sl[u] = __ldg(sc_lo + it * 4); sh[u] = __ldg(sc_hi + it * 4);
      }
    }
    __syncthreads();                                // previous chunk fully consumed
    const int kc = min(MXG_KC, K - k0);
    // stage the chunk: 16-byte loads, four in flight per thread before any is converted (the loads come from L2 and
    // a dependent load-convert-store chain would leave the CTA waiting on latency)
    const int vpr = kc >> 3, total = mts * 16 * vpr;
    for (int base = threadIdx.x; base < total; base += 256 * 4) {
      uint4 gv[4], uv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = base + j * 256;
        gv[j] = make_uint4(0u, 0u, 0u, 0u); uv[j] = gv[j];
        if (i < total) {
          const int r = i / vpr, k = (i - r * vpr) * 8;
          if (r < nrows) {
            const __nv_bfloat16* xr = x + static_cast<size_t>(row0 + r) * ldx + k0 + k;
            gv[j] = *reinterpret_cast<const uint4*>(xr);
            if (act) uv[j] = *reinterpret_cast<const uint4*>(xr + K);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = base + j * 256;
        if (i >= total) break;
        const int r = i / vpr, k = (i - r * vpr) * 8;
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv[j]);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv[j]);
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 gg = __bfloat1622float2(gp[q]);
          if (act) {
            float2 uu = __bfloat1622float2(up[q]);
            if (limit > 0.f) {
              gg.x = fminf(gg.x, limit); gg.y = fminf(gg.y, limit);
              uu.x = fminf(fmaxf(uu.x, -limit), limit); uu.y = fminf(fmaxf(uu.y, -limit), limit);
            }
            gg.x = gg.x / (1.f + __expf(-gg.x)) * uu.x; gg.y = gg.y / (1.f + __expf(-gg.y)) * uu.y;
          }
          h[q] = __floats2half2_rn(gg.x, gg.y);
        }
        // elements k..k+3 and k+4..k+7 are two consecutive 4-groups of one lane's 32-k run
        const int kk = k & 127;
        __half* dst = xs + r * XS + (k - kk) + ((kk & 31) >> 2) * 16 + (kk >> 5) * 4;
        *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]));
        *reinterpret_cast<uint2*>(dst + 16) = make_uint2(*reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
      }
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < IPC; ++u) {
      if (k0 + u * 128 >= K) break;
      const uint32_t* pl = reinterpret_cast<const uint32_t*>(&wl[u]);
      const uint32_t* ph = reinterpret_cast<const uint32_t*>(&wh[u]);
      const __half2 hl = e8m0_h2(sl[u]), hh = e8m0_h2(sh[u]);
      const __half* xk = xs + g * XS + u * 128 + t * 4;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const uint32_t vl = pl[s >> 1] >> ((s & 1) * 16), vh = ph[s >> 1] >> ((s & 1) * 16);
        const uint32_t b0l = fp4x2_to_h2(static_cast<uint8_t>(vl & 0xffu), hl), b1l = fp4x2_to_h2(static_cast<uint8_t>((vl >> 8) & 0xffu), hl);
        const uint32_t b0h = fp4x2_to_h2(static_cast<uint8_t>(vh & 0xffu), hh), b1h = fp4x2_to_h2(static_cast<uint8_t>((vh >> 8) & 0xffu), hh);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          if (m < mts) {
            const uint2 av = *reinterpret_cast<const uint2*>(xk + (m * 16) * XS + s * 16);
            const uint2 bv = *reinterpret_cast<const uint2*>(xk + (m * 16 + 8) * XS + s * 16);
            mma16816(acc[m][0], av.x, bv.x, av.y, bv.y, b0l, b1l);
            mma16816(acc[m][1], av.x, bv.x, av.y, bv.y, b0h, b1h);
          }
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    if (m >= mts) break;
#pragma unroll
    for (int hh2 = 0; hh2 < 2; ++hh2) {
      const int r = m * 16 + g + hh2 * 8;
      if (r >= nrows) continue;
      const size_t o = static_cast<size_t>(row0 + r) * ldy + n0 + 2 * t;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float v0 = acc[m][nt][2 * hh2], v1 = acc[m][nt][2 * hh2 + 1];
        if (out_f32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(y) + o + nt * 8) = make_float2(v0, v1);
        else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(y) + o + nt * 8) = __floats2bfloat162_rn(v0, v1);
      }
    }
  }
}

}  // namespace spark

// MXFP4 experts, rows in expert order; tiles = the 128-row tile list of the MoE sort (max_tiles allocated, *ntile valid).
// x bf16 [P, K] (act 0) or [P, 2K] = [gate | up] (act 1); y [P, N] bf16 or fp32.  N % 128 == 0, K % 128 == 0.
extern "C" int spark_mx_mgemm(const void* x, int ldx, const void* W, const void* scales, long long w_expert_stride,
                              long long s_expert_stride, const void* tiles, const int* ntile, int max_tiles, void* y, int ldy,
                              int out_f32, int N, int K, int act, float limit, cudaStream_t s) {
  if (max_tiles <= 0) return 0;
  if (N % 128 || K % 128 || (ldx & 7) || (ldy & 1)) return -5;
  constexpr int smem = spark::MXG_ROWS * (spark::MXG_KC + 16) * 2;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(spark::mx_mgemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr = true; }
  spark::mx_mgemm_kernel<<<dim3(N / 128, 2 * max_tiles), 256, smem, s>>>((const __nv_bfloat16*)x, ldx, (const uint8_t*)W,
                                                                     (const uint8_t*)scales, w_expert_stride, s_expert_stride,
                                                                     (const int4*)tiles, ntile, y, ldy, out_f32, N, K, act, limit);
  return spark_launch_rc(__func__);
}
