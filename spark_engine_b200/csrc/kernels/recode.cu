// GEMV over the load-time re-codings of dense weights (<= 16 rows): Q8 (int8 + fp32 scale per row and 128 k),
// Q4 (4-bit codes + fp32 (scale, minimum) per row and 64 k, w = code * scale + minimum) and FP8 per row (e4m3 codes
// + one fp32 scale per row; the codes convert to fp16 exactly and share the Q8 data path, the scale is applied to
// each group's partial dot product).
// Same scheme as the micro-scaled GEMV: 16-byte (Q8) or 8-byte (Q4) pieces of a weight row go straight into
// `mma.sync.m16n8k16` B fragments as exact fp16 integers, one warp iteration covers exactly one scale group, the
// group's integer dot products are scaled in fp32 (Q4 adds minimum * sum of the activations of the group), the 8 warps
// of a CTA split K in a fixed pattern and are summed in warp order.  Run-to-run bitwise equal, rows independent.
// Reference: engine-rs/shim/q8.cuh, q4d.cuh, qwen_q8.cu (int8 / int4 skinny GEMMs).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "../common/ptx.cuh"

namespace spark {

constexpr int RCV_WARPS = 8;
constexpr int RCV_COLS = 16;

__device__ __forceinline__ uint32_t rc_s8x2_to_h2(uint32_t v16) {      // two int8 -> half2, exact
  const uint32_t u = (v16 & 0xFFFFu) ^ 0x8080u;
  const uint32_t packed = __byte_perm(u, 0x64646464u, 0x7170);          // bytes {b0, 0x64, b1, 0x64}
  const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&packed), __float2half2_rn(1152.f));
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t rc_e4m3x2_to_h2(uint32_t v16) {    // two e4m3 codes -> half2, exact
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v16 & 0xFFFFu), __NV_E4M3);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t rc_u4x2_to_h2(uint32_t v8) {       // two 4-bit codes (low nibble first) -> half2
  const uint32_t packed = (v8 & 0x0Fu) | ((v8 & 0xF0u) << 12) | 0x64006400u;
  const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&packed), __float2half2_rn(1024.f));
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void rc_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Q4 = false: W int8 [N,K], sc fp32 [N, K/128].  Q4 = true: W nibbles [N, K/2], sc fp32 [N, K/64, 2].
// One warp iteration = 64 k (Q8: 4 lanes x 16 bytes; Q4: 4 lanes x 8 bytes).
// F8 (with Q4 = false): W e4m3 [N,K], sc fp32 [N].
template <bool Q4, int RB, typename TO, bool F8 = false>
__global__ void __launch_bounds__(RCV_WARPS * 32)
coded_gemv_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const uint8_t* __restrict__ W, const float* __restrict__ sc,
                  TO* __restrict__ y, int ldy, int R, int N, int K) {
  extern __shared__ __align__(16) uint8_t smem_rc[];
  const int XS = K + 8;
  __half* xs = reinterpret_cast<__half*>(smem_rc);                                  // [RB][XS]
  float* red = reinterpret_cast<float*>(smem_rc + static_cast<size_t>(RB) * XS * 2);   // [warps][16][16]
  float* xsum = red + RCV_WARPS * 256;                                              // [RB][K/64] (Q4 only)
  const int G64 = K >> 6;
  for (int i = threadIdx.x; i < RB * (K >> 1); i += blockDim.x) {
    const int r = i / (K >> 1), k = (i - r * (K >> 1)) * 2;
    float2 v = make_float2(0.f, 0.f);
    if (r < R) v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(r) * ldx + k));
    *reinterpret_cast<__half2*>(xs + r * XS + k) = __floats2half2_rn(v.x, v.y);
  }
  __syncthreads();
  if (Q4) {        // sums of the (fp16-rounded) activations per 64-k group, for the minimum term
    for (int i = threadIdx.x; i < RB * G64; i += blockDim.x) {
      const int r = i / G64, gq = i - r * G64;
      float s = 0.f;
      for (int k = 0; k < 64; ++k) s += __half2float(xs[r * XS + gq * 64 + k]);
      xsum[i] = s;
    }
    __syncthreads();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * RCV_COLS;
  const int iters = K >> 6;
  constexpr int BT = Q4 ? 8 : 16;                                  // bytes per lane and iteration
  const size_t row_bytes = Q4 ? (K >> 1) : K;
  const uint8_t* w_lo = W + static_cast<size_t>(n0 + g) * row_bytes + t * BT;
  const uint8_t* w_hi = w_lo + 8 * row_bytes;
  const __half* xa = xs + (g < RB ? g : 0) * XS + t * 16;
  const __half* xb = xs + ((g + 8) < RB ? (g + 8) : 0) * XS + t * 16;
  const bool has_a = g < RB, has_b = (g + 8) < RB;
  // scale addresses of this lane's two output columns per n-tile (columns 2t, 2t+1 of the accumulator fragment)
  const int c00 = n0 + 2 * t, c01 = c00 + 1, c10 = c00 + 8, c11 = c00 + 9;
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  constexpr int U = 4;
  for (int it0 = warp; it0 < iters; it0 += RCV_WARPS * U) {
    uint4 wl[U], wh[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int it = it0 + u * RCV_WARPS;
      if (it < iters) {
        if (Q4) {
          const uint2 a = __ldg(reinterpret_cast<const uint2*>(w_lo + static_cast<size_t>(it) * 32));
          const uint2 b = __ldg(reinterpret_cast<const uint2*>(w_hi + static_cast<size_t>(it) * 32));
          wl[u] = make_uint4(a.x, a.y, 0u, 0u); wh[u] = make_uint4(b.x, b.y, 0u, 0u);
        } else {
          wl[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + static_cast<size_t>(it) * 64));
          wh[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + static_cast<size_t>(it) * 64));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int it = it0 + u * RCV_WARPS;
      if (it >= iters) break;
      float c[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const uint32_t* pl = reinterpret_cast<const uint32_t*>(&wl[u]);
      const uint32_t* ph = reinterpret_cast<const uint32_t*>(&wh[u]);
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        uint2 av = make_uint2(0u, 0u), bv = make_uint2(0u, 0u);
        if (has_a) av = *reinterpret_cast<const uint2*>(xa + it * 64 + s * 4);
        if (has_b) bv = *reinterpret_cast<const uint2*>(xb + it * 64 + s * 4);
        uint32_t b0l, b1l, b0h, b1h;
        if (Q4) {
          const uint32_t vl = pl[s >> 1] >> ((s & 1) * 16), vh = ph[s >> 1] >> ((s & 1) * 16);
          b0l = rc_u4x2_to_h2(vl & 0xFFu); b1l = rc_u4x2_to_h2((vl >> 8) & 0xFFu);
          b0h = rc_u4x2_to_h2(vh & 0xFFu); b1h = rc_u4x2_to_h2((vh >> 8) & 0xFFu);
        } else if (F8) {
          b0l = rc_e4m3x2_to_h2(pl[s]); b1l = rc_e4m3x2_to_h2(pl[s] >> 16);
          b0h = rc_e4m3x2_to_h2(ph[s]); b1h = rc_e4m3x2_to_h2(ph[s] >> 16);
        } else {
          b0l = rc_s8x2_to_h2(pl[s]); b1l = rc_s8x2_to_h2(pl[s] >> 16);
          b0h = rc_s8x2_to_h2(ph[s]); b1h = rc_s8x2_to_h2(ph[s] >> 16);
        }
        rc_mma(c[0], av.x, bv.x, av.y, bv.y, b0l, b1l);
        rc_mma(c[1], av.x, bv.x, av.y, bv.y, b0h, b1h);
      }
      if (Q4) {
        const float2 s00 = __ldg(reinterpret_cast<const float2*>(sc) + static_cast<size_t>(c00) * G64 + it);
        const float2 s01 = __ldg(reinterpret_cast<const float2*>(sc) + static_cast<size_t>(c01) * G64 + it);
        const float2 s10 = __ldg(reinterpret_cast<const float2*>(sc) + static_cast<size_t>(c10) * G64 + it);
        const float2 s11 = __ldg(reinterpret_cast<const float2*>(sc) + static_cast<size_t>(c11) * G64 + it);
        const float xa_s = has_a ? xsum[g * G64 + it] : 0.f, xb_s = has_b ? xsum[(g + 8) * G64 + it] : 0.f;
        acc[0][0] += s00.x * c[0][0] + s00.y * xa_s; acc[0][1] += s01.x * c[0][1] + s01.y * xa_s;
        acc[0][2] += s00.x * c[0][2] + s00.y * xb_s; acc[0][3] += s01.x * c[0][3] + s01.y * xb_s;
        acc[1][0] += s10.x * c[1][0] + s10.y * xa_s; acc[1][1] += s11.x * c[1][1] + s11.y * xa_s;
        acc[1][2] += s10.x * c[1][2] + s10.y * xb_s; acc[1][3] += s11.x * c[1][3] + s11.y * xb_s;
      } else {
        const int gq = F8 ? 0 : it >> 1, G128 = F8 ? 1 : K >> 7;
        const float s00 = __ldg(sc + static_cast<size_t>(c00) * G128 + gq), s01 = __ldg(sc + static_cast<size_t>(c01) * G128 + gq);
        const float s10 = __ldg(sc + static_cast<size_t>(c10) * G128 + gq), s11 = __ldg(sc + static_cast<size_t>(c11) * G128 + gq);
        acc[0][0] = fmaf(s00, c[0][0], acc[0][0]); acc[0][1] = fmaf(s01, c[0][1], acc[0][1]);
        acc[0][2] = fmaf(s00, c[0][2], acc[0][2]); acc[0][3] = fmaf(s01, c[0][3], acc[0][3]);
        acc[1][0] = fmaf(s10, c[1][0], acc[1][0]); acc[1][1] = fmaf(s11, c[1][1], acc[1][1]);
        acc[1][2] = fmaf(s10, c[1][2], acc[1][2]); acc[1][3] = fmaf(s11, c[1][3], acc[1][3]);
      }
    }
  }
  float* rw = red + warp * 256;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    rw[g * 16 + nt * 8 + 2 * t] = acc[nt][0];
    rw[g * 16 + nt * 8 + 2 * t + 1] = acc[nt][1];
    rw[(g + 8) * 16 + nt * 8 + 2 * t] = acc[nt][2];
    rw[(g + 8) * 16 + nt * 8 + 2 * t + 1] = acc[nt][3];
  }
  __syncthreads();
  const int row = threadIdx.x >> 4, col = threadIdx.x & 15;
  if (row < R && n0 + col < N) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < RCV_WARPS; ++w) v += red[w * 256 + row * 16 + col];
    y[static_cast<size_t>(row) * ldy + n0 + col] = static_cast<TO>(v);
  }
}

template <bool Q4, int RB, typename TO, bool F8 = false>
static int launch_coded(const void* x, int ldx, const void* W, const float* sc, void* y, int ldy, int R, int N, int K,
                        cudaStream_t s) {
  auto kern = coded_gemv_kernel<Q4, RB, TO, F8>;
  const int smem = RB * (K + 8) * 2 + RCV_WARPS * 256 * 4 + (Q4 ? RB * (K / 64) * 4 : 0);
  if (smem > 200 * 1024) return -6;
  static bool done = false;
  if (!done) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); done = true; }
  kern<<<N / RCV_COLS, RCV_WARPS * 32, smem, s>>>((const __nv_bfloat16*)x, ldx, (const uint8_t*)W, sc, (TO*)y, ldy, R, N, K);
  return spark_launch_rc(__func__);
}

}  // namespace spark

using namespace spark;

// fmt 2 = Q8, 3 = Q4, 4 = FP8 per row.  R <= 16 rows of bf16 activations; K % 128 == 0, N % 16 == 0.
extern "C" int spark_coded_gemv(const void* x, int ldx, const void* W, const float* scales, int fmt, void* y, int ldy, int R,
                                int N, int K, int out_f32, cudaStream_t s) {
  if (R <= 0) return 0;
  if (R > 16 || N % 16 || K % 128 || (fmt != 2 && fmt != 3 && fmt != 4)) return -5;
#define SPARK_RC(Q, RB)                                                                              \
  (out_f32 ? launch_coded<Q, RB, float>(x, ldx, W, scales, y, ldy, R, N, K, s)                      \
           : launch_coded<Q, RB, __nv_bfloat16>(x, ldx, W, scales, y, ldy, R, N, K, s))
  if (fmt == 2) return R <= 4 ? SPARK_RC(false, 4) : SPARK_RC(false, 16);
  if (fmt == 4) {
    if (R <= 4) return out_f32 ? launch_coded<false, 4, float, true>(x, ldx, W, scales, y, ldy, R, N, K, s)
                               : launch_coded<false, 4, __nv_bfloat16, true>(x, ldx, W, scales, y, ldy, R, N, K, s);
    return out_f32 ? launch_coded<false, 16, float, true>(x, ldx, W, scales, y, ldy, R, N, K, s)
                   : launch_coded<false, 16, __nv_bfloat16, true>(x, ldx, W, scales, y, ldy, R, N, K, s);
  }
  return R <= 4 ? SPARK_RC(true, 4) : SPARK_RC(true, 16);
#undef SPARK_RC
}
