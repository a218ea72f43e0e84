// EXL3 GEMV for <= 16 rows (decode / verify rows, MoE (row, expert) pairs):
//   y = had128( had128(x * suh) @ inner ) * svh
// One launch: input Hadamard, trellis decode, product, output Hadamard.  Grid (N/128, S, items) with a
// thread-block cluster of S CTAs along the K-slices of one 128-column strip: every CTA streams the
// 128-byte tiles of its slice (all loads of a warp are issued before the first decode, so one DRAM
// round trip covers 16 tiles), decodes 8 weights per lane straight into m16n8k16 B fragments and
// multiplies with the <= 16 activation rows; every CTA then stores its partial strip into the shared
// memory of cluster rank 0 (distributed shared memory), which sums the slices in slice order (no global
// scratch, no atomics), applies the output Hadamard transform and scales.  Fixed reduction order => bitwise reproducible and independent of the rows in flight.
// M <= 16 is bandwidth / decode-ALU bound, so the warp-level MMA feeds it; GEMM-shaped EXL3 work goes
// through exl3_reconstruct to the tcgen05 GEMM.
// Replaces engine-rs/shim/qwen_exl3.cuh:427-626 (gemv_kernel / gemv_fused_kernel / finish_kernel) and
// the decode half of moe_exl3.cuh:273-399.
#include "exl3_common.cuh"
#include "../common/comm.cuh"
#include "../common/decode.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace spark {

struct Exl3GemvArgs {
  const __nv_bfloat16* x; int ldx;             // activations [rows, K] (or [rows, 2K] = [gate | up] when act == 1)
  const uint32_t* trellis;                      // [E][K/16][N/16][32] words (4 bpw)
  const __half* suh; const __half* svh;         // [E][K], [E][N]
  long long t_stride, suh_stride, svh_stride;   // per expert, in elements
  void* y; int ldy; int out_f32;                // [items*R, N]
  const int* pair_expert; const int* pair_row;
  int R, K, N, S, act; float limit;
  int fuse_ar;                                  // 1: row-parallel layer under TP: the epilogue pushes the strip to every
  ArRows ar;                                    //    rank's slots and raises the flag; a tail launch reduces the rows
  int pairs_early;                              // pair tables were written at least two launches back: they may be read
};                                              // (and the weight loads issued) before the dependency wait

#ifndef SPARK_EXL3_MINB
#define SPARK_EXL3_MINB 6   // 40 registers: 6 CTAs (48 warps) per SM; measured faster than 4 (64 regs) or 2 (94 regs)
#endif
constexpr int EXL3_MAX_KS = 2048;              // K-slice per CTA (activation slice lives in shared memory)

// Fused all-reduce, push side (kept out of line so that it costs the GEMV no registers): the last strip of this rank
// to finish raises this rank's flag on every peer.  The reduction itself (wait for every rank's flag, rank-ordered
// sum + residual + RMSNorm) runs as a second launch with one CTA per row (ar_tail_kernel): a single finisher CTA
// serialised all rows (measured 29 us for 4 rows against 6 + 11 us for the GEMV and a stand-alone all-reduce).
__device__ __noinline__ void exl3_fused_ar_arrive(const Exl3GemvArgs& a) {
  const uint32_t seq = comm_seq(a.ar.seq_ptr, a.ar.seq);
  __syncthreads();
  if (threadIdx.x == 0) {
    ArRows ar = a.ar;
    ar.seq_ptr = nullptr;                                  // the tail kernel closes the sequence
    ar_arrive_and_is_last(ar, seq, gridDim.x);
  }
}

template <int CB, bool HI>       // HI: more than 8 activation rows (the upper half of the MMA tile is live)
__global__ void __launch_bounds__(256, SPARK_EXL3_MINB)
exl3_gemv_kernel(const __grid_constant__ Exl3GemvArgs a) {
  // (the argument block stays in constant memory: a local copy would put every field access on the stack)
  // Weight loads depend on no earlier launch; everything else is read after the dependency wait.
  const bool early = a.pair_expert == nullptr || a.pairs_early;
  if (!early) pdl_wait();
  if (a.pair_expert && a.pair_expert[blockIdx.z] < 0) {         // expert on another rank (whole cluster leaves)
    if (early) pdl_wait();
    return;
  }
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  __half* xh = reinterpret_cast<__half*>(smem_dyn);          // [16][Ks + 8]
  cg::cluster_group cluster = cg::this_cluster();
  const int strip = blockIdx.x, slice = blockIdx.y, item = blockIdx.z;
  const int NT = a.N >> 4;
  const int Ks = a.K / a.S, kts = Ks >> 4;
  const int ldh = Ks + 8;
  float* red = reinterpret_cast<float*>(smem_dyn + 16 * ldh * 2);   // [S][R][128]: slice partials, used on rank 0
  const int k_begin = slice * Ks;
  const int e = a.pair_expert ? a.pair_expert[item] : 0;
  const int xr0 = a.pair_row ? a.pair_row[item] : item * a.R;
  const int R = a.R;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // every CTA of the cluster must be running before its shared memory is written remotely: arrive now, wait
  // right before the first remote store
  if (a.S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  // ---- issue this warp's trellis loads first (they do not depend on the prologue)
  const int nt = strip * 8 + warp;
  const uint32_t* tw = a.trellis + e * a.t_stride + (static_cast<size_t>(slice) * kts * NT + nt) * 32 + lane;
  // (kts is a multiple of 8: batches of 8 tiles, the next batch is in flight while one is decoded)
  uint32_t cur[8], nxt[8];
  const size_t tstep = static_cast<size_t>(NT) * 32;
#pragma unroll
  for (int u = 0; u < 8; ++u) cur[u] = __ldg(tw + u * tstep);
  if (kts > 8) {
#pragma unroll
    for (int u = 0; u < 8; ++u) nxt[u] = __ldg(tw + (8 + u) * tstep);
  }

  if (early) pdl_wait();
  // ---- prologue: xh = had128(x * suh) / sqrt(128) for this K-slice; one warp per (row, 128-block)
  const __half* suh = a.suh + e * a.suh_stride + k_begin;
  const int nblk = Ks >> 7;
  for (int job = warp; job < R * nblk; job += 8) {
    const int r = job / nblk, b = job - r * nblk;
    const __nv_bfloat16* xr = a.x + static_cast<size_t>(xr0 + r) * a.ldx + k_begin + b * 128 + lane * 4;
    float v[4];
    if (a.act == 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float gg = __bfloat162float(xr[i]), uu = __bfloat162float(xr[a.K + i]);
        if (a.limit > 0.f) { gg = fminf(gg, a.limit); uu = fminf(fmaxf(uu, -a.limit), a.limit); }
        v[i] = gg / (1.f + __expf(-gg)) * uu;
      }
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(xr);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
      v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
    }
    const uint2 sraw = *reinterpret_cast<const uint2*>(suh + b * 128 + lane * 4);
    const __half2* sp = reinterpret_cast<const __half2*>(&sraw);
    const float2 s0 = __half22float2(sp[0]), s1 = __half22float2(sp[1]);
    v[0] *= s0.x; v[1] *= s0.y; v[2] *= s1.x; v[3] *= s1.y;
    fwht128_warp(v, lane);
    __half2 h0 = __floats2half2_rn(v[0] * INV_SQRT_128, v[1] * INV_SQRT_128);
    __half2 h1 = __floats2half2_rn(v[2] * INV_SQRT_128, v[3] * INV_SQRT_128);
    uint2 o; o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(xh + r * ldh + b * 128 + lane * 4) = o;
  }
  if (R < 16) {            // the zero row read by lanes without an activation row
    for (int i = threadIdx.x; i < (Ks >> 1); i += blockDim.x) reinterpret_cast<uint32_t*>(xh + R * ldh)[i] = 0u;
  }
  __syncthreads();

  // ---- main loop.  Lanes whose activation row does not exist read a zeroed row, so the loop has no selects.
  float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
  const bool lo_row = g < R, hi_row = (g + 8) < R;
  const __half* row_lo = xh + (lo_row ? g : R) * ldh + 2 * t;
  const __half* row_hi = xh + (hi_row ? g + 8 : R) * ldh + 2 * t;
#pragma unroll 1
  for (int kb = 0; kb < kts; kb += 8) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t prev = __shfl_sync(0xffffffffu, cur[u], (lane + 31) & 31);
      uint32_t w[4];
      exl3_decode8_b4<CB>(cur[u], prev, w);
      uint32_t af[4];
      af[0] = *reinterpret_cast<const uint32_t*>(row_lo + (kb + u) * 16);
      af[2] = *reinterpret_cast<const uint32_t*>(row_lo + (kb + u) * 16 + 8);
      if (HI) {
        af[1] = *reinterpret_cast<const uint32_t*>(row_hi + (kb + u) * 16);
        af[3] = *reinterpret_cast<const uint32_t*>(row_hi + (kb + u) * 16 + 8);
      } else {
        af[1] = 0u; af[3] = 0u;
      }
      mma_f16_16816(d0, af, w[0], w[1]);       // columns 0..7 of the n-tile
      mma_f16_16816(d1, af, w[2], w[3]);       // columns 8..15
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) cur[u] = nxt[u];
    if (kb + 16 < kts) {
#pragma unroll
      for (int u = 0; u < 8; ++u) nxt[u] = __ldg(tw + (kb + 16 + u) * tstep);
    }
  }
  // This CTA's weight stream is done: let the next kernel's CTAs start (they issue their own weight loads while this
  // grid reduces and stores).  Triggering earlier only makes the two kernels' loads compete (measured: slower).
  pdl_trigger();
  // ---- every CTA pushes its partial strip into the shared memory of cluster rank 0 (plain remote stores,
  //      no round trip), one cluster barrier, then rank 0 sums the slices in rank order:
  //      y = had128(sum) * svh.
  {
    if (a.S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    float* dst = (a.S > 1 ? cluster.map_shared_rank(red, 0) : red) + static_cast<size_t>(slice) * R * 128;
    const int c = warp * 16 + 2 * t;
    if (lo_row) {
      *reinterpret_cast<float2*>(dst + g * 128 + c) = make_float2(d0[0], d0[1]);
      *reinterpret_cast<float2*>(dst + g * 128 + c + 8) = make_float2(d1[0], d1[1]);
    }
    if (hi_row) {
      *reinterpret_cast<float2*>(dst + (g + 8) * 128 + c) = make_float2(d0[2], d0[3]);
      *reinterpret_cast<float2*>(dst + (g + 8) * 128 + c + 8) = make_float2(d1[2], d1[3]);
    }
  }
  if (a.S > 1) cluster.sync(); else __syncthreads();
  if (slice != 0) return;
  const __half* svh = a.svh + e * a.svh_stride + strip * 128;
  for (int r = warp; r < R; r += 8) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < a.S; ++s) {
      const float4 p = *reinterpret_cast<const float4*>(red + (static_cast<size_t>(s) * R + r) * 128 + lane * 4);
      v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
    }
    fwht128_warp(v, lane);
    const uint2 sraw = *reinterpret_cast<const uint2*>(svh + lane * 4);
    const __half2* sp = reinterpret_cast<const __half2*>(&sraw);
    const float2 s0 = __half22float2(sp[0]), s1 = __half22float2(sp[1]);
    v[0] *= INV_SQRT_128 * s0.x; v[1] *= INV_SQRT_128 * s0.y; v[2] *= INV_SQRT_128 * s1.x; v[3] *= INV_SQRT_128 * s1.y;
    if (a.fuse_ar) {
      // fused all-reduce: this rank's partial strip goes straight into slot[rank] of every peer's arena
      const uint32_t ar_seq = comm_seq(a.ar.seq_ptr, a.ar.seq);
      if (a.ar.ll_off >= 0) {                     // decode rows: {value, sequence} words, the tail polls the data itself
        for (int p = 0; p < a.ar.c.world; ++p) {
          uint4* dst = ll_slot(a.ar.c.peers[p], a.ar.ll_off, ar_seq, a.ar.c.world, a.ar.c.rank, r, a.ar.N, strip * 128 + lane * 4);
          st_ll(dst, v[0], v[1], ar_seq);
          st_ll(dst + 1, v[2], v[3], ar_seq);
        }
        continue;
      }
      const size_t so = static_cast<size_t>(ar_seq & 1) * a.ar.c.world * a.ar.rows_cap * a.ar.N +
                        (static_cast<size_t>(a.ar.c.rank) * a.ar.rows_cap + r) * a.ar.N + strip * 128 + lane * 4;
      for (int p = 0; p < a.ar.c.world; ++p)
        st_f4(reinterpret_cast<float*>(a.ar.c.peers[p] + a.ar.slot_off) + so, make_float4(v[0], v[1], v[2], v[3]));
      continue;
    }
    const size_t o = static_cast<size_t>(item * R + r) * a.ldy + strip * 128 + lane * 4;
    if (a.out_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + o) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      __nv_bfloat162 b0 = __floats2bfloat162_rn(v[0], v[1]), b1 = __floats2bfloat162_rn(v[2], v[3]);
      uint2 ov; ov.x = *reinterpret_cast<uint32_t*>(&b0); ov.y = *reinterpret_cast<uint32_t*>(&b1);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.y) + o) = ov;
    }
  }
  if (a.fuse_ar && a.ar.ll_off < 0) exl3_fused_ar_arrive(a);
}

}  // namespace spark

using namespace spark;

// rows_per_item <= 16; K, N multiples of 128; S in 1..8 with (K/128) % S == 0 and K/S <= 2048.
// codebook: 0 mul1, 1 mcg.  ldx, ldy multiples of 4 elements.
extern "C" int spark_exl3_gemv(const void* x, int ldx, const void* trellis, const void* suh, const void* svh,
                               long long t_stride_words, long long suh_stride, long long svh_stride, void* y, int ldy,
                               int out_f32, const int* pair_expert, const int* pair_row, int items, int rows_per_item,
                               int K, int N, int S, int act, float limit, int codebook, cudaStream_t s, const void* ar_args,
                               int pairs_early) {
  if (items <= 0 || rows_per_item <= 0) return 0;
  if (rows_per_item > 16 || (K & 127) || (N & 127) || S < 1 || S > 8 || ((K >> 7) % S) || K / S > EXL3_MAX_KS) return -5;
  if ((ldx & 3) || (ldy & 3)) return -5;
  Exl3GemvArgs a;
  a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.trellis = (const uint32_t*)trellis;
  a.suh = (const __half*)suh; a.svh = (const __half*)svh;
  a.t_stride = t_stride_words; a.suh_stride = suh_stride; a.svh_stride = svh_stride;
  a.y = y; a.ldy = ldy; a.out_f32 = out_f32;
  a.pair_expert = pair_expert; a.pair_row = pair_row;
  a.R = rows_per_item; a.K = K; a.N = N; a.S = S; a.act = act; a.limit = limit;
  a.fuse_ar = 0;
  a.pairs_early = pairs_early;
  if (ar_args) {
    if (items != 1) return -5;
    a.fuse_ar = 1;
    a.ar = *static_cast<const ArRows*>(ar_args);
  }
  const size_t smem_bytes = 16 * (K / S + 8) * 2 + S * rows_per_item * 128 * 4;
  const bool hi = rows_per_item > 8;
  void (*kern)(Exl3GemvArgs) = codebook == 0 ? (hi ? exl3_gemv_kernel<0, true> : exl3_gemv_kernel<0, false>)
                                             : (hi ? exl3_gemv_kernel<1, true> : exl3_gemv_kernel<1, false>);
  {
    static bool done[4] = {false, false, false, false};
    const int id = (codebook ? 2 : 0) + (hi ? 1 : 0);
    if (!done[id]) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * (EXL3_MAX_KS + 8) * 2 + 8 * 16 * 128 * 4);
      done[id] = true;
    }
  }
  cudaError_t err = spark_launch_pdl(kern, dim3(N / 128, S, items), dim3(256), smem_bytes, s, dim3(1, S, 1), a);
  return err == cudaSuccess ? 0 : -4;
}
