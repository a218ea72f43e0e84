// Gated-DeltaNet prefill in chunked (WY) form: 64-token chunks, all matrix work on tensor cores (tf32 MMA, fp32
// accumulate), the state carried through a short sequential pass.
//
// Per value head, with d_t = exp(g_t), D_t = prod_{j<=t} d_j inside a chunk, S0 the state entering the chunk
// (S is [Dv, Dk]; row i is what one thread of the sequential kernel owns):
//     u_t = beta_t (v_t - d_t S_{t-1} k_t),   S_t = d_t S_{t-1} + u_t k_t^T,   o_t = S_t q_t
// unrolls to
//     (I + A) U = diag(beta) V - diag(beta D) K S0^T,     A_tj = beta_t (D_t/D_j) (k_t.k_j)  (j < t)
//     O = diag(D) Q S0^T + P U,                           P_tj = (D_t/D_j) (q_t.k_j)         (j <= t)
//     S_C = D_C S0 + U^T diag(D_C / D) K
// so with T = (I + A)^-1 everything that does not involve S0 is computed for all chunks in parallel:
//   kernel 1 (chunk, head):  conv(k=4)+SiLU, L2 norms, gates;  K K^T, Q K^T -> A, P;  T by forward substitution;
//                            W = T diag(beta D) K,  Ut = T diag(beta) V,  Qt = diag(D) Q,  Kt = diag(D_C/D) K
//   kernel 2 (v-slice, head, segment), sequential over the chunks of one sequence, S kept in registers:
//                            U = Ut - W S0^T;  O = Qt S0^T + P U;  S <- D_C S + U^T Kt
//                            (the Dv rows of S are independent, so a head is split over 4 CTAs of 32 rows)
//   kernel 3 (chunk, head):  RMSNorm(o) * w * sigmoid(z) -> bf16
// All decay ratios are exp() of non-positive numbers: nothing can overflow.  Operands are rounded to tf32
// (10-bit mantissa) once, when they are written; sums are fp32.  Decode and verify rows keep using the
// sequential kernel (bitwise chained == one-pass there); this path serves committed segments of >= 64 rows.
// Reference: engine-rs/shim/qwen_gdn.cu rows_kernel / rows4_kernel (sequential over rows, 4 rows per step).
#include "../common/ptx.cuh"

namespace spark {

constexpr int GC = 64;            // chunk length
constexpr int GD = 128;           // head dim (k and v)
constexpr int LD128 = 136;        // smem row stride of 128-wide arrays (8 mod 32: conflict-free fragment loads)
constexpr int LD64 = 72;
constexpr int LD32 = 40;
constexpr int GVS = 32;           // value rows of S per CTA in the state pass
// workspace per (chunk, head), floats
constexpr int WS_W = 0, WS_UT = GC * GD, WS_QT = 2 * GC * GD, WS_KT = 3 * GC * GD, WS_P = 4 * GC * GD,
              WS_DC = 4 * GC * GD + GC * GC, WS_STRIDE = 4 * GC * GD + GC * GC + 64;

__device__ __forceinline__ float tf32r(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], float a0, float a1, float a2, float a3, float b0, float b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)), "r"(__float_as_uint(a2)), "r"(__float_as_uint(a3)),
                 "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- kernel 1
// grid (chunks, Hv); 256 threads
__global__ void __launch_bounds__(256)
gdn_chunk_prep_kernel(const __nv_bfloat16* __restrict__ proj, int ldp, const __nv_bfloat16* __restrict__ ab, int ldab,
                      const float* __restrict__ conv_w, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                      const float* __restrict__ tail, const int* __restrict__ seg, const int* __restrict__ chunks,
                      float* __restrict__ ws, int Hk, int Hv, float eps) {
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                          // [64][136]
  float* Ks = Qs + GC * LD128;
  float* Vs = Ks + GC * LD128;
  float* As = Vs + GC * LD128;             // [64][72]   A, later T diag(beta D)
  float* Ts = As + GC * LD64;              // [64][72]   T, later T diag(beta)
  float* beta_s = Ts + GC * LD64;          // [64]
  float* G_s = beta_s + GC;                // [64] cumulative log decay
  const int ci = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sg = chunks[2 * ci], c = chunks[2 * ci + 1];
  const int slot = seg[sg * 4], r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2];
  const int t0 = c * GC, nv = min(GC, n - t0);
  const int hk = h / (Hv / Hk);
  float* wsb = ws + (static_cast<size_t>(ci) * Hv + h) * WS_STRIDE;

  // ---- conv + SiLU + L2 norms: warp w owns rows 8w..8w+7 (sliding window), lane owns channels lane+32cc
  {
    const float* tl = tail + (static_cast<size_t>(slot) * 3 * Hv + h) * 3 * GD;
    const float qscale = rsqrtf(static_cast<float>(GD));
    float hq[4][3], hk_[4][3], hv[4][3], wq[4][4], wk[4][4], wv[4][4];
    int chq[4], chk[4], chv[4];
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int i = lane + 32 * cc;
      chq[cc] = hk * GD + i; chk[cc] = Hk * GD + hk * GD + i; chv[cc] = 2 * Hk * GD + h * GD + i;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        wq[cc][j] = conv_w[chq[cc] * 4 + j]; wk[cc][j] = conv_w[chk[cc] * 4 + j]; wv[cc][j] = conv_w[chv[cc] * 4 + j];
      }
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int p = t0 + warp * 8 - 3 + j;            // position in the segment of history entry j
        if (p < 0) {
          const float* t = tl + static_cast<size_t>(p + 3) * Hv * 3 * GD;
          hq[cc][j] = t[i]; hk_[cc][j] = t[GD + i]; hv[cc][j] = t[2 * GD + i];
        } else if (p < n) {
          const __nv_bfloat16* pr = proj + static_cast<size_t>(r0 + p) * ldp;
          hq[cc][j] = __bfloat162float(pr[chq[cc]]); hk_[cc][j] = __bfloat162float(pr[chk[cc]]);
          hv[cc][j] = __bfloat162float(pr[chv[cc]]);
        } else { hq[cc][j] = 0.f; hk_[cc][j] = 0.f; hv[cc][j] = 0.f; }
      }
    }
    for (int rr = 0; rr < 8; ++rr) {
      const int r = warp * 8 + rr;
      float q[4], k[4], v[4], q2 = 0.f, k2 = 0.f;
      if (r < nv) {
        const __nv_bfloat16* pr = proj + static_cast<size_t>(r0 + t0 + r) * ldp;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const float xq = __bfloat162float(pr[chq[cc]]), xk = __bfloat162float(pr[chk[cc]]), xv = __bfloat162float(pr[chv[cc]]);
          q[cc] = silu(hq[cc][0] * wq[cc][0] + hq[cc][1] * wq[cc][1] + hq[cc][2] * wq[cc][2] + xq * wq[cc][3]);
          k[cc] = silu(hk_[cc][0] * wk[cc][0] + hk_[cc][1] * wk[cc][1] + hk_[cc][2] * wk[cc][2] + xk * wk[cc][3]);
          v[cc] = silu(hv[cc][0] * wv[cc][0] + hv[cc][1] * wv[cc][1] + hv[cc][2] * wv[cc][2] + xv * wv[cc][3]);
          hq[cc][0] = hq[cc][1]; hq[cc][1] = hq[cc][2]; hq[cc][2] = xq;
          hk_[cc][0] = hk_[cc][1]; hk_[cc][1] = hk_[cc][2]; hk_[cc][2] = xk;
          hv[cc][0] = hv[cc][1]; hv[cc][1] = hv[cc][2]; hv[cc][2] = xv;
          q2 = fmaf(q[cc], q[cc], q2); k2 = fmaf(k[cc], k[cc], k2);
        }
        q2 = warp_sum(q2); k2 = warp_sum(k2);
        const float qn = rsqrtf(q2 + eps) * qscale, kn = rsqrtf(k2 + eps);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) { q[cc] *= qn; k[cc] *= kn; }
      } else {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) { q[cc] = 0.f; k[cc] = 0.f; v[cc] = 0.f; }
      }
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int i = lane + 32 * cc;
        Qs[r * LD128 + i] = tf32r(q[cc]); Ks[r * LD128 + i] = tf32r(k[cc]); Vs[r * LD128 + i] = tf32r(v[cc]);
      }
    }
  }
  if (tid < GC) {
    float beta = 0.f, lg = 0.f;
    if (tid < nv) {
      const float bl = __bfloat162float(ab[static_cast<size_t>(r0 + t0 + tid) * ldab + h]);
      const float al = __bfloat162float(ab[static_cast<size_t>(r0 + t0 + tid) * ldab + Hv + h]);
      beta = 1.f / (1.f + __expf(-bl));
      const float xa = al + dt_bias[h];
      const float sp = xa > 20.f ? xa : log1pf(__expf(xa));
      lg = -__expf(A_log[h]) * sp;
    }
    beta_s[tid] = beta;
    G_s[tid] = lg;
  }
  __syncthreads();
  {                                                  // inclusive prefix sum of the log decays
    float gsum = 0.f;
    if (tid < GC)
      for (int j = 0; j <= tid; ++j) gsum += G_s[j];
    __syncthreads();
    if (tid < GC) G_s[tid] = gsum;
    __syncthreads();
  }

  const int g = lane >> 2, t = lane & 3;
  // ---- K K^T and Q K^T (lower triangle only): warp -> m-tile (warp&3), n-tiles 4*(warp>>2) .. +4
  {
    const int mt = warp & 3, nt0 = (warp >> 2) * 4;
    float ckk[4][4], cqk[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) { ckk[a][b] = 0.f; cqk[a][b] = 0.f; }
    const float* ka = Ks + (mt * 16 + g) * LD128 + t;
    const float* qa = Qs + (mt * 16 + g) * LD128 + t;
    for (int ks = 0; ks < GD / 8; ++ks) {
      const float k0 = ka[ks * 8], k1 = ka[8 * LD128 + ks * 8], k2 = ka[ks * 8 + 4], k3 = ka[8 * LD128 + ks * 8 + 4];
      const float q0 = qa[ks * 8], q1 = qa[8 * LD128 + ks * 8], q2 = qa[ks * 8 + 4], q3 = qa[8 * LD128 + ks * 8 + 4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int nt = nt0 + a;
        if (nt * 8 > mt * 16 + 15) continue;                      // strictly above the diagonal
        const float* kb = Ks + (nt * 8 + g) * LD128 + ks * 8 + t;
        const float b0 = kb[0], b1 = kb[4];
        mma_tf32(ckk[a], k0, k1, k2, k3, b0, b1);
        mma_tf32(cqk[a], q0, q1, q2, q3, b0, b1);
      }
    }
    float* Pg = wsb + WS_P;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int nt = nt0 + a;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = mt * 16 + g + (e >> 1) * 8, col = nt * 8 + 2 * t + (e & 1);
        float av = 0.f, pv = 0.f;
        if (col <= row) {
          const float dec = __expf(G_s[row] - G_s[col]);
          pv = dec * cqk[a][e];
          if (col < row) av = beta_s[row] * dec * ckk[a][e];
        }
        As[row * LD64 + col] = av;
        Pg[row * GC + col] = tf32r(pv);
      }
    }
  }
  __syncthreads();
  // ---- T = (I + A)^-1: thread c owns column c (forward substitution, column in registers)
  if (tid < GC) {
    float tc[GC];
#pragma unroll
    for (int i = 0; i < GC; ++i) {
      float s = (i == tid) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s = fmaf(-As[i * LD64 + j], tc[j], s);
      tc[i] = s;
    }
#pragma unroll
    for (int i = 0; i < GC; ++i) Ts[i * LD64 + tid] = tc[i];
  }
  __syncthreads();
  // As <- T diag(beta D), Ts <- T diag(beta)
  for (int idx = tid; idx < GC * GC; idx += 256) {
    const int i = idx >> 6, j = idx & 63;
    const float tv = Ts[i * LD64 + j];
    As[i * LD64 + j] = tf32r(tv * beta_s[j] * __expf(G_s[j]));
    Ts[i * LD64 + j] = tf32r(tv * beta_s[j]);
  }
  __syncthreads();
  // ---- W = As K, Ut = Ts V: warp -> m-tile (warp&3), n-tiles 8*(warp>>2) .. +8; k-steps up to the diagonal
  {
    const int mt = warp & 3, nt0 = (warp >> 2) * 8;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const float* Am = which == 0 ? As : Ts;
      const float* Bm = which == 0 ? Ks : Vs;
      float acc[8][4];
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
      const float* aa = Am + (mt * 16 + g) * LD64 + t;
      for (int ks = 0; ks < 2 * (mt + 1); ++ks) {
        const float a0 = aa[ks * 8], a1 = aa[8 * LD64 + ks * 8], a2 = aa[ks * 8 + 4], a3 = aa[8 * LD64 + ks * 8 + 4];
#pragma unroll
        for (int a = 0; a < 8; ++a) {
          const float* bb = Bm + (ks * 8 + t) * LD128 + (nt0 + a) * 8 + g;
          mma_tf32(acc[a], a0, a1, a2, a3, bb[0], bb[4 * LD128]);
        }
      }
      float* Og = wsb + (which == 0 ? WS_W : WS_UT);
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        const int col = (nt0 + a) * 8 + 2 * t, row = mt * 16 + g;
        float2 lo = make_float2(acc[a][0], acc[a][1]), hi = make_float2(acc[a][2], acc[a][3]);
        if (which == 0) { lo.x = tf32r(lo.x); lo.y = tf32r(lo.y); hi.x = tf32r(hi.x); hi.y = tf32r(hi.y); }
        *reinterpret_cast<float2*>(Og + row * GD + col) = lo;
        *reinterpret_cast<float2*>(Og + (row + 8) * GD + col) = hi;
      }
    }
  }
  // ---- Qt = diag(D) Q, Kt = diag(D_C / D) K
  const float Gl = G_s[GC - 1];
  for (int idx = tid; idx < GC * GD; idx += 256) {
    const int r = idx >> 7, i = idx & 127;
    wsb[WS_QT + idx] = tf32r(Qs[r * LD128 + i] * __expf(G_s[r]));
    wsb[WS_KT + idx] = tf32r(Ks[r * LD128 + i] * __expf(Gl - G_s[r]));
  }
  if (tid == 0) wsb[WS_DC] = __expf(Gl);
}

// ---------------------------------------------------------------------------------------------- kernel 2
// grid (4, Hv, nseg); 128 threads; sequential over the chunks of one segment
__global__ void __launch_bounds__(128)
gdn_chunk_state_kernel(const float* __restrict__ ws, const int* __restrict__ seg, const int* __restrict__ seg_chunk0,
                       const __nv_bfloat16* __restrict__ proj, int ldp, float* __restrict__ S, float* __restrict__ tail,
                       float* __restrict__ o_raw, int ldo, int Hk, int Hv) {
  extern __shared__ __align__(16) float sm[];
  float* Wsm = sm;                          // [64][136]
  float* Qsm = Wsm + GC * LD128;
  float* Ksm = Qsm + GC * LD128;
  float* Psm = Ksm + GC * LD128;            // [64][72]
  float* Usm = Psm + GC * LD64;             // [64][40]  Ut, then U
  float* Ssm = Usm + GC * LD32;             // [32][136]
  const int vs = blockIdx.x, h = blockIdx.y, sg = blockIdx.z;
  const int ci0 = seg_chunk0[sg];
  if (ci0 < 0) return;
  const int slot = seg[sg * 4], r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2];
  const int nch = (n + GC - 1) / GC;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int v0 = vs * GVS;
  // S accumulator fragments: warp -> v rows 16*(warp&1).., k columns 64*(warp>>1)..
  const int smt = warp & 1, sng = warp >> 1;
  float sacc[8][4];
  float* Sg = S + ((static_cast<size_t>(slot) * Hv + h) * GD + v0) * GD;
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int col = sng * 64 + a * 8 + 2 * t, row = smt * 16 + g;
    const float2 lo = *reinterpret_cast<const float2*>(Sg + row * GD + col);
    const float2 hi = *reinterpret_cast<const float2*>(Sg + (row + 8) * GD + col);
    sacc[a][0] = lo.x; sacc[a][1] = lo.y; sacc[a][2] = hi.x; sacc[a][3] = hi.y;
    Ssm[row * LD128 + col] = tf32r(lo.x); Ssm[row * LD128 + col + 1] = tf32r(lo.y);
    Ssm[(row + 8) * LD128 + col] = tf32r(hi.x); Ssm[(row + 8) * LD128 + col + 1] = tf32r(hi.y);
  }
  for (int c = 0; c < nch; ++c) {
    const float* wsb = ws + (static_cast<size_t>(ci0 + c) * Hv + h) * WS_STRIDE;
    // ---- stage this chunk's operands
    for (int idx = tid; idx < GC * GD / 4; idx += 128) {
      const int r = idx >> 5, c4 = (idx & 31) * 4;
      cp_async16(Wsm + r * LD128 + c4, wsb + WS_W + r * GD + c4);
      cp_async16(Qsm + r * LD128 + c4, wsb + WS_QT + r * GD + c4);
      cp_async16(Ksm + r * LD128 + c4, wsb + WS_KT + r * GD + c4);
    }
    for (int idx = tid; idx < GC * GC / 4; idx += 128) {
      const int r = idx >> 4, c4 = (idx & 15) * 4;
      cp_async16(Psm + r * LD64 + c4, wsb + WS_P + r * GC + c4);
    }
    for (int idx = tid; idx < GC * GVS / 4; idx += 128) {
      const int r = idx >> 3, c4 = (idx & 7) * 4;
      cp_async16(Usm + r * LD32 + c4, wsb + WS_UT + r * GD + v0 + c4);
    }
    cp_async_wait_all();
    __syncthreads();
    const float dc = wsb[WS_DC];
    // ---- X = W S0^T and O = Qt S0^T: warp -> token rows 16*warp.., 4 n-tiles (32 v columns), 16 k-steps
    float xacc[4][4], oacc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) { xacc[a][b] = 0.f; oacc[a][b] = 0.f; }
    {
      const float* wa = Wsm + (warp * 16 + g) * LD128 + t;
      const float* qa = Qsm + (warp * 16 + g) * LD128 + t;
#pragma unroll 4
      for (int ks = 0; ks < GD / 8; ++ks) {
        const float w0 = wa[ks * 8], w1 = wa[8 * LD128 + ks * 8], w2 = wa[ks * 8 + 4], w3 = wa[8 * LD128 + ks * 8 + 4];
        const float q0 = qa[ks * 8], q1 = qa[8 * LD128 + ks * 8], q2 = qa[ks * 8 + 4], q3 = qa[8 * LD128 + ks * 8 + 4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float* sb = Ssm + (a * 8 + g) * LD128 + ks * 8 + t;
          const float b0 = sb[0], b1 = sb[4];
          mma_tf32(xacc[a], w0, w1, w2, w3, b0, b1);
          mma_tf32(oacc[a], q0, q1, q2, q3, b0, b1);
        }
      }
    }
    // ---- U = Ut - X (each element is read and written by the same thread)
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int col = a * 8 + 2 * t, row = warp * 16 + g;
      float* u0 = Usm + row * LD32 + col;
      float* u1 = Usm + (row + 8) * LD32 + col;
      u0[0] = tf32r(u0[0] - xacc[a][0]); u0[1] = tf32r(u0[1] - xacc[a][1]);
      u1[0] = tf32r(u1[0] - xacc[a][2]); u1[1] = tf32r(u1[1] - xacc[a][3]);
    }
    __syncthreads();
    // ---- O += P U (P is lower triangular: k-steps up to this warp's diagonal block)
    {
      const float* pa = Psm + (warp * 16 + g) * LD64 + t;
      for (int ks = 0; ks < 2 * (warp + 1); ++ks) {
        const float p0 = pa[ks * 8], p1 = pa[8 * LD64 + ks * 8], p2 = pa[ks * 8 + 4], p3 = pa[8 * LD64 + ks * 8 + 4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float* ub = Usm + (ks * 8 + t) * LD32 + a * 8 + g;
          mma_tf32(oacc[a], p0, p1, p2, p3, ub[0], ub[4 * LD32]);
        }
      }
      const int nvr = min(GC, n - c * GC);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int col = h * GD + v0 + a * 8 + 2 * t, row = warp * 16 + g;
        if (row < nvr)
          *reinterpret_cast<float2*>(o_raw + static_cast<size_t>(r0 + c * GC + row) * ldo + col) = make_float2(oacc[a][0], oacc[a][1]);
        if (row + 8 < nvr)
          *reinterpret_cast<float2*>(o_raw + static_cast<size_t>(r0 + c * GC + row + 8) * ldo + col) = make_float2(oacc[a][2], oacc[a][3]);
      }
    }
    // ---- S <- D_C S + U^T Kt: A[m = v][k = j] = U[j][v], B[k = j][n] = Kt[j][n]
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) sacc[a][b] *= dc;
    for (int ks = 0; ks < GC / 8; ++ks) {
      const float* ua = Usm + (ks * 8 + t) * LD32 + smt * 16 + g;
      const float a0 = ua[0], a1 = ua[8], a2 = ua[4 * LD32], a3 = ua[4 * LD32 + 8];
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        const float* kb = Ksm + (ks * 8 + t) * LD128 + sng * 64 + a * 8 + g;
        mma_tf32(sacc[a], a0, a1, a2, a3, kb[0], kb[4 * LD128]);
      }
    }
    __syncthreads();            // every warp is done with the old S and with this chunk's operands
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int col = sng * 64 + a * 8 + 2 * t, row = smt * 16 + g;
      Ssm[row * LD128 + col] = tf32r(sacc[a][0]); Ssm[row * LD128 + col + 1] = tf32r(sacc[a][1]);
      Ssm[(row + 8) * LD128 + col] = tf32r(sacc[a][2]); Ssm[(row + 8) * LD128 + col + 1] = tf32r(sacc[a][3]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int col = sng * 64 + a * 8 + 2 * t, row = smt * 16 + g;
    *reinterpret_cast<float2*>(Sg + row * GD + col) = make_float2(sacc[a][0], sacc[a][1]);
    *reinterpret_cast<float2*>(Sg + (row + 8) * GD + col) = make_float2(sacc[a][2], sacc[a][3]);
  }
  if (vs == 0) {          // conv history for the next call: raw inputs of the last three positions
    const int hk = h / (Hv / Hk), i = tid;
    float* tl = tail + (static_cast<size_t>(slot) * 3 * Hv + h) * 3 * GD;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const __nv_bfloat16* pr = proj + static_cast<size_t>(r0 + n - 3 + j) * ldp;
      float* tj = tl + static_cast<size_t>(j) * Hv * 3 * GD;
      tj[i] = __bfloat162float(pr[hk * GD + i]);
      tj[GD + i] = __bfloat162float(pr[Hk * GD + hk * GD + i]);
      tj[2 * GD + i] = __bfloat162float(pr[2 * Hk * GD + h * GD + i]);
    }
  }
}

// ---------------------------------------------------------------------------------------------- kernel 3
// grid (chunks, Hv); 256 threads: warp w -> rows 8w..8w+7 of the chunk
__global__ void __launch_bounds__(256)
gdn_chunk_out_kernel(const float* __restrict__ o_raw, int ldo, const __nv_bfloat16* __restrict__ proj, int ldp,
                     const float* __restrict__ norm_w, const int* __restrict__ seg, const int* __restrict__ chunks,
                     __nv_bfloat16* __restrict__ out, int ldout, int Hk, int Hv, float eps) {
  const int ci = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sg = chunks[2 * ci], c = chunks[2 * ci + 1];
  const int r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2];
  const int zc = 2 * Hk * GD + Hv * GD + h * GD + lane * 4;
  const float4 nw = *reinterpret_cast<const float4*>(norm_w + lane * 4);
  for (int rr = 0; rr < 8; ++rr) {
    const int tt = c * GC + warp * 8 + rr;
    if (tt >= n) break;
    const size_t row = static_cast<size_t>(r0 + tt);
    const float4 o = *reinterpret_cast<const float4*>(o_raw + row * ldo + h * GD + lane * 4);
    const float o2 = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
    const float rs = rsqrtf(o2 / GD + eps);
    const uint2 zr = *reinterpret_cast<const uint2*>(proj + row * ldp + zc);
    const float2 z0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&zr.x));
    const float2 z1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&zr.y));
    const __nv_bfloat162 b0 = __floats2bfloat162_rn(o.x * rs * nw.x / (1.f + __expf(-z0.x)), o.y * rs * nw.y / (1.f + __expf(-z0.y)));
    const __nv_bfloat162 b1 = __floats2bfloat162_rn(o.z * rs * nw.z / (1.f + __expf(-z1.x)), o.w * rs * nw.w / (1.f + __expf(-z1.y)));
    uint2 ov; ov.x = *reinterpret_cast<const uint32_t*>(&b0); ov.y = *reinterpret_cast<const uint32_t*>(&b1);
    *reinterpret_cast<uint2*>(out + row * ldout + h * GD + lane * 4) = ov;
  }
}

}  // namespace spark

using namespace spark;

extern "C" long long spark_gdn_chunk_ws_floats(int n_chunks, int Hv) {
  return static_cast<long long>(n_chunks) * Hv * WS_STRIDE;
}

// chunks: int [n_chunks][2] = (segment, chunk in segment); seg_chunk0: int [nseg] first chunk of a segment or -1
// (segment not served here).  head_dim must be 128; o_raw fp32 [R, Hv*128]; ws from spark_gdn_chunk_ws_floats.
extern "C" int spark_gdn_chunk_prefill(const void* proj, int ldp, const void* ab, int ldab, const float* conv_w,
                                       const float* A_log, const float* dt_bias, const float* norm_w, float* S, float* tail,
                                       const int* seg, int nseg, const int* chunks, int n_chunks, const int* seg_chunk0,
                                       float* ws, float* o_raw, void* out, int ldo, int Hk, int Hv, int D, float eps,
                                       cudaStream_t s) {
  if (n_chunks <= 0) return 0;
  if (D != GD || Hv % Hk) return -5;
  constexpr int SM1 = (3 * GC * LD128 + 2 * GC * LD64 + 2 * GC) * 4;
  constexpr int SM2 = (3 * GC * LD128 + GC * LD64 + GC * LD32 + GVS * LD128) * 4;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM1);
    cudaFuncSetAttribute(gdn_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM2);
    attr = true;
  }
  gdn_chunk_prep_kernel<<<dim3(n_chunks, Hv), 256, SM1, s>>>((const __nv_bfloat16*)proj, ldp, (const __nv_bfloat16*)ab, ldab,
                                                              conv_w, A_log, dt_bias, tail, seg, chunks, ws, Hk, Hv, eps);
  gdn_chunk_state_kernel<<<dim3(GD / GVS, Hv, nseg), 128, SM2, s>>>(ws, seg, seg_chunk0, (const __nv_bfloat16*)proj, ldp, S,
                                                                    tail, o_raw, Hv * GD, Hk, Hv);
  gdn_chunk_out_kernel<<<dim3(n_chunks, Hv), 256, 0, s>>>(o_raw, Hv * GD, (const __nv_bfloat16*)proj, ldp, norm_w, seg, chunks,
                                                          (__nv_bfloat16*)out, ldo, Hk, Hv, eps);
  return spark_launch_rc(__func__);
}
