// Kimi-delta-attention prefill in chunked form: 16-token chunks, per-channel decay, matrix work on tensor cores
// (tf32 MMA, fp32 accumulate), the state carried through a short sequential pass.
//
// Per head, with the per-channel decay d_t = exp(lam_t) in R^Dk, G_t = sum_{j<=t} lam_j inside a chunk and S0 the state
// entering the chunk (S is [Dv, Dk]):
//     u_t = beta_t (v_t - S_{t-1} diag(d_t) k_t),   S_t = S_{t-1} diag(d_t) + u_t k_t^T,   o_t = S_t q_t
// unrolls, with K+ = K.exp(G), K- = K.exp(-G), Q+ = Q.exp(G), to
//     (I + A) U = diag(beta) V - diag(beta) K+ S0^T,     A_tj = beta_t (K+_t . K-_j)  (j < t)
//     O = Q+ S0^T + P U,                                 P_tj = Q+_t . K-_j           (j <= t)
//     S_C = S0 diag(exp(G_C)) + U^T (K- . exp(G_C))
// The log decay of one step lies in (-5, 0) by construction (lam = -5 sigmoid(..)), so over 16 steps |G| < 80 and
// exp(-G) stays inside fp32: that is why the chunk is 16 tokens long here (64 in the scalar-decay kernel).
//   kernel 1 (chunk, head):  conv(k=4)+SiLU, L2 norms, gates and their prefix sums; K+ K-^T, Q+ K-^T -> A, P; T = (I+A)^-1;
//                            W = T diag(beta) K+,  Ut = T diag(beta) V,  Qt = Q+,  Kt = K- . exp(G_C),  Dc = exp(G_C)
//   kernel 2 (v-slice, head, segment), sequential over chunks, S in registers:
//                            U = Ut - W S0^T;  O = Qt S0^T + P U;  S <- S diag(Dc) + U^T Kt
//   kernel 3 (chunk, head):  o_norm * RMS(o) * sigmoid(g2) -> bf16
// Decode and verify rows keep using the sequential kernel.  Reference: reference/glm53/kda.py:35-77 (math),
// engine-rs/shim/kda.cu recurrent_lane_sequence6 (sequential rows).
#include "../common/ptx.cuh"

namespace spark {

constexpr int KC = 16;            // chunk length
constexpr int KD = 128;           // head dim
constexpr int KLD = 136;          // smem row stride of 128-wide arrays
constexpr int KLC = 24;           // smem row stride of 16-wide arrays (8 mod 16: conflict-free fragment loads)
constexpr int KLV = 40;           // 32-wide arrays
constexpr int KVS = 32;           // value rows of S per CTA in the state pass
// workspace per (chunk, head), floats
constexpr int KW_W = 0, KW_UT = KC * KD, KW_QT = 2 * KC * KD, KW_KT = 3 * KC * KD, KW_P = 4 * KC * KD,
              KW_DC = 4 * KC * KD + KC * KC, KW_STRIDE = 4 * KC * KD + KC * KC + KD;

__device__ __forceinline__ float k_tf32r(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ void k_mma(float (&c)[4], float a0, float a1, float a2, float a3, float b0, float b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)), "r"(__float_as_uint(a2)), "r"(__float_as_uint(a3)),
                 "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}
__device__ __forceinline__ float k_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ void k_cp16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// ---------------------------------------------------------------------------------------------- kernel 1
// grid (chunks, H); 128 threads
__global__ void __launch_bounds__(128)
kda_chunk_prep_kernel(const __nv_bfloat16* __restrict__ pre, int ldp, const float* __restrict__ g1, int ldg,
                      const __nv_bfloat16* __restrict__ lr, int ldl, int beta_off, const float* __restrict__ conv_w,
                      const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ tail,
                      const int* __restrict__ seg, const int* __restrict__ chunks, float* __restrict__ ws, int H) {
  __shared__ float Qs[KC * KLD], Ks[KC * KLD], Vs[KC * KLD], Gs[KC * KLD];   // Q+ | K+ | V | K- (after step 3)
  __shared__ float As[KC * KLC], Ts[KC * KLC], beta_s[KC];
  const int ci = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sg = chunks[2 * ci], c = chunks[2 * ci + 1];
  const int slot = seg[sg * 4], r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2];
  const int t0 = c * KC, nv = min(KC, n - t0);
  const int nn = H * KD;
  float* wsb = ws + (static_cast<size_t>(ci) * H + h) * KW_STRIDE;
  // ---- conv + SiLU + L2 norms: warp w owns rows 4w..4w+3 (sliding window), lane owns channels lane+32cc
  {
    const float* tl = tail + static_cast<size_t>(slot) * 3 * 3 * nn;
    const float qscale = rsqrtf(static_cast<float>(KD));
    float hq[4][3], hk[4][3], hv[4][3], wq[4][4], wk[4][4], wv[4][4];
    int chq[4], chk[4], chv[4];
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int i = lane + 32 * cc;
      chq[cc] = h * KD + i; chk[cc] = nn + h * KD + i; chv[cc] = 2 * nn + h * KD + i;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        wq[cc][j] = conv_w[chq[cc] * 4 + j]; wk[cc][j] = conv_w[chk[cc] * 4 + j]; wv[cc][j] = conv_w[chv[cc] * 4 + j];
      }
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int p = t0 + warp * 4 - 3 + j;
        if (p < 0) {
          const float* t = tl + static_cast<size_t>(p + 3) * 3 * nn;
          hq[cc][j] = t[chq[cc]]; hk[cc][j] = t[chk[cc]]; hv[cc][j] = t[chv[cc]];
        } else if (p < n) {
          const __nv_bfloat16* pr = pre + static_cast<size_t>(r0 + p) * ldp;
          hq[cc][j] = __bfloat162float(pr[chq[cc]]); hk[cc][j] = __bfloat162float(pr[chk[cc]]); hv[cc][j] = __bfloat162float(pr[chv[cc]]);
        } else { hq[cc][j] = 0.f; hk[cc][j] = 0.f; hv[cc][j] = 0.f; }
      }
    }
    for (int rr = 0; rr < 4; ++rr) {
      const int r = warp * 4 + rr;
      float q[4], k[4], v[4], q2 = 0.f, k2 = 0.f;
      if (r < nv) {
        const __nv_bfloat16* pr = pre + static_cast<size_t>(r0 + t0 + r) * ldp;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const float xq = __bfloat162float(pr[chq[cc]]), xk = __bfloat162float(pr[chk[cc]]), xv = __bfloat162float(pr[chv[cc]]);
          q[cc] = k_silu(hq[cc][0] * wq[cc][0] + hq[cc][1] * wq[cc][1] + hq[cc][2] * wq[cc][2] + xq * wq[cc][3]);
          k[cc] = k_silu(hk[cc][0] * wk[cc][0] + hk[cc][1] * wk[cc][1] + hk[cc][2] * wk[cc][2] + xk * wk[cc][3]);
          v[cc] = k_silu(hv[cc][0] * wv[cc][0] + hv[cc][1] * wv[cc][1] + hv[cc][2] * wv[cc][2] + xv * wv[cc][3]);
          hq[cc][0] = hq[cc][1]; hq[cc][1] = hq[cc][2]; hq[cc][2] = xq;
          hk[cc][0] = hk[cc][1]; hk[cc][1] = hk[cc][2]; hk[cc][2] = xk;
          hv[cc][0] = hv[cc][1]; hv[cc][1] = hv[cc][2]; hv[cc][2] = xv;
          q2 = fmaf(q[cc], q[cc], q2); k2 = fmaf(k[cc], k[cc], k2);
        }
        q2 = warp_sum(q2); k2 = warp_sum(k2);
        const float qn = rsqrtf(q2 + 1e-6f) * qscale, kn = rsqrtf(k2 + 1e-6f);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) { q[cc] *= qn; k[cc] *= kn; }
      } else {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) { q[cc] = 0.f; k[cc] = 0.f; v[cc] = 0.f; }
      }
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int i = lane + 32 * cc;
        Qs[r * KLD + i] = q[cc]; Ks[r * KLD + i] = k[cc]; Vs[r * KLD + i] = k_tf32r(v[cc]);
      }
    }
  }
  if (tid < KC) beta_s[tid] = tid < nv ? 1.f / (1.f + __expf(-__bfloat162float(lr[static_cast<size_t>(r0 + t0 + tid) * ldl + beta_off + h]))) : 0.f;
  __syncthreads();
  // ---- per-channel decay: thread = channel; prefix sums over the rows; Q+ = Q e^G, K+ = K e^G, K- = K e^-G
  {
    const int ch = tid;
    const float a_exp = __expf(A_log[h]), dtb = dt_bias[h * KD + ch];
    float G = 0.f;
    for (int r = 0; r < KC; ++r) {
      if (r < nv) G += -5.f / (1.f + __expf(-a_exp * (g1[static_cast<size_t>(r0 + t0 + r) * ldg + h * KD + ch] + dtb)));
      const float ep = __expf(G), em = __expf(-G);
      const float k = Ks[r * KLD + ch];
      Qs[r * KLD + ch] = k_tf32r(Qs[r * KLD + ch] * ep);
      Ks[r * KLD + ch] = k_tf32r(k * ep);
      Gs[r * KLD + ch] = k_tf32r(k * em);
    }
    const float eC = __expf(G);
    wsb[KW_DC + ch] = eC;
    // Qt and Kt rows for the state pass
    for (int r = 0; r < KC; ++r) {
      wsb[KW_QT + r * KD + ch] = Qs[r * KLD + ch];
      wsb[KW_KT + r * KD + ch] = k_tf32r(Gs[r * KLD + ch] * eC);
    }
  }
  __syncthreads();
  const int g = lane >> 2, t = lane & 3;
  // ---- K+ K-^T (warps 0,1) and Q+ K-^T (warps 2,3): one m16 tile, n-tile = warp & 1, 16 k-steps
  {
    const float* am = (warp < 2 ? Ks : Qs) + g * KLD + t;
    const int nt = warp & 1;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int ks = 0; ks < KD / 8; ++ks) {
      const float* bb = Gs + (nt * 8 + g) * KLD + ks * 8 + t;
      k_mma(acc, am[ks * 8], am[8 * KLD + ks * 8], am[ks * 8 + 4], am[8 * KLD + ks * 8 + 4], bb[0], bb[4]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = g + (e >> 1) * 8, col = nt * 8 + 2 * t + (e & 1);
      if (warp < 2) As[row * KLC + col] = col < row ? beta_s[row] * acc[e] : 0.f;
      else wsb[KW_P + row * KC + col] = col <= row ? k_tf32r(acc[e]) : 0.f;
    }
  }
  __syncthreads();
  // ---- T = (I + A)^-1 by forward substitution, column per thread; then T diag(beta)
  if (tid < KC) {
    float tc[KC];
#pragma unroll
    for (int i = 0; i < KC; ++i) {
      float s = (i == tid) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s = fmaf(-As[i * KLC + j], tc[j], s);
      tc[i] = s;
    }
    const float b = beta_s[tid];
#pragma unroll
    for (int i = 0; i < KC; ++i) Ts[i * KLC + tid] = k_tf32r(tc[i] * b);
  }
  __syncthreads();
  // ---- W = Ts K+, Ut = Ts V: M = 16, K = 16 (2 k-steps), N = 128: warp -> n-tiles 4*warp .. +4
  {
    const float* aa = Ts + g * KLC + t;
    const float a0[2] = {aa[0], aa[8]}, a1[2] = {aa[8 * KLC], aa[8 * KLC + 8]}, a2[2] = {aa[4], aa[12]},
                a3[2] = {aa[8 * KLC + 4], aa[8 * KLC + 12]};
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const float* Bm = which == 0 ? Ks : Vs;
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int nt = warp * 4 + a;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          const float* bb = Bm + (ks * 8 + t) * KLD + nt * 8 + g;
          k_mma(acc, a0[ks], a1[ks], a2[ks], a3[ks], bb[0], bb[4 * KLD]);
        }
        float* og = wsb + (which == 0 ? KW_W : KW_UT) + g * KD + nt * 8 + 2 * t;
        if (which == 0) { acc[0] = k_tf32r(acc[0]); acc[1] = k_tf32r(acc[1]); acc[2] = k_tf32r(acc[2]); acc[3] = k_tf32r(acc[3]); }
        *reinterpret_cast<float2*>(og) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2*>(og + 8 * KD) = make_float2(acc[2], acc[3]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- kernel 2
// grid (4, H, nseg); 128 threads; sequential over the chunks of one segment
__global__ void __launch_bounds__(128)
kda_chunk_state_kernel(const float* __restrict__ ws, const int* __restrict__ seg, const int* __restrict__ seg_chunk0,
                       const __nv_bfloat16* __restrict__ pre, int ldp, float* __restrict__ S, float* __restrict__ tail,
                       float* __restrict__ o_raw, int ldo, int H) {
  __shared__ __align__(16) float Wsm[KC * KLD], Qsm[KC * KLD], Ksm[KC * KLD], Ssm[KVS * KLD];
  __shared__ __align__(16) float Psm[KC * KLC], Usm[KC * KLV], Dsm[KD];
  const int vs = blockIdx.x, h = blockIdx.y, sg = blockIdx.z;
  const int ci0 = seg_chunk0[sg];
  if (ci0 < 0) return;
  const int slot = seg[sg * 4], r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2];
  const int nch = (n + KC - 1) / KC;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int v0 = vs * KVS;
  const int smt = warp & 1, sng = warp >> 1;          // S fragments: v rows 16*smt.., k columns 64*sng..
  float sacc[8][4];
  float* Sg = S + ((static_cast<size_t>(slot) * H + h) * KD + v0) * KD;
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int col = sng * 64 + a * 8 + 2 * t, row = smt * 16 + g;
    const float2 lo = *reinterpret_cast<const float2*>(Sg + row * KD + col);
    const float2 hi = *reinterpret_cast<const float2*>(Sg + (row + 8) * KD + col);
    sacc[a][0] = lo.x; sacc[a][1] = lo.y; sacc[a][2] = hi.x; sacc[a][3] = hi.y;
    Ssm[row * KLD + col] = k_tf32r(lo.x); Ssm[row * KLD + col + 1] = k_tf32r(lo.y);
    Ssm[(row + 8) * KLD + col] = k_tf32r(hi.x); Ssm[(row + 8) * KLD + col + 1] = k_tf32r(hi.y);
  }
  for (int c = 0; c < nch; ++c) {
    const float* wsb = ws + (static_cast<size_t>(ci0 + c) * H + h) * KW_STRIDE;
    for (int idx = tid; idx < KC * KD / 4; idx += 128) {
      const int r = idx >> 5, c4 = (idx & 31) * 4;
      k_cp16(Wsm + r * KLD + c4, wsb + KW_W + r * KD + c4);
      k_cp16(Qsm + r * KLD + c4, wsb + KW_QT + r * KD + c4);
      k_cp16(Ksm + r * KLD + c4, wsb + KW_KT + r * KD + c4);
    }
    if (tid < KC * KC / 4) { const int r = tid >> 2, c4 = (tid & 3) * 4; k_cp16(Psm + r * KLC + c4, wsb + KW_P + r * KC + c4); }
    { const int r = tid >> 3, c4 = (tid & 7) * 4; k_cp16(Usm + r * KLV + c4, wsb + KW_UT + r * KD + v0 + c4); }
    if (tid < KD / 4) k_cp16(Dsm + tid * 4, wsb + KW_DC + tid * 4);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    // ---- X = W S0^T and O = Qt S0^T: one m16 tile of tokens, warp -> n-tile (8 v columns), 16 k-steps
    float xacc[4] = {0.f, 0.f, 0.f, 0.f}, oacc[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const float* wa = Wsm + g * KLD + t;
      const float* qa = Qsm + g * KLD + t;
#pragma unroll 4
      for (int ks = 0; ks < KD / 8; ++ks) {
        const float* sb = Ssm + (warp * 8 + g) * KLD + ks * 8 + t;
        const float b0 = sb[0], b1 = sb[4];
        k_mma(xacc, wa[ks * 8], wa[8 * KLD + ks * 8], wa[ks * 8 + 4], wa[8 * KLD + ks * 8 + 4], b0, b1);
        k_mma(oacc, qa[ks * 8], qa[8 * KLD + ks * 8], qa[ks * 8 + 4], qa[8 * KLD + ks * 8 + 4], b0, b1);
      }
    }
    {   // U = Ut - X (each element is read and written by the same thread)
      const int col = warp * 8 + 2 * t;
      float* u0 = Usm + g * KLV + col;
      float* u1 = Usm + (g + 8) * KLV + col;
      u0[0] = k_tf32r(u0[0] - xacc[0]); u0[1] = k_tf32r(u0[1] - xacc[1]);
      u1[0] = k_tf32r(u1[0] - xacc[2]); u1[1] = k_tf32r(u1[1] - xacc[3]);
    }
    __syncthreads();
    {   // O += P U (2 k-steps), store the valid rows
      const float* pa = Psm + g * KLC + t;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const float* ub = Usm + (ks * 8 + t) * KLV + warp * 8 + g;
        k_mma(oacc, pa[ks * 8], pa[8 * KLC + ks * 8], pa[ks * 8 + 4], pa[8 * KLC + ks * 8 + 4], ub[0], ub[4 * KLV]);
      }
      const int nvr = min(KC, n - c * KC);
      const int col = h * KD + v0 + warp * 8 + 2 * t;
      if (g < nvr) *reinterpret_cast<float2*>(o_raw + static_cast<size_t>(r0 + c * KC + g) * ldo + col) = make_float2(oacc[0], oacc[1]);
      if (g + 8 < nvr) *reinterpret_cast<float2*>(o_raw + static_cast<size_t>(r0 + c * KC + g + 8) * ldo + col) = make_float2(oacc[2], oacc[3]);
    }
    // ---- S <- S diag(Dc) + U^T Kt
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int col = sng * 64 + a * 8 + 2 * t;
      const float d0 = Dsm[col], d1 = Dsm[col + 1];
      sacc[a][0] *= d0; sacc[a][1] *= d1; sacc[a][2] *= d0; sacc[a][3] *= d1;
    }
#pragma unroll
    for (int ks = 0; ks < KC / 8; ++ks) {
      const float* ua = Usm + (ks * 8 + t) * KLV + smt * 16 + g;
      const float a0 = ua[0], a1 = ua[8], a2 = ua[4 * KLV], a3 = ua[4 * KLV + 8];
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        const float* kb = Ksm + (ks * 8 + t) * KLD + sng * 64 + a * 8 + g;
        k_mma(sacc[a], a0, a1, a2, a3, kb[0], kb[4 * KLD]);
      }
    }
    __syncthreads();            // every warp is done with the old S and with this chunk's operands
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int col = sng * 64 + a * 8 + 2 * t, row = smt * 16 + g;
      Ssm[row * KLD + col] = k_tf32r(sacc[a][0]); Ssm[row * KLD + col + 1] = k_tf32r(sacc[a][1]);
      Ssm[(row + 8) * KLD + col] = k_tf32r(sacc[a][2]); Ssm[(row + 8) * KLD + col + 1] = k_tf32r(sacc[a][3]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 8; ++a) {
    const int col = sng * 64 + a * 8 + 2 * t, row = smt * 16 + g;
    *reinterpret_cast<float2*>(Sg + row * KD + col) = make_float2(sacc[a][0], sacc[a][1]);
    *reinterpret_cast<float2*>(Sg + (row + 8) * KD + col) = make_float2(sacc[a][2], sacc[a][3]);
  }
  if (vs == 0) {          // conv history for the next call: raw inputs of the last three positions
    const int nn = H * KD, i = tid;
    float* tl = tail + static_cast<size_t>(slot) * 3 * 3 * nn;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const __nv_bfloat16* pr = pre + static_cast<size_t>(r0 + n - 3 + j) * ldp;
      tl[j * 3 * nn + h * KD + i] = __bfloat162float(pr[h * KD + i]);
      tl[j * 3 * nn + nn + h * KD + i] = __bfloat162float(pr[nn + h * KD + i]);
      tl[j * 3 * nn + 2 * nn + h * KD + i] = __bfloat162float(pr[2 * nn + h * KD + i]);
    }
  }
}

// ---------------------------------------------------------------------------------------------- kernel 3
// grid (chunks, H); 128 threads: warp w -> rows 4w..4w+3 of the chunk
__global__ void __launch_bounds__(128)
kda_chunk_out_kernel(const float* __restrict__ o_raw, int ldo, const float* __restrict__ g2, int ldg,
                     const float* __restrict__ o_norm, const int* __restrict__ seg, const int* __restrict__ chunks,
                     __nv_bfloat16* __restrict__ out, int ldout, int H) {
  const int ci = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sg = chunks[2 * ci], c = chunks[2 * ci + 1];
  const int r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2];
  const float4 nw = *reinterpret_cast<const float4*>(o_norm + lane * 4);
  for (int rr = 0; rr < 4; ++rr) {
    const int tt = c * KC + warp * 4 + rr;
    if (tt >= n) break;
    const size_t row = static_cast<size_t>(r0 + tt);
    const float4 o = *reinterpret_cast<const float4*>(o_raw + row * ldo + h * KD + lane * 4);
    const float o2 = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
    const float rs = rsqrtf(o2 / KD + 1e-5f);
    const float4 gt = *reinterpret_cast<const float4*>(g2 + row * ldg + h * KD + lane * 4);
    const __nv_bfloat162 b0 = __floats2bfloat162_rn(nw.x * o.x * rs / (1.f + __expf(-gt.x)), nw.y * o.y * rs / (1.f + __expf(-gt.y)));
    const __nv_bfloat162 b1 = __floats2bfloat162_rn(nw.z * o.z * rs / (1.f + __expf(-gt.z)), nw.w * o.w * rs / (1.f + __expf(-gt.w)));
    uint2 ov; ov.x = *reinterpret_cast<const uint32_t*>(&b0); ov.y = *reinterpret_cast<const uint32_t*>(&b1);
    *reinterpret_cast<uint2*>(out + row * ldout + h * KD + lane * 4) = ov;
  }
}

}  // namespace spark

using namespace spark;

extern "C" long long spark_kda_chunk_ws_floats(int n_chunks, int H) { return static_cast<long long>(n_chunks) * H * KW_STRIDE; }

// chunks: int [n_chunks][2] = (segment, 16-row chunk in segment); seg_chunk0: int [nseg] first chunk of a segment or -1.
// head_dim must be 128; o_raw fp32 [R, H*128]; ws from spark_kda_chunk_ws_floats.
extern "C" int spark_kda_chunk_prefill(const void* pre, int ldp, const float* g1, const float* g2, int ldg, const void* lr,
                                       int ldl, int beta_off, const float* conv_w, const float* A_log, const float* dt_bias,
                                       const float* o_norm, float* S, float* tail, const int* seg, int nseg, const int* chunks,
                                       int n_chunks, const int* seg_chunk0, float* ws, float* o_raw, void* out, int ldo, int H,
                                       int D, cudaStream_t s) {
  if (n_chunks <= 0) return 0;
  if (D != KD) return -5;
  kda_chunk_prep_kernel<<<dim3(n_chunks, H), 128, 0, s>>>((const __nv_bfloat16*)pre, ldp, g1, ldg, (const __nv_bfloat16*)lr, ldl,
                                                          beta_off, conv_w, A_log, dt_bias, tail, seg, chunks, ws, H);
  kda_chunk_state_kernel<<<dim3(KD / KVS, H, nseg), 128, 0, s>>>(ws, seg, seg_chunk0, (const __nv_bfloat16*)pre, ldp, S, tail,
                                                                 o_raw, H * KD, H);
  kda_chunk_out_kernel<<<dim3(n_chunks, H), 128, 0, s>>>(o_raw, H * KD, g2, ldg, o_norm, seg, chunks, (__nv_bfloat16*)out, ldo, H);
  return spark_launch_rc(__func__);
}
