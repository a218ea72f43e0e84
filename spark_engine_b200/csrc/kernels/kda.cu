// Kimi-delta-attention decode / verify / sequential-prefill kernel (one launch per layer):
//   depthwise causal conv (k=4) + SiLU on q,k,v -> L2-norm q,k (q scaled D^-0.5) -> per row
//   S <- S diag(exp(lam));  v' = beta (v - S k);  S <- S + v' k^T;  o = S q  ->  o_norm * RMS(o) * sigmoid(g2)
// with the per-channel log decay lam = -5 / (1 + exp(-exp(A_log) (g1 + dt_bias))) (g1, g2 = the low-rank gate
// projections, computed by the GEMV/GEMM kernels before this launch).
// Grid (head, segment); D x SPLIT threads; SPLIT adjacent lanes share state row S[h, i, :] (each holds D/SPLIT
// columns in registers for the whole segment; partial dot products meet through one shuffle).
// `commit` = 0 leaves state and conv history untouched (speculative verify); a later launch with the accepted
// row counts replays and commits.
// Reference: reference/glm53/kda.py:35-77 (math); engine-rs/shim/kda.cu (recurrent_lane_sequence*, kda_gates,
// kda_prep, kda_out), kda_conv_chain.cu.
#include "../common/ptx.cuh"

namespace spark {

template <int D, int SPLIT, bool PF>
__global__ void __launch_bounds__(D * SPLIT)
kda_seq_kernel(const __nv_bfloat16* __restrict__ pre, int ldp,          // [R, 3*H*D]  q | k | v before the conv
               const float* __restrict__ g1, const float* __restrict__ g2, int ldg,   // [R, H*D] each
               const __nv_bfloat16* __restrict__ lr, int ldl, int beta_off,            // beta logits at lr[:, beta_off + h]
               const float* __restrict__ conv_w,                         // [3*H*D, 4]
               const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ o_norm,
               float* __restrict__ S,                                    // [slots, H, D, D]
               float* __restrict__ tail,                                 // [slots, 3, 3*H*D]
               const int* __restrict__ seg, const int* __restrict__ n_rows,
               __nv_bfloat16* __restrict__ out, int ldo, int H, int commit,
               const int* __restrict__ path, int path_ld) {             // optional [nseg, path_ld]: the rows a segment walks
  // With `path` a segment is one root-to-node walk of a verification tree (see gdn.cu): step t reads batch row
  // path[sg][t]; only the last step's output is kept unless the walk is being committed.
  constexpr int DS = D / SPLIT, NW = D * SPLIT / 32;
  const int h = blockIdx.x, sg = blockIdx.y, i = threadIdx.x / SPLIT, part = threadIdx.x % SPLIT;
  const int slot = seg[sg * 4 + 0], r0 = seg[sg * 4 + 1];
  int n = seg[sg * 4 + 2];
  if (n_rows != nullptr) n = min(n, n_rows[sg]);
  if (n <= 0) return;
  const int nn = H * D;
  const int cq = h * D + i, ck = nn + h * D + i, cv = 2 * nn + h * D + i;
  __shared__ float sq[D], sk[D], sdec[D], red[2][NW], sred[NW];
  float s[DS];
  float* Srow = S + ((static_cast<size_t>(slot) * H + h) * D + i) * D + part * DS;
#pragma unroll
  for (int j = 0; j < DS; j += 4) {
    float4 t = *reinterpret_cast<const float4*>(Srow + j);
    s[j] = t.x; s[j + 1] = t.y; s[j + 2] = t.z; s[j + 3] = t.w;
  }
  float hq[3], hk_[3], hv[3];
  float* tl = tail + static_cast<size_t>(slot) * 3 * 3 * nn;
#pragma unroll
  for (int j = 0; j < 3; ++j) { hq[j] = tl[j * 3 * nn + cq]; hk_[j] = tl[j * 3 * nn + ck]; hv[j] = tl[j * 3 * nn + cv]; }
  const float wq[4] = {conv_w[cq * 4], conv_w[cq * 4 + 1], conv_w[cq * 4 + 2], conv_w[cq * 4 + 3]};
  const float wk[4] = {conv_w[ck * 4], conv_w[ck * 4 + 1], conv_w[ck * 4 + 2], conv_w[ck * 4 + 3]};
  const float wv[4] = {conv_w[cv * 4], conv_w[cv * 4 + 1], conv_w[cv * 4 + 2], conv_w[cv * 4 + 3]};
  const float a_exp = __expf(A_log[h]);
  const float dtb = dt_bias[h * D + i];
  const float nw = o_norm[i];
  const float qscale = rsqrtf(static_cast<float>(D));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* pq = sq + part * DS;
  const float* pk = sk + part * DS;
  const float* pd = sdec + part * DS;

  // PF (several rows per segment): the inputs of row t + 1 are fetched while row t is computed (nothing in them depends
  // on the recurrence); single-row decode launches keep each load next to its use (see gdn.cu).
  struct RowIn { float xq, xk, xv, g1, g2, bl; size_t r; };
  auto fetch = [&](int t) {
    RowIn in;
    in.r = static_cast<size_t>(path != nullptr ? path[sg * path_ld + t] : r0 + t);
    const __nv_bfloat16* pr = pre + in.r * ldp;
    in.xq = __bfloat162float(pr[cq]); in.xk = __bfloat162float(pr[ck]); in.xv = __bfloat162float(pr[cv]);
    in.g1 = g1[in.r * ldg + h * D + i];
    if (PF) {
      in.g2 = g2[in.r * ldg + h * D + i];
      in.bl = __bfloat162float(lr[in.r * ldl + beta_off + h]);
    }
    return in;
  };
  RowIn nxt = fetch(0);
  for (int t = 0; t < n; ++t) {
    RowIn cur = nxt;
    if (PF && t + 1 < n) nxt = fetch(t + 1);
    if (!PF && t > 0) cur = fetch(t);
    const size_t r = cur.r;
    const float xq = cur.xq, xk = cur.xk, xv = cur.xv;
    float q = hq[0] * wq[0] + hq[1] * wq[1] + hq[2] * wq[2] + xq * wq[3];
    float k = hk_[0] * wk[0] + hk_[1] * wk[1] + hk_[2] * wk[2] + xk * wk[3];
    float v = hv[0] * wv[0] + hv[1] * wv[1] + hv[2] * wv[2] + xv * wv[3];
    hq[0] = hq[1]; hq[1] = hq[2]; hq[2] = xq;
    hk_[0] = hk_[1]; hk_[1] = hk_[2]; hk_[2] = xk;
    hv[0] = hv[1]; hv[1] = hv[2]; hv[2] = xv;
    q = q / (1.f + __expf(-q)); k = k / (1.f + __expf(-k)); v = v / (1.f + __expf(-v));
    float q2 = warp_sum(q * q), k2 = warp_sum(k * k);
    if (lane == 0) { red[0][warp] = q2; red[1][warp] = k2; }
    // decay of key channel i for this row
    const float lam = -5.f / (1.f + __expf(-a_exp * (cur.g1 + dtb)));
    sdec[i] = __expf(lam);
    __syncthreads();
    q2 = 0.f; k2 = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) { q2 += red[0][w]; k2 += red[1][w]; }
    q2 *= 1.f / SPLIT; k2 *= 1.f / SPLIT;              // every channel was counted by its SPLIT lanes
    sq[i] = q * rsqrtf(q2 + 1e-6f) * qscale;
    sk[i] = k * rsqrtf(k2 + 1e-6f);
    __syncthreads();
    if (!PF) cur.bl = __bfloat162float(lr[r * ldl + beta_off + h]);
    const float beta = 1.f / (1.f + __expf(-cur.bl));
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < DS; ++j) { s[j] *= pd[j]; dot = fmaf(s[j], pk[j], dot); }
    if (SPLIT == 2) dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    const float vp = beta * (v - dot);
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < DS; ++j) { s[j] = fmaf(vp, pk[j], s[j]); o = fmaf(s[j], pq[j], o); }
    if (SPLIT == 2) o += __shfl_xor_sync(0xffffffffu, o, 1);
    float o2 = warp_sum(o * o);
    if (lane == 0) sred[warp] = o2;
    __syncthreads();
    o2 = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) o2 += sred[w];
    o2 *= 1.f / SPLIT;
    const float gate = PF ? cur.g2 : g2[r * ldg + h * D + i];
    const float res = nw * (o * rsqrtf(o2 / D + 1e-5f)) / (1.f + __expf(-gate));
    if (part == 0 && (path == nullptr || commit || t == n - 1)) out[r * ldo + h * D + i] = __float2bfloat16(res);
    __syncthreads();
  }
  if (commit) {
#pragma unroll
    for (int j = 0; j < DS; j += 4) *reinterpret_cast<float4*>(Srow + j) = make_float4(s[j], s[j + 1], s[j + 2], s[j + 3]);
    if (part == 0) {
#pragma unroll
      for (int j = 0; j < 3; ++j) { tl[j * 3 * nn + cq] = hq[j]; tl[j * 3 * nn + ck] = hk_[j]; tl[j * 3 * nn + cv] = hv[j]; }
    }
  }
}

}  // namespace spark

using namespace spark;

extern "C" int spark_kda_seq(const void* pre, int ldp, const float* g1, const float* g2, int ldg, const void* lr, int ldl,
                             int beta_off, const float* conv_w, const float* A_log, const float* dt_bias,
                             const float* o_norm, float* S, float* tail, const int* seg, const int* n_rows, int nseg,
                             void* out, int ldo, int H, int D, int commit, cudaStream_t s, const int* path, int path_ld, int multi_row) {
  if (nseg <= 0) return 0;
  dim3 grid(H, nseg);
#define SPARK_KDA(DD, SP, PFV)                                                                                            \
  kda_seq_kernel<DD, SP, PFV><<<grid, DD * SP, 0, s>>>((const __nv_bfloat16*)pre, ldp, g1, g2, ldg, (const __nv_bfloat16*)lr, ldl,  \
                                         beta_off, conv_w, A_log, dt_bias, o_norm, S, tail, seg, n_rows,             \
                                         (__nv_bfloat16*)out, ldo, H, commit, path, path_ld)
  if (D == 128) { if (multi_row) SPARK_KDA(128, 2, true); else SPARK_KDA(128, 2, false); }
  else if (D == 64) { if (multi_row) SPARK_KDA(64, 1, true); else SPARK_KDA(64, 1, false); }
  else if (D == 32) { if (multi_row) SPARK_KDA(32, 1, true); else SPARK_KDA(32, 1, false); }
  else return -5;
#undef SPARK_KDA
  return spark_launch_rc(__func__);
}
