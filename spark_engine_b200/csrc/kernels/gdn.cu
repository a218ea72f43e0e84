// Gated-DeltaNet decode / verify / sequential-prefill kernel (one launch per layer):
//   depthwise causal conv (k=4) + SiLU on q,k,v  ->  L2-norm q,k (q scaled D^-0.5)  ->  per row
//   S <- e^g S;  v' = beta (v - S k);  S <- S + v' k^T;  o = S q   ->  RMSNorm(o) * w * sigmoid(z).
// Grid (value head, segment); D * SPLIT threads; the SPLIT lanes of row i own state row S[h, i, :] in registers
// for the whole segment, so decode touches the state once.  Rows of a segment run in order with the
// oracle's operation order; `commit` = 0 leaves state and conv tails untouched (speculative verify),
// a later launch with the accepted row counts replays and commits (device-side counts `n_rows`).
// Conv tails are kept per value head ([slot, 3, Hv, 3D]: that head's q, k and v channels) so that no
// two CTAs ever write the same tail entry.
// Reference: engine-rs/shim/qwen_gdn.cu:45-190 (conv/recur kernels), :636-816 (launch shapes).
#include "../common/decode.cuh"

namespace spark {

// SPLIT lanes share one state row: lane `part` keeps columns [part * D/SPLIT, (part + 1) * D/SPLIT) in registers.  With
// D = 128 a whole row per thread (128 floats + temporaries) does not fit the register file and the compiler parks the
// state in local memory (ptxas: 32 registers, 2.6 KB of spills per thread); two lanes per row keep it in registers.
template <int D, int SPLIT, bool PF>
__global__ void __launch_bounds__(D * SPLIT)
gdn_seq_kernel(const __nv_bfloat16* __restrict__ proj, int ldp,      // [R, 2*Hk*D + 2*Hv*D]  q | k | v | z
               const __nv_bfloat16* __restrict__ ab, int ldab,       // [R, 2*Hv]  b | a
               const float* __restrict__ conv_w,                     // [2*Hk*D + Hv*D, 4]
               const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ norm_w,
               float* __restrict__ S,                                // [slots, Hv, D, D]
               float* __restrict__ tail,                             // [slots, 3, Hv, 3*D]
               const int* __restrict__ seg,                          // [nseg, 4] slot, r0, n, pos0
               const int* __restrict__ n_rows,                       // optional [nseg]: rows to process
               __nv_bfloat16* __restrict__ out, int ldo,             // [R, Hv*D]
               int Hk, int Hv, float eps, int commit,
               const int* __restrict__ path, int path_ld) {          // optional [nseg, path_ld]: the rows a segment walks
  // With `path` a segment is one root-to-node walk of a verification tree: step t reads batch row path[sg][t] (n_rows[sg]
  // of them) from the committed state, and only the last step's output is kept unless the walk is being committed.
  constexpr int DS = D / SPLIT, NW = D * SPLIT / 32;
  const int h = blockIdx.x, sg = blockIdx.y, i = threadIdx.x / SPLIT, part = threadIdx.x % SPLIT;
  // The segment table, the state and the conv history were last written at least two launches back (plan staging,
  // this layer's launch of the previous round): they are fetched before the dependency wait, so the 64 KB state of
  // the head streams in while the input projection that precedes this kernel drains.
  const int slot = seg[sg * 4 + 0], r0 = seg[sg * 4 + 1];
  int n = seg[sg * 4 + 2];
  const int hk = h / (Hv / Hk);
  const int cq = hk * D + i, ck = Hk * D + hk * D + i, cv = 2 * Hk * D + h * D + i;   // conv channels
  const int zc = 2 * Hk * D + Hv * D + h * D + i;                                       // z column
  __shared__ float sq[D], sk[D], red[2][NW];
  __shared__ float sred[NW];

  float s[DS];
  float* Srow = S + ((static_cast<size_t>(slot) * Hv + h) * D + i) * D + part * DS;
#pragma unroll
  for (int j = 0; j < DS; j += 4) {
    float4 t = *reinterpret_cast<const float4*>(Srow + j);
    s[j] = t.x; s[j + 1] = t.y; s[j + 2] = t.z; s[j + 3] = t.w;
  }
  // conv history (pre-activation inputs of the 3 previous positions), oldest first
  float hq[3], hk_[3], hv[3];
  float* tl = tail + (static_cast<size_t>(slot) * 3 * Hv + h) * 3 * D;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const float* t = tl + static_cast<size_t>(j) * Hv * 3 * D;
    hq[j] = t[i]; hk_[j] = t[D + i]; hv[j] = t[2 * D + i];
  }
  const float wq[4] = {conv_w[cq * 4], conv_w[cq * 4 + 1], conv_w[cq * 4 + 2], conv_w[cq * 4 + 3]};
  const float wk[4] = {conv_w[ck * 4], conv_w[ck * 4 + 1], conv_w[ck * 4 + 2], conv_w[ck * 4 + 3]};
  const float wv[4] = {conv_w[cv * 4], conv_w[cv * 4 + 1], conv_w[cv * 4 + 2], conv_w[cv * 4 + 3]};
  pdl_wait();
  pdl_trigger();
  if (n_rows != nullptr) n = min(n, n_rows[sg]);
  if (n <= 0) return;
  const float a_neg = -__expf(A_log[h]);
  const float dtb = dt_bias[h];
  const float nw = norm_w[i];
  const float qscale = rsqrtf(static_cast<float>(D));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* pq = sq + part * DS;
  const float* pk = sk + part * DS;

  // PF (launches with several rows per segment): the inputs of row t + 1 are fetched while row t is computed (nothing in
  // them depends on the recurrence).  Single-row decode launches keep each load next to its use.
  struct RowIn { float xq, xk, xv, bl, al, z; int row; };
  auto fetch = [&](int t) {
    RowIn r;
    r.row = path != nullptr ? path[sg * path_ld + t] : r0 + t;
    const __nv_bfloat16* pr = proj + static_cast<size_t>(r.row) * ldp;
    r.xq = __bfloat162float(pr[cq]); r.xk = __bfloat162float(pr[ck]); r.xv = __bfloat162float(pr[cv]);
    if (PF) {
      r.z = __bfloat162float(pr[zc]);
      r.bl = __bfloat162float(ab[static_cast<size_t>(r.row) * ldab + h]);
      r.al = __bfloat162float(ab[static_cast<size_t>(r.row) * ldab + Hv + h]);
    }
    return r;
  };
  RowIn nxt = fetch(0);
  for (int t = 0; t < n; ++t) {
    RowIn cur = nxt;
    if (PF && t + 1 < n) nxt = fetch(t + 1);
    if (!PF && t > 0) cur = fetch(t);
    const int row = cur.row;
    const float xq = cur.xq, xk = cur.xk, xv = cur.xv;
    float q = hq[0] * wq[0] + hq[1] * wq[1] + hq[2] * wq[2] + xq * wq[3];
    float k = hk_[0] * wk[0] + hk_[1] * wk[1] + hk_[2] * wk[2] + xk * wk[3];
    float v = hv[0] * wv[0] + hv[1] * wv[1] + hv[2] * wv[2] + xv * wv[3];
    hq[0] = hq[1]; hq[1] = hq[2]; hq[2] = xq;
    hk_[0] = hk_[1]; hk_[1] = hk_[2]; hk_[2] = xk;
    hv[0] = hv[1]; hv[1] = hv[2]; hv[2] = xv;
    q = q / (1.f + __expf(-q)); k = k / (1.f + __expf(-k)); v = v / (1.f + __expf(-v));
    // L2 norms of q and k over the D channels of this head (every channel is counted by its SPLIT lanes)
    float q2 = warp_sum(q * q), k2 = warp_sum(k * k);
    if (lane == 0) { red[0][warp] = q2; red[1][warp] = k2; }
    __syncthreads();
    q2 = 0.f; k2 = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) { q2 += red[0][w]; k2 += red[1][w]; }
    q2 *= 1.f / SPLIT; k2 *= 1.f / SPLIT;
    sq[i] = q * rsqrtf(q2 + eps) * qscale;
    sk[i] = k * rsqrtf(k2 + eps);
    __syncthreads();
    if (!PF) {
      cur.bl = __bfloat162float(ab[static_cast<size_t>(row) * ldab + h]);
      cur.al = __bfloat162float(ab[static_cast<size_t>(row) * ldab + Hv + h]);
    }
    const float beta = 1.f / (1.f + __expf(-cur.bl));
    const float xa = cur.al + dtb;
    const float sp = xa > 20.f ? xa : log1pf(__expf(xa));          // softplus
    const float dec = __expf(a_neg * sp);
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < DS; ++j) { s[j] *= dec; dot = fmaf(s[j], pk[j], dot); }
    if (SPLIT == 2) dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    const float vp = beta * (v - dot);
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < DS; ++j) { s[j] = fmaf(vp, pk[j], s[j]); o = fmaf(s[j], pq[j], o); }
    if (SPLIT == 2) o += __shfl_xor_sync(0xffffffffu, o, 1);
    // RMSNorm over the head's D outputs, gate with sigmoid(z)
    float o2 = warp_sum(o * o);
    if (lane == 0) sred[warp] = o2;
    __syncthreads();
    o2 = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) o2 += sred[w];
    o2 *= 1.f / SPLIT;
    if (!PF) cur.z = __bfloat162float(proj[static_cast<size_t>(row) * ldp + zc]);
    const float res = o * rsqrtf(o2 / D + eps) * nw / (1.f + __expf(-cur.z));
    if (part == 0 && (path == nullptr || commit || t == n - 1))
      out[static_cast<size_t>(row) * ldo + h * D + i] = __float2bfloat16(res);
    __syncthreads();     // sq/sk/red reused by the next row
  }
  if (commit) {
#pragma unroll
    for (int j = 0; j < DS; j += 4) *reinterpret_cast<float4*>(Srow + j) = make_float4(s[j], s[j + 1], s[j + 2], s[j + 3]);
    if (part == 0) {
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        float* t = tl + static_cast<size_t>(j) * Hv * 3 * D;
        t[i] = hq[j]; t[D + i] = hk_[j]; t[2 * D + i] = hv[j];
      }
    }
  }
}

}  // namespace spark

using namespace spark;

extern "C" int spark_gdn_seq(const void* proj, int ldp, const void* ab, int ldab, const float* conv_w,
                             const float* A_log, const float* dt_bias, const float* norm_w, float* S, float* tail,
                             const int* seg, const int* n_rows, int nseg, void* out, int ldo, int Hk, int Hv, int D,
                             float eps, int commit, cudaStream_t s, const int* path, int path_ld, int multi_row) {
  if (nseg <= 0) return 0;
  dim3 grid(Hv, nseg);
  cudaError_t e = cudaSuccess;
#define SPARK_GDN(DD, SP, PFV)                                                                                          \
  e = spark_launch_pdl(gdn_seq_kernel<DD, SP, PFV>, grid, dim3(DD * SP), 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)proj, ldp, \
                       (const __nv_bfloat16*)ab, ldab, conv_w, A_log, dt_bias, norm_w, S, tail, seg, n_rows,             \
                       (__nv_bfloat16*)out, ldo, Hk, Hv, eps, commit, path, path_ld)
  const bool pf = multi_row != 0;
  if (D == 128) { if (pf) SPARK_GDN(128, 2, true); else SPARK_GDN(128, 2, false); }
  else if (D == 64) { if (pf) SPARK_GDN(64, 1, true); else SPARK_GDN(64, 1, false); }
  else if (D == 32) { if (pf) SPARK_GDN(32, 1, true); else SPARK_GDN(32, 1, false); }
#undef SPARK_GDN
  else
    return -5;
  return e == cudaSuccess ? 0 : -4;
}
