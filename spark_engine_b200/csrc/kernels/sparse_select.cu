// Block-sparse key selection for the sparse attention layers (QSA / DSA style indexers).
//   idx_score : score[r, b] = sum over indexer heads of relu(q_h . pooled_key_b) * scale   (optionally weighted
//               per head: DSA `weights_proj`), for the complete blocks b < vis(r) = (pos+1)/block
//   topk_select: exact top-k blocks per row, ties -> lowest block index, emitted in ascending block order and
//               expanded to token indices, followed by the tail tokens vis*block .. pos of the open block.
//               Rows with vis <= k select every token (no scoring needed).
// Exactness and a deterministic order matter: the selected list drives attention, and N-stream decode must equal
// 1-stream decode bit for bit.  The threshold comes from a 4-pass 8-bit radix select over the float bits (scores
// are >= 0, so their bit patterns sort like unsigned integers), one CTA per row.
// Reference: engine-rs/shim/qwen_qsa.cu:903-1076 (score_kernel, select_kernel), topk_select.cuh,
// dataflow.cu:159-336 (dsa_score*), dsa_index.cu:225 (dsa_topk_rows).
#include "../common/ptx.cuh"

namespace spark {

// grid (ceil(nb_max/8), R), 256 threads: warp w of CTA x scores block x*8+w.  idx_dim <= 128 (4 dims per lane).
__global__ void __launch_bounds__(256)
idx_score_kernel(const float* __restrict__ qi, int H, int Dm, const float* __restrict__ pool, const long long* __restrict__ row_kv,
                 const int* __restrict__ pos, int block, const float* __restrict__ head_w, float scale,
                 float* __restrict__ score, int ld) {
  const int r = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * 8 + warp;
  const int vis = (pos[r] + 1) / block;
  if (b >= vis) return;
  const float* kc = pool + (row_kv[r] / block + b) * Dm;
  float k[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) k[j] = (lane * 4 + j) < Dm ? kc[lane * 4 + j] : 0.f;
  float acc = 0.f;
  for (int h = 0; h < H; ++h) {
    const float* q = qi + (static_cast<size_t>(r) * H + h) * Dm;
    float d = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) if (lane * 4 + j < Dm) d = fmaf(q[lane * 4 + j], k[j], d);
    d = warp_sum(d);
    d = fmaxf(d, 0.f) * scale;
    acc += head_w ? head_w[static_cast<size_t>(r) * H + h] * d : d;
  }
  if (lane == 0) score[static_cast<size_t>(r) * ld + b] = acc;
}

// ------------------------------------------------------------------------------------------------------------
// The same scores for prefill rows on tensor cores.  The M side of the MMA tiles is (row, head): 64 consecutive
// [row][head] query vectors of one segment (64 / H rows) are staged once, pooled-key tiles of 64 blocks are streamed
// with cp.async (double buffered), S = Q K^T runs as 3xTF32 (every operand split into a TF32 head and a TF32 remainder,
// three m16n8k8 MMAs per product: fp32-grade scores, so a row selects the same blocks whether it is scored here or by
// the decode kernel), then relu x scale x head weight goes through shared memory where the H heads of a row are summed
// in head order.  Blocks beyond a row's visible range get values nobody reads.
// Reference: engine-rs/shim/ds41_attn.cu:447-824, dataflow.cu:159-336 (tensor-core indexer scoring for prefill rows).
constexpr int IS_M = 64, IS_N = 64;

__device__ __forceinline__ void is_cp16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc));
}
__device__ __forceinline__ void is_split(float x, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(x - __uint_as_float(hi)));
}
__device__ __forceinline__ void is_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (ceil(max segment rows / (64 / H)), segments); 256 threads: warps w and w + 4 share the 16 (row, head) pairs of
// M tile w & 3 and take four of the eight 8-block column tiles each (shared memory allows one CTA per SM, so the
// second set of warps is what hides the fragment-load latency).  H in {1, 2, 4, ..., 64}, Dm % 8 == 0, Dm <= 128.
// seg: int [nseg][4] = slot, first row, rows, first position.
__global__ void __launch_bounds__(256)
idx_score_mma_kernel(const float* __restrict__ qi, int H, int Dm, const float* __restrict__ pool,
                     const long long* __restrict__ row_kv, const int* __restrict__ seg, int block,
                     const float* __restrict__ head_w, float scale, float* __restrict__ score, int ld) {
  extern __shared__ __align__(16) uint8_t smem_is[];
  const int LQ = Dm + 4;                                             // row stride in floats: rows fall on different banks
  float* Qs = reinterpret_cast<float*>(smem_is);                     // [64][LQ]
  float* Ks = Qs + IS_M * LQ;                                        // [2][64][LQ]
  float* Ss = Ks + 2 * IS_N * LQ;                                    // [64][65]
  const int sg = blockIdx.y, rpc = IS_M / H;
  const int r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2], pos0 = seg[sg * 4 + 3];
  const int q0 = blockIdx.x * rpc;                                   // first row of this CTA inside the segment
  if (q0 >= n) return;
  const int rows_valid = min(rpc, n - q0);
  const int nb = (pos0 + q0 + rows_valid) / block;                   // blocks visible to the CTA's last row
  if (nb <= 0) return;
  const int ntiles = (nb + IS_N - 1) / IS_N;
  const float* kbase = pool + (row_kv[r0] / block) * Dm;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int VPR = Dm >> 2;                                           // 16-byte vectors per row
  for (int i = tid; i < IS_M * VPR; i += 256) {
    const int m = i / VPR, v = i - m * VPR;
    const int mm = min(m, rows_valid * H - 1);                       // padded (row, head) pairs repeat the last valid one
    is_cp16(Qs + m * LQ + v * 4, qi + (static_cast<size_t>(r0 + q0) * H + mm) * Dm + v * 4);
  }
  auto load_k = [&](int j, int buf) {
    float* kd = Ks + buf * IS_N * LQ;
    for (int i = tid; i < IS_N * VPR; i += 256) {
      const int r = i / VPR, v = i - r * VPR;
      const int b = j * IS_N + r;
      if (b < nb) is_cp16(kd + r * LQ + v * 4, kbase + static_cast<size_t>(b) * Dm + v * 4);
      else *reinterpret_cast<float4*>(kd + r * LQ + v * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  load_k(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  // weights of this thread's two (row, head) pairs: accumulator rows g and g + 8 of the warp's 16
  const int m_lo = (warp & 3) * 16 + g, m_hi = m_lo + 8, nt0 = (warp >> 2) * 4;
  const int mv_lo = min(m_lo, rows_valid * H - 1), mv_hi = min(m_hi, rows_valid * H - 1);
  const float w_lo = scale * (head_w ? head_w[static_cast<size_t>(r0 + q0) * H + mv_lo] : 1.f);
  const float w_hi = scale * (head_w ? head_w[static_cast<size_t>(r0 + q0) * H + mv_hi] : 1.f);
  for (int j = 0; j < ntiles; ++j) {
    const int buf = j & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                                 // tile j landed; Ss of tile j-1 has been read
    if (j + 1 < ntiles) { load_k(j + 1, buf ^ 1); asm volatile("cp.async.commit_group;" ::: "memory"); }
    const float* kb = Ks + buf * IS_N * LQ;
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { s[i][0] = 0.f; s[i][1] = 0.f; s[i][2] = 0.f; s[i][3] = 0.f; }
    for (int ks = 0; ks < Dm / 8; ++ks) {
      uint32_t ah[4], al[4];
      is_split(Qs[m_lo * LQ + ks * 8 + t], ah[0], al[0]);
      is_split(Qs[m_hi * LQ + ks * 8 + t], ah[1], al[1]);
      is_split(Qs[m_lo * LQ + ks * 8 + t + 4], ah[2], al[2]);
      is_split(Qs[m_hi * LQ + ks * 8 + t + 4], ah[3], al[3]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        uint32_t bh0, bl0, bh1, bl1;
        is_split(kb[((nt0 + nt) * 8 + g) * LQ + ks * 8 + t], bh0, bl0);
        is_split(kb[((nt0 + nt) * 8 + g) * LQ + ks * 8 + t + 4], bh1, bl1);
        is_mma(s[nt], al, bh0, bh1);                                 // small terms first
        is_mma(s[nt], ah, bl0, bl1);
        is_mma(s[nt], ah, bh0, bh1);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int c = (nt0 + nt) * 8 + 2 * t;
      Ss[m_lo * 65 + c] = fmaxf(s[nt][0], 0.f) * w_lo; Ss[m_lo * 65 + c + 1] = fmaxf(s[nt][1], 0.f) * w_lo;
      Ss[m_hi * 65 + c] = fmaxf(s[nt][2], 0.f) * w_hi; Ss[m_hi * 65 + c + 1] = fmaxf(s[nt][3], 0.f) * w_hi;
    }
    __syncthreads();
    for (int i = tid; i < rows_valid * IS_N; i += 256) {
      const int rq = i >> 6, c = i & 63, b = j * IS_N + c;
      if (b >= nb) continue;
      float acc = 0.f;
      for (int h = 0; h < H; ++h) acc += Ss[(rq * H + h) * 65 + c];
      score[static_cast<size_t>(r0 + q0 + rq) * ld + b] = acc;
    }
  }
}

__device__ __forceinline__ int block_excl_scan(int v, int* warp_tot, int& total) {
  // exclusive prefix sum over the 1024 threads of the CTA; `total` = sum over all threads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += t; }
    warp_tot[lane] = w;                       // inclusive over warps
  }
  __syncthreads();
  total = warp_tot[31];
  const int base = warp ? warp_tot[warp - 1] : 0;
  __syncthreads();
  return base + inc - v;
}

// float bits -> unsigned key with the same order (negative scores sort below positive ones, -0 == +0)
__device__ __forceinline__ uint32_t order_key(uint32_t b) {
  if (b == 0x80000000u) b = 0u;
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// grid R, 1024 threads.  sel [R, sel_ld] token indices, sel_n [R].  `window` > 0: the last `window` positions are
// always visible (sliding window); selected blocks are emitted only up to the start of that range, so no token
// appears twice.
__global__ void __launch_bounds__(1024)
topk_select_kernel(const float* __restrict__ score, int ld, const int* __restrict__ pos, int block, int k, int window,
                   int* __restrict__ sel, int sel_ld, int* __restrict__ sel_n) {
  __shared__ int s_straddle;
  __shared__ int hist[256];
  __shared__ int warp_tot[32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  const int r = blockIdx.x, t = threadIdx.x;
  const int p = pos[r];
  const int vis = (p + 1) / block;
  int* out = sel + static_cast<size_t>(r) * sel_ld;
  if (vis <= k) {                                  // every token is visible
    for (int i = t; i <= p; i += 1024) out[i] = i;
    if (t == 0) sel_n[r] = p + 1;
    return;
  }
  const uint32_t* s = reinterpret_cast<const uint32_t*>(score + static_cast<size_t>(r) * ld);
  // ---- radix select: the k-th largest key
  uint32_t prefix = 0, mask = 0;
  int need = k;
  for (int pass = 3; pass >= 0; --pass) {
    for (int i = t; i < 256; i += 1024) hist[i] = 0;
    __syncthreads();
    const int shift = pass * 8;
    for (int i = t; i < vis; i += 1024) {
      const uint32_t key = order_key(s[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (t == 0) {
      int acc = 0, d = 255;
      for (; d > 0; --d) { if (acc + hist[d] >= need) break; acc += hist[d]; }
      s_prefix = prefix | (static_cast<uint32_t>(d) << shift);
      s_need = need - acc;                         // still needed among keys with this digit
    }
    __syncthreads();
    prefix = s_prefix; need = s_need;
    mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t thr = prefix;                     // k-th largest key; `need` of the keys equal to thr are taken
  // ---- emit in ascending block order; blocks that reach into the always-visible range [lo, p] are cut there
  const int tail0 = vis * block;
  const int lo = window > 0 ? min(max(0, p + 1 - window), tail0) : tail0;
  const int sb = lo / block;                       // block that straddles lo (when lo is not a block boundary)
  if (t == 0) s_straddle = 0;
  __syncthreads();
  int n_out = 0, eq_taken = 0;
  for (int base = 0; base < vis; base += 1024) {
    const int i = base + t;
    const uint32_t key = i < vis ? order_key(s[i]) : 0u;
    const int is_eq = (i < vis && key == thr) ? 1 : 0;
    int tot_eq;
    const int eq_rank = block_excl_scan(is_eq, warp_tot, tot_eq);
    const int take = (i < vis) && (key > thr || (is_eq && eq_taken + eq_rank < need));
    const int full = take && (i + 1) * block <= lo;
    if (take && !full && i == sb && lo > sb * block) s_straddle = 1;
    int tot_take;
    const int o = block_excl_scan(full ? 1 : 0, warp_tot, tot_take);
    if (full) {
      const int dst = (n_out + o) * block;
      for (int j = 0; j < block; ++j) out[dst + j] = i * block + j;
    }
    n_out += tot_take;
    eq_taken += tot_eq;
  }
  __syncthreads();
  int cnt = n_out * block;
  if (s_straddle) {
    const int m = lo - sb * block;
    if (t < m) out[cnt + t] = sb * block + t;
    cnt += m;
  }
  // ---- the always-visible range: window and the tokens of the open block
  for (int i = t; i <= p - lo; i += 1024) out[cnt + i] = lo + i;
  if (t == 0) sel_n[r] = cnt + (p - lo + 1);
}

// ------------------------------------------------------------------------------------------------------------
// Multi-CTA form of the same exact selection for very long contexts (>= 128K candidates per row, where one CTA per row
// leaves a decode round of a few rows on a handful of SMs): C CTAs per row, each owning one slice of the candidates.
//   mc_hist   x3  pass 2, 1, 0 over key digits of 11 / 11 / 10 bits: every CTA first resolves the passes already
//                 finished from the row's global histograms (a block-wide suffix scan of 2048 bins), then adds its
//                 slice's digits of the current pass to the global histogram through a shared-memory one.
//   mc_count      per slice: keys above the threshold in fully selectable blocks, keys equal to it, and those of
//                 them in fully selectable blocks.
//   mc_emit       a CTA sums the counts of the slices before it (ties go to the lowest indices, so the equal keys a
//                 slice may take are what earlier slices left), emits its slice in ascending block order; the last
//                 CTA adds the straddling block, the always-visible range and the count.
// Launches depend on one another only through stream order: no CTA waits for another.  Output identical to
// topk_select_kernel.  Reference: engine-rs/shim/ds41_attn.cu:825-942 (multi-CTA radix select).
constexpr int MC_BINS = 2048;

__device__ __forceinline__ int mc_digit(uint32_t key, int pass) {
  return pass == 2 ? static_cast<int>(key >> 21) : (pass == 1 ? static_cast<int>((key >> 10) & 2047u) : static_cast<int>(key & 1023u));
}
__device__ __forceinline__ uint32_t mc_place(int d, int pass) {
  return pass == 2 ? static_cast<uint32_t>(d) << 21 : (pass == 1 ? static_cast<uint32_t>(d) << 10 : static_cast<uint32_t>(d));
}
__device__ __forceinline__ uint32_t mc_mask(int pass) {       // bits decided once passes > `pass`... down to `pass` are done
  return pass == 2 ? 0xFFE00000u : (pass == 1 ? 0xFFFFFC00u : 0xFFFFFFFFu);
}

// Resolves passes 2 .. last (inclusive) from the row's global histograms; all 1024 threads call it.
__device__ void mc_resolve(const int* __restrict__ gh, int last, int k, int* warp_tot, int* s_pair, uint32_t& prefix, int& need) {
  prefix = 0u;
  need = k;
  for (int pass = 2; pass >= last; --pass) {
    const int* h = gh + pass * MC_BINS;
    // thread t owns bins 2047 - 2t and 2046 - 2t: an exclusive scan in thread order counts the keys with larger digits
    const int h0 = h[MC_BINS - 1 - 2 * threadIdx.x], h1 = h[MC_BINS - 2 - 2 * threadIdx.x];
    int tot;
    const int before = block_excl_scan(h0 + h1, warp_tot, tot);
    if (before < need && before + h0 >= need) { s_pair[0] = MC_BINS - 1 - 2 * threadIdx.x; s_pair[1] = need - before; }
    else if (before + h0 < need && before + h0 + h1 >= need) { s_pair[0] = MC_BINS - 2 - 2 * threadIdx.x; s_pair[1] = need - before - h0; }
    __syncthreads();
    prefix |= mc_place(s_pair[0], pass);
    need = s_pair[1];
    __syncthreads();
  }
}

__device__ __forceinline__ void mc_slice(int vis, int C, int c, int& i0, int& i1) {
  const int chunk = ((vis + C - 1) / C + 31) & ~31;
  i0 = min(vis, c * chunk);
  i1 = min(vis, i0 + chunk);
}

// grid (C, R), 1024 threads.  ghist [R, 3, 2048] zeroed before pass 2.
__global__ void __launch_bounds__(1024)
mc_hist_kernel(const float* __restrict__ score, int ld, const int* __restrict__ pos, int block, int k, int pass,
               int* __restrict__ ghist) {
  __shared__ int hist[MC_BINS];
  __shared__ int warp_tot[32];
  __shared__ int s_pair[2];
  const int r = blockIdx.y, t = threadIdx.x;
  const int vis = (pos[r] + 1) / block;
  if (vis <= k) return;
  int* gh = ghist + static_cast<size_t>(r) * 3 * MC_BINS;
  uint32_t prefix = 0u;
  int need = k;
  if (pass < 2) mc_resolve(gh, pass + 1, k, warp_tot, s_pair, prefix, need);
  const uint32_t mask = pass < 2 ? mc_mask(pass + 1) : 0u;
  hist[t] = 0; hist[t + 1024] = 0;
  __syncthreads();
  int i0, i1;
  mc_slice(vis, gridDim.x, blockIdx.x, i0, i1);
  const uint32_t* s = reinterpret_cast<const uint32_t*>(score + static_cast<size_t>(r) * ld);
  for (int i = i0 + t; i < i1; i += 1024) {
    const uint32_t key = order_key(s[i]);
    if ((key & mask) == prefix) atomicAdd(&hist[mc_digit(key, pass)], 1);
  }
  __syncthreads();
  for (int b = t; b < MC_BINS; b += 1024)
    if (hist[b]) atomicAdd(&gh[pass * MC_BINS + b], hist[b]);
}

__device__ __forceinline__ int mc_lo(int p, int vis, int block, int window) {
  const int tail0 = vis * block;
  return window > 0 ? min(max(0, p + 1 - window), tail0) : tail0;
}

// grid (C, R), 1024 threads.  counts [R, C, 3] = {above threshold and full, equal, equal and full}
__global__ void __launch_bounds__(1024)
mc_count_kernel(const float* __restrict__ score, int ld, const int* __restrict__ pos, int block, int k, int window,
                const int* __restrict__ ghist, int* __restrict__ counts) {
  __shared__ int warp_tot[32];
  __shared__ int s_pair[2];
  __shared__ int s_cnt[3];
  const int r = blockIdx.y, t = threadIdx.x, p = pos[r];
  const int vis = (p + 1) / block;
  if (vis <= k) return;
  uint32_t thr;
  int need;
  mc_resolve(ghist + static_cast<size_t>(r) * 3 * MC_BINS, 0, k, warp_tot, s_pair, thr, need);
  if (t < 3) s_cnt[t] = 0;
  __syncthreads();
  const int nfull = mc_lo(p, vis, block, window) / block;        // blocks 0 .. nfull-1 lie below the always-visible range
  int i0, i1;
  mc_slice(vis, gridDim.x, blockIdx.x, i0, i1);
  const uint32_t* s = reinterpret_cast<const uint32_t*>(score + static_cast<size_t>(r) * ld);
  int gt_full = 0, eq = 0, eq_full = 0;
  for (int i = i0 + t; i < i1; i += 1024) {
    const uint32_t key = order_key(s[i]);
    gt_full += key > thr && i < nfull;
    eq += key == thr;
    eq_full += key == thr && i < nfull;
  }
  gt_full = __reduce_add_sync(0xffffffffu, gt_full); eq = __reduce_add_sync(0xffffffffu, eq);
  eq_full = __reduce_add_sync(0xffffffffu, eq_full);
  if ((t & 31) == 0) { atomicAdd(&s_cnt[0], gt_full); atomicAdd(&s_cnt[1], eq); atomicAdd(&s_cnt[2], eq_full); }
  __syncthreads();
  if (t < 3) counts[(static_cast<size_t>(r) * gridDim.x + blockIdx.x) * 3 + t] = s_cnt[t];
}

// grid (C, R), 1024 threads.
__global__ void __launch_bounds__(1024)
mc_emit_kernel(const float* __restrict__ score, int ld, const int* __restrict__ pos, int block, int k, int window,
               const int* __restrict__ ghist, const int* __restrict__ counts, int* __restrict__ sel, int sel_ld,
               int* __restrict__ sel_n) {
  __shared__ int warp_tot[32];
  __shared__ int s_pair[2];
  __shared__ int s_before[2];
  const int r = blockIdx.y, t = threadIdx.x, p = pos[r], C = gridDim.x, c = blockIdx.x;
  const int vis = (p + 1) / block;
  int* out = sel + static_cast<size_t>(r) * sel_ld;
  if (vis <= k) {                                  // every token is visible
    for (int i = c * 1024 + t; i <= p; i += C * 1024) out[i] = i;
    if (c == 0 && t == 0) sel_n[r] = p + 1;
    return;
  }
  uint32_t thr;
  int need;
  mc_resolve(ghist + static_cast<size_t>(r) * 3 * MC_BINS, 0, k, warp_tot, s_pair, thr, need);
  const int lo = mc_lo(p, vis, block, window);
  const int nfull = lo / block;
  const int* cn = counts + static_cast<size_t>(r) * C * 3;
  if (t == 0) {
    int eq_before = 0, full_before = 0;
    for (int q = 0; q < c; ++q) {
      full_before += cn[q * 3] + min(cn[q * 3 + 2], max(0, need - eq_before));
      eq_before += cn[q * 3 + 1];
    }
    s_before[0] = eq_before; s_before[1] = full_before;
  }
  __syncthreads();
  int eq_taken = s_before[0], n_out = s_before[1];
  int i0, i1;
  mc_slice(vis, C, c, i0, i1);
  const uint32_t* s = reinterpret_cast<const uint32_t*>(score + static_cast<size_t>(r) * ld);
  for (int base = i0; base < i1; base += 1024) {
    const int i = base + t;
    const uint32_t key = i < i1 ? order_key(s[i]) : 0u;
    const int is_eq = (i < i1 && key == thr) ? 1 : 0;
    int tot_eq;
    const int eq_rank = block_excl_scan(is_eq, warp_tot, tot_eq);
    const int take = (i < i1) && (key > thr || (is_eq && eq_taken + eq_rank < need));
    const int full = take && i < nfull;
    int tot_take;
    const int o = block_excl_scan(full ? 1 : 0, warp_tot, tot_take);
    if (full) {
      const int dst = (n_out + o) * block;
      for (int j = 0; j < block; ++j) out[dst + j] = i * block + j;
    }
    n_out += tot_take;
    eq_taken += tot_eq;
  }
  if (c != C - 1) return;
  // ---- last CTA: n_out is the row's total; the block that straddles lo, then the always-visible range
  int cnt = n_out * block;
  const int sb = nfull;
  if (lo > sb * block && sb < vis) {               // lo inside block sb: is sb selected?
    const uint32_t ksb = order_key(s[sb]);
    int taken = ksb > thr;
    if (ksb == thr) {
      // rank of sb among the equal keys = equal keys of the slices before sb's + those before sb inside its slice
      const int chunk = ((vis + C - 1) / C + 31) & ~31;
      const int cs = sb / chunk;
      int part = 0;
      for (int i = cs * chunk + t; i < sb; i += 1024) part += order_key(s[i]) == thr;
      int tot;
      block_excl_scan(part, warp_tot, tot);
      int eq_b = tot;
      for (int q = 0; q < cs; ++q) eq_b += cn[q * 3 + 1];
      taken = eq_b < need;
    }
    if (taken) {
      const int m = lo - sb * block;
      if (t < m) out[cnt + t] = sb * block + t;
      cnt += m;
    }
  }
  for (int i = t; i <= p - lo; i += 1024) out[cnt + i] = lo + i;
  if (t == 0) sel_n[r] = cnt + (p - lo + 1);
}

}  // namespace spark

using namespace spark;

extern "C" int spark_idx_score(const float* qi, int R, int H, int Dm, const float* pool, const long long* row_kv,
                               const int* pos, int block, const float* head_w, float scale, float* score, int ld,
                               int nb_max, cudaStream_t s) {
  if (R <= 0 || nb_max <= 0) return 0;
  if (Dm > 128) return -5;
  idx_score_kernel<<<dim3((nb_max + 7) / 8, R), 256, 0, s>>>(qi, H, Dm, pool, row_kv, pos, block, head_w, scale, score, ld);
  return spark_launch_rc(__func__);
}

// Prefill rows (whole segments): tensor-core scoring.  H a power of two <= 64, Dm % 8 == 0, Dm <= 128.
extern "C" int spark_idx_score_mma(const float* qi, int H, int Dm, const float* pool, const long long* row_kv, const int* seg,
                                   int nseg, int max_rows, int block, const float* head_w, float scale, float* score, int ld,
                                   cudaStream_t s) {
  if (nseg <= 0 || max_rows <= 0) return 0;
  if (H < 1 || H > 64 || (H & (H - 1)) || (Dm & 7) || Dm > 128 || Dm < 8) return -5;
  const int smem = (3 * 64 * (Dm + 4) + 64 * 65) * 4;
  static bool done = false;
  if (!done) { cudaFuncSetAttribute(idx_score_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024); done = true; }
  const int rpc = 64 / H;
  idx_score_mma_kernel<<<dim3((max_rows + rpc - 1) / rpc, nseg), 256, smem, s>>>(qi, H, Dm, pool, row_kv, seg, block, head_w, scale,
                                                                                score, ld);
  return spark_launch_rc(__func__);
}

extern "C" int spark_topk_select(const float* score, int ld, const int* pos, int R, int block, int k, int* sel,
                                 int sel_ld, int* sel_n, cudaStream_t s, int window) {
  if (R <= 0) return 0;
  if (sel_ld < k * block + block + window || window < 0) return -5;
  topk_select_kernel<<<R, 1024, 0, s>>>(score, ld, pos, block, k, window, sel, sel_ld, sel_n);
  return spark_launch_rc(__func__);
}

// Multi-CTA exact selection: `ctas` CTAs per row (<= 64); work: int32 [R * (3 * 2048 + 3 * ctas)] scratch.
extern "C" int spark_topk_select_mc(const float* score, int ld, const int* pos, int R, int block, int k, int* sel,
                                    int sel_ld, int* sel_n, cudaStream_t s, int window, int ctas, int* work) {
  if (R <= 0) return 0;
  if (sel_ld < k * block + block + window || window < 0 || ctas < 1 || ctas > 64 || !work) return -5;
  int* ghist = work;
  int* counts = work + static_cast<size_t>(R) * 3 * MC_BINS;
  if (cudaMemsetAsync(ghist, 0, static_cast<size_t>(R) * 3 * MC_BINS * sizeof(int), s) != cudaSuccess) return -4;
  const dim3 grid(ctas, R);
  for (int pass = 2; pass >= 0; --pass) mc_hist_kernel<<<grid, 1024, 0, s>>>(score, ld, pos, block, k, pass, ghist);
  mc_count_kernel<<<grid, 1024, 0, s>>>(score, ld, pos, block, k, window, ghist, counts);
  mc_emit_kernel<<<grid, 1024, 0, s>>>(score, ld, pos, block, k, window, ghist, counts, sel, sel_ld, sel_n);
  return spark_launch_rc(__func__);
}
