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

extern "C" int spark_topk_select(const float* score, int ld, const int* pos, int R, int block, int k, int* sel,
                                 int sel_ld, int* sel_n, cudaStream_t s, int window) {
  if (R <= 0) return 0;
  if (sel_ld < k * block + block + window || window < 0) return -5;
  topk_select_kernel<<<R, 1024, 0, s>>>(score, ld, pos, block, k, window, sel, sel_ld, sel_n);
  return spark_launch_rc(__func__);
}
