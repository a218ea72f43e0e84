// Candidate selection of a feature-conditioned drafter: for each of J future positions the sub-vocabulary head's logits
// become log-probabilities and the K best (sorted, ties -> lowest id) become the position's candidates; low-rank
// embeddings of the candidates give pairwise edge scores between consecutive positions and one warp walks the greedy
// path (best unary + edge from the chosen predecessor).  Two launches per drafter step, no host round trip.
// Reference: engine-rs/src/dflash.rs:876-1016 (Candidates{ids, unary, edges, path, conf}), shim/draft_selector.cu:14,
// draft_head4.cu:12-162 (the head itself runs on the int4 / bf16 GEMV kernels of this library).
#include "../common/decode.cuh"

namespace spark {

constexpr int DK_MAX = 32;      // candidates per position
constexpr int DJ_MAX = 8;       // future positions

// greater-or-NaN order of a (value, index) pair: NaN beats numbers, equal values -> lowest index
__device__ __forceinline__ bool better(float a, int ia, float b, int ib) {
  if (a != a) return (b != b) ? ia < ib : true;
  if (b != b) return false;
  return a == b ? ia < ib : a > b;
}

// grid J, 256 threads; logits [J, V] -> ids [J, K] (int32), unary [J, K] log-probabilities, descending
__global__ void __launch_bounds__(256) draft_topk_kernel(const float* __restrict__ logits, int V, int K, int* __restrict__ ids,
                                                         float* __restrict__ unary) {
  __shared__ float rv[8];
  __shared__ int ri[8];
  __shared__ float lse_s;
  __shared__ int taken[DK_MAX];
  pdl_wait();
  pdl_trigger();
  const int j = blockIdx.x, t = threadIdx.x;
  const float* x = logits + static_cast<size_t>(j) * V;
  float m = -INFINITY;
  for (int v = t; v < V; v += 256) m = fmaxf(m, x[v]);
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o));
  if ((t & 31) == 0) rv[t >> 5] = m;
  __syncthreads();
  m = rv[0];
  for (int w = 1; w < 8; ++w) m = fmaxf(m, rv[w]);
  __syncthreads();
  float s = 0.f;
  for (int v = t; v < V; v += 256) s += expf(x[v] - m);
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(~0u, s, o);
  if ((t & 31) == 0) rv[t >> 5] = s;
  __syncthreads();
  if (t == 0) {
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += rv[w];
    lse_s = m + logf(tot);
  }
  __syncthreads();
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY;
    int bi = INT_MAX;
    for (int v = t; v < V; v += 256) {
      bool used = false;
      for (int q = 0; q < k; ++q) used |= (taken[q] == v);
      if (!used && better(x[v], v, bv, bi)) { bv = x[v]; bi = v; }
    }
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(~0u, bv, o);
      const int oi = __shfl_xor_sync(~0u, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if ((t & 31) == 0) { rv[t >> 5] = bv; ri[t >> 5] = bi; }
    __syncthreads();
    if (t == 0) {
      for (int w = 1; w < 8; ++w)
        if (better(rv[w], ri[w], rv[0], ri[0])) { rv[0] = rv[w]; ri[0] = ri[w]; }
      taken[k] = ri[0];
      ids[j * K + k] = ri[0];
      unary[j * K + k] = rv[0] - lse_s;
    }
    __syncthreads();
  }
}

// one CTA: edges[j][a][b] = <eu[j][a], ev[j+1][b]> for j < J-1, then the greedy path on warp 0.
// eu, ev: [J, K, r] projections of the candidates' embeddings; path [J] candidate index, tok [J] token id, conf [J].
__global__ void __launch_bounds__(256) draft_path_kernel(const float* __restrict__ unary, const int* __restrict__ ids,
                                                         const float* __restrict__ eu, const float* __restrict__ ev, int J, int K,
                                                         int r, float* __restrict__ edges, int* __restrict__ path,
                                                         int* __restrict__ tok, float* __restrict__ conf) {
  pdl_wait();
  pdl_trigger();
  const int t = threadIdx.x;
  for (int e = t; e < (J - 1) * K * K; e += 256) {
    const int j = e / (K * K), a = (e / K) % K, b = e % K;
    const float* u = eu + (static_cast<size_t>(j) * K + a) * r;
    const float* v = ev + (static_cast<size_t>(j + 1) * K + b) * r;
    float s = 0.f;
    for (int q = 0; q < r; ++q) s += u[q] * v[q];
    edges[e] = s;
  }
  __syncthreads();
  if (t >= 32) return;
  int prev = 0;
  for (int j = 0; j < J; ++j) {
    float val = -INFINITY;
    int idx = INT_MAX;
    if (t < K) {
      val = unary[j * K + t] + (j > 0 ? edges[((j - 1) * K + prev) * K + t] : 0.f);
      idx = t;
    }
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(~0u, val, o);
      const int oi = __shfl_xor_sync(~0u, idx, o);
      if (better(ov, oi, val, idx)) { val = ov; idx = oi; }
    }
    prev = idx;
    if (t == 0) {
      path[j] = prev;
      tok[j] = ids[j * K + prev];
      conf[j] = expf(unary[j * K + prev]);
    }
  }
}

}  // namespace spark

using namespace spark;

extern "C" int spark_draft_topk(const float* logits, int J, int V, int K, int* ids, float* unary, cudaStream_t s) {
  if (J <= 0) return 0;
  if (K < 1 || K > DK_MAX || K > V) return -5;
  const cudaError_t e = spark_launch_pdl(draft_topk_kernel, dim3(J), dim3(256), 0, s, dim3(1, 1, 1), logits, V, K, ids, unary);
  return e == cudaSuccess ? 0 : -4;
}
extern "C" int spark_draft_path(const float* unary, const int* ids, const float* eu, const float* ev, int J, int K, int r,
                                float* edges, int* path, int* tok, float* conf, cudaStream_t s) {
  if (J <= 0) return 0;
  if (K < 1 || K > DK_MAX || J > DJ_MAX) return -5;
  const cudaError_t e = spark_launch_pdl(draft_path_kernel, dim3(1), dim3(256), 0, s, dim3(1, 1, 1), unary, ids, eu, ev, J, K, r, edges,
                                         path, tok, conf);
  return e == cudaSuccess ? 0 : -4;
}
