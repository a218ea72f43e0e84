// MoE routing and combine kernels.
//   moe_route    : router scores -> top-k (ties -> lowest expert id) -> renormalised weights; three
//                  router kinds (softmax-renorm, sigmoid+bias x scale, sqrt-softplus+bias x scale);
//                  also emits the (row, expert) pair table the grouped GEMV/GEMM kernels consume.
//   moe_sort     : stable counting sort of the (row, slot) pairs by expert -> permuted row list, expert
//                  offsets and the <=128-row tile list of the grouped tcgen05 GEMM (int atomics only,
//                  order inside an expert = ascending pair index, so the result is deterministic).
//   moe_combine  : residual += sum over slots (slot order) of weight * expert output (+ gated shared).
// Reference: engine-rs/shim/qwen_moe.cu:10-92, dataflow.cu:370-572, ds41_ops.cu:375-421 (routers);
// moe_exl3.cuh:141-231 (count/scan/fill), :1085 (slot-order combine).
#include "../common/ptx.cuh"

namespace spark {

constexpr int ROUTE_THREADS = 256;
constexpr int ROUTE_MAXE_PER_THREAD = 4;     // up to 1024 experts

// kind: 0 softmax, 1 sigmoid+bias, 2 sqrt(softplus)+bias
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const float* __restrict__ logits, int ld, int E, int top_k, int kind, const float* __restrict__ bias,
                 float scale, int shared_gate, float* __restrict__ wts, int* __restrict__ ids,
                 int* __restrict__ pair_row, float* __restrict__ sg, int e_lo, int e_hi) {
  __shared__ float rv[ROUTE_THREADS / 32];
  __shared__ int ri[ROUTE_THREADS / 32];
  __shared__ float bv; __shared__ int bidx;
  __shared__ float sel_p[32];
  const int r = blockIdx.x, t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const float* x = logits + static_cast<size_t>(r) * ld;
  float p[ROUTE_MAXE_PER_THREAD], s[ROUTE_MAXE_PER_THREAD];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < ROUTE_MAXE_PER_THREAD; ++j) {
    const int e = t + j * ROUTE_THREADS;
    p[j] = e < E ? x[e] : -INFINITY;
    mx = fmaxf(mx, p[j]);
  }
  if (kind == 0) {
    mx = warp_max(mx);
    if (lane == 0) rv[warp] = mx;
    __syncthreads();
    mx = rv[0];
    for (int w = 1; w < ROUTE_THREADS / 32; ++w) mx = fmaxf(mx, rv[w]);
    __syncthreads();
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAXE_PER_THREAD; ++j) {
      const int e = t + j * ROUTE_THREADS;
      p[j] = e < E ? expf(p[j] - mx) : 0.f;
      sum += p[j];
    }
    sum = warp_sum(sum);
    if (lane == 0) rv[warp] = sum;
    __syncthreads();
    sum = 0.f;
    for (int w = 0; w < ROUTE_THREADS / 32; ++w) sum += rv[w];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < ROUTE_MAXE_PER_THREAD; ++j) { p[j] = p[j] / sum; s[j] = p[j]; }
  } else {
#pragma unroll
    for (int j = 0; j < ROUTE_MAXE_PER_THREAD; ++j) {
      const int e = t + j * ROUTE_THREADS;
      if (e < E) {
        const float v = p[j];
        if (kind == 1) p[j] = 1.f / (1.f + expf(-v));
        else p[j] = sqrtf(v > 20.f ? v : log1pf(expf(v)));
        s[j] = p[j] + (bias ? bias[e] : 0.f);
      } else { p[j] = 0.f; s[j] = -INFINITY; }
    }
  }
#pragma unroll
  for (int j = 0; j < ROUTE_MAXE_PER_THREAD; ++j) if (t + j * ROUTE_THREADS >= E) s[j] = -INFINITY;
  for (int k = 0; k < top_k; ++k) {
    float best = -INFINITY; int bi = 0x7fffffff; float bp = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAXE_PER_THREAD; ++j) {
      const int e = t + j * ROUTE_THREADS;
      if (s[j] > best || (s[j] == best && e < bi && s[j] != -INFINITY)) { best = s[j]; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { rv[warp] = best; ri[warp] = bi; }
    __syncthreads();
    if (t == 0) {
      for (int w = 1; w < ROUTE_THREADS / 32; ++w)
        if (rv[w] > best || (rv[w] == best && ri[w] < bi)) { best = rv[w]; bi = ri[w]; }
      bv = best; bidx = bi;
    }
    __syncthreads();
    const int win = bidx;
    if ((win % ROUTE_THREADS) == t) {
      const int j = win / ROUTE_THREADS;
#pragma unroll
      for (int jj = 0; jj < ROUTE_MAXE_PER_THREAD; ++jj) if (jj == j) { bp = p[jj]; s[jj] = -INFINITY; }
      sel_p[k] = bp;
      // expert-parallel ranks keep only their own experts [e_lo, e_hi): others become -1 (skipped downstream)
      ids[static_cast<size_t>(r) * top_k + k] = (win >= e_lo && win < e_hi) ? win - e_lo : -1;
      if (pair_row) pair_row[static_cast<size_t>(r) * top_k + k] = r;
    }
    __syncthreads();
  }
  if (t == 0) {
    float sum = 0.f;
    for (int k = 0; k < top_k; ++k) sum += sel_p[k];
    sum = fmaxf(sum, 1e-20f);
    for (int k = 0; k < top_k; ++k) wts[static_cast<size_t>(r) * top_k + k] = sel_p[k] / sum * scale;
    if (shared_gate) sg[r] = 1.f / (1.f + expf(-x[E]));
  }
}

// ---------------------------------------------------------------------------------- counting sort
// One CTA.  ids [P] expert per pair (P = R*top_k).  Outputs: perm[P] (pair index in expert order),
// offsets[E+1], tile_list[int4] of <=128-row tiles {row0, row_end, expert, 0}, tile_count.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ perm, int* __restrict__ inv_perm,
                int* __restrict__ offsets, int4* __restrict__ tile_list, int* __restrict__ tile_count) {
  extern __shared__ int sh[];          // counts[E], starts[E+1]
  int* cnt = sh; int* start = sh + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < P; i += blockDim.x) if (ids[i] >= 0) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = acc; offsets[e] = acc;
      for (int r0 = 0; r0 < cnt[e]; r0 += 128) tile_list[nt++] = make_int4(acc + r0, acc + cnt[e], e, 0);
      acc += cnt[e];
    }
    start[E] = acc; offsets[E] = acc; *tile_count = nt;
  }
  __syncthreads();
  // stable placement: pair i goes to start[e] + (number of earlier pairs with the same expert)
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0) { if (inv_perm) inv_perm[i] = -1; continue; }   // not a local expert
    int rank = 0;
    for (int j = 0; j < i; ++j) rank += (ids[j] == e);     // P is small on the decode path
    perm[start[e] + rank] = i;
    if (inv_perm) inv_perm[i] = start[e] + rank;
  }
}

// Prefill-size stable sort: rank of pair i inside its expert = exclusive count over earlier pairs.
// Two passes over blocks of pairs with per-block histograms (deterministic, int atomics only in smem).
__global__ void moe_hist_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ block_hist) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < P && ids[i] >= 0) atomicAdd(&sh[ids[i]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[static_cast<size_t>(blockIdx.x) * E + e] = sh[e];
}
// one CTA: exclusive scan over blocks per expert, expert offsets, tile list
__global__ void __launch_bounds__(1024)
moe_scan_kernel(int* __restrict__ block_hist, int nblocks, int E, int* __restrict__ offsets,
                int4* __restrict__ tile_list, int* __restrict__ tile_count) {
  extern __shared__ int tot[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int acc = 0;
    for (int b = 0; b < nblocks; ++b) { int c = block_hist[static_cast<size_t>(b) * E + e]; block_hist[static_cast<size_t>(b) * E + e] = acc; acc += c; }
    tot[e] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = acc;
      for (int r0 = 0; r0 < tot[e]; r0 += 128) tile_list[nt++] = make_int4(acc + r0, acc + tot[e], e, 0);
      acc += tot[e];
    }
    offsets[E] = acc; *tile_count = nt;
  }
}
__global__ void moe_place_kernel(const int* __restrict__ ids, int P, int E, const int* __restrict__ block_hist,
                                 const int* __restrict__ offsets, int* __restrict__ perm, int* __restrict__ inv_perm) {
  extern __shared__ int sid[];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  sid[threadIdx.x] = i < P ? ids[i] : -1;
  __syncthreads();
  if (i >= P) return;
  const int e = sid[threadIdx.x];
  if (e < 0) { if (inv_perm) inv_perm[i] = -1; return; }
  int rank = 0;
  for (int j = 0; j < threadIdx.x; ++j) rank += (sid[j] == e);
  const int dst = offsets[e] + block_hist[static_cast<size_t>(blockIdx.x) * E + e] + rank;
  perm[dst] = i;
  if (inv_perm) inv_perm[i] = dst;
}

// ---------------------------------------------------------------------------------- combine
// res[R,H] += sum_slot w[r,slot] * y[pair_pos(r,slot), :] (+ sg[r] * shared[r,:]).  y fp32 or bf16.
template <typename TY>
__global__ void moe_combine_kernel(float* __restrict__ res, const TY* __restrict__ y, const int* __restrict__ inv_perm,
                                   const float* __restrict__ wts, int top_k, const __nv_bfloat16* __restrict__ shared,
                                   const float* __restrict__ sg, int H, __nv_bfloat16* __restrict__ out_bf16,
                                   const int* __restrict__ pair_expert) {
  const int r = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
#pragma unroll 4
    for (int k = 0; k < top_k; ++k) {
      const int pi = r * top_k + k;
      if (pair_expert && pair_expert[pi] < 0) continue;          // expert lives on another rank
      const int row = inv_perm ? inv_perm[pi] : pi;
      acc = fmaf(wts[pi], static_cast<float>(y[static_cast<size_t>(row) * H + i]), acc);
    }
    if (shared) {
      const float s = __bfloat162float(shared[static_cast<size_t>(r) * H + i]);
      acc += sg ? sg[r] * s : s;
    }
    if (res) res[static_cast<size_t>(r) * H + i] += acc;
    if (out_bf16) out_bf16[static_cast<size_t>(r) * H + i] = __float2bfloat16(acc);
  }
}

}  // namespace spark

using namespace spark;

extern "C" int spark_moe_route(const float* logits, int ld, int R, int E, int top_k, int kind, const float* bias,
                               float scale, int shared_gate, float* wts, int* ids, int* pair_row, float* sg,
                               cudaStream_t s, int e_lo, int e_hi) {
  if (R <= 0) return 0;
  if (E > ROUTE_THREADS * ROUTE_MAXE_PER_THREAD || top_k > 32) return -5;
  moe_route_kernel<<<R, ROUTE_THREADS, 0, s>>>(logits, ld, E, top_k, kind, bias, scale, shared_gate, wts, ids, pair_row, sg, e_lo, e_hi);
  return spark_launch_rc(__func__);
}

// Scratch `block_hist` must hold ceil(P/256) * E ints when P > 2048.
extern "C" int spark_moe_sort(const int* ids, int P, int E, int* perm, int* inv_perm, int* offsets, void* tile_list,
                              int* tile_count, int* block_hist, cudaStream_t s) {
  if (P <= 0) return 0;
  if (P <= 2048) {
    moe_sort_kernel<<<1, 1024, (2 * E + 1) * sizeof(int), s>>>(ids, P, E, perm, inv_perm, offsets, (int4*)tile_list, tile_count);
  } else {
    const int nb = (P + 255) / 256;
    moe_hist_kernel<<<nb, 256, E * sizeof(int), s>>>(ids, P, E, block_hist);
    moe_scan_kernel<<<1, 1024, E * sizeof(int), s>>>(block_hist, nb, E, offsets, (int4*)tile_list, tile_count);
    moe_place_kernel<<<nb, 256, 256 * sizeof(int), s>>>(ids, P, E, block_hist, offsets, perm, inv_perm);
  }
  return spark_launch_rc(__func__);
}

extern "C" int spark_moe_combine(float* res, const void* y, int y_f32, const int* inv_perm, const float* wts, int R,
                                 int top_k, const void* shared, const float* sg, int H, void* out_bf16, cudaStream_t s,
                                 const int* pair_expert) {
  if (R <= 0) return 0;
  if (y_f32)
    moe_combine_kernel<float><<<dim3(R, (H + 255) / 256), 256, 0, s>>>(res, (const float*)y, inv_perm, wts, top_k, (const __nv_bfloat16*)shared, sg, H,
                                                (__nv_bfloat16*)out_bf16, pair_expert);
  else
    moe_combine_kernel<__nv_bfloat16><<<dim3(R, (H + 255) / 256), 256, 0, s>>>(res, (const __nv_bfloat16*)y, inv_perm, wts, top_k,
                                                        (const __nv_bfloat16*)shared, sg, H, (__nv_bfloat16*)out_bf16, pair_expert);
  return spark_launch_rc(__func__);
}
