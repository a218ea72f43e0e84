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
#include "../common/decode.cuh"

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


// ---------------------------------------------------------------------------------- decode router (fused)
// One launch for <= 16 rows: router GEMV over the E (+1 shared-gate) columns, then the CTA that finishes last
// (integer arrival counter, nobody waits) scores, picks the top-k experts of every row with one warp per row and
// writes the pair tables the expert GEMVs read: ids / weights / source row for top_k routed slots plus an optional
// shared-expert slot (the shared expert is stored as one more matrix of the expert stack, so it is just another
// pair; under tensor parallelism row r's shared pair belongs to rank r % world).
// Replaces three launches (norm, GEMV, route); reference: engine-rs/shim/qwen_moe.cu:10-92, dataflow.cu:370-572.
struct RouterArgs {
  const __nv_bfloat16* x; int ldx;           // [R, K]
  const __nv_bfloat16* Wg; int ldw;          // [E (+1), K]
  float* logits; int ld;                     // scratch [R, ld]
  int R, K, E, top_k, kind;                  // kind: 0 softmax, 1 sigmoid+bias, 2 sqrt(softplus)+bias
  const float* bias; float scale; int shared_gate;
  int slots;                                 // top_k, or top_k + 1 when the shared expert is a pair
  int shared_expert;                         // index of the shared expert in the local stack (slot top_k)
  int e_lo, e_hi, rank, world;
  float* wts; int* ids; int* pair_row;       // [R, slots]
  float* sg;                                 // optional [R]: shared gate (when the shared expert is NOT a pair)
  int* counter;
};

constexpr int ROUTER_RB = 16;

template <int EPL>
__global__ void __launch_bounds__(256)
moe_router_topk_kernel(const __grid_constant__ RouterArgs a) {
  extern __shared__ __align__(16) uint8_t smem_router[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_router);     // [R][K]
  __shared__ int last_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int R = a.R, K = a.K;
  // the gate matrix depends on no earlier launch: its first batch of loads is in flight before the dependency wait
  const int NE = a.E + (a.shared_gate ? 1 : 0);
  const int n0 = blockIdx.x * 8 + warp;                    // one gate column per warp
  const uint4* w0 = reinterpret_cast<const uint4*>(a.Wg + static_cast<size_t>(n0 < NE ? n0 : 0) * a.ldw);
  constexpr int BATCH = 8;                                 // weight loads in flight per lane
  const int KV = K >> 3;
  uint4 wa[BATCH];
#pragma unroll
  for (int u = 0; u < BATCH; ++u) {
    const int kv = lane + 32 * u;
    wa[u] = kv < KV ? __ldg(w0 + kv) : make_uint4(0u, 0u, 0u, 0u);
  }
  pdl_wait();
  pdl_trigger();
  const int KV8 = K >> 3;
  for (int i = tid; i < R * KV8; i += 256) {
    const int r = i / KV8, kv = i - r * KV8;
    reinterpret_cast<uint4*>(xs)[i] = *reinterpret_cast<const uint4*>(a.x + static_cast<size_t>(r) * a.ldx + kv * 8);
  }
  __syncthreads();
  // ---- GEMV: this CTA's 8 gate columns (one per warp), all rows; one warp per output => fixed reduction order
  if (n0 < NE) {
    float acc0[ROUTER_RB];
#pragma unroll
    for (int r = 0; r < ROUTER_RB; ++r) acc0[r] = 0.f;
    for (int kv0 = lane; kv0 < KV; kv0 += 32 * BATCH) {
      if (kv0 != lane) {
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
          const int kv = kv0 + 32 * u;
          wa[u] = kv < KV ? __ldg(w0 + kv) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int kv = kv0 + 32 * u;
        if (kv >= KV) break;
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&wa[u]);
        float fa[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t0 = __bfloat1622float2(pa[i]);
          fa[2 * i] = t0.x; fa[2 * i + 1] = t0.y;
        }
#pragma unroll
        for (int r = 0; r < ROUTER_RB; ++r) {
          if (r < R) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(r) * K + kv * 8);
            const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 t = __bfloat1622float2(px[i]);
              acc0[r] = fmaf(fa[2 * i], t.x, acc0[r]); acc0[r] = fmaf(fa[2 * i + 1], t.y, acc0[r]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < ROUTER_RB; ++r) {
      if (r < R) {
        const float s0 = warp_sum(acc0[r]);
        if (lane == 0) a.logits[static_cast<size_t>(r) * a.ld + n0] = s0;
      }
    }
  }
  // ---- arrival: the last CTA to get here routes every row
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int old = atomicAdd(a.counter, 1);
    last_s = old == static_cast<int>(gridDim.x) - 1;
    if (last_s) *a.counter = 0;
  }
  __syncthreads();
  if (!last_s) return;
  // (the writers fenced before they arrived; the logits are read with L2 loads, so no reader-side fence)
  // EPL experts per lane (E <= 32 * EPL).  The k selection rounds are a serial chain, so each round is kept short: the
  // lane's best candidate comes from a max TREE over its EPL scores and a bit mask of the positions that hold it
  // (lowest position = lowest expert id), not from a serial compare chain (timed inside the kernel: the serial form spent 5.8 us per group of rows).
  const int nj = (a.E + 31) >> 5;
  auto lane_best = [&](const float (&s)[EPL], float& best, int& bj) {
    float m[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) m[j] = s[j];
#pragma unroll
    for (int w = EPL / 2; w >= 1; w >>= 1)
#pragma unroll
      for (int j = 0; j < w; ++j) m[j] = fmaxf(m[j], m[j + w]);
    best = m[0];
    unsigned mask = 0u;
#pragma unroll
    for (int j = 0; j < EPL; ++j) mask |= (s[j] == best ? 1u : 0u) << j;
    bj = __ffs(mask) - 1;
    if (bj < 0) bj = 0;
  };
  for (int r = warp; r < R; r += 8) {
    const float* lg = a.logits + static_cast<size_t>(r) * a.ld;
    float p[EPL], s[EPL];                                   // p: what the weights are made of; s: selection score
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = lane + 32 * j;
      p[j] = (j < nj && e < a.E) ? __ldcg(lg + e) : -INFINITY;
      s[j] = p[j];
      mx = fmaxf(mx, p[j]);
    }
    if (a.kind == 0) {
      // softmax -> top-k -> renormalise: the softmax denominator cancels, so experts are ranked by their logits and
      // only the k winners are exponentiated
      mx = warp_max(mx);
    } else {
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const int e = lane + 32 * j;
        if (j < nj && e < a.E) {
          const float v = p[j];
          p[j] = a.kind == 1 ? 1.f / (1.f + expf(-v)) : sqrtf(v > 20.f ? v : log1pf(expf(v)));
          s[j] = p[j] + (a.bias ? a.bias[e] : 0.f);
        } else { p[j] = 0.f; s[j] = -INFINITY; }
      }
    }
    float selp = 0.f; int seli = -1;                        // lane k keeps slot k's weight numerator and expert
    float tot = 0.f;
    // A round: warp maximum of the candidates' order-preserving integer keys (one redux), lowest expert id among the
    // lanes that hold it (one redux), the winning lane takes its expert out and finds its next best.
    float best; int bj;
    lane_best(s, best, bj);
    for (int k = 0; k < a.top_k; ++k) {
      const uint32_t bits = __float_as_uint(best);
      const uint32_t key = best == -INFINITY ? 0u : (bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u));
      const uint32_t wmax = __reduce_max_sync(0xffffffffu, key);
      const int cand = (key == wmax && key != 0u) ? lane + 32 * bj : 0x7fffffff;
      const int wi = __reduce_min_sync(0xffffffffu, cand);
      float bp = 0.f;
      if (wi == cand && wi != 0x7fffffff) {                 // this lane owns the winner
#pragma unroll
        for (int j = 0; j < EPL; ++j) if (j == bj) { bp = p[j]; s[j] = -INFINITY; }
        if (a.kind == 0) bp = __expf(bp - mx);
        lane_best(s, best, bj);
      }
      const float wp = __shfl_sync(0xffffffffu, bp, wi & 31);
      if (lane == k) { selp = wp; seli = wi; }
      tot += wp;                                            // slot order, identical on every lane
    }
    tot = fmaxf(tot, 1e-20f);
    const size_t o = static_cast<size_t>(r) * a.slots;
    if (lane < a.top_k) {
      a.wts[o + lane] = selp / tot * a.scale;
      a.ids[o + lane] = (seli >= a.e_lo && seli < a.e_hi) ? seli - a.e_lo : -1;
      if (a.pair_row) a.pair_row[o + lane] = r;
    }
    if (lane == 0) {
      const float g = a.shared_gate ? 1.f / (1.f + __expf(-__ldcg(lg + a.E))) : 1.f;
      if (a.slots > a.top_k) {
        a.wts[o + a.top_k] = g;
        a.ids[o + a.top_k] = (r % a.world) == a.rank ? a.shared_expert : -1;
        if (a.pair_row) a.pair_row[o + a.top_k] = r;
      }
      if (a.sg) a.sg[r] = g;
    }
  }
}

// Decode combine fused with the residual update and the next RMSNorm: one CTA per row.
//   res[r] += sum over slots (slot order) of weight * y[pair] (+ gated shared);  h[r] = rmsnorm(res[r]) * w  (bf16)
// Replaces combine + add_rmsnorm (two launches); reference: engine-rs/shim/moe_exl3.cuh:1381 finish_combine_kernel.
__global__ void __launch_bounds__(1024)
moe_combine_norm_kernel(const float* __restrict__ y, const float* __restrict__ wts, const int* __restrict__ ids, int slots,
                        int H, float* __restrict__ res, const float* __restrict__ norm_w, float eps, int one_plus,
                        __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ shared,
                        const float* __restrict__ sg) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  float4 keep[2];                                          // H <= 2 * 4 * blockDim.x
  float ss = 0.f;
  int ki = 0;
  for (int col = threadIdx.x * 4; col < H; col += blockDim.x * 4, ++ki) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < slots; k0 += 4) {                // four slots' loads in flight; summed in slot order
      float4 v[4]; float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int pi = r * slots + k0 + u;
        const bool live = (k0 + u) < slots && ids[pi] >= 0;
        w[u] = live ? wts[pi] : 0.f;
        v[u] = live ? __ldcg(reinterpret_cast<const float4*>(y + static_cast<size_t>(pi) * H + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        acc.x = fmaf(w[u], v[u].x, acc.x); acc.y = fmaf(w[u], v[u].y, acc.y);
        acc.z = fmaf(w[u], v[u].z, acc.z); acc.w = fmaf(w[u], v[u].w, acc.w);
      }
    }
    if (shared) {
      const uint2 raw = *reinterpret_cast<const uint2*>(shared + static_cast<size_t>(r) * H + col);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 f0 = __bfloat1622float2(p2[0]), f1 = __bfloat1622float2(p2[1]);
      const float g = sg ? sg[r] : 1.f;
      acc.x += g * f0.x; acc.y += g * f0.y; acc.z += g * f1.x; acc.w += g * f1.y;
    }
    float* rp = res + static_cast<size_t>(r) * H + col;
    float4 o4 = *reinterpret_cast<const float4*>(rp);
    o4.x += acc.x; o4.y += acc.y; o4.z += acc.z; o4.w += acc.w;
    *reinterpret_cast<float4*>(rp) = o4;
    ss += o4.x * o4.x + o4.y * o4.y + o4.z * o4.z + o4.w * o4.w;
    if (ki < 2) keep[ki] = o4;
  }
  ss = warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < nw; ++w) tot += red[w];              // fixed order
  const float rs = rsqrtf(tot / H + eps);
  ki = 0;
  for (int col = threadIdx.x * 4; col < H; col += blockDim.x * 4, ++ki) {
    const float4 v = keep[ki < 2 ? ki : 1];
    const float4 g = *reinterpret_cast<const float4*>(norm_w + col);
    const float o = one_plus ? 1.f : 0.f;
    __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x * rs * (g.x + o), v.y * rs * (g.y + o));
    __nv_bfloat162 b1 = __floats2bfloat162_rn(v.z * rs * (g.z + o), v.w * rs * (g.w + o));
    uint2 ov; ov.x = *reinterpret_cast<uint32_t*>(&b0); ov.y = *reinterpret_cast<uint32_t*>(&b1);
    *reinterpret_cast<uint2*>(h + static_cast<size_t>(r) * H + col) = ov;
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
// one CTA: exclusive scan over blocks per expert, expert offsets, tile list.  Every step is parallel over the experts
// (two block-wide scans: rows per expert -> offsets, tiles per expert -> first tile), each expert's thread writes its
// own tiles; a single thread walking the 512 experts took 72 us per layer of a prefill chunk.
__global__ void __launch_bounds__(1024)
moe_scan_kernel(int* __restrict__ block_hist, int nblocks, int E, int* __restrict__ offsets,
                int4* __restrict__ tile_list, int* __restrict__ tile_count) {
  extern __shared__ int tot[];                         // [E]
  __shared__ int sa[1024], sb[1024];
  const int e = threadIdx.x;
  int mine = 0;
  if (e < E) {
    int acc = 0;
    for (int b = 0; b < nblocks; ++b) { int c = block_hist[static_cast<size_t>(b) * E + e]; block_hist[static_cast<size_t>(b) * E + e] = acc; acc += c; }
    tot[e] = acc;
    mine = acc;
  }
  const int my_tiles = (mine + 127) / 128;
  sa[e] = mine; sb[e] = my_tiles;
  __syncthreads();
  for (int st = 1; st < 1024; st <<= 1) {               // inclusive scans of rows and of tiles
    const int a = e >= st ? sa[e - st] : 0, b = e >= st ? sb[e - st] : 0;
    __syncthreads();
    sa[e] += a; sb[e] += b;
    __syncthreads();
  }
  if (e < E) {
    const int off = sa[e] - mine, t0 = sb[e] - my_tiles;
    offsets[e] = off;
    for (int i = 0; i < my_tiles; ++i) tile_list[t0 + i] = make_int4(off + i * 128, off + mine, e, 0);
    if (e == E - 1) { offsets[E] = sa[e]; *tile_count = sb[e]; }
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
  if (E > 1024) return -5;                     // one thread per expert in the scan
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

// Fused decode router: see moe_router_topk_kernel.  `logits` scratch [R, ld] fp32 (ld >= E + 1), `counter` one int
// that is zero between launches.  x bf16 [R, K].
extern "C" int spark_moe_router_topk(const void* x, int ldx, const void* Wg, int ldw, float* logits,
                                     int ld, int R, int K, int E, int top_k, int kind, const float* bias, float scale,
                                     int shared_gate, int slots, int shared_expert, int e_lo, int e_hi, int rank, int world,
                                     float* wts, int* ids, int* pair_row, float* sg, int* counter, cudaStream_t s) {
  if (R <= 0) return 0;
  if (R > ROUTER_RB || E > 1024 || top_k > 32 || (K & 7) || slots < top_k || slots > top_k + 1 || ld < E + (shared_gate ? 1 : 0))
    return -5;
  RouterArgs a;
  a.x = (const __nv_bfloat16*)x; a.ldx = ldx;
  a.Wg = (const __nv_bfloat16*)Wg; a.ldw = ldw; a.logits = logits; a.ld = ld;
  a.R = R; a.K = K; a.E = E; a.top_k = top_k; a.kind = kind; a.bias = bias; a.scale = scale; a.shared_gate = shared_gate;
  a.slots = slots; a.shared_expert = shared_expert; a.e_lo = e_lo; a.e_hi = e_hi; a.rank = rank; a.world = world < 1 ? 1 : world;
  a.wts = wts; a.ids = ids; a.pair_row = pair_row; a.sg = sg; a.counter = counter;
  const int NE = E + (shared_gate ? 1 : 0);
  const size_t smem = static_cast<size_t>(R) * K * 2;
  if (smem > 200 * 1024) return -6;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(moe_router_topk_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(moe_router_topk_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_set = true;
  }
  const cudaError_t err = E <= 512
      ? spark_launch_pdl(moe_router_topk_kernel<16>, dim3((NE + 7) / 8), dim3(256), smem, s, dim3(1, 1, 1), a)
      : spark_launch_pdl(moe_router_topk_kernel<32>, dim3((NE + 7) / 8), dim3(256), smem, s, dim3(1, 1, 1), a);
  return err == cudaSuccess ? 0 : -4;
}

// res fp32 [R, H] (in/out), h bf16 [R, H] out; y fp32 [R * slots, H] in pair order.
extern "C" int spark_moe_combine_norm(const float* y, const float* wts, const int* ids, int R, int slots, int H, float* res,
                                      const float* norm_w, float eps, int one_plus, void* h, const void* shared,
                                      const float* sg, cudaStream_t s) {
  if (R <= 0) return 0;
  int th = H / 4;
  if (H % 128 || th > 2048) return -5;
  if (th > 1024) th = 1024;
  const cudaError_t err = spark_launch_pdl(moe_combine_norm_kernel, dim3(R), dim3(th), 0, s, dim3(1, 1, 1), y, wts, ids, slots, H,
                                           res, norm_w, eps, one_plus, (__nv_bfloat16*)h, (const __nv_bfloat16*)shared, sg);
  return err == cudaSuccess ? 0 : -4;
}
