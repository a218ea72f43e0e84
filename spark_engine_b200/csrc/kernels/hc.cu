// Hyper-connection sites: the residual is S parallel streams [T, S, D] (fp32); every block reads ONE mixed row and
// writes its output back into all streams.
//
//   mHC (GLM-style):   m = (flat(res) . fn^T) * rsqrt(mean(flat^2) + eps)              2S + S^2 logits per row
//                      pre = sigmoid(m[:S] s0 + b) + 1e-6, post = 2 sigmoid(m[S:2S] s1 + b),
//                      comb = sinkhorn(softmax(m[2S:] s2 + b) + 1e-6, iters)
//                      layer_in = rmsnorm(sum_s pre[s] res[s]) * norm
//                      after the block: res'[j] = sum_i comb[i][j] res[i] + post[j] x
//   gated HC (Qwen-style): n = rms(res) (1 + norm); t = silu(flat(n) . down^T / S); post = 2 sigmoid(flat(n) . inject^T / S)
//                      g = sigmoid(t . up^T); layer_in = mean_s(g n); after the block: res'[s] = res[s] + post[s] x
//
// One kernel per site does [apply the previous site's update] -> [this site's logits] in a single pass over the
// streams: grid (row, chunk of D, group of logits); a CTA forms its chunk of the updated streams in registers (one
// CTA of the chunk stores them, out of place), accumulates its share of the logits, and the LAST CTA of a row to
// arrive (ticket counter, no CTA ever waits on another) sums the partials in chunk order (deterministic), runs the
// S x S Sinkhorn on 16 lanes and produces the mixed row.  The gated site needs the logits before it can form g, so
// its mixed row is a second launch.
// Reference: shim/mhc.cu:27-517 (pre/post, Sinkhorn(20)), qwen_hc.cu:23-477, ds41_hc.cu:27-355, glm53/mhc.py:31-60,
// qwen38/model.py:65-82.
#include "../common/decode.cuh"

namespace spark {

constexpr int HC_S = 4;                 // streams
constexpr int HC_NL = 2 * HC_S + HC_S * HC_S;
constexpr int HC_THREADS = 128;
constexpr int HC_DC = HC_THREADS * 4;   // columns of D per CTA
constexpr int HC_ZG = 3;                // CTAs that share one chunk of a row, each owning HC_NL / HC_ZG logits
constexpr int HC_LG = HC_NL / HC_ZG;    // logits per CTA

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

template <int N>
__device__ __forceinline__ void block_sum(float (&v)[N], float* red /* [4][N] */) {
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int o = 16; o; o >>= 1) v[i] += __shfl_xor_sync(~0u, v[i], o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0)
#pragma unroll
    for (int i = 0; i < N; ++i) red[w * N + i] = v[i];
  __syncthreads();
  if (threadIdx.x == 0)
#pragma unroll
    for (int i = 0; i < N; ++i) {
      float s = 0.f;
      for (int k = 0; k < HC_THREADS / 32; ++k) s += red[k * N + i];
      red[i] = s;
    }
  __syncthreads();
}

__device__ __forceinline__ float4 ld_x4(const void* x, int x_f32, size_t i) {
  if (x_f32) return *reinterpret_cast<const float4*>(static_cast<const float*>(x) + i);
  const uint2 r = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(x) + i);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 ld_w4(const __nv_bfloat16* w, size_t i) { return ld_x4(w, 0, i); }

// ------------------------------------------------------------------------------------------------ mHC
// mode: 0 = update only (no next site), 1 = full pre (logits, Sinkhorn, contraction, RMSNorm), 2 = stream mean + RMSNorm
struct MhcArgs {
  const float* res;           // [T, S, D] streams before the pending update
  const void* x;              // [T, D] block output of the previous site (nullptr: no update)
  int x_f32;
  const float* post_in;       // [T, S]
  const float* comb_in;       // [T, S, S]
  const __nv_bfloat16* fn;    // [NL, S*D]
  const float* scale;         // [3]
  const float* base;          // [NL]
  const float* norm;          // [D]
  __nv_bfloat16* h;           // [T, D] mixed, normed row
  float* mean_out;            // mode 2: [T, D] fp32 stream mean
  float* post_out;            // [T, S]
  float* comb_out;            // [T, S, S]
  float* partial;             // [T, NS, NL + 1]
  int* counter;               // [T], zero; the last CTA resets it
  float* res_out;             // [T, S, D] updated streams (written when x != nullptr; several CTAs read one chunk of
                              // `res`, so the update is never in place)
  int D, iters, mode;
  float eps;
};

__global__ void __launch_bounds__(HC_THREADS) mhc_site_kernel(MhcArgs a) {
  extern __shared__ float sm[];                       // [D] mixed row of the finishing CTA
  __shared__ float red[(HC_THREADS / 32) * (HC_LG + 1)];
  __shared__ float msum[HC_NL + 1];
  __shared__ float pre_s[HC_S];
  __shared__ int last_s;
  // grid (row, chunk of D, logit group): the groups of a chunk all form the updated streams in registers, group 0 stores them
  const int row = blockIdx.x, c = blockIdx.y, zg = blockIdx.z, NS = gridDim.y, NZ = gridDim.z, D = a.D, t = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  const float* R = a.res + static_cast<size_t>(row) * HC_S * D;
  float comb[HC_S][HC_S], post[HC_S];
  if (a.x != nullptr) {
#pragma unroll
    for (int i = 0; i < HC_S; ++i) {
      post[i] = a.post_in[row * HC_S + i];
#pragma unroll
      for (int j = 0; j < HC_S; ++j) comb[i][j] = a.comb_in[(row * HC_S + i) * HC_S + j];
    }
  }
  float acc[HC_LG + 1];
#pragma unroll
  for (int l = 0; l <= HC_LG; ++l) acc[l] = 0.f;
  const int d = c * HC_DC + t * 4;
  if (d < D) {
    float4 v[HC_S];
#pragma unroll
    for (int s = 0; s < HC_S; ++s) v[s] = *reinterpret_cast<const float4*>(R + static_cast<size_t>(s) * D + d);
    if (a.x != nullptr) {
      const float4 xv = ld_x4(a.x, a.x_f32, static_cast<size_t>(row) * D + d);
      float4 n[HC_S];
#pragma unroll
      for (int j = 0; j < HC_S; ++j) {
        n[j] = make_float4(post[j] * xv.x, post[j] * xv.y, post[j] * xv.z, post[j] * xv.w);
#pragma unroll
        for (int i = 0; i < HC_S; ++i) {
          n[j].x += comb[i][j] * v[i].x; n[j].y += comb[i][j] * v[i].y;
          n[j].z += comb[i][j] * v[i].z; n[j].w += comb[i][j] * v[i].w;
        }
      }
#pragma unroll
      for (int s = 0; s < HC_S; ++s) v[s] = n[s];
    }
    if (a.mode == 1) {
      float4 w[HC_S][HC_LG];                            // all of this thread's weight loads in flight together
#pragma unroll
      for (int s = 0; s < HC_S; ++s)
#pragma unroll
        for (int l = 0; l < HC_LG; ++l) w[s][l] = ld_w4(a.fn, (static_cast<size_t>(zg * HC_LG + l) * HC_S + s) * D + d);
#pragma unroll
      for (int s = 0; s < HC_S; ++s) {
        acc[HC_LG] += v[s].x * v[s].x + v[s].y * v[s].y + v[s].z * v[s].z + v[s].w * v[s].w;
#pragma unroll
        for (int l = 0; l < HC_LG; ++l) acc[l] += v[s].x * w[s][l].x + v[s].y * w[s][l].y + v[s].z * w[s][l].z + v[s].w * w[s][l].w;
      }
    }
    if (a.x != nullptr && zg == 0) {
      float* W = a.res_out + static_cast<size_t>(row) * HC_S * D;
#pragma unroll
      for (int s = 0; s < HC_S; ++s) *reinterpret_cast<float4*>(W + static_cast<size_t>(s) * D + d) = v[s];
    }
  }
  if (a.mode == 0) return;
  if (a.mode == 1) {
    block_sum<HC_LG + 1>(acc, red);
    float* P = a.partial + (static_cast<size_t>(row) * NS + c) * (HC_NL + 1);
    if (t < HC_LG) P[zg * HC_LG + t] = red[t];
    if (t == HC_LG && zg == 0) P[HC_NL] = red[HC_LG];
  }
  __threadfence();
  __syncthreads();
  if (t == 0) last_s = (atomicAdd(a.counter + row, 1) == NS * NZ - 1);
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const float* Rn = a.x != nullptr ? a.res_out + static_cast<size_t>(row) * HC_S * D : R;
  if (t == 0) a.counter[row] = 0;
  if (a.mode == 1) {
    if (t <= HC_NL) {
      float s = 0.f;
      for (int k = 0; k < NS; ++k) s += __ldcg(a.partial + (static_cast<size_t>(row) * NS + k) * (HC_NL + 1) + t);
      msum[t] = s;
    }
    __syncthreads();
    const float inv = rsqrtf(msum[HC_NL] / static_cast<float>(HC_S * D) + a.eps);
    if (t < HC_S) {
      pre_s[t] = sigmoidf_(msum[t] * inv * a.scale[0] + a.base[t]) + 1e-6f;
      a.post_out[row * HC_S + t] = 2.f * sigmoidf_(msum[HC_S + t] * inv * a.scale[1] + a.base[HC_S + t]);
    }
    if (t < 32) {
      // Sinkhorn on 16 lanes: lane = i * S + j holds comb[i][j]; row sums run over j (xor 1, 2), column sums over i (xor 4, 8)
      const int e = t & 15;
      float z = msum[2 * HC_S + e] * inv * a.scale[2] + a.base[2 * HC_S + e];
      float mx = fmaxf(z, __shfl_xor_sync(~0u, z, 1));
      mx = fmaxf(mx, __shfl_xor_sync(~0u, mx, 2));
      float p = expf(z - mx);
      float sum = p + __shfl_xor_sync(~0u, p, 1);
      sum += __shfl_xor_sync(~0u, sum, 2);
      float cb = p / sum + 1e-6f;
      float cs = cb + __shfl_xor_sync(~0u, cb, 4);
      cs += __shfl_xor_sync(~0u, cs, 8);
      cb /= (cs + 1e-6f);
      for (int it = 1; it < a.iters; ++it) {
        float rs = cb + __shfl_xor_sync(~0u, cb, 1);
        rs += __shfl_xor_sync(~0u, rs, 2);
        cb /= (rs + 1e-6f);
        cs = cb + __shfl_xor_sync(~0u, cb, 4);
        cs += __shfl_xor_sync(~0u, cs, 8);
        cb /= (cs + 1e-6f);
      }
      if (t < 16) a.comb_out[row * HC_S * HC_S + e] = cb;
    }
  } else if (t < HC_S) {
    pre_s[t] = 1.f / HC_S;
  }
  __syncthreads();
  // the mixed row: sum_s pre[s] res'[s] (the other CTAs' chunks come through L2), then RMSNorm
  float ss[1] = {0.f};
  for (int i = t * 4; i < D; i += HC_THREADS * 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < HC_S; ++s) {
      const float4 x = __ldcg(reinterpret_cast<const float4*>(Rn + static_cast<size_t>(s) * D + i));
      v.x += pre_s[s] * x.x; v.y += pre_s[s] * x.y; v.z += pre_s[s] * x.z; v.w += pre_s[s] * x.w;
    }
    *reinterpret_cast<float4*>(sm + i) = v;
    ss[0] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  block_sum<1>(ss, red);
  const float r = rsqrtf(red[0] / static_cast<float>(D) + a.eps);
  for (int i = t; i < D; i += HC_THREADS) {
    a.h[static_cast<size_t>(row) * D + i] = __float2bfloat16(sm[i] * r * a.norm[i]);
    if (a.mode == 2) a.mean_out[static_cast<size_t>(row) * D + i] = sm[i];
  }
}

// ------------------------------------------------------------------------------------------------ gated HC
constexpr int GH_R = 32;                // rank of the gate's bottleneck
constexpr int GH_NL = GH_R + HC_S;      // down rows + inject rows

constexpr int GH_ZG = 4;                // CTAs that share one chunk of a row
constexpr int GH_LG = GH_NL / GH_ZG;    // gate / inject rows per CTA

struct GatedArgs {
  const float* res;           // [T, S, D] streams before the pending update
  float* res_out;             // [T, S, D] updated streams (written when x != nullptr, never in place)
  const void* x;              // [T, D] previous block output (nullptr: no update)
  int x_f32;
  const float* post_in;       // [T, S]
  const float* norm;          // [S, D]
  const __nv_bfloat16* down;  // [GH_R, S*D]
  const __nv_bfloat16* inject;  // [S, S*D] or nullptr
  const __nv_bfloat16* up;    // [S*D, GH_R]
  float* tvec;                // [T, GH_R + S]: t, then the per-stream rms factors
  float* post_out;            // [T, S]
  __nv_bfloat16* h;           // [T, D] bf16 mixed row
  float* h_f32;               // optional fp32 copy of the mixed row
  float* partial;             // [T, NS, GH_NL * S + S]
  int* counter;
  int D;
  float eps;
};

// pass 1: update, per-stream square sums and per-stream partial dots; the last CTA folds the rms factors in
__global__ void __launch_bounds__(HC_THREADS) hc_gated_logits_kernel(GatedArgs a) {
  constexpr int NA = GH_NL * HC_S + HC_S;          // a row's partial record: [row l][stream s] dots, then S square sums
  constexpr int NC = GH_LG * HC_S + HC_S;          // what one CTA accumulates
  __shared__ float red[(HC_THREADS / 32) * NC];
  __shared__ float tot[NA];
  __shared__ int last_s;
  const int row = blockIdx.x, c = blockIdx.y, zg = blockIdx.z, NS = gridDim.y, D = a.D, t = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  const float* R = a.res + static_cast<size_t>(row) * HC_S * D;
  float acc[NC];
#pragma unroll
  for (int l = 0; l < NC; ++l) acc[l] = 0.f;
  const int d = c * HC_DC + t * 4;
  const int nl = a.inject != nullptr ? GH_NL : GH_R;
  if (d < D) {
    float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.x != nullptr) xv = ld_x4(a.x, a.x_f32, static_cast<size_t>(row) * D + d);
    float4 w[GH_LG];
#pragma unroll
    for (int s = 0; s < HC_S; ++s) {
#pragma unroll
      for (int q = 0; q < GH_LG; ++q) {
        const int l = zg * GH_LG + q;
        if (l < nl) {
          const __nv_bfloat16* wrow = l < GH_R ? a.down + (static_cast<size_t>(l) * HC_S + s) * D
                                               : a.inject + (static_cast<size_t>(l - GH_R) * HC_S + s) * D;
          w[q] = ld_w4(wrow, d);
        } else {
          w[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      float4 v = *reinterpret_cast<const float4*>(R + static_cast<size_t>(s) * D + d);
      if (a.x != nullptr) {
        const float p = a.post_in[row * HC_S + s];
        v.x += p * xv.x; v.y += p * xv.y; v.z += p * xv.z; v.w += p * xv.w;
        if (zg == 0) *reinterpret_cast<float4*>(a.res_out + (static_cast<size_t>(row) * HC_S + s) * D + d) = v;
      }
      acc[GH_LG * HC_S + s] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      const float4 g = *reinterpret_cast<const float4*>(a.norm + static_cast<size_t>(s) * D + d);
      v.x *= 1.f + g.x; v.y *= 1.f + g.y; v.z *= 1.f + g.z; v.w *= 1.f + g.w;
#pragma unroll
      for (int q = 0; q < GH_LG; ++q) acc[q * HC_S + s] += v.x * w[q].x + v.y * w[q].y + v.z * w[q].z + v.w * w[q].w;
    }
  }
  block_sum<NC>(acc, red);
  float* P = a.partial + (static_cast<size_t>(row) * NS + c) * NA;
  if (t < GH_LG * HC_S) P[zg * GH_LG * HC_S + t] = red[t];
  if (zg == 0 && t >= GH_LG * HC_S && t < NC) P[GH_NL * HC_S + (t - GH_LG * HC_S)] = red[t];
  __threadfence();
  __syncthreads();
  if (t == 0) last_s = (atomicAdd(a.counter + row, 1) == NS * static_cast<int>(gridDim.z) - 1);
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  for (int i = t; i < NA; i += HC_THREADS) {
    float s = 0.f;
    for (int k = 0; k < NS; ++k) s += __ldcg(a.partial + (static_cast<size_t>(row) * NS + k) * NA + i);
    tot[i] = s;
  }
  __syncthreads();
  if (t < GH_NL) {
    float dot = 0.f;
#pragma unroll
    for (int s = 0; s < HC_S; ++s) dot += tot[t * HC_S + s] * rsqrtf(tot[GH_NL * HC_S + s] / static_cast<float>(D) + a.eps);
    dot /= static_cast<float>(HC_S);
    if (t < GH_R) a.tvec[row * (GH_R + HC_S) + t] = dot / (1.f + __expf(-dot));        // silu
    else if (a.inject != nullptr) a.post_out[row * HC_S + (t - GH_R)] = 2.f * sigmoidf_(dot);
  }
  if (t < HC_S) a.tvec[row * (GH_R + HC_S) + GH_R + t] = rsqrtf(tot[GH_NL * HC_S + t] / static_cast<float>(D) + a.eps);
  if (t == 0) a.counter[row] = 0;
}

// pass 2: g = sigmoid(t . up^T), mixed = mean_s(g n)
__global__ void __launch_bounds__(HC_THREADS) hc_gated_mix_kernel(GatedArgs a) {
  __shared__ float tv[GH_R + HC_S];
  const int row = blockIdx.x, D = a.D, t = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  if (t < GH_R + HC_S) tv[t] = a.tvec[row * (GH_R + HC_S) + t];
  __syncthreads();
  const float* R = (a.x != nullptr ? a.res_out : a.res) + static_cast<size_t>(row) * HC_S * D;
  const int d = blockIdx.y * HC_DC + t * 4;
  if (d >= D) return;
  float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < HC_S; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(R + static_cast<size_t>(s) * D + d);
    const float4 g = *reinterpret_cast<const float4*>(a.norm + static_cast<size_t>(s) * D + d);
    const float n[4] = {v.x * tv[GH_R + s] * (1.f + g.x), v.y * tv[GH_R + s] * (1.f + g.y), v.z * tv[GH_R + s] * (1.f + g.z),
                        v.w * tv[GH_R + s] * (1.f + g.w)};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat16* u = a.up + (static_cast<size_t>(s) * D + d + e) * GH_R;
      float z = 0.f;
#pragma unroll
      for (int r = 0; r < GH_R; r += 8) {
        const uint4 q = *reinterpret_cast<const uint4*>(u + r);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(p[k]);
          z += tv[r + 2 * k] * f.x + tv[r + 2 * k + 1] * f.y;
        }
      }
      out[e] += sigmoidf_(z) * n[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float m = out[e] / static_cast<float>(HC_S);
    a.h[static_cast<size_t>(row) * D + d + e] = __float2bfloat16(m);
    if (a.h_f32 != nullptr) a.h_f32[static_cast<size_t>(row) * D + d + e] = m;
  }
}

// gate of the hashed n-gram embedding: d = <rms(key) nk, rms(x) nq> / sqrt(H); x += sigmoid(sign(d) sqrt(max(|d|, eps))) * value
__global__ void ngram_gate_kernel(float* __restrict__ x, const float* __restrict__ key, const float* __restrict__ val,
                                  const float* __restrict__ nk, const float* __restrict__ nq, int H, float eps) {
  __shared__ float red[3 * 32];
  const int row = blockIdx.x, t = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  float* X = x + static_cast<size_t>(row) * H;
  const float* K = key + static_cast<size_t>(row) * H;
  float sk = 0.f, sx = 0.f, dot = 0.f;
  for (int i = t; i < H; i += blockDim.x) {
    const float k = K[i], v = X[i];
    sk += k * k; sx += v * v; dot += k * nk[i] * v * nq[i];
  }
  for (int o = 16; o; o >>= 1) {
    sk += __shfl_xor_sync(~0u, sk, o); sx += __shfl_xor_sync(~0u, sx, o); dot += __shfl_xor_sync(~0u, dot, o);
  }
  if ((t & 31) == 0) { red[(t >> 5) * 3] = sk; red[(t >> 5) * 3 + 1] = sx; red[(t >> 5) * 3 + 2] = dot; }
  __syncthreads();
  sk = sx = dot = 0.f;
  for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) { sk += red[w * 3]; sx += red[w * 3 + 1]; dot += red[w * 3 + 2]; }
  const float dd = dot * rsqrtf(sk / H + eps) * rsqrtf(sx / H + eps) * rsqrtf(static_cast<float>(H));
  const float mag = sqrtf(fmaxf(fabsf(dd), eps));
  const float gate = sigmoidf_(dd > 0.f ? mag : (dd < 0.f ? -mag : 0.f));
  const float* V = val + static_cast<size_t>(row) * H;
  for (int i = t; i < H; i += blockDim.x) X[i] += gate * V[i];
}

}  // namespace spark

using namespace spark;

extern "C" int spark_hc_chunks(int D) { return (D + HC_DC - 1) / HC_DC; }
extern "C" int spark_hc_partial_floats(int T, int D, int gated) {
  return T * spark_hc_chunks(D) * (gated ? GH_NL * HC_S + HC_S : HC_NL + 1);
}

// mHC site.  mode 0 = apply the update only, 1 = update (if x) + pre for the next block, 2 = update + stream mean + RMSNorm.
// The updated streams go to `res_out` (a different buffer than `res`); without an update `res` is only read.
extern "C" int spark_mhc_site(const float* res, int T, int S, int D, const void* x, int x_f32, const float* post_in,
                              const float* comb_in, const void* fn, const float* scale, const float* base, const float* norm,
                              void* h, float* mean_out, float* post_out, float* comb_out, float* partial, int* counter,
                              int iters, float eps, int mode, cudaStream_t s, float* res_out) {
  if (T <= 0) return 0;
  if (S != HC_S || D % 4 != 0 || D > 16384) return -5;
  MhcArgs a{res, x, x_f32, post_in, comb_in, static_cast<const __nv_bfloat16*>(fn), scale, base, norm,
            static_cast<__nv_bfloat16*>(h), mean_out, post_out, comb_out, partial, counter, res_out, D, iters, mode, eps};
  if (x != nullptr && (res_out == nullptr || res_out == res)) return -5;
  const int nz = mode == 1 ? HC_ZG : 1;
  const size_t smem = static_cast<size_t>(D) * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(mhc_site_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  const cudaError_t e = spark_launch_pdl(mhc_site_kernel, dim3(T, spark_hc_chunks(D), nz), dim3(HC_THREADS), smem, s, dim3(1, 1, 1), a);
  return e == cudaSuccess ? 0 : -4;
}

// Gated site: two launches (logits, then the mixed row).  `inject` == nullptr: no post (the final site).
extern "C" int spark_hc_gated_site(const float* res, int T, int S, int D, int rank, const void* x, int x_f32, const float* post_in,
                                   const float* norm, const void* down, const void* inject, const void* up, float* tvec,
                                   float* post_out, void* h, float* h_f32, float* partial, int* counter, float eps,
                                   cudaStream_t s, float* res_out) {
  if (T <= 0) return 0;
  if (S != HC_S || rank != GH_R || D % 4 != 0) return -5;
  if (x != nullptr && (res_out == nullptr || res_out == res)) return -5;
  GatedArgs a{res, res_out, x, x_f32, post_in, norm, static_cast<const __nv_bfloat16*>(down), static_cast<const __nv_bfloat16*>(inject),
              static_cast<const __nv_bfloat16*>(up), tvec, post_out, static_cast<__nv_bfloat16*>(h), h_f32, partial, counter, D, eps};
  cudaError_t e = spark_launch_pdl(hc_gated_logits_kernel, dim3(T, spark_hc_chunks(D), GH_ZG), dim3(HC_THREADS), 0, s, dim3(1, 1, 1), a);
  if (e != cudaSuccess) return -4;
  e = spark_launch_pdl(hc_gated_mix_kernel, dim3(T, spark_hc_chunks(D)), dim3(HC_THREADS), 0, s, dim3(1, 1, 1), a);
  return e == cudaSuccess ? 0 : -4;
}

// Residual update of a gated site on its own (after the last block, before the final site has no next logits to share a pass with).
extern "C" int spark_ngram_gate(float* x, const float* key, const float* val, const float* nk, const float* nq, int R, int H,
                                float eps, cudaStream_t s) {
  if (R <= 0) return 0;
  const cudaError_t e = spark_launch_pdl(ngram_gate_kernel, dim3(R), dim3(256), 0, s, dim3(1, 1, 1), x, key, val, nk, nq, H, eps);
  return e == cudaSuccess ? 0 : -4;
}
