// Row-wise elementwise kernels: embedding gather, (add +) RMSNorm, SwiGLU, arg-max, copies.
// Activations are bf16, the residual stream and norm weights are fp32.  One CTA per row, 16-byte
// accesses.  Replaces engine-rs/shim/ds41_ops.cu:17-239 (rms_norm*), kda.cu:1036 (rms_rows),
// shared_gu.cu:38-65 and the ATen row ops of the eager path.
#include "../common/decode.cuh"

namespace spark {

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += sh[i];      // fixed order: every thread gets the same bits
  __syncthreads();
  return t;
}

// res[R,H] fp32 (in/out) += delta (bf16 or fp32, optional); out[R,H] bf16 = rmsnorm(res) * w.
template <typename TD>
__global__ void add_rmsnorm_kernel(const TD* __restrict__ delta, float* __restrict__ res, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ out, int H, float eps, int one_plus) {
  __shared__ float sh[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  float* x = res + static_cast<size_t>(r) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = x[i];
    if (delta != nullptr) { v += static_cast<float>(delta[static_cast<size_t>(r) * H + i]); x[i] = v; }
    ss += v * v;
  }
  const float tot = block_sum(ss, sh);
  const float rs = rsqrtf(tot / H + eps);
  if (out != nullptr)
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float g = one_plus ? 1.f + w[i] : w[i];
      out[static_cast<size_t>(r) * H + i] = __float2bfloat16(x[i] * rs * g);
    }
}

// x bf16 [R,H] -> out bf16 (no residual)
__global__ void rmsnorm_bf16_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                    __nv_bfloat16* __restrict__ out, int H, float eps, int one_plus) {
  __shared__ float sh[32];
  const int r = blockIdx.x;
  const __nv_bfloat16* xr = x + static_cast<size_t>(r) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = __bfloat162float(xr[i]); ss += v * v; }
  const float rs = rsqrtf(block_sum(ss, sh) / H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float g = one_plus ? 1.f + w[i] : w[i];
    out[static_cast<size_t>(r) * H + i] = __float2bfloat16(__bfloat162float(xr[i]) * rs * g);
  }
}

// A token id outside [0, V) never reaches memory: its row is zero and the status word records {ST_BOUNDS, row, id}
// (ids come from clients; the host also validates them, this is the last line).
__global__ void embed_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int H, int V, int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int id = ids[r];
  if (id < 0 || id >= V) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[static_cast<size_t>(r) * H + i] = 0.f;
    if (threadIdx.x == 0 && status) set_status(status, ST_BOUNDS, r, id, V);
    return;
  }
  const __nv_bfloat16* src = table + static_cast<size_t>(id) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[static_cast<size_t>(r) * H + i] = __bfloat162float(src[i]);
}

// End of a device-fed decode round (one row per sequence): the sampled ids become the next round's input ids and
// every position advances by one, so a captured round can be replayed without the host in between.
// dev = packed plan [ids R | pos R | row_pos0 R | seg n*4] with R == n.
__global__ void decode_advance_kernel(int* __restrict__ dev, const int* __restrict__ out_ids, int n) {
  pdl_wait();
  pdl_trigger();
  const int i = threadIdx.x;
  if (i < n) {
    dev[i] = out_ids[i];
    dev[n + i] += 1;
    dev[2 * n + i] += 1;
    dev[3 * n + 4 * i + 3] += 1;
  }
}

// gu bf16 [R, 2F] = [gate | up] -> out bf16 [R, F]
// grid (R, column chunks): a decode-size batch still spreads over many CTAs (one CTA per row walked 12288 columns in 48
// dependent steps: 30 us for 4 rows)
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int F, float limit) {
  const int r = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < F; i += blockDim.x * gridDim.y) {
    float g = __bfloat162float(gu[static_cast<size_t>(r) * 2 * F + i]);
    float u = __bfloat162float(gu[static_cast<size_t>(r) * 2 * F + F + i]);
    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    out[static_cast<size_t>(r) * F + i] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
  }
}

// arg-max per row, ties -> lowest index.  Two stages so that a 150K-wide vocabulary is scanned by many
// CTAs: stage 1 grid (R, chunks) writes (value, index) packets, stage 2 (one warp per row) picks the winner.
__device__ __forceinline__ void argmax_combine(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
}

__global__ void __launch_bounds__(256)
argmax_part_kernel(const float* __restrict__ logits, int V, float* __restrict__ pv, int* __restrict__ pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, c = blockIdx.y, nc = gridDim.y;
  const int per = (V + nc - 1) / nc;
  const int i0 = c * per, i1 = min(V, i0 + per);
  const float* x = logits + static_cast<size_t>(r) * V;
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += 256 * 4) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = (i + u * 256) < i1 ? x[i + u * 256] : -INFINITY;
#pragma unroll
    for (int u = 0; u < 4; ++u) if (v[u] > best) { best = v[u]; bi = i + u * 256; }   // ascending i: first max kept
  }
  for (int o = 16; o > 0; o >>= 1)
    argmax_combine(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) argmax_combine(best, bi, sv[i], si[i]);
    pv[r * nc + c] = best; pi[r * nc + c] = bi;
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int nc,
                                    int* __restrict__ out_id, float* __restrict__ out_val) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < nc; i += 32) argmax_combine(best, bi, pv[r * nc + i], pi[r * nc + i]);
  for (int o = 16; o > 0; o >>= 1)
    argmax_combine(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (threadIdx.x == 0) { out_id[r] = bi; if (out_val) out_val[r] = best; }
}

// out f32 [R,H] = x f32 + add (bf16 or f32): residual add without a norm (last layer).
template <typename TD>
__global__ void add_kernel(const TD* __restrict__ delta, float* __restrict__ res, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < n) res[i] += static_cast<float>(delta[i]);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < n) y[i] = __float2bfloat16(x[i]);
}

// gather rows: out[i, :] = src[idx[i], :]  (bf16, 16-byte vectors; H % 8 == 0)
__global__ void gather_rows_bf16_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx,
                                        __nv_bfloat16* __restrict__ out, int H) {
  const int r = blockIdx.x;
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(idx[r]) * H);
  uint4* d = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) d[i] = s[i];
}

}  // namespace spark

using namespace spark;

// Gumbel-max sampling noise, in place: x[r][v] = x[r][v] / T_r + g(seed_r, pos_r, off + v) for rows with T_r > 0
// (rows with T_r <= 0 stay greedy).  g = -log(-log u), u a splitmix64 hash of (seed, position, global vocabulary id),
// so every rank of a vocabulary-parallel head perturbs its slice with the noise of the global ids and the arg-max over
// ranks is the token a single GPU would draw.  Double-precision logs keep it equal to the host oracle after rounding.
// Reference: engine-rs/src/sampling.rs:20-170, shim/latent.cu:840-940.
static __device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
static __global__ void gumbel_perturb_kernel(float* __restrict__ x, int V, int ldx, const float* __restrict__ temp,
                                      const long long* __restrict__ seed, const long long* __restrict__ pos, int off) {
  const int r = blockIdx.y;
  const float T = temp[r];
  if (!(T > 0.f)) return;
  const unsigned long long key = ((unsigned long long)seed[r] * 0x9E3779B97F4A7C15ull) ^
                                 ((unsigned long long)(pos[r] + 1) * 0xBF58476D1CE4E5B9ull);
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < V; v += gridDim.x * blockDim.x) {
    const unsigned long long h = mix64((unsigned long long)(v + off) * 0x9E3779B97F4A7C15ull + key);
    const double u = ((double)(h >> 11) + 0.5) * (1.0 / 9007199254740992.0);
    const float g = (float)(-log(-log(u)));
    float* p = x + (size_t)r * ldx + v;
    *p = *p / T + g;
  }
}

// softmax(logits)[token] for one row from vocabulary slices: every rank reduces its slice to (max, sum exp(l - max)) and
// the slice that holds the token contributes its logit; `final` combines the per-rank pairs.  Used for the drafter's
// confidence (the draft-length policies read it), so all ranks must get the same number: the per-rank pairs travel
// through the rank-ordered all-reduce.  ms: [R, ld] with rank r's pair at columns 2r, 2r+1; lt: [R] (zero unless owned).
// Reference: engine-rs/src/sampling.rs:120-170 (confidence of the sampled draft), shim/draft_selector.cu:14.
static __global__ void token_prob_part_kernel(const float* __restrict__ logits, int V, int ldx, const int* __restrict__ ids,
                                              int off, int rank, float* __restrict__ ms, int ld, float* __restrict__ lt) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, t = threadIdx.x;
  const float* x = logits + (size_t)r * ldx;
  __shared__ float red[32];
  float m = -INFINITY;
  for (int v = t; v < V; v += blockDim.x) m = fmaxf(m, x[v]);
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o));
  if ((t & 31) == 0) red[t >> 5] = m;
  __syncthreads();
  m = red[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  float s = 0.f;
  for (int v = t; v < V; v += blockDim.x) s += __expf(x[v] - m);
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(~0u, s, o);
  if ((t & 31) == 0) red[t >> 5] = s;
  __syncthreads();
  if (t == 0) {
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
    ms[(size_t)r * ld + 2 * rank] = m;
    ms[(size_t)r * ld + 2 * rank + 1] = tot;
    const int id = ids[r] - off;
    lt[r] = (id >= 0 && id < V) ? x[id] : 0.f;
  }
}
static __global__ void token_prob_final_kernel(const float* __restrict__ ms, int ld, int world, const float* __restrict__ lt,
                                               float* __restrict__ out, int R) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  float M = -INFINITY;
  for (int k = 0; k < world; ++k) M = fmaxf(M, ms[(size_t)r * ld + 2 * k]);
  float S = 0.f;
  for (int k = 0; k < world; ++k) S += ms[(size_t)r * ld + 2 * k + 1] * __expf(ms[(size_t)r * ld + 2 * k] - M);
  out[r] = __expf(lt[r] - M) / S;
}

extern "C" void spark_add_rmsnorm(const void* delta, int delta_f32, float* res, const float* w, void* out, int R, int H,
                                  float eps, int one_plus, cudaStream_t s) {
  if (R <= 0) return;
  int th = H >= 2048 ? 512 : 256;
  if (delta_f32)
    spark_launch_pdl(add_rmsnorm_kernel<float>, dim3(R), dim3(th), 0, s, dim3(1, 1, 1), (const float*)delta, res, w,
                     (__nv_bfloat16*)out, H, eps, one_plus);
  else
    spark_launch_pdl(add_rmsnorm_kernel<__nv_bfloat16>, dim3(R), dim3(th), 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)delta, res, w,
                     (__nv_bfloat16*)out, H, eps, one_plus);
}
extern "C" void spark_rmsnorm_bf16(const void* x, const float* w, void* out, int R, int H, float eps, int one_plus,
                                   cudaStream_t s) {
  if (R <= 0) return;
  rmsnorm_bf16_kernel<<<R, 256, 0, s>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)out, H, eps, one_plus);
}
extern "C" void spark_embed(const void* table, const int* ids, float* out, int R, int H, cudaStream_t s, int V, int* status) {
  if (R <= 0) return;
  spark_launch_pdl(embed_kernel, dim3(R), dim3(256), 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)table, ids, out, H, V, status);
}
extern "C" int spark_decode_advance(int* dev, const int* out_ids, int n, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n > 1024) return -5;
  const cudaError_t e = spark_launch_pdl(decode_advance_kernel, dim3(1), dim3(((n + 31) / 32) * 32), 0, s, dim3(1, 1, 1), dev, out_ids, n);
  return e == cudaSuccess ? 0 : -4;
}
extern "C" void spark_swiglu(const void* gu, void* out, int R, int F, float limit, cudaStream_t s) {
  if (R <= 0) return;
  int ny = (F + 1023) / 1024;                       // <= 4 columns per thread while the grid stays below ~4 waves
  while (ny > 1 && static_cast<long long>(R) * ny > 148 * 16) ny = (ny + 1) / 2;
  swiglu_kernel<<<dim3(R, ny), 256, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, F, limit);
}
// part_v / part_i: scratch of R * 64 entries each.
extern "C" void spark_argmax(const float* logits, int R, int V, int* out_id, float* out_val, float* part_v, int* part_i,
                             cudaStream_t s) {
  if (R <= 0) return;
  const int nc = V >= 65536 ? 64 : (V >= 4096 ? 8 : 1);
  spark_launch_pdl(argmax_part_kernel, dim3(R, nc), dim3(256), 0, s, dim3(1, 1, 1), logits, V, part_v, part_i);
  spark_launch_pdl(argmax_final_kernel, dim3(R), dim3(32), 0, s, dim3(1, 1, 1), (const float*)part_v, (const int*)part_i, nc, out_id,
                   out_val);
}
extern "C" int spark_gumbel_perturb(float* x, int R, int V, int ldx, const float* temp, const long long* seed,
                                    const long long* pos, int off, cudaStream_t s) {
  if (R <= 0 || V <= 0) return 0;
  if (R > 65535) return -5;
  const int bx = V >= 65536 ? 32 : (V >= 4096 ? 8 : 1);
  gumbel_perturb_kernel<<<dim3(bx, R), 256, 0, s>>>(x, V, ldx, temp, seed, pos, off);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int spark_token_prob_part(const float* logits, int R, int V, int ldx, const int* ids, int off, int rank, float* ms,
                                     int ld, float* lt, cudaStream_t s) {
  if (R <= 0) return 0;
  const cudaError_t e = spark_launch_pdl(token_prob_part_kernel, dim3(R), dim3(1024), 0, s, dim3(1, 1, 1), logits, V, ldx, ids, off,
                                         rank, ms, ld, lt);
  return e == cudaSuccess ? 0 : -4;
}
extern "C" int spark_token_prob_final(const float* ms, int ld, int world, const float* lt, float* out, int R, cudaStream_t s) {
  if (R <= 0) return 0;
  const cudaError_t e = spark_launch_pdl(token_prob_final_kernel, dim3((R + 63) / 64), dim3(64), 0, s, dim3(1, 1, 1), ms, ld, world,
                                         lt, out, R);
  return e == cudaSuccess ? 0 : -4;
}
extern "C" void spark_add(const void* delta, int delta_f32, float* res, long n, cudaStream_t s) {
  if (n <= 0) return;
  unsigned b = (unsigned)((n + 255) / 256);
  if (delta_f32) add_kernel<float><<<b, 256, 0, s>>>((const float*)delta, res, (size_t)n);
  else add_kernel<__nv_bfloat16><<<b, 256, 0, s>>>((const __nv_bfloat16*)delta, res, (size_t)n);
}
extern "C" void spark_f32_to_bf16(const float* x, void* y, long n, cudaStream_t s) {
  if (n <= 0) return;
  f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, (__nv_bfloat16*)y, (size_t)n);
}
extern "C" void spark_gather_rows_bf16(const void* src, const int* idx, void* out, int R, int H, cudaStream_t s) {
  if (R <= 0) return;
  gather_rows_bf16_kernel<<<R, 256, 0, s>>>((const __nv_bfloat16*)src, idx, (__nv_bfloat16*)out, H);
}
