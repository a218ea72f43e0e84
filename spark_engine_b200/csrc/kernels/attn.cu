// Softmax GQA attention for decode / verify rows over a contiguous-per-sequence KV pool.
//   attn_prep   : per (row, head) Gemma-RMS q/k norm + partial NeoX RoPE; K,V appended to the pool at
//                 kv_base[slot] + pos (bf16, or e4m3 with one fp32 scale per (token, head)); indexer
//                 query norm+rope, raw indexer key append, and the mean-pooled (then normed + roped)
//                 key of every 4-token block this row completes.
//   attn_decode : split-KV (256 tokens per CTA): scores -> per-head softmax stats -> P.V, partials
//                 (m, l, o) to scratch;  tokens are either the row's whole context or a selected list
//                 (block-sparse top-k + tail).
//   attn_merge  : fixed-order merge of the splits, sigmoid output gate, bf16 out.
// All reductions have a fixed order (no float atomics): run-to-run bitwise equal, and a row's result is
// independent of the other rows in the batch.
// Reference: engine-rs/shim/qwen_qsa.cu:69-178 (prep/pool), :215-882 (attn_* / attn_combine).
#include "../common/decode.cuh"
#include <cuda_fp8.h>

namespace spark {

struct AttnDims {
  int Hq, Hkv, D, rope_dim, gated, qk_norm, idx_heads, idx_dim, block, fp8;
  float eps;
};

// ------------------------------------------------------------------------------------------ prep
// grid (R, Hq + 2*Hkv + idx_heads + (idx_dim ? 1 : 0)); 128 threads; thread t owns dims t and t+128.
__global__ void __launch_bounds__(128)
attn_prep_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, AttnDims a,
                 const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                 const float* __restrict__ iq_norm, const float* __restrict__ ik_norm,
                 const double* __restrict__ inv_freq,
                 const int* __restrict__ pos, const long long* __restrict__ row_kv,   // kv_base[slot] per row
                 const int* __restrict__ row_j,                                       // row index inside its segment
                 __nv_bfloat16* __restrict__ qbuf,                                    // [R, Hq, D]
                 void* __restrict__ kc, void* __restrict__ vc,                        // [tokens, Hkv, D]
                 float* __restrict__ ks, float* __restrict__ vs,                      // fp8 scales [tokens, Hkv]
                 float* __restrict__ qi_buf,                                          // [R, idx_heads, idx_dim]
                 float* __restrict__ ik_raw, float* __restrict__ ik_pool) {
  __shared__ float red[4];
  __shared__ float vals[256];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, job = blockIdx.y, t = threadIdx.x;
  const int qw = a.D * (a.gated ? 2 : 1);
  const int nq = a.Hq * qw, nkv = a.Hkv * a.D;
  const int p = pos[r];
  const long long tok = row_kv[r] + p;
  const __nv_bfloat16* row = qkv + static_cast<size_t>(r) * ld;
  int kind, head, dim, off;            // kind 0 q, 1 k, 2 v, 3 indexer q, 4 indexer key
  if (job < a.Hq) { kind = 0; head = job; dim = a.D; off = head * qw; }
  else if (job < a.Hq + a.Hkv) { kind = 1; head = job - a.Hq; dim = a.D; off = nq + head * a.D; }
  else if (job < a.Hq + 2 * a.Hkv) { kind = 2; head = job - a.Hq - a.Hkv; dim = a.D; off = nq + nkv + head * a.D; }
  else if (job < a.Hq + 2 * a.Hkv + a.idx_heads) { kind = 3; head = job - a.Hq - 2 * a.Hkv; dim = a.idx_dim; off = nq + 2 * nkv + head * a.idx_dim; }
  else { kind = 4; head = 0; dim = a.idx_dim; off = nq + 2 * nkv + a.idx_heads * a.idx_dim; }

  int rope = a.rope_dim, rp = p;
  const float* nw = nullptr;
  bool norm = false;
  float x0 = 0.f, x1 = 0.f;
  if (kind == 4) {
    // raw key of this row; pooled key only when this row completes a block
    for (int d = t; d < dim; d += 128) ik_raw[tok * dim + d] = __bfloat162float(row[off + d]);
    if ((p + 1) % a.block != 0) return;
    // mean of the block's raw keys BEFORE norm + rope at the block's first position
    for (int d = t; d < dim; d += 128) {
      float s = 0.f;
      for (int b = 0; b < a.block; ++b) {
        const int back = a.block - 1 - b;                 // rows p-back .. p
        float v;
        if (back <= row_j[r]) v = __bfloat162float(qkv[static_cast<size_t>(r - back) * ld + off + d]);   // same launch
        else v = ik_raw[(tok - back) * dim + d];                                                          // earlier step
        s += v;
      }
      vals[d] = s / a.block;
    }
    __syncthreads();
    x0 = t < dim ? vals[t] : 0.f; x1 = (t + 128) < dim ? vals[t + 128] : 0.f;
    norm = true; nw = ik_norm; rp = p + 1 - a.block; rope = min(a.rope_dim, dim);
  } else {
    x0 = t < dim ? __bfloat162float(row[off + t]) : 0.f;
    x1 = (t + 128) < dim ? __bfloat162float(row[off + t + 128]) : 0.f;
    if (kind == 0) { norm = a.qk_norm; nw = q_norm; }
    if (kind == 1) { norm = a.qk_norm; nw = k_norm; }
    if (kind == 3) { norm = true; nw = iq_norm; rope = min(a.rope_dim, dim); }
    if (kind == 2) rope = 0;
  }
  if (norm) {
    float ss = warp_sum(x0 * x0 + x1 * x1);
    if ((t & 31) == 0) red[t >> 5] = ss;
    __syncthreads();
    ss = red[0] + red[1] + red[2] + red[3];
    const float rs = rsqrtf(ss / dim + a.eps);
    if (t < dim) x0 = x0 * rs * (1.f + nw[t]);
    if (t + 128 < dim) x1 = x1 * rs * (1.f + nw[t + 128]);
  }
  __syncthreads();
  vals[t] = x0; vals[t + 128] = x1;
  __syncthreads();
  if (rope > 0) {
    const int half = rope / 2;
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int d = t + rep * 128;
      if (d < rope) {
        const int i = d < half ? d : d - half;
        const float ang = static_cast<float>(static_cast<double>(rp) * inv_freq[i]);
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const float a1 = vals[i], a2 = vals[i + half];
        const float o = d < half ? a1 * cs - a2 * sn : a2 * cs + a1 * sn;
        if (rep == 0) x0 = o; else x1 = o;
      }
    }
  }
  // ---- write
  if (kind == 0) {
    __nv_bfloat16* dst = qbuf + (static_cast<size_t>(r) * a.Hq + head) * a.D;
    if (t < dim) dst[t] = __float2bfloat16(x0);
    if (t + 128 < dim) dst[t + 128] = __float2bfloat16(x1);
  } else if (kind == 1 || kind == 2) {
    const size_t o = (static_cast<size_t>(tok) * a.Hkv + head) * a.D;
    if (a.fp8) {
      float am = warp_max(fmaxf(fabsf(x0), fabsf(x1)));
      __syncthreads();
      if ((t & 31) == 0) red[t >> 5] = am;
      __syncthreads();
      am = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
      const float sc = fmaxf(am, 1e-8f) / 448.f;
      __nv_fp8_e4m3* dst = reinterpret_cast<__nv_fp8_e4m3*>(kind == 1 ? kc : vc) + o;
      if (t < dim) dst[t] = __nv_fp8_e4m3(x0 / sc);
      if (t + 128 < dim) dst[t + 128] = __nv_fp8_e4m3(x1 / sc);
      if (t == 0) (kind == 1 ? ks : vs)[static_cast<size_t>(tok) * a.Hkv + head] = sc;
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(kind == 1 ? kc : vc) + o;
      if (t < dim) dst[t] = __float2bfloat16(x0);
      if (t + 128 < dim) dst[t + 128] = __float2bfloat16(x1);
    }
  } else if (kind == 3) {
    float* dst = qi_buf + (static_cast<size_t>(r) * a.idx_heads + head) * dim;
    if (t < dim) dst[t] = x0;
    if (t + 128 < dim) dst[t + 128] = x1;
  } else {
    float* dst = ik_pool + (tok / a.block) * dim;
    if (t < dim) dst[t] = x0;
    if (t + 128 < dim) dst[t + 128] = x1;
  }
}

// ------------------------------------------------------------------------------------------ decode
constexpr int ATT_TS = 64;         // tokens per split
constexpr int ATT_MAXREP = 8;

template <bool FP8>
__device__ __forceinline__ float kv_load(const void* base, size_t idx) {
  if (FP8) return static_cast<float>(reinterpret_cast<const __nv_fp8_e4m3*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

// grid (R, Hkv, nsplit); 256 threads.
template <bool FP8>
__global__ void __launch_bounds__(256)
attn_decode_kernel(const __nv_bfloat16* __restrict__ qbuf, const void* __restrict__ kc, const void* __restrict__ vc,
                   const float* __restrict__ ks, const float* __restrict__ vs,
                   const int* __restrict__ pos, const long long* __restrict__ row_kv,
                   const int* __restrict__ sel, const int* __restrict__ sel_n, int sel_ld,
                   float* __restrict__ part_o, float* __restrict__ part_ml,   // [R,Hq,nsplit,D], [R,Hq,nsplit,2]
                   int Hq, int Hkv, int D, float scale) {
  __shared__ float sc[ATT_MAXREP][ATT_TS];
  __shared__ float sq[ATT_MAXREP][256];
  __shared__ int stok[ATT_TS];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z, nsplit = gridDim.z;
  const int rep = Hq / Hkv;
  const int n_ctx = sel ? sel_n[r] : pos[r] + 1;
  const int t0 = sp * ATT_TS;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const size_t pbase = ((static_cast<size_t>(r) * Hq + hk * rep) * nsplit + sp);
  if (t0 >= n_ctx) {                     // empty split: neutral partial
    if (t < rep) { part_ml[(pbase + static_cast<size_t>(t) * nsplit) * 2] = -INFINITY; part_ml[(pbase + static_cast<size_t>(t) * nsplit) * 2 + 1] = 0.f; }
    return;
  }
  const int nt = min(ATT_TS, n_ctx - t0);
  const long long base = row_kv[r];
  for (int i = t; i < nt; i += 256) stok[i] = sel ? sel[static_cast<size_t>(r) * sel_ld + t0 + i] : t0 + i;
  for (int i = t; i < rep * 256; i += 256) {
    const int h = i >> 8, d = i & 255;
    sq[h][d] = d < D ? __bfloat162float(qbuf[(static_cast<size_t>(r) * Hq + hk * rep + h) * D + d]) : 0.f;
  }
  __syncthreads();
  // phase 1: scores.  warp per token, lane covers dims [8*lane, 8*lane+8)
  for (int i = warp; i < nt; i += 8) {
    const size_t ko = (static_cast<size_t>(base + stok[i]) * Hkv + hk) * D;
    float kf[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { const int d = lane * 8 + j; kf[j] = d < D ? kv_load<FP8>(kc, ko + d) : 0.f; }
    const float ksc = FP8 ? ks[static_cast<size_t>(base + stok[i]) * Hkv + hk] : 1.f;
    for (int h = 0; h < rep; ++h) {
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) a = fmaf(kf[j], sq[h][lane * 8 + j], a);
      a = warp_sum(a);
      if (lane == 0) sc[h][i] = a * scale * ksc;
    }
  }
  __syncthreads();
  // phase 2: per-head softmax statistics (warp h owns head h)
  if (warp < rep) {
    float m = -INFINITY;
    for (int i = lane; i < nt; i += 32) m = fmaxf(m, sc[warp][i]);
    m = warp_max(m);
    float l = 0.f;
    for (int i = lane; i < nt; i += 32) {
      float pexp = __expf(sc[warp][i] - m);
      if (FP8) pexp *= vs[static_cast<size_t>(base + stok[i]) * Hkv + hk];   // fold the V scale into P
      sc[warp][i] = pexp;
    }
    __syncwarp();
    // l must not include the V scale: recompute from exp only when FP8
    for (int i = lane; i < nt; i += 32) {
      float e = sc[warp][i];
      if (FP8) e /= vs[static_cast<size_t>(base + stok[i]) * Hkv + hk];
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) {
      part_ml[(pbase + static_cast<size_t>(warp) * nsplit) * 2] = m;
      part_ml[(pbase + static_cast<size_t>(warp) * nsplit) * 2 + 1] = l;
    }
  }
  __syncthreads();
  // phase 3: o[h][d] = sum_tok p[h][tok] v[tok][d]; thread d owns one output dim
  if (t < D) {
    float o[ATT_MAXREP];
#pragma unroll
    for (int h = 0; h < ATT_MAXREP; ++h) o[h] = 0.f;
    for (int i0 = 0; i0 < nt; i0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = (i0 + u) < nt ? kv_load<FP8>(vc, (static_cast<size_t>(base + stok[i0 + u]) * Hkv + hk) * D + t) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i0 + u < nt) {
#pragma unroll
          for (int h = 0; h < ATT_MAXREP; ++h) if (h < rep) o[h] = fmaf(sc[h][i0 + u], v[u], o[h]);
        }
    }
#pragma unroll
    for (int h = 0; h < ATT_MAXREP; ++h)
      if (h < rep) part_o[(pbase + static_cast<size_t>(h) * nsplit) * D + t] = o[h];
  }
}

// grid (R, Hq); D threads (<= 256).  Splits merged in ascending order.
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int nsplit,
                                  const __nv_bfloat16* __restrict__ qkv, int ld, int gated, int Hq, int D,
                                  __nv_bfloat16* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const size_t pb = (static_cast<size_t>(r) * Hq + h) * nsplit;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(pb + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float m = part_ml[(pb + s) * 2];
    if (m == -INFINITY) continue;
    const float w = __expf(m - M);
    l += w * part_ml[(pb + s) * 2 + 1];
    o += w * part_o[(pb + s) * D + d];
  }
  float res = o / l;
  if (gated) {
    const float g = __bfloat162float(qkv[static_cast<size_t>(r) * ld + h * 2 * D + D + d]);
    res = res / (1.f + __expf(-g));
  }
  out[(static_cast<size_t>(r) * Hq + h) * D + d] = __float2bfloat16(res);
}

}  // namespace spark

using namespace spark;

extern "C" int spark_attn_prep(const void* qkv, int ld, int R, int Hq, int Hkv, int D, int rope_dim, int gated,
                               int qk_norm, int idx_heads, int idx_dim, int block, int fp8, float eps,
                               const float* q_norm, const float* k_norm, const float* iq_norm, const float* ik_norm,
                               const double* inv_freq, const int* pos, const long long* row_kv, const int* row_j,
                               void* qbuf, void* kc, void* vc, float* ks, float* vs, float* qi_buf, float* ik_raw,
                               float* ik_pool, cudaStream_t s) {
  if (R <= 0) return 0;
  if (D > 256 || idx_dim > 256) return -5;
  AttnDims a{Hq, Hkv, D, rope_dim, gated, qk_norm, idx_heads, idx_dim, block, fp8, eps};
  dim3 grid(R, Hq + 2 * Hkv + idx_heads + (idx_dim > 0 ? 1 : 0));
  const cudaError_t err = spark_launch_pdl(attn_prep_kernel, grid, dim3(128), 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)qkv, ld, a,
                                           q_norm, k_norm, iq_norm, ik_norm, inv_freq, pos, row_kv, row_j, (__nv_bfloat16*)qbuf,
                                           kc, vc, ks, vs, qi_buf, ik_raw, ik_pool);
  return err == cudaSuccess ? 0 : -4;
}

extern "C" int spark_attn_decode(const void* qbuf, const void* kc, const void* vc, const float* ks, const float* vs,
                                 int fp8, const int* pos, const long long* row_kv, const int* sel, const int* sel_n,
                                 int sel_ld, float* part_o, float* part_ml, int nsplit, const void* qkv, int ld,
                                 int gated, int R, int Hq, int Hkv, int D, float scale, void* out, cudaStream_t s) {
  if (R <= 0) return 0;
  if (D > 256 || Hq / Hkv > ATT_MAXREP) return -5;
  dim3 grid(R, Hkv, nsplit);
  cudaError_t err;
  if (fp8)
    err = spark_launch_pdl(attn_decode_kernel<true>, grid, dim3(256), 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)qbuf, kc, vc, ks, vs,
                           pos, row_kv, sel, sel_n, sel_ld, part_o, part_ml, Hq, Hkv, D, scale);
  else
    err = spark_launch_pdl(attn_decode_kernel<false>, grid, dim3(256), 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)qbuf, kc, vc, ks, vs,
                           pos, row_kv, sel, sel_n, sel_ld, part_o, part_ml, Hq, Hkv, D, scale);
  if (err != cudaSuccess) return -4;
  err = spark_launch_pdl(attn_merge_kernel, dim3(R, Hq), dim3(D), 0, s, dim3(1, 1, 1), (const float*)part_o, (const float*)part_ml,
                         nsplit, (const __nv_bfloat16*)qkv, ld, gated, Hq, D, (__nv_bfloat16*)out);
  return err == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory (declared in attn_noalloc.h; this entry
// point has no counterpart in the reference).  Same kernels as spark_attn_decode, but the split partials live
// in a fixed array inside this library instead of a caller-provided scratch buffer.
#include "attn_noalloc.h"
#include <cstdio>
#include <mutex>

static __device__ __align__(256) float g_noalloc_scratch[SPARK_ATTN_NOALLOC_MAX_FLOATS];

// `g_noalloc_scratch` names a host-side shadow here; the device address is looked up once per device.
static float* noalloc_scratch_for_current_device(cudaError_t* err) {
  static std::mutex mu;
  static float* ptrs[64] = {nullptr};
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (*err != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<float*>(p);
  }
  return ptrs[dev];
}

extern "C" int spark_attn_decode_noalloc(const void* qbuf, const void* kc, const void* vc, const float* ks,
                                         const float* vs, int fp8, const int* pos, const long long* row_kv,
                                         const int* sel, const int* sel_n, int sel_ld, int nsplit, const void* qkv,
                                         int ld, int gated, int R, int Hq, int Hkv, int D, float scale, void* out,
                                         cudaStream_t s) {
  if (R <= 0) return 0;
  if (D > 256 || Hq / Hkv > ATT_MAXREP || nsplit <= 0) return -5;
  const long long need = static_cast<long long>(R) * Hq * nsplit * (D + 2);
  if (need > SPARK_ATTN_NOALLOC_MAX_FLOATS) {
    fprintf(stderr, "spark_attn_decode_noalloc: rows*heads*splits*(head_dim+2) = %lld floats exceeds the built-in "
                    "scratch of %lld floats; use spark_attn_decode with a caller-provided buffer\n",
            need, static_cast<long long>(SPARK_ATTN_NOALLOC_MAX_FLOATS));
    return SPARK_ATTN_NOALLOC_TOO_LARGE;
  }
  cudaError_t err;
  float* scratch = noalloc_scratch_for_current_device(&err);
  if (scratch == nullptr) {
    fprintf(stderr, "spark_attn_decode_noalloc: scratch symbol lookup failed: %s\n", cudaGetErrorString(err));
    return -4;
  }
  float* part_o = scratch;
  float* part_ml = scratch + static_cast<size_t>(R) * Hq * nsplit * D;
  dim3 grid(R, Hkv, nsplit);
  if (fp8)
    attn_decode_kernel<true><<<grid, 256, 0, s>>>((const __nv_bfloat16*)qbuf, kc, vc, ks, vs, pos, row_kv, sel, sel_n, sel_ld,
                                                  part_o, part_ml, Hq, Hkv, D, scale);
  else
    attn_decode_kernel<false><<<grid, 256, 0, s>>>((const __nv_bfloat16*)qbuf, kc, vc, ks, vs, pos, row_kv, sel, sel_n, sel_ld,
                                                   part_o, part_ml, Hq, Hkv, D, scale);
  attn_merge_kernel<<<dim3(R, Hq), D, 0, s>>>(part_o, part_ml, nsplit, (const __nv_bfloat16*)qkv, ld, gated, Hq, D,
                                              (__nv_bfloat16*)out);
  return spark_launch_rc(__func__);
}
