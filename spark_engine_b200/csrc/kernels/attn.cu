// Softmax GQA attention for decode / verify rows over a contiguous-per-sequence KV pool.
//   attn_prep   : per (row, head) Gemma-RMS q/k norm + partial NeoX RoPE; K,V appended to the pool at
//                 kv_base[slot] + pos (bf16, or e4m3 with one fp32 scale per (token, head)); indexer
//                 query norm+rope, raw indexer key append, and the mean-pooled (then normed + roped)
//                 key of every 4-token block this row completes.
//   attn_decode : split-KV (64 tokens per CTA) on warp-level tensor-core MMAs: scores -> per-head softmax
//                 stats -> P.V, partials (m, l, o) to scratch;  tokens are either the row's whole context or a
//                 selected list (block-sparse top-k + tail); optional ancestor mask for tree verification.
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
                 const int* __restrict__ row_pos0,                                    // tree verify: first in-flight position
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
  // KV row of this token: its position for chains; for tree rows (row_pos0 given) the in-flight slot pos0 + j, because
  // sibling nodes share a position (the rotary angle still uses the position)
  const long long tok = row_kv[r] + (row_pos0 ? row_pos0[r] + row_j[r] : p);
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
    if (row_pos0 != nullptr) return;          // tree rows: blocks are pooled when the accepted path is committed
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


// ------------------------------------------------------------------------------------------ decode (tensor cores)
// Split-KV decode / verify attention: grid (row, kv head, split of 64 tokens), 4 warps.  The split's K and V rows
// (the row's context, or its selected-token list) are requested with cp.async in one go -- 64 KB in flight per CTA
// for head_dim 256 -- so a split costs one memory round trip instead of one per group of tokens.  The q heads that
// share the kv head are the M dimension of the warp-level MMA (<= 16), S = Q K^T and O = P V run on m16n8k16 bf16
// with fp32 accumulation; V fragments come from ldmatrix.trans.  FP8 KV (e4m3 + one fp32 scale per token and head)
// is converted to bf16 tiles in shared memory, the scales are folded into S and P.
// Tree verification: `anc` holds, per row, the bitmask of segment-local rows it may attend to (itself and its
// ancestors); tokens at or beyond the segment's first in-flight position (`row_pos0`) are kept only if their bit is
// set, committed tokens are always visible.  Chains pass anc == nullptr (causal by the context length).
// Splits are merged in ascending order by attn_merge_kernel: fixed order, a row never depends on its batch mates.
// Replaces engine-rs/shim/qwen_qsa.cu:421-882 (attn_tc / attn_tcp / attn_combine) and the tree paths of
// engine-rs/src/mla_latent.rs:472-773 for GQA layers.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(smem)));
}

struct AttnDecodeArgs {
  const __nv_bfloat16* qbuf; const void* kc; const void* vc; const float* ks; const float* vs;
  const int* pos; const long long* row_kv; const int* sel; const int* sel_n; int sel_ld;
  const int* row_pos0; const int* row_j; const uint32_t* anc;     // optional (tree verify / explicit in-flight index)
  float* part_o; float* part_ml; int Hq, Hkv; float scale;
  int chunks;                        // 64-token tiles per split (>= 1)
};

constexpr int ATT_ROWS = 16;       // q heads per kv head, padded to the MMA's M

template <int D, bool FP8>
__global__ void __launch_bounds__(128)
attn_decode_tc_kernel(const __grid_constant__ AttnDecodeArgs a) {
  constexpr int LD = D + 8;                                   // bf16 elements per tile row (16-byte padded)
  constexpr int NT = D / 32;                                  // 8-wide dim tiles per warp
  extern __shared__ __align__(16) uint8_t smem_att[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_att);                  // [16][LD]
  __nv_bfloat16* Ks = Qs + ATT_ROWS * LD;                                           // [64][LD]
  __nv_bfloat16* Vs = Ks + ATT_TS * LD;                                             // [64][LD]
  float* Ss = reinterpret_cast<float*>(Vs + ATT_TS * LD);                           // [16][68]
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(Ss + ATT_ROWS * 68);         // [16][72]
  int* stok = reinterpret_cast<int*>(Ps + ATT_ROWS * 72);                           // [64]
  float* ksc = reinterpret_cast<float*>(stok + ATT_TS);                             // [64]
  float* vsc = ksc + ATT_TS;                                                        // [64]
  uint8_t* stage = reinterpret_cast<uint8_t*>(vsc + ATT_TS);                        // FP8: [2][64][D] bytes
  __shared__ float m_run[ATT_ROWS], l_run[ATT_ROWS], alpha[ATT_ROWS];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z, nsplit = gridDim.z;
  const int rep = a.Hq / a.Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int pos0 = a.row_pos0 ? a.row_pos0[r] : 0;
  const int n_ctx = a.sel ? a.sel_n[r] : (a.row_pos0 ? pos0 + a.row_j[r] + 1 : a.pos[r] + 1);
  // a split is `chunks` tiles of 64 tokens walked in order with a running (max, sum): decode rounds use one tile per
  // split (parallelism over splits), prefill-size batches walk the whole row in one CTA (no partials to merge)
  const int span = a.chunks * ATT_TS;
  const int s0 = sp * span;
  const size_t pbase = (static_cast<size_t>(r) * a.Hq + hk * rep) * nsplit + sp;
  if (s0 >= n_ctx) {                     // empty split: neutral partial
    if (tid < rep) { a.part_ml[(pbase + static_cast<size_t>(tid) * nsplit) * 2] = -INFINITY; a.part_ml[(pbase + static_cast<size_t>(tid) * nsplit) * 2 + 1] = 0.f; }
    return;
  }
  const int s1 = min(n_ctx, s0 + span);
  const long long base = a.row_kv[r];
  const uint32_t anc = a.anc ? a.anc[r] : 0xffffffffu;
  if (tid < ATT_ROWS) { m_run[tid] = -INFINITY; l_run[tid] = 0.f; alpha[tid] = 1.f; }
  for (int i = tid; i < ATT_ROWS * (D / 8); i += 128) {       // queries of the heads that share this kv head
    const int h = i / (D / 8), c = i - h * (D / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (h < rep) v = *reinterpret_cast<const uint4*>(a.qbuf + (static_cast<size_t>(r) * a.Hq + hk * rep + h) * D + c * 8);
    *reinterpret_cast<uint4*>(Qs + h * LD + c * 8) = v;
  }
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }

  for (int t0 = s0; t0 < s1; t0 += ATT_TS) {
    const int nt = min(ATT_TS, s1 - t0);
    if (tid < ATT_TS) {
      int tk = -1;
      if (tid < nt) {
        tk = a.sel ? a.sel[static_cast<size_t>(r) * a.sel_ld + t0 + tid] : t0 + tid;
        if (a.anc && tk >= pos0 && !((anc >> min(tk - pos0, 31)) & 1u)) tk = -1;      // not an ancestor of this row
      }
      stok[tid] = tk;
      if (FP8) {
        ksc[tid] = tk >= 0 ? a.ks[static_cast<size_t>(base + tk) * a.Hkv + hk] : 0.f;
        vsc[tid] = tk >= 0 ? a.vs[static_cast<size_t>(base + tk) * a.Hkv + hk] : 0.f;
      }
    }
    __syncthreads();
    // ---- request the whole tile: K and V rows (16-byte pieces), zero rows for masked / missing tokens
    constexpr int ROWB = FP8 ? D : D * 2;                       // bytes per token row in the cache
    constexpr int CH = ROWB / 16;
    for (int i = tid; i < ATT_TS * CH; i += 128) {
      const int tok = i / CH, c = i - tok * CH;
      const int tk = stok[tok];
      uint8_t* dk = FP8 ? stage + tok * D + c * 16 : reinterpret_cast<uint8_t*>(Ks + tok * LD) + c * 16;
      uint8_t* dv = FP8 ? stage + (ATT_TS + tok) * D + c * 16 : reinterpret_cast<uint8_t*>(Vs + tok * LD) + c * 16;
      if (tk >= 0) {
        const size_t off = (static_cast<size_t>(base + tk) * a.Hkv + hk) * ROWB + c * 16;
        cp_async16(dk, reinterpret_cast<const uint8_t*>(a.kc) + off);
        cp_async16(dv, reinterpret_cast<const uint8_t*>(a.vc) + off);
      } else {
        *reinterpret_cast<uint4*>(dk) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(dv) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_wait_all();
    __syncthreads();
    if (FP8) {                                                  // e4m3 bytes -> bf16 tiles (scales applied to S and P)
      for (int i = tid; i < ATT_TS * (D / 4); i += 128) {
        const int tok = i / (D / 4), c = i - tok * (D / 4);
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint32_t raw = *reinterpret_cast<const uint32_t*>(stage + (which * ATT_TS + tok) * D + c * 4);
          const __nv_fp8_e4m3* f8 = reinterpret_cast<const __nv_fp8_e4m3*>(&raw);
          __nv_bfloat162 b0 = __floats2bfloat162_rn(static_cast<float>(f8[0]), static_cast<float>(f8[1]));
          __nv_bfloat162 b1 = __floats2bfloat162_rn(static_cast<float>(f8[2]), static_cast<float>(f8[3]));
          uint2 ov; ov.x = *reinterpret_cast<uint32_t*>(&b0); ov.y = *reinterpret_cast<uint32_t*>(&b1);
          *reinterpret_cast<uint2*>((which ? Vs : Ks) + tok * LD + c * 4) = ov;
        }
      }
      __syncthreads();
    }
    // ---- S = Q K^T: warp w owns tokens [16w, 16w + 16)
    {
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
      const __nv_bfloat16* q_lo = Qs + g * LD + 2 * t;
      const __nv_bfloat16* q_hi = Qs + (g + 8) * LD + 2 * t;
      const __nv_bfloat16* k0 = Ks + (warp * 16 + g) * LD + 2 * t;
      const __nv_bfloat16* k1 = Ks + (warp * 16 + 8 + g) * LD + 2 * t;
#pragma unroll 4
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(q_lo + kk * 16), a1 = *reinterpret_cast<const uint32_t*>(q_hi + kk * 16);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(q_lo + kk * 16 + 8), a3 = *reinterpret_cast<const uint32_t*>(q_hi + kk * 16 + 8);
        mma_bf16_16816(c0, a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(k0 + kk * 16), *reinterpret_cast<const uint32_t*>(k0 + kk * 16 + 8));
        mma_bf16_16816(c1, a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(k1 + kk * 16), *reinterpret_cast<const uint32_t*>(k1 + kk * 16 + 8));
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float* c = j ? c1 : c0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = g + (e >> 1) * 8, tok = warp * 16 + j * 8 + 2 * t + (e & 1);
          float v = c[e] * a.scale;
          if (FP8) v *= ksc[tok];
          Ss[row * 68 + tok] = stok[tok] >= 0 ? v : -INFINITY;
        }
      }
    }
    __syncthreads();
    // ---- running softmax statistics; P in bf16 relative to the new running maximum (the row sum uses the same
    //      rounded values); alpha rescales what was accumulated under the old maximum
    for (int row = warp * 4; row < warp * 4 + 4; ++row) {
      const float s0v = Ss[row * 68 + lane], s1v = Ss[row * 68 + lane + 32];
      const float mo = m_run[row];
      const float m = fmaxf(mo, warp_max(fmaxf(s0v, s1v)));
      float p0 = m == -INFINITY ? 0.f : __expf(s0v - m), p1 = m == -INFINITY ? 0.f : __expf(s1v - m);
      p0 = __bfloat162float(__float2bfloat16(p0)); p1 = __bfloat162float(__float2bfloat16(p1));
      const float l = warp_sum(p0 + p1);
      Ps[row * 72 + lane] = __float2bfloat16(FP8 ? p0 * vsc[lane] : p0);
      Ps[row * 72 + lane + 32] = __float2bfloat16(FP8 ? p1 * vsc[lane + 32] : p1);
      if (lane == 0) {
        const float al = (mo == -INFINITY) ? 0.f : __expf(mo - m);
        alpha[row] = al;
        l_run[row] = l_run[row] * al + l;
        m_run[row] = m;
      }
    }
    __syncthreads();
    // ---- O = alpha O + P V: warp w owns dims [w D/4, (w+1) D/4)
    {
      const float al_lo = alpha[g], al_hi = alpha[g + 8];
#pragma unroll
      for (int j = 0; j < NT; ++j) { o[j][0] *= al_lo; o[j][1] *= al_lo; o[j][2] *= al_hi; o[j][3] *= al_hi; }
      const __nv_bfloat16* p_lo = Ps + g * 72 + 2 * t;
      const __nv_bfloat16* p_hi = Ps + (g + 8) * 72 + 2 * t;
#pragma unroll
      for (int kk = 0; kk < ATT_TS / 16; ++kk) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(p_lo + kk * 16), a1 = *reinterpret_cast<const uint32_t*>(p_hi + kk * 16);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(p_lo + kk * 16 + 8), a3 = *reinterpret_cast<const uint32_t*>(p_hi + kk * 16 + 8);
        const __nv_bfloat16* vrow = Vs + (kk * 16 + (lane & 15)) * LD + warp * (D / 4);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          uint32_t b0, b1;
          ldmatrix_x2_trans(b0, b1, vrow + j * 8);
          mma_bf16_16816(o[j], a0, a1, a2, a3, b0, b1);
        }
      }
    }
    __syncthreads();                     // the next tile overwrites K, V, P and the token list
  }
  if (tid < rep) {
    a.part_ml[(pbase + static_cast<size_t>(tid) * nsplit) * 2] = m_run[tid];
    a.part_ml[(pbase + static_cast<size_t>(tid) * nsplit) * 2 + 1] = l_run[tid];
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int d = warp * (D / 4) + j * 8 + 2 * t;
    if (g < rep) *reinterpret_cast<float2*>(a.part_o + (pbase + static_cast<size_t>(g) * nsplit) * D + d) = make_float2(o[j][0], o[j][1]);
    if (g + 8 < rep) *reinterpret_cast<float2*>(a.part_o + (pbase + static_cast<size_t>(g + 8) * nsplit) * D + d) = make_float2(o[j][2], o[j][3]);
  }
}

template <int D, bool FP8>
static size_t attn_decode_tc_smem() {
  return static_cast<size_t>(ATT_ROWS + 2 * ATT_TS) * (D + 8) * 2 + ATT_ROWS * 68 * 4 + ATT_ROWS * 72 * 2 + ATT_TS * 12 +
         (FP8 ? 2 * ATT_TS * D : 0);
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
                               float* ik_pool, cudaStream_t s, const int* row_pos0) {
  if (R <= 0) return 0;
  if (D > 256 || idx_dim > 256) return -5;
  AttnDims a{Hq, Hkv, D, rope_dim, gated, qk_norm, idx_heads, idx_dim, block, fp8, eps};
  dim3 grid(R, Hq + 2 * Hkv + idx_heads + (idx_dim > 0 ? 1 : 0));
  const cudaError_t err = spark_launch_pdl(attn_prep_kernel, grid, dim3(128), 0, s, dim3(1, 1, 1), (const __nv_bfloat16*)qkv, ld, a,
                                           q_norm, k_norm, iq_norm, ik_norm, inv_freq, pos, row_kv, row_j, row_pos0, (__nv_bfloat16*)qbuf,
                                           kc, vc, ks, vs, qi_buf, ik_raw, ik_pool);
  return err == cudaSuccess ? 0 : -4;
}

// Launches split + merge for both entry points.  head_dim 64 / 128 / 256 with <= 16 q heads per kv head runs the
// tensor-core kernel; anything else the scalar one (no tree mask there).
template <int D, bool FP8>
static cudaError_t launch_decode_tc(const AttnDecodeArgs& a, dim3 grid, cudaStream_t s, bool pdl) {
  auto kern = attn_decode_tc_kernel<D, FP8>;
  const size_t smem = attn_decode_tc_smem<D, FP8>();
  static bool attr_set = false;
  if (!attr_set) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); attr_set = true; }
  if (pdl) return spark_launch_pdl(kern, grid, dim3(128), smem, s, dim3(1, 1, 1), a);
  kern<<<grid, 128, smem, s>>>(a);
  return cudaGetLastError();
}

static int attn_decode_launch(const void* qbuf, const void* kc, const void* vc, const float* ks, const float* vs, int fp8,
                              const int* pos, const long long* row_kv, const int* sel, const int* sel_n, int sel_ld,
                              const int* row_pos0, const int* row_j, const uint32_t* anc, float* part_o, float* part_ml,
                              int nsplit, const void* qkv, int ld, int gated, int R, int Hq, int Hkv, int D, float scale,
                              void* out, cudaStream_t s, bool pdl, int chunks = 1) {
  dim3 grid(R, Hkv, nsplit);
  const int rep = Hq / Hkv;
  cudaError_t err;
  if ((D == 64 || D == 128 || D == 256) && rep <= ATT_ROWS && (row_pos0 == nullptr) == (row_j == nullptr)) {
    AttnDecodeArgs a{(const __nv_bfloat16*)qbuf, kc, vc, ks, vs, pos, row_kv, sel, sel_n, sel_ld, row_pos0, row_j, anc,
                     part_o, part_ml, Hq, Hkv, scale, chunks < 1 ? 1 : chunks};
    if (D == 64) err = fp8 ? launch_decode_tc<64, true>(a, grid, s, pdl) : launch_decode_tc<64, false>(a, grid, s, pdl);
    else if (D == 128) err = fp8 ? launch_decode_tc<128, true>(a, grid, s, pdl) : launch_decode_tc<128, false>(a, grid, s, pdl);
    else err = fp8 ? launch_decode_tc<256, true>(a, grid, s, pdl) : launch_decode_tc<256, false>(a, grid, s, pdl);
  } else {
    if (D > 256 || rep > ATT_MAXREP || anc != nullptr || chunks > 1) return -5;
    if (fp8)
      attn_decode_kernel<true><<<grid, 256, 0, s>>>((const __nv_bfloat16*)qbuf, kc, vc, ks, vs, pos, row_kv, sel, sel_n, sel_ld,
                                                    part_o, part_ml, Hq, Hkv, D, scale);
    else
      attn_decode_kernel<false><<<grid, 256, 0, s>>>((const __nv_bfloat16*)qbuf, kc, vc, ks, vs, pos, row_kv, sel, sel_n, sel_ld,
                                                     part_o, part_ml, Hq, Hkv, D, scale);
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) return -4;
  if (pdl)
    err = spark_launch_pdl(attn_merge_kernel, dim3(R, Hq), dim3(D), 0, s, dim3(1, 1, 1), (const float*)part_o, (const float*)part_ml,
                           nsplit, (const __nv_bfloat16*)qkv, ld, gated, Hq, D, (__nv_bfloat16*)out);
  else {
    attn_merge_kernel<<<dim3(R, Hq), D, 0, s>>>(part_o, part_ml, nsplit, (const __nv_bfloat16*)qkv, ld, gated, Hq, D, (__nv_bfloat16*)out);
    err = cudaGetLastError();
  }
  return err == cudaSuccess ? 0 : -4;
}

// row_pos0 / row_j (both or neither): first in-flight position of the row's segment and the row's index inside it (the
// row's KV entry sits at row_pos0 + row_j); anc: optional per-row ancestor bitmask over segment rows (tree verify).
extern "C" int spark_attn_decode(const void* qbuf, const void* kc, const void* vc, const float* ks, const float* vs,
                                 int fp8, const int* pos, const long long* row_kv, const int* sel, const int* sel_n,
                                 int sel_ld, float* part_o, float* part_ml, int nsplit, const void* qkv, int ld,
                                 int gated, int R, int Hq, int Hkv, int D, float scale, void* out, cudaStream_t s,
                                 const int* row_pos0, const int* row_j, const unsigned* anc, int chunks) {
  if (R <= 0) return 0;
  return attn_decode_launch(qbuf, kc, vc, ks, vs, fp8, pos, row_kv, sel, sel_n, sel_ld, row_pos0, row_j, anc, part_o, part_ml,
                            nsplit, qkv, ld, gated, R, Hq, Hkv, D, scale, out, s, true, chunks);
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
  if (D > 256 || Hq / Hkv > ATT_ROWS || nsplit <= 0) return -5;
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
  return attn_decode_launch(qbuf, kc, vc, ks, vs, fp8, pos, row_kv, sel, sel_n, sel_ld, nullptr, nullptr, nullptr, part_o,
                            part_ml, nsplit, qkv, ld, gated, R, Hq, Hkv, D, scale, out, s, false);
}
