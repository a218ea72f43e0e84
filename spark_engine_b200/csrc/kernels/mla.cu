// Multi-head latent attention (absorbed form) on a latent KV cache, with the DSA indexer state.
//
//   mla_prep_kernel   per row: RMSNorm of the q and kv low-rank activations, RoPE of the shared rope key, latent row
//                     [kv_lora | rope] appended to the cache; indexer key (LayerNorm), pool gate and per-head index
//                     weights; when the row closes a 4-token pool: pooled key = sum_j softmax_j(gate_j + ape_j) key_j.
//   mla_qrope_kernel  rotary part of the queries into the tail of the absorbed query rows.
//   mla_decode_kernel scores, softmax and P.V over one 64-token split of a row's visible tokens for ALL heads of the
//                     row at once: the heads are the M dimension of the MMA tiles (every head reads the same latent
//                     row, which is both key and value), so the latent tile is fetched once per split and used by
//                     64 heads.  mma.sync m16n8k16 bf16, ldmatrix-fed; token gather by cp.async from the selection.
//   mla_merge_kernel  ordered merge of the splits (+ attention sink in the denominator), bf16 latent-space output.
// FP8 cache rows (lat_fp8): [kv_lora e4m3 | 4 fp32 tile scales (tiles of kv_lora / max(1, kv_lora / 128)) | rope bf16],
// 656 bytes instead of 1152 for 512 + 64; the decode kernel copies the packed row into the tail of its bf16 tile row and
// a warp expands it in place.
// The visible tokens of a row come from the top-k pool selection (sparse_select.cu) or are 0..pos.
// Reference: engine-rs/shim/latent.cu (sparse_latent*, latent_tc16*, merge_latent), ds41_attn.cu:90-424,
// engine-rs/src/mla_latent.rs:36-38,196-248, dsa.rs:127-230; FP8 rows: latent.cu:25-47.
#include <cuda_fp8.h>
#include "../common/ptx.cuh"

namespace spark {

struct MlaDims {
  int q_lora, kv_lora, rope, idx_dim, idx_heads, pool;
  float eps;
};

__device__ __forceinline__ float block_sum_128(float v, float* red) {      // 128 threads
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  const float t = red[0] + red[1] + red[2] + red[3];
  __syncthreads();
  return t;
}

// LayerNorm'ed indexer key and gate of row `a` for channel d (whole block cooperates on the statistics)
__device__ __forceinline__ void idx_key_gate(const __nv_bfloat16* a, int o1, int Dm, const float* lw, const float* lb,
                                             float* red, float& key, float& gate) {
  const int d = threadIdx.x;
  const float x = d < Dm ? __bfloat162float(a[o1 + d]) : 0.f;
  const float mu = block_sum_128(x, red) / Dm;
  const float dv = d < Dm ? x - mu : 0.f;
  const float var = block_sum_128(dv * dv, red) / Dm;
  key = d < Dm ? dv * rsqrtf(var + 1e-6f) * lw[d] + lb[d] : 0.f;
  gate = d < Dm ? __bfloat162float(a[o1 + Dm + d]) : 0.f;
}

// grid R; 128 threads.  a: [R, q_lora + kv_lora + rope + 2*idx_dim + idx_heads] bf16.
__global__ void __launch_bounds__(128)
mla_prep_kernel(const __nv_bfloat16* __restrict__ a, int lda, MlaDims dm, const float* __restrict__ q_norm,
                const float* __restrict__ kv_norm, const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                const float* __restrict__ ape, const double* __restrict__ inv_freq, const int* __restrict__ pos,
                const long long* __restrict__ row_kv, const int* __restrict__ row_j,
                __nv_bfloat16* __restrict__ cq, __nv_bfloat16* __restrict__ lat, float* __restrict__ ik,
                float* __restrict__ ig, float* __restrict__ pool, float* __restrict__ hw,
                const int* __restrict__ row_pos0, int lat_fp8) {
  __shared__ float red[4];
  __shared__ int tmax[4];
  const int r = blockIdx.x, t = threadIdx.x;
  const __nv_bfloat16* ar = a + static_cast<size_t>(r) * lda;
  const int p = pos[r];
  // rows of a verification tree (row_pos0 given) are rotated at their depth position p but stored at the slot of
  // their node, first in-flight slot + node index; their pools are finished when the accepted path is compacted
  const long long tok = row_kv[r] + (row_pos0 ? row_pos0[r] + row_j[r] : p);
  const int KW = dm.kv_lora + dm.rope;
  // q low-rank activation
  float ss = 0.f;
  for (int i = t; i < dm.q_lora; i += 128) { const float x = __bfloat162float(ar[i]); ss = fmaf(x, x, ss); }
  float rs = rsqrtf(block_sum_128(ss, red) / dm.q_lora + dm.eps);
  for (int i = t; i < dm.q_lora; i += 128)
    cq[static_cast<size_t>(r) * dm.q_lora + i] = __float2bfloat16(__bfloat162float(ar[i]) * rs * q_norm[i]);
  // latent row
  const __nv_bfloat16* akv = ar + dm.q_lora;
  ss = 0.f;
  for (int i = t; i < dm.kv_lora; i += 128) { const float x = __bfloat162float(akv[i]); ss = fmaf(x, x, ss); }
  rs = rsqrtf(block_sum_128(ss, red) / dm.kv_lora + dm.eps);
  __nv_bfloat16* lrow = lat + tok * KW;
  if (lat_fp8) {
    const int nt8 = max(1, dm.kv_lora >> 7), tw = dm.kv_lora / nt8;
    uint8_t* brow = reinterpret_cast<uint8_t*>(lat) + tok * (dm.kv_lora + 16 + 2 * dm.rope);
    if (t < 4) tmax[t] = 0;
    __syncthreads();
    for (int i = t; i < dm.kv_lora; i += 128)
      atomicMax(&tmax[i / tw], __float_as_int(fabsf(__bfloat162float(akv[i]) * rs * kv_norm[i])));   // non-negative floats order as ints
    __syncthreads();
    for (int i = t; i < dm.kv_lora; i += 128) {
      const float amax = __int_as_float(tmax[i / tw]);
      const float sc = amax > 0.f ? amax / 448.f : 1.f;
      brow[i] = __nv_cvt_float_to_fp8(__bfloat162float(akv[i]) * rs * kv_norm[i] / sc, __NV_SATFINITE, __NV_E4M3);
    }
    if (t < 4) {
      const float amax = __int_as_float(tmax[t]);
      reinterpret_cast<float*>(brow + dm.kv_lora)[t] = t < nt8 ? (amax > 0.f ? amax / 448.f : 1.f) : 0.f;
    }
    lrow = reinterpret_cast<__nv_bfloat16*>(brow + dm.kv_lora + 16) - dm.kv_lora;     // rope tail written below
  } else {
    for (int i = t; i < dm.kv_lora; i += 128) lrow[i] = __float2bfloat16(__bfloat162float(akv[i]) * rs * kv_norm[i]);
  }
  const int half = dm.rope >> 1;
  for (int i = t; i < half; i += 128) {
    const float x1 = __bfloat162float(akv[dm.kv_lora + i]), x2 = __bfloat162float(akv[dm.kv_lora + half + i]);
    const float ang = static_cast<float>(static_cast<double>(p) * inv_freq[i]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    lrow[dm.kv_lora + i] = __float2bfloat16(x1 * cs - x2 * sn);
    lrow[dm.kv_lora + half + i] = __float2bfloat16(x2 * cs + x1 * sn);
  }
  // indexer state
  const int o1 = dm.q_lora + KW, Dm = dm.idx_dim;
  float key, gate;
  idx_key_gate(ar, o1, Dm, ln_w, ln_b, red, key, gate);
  if (t < Dm) { ik[tok * Dm + t] = key; ig[tok * Dm + t] = gate; }
  if (t < dm.idx_heads) hw[static_cast<size_t>(r) * dm.idx_heads + t] = __bfloat162float(ar[o1 + 2 * Dm + t]) * rsqrtf(static_cast<float>(dm.idx_heads));
  if (!row_pos0 && (p + 1) % dm.pool == 0) {
    // this row closes a pool: gates/keys of the earlier tokens come from this launch's rows when they belong to
    // the same segment (their cache entries may not be written yet), else from the cache
    float gmax = gate + ape[(dm.pool - 1) * Dm + (t < Dm ? t : 0)];
    float kj[8], gj[8];
    kj[dm.pool - 1] = key; gj[dm.pool - 1] = gmax;
    for (int j = 0; j < dm.pool - 1; ++j) {
      const int back = dm.pool - 1 - j;                         // rows before this one
      float k2, g2;
      if (back <= row_j[r]) {
        idx_key_gate(a + static_cast<size_t>(r - back) * lda, o1, Dm, ln_w, ln_b, red, k2, g2);
      } else {
        k2 = t < Dm ? ik[(tok - back) * Dm + t] : 0.f;
        g2 = t < Dm ? ig[(tok - back) * Dm + t] : 0.f;
      }
      g2 += ape[j * Dm + (t < Dm ? t : 0)];
      kj[j] = k2; gj[j] = g2;
      gmax = fmaxf(gmax, g2);
    }
    float den = 0.f, num = 0.f;
    for (int j = 0; j < dm.pool; ++j) { const float e = __expf(gj[j] - gmax); den += e; num = fmaf(e, kj[j], num); }
    if (t < Dm) pool[(row_kv[r] / dm.pool + p / dm.pool) * Dm + t] = num / den;
  }
}

// grid (R, H); rope/2 threads.  qb: [R, H*(D+rope) + ...] bf16; q_full: [R, H, kv_lora + rope] bf16 (tail written here)
__global__ void mla_qrope_kernel(const __nv_bfloat16* __restrict__ qb, int ldq, int D, int rope, int kv_lora,
                                 const double* __restrict__ inv_freq, const int* __restrict__ pos,
                                 __nv_bfloat16* __restrict__ q_full, int H) {
  const int r = blockIdx.x, h = blockIdx.y, i = threadIdx.x, half = rope >> 1;
  if (i >= half) return;
  const __nv_bfloat16* q = qb + static_cast<size_t>(r) * ldq + h * (D + rope) + D;
  const float x1 = __bfloat162float(q[i]), x2 = __bfloat162float(q[half + i]);
  const float ang = static_cast<float>(static_cast<double>(pos[r]) * inv_freq[i]);
  float sn, cs;
  sincosf(ang, &sn, &cs);
  __nv_bfloat16* o = q_full + (static_cast<size_t>(r) * H + h) * (kv_lora + rope) + kv_lora;
  o[i] = __float2bfloat16(x1 * cs - x2 * sn);
  o[half + i] = __float2bfloat16(x2 * cs + x1 * sn);
}

// ------------------------------------------------------------------------------------------------ attention
constexpr int MLA_TS = 64;          // tokens per split

__device__ __forceinline__ void mla_cp16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void mla_ldsm4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mla_ldsm4t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mla_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (R, ceil(nsplit / spc)); 256 threads; a CTA walks `spc` consecutive splits.  HM = 16-head MMA tiles (H <= 16*HM).  KW = kv_lora + rope (multiple of 16),
// L = kv_lora (multiple of 16).
template <int HM>
__global__ void __launch_bounds__(256)
mla_decode_kernel(const __nv_bfloat16* __restrict__ q_full,      // [R, H, KW]
                  const __nv_bfloat16* __restrict__ lat,         // [tokens, KW]
                  const int* __restrict__ pos, const long long* __restrict__ row_kv, const int* __restrict__ sel,
                  const int* __restrict__ sel_n, int sel_ld, float* __restrict__ part_o,   // [R, H, nsplit, L]
                  float* __restrict__ part_ml,                   // [R, H, nsplit, 2]
                  int H, int KW, int L, float scale, int nsplit, int spc,
                  const int* __restrict__ row_pos0, const int* __restrict__ row_j, const int* __restrict__ anc,
                  int lat_fp8) {
  extern __shared__ __align__(16) uint8_t smem_mla[];
  const int LDK = KW + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_mla);          // [HM*16][LDK]
  __nv_bfloat16* Ls = Qs + HM * 16 * LDK;                                   // [64][LDK]
  float* Ss = reinterpret_cast<float*>(Ls + MLA_TS * LDK);                  // [HM*16][65]
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(Ss + HM * 16 * 65);  // [HM*16][72]
  __shared__ int stok[MLA_TS];
  const int r = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  // tree rows (anc given, no selection): the committed context [0, first in-flight slot) plus the in-flight slots
  // of the row's ancestors and its own, bit j of anc[r] = node j of the sequence is visible
  const bool tree = anc != nullptr;
  const int tp0 = tree ? row_pos0[r] : 0;
  const unsigned amask = tree ? static_cast<unsigned>(anc[r]) : 0u;
  const int n_ctx = sel ? sel_n[r] : (tree ? tp0 + row_j[r] + 1 : pos[r] + 1);
  const long long base = row_kv[r];
  const int VPR = KW >> 3;
  // the row's queries (all heads) are staged once and serve every split this CTA walks through
  for (int i = tid; i < HM * 16 * VPR; i += 256) {
    const int h = i / VPR, v = i - h * VPR;
    if (h < H) mla_cp16(Qs + h * LDK + v * 8, q_full + (static_cast<size_t>(r) * H + h) * KW + v * 8);
    else *reinterpret_cast<uint4*>(Qs + h * LDK + v * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  for (int sp = blockIdx.y * spc; sp < min(nsplit, (blockIdx.y + 1) * spc); ++sp) {
  const int t0 = sp * MLA_TS;
  const size_t pb = (static_cast<size_t>(r) * H) * nsplit + sp;
  if (t0 >= n_ctx) {                                           // empty split: neutral partial
    for (int h = tid; h < H; h += 256) {
      part_ml[(pb + static_cast<size_t>(h) * nsplit) * 2] = -INFINITY;
      part_ml[(pb + static_cast<size_t>(h) * nsplit) * 2 + 1] = 0.f;
    }
    continue;
  }
  const int nt = min(MLA_TS, n_ctx - t0);
  __syncthreads();                                             // the previous split's tiles are no longer read
  if (tid < MLA_TS) stok[tid] = tid < nt ? (sel ? sel[static_cast<size_t>(r) * sel_ld + t0 + tid] : t0 + tid) : -1;
  __syncthreads();
  if (!lat_fp8) {
    for (int i = tid; i < MLA_TS * VPR; i += 256) {
      const int k = i / VPR, v = i - k * VPR;
      if (stok[k] >= 0) mla_cp16(Ls + k * LDK + v * 8, lat + (base + stok[k]) * KW + v * 8);
      else *reinterpret_cast<uint4*>(Ls + k * LDK + v * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
  } else {
    // packed rows land at byte L of their tile row (the row is 2 KW + 16 bytes, the packed row L + 16 + 2 rope), then
    // one warp per row expands them in place: every lane reads its 16 codes, its scale and its piece of the rope
    // tail into registers before any lane writes
    const int RB = L + 16 + 2 * (KW - L), CH = RB >> 4;
    const uint8_t* lat8 = reinterpret_cast<const uint8_t*>(lat);
    for (int i = tid; i < MLA_TS * CH; i += 256) {
      const int k = i / CH, v = i - k * CH;
      if (stok[k] >= 0) mla_cp16(reinterpret_cast<uint8_t*>(Ls + k * LDK) + L + v * 16, lat8 + (base + stok[k]) * RB + v * 16);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    const int nt8 = max(1, L >> 7), tw = L / nt8, rch = (KW - L) >> 3;
    for (int k = warp; k < MLA_TS; k += 8) {
      uint8_t* rowb = reinterpret_cast<uint8_t*>(Ls + k * LDK);
      if (stok[k] < 0) {
        for (int v = lane; v < VPR; v += 32) *reinterpret_cast<uint4*>(rowb + v * 16) = make_uint4(0u, 0u, 0u, 0u);
        continue;
      }
      const bool mine = lane < (L >> 4);
      uint4 q = make_uint4(0u, 0u, 0u, 0u), rp = q;
      float sc = 0.f;
      if (mine) {
        q = *reinterpret_cast<const uint4*>(rowb + L + lane * 16);
        sc = *reinterpret_cast<const float*>(rowb + 2 * L + (lane * 16 / tw) * 4);
      }
      if (lane < rch) rp = *reinterpret_cast<const uint4*>(rowb + 2 * L + 16 + lane * 16);
      __syncwarp();
      if (mine) {
        const uint16_t* q2 = reinterpret_cast<const uint16_t*>(&q);
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(q2[j], __NV_E4M3);
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
          const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * sc, f.y * sc);
          o[j] = *reinterpret_cast<const uint32_t*>(&b);
        }
        *reinterpret_cast<uint4*>(rowb + lane * 32) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(rowb + lane * 32 + 16) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      if (lane < rch) *reinterpret_cast<uint4*>(rowb + 2 * L + lane * 16) = rp;
    }
    __syncthreads();
  }
  // ---- phase 1: S[h][tok] for this warp's 8 tokens, all head tiles
  {
    float s[HM][4];
#pragma unroll
    for (int m = 0; m < HM; ++m) { s[m][0] = 0.f; s[m][1] = 0.f; s[m][2] = 0.f; s[m][3] = 0.f; }
    for (int ks = 0; ks < KW / 16; ks += 2) {
      // B: tokens 8*warp..+7; matrices (k0..7), (k8..15) of step ks and of step ks+1
      uint32_t b[4];
      const bool two = ks + 1 < KW / 16;
      mla_ldsm4(b, Ls + (warp * 8 + (lane & 7)) * LDK + ks * 16 + (two ? (lane >> 3) * 8 : ((lane >> 3) & 1) * 8));
#pragma unroll
      for (int m = 0; m < HM; ++m) {
        uint32_t a[4];
        mla_ldsm4(a, Qs + (m * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + ks * 16 + (lane >> 4) * 8);
        mla_mma(s[m], a, b[0], b[1]);
        if (two) {
          mla_ldsm4(a, Qs + (m * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (ks + 1) * 16 + (lane >> 4) * 8);
          mla_mma(s[m], a, b[2], b[3]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < HM; ++m) {
      const int c = warp * 8 + 2 * t;
      Ss[(m * 16 + g) * 65 + c] = s[m][0] * scale; Ss[(m * 16 + g) * 65 + c + 1] = s[m][1] * scale;
      Ss[(m * 16 + g + 8) * 65 + c] = s[m][2] * scale; Ss[(m * 16 + g + 8) * 65 + c + 1] = s[m][3] * scale;
    }
  }
  __syncthreads();
  // ---- phase 2: per-head softmax statistics over the split; P (bf16) for the second product
  for (int h = warp; h < HM * 16; h += 8) {
    bool v0 = lane < nt, v1 = lane + 32 < nt;
    if (tree) {
      const int k0 = t0 + lane - tp0, k1 = k0 + 32;
      v0 = v0 && (k0 < 0 || (k0 < 32 && ((amask >> k0) & 1u)));
      v1 = v1 && (k1 < 0 || (k1 < 32 && ((amask >> k1) & 1u)));
    }
    const float s0 = v0 ? Ss[h * 65 + lane] : -INFINITY;
    const float s1 = v1 ? Ss[h * 65 + lane + 32] : -INFINITY;
    const float m = warp_max(fmaxf(s0, s1));                     // -inf when the split holds no visible token
    const float e0 = v0 ? __expf(s0 - m) : 0.f, e1 = v1 ? __expf(s1 - m) : 0.f;
    const float l = warp_sum(e0 + e1);
    Ps[h * 72 + lane] = __float2bfloat16(e0);
    Ps[h * 72 + lane + 32] = __float2bfloat16(e1);
    if (lane == 0 && h < H) {
      part_ml[(pb + static_cast<size_t>(h) * nsplit) * 2] = m;
      part_ml[(pb + static_cast<size_t>(h) * nsplit) * 2 + 1] = l;
    }
  }
  __syncthreads();
  // ---- phase 3: O[h][d] = sum_tok P[h][tok] lat[tok][d]; column pairs (16 wide) round-robin over the warps
  for (int np = warp; np < L / 16; np += 8) {
    float o[HM][2][4];
#pragma unroll
    for (int m = 0; m < HM; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) { o[m][0][j] = 0.f; o[m][1][j] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < MLA_TS / 16; ++kk) {
      uint32_t b[4];
      mla_ldsm4t(b, Ls + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDK + np * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int m = 0; m < HM; ++m) {
        uint32_t a[4];
        mla_ldsm4(a, Ps + (m * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * 72 + kk * 16 + (lane >> 4) * 8);
        mla_mma(o[m][0], a, b[0], b[1]);
        mla_mma(o[m][1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int m = 0; m < HM; ++m) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int h = m * 16 + g + hh * 8;
        if (h < H) {
          float* dst = part_o + (pb + static_cast<size_t>(h) * nsplit) * L + np * 16 + 2 * t;
          *reinterpret_cast<float2*>(dst) = make_float2(o[m][0][2 * hh], o[m][0][2 * hh + 1]);
          *reinterpret_cast<float2*>(dst + 8) = make_float2(o[m][1][2 * hh], o[m][1][2 * hh + 1]);
        }
      }
    }
  }
  }   // splits of this CTA
  asm volatile("cp.async.wait_all;" ::: "memory");               // the query copy, if every split was empty
}

// grid (R, ceil(H / hpc)); 256 threads.  Splits merged in ascending order; `sink` (per head, optional) joins the
// denominator.  A CTA owns `hpc` heads of one row: the per-head weights of the splits are computed once into shared
// memory, then the threads sweep the hpc x L outputs with 16-byte loads.  The launcher picks hpc so that a decode
// round of a few rows still fills the SMs (one head per CTA), while a prefill chunk keeps one CTA per row.
__global__ void __launch_bounds__(256)
mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int nsplit, const float* __restrict__ sink,
                 int H, int L, int hpc, __nv_bfloat16* __restrict__ out) {
  extern __shared__ float wts[];                        // [hpc][nsplit]: exp(m_s - M) / l
  const int r = blockIdx.x, h0 = blockIdx.y * hpc;
  const int nh = min(hpc, H - h0);
  for (int hl = threadIdx.x; hl < nh; hl += blockDim.x) {
    const int h = h0 + hl;
    const size_t pb = (static_cast<size_t>(r) * H + h) * nsplit;
    float M = sink ? sink[h] : -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(pb + s) * 2]);
    float l = sink ? __expf(sink[h] - M) : 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float m = part_ml[(pb + s) * 2];
      if (m != -INFINITY) l += __expf(m - M) * part_ml[(pb + s) * 2 + 1];
    }
    const float inv = 1.f / l;
    for (int s = 0; s < nsplit; ++s) {
      const float m = part_ml[(pb + s) * 2];
      wts[hl * nsplit + s] = m != -INFINITY ? __expf(m - M) * inv : 0.f;
    }
  }
  __syncthreads();
  const int L4 = L >> 2;
  for (int i = threadIdx.x; i < nh * L4; i += blockDim.x) {
    const int hl = i / L4, d = (i - hl * L4) * 4, h = h0 + hl;
    const size_t pb = (static_cast<size_t>(r) * H + h) * nsplit;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < nsplit; ++s) {
      const float w = wts[hl * nsplit + s];
      if (w != 0.f) {
        const float4 p = *reinterpret_cast<const float4*>(part_o + (pb + s) * L + d);
        o.x = fmaf(w, p.x, o.x); o.y = fmaf(w, p.y, o.y); o.z = fmaf(w, p.z, o.z); o.w = fmaf(w, p.w, o.w);
      }
    }
    const __nv_bfloat162 b0 = __floats2bfloat162_rn(o.x, o.y), b1 = __floats2bfloat162_rn(o.z, o.w);
    uint2 ov; ov.x = *reinterpret_cast<const uint32_t*>(&b0); ov.y = *reinterpret_cast<const uint32_t*>(&b1);
    *reinterpret_cast<uint2*>(out + (static_cast<size_t>(r) * H + h) * L + d) = ov;
  }
}

}  // namespace spark

using namespace spark;

// Shapes the packed FP8 rows cover: at most four scale tiles, 16 codes per lane of one warp, 16-byte pieces.
static bool mla_fp8_ok(int kv_lora, int rope) {
  const int nt8 = kv_lora >= 128 ? kv_lora / 128 : 1;
  return kv_lora <= 512 && kv_lora % 16 == 0 && kv_lora % nt8 == 0 && (kv_lora / nt8) % 16 == 0 && rope % 8 == 0 && rope <= 256;
}

extern "C" int spark_mla_prep(const void* a, int lda, int R, int q_lora, int kv_lora, int rope, int idx_dim, int idx_heads,
                              int pool_sz, float eps, const float* q_norm, const float* kv_norm, const float* ln_w,
                              const float* ln_b, const float* ape, const double* inv_freq, const int* pos,
                              const long long* row_kv, const int* row_j, void* cq, void* lat, float* ik, float* ig,
                              float* pool, float* hw, cudaStream_t s, const int* row_pos0, int lat_fp8) {
  if (R <= 0) return 0;
  if (idx_dim > 128 || idx_heads > 128 || pool_sz > 8 || pool_sz < 1 || (rope & 1)) return -5;
  if (lat_fp8 && !mla_fp8_ok(kv_lora, rope)) return -5;
  MlaDims dm{q_lora, kv_lora, rope, idx_dim, idx_heads, pool_sz, eps};
  mla_prep_kernel<<<R, 128, 0, s>>>((const __nv_bfloat16*)a, lda, dm, q_norm, kv_norm, ln_w, ln_b, ape, inv_freq, pos, row_kv,
                                    row_j, (__nv_bfloat16*)cq, (__nv_bfloat16*)lat, ik, ig, pool, hw, row_pos0, lat_fp8);
  return spark_launch_rc(__func__);
}

extern "C" int spark_mla_qrope(const void* qb, int ldq, int R, int H, int D, int rope, int kv_lora, const double* inv_freq,
                               const int* pos, void* q_full, cudaStream_t s) {
  if (R <= 0 || rope <= 0) return 0;
  if (rope > 512) return -5;
  mla_qrope_kernel<<<dim3(R, H), (rope / 2 + 31) / 32 * 32, 0, s>>>((const __nv_bfloat16*)qb, ldq, D, rope, kv_lora, inv_freq, pos,
                                                                    (__nv_bfloat16*)q_full, H);
  return spark_launch_rc(__func__);
}

// part_o: fp32 [R, H, nsplit, L]; part_ml: fp32 [R, H, nsplit, 2]; out: bf16 [R, H, L].
extern "C" int spark_mla_attn(const void* q_full, const void* lat, const int* pos, const long long* row_kv, const int* sel,
                              const int* sel_n, int sel_ld, float* part_o, float* part_ml, int nsplit, const float* sink,
                              int R, int H, int kv_lora, int rope, float scale, void* out, cudaStream_t s,
                              const int* row_pos0, const int* row_j, const int* anc, int lat_fp8) {
  if (R <= 0) return 0;
  const int KW = kv_lora + rope;
  if (lat_fp8 && !mla_fp8_ok(kv_lora, rope)) return -5;
  if (H > 64 || (KW & 15) || (kv_lora & 15) || nsplit <= 0) return -5;
  if (anc && (sel || !row_pos0 || !row_j)) return -5;          // tree rows read a dense context
  const int HM = H <= 16 ? 1 : (H <= 32 ? 2 : 4);
  const int smem = (HM * 16 + MLA_TS) * (KW + 8) * 2 + HM * 16 * 65 * 4 + HM * 16 * 72 * 2;
  if (smem > 200 * 1024) return -6;
  void (*kern)(const __nv_bfloat16*, const __nv_bfloat16*, const int*, const long long*, const int*, const int*, int, float*,
               float*, int, int, int, float, int, int, const int*, const int*, const int*, int) = HM == 1 ? mla_decode_kernel<1> : (HM == 2 ? mla_decode_kernel<2> : mla_decode_kernel<4>);
  static bool done[3] = {false, false, false};
  const int id = HM == 1 ? 0 : (HM == 2 ? 1 : 2);
  if (!done[id]) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); done[id] = true; }
  // few rows (decode): one split per CTA for parallelism; many rows (prefill): a CTA per row walks all its splits
  const int spc = R >= 128 ? nsplit : (R >= 32 ? 4 : 1);
  kern<<<dim3(R, (nsplit + spc - 1) / spc), 256, smem, s>>>((const __nv_bfloat16*)q_full, (const __nv_bfloat16*)lat, pos, row_kv,
                                                            sel, sel_n, sel_ld, part_o, part_ml, H, KW, kv_lora, scale, nsplit, spc,
                                                            row_pos0, row_j, anc, lat_fp8);
  if (H * nsplit * 4 > 48 * 1024) return -6;
  int hpc = H;                                          // heads per merge CTA: enough CTAs for two per SM when rows are few
  while (hpc > 1 && R * ((H + hpc - 1) / hpc) < 296) hpc = (hpc + 1) / 2;
  const int L4 = kv_lora >> 2;
  const int mthreads = hpc * L4 >= 256 ? 256 : ((hpc * L4 + 31) / 32 * 32);
  mla_merge_kernel<<<dim3(R, (H + hpc - 1) / hpc), mthreads, hpc * nsplit * 4, s>>>(part_o, part_ml, nsplit, sink, H, kv_lora, hpc,
                                                                                  (__nv_bfloat16*)out);
  return spark_launch_rc(__func__);
}
