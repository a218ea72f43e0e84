// Causal GQA attention for prefill segments (dense context, bf16 KV cache): flash-style streaming softmax on
// tensor cores.  One CTA = 64 query rows of one q head; 4 warps x 16 rows; key/value tiles of 64 tokens are
// double-buffered with cp.async; S = Q K^T and O += P V run on mma.sync m16n8k16 (bf16, fp32 accumulate) with
// ldmatrix-fed fragments; P never leaves registers.  The rows of a segment see the committed prefix of their
// sequence (already in the cache) plus the rows before them in the segment (stored by the prep kernel of the same
// step).  Epilogue: 1/l, optional sigmoid output gate, bf16 store.  One CTA owns a (row tile, head) from first key
// to last, so results are run-to-run identical.
// Serves: GQA / QSA layers while the context is below the sparse-selection threshold (engine-rs/shim/qwen_qsa.cu
// attn paths; the reference runs prefill rows through the same per-row kernel as decode).
#include "../common/ptx.cuh"

namespace spark {

constexpr int PF_BM = 64, PF_BN = 64;

__device__ __forceinline__ void pf_cp16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// grid (row tiles, Hq, segments); 128 threads.  MASK: rows also carry a bit per 4-token key block (bmask [R, mw] words,
// bit b of a row = block b may be attended): block-sparse selections of a few thousand tokens run through the dense
// tiles with the unselected blocks masked, which beats one gathering CTA per row while the context is short enough.
template <int D, bool MASK>
__global__ void __launch_bounds__(128)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ qbuf,        // [R, Hq, D]
                    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,   // [tokens, Hkv, D]
                    const long long* __restrict__ row_kv, const int* __restrict__ seg,
                    const __nv_bfloat16* __restrict__ qkv, int ld, int gated,
                    __nv_bfloat16* __restrict__ out, int Hq, int Hkv, float scale_log2,
                    const uint32_t* __restrict__ bmask, int mw) {
  constexpr int LDS = D + 8;                                // smem row stride (elements): 16 bytes past a 128-byte multiple
  extern __shared__ __align__(16) uint8_t smem_pf[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_pf);        // [64][LDS]
  __nv_bfloat16* Ks = Qs + PF_BM * LDS;                                  // [2][64][LDS]
  __nv_bfloat16* Vs = Ks + 2 * PF_BN * LDS;                              // [2][64][LDS]
  const int sg = blockIdx.z, h = blockIdx.y;
  const int qt = gridDim.x - 1 - blockIdx.x;                 // longest row tiles (most key tiles) are scheduled first
  const int r0 = seg[sg * 4 + 1], n = seg[sg * 4 + 2], pos0 = seg[sg * 4 + 3];
  if (qt * PF_BM >= n) return;
  const int hk = h / (Hq / Hkv);
  const long long base = row_kv[r0];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int rows_valid = min(PF_BM, n - qt * PF_BM);
  const int nkeys = pos0 + qt * PF_BM + rows_valid;           // keys visible to the last valid row of the tile
  const int ntiles = (nkeys + PF_BN - 1) / PF_BN;
  constexpr int VPR = D / 8;                                  // 16-byte vectors per row

  auto load_kv = [&](int j, int buf) {
    __nv_bfloat16* kd = Ks + buf * PF_BN * LDS;
    __nv_bfloat16* vd = Vs + buf * PF_BN * LDS;
    for (int i = tid; i < PF_BN * VPR; i += 128) {
      const int r = i / VPR, v = i - r * VPR;
      const int key = j * PF_BN + r;
      if (key < nkeys) {
        const size_t off = (static_cast<size_t>(base + key) * Hkv + hk) * D + v * 8;
        pf_cp16(kd + r * LDS + v * 8, kc + off);
        pf_cp16(vd + r * LDS + v * 8, vc + off);
      } else {
        *reinterpret_cast<uint4*>(kd + r * LDS + v * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vd + r * LDS + v * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  for (int i = tid; i < PF_BM * VPR; i += 128) {
    const int r = i / VPR, v = i - r * VPR;
    const int rr = min(r, rows_valid - 1);                     // padded rows repeat the last valid row
    pf_cp16(Qs + r * LDS + v * 8, qbuf + (static_cast<size_t>(r0 + qt * PF_BM + rr) * Hq + h) * D + v * 8);
  }
  load_kv(0, 0);
  pf_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  // query positions of this thread's two rows (padded rows: the last valid row's)
  const int p_lo = pos0 + qt * PF_BM + min(warp * 16 + g, rows_valid - 1);
  const int p_hi = pos0 + qt * PF_BM + min(warp * 16 + g + 8, rows_valid - 1);
  const uint32_t* bm_lo = MASK ? bmask + static_cast<size_t>(r0 + p_lo - pos0) * mw : nullptr;
  const uint32_t* bm_hi = MASK ? bmask + static_cast<size_t>(r0 + p_hi - pos0) * mw : nullptr;

  for (int j = 0; j < ntiles; ++j) {
    const int buf = j & 1;
    pf_wait<0>();
    __syncthreads();
    if (j + 1 < ntiles) { load_kv(j + 1, buf ^ 1); pf_commit(); }
    const __nv_bfloat16* kb = Ks + buf * PF_BN * LDS;
    const __nv_bfloat16* vb = Vs + buf * PF_BN * LDS;
    // ---- S = Q K^T : 16 rows x 64 keys per warp
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = 0.f; s[i][1] = 0.f; s[i][2] = 0.f; s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldsm4(a, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldsm4(b, kb + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * LDS + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], a, b[0], b[1]);
        mma_bf16(s[2 * np + 1], a, b[2], b[3]);
      }
    }
    // ---- scale, causal mask, streaming softmax
    const int k0 = j * PF_BN;
    const bool need_mask = k0 + PF_BN - 1 > pos0 + qt * PF_BM;
    // 16 block bits of this 64-key tile for the thread's two rows (a word covers two tiles)
    const uint32_t sel_lo = MASK ? (__ldg(bm_lo + (j >> 1)) >> ((j & 1) * 16)) : 0u;
    const uint32_t sel_hi = MASK ? (__ldg(bm_hi + (j >> 1)) >> ((j & 1) * 16)) : 0u;
    float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[i][e] * scale_log2;
        if (need_mask) {
          const int key = k0 + i * 8 + 2 * t + (e & 1);
          if (key > ((e >> 1) ? p_hi : p_lo)) v = -INFINITY;
        }
        if (MASK && !((((e >> 1) ? sel_hi : sel_lo) >> (i * 2 + (t >> 1))) & 1u)) v = -INFINITY;
        s[i][e] = v;
      }
      mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    // dense: key 0 is visible to every row, so mx is finite.  Masked: a row may have seen no key yet (mx = -inf):
    // exponentials are then taken against 0, every term is exp2(-inf) = 0 and the running sums stay 0.
    const float f_lo = (MASK && mx_lo == -INFINITY) ? 0.f : mx_lo, f_hi = (MASK && mx_hi == -INFINITY) ? 0.f : mx_hi;
    const float c_lo = exp2f(m_lo - f_lo), c_hi = exp2f(m_hi - f_hi);
    m_lo = mx_lo; m_hi = mx_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s[i][0] = exp2f(s[i][0] - f_lo); s[i][1] = exp2f(s[i][1] - f_lo);
      s[i][2] = exp2f(s[i][2] - f_hi); s[i][3] = exp2f(s[i][3] - f_hi);
      sum_lo += s[i][0] + s[i][1]; sum_hi += s[i][2] + s[i][3];
    }
    l_lo = l_lo * c_lo + sum_lo; l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi; }
    // ---- O += P V : P from the score registers (bf16), V fragments via transposed ldmatrix
#pragma unroll
    for (int kk = 0; kk < PF_BN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]); a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]); a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        uint32_t b[4];
        ldsm4t(b, vb + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + np * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * np], a, b[0], b[1]);
        mma_bf16(o[2 * np + 1], a, b[2], b[3]);
      }
    }
  }
  // ---- epilogue: row sums over the quad, normalise, gate, store
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = 1.f / l_lo, inv_hi = 1.f / l_hi;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int rl = warp * 16 + g + hh * 8;
    if (rl >= rows_valid) continue;
    const size_t r = static_cast<size_t>(r0 + qt * PF_BM + rl);
    const float inv = hh ? inv_hi : inv_lo;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int d = i * 8 + 2 * t;
      float v0 = o[i][2 * hh] * inv, v1 = o[i][2 * hh + 1] * inv;
      if (gated) {
        const float2 gt = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qkv + r * ld + h * 2 * D + D + d));
        v0 = v0 / (1.f + __expf(-gt.x)); v1 = v1 / (1.f + __expf(-gt.y));
      }
      *reinterpret_cast<__nv_bfloat162*>(out + (r * Hq + h) * D + d) = __floats2bfloat162_rn(v0, v1);
    }
  }
}

template <int D, bool MASK>
static int launch_prefill(const void* qbuf, const void* kc, const void* vc, const long long* row_kv, const int* seg, int nseg,
                          int max_rows, const void* qkv, int ld, int gated, void* out, int Hq, int Hkv, float scale,
                          cudaStream_t s, const uint32_t* bmask = nullptr, int mw = 0) {
  auto kern = attn_prefill_kernel<D, MASK>;
  constexpr int smem = (PF_BM + 4 * PF_BN) * (D + 8) * 2;
  static bool done = false;
  if (!done) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); done = true; }
  dim3 grid((max_rows + PF_BM - 1) / PF_BM, Hq, nseg);
  kern<<<grid, 128, smem, s>>>((const __nv_bfloat16*)qbuf, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, row_kv, seg,
                               (const __nv_bfloat16*)qkv, ld, gated, (__nv_bfloat16*)out, Hq, Hkv,
                               scale * 1.4426950408889634f, bmask, mw);
  return spark_launch_rc(__func__);
}

// grid R, 256 threads: the row's selected token list -> one bit per 4-token block (the always-visible tail is part of
// the list, so its blocks are set as well; keys past the row's position are cut by the causal test).
__global__ void __launch_bounds__(256)
sel_blockmask_kernel(const int* __restrict__ sel, const int* __restrict__ sel_n, int sel_ld, uint32_t* __restrict__ bmask,
                     int mw) {
  extern __shared__ uint32_t bits[];
  const int r = blockIdx.x;
  for (int i = threadIdx.x; i < mw; i += blockDim.x) bits[i] = 0u;
  __syncthreads();
  const int n = sel_n[r];
  const int* row = sel + static_cast<size_t>(r) * sel_ld;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int b = row[i] >> 2;
    if ((b >> 5) < mw) atomicOr(&bits[b >> 5], 1u << (b & 31));
  }
  __syncthreads();
  for (int i = threadIdx.x; i < mw; i += blockDim.x) bmask[static_cast<size_t>(r) * mw + i] = bits[i];
}

}  // namespace spark

using namespace spark;

// Dense causal attention over bf16 caches for whole segments.  seg: int [nseg][4] = slot, first row, rows, first
// position; max_rows = longest segment.  head_dim 64, 128 or 256.
extern "C" int spark_attn_prefill(const void* qbuf, const void* kc, const void* vc, const long long* row_kv, const int* seg,
                                  int nseg, int max_rows, const void* qkv, int ld, int gated, void* out, int Hq, int Hkv,
                                  int D, float scale, cudaStream_t s) {
  if (nseg <= 0 || max_rows <= 0) return 0;
  if (Hq % Hkv) return -5;
  if (D == 256) return launch_prefill<256, false>(qbuf, kc, vc, row_kv, seg, nseg, max_rows, qkv, ld, gated, out, Hq, Hkv, scale, s);
  if (D == 128) return launch_prefill<128, false>(qbuf, kc, vc, row_kv, seg, nseg, max_rows, qkv, ld, gated, out, Hq, Hkv, scale, s);
  if (D == 64) return launch_prefill<64, false>(qbuf, kc, vc, row_kv, seg, nseg, max_rows, qkv, ld, gated, out, Hq, Hkv, scale, s);
  return -5;
}

// The same tiles for rows with a block-sparse selection (4-token blocks): sel / sel_n are the per-row token lists of the
// selection kernels (R rows, plan order), bmask a scratch of R * mw words with mw >= ceil(max context / 128).
extern "C" int spark_attn_prefill_masked(const void* qbuf, const void* kc, const void* vc, const long long* row_kv,
                                         const int* seg, int nseg, int max_rows, const void* qkv, int ld, int gated, void* out,
                                         int Hq, int Hkv, int D, float scale, const int* sel, const int* sel_n, int sel_ld,
                                         int R, unsigned* bmask, int mw, cudaStream_t s) {
  if (nseg <= 0 || max_rows <= 0 || R <= 0) return 0;
  if (Hq % Hkv || mw <= 0 || mw > 8192 || !sel || !sel_n || !bmask) return -5;
  sel_blockmask_kernel<<<R, 256, mw * 4, s>>>(sel, sel_n, sel_ld, bmask, mw);
  if (D == 256) return launch_prefill<256, true>(qbuf, kc, vc, row_kv, seg, nseg, max_rows, qkv, ld, gated, out, Hq, Hkv, scale, s, bmask, mw);
  if (D == 128) return launch_prefill<128, true>(qbuf, kc, vc, row_kv, seg, nseg, max_rows, qkv, ld, gated, out, Hq, Hkv, scale, s, bmask, mw);
  if (D == 64) return launch_prefill<64, true>(qbuf, kc, vc, row_kv, seg, nseg, max_rows, qkv, ld, gated, out, Hq, Hkv, scale, s, bmask, mw);
  return -5;
}
