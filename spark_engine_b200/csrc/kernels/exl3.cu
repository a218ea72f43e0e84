// EXL3 (trellis-coded, 4 bits/weight, `mul1` or `mcg` codebook) kernels.
//
//   y = had128( had128(x * suh) @ inner ) * svh,  inner[K,N] = codebook(trellis states)
//
// exl3_gemv  (<= 16 rows, decode / verify / MoE pairs): one launch does the input Hadamard, the
//   trellis decode, the product and the output Hadamard.  Grid (N/128, S, items): a CTA owns a
//   128-column strip and one K-slice; warp w streams the 128-byte tiles of its 16-column n-tile
//   (one coalesced word per lane, previous lane's word by shuffle), decodes 8 weights per lane
//   straight into m16n8k16 B fragments (the trellis stream order IS the fragment order) and feeds
//   mma.sync with the <=16 activation rows as A.  M <= 16 is decode-ALU / bandwidth bound, so the
//   warp-level MMA is used here; GEMM-shaped EXL3 work goes to tcgen05 through exl3_reconstruct.
//   K-slices are summed in slice order by the last-arriving CTA of a strip (integer counter only),
//   so results are deterministic and independent of the number of rows in flight.
// exl3_reconstruct: inner -> fp16 [N,K] (K-major B operand of the tcgen05 GEMM).
// exl3_had_rows   : y = had128(x * scale) row-wise (prologue / epilogue of the GEMM path).
//
// Format contract: engine-rs/shim/qwen_exl3.cuh:17-117 (decode), :427-626 (gemv/finish kernels);
// reference/qwen38/exl3.py:66-110.
#include "../common/ptx.cuh"

namespace spark {

constexpr uint32_t EXL3_MUL1 = 0x83DCD12Du;
constexpr uint32_t EXL3_MCG = 0xCBAC1FEDu;

// two trellis states -> two fp16 weights packed in a half2
template <int CB>
__device__ __forceinline__ uint32_t exl3_pair(uint32_t s0, uint32_t s1) {
  if (CB == 0) {   // mul1: fp16(1024 + bytesum) * k_inv + k_bias, fused (one rounding)
    const uint32_t a = __dp4a(s0 * EXL3_MUL1, 0x01010101u, 0x6400u);     // 0x6400 | sum  == fp16(1024+sum)
    const uint32_t b = __dp4a(s1 * EXL3_MUL1, 0x01010101u, 0x6400u);
    const uint32_t packed = a | (b << 16);
    const __half2 inv = __halves2half2(__ushort_as_half(0x1eee), __ushort_as_half(0x1eee));
    const __half2 bias = __halves2half2(__ushort_as_half(0xc931), __ushort_as_half(0xc931));
    const __half2 v = __hfma2(*reinterpret_cast<const __half2*>(&packed), inv, bias);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {         // mcg: fp16(lo16) + fp16(hi16) of the masked product
    const uint32_t y0 = ((s0 * EXL3_MCG) & 0x8FFF8FFFu) ^ 0x3B603B60u;
    const uint32_t y1 = ((s1 * EXL3_MCG) & 0x8FFF8FFFu) ^ 0x3B603B60u;
    const uint32_t lo = (y0 & 0xFFFFu) | (y1 << 16);
    const uint32_t hi = (y0 >> 16) | (y1 & 0xFFFF0000u);
    const __half2 v = __hadd2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&hi));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// 4-bit tile: lane l holds word l of the tile (32 words); decodes stream positions 8l..8l+7.
// State j = 16 bits of the (prev:cur) window ending 4(j+1) bits into `cur` (MSB-first stream).
template <int CB>
__device__ __forceinline__ void exl3_decode8_b4(uint32_t cur, uint32_t prev, uint32_t (&w)[4]) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint32_t s0 = __funnelshift_r(cur, prev, 28 - 8 * p) & 0xFFFFu;
    const uint32_t s1 = __funnelshift_r(cur, prev, 24 - 8 * p) & 0xFFFFu;
    w[p] = exl3_pair<CB>(s0, s1);
  }
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// in-place 128-point Walsh-Hadamard / sqrt(128) over rows of `buf` ([rows][ld] floats), columns
// [c0, c0+128); all threads of the CTA cooperate (blockDim.x threads).
__device__ __forceinline__ void fwht128_rows(float* buf, int ld, int rows, int nblk) {
  // element index space: rows * nblk * 64 butterflies per stage
  const int total = rows * nblk * 64;
  for (int st = 1; st < 128; st <<= 1) {
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int r = i / (nblk * 64), rem = i - r * (nblk * 64);
      const int b = rem >> 6, j = rem & 63;
      const int lo = ((j & ~(st - 1)) << 1) | (j & (st - 1));
      float* p = buf + r * ld + b * 128 + lo;
      const float x = p[0], y = p[st];
      p[0] = x + y; p[st] = x - y;
    }
    __syncthreads();
  }
}

struct Exl3GemvArgs {
  const __nv_bfloat16* x; int ldx;             // activations [rows, K] (or [rows, 2K] when act == 1)
  const uint32_t* trellis;                      // [E][K/16][N/16][32] words (4 bpw)
  const __half* suh; const __half* svh;         // [E][K], [E][N]
  long long t_stride, suh_stride, svh_stride;   // per expert, in elements
  void* y; int ldy; int out_f32;                // [items*R, N]
  float* partial;                               // scratch [items][S][16][N]
  int* counters;                                // scratch [items][N/128], zero between launches
  const int* pair_expert; const int* pair_row;
  int R, K, N, S, act; float limit;
};

template <int CB>
__global__ void __launch_bounds__(256)
exl3_gemv_kernel(Exl3GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem_exl3[];
  const int strip = blockIdx.x, slice = blockIdx.y, item = blockIdx.z;
  const int KT = a.K >> 4, NT = a.N >> 4;
  const int kts = KT / a.S;                    // k-tiles per slice (multiple of 8)
  const int Ks = kts << 4;
  const int k_begin = slice * Ks;
  const int e = a.pair_expert ? a.pair_expert[item] : 0;
  const int xr0 = a.pair_row ? a.pair_row[item] : item * a.R;
  const int R = a.R;
  float* xf = reinterpret_cast<float*>(smem_exl3);                       // [R][Ks] fp32 for the FWHT
  const int ldh = Ks + 8;
  __half* xh = reinterpret_cast<__half*>(smem_exl3 + static_cast<size_t>(R) * Ks * 4);   // [16][ldh]
  __shared__ int s_last;

  // ---- prologue: xh = had128(x * suh) for this K-slice
  const __half* suh = a.suh + e * a.suh_stride;
  for (int i = threadIdx.x; i < R * Ks; i += blockDim.x) {
    const int r = i / Ks, k = i - r * Ks;
    const __nv_bfloat16* xr = a.x + static_cast<size_t>(xr0 + r) * a.ldx;
    float v;
    if (a.act == 1) {
      float g = __bfloat162float(xr[k_begin + k]), u = __bfloat162float(xr[a.K + k_begin + k]);
      if (a.limit > 0.f) { g = fminf(g, a.limit); u = fminf(fmaxf(u, -a.limit), a.limit); }
      v = g / (1.f + __expf(-g)) * u;
    } else {
      v = __bfloat162float(xr[k_begin + k]);
    }
    xf[i] = v * __half2float(suh[k_begin + k]);
  }
  __syncthreads();
  fwht128_rows(xf, Ks, R, Ks >> 7);
  for (int i = threadIdx.x; i < 16 * Ks; i += blockDim.x) {
    const int r = i / Ks, k = i - r * Ks;
    xh[r * ldh + k] = __float2half(r < R ? xf[r * Ks + k] * 0.08838834764831845f : 0.f);
  }
  __syncthreads();

  // ---- main loop: warp w owns n-tile strip*8 + w
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int nt = strip * 8 + warp;
  const uint32_t* tw = a.trellis + e * a.t_stride + (static_cast<size_t>(slice) * kts * NT + nt) * 32 + lane;
  float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
  constexpr int UN = 4;
  for (int kt = 0; kt < kts; kt += UN) {
    uint32_t cur[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) cur[u] = (kt + u < kts) ? __ldg(tw + static_cast<size_t>(kt + u) * NT * 32) : 0u;
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      if (kt + u < kts) {
        const uint32_t prev = __shfl_sync(0xffffffffu, cur[u], (lane + 31) & 31);
        uint32_t w[4];
        exl3_decode8_b4<CB>(cur[u], prev, w);
        uint32_t af[4];
        const __half* xa = xh + (kt + u) * 16 + 2 * t;
        af[0] = *reinterpret_cast<const uint32_t*>(xa + g * ldh);
        af[1] = *reinterpret_cast<const uint32_t*>(xa + (g + 8) * ldh);
        af[2] = *reinterpret_cast<const uint32_t*>(xa + g * ldh + 8);
        af[3] = *reinterpret_cast<const uint32_t*>(xa + (g + 8) * ldh + 8);
        mma_f16_16816(d0, af, w[0], w[1]);       // columns 0..7 of the n-tile
        mma_f16_16816(d1, af, w[2], w[3]);       // columns 8..15
      }
    }
  }
  __syncthreads();                               // xf is reused as the strip buffer [16][128]
  float* sb = xf;
  {
    const int c = warp * 16 + 2 * t;
    sb[g * 128 + c] = d0[0]; sb[g * 128 + c + 1] = d0[1];
    sb[(g + 8) * 128 + c] = d0[2]; sb[(g + 8) * 128 + c + 1] = d0[3];
    sb[g * 128 + c + 8] = d1[0]; sb[g * 128 + c + 9] = d1[1];
    sb[(g + 8) * 128 + c + 8] = d1[2]; sb[(g + 8) * 128 + c + 9] = d1[3];
  }
  __syncthreads();
  if (a.S > 1) {
    float* part = a.partial + ((static_cast<size_t>(item) * a.S + slice) * 16) * a.N + strip * 128;
    for (int i = threadIdx.x; i < R * 128; i += blockDim.x) part[static_cast<size_t>(i >> 7) * a.N + (i & 127)] = sb[i];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int old = atomicAdd(&a.counters[item * gridDim.x + strip], 1);
      s_last = (old == a.S - 1);
      if (s_last) a.counters[item * gridDim.x + strip] = 0;       // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < R * 128; i += blockDim.x) {
      float acc = 0.f;
      for (int s = 0; s < a.S; ++s)                 // fixed slice order
        acc += __ldcg(a.partial + ((static_cast<size_t>(item) * a.S + s) * 16 + (i >> 7)) * a.N + strip * 128 + (i & 127));
      sb[i] = acc;
    }
    __syncthreads();
  }
  // ---- epilogue: y = had128(acc) * svh
  fwht128_rows(sb, 128, R, 1);
  const __half* svh = a.svh + e * a.svh_stride + strip * 128;
  for (int i = threadIdx.x; i < R * 128; i += blockDim.x) {
    const int r = i >> 7, c = i & 127;
    const float v = sb[i] * 0.08838834764831845f * __half2float(svh[c]);
    const size_t o = static_cast<size_t>(item * R + r) * a.ldy + strip * 128 + c;
    if (a.out_f32) reinterpret_cast<float*>(a.y)[o] = v;
    else reinterpret_cast<__nv_bfloat16*>(a.y)[o] = __float2bfloat16(v);
  }
}

// inner -> fp16 Wt[N, K] (K contiguous).  One warp per tile.
template <int CB>
__global__ void exl3_reconstruct_kernel(const uint32_t* __restrict__ trellis, __half* __restrict__ Wt, int K, int N,
                                        int E) {
  const int KT = K >> 4, NT = N >> 4;
  const long long per = static_cast<long long>(KT) * NT;
  long long tile = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (tile >= per * E) return;
  const int lane = threadIdx.x & 31;
  const uint32_t cur = __ldg(trellis + tile * 32 + lane);
  const long long e = tile / per;
  tile -= e * per;
  Wt += e * static_cast<long long>(N) * K;
  const int kt = static_cast<int>(tile / NT), nt = static_cast<int>(tile % NT);
  const uint32_t prev = __shfl_sync(0xffffffffu, cur, (lane + 31) & 31);
  uint32_t w[4];
  exl3_decode8_b4<CB>(cur, prev, w);
  const int r0 = (lane & 3) * 2, c0 = lane >> 2;
  uint32_t* dst0 = reinterpret_cast<uint32_t*>(Wt + static_cast<size_t>(nt * 16 + c0) * K + kt * 16);
  uint32_t* dst1 = reinterpret_cast<uint32_t*>(Wt + static_cast<size_t>(nt * 16 + c0 + 8) * K + kt * 16);
  dst0[r0 >> 1] = w[0]; dst0[(r0 + 8) >> 1] = w[1];
  dst1[r0 >> 1] = w[2]; dst1[(r0 + 8) >> 1] = w[3];
}

// y[r, :] = had128(x[r, :] * scale[:]) (pre) or had128(x[r, :]) * scale[:] (post); 128-blocks along the row.
template <typename TI, typename TOUT>
__global__ void __launch_bounds__(128)
exl3_had_rows_kernel(const TI* __restrict__ x, int ldx, const __half* __restrict__ scale, TOUT* __restrict__ y, int ldy,
                     int post, const int* __restrict__ row_expert, long long expert_stride) {
  __shared__ float b[128];
  const int r = blockIdx.x, blk = blockIdx.y, t = threadIdx.x;
  float v = static_cast<float>(x[static_cast<size_t>(r) * ldx + blk * 128 + t]);
  const __half* srow = scale + (row_expert ? row_expert[r] * expert_stride : 0);
  const float sc = __half2float(srow[blk * 128 + t]);
  if (!post) v *= sc;
  b[t] = v;
  __syncthreads();
  for (int st = 1; st < 128; st <<= 1) {
    const float me = b[t], other = b[t ^ st];
    __syncthreads();
    b[t] = (t & st) ? other - me : me + other;
    __syncthreads();
  }
  v = b[t] * 0.08838834764831845f;
  if (post) v *= sc;
  y[static_cast<size_t>(r) * ldy + blk * 128 + t] = static_cast<TOUT>(v);
}

}  // namespace spark

using namespace spark;

extern "C" long long spark_exl3_gemv_scratch_floats(int items, int S, int N) { return (long long)items * S * 16 * N; }

// rows_per_item <= 16; K, N multiples of 128; (K/128) % S == 0.  codebook: 0 mul1, 1 mcg.
extern "C" int spark_exl3_gemv(const void* x, int ldx, const void* trellis, const void* suh, const void* svh,
                               long long t_stride_words, long long suh_stride, long long svh_stride, void* y, int ldy,
                               int out_f32, float* partial, int* counters, const int* pair_expert, const int* pair_row,
                               int items, int rows_per_item, int K, int N, int S, int act, float limit, int codebook,
                               cudaStream_t s) {
  if (items <= 0 || rows_per_item <= 0) return 0;
  if (rows_per_item > 16 || (K & 127) || (N & 127) || S < 1 || ((K >> 7) % S)) return -5;
  Exl3GemvArgs a;
  a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.trellis = (const uint32_t*)trellis;
  a.suh = (const __half*)suh; a.svh = (const __half*)svh;
  a.t_stride = t_stride_words; a.suh_stride = suh_stride; a.svh_stride = svh_stride;
  a.y = y; a.ldy = ldy; a.out_f32 = out_f32; a.partial = partial; a.counters = counters;
  a.pair_expert = pair_expert; a.pair_row = pair_row;
  a.R = rows_per_item; a.K = K; a.N = N; a.S = S; a.act = act; a.limit = limit;
  const int Ks = K / S;
  size_t smem = static_cast<size_t>(rows_per_item) * Ks * 4 + 16 * static_cast<size_t>(Ks + 8) * 2;
  if (smem < 16 * 128 * 4) smem = 16 * 128 * 4;
  if (smem > 200 * 1024) return -6;
  dim3 grid(N / 128, S, items);
  if (codebook == 0) {
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(exl3_gemv_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); done = true; }
    exl3_gemv_kernel<0><<<grid, 256, smem, s>>>(a);
  } else {
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(exl3_gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); done = true; }
    exl3_gemv_kernel<1><<<grid, 256, smem, s>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// E stacked tensors (experts) in one launch: trellis [E][K/16][N/16][32 words] -> Wt [E][N][K].
extern "C" int spark_exl3_reconstruct(const void* trellis, void* Wt, int K, int N, int codebook, cudaStream_t s, int E) {
  const long long tiles = (long long)(K >> 4) * (N >> 4) * E;
  const unsigned blocks = (unsigned)((tiles * 32 + 255) / 256);
  if (codebook == 0) exl3_reconstruct_kernel<0><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E);
  else exl3_reconstruct_kernel<1><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// pre (post = 0): x bf16 -> y fp16 = had128(x * scale);  post = 1: x fp32 -> y bf16 = had128(x) * scale.
// row_expert (optional): per-row expert id selecting scale + row_expert[r] * expert_stride.
extern "C" int spark_exl3_had_rows(const void* x, int ldx, const void* scale, void* y, int ldy, int R, int C, int post,
                                   const int* row_expert, cudaStream_t s, long long expert_stride) {
  if (R <= 0) return 0;
  if (C & 127) return -5;
  dim3 grid(R, C / 128);
  if (!post) exl3_had_rows_kernel<__nv_bfloat16, __half><<<grid, 128, 0, s>>>((const __nv_bfloat16*)x, ldx, (const __half*)scale, (__half*)y, ldy, 0, row_expert, expert_stride);
  else exl3_had_rows_kernel<float, __nv_bfloat16><<<grid, 128, 0, s>>>((const float*)x, ldx, (const __half*)scale, (__nv_bfloat16*)y, ldy, 1, row_expert, expert_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
