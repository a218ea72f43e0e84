// EXL3 helpers for the GEMM (prefill) path:
//   exl3_reconstruct: trellis -> inner codebook weights as fp16 [N,K] (K-major B operand of the tcgen05 GEMM),
//                     all experts of a stacked tensor in one launch;
//   exl3_had_rows   : y = had128(x * scale) (input side, fp16 out) or had128(x) * scale (output side, bf16 out),
//                     with an optional per-row expert index selecting the scale vector.
// Format contract: engine-rs/shim/qwen_exl3.cuh:17-117,634-661; reference/qwen38/exl3.py:66-110.
#include "exl3_common.cuh"

namespace spark {

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

// Any bit width (2..8 bits/weight: checkpoints mix 3 to 6 bits per tensor, heads often 6): a tile is 8 * bits words;
// the state of stream position t is the 16 bits that start at bit ((t + 1) * bits - 16) of the tail-biting ring, read
// MSB-first over little-endian 32-bit words.  Lane l still decodes positions 8l .. 8l+7, so the fragment assembly
// and the store pattern are those of the 4-bit kernel; only the window extraction reads its two words per state
// from memory (L1) instead of from the lane's own register.
template <int CB>
__global__ void exl3_reconstruct_bits_kernel(const uint32_t* __restrict__ trellis, __half* __restrict__ Wt, int K, int N,
                                             int E, int bits) {
  const int KT = K >> 4, NT = N >> 4;
  const long long per = static_cast<long long>(KT) * NT;
  long long tile = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (tile >= per * E) return;
  const int lane = threadIdx.x & 31;
  const int n_words = 8 * bits, n_bits = 256 * bits;
  const uint32_t* tw = trellis + tile * n_words;
  uint32_t st[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int first = (8 * lane + j + 1) * bits - 16;
    if (first < 0) first += n_bits;
    const int wi = first >> 5, off = first & 31;
    const uint32_t hi = __ldg(tw + wi), lo = __ldg(tw + (wi + 1 == n_words ? 0 : wi + 1));
    st[j] = __funnelshift_l(lo, hi, off) >> 16;
  }
  const long long e = tile / per;
  tile -= e * per;
  Wt += e * static_cast<long long>(N) * K;
  const int kt = static_cast<int>(tile / NT), nt = static_cast<int>(tile % NT);
  uint32_t w[4];
  w[0] = exl3_pair<CB>(st[0], st[1]); w[1] = exl3_pair<CB>(st[2], st[3]);
  w[2] = exl3_pair<CB>(st[4], st[5]); w[3] = exl3_pair<CB>(st[6], st[7]);
  const int r0 = (lane & 3) * 2, c0 = lane >> 2;
  uint32_t* dst0 = reinterpret_cast<uint32_t*>(Wt + static_cast<size_t>(nt * 16 + c0) * K + kt * 16);
  uint32_t* dst1 = reinterpret_cast<uint32_t*>(Wt + static_cast<size_t>(nt * 16 + c0 + 8) * K + kt * 16);
  dst0[r0 >> 1] = w[0]; dst0[(r0 + 8) >> 1] = w[1];
  dst1[r0 >> 1] = w[2]; dst1[(r0 + 8) >> 1] = w[3];
}

// y[r, :] = had128(x[r, :] * scale[:]) (pre) or had128(x[r, :]) * scale[:] (post); 128-blocks along the row.
// One warp per 128-block: a lane keeps 4 consecutive elements (one 8- or 16-byte load), the strides 1 and 2 of the
// butterfly run in registers and the strides 4..64 through five shuffles -- the same additions in the same order as a
// shared-memory butterfly, without its 14 barriers per block (this pass was 0.76 TB/s as one block per CTA).
template <typename T> __device__ __forceinline__ void ld4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void ld4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void ld4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
}
__device__ __forceinline__ void st4(__half* p, const float (&v)[4]) {
  const __half2 a = __floats2half2_rn(v[0], v[1]), c = __floats2half2_rn(v[2], v[3]);
  uint2 o; o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&c);
  *reinterpret_cast<uint2*>(p) = o;
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), c = __floats2bfloat162_rn(v[2], v[3]);
  uint2 o; o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&c);
  *reinterpret_cast<uint2*>(p) = o;
}

template <typename TI, typename TOUT>
__global__ void __launch_bounds__(256)
exl3_had_rows_kernel(const TI* __restrict__ x, int ldx, const __half* __restrict__ scale, TOUT* __restrict__ y, int ldy,
                     int post, const int* __restrict__ row_expert, long long expert_stride, int nblk, long long total) {
  const int lane = threadIdx.x & 31;
  const long long w = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);      // (row, 128-block) of this warp
  if (w >= total) return;
  const int r = static_cast<int>(w / nblk), blk = static_cast<int>(w - static_cast<long long>(r) * nblk);
  const int c0 = blk * 128 + lane * 4;
  float v[4];
  ld4(x + static_cast<size_t>(r) * ldx + c0, v);
  const __half* srow = scale + (row_expert ? row_expert[r] * expert_stride : 0);
  const uint2 sraw = *reinterpret_cast<const uint2*>(srow + c0);
  const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sraw.x));
  const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sraw.y));
  const float sc[4] = {s01.x, s01.y, s23.x, s23.y};
  if (!post) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= sc[i];
  }
  // strides 1, 2: inside the lane (element i pairs with i ^ stride; the upper one takes lower - upper)
  {
    const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
    v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
  }
  // strides 4 .. 64: lane ^ 1 .. lane ^ 16
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? other - v[i] : v[i] + other;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] *= 0.08838834764831845f;
    if (post) v[i] *= sc[i];
  }
  st4(y + static_cast<size_t>(r) * ldy + c0, v);
}

}  // namespace spark

using namespace spark;

// E stacked tensors (experts) in one launch: trellis [E][K/16][N/16][32 words] -> Wt [E][N][K].
extern "C" int spark_exl3_reconstruct(const void* trellis, void* Wt, int K, int N, int codebook, cudaStream_t s, int E) {
  const long long tiles = (long long)(K >> 4) * (N >> 4) * E;
  const unsigned blocks = (unsigned)((tiles * 32 + 255) / 256);
  if (codebook == 0) exl3_reconstruct_kernel<0><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E);
  else exl3_reconstruct_kernel<1><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E);
  return spark_launch_rc(__func__);
}

// The same for any bit width 2..8 (trellis [E][K/16][N/16][8 * bits words]).
extern "C" int spark_exl3_reconstruct_bits(const void* trellis, void* Wt, int K, int N, int codebook, cudaStream_t s, int E,
                                           int bits) {
  if (bits < 2 || bits > 8 || (K & 15) || (N & 15) || E < 1) return -5;
  const long long tiles = (long long)(K >> 4) * (N >> 4) * E;
  const unsigned blocks = (unsigned)((tiles * 32 + 255) / 256);
  if (codebook == 0) exl3_reconstruct_bits_kernel<0><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E, bits);
  else exl3_reconstruct_bits_kernel<1><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E, bits);
  return spark_launch_rc(__func__);
}

// pre (post = 0): x bf16 -> y fp16 = had128(x * scale);  post = 1: x fp32 -> y bf16 = had128(x) * scale.
// row_expert (optional): per-row expert id selecting scale + row_expert[r] * expert_stride.
extern "C" int spark_exl3_had_rows(const void* x, int ldx, const void* scale, void* y, int ldy, int R, int C, int post,
                                   const int* row_expert, cudaStream_t s, long long expert_stride) {
  if (R <= 0) return 0;
  if (C & 127) return -5;
  if ((ldx & 3) || (ldy & 3)) return -5;               // 8- / 16-byte vector accesses along the rows
  const int nblk = C / 128;
  const long long total = static_cast<long long>(R) * nblk;
  const unsigned grid = static_cast<unsigned>((total + 7) / 8);
  if (!post) exl3_had_rows_kernel<__nv_bfloat16, __half><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, ldx, (const __half*)scale, (__half*)y, ldy, 0, row_expert, expert_stride, nblk, total);
  else exl3_had_rows_kernel<float, __nv_bfloat16><<<grid, 256, 0, s>>>((const float*)x, ldx, (const __half*)scale, (__nv_bfloat16*)y, ldy, 1, row_expert, expert_stride, nblk, total);
  return spark_launch_rc(__func__);
}
