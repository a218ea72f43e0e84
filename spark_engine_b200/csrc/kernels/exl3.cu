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

// E stacked tensors (experts) in one launch: trellis [E][K/16][N/16][32 words] -> Wt [E][N][K].
extern "C" int spark_exl3_reconstruct(const void* trellis, void* Wt, int K, int N, int codebook, cudaStream_t s, int E) {
  const long long tiles = (long long)(K >> 4) * (N >> 4) * E;
  const unsigned blocks = (unsigned)((tiles * 32 + 255) / 256);
  if (codebook == 0) exl3_reconstruct_kernel<0><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E);
  else exl3_reconstruct_kernel<1><<<blocks, 256, 0, s>>>((const uint32_t*)trellis, (__half*)Wt, K, N, E);
  return spark_launch_rc(__func__);
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
  return spark_launch_rc(__func__);
}
