// EXL3 grouped GEMM for prefill-size MoE batches: rows in expert order, <= 64 rows per work item.
//   y[rows of the item] = had128( xh @ inner_e ) * svh_e       (xh = had128(x * suh_e) computed by a pre-pass)
// The trellis of an expert is decoded ONCE per item and reused by up to four 16-row MMA tiles, so the expert
// weights cross HBM in their packed form only (0.5 byte per weight) instead of being expanded to fp16 and read
// back by a GEMM (4.5 bytes per weight): with ~20..80 rows per expert the work is bound by the integer decode,
// not by tensor throughput, which is why the warp-level MMA carries it.
// Grid (groups of 4 strips of 128 columns, S, work items) with a cluster of S CTAs along K.  A CTA copies its
// K-slice of the item's rows into shared memory once and walks through its strips; each warp streams one
// 16-column n-tile of the strip (batches of 8 packed tiles in flight, the next strip's first batches are requested
// before the reduction of the current one) and feeds every decoded B fragment to all live row tiles.  The slice partials are
// reduce-scattered through distributed shared memory (CTA s owns 64/S rows), summed in slice order, and the
// owner applies the output Hadamard and scale.  Fixed order => bitwise reproducible.
// Reference: engine-rs/shim/moe_exl3.cuh:521-1233 (gemm_grouped / gux / gu2 kernels, mma.sync m16n8k16).
#include "exl3_common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace spark {

struct Exl3MgemmArgs {
  const __half* xh; int ldx;                    // [P, K] fp16, rows in expert order, input Hadamard applied
  const uint32_t* trellis; const __half* svh;   // [E][K/16][N/16][32], [E][N]
  long long t_stride, svh_stride;
  const int4* tiles; const int* ntile;          // 128-row tiles {row0, row_end, expert, 0} and their count
  void* y; int ldy; int out_f32;                // [P, N]
  int K, N, S;
};

constexpr int MG_STRIPS = 4;     // 128-column strips a CTA walks through with one staged copy of its rows

// MT = 16-row MMA tiles per work item (2: items of <= 32 rows, 4: <= 64 rows; fewer accumulators -> more CTAs per SM)
template <int CB, int MT>
__global__ void __launch_bounds__(256, MT == 2 ? 3 : 2)
exl3_mgemm_kernel(const __grid_constant__ Exl3MgemmArgs a) {
  constexpr int ROWS = 16 * MT, PER_TILE = 128 / ROWS;
  const int tile = blockIdx.z / PER_TILE, part = blockIdx.z % PER_TILE;
  if (tile >= *a.ntile) return;
  const int4 td = a.tiles[tile];
  const int row0 = td.x + part * ROWS;
  const int nrows = min(min(td.x + 128, td.y) - row0, ROWS);
  if (nrows <= 0) return;                                       // uniform over the cluster
  const int e = td.z;
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  cg::cluster_group cluster = cg::this_cluster();
  const int slice = blockIdx.y;
  const int NT = a.N >> 4;
  const int Ks = a.K / a.S, kts = Ks >> 4;
  const int ldh = Ks + 8;
  __half* xs = reinterpret_cast<__half*>(smem_dyn);                               // [ROWS][Ks + 8]
  float* red0 = reinterpret_cast<float*>(smem_dyn + ROWS * ldh * 2);              // 2 x [S][ROWS/S][128]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int mts = (nrows + 15) >> 4;
  const int strip0 = blockIdx.x * MG_STRIPS, nstrips = min(MG_STRIPS, (a.N >> 7) - strip0);
  // every CTA of the cluster must be running before its shared memory is written remotely: arrive now, wait
  // right before the first remote store
  if (a.S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  const size_t tstep = static_cast<size_t>(NT) * 32;
  const uint32_t* tw = a.trellis + e * a.t_stride + (static_cast<size_t>(slice) * kts * NT + strip0 * 8 + warp) * 32 + lane;
  // packed tiles arrive in batches of 8 per warp; batches are numbered across the strips of this CTA and the one
  // two ahead of the batch being decoded is always in flight
  const int nb = kts >> 3, nbatch = nb * nstrips;
  uint32_t cur[8], nxt[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) cur[u] = __ldg(tw + u * tstep);
  if (nbatch > 1) {
    const uint32_t* t1 = nb > 1 ? tw + 8 * tstep : tw + 8 * 32;
#pragma unroll
    for (int u = 0; u < 8; ++u) nxt[u] = __ldg(t1 + u * tstep);
  }
  // ---- stage the K-slice of the item's rows once (zero rows up to the next multiple of 16)
  {
    const int vec = Ks >> 3;                                   // 16-byte vectors per row
    const __half* src = a.xh + static_cast<size_t>(row0) * a.ldx + slice * Ks;
    for (int i = threadIdx.x; i < mts * 16 * vec; i += 256) {
      const int r = i / vec, v = i - r * vec;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (r < nrows) val = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * a.ldx + v * 8);
      *reinterpret_cast<uint4*>(xs + r * ldh + v * 8) = val;
    }
  }
  __syncthreads();
  const int rp = ROWS / a.S;
  const __half* xa = xs + g * ldh + 2 * t;

#pragma unroll 1
  for (int si = 0; si < nstrips; ++si) {
    const int strip = strip0 + si;
    float d[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) { d[m][0][j] = 0.f; d[m][1][j] = 0.f; }
#pragma unroll 1
    for (int kb = 0; kb < kts; kb += 8) {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t prev = __shfl_sync(0xffffffffu, cur[u], (lane + 31) & 31);
        uint32_t w[4];
        exl3_decode8_b4<CB>(cur[u], prev, w);
        const __half* xk = xa + (kb + u) * 16;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m < mts) {
            uint32_t af[4];
            af[0] = *reinterpret_cast<const uint32_t*>(xk + (m * 16) * ldh);
            af[1] = *reinterpret_cast<const uint32_t*>(xk + (m * 16 + 8) * ldh);
            af[2] = *reinterpret_cast<const uint32_t*>(xk + (m * 16) * ldh + 8);
            af[3] = *reinterpret_cast<const uint32_t*>(xk + (m * 16 + 8) * ldh + 8);
            mma_f16_16816(d[m][0], af, w[0], w[1]);
            mma_f16_16816(d[m][1], af, w[2], w[3]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) cur[u] = nxt[u];
      const int gb = si * nb + (kb >> 3) + 2;                  // batch to request now
      if (gb < nbatch) {
        const int st = gb / nb, bi = gb - st * nb;
        const uint32_t* tn = tw + st * 8 * 32 + static_cast<size_t>(bi) * 8 * tstep;
#pragma unroll
        for (int u = 0; u < 8; ++u) nxt[u] = __ldg(tn + u * tstep);
      }
    }
    // ---- reduce-scatter of the slice partials inside the cluster: CTA o owns rows [o*rp, (o+1)*rp)
    float* red = red0 + (si & 1) * ROWS * 128;
    if (a.S > 1 && si == 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < mts) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = m * 16 + g + hh * 8;
          if (r < nrows) {
            const int owner = r / rp;
            float* dst = (a.S > 1 ? cluster.map_shared_rank(red, owner) : red) +
                         (static_cast<size_t>(slice) * rp + (r - owner * rp)) * 128 + warp * 16 + 2 * t;
            *reinterpret_cast<float2*>(dst) = make_float2(d[m][0][2 * hh], d[m][0][2 * hh + 1]);
            *reinterpret_cast<float2*>(dst + 8) = make_float2(d[m][1][2 * hh], d[m][1][2 * hh + 1]);
          }
        }
      }
    }
    if (a.S > 1) cluster.sync(); else __syncthreads();
    const __half* svh = a.svh + e * a.svh_stride + strip * 128;
    const uint2 sraw = *reinterpret_cast<const uint2*>(svh + lane * 4);
    const __half2* sp = reinterpret_cast<const __half2*>(&sraw);
    const float2 s0 = __half22float2(sp[0]), s1 = __half22float2(sp[1]);
    for (int rl = warp; rl < rp; rl += 8) {
      const int r = slice * rp + rl;
      if (r >= nrows) break;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < a.S; ++s) {
        const float4 p = *reinterpret_cast<const float4*>(red + (static_cast<size_t>(s) * rp + rl) * 128 + lane * 4);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
      }
      fwht128_warp(v, lane);
      v[0] *= INV_SQRT_128 * s0.x; v[1] *= INV_SQRT_128 * s0.y; v[2] *= INV_SQRT_128 * s1.x; v[3] *= INV_SQRT_128 * s1.y;
      const size_t o = static_cast<size_t>(row0 + r) * a.ldy + strip * 128 + lane * 4;
      if (a.out_f32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + o) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
        __nv_bfloat162 b0 = __floats2bfloat162_rn(v[0], v[1]), b1 = __floats2bfloat162_rn(v[2], v[3]);
        uint2 ov; ov.x = *reinterpret_cast<uint32_t*>(&b0); ov.y = *reinterpret_cast<uint32_t*>(&b1);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.y) + o) = ov;
      }
    }
  }
}

}  // namespace spark

using namespace spark;

// xh fp16 [P, K] (input Hadamard applied), rows in expert order; tiles = the 128-row tile list of the MoE sort
// (max_tiles entries allocated, *ntile valid).  K, N multiples of 128; S in {1,2,4,8} with (K/128) % S == 0.
template <int CB, int MT>
static int launch_mgemm(const Exl3MgemmArgs& a, int max_tiles, cudaStream_t s) {
  constexpr int ROWS = 16 * MT;
  const int smem = ROWS * (a.K / a.S + 8) * 2 + 2 * ROWS * 128 * 4;
  if (smem > 200 * 1024) return -6;
  void (*kern)(Exl3MgemmArgs) = exl3_mgemm_kernel<CB, MT>;
  static bool done = false;
  if (!done) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); done = true; }
  cudaLaunchConfig_t cfg = {};
  const int strips = a.N / 128;
  cfg.gridDim = dim3((strips + MG_STRIPS - 1) / MG_STRIPS, a.S, (128 / ROWS) * max_tiles);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = a.S; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, a) == cudaSuccess ? 0 : -4;
}

// xh fp16 [P, K] (input Hadamard applied), rows in expert order; tiles = the 128-row tile list of the MoE sort
// (max_tiles entries allocated, *ntile valid).  K, N multiples of 128; S in {1,2,4,8} with (K/128) % S == 0.
// rows_per_item: 32 or 64 (work item = that many rows of one expert; 32 suits ~<= 24 rows per expert on average).
extern "C" int spark_exl3_mgemm(const void* xh, int ldx, const void* trellis, const void* svh, long long t_stride_words,
                                long long svh_stride, const void* tiles, const int* ntile, int max_tiles, void* y, int ldy,
                                int out_f32, int K, int N, int S, int codebook, int rows_per_item, cudaStream_t s) {
  if (max_tiles <= 0) return 0;
  if ((K & 127) || (N & 127) || !(S == 1 || S == 2 || S == 4 || S == 8) || ((K >> 7) % S) || (ldx & 7) || (ldy & 3)) return -5;
  if (rows_per_item != 32 && rows_per_item != 64) return -5;
  Exl3MgemmArgs a;
  a.xh = (const __half*)xh; a.ldx = ldx; a.trellis = (const uint32_t*)trellis; a.svh = (const __half*)svh;
  a.t_stride = t_stride_words; a.svh_stride = svh_stride; a.tiles = (const int4*)tiles; a.ntile = ntile;
  a.y = y; a.ldy = ldy; a.out_f32 = out_f32; a.K = K; a.N = N; a.S = S;
  if (codebook == 0) return rows_per_item == 32 ? launch_mgemm<0, 2>(a, max_tiles, s) : launch_mgemm<0, 4>(a, max_tiles, s);
  return rows_per_item == 32 ? launch_mgemm<1, 2>(a, max_tiles, s) : launch_mgemm<1, 4>(a, max_tiles, s);
}
