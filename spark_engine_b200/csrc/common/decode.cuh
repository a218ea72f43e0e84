// Building blocks shared by the decode-round kernels (<= 16 rows per launch).
//
// Deferred RMSNorm.  A decode round never materialises the normalised hidden rows.  The kernel that
// finishes a residual update (output projection, MoE combine, fused all-reduce) adds its result into the
// fp32 residual stream and leaves, per 128-column strip and row, the partial sum of squares of the new
// residual (`ResOut`).  Every consumer (the next projection GEMV, the router, the expert gate/up GEMV,
// lm_head) rebuilds rstd from those partials in a fixed order and normalises the rows while it stages
// them (`NormIn`).  No norm launch, no serial tail, and the result of a row does not depend on the other
// rows of the batch.  The reference fuses the same pair the other way round (norm folded into the
// producing kernel's finisher CTA: engine-rs/shim/qwen_exl3.cuh:459 gemv_fused_kernel, mhc.cu:282).
//
// Programmatic dependent launch.  Decode kernels are launched with the programmatic-stream-serialisation
// attribute: a kernel's CTAs may start while its predecessor drains, issue the loads that depend on
// nothing but weights, and then `pdl_wait()` (griddepcontrol.wait: predecessor complete, its writes
// visible).  Every kernel calls `pdl_trigger()` only AFTER its own wait, so "my successor runs" implies
// "my predecessor's predecessor is complete" and data produced two launches back may be read before the
// wait.  Reference: engine-rs/shim/pdl.cuh:20-41, ds41_ops.cu:593-685.
#pragma once
#include "ptx.cuh"

namespace spark {

struct NormIn {
  const float* res;      // [rows, H] fp32 residual stream (nullptr: the kernel reads its plain bf16 input)
  const float* ssq;      // [nparts][ssq_ld] partial sums of squares per row
  const float* w;        // [H] norm weights
  int nparts, ssq_ld, H;
  float eps;
  int one_plus;          // Gemma-style (1 + w)
};

struct ResOut {
  float* res;            // [rows, H] fp32 residual stream (nullptr: the kernel writes its plain output)
  float* ssq;            // [H/128][ssq_ld]: ssq[strip][row] = sum over the strip's columns of res'^2
  int ssq_ld;
};

// rstd of one row, rebuilt by a whole warp from the strip partials (same code, same order everywhere).
__device__ __forceinline__ float norm_rstd(const NormIn& n, int row, int lane) {
  float s = 0.f;
  for (int p = lane; p < n.nparts; p += 32) s += __ldcg(n.ssq + static_cast<size_t>(p) * n.ssq_ld + row);
  s = warp_sum(s);
  return rsqrtf(s / static_cast<float>(n.H) + n.eps);
}

// four consecutive normalised elements of a row, rounded to bf16 like a materialised norm output would be
__device__ __forceinline__ void norm_apply4(const NormIn& n, const float4& x, const float4& g, float rstd, float (&v)[4]) {
  const float o = n.one_plus ? 1.f : 0.f;
  v[0] = __bfloat162float(__float2bfloat16(x.x * rstd * (g.x + o)));
  v[1] = __bfloat162float(__float2bfloat16(x.y * rstd * (g.y + o)));
  v[2] = __bfloat162float(__float2bfloat16(x.z * rstd * (g.z + o)));
  v[3] = __bfloat162float(__float2bfloat16(x.w * rstd * (g.w + o)));
}
// whole warp: the row's elements, weights and strip partials are all requested before anything waits on them
__device__ __forceinline__ void norm_row4(const NormIn& n, int row, int col, int lane, float (&v)[4]) {
  const float4 x = __ldcg(reinterpret_cast<const float4*>(n.res + static_cast<size_t>(row) * n.H + col));
  const float4 g = __ldg(reinterpret_cast<const float4*>(n.w + col));
  norm_apply4(n, x, g, norm_rstd(n, row, lane), v);
}
__device__ __forceinline__ void norm_load4(const NormIn& n, int row, int col, float rstd, float (&v)[4]) {
  const float4 x = __ldcg(reinterpret_cast<const float4*>(n.res + static_cast<size_t>(row) * n.H + col));
  const float4 g = __ldg(reinterpret_cast<const float4*>(n.w + col));
  const float o = n.one_plus ? 1.f : 0.f;
  v[0] = __bfloat162float(__float2bfloat16(x.x * rstd * (g.x + o)));
  v[1] = __bfloat162float(__float2bfloat16(x.y * rstd * (g.y + o)));
  v[2] = __bfloat162float(__float2bfloat16(x.z * rstd * (g.z + o)));
  v[3] = __bfloat162float(__float2bfloat16(x.w * rstd * (g.w + o)));
}

}  // namespace spark

// ---------------------------------------------------------------------------------------- host side
// Launch with the programmatic-dependency attribute (the kernel MUST call pdl_wait() before it touches anything
// an earlier launch wrote).  SPARK_PDL=0 turns the attribute off (plain stream order) for A/B timing.
#include <cstdlib>
static inline bool spark_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = std::getenv("SPARK_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t spark_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                           dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = cluster.x; attr[na].val.clusterDim.y = cluster.y; attr[na].val.clusterDim.z = cluster.z;
    ++na;
  }
  if (spark_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr; cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
