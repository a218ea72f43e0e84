// Launch plumbing shared by the decode-round kernels (<= 16 rows per launch).
//
// Programmatic dependent launch.  Decode kernels are launched with the programmatic-stream-serialisation
// attribute: a kernel's CTAs may start while its predecessor drains, issue the loads that depend on
// nothing but weights, and then `pdl_wait()` (griddepcontrol.wait: predecessor complete, its writes
// visible).  Every kernel calls `pdl_trigger()` only AFTER its own wait, so "my successor runs" implies
// "my predecessor's predecessor is complete" and data produced two launches back may be read before the
// wait.  Reference: engine-rs/shim/pdl.cuh:20-41, ds41_ops.cu:593-685.
#pragma once
#include "ptx.cuh"

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
