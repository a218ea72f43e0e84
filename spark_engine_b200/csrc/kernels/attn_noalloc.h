// Decode attention without any allocation.  This entry point has no counterpart in the reference.
//
// Who needs it: code that runs where device memory cannot be allocated -- a host that drives the engine from
// inside a CUDA-graph capture or a real-time loop where cudaMalloc (a synchronising, possibly failing call) is
// forbidden, an embedding process that hands this library a fixed memory budget and no allocator, or a plain C
// caller without PyTorch's caching allocator behind it.  spark_attn_decode needs a scratch buffer for the
// per-split partial results; here that buffer is a fixed array compiled into the library.
//
// Contract
//   * Inputs and outputs are the caller's (same meaning as spark_attn_decode); nothing is allocated or freed,
//     by this call or by anything it calls.
//   * The built-in scratch holds SPARK_ATTN_NOALLOC_MAX_FLOATS floats (16 MiB).  Every GPU whose context
//     loads this library carries that array until the process exits.  A call needs
//     rows * q_heads * splits * (head_dim + 2) floats; a larger request is refused with
//     SPARK_ATTN_NOALLOC_TOO_LARGE and a message on stderr, and nothing is launched.
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress, with that
//     device current).  Make that first call outside any stream capture.
//   * All calls on a device share the one array, and it keeps whatever the previous call left in it.  The
//     kernels write every partial they later read, so nothing has to be cleared between calls; but two calls
//     whose kernels overlap on the GPU (different streams, no ordering between them) race on the array.
//     Serialise them.
#pragma once
#include <cuda_runtime.h>

#define SPARK_ATTN_NOALLOC_MAX_FLOATS (4ll << 20)
#define SPARK_ATTN_NOALLOC_TOO_LARGE (-22)

#ifdef __cplusplus
extern "C" {
#endif
// qbuf [R,Hq,D] bf16 queries (normed, roped); kc/vc KV pool [tokens,Hkv,D] bf16 (or e4m3 with ks/vs fp32 scales
// [tokens,Hkv] when fp8 != 0); pos [R] position of each row; row_kv [R] first KV row of each row's sequence;
// sel/sel_n optional selected-token lists [R, sel_ld] / [R]; nsplit = ceil(max context / 64); qkv/ld/gated: the
// fused projection rows holding the per-head output gate; out [R, Hq*D] bf16.  Returns 0, a negative launch
// error, or SPARK_ATTN_NOALLOC_TOO_LARGE.
int spark_attn_decode_noalloc(const void* qbuf, const void* kc, const void* vc, const float* ks, const float* vs,
                              int fp8, const int* pos, const long long* row_kv, const int* sel, const int* sel_n,
                              int sel_ld, int nsplit, const void* qkv, int ld, int gated, int R, int Hq, int Hkv,
                              int D, float scale, void* out, cudaStream_t s);
#ifdef __cplusplus
}
#endif
