// Expert-parallel MoE all-to-all over peer memory (NVLink P2P stores issued from the kernels).
//
//   ep_dispatch : one CTA per token: router top-k (softmax-renorm, ties -> lowest expert id), FP8 e4m3
//                 quantisation of the row with one fp32 scale per 128 elements (done ONCE per token), and a
//                 direct scatter of {fp8 row, scales, (token, slot, expert, weight)} into the receive slab of
//                 every selected expert's owner.  Slots are reserved with a LOCAL counter per destination
//                 (each source owns a sub-slab on every destination), so no remote atomics are needed.
//                 The last CTA publishes the per-destination counts and raises the flags.
//   ep_recv     : owner side: bounded wait for every source's flag, then dequantise the received rows into a
//                 compact bf16 matrix + local expert ids (the grouped GEMM's input) and keep the metadata.
//   ep_combine_push   : owner side: every expert output row goes back into slot (token, k) of the return buffer
//                 of the token's home rank.
//   ep_combine_reduce : home side: bounded wait, then out[t] = sum over slots IN SLOT ORDER of w * row
//                 (+ residual).  Arrival order never affects a result: rows are addressed by (token, slot).
// The reference has no expert parallelism (one GPU per node, experts split by intermediate dimension,
// engine-rs/src/moefast.rs:126-147); the counting-sort grouping and slot-order combine it uses
// (engine-rs/shim/moe_exl3.cuh:141-231,1085) carry over to the owner side.
#include "../common/comm.cuh"
#include <cuda_fp8.h>

namespace spark {

struct EpLayout {
  long long slab_off;      // receive slab: [world(src)][cap][row_bytes]
  long long count_off;     // int [world(src)]: rows sent by src
  long long flag_off;      // u32 [world]: dispatch flags
  long long ret_off;       // return buffer on the home rank: bf16 [T_cap * top_k][H]
  long long ret_flag_off;  // u32 [world]: combine flags
  int cap;                 // rows per (src, dst) sub-slab
  int row_bytes;           // H + ep_scale_bytes(H) + 16
  uint32_t* seq_ptr;       // optional device-side sequence counter (graph replay)
};

constexpr int EP_THREADS = 256;

// Bytes of the per-row scale area (one fp32 per 128 elements), padded to 16 bytes so that the metadata that follows
// and the 16-byte row copies stay aligned for every H that is a multiple of 128.
__host__ __device__ constexpr int ep_scale_bytes(int H) { return (((H >> 7) * 4) + 15) & ~15; }

// grid T, 256 threads; H % 2048 == 0 is not required: thread handles 8 consecutive elements per pass.
__global__ void __launch_bounds__(EP_THREADS)
ep_dispatch_kernel(CommCtx c, EpLayout L, uint32_t seq, const __nv_bfloat16* __restrict__ x, int H,
                   const float* __restrict__ logits, int ld, int E, int top_k,
                   float* __restrict__ wts, int* __restrict__ ids, int* __restrict__ send_count,
                   int* __restrict__ done_counter) {
  extern __shared__ __align__(16) uint8_t sm[];
  uint8_t* q = sm;                                          // [H] fp8
  float* scales = reinterpret_cast<float*>(sm + H);         // [H/128]
  __shared__ float rv[EP_THREADS / 32];
  __shared__ int ri[EP_THREADS / 32];
  __shared__ int sel_id[32];
  __shared__ float sel_p[32];
  __shared__ int sel_pos[32];
  seq = comm_seq(L.seq_ptr, seq);
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int epr = E / c.world;

  // ---- router: softmax over E, top-k, renormalise
  const float* lg = logits + static_cast<size_t>(t) * ld;
  float p[4], s[4];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 4; ++j) { const int e = tid + j * EP_THREADS; p[j] = e < E ? lg[e] : -INFINITY; mx = fmaxf(mx, p[j]); }
  mx = warp_max(mx);
  if (lane == 0) rv[warp] = mx;
  __syncthreads();
  mx = rv[0];
  for (int w = 1; w < EP_THREADS / 32; ++w) mx = fmaxf(mx, rv[w]);
  __syncthreads();
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { const int e = tid + j * EP_THREADS; p[j] = e < E ? expf(p[j] - mx) : 0.f; sum += p[j]; }
  sum = warp_sum(sum);
  if (lane == 0) rv[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < EP_THREADS / 32; ++w) sum += rv[w];
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) { p[j] /= sum; s[j] = (tid + j * EP_THREADS) < E ? p[j] : -INFINITY; }
  for (int k = 0; k < top_k; ++k) {
    float best = -INFINITY; int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 4; ++j) { const int e = tid + j * EP_THREADS; if (s[j] > best) { best = s[j]; bi = e; } }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { rv[warp] = best; ri[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < EP_THREADS / 32; ++w) if (rv[w] > best || (rv[w] == best && ri[w] < bi)) { best = rv[w]; bi = ri[w]; }
      sel_id[k] = bi;
    }
    __syncthreads();
    const int win = sel_id[k];
    if ((win % EP_THREADS) == tid) {
#pragma unroll
      for (int j = 0; j < 4; ++j) if (j == win / EP_THREADS) { sel_p[k] = p[j]; s[j] = -INFINITY; }
    }
    __syncthreads();
  }
  if (tid == 0) {
    float tot = 0.f;
    for (int k = 0; k < top_k; ++k) tot += sel_p[k];
    tot = fmaxf(tot, 1e-20f);
    for (int k = 0; k < top_k; ++k) {
      sel_p[k] /= tot;
      wts[static_cast<size_t>(t) * top_k + k] = sel_p[k];
      ids[static_cast<size_t>(t) * top_k + k] = sel_id[k];
      sel_pos[k] = atomicAdd(&send_count[sel_id[k] / epr], 1);      // local reservation in (this src -> dst)
    }
  }
  // ---- quantise the row once: e4m3 with one scale per 128 elements (8 elements per thread per pass)
  const __nv_bfloat16* xr = x + static_cast<size_t>(t) * H;
  for (int base = tid * 8; base < H; base += EP_THREADS * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + base);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8]; float am = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(p2[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; am = fmaxf(am, fmaxf(fabsf(v.x), fabsf(v.y))); }
    // 16 consecutive threads cover one 128-element block
    for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float sc = fmaxf(am, 1e-4f) / 448.f;
    if ((tid & 15) == 0) scales[base >> 7] = sc;
    const float inv = 1.f / sc;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(f[i] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
      hi |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(f[4 + i] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    }
    *reinterpret_cast<uint2*>(q + base) = make_uint2(lo, hi);
  }
  __syncthreads();
  // ---- scatter to the owners
  const int payload16 = (H + ep_scale_bytes(H)) >> 4;            // 16-byte vectors of fp8 row + scales
  for (int k = 0; k < top_k; ++k) {
    const int e = sel_id[k], dst = e / epr, pos = sel_pos[k];
    if (pos >= L.cap) { if (tid == 0) set_status(c.status, ST_BOUNDS, dst, pos, L.cap); continue; }
    uint8_t* row = c.peers[dst] + L.slab_off + (static_cast<size_t>(c.rank) * L.cap + pos) * L.row_bytes;
    for (int i = tid; i < payload16; i += EP_THREADS) reinterpret_cast<uint4*>(row)[i] = reinterpret_cast<const uint4*>(sm)[i];
    if (tid == 0) {
      int4 meta; meta.x = t; meta.y = k; meta.z = e - dst * epr; meta.w = __float_as_int(sel_p[k]);
      *reinterpret_cast<int4*>(row + H + ep_scale_bytes(H)) = meta;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    if (atomicAdd(done_counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *done_counter = 0;
      for (int d = 0; d < c.world; ++d) {
        const int n = min(send_count[d], L.cap);
        *reinterpret_cast<volatile int*>(c.peers[d] + L.count_off + c.rank * 4) = n;
        send_count[d] = 0;
      }
      __threadfence_system();
      for (int d = 0; d < c.world; ++d) st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peers[d] + L.flag_off) + c.rank, seq);
    }
  }
}

// Owner side.  grid-stride over received rows; writes A rows (bf16, compact: source-major), local expert ids,
// metadata {src, token, slot, weight} and the total row count.
__global__ void __launch_bounds__(256)
ep_recv_kernel(CommCtx c, EpLayout L, uint32_t seq, int H, __nv_bfloat16* __restrict__ a_rows,
               int* __restrict__ expert_local, int4* __restrict__ meta_out, int* __restrict__ total) {
  seq = comm_seq(L.seq_ptr, seq);
  __shared__ int base[COMM_MAX_RANKS + 1];
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world && !wait_flag(c, reinterpret_cast<const uint32_t*>(c.peers[c.rank] + L.flag_off) + threadIdx.x, seq, threadIdx.x)) ok_s = 0;
  __syncthreads();
  if (!ok_s) { if (blockIdx.x == 0 && threadIdx.x == 0) *total = 0; return; }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int s = 0; s < c.world; ++s) { base[s] = acc; acc += *reinterpret_cast<const volatile int*>(c.peers[c.rank] + L.count_off + s * 4); }
    base[c.world] = acc;
    if (blockIdx.x == 0) *total = acc;
  }
  __syncthreads();
  const int P = base[c.world];
  for (int i = blockIdx.x; i < P; i += gridDim.x) {
    int src = 0;
    while (i >= base[src + 1]) ++src;
    const int pos = i - base[src];
    const uint8_t* row = c.peers[c.rank] + L.slab_off + (static_cast<size_t>(src) * L.cap + pos) * L.row_bytes;
    const float* sc = reinterpret_cast<const float*>(row + H);
    for (int b = threadIdx.x * 8; b < H; b += blockDim.x * 8) {
      const uint2 raw = *reinterpret_cast<const uint2*>(row + b);
      const float s = sc[b >> 7];
      const __nv_fp8_e4m3* f8 = reinterpret_cast<const __nv_fp8_e4m3*>(&raw);
      __nv_bfloat162 o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(static_cast<float>(f8[2 * j]) * s, static_cast<float>(f8[2 * j + 1]) * s);
      *reinterpret_cast<uint4*>(a_rows + static_cast<size_t>(i) * H + b) = *reinterpret_cast<uint4*>(o);
    }
    if (threadIdx.x == 0) {
      const int4 m = *reinterpret_cast<const int4*>(row + H + ep_scale_bytes(H));
      expert_local[i] = m.z;
      meta_out[i] = make_int4(src, m.x, m.y, m.w);
    }
  }
}

// Owner side: y [P, H] bf16 (row i belongs to meta[i]) -> return buffer of the home rank at (token, slot).
__global__ void __launch_bounds__(256)
ep_combine_push_kernel(CommCtx c, EpLayout L, uint32_t seq, int H, int top_k, const __nv_bfloat16* __restrict__ y,
                       const int4* __restrict__ meta, const int* __restrict__ total, int* __restrict__ done_counter) {
  seq = comm_seq(L.seq_ptr, seq);
  const int P = *total;
  for (int i = blockIdx.x; i < P; i += gridDim.x) {
    const int4 m = meta[i];
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c.peers[m.x] + L.ret_off) + (static_cast<size_t>(m.y) * top_k + m.z) * H;
    const uint4* src = reinterpret_cast<const uint4*>(y + static_cast<size_t>(i) * H);
    for (int b = threadIdx.x; b < (H >> 3); b += blockDim.x) reinterpret_cast<uint4*>(dst)[b] = src[b];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(done_counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *done_counter = 0;
      for (int d = 0; d < c.world; ++d) st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peers[d] + L.ret_flag_off) + c.rank, seq);
    }
  }
}

// Home side: grid T.  out[t] (bf16) = sum_k w[t,k] * ret[t,k,:]; optionally res[t] (fp32) += the same.
__global__ void __launch_bounds__(256)
ep_combine_reduce_kernel(CommCtx c, EpLayout L, uint32_t seq, int H, int top_k, const float* __restrict__ wts,
                         float* __restrict__ res, __nv_bfloat16* __restrict__ out) {
  seq = comm_seq(L.seq_ptr, seq);
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world && !wait_flag(c, reinterpret_cast<const uint32_t*>(c.peers[c.rank] + L.ret_flag_off) + threadIdx.x, seq, threadIdx.x)) ok_s = 0;
  __syncthreads();
  if (!ok_s) return;
  const int t = blockIdx.x;
  const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(c.peers[c.rank] + L.ret_off) + static_cast<size_t>(t) * top_k * H;
  for (int b = threadIdx.x * 8; b < H; b += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top_k; ++k) {                      // slot order
      const float w = wts[static_cast<size_t>(t) * top_k + k];
      const uint4 raw = *reinterpret_cast<const uint4*>(ret + static_cast<size_t>(k) * H + b);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 v = __bfloat1622float2(p2[j]); acc[2 * j] = fmaf(w, v.x, acc[2 * j]); acc[2 * j + 1] = fmaf(w, v.y, acc[2 * j + 1]); }
    }
    if (res) {
      float* r = res + static_cast<size_t>(t) * H + b;
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] += acc[j];
    }
    if (out) {
      __nv_bfloat162 o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + b) = *reinterpret_cast<uint4*>(o);
    }
  }
}

}  // namespace spark

using namespace spark;

struct HostCtxE { void* peers[8]; int rank, world; unsigned long long wait_ns; int* status; };
static CommCtx to_ctx_e(const HostCtxE* h) {
  CommCtx c;
  for (int i = 0; i < COMM_MAX_RANKS; ++i) c.peers[i] = static_cast<uint8_t*>(h->peers[i]);
  c.rank = h->rank; c.world = h->world; c.wait_ns = h->wait_ns; c.status = h->status;
  return c;
}

extern "C" int spark_ep_row_bytes(int H) { return H + ep_scale_bytes(H) + 16; }

extern "C" int spark_ep_dispatch(const HostCtxE* h, const EpLayout* L, unsigned seq, const void* x, int T, int H,
                                 const float* logits, int ld, int E, int top_k, float* wts, int* ids, int* send_count,
                                 int* done_counter, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 128 || E > 1024 || top_k > 32 || E % h->world || L->row_bytes != H + ep_scale_bytes(H) + 16) return -5;
  const int smem = H + ep_scale_bytes(H);
  ep_dispatch_kernel<<<T, EP_THREADS, smem, s>>>(to_ctx_e(h), *L, seq, (const __nv_bfloat16*)x, H, logits, ld, E, top_k, wts,
                                                  ids, send_count, done_counter);
  return spark_launch_rc(__func__);
}

// A rank with no tokens still has to raise its flags: dispatch with T == 0 goes through this.
__global__ void ep_empty_flags_kernel(CommCtx c, EpLayout L, uint32_t seq, int which) {
  seq = comm_seq(L.seq_ptr, seq);
  const int d = threadIdx.x;
  if (d < c.world) {
    if (which == 0) *reinterpret_cast<volatile int*>(c.peers[d] + L.count_off + c.rank * 4) = 0;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(c.peers[d] + (which == 0 ? L.flag_off : L.ret_flag_off)) + c.rank, seq);
  }
}
extern "C" int spark_ep_empty(const HostCtxE* h, const EpLayout* L, unsigned seq, int which, cudaStream_t s) {
  ep_empty_flags_kernel<<<1, 32, 0, s>>>(to_ctx_e(h), *L, seq, which);
  return spark_launch_rc(__func__);
}

extern "C" int spark_ep_recv(const HostCtxE* h, const EpLayout* L, unsigned seq, int H, void* a_rows, int* expert_local,
                             void* meta_out, int* total, int max_rows, cudaStream_t s) {
  int grid = max_rows < 1184 ? (max_rows > 0 ? max_rows : 1) : 1184;
  ep_recv_kernel<<<grid, 256, 0, s>>>(to_ctx_e(h), *L, seq, H, (__nv_bfloat16*)a_rows, expert_local, (int4*)meta_out, total);
  return spark_launch_rc(__func__);
}

extern "C" int spark_ep_combine_push(const HostCtxE* h, const EpLayout* L, unsigned seq, int H, int top_k, const void* y,
                                     const void* meta, const int* total, int* done_counter, int max_rows, cudaStream_t s) {
  int grid = max_rows < 1184 ? (max_rows > 0 ? max_rows : 1) : 1184;
  ep_combine_push_kernel<<<grid, 256, 0, s>>>(to_ctx_e(h), *L, seq, H, top_k, (const __nv_bfloat16*)y, (const int4*)meta, total,
                                              done_counter);
  return spark_launch_rc(__func__);
}

extern "C" int spark_ep_combine_reduce(const HostCtxE* h, const EpLayout* L, unsigned seq, int T, int H, int top_k,
                                       const float* wts, float* res, void* out, cudaStream_t s) {
  if (T <= 0) return 0;
  ep_combine_reduce_kernel<<<T, 256, 0, s>>>(to_ctx_e(h), *L, seq, H, top_k, wts, res, (__nv_bfloat16*)out);
  return spark_launch_rc(__func__);
}
