// Device-side building blocks of the peer-memory collectives (NVLink P2P loads/stores inside kernels).
//
// Every rank owns an arena; `CommCtx` carries the base pointer of every rank's arena as mapped into
// this process (IPC), so a kernel addresses a peer's buffer as peers[p] + offset.  Signalling uses
// monotonically increasing sequence numbers written with st.release.sys and polled with
// ld.acquire.sys.  EVERY wait is bounded by a wall-clock budget (%globaltimer): when it runs out the
// kernel records {ST_TIMEOUT_PEER_FLAG, peer, expected, seen} in the status word and returns, so a
// missing peer can never hang the GPU (the reference traps after 2^34 polls, engine-rs/shim/rdma_ar.cu:83).
// No TMA, and in particular no multicast load, ever touches peer memory here.
#pragma once
#include "ptx.cuh"

namespace spark {

constexpr int COMM_MAX_RANKS = 8;

struct CommCtx {
  uint8_t* peers[COMM_MAX_RANKS];   // arena base of every rank (peers[rank] = local arena)
  int rank, world;
  unsigned long long wait_ns;       // budget of one device-side wait
  int* status;                      // local status word (int[4])
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Flag store that follows a fence.acq_rel.sys issued by the same thread: fence + relaxed store is a release pattern, and
// unlike st.release (a fence of its own per store) the stores to the 2..8 peers go out back to back.  With one
// st.release per peer the flag fan-out of an 8-rank all-reduce alone took ~15 us.
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Wait until *flag >= expect (sequence numbers only grow).  false = budget exhausted (status recorded).
__device__ __forceinline__ bool wait_flag(const CommCtx& c, const uint32_t* flag, uint32_t expect, int peer) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t seen = 0;
  for (;;) {
    seen = ld_acquire_sys(flag);
    if (static_cast<int32_t>(seen - expect) >= 0) return true;
    if (globaltimer_ns() - t0 > c.wait_ns) break;
    __nanosleep(40);
  }
  set_status(c.status, ST_TIMEOUT_PEER_FLAG, peer, static_cast<int>(expect), static_cast<int>(seen));
  return false;
}

// 16-byte vector helpers
__device__ __forceinline__ float4 ld_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st_f4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

// ------------------------------------------------------------------------------------------ one-shot AR
struct ArRows {
  CommCtx c;
  long long slot_off;        // float slots [2][world][rows_cap * N]
  long long flag_off;        // u32 [world]
  uint32_t seq;
  int rows_cap, R, N;
  const void* in; int in_f32;            // local partial rows [R, N]
  int* counter;                          // local, zero between launches
  float* res;                            // optional fp32 residual [R, N] (in/out): res += sum
  const float* norm_w; float eps;        // optional RMSNorm weights
  void* out; int out_f32;                // sum (no norm) or normed rows; bf16 or fp32 [R, N]
  uint32_t* seq_ptr;                     // optional device-side sequence counter (CUDA-graph replay): the kernel
                                         // uses *seq_ptr + 1 and the last CTA stores it back
  // optional producer of the local rows: the slot-order combine of a decode-round MoE (in == nullptr):
  //   row r = sum_k moe_w[r, k] * moe_y[r * slots + k, :]  (pairs with moe_ids < 0 belong to other ranks)
  //           (+ moe_sg[r] * moe_shared[r, :])
  const float* moe_y; const float* moe_w; const int* moe_ids; int moe_slots;
  const __nv_bfloat16* moe_shared; const float* moe_sg;
  long long ll_off;                      // >= 0: decode rounds travel as {value, sequence} words in this region (see below)
};

// Low-latency wire format of the decode all-reduce (R <= AR_LL_ROWS rows): every element travels as an 8-byte
// {value, sequence} word, so a receiver knows a value has arrived by looking at the value itself -- no fence, no arrival
// counter, no flag fan-out and no flag poll between the pushes and the sum.  A 16-byte store carries two such words;
// its 8-byte halves are single-copy atomic and the reader checks both sequence fields.  Region: u64 [2][world][16 * N],
// the set alternates with the parity of the sequence number (a rank can only push number k + 2 after it finished k + 1,
// which needed every rank's k + 1 pushes, which every rank issued after finishing k).
// Reference: engine-rs/shim/rdma_arn.cu:129-164 (flag-in-data wire format of the decode all-reduce).
constexpr int AR_LL_ROWS = 16;
__device__ __forceinline__ void st_ll(uint4* p, float a, float b, uint32_t seq) {
  asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(a)), "r"(seq),
               "r"(__float_as_uint(b)), "r"(seq) : "memory");
}
__device__ __forceinline__ uint4 ld_ll(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// 16-byte slot that holds elements [i, i + 2) of row r as pushed by rank `src`, in the arena that `base` points at
__device__ __forceinline__ uint4* ll_slot(uint8_t* base, long long ll_off, uint32_t seq, int world, int src, int r, int N, int i) {
  const size_t set = static_cast<size_t>(seq & 1) * world * AR_LL_ROWS * N;
  return reinterpret_cast<uint4*>(base + ll_off) + (set + (static_cast<size_t>(src) * AR_LL_ROWS + r) * N + i) / 2;
}

// Four consecutive elements of this rank's partial row: from `in`, or combined from the expert outputs.
__device__ __forceinline__ float4 ar_local4(const ArRows& a, int r, int i) {
  if (a.in != nullptr) {
    if (a.in_f32) return ld_f4(reinterpret_cast<const float*>(a.in) + static_cast<size_t>(r) * a.N + i);
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.in) + static_cast<size_t>(r) * a.N + i);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 f0 = __bfloat1622float2(p2[0]), f1 = __bfloat1622float2(p2[1]);
    return make_float4(f0.x, f0.y, f1.x, f1.y);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k0 = 0; k0 < a.moe_slots; k0 += 4) {            // four slots' loads in flight; summed in slot order
    float4 v[4]; float w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int pi = r * a.moe_slots + k0 + u;
      const bool live = (k0 + u) < a.moe_slots && a.moe_ids[pi] >= 0;
      w[u] = live ? a.moe_w[pi] : 0.f;
      v[u] = live ? ld_f4(a.moe_y + static_cast<size_t>(pi) * a.N + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      acc.x = fmaf(w[u], v[u].x, acc.x); acc.y = fmaf(w[u], v[u].y, acc.y);
      acc.z = fmaf(w[u], v[u].z, acc.z); acc.w = fmaf(w[u], v[u].w, acc.w);
    }
  }
  if (a.moe_shared != nullptr) {
    const uint2 raw = *reinterpret_cast<const uint2*>(a.moe_shared + static_cast<size_t>(r) * a.N + i);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 f0 = __bfloat1622float2(p2[0]), f1 = __bfloat1622float2(p2[1]);
    const float g = a.moe_sg ? a.moe_sg[r] : 1.f;
    acc.x += g * f0.x; acc.y += g * f0.y; acc.z += g * f1.x; acc.w += g * f1.y;
  }
  return acc;
}

// Sequence number of this launch: from the device counter when there is one (replayed graphs), else the
// host-provided value.
__device__ __forceinline__ uint32_t comm_seq(const uint32_t* seq_ptr, uint32_t host_seq) {
  return seq_ptr ? *reinterpret_cast<const volatile uint32_t*>(seq_ptr) + 1u : host_seq;
}

// Shared tail: wait for every rank's flag, then rows r = first, first+stride, ...: rank-ordered sum
// (+ residual)(+ RMSNorm).  Called by whole CTAs (blockDim.x threads).
__device__ __forceinline__ void ar_rows_tail(const ArRows& a, uint32_t seq, int first_row, int row_stride, float* red_smem) {
  const int W = a.c.world;
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < W) {
    if (!wait_flag(a.c, reinterpret_cast<const uint32_t*>(a.c.peers[a.c.rank] + a.flag_off) + threadIdx.x, seq, threadIdx.x))
      ok_s = 0;
  }
  __syncthreads();
  if (!ok_s) return;
  const float* slots = reinterpret_cast<const float*>(a.c.peers[a.c.rank] + a.slot_off) +
                       static_cast<size_t>(seq & 1) * W * a.rows_cap * a.N;
  for (int r = first_row; r < a.R; r += row_stride) {
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < a.N; i += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < W; ++p) {                       // fixed rank order
        const float4 v = ld_f4(slots + (static_cast<size_t>(p) * a.rows_cap + r) * a.N + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (a.res) {
        float4 rv = ld_f4(a.res + static_cast<size_t>(r) * a.N + i);
        acc.x += rv.x; acc.y += rv.y; acc.z += rv.z; acc.w += rv.w;
        st_f4(a.res + static_cast<size_t>(r) * a.N + i, acc);
      }
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
      if (!a.norm_w) {
        if (a.out_f32) st_f4(reinterpret_cast<float*>(a.out) + static_cast<size_t>(r) * a.N + i, acc);
        else {
          __nv_bfloat162 b0 = __floats2bfloat162_rn(acc.x, acc.y), b1 = __floats2bfloat162_rn(acc.z, acc.w);
          uint2 o; o.x = *reinterpret_cast<uint32_t*>(&b0); o.y = *reinterpret_cast<uint32_t*>(&b1);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + static_cast<size_t>(r) * a.N + i) = o;
        }
      } else if (!a.res) {
        // no residual buffer to re-read from: stash the sum in the fp32 output slot of this rank's parity set
        st_f4(const_cast<float*>(slots) + (static_cast<size_t>(a.c.rank) * a.rows_cap + r) * a.N + i, acc);
      }
    }
    if (a.norm_w) {
      ss = warp_sum(ss);
      if ((threadIdx.x & 31) == 0) red_smem[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red_smem[w];
      __syncthreads();
      const float rs = rsqrtf(tot / a.N + a.eps);
      const float* src = a.res ? a.res + static_cast<size_t>(r) * a.N
                               : slots + (static_cast<size_t>(a.c.rank) * a.rows_cap + r) * a.N;
      for (int i = threadIdx.x * 4; i < a.N; i += blockDim.x * 4) {
        const float4 v = ld_f4(src + i), g = ld_f4(a.norm_w + i);
        const float4 o4 = make_float4(v.x * rs * g.x, v.y * rs * g.y, v.z * rs * g.z, v.w * rs * g.w);
        if (a.out_f32) st_f4(reinterpret_cast<float*>(a.out) + static_cast<size_t>(r) * a.N + i, o4);
        else {
          __nv_bfloat162 b0 = __floats2bfloat162_rn(o4.x, o4.y), b1 = __floats2bfloat162_rn(o4.z, o4.w);
          uint2 o; o.x = *reinterpret_cast<uint32_t*>(&b0); o.y = *reinterpret_cast<uint32_t*>(&b1);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + static_cast<size_t>(r) * a.N + i) = o;
        }
      }
    }
  }
}

// Signal "all my rows are in every peer's slot": called by one thread after the CTA's pushes are fenced.
__device__ __forceinline__ bool ar_arrive_and_is_last(const ArRows& a, uint32_t seq, int n_ctas) {
  __threadfence_system();
  const int old = atomicAdd(a.counter, 1);
  if (old != n_ctas - 1) return false;
  *a.counter = 0;
  for (int p = 0; p < a.c.world; ++p)      // (the fence above orders this rank's pushes before the flags)
    st_relaxed_sys(reinterpret_cast<uint32_t*>(a.c.peers[p] + a.flag_off) + a.c.rank, seq);
  if (a.seq_ptr) *a.seq_ptr = seq;       // every CTA of this launch has read the counter before arriving
  return true;
}


}  // namespace spark
