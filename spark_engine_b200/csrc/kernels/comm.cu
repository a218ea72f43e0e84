// Peer-memory collectives over NVLink / NVSwitch (P2P loads and stores issued from ordinary CTAs).
//
//   arena management : cudaMalloc'd arena per rank, cudaIpc handle export / import
//   barrier          : sequence-number barrier across ranks
//   allreduce_rows   : one-shot all-reduce of R rows (push to every peer, rank-ordered fp32 sum), optionally
//                      fused with residual add + RMSNorm  (decode / verify rows)
//   rs_push / rs_finish / ag_wait : reduce-scatter by row blocks (+ residual + RMSNorm on the owned rows) and
//                      all-gather of the result (prefill, sequence-parallel style)
//   ag_push          : all-gather of row blocks into every peer's arena (prologue of the AG-fused GEMM)
//   ep_dispatch / ep_combine : expert-parallel all-to-all, see ep.cu
//
// Sums are taken in rank order from fp32 slots, so every rank computes bit-identical results and the
// result equals the local rank-ordered sum (the contract of the reference's RDMA transport,
// engine-rs/shim/rdma_arn.cu:84-125,104-113).  Two slot sets alternate by sequence parity: a rank can only
// reach sequence s+2 after every peer has finished reading set s.
#include "../common/comm.cuh"
#include "../common/decode.cuh"

namespace spark {

// ------------------------------------------------------------------------------------------ barrier
// flags: u32 [world] in every arena at flag_off.  Rank r writes seq into slot r of every peer, then waits
// for all slots of its own arena.
__global__ void comm_barrier_kernel(CommCtx c, long long flag_off, uint32_t seq) {
  const int p = threadIdx.x;
  if (p < c.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(c.peers[p] + flag_off) + c.rank, seq);
    wait_flag(c, reinterpret_cast<const uint32_t*>(c.peers[c.rank] + flag_off) + p, seq, p);
  }
}

// (ArRows, ar_rows_tail and ar_arrive_and_is_last live in comm.cuh: the fused GEMV epilogues share them)

// grid = R CTAs (one row each), 256 threads.  N % 4 == 0.
__global__ void __launch_bounds__(256)
allreduce_rows_kernel(ArRows a_in) {
  pdl_wait();
  pdl_trigger();
  ArRows a = a_in;
  a.seq = comm_seq(a.seq_ptr, a.seq);
  __shared__ float red[8];
  __shared__ int last_s;
  const int r = blockIdx.x, W = a.c.world;
  const size_t set = static_cast<size_t>(a.seq & 1) * W * a.rows_cap * a.N;
  for (int i = threadIdx.x * 4; i < a.N; i += blockDim.x * 4) {
    const float4 v = ar_local4(a, r, i);
    for (int p = 0; p < W; ++p) {
      float* dst = reinterpret_cast<float*>(a.c.peers[p] + a.slot_off) + set + (static_cast<size_t>(a.c.rank) * a.rows_cap + r) * a.N + i;
      st_f4(dst, v);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) last_s = ar_arrive_and_is_last(a, a.seq, gridDim.x) ? 1 : 0;
  __syncthreads();
  // every CTA finishes its own row once all flags are in
  ar_rows_tail(a, a.seq, r, gridDim.x, red);
}

// Low-latency all-reduce (wire format: comm.cuh).  grid = R CTAs (one row each), 256 threads, N <= 8192, N % 4 == 0.
// PUSH = false: the rows were pushed by another kernel's epilogue (the row-parallel EXL3 GEMV); this launch only sums.
template <bool PUSH>
__global__ void __launch_bounds__(256)
allreduce_rows_ll_kernel(ArRows a_in) {
  const long long ll_off = a_in.ll_off;
  pdl_wait();
  pdl_trigger();
  ArRows a = a_in;
  const uint32_t seq = comm_seq(a.seq_ptr, a.seq);
  __shared__ float red[8];
  const int r = blockIdx.x, W = a.c.world, N = a.N;
  constexpr int KEEP = 8;                                                         // float4 per thread: N <= 256 * 4 * KEEP
  float4 keep[KEEP];
#pragma unroll
  for (int ki = 0; ki < KEEP; ++ki) {
    const int i = threadIdx.x * 4 + ki * 1024;
    if (i >= N) break;
    if (!PUSH) break;
    const float4 v = ar_local4(a, r, i);
    for (int p = 0; p < W; ++p) {
      uint4* dst = ll_slot(a.c.peers[p], ll_off, seq, W, a.c.rank, r, N, i);
      st_ll(dst, v.x, v.y, seq);
      st_ll(dst + 1, v.z, v.w, seq);
    }
  }
  // rank-ordered sum of the row: every word is polled until it carries this launch's sequence number (bounded)
  const unsigned long long t0 = globaltimer_ns();
  float ss = 0.f;
#pragma unroll
  for (int ki = 0; ki < KEEP; ++ki) {
    const int i = threadIdx.x * 4 + ki * 1024;
    if (i >= N) break;
    // every peer's words are requested together (one memory latency for the whole set, not one per peer); words that
    // do not carry this launch's sequence number yet are asked for again
    uint4 w0[COMM_MAX_RANKS], w1[COMM_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < COMM_MAX_RANKS; ++p) {
      if (p < W) {
        const uint4* src = ll_slot(a.c.peers[a.c.rank], ll_off, seq, W, p, r, N, i);
        w0[p] = ld_ll(src); w1[p] = ld_ll(src + 1);
      }
    }
    for (;;) {
      bool ready = true;
#pragma unroll
      for (int p = 0; p < COMM_MAX_RANKS; ++p)
        if (p < W && (w0[p].y != seq || w0[p].w != seq || w1[p].y != seq || w1[p].w != seq)) ready = false;
      if (ready) break;
      if (globaltimer_ns() - t0 > a.c.wait_ns) {
        set_status(a.c.status, ST_TIMEOUT_PEER_FLAG, -1, static_cast<int>(seq), static_cast<int>(w0[0].y));
        break;
      }
#pragma unroll
      for (int p = 0; p < COMM_MAX_RANKS; ++p) {
        if (p < W && (w0[p].y != seq || w0[p].w != seq || w1[p].y != seq || w1[p].w != seq)) {
          const uint4* src = ll_slot(a.c.peers[a.c.rank], ll_off, seq, W, p, r, N, i);
          w0[p] = ld_ll(src); w1[p] = ld_ll(src + 1);
        }
      }
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < COMM_MAX_RANKS; ++p) {               // fixed rank order
      if (p < W) {
        acc.x += __uint_as_float(w0[p].x); acc.y += __uint_as_float(w0[p].z);
        acc.z += __uint_as_float(w1[p].x); acc.w += __uint_as_float(w1[p].z);
      }
    }
    if (a.res) {
      const float4 rv = ld_f4(a.res + static_cast<size_t>(r) * N + i);
      acc.x += rv.x; acc.y += rv.y; acc.z += rv.z; acc.w += rv.w;
      st_f4(a.res + static_cast<size_t>(r) * N + i, acc);
    }
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    keep[ki] = acc;
  }
  float rs = 1.f;
  if (a.norm_w) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += red[w];
    rs = rsqrtf(tot / N + a.eps);
  }
#pragma unroll
  for (int ki = 0; ki < KEEP; ++ki) {
    const int i = threadIdx.x * 4 + ki * 1024;
    if (i >= N) break;
    float4 v = keep[ki];
    if (a.norm_w) { const float4 g = ld_f4(a.norm_w + i); v.x *= rs * g.x; v.y *= rs * g.y; v.z *= rs * g.z; v.w *= rs * g.w; }
    if (a.out_f32) st_f4(reinterpret_cast<float*>(a.out) + static_cast<size_t>(r) * N + i, v);
    else {
      __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
      uint2 o; o.x = *reinterpret_cast<uint32_t*>(&b0); o.y = *reinterpret_cast<uint32_t*>(&b1);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + static_cast<size_t>(r) * N + i) = o;
    }
  }
  // the last CTA to finish publishes the sequence number for the next launch (every CTA read it at entry)
  __syncthreads();
  if (threadIdx.x == 0 && a.seq_ptr) {
    if (atomicAdd(a.counter, 1) == static_cast<int>(gridDim.x) - 1) { *a.counter = 0; *a.seq_ptr = seq; }
  }
}

// ------------------------------------------------------------------------------------------ vocabulary-parallel arg-max
// Every rank scores its slice of the vocabulary; only (value, index) packets travel.  Stage 1 (many CTAs per row)
// leaves per-chunk winners; stage 2 (one warp per row) picks the local winner, stores the packet {value, global id}
// into slot [rank][row] of every peer, raises the flags once all rows are out, waits (bounded) for every rank's
// flag and picks the global winner in rank order (ties -> lowest id), so all ranks agree bit for bit.
// Reference: engine-rs/src/head_select.rs:42-67, shim/latent.cu:901-940 (gumbel_argmax_part / _packet).
struct PkArgs {
  CommCtx c;
  long long slot_off;        // float2-sized packets [2][world][rows_cap]
  long long flag_off;        // u32 [world]
  uint32_t* seq_ptr;         // device-side sequence counter
  int* counter;
  int rows_cap, vocab_off;
};

__global__ void __launch_bounds__(256)
tp_argmax_part_kernel(const float* __restrict__ logits, int V, float* __restrict__ pv, int* __restrict__ pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, c = blockIdx.y, nc = gridDim.y;
  const int per = (V + nc - 1) / nc;
  const int i0 = c * per, i1 = min(V, i0 + per);
  const float* x = logits + static_cast<size_t>(r) * V;
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += 256) {
    const float v = x[i];
    if (v > best) { best = v; bi = i; }                   // ascending i per thread: first maximum kept
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) if (sv[i] > best || (sv[i] == best && si[i] < bi)) { best = sv[i]; bi = si[i]; }
    pv[r * nc + c] = best; pi[r * nc + c] = bi;
  }
}

// grid R (<= 64, all co-resident), 32 threads
__global__ void tp_argmax_packets_kernel(PkArgs a, const float* __restrict__ pv, const int* __restrict__ pi, int nc,
                                         int* __restrict__ out_id) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, lane = threadIdx.x, W = a.c.world;
  const uint32_t seq = comm_seq(a.seq_ptr, 0);
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int i = lane; i < nc; i += 32) {
    const float v = pv[r * nc + i]; const int ix = pi[r * nc + i];
    if (v > best || (v == best && ix < bi)) { best = v; bi = ix; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const size_t set = static_cast<size_t>(seq & 1) * W * a.rows_cap;
  if (lane < W) {
    float2 pk; pk.x = best; pk.y = __int_as_float(bi + a.vocab_off);
    *reinterpret_cast<float2*>(a.c.peers[lane] + a.slot_off + (set + static_cast<size_t>(a.c.rank) * a.rows_cap + r) * 8) = pk;
  }
  __syncwarp();
  if (lane == 0) {
    __threadfence_system();
    if (atomicAdd(a.counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *a.counter = 0;
      for (int p = 0; p < W; ++p) st_relaxed_sys(reinterpret_cast<uint32_t*>(a.c.peers[p] + a.flag_off) + a.c.rank, seq);
      *a.seq_ptr = seq;
    }
  }
  bool ok = true;
  if (lane < W) ok = wait_flag(a.c, reinterpret_cast<const uint32_t*>(a.c.peers[a.c.rank] + a.flag_off) + lane, seq, lane);
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) { if (lane == 0) out_id[r] = 0; return; }
  if (lane == 0) {
    float gv = -INFINITY; int gi = 0x7fffffff;
    for (int p = 0; p < W; ++p) {                          // rank order; ties -> lowest id
      const float* q = reinterpret_cast<const float*>(a.c.peers[a.c.rank] + a.slot_off + (set + static_cast<size_t>(p) * a.rows_cap + r) * 8);
      const float pvx = __ldcg(q);
      const int ix = __float_as_int(__ldcg(q + 1));
      if (pvx > gv || (pvx == gv && ix < gi)) { gv = pvx; gi = ix; }
    }
    out_id[r] = gi;
  }
}

// ------------------------------------------------------------------------------------------ RS / AG by rows
struct RsAg {
  CommCtx c;
  long long slot_off;        // float partial slots on the OWNER: [world(src)][rows_per_rank * N]
  long long out_off;         // gathered result rows in every arena: bf16 [M, N]
  long long flag_rs_off, flag_ag_off;   // u32 [world] each
  uint32_t seq;
  int M, N, rows_per_rank;   // M = world * rows_per_rank (padded)
  const void* in; int in_f32;            // local partial [M, N]
  int* counter;
  float* res;                            // fp32 residual of the OWNED rows [rows_per_rank, N] (optional)
  const float* norm_w; float eps;
  uint32_t* seq_ptr;
};

// push every row block to its owner (grid-stride over rows), then flag all owners
__global__ void __launch_bounds__(256)
rs_push_kernel(RsAg a_in) {
  RsAg a = a_in;
  a.seq = comm_seq(a.seq_ptr, a.seq);
  const int W = a.c.world;
  for (int row = blockIdx.x; row < a.M; row += gridDim.x) {
    const int owner = row / a.rows_per_rank, lr = row - owner * a.rows_per_rank;
    float* dst = reinterpret_cast<float*>(a.c.peers[owner] + a.slot_off) + (static_cast<size_t>(a.c.rank) * a.rows_per_rank + lr) * a.N;
    for (int i = threadIdx.x * 4; i < a.N; i += blockDim.x * 4) {
      float4 v;
      if (a.in_f32) v = ld_f4(reinterpret_cast<const float*>(a.in) + static_cast<size_t>(row) * a.N + i);
      else {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.in) + static_cast<size_t>(row) * a.N + i);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 f0 = __bfloat1622float2(p2[0]), f1 = __bfloat1622float2(p2[1]);
        v = make_float4(f0.x, f0.y, f1.x, f1.y);
      }
      st_f4(dst + i, v);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *a.counter = 0;
      for (int p = 0; p < W; ++p) st_relaxed_sys(reinterpret_cast<uint32_t*>(a.c.peers[p] + a.flag_rs_off) + a.c.rank, a.seq);
    }
  }
}

// owner: wait all sources, rank-ordered sum (+ residual + RMSNorm) of the owned rows, push the bf16 result row
// into every peer's gathered buffer, then flag.  grid-stride over the owned rows.
__global__ void __launch_bounds__(256)
rs_finish_ag_push_kernel(RsAg a_in) {
  RsAg a = a_in;
  a.seq = comm_seq(a.seq_ptr, a.seq);
  __shared__ float red[8];
  __shared__ int ok_s;
  const int W = a.c.world;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < W && !wait_flag(a.c, reinterpret_cast<const uint32_t*>(a.c.peers[a.c.rank] + a.flag_rs_off) + threadIdx.x, a.seq, threadIdx.x)) ok_s = 0;
  __syncthreads();
  if (ok_s) {
    const float* slots = reinterpret_cast<const float*>(a.c.peers[a.c.rank] + a.slot_off);
    for (int lr = blockIdx.x; lr < a.rows_per_rank; lr += gridDim.x) {
      float ss = 0.f;
      float4 keep[4];                    // N <= 256 threads * 4 * 4 = 4096 per pass; larger N loops twice
      int ki = 0;
      for (int i = threadIdx.x * 4; i < a.N; i += blockDim.x * 4, ++ki) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < W; ++p) {
          const float4 v = ld_f4(slots + (static_cast<size_t>(p) * a.rows_per_rank + lr) * a.N + i);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (a.res) {
          const float4 rv = ld_f4(a.res + static_cast<size_t>(lr) * a.N + i);
          acc.x += rv.x; acc.y += rv.y; acc.z += rv.z; acc.w += rv.w;
          st_f4(a.res + static_cast<size_t>(lr) * a.N + i, acc);
        }
        ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
        if (ki < 4) keep[ki] = acc;
      }
      float rs = 1.f;
      if (a.norm_w) {
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < 8; ++w) tot += red[w];
        __syncthreads();
        rs = rsqrtf(tot / a.N + a.eps);
      }
      const int grow = a.c.rank * a.rows_per_rank + lr;
      ki = 0;
      for (int i = threadIdx.x * 4; i < a.N; i += blockDim.x * 4, ++ki) {
        float4 v = keep[ki < 4 ? ki : 3];
        if (a.norm_w) { const float4 g = ld_f4(a.norm_w + i); v.x *= rs * g.x; v.y *= rs * g.y; v.z *= rs * g.z; v.w *= rs * g.w; }
        __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
        uint2 o; o.x = *reinterpret_cast<uint32_t*>(&b0); o.y = *reinterpret_cast<uint32_t*>(&b1);
        for (int p = 0; p < W; ++p)
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.c.peers[p] + a.out_off) + static_cast<size_t>(grow) * a.N + i) = o;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(a.counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *a.counter = 0;
      for (int p = 0; p < W; ++p) st_relaxed_sys(reinterpret_cast<uint32_t*>(a.c.peers[p] + a.flag_ag_off) + a.c.rank, a.seq);
    }
  }
}

// Waits for every rank's flag; with a device counter and `bump` it closes the sequence (stores seq back).
__global__ void wait_flags_kernel(CommCtx c, long long flag_off, uint32_t seq, uint32_t* seq_ptr, int bump) {
  seq = comm_seq(seq_ptr, seq);
  if (threadIdx.x < c.world)
    wait_flag(c, reinterpret_cast<const uint32_t*>(c.peers[c.rank] + flag_off) + threadIdx.x, seq, threadIdx.x);
  __syncthreads();
  if (threadIdx.x == 0 && seq_ptr && bump) *seq_ptr = seq;
}
__global__ void seq_bump_kernel(uint32_t* seq_ptr) { *seq_ptr = *seq_ptr + 1u; }

// ------------------------------------------------------------------------------------------ AG push
// Copy this rank's row block x [rows, K] (bf16) into every peer's gathered buffer at row rank*rows, then flag.
__global__ void __launch_bounds__(256)
ag_push_kernel(CommCtx c, const __nv_bfloat16* __restrict__ x, int rows, int K, long long buf_off, long long flag_off,
               uint32_t seq, int* counter, const uint32_t* seq_ptr) {
  seq = comm_seq(seq_ptr, seq);
  const int W = c.world;
  const int KV = K >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * K);
    for (int i = threadIdx.x; i < KV; i += blockDim.x) {
      const uint4 v = src[i];
      for (int p = 0; p < W; ++p)
        reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(c.peers[p] + buf_off) + (static_cast<size_t>(c.rank) * rows + r) * K)[i] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *counter = 0;
      for (int p = 0; p < W; ++p) st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peers[p] + flag_off) + c.rank, seq);
    }
  }
}

}  // namespace spark

using namespace spark;

// ------------------------------------------------------------------------------------------ host API
extern "C" void* spark_arena_alloc(long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, bytes);
  return p;
}
extern "C" void spark_arena_free(void* p) { cudaFree(p); }
extern "C" int spark_ipc_get_handle(void* p, void* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -1;
  memcpy(out64, &h, sizeof(h));
  return 0;
}
extern "C" void* spark_ipc_open_handle(const void* in64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return nullptr;
  return p;
}
extern "C" void spark_ipc_close(void* p) { cudaIpcCloseMemHandle(p); }

struct HostCtx { void* peers[8]; int rank, world; unsigned long long wait_ns; int* status; };
static CommCtx to_ctx(const HostCtx* h) {
  CommCtx c;
  for (int i = 0; i < COMM_MAX_RANKS; ++i) c.peers[i] = static_cast<uint8_t*>(h->peers[i]);
  c.rank = h->rank; c.world = h->world; c.wait_ns = h->wait_ns; c.status = h->status;
  return c;
}

extern "C" int spark_comm_barrier(const HostCtx* h, long long flag_off, unsigned seq, cudaStream_t s) {
  comm_barrier_kernel<<<1, 32, 0, s>>>(to_ctx(h), flag_off, seq);
  return spark_launch_rc(__func__);
}

// Many rows (prefill): two launches.  A CTA that waits for a peer's flag must never keep one of its own
// grid's CTAs from running (the peer's flag needs ALL of that peer's CTAs to have pushed, and vice versa), so
// the push kernel never waits and the tail kernel only waits for flags that push kernels raise.
__global__ void __launch_bounds__(256)
ar_push_kernel(ArRows a_in) {
  ArRows a = a_in;
  a.seq = comm_seq(a.seq_ptr, a.seq);
  a.seq_ptr = nullptr;                                   // the tail kernel closes the sequence
  const int W = a.c.world;
  const size_t set = static_cast<size_t>(a.seq & 1) * W * a.rows_cap * a.N;
  for (int r = blockIdx.x; r < a.R; r += gridDim.x) {
    for (int i = threadIdx.x * 4; i < a.N; i += blockDim.x * 4) {
      const float4 v = ar_local4(a, r, i);
      for (int p = 0; p < W; ++p)
        st_f4(reinterpret_cast<float*>(a.c.peers[p] + a.slot_off) + set + (static_cast<size_t>(a.c.rank) * a.rows_cap + r) * a.N + i, v);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) ar_arrive_and_is_last(a, a.seq, gridDim.x);
}

__global__ void __launch_bounds__(256)
ar_tail_kernel(ArRows a_in, int* tail_counter) {
  __shared__ float red[8];
  pdl_wait();
  pdl_trigger();
  ArRows a = a_in;
  a.seq = comm_seq(a.seq_ptr, a.seq);
  ar_rows_tail(a, a.seq, blockIdx.x, gridDim.x, red);
  __syncthreads();
  if (threadIdx.x == 0 && a.seq_ptr) {                   // last CTA of the tail closes the sequence
    __threadfence();
    if (atomicAdd(tail_counter, 1) == static_cast<int>(gridDim.x) - 1) { *tail_counter = 0; *a.seq_ptr = a.seq; }
  }
}

// CTAs of the one-kernel form that are certainly co-resident on an otherwise idle device (occupancy query).  A CTA
// of that form waits for flags that every rank raises only after ALL of its CTAs have pushed; CTAs of this grid
// that are not resident yet can still start later (no other grid depends on this one), so the wait always ends,
// but the form is only used well below this number so that it normally ends at once.
static int ar_coresident_limit() {
  static int limit = 0;
  if (limit == 0) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_rows_kernel, 256, 0);
    limit = sms * (per_sm > 0 ? per_sm : 1) / 4;
    if (limit < 1) limit = 1;
  }
  return limit;
}

// moe: optional {y, wts, ids, slots, shared, sg} = the local rows are the slot-order combine of a decode MoE (in == null).
struct ArMoe { const float* y; const float* w; const int* ids; int slots; const void* shared; const float* sg; };

extern "C" int spark_allreduce_rows(const HostCtx* h, long long slot_off, long long flag_off, unsigned seq, int rows_cap,
                                    int R, int N, const void* in, int in_f32, int* counter, float* res,
                                    const float* norm_w, float eps, void* out, int out_f32, cudaStream_t s, void* seq_ptr,
                                    const ArMoe* moe, long long ll_off) {
  if (R <= 0) return 0;
  if (N % 4 || R > rows_cap) return -5;
  if ((in == nullptr) == (moe == nullptr)) return -5;
  ArRows a;
  a.c = to_ctx(h); a.slot_off = slot_off; a.flag_off = flag_off; a.seq = seq; a.rows_cap = rows_cap; a.R = R; a.N = N;
  a.in = in; a.in_f32 = in_f32; a.counter = counter; a.res = res; a.norm_w = norm_w; a.eps = eps; a.out = out; a.out_f32 = out_f32; a.seq_ptr = (uint32_t*)seq_ptr;
  a.moe_y = nullptr; a.moe_w = nullptr; a.moe_ids = nullptr; a.moe_slots = 0; a.moe_shared = nullptr; a.moe_sg = nullptr;
  a.ll_off = ll_off;
  if (moe) {
    a.moe_y = moe->y; a.moe_w = moe->w; a.moe_ids = moe->ids; a.moe_slots = moe->slots;
    a.moe_shared = (const __nv_bfloat16*)moe->shared; a.moe_sg = moe->sg;
  }
  if (ll_off >= 0 && R <= AR_LL_ROWS && N <= 8192 && seq_ptr != nullptr && R <= ar_coresident_limit()) {
    const cudaError_t e = spark_launch_pdl(allreduce_rows_ll_kernel<true>, dim3(R), dim3(256), 0, s, dim3(1, 1, 1), a);
    return e == cudaSuccess ? 0 : -4;
  }
  if (R <= 64 && R <= ar_coresident_limit()) {       // one kernel pushes, signals, waits and reduces
    const cudaError_t e = spark_launch_pdl(allreduce_rows_kernel, dim3(R), dim3(256), 0, s, dim3(1, 1, 1), a);
    return e == cudaSuccess ? 0 : -4;
  }
  ar_push_kernel<<<R < 592 ? R : 592, 256, 0, s>>>(a);
  ar_tail_kernel<<<R < 296 ? R : 296, 256, 0, s>>>(a, counter + 1);
  return spark_launch_rc(__func__);
}

// Reduce-scatter by row blocks (+ residual + RMSNorm on the owned rows) then all-gather of the bf16 result into
// every arena at out_off.  M must be world * rows_per_rank.  Three launches; the last only waits.
extern "C" int spark_rs_ag_rows(const HostCtx* h, long long slot_off, long long out_off, long long flag_rs_off,
                                long long flag_ag_off, unsigned seq, int M, int N, int rows_per_rank, const void* in,
                                int in_f32, int* counter, float* res, const float* norm_w, float eps, int push_only,
                                cudaStream_t s, void* seq_ptr) {
  if (M <= 0) return 0;
  if (N % 4 || N > 4096) return -5;
  RsAg a;
  a.c = to_ctx(h); a.slot_off = slot_off; a.out_off = out_off; a.flag_rs_off = flag_rs_off; a.flag_ag_off = flag_ag_off;
  a.seq = seq; a.M = M; a.N = N; a.rows_per_rank = rows_per_rank; a.in = in; a.in_f32 = in_f32; a.counter = counter;
  a.res = res; a.norm_w = norm_w; a.eps = eps; a.seq_ptr = (uint32_t*)seq_ptr;
  if (push_only != 2) {
    int grid = M < 592 ? M : 592;
    rs_push_kernel<<<grid, 256, 0, s>>>(a);
  }
  if (push_only == 1) return spark_launch_rc(__func__);
  int grid2 = rows_per_rank < 592 ? rows_per_rank : 592;
  a.counter = counter + 1;
  rs_finish_ag_push_kernel<<<grid2, 256, 0, s>>>(a);
  wait_flags_kernel<<<1, 32, 0, s>>>(a.c, flag_ag_off, seq, (uint32_t*)seq_ptr, 1);
  return spark_launch_rc(__func__);
}

extern "C" int spark_ag_push(const HostCtx* h, const void* x, int rows, int K, long long buf_off, long long flag_off,
                             unsigned seq, int* counter, cudaStream_t s, const void* seq_ptr) {
  if (rows <= 0) return 0;
  if (K % 8) return -5;
  int grid = rows < 296 ? rows : 296;
  ag_push_kernel<<<grid, 256, 0, s>>>(to_ctx(h), (const __nv_bfloat16*)x, rows, K, buf_off, flag_off, seq, counter, (const uint32_t*)seq_ptr);
  return spark_launch_rc(__func__);
}

extern "C" int spark_seq_bump(void* seq_ptr, cudaStream_t s) {
  seq_bump_kernel<<<1, 1, 0, s>>>((uint32_t*)seq_ptr);
  return spark_launch_rc(__func__);
}
extern "C" int spark_wait_flags(const HostCtx* h, long long flag_off, unsigned seq, cudaStream_t s) {
  wait_flags_kernel<<<1, 32, 0, s>>>(to_ctx(h), flag_off, seq, nullptr, 0);
  return spark_launch_rc(__func__);
}

// Wait on a flag region using the device-side sequence counter (value + 1); bump != 0 stores it back.
extern "C" int spark_wait_flags_dev(const HostCtx* h, long long flag_off, void* seq_ptr, int bump, cudaStream_t s) {
  wait_flags_kernel<<<1, 32, 0, s>>>(to_ctx(h), flag_off, 0, (uint32_t*)seq_ptr, bump);
  return spark_launch_rc(__func__);
}

// Vocabulary-parallel greedy sampling: logits fp32 [R, V_local] -> out_id [R] (global ids, identical on all ranks).
// part_v / part_i: scratch of R * 64 entries each; seq_ptr: device sequence counter of this channel.
extern "C" int spark_tp_argmax(const HostCtx* h, long long slot_off, long long flag_off, void* seq_ptr, int* counter,
                               int rows_cap, const float* logits, int R, int V, int vocab_off, float* part_v, int* part_i,
                               int* out_id, cudaStream_t s) {
  if (R <= 0) return 0;
  if (R > rows_cap || R > 64 || seq_ptr == nullptr) return -5;
  const int nc = V >= 16384 ? 64 : (V >= 2048 ? 8 : 1);
  cudaError_t e = spark_launch_pdl(tp_argmax_part_kernel, dim3(R, nc), dim3(256), 0, s, dim3(1, 1, 1), logits, V, part_v, part_i);
  if (e != cudaSuccess) return -4;
  PkArgs a;
  a.c = to_ctx(h); a.slot_off = slot_off; a.flag_off = flag_off; a.seq_ptr = (uint32_t*)seq_ptr; a.counter = counter;
  a.rows_cap = rows_cap; a.vocab_off = vocab_off;
  e = spark_launch_pdl(tp_argmax_packets_kernel, dim3(R), dim3(32), 0, s, dim3(1, 1, 1), a, (const float*)part_v, (const int*)part_i, nc, out_id);
  return e == cudaSuccess ? 0 : -4;
}

// Second half of an all-reduce whose pushes were made by another kernel's epilogue (the row-parallel EXL3 GEMV):
// one CTA per row waits (bounded) for every rank's flag, sums in rank order (+ residual)(+ RMSNorm), and the last CTA
// closes the sequence.  `counter` + 1 is the tail's own arrival counter.
extern "C" int spark_allreduce_tail(const HostCtx* h, long long slot_off, long long flag_off, int rows_cap, int R, int N,
                                    int* counter, float* res, const float* norm_w, float eps, void* out, int out_f32,
                                    cudaStream_t s, void* seq_ptr, long long ll_off) {
  if (R <= 0) return 0;
  if (N % 4 || R > rows_cap || seq_ptr == nullptr) return -5;
  ArRows a;
  a.c = to_ctx(h); a.slot_off = slot_off; a.flag_off = flag_off; a.seq = 0; a.rows_cap = rows_cap; a.R = R; a.N = N;
  a.in = nullptr; a.in_f32 = 0; a.counter = counter; a.res = res; a.norm_w = norm_w; a.eps = eps; a.out = out; a.out_f32 = out_f32;
  a.seq_ptr = (uint32_t*)seq_ptr;
  a.moe_y = nullptr; a.moe_w = nullptr; a.moe_ids = nullptr; a.moe_slots = 0; a.moe_shared = nullptr; a.moe_sg = nullptr;
  a.ll_off = ll_off;
  if (ll_off >= 0 && R <= AR_LL_ROWS && N <= 8192) {       // the pushing kernel used the low-latency wire format too
    const cudaError_t e = spark_launch_pdl(allreduce_rows_ll_kernel<false>, dim3(R), dim3(256), 0, s, dim3(1, 1, 1), a);
    return e == cudaSuccess ? 0 : -4;
  }
  const cudaError_t e = spark_launch_pdl(ar_tail_kernel, dim3(R < 296 ? R : 296), dim3(256), 0, s, dim3(1, 1, 1), a, counter + 1);
  return e == cudaSuccess ? 0 : -4;
}
