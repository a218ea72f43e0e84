// Persistent warp-specialised tcgen05 GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  (bf16 in, fp32
// accumulate in TMEM).  One CTA per SM; warp 0 = TMA producer, warp 1 = MMA issuer (one elected
// thread issues tcgen05.mma), warps 2..5 = epilogue (tcgen05.ld from TMEM, 32 lanes each).
// A and B tiles arrive by TMA (128-byte swizzle, K-major) into a multi-stage ring guarded by
// mbarriers; two TMEM accumulator stages let the epilogue of tile i overlap the mainloop of tile i+1.
//
// The mainloop is shared by every GEMM-shaped op of the engine; the epilogue is a functor:
// plain store, SwiGLU over a [gate | up] tile pair, slot-weighted MoE scatter, and the fused
// row-parallel epilogue that pushes partial tiles to peer GPUs.  `GROUPED` reads a tile list
// (ragged row ranges per expert) instead of a regular M x N grid.
//
// Replaces the reference's cuBLAS/ATen prefill GEMMs (engine-rs/shim/shim.cpp:253-288,1028-1106) and
// its mma.sync grouped GEMMs (engine-rs/shim/moe_exl3.cuh:521-1233); none of those has a tcgen05 path.
#pragma once
#include "../common/comm.cuh"

namespace spark {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_ACC_STAGES = 2;

struct GemmArgs {
  int M, N, K;                 // logical problem (GROUPED: M = total permuted rows, N = per-expert N)
  int num_n_tiles;             // tiles along N (of BN, or BN/2 outputs in gate-up mode)
  int num_tiles;               // total tiles
  const int4* tile_list;       // GROUPED: per m-tile {a_row0, row_end, expert, 0}
  const int* tile_count;       // GROUPED: device-side number of m-tiles (nullable -> num_tiles fixed)
  int b_rows_per_expert;       // GROUPED: rows of B per expert
  int ab_fmt;                  // operand format of A and B: 1 = bf16, 0 = fp16
  int gate_up_F;               // > 0: B rows [f0, f0+BN/2) and [F+f0, ...) form one tile (SwiGLU epilogue)
  int* status;
  // all-gather fused into the A operand: rows [src*ag_rows, (src+1)*ag_rows) of A were pushed into the local
  // arena by rank src; the TMA producer waits (bounded) for flag[src] >= ag_seq before the first tile of
  // that block and visits its own block first.  ag_flags == nullptr: plain GEMM.
  const uint32_t* ag_flags; uint32_t ag_seq; int ag_rows, ag_rank, ag_world; unsigned long long ag_wait_ns;
  const uint32_t* ag_seq_ptr;
};

struct TileCoord {
  int a_row0, row_end, b_row_a, b_row_b, out_col0, expert;
};

template <int BN, bool GROUPED>
__device__ __forceinline__ TileCoord tile_coord(const GemmArgs& g, int t) {
  TileCoord c;
  int mt = t / g.num_n_tiles, nt = t % g.num_n_tiles;
  int b_base = 0;
  if (GROUPED) {
    int4 e = g.tile_list[mt];
    c.a_row0 = e.x; c.row_end = e.y; c.expert = e.z;
    b_base = e.z * g.b_rows_per_expert;
  } else {
    if (g.ag_flags != nullptr) {          // rotate the m-tiles so that this rank's own row block comes first
      const int num_m = g.num_tiles / g.num_n_tiles;
      const int per = (g.ag_rows + GEMM_BM - 1) / GEMM_BM;
      mt = (mt + g.ag_rank * per) % num_m;
    }
    c.a_row0 = mt * GEMM_BM; c.row_end = g.M; c.expert = 0;
  }
  if (g.gate_up_F > 0) {
    int f0 = nt * (BN / 2);
    c.b_row_a = b_base + f0;
    c.b_row_b = b_base + g.gate_up_F + f0;
    c.out_col0 = f0;
  } else {
    c.b_row_a = b_base + nt * BN;
    c.b_row_b = c.b_row_a + 128;
    c.out_col0 = nt * BN;
  }
  return c;
}

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BAR_BYTES = 256;
  static constexpr int XPOSE_BYTES = 4 * 32 * 33 * 4;                     // per-epilogue-warp transpose tile (coalesced pushes)
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + XPOSE_BYTES + 1024;   // + alignment slack
};

// Epilogue functor contract:
//   __device__ void operator()(const TileCoord& tc, int row, int col, const float (&v)[32]) const
// `row` is a valid global row (< tc.row_end), `col` the first of 32 consecutive output columns
// (col + 32 may exceed N: the functor guards).  In gate-up mode `v` already holds silu(g)*u.
template <int BN, class Epi, bool GROUPED>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    GemmArgs g, Epi epi) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  constexpr int TMEM_COLS = GEMM_ACC_STAGES * BN;       // 256 or 512 (power of two)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + GEMM_ACC_STAGES;
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + GEMM_ACC_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = (g.K + GEMM_BK - 1) / GEMM_BK;
  int num_tiles = g.num_tiles;
  if (GROUPED && g.tile_count != nullptr) num_tiles = (*g.tile_count) * g.num_n_tiles;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < GEMM_ACC_STAGES; ++s) { mbar_init(&tmem_full[s], 1); mbar_init(&tmem_empty[s], 4); }
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc<TMEM_COLS>(tmem_base_ptr); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      uint32_t ag_seen = 0;                 // bit src set: rank src's block has arrived
      const uint32_t ag_seq = comm_seq(g.ag_seq_ptr, g.ag_seq);
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        TileCoord tc = tile_coord<BN, GROUPED>(g, t);
        if (!GROUPED && g.ag_flags != nullptr) {
          // a 128-row tile may straddle two source blocks when ag_rows % 128 != 0: wait for both
          const int s0 = tc.a_row0 / g.ag_rows, s1 = min(g.ag_world - 1, (tc.a_row0 + GEMM_BM - 1) / g.ag_rows);
          for (int src = s0; src <= s1 && ok; ++src) {
            if (src == g.ag_rank || (ag_seen >> src) & 1u) continue;
            CommCtx cc; cc.wait_ns = g.ag_wait_ns; cc.status = g.status;
            if (!wait_flag(cc, g.ag_flags + src, ag_seq, src)) { ok = false; break; }
            ag_seen |= 1u << src;
            asm volatile("fence.proxy.async;" ::: "memory");   // peer's generic-proxy stores -> our TMA reads
          }
          if (!ok) break;
        }
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            set_status(g.status, ST_TIMEOUT_MBAR_EMPTY, blockIdx.x, t, kb); ok = false; break;
          }
          uint8_t* a_dst = smem + stage * S::STAGE_BYTES;
          uint8_t* b_dst = a_dst + S::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full_bar[stage], kb * GEMM_BK, tc.a_row0);
          tma_load_2d(b_dst, &tmB, &full_bar[stage], kb * GEMM_BK, tc.b_row_a);
          if (BN == 256) tma_load_2d(b_dst + 128 * GEMM_BK * 2, &tmB, &full_bar[stage], kb * GEMM_BK, tc.b_row_b);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(g.ab_fmt, g.ab_fmt, GEMM_BM, BN);   // 16-bit x 16-bit -> f32
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          set_status(g.status, ST_TIMEOUT_TMEM_EMPTY, blockIdx.x, t, acc); break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            set_status(g.status, ST_TIMEOUT_MBAR_FULL, blockIdx.x, t, kb); ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint64_t a_desc = make_smem_desc_sw128(a_addr);
          const uint64_t b_desc = make_smem_desc_sw128(a_addr + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // 16 bf16 = 32 bytes along K inside the swizzled row: +2 in the encoded address
            umma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);          // frees the smem stage when these MMAs finish
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full[acc]);              // accumulator complete
        if (++acc == GEMM_ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, 128 TMEM lanes)
    const int quarter = warp & 3;                  // TMEM lanes [32*quarter, +32) belong to this warp
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      TileCoord tc = tile_coord<BN, GROUPED>(g, t);
      // warp-uniform result: tcgen05.ld below needs the whole warp
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase))) {
        set_status(g.status, ST_TIMEOUT_TMEM_FULL, blockIdx.x, t, acc); break;
      }
      tc_fence_after();
      const int row = tc.a_row0 + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (g.gate_up_F > 0) {
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(t_addr + c, rg);
          tmem_ld_32x32(t_addr + BN / 2 + c, ru);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = epi.act(__uint_as_float(rg[i]), __uint_as_float(ru[i]));
          if (row < tc.row_end) epi(tc, row, tc.out_col0 + c, v);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + c, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if constexpr (Epi::kWarpTile) {
            // remote stores want whole 128-byte lines: transpose the warp's 32 x 32 block through shared memory so
            // that the 32 lanes write 32 consecutive floats of one row per instruction
            float* xp = reinterpret_cast<float*>(smem + STAGES * S::STAGE_BYTES + S::BAR_BYTES) + quarter * 32 * 33;
#pragma unroll
            for (int i = 0; i < 32; ++i) xp[lane * 33 + i] = v[i];
            __syncwarp();
            epi.warp_tile(tc, tc.a_row0 + quarter * 32, tc.out_col0 + c, xp, lane);
            __syncwarp();
          } else {
            if (row < tc.row_end) epi(tc, row, tc.out_col0 + c, v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == GEMM_ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }
  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<TMEM_COLS>(tmem_base); }
  if (threadIdx.x == 0) epi.cta_done(gridDim.x);
}

// ---------------------------------------------------------------- epilogues
struct EpiStoreBf16 {
  static constexpr bool kWarpTile = false;
  __nv_bfloat16* C; int ldc; int N;
  __device__ __forceinline__ void cta_done(int) const {}
  __device__ __forceinline__ float act(float g, float u) const { return g; }
  __device__ __forceinline__ void operator()(const TileCoord&, int row, int col, const float (&v)[32]) const {
    __nv_bfloat16* dst = C + static_cast<size_t>(row) * ldc + col;
    if (col + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 o;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[i], v[i + 1]), p1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), p3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
        o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
        o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
        *reinterpret_cast<uint4*>(dst + i) = o;
      }
    } else {
      for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = __float2bfloat16(v[i]);
    }
  }
};

struct EpiStoreF32 {
  static constexpr bool kWarpTile = false;
  float* C; int ldc; int N;
  __device__ __forceinline__ void cta_done(int) const {}
  __device__ __forceinline__ float act(float g, float u) const { return g; }
  __device__ __forceinline__ void operator()(const TileCoord&, int row, int col, const float (&v)[32]) const {
    float* dst = C + static_cast<size_t>(row) * ldc + col;
    if (col + 32 <= N && (ldc & 3) == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
      for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = v[i];
    }
  }
};

// SwiGLU (optionally clamped) over a [gate | up] tile pair -> bf16 [rows, F].
struct EpiSwigluBf16 {
  static constexpr bool kWarpTile = false;
  __nv_bfloat16* C; int ldc; int N; float limit;
  __device__ __forceinline__ void cta_done(int) const {}
  __device__ __forceinline__ float act(float g, float u) const {
    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    return g / (1.f + __expf(-g)) * u;
  }
  __device__ __forceinline__ void operator()(const TileCoord& tc, int row, int col, const float (&v)[32]) const {
    EpiStoreBf16 st{C, ldc, N};
    st(tc, row, col, v);
  }
};

// Row-parallel GEMM under tensor parallelism: the fp32 partial tile goes straight to the rank that owns the
// row block (reduce-scatter by rows over NVLink, plain P2P stores from the epilogue warps); the CTA that
// finishes last on this rank raises the "my partials are delivered" flag on every owner.  The owners then
// sum the slots in rank order (+ residual + RMSNorm) and all-gather the result (comm.cu rs_finish_ag_push).
struct EpiPushRS {
  static constexpr bool kWarpTile = true;
  uint8_t* peers[COMM_MAX_RANKS];
  long long slot_off, flag_off;        // float slots [world(src)][rows_per_rank * N] on the owner; u32 flags [world]
  int rank, world, rows_per_rank, N;
  uint32_t seq;
  int* counter;
  const uint32_t* seq_ptr;
  __device__ __forceinline__ float act(float g, float u) const { return g; }
  __device__ __forceinline__ void operator()(const TileCoord&, int row, int col, const float (&v)[32]) const {
    const int owner = row / rows_per_rank, lr = row - owner * rows_per_rank;
    float* dst = reinterpret_cast<float*>(peers[owner] + slot_off) + (static_cast<size_t>(rank) * rows_per_rank + lr) * N + col;
    if (col + 32 <= N) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
      for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = v[i];
    }
  }
  // xp: the warp's 32 x 32 block, row-major with stride 33; rows row0..row0+31, columns col..col+31
  __device__ __forceinline__ void warp_tile(const TileCoord& tc, int row0, int col, const float* xp, int lane) const {
    if (col + lane >= N) return;
#pragma unroll 4
    for (int r = 0; r < 32; ++r) {
      const int row = row0 + r;
      if (row >= tc.row_end) break;
      const int owner = row / rows_per_rank, lr = row - owner * rows_per_rank;
      float* dst = reinterpret_cast<float*>(peers[owner] + slot_off) + (static_cast<size_t>(rank) * rows_per_rank + lr) * N + col;
      dst[lane] = xp[r * 33 + lane];
    }
  }
  __device__ __forceinline__ void cta_done(int n_ctas) const {
    __threadfence_system();
    if (atomicAdd(counter, 1) == n_ctas - 1) {
      *counter = 0;
      const uint32_t sq = comm_seq(seq_ptr, seq);
      for (int p = 0; p < world; ++p) st_relaxed_sys(reinterpret_cast<uint32_t*>(peers[p] + flag_off) + rank, sq);
    }
  }
};

// Grouped down-projection: rows are (token, slot) pairs in expert order; write fp32 partial rows
// that the combine kernel sums in slot order (deterministic).
using EpiGroupedF32 = EpiStoreF32;

}  // namespace spark
