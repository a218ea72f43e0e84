// Block-scaled FP8 GEMM on tcgen05:  C[M,N] = (A . sfa)[M,K] (B . sfb)[N,K]^T with e4m3 operands and one E8M0 scale per
// 32 elements along K for every row of A and of B (MXFP8), accumulated in fp32 in TMEM.  The scales are applied by the
// tensor core itself (`tcgen05.mma.kind::mxf8f6f4.block_scale`): no dequantised copy of the weights ever exists.
//
// Same skeleton as the bf16 GEMM (persistent CTAs, warp 0 = TMA producer, warp 1 = one-thread MMA issuer, warps 2..5 =
// epilogue, 128-byte-swizzled K-major tiles, two TMEM accumulator stages), plus the scale-factor path:
//   * scales live in global memory in the layout the tensor core wants, one 512-byte block per (128 rows, 128 k):
//     byte (row % 32) * 16 + (row / 32) * 4 + (k / 32) % 4  (act_quant / weight preparation write this directly);
//   * the producer fetches the block of A and of B with a bulk copy onto the stage's full barrier;
//   * the MMA thread copies both blocks to tensor memory (`tcgen05.cp.32x128b.warpx4`: 32 rows x 16 bytes, replicated
//     to the four lane quadrants) and issues four K=32 MMAs per stage whose descriptors select scale byte 0..3.
// Tile 128 x 128 x 128 bytes of K; TMEM: 2 x 128 accumulator columns + 8 scale columns per stage.
// Every wait is bounded (status word + normal teardown).  Reference paths replaced: engine-rs/shim/ds41_mx.cu
// fp8_gemm_mx* (warp-level block-scaled mma.sync), fp8.cu / fp8pf.cu (wmma + scale promotion).
#include "../common/ptx.cuh"
#include <cstdlib>
#include <mutex>

namespace spark {

constexpr int MX_BM = 128, MX_BN = 128, MX_BK = 128;       // BK in elements = bytes (fp8)
constexpr int MX_STAGES = 5;
constexpr int MX_ACC_STAGES = 2;
constexpr int MX_THREADS = 192;
constexpr int MX4_THREADS = 224;       // grouped MXFP4 kernel: + one warp that fetches the scale blocks
constexpr int MX_A_BYTES = MX_BM * MX_BK, MX_B_BYTES = MX_BN * MX_BK, MX_SF_BYTES = 512;
constexpr int MX_STAGE_BYTES = MX_A_BYTES + MX_B_BYTES + 2 * MX_SF_BYTES;
constexpr int MX_SMEM = MX_STAGES * MX_STAGE_BYTES + 256 + 1024;
constexpr int MX_TMEM_COLS = 512;                           // 256 accumulator + 40 scale columns, power of two
constexpr int MX_SF_COL0 = MX_ACC_STAGES * MX_BN;

struct MxGemmArgs {
  int M, N, K;
  const uint8_t* sfa; const uint8_t* sfb;     // [ceil(M/128)][K/128][512], [ceil(N/128)][K/128][512]
  void* C; int ldc; int out_f32;
  int* status;
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 consecutive 32-bit TMEM columns, replicated over the 4 lane quadrants
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// un-swizzled K-major descriptor of a 32 x 16-byte block: 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(16 >> 4) << 16;        // leading byte offset (one 16-byte column only)
  d |= static_cast<uint64_t>(128 >> 4) << 32;       // stride byte offset between 8-row groups
  d |= 1ull << 46;                                  // descriptor version of this architecture
  return d;
}
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t tsfa,
                                          uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb) : "memory");
}
// block-scaled instruction descriptor: [4,6) B scale byte, [7,10) A format, [10,13) B format (0 = e4m3), [17,23) N>>3,
// bit 23 scale format (1 = E8M0), [24,29) M>>4, [29,31) A scale byte, bit 31 K size (0 = 32 for 8-bit operands)
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t M, uint32_t N) {
  return ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24);
}

__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, MxGemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + MX_STAGES * MX_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + MX_STAGES;
  uint64_t* tmem_full = empty_bar + MX_STAGES;
  uint64_t* tmem_empty = tmem_full + MX_ACC_STAGES;
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + MX_ACC_STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = g.K / MX_BK;
  const int mt_n = (g.M + MX_BM - 1) / MX_BM, nt_n = (g.N + MX_BN - 1) / MX_BN;
  const int num_tiles = mt_n * nt_n;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < MX_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < MX_ACC_STAGES; ++s) { mbar_init(&tmem_full[s], 1); mbar_init(&tmem_empty[s], 4); }
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc<MX_TMEM_COLS>(tmem_base_ptr); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int mt = t / nt_n, nt = t % nt_n;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            set_status(g.status, ST_TIMEOUT_MBAR_EMPTY, blockIdx.x, t, kb); ok = false; break;
          }
          uint8_t* a_dst = smem + stage * MX_STAGE_BYTES;
          uint8_t* b_dst = a_dst + MX_A_BYTES;
          uint8_t* sfa_dst = b_dst + MX_B_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], MX_STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full_bar[stage], kb * MX_BK, mt * MX_BM);
          tma_load_2d(b_dst, &tmB, &full_bar[stage], kb * MX_BK, nt * MX_BN);
          bulk_load(sfa_dst, g.sfa + (static_cast<size_t>(mt) * num_k + kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[stage]);
          bulk_load(sfa_dst + MX_SF_BYTES, g.sfb + (static_cast<size_t>(nt) * num_k + kb) * MX_SF_BYTES, MX_SF_BYTES,
                    &full_bar[stage]);
          if (++stage == MX_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc0 = make_idesc_mx(MX_BM, MX_BN);
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          set_status(g.status, ST_TIMEOUT_TMEM_EMPTY, blockIdx.x, t, acc); break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * MX_BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            set_status(g.status, ST_TIMEOUT_MBAR_FULL, blockIdx.x, t, kb); ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * MX_STAGE_BYTES);
          const uint64_t a_desc = make_smem_desc_sw128(a_addr);
          const uint64_t b_desc = make_smem_desc_sw128(a_addr + MX_A_BYTES);
          const uint32_t tsfa = tmem_base + MX_SF_COL0 + stage * 8, tsfb = tsfa + 4;
          tmem_cp_32x128b_x4(tsfa, make_sf_desc(a_addr + MX_A_BYTES + MX_B_BYTES));
          tmem_cp_32x128b_x4(tsfb, make_sf_desc(a_addr + MX_A_BYTES + MX_B_BYTES + MX_SF_BYTES));
#pragma unroll
          for (int k = 0; k < MX_BK / 32; ++k) {
            // 32 fp8 = 32 bytes along K inside the swizzled row: +2 in the encoded address; scale byte k of the block
            const uint32_t idesc = idesc0 | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29);
            umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, tsfa, tsfb, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == MX_STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full[acc]);
        if (++acc == MX_ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int mt = t / nt_n, nt = t % nt_n;
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase))) {
        set_status(g.status, ST_TIMEOUT_TMEM_FULL, blockIdx.x, t, acc); break;
      }
      tc_fence_after();
      const int row = mt * MX_BM + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + acc * MX_BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < MX_BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c, r);
        tmem_ld_wait();
        const int col = nt * MX_BN + c;
        if (row < g.M) {
          if (g.out_f32) {
            float* dst = reinterpret_cast<float*>(g.C) + static_cast<size_t>(row) * g.ldc + col;
            for (int i = 0; i < 32 && col + i < g.N; ++i) dst[i] = __uint_as_float(r[i]);
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C) + static_cast<size_t>(row) * g.ldc + col;
            if (col + 32 <= g.N && (g.ldc & 7) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 o;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + i) = o;
              }
            } else {
              for (int i = 0; i < 32 && col + i < g.N; ++i) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == MX_ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<MX_TMEM_COLS>(tmem_base); }
}

// ------------------------------------------------------------------------------------------------------------------
// Grouped MoE GEMM with MXFP4 expert weights: for every work item (a run of <= 128 activation rows routed to one
// expert) and every 128-column tile of that expert, C[rows, cols] = (A . sfa)(W_e . sfw)^T with A in MXFP8 (e4m3 + one
// E8M0 per 32 k) and W_e in MXFP4 (e2m1 + one E8M0 per 32 k).  The packed nibbles go from global memory to the tensor
// core untouched: the tensor map type 16U4_ALIGN16B makes TMA expand 16 nibbles (8 bytes) into the 16-byte padded
// slots that `tcgen05.mma.kind::mxf8f6f4` reads for a 4-bit operand, so a 128-k slice of a weight row is 128 bytes of
// shared memory exactly like an fp8 row, and the descriptors of the fp8 kernel apply unchanged (B format = e2m1).
// Items with <= 16 rows (decode: one row per (token, expert) pair) fetch a 16-row activation box instead of 128 rows;
// the other rows of the tile are whatever shared memory held, which only reaches accumulator rows that are never
// stored.  The A scale blocks are tile-local (row r of the item, not of the matrix): mx_sf_tile_blocks_kernel.
// Reference paths replaced: engine-rs/shim/ds41_mx.cu (mxfp4 expert GEMMs through dequantised tiles).
struct Mx4Args {
  const int4* items;          // (first A row, rows, expert, first C row)
  const int* n_items;         // device count (<= max_items)
  int max_items;
  int N, K;                   // per expert
  const uint8_t* sfa;         // [max_items][K/128][512]
  const uint8_t* sfw;         // [E * N/128][K/128][512]
  void* C; int ldc; int out_f32;
  int* status;
  uint32_t w_tx_bytes;        // bytes one weight tile adds to the stage barrier's transaction count (packed size)
  int burst;                  // k-blocks whose tile loads are issued together (1 .. stages / 2)
};

// SMALL: every item has <= 16 rows (decode pairs).  The operands are swapped: the weight tile is the 128-row M
// operand, the 16-row activation box the N operand, so the accumulator is [128 weight rows, 16 activation rows] and
// the tensor pipe does an eighth of the work per weight byte.  A stage is 19 KB (2 KB activations, 16 KB weights,
// two scale blocks) and ten stages fit.
template <bool SMALL>
struct Mx4Cfg {
  static constexpr int STAGES = SMALL ? 10 : MX_STAGES;
  static constexpr int A_REGION = SMALL ? 16 * MX_BK : MX_A_BYTES;
  static constexpr int B_OFF = STAGES * A_REGION;
  static constexpr int SF_OFF = B_OFF + STAGES * MX_B_BYTES;
  static constexpr int BAR_OFF = SF_OFF + STAGES * 2 * MX_SF_BYTES;
  static constexpr int SMEM = BAR_OFF + 256 + 1024;
};

template <bool SMALL>
__global__ void __launch_bounds__(MX4_THREADS, 1)
moe_mxfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA16,
                 const __grid_constant__ CUtensorMap tmW, Mx4Args g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using Cfg = Mx4Cfg<SMALL>;
  constexpr int STAGES = Cfg::STAGES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + MX_ACC_STAGES;
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + MX_ACC_STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = g.K / MX_BK;
  const int nt_n = g.N / MX_BN;
  const int n_items = min(*g.n_items, g.max_items);
  const int num_tiles = n_items * nt_n;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmA16);
    tma_prefetch_desc(&tmW);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 2); mbar_init(&empty_bar[s], 1); }    // two producers
    for (int s = 0; s < MX_ACC_STAGES; ++s) { mbar_init(&tmem_full[s], 1); mbar_init(&tmem_empty[s], 4); }
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc<MX_TMEM_COLS>(tmem_base_ptr); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int it = t / nt_n, nt = t - it * nt_n;
        const int4 item = g.items[it];
        if (item.z < 0 || item.y <= 0) continue;                 // expert of another rank / empty item
        if (SMALL && item.y > 16) { set_status(g.status, ST_BOUNDS, blockIdx.x, t, item.y); break; }
        const bool small = SMALL || item.y <= 16;
        const uint32_t a_bytes = small ? 16 * MX_BK : MX_A_BYTES;
        // the tile loads can go out in bursts of `burst` k-blocks (adjacent 64-byte row pieces requested together);
        // measured neutral on B200, so the default is 1
        for (int kb0 = 0; kb0 < num_k && ok; kb0 += g.burst) {
          const int nb = min(g.burst, num_k - kb0);
          int st = stage; uint32_t ph = phase;
          for (int j = 0; j < nb; ++j) {
            if (!mbar_wait(&empty_bar[st], ph ^ 1)) {
              set_status(g.status, ST_TIMEOUT_MBAR_EMPTY, blockIdx.x, t, kb0 + j); ok = false; break;
            }
            if (++st == STAGES) { st = 0; ph ^= 1; }
          }
          if (!ok) break;
          for (int j = 0; j < nb; ++j) {
            const int kb = kb0 + j;
            uint8_t* a_dst = smem + stage * Cfg::A_REGION;
            uint8_t* b_dst = smem + Cfg::B_OFF + stage * MX_B_BYTES;
            mbar_arrive_expect_tx(&full_bar[stage], a_bytes + g.w_tx_bytes);
            tma_load_2d(a_dst, small ? &tmA16 : &tmA, &full_bar[stage], kb * MX_BK, item.x);
            tma_load_2d(b_dst, &tmW, &full_bar[stage], kb * MX_BK, item.z * g.N + nt * MX_BN);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 6) {
    // second producer: the two scale blocks of every stage, so that the tile loads and the scale copies are issued
    // by different threads
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int it = t / nt_n, nt = t - it * nt_n;
        const int4 item = g.items[it];
        if (item.z < 0 || item.y <= 0) continue;
        if (SMALL && item.y > 16) break;
        const uint8_t* sa = g.sfa + static_cast<size_t>(it) * num_k * MX_SF_BYTES;
        const uint8_t* sw = g.sfw + static_cast<size_t>(item.z * nt_n + nt) * num_k * MX_SF_BYTES;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            set_status(g.status, ST_TIMEOUT_MBAR_EMPTY, blockIdx.x, t, -kb - 1); ok = false; break;
          }
          uint8_t* sf_dst = smem + Cfg::SF_OFF + stage * 2 * MX_SF_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], 2 * MX_SF_BYTES);
          bulk_load(sf_dst, sa + static_cast<size_t>(kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[stage]);
          bulk_load(sf_dst + MX_SF_BYTES, sw + static_cast<size_t>(kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // 128-row tiles: D[activation rows, weight rows], weights are operand B (format e2m1 in bits [10,13)).
      // SMALL: operands swapped, D[weight rows, 16 activation rows]: the MMA is 128 x 16 x 32 instead of
      // 128 x 128 x 32, an eighth of the tensor-pipe time per weight byte, which is what lets the decode shape run at
      // memory speed (with the 128-wide form the tensor pipe, padded 1 row -> 128, was the limit at 0.4 us per stage).
      const uint32_t idesc0 = SMALL ? (make_idesc_mx(MX_BN, 16) | (5u << 7)) : (make_idesc_mx(MX_BM, MX_BN) | (5u << 10));
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int4 item = g.items[t / nt_n];
        if (item.z < 0 || item.y <= 0) continue;
        if (SMALL && item.y > 16) break;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          set_status(g.status, ST_TIMEOUT_TMEM_EMPTY, blockIdx.x, t, acc); break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * MX_BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            set_status(g.status, ST_TIMEOUT_MBAR_FULL, blockIdx.x, t, kb); ok = false; break;
          }
          tc_fence_after();
          const uint32_t s0 = smem_u32(smem);
          const uint64_t x_desc = make_smem_desc_sw128(s0 + stage * Cfg::A_REGION);            // activations
          const uint64_t w_desc = make_smem_desc_sw128(s0 + Cfg::B_OFF + stage * MX_B_BYTES);  // weights
          const uint64_t a_desc = SMALL ? w_desc : x_desc, b_desc = SMALL ? x_desc : w_desc;
          const uint32_t sf_addr = s0 + Cfg::SF_OFF + stage * 2 * MX_SF_BYTES;                 // [activations | weights]
          const uint32_t tsfa = tmem_base + MX_SF_COL0 + stage * 8, tsfb = tsfa + 4;
          tmem_cp_32x128b_x4(tsfa, make_sf_desc(sf_addr + (SMALL ? MX_SF_BYTES : 0)));
          tmem_cp_32x128b_x4(tsfb, make_sf_desc(sf_addr + (SMALL ? 0 : MX_SF_BYTES)));
#pragma unroll
          for (int k = 0; k < MX_BK / 32; ++k) {
            const uint32_t idesc = idesc0 | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29);
            umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, tsfa, tsfb, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        if (++acc == MX_ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int it = t / nt_n, nt = t - it * nt_n;
      const int4 item = g.items[it];
      if (item.z < 0 || item.y <= 0) continue;
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_phase))) {
        set_status(g.status, ST_TIMEOUT_TMEM_FULL, blockIdx.x, t, acc); break;
      }
      tc_fence_after();
      const int r = quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + acc * MX_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (SMALL) {
        // lane = weight row (output column), TMEM column j = activation row j of the item
        uint32_t v[32];
        tmem_ld_32x32(t_addr, v);
        tmem_ld_wait();
        const int col = nt * MX_BN + r;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j < item.y) {
            const size_t o = (static_cast<size_t>(item.w) + j) * g.ldc + col;
            if (g.out_f32) reinterpret_cast<float*>(g.C)[o] = __uint_as_float(v[j]);
            else reinterpret_cast<__nv_bfloat16*>(g.C)[o] = __float2bfloat16(__uint_as_float(v[j]));
          }
        }
      } else
      // a warp whose 32 rows all lie past the item's rows has nothing to read
      if (quarter * 32 < item.y) {
#pragma unroll 1
        for (int c = 0; c < MX_BN; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(t_addr + c, v);
          tmem_ld_wait();
          const int col = nt * MX_BN + c;
          if (r < item.y) {
            const size_t row = static_cast<size_t>(item.w) + r;
            if (g.out_f32) {
              float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(g.C) + row * g.ldc + col);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]),
                                     __uint_as_float(v[4 * i + 3]));
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C) + row * g.ldc + col;
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 o;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + i) = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == MX_ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<MX_TMEM_COLS>(tmem_base); }
}

// Work items of the grouped kernel.  mode 0: from the expert-sorted tile list (first row, end row, expert): one item
// per tile, C rows = A rows.  mode 1: one item per (token, expert) pair: A row = pair_row[p] (or p), C row = p.
__global__ void mx4_items_kernel(int mode, const int4* __restrict__ tiles, const int* __restrict__ ntile,
                                 const int* __restrict__ pair_expert, const int* __restrict__ pair_row, int pairs,
                                 int max_items, int4* __restrict__ items, int* __restrict__ n_items) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = mode == 0 ? min(*ntile, max_items) : min(pairs, max_items);
  if (i == 0) *n_items = n;
  if (i >= max_items) return;
  int4 it = make_int4(0, 0, -1, 0);
  if (i < n) {
    if (mode == 0) {
      const int4 td = tiles[i];
      it = make_int4(td.x, min(128, td.y - td.x), td.z, td.x);
    } else {
      it = make_int4(pair_row ? pair_row[i] : i, 1, pair_expert[i], i);
    }
  }
  items[i] = it;
}

// Activation scale bytes [R, K/32] (row-major) -> item-local blocks [max_items][K/128][512]: byte
// (r % 32) * 16 + (r / 32) * 4 + k32 % 4 of block (item, k128) is the scale of row item.x + r; rows past the item's
// end read exponent 0.
__global__ void mx_sf_tile_blocks_kernel(const uint8_t* __restrict__ sf, const int4* __restrict__ items,
                                         const int* __restrict__ n_items, int max_items, int kblocks32,
                                         uint8_t* __restrict__ out) {
  const int kb128 = kblocks32 >> 2;
  const int it = blockIdx.x;
  if (it >= min(*n_items, max_items)) return;
  const int4 item = items[it];
  for (int i = threadIdx.x; i < kb128 * 512; i += blockDim.x) {
    const int kt = i >> 9, within = i & 511;
    const int r32 = within >> 4, q = (within >> 2) & 3, kk = within & 3;
    const int r = q * 32 + r32;
    uint8_t v = 0;
    if (item.z >= 0 && r < item.y) v = sf[static_cast<size_t>(item.x + r) * kblocks32 + kt * 4 + kk];
    out[(static_cast<size_t>(it) * kb128 + kt) * 512 + within] = v;
  }
}

// Work items and their activation scale blocks in one launch (one block per item): the decode path runs this twice
// per MoE layer, and a launch saved there is worth more than the few redundant loads.
__global__ void mx4_prep_kernel(int mode, const int4* __restrict__ tiles, const int* __restrict__ ntile,
                                const int* __restrict__ pair_expert, const int* __restrict__ pair_row, int pairs,
                                int max_items, const uint8_t* __restrict__ sf, int kblocks32, int4* __restrict__ items,
                                int* __restrict__ n_items, uint8_t* __restrict__ out) {
  const int i = blockIdx.x;
  const int n = mode == 0 ? min(*ntile, max_items) : min(pairs, max_items);
  int4 item = make_int4(0, 0, -1, 0);
  if (i < n) {
    if (mode == 0) {
      const int4 td = tiles[i];
      item = make_int4(td.x, min(128, td.y - td.x), td.z, td.x);
    } else {
      item = make_int4(pair_row ? pair_row[i] : i, 1, pair_expert[i], i);
    }
  }
  if (threadIdx.x == 0) {
    items[i] = item;
    if (i == 0) *n_items = n;
  }
  if (i >= n) return;
  const int kb128 = kblocks32 >> 2;
  for (int j = threadIdx.x; j < kb128 * 512; j += blockDim.x) {
    const int kt = j >> 9, within = j & 511;
    const int r32 = within >> 4, q = (within >> 2) & 3, kk = within & 3;
    const int r = q * 32 + r32;
    uint8_t v = 0;
    if (item.z >= 0 && r < item.y) v = sf[static_cast<size_t>(item.x + r) * kblocks32 + kt * 4 + kk];
    out[(static_cast<size_t>(i) * kb128 + kt) * 512 + within] = v;
  }
}

// Scale bytes [rows, K/32] (row-major) -> the tensor core's block layout [ceil(rows/128)][K/128][512]; rows past the
// end get exponent 0 (scale 2^-127: their products vanish and are never stored anyway).
__global__ void mx_sf_to_blocks_kernel(const uint8_t* __restrict__ sf, uint8_t* __restrict__ out, int rows, int kblocks32) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int kb128 = kblocks32 >> 2;
  const long long total = static_cast<long long>((rows + 127) / 128) * kb128 * 512;
  if (i >= total) return;
  const int within = static_cast<int>(i & 511);
  const long long blk = i >> 9;
  const int kt = static_cast<int>(blk % kb128);
  const int rt = static_cast<int>(blk / kb128);
  const int r32 = within >> 4, q = (within >> 2) & 3, kk = within & 3;
  const int row = rt * 128 + q * 32 + r32;
  out[i] = row < rows ? sf[static_cast<size_t>(row) * kblocks32 + kt * 4 + kk] : 0;
}

typedef CUresult (*EncodeTiledFnMx)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFnMx encode_fn_mx() {
  static EncodeTiledFnMx fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnMx>(p);
  });
  return fn;
}
static int make_tmap_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t K, uint64_t ld, uint32_t box_rows = 128) {
  EncodeTiledFnMx fn = encode_fn_mx();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld & 15)) return -2;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {MX_BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// packed e2m1 [rows, K/2 bytes]: 128 nibbles of a row (64 bytes of global memory) land as 128 bytes of shared memory
static int make_tmap_u4(CUtensorMap* m, const void* base, uint64_t rows, uint64_t K) {
  EncodeTiledFnMx fn = encode_fn_mx();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 31) || ((K / 2) & 31) || (K & 127)) return -2;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K / 2};
  cuuint32_t box[2] = {MX_BK, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace spark

using namespace spark;

extern "C" int spark_mx4_items(int mode, const void* tiles, const int* ntile, const int* pair_expert, const int* pair_row,
                               int pairs, int max_items, void* items, int* n_items, cudaStream_t stream) {
  if (max_items <= 0) return 0;
  mx4_items_kernel<<<(max_items + 127) / 128, 128, 0, stream>>>(mode, (const int4*)tiles, ntile, pair_expert, pair_row, pairs,
                                                                max_items, (int4*)items, n_items);
  return spark_launch_rc(__func__);
}

extern "C" int spark_mx_sf_tile_blocks(const void* sf, const void* items, const int* n_items, int max_items, int kblocks32,
                                       void* out, cudaStream_t stream) {
  if (max_items <= 0 || kblocks32 <= 0) return 0;
  if (kblocks32 % 4) return -5;
  mx_sf_tile_blocks_kernel<<<max_items, 256, 0, stream>>>((const uint8_t*)sf, (const int4*)items, n_items, max_items, kblocks32,
                                                         (uint8_t*)out);
  return spark_launch_rc(__func__);
}

extern "C" int spark_mx4_prep(int mode, const void* tiles, const int* ntile, const int* pair_expert, const int* pair_row,
                              int pairs, int max_items, const void* sf, int kblocks32, void* items, int* n_items, void* out,
                              cudaStream_t stream) {
  if (max_items <= 0 || kblocks32 <= 0) return 0;
  if (kblocks32 % 4) return -5;
  mx4_prep_kernel<<<max_items, 256, 0, stream>>>(mode, (const int4*)tiles, ntile, pair_expert, pair_row, pairs, max_items,
                                                 (const uint8_t*)sf, kblocks32, (int4*)items, n_items, (uint8_t*)out);
  return spark_launch_rc(__func__);
}

// A e4m3 [rows_a, K] (row stride lda bytes); W packed e2m1 [E * N, K / 2]; sfa item-local blocks
// (spark_mx_sf_tile_blocks), sfw blocks of the flattened [E * N, K / 32] scales (spark_mx_sf_to_blocks);
// C [*, ldc] bf16 or fp32.  N % 128 == 0, K % 128 == 0.  small != 0: every item has <= 16 rows (ten-stage variant).
extern "C" int spark_moe_mxfp4(const void* A, int lda, int rows_a, const void* W, const void* sfa, const void* sfw,
                               const void* items, const int* n_items, int max_items, int E, int N, int K, void* C, int ldc,
                               int out_f32, int small, int* status, cudaStream_t stream) {
  if (max_items <= 0 || rows_a <= 0) return 0;
  if (K % MX_BK || N % MX_BN || (ldc & 7) || (reinterpret_cast<uintptr_t>(C) & 15)) return -5;
  CUtensorMap tA, tA16, tW;
  int r = make_tmap_u8(&tA, A, rows_a, K, lda);
  if (r) return r;
  r = make_tmap_u8(&tA16, A, rows_a, K, lda, 16);
  if (r) return r;
  r = make_tmap_u4(&tW, W, static_cast<uint64_t>(E) * N, K);
  if (r) return r - 10;
  // a 16U4_ALIGN16B copy completes the barrier with the packed bytes it read (64 per row), not the 128 it writes
  const uint32_t w_tx = MX_B_BYTES / 2;
  static const int burst_env = [] { const char* e = getenv("SPARK_MX4_BURST"); return e ? atoi(e) : 0; }();   // tuning knob
  int burst = burst_env > 0 ? burst_env : 1;
  const int max_burst = (small ? Mx4Cfg<true>::STAGES : Mx4Cfg<false>::STAGES) / 2;
  if (burst > max_burst) burst = max_burst;
  if (burst < 1) burst = 1;
  Mx4Args g{(const int4*)items, n_items, max_items, N, K, (const uint8_t*)sfa, (const uint8_t*)sfw, C, ldc, out_f32, status, w_tx,
            burst};
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(moe_mxfp4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Mx4Cfg<false>::SMEM);
    cudaFuncSetAttribute(moe_mxfp4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Mx4Cfg<true>::SMEM);
    attr_done = true;
  }
  static int sms = 0;
  if (!sms) { int dev; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const long long tiles = static_cast<long long>(max_items) * (N / MX_BN);
  const int grid = tiles < sms ? static_cast<int>(tiles) : sms;
  if (small) moe_mxfp4_kernel<true><<<grid, MX4_THREADS, Mx4Cfg<true>::SMEM, stream>>>(tA, tA16, tW, g);
  else moe_mxfp4_kernel<false><<<grid, MX4_THREADS, Mx4Cfg<false>::SMEM, stream>>>(tA, tA16, tW, g);
  return spark_launch_rc(__func__);
}

// A e4m3 [M,K] (row stride lda bytes), B e4m3 [N,K]; sfa / sfb in block layout (spark_mx_sf_to_blocks); K % 128 == 0.
extern "C" int spark_gemm_mxfp8(const void* A, const void* B, const void* sfa, const void* sfb, void* C, int M, int N, int K,
                                int lda, int ldb, int ldc, int out_f32, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % MX_BK) return -5;
  CUtensorMap tA, tB;
  int r = make_tmap_u8(&tA, A, M, K, lda);
  if (r) return r;
  r = make_tmap_u8(&tB, B, N, K, ldb);
  if (r) return r;
  MxGemmArgs g{M, N, K, (const uint8_t*)sfa, (const uint8_t*)sfb, C, ldc, out_f32, status};
  static bool attr_done = false;
  if (!attr_done) { cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MX_SMEM); attr_done = true; }
  static int sms = 0;
  if (!sms) { int dev; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const int tiles = ((M + MX_BM - 1) / MX_BM) * ((N + MX_BN - 1) / MX_BN);
  gemm_mxfp8_kernel<<<tiles < sms ? tiles : sms, MX_THREADS, MX_SMEM, stream>>>(tA, tB, g);
  return spark_launch_rc(__func__);
}

extern "C" int spark_mx_sf_to_blocks(const void* sf, void* out, int rows, int kblocks32, cudaStream_t stream) {
  if (rows <= 0 || kblocks32 <= 0) return 0;
  if (kblocks32 % 4) return -5;
  const long long total = static_cast<long long>((rows + 127) / 128) * (kblocks32 / 4) * 512;
  mx_sf_to_blocks_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>((const uint8_t*)sf, (uint8_t*)out, rows,
                                                                                         kblocks32);
  return spark_launch_rc(__func__);
}
