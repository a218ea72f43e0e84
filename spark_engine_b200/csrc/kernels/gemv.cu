// Skinny GEMV for decode / verify rows:  y[R,N] = x[R,K] W[N,K]^T with R <= 16, bf16 weights.
// Bandwidth-bound: each warp streams two weight rows with 16-byte loads while the activation rows
// sit in shared memory; every output is produced by ONE warp with a fixed reduction order, so a row's
// result does not depend on how many other rows are in the batch (batch-invariant decode, as
// engine-rs/src/forward.rs:536-544 requires) and two runs are bitwise equal.
// The `item` dimension (blockIdx.y) turns it into the MoE decode GEMV: item i multiplies its own
// activation row by expert pair_expert[i]'s matrix.
// Replaces engine-rs/shim/gemv.cu:8-72, qwen_f16.cu:14-258, dataflow.cu:772 bf16w_rows.
#include "../common/decode.cuh"

namespace spark {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_COLS = 2;      // output columns per warp

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// act: 0 none; 1 = input is [gate | up] (2K wide), x := swiglu(gate, up) computed while staging.
template <int RB, typename TO>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ W,
                 long long expert_stride, int ldw, TO* __restrict__ y, int ldy, int rows_per_item, int N, int K,
                 const int* __restrict__ pair_expert, const int* __restrict__ pair_row, int act, float limit,
                 long long x_item_stride, long long y_item_stride, int cpc) {
  extern __shared__ __align__(16) uint8_t smem_gemv[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_gemv);     // [RB][K]
  const int item = blockIdx.y;
  pdl_wait();                                            // rows (and pair tables) come from earlier launches
  if (pair_expert && pair_expert[item] < 0) return;      // pair of an expert that lives on another rank
  // strided items (either stride non-zero): item i reads rows x + i * x_item_stride + r * ldx and writes rows
  // y + i * y_item_stride + r * ldy, e.g. the per-head slices of a [rows, heads, dim] tensor
  const bool strided = (x_item_stride | y_item_stride) != 0;
  if (strided) { x += item * x_item_stride; y += item * y_item_stride; }
  const int xr0 = strided ? 0 : (pair_row ? pair_row[item] : item * rows_per_item);
  const int yr0 = strided ? 0 : item * rows_per_item;
  const __nv_bfloat16* Wb = W + (pair_expert ? static_cast<long long>(pair_expert[item]) * expert_stride : 0);
  const int R = rows_per_item;
  // stage activations (zero rows beyond R); plain rows are copied as 16-byte vectors
  if (act == 0) {
    const int KV8 = K >> 3;
    for (int i = threadIdx.x; i < RB * KV8; i += blockDim.x) {
      const int r = i / KV8, kv = i - r * KV8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < R) v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(xr0 + r) * ldx + kv * 8);
      reinterpret_cast<uint4*>(xs)[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < RB * K; i += blockDim.x) {
      const int r = i / K, k = i - r * K;
      float v = 0.f;
      if (r < R) {
        const __nv_bfloat16* xr = x + static_cast<size_t>(xr0 + r) * ldx;
        float g = __bfloat162float(xr[k]), u = __bfloat162float(xr[K + k]);
        if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        v = g / (1.f + __expf(-g)) * u;
      }
      xs[i] = __float2bfloat16(v);
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a CTA covers `cpc` groups of 16 output columns, so that wide projections (lm_head) stage the rows once per
  // 16 * cpc columns instead of once per 16
  for (int cg = 0; cg < cpc; ++cg) {
  const int n0 = ((blockIdx.x * cpc + cg) * GEMV_WARPS + warp) * GEMV_COLS;
  if (n0 >= N) return;
  const bool two = (n0 + 1) < N;
  const uint4* w0 = reinterpret_cast<const uint4*>(Wb + static_cast<size_t>(n0) * ldw);
  const uint4* w1 = reinterpret_cast<const uint4*>(Wb + static_cast<size_t>(two ? n0 + 1 : n0) * ldw);
  float acc0[RB], acc1[RB];
#pragma unroll
  for (int r = 0; r < RB; ++r) { acc0[r] = 0.f; acc1[r] = 0.f; }
  const int KV = K >> 3;                        // 16-byte vectors per row
  constexpr int BATCH = 8;                      // loads in flight per lane and column
  for (int kv0 = lane; kv0 < KV; kv0 += 32 * BATCH) {
    uint4 ra[BATCH], rb[BATCH];
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      const int kv = kv0 + 32 * u;
      ra[u] = kv < KV ? __ldg(w0 + kv) : make_uint4(0u, 0u, 0u, 0u);
      rb[u] = kv < KV ? __ldg(w1 + kv) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      const int kv = kv0 + 32 * u;
      if (kv < KV) {
        float a[8], b[8];
        unpack8(ra[u], a);
        unpack8(rb[u], b);
#pragma unroll
        for (int r = 0; r < RB; ++r) {
          float xv[8];
          unpack8(*reinterpret_cast<const uint4*>(xs + r * K + kv * 8), xv);
#pragma unroll
          for (int i = 0; i < 8; ++i) { acc0[r] = fmaf(a[i], xv[i], acc0[r]); acc1[r] = fmaf(b[i], xv[i], acc1[r]); }
        }
      }
    }
  }
  if (cg == cpc - 1) pdl_trigger();                      // weight stream done: the next kernel may start its loads
#pragma unroll
  for (int r = 0; r < RB; ++r) { acc0[r] = warp_sum(acc0[r]); acc1[r] = warp_sum(acc1[r]); }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      if (r < R) {
        TO* yr = y + static_cast<size_t>(yr0 + r) * ldy;
        yr[n0] = static_cast<TO>(acc0[r]);
        if (two) yr[n0 + 1] = static_cast<TO>(acc1[r]);
      }
    }
  }
  }
}

template <int RB, typename TO>
static int launch_gemv(const void* x, int ldx, const void* W, long long es, int ldw, void* y, int ldy, int items,
                       int rows, int N, int K, const int* pe, const int* pr, int act, float limit, cudaStream_t s,
                       long long xis = 0, long long yis = 0) {
  auto kern = gemv_bf16_kernel<RB, TO>;
  const int smem = RB * K * 2;
  if (smem > 48 * 1024) {
    static int set_for = 0;
    if (smem > set_for) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); set_for = 200 * 1024; }
  }
  if (smem > 200 * 1024) return -6;
  const int groups = (N + GEMV_WARPS * GEMV_COLS - 1) / (GEMV_WARPS * GEMV_COLS);
  int cpc = (groups + 1183) / 1184;                  // keep wide grids near 8 CTAs x 148 SMs
  if (cpc < 1) cpc = 1;
  if (cpc > 8) cpc = 8;
  dim3 grid((groups + cpc - 1) / cpc, items);
  const cudaError_t err = spark_launch_pdl(kern, grid, dim3(GEMV_WARPS * 32), smem, s, dim3(1, 1, 1),
                                           (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, es, ldw, (TO*)y, ldy, rows, N, K,
                                           pe, pr, act, limit, xis, yis, cpc);
  return err == cudaSuccess ? 0 : -4;
}

// Wide projections (lm_head: N >= 2048 columns, every column read once) with the rows as the N side of
// mma.sync m16n8k16: a warp owns 16 weight rows, lane (g, t) loads 16 contiguous bytes of rows g and g + 8 per
// 32 k and uses them as the A fragments of two MMAs; the same permutation of k is applied to the activation
// fragment (one 16-byte shared-memory load per lane), which leaves every dot product unchanged.  No unpacking,
// no cross-lane reduction: about 8 warp-instructions per KB of weights instead of about 30 x rows.  Which kernel
// runs depends on (N, K) only, never on the number of rows, and every output element is one fixed chain of
// MMAs over k, so a row's logits do not depend on the batch it is in.
constexpr int GEMV_MMA_PAD = 8;   // bf16 of padding per staged activation row: spreads rows over the banks

__device__ __forceinline__ void gemv_mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// KS = false: a warp owns 16 weight rows over the whole of K (heads of >= 150K rows).  KS = true: a CTA owns 16 weight
// rows, its 8 warps split K and their partial tiles are summed in warp order through shared memory (projections of
// a few thousand rows, where one warp per 16 rows would leave most SMs idle).
template <int NT, typename TO, bool KS>
__global__ void __launch_bounds__(GEMV_WARPS * 32, NT == 1 ? 3 : 2)      // <= 85 registers: three CTAs of loads in flight per SM
gemv_wide_mma_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ W, int ldw,
                     TO* __restrict__ y, int ldy, int R, int N, int K, int cpc) {
  extern __shared__ __align__(16) uint8_t smem_gemv[];
  __shared__ float red[KS ? GEMV_WARPS : 1][NT * 4][32];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_gemv);     // [NT * 8][K + GEMV_MMA_PAD]
  const int lds = K + GEMV_MMA_PAD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int KC = K >> 5;                                 // 32-wide k chunks
  const int per = (KC + GEMV_WARPS - 1) / GEMV_WARPS;
  const int kb = KS ? min(KC, warp * per) : 0, ke = KS ? min(KC, kb + per) : KC;    // this warp's chunks
  constexpr int BATCH = NT == 1 ? 6 : 8;                 // chunks in flight per lane and weight row (fits the register budget)
  uint4 ra[BATCH], rb[BATCH];
  auto rows_of = [&](int cg, const uint4*& w0, const uint4*& w1) -> int {
    const int n0 = KS ? blockIdx.x * 16 : ((blockIdx.x * cpc + cg) * GEMV_WARPS + warp) * 16;
    w0 = reinterpret_cast<const uint4*>(W + static_cast<size_t>(min(n0 + g, N - 1)) * ldw) + t;
    w1 = reinterpret_cast<const uint4*>(W + static_cast<size_t>(min(n0 + g + 8, N - 1)) * ldw) + t;
    return n0;
  };
  auto load = [&](const uint4* w0, const uint4* w1, int kc0) {
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      const bool in = kc0 + u < ke;
      ra[u] = in ? __ldg(w0 + (kc0 + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
      rb[u] = in ? __ldg(w1 + (kc0 + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  const uint4 *w0, *w1;
  int n0 = rows_of(0, w0, w1);
  pdl_wait();
  if (n0 < N) load(w0, w1, kb);                          // in flight while the rows are staged
  const int KV8 = K >> 3;
  for (int i = threadIdx.x; i < NT * 8 * KV8; i += blockDim.x) {
    const int r = i / KV8, kv = i - r * KV8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < R) v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ldx + kv * 8);
    *reinterpret_cast<uint4*>(xs + r * lds + kv * 8) = v;
  }
  __syncthreads();
  for (int cg = 0; cg < (KS ? 1 : cpc); ++cg) {
    if (cg) { n0 = rows_of(cg, w0, w1); if (n0 < N) load(w0, w1, kb); }
    if (n0 >= N) break;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
    for (int kc0 = kb; kc0 < ke; kc0 += BATCH) {
      if (kc0 != kb) load(w0, w1, kc0);
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        if (kc0 + u < ke) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 xb = *reinterpret_cast<const uint4*>(xs + (nt * 8 + g) * lds + (kc0 + u) * 32 + t * 8);
            gemv_mma16816(acc[nt], ra[u].x, rb[u].x, ra[u].y, rb[u].y, xb.x, xb.y);
            gemv_mma16816(acc[nt], ra[u].z, rb[u].z, ra[u].w, rb[u].w, xb.z, xb.w);
          }
        }
      }
    }
    if (KS) {
      // the CTA's 16 weight rows: partial tiles of the 8 warps, summed in warp order
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) red[warp][nt * 4 + j][lane] = acc[nt][j];
      __syncthreads();
      for (int i = threadIdx.x; i < NT * 4 * 32; i += blockDim.x) {
        const int slot = i >> 5, ln = i & 31, nt = slot >> 2, j = slot & 3;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) v += red[w][slot][ln];
        const int r = nt * 8 + 2 * (ln & 3) + (j & 1), n = n0 + (ln >> 2) + (j >> 1) * 8;
        if (r < R && n < N) y[static_cast<size_t>(r) * ldy + n] = static_cast<TO>(v);
      }
    } else {
      // accumulator (g, t): weight rows n0 + g and n0 + g + 8, activation rows nt * 8 + 2t and + 1
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = nt * 8 + 2 * t + (j & 1), n = n0 + g + (j >> 1) * 8;
          if (r < R && n < N) y[static_cast<size_t>(r) * ldy + n] = static_cast<TO>(acc[nt][j]);
        }
      }
    }
  }
  pdl_trigger();
}

template <int NT, typename TO, bool KS>
static int launch_gemv_wide_as(const void* x, int ldx, const void* W, int ldw, void* y, int ldy, int rows, int N, int K,
                               cudaStream_t s) {
  auto kern = gemv_wide_mma_kernel<NT, TO, KS>;
  const int smem = NT * 8 * (K + GEMV_MMA_PAD) * 2;
  if (smem > 200 * 1024) return -6;
  if (smem > 48 * 1024) {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); set = true; }
  }
  const int groups = KS ? (N + 15) / 16 : (N + GEMV_WARPS * 16 - 1) / (GEMV_WARPS * 16);
  int cpc = KS ? 1 : (groups + 2367) / 2368;         // short CTAs: the tail of the last wave stays small
  if (cpc < 1) cpc = 1;
  dim3 grid((groups + cpc - 1) / cpc);
  const cudaError_t err = spark_launch_pdl(kern, grid, dim3(GEMV_WARPS * 32), smem, s, dim3(1, 1, 1),
                                           (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, ldw, (TO*)y, ldy, rows, N, K, cpc);
  return err == cudaSuccess ? 0 : -4;
}

// Fewer than 8 x 148 tiles of 16 weight rows: split K over the warps of a CTA instead of giving every warp its own tile
// (depends on N only, so a row's result does not change with the batch it is in).
template <int NT, typename TO>
static int launch_gemv_wide(const void* x, int ldx, const void* W, int ldw, void* y, int ldy, int rows, int N, int K,
                            cudaStream_t s) {
  return (N + 15) / 16 < 8 * 148 ? launch_gemv_wide_as<NT, TO, true>(x, ldx, W, ldw, y, ldy, rows, N, K, s)
                                 : launch_gemv_wide_as<NT, TO, false>(x, ldx, W, ldw, y, ldy, rows, N, K, s);
}

// Shapes the wide kernel takes: one item, no activation, no expert tables, K a multiple of 32 and small enough that
// 16 staged rows fit in shared memory (the choice must not depend on the number of rows: a row's result may not
// change with the batch it is in).
static bool gemv_wide_ok(int ldx, int ldw, int items, int N, int K, const int* pe, const int* pr, int act) {
  return items == 1 && !pe && !pr && act == 0 && N >= 2048 && (K & 31) == 0 && (ldx & 7) == 0 && (ldw & 7) == 0 &&
         16 * (K + GEMV_MMA_PAD) * 2 <= 200 * 1024;
}

}  // namespace spark

using namespace spark;

// items x rows_per_item rows; K % 8 == 0; out_f32 selects fp32 or bf16 output.
extern "C" int spark_gemv_bf16(const void* x, int ldx, const void* W, long long expert_stride, int ldw, void* y, int ldy,
                               int items, int rows_per_item, int N, int K, const int* pair_expert, const int* pair_row,
                               int act, float limit, int out_f32, cudaStream_t s) {
  if (items <= 0 || rows_per_item <= 0) return 0;
  if (K % 8 || rows_per_item > 16) return -5;
  if (gemv_wide_ok(ldx, ldw, items, N, K, pair_expert, pair_row, act) &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15) == 0) {
    if (rows_per_item <= 8)
      return out_f32 ? launch_gemv_wide<1, float>(x, ldx, W, ldw, y, ldy, rows_per_item, N, K, s)
                     : launch_gemv_wide<1, __nv_bfloat16>(x, ldx, W, ldw, y, ldy, rows_per_item, N, K, s);
    return out_f32 ? launch_gemv_wide<2, float>(x, ldx, W, ldw, y, ldy, rows_per_item, N, K, s)
                   : launch_gemv_wide<2, __nv_bfloat16>(x, ldx, W, ldw, y, ldy, rows_per_item, N, K, s);
  }
#define SPARK_GEMV_CASE(RB)                                                                                          \
  if (rows_per_item <= RB)                                                                                           \
    return out_f32 ? launch_gemv<RB, float>(x, ldx, W, expert_stride, ldw, y, ldy, items, rows_per_item, N, K,       \
                                            pair_expert, pair_row, act, limit, s)                                    \
                   : launch_gemv<RB, __nv_bfloat16>(x, ldx, W, expert_stride, ldw, y, ldy, items, rows_per_item, N,  \
                                                    K, pair_expert, pair_row, act, limit, s);
  SPARK_GEMV_CASE(1)
  SPARK_GEMV_CASE(2)
  SPARK_GEMV_CASE(4)
  SPARK_GEMV_CASE(8)
  SPARK_GEMV_CASE(16)
#undef SPARK_GEMV_CASE
  return -5;
}

// Strided items: item i multiplies rows x + i * x_item_stride + r * ldx (r < rows_per_item) by expert
// pair_expert[i] (or W itself) and writes y + i * y_item_stride + r * ldy.  Used for per-head projections of
// [rows, heads, dim] tensors: every head's matrix is streamed once for all rows.  Strides in elements; the item
// offsets must keep x 16-byte aligned.
extern "C" int spark_gemv_bf16_items(const void* x, int ldx, long long x_item_stride, const void* W, long long expert_stride,
                                     int ldw, void* y, int ldy, long long y_item_stride, int items, int rows_per_item, int N,
                                     int K, const int* pair_expert, int out_f32, cudaStream_t s) {
  if (items <= 0 || rows_per_item <= 0) return 0;
  if (K % 8 || rows_per_item > 16 || (x_item_stride & 7) || (ldx & 7) || (x_item_stride | y_item_stride) == 0) return -5;
#define SPARK_GEMV_ITEMS(RB)                                                                                         \
  if (rows_per_item <= RB)                                                                                           \
    return out_f32 ? launch_gemv<RB, float>(x, ldx, W, expert_stride, ldw, y, ldy, items, rows_per_item, N, K,       \
                                            pair_expert, nullptr, 0, 0.f, s, x_item_stride, y_item_stride)           \
                   : launch_gemv<RB, __nv_bfloat16>(x, ldx, W, expert_stride, ldw, y, ldy, items, rows_per_item, N,  \
                                                    K, pair_expert, nullptr, 0, 0.f, s, x_item_stride, y_item_stride);
  SPARK_GEMV_ITEMS(1)
  SPARK_GEMV_ITEMS(2)
  SPARK_GEMV_ITEMS(4)
  SPARK_GEMV_ITEMS(8)
  SPARK_GEMV_ITEMS(16)
#undef SPARK_GEMV_ITEMS
  return -5;
}
