// Host entry points of the tcgen05 GEMM family (C ABI: raw pointers, shapes, stream).
#include "gemm_sm100.cuh"
#include <mutex>

namespace spark {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// K-major 2D bf16 tensor [rows, K] with row stride ld (elements); box = 64 x 128, 128-byte swizzle.
// Out-of-range rows / K are zero-filled by the hardware, so ragged M, N and K need no padding.
int make_tmap_bf16(CUtensorMap* m, const void* base, uint64_t rows, uint64_t K, uint64_t ld, int box_rows, int fmt = 1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {GEMM_BK, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

static int num_sms() {
  static int n = 0;
  if (!n) { int dev; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); }
  return n;
}

template <int BN, class Epi, bool GROUPED>
static int launch(const CUtensorMap& tA, const CUtensorMap& tB, const GemmArgs& g, const Epi& epi, int grid,
                  cudaStream_t stream) {
  auto kern = gemm_tcgen05_kernel<BN, Epi, GROUPED>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL);
    attr_done = true;
  }
  kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(tA, tB, g, epi);
  return spark_launch_rc(__func__);
}

}  // namespace spark

using namespace spark;

// C[M,N] = A[M,K] B[N,K]^T.  out_f32: 0 -> bf16 C, 1 -> fp32 C.  Returns 0 or a negative error.
extern "C" int spark_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                               int ldc, int out_f32, int fmt, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap tA, tB;
  int r = make_tmap_bf16(&tA, A, M, K, lda, 128, fmt);
  if (r) return r;
  r = make_tmap_bf16(&tB, B, N, K, ldb, 128, fmt);
  if (r) return r;
  GemmArgs g{};
  g.M = M; g.N = N; g.K = K; g.status = status; g.ab_fmt = fmt;
  const int mt = (M + GEMM_BM - 1) / GEMM_BM;
  if (N > 128) {
    g.num_n_tiles = (N + 255) / 256; g.num_tiles = mt * g.num_n_tiles;
    int grid = g.num_tiles < num_sms() ? g.num_tiles : num_sms();
    if (out_f32) return launch<256, EpiStoreF32, false>(tA, tB, g, EpiStoreF32{(float*)C, ldc, N}, grid, stream);
    return launch<256, EpiStoreBf16, false>(tA, tB, g, EpiStoreBf16{(__nv_bfloat16*)C, ldc, N}, grid, stream);
  }
  g.num_n_tiles = (N + 127) / 128; g.num_tiles = mt * g.num_n_tiles;
  int grid = g.num_tiles < num_sms() ? g.num_tiles : num_sms();
  if (out_f32) return launch<128, EpiStoreF32, false>(tA, tB, g, EpiStoreF32{(float*)C, ldc, N}, grid, stream);
  return launch<128, EpiStoreBf16, false>(tA, tB, g, EpiStoreBf16{(__nv_bfloat16*)C, ldc, N}, grid, stream);
}

// SwiGLU-fused: C[M,F] = act(A B_gate^T) * (A B_up^T) with B = [gate rows (F) | up rows (F)], F % 128 == 0.
extern "C" int spark_gemm_bf16_swiglu(const void* A, const void* B, void* C, int M, int F, int K, int lda, int ldb,
                                      int ldc, float limit, int* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (F % 128) return -5;
  CUtensorMap tA, tB;
  int r = make_tmap_bf16(&tA, A, M, K, lda, 128);
  if (r) return r;
  r = make_tmap_bf16(&tB, B, 2 * F, K, ldb, 128);
  if (r) return r;
  GemmArgs g{};
  g.M = M; g.N = F; g.K = K; g.status = status; g.gate_up_F = F; g.ab_fmt = 1;
  g.num_n_tiles = F / 128; g.num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * g.num_n_tiles;
  int grid = g.num_tiles < num_sms() ? g.num_tiles : num_sms();
  return launch<256, EpiSwigluBf16, false>(tA, tB, g, EpiSwigluBf16{(__nv_bfloat16*)C, ldc, F, limit}, grid, stream);
}

// Grouped (MoE) GEMM over a device-side tile list: rows of A are (token, slot) pairs permuted into
// expert order; tile_list[i] = {a_row0, row_end, expert, 0}; *tile_count m-tiles are valid.
//   mode 0: C[rows, N] fp32 = A B_e^T          (down projection; combine sums slots later)
//   mode 1: C[rows, F] bf16 = swiglu(A B_e^T)  (B_e = [gate | up], N = F)
extern "C" int spark_gemm_grouped_bf16(const void* A, const void* B, void* C, int total_rows, int N, int K,
                                       int lda, int ldb, int ldc, int n_experts, int b_rows_per_expert,
                                       const void* tile_list, const int* tile_count, int max_m_tiles, int mode,
                                       float limit, int fmt, int* status, cudaStream_t stream) {
  if (total_rows <= 0 || max_m_tiles <= 0) return 0;
  CUtensorMap tA, tB;
  int r = make_tmap_bf16(&tA, A, total_rows, K, lda, 128, fmt);
  if (r) return r;
  r = make_tmap_bf16(&tB, B, (uint64_t)n_experts * b_rows_per_expert, K, ldb, 128, fmt);
  if (r) return r;
  GemmArgs g{};
  g.M = total_rows; g.N = N; g.K = K; g.status = status; g.ab_fmt = fmt;
  g.tile_list = reinterpret_cast<const int4*>(tile_list); g.tile_count = tile_count;
  g.b_rows_per_expert = b_rows_per_expert;
  if (mode == 1) {
    if (N % 128) return -5;
    g.gate_up_F = N; g.num_n_tiles = N / 128; g.num_tiles = max_m_tiles * g.num_n_tiles;
    return launch<256, EpiSwigluBf16, true>(tA, tB, g, EpiSwigluBf16{(__nv_bfloat16*)C, ldc, N, limit}, num_sms(), stream);
  }
  if (N % 256 == 0) {
    g.num_n_tiles = N / 256; g.num_tiles = max_m_tiles * g.num_n_tiles;
    return launch<256, EpiStoreF32, true>(tA, tB, g, EpiStoreF32{(float*)C, ldc, N}, num_sms(), stream);
  }
  g.num_n_tiles = (N + 127) / 128; g.num_tiles = max_m_tiles * g.num_n_tiles;
  return launch<128, EpiStoreF32, true>(tA, tB, g, EpiStoreF32{(float*)C, ldc, N}, num_sms(), stream);
}

// Row-parallel GEMM fused with the reduce-scatter of its output: C is never materialised locally; the epilogue
// writes fp32 partial tiles into the owner rank's arena and flags the owners when this rank is done.
// M must equal world * rows_per_rank (pad rows are computed from zero-filled A and pushed as zeros).
struct HostPush { void* peers[8]; long long slot_off, flag_off; int rank, world, rows_per_rank; unsigned seq; int* counter; void* seq_ptr; };
extern "C" int spark_gemm_bf16_push_rs(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int fmt,
                                       const HostPush* hp, int* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N % 4) return -5;
  CUtensorMap tA, tB;
  int r = make_tmap_bf16(&tA, A, M, K, lda, 128, fmt);
  if (r) return r;
  r = make_tmap_bf16(&tB, B, N, K, ldb, 128, fmt);
  if (r) return r;
  GemmArgs g{};
  g.M = M; g.N = N; g.K = K; g.status = status; g.ab_fmt = fmt;
  EpiPushRS epi;
  for (int i = 0; i < 8; ++i) epi.peers[i] = static_cast<uint8_t*>(hp->peers[i]);
  epi.slot_off = hp->slot_off; epi.flag_off = hp->flag_off; epi.rank = hp->rank; epi.world = hp->world;
  epi.rows_per_rank = hp->rows_per_rank; epi.N = N; epi.seq = hp->seq; epi.counter = hp->counter;
  epi.seq_ptr = static_cast<const uint32_t*>(hp->seq_ptr);
  const int mt = (M + GEMM_BM - 1) / GEMM_BM;
  if (N > 128) {
    g.num_n_tiles = (N + 255) / 256; g.num_tiles = mt * g.num_n_tiles;
    int grid = g.num_tiles < num_sms() ? g.num_tiles : num_sms();
    return launch<256, EpiPushRS, false>(tA, tB, g, epi, grid, stream);
  }
  g.num_n_tiles = (N + 127) / 128; g.num_tiles = mt * g.num_n_tiles;
  int grid = g.num_tiles < num_sms() ? g.num_tiles : num_sms();
  return launch<128, EpiPushRS, false>(tA, tB, g, epi, grid, stream);
}

// Column-parallel GEMM with the all-gather of its input fused in: A is the gathered buffer in the local arena
// ([world * ag_rows, K], block src written by rank src, see spark_ag_push); tiles of a block start as soon as
// that block's flag arrives, the local block first.
extern "C" int spark_gemm_bf16_ag(const void* A_gathered, const void* B, void* C, int M, int N, int K, int ldb, int ldc,
                                  int out_f32, const void* ag_flags, unsigned ag_seq, int ag_rows, int rank, int world,
                                  unsigned long long wait_ns, int* status, cudaStream_t stream, const void* seq_ptr) {
  if (M <= 0) return 0;
  CUtensorMap tA, tB;
  int r = make_tmap_bf16(&tA, A_gathered, M, K, K, 128, 1);
  if (r) return r;
  r = make_tmap_bf16(&tB, B, N, K, ldb, 128, 1);
  if (r) return r;
  GemmArgs g{};
  g.M = M; g.N = N; g.K = K; g.status = status; g.ab_fmt = 1;
  g.ag_flags = static_cast<const uint32_t*>(ag_flags); g.ag_seq = ag_seq; g.ag_rows = ag_rows; g.ag_rank = rank;
  g.ag_world = world; g.ag_wait_ns = wait_ns; g.ag_seq_ptr = static_cast<const uint32_t*>(seq_ptr);
  const int mt = (M + GEMM_BM - 1) / GEMM_BM;
  if (N > 128) {
    g.num_n_tiles = (N + 255) / 256; g.num_tiles = mt * g.num_n_tiles;
    int grid = g.num_tiles < num_sms() ? g.num_tiles : num_sms();
    if (out_f32) return launch<256, EpiStoreF32, false>(tA, tB, g, EpiStoreF32{(float*)C, ldc, N}, grid, stream);
    return launch<256, EpiStoreBf16, false>(tA, tB, g, EpiStoreBf16{(__nv_bfloat16*)C, ldc, N}, grid, stream);
  }
  g.num_n_tiles = (N + 127) / 128; g.num_tiles = mt * g.num_n_tiles;
  int grid = g.num_tiles < num_sms() ? g.num_tiles : num_sms();
  if (out_f32) return launch<128, EpiStoreF32, false>(tA, tB, g, EpiStoreF32{(float*)C, ldc, N}, grid, stream);
  return launch<128, EpiStoreBf16, false>(tA, tB, g, EpiStoreBf16{(__nv_bfloat16*)C, ldc, N}, grid, stream);
}
