// tcgen05 GEMM for 16-bit inputs with fp32 accumulation in TMEM.
//
//   C[b] = act(alpha * A[b] . B[b]^T + beta * C[b] + bias)
//
// A is logically M x K, B logically N x K.  Each operand may be stored with K
// contiguous ("K-major": A as [M][K], B as [N][K]) or with its M/N dimension
// contiguous ("MN-major": A as [K][M], B as [K][N]), so all of forward
// (x.W^T), data gradient (dy.W) and weight gradient (dy^T.x) run without a
// transpose pass.  Replaces the cuBLAS calls behind the reference's
// fully_connected (src/layers/learning/fully_connected.cpp:511-636),
// channelwise_fully_connected and matmul layers
// (src/layers/math/matmul.cpp:419-584, strided-batched).
#include "tc_pipeline.cuh"

namespace lb {

template <int BN_>
struct GemmPolicy {
  static constexpr int BN = BN_;
  static constexpr int kEpiGroups = 2;       // two tiles' epilogues in flight (tc_pipeline.cuh)
  using G = StageGeom<BN>;

  struct Params {
    int M, N, K, batch;
    int tiles_m, tiles_n;
    int num_tiles, k_iters;
    int a_mn, b_mn, in_dtype;
    long long strideC;
    EpiParams epi;
  };
  struct Tile {
    int m0, n0, b;
  };

  __device__ static Tile decode(const Params& p, int t) {
    const int per_batch = p.tiles_m * p.tiles_n;
    Tile tl;
    tl.b = t / per_batch;
    const int r = t - tl.b * per_batch;
    const int nb = r / p.tiles_m;
    tl.n0 = nb * BN;
    tl.m0 = (r - nb * p.tiles_m) * kBM;
    return tl;
  }
  __device__ static uint32_t stage_bytes(const Params&, const Tile&, int) {
    return G::kStageBytes;
  }
  __device__ static void load(const Params& p, const Tile& tl, int k, uint32_t sA, uint32_t sB,
                              uint32_t bar, const CUtensorMap* tmA, const CUtensorMap* tmB,
                              int lane) {
    const int k0 = k * kBK;
    // boxes of the A operand go out from lanes 0.., boxes of B from lanes 8..
    if (!p.a_mn) {
      if (lane == 0) tma_load_3d(sA, tmA, bar, k0, tl.m0, tl.b);  // box {64 k, 128 rows}
    } else if (lane < kBM / 64) {                                 // box {64 m, 64 k-rows}
      tma_load_3d(sA + lane * 8192, tmA, bar, tl.m0 + lane * 64, k0, tl.b);
    }
    if (!p.b_mn) {
      if (lane == 8) tma_load_3d(sB, tmB, bar, k0, tl.n0, tl.b);  // box {64 k, BN rows}
    } else if (lane >= 8 && lane < 8 + BN / 64) {
      const int j = lane - 8;
      tma_load_3d(sB + j * 8192, tmB, bar, tl.n0 + j * 64, k0, tl.b);
    }
  }
  __device__ static uint32_t idesc(const Params& p) {
    return make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, p.a_mn, p.b_mn, kBM, BN);
  }
  __device__ static void mma(const Params& p, int, uint32_t sA, uint32_t sB, uint32_t tmem_acc,
                             uint32_t idesc, bool first) {
    // K-major: 16 elements = 32 bytes along the swizzled row.
    // MN-major: 16 k-rows of 128 bytes.
    // The four descriptors of a stage differ in the start-address field of the low word.
    const uint64_t a0 = p.a_mn ? make_smem_desc(0, 8192, 1024, kLayoutSw128)
                               : make_smem_desc(0, 16, 1024, kLayoutSw128);
    const uint64_t b0 = p.b_mn ? make_smem_desc(0, 8192, 1024, kLayoutSw128)
                               : make_smem_desc(0, 16, 1024, kLayoutSw128);
    const uint32_t a_hi = (uint32_t)(a0 >> 32), b_hi = (uint32_t)(b0 >> 32);
    const uint32_t a_lo = (uint32_t)a0 + (sA >> 4), b_lo = (uint32_t)b0 + (sB >> 4);
    const uint32_t a_step = p.a_mn ? (2048u >> 4) : (32u >> 4);
    const uint32_t b_step = p.b_mn ? (2048u >> 4) : (32u >> 4);
#pragma unroll
    for (int kk = 0; kk < kBK / 16; ++kk)
      umma_f16_lo(tmem_acc, a_lo + kk * a_step, a_hi, b_lo + kk * b_step, b_hi, idesc,
                  (first && kk == 0) ? 0u : 1u);
  }
  __device__ static bool row_addr(const Params& p, const Tile& tl, int row, long long& off) {
    const int m = tl.m0 + row;
    off = (long long)tl.b * p.strideC + (long long)m * p.epi.ldc;
    return m < p.M;
  }
  __device__ static int row_index(const Params&, const Tile& tl, int row) { return tl.m0 + row; }
  __device__ static int col0(const Params&, const Tile& tl) { return tl.n0; }
  __device__ static int ncols(const Params& p) { return p.N; }
};

template <int BN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB,
                       typename GemmPolicy<BN>::Params p, const lbhost::SplitKOffer& offer,
                       cudaStream_t stream) {
  using P = GemmPolicy<BN>;
  using G = StageGeom<BN>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(tc_persistent_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         G::kSmemBytes);
    configured = true;
  }
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n * p.batch;
  p.k_iters = (p.K + kBK - 1) / kBK;
  // a skinny product (few tiles, long K, e.g. a wide fully-connected layer on a small
  // mini-batch) is cut along K so that all SMs stream the weights
  if (p.epi.rs_ranks == 0 && p.epi.bcast_ranks == 0) {
    p.epi.k_splits = lbhost::plan_splitk(offer, p.num_tiles, p.k_iters, BN);
    p.epi.sk_ws = offer.ws;
  }
  const int items = p.num_tiles * p.epi.k_splits;
  const int grid = items < lbhost::sm_count() ? items : lbhost::sm_count();
  tc_persistent_kernel<P><<<grid, tc_threads<P>(), G::kSmemBytes, stream>>>(tmA, tmB, p,
                                                                       lbhost::status_word());
  int rc = (int)cudaGetLastError();
  if (rc == 0 && p.epi.k_splits > 1) rc = launch_splitk_reduce<P>(p, stream);
  return rc;
}

}  // namespace lb

extern "C" {

// Returns 0 on success, a cudaError_t (>0) on launch failure, -1 on a bad argument.
//   a_mn = 0: A stored [M][K] with row pitch lda;  a_mn = 1: A stored [K][M] with row pitch lda
//   b_mn = 0: B stored [N][K] with row pitch ldb;  b_mn = 1: B stored [K][N] with row pitch ldb
//   lda/ldb (elements) must be multiples of 8 and bases 16-byte aligned (TMA).
//   in_dtype: 0 fp16, 1 bf16.  out_dtype: 0 fp16, 1 bf16, 2 fp32.
int lb_gemm_bcast_tc(const void* A, const void* B, void* C, const float* bias, int M, int N, int K,
                     int batch, long long lda, long long ldb, long long ldc, long long strideA,
                     long long strideB, long long strideC, int a_mn, int b_mn, int in_dtype,
                     int out_dtype, float alpha, float beta, int bias_mode, int act, float act_param,
                     int bn_hint, void* const* bcast_ptrs, int bcast_ranks, void* stream_);

int lb_gemm_tc(const void* A, const void* B, void* C, const float* bias, int M, int N, int K,
               int batch, long long lda, long long ldb, long long ldc, long long strideA,
               long long strideB, long long strideC, int a_mn, int b_mn, int in_dtype,
               int out_dtype, float alpha, float beta, int bias_mode, int act, float act_param,
               int bn_hint, void* stream_) {
  return lb_gemm_bcast_tc(A, B, C, bias, M, N, K, batch, lda, ldb, ldc, strideA, strideB, strideC,
                          a_mn, b_mn, in_dtype, out_dtype, alpha, beta, bias_mode, act, act_param,
                          bn_hint, nullptr, 0, stream_);
}

// Same product with the all-gather epilogue: bcast_ptrs[q] is the (peer-mapped) address that
// C has on rank q (entry of this rank = C); every finished tile is stored into all of them.
// Needs a 16-bit output, beta == 0, N a multiple of 32 and 16-byte aligned rows; the caller
// runs a rendezvous of the ranks before the outputs are read.
int lb_gemm_bcast_tc(const void* A, const void* B, void* C, const float* bias, int M, int N, int K,
                     int batch, long long lda, long long ldb, long long ldc, long long strideA,
                     long long strideB, long long strideC, int a_mn, int b_mn, int in_dtype,
                     int out_dtype, float alpha, float beta, int bias_mode, int act, float act_param,
                     int bn_hint, void* const* bcast_ptrs, int bcast_ranks, void* stream_) {
  using namespace lb;
  const lbhost::SplitKOffer offer = lbhost::take_splitk_offer();   // holds for this call only
  if (bcast_ranks < 0 || bcast_ranks > 8) return -1;
  if (bcast_ranks > 0) {
    if (!bcast_ptrs || out_dtype == kF32 || beta != 0.f || N % 32 || ldc % 8) return -1;
    for (int q = 0; q < bcast_ranks; ++q)
      if (!bcast_ptrs[q] || (reinterpret_cast<uintptr_t>(bcast_ptrs[q]) & 15)) return -1;
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return -1;
  if ((lda % 8) || (ldb % 8) || (strideA % 8) || (strideB % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;

  int BN = bn_hint;
  if (BN != 64 && BN != 128 && BN != 256) {
    // Heuristic: the widest tile that still gives every SM a tile.
    const long long t256 = (long long)((M + 127) / 128) * ((N + 255) / 256) * batch;
    const long long t128 = (long long)((M + 127) / 128) * ((N + 127) / 128) * batch;
    if (N > 128 && t256 >= lbhost::sm_count()) BN = 256;
    else if (N > 64 && t128 >= lbhost::sm_count() / 2) BN = 128;
    else BN = N > 64 ? 128 : 64;
  }

  CUtensorMap tmA, tmB;
  const uint64_t sa = strideA > 0 ? (uint64_t)strideA : (uint64_t)lda * (a_mn ? K : M);
  const uint64_t sb = strideB > 0 ? (uint64_t)strideB : (uint64_t)ldb * (b_mn ? K : N);
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!a_mn) { dims[0] = K; dims[1] = M; box[0] = 64; box[1] = 128; }
    else       { dims[0] = M; dims[1] = K; box[0] = 64; box[1] = 64; }
    dims[2] = batch; box[2] = 1;
    strides[0] = (uint64_t)lda * 2; strides[1] = sa * 2;
    if (!lbhost::encode_tmap(&tmA, in_dtype, 3, A, dims, strides, box, nullptr, 128)) return -1;
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!b_mn) { dims[0] = K; dims[1] = N; box[0] = 64; box[1] = (uint32_t)BN; }
    else       { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = 64; }
    dims[2] = batch; box[2] = 1;
    strides[0] = (uint64_t)ldb * 2; strides[1] = sb * 2;
    if (!lbhost::encode_tmap(&tmB, in_dtype, 3, B, dims, strides, box, nullptr, 128)) return -1;
  }

  EpiParams e;
  e.C = C; e.bias = bias; e.alpha = alpha; e.beta = beta; e.out_dtype = out_dtype;
  e.bias_mode = bias ? bias_mode : 0; e.act = act; e.act_param = act_param; e.ldc = ldc;
  e.bcast_ranks = bcast_ranks;
  for (int q = 0; q < bcast_ranks; ++q) e.bcast_ptr[q] = bcast_ptrs[q];

#define LB_LAUNCH(BN_)                                                        \
  {                                                                           \
    GemmPolicy<BN_>::Params p;                                                \
    p.M = M; p.N = N; p.K = K; p.batch = batch; p.a_mn = a_mn; p.b_mn = b_mn; \
    p.in_dtype = in_dtype; p.strideC = strideC; p.epi = e;                    \
    return launch_gemm<BN_>(tmA, tmB, p, offer, stream);                          \
  }
  if (BN == 256) LB_LAUNCH(256)
  if (BN == 128) LB_LAUNCH(128)
  LB_LAUNCH(64)
#undef LB_LAUNCH
}

}  // extern "C"
