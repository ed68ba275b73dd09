// First-layer convolution kernels for inputs with at most 8 channels (stored as exactly
// 8 = one 16-byte vector per pixel), 3x3x3 / 1x3x3 filters, stride 1, dilation 1.
//
// With 16 bytes per pixel a row of W consecutive pixels is a dense array of 16-byte
// vectors, which is exactly the core-matrix row pitch of the un-swizzled tcgen05 operand
// layouts.  The kernels exploit that to apply the kw taps WITHOUT re-loading or
// re-arranging data:
//
//  forward:  A is K-major, un-swizzled, row pitch 16 B, K-chunk pitch (LBO) 16 B, so
//            A[m][k] = slab[8 m + k]: row m sees pixels m, m+1 (one UMMA, K = 16) and
//            m+2, m+3 (second UMMA); the filter is laid out [kd*kh][Kout][kw(4) x c(8)] with
//            the kw = 3 column zero.  One TMA box of (W+2) pixels per (kd, kh) feeds 128
//            output pixels; there is no im2col and no per-tap reload.
//
//  wgrad:    A is MN-major, un-swizzled, with the M-block pitch (SBO) equal to one pixel
//            (16 B): M = 16 shifts x 8 channels, of which shifts 0..2 are the kw taps.  One
//            accumulator per (kd, kh) (9 x 32 TMEM columns for 32 output channels); a CTA
//            streams 64-pixel bricks (one x slab + one dy brick per stage) and finally adds
//            its partial dW with fp32 atomics.
//
// These replace the generic implicit-GEMM path for the layer where it is weakest (tiny
// reduction per tap, 27 reloads of the same pixels); the reference relies on cuDNN here
// (src/layers/learning/base_convolution.cpp:462-814).
#include "tc_pipeline.cuh"

namespace lb {

constexpr uint32_t kLayoutNone = 0;

struct C8Geom {
  int N, D, H, W;       // input spatial dims (C is 8)
  int Kout;
  int kd, kh;           // kw is 3
  int pd, ph;           // pw is 1
  int Do;               // output depth = D + 2 pd - kd + 1 (pd = 0 when halos carry the padding)
};

// ------------------------------------------------------------------------- forward
// A stage holds one (kd, kh) slab (<= 144 pixels = 2304 B) and its 2 KB filter slice.  The
// stages are tiny, so the ring is made deep: with ~1 us of load latency it is the number
// of bytes in flight, not the copy engine, that bounds this kernel.
template <int BN>
struct C8StageGeom {
  static constexpr int kABytes = 2304;
  static constexpr int kBBytes = BN * 64;
  static constexpr int kStageBytes = kABytes + kBBytes;     // multiple of 128
  static constexpr int kStages = 32;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
};

template <int BN_>
struct ConvC8FwdPolicy {
  static constexpr int BN = BN_;
  using G = C8StageGeom<BN>;
  struct Params {
    C8Geom g;
    int TW, tiles_w;
    int half_px;   // pixels per slab box: a multiple of 8 (128 B) so both boxes land aligned
    int num_tiles, k_iters, in_dtype;
    long long o_sn, o_sd, o_sh, o_sw;
    EpiParams epi;
  };
  struct Tile { int n, d, h, w0; };

  __device__ static Tile decode(const Params& p, int t) {
    Tile tl;
    int r = t;
    const int tw = r % p.tiles_w; r /= p.tiles_w;
    tl.h = r % p.g.H; r /= p.g.H;
    tl.d = r % p.g.Do; r /= p.g.Do;
    tl.n = r;
    tl.w0 = tw * p.TW;
    return tl;
  }
  __device__ static uint32_t stage_bytes(const Params& p, const Tile&, int) {
    return (uint32_t)(2 * p.half_px * 16 + BN * 64);
  }
  __device__ static void load(const Params& p, const Tile& tl, int k, uint32_t sA, uint32_t sB,
                              uint32_t bar, const CUtensorMap* tmA, const CUtensorMap* tmB,
                              int lane) {
    if (lane > 2) return;
    const int a = k / p.g.kh, b = k - a * p.g.kh;
    // Slab of 2 * half_px >= TW + 3 pixels starting one pixel left of the tile (TMA zero fill
    // supplies the padding).
    // The tensor map views the 16-byte pixels as pairs of 8-byte units so that a row of
    // pixels is ONE long TMA row instead of one 16-byte request per pixel; the slab comes
    // as two boxes of half_px pixels each; TMA destinations must be 128-byte aligned.
    const int half = p.half_px;
    const int h = tl.h - p.g.ph + b, d = tl.d - p.g.pd + a;
    if (lane == 0) tma_load_4d(sA, tmA, bar, (tl.w0 - 1) * 2, h, d, tl.n);
    if (lane == 1) tma_load_4d(sA + half * 16, tmA, bar, (tl.w0 - 1 + half) * 2, h, d, tl.n);
    if (lane == 2) tma_load_2d(sB, tmB, bar, 0, k);   // packed filter of tap-row k: one 2 KB row
  }
  __device__ static uint32_t idesc(const Params& p) {
    return make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 0, 0, kBM, BN);
  }
  __device__ static void mma(const Params&, int, uint32_t sA, uint32_t sB, uint32_t tmem_acc,
                             uint32_t idesc, bool first) {
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      // A: rows 16 B apart (SBO = 8 rows = 128 B), the two 8-element K chunks 16 B apart.
      const uint64_t ad = make_smem_desc(sA + kk * 32, 16, 128, kLayoutNone);
      // B: un-swizzled core-matrix order [k-chunk(4)][BN rows][8 elements]: rows 16 B apart,
      // 8-row groups 128 B apart (SBO), K chunks BN*16 B apart (LBO); 2 chunks per UMMA
      const uint64_t bd = make_smem_desc(sB + kk * 2 * BN * 16, BN * 16, 128, kLayoutNone);
      umma_f16(tmem_acc, ad, bd, idesc, (first && kk == 0) ? 0u : 1u);
    }
  }
  __device__ static bool row_addr(const Params& p, const Tile& tl, int row, long long& off) {
    const int w = tl.w0 + row;
    off = tl.n * p.o_sn + tl.d * p.o_sd + tl.h * p.o_sh + (long long)w * p.o_sw;
    return row < p.TW && w < p.g.W;
  }
  __device__ static int row_index(const Params&, const Tile&, int row) { return row; }
  __device__ static int col0(const Params&, const Tile&) { return 0; }
  __device__ static int ncols(const Params& p) { return p.g.Kout; }
};

template <int BN>
static int launch_c8_fwd(const CUtensorMap& tmA, const CUtensorMap& tmB,
                         typename ConvC8FwdPolicy<BN>::Params p, cudaStream_t stream) {
  using P = ConvC8FwdPolicy<BN>;
  using G = typename P::G;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(tc_persistent_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         G::kSmemBytes);
    configured = true;
  }
  const int grid = p.num_tiles < lbhost::sm_count() ? p.num_tiles : lbhost::sm_count();
  tc_persistent_kernel<P><<<grid, kTcThreads, G::kSmemBytes, stream>>>(tmA, tmB, p,
                                                                       lbhost::status_word());
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------- wgrad
struct C8WgradParams {
  C8Geom g;
  int bricks_w, bricks_total, splits;
  int taps2;            // kd * kh accumulators
  int BN, tmem_cols, in_dtype;
  int cin;              // real input channels (<= 8): rows of padded channels are not written
  int stage_bytes, stages, slab_bytes;
  float alpha;
  float* dW;
  long long s_tap, s_k, s_c;   // tap = (a*kh + b)*3 + kw
};

struct C8Shared {
  uint64_t full[6];
  uint64_t empty[6];
  uint64_t done;
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kC8Brick = 64;        // pixels per pipeline stage
constexpr int kC8SlabPix = 80;      // 64 + 16 shifts

__global__ void __launch_bounds__(192, 1)
conv_c8_wgrad_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDy,
                     const C8WgradParams p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ C8Shared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const int S = p.stages;
  const C8Geom& g = p.g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    mbar_init(smem_u32(&sh.done), 1);
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sh.tmem_base), p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  const int split = blockIdx.x;
  const int my_bricks = (p.bricks_total - split + p.splits - 1) / p.splits;

  if (warp == 4) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int b = split; b < p.bricks_total && ok; b += p.splits, ++it) {
        int r = b;
        const int bw = r % p.bricks_w; r /= p.bricks_w;
        const int h = r % g.H; r /= g.H;
        const int d = r % g.Do; r /= g.Do;
        const int n = r;
        const int w0 = bw * kC8Brick;
        const uint32_t s = it % S, ph = (it / S) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.empty[s]), ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutStageEmpty);
          ok = false;
          break;
        }
        const uint32_t sA = smem_base + s * p.stage_bytes;
        const uint32_t sB = sA + p.slab_bytes;
        const uint32_t bar = smem_u32(&sh.full[s]);
        mbar_expect_tx(bar, (uint32_t)(p.taps2 * kC8SlabPix * 16 + kC8Brick * p.BN * 2));
        // x slab: [kd][kh][80 pixels][8 ch]; dy brick: [64 pixels][BN]
        tma_load_4d(sA, &tmX, bar, (w0 - 1) * 2, h - g.ph, d - g.pd, n);   // 8-byte units
        tma_load_5d(sB, &tmDy, bar, 0, w0, h, d, n);
      }
      if (!ok || *abort_flag) {
        const uint32_t pending = it < (uint32_t)S ? it : (uint32_t)S;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t q = it - 1 - j;
          mbar_wait_budget_only(smem_u32(&sh.full[q % S]), (q / S) & 1);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 1, 1, 128, (uint32_t)p.BN);
      const uint32_t b_row = p.BN == 32 ? 64u : 128u;
      const uint32_t b_layout = p.BN == 32 ? kLayoutSw64 : kLayoutSw128;
      uint32_t it = 0;
      bool ok = true;
      for (int b = split; b < p.bricks_total && ok; b += p.splits, ++it) {
        const uint32_t s = it % S, ph = (it / S) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmaFull);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sA = smem_base + s * p.stage_bytes;
        const uint32_t sB = sA + p.slab_bytes;
        for (int t2 = 0; t2 < p.taps2; ++t2) {
          const uint32_t slab = sA + t2 * (kC8SlabPix * 16);
#pragma unroll
          for (int kk = 0; kk < kC8Brick / 16; ++kk) {
            // A (MN-major, un-swizzled): 8 channels contiguous, M blocks (= pixel shifts)
            // 16 B apart (SBO), k rows (= pixels) 16 B apart, 8-pixel groups 128 B apart (LBO)
            const uint64_t ad = make_smem_desc(slab + kk * 256, 128, 16, kLayoutNone);
            const uint64_t bd = make_smem_desc(sB + kk * 16 * b_row, 8192, 8 * b_row, b_layout);
            umma_f16(tmem_base + t2 * p.BN, ad, bd, idesc, (it == 0 && kk == 0) ? 0u : 1u);
          }
        }
        umma_commit(smem_u32(&sh.empty[s]));
      }
      if (ok) umma_commit(smem_u32(&sh.done));
    }
  } else {
    const bool landed =
        my_bricks > 0 &&
        __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&sh.done), 0, abort_flag));
    if (my_bricks > 0 && !landed && lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
    if (landed && warp == 0) {   // rows 0..23 (shifts 0..2) carry the result: warp 0 only
      tc_fence_after();
      const int shift = lane >> 3, ch = lane & 7;
      for (int t2 = 0; t2 < p.taps2; ++t2) {
        for (int c = 0; c < p.BN; c += 32) {
          if (c >= g.Kout) break;
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + t2 * p.BN + c, r);
          tmem_ld_wait();
          if (shift < 3 && ch < p.cin) {
            float* dst = p.dW + (long long)(t2 * 3 + shift) * p.s_tap + ch * p.s_c;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int k = c + j;
              if (k < g.Kout) atomicAdd(dst + k * p.s_k, p.alpha * __uint_as_float(r[j]));
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

}  // namespace lb

extern "C" {

// x: [N][D][H][W][8] (strides xs in elements, pixels dense); w: [kd*kh][4 (kw, kw = 3 zero)]
// [32 (output channel, zero rows beyond Kout)][8 (input channel)]; y: [N][D][H][W][Kout].
// geom: N D H W Kout kd kh pd ph Do (10 ints).  kw = 3, pad_w = 1, stride 1.
int lb_conv_c8_fwd(const void* x, const void* w, void* y, const float* bias, const int* geom,
                   const long long* xs, const long long* ys, int in_dtype, int out_dtype,
                   int act, float act_param, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  C8Geom g;
  memcpy(&g, geom, sizeof(g));
  if (g.Kout > 32 || g.Kout % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -1;
  if (xs[3] != 8 || (g.W & 1)) return -1;   // dense 8-channel pixels, even width
  const int TW = g.W < 128 ? g.W : 128;
  const int half_px = (((TW + 3 + 1) / 2) + 7) / 8 * 8;
  CUtensorMap tmA, tmB;
  {
    // pixels viewed as pairs of 8-byte units: one image row = one TMA row of 2 W units
    uint64_t dims[4] = {(uint64_t)g.W * 2, (uint64_t)g.H, (uint64_t)g.D, (uint64_t)g.N};
    uint64_t strides[3] = {(uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2, (uint64_t)xs[0] * 2};
    uint32_t box[4] = {(uint32_t)(half_px * 2), 1, 1, 1};
    if (!lbhost::encode_tmap(&tmA, kI64, 4, x, dims, strides, box, nullptr, 0)) return -1;
  }
  const int BN = 32;
  {
    // packed filter: [kd*kh][4 k-chunks][32 rows][8 elements] = 2 KB per tap-row
    uint64_t dims[2] = {256, (uint64_t)(g.kd * g.kh)};
    uint64_t strides[1] = {2048};
    uint32_t box[2] = {256, 1};
    if (!lbhost::encode_tmap(&tmB, kI64, 2, w, dims, strides, box, nullptr, 0)) return -1;
  }
#define LB_LAUNCH(BN_)                                                                 \
  {                                                                                    \
    ConvC8FwdPolicy<BN_>::Params p;                                                    \
    p.g = g; p.TW = TW; p.half_px = half_px; p.tiles_w = (g.W + TW - 1) / TW;                             \
    p.num_tiles = p.tiles_w * g.H * g.Do * g.N; p.k_iters = g.kd * g.kh;                \
    p.in_dtype = in_dtype;                                                             \
    p.o_sn = ys[0]; p.o_sd = ys[1]; p.o_sh = ys[2]; p.o_sw = ys[3];                    \
    p.epi.C = y; p.epi.bias = bias; p.epi.alpha = 1.f; p.epi.beta = 0.f;               \
    p.epi.out_dtype = out_dtype; p.epi.bias_mode = bias ? 1 : 0; p.epi.act = act;      \
    p.epi.act_param = act_param; p.epi.ldc = ys[3];                                    \
    return launch_c8_fwd<BN_>(tmA, tmB, p, stream);                                    \
  }
  (void)BN;
  LB_LAUNCH(32)
#undef LB_LAUNCH
}

// dW element (tap = (a*kh + b)*3 + kw, k, c) at tap*s_tap + k*s_k + c*s_c; ADDS alpha * grad.
// Requires W % 64 == 0 is NOT needed (edges are zero-filled), Kout in {32, 64}-ish (<= 64, % 8).
int lb_conv_c8_wgrad(const void* x, const void* dy, float* dW, const int* geom,
                     const long long* xs, const long long* ys, long long s_tap, long long s_k,
                     long long s_c, int cin, int in_dtype, float alpha, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  C8WgradParams p;
  memcpy(&p.g, geom, sizeof(C8Geom));
  p.cin = cin < 8 ? cin : 8;
  const C8Geom& g = p.g;
  if (g.Kout > 64 || g.Kout % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15)) return -1;
  p.taps2 = g.kd * g.kh;
  p.BN = g.Kout > 32 ? 64 : 32;
  if (p.taps2 * p.BN > 512) return -1;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.taps2 * p.BN) p.tmem_cols *= 2;
  p.slab_bytes = ((p.taps2 * kC8SlabPix * 16) + 1023) & ~1023;
  p.stage_bytes = p.slab_bytes + kC8Brick * p.BN * 2;
  p.stages = 200 * 1024 / p.stage_bytes;
  if (p.stages > 6) p.stages = 6;
  p.bricks_w = (g.W + kC8Brick - 1) / kC8Brick;
  p.bricks_total = p.bricks_w * g.H * g.Do * g.N;
  int splits = lbhost::sm_count();
  if (splits > p.bricks_total) splits = p.bricks_total;
  p.splits = splits;
  p.in_dtype = in_dtype;
  p.alpha = alpha;
  p.dW = dW;
  p.s_tap = s_tap; p.s_k = s_k; p.s_c = s_c;
  CUtensorMap tmX, tmDy;
  {
    if (xs[3] != 8) return -1;
    uint64_t dims[4] = {(uint64_t)g.W * 2, (uint64_t)g.H, (uint64_t)g.D, (uint64_t)g.N};
    uint64_t strides[3] = {(uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2, (uint64_t)xs[0] * 2};
    uint32_t box[4] = {(uint32_t)kC8SlabPix * 2, (uint32_t)g.kh, (uint32_t)g.kd, 1};
    if (!lbhost::encode_tmap(&tmX, kI64, 4, x, dims, strides, box, nullptr, 0)) return -1;
  }
  {
    uint64_t dims[5] = {(uint64_t)g.Kout, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.Do, (uint64_t)g.N};
    uint64_t strides[4] = {(uint64_t)ys[3] * 2, (uint64_t)ys[2] * 2, (uint64_t)ys[1] * 2,
                           (uint64_t)ys[0] * 2};
    uint32_t box[5] = {(uint32_t)p.BN, (uint32_t)kC8Brick, 1, 1, 1};
    if (!lbhost::encode_tmap(&tmDy, in_dtype, 5, dy, dims, strides, box, nullptr, p.BN * 2)) return -1;
  }
  const int smem = p.stages * p.stage_bytes + 1024;
  static int configured_smem = 0;
  if (smem > configured_smem) {
    cudaFuncSetAttribute(conv_c8_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured_smem = smem;
  }
  conv_c8_wgrad_kernel<<<p.splits, 192, smem, stream>>>(tmX, tmDy, p, lbhost::status_word());
  return (int)cudaGetLastError();
}

}  // extern "C"
