// tcgen05 implicit-GEMM convolution (1-D/2-D/3-D, stride, dilation) on channels-last
// tensors.  Activations are [N][D][H][W][C] (2-D uses D = 1), filters are
// [tap][Kout][C] with tap = (kd*KH + kh)*KW + kw.
//
// The GEMM view: rows = 128 output pixels of a (TN x TD x TH x TW) brick, columns =
// output channels, reduction = taps x input channels.  For every (tap, channel block)
// the producer issues ONE 5-D TMA box load whose origin is the brick origin shifted by
// the tap offset; out-of-range coordinates are zero-filled by the TMA unit, which is
// the convolution padding.  Strided convolutions use the tensor map's element strides.
// The same kernel computes the data gradient of a stride-1 convolution when it is
// given dy, the tap-flipped / channel-transposed filter and padding dil*(k-1)-pad.
//
// Stands in for the cuDNN calls of the reference's base_convolution layer
// (src/layers/learning/base_convolution.cpp:462-814).
#include "conv_geom.cuh"
#include "tc_pipeline.cuh"
#include <algorithm>

namespace lb {

template <int BN_>
struct ConvFwdPolicy {
  static constexpr int BN = BN_;
  static constexpr int kEpiGroups = 2;       // two tiles' epilogues in flight (tc_pipeline.cuh)
  using G = StageGeom<BN>;

  struct Params {
    ConvGeom g;
    int TW, TH, TD, TN, rows_used;
    int tiles_w, tiles_h, tiles_d, tiles_nb, tiles_col;
    int Cb, cblocks, slices, slices_per_stage, layout_type;
    int num_tiles, k_iters, in_dtype;
    long long o_sn, o_sd, o_sh, o_sw;  // output strides in elements
    // divisions by run-time values as multiply-high (the producer and the MMA issuer are
    // single threads: a plain division costs them 100+ cycles)
    FastDiv fd_tiles_col, fd_tiles_w, fd_tiles_h, fd_tiles_d, fd_cblocks, fd_khw, fd_kw;
    FastDiv fd_TW, fd_TH, fd_TD;
    EpiParams epi;
    HaloSync hs;                       // halo exchange with the depth neighbours (distconv)
  };
  struct Tile {
    int n0, d0, h0, w0, col0;
  };
  using HasHalo = void;
  __device__ static const HaloSync& halo(const Params& p) { return p.hs; }
  __device__ static int tile_halo(const Params& p, const Tile& tl) {
    // input planes of the brick: [d0 * sd - pd, (d0 + TD - 1) * sd - pd + (kd - 1) * dd]
    const int lo = tl.d0 * p.g.sd - p.g.pd;
    const int hi = (tl.d0 + p.TD - 1) * p.g.sd - p.g.pd + (p.g.kd - 1) * p.g.dd;
    return (lo < (int)p.hs.h ? 1 : 0) | (hi >= (int)(p.hs.h + p.hs.dl) ? 2 : 0);
  }

  __device__ static Tile decode(const Params& p, int t) {
    Tile tl;
    uint32_t r = (uint32_t)t, ucb, utw, uth, utd;
    p.fd_tiles_col.divmod(r, r, ucb);
    p.fd_tiles_w.divmod(r, r, utw);
    p.fd_tiles_h.divmod(r, r, uth);
    p.fd_tiles_d.divmod(r, r, utd);
    const int cb = (int)ucb, tw = (int)utw, th = (int)uth;
    int td = (int)utd;
    if (p.hs.enabled) td = halo_rotate(td, p.tiles_d);   // the brick that needs the top halo goes last
    tl.col0 = cb * BN;
    tl.w0 = tw * p.TW; tl.h0 = th * p.TH; tl.d0 = td * p.TD; tl.n0 = (int)r * p.TN;
    return tl;
  }
  __device__ static int slices_in(const Params& p, int k) {
    const int rem = p.slices - k * p.slices_per_stage;
    return rem < p.slices_per_stage ? rem : p.slices_per_stage;
  }
  __device__ static uint32_t stage_bytes(const Params& p, const Tile&, int k) {
    return (uint32_t)slices_in(p, k) * (uint32_t)((p.rows_used + BN) * p.Cb * 2);
  }
  __device__ static void load(const Params& p, const Tile& tl, int k, uint32_t sA, uint32_t sB,
                              uint32_t bar, const CUtensorMap* tmA, const CUtensorMap* tmB,
                              int lane) {
    const ConvGeom& g = p.g;
    const int ns = slices_in(p, k);
    // lane 2j issues the activation box of slice j, lane 2j+1 its filter box
    const int j = lane >> 1;
    if (j >= ns) return;
    const int sl = k * p.slices_per_stage + j;
    const int tap = (int)p.fd_cblocks.div((uint32_t)sl);
    const int c0 = (sl - tap * p.cblocks) * p.Cb;
    if ((lane & 1) == 0) {
      uint32_t ua, rem, ub, uc;
      p.fd_khw.divmod((uint32_t)tap, ua, rem);
      p.fd_kw.divmod(rem, ub, uc);
      const int a = (int)ua, b = (int)ub, c = (int)uc;
      tma_load_5d(sA + j * (kBM * p.Cb * 2), tmA, bar, c0,
                  tl.w0 * g.sw - g.pw + c * g.dw,
                  tl.h0 * g.sh - g.ph + b * g.dh,
                  tl.d0 * g.sd - g.pd + a * g.dd, tl.n0);
    } else {
      tma_load_3d(sB + j * (BN * p.Cb * 2), tmB, bar, c0, tl.col0, tap);
    }
  }
  __device__ static uint32_t idesc(const Params& p) {
    return make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 0, 0, kBM, BN);
  }
  __device__ static void mma(const Params& p, int k, uint32_t sA, uint32_t sB, uint32_t tmem_acc,
                             uint32_t idesc, bool first) {
    // A stage holds 64 / Cb slices of Cb channels: four MMAs of K = 16 whatever Cb is.  MMA i
    // reads slice i / (Cb / 16), K step i % (Cb / 16); descriptors differ in the low word.
    const int ns = slices_in(p, k);
    const uint64_t d0 = make_smem_desc(0, 16, 8u * p.Cb * 2u, p.layout_type);
    const uint32_t hi = (uint32_t)(d0 >> 32);
    const uint32_t a_lo = (uint32_t)d0 + (sA >> 4), b_lo = (uint32_t)d0 + (sB >> 4);
    const uint32_t a_slice = (uint32_t)(kBM * p.Cb * 2) >> 4, b_slice = (uint32_t)(BN * p.Cb * 2) >> 4;
    const int per = p.Cb >> 4;                    // MMAs per slice: 4, 2 or 1
    const int sh = per == 4 ? 2 : (per == 2 ? 1 : 0);
    const int count = ns * per;
    uint32_t acc = first ? 0u : 1u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < count) {
        const uint32_t j = (uint32_t)i >> sh, kk = (uint32_t)i & (uint32_t)(per - 1);
        umma_f16_lo(tmem_acc, a_lo + j * a_slice + 2 * kk, hi, b_lo + j * b_slice + 2 * kk, hi, idesc, acc);
        acc = 1u;
      }
    }
  }
  __device__ static bool row_addr(const Params& p, const Tile& tl, int row, long long& off) {
    uint32_t r = (uint32_t)row, utw, uth, utd;
    p.fd_TW.divmod(r, r, utw);
    p.fd_TH.divmod(r, r, uth);
    p.fd_TD.divmod(r, r, utd);
    const int tw = (int)utw, th = (int)uth, td = (int)utd;
    const int n = tl.n0 + (int)r, d = tl.d0 + td, h = tl.h0 + th, w = tl.w0 + tw;
    off = n * p.o_sn + d * p.o_sd + h * p.o_sh + w * p.o_sw;
    return row < p.rows_used && n < p.g.N && d < p.g.Do && h < p.g.Ho && w < p.g.Wo;
  }
  __device__ static int row_index(const Params&, const Tile&, int row) { return row; }
  __device__ static int col0(const Params&, const Tile& tl) { return tl.col0; }
  __device__ static int ncols(const Params& p) { return p.g.Kout; }
};

static int largest_tile(int extent, int limit) {
  // Largest tile <= limit along a dimension: the whole extent if it fits, otherwise the
  // largest divisor of the extent unless that wastes more than half of the limit.
  if (extent <= limit) return extent;
  int best = 1;
  for (int t = limit; t >= 1; --t)
    if (extent % t == 0) { best = t; break; }
  return best * 2 > limit ? best : limit;
}

template <int BN>
static int launch_conv(const CUtensorMap& tmA, const CUtensorMap& tmB,
                       typename ConvFwdPolicy<BN>::Params p, const lbhost::SplitKOffer& offer,
                       cudaStream_t stream) {
  using P = ConvFwdPolicy<BN>;
  using G = StageGeom<BN>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(tc_persistent_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         G::kSmemBytes);
    configured = true;
  }
  p.tiles_col = (p.g.Kout + BN - 1) / BN;
  p.num_tiles = p.tiles_col * p.tiles_w * p.tiles_h * p.tiles_d * p.tiles_nb;
  {
    const long long dmax = std::max({p.tiles_col, p.tiles_w, p.tiles_h, p.tiles_d, 128});
    if ((long long)p.num_tiles * dmax >= (1ll << 32)) return -1;   // range of the fast divisions
  }
  p.fd_tiles_col = FastDiv((uint32_t)p.tiles_col);
  p.fd_tiles_w = FastDiv((uint32_t)p.tiles_w);
  p.fd_tiles_h = FastDiv((uint32_t)p.tiles_h);
  p.fd_tiles_d = FastDiv((uint32_t)p.tiles_d);
  p.fd_cblocks = FastDiv((uint32_t)p.cblocks);
  p.fd_khw = FastDiv((uint32_t)(p.g.kh * p.g.kw));
  p.fd_kw = FastDiv((uint32_t)p.g.kw);
  p.fd_TW = FastDiv((uint32_t)p.TW);
  p.fd_TH = FastDiv((uint32_t)p.TH);
  p.fd_TD = FastDiv((uint32_t)p.TD);
  // few bricks, long reduction (the deep layers of a network on a small batch): split it
  p.epi.k_splits = lbhost::plan_splitk(offer, p.num_tiles, p.k_iters, BN);
  p.epi.sk_ws = offer.ws;
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

// Forward convolution / stride-1 data gradient.
//   x: [N][D][H][W][C] with element strides (xs_n, xs_d, xs_h, xs_w), C contiguous
//   w: [taps][Kout][C] contiguous, same dtype as x
//   y: [N][Do][Ho][Wo][Kout] with element strides (ys_*), Kout contiguous (ldc = ys_w)
// geom: 21 ints = N D H W C Do Ho Wo Kout kd kh kw pd ph pw sd sh sw dd dh dw
int lb_conv_fwd_halo_tc(const void* x, const void* w, void* y, const float* bias, const int* geom,
                        const long long* xs, const long long* ys, int in_dtype, int out_dtype,
                        float alpha, float beta, int act, float act_param, const void* halo,
                        void* stream_);

int lb_conv_fwd_tc(const void* x, const void* w, void* y, const float* bias, const int* geom,
                   const long long* xs, const long long* ys, int in_dtype, int out_dtype,
                   float alpha, float beta, int act, float act_param, void* stream_) {
  return lb_conv_fwd_halo_tc(x, w, y, bias, geom, xs, ys, in_dtype, out_dtype, alpha, beta, act,
                             act_param, nullptr, stream_);
}

// `halo` (optional): a HaloSyncArgs.  x is then this rank's extended tensor
// [N][Dl + 2h][H][W][C] in symmetric memory (dense planes, pd == 0): the kernel sends the
// boundary planes to the depth neighbours itself and waits for theirs before the first tile
// that reads a halo plane.
int lb_conv_fwd_halo_tc(const void* x, const void* w, void* y, const float* bias, const int* geom,
                        const long long* xs, const long long* ys, int in_dtype, int out_dtype,
                        float alpha, float beta, int act, float act_param, const void* halo,
                        void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const lbhost::SplitKOffer offer = lbhost::take_splitk_offer();   // holds for this call only
  ConvGeom g;
  static_assert(sizeof(ConvGeom) == 21 * sizeof(int), "geom layout");
  memcpy(&g, geom, sizeof(g));
  if (g.C % 8 != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -1;
  for (int i = 0; i < 4; ++i)
    if (xs[i] % 8) return -1;

  // Stride-1 convolutions whose whole filter fits in shared memory take the halo-slab
  // kernel: one TMA box per (tile, filter plane) instead of one per tap.
  {
    const int rc = lb_conv_slab_fwd(x, w, y, bias, geom, xs, ys, in_dtype, out_dtype, alpha, beta,
                                    act, act_param, halo, stream_);
    if (rc != -2) return rc;
  }

  const int Cb = g.C >= 64 ? 64 : (g.C >= 32 ? 32 : 16);
  const int TW = largest_tile(g.Wo, 128);
  const int TH = largest_tile(g.Ho, 128 / TW);
  const int TD = largest_tile(g.Do, 128 / (TW * TH));
  const int TN = largest_tile(g.N, 128 / (TW * TH * TD));
  const uint32_t bw = (TW - 1) * g.sw + 1, bh = (TH - 1) * g.sh + 1, bd = (TD - 1) * g.sd + 1;
  if (bw > 256 || bh > 256 || bd > 256) return -1;

  HaloSync hsync;
  if (halo && (g.pd != 0 || xs[3] != g.C || xs[2] != (long long)g.W * g.C ||
               xs[1] != (long long)g.H * g.W * g.C)) return -1;
  if (!make_halo_sync(hsync, reinterpret_cast<const HaloSyncArgs*>(halo), x, g.N, g.D,
                      (long long)g.H * g.W * g.C * 2, xs[0] * 2)) return -1;

  CUtensorMap tmA, tmB;
  {
    uint64_t dims[5] = {(uint64_t)g.C, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.D, (uint64_t)g.N};
    uint64_t strides[4] = {(uint64_t)xs[3] * 2, (uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2,
                           (uint64_t)xs[0] * 2};
    uint32_t box[5] = {(uint32_t)Cb, bw, bh, bd, (uint32_t)TN};
    uint32_t es[5] = {1, (uint32_t)g.sw, (uint32_t)g.sh, (uint32_t)g.sd, 1};
    if (!lbhost::encode_tmap(&tmA, in_dtype, 5, x, dims, strides, box, es, Cb * 2)) return -1;
  }
  int BN = g.Kout > 128 ? 256 : (g.Kout > 64 ? 128 : (g.Kout > 32 ? 64 : 32));
  {
    const int taps = g.kd * g.kh * g.kw;
    uint64_t dims[3] = {(uint64_t)g.C, (uint64_t)g.Kout, (uint64_t)taps};
    uint64_t strides[2] = {(uint64_t)g.C * 2, (uint64_t)g.C * g.Kout * 2};
    uint32_t box[3] = {(uint32_t)Cb, (uint32_t)BN, 1};
    if (!lbhost::encode_tmap(&tmB, in_dtype, 3, w, dims, strides, box, nullptr, Cb * 2)) return -1;
  }

#define LB_LAUNCH(BN_)                                                                   \
  {                                                                                      \
    ConvFwdPolicy<BN_>::Params p;                                                        \
    p.g = g; p.TW = TW; p.TH = TH; p.TD = TD; p.TN = TN; p.rows_used = TW * TH * TD * TN; \
    p.tiles_w = (g.Wo + TW - 1) / TW; p.tiles_h = (g.Ho + TH - 1) / TH;                  \
    p.tiles_d = (g.Do + TD - 1) / TD; p.tiles_nb = (g.N + TN - 1) / TN;                  \
    p.Cb = Cb; p.cblocks = (g.C + Cb - 1) / Cb;                                          \
    p.slices = g.kd * g.kh * g.kw * p.cblocks; p.slices_per_stage = 64 / Cb;             \
    p.layout_type = Cb == 64 ? kLayoutSw128 : (Cb == 32 ? kLayoutSw64 : kLayoutSw32);    \
    p.k_iters = (p.slices + p.slices_per_stage - 1) / p.slices_per_stage;                \
    p.in_dtype = in_dtype;                                                               \
    p.o_sn = ys[0]; p.o_sd = ys[1]; p.o_sh = ys[2]; p.o_sw = ys[3];                      \
    p.epi.C = y; p.epi.bias = bias; p.epi.alpha = alpha; p.epi.beta = beta;              \
    p.epi.out_dtype = out_dtype; p.epi.bias_mode = bias ? 1 : 0; p.epi.act = act;        \
    p.epi.act_param = act_param; p.epi.ldc = ys[3];                                      \
    p.hs = hsync;                                                                        \
    return launch_conv<BN_>(tmA, tmB, p, offer, stream);                                      \
  }
  if (BN == 256) LB_LAUNCH(256)
  if (BN == 128) LB_LAUNCH(128)
  if (BN == 64) LB_LAUNCH(64)
  LB_LAUNCH(32)
#undef LB_LAUNCH
}

}  // extern "C"
