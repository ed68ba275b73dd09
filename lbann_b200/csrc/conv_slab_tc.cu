// Halo-slab forward convolution (stride 1, no dilation) for filters that fit in shared
// memory: 3x3x3 convolutions with few channels on large images, where the implicit-GEMM
// kernel of conv_tc.cu is bound by the ~300 cycles that every TMA box costs its issuer.
//
// Output pixels of one image plane are numbered along a PADDED row pitch
// Wp = Wo + kw - 1:  q = h * Wp + w.  A tile is 128 consecutive q (rows with w >= Wo or
// h >= Ho are computed and thrown away, a loss of (kw - 1) / Wp).  For filter plane `a`
// the tile needs input rows l0 - ph .. l0 - ph + nl - 1 (l0 = first output row of the
// tile) and all Wp columns starting at -pw: ONE 5-D TMA box {Cb, Wp, nl, 1, 1}, whose
// out-of-range parts the copy engine fills with zeros (the padding).  In that slab the
// operand row of output q for tap (b, c) is  (q - l0 * Wp) + b * Wp + c : every tap is
// the same matrix at a different start row, so the kh * kw taps of a plane are UMMA
// descriptors into one slab and a tile costs kd * cblocks boxes instead of
// kd * kh * kw * cblocks * 2.  The filter ([tap][Kout][C], all taps) is loaded once per
// CTA.  The swizzle of both operands is a function of the absolute shared-memory
// address, so shifting an operand by whole rows keeps it consistent with what TMA wrote.
//
// Also computes the data gradient of such a convolution (tap-flipped, channel-
// transposed filter and padding k - 1 - pad), like the kernel it stands in for.
// Reference counterpart: the cuDNN calls of src/layers/learning/base_convolution.cpp:462-814.
#include "conv_geom.cuh"
#include "halo_sync.cuh"
#include "tc_pipeline.cuh"

namespace lb {

constexpr int kSlabMaxStages = 8;

struct SlabParams {
  ConvGeom g;
  int Wp, nl;                 // padded row pitch, input rows per slab
  int tiles_plane, num_tiles; // tiles per output plane, total
  int Cb, cblocks, layout_type, taps;
  int slab_bytes, stage_bytes, stages, filter_bytes;
  int in_dtype;
  long long o_sn, o_sd, o_sh, o_sw;
  FastDiv fd_tiles_plane, fd_Do, fd_Wp;   // tile decode without run-time divisions
  EpiParams epi;
  HaloSync hs;                // halo exchange with the depth neighbours inside this kernel
};

struct SlabShared {
  uint64_t full[kSlabMaxStages];
  uint64_t empty[kSlabMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t filter_ready;
  uint32_t tmem_base;
  int abort_flag;
};

// The MMAs of one filter plane on one slab, straight-line: with loops over run-time tap counts
// the issuing thread spent ~90-120 cycles per tcgen05.mma on counters and branches, twice what
// the instruction takes to execute at N <= 64 (48 cycles); unrolled it issues at that rate.
template <int KSTEPS, int KH, int KW>
__device__ __forceinline__ void slab_issue_plane(uint32_t tmem_acc, uint32_t a_line, uint32_t bd,
                                                 uint32_t line_step, uint32_t pix_step,
                                                 uint32_t tap_step, uint32_t d_hi, uint32_t idesc,
                                                 uint32_t& accum) {
#pragma unroll
  for (int b = 0; b < KH; ++b) {
#pragma unroll
    for (int c = 0; c < KW; ++c) {
      const uint32_t ad = a_line + b * line_step + c * pix_step;
      const uint32_t bt = bd + (b * KW + c) * tap_step;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        umma_f16_lo(tmem_acc, ad + 2 * kk, d_hi, bt + 2 * kk, d_hi, idesc, accum);
        accum = 1u;
      }
    }
  }
}

constexpr int kSlabThreads = 64 + 2 * 128;     // 8 epilogue warps, producer, MMA issuer

template <int BN>
__global__ void __launch_bounds__(kSlabThreads, 1)
conv_slab_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                 const SlabParams p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ SlabShared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_filter = smem_base;
  const uint32_t s_stage0 = smem_base + p.filter_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const int S = p.stages;
  const ConvGeom& g = p.g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&sh.tmem_full[a]), 1);
      mbar_init(smem_u32(&sh.tmem_empty[a]), 4);
    }
    mbar_init(smem_u32(&sh.filter_ready), 1);
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sh.tmem_base), 2 * BN < 32 ? 32 : 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  const HaloSync& hs = p.hs;

  if (hs.enabled && warp < 4) {
    // the epilogue warps have nothing to do until the first accumulator is complete: they
    // send this rank's boundary planes to the neighbours meanwhile
    halo_push(hs, threadIdx.x, 128, blockIdx.x, gridDim.x);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 0) halo_signal(hs);
  }

  if (warp == 4) {
    if (lane == 0) {
      // filter: one box per channel block, [cblock][tap][BN rows][Cb]
      const uint32_t fbar = smem_u32(&sh.filter_ready);
      mbar_expect_tx(fbar, (uint32_t)p.filter_bytes);
      for (int j = 0; j < p.cblocks; ++j)
        tma_load_3d(s_filter + j * (p.filter_bytes / p.cblocks), &tmW, fbar, j * p.Cb, 0, 0);
      uint32_t it = 0;
      bool ok = true;
      // halo planes: input planes [0, h) come from the rank above, [h + dl, dl + 2h) from below
      const uint32_t halo_target =
          hs.enabled ? (*reinterpret_cast<volatile uint32_t*>(hs.local) + 1u) * gridDim.x : 0u;
      bool top_ok = !hs.enabled || hs.top_flag == nullptr;
      bool bot_ok = !hs.enabled || hs.bot_flag == nullptr;
      RingPos rp;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        uint32_t ti, r, dd, nn;
        p.fd_tiles_plane.divmod((uint32_t)t, r, ti);
        p.fd_Do.divmod(r, nn, dd);
        const int d = hs.enabled ? halo_rotate((int)dd, g.Do) : (int)dd, n = (int)nn;
        const int l0 = (int)p.fd_Wp.div(ti * 128u);
        for (int a = 0; a < g.kd && ok; ++a) {
          const int plane_in = d - g.pd + a;
          if (!top_ok && plane_in < hs.h) {
            top_ok = halo_wait(hs.top_flag, halo_target, status, abort_flag);
            if (!top_ok) { ok = false; break; }
          }
          if (!bot_ok && plane_in >= hs.h + hs.dl) {
            bot_ok = halo_wait(hs.bot_flag, halo_target, status, abort_flag);
            if (!bot_ok) { ok = false; break; }
          }
          for (int j = 0; j < p.cblocks; ++j, ++it) {
            const uint32_t s = rp.s;
            if (!mbar_wait_bounded(smem_u32(&sh.empty[s]), rp.ph ^ 1, abort_flag)) {
              raise_status(status, abort_flag, kTimeoutStageEmpty);
              ok = false;
              break;
            }
            const uint32_t bar = smem_u32(&sh.full[s]);
            mbar_expect_tx(bar, (uint32_t)p.slab_bytes);
            tma_load_5d(s_stage0 + s * p.stage_bytes, &tmX, bar, j * p.Cb, -g.pw, l0 - g.ph,
                        d - g.pd + a, n);
            rp.advance((uint32_t)S);
          }
        }
      }
      if (!ok || *abort_flag) {
        const uint32_t pending = it < (uint32_t)S ? it : (uint32_t)S;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t q = it - 1 - j;
          mbar_wait_budget_only(smem_u32(&sh.full[q % S]), (q / S) & 1);
        }
        mbar_wait_budget_only(smem_u32(&sh.filter_ready), 0);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // Everything between two tcgen05.mma of this loop is on the critical path of the CTA
      // (one thread issues all of them): descriptors differ in the start-address field of
      // their low word only, and the tap offsets are running sums.
      const uint32_t idesc = make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 0, 0, 128, BN);
      const uint32_t row_bytes = p.Cb * 2;
      const uint64_t desc0 = make_smem_desc(0, 16, 8 * row_bytes, p.layout_type);
      const uint32_t d_lo = (uint32_t)desc0, d_hi = (uint32_t)(desc0 >> 32);
      const uint32_t tap_step = (BN * row_bytes) >> 4;            // one tap of the filter
      const uint32_t pix_step = row_bytes >> 4;                   // one pixel along a row
      const uint32_t line_step = ((uint32_t)p.Wp * row_bytes) >> 4;   // one image row in the slab
      const uint32_t fblock = ((uint32_t)p.filter_bytes / (uint32_t)p.cblocks) >> 4;
      const uint32_t plane_step = (uint32_t)(g.kh * g.kw) * tap_step;
      const uint32_t stage_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t ksteps = (uint32_t)p.Cb / 16u;
      const uint32_t kh = (uint32_t)g.kh, kw = (uint32_t)g.kw, kd = (uint32_t)g.kd;
      const uint32_t cblocks = (uint32_t)p.cblocks;
      const bool plane33 = kh == 3 && kw == 3;
      bool ok = mbar_wait_bounded(smem_u32(&sh.filter_ready), 0, abort_flag);
      if (!ok) raise_status(status, abort_flag, kTimeoutTmaFull);
      uint32_t lt = 0;
      RingPos rp;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x, ++lt) {
        uint32_t ti, r;
        p.fd_tiles_plane.divmod((uint32_t)t, r, ti);
        const uint32_t q0 = ti * 128u;
        const uint32_t row0 = q0 - p.fd_Wp.div(q0) * (uint32_t)p.Wp;   // first operand row in the slab
        const uint32_t acc = lt & 1, acc_ph = (lt >> 1) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.tmem_empty[acc]), acc_ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmemEmpty);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * BN;
        const uint32_t a_tile = d_lo + ((s_stage0 + row0 * row_bytes) >> 4);
        uint32_t accum = 0;
        uint32_t b_plane = d_lo + (s_filter >> 4);
        for (uint32_t a = 0; a < kd && ok; ++a, b_plane += plane_step) {
          uint32_t b_blk = b_plane;
          for (uint32_t j = 0; j < cblocks; ++j, b_blk += fblock) {
            if (!mbar_wait_bounded(smem_u32(&sh.full[rp.s]), rp.ph, abort_flag)) {
              raise_status(status, abort_flag, kTimeoutTmaFull);
              ok = false;
              break;
            }
            tc_fence_after();
            uint32_t a_line = a_tile + rp.s * stage_step;
            uint32_t bd = b_blk;
            if (plane33 && ksteps == 2) {
              slab_issue_plane<2, 3, 3>(tmem_acc, a_line, bd, line_step, pix_step, tap_step, d_hi, idesc, accum);
            } else if (plane33 && ksteps == 4) {
              slab_issue_plane<4, 3, 3>(tmem_acc, a_line, bd, line_step, pix_step, tap_step, d_hi, idesc, accum);
            } else if (plane33 && ksteps == 1) {
              slab_issue_plane<1, 3, 3>(tmem_acc, a_line, bd, line_step, pix_step, tap_step, d_hi, idesc, accum);
            } else {
              for (uint32_t b = 0; b < kh; ++b, a_line += line_step) {
                uint32_t ad = a_line;
                for (uint32_t c = 0; c < kw; ++c, ad += pix_step, bd += tap_step) {
                  for (uint32_t kk = 0; kk < ksteps; ++kk) {
                    umma_f16_lo(tmem_acc, ad + 2 * kk, d_hi, bd + 2 * kk, d_hi, idesc, accum);
                    accum = 1u;
                  }
                }
              }
            }
            umma_commit(smem_u32(&sh.empty[rp.s]));
            rp.advance((uint32_t)S);
          }
        }
        if (ok) umma_commit(smem_u32(&sh.tmem_full[acc]));
      }
    }
  } else {
    // Two epilogue groups of four warps (warps 0-3 and 6-9), one per accumulator: group eg
    // drains this CTA's tiles eg, eg + 2, ...  With a single warp per scheduler the epilogue
    // of a tile (TMEM load, conversion, row stores) shows its full latency and outlasts the
    // tile's MMAs for layers with few input channels; two tiles in flight hide it.
    const int eg = warp >= 6 ? 1 : 0;
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may read
    uint32_t use = 0;
    const EpiParams& e = p.epi;
    for (long long tl = (long long)blockIdx.x + (long long)eg * gridDim.x; tl < p.num_tiles;
         tl += 2ll * gridDim.x, ++use) {
      const int t = (int)tl;
      uint32_t ti, r, dd, nn;
      p.fd_tiles_plane.divmod((uint32_t)t, r, ti);
      p.fd_Do.divmod(r, nn, dd);
      const int d = hs.enabled ? halo_rotate((int)dd, g.Do) : (int)dd, n = (int)nn;
      const uint32_t acc = (uint32_t)eg, acc_ph = use & 1u;
      const bool landed = __all_sync(
          0xffffffffu, mbar_wait_bounded(smem_u32(&sh.tmem_full[acc]), acc_ph, abort_flag));
      if (!landed) {
        if (lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
        break;
      }
      tc_fence_after();
      const int row = quarter * 32 + lane;
      const uint32_t q = ti * 128u + (uint32_t)row;
      const int h = (int)p.fd_Wp.div(q), w = (int)q - h * p.Wp;
      const long long row_off = n * p.o_sn + d * p.o_sd + h * p.o_sh + (long long)w * p.o_sw;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      tc_epilogue_rows<BN>(TmemSrc{taddr}, h < g.Ho && w < g.Wo, row_off, 0, g.Kout, row, e);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[acc]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (hs.enabled && threadIdx.x == 0) halo_finish(hs, gridDim.x);
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN < 32 ? 32 : 2 * BN);
  }
}

template <int BN>
static int launch_slab(const CUtensorMap& tmX, const CUtensorMap& tmW, const SlabParams& p,
                       int smem, cudaStream_t stream) {
  static int configured = 0;
  if (configured < smem) {
    cudaFuncSetAttribute(conv_slab_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = smem;
  }
  const int grid = p.num_tiles < lbhost::sm_count() ? p.num_tiles : lbhost::sm_count();
  conv_slab_kernel<BN><<<grid, kSlabThreads, smem, stream>>>(tmX, tmW, p, lbhost::status_word());
  return (int)cudaGetLastError();
}

}  // namespace lb

extern "C" int lb_conv_slab_fwd(const void* x, const void* w, void* y, const float* bias,
                                const int* geom, const long long* xs, const long long* ys,
                                int in_dtype, int out_dtype, float alpha, float beta, int act,
                                float act_param, const void* halo, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  SlabParams p;
  memcpy(&p.g, geom, sizeof(ConvGeom));
  const ConvGeom& g = p.g;
  if (g.sd != 1 || g.sh != 1 || g.sw != 1 || g.dd != 1 || g.dh != 1 || g.dw != 1) return -2;
  if (g.Kout > 128 || g.C % 16) return -2;
  p.Cb = g.C % 64 == 0 ? 64 : (g.C % 32 == 0 ? 32 : 16);
  p.cblocks = g.C / p.Cb;
  p.layout_type = p.Cb == 64 ? kLayoutSw128 : (p.Cb == 32 ? kLayoutSw64 : kLayoutSw32);
  p.taps = g.kd * g.kh * g.kw;
  const int BN = g.Kout > 64 ? 128 : (g.Kout > 32 ? 64 : 32);
  p.filter_bytes = p.cblocks * p.taps * BN * p.Cb * 2;
  p.filter_bytes = (p.filter_bytes + 1023) & ~1023;
  p.Wp = g.Wo + g.kw - 1;
  // Worth it only where rows are long (little waste) and images big enough to amortise
  // the filter load; TMA boxes are limited to 256 elements per dimension.
  if (p.Wp > 256 || g.Wo < 24 || g.kw * g.kh < 2) return -2;
  p.nl = (p.Wp - 1 + 127) / p.Wp + 1 + (g.kh - 1);
  if (p.nl > 256 || p.taps > 256) return -2;
  p.slab_bytes = p.nl * p.Wp * p.Cb * 2;
  // operand rows may run (kw - 1) rows past the slab for discarded outputs: keep them inside
  p.stage_bytes = (p.slab_bytes + g.kw * p.Cb * 2 + 1023) & ~1023;
  const int budget = 224 * 1024 - p.filter_bytes;
  if (budget < 2 * p.stage_bytes) return -2;
  p.stages = budget / p.stage_bytes;
  if (p.stages > kSlabMaxStages) p.stages = kSlabMaxStages;
  p.tiles_plane = (g.Ho * p.Wp + 127) / 128;
  p.num_tiles = p.tiles_plane * g.Do * g.N;
  if ((long long)p.num_tiles * p.tiles_plane >= (1ll << 32) || (long long)p.num_tiles * g.Do >= (1ll << 32))
    return -2;                      // beyond the exact range of the multiply-high divisions
  p.fd_tiles_plane = FastDiv((uint32_t)p.tiles_plane);
  p.fd_Do = FastDiv((uint32_t)g.Do);
  p.fd_Wp = FastDiv((uint32_t)p.Wp);
  p.in_dtype = in_dtype;
  p.o_sn = ys[0]; p.o_sd = ys[1]; p.o_sh = ys[2]; p.o_sw = ys[3];
  p.epi.C = y; p.epi.bias = bias; p.epi.alpha = alpha; p.epi.beta = beta;
  p.epi.out_dtype = out_dtype; p.epi.bias_mode = bias ? 1 : 0; p.epi.act = act;
  p.epi.act_param = act_param; p.epi.ldc = ys[3];
  if (halo && (g.pd != 0 || xs[2] != (long long)g.W * g.C || xs[3] != g.C)) return -1;
  if (!make_halo_sync(p.hs, reinterpret_cast<const HaloSyncArgs*>(halo), x, g.N, g.D,
                      (long long)g.H * g.W * g.C * 2, xs[0] * 2)) return -1;
  if (halo && xs[1] != (long long)g.H * g.W * g.C) return -1;

  CUtensorMap tmX, tmW;
  {
    uint64_t dims[5] = {(uint64_t)g.C, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.D, (uint64_t)g.N};
    uint64_t strides[4] = {(uint64_t)xs[3] * 2, (uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2,
                           (uint64_t)xs[0] * 2};
    uint32_t box[5] = {(uint32_t)p.Cb, (uint32_t)p.Wp, (uint32_t)p.nl, 1, 1};
    if (!lbhost::encode_tmap(&tmX, in_dtype, 5, x, dims, strides, box, nullptr, p.Cb * 2)) return -1;
  }
  {
    uint64_t dims[3] = {(uint64_t)g.C, (uint64_t)g.Kout, (uint64_t)p.taps};
    uint64_t strides[2] = {(uint64_t)g.C * 2, (uint64_t)g.C * g.Kout * 2};
    uint32_t box[3] = {(uint32_t)p.Cb, (uint32_t)BN, (uint32_t)p.taps};
    if (!lbhost::encode_tmap(&tmW, in_dtype, 3, w, dims, strides, box, nullptr, p.Cb * 2)) return -1;
  }
  const int smem = p.filter_bytes + p.stages * p.stage_bytes + 1024;
  if (BN == 128) return launch_slab<128>(tmX, tmW, p, smem, stream);
  if (BN == 64) return launch_slab<64>(tmX, tmW, p, smem, stream);
  return launch_slab<32>(tmX, tmW, p, smem, stream);
}
