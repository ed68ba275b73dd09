// First-layer convolution kernels for inputs with at most 8 channels (4 or 8 channels per
// pixel in memory, i.e. 8- or 16-byte pixels), kd x kh x 3 filters, stride 1, dilation 1.
//
// With so few channels the reduction per tap is tiny, and a tcgen05.mma costs ~104
// cycles however little of it is used, so the generic implicit-GEMM path (one operand
// slice per tap) wastes almost all of every instruction here.  Both kernels therefore
// bring ONE halo slab per tile with TMA and let the four epilogue warps unfold it in
// shared memory into a dense operand whose rows / columns are (tap, channel):
//
//  forward:  A = [pixel][(tap, channel)] K-major, 7 UMMAs per 128 pixels for a 3x3x3
//            filter on 4-channel pixels; the packed filter stays in shared memory.
//  wgrad:    A = the same bytes read MN-major (M = (tap, channel), K = pixel), B = the dy
//            brick as TMA delivers it; 8 UMMAs per 128 pixels, one accumulator tile per
//            CTA, partial dW added with fp32 atomics at the end.
//
// The reference relies on cuDNN for this layer
// (src/layers/learning/base_convolution.cpp:462-814).
#include "tc_pipeline.cuh"
#include <algorithm>

namespace lb {

constexpr uint32_t kLayoutNone = 0;

struct C8Geom {
  int N, D, H, W;       // input spatial dims
  int Kout;
  int kd, kh;           // kw is 3
  int pd, ph;           // pw is 1
  int Do;               // output depth = D + 2 pd - kd + 1 (pd = 0 when halos carry the padding)
};

// Unfold one pixel: gather its taps from the halo slab (3 kw taps from each of the
// kd * kh slab rows) and store them as 16-byte K chunks, 128 B apart, of the operand row.
// All loads of a pixel are issued before the first store so that their latencies overlap;
// TAPS2 > 0 fixes kd * kh at compile time (full unrolling), TAPS2 = 0 is the generic loop.
// RPITCH > 0 (with TAPS2 = 9, a 3 x 3 tap plane): the slab has RPITCH rows per depth plane
// instead of 3, i.e. it is a window of a larger slab shared by several tiles.
template <int CR, int TAPS2, int RPITCH = 0>
__device__ __forceinline__ void c8_unfold_pixel(uint32_t src_px, uint32_t dst, int taps2,
                                                int row_bytes) {
  if constexpr (TAPS2 > 0 && CR == 4) {
    uint2 v[TAPS2 * 3 + 1];
#pragma unroll
    for (int r = 0; r < TAPS2; ++r) {
      const int row = RPITCH > 0 ? (r / 3) * RPITCH + (r % 3) : r;
#pragma unroll
      for (int c = 0; c < 3; ++c) v[r * 3 + c] = lds64(src_px + row * row_bytes + c * 8);
    }
    v[TAPS2 * 3] = make_uint2(0u, 0u);
#pragma unroll
    for (int mb = 0; mb < (TAPS2 * 3 + 1) / 2; ++mb)
      sts128(dst + mb * 128, make_uint4(v[2 * mb].x, v[2 * mb].y, v[2 * mb + 1].x, v[2 * mb + 1].y));
  } else if constexpr (TAPS2 > 0) {
#pragma unroll
    for (int r = 0; r < TAPS2; ++r) {
      uint4 v[3];
#pragma unroll
      for (int c = 0; c < 3; ++c) v[c] = lds128(src_px + r * row_bytes + c * 16);
#pragma unroll
      for (int c = 0; c < 3; ++c) sts128(dst + (r * 3 + c) * 128, v[c]);
    }
  } else if constexpr (CR == 4) {
    const int taps = taps2 * 3;
    for (int mb = 0; mb < (taps + 1) / 2; ++mb) {
      const int t0 = 2 * mb, t1 = 2 * mb + 1;
      const int r0 = t0 / 3, c0 = t0 - r0 * 3;
      const int r1 = t1 / 3, c1 = t1 - r1 * 3;
      uint2 lo = lds64(src_px + r0 * row_bytes + c0 * 8);
      uint2 hi = make_uint2(0u, 0u);
      if (t1 < taps) hi = lds64(src_px + r1 * row_bytes + c1 * 8);
      sts128(dst + mb * 128, make_uint4(lo.x, lo.y, hi.x, hi.y));
    }
  } else {
    for (int r = 0; r < taps2; ++r) {
#pragma unroll
      for (int c = 0; c < 3; ++c)
        sts128(dst + (r * 3 + c) * 128, lds128(src_px + r * row_bytes + c * 16));
    }
  }
}

__device__ __forceinline__ void c8_unfold(int cr, int taps2, uint32_t slab, int slab_lead, int px,
                                          uint32_t dst, int row_bytes) {
  if (cr == 4) {
    const uint32_t src_px = slab + (slab_lead + px) * 8;
    if (taps2 == 9) c8_unfold_pixel<4, 9>(src_px, dst, taps2, row_bytes);
    else if (taps2 == 3) c8_unfold_pixel<4, 3>(src_px, dst, taps2, row_bytes);
    else c8_unfold_pixel<4, 0>(src_px, dst, taps2, row_bytes);
  } else {
    const uint32_t src_px = slab + (slab_lead + px) * 16;
    if (taps2 == 9) c8_unfold_pixel<8, 9>(src_px, dst, taps2, row_bytes);
    else if (taps2 == 3) c8_unfold_pixel<8, 3>(src_px, dst, taps2, row_bytes);
    else c8_unfold_pixel<8, 0>(src_px, dst, taps2, row_bytes);
  }
}

// ------------------------------------------------------------------------- forward
// y[pixel][k] = sum over (tap, channel) of x[pixel + tap][channel] * w[k][tap][channel], as a
// GEMM with M = 128 pixels of one image row, N = Kout, K = (tap, channel).  A tcgen05.mma
// costs ~104 cycles whatever N <= 128 is, so the tile time is the number of UMMAs: the
// four epilogue warps first unfold the tile's halo slab into the canonical un-swizzled
// K-major operand [pixel][(tap, channel)] in shared memory, which makes every K element
// useful: 27 taps x 4 channels = 108 -> 7 UMMAs per tile (14 with 8-channel pixels)
// against 18 when each (kd, kh) slab row is fed through shifted descriptors.
//
// Per tile ONE 5-D TMA box brings the slab [kd][kh][chunks][128 B].  The tensor map
// splits W into 128-byte chunks (dim 0: 16 units of 8 bytes, dim 1: chunk index), which
// lifts the 256-element limit of a box dimension while the rows still land back to
// back; the chunk left of the tile and chunks beyond W are zero-filled and supply the
// padding along W, rows outside H / D likewise.  Pixels are 8 bytes (4 channels) or 16.
// The filter, packed on the host as [K chunk of 8][32 rows][8], stays in shared memory.
// A run of MMAs along K into one accumulator, straight-line for the step counts the first-layer
// shapes have (a rolled loop costs the issuing thread ~100 cycles per MMA, the MMA itself 44).
template <int KSTEPS>
__device__ __forceinline__ void c8_issue_run(uint32_t acc, uint32_t ad, uint32_t a_hi, uint32_t bd,
                                             uint32_t b_hi, uint32_t idesc, uint32_t a_step,
                                             uint32_t b_step, uint32_t first) {
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk)
    umma_f16_lo(acc, ad + kk * a_step, a_hi, bd + kk * b_step, b_hi, idesc, kk ? 1u : first);
}
__device__ __forceinline__ void c8_issue(int ksteps, uint32_t acc, uint32_t ad, uint32_t a_hi,
                                         uint32_t bd, uint32_t b_hi, uint32_t idesc, uint32_t a_step,
                                         uint32_t b_step, uint32_t first) {
  switch (ksteps) {
    case 3: c8_issue_run<3>(acc, ad, a_hi, bd, b_hi, idesc, a_step, b_step, first); break;
    case 5: c8_issue_run<5>(acc, ad, a_hi, bd, b_hi, idesc, a_step, b_step, first); break;
    case 7: c8_issue_run<7>(acc, ad, a_hi, bd, b_hi, idesc, a_step, b_step, first); break;
    case 8: c8_issue_run<8>(acc, ad, a_hi, bd, b_hi, idesc, a_step, b_step, first); break;
    case 14: c8_issue_run<14>(acc, ad, a_hi, bd, b_hi, idesc, a_step, b_step, first); break;
    default:
      for (int kk = 0; kk < ksteps; ++kk)
        umma_f16_lo(acc, ad + kk * a_step, a_hi, bd + kk * b_step, b_hi, idesc, kk ? 1u : first);
  }
}

constexpr int kC8MaxStages = 12;
// Worker groups of four warps.  A group unfolds a tile and later runs its epilogue; with a
// single warp per scheduler every dependent instruction shows its full latency, so the
// groups take tiles in turn (tile i belongs to group i % G, with its own operand buffer
// and accumulator) and overlap one another's latencies.
constexpr int kC8Groups = 4;
constexpr int kC8Threads = 64 + 128 * kC8Groups;

struct C8FwdParams {
  C8Geom g;
  int tiles_w, num_tiles, taps2, taps;
  int cr;                      // channels per pixel in memory: 4 or 8
  int mb_pad;                  // 16-byte K chunks per pixel in the unfolded operand (16 or 32)
  int ksteps;                  // UMMAs per tile
  int groups;                  // worker groups (<= kC8Groups)
  int slab_row_bytes, slab_lead, stage_bytes, stages, filter_bytes;
  int in_dtype;
  const void* w;               // packed filter in global memory
  long long o_sn, o_sd, o_sh, o_sw;
  FastDiv fd_tiles_w, fd_H, fd_Do;   // tile decode without run-time divisions
  EpiParams epi;
};

struct C8FwdShared {
  uint64_t full[kC8MaxStages];
  uint64_t empty[kC8MaxStages];
  uint64_t a_ready[kC8Groups];
  uint64_t tmem_full[kC8Groups];
  uint64_t tmem_empty[kC8Groups];
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kC8Threads, 1)
conv_c8_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const C8FwdParams p, int* status) {
  constexpr int BN = 32;
  const int G = p.groups;                        // worker groups in this launch: 2 to 4
  const int kProducerWarp = 4 * G, kMmaWarp = 4 * G + 1;
  constexpr int kTmemCols = 128;
  extern __shared__ uint8_t smem_raw[];
  __shared__ C8FwdShared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_bytes = 16u * p.mb_pad * 128u;
  const uint32_t s_a0 = smem_base;                               // G unfolded operands
  const uint32_t s_filter = smem_base + G * a_bytes;
  const uint32_t s_stage0 = s_filter + p.filter_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const int S = p.stages;
  const C8Geom& g = p.g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 4);      // one arrive per unfolding warp
    }
    for (int a = 0; a < kC8Groups; ++a) {
      mbar_init(smem_u32(&sh.a_ready[a]), 4);
      mbar_init(smem_u32(&sh.tmem_full[a]), 1);
      mbar_init(smem_u32(&sh.tmem_empty[a]), 4);
    }
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp && lane == 0) tma_prefetch_desc(&tmX);
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sh.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  if (warp < 4 * G) {
    // zero the operand buffers (K chunks that no tap fills must read as zero) and bring
    // the filter in with plain loads; both are then published to the tensor core's proxy
    uint4* az = reinterpret_cast<uint4*>(smem_raw + (s_a0 - smem_u32(smem_raw)));
    for (uint32_t i = threadIdx.x; i < G * a_bytes / 16; i += 128 * G) az[i] = make_uint4(0, 0, 0, 0);
    uint4* fz = reinterpret_cast<uint4*>(smem_raw + (s_filter - smem_u32(smem_raw)));
    const uint4* fw = reinterpret_cast<const uint4*>(p.w);
    for (uint32_t i = threadIdx.x; i < (uint32_t)p.filter_bytes / 16; i += 128 * G) fz[i] = fw[i];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  const int chunk_px = p.cr == 4 ? 16 : 8;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      // tile index -> (tw, h, d, n), advanced incrementally: no divisions in the loop
      int t = blockIdx.x;
      int tw = t % p.tiles_w, r = t / p.tiles_w;
      int h = r % g.H; r /= g.H;
      int d = r % g.Do, n = r / g.Do;
      const int step_tw = gridDim.x % p.tiles_w, step_r = gridDim.x / p.tiles_w;
      const int step_h = step_r % g.H, step_r2 = step_r / g.H;
      const int step_d = step_r2 % g.Do, step_n = step_r2 / g.Do;
      RingPos rp;
      for (; t < p.num_tiles; t += gridDim.x, ++it) {
        const uint32_t s = rp.s;
        if (!mbar_wait_bounded(smem_u32(&sh.empty[s]), rp.ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutStageEmpty);
          ok = false;
          break;
        }
        rp.advance((uint32_t)S);
        const uint32_t bar = smem_u32(&sh.full[s]);
        mbar_expect_tx(bar, (uint32_t)(p.taps2 * p.slab_row_bytes));
        tma_load_5d(s_stage0 + s * p.stage_bytes, &tmX, bar, 0, tw * (128 / chunk_px) - 1,
                    h - g.ph, d - g.pd, n);
        // mixed-radix add of the grid stride
        tw += step_tw;
        int c = 0;
        if (tw >= p.tiles_w) { tw -= p.tiles_w; c = 1; }
        h += step_h + c; c = 0;
        if (h >= g.H) { h -= g.H; c = 1; }
        d += step_d + c; c = 0;
        if (d >= g.Do) { d -= g.Do; c = 1; }
        n += step_n + c;
      }
      if (!ok || *abort_flag) {
        const uint32_t pending = it < (uint32_t)S ? it : (uint32_t)S;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t q = it - 1 - j;
          mbar_wait_budget_only(smem_u32(&sh.full[q % S]), (q / S) & 1);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 0, 0, 128, BN);
      // A (K-major, un-swizzled): core matrix = 8 pixels x 16 B; K chunks 128 B apart (LBO),
      // 8-pixel groups mb_pad * 128 B apart (SBO).  B: [K chunk][BN rows][16 B]: K chunks
      // BN * 16 B apart (LBO), 8-row groups 128 B apart (SBO).  One UMMA = 2 K chunks.
      const uint64_t a_desc0 = make_smem_desc(0, 128, p.mb_pad * 128, kLayoutNone);
      const uint64_t b_desc0 = make_smem_desc(s_filter, BN * 16, 128, kLayoutNone);
      const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
      const uint32_t a_lo0 = (uint32_t)a_desc0 + (s_a0 >> 4), b_lo0 = (uint32_t)b_desc0;
      const uint32_t a_buf_step = a_bytes >> 4;
      const int ksteps = p.ksteps;
      bool ok = true;
      RingPos gp;                                   // which worker group's buffers: (j, parity)
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x, gp.advance((uint32_t)G)) {
        const uint32_t j = gp.s, jph = gp.ph;
        if (!mbar_wait_bounded(smem_u32(&sh.tmem_empty[j]), jph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmemEmpty);
          ok = false;
          break;
        }
        if (!mbar_wait_bounded(smem_u32(&sh.a_ready[j]), jph, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmaFull);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t ad = a_lo0 + j * a_buf_step;
        uint32_t bd = b_lo0;
        const uint32_t tmem_acc = tmem_base + j * BN;
        constexpr uint32_t kAStep = (2 * 128) >> 4, kBStep = (2 * BN * 16) >> 4;
        c8_issue(ksteps, tmem_acc, ad, a_hi, bd, b_hi, idesc, kAStep, kBStep, 0u);
        // one commit tells the group both that its accumulator is complete and that its
        // operand buffer may be overwritten (every barrier operation costs this thread ~80 cycles)
        umma_commit(smem_u32(&sh.tmem_full[j]));
      }
    }
  } else {
    const int group = warp >> 2;                    // tiles group, group + G, ... of this CTA
    const int wq = warp & 3;                        // TMEM lane quarter of this warp
    const int px = wq * 32 + lane;                  // pixel of the tile this thread unfolds
    const uint32_t dst_px = (px >> 3) * (p.mb_pad * 128) + (px & 7) * 16;
    const EpiParams& e = p.epi;
    const uint32_t j = group;
    int t_prev = -1;
    uint32_t use = 0;                               // how often this group used its buffers
    // ring position of tile `it` = group, group + G, ...: advanced by G stages per round
    uint32_t rs = (uint32_t)group % (uint32_t)S, rph = ((uint32_t)group / (uint32_t)S) & 1u;
    for (uint32_t it = group;; it += G, ++use) {
      const long long tl = (long long)blockIdx.x + (long long)it * gridDim.x;
      const bool have = tl < p.num_tiles;
      const int t = (int)tl;
      if (have) {
        // ---- unfold tile `it` ---------------------------------------------------------
        const uint32_t s = rs, ph = rph;
        rs += (uint32_t)G;
        if (rs >= (uint32_t)S) { rs -= (uint32_t)S; rph ^= 1u; }
        bool good = mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag);
        // the MMAs of this group's previous tile have read the operand buffer
        good = good && (use == 0 ||
                        mbar_wait_bounded(smem_u32(&sh.tmem_full[j]), (use - 1) & 1, abort_flag));
        if (!__all_sync(0xffffffffu, good)) {
          if (lane == 0) raise_status(status, abort_flag, kTimeoutTmaFull);
          break;
        }
        const uint32_t sX = s_stage0 + s * p.stage_bytes;
        const uint32_t dst = s_a0 + j * a_bytes + dst_px;
        c8_unfold(p.cr, p.taps2, sX, p.slab_lead, px, dst, p.slab_row_bytes);
        // publish the generic-proxy writes to the tensor core's proxy, then signal
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&sh.a_ready[j]));
          mbar_arrive(smem_u32(&sh.empty[s]));       // the slab is no longer needed
        }
      }
      // ---- epilogue of this group's previous tile (its UMMAs ran meanwhile) ------------
      if (t_prev >= 0) {
        const uint32_t acc_ph = (use - 1) & 1;
        uint32_t r, utw, uh, ud, un;
        p.fd_tiles_w.divmod((uint32_t)t_prev, r, utw);
        p.fd_H.divmod(r, r, uh);
        p.fd_Do.divmod(r, un, ud);
        const int tw = (int)utw, h = (int)uh, d = (int)ud, n = (int)un;
        const bool landed = __all_sync(
            0xffffffffu, mbar_wait_bounded(smem_u32(&sh.tmem_full[j]), acc_ph, abort_flag));
        if (!landed) {
          if (lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
          break;
        }
        tc_fence_after();
        const int row = wq * 32 + lane;
        const int w = tw * 128 + row;
        const long long row_off = n * p.o_sn + d * p.o_sd + h * p.o_sh + (long long)w * p.o_sw;
        const uint32_t taddr = tmem_base + j * BN + (static_cast<uint32_t>(wq * 32) << 16);
        tc_epilogue_rows<BN>(TmemSrc{taddr}, w < g.W, row_off, 0, g.Kout, row, e);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[j]));
      }
      if (!have) break;
      t_prev = t;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------- forward + 2 x 2 x 2 max pooling in one pass
// The first layer's output is the largest tensor of the network (128^3 x 32 channels per
// sample in CosmoFlow) and its only reader is the pooling layer behind the activation.
// This kernel never writes it: a CTA takes SUPER-TILES of four row tiles, (plane 2dp or
// 2dp + 1) x (row 2hp or 2hp + 1), one per worker group.  One TMA box brings the 4 x 4-row
// slab that the four tiles share; each group unfolds its own 3 x 3-row window of it, the
// MMA thread fills four accumulators, and every group then pools 8 of the 32 channels over
// all four accumulators (the 2 x 2 window in depth and height comes from the four tiles,
// the one along W from the neighbouring TMEM lane through a shuffle).  Written: the pooled
// tensor, and one byte per pooled element with the arg-max position in scan order
// (bits 0-6) and "maximum positive" (bit 7) - the layout pool_bwd_tiled_idx_kernel reads,
// so the backward pass is the same as for the separate pooling kernel.  Two sets of
// accumulators alternate between super-tiles.
// 4-channel pixels, 3 x 3 x 3 filter only.
struct C8PoolParams {
  C8Geom g;
  int tiles_w, num_super, Hp, Dp, Wp;
  int mb_pad, ksteps;
  int slab_row_bytes, slab_lead, stage_bytes, stages, filter_bytes;
  int in_dtype, out_dtype, act;
  float act_param;
  const void* w;
  const float* bias;
  void* y;
  uint8_t* idx;
  long long o_sn, o_sd, o_sh, o_sw;   // strides of the pooled output, in elements
  FastDiv fd_tiles_w, fd_Hp, fd_Dp;
};

struct C8PoolShared {
  uint64_t full[kC8MaxStages];
  uint64_t empty[kC8MaxStages];
  uint64_t a_ready[4];
  uint64_t tmem_full[2][4];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "r"(taddr));
}

// The maximum is taken on the fp32 accumulators (3 instructions per value); bias,
// activation and the rounding to 16 bits are monotonic (leaky slope >= 0), so they are applied
// to the eight winners only and give the same pooled values as pooling the rounded tensor.
// Where two values of a window differ only below the 16-bit rounding, the arg-max recorded is
// the larger fp32 value rather than the first in scan order.
template <typename T, int ACT>
__device__ __forceinline__ void c8_pool_epilogue(const C8PoolParams& p, uint32_t taddr, int col0,
                                                 int lane, bool in_range, long long y_off,
                                                 long long idx_off) {
  uint32_t r[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a) tmem_ld_32x8(taddr + a * 32, r[a]);
  tmem_ld_wait();
  const int par = lane & 1;
  float best[8];
  int pos[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    best[c] = -INFINITY;
    pos[c] = 0;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const float v = __uint_as_float(r[a][c]);
      const bool gt = v > best[c];
      best[c] = gt ? v : best[c];
      pos[c] = gt ? 2 * a + par : pos[c];
    }
  }
  // the neighbouring pixel along W: the larger value wins, on equal values the earlier
  // position in scan order
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float ov = __shfl_xor_sync(0xffffffffu, best[c], 1);
    const int op = __shfl_xor_sync(0xffffffffu, pos[c], 1);
    const bool take = ov > best[c] || (ov == best[c] && op < pos[c]);
    best[c] = take ? ov : best[c];
    pos[c] = take ? op : pos[c];
  }
  if (!in_range) return;
  if (p.bias) {
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + col0));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + 4));
    best[0] += b0.x; best[1] += b0.y; best[2] += b0.z; best[3] += b0.w;
    best[4] += b1.x; best[5] += b1.y; best[6] += b1.z; best[7] += b1.w;
  }
  uint4 o;
  T* oe = reinterpret_cast<T*>(&o);
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float v = best[c];
    if (ACT == kActRelu) v = fmaxf(v, 0.f);
    else if (ACT == kActLeaky) v = v > 0.f ? v : v * p.act_param;
    oe[c] = from_f32<T>(v);
    const uint32_t byte = (uint32_t)pos[c] | (to_f32<T>(oe[c]) > 0.f ? 0x80u : 0u);
    if (c < 4) lo |= byte << (8 * c);
    else hi |= byte << (8 * (c - 4));
  }
  if (par == 0) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.y) + y_off) = o;
  else *reinterpret_cast<uint2*>(p.idx + idx_off) = make_uint2(lo, hi);
}

template <typename T>
__device__ __forceinline__ void c8_pool_epilogue_act(const C8PoolParams& p, uint32_t taddr, int col0,
                                                     int lane, bool in_range, long long y_off,
                                                     long long idx_off) {
  if (p.act == kActLeaky) c8_pool_epilogue<T, kActLeaky>(p, taddr, col0, lane, in_range, y_off, idx_off);
  else if (p.act == kActRelu) c8_pool_epilogue<T, kActRelu>(p, taddr, col0, lane, in_range, y_off, idx_off);
  else c8_pool_epilogue<T, kActNone>(p, taddr, col0, lane, in_range, y_off, idx_off);
}

constexpr int kC8PoolThreads = 64 + 128 * 4;

__global__ void __launch_bounds__(kC8PoolThreads, 1)
conv_c8_fwd_pool_kernel(const __grid_constant__ CUtensorMap tmX, const C8PoolParams p, int* status) {
  constexpr int BN = 32;
  constexpr int G = 4;
  constexpr int kProducerWarp = 4 * G, kMmaWarp = 4 * G + 1;
  constexpr int kTmemCols = 256;                 // two sets of four 32-column accumulators
  extern __shared__ uint8_t smem_raw[];
  __shared__ C8PoolShared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_bytes = 16u * p.mb_pad * 128u;
  const uint32_t s_a0 = smem_base;
  const uint32_t s_filter = smem_base + G * a_bytes;
  const uint32_t s_stage0 = s_filter + p.filter_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const int S = p.stages;
  const C8Geom& g = p.g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 4 * G);   // one arrive per unfolding warp
    }
    for (int a = 0; a < G; ++a) {
      mbar_init(smem_u32(&sh.a_ready[a]), 4);
      mbar_init(smem_u32(&sh.tmem_full[0][a]), 1);
      mbar_init(smem_u32(&sh.tmem_full[1][a]), 1);
    }
    mbar_init(smem_u32(&sh.tmem_empty[0]), 4 * G);
    mbar_init(smem_u32(&sh.tmem_empty[1]), 4 * G);
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp && lane == 0) tma_prefetch_desc(&tmX);
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sh.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  if (warp < 4 * G) {
    uint4* az = reinterpret_cast<uint4*>(smem_raw + (s_a0 - smem_u32(smem_raw)));
    for (uint32_t i = threadIdx.x; i < G * a_bytes / 16; i += 128 * G) az[i] = make_uint4(0, 0, 0, 0);
    uint4* fz = reinterpret_cast<uint4*>(smem_raw + (s_filter - smem_u32(smem_raw)));
    const uint4* fw = reinterpret_cast<const uint4*>(p.w);
    for (uint32_t i = threadIdx.x; i < (uint32_t)p.filter_bytes / 16; i += 128 * G) fz[i] = fw[i];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      RingPos rp;
      for (int q = blockIdx.x; q < p.num_super; q += gridDim.x, ++it) {
        const uint32_t s = rp.s;
        if (!mbar_wait_bounded(smem_u32(&sh.empty[s]), rp.ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutStageEmpty);
          ok = false;
          break;
        }
        rp.advance((uint32_t)S);
        uint32_t r, tw, hp, dp, n;
        p.fd_tiles_w.divmod((uint32_t)q, r, tw);
        p.fd_Hp.divmod(r, r, hp);
        p.fd_Dp.divmod(r, n, dp);
        const uint32_t bar = smem_u32(&sh.full[s]);
        mbar_expect_tx(bar, (uint32_t)p.stage_bytes);
        // 16 pixels of 8 bytes per 128-byte chunk; the chunk left of the tile carries the
        // padding along W, rows / planes outside the tensor are zero-filled
        tma_load_5d(s_stage0 + s * p.stage_bytes, &tmX, bar, 0, (int)tw * 8 - 1,
                    2 * (int)hp - g.ph, 2 * (int)dp - g.pd, (int)n);
      }
      if (!ok || *abort_flag) {
        const uint32_t pending = it < (uint32_t)S ? it : (uint32_t)S;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t qq = it - 1 - j;
          mbar_wait_budget_only(smem_u32(&sh.full[qq % S]), (qq / S) & 1);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 0, 0, 128, BN);
      const uint64_t a_desc0 = make_smem_desc(0, 128, p.mb_pad * 128, kLayoutNone);
      const uint64_t b_desc0 = make_smem_desc(s_filter, BN * 16, 128, kLayoutNone);
      const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
      const uint32_t a_lo0 = (uint32_t)a_desc0 + (s_a0 >> 4), b_lo0 = (uint32_t)b_desc0;
      const uint32_t a_buf_step = a_bytes >> 4;
      constexpr uint32_t kAStep = (2 * 128) >> 4, kBStep = (2 * BN * 16) >> 4;
      const int ksteps = p.ksteps;
      bool ok = true;
      uint32_t k = 0;
      for (int q = blockIdx.x; q < p.num_super && ok; q += gridDim.x, ++k) {
        const uint32_t set = k & 1u, u = k >> 1;
        if (!mbar_wait_bounded(smem_u32(&sh.tmem_empty[set]), (u & 1u) ^ 1u, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmemEmpty);
          break;
        }
#pragma unroll
        for (int j = 0; j < G; ++j) {
          if (!mbar_wait_bounded(smem_u32(&sh.a_ready[j]), k & 1u, abort_flag)) {
            raise_status(status, abort_flag, kTimeoutTmaFull);
            ok = false;
            break;
          }
          tc_fence_after();
          c8_issue(ksteps, tmem_base + set * (G * BN) + j * BN, a_lo0 + j * a_buf_step, a_hi, b_lo0,
                   b_hi, idesc, kAStep, kBStep, 0u);
          umma_commit(smem_u32(&sh.tmem_full[set][j]));
        }
      }
    }
  } else {
    const int group = warp >> 2;                    // sub-tile: plane offset group >> 1, row offset group & 1
    const int wq = warp & 3;
    const int px = wq * 32 + lane;
    const uint32_t dst = s_a0 + group * a_bytes + (px >> 3) * (p.mb_pad * 128) + (px & 7) * 16;
    const uint32_t sub_off = (uint32_t)(((group >> 1) * 4 + (group & 1)) * p.slab_row_bytes) +
                             (uint32_t)(p.slab_lead + px) * 8u;
    const int col0 = group * 8;
    RingPos rp;
    for (uint32_t k = 0;; ++k) {
      const long long ql = (long long)blockIdx.x + (long long)k * gridDim.x;
      const bool have = ql < p.num_super;
      if (have) {
        const uint32_t s = rp.s, ph = rp.ph;
        rp.advance((uint32_t)S);
        bool good = mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag);
        // the MMAs of this group's previous tile have read its operand buffer
        good = good && (k == 0 || mbar_wait_bounded(smem_u32(&sh.tmem_full[(k - 1) & 1u][group]),
                                                    ((k - 1) >> 1) & 1u, abort_flag));
        if (!__all_sync(0xffffffffu, good)) {
          if (lane == 0) raise_status(status, abort_flag, kTimeoutTmaFull);
          break;
        }
        c8_unfold_pixel<4, 9, 4>(s_stage0 + s * p.stage_bytes + sub_off, dst, 9, p.slab_row_bytes);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&sh.a_ready[group]));
          mbar_arrive(smem_u32(&sh.empty[s]));
        }
      }
      if (k >= 1) {
        // ---- pool the previous super-tile: 8 channels of all four accumulators -----------
        const uint32_t kp = k - 1, set = kp & 1u, par = (kp >> 1) & 1u;
        bool landed = true;
#pragma unroll
        for (int a = 0; a < G; ++a)
          landed = landed && mbar_wait_bounded(smem_u32(&sh.tmem_full[set][a]), par, abort_flag);
        if (!__all_sync(0xffffffffu, landed)) {
          if (lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
          break;
        }
        tc_fence_after();
        if (col0 < g.Kout) {
          const uint32_t qp = (uint32_t)(ql - gridDim.x);
          uint32_t r, tw, hp, dp, n;
          p.fd_tiles_w.divmod(qp, r, tw);
          p.fd_Hp.divmod(r, r, hp);
          p.fd_Dp.divmod(r, n, dp);
          const int w = (int)tw * 128 + px;
          const int wp = w >> 1;
          const long long y_off = (long long)n * p.o_sn + (long long)dp * p.o_sd +
                                  (long long)hp * p.o_sh + (long long)wp * p.o_sw + col0;
          const long long idx_off =
              ((((long long)n * p.Dp + dp) * p.Hp + hp) * p.Wp + wp) * g.Kout + col0;
          const uint32_t taddr = tmem_base + set * (G * BN) + col0 + (static_cast<uint32_t>(wq * 32) << 16);
          if (p.out_dtype == kBF16)
            c8_pool_epilogue_act<__nv_bfloat16>(p, taddr, col0, lane, w < g.W, y_off, idx_off);
          else
            c8_pool_epilogue_act<__half>(p, taddr, col0, lane, w < g.W, y_off, idx_off);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[set]));
      }
      if (!have) break;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------- wgrad
// dW[tap][k][c] = sum over pixels of x[pixel + tap][c] * dy[pixel][k], as a GEMM with
// M = (tap, channel), N = output channel, K = pixel.  A tcgen05.mma costs ~104 cycles for any
// N <= 128, so what counts is the number of UMMAs per pixel: reading the taps straight
// from a halo slab through shifted descriptors fills only 3 of the 16 row blocks of a
// UMMA (the kw shifts of one slab row).  Instead the four otherwise idle warps unfold
// the slab in shared memory into the canonical un-swizzled MN-major operand
// [pixel][(tap, channel)], whose rows are all useful: with 4-channel pixels the 27 taps
// of a 3x3x3 filter fit ONE 128-row tile and a brick of 128 pixels takes 8 UMMAs.
//
// Per brick (<= 128 pixels of one image row) the producer issues two TMA boxes: the
// halo slab [kd][kh][chunks][128 B] and the dy brick [pixel][Kout] (swizzled, MN-major B
// operand).  Pixels are 8 bytes (4 channels) or 16 bytes (8 channels).
constexpr int kWgBrick = 128;

struct C8WgradParams {
  C8Geom g;
  int bricks_w, bricks_total, splits;
  int taps2, taps;      // kd * kh, kd * kh * 3
  int cr;               // channels per pixel in memory: 4 or 8
  int cin;              // real input channels (<= cr): rows of padded channels are not written
  int BN, in_dtype;
  int m_tiles;          // 128-row tiles of (tap, channel) rows: 1 or 2
  int mb_pad;           // 16-byte row blocks per pixel in the unfolded operand (16 or 32)
  int slab_row_bytes, slab_bytes, slab_lead;   // slab_lead: slab index of pixel w0 - 1
  int stage_bytes, stages;
  int groups;           // worker groups unfolding bricks in turn (<= kC8Groups)
  float alpha;
  float* dW;
  long long s_tap, s_k, s_c;   // tap = (a*kh + b)*3 + kw
  FastDiv fd_bricks_w, fd_H, fd_Do;  // brick decode without run-time divisions
};

constexpr int kWgMaxStages = 8;
struct C8WgShared {
  uint64_t full[kWgMaxStages];
  uint64_t empty[kWgMaxStages];
  uint64_t a_ready[kC8Groups];
  uint64_t a_free[kC8Groups];
  uint64_t done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kC8Threads, 1)
conv_c8_wgrad_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDy,
                     const C8WgradParams p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ C8WgShared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const int S = p.stages;
  const C8Geom& g = p.g;
  const uint32_t a_bytes = 16u * p.mb_pad * 128u;          // 16 pixel groups x row blocks x 128 B
  const int G = p.groups;
  const int kProducerWarp = 4 * G, kMmaWarp = 4 * G + 1;
  const uint32_t s_a0 = smem_base;                          // G unfolded operands
  const uint32_t s_stage0 = smem_base + G * a_bytes;
  const int tmem_cols = p.m_tiles * p.BN < 32 ? 32 : p.m_tiles * p.BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int j = 0; j < kC8Groups; ++j) {
      mbar_init(smem_u32(&sh.a_ready[j]), 4);   // one arrive per unfolding warp
      mbar_init(smem_u32(&sh.a_free[j]), 1);
    }
    mbar_init(smem_u32(&sh.done), 1);
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmDy);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sh.tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  const int split = blockIdx.x;
  const int my_bricks = (p.bricks_total - split + p.splits - 1) / p.splits;
  const int bw_px = g.W < kWgBrick ? g.W : kWgBrick;        // pixels per brick
  const int k_steps = (bw_px + 15) / 16;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      RingPos rp;
      for (int b = split; b < p.bricks_total && ok; b += p.splits, ++it) {
        uint32_t r, ubw, uh, ud, un;
        p.fd_bricks_w.divmod((uint32_t)b, r, ubw);
        p.fd_H.divmod(r, r, uh);
        p.fd_Do.divmod(r, un, ud);
        const int bw = (int)ubw, h = (int)uh, d = (int)ud, n = (int)un;
        const uint32_t s = rp.s;
        if (!mbar_wait_bounded(smem_u32(&sh.empty[s]), rp.ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutStageEmpty);
          ok = false;
          break;
        }
        rp.advance((uint32_t)S);
        const uint32_t sX = s_stage0 + s * p.stage_bytes;
        const uint32_t sDy = sX + p.slab_bytes;
        const uint32_t bar = smem_u32(&sh.full[s]);
        mbar_expect_tx(bar, (uint32_t)(p.taps2 * p.slab_row_bytes + kWgBrick * p.BN * 2));
        // chunk coordinate: one chunk (128 B) left of the brick
        const int chunk_px = p.cr == 4 ? 16 : 8;
        tma_load_5d(sX, &tmX, bar, 0, bw * (kWgBrick / chunk_px) - 1, h - g.ph, d - g.pd, n);
        tma_load_5d(sDy, &tmDy, bar, 0, bw * kWgBrick, h, d, n);
      }
      if (!ok || *abort_flag) {
        const uint32_t pending = it < (uint32_t)S ? it : (uint32_t)S;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t q = it - 1 - j;
          mbar_wait_budget_only(smem_u32(&sh.full[q % S]), (q / S) & 1);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 1, 1, 128, (uint32_t)p.BN);
      // A (MN-major, un-swizzled): core matrix = 8 pixels x 16 B; row blocks 128 B apart
      // (SBO), 8-pixel groups mb_pad * 128 B apart (LBO); one UMMA = 2 pixel groups.
      const uint64_t a_desc0 = make_smem_desc(0, p.mb_pad * 128, 128, kLayoutNone);
      const uint32_t b_row = p.BN == 32 ? 64u : 128u;
      const uint64_t b_desc0 =
          make_smem_desc(0, 8192, 8 * b_row, p.BN == 32 ? kLayoutSw64 : kLayoutSw128);
      const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
      const uint32_t a_lo0 = (uint32_t)a_desc0 + (s_a0 >> 4);
      const uint32_t b_lo0 = (uint32_t)b_desc0 + ((s_stage0 + (uint32_t)p.slab_bytes) >> 4);
      const uint32_t a_buf_step = a_bytes >> 4, stage_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t a_kstep = (2u * p.mb_pad * 128u) >> 4;     // two pixel groups
      const uint32_t b_kstep = (16u * b_row) >> 4;              // sixteen pixel rows
      const uint32_t BNu = (uint32_t)p.BN;
      const int m_tiles = p.m_tiles;
      uint32_t first = 0;                           // 0 for the MMAs that start an accumulator
      bool ok = true;
      RingPos rp, gp;
      for (int b = split; b < p.bricks_total && ok; b += p.splits) {
        const uint32_t s = rp.s, j = gp.s;
        if (!mbar_wait_bounded(smem_u32(&sh.full[s]), rp.ph, abort_flag) ||
            !mbar_wait_bounded(smem_u32(&sh.a_ready[j]), gp.ph, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmaFull);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t ad0 = a_lo0 + j * a_buf_step;
        const uint32_t bd0 = b_lo0 + s * stage_step;
        for (int mt = 0; mt < m_tiles; ++mt) {
          const uint32_t ad = ad0 + (uint32_t)mt * ((16u * 128u) >> 4);
          const uint32_t acc = tmem_base + (uint32_t)mt * BNu;
          c8_issue(k_steps, acc, ad, a_hi, bd0, b_hi, idesc, a_kstep, b_kstep, first);
        }
        first = 1u;
        umma_commit(smem_u32(&sh.empty[s]));
        umma_commit(smem_u32(&sh.a_free[j]));
        rp.advance((uint32_t)S);
        gp.advance((uint32_t)G);
      }
      if (ok) umma_commit(smem_u32(&sh.done));
    }
  } else {
    // ---- unfold: group `warp / 4` takes bricks group, group + G, ...; a thread owns a pixel
    const int group = warp >> 2, wq = warp & 3;
    const int px = wq * 32 + lane;                  // 0..127
    const uint32_t dst_px = (px >> 3) * (p.mb_pad * 128) + (px & 7) * 16;
    const uint32_t j = group;
    bool ok = true;
    uint32_t use = 0;
    uint32_t rs = (uint32_t)group % (uint32_t)S, rph = ((uint32_t)group / (uint32_t)S) & 1u;
    for (uint32_t it = group; (long long)split + (long long)it * p.splits < p.bricks_total;
         it += G, ++use) {
      const uint32_t s = rs, ph = rph;
      rs += (uint32_t)G;
      if (rs >= (uint32_t)S) { rs -= (uint32_t)S; rph ^= 1u; }
      const uint32_t jph = use & 1;
      bool good = mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag);
      good = good && mbar_wait_bounded(smem_u32(&sh.a_free[j]), jph ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, good)) {
        if (lane == 0) raise_status(status, abort_flag, kTimeoutTmaFull);
        ok = false;
        break;
      }
      const uint32_t sX = s_stage0 + s * p.stage_bytes;
      const uint32_t dst = s_a0 + j * a_bytes + dst_px;
      c8_unfold(p.cr, p.taps2, sX, p.slab_lead, px, dst, p.slab_row_bytes);
      // make the generic-proxy writes visible to the tensor core (async proxy), then signal
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh.a_ready[j]));
    }
    // ---- epilogue: D row m = tap * cr + channel ----------------------------------------
    const bool landed =
        group == 0 && ok && my_bricks > 0 &&
        __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&sh.done), 0, abort_flag));
    if (group == 0 && ok && my_bricks > 0 && !landed && lane == 0)
      raise_status(status, abort_flag, kTimeoutTmemFull);
    if (landed) {
      tc_fence_after();
      for (int mt = 0; mt < p.m_tiles; ++mt) {
        const int m = mt * 128 + warp * 32 + lane;
        const int tap = m / p.cr, ch = m - tap * p.cr;
        const bool row_ok = tap < p.taps && ch < p.cin;
        for (int c = 0; c < p.BN; c += 32) {
          if (c >= g.Kout) break;
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(tmem_base + mt * p.BN + c + (static_cast<uint32_t>(warp * 32) << 16), r);
          tmem_ld_wait();
          if (row_ok) {
            float* dst = p.dW + (long long)tap * p.s_tap + ch * p.s_c;
#pragma unroll
            for (int q = 0; q < 32; ++q) {
              const int k = c + q;
              if (k < g.Kout) atomicAdd(dst + k * p.s_k, p.alpha * __uint_as_float(r[q]));
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

}  // namespace lb

extern "C" {

// x: [N][D][H][W][cr] with cr = xs[3] = 4 or 8 channels per pixel (dense); W a multiple of
// 16 (cr = 4) or 8.  w: filter packed as [K chunk][32 rows (output channel, zero beyond
// Kout)][8], K = tap * cr + channel with tap = (a*kh + b)*3 + kw, zero-padded to a multiple
// of 16.  y: [N][Do][H][W][Kout].  geom: N D H W Kout kd kh pd ph Do.  kw = 3, pad_w = 1.
int lb_conv_c8_fwd(const void* x, const void* w, void* y, const float* bias, const int* geom,
                   const long long* xs, const long long* ys, int in_dtype, int out_dtype,
                   int act, float act_param, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  C8FwdParams p;
  memcpy(&p.g, geom, sizeof(C8Geom));
  const C8Geom& g = p.g;
  if (g.Kout > 32 || g.Kout % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -1;
  p.cr = (int)xs[3];
  if (p.cr != 4 && p.cr != 8) return -1;
  const int chunk_px = p.cr == 4 ? 16 : 8;
  if (g.W % chunk_px) return -1;
  p.taps2 = g.kd * g.kh;
  p.taps = p.taps2 * 3;
  const int kchunks = (p.taps * p.cr + 7) / 8;
  p.ksteps = (kchunks + 1) / 2;
  if (p.ksteps > 16) return -1;
  p.mb_pad = p.ksteps > 8 ? 32 : 16;
  p.filter_bytes = (2 * p.ksteps * 32 * 16 + 1023) & ~1023;
  p.slab_lead = chunk_px - 1;
  const int nchunks = (p.slab_lead + 128 + 2 + chunk_px - 1) / chunk_px;
  p.slab_row_bytes = nchunks * 128;
  p.stage_bytes = p.taps2 * p.slab_row_bytes;
  // as many worker groups as leave room for a few slab stages beside their operand buffers
  p.groups = kC8Groups;
  int fixed = p.groups * 16 * p.mb_pad * 128 + p.filter_bytes;
  while (p.groups > 2 && (224 * 1024 - fixed) / p.stage_bytes < 3) {
    --p.groups;
    fixed = p.groups * 16 * p.mb_pad * 128 + p.filter_bytes;
  }
  p.stages = (224 * 1024 - fixed) / p.stage_bytes;
  if (p.stages > kC8MaxStages) p.stages = kC8MaxStages;
  if (p.stages < 2) return -1;
  p.tiles_w = (g.W + 127) / 128;
  p.num_tiles = p.tiles_w * g.H * g.Do * g.N;
  {   // exact range of the multiply-high divisions
    const long long dmax = std::max(std::max(p.tiles_w, g.H), g.Do);
    if ((long long)p.num_tiles * dmax >= (1ll << 32)) return -1;
  }
  p.fd_tiles_w = FastDiv((uint32_t)p.tiles_w);
  p.fd_H = FastDiv((uint32_t)g.H);
  p.fd_Do = FastDiv((uint32_t)g.Do);
  p.in_dtype = in_dtype;
  p.w = w;
  p.o_sn = ys[0]; p.o_sd = ys[1]; p.o_sh = ys[2]; p.o_sw = ys[3];
  p.epi.C = y; p.epi.bias = bias; p.epi.alpha = 1.f; p.epi.beta = 0.f;
  p.epi.out_dtype = out_dtype; p.epi.bias_mode = bias ? 1 : 0; p.epi.act = act;
  p.epi.act_param = act_param; p.epi.ldc = ys[3];
  CUtensorMap tmX;
  {
    // dims: 8-byte unit within a 128-byte chunk, chunk, H, D, N
    uint64_t dims[5] = {16, (uint64_t)(g.W / chunk_px), (uint64_t)g.H, (uint64_t)g.D,
                        (uint64_t)g.N};
    uint64_t strides[4] = {128, (uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2, (uint64_t)xs[0] * 2};
    uint32_t box[5] = {16, (uint32_t)nchunks, (uint32_t)g.kh, (uint32_t)g.kd, 1};
    if (!lbhost::encode_tmap(&tmX, kI64, 5, x, dims, strides, box, nullptr, 0)) return -1;
  }
  const int smem = fixed + p.stages * p.stage_bytes + 1024;
  static int configured = 0;
  if (configured < smem) {
    cudaFuncSetAttribute(conv_c8_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = smem;
  }
  const int grid = p.num_tiles < lbhost::sm_count() ? p.num_tiles : lbhost::sm_count();
  conv_c8_fwd_kernel<<<grid, 64 + 128 * p.groups, smem, stream>>>(tmX, p, lbhost::status_word());
  return (int)cudaGetLastError();
}

// Convolution (3 x 3 x 3, 4-channel pixels) + bias + activation + 2 x 2 x 2 max pooling,
// stride 2, in one kernel.  x, w, geom, xs as for lb_conv_c8_fwd (xs[3] must be 4).
// y: pooled output [N][Do/2][H/2][W/2][Kout] with element strides ys; idx: one byte per
// pooled element, contiguous, in the layout of lb_pool_fwd_tiled.  Returns -2 when the
// shape is not covered (the caller then runs the two kernels separately).
int lb_conv_c8_fwd_pool(const void* x, const void* w, void* y, void* idx, const float* bias,
                        const int* geom, const long long* xs, const long long* ys, int in_dtype,
                        int out_dtype, int act, float act_param, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  C8PoolParams p;
  memcpy(&p.g, geom, sizeof(C8Geom));
  const C8Geom& g = p.g;
  if (g.Kout > 32 || g.Kout % 8) return -2;
  if (xs[3] != 4 || g.kd != 3 || g.kh != 3 || g.ph != 1) return -2;
  if (g.W % 16 || g.H % 2 || g.Do % 2) return -2;
  if (out_dtype != kF16 && out_dtype != kBF16) return -2;
  if (act != kActNone && act != kActRelu && !(act == kActLeaky && act_param >= 0.f)) return -2;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return -2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(idx) & 7))
    return -1;
  if (ys[0] % 8 || ys[1] % 8 || ys[2] % 8 || ys[3] % 8) return -2;
  const int chunk_px = 16;
  const int kchunks = (27 * 4 + 7) / 8;
  p.ksteps = (kchunks + 1) / 2;                      // 7
  p.mb_pad = 16;
  p.filter_bytes = (2 * p.ksteps * 32 * 16 + 1023) & ~1023;
  p.slab_lead = chunk_px - 1;
  const int nchunks = (p.slab_lead + 128 + 2 + chunk_px - 1) / chunk_px;
  p.slab_row_bytes = nchunks * 128;
  p.stage_bytes = 16 * p.slab_row_bytes;             // 4 planes x 4 rows
  const int fixed = 4 * 16 * p.mb_pad * 128 + p.filter_bytes;
  p.stages = (224 * 1024 - fixed) / p.stage_bytes;
  if (p.stages > kC8MaxStages) p.stages = kC8MaxStages;
  if (p.stages < 2) return -2;
  p.tiles_w = (g.W + 127) / 128;
  p.Hp = g.H / 2; p.Dp = g.Do / 2; p.Wp = g.W / 2;
  const long long num_super = (long long)p.tiles_w * p.Hp * p.Dp * g.N;
  {
    const long long dmax = std::max(std::max(p.tiles_w, p.Hp), p.Dp);
    if (num_super * dmax >= (1ll << 32) || num_super >= (1ll << 31)) return -2;
  }
  p.num_super = (int)num_super;
  if (p.num_super <= 0) return 0;
  p.fd_tiles_w = FastDiv((uint32_t)p.tiles_w);
  p.fd_Hp = FastDiv((uint32_t)p.Hp);
  p.fd_Dp = FastDiv((uint32_t)p.Dp);
  p.in_dtype = in_dtype; p.out_dtype = out_dtype; p.act = act; p.act_param = act_param;
  p.w = w; p.bias = bias; p.y = y; p.idx = static_cast<uint8_t*>(idx);
  p.o_sn = ys[0]; p.o_sd = ys[1]; p.o_sh = ys[2]; p.o_sw = ys[3];
  CUtensorMap tmX;
  {
    uint64_t dims[5] = {16, (uint64_t)(g.W / chunk_px), (uint64_t)g.H, (uint64_t)g.D,
                        (uint64_t)g.N};
    uint64_t strides[4] = {128, (uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2, (uint64_t)xs[0] * 2};
    uint32_t box[5] = {16, (uint32_t)nchunks, 4, 4, 1};
    if (!lbhost::encode_tmap(&tmX, kI64, 5, x, dims, strides, box, nullptr, 0)) return -1;
  }
  const int smem = fixed + p.stages * p.stage_bytes + 1024;
  static int configured = 0;
  if (configured < smem) {
    cudaFuncSetAttribute(conv_c8_fwd_pool_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = smem;
  }
  const int grid = p.num_super < lbhost::sm_count() ? p.num_super : lbhost::sm_count();
  conv_c8_fwd_pool_kernel<<<grid, kC8PoolThreads, smem, stream>>>(tmX, p, lbhost::status_word());
  return (int)cudaGetLastError();
}

// dW element (tap = (a*kh + b)*3 + kw, k, c) at tap*s_tap + k*s_k + c*s_c; ADDS alpha * grad.
// x pixels hold xs[3] = 4 or 8 channels (8 or 16 bytes, dense); W must be a multiple of
// 16 (4-channel pixels) or 8; Kout <= 64 and a multiple of 8; kd * kh * 3 * channels <= 256.
int lb_conv_c8_wgrad(const void* x, const void* dy, float* dW, const int* geom,
                     const long long* xs, const long long* ys, long long s_tap, long long s_k,
                     long long s_c, int cin, int in_dtype, float alpha, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  C8WgradParams p;
  memcpy(&p.g, geom, sizeof(C8Geom));
  const C8Geom& g = p.g;
  p.cr = (int)xs[3];
  if (p.cr != 4 && p.cr != 8) return -1;
  p.cin = cin < p.cr ? cin : p.cr;
  if (g.Kout > 64 || g.Kout % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15)) return -1;
  const int chunk_px = p.cr == 4 ? 16 : 8;
  if (g.W % chunk_px) return -1;
  p.taps2 = g.kd * g.kh;
  p.taps = p.taps2 * 3;
  const int rows = p.taps * p.cr;
  if (rows > 256) return -1;
  p.m_tiles = rows > 128 ? 2 : 1;
  p.mb_pad = 16 * p.m_tiles;
  p.BN = g.Kout > 32 ? 64 : 32;
  p.slab_lead = chunk_px - 1;
  const int nchunks = (p.slab_lead + kWgBrick + 2 + chunk_px - 1) / chunk_px;
  p.slab_row_bytes = nchunks * 128;
  p.slab_bytes = (p.taps2 * p.slab_row_bytes + 1023) & ~1023;
  p.stage_bytes = p.slab_bytes + kWgBrick * p.BN * 2;
  p.groups = kC8Groups;
  int a_total = p.groups * 16 * p.mb_pad * 128;
  while (p.groups > 2 && (224 * 1024 - a_total) / p.stage_bytes < 3) {
    --p.groups;
    a_total = p.groups * 16 * p.mb_pad * 128;
  }
  p.stages = (224 * 1024 - a_total) / p.stage_bytes;
  if (p.stages > kWgMaxStages) p.stages = kWgMaxStages;
  if (p.stages < 2) return -1;
  p.bricks_w = (g.W + kWgBrick - 1) / kWgBrick;
  p.bricks_total = p.bricks_w * g.H * g.Do * g.N;
  {
    const long long dmax = std::max(std::max(p.bricks_w, g.H), g.Do);
    if ((long long)p.bricks_total * dmax >= (1ll << 32)) return -1;
  }
  p.fd_bricks_w = FastDiv((uint32_t)p.bricks_w);
  p.fd_H = FastDiv((uint32_t)g.H);
  p.fd_Do = FastDiv((uint32_t)g.Do);
  int splits = lbhost::sm_count();
  if (splits > p.bricks_total) splits = p.bricks_total;
  p.splits = splits;
  p.in_dtype = in_dtype;
  p.alpha = alpha;
  p.dW = dW;
  p.s_tap = s_tap; p.s_k = s_k; p.s_c = s_c;
  CUtensorMap tmX, tmDy;
  {
    // dims: 8-byte unit within a 128-byte chunk, chunk, H, D, N
    uint64_t dims[5] = {16, (uint64_t)(g.W / chunk_px), (uint64_t)g.H, (uint64_t)g.D,
                        (uint64_t)g.N};
    uint64_t strides[4] = {128, (uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2, (uint64_t)xs[0] * 2};
    uint32_t box[5] = {16, (uint32_t)nchunks, (uint32_t)g.kh, (uint32_t)g.kd, 1};
    if (!lbhost::encode_tmap(&tmX, kI64, 5, x, dims, strides, box, nullptr, 0)) return -1;
  }
  {
    uint64_t dims[5] = {(uint64_t)g.Kout, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.Do, (uint64_t)g.N};
    uint64_t strides[4] = {(uint64_t)ys[3] * 2, (uint64_t)ys[2] * 2, (uint64_t)ys[1] * 2,
                           (uint64_t)ys[0] * 2};
    uint32_t box[5] = {(uint32_t)p.BN, (uint32_t)kWgBrick, 1, 1, 1};
    if (!lbhost::encode_tmap(&tmDy, in_dtype, 5, dy, dims, strides, box, nullptr, p.BN * 2)) return -1;
  }
  const int smem = a_total + p.stages * p.stage_bytes + 1024;
  static int configured_smem = 0;
  if (smem > configured_smem) {
    cudaFuncSetAttribute(conv_c8_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured_smem = smem;
  }
  conv_c8_wgrad_kernel<<<p.splits, 64 + 128 * p.groups, smem, stream>>>(tmX, tmDy, p, lbhost::status_word());
  return (int)cudaGetLastError();
}

}  // extern "C"
