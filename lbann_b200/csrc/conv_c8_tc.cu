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
// One CTA per SM walks tiles of 128 pixels along W.  Per tile a SINGLE 5-D TMA box brings
// the whole input neighbourhood: kd x kh rows of 144 pixels (8 left of the tile start to
// 136 right of it), and the packed filter (2 KB per (kd, kh) row) stays in shared memory
// for the life of the CTA.  A kw tap is a 16-byte shift of the operand start address, so
// a tile costs one copy instruction and 2 * kd * kh UMMAs; the copy engine's per-box
// set-up time (a few hundred cycles, whatever the box size) is paid once per tile
// instead of once per tap row.
//
// The tensor map splits W into 8-pixel chunks (dim 0: 16 units of 8 bytes, dim 1: chunk
// index, stride 128 B), which lifts the 256-element limit of a box dimension while the
// rows still land back to back: [kd][kh][18 chunks][128 B].  Chunk -1 and chunks beyond
// W / 8 are zero-filled and supply the padding along W; rows outside H / D likewise.
constexpr int kC8SlabChunks = 18;                       // 144 pixels
constexpr int kC8RowBytes = kC8SlabChunks * 128;        // 2304
constexpr int kC8MaxStages = 12;

struct C8FwdParams {
  C8Geom g;
  int tiles_w, num_tiles, taps2, stages, stage_bytes, in_dtype;
  long long o_sn, o_sd, o_sh, o_sw;
  EpiParams epi;
};

struct C8FwdShared {
  uint64_t full[kC8MaxStages];
  uint64_t empty[kC8MaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t filter_ready;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(192, 1)
conv_c8_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const C8FwdParams p, int* status) {
  constexpr int BN = 32;
  extern __shared__ uint8_t smem_raw[];
  __shared__ C8FwdShared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_filter = smem_base;                           // taps2 * 2048 bytes
  const uint32_t s_stage0 = smem_base + p.taps2 * 2048;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const int S = p.stages;
  const C8Geom& g = p.g;

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
    tmem_alloc(smem_u32(&sh.tmem_base), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 4) {
    if (lane == 0) {
      // filter: one box of taps2 rows x 2 KB, once
      mbar_expect_tx(smem_u32(&sh.filter_ready), (uint32_t)p.taps2 * 2048u);
      tma_load_2d(s_filter, &tmW, smem_u32(&sh.filter_ready), 0, 0);
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
      for (; t < p.num_tiles; t += gridDim.x, ++it) {
        const uint32_t s = it % S, ph = (it / S) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.empty[s]), ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutStageEmpty);
          ok = false;
          break;
        }
        const uint32_t bar = smem_u32(&sh.full[s]);
        LB_TRACE_AT(0, 2 * it);
        mbar_expect_tx(bar, (uint32_t)p.stage_bytes);
        tma_load_5d(s_stage0 + s * p.stage_bytes, &tmX, bar, 0, tw * 16 - 1, h - g.ph,
                    d - g.pd, n);
        LB_TRACE_AT(0, 2 * it + 1);
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
        mbar_wait_budget_only(smem_u32(&sh.filter_ready), 0);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 0, 0, 128, BN);
      // A: rows (pixels) 16 B apart, 8-row groups 128 B apart (SBO), the two 8-element K
      // chunks of one UMMA 16 B apart (LBO): K = 16 spans pixels m and m + 1.
      // B: [k-chunk(4)][BN rows][8 elements]: rows 16 B apart, 8-row groups 128 B (SBO),
      // K chunks BN * 16 B apart (LBO).
      const uint64_t a_desc0 = make_smem_desc(0, 16, 128, kLayoutNone);
      const uint64_t b_desc0 = make_smem_desc(0, BN * 16, 128, kLayoutNone);
      bool ok = mbar_wait_bounded(smem_u32(&sh.filter_ready), 0, abort_flag);
      if (!ok) raise_status(status, abort_flag, kTimeoutTmaFull);
      uint32_t it = 0;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x, ++it) {
        const uint32_t acc = it & 1, acc_ph = (it >> 1) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.tmem_empty[acc]), acc_ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmemEmpty);
          ok = false;
          break;
        }
        const uint32_t s = it % S, ph = (it / S) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmaFull);
          ok = false;
          break;
        }
        tc_fence_after();
        LB_TRACE_AT(1, it);
        // pixel w0 - 1 sits 7 pixels into the slab row
        uint64_t ad = a_desc0 + ((s_stage0 + s * p.stage_bytes + 7 * 16) >> 4);
        uint64_t bd = b_desc0 + (s_filter >> 4);
        const uint32_t tmem_acc = tmem_base + acc * BN;
        for (int t2 = 0; t2 < p.taps2; ++t2) {
          umma_f16(tmem_acc, ad, bd, idesc, t2 == 0 ? 0u : 1u);
          umma_f16(tmem_acc, ad + 2, bd + (2 * BN * 16 >> 4), idesc, 1u);
          ad += kC8RowBytes >> 4;
          bd += 2048 >> 4;
        }
        umma_commit(smem_u32(&sh.empty[s]));
        umma_commit(smem_u32(&sh.tmem_full[acc]));
        LB_TRACE_AT(2, it);
      }
    }
  } else {
    uint32_t it = 0;
    const EpiParams& e = p.epi;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++it) {
      int r = t;
      const int tw = r % p.tiles_w; r /= p.tiles_w;
      const int h = r % g.H; r /= g.H;
      const int d = r % g.Do, n = r / g.Do;
      const uint32_t acc = it & 1, acc_ph = (it >> 1) & 1;
      const bool landed = __all_sync(
          0xffffffffu, mbar_wait_bounded(smem_u32(&sh.tmem_full[acc]), acc_ph, abort_flag));
      if (!landed) {
        if (lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
        break;
      }
      tc_fence_after();
      if (threadIdx.x == 0) LB_TRACE_AT(3, 2 * it);
      const int row = warp * 32 + lane;
      const int w = tw * 128 + row;
      const long long row_off = n * p.o_sn + d * p.o_sd + h * p.o_sh + (long long)w * p.o_sw;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(warp * 32) << 16);
      tc_epilogue_rows<BN>(taddr, w < g.W, row_off, 0, g.Kout, row, e, it);
      tc_fence_before();
      __syncwarp();
      if (threadIdx.x == 0) LB_TRACE_AT(3, 2 * it + 1);
      if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[acc]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
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
  float alpha;
  float* dW;
  long long s_tap, s_k, s_c;   // tap = (a*kh + b)*3 + kw
};

constexpr int kWgMaxStages = 8;
struct C8WgShared {
  uint64_t full[kWgMaxStages];
  uint64_t empty[kWgMaxStages];
  uint64_t a_ready[2];
  uint64_t a_free[2];
  uint64_t done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(192, 1)
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
  const uint32_t s_a0 = smem_base;                          // two unfolded operands
  const uint32_t s_stage0 = smem_base + 2 * a_bytes;
  const int tmem_cols = p.m_tiles * p.BN < 32 ? 32 : p.m_tiles * p.BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int j = 0; j < 2; ++j) {
      mbar_init(smem_u32(&sh.a_ready[j]), 4);   // one arrive per unfolding warp
      mbar_init(smem_u32(&sh.a_free[j]), 1);
    }
    mbar_init(smem_u32(&sh.done), 1);
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmDy);
  }
  if (warp == 5) {
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
        const uint32_t s = it % S, ph = (it / S) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.empty[s]), ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutStageEmpty);
          ok = false;
          break;
        }
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
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 1, 1, 128, (uint32_t)p.BN);
      // A (MN-major, un-swizzled): core matrix = 8 pixels x 16 B; row blocks 128 B apart
      // (SBO), 8-pixel groups mb_pad * 128 B apart (LBO); one UMMA = 2 pixel groups.
      const uint64_t a_desc0 = make_smem_desc(0, p.mb_pad * 128, 128, kLayoutNone);
      const uint32_t b_row = p.BN == 32 ? 64u : 128u;
      const uint64_t b_desc0 =
          make_smem_desc(0, 8192, 8 * b_row, p.BN == 32 ? kLayoutSw64 : kLayoutSw128);
      uint32_t it = 0;
      bool ok = true;
      for (int b = split; b < p.bricks_total && ok; b += p.splits, ++it) {
        const uint32_t s = it % S, ph = (it / S) & 1;
        const uint32_t j = it & 1, jph = (it >> 1) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag) ||
            !mbar_wait_bounded(smem_u32(&sh.a_ready[j]), jph, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmaFull);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sDy = s_stage0 + s * p.stage_bytes + p.slab_bytes;
        const uint64_t ad0 = a_desc0 + ((s_a0 + j * a_bytes) >> 4);
        const uint64_t bd0 = b_desc0 + (sDy >> 4);
        for (int mt = 0; mt < p.m_tiles; ++mt) {
          uint64_t ad = ad0 + ((mt * 16 * 128) >> 4);
          uint64_t bd = bd0;
          for (int kk = 0; kk < k_steps; ++kk) {
            umma_f16(tmem_base + mt * p.BN, ad, bd, idesc, (it == 0 && kk == 0) ? 0u : 1u);
            ad += (2 * p.mb_pad * 128) >> 4;     // two pixel groups
            bd += (16 * b_row) >> 4;             // sixteen pixel rows
          }
        }
        umma_commit(smem_u32(&sh.empty[s]));
        umma_commit(smem_u32(&sh.a_free[j]));
      }
      if (ok) umma_commit(smem_u32(&sh.done));
    }
  } else {
    // ---- unfold: thread t owns pixel t of the brick -------------------------------
    const int px = threadIdx.x;                     // 0..127
    const uint32_t dst_px = (px >> 3) * (p.mb_pad * 128) + (px & 7) * 16;
    uint32_t it = 0;
    bool ok = true;
    for (int b = split; b < p.bricks_total && ok; b += p.splits, ++it) {
      const uint32_t s = it % S, ph = (it / S) & 1;
      const uint32_t j = it & 1, jph = (it >> 1) & 1;
      bool good = mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag);
      good = good && mbar_wait_bounded(smem_u32(&sh.a_free[j]), jph ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, good)) {
        if (lane == 0) raise_status(status, abort_flag, kTimeoutTmaFull);
        ok = false;
        break;
      }
      const uint32_t sX = s_stage0 + s * p.stage_bytes;
      const uint32_t dst = s_a0 + j * a_bytes + dst_px;
      if (p.cr == 4) {
        // 8-byte pixels: a 16-byte row block holds two taps
        const uint32_t src_px = sX + (p.slab_lead + px) * 8;
        for (int mb = 0; mb < (p.taps + 1) / 2; ++mb) {
          const int t0 = 2 * mb, t1 = 2 * mb + 1;
          const int r0 = t0 / 3, c0 = t0 - r0 * 3;
          const int r1 = t1 / 3, c1 = t1 - r1 * 3;
          uint2 lo = lds64(src_px + r0 * p.slab_row_bytes + c0 * 8);
          uint2 hi = make_uint2(0u, 0u);
          if (t1 < p.taps) hi = lds64(src_px + r1 * p.slab_row_bytes + c1 * 8);
          sts128(dst + mb * 128, make_uint4(lo.x, lo.y, hi.x, hi.y));
        }
      } else {
        const uint32_t src_px = sX + (p.slab_lead + px) * 16;
        for (int t = 0; t < p.taps; ++t) {
          const int r0 = t / 3, c0 = t - r0 * 3;
          sts128(dst + t * 128, lds128(src_px + r0 * p.slab_row_bytes + c0 * 16));
        }
      }
      // make the generic-proxy writes visible to the tensor core (async proxy), then signal
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh.a_ready[j]));
    }
    // ---- epilogue: D row m = tap * cr + channel ----------------------------------------
    const bool landed =
        ok && my_bricks > 0 &&
        __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&sh.done), 0, abort_flag));
    if (ok && my_bricks > 0 && !landed && lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
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
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
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
  if (g.W % 8) return -1;                    // the W axis is cut into 8-pixel chunks
  const int taps2 = g.kd * g.kh;
  if (taps2 < 1 || taps2 > 16) return -1;
  CUtensorMap tmX, tmW;
  {
    // dims: 8-byte unit within an 8-pixel chunk, chunk, H, D, N
    uint64_t dims[5] = {16, (uint64_t)g.W / 8, (uint64_t)g.H, (uint64_t)g.D, (uint64_t)g.N};
    uint64_t strides[4] = {128, (uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2, (uint64_t)xs[0] * 2};
    uint32_t box[5] = {16, (uint32_t)kC8SlabChunks, (uint32_t)g.kh, (uint32_t)g.kd, 1};
    if (!lbhost::encode_tmap(&tmX, kI64, 5, x, dims, strides, box, nullptr, 0)) return -1;
  }
  {
    // packed filter: [kd*kh][4 k-chunks][32 rows][8 elements] = 2 KB per tap-row
    uint64_t dims[2] = {256, (uint64_t)taps2};
    uint64_t strides[1] = {2048};
    uint32_t box[2] = {256, (uint32_t)taps2};
    if (!lbhost::encode_tmap(&tmW, kI64, 2, w, dims, strides, box, nullptr, 0)) return -1;
  }
  C8FwdParams p;
  p.g = g;
  p.taps2 = taps2;
  p.tiles_w = (g.W + 127) / 128;
  p.num_tiles = p.tiles_w * g.H * g.Do * g.N;
  p.stage_bytes = taps2 * kC8RowBytes;
  p.stages = (200 * 1024 - taps2 * 2048) / p.stage_bytes;
  if (p.stages > kC8MaxStages) p.stages = kC8MaxStages;
  if (p.stages < 2) return -1;
  p.in_dtype = in_dtype;
  p.o_sn = ys[0]; p.o_sd = ys[1]; p.o_sh = ys[2]; p.o_sw = ys[3];
  p.epi.C = y; p.epi.bias = bias; p.epi.alpha = 1.f; p.epi.beta = 0.f;
  p.epi.out_dtype = out_dtype; p.epi.bias_mode = bias ? 1 : 0; p.epi.act = act;
  p.epi.act_param = act_param; p.epi.ldc = ys[3];
  const int smem = taps2 * 2048 + p.stages * p.stage_bytes + 1024;
  static int configured = 0;
  if (configured < smem) {
    cudaFuncSetAttribute(conv_c8_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = smem;
  }
  const int grid = p.num_tiles < lbhost::sm_count() ? p.num_tiles : lbhost::sm_count();
  conv_c8_fwd_kernel<<<grid, 192, smem, stream>>>(tmX, tmW, p, lbhost::status_word());
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
  const int a_total = 2 * 16 * p.mb_pad * 128;
  p.stages = (224 * 1024 - a_total) / p.stage_bytes;
  if (p.stages > kWgMaxStages) p.stages = kWgMaxStages;
  if (p.stages < 2) return -1;
  p.bricks_w = (g.W + kWgBrick - 1) / kWgBrick;
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
  conv_c8_wgrad_kernel<<<p.splits, 192, smem, stream>>>(tmX, tmDy, p, lbhost::status_word());
  return (int)cudaGetLastError();
}

}  // extern "C"
