// tcgen05 filter-gradient kernel for channels-last convolutions:
//
//   dW[tap][k][c] += alpha * sum_pixels dy[pixel][k] * x[pixel*stride - pad + tap*dil][c]
//
// GEMM view: the reduction runs over output pixels, 64 at a time (one TMA brick per
// pipeline stage); both operands are "MN-major" (pixel rows, channels contiguous), so
// x and dy are consumed exactly as they sit in memory.  The accumulator rows stack
// several (tap, channel-block) slices: with Cb = 16/32/64 channels per slice an M = 128
// accumulator holds 8/4/2 slices, and a CTA keeps up to four such accumulators in TMEM,
// so one pass over its pixels yields up to 32 taps x 16 channels (CosmoFlow's first
// layer needs a single pass for all 27 taps).  The pixel range is split over CTAs and
// the partial results are added with fp32 atomics into the (pre-scaled) gradient buffer,
// matching the reference's dst_scale / grad_scale accumulation contract
// (src/layers/learning/base_convolution.cpp:1397-1445).
#include "common.cuh"

namespace lb {

struct WgradGeom {
  int N, D, H, W, C;
  int Do, Ho, Wo, Kout;
  int kd, kh, kw;
  int pd, ph, pw;
  int sd, sh, sw;
  int dd, dh, dw;
};

struct WgradParams {
  WgradGeom g;
  int TW, TH, TD, TN, rows_used;        // pixel brick (<= 64 rows)
  int bricks_w, bricks_h, bricks_d, bricks_n, bricks_total;
  int Cb, cblocks, slices_total, spg;   // spg = slices per accumulator = 128 / Cb
  int groups_total, G, group_sets;      // G accumulators per CTA
  int BN, n_tiles, splits;
  int a_layout, b_layout;
  int stage_bytes, stages, a_bytes;     // a_bytes = G * 16384
  int tmem_cols, in_dtype;
  float alpha;
  float* dW;
  long long s_tap, s_k, s_c;            // output strides in elements
  FastDiv fd_bw, fd_bh, fd_bd;          // brick decode without run-time divisions
};

struct WgradShared {
  uint64_t full[4];
  uint64_t empty[4];
  uint64_t done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(192, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmDy,
                  const WgradParams p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ WgradShared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const int S = p.stages;

  // Rows of a stage that no TMA box covers must read as zero: they are part of the
  // reduction.  TMA only ever writes the first rows_used rows, so one clear suffices.
  {
    uint8_t* base = smem_raw + (smem_base - smem_u32(smem_raw));
    uint4* q = reinterpret_cast<uint4*>(base);
    const int n16 = S * p.stage_bytes / 16;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) q[i] = make_uint4(0, 0, 0, 0);
  }
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
  // make the generic-proxy zero fill visible to the async proxy (TMA / MMA reads)
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  // work decomposition
  int wi = blockIdx.x;
  const int split = wi % p.splits; wi /= p.splits;
  const int nt = wi % p.n_tiles;   wi /= p.n_tiles;
  const int gs = wi;
  const int n0 = nt * p.BN;
  const int g_first = gs * p.G;
  const int g_count = min(p.G, p.groups_total - g_first);
  const WgradGeom& g = p.g;

  if (warp == 4) {
    // The whole warp walks the bricks: lane 0 owns the barrier protocol, and the
    // boxes of one stage go out from different lanes so that they enter the
    // copy engine side by side instead of one after another.  What a lane loads is
    // the same for every brick (which box, which tap, which channel block), so it is
    // worked out once; per brick only the brick origin changes.
    uint32_t it = 0;
    bool ok = true;
    // slices this CTA loads per brick (the same for every brick)
    int nsl = 0;
    for (int gi = 0; gi < g_count; ++gi)
      nsl += min(p.spg, p.slices_total - (g_first + gi) * p.spg);
    const int ndy = p.BN == 32 ? 1 : p.BN / 64;
    const int njobs = ndy + g_count * p.spg;
    // this lane's jobs q = lane, lane + 32 (at most two: njobs <= 4 + 4 * 8)
    struct Job { int kind; uint32_t dst; int c0, ow, oh, od; };   // kind 0 none, 1 dy box, 2 x slice
    Job jobs[2];
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const int q = lane + 32 * jj;
      Job jb = {0, 0u, 0, 0, 0, 0};
      if (q < ndy) {
        jb.kind = 1; jb.dst = (uint32_t)p.a_bytes + q * 8192u; jb.c0 = n0 + q * 64;
      } else if (q < njobs) {
        const int gi = (q - ndy) / p.spg, j = (q - ndy) - gi * p.spg;
        const int sl = (g_first + gi) * p.spg + j;
        if (sl < p.slices_total) {
          const int tap = sl / p.cblocks;
          const int ta = tap / (g.kh * g.kw), tb = (tap / g.kw) % g.kh, tc = tap % g.kw;
          jb.kind = 2; jb.dst = gi * 16384u + j * (64u * p.Cb * 2u);
          jb.c0 = (sl - tap * p.cblocks) * p.Cb;
          jb.ow = tc * g.dw - g.pw; jb.oh = tb * g.dh - g.ph; jb.od = ta * g.dd - g.pd;
        }
      }
      jobs[jj] = jb;
    }
    const uint32_t tx_bytes = (uint32_t)(p.rows_used * 2 * (nsl * p.Cb + p.BN));
    RingPos rp;
    for (int b = split; b < p.bricks_total && ok; b += p.splits, ++it) {
      uint32_t r, bw, bh, bd, nb;
      p.fd_bw.divmod((uint32_t)b, r, bw);
      p.fd_bh.divmod(r, r, bh);
      p.fd_bd.divmod(r, nb, bd);
      const int w0 = bw * p.TW, h0 = bh * p.TH, d0 = bd * p.TD, nn0 = nb * p.TN;
      const uint32_t sA = smem_base + rp.s * p.stage_bytes;
      const uint32_t bar = smem_u32(&sh.full[rp.s]);
      int go = 1;
      if (lane == 0) {
        if (!mbar_wait_bounded(smem_u32(&sh.empty[rp.s]), rp.ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutStageEmpty);
          go = 0;
        } else {
          // every slice brings rows_used * Cb * 2 bytes, dy brings rows_used * BN * 2
          mbar_expect_tx(bar, tx_bytes);
        }
      }
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) {
        ok = false;
        break;
      }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const Job& jb = jobs[jj];
        if (jb.kind == 1) {
          tma_load_5d(sA + jb.dst, &tmDy, bar, jb.c0, w0, h0, d0, nn0);
        } else if (jb.kind == 2) {
          tma_load_5d(sA + jb.dst, &tmX, bar, jb.c0, w0 * g.sw + jb.ow, h0 * g.sh + jb.oh,
                      d0 * g.sd + jb.od, nn0);
        }
      }
      __syncwarp();
      rp.advance((uint32_t)S);
    }
    if (lane == 0) {
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
      // descriptors differ in the start-address field of the low word only; four MMAs per
      // accumulator and stage, issued straight-line (see slab_issue_plane for why)
      const uint32_t idesc =
          make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, 1, 1, 128, (uint32_t)p.BN);
      const uint32_t a_lbo = 64u * p.Cb * 2u, a_sbo = 8u * p.Cb * 2u, a_adv = (16u * p.Cb * 2u) >> 4;
      const uint32_t b_row = (p.BN == 32) ? 64u : 128u;
      const uint32_t b_lbo = 8192u, b_sbo = 8u * b_row, b_adv = (16u * b_row) >> 4;
      const uint64_t a_desc = make_smem_desc(0, a_lbo, a_sbo, p.a_layout);
      const uint64_t b_desc = make_smem_desc(0, b_lbo, b_sbo, p.b_layout);
      const uint32_t a_lo0 = (uint32_t)a_desc, a_hi = (uint32_t)(a_desc >> 32);
      const uint32_t b_lo0 = (uint32_t)b_desc, b_hi = (uint32_t)(b_desc >> 32);
      const uint32_t stage_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t a_base = a_lo0 + (smem_base >> 4);
      const uint32_t b_base = b_lo0 + ((smem_base + (uint32_t)p.a_bytes) >> 4);
      const uint32_t BNu = (uint32_t)p.BN;
      uint32_t accum = 0;
      bool ok = true;
      RingPos rp;
      for (int b = split; b < p.bricks_total && ok; b += p.splits) {
        if (!mbar_wait_bounded(smem_u32(&sh.full[rp.s]), rp.ph, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmaFull);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = a_base + rp.s * stage_step, sb = b_base + rp.s * stage_step;
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          if (gi < g_count) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_f16_lo(tmem_base + gi * BNu, sa + gi * 1024u + kk * a_adv, a_hi, sb + kk * b_adv,
                          b_hi, idesc, kk == 0 ? accum : 1u);   // the first MMA of an accumulator overwrites
          }
        }
        accum = 1u;
        umma_commit(smem_u32(&sh.empty[rp.s]));
        rp.advance((uint32_t)S);
      }
      if (ok) umma_commit(smem_u32(&sh.done));
    }
  } else {
    // epilogue: wait for the whole reduction of this CTA, then atomically add to dW
    const int my_bricks = (p.bricks_total - split + p.splits - 1) / p.splits;
    const bool landed =
        my_bricks > 0 &&
        __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&sh.done), 0, abort_flag));
    if (my_bricks > 0 && !landed && lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
    if (landed) {
      tc_fence_after();
      const int row = warp * 32 + lane;
      for (int gi = 0; gi < g_count; ++gi) {
        const int sl = (g_first + gi) * p.spg + row / p.Cb;
        const int tap = sl / p.cblocks;
        const int ch = (sl - tap * p.cblocks) * p.Cb + row % p.Cb;
        const bool row_ok = sl < p.slices_total && ch < g.C;
        for (int c = 0; c < p.BN; c += 32) {
          if (n0 + c >= g.Kout) break;
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + gi * p.BN + c + ((uint32_t)(warp * 32) << 16), r);
          tmem_ld_wait();
          if (row_ok) {
            float* dst = p.dW + tap * p.s_tap + ch * p.s_c;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int k = n0 + c + j;
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

static int wg_largest_tile(int extent, int limit) {
  if (extent <= limit) return extent;
  int best = 1;
  for (int t = limit; t >= 1; --t)
    if (extent % t == 0) { best = t; break; }
  return best * 2 > limit ? best : limit;
}

}  // namespace lb

extern "C" {

// x:  [N][D][H][W][C] (strides xs, C contiguous), dy: [N][Do][Ho][Wo][Kout] (strides ys).
// dW: fp32, element (tap, k, c) at tap*s_tap + k*s_k + c*s_c; the kernel ADDS alpha * grad.
// geom as in lb_conv_fwd_tc.  Requires C % 8 == 0 and Kout % 8 == 0.
int lb_conv_wgrad_tc(const void* x, const void* dy, float* dW, const int* geom,
                     const long long* xs, const long long* ys, long long s_tap, long long s_k,
                     long long s_c, int in_dtype, float alpha, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  WgradParams p;
  static_assert(sizeof(WgradGeom) == 21 * sizeof(int), "geom layout");
  memcpy(&p.g, geom, sizeof(WgradGeom));
  const WgradGeom& g = p.g;
  if (g.C % 8 || g.Kout % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15)) return -1;
  for (int i = 0; i < 4; ++i)
    if (xs[i] % 8 || ys[i] % 8) return -1;

  p.Cb = g.C >= 64 ? 64 : (g.C >= 32 ? 32 : 16);
  p.cblocks = (g.C + p.Cb - 1) / p.Cb;
  p.slices_total = g.kd * g.kh * g.kw * p.cblocks;
  p.spg = 128 / p.Cb;
  p.groups_total = (p.slices_total + p.spg - 1) / p.spg;
  p.BN = g.Kout > 128 ? 256 : (g.Kout > 64 ? 128 : (g.Kout > 32 ? 64 : 32));
  p.n_tiles = (g.Kout + p.BN - 1) / p.BN;
  p.G = 512 / p.BN < 4 ? 512 / p.BN : 4;
  if (p.G > p.groups_total) p.G = p.groups_total;
  p.group_sets = (p.groups_total + p.G - 1) / p.G;
  p.a_layout = p.Cb == 64 ? kLayoutSw128 : (p.Cb == 32 ? kLayoutSw64 : kLayoutSw32);
  p.b_layout = p.BN == 32 ? kLayoutSw64 : kLayoutSw128;
  p.a_bytes = p.G * 16384;
  p.stage_bytes = p.a_bytes + 64 * p.BN * 2;
  p.stages = 200 * 1024 / p.stage_bytes;
  if (p.stages > 4) p.stages = 4;
  if (p.stages < 1) return -1;
  int cols = p.G * p.BN;
  p.tmem_cols = 32;
  while (p.tmem_cols < cols) p.tmem_cols *= 2;

  p.TW = wg_largest_tile(g.Wo, 64);
  p.TH = wg_largest_tile(g.Ho, 64 / p.TW);
  p.TD = wg_largest_tile(g.Do, 64 / (p.TW * p.TH));
  p.TN = wg_largest_tile(g.N, 64 / (p.TW * p.TH * p.TD));
  p.rows_used = p.TW * p.TH * p.TD * p.TN;
  p.bricks_w = (g.Wo + p.TW - 1) / p.TW;
  p.bricks_h = (g.Ho + p.TH - 1) / p.TH;
  p.bricks_d = (g.Do + p.TD - 1) / p.TD;
  p.bricks_n = (g.N + p.TN - 1) / p.TN;
  p.bricks_total = p.bricks_w * p.bricks_h * p.bricks_d * p.bricks_n;
  if ((long long)p.bricks_total * 256 >= (1ll << 32)) return -1;
  p.fd_bw = FastDiv((uint32_t)p.bricks_w);
  p.fd_bh = FastDiv((uint32_t)p.bricks_h);
  p.fd_bd = FastDiv((uint32_t)p.bricks_d);

  const int base_ctas = p.group_sets * p.n_tiles;
  int splits = (2 * lbhost::sm_count() + base_ctas - 1) / base_ctas;
  // keep at least 8 bricks per CTA so the pipeline fill is amortised
  if (splits > (p.bricks_total + 7) / 8) splits = (p.bricks_total + 7) / 8;
  if (splits < 1) splits = 1;
  p.splits = splits;
  p.in_dtype = in_dtype;
  p.alpha = alpha;
  p.dW = dW;
  p.s_tap = s_tap; p.s_k = s_k; p.s_c = s_c;

  const uint32_t bw = (p.TW - 1) * g.sw + 1, bh = (p.TH - 1) * g.sh + 1, bd = (p.TD - 1) * g.sd + 1;
  if (bw > 256 || bh > 256 || bd > 256) return -1;
  CUtensorMap tmX, tmDy;
  {
    uint64_t dims[5] = {(uint64_t)g.C, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.D, (uint64_t)g.N};
    uint64_t strides[4] = {(uint64_t)xs[3] * 2, (uint64_t)xs[2] * 2, (uint64_t)xs[1] * 2,
                           (uint64_t)xs[0] * 2};
    uint32_t box[5] = {(uint32_t)p.Cb, bw, bh, bd, (uint32_t)p.TN};
    uint32_t es[5] = {1, (uint32_t)g.sw, (uint32_t)g.sh, (uint32_t)g.sd, 1};
    if (!lbhost::encode_tmap(&tmX, in_dtype, 5, x, dims, strides, box, es, p.Cb * 2)) return -1;
  }
  {
    uint64_t dims[5] = {(uint64_t)g.Kout, (uint64_t)g.Wo, (uint64_t)g.Ho, (uint64_t)g.Do,
                        (uint64_t)g.N};
    uint64_t strides[4] = {(uint64_t)ys[3] * 2, (uint64_t)ys[2] * 2, (uint64_t)ys[1] * 2,
                           (uint64_t)ys[0] * 2};
    const uint32_t inner = p.BN == 32 ? 32 : 64;
    uint32_t box[5] = {inner, (uint32_t)p.TW, (uint32_t)p.TH, (uint32_t)p.TD, (uint32_t)p.TN};
    if (!lbhost::encode_tmap(&tmDy, in_dtype, 5, dy, dims, strides, box, nullptr, inner * 2))
      return -1;
  }
  const int smem = p.stages * p.stage_bytes + 1024;
  static int configured_smem = 0;
  if (smem > configured_smem) {
    cudaFuncSetAttribute(conv_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured_smem = smem;
  }
  const int grid = p.group_sets * p.n_tiles * p.splits;
  conv_wgrad_kernel<<<grid, 192, smem, stream>>>(tmX, tmDy, p, lbhost::status_word());
  return (int)cudaGetLastError();
}

}  // extern "C"
