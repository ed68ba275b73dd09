// Persistent warp-specialised tcgen05 pipeline shared by the GEMM and the
// implicit-GEMM convolution kernels.
//
//   warp 4      : TMA producer (one elected lane) - fills a ring of smem stages
//   warp 5      : TMEM allocator + MMA issuer (one elected lane) - tcgen05.mma into
//                 one of two TMEM accumulators, tcgen05.commit frees stages
//   warps 0..3  : epilogue - tcgen05.ld the finished accumulator (lane quarter =
//                 warp id), apply alpha/beta/bias/activation, store to global
//
// The two accumulators let the epilogue of tile i overlap the main loop of tile
// i+1.  One CTA per SM; tiles are dealt round-robin (static persistent schedule).
// A `Policy` supplies tile decoding, the per-stage TMA loads, the per-stage MMA
// issue and the row -> output address map.
#pragma once
#include "common.cuh"
#include <type_traits>
#include "halo_sync.cuh"

namespace lb {

constexpr int kBM = 128;       // accumulator rows = TMEM lanes
constexpr int kBK = 64;        // K elements per pipeline stage (16-bit types)
constexpr int kTcThreads = 192;
constexpr int kMaxStages = 32;

struct EpiParams {
  void* C;            // output
  const float* bias;  // fp32 bias or nullptr
  float alpha;        // scale of the accumulator
  float beta;         // scale of the existing output (0 = overwrite)
  int out_dtype;      // DType
  int bias_mode;      // 0 none, 1 per column, 2 per row
  int act;            // Act
  float act_param;
  long long ldc;      // elements between consecutive output rows
  // Reduce-scatter epilogue (fused GEMM -> reduce-scatter): when rs_ranks > 0 the tile is
  // not stored but ADDED (fp32 atomics, over NVLink for remote owners) into the output
  // shard of the rank that owns the row: owner = row / rs_rows, buffer rs_ptr[owner] with
  // row pitch ldc.  alpha applies; bias, beta and activation do not.
  int rs_ranks = 0;
  int rs_rows = 0;
  int rs_store = 0;   // 1: plain stores (every source rank has its own slot at the owner)
  float* rs_ptr[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // All-gather epilogue (fused GEMM -> all-gather): when bcast_ranks > 0 the finished tile is
  // stored at the same offset into the output of EVERY rank (bcast_ptr[q], peer mapped; the
  // entry of this rank is its own C), so each rank's column block of a model-parallel
  // product lands in all replicas without a separate collective.  16-bit outputs, beta == 0.
  int bcast_ranks = 0;
  void* bcast_ptr[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // Split-K (k_splits > 1): the reduction of a tile is cut into k_splits ranges that run as
  // separate work items, so a problem with few output tiles and a long reduction still fills
  // the GPU.  Every item stores its fp32 accumulators into sk_ws[tile][split][128][BN] and is
  // done; tc_splitk_reduce_kernel, launched behind it, sums the partials of every output
  // element in split order (one warp per output row, lanes along the row), applies the
  // epilogue and stores.
  int k_splits = 1;
  float* sk_ws = nullptr;
};

template <int BN>
struct StageGeom {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages =
      (200 * 1024 / kStageBytes) > 6 ? 6 : (200 * 1024 / kStageBytes);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);  // power of two by BN choice
};

struct TcShared {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Epilogue of one accumulator tile for one warp: reads this warp's 32 TMEM lanes in
// chunks of 32 columns, applies alpha / bias / beta / activation and stores the row.
// The activation kind is switched on ONCE per chunk, outside the element loops: a switch
// inside a 32-way unrolled loop made 32 copies of every activation's code, and walking
// that much code (instruction-cache misses, 32 indirect branches) cost ~200 cycles per
// element.
__device__ __forceinline__ void tc_apply_act32(float (&v)[32], int act, float prm) {
  switch (act) {
    case kActNone:
      break;
    case kActRelu:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
      break;
    case kActLeaky:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : prm * v[j];
      break;
    default:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], act, prm);
      break;
  }
}

// Where the epilogue takes a row's 32-column chunk of accumulators from.
struct TmemSrc {                 // this warp's lanes of a TMEM accumulator
  uint32_t taddr;
  __device__ __forceinline__ void load(int c, float (&v)[32]) const {
    uint32_t r[32];
    __syncwarp();  // tcgen05.ld is warp-collective: rejoin lanes that skipped a masked row
    tmem_ld_32x32(taddr + c, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  }
};
template <int BN, class Src>
__device__ __forceinline__ void tc_epilogue_rows(const Src& src, bool row_ok, long long row_off,
                                                 int n0, int n_total, int row_index,
                                                 const EpiParams& e) {
  const float alpha = e.alpha, beta = e.beta;
  const int bias_mode = e.bias_mode, act = e.act, out_dtype = e.out_dtype;
  const float row_bias = bias_mode == 2 ? e.bias[row_index] : 0.f;
#pragma unroll 1
  for (int c = 0; c < BN; c += 32) {
    if (n0 + c >= n_total) break;  // warp-uniform
    float v[32];
    src.load(c, v);
    if (!row_ok) continue;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = v[j] * alpha + row_bias;
    const long long off = row_off + n0 + c;
    const int ncol = min(32, n_total - (n0 + c));
    const bool full = ncol == 32;
    if (e.rs_ranks > 0) {
      const int owner = row_index / e.rs_rows;
      float* dst = e.rs_ptr[owner] + (long long)(row_index - owner * e.rs_rows) * e.ldc + n0 + c;
      if (e.rs_store) {
        if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < ncol) dst[j] = v[j];
        }
      } else if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          atomicAdd(reinterpret_cast<float4*>(dst + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncol) atomicAdd(dst + j, v[j]);
      }
      continue;
    }
    if (bias_mode == 1) {
      const float* bp = e.bias + n0 + c;
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += __ldg(bp + j);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncol) v[j] += __ldg(bp + j);
      }
    }
    if (beta != 0.f) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncol) v[j] += beta * load_as_f32(e.C, off + j, out_dtype);
    }
    tc_apply_act32(v, act, e.act_param);
    if (out_dtype == kF32) {
      float* dst = reinterpret_cast<float*>(e.C) + off;
      if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncol) dst[j] = v[j];
      }
    } else {
      uint16_t* dst = reinterpret_cast<uint16_t*>(e.C) + off;
      uint32_t q[16];
      if (out_dtype == kBF16) {
#pragma unroll
        for (int j = 0; j < 16; ++j) q[j] = pack2(v[2 * j], v[2 * j + 1], kBF16);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) q[j] = pack2(v[2 * j], v[2 * j + 1], kF16);
      }
      if (e.bcast_ranks > 0 && full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
        // the same 64 bytes to every rank's copy of the output (peer stores over NVLink)
#pragma unroll
        for (int rk = 0; rk < 8; ++rk) {
          if (rk >= e.bcast_ranks) break;
          uint16_t* pd = reinterpret_cast<uint16_t*>(e.bcast_ptr[rk]) + off;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(pd + 8 * j) =
                make_uint4(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
        }
      } else if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(dst + 8 * j) =
              make_uint4(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncol) dst[j] = static_cast<uint16_t>(j & 1 ? q[j >> 1] >> 16 : q[j >> 1] & 0xffffu);
      }
    }
  }
}

// Split-K: this warp's 32 rows of the accumulator go to the workspace as they are.
template <int BN>
__device__ __forceinline__ void tc_splitk_store(uint32_t taddr, float* row, bool row_ok, int n0,
                                                int n_total) {
#pragma unroll 1
  for (int c = 0; c < BN; c += 32) {
    if (n0 + c >= n_total) break;  // warp-uniform
    uint32_t r[32];
    __syncwarp();
    tmem_ld_32x32(taddr + c, r);
    tmem_ld_wait();
    if (!row_ok) continue;
    float4* dst = reinterpret_cast<float4*>(row + c);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      __stcg(dst + j, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
  }
}

// A policy may reserve the LAST `Policy::helpers(p)` CTAs of the grid for work of its own
// (e.g. copying a peer's operand shard into local memory while the other CTAs multiply):
// such a CTA runs Policy::helper_cta and leaves before any tile machinery is set up.
template <class Policy, class = void>
struct TcHelpers {
  __device__ static int count(const typename Policy::Params&) { return 0; }
  __device__ static void run(const typename Policy::Params&, int, int, uint8_t*, int*) {}
};
template <class Policy>
struct TcHelpers<Policy, typename Policy::HasHelpers> {
  __device__ static int count(const typename Policy::Params& p) { return Policy::helpers(p); }
  __device__ static void run(const typename Policy::Params& p, int index, int n, uint8_t* smem,
                             int* status) {
    Policy::helper_cta(p, index, n, smem, status);
  }
};

// A policy whose operand A is a depth-partitioned tensor with halo planes (`using HasHalo =
// void;`) exposes the exchange state (`halo(p)`) and tells which halos a tile reads
// (`tile_halo(p, tile)`: bit 0 = planes from the rank above, bit 1 = from the rank below).
template <class Policy, class = void>
struct TcHalo {
  static constexpr bool kHas = false;
  __device__ static const HaloSync* get(const typename Policy::Params&) { return nullptr; }
  __device__ static int touches(const typename Policy::Params&, const typename Policy::Tile&) {
    return 0;
  }
};
template <class Policy>
struct TcHalo<Policy, typename Policy::HasHalo> {
  static constexpr bool kHas = true;
  __device__ static const HaloSync* get(const typename Policy::Params& p) { return &Policy::halo(p); }
  __device__ static int touches(const typename Policy::Params& p, const typename Policy::Tile& t) {
    return Policy::tile_halo(p, t);
  }
};

// A policy may bring its own epilogue (`using HasEpilogue = void;` plus a static
// `epilogue(...)`); the default is tc_epilogue_rows.
template <class Policy, class = void>
struct TcEpilogue {
  static constexpr bool kSplitK = true;     // the default epilogue can finish a split-K tile
  __device__ static void run(uint32_t taddr, bool row_ok, long long row_off, int n0, int n_total,
                             int row_index, const EpiParams& e, const typename Policy::Params&) {
    tc_epilogue_rows<Policy::BN>(TmemSrc{taddr}, row_ok, row_off, n0, n_total, row_index, e);
  }
};
template <class Policy>
struct TcEpilogue<Policy, typename Policy::HasEpilogue> {
  static constexpr bool kSplitK = false;
  __device__ static void run(uint32_t taddr, bool row_ok, long long row_off, int n0, int n_total,
                             int row_index, const EpiParams& e, const typename Policy::Params& p) {
    Policy::epilogue(taddr, row_ok, row_off, n0, n_total, row_index, e, p);
  }
};

// Epilogue groups of a policy: four warps each (0-3, and 6-9 for the second).  With two
// groups each owns one of the two accumulators and drains every other tile of the CTA, so
// that two tiles' epilogues are in flight: with a single warp per scheduler the TMEM load,
// conversion and row stores of a tile show their full latency, which outlasts the MMAs of
// tiles with a short reduction (convolutions with few channels, 1x1 convolutions).
// A policy opts in with `static constexpr int kEpiGroups = 2`.
template <class Policy, class = void>
struct TcEpiGroups { static constexpr int value = 1; };
template <class Policy>
struct TcEpiGroups<Policy, std::void_t<decltype(Policy::kEpiGroups)>> {
  static constexpr int value = Policy::kEpiGroups;
};
template <class Policy>
constexpr int tc_threads() { return 64 + 128 * TcEpiGroups<Policy>::value; }

template <class Policy>
__global__ void __launch_bounds__(tc_threads<Policy>(), 1)
tc_persistent_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ typename Policy::Params p, int* status) {
  constexpr int BN = Policy::BN;
  using G = typename Policy::G;
  constexpr int S = G::kStages;

  extern __shared__ uint8_t smem_raw[];
  __shared__ TcShared sh;

  const int n_helpers = TcHelpers<Policy>::count(p);
  const int n_workers = (int)gridDim.x - n_helpers;      // CTAs that walk tiles
  if ((int)blockIdx.x >= n_workers) {
    TcHelpers<Policy>::run(p, (int)blockIdx.x - n_workers, n_helpers, smem_raw, status);
    return;
  }

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&sh.tmem_full[a]), 1);
      mbar_init(smem_u32(&sh.tmem_empty[a]), 4);  // one arrive per epilogue warp
    }
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sh.tmem_base), G::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  // Work items: (tile, split) pairs, the splits of a tile next to one another.
  const int k_iters = p.k_iters;
  const int splits = TcEpilogue<Policy>::kSplitK && p.epi.k_splits > 1 ? p.epi.k_splits : 1;
  const int num_items = p.num_tiles * splits;
  const HaloSync* hs = TcHalo<Policy>::get(p);
  const bool halo_on = TcHalo<Policy>::kHas && hs->enabled;

  if (halo_on && warp < 4) {
    // idle until the first accumulator completes: send the boundary planes to the neighbours
    halo_push(*hs, threadIdx.x, 128, blockIdx.x, n_workers);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 0) halo_signal(*hs);
  }

  if (warp == 4) {
    // ------------------------------ producer --------------------------------
    // The whole warp runs the loop: lane 0 waits for the stage and arms its barrier, then
    // every lane may issue one of the stage's TMA boxes (Policy::load picks by lane), so
    // the boxes of a stage enter the copy engine side by side instead of one after another.
    uint32_t it = 0;
    bool ok = true;
    const uint32_t halo_target =
        halo_on ? (*reinterpret_cast<volatile uint32_t*>(hs->local) + 1u) * (uint32_t)n_workers : 0u;
    int halo_need = halo_on ? ((hs->top_flag ? 1 : 0) | (hs->bot_flag ? 2 : 0)) : 0;
    for (int w = blockIdx.x; w < num_items && ok; w += n_workers) {
      const int t = w / splits, sp = w - t * splits;
      const int k_begin = (int)((long long)sp * k_iters / splits);
      const int k_end = (int)((long long)(sp + 1) * k_iters / splits);
      const typename Policy::Tile tile = Policy::decode(p, t);
      if (halo_need) {
        // first tile of this CTA that reads planes a neighbour sends: wait for them (bounded)
        const int touch = TcHalo<Policy>::touches(p, tile) & halo_need;
        int good = 1;
        if (touch && lane == 0) {
          if ((touch & 1) && !halo_wait(hs->top_flag, halo_target, status, abort_flag)) good = 0;
          if (good && (touch & 2) && !halo_wait(hs->bot_flag, halo_target, status, abort_flag)) good = 0;
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          ok = false;
          break;
        }
        halo_need &= ~touch;
      }
      for (int k = k_begin; k < k_end; ++k, ++it) {
        const uint32_t s = it % S;
        const uint32_t ph = (it / S) & 1;
        int good = 1;
        const uint32_t bar = smem_u32(&sh.full[s]);
        if (lane == 0) {
          good = mbar_wait_bounded(smem_u32(&sh.empty[s]), ph ^ 1, abort_flag) ? 1 : 0;
          if (good) mbar_expect_tx(bar, Policy::stage_bytes(p, tile, k));
          else raise_status(status, abort_flag, kTimeoutStageEmpty);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          ok = false;
          break;
        }
        const uint32_t sA = smem_base + s * G::kStageBytes;
        const uint32_t sB = sA + G::kABytes;
        Policy::load(p, tile, k, sA, sB, bar, &tmA, &tmB, lane);
      }
    }
    // Drain: every load issued must have landed before the CTA's shared memory goes away.
    // Loads whose consumer already waited have landed; the last min(it, S) stages may
    // still be in flight if the consumer gave up.
    if (lane == 0 && (!ok || *abort_flag)) {
      const uint32_t pending = it < (uint32_t)S ? it : (uint32_t)S;
      for (uint32_t j = 0; j < pending; ++j) {
        const uint32_t q = it - 1 - j;
        mbar_wait_budget_only(smem_u32(&sh.full[q % S]), (q / S) & 1);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = Policy::idesc(p);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_items && ok; w += n_workers, ++local_tile) {
        const int sp = w % splits;
        const int k_begin = (int)((long long)sp * k_iters / splits);
        const int k_end = (int)((long long)(sp + 1) * k_iters / splits);
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait_bounded(smem_u32(&sh.tmem_empty[acc]), acc_ph ^ 1, abort_flag)) {
          raise_status(status, abort_flag, kTimeoutTmemEmpty);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * BN;
        for (int k = k_begin; k < k_end; ++k, ++it) {
          const uint32_t s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait_bounded(smem_u32(&sh.full[s]), ph, abort_flag)) {
            raise_status(status, abort_flag, kTimeoutTmaFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_base + s * G::kStageBytes;
          const uint32_t sB = sA + G::kABytes;
          Policy::mma(p, k, sA, sB, tmem_acc, idesc, /*first=*/k == k_begin);
          umma_commit(smem_u32(&sh.empty[s]));  // frees the stage when the MMAs retire
        }
        if (ok) umma_commit(smem_u32(&sh.tmem_full[acc]));
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    constexpr int EG = TcEpiGroups<Policy>::value;
    const int eg = (EG > 1 && warp >= 6) ? 1 : 0;
    const int quarter = warp & 3;                    // TMEM lane quarter this warp may read
    uint32_t local_tile = (uint32_t)eg;
    bool ok = true;
    for (long long wl = (long long)blockIdx.x + (long long)eg * n_workers; wl < num_items && ok;
         wl += (long long)EG * n_workers, local_tile += EG) {
      const int w = (int)wl;
      const int t = w / splits;
      const typename Policy::Tile tile = Policy::decode(p, t);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      // The verdict is made warp-uniform: tcgen05.ld below is a warp-collective.
      const bool landed = __all_sync(
          0xffffffffu, mbar_wait_bounded(smem_u32(&sh.tmem_full[acc]), acc_ph, abort_flag));
      if (!landed) {
        if (lane == 0) raise_status(status, abort_flag, kTimeoutTmemFull);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = quarter * 32 + lane;
      long long row_off = 0;
      const bool row_ok = Policy::row_addr(p, tile, row, row_off);
      const int n0 = Policy::col0(p, tile);
      const int n_total = Policy::ncols(p);
      const int row_index = Policy::row_index(p, tile, row);
      const EpiParams& e = p.epi;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (splits == 1) {
        TcEpilogue<Policy>::run(taddr, row_ok, row_off, n0, n_total, row_index, e, p);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[acc]));
      } else {
        tc_splitk_store<BN>(taddr, e.sk_ws + ((long long)w * kBM + row) * BN, row_ok, n0, n_total);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[acc]));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (halo_on && threadIdx.x == 0) halo_finish(*hs, n_workers);
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, G::kTmemCols);
  }
}

// Second half of a split-K product: one warp per output row of a tile, lanes along the row.
// Sums the k_splits partials of every element in split order, so the result does not depend
// on how the items were scheduled, then alpha / bias / beta / activation and the store.
constexpr int kSplitReduceThreads = 256;

template <class Policy>
__global__ void __launch_bounds__(kSplitReduceThreads)
tc_splitk_reduce_kernel(const __grid_constant__ typename Policy::Params p) {
  constexpr int BN = Policy::BN;
  const long long wg = (long long)blockIdx.x * (kSplitReduceThreads / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int t = (int)(wg / kBM), row = (int)(wg % kBM);
  if (t >= p.num_tiles) return;
  const typename Policy::Tile tile = Policy::decode(p, t);
  long long row_off = 0;
  if (!Policy::row_addr(p, tile, row, row_off)) return;
  const int n0 = Policy::col0(p, tile);
  const int n_total = Policy::ncols(p);
  const EpiParams& e = p.epi;
  const int splits = e.k_splits;
  const long long split_stride = (long long)kBM * BN;
  const float* base = e.sk_ws + ((long long)t * splits * kBM + row) * BN;
  const float row_bias = e.bias_mode == 2 ? e.bias[Policy::row_index(p, tile, row)] : 0.f;
  for (int c = lane * 4; c < BN; c += 128) {
    if (n0 + c >= n_total) break;
    const float* src = base + c;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
      const float4 q0 = __ldcg(reinterpret_cast<const float4*>(src + (s + 0) * split_stride));
      const float4 q1 = __ldcg(reinterpret_cast<const float4*>(src + (s + 1) * split_stride));
      const float4 q2 = __ldcg(reinterpret_cast<const float4*>(src + (s + 2) * split_stride));
      const float4 q3 = __ldcg(reinterpret_cast<const float4*>(src + (s + 3) * split_stride));
      a.x += q0.x; a.y += q0.y; a.z += q0.z; a.w += q0.w;
      a.x += q1.x; a.y += q1.y; a.z += q1.z; a.w += q1.w;
      a.x += q2.x; a.y += q2.y; a.z += q2.z; a.w += q2.w;
      a.x += q3.x; a.y += q3.y; a.z += q3.z; a.w += q3.w;
    }
    for (; s < splits; ++s) {
      const float4 q = __ldcg(reinterpret_cast<const float4*>(src + s * split_stride));
      a.x += q.x; a.y += q.y; a.z += q.z; a.w += q.w;
    }
    float v[4] = {a.x, a.y, a.z, a.w};
    const int ncol = min(4, n_total - (n0 + c));
    const long long off = row_off + n0 + c;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j >= ncol) break;
      float x = v[j] * e.alpha + row_bias;
      if (e.bias_mode == 1) x += __ldg(e.bias + n0 + c + j);
      if (e.beta != 0.f) x += e.beta * load_as_f32(e.C, off + j, e.out_dtype);
      v[j] = apply_act(x, e.act, e.act_param);
    }
    if (e.out_dtype == kF32) {
      float* dst = reinterpret_cast<float*>(e.C) + off;
      if (ncol == 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
        for (int j = 0; j < ncol; ++j) dst[j] = v[j];
      }
    } else {
      uint16_t* dst = reinterpret_cast<uint16_t*>(e.C) + off;
      const uint32_t lo = pack2(v[0], v[1], e.out_dtype), hi = pack2(v[2], v[3], e.out_dtype);
      if (ncol == 4 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
      } else {
        for (int j = 0; j < ncol; ++j) {
          const uint32_t q = j < 2 ? lo : hi;
          dst[j] = static_cast<uint16_t>(j & 1 ? q >> 16 : q & 0xffffu);
        }
      }
    }
  }
}

// Host side: launches the reduction behind a split product.
template <class Policy>
static int launch_splitk_reduce(const typename Policy::Params& p, cudaStream_t stream) {
  const long long rows = (long long)p.num_tiles * kBM;
  const int per_block = kSplitReduceThreads / 32;
  const int blocks = (int)((rows + per_block - 1) / per_block);
  tc_splitk_reduce_kernel<Policy><<<blocks, kSplitReduceThreads, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace lb
