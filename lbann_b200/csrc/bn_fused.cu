// Batch normalisation as ONE kernel per direction, cross-GPU statistics included.
//
// The reference runs distconv batch norm as stage 1 (local sums) -> all-reduce of 2 C
// accumulators -> stage 2 (normalise), and the same again backwards
// (src/layers/regularizers/batch_normalization.cu:377-497).  Here one cooperative kernel does
// all of it:
//
//   1. every block adds its partial sums into a small replicated accumulator (L2 atomics);
//   2. grid barrier; block 0 adds the replicas up and - when the statistics span several
//      ranks - stores its 2 C floats into its slot of every peer's staging buffer (plain peer
//      stores over NVLink), meets the peers at a bounded flag rendezvous, sums the slots and
//      publishes the total; grid barrier;
//   3. every block normalises its rows with the total (the second read of x hits the L2 for
//      activations that fit).
//
// Backward: the same shape with (sum g, sum g (x - mean)) as the accumulators; the parameter
// gradients are added to the gradient arena by block 0, the (dmean, dvar) pair crosses the
// ranks.  Grid barriers are counters in a per-layer workspace that only grow (a launch
// carries no per-step argument, so the kernel can sit in a replayed CUDA graph); the kernel
// is launched cooperatively, which guarantees that all blocks are resident.  Every wait is
// bounded and reports through the status word.
#include <cooperative_groups.h>

#include "comm_sync.cuh"

namespace lb {

constexpr int kBnReplicas = 16;

template <typename T>
__device__ __forceinline__ void bnf_ld8(const T* p, float (&f)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ void bnf_st8(T* p, const float (&f)[8]) {
  uint4 q;
  T* e = reinterpret_cast<T*>(&q);
#pragma unroll
  for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(f[j]);
  *reinterpret_cast<uint4*>(p) = q;
}

// Sum of an 8-wide register array over the threads of a block that share threadIdx.x; valid
// where threadIdx.y == 0.  `sm`: blockDim.y * 8 * blockDim.x floats.
__device__ __forceinline__ void bnf_reduce_y(float (&a)[8], float* sm) {
  const int bx = blockDim.x;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[(threadIdx.y * 8 + j) * bx + threadIdx.x] = a[j];
  __syncthreads();
  if (threadIdx.y == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.f;
      for (int w = 0; w < (int)blockDim.y; ++w) t += sm[(w * 8 + j) * bx + threadIdx.x];
      a[j] = t;
    }
  }
}

// Workspace of one layer and direction (fp32 words, zero before the first launch):
//   [0] launches completed   [1] arrivals at the grid barrier (grows by the block count per launch)
//   [2] totals published (grows by 1 per launch)        [3] unused
//   [4 .. 4 + width)                totals of this launch
//   [4 + width ..)                  two accumulators (parity of the launch) x replicas x width
struct BnWork {
  unsigned* ctl;
  float* total;
  float* acc;
};
__device__ __forceinline__ BnWork bn_work(float* ws, int width) {
  BnWork w;
  w.ctl = reinterpret_cast<unsigned*>(ws);
  w.total = ws + 4;
  w.acc = ws + 4 + width;
  return w;
}

// Bounded wait until *p (only ever growing) has reached `target`.
__device__ __forceinline__ bool bn_wait_counter(const unsigned* p, unsigned target, int* status) {
  const volatile unsigned* vp = p;
  if ((int)(*vp - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  const uint64_t budget = peer_wait_budget_ns(status);
  unsigned spins = 0;
  while ((int)(*vp - target) < 0) {
    if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > budget) {
      if (status) atomicCAS(status, 0, kTimeoutPeerFlag);
      return false;
    }
  }
  return true;
}

// All blocks arrive (one arrival per block and launch); a block that passes `wait` returns
// once all `nblocks` arrivals of this launch are in.
__device__ __forceinline__ bool bn_grid_arrive_wait(unsigned* ctl, unsigned epoch, unsigned nblocks,
                                                    bool wait, int* status) {
  __shared__ int ok_sh;
  __syncthreads();
  if (threadIdx.x == 0 && threadIdx.y == 0) {
    __threadfence();
    atomicAdd(ctl + 1, 1u);
    ok_sh = 1;
    if (wait) ok_sh = bn_wait_counter(ctl + 1, (epoch + 1u) * nblocks, status) ? 1 : 0;
    __threadfence();
  }
  __syncthreads();
  return ok_sh != 0;
}

// All threads of a block: wait (thread 0 spins) until *p has reached `target`.
__device__ __forceinline__ bool bn_wait_block(const unsigned* p, unsigned target, int* status) {
  __shared__ int ok_sh2;
  if (threadIdx.x == 0 && threadIdx.y == 0) {
    ok_sh2 = bn_wait_counter(p, target, status) ? 1 : 0;
    __threadfence();
  }
  __syncthreads();
  return ok_sh2 != 0;
}

// Block 0, all threads: sum of `width` floats over the ranks of the group through the
// staging slots ([world][slot_stride] fp32 in every rank's staging buffer).
__device__ __forceinline__ bool bn_cross_rank_sum(const PeerPtrs& pp, int rank, int world,
                                                  float* vec, int width, long long slot_stride,
                                                  uint32_t* ctr, int* status) {
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, nthr = blockDim.x * blockDim.y;
  for (int i = tid; i < width; i += nthr) {
    const float v = vec[i];
    for (int q = 0; q < world; ++q)
      reinterpret_cast<float*>(pp.buf[q])[(long long)rank * slot_stride + i] = v;
  }
  if (!block_rendezvous_row(pp, rank, world, 2 * kCommBlocks, tid, ctr, status)) return false;
  const float* mine = reinterpret_cast<const float*>(pp.buf[rank]);
  for (int i = tid; i < width; i += nthr) {
    float a = 0.f;
    for (int q = 0; q < world; ++q) a += __ldcg(mine + (long long)q * slot_stride + i);
    vec[i] = a;
  }
  // the slots may be overwritten by the peers' next call only after everybody has read
  return block_rendezvous_row(pp, rank, world, 3 * kCommBlocks, tid, ctr, status);
}

struct BnFusedArgs {
  const void* x;
  const void* dy;        // backward
  const void* yact;      // output of the fused activation (backward mask), or null
  void* out;             // y (forward) / dx (backward)
  const float* scale;
  const float* bias;
  float* stats;          // [2 C]: mean, var (written forward, read backward)
  float* run_mean;
  float* run_var;
  float* dscale;         // gradient arena slices (backward), added to
  float* dbias;
  float* ws;
  long long rows, rows_per_block;
  int C, act;
  float count, correction, eps, decay, act_param;
  int rank, world;
  long long slot_stride;
  uint32_t* ctr;
  PeerPtrs pp;
};

template <typename T>
__global__ void __launch_bounds__(256)
bn_fused_fwd_kernel(const BnFusedArgs a, int* status) {
  __shared__ float sm[256 * 8];
  const int C = a.C, cv = C / 8, width = 2 * C;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = v < cv;
  const unsigned nblocks = gridDim.x * gridDim.y;
  const bool lead = blockIdx.x == 0 && blockIdx.y == 0;
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, nthr = blockDim.x * blockDim.y;
  BnWork w = bn_work(a.ws, width);
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(w.ctl);
  float* acc = w.acc + (size_t)(epoch & 1u) * kBnReplicas * width;
  const T* x = reinterpret_cast<const T*>(a.x);
  const long long r0 = (long long)blockIdx.y * a.rows_per_block;
  const long long r1 = min(a.rows, r0 + a.rows_per_block);

  // ---- 1. partial sums
  float s[8], ss[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.f; ss[j] = 0.f; }
  if (valid) {
    const T* base = x + v * 8;
    const long long step = blockDim.y;
    long long r = r0 + threadIdx.y;
    for (; r + 3 * step < r1; r += 4 * step) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = *reinterpret_cast<const uint4*>(base + (r + u * step) * C);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const T* e = reinterpret_cast<const T*>(&q[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float f = to_f32<T>(e[j]);
          s[j] += f;
          ss[j] += f * f;
        }
      }
    }
    for (; r < r1; r += step) {
      float f[8];
      bnf_ld8<T>(base + r * C, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) { s[j] += f[j]; ss[j] += f[j] * f[j]; }
    }
  }
  bnf_reduce_y(s, sm);
  bnf_reduce_y(ss, sm);
  if (valid && threadIdx.y == 0) {
    float* out = acc + (size_t)(blockIdx.y % kBnReplicas) * width;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(out + v * 8 + j, s[j]);
      atomicAdd(out + C + v * 8 + j, ss[j]);
    }
  }

  // ---- 2. grid barrier; the lead block forms the total (over the ranks too)
  bool ok = bn_grid_arrive_wait(w.ctl, epoch, nblocks, lead, status);
  if (lead) {
    if (ok) {
      for (int i = tid; i < width; i += nthr) {
        float t = 0.f;
        for (int rp = 0; rp < kBnReplicas; ++rp) {
          t += __ldcg(acc + (size_t)rp * width + i);
          acc[(size_t)rp * width + i] = 0.f;          // ready for the launch after the next
        }
        w.total[i] = t;
      }
      __syncthreads();
      if (a.world > 1)
        ok = bn_cross_rank_sum(a.pp, a.rank, a.world, w.total, width, a.slot_stride, a.ctr, status);
    }
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      atomicAdd(w.ctl + 2, 1u);                 // totals published (also on failure: nobody hangs)
      atomicAdd(w.ctl, 1u);                     // every block has read the launch count by now
    }
  }
  if (!bn_wait_block(w.ctl + 2, epoch + 1u, status) || !ok) return;

  // ---- 3. normalise
  if (!valid) return;
  float mean[8], mul[8], add[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = v * 8 + j;
    const float m = __ldcg(w.total + c) / a.count;
    const float sq = __ldcg(w.total + C + c) / a.count;
    float var = a.count * (sq - m * m) / (a.count - a.correction);
    var = var > a.eps ? var : a.eps;
    const float rstd = rsqrtf(var + a.eps);
    mean[j] = m;
    mul[j] = rstd * (a.scale ? a.scale[c] : 1.f);
    add[j] = a.bias ? a.bias[c] : 0.f;
    if (blockIdx.y == 0 && threadIdx.y == 0) {
      a.stats[c] = m;
      a.stats[C + c] = var;
      if (a.run_mean) {
        a.run_mean[c] = a.decay * a.run_mean[c] + (1.f - a.decay) * m;
        a.run_var[c] = a.decay * a.run_var[c] + (1.f - a.decay) * var;
      }
    }
  }
  T* y = reinterpret_cast<T*>(a.out);
#pragma unroll 4
  for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
    float f[8];
    bnf_ld8<T>(x + r * C + v * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float o = (f[j] - mean[j]) * mul[j] + add[j];
      if (a.act == 1) o = o > 0.f ? o : 0.f;
      else if (a.act == 2) o = o > 0.f ? o : a.act_param * o;
      f[j] = o;
    }
    bnf_st8<T>(y + r * C + v * 8, f);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
bn_fused_bwd_kernel(const BnFusedArgs a, int* status) {
  __shared__ float sm[256 * 8];
  const int C = a.C, cv = C / 8, width = 2 * C;      // accumulators: S1 = sum g, S2 = sum g (x - mean)
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = v < cv;
  const unsigned nblocks = gridDim.x * gridDim.y;
  const bool lead = blockIdx.x == 0 && blockIdx.y == 0;
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, nthr = blockDim.x * blockDim.y;
  BnWork w = bn_work(a.ws, width);
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(w.ctl);
  float* acc = w.acc + (size_t)(epoch & 1u) * kBnReplicas * width;
  const T* x = reinterpret_cast<const T*>(a.x);
  const T* dy = reinterpret_cast<const T*>(a.dy);
  const T* ya = reinterpret_cast<const T*>(a.yact);
  const int act = ya ? a.act : 0;
  const long long r0 = (long long)blockIdx.y * a.rows_per_block;
  const long long r1 = min(a.rows, r0 + a.rows_per_block);

  float mean[8], s1[8], s2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    mean[j] = a.stats[valid ? v * 8 + j : 0];
    s1[j] = s2[j] = 0.f;
  }
  if (valid) {
#pragma unroll 4
    for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
      float fx[8], fg[8], fy[8];
      bnf_ld8<T>(x + r * C + v * 8, fx);
      bnf_ld8<T>(dy + r * C + v * 8, fg);
      if (act) bnf_ld8<T>(ya + r * C + v * 8, fy);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float g = fg[j];
        if (act == 1) g = fy[j] > 0.f ? g : 0.f;
        else if (act == 2) g = fy[j] > 0.f ? g : a.act_param * g;
        s1[j] += g;
        s2[j] += g * (fx[j] - mean[j]);
      }
    }
  }
  bnf_reduce_y(s1, sm);
  bnf_reduce_y(s2, sm);
  if (valid && threadIdx.y == 0) {
    float* out = acc + (size_t)(blockIdx.y % kBnReplicas) * width;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(out + v * 8 + j, s1[j]);
      atomicAdd(out + C + v * 8 + j, s2[j]);
    }
  }

  bool ok = bn_grid_arrive_wait(w.ctl, epoch, nblocks, lead, status);
  if (lead) {
    if (ok) {
      for (int i = tid; i < width; i += nthr) {
        float t = 0.f;
        for (int rp = 0; rp < kBnReplicas; ++rp) {
          t += __ldcg(acc + (size_t)rp * width + i);
          acc[(size_t)rp * width + i] = 0.f;
        }
        w.total[i] = t;
      }
      __syncthreads();
      // parameter gradients are local sums (the gradient reduction of the step sums the ranks)
      for (int c = tid; c < C; c += nthr) {
        const float rstd = rsqrtf(a.stats[C + c] + a.eps);
        if (a.dscale) a.dscale[c] += w.total[C + c] * rstd;
        if (a.dbias) a.dbias[c] += w.total[c];
      }
      __syncthreads();
      if (a.world > 1)
        ok = bn_cross_rank_sum(a.pp, a.rank, a.world, w.total, width, a.slot_stride, a.ctr, status);
    }
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      atomicAdd(w.ctl + 2, 1u);
      atomicAdd(w.ctl, 1u);
    }
  }
  if (!bn_wait_block(w.ctl + 2, epoch + 1u, status) || !ok) return;
  if (!valid) return;

  // dx = g scale rstd + dmean / n + dvar 2 (x - mean) / (n - corr), with
  // dmean = -scale rstd S1 and dvar = -scale rstd^3 S2 / 2 (reference :302-371)
  float k0[8], k1[8], k2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = v * 8 + j;
    const float rstd = rsqrtf(a.stats[C + c] + a.eps);
    const float sc = a.scale ? a.scale[c] : 1.f;
    const float S1 = __ldcg(w.total + c), S2 = __ldcg(w.total + C + c);
    k0[j] = sc * rstd;
    k1[j] = -sc * rstd * S1 / a.count;
    k2[j] = -0.5f * sc * rstd * rstd * rstd * S2 * 2.f / (a.count - a.correction);
  }
  T* dx = reinterpret_cast<T*>(a.out);
#pragma unroll 4
  for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
    float fx[8], fg[8], fy[8];
    bnf_ld8<T>(x + r * C + v * 8, fx);
    bnf_ld8<T>(dy + r * C + v * 8, fg);
    if (act) bnf_ld8<T>(ya + r * C + v * 8, fy);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = fg[j];
      if (act == 1) g = fy[j] > 0.f ? g : 0.f;
      else if (act == 2) g = fy[j] > 0.f ? g : a.act_param * g;
      fx[j] = g * k0[j] + k1[j] + k2[j] * (fx[j] - mean[j]);
    }
    bnf_st8<T>(dx + r * C + v * 8, fx);
  }
}

struct BnGrid {
  dim3 grid, block;
  long long rows_per_block;
};

// Blocks of (bx channel vectors) x (256 / bx row lanes); as many row bands as fit on the
// device at once (the kernel waits on other blocks, so all of them must be resident).
template <typename K>
static BnGrid bn_fused_grid(K kernel, long long rows, int C) {
  BnGrid g;
  const int cv = C / 8;
  const int bx = cv >= 32 ? 32 : (cv >= 16 ? 16 : (cv >= 8 ? 8 : (cv >= 4 ? 4 : (cv >= 2 ? 2 : 1))));
  const int by = 256 / bx;
  g.block = dim3(bx, by, 1);
  const int gx = (cv + bx - 1) / bx;
  int per_sm = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 4) per_sm = 4;
  long long cap = (long long)lbhost::sm_count() * per_sm / gx;
  if (cap < 1) cap = 1;
  long long gy = (rows + by - 1) / by;
  if (gy > cap) gy = cap;
  if (gy < 1) gy = 1;
  g.rows_per_block = (rows + gy - 1) / gy;
  g.grid = dim3(gx, (unsigned)((rows + g.rows_per_block - 1) / g.rows_per_block), 1);
  return g;
}

template <typename T>
static int bn_fused_launch(bool forward, BnFusedArgs& a, cudaStream_t stream) {
  auto kernel = forward ? bn_fused_fwd_kernel<T> : bn_fused_bwd_kernel<T>;
  BnGrid g = bn_fused_grid(kernel, a.rows, a.C);
  if ((long long)g.grid.x * g.grid.y > (long long)lbhost::sm_count() * 4) return -2;
  a.rows_per_block = g.rows_per_block;
  int* status = lbhost::status_word();
  void* params[2] = {&a, &status};
  return (int)cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), g.grid, g.block, params, 0,
                                          stream);
}

}  // namespace lb

extern "C" {

// fp32 words of the per-layer, per-direction workspace (zero before the first launch).
int lb_bn_fused_ws_floats(int C) { return 4 + 2 * C + 2 * lb::kBnReplicas * 2 * C; }

// Training-mode batch norm forward in one cooperative launch.  x, y: [rows][C] channels-last,
// 16-bit, C % 8 == 0.  stats [2 C] receives (mean, variance).  world > 1: the sums are taken
// over the ranks of the group through `staging` (every rank's staging buffer, peer mapped,
// slots of slot_stride floats) and the flag rows of `pads`; count is the element count per
// channel over all those ranks.  Returns -2 when the shape is not covered.
int lb_bn_fused_fwd(const void* x, const float* scale, const float* bias, void* y, float* stats,
                    float* run_mean, float* run_var, float* ws, long long rows, int C, float count,
                    float correction, float eps, float decay, int act, float act_param, int dtype,
                    void* const* staging, void* const* pads, int rank, int world,
                    long long slot_stride, unsigned* ctr, void* stream_) {
  using namespace lb;
  if (C % 8 || C < 8 || rows < 1 || 2 * C > 4096) return -2;
  if (world > 1 && (!staging || !pads || !ctr || world > kMaxRanks || 2 * C > slot_stride)) return -1;
  BnFusedArgs a;
  memset(&a, 0, sizeof(a));
  a.x = x; a.out = y; a.scale = scale; a.bias = bias; a.stats = stats; a.run_mean = run_mean;
  a.run_var = run_var; a.ws = ws; a.rows = rows; a.C = C; a.act = act; a.count = count;
  a.correction = correction; a.eps = eps; a.decay = decay; a.act_param = act_param;
  a.rank = rank; a.world = world < 1 ? 1 : world; a.slot_stride = slot_stride; a.ctr = ctr;
  if (a.world > 1) a.pp = make_ptrs(staging, pads, a.world);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == kBF16) return bn_fused_launch<__nv_bfloat16>(true, a, stream);
  if (dtype == kF16) return bn_fused_launch<__half>(true, a, stream);
  return -2;
}

// Backward of the above: dx from (x, dy, stats); `yact` (optional) is the output of the fused
// activation, whose sign masks dy; dscale / dbias (optional) are ADDED to.
int lb_bn_fused_bwd(const void* x, const void* dy, const void* yact, const float* stats,
                    const float* scale, void* dx, float* dscale, float* dbias, float* ws,
                    long long rows, int C, float count, float correction, float eps, int act,
                    float act_param, int dtype, void* const* staging, void* const* pads, int rank,
                    int world, long long slot_stride, unsigned* ctr, void* stream_) {
  using namespace lb;
  if (C % 8 || C < 8 || rows < 1 || 2 * C > 4096) return -2;
  if (world > 1 && (!staging || !pads || !ctr || world > kMaxRanks || 2 * C > slot_stride)) return -1;
  BnFusedArgs a;
  memset(&a, 0, sizeof(a));
  a.x = x; a.dy = dy; a.yact = yact; a.out = dx; a.scale = scale; a.stats = const_cast<float*>(stats);
  a.dscale = dscale; a.dbias = dbias; a.ws = ws; a.rows = rows; a.C = C; a.act = act; a.count = count;
  a.correction = correction; a.eps = eps; a.act_param = act_param;
  a.rank = rank; a.world = world < 1 ? 1 : world; a.slot_stride = slot_stride; a.ctr = ctr;
  if (a.world > 1) a.pp = make_ptrs(staging, pads, a.world);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == kBF16) return bn_fused_launch<__nv_bfloat16>(false, a, stream);
  if (dtype == kF16) return bn_fused_launch<__half>(false, a, stream);
  return -2;
}

}  // extern "C"
