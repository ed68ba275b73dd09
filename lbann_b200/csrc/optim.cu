// Fused optimizer kernels over a flat parameter arena.
//
// All trainable weights of a model live in one fp32 "master" arena; gradients and
// optimizer state live in parallel arenas with the same offsets.  One launch updates
// every weight tensor: a device-resident segment table gives each tensor its offset,
// length, learning rate and hyper-parameters, and every block looks its segment up by
// binary search.  The same kernel refreshes the 16-bit compute copy of the weights
// (the reference keeps typed weight proxies in sync separately,
// include/lbann/weights/weights_proxy.hpp:77-350) and can fold in gradient
// unscaling for mixed precision.
//
// Update rules follow the reference kernels exactly:
//   SGD       src/optimizers/sgd.cu:36-108      v = mu v + g ; x -= lr v   (Nesterov: x -= lr (mu v + g))
//   Adam      src/optimizers/adam.cu:36-96      non-finite g skipped; x -= corr*m1/(sqrt(m2)+eps) + lr*wd*x
//   AdaGrad   src/optimizers/adagrad.cu         c += g^2 ; x -= lr g/(sqrt(c)+eps)
//   RMSprop   src/optimizers/rmsprop.cu         c = d c + (1-d) g^2 ; x -= lr g/(sqrt(c)+eps)
// AMP helper: unscale + finite check (src/utils/amp.cu:36-120); squared-norm reduction
// (src/objective_functions/weight_regularization/l2.cu, src/callbacks/gradient_clipping.cpp).
#include "common.cuh"

namespace lb {

enum OptKind : int { kOptSgd = 0, kOptAdam = 1, kOptAdagrad = 2, kOptRmsprop = 3 };

// 64-byte segment descriptor (one per weight tensor), mirrored in lbann_b200/ops/optim.py
struct OptSegment {
  long long offset;   // first element in the arenas
  long long count;    // number of elements
  int kind;           // OptKind, -1 = frozen / no optimizer
  int nesterov;
  float lr;           // SGD/AdaGrad/RMSprop: learning rate.  Adam: lr (for weight decay)
  float p0;           // SGD: momentum       Adam: beta1      RMSprop: decay
  float p1;           //                     Adam: beta2
  float eps;
  float wd;           // Adam: decoupled weight decay coefficient (multiplied by lr)
  float corr;         // unused on entry; the kernel derives it from the device step counter
  float l2;           // L2 regularisation coefficient folded into the gradient (g += l2 * x)
  float pad[3];
};
static_assert(sizeof(OptSegment) == 64, "segment layout");

constexpr int kOptChunk = 1024;  // elements per block iteration; tensors are padded to this

__device__ __forceinline__ int find_segment(const OptSegment* segs, int nseg, long long pos) {
  int lo = 0, hi = nseg - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (segs[mid].offset <= pos) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// grad_dtype: dtype of the gradient arena (fp32 or 16-bit).  inv_scale multiplies g first
// (AMP unscale / gradient averaging / clipping).  w16 (optional): 16-bit copy of the weights.
template <typename G, typename W16>
__global__ void fused_optimizer_kernel(float* __restrict__ w, const G* __restrict__ grad,
                                       float* __restrict__ s0, float* __restrict__ s1,
                                       W16* __restrict__ w16, const OptSegment* __restrict__ segs,
                                       int nseg, long long total, float inv_scale,
                                       const int* __restrict__ skip_flag,
                                       const int* __restrict__ step_ptr,
                                       const float* __restrict__ lr_scale_ptr,
                                       const float* __restrict__ inv_scale_dev) {
  if (skip_flag && *skip_flag) return;  // AMP overflow: the whole step is skipped
  // AMP: the inverse loss scale of this step's gradients, kept on the device; the gradients
  // are then unscaled here, in registers, instead of by a pass of their own
  if (inv_scale_dev) inv_scale *= *inv_scale_dev;
  // The step number and a global learning-rate multiplier live in device memory so that a
  // captured CUDA graph sees fresh values on every replay.
  const float step_t = step_ptr ? (float)(*step_ptr) : 1.f;
  const float lr_mul = lr_scale_ptr ? *lr_scale_ptr : 1.f;
  const long long nchunks = (total + kOptChunk - 1) / kOptChunk;
  for (long long ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
    const long long base = ch * kOptChunk;
    const int si = find_segment(segs, nseg, base);
    OptSegment sg = segs[si];
    sg.lr *= lr_mul;
    if (sg.kind == kOptAdam)
      sg.corr = sg.lr * sqrtf(1.f - powf(sg.p1, step_t)) / (1.f - powf(sg.p0, step_t));
    const long long end = sg.offset + sg.count;
    for (int t = threadIdx.x; t < kOptChunk; t += blockDim.x) {
      const long long i = base + t;
      if (i >= end || i >= total) break;
      float x = w[i];
      if (sg.kind >= 0) {
        float g = to_f32<G>(grad[i]) * inv_scale;
        if (sg.l2 != 0.f) g += sg.l2 * x;
        if (sg.kind == kOptSgd) {
          if (sg.p0 != 0.f) {
            float v = sg.p0 * s0[i] + g;
            s0[i] = v;
            x -= sg.lr * (sg.nesterov ? (sg.p0 * v + g) : v);
          } else {
            x -= sg.lr * g;
          }
        } else if (sg.kind == kOptAdam) {
          if (isfinite(g)) {
            const float m1 = sg.p0 * s0[i] + (1.f - sg.p0) * g;
            const float m2 = sg.p1 * s1[i] + (1.f - sg.p1) * g * g;
            s0[i] = m1; s1[i] = m2;
            x -= sg.corr * (m1 / (sqrtf(m2) + sg.eps)) + sg.lr * sg.wd * x;
          }
        } else if (sg.kind == kOptAdagrad) {
          const float c = s0[i] + g * g;
          s0[i] = c;
          x -= sg.lr * g / (sqrtf(c) + sg.eps);
        } else {
          const float c = sg.p0 * s0[i] + (1.f - sg.p0) * g * g;
          s0[i] = c;
          x -= sg.lr * g / (sqrtf(c) + sg.eps);
        }
        w[i] = x;
      }
      if (w16) w16[i] = from_f32<W16>(x);
    }
  }
}


// ---------------------------------------------------------------------------------
// One element of any of the update rules above; s0 / s1 are updated in place.
__device__ __forceinline__ float opt_update_one(const OptSegment& sg, float x, float g, float& s0,
                                                float& s1) {
  if (sg.l2 != 0.f) g += sg.l2 * x;
  if (sg.kind == kOptSgd) {
    if (sg.p0 != 0.f) {
      const float v = sg.p0 * s0 + g;
      s0 = v;
      x -= sg.lr * (sg.nesterov ? (sg.p0 * v + g) : v);
    } else {
      x -= sg.lr * g;
    }
  } else if (sg.kind == kOptAdam) {
    if (isfinite(g)) {
      const float m1 = sg.p0 * s0 + (1.f - sg.p0) * g;
      const float m2 = sg.p1 * s1 + (1.f - sg.p1) * g * g;
      s0 = m1; s1 = m2;
      x -= sg.corr * (m1 / (sqrtf(m2) + sg.eps)) + sg.lr * sg.wd * x;
    }
  } else if (sg.kind == kOptAdagrad) {
    const float c = s0 + g * g;
    s0 = c;
    x -= sg.lr * g / (sqrtf(c) + sg.eps);
  } else {
    const float c = sg.p0 * s0 + (1.f - sg.p0) * g * g;
    s0 = c;
    x -= sg.lr * g / (sqrtf(c) + sg.eps);
  }
  return x;
}

// Peers of a sharded update: the fp32 master arenas of the ranks of the group (index = rank).
struct OptPeers {
  float* w[8];
};

// Ownership of the arena when the optimizer is sharded over `world` ranks: blocks of
// `own_chunks` chunks are dealt round-robin, block b belongs to rank b % world.  Any long
// range of the arena is then spread evenly over the ranks, whichever weight tensors it holds.
__device__ __forceinline__ bool chunk_owned(long long ch, int rank, int world, int own_chunks) {
  return world <= 1 || (int)((ch / own_chunks) % world) == rank;
}

// Vectorised update of the chunks this rank owns (all chunks when world == 1): four
// elements per thread and 16-byte accesses.  With peers, the new fp32 values of an owned
// chunk are also STORED into every other rank's master arena over NVLink, which is the
// all-gather that follows a sharded update (rank q then only casts its arena to 16 bits);
// gradients and optimizer state are touched on the owner alone.
template <typename G, typename W16>
__global__ void __launch_bounds__(256)
fused_optimizer_vec_kernel(float* __restrict__ w, const G* __restrict__ grad,
                           float* __restrict__ s0, float* __restrict__ s1, W16* __restrict__ w16,
                           const OptSegment* __restrict__ segs, int nseg, long long total,
                           float inv_scale, const int* __restrict__ skip_flag,
                           const int* __restrict__ step_ptr,
                           const float* __restrict__ lr_scale_ptr,
                           const float* __restrict__ inv_scale_dev, int rank, int world,
                           int own_chunks, OptPeers peers, int compact_state) {
  if (skip_flag && *skip_flag) return;
  if (inv_scale_dev) inv_scale *= *inv_scale_dev;
  const float step_t = step_ptr ? (float)(*step_ptr) : 1.f;
  const float lr_mul = lr_scale_ptr ? *lr_scale_ptr : 1.f;
  const long long nchunks = (total + kOptChunk - 1) / kOptChunk;
  // owned chunks are enumerated densely so that every block of the grid has work
  const long long nblocks = (nchunks + own_chunks - 1) / own_chunks;
  const long long mine = world <= 1 ? nblocks : (nblocks - rank + world - 1) / world;
  const long long nowned = mine * own_chunks;
  const bool has_s1 = s1 != s0;
  for (long long k = blockIdx.x; k < nowned; k += gridDim.x) {
    const long long ch = world <= 1 ? k
                                    : ((k / own_chunks) * world + rank) * own_chunks + k % own_chunks;
    if (ch >= nchunks) continue;
    const long long base = ch * kOptChunk;
    const int si = find_segment(segs, nseg, base);
    OptSegment sg = segs[si];
    sg.lr *= lr_mul;
    if (sg.kind == kOptAdam)
      sg.corr = sg.lr * sqrtf(1.f - powf(sg.p1, step_t)) / (1.f - powf(sg.p0, step_t));
    long long end = sg.offset + sg.count;
    if (end > total) end = total;
    const long long i = base + 4 * (long long)threadIdx.x;
    if (i >= end) continue;
    const int nv = end - i >= 4 ? 4 : (int)(end - i);
    // optimizer state: at the element's arena offset, or - when only the owned blocks have
    // state storage - at its position in the dense enumeration of this rank's chunks
    const long long is = compact_state ? k * kOptChunk + 4 * (long long)threadIdx.x : i;
    float x[4], g[4], a0[4], a1[4];
    if (nv == 4) {
      const float4 xv = *reinterpret_cast<const float4*>(w + i);
      x[0] = xv.x; x[1] = xv.y; x[2] = xv.z; x[3] = xv.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) x[j] = j < nv ? w[i + j] : 0.f;
    }
    if (sg.kind >= 0) {
      if (nv == 4) {
        if (sizeof(G) == 4) {
          const float4 gv = *reinterpret_cast<const float4*>(grad + i);
          g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
        } else {
          const uint2 gv = *reinterpret_cast<const uint2*>(grad + i);
          const G* e = reinterpret_cast<const G*>(&gv);
#pragma unroll
          for (int j = 0; j < 4; ++j) g[j] = to_f32<G>(e[j]);
        }
        const float4 v0 = *reinterpret_cast<const float4*>(s0 + is);
        a0[0] = v0.x; a0[1] = v0.y; a0[2] = v0.z; a0[3] = v0.w;
        if (has_s1) {
          const float4 v1 = *reinterpret_cast<const float4*>(s1 + is);
          a1[0] = v1.x; a1[1] = v1.y; a1[2] = v1.z; a1[3] = v1.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          g[j] = j < nv ? to_f32<G>(grad[i + j]) : 0.f;
          a0[j] = j < nv ? s0[is + j] : 0.f;
          a1[j] = (j < nv && has_s1) ? s1[is + j] : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) x[j] = opt_update_one(sg, x[j], g[j] * inv_scale, a0[j], a1[j]);
      if (nv == 4) {
        *reinterpret_cast<float4*>(s0 + is) = make_float4(a0[0], a0[1], a0[2], a0[3]);
        if (has_s1 && sg.kind == kOptAdam)
          *reinterpret_cast<float4*>(s1 + is) = make_float4(a1[0], a1[1], a1[2], a1[3]);
        *reinterpret_cast<float4*>(w + i) = make_float4(x[0], x[1], x[2], x[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j >= nv) continue;
          s0[is + j] = a0[j];
          if (has_s1 && sg.kind == kOptAdam) s1[is + j] = a1[j];
          w[i + j] = x[j];
        }
      }
    }
    if (world > 1 && sg.kind >= 0) {   // frozen tensors are not the optimizer's to publish
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float* dst = peers.w[q];
        if (!dst) continue;
        if (nv == 4) {
          *reinterpret_cast<float4*>(dst + i) = make_float4(x[0], x[1], x[2], x[3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (j < nv) dst[i + j] = x[j];
        }
      }
    }
    if (w16 && world <= 1) {
      if (nv == 4) {
        uint2 o;
        W16* e = reinterpret_cast<W16*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) e[j] = from_f32<W16>(x[j]);
        *reinterpret_cast<uint2*>(w16 + i) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < nv) w16[i + j] = from_f32<W16>(x[j]);
      }
    }
  }
}

// flag |= any non-finite; optionally g *= inv_scale in place.
template <typename G>
__global__ void unscale_check_kernel(G* __restrict__ grad, long long n, float inv_scale,
                                     const float* __restrict__ inv_scale_dev, int write_back,
                                     int* __restrict__ flag, int rank, int world, int own_chunks) {
  if (inv_scale_dev) inv_scale = *inv_scale_dev;     // loss scale kept on the device
  bool bad = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    // sharded update: only the owner holds the reduced gradient of a chunk
    if (!chunk_owned(i / kOptChunk, rank, world, own_chunks)) continue;
    const float g = to_f32<G>(grad[i]) * inv_scale;
    if (!isfinite(g)) bad = true;
    if (write_back) grad[i] = from_f32<G>(g);
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(flag, 1);
}

// Loss-scale schedule of automatic mixed precision, on the device so that a training step
// needs no host decision (src/models/model.cpp:1796-1824 is the schedule): after an overflow
// the scale shrinks and the step is skipped, after `interval` clean steps it grows.
// state = {scale, 1 / scale, clean steps, consecutive skipped steps, 1 / scale of the step
// that just ran (what the optimizer unscales this step's gradients with)}; reduced: the overflow
// flag after the max-reduction over the ranks (nullptr on one rank); flag: this rank's flag
// on entry, the decision the optimizer reads on exit.
__global__ void amp_update_kernel(float* __restrict__ state, const float* __restrict__ reduced,
                                  int* __restrict__ flag, float growth, float backoff,
                                  float interval) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const bool bad = reduced ? (*reduced > 0.f) : (*flag != 0);
  *flag = bad ? 1 : 0;
  float scale = state[0], good = state[2], skipped = state[3];
  state[4] = state[1];
  if (bad) {
    scale *= backoff;
    good = 0.f;
    skipped += 1.f;
  } else {
    skipped = 0.f;
    good += 1.f;
    if (good >= interval) {
      scale *= growth;
      good = 0.f;
    }
  }
  state[0] = scale;
  state[1] = 1.f / scale;
  state[2] = good;
  state[3] = skipped;
}

// out[0] += sum x^2
template <typename G>
__global__ void sqnorm_kernel(const G* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f32<G>(x[i]);
    s += v * v;
  }
  s = warp_sum(s);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = s;
  __syncthreads();
  if (warp == 0) {
    float r = lane < (blockDim.x >> 5) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    if (lane == 0) atomicAdd(out, r);
  }
}

// dst = cast(src) with scale (weights fp32 -> 16-bit copy, gradient casts)
template <typename S, typename D>
__global__ void cast_scale_kernel(const S* __restrict__ src, D* __restrict__ dst, long long n,
                                  float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = from_f32<D>(to_f32<S>(src[i]) * scale);
}

static int flat_grid(long long n, int per_block) {
  const long long blocks = (n + per_block - 1) / per_block;
  const long long cap = (long long)lbhost::sm_count() * 8;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace lb

extern "C" {

int lb_opt_segment_bytes() { return (int)sizeof(lb::OptSegment); }
int lb_opt_chunk() { return lb::kOptChunk; }

// step_ptr: device int holding the 1-based step number (Adam bias correction);
// lr_scale_ptr: optional device float multiplied into every learning rate.
// w, s0, s1: fp32 arenas.  grad: arena of grad_dtype.  w16: optional 16-bit weight copy of
// w16_dtype (pass null to skip).  segs: device array of nseg OptSegment sorted by offset.
int lb_fused_optimizer(float* w, const void* grad, float* s0, float* s1, void* w16,
                       const void* segs, int nseg, long long total, float inv_scale,
                       const int* skip_flag, const int* step_ptr, const float* lr_scale_ptr,
                       const float* inv_scale_dev, int grad_dtype, int w16_dtype, void* stream_) {
  using namespace lb;
  if (total <= 0 || nseg <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = flat_grid(total, kOptChunk);
  const OptSegment* sg = reinterpret_cast<const OptSegment*>(segs);
#define LB_OPT(G, W)                                                                      \
  fused_optimizer_kernel<G, W><<<grid, 256, 0, s>>>(w, (const G*)grad, s0, s1, (W*)w16, sg, \
                                                    nseg, total, inv_scale, skip_flag,     \
                                                    step_ptr, lr_scale_ptr, inv_scale_dev)
  const bool wb = (w16_dtype == kBF16);
  if (grad_dtype == kF32) { if (wb) LB_OPT(float, __nv_bfloat16); else LB_OPT(float, __half); }
  else if (grad_dtype == kBF16) { if (wb) LB_OPT(__nv_bfloat16, __nv_bfloat16); else LB_OPT(__nv_bfloat16, __half); }
  else { if (wb) LB_OPT(__half, __nv_bfloat16); else LB_OPT(__half, __half); }
#undef LB_OPT
  return (int)cudaGetLastError();
}

int lb_amp_update(float* state, const float* reduced, int* flag, float growth, float backoff,
                  float interval, void* stream_) {
  lb::amp_update_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      state, reduced, flag, growth, backoff, interval);
  return (int)cudaGetLastError();
}

// inv_scale_dev: when not null the factor is read from device memory instead of `inv_scale`.
int lb_unscale_check_owned(void* grad, long long n, float inv_scale, const float* inv_scale_dev,
                           int write_back, int* flag, int dtype, int rank, int world,
                           int own_chunks, void* stream_) {
  using namespace lb;
  if (n <= 0) return 0;
  if (world < 1 || rank < 0 || rank >= world || own_chunks < 1) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = flat_grid(n, 2048);
  if (dtype == kF32) unscale_check_kernel<float><<<grid, 256, 0, s>>>((float*)grad, n, inv_scale, inv_scale_dev, write_back, flag, rank, world, own_chunks);
  else if (dtype == kBF16) unscale_check_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)grad, n, inv_scale, inv_scale_dev, write_back, flag, rank, world, own_chunks);
  else unscale_check_kernel<__half><<<grid, 256, 0, s>>>((__half*)grad, n, inv_scale, inv_scale_dev, write_back, flag, rank, world, own_chunks);
  return (int)cudaGetLastError();
}

int lb_unscale_check(void* grad, long long n, float inv_scale, const float* inv_scale_dev,
                     int write_back, int* flag, int dtype, void* stream_) {
  return lb_unscale_check_owned(grad, n, inv_scale, inv_scale_dev, write_back, flag, dtype, 0, 1, 1,
                                stream_);
}

// Sharded form of lb_fused_optimizer: updates the chunks that `rank` owns (blocks of
// own_chunks chunks dealt round-robin over `world` ranks) and stores their new fp32 values
// into the master arenas of the other ranks (peer_w: host array of `world` device pointers,
// peer-mapped; entry `rank` is ignored).  With world == 1 it is the whole update and also
// refreshes the 16-bit copy; with world > 1 the 16-bit copy is left to a cast of the arena
// once every rank's stores have landed.
// compact_state != 0: s0 / s1 hold state for the owned blocks only, densely, in block order
// (owned block j = arena block j * world + rank): ceil-divided share of the arena per rank.
int lb_fused_optimizer_sharded2(float* w, const void* grad, float* s0, float* s1, void* w16,
                                const void* segs, int nseg, long long total, float inv_scale,
                                const int* skip_flag, const int* step_ptr,
                                const float* lr_scale_ptr, const float* inv_scale_dev,
                                int grad_dtype, int w16_dtype, int rank, int world, int own_chunks,
                                void* const* peer_w, int compact_state, void* stream_) {
  using namespace lb;
  if (total <= 0 || nseg <= 0) return 0;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || own_chunks < 1) return -1;
  if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(grad) |
       reinterpret_cast<uintptr_t>(s0) | reinterpret_cast<uintptr_t>(s1)) & 15) return -1;
  OptPeers peers;
  for (int r = 0; r < 8; ++r) {
    peers.w[r] = (world > 1 && r < world && r != rank && peer_w) ? (float*)peer_w[r] : nullptr;
    if (reinterpret_cast<uintptr_t>(peers.w[r]) & 15) return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long nchunks = (total + kOptChunk - 1) / kOptChunk;
  const int grid = flat_grid((nchunks + world - 1) / world * kOptChunk, kOptChunk);
  const OptSegment* sg = reinterpret_cast<const OptSegment*>(segs);
#define LB_OPTV(G, W)                                                                        \
  fused_optimizer_vec_kernel<G, W><<<grid, 256, 0, s>>>(                                     \
      w, (const G*)grad, s0, s1, (W*)w16, sg, nseg, total, inv_scale, skip_flag, step_ptr,   \
      lr_scale_ptr, inv_scale_dev, rank, world, own_chunks, peers, compact_state)
  const bool wb = (w16_dtype == kBF16);
  if (grad_dtype == kF32) { if (wb) LB_OPTV(float, __nv_bfloat16); else LB_OPTV(float, __half); }
  else if (grad_dtype == kBF16) { if (wb) LB_OPTV(__nv_bfloat16, __nv_bfloat16); else LB_OPTV(__nv_bfloat16, __half); }
  else { if (wb) LB_OPTV(__half, __nv_bfloat16); else LB_OPTV(__half, __half); }
#undef LB_OPTV
  return (int)cudaGetLastError();
}

int lb_fused_optimizer_sharded(float* w, const void* grad, float* s0, float* s1, void* w16,
                               const void* segs, int nseg, long long total, float inv_scale,
                               const int* skip_flag, const int* step_ptr,
                               const float* lr_scale_ptr, const float* inv_scale_dev,
                               int grad_dtype, int w16_dtype, int rank, int world, int own_chunks,
                               void* const* peer_w, void* stream_) {
  return lb_fused_optimizer_sharded2(w, grad, s0, s1, w16, segs, nseg, total, inv_scale, skip_flag,
                                     step_ptr, lr_scale_ptr, inv_scale_dev, grad_dtype, w16_dtype,
                                     rank, world, own_chunks, peer_w, 0, stream_);
}

int lb_sqnorm(const void* x, long long n, float* out, int dtype, void* stream_) {
  using namespace lb;
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = flat_grid(n, 4096);
  if (dtype == kF32) sqnorm_kernel<float><<<grid, 256, 0, s>>>((const float*)x, n, out);
  else if (dtype == kBF16) sqnorm_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, n, out);
  else sqnorm_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, n, out);
  return (int)cudaGetLastError();
}

int lb_cast_scale(const void* src, void* dst, long long n, float scale, int src_dtype,
                  int dst_dtype, void* stream_) {
  using namespace lb;
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = flat_grid(n, 2048);
#define LB_CAST(S, D) cast_scale_kernel<S, D><<<grid, 256, 0, s>>>((const S*)src, (D*)dst, n, scale)
  if (src_dtype == kF32 && dst_dtype == kBF16) LB_CAST(float, __nv_bfloat16);
  else if (src_dtype == kF32 && dst_dtype == kF16) LB_CAST(float, __half);
  else if (src_dtype == kF32 && dst_dtype == kF32) LB_CAST(float, float);
  else if (src_dtype == kBF16 && dst_dtype == kF32) LB_CAST(__nv_bfloat16, float);
  else if (src_dtype == kF16 && dst_dtype == kF32) LB_CAST(__half, float);
  else if (src_dtype == kBF16 && dst_dtype == kBF16) LB_CAST(__nv_bfloat16, __nv_bfloat16);
  else if (src_dtype == kF16 && dst_dtype == kF16) LB_CAST(__half, __half);
  else return -1;
#undef LB_CAST
  return (int)cudaGetLastError();
}

}  // extern "C"
