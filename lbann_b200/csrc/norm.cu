// Normalisation kernels.
//
// Layer norm (rows = samples x leading dims, columns = normalised size), forward and
// backward with optional scale / bias, statistics in fp32
// (reference: src/layers/regularizers/layer_norm.cu:257-330,576-644).
//
// Batch norm on channels-last data (rows = N x spatial, columns = channels) in three
// phases so a cross-GPU reduction of the 2C partial sums can be placed between them
// (reference: src/layers/regularizers/batch_normalization.cu:64-371; the variance uses
// the same Bessel correction and epsilon clamp, :139-146):
//   bn_partial_sums   -> sums[2][C]            (sum x, sum x^2)
//   bn_finalize_apply -> mean/var/running stats, y = (x-mean)*rsqrt(var+eps)*scale+bias
//   bn_bwd_sums       -> dscale, dbias, dmean, dvar partials; bn_bwd_apply -> dx
// Instance norm reuses the batch-norm kernels with one "batch" per sample.
#include "common.cuh"

namespace lb {

template <typename T>
__device__ __forceinline__ void ld8n(const T* p, float (&f)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ void st8n(T* p, const float (&f)[8]) {
  uint4 q;
  T* e = reinterpret_cast<T*>(&q);
#pragma unroll
  for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(f[j]);
  *reinterpret_cast<uint4*>(p) = q;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

// ------------------------------- layer norm ---------------------------------
// One block per row (grid-stride over rows).  cols may be any size; vector path when
// cols % 8 == 0 and pointers are 16-byte aligned (16-bit types) else scalar.
template <typename T>
__global__ void layer_norm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ scale,
                                      const float* __restrict__ bias, T* __restrict__ y,
                                      float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                      long long rows, int cols, float eps) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    float s = 0.f, ss = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = to_f32<T>(xr[c]);
      s += v; ss += v * v;
    }
    s = block_sum(s, scratch);
    ss = block_sum(ss, scratch);
    const float mean = s / cols;
    float var = ss / cols - mean * mean;
    var = var > 0.f ? var : 0.f;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) { mean_out[r] = mean; rstd_out[r] = rstd; }
    T* yr = y + r * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float v = (to_f32<T>(xr[c]) - mean) * rstd;
      if (scale) v *= scale[c];
      if (bias) v += bias[c];
      yr[c] = from_f32<T>(v);
    }
  }
}

// dx for one row per block; dscale/dbias accumulated with atomics into fp32 buffers.
template <typename T>
__global__ void layer_norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                      const float* __restrict__ scale,
                                      const float* __restrict__ mean_in,
                                      const float* __restrict__ rstd_in, T* __restrict__ dx,
                                      float* __restrict__ dscale, float* __restrict__ dbias,
                                      long long rows, int cols) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    const T* gr = dy + r * cols;
    const float mean = mean_in[r], rstd = rstd_in[r];
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float xh = (to_f32<T>(xr[c]) - mean) * rstd;
      const float g = to_f32<T>(gr[c]) * (scale ? scale[c] : 1.f);
      s1 += g; s2 += g * xh;
    }
    s1 = block_sum(s1, scratch) / cols;
    s2 = block_sum(s2, scratch) / cols;
    T* dr = dx + r * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float xh = (to_f32<T>(xr[c]) - mean) * rstd;
      const float gy = to_f32<T>(gr[c]);
      const float g = gy * (scale ? scale[c] : 1.f);
      dr[c] = from_f32<T>((g - s1 - xh * s2) * rstd);
    }
  }
}

// Column reductions for dscale / dbias: each block owns a band of rows and a tile of
// 32*VEC columns; partial sums are combined with atomics.
template <typename T>
__global__ void layer_norm_param_grad_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                             const float* __restrict__ mean_in,
                                             const float* __restrict__ rstd_in,
                                             float* __restrict__ dscale, float* __restrict__ dbias,
                                             long long rows, int cols, long long rows_per_block) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  float a = 0.f, b = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const float g = to_f32<T>(dy[r * cols + c]);
    a += g * (to_f32<T>(x[r * cols + c]) - mean_in[r]) * rstd_in[r];
    b += g;
  }
  if (dscale) atomicAdd(dscale + c, a);
  if (dbias) atomicAdd(dbias + c, b);
}

// Sum an 8-wide register array over threadIdx.y; the result is valid where threadIdx.y == 0.
// blockDim.x is a power of two <= 32 and the block has 256 threads.  Lanes of a warp that
// share threadIdx.x are combined with shuffles first, so shared memory only carries one
// partial per warp and the closing serial sum is 8 terms long (it used to be blockDim.y
// terms, which left the memory system idle for microseconds at the end of every block).
// `sm` holds 8 warps x 8 values x blockDim.x floats.  Every thread of the block must call it.
__device__ __forceinline__ void reduce_over_y(float (&a)[8], float* sm) {
  const int bx = blockDim.x;
  for (int off = bx; off < 32; off <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += __shfl_xor_sync(0xffffffffu, a[j], off);
  }
  const int tid = threadIdx.y * bx + threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, nw = (bx * blockDim.y) >> 5;
  __syncthreads();
  if (lane < bx) {
#pragma unroll
    for (int j = 0; j < 8; ++j) sm[(warp * 8 + j) * bx + lane] = a[j];
  }
  __syncthreads();
  if (threadIdx.y == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.f;
      for (int w = 0; w < nw; ++w) t += sm[(w * 8 + j) * bx + threadIdx.x];
      a[j] = t;
    }
  }
}

// dscale / dbias of layer norm for 16-bit tensors with cols % 8 == 0: a thread owns eight
// columns (one 16-byte load per tensor and row), the 8 row lanes of a block stride over a band
// of rows four at a time, the band is folded over threadIdx.y and added with atomics.  Reads
// x and dy once at vector width (the one-column-per-thread kernel above moved 2 bytes per
// load and ran at ~0.5 TB/s).
template <typename T>
__global__ void __launch_bounds__(256)
layer_norm_param_grad8_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                              const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                              float* __restrict__ dscale, float* __restrict__ dbias, long long rows,
                              int cols, long long rows_per_block) {
  __shared__ float sm[256 * 8];
  const int cv = cols / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = v < cv;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  float a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.f;
  if (active) {
    const long long base = (long long)v * 8;
    const int ny = blockDim.y;
    long long r = r0 + threadIdx.y;
    for (; r + 3LL * ny < r1; r += 4LL * ny) {
      float fx[4][8], fg[4][8], mu[4], rs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        ld8n<T>(x + (r + (long long)u * ny) * cols + base, fx[u]);
        ld8n<T>(dy + (r + (long long)u * ny) * cols + base, fg[u]);
        mu[u] = mean_in[r + (long long)u * ny];
        rs[u] = rstd_in[r + (long long)u * ny];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a[j] += fg[u][j] * (fx[u][j] - mu[u]) * rs[u];
          b[j] += fg[u][j];
        }
      }
    }
    for (; r < r1; r += ny) {
      float fx[8], fg[8];
      ld8n<T>(x + r * cols + base, fx);
      ld8n<T>(dy + r * cols + base, fg);
      const float mu = mean_in[r], rs = rstd_in[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] += fg[j] * (fx[j] - mu) * rs;
        b[j] += fg[j];
      }
    }
  }
  reduce_over_y(a, sm);
  reduce_over_y(b, sm);
  if (active && threadIdx.y == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (dscale) atomicAdd(dscale + v * 8 + j, a[j]);
      if (dbias) atomicAdd(dbias + v * 8 + j, b[j]);
    }
  }
}

// ------------------------------- batch norm ---------------------------------
// x: [groups][rows][C] channels-last; each group has its own statistics (groups = 1 for
// batch norm, = N for instance norm).  Threads: x -> 8-channel vectors, y -> row lanes.
template <typename T>
__global__ void bn_partial_sums_kernel(const T* __restrict__ x, float* __restrict__ sums,
                                       long long rows, int C, long long rows_per_block,
                                       int replicas) {
  __shared__ float sm[256 * 8];
  const int cv = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int grp = blockIdx.z;
  const bool valid = v < cv;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  float s[8], ss[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.f; ss[j] = 0.f; }
  const T* base = x + ((long long)grp * rows) * C + v * 8;
  if (valid) {
    // four rows' loads are issued before the first is used (the pass is a pure streaming
    // read, so bytes in flight per thread are what sets its bandwidth)
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
      ld8n<T>(base + r * C, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) { s[j] += f[j]; ss[j] += f[j] * f[j]; }
    }
  }
  reduce_over_y(s, sm);
  reduce_over_y(ss, sm);
  if (valid && threadIdx.y == 0) {
    // Hundreds of blocks add into the same few cache lines, and the L2 serialises atomics on
    // a line (592 blocks x 32 floats per line cost 37 us on a 51 MB activation, four times the
    // read itself): the blocks are spread over `replicas` copies that the caller sums.
    float* out = sums + ((long long)(blockIdx.y % replicas) * gridDim.z + grp) * 2 * C;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(out + v * 8 + j, s[j]);
      atomicAdd(out + C + v * 8 + j, ss[j]);
    }
  }
}

// stats[grp] = {mean[C], var[C]} computed from sums (already reduced over all ranks),
// `count` = elements per channel over all ranks.  Running statistics are updated by the
// first row-block.  act: 0 none, 1 relu, 2 leaky(act_param).
template <typename T>
__global__ void bn_finalize_apply_kernel(const T* __restrict__ x, const float* __restrict__ sums,
                                         const float* __restrict__ scale,
                                         const float* __restrict__ bias, T* __restrict__ y,
                                         float* __restrict__ stats, float* __restrict__ run_mean,
                                         float* __restrict__ run_var, long long rows, int C,
                                         long long rows_per_block, float count, float correction,
                                         float eps, float decay, int act, float act_param) {
  const int cv = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int grp = blockIdx.z;
  if (v >= cv) return;
  float mean[8], mul[8], add[8];
  const float* sg = sums + (long long)grp * 2 * C;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = v * 8 + j;
    const float m = sg[c] / count;
    const float sq = sg[C + c] / count;
    float var = count * (sq - m * m) / (count - correction);
    var = var > eps ? var : eps;
    const float rstd = rsqrtf(var + eps);
    mean[j] = m;
    mul[j] = rstd * (scale ? scale[c] : 1.f);
    add[j] = bias ? bias[c] : 0.f;
    if (blockIdx.y == 0 && threadIdx.y == 0) {
      stats[(long long)grp * 2 * C + c] = m;
      stats[(long long)grp * 2 * C + C + c] = var;
      if (run_mean) {
        run_mean[c] = decay * run_mean[c] + (1.f - decay) * m;
        run_var[c] = decay * run_var[c] + (1.f - decay) * var;
      }
    }
  }
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  const long long base = ((long long)grp * rows) * C + v * 8;
#pragma unroll 4
  for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
    float f[8];
    ld8n<T>(x + base + r * C, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float o = (f[j] - mean[j]) * mul[j] + add[j];
      if (act == 1) o = o > 0.f ? o : 0.f;
      else if (act == 2) o = o > 0.f ? o : act_param * o;
      f[j] = o;
    }
    st8n<T>(y + base + r * C, f);
  }
}

// Inference / fixed statistics: y = (x - mean) * rsqrt(var + eps) * scale + bias
template <typename T>
__global__ void bn_apply_fixed_kernel(const T* __restrict__ x, const float* __restrict__ mean_in,
                                      const float* __restrict__ var_in,
                                      const float* __restrict__ scale,
                                      const float* __restrict__ bias, T* __restrict__ y,
                                      long long rows, int C, long long rows_per_block, float eps,
                                      int act, float act_param) {
  const int cv = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= cv) return;
  float mean[8], mul[8], add[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = v * 8 + j;
    mean[j] = mean_in[c];
    mul[j] = rsqrtf(var_in[c] + eps) * (scale ? scale[c] : 1.f);
    add[j] = bias ? bias[c] : 0.f;
  }
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
#pragma unroll 4
  for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
    float f[8];
    ld8n<T>(x + r * C + v * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float o = (f[j] - mean[j]) * mul[j] + add[j];
      if (act == 1) o = o > 0.f ? o : 0.f;
      else if (act == 2) o = o > 0.f ? o : act_param * o;
      f[j] = o;
    }
    st8n<T>(y + r * C + v * 8, f);
  }
}

// bsums[grp] = {dscale[C], dbias[C], dmean[C], dvar[C]} partials (reference :250-300).
// If act != 0 the gradient is first masked with the sign of the activation output y.
template <typename T>
__global__ void bn_bwd_sums_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                   const T* __restrict__ y, const float* __restrict__ stats,
                                   const float* __restrict__ scale, float* __restrict__ bsums,
                                   long long rows, int C, long long rows_per_block, float eps,
                                   int act, float act_param, int replicas) {
  __shared__ float sm[256 * 8];
  const int cv = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int grp = blockIdx.z;
  const bool valid = v < cv;
  // Two running sums per channel are enough: S1 = sum g and S2 = sum g (x - mean); the four
  // outputs are linear in them (dscale = S2 rstd, dbias = S1, dmean = -scale rstd S1,
  // dvar = -scale rstd^3 S2 / 2), which halves the registers and the block reductions.
  float mean[8], s1[8], s2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = valid ? v * 8 + j : 0;
    mean[j] = stats[(long long)grp * 2 * C + c];
    s1[j] = s2[j] = 0.f;
  }
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  const long long base = ((long long)grp * rows) * C + v * 8;
  if (valid) {
#pragma unroll 4
    for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
      float fx[8], fg[8], fy[8];
      ld8n<T>(x + base + r * C, fx);
      ld8n<T>(dy + base + r * C, fg);
      if (act) ld8n<T>(y + base + r * C, fy);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float g = fg[j];
        if (act == 1) g = fy[j] > 0.f ? g : 0.f;
        else if (act == 2) g = fy[j] > 0.f ? g : act_param * g;
        s1[j] += g;
        s2[j] += g * (fx[j] - mean[j]);
      }
    }
  }
  reduce_over_y(s1, sm);
  reduce_over_y(s2, sm);
  if (valid && threadIdx.y == 0) {
    float* out = bsums + ((long long)(blockIdx.y % replicas) * gridDim.z + grp) * 4 * C;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = v * 8 + j;
      const float rstd = rsqrtf(stats[(long long)grp * 2 * C + C + c] + eps);
      const float sc = scale ? scale[c] : 1.f;
      atomicAdd(out + c, s2[j] * rstd);
      atomicAdd(out + C + c, s1[j]);
      atomicAdd(out + 2 * C + c, -sc * rstd * s1[j]);
      atomicAdd(out + 3 * C + c, -0.5f * sc * rstd * rstd * rstd * s2[j]);
    }
  }
}

// dx = dxhat*rstd + dmean/n + dvar*2/(n-corr)*(x-mean)   (reference :302-371)
template <typename T>
__global__ void bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                    const T* __restrict__ y, const float* __restrict__ stats,
                                    const float* __restrict__ scale,
                                    const float* __restrict__ bsums, T* __restrict__ dx,
                                    long long rows, int C, long long rows_per_block, float count,
                                    float correction, float eps, int act, float act_param) {
  const int cv = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int grp = blockIdx.z;
  if (v >= cv) return;
  float mean[8], k0[8], k1[8], k2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = v * 8 + j;
    mean[j] = stats[(long long)grp * 2 * C + c];
    const float rstd = rsqrtf(stats[(long long)grp * 2 * C + C + c] + eps);
    k0[j] = (scale ? scale[c] : 1.f) * rstd;
    k1[j] = bsums[(long long)grp * 4 * C + 2 * C + c] / count;
    k2[j] = bsums[(long long)grp * 4 * C + 3 * C + c] * 2.f / (count - correction);
  }
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  const long long base = ((long long)grp * rows) * C + v * 8;
#pragma unroll 4
  for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
    float fx[8], fg[8], fy[8];
    ld8n<T>(x + base + r * C, fx);
    ld8n<T>(dy + base + r * C, fg);
    if (act) ld8n<T>(y + base + r * C, fy);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = fg[j];
      if (act == 1) g = fy[j] > 0.f ? g : 0.f;
      else if (act == 2) g = fy[j] > 0.f ? g : act_param * g;
      fx[j] = g * k0[j] + k1[j] + k2[j] * (fx[j] - mean[j]);
    }
    st8n<T>(dx + base + r * C, fx);
  }
}

struct BnLaunch {
  dim3 grid, block;
  long long rows_per_block;
};
static BnLaunch bn_shape(long long rows, int C, int groups) {
  BnLaunch l;
  const int cv = C / 8;
  const int bx = cv >= 32 ? 32 : (cv >= 16 ? 16 : (cv >= 8 ? 8 : (cv >= 4 ? 4 : (cv >= 2 ? 2 : 1))));
  const int by = 256 / bx;
  l.block = dim3(bx, by, 1);
  const int gx = (cv + bx - 1) / bx;
  long long want = (long long)lbhost::sm_count() * 4 / (gx * groups);
  if (want < 1) want = 1;
  long long rpb = (rows + want - 1) / want;
  if (rpb < by) rpb = by;
  l.rows_per_block = rpb;
  l.grid = dim3(gx, (unsigned)((rows + rpb - 1) / rpb), groups);
  return l;
}

}  // namespace lb

#define LB_DISPATCH_16(dtype, ...)                                   \
  if (dtype == lb::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else if (dtype == lb::kF16) { using T = __half; __VA_ARGS__; }     \
  else return -1;
#define LB_DISPATCH_ALL(dtype, ...)                                  \
  if (dtype == lb::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else if (dtype == lb::kF16) { using T = __half; __VA_ARGS__; }     \
  else { using T = float; __VA_ARGS__; }

extern "C" {

int lb_layer_norm_fwd(const void* x, const float* scale, const float* bias, void* y, float* mean,
                      float* rstd, long long rows, int cols, float eps, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int threads = cols >= 1024 ? 256 : (cols >= 256 ? 128 : 64);
  const long long cap = (long long)lbhost::sm_count() * 16;
  const int grid = (int)(rows < cap ? rows : cap);
  LB_DISPATCH_ALL(dtype, (layer_norm_fwd_kernel<T><<<grid, threads, 0, s>>>(
                             (const T*)x, scale, bias, (T*)y, mean, rstd, rows, cols, eps)));
  return (int)cudaGetLastError();
}

// dscale / dbias (fp32, may be null) are ACCUMULATED into.
int lb_layer_norm_bwd(const void* x, const void* dy, const float* scale, const float* mean,
                      const float* rstd, void* dx, float* dscale, float* dbias, long long rows,
                      int cols, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int threads = cols >= 1024 ? 256 : (cols >= 256 ? 128 : 64);
  const long long cap = (long long)lbhost::sm_count() * 16;
  const int grid = (int)(rows < cap ? rows : cap);
  LB_DISPATCH_ALL(dtype, (layer_norm_bwd_kernel<T><<<grid, threads, 0, s>>>(
                             (const T*)x, (const T*)dy, scale, mean, rstd, (T*)dx, dscale, dbias,
                             rows, cols)));
  if ((dscale || dbias) && dtype != kF32 && cols % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0) {
    const int cv = cols / 8;
    int bx = 32;
    while (bx > 1 && bx / 2 >= cv) bx /= 2;           // power of two <= 32 covering the vectors
    dim3 block(bx, 256 / bx);
    const int gx = (cv + bx - 1) / bx;
    long long bands = (long long)lbhost::sm_count() * 4 / gx;
    if (bands < 1) bands = 1;
    const long long min_rows = 4LL * block.y;            // at least one unrolled round per block
    if (bands > (rows + min_rows - 1) / min_rows) bands = (rows + min_rows - 1) / min_rows;
    const long long rpb = (rows + bands - 1) / bands;
    dim3 g(gx, (unsigned)((rows + rpb - 1) / rpb));
    LB_DISPATCH_16(dtype, (layer_norm_param_grad8_kernel<T><<<g, block, 0, s>>>(
                              (const T*)x, (const T*)dy, mean, rstd, dscale, dbias, rows, cols, rpb)));
  } else if (dscale || dbias) {
    const int gx = (cols + 127) / 128;
    long long bands = (long long)lbhost::sm_count() * 2 / gx;
    if (bands < 1) bands = 1;
    if (bands > rows) bands = rows;
    const long long rpb = (rows + bands - 1) / bands;
    dim3 g(gx, (unsigned)((rows + rpb - 1) / rpb));
    LB_DISPATCH_ALL(dtype, (layer_norm_param_grad_kernel<T><<<g, 128, 0, s>>>(
                               (const T*)x, (const T*)dy, mean, rstd, dscale, dbias, rows, cols,
                               rpb)));
  }
  return (int)cudaGetLastError();
}

// sums: fp32 [groups][2][C], must be zero on entry.  C % 8 == 0.
// sums: fp32 [replicas][groups][2][C], zero on entry; the caller adds the replicas up.
int lb_bn_partial_sums(const void* x, float* sums, long long rows, int C, int groups, int dtype,
                       int replicas, void* stream_) {
  using namespace lb;
  if (C % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  BnLaunch l = bn_shape(rows, C, groups);
  LB_DISPATCH_16(dtype, (bn_partial_sums_kernel<T><<<l.grid, l.block, 0, s>>>(
                            (const T*)x, sums, rows, C, l.rows_per_block, replicas < 1 ? 1 : replicas)));
  return (int)cudaGetLastError();
}

int lb_bn_finalize_apply(const void* x, const float* sums, const float* scale, const float* bias,
                         void* y, float* stats, float* run_mean, float* run_var, long long rows,
                         int C, int groups, float count, float correction, float eps, float decay,
                         int act, float act_param, int dtype, void* stream_) {
  using namespace lb;
  if (C % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  BnLaunch l = bn_shape(rows, C, groups);
  LB_DISPATCH_16(dtype, (bn_finalize_apply_kernel<T><<<l.grid, l.block, 0, s>>>(
                            (const T*)x, sums, scale, bias, (T*)y, stats, run_mean, run_var, rows,
                            C, l.rows_per_block, count, correction, eps, decay, act, act_param)));
  return (int)cudaGetLastError();
}

int lb_bn_apply_fixed(const void* x, const float* mean, const float* var, const float* scale,
                      const float* bias, void* y, long long rows, int C, float eps, int act,
                      float act_param, int dtype, void* stream_) {
  using namespace lb;
  if (C % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  BnLaunch l = bn_shape(rows, C, 1);
  LB_DISPATCH_16(dtype, (bn_apply_fixed_kernel<T><<<l.grid, l.block, 0, s>>>(
                            (const T*)x, mean, var, scale, bias, (T*)y, rows, C, l.rows_per_block,
                            eps, act, act_param)));
  return (int)cudaGetLastError();
}

// bsums: fp32 [replicas][groups][4][C], zero on entry; the caller adds the replicas up.
int lb_bn_bwd_sums(const void* x, const void* dy, const void* y, const float* stats,
                   const float* scale, float* bsums, long long rows, int C, int groups, float eps,
                   int act, float act_param, int dtype, int replicas, void* stream_) {
  using namespace lb;
  if (C % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  BnLaunch l = bn_shape(rows, C, groups);
  LB_DISPATCH_16(dtype, (bn_bwd_sums_kernel<T><<<l.grid, l.block, 0, s>>>(
                            (const T*)x, (const T*)dy, (const T*)y, stats, scale, bsums, rows, C,
                            l.rows_per_block, eps, act, act_param, replicas < 1 ? 1 : replicas)));
  return (int)cudaGetLastError();
}

int lb_bn_bwd_apply(const void* x, const void* dy, const void* y, const float* stats,
                    const float* scale, const float* bsums, void* dx, long long rows, int C,
                    int groups, float count, float correction, float eps, int act,
                    float act_param, int dtype, void* stream_) {
  using namespace lb;
  if (C % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  BnLaunch l = bn_shape(rows, C, groups);
  LB_DISPATCH_16(dtype, (bn_bwd_apply_kernel<T><<<l.grid, l.block, 0, s>>>(
                            (const T*)x, (const T*)dy, (const T*)y, stats, scale, bsums, (T*)dx,
                            rows, C, l.rows_per_block, count, correction, eps, act, act_param)));
  return (int)cudaGetLastError();
}

}  // extern "C"
