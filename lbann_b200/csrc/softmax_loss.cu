// Row softmax family and per-sample losses.
//
//   softmax / log-softmax forward and backward over the last (contiguous) dimension,
//   with an optional causal mask and input scale (the attention softmax)
//     reference: src/layers/activations/softmax.cu, log_softmax.cu,
//                src/layers/misc/channelwise_softmax.cu:238-319,489-519
//   fused softmax + cross-entropy against integer labels (value and gradient identical to
//   softmax followed by cross_entropy(use_labels); out-of-range label contributes 0)
//     reference: src/layers/loss/cross_entropy.cu:55-73
//   cross-entropy on probabilities (-sum y log yhat over y > 0), mean squared / absolute
//   error, L1 norm, squared L2 norm: one value per sample
//     reference: src/layers/loss/{cross_entropy,mean_squared_error,mean_absolute_error,
//                l1_norm,l2_norm2}.cu
//   categorical / top-k accuracy per sample
//     reference: src/layers/loss/categorical_accuracy.cu, top_k_categorical_accuracy.cu
#include "common.cuh"

namespace lb {

__device__ __forceinline__ float block_reduce_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? scratch[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_reduce_max(float v, float* scratch) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

// mode 0: softmax, 1: log-softmax.  causal_period > 0: row r may only see columns
// <= (r % causal_period) (rows of an S x S score matrix, S = causal_period).
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows,
                                   int cols, int mode, float in_scale, int causal_period) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    T* yr = y + r * cols;
    const int limit = causal_period > 0 ? min(cols, (int)(r % causal_period) + 1) : cols;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < limit; c += blockDim.x) m = fmaxf(m, to_f32<T>(xr[c]) * in_scale);
    m = block_reduce_max(m, scratch);
    float s = 0.f;
    for (int c = threadIdx.x; c < limit; c += blockDim.x) s += __expf(to_f32<T>(xr[c]) * in_scale - m);
    s = block_reduce_sum(s, scratch);
    const float inv = 1.f / s, lse = m + __logf(s);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float o;
      if (c < limit) {
        const float v = to_f32<T>(xr[c]) * in_scale;
        o = mode == 0 ? __expf(v - m) * inv : v - lse;
      } else {
        o = mode == 0 ? 0.f : -INFINITY;
      }
      yr[c] = from_f32<T>(o);
    }
  }
}

// softmax: dx = y * (dy - sum(y*dy)) * in_scale ; log-softmax: dx = (dy - exp(y)*sum(dy)) * in_scale
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                                   T* __restrict__ dx, long long rows, int cols, int mode,
                                   float in_scale, int causal_period) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* yr = y + r * cols;
    const T* gr = dy + r * cols;
    T* dr = dx + r * cols;
    const int limit = causal_period > 0 ? min(cols, (int)(r % causal_period) + 1) : cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < limit; c += blockDim.x) {
      const float g = to_f32<T>(gr[c]);
      s += mode == 0 ? g * to_f32<T>(yr[c]) : g;
    }
    s = block_reduce_sum(s, scratch);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float o = 0.f;
      if (c < limit) {
        const float g = to_f32<T>(gr[c]), yy = to_f32<T>(yr[c]);
        o = (mode == 0 ? yy * (g - s) : g - __expf(yy) * s) * in_scale;
      }
      dr[c] = from_f32<T>(o);
    }
  }
}

// Fused softmax + cross entropy with integer labels.  loss[r] = lse - x[label] (0 if the
// label is out of range); lse[r] saved for backward.
template <typename T>
__global__ void softmax_ce_fwd_kernel(const T* __restrict__ x, const long long* __restrict__ labels,
                                      float* __restrict__ loss, float* __restrict__ lse_out,
                                      long long rows, int cols) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, to_f32<T>(xr[c]));
    m = block_reduce_max(m, scratch);
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(to_f32<T>(xr[c]) - m);
    s = block_reduce_sum(s, scratch);
    if (threadIdx.x == 0) {
      const float lse = m + logf(s);
      lse_out[r] = lse;
      const long long lab = labels[r];
      loss[r] = (lab >= 0 && lab < cols) ? lse - to_f32<T>(xr[lab]) : 0.f;
    }
  }
}

// dx[r][c] = dloss[r] * (softmax - onehot)  (zero row if label out of range)
template <typename T>
__global__ void softmax_ce_bwd_kernel(const T* __restrict__ x, const long long* __restrict__ labels,
                                      const float* __restrict__ lse, const float* __restrict__ dloss,
                                      float dloss_scalar, T* __restrict__ dx, long long rows,
                                      int cols) {
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    T* dr = dx + r * cols;
    const long long lab = labels[r];
    const bool ok = lab >= 0 && lab < cols;
    const float g = ok ? (dloss ? dloss[r] : dloss_scalar) : 0.f;
    const float l = lse[r];
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float p = __expf(to_f32<T>(xr[c]) - l);
      dr[c] = from_f32<T>(g * (p - (c == lab ? 1.f : 0.f)));
    }
  }
}

// Long rows of 16-bit logits (a vocabulary): one pass with 16-byte loads and a running
// (max, sum) pair per thread; the two-pass scalar kernel above read a 100 KB row twice, two
// bytes per load, and ran at a tenth of the copy rate.  cols % 8 == 0, rows 16-byte aligned.
template <typename T>
__global__ void softmax_ce_fwd_vec_kernel(const T* __restrict__ x, const long long* __restrict__ labels,
                                          float* __restrict__ loss, float* __restrict__ lse_out,
                                          long long rows, int cols) {
  __shared__ float scratch[32];
  const int nv = cols / 8;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 q = xv[i];
      const T* e = reinterpret_cast<const T*>(&q);
      float f[8];
      float lm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) { f[j] = to_f32<T>(e[j]); lm = fmaxf(lm, f[j]); }
      if (lm > m) {
        s *= __expf(m - lm);      // m == -inf: s is 0 and stays 0
        m = lm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    }
    const float M = block_reduce_max(m, scratch);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - M);
    s = block_reduce_sum(s, scratch);
    if (threadIdx.x == 0) {
      const float lse = M + logf(s);
      lse_out[r] = lse;
      const long long lab = labels[r];
      loss[r] = (lab >= 0 && lab < cols) ? lse - to_f32<T>(xr[lab]) : 0.f;
    }
  }
}
template <typename T>
__global__ void softmax_ce_bwd_vec_kernel(const T* __restrict__ x, const long long* __restrict__ labels,
                                          const float* __restrict__ lse, const float* __restrict__ dloss,
                                          float dloss_scalar, T* __restrict__ dx, long long rows,
                                          int cols) {
  const int nv = cols / 8;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* xv = reinterpret_cast<const uint4*>(x + r * cols);
    uint4* dv = reinterpret_cast<uint4*>(dx + r * cols);
    const long long lab = labels[r];
    const bool ok = lab >= 0 && lab < cols;
    const float g = ok ? (dloss ? dloss[r] : dloss_scalar) : 0.f;
    const float l = lse[r];
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 q = xv[i];
      const T* e = reinterpret_cast<const T*>(&q);
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p = __expf(to_f32<T>(e[j]) - l);
        oe[j] = from_f32<T>(g * (p - ((long long)i * 8 + j == lab ? 1.f : 0.f)));
      }
      dv[i] = o;
    }
  }
}

// Short rows (a handful of classes per voxel, as in segmentation): one THREAD per row, so a
// warp covers 32 consecutive rows and its loads are contiguous; the block-per-row kernels
// above spend their time in two block reductions over three values.
template <typename T>
__global__ void softmax_ce_fwd_short_kernel(const T* __restrict__ x,
                                            const long long* __restrict__ labels,
                                            float* __restrict__ loss, float* __restrict__ lse_out,
                                            long long rows, int cols) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
       r += (long long)gridDim.x * blockDim.x) {
    const T* xr = x + r * cols;
    float m = -INFINITY;
    for (int c = 0; c < cols; ++c) m = fmaxf(m, to_f32<T>(xr[c]));
    float s = 0.f;
    for (int c = 0; c < cols; ++c) s += __expf(to_f32<T>(xr[c]) - m);
    const float lse = m + logf(s);
    lse_out[r] = lse;
    const long long lab = labels[r];
    loss[r] = (lab >= 0 && lab < cols) ? lse - to_f32<T>(xr[lab]) : 0.f;
  }
}

template <typename T>
__global__ void softmax_ce_bwd_short_kernel(const T* __restrict__ x,
                                            const long long* __restrict__ labels,
                                            const float* __restrict__ lse,
                                            const float* __restrict__ dloss, float dloss_scalar,
                                            T* __restrict__ dx, long long rows, int cols) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
       r += (long long)gridDim.x * blockDim.x) {
    const T* xr = x + r * cols;
    T* dr = dx + r * cols;
    const long long lab = labels[r];
    const bool ok = lab >= 0 && lab < cols;
    const float g = ok ? (dloss ? dloss[r] : dloss_scalar) : 0.f;
    const float l = lse[r];
    for (int c = 0; c < cols; ++c) {
      const float p = __expf(to_f32<T>(xr[c]) - l);
      dr[c] = from_f32<T>(g * (p - (c == lab ? 1.f : 0.f)));
    }
  }
}

constexpr int kShortRowCols = 32;
static int short_row_grid(long long rows) {
  long long b = (rows + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 16;
  if (b > cap) b = cap;
  return (int)(b > 0 ? b : 1);
}

// Per-sample reductions of two inputs.  kind: 0 = CE on probabilities (-sum t*log(p), t>0),
// 1 = MSE (mean of squared diff), 2 = MAE (mean abs diff), 3 = L1 norm of a, 4 = L2^2 of a.
template <typename T>
__global__ void sample_loss_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                       float* __restrict__ out, long long rows, long long cols,
                                       int kind) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* ar = a + r * cols;
    const T* br = b ? b + r * cols : nullptr;
    float s = 0.f;
    for (long long c = threadIdx.x; c < cols; c += blockDim.x) {
      const float p = to_f32<T>(ar[c]);
      const float t = br ? to_f32<T>(br[c]) : 0.f;
      switch (kind) {
        case 0: if (t > 0.f) s += -t * logf(p); break;
        case 1: s += (p - t) * (p - t); break;
        case 2: s += fabsf(p - t); break;
        case 3: s += fabsf(p); break;
        default: s += p * p; break;
      }
    }
    s = block_reduce_sum(s, scratch);
    if (threadIdx.x == 0) out[r] = (kind == 1 || kind == 2) ? s / cols : s;
  }
}

// Gradients: da (and db where defined) given dloss per sample.
template <typename T>
__global__ void sample_loss_bwd_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                       const float* __restrict__ dloss, T* __restrict__ da,
                                       T* __restrict__ db, long long rows, long long cols,
                                       int kind) {
  const long long total = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float g = dloss[i / cols];
    const float p = to_f32<T>(a[i]);
    const float t = b ? to_f32<T>(b[i]) : 0.f;
    float ga = 0.f, gb = 0.f;
    switch (kind) {
      case 0: if (t > 0.f) { ga = -g * t / p; gb = -g * logf(p); } break;
      case 1: ga = 2.f * (p - t) * g / cols; gb = -ga; break;
      case 2: ga = (p > t ? 1.f : (p < t ? -1.f : 0.f)) * g / cols; gb = -ga; break;
      case 3: ga = (p > 0.f ? 1.f : (p < 0.f ? -1.f : 0.f)) * g; break;
      default: ga = 2.f * p * g; break;
    }
    if (da) da[i] = from_f32<T>(ga);
    if (db) db[i] = from_f32<T>(gb);
  }
}

// out[r] = 1 if the label's score is among the k largest of the row (ties broken towards
// lower indices, as a stable descending sort would), else 0.  labels: integer class ids.
template <typename T>
__global__ void topk_accuracy_kernel(const T* __restrict__ x, const long long* __restrict__ labels,
                                     float* __restrict__ out, long long rows, int cols, int k) {
  __shared__ float scratch[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    const long long lab = labels[r];
    float cnt = 0.f;
    if (lab >= 0 && lab < cols) {
      const float v = to_f32<T>(xr[lab]);
      for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float o = to_f32<T>(xr[c]);
        if (o > v || (o == v && c < lab)) cnt += 1.f;
      }
    }
    cnt = block_reduce_sum(cnt, scratch);
    if (threadIdx.x == 0) out[r] = (lab >= 0 && lab < cols && cnt < k) ? 1.f : 0.f;
  }
}

static int row_grid(long long rows) {
  const long long cap = (long long)lbhost::sm_count() * 16;
  return (int)(rows < cap ? (rows > 0 ? rows : 1) : cap);
}
static int row_threads(long long cols) { return cols >= 2048 ? 256 : (cols >= 512 ? 128 : 64); }

}  // namespace lb

#define LB_DISPATCH_ALL(dtype, ...)                                  \
  if (dtype == lb::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else if (dtype == lb::kF16) { using T = __half; __VA_ARGS__; }     \
  else { using T = float; __VA_ARGS__; }

extern "C" {

int lb_softmax_fwd(const void* x, void* y, long long rows, int cols, int mode, float in_scale,
                   int causal_period, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  LB_DISPATCH_ALL(dtype, (softmax_fwd_kernel<T><<<row_grid(rows), row_threads(cols), 0, s>>>(
                             (const T*)x, (T*)y, rows, cols, mode, in_scale, causal_period)));
  return (int)cudaGetLastError();
}
int lb_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int cols, int mode,
                   float in_scale, int causal_period, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  LB_DISPATCH_ALL(dtype, (softmax_bwd_kernel<T><<<row_grid(rows), row_threads(cols), 0, s>>>(
                             (const T*)y, (const T*)dy, (T*)dx, rows, cols, mode, in_scale,
                             causal_period)));
  return (int)cudaGetLastError();
}
int lb_softmax_ce_fwd(const void* x, const long long* labels, float* loss, float* lse,
                      long long rows, int cols, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (cols <= kShortRowCols && rows >= 4096) {
    LB_DISPATCH_ALL(dtype, (softmax_ce_fwd_short_kernel<T><<<short_row_grid(rows), 256, 0, s>>>(
                               (const T*)x, labels, loss, lse, rows, cols)));
    return (int)cudaGetLastError();
  }
  if (dtype != kF32 && cols % 8 == 0 && cols >= 2048 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    if (dtype == kBF16)
      softmax_ce_fwd_vec_kernel<__nv_bfloat16><<<row_grid(rows), 256, 0, s>>>(
          (const __nv_bfloat16*)x, labels, loss, lse, rows, cols);
    else
      softmax_ce_fwd_vec_kernel<__half><<<row_grid(rows), 256, 0, s>>>((const __half*)x, labels, loss,
                                                                        lse, rows, cols);
    return (int)cudaGetLastError();
  }
  LB_DISPATCH_ALL(dtype, (softmax_ce_fwd_kernel<T><<<row_grid(rows), row_threads(cols), 0, s>>>(
                             (const T*)x, labels, loss, lse, rows, cols)));
  return (int)cudaGetLastError();
}
int lb_softmax_ce_bwd(const void* x, const long long* labels, const float* lse, const float* dloss,
                      float dloss_scalar, void* dx, long long rows, int cols, int dtype,
                      void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (cols <= kShortRowCols && rows >= 4096) {
    LB_DISPATCH_ALL(dtype, (softmax_ce_bwd_short_kernel<T><<<short_row_grid(rows), 256, 0, s>>>(
                               (const T*)x, labels, lse, dloss, dloss_scalar, (T*)dx, rows, cols)));
    return (int)cudaGetLastError();
  }
  if (dtype != kF32 && cols % 8 == 0 && cols >= 2048 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0) {
    if (dtype == kBF16)
      softmax_ce_bwd_vec_kernel<__nv_bfloat16><<<row_grid(rows), 256, 0, s>>>(
          (const __nv_bfloat16*)x, labels, lse, dloss, dloss_scalar, (__nv_bfloat16*)dx, rows, cols);
    else
      softmax_ce_bwd_vec_kernel<__half><<<row_grid(rows), 256, 0, s>>>(
          (const __half*)x, labels, lse, dloss, dloss_scalar, (__half*)dx, rows, cols);
    return (int)cudaGetLastError();
  }
  LB_DISPATCH_ALL(dtype, (softmax_ce_bwd_kernel<T><<<row_grid(rows), row_threads(cols), 0, s>>>(
                             (const T*)x, labels, lse, dloss, dloss_scalar, (T*)dx, rows, cols)));
  return (int)cudaGetLastError();
}
int lb_sample_loss_fwd(const void* a, const void* b, float* out, long long rows, long long cols,
                       int kind, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  LB_DISPATCH_ALL(dtype, (sample_loss_fwd_kernel<T><<<row_grid(rows), 256, 0, s>>>(
                             (const T*)a, (const T*)b, out, rows, cols, kind)));
  return (int)cudaGetLastError();
}
int lb_sample_loss_bwd(const void* a, const void* b, const float* dloss, void* da, void* db,
                       long long rows, long long cols, int kind, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long total = rows * cols;
  const long long blocks = (total + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 16;
  const int grid = (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
  LB_DISPATCH_ALL(dtype, (sample_loss_bwd_kernel<T><<<grid, 256, 0, s>>>(
                             (const T*)a, (const T*)b, dloss, (T*)da, (T*)db, rows, cols, kind)));
  return (int)cudaGetLastError();
}
int lb_topk_accuracy(const void* x, const long long* labels, float* out, long long rows, int cols,
                     int k, int dtype, void* stream_) {
  using namespace lb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  LB_DISPATCH_ALL(dtype, (topk_accuracy_kernel<T><<<row_grid(rows), row_threads(cols), 0, s>>>(
                             (const T*)x, labels, out, rows, cols, k)));
  return (int)cudaGetLastError();
}

}  // extern "C"
