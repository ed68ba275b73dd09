// Max / average pooling forward and backward on channels-last tensors
// ([N][D][H][W][C], 2-D uses D = 1), 8 channels (16 bytes) per thread.
// Modes follow the reference's pooling layer (include/lbann/layers/transform/pooling.hpp:56-66):
// 0 = max, 1 = average counting padding, 2 = average not counting padding.
// The backward pass is a gather (no atomics, deterministic): every input position
// visits the windows that contain it; for max pooling the gradient goes to the first
// maximum of a window in scan order, which is recomputed from x.
#include "common.cuh"

namespace lb {

struct PoolGeom {
  int N, D, H, W, C;
  int Do, Ho, Wo;
  int kd, kh, kw;
  int pd, ph, pw;
  int sd, sh, sw;
  int mode;
};

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&f)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&f)[8]) {
  uint4 q;
  T* e = reinterpret_cast<T*>(&q);
#pragma unroll
  for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(f[j]);
  *reinterpret_cast<uint4*>(p) = q;
}

// `idx` (optional, max pooling): one byte per output element, dense [N][Do][Ho][Wo][C]: the
// position of the first maximum in the window's scan order (kd, kh, kw nested) in bits 0-6
// and "the maximum is positive" in bit 7.  The backward kernel of non-overlapping windows
// then needs neither x nor y: it reads dy and these bytes (0.2 GB instead of 1.2 GB for
// the first pooling layer of CosmoFlow).
template <typename T>
__global__ void pool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, PoolGeom g,
                                long long xs_n, long long xs_d, long long xs_h, long long xs_w,
                                long long y_sn, long long total, uint8_t* __restrict__ idx) {
  const int cv = g.C / 8;
  const long long per_sample = (long long)g.Do * g.Ho * g.Wo * g.C;   // dense part of a sample
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int c8 = r % cv; r /= cv;
    const int ow = r % g.Wo; r /= g.Wo;
    const int oh = r % g.Ho; r /= g.Ho;
    const int od = r % g.Do; r /= g.Do;
    const int n = (int)r;
    float acc[8];
    int arg[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[j] = g.mode == 0 ? -INFINITY : 0.f; arg[j] = 0; }
    int count = 0;
    for (int a = 0; a < g.kd; ++a) {
      const int id = od * g.sd - g.pd + a;
      if (id < 0 || id >= g.D) continue;
      for (int b = 0; b < g.kh; ++b) {
        const int ih = oh * g.sh - g.ph + b;
        if (ih < 0 || ih >= g.H) continue;
        for (int c = 0; c < g.kw; ++c) {
          const int iw = ow * g.sw - g.pw + c;
          if (iw < 0 || iw >= g.W) continue;
          float f[8];
          ld8<T>(x + n * xs_n + id * xs_d + ih * xs_h + iw * xs_w + c8 * 8, f);
          if (idx) {
            const int pos = (a * g.kh + b) * g.kw + c;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (f[j] > acc[j]) { acc[j] = f[j]; arg[j] = pos; }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = g.mode == 0 ? fmaxf(acc[j], f[j]) : acc[j] + f[j];
          }
          ++count;
        }
      }
    }
    if (idx) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= (uint32_t)((arg[j] & 0x7f) | (acc[j] > 0.f ? 0x80 : 0)) << (8 * j);
        hi |= (uint32_t)((arg[j + 4] & 0x7f) | (acc[j + 4] > 0.f ? 0x80 : 0)) << (8 * j);
      }
      *reinterpret_cast<uint2*>(idx + i * 8) = make_uint2(lo, hi);
    }
    if (g.mode == 1) {
      const float inv = 1.f / (g.kd * g.kh * g.kw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= inv;
    } else if (g.mode == 2) {
      const float inv = count > 0 ? 1.f / count : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= inv;
    }
    st8<T>(y + n * y_sn + (i * 8 - n * per_sample), acc);
  }
}

__device__ __forceinline__ int ceil_div_pos(int a, int b) { return a >= 0 ? (a + b - 1) / b : 0; }

template <typename T>
__global__ void pool_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                T* __restrict__ dx, PoolGeom g, long long xs_n, long long xs_d,
                                long long xs_h, long long xs_w, long long total) {
  const int cv = g.C / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int c8 = r % cv; r /= cv;
    const int iw = r % g.W; r /= g.W;
    const int ih = r % g.H; r /= g.H;
    const int id = r % g.D; r /= g.D;
    const int n = (int)r;
    float xin[8], acc[8];
    const T* xn = x + n * xs_n + c8 * 8;
    if (g.mode == 0) ld8<T>(xn + id * xs_d + ih * xs_h + iw * xs_w, xin);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // windows (od, oh, ow) containing this input position
    const int od_lo = ceil_div_pos(id + g.pd - g.kd + 1, g.sd), od_hi = min((id + g.pd) / g.sd, g.Do - 1);
    const int oh_lo = ceil_div_pos(ih + g.ph - g.kh + 1, g.sh), oh_hi = min((ih + g.ph) / g.sh, g.Ho - 1);
    const int ow_lo = ceil_div_pos(iw + g.pw - g.kw + 1, g.sw), ow_hi = min((iw + g.pw) / g.sw, g.Wo - 1);
    for (int od = od_lo; od <= od_hi; ++od)
      for (int oh = oh_lo; oh <= oh_hi; ++oh)
        for (int ow = ow_lo; ow <= ow_hi; ++ow) {
          float gy[8];
          ld8<T>(dy + ((((long long)n * g.Do + od) * g.Ho + oh) * g.Wo + ow) * g.C + c8 * 8, gy);
          if (g.mode == 0) {
            // am I the first maximum of this window?
            bool first[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) first[j] = true;
            for (int a = 0; a < g.kd; ++a) {
              const int zd = od * g.sd - g.pd + a;
              if (zd < 0 || zd >= g.D) continue;
              for (int b = 0; b < g.kh; ++b) {
                const int zh = oh * g.sh - g.ph + b;
                if (zh < 0 || zh >= g.H) continue;
                for (int c = 0; c < g.kw; ++c) {
                  const int zw = ow * g.sw - g.pw + c;
                  if (zw < 0 || zw >= g.W) continue;
                  if (zd == id && zh == ih && zw == iw) continue;
                  const bool before = (zd < id) || (zd == id && (zh < ih || (zh == ih && zw < iw)));
                  float f[8];
                  ld8<T>(xn + zd * xs_d + zh * xs_h + zw * xs_w, f);
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (f[j] > xin[j] || (before && f[j] == xin[j])) first[j] = false;
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (first[j]) acc[j] += gy[j];
          } else if (g.mode == 1) {
            const float inv = 1.f / (g.kd * g.kh * g.kw);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += gy[j] * inv;
          } else {
            const int d0 = max(od * g.sd - g.pd, 0), d1 = min(od * g.sd - g.pd + g.kd, g.D);
            const int h0 = max(oh * g.sh - g.ph, 0), h1 = min(oh * g.sh - g.ph + g.kh, g.H);
            const int w0 = max(ow * g.sw - g.pw, 0), w1 = min(ow * g.sw - g.pw + g.kw, g.W);
            const float inv = 1.f / ((d1 - d0) * (h1 - h0) * (w1 - w0));
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += gy[j] * inv;
          }
        }
    st8<T>(dx + i * 8, acc);
  }
}

static int pool_grid(long long total) {
  const long long blocks = (total + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace lb

extern "C" {

// geom: 18 ints = N D H W C Do Ho Wo kd kh kw pd ph pw sd sh sw mode.  C % 8 == 0.
// y and dx are dense NDHWC; x may be strided (xs = n, d, h, w strides in elements).
int lb_pool_fwd_strided(const void* x, void* y, const int* geom, const long long* xs,
                        long long y_sn, int dtype, void* stream_);
int lb_pool_fwd_idx(const void* x, void* y, void* idx, const int* geom, const long long* xs,
                    long long y_sn, int dtype, void* stream_);
int lb_pool_fwd(const void* x, void* y, const int* geom, const long long* xs, int dtype,
                void* stream_) {
  return lb_pool_fwd_strided(x, y, geom, xs, 0, dtype, stream_);
}

// y_sn: elements between consecutive samples of y (0 = dense); a sample itself is dense.
int lb_pool_fwd_strided(const void* x, void* y, const int* geom, const long long* xs,
                        long long y_sn, int dtype, void* stream_) {
  return lb_pool_fwd_idx(x, y, nullptr, geom, xs, y_sn, dtype, stream_);
}

// Max pooling that also records where each maximum sits (see pool_fwd_kernel); idx: dense
// bytes [N][Do][Ho][Wo][C], 8-byte aligned, windows of at most 128 positions.
int lb_pool_fwd_idx(const void* x, void* y, void* idx, const int* geom, const long long* xs,
                    long long y_sn, int dtype, void* stream_) {
  using namespace lb;
  PoolGeom g;
  memcpy(&g, geom, sizeof(g));
  if (g.C % 8) return -1;
  if (idx && (g.mode != 0 || g.kd * g.kh * g.kw > 128 || (reinterpret_cast<uintptr_t>(idx) & 7)))
    return -1;
  if (y_sn == 0) y_sn = (long long)g.Do * g.Ho * g.Wo * g.C;
  if (y_sn % 8 || (reinterpret_cast<uintptr_t>(y) & 15)) return -1;
  const long long total = (long long)g.N * g.Do * g.Ho * g.Wo * (g.C / 8);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == kBF16)
    pool_fwd_kernel<__nv_bfloat16><<<pool_grid(total), 256, 0, s>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)y, g, xs[0], xs[1], xs[2], xs[3], y_sn, total,
        (uint8_t*)idx);
  else if (dtype == kF16)
    pool_fwd_kernel<__half><<<pool_grid(total), 256, 0, s>>>((const __half*)x, (__half*)y, g,
                                                             xs[0], xs[1], xs[2], xs[3], y_sn, total,
                                                             (uint8_t*)idx);
  else
    return -1;
  return (int)cudaGetLastError();
}

int lb_pool_bwd(const void* x, const void* dy, void* dx, const int* geom, const long long* xs,
                int dtype, void* stream_) {
  using namespace lb;
  PoolGeom g;
  memcpy(&g, geom, sizeof(g));
  if (g.C % 8) return -1;
  const long long total = (long long)g.N * g.D * g.H * g.W * (g.C / 8);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == kBF16)
    pool_bwd_kernel<__nv_bfloat16><<<pool_grid(total), 256, 0, s>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, g, xs[0], xs[1],
        xs[2], xs[3], total);
  else if (dtype == kF16)
    pool_bwd_kernel<__half><<<pool_grid(total), 256, 0, s>>>(
        (const __half*)x, (const __half*)dy, (__half*)dx, g, xs[0], xs[1], xs[2], xs[3], total);
  else
    return -1;
  return (int)cudaGetLastError();
}

}  // extern "C"
