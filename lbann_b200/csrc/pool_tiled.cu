// Backward of non-overlapping max pooling (window == stride, no padding, input extents
// divisible by the window) on channels-last tensors, optionally fused with the gradient
// of a ReLU / leaky-ReLU that produced the pooled tensor:
//
//   dx[p] = (p is the first maximum of its window) ? dy[window] * act'(x[p]) : 0
//
// One thread owns one window and 8 channels: it reads the window once, finds the arg-max
// and writes every dx position of the window, so dx is written exactly once and x is read
// exactly once (the general gather kernel in pool.cu re-scans windows per input element).
// This is the shape of every pooling layer of CosmoFlow and U-Net
// (reference: cuDNN pooling backward, src/layers/transform/pooling.cpp:129-176, followed
// by a separate activation backward kernel).
#include "common.cuh"

namespace lb {

struct TiledPoolGeom {
  int N, D, H, W, C;     // input dims
  int kd, kh, kw;        // window == stride
};

template <typename T>
__global__ void pool_bwd_tiled_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                      T* __restrict__ dx, TiledPoolGeom g, int act,
                                      float act_param, long long dx_sn, long long total) {
  const int cv = g.C / 8;
  const int Do = g.D / g.kd, Ho = g.H / g.kh, Wo = g.W / g.kw;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int c8 = r % cv; r /= cv;
    const int ow = r % Wo; r /= Wo;
    const int oh = r % Ho; r /= Ho;
    const int od = r % Do; r /= Do;
    const long long n = r;
    float best[8], gy[8], bestx[8];
    int arg[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; arg[j] = 0; bestx[j] = 0.f; }
    {
      uint4 q = *reinterpret_cast<const uint4*>(dy + i * 8);
      const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) gy[j] = to_f32<T>(e[j]);
    }
    const long long base = (((n * g.D + (long long)od * g.kd) * g.H + (long long)oh * g.kh) * g.W +
                            (long long)ow * g.kw) * g.C + c8 * 8;
    // dx may leave a gap between samples (it is then the inside of a tensor with halo planes)
    const long long dbase = base + n * (dx_sn - (long long)g.D * g.H * g.W * g.C);
    int pos = 0;
    for (int a = 0; a < g.kd; ++a)
      for (int b = 0; b < g.kh; ++b)
        for (int c = 0; c < g.kw; ++c, ++pos) {
          const long long off = base + (((long long)a * g.H + b) * g.W + c) * g.C;
          uint4 q = *reinterpret_cast<const uint4*>(x + off);
          const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float v = to_f32<T>(e[j]);
            if (v > best[j]) { best[j] = v; arg[j] = pos; }
          }
        }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f = 1.f;
      if (act == kActRelu) f = best[j] > 0.f ? 1.f : 0.f;
      else if (act == kActLeaky) f = best[j] > 0.f ? 1.f : act_param;
      gy[j] *= f;
    }
    pos = 0;
    for (int a = 0; a < g.kd; ++a)
      for (int b = 0; b < g.kh; ++b)
        for (int c = 0; c < g.kw; ++c, ++pos) {
          const long long off = base + (((long long)a * g.H + b) * g.W + c) * g.C;
          uint4 q;
          T* e = reinterpret_cast<T*>(&q);
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(arg[j] == pos ? gy[j] : 0.f);
          *reinterpret_cast<uint4*>(dx + off + (dbase - base)) = q;
        }
  }
}

// Forward of the same windows: a thread owns one window and 8 channels, issues all of the
// window's 16-byte loads before the first comparison (a 2x2x2 window keeps eight loads in
// flight per thread) and records the position of the first maximum (bits 0-6) and whether it
// is positive (bit 7) in one byte per output element.  y may leave a gap between samples.
template <typename T, int KD, int KH, int KW>
__global__ void pool_fwd_tiled_kernel(const T* __restrict__ x, T* __restrict__ y,
                                      uint8_t* __restrict__ idx, TiledPoolGeom g, long long xs_n,
                                      long long xs_d, long long xs_h, long long xs_w,
                                      long long y_sn, long long total) {
  const int cv = g.C / 8;
  const int Do = g.D / KD, Ho = g.H / KH, Wo = g.W / KW;
  const long long per_sample = (long long)Do * Ho * Wo * g.C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int c8 = r % cv; r /= cv;
    const int ow = r % Wo; r /= Wo;
    const int oh = r % Ho; r /= Ho;
    const int od = r % Do; r /= Do;
    const long long n = r;
    const T* base = x + n * xs_n + (long long)od * KD * xs_d + (long long)oh * KH * xs_h +
                    (long long)ow * KW * xs_w + c8 * 8;
    uint4 q[KD * KH * KW];
#pragma unroll
    for (int a = 0; a < KD; ++a)
#pragma unroll
      for (int b = 0; b < KH; ++b)
#pragma unroll
        for (int c = 0; c < KW; ++c)
          q[(a * KH + b) * KW + c] = *reinterpret_cast<const uint4*>(base + a * xs_d + b * xs_h + c * xs_w);
    float best[8];
    int arg[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; arg[j] = 0; }
#pragma unroll
    for (int pos = 0; pos < KD * KH * KW; ++pos) {
      const T* e = reinterpret_cast<const T*>(&q[pos]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = to_f32<T>(e[j]);
        const bool gt = v > best[j];
        best[j] = gt ? v : best[j];
        arg[j] = gt ? pos : arg[j];
      }
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) oe[j] = from_f32<T>(best[j]);
    *reinterpret_cast<uint4*>(y + n * y_sn + (i * 8 - n * per_sample)) = o;
    if (idx) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= (uint32_t)(arg[j] | (best[j] > 0.f ? 0x80 : 0)) << (8 * j);
        hi |= (uint32_t)(arg[j + 4] | (best[j + 4] > 0.f ? 0x80 : 0)) << (8 * j);
      }
      *reinterpret_cast<uint2*>(idx + i * 8) = make_uint2(lo, hi);
    }
  }
}

// The same from the positions recorded by the forward kernel (pool.cu: one byte per output
// element, bits 0-6 the arg-max in scan order, bit 7 "maximum positive"): reads dy and the
// bytes, writes dx once.
template <typename T>
__global__ void pool_bwd_tiled_idx_kernel(const uint8_t* __restrict__ idx, const T* __restrict__ dy,
                                          T* __restrict__ dx, TiledPoolGeom g, int act,
                                          float act_param, long long dx_sn, long long total) {
  const int cv = g.C / 8;
  const int Do = g.D / g.kd, Ho = g.H / g.kh, Wo = g.W / g.kw;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int c8 = r % cv; r /= cv;
    const int ow = r % Wo; r /= Wo;
    const int oh = r % Ho; r /= Ho;
    const int od = r % Do; r /= Do;
    const long long n = r;
    float gy[8];
    int arg[8];
    {
      const uint4 q = *reinterpret_cast<const uint4*>(dy + i * 8);
      const T* e = reinterpret_cast<const T*>(&q);
      const uint2 b = *reinterpret_cast<const uint2*>(idx + i * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t v = ((j < 4 ? b.x : b.y) >> (8 * (j & 3))) & 0xffu;
        arg[j] = (int)(v & 0x7fu);
        float f = 1.f;
        if (act == kActRelu) f = (v & 0x80u) ? 1.f : 0.f;
        else if (act == kActLeaky) f = (v & 0x80u) ? 1.f : act_param;
        gy[j] = to_f32<T>(e[j]) * f;
      }
    }
    const long long base = n * dx_sn + ((((long long)od * g.kd) * g.H + (long long)oh * g.kh) * g.W +
                                        (long long)ow * g.kw) * g.C + c8 * 8;
    int pos = 0;
    for (int a = 0; a < g.kd; ++a)
      for (int b = 0; b < g.kh; ++b)
        for (int c = 0; c < g.kw; ++c, ++pos) {
          const long long off = base + (((long long)a * g.H + b) * g.W + c) * g.C;
          uint4 q;
          T* e = reinterpret_cast<T*>(&q);
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(arg[j] == pos ? gy[j] : 0.f);
          *reinterpret_cast<uint4*>(dx + off) = q;
        }
  }
}

}  // namespace lb

extern "C" {

// geom: N D H W C kd kh kw (8 ints); x, dx dense NDHWC, dy dense [N][D/kd][H/kh][W/kw][C].
// act: 0 none, 1 relu, 2 leaky(act_param) - derivative taken from the sign of x.
int lb_pool_bwd_tiled_strided(const void* x, const void* dy, void* dx, const int* geom, int act,
                              float act_param, long long dx_sn, int dtype, void* stream_);
int lb_pool_bwd_tiled(const void* x, const void* dy, void* dx, const int* geom, int act,
                      float act_param, int dtype, void* stream_) {
  return lb_pool_bwd_tiled_strided(x, dy, dx, geom, act, act_param, 0, dtype, stream_);
}

// dx_sn: elements between consecutive samples of dx (0 = dense).
int lb_pool_bwd_tiled_strided(const void* x, const void* dy, void* dx, const int* geom, int act,
                              float act_param, long long dx_sn, int dtype, void* stream_) {
  using namespace lb;
  TiledPoolGeom g;
  memcpy(&g, geom, sizeof(g));
  if (g.C % 8 || g.D % g.kd || g.H % g.kh || g.W % g.kw) return -1;
  if (dx_sn == 0) dx_sn = (long long)g.D * g.H * g.W * g.C;
  if (dx_sn % 8 || (reinterpret_cast<uintptr_t>(dx) & 15)) return -1;
  const long long total = (long long)g.N * (g.D / g.kd) * (g.H / g.kh) * (g.W / g.kw) * (g.C / 8);
  if (total <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long blocks = (total + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 32;
  const int grid = (int)(blocks < cap ? blocks : cap);
  if (dtype == kBF16)
    pool_bwd_tiled_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, g, act, act_param, dx_sn, total);
  else if (dtype == kF16)
    pool_bwd_tiled_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, (const __half*)dy,
                                                       (__half*)dx, g, act, act_param, dx_sn, total);
  else
    return -1;
  return (int)cudaGetLastError();
}

// Forward max pooling over non-overlapping 2x2x2 / 1x2x2 / 2x2 windows (the shapes of every
// pooling layer of CosmoFlow, U-Net and the ResNet stem are covered by 2 and 3).  Returns -2
// for other windows: the caller then uses the general kernel.  x strided (xs: n, d, h, w in
// elements), y dense per sample with y_sn elements between samples, idx optional.
int lb_pool_fwd_tiled(const void* x, void* y, void* idx, const int* geom, const long long* xs,
                      long long y_sn, int dtype, void* stream_) {
  using namespace lb;
  TiledPoolGeom g;
  memcpy(&g, geom, sizeof(g));
  if (g.C % 8 || g.D % g.kd || g.H % g.kh || g.W % g.kw) return -2;
  const bool k222 = g.kd == 2 && g.kh == 2 && g.kw == 2, k122 = g.kd == 1 && g.kh == 2 && g.kw == 2;
  if (!k222 && !k122) return -2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || xs[0] % 8 || xs[1] % 8 || xs[2] % 8 || xs[3] % 8) return -2;
  const long long per_sample = (long long)(g.D / g.kd) * (g.H / g.kh) * (g.W / g.kw) * g.C;
  if (y_sn == 0) y_sn = per_sample;
  if (y_sn % 8 || (reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(idx) & 7)) return -1;
  const long long total = (long long)g.N * per_sample / 8;
  if (total <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long blocks = (total + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 32;
  const int grid = (int)(blocks < cap ? blocks : cap);
#define LB_POOL_FWD(T, KD)                                                                         \
  pool_fwd_tiled_kernel<T, KD, 2, 2><<<grid, 256, 0, s>>>((const T*)x, (T*)y, (uint8_t*)idx, g, xs[0], \
                                                          xs[1], xs[2], xs[3], y_sn, total)
  if (dtype == kBF16) { if (k222) LB_POOL_FWD(__nv_bfloat16, 2); else LB_POOL_FWD(__nv_bfloat16, 1); }
  else if (dtype == kF16) { if (k222) LB_POOL_FWD(__half, 2); else LB_POOL_FWD(__half, 1); }
  else return -2;
#undef LB_POOL_FWD
  return (int)cudaGetLastError();
}

// idx: the bytes written by lb_pool_fwd_idx / lb_pool_fwd_tiled for the same geometry.
int lb_pool_bwd_tiled_idx(const void* idx, const void* dy, void* dx, const int* geom, int act,
                          float act_param, long long dx_sn, int dtype, void* stream_) {
  using namespace lb;
  TiledPoolGeom g;
  memcpy(&g, geom, sizeof(g));
  if (g.C % 8 || g.D % g.kd || g.H % g.kh || g.W % g.kw || g.kd * g.kh * g.kw > 128) return -1;
  if (dx_sn == 0) dx_sn = (long long)g.D * g.H * g.W * g.C;
  if (dx_sn % 8 || (reinterpret_cast<uintptr_t>(dx) & 15) || (reinterpret_cast<uintptr_t>(idx) & 7)) return -1;
  const long long total = (long long)g.N * (g.D / g.kd) * (g.H / g.kh) * (g.W / g.kw) * (g.C / 8);
  if (total <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long blocks = (total + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 32;
  const int grid = (int)(blocks < cap ? blocks : cap);
  if (dtype == kBF16)
    pool_bwd_tiled_idx_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        (const uint8_t*)idx, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, g, act, act_param, dx_sn, total);
  else if (dtype == kF16)
    pool_bwd_tiled_idx_kernel<__half><<<grid, 256, 0, s>>>((const uint8_t*)idx, (const __half*)dy,
                                                           (__half*)dx, g, act, act_param, dx_sn, total);
  else
    return -1;
  return (int)cudaGetLastError();
}

}  // extern "C"
