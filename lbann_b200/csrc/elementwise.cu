// Entrywise operator set (forward and backward) with 16-byte vectorised I/O in
// fp32 / bf16 / fp16.  One kernel body, op selected by code; the math runs in fp32.
// Covers the reference's operator layers (src/operators/math/{unary,binary,
// binary_with_constant,clamp,select,abs}.cu, src/operators/activations/activations.cu,
// src/operators/loss/entrywise.cu) and the activation layers relu / leaky_relu / elu /
// identity (src/layers/activations/*.cu).
#include "common.cuh"

namespace lb {

// Keep in sync with lbann_b200/ops/elementwise.py
enum UnaryOp : int {
  U_IDENTITY = 0, U_LOGICAL_NOT, U_ABS, U_NEGATIVE, U_SIGN, U_ROUND, U_CEIL, U_FLOOR,
  U_RECIPROCAL, U_SQUARE, U_SQRT, U_RSQRT, U_SAFE_RECIPROCAL, U_EXP, U_EXPM1, U_LOG, U_LOG1P,
  U_COS, U_SIN, U_TAN, U_ACOS, U_ASIN, U_ATAN, U_COSH, U_SINH, U_TANH, U_ACOSH, U_ASINH,
  U_ATANH, U_ERF, U_ERFINV, U_GELU, U_LOG_SIGMOID, U_SELU, U_SIGMOID, U_SOFTPLUS, U_SOFTSIGN,
  U_RELU, U_LEAKY_RELU, U_ELU, U_ADD_CONST, U_SCALE, U_SUB_CONST, U_CONST_SUB, U_MAX_CONST,
  U_MIN_CONST, U_EQ_CONST, U_NE_CONST, U_LT_CONST, U_LE_CONST, U_GT_CONST, U_GE_CONST, U_CLAMP,
  U_GELU_TANH, U_COUNT
};
enum BinaryOp : int {
  B_ADD = 0, B_SUB, B_MUL, B_DIV, B_MOD, B_POW, B_SAFE_DIV, B_SQ_DIFF, B_MAX, B_MIN, B_EQ, B_NE,
  B_LT, B_LE, B_GT, B_GE, B_AND, B_OR, B_XOR, B_BCE, B_SIGMOID_BCE, B_BOOL_ACC, B_BOOL_FN,
  B_BOOL_FP, B_ADD_RELU, B_COUNT
};

__device__ __forceinline__ float unary_fwd(int op, float x, float p0, float p1) {
  switch (op) {
    case U_IDENTITY: return x;
    case U_LOGICAL_NOT: return x != 0.f ? 0.f : 1.f;
    case U_ABS: return fabsf(x);
    case U_NEGATIVE: return -x;
    case U_SIGN: return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f);
    case U_ROUND: return roundf(x);
    case U_CEIL: return ceilf(x);
    case U_FLOOR: return floorf(x);
    case U_RECIPROCAL: return 1.f / x;
    case U_SQUARE: return x * x;
    case U_SQRT: return sqrtf(x);
    case U_RSQRT: return rsqrtf(x);
    case U_SAFE_RECIPROCAL: { float y = 1.f / x; return isfinite(y) ? y : 0.f; }
    case U_EXP: return expf(x);
    case U_EXPM1: return expm1f(x);
    case U_LOG: return logf(x);
    case U_LOG1P: return log1pf(x);
    case U_COS: return cosf(x);
    case U_SIN: return sinf(x);
    case U_TAN: return tanf(x);
    case U_ACOS: return acosf(x);
    case U_ASIN: return asinf(x);
    case U_ATAN: return atanf(x);
    case U_COSH: return coshf(x);
    case U_SINH: return sinhf(x);
    case U_TANH: return tanhf(x);
    case U_ACOSH: return acoshf(x);
    case U_ASINH: return asinhf(x);
    case U_ATANH: return atanhf(x);
    case U_ERF: return erff(x);
    case U_ERFINV: return erfinvf(x);
    case U_GELU: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case U_GELU_TANH: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case U_LOG_SIGMOID: return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x));
    case U_SELU: {
      const float a = 1.6732632423543772f, s = 1.0507009873554805f;
      return x > 0.f ? s * x : s * a * expm1f(x);
    }
    case U_SIGMOID: return 1.f / (1.f + expf(-x));
    case U_SOFTPLUS: return x > 0.f ? x + log1pf(expf(-x)) : log1pf(expf(x));
    case U_SOFTSIGN: return x / (1.f + fabsf(x));
    case U_RELU: return x > 0.f ? x : 0.f;
    case U_LEAKY_RELU: return x > 0.f ? x : p0 * x;
    case U_ELU: return x > 0.f ? x : p0 * expm1f(x);
    case U_ADD_CONST: return x + p0;
    case U_SCALE: return x * p0;
    case U_SUB_CONST: return x - p0;
    case U_CONST_SUB: return p0 - x;
    case U_MAX_CONST: return fmaxf(x, p0);
    case U_MIN_CONST: return fminf(x, p0);
    case U_EQ_CONST: return x == p0 ? 1.f : 0.f;
    case U_NE_CONST: return x != p0 ? 1.f : 0.f;
    case U_LT_CONST: return x < p0 ? 1.f : 0.f;
    case U_LE_CONST: return x <= p0 ? 1.f : 0.f;
    case U_GT_CONST: return x > p0 ? 1.f : 0.f;
    case U_GE_CONST: return x >= p0 ? 1.f : 0.f;
    case U_CLAMP: return fminf(fmaxf(x, p0), p1);
    default: return x;
  }
}

// d(op)/dx * dy
__device__ __forceinline__ float unary_bwd(int op, float x, float dy, float p0, float p1) {
  switch (op) {
    case U_IDENTITY: return dy;
    case U_ABS: return x > 0.f ? dy : (x < 0.f ? -dy : 0.f);
    case U_NEGATIVE: return -dy;
    case U_RECIPROCAL: return -dy / (x * x);
    case U_SQUARE: return 2.f * x * dy;
    case U_SQRT: return dy / (2.f * sqrtf(x));
    case U_RSQRT: { const float s = sqrtf(x); return -dy / (2.f * x * s); }
    case U_SAFE_RECIPROCAL: { float y = 1.f / x; return isfinite(y) ? -dy * y * y : 0.f; }
    case U_EXP: return dy * expf(x);
    case U_EXPM1: return dy * expf(x);
    case U_LOG: return dy / x;
    case U_LOG1P: return dy / (x + 1.f);
    case U_COS: return -dy * sinf(x);
    case U_SIN: return dy * cosf(x);
    case U_TAN: { const float c = cosf(x); return dy / (c * c); }
    case U_ACOS: return -dy / sqrtf(1.f - x * x);
    case U_ASIN: return dy / sqrtf(1.f - x * x);
    case U_ATAN: return dy / (1.f + x * x);
    case U_COSH: return dy * sinhf(x);
    case U_SINH: return dy * coshf(x);
    case U_TANH: { const float c = coshf(x); return dy / (c * c); }
    case U_ACOSH: return dy / (sqrtf(x - 1.f) * sqrtf(x + 1.f));
    case U_ASINH: return dy / sqrtf(x * x + 1.f);
    case U_ATANH: return dy / (1.f - x * x);
    case U_ERF: return dy * 1.1283791670955126f * expf(-x * x);
    case U_ERFINV: { const float y = erfinvf(x); return dy * 0.8862269254527580f * expf(y * y); }
    case U_GELU: {
      const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
      const float pdf = 0.3989422804014327f * expf(-0.5f * x * x);
      return dy * (cdf + x * pdf);
    }
    case U_GELU_TANH: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float t = tanhf(u);
      const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
      return dy * (0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du);
    }
    case U_LOG_SIGMOID: return dy / (1.f + expf(x));
    case U_SELU: {
      const float a = 1.6732632423543772f, s = 1.0507009873554805f;
      return x > 0.f ? dy * s : dy * s * a * expf(x);
    }
    case U_SIGMOID: { const float s = 1.f / (1.f + expf(-x)); return dy * s * (1.f - s); }
    case U_SOFTPLUS: return dy / (1.f + expf(-x));
    case U_SOFTSIGN: { const float d = 1.f + fabsf(x); return dy / (d * d); }
    case U_RELU: return x > 0.f ? dy : 0.f;
    case U_LEAKY_RELU: return x > 0.f ? dy : p0 * dy;
    case U_ELU: return x > 0.f ? dy : dy * p0 * expf(x);
    case U_ADD_CONST: return dy;
    case U_SCALE: return dy * p0;
    case U_SUB_CONST: return dy;
    case U_CONST_SUB: return -dy;
    case U_MAX_CONST: return x > p0 ? dy : 0.f;
    case U_MIN_CONST: return x < p0 ? dy : 0.f;
    case U_CLAMP: return (x > p0 && x < p1) ? dy : 0.f;
    default: return 0.f;  // piecewise-constant ops
  }
}

__device__ __forceinline__ float binary_fwd(int op, float a, float b) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return a / b;
    case B_MOD: return fmodf(a, b);
    case B_POW: return powf(a, b);
    case B_SAFE_DIV: { const float y = a / b; return isfinite(y) ? y : 0.f; }
    case B_SQ_DIFF: return (a - b) * (a - b);
    case B_MAX: return fmaxf(a, b);
    case B_MIN: return fminf(a, b);
    case B_EQ: return a == b ? 1.f : 0.f;
    case B_NE: return a != b ? 1.f : 0.f;
    case B_LT: return a < b ? 1.f : 0.f;
    case B_LE: return a <= b ? 1.f : 0.f;
    case B_GT: return a > b ? 1.f : 0.f;
    case B_GE: return a >= b ? 1.f : 0.f;
    case B_AND: return (a != 0.f && b != 0.f) ? 1.f : 0.f;
    case B_OR: return (a != 0.f || b != 0.f) ? 1.f : 0.f;
    case B_XOR: return ((a != 0.f) != (b != 0.f)) ? 1.f : 0.f;
    case B_BCE: {  // a = prediction in (0,1), b = target
      float y = 0.f;
      if (b > 0.f) y += -b * logf(a);
      if (b < 1.f) y += -(1.f - b) * logf(1.f - a);
      return y;
    }
    case B_SIGMOID_BCE: {  // a = logit, b = target
      const float z = fmaxf(0.f, fminf(b, 1.f));
      return a > 0.f ? (1.f - z) * a + log1pf(expf(-a)) : -a * z + log1pf(expf(a));
    }
    case B_BOOL_ACC: return ((a >= 0.5f) == (b >= 0.5f)) ? 1.f : 0.f;
    case B_BOOL_FN: return (!(a >= 0.5f) && (b >= 0.5f)) ? 1.f : 0.f;
    case B_BOOL_FP: return ((a >= 0.5f) && !(b >= 0.5f)) ? 1.f : 0.f;
    case B_ADD_RELU: return fmaxf(a + b, 0.f);      // residual addition + ReLU in one pass
    default: return 0.f;
  }
}

__device__ __forceinline__ void binary_bwd(int op, float a, float b, float dy, float& da,
                                           float& db) {
  da = 0.f; db = 0.f;
  switch (op) {
    case B_ADD: da = dy; db = dy; break;
    case B_ADD_RELU: da = (a + b) > 0.f ? dy : 0.f; db = da; break;
    case B_SUB: da = dy; db = -dy; break;
    case B_MUL: da = dy * b; db = dy * a; break;
    case B_DIV: da = dy / b; db = -dy * a / (b * b); break;
    case B_MOD: da = dy; db = -dy * truncf(a / b); break;
    case B_POW: da = dy * b * powf(a, b - 1.f); db = dy * logf(a) * powf(a, b); break;
    case B_SAFE_DIV: {
      const float y = a / b;
      if (isfinite(y)) { da = dy / b; db = -dy * a / (b * b); }
      break;
    }
    case B_SQ_DIFF: da = 2.f * (a - b) * dy; db = -da; break;
    case B_MAX:
      if (a > b) da = dy; else if (b > a) db = dy; else { da = 0.5f * dy; db = 0.5f * dy; }
      break;
    case B_MIN:
      if (a < b) da = dy; else if (b < a) db = dy; else { da = 0.5f * dy; db = 0.5f * dy; }
      break;
    case B_BCE:
      if (b > 0.f) { da += -b / a * dy; db += -logf(a) * dy; }
      if (b < 1.f) { da += (1.f - b) / (1.f - a) * dy; db += logf(1.f - a) * dy; }
      break;
    case B_SIGMOID_BCE: {
      const float z = fmaxf(0.f, fminf(b, 1.f));
      if (a > 0.f) { da = (1.f - z - 1.f / (1.f + expf(a))) * dy; db = -a * dy; }
      else         { da = (-z + 1.f / (1.f + expf(-a))) * dy; db = -a * dy; }
      break;
    }
    default: break;
  }
}

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); T v[16 / sizeof(T)]; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, long long i, long long n, float (&f)[8],
                                         bool aligned) {
  constexpr int V = 16 / sizeof(T);
  if (aligned && i + V <= n) {
    uint4 q = *reinterpret_cast<const uint4*>(p + i);
    const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int j = 0; j < V; ++j) f[j] = to_f32<T>(e[j]);
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) f[j] = (i + j < n) ? to_f32<T>(p[i + j]) : 0.f;
  }
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, long long i, long long n, const float (&f)[8],
                                          bool aligned) {
  constexpr int V = 16 / sizeof(T);
  if (aligned && i + V <= n) {
    uint4 q;
    T* e = reinterpret_cast<T*>(&q);
#pragma unroll
    for (int j = 0; j < V; ++j) e[j] = from_f32<T>(f[j]);
    *reinterpret_cast<uint4*>(p + i) = q;
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j)
      if (i + j < n) p[i + j] = from_f32<T>(f[j]);
  }
}

// The operator is chosen ONCE per thread, outside the element loops: with the switch of
// unary_fwd inside an eight-way unrolled loop every element walked a jump table and eight
// copies of all ~60 operators' code (GELU on 134 M bf16 values ran at 1.5 TB/s instead of the
// copy rate).  Dispatch is a compile-time binary search over the operator codes; each leaf is
// the grid-stride loop with the operator as a constant.
template <typename T, int OP>
__device__ __forceinline__ void unary_body(const T* __restrict__ x, const T* __restrict__ dy,
                                           T* __restrict__ out, long long n, int mode, float p0,
                                           float p1, int aligned) {
  constexpr int V = 16 / sizeof(T);
  const long long stride = (long long)gridDim.x * blockDim.x * V;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    float fx[8], fd[8], fo[8];
    load_vec<T>(x, i, n, fx, aligned);
    if (mode == 0) {
#pragma unroll
      for (int j = 0; j < V; ++j) fo[j] = unary_fwd(OP, fx[j], p0, p1);
    } else {
      load_vec<T>(dy, i, n, fd, aligned);
#pragma unroll
      for (int j = 0; j < V; ++j) fo[j] = unary_bwd(OP, fx[j], fd[j], p0, p1);
    }
    store_vec<T>(out, i, n, fo, aligned);
  }
}
template <typename T, int LO, int HI>
struct UnaryDispatch {
  __device__ __forceinline__ static void run(int op, const T* x, const T* dy, T* out, long long n,
                                             int mode, float p0, float p1, int aligned) {
    if constexpr (LO == HI) {
      unary_body<T, LO>(x, dy, out, n, mode, p0, p1, aligned);
    } else {
      constexpr int MID = (LO + HI) / 2;
      if (op <= MID) UnaryDispatch<T, LO, MID>::run(op, x, dy, out, n, mode, p0, p1, aligned);
      else UnaryDispatch<T, MID + 1, HI>::run(op, x, dy, out, n, mode, p0, p1, aligned);
    }
  }
};

// mode 0: y = f(x); mode 1: dx = f'(x) dy
template <typename T>
__global__ void unary_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out,
                             long long n, int op, int mode, float p0, float p1, int aligned) {
  UnaryDispatch<T, 0, U_COUNT - 1>::run(op, x, dy, out, n, mode, p0, p1, aligned);
}

template <typename T, int OP>
__device__ __forceinline__ void binary_body(const T* __restrict__ a, const T* __restrict__ b,
                                            const T* __restrict__ dy, T* __restrict__ out0,
                                            T* __restrict__ out1, long long n, int mode, int aligned) {
  constexpr int V = 16 / sizeof(T);
  const long long stride = (long long)gridDim.x * blockDim.x * V;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    float fa[8], fb[8], fd[8], o0[8], o1[8];
    load_vec<T>(a, i, n, fa, aligned);
    load_vec<T>(b, i, n, fb, aligned);
    if (mode == 0) {
#pragma unroll
      for (int j = 0; j < V; ++j) o0[j] = binary_fwd(OP, fa[j], fb[j]);
    } else {
      load_vec<T>(dy, i, n, fd, aligned);
#pragma unroll
      for (int j = 0; j < V; ++j) binary_bwd(OP, fa[j], fb[j], fd[j], o0[j], o1[j]);
    }
    store_vec<T>(out0, i, n, o0, aligned);
    if (mode == 1 && out1) store_vec<T>(out1, i, n, o1, aligned);
  }
}
template <typename T, int LO, int HI>
struct BinaryDispatch {
  __device__ __forceinline__ static void run(int op, const T* a, const T* b, const T* dy, T* out0,
                                             T* out1, long long n, int mode, int aligned) {
    if constexpr (LO == HI) {
      binary_body<T, LO>(a, b, dy, out0, out1, n, mode, aligned);
    } else {
      constexpr int MID = (LO + HI) / 2;
      if (op <= MID) BinaryDispatch<T, LO, MID>::run(op, a, b, dy, out0, out1, n, mode, aligned);
      else BinaryDispatch<T, MID + 1, HI>::run(op, a, b, dy, out0, out1, n, mode, aligned);
    }
  }
};

// mode 0: y = f(a, b); mode 1: (da, db) = grad.
template <typename T>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b,
                              const T* __restrict__ dy, T* __restrict__ out0, T* __restrict__ out1,
                              long long n, int op, int mode, int aligned) {
  BinaryDispatch<T, 0, B_COUNT - 1>::run(op, a, b, dy, out0, out1, n, mode, aligned);
}

// out = sum_k scale[k] * in[k]  (the Sum / WeightedSum layers and residual adds)
template <typename T>
__global__ void weighted_sum_kernel(const T* const* __restrict__ ins, const float* __restrict__ scales,
                                    int k, T* __restrict__ out, long long n, int aligned) {
  constexpr int V = 16 / sizeof(T);
  const long long stride = (long long)gridDim.x * blockDim.x * V;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int t = 0; t < k; ++t) {
      float f[8];
      load_vec<T>(ins[t], i, n, f, aligned);
      const float s = scales[t];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += s * f[j];
    }
    store_vec<T>(out, i, n, acc, aligned);
  }
}

static int grid_for(long long n, int vec) {
  const long long blocks = (n + 256LL * vec - 1) / (256LL * vec);
  const long long cap = (long long)lbhost::sm_count() * 8;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

static int all_aligned(std::initializer_list<const void*> ps) {
  for (const void* p : ps)
    if (p && (reinterpret_cast<uintptr_t>(p) & 15)) return 0;
  return 1;
}

}  // namespace lb

extern "C" {

int lb_unary(const void* x, const void* dy, void* out, long long n, int op, int mode, float p0,
             float p1, int dtype, void* stream_) {
  using namespace lb;
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int al = all_aligned({x, dy, out});
  if (dtype == kF32)
    unary_kernel<float><<<grid_for(n, 4), 256, 0, s>>>((const float*)x, (const float*)dy,
                                                       (float*)out, n, op, mode, p0, p1, al);
  else if (dtype == kBF16)
    unary_kernel<__nv_bfloat16><<<grid_for(n, 8), 256, 0, s>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)out, n, op, mode, p0, p1, al);
  else
    unary_kernel<__half><<<grid_for(n, 8), 256, 0, s>>>((const __half*)x, (const __half*)dy,
                                                        (__half*)out, n, op, mode, p0, p1, al);
  return (int)cudaGetLastError();
}

int lb_binary(const void* a, const void* b, const void* dy, void* out0, void* out1, long long n,
              int op, int mode, int dtype, void* stream_) {
  using namespace lb;
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int al = all_aligned({a, b, dy, out0, out1});
  if (dtype == kF32)
    binary_kernel<float><<<grid_for(n, 4), 256, 0, s>>>((const float*)a, (const float*)b,
                                                        (const float*)dy, (float*)out0,
                                                        (float*)out1, n, op, mode, al);
  else if (dtype == kBF16)
    binary_kernel<__nv_bfloat16><<<grid_for(n, 8), 256, 0, s>>>(
        (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (const __nv_bfloat16*)dy,
        (__nv_bfloat16*)out0, (__nv_bfloat16*)out1, n, op, mode, al);
  else
    binary_kernel<__half><<<grid_for(n, 8), 256, 0, s>>>((const __half*)a, (const __half*)b,
                                                         (const __half*)dy, (__half*)out0,
                                                         (__half*)out1, n, op, mode, al);
  return (int)cudaGetLastError();
}

// ins: device array of k pointers, scales: device array of k floats.
int lb_weighted_sum(const void* const* ins, const float* scales, int k, void* out, long long n,
                    int dtype, int aligned, void* stream_) {
  using namespace lb;
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == kF32)
    weighted_sum_kernel<float><<<grid_for(n, 4), 256, 0, s>>>((const float* const*)ins, scales, k,
                                                              (float*)out, n, aligned);
  else if (dtype == kBF16)
    weighted_sum_kernel<__nv_bfloat16><<<grid_for(n, 8), 256, 0, s>>>(
        (const __nv_bfloat16* const*)ins, scales, k, (__nv_bfloat16*)out, n, aligned);
  else
    weighted_sum_kernel<__half><<<grid_for(n, 8), 256, 0, s>>>((const __half* const*)ins, scales,
                                                               k, (__half*)out, n, aligned);
  return (int)cudaGetLastError();
}

}  // extern "C"
