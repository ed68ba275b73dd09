// Weight gradient of a fully-connected layer for SHORT mini-batches:
//   out[m][n] = beta * out[m][n] + alpha * sum_k a[k][m] * b[k][n],   k < K <= 32
// a = dy [K, M], b = x [K, N] (16-bit, row-major), out fp32 [M, N].
//
// With K of 8 (one sample per row) the product has 16 FLOPs per 4-byte output element, so the
// operation is bound by the fp32 read-modify-write of `out`; a tensor-core tile pipeline only
// adds latency.  Every thread keeps its four columns of b for all K rows in registers, walks
// over a strip of rows m and updates one float4 of `out` per row; a[.][m] comes from shared
// memory as a broadcast.  The reference computes this product as a distributed GEMM
// (src/layers/learning/fully_connected.cpp:638-808).
#include "common.cuh"

namespace lb {

constexpr int kOuterMaxK = 32;
constexpr int kOuterRows = 32;      // rows of `out` per block (power of two)

template <typename T, int K>
__global__ void __launch_bounds__(256)
outer_accum_kernel(const T* __restrict__ a, const T* __restrict__ b, float* __restrict__ out,
                   int M, long long N, float alpha, float beta) {
  __shared__ float sa[K][kOuterRows];
  const int m0 = blockIdx.y * kOuterRows;
  for (int i = threadIdx.x; i < K * kOuterRows; i += blockDim.x) {
    const int k = i / kOuterRows, m = i - k * kOuterRows;
    sa[k][m] = m0 + m < M ? alpha * to_f32<T>(a[(long long)k * M + m0 + m]) : 0.f;
  }
  __syncthreads();
  const long long n = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (n >= N) return;
  float bv[K][4];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const uint2 raw = *reinterpret_cast<const uint2*>(b + (long long)k * N + n);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) bv[k][j] = to_f32<T>(e[j]);
  }
  const int rows = M - m0 < kOuterRows ? M - m0 : kOuterRows;
  // eight rows at a time: their read-modify-write loads are all issued before the first is
  // used, which is what keeps enough bytes in flight for a memory-bound kernel
  constexpr int G = 8;
  for (int mb = 0; mb < rows; mb += G) {
    float4 acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (beta != 0.f && mb + g < rows)
        acc[g] = *reinterpret_cast<const float4*>(out + (long long)(m0 + mb + g) * N + n);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      acc[g].x *= beta; acc[g].y *= beta; acc[g].z *= beta; acc[g].w *= beta;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const float av = sa[k][(mb + g) & (kOuterRows - 1)];
        acc[g].x = fmaf(av, bv[k][0], acc[g].x);
        acc[g].y = fmaf(av, bv[k][1], acc[g].y);
        acc[g].z = fmaf(av, bv[k][2], acc[g].z);
        acc[g].w = fmaf(av, bv[k][3], acc[g].w);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
      if (mb + g < rows)
        *reinterpret_cast<float4*>(out + (long long)(m0 + mb + g) * N + n) = acc[g];
  }
}

template <typename T>
static int launch_outer(const void* a, const void* b, float* out, int K, int M, long long N,
                        float alpha, float beta, cudaStream_t s) {
  dim3 grid((unsigned)((N / 4 + 255) / 256), (unsigned)((M + kOuterRows - 1) / kOuterRows));
  // only exact row counts are instantiated: a larger K would read rows that do not exist
  switch (K) {
    case 1: outer_accum_kernel<T, 1><<<grid, 256, 0, s>>>((const T*)a, (const T*)b, out, M, N, alpha, beta); break;
    case 2: outer_accum_kernel<T, 2><<<grid, 256, 0, s>>>((const T*)a, (const T*)b, out, M, N, alpha, beta); break;
    case 4: outer_accum_kernel<T, 4><<<grid, 256, 0, s>>>((const T*)a, (const T*)b, out, M, N, alpha, beta); break;
    case 8: outer_accum_kernel<T, 8><<<grid, 256, 0, s>>>((const T*)a, (const T*)b, out, M, N, alpha, beta); break;
    case 16: outer_accum_kernel<T, 16><<<grid, 256, 0, s>>>((const T*)a, (const T*)b, out, M, N, alpha, beta); break;
    default: return -2;
  }
  return (int)cudaGetLastError();
}

}  // namespace lb

extern "C" {

// Returns -2 when the shape is not covered (K not in {1, 2, 4, 8, 16}, N not a multiple of 4,
// misaligned pointers): the caller then uses the tensor-core GEMM.
int lb_outer_accum(const void* a, const void* b, float* out, int K, int M, long long N,
                   float alpha, float beta, int dtype, void* stream_) {
  using namespace lb;
  if (K < 1 || K > kOuterMaxK || M < 1 || N < 4 || (N & 3)) return -2;
  if ((reinterpret_cast<uintptr_t>(b) & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == kF16) return launch_outer<__half>(a, b, out, K, M, N, alpha, beta, s);
  if (dtype == kBF16) return launch_outer<__nv_bfloat16>(a, b, out, K, M, N, alpha, beta, s);
  return -2;
}

}  // extern "C"
