// Allocation-free per-column reduction (see no_alloc.h for the contract).
#include "no_alloc.h"

#include <cstdio>

#include "common.cuh"

namespace lb {

// The workspace: [2][kMaxCols] fp32 partial sums, cleared at the start of every call.
constexpr int kNoAllocMaxCols = LB_COLUMN_SUMS_NOALLOC_MAX_COLS;
static __device__ __align__(256) float g_colsum_scratch[2 * kNoAllocMaxCols];

constexpr int kNoAllocMaxDevices = 64;
static float* g_scratch_ptr[kNoAllocMaxDevices] = {nullptr};

// One thread per 8-column vector; blockDim.y threads walk the rows of the block's chunk,
// are combined through shared memory, and row 0 adds the block's partial sums to the
// workspace with fp32 atomics.
template <typename T>
__global__ void colsum_scratch_kernel(const T* __restrict__ x, float* __restrict__ scratch,
                                      long long rows, int C, long long rows_per_block) {
  __shared__ float sm[8][32][17];       // [row lane][vector][8 sums + 8 squares (+1 pad)]
  const int cv = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = v < cv;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  float s[8], ss[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.f; ss[j] = 0.f; }
  if (valid) {
    for (long long r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
      const uint4 q = *reinterpret_cast<const uint4*>(x + r * C + v * 8);
      const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = to_f32<T>(e[j]);
        s[j] += f;
        ss[j] += f * f;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sm[threadIdx.y][threadIdx.x][j] = s[j];
    sm[threadIdx.y][threadIdx.x][8 + j] = ss[j];
  }
  __syncthreads();
  if (threadIdx.y == 0 && valid) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float acc = 0.f;
      for (int y = 0; y < (int)blockDim.y; ++y) acc += sm[y][threadIdx.x][j];
      const int col = v * 8 + (j & 7);
      atomicAdd(scratch + (j < 8 ? 0 : kNoAllocMaxCols) + col, acc);
    }
  }
}

__global__ void colsum_copy_out_kernel(const float* __restrict__ scratch, float* __restrict__ out,
                                       int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < C) {
    out[c] = scratch[c];
    out[C + c] = scratch[kNoAllocMaxCols + c];
  }
}

}  // namespace lb

extern "C" int lb_column_sums_noalloc(const void* x, float* out, long long rows, int cols,
                                      int dtype, void* stream_) {
  using namespace lb;
  if (!x || !out || rows < 0 || cols <= 0 || (cols % 8) || (dtype != kF16 && dtype != kBF16))
    return -1;
  if (reinterpret_cast<uintptr_t>(x) & 15) return -1;
  if (cols > kNoAllocMaxCols) {
    fprintf(stderr,
            "lb_column_sums_noalloc: %d columns exceed the built-in workspace of %d columns\n",
            cols, kNoAllocMaxCols);
    return -2;
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return (int)err;
  if (dev < 0 || dev >= kNoAllocMaxDevices) return -1;
  if (g_scratch_ptr[dev] == nullptr) {
    // first call on this device: look the workspace up (once; keep it out of stream capture)
    float* ptr = nullptr;
    err = cudaGetSymbolAddress((void**)&ptr, g_colsum_scratch);
    if (err != cudaSuccess) return (int)err;
    g_scratch_ptr[dev] = ptr;
  }
  float* scratch = g_scratch_ptr[dev];
  // the sums accumulate with atomics: the part of the workspace in use must start at zero
  err = cudaMemsetAsync(scratch, 0, sizeof(float) * cols, stream);
  if (err != cudaSuccess) return (int)err;
  err = cudaMemsetAsync(scratch + kNoAllocMaxCols, 0, sizeof(float) * cols, stream);
  if (err != cudaSuccess) return (int)err;
  if (rows > 0) {
    const int cv = cols / 8;
    dim3 block(32, 8);
    const int gx = (cv + 31) / 32;
    long long want = (4LL * lbhost::sm_count() + gx - 1) / gx;
    long long by = (rows + 63) / 64;          // at least 64 rows per block
    if (by > want) by = want;
    if (by < 1) by = 1;
    const long long rpb = (rows + by - 1) / by;
    dim3 grid(gx, (unsigned)by);
    if (dtype == kF16)
      colsum_scratch_kernel<__half><<<grid, block, 0, stream>>>((const __half*)x, scratch, rows,
                                                                cols, rpb);
    else
      colsum_scratch_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)x,
                                                                       scratch, rows, cols, rpb);
    err = cudaGetLastError();
    if (err != cudaSuccess) return (int)err;
  }
  colsum_copy_out_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(scratch, out, cols);
  return (int)cudaGetLastError();
}
