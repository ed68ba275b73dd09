// Planar to pixel-interleaved layout for the first layer: [N][C][S] (S = D*H*W spatial
// positions, C <= CR channels) -> [N][S][CR] with the missing channels zero.  The
// first-layer kernels (conv_c8_tc.cu) read 8- or 16-byte pixels; samples arrive planar
// from the data readers.  A thread takes 8 consecutive positions: one 16-byte load per
// channel, 8 * CR * 2 contiguous bytes out.
#include "common.cuh"

namespace lb {

template <int CR>
__global__ void __launch_bounds__(256)
planar_to_pixels_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, int C,
                        long long S, long long xs_n, long long total8) {
  const long long s8 = S / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8;
       i += (long long)gridDim.x * blockDim.x) {
    const long long n = i / s8, s = (i - n * s8) * 8;
    uint4 v[CR];
#pragma unroll
    for (int c = 0; c < CR; ++c) {
      v[c] = make_uint4(0u, 0u, 0u, 0u);
      if (c < C) v[c] = __ldg(reinterpret_cast<const uint4*>(x + n * xs_n + c * S + s));
    }
    uint4* dst = reinterpret_cast<uint4*>(y + (n * S + s) * CR);
    // position j of channel c sits in half j of v[c]; output pixel j = (v[0][j], v[1][j], ...)
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      uint32_t lo[CR], hi[CR];                 // the two pixels j, j + 1, one half per channel
#pragma unroll
      for (int c = 0; c < CR; ++c) {
        const uint32_t w = j == 0 ? v[c].x : j == 2 ? v[c].y : j == 4 ? v[c].z : v[c].w;
        lo[c] = w & 0xffffu;
        hi[c] = w >> 16;
      }
      if (CR == 4) {
        dst[j / 2] = make_uint4(lo[0] | (lo[1] << 16), lo[2] | (lo[3] << 16), hi[0] | (hi[1] << 16),
                                hi[2] | (hi[3] << 16));
      } else {
        dst[j] = make_uint4(lo[0] | (lo[1] << 16), lo[2] | (lo[3] << 16), lo[4] | (lo[5] << 16),
                            lo[6] | (lo[7] << 16));
        dst[j + 1] = make_uint4(hi[0] | (hi[1] << 16), hi[2] | (hi[3] << 16), hi[4] | (hi[5] << 16),
                                hi[6] | (hi[7] << 16));
      }
    }
  }
}

}  // namespace lb

// x: N samples of C planes of S 16-bit values, sample stride xs_n elements, planes dense;
// y: [N][S][cr] dense, cr = 4 or 8 >= C.  S a multiple of 8, both 16-byte aligned.
extern "C" int lb_planar_to_pixels(const void* x, void* y, int N, int C, long long S, long long xs_n,
                                   int cr, void* stream_) {
  using namespace lb;
  if ((cr != 4 && cr != 8) || C > cr || C < 1 || S % 8 || xs_n % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15)) return -1;
  const long long total8 = (long long)N * (S / 8);
  if (total8 <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long blocks = (total8 + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 16;
  const int grid = (int)(blocks < cap ? blocks : cap);
  if (cr == 4)
    planar_to_pixels_kernel<4><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint16_t*)y, C, S, xs_n, total8);
  else
    planar_to_pixels_kernel<8><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint16_t*)y, C, S, xs_n, total8);
  return (int)cudaGetLastError();
}
