// Convolution filters for the implicit-GEMM kernels, repacked from the fp32 master copy in
// ONE launch per layer and optimizer step:
//   fwd  [tap][Kp][Cp]            = w[k][c][tap]                 (forward operand)
//   dgrad[tap][Cp][Kp]            = w[k][c][taps - 1 - tap]      (data-gradient operand: taps
//                                                                 reversed, channel roles swapped)
// Kp / Cp are the channel counts padded to the kernels' granularity; padding is zero.  The
// reference keeps filters in the vendor library's layout and has no such step.
#include "common.cuh"

namespace lb {

template <typename T>
__global__ void __launch_bounds__(256)
pack_filter_kernel(const float* __restrict__ w, T* __restrict__ fwd, T* __restrict__ dgrad, int K,
                   int C, int taps, int Kp, int Cp) {
  const long long total = (long long)taps * Kp * Cp;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cp);
    const int k = (int)((i / Cp) % Kp);
    const int t = (int)(i / ((long long)Cp * Kp));
    const float v = (k < K && c < C) ? w[((long long)k * C + c) * taps + t] : 0.f;
    const T o = from_f32<T>(v);
    if (fwd) fwd[i] = o;
    if (dgrad) dgrad[((long long)(taps - 1 - t) * Cp + c) * Kp + k] = o;
  }
}

}  // namespace lb

extern "C" int lb_pack_filter(const float* w, void* fwd, void* dgrad, int K, int C, int taps, int Kp,
                              int Cp, int dtype, void* stream_) {
  using namespace lb;
  if (K < 1 || C < 1 || taps < 1 || Kp < K || Cp < C) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long total = (long long)taps * Kp * Cp;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (dtype == kF16)
    pack_filter_kernel<__half><<<(int)blocks, 256, 0, s>>>(w, (__half*)fwd, (__half*)dgrad, K, C, taps, Kp, Cp);
  else if (dtype == kBF16)
    pack_filter_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, s>>>(w, (__nv_bfloat16*)fwd, (__nv_bfloat16*)dgrad, K, C, taps, Kp, Cp);
  else if (dtype == kF32)
    pack_filter_kernel<float><<<(int)blocks, 256, 0, s>>>(w, (float*)fwd, (float*)dgrad, K, C, taps, Kp, Cp);
  else
    return -1;
  return (int)cudaGetLastError();
}
