// Geometry record shared by the convolution kernels (21 ints, filled by the host caller).
#pragma once

namespace lb {

struct ConvGeom {
  int N, D, H, W, C;
  int Do, Ho, Wo, Kout;
  int kd, kh, kw;
  int pd, ph, pw;
  int sd, sh, sw;
  int dd, dh, dw;
};

}  // namespace lb

// Halo-slab variant of the forward convolution (conv_slab_tc.cu): same arguments as
// lb_conv_fwd_tc; returns -2 when the shape is not one it handles.
extern "C" int lb_conv_slab_fwd(const void* x, const void* w, void* y, const float* bias,
                                const int* geom, const long long* xs, const long long* ys,
                                int in_dtype, int out_dtype, float alpha, float beta, int act,
                                float act_param, const void* halo, void* stream_);
