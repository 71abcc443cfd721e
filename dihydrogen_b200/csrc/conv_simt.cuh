// Interfaces between the convolution front end (conv.cu) and its kernel
// families.
#pragma once

#include "common.cuh"

namespace dcb
{

// Everything a convolution kernel needs to know about one problem.  Spatial
// arrays are ordered D, H, W; a 2-D problem has extent 1, filter 1, pad 0,
// stride 1 in slot 0.
struct ConvGeom
{
    int n, c, k;
    int in[3], out[3];
    int f[3], pad[3], stride[3], dil[3];
    long long xs_n, xs_c, xs[3]; // element strides of the input window
    long long ys_n, ys_c, ys[3]; // element strides of the output window
};

// fp32 CUDA-core kernels -------------------------------------------------
int32_t simt_conv_fwd(const ConvGeom& g, float alpha, const float* x,
                      const float* w, float beta, float* y,
                      cudaStream_t stream);
// Gather form of the adjoint w.r.t. the input; any stride / dilation.
int32_t simt_conv_bwd_data(const ConvGeom& g, float alpha, const float* w,
                           const float* dy, float beta, float* dx,
                           cudaStream_t stream);
size_t simt_conv_bwd_filter_workspace(const ConvGeom& g);
int32_t simt_conv_bwd_filter(const ConvGeom& g, float alpha, const float* x,
                             const float* dy, float beta, float* dw,
                             float* workspace, cudaStream_t stream);
// w2[c][k][flipped taps] = w[k][c][taps]: turns a stride-1 backward-data into
// a forward correlation of dy.
int32_t flip_transpose_filter(const float* w, float* w2, int k, int c,
                              int taps, cudaStream_t stream);

} // namespace dcb
