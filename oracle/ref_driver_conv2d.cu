// TEST INFRASTRUCTURE ONLY.  C-ABI launch shim around the reference's plain 2-D im2col / col2im
// device kernels (conv2d/lib/conv2d_cuda_kernel.cu, compiled in place and linked with this
// file); launchers declared in conv2d/lib/conv2d_cuda_kernel.h:11-32.
#include <cuda_runtime.h>
#include "conv2d_cuda_kernel.h"

extern "C" {
int refc2d_im2col(const float* x_n, int C, const int* in, const int* out, const int* k, const int* pad,
                  const int* stride, const int* dil, float* col) {
    im2col(0, x_n, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1], stride[0], stride[1], dil[0],
           dil[1], col);
    return (int)cudaGetLastError();
}
int refc2d_col2im(const float* col, int C, const int* in, const int* out, const int* k, const int* pad,
                  const int* stride, const int* dil, float* dx_n) {
    col2im(0, col, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1], stride[0], stride[1], dil[0],
           dil[1], dx_n);
    return (int)cudaGetLastError();
}
}
