// TEST INFRASTRUCTURE ONLY.  C-ABI launch shim around the reference's fp32 2-D device kernels
// (deform2d/lib/deform_conv2d_cuda_kernel.cu, compiled in place and linked with this file);
// launchers declared in deform2d/lib/deform_conv2d_cuda_kernel.h:11-41 (no dilation argument).
#include <cuda_runtime.h>
#include "deform_conv2d_cuda_kernel.h"

extern "C" {
int ref2d_im2col(const float* x_n, const float* off_n, int C, const int* in, const int* out, const int* k,
                 const int* pad, const int* stride, int cpg, float* col) {
    deformable_im2col(0, x_n, off_n, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1], stride[0],
                      stride[1], cpg, col);
    return (int)cudaGetLastError();
}
int ref2d_col2im_input(const float* col, const float* off_n, int C, const int* in, const int* out, const int* k,
                       const int* pad, const int* stride, int cpg, float* dx_n) {
    deformable_col2im_input(0, col, off_n, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1],
                            stride[0], stride[1], cpg, dx_n);
    return (int)cudaGetLastError();
}
int ref2d_col2im_offset(const float* col, const float* x_n, const float* off_n, int C, const int* in,
                        const int* out, const int* k, const int* pad, const int* stride, int cpg,
                        float* doff_n) {
    deformable_col2im_offset(0, col, x_n, off_n, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1],
                             stride[0], stride[1], cpg, doff_n);
    return (int)cudaGetLastError();
}
}
