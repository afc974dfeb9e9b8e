// TEST INFRASTRUCTURE ONLY.  C-ABI launch shim around the reference's fp64 2-D device kernels
// (deform2d_double/lib/deform_conv2d_cuda_kernel.cu, compiled in place and linked with this
// file); launchers declared in deform2d_double/lib/deform_conv2d_cuda_kernel.h:11-44.
#include <cuda_runtime.h>
#include "deform_conv2d_cuda_kernel.h"

extern "C" {
int ref2dd_im2col(const double* x_n, const double* off_n, int C, const int* in, const int* out, const int* k,
                  const int* pad, const int* stride, const int* dil, int cpg, double* col) {
    deformable_im2col(0, x_n, off_n, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1], stride[0],
                      stride[1], dil[0], dil[1], cpg, col);
    return (int)cudaGetLastError();
}
int ref2dd_col2im_input(const double* col, const double* off_n, int C, const int* in, const int* out,
                        const int* k, const int* pad, const int* stride, const int* dil, int cpg, double* dx_n) {
    deformable_col2im_input(0, col, off_n, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1],
                            stride[0], stride[1], dil[0], dil[1], cpg, dx_n);
    return (int)cudaGetLastError();
}
int ref2dd_col2im_offset(const double* col, const double* x_n, const double* off_n, int C, const int* in,
                         const int* out, const int* k, const int* pad, const int* stride, const int* dil,
                         int cpg, double* doff_n) {
    deformable_col2im_offset(0, col, x_n, off_n, C, in[0], in[1], out[0], out[1], k[0], k[1], pad[0], pad[1],
                             stride[0], stride[1], dil[0], dil[1], cpg, doff_n);
    return (int)cudaGetLastError();
}
}
