// TEST INFRASTRUCTURE ONLY.  C-ABI launch shim around the reference's own 3-D device kernels
// (deform3d/lib/deform_conv3d_cuda_kernel.cu, compiled in place from the reference checkout and
// linked with this file).  It forwards raw device pointers to the reference's host launchers
// declared in deform3d/lib/deform_conv3d_cuda_kernel.h:11-47, one sample per call like
// deform3d/lib/deform_conv3d_cuda.cpp:105-118, 231-251, 283-292.
#include <cuda_runtime.h>
#include "deform_conv3d_cuda_kernel.h"

extern "C" {
int ref3d_im2col(const float* x_n, const float* off_n, int C, const int* in, const int* out, const int* k,
                 const int* pad, const int* stride, const int* dil, int cpg, float* col) {
    deformable_im2col<float>(0, x_n, off_n, C, in[0], in[1], in[2], out[0], out[1], out[2], k[0], k[1], k[2],
                             pad[0], pad[1], pad[2], stride[0], stride[1], stride[2], dil[0], dil[1], dil[2],
                             cpg, col);
    return (int)cudaGetLastError();
}
int ref3d_col2im_input(const float* col, const float* off_n, int C, const int* in, const int* out, const int* k,
                       const int* pad, const int* stride, const int* dil, int cpg, float* dx_n) {
    deformable_col2im_input<float>(0, col, off_n, C, in[0], in[1], in[2], out[0], out[1], out[2], k[0], k[1],
                                   k[2], pad[0], pad[1], pad[2], stride[0], stride[1], stride[2], dil[0], dil[1],
                                   dil[2], cpg, dx_n);
    return (int)cudaGetLastError();
}
int ref3d_col2im_offset(const float* col, const float* x_n, const float* off_n, int C, const int* in,
                        const int* out, const int* k, const int* pad, const int* stride, const int* dil, int cpg,
                        float* doff_n) {
    deformable_col2im_offset<float>(0, col, x_n, off_n, C, in[0], in[1], in[2], out[0], out[1], out[2], k[0],
                                    k[1], k[2], pad[0], pad[1], pad[2], stride[0], stride[1], stride[2], dil[0],
                                    dil[1], dil[2], cpg, doff_n);
    return (int)cudaGetLastError();
}
}
