// Internal interfaces between the C-ABI layer (dcn_api.cu) and the kernel files of libdcn.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "dcn_common.cuh"

namespace dcn {

// EXACT-precision (SIMT) launchers, dcn_simt.cu.  dtype: 0 fp32, 1 fp64.  Return 0 or -5 (launch failure).
int simt_forward(const Geom& g, int dtype, int ndim, int deform, const void* x, const void* off, const void* w,
                 const void* bias, void* y, cudaStream_t st);
int simt_backward_data(const Geom& g, int dtype, int ndim, int deform, const void* x, const void* off,
                       const void* w, const void* dy, void* dx, void* doff, cudaStream_t st);
int simt_backward_weight(const Geom& g, int dtype, int ndim, int deform, const void* x, const void* off,
                         const void* dy, void* dw, cudaStream_t st);
// latency-shaped kernels for very small fp32 deformable problems (dcn_simt_small.cuh)
bool simt_small_supported(const Geom& g, int dtype, int ndim, int deform);
int simt_small_forward(const Geom& g, int ndim, const void* x, const void* off, const void* w, const void* bias,
                       void* y, cudaStream_t st);
int simt_small_backward(const Geom& g, int ndim, const void* x, const void* off, const void* w, const void* dy,
                        void* dx, void* doff, void* dw, cudaStream_t st);
// fused layer forward for small problems: offsets computed in the kernel (gq: the offset-producing convolution)
bool simt_small_layer_supported(const Geom& g, const Geom& gq, int dtype, int ndim);
int simt_small_layer_forward(const Geom& g, const Geom& gq, int ndim, const void* x, const void* w_off, const void* b_off,
                             const void* w, const void* bias, void* offsets, void* y, cudaStream_t st);
int simt_small_layer_backward(const Geom& g, const Geom& gq, int ndim, const void* x, const void* offsets,
                              const void* w_off, const void* w, const void* dy, void* dx, void* dw_off, void* db_off,
                              void* dw, cudaStream_t st);
bool simt_backward_both_supported(const Geom& g, int dtype);
int simt_backward_both(const Geom& g, int ndim, int deform, const void* x, const void* off, const void* w,
                       const void* dy, void* dx, void* doff, void* dw, cudaStream_t st);
int bias_grad(const Geom& g, int dtype, const void* dy, void* dbias, cudaStream_t st);
int debug_points(const Geom& g, int dtype, int ndim, const void* off, int n, void* coords, int32_t* valid,
                 int32_t* lo, int32_t* hi, cudaStream_t st);

// BF16 tensor-core (tcgen05) path, dcn_tc.cu.  fp32 tensors only.
bool tc_supported(const Geom& g, int ndim, int deform);
size_t tc_workspace_bytes(const Geom& g, int ndim, int pass);
int tc_forward(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
               const float* bias, float* y, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_backward_data(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
                     const float* dy, float* dx, float* doff, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_backward_weight(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* dy,
                       float* dw, void* ws, size_t ws_bytes, cudaStream_t st);
size_t tc_backward_workspace_bytes(const Geom& g);
int tc_backward(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
                const float* dy, const void* xcl_in, float* dx, float* doff, float* dw, void* ws, size_t ws_bytes,
                cudaStream_t st);
// deformable layer = offset-producing plain convolution (gq) + deformable convolution (g) of the same input
size_t tc_layer_workspace_bytes(const Geom& g, const Geom& gq, int ndim, int pass);
int tc_layer_forward(const Geom& g, const Geom& gq, int ndim, const float* x, const float* w_off, const float* b_off,
                     const float* w, const float* bias, float* offsets, float* y, void* ws, size_t ws_bytes,
                     cudaStream_t st);
int tc_layer_backward(const Geom& g, const Geom& gq, int ndim, const float* x, const float* offsets, const float* w_off,
                      const float* w, const float* dy, const void* xcl_in, float* dx, float* dw_off, float* dw,
                      float** doff_out, void* ws, size_t ws_bytes, cudaStream_t st);
int tc_forward_static(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
                      const float* bias, float* y, cudaStream_t st);
size_t tc_static_scratch_bytes();
int tc_check_status(cudaStream_t st);
int tc_debug_expire_wait(int* gave_up, cudaStream_t st);
int tc_launch_count(const Geom& g, int ndim, int deform, int pass);
int tc_debug_points(const Geom& g, int ndim, int deform, const float* off, int n, float* coords, int32_t* valid,
                    int32_t* lo, int32_t* hi, void* ws, size_t ws_bytes, cudaStream_t st);

}  // namespace dcn
