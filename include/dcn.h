/*
 * dcn.h -- C ABI of the B200 (sm_100a) deformable-convolution library, libdcn.so.
 *
 * The library replaces the hot path of lshiwjx/deform_conv3d_pytorch_op: the host launchers the
 * reference exports through its FFI layer plus the device kernels and cuBLAS GEMMs they drive
 * (reference paths below are relative to that project's root):
 *
 *   deform3d/lib/deform_conv3d_cuda.h:12-34          3-D deformable conv, fp32
 *   deform2d/lib/deform_conv2d_cuda.h:12-31          2-D deformable conv, fp32 (no dilation / groups)
 *   deform2d_double/lib/deform_conv2d_cuda.h:12-34   2-D deformable conv, fp64
 *   conv2d/lib/conv2d_cuda.h:17-39                   plain 2-D conv, fp32
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; all tensor pointers are DEVICE pointers to contiguous
 *     NC(L)HW storage on the current device; `stream` is a cudaStream_t passed as void*;
 *   - nothing is allocated, nothing synchronises: work is enqueued on `stream` and the call
 *     returns; the caller owns every buffer including the workspace;
 *   - re-entrant and thread-safe: inputs are never modified (the reference launchers temporarily
 *     reshape `weight`) and the library keeps no state between calls, with two exceptions that
 *     are process-wide per device: the sticky status word read by dcn_check_status, and the fixed
 *     scratch array of dcn_forward_static_scratch (calls of that entry point must be serialised);
 *   - the generic dcn_* functions return DCN_OK (0) or a negative dcn_status; the
 *     reference-named wrappers at the bottom return 1 on success like the functions they
 *     replace, and a negative dcn_status where the reference would have raised THError.
 *
 * Tensor layouts (identical to the reference)
 *   input   [N, C, (L,) H, W]
 *   weight  [O, C/G, (kl,) kh, kw]
 *   offset  [N, dg*kv*D, out...]   channel = ((g*kv + tap)*D + d), d in (l,h,w) / (h,w) order,
 *                                  tap row-major over the kernel, dg = C / cpg
 *   output  [N, O, out...]         out_i = (in_i + 2*pad_i - k_i)/stride_i + 1 for the deformable
 *                                  operators (dilation ignored, as the reference does) and the
 *                                  usual dilation-aware size for the plain convolution.
 */
#ifndef DCN_H_
#define DCN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dcn_status {
    DCN_OK = 0,
    DCN_ERR_NULL = -1,         /* a required pointer is NULL */
    DCN_ERR_SHAPE = -2,        /* sizes violate the reference's shape_check contract */
    DCN_ERR_UNSUPPORTED = -3,  /* dtype / precision / ndim combination not provided */
    DCN_ERR_WORKSPACE = -4,    /* workspace missing, too small or misaligned */
    DCN_ERR_CUDA = -5,         /* a CUDA runtime call or launch failed */
    DCN_ERR_TIMEOUT = -6,      /* a bounded device-side wait gave up (reported by dcn_check_status) */
    DCN_ERR_ALIGN = -7,        /* a pointer is not aligned for the element type */
    DCN_ERR_LIMIT = -8         /* problem exceeds a fixed capacity of the entry point */
} dcn_status;

enum { DCN_F32 = 0, DCN_F64 = 1 };
/* EXACT: SIMT kernels computing in the tensor dtype (fp32 / fp64).
 * BF16 : fp32 tensors in and out, sampled patches and weights rounded to bf16, tcgen05 MMA with
 *        fp32 accumulation in tensor memory.  Coordinates and interpolation stay fp32. */
enum { DCN_PREC_EXACT = 0, DCN_PREC_BF16 = 1 };
enum { DCN_PASS_FORWARD = 0, DCN_PASS_BACKWARD_DATA = 1, DCN_PASS_BACKWARD_WEIGHT = 2, DCN_PASS_BACKWARD = 3 };

/* One operator instance.  For ndim == 2 only the LAST two slots of each triple are used
 * (slot 0 must hold in=1, k=1, stride=1, pad=0, dil=1). */
typedef struct dcn_problem {
    int32_t ndim;             /* 2 or 3 */
    int32_t dtype;            /* DCN_F32 / DCN_F64 */
    int32_t precision;        /* DCN_PREC_* */
    int32_t deformable;       /* 1: sample at offset positions; 0: plain convolution (offset unused) */
    int32_t std_size_rule;    /* 0: reference deformable size rule (dilation ignored); 1: dilation-aware */
    int32_t oob_offset_grad;  /* 3-D only. 1: reproduce the reference's pull-back term for invalid
                                 samples (deform3d/lib/deform_conv3d_cuda_kernel.cu:470-481); 0: zero */
    int32_t N, C, O;          /* batch, input channels, output channels */
    int32_t G;                /* convolution groups */
    int32_t cpg;              /* channels per deformable group (the reference's channel_per_group) */
    int32_t in[3], k[3], stride[3], pad[3], dil[3];
    int32_t channels_last;    /* 0: x, y and their gradients are [N, channels, spatial] as in the reference.
                                 1: they are [N, spatial, channels] (torch channels_last / channels_last_3d
                                 storage), so no layout pass runs around the kernels; offsets and their
                                 gradient stay [N, dg*kv*D, out spatial], weights [O, C/G, k].  DCN_PREC_BF16
                                 only.  The reference has no such layout (its tensors are always NCHW). */
} dcn_problem;

int dcn_version(void);
const char* dcn_status_string(int status);

/* Output spatial size under the problem's size rule; out[0] = 1 for ndim == 2.
 * Replaces input_to_output, deform3d/lib/deform_conv3d_cuda.cpp:15-17 and conv2d/lib/conv2d_cuda.cpp:20-22. */
int dcn_output_size(const dcn_problem* p, int32_t out[3]);

/* Argument contract of the reference's shape_check (deform3d/lib/deform_conv3d_cuda.cpp:24-87,
 * conv2d/lib/conv2d_cuda.cpp:29-74) on sizes alone.  DCN_OK or DCN_ERR_SHAPE / DCN_ERR_UNSUPPORTED. */
int dcn_validate(const dcn_problem* p);

/* 1 if the problem's precision can be served (EXACT always can; BF16 needs fp32 tensors and channel
 * counts per convolution group and per deformable group that are multiples of 8), else 0. */
int dcn_precision_supported(const dcn_problem* p);

/* Scratch bytes `pass` needs (0 for the EXACT precision).  The workspace must be 256-byte aligned. */
size_t dcn_workspace_bytes(const dcn_problem* p, int pass);

/* Number of kernel launches `pass` enqueues for this problem (memsets not counted); used by callers
 * that account for launches.  0 on an invalid problem. */
int dcn_launch_count(const dcn_problem* p, int pass);

/* y = conv(x sampled at offset, weight) + bias.  `offset` may be NULL when deformable == 0, `bias` may
 * be NULL.  y is overwritten.  Replaces deform_conv_forward_cuda (deform3d/lib/deform_conv3d_cuda.cpp:90-165)
 * and the Python-side bias add (deform3d/deform_conv3d_functions/deform_conv3d_function.py:41-42). */
int dcn_forward(const dcn_problem* p, const void* x, const void* offset, const void* weight, const void* bias,
                void* y, void* workspace, size_t workspace_bytes, void* stream);

/* Forward pass that allocates nothing and needs no workspace (no counterpart in the reference, which
 * leaves all allocation to its Python layer).  It is for callers that cannot hand over scratch memory:
 * code running where device allocation is forbidden or would stall the pipeline -- an inference plugin's
 * enqueue hook, a real-time loop, a process whose memory pool already owns the whole device.
 * Same arithmetic and results as dcn_forward with precision DCN_PREC_BF16 (other precisions are refused
 * with DCN_ERR_UNSUPPORTED).  The scratch is a fixed array inside the library image of
 * dcn_static_scratch_bytes() bytes (32 MiB), held on every device that loads the library until the process
 * exits; a problem whose forward workspace (dcn_workspace_bytes) exceeds it is refused with DCN_ERR_LIMIT
 * before anything is launched.  The first call on each device resolves the array's device address (this
 * may load the library's device code), so make that first call outside any stream capture.  All calls on a
 * device share the one array, which keeps the previous call's contents; this pass overwrites every byte it
 * later reads, so nothing needs clearing, but two calls whose kernels overlap on the GPU (different
 * streams, or different host threads) race on it: serialise them.  The resolved address is cached per device
 * ordinal for the life of the process and does not survive cudaDeviceReset or the destruction of the device's
 * primary context.  With CUDA's lazy module loading the first launch of each kernel variant (2-D / 3-D,
 * deformable / plain, reference / channels-last layout) may load device code as well: call once per kind of
 * problem before any stream capture. */
size_t dcn_static_scratch_bytes(void);
int dcn_forward_static_scratch(const dcn_problem* p, const void* x, const void* offset, const void* weight,
                               const void* bias, void* y, void* stream);

/* Gradients w.r.t. input and offset.  Either of dx / doffset may be NULL (not wanted).
 * dx ACCUMULATES into the caller's buffer (zero it first, as the reference's Python does,
 * deform_conv3d_function.py:53); doffset is OVERWRITTEN (reference kernel stores with `=`).
 * Replaces deform_conv_backward_input_offset_cuda (deform3d/lib/deform_conv3d_cuda.cpp:168-262). */
int dcn_backward_data(const dcn_problem* p, const void* x, const void* offset, const void* weight, const void* dy,
                      void* dx, void* doffset, void* workspace, size_t workspace_bytes, void* stream);

/* Gradient w.r.t. weight (ACCUMULATES into the caller's zeroed buffer, like the reference's beta = 1 GEMM)
 * and, if dbias != NULL, w.r.t. bias (overwritten).  Replaces deform_conv_backward_weight_cuda
 * (deform3d/lib/deform_conv3d_cuda.cpp:265-336) and the Python-side bias gradient
 * (deform_conv3d_function.py:73-74). */
int dcn_backward_weight(const dcn_problem* p, const void* x, const void* offset, const void* dy, void* dweight,
                        void* dbias, void* workspace, size_t workspace_bytes, void* stream);

/* All gradients in one call (any of dx / doffset / dweight / dbias may be NULL = not wanted).  Unlike the two
 * calls above, EVERY output is OVERWRITTEN: no zero fill by the caller.  The passes share their scratch
 * (workspace of dcn_workspace_bytes(p, DCN_PASS_BACKWARD) bytes).  `x_channels_last`, if not NULL, is the
 * channels-last bf16 copy of x that dcn_forward (precision BF16, same problem, same x) left at the START of
 * its workspace; passing it saves rebuilding it.  It is ignored by the EXACT precision.
 * Replaces deform_conv_backward_input_offset_cuda + deform_conv_backward_weight_cuda + the Python-side bias
 * gradient (deform3d/deform_conv3d_functions/deform_conv3d_function.py:46-77) as one unit. */
int dcn_backward(const dcn_problem* p, const void* x, const void* offset, const void* weight, const void* dy,
                 const void* x_channels_last, void* dx, void* doffset, void* dweight, void* dbias, void* workspace,
                 size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Deformable layer: the caller pattern of the reference's model scripts in one call -- a plain
 * convolution of x produces the offsets, the deformable convolution of the same x consumes them
 * (deform3d/test_model.py:18-30, deform2d/test_model.py:19-31, where the two are separate modules
 * and the offsets make a round trip through the framework's allocator).
 * The offset-producing convolution is fixed by the deformable problem p: same input, taps, stride and
 * padding, dilation 1 (the only one whose output size matches the deformable size rule), one group,
 * dg*kv*D output channels, weight [dg*kv*D, C, k...], optional bias [dg*kv*D];
 * dcn_offset_conv_problem fills q with it.  Offsets are always [N, dg*kv*D, out...], also with
 * channels_last activations.
 * With precision BF16 one channels-last bf16 copy of x serves both convolutions of the forward pass
 * and all gradient kernels of the backward pass, and the offsets are read back while still in L2;
 * with precision EXACT the calls below are the composition of the generic entry points.
 * ------------------------------------------------------------------------------------------- */
int dcn_offset_conv_problem(const dcn_problem* p, dcn_problem* q);

/* Scratch bytes of dcn_layer_forward (pass = DCN_PASS_FORWARD) / dcn_layer_backward (DCN_PASS_BACKWARD). */
size_t dcn_layer_workspace_bytes(const dcn_problem* p, int pass);

/* Kernel launches of dcn_layer_forward / dcn_layer_backward when every gradient is wanted (memsets not counted).
 * A small fp32 problem under precision EXACT takes ONE forward launch: the offsets are formed inside the kernel,
 * from the plain patch of the CTA's positions, and stay in shared memory for the sampling that follows (they are
 * written out once, for the backward pass), and a zero-fill launch plus ONE backward launch in which the offset
 * gradient stays in shared memory and is pushed through the offset-producing convolution in place. */
int dcn_layer_launch_count(const dcn_problem* p, int pass);

/* offset = conv(x, offset_weight) + offset_bias;  y = deform_conv(x, offset, weight) + bias.
 * `offset` (written) and `y` (written) are caller buffers; keep `offset` for the backward pass.
 * BF16: the channels-last bf16 copy of x is left at the START of the workspace, as dcn_forward does. */
int dcn_layer_forward(const dcn_problem* p, const void* x, const void* offset_weight, const void* offset_bias,
                      const void* weight, const void* bias, void* offset, void* y, void* workspace,
                      size_t workspace_bytes, void* stream);

/* Gradients of the layer: dx (through the sampled values AND through the offsets), doffset_weight,
 * doffset_bias, dweight, dbias; any may be NULL, every output is OVERWRITTEN.  The offset gradient itself
 * lives in the workspace.  `x_channels_last` as in dcn_backward. */
int dcn_layer_backward(const dcn_problem* p, const void* x, const void* offset, const void* offset_weight,
                       const void* weight, const void* dy, const void* x_channels_last, void* dx,
                       void* doffset_weight, void* doffset_bias, void* dweight, void* dbias, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Debug aid for the bit-exactness tests: for sample `n` writes, for every (deformable group, tap,
 * output position), the sampling coordinate (tensor dtype, [dg,kv,ov,ndim]), validity (int32
 * [dg,kv,ov]) and the low / high corner index per axis (int32 [dg,kv,ov,ndim], -1 when invalid),
 * computed by the same device routine the kernels use. */
int dcn_debug_points(const dcn_problem* p, const void* offset, int32_t n, void* coords, int32_t* valid,
                     int32_t* lo, int32_t* hi, void* stream);

/* Same outputs as dcn_debug_points, taken from the sampling-point entries the tensor-core backward-data kernel
 * of the 2-D deformable operator consumes: the entry pre-pass runs over the whole batch into `workspace`
 * (dcn_workspace_bytes(p, DCN_PASS_BACKWARD) bytes, where the backward pass keeps them) and sample n's entries are
 * decoded (corner indices, validity, coordinate = low corner + fraction; valid = -1 flags an entry whose two
 * encodings of the low corner disagree).  DCN_ERR_UNSUPPORTED where that kernel does not take the problem
 * (3-D, more than 16 taps, planes too large for shared memory).  fp32 tensors, precision BF16. */
int dcn_debug_tc_points(const dcn_problem* p, const void* offset, int32_t n, void* coords, int32_t* valid,
                        int32_t* lo, int32_t* hi, void* workspace, size_t workspace_bytes, void* stream);

/* Test aid for the error path of the bounded device-side waits: launches one thread that waits, with a limit of
 * about a millisecond, on a barrier nothing arrives on.  The wait gives up, the kernel returns normally (nothing
 * traps, the context stays usable), *gave_up (device pointer, may be NULL) is set to 1 and the next
 * dcn_check_status reports DCN_ERR_TIMEOUT.  No counterpart in the reference (its kernels have no error path). */
int dcn_debug_expire_wait(int32_t* gave_up, void* stream);

/* Reads and clears the sticky device-side status word of the tensor-core kernels (bounded waits that
 * gave up).  Synchronises `stream`.  DCN_OK or DCN_ERR_TIMEOUT. */
int dcn_check_status(void* stream);

/* ---------------------------------------------------------------------------------------------
 * Reference-named wrappers: one per symbol of the reference's four FFI headers, same argument
 * order, with each THCudaTensor replaced by its device pointer and the sizes the reference reads
 * from the tensor header made explicit.  `columns` (the caller-provided im2col scratch of the
 * reference) is not needed and has no counterpart.  Return 1 on success.
 * ------------------------------------------------------------------------------------------- */

/* deform3d/lib/deform_conv3d_cuda.h:12-18 */
int dcn_deform3d_deform_conv_forward_cuda(
    const float* input, const float* weight, const float* offset, float* output,
    int N, int C, int L, int H, int W, int O, int kl, int kh, int kw,
    int pad_l, int pad_h, int pad_w, int stride_l, int stride_h, int stride_w,
    int dilation_l, int dilation_h, int dilation_w, int channel_per_deformable_group, int group, void* stream);
/* deform3d/lib/deform_conv3d_cuda.h:20-26 */
int dcn_deform3d_deform_conv_backward_input_offset_cuda(
    const float* input, const float* weight, const float* offset, const float* grad_output,
    float* grad_input, float* grad_offset,
    int N, int C, int L, int H, int W, int O, int kl, int kh, int kw,
    int pad_l, int pad_h, int pad_w, int stride_l, int stride_h, int stride_w,
    int dilation_l, int dilation_h, int dilation_w, int channel_per_deformable_group, int group, void* stream);
/* deform3d/lib/deform_conv3d_cuda.h:28-34 */
int dcn_deform3d_deform_conv_backward_weight_cuda(
    const float* input, const float* offset, const float* grad_output, float* grad_weight,
    int N, int C, int L, int H, int W, int O, int kl, int kh, int kw,
    int pad_l, int pad_h, int pad_w, int stride_l, int stride_h, int stride_w,
    int dilation_l, int dilation_h, int dilation_w, int channel_per_deformable_group, int group, void* stream);

/* deform2d/lib/deform_conv2d_cuda.h:12-17 */
int dcn_deform2d_deform_conv_forward_cuda(
    const float* input, const float* weight, const float* offset, float* output,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int channel_per_deformable_group, void* stream);
/* deform2d/lib/deform_conv2d_cuda.h:19-24 */
int dcn_deform2d_deform_conv_backward_input_offset_cuda(
    const float* input, const float* weight, const float* offset, const float* grad_output,
    float* grad_input, float* grad_offset,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int channel_per_deformable_group, void* stream);
/* deform2d/lib/deform_conv2d_cuda.h:26-31 */
int dcn_deform2d_deform_conv_backward_weight_cuda(
    const float* input, const float* offset, const float* grad_output, float* grad_weight,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int channel_per_deformable_group, void* stream);

/* deform2d_double/lib/deform_conv2d_cuda.h:12-18 */
int dcn_deform2d_double_deform_conv_forward_cuda(
    const double* input, const double* weight, const double* offset, double* output,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
    int channel_per_deformable_group, int group, void* stream);
/* deform2d_double/lib/deform_conv2d_cuda.h:20-26 */
int dcn_deform2d_double_deform_conv_backward_input_offset_cuda(
    const double* input, const double* weight, const double* offset, const double* grad_output,
    double* grad_input, double* grad_offset,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
    int channel_per_deformable_group, int group, void* stream);
/* deform2d_double/lib/deform_conv2d_cuda.h:28-34 */
int dcn_deform2d_double_deform_conv_backward_weight_cuda(
    const double* input, const double* offset, const double* grad_output, double* grad_weight,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
    int channel_per_deformable_group, int group, void* stream);

/* conv2d/lib/conv2d_cuda.h:17-23 */
int dcn_conv2d_conv_forward_cuda(
    const float* input, const float* weight, float* output,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void* stream);
/* conv2d/lib/conv2d_cuda.h:25-31 */
int dcn_conv2d_conv_backward_input_cuda(
    const float* weight, const float* grad_output, float* grad_input,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void* stream);
/* conv2d/lib/conv2d_cuda.h:33-39 */
int dcn_conv2d_conv_backward_weight_cuda(
    const float* input, const float* grad_output, float* grad_weight,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DCN_H_ */
