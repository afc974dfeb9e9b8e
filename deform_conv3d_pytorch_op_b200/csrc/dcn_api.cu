// C-ABI layer of libdcn: argument validation (the reference's shape_check contract restated on plain
// sizes), geometry set-up and dispatch to the kernel files.  Declarations and the reference line each
// entry point replaces are in include/dcn.h.
#include "../../include/dcn.h"
#include "dcn_internal.h"

namespace {

using dcn::Geom;

int out_size_1d(int in, int pad, int k, int stride, int dil, int std_rule) {
    // deformable packages: deform3d/lib/deform_conv3d_cuda.cpp:15-17 (dilation ignored)
    // plain conv:          conv2d/lib/conv2d_cuda.cpp:20-22
    if (std_rule) return (in + 2 * pad - dil * (k - 1) - 1) / stride + 1;
    return (in + 2 * pad - k) / stride + 1;
}

int validate(const dcn_problem* p) {
    if (p == nullptr) return DCN_ERR_NULL;
    if (p->ndim != 2 && p->ndim != 3) return DCN_ERR_UNSUPPORTED;
    if (p->dtype != DCN_F32 && p->dtype != DCN_F64) return DCN_ERR_UNSUPPORTED;
    if (p->precision != DCN_PREC_EXACT && p->precision != DCN_PREC_BF16) return DCN_ERR_UNSUPPORTED;
    if (p->precision == DCN_PREC_BF16 && p->dtype != DCN_F32) return DCN_ERR_UNSUPPORTED;
    if (p->channels_last != 0 && p->channels_last != 1) return DCN_ERR_UNSUPPORTED;
    if (p->channels_last && p->precision != DCN_PREC_BF16) return DCN_ERR_UNSUPPORTED;   // the SIMT kernels are NCHW
    if (p->N < 1 || p->C < 1 || p->O < 1 || p->G < 1) return DCN_ERR_SHAPE;
    if (p->C % p->G != 0 || p->O % p->G != 0) return DCN_ERR_SHAPE;            // deform_conv3d_model.py:32-35
    if (p->deformable) {
        if (p->cpg < 1 || p->C % p->cpg != 0) return DCN_ERR_SHAPE;           // offset channel count must be whole
    }
    long long iv = 1, ov = 1, kv = 1;
    for (int d = 0; d < 3; ++d) {
        if (p->ndim == 2 && d == 0) {
            if (p->in[0] != 1 || p->k[0] != 1 || p->stride[0] != 1 || p->pad[0] != 0 || p->dil[0] != 1)
                return DCN_ERR_SHAPE;
        }
        if (p->in[d] < 1 || p->k[d] < 1 || p->stride[d] < 1 || p->pad[d] < 0 || p->dil[d] < 1) return DCN_ERR_SHAPE;
        const int o = out_size_1d(p->in[d], p->pad[d], p->k[d], p->stride[d], p->dil[d], p->std_size_rule);
        if (o < 1) return DCN_ERR_SHAPE;
        iv *= p->in[d]; ov *= o; kv *= p->k[d];
    }
    // index ranges the kernels assume (32-bit flattened positions and per-sample plane offsets)
    if ((long long)p->N * ov >= (1ll << 31) || (long long)p->N * iv >= (1ll << 31)) return DCN_ERR_LIMIT;
    if ((long long)p->C * iv >= (1ll << 31) || (long long)(p->C / p->G) * kv >= (1ll << 31)) return DCN_ERR_LIMIT;
    if (p->deformable && (long long)(p->C / p->cpg) * kv * p->ndim * ov >= (1ll << 31)) return DCN_ERR_LIMIT;
    return DCN_OK;
}

void make_geom(const dcn_problem* p, Geom& g) {
    g.N = p->N; g.C = p->C; g.O = p->O; g.G = p->G;
    g.cpg = p->deformable ? p->cpg : p->C;
    g.dg = p->C / g.cpg;
    g.iv = g.ov = g.kv = 1;
    for (int d = 0; d < 3; ++d) {
        g.in[d] = p->in[d]; g.k[d] = p->k[d]; g.stride[d] = p->stride[d]; g.pad[d] = p->pad[d]; g.dil[d] = p->dil[d];
        g.out[d] = out_size_1d(p->in[d], p->pad[d], p->k[d], p->stride[d], p->dil[d], p->std_size_rule);
        g.iv *= g.in[d]; g.ov *= g.out[d]; g.kv *= g.k[d];
    }
    g.Cg = g.C / g.G; g.Og = g.O / g.G; g.Kg = g.Cg * g.kv;
    g.oob = (p->ndim == 3 && p->deformable && p->oob_offset_grad) ? 1 : 0;
    g.cl = p->channels_last ? 1 : 0;
    g.P = (long long)g.N * g.ov;
    g.d_ov.init(g.ov); g.d_ow.init(g.out[2]); g.d_oh.init(g.out[1]);
    g.d_kw.init(g.k[2]); g.d_kh.init(g.k[1]); g.d_kv.init(g.kv);
    g.d_Cg.init(g.Cg); g.d_cpg.init(g.cpg);
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

bool workspace_ok(const void* ws, size_t have, size_t need) {
    if (need == 0) return true;
    return ws != nullptr && have >= need && aligned(ws, 256);
}

int check_ptrs(const dcn_problem* p, std::initializer_list<const void*> ptrs) {
    const size_t es = p->dtype == DCN_F64 ? 8 : 4;
    for (const void* q : ptrs)
        if (q != nullptr && !aligned(q, es)) return DCN_ERR_ALIGN;
    return DCN_OK;
}

}  // namespace

extern "C" {

int dcn_version(void) { return 100; }

const char* dcn_status_string(int s) {
    switch (s) {
        case DCN_OK: return "ok";
        case DCN_ERR_NULL: return "a required pointer is NULL";
        case DCN_ERR_SHAPE: return "sizes violate the operator's shape contract";
        case DCN_ERR_UNSUPPORTED: return "dtype / precision / dimensionality not supported";
        case DCN_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case DCN_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
        case DCN_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case DCN_ERR_ALIGN: return "pointer not aligned for the element type";
        case DCN_ERR_LIMIT: return "problem exceeds a fixed capacity";
        default: return "unknown status";
    }
}

int dcn_output_size(const dcn_problem* p, int32_t out[3]) {
    if (p == nullptr || out == nullptr) return DCN_ERR_NULL;
    const int v = validate(p);
    if (v != DCN_OK) return v;
    for (int d = 0; d < 3; ++d)
        out[d] = out_size_1d(p->in[d], p->pad[d], p->k[d], p->stride[d], p->dil[d], p->std_size_rule);
    return DCN_OK;
}

int dcn_validate(const dcn_problem* p) { return validate(p); }

int dcn_precision_supported(const dcn_problem* p) {
    if (validate(p) != DCN_OK) return 0;
    if (p->precision == DCN_PREC_EXACT) return 1;
    Geom g;
    make_geom(p, g);
    return dcn::tc_supported(g, p->ndim, p->deformable) ? 1 : 0;
}

size_t dcn_workspace_bytes(const dcn_problem* p, int pass) {
    if (validate(p) != DCN_OK || p->precision == DCN_PREC_EXACT) return 0;
    Geom g;
    make_geom(p, g);
    if (!dcn::tc_supported(g, p->ndim, p->deformable)) return 0;
    if (pass == DCN_PASS_BACKWARD) return dcn::tc_backward_workspace_bytes(g);
    return dcn::tc_workspace_bytes(g, p->ndim, pass);
}

int dcn_launch_count(const dcn_problem* p, int pass) {
    if (validate(p) != DCN_OK) return 0;
    Geom g;
    make_geom(p, g);
    if (p->precision == DCN_PREC_EXACT) {
        if (pass != DCN_PASS_BACKWARD) return 1;
        if (dcn::simt_small_supported(g, p->dtype, p->ndim, p->deformable)) return 2;      // zero fill + one kernel
        return dcn::simt_backward_both_supported(g, p->dtype) ? 1 : 2;
    }
    if (!dcn::tc_supported(g, p->ndim, p->deformable)) return 0;
    return dcn::tc_launch_count(g, p->ndim, p->deformable, pass);
}

int dcn_forward(const dcn_problem* p, const void* x, const void* offset, const void* weight, const void* bias,
                void* y, void* ws, size_t ws_bytes, void* stream) {
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (x == nullptr || weight == nullptr || y == nullptr || (p->deformable && offset == nullptr)) return DCN_ERR_NULL;
    const int a = check_ptrs(p, {x, offset, weight, bias, y});
    if (a != DCN_OK) return a;
    Geom g;
    make_geom(p, g);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p->precision == DCN_PREC_BF16) {
        if (!dcn::tc_supported(g, p->ndim, p->deformable)) return DCN_ERR_UNSUPPORTED;
        if (!workspace_ok(ws, ws_bytes, dcn::tc_workspace_bytes(g, p->ndim, DCN_PASS_FORWARD))) return DCN_ERR_WORKSPACE;
        return dcn::tc_forward(g, p->ndim, p->deformable, (const float*)x, (const float*)offset,
                               (const float*)weight, (const float*)bias, (float*)y, ws, ws_bytes, st);
    }
    if (dcn::simt_small_supported(g, p->dtype, p->ndim, p->deformable))
        return dcn::simt_small_forward(g, p->ndim, x, offset, weight, bias, y, st);
    return dcn::simt_forward(g, p->dtype, p->ndim, p->deformable, x, offset, weight, bias, y, st);
}

size_t dcn_static_scratch_bytes(void) { return dcn::tc_static_scratch_bytes(); }

int dcn_forward_static_scratch(const dcn_problem* p, const void* x, const void* offset, const void* weight,
                               const void* bias, void* y, void* stream) {
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (p->precision != DCN_PREC_BF16) return DCN_ERR_UNSUPPORTED;     // the EXACT path has no scratch to replace
    if (x == nullptr || weight == nullptr || y == nullptr || (p->deformable && offset == nullptr)) return DCN_ERR_NULL;
    const int a = check_ptrs(p, {x, offset, weight, bias, y});
    if (a != DCN_OK) return a;
    Geom g;
    make_geom(p, g);
    if (!dcn::tc_supported(g, p->ndim, p->deformable)) return DCN_ERR_UNSUPPORTED;
    if (dcn::tc_workspace_bytes(g, p->ndim, DCN_PASS_FORWARD) > dcn::tc_static_scratch_bytes()) return DCN_ERR_LIMIT;
    return dcn::tc_forward_static(g, p->ndim, p->deformable, (const float*)x, (const float*)offset,
                                  (const float*)weight, (const float*)bias, (float*)y,
                                  static_cast<cudaStream_t>(stream));
}

int dcn_backward_data(const dcn_problem* p, const void* x, const void* offset, const void* weight, const void* dy,
                      void* dx, void* doffset, void* ws, size_t ws_bytes, void* stream) {
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (weight == nullptr || dy == nullptr) return DCN_ERR_NULL;
    if (p->deformable && (x == nullptr || offset == nullptr)) return DCN_ERR_NULL;
    if (dx == nullptr && doffset == nullptr) return DCN_OK;
    const int a = check_ptrs(p, {x, offset, weight, dy, dx, doffset});
    if (a != DCN_OK) return a;
    Geom g;
    make_geom(p, g);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p->precision == DCN_PREC_BF16) {
        if (!dcn::tc_supported(g, p->ndim, p->deformable)) return DCN_ERR_UNSUPPORTED;
        if (!workspace_ok(ws, ws_bytes, dcn::tc_workspace_bytes(g, p->ndim, DCN_PASS_BACKWARD_DATA)))
            return DCN_ERR_WORKSPACE;
        return dcn::tc_backward_data(g, p->ndim, p->deformable, (const float*)x, (const float*)offset,
                                     (const float*)weight, (const float*)dy, (float*)dx, (float*)doffset, ws,
                                     ws_bytes, st);
    }
    return dcn::simt_backward_data(g, p->dtype, p->ndim, p->deformable, x, offset, weight, dy, dx,
                                   p->deformable ? doffset : nullptr, st);
}

int dcn_backward_weight(const dcn_problem* p, const void* x, const void* offset, const void* dy, void* dweight,
                        void* dbias, void* ws, size_t ws_bytes, void* stream) {
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (x == nullptr || dy == nullptr || (p->deformable && offset == nullptr)) return DCN_ERR_NULL;
    if (dweight == nullptr && dbias == nullptr) return DCN_OK;
    const int a = check_ptrs(p, {x, offset, dy, dweight, dbias});
    if (a != DCN_OK) return a;
    Geom g;
    make_geom(p, g);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int r = DCN_OK;
    if (dweight != nullptr) {
        if (p->precision == DCN_PREC_BF16) {
            if (!dcn::tc_supported(g, p->ndim, p->deformable)) return DCN_ERR_UNSUPPORTED;
            if (!workspace_ok(ws, ws_bytes, dcn::tc_workspace_bytes(g, p->ndim, DCN_PASS_BACKWARD_WEIGHT)))
                return DCN_ERR_WORKSPACE;
            r = dcn::tc_backward_weight(g, p->ndim, p->deformable, (const float*)x, (const float*)offset,
                                        (const float*)dy, (float*)dweight, ws, ws_bytes, st);
        } else {
            r = dcn::simt_backward_weight(g, p->dtype, p->ndim, p->deformable, x, offset, dy, dweight, st);
        }
        if (r != DCN_OK) return r;
    }
    if (dbias != nullptr) r = dcn::bias_grad(g, p->dtype, dy, dbias, st);
    return r;
}

int dcn_backward(const dcn_problem* p, const void* x, const void* offset, const void* weight, const void* dy,
                 const void* x_channels_last, void* dx, void* doffset, void* dweight, void* dbias, void* ws,
                 size_t ws_bytes, void* stream) {
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (x == nullptr || weight == nullptr || dy == nullptr || (p->deformable && offset == nullptr)) return DCN_ERR_NULL;
    const int a = check_ptrs(p, {x, offset, weight, dy, dx, doffset, dweight, dbias});
    if (a != DCN_OK) return a;
    Geom g;
    make_geom(p, g);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int r = DCN_OK;
    if (dx != nullptr || doffset != nullptr || dweight != nullptr) {
        if (p->precision == DCN_PREC_BF16) {
            if (!dcn::tc_supported(g, p->ndim, p->deformable)) return DCN_ERR_UNSUPPORTED;
            if (!workspace_ok(ws, ws_bytes, dcn::tc_backward_workspace_bytes(g))) return DCN_ERR_WORKSPACE;
            if (x_channels_last != nullptr && !aligned(x_channels_last, 16)) return DCN_ERR_ALIGN;
            r = dcn::tc_backward(g, p->ndim, p->deformable, (const float*)x, (const float*)offset, (const float*)weight,
                                 (const float*)dy, x_channels_last, (float*)dx, (float*)doffset, (float*)dweight, ws,
                                 ws_bytes, st);
        } else {
            const size_t es = p->dtype == DCN_F64 ? 8 : 4;
            const bool small = dcn::simt_small_supported(g, p->dtype, p->ndim, p->deformable);
            // (the small-problem path zero-fills its outputs itself, in one launch that its main kernel overlaps)
            if (!small && dx != nullptr && cudaMemsetAsync(dx, 0, (size_t)g.N * g.C * g.iv * es, st) != cudaSuccess)
                return DCN_ERR_CUDA;
            if (!small && dweight != nullptr && cudaMemsetAsync(dweight, 0, (size_t)g.O * g.Cg * g.kv * es, st) != cudaSuccess)
                return DCN_ERR_CUDA;
            const bool all = dx != nullptr && dweight != nullptr && (!p->deformable || doffset != nullptr);
            if (small) {
                r = dcn::simt_small_backward(g, p->ndim, x, offset, weight, dy, dx, doffset, dweight, st);
            } else if (all && dcn::simt_backward_both_supported(g, p->dtype)) {
                r = dcn::simt_backward_both(g, p->ndim, p->deformable, x, offset, weight, dy, dx,
                                            p->deformable ? doffset : nullptr, dweight, st);     // one launch
            } else {
                if (dx != nullptr || doffset != nullptr)
                    r = dcn::simt_backward_data(g, p->dtype, p->ndim, p->deformable, x, offset, weight, dy, dx,
                                                p->deformable ? doffset : nullptr, st);
                if (r == DCN_OK && dweight != nullptr)
                    r = dcn::simt_backward_weight(g, p->dtype, p->ndim, p->deformable, x, offset, dy, dweight, st);
            }
        }
        if (r != DCN_OK) return r;
    }
    if (dbias != nullptr) r = dcn::bias_grad(g, p->dtype, dy, dbias, st);
    return r;
}

int dcn_debug_points(const dcn_problem* p, const void* offset, int32_t n, void* coords, int32_t* valid,
                     int32_t* lo, int32_t* hi, void* stream) {
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (!p->deformable) return DCN_ERR_UNSUPPORTED;
    if (offset == nullptr || coords == nullptr || valid == nullptr || lo == nullptr || hi == nullptr) return DCN_ERR_NULL;
    if (n < 0 || n >= p->N) return DCN_ERR_SHAPE;
    Geom g;
    make_geom(p, g);
    return dcn::debug_points(g, p->dtype, p->ndim, offset, n, coords, valid, lo, hi, static_cast<cudaStream_t>(stream));
}

int dcn_debug_tc_points(const dcn_problem* p, const void* offset, int32_t n, void* coords, int32_t* valid,
                        int32_t* lo, int32_t* hi, void* ws, size_t ws_bytes, void* stream) {
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (!p->deformable || p->precision != DCN_PREC_BF16) return DCN_ERR_UNSUPPORTED;
    if (offset == nullptr || coords == nullptr || valid == nullptr || lo == nullptr || hi == nullptr) return DCN_ERR_NULL;
    if (n < 0 || n >= p->N) return DCN_ERR_SHAPE;
    Geom g;
    make_geom(p, g);
    if (!dcn::tc_supported(g, p->ndim, p->deformable)) return DCN_ERR_UNSUPPORTED;
    if (!workspace_ok(ws, ws_bytes, dcn::tc_backward_workspace_bytes(g))) return DCN_ERR_WORKSPACE;
    return dcn::tc_debug_points(g, p->ndim, p->deformable, (const float*)offset, n, (float*)coords, valid, lo, hi, ws,
                                ws_bytes, static_cast<cudaStream_t>(stream));
}

int dcn_debug_expire_wait(int32_t* gave_up, void* stream) {
    return dcn::tc_debug_expire_wait(gave_up, static_cast<cudaStream_t>(stream));
}

int dcn_check_status(void* stream) { return dcn::tc_check_status(static_cast<cudaStream_t>(stream)); }

// ------------------------------------------------------------------------------------------------
// Deformable layer: offset-producing convolution + deformable convolution of the same input
// ------------------------------------------------------------------------------------------------
int dcn_offset_conv_problem(const dcn_problem* p, dcn_problem* q) {
    if (p == nullptr || q == nullptr) return DCN_ERR_NULL;
    const int v = validate(p);
    if (v != DCN_OK) return v;
    if (!p->deformable) return DCN_ERR_UNSUPPORTED;
    *q = *p;
    int kv = 1;
    for (int d = 0; d < 3; ++d) {
        kv *= p->k[d];
        q->dil[d] = 1;          // the deformable size rule ignores dilation: only dilation 1 gives the same output size
    }
    q->O = (p->C / p->cpg) * kv * p->ndim;
    q->G = 1;
    q->cpg = p->C;
    q->deformable = 0;
    q->std_size_rule = 1;
    q->oob_offset_grad = 0;
    q->channels_last = 0;       // offsets are [N, dg*kv*D, out...] whatever the layout of x
    return validate(q);
}

static size_t layer_doff_bytes(const dcn_problem* p, const Geom& g) {
    const size_t es = p->dtype == DCN_F64 ? 8 : 4;
    return ((size_t)g.N * g.dg * g.kv * p->ndim * g.ov * es + 255) / 256 * 256;
}

size_t dcn_layer_workspace_bytes(const dcn_problem* p, int pass) {
    dcn_problem q;
    if (dcn_offset_conv_problem(p, &q) != DCN_OK) return 0;
    Geom g, gq;
    make_geom(p, g);
    make_geom(&q, gq);
    if (p->precision == DCN_PREC_EXACT) return pass == DCN_PASS_FORWARD ? 0 : layer_doff_bytes(p, g);
    if (!dcn::tc_supported(g, p->ndim, 1) || !dcn::tc_supported(gq, p->ndim, 0)) return 0;
    return dcn::tc_layer_workspace_bytes(g, gq, p->ndim, pass == DCN_PASS_FORWARD ? 0 : 3);
}

int dcn_layer_launch_count(const dcn_problem* p, int pass) {
    dcn_problem q;
    if (dcn_offset_conv_problem(p, &q) != DCN_OK) return 0;
    Geom g, gq;
    make_geom(p, g);
    make_geom(&q, gq);
    if (pass == DCN_PASS_FORWARD) {
        if (p->precision == DCN_PREC_EXACT && dcn::simt_small_layer_supported(g, gq, p->dtype, p->ndim)) return 1;
        // (bf16: the input copy is built once for both convolutions)
        const int both = dcn_launch_count(&q, DCN_PASS_FORWARD) + dcn_launch_count(p, DCN_PASS_FORWARD);
        return p->precision == DCN_PREC_BF16 && both > 0 ? both - 1 : both;
    }
    if (pass != DCN_PASS_BACKWARD) return 0;
    if (p->precision == DCN_PREC_EXACT && dcn::simt_small_layer_supported(g, gq, p->dtype, p->ndim)) return 2;
    const int main = dcn_launch_count(p, DCN_PASS_BACKWARD);
    const int rest = dcn_launch_count(&q, DCN_PASS_BACKWARD_DATA) + dcn_launch_count(&q, DCN_PASS_BACKWARD_WEIGHT);
    if (main == 0 || rest == 0) return 0;
    // bf16: the plain convolution's two gradient kernels share the packed dOffset and take the input copy over
    return p->precision == DCN_PREC_BF16 ? main + rest - 2 : main + rest;
}

int dcn_layer_forward(const dcn_problem* p, const void* x, const void* offset_weight, const void* offset_bias,
                      const void* weight, const void* bias, void* offset, void* y, void* ws, size_t ws_bytes,
                      void* stream) {
    dcn_problem q;
    const int v = dcn_offset_conv_problem(p, &q);
    if (v != DCN_OK) return v;
    if (x == nullptr || offset_weight == nullptr || weight == nullptr || offset == nullptr || y == nullptr)
        return DCN_ERR_NULL;
    const int a = check_ptrs(p, {x, offset_weight, offset_bias, weight, bias, offset, y});
    if (a != DCN_OK) return a;
    if (p->precision == DCN_PREC_EXACT) {
        Geom g, gq;
        make_geom(p, g);
        make_geom(&q, gq);
        if (dcn::simt_small_layer_supported(g, gq, p->dtype, p->ndim))      // one kernel, offsets formed on the SM
            return dcn::simt_small_layer_forward(g, gq, p->ndim, x, offset_weight, offset_bias, weight, bias, offset, y,
                                                 static_cast<cudaStream_t>(stream));
        const int r = dcn_forward(&q, x, nullptr, offset_weight, offset_bias, offset, nullptr, 0, stream);
        if (r != DCN_OK) return r;
        return dcn_forward(p, x, offset, weight, bias, y, nullptr, 0, stream);
    }
    if (p->dtype != DCN_F32) return DCN_ERR_UNSUPPORTED;
    Geom g, gq;
    make_geom(p, g);
    make_geom(&q, gq);
    if (!dcn::tc_supported(g, p->ndim, 1) || !dcn::tc_supported(gq, p->ndim, 0)) return DCN_ERR_UNSUPPORTED;
    if (!workspace_ok(ws, ws_bytes, dcn::tc_layer_workspace_bytes(g, gq, p->ndim, 0))) return DCN_ERR_WORKSPACE;
    return dcn::tc_layer_forward(g, gq, p->ndim, (const float*)x, (const float*)offset_weight, (const float*)offset_bias,
                                 (const float*)weight, (const float*)bias, (float*)offset, (float*)y, ws, ws_bytes,
                                 static_cast<cudaStream_t>(stream));
}

int dcn_layer_backward(const dcn_problem* p, const void* x, const void* offset, const void* offset_weight,
                       const void* weight, const void* dy, const void* x_channels_last, void* dx,
                       void* doffset_weight, void* doffset_bias, void* dweight, void* dbias, void* ws, size_t ws_bytes,
                       void* stream) {
    dcn_problem q;
    const int v = dcn_offset_conv_problem(p, &q);
    if (v != DCN_OK) return v;
    if (x == nullptr || offset == nullptr || offset_weight == nullptr || weight == nullptr || dy == nullptr)
        return DCN_ERR_NULL;
    const int a = check_ptrs(p, {x, offset, offset_weight, weight, dy, dx, doffset_weight, doffset_bias, dweight, dbias});
    if (a != DCN_OK) return a;
    Geom g, gq;
    make_geom(p, g);
    make_geom(&q, gq);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool chain = dx != nullptr || doffset_weight != nullptr || doffset_bias != nullptr;
    if (p->precision == DCN_PREC_EXACT && dcn::simt_small_layer_supported(g, gq, p->dtype, p->ndim)) {
        // one zero fill + one kernel: the offset gradient stays in shared memory and is pushed through the
        // offset-producing convolution there
        int r = DCN_OK;
        if (dx != nullptr || doffset_weight != nullptr || doffset_bias != nullptr || dweight != nullptr)
            r = dcn::simt_small_layer_backward(g, gq, p->ndim, x, offset, offset_weight, weight, dy, dx, doffset_weight,
                                               doffset_bias, dweight, st);
        if (r == DCN_OK && dbias != nullptr) r = dcn::bias_grad(g, p->dtype, dy, dbias, st);
        return r;
    }
    if (p->precision == DCN_PREC_EXACT) {
        if (chain && !workspace_ok(ws, ws_bytes, layer_doff_bytes(p, g))) return DCN_ERR_WORKSPACE;
        void* doff = chain ? ws : nullptr;
        int r = dcn_backward(p, x, offset, weight, dy, nullptr, dx, doff, dweight, dbias, nullptr, 0, stream);
        if (r != DCN_OK || !chain) return r;
        if (dx != nullptr) {                                            // accumulates into the dx just written
            r = dcn_backward_data(&q, nullptr, nullptr, offset_weight, doff, dx, nullptr, nullptr, 0, stream);
            if (r != DCN_OK) return r;
        }
        if (doffset_weight != nullptr) {
            const size_t es = p->dtype == DCN_F64 ? 8 : 4;
            if (cudaMemsetAsync(doffset_weight, 0, (size_t)gq.O * gq.Cg * gq.kv * es, st) != cudaSuccess) return DCN_ERR_CUDA;
        }
        if (doffset_weight != nullptr || doffset_bias != nullptr)
            r = dcn_backward_weight(&q, x, nullptr, doff, doffset_weight, doffset_bias, nullptr, 0, stream);
        return r;
    }
    if (p->dtype != DCN_F32) return DCN_ERR_UNSUPPORTED;
    if (!dcn::tc_supported(g, p->ndim, 1) || !dcn::tc_supported(gq, p->ndim, 0)) return DCN_ERR_UNSUPPORTED;
    if (!workspace_ok(ws, ws_bytes, dcn::tc_layer_workspace_bytes(g, gq, p->ndim, 3))) return DCN_ERR_WORKSPACE;
    if (x_channels_last != nullptr && !aligned(x_channels_last, 16)) return DCN_ERR_ALIGN;
    float* doff = nullptr;
    int r = dcn::tc_layer_backward(g, gq, p->ndim, (const float*)x, (const float*)offset, (const float*)offset_weight,
                                   (const float*)weight, (const float*)dy, x_channels_last, (float*)dx,
                                   (float*)doffset_weight, (float*)dweight, doffset_bias != nullptr ? &doff : nullptr, ws,
                                   ws_bytes, st);
    if (r != DCN_OK) return r;
    if (dbias != nullptr) {
        r = dcn::bias_grad(g, p->dtype, dy, dbias, st);
        if (r != DCN_OK) return r;
    }
    if (doffset_bias != nullptr) r = dcn::bias_grad(gq, p->dtype, doff, doffset_bias, st);
    return r;
}

// ------------------------------------------------------------------------------------------------
// Reference-named wrappers
// ------------------------------------------------------------------------------------------------
static dcn_problem make3d(int dtype, int N, int C, int L, int H, int W, int O, int kl, int kh, int kw, int pl, int ph,
                          int pw, int sl, int sh, int sw, int dl, int dh, int dw, int cpg, int group, int deform,
                          int std_rule, int ndim) {
    dcn_problem p;
    p.ndim = ndim; p.dtype = dtype; p.precision = DCN_PREC_EXACT; p.deformable = deform;
    p.std_size_rule = std_rule; p.oob_offset_grad = 1;
    p.N = N; p.C = C; p.O = O; p.G = group; p.cpg = cpg;
    p.in[0] = L; p.in[1] = H; p.in[2] = W;
    p.k[0] = kl; p.k[1] = kh; p.k[2] = kw;
    p.pad[0] = pl; p.pad[1] = ph; p.pad[2] = pw;
    p.stride[0] = sl; p.stride[1] = sh; p.stride[2] = sw;
    p.dil[0] = dl; p.dil[1] = dh; p.dil[2] = dw;
    p.channels_last = 0;
    return p;
}
static int legacy(int r) { return r == DCN_OK ? 1 : r; }

#define DCN_P3D make3d(DCN_F32, N, C, L, H, W, O, kl, kh, kw, pad_l, pad_h, pad_w, stride_l, stride_h, stride_w, \
                       dilation_l, dilation_h, dilation_w, channel_per_deformable_group, group, 1, 0, 3)

int dcn_deform3d_deform_conv_forward_cuda(
    const float* input, const float* weight, const float* offset, float* output,
    int N, int C, int L, int H, int W, int O, int kl, int kh, int kw,
    int pad_l, int pad_h, int pad_w, int stride_l, int stride_h, int stride_w,
    int dilation_l, int dilation_h, int dilation_w, int channel_per_deformable_group, int group, void* stream) {
    dcn_problem p = DCN_P3D;
    return legacy(dcn_forward(&p, input, offset, weight, nullptr, output, nullptr, 0, stream));
}
int dcn_deform3d_deform_conv_backward_input_offset_cuda(
    const float* input, const float* weight, const float* offset, const float* grad_output,
    float* grad_input, float* grad_offset,
    int N, int C, int L, int H, int W, int O, int kl, int kh, int kw,
    int pad_l, int pad_h, int pad_w, int stride_l, int stride_h, int stride_w,
    int dilation_l, int dilation_h, int dilation_w, int channel_per_deformable_group, int group, void* stream) {
    dcn_problem p = DCN_P3D;
    return legacy(dcn_backward_data(&p, input, offset, weight, grad_output, grad_input, grad_offset, nullptr, 0, stream));
}
int dcn_deform3d_deform_conv_backward_weight_cuda(
    const float* input, const float* offset, const float* grad_output, float* grad_weight,
    int N, int C, int L, int H, int W, int O, int kl, int kh, int kw,
    int pad_l, int pad_h, int pad_w, int stride_l, int stride_h, int stride_w,
    int dilation_l, int dilation_h, int dilation_w, int channel_per_deformable_group, int group, void* stream) {
    dcn_problem p = DCN_P3D;
    return legacy(dcn_backward_weight(&p, input, offset, grad_output, grad_weight, nullptr, nullptr, 0, stream));
}

#define DCN_P2D make3d(DCN_F32, N, C, 1, H, W, O, 1, kh, kw, 0, pad_h, pad_w, 1, stride_h, stride_w, 1, 1, 1, \
                       channel_per_deformable_group, 1, 1, 0, 2)

int dcn_deform2d_deform_conv_forward_cuda(
    const float* input, const float* weight, const float* offset, float* output,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int channel_per_deformable_group, void* stream) {
    dcn_problem p = DCN_P2D;
    return legacy(dcn_forward(&p, input, offset, weight, nullptr, output, nullptr, 0, stream));
}
int dcn_deform2d_deform_conv_backward_input_offset_cuda(
    const float* input, const float* weight, const float* offset, const float* grad_output,
    float* grad_input, float* grad_offset,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int channel_per_deformable_group, void* stream) {
    dcn_problem p = DCN_P2D;
    return legacy(dcn_backward_data(&p, input, offset, weight, grad_output, grad_input, grad_offset, nullptr, 0, stream));
}
int dcn_deform2d_deform_conv_backward_weight_cuda(
    const float* input, const float* offset, const float* grad_output, float* grad_weight,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int channel_per_deformable_group, void* stream) {
    dcn_problem p = DCN_P2D;
    return legacy(dcn_backward_weight(&p, input, offset, grad_output, grad_weight, nullptr, nullptr, 0, stream));
}

#define DCN_P2DD make3d(DCN_F64, N, C, 1, H, W, O, 1, kh, kw, 0, pad_h, pad_w, 1, stride_h, stride_w, 1, dilation_h, \
                        dilation_w, channel_per_deformable_group, group, 1, 0, 2)

int dcn_deform2d_double_deform_conv_forward_cuda(
    const double* input, const double* weight, const double* offset, double* output,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
    int channel_per_deformable_group, int group, void* stream) {
    dcn_problem p = DCN_P2DD;
    return legacy(dcn_forward(&p, input, offset, weight, nullptr, output, nullptr, 0, stream));
}
int dcn_deform2d_double_deform_conv_backward_input_offset_cuda(
    const double* input, const double* weight, const double* offset, const double* grad_output,
    double* grad_input, double* grad_offset,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
    int channel_per_deformable_group, int group, void* stream) {
    dcn_problem p = DCN_P2DD;
    return legacy(dcn_backward_data(&p, input, offset, weight, grad_output, grad_input, grad_offset, nullptr, 0, stream));
}
int dcn_deform2d_double_deform_conv_backward_weight_cuda(
    const double* input, const double* offset, const double* grad_output, double* grad_weight,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
    int channel_per_deformable_group, int group, void* stream) {
    dcn_problem p = DCN_P2DD;
    return legacy(dcn_backward_weight(&p, input, offset, grad_output, grad_weight, nullptr, nullptr, 0, stream));
}

#define DCN_PC2D make3d(DCN_F32, N, C, 1, H, W, O, 1, kh, kw, 0, pad_h, pad_w, 1, stride_h, stride_w, 1, dilation_h, \
                        dilation_w, C, group, 0, 1, 2)

int dcn_conv2d_conv_forward_cuda(
    const float* input, const float* weight, float* output,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void* stream) {
    dcn_problem p = DCN_PC2D;
    return legacy(dcn_forward(&p, input, nullptr, weight, nullptr, output, nullptr, 0, stream));
}
int dcn_conv2d_conv_backward_input_cuda(
    const float* weight, const float* grad_output, float* grad_input,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void* stream) {
    dcn_problem p = DCN_PC2D;
    return legacy(dcn_backward_data(&p, nullptr, nullptr, weight, grad_output, grad_input, nullptr, nullptr, 0, stream));
}
int dcn_conv2d_conv_backward_weight_cuda(
    const float* input, const float* grad_output, float* grad_weight,
    int N, int C, int H, int W, int O, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void* stream) {
    dcn_problem p = DCN_PC2D;
    return legacy(dcn_backward_weight(&p, input, nullptr, grad_output, grad_weight, nullptr, nullptr, 0, stream));
}

}  // extern "C"
