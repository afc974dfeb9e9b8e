// TEST INFRASTRUCTURE ONLY -- not part of the shipped operator.
//
// CPU restatement of the reference's per-sample device kernels (the reference has no CPU
// path of its own; its kernels are CUDA only).  Only the tests, the smoke check and the
// CPU-baseline leg of the benchmark may load this library; the product path never does.
//
// Every function follows one reference kernel, cited by file:line (paths are relative to
// the reference project root):
//   sample geometry + bilinear / trilinear value
//       deform3d/lib/deform_conv3d_cuda_kernel.cu:12-59        (Tri_Linear)
//       deform2d/lib/deform_conv2d_cuda_kernel.cu:12-43        (Bi_Linear, fp32)
//       deform2d_double/lib/deform_conv2d_cuda_kernel.cu:25-56 (Bi_Linear, fp64)
//   deformable im2col
//       deform3d/lib/deform_conv3d_cuda_kernel.cu:62-131
//       deform2d/lib/deform_conv2d_cuda_kernel.cu:46-108       (no dilation == dilation 1)
//       deform2d_double/lib/deform_conv2d_cuda_kernel.cu:59-124
//   col2im to the input gradient
//       deform3d/lib/deform_conv3d_cuda_kernel.cu:175-298
//       deform2d/lib/deform_conv2d_cuda_kernel.cu:138-223
//       deform2d_double/lib/deform_conv2d_cuda_kernel.cu:155-241
//   col2im to the offset gradient
//       deform3d/lib/deform_conv3d_cuda_kernel.cu:340-485      (with the out-of-bounds term :470-481)
//       deform2d/lib/deform_conv2d_cuda_kernel.cu:250-347
//       deform2d_double/lib/deform_conv2d_cuda_kernel.cu:270-368
//   plain im2col / col2im
//       conv2d/lib/conv2d_cuda_kernel.cu:25-71, 101-146
//
// The per-sample / per-group host loops and the three GEMMs of the reference launchers
// (deform3d/lib/deform_conv3d_cuda.cpp:90-336 and siblings) are restated in oracle.py.
//
// Arithmetic notes.  Sampling coordinates are formed exactly as the reference does: an
// int32 base (out*stride - pad + tap*dilation) converted to the tensor type and added to the
// offset with a single rounding.  Built with -ffp-contract=off so that no multiply-add is
// fused on the host; the coordinate path contains no multiply, so it is bit-identical to the
// device code regardless of contraction.  2-D problems are passed with a leading unit
// dimension (in[0]=out[0]=k[0]=1, pad[0]=0, stride[0]=1, dil[0]=1) and ndim=2.

#include <cstdint>
#include <cstring>
#include <cmath>

namespace {

struct Geo {
    int ndim;               // 2 or 3
    int C;                  // input channels
    int in[3], out[3], k[3], pad[3], stride[3], dil[3];
    int cpg;                // channels per deformable group
    int iv() const { return in[0] * in[1] * in[2]; }
    int ov() const { return out[0] * out[1] * out[2]; }
    int kv() const { return k[0] * k[1] * k[2]; }
};

Geo make_geo(int ndim, int C, const int* in, const int* out, const int* k, const int* pad,
             const int* stride, const int* dil, int cpg) {
    Geo g;
    g.ndim = ndim;
    g.C = C;
    g.cpg = cpg;
    for (int d = 0; d < 3; ++d) {
        g.in[d] = in[d]; g.out[d] = out[d]; g.k[d] = k[d];
        g.pad[d] = pad[d]; g.stride[d] = stride[d]; g.dil[d] = dil[d];
    }
    return g;
}

// One sampling point: coordinates, validity, the corner indices and per-axis weights.
template <typename T>
struct Pt {
    T p[3];
    bool valid;
    int lo[3], hi[3];
    T lw[3], hw[3];   // lw = p - lo ("l_width" ...), hw = 1 - lw
};

// Axes used: 3-D uses 0,1,2 (l,h,w); 2-D uses 1,2 (h,w).  d0 = first active axis.
template <typename T>
inline Pt<T> locate(const Geo& g, const T* off_n, int grp, int tap, const int o[3], const int t[3]) {
    Pt<T> s;
    const int ov = g.ov();
    const int nd = g.ndim;
    const int d0 = 3 - nd;
    const int opos = (o[0] * g.out[1] + o[1]) * g.out[2] + o[2];
    const T* base = off_n + (size_t)(grp * g.kv() + tap) * nd * ov;
    s.valid = true;
    for (int d = 0; d < 3; ++d) { s.p[d] = 0; s.lo[d] = s.hi[d] = 0; s.lw[d] = 0; s.hw[d] = 1; }
    for (int d = d0; d < 3; ++d) {
        const int ib = o[d] * g.stride[d] - g.pad[d] + t[d] * g.dil[d];   // pure int32
        const T pd = (T)ib + base[(size_t)(d - d0) * ov + opos];          // one rounding
        s.p[d] = pd;
        if (!(pd > (T)-1 && pd < (T)g.in[d])) s.valid = false;
    }
    if (s.valid) {
        for (int d = d0; d < 3; ++d) {
            const T pd = s.p[d];
            const int lo = (int)pd;                                       // truncation toward zero
            const int hi = (pd >= (T)(g.in[d] - 1) || pd <= (T)0) ? lo : lo + 1;
            s.lo[d] = lo; s.hi[d] = hi;
            s.lw[d] = pd - (T)lo;
            s.hw[d] = (T)1 - s.lw[d];
        }
    }
    return s;
}

inline int lin(const Geo& g, int l, int h, int w) { return (l * g.in[1] + h) * g.in[2] + w; }

template <typename T>
inline T interp(const Geo& g, const T* plane, const Pt<T>& s) {
    if (g.ndim == 2) {
        const T c00 = plane[lin(g, 0, s.lo[1], s.lo[2])];
        const T c01 = plane[lin(g, 0, s.lo[1], s.hi[2])];
        const T c10 = plane[lin(g, 0, s.hi[1], s.lo[2])];
        const T c11 = plane[lin(g, 0, s.hi[1], s.hi[2])];
        const T c0 = c00 * s.hw[2] + c01 * s.lw[2];
        const T c1 = c10 * s.hw[2] + c11 * s.lw[2];
        return c0 * s.hw[1] + c1 * s.lw[1];
    }
    const T c000 = plane[lin(g, s.lo[0], s.lo[1], s.lo[2])];
    const T c001 = plane[lin(g, s.lo[0], s.lo[1], s.hi[2])];
    const T c010 = plane[lin(g, s.lo[0], s.hi[1], s.lo[2])];
    const T c011 = plane[lin(g, s.lo[0], s.hi[1], s.hi[2])];
    const T c100 = plane[lin(g, s.hi[0], s.lo[1], s.lo[2])];
    const T c101 = plane[lin(g, s.hi[0], s.lo[1], s.hi[2])];
    const T c110 = plane[lin(g, s.hi[0], s.hi[1], s.lo[2])];
    const T c111 = plane[lin(g, s.hi[0], s.hi[1], s.hi[2])];
    const T c00 = c000 * s.hw[2] + c001 * s.lw[2];
    const T c01 = c010 * s.hw[2] + c011 * s.lw[2];
    const T c10 = c100 * s.hw[2] + c101 * s.lw[2];
    const T c11 = c110 * s.hw[2] + c111 * s.lw[2];
    const T c0 = c00 * s.hw[1] + c01 * s.lw[1];
    const T c1 = c10 * s.hw[1] + c11 * s.lw[1];
    return c0 * s.hw[0] + c1 * s.lw[0];
}

inline void unravel_tap(const Geo& g, int tap, int t[3]) {
    t[2] = tap % g.k[2];
    t[1] = tap / g.k[2] % g.k[1];
    t[0] = tap / g.k[2] / g.k[1];
}
inline void unravel_out(const Geo& g, int pos, int o[3]) {
    o[2] = pos % g.out[2];
    o[1] = pos / g.out[2] % g.out[1];
    o[0] = pos / g.out[2] / g.out[1];
}

// col[(c,tap), pos] = sampled value or 0
template <typename T>
void deform_im2col(const Geo& g, const T* x_n, const T* off_n, T* col) {
    const int ov = g.ov(), kv = g.kv(), iv = g.iv();
#pragma omp parallel for schedule(static)
    for (int row = 0; row < g.C * kv; ++row) {
        const int c = row / kv, tap = row % kv;
        int t[3]; unravel_tap(g, tap, t);
        const int grp = c / g.cpg;
        const T* plane = x_n + (size_t)c * iv;
        T* dst = col + (size_t)row * ov;
        for (int pos = 0; pos < ov; ++pos) {
            int o[3]; unravel_out(g, pos, o);
            const Pt<T> s = locate<T>(g, off_n, grp, tap, o, t);
            dst[pos] = s.valid ? interp<T>(g, plane, s) : (T)0;
        }
    }
}

// dx_n[c, corner] += weight * col   (caller zero-fills dx_n, as the reference's Python does)
template <typename T>
void deform_col2im_input(const Geo& g, const T* col, const T* off_n, T* dx_n) {
    const int ov = g.ov(), kv = g.kv(), iv = g.iv();
#pragma omp parallel for schedule(static)
    for (int c = 0; c < g.C; ++c) {
        const int grp = c / g.cpg;
        T* plane = dx_n + (size_t)c * iv;
        for (int pos = 0; pos < ov; ++pos) {
            int o[3]; unravel_out(g, pos, o);
            for (int tap = 0; tap < kv; ++tap) {
                int t[3]; unravel_tap(g, tap, t);
                const Pt<T> s = locate<T>(g, off_n, grp, tap, o, t);
                if (!s.valid) continue;
                const T v = col[(size_t)(c * kv + tap) * ov + pos];
                if (g.ndim == 2) {
                    plane[lin(g, 0, s.lo[1], s.lo[2])] += s.hw[1] * s.hw[2] * v;
                    plane[lin(g, 0, s.lo[1], s.hi[2])] += s.hw[1] * s.lw[2] * v;
                    plane[lin(g, 0, s.hi[1], s.lo[2])] += s.lw[1] * s.hw[2] * v;
                    plane[lin(g, 0, s.hi[1], s.hi[2])] += s.lw[1] * s.lw[2] * v;
                } else {
                    plane[lin(g, s.lo[0], s.lo[1], s.lo[2])] += s.hw[0] * s.hw[1] * s.hw[2] * v;
                    plane[lin(g, s.lo[0], s.lo[1], s.hi[2])] += s.hw[0] * s.hw[1] * s.lw[2] * v;
                    plane[lin(g, s.lo[0], s.hi[1], s.lo[2])] += s.hw[0] * s.lw[1] * s.hw[2] * v;
                    plane[lin(g, s.lo[0], s.hi[1], s.hi[2])] += s.hw[0] * s.lw[1] * s.lw[2] * v;
                    plane[lin(g, s.hi[0], s.lo[1], s.lo[2])] += s.lw[0] * s.hw[1] * s.hw[2] * v;
                    plane[lin(g, s.hi[0], s.lo[1], s.hi[2])] += s.lw[0] * s.hw[1] * s.lw[2] * v;
                    plane[lin(g, s.hi[0], s.hi[1], s.lo[2])] += s.lw[0] * s.lw[1] * s.hw[2] * v;
                    plane[lin(g, s.hi[0], s.hi[1], s.hi[2])] += s.lw[0] * s.lw[1] * s.lw[2] * v;
                }
            }
        }
    }
}

// doff_n[(grp,tap,d), pos] = sum over the group's channels of col * d(val)/d(p_d)
// oob_ref != 0 adds the 3-D reference's pull-back term for invalid samples (threshold is
// in[0] for every axis, as the reference compares h and w against input_l too).
template <typename T>
void deform_col2im_offset(const Geo& g, const T* col, const T* x_n, const T* off_n, int oob_ref,
                          T* doff_n) {
    const int ov = g.ov(), kv = g.kv(), iv = g.iv();
    const int nd = g.ndim, d0 = 3 - nd;
    const int dg = g.C / g.cpg;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < dg * kv * nd; ++row) {
        const int comp = row % nd;             // 0..nd-1 in (l,)h,w order
        const int tap = row / nd % kv;
        const int grp = row / nd / kv;
        const int ax = comp + d0;              // axis index 0..2
        int t[3]; unravel_tap(g, tap, t);
        for (int pos = 0; pos < ov; ++pos) {
            int o[3]; unravel_out(g, pos, o);
            const Pt<T> s = locate<T>(g, off_n, grp, tap, o, t);
            T val = 0;
            for (int i = 0; i < g.cpg; ++i) {
                const int c = grp * g.cpg + i;
                const T cv = col[(size_t)(c * kv + tap) * ov + pos];
                const T* plane = x_n + (size_t)c * iv;
                if (s.valid) {
                    if (nd == 2) {
                        const T c00 = plane[lin(g, 0, s.lo[1], s.lo[2])];
                        const T c01 = plane[lin(g, 0, s.lo[1], s.hi[2])];
                        const T c10 = plane[lin(g, 0, s.hi[1], s.lo[2])];
                        const T c11 = plane[lin(g, 0, s.hi[1], s.hi[2])];
                        if (comp == 0)
                            val += cv * (c11 * s.lw[2] + c10 * s.hw[2] - c01 * s.lw[2] - c00 * s.hw[2]);
                        else
                            val += cv * (c01 * s.hw[1] + c11 * s.lw[1] - c00 * s.hw[1] - c10 * s.lw[1]);
                    } else {
                        const T c000 = plane[lin(g, s.lo[0], s.lo[1], s.lo[2])];
                        const T c001 = plane[lin(g, s.lo[0], s.lo[1], s.hi[2])];
                        const T c010 = plane[lin(g, s.lo[0], s.hi[1], s.lo[2])];
                        const T c011 = plane[lin(g, s.lo[0], s.hi[1], s.hi[2])];
                        const T c100 = plane[lin(g, s.hi[0], s.lo[1], s.lo[2])];
                        const T c101 = plane[lin(g, s.hi[0], s.lo[1], s.hi[2])];
                        const T c110 = plane[lin(g, s.hi[0], s.hi[1], s.lo[2])];
                        const T c111 = plane[lin(g, s.hi[0], s.hi[1], s.hi[2])];
                        const T lwW = s.lw[2], hwW = s.hw[2], lwH = s.lw[1], hwH = s.hw[1];
                        const T lwL = s.lw[0], hwL = s.hw[0];
                        if (comp == 0)
                            val += cv * (c100 * hwH * hwW + c101 * hwH * lwW + c110 * lwH * hwW + c111 * lwH * lwW
                                         - c000 * hwH * hwW - c001 * hwH * lwW - c010 * lwH * hwW - c011 * lwH * lwW);
                        else if (comp == 1)
                            val += cv * (c010 * hwL * hwW + c011 * hwL * lwW + c110 * lwL * hwW + c111 * lwL * lwW
                                         - c000 * hwL * hwW - c001 * hwL * lwW - c100 * lwL * hwW - c101 * lwL * lwW);
                        else
                            val += cv * (c001 * hwH * hwL + c101 * hwH * lwL + c011 * lwH * hwL + c111 * lwH * lwL
                                         - c000 * hwH * hwL - c100 * hwH * lwL - c010 * lwH * hwL - c110 * lwH * lwL);
                    }
                } else if (nd == 3 && oob_ref) {
                    const T pd = s.p[ax];
                    const T mag = cv > (T)0 ? cv : -cv;
                    if (pd <= (T)-1) val += -mag;
                    else if (pd >= (T)g.in[0]) val += mag;
                }
            }
            doff_n[(size_t)row * ov + pos] = val;
        }
    }
}

// Plain im2col / col2im (integer taps, zero padding); dilation-aware.
template <typename T>
void plain_im2col(const Geo& g, const T* x_n, T* col) {
    const int ov = g.ov(), kv = g.kv(), iv = g.iv();
#pragma omp parallel for schedule(static)
    for (int row = 0; row < g.C * kv; ++row) {
        const int c = row / kv, tap = row % kv;
        int t[3]; unravel_tap(g, tap, t);
        const T* plane = x_n + (size_t)c * iv;
        for (int pos = 0; pos < ov; ++pos) {
            int o[3]; unravel_out(g, pos, o);
            int q[3]; bool ok = true;
            for (int d = 0; d < 3; ++d) {
                q[d] = o[d] * g.stride[d] - g.pad[d] + t[d] * g.dil[d];
                if (!(q[d] > -1 && q[d] < g.in[d])) ok = false;
            }
            col[(size_t)row * ov + pos] = ok ? plane[lin(g, q[0], q[1], q[2])] : (T)0;
        }
    }
}

template <typename T>
void plain_col2im(const Geo& g, const T* col, T* dx_n) {
    const int ov = g.ov(), kv = g.kv(), iv = g.iv();
#pragma omp parallel for schedule(static)
    for (int c = 0; c < g.C; ++c) {
        T* plane = dx_n + (size_t)c * iv;
        for (int pos = 0; pos < ov; ++pos) {
            int o[3]; unravel_out(g, pos, o);
            for (int tap = 0; tap < kv; ++tap) {
                int t[3]; unravel_tap(g, tap, t);
                int q[3]; bool ok = true;
                for (int d = 0; d < 3; ++d) {
                    q[d] = o[d] * g.stride[d] - g.pad[d] + t[d] * g.dil[d];
                    if (!(q[d] > -1 && q[d] < g.in[d])) ok = false;
                }
                if (ok) plane[lin(g, q[0], q[1], q[2])] += col[(size_t)(c * kv + tap) * ov + pos];
            }
        }
    }
}

// Debug dump used by the bit-exactness tests: for every (grp, tap, pos) the coordinate bits,
// validity and the low / high corner index per axis.
template <typename T>
void dump_points(const Geo& g, const T* off_n, T* p_out, int32_t* valid_out, int32_t* lo_out,
                 int32_t* hi_out) {
    const int ov = g.ov(), kv = g.kv();
    const int nd = g.ndim, d0 = 3 - nd;
    const int dg = g.C / g.cpg;
    for (int grp = 0; grp < dg; ++grp)
        for (int tap = 0; tap < kv; ++tap) {
            int t[3]; unravel_tap(g, tap, t);
            for (int pos = 0; pos < ov; ++pos) {
                int o[3]; unravel_out(g, pos, o);
                const Pt<T> s = locate<T>(g, off_n, grp, tap, o, t);
                const size_t e = ((size_t)(grp * kv + tap)) * ov + pos;
                valid_out[e] = s.valid ? 1 : 0;
                for (int d = d0; d < 3; ++d) {
                    p_out[e * nd + (d - d0)] = s.p[d];
                    lo_out[e * nd + (d - d0)] = s.valid ? s.lo[d] : -1;
                    hi_out[e * nd + (d - d0)] = s.valid ? s.hi[d] : -1;
                }
            }
        }
}

}  // namespace

#define ORC_GEO_ARGS int ndim, int C, const int* in, const int* out, const int* k, const int* pad, \
                     const int* stride, const int* dil, int cpg
#define ORC_GEO make_geo(ndim, C, in, out, k, pad, stride, dil, cpg)

extern "C" {

void orc_deform_im2col_f32(ORC_GEO_ARGS, const float* x_n, const float* off_n, float* col) {
    deform_im2col<float>(ORC_GEO, x_n, off_n, col);
}
void orc_deform_im2col_f64(ORC_GEO_ARGS, const double* x_n, const double* off_n, double* col) {
    deform_im2col<double>(ORC_GEO, x_n, off_n, col);
}
void orc_deform_col2im_input_f32(ORC_GEO_ARGS, const float* col, const float* off_n, float* dx_n) {
    deform_col2im_input<float>(ORC_GEO, col, off_n, dx_n);
}
void orc_deform_col2im_input_f64(ORC_GEO_ARGS, const double* col, const double* off_n, double* dx_n) {
    deform_col2im_input<double>(ORC_GEO, col, off_n, dx_n);
}
void orc_deform_col2im_offset_f32(ORC_GEO_ARGS, const float* col, const float* x_n, const float* off_n,
                                  int oob_ref, float* doff_n) {
    deform_col2im_offset<float>(ORC_GEO, col, x_n, off_n, oob_ref, doff_n);
}
void orc_deform_col2im_offset_f64(ORC_GEO_ARGS, const double* col, const double* x_n, const double* off_n,
                                  int oob_ref, double* doff_n) {
    deform_col2im_offset<double>(ORC_GEO, col, x_n, off_n, oob_ref, doff_n);
}
void orc_im2col_f32(ORC_GEO_ARGS, const float* x_n, float* col) { plain_im2col<float>(ORC_GEO, x_n, col); }
void orc_im2col_f64(ORC_GEO_ARGS, const double* x_n, double* col) { plain_im2col<double>(ORC_GEO, x_n, col); }
void orc_col2im_f32(ORC_GEO_ARGS, const float* col, float* dx_n) { plain_col2im<float>(ORC_GEO, col, dx_n); }
void orc_col2im_f64(ORC_GEO_ARGS, const double* col, double* dx_n) { plain_col2im<double>(ORC_GEO, col, dx_n); }
void orc_dump_points_f32(ORC_GEO_ARGS, const float* off_n, float* p, int32_t* valid, int32_t* lo, int32_t* hi) {
    dump_points<float>(ORC_GEO, off_n, p, valid, lo, hi);
}
void orc_dump_points_f64(ORC_GEO_ARGS, const double* off_n, double* p, int32_t* valid, int32_t* lo, int32_t* hi) {
    dump_points<double>(ORC_GEO, off_n, p, valid, lo, hi);
}
int orc_abi_version(void) { return 1; }

}  // extern "C"
