// Shared device-side geometry and sampling routines of libdcn (sm_100a).
//
// The sampling rule is the reference's (paths relative to the reference project root):
//   coordinate   deform3d/lib/deform_conv3d_cuda_kernel.cu:87-89,117-119   int32 base + offset, one rounding
//   validity     deform3d/lib/deform_conv3d_cuda_kernel.cu:123-124         p > -1 && p < size on every axis
//   corners      deform3d/lib/deform_conv3d_cuda_kernel.cu:21-26           low = trunc(p); high = low on the
//                                                                          edges (p <= 0 or p >= size-1)
//   weights      deform3d/lib/deform_conv3d_cuda_kernel.cu:40-45           lw = p - low, hw = 1 - lw
// The 2-D packages use the same rule on (h, w): deform2d/lib/deform_conv2d_cuda_kernel.cu:17-33,95-100.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dcn {

// Division by a runtime constant through a multiply-high and a shift (n < 2^31).
struct FastDiv {
    uint32_t d, mul, shr;
    __host__ void init(uint32_t div) {
        d = div;
        if (div <= 1) { mul = 0; shr = 0; d = 1; return; }
        uint32_t lg = 0;
        while ((1u << lg) < div) ++lg;          // ceil(log2(div))
        const uint64_t pw = 1ull << (31 + lg);
        mul = (uint32_t)((pw + div - 1) / div);
        shr = lg - 1;
    }
    __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
        return d == 1 ? n : (__umulhi(n, mul) >> shr);
#else
        return d == 1 ? n : (uint32_t)(((uint64_t)n * mul) >> 32) >> shr;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = div(n);
        r = n - q * d;
    }
};

// Problem geometry as the kernels see it.  Axis order is (l, h, w); 2-D problems keep a unit l axis.
struct Geom {
    int N, C, O, G, cpg, dg;
    int in[3], out[3], k[3], stride[3], pad[3], dil[3];
    int iv, ov, kv;      // products of in / out / k
    int Cg, Og, Kg;      // per convolution group: input channels, output channels, Cg*kv
    int oob;             // 3-D: reference pull-back term for invalid samples in the offset gradient
    int cl;              // x, y and their gradients are stored channels-last ([N, spatial, channels])
    long long P;         // N * ov  (flattened output positions)
    FastDiv d_ov, d_ow, d_oh, d_kw, d_kh, d_kv, d_Cg, d_cpg;
};

template <typename T, int D>
struct Pt {
    bool valid;
    T p[D];         // sampling coordinate per active axis ((l,) h, w)
    int lo[D], hi[D];
    T lw[D], hw[D];
};

struct OutPos {          // decomposition of a flattened output position
    int n;               // sample
    int opos;            // position inside the sample's output volume
    int base[3];         // o*stride - pad per axis (int32, as the reference forms it)
};

__device__ __forceinline__ OutPos decompose_pos(const Geom& g, long long P) {
    OutPos r;
    uint32_t n, opos;
    g.d_ov.divmod((uint32_t)P, n, opos);
    r.n = (int)n;
    r.opos = (int)opos;
    uint32_t q, ow, ol, oh;
    g.d_ow.divmod(opos, q, ow);
    g.d_oh.divmod(q, ol, oh);
    r.base[0] = (int)ol * g.stride[0] - g.pad[0];
    r.base[1] = (int)oh * g.stride[1] - g.pad[1];
    r.base[2] = (int)ow * g.stride[2] - g.pad[2];
    return r;
}

__device__ __forceinline__ void decompose_tap(const Geom& g, int tap, int t[3]) {
    uint32_t q, tw, tl, th;
    g.d_kw.divmod((uint32_t)tap, q, tw);
    g.d_kh.divmod(q, tl, th);
    t[0] = (int)tl; t[1] = (int)th; t[2] = (int)tw;
}

// Validity, corners and weights of a point whose coordinates s.p are set (the reference's rule, see the top of
// this file).
template <typename T, int D>
__device__ __forceinline__ void finish_point(const Geom& g, Pt<T, D>& s) {
    bool ok = true;
#pragma unroll
    for (int a = 0; a < D; ++a) {
        const int ax = a + (3 - D);
        ok = ok && (s.p[a] > (T)-1) && (s.p[a] < (T)g.in[ax]);
    }
    s.valid = ok;
    if (ok) {
#pragma unroll
        for (int a = 0; a < D; ++a) {
            const int ax = a + (3 - D);
            const T pd = s.p[a];
            const int lo = (int)pd;                               // cvt.rzi: truncation toward zero
            const int hi = (pd >= (T)(g.in[ax] - 1) || pd <= (T)0) ? lo : lo + 1;
            s.lo[a] = lo;
            s.hi[a] = hi;
            s.lw[a] = pd - (T)lo;
            s.hw[a] = (T)1 - s.lw[a];
        }
    }
}

// Locate one sampling point from its D offset values (axis order (l,) h, w).
template <typename T, int D>
__device__ __forceinline__ void locate_with(const Geom& g, const T (&offv)[D], int tap, const OutPos& op,
                                            Pt<T, D>& s) {
    int t[3];
    decompose_tap(g, tap, t);
#pragma unroll
    for (int a = 0; a < D; ++a) {
        const int ax = a + (3 - D);
        const int ib = op.base[ax] + t[ax] * g.dil[ax];
        s.p[a] = (T)ib + offv[a];                                 // single rounding, no multiply
    }
    finish_point<T, D>(g, s);
}

// Address of the first offset component of (grp, tap) at this output position; components are ov apart.
template <typename T, int D>
__device__ __forceinline__ const T* offset_ptr(const Geom& g, const T* __restrict__ off_n, int grp, int tap,
                                               const OutPos& op) {
    // (grp * kv + tap) * D * ov + opos stays below 2^31 inside one sample (checked on the host)
    return off_n + (uint32_t)((grp * g.kv + tap) * D) * (uint32_t)g.ov + (uint32_t)op.opos;
}

// Offset block [dg*kv*D, ov] of sample n: one unsigned 32 x 32 -> 64-bit product instead of a chain of 64-bit ones.
template <typename T, int D>
__device__ __forceinline__ const T* offset_block(const Geom& g, const T* __restrict__ off, int n) {
    return off + (uint64_t)(uint32_t)n * (uint64_t)(uint32_t)(g.dg * g.kv * D * g.ov);
}

// Locate one sampling point.  off_n points at the sample's offset block [dg*kv*D, ov].
template <typename T, int D>
__device__ __forceinline__ void locate(const Geom& g, const T* __restrict__ off_n, int grp, int tap,
                                       const OutPos& op, Pt<T, D>& s) {
    const T* ob = offset_ptr<T, D>(g, off_n, grp, tap, op);
    T offv[D];
#pragma unroll
    for (int a = 0; a < D; ++a) offv[a] = __ldg(ob + (size_t)a * g.ov);
    locate_with<T, D>(g, offv, tap, op, s);
}

// Integer tap location of the plain convolution (conv2d/lib/conv2d_cuda_kernel.cu:60-67).
template <int D>
__device__ __forceinline__ bool locate_plain(const Geom& g, int tap, const OutPos& op, int& idx) {
    int t[3];
    decompose_tap(g, tap, t);
    bool ok = true;
    int q[3] = {0, 0, 0};
#pragma unroll
    for (int a = 0; a < D; ++a) {
        const int ax = a + (3 - D);
        q[ax] = op.base[ax] + t[ax] * g.dil[ax];
        ok = ok && q[ax] > -1 && q[ax] < g.in[ax];
    }
    idx = (q[0] * g.in[1] + q[1]) * g.in[2] + q[2];
    return ok;
}

// Linear indices of the 2^D corners; bit (D-1-a) of the corner number selects high on axis a,
// so corner numbering is c[l][h][w] with w the fastest bit, like the reference's c000..c111.
template <typename T, int D>
__device__ __forceinline__ void corner_indices(const Geom& g, const Pt<T, D>& s, int idx[1 << D]) {
    if (D == 2) {
        const int r0 = s.lo[0] * g.in[2], r1 = s.hi[0] * g.in[2];
        idx[0] = r0 + s.lo[1]; idx[1] = r0 + s.hi[1];
        idx[2] = r1 + s.lo[1]; idx[3] = r1 + s.hi[1];
    } else {
        const int hw = g.in[1] * g.in[2];
        const int l0 = s.lo[0] * hw, l1 = s.hi[0] * hw;
        const int h0 = s.lo[1] * g.in[2], h1 = s.hi[1] * g.in[2];
        idx[0] = l0 + h0 + s.lo[2]; idx[1] = l0 + h0 + s.hi[2];
        idx[2] = l0 + h1 + s.lo[2]; idx[3] = l0 + h1 + s.hi[2];
        idx[4] = l1 + h0 + s.lo[2]; idx[5] = l1 + h0 + s.hi[2];
        idx[6] = l1 + h1 + s.lo[2]; idx[7] = l1 + h1 + s.hi[2];
    }
}

// Interpolated value in the reference's order: along w, then h, then l.
template <typename T, int D>
__device__ __forceinline__ T interp(const Pt<T, D>& s, const T c[1 << D]) {
    if (D == 2) {
        const T c0 = c[0] * s.hw[1] + c[1] * s.lw[1];
        const T c1 = c[2] * s.hw[1] + c[3] * s.lw[1];
        return c0 * s.hw[0] + c1 * s.lw[0];
    } else {
        const T c00 = c[0] * s.hw[2] + c[1] * s.lw[2];
        const T c01 = c[2] * s.hw[2] + c[3] * s.lw[2];
        const T c10 = c[4] * s.hw[2] + c[5] * s.lw[2];
        const T c11 = c[6] * s.hw[2] + c[7] * s.lw[2];
        const T c0 = c00 * s.hw[1] + c01 * s.lw[1];
        const T c1 = c10 * s.hw[1] + c11 * s.lw[1];
        return c0 * s.hw[0] + c1 * s.lw[0];
    }
}

// Scatter weights per corner: product of the per-axis weights in l*h*w order
// (deform3d/lib/deform_conv3d_cuda_kernel.cu:264-295).
template <typename T, int D>
__device__ __forceinline__ void corner_weights(const Pt<T, D>& s, T w[1 << D]) {
    if (D == 2) {
        w[0] = s.hw[0] * s.hw[1]; w[1] = s.hw[0] * s.lw[1];
        w[2] = s.lw[0] * s.hw[1]; w[3] = s.lw[0] * s.lw[1];
    } else {
        const T a00 = s.hw[0] * s.hw[1], a01 = s.hw[0] * s.lw[1];
        const T a10 = s.lw[0] * s.hw[1], a11 = s.lw[0] * s.lw[1];
        w[0] = a00 * s.hw[2]; w[1] = a00 * s.lw[2];
        w[2] = a01 * s.hw[2]; w[3] = a01 * s.lw[2];
        w[4] = a10 * s.hw[2]; w[5] = a10 * s.lw[2];
        w[6] = a11 * s.hw[2]; w[7] = a11 * s.lw[2];
    }
}

// d(value)/d(p_a) for every active axis (deform3d/lib/deform_conv3d_cuda_kernel.cu:444-465,
// deform2d/lib/deform_conv2d_cuda_kernel.cu:329-339).
template <typename T, int D>
__device__ __forceinline__ void interp_grad(const Pt<T, D>& s, const T c[1 << D], T gr[D]) {
    if (D == 2) {
        gr[0] = c[3] * s.lw[1] + c[2] * s.hw[1] - c[1] * s.lw[1] - c[0] * s.hw[1];
        gr[1] = c[1] * s.hw[0] + c[3] * s.lw[0] - c[0] * s.hw[0] - c[2] * s.lw[0];
    } else {
        const T hL = s.hw[0], lL = s.lw[0], hH = s.hw[1], lH = s.lw[1], hW = s.hw[2], lW = s.lw[2];
        gr[0] = c[4] * hH * hW + c[5] * hH * lW + c[6] * lH * hW + c[7] * lH * lW
              - c[0] * hH * hW - c[1] * hH * lW - c[2] * lH * hW - c[3] * lH * lW;
        gr[1] = c[2] * hL * hW + c[3] * hL * lW + c[6] * lL * hW + c[7] * lL * lW
              - c[0] * hL * hW - c[1] * hL * lW - c[4] * lL * hW - c[5] * lL * lW;
        gr[2] = c[1] * hH * hL + c[5] * hH * lL + c[3] * lH * hL + c[7] * lH * lL
              - c[0] * hH * hL - c[4] * hH * lL - c[2] * lH * hL - c[6] * lH * lL;
    }
}

// The reference's pull-back term for an invalid 3-D sample: -|v| if p_a <= -1, +|v| if p_a >= in[0]
// (the length is used as the threshold on every axis; deform3d/lib/deform_conv3d_cuda_kernel.cu:470-481).
template <typename T>
__device__ __forceinline__ T oob_term(const Geom& g, T pa, T v) {
    const T mag = v > (T)0 ? v : -v;
    if (pa <= (T)-1) return -mag;
    if (pa >= (T)g.in[0]) return mag;
    return (T)0;
}

}  // namespace dcn
