// Exact fp32 kernels for problems so small that latency, not throughput, is what they cost (included by
// dcn_simt.cu inside its anonymous namespace).  A problem like N=2, 16->32 channels, 32x32 (57 MFLOP per step) has
// a roofline time below one kernel launch; the tiled kernels spend ~25 us on it because a few CTAs walk the K loop
// with a dependent offset -> corner -> FMA chain per chunk.  Here a CTA takes kSmallTP output positions of one
// convolution group and does each phase once for all of K, every phase spread over all 1024 threads:
//   forward    weights of the group -> shared; sampling points; sampled patch [TP][Kg] -> shared; y = W * patch
//   backward   (one launch for dX, dOffset and dW)  weights, dy tile, points -> shared;
//              col = W^T dy per (position, k), consumed at once by the input-gradient scatter, the
//              offset-gradient sum (shared-memory accumulators) and the recomputed patch; dW += dy * patch^T
// Same arithmetic rules as the tiled kernels: locate / finish_point, interp, corner_weights, interp_grad, oob_term.
#pragma once

constexpr int kSmallThreads = 1024;      // one CTA per SM, eight warps per scheduler: the phases are latency chains

struct SmallDims {
    int TP;          // output positions per CTA
    int ndg;         // deformable groups a convolution group's channels touch
    int smem_fwd, smem_bwd;
};

// deformable groups overlapping the channels [j*Cg, (j+1)*Cg): first index and count
__host__ __device__ inline void small_dg_range(const Geom& g, int j, int& grp0, int& n) {
    grp0 = (j * g.Cg) / g.cpg;
    n = ((j + 1) * g.Cg - 1) / g.cpg - grp0 + 1;
}

inline SmallDims small_dims(const Geom& g, int D) {
    SmallDims d;
    d.ndg = 1;
    for (int j = 0; j < g.G; ++j) {
        int g0, n;
        small_dg_range(g, j, g0, n);
        if (n > d.ndg) d.ndg = n;
    }
    d.TP = 16;
    auto fwd = [&](int tp) { return 4 * (g.Og * g.Kg + tp * (g.Kg + 1) + tp * g.kv * d.ndg * (D + 1)); };
    auto bwd = [&](int tp) {
        return 4 * (g.Og * g.Kg + g.Og * tp + tp * (g.Kg + 1) + tp * g.kv * d.ndg * (D + 1) + tp * g.kv * d.ndg * D);
    };
    // within shared memory, and enough CTAs to reach most SMs where the problem has the positions for it
    while (d.TP > 4 && (bwd(d.TP) > 96 * 1024 || (g.P + d.TP - 1) / d.TP * g.G < 96)) d.TP /= 2;
    d.smem_fwd = fwd(d.TP);
    d.smem_bwd = bwd(d.TP);
    return d;
}

// One sampling point per (position of the tile, tap, deformable group of the conv group): its D coordinates
// and a validity word, positions fastest so that the offset loads coalesce.
template <int D>
__device__ __forceinline__ void small_points(const Geom& g, const float* __restrict__ off, int j, int TP, int ndg,
                                             long long P0, float* __restrict__ pts) {
    int grp0, n_;
    small_dg_range(g, j, grp0, n_);
    for (int e = threadIdx.x; e < TP * g.kv * ndg; e += kSmallThreads) {
        const int pl = e % TP, r = e / TP, tap = r % g.kv, gl = r / g.kv;
        float* dst = pts + (size_t)e * (D + 1);
        const long long P = P0 + pl;
        bool ok = false;
        if (P < g.P && gl < n_) {
            const OutPos op = decompose_pos(g, P);
            Pt<float, D> s;
            locate<float, D>(g, offset_block<float, D>(g, off, op.n), grp0 + gl, tap, op, s);
#pragma unroll
            for (int a = 0; a < D; ++a) dst[a] = s.p[a];
            ok = true;
        }
        dst[D] = ok ? 1.f : 0.f;
    }
}

// The point of entry e as the tiled kernels would have located it (same finish_point).
template <int D>
__device__ __forceinline__ bool small_load_point(const Geom& g, const float* __restrict__ pts, int e, Pt<float, D>& s) {
    const float* src = pts + (size_t)e * (D + 1);
    if (src[D] == 0.f) { s.valid = false; return false; }
#pragma unroll
    for (int a = 0; a < D; ++a) s.p[a] = src[a];
    finish_point<float, D>(g, s);
    return true;                                         // the position exists (the point may still be invalid)
}

template <int D>
__global__ void __launch_bounds__(kSmallThreads)
small_forward_kernel(const Geom g, const float* __restrict__ x, const float* __restrict__ off,
                     const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ y,
                     const int TP, const int ndg) {
    extern __shared__ float sm_small[];
    float* Ws = sm_small;                                 // [Og][Kg]
    float* smp = Ws + g.Og * g.Kg;                        // [TP][Kg + 1]
    float* pts = smp + TP * (g.Kg + 1);                   // [ndg][kv][TP][D + 1]
    const int j = blockIdx.y;
    const long long P0 = (long long)blockIdx.x * TP;
    int grp0, n_;
    small_dg_range(g, j, grp0, n_);
    for (int i = threadIdx.x; i < g.Og * g.Kg; i += kSmallThreads) Ws[i] = __ldg(w + (size_t)j * g.Og * g.Kg + i);
    small_points<D>(g, off, j, TP, ndg, P0, pts);
    __syncthreads();
    // (unrolled so that the corner loads of several items are in flight together: the phase is one round of
    // global-memory latency, not one per item)
#pragma unroll 4
    for (int it = threadIdx.x; it < TP * g.Kg; it += kSmallThreads) {
        const int pl = it % TP, k = it / TP;
        uint32_t cl, tap;
        g.d_kv.divmod((uint32_t)k, cl, tap);
        const int c = j * g.Cg + (int)cl;
        const int gl = (int)g.d_cpg.div((uint32_t)c) - grp0;
        Pt<float, D> s;
        float val = 0.f;
        if (small_load_point<D>(g, pts, (gl * g.kv + (int)tap) * TP + pl, s) && s.valid) {
            uint32_t n = g.d_ov.div((uint32_t)(P0 + pl));
            const float* plane = x + ((size_t)n * g.C + c) * g.iv;
            int idx[1 << D];
            corner_indices<float, D>(g, s, idx);
            float cv[1 << D];
#pragma unroll
            for (int i = 0; i < (1 << D); ++i) cv[i] = __ldg(plane + idx[i]);
            val = interp<float, D>(s, cv);
        }
        smp[pl * (g.Kg + 1) + k] = val;
    }
    __syncthreads();
    // y = W * patch: S adjacent lanes share one output and split K among them (S a power of two that divides 32)
    const int outs = TP * g.Og;
    int S = 1;
    while (S < 8 && outs * (S * 2) <= kSmallThreads) S *= 2;
    for (int base = 0; base < outs * S; base += kSmallThreads) {
        const int t = base + (int)threadIdx.x;
        const int it = t / S, sub = t % S;
        const bool live = it < outs;
        const int pl = live ? it % TP : 0, ol = live ? it / TP : 0;
        const float* wr = Ws + ol * g.Kg;
        const float* sr = smp + pl * (g.Kg + 1);
        float a2[2] = {0.f, 0.f};
        int k = sub;
        for (; k + S < g.Kg; k += 2 * S) {
            a2[0] = fmaf(wr[k], sr[k], a2[0]);
            a2[1] = fmaf(wr[k + S], sr[k + S], a2[1]);
        }
        if (k < g.Kg) a2[0] = fmaf(wr[k], sr[k], a2[0]);
        float acc = a2[0] + a2[1];
        for (int m = S / 2; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
        const long long P = P0 + pl;
        if (!live || sub != 0 || P >= g.P) continue;
        uint32_t n, opos;
        g.d_ov.divmod((uint32_t)P, n, opos);
        const int o = j * g.Og + ol;
        y[((size_t)n * g.O + o) * g.ov + opos] = acc + (bias != nullptr ? __ldg(bias + o) : 0.f);
    }
}

// ---------------------------------------------------------------------------------------------------
// Fused layer forward for small problems: the offsets are computed INSIDE the kernel, from the plain (integer-tap,
// dilation 1) patch of the CTA's positions and the offset-producing convolution's weights, and stay in shared
// memory for the sampling that follows; they are also written out once, because the backward pass reads them.
// gq: geometry of the offset-producing convolution (one group, dg*kv*D output channels, dilation 1).
// Extra shared memory behind the forward kernel's: plain patch [TP][C*kv], offsets [ndg][kv][D][TP], the rows of the
// offset weights of this CTA's deformable groups.
// ---------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kSmallThreads)
small_layer_forward_kernel(const Geom g, const Geom gq, const float* __restrict__ x, const float* __restrict__ w_off,
                           const float* __restrict__ b_off, const float* __restrict__ w,
                           const float* __restrict__ bias, float* __restrict__ offsets, float* __restrict__ y,
                           const int TP, const int ndg) {
    extern __shared__ float sm_small[];
    float* Ws = sm_small;                                 // [Og][Kg]
    float* smp = Ws + g.Og * g.Kg;                        // [TP][Kg + 1]
    float* pts = smp + TP * (g.Kg + 1);                   // [ndg][kv][TP][D + 1]
    float* pp = pts + TP * g.kv * ndg * (D + 1);          // [TP][Kq + 1] plain patch of all C channels
    float* offs = pp + TP * (gq.Kg + 1);                  // [ndg][kv][D][TP]
    float* Wq = offs + ndg * g.kv * D * TP;               // [ndg * kv * D][Kq] rows of the offset weights this CTA needs
    const int j = blockIdx.y;
    const long long P0 = (long long)blockIdx.x * TP;
    const int Kq = gq.Kg;                                 // C * kv
    int grp0, n_;
    small_dg_range(g, j, grp0, n_);
    for (int i = threadIdx.x; i < g.Og * g.Kg; i += kSmallThreads) Ws[i] = __ldg(w + (size_t)j * g.Og * g.Kg + i);
    // the offset channels of this CTA's deformable groups are consecutive rows of the offset weights
    for (int i = threadIdx.x; i < n_ * g.kv * D * Kq; i += kSmallThreads)
        Wq[i] = __ldg(w_off + (size_t)grp0 * g.kv * D * Kq + i);
    // plain patch: x at the integer taps of the offset-producing convolution
    for (int it = threadIdx.x; it < TP * Kq; it += kSmallThreads) {
        const int pl = it % TP, k = it / TP;
        const long long P = P0 + pl;
        float v = 0.f;
        if (P < g.P) {
            uint32_t c, tap;
            g.d_kv.divmod((uint32_t)k, c, tap);
            const OutPos op = decompose_pos(gq, P);
            int idx;
            if (locate_plain<D>(gq, (int)tap, op, idx)) v = __ldg(x + ((size_t)op.n * g.C + c) * g.iv + idx);
        }
        pp[pl * (Kq + 1) + k] = v;
    }
    __syncthreads();
    // offsets of the deformable groups this convolution group touches: one warp per (offset channel, position) pair,
    // lanes over the contraction index
    {
        const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
        const int per_grp = g.kv * D;
        for (int item = warp; item < n_ * per_grp * TP; item += kSmallThreads / 32) {
            const int pl = item % TP, r = item / TP;            // r = gl * kv * D + tap * D + a
            const int oc = grp0 * per_grp + r;                  // offset channel ((grp * kv + tap) * D + a)
            const float* wr = Wq + (size_t)r * Kq;
            const float* pr = pp + pl * (Kq + 1);
            float acc = 0.f;
            for (int k = lane; k < Kq; k += 32) acc = fmaf(wr[k], pr[k], acc);
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
            if (lane == 0) {
                const float v = acc + (b_off != nullptr ? __ldg(b_off + oc) : 0.f);
                offs[r * TP + pl] = v;
                const long long P = P0 + pl;
                if (P < g.P && offsets != nullptr) {
                    uint32_t n, opos;
                    g.d_ov.divmod((uint32_t)P, n, opos);
                    offsets[((size_t)n * gq.O + oc) * g.ov + opos] = v;
                }
            }
        }
    }
    __syncthreads();
    // sampling points from the offsets in shared memory (same rule: locate_with)
    for (int e = threadIdx.x; e < TP * g.kv * ndg; e += kSmallThreads) {
        const int pl = e % TP, r = e / TP, tap = r % g.kv, gl = r / g.kv;
        float* dst = pts + (size_t)e * (D + 1);
        const long long P = P0 + pl;
        bool ok = false;
        if (P < g.P && gl < n_) {
            const OutPos op = decompose_pos(g, P);
            float offv[D];
#pragma unroll
            for (int a = 0; a < D; ++a) offv[a] = offs[((gl * g.kv + tap) * D + a) * TP + pl];
            Pt<float, D> s;
            locate_with<float, D>(g, offv, tap, op, s);
#pragma unroll
            for (int a = 0; a < D; ++a) dst[a] = s.p[a];
            ok = true;
        }
        dst[D] = ok ? 1.f : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int it = threadIdx.x; it < TP * g.Kg; it += kSmallThreads) {
        const int pl = it % TP, k = it / TP;
        uint32_t cl, tap;
        g.d_kv.divmod((uint32_t)k, cl, tap);
        const int c = j * g.Cg + (int)cl;
        const int gl = (int)g.d_cpg.div((uint32_t)c) - grp0;
        Pt<float, D> s;
        float val = 0.f;
        if (small_load_point<D>(g, pts, (gl * g.kv + (int)tap) * TP + pl, s) && s.valid) {
            uint32_t n = g.d_ov.div((uint32_t)(P0 + pl));
            const float* plane = x + ((size_t)n * g.C + c) * g.iv;
            int idx[1 << D];
            corner_indices<float, D>(g, s, idx);
            float cv[1 << D];
#pragma unroll
            for (int i = 0; i < (1 << D); ++i) cv[i] = __ldg(plane + idx[i]);
            val = interp<float, D>(s, cv);
        }
        smp[pl * (g.Kg + 1) + k] = val;
    }
    __syncthreads();
    const int outs = TP * g.Og;
    int S = 1;
    while (S < 8 && outs * (S * 2) <= kSmallThreads) S *= 2;
    for (int base = 0; base < outs * S; base += kSmallThreads) {
        const int t = base + (int)threadIdx.x;
        const int it = t / S, sub = t % S;
        const bool live = it < outs;
        const int pl = live ? it % TP : 0, ol = live ? it / TP : 0;
        const float* wr = Ws + ol * g.Kg;
        const float* sr = smp + pl * (g.Kg + 1);
        float a2[2] = {0.f, 0.f};
        int k = sub;
        for (; k + S < g.Kg; k += 2 * S) {
            a2[0] = fmaf(wr[k], sr[k], a2[0]);
            a2[1] = fmaf(wr[k + S], sr[k + S], a2[1]);
        }
        if (k < g.Kg) a2[0] = fmaf(wr[k], sr[k], a2[0]);
        float acc = a2[0] + a2[1];
        for (int m = S / 2; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
        const long long P = P0 + pl;
        if (!live || sub != 0 || P >= g.P) continue;
        uint32_t n, opos;
        g.d_ov.divmod((uint32_t)P, n, opos);
        const int o = j * g.Og + ol;
        y[((size_t)n * g.O + o) * g.ov + opos] = acc + (bias != nullptr ? __ldg(bias + o) : 0.f);
    }
}

inline bool small_supported(const Geom& g, int dtype, int ndim, int deform);

inline size_t small_layer_smem(const Geom& g, const Geom& gq, int D) {
    const SmallDims d = small_dims(g, D);
    return (size_t)d.smem_fwd + 4 * ((size_t)d.TP * (gq.Kg + 1) + (size_t)d.ndg * g.kv * D * d.TP +
                                     (size_t)d.ndg * g.kv * D * gq.Kg);
}

// the fused layer forward: a small problem whose plain patch also fits, with the same output positions for both
// convolutions (which dcn_offset_conv_problem guarantees)
inline bool small_layer_supported(const Geom& g, const Geom& gq, int dtype, int ndim) {
    if (!small_supported(g, dtype, ndim, 1)) return false;
    if ((double)g.P * gq.Kg * gq.O > 16777216.0) return false;
    const SmallDims d = small_dims(g, ndim);
    const size_t bwd = (size_t)d.smem_bwd + 4 * ((size_t)d.TP * (gq.Kg + 1) + (size_t)d.ndg * g.kv * ndim * gq.Kg);
    return small_layer_smem(g, gq, ndim) <= 96 * 1024 && bwd <= 96 * 1024 && gq.ov == g.ov && gq.P == g.P;
}

template <int D>
int launch_small_layer_forward(const Geom& g, const Geom& gq, const float* x, const float* w_off, const float* b_off,
                               const float* w, const float* bias, float* offsets, float* y, cudaStream_t st) {
    const SmallDims d = small_dims(g, D);
    const int smem = (int)small_layer_smem(g, gq, D);
    auto kern = small_layer_forward_kernel<D>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return -5;
    dim3 grid((unsigned)((g.P + d.TP - 1) / d.TP), (unsigned)g.G);
    kern<<<grid, kSmallThreads, smem, st>>>(g, gq, x, w_off, b_off, w, bias, offsets, y, d.TP, d.ndg);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// dx and dw must be zero-filled by the launch before this one (see launch_small_backward); doff is written with
// plain stores when DOFF_PLAIN (one conv group: a CTA then holds every channel of the deformable groups it touches),
// else added to a zero-filled doff.
// LAYER: the backward pass of the whole layer (offset-producing convolution + deformable convolution) in this one
// launch.  The offset gradient then is no output: it stays in the shared-memory accumulators and is pushed through
// the offset-producing convolution here -- its bias and weight gradients from the plain patch of the CTA's positions,
// its input gradient added to dx at the integer taps.  `lay` carries that convolution (gq: its geometry).
struct SmallLayer {
    const float* w_off;      // [dg*kv*D][C*kv]
    float* dw_off;           // zero-filled before this launch; may be null
    float* db_off;           // zero-filled before this launch; may be null
};

template <int D, bool DOFF_PLAIN, bool LAYER>
__global__ void __launch_bounds__(kSmallThreads)
small_backward_kernel(const Geom g, const float* __restrict__ x, const float* __restrict__ off,
                      const float* __restrict__ w, const float* __restrict__ dy, float* __restrict__ dx,
                      float* __restrict__ doff, float* __restrict__ dw, const int TP, const int ndg,
                      const Geom gq, const SmallLayer lay) {
    extern __shared__ float sm_small[];
    float* Ws = sm_small;                                 // [Og][Kg]
    float* dys = Ws + g.Og * g.Kg;                        // [Og][TP]
    float* smp = dys + g.Og * TP;                         // [TP][Kg + 1]
    float* pts = smp + TP * (g.Kg + 1);                   // [ndg][kv][TP][D + 1]
    float* dacc = pts + TP * g.kv * ndg * (D + 1);        // [ndg][kv][TP][D]
    float* pp = dacc + TP * g.kv * ndg * D;               // LAYER: [TP][Kq + 1] plain patch, all C channels
    float* Wq = pp + (LAYER ? TP * (gq.Kg + 1) : 0);      // LAYER: [ndg * kv * D][Kq] offset-weight rows of this CTA
    const bool want_doff = LAYER || doff != nullptr;
    const int j = blockIdx.y;
    const long long P0 = (long long)blockIdx.x * TP;
    int grp0, n_;
    small_dg_range(g, j, grp0, n_);
    for (int i = threadIdx.x; i < g.Og * g.Kg; i += kSmallThreads) Ws[i] = __ldg(w + (size_t)j * g.Og * g.Kg + i);
    for (int i = threadIdx.x; i < g.Og * TP; i += kSmallThreads) {
        const int pl = i % TP, ol = i / TP;
        const long long P = P0 + pl;
        float v = 0.f;
        if (P < g.P) {
            uint32_t n, opos;
            g.d_ov.divmod((uint32_t)P, n, opos);
            v = __ldg(dy + ((size_t)n * g.O + j * g.Og + ol) * g.ov + opos);
        }
        dys[ol * TP + pl] = v;
    }
    for (int i = threadIdx.x; i < TP * g.kv * ndg * D; i += kSmallThreads) dacc[i] = 0.f;
    if (LAYER) {
        const int Kq = gq.Kg;
        for (int i = threadIdx.x; i < n_ * g.kv * D * Kq; i += kSmallThreads)
            Wq[i] = __ldg(lay.w_off + (size_t)grp0 * g.kv * D * Kq + i);
        for (int it = threadIdx.x; it < TP * Kq; it += kSmallThreads) {
            const int pl = it % TP, k = it / TP;
            const long long P = P0 + pl;
            float v = 0.f;
            if (P < g.P) {
                uint32_t c, tap;
                g.d_kv.divmod((uint32_t)k, c, tap);
                const OutPos op = decompose_pos(gq, P);
                int idx;
                if (locate_plain<D>(gq, (int)tap, op, idx)) v = __ldg(x + ((size_t)op.n * g.C + c) * g.iv + idx);
            }
            pp[pl * (Kq + 1) + k] = v;
        }
    }
    small_points<D>(g, off, j, TP, ndg, P0, pts);
    __syncthreads();
    // Everything above only reads inputs.  The outputs are zero-filled by the launch before this one, which this
    // kernel may overlap (programmatic dependent launch): wait for it here, before the first addition.
    asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll 2
    for (int it = threadIdx.x; it < TP * g.Kg; it += kSmallThreads) {
        const int pl = it % TP, k = it / TP;
        uint32_t cl, tap;
        g.d_kv.divmod((uint32_t)k, cl, tap);
        const int c = j * g.Cg + (int)cl;
        const int gl = (int)g.d_cpg.div((uint32_t)c) - grp0;
        const int e = (gl * g.kv + (int)tap) * TP + pl;
        Pt<float, D> s;
        float val = 0.f;
        if (small_load_point<D>(g, pts, e, s)) {
            float c4[4] = {0.f, 0.f, 0.f, 0.f};
            int ol = 0;
            for (; ol + 4 <= g.Og; ol += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) c4[u] = fmaf(Ws[(ol + u) * g.Kg + k], dys[(ol + u) * TP + pl], c4[u]);
            }
            for (; ol < g.Og; ++ol) c4[0] = fmaf(Ws[ol * g.Kg + k], dys[ol * TP + pl], c4[0]);
            const float col = (c4[0] + c4[1]) + (c4[2] + c4[3]);
            if (s.valid) {
                const uint32_t n = g.d_ov.div((uint32_t)(P0 + pl));
                const size_t pbase = ((size_t)n * g.C + c) * g.iv;
                int idx[1 << D];
                corner_indices<float, D>(g, s, idx);
                float cv[1 << D];
#pragma unroll
                for (int i = 0; i < (1 << D); ++i) cv[i] = __ldg(x + pbase + idx[i]);
                val = interp<float, D>(s, cv);
                if (dx != nullptr) {
                    float cw[1 << D];
                    corner_weights<float, D>(s, cw);
#pragma unroll
                    for (int i = 0; i < (1 << D); ++i) atomicAdd(dx + pbase + idx[i], cw[i] * col);
                }
                if (want_doff) {
                    float gr[D];
                    interp_grad<float, D>(s, cv, gr);
#pragma unroll
                    for (int a = 0; a < D; ++a) atomicAdd(dacc + (size_t)e * D + a, col * gr[a]);
                }
            } else if (D == 3 && g.oob && want_doff) {
#pragma unroll
                for (int a = 0; a < D; ++a) {
                    const float t = oob_term<float>(g, s.p[a], col);
                    if (t != 0.f) atomicAdd(dacc + (size_t)e * D + a, t);
                }
            }
        }
        smp[pl * (g.Kg + 1) + k] = val;
    }
    __syncthreads();
    if (dw != nullptr) {
        for (int it = threadIdx.x; it < g.Og * g.Kg; it += kSmallThreads) {
            const int k = it % g.Kg, ol = it / g.Kg;
            float a2[2] = {0.f, 0.f};
            for (int pl = 0; pl < TP; pl += 2) {           // TP is even
                a2[0] = fmaf(dys[ol * TP + pl], smp[pl * (g.Kg + 1) + k], a2[0]);
                a2[1] = fmaf(dys[ol * TP + pl + 1], smp[(pl + 1) * (g.Kg + 1) + k], a2[1]);
            }
            const float acc = a2[0] + a2[1];
            if (acc != 0.f) atomicAdd(dw + ((size_t)j * g.Og + ol) * g.Kg + k, acc);
        }
    }
    if (LAYER) {
        // dacc row r = (gl * kv + tap) * D + a at position pl: dacc[((gl * kv + tap) * TP + pl) * D + a]
        const int Kq = gq.Kg, rows = n_ * g.kv * D;
        auto dval = [&](int r, int pl) { return dacc[((r / D) * TP + pl) * D + (r % D)]; };
        if (lay.db_off != nullptr) {
            for (int r = threadIdx.x; r < rows; r += kSmallThreads) {
                float sum = 0.f;
                for (int pl = 0; pl < TP; ++pl) sum += dval(r, pl);
                if (sum != 0.f) atomicAdd(lay.db_off + grp0 * g.kv * D + r, sum);
            }
        }
        if (lay.dw_off != nullptr) {
            for (int it = threadIdx.x; it < rows * Kq; it += kSmallThreads) {
                const int k = it % Kq, r = it / Kq;
                float sum = 0.f;
                for (int pl = 0; pl < TP; ++pl) sum = fmaf(dval(r, pl), pp[pl * (Kq + 1) + k], sum);
                if (sum != 0.f) atomicAdd(lay.dw_off + (size_t)(grp0 * g.kv * D + r) * Kq + k, sum);
            }
        }
        if (dx != nullptr) {
            for (int it = threadIdx.x; it < TP * Kq; it += kSmallThreads) {
                const int pl = it % TP, k = it / TP;
                const long long P = P0 + pl;
                if (P >= g.P) continue;
                uint32_t c, tap;
                g.d_kv.divmod((uint32_t)k, c, tap);
                const OutPos op = decompose_pos(gq, P);
                int idx;
                if (!locate_plain<D>(gq, (int)tap, op, idx)) continue;
                float sum = 0.f;
                for (int r = 0; r < rows; ++r) sum = fmaf(Wq[(size_t)r * Kq + k], dval(r, pl), sum);
                if (sum != 0.f) atomicAdd(dx + ((size_t)op.n * g.C + c) * g.iv + idx, sum);
            }
        }
    }
    if (!LAYER && doff != nullptr) {
        for (int i = threadIdx.x; i < TP * g.kv * ndg * D; i += kSmallThreads) {
            const int a = i % D, e = i / D;
            const int pl = e % TP, r = e / TP, tap = r % g.kv, gl = r / g.kv;
            const long long P = P0 + pl;
            if (P >= g.P || gl >= n_) continue;
            uint32_t n, opos;
            g.d_ov.divmod((uint32_t)P, n, opos);
            float* dst = doff + ((size_t)n * g.dg * g.kv * D + (size_t)((grp0 + gl) * g.kv + tap) * D + a) * g.ov + opos;
            if (DOFF_PLAIN) *dst = dacc[i];
            else if (dacc[i] != 0.f) atomicAdd(dst, dacc[i]);
        }
    }
}

// fp32 deformable problems of at most 2^25 multiply-adds per pass whose group weights fit the shared memory.
inline bool small_supported(const Geom& g, int dtype, int ndim, int deform) {
    if (dtype != 0 || !deform) return false;
    // multiply-adds per pass up to which these kernels are taken (DCN_SMALL_LOG2 overrides the exponent)
    static const double limit = [] {
        const char* e = getenv("DCN_SMALL_LOG2");
        const int lg = e != nullptr ? atoi(e) : 25;     // measured crossover with the tiled kernels: 2^25 .. 2^25.2
        return (double)(1ull << (lg < 0 ? 0 : (lg > 40 ? 40 : lg)));
    }();
    if ((double)g.P * g.Kg * g.Og * g.G > limit) return false;
    const SmallDims d = small_dims(g, ndim);
    return d.smem_bwd <= 96 * 1024 && d.smem_fwd <= 96 * 1024;
}

template <int D>
int launch_small_forward(const Geom& g, const float* x, const float* off, const float* w, const float* bias, float* y,
                         cudaStream_t st) {
    const SmallDims d = small_dims(g, D);
    auto kern = small_forward_kernel<D>;
    if (d.smem_fwd > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, d.smem_fwd) != cudaSuccess) return -5;
    dim3 grid((unsigned)((g.P + d.TP - 1) / d.TP), (unsigned)g.G);
    kern<<<grid, kSmallThreads, d.smem_fwd, st>>>(g, x, off, w, bias, y, d.TP, d.ndg);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Zero fill of up to five output buffers in one launch; lets the dependent launch start at once.
struct ZeroList {
    float4* p[5];
    size_t n4[5];
};
__global__ void __launch_bounds__(256)
small_zero_kernel(const ZeroList z) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int b = 0; b < 5; ++b)
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < z.n4[b]; i += stride) z.p[b][i] = zero;
}

inline bool small_pdl_enabled() {
    static const bool off = [] { const char* e = getenv("DCN_PDL"); return e != nullptr && e[0] == '0'; }();
    return !off;
}

// dX, dW (dOffset with several convolution groups; the offset-producing convolution's gradients in layer mode) are
// zero-filled here: by one kernel when the buffers allow 16-byte stores, and then the main kernel is launched as its
// programmatic dependent, so that its input-only prologue (weights, dy tile, sampling points) runs while the zero
// fill is still in flight.
// lay / gq: null for the operator alone; else the layer's backward pass (doff is then not an output).
template <int D>
int launch_small_backward(const Geom& g, const float* x, const float* off, const float* w, const float* dy, float* dx,
                          float* doff, float* dw, cudaStream_t st, const Geom* gq = nullptr,
                          const SmallLayer* lay = nullptr) {
    const SmallDims d = small_dims(g, D);
    const bool layer = lay != nullptr;
    dim3 grid((unsigned)((g.P + d.TP - 1) / d.TP), (unsigned)g.G);
    float* bufs[5] = {dx, dw, (!layer && g.G > 1) ? doff : nullptr, layer ? lay->dw_off : nullptr,
                      layer ? lay->db_off : nullptr};
    const size_t lens[5] = {(size_t)g.N * g.C * g.iv, (size_t)g.O * g.Cg * g.kv, (size_t)g.N * g.dg * g.kv * D * g.ov,
                            layer ? (size_t)gq->O * gq->Kg : 0, layer ? (size_t)gq->O : 0};
    bool pdl = small_pdl_enabled();
    ZeroList z;
    size_t most = 0;
    for (int b = 0; b < 5; ++b) {
        const size_t n = bufs[b] != nullptr ? lens[b] : 0;
        if (n % 4 != 0 || (reinterpret_cast<uintptr_t>(bufs[b]) & 15) != 0) pdl = false;
        z.p[b] = reinterpret_cast<float4*>(bufs[b]);
        z.n4[b] = n / 4;
        if (n / 4 > most) most = n / 4;
    }
    if (pdl) {
        size_t blocks = (most + 255) / 256;
        if (blocks < 1) blocks = 1;
        if (blocks > 296) blocks = 296;
        small_zero_kernel<<<(unsigned)blocks, 256, 0, st>>>(z);
        if (cudaGetLastError() != cudaSuccess) return -5;
    } else {
        for (int b = 0; b < 5; ++b)
            if (bufs[b] != nullptr && cudaMemsetAsync(bufs[b], 0, lens[b] * sizeof(float), st) != cudaSuccess) return -5;
    }
    size_t smem = (size_t)d.smem_bwd;
    if (layer) smem += 4 * ((size_t)d.TP * (gq->Kg + 1) + (size_t)d.ndg * g.kv * D * gq->Kg);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kSmallThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    const Geom gq_v = layer ? *gq : g;
    const SmallLayer lay_v = layer ? *lay : SmallLayer{nullptr, nullptr, nullptr};
    auto go = [&](auto kern) {
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return cudaErrorInvalidValue;
        return cudaLaunchKernelEx(&cfg, kern, g, x, off, w, dy, dx, doff, dw, d.TP, d.ndg, gq_v, lay_v);
    };
    cudaError_t e;
    if (layer) e = go(small_backward_kernel<D, true, true>);
    else if (g.G == 1) e = go(small_backward_kernel<D, true, false>);
    else e = go(small_backward_kernel<D, false, false>);
    return (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -5;
}
