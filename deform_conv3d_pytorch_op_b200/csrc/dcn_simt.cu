// EXACT-precision kernels of libdcn: fused sampling + contraction on the CUDA cores, computing in
// the tensor dtype (fp32 or fp64) directly on the caller's NC(L)HW tensors, no scratch memory.
//
// They replace the reference's im2col -> cuBLAS GEMM -> col2im pipeline
// (deform3d/lib/deform_conv3d_cuda.cpp:90-336 with the kernels of
// deform3d/lib/deform_conv3d_cuda_kernel.cu:62-131, 175-298, 340-485, and the 2-D / plain-conv
// twins) with three tiled kernels that never materialise the column buffer:
//   forward          y[o, P]    = sum_k W[o, k] * sample(k, P)           (+ bias)
//   backward data    col[k, P]  = sum_o W[o, k] * dy[o, P], consumed in registers by the
//                    input-gradient scatter and the offset-gradient reduction
//   backward weight  dW[o, k]  += sum_P dy[o, P] * sample(k, P)          (split over P, fp atomics)
// P runs over the whole batch (N * out volume): the reference's serial per-sample loop is gone.
#include "dcn_internal.h"

#include <stdlib.h>
#include <type_traits>

namespace dcn {

namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ void atomic_add(T* addr, T v) { atomicAdd(addr, v); }

// ---------------------------------------------------------------------------------------------
// Sampled value for GEMM-K index k (reference order: k = c_local * kv + tap) of conv group j.
// ---------------------------------------------------------------------------------------------
template <typename T, int D, bool DEFORM>
__device__ __forceinline__ T sample_value(const Geom& g, const T* __restrict__ x, const T* __restrict__ off,
                                          int j, int k, const OutPos& op) {
    uint32_t cl, tap;
    g.d_kv.divmod((uint32_t)k, cl, tap);
    const int c = j * g.Cg + (int)cl;
    const T* plane = x + ((size_t)op.n * g.C + c) * g.iv;
    if (DEFORM) {
        const int grp = (int)g.d_cpg.div((uint32_t)c);
        Pt<T, D> s;
        locate<T, D>(g, off + (size_t)op.n * g.dg * g.kv * D * g.ov, grp, (int)tap, op, s);
        if (!s.valid) return (T)0;
        int idx[1 << D];
        corner_indices<T, D>(g, s, idx);
        T cv[1 << D];
#pragma unroll
        for (int i = 0; i < (1 << D); ++i) cv[i] = __ldg(plane + idx[i]);
        return interp<T, D>(s, cv);
    } else {
        int idx;
        return locate_plain<D>(g, (int)tap, op, idx) ? __ldg(plane + idx) : (T)0;
    }
}

// ---------------------------------------------------------------------------------------------
// forward
// grid.x: tiles of BN flattened positions; grid.y: G * ceil(Og / BM)
// ---------------------------------------------------------------------------------------------
// BM output channels per CTA: every sampled element is gathered once per BM-row tile, and the gathers (scattered
// 4-byte loads, one L1 tag look-up each) are what bounds this kernel, so wide problems take 256-row tiles.
template <typename T, int D, bool DEFORM, int BM>
__global__ void __launch_bounds__(kThreads)
simt_forward_kernel(const Geom g, const T* __restrict__ x, const T* __restrict__ off, const T* __restrict__ w,
                    const T* __restrict__ bias, T* __restrict__ y) {
    constexpr int BN = 64, BK = 16, TM = BM / 16, TN = 4;
    __shared__ T As[BK][BM + 4];
    __shared__ T Bs[BK][BN + 4];

    const int tid = threadIdx.x;
    const int mt_per_group = (g.Og + BM - 1) / BM;
    const int j = blockIdx.y / mt_per_group;
    const int o0 = (blockIdx.y % mt_per_group) * BM;     // within the group
    const long long P0 = (long long)blockIdx.x * BN;

    const int tx = tid % 16, ty = tid / 16;

    // this thread's sampling column
    const int bn = tid % BN;
    const long long Pb = P0 + bn;
    const bool pb_ok = Pb < g.P;
    OutPos opb = decompose_pos(g, pb_ok ? Pb : 0);

    T acc[TM][TN];
#pragma unroll
    for (int a = 0; a < TM; ++a)
#pragma unroll
        for (int b = 0; b < TN; ++b) acc[a][b] = (T)0;

    const T* wg = w + (size_t)j * g.Og * g.Kg;

    for (int k0 = 0; k0 < g.Kg; k0 += BK) {
        // A: weights  As[kk][m] = W[j*Og + o0 + m][k0 + kk]
#pragma unroll
        for (int i = 0; i < (BM * BK) / kThreads; ++i) {
            const int e = tid + i * kThreads;
            const int kk = e % BK, m = e / BK;
            const int o = o0 + m, k = k0 + kk;
            As[kk][m] = (o < g.Og && k < g.Kg) ? __ldg(wg + (size_t)o * g.Kg + k) : (T)0;
        }
        // B: sampled patch  Bs[kk][n]
#pragma unroll
        for (int i = 0; i < (BN * BK) / kThreads; ++i) {
            const int kk = tid / BN + i * (kThreads / BN);
            const int k = k0 + kk;
            T v = (T)0;
            if (pb_ok && k < g.Kg) v = sample_value<T, D, DEFORM>(g, x, off, j, k, opb);
            Bs[kk][bn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            T a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int i = 0; i < TN; ++i) b[i] = Bs[kk][tx * TN + i];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int q = 0; q < TN; ++q) acc[i][q] += a[i] * b[q];
        }
        __syncthreads();
    }

    // epilogue
#pragma unroll
    for (int q = 0; q < TN; ++q) {
        const long long P = P0 + tx * TN + q;
        if (P >= g.P) continue;
        uint32_t n, opos;
        g.d_ov.divmod((uint32_t)P, n, opos);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int ol = o0 + ty * TM + i;
            if (ol >= g.Og) continue;
            const int o = j * g.Og + ol;
            T v = acc[i][q];
            if (bias != nullptr) v += __ldg(bias + o);
            y[((size_t)n * g.O + o) * g.ov + opos] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// backward data: input gradient (scatter) + offset gradient (reduction over the group's channels)
// Tile rows are ordered (tap, c_local) so that one tile holds many channels of the same tap.
// grid.x: tiles of BN positions; grid.y: G * ceil(Kg / BM)
// ---------------------------------------------------------------------------------------------
template <typename T, int D, bool DEFORM>
__device__ __forceinline__ void
simt_backward_data_body(const uint3 bid, const Geom g, const T* __restrict__ x, const T* __restrict__ off,
                          const T* __restrict__ w, const T* __restrict__ dy, T* __restrict__ dx,
                          T* __restrict__ doff) {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    // main loop: As[BK][BM+4], Bs[BK][BN+4]; epilogue: S[BM][BN+1]
    constexpr int kMain = BK * (BM + 4) + BK * (BN + 4);
    constexpr int kEpi = BM * (BN + 1);
    __shared__ T smem[kMain > kEpi ? kMain : kEpi];
    __shared__ int row_key[BM];
    T (*As)[BM + 4] = reinterpret_cast<T (*)[BM + 4]>(smem);
    T (*Bs)[BN + 4] = reinterpret_cast<T (*)[BN + 4]>(smem + BK * (BM + 4));
    T (*S)[BN + 1] = reinterpret_cast<T (*)[BN + 1]>(smem);

    const int tid = threadIdx.x;
    const int mt_per_group = (g.Kg + BM - 1) / BM;
    const int j = bid.y / mt_per_group;
    const int m0 = (bid.y % mt_per_group) * BM;
    const long long P0 = (long long)bid.x * BN;
    const int tx = tid % 16, ty = tid / 16;

    T acc[TM][TN];
#pragma unroll
    for (int a = 0; a < TM; ++a)
#pragma unroll
        for (int b = 0; b < TN; ++b) acc[a][b] = (T)0;

    const T* wg = w + (size_t)j * g.Og * g.Kg;

    // this thread's dy column in the B load
    const int bn = tid % BN;
    const long long Pb = P0 + bn;
    const bool pb_ok = Pb < g.P;
    uint32_t nb = 0, oposb = 0;
    if (pb_ok) g.d_ov.divmod((uint32_t)Pb, nb, oposb);
    const T* dyb = dy + ((size_t)nb * g.O + (size_t)j * g.Og) * g.ov + oposb;

    // this thread's weight column in the A load: row m = (tap, cl) -> W index cl*kv + tap
    const int am = tid % BM;
    int a_widx = -1;
    if (m0 + am < g.Kg) {
        uint32_t tap, cl;
        g.d_Cg.divmod((uint32_t)(m0 + am), tap, cl);
        a_widx = (int)cl * g.kv + (int)tap;
    }

    for (int o0 = 0; o0 < g.Og; o0 += BK) {
#pragma unroll
        for (int i = 0; i < (BM * BK) / kThreads; ++i) {
            const int kk = tid / BM + i * (kThreads / BM);
            const int o = o0 + kk;
            As[kk][am] = (a_widx >= 0 && o < g.Og) ? __ldg(wg + (size_t)o * g.Kg + a_widx) : (T)0;
        }
#pragma unroll
        for (int i = 0; i < (BN * BK) / kThreads; ++i) {
            const int kk = tid / BN + i * (kThreads / BN);
            const int o = o0 + kk;
            Bs[kk][bn] = (pb_ok && o < g.Og) ? __ldg(dyb + (size_t)o * g.ov) : (T)0;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            T a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int i = 0; i < TN; ++i) b[i] = Bs[kk][tx * TN + i];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int q = 0; q < TN; ++q) acc[i][q] += a[i] * b[q];
        }
        __syncthreads();
    }

    // ---- epilogue: acc[i][q] = col[(tap, cl) = m0 + ty*TM + i, P0 + tx*TN + q] ----
    T gcon[TM][TN][D];   // offset-gradient contributions
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int q = 0; q < TN; ++q)
#pragma unroll
            for (int a = 0; a < D; ++a) gcon[i][q][a] = (T)0;

    // row bookkeeping: tap / channel / deformable group of each of this thread's rows
    int r_tap[TM], r_c[TM], r_grp[TM];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m < g.Kg) {
            uint32_t tap, cl;
            g.d_Cg.divmod((uint32_t)m, tap, cl);
            r_tap[i] = (int)tap;
            r_c[i] = j * g.Cg + (int)cl;
            r_grp[i] = (int)g.d_cpg.div((uint32_t)r_c[i]);
        } else {
            r_tap[i] = -1; r_c[i] = 0; r_grp[i] = 0;
        }
    }
    if (tid < BM) {
        const int m = m0 + tid;
        int key = -1;
        if (m < g.Kg) {
            uint32_t tap, cl;
            g.d_Cg.divmod((uint32_t)m, tap, cl);
            const int c = j * g.Cg + (int)cl;
            key = (int)g.d_cpg.div((uint32_t)c) * g.kv + (int)tap;
        }
        row_key[tid] = key;
    }

#pragma unroll
    for (int q = 0; q < TN; ++q) {
        const long long P = P0 + tx * TN + q;
        if (P >= g.P) continue;
        const OutPos op = decompose_pos(g, P);
        if (DEFORM) {
            const T* off_n = off + (size_t)op.n * g.dg * g.kv * D * g.ov;
            Pt<T, D> s;
            int idx[1 << D];
            T cw[1 << D];
            int have_tap = -2, have_grp = -2;
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                if (r_tap[i] < 0) continue;
                if (r_tap[i] != have_tap || r_grp[i] != have_grp) {
                    locate<T, D>(g, off_n, r_grp[i], r_tap[i], op, s);
                    have_tap = r_tap[i]; have_grp = r_grp[i];
                    if (s.valid) {
                        corner_indices<T, D>(g, s, idx);
                        corner_weights<T, D>(s, cw);
                    }
                }
                const T v = acc[i][q];
                const size_t plane = ((size_t)op.n * g.C + r_c[i]) * g.iv;
                if (s.valid) {
                    if (doff != nullptr) {
                        T cv[1 << D], gr[D];
#pragma unroll
                        for (int e = 0; e < (1 << D); ++e) cv[e] = __ldg(x + plane + idx[e]);
                        interp_grad<T, D>(s, cv, gr);
#pragma unroll
                        for (int a = 0; a < D; ++a) gcon[i][q][a] = v * gr[a];
                    }
                    if (dx != nullptr) {
#pragma unroll
                        for (int e = 0; e < (1 << D); ++e) atomic_add(dx + plane + idx[e], cw[e] * v);
                    }
                } else if (D == 3 && g.oob) {
#pragma unroll
                    for (int a = 0; a < D; ++a) gcon[i][q][a] = oob_term<T>(g, s.p[a], v);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                if (r_tap[i] < 0) continue;
                int idx;
                if (dx != nullptr && locate_plain<D>(g, r_tap[i], op, idx))
                    atomic_add(dx + ((size_t)op.n * g.C + r_c[i]) * g.iv + idx, acc[i][q]);
            }
        }
    }

    if (DEFORM && doff != nullptr) {
        // reduce over the rows of the tile that share (group, tap); one atomic per run
        const int rc = tid % BN;            // column handled in the reduction
        const int seg = tid / BN;           // rows seg*16 .. seg*16+15
        const long long Pr = P0 + rc;
        uint32_t nr = 0, oposr = 0;
        if (Pr < g.P) g.d_ov.divmod((uint32_t)Pr, nr, oposr);
        T* doff_n = doff + (size_t)nr * g.dg * g.kv * D * g.ov + oposr;
#pragma unroll
        for (int a = 0; a < D; ++a) {
            __syncthreads();
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int q = 0; q < TN; ++q) S[ty * TM + i][tx * TN + q] = gcon[i][q][a];
            __syncthreads();
            if (Pr < g.P) {
                constexpr int kRows = BM / (kThreads / BN);
                int key = -1;
                T sum = (T)0;
                for (int r = seg * kRows; r < (seg + 1) * kRows; ++r) {
                    const int kr = row_key[r];
                    if (kr != key) {
                        if (key >= 0) atomic_add(doff_n + ((size_t)key * D + a) * g.ov, sum);
                        key = kr;
                        sum = (T)0;
                    }
                    sum += S[r][rc];
                }
                if (key >= 0) atomic_add(doff_n + ((size_t)key * D + a) * g.ov, sum);
            }
        }
    }
}

template <typename T, int D, bool DEFORM>
__global__ void __launch_bounds__(kThreads)
simt_backward_data_kernel(const Geom g, const T* __restrict__ x, const T* __restrict__ off,
                          const T* __restrict__ w, const T* __restrict__ dy, T* __restrict__ dx,
                          T* __restrict__ doff) {
    simt_backward_data_body<T, D, DEFORM>(blockIdx, g, x, off, w, dy, dx, doff);
}

// ---------------------------------------------------------------------------------------------
// backward weight: dW[o, k] += sum_P dy[o, P] * sample(k, P);  grid.z splits the position range
// grid.x: ceil(Kg / BN) ; grid.y: G * ceil(Og / BM)
// ---------------------------------------------------------------------------------------------
template <typename T, int D, bool DEFORM, int BM = 64>
__device__ __forceinline__ void
simt_backward_weight_body(const uint3 bid, const Geom g, const T* __restrict__ x, const T* __restrict__ off,
                            const T* __restrict__ dy, T* __restrict__ dw, int chunks_per_split) {
    constexpr int BN = 64, BK = 16, TM = BM / 16, TN = 4;
    __shared__ T As[BK][BM + 4];
    __shared__ T Bs[BK][BN + 4];

    const int tid = threadIdx.x;
    const int mt_per_group = (g.Og + BM - 1) / BM;
    const int j = bid.y / mt_per_group;
    const int o0 = (bid.y % mt_per_group) * BM;
    const int k0 = bid.x * BN;
    const int tx = tid % 16, ty = tid / 16;

    T acc[TM][TN];
#pragma unroll
    for (int a = 0; a < TM; ++a)
#pragma unroll
        for (int b = 0; b < TN; ++b) acc[a][b] = (T)0;

    const long long total_chunks = (g.P + BK - 1) / BK;
    long long c_begin = (long long)bid.z * chunks_per_split;
    long long c_end = c_begin + chunks_per_split;
    if (c_end > total_chunks) c_end = total_chunks;

    const int kk = tid % BK;          // this thread's position inside the chunk (both loads)
    const int rr = tid / BK;          // 0..15

    for (long long ch = c_begin; ch < c_end; ++ch) {
        const long long P = ch * BK + kk;
        const bool ok = P < g.P;
        const OutPos op = decompose_pos(g, ok ? P : 0);
        const T* dyp = dy + ((size_t)op.n * g.O + (size_t)j * g.Og) * g.ov + op.opos;
#pragma unroll
        for (int i = 0; i < BM / 16; ++i) {
            const int m = rr + i * 16;
            const int o = o0 + m;
            As[kk][m] = (ok && o < g.Og) ? __ldg(dyp + (size_t)o * g.ov) : (T)0;
        }
#pragma unroll
        for (int i = 0; i < BN / 16; ++i) {
            const int nn = rr + i * 16;
            const int k = k0 + nn;
            T v = (T)0;
            if (ok && k < g.Kg) v = sample_value<T, D, DEFORM>(g, x, off, j, k, op);
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < BK; ++q) {
            T a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[q][ty * TM + i];
#pragma unroll
            for (int i = 0; i < TN; ++i) b[i] = Bs[q][tx * TN + i];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int e = 0; e < TN; ++e) acc[i][e] += a[i] * b[e];
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int ol = o0 + ty * TM + i;
        if (ol >= g.Og) continue;
#pragma unroll
        for (int e = 0; e < TN; ++e) {
            const int k = k0 + tx * TN + e;
            if (k >= g.Kg) continue;
            atomic_add(dw + ((size_t)(j * g.Og + ol)) * g.Kg + k, acc[i][e]);
        }
    }
}

// dbias[o] = sum over n and positions of dy  (deform3d/deform_conv3d_functions/deform_conv3d_function.py:73-74)
// (BM: as in the forward kernel, the sampled elements of a position chunk serve BM output channels)
template <typename T, int D, bool DEFORM, int BM>
__global__ void __launch_bounds__(kThreads)
simt_backward_weight_kernel(const Geom g, const T* __restrict__ x, const T* __restrict__ off,
                            const T* __restrict__ dy, T* __restrict__ dw, int chunks_per_split) {
    simt_backward_weight_body<T, D, DEFORM, BM>(blockIdx, g, x, off, dy, dw, chunks_per_split);
}

// Both backward passes in one launch, for problems so small that the launch itself is what they cost: the first
// gd.x * gd.y blocks are the blocks of the data pass, the others those of the weight pass (fp32: the two bodies'
// static shared memory together stays under 48 KB).
template <int D, bool DEFORM>
__global__ void __launch_bounds__(kThreads)
simt_backward_both_kernel(const Geom g, const float* __restrict__ x, const float* __restrict__ off,
                          const float* __restrict__ w, const float* __restrict__ dy, float* __restrict__ dx,
                          float* __restrict__ doff, float* __restrict__ dw, const uint3 gd, const uint3 gw,
                          int chunks_per_split) {
    const unsigned nd = gd.x * gd.y;
    if (blockIdx.x < nd) {
        simt_backward_data_body<float, D, DEFORM>(make_uint3(blockIdx.x % gd.x, blockIdx.x / gd.x, 0), g, x, off, w, dy,
                                                  dx, doff);
    } else {
        const unsigned r = blockIdx.x - nd;
        simt_backward_weight_body<float, D, DEFORM>(make_uint3(r % gw.x, (r / gw.x) % gw.y, r / (gw.x * gw.y)), g, x, off,
                                                    dy, dw, chunks_per_split);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
bias_grad_kernel(const Geom g, const T* __restrict__ dy, T* __restrict__ dbias) {
    __shared__ T red[kThreads];
    const int o = blockIdx.x;
    T s = (T)0;
    for (int n = 0; n < g.N; ++n) {
        const T* p = dy + ((size_t)n * g.O + o) * g.ov;
        for (int i = threadIdx.x; i < g.ov; i += kThreads) s += p[i];
    }
    red[threadIdx.x] = s;
    __syncthreads();
    for (int st = kThreads / 2; st > 0; st >>= 1) {
        if (threadIdx.x < st) red[threadIdx.x] += red[threadIdx.x + st];
        __syncthreads();
    }
    if (threadIdx.x == 0) dbias[o] = red[0];
}

// Same for a channels-last dy [N * ov positions][O]: a block sums one channel over all positions.
template <typename T>
__global__ void __launch_bounds__(kThreads)
bias_grad_cl_kernel(const Geom g, const T* __restrict__ dy, T* __restrict__ dbias) {
    __shared__ T red[kThreads];
    const int o = blockIdx.x;
    T s = (T)0;
    for (long long P = threadIdx.x; P < g.P; P += kThreads) s += dy[(size_t)P * g.O + o];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int st = kThreads / 2; st > 0; st >>= 1) {
        if (threadIdx.x < st) red[threadIdx.x] += red[threadIdx.x + st];
        __syncthreads();
    }
    if (threadIdx.x == 0) dbias[o] = red[0];
}

template <typename T, int D>
__global__ void debug_points_kernel(const Geom g, const T* __restrict__ off, int n, T* __restrict__ coords,
                                    int32_t* __restrict__ valid, int32_t* __restrict__ lo,
                                    int32_t* __restrict__ hi) {
    const long long total = (long long)g.dg * g.kv * g.ov;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(e % g.ov);
        const int tap = (int)(e / g.ov % g.kv);
        const int grp = (int)(e / g.ov / g.kv);
        const OutPos op = decompose_pos(g, (long long)n * g.ov + pos);
        Pt<T, D> s;
        locate<T, D>(g, off + (size_t)n * g.dg * g.kv * D * g.ov, grp, tap, op, s);
        valid[e] = s.valid ? 1 : 0;
#pragma unroll
        for (int a = 0; a < D; ++a) {
            coords[e * D + a] = s.p[a];
            lo[e * D + a] = s.valid ? s.lo[a] : -1;
            hi[e * D + a] = s.valid ? s.hi[a] : -1;
        }
    }
}

template <typename T, int D, bool DEFORM>
int launch_forward(const Geom& g, const void* x, const void* off, const void* w, const void* bias, void* y,
                   cudaStream_t st) {
    if constexpr (std::is_same<T, float>::value) {
        if (g.Og > 128) {
            dim3 grid((unsigned)((g.P + 63) / 64), (unsigned)(g.G * ((g.Og + 255) / 256)));
            simt_forward_kernel<T, D, DEFORM, 256><<<grid, kThreads, 0, st>>>(g, (const T*)x, (const T*)off, (const T*)w,
                                                                              (const T*)bias, (T*)y);
            return cudaGetLastError() == cudaSuccess ? 0 : -5;
        }
    }
    dim3 grid((unsigned)((g.P + 63) / 64), (unsigned)(g.G * ((g.Og + 127) / 128)));
    simt_forward_kernel<T, D, DEFORM, 128><<<grid, kThreads, 0, st>>>(g, (const T*)x, (const T*)off, (const T*)w,
                                                                      (const T*)bias, (T*)y);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <typename T, int D, bool DEFORM>
int launch_backward_data(const Geom& g, const void* x, const void* off, const void* w, const void* dy, void* dx,
                         void* doff, cudaStream_t st) {
    if (DEFORM && doff != nullptr) {
        const size_t bytes = (size_t)g.N * g.dg * g.kv * D * g.ov * sizeof(T);
        if (cudaMemsetAsync(doff, 0, bytes, st) != cudaSuccess) return -5;
    }
    dim3 grid((unsigned)((g.P + 63) / 64), (unsigned)(g.G * ((g.Kg + 63) / 64)));
    simt_backward_data_kernel<T, D, DEFORM><<<grid, kThreads, 0, st>>>(
        g, (const T*)x, (const T*)off, (const T*)w, (const T*)dy, (T*)dx, (T*)doff);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Work split of the weight pass: (grid, position chunks per split).
inline void weight_grid(const Geom& g, dim3& grid, int& cps, int bm = 64) {
    const long long chunks = (g.P + 15) / 16;
    const long long tiles = (long long)((g.Kg + 63) / 64) * g.G * ((g.Og + bm - 1) / bm);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) sms = 148;
    long long splits = ((long long)sms * 8 + tiles - 1) / tiles;      // ~8 CTAs per SM overall, >= 8 chunks per split
    if (splits > chunks / 8) splits = chunks / 8;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    cps = (int)((chunks + splits - 1) / splits);
    splits = (chunks + cps - 1) / cps;
    grid = dim3((unsigned)((g.Kg + 63) / 64), (unsigned)(g.G * ((g.Og + bm - 1) / bm)), (unsigned)splits);
}

template <typename T, int D, bool DEFORM>
int launch_backward_weight(const Geom& g, const void* x, const void* off, const void* dy, void* dw,
                           cudaStream_t st) {
    dim3 grid;
    int cps;
    if constexpr (std::is_same<T, float>::value) {
        if (g.Og > 64) {
            const int bm = g.Og > 128 ? 256 : 128;
            weight_grid(g, grid, cps, bm);
            if (bm == 256)
                simt_backward_weight_kernel<T, D, DEFORM, 256><<<grid, kThreads, 0, st>>>(g, (const T*)x, (const T*)off,
                                                                                         (const T*)dy, (T*)dw, cps);
            else
                simt_backward_weight_kernel<T, D, DEFORM, 128><<<grid, kThreads, 0, st>>>(g, (const T*)x, (const T*)off,
                                                                                         (const T*)dy, (T*)dw, cps);
            return cudaGetLastError() == cudaSuccess ? 0 : -5;
        }
    }
    weight_grid(g, grid, cps);
    simt_backward_weight_kernel<T, D, DEFORM, 64><<<grid, kThreads, 0, st>>>(g, (const T*)x, (const T*)off,
                                                                             (const T*)dy, (T*)dw, cps);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <int D, bool DEFORM>
int launch_backward_both(const Geom& g, const float* x, const float* off, const float* w, const float* dy, float* dx,
                         float* doff, float* dw, cudaStream_t st) {
    const dim3 gd((unsigned)((g.P + 63) / 64), (unsigned)(g.G * ((g.Kg + 63) / 64)));
    dim3 gw;
    int cps;
    weight_grid(g, gw, cps);
    const unsigned total = gd.x * gd.y + gw.x * gw.y * gw.z;
    simt_backward_both_kernel<D, DEFORM><<<total, kThreads, 0, st>>>(g, x, off, w, dy, dx, doff, dw,
                                                                     make_uint3(gd.x, gd.y, 1), make_uint3(gw.x, gw.y, gw.z), cps);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#include "dcn_simt_small.cuh"

}  // namespace

bool simt_small_supported(const Geom& g, int dtype, int ndim, int deform) { return small_supported(g, dtype, ndim, deform); }

int simt_small_forward(const Geom& g, int ndim, const void* x, const void* off, const void* w, const void* bias,
                       void* y, cudaStream_t st) {
    if (ndim == 2) return launch_small_forward<2>(g, (const float*)x, (const float*)off, (const float*)w, (const float*)bias, (float*)y, st);
    return launch_small_forward<3>(g, (const float*)x, (const float*)off, (const float*)w, (const float*)bias, (float*)y, st);
}

bool simt_small_layer_supported(const Geom& g, const Geom& gq, int dtype, int ndim) {
    return small_layer_supported(g, gq, dtype, ndim);
}

int simt_small_layer_forward(const Geom& g, const Geom& gq, int ndim, const void* x, const void* w_off, const void* b_off,
                             const void* w, const void* bias, void* offsets, void* y, cudaStream_t st) {
    if (ndim == 2) return launch_small_layer_forward<2>(g, gq, (const float*)x, (const float*)w_off, (const float*)b_off, (const float*)w, (const float*)bias, (float*)offsets, (float*)y, st);
    return launch_small_layer_forward<3>(g, gq, (const float*)x, (const float*)w_off, (const float*)b_off, (const float*)w, (const float*)bias, (float*)offsets, (float*)y, st);
}

int simt_small_layer_backward(const Geom& g, const Geom& gq, int ndim, const void* x, const void* offsets,
                              const void* w_off, const void* w, const void* dy, void* dx, void* dw_off, void* db_off,
                              void* dw, cudaStream_t st) {
    const SmallLayer lay{(const float*)w_off, (float*)dw_off, (float*)db_off};
    if (ndim == 2) return launch_small_backward<2>(g, (const float*)x, (const float*)offsets, (const float*)w, (const float*)dy, (float*)dx, nullptr, (float*)dw, st, &gq, &lay);
    return launch_small_backward<3>(g, (const float*)x, (const float*)offsets, (const float*)w, (const float*)dy, (float*)dx, nullptr, (float*)dw, st, &gq, &lay);
}

int simt_small_backward(const Geom& g, int ndim, const void* x, const void* off, const void* w, const void* dy,
                        void* dx, void* doff, void* dw, cudaStream_t st) {
    if (ndim == 2) return launch_small_backward<2>(g, (const float*)x, (const float*)off, (const float*)w, (const float*)dy, (float*)dx, (float*)doff, (float*)dw, st);
    return launch_small_backward<3>(g, (const float*)x, (const float*)off, (const float*)w, (const float*)dy, (float*)dx, (float*)doff, (float*)dw, st);
}

// fp32 problems whose two backward grids together stay small take one launch for both passes (all outputs must be
// wanted and zero-filled by the caller, as for the separate launchers).
bool simt_backward_both_supported(const Geom& g, int dtype) {
    if (dtype != 0) return false;
    const long long nd = ((g.P + 63) / 64) * (long long)g.G * ((g.Kg + 63) / 64);
    return nd <= 4096;
}

int simt_backward_both(const Geom& g, int ndim, int deform, const void* x, const void* off, const void* w,
                       const void* dy, void* dx, void* doff, void* dw, cudaStream_t st) {
    const float *xf = (const float*)x, *of = (const float*)off, *wf = (const float*)w, *dyf = (const float*)dy;
    float *dxf = (float*)dx, *dof = (float*)doff, *dwf = (float*)dw;
    if (deform && doff != nullptr &&
        cudaMemsetAsync(doff, 0, (size_t)g.N * g.dg * g.kv * ndim * g.ov * sizeof(float), st) != cudaSuccess)
        return -5;
    if (ndim == 2) return deform ? launch_backward_both<2, true>(g, xf, of, wf, dyf, dxf, dof, dwf, st)
                                 : launch_backward_both<2, false>(g, xf, of, wf, dyf, dxf, dof, dwf, st);
    return deform ? launch_backward_both<3, true>(g, xf, of, wf, dyf, dxf, dof, dwf, st)
                  : launch_backward_both<3, false>(g, xf, of, wf, dyf, dxf, dof, dwf, st);
}

#define DCN_DISPATCH(FN, ...)                                                                     \
    do {                                                                                          \
        if (dtype == 0) {                                                                         \
            if (ndim == 2) return deform ? FN<float, 2, true>(__VA_ARGS__) : FN<float, 2, false>(__VA_ARGS__);   \
            return deform ? FN<float, 3, true>(__VA_ARGS__) : FN<float, 3, false>(__VA_ARGS__);   \
        } else {                                                                                  \
            if (ndim == 2) return deform ? FN<double, 2, true>(__VA_ARGS__) : FN<double, 2, false>(__VA_ARGS__); \
            return deform ? FN<double, 3, true>(__VA_ARGS__) : FN<double, 3, false>(__VA_ARGS__); \
        }                                                                                         \
    } while (0)

int simt_forward(const Geom& g, int dtype, int ndim, int deform, const void* x, const void* off, const void* w,
                 const void* bias, void* y, cudaStream_t st) {
    DCN_DISPATCH(launch_forward, g, x, off, w, bias, y, st);
}

int simt_backward_data(const Geom& g, int dtype, int ndim, int deform, const void* x, const void* off,
                       const void* w, const void* dy, void* dx, void* doff, cudaStream_t st) {
    DCN_DISPATCH(launch_backward_data, g, x, off, w, dy, dx, doff, st);
}

int simt_backward_weight(const Geom& g, int dtype, int ndim, int deform, const void* x, const void* off,
                         const void* dy, void* dw, cudaStream_t st) {
    DCN_DISPATCH(launch_backward_weight, g, x, off, dy, dw, st);
}

int bias_grad(const Geom& g, int dtype, const void* dy, void* dbias, cudaStream_t st) {
    if (g.cl) bias_grad_cl_kernel<float><<<g.O, kThreads, 0, st>>>(g, (const float*)dy, (float*)dbias);
    else if (dtype == 0) bias_grad_kernel<float><<<g.O, kThreads, 0, st>>>(g, (const float*)dy, (float*)dbias);
    else bias_grad_kernel<double><<<g.O, kThreads, 0, st>>>(g, (const double*)dy, (double*)dbias);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int debug_points(const Geom& g, int dtype, int ndim, const void* off, int n, void* coords, int32_t* valid,
                 int32_t* lo, int32_t* hi, cudaStream_t st) {
    const long long total = (long long)g.dg * g.kv * g.ov;
    const int blocks = (int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
    if (dtype == 0) {
        if (ndim == 2) debug_points_kernel<float, 2><<<blocks, 256, 0, st>>>(g, (const float*)off, n, (float*)coords, valid, lo, hi);
        else debug_points_kernel<float, 3><<<blocks, 256, 0, st>>>(g, (const float*)off, n, (float*)coords, valid, lo, hi);
    } else {
        if (ndim == 2) debug_points_kernel<double, 2><<<blocks, 256, 0, st>>>(g, (const double*)off, n, (double*)coords, valid, lo, hi);
        else debug_points_kernel<double, 3><<<blocks, 256, 0, st>>>(g, (const double*)off, n, (double*)coords, valid, lo, hi);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace dcn
