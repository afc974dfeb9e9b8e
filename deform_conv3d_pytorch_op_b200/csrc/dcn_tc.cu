// BF16 tensor-core path of libdcn (sm_100a): implicit-GEMM kernels on tcgen05 with accumulators in tensor
// memory.  fp32 tensors in and out; sampled patches, weights and output gradients are rounded to bf16 on
// their way into shared memory; coordinates, interpolation weights and accumulation stay fp32.
//
// Replaces, without ever materialising the reference's column buffer:
//   forward          deformable_im2col + SGEMM       (deform3d/lib/deform_conv3d_cuda.cpp:105-149)
//   backward data    SGEMM + col2im_offset + col2im  (deform3d/lib/deform_conv3d_cuda.cpp:186-251)
//   backward weight  deformable_im2col + SGEMM(b=1)  (deform3d/lib/deform_conv3d_cuda.cpp:278-321)
//
// Internal layouts (workspace):
//   x_cl   [N][in volume][C] bf16      channels-last copy of the input: the C/dg channels that share one
//                                      sampling point are contiguous, so one corner fetch is a 16-byte load
//   w_pk   pre-swizzled 128x64 bf16 operand tiles of the weight, GEMM-K ordered (tap, channel)
//   dx_cl  [N][in volume][C] fp32      channels-last input-gradient accumulator (backward data)
//
// Requirements (dcn_precision_supported): fp32 tensors, C/G and C/dg multiples of 8.
#include <stdlib.h>

#include "dcn_internal.h"
#include "dcn_tc_common.cuh"

namespace dcn {

using namespace tc;

namespace {

constexpr int kTileN = 128;            // output positions per tile
constexpr int kTileK = 64;             // bf16 elements per K chunk (one 128-byte swizzled row)
constexpr int kTileBytes = 128 * 128;  // one 128-row operand tile: 16 KB
constexpr int kProducerWarps = 8;
constexpr int kEpilogueWarps = 4;

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct TcDims {
    int KC;         // K chunks per group: ceil(kv*Cg / 64)
    int MT;         // 128-row output-channel tiles per group
    int MB;         // o-blocks per group (each up to 2 m-tiles sharing the sampled operand)
    long long PT;   // position tiles
};

TcDims tc_dims(const Geom& g) {
    TcDims d;
    d.KC = (g.kv * g.Cg + kTileK - 1) / kTileK;
    d.MT = (g.Og + 127) / 128;
    d.MB = (d.MT + 1) / 2;
    d.PT = (g.P + kTileN - 1) / kTileN;
    return d;
}

// ---------------------------------------------------------------------------------------------------
// Pre-pass 1: NC(L)HW fp32 -> N(L)HWC bf16
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
to_channels_last_bf16(const float* __restrict__ x, __nv_bfloat16* __restrict__ xcl, int C, int iv) {
    // tile of 64 channels x 32 positions: 128-byte reads along the positions, 128-byte writes of bf16 pairs along
    // the channels (C is a multiple of 8, so a pair never straddles the end)
    __shared__ float tile[64][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 64;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    const float* xn = x + (size_t)n * C * iv;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = c0 + ty + i * 8, p = p0 + tx;
        tile[ty + i * 8][tx] = (c < C && p < iv) ? __ldg(xn + (size_t)c * iv + p) : 0.f;
    }
    __syncthreads();
    uint32_t* on = reinterpret_cast<uint32_t*>(xcl + (size_t)n * iv * C);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = p0 + ty + i * 8, c = c0 + 2 * tx;
        if (p < iv && c < C) on[((size_t)p * C + c) >> 1] = pack_bf16x2(tile[2 * tx][ty + i * 8], tile[2 * tx + 1][ty + i * 8]);
    }
}

// ---------------------------------------------------------------------------------------------------
// Pre-pass 2: weights.  Step one reorders and rounds the weight once, with coalesced reads and writes:
//   W [O][Cg][kv] fp32  ->  Wt [O][kv * Cg] bf16,  GEMM-K order k' = tap * Cg + c
// (a block takes one output channel and walks its row in pieces of 64 input channels through shared memory;
// reading W directly in k' order would be a stride-kv gather, 8 to 27 times the traffic).  It also raises
// *wmax_bits to the bit pattern of max|W| when asked to.  The operand tiles of the three passes are then cut out
// of Wt, every tile row being a contiguous run of it.
// ---------------------------------------------------------------------------------------------------
constexpr int kWtChunk = 64;       // input channels per shared-memory piece

__global__ void __launch_bounds__(256)
weight_to_kmajor_bf16(const Geom g, const float* __restrict__ w, __nv_bfloat16* __restrict__ wt,
                      unsigned int* __restrict__ wmax_bits) {
    extern __shared__ float wrow[];                                  // [<= 64 channels][kv]
    const int o = blockIdx.x;
    const float* src = w + (size_t)o * g.Cg * g.kv;
    __nv_bfloat16* dst = wt + (size_t)o * g.Kg;
    float mx = 0.f;
    {
        const int c0 = blockIdx.y * kWtChunk;                        // one piece of 64 channels per block
        const int nc = g.Cg - c0 < kWtChunk ? g.Cg - c0 : kWtChunk;
        for (int i = threadIdx.x; i < nc * g.kv; i += blockDim.x) {
            const float v = __ldg(src + (size_t)c0 * g.kv + i);
            wrow[i] = v;
            mx = fmaxf(mx, fabsf(v));
        }
        __syncthreads();
        // pairs of channels of one tap: consecutive threads write consecutive 4-byte words of a tap's row segment
        const int np = nc / 2;                                       // channel counts are multiples of 8
        for (int i = threadIdx.x; i < np * g.kv; i += blockDim.x) {
            const int tap = i / np, cp = i - tap * np;
            const uint32_t v = pack_bf16x2(wrow[(2 * cp) * g.kv + tap], wrow[(2 * cp + 1) * g.kv + tap]);
            *reinterpret_cast<uint32_t*>(dst + (size_t)tap * g.Cg + c0 + 2 * cp) = v;
        }
    }
    if (wmax_bits != nullptr) {
        const unsigned int m = __reduce_max_sync(0xffffffffu, __float_as_uint(mx));
        if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(wmax_bits, m);
    }
}

size_t wt_bytes(const Geom& g) { return align_up((size_t)g.O * g.Kg * 2, 256); }

int launch_weight_to_kmajor(const Geom& g, const float* w, __nv_bfloat16* wt, unsigned int* wmax_bits, cudaStream_t st) {
    const int smem = kWtChunk * g.kv * (int)sizeof(float);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(weight_to_kmajor_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return -5;
    weight_to_kmajor_bf16<<<dim3((unsigned)g.O, (unsigned)((g.Cg + kWtChunk - 1) / kWtChunk)), 256, smem, st>>>(g, w, wt, wmax_bits);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Wt -> swizzled K-major bf16 tiles [G][MT][KC][128 rows x 64 k'] of the forward pass.  Rows >= Og and
// k' >= kv*Cg are zero.  One thread per 16-byte chunk (8 consecutive k').
__global__ void __launch_bounds__(256)
pack_weight_fwd(const Geom g, const __nv_bfloat16* __restrict__ wt, uint8_t* __restrict__ wpk, int MT, int KC) {
    const int tile = blockIdx.x;                  // (j * MT + mt) * KC + kc
    const int kc = tile % KC, mt = (tile / KC) % MT, j = tile / KC / MT;
    uint8_t* dst = wpk + (size_t)tile * kTileBytes;
    for (int e = threadIdx.x; e < 128 * 8; e += blockDim.x) {
        const int row = e / 8, chunk = e % 8;
        const int o = mt * 128 + row;
        const int kp = kc * kTileK + chunk * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (o < g.Og && kp < g.Kg)                // Kg is a multiple of 8: a chunk is inside or outside as a whole
            v = __ldg(reinterpret_cast<const uint4*>(wt + (size_t)(j * g.Og + o) * g.Kg + kp));
        *reinterpret_cast<uint4*>(dst + swz_offset(row, chunk)) = v;
    }
}

// ---------------------------------------------------------------------------------------------------
// Sampling of one 16-byte chunk (8 consecutive channels of one tap, one deformable group) at one output
// position, from the channels-last bf16 input.  Returns 8 bf16 packed in 4 words.
// ---------------------------------------------------------------------------------------------------
template <int D, bool DEFORM>
__device__ __forceinline__ uint4 sample_chunk(const Geom& g, const __nv_bfloat16* __restrict__ xcl,
                                              const float* __restrict__ off, const OutPos& op, int tap, int c,
                                              int grp) {
    const uint32_t pix_bytes = (uint32_t)g.C * 2u;
    const void* xn = ptr_mad_u32(xcl + c, (uint32_t)op.n * (uint32_t)g.iv, pix_bytes);
    if (!DEFORM) {
        int idx;
        if (!locate_plain<D>(g, tap, op, idx)) return make_uint4(0, 0, 0, 0);
        return __ldg(static_cast<const uint4*>(ptr_mad_u32(xn, (uint32_t)idx, pix_bytes)));
    }
    Pt<float, D> s;
    locate<float, D>(g, offset_block<float, D>(g, off, op.n), grp, tap, op, s);
    if (!s.valid) return make_uint4(0, 0, 0, 0);
    int idx[1 << D];
    float cw[1 << D];
    corner_indices<float, D>(g, s, idx);
    corner_weights<float, D>(s, cw);
    uint4 q[1 << D];
#pragma unroll
    for (int e = 0; e < (1 << D); ++e) q[e] = __ldg(static_cast<const uint4*>(ptr_mad_u32(xn, (uint32_t)idx[e], pix_bytes)));
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int e = 0; e < (1 << D); ++e) {
        const uint32_t wd[4] = {q[e].x, q[e].y, q[e].z, q[e].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] = fmaf(cw[e], bf16_lo(wd[i]), acc[2 * i]);
            acc[2 * i + 1] = fmaf(cw[e], bf16_hi(wd[i]), acc[2 * i + 1]);
        }
    }
    return make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                      pack_bf16x2(acc[6], acc[7]));
}

int sm_count() {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
}

#include "dcn_tc_fwd_direct.cuh"
#include "dcn_tc_sampler.cuh"
#include "dcn_tc_fwd.cuh"

struct FwdWorkspace {
    size_t xcl_off, xcl_bytes, wpk_off, wpk_bytes, wt_off, total;
};
FwdWorkspace fwd_workspace(const Geom& g) {
    const TcDims d = tc_dims(g);
    FwdWorkspace w;
    w.xcl_off = 0;
    w.xcl_bytes = align_up((size_t)g.N * g.iv * g.C * 2, 256);
    w.wpk_off = w.xcl_bytes;
    w.wpk_bytes = align_up((size_t)g.G * d.MT * d.KC * kTileBytes, 256);
    w.wt_off = w.wpk_off + w.wpk_bytes;
    w.total = w.wt_off + wt_bytes(g);
    return w;
}

// fp32 -> bf16 of an input that already is channels-last (8 elements per thread; C is a multiple of 8)
__global__ void __launch_bounds__(256)
cast_bf16(const float* __restrict__ x, __nv_bfloat16* __restrict__ xcl, size_t n8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * i);
        const float4 b = __ldg(reinterpret_cast<const float4*>(x) + 2 * i + 1);
        reinterpret_cast<uint4*>(xcl)[i] = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w),
                                                      pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
    }
}

int launch_channels_last(const Geom& g, const float* x, __nv_bfloat16* xcl, cudaStream_t st) {
    if (g.cl) {
        if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return -7;      // vector loads
        const size_t n8 = (size_t)g.N * g.iv * g.C / 8;
        const size_t want = (n8 + 255) / 256;
        const int blocks = (int)(want < (size_t)(8 * sm_count()) ? want : (size_t)(8 * sm_count()));
        cast_bf16<<<blocks, 256, 0, st>>>(x, xcl, n8);
        return cudaGetLastError() == cudaSuccess ? 0 : -5;
    }
    dim3 grid((unsigned)((g.iv + 31) / 32), (unsigned)((g.C + 63) / 64), (unsigned)g.N);
    to_channels_last_bf16<<<grid, 256, 0, st>>>(x, xcl, g.C, g.iv);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#include "dcn_tc_wgrad.cuh"
#include "dcn_tc_wgrad2.cuh"
#include "dcn_tc_dgrad.cuh"
#include "dcn_tc_dgrad2.cuh"
#include "dcn_tc_bwd2d.cuh"

struct BwdWeightWorkspace {
    size_t xcl_off, dpk_off, dwpk_off, total;
};
BwdWeightWorkspace bwd_weight_workspace(const Geom& g) {
    const WgDims d = wg_dims(g);
    BwdWeightWorkspace w;
    w.xcl_off = 0;
    w.dpk_off = align_up((size_t)g.N * g.iv * g.C * 2, 256);
    w.dwpk_off = w.dpk_off + align_up((size_t)g.G * d.MT * d.PC * kTileBytes, 256);
    w.total = w.dwpk_off + align_up(dwpk_bytes(g), 256);
    return w;
}

struct BwdDataWorkspace {
    size_t xcl_off, dpk_off, wpk_off, scale_off, wt_off, dxcl_off, dxcl_bytes, dwpk_off, gath_off, total;   // dwpk: fused backward only; gath: forward workspace of the transposed convolution
};
size_t gather_dgrad_bytes(const Geom& g);      // 0 unless the problem can take the gather form (any ndim)
BwdDataWorkspace bwd_data_workspace(const Geom& g) {
    const DgDims d = dg_dims(g);
    BwdDataWorkspace w;
    w.xcl_off = 0;
    w.dpk_off = align_up((size_t)g.N * g.iv * g.C * 2, 256);
    w.wpk_off = w.dpk_off + align_up((size_t)g.G * d.MT * d.PC2 * kTileBytes, 256);
    size_t wpk_bytes = (size_t)g.G * d.NB * d.OC * 2 * kTileBytes;
    if (g.Cg % 8 == 0 && b2_wpk_bytes(g) > wpk_bytes) wpk_bytes = b2_wpk_bytes(g);   // slab-wise tiles of dcn_tc_bwd2d.cuh
    w.scale_off = w.wpk_off + align_up(wpk_bytes, 256);
    w.wt_off = w.scale_off + 256;                      // two words: bit patterns of max|dy| and max|W|
    w.dxcl_off = w.wt_off + wt_bytes(g);
    w.dxcl_bytes = align_up((size_t)g.N * g.iv * g.C * 4, 256);
    // the shared-memory-accumulating kernel has no channels-last dX scratch; its sampling-point entries live there
    if (g.Cg % 8 == 0 && b2_points_bytes(g) > w.dxcl_bytes) w.dxcl_bytes = align_up(b2_points_bytes(g), 256);
    w.dwpk_off = w.dxcl_off + w.dxcl_bytes;
    w.gath_off = w.dwpk_off + align_up(dwpk_bytes(g), 256);
    w.total = w.gath_off + gather_dgrad_bytes(g);
    return w;
}

// ---------------------------------------------------------------------------------------------------
// Plain convolution, stride 1: the input gradient is itself a plain convolution of dy (taps mirrored, weights
// transposed within each group, padding dil*(k-1) - pad), so it runs on the FORWARD kernel as a gather -- every
// dX element written once, no reductions -- instead of the scatter the deformable operator needs.
// gt: that convolution's geometry (C and O swapped, input and output sizes swapped).
// ---------------------------------------------------------------------------------------------------
bool transposed_geom(const Geom& g, int ndim, Geom& gt) {
    gt = g;
    gt.C = g.O; gt.O = g.C;
    gt.cpg = gt.C; gt.dg = 1; gt.oob = 0;
    gt.iv = g.ov; gt.ov = g.iv;
    for (int d = 0; d < 3; ++d) {
        if (g.stride[d] != 1) return false;
        gt.in[d] = g.out[d]; gt.out[d] = g.in[d];
        gt.pad[d] = g.dil[d] * (g.k[d] - 1) - g.pad[d];
        if (gt.pad[d] < 0) return false;
        if (gt.in[d] + 2 * gt.pad[d] - g.dil[d] * (g.k[d] - 1) != gt.out[d]) return false;
    }
    gt.Cg = g.Og; gt.Og = g.Cg; gt.Kg = gt.Cg * gt.kv;
    gt.P = (long long)gt.N * gt.ov;
    gt.d_ov.init(gt.ov); gt.d_ow.init(gt.out[2]); gt.d_oh.init(gt.out[1]);
    gt.d_Cg.init(gt.Cg); gt.d_cpg.init(gt.cpg);
    (void)ndim;
    return gt.Cg % 8 == 0 && gt.N <= 65535;
}

bool use_gather_dgrad(const Geom& g, int ndim, int deform, Geom& gt) {
    static const bool off = [] { const char* e = getenv("DCN_GATHER_DGRAD"); return e != nullptr && e[0] == '0'; }();
    return !off && !deform && transposed_geom(g, ndim, gt);
}

// Wt'[c][tap' * Og + ol] = W[j*Og + ol][cl][kv - 1 - tap'] (c = j*Cg + cl) as bf16: the k-major weights of the
// transposed convolution, in the layout pack_weight_fwd reads.
__global__ void __launch_bounds__(256)
weight_flip_to_kmajor_bf16(const Geom g, const float* __restrict__ w, __nv_bfloat16* __restrict__ wt) {
    const long long total = (long long)g.C * g.kv * g.Og;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int ol = (int)(i % g.Og);
        const long long r = i / g.Og;
        const int tap = (int)(r % g.kv);
        const int c = (int)(r / g.kv);
        const int j = c / g.Cg, cl = c - j * g.Cg;
        wt[i] = __float2bfloat16_rn(__ldg(w + ((size_t)(j * g.Og + ol) * g.Cg + cl) * g.kv + (g.kv - 1 - tap)));
    }
}

size_t gather_dgrad_bytes(const Geom& g) {
    Geom gt;
    if (g.dg != 1 || g.cpg != g.C) return 0;                     // deformable problems never take it
    if (!transposed_geom(g, 3, gt)) return 0;
    return align_up(fwd_workspace(gt).total, 256);
}

// dX of a plain stride-1 convolution through the forward kernel.  add: dX already holds a partial result (the
// layer's deformable part, or the accumulating entry point): the tiles are added to it with reductions.
// dx_cl: dX is stored channels-last (it may differ from the layout of dy: the layer's dOffset is always channel-first).
int run_gather_dgrad(const Geom& g, const Geom& gt, int ndim, const float* w, const float* dy, float* dx, bool add,
                     bool dx_cl, void* ws, cudaStream_t st) {
    const FwdWorkspace l = fwd_workspace(gt);
    uint8_t* base = static_cast<uint8_t*>(ws);
    __nv_bfloat16* dycl = reinterpret_cast<__nv_bfloat16*>(base + l.xcl_off);
    uint8_t* wpk = base + l.wpk_off;
    __nv_bfloat16* wt = reinterpret_cast<__nv_bfloat16*>(base + l.wt_off);
    const TcDims d = tc_dims(gt);
    int r = launch_channels_last(gt, dy, dycl, st);              // gt.cl == g.cl: dy has the layout of y
    if (r != 0) return r;
    {
        const long long total = (long long)g.C * g.kv * g.Og;
        const int blocks = (int)((total + 255) / 256 < 8ll * sm_count() ? (total + 255) / 256 : 8ll * sm_count());
        weight_flip_to_kmajor_bf16<<<blocks, 256, 0, st>>>(g, w, wt);
        if (cudaGetLastError() != cudaSuccess) return -5;
    }
    pack_weight_fwd<<<gt.G * d.MT * d.KC, 256, 0, st>>>(gt, wt, wpk, d.MT, d.KC);
    if (cudaGetLastError() != cudaSuccess) return -5;
    Geom gk = gt;
    gk.cl = dx_cl ? 1 : 0;
    // add: the tiles leave through reductions into the dX that is already there
    return ndim == 2 ? launch_tc_forward<2, false>(gk, dycl, nullptr, wpk, nullptr, dx, st, add)
                     : launch_tc_forward<3, false>(gk, dycl, nullptr, wpk, nullptr, dx, st, add);
}

// The shared-memory-accumulating backward-data kernel is taken whenever it fits (DCN_BWD2D=0 forces the
// global-reduction kernels, for A/B measurements).
bool use_bwd2d(const Geom& g, int ndim, int deform) {
    static const bool off = [] { const char* e = getenv("DCN_BWD2D"); return e != nullptr && e[0] == '0'; }();
    return !off && b2_supported(g, ndim, deform);
}

// dy packed (max|dy| taken on the way), slab-wise weight tiles (max|W|), cleared dOffset, then the kernel.
int run_bwd2d(const Geom& g, const __nv_bfloat16* xcl, const float* off, const float* w, const float* dy, uint8_t* dpk,
              uint8_t* wpk, __nv_bfloat16* wt, unsigned int* scale, uint4* pts, float* dx, float* doff, bool accumulate,
              cudaStream_t st) {
    const B2Dims d = b2_dims(g);
    {
        const long long total = (long long)g.N * g.dg * g.kv * g.ov;
        const long long want = (total + 255) / 256;
        const int blocks = (int)(want < 16ll * sm_count() ? want : 16ll * sm_count());
        b2_points_kernel<<<blocks, 256, 0, st>>>(g, off, pts, d.Wp, d.W2);
        if (cudaGetLastError() != cudaSuccess) return -5;
    }
    if (cudaMemsetAsync(scale, 0, 8, st) != cudaSuccess) return -5;
    int r = launch_pack_dy(g, dy, dpk, d.MT, d.PC, st, scale);
    if (r != 0) return r;
    r = launch_weight_to_kmajor(g, w, wt, scale + 1, st);
    if (r != 0) return r;
    pack_weight_slab<<<g.G * d.SL * d.OC, 256, 0, st>>>(g, wt, wpk, d.SL, d.OC);
    if (cudaGetLastError() != cudaSuccess) return -5;
    if (doff != nullptr &&
        cudaMemsetAsync(doff, 0, (size_t)g.N * g.dg * g.kv * 2 * g.ov * sizeof(float), st) != cudaSuccess)
        return -5;
    return launch_tc_bwd2d(g, xcl, pts, dpk, wpk, scale, dx, doff, accumulate, st);
}

}  // namespace

bool tc_supported(const Geom& g, int ndim, int deform) {
    (void)ndim;
    if (g.Cg % 8 != 0) return false;
    if (deform && g.cpg % 8 != 0) return false;
    if (g.N > 65535) return false;
    return true;
}

size_t tc_workspace_bytes(const Geom& g, int ndim, int pass) {
    (void)ndim;
    if (pass == 0) return fwd_workspace(g).total;
    if (pass == 1) return bwd_data_workspace(g).total;
    return bwd_weight_workspace(g).total;
}

// Kernels a pass enqueues when every gradient is wanted (memsets not counted).
int tc_launch_count(const Geom& g, int ndim, int deform, int pass) {
    const bool b2 = use_bwd2d(g, ndim, deform);
    Geom gt;
    const bool gather = use_gather_dgrad(g, ndim, deform, gt);
    if (pass == 0) return 4;      // channels-last copy, weight reorder, weight tiles, implicit GEMM
    if (gather && pass == 1) return 4;      // dy copy, mirrored weights, weight tiles, forward kernel on dy (adds into dX)
    if (gather && pass == 3) return 8;      // the first four of those + input copy, dy pack, wgrad, dW unpack
    if (pass == 1) {
        if (b2) return 6;         // input copy, sampling points, dy pack, weight reorder, slab tiles, GEMM + scatter
        return g.cl ? 5 : 6;      // input copy, dy pack, weight reorder, weight tiles, GEMM + scatter, (dx transpose-add)
    }
    if (pass == 2) return 4;      // channels-last copy, dy pack, implicit GEMM, dW unpack
    // fused backward (input copy taken over from the forward pass when the caller hands it in: counted here)
    if (b2) return 8;             // input copy, points, dy pack, weight reorder, slab tiles, dgrad, wgrad, dW unpack
    return g.cl ? 7 : 8;          // input copy, dy pack, weight reorder, weight tiles, dgrad, (dx transpose,) wgrad, dW unpack
}

int tc_debug_points(const Geom& g, int ndim, int deform, const float* off, int n, float* coords, int32_t* valid,
                    int32_t* lo, int32_t* hi, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!b2_supported(g, ndim, deform)) return -3;
    const BwdDataWorkspace l = bwd_data_workspace(g);
    if (ws_bytes < l.total) return -4;
    uint4* pts = reinterpret_cast<uint4*>(static_cast<uint8_t*>(ws) + l.dxcl_off);
    const B2Dims d = b2_dims(g);
    const long long total = (long long)g.N * g.dg * g.kv * g.ov;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 16ll * sm_count() ? want : 16ll * sm_count());
    b2_points_kernel<<<blocks, 256, 0, st>>>(g, off, pts, d.Wp, d.W2);
    if (cudaGetLastError() != cudaSuccess) return -5;
    b2_points_decode_kernel<<<blocks, 256, 0, st>>>(g, pts, n, d.Wp, d.W2, coords, valid, lo, hi);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// `xcl_in`: a channels-last bf16 copy of x that already exists (the workspace's own copy is then not built).
static int tc_forward_x(const Geom& g, int ndim, int deform, const float* x, const __nv_bfloat16* xcl_in, const float* off,
                        const float* w, const float* bias, float* y, void* ws, size_t ws_bytes, cudaStream_t st) {
    const FwdWorkspace l = fwd_workspace(g);
    if (ws_bytes < l.total) return -4;
    uint8_t* base = static_cast<uint8_t*>(ws);
    const __nv_bfloat16* xcl = xcl_in;
    uint8_t* wpk = base + l.wpk_off;
    const TcDims d = tc_dims(g);
    int r = 0;
    if (xcl == nullptr) {
        __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(base + l.xcl_off);
        r = launch_channels_last(g, x, mine, st);
        if (r != 0) return r;
        xcl = mine;
    }
    __nv_bfloat16* wt = reinterpret_cast<__nv_bfloat16*>(base + l.wt_off);
    r = launch_weight_to_kmajor(g, w, wt, nullptr, st);
    if (r != 0) return r;
    pack_weight_fwd<<<g.G * d.MT * d.KC, 256, 0, st>>>(g, wt, wpk, d.MT, d.KC);
    if (cudaGetLastError() != cudaSuccess) return -5;
    if (ndim == 2) return deform ? launch_tc_forward<2, true>(g, xcl, off, wpk, bias, y, st)
                                 : launch_tc_forward<2, false>(g, xcl, off, wpk, bias, y, st);
    return deform ? launch_tc_forward<3, true>(g, xcl, off, wpk, bias, y, st)
                  : launch_tc_forward<3, false>(g, xcl, off, wpk, bias, y, st);
}

int tc_forward(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
               const float* bias, float* y, void* ws, size_t ws_bytes, cudaStream_t st) {
    return tc_forward_x(g, ndim, deform, x, nullptr, off, w, bias, y, ws, ws_bytes, st);
}

int tc_backward_data(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
                     const float* dy, float* dx, float* doff, void* ws, size_t ws_bytes, cudaStream_t st) {
    const BwdDataWorkspace l = bwd_data_workspace(g);
    if (ws_bytes < l.total) return -4;
    uint8_t* base = static_cast<uint8_t*>(ws);
    __nv_bfloat16* xcl = reinterpret_cast<__nv_bfloat16*>(base + l.xcl_off);
    uint8_t* dpk = base + l.dpk_off;
    uint8_t* wpk = base + l.wpk_off;
    if (g.cl && dx != nullptr && (reinterpret_cast<uintptr_t>(dx) & 15) != 0) return -7;   // 16-byte reductions
    // a channels-last dx is the scatter target itself (this entry point accumulates into dx)
    float* dxcl = dx == nullptr ? nullptr : (g.cl ? dx : reinterpret_cast<float*>(base + l.dxcl_off));
    if (!deform) doff = nullptr;
    const DgDims d = dg_dims(g);
    int r = 0;
    if (deform) {
        r = launch_channels_last(g, x, xcl, st);
        if (r != 0) return r;
    }
    if (use_bwd2d(g, ndim, deform))
        return run_bwd2d(g, xcl, off, w, dy, dpk, wpk, reinterpret_cast<__nv_bfloat16*>(base + l.wt_off),
                         reinterpret_cast<unsigned int*>(base + l.scale_off),
                         reinterpret_cast<uint4*>(base + l.dxcl_off), dx, doff, true, st);
    {
        Geom gt;
        if (dx != nullptr && use_gather_dgrad(g, ndim, deform, gt))          // plain, stride 1: a gather, added to dx
            return run_gather_dgrad(g, gt, ndim, w, dy, dx, true, g.cl != 0, base + l.gath_off, st);
    }
    r = launch_pack_dy(g, dy, dpk, d.MT, d.PC2, st);
    if (r != 0) return r;
    r = launch_weight_to_kmajor(g, w, reinterpret_cast<__nv_bfloat16*>(base + l.wt_off), nullptr, st);
    if (r != 0) return r;
    pack_weight_bwd<<<g.G * d.NB * d.OC, 256, 0, st>>>(g, reinterpret_cast<const __nv_bfloat16*>(base + l.wt_off), wpk,
                                                       d.NB, d.OC);
    if (cudaGetLastError() != cudaSuccess) return -5;
    if (dxcl != nullptr && !g.cl && cudaMemsetAsync(dxcl, 0, (size_t)g.N * g.iv * g.C * 4, st) != cudaSuccess) return -5;
    if (doff != nullptr &&
        cudaMemsetAsync(doff, 0, (size_t)g.N * g.dg * g.kv * ndim * g.ov * sizeof(float), st) != cudaSuccess)
        return -5;
    if (ndim == 2) r = deform ? launch_tc_dgrad<2, true>(g, xcl, off, dpk, wpk, dxcl, doff, st)
                              : launch_tc_dgrad<2, false>(g, xcl, off, dpk, wpk, dxcl, doff, st);
    else r = deform ? launch_tc_dgrad<3, true>(g, xcl, off, dpk, wpk, dxcl, doff, st)
                    : launch_tc_dgrad<3, false>(g, xcl, off, dpk, wpk, dxcl, doff, st);
    if (r != 0) return r;
    if (dx != nullptr && !g.cl) {
        dim3 grid((unsigned)((g.iv + 31) / 32), (unsigned)((g.C + 31) / 32), (unsigned)g.N);
        from_channels_last<true><<<grid, 256, 0, st>>>(dxcl, dx, g.C, g.iv);
        if (cudaGetLastError() != cudaSuccess) return -5;
    }
    return 0;
}

int tc_backward_weight(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* dy,
                       float* dw, void* ws, size_t ws_bytes, cudaStream_t st) {
    const BwdWeightWorkspace l = bwd_weight_workspace(g);
    if (ws_bytes < l.total) return -4;
    uint8_t* base = static_cast<uint8_t*>(ws);
    __nv_bfloat16* xcl = reinterpret_cast<__nv_bfloat16*>(base + l.xcl_off);
    uint8_t* dpk = base + l.dpk_off;
    const WgDims d = wg_dims(g);
    int r = launch_channels_last(g, x, xcl, st);
    if (r != 0) return r;
    r = launch_pack_dy(g, dy, dpk, d.MT, d.PC, st);
    if (r != 0) return r;
    float* dwpk = reinterpret_cast<float*>(base + l.dwpk_off);
    if (ndim == 2) r = deform ? launch_tc_wgrad<2, true>(g, xcl, off, dpk, dwpk, st)
                              : launch_tc_wgrad<2, false>(g, xcl, off, dpk, dwpk, st);
    else r = deform ? launch_tc_wgrad<3, true>(g, xcl, off, dpk, dwpk, st)
                    : launch_tc_wgrad<3, false>(g, xcl, off, dpk, dwpk, st);
    if (r != 0) return r;
    return dwpk_fold<true>(g, dwpk, dw, st);         // this entry point accumulates into dW
}

// ---------------------------------------------------------------------------------------------------
// Fused backward: all requested gradients in one call.  The channels-last input copy and the packed dy are
// built once and shared by the data and weight kernels (or the input copy is taken over from the forward
// pass), and every output is overwritten, so no caller-side zero fill and no read-modify-write of dx.
// ---------------------------------------------------------------------------------------------------
size_t tc_backward_workspace_bytes(const Geom& g) { return bwd_data_workspace(g).total; }

int tc_backward(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
                const float* dy, const void* xcl_in, float* dx, float* doff, float* dw, void* ws, size_t ws_bytes,
                cudaStream_t st) {
    const BwdDataWorkspace l = bwd_data_workspace(g);
    if (ws_bytes < l.total) return -4;
    uint8_t* base = static_cast<uint8_t*>(ws);
    const __nv_bfloat16* xcl = static_cast<const __nv_bfloat16*>(xcl_in);
    uint8_t* dpk = base + l.dpk_off;
    uint8_t* wpk = base + l.wpk_off;
    if (g.cl && dx != nullptr && (reinterpret_cast<uintptr_t>(dx) & 15) != 0) return -7;   // 16-byte reductions
    // a channels-last dx is the scatter target itself (zero-filled here: this entry point overwrites)
    float* dxcl = dx == nullptr ? nullptr : (g.cl ? dx : reinterpret_cast<float*>(base + l.dxcl_off));
    if (!deform) doff = nullptr;
    const DgDims d = dg_dims(g);
    int r = 0;
    const bool need_x = dw != nullptr || (deform && (dx != nullptr || doff != nullptr));
    if (xcl == nullptr && need_x) {
        __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(base + l.xcl_off);
        r = launch_channels_last(g, x, mine, st);
        if (r != 0) return r;
        xcl = mine;
    }
    const bool b2 = (dx != nullptr || doff != nullptr) && use_bwd2d(g, ndim, deform);
    if (b2) {
        r = run_bwd2d(g, xcl, off, w, dy, dpk, wpk, reinterpret_cast<__nv_bfloat16*>(base + l.wt_off),
                      reinterpret_cast<unsigned int*>(base + l.scale_off),
                      reinterpret_cast<uint4*>(base + l.dxcl_off), dx, doff, false, st);
        if (r != 0) return r;
    } else {
        r = launch_pack_dy(g, dy, dpk, d.MT, d.PC2, st);
        if (r != 0) return r;
    }
    Geom gt;
    const bool gather = !b2 && dx != nullptr && use_gather_dgrad(g, ndim, deform, gt);
    if (gather) {                                                          // plain, stride 1: dX as a gather
        r = run_gather_dgrad(g, gt, ndim, w, dy, dx, false, g.cl != 0, base + l.gath_off, st);
        if (r != 0) return r;
    }
    if (!b2 && !gather && (dx != nullptr || doff != nullptr)) {
        r = launch_weight_to_kmajor(g, w, reinterpret_cast<__nv_bfloat16*>(base + l.wt_off), nullptr, st);
        if (r != 0) return r;
        pack_weight_bwd<<<g.G * d.NB * d.OC, 256, 0, st>>>(g, reinterpret_cast<const __nv_bfloat16*>(base + l.wt_off), wpk,
                                                           d.NB, d.OC);
        if (cudaGetLastError() != cudaSuccess) return -5;
        if (dxcl != nullptr && cudaMemsetAsync(dxcl, 0, (size_t)g.N * g.iv * g.C * 4, st) != cudaSuccess) return -5;
        if (doff != nullptr &&
            cudaMemsetAsync(doff, 0, (size_t)g.N * g.dg * g.kv * ndim * g.ov * sizeof(float), st) != cudaSuccess)
            return -5;
        if (ndim == 2) r = deform ? launch_tc_dgrad<2, true>(g, xcl, off, dpk, wpk, dxcl, doff, st)
                                  : launch_tc_dgrad<2, false>(g, xcl, off, dpk, wpk, dxcl, doff, st);
        else r = deform ? launch_tc_dgrad<3, true>(g, xcl, off, dpk, wpk, dxcl, doff, st)
                        : launch_tc_dgrad<3, false>(g, xcl, off, dpk, wpk, dxcl, doff, st);
        if (r != 0) return r;
        if (dx != nullptr && !g.cl) {
            dim3 grid((unsigned)((g.iv + 31) / 32), (unsigned)((g.C + 31) / 32), (unsigned)g.N);
            from_channels_last<false><<<grid, 256, 0, st>>>(dxcl, dx, g.C, g.iv);
            if (cudaGetLastError() != cudaSuccess) return -5;
        }
    }
    if (dw != nullptr) {
        float* dwpk = reinterpret_cast<float*>(base + l.dwpk_off);
        // the weight kernel reads dy tiles with the same layout and stride (PC2 == wg_dims().PC)
        if (ndim == 2) r = deform ? launch_tc_wgrad<2, true>(g, xcl, off, dpk, dwpk, st)
                                  : launch_tc_wgrad<2, false>(g, xcl, off, dpk, dwpk, st);
        else r = deform ? launch_tc_wgrad<3, true>(g, xcl, off, dpk, dwpk, st)
                        : launch_tc_wgrad<3, false>(g, xcl, off, dpk, dwpk, st);
        if (r != 0) return r;
        r = dwpk_fold<false>(g, dwpk, dw, st);       // the fused entry point overwrites dW
        if (r != 0) return r;
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------------
// Deformable layer: the plain convolution that produces the offsets (geometry gq: same input, taps, stride and
// padding, dilation 1, one group, dg*kv*D output channels, channel-first output whatever the layout of x)
// followed by the deformable convolution (geometry g) of the same input.  One channels-last bf16 copy of x
// serves both convolutions in the forward pass and all four gradient kernels in the backward pass; the offsets
// are written once and read back while they are still in L2.
// Workspaces: forward  [ forward workspace of g (its start holds the input copy) | forward workspace of gq ]
//             backward [ dOffset | backward workspace of g | backward workspace of gq ]
// ---------------------------------------------------------------------------------------------------
static size_t layer_doff_bytes(const Geom& g, int ndim) {
    return align_up((size_t)g.N * g.dg * g.kv * ndim * g.ov * sizeof(float), 256);
}

size_t tc_layer_workspace_bytes(const Geom& g, const Geom& gq, int ndim, int pass) {
    if (pass == 0) return fwd_workspace(g).total + align_up(fwd_workspace(gq).total, 256);
    return layer_doff_bytes(g, ndim) + align_up(bwd_data_workspace(g).total, 256) + align_up(bwd_data_workspace(gq).total, 256);
}

int tc_layer_forward(const Geom& g, const Geom& gq, int ndim, const float* x, const float* w_off, const float* b_off,
                     const float* w, const float* bias, float* offsets, float* y, void* ws, size_t ws_bytes,
                     cudaStream_t st) {
    if (ws_bytes < tc_layer_workspace_bytes(g, gq, ndim, 0)) return -4;
    uint8_t* base = static_cast<uint8_t*>(ws);
    const size_t main_bytes = align_up(fwd_workspace(g).total, 256);
    __nv_bfloat16* xcl = reinterpret_cast<__nv_bfloat16*>(base + fwd_workspace(g).xcl_off);
    int r = launch_channels_last(g, x, xcl, st);
    if (r != 0) return r;
    r = tc_forward_x(gq, ndim, 0, x, xcl, nullptr, w_off, b_off, offsets, base + main_bytes, ws_bytes - main_bytes, st);
    if (r != 0) return r;
    return tc_forward_x(g, ndim, 1, x, xcl, offsets, w, bias, y, base, main_bytes, st);
}

// Gradients of the offset-producing convolution given dOffset: its input gradient is ADDED to dx (which the
// deformable part has already written, in the layout of g), its weight gradient overwrites dw_off.
static int plain_backward_into(const Geom& gq, int ndim, bool dx_channels_last, const __nv_bfloat16* xcl,
                               const float* w_off, const float* dyq, float* dx, float* dw_off, void* ws,
                               cudaStream_t st) {
    const BwdDataWorkspace l = bwd_data_workspace(gq);
    uint8_t* base = static_cast<uint8_t*>(ws);
    uint8_t* dpk = base + l.dpk_off;
    uint8_t* wpk = base + l.wpk_off;
    const DgDims d = dg_dims(gq);
    int r = launch_pack_dy(gq, dyq, dpk, d.MT, d.PC2, st);
    if (r != 0) return r;
    Geom gt;
    if (dx != nullptr && use_gather_dgrad(gq, ndim, 0, gt)) {      // stride 1: a gather, added to the dX already there
        r = run_gather_dgrad(gq, gt, ndim, w_off, dyq, dx, true, dx_channels_last, base + l.gath_off, st);
        if (r != 0) return r;
        dx = nullptr;                                              // done
    }
    if (dx != nullptr) {
        __nv_bfloat16* wt = reinterpret_cast<__nv_bfloat16*>(base + l.wt_off);
        r = launch_weight_to_kmajor(gq, w_off, wt, nullptr, st);
        if (r != 0) return r;
        pack_weight_bwd<<<gq.G * d.NB * d.OC, 256, 0, st>>>(gq, wt, wpk, d.NB, d.OC);
        if (cudaGetLastError() != cudaSuccess) return -5;
        float* dxcl = dx_channels_last ? dx : reinterpret_cast<float*>(base + l.dxcl_off);
        if (!dx_channels_last && cudaMemsetAsync(dxcl, 0, (size_t)gq.N * gq.iv * gq.C * 4, st) != cudaSuccess) return -5;
        r = ndim == 2 ? launch_tc_dgrad<2, false>(gq, xcl, nullptr, dpk, wpk, dxcl, nullptr, st)
                      : launch_tc_dgrad<3, false>(gq, xcl, nullptr, dpk, wpk, dxcl, nullptr, st);
        if (r != 0) return r;
        if (!dx_channels_last) {
            dim3 grid((unsigned)((gq.iv + 31) / 32), (unsigned)((gq.C + 31) / 32), (unsigned)gq.N);
            from_channels_last<true><<<grid, 256, 0, st>>>(dxcl, dx, gq.C, gq.iv);
            if (cudaGetLastError() != cudaSuccess) return -5;
        }
    }
    if (dw_off != nullptr) {
        float* dwpk = reinterpret_cast<float*>(base + l.dwpk_off);
        r = ndim == 2 ? launch_tc_wgrad<2, false>(gq, xcl, nullptr, dpk, dwpk, st)
                      : launch_tc_wgrad<3, false>(gq, xcl, nullptr, dpk, dwpk, st);
        if (r != 0) return r;
        r = dwpk_fold<false>(gq, dwpk, dw_off, st);
        if (r != 0) return r;
    }
    return 0;
}

int tc_layer_backward(const Geom& g, const Geom& gq, int ndim, const float* x, const float* offsets, const float* w_off,
                      const float* w, const float* dy, const void* xcl_in, float* dx, float* dw_off, float* dw,
                      float** doff_out, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (ws_bytes < tc_layer_workspace_bytes(g, gq, ndim, 3)) return -4;
    uint8_t* base = static_cast<uint8_t*>(ws);
    float* doff = reinterpret_cast<float*>(base);
    uint8_t* ws_main = base + layer_doff_bytes(g, ndim);
    const size_t main_bytes = align_up(bwd_data_workspace(g).total, 256);
    uint8_t* ws_q = ws_main + main_bytes;
    const __nv_bfloat16* xcl = static_cast<const __nv_bfloat16*>(xcl_in);
    if (xcl == nullptr) {
        __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(ws_main + bwd_data_workspace(g).xcl_off);
        const int r0 = launch_channels_last(g, x, mine, st);
        if (r0 != 0) return r0;
        xcl = mine;
    }
    const bool chain = dx != nullptr || dw_off != nullptr || doff_out != nullptr;     // dOffset is needed downstream
    int r = tc_backward(g, ndim, 1, x, offsets, w, dy, xcl, dx, chain ? doff : nullptr, dw, ws_main, main_bytes, st);
    if (r != 0) return r;
    if (doff_out != nullptr) *doff_out = doff;
    if (dx == nullptr && dw_off == nullptr) return 0;
    return plain_backward_into(gq, ndim, g.cl != 0, xcl, w_off, doff, dx, dw_off, ws_q, st);
}

// ---------------------------------------------------------------------------------------------------
// Forward pass for callers that must not allocate: the scratch (channels-last bf16 copy of the input and
// the packed weight tiles) lives in a fixed array that is part of the library image instead of a
// caller-provided workspace.  Every device that loads the library holds kStaticScratchBytes until the
// process exits.  In host code the array's name is only a stand-in for the symbol; the device address is
// obtained once per device with cudaGetSymbolAddress while that device is current.
// ---------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = (size_t)32 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

size_t tc_static_scratch_bytes() { return kStaticScratchBytes; }

int tc_forward_static(const Geom& g, int ndim, int deform, const float* x, const float* off, const float* w,
                      const float* bias, float* y, cudaStream_t st) {
    constexpr int kMaxDevices = 64;
    static void* volatile scratch_of_device[kMaxDevices] = {};
    if (fwd_workspace(g).total > kStaticScratchBytes) return -8;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return -5;
    if (dev < 0 || dev >= kMaxDevices) return -8;
    void* ptr = scratch_of_device[dev];
    if (ptr == nullptr) {
        // first call on this device: resolve the array's device address (may load the module)
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return -5;
        scratch_of_device[dev] = ptr;      // racing first calls resolve the same address
    }
    return tc_forward(g, ndim, deform, x, off, w, bias, y, ptr, kStaticScratchBytes, st);
}

// A wait that cannot complete: one thread waits, with a limit of about a millisecond, on a barrier nothing ever
// arrives on.  It must give up, raise the status word and return -- the path every pipeline role of the kernels
// above takes when its bounded wait runs out.  For the test of that path only.
namespace {
__global__ void expire_wait_kernel(long long limit_cycles, int* gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_barrier_init();
        const bool ok = mbar_wait(&bar, 0, limit_cycles);
        if (gave_up != nullptr) *gave_up = ok ? 0 : 1;
    }
}
}  // namespace

int tc_debug_expire_wait(int* gave_up, cudaStream_t st) {
    expire_wait_kernel<<<1, 32, 0, st>>>(2000000ll, gave_up);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int tc_check_status(cudaStream_t st) {
    if (cudaStreamSynchronize(st) != cudaSuccess) return -5;
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)) != cudaSuccess) return -5;
    if (v != 0) {
        const unsigned int z = 0;
        cudaMemcpyToSymbol(g_tc_status, &z, sizeof(z));
        return -6;
    }
    return 0;
}

}  // namespace dcn
