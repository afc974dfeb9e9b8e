// Input and offset gradients on tcgen05, row-wise epilogue variant (included by dcn_tc.cu inside its anonymous
// namespace): every epilogue thread keeps its output position for the scatter as well.  Fallback of
// dcn_tc_dgrad2.cuh for channel-group sizes that variant does not take; also defines the packers, the
// work decomposition and the GEMM description shared by both.
//
//   col[P, k'] = sum over o of dy[o, P] * W[o, k']                    k' = tap * Cg + c
// is produced tile by tile in tensor memory and consumed there: the epilogue threads (one per output
// position) re-locate the sampling point of every (deformable group, tap), then
//   input gradient : channels-last fp32 accumulator dx_cl[n, corner, c..c+7] += weight(corner) * col
//                    with 16-byte vector reductions (8 consecutive channels per corner),
//   offset gradient: dot products of col with the corner values over the group's channels, kept in
//                    registers (the channel axis lies along the thread's own columns), combined with the
//                    interpolation-weight derivatives and added to dOffset once per (group, tap, position).
// The reference's column buffer (col) never reaches memory.
//   A operand: dy, bf16, pack_dy tiles read as MN-major [64 o rows][64 P per 128-byte row], two P halves
//   B operand: W^T, bf16, pre-packed [k' rows][64 o per 128-byte row]              -> K-major
#pragma once

constexpr int kDgStages = 4;
constexpr int kDgEpiWarps = 8;
constexpr int kDgThreads = 32 * (2 + kDgEpiWarps);

struct DgSmem {
    // per stage: A (2 halves x 8 KB) | B (256 rows x 128 B = 32 KB)
    static constexpr int kStageBytes = kTileBytes + 2 * kTileBytes;
    static constexpr int kBarOffset = kDgStages * kStageBytes;
    static constexpr int kTotal = kBarOffset + (2 * kDgStages + 4) * 8 + 16;
};

// Wt [O][kv * Cg] bf16 (k' order) -> bf16 tiles [G][NB][OC][256 k' rows x 64 o], swizzled K-major: the transpose of a
// 64 x 256 piece of Wt through shared memory, 512-byte row reads and 128-byte tile-row writes.
__global__ void __launch_bounds__(256)
pack_weight_bwd(const Geom g, const __nv_bfloat16* __restrict__ wt, uint8_t* __restrict__ wpk, int NB, int OC) {
    __shared__ __align__(16) uint16_t piece[64][256 + 8];   // [o][k'], rows padded against bank conflicts
    const int tile = blockIdx.x;                          // (j * NB + nb) * OC + oc
    const int oc = tile % OC, nb = (tile / OC) % NB, j = tile / OC / NB;
    uint8_t* dst = wpk + (size_t)tile * (2 * kTileBytes);
    const uint16_t* src = reinterpret_cast<const uint16_t*>(wt);
    for (int e = threadIdx.x; e < 64 * 32; e += blockDim.x) {
        const int ol = e / 32, part = e % 32;
        const int o = oc * 64 + ol, kq = nb * 256 + part * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (o < g.Og && kq < g.Kg) v = __ldg(reinterpret_cast<const uint4*>(src + (size_t)(j * g.Og + o) * g.Kg + kq));
        *reinterpret_cast<uint4*>(&piece[ol][part * 8]) = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 256 * 8; e += blockDim.x) {
        const int row = e % 256, chunk = e / 256;         // consecutive threads read consecutive k' of one o
        uint32_t pk[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            pk[q] = (uint32_t)piece[chunk * 8 + 2 * q][row] | ((uint32_t)piece[chunk * 8 + 2 * q + 1][row] << 16);
        *reinterpret_cast<uint4*>(dst + swz_offset(row, chunk)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

// dx[n, c, p] (+)= dx_cl[n, p, c]
template <bool ACCUMULATE>
__global__ void __launch_bounds__(256)
from_channels_last(const float* __restrict__ dxcl, float* __restrict__ dx, int C, int iv) {
    __shared__ float tile[32][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    const float* in = dxcl + (size_t)n * iv * C;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = p0 + ty + i * 8, c = c0 + tx;
        tile[ty + i * 8][tx] = (p < iv && c < C) ? in[(size_t)p * C + c] : 0.f;
    }
    __syncthreads();
    float* out = dx + (size_t)n * C * iv;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + i * 8, p = p0 + tx;
        if (c < C && p < iv) {
            if (ACCUMULATE) out[(size_t)c * iv + p] += tile[tx][ty + i * 8];
            else out[(size_t)c * iv + p] = tile[tx][ty + i * 8];
        }
    }
}

template <int D, bool DEFORM>
__global__ void __launch_bounds__(kDgThreads, 1)
tc_dgrad_rowwise_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const float* __restrict__ off,
                const uint8_t* __restrict__ dpk, const uint8_t* __restrict__ wpk, float* __restrict__ dxcl,
                float* __restrict__ doff, const int MT, const int NB, const int NW, const int OC,
                const long long PC2, const long long PT) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + DgSmem::kBarOffset);
    uint64_t* empty = full + kDgStages;
    uint64_t* acc_full = empty + kDgStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDgStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], kDgEpiWarps);
        }
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = make_idesc(128, NW, 1, 0);   // A MN-major, B K-major
    const long long n_tiles = (long long)g.G * PT * NB;
    const uint32_t b_bytes = (uint32_t)NW * 128u;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0, tl = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tl) {
                const uint32_t b = tl & 1;
                ok = mbar_wait(&acc_empty[b], ((tl >> 1) & 1) ^ 1);
                tc_fence_after();
                for (int oc = 0; oc < OC && ok; ++oc, ++it) {
                    const uint32_t s = it % kDgStages;
                    ok = mbar_wait(&full[s], (it / kDgStages) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem + s * DgSmem::kStageBytes);
                    const uint32_t b_base = a_base + kTileBytes;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t ad = make_desc(a_base + k * 2048, 8192, 1024);
                        const uint64_t bd = make_desc(b_base + k * 32, 16, 1024);
                        umma_bf16(tmem_base + b * 256, ad, bd, idesc, (oc > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[b]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int nb = (int)(t % NB);
                const long long pt = (t / NB) % PT;
                const int j = (int)(t / NB / PT);
                for (int oc = 0; oc < OC && ok; ++oc, ++it) {
                    const uint32_t s = it % kDgStages;
                    ok = mbar_wait(&empty[s], ((it / kDgStages) & 1) ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&full[s], (uint32_t)kTileBytes + b_bytes);
                    uint8_t* a_dst = smem + s * DgSmem::kStageBytes;
                    const int mt = oc / 2, half = oc % 2;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint8_t* src = dpk + (((size_t)j * MT + mt) * PC2 + (pt * 2 + h)) * kTileBytes + half * 8192;
                        bulk_g2s(a_dst + h * 8192, src, 8192, &full[s]);
                    }
                    const uint8_t* wsrc = wpk + (((size_t)j * NB + nb) * OC + oc) * (2 * kTileBytes);
                    bulk_g2s(a_dst + kTileBytes, wsrc, b_bytes, &full[s]);
                }
            }
        }
    } else {
        // ------------------------------------------------ epilogue: one thread per output position
        const int q = warp & 3;
        const int half = (warp - 2) / 4;                // which 128-column half of the tile
        const int kq_total = g.kv * g.Cg;
        uint32_t tl = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tl) {
            const int nb = (int)(t % NB);
            const long long pt = (t / NB) % PT;
            const int j = (int)(t / NB / PT);
            const uint32_t b = tl & 1;
            const long long P = pt * 128 + q * 32 + lane;
            const bool p_ok = P < g.P;
            const OutPos op = decompose_pos(g, p_ok ? P : 0);
            const float* off_n = DEFORM ? off + (size_t)op.n * g.dg * g.kv * D * g.ov : nullptr;

            ok = mbar_wait(&acc_full[b], (tl >> 1) & 1);
            if (!ok) break;
            tc_fence_after();

            int key = -1;
            Pt<float, D> s;
            s.valid = false;
            int idx[1 << D];
            float cw[1 << D];
            float T[1 << D];
            float S = 0.f;
#pragma unroll
            for (int e = 0; e < (1 << D); ++e) { idx[e] = 0; cw[e] = 0.f; T[e] = 0.f; }

            auto flush = [&]() {
                if (!DEFORM || key < 0 || doff == nullptr) return;
                float gr[D];
                if (s.valid) {
                    interp_grad<float, D>(s, T, gr);
                } else {
#pragma unroll
                    for (int a = 0; a < D; ++a) gr[a] = (D == 3 && g.oob) ? oob_term<float>(g, s.p[a], S) : 0.f;
                }
                float* dst = doff + ((size_t)op.n * g.dg * g.kv * D + (size_t)key * D) * g.ov + op.opos;
#pragma unroll
                for (int a = 0; a < D; ++a)
                    if (gr[a] != 0.f) atomicAdd(dst + (size_t)a * g.ov, gr[a]);
            };

            for (int cc = 0; cc < 4; ++cc) {
                const int col0 = half * 128 + cc * 32;
                if (col0 >= NW) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + b * 256 + col0, v);
                tmem_ld_wait();
                if (!p_ok) continue;
#pragma unroll
                for (int sc = 0; sc < 4; ++sc) {
                    const int kq = nb * 256 + col0 + sc * 8;
                    if (kq >= kq_total) break;
                    uint32_t tap, cl;
                    g.d_Cg.divmod((uint32_t)kq, tap, cl);
                    const int c = j * g.Cg + (int)cl;
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[sc * 8 + i]);
                    if (DEFORM) {
                        const int grp = (int)g.d_cpg.div((uint32_t)c);
                        const int k2 = grp * g.kv + (int)tap;
                        if (k2 != key) {
                            flush();
                            key = k2;
                            locate<float, D>(g, off_n, grp, (int)tap, op, s);
                            if (s.valid) {
                                corner_indices<float, D>(g, s, idx);
                                corner_weights<float, D>(s, cw);
                            }
                            S = 0.f;
#pragma unroll
                            for (int e = 0; e < (1 << D); ++e) T[e] = 0.f;
                        }
                        if (s.valid) {
                            const size_t base = ((size_t)op.n * g.iv) * g.C + c;
#pragma unroll
                            for (int e = 0; e < (1 << D); ++e) {
                                const size_t a = base + (size_t)idx[e] * g.C;
                                if (doff != nullptr) {
                                    const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xcl + a));
                                    float d = T[e];
                                    d = fmaf(f[0], bf16_lo(xv.x), d); d = fmaf(f[1], bf16_hi(xv.x), d);
                                    d = fmaf(f[2], bf16_lo(xv.y), d); d = fmaf(f[3], bf16_hi(xv.y), d);
                                    d = fmaf(f[4], bf16_lo(xv.z), d); d = fmaf(f[5], bf16_hi(xv.z), d);
                                    d = fmaf(f[6], bf16_lo(xv.w), d); d = fmaf(f[7], bf16_hi(xv.w), d);
                                    T[e] = d;
                                }
                                if (dxcl != nullptr) {
                                    const float wv = cw[e];
                                    atomicAdd(reinterpret_cast<float4*>(dxcl + a),
                                              make_float4(wv * f[0], wv * f[1], wv * f[2], wv * f[3]));
                                    atomicAdd(reinterpret_cast<float4*>(dxcl + a + 4),
                                              make_float4(wv * f[4], wv * f[5], wv * f[6], wv * f[7]));
                                }
                            }
                        } else if (D == 3 && g.oob) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) S += fabsf(f[i]);
                        }
                    } else {
                        int pidx;
                        if (dxcl != nullptr && locate_plain<D>(g, (int)tap, op, pidx)) {
                            const size_t a = ((size_t)op.n * g.iv + pidx) * g.C + c;
                            atomicAdd(reinterpret_cast<float4*>(dxcl + a), make_float4(f[0], f[1], f[2], f[3]));
                            atomicAdd(reinterpret_cast<float4*>(dxcl + a + 4), make_float4(f[4], f[5], f[6], f[7]));
                        }
                    }
                }
            }
            flush();
            tc_fence_before();
            mbar_arrive_warp(&acc_empty[b]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

struct DgDims {
    int MT, NB, NW, OC;
    long long PC2, PT;
};

inline DgDims dg_dims(const Geom& g) {
    DgDims d;
    d.MT = (g.Og + 127) / 128;
    const int kq = g.kv * g.Cg;
    d.NB = (kq + 255) / 256;
    d.NW = kq >= 256 ? 256 : ((kq + 63) / 64) * 64;
    d.OC = (g.Og + 63) / 64;
    d.PT = (g.P + 127) / 128;
    d.PC2 = d.PT * 2;
    return d;
}

template <int D, bool DEFORM>
int launch_tc_dgrad_rowwise(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* dpk,
                    const uint8_t* wpk, float* dxcl, float* doff, cudaStream_t st) {
    const DgDims d = dg_dims(g);
    const int smem = DgSmem::kTotal + 1024;
    auto kern = tc_dgrad_rowwise_kernel<D, DEFORM>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    const long long tiles = (long long)g.G * d.PT * d.NB;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kern<<<grid, kDgThreads, smem, st>>>(g, xcl, off, dpk, wpk, dxcl, doff, d.MT, d.NB, d.NW, d.OC, d.PC2, d.PT);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
