// Input and offset gradients on tcgen05 with a transposed, warp-aggregated epilogue (included by dcn_tc.cu
// inside its anonymous namespace).  GEMM, operands, pipeline and tile order are those of dcn_tc_dgrad.cuh:
//   col[P, k'] = sum over o of dy[o, P] * W[o, k']        one tensor-memory lane = one output position.
//
// Epilogue, per warp and per chunk of 32 columns (32 channels of one tap):
//   phase A  (thread = position)  tcgen05.ld the 32 columns, stage them in shared memory, and when the chunk
//            starts a new (deformable group, tap) key, locate the position's sampling point and publish its
//            corner indices and corner weights;
//   phase B  (lane = (row mod 4, channel quad))  8 lanes cover 32 consecutive channels = 128 contiguous bytes
//            of the channels-last tensors, so one warp-wide vector reduction adds 4 full 128-byte lines into
//            dx_cl (instead of 32 scattered 16-byte pieces), and the input values for the offset gradient
//            arrive as contiguous 64-byte row segments; the per-corner dot products over the channels are
//            accumulated per lane and, when the key ends, reduced across the lanes of the key with shuffles;
//   flush    (thread = position again) the 2^D dot products become the D offset-gradient components through
//            the interpolation-weight derivatives and are added to dOffset, coalesced along positions.
// Taken when key boundaries fall on multiples of U = 32 or 16 channels (U = min(32, cpg, Cg) divides Cg and cpg):
// a 32-column chunk then holds one or two whole keys.  Other channel-group sizes use the row-wise variant.
#pragma once

constexpr int kDg2Stages = 2;

template <int D, bool DEFORM>
struct alignas(16) DgEntry {
    int idx[1 << D];  // corner positions in the whole channels-last tensor (sample * in volume + corner); idx[0] < 0: invalid
    float cw[1 << D];
};

template <int D, bool DEFORM, int EW, int U>
struct Dg2Smem {
    static constexpr int kSlots = 32 / U;                                      // keys per 32-column chunk
    static constexpr int kStageBytes = 3 * kTileBytes;                         // A 16 KB | B 32 KB
    static constexpr int kStagesBytes = kDg2Stages * kStageBytes;
    static constexpr int kColFloats = 32 * 36;                                 // per warp: 32 rows x (32 + 4 pad)
    static constexpr int kTotStride = 9;                                       // 2^D + 1 totals per row (D = 3)
    static constexpr int kTotFloats = kSlots * 32 * kTotStride;                // per warp
    static constexpr int kEntryBytes = kSlots * 32 * (int)sizeof(DgEntry<D, DEFORM>);   // per warp: slots x 32 rows
    static constexpr int kWarpBytes = (kColFloats + kTotFloats) * 4 + kEntryBytes;
    static constexpr int kBarOffset = kStagesBytes + EW * kWarpBytes;
    static constexpr int kTotal = kBarOffset + (2 * kDg2Stages + 4) * 8 + 16;
};

// EW epilogue warps: 8 (each 128 columns of the tile) or 16 (each 64 columns).
// U: channel granularity of the keys, 32 (one key per 32-column chunk) or 16 (two keys per chunk).
template <int D, bool DEFORM, int EW, int U>
__global__ void __launch_bounds__(32 * (2 + EW), 1)
tc_dgrad_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const float* __restrict__ off,
                const uint8_t* __restrict__ dpk, const uint8_t* __restrict__ wpk, float* __restrict__ dxcl,
                float* __restrict__ doff, const int MT, const int NB, const int NW, const int OC,
                const long long PC2, const long long PT) {
    using SM = Dg2Smem<D, DEFORM, EW, U>;
    using Entry = DgEntry<D, DEFORM>;
    constexpr int NC = 1 << D;
    constexpr int NS = 32 / U;                   // keys (slots) per chunk
    constexpr int LG = U / 4;                    // lanes that share a key within a row
    constexpr int kColsPerWarp = 256 / (EW / 4);
    extern __shared__ __align__(1024) uint8_t smem_dg2[];     // the kernel has no static shared memory: base is 1024-aligned
    uint8_t* smem = smem_dg2;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM::kBarOffset);
    uint64_t* empty = full + kDg2Stages;
    uint64_t* acc_full = empty + kDg2Stages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDg2Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], EW);
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
                    const uint32_t s = it % kDg2Stages;
                    ok = mbar_wait(&full[s], (it / kDg2Stages) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem + s * SM::kStageBytes);
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
                    const uint32_t s = it % kDg2Stages;
                    ok = mbar_wait(&empty[s], ((it / kDg2Stages) & 1) ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&full[s], (uint32_t)kTileBytes + b_bytes);
                    uint8_t* a_dst = smem + s * SM::kStageBytes;
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
        // ------------------------------------------------ epilogue
        const int ew = warp - 2;
        const int q = warp & 3;                         // tensor-memory lane quarter
        const int part = ew / 4;                        // which column range of the tile
        float* colS = reinterpret_cast<float*>(smem + SM::kStagesBytes + (size_t)ew * SM::kWarpBytes);   // [32][36]
        float* tot = colS + SM::kColFloats;                                                               // [32][12]
        Entry* ent = reinterpret_cast<Entry*>(tot + SM::kTotFloats);                                      // [32]
        const int kq_total = g.kv * g.Cg;
        const int r4 = lane >> 3, cq = lane & 7;        // phase-B coordinates of this lane
        const int my_slot = (cq * 4) / U;
        const bool want_x = DEFORM && doff != nullptr;
        uint32_t tl = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tl) {
            const int nb = (int)(t % NB);
            const long long pt = (t / NB) % PT;
            const int j = (int)(t / NB / PT);
            const uint32_t b = tl & 1;
            const long long P = pt * 128 + q * 32 + lane;          // phase-A position of this thread
            const bool p_ok = P < g.P;
            const OutPos op = decompose_pos(g, p_ok ? P : 0);
            const float* off_n = DEFORM ? off + (size_t)op.n * g.dg * g.kv * D * g.ov : nullptr;

            ok = mbar_wait(&acc_full[b], (tl >> 1) & 1);
            if (!ok) break;
            tc_fence_after();

            int key[NS];
            Pt<float, D> pts[NS];
#pragma unroll
            for (int sl = 0; sl < NS; ++sl) { key[sl] = -1; pts[sl].valid = false; }

            // position-owning thread: turn the accumulated dot products of a finished key into offset gradients
            auto flush = [&](int sl) {
                if (!DEFORM || doff == nullptr || key[sl] < 0) return;
                __syncwarp();
                if (p_ok) {
                    const float* tp = tot + (sl * 32 + lane) * SM::kTotStride;
                    float tv[NC];
#pragma unroll
                    for (int e = 0; e < NC; ++e) tv[e] = tp[e];
                    float gr[D];
                    if (pts[sl].valid) {
                        interp_grad<float, D>(pts[sl], tv, gr);
                    } else {
                        const float stot = tp[NC];
#pragma unroll
                        for (int a = 0; a < D; ++a) gr[a] = (D == 3 && g.oob) ? oob_term<float>(g, pts[sl].p[a], stot) : 0.f;
                    }
                    float* dst = doff + ((size_t)op.n * g.dg * g.kv * D + (size_t)key[sl] * D) * g.ov + op.opos;
#pragma unroll
                    for (int a = 0; a < D; ++a)
                        if (gr[a] != 0.f) atomicAdd(dst + (size_t)a * g.ov, gr[a]);
                }
            };

            for (int cc = 0; cc < kColsPerWarp / 32; ++cc) {
                const int col0 = part * kColsPerWarp + cc * 32;
                if (col0 >= NW) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + b * 256 + col0, v);
                tmem_ld_wait();
                const int kq0 = nb * 256 + col0;
                if (kq0 >= kq_total) break;
                int nkey[NS], ch0[NS];
#pragma unroll
                for (int sl = 0; sl < NS; ++sl) {
                    nkey[sl] = -1; ch0[sl] = 0;
                    const int kq = kq0 + sl * U;
                    if (kq < kq_total) {
                        uint32_t tap, cl;
                        g.d_Cg.divmod((uint32_t)kq, tap, cl);
                        ch0[sl] = j * g.Cg + (int)cl;                 // first channel of the slot
                        nkey[sl] = DEFORM ? (int)g.d_cpg.div((uint32_t)ch0[sl]) * g.kv + (int)tap : (int)tap;
                    }
                }
#pragma unroll
                for (int sl = 0; sl < NS; ++sl) {
                    if (nkey[sl] == key[sl]) continue;
                    flush(sl);
                    key[sl] = nkey[sl];
                    // phase A: locate the point of the new key and publish it; reset the key's accumulators
                    Entry e;
#pragma unroll
                    for (int i = 0; i < NC; ++i) { e.idx[i] = -1; e.cw[i] = 0.f; }
                    const int nbase = op.n * g.iv;            // N * in volume < 2^31 (checked on the host)
                    pts[sl].valid = false;
                    if (p_ok && nkey[sl] >= 0) {
                        if (DEFORM) {
                            const int grp = nkey[sl] / g.kv, tp = nkey[sl] - grp * g.kv;
                            locate<float, D>(g, off_n, grp, tp, op, pts[sl]);
                            if (pts[sl].valid) {
                                corner_indices<float, D>(g, pts[sl], e.idx);
                                corner_weights<float, D>(pts[sl], e.cw);
#pragma unroll
                                for (int i = 0; i < NC; ++i) e.idx[i] += nbase;
                            }
                        } else {
                            int pidx;
                            if (locate_plain<D>(g, nkey[sl], op, pidx)) {
                                e.idx[0] = nbase + pidx;
                                e.cw[0] = 1.f;
                            }
                        }
                    }
                    __syncwarp();
                    const int4* src = reinterpret_cast<const int4*>(&e);
                    int4* dst = reinterpret_cast<int4*>(ent + sl * 32 + lane);
#pragma unroll
                    for (int i = 0; i < (int)(sizeof(Entry) / 16); ++i) dst[i] = src[i];
#pragma unroll
                    for (int i = 0; i <= NC; ++i) tot[(sl * 32 + lane) * SM::kTotStride + i] = 0.f;
                }
                // stage the 32 columns of this thread's position
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    *reinterpret_cast<uint4*>(colS + lane * 36 + 4 * i) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                __syncwarp();
                // phase B: the entry and the input values of row iteration rr+1 are fetched while rr is consumed
                const int cbase = ch0[my_slot] + (cq * 4) % U;        // first of this lane's 4 channels
                const bool lane_ok = nkey[my_slot] >= 0;
                constexpr int NE = DEFORM ? NC : 1;
                struct RowData {
                    float4 c4;
                    float cw[NE];
                    int idx[NE];
                    uint2 xv[NE];
                    int valid;
                };
                auto fetch = [&](int rr, RowData& rd) {
                    const int row = rr * 4 + r4;
                    const Entry* ep = ent + my_slot * 32 + row;
                    rd.c4 = *reinterpret_cast<const float4*>(colS + row * 36 + cq * 4);
#pragma unroll
                    for (int i = 0; i < (NE + 3) / 4; ++i) {
                        const int4 ti = reinterpret_cast<const int4*>(ep->idx)[i];
                        const float4 tw = reinterpret_cast<const float4*>(ep->cw)[i];
                        const int ii[4] = {ti.x, ti.y, ti.z, ti.w};
                        const float ww[4] = {tw.x, tw.y, tw.z, tw.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (4 * i + k < NE) {
                                rd.idx[4 * i + k] = ii[k];
                                rd.cw[4 * i + k] = ww[k];
                            }
                        }
                    }
                    // unsigned 32 x 32 -> 64-bit products (one multiply-add each); plain C++ so that the pointers
                    // stay provably global
                    rd.valid = (lane_ok && rd.idx[0] >= 0) ? 1 : 0;
                    const __nv_bfloat16* xb = xcl + cbase;
#pragma unroll
                    for (int e = 0; e < NE; ++e)
                        rd.xv[e] = (want_x && rd.valid)
                                       ? __ldg(reinterpret_cast<const uint2*>(xb + (uint64_t)(uint32_t)rd.idx[e] * (uint32_t)g.C))
                                       : make_uint2(0, 0);
                };
                auto consume = [&](int rr, const RowData& rd) {
                    const int row = rr * 4 + r4;
                    float d[NC];
#pragma unroll
                    for (int e = 0; e < NC; ++e) d[e] = 0.f;
                    float sabs = 0.f;
                    if (rd.valid) {
                        float* db = dxcl + cbase;
#pragma unroll
                        for (int e = 0; e < NE; ++e) {
                            if (want_x) {
                                float a = fmaf(rd.c4.x, bf16_lo(rd.xv[e].x), 0.f);
                                a = fmaf(rd.c4.y, bf16_hi(rd.xv[e].x), a);
                                a = fmaf(rd.c4.z, bf16_lo(rd.xv[e].y), a);
                                d[e] = fmaf(rd.c4.w, bf16_hi(rd.xv[e].y), a);
                            }
                            if (dxcl != nullptr) {
                                const float wv = rd.cw[e];
                                atomicAdd(reinterpret_cast<float4*>(db + (uint64_t)(uint32_t)rd.idx[e] * (uint32_t)g.C),
                                          make_float4(wv * rd.c4.x, wv * rd.c4.y, wv * rd.c4.z, wv * rd.c4.w));
                            }
                        }
                    } else if (DEFORM && D == 3 && g.oob && lane_ok) {
                        sabs = fabsf(rd.c4.x) + fabsf(rd.c4.y) + fabsf(rd.c4.z) + fabsf(rd.c4.w);
                    }
                    if (want_x) {
                        // transposing butterfly over the LG lanes that share the key: each step halves the set of
                        // corners a lane is responsible for; `base` is the first corner this lane ends up holding
                        int width = NC, base = 0;
#pragma unroll
                        for (int bit = LG / 2; bit >= 1; bit >>= 1) {
                            if (width > 1) {
                                const int hw = width / 2;
#pragma unroll
                                for (int i = 0; i < NC / 2; ++i) {
                                    if (i < hw) {
                                        const float keep = (cq & bit) ? d[hw + i] : d[i];
                                        const float send = (cq & bit) ? d[i] : d[hw + i];
                                        d[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                                    }
                                }
                                if (cq & bit) base += hw;
                                width = hw;
                            } else {
                                d[0] += __shfl_xor_sync(0xffffffffu, d[0], bit);
                            }
                        }
                        // lanes that hold a duplicate after the plain-add steps (2-D with 8 lanes) stay silent
                        const bool writer = (NC >= LG) || ((cq & (LG / NC - 1)) == 0);
                        if (writer) {
                            float* tp = tot + (my_slot * 32 + row) * SM::kTotStride + base;
#pragma unroll
                            for (int i = 0; i < NC; ++i)
                                if (i < width) tp[i] += d[i];
                        }
                        if (D == 3 && g.oob) {
#pragma unroll
                            for (int bit = LG / 2; bit >= 1; bit >>= 1) sabs += __shfl_xor_sync(0xffffffffu, sabs, bit);
                            if ((cq & (LG - 1)) == 0) tot[(my_slot * 32 + row) * SM::kTotStride + NC] += sabs;
                        }
                    }
                };
                if constexpr (D == 2 || !DEFORM || EW == 8) {
                    RowData ra, rb;
                    fetch(0, ra);
#pragma unroll
                    for (int rr = 0; rr < 8; rr += 2) {
                        fetch(rr + 1, rb);
                        consume(rr, ra);
                        if (rr + 2 < 8) fetch(rr + 2, ra);
                        consume(rr + 1, rb);
                    }
                } else {
                    // 3-D with 16 epilogue warps: one row at a time (register budget), the warps overlap each other
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) {
                        RowData ra;
                        fetch(rr, ra);
                        consume(rr, ra);
                    }
                }
            }
#pragma unroll
            for (int sl = 0; sl < NS; ++sl) flush(sl);
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

// Channel granularity of the (deformable group, tap) keys if the transposed epilogue can take the problem, else 0.
inline int dgrad_key_unit(const Geom& g, int deform) {
    int u = 32;
    if (g.Cg < u) u = g.Cg;
    if (deform && g.cpg < u) u = g.cpg;
    if (u != 32 && u != 16) return 0;
    if (g.Cg % u != 0) return 0;
    if (deform && g.cpg % u != 0) return 0;
    return u;
}

template <int D, bool DEFORM, int EW, int U>
int launch_tc_dgrad_t(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* dpk,
                      const uint8_t* wpk, float* dxcl, float* doff, cudaStream_t st) {
    const DgDims d = dg_dims(g);
    const int smem = Dg2Smem<D, DEFORM, EW, U>::kTotal;
    static_assert(Dg2Smem<D, DEFORM, EW, U>::kTotal <= kSmemLimit, "dgrad epilogue staging does not fit");
    auto kern = tc_dgrad_kernel<D, DEFORM, EW, U>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    const long long tiles = (long long)g.G * d.PT * d.NB;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kern<<<grid, 32 * (2 + EW), smem, st>>>(g, xcl, off, dpk, wpk, dxcl, doff, d.MT, d.NB, d.NW, d.OC, d.PC2, d.PT);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <int D, bool DEFORM>
int launch_tc_dgrad(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* dpk,
                    const uint8_t* wpk, float* dxcl, float* doff, cudaStream_t st) {
    const int u = dgrad_key_unit(g, DEFORM ? 1 : 0);
    if (u == 32) return launch_tc_dgrad_t<D, DEFORM, 16, 32>(g, xcl, off, dpk, wpk, dxcl, doff, st);
    // two keys per chunk double the per-warp staging: 8 epilogue warps
    if (u == 16) return launch_tc_dgrad_t<D, DEFORM, 8, 16>(g, xcl, off, dpk, wpk, dxcl, doff, st);
    return launch_tc_dgrad_rowwise<D, DEFORM>(g, xcl, off, dpk, wpk, dxcl, doff, st);
}
