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
// Taken when key boundaries fall on multiples of 32 channels (Cg and cpg multiples of 32); the code also handles
// 16-channel keys (two keys per chunk), which the dispatcher currently leaves to the row-wise variant.
#pragma once

constexpr int kDg2Stages = 3;

template <int D, bool DEFORM>
struct alignas(16) DgEntry {
    int idx[1 << D];
    float cw[1 << D];
    int n;            // sample index
    int valid;
    int pad[2];
};

template <int D, bool DEFORM>
struct Dg2Smem {
    static constexpr int kStageBytes = 3 * kTileBytes;                         // A 16 KB | B 32 KB
    static constexpr int kStagesBytes = kDg2Stages * kStageBytes;
    static constexpr int kColFloats = 32 * 36;                                 // per warp: 32 rows x (32 + 4 pad)
    static constexpr int kEntryBytes = 2 * 32 * (int)sizeof(DgEntry<D, DEFORM>);   // per warp: 2 slots x 32 rows
    static constexpr int kWarpBytes = kColFloats * 4 + kEntryBytes;
    static constexpr int kBarOffset = kStagesBytes + kDgEpiWarps * kWarpBytes;
    static constexpr int kTotal = kBarOffset + (2 * kDg2Stages + 4) * 8 + 16;
};

template <int D, bool DEFORM>
__global__ void __launch_bounds__(kDgThreads, 1)
tc_dgrad_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const float* __restrict__ off,
                const uint8_t* __restrict__ dpk, const uint8_t* __restrict__ wpk, float* __restrict__ dxcl,
                float* __restrict__ doff, const int MT, const int NB, const int NW, const int OC,
                const long long PC2, const long long PT, const int u) {
    using SM = Dg2Smem<D, DEFORM>;
    using Entry = DgEntry<D, DEFORM>;
    constexpr int NC = 1 << D;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
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
            mbar_init(&acc_empty[b], kDgEpiWarps * 32);
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
        const int ew = warp - 2;                        // 0..7
        const int q = warp & 3;                         // tensor-memory lane quarter
        const int half = ew / 4;                        // which 128-column half of the tile
        float* colS = reinterpret_cast<float*>(smem + SM::kStagesBytes + (size_t)ew * SM::kWarpBytes);   // [32][36]
        Entry* ent = reinterpret_cast<Entry*>(colS + SM::kColFloats);                                     // [2][32]
        const int kq_total = g.kv * g.Cg;
        const int ns = 32 / u;                          // keys (slots) per 32-column chunk: 1 or 2
        // phase-B coordinates of this lane
        const int r4 = lane >> 3, cq = lane & 7;
        const int my_slot = (cq * 4) / u;
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

            // per-slot state: phase A keeps the located point, phase B the running dot products
            int key[2] = {-1, -1};
            Pt<float, D> pts[2];
            pts[0].valid = pts[1].valid = false;
            float T[8][NC];                // [row iteration][corner] for this lane's slot
            float S[8];
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                S[rr] = 0.f;
#pragma unroll
                for (int e = 0; e < NC; ++e) T[rr][e] = 0.f;
            }

            // reduce this lane's accumulators over the lanes of its key and hand the totals of slot `sl` to the
            // position-owning threads, which turn them into offset-gradient components
            auto flush = [&](int sl) {
                if (!DEFORM || doff == nullptr) return;
                __syncwarp();
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    float vals[NC + 1];
#pragma unroll
                    for (int e = 0; e < NC; ++e) vals[e] = T[rr][e];
                    vals[NC] = S[rr];
#pragma unroll
                    for (int e = 0; e <= NC; ++e) {
                        float v = vals[e];
                        v += __shfl_xor_sync(0xffffffffu, v, 1);
                        v += __shfl_xor_sync(0xffffffffu, v, 2);
                        if (u == 32) v += __shfl_xor_sync(0xffffffffu, v, 4);
                        vals[e] = v;
                    }
                    if (my_slot == sl && (cq * 4) % u == 0) {
#pragma unroll
                        for (int e = 0; e <= NC; ++e) colS[(rr * 4 + r4) * 36 + e] = vals[e];
                    }
                    if (my_slot == sl) {
                        S[rr] = 0.f;
#pragma unroll
                        for (int e = 0; e < NC; ++e) T[rr][e] = 0.f;
                    }
                }
                __syncwarp();
                if (p_ok && key[sl] >= 0) {
                    float tot[NC];
#pragma unroll
                    for (int e = 0; e < NC; ++e) tot[e] = colS[lane * 36 + e];
                    const float stot = colS[lane * 36 + NC];
                    float gr[D];
                    if (pts[sl].valid) {
                        interp_grad<float, D>(pts[sl], tot, gr);
                    } else {
#pragma unroll
                        for (int a = 0; a < D; ++a) gr[a] = (D == 3 && g.oob) ? oob_term<float>(g, pts[sl].p[a], stot) : 0.f;
                    }
                    float* dst = doff + ((size_t)op.n * g.dg * g.kv * D + (size_t)key[sl] * D) * g.ov + op.opos;
#pragma unroll
                    for (int a = 0; a < D; ++a)
                        if (gr[a] != 0.f) atomicAdd(dst + (size_t)a * g.ov, gr[a]);
                }
                __syncwarp();
            };

            for (int cc = 0; cc < 4; ++cc) {
                const int col0 = half * 128 + cc * 32;
                if (col0 >= NW) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + b * 256 + col0, v);
                tmem_ld_wait();
                const int kq0 = nb * 256 + col0;
                if (kq0 >= kq_total) break;
                // keys of the chunk's slots (uniform across the warp)
                int nkey[2], ch0[2];
#pragma unroll
                for (int sl = 0; sl < 2; ++sl) {
                    nkey[sl] = -1; ch0[sl] = 0;
                    const int kq = kq0 + sl * u;
                    if (sl < ns && kq < kq_total) {
                        uint32_t tap, cl;
                        g.d_Cg.divmod((uint32_t)kq, tap, cl);
                        ch0[sl] = j * g.Cg + (int)cl;
                        nkey[sl] = DEFORM ? (int)g.d_cpg.div((uint32_t)ch0[sl]) * g.kv + (int)tap : (int)tap;
                    }
                }
                // a slot whose key changes first hands over the finished key
#pragma unroll
                for (int sl = 0; sl < 2; ++sl) {
                    if (sl < ns && nkey[sl] != key[sl]) {
                        if (key[sl] >= 0) flush(sl);
                        key[sl] = nkey[sl];
                        // phase A: locate and publish
                        Entry e;
                        e.n = op.n; e.valid = 0; e.pad[0] = e.pad[1] = 0;
#pragma unroll
                        for (int i = 0; i < NC; ++i) { e.idx[i] = 0; e.cw[i] = 0.f; }
                        pts[sl].valid = false;
                        if (p_ok && nkey[sl] >= 0) {
                            if (DEFORM) {
                                const int grp = nkey[sl] / g.kv, tap = nkey[sl] - grp * g.kv;
                                locate<float, D>(g, off_n, grp, tap, op, pts[sl]);
                                if (pts[sl].valid) {
                                    corner_indices<float, D>(g, pts[sl], e.idx);
                                    corner_weights<float, D>(pts[sl], e.cw);
                                    e.valid = 1;
                                }
                            } else {
                                int pidx;
                                if (locate_plain<D>(g, nkey[sl], op, pidx)) {
                                    e.valid = 1;
                                    e.idx[0] = pidx;
                                    e.cw[0] = 1.f;
                                }
                            }
                        }
                        __syncwarp();
                        {
                            const int4* src = reinterpret_cast<const int4*>(&e);
                            int4* dst = reinterpret_cast<int4*>(ent + sl * 32 + lane);
#pragma unroll
                            for (int i = 0; i < (int)(sizeof(Entry) / 16); ++i) dst[i] = src[i];
                        }
                    }
                }
                // stage the 32 columns of this thread's position
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    *reinterpret_cast<uint4*>(colS + lane * 36 + 4 * i) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                __syncwarp();
                // phase B: the entry and the input values of row iteration rr+1 are fetched while rr is consumed
                const int cbase = ch0[my_slot] + (cq * 4) % u;          // first of this lane's 4 channels
                const bool lane_ok = nkey[my_slot] >= 0;
                constexpr int NE = DEFORM ? NC : 1;
                struct RowData {
                    float4 c4;
                    float cw[NE];
                    size_t addr[NE];
                    uint2 xv[NE];
                    int valid;
                };
                const bool want_x = DEFORM && doff != nullptr;
                auto fetch = [&](int rr, RowData& rd) {
                    const int row = rr * 4 + r4;
                    const Entry* ep = ent + my_slot * 32 + row;
                    const int4 hdr = *reinterpret_cast<const int4*>(&ep->n);      // n, valid, pad, pad
                    rd.c4 = *reinterpret_cast<const float4*>(colS + row * 36 + cq * 4);
                    rd.valid = lane_ok ? hdr.y : 0;
                    const size_t base = (size_t)hdr.x * g.iv * g.C + cbase;
#pragma unroll
                    for (int i = 0; i < (NE + 3) / 4; ++i) {
                        const int4 ti = reinterpret_cast<const int4*>(ep->idx)[i];
                        const float4 tw = reinterpret_cast<const float4*>(ep->cw)[i];
                        const int ii[4] = {ti.x, ti.y, ti.z, ti.w};
                        const float ww[4] = {tw.x, tw.y, tw.z, tw.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (4 * i + k < NE) {
                                rd.addr[4 * i + k] = base + (size_t)ii[k] * g.C;
                                rd.cw[4 * i + k] = ww[k];
                            }
                        }
                    }
#pragma unroll
                    for (int e = 0; e < NE; ++e)
                        rd.xv[e] = (want_x && rd.valid) ? __ldg(reinterpret_cast<const uint2*>(xcl + rd.addr[e])) : make_uint2(0, 0);
                };
                auto consume = [&](int rr, const RowData& rd) {
                    if (rd.valid) {
#pragma unroll
                        for (int e = 0; e < NE; ++e) {
                            if (want_x) {
                                float d = T[rr][e];
                                d = fmaf(rd.c4.x, bf16_lo(rd.xv[e].x), d); d = fmaf(rd.c4.y, bf16_hi(rd.xv[e].x), d);
                                d = fmaf(rd.c4.z, bf16_lo(rd.xv[e].y), d); d = fmaf(rd.c4.w, bf16_hi(rd.xv[e].y), d);
                                T[rr][e] = d;
                            }
                            if (dxcl != nullptr) {
                                const float wv = rd.cw[e];
                                atomicAdd(reinterpret_cast<float4*>(dxcl + rd.addr[e]),
                                          make_float4(wv * rd.c4.x, wv * rd.c4.y, wv * rd.c4.z, wv * rd.c4.w));
                            }
                        }
                    } else if (DEFORM && D == 3 && g.oob && lane_ok) {
                        S[rr] += fabsf(rd.c4.x) + fabsf(rd.c4.y) + fabsf(rd.c4.z) + fabsf(rd.c4.w);
                    }
                };
                RowData ra, rb;
                fetch(0, ra);
#pragma unroll
                for (int rr = 0; rr < 8; rr += 2) {
                    fetch(rr + 1, rb);
                    consume(rr, ra);
                    if (rr + 2 < 8) fetch(rr + 2, ra);
                    consume(rr + 1, rb);
                }
            }
#pragma unroll
            for (int sl = 0; sl < 2; ++sl)
                if (sl < ns && key[sl] >= 0) flush(sl);
            tc_fence_before();
            mbar_arrive(&acc_empty[b]);
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
    if (u != 32) return 0;      // with 16-channel keys the per-key hand-over costs more than the aggregation saves
    if (g.Cg % u != 0) return 0;
    if (deform && g.cpg % u != 0) return 0;
    return u;
}

template <int D, bool DEFORM>
int launch_tc_dgrad(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* dpk,
                    const uint8_t* wpk, float* dxcl, float* doff, cudaStream_t st) {
    const int u = dgrad_key_unit(g, DEFORM ? 1 : 0);
    if (u == 0) return launch_tc_dgrad_rowwise<D, DEFORM>(g, xcl, off, dpk, wpk, dxcl, doff, st);
    const DgDims d = dg_dims(g);
    const int smem = Dg2Smem<D, DEFORM>::kTotal + 1024;
    auto kern = tc_dgrad_kernel<D, DEFORM>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    const long long tiles = (long long)g.G * d.PT * d.NB;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kern<<<grid, kDgThreads, smem, st>>>(g, xcl, off, dpk, wpk, dxcl, doff, d.MT, d.NB, d.NW, d.OC, d.PC2, d.PT, u);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
