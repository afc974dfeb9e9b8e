// Forward implicit GEMM, direct-sampling variant (included by dcn_tc.cu inside its anonymous namespace).
// Same tiling, operand layout and MMA issue as dcn_tc_fwd.cuh, but each producer thread locates its own
// sampling points instead of reading a coordinate table.  Used when a K chunk touches so many distinct
// (deformable group, tap) keys (very small channel groups) that the coordinate table would not fit in shared
// memory next to the operand stages.
#pragma once

constexpr int kDirectStages = 4;
constexpr int kFwdDirectThreads = 32 * (2 + kProducerWarps + kEpilogueWarps);

// ---------------------------------------------------------------------------------------------------
// Forward implicit GEMM.  Persistent CTAs, one per SM; warp roles:
//   warp 0      MMA issue (one elected lane) and tensor-memory allocation
//   warp 1      weight-tile loader (bulk async copies, one elected lane)
//   warps 2-9   producers: sample the input patch tile straight into the swizzled B operand
//   warps 10-13 epilogue: tensor memory -> registers -> (+bias) -> y
// Tile = (conv group, block of up to 256 output channels, 128 output positions).  The sampled operand of a
// K chunk is shared by both 128-row halves of the output-channel block.
// ---------------------------------------------------------------------------------------------------
struct FwdDirectSmem {
    // per stage: A0 | A1 | B, 16 KB each
    static constexpr int kStageBytes = 3 * kTileBytes;
    static constexpr int kBarOffset = kDirectStages * kStageBytes;
    // barriers: full[S], empty[S], acc_full[2], acc_empty[2]; then the tensor-memory base address
    static constexpr int kTotal = kBarOffset + (2 * kDirectStages + 4) * 8 + 16;
};

template <int D, bool DEFORM>
__global__ void __launch_bounds__(kFwdDirectThreads, 1)
tc_forward_direct_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const float* __restrict__ off,
                  const uint8_t* __restrict__ wpk, const float* __restrict__ bias, float* __restrict__ y,
                  const int KC, const int MT, const int MB, const long long PT) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + FwdDirectSmem::kBarOffset);
    uint64_t* empty = full + kDirectStages;
    uint64_t* acc_full = empty + kDirectStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDirectStages; ++s) {
            mbar_init(&full[s], kProducerWarps + 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], kEpilogueWarps);
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

    const long long n_tiles = (long long)g.G * MB * PT;
    constexpr uint32_t kIdesc = make_idesc(128, kTileN, 0, 0);

    if (warp == 0) {
        // ------------------------------------------------ MMA issue
        if (lane == 0) {
            uint32_t it = 0, tl = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tl) {
                const int mb = (int)((t / PT) % MB);
                const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
                const uint32_t b = tl & 1;
                ok = mbar_wait(&acc_empty[b], ((tl >> 1) & 1) ^ 1);
                tc_fence_after();
                for (int kc = 0; kc < KC && ok; ++kc, ++it) {
                    const uint32_t s = it % kDirectStages;
                    ok = mbar_wait(&full[s], (it / kDirectStages) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem + s * FwdDirectSmem::kStageBytes);
                    const uint32_t b_base = a_base + 2 * kTileBytes;
                    for (int mt = 0; mt < mtb; ++mt) {
#pragma unroll
                        for (int k = 0; k < kTileK / 16; ++k) {
                            const uint64_t ad = make_desc(a_base + mt * kTileBytes + k * 32, 16, 1024);
                            const uint64_t bd = make_desc(b_base + k * 32, 16, 1024);
                            umma_bf16(tmem_base + b * 256 + mt * 128, ad, bd, kIdesc, (kc > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[b]);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ weight loader
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int mb = (int)((t / PT) % MB);
                const int j = (int)(t / PT / MB);
                const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
                for (int kc = 0; kc < KC && ok; ++kc, ++it) {
                    const uint32_t s = it % kDirectStages;
                    ok = mbar_wait(&empty[s], ((it / kDirectStages) & 1) ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&full[s], (uint32_t)(mtb * kTileBytes));
                    for (int mt = 0; mt < mtb; ++mt) {
                        const uint8_t* src = wpk + ((size_t)(j * MT + mb * 2 + mt) * KC + kc) * kTileBytes;
                        bulk_g2s(smem + s * FwdDirectSmem::kStageBytes + mt * kTileBytes, src, kTileBytes, &full[s]);
                    }
                }
            }
        }
    } else if (warp < 2 + kProducerWarps) {
        // ------------------------------------------------ producers
        const int ptid = threadIdx.x - 64;          // 0..255
        const int chunk = ptid % 8;                 // 16-byte chunk of the 128-byte row
        const int row0 = ptid / 8;                  // rows row0 + 32*i
        uint32_t it = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const long long pt = t % PT;
            const int j = (int)(t / PT / MB);
            OutPos op[4];
            bool pok[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const long long P = pt * kTileN + row0 + 32 * i;
                pok[i] = P < g.P;
                op[i] = decompose_pos(g, pok[i] ? P : 0);
            }
            for (int kc = 0; kc < KC && ok; ++kc, ++it) {
                const uint32_t s = it % kDirectStages;
                const int kp = kc * kTileK + chunk * 8;
                const bool kok = kp < g.kv * g.Cg;
                uint32_t tap = 0, cl = 0;
                g.d_Cg.divmod((uint32_t)(kok ? kp : 0), tap, cl);
                const int c = j * g.Cg + (int)cl;
                const int grp = (int)g.d_cpg.div((uint32_t)c);
                uint4 v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[i] = make_uint4(0, 0, 0, 0);
                    if (kok && pok[i]) v[i] = sample_chunk<D, DEFORM>(g, xcl, off, op[i], (int)tap, c, grp);
                }
                ok = mbar_wait(&empty[s], ((it / kDirectStages) & 1) ^ 1);
                if (!ok) break;
                const uint32_t b_base = smem_u32(smem + s * FwdDirectSmem::kStageBytes + 2 * kTileBytes);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    st_shared_v4(b_base + swz_offset(row0 + 32 * i, chunk), v[i].x, v[i].y, v[i].z, v[i].w);
                fence_proxy_async_smem();
                mbar_arrive_warp(&full[s]);
            }
        }
    } else {
        // ------------------------------------------------ epilogue
        const int q = warp & 3;                     // tensor-memory lane quarter this warp may access
        uint32_t tl = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tl) {
            const long long pt = t % PT;
            const int mb = (int)((t / PT) % MB);
            const int j = (int)(t / PT / MB);
            const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
            const uint32_t b = tl & 1;
            ok = mbar_wait(&acc_full[b], (tl >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            for (int mt = 0; mt < mtb; ++mt) {
                const int ol = (mb * 2 + mt) * 128 + q * 32 + lane;      // output channel within the group
                const bool o_ok = ol < g.Og;
                const int o = j * g.Og + ol;
                const float bv = (bias != nullptr && o_ok) ? __ldg(bias + o) : 0.f;
#pragma unroll 1
                for (int cc = 0; cc < kTileN / 32; ++cc) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + b * 256 + mt * 128 + cc * 32, v);
                    tmem_ld_wait();
                    const long long P0 = pt * kTileN + cc * 32;
                    if (!o_ok || P0 >= g.P) continue;
                    if (g.cl) {
                        // channels-last y: the 32 lanes of the warp hold 32 consecutive channels of a position
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (P0 + i < g.P) y[(size_t)(P0 + i) * g.O + o] = __uint_as_float(v[i]) + bv;
                        continue;
                    }
                    uint32_t n0, opos0;
                    g.d_ov.divmod((uint32_t)P0, n0, opos0);
                    float* dst = y + ((size_t)n0 * g.O + o) * g.ov + opos0;
                    const bool fast = (opos0 + 32 <= (uint32_t)g.ov) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
                    if (fast) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<float4*>(dst + 4 * i) =
                                make_float4(__uint_as_float(v[4 * i]) + bv, __uint_as_float(v[4 * i + 1]) + bv,
                                            __uint_as_float(v[4 * i + 2]) + bv, __uint_as_float(v[4 * i + 3]) + bv);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const long long P = P0 + i;
                            if (P < g.P) {
                                uint32_t n, opos;
                                g.d_ov.divmod((uint32_t)P, n, opos);
                                y[((size_t)n * g.O + o) * g.ov + opos] = __uint_as_float(v[i]) + bv;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_warp(&acc_empty[b]);
        }
    }

    // teardown: every role has left its loop (normally or after a bounded wait gave up)
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int D, bool DEFORM>
int launch_tc_forward_direct(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* wpk,
                      const float* bias, float* y, cudaStream_t st) {
    const TcDims d = tc_dims(g);
    const int smem = FwdDirectSmem::kTotal + 1024;
    auto kern = tc_forward_direct_kernel<D, DEFORM>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    const long long tiles = (long long)g.G * d.MB * d.PT;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kern<<<grid, kFwdDirectThreads, smem, st>>>(g, xcl, off, wpk, bias, y, d.KC, d.MT, d.MB, d.PT);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

