// Weight gradient on tcgen05 (included by dcn_tc.cu inside its anonymous namespace).
//
//   dW[o, k'] += sum over positions P of dy[o, P] * sample(k', P)          k' = tap * Cg + c
//
// GEMM view: M = output channels (128-row tiles, up to two per CTA), N = a block of up to 256 k' columns,
// K = output positions, 64 per pipeline stage.  One CTA owns one (group, o-block, k'-block) and a slice of
// the position range; partial sums are added with 16-byte fp32 reductions to a packed, zero-filled scratch
// dwpk[o][k'] (tiny and L2-resident) that unpack_dw folds into dW's [O][Cg][kv] layout afterwards.
//   A operand: dy, bf16, pre-packed by pack_dy into swizzled [128 o][64 P] tiles  -> K-major, bulk-copied
//   B operand: sampled patch, [64 P rows][64 k' per 128-byte row] sub-tiles        -> MN-major, produced here
// Warps: 0 MMA issue, 1 dy-tile loader, 2-5 coordinate warps (warp k fills the table of every 4th stage, as in
// dcn_tc_fwd.cuh; after the last table the same warps are the epilogue), 6-21 gather warps (dcn_tc_sampler.cuh).
// The k' block of a CTA is fixed, so the (deformable group, tap) key of every chunk column and the slot
// numbering are computed once.
#pragma once

constexpr int kWgCoordWarps = 4;
constexpr int kWgGatherWarps = 16;
constexpr int kWgMaxTabs = 6;
constexpr int kWgOffRing = 2 * kWgCoordWarps;       // two private offset staging buffers per coordinate warp
constexpr int kWg2Threads = 32 * (2 + kWgCoordWarps + kWgGatherWarps);

struct Wg2Ctl {
    uint64_t full[kMaxStages], empty[kMaxStages], acc_full, tab_full[kWgMaxTabs], tab_empty[kWgMaxTabs];
    uint32_t tmem_base;
    int slot_of_chunk[32];
    int key_of_slot[32];
    int nslots;
};

template <int D, bool DEFORM>
__global__ void __launch_bounds__(kWg2Threads, 1)
tc_wgrad_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const float* __restrict__ off,
                const uint8_t* __restrict__ dpk, float* __restrict__ dw, const int MT, const int MB,
                const int NB, const int NW, const long long PC, const int chunks_per_split, const int n_stages,
                const int max_slots, const int n_tabs, const int a_tiles) {
    using Entry = TabEntry<D, DEFORM>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int stage_bytes = a_tiles * kTileBytes + 4 * 8192;          // A tiles | B (4 sub-tiles of 8 KB)
    Entry* tab = reinterpret_cast<Entry*>(smem + (size_t)n_stages * stage_bytes);        // [n_tabs][max_slots][64]
    float* ostage = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tab) +
                                             (size_t)n_tabs * max_slots * 64 * sizeof(Entry));   // [kWgOffRing][max_slots][D][64]
    Wg2Ctl* ctl = reinterpret_cast<Wg2Ctl*>(ostage + (size_t)kWgOffRing * max_slots * D * 64);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    const int nb = blockIdx.x % NB;                     // k' block
    const int mb = (blockIdx.x / NB) % MB;              // o block (two 128-row tiles)
    const int j = blockIdx.x / NB / MB;                 // conv group
    const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
    const long long c_begin = (long long)blockIdx.y * chunks_per_split;
    long long c_end = c_begin + chunks_per_split;
    if (c_end > PC) c_end = PC;
    const int n_chunks = (int)(c_end - c_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl->full[s], kWgGatherWarps + 1);
            mbar_init(&ctl->empty[s], 1);
        }
        mbar_init(&ctl->acc_full, 1);
        for (int b = 0; b < kWgMaxTabs; ++b) {
            mbar_init(&ctl->tab_full[b], 1);                  // the coordinate warp that filled it
            mbar_init(&ctl->tab_empty[b], kWgGatherWarps);
        }
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&ctl->tmem_base, 512);
        tmem_relinquish();
    }
    if (warp == 2) {
        // keys of the NW/8 chunk columns of this k' block, numbered into slots (once per CTA)
        int tap_, c_;
        const int key = chunk_key(g, j, nb * kWgNMax + lane * 8, tap_, c_);
        const SlotInfo si = make_slots(key, lane, NW / 8);
        ctl->slot_of_chunk[lane] = lane < NW / 8 ? si.my_slot : 0;
        for (int sl = 0; sl < si.nslots; ++sl) {
            const int k = slot_key(si, sl);
            if (lane == 0) ctl->key_of_slot[sl] = k;
        }
        if (lane == 0) ctl->nslots = si.nslots;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    const uint32_t idesc = make_idesc(128, NW, 0, 1);   // A K-major, B MN-major
    const int nslots = ctl->nslots;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            Ring rs;
            for (int it = 0; it < n_chunks && ok; ++it, rs.next(n_stages)) {
                const uint32_t s = rs.i;
                ok = mbar_wait(&ctl->full[s], rs.ph);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_base = smem_u32(smem + (size_t)s * stage_bytes);
                const uint32_t b_base = a_base + a_tiles * kTileBytes;
                const uint64_t ad0 = make_desc(a_base, 16, 1024);       // see dcn_tc_fwd.cuh: only the start address moves
                const uint64_t bd0 = make_desc(b_base, 8192, 1024);
                for (int mt = 0; mt < mtb; ++mt) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        umma_bf16(tmem_base + mt * 256, ad0 + (uint64_t)((mt * kTileBytes + k * 32) >> 4),
                                  bd0 + (uint64_t)((k * 2048) >> 4), idesc, (it > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&ctl->empty[s]);
            }
            if (ok) umma_commit(&ctl->acc_full);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            Ring rs;
            for (int it = 0; it < n_chunks && ok; ++it, rs.next(n_stages)) {
                const uint32_t s = rs.i;
                ok = mbar_wait(&ctl->empty[s], rs.ph ^ 1u);
                if (!ok) break;
                mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)(mtb * kTileBytes));
                for (int mt = 0; mt < mtb; ++mt) {
                    const uint8_t* src = dpk + (((size_t)j * MT + mb * 2 + mt) * PC + (c_begin + it)) * kTileBytes;
                    bulk_g2s(smem + (size_t)s * stage_bytes + mt * kTileBytes, src, kTileBytes, &ctl->full[s]);
                }
            }
        }
    } else if (warp < 2 + kWgCoordWarps) {
        // ------------------------------------------------ coordinate warps, then epilogue
        // Warp cw fills the tables of chunks cw, cw + 4, ...; a thread owns position rows lane and lane + 32.  The
        // offsets of a chunk are fetched (4-byte cp.async) into one of the warp's two staging buffers while the
        // warp's previous chunk is being filled.
        const int cw = warp - 2;
        float* my_ost = ostage + (size_t)cw * 2 * max_slots * D * 64;
        auto prefetch = [&](int itp, uint32_t buf) {
            if (DEFORM && itp < n_chunks) {
                float* dst = my_ost + (size_t)buf * max_slots * D * 64;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int row = lane + 32 * i;
                    const long long P = (c_begin + itp) * 64 + row;
                    if (P >= g.P) continue;
                    const OutPos op = decompose_pos(g, P);
                    for (int sl = 0; sl < nslots; ++sl) {
                        const int key = ctl->key_of_slot[sl];
                        if (key < 0) continue;
                        uint32_t grp, tap;
                        g.d_kv.divmod((uint32_t)key, grp, tap);
                        const float* src = offset_ptr<float, D>(g, offset_block<float, D>(g, off, op.n), (int)grp, (int)tap, op);
#pragma unroll
                        for (int a = 0; a < D; ++a) cp_async4(dst + (size_t)(sl * D + a) * 64 + row, src + (size_t)a * g.ov);
                    }
                }
            }
            cp_async_commit();
        };
        prefetch(cw, 0);
        prefetch(cw + kWgCoordWarps, 1);
        bool ok = true;
        Ring rt;
        for (int i = 0; i < cw; ++i) rt.next(n_tabs);
        uint32_t k = 0;
        for (int it = cw; it < n_chunks && ok; it += kWgCoordWarps, ++k) {
            const uint32_t tb = rt.i;
            ok = mbar_wait(&ctl->tab_empty[tb], rt.ph ^ 1u);
            if (!ok) break;
            cp_async_wait<1>();             // this chunk's offsets have landed; the next chunk's may be in flight
            const float* src = my_ost + (size_t)(k & 1u) * max_slots * D * 64;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int row = lane + 32 * i;
                const long long P = (c_begin + it) * 64 + row;
                const bool pok = P < g.P;
                const OutPos op = decompose_pos(g, pok ? P : 0);
                for (int sl = 0; sl < nslots; ++sl) {
                    const int key = ctl->key_of_slot[sl];
                    float offv[D];
#pragma unroll
                    for (int a = 0; a < D; ++a) offv[a] = (DEFORM && key >= 0 && pok) ? src[(size_t)(sl * D + a) * 64 + row] : 0.f;
                    fill_entry_from<D, DEFORM>(g, offv, op, pok, key, tab + ((size_t)tb * max_slots + sl) * 64 + row);
                }
            }
            mbar_arrive_warp(&ctl->tab_full[tb]);
            prefetch(it + 2 * kWgCoordWarps, k & 1u);      // into the buffer just read
            for (int i = 0; i < kWgCoordWarps; ++i) rt.next(n_tabs);
        }
        cp_async_wait<0>();
        // ------------------------------------------------ epilogue: partial dW of this CTA -> atomics
        const int q = warp & 3;
        if (ok && n_chunks > 0 && mbar_wait(&ctl->acc_full, 0)) {
            tc_fence_after();
            for (int mt = 0; mt < mtb; ++mt) {
                const int ol = (mb * 2 + mt) * 128 + q * 32 + lane;
                const bool o_ok = ol < g.Og;
                // The partial sums of this position split go to ITS slice of the packed scratch
                // dwpk[split][G][MB*256 rows][NB*256 columns] with plain 16-byte stores: every element a slice's
                // reader touches is written exactly once, and unpack_dw adds the slices in split order, so dW does
                // not depend on the order in which the CTAs finish.
                float* dwo = dw + (size_t)blockIdx.y * wg_slice_elems(gridDim.x) +
                             ((size_t)j * MB * 256 + (o_ok ? ol : 0)) * ((size_t)NB * kWgNMax) + (size_t)nb * kWgNMax;
                for (int cc = 0; cc < NW / 16; ++cc) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + mt * 256 + cc * 16, v);
                    tmem_ld_wait();
                    if (!o_ok) continue;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int kq = nb * kWgNMax + cc * 16 + 4 * i;
                        if (kq < g.kv * g.Cg)
                            *reinterpret_cast<float4*>(dwo + cc * 16 + 4 * i) =
                                make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                            __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------ gather warps
        const int gtid = threadIdx.x - 32 * (2 + kWgCoordWarps);  // 0..511
        const int cj = gtid % 32;                   // chunk column (8 channels) inside the k' block
        const int row0 = gtid / 32;                 // rows row0 + RS*i, i = 0..RT-1
        constexpr int NQ = DEFORM ? (1 << D) : 1;
        constexpr int RS = kWgGatherWarps;                         // row stride between a thread's rows
        constexpr int RT = 64 / RS;                                // rows per thread and stage
        constexpr int RPP = (D == 3 && DEFORM) ? 1 : 2;            // rows per pass: 8 loads in flight
        constexpr int PPS = RT / RPP;                              // passes per stage
        constexpr bool kOverlap = false;                           // one pass at a time: 80 registers per thread
        const bool col_ok = cj * 8 < NW;
        int tap_, cch;
        chunk_key(g, j, nb * kWgNMax + cj * 8, tap_, cch);
        const int sl = ctl->slot_of_chunk[cj];
        const uint32_t sub_off = (uint32_t)(cj / 8) * 8192u + (uint32_t)(a_tiles * kTileBytes);
        struct Pass {
            uint4 q[RPP][NQ];
            float w[RPP][NQ];
            uint32_t s, ph;
            int h;
        };
        const uint32_t tab_s = smem_u32(tab);
        const uint32_t pix_bytes = (uint32_t)g.C * 2u;
        int cit = 0, ch = 0;
        Ring rtab, rstg;
        bool failed = false;
        auto issue = [&](Pass& p) -> bool {
            if (cit >= n_chunks || failed) return false;
            const uint32_t tb = rtab.i;
            if (ch == 0) {
                if (!mbar_wait(&ctl->tab_full[tb], rtab.ph)) { failed = true; return false; }
            }
            const uint32_t trow_s = tab_s + ((tb * (uint32_t)max_slots + (uint32_t)sl) * 64u) * (uint32_t)sizeof(Entry);
#pragma unroll
            for (int r = 0; r < RPP; ++r) {
                const int row = row0 + RS * (ch * RPP + r);
                const long long P = (c_begin + cit) * 64 + row;
                uint32_t n = 0;
                if (P < g.P) n = g.d_ov.div((uint32_t)P);
                if (col_ok) {
                    gather_issue_s<D, DEFORM>(trow_s + (uint32_t)row * (uint32_t)sizeof(Entry),
                                              xcl + (uint64_t)(n * (uint32_t)g.iv) * (uint32_t)g.C + cch, pix_bytes, p.q[r], p.w[r]);
                } else {
#pragma unroll
                    for (int e = 0; e < NQ; ++e) { p.q[r][e] = make_uint4(0, 0, 0, 0); p.w[r][e] = 0.f; }
                }
            }
            p.s = rstg.i;
            p.ph = rstg.ph;
            p.h = ch;
            if (ch == PPS - 1) mbar_arrive_warp(&ctl->tab_empty[tb]);
            if (++ch == PPS) { ch = 0; ++cit; rtab.next(n_tabs); rstg.next(n_stages); }
            return true;
        };
        auto finish = [&](Pass& p) -> bool {
            const uint32_t s = p.s;
            if (p.h == 0) {
                if (!mbar_wait(&ctl->empty[s], p.ph ^ 1u)) { failed = true; return false; }
            }
            if (col_ok) {
                const uint32_t b_base = smem_u32(smem + (size_t)s * stage_bytes) + sub_off;
#pragma unroll
                for (int r = 0; r < RPP; ++r) {
                    const uint4 v = gather_finish_w<D, DEFORM>(p.q[r], p.w[r]);
                    st_shared_v4(b_base + swz_offset(row0 + RS * (p.h * RPP + r), cj % 8), v.x, v.y, v.z, v.w);
                }
            }
            if (p.h == PPS - 1) {
                fence_proxy_async_smem();
                mbar_arrive_warp(&ctl->full[s]);
            }
            return true;
        };
        if constexpr (kOverlap) {
            Pass pa, pb;
            bool ha = issue(pa);
            while (ha) {
                const bool hb = issue(pb);
                if (!finish(pa)) break;
                if (!hb) break;
                ha = issue(pa);
                if (!finish(pb)) break;
            }
        } else {
            Pass pa;
            while (issue(pa)) {
                if (!finish(pa)) break;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Largest number of distinct keys among the chunk columns of any 256-wide k' block.
inline int max_slots_per_block(const Geom& g) { return max_slots_per_chunk(g, 32); }

template <int D, bool DEFORM>
int launch_tc_wgrad(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* dpk, float* dw,
                    cudaStream_t st) {
    const WgDims d = wg_dims(g);
    const int a_tiles = d.MT >= 2 ? 2 : 1;
    const int stage_bytes = a_tiles * kTileBytes + 4 * 8192;
    const int max_slots = max_slots_per_block(g);
    const size_t tab_one = (size_t)max_slots * 64 * sizeof(TabEntry<D, DEFORM>);
    const size_t ost_bytes = (size_t)kWgOffRing * max_slots * D * 64 * sizeof(float);
    auto need = [&](int stages, int tabs) {
        return (long long)stages * stage_bytes + (long long)tabs * tab_one + ost_bytes + sizeof(Wg2Ctl) + 1024;
    };
    // table ring of at least four (see launch_tc_forward), preferably deeper than the four coordinate warps
    int stages = 0, n_tabs = 0;
    const int pref[][2] = {{3, 6}, {3, 5}, {2, 6}, {2, 5}, {3, 4}, {2, 4}};
    for (const auto& c : pref) {
        if (need(c[0], c[1]) <= kSmemLimit) { stages = c[0]; n_tabs = c[1]; break; }
    }
    if (stages == 0 || max_slots > 32) return launch_tc_wgrad_direct<D, DEFORM>(g, xcl, off, dpk, dw, st);
    const int smem = (int)need(stages, n_tabs);
    auto kern = tc_wgrad_kernel<D, DEFORM>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    dim3 grid((unsigned)(g.G * d.MB * d.NB), (unsigned)d.splits);
    kern<<<grid, kWg2Threads, smem, st>>>(g, xcl, off, dpk, dw, d.MT, d.MB, d.NB, d.NW, d.PC, d.cps, stages, max_slots,
                                          n_tabs, a_tiles);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
