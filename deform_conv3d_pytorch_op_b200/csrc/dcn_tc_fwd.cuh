// Forward implicit GEMM on tcgen05 (included by dcn_tc.cu inside its anonymous namespace).
//
//   y[o, P] = sum over k' of W[o, k'] * sample(k', P)  (+ bias)            k' = tap * Cg + c
//
// Persistent CTAs, one per SM; 6 + GW warps:
//   warp 0       MMA issue (one elected lane) and tensor-memory allocation
//   warp 1       weight-tile loader (bulk async copies, one elected lane)
//   warps 2-5    coordinate warps (dcn_tc_sampler.cuh).  Warp k fills the whole table of every 4th pipeline stage
//                (k, k+4, ...): the chain offsets -> coordinates -> corner table of one stage is long and serial,
//                so four stages are in production at once.  The same warps drain finished accumulators
//                (tensor memory -> registers -> (+bias) -> y) whenever they have no table to fill, so the
//                epilogue costs no warps of its own.
//   warps 6..    GW gather warps: build the sampled, interpolated patch tile straight into the swizzled B
//                operand, all of them on the same stage (splitting them into groups that take alternate
//                stages measured slower).
// Tile = (conv group, block of up to 256 output channels, 128 output positions).  The sampled operand of a
// K chunk is shared by both 128-row halves of the output-channel block.
#pragma once

constexpr int kMaxStages = 4;
constexpr int kFwdCoordWarps = 4;               // forward: coordinate + epilogue warps, one per tensor-memory lane quarter
constexpr int fwd_threads(int gw) { return 32 * (2 + kFwdCoordWarps + gw); }
constexpr int kFwdStageBytes = 3 * kTileBytes;      // A0 | A1 | B
constexpr int kSmemLimit = 232448;                   // 227 KB opt-in maximum per CTA

constexpr int kFwdMaxTabs = 6;
constexpr int kFwdOffRing = 2 * kFwdCoordWarps;   // two private offset staging buffers per coordinate warp

struct FwdCtl {            // lives behind the stages, the tables and the offset staging ring
    uint64_t full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2], tab_full[kFwdMaxTabs], tab_empty[kFwdMaxTabs];
    uint32_t tmem_base;
    int slot_of_chunk[kFwdMaxTabs][8];
};

// How the work items of the persistent CTAs map to (tile, K range).  Items [0, T0) split every tile KS0 ways
// (KS0 = 1: whole tiles); items from T0 on split the tiles from tile1 on KS1 ways.  The second region is the
// tail of a grid that does not divide evenly: the tiles left over after the last full wave are split along K so
// that the last wave is a fraction of a tile long instead of a whole one.  Split tiles add into a zero-filled y.
struct FwdSplit {
    long long T0, tile1, n_items;
    int KS0, cpk0, KS1, cpk1;
    int acc;            // y already holds a partial result: every tile is added to it with reductions
};
struct FwdItem {
    long long tt;       // tile index ((j * MB + mb) * PT + pt)
    int ks, kc0, kc1;   // split number and its K chunks [kc0, kc1)
    bool atomic;        // partial sum of a split tile
};
__device__ __forceinline__ FwdItem fwd_item(const FwdSplit& sp, long long t, int KC) {
    const bool tail = t >= sp.T0;
    const long long r = tail ? t - sp.T0 : t;
    const int KS = tail ? sp.KS1 : sp.KS0, cpk = tail ? sp.cpk1 : sp.cpk0;
    FwdItem it;
    it.ks = (int)(r % KS);
    it.tt = (tail ? sp.tile1 : 0) + r / KS;
    it.kc0 = it.ks * cpk;
    it.kc1 = (it.kc0 + cpk < KC) ? it.kc0 + cpk : KC;
    it.atomic = KS > 1 || sp.acc != 0;
    return it;
}

template <int D, bool DEFORM, int GW>
__global__ void __launch_bounds__(fwd_threads(GW), 1)
tc_forward_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const float* __restrict__ off,
                  const uint8_t* __restrict__ wpk, const float* __restrict__ bias, float* __restrict__ y,
                  const int KC, const int MT, const int MB, const long long PT, const int n_stages,
                  const int max_slots, const int n_tabs, const FwdSplit sp) {
    // Work items: see FwdSplit.  With few position tiles and a long K every tile is split (small batches, late
    // layers of a network); otherwise only the tiles of the last, partial wave are.
    using Entry = TabEntry<D, DEFORM>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    Entry* tab = reinterpret_cast<Entry*>(smem + n_stages * kFwdStageBytes);          // [n_tabs][max_slots][128]
    float* ostage = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tab) +
                                             (size_t)n_tabs * max_slots * 128 * sizeof(Entry));   // [kFwdOffRing][max_slots][D][128]
    FwdCtl* ctl = reinterpret_cast<FwdCtl*>(ostage + (size_t)kFwdOffRing * max_slots * D * 128);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl->full[s], GW + 1);            // one arrival per gather warp + the loader
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], kFwdCoordWarps);
        }
        for (int b = 0; b < kFwdMaxTabs; ++b) {
            mbar_init(&ctl->tab_full[b], 1);             // the coordinate warp that filled it
            mbar_init(&ctl->tab_empty[b], GW);           // the gather warps that read it
        }
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&ctl->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    const long long n_tiles = sp.n_items;
    constexpr uint32_t kIdesc = make_idesc(128, kTileN, 0, 0);

    if (warp == 0) {
        // ------------------------------------------------ MMA issue
        if (lane == 0) {
            uint32_t tl = 0;
            Ring rs;
            bool ok = true;
            for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tl) {
                const FwdItem wi = fwd_item(sp, t, KC);
                const long long tt = wi.tt;
                const int mb = (int)((tt / PT) % MB);
                const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
                const int kc0 = wi.kc0, kc1 = wi.kc1;
                const uint32_t b = tl & 1;
                ok = mbar_wait(&ctl->acc_empty[b], ((tl >> 1) & 1) ^ 1);
                tc_fence_after();
                for (int kc = kc0; kc < kc1 && ok; ++kc, rs.next(n_stages)) {
                    const uint32_t s = rs.i;
                    ok = mbar_wait(&ctl->full[s], rs.ph);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem + s * kFwdStageBytes);
                    const uint32_t b_base = a_base + 2 * kTileBytes;
                    // one descriptor per operand and stage; the K step and the second M tile only move the
                    // start-address field (units of 16 bytes), which cannot carry out of its 14 bits
                    const uint64_t ad0 = make_desc(a_base, 16, 1024);
                    const uint64_t bd0 = make_desc(b_base, 16, 1024);
                    for (int mt = 0; mt < mtb; ++mt) {
#pragma unroll
                        for (int k = 0; k < kTileK / 16; ++k) {
                            umma_bf16(tmem_base + b * 256 + mt * 128, ad0 + (uint64_t)((mt * kTileBytes + k * 32) >> 4),
                                      bd0 + (uint64_t)((k * 32) >> 4), kIdesc, (kc > kc0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&ctl->empty[s]);
                }
                if (ok) umma_commit(&ctl->acc_full[b]);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ weight loader
        if (lane == 0) {
            Ring rs;
            bool ok = true;
            for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const FwdItem wi = fwd_item(sp, t, KC);
                const long long tt = wi.tt;
                const int mb = (int)((tt / PT) % MB);
                const int j = (int)(tt / PT / MB);
                const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
                const int kc0 = wi.kc0, kc1 = wi.kc1;
                for (int kc = kc0; kc < kc1 && ok; ++kc, rs.next(n_stages)) {
                    const uint32_t s = rs.i;
                    ok = mbar_wait(&ctl->empty[s], rs.ph ^ 1u);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)(mtb * kTileBytes));
                    for (int mt = 0; mt < mtb; ++mt) {
                        const uint8_t* src = wpk + ((size_t)(j * MT + mb * 2 + mt) * KC + kc) * kTileBytes;
                        bulk_g2s(smem + s * kFwdStageBytes + mt * kTileBytes, src, kTileBytes, &ctl->full[s]);
                    }
                }
            }
        }
    } else if (warp < 2 + kFwdCoordWarps) {
        // ------------------------------------------------ coordinate + epilogue warps
        const int cw = warp - 2;                    // takes stages cw, cw + 4, ... of this CTA's stage sequence
        const int q = warp & 3;                     // tensor-memory lane quarter this warp may access
        constexpr int CR = 4;                       // table rows per thread: lane + 32 * i
        struct Cur {
            long long t, pt;
            int kc, kc_end, j;
            uint32_t tl;            // how many tiles of this CTA came before t
        };
        auto init_tile = [&](Cur& c) {
            const FwdItem wi = fwd_item(sp, c.t, KC);
            c.pt = wi.tt % PT;
            c.j = (int)(wi.tt / PT / MB);
            c.kc = wi.kc0;
            c.kc_end = wi.kc1;
        };
        auto skip = [&](Cur& c, int n) {            // n stages further
            for (int i = 0; i < n && c.t < n_tiles; ++i) {
                if (++c.kc == c.kc_end) {
                    c.t += gridDim.x;
                    ++c.tl;
                    if (c.t < n_tiles) init_tile(c);
                }
            }
        };
        auto stage_slots = [&](const Cur& c) {
            int tap_, c_;
            const int key = chunk_key(g, c.j, c.kc * kTileK + (lane & 7) * 8, tap_, c_);
            return make_slots(key, lane, 8);
        };
        // Offsets of a stage are fetched with 4-byte cp.async into one of this warp's two staging buffers while
        // the warp's previous stage is being filled, so their latency is off the critical path.
        float* my_ost = ostage + (size_t)cw * 2 * max_slots * D * 128;
        auto prefetch = [&](const Cur& c, uint32_t buf) {
            if (DEFORM && c.t < n_tiles) {
                const SlotInfo si = stage_slots(c);
                float* dst = my_ost + (size_t)buf * max_slots * D * 128;
                for (int sl = 0; sl < si.nslots; ++sl) {
                    const int key = slot_key(si, sl);
                    if (key < 0) continue;
                    uint32_t grp, tap;
                    g.d_kv.divmod((uint32_t)key, grp, tap);
#pragma unroll
                    for (int i = 0; i < CR; ++i) {
                        const long long P = c.pt * kTileN + lane + 32 * i;
                        if (P >= g.P) continue;
                        const OutPos op = decompose_pos(g, P);
                        const float* src = offset_ptr<float, D>(g, offset_block<float, D>(g, off, op.n), (int)grp, (int)tap, op);
#pragma unroll
                        for (int a = 0; a < D; ++a)
                            cp_async4(dst + (size_t)(sl * D + a) * 128 + lane + 32 * i, src + (size_t)a * g.ov);
                    }
                }
            }
            cp_async_commit();
        };
        Cur cur;
        cur.t = blockIdx.x; cur.pt = 0; cur.kc = 0; cur.kc_end = 0; cur.j = 0; cur.tl = 0;
        if (cur.t < n_tiles) init_tile(cur);
        skip(cur, cw);
        Ring rt;
        for (int i = 0; i < cw; ++i) rt.next(n_tabs);
        prefetch(cur, 0);
        {
            Cur pre = cur;
            skip(pre, kFwdCoordWarps);
            prefetch(pre, 1);
        }
        uint32_t it = 0;                // stages this warp has filled
        long long et = blockIdx.x;      // next tile whose accumulator this warp drains
        uint32_t etl = 0;               // ... and how many tiles of this CTA came before it
        bool waiting = false;
        long long t0 = 0;
        while (true) {
            const bool more = cur.t < n_tiles;
            if (!more && et >= n_tiles) break;
            const bool tab_free = more && mbar_try_wait(&ctl->tab_empty[rt.i], rt.ph ^ 1u);
            // Drain an accumulator when there is no table to fill (the ring is full, or the tables are done) or
            // when the tables of the tile that needs the accumulator's buffer are about to be filled.
            if (et < n_tiles && (!tab_free || cur.tl >= etl + 2) &&
                mbar_try_wait(&ctl->acc_full[etl & 1], (etl >> 1) & 1)) {
                waiting = false;
                tc_fence_after();
                const uint32_t b = etl & 1;
                const FwdItem wi = fwd_item(sp, et, KC);
                const int ks = wi.ks;
                const bool plain = !wi.atomic;
                const long long tt = wi.tt;
                const long long pt = tt % PT;
                const int mb = (int)((tt / PT) % MB);
                const int j = (int)(tt / PT / MB);
                const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
                for (int mt = 0; mt < mtb; ++mt) {
                    const int ol = (mb * 2 + mt) * 128 + q * 32 + lane;      // output channel within the group
                    const bool o_ok = ol < g.Og;
                    const int o = j * g.Og + ol;
                    const float bv = (bias != nullptr && o_ok && ks == 0) ? __ldg(bias + o) : 0.f;
#pragma unroll 1
                    for (int cc = 0; cc < kTileN / 16; ++cc) {
                        uint32_t v[16];
                        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + b * 256 + mt * 128 + cc * 16, v);
                        tmem_ld_wait();
                        const long long P0 = pt * kTileN + cc * 16;
                        if (!o_ok || P0 >= g.P) continue;
                        if (g.cl) {
                            // channels-last y: the 32 lanes of the warp hold 32 consecutive channels of a position
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                if (P0 + i < g.P) {
                                    float* d1 = y + (size_t)(P0 + i) * g.O + o;
                                    if (plain) *d1 = __uint_as_float(v[i]) + bv;
                                    else atomicAdd(d1, __uint_as_float(v[i]) + bv);
                                }
                            }
                            continue;
                        }
                        uint32_t n0, opos0;
                        g.d_ov.divmod((uint32_t)P0, n0, opos0);
                        float* dst = y + ((size_t)n0 * g.O + o) * g.ov + opos0;
                        const bool fast = (opos0 + 16 <= (uint32_t)g.ov) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
                        if (fast) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float4 val = make_float4(__uint_as_float(v[4 * i]) + bv, __uint_as_float(v[4 * i + 1]) + bv,
                                                               __uint_as_float(v[4 * i + 2]) + bv, __uint_as_float(v[4 * i + 3]) + bv);
                                if (plain) *reinterpret_cast<float4*>(dst + 4 * i) = val;
                                else atomicAdd(reinterpret_cast<float4*>(dst + 4 * i), val);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const long long P = P0 + i;
                                if (P < g.P) {
                                    uint32_t n, opos;
                                    g.d_ov.divmod((uint32_t)P, n, opos);
                                    float* d1 = y + ((size_t)n * g.O + o) * g.ov + opos;
                                    if (plain) *d1 = __uint_as_float(v[i]) + bv;
                                    else atomicAdd(d1, __uint_as_float(v[i]) + bv);
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive_warp(&ctl->acc_empty[b]);
                et += gridDim.x;
                ++etl;
                continue;
            }
            if (tab_free) {
                waiting = false;
                cp_async_wait<1>();             // this stage's offsets have landed; the next stage's may be in flight
                const uint32_t tb = rt.i;
                const SlotInfo si = stage_slots(cur);
                if (lane < 8) ctl->slot_of_chunk[tb][lane] = si.my_slot;
                const float* src = my_ost + (size_t)(it & 1u) * max_slots * D * 128;
                for (int sl = 0; sl < si.nslots; ++sl) {
                    const int key = slot_key(si, sl);
#pragma unroll
                    for (int i = 0; i < CR; ++i) {
                        const long long P = cur.pt * kTileN + lane + 32 * i;
                        const bool pok = P < g.P;
                        const OutPos op = decompose_pos(g, pok ? P : 0);
                        float offv[D];
#pragma unroll
                        for (int a = 0; a < D; ++a)
                            offv[a] = (DEFORM && key >= 0 && pok) ? src[(size_t)(sl * D + a) * 128 + lane + 32 * i] : 0.f;
                        fill_entry_from<D, DEFORM>(g, offv, op, pok, key, tab + ((size_t)tb * max_slots + sl) * 128 + lane + 32 * i);
                    }
                }
                mbar_arrive_warp(&ctl->tab_full[tb]);
                skip(cur, kFwdCoordWarps);
                for (int i = 0; i < kFwdCoordWarps; ++i) rt.next(n_tabs);
                {
                    Cur pre = cur;              // the stage after the next one goes into the buffer just read
                    skip(pre, kFwdCoordWarps);
                    prefetch(pre, it & 1u);
                }
                ++it;
                continue;
            }
            // nothing to do yet: bounded wait for either event
            __nanosleep(200);
            if (!waiting) {
                waiting = true;
                t0 = clock64();
            } else if (clock64() - t0 > kWaitCycles) {
                atomicOr(&g_tc_status, 1u);
                break;
            }
        }
        cp_async_wait<0>();
    } else {
        // ------------------------------------------------ gather warps
        // Within a thread a stage is produced in passes of RPP rows; where the registers allow it the loads
        // of the next pass are in flight while the current one is interpolated and stored.
        const int gtid = threadIdx.x - 32 * (2 + kFwdCoordWarps);   // 0..GW*32-1
        const int chunk = gtid % 8;                 // 16-byte chunk of the 128-byte row
        const int row0 = gtid / 8;                  // rows row0 + RS*i, i = 0..RT-1
        constexpr int NQ = DEFORM ? (1 << D) : 1;
        constexpr int RT = 128 * 8 / (GW * 32);     // rows per thread and stage
        constexpr int RS = GW * 4;                  // row stride between a thread's rows
        constexpr int RPP = (RT >= 2 && !(D == 3 && DEFORM && GW > 8)) ? 2 : 1;   // rows per pass (16 or 8 loads)
        constexpr int PPS = RT / RPP;               // passes per stage
        // 2-D: two passes in flight (16 loads); 3-D: one pass already has 16 loads in flight, and two would
        // not fit the register file.
        constexpr bool kOverlap = (D == 2 || !DEFORM) && PPS >= 2 && GW <= 10;
        struct Pass {
            uint4 q[RPP][NQ];
            float w[RPP][NQ];
            uint32_t s, ph;     // operand stage of this pass and the phase of its barriers
            int h;
        };
        // issue cursor: stage sequence (tile, K chunk) of this CTA
        long long ct = blockIdx.x, cpt = 0;
        int ckc = 0, ckc_end = 0, ch = 0, cj = 0, cc = 0, csl = 0;
        Ring rtab, rstg;            // table buffer and operand stage of the issue cursor
        bool failed = false;
        const uint32_t tab_s = smem_u32(tab);
        const uint32_t pix_bytes = (uint32_t)g.C * 2u;
        const __nv_bfloat16* xbase[RT];         // channels-last base of the sample of each of this thread's rows
        auto init_tile = [&]() {
            const FwdItem wi = fwd_item(sp, ct, KC);
            cpt = wi.tt % PT;
            cj = (int)(wi.tt / PT / MB);
            ckc = wi.kc0;
            ckc_end = wi.kc1;
#pragma unroll
            for (int i = 0; i < RT; ++i) {
                const long long P = cpt * kTileN + row0 + RS * i;
                uint32_t n = 0;
                if (P < g.P) n = g.d_ov.div((uint32_t)P);
                xbase[i] = xcl + (uint64_t)(n * (uint32_t)g.iv) * (uint32_t)g.C;
            }
        };
        auto next_stage = [&]() {
            rtab.next(n_tabs);
            rstg.next(n_stages);
            if (++ckc == ckc_end) {
                ct += gridDim.x;
                if (ct < n_tiles) init_tile();
            }
        };
        if (ct < n_tiles) init_tile();
        auto issue = [&](Pass& p) -> bool {
            if (ct >= n_tiles || failed) return false;
            const uint32_t tb = rtab.i;
            if (ch == 0) {
                const bool okw = mbar_wait(&ctl->tab_full[tb], rtab.ph); if (!okw) { failed = true; return false; }
                csl = ctl->slot_of_chunk[tb][chunk];
                const int kp = ckc * kTileK + chunk * 8;
                uint32_t tap, cl;
                g.d_Cg.divmod((uint32_t)(kp < g.kv * g.Cg ? kp : 0), tap, cl);
                cc = cj * g.Cg + (int)cl;
            }
            const uint32_t trow_s = tab_s + ((tb * (uint32_t)max_slots + (uint32_t)csl) * 128u) * (uint32_t)sizeof(Entry);
#pragma unroll
            for (int hh = 0; hh < PPS; ++hh) {
                if (hh == ch) {
#pragma unroll
                    for (int r = 0; r < RPP; ++r) {
                        const int i = hh * RPP + r;
                        gather_issue_s<D, DEFORM>(trow_s + (uint32_t)(row0 + RS * i) * (uint32_t)sizeof(Entry),
                                                  xbase[i] + cc, pix_bytes, p.q[r], p.w[r]);
                    }
                }
            }
            p.s = rstg.i;
            p.ph = rstg.ph;
            p.h = ch;
            if (ch == PPS - 1) mbar_arrive_warp(&ctl->tab_empty[tb]);   // this warp is done with the stage's table
            if (++ch == PPS) {
                ch = 0;
                next_stage();
            }
            return true;
        };
        auto finish = [&](Pass& p) -> bool {
            const uint32_t s = p.s;
            if (p.h == 0) {
                const bool okw = mbar_wait(&ctl->empty[s], p.ph ^ 1u); if (!okw) { failed = true; return false; }
            }
            const uint32_t b_base = smem_u32(smem + s * kFwdStageBytes + 2 * kTileBytes);
#pragma unroll
            for (int r = 0; r < RPP; ++r) {
                const uint4 v = gather_finish_w<D, DEFORM>(p.q[r], p.w[r]);
                st_shared_v4(b_base + swz_offset(row0 + RS * (p.h * RPP + r), chunk), v.x, v.y, v.z, v.w);
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

    // teardown: every role has left its loop (normally or after a bounded wait gave up)
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Largest number of distinct (deformable group, tap) keys any 64-wide K chunk touches.
inline int max_slots_per_chunk(const Geom& g, int cols_per_chunk) {
    const int kq = g.kv * g.Cg;
    int best = 1;
    for (int j = 0; j < g.G; ++j) {
        for (int k0 = 0; k0 < kq; k0 += cols_per_chunk * 8) {
            int slots = 0, prev = -2;
            for (int c8 = 0; c8 < cols_per_chunk; ++c8) {
                const int kp = k0 + c8 * 8;
                int key = -1;
                if (kp < kq) {
                    const int tap = kp / g.Cg, cl = kp % g.Cg;
                    key = ((j * g.Cg + cl) / g.cpg) * g.kv + tap;
                }
                if (c8 == 0 || key != prev) ++slots;
                prev = key;
            }
            if (slots > best) best = slots;
        }
    }
    return best;
}

// accumulate: add to what y holds (no zero fill; every tile leaves through reductions)
template <int D, bool DEFORM>
int launch_tc_forward(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* wpk,
                      const float* bias, float* y, cudaStream_t st, bool accumulate = false) {
    const TcDims d = tc_dims(g);
    const int max_slots = max_slots_per_chunk(g, 8);
    const size_t tab_one = (size_t)max_slots * 128 * sizeof(TabEntry<D, DEFORM>);
    const size_t ost_bytes = (size_t)kFwdOffRing * max_slots * D * 128 * sizeof(float);
    auto need = [&](int stages, int tabs) {
        return (long long)stages * kFwdStageBytes + (long long)tabs * tab_one + ost_bytes + sizeof(FwdCtl) + 1024;
    };
    // The four coordinate warps work on four tables at once and wait on the barriers of a table buffer by phase
    // parity, which is only sound while no warp runs two laps of the ring ahead of another: with the tables
    // consumed in order that holds for rings of four and more.  A ring of five or six comes before the fourth
    // operand stage (the stage count hardly matters: the producers, not the MMA, bound a stage).
    int stages = 0, n_tabs = 0;
    const int pref[][2] = {{4, 6}, {4, 5}, {3, 6}, {3, 5}, {4, 4}, {3, 4}, {2, 6}, {2, 5}, {2, 4}};
    for (const auto& c : pref) {
        if (need(c[0], c[1]) <= kSmemLimit) { stages = c[0]; n_tabs = c[1]; break; }
    }
    if (stages == 0) {
        if (accumulate) return -5;                  // (the direct variant overwrites)
        return launch_tc_forward_direct<D, DEFORM>(g, xcl, off, wpk, bias, y, st);   // table too large
    }
    const int smem = (int)need(stages, n_tabs);
    constexpr int GW = 16;
    auto kern = tc_forward_kernel<D, DEFORM, GW>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    // split the K range when there are fewer tiles than SMs (small batches / late layers of a network)
    const long long base_tiles = (long long)g.G * d.MB * d.PT;
    const int S = sm_count();
    FwdSplit sp;
    sp.acc = accumulate ? 1 : 0;
    sp.KS0 = 1;
    if (base_tiles * 2 <= S) {
        sp.KS0 = (int)(S / base_tiles);
        if (sp.KS0 > d.KC / 8) sp.KS0 = d.KC / 8;          // at least 8 chunks per split
        if (sp.KS0 < 1) sp.KS0 = 1;
    }
    sp.cpk0 = (d.KC + sp.KS0 - 1) / sp.KS0;
    sp.KS0 = (d.KC + sp.cpk0 - 1) / sp.cpk0;
    sp.T0 = base_tiles * sp.KS0;
    sp.tile1 = base_tiles;
    sp.KS1 = 1;
    sp.cpk1 = d.KC;
    sp.n_items = sp.T0;
    if (sp.KS0 > 1) {
        if (!accumulate && cudaMemsetAsync(y, 0, (size_t)g.N * g.O * g.ov * sizeof(float), st) != cudaSuccess) return -5;
    } else if (!accumulate && g.G * d.MB == 1 && base_tiles > S && base_tiles % S != 0) {
        // Tail of an uneven grid: the R tiles left after the last full wave are split along K into as many pieces
        // as there are SMs to take them.  With one (group, channel block) the tile index is the position tile, so
        // the tail is the position range [P0, P) and only that part of y is zero-filled.
        const long long R = base_tiles % S;
        int ks1 = (int)(S / R);
        if (ks1 > d.KC / 8) ks1 = d.KC / 8;
        if (ks1 >= 2) {
            sp.cpk1 = (d.KC + ks1 - 1) / ks1;
            sp.KS1 = (d.KC + sp.cpk1 - 1) / sp.cpk1;
            sp.T0 = base_tiles - R;
            sp.tile1 = sp.T0;
            sp.n_items = sp.T0 + R * sp.KS1;
            const long long P0 = sp.T0 * kTileN;
            if (g.cl) {
                if (cudaMemsetAsync(y + (size_t)P0 * g.O, 0, (size_t)(g.P - P0) * g.O * sizeof(float), st) != cudaSuccess)
                    return -5;
            } else {
                long long n0 = P0 / g.ov;
                const long long o0 = P0 % g.ov;
                if (o0 != 0) {      // the sample the tail starts in: the positions [o0, ov) of every channel
                    if (cudaMemset2DAsync(y + (size_t)n0 * g.O * g.ov + o0, (size_t)g.ov * sizeof(float), 0,
                                          (size_t)(g.ov - o0) * sizeof(float), (size_t)g.O, st) != cudaSuccess)
                        return -5;
                    ++n0;
                }
                if (n0 < g.N &&
                    cudaMemsetAsync(y + (size_t)n0 * g.O * g.ov, 0, (size_t)(g.N - n0) * g.O * g.ov * sizeof(float), st) !=
                        cudaSuccess)
                    return -5;
            }
        }
    }
    const int grid = (int)(sp.n_items < S ? sp.n_items : S);
    kern<<<grid, fwd_threads(GW), smem, st>>>(g, xcl, off, wpk, bias, y, d.KC, d.MT, d.MB, d.PT, stages, max_slots, n_tabs, sp);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
