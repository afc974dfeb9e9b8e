// Weight gradient on tcgen05, direct-sampling variant (included by dcn_tc.cu inside its anonymous namespace):
// each producer thread locates its own sampling points.  Fallback of dcn_tc_wgrad2.cuh for problems whose
// coordinate table does not fit in shared memory; also defines pack_dy and the work decomposition.
//
//   dW[o, k'] += sum over positions P of dy[o, P] * sample(k', P)          k' = tap * Cg + c
//
// GEMM view: M = output channels (128-row tiles, up to two per CTA), N = a block of up to 256 k' columns,
// K = output positions, 64 per pipeline stage.  One CTA owns one (group, o-block, k'-block) and a slice of
// the position range; partial sums are added with 16-byte fp32 reductions to the packed scratch dwpk[o][k']
// (tiny and L2-resident), which unpack_dw folds into dW afterwards.
//   A operand: dy, bf16, pre-packed by pack_dy into swizzled [128 o][64 P] tiles  -> K-major, bulk-copied
//   B operand: sampled patch, [64 P rows][64 k' per 128-byte row] sub-tiles        -> MN-major, produced here
#pragma once

constexpr int kWgStages = 3;
constexpr int kWgNMax = 256;
// elements of one position split's slice of the packed dW scratch; `items` = G * MB * NB (the kernels' gridDim.x)
__host__ __device__ inline size_t wg_slice_elems(unsigned items) { return (size_t)items * 256 * kWgNMax; }
constexpr int kWgThreads = 32 * (2 + kProducerWarps + kEpilogueWarps);

struct WgSmem {
    // per stage: A0 | A1 (16 KB each) | B (4 sub-tiles of 8 KB)
    static constexpr int kStageBytes = 2 * kTileBytes + 4 * 8192;
    static constexpr int kBarOffset = kWgStages * kStageBytes;
    static constexpr int kTotal = kBarOffset + (2 * kWgStages + 1) * 8 + 16;
};

// dy [N, O, ov] fp32 -> bf16 tiles [G][MT][PC][128 o rows x 64 positions], swizzled; rows >= Og and
// positions >= P are zero.  Used by both backward kernels.
// If absmax_bits is not null it is raised to the bit pattern of max|dy| (non-negative floats order like their bits).
__global__ void __launch_bounds__(256)
pack_dy(const Geom g, const float* __restrict__ dy, uint8_t* __restrict__ dpk, int MT, long long PC,
        unsigned int* __restrict__ absmax_bits) {
    const long long pc = blockIdx.x;
    const int mt = blockIdx.y % MT, j = blockIdx.y / MT;
    uint8_t* dst = dpk + (((size_t)j * MT + mt) * PC + pc) * kTileBytes;
    const int lane = threadIdx.x % 32, wrp = threadIdx.x / 32;
    // lane handles positions 2*lane, 2*lane+1 of the 64; each warp walks rows wrp, wrp+8, ...
    const long long P0 = pc * 64 + 2 * lane;
    uint32_t n0 = 0, op0 = 0, n1 = 0, op1 = 0;
    const bool ok0 = P0 < g.P, ok1 = P0 + 1 < g.P;
    if (ok0) g.d_ov.divmod((uint32_t)P0, n0, op0);
    if (ok1) g.d_ov.divmod((uint32_t)(P0 + 1), n1, op1);
    float mx = 0.f;
    // both positions in one sample and 8-byte aligned (even ov, aligned dy): one 8-byte load per row
    const bool pair = ok1 && n0 == n1 && (g.ov & 1) == 0 && (reinterpret_cast<uintptr_t>(dy) & 7) == 0;
    for (int row = wrp; row < 128; row += 8) {      // (forcing this loop to unroll 8-fold measured 20 % slower)
        const int ol = mt * 128 + row;
        float a = 0.f, b = 0.f;
        if (ol < g.Og) {
            const int o = j * g.Og + ol;
            if (pair) {
                const float2 t = __ldg(reinterpret_cast<const float2*>(dy + ((size_t)n0 * g.O + o) * g.ov + op0));
                a = t.x; b = t.y;
            } else {
                if (ok0) a = __ldg(dy + ((size_t)n0 * g.O + o) * g.ov + op0);
                if (ok1) b = __ldg(dy + ((size_t)n1 * g.O + o) * g.ov + op1);
            }
        }
        mx = fmaxf(mx, fmaxf(fabsf(a), fabsf(b)));
        const uint32_t chunk = lane / 4;            // 8 positions per 16-byte chunk
        *reinterpret_cast<uint32_t*>(dst + swz_offset(row, chunk) + (lane % 4) * 4) = pack_bf16x2(a, b);
    }
    if (absmax_bits != nullptr) {
        __shared__ unsigned int blk_max;
        if (threadIdx.x == 0) blk_max = 0u;
        __syncthreads();
        const unsigned int m = __reduce_max_sync(0xffffffffu, __float_as_uint(mx));
        if (lane == 0 && m != 0) atomicMax(&blk_max, m);
        __syncthreads();
        if (threadIdx.x == 0 && blk_max != 0) atomicMax(absmax_bits, blk_max);
    }
}

// Same tiles from a channels-last dy [N * ov positions][O]: a thread packs 8 consecutive positions of one
// output channel (one 16-byte chunk); consecutive threads take consecutive channels, so the reads coalesce.
__global__ void __launch_bounds__(256)
pack_dy_cl(const Geom g, const float* __restrict__ dy, uint8_t* __restrict__ dpk, int MT, long long PC) {
    const long long pc = blockIdx.x;
    const int mt = blockIdx.y % MT, j = blockIdx.y / MT;
    uint8_t* dst = dpk + (((size_t)j * MT + mt) * PC + pc) * kTileBytes;
    for (int item = threadIdx.x; item < 128 * 8; item += 256) {
        const int row = item % 128, chunk = item / 128;
        const int ol = mt * 128 + row;
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const long long P = pc * 64 + chunk * 8 + e;
            v[e] = (ol < g.Og && P < g.P) ? __ldg(dy + (size_t)P * g.O + j * g.Og + ol) : 0.f;
        }
        *reinterpret_cast<uint4*>(dst + swz_offset(row, chunk)) =
            make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    }
}

inline int launch_pack_dy(const Geom& g, const float* dy, uint8_t* dpk, int MT, long long PC, cudaStream_t st,
                          unsigned int* absmax_bits = nullptr) {
    const dim3 grid((unsigned)PC, (unsigned)(g.G * MT));
    if (g.cl) pack_dy_cl<<<grid, 256, 0, st>>>(g, dy, dpk, MT, PC);
    else pack_dy<<<grid, 256, 0, st>>>(g, dy, dpk, MT, PC, absmax_bits);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <int D, bool DEFORM>
__global__ void __launch_bounds__(kWgThreads, 1)
tc_wgrad_direct_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const float* __restrict__ off,
                const uint8_t* __restrict__ dpk, float* __restrict__ dw, const int MT, const int MB,
                const int NB, const int NW, const long long PC, const int chunks_per_split) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + WgSmem::kBarOffset);
    uint64_t* empty = full + kWgStages;
    uint64_t* acc_full = empty + kWgStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    // work item of this CTA
    const int nb = blockIdx.x % NB;                     // k' block
    const int mb = (blockIdx.x / NB) % MB;              // o block (two 128-row tiles)
    const int j = blockIdx.x / NB / MB;                 // conv group
    const int mtb = (MT - mb * 2) >= 2 ? 2 : 1;
    const long long c_begin = (long long)blockIdx.y * chunks_per_split;
    long long c_end = c_begin + chunks_per_split;
    if (c_end > PC) c_end = PC;
    const int n_chunks = (int)(c_end - c_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWgStages; ++s) {
            mbar_init(&full[s], kProducerWarps + 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
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
    const uint32_t idesc = make_idesc(128, NW, 0, 1);   // A K-major, B MN-major

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < n_chunks && ok; ++it) {
                const uint32_t s = it % kWgStages;
                ok = mbar_wait(&full[s], (it / kWgStages) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_base = smem_u32(smem + s * WgSmem::kStageBytes);
                const uint32_t b_base = a_base + 2 * kTileBytes;
                for (int mt = 0; mt < mtb; ++mt) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t ad = make_desc(a_base + mt * kTileBytes + k * 32, 16, 1024);
                        const uint64_t bd = make_desc(b_base + k * 2048, 8192, 1024);
                        umma_bf16(tmem_base + mt * 256, ad, bd, idesc, (it > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(acc_full);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < n_chunks && ok; ++it) {
                const uint32_t s = it % kWgStages;
                ok = mbar_wait(&empty[s], ((it / kWgStages) & 1) ^ 1);
                if (!ok) break;
                mbar_arrive_expect_tx(&full[s], (uint32_t)(mtb * kTileBytes));
                for (int mt = 0; mt < mtb; ++mt) {
                    const uint8_t* src = dpk + (((size_t)j * MT + mb * 2 + mt) * PC + (c_begin + it)) * kTileBytes;
                    bulk_g2s(smem + s * WgSmem::kStageBytes + mt * kTileBytes, src, kTileBytes, &full[s]);
                }
            }
        }
    } else if (warp < 2 + kProducerWarps) {
        const int ptid = threadIdx.x - 64;          // 0..255
        const int cj = ptid % 32;                   // k' chunk column (8 channels) inside the block
        const int row0 = ptid / 32;                 // rows row0 + 8*i
        const int kp = nb * kWgNMax + cj * 8;
        const bool kok = (cj * 8 < NW) && kp < g.kv * g.Cg;
        uint32_t tap = 0, cl = 0;
        g.d_Cg.divmod((uint32_t)(kok ? kp : 0), tap, cl);
        const int c = j * g.Cg + (int)cl;
        const int grp = (int)g.d_cpg.div((uint32_t)c);
        const uint32_t sub_off = (uint32_t)(cj / 8) * 8192u;
        bool ok = true;
        for (int it = 0; it < n_chunks && ok; ++it) {
            const uint32_t s = it % kWgStages;
            const long long Pc = (c_begin + it) * 64;
            uint4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = make_uint4(0, 0, 0, 0);
                const long long P = Pc + row0 + 8 * i;
                if (kok && P < g.P) {
                    const OutPos op = decompose_pos(g, P);
                    v[i] = sample_chunk<D, DEFORM>(g, xcl, off, op, (int)tap, c, grp);
                }
            }
            ok = mbar_wait(&empty[s], ((it / kWgStages) & 1) ^ 1);
            if (!ok) break;
            if (cj * 8 < NW) {
                const uint32_t b_base = smem_u32(smem + s * WgSmem::kStageBytes + 2 * kTileBytes) + sub_off;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    st_shared_v4(b_base + swz_offset(row0 + 8 * i, cj % 8), v[i].x, v[i].y, v[i].z, v[i].w);
            }
            fence_proxy_async_smem();
            mbar_arrive_warp(&full[s]);
        }
    } else {
        const int q = warp & 3;
        if (n_chunks > 0 && mbar_wait(acc_full, 0)) {
            tc_fence_after();
            for (int mt = 0; mt < mtb; ++mt) {
                const int ol = (mb * 2 + mt) * 128 + q * 32 + lane;
                const bool o_ok = ol < g.Og;
                // partial sums of this position split: plain stores into its slice of the packed scratch
                // dwpk[split][G][MB*256 rows][NB*256 columns] (added up in split order by unpack_dw)
                float* dwo = dw + (size_t)blockIdx.y * wg_slice_elems(gridDim.x) +
                             ((size_t)j * MB * 256 + (o_ok ? ol : 0)) * ((size_t)NB * kWgNMax) + (size_t)nb * kWgNMax;
                for (int cc = 0; cc < NW / 32; ++cc) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + mt * 256 + cc * 32, v);
                    tmem_ld_wait();
                    if (!o_ok) continue;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int kq = nb * kWgNMax + cc * 32 + 4 * i;
                        if (kq < g.kv * g.Cg)
                            *reinterpret_cast<float4*>(dwo + cc * 32 + 4 * i) =
                                make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                            __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                    }
                }
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

struct WgDims {
    int MT, MB, NB, NW;
    long long PC;
    int splits, cps;
};

inline WgDims wg_dims(const Geom& g) {
    WgDims d;
    d.MT = (g.Og + 127) / 128;
    d.MB = (d.MT + 1) / 2;
    const int kq = g.kv * g.Cg;
    d.NB = (kq + kWgNMax - 1) / kWgNMax;
    d.NW = kq >= kWgNMax ? kWgNMax : ((kq + 63) / 64) * 64;
    d.PC = 2 * ((g.P + 127) / 128);     // 64-position chunks, even count (shared tile layout with dgrad)
    const long long items = (long long)g.G * d.MB * d.NB;
    long long splits = sm_count() / items;      // floor: the whole grid must fit in one wave (one CTA per SM)
    if (splits > d.PC) splits = d.PC;
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    d.cps = (int)((d.PC + splits - 1) / splits);
    d.splits = (int)((d.PC + d.cps - 1) / d.cps);
    return d;
}

// dwpk[split][G][rows][cols] (k' = tap * Cg + c along the columns) -> dW [O][Cg][kv] of the reference layout, the
// position splits added in split order (deterministic); ACC adds to dW (the separate weight-gradient entry point
// accumulates), else dW is overwritten.
template <bool ACC>
__global__ void __launch_bounds__(256)
unpack_dw(const Geom g, const float* __restrict__ dwpk, float* __restrict__ dw, int rows, int cols, int splits,
          size_t slice) {
    const long long total = (long long)g.O * g.Cg * g.kv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int tap = (int)(i % g.kv);
        const long long oc = i / g.kv;
        const int c = (int)(oc % g.Cg);
        const int o = (int)(oc / g.Cg);
        const int j = o / g.Og, ol = o - j * g.Og;
        const float* src = dwpk + ((size_t)j * rows + ol) * cols + (size_t)tap * g.Cg + c;
        // loads in batches of eight (independent, all in flight), additions in split order
        float v = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) t[u] = (s0 + u < splits) ? __ldg(src + (size_t)(s0 + u) * slice) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (s0 + u < splits) v = (s0 + u == 0) ? t[u] : v + t[u];
        }
        if (ACC) dw[i] += v;
        else dw[i] = v;
    }
}

inline size_t dwpk_bytes(const Geom& g) {
    const WgDims d = wg_dims(g);
    return (size_t)d.splits * wg_slice_elems(g.G * d.MB * d.NB) * sizeof(float);
}

template <bool ACC>
int dwpk_fold(const Geom& g, const float* dwpk, float* dw, cudaStream_t st) {
    const WgDims d = wg_dims(g);
    const long long total = (long long)g.O * g.Cg * g.kv;
    const int blocks = (int)((total + 255) / 256 < 16 * sm_count() ? (total + 255) / 256 : 16 * sm_count());
    unpack_dw<ACC><<<blocks, 256, 0, st>>>(g, dwpk, dw, d.MB * 256, d.NB * kWgNMax, d.splits,
                                           wg_slice_elems(g.G * d.MB * d.NB));
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

template <int D, bool DEFORM>
int launch_tc_wgrad_direct(const Geom& g, const __nv_bfloat16* xcl, const float* off, const uint8_t* dpk, float* dw,
                    cudaStream_t st) {
    const WgDims d = wg_dims(g);
    const int smem = WgSmem::kTotal + 1024;
    auto kern = tc_wgrad_direct_kernel<D, DEFORM>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    dim3 grid((unsigned)(g.G * d.MB * d.NB), (unsigned)d.splits);
    kern<<<grid, kWgThreads, smem, st>>>(g, xcl, off, dpk, dw, d.MT, d.MB, d.NB, d.NW, d.PC, d.cps);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
