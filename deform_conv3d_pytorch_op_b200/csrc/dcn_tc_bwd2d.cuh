// Input and offset gradients of the 2-D deformable convolution with the input gradient accumulated in shared
// memory (included by dcn_tc.cu inside its anonymous namespace).
//
// The scatter of the input gradient (the reference's deformable_col2im_input: four fp32 atomics per sample,
// deform2d/lib/deform_conv2d_cuda_kernel.cu:205-220) is what bounds the backward pass: through global memory it
// is 925 M fp32 additions at configuration 2, and the SM -> L2 reduction path sustains 5.5 of them per clock and
// SM.  Here one CTA owns one (sample, slab of 8 input channels) at a time and keeps that slab's whole input
// plane in shared memory, so every addition is a shared-memory atomic and dX is written once.
//
// Fixed point.  Shared-memory atomics are native (one warp instruction per clock) for integers only; fp32 ones
// are compare-and-swap loops that run slower than the global path (measured).  The plane therefore accumulates
// in 32-bit fixed point: every term w * col is scaled by a power of two chosen from a bound on |col| (output
// channels per group x max|dy| x max|W|, both maxima taken by the packing pre-passes), so that one term is at
// most 2^21 and the quantisation step is 2^-21 of the largest possible term.  The magnitudes of all terms added
// to the plane are summed in a shared counter before they are added; while that sum stays below 2^30 no element
// can have overflowed and plain reductions are used.  Once it is spent, every addition looks at the element it
// found (atom with return) and an element that has reached 2^30 is exchanged with zero and its value added to
// dX in global memory at once, so the accumulation cannot overflow for any input.
//
// Bank conflicts.  The plane is stored in 2 x 2 pixel blocks of 128 bytes: word = block * 32 + class * 8 + c with
// class = (h & 1) * 2 + (w & 1), so the bank is class * 8 + c whatever the block.  The four corners of a sample
// always have four different classes (where two corners coincide, the twin of the other parity gets weight 0 and
// the coinciding one the sum of both weights).  A thread owns one output position and all 8 channels; in round
// r of 4 and step k of 8, lane l adds channel ((l & 7) + k) & 7 of its corner of class r ^ (l >> 3): the 32 lanes
// of the instruction then hit 32 different banks for any offsets, one wavefront per instruction.
//
// GEMM (per position tile of 128, 32 output channels per pipeline stage):
//   col[P, (tap, c)] = sum over o of dy[o, P] * W[o, c, tap]        N = kv * 8 columns (padded to 16)
//   A operand: dy, pack_dy tiles read MN-major (two 64-position halves)      B operand: the slab's W^T, K-major,
//   resident in shared memory for the whole (sample, slab)
// Offset gradient (the reference's deformable_col2im_offset, deform2d/lib/deform_conv2d_cuda_kernel.cu:250-347):
// the same thread reads the 4 corner rows of the slab's input plane (bf16, also in shared memory), forms the
// per-corner dot products with its 8 col values and adds the slab's share to dOffset with reductions that
// coalesce along the positions.
#pragma once

constexpr int kB2EpiWarps = 12;                       // three per tensor-memory lane quarter (four measured slower)
constexpr int kB2WQ = kB2EpiWarps / 4;                // warps per quarter: the taps of a position are dealt round-robin
constexpr int kB2Threads = 32 * (2 + kB2EpiWarps);
constexpr int kB2StageBytes = 8192;                   // 32 output channels x 128 positions of dy
constexpr int kB2TermBits = 21;                       // |one fixed-point term| <= 2^21
constexpr int kB2MaxStages = 8;

struct B2Dims {
    int SL;          // slabs of 8 channels per convolution group
    int NW;          // GEMM N: kv * 8 rounded up to a multiple of 16
    int OC;          // 64-wide chunks of the output channels of a group (weight tiles)
    int OS;          // 32-wide pipeline stages of the output channels of a group
    int MT;          // 128-row dy tiles per group
    long long PC;    // 64-position chunks of the packed dy
    int Wp, W2, H2;  // x-plane row pitch in pixels; plane size in 2 x 2 blocks
    int w_chunk;     // bytes of one weight tile: kv * 8 rows of 128 bytes
    int w_bytes, stages, plane_bytes, xs_bytes, smem_bytes;
    long long items;
};

inline B2Dims b2_dims(const Geom& g) {
    B2Dims d;
    d.SL = g.Cg / 8;
    d.NW = ((g.kv * 8 + 15) / 16) * 16;
    d.OC = (g.Og + 63) / 64;
    d.OS = (g.Og + 31) / 32;
    d.MT = (g.Og + 127) / 128;
    d.PC = 2 * ((g.P + 127) / 128);
    d.Wp = (g.in[2] + 1) / 2 * 2;
    d.W2 = d.Wp / 2;
    d.H2 = (g.in[1] + 1) / 2;
    d.w_chunk = g.kv * 1024;
    // the MMA reads NW rows of a weight tile; the rows past kv * 8 of the last tile fall into the stage ring
    d.w_bytes = d.OC * d.w_chunk;
    d.plane_bytes = d.H2 * d.W2 * 128;
    d.xs_bytes = 2 * d.H2 * d.Wp * 16;
    const int fixed = d.w_bytes + d.plane_bytes + d.xs_bytes + 512;
    int room = (kSmemLimit - fixed) / kB2StageBytes;
    d.stages = room > kB2MaxStages ? kB2MaxStages : room;
    d.smem_bytes = fixed + d.stages * kB2StageBytes;
    d.items = (long long)g.N * g.G * d.SL;
    return d;
}

// Whether the shared-memory-accumulating kernel takes the problem: 2-D deformable, up to 16 taps (two
// accumulators of kv * 8 columns), and the slab's input plane (fixed-point dX + bf16 x) and weights fit next
// to at least three pipeline stages.
inline bool b2_supported(const Geom& g, int ndim, int deform) {
    if (ndim != 2 || !deform || g.cl) return false;
    if (g.kv > 16 || g.Cg % 8 != 0 || g.cpg % 8 != 0) return false;
    return b2_dims(g).stages >= 3;
}

size_t b2_wpk_bytes(const Geom& g) {
    const B2Dims d = b2_dims(g);
    return (size_t)g.G * d.SL * d.w_bytes + 2048;     // + the rows an MMA reads past the last tile
}

// Wt [O][kv * Cg] bf16 (k' order) -> per (group, slab, 64-channel chunk of o) one K-major bf16 tile
// [kv * 8 rows][64 o], row = tap * 8 + (channel within the slab), swizzled; o >= Og is zero.  The 8 channels of a
// (slab, tap) are 16 contiguous bytes of Wt.
__global__ void __launch_bounds__(256)
pack_weight_slab(const Geom g, const __nv_bfloat16* __restrict__ wt, uint8_t* __restrict__ wpk, int SL, int OC) {
    __shared__ __align__(16) uint16_t piece[64][16 * 8 + 8];        // [o][tap * 8 + c], up to 16 taps
    const int tile = blockIdx.x;                          // (j * SL + slab) * OC + oc
    const int oc = tile % OC, slab = (tile / OC) % SL, j = tile / OC / SL;
    uint8_t* dst = wpk + (size_t)tile * g.kv * 1024;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(wt);
    for (int e = threadIdx.x; e < 64 * g.kv; e += blockDim.x) {
        const int ol = e / g.kv, tap = e - ol * g.kv;
        const int o = oc * 64 + ol;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (o < g.Og) v = __ldg(reinterpret_cast<const uint4*>(src + (size_t)(j * g.Og + o) * g.Kg + (size_t)tap * g.Cg + slab * 8));
        *reinterpret_cast<uint4*>(&piece[ol][tap * 8]) = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < g.kv * 64; e += blockDim.x) {
        const int row = e % (g.kv * 8), chunk = e / (g.kv * 8);
        uint32_t pk[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            pk[q] = (uint32_t)piece[chunk * 8 + 2 * q][row] | ((uint32_t)piece[chunk * 8 + 2 * q + 1][row] << 16);
        *reinterpret_cast<uint4*>(dst + swz_offset(row, chunk)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

// Sampling points, located once for all channel slabs of a deformable group.  One 16-byte entry per (sample,
// deformable group, tap, output position), positions contiguous:
//   x  bits 0-19 byte offset of the (lo_h, lo_w) pixel in the blocked dX plane | bits 27-28 its class
//      | bit 29 hi_w != lo_w | bit 30 hi_h != lo_h | bit 31 valid
//   y  lo_h * Wp + lo_w (pixel index in the linear x plane)      z, w  the fractions lw_h, lw_w (fp32 bits)
// An invalid point has bits 29-31 and the fractions zero and names some pixel inside the plane (the tap's
// undeformed position, clamped): the kernel adds zeros there, and spreading those zeros over the plane keeps
// them from colliding on one address.
// The point is located exactly as everywhere else in the library (locate: int32 base + offset in one fp32
// rounding, validity, truncation, edge rule); dcn_debug_tc_points decodes these entries for the bit-exactness test.
__global__ void __launch_bounds__(256)
b2_points_kernel(const Geom g, const float* __restrict__ off, uint4* __restrict__ pts, int Wp, int W2) {
    const long long total = (long long)g.N * g.dg * g.kv * g.ov;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        uint32_t q1, pos, q2, tap, n, grp;
        g.d_ov.divmod((uint32_t)e, q1, pos);
        g.d_kv.divmod(q1, q2, tap);
        n = q2 / (uint32_t)g.dg;
        grp = q2 - n * (uint32_t)g.dg;
        const OutPos op = decompose_pos(g, (long long)n * g.ov + pos);
        Pt<float, 2> s;
        locate<float, 2>(g, offset_block<float, 2>(g, off, (int)n), (int)grp, (int)tap, op, s);
        uint4 r = make_uint4(0u, 0u, 0u, 0u);
        int h0, w0;
        if (s.valid) {
            h0 = s.lo[0];
            w0 = s.lo[1];
            r.x = ((s.hi[1] != w0 ? 1u : 0u) << 29) | ((s.hi[0] != h0 ? 1u : 0u) << 30) | (1u << 31);
            r.z = __float_as_uint(s.lw[0]);
            r.w = __float_as_uint(s.lw[1]);
        } else {
            h0 = op.base[1] < 0 ? 0 : (op.base[1] >= g.in[1] ? g.in[1] - 1 : op.base[1]);
            w0 = op.base[2] < 0 ? 0 : (op.base[2] >= g.in[2] ? g.in[2] - 1 : op.base[2]);
        }
        const uint32_t cls = (uint32_t)((h0 & 1) * 2 + (w0 & 1));
        r.x |= (uint32_t)(((h0 >> 1) * W2 + (w0 >> 1)) * 128) + cls * 32u + (cls << 27);
        r.y = (uint32_t)(h0 * Wp + w0);
        pts[e] = r;
    }
}

size_t b2_points_bytes(const Geom& g) { return (size_t)g.N * g.dg * g.kv * g.ov * 16; }

// Decodes the entries of sample n into the layout of dcn_debug_points (coords [dg,kv,ov,2], valid [dg,kv,ov],
// lo / hi [dg,kv,ov,2], -1 when invalid).  The coordinate is rebuilt as lo + lw, which is exact.  An entry whose
// plane address does not decode to the same low corner as its x-plane index is reported as valid = -1.
__global__ void __launch_bounds__(256)
b2_points_decode_kernel(const Geom g, const uint4* __restrict__ pts, int n, int Wp, int W2, float* __restrict__ coords,
                        int32_t* __restrict__ valid, int32_t* __restrict__ lo, int32_t* __restrict__ hi) {
    const long long total = (long long)g.dg * g.kv * g.ov;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const uint4 r = pts[(size_t)n * total + e];
        const bool v = (r.x >> 31) != 0u;
        int h0 = -1, w0 = -1, h1 = -1, w1 = -1, vv = 0;
        float ph = 0.f, pw = 0.f;
        if (v) {
            h0 = (int)(r.y / (uint32_t)Wp);
            w0 = (int)(r.y % (uint32_t)Wp);
            h1 = h0 + (int)((r.x >> 30) & 1u);
            w1 = w0 + (int)((r.x >> 29) & 1u);
            ph = (float)h0 + __uint_as_float(r.z);
            pw = (float)w0 + __uint_as_float(r.w);
            const uint32_t a = r.x & 0xFFFFFu, blk = a >> 7, cls = (a >> 5) & 3u;
            const int ah = (int)(blk / (uint32_t)W2) * 2 + (int)(cls >> 1), aw = (int)(blk % (uint32_t)W2) * 2 + (int)(cls & 1u);
            vv = (ah == h0 && aw == w0 && cls == ((r.x >> 27) & 3u)) ? 1 : -1;
        }
        valid[e] = vv;
        coords[e * 2] = ph; coords[e * 2 + 1] = pw;
        lo[e * 2] = h0; lo[e * 2 + 1] = w0;
        hi[e * 2] = h1; hi[e * 2 + 1] = w1;
    }
}

// 32 lanes x 8 consecutive 32-bit columns of tensor memory.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void b2_epi_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kB2EpiWarps) : "memory");
}

__device__ __forceinline__ int atom_shared_add(uint32_t addr, int v) {
    int old;
    asm volatile("atom.shared.add.s32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void red_shared_add(uint32_t addr, int v) {
    asm volatile("red.shared.add.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int atom_shared_exch(uint32_t addr, int v) {
    int old;
    asm volatile("atom.shared.exch.b32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}

struct B2Item {
    int n, j, slab;
    int ch0;            // first input channel of the slab
    long long c0;       // first 64-position chunk of the sample's tiles
    int tiles;          // 128-position tiles covering the sample
};
__device__ __forceinline__ B2Item b2_item(const Geom& g, long long item, int SL) {
    B2Item r;
    r.slab = (int)(item % SL);
    r.j = (int)((item / SL) % g.G);
    r.n = (int)(item / SL / g.G);
    r.ch0 = r.j * g.Cg + r.slab * 8;
    const long long p0 = (long long)r.n * g.ov;
    r.c0 = p0 / 64;
    r.tiles = (int)((p0 + g.ov - r.c0 * 64 + 127) / 128);
    return r;
}

struct B2Ctl {
    uint64_t full[kB2MaxStages], empty[kB2MaxStages], acc_full[2], acc_empty[2], w_full, w_empty;
    uint32_t tmem_base;
    uint32_t abort_flag;        // raised by an epilogue warp whose bounded wait gave up
    unsigned int budget;        // magnitudes added to the plane so far, in units of 256 fixed-point steps
};

// ACC: dX accumulates into the caller's buffer (separate backward-data entry point); otherwise this kernel
// zero-fills the part of dX it owns before it adds to it.
// FULL: both gradients are wanted and the tap count is a whole number of tap groups per warp residue (the common
// case: 3 x 3), so the per-tap tests of those conditions fold away at compile time.
template <bool ACC, bool FULL>
__global__ void __launch_bounds__(kB2Threads, 1)
tc_bwd2d_kernel(const Geom g, const __nv_bfloat16* __restrict__ xcl, const uint4* __restrict__ pts,
                const uint8_t* __restrict__ dpk, const uint8_t* __restrict__ wpk,
                const unsigned int* __restrict__ scale_bits, float* __restrict__ dx, float* __restrict__ doff,
                const B2Dims d, const FastDiv d_iw, const FastDiv d_w2) {
    extern __shared__ __align__(1024) uint8_t smem_b2[];
    uint8_t* wres = smem_b2;                                    // resident weight tiles of the current slab
    uint8_t* ring = wres + d.w_bytes;                           // dy stages
    int* plane = reinterpret_cast<int*>(ring + d.stages * kB2StageBytes);
    uint8_t* xs = reinterpret_cast<uint8_t*>(plane) + d.plane_bytes;
    B2Ctl* ctl = reinterpret_cast<B2Ctl*>(xs + d.xs_bytes);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t NS = (uint32_t)d.stages;

    if (threadIdx.x == 0) {
        ctl->abort_flag = 0;
        for (int s = 0; s < kB2MaxStages; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], kB2EpiWarps);
        }
        mbar_init(&ctl->w_full, 1);
        mbar_init(&ctl->w_empty, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        tmem_alloc(&ctl->tmem_base, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    const uint32_t idesc = make_idesc(128, d.NW, 1, 0);   // A MN-major, B K-major

    if (warp == 0) {
        // ------------------------------------------------ MMA issue
        if (lane == 0) {
            uint32_t tl = 0, il = 0;
            Ring rs;
            bool ok = true;
            const uint32_t w_base = smem_u32(wres);
            for (long long item = blockIdx.x; item < d.items && ok; item += gridDim.x, ++il) {
                const B2Item wi = b2_item(g, item, d.SL);
                ok = mbar_wait(&ctl->w_full, il & 1);
                for (int t = 0; t < wi.tiles && ok; ++t, ++tl) {
                    const uint32_t b = tl & 1;
                    ok = mbar_wait(&ctl->acc_empty[b], ((tl >> 1) & 1) ^ 1);
                    tc_fence_after();
                    for (int os = 0; os < d.OS && ok; ++os, rs.next(NS)) {
                        ok = mbar_wait(&ctl->full[rs.i], rs.ph);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t a_base = smem_u32(ring + rs.i * kB2StageBytes);
                        const uint32_t b_base = w_base + (uint32_t)(os >> 1) * (uint32_t)d.w_chunk + (uint32_t)(os & 1) * 64u;
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const uint64_t ad = make_desc(a_base + k * 2048, 4096, 1024);
                            const uint64_t bd = make_desc(b_base + k * 32, 16, 1024);
                            umma_bf16(tmem_base + b * 128, ad, bd, idesc, (os > 0 || k > 0) ? 1u : 0u);
                        }
                        umma_commit(&ctl->empty[rs.i]);
                    }
                    if (ok) umma_commit(&ctl->acc_full[b]);
                }
                if (ok) umma_commit(&ctl->w_empty);       // the slab's weights have been read for the last time
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ operand loader
        if (lane == 0) {
            Ring rs;
            uint32_t il = 0;
            bool ok = true;
            for (long long item = blockIdx.x; item < d.items && ok; item += gridDim.x, ++il) {
                const B2Item wi = b2_item(g, item, d.SL);
                ok = mbar_wait(&ctl->w_empty, (il & 1) ^ 1);
                if (!ok) break;
                mbar_arrive_expect_tx(&ctl->w_full, (uint32_t)d.w_bytes);
                for (int oc = 0; oc < d.OC; ++oc)
                    bulk_g2s(wres + oc * d.w_chunk, wpk + ((size_t)wi.j * d.SL + wi.slab) * d.w_bytes + (size_t)oc * d.w_chunk,
                             (uint32_t)d.w_chunk, &ctl->w_full);
                for (int t = 0; t < wi.tiles && ok; ++t) {
                    for (int os = 0; os < d.OS && ok; ++os, rs.next(NS)) {
                        ok = mbar_wait(&ctl->empty[rs.i], rs.ph ^ 1u);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&ctl->full[rs.i], (uint32_t)kB2StageBytes);
                        uint8_t* a_dst = ring + rs.i * kB2StageBytes;
                        const int mt = os / 4, quarter = os % 4;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            long long ch = wi.c0 + 2 * t + h;
                            if (ch >= d.PC) ch = d.PC - 1;       // past the packed range: rows masked by the epilogue
                            const uint8_t* src = dpk + (((size_t)wi.j * d.MT + mt) * d.PC + ch) * kTileBytes + quarter * 4096;
                            bulk_g2s(a_dst + h * 4096, src, 4096, &ctl->full[rs.i]);
                        }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------ epilogue
        const int ew = warp - 2;
        const int q = warp & 3;                         // tensor-memory lane quarter
        const int kq = ew / 4;                          // which of the quarter's warps
        const int etid = ew * 32 + lane;                // 0 .. 383
        constexpr int ET = 32 * kB2EpiWarps;
        const uint32_t plane_s = smem_u32(plane);
        const uint32_t xs_s = smem_u32(xs);
        const int W = g.in[2], Wp = d.Wp;
        const bool want_dx = FULL || dx != nullptr;
        const bool want_off = FULL || doff != nullptr;
        const uint32_t lane_j = (uint32_t)lane & 7u, lane_g = (uint32_t)lane >> 3;
        uint32_t ck4[8];                                // byte offset of this lane's channel in step k
#pragma unroll
        for (int k = 0; k < 8; ++k) ck4[k] = ((lane_j + (uint32_t)k) & 7u) << 2;

        // fixed-point scale: one term |w * col| <= 4 * Og * max|dy| * max|W| (corner weights reach 2 per axis in the
        // one-pixel border band, where the low weight is 1 - lw with lw in (-1, 0))
        const float bound = (float)g.Og * __uint_as_float(scale_bits[0]) * __uint_as_float(scale_bits[1]) * 1.01f;
        const int ex = (int)((__float_as_uint(bound) >> 23) & 0xffu) - 127;            // bound < 2^(ex + 1)
        float fx_scale, fx_inv;
        if (!(bound < 3.0e38f)) {                       // inf or NaN in dy / W: poison dX like fp32 arithmetic would
            fx_scale = 0.f;
            fx_inv = __uint_as_float(0x7fc00000u);
        } else {
            int se = kB2TermBits - 3 - ex;              // 4 * bound * 2^se < 2^21
            se = se > 100 ? 100 : (se < -100 ? -100 : se);
            fx_scale = __uint_as_float((uint32_t)(127 + se) << 23);
            fx_inv = __uint_as_float((uint32_t)(127 - se) << 23);
        }

        // A sampling point as the epilogue needs it.
        struct TapPt {
            uint32_t xpix;      // lo_h * Wp + lo_w in the linear x plane
            uint32_t a00;       // byte address of the (lo_h, lo_w) pixel in the blocked dX plane
            int adh, adw;       // steps to the pixel of the other row / column parity
            uint32_t cls;       // class of (lo_h, lo_w)
            float lw0, lw1;
            bool valid, sh, sw; // sh / sw: the high corner differs from the low one along h / w
        };
        constexpr int TG = 3;                           // taps of one group: k3, k3 + WQ, k3 + 2 WQ (+ 3 WQ per further group)
        constexpr int WQ = kB2WQ;
        uint32_t tl = 0;
        bool ok = true;
        for (long long item = blockIdx.x; item < d.items && ok; item += gridDim.x) {
            const B2Item wi = b2_item(g, item, d.SL);
            const int grp = (int)g.d_cpg.div((uint32_t)wi.ch0);
            const uint4* pts_n = pts + (size_t)(wi.n * g.dg + grp) * g.kv * g.ov;
            float* dx_n = want_dx ? dx + (size_t)wi.n * g.C * g.iv + (size_t)wi.ch0 * g.iv : nullptr;
            float* doff_n = want_off ? doff + ((size_t)wi.n * g.dg + grp) * g.kv * 2 * g.ov : nullptr;
            const long long pbeg = (long long)wi.n * g.ov, pend = pbeg + g.ov;
            const long long Pfirst = wi.c0 * 64 + q * 32 + lane;

            // entries of the first tap group of the first tile (later groups are fetched one group ahead)
            uint4 ent[TG];
            auto fetch_points = [&](long long P, int tg) {
                const bool in = P >= pbeg && P < pend;
#pragma unroll
                for (int u = 0; u < TG; ++u) {
                    const int tap = tg + WQ * u;
                    ent[u] = (in && (FULL || tap < g.kv)) ? __ldg(pts_n + (uint32_t)tap * (uint32_t)g.ov + (uint32_t)(P - pbeg))
                                                : make_uint4(0u, 0u, 0u, 0u);
                }
            };
            fetch_points(Pfirst, (kq + (int)tl) % WQ);

            // ---- set-up: clear the fixed-point plane, bring in the slab's input plane, own the dX slab
            if (want_dx) {
                for (int i = etid; i < d.plane_bytes / 16; i += ET)
                    st_shared_v4(plane_s + (uint32_t)i * 16u, 0u, 0u, 0u, 0u);
                if (!ACC)
                    for (int i = etid; i < 8 * g.iv; i += ET) dx_n[i] = 0.f;
                if (etid == 0) ctl->budget = 0u;
            }
            if (want_off) {
                const __nv_bfloat16* xn = xcl + (size_t)wi.n * g.iv * g.C + wi.ch0;
                for (int i = etid; i < g.iv; i += ET) {
                    uint32_t r, c;
                    d_iw.divmod((uint32_t)i, r, c);
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(xn + (size_t)i * g.C));
                    st_shared_v4(xs_s + (r * (uint32_t)Wp + c) * 16u, v.x, v.y, v.z, v.w);
                }
            }
            b2_epi_barrier();

            for (int t = 0; t < wi.tiles && ok; ++t, ++tl) {
                const uint32_t b = tl & 1;
                const long long P = Pfirst + 128ll * t;
                const bool p_ok = P >= pbeg && P < pend;
                const uint32_t opos = p_ok ? (uint32_t)(P - pbeg) : 0u;
                // the warps of a quarter take turns at the tap residues, so that the uneven share evens out over tiles
                const int k3 = (kq + (int)tl) % WQ, k3n = (kq + (int)tl + 1) % WQ;
                for (int tg = k3; tg < g.kv; tg += WQ * TG) {
                    // ---- sampling points of this group from the entries fetched a group ago.  An invalid point is an
                    // all-zero entry: first block of the plane, zero weights, so the code below runs without
                    // divergence and its lanes add zeros to addresses that still differ from every other lane's.
                    TapPt tp[TG];
#pragma unroll
                    for (int u = 0; u < TG; ++u) {
                        const uint32_t ex_ = ent[u].x;
                        const bool sh = (ex_ >> 30) & 1u, sw = (ex_ >> 29) & 1u;
                        tp[u].valid = (ex_ >> 31) != 0u;
                        tp[u].sh = sh;
                        tp[u].sw = sw;
                        tp[u].xpix = ent[u].y;
                        tp[u].a00 = plane_s + (ex_ & 0xFFFFFu);
                        tp[u].cls = (ex_ >> 27) & 3u;
                        // the pixel of the other parity: the high corner, or (where the corners coincide) the
                        // twin inside the same block, which only ever receives zeros
                        tp[u].adw = (tp[u].cls & 1u) ? (sw ? 96 : -32) : 32;
                        tp[u].adh = (tp[u].cls & 2u) ? (sh ? d.W2 * 128 - 64 : -64) : 64;
                        tp[u].lw0 = __uint_as_float(ent[u].z);
                        tp[u].lw1 = __uint_as_float(ent[u].w);
                    }
                    // ---- entries of the next group (this tile's, or the next tile's first one)
                    const bool last_group = tg + WQ * TG >= g.kv;
                    if (!last_group) fetch_points(P, tg + WQ * TG);
                    else if (t + 1 < wi.tiles) fetch_points(P + 128, k3n);

                    // ---- col values of the group out of tensor memory; the accumulator is released once the
                    // position's last values are in registers
                    if (tg == k3) {
                        ok = mbar_wait(&ctl->acc_full[b], (tl >> 1) & 1);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    float f[TG][8];
#pragma unroll
                    for (int u = 0; u < TG; ++u) {
                        uint32_t v[8];
                        const int tap = tg + WQ * u;
                        tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + b * 128 + ((FULL || tap < g.kv) ? tap : 0) * 8, v);
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[u][i] = __uint_as_float(v[i]);
                    }
                    tmem_ld_wait();
                    if (last_group) {
                        tc_fence_before();
                        mbar_arrive_warp(&ctl->acc_empty[b]);
                    }
                    // ---- budget: while the magnitudes of all terms ever added to the plane sum to less than 2^30
                    // no element can have overflowed, so plain reductions (no return value) are safe
                    bool fast = true;
                    if (want_dx) {
                        float mag = 0.f;
#pragma unroll
                        for (int u = 0; u < TG; ++u) {
                            float sa = 0.f;
#pragma unroll
                            for (int i = 0; i < 8; ++i) sa += fabsf(f[u][i]);
                            const float h0 = fabsf(1.f - tp[u].lw0) + fabsf(tp[u].lw0), h1 = fabsf(1.f - tp[u].lw1) + fabsf(tp[u].lw1);
                            mag = fmaf(tp[u].valid ? sa : 0.f, h0 * h1, mag);
                        }
                        // units of 256 fixed-point steps, rounded up, plus the rounding of the 96 terms themselves
                        const unsigned int mine = (unsigned int)(mag * fx_scale * (1.f / 256.f)) + 2u;
                        const unsigned int wsum = __reduce_add_sync(0xffffffffu, mine);
                        unsigned int before = 0;
                        if (lane == 0) before = atomicAdd(&ctl->budget, wsum);
                        before = __shfl_sync(0xffffffffu, before, 0);
                        fast = before + wsum < (1u << 22) - (1u << 16);
                    }

#pragma unroll
                    for (int u = 0; u < TG; ++u) {
                        const int tap = tg + WQ * u;
                        if (!FULL && tap >= g.kv) break;        // warp-uniform
                        const bool sh = tp[u].sh, sw = tp[u].sw;
                        const float lw0 = tp[u].lw0, lw1 = tp[u].lw1, hw0 = 1.f - lw0, hw1 = 1.f - lw1;
                        if (want_off) {
                            const uint32_t xdh = sh ? (uint32_t)Wp : 0u, xdw = sw ? 1u : 0u;
                            const uint32_t xp[4] = {tp[u].xpix, tp[u].xpix + xdw, tp[u].xpix + xdh, tp[u].xpix + xdh + xdw};
                            float T[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const uint4 xv = lds128(xs_s + xp[e] * 16u);
                                float a = f[u][0] * bf16_lo(xv.x);
                                a = fmaf(f[u][1], bf16_hi(xv.x), a);
                                a = fmaf(f[u][2], bf16_lo(xv.y), a);
                                a = fmaf(f[u][3], bf16_hi(xv.y), a);
                                a = fmaf(f[u][4], bf16_lo(xv.z), a);
                                a = fmaf(f[u][5], bf16_hi(xv.z), a);
                                a = fmaf(f[u][6], bf16_lo(xv.w), a);
                                T[e] = fmaf(f[u][7], bf16_hi(xv.w), a);
                            }
                            // deform2d/lib/deform_conv2d_cuda_kernel.cu:329-339, same expression order as interp_grad
                            const float g0 = T[3] * lw1 + T[2] * hw1 - T[1] * lw1 - T[0] * hw1;
                            const float g1 = T[1] * hw0 + T[3] * lw0 - T[0] * hw0 - T[2] * lw0;
                            float* dst = doff_n + (uint32_t)(tap * 2) * (uint32_t)g.ov + opos;
                            if (tp[u].valid) {
                                atomicAdd(dst, g0);
                                atomicAdd(dst + g.ov, g1);
                            }
                        }
                        if (want_dx) {
                            // per-axis weights of the low pixel and of the pixel of the other parity
                            const float wh[2] = {sh ? hw0 : hw0 + lw0, sh ? lw0 : 0.f};
                            const float ww[2] = {sw ? hw1 : hw1 + lw1, sw ? lw1 : 0.f};
                            // rotate the 8 col values so that step k holds channel (lane_j + k) & 7
                            float fa[8], fr[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) fa[i] = (lane_j & 4u) ? f[u][(i + 4) & 7] : f[u][i];
#pragma unroll
                            for (int i = 0; i < 8; ++i) fr[i] = (lane_j & 2u) ? fa[(i + 2) & 7] : fa[i];
#pragma unroll
                            for (int i = 0; i < 8; ++i) fa[i] = (lane_j & 1u) ? fr[(i + 1) & 7] : fr[i];
                            // in round r this lane takes its corner of class r ^ lane_g, i.e. corner r ^ m
                            const uint32_t m = tp[u].cls ^ lane_g;
                            const float vs = tp[u].valid ? fx_scale : 0.f;
                            uint32_t ar[4];
                            float wr[4];
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                const uint32_t e = (uint32_t)r ^ m;
                                ar[r] = tp[u].a00 + ((e & 2u) ? tp[u].adh : 0) + ((e & 1u) ? tp[u].adw : 0);
                                wr[r] = ((e & 2u) ? wh[1] : wh[0]) * ((e & 1u) ? ww[1] : ww[0]) * vs;
                            }
                            if (fast) {
#pragma unroll
                                for (int r = 0; r < 4; ++r) {
#pragma unroll
                                    for (int k = 0; k < 8; ++k) {
                                        const int term = __float_as_int(fmaf(fa[k], wr[r], 12582912.f)) - 0x4B400000;
                                        red_shared_add(ar[r] + ck4[k], term);
                                    }
                                }
                            } else {
                                // the budget is spent: every addition looks at the element it found, and one that
                                // had reached 2^30 is taken out and added to dX right away
#pragma unroll
                                for (int r = 0; r < 4; ++r) {
#pragma unroll
                                    for (int k = 0; k < 8; ++k) {
                                        const int term = __float_as_int(fmaf(fa[k], wr[r], 12582912.f)) - 0x4B400000;
                                        const uint32_t addr = ar[r] + ck4[k];
                                        const int old = atom_shared_add(addr, term);
                                        if ((old ^ (old << 1)) < 0) {
                                            const int got = atom_shared_exch(addr, 0);
                                            const uint32_t wofs = (addr - plane_s) >> 2;          // word in the plane
                                            uint32_t bh, bw;
                                            d_w2.divmod(wofs >> 5, bh, bw);
                                            const uint32_t cl = (wofs >> 3) & 3u, c = wofs & 7u;
                                            const uint32_t hh = bh * 2 + (cl >> 1), wc = bw * 2 + (cl & 1u);
                                            atomicAdd(dx_n + (size_t)c * g.iv + hh * W + wc, (float)got * fx_inv);
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
            }

            // ---- read-out: plane -> dX (reductions: early spills may already have landed there).  The epilogue
            // warps pass the item's barriers together; a warp whose wait gave up tells the others to stop as well.
            if (!ok) ctl->abort_flag = 1;
            b2_epi_barrier();
            if (*reinterpret_cast<volatile uint32_t*>(&ctl->abort_flag) != 0) ok = false;
            if (want_dx && ok) {
                // a thread takes 4 channels of one pixel (16 bytes); a quarter warp covers one 128-byte block
                const int n16 = d.plane_bytes / 16;
                for (int i = etid; i < n16; i += ET) {
                    const uint4 v = lds128(plane_s + (uint32_t)i * 16u);
                    uint32_t bh, bw;
                    d_w2.divmod((uint32_t)i >> 3, bh, bw);
                    const uint32_t cl = ((uint32_t)i >> 1) & 3u, c4 = ((uint32_t)i & 1u) * 4u;
                    const uint32_t hh = bh * 2 + (cl >> 1), wc = bw * 2 + (cl & 1u);
                    if (hh < (uint32_t)g.in[1] && wc < (uint32_t)W) {
                        float* dc = dx_n + (size_t)c4 * g.iv + hh * W + wc;
                        const int vv[4] = {(int)v.x, (int)v.y, (int)v.z, (int)v.w};
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (vv[c] != 0) atomicAdd(dc + (size_t)c * g.iv, (float)vv[c] * fx_inv);
                    }
                }
            }
            b2_epi_barrier();          // the plane is cleared again by the next item's set-up
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 256);
    }
}

// scale_bits: two words, zeroed by the caller and raised by the packing passes (max|dy|, max|W| as bit patterns).
int launch_tc_bwd2d(const Geom& g, const __nv_bfloat16* xcl, const uint4* pts, const uint8_t* dpk, const uint8_t* wpk,
                    const unsigned int* scale_bits, float* dx, float* doff, bool accumulate, cudaStream_t st) {
    const B2Dims d = b2_dims(g);
    FastDiv d_iw, d_w2;
    d_iw.init((uint32_t)g.in[2]);
    d_w2.init((uint32_t)d.W2);
    const int grid = (int)(d.items < sm_count() ? d.items : sm_count());
    const bool full = dx != nullptr && doff != nullptr && g.kv % (kB2WQ * 3) == 0;
    auto go = [&](auto kern) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, d.smem_bytes) != cudaSuccess) return false;
        kern<<<grid, kB2Threads, d.smem_bytes, st>>>(g, xcl, pts, dpk, wpk, scale_bits, dx, doff, d, d_iw, d_w2);
        return true;
    };
    bool launched;
    if (accumulate) launched = full ? go(tc_bwd2d_kernel<true, true>) : go(tc_bwd2d_kernel<true, false>);
    else launched = full ? go(tc_bwd2d_kernel<false, true>) : go(tc_bwd2d_kernel<false, false>);
    if (!launched) return -5;
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
