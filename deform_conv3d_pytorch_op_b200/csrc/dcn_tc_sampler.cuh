// Sampling front end shared by the tensor-core forward and weight-gradient kernels (included by dcn_tc.cu
// inside its anonymous namespace).
//
// Work is split between two kinds of warps so that the two dependent memory latencies of a sample (offset
// load -> corner gathers) sit in different warps and overlap:
//   coordinate warps  read the offsets (coalesced along positions), locate the sampling point exactly as the
//                     reference does (fp32, one rounding) and publish, per (position row, key), the 2^D
//                     corner indices and corner weights in a shared-memory table; a key is one
//                     (deformable group, tap) pair, and a K chunk touches only a few distinct keys;
//   gather warps      read a table entry (broadcast to the 8 lanes that share a row), fetch 2^D 16-byte
//                     vectors of 8 bf16 channels from the channels-last input, interpolate in fp32 with packed
//                     two-wide FMAs, round to bf16 and store one 16-byte chunk of the swizzled operand tile.
#pragma once

template <int D, bool DEFORM>
struct alignas(16) TabEntry {
    int idx[1 << D];      // linear index of each corner inside the sample's input volume; idx[0] < 0: invalid
    float w[1 << D];      // corner weights (products of the per-axis weights)
};
template <int D>
struct alignas(16) TabEntry<D, false> {
    int idx[4];           // idx[0] = integer tap location or -1
};

// key of an 8-channel chunk column starting at GEMM-K index kp (k' = tap * Cg + c): grp * kv + tap, -1 past the end
__device__ __forceinline__ int chunk_key(const Geom& g, int j, int kp, int& tap_out, int& c_out) {
    if (kp >= g.kv * g.Cg) { tap_out = 0; c_out = 0; return -1; }
    uint32_t tap, cl;
    g.d_Cg.divmod((uint32_t)kp, tap, cl);
    const int c = j * g.Cg + (int)cl;
    tap_out = (int)tap;
    c_out = c;
    return (int)g.d_cpg.div((uint32_t)c) * g.kv + (int)tap;
}

// 4-byte asynchronous global -> shared copy (offset prefetch of the coordinate warps) and its group control.
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Keys of the chunk columns handled by lanes 0..ncols-1 of a warp, run-length numbered into slots.
struct SlotInfo {
    int my_key;        // key of column `lane` (lanes >= ncols: undefined)
    uint32_t news;     // bit c set: column c starts a new slot
    int my_slot;       // slot of column `lane`
    int nslots;
};
__device__ __forceinline__ SlotInfo make_slots(int my_key, int lane, int ncols) {
    SlotInfo r;
    r.my_key = my_key;
    const int prev = __shfl_up_sync(0xffffffffu, my_key, 1);
    const bool is_new = lane < ncols && (lane == 0 || my_key != prev);
    r.news = __ballot_sync(0xffffffffu, is_new);
    r.my_slot = __popc(r.news & ((2u << lane) - 1u)) - 1;
    r.nslots = __popc(r.news);
    return r;
}
// key of slot sl (all lanes)
__device__ __forceinline__ int slot_key(const SlotInfo& si, int sl) {
    const int col = __fns(si.news, 0, sl + 1);
    return __shfl_sync(0xffffffffu, si.my_key, col);
}

// Coordinate-warp side: fill one table entry from the D offset values of its point (prefetched into shared
// memory).
template <int D, bool DEFORM>
__device__ __forceinline__ void fill_entry_from(const Geom& g, const float (&offv)[D], const OutPos& op, bool pos_ok,
                                                int key, TabEntry<D, DEFORM>* e) {
    if constexpr (DEFORM) {
        int4* ei = reinterpret_cast<int4*>(e->idx);
        float4* ew = reinterpret_cast<float4*>(e->w);
        Pt<float, D> s;
        s.valid = false;
        if (pos_ok && key >= 0) {
            uint32_t grp_, tap_;
            g.d_kv.divmod((uint32_t)key, grp_, tap_);
            const int tap = (int)tap_;
            locate_with<float, D>(g, offv, tap, op, s);
        }
        int idx[1 << D];
        float cw[1 << D];
        if (s.valid) {
            corner_indices<float, D>(g, s, idx);
            corner_weights<float, D>(s, cw);
        } else {
#pragma unroll
            for (int i = 0; i < (1 << D); ++i) { idx[i] = -1; cw[i] = 0.f; }
        }
#pragma unroll
        for (int q = 0; q < (1 << D) / 4; ++q) {
            ei[q] = make_int4(idx[4 * q], idx[4 * q + 1], idx[4 * q + 2], idx[4 * q + 3]);
            ew[q] = make_float4(cw[4 * q], cw[4 * q + 1], cw[4 * q + 2], cw[4 * q + 3]);
        }
    } else {
        int pidx = -1;
        if (pos_ok && key >= 0) {
            const int tap = (int)((uint32_t)key - g.d_kv.div((uint32_t)key) * (uint32_t)g.kv);
            int t;
            if (locate_plain<D>(g, tap, op, t)) pidx = t;
        }
        *reinterpret_cast<int4*>(e->idx) = make_int4(pidx, 0, 0, 0);
    }
}

__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// two fp32 FMAs in one instruction (sm_100)
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Gather-warp side, step 1: issue the corner loads of one entry.  The entry at shared address `entry_s`, the 8 channels at `xrow` (sample base +
// channel), `pix_bytes` = bytes between consecutive input positions of the channels-last copy.  Loads of an
// invalid entry are predicated off (no divergent branch); its weights are zero.
template <int D, bool DEFORM>
__device__ __forceinline__ void gather_issue_s(uint32_t entry_s, const __nv_bfloat16* __restrict__ xrow,
                                               uint32_t pix_bytes, uint4 (&q)[DEFORM ? (1 << D) : 1],
                                               float (&w)[DEFORM ? (1 << D) : 1]) {
    constexpr int NQ = DEFORM ? (1 << D) : 1;
    constexpr int NI = DEFORM ? (1 << D) : 4;
    uint32_t idx[NI];
#pragma unroll
    for (int i = 0; i < NI / 4; ++i) {
        const uint4 t = lds128(entry_s + 16 * i);
        idx[4 * i] = t.x; idx[4 * i + 1] = t.y; idx[4 * i + 2] = t.z; idx[4 * i + 3] = t.w;
    }
    if constexpr (DEFORM) {
#pragma unroll
        for (int i = 0; i < NQ / 4; ++i) {
            const uint4 t = lds128(entry_s + 4 * NI + 16 * i);
            w[4 * i] = __uint_as_float(t.x); w[4 * i + 1] = __uint_as_float(t.y);
            w[4 * i + 2] = __uint_as_float(t.z); w[4 * i + 3] = __uint_as_float(t.w);
        }
    } else {
        w[0] = 1.f;
    }
    const bool valid = (int)idx[0] >= 0;
#pragma unroll
    for (int i = 0; i < NQ; ++i)
        q[i] = valid ? __ldg(static_cast<const uint4*>(ptr_mad_u32(xrow, idx[i], pix_bytes))) : make_uint4(0, 0, 0, 0);
}

template <int D, bool DEFORM>
__device__ __forceinline__ uint4 gather_finish_w(const uint4 (&q)[DEFORM ? (1 << D) : 1],
                                                 const float (&w)[DEFORM ? (1 << D) : 1]) {
    if constexpr (!DEFORM) return q[0];
#ifndef DCN_INTERP_FP32
    // Packed bf16 arithmetic: 16 two-wide FMAs per 8 channels and no unpacking, against 16 two-wide fp32 FMAs plus
    // 32 unpack and pack operations (build with -DDCN_INTERP_FP32 for the fp32 form).  The sampled value is rounded
    // to bf16 for the MMA either way; rounding the partial sums too raises the measured error of y / dW at the
    // tensor-core test shapes from 3.3e-3 to 4.6e-3 of max|ref| (gate 2e-2) and takes 7-8 % off both kernels.
    else {
        uint32_t acc[4];
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            const uint32_t w2 = pack_bf16x2(w[c], w[c]);
            const uint32_t wd[4] = {q[c].x, q[c].y, q[c].z, q[c].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (c == 0) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(acc[i]) : "r"(w2), "r"(wd[i]));
                else asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(acc[i]) : "r"(w2), "r"(wd[i]), "r"(acc[i]));
            }
        }
        return make_uint4(acc[0], acc[1], acc[2], acc[3]);
    }
#else
    else {
        uint64_t acc[4];
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            const uint64_t w2 = pack_f32x2(w[c], w[c]);
            const uint32_t wd[4] = {q[c].x, q[c].y, q[c].z, q[c].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint64_t xv = pack_f32x2(bf16_lo(wd[i]), bf16_hi(wd[i]));
                acc[i] = (c == 0) ? fmul2(w2, xv) : ffma2(w2, xv, acc[i]);       // 0 + w*x == w*x exactly
            }
        }
        uint32_t out[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            unpack_f32x2(acc[i], lo, hi);
            out[i] = pack_bf16x2(lo, hi);
        }
        return make_uint4(out[0], out[1], out[2], out[3]);
    }
#endif
}
