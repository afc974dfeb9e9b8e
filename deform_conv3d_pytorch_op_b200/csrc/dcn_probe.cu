// Measurement probes for the two memory access patterns that bound the tensor-core kernels, built into their
// own small library (libdcn_probe.so) and used only by bench.py --probe: they are not part of the operator's
// C ABI.  Both touch pseudo-random 128-byte lines of a buffer with the lane layout of the kernels (8 lanes x
// 16 bytes = one line, four lines per warp instruction):
//   scatter: red.global.add.v4.f32, the input-gradient epilogue's reduction into the channels-last dX;
//   gather : 16-byte read-only loads, the corner fetches of the forward and weight-gradient producers.
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ uint32_t mix(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

__global__ void __launch_bounds__(512)
scatter_probe(float* __restrict__ buf, uint32_t n_lines, int reps) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;      // one line per 8 lanes
    const float4 v = make_float4(1.f, 1.f, 1.f, 1.f);
    for (int r = 0; r < reps; r += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t line = mix(slot * 0x9e3779b9u + (uint32_t)(r + u)) % n_lines;
            atomicAdd(reinterpret_cast<float4*>(buf + (size_t)line * 32 + (lane & 7) * 4), v);
        }
    }
}

__global__ void __launch_bounds__(512)
gather_probe(const uint4* __restrict__ buf, uint32_t n_lines, int reps, uint32_t* __restrict__ sink) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    uint32_t acc = 0;
    for (int r = 0; r < reps; r += 8) {
        uint4 q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t line = mix(slot * 0x9e3779b9u + (uint32_t)(r + u)) % n_lines;
            q[u] = __ldg(buf + (size_t)line * 8 + (lane & 7));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) acc ^= q[u].x ^ q[u].y ^ q[u].z ^ q[u].w;
    }
    if (acc == 0x12345678u) *sink = acc;       // keeps the loads alive
}

}  // namespace

extern "C" {

// `bytes` of `buf` (a multiple of 128, 16-byte aligned) are the target; every thread of `blocks` x 512 issues
// `reps` (a multiple of 8) accesses of 16 bytes.  Returns 0, or -5 when the launch failed.
int dcn_probe_scatter(float* buf, size_t bytes, int blocks, int reps, void* stream) {
    if (buf == nullptr || bytes < 128 || blocks < 1 || reps < 8) return -1;
    scatter_probe<<<blocks, 512, 0, static_cast<cudaStream_t>(stream)>>>(buf, (uint32_t)(bytes / 128), reps);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int dcn_probe_gather(const void* buf, size_t bytes, int blocks, int reps, uint32_t* sink, void* stream) {
    if (buf == nullptr || sink == nullptr || bytes < 128 || blocks < 1 || reps < 8) return -1;
    gather_probe<<<blocks, 512, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(buf),
                                                                         (uint32_t)(bytes / 128), reps, sink);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
