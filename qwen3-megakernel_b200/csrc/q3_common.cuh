// Shared device helpers and model geometry for the Qwen3-0.6B engine (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace q3 {

constexpr int HIDDEN = 1024;
constexpr int Q_HEADS = 16;
constexpr int KV_HEADS = 8;
constexpr int HEAD_DIM = 128;
constexpr int Q_DIM = Q_HEADS * HEAD_DIM;     // 2048
constexpr int KV_DIM = KV_HEADS * HEAD_DIM;   // 1024
constexpr int QKV_DIM = Q_DIM + 2 * KV_DIM;   // 4096: q | k | v
constexpr int INTER = 3072;
constexpr float EPS = 1e-6f;
constexpr float ATTN_SCALE = 0.08838834764831845f;  // 128^-0.5

typedef unsigned short bf16_raw;

// ---- bf16 <-> fp32 ---------------------------------------------------------------------------
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ float bf_to_f(bf16_raw h) { return __uint_as_float(((uint32_t)h) << 16); }
__device__ __forceinline__ bf16_raw f_to_bf(float f) {  // round to nearest even, NaN-safe
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// ---- warp / block reductions -----------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of NW warps.  `red` holds >= NW floats.  Two __syncthreads; every thread gets the sum.
template <int NW>
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = (l < NW) ? red[l] : 0.f;
    return warp_sum(t);
}

// ---- activation vectors in shared memory -----------------------------------------------------
// A weight row is streamed as 16-byte units: unit j of a lane holds elements [j*256 + lane*8, +8).
// The matching eight activations are fetched as two float4.  To keep both fetches free of bank
// conflicts the vector is stored "lane-interleaved": inside every 256-element block, element
// lane*8 + h*4 + i sits at h*128 + lane*4 + i.
__device__ __forceinline__ int act_slot(int e) {
    const int o = e & 255;
    return (e & ~255) | (((o >> 2) & 1) << 7) | ((o >> 3) << 2) | (o & 3);
}

// dot of 8 bf16 weights (one uint4) with the eight activations of unit j for this lane
__device__ __forceinline__ float dot8(const uint4& w, const float* __restrict__ xs, int j, int lane) {
    const float4 a = *reinterpret_cast<const float4*>(xs + j * 256 + lane * 4);
    const float4 b = *reinterpret_cast<const float4*>(xs + j * 256 + 128 + lane * 4);
    float s = bf_lo(w.x) * a.x;
    s = fmaf(bf_hi(w.x), a.y, s);
    s = fmaf(bf_lo(w.y), a.z, s);
    s = fmaf(bf_hi(w.y), a.w, s);
    s = fmaf(bf_lo(w.z), b.x, s);
    s = fmaf(bf_hi(w.z), b.y, s);
    s = fmaf(bf_lo(w.w), b.z, s);
    s = fmaf(bf_hi(w.w), b.w, s);
    return s;
}

// streaming 16-byte load that does not pollute L1 (weights are read once per step)
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Prefetch loads write straight into the registers that hold the row until it is used: the zero for a row past the
// cache and the predicated load sit in one asm statement, so that no select or move consumes the loaded value (which
// would park the warp until the row has arrived, at the place where it was only meant to be requested).
__device__ __forceinline__ void ld_row16(uint4& d, const void* ptr, bool live) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
                 "@p ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
                 : "=&r"(d.x), "=&r"(d.y), "=&r"(d.z), "=&r"(d.w) : "l"(ptr), "r"((int)live));
}
__device__ __forceinline__ void ld_row8(uint32_t& a, uint32_t& b, const void* ptr, bool live) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\t"
                 "@p ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n\t}"
                 : "=&r"(a), "=&r"(b) : "l"(ptr), "r"((int)live));
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// The layered path is a chain of short kernels.  Each one lets its successor start launching at once
// (`pdl_launch`) and itself waits for its predecessor's results only after its own set-up (`pdl_wait`, which
// returns immediately for a kernel that was launched without the attribute), so that launch latency and
// prologues overlap the tail of the kernel before.
#ifndef Q3_PDL
#define Q3_PDL 1
#endif
__device__ __forceinline__ void pdl_launch() {
#if Q3_PDL
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_wait() {
#if Q3_PDL
    asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = Q3_PDL;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- device status words ----------------------------------------------------------------------
// [0] error code (0 = fine), [1] phase / site id, [2] CTA index, [3] observed value.
enum : uint32_t { ST_OK = 0, ST_BARRIER_TIMEOUT = 1, ST_MBAR_TIMEOUT = 2, ST_BAD_TOKEN = 3, ST_PEER_TIMEOUT = 4, ST_BAD_LEN = 5 };

__device__ __forceinline__ void report(uint32_t* status, uint32_t code, uint32_t site, uint32_t value) {
    if (atomicCAS(status, 0u, code) == 0u) {
        status[1] = site;
        status[2] = blockIdx.x;
        status[3] = value;
    }
}

}  // namespace q3
