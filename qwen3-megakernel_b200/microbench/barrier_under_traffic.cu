// Grid-barrier latency under background weight streaming.
//
// 148 co-resident CTAs (cooperative launch) run a loop of {write 28 floats, grid barrier, read a 1024-float vector}
// while extra warps of every CTA stream a large buffer into shared memory, either as TMA bulk copies (mode 1),
// as plain loads (mode 2) or as 16-byte cp.async copies (mode 3), paced by nanosleep.  Prints the time per
// barrier round and the background bandwidth: the evidence behind the persistent decode kernel's choice of
// cp.async producers over bulk copies.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o barrier_under_traffic barrier_under_traffic.cu
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("%s: %s\n", #x, cudaGetErrorString(e)); return 1; } } while (0)
__device__ __forceinline__ unsigned long long gns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ uint32_t su32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// mode 0: no background; 1: TMA bulk copies of `chunk` bytes every `pace` ns; 2: LDG by the extra warp
template <int NP>
__global__ void __launch_bounds__(512 + 32 * NP, 1) k(unsigned* cnt, float* data, float* sink, int iters, const unsigned char* big, size_t per_cta,
                                            int mode, int chunk, int pace, unsigned long long* tout, unsigned long long* bytes_out, volatile int* stop) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bars[8];
    const int tid = threadIdx.x, c = blockIdx.x, G = gridDim.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { for (int i = 0; i < 8; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(su32(&bars[i]))); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    __syncthreads();
    if (warp >= 16) {
        unsigned long long moved = 0;
        const int pw = warp - 16;
        const unsigned char* base = big + (size_t)c * per_cta + (size_t)pw * (per_cta / NP);
        if (mode != 3 && pw > 0) return;
        if (mode == 1 && lane == 0) {
            const int depth = 8;
            size_t off = 0; int kq = 0;
            while (!*stop) {
                const int s = kq % depth;
                if (kq >= depth) { const unsigned par = ((kq - depth) / depth) & 1; unsigned ok = 0;
                    while (!ok) asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(su32(&bars[s])), "r"(par) : "memory"); }
                asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(su32(&bars[s])), "r"(chunk) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(su32(smem + (size_t)s * chunk)), "l"(base + off), "r"(chunk), "r"(su32(&bars[s])) : "memory");
                off += chunk; if (off + chunk > per_cta) off = 0; moved += chunk; ++kq;
                if (pace > 0) __nanosleep(pace);
            }
            // drain
            for (int j = (kq > depth ? kq - depth : 0); j < kq; ++j) { const int s = j % depth; const unsigned par = (j / depth) & 1; unsigned ok = 0;
                while (!ok) asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(su32(&bars[s])), "r"(par) : "memory"); }
            bytes_out[c] = moved;
        } else if (mode == 2) {
            size_t off = 0; uint4 acc = make_uint4(0, 0, 0, 0);
            while (!*stop) {
                uint4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w) : "l"(base + off + (size_t)(j * 32 + lane) * 16));
#pragma unroll
                for (int j = 0; j < 8; ++j) acc.x ^= v[j].x ^ v[j].w;
                off += 4096; if (off + 4096 > per_cta) off = 0; moved += 4096;
                if (pace > 0) __nanosleep(pace);
            }
            if (acc.x == 0x12345678) sink[0] = 1.f;
            if (lane == 0) bytes_out[c] = moved;
        } else if (mode == 3) {   // cp.async (LDGSTS) 16 B per lane, 16 per lane per group (8 KB per group), 4 groups in flight
            size_t off = 0;
            int g = 0;
            while (!*stop) {
                unsigned char* dst = smem + (size_t)pw * 65536 + (size_t)(g & 7) * 8192;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(su32(dst + (j * 32 + lane) * 16)), "l"(base + off + (size_t)(j * 32 + lane) * 16) : "memory");
                asm volatile("cp.async.commit_group;" ::: "memory");
                if (chunk == 8192) asm volatile("cp.async.wait_group 7;" ::: "memory"); else asm volatile("cp.async.wait_group 3;" ::: "memory");
                off += 8192; if (off + 8192 > per_cta / NP) off = 0; moved += 8192; ++g;
                if (pace > 0) __nanosleep(pace);
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            if (lane == 0) atomicAdd(&bytes_out[c], moved);
        } else if (lane == 0) bytes_out[c] = 0;
        return;
    }
    unsigned target = 0; float acc = 0.f;
    unsigned long long t0 = gns();
    for (int it = 0; it < iters; ++it) {
        float* buf = data + (size_t)(it & 1) * 4096;
        if ((tid & 31) == 0 && (tid >> 5) < 14) { __stcg(buf + c * 27 + (tid >> 5) * 2, acc + it); __stcg(buf + c * 27 + (tid >> 5) * 2 + 1, acc); }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        target += G;
        if (tid == 0) {
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
            unsigned v;
            do { asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory"); } while ((int)(v - target) < 0);
            asm volatile("fence.acquire.gpu;" ::: "memory");
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        float2 a = __ldcg(reinterpret_cast<const float2*>(buf) + tid);
        acc += a.x + a.y;
    }
    unsigned long long t1 = gns();
    if (tid == 0) { tout[c] = t1 - t0; __threadfence(); if (atomicAdd(cnt + 4, 1u) == (unsigned)G - 1) *stop = 1; }
    // every CTA's producer must stop: stop is set by the last CTA to finish
    sink[c * 512 + tid] = acc;
}

template <int NP>
int run_cfg(unsigned* cnt, float* data, float* sink, int iters, unsigned char* big, size_t per, int mode, int chunk, int pace, unsigned long long* tout, unsigned long long* bout, int* stop) {
    CK(cudaFuncSetAttribute(k<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    CK(cudaMemset(cnt, 0, 256)); CK(cudaMemset(stop, 0, 4)); CK(cudaMemset(bout, 0, 148 * 8));
    int G = 148; size_t p2 = per;
    void* args[] = {&cnt, &data, &sink, &iters, &big, &p2, &mode, &chunk, &pace, &tout, &bout, &stop};
    CK(cudaLaunchCooperativeKernel((void*)k<NP>, dim3(G), dim3(512 + 32 * NP), args, (size_t)(mode == 1 ? 8 * chunk : (mode == 3 ? NP * 65536 : 0)), 0));
    CK(cudaDeviceSynchronize());
    unsigned long long h[148], b[148]; CK(cudaMemcpy(h, tout, sizeof(h), cudaMemcpyDeviceToHost)); CK(cudaMemcpy(b, bout, sizeof(b), cudaMemcpyDeviceToHost));
    unsigned long long mx = 0, bytes = 0; for (int i = 0; i < G; ++i) { if (h[i] > mx) mx = h[i]; bytes += b[i]; }
    printf("NP %d mode %d chunk %5d pace %4d: %5.0f ns per barrier+payload, background %.2f TB/s\n", NP, mode, chunk, pace, (double)mx / iters, (double)bytes / mx / 1000.0);
    return 0;
}

int main() {
    const size_t per = (size_t)8 * 1024 * 1024, total = 148 * per;
    unsigned char* big; CK(cudaMalloc(&big, total)); CK(cudaMemset(big, 1, total));
    unsigned* cnt; float *data, *sink; unsigned long long *tout, *bout; int* stop;
    CK(cudaMalloc(&cnt, 256)); CK(cudaMalloc(&data, 2 * 4096 * 4)); CK(cudaMemset(data, 0, 2 * 4096 * 4));
    CK(cudaMalloc(&sink, 148 * 544 * 4)); CK(cudaMalloc(&tout, 148 * 8)); CK(cudaMalloc(&bout, 148 * 8)); CK(cudaMalloc(&stop, 4));
    int iters = 3000;
    run_cfg<1>(cnt, data, sink, iters, big, per, 0, 0, 0, tout, bout, stop);
    for (int pace : {4000, 2000, 1000, 400, 250, 100, 0}) run_cfg<1>(cnt, data, sink, iters, big, per, 1, 16384, pace, tout, bout, stop);
    for (int pace : {1000, 400, 200, 100, 0}) run_cfg<1>(cnt, data, sink, iters, big, per, 3, 8192, pace, tout, bout, stop);
    for (int pace : {1000, 400, 200, 100, 0}) run_cfg<2>(cnt, data, sink, iters, big, per, 3, 8192, pace, tout, bout, stop);
    return 0;
}
