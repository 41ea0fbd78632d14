// TMA bulk-copy (cp.async.bulk) streaming throughput against copy size: every CTA streams its share of a 1.2 GB
// buffer through a shared-memory ring.  Shows the fixed cost per bulk copy (about 230 ns of TMA time whatever the
// size): 2 KB copies cap at 1.25 TB/s over the GPU, 16 KB copies stream above 7 TB/s.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tma_copy_size tma_copy_size.cu
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("%s: %s\n", #x, cudaGetErrorString(e)); return 1; } } while (0)
__device__ __forceinline__ uint32_t su32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__global__ void __launch_bounds__(64, 1) tma_stream(const unsigned char* src, size_t per_cta, int chunk, int depth, unsigned long long* out) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bars[64];
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < depth; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(su32(&bars[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const unsigned char* base = src + (size_t)blockIdx.x * per_cta;
    const int n = (int)(per_cta / chunk);
    unsigned long long t0 = 0, t1 = 0;
    if (tid == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (int k = 0; k < n + depth; ++k) {
            if (k >= depth) {   // wait for chunk k - depth (the ring slot is then free again)
                const int s = (k - depth) % depth; const unsigned par = ((k - depth) / depth) & 1;
                unsigned ok = 0;
                while (!ok) asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(su32(&bars[s])), "r"(par) : "memory");
            }
            if (k < n) {
                const int s = k % depth;
                asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(su32(&bars[s])), "r"(chunk) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(su32(smem + (size_t)s * chunk)), "l"(base + (size_t)k * chunk), "r"(chunk), "r"(su32(&bars[s])) : "memory");
            }
        }
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        out[blockIdx.x] = t1 - t0;
    }
}
int main() {
    const size_t total = (size_t)148 * 8 * 1024 * 1024;   // 1.16 GB
    unsigned char* d; CK(cudaMalloc(&d, total)); CK(cudaMemset(d, 1, total));
    unsigned long long* out; CK(cudaMalloc(&out, 148 * 8));
    CK(cudaFuncSetAttribute(tma_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const int chunks[] = {2048, 4096, 8192, 16384, 32768};
    const int inflight_kb[] = {8, 16, 32, 64, 128};
    for (int ci = 0; ci < 5; ++ci) for (int fi = 0; fi < 5; ++fi) {
        const int chunk = chunks[ci]; const int depth = inflight_kb[fi] * 1024 / chunk;
        if (depth < 1 || depth > 64) continue;
        const size_t per = (size_t)8 * 1024 * 1024;
        for (int rep = 0; rep < 2; ++rep) { tma_stream<<<148, 64, (size_t)depth * chunk>>>(d, per, chunk, depth, out); CK(cudaDeviceSynchronize()); }
        unsigned long long h[148]; CK(cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost));
        unsigned long long mx = 0; for (int i = 0; i < 148; ++i) if (h[i] > mx) mx = h[i];
        printf("chunk %5d B, in flight %3d KB/SM (depth %2d): %.0f GB/s\n", chunk, inflight_kb[fi], depth, (double)total / mx);
    }
    return 0;
}
