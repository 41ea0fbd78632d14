// How long does a CTA need to ISSUE a burst of cp.async (16-byte LDGSTS) copies, and how long until the burst has
// landed, when every SM of the GPU does the same at the same moment?  480 threads of each of 148 CTAs issue
// `per_thread` copies from cold global memory (a different region every repetition), stamp the clock, then wait for
// completion.  The issue time tells how many bytes the load/store path accepts before the issuing warps stall, i.e.
// how much a kernel may issue in a window where its warps are needed again soon.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o cp_async_issue cp_async_issue.cu
#include <algorithm>
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("%s: %s\n", #x, cudaGetErrorString(e)); return 1; } } while (0)
constexpr int THREADS = 480;
__global__ void __launch_bounds__(THREADS, 1) burst(const unsigned char* src, size_t per_cta, int per_thread, unsigned long long* out) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const unsigned char* base = src + (size_t)blockIdx.x * per_cta;
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    __syncthreads();
    const long long t0 = clock64();
    for (int k = 0; k < per_thread; ++k) {
        const int i = k * THREADS + tid;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 16), "l"(base + (size_t)i * 16) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const long long t1 = clock64();
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const long long t2 = clock64();
    __syncthreads();
    // slowest warp of the CTA: lane 0 of every warp records, the host takes the maximum
    if ((tid & 31) == 0) {
        out[((size_t)blockIdx.x * 16 + (tid >> 5)) * 2] = (unsigned long long)(t1 - t0);
        out[((size_t)blockIdx.x * 16 + (tid >> 5)) * 2 + 1] = (unsigned long long)(t2 - t0);
    }
}
int main() {
    const size_t per_cta = (size_t)256 * 1024, reps = 8;
    const size_t total = (size_t)148 * per_cta * reps;   // 310 MB: every repetition reads a region no cache holds
    unsigned char* d; CK(cudaMalloc(&d, total)); CK(cudaMemset(d, 1, total));
    unsigned long long* out; CK(cudaMalloc(&out, 148 * 16 * 2 * 8)); CK(cudaMemset(out, 0, 148 * 16 * 2 * 8));
    CK(cudaFuncSetAttribute(burst, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    int dev = 0, khz = 0; CK(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    const int per_thread[] = {1, 2, 4, 6, 8, 12, 17, 24, 28};
    for (int pi = 0; pi < 9; ++pi) {
        double issue = 0, land = 0;
        for (size_t r = 0; r < reps; ++r) {
            burst<<<148, THREADS, 224 * 1024>>>(d + r * 148 * per_cta, per_cta, per_thread[pi], out);
            CK(cudaDeviceSynchronize());
            static unsigned long long h[148 * 16 * 2];
            CK(cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost));
            unsigned long long is[148], ld[148];
            for (int c = 0; c < 148; ++c) {
                is[c] = ld[c] = 0;
                for (int w = 0; w < 15; ++w) { is[c] = std::max(is[c], h[(c * 16 + w) * 2]); ld[c] = std::max(ld[c], h[(c * 16 + w) * 2 + 1]); }
            }
            std::sort(is, is + 148); std::sort(ld, ld + 148);
            if (r >= 2) { issue += is[74]; land += ld[74]; }   // median CTA, first two repetitions are warm-up
        }
        issue /= (reps - 2); land /= (reps - 2);
        const double kb = per_thread[pi] * THREADS * 16 / 1024.0;
        printf("%5.1f KB per SM: issued after %6.0f cycles, landed after %6.0f cycles (%.2f us at the SM clock); %.0f GB/s over the GPU\n",
               kb, issue, land, land / (khz / 1e3), 148 * kb * 1024 / (land / (khz * 1e3)) / 1e9);
    }
    return 0;
}
