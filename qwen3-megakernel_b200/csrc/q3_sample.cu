// Temperature / top-k sampling over the fp32 logits a decode step writes.
//
// The reference decodes greedily inside its kernel and leaves sampling to the caller, who gets the fp32
// logits for that purpose (csrc/qwen3_step.cu:175 writes them, qwen3mk/kernel.py:44-50 returns them).  This is
// that next step on the GPU, so that a sampled token can feed the following launch without a trip to the host.
//
// One block of 1024 threads per row; every pass streams the row (593 KB for the full vocabulary, L2 resident after
// the first pass):
//   1. the row maximum, together with the first histogram of
//   2. top-k: the k-th largest logit by a radix select over the order-preserving integer image of the floats
//      (three passes of 11, 11 and 10 bits, a histogram in shared memory each; coalesced, strided reads); every
//      logit >= that value is kept, so ties at the threshold are all kept;
//   3. weights w_i = exp((l_i - max) / T) of the kept logits, summed per thread over a contiguous chunk of the
//      row (index order matters from here on), then scanned over the block;
//   4. the token is the first index whose inclusive prefix sum exceeds u * total, u in [0, 1) supplied per row
//      by the caller (a seeded generator on the host side keeps runs reproducible); the thread whose chunk
//      brackets the target walks its chunk in the same order it summed it.
// T <= 0 or k == 1 degenerate to the arg-max (ties -> lowest index), like the decode kernels.
#include "q3_engine.h"

namespace q3 {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned ordered_key(float f) {   // monotonic in the float's value
    const unsigned b = __float_as_uint(f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, int vocab, float temperature, int top_k,
                                                               const float* __restrict__ uniform, long long* __restrict__ out) {
    __shared__ float s_f[SAMPLE_THREADS];
    __shared__ int s_i[SAMPLE_THREADS];
    __shared__ unsigned s_hist[2048];
    __shared__ unsigned s_prefix, s_need;
    __shared__ float s_total;
    __shared__ int s_pick;
    const int tid = threadIdx.x, row_id = blockIdx.x;
    const float* row = logits + (size_t)row_id * vocab;
    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int i0 = min(vocab, tid * chunk), i1 = min(vocab, i0 + chunk);
    const bool select = top_k > 1 && top_k < vocab && temperature > 0.f;

    // ---- 1. maximum (and its lowest index); the histogram of the keys' top 11 bits on the side ----
    for (int b = tid; b < 2048; b += SAMPLE_THREADS) s_hist[b] = 0u;
    __syncthreads();
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }   // a thread's indices ascend: the first maximum is the lowest
        if (select) atomicAdd(&s_hist[ordered_key(v) >> 21], 1u);
    }
    s_f[tid] = bv; s_i[tid] = bi;
    __syncthreads();
    for (int o = SAMPLE_THREADS / 2; o > 0; o >>= 1) {
        if (tid < o) {
            const float v = s_f[tid + o];
            const int ix = s_i[tid + o];
            if (v > s_f[tid] || (v == s_f[tid] && ix < s_i[tid])) { s_f[tid] = v; s_i[tid] = ix; }
        }
        __syncthreads();
    }
    const float vmax = s_f[0];
    const int imax = s_i[0];
    __syncthreads();
    if (!(temperature > 0.f) || top_k == 1) {
        if (tid == 0) out[row_id] = imax;
        return;
    }

    // ---- 2. threshold: the k-th largest key (0 keeps everything) ----
    unsigned thresh = 0u;
    if (select) {
        if (tid == 0) { s_prefix = 0u; s_need = (unsigned)top_k; }
        __syncthreads();
        // digit d of a key: bits [shift, shift + width)
        for (int pass = 0; pass < 3; ++pass) {
            const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0), width = pass == 2 ? 10 : 11;
            const unsigned prefix = s_prefix;
            if (pass > 0) {
                for (int b = tid; b < 2048; b += SAMPLE_THREADS) s_hist[b] = 0u;
                __syncthreads();
                const unsigned mask = 0xffffffffu << (shift + width);
                for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                    const unsigned k = ordered_key(row[i]);
                    if ((k & mask) == prefix) atomicAdd(&s_hist[(k >> shift) & ((1u << width) - 1u)], 1u);
                }
                __syncthreads();
            }
            if (tid == 0) {   // walk the bins from the top until `need` keys are covered
                unsigned need = s_need, b = (1u << width) - 1u;
                for (;; --b) {
                    const unsigned n = s_hist[b];
                    if (n >= need || b == 0u) break;
                    need -= n;
                }
                s_need = need;
                s_prefix = prefix | (b << shift);
            }
            __syncthreads();
        }
        thresh = s_prefix;
    }

    // ---- 3. weights of the kept logits: per-thread chunk sums, then a scan over the block ----
    const float inv_t = 1.f / temperature;
    float mine = 0.f;
    for (int i = i0; i < i1; ++i) {
        const float v = row[i];
        if (ordered_key(v) >= thresh) mine += __expf((v - vmax) * inv_t);
    }
    s_f[tid] = mine;
    __syncthreads();
    // inclusive scan (Hillis-Steele over 1024 entries)
    for (int o = 1; o < SAMPLE_THREADS; o <<= 1) {
        const float add = (tid >= o) ? s_f[tid - o] : 0.f;
        __syncthreads();
        s_f[tid] += add;
        __syncthreads();
    }
    if (tid == SAMPLE_THREADS - 1) { s_total = s_f[tid]; s_pick = -1; }
    __syncthreads();

    // ---- 4. the first index whose inclusive prefix exceeds u * total ----
    const float target = uniform[row_id] * s_total;
    const float before = tid ? s_f[tid - 1] : 0.f;   // the scanned prefixes partition [0, total) exactly
    if (mine > 0.f && before <= target && target < s_f[tid]) {
        float run = before;
        int pick = -1, last_kept = -1;
        for (int i = i0; i < i1; ++i) {
            const float v = row[i];
            if (ordered_key(v) >= thresh) {
                run += __expf((v - vmax) * inv_t);
                last_kept = i;
                if (run > target) { pick = i; break; }
            }
        }
        s_pick = pick >= 0 ? pick : last_kept;   // rounding may leave the target a hair beyond the chunk's own sum
    }
    __syncthreads();
    if (tid == 0) out[row_id] = s_pick >= 0 ? s_pick : imax;   // u * total rounded up to the total: the mode is as good a token as any
}

}  // namespace q3

extern "C" int q3_sample(const float* logits, int32_t batch, int32_t vocab, float temperature, int32_t top_k,
                         const float* uniform, int64_t* out_tokens, void* stream) {
    if (!logits || !out_tokens) return q3::engine_fail(nullptr, Q3_ERR_INVALID, "q3_sample: logits and out_tokens are required");
    if (batch < 1 || vocab < 1 || top_k < 0) return q3::engine_fail(nullptr, Q3_ERR_INVALID, "q3_sample: batch=%d vocab=%d top_k=%d out of range", batch, vocab, top_k);
    if (temperature > 0.f && top_k != 1 && !uniform) return q3::engine_fail(nullptr, Q3_ERR_INVALID, "q3_sample: sampling needs one uniform number per row");
    q3::sample_kernel<<<batch, q3::SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, vocab, temperature, top_k, uniform,
                                                                              reinterpret_cast<long long*>(out_tokens));
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return q3::engine_fail(nullptr, Q3_ERR_CUDA, "q3_sample: %s", cudaGetErrorString(err));
    return Q3_OK;
}
