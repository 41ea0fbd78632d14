// Causal attention for prefill: one prompt, positions 0..T-1, K/V rows read from the bf16 cache that
// head_prep has just filled.  Flash-attention tiling on mma.sync.m16n8k16: a block owns 64 queries
// of one head (4 warps x 16 rows), walks the key tiles up to its diagonal, keeps scores, the running
// max / sum and the output tile in registers.  Q enters as two bf16 terms (hi + lo) so the scores
// carry fp32-grade accuracy into the exponent; probabilities are rounded to bf16 for P.V, the
// accumulation is fp32.  GQA: query head h reads kv head h / 2.
//
// Replaces the [16, T, T] masked score matrix of the reference's prefill (qwen3mk/prefill.py:71-75).
#include "q3_engine.h"

namespace q3 {

constexpr int PA_ROW = 136;   // elements between K / V rows in shared memory: 128 + 8 of padding (ldmatrix bank spread)

__device__ __forceinline__ uint32_t pa_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pa_ldsm(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pa_ldsm_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pa_pack(float lo, float hi) { return (uint32_t)f_to_bf(lo) | ((uint32_t)f_to_bf(hi) << 16); }

struct PrefillAttnArgs {
    const float* qkv;        // [T, 4096] fp32 after head_prep (q normalised + RoPE, unscaled)
    const bf16_raw* kcache;  // layer slice [cap, 8, 128]
    const bf16_raw* vcache;
    float* attn;             // [T, 2048]
    int T;
    int paired;              // the grid has half as many blocks as query tiles (long prompts)
};

__global__ void __launch_bounds__(128) prefill_attn_kernel(const PrefillAttnArgs a) {
    __shared__ __align__(16) bf16_raw sK[64 * PA_ROW];
    __shared__ __align__(16) bf16_raw sV[64 * PA_ROW];
    const int h = blockIdx.y, kvh = h >> 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, q4 = lane & 3;
    // Causal work grows with the query tile's index: a block takes tile i and then tile n - 1 - i, so that every block
    // walks n + 1 key tiles and the grid is one even wave instead of two ragged ones.
    const int n_qt = (a.T + 63) / 64;
    for (int pass = 0; pass < 2; ++pass) {
    const int qt = pass ? n_qt - 1 - (int)blockIdx.x : (int)blockIdx.x;
    if (pass && (!a.paired || qt <= (int)blockIdx.x)) break;   // unpaired grid; or the middle tile of an odd count, done in pass 0
    const int row0 = qt * 64 + warp * 16 + g, row1 = row0 + 8;   // this thread's two query rows

    // ---- Q fragments, scaled, as hi + lo bf16 ----
    uint32_t qh[8][4], ql[8][4];
    {
        const float* q0 = a.qkv + (size_t)min(row0, a.T - 1) * QKV_DIM + h * HEAD_DIM;
        const float* q1 = a.qkv + (size_t)min(row1, a.T - 1) * QKV_DIM + h * HEAD_DIM;
#pragma unroll
        for (int d = 0; d < 8; ++d) {
            const float2 v[4] = {*reinterpret_cast<const float2*>(q0 + 16 * d + 2 * q4), *reinterpret_cast<const float2*>(q1 + 16 * d + 2 * q4),
                                 *reinterpret_cast<const float2*>(q0 + 16 * d + 8 + 2 * q4), *reinterpret_cast<const float2*>(q1 + 16 * d + 8 + 2 * q4)};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x = v[i].x * ATTN_SCALE, y = v[i].y * ATTN_SCALE;
                const bf16_raw xh = f_to_bf(x), yh = f_to_bf(y);
                qh[d][i] = (uint32_t)xh | ((uint32_t)yh << 16);
                ql[d][i] = pa_pack(x - bf_to_f(xh), y - bf_to_f(yh));
            }
        }
    }
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const bf16_raw* kbase = a.kcache + kvh * HEAD_DIM;
    const bf16_raw* vbase = a.vcache + kvh * HEAD_DIM;
    for (int kt = 0; kt <= qt; ++kt) {
        __syncthreads();   // the previous tile is consumed
        for (int i = tid; i < 64 * 16; i += 128) {   // 64 keys x 16 chunks of 16 bytes, K and V
            const int r = i >> 4, ck = i & 15;
            const int key = min(kt * 64 + r, a.T - 1);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(pa_smem(sK + r * PA_ROW + ck * 8)), "l"(kbase + (size_t)key * KV_DIM + ck * 8) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(pa_smem(sV + r * PA_ROW + ck * 8)), "l"(vbase + (size_t)key * KV_DIM + ck * 8) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        // ---- S = Q K^T for 16 rows x 64 keys ----
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int dd = 0; dd < 4; ++dd) {   // two 16-dim k-tiles per ldmatrix.x4
                uint32_t kb[4];
                const int mi = lane >> 3, r = lane & 7;
                pa_ldsm(kb, pa_smem(sK + (8 * j + r) * PA_ROW + 32 * dd + 8 * (mi & 1) + 16 * (mi >> 1)));
                pa_mma(s[j], qh[2 * dd], kb[0], kb[1]);
                pa_mma(s[j], ql[2 * dd], kb[0], kb[1]);
                pa_mma(s[j], qh[2 * dd + 1], kb[2], kb[3]);
                pa_mma(s[j], ql[2 * dd + 1], kb[2], kb[3]);
            }
        }
        // ---- causal mask on the diagonal tile, online softmax ----
        if (kt == qt) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int key = kt * 64 + 8 * j + 2 * q4;
                if (key > row0) s[j][0] = -INFINITY;
                if (key + 1 > row0) s[j][1] = -INFINITY;
                if (key > row1) s[j][2] = -INFINITY;
                if (key + 1 > row1) s[j][3] = -INFINITY;
            }
        }
        float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) { t0 = fmaxf(t0, fmaxf(s[j][0], s[j][1])); t1 = fmaxf(t1, fmaxf(s[j][2], s[j][3])); }
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
        t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
        const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);   // finite: key 0 is visible to every row
        const float c0 = __expf(m0 - n0), c1 = __expf(m1 - n1);
        m0 = n0; m1 = n1;
        float p0 = 0.f, p1 = 0.f;
        uint32_t pf[4][4];   // P as A fragments: k-tile kk = keys 16 kk .. 16 kk + 15
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float e0 = __expf(s[j][0] - n0), e1 = __expf(s[j][1] - n0), e2 = __expf(s[j][2] - n1), e3 = __expf(s[j][3] - n1);
            p0 += e0 + e1; p1 += e2 + e3;
            pf[j >> 1][(j & 1) * 2] = pa_pack(e0, e1);
            pf[j >> 1][(j & 1) * 2 + 1] = pa_pack(e2, e3);
        }
        l0 = l0 * c0 + p0; l1 = l1 * c1 + p1;
#pragma unroll
        for (int n = 0; n < 16; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int nn = 0; nn < 8; ++nn) {   // two 8-dim n-tiles per ldmatrix.x4.trans
                uint32_t vb[4];
                const int mi = lane >> 3, r = lane & 7;
                pa_ldsm_t(vb, pa_smem(sV + (16 * kk + 8 * (mi & 1) + r) * PA_ROW + 8 * (2 * nn + (mi >> 1))));
                pa_mma(o[2 * nn], pf[kk], vb[0], vb[1]);
                pa_mma(o[2 * nn + 1], pf[kk], vb[2], vb[3]);
            }
        }
    }
    // row sums live in the four lanes of a quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
        if (row0 < a.T) *reinterpret_cast<float2*>(a.attn + (size_t)row0 * Q_DIM + h * HEAD_DIM + 8 * n + 2 * q4) = make_float2(o[n][0] * i0, o[n][1] * i0);
        if (row1 < a.T) *reinterpret_cast<float2*>(a.attn + (size_t)row1 * Q_DIM + h * HEAD_DIM + 8 * n + 2 * q4) = make_float2(o[n][2] * i1, o[n][3] * i1);
    }
    }   // pass
}

cudaError_t launch_prefill_attn(const float* qkv, const void* kcache_layer, const void* vcache_layer, float* attn, int T, cudaStream_t st) {
    const int n_qt = (T + 63) / 64;
    const int paired = n_qt >= 16 ? 1 : 0;   // short prompts need every tile as a block of its own to fill the GPU
    PrefillAttnArgs a{qkv, reinterpret_cast<const bf16_raw*>(kcache_layer), reinterpret_cast<const bf16_raw*>(vcache_layer), attn, T, paired};
    prefill_attn_kernel<<<dim3(paired ? (n_qt + 1) / 2 : n_qt, Q_HEADS), 128, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace q3
