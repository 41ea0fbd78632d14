// Causal attention for prefill on the 5th-generation tensor cores: tcgen05.mma with accumulators in TMEM, K/V tiles
// brought in by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a two-stage mbarrier pipeline.
//
// One CTA owns 64 query positions of ONE KV HEAD GROUP: its M = 128 rows are the two query heads of the group (rows
// 0..63 head 2g, rows 64..127 head 2g + 1), so every K/V tile is fetched once for both heads (GQA sharing).  It walks
// the key tiles (128 keys) up to its diagonal:
//     S  = Q K^T      M 128 x N 128 keys x K 128 dims: Q as TWO bf16 planes (hi + lo, so the scores carry fp32-grade
//                     accuracy into the exponent), both K-major operands      -> TMEM columns [0, 128) / [128, 256)
//     P  = exp(S - m) sixteen warps, four threads per row (32 keys each): tcgen05.ld, causal mask on the diagonal tile,
//                     running max / sum, P rounded to bf16 into shared memory in the K-major swizzled operand layout
//     PV = P V        M 128 x N 128 dims x K 128 keys; V is the MN-major B operand straight from its TMA tile
//                                                                             -> TMEM columns [256, 384) / [384, 512)
//     O  = O c + PV   in registers (32 dims per thread), rescaled by c = exp(m_old - m_new); written at the end as the
//                     bf16 plane(s) the Wo GEMM reads, so no fp32 round trip and no separate splitting kernel
// S and PV are double-buffered in TMEM (all 512 columns): the MMA thread issues S of tile t + 1 before it waits for P
// of tile t, and the softmax warps fold PV of tile t - 1 into O after they have posted P of tile t, so the exponentials
// (the bottleneck: 16 K of them per tile on the SFUs) run back to back while the tensor pipe works beside them.
// Long prompts launch one block per (query tile, kv group) in order of work (a query tile has 1..n key tiles), so that
// the SMs that finish early pick up the light tiles; short ones a (query tile, kv group) grid.  Every mbarrier wait is
// bounded.
//
// Replaces the [16, T, T] masked score matrix of the reference's prefill (qwen3mk/prefill.py:71-75).
#include <cuda.h>

#include "q3_engine.h"
#include "q3_gemm_tc.h"

namespace q3 {

constexpr int AT_PARTS = 4;               // threads per row in the softmax: each takes 128 / AT_PARTS columns of S and of O
constexpr int AT_SOFT = 128 * AT_PARTS;   // softmax / output threads: warps 0..15
constexpr int AT_THREADS = AT_SOFT + 64;  // + warp 16 TMA producer, warp 17 MMA issuer and TMEM owner
constexpr int AT_QT = 64;                 // query positions per CTA pass
constexpr int AT_KT = 128;                // keys per tile
constexpr int AT_STAGES = 2;
constexpr uint32_t AT_BOX = 128 * 128;    // bytes of one [128 rows x 64 columns] bf16 box, 128-byte swizzle
constexpr uint32_t AT_Q_BYTES = 2 * AT_BOX, AT_P_BYTES = 2 * AT_BOX, AT_KV_BYTES = 2 * AT_BOX;   // 128 x 128 bf16 = two boxes
// Q hi, Q lo, P, stages x (K, V) = 224 KB; with the 3 KB of static shared memory below that is all an SM has, so the
// dynamic part must start 1024-aligned by itself (the extern array is declared so) and the static part must stay <= 3 KB
constexpr size_t AT_SMEM = 2 * AT_Q_BYTES + AT_P_BYTES + AT_STAGES * 2 * AT_KV_BYTES;
constexpr unsigned long long AT_WAIT_NS = 200ull * 1000 * 1000;

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long at_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t* status, uint32_t site) {
    unsigned it = 0;
    unsigned long long t0 = 0;
    for (;;) {
        uint32_t ok;
        // test_wait, not try_wait: a try_wait on a phase that is not complete yet parks the thread for a while, and a tile
        // has eight hand-offs between the MMA thread and the softmax warps
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(at_smem(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if ((++it & 63u) == 0) {
            const unsigned long long t = at_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > AT_WAIT_NS) {
                if (status) report(status, ST_MBAR_TIMEOUT, site, parity);
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart (as in the GEMM)
__device__ __forceinline__ uint64_t at_desc_k(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand (V: rows = keys = the K index, 64 contiguous dims per 128-byte row), 128-byte swizzle: the next 64
// dims are one box further (leading byte offset), the next 8 keys 1024 bytes further (stride byte offset)
__device__ __forceinline__ uint64_t at_desc_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(AT_BOX >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// byte offset of element (row, col) of a [128 x 128] bf16 operand stored as two swizzled boxes of 64 columns
__device__ __forceinline__ uint32_t at_swz(int row, int col) {
    const int box = col >> 6, c = col & 63;
    return (uint32_t)box * AT_BOX + (uint32_t)row * 128u + (uint32_t)((((c >> 3) ^ (row & 7)) << 4) + ((c & 7) << 1));
}

// The special-function pipe (16 results a cycle and SM) is this kernel's bottleneck: a tile needs 16 K exponentials and
// the conversion of 16 K probabilities to bf16.  So: one ex2 per element (log2(e) is folded into the scale of Q) and one
// conversion per PAIR of elements.
__device__ __forceinline__ float at_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t at_pack_bf16(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

__device__ __forceinline__ void at_ld32(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}

struct PrefillAttnTcArgs {
    const float* qkv;     // [T, 4096] fp32 after head_prep (q normalised + RoPE, unscaled)
    bf16_raw* planes;     // [nsplit][plane_rows][2048] bf16: the output, already split for the Wo GEMM (hi, then lo = what hi left)
    int plane_rows, nsplit;
    int T;
    int paired;           // the grid has half as many blocks as query tiles
    int heavy_first;      // a one-dimensional grid of (query tile, kv group) blocks, the tiles with the most key tiles first
    uint32_t* status;
};

__global__ void __launch_bounds__(AT_THREADS, 1) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                                        const __grid_constant__ CUtensorMap tm_v, const PrefillAttnTcArgs a) {
    extern __shared__ __align__(1024) unsigned char at_raw[];
    __shared__ __align__(8) uint64_t k_full[AT_STAGES], v_full[AT_STAGES], k_empty[AT_STAGES], v_empty[AT_STAGES], s_full[2], p_full, o_full[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    // Per-row partial maxima of the four column parts, exchanged once per key tile with ONE barrier: two buffers, picked by the
    // tile's parity, so that a warp that is a tile ahead never overwrites what a slower one has yet to read.  Stored as bf16
    // rounded UP (the shared maximum only has to be an upper bound that every thread of the row agrees on), which keeps the
    // two buffers in the 2 KB the kernel has left.  The same bytes hold the fp32 partial sums at the end.
    __shared__ __align__(16) unsigned short pm16[2][AT_PARTS][128];
    float (*pm)[128] = reinterpret_cast<float (*)[128]>(&pm16[0][0][0]);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = a.heavy_first ? (int)blockIdx.x % KV_HEADS : (int)blockIdx.y;   // kv head; query heads 2g and 2g + 1
    unsigned char* sQh = at_raw;
    unsigned char* sQl = sQh + AT_Q_BYTES;
    unsigned char* sP = sQl + AT_Q_BYTES;
    unsigned char* sKV = sP + AT_P_BYTES;           // stage s: K at s * 2 * AT_KV_BYTES, V right after it

    if (tid == 0) {
        for (int s = 0; s < AT_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&k_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&v_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&k_empty[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&v_empty[s])) : "memory");
        }
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&s_full[b])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(at_smem(&o_full[b])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(&p_full)), "r"(AT_SOFT) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_flag = 0;
    }
    if (warp == AT_SOFT / 32 + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(&tmem_base_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    const int n_qt = (a.T + AT_QT - 1) / AT_QT;
    int it0 = 0;                                    // key tiles consumed before this pass: every barrier's phase is counted on it
    for (int pass = 0; pass < 2; ++pass) {
        const int qt = a.heavy_first ? n_qt - 1 - (int)blockIdx.x / KV_HEADS : (pass ? n_qt - 1 - (int)blockIdx.x : (int)blockIdx.x);
        if (pass && (a.heavy_first || !a.paired || qt <= (int)blockIdx.x)) break;
        const int q0 = qt * AT_QT;
        const int n_kt = (q0 + AT_QT - 1) / AT_KT + 1;          // key tiles up to and including the diagonal one

        // ---- Q of both heads, scaled, as hi + lo bf16 planes in the operand layout (all 320 threads) ----
        for (int i = tid; i < 128 * 32; i += AT_THREADS) {       // 128 rows x 32 groups of 4 dims
            const int row = i >> 5, c4 = (i & 31) * 4;
            const int pos = min(q0 + (row & 63), a.T - 1), head = 2 * g + (row >> 6);
            const float4 v = *reinterpret_cast<const float4*>(a.qkv + (size_t)pos * QKV_DIM + head * HEAD_DIM + c4);
            constexpr float QS = ATTN_SCALE * 1.4426950408889634f;   // scores in units of log2: probabilities are ex2(s - m)
            const float x[4] = {v.x * QS, v.y * QS, v.z * QS, v.w * QS};
            bf16_raw h[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) { h[j] = f_to_bf(x[j]); l[j] = f_to_bf(x[j] - bf_to_f(h[j])); }
            const uint32_t off = at_swz(row, c4);
            *reinterpret_cast<uint2*>(sQh + off) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
            *reinterpret_cast<uint2*>(sQl + off) = make_uint2((uint32_t)l[0] | ((uint32_t)l[1] << 16), (uint32_t)l[2] | ((uint32_t)l[3] << 16));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();

        if (warp == AT_SOFT / 32) {
            // ------------------------------------------------------------------ TMA producer
            if (lane == 0) {
                // K and V of a tile share a stage but are released separately: the K half is free as soon as S of its tile has
                // been computed, a whole tile before the V half (after PV), so the next K is on its way that much earlier
                for (int t = 0; t < n_kt; ++t) {
                    const int it = it0 + t, s = it % AT_STAGES;
                    unsigned char* sk = sKV + (size_t)s * 2 * AT_KV_BYTES;
                    unsigned char* sv = sk + AT_KV_BYTES;
                    if (it >= AT_STAGES && !at_wait(&k_empty[s], ((it / AT_STAGES) - 1) & 1, &abort_flag, a.status, 40)) break;
                    asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(&k_full[s])), "r"(AT_KV_BYTES) : "memory");
#pragma unroll
                    for (int b = 0; b < 2; ++b)        // the two 64-dim halves of the head
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(at_smem(sk + b * AT_BOX)), "l"(&tm_k), "r"(g * HEAD_DIM + 64 * b), "r"(t * AT_KT), "r"(at_smem(&k_full[s])) : "memory");
                    if (it >= AT_STAGES && !at_wait(&v_empty[s], ((it / AT_STAGES) - 1) & 1, &abort_flag, a.status, 47)) break;
                    asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(&v_full[s])), "r"(AT_KV_BYTES) : "memory");
#pragma unroll
                    for (int b = 0; b < 2; ++b)
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(at_smem(sv + b * AT_BOX)), "l"(&tm_v), "r"(g * HEAD_DIM + 64 * b), "r"(t * AT_KT), "r"(at_smem(&v_full[s])) : "memory");
                }
            }
        } else if (warp == AT_SOFT / 32 + 1) {
            // ------------------------------------------------------------------ MMA issuer
            if (lane == 0) {
                // D fp32, A and B bf16, M 128, N 128; bit 16: B is MN-major (V)
                const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                const uint32_t idesc_o = idesc_s | (1u << 16);
                auto issue_s = [&](int t) -> bool {    // S = (Q hi + Q lo) K^T of key tile t, into S buffer it & 1
                    const int it = it0 + t, s = it % AT_STAGES;
                    if (!at_wait(&k_full[s], (it / AT_STAGES) & 1, &abort_flag, a.status, 41)) return false;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sk = at_smem(sKV + (size_t)s * 2 * AT_KV_BYTES);
#pragma unroll
                    for (int plane = 0; plane < 2; ++plane) {
                        const uint32_t sq = at_smem(plane ? sQl : sQh);
#pragma unroll
                        for (int k = 0; k < 8; ++k) {  // 16 dims a step: four steps per 64-dim box
                            const uint32_t o = (uint32_t)(k >> 2) * AT_BOX + (uint32_t)(k & 3) * 32u;
                            const uint64_t da = at_desc_k(sq + o), db = at_desc_k(sk + o);
                            const uint32_t acc = (plane | k) ? 1u : 0u;
                            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                         "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                                         ::"r"(tmem_base + (uint32_t)(it & 1) * 128u), "l"(da), "l"(db), "r"(idesc_s), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
                        }
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(&s_full[it & 1])) : "memory");
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(&k_empty[s])) : "memory");
                    return true;
                };
                bool ok = issue_s(0);
                for (int t = 0; t < n_kt && ok; ++t) {
                    const int it = it0 + t, s = it % AT_STAGES;
                    // S of the next tile first: its buffer was read before P of tile t - 1 was posted, and the exponentials of
                    // tile t can be followed by those of tile t + 1 without waiting for the tensor pipe
                    if (t + 1 < n_kt) ok = issue_s(t + 1);
                    ok = ok && at_wait(&p_full, it & 1, &abort_flag, a.status, 42) && at_wait(&v_full[s], (it / AT_STAGES) & 1, &abort_flag, a.status, 43);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sv = at_smem(sKV + (size_t)s * 2 * AT_KV_BYTES + AT_KV_BYTES), sp = at_smem(sP);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {      // 16 keys a step; PV buffer it & 1 (its previous tenant, tile t - 2, was folded into O before P of tile t was posted)
                        const uint64_t da = at_desc_k(sp + (uint32_t)(k >> 2) * AT_BOX + (uint32_t)(k & 3) * 32u);
                        const uint64_t db = at_desc_mn(sv + (uint32_t)k * 2048u);
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                                     ::"r"(tmem_base + 256u + (uint32_t)(it & 1) * 128u), "l"(da), "l"(db), "r"(idesc_o), "r"(k ? 1u : 0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(&o_full[it & 1])) : "memory");
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(&v_empty[s])) : "memory");
                }
            }
        } else {
            // ------------------------------------------------------------------ softmax and output: row = TMEM lane, part = 32 columns
            const int row = (warp & 3) * 32 + lane, part = warp >> 2;
            const int qpos = q0 + (row & 63);
            const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(part * 32);
            float o[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = 0.f;
            float m = -INFINITY, lsum = 0.f, c_prev = 1.f;
            bool ok = true;
            // O = O c + PV of tile `it` (this thread's 32 dims), once its MMAs have completed
            auto fold = [&](int it, float c) -> bool {
                if (!at_wait(&o_full[it & 1], (it >> 1) & 1, &abort_flag, a.status, 45)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t v0[32];
                at_ld32(v0, trow + 256u + (uint32_t)(it & 1) * 128u);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; ++j) o[j] = fmaf(o[j], c, __uint_as_float(v0[j]));
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                return true;
            };
            for (int t = 0; t < n_kt && ok; ++t) {
                const int it = it0 + t;
                ok = at_wait(&s_full[it & 1], (it >> 1) & 1, &abort_flag, a.status, 44);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t r0[32];
                at_ld32(r0, trow + (uint32_t)(it & 1) * 128u);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int key0 = t * AT_KT + part * 32;
                if (t == n_kt - 1) {   // the diagonal tile: causal mask (it also hides keys past the prompt)
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (key0 + j > qpos) r0[j] = 0xff800000u;            // -inf
                }
                float tmax = -INFINITY;
#pragma unroll
                for (int j = 0; j < 32; ++j) tmax = fmaxf(tmax, __uint_as_float(r0[j]));
                {
                    const uint32_t tb = __float_as_uint(tmax);   // towards +inf: truncation for negative values, carry for positive ones
                    pm16[it & 1][part][row] = (unsigned short)((tb & 0x80000000u) ? (tb >> 16) : ((tb + 0xffffu) >> 16));
                }
                asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFT) : "memory");
                float mn = m;                                   // finite from the first tile on: key 0 is visible to every row
#pragma unroll
                for (int q = 0; q < AT_PARTS; ++q) mn = fmaxf(mn, __uint_as_float((uint32_t)pm16[it & 1][q][row] << 16));
                const float c = at_ex2(m - mn);
                m = mn;
                float psum = 0.f;
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float e0 = at_ex2(__uint_as_float(r0[2 * j]) - mn), e1 = at_ex2(__uint_as_float(r0[2 * j + 1]) - mn);
                    psum += e0 + e1;
                    pk[j] = at_pack_bf16(e0, e1);
                }
                lsum = lsum * c + psum;
                // the P buffer is free once PV of the previous tile has completed (long ago in practice)
                if (t > 0 && !at_wait(&o_full[(it - 1) & 1], ((it - 1) >> 1) & 1, &abort_flag, a.status, 46)) { ok = false; break; }
                // P[row][32 part .. 32 part + 31]: four 16-byte chunks of box part / 2, chunk slots 4 (part & 1) + ch
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
                    *reinterpret_cast<uint4*>(sP + (uint32_t)(part >> 1) * AT_BOX + (uint32_t)row * 128u + (uint32_t)((((part & 1) * 4 + ch) ^ (row & 7)) << 4)) =
                        make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(at_smem(&p_full)) : "memory");
                // fold the PREVIOUS tile's PV into O while the tensor pipe works on this one
                if (t > 0) ok = fold(it - 1, c_prev);
                c_prev = c;
            }
            if (ok) ok = fold(it0 + n_kt - 1, c_prev);
            // the row sum is split over the parts' key ranges
            asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFT) : "memory");   // the last tile's maxima have been read
            pm[part][row] = lsum;
            asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFT) : "memory");
            float ltot = 0.f;
#pragma unroll
            for (int q = 0; q < AT_PARTS; ++q) ltot += pm[q][row];
            const float inv = 1.f / ltot;
            if (ok && qpos < a.T) {   // 32 dims = 64 contiguous bytes per plane
                const size_t off = (size_t)qpos * Q_DIM + (2 * g + (row >> 6)) * HEAD_DIM + part * 32;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float x = o[j + 2 * q] * inv, y = o[j + 2 * q + 1] * inv;
                        hi[q] = at_pack_bf16(x, y);
                        lo[q] = at_pack_bf16(x - bf_lo(hi[q]), y - bf_hi(hi[q]));
                    }
                    *reinterpret_cast<uint4*>(a.planes + off + j) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    if (a.nsplit > 1) *reinterpret_cast<uint4*>(a.planes + (size_t)a.plane_rows * Q_DIM + off + j) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
        }
        it0 += n_kt;
        __syncthreads();   // every MMA of this pass has completed (the last O was read): Q and P may be rewritten
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == AT_SOFT / 32 + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

cudaError_t launch_prefill_attn_tc(const float* qkv, const void* kcache_layer, const void* vcache_layer, int cap_rows, void* planes,
                                   int plane_rows, int nsplit, int T, uint32_t* status, cudaStream_t st) {
    if (nsplit < 1 || nsplit > 2) return cudaErrorInvalidValue;
    CUtensorMap tk, tv;
    // the layer's cache as a [cap_rows, 1024] bf16 matrix; boxes of 64 columns x 128 rows (keys past the cache read as zeros)
    if (!tc_cached_map(kcache_layer, (uint64_t)cap_rows, (uint64_t)KV_DIM, AT_KT, &tk)) return cudaErrorUnknown;
    if (!tc_cached_map(vcache_layer, (uint64_t)cap_rows, (uint64_t)KV_DIM, AT_KT, &tv)) return cudaErrorUnknown;
    {
        static bool attr_set[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        if (!attr_set[dev]) {   // (a benign race between host threads: the attribute is set to the same value)
            e = cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM);
            if (e != cudaSuccess) return e;
            attr_set[dev] = true;
        }
    }
    const int n_qt = (T + AT_QT - 1) / AT_QT;
    // More blocks than SMs: one block per (query tile, kv group), dispatched in the order of their work (a query tile has
    // 1..n key tiles), so that the SMs that finish early pick up the light tiles: greedy longest-first over all 148 SMs,
    // where pairing a light with a heavy tile per CTA used 128 of them (measured at 2048 tokens: see the profile).
    const int heavy_first = n_qt * KV_HEADS > 148 ? 1 : 0, paired = 0;
    PrefillAttnTcArgs a{qkv, reinterpret_cast<bf16_raw*>(planes), plane_rows, nsplit, T, paired, heavy_first, status};
    const dim3 grid = heavy_first ? dim3(n_qt * KV_HEADS) : dim3(paired ? (n_qt + 1) / 2 : n_qt, KV_HEADS);
    prefill_attn_tc_kernel<<<grid, AT_THREADS, AT_SMEM, st>>>(tk, tv, a);
    return cudaGetLastError();
}

}  // namespace q3
