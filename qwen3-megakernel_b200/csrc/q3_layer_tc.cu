// One persistent launch for everything of a decoder layer that is not attention, for decode batches of 4..64 sequences:
//
//     x += attn @ Wo^T  |  gate, up = (g2 * x) @ [Wg; Wu]^T  |  x += (silu(r2 gate) * (r2 up)) @ Wd^T  |
//     q, k, v (next layer) = (g1' * x) @ [Wq; Wk; Wv]^T
//
// (| = a grid barrier).  The layered path had ten launches for this, each with its own prologue, pipeline fill and tail;
// here one CTA per SM stays resident, the weight tiles of the NEXT phase are already on their way through the TMA ring
// while a phase's epilogue and the barrier run (weights are nobody's output, so the producer warp never waits for a
// barrier), and what used to be separate kernels between the GEMMs happens where the B operand is built:
//
//   * a phase's work is cut into (128 weight rows) x (a slice of K) units, one per CTA; the unit's activations - 32 or 64
//     tokens x 64 k per k block - are read as fp32 from L2, transformed (norm gain / SiLU * up), split into three bf16 planes (hi + mid + lo = the fp32 value) and written straight into shared
//     memory in the 128-byte-swizzled K-major layout tcgen05.mma reads; nothing goes through HBM as bf16 planes;
//   * RMS norm without a pass over the row: y = W (g * x * r) = r * (W (g * x)) for the per-token scalar r, so the GEMM
//     runs on g * x, the CTAs of weight tile 0 add the row sums of x^2 into a per-token accumulator on the side, and the
//     CONSUMER of the GEMM's output (the SiLU of the next phase, the head preparation of the attention kernel) applies
//     r = rsqrt(ssq / 1024 + eps);
//   * the residual stream is updated in place: the split-K partial tiles of Wo and down are added onto x itself.
//
// tcgen05.mma (kind::f16, M 128 weight rows x N tokens, fp32 accumulator in TMEM) is issued by one thread; sixteen warps
// build B and read the accumulator back (tcgen05.ld) for the epilogue's fp32 reds.  Every wait is bounded.
//
// Replaces, for batches, the phases 2-6 of the reference's layer loop (csrc/qwen3_step.cu:566-727: Wo + residual,
// norm, gate/up, SiLU, down + residual, norm, q/k/v), which there serve one sequence.
#include <cuda.h>

#include "q3_engine.h"
#include "q3_gemm_tc.h"
#include "q3_layer_tc.h"

namespace q3 {

constexpr int LK_WORKERS = 512;                 // warps 2..17: B builders and epilogue
constexpr int LK_THREADS = 64 + LK_WORKERS;     // warp 0: TMA producer (weights), warp 1: MMA issuer and TMEM owner
constexpr int LK_SYNCED = LK_THREADS - 32;      // the threads of a grid barrier: everyone but the producer warp
constexpr int LK_A_STAGES = 8;                  // weight tiles in flight: 8 x 16 KB
constexpr int LK_B_SLOTS = 3;
constexpr uint32_t LK_A_BYTES = 128 * 128;      // 128 weight rows x 64 k bf16
constexpr int LK_MAX_PHASES = 4;
constexpr bool LK_WORKER_SPIN = false;   // the workers' waits park (try_wait)
constexpr int LK_CHUNK = 6;                     // k blocks whose activations a builder thread requests at once (three with two source arrays)

enum { LK_ZERO = 0, LK_WO = 1, LK_GU = 2, LK_DN = 3, LK_QKV = 4 };

__device__ __forceinline__ uint32_t lk_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long lk_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

struct LkCtx {
    volatile int* abort_flag;
    uint32_t* status;
    unsigned long long wait_ns;
};

// SPIN: poll (mbarrier.test_wait; the lowest latency, for the two single-thread roles).  Otherwise try_wait, which parks
// the thread until the phase completes or a time slice ends and leaves the issue slots to the warps that still build
// (measured equal to polling for the phase times).
template <bool SPIN>
__device__ __forceinline__ bool lk_wait(uint64_t* bar, uint32_t parity, const LkCtx& cx, uint32_t site) {
    unsigned it = 0;
    unsigned long long t0 = 0;
    for (;;) {
        uint32_t ok;
        if (SPIN)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(lk_smem(bar)), "r"(parity) : "memory");
        else
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(lk_smem(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if (*cx.abort_flag) return false;
        if ((++it & 63u) == 0) {
            const unsigned long long t = lk_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > cx.wait_ns) {
                report(cx.status, ST_MBAR_TIMEOUT, site, parity);
                *cx.abort_flag = 1;
                return false;
            }
        }
    }
}

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t lk_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// The unit of CTA c in a phase: weight tile mt, k blocks [kb0, kb0 + nkb).  A phase has MT tiles of KB k blocks each;
// every tile is cut into S = min(G / MT, KB) slices of K, the CTAs beyond MT * S have no unit in this phase.
struct LkUnit {
    int has, mt, kb0, nkb;
};
__device__ __forceinline__ void lk_shape(int kind, int& MT, int& KB) {
    MT = kind == LK_WO ? HIDDEN / 128 : kind == LK_GU ? 2 * INTER / 128 : kind == LK_DN ? HIDDEN / 128 : QKV_DIM / 128;
    KB = kind == LK_WO ? Q_DIM / 64 : kind == LK_DN ? INTER / 64 : HIDDEN / 64;
}
__device__ __forceinline__ LkUnit lk_unit(int kind, int c, int G) {
    LkUnit u{0, 0, 0, 0};
    if (kind == LK_ZERO) return u;
    int MT, KB;
    lk_shape(kind, MT, KB);
    int S = G / MT;
    if (S > KB) S = KB;
    if (S < 1 || c >= MT * S) return u;
    u.has = 1;
    u.mt = c / S;
    const int sl = c % S;
    u.kb0 = sl * KB / S;
    u.nkb = (sl + 1) * KB / S - u.kb0;
    return u;
}

struct LkArgs {
    float* x;                 // [n_tok, 1024] residual stream, updated in place
    float* qkv;               // [n_tok, 4096] raw projections of the next layer (accumulated; unnormalised: see ssq)
    float* gate;              // [n_tok, 3072]
    float* up;                // [n_tok, 3072]
    float* ssq;               // [2][64]: row sums of x^2 behind the q/k/v GEMM ([0]) and behind the gate/up GEMM ([1])
    const float* attn;        // [n_tok, 2048] attention output (merged over the splits by the attention kernel)
    const bf16_raw* gain_ffn; // ln2 of this layer [1024]
    const bf16_raw* gain_qkv; // ln1 of the layer the q/k/v phase serves [1024]
    unsigned long long* sync; // [0] arrival counter (only ever grows), [1] its value when this launch started
    uint32_t* status;
    unsigned long long wait_ns;
    int layer;                // weights of Wo / gate / up / down
    int layer_qkv;            // weights of the q/k/v phase
    int n_tok;
    int n_phases;
    int phase[LK_MAX_PHASES];
};

// all worker threads of all CTAs clear n floats (n a multiple of 4, p 16-byte aligned)
__device__ __forceinline__ void lk_zero(float* p, int n, int c, int G, int wt) {
    const int n4 = n >> 2;
    const int i0 = (int)((long long)c * n4 / G), i1 = (int)((long long)(c + 1) * n4 / G);
    for (int i = i0 + wt; i < i1; i += LK_WORKERS) reinterpret_cast<float4*>(p)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

template <int N>
__device__ __forceinline__ void lk_tmem_ld(uint32_t (&r)[N], uint32_t taddr);
template <>
__device__ __forceinline__ void lk_tmem_ld<8>(uint32_t (&r)[8], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
template <>
__device__ __forceinline__ void lk_tmem_ld<32>(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
template <>
__device__ __forceinline__ void lk_tmem_ld<16>(uint32_t (&r)[16], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

// BN: the token tile (32 or 64).
template <int BN>
__global__ void __launch_bounds__(LK_THREADS, 1) layer_tc_kernel(const __grid_constant__ CUtensorMap tm_wq, const __grid_constant__ CUtensorMap tm_wk,
                                                                 const __grid_constant__ CUtensorMap tm_wv, const __grid_constant__ CUtensorMap tm_wo,
                                                                 const __grid_constant__ CUtensorMap tm_wg, const __grid_constant__ CUtensorMap tm_wu,
                                                                 const __grid_constant__ CUtensorMap tm_wd, const LkArgs a) {
    constexpr uint32_t PLANE = BN * 128, B_BYTES = 3 * PLANE;
    // the three planes of a slot lie one after the other: ONE B operand of 3 BN columns, one tcgen05.mma per k step (an
    // instruction costs about 150 clocks here whatever its N); the epilogue adds the three column groups
    constexpr uint32_t TMEM_COLS = 3 * BN <= 128 ? 128u : 256u;
    extern __shared__ __align__(1024) unsigned char lk_raw[];
    __shared__ __align__(8) uint64_t a_full[LK_A_STAGES], a_empty[LK_A_STAGES], b_ready[LK_B_SLOTS], b_free[LK_B_SLOTS], acc_full;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, G = gridDim.x;
    unsigned char* sA = lk_raw;
    unsigned char* sB = lk_raw + LK_A_STAGES * LK_A_BYTES;
    const LkCtx cx{&abort_flag, a.status, a.wait_ns};

    if (tid == 0) {
        for (int s = 0; s < LK_A_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(lk_smem(&a_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(lk_smem(&a_empty[s])) : "memory");
        }
        for (int s = 0; s < LK_B_SLOTS; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(lk_smem(&b_ready[s])), "r"(BN * 8) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(lk_smem(&b_free[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(lk_smem(&acc_full)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_flag = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lk_smem(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    // the counter's value when this launch started: CTA 0 stores the value for the next launch after the last barrier,
    // which every CTA reaches only after it has read this one
    const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(a.sync + 1);

    // Arrive at the grid barrier and wait for all G CTAs (the threads of warps 1..9; the producer warp runs ahead).
    int barriers = 0;
    auto grid_barrier = [&]() {
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"n"(LK_SYNCED) : "memory");
        ++barriers;
        if (tid == 64) {
            const unsigned long long target = epoch + (unsigned long long)G * (unsigned long long)barriers;
            __threadfence();
            asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(a.sync), "l"(1ull) : "memory");
            unsigned it = 0;
            unsigned long long t0 = 0;
            while (!abort_flag) {
                unsigned long long v;
                asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(a.sync) : "memory");
                if (v >= target) break;
                if ((++it & 63u) == 0) {
                    if (*reinterpret_cast<volatile uint32_t*>(a.status) != 0u) { abort_flag = 1; break; }   // another CTA gave up
                    const unsigned long long t = lk_ns();
                    if (t0 == 0) t0 = t;
                    else if (t - t0 > a.wait_ns) {
                        report(a.status, ST_BARRIER_TIMEOUT, 600u + (uint32_t)barriers, (uint32_t)(v - epoch));
                        abort_flag = 1;
                    }
                }
            }
            __threadfence();
        }
        asm volatile("bar.sync 1, %0;" ::"n"(LK_SYNCED) : "memory");
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    };

    if (warp == 0) {
        // ---------------------------------------------------------------------- TMA producer: weight tiles of every phase
        if (lane == 0) {
            int ai = 0;
            for (int ph = 0; ph < a.n_phases && !abort_flag; ++ph) {
                const int kind = a.phase[ph];
                const LkUnit u = lk_unit(kind, c, G);
                if (!u.has) continue;
                const CUtensorMap* tm;
                int row0;
                if (kind == LK_WO) { tm = &tm_wo; row0 = a.layer * HIDDEN + u.mt * 128; }
                else if (kind == LK_DN) { tm = &tm_wd; row0 = a.layer * HIDDEN + u.mt * 128; }
                else if (kind == LK_GU) {
                    const bool up = u.mt >= INTER / 128;
                    tm = up ? &tm_wu : &tm_wg;
                    row0 = a.layer * INTER + (u.mt - (up ? INTER / 128 : 0)) * 128;
                } else {
                    if (u.mt < Q_DIM / 128) { tm = &tm_wq; row0 = a.layer_qkv * Q_DIM + u.mt * 128; }
                    else if (u.mt < (Q_DIM + KV_DIM) / 128) { tm = &tm_wk; row0 = a.layer_qkv * KV_DIM + (u.mt - Q_DIM / 128) * 128; }
                    else { tm = &tm_wv; row0 = a.layer_qkv * KV_DIM + (u.mt - (Q_DIM + KV_DIM) / 128) * 128; }
                }
                for (int kb = 0; kb < u.nkb; ++kb, ++ai) {
                    const int s = ai % LK_A_STAGES;
                    if (ai >= LK_A_STAGES && !lk_wait<true>(&a_empty[s], ((ai / LK_A_STAGES) - 1) & 1, cx, 60)) break;
                    asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(lk_smem(&a_full[s])), "r"(LK_A_BYTES) : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(lk_smem(sA + (size_t)s * LK_A_BYTES)), "l"(tm), "r"((u.kb0 + kb) * 64), "r"(row0), "r"(lk_smem(&a_full[s])) : "memory");
                }
            }
            if (abort_flag) {   // nobody consumes the tiles still on their way: let them land before the CTA leaves (bounded)
                for (int j = ai > LK_A_STAGES ? ai - LK_A_STAGES : 0; j < ai; ++j) {
                    uint32_t ok = 0;
                    for (int it = 0; it < (1 << 16) && !ok; ++it)
                        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                     : "=r"(ok) : "r"(lk_smem(&a_full[j % LK_A_STAGES])), "r"((uint32_t)((j / LK_A_STAGES) & 1)) : "memory");
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------------- MMA issuer
        int ai = 0, bi = 0;
        for (int ph = 0; ph < a.n_phases; ++ph) {
            const LkUnit u = lk_unit(a.phase[ph], c, G);
            if (lane == 0 && u.has && !abort_flag) {
                // D fp32, A and B bf16, both K-major, M 128, N = BN
                const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((3 * BN) >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                bool ok = true;
                for (int kb = 0; kb < u.nkb && ok; ++kb, ++ai, ++bi) {
                    const int s = ai % LK_A_STAGES, sb = bi % LK_B_SLOTS;
                    ok = lk_wait<true>(&b_ready[sb], (bi / LK_B_SLOTS) & 1, cx, 62);
                    ok = ok && lk_wait<true>(&a_full[s], (ai / LK_A_STAGES) & 1, cx, 61);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t wa = lk_smem(sA + (size_t)s * LK_A_BYTES), xb = lk_smem(sB + (size_t)sb * B_BYTES);
                    {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t da = lk_desc(wa + k * 32), db = lk_desc(xb + k * 32);
                            const uint32_t accumulate = (kb | k) ? 1u : 0u;
                            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                         "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                                         ::"r"(tmem_base), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
                        }
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(lk_smem(&a_empty[s])) : "memory");
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(lk_smem(&b_free[sb])) : "memory");
                }
                if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(lk_smem(&acc_full)) : "memory");
            } else if (u.has) {
                ai += u.nkb; bi += u.nkb;
            }
            // lane 0's counters are the ones that matter; keep the others in step
            ai = __shfl_sync(0xffffffffu, ai, 0);
            bi = __shfl_sync(0xffffffffu, bi, 0);
            __syncwarp();
            if (ph + 1 < a.n_phases) grid_barrier();
        }
    } else {
        // ---------------------------------------------------------------------- workers: clear, build B, epilogue
        const int wt = tid - 64;
        // B builders: TPT = 8 threads per token, 8 k each = one 16-byte chunk per plane (with the 32-token tile half the
        // workers build)
        const int t = wt >> 3, kq = (wt & 7) * 8;
        const bool builder = wt < BN * 8;
        const bool live = builder && t < a.n_tok;
        const int quad = warp & 3, part = (warp - 2) >> 2;          // TMEM lanes [32 quad, +32), columns [part BN/4, +BN/4)
        int bi = 0, ui = 0;
        for (int ph = 0; ph < a.n_phases; ++ph) {
            const int kind = a.phase[ph];
            const LkUnit u = lk_unit(kind, c, G);
            // ---- buffers nobody reads or adds into during this phase ----
            if (kind == LK_ZERO || kind == LK_WO) {
                lk_zero(a.qkv, a.n_tok * QKV_DIM, c, G, wt);
                if (c == G - 1 && wt < 64) a.ssq[wt] = 0.f;
            }
            if (kind == LK_ZERO || (kind == LK_QKV && a.n_phases == LK_MAX_PHASES)) {
                lk_zero(a.gate, a.n_tok * INTER, c, G, wt);
                lk_zero(a.up, a.n_tok * INTER, c, G, wt);
                if (c == G - 1 && wt < 64) a.ssq[64 + wt] = 0.f;
            }
            if (u.has && !abort_flag) {
                bool ok = true;
                if (builder) {
                    // ---- B operand: three bf16 planes of the transformed activations.  All loads of up to LK_CHUNK k
                    // blocks are requested before the first one is used: a build is one L2 round trip, not one per block
                    const bool two = kind == LK_DN;                 // two source arrays (gate and up)
                    const int ld = kind == LK_WO ? Q_DIM : kind == LK_DN ? INTER : HIDDEN;
                    const float* src0 = (kind == LK_WO ? a.attn : kind == LK_DN ? a.gate : a.x) + (size_t)t * ld + kq;
                    const float* src1 = a.up + (size_t)t * INTER + kq;
                    const bf16_raw* gain = kind == LK_GU ? a.gain_ffn : a.gain_qkv;
                    const bool sums = (kind == LK_GU || kind == LK_QKV) && u.mt == 0;   // the CTAs of weight tile 0 cover every k once
                    float r_tok = 1.f, ss = 0.f;
                    if (kind == LK_DN && live) r_tok = rsqrtf(__ldcg(a.ssq + 64 + t) / (float)HIDDEN + EPS);
                    const int per = two ? LK_CHUNK / 2 : LK_CHUNK;  // k blocks per round of loads
                    // one k block's eight values -> three planes -> the B slot; false when a wait gave up
                    auto emit = [&](const float (&v)[8]) -> bool {
                        // hi + mid + lo by TRUNCATION: each plane takes the next eight significant bits, so the three of them
                        // hold the fp32 value exactly (as rounding does), at the price of a mask and a byte permute on the
                        // full-rate integer pipe instead of conversions
                        uint32_t hi[4], mid[4], lo[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float v0 = v[2 * i], v1 = v[2 * i + 1];
                            const uint32_t a0 = __float_as_uint(v0), a1 = __float_as_uint(v1);
                            hi[i] = __byte_perm(a0, a1, 0x7632);
                            const float r0 = v0 - __uint_as_float(a0 & 0xffff0000u), r1 = v1 - __uint_as_float(a1 & 0xffff0000u);
                            const uint32_t b0 = __float_as_uint(r0), b1 = __float_as_uint(r1);
                            mid[i] = __byte_perm(b0, b1, 0x7632);
                            const float s0 = r0 - __uint_as_float(b0 & 0xffff0000u), s1 = r1 - __uint_as_float(b1 & 0xffff0000u);
                            lo[i] = __byte_perm(__float_as_uint(s0), __float_as_uint(s1), 0x7632);
                        }
                        const int sb = bi % LK_B_SLOTS;
                        if (bi >= LK_B_SLOTS && !lk_wait<LK_WORKER_SPIN>(&b_free[sb], ((bi / LK_B_SLOTS) - 1) & 1, cx, 63)) return false;
                        // the token's 128-byte row of each plane, 16-byte chunks swizzled by the row
                        unsigned char* dst = sB + (size_t)sb * B_BYTES + (size_t)t * 128 + (uint32_t)(((kq >> 3) ^ (t & 7)) << 4);
                        *reinterpret_cast<uint4*>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4*>(dst + PLANE) = make_uint4(mid[0], mid[1], mid[2], mid[3]);
                        *reinterpret_cast<uint4*>(dst + 2 * PLANE) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(lk_smem(&b_ready[sb])) : "memory");
                        ++bi;
                        return true;
                    };
                    auto load8 = [&](float (&d)[8], const float* sp, bool on) {
                        float4 lo4 = make_float4(0.f, 0.f, 0.f, 0.f), hi4 = lo4;
                        if (on) { lo4 = __ldcg(reinterpret_cast<const float4*>(sp)); hi4 = __ldcg(reinterpret_cast<const float4*>(sp) + 1); }
                        d[0] = lo4.x; d[1] = lo4.y; d[2] = lo4.z; d[3] = lo4.w; d[4] = hi4.x; d[5] = hi4.y; d[6] = hi4.z; d[7] = hi4.w;
                    };
                    for (int kb0 = 0; kb0 < u.nkb && ok; kb0 += per) {
                        float q[LK_CHUNK][8];
                        if (two) {
#pragma unroll
                            for (int j = 0; j < LK_CHUNK / 2; ++j) {
                                const bool on = live && kb0 + j < u.nkb;
                                load8(q[2 * j], src0 + (size_t)(u.kb0 + kb0 + j) * 64, on);
                                load8(q[2 * j + 1], src1 + (size_t)(u.kb0 + kb0 + j) * 64, on);
                            }
                            // transform in place, all k blocks at once (independent chains for the scheduler to interleave)
#pragma unroll
                            for (int j = 0; j < LK_CHUNK / 2; ++j)
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const float gg = q[2 * j][i] * r_tok;
                                    q[2 * j][i] = __fdividef(gg, 1.f + __expf(-gg)) * (q[2 * j + 1][i] * r_tok);
                                }
#pragma unroll
                            for (int j = 0; j < LK_CHUNK / 2; ++j)
                                if (ok && kb0 + j < u.nkb) ok = emit(q[2 * j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < LK_CHUNK; ++j) load8(q[j], src0 + (size_t)(u.kb0 + kb0 + j) * 64, live && kb0 + j < u.nkb);
                            if (kind != LK_WO) {   // the norm gain; the row's scale is applied by the consumer of the GEMM
#pragma unroll
                                for (int j = 0; j < LK_CHUNK; ++j) {
                                    if (kb0 + j < u.nkb) {
                                        const uint4 gg = *reinterpret_cast<const uint4*>(gain + (size_t)(u.kb0 + kb0 + j) * 64 + kq);
                                        const float gf[8] = {bf_lo(gg.x), bf_hi(gg.x), bf_lo(gg.y), bf_hi(gg.y), bf_lo(gg.z), bf_hi(gg.z), bf_lo(gg.w), bf_hi(gg.w)};
#pragma unroll
                                        for (int i = 0; i < 8; ++i) { ss = fmaf(q[j][i], q[j][i], ss); q[j][i] *= gf[i]; }
                                    }
                                }
                            }
#pragma unroll
                            for (int j = 0; j < LK_CHUNK; ++j)
                                if (ok && kb0 + j < u.nkb) ok = emit(q[j]);
                        }
                    }
                    if (sums) {   // (uniform over the warp: the kind and the tile are the CTA's)
                        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                        if (live && kq == 0) atomicAdd(a.ssq + (kind == LK_GU ? 64 : 0) + t, ss);
                    }
                } else {
                    bi += u.nkb;
                }
                // ---- epilogue: the partial tile is added into the output (x itself for Wo and down) ----
                if (ok) ok = lk_wait<LK_WORKER_SPIN>(&acc_full, ui & 1, cx, 64);
                ++ui;
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    float* out;
                    int ldo, col0;
                    if (kind == LK_WO || kind == LK_DN) { out = a.x; ldo = HIDDEN; col0 = u.mt * 128; }
                    else if (kind == LK_GU) {
                        const bool up = u.mt >= INTER / 128;
                        out = up ? a.up : a.gate; ldo = INTER; col0 = (u.mt - (up ? INTER / 128 : 0)) * 128;
                    } else { out = a.qkv; ldo = QKV_DIM; col0 = u.mt * 128; }
                    constexpr int NC = BN / 4;
                    uint32_t r[NC], r1[NC], r2[NC];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(part * NC);
                    lk_tmem_ld<NC>(r, taddr);
                    lk_tmem_ld<NC>(r1, taddr + (uint32_t)BN);
                    lk_tmem_ld<NC>(r2, taddr + (uint32_t)(2 * BN));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < NC; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r1[j]) + __uint_as_float(r2[j]));
                    float* dst = out + col0 + quad * 32 + lane;
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        const int tok = part * NC + j;
                        if (tok < a.n_tok) atomicAdd(dst + (size_t)tok * ldo, __uint_as_float(r[j]));
                    }
                }
            } else if (u.has) {
                bi += u.nkb; ++ui;
            }
            if (ph + 1 < a.n_phases) grid_barrier();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (c == 0 && tid == 64 && !abort_flag) a.sync[1] = epoch + (unsigned long long)G * (unsigned long long)(a.n_phases - 1);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static size_t lk_smem_bytes(int bn) { return (size_t)LK_A_STAGES * LK_A_BYTES + (size_t)LK_B_SLOTS * 3 * bn * 128; }

bool layer_tc_supports(const q3_engine* e, int batch) {
    return e->lk_state != nullptr && e->planes != nullptr && batch >= Q3_TC_MIN_BATCH && batch <= 64 && e->sm_count >= 2 * INTER / 128;
}

cudaError_t launch_layer_tc(q3_engine* e, int mode, int layer, int n_tok, cudaStream_t st) {
    const q3_weights& w = e->w;
    const int L = e->cfg.n_layers;
    CUtensorMap tm[7];
    const void* ptr[7] = {w.wq, w.wk, w.wv, w.wo, w.wg, w.wu, w.wd};
    const uint64_t rows[7] = {(uint64_t)L * Q_DIM, (uint64_t)L * KV_DIM, (uint64_t)L * KV_DIM, (uint64_t)L * HIDDEN,
                              (uint64_t)L * INTER, (uint64_t)L * INTER, (uint64_t)L * HIDDEN};
    const uint64_t cols[7] = {HIDDEN, HIDDEN, HIDDEN, Q_DIM, HIDDEN, HIDDEN, INTER};
    for (int i = 0; i < 7; ++i)
        if (!tc_cached_map(ptr[i], rows[i], cols[i], 128, &tm[i])) return cudaErrorUnknown;

    LkArgs a{};
    a.x = e->x; a.qkv = e->qkv; a.gate = e->gate; a.up = e->up;
    a.ssq = reinterpret_cast<float*>(e->lk_state);
    a.sync = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(e->lk_state) + 512);
    a.attn = e->attn;
    a.status = e->status;
    a.wait_ns = (e->cfg.wait_limit_us > 0 ? (unsigned long long)e->cfg.wait_limit_us : 200000ull) * 1000ull;
    a.n_tok = n_tok;
    const bf16_raw* ln1 = reinterpret_cast<const bf16_raw*>(w.ln1);
    const bf16_raw* ln2 = reinterpret_cast<const bf16_raw*>(w.ln2);
    if (mode == LK_MODE_FIRST) {
        a.layer = 0; a.layer_qkv = 0;
        a.n_phases = 2; a.phase[0] = LK_ZERO; a.phase[1] = LK_QKV;
    } else {
        a.layer = layer; a.layer_qkv = layer + 1;
        a.phase[0] = LK_WO; a.phase[1] = LK_GU; a.phase[2] = LK_DN; a.phase[3] = LK_QKV;
        a.n_phases = mode == LK_MODE_LAST ? 3 : 4;
    }
    a.gain_ffn = ln2 + (size_t)a.layer * HIDDEN;
    a.gain_qkv = ln1 + (size_t)(a.layer_qkv < L ? a.layer_qkv : 0) * HIDDEN;

    const int bn = n_tok <= 32 ? 32 : 64;
    auto kernel = bn == 32 ? layer_tc_kernel<32> : layer_tc_kernel<64>;
    const size_t smem = lk_smem_bytes(bn);
    {
        static bool attr_set[64][2] = {};
        int dev = 0;
        cudaError_t err = cudaGetDevice(&dev);
        if (err != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        if (!attr_set[dev][bn == 64]) {   // (a benign race between host threads: the attribute is set to the same value)
            err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess) return err;
            attr_set[dev][bn == 64] = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(e->sm_count); cfg.blockDim = dim3(LK_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;   // the grid barriers need every CTA resident
    at[0].val.cooperative = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[6], a);
}

}  // namespace q3
