// Tensor-core GEMM for prefill and large-batch decode: out[t, n] (+)= sum_k W[n, k] * X[t, k].
//
// Blackwell path: TMA (cp.async.bulk.tensor, 128-byte swizzle) stages W and X tiles in shared memory,
// one elected thread issues tcgen05.mma (kind::f16, bf16 operands, fp32 accumulator in TMEM), four
// warps read the accumulator back with tcgen05.ld and store it.  The weight matrix is the M operand
// (128 weight rows per tile) and the tokens are the N operand, so a decode batch of 32..256 tokens is
// one N tile and every weight byte crosses HBM once.
//
// Exact activations: the fp32 activations are passed as up to three bf16 planes (hi, mid, lo with
// X = hi + mid + lo); each W tile is multiplied with every plane into the same accumulator.  With
// three planes the result equals the fp32 product of the bf16 weights up to accumulation order;
// large-batch decode uses that (the extra MMAs are free while the weights stream from HBM), prefill
// uses one or two planes.
//
// Replaces the dense `xn @ w.T` products of the reference's PyTorch prefill (qwen3mk/prefill.py:61-80).
#include <cuda.h>

#include <mutex>
#include <vector>

#include "q3_engine.h"
#include "q3_gemm_tc.h"

namespace q3 {

constexpr int MAX_DEVICES = 64;
static std::mutex& host_lock() { static std::mutex m; return m; }   // guards the per-device set-up flags and the tensor-map cache

constexpr int TC_THREADS = 192;    // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..5: epilogue
constexpr int TC_BM = 128;         // weight rows per tile (UMMA M)
constexpr int TC_BK = 64;          // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr unsigned long long TC_WAIT_NS = 200ull * 1000 * 1000;

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long tc_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

// bounded mbarrier wait; on timeout sets *abort_flag and returns false
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t* status, uint32_t site) {
    unsigned it = 0;
    unsigned long long t0 = 0;
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(tc_smem(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if ((++it & 63u) == 0) {
            const unsigned long long t = tc_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > TC_WAIT_NS) {
                report(status, ST_MBAR_TIMEOUT, site, parity);
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, 8-row
// groups 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell)
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);        // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused with swizzle), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                              // version
    d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void tc_ld32(uint32_t (&r)[32], uint32_t taddr) {   // 32 columns of this warp's 32 TMEM lanes; no wait
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w0,
                                                                const __grid_constant__ CUtensorMap tm_w1,
                                                                const __grid_constant__ CUtensorMap tm_w2,
                                                                const __grid_constant__ CUtensorMap tm_x, const GemmTcParams p) {
    extern __shared__ __align__(1024) unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // which weight matrix this tile belongs to (grouped launches), and its first row inside that matrix
    int grp = 0, tile = blockIdx.x;
    if (p.n_groups > 1) {
        if (tile >= p.g_tiles[0]) { tile -= p.g_tiles[0]; grp = 1; }
        if (grp == 1 && p.n_groups > 2 && tile >= p.g_tiles[1]) { tile -= p.g_tiles[1]; grp = 2; }
    }
    const CUtensorMap* tm_w = grp == 0 ? &tm_w0 : (grp == 1 ? &tm_w1 : &tm_w2);
    float* const out = p.n_groups > 1 ? (grp == 0 ? p.g_out[0] : grp == 1 ? p.g_out[1] : p.g_out[2]) : p.out;
    const int ldo = p.n_groups > 1 ? (grp == 0 ? p.g_ldo[0] : grp == 1 ? p.g_ldo[1] : p.g_ldo[2]) : p.ldo;
    const int n_rows = p.n_groups > 1 ? (grp == 0 ? p.g_tiles[0] : grp == 1 ? p.g_tiles[1] : p.g_tiles[2]) * TC_BM : p.n_rows;
    const int m0 = tile * TC_BM;                // first weight row of this tile
    const int n0 = blockIdx.y * BN;             // first token of this tile
    // split-K: grid.z slices of the k blocks; partial tiles are added into `out` with fp32 atomics
    const int kb_begin = blockIdx.z * p.kb_per_split;
    const int nkb = min(p.K / TC_BK - kb_begin, p.kb_per_split);
    const int nsplit = p.nsplit;
    const uint32_t a_bytes = TC_BM * TC_BK * 2, b_bytes = BN * TC_BK * 2;
    const uint32_t stage_bytes = a_bytes + nsplit * b_bytes;
    const int stages = p.stages;
    // 1024-byte aligned base (the swizzle pattern repeats every 1024 bytes)
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&full_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&empty_bar[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&acc_bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_flag = 0;
    }
    // The planes of a stage lie one after the other in shared memory, each BN rows of 128 bytes: up to 256 rows they are
    // ONE B operand of nsplit * BN columns, so a k step is one tcgen05.mma instead of nsplit (an instruction costs about 150
    // clocks here whatever its N), and the epilogue adds the planes' column groups.  Beyond 256 columns: one MMA per plane
    // into the same BN columns.
    const bool wide = nsplit > 1 && nsplit * BN <= 256;
    const uint32_t tmem_cols = wide ? (nsplit * BN <= 128 ? 128u : 256u) : (uint32_t)(BN < 32 ? 32 : BN);
    if (warp == 1) {   // TMEM allocation: one warp, power-of-two column count >= 32
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    // Barriers and the accumulator are set up.  The successor may start its own set-up now; this kernel waits for its
    // predecessor only where it first touches what that one produced: the weights are nobody's output, so their tiles
    // are requested BEFORE the wait (their HBM latency overlaps the predecessor's tail), the activation planes and
    // the output stores come after it.
    pdl_launch();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const int ahead = min(nkb, stages);   // the first ring of stages: weight tiles before the wait
            for (int kb = 0; kb < ahead; ++kb) {
                unsigned char* st = base + (size_t)kb * stage_bytes;
                asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(&full_bar[kb])), "r"(stage_bytes) : "memory");
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(tc_smem(st)), "l"(tm_w), "r"((kb_begin + kb) * TC_BK), "r"(m0), "r"(tc_smem(&full_bar[kb])) : "memory");
            }
            pdl_wait();
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % stages;
                if (kb >= stages && !tc_wait(&empty_bar[s], ((kb / stages) - 1) & 1, &abort_flag, p.status, 30)) break;
                unsigned char* st = base + (size_t)s * stage_bytes;
                if (kb >= ahead) {
                    asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(&full_bar[s])), "r"(stage_bytes) : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(tc_smem(st)), "l"(tm_w), "r"((kb_begin + kb) * TC_BK), "r"(m0), "r"(tc_smem(&full_bar[s])) : "memory");
                }
                for (int sp = 0; sp < nsplit; ++sp)
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(tc_smem(st + a_bytes + sp * b_bytes)), "l"(&tm_x), "r"((kb_begin + kb) * TC_BK), "r"(sp * p.plane_rows + n0),
                                   "r"(tc_smem(&full_bar[s])) : "memory");
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: D fp32, A and B bf16, both K-major, N = BN (or all planes side by side), M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((wide ? nsplit * BN : BN) >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            const int n_mma = wide ? 1 : nsplit;
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % stages;
                ok = tc_wait(&full_bar[s], (kb / stages) & 1, &abort_flag, p.status, 31);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = tc_smem(base + (size_t)s * stage_bytes);
                for (int sp = 0; sp < n_mma; ++sp) {
                    const uint32_t sb = sa + a_bytes + sp * b_bytes;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        const uint64_t da = tc_desc(sa + k * 32), db = tc_desc(sb + k * 32);
                        const uint32_t accumulate = (kb | sp | k) ? 1u : 0u;
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                                     ::"r"(tmem_base), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
                    }
                }
                // the stage may be overwritten once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&empty_bar[s])) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&acc_bar)) : "memory");
        }
    } else {
        // ------------------------------------------------------------------ epilogue: TMEM -> registers -> global
        const int quad = warp & 3;                      // TMEM lanes [32 quad, 32 quad + 32) belong to this warp
        const bool ok = tc_wait(&acc_bar, 0, &abort_flag, p.status, 32);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_wait();   // before the first store (the output may be something the predecessor still reads)
        if (ok) {
            const int row = m0 + quad * 32 + lane;      // weight row = output column
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32);
                tc_ld32(r, taddr);
                if constexpr (BN >= 64) {
                    // all column groups of these tokens are requested before the one wait (a TMEM round trip each otherwise:
                    // batch 64 x 1024 2478 -> 2424 us per step).  Not for the 32-token tile: the 64 extra registers cost it
                    // two of its five CTAs per SM (batch 8 x 1024 1083 -> 1153 us).
                    uint32_t q1[32], q2[32];
                    if (wide) {
                        tc_ld32(q1, taddr + (uint32_t)BN);
                        if (nsplit > 2) tc_ld32(q2, taddr + (uint32_t)(2 * BN));
                    }
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (wide) {   // add the other planes' columns of the same tokens
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            float v = __uint_as_float(r[j]) + __uint_as_float(q1[j]);
                            if (nsplit > 2) v += __uint_as_float(q2[j]);
                            r[j] = __float_as_uint(v);
                        }
                    }
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (wide) {
                        for (int sp = 1; sp < nsplit; ++sp) {
                            uint32_t q[32];
                            tc_ld32(q, taddr + (uint32_t)(sp * BN));
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
                        }
                    }
                }
                if (row < n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int t = n0 + c * 32 + j;
                        if (t < p.n_tok) {
                            float v = __uint_as_float(r[j]);
                            float* dst = out + (size_t)t * ldo + row;
                            if (p.epi == TC_EPI_ATOMIC) {
                                atomicAdd(dst, v);   // split-K: `out` already holds zero or the residual
                            } else {
                                if (p.epi == TC_EPI_RESID) v += p.resid[(size_t)t * p.ldr + row];
                                *dst = v;
                            }
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// The same GEMM for prompts as a PERSISTENT kernel: one CTA per SM walks a list of work items (a tile of 128 weight rows x
// 256 tokens).  What the one-tile-per-CTA kernel does in
// series - fill the pipeline, the MMAs, the read-back of 128 KB of accumulator - overlaps here:
//   * the TMA ring never drains between items (the producer runs ahead into the next item's k blocks),
//   * two accumulators in TMEM (2 x 256 columns = all of it): the epilogue warps read item i out while the MMA thread
//     already accumulates item i + 1,
//   * N = 256 per tcgen05.mma halves the shared-memory operand traffic per flop against N = 128.
// Items are numbered with the weight tile fastest, so that the CTAs of a round share a few token tiles in L2.
// ------------------------------------------------------------------------------------------------
//
// DUAL: the FFN's gate and up in one item - the same 128 rows of Wg and of Wu against a tile of 128 tokens, four
// accumulators of 128 columns - and an epilogue that writes silu(gate) * up as the bf16 plane the down GEMM reads.  The
// fp32 gate and up matrices (2 x 25 MB per layer at 2048 tokens) and the kernel that read them back are gone, and the
// exponentials of the epilogue hide behind the next item's MMAs.
constexpr int TP_BN = 256;
constexpr int TP_THREADS = 64 + 256;   // warp 0: TMA, warp 1: MMA, warps 2..9: epilogue (two warps per TMEM lane quadrant, half the columns each)
struct GemmPersistItems {
    int n_items, m_tiles, n_ttiles;   // items = token tiles x weight tiles
    bf16_raw* silu_out;               // DUAL: [silu_rows][n_rows] bf16
    int silu_rows;                    // rows of that plane (multiple of 128): rows past the prompt are written as zeros
};

template <bool DUAL>
__global__ void __launch_bounds__(TP_THREADS, 1) gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap tm_w0,
                                                                        const __grid_constant__ CUtensorMap tm_w1,
                                                                        const __grid_constant__ CUtensorMap tm_w2,
                                                                        const __grid_constant__ CUtensorMap tm_x, const GemmTcParams p,
                                                                        const GemmPersistItems w) {
    constexpr int BN = DUAL ? 128 : TP_BN;          // tokens per item
    constexpr int ACC = DUAL ? 2 * BN : BN;         // TMEM columns of one accumulator buffer (DUAL: gate | up)
    extern __shared__ __align__(1024) unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsplit = p.nsplit, stages = p.stages;
    const uint32_t a_bytes = (DUAL ? 2 : 1) * TC_BM * TC_BK * 2, b_bytes = BN * TC_BK * 2;   // DUAL: the Wg tile, then the Wu tile
    const uint32_t stage_bytes = a_bytes + nsplit * b_bytes;
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&full_bar[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&empty_bar[s])) : "memory");
        }
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&acc_full[b])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 256;" ::"r"(tc_smem(&acc_empty[b])) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        abort_flag = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"((uint32_t)(2 * ACC)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch();

    // item -> (k slice, token tile, weight tile -> matrix of a grouped launch and row inside it)
    struct Item { int grp, m0, n0, kb_begin, nkb; };
    auto decode = [&](int it) {
        Item r;
        const int per_slice = w.m_tiles * w.n_ttiles;
        const int ks = it / per_slice, rem = it - ks * per_slice;
        int tile = rem % w.m_tiles;
        r.n0 = (rem / w.m_tiles) * BN;
        r.grp = 0;
        if (!DUAL && p.n_groups > 1) {
            if (tile >= p.g_tiles[0]) { tile -= p.g_tiles[0]; r.grp = 1; }
            if (r.grp == 1 && p.n_groups > 2 && tile >= p.g_tiles[1]) { tile -= p.g_tiles[1]; r.grp = 2; }
        }
        r.m0 = tile * TC_BM;
        r.kb_begin = ks * p.kb_per_split;
        r.nkb = min(p.K / TC_BK - r.kb_begin, p.kb_per_split);
        return r;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            pdl_wait();
            int gi = 0;
            for (int it = blockIdx.x; it < w.n_items && !abort_flag; it += gridDim.x) {
                const Item r = decode(it);
                const CUtensorMap* tm_w = r.grp == 0 ? &tm_w0 : (r.grp == 1 ? &tm_w1 : &tm_w2);
                for (int kb = 0; kb < r.nkb; ++kb, ++gi) {
                    const int s = gi % stages;
                    if (gi >= stages && !tc_wait(&empty_bar[s], ((gi / stages) - 1) & 1, &abort_flag, p.status, 36)) break;
                    unsigned char* st = base + (size_t)s * stage_bytes;
                    asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(tc_smem(&full_bar[s])), "r"(stage_bytes) : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(tc_smem(st)), "l"(tm_w), "r"((r.kb_begin + kb) * TC_BK), "r"(r.m0), "r"(tc_smem(&full_bar[s])) : "memory");
                    if (DUAL)
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(tc_smem(st + a_bytes / 2)), "l"(&tm_w1), "r"((r.kb_begin + kb) * TC_BK), "r"(r.m0), "r"(tc_smem(&full_bar[s])) : "memory");
                    for (int sp = 0; sp < nsplit; ++sp)
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(tc_smem(st + a_bytes + sp * b_bytes)), "l"(&tm_x), "r"((r.kb_begin + kb) * TC_BK), "r"(sp * p.plane_rows + r.n0),
                                       "r"(tc_smem(&full_bar[s])) : "memory");
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            int gi = 0, li = 0;
            bool ok = true;
            for (int it = blockIdx.x; it < w.n_items && ok; it += gridDim.x, ++li) {
                const Item r = decode(it);
                const int acc = li & 1;
                // the accumulator is free once the epilogue warps have read its previous tenant out
                if (li >= 2) ok = tc_wait(&acc_empty[acc], ((li >> 1) - 1) & 1, &abort_flag, p.status, 37);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < r.nkb && ok; ++kb, ++gi) {
                    const int s = gi % stages;
                    ok = tc_wait(&full_bar[s], (gi / stages) & 1, &abort_flag, p.status, 38);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = tc_smem(base + (size_t)s * stage_bytes);
                    for (int sp = 0; sp < nsplit; ++sp) {
                        const uint32_t sb = sa + a_bytes + sp * b_bytes;
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k) {
                            const uint64_t da = tc_desc(sa + k * 32), db = tc_desc(sb + k * 32);
                            const uint32_t accumulate = (kb | sp | k) ? 1u : 0u;
                            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                         "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                                         ::"r"(tmem_base + (uint32_t)(acc * ACC)), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
                            if (DUAL) {
                                const uint64_t du = tc_desc(sa + a_bytes / 2 + k * 32);
                                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                                             ::"r"(tmem_base + (uint32_t)(acc * ACC + BN)), "l"(du), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
                            }
                        }
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&empty_bar[s])) : "memory");
                }
                if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&acc_full[acc])) : "memory");
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: TMEM -> registers -> global
        const int quad = warp & 3, half = (warp - 2) >> 2;   // TMEM lanes [32 quad, +32), columns [half BN / 2, + BN / 2)
        pdl_wait();   // before the first store (the output may be something the predecessor still reads)
        int li = 0;
        bool ok = true;
        for (int it = blockIdx.x; it < w.n_items && ok; it += gridDim.x, ++li) {
            const Item r = decode(it);
            const int acc = li & 1;
            float* const out = p.n_groups > 1 ? (r.grp == 0 ? p.g_out[0] : r.grp == 1 ? p.g_out[1] : p.g_out[2]) : p.out;
            const int ldo = p.n_groups > 1 ? (r.grp == 0 ? p.g_ldo[0] : r.grp == 1 ? p.g_ldo[1] : p.g_ldo[2]) : p.ldo;
            ok = tc_wait(&acc_full[acc], (li >> 1) & 1, &abort_flag, p.status, 39);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = r.m0 + quad * 32 + lane;    // weight row = output column (every tile is a full 128 rows)
            if (DUAL) {
                // Reading TMEM while the MMAs of the next item run costs about a microsecond per round trip, whatever its width:
                // two rounds of 64 tokens (gate and up requested together, one wait) instead of sixteen narrow ones
                for (int c = half; c == half; ++c) {   // 64 tokens: this warp's half of the item
                    if (r.n0 + c * 64 >= w.silu_rows) break;
                    uint32_t g[64], u[64];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * ACC + c * 64);
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
                                 : "=r"(g[0]), "=r"(g[1]), "=r"(g[2]), "=r"(g[3]), "=r"(g[4]), "=r"(g[5]), "=r"(g[6]), "=r"(g[7]), "=r"(g[8]), "=r"(g[9]), "=r"(g[10]), "=r"(g[11]), "=r"(g[12]), "=r"(g[13]), "=r"(g[14]), "=r"(g[15]), "=r"(g[16]), "=r"(g[17]), "=r"(g[18]), "=r"(g[19]), "=r"(g[20]), "=r"(g[21]), "=r"(g[22]), "=r"(g[23]), "=r"(g[24]), "=r"(g[25]), "=r"(g[26]), "=r"(g[27]), "=r"(g[28]), "=r"(g[29]), "=r"(g[30]), "=r"(g[31]), "=r"(g[32]), "=r"(g[33]), "=r"(g[34]), "=r"(g[35]), "=r"(g[36]), "=r"(g[37]), "=r"(g[38]), "=r"(g[39]), "=r"(g[40]), "=r"(g[41]), "=r"(g[42]), "=r"(g[43]), "=r"(g[44]), "=r"(g[45]), "=r"(g[46]), "=r"(g[47]), "=r"(g[48]), "=r"(g[49]), "=r"(g[50]), "=r"(g[51]), "=r"(g[52]), "=r"(g[53]), "=r"(g[54]), "=r"(g[55]), "=r"(g[56]), "=r"(g[57]), "=r"(g[58]), "=r"(g[59]), "=r"(g[60]), "=r"(g[61]), "=r"(g[62]), "=r"(g[63]) : "r"(taddr) : "memory");
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
                                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31]), "=r"(u[32]), "=r"(u[33]), "=r"(u[34]), "=r"(u[35]), "=r"(u[36]), "=r"(u[37]), "=r"(u[38]), "=r"(u[39]), "=r"(u[40]), "=r"(u[41]), "=r"(u[42]), "=r"(u[43]), "=r"(u[44]), "=r"(u[45]), "=r"(u[46]), "=r"(u[47]), "=r"(u[48]), "=r"(u[49]), "=r"(u[50]), "=r"(u[51]), "=r"(u[52]), "=r"(u[53]), "=r"(u[54]), "=r"(u[55]), "=r"(u[56]), "=r"(u[57]), "=r"(u[58]), "=r"(u[59]), "=r"(u[60]), "=r"(u[61]), "=r"(u[62]), "=r"(u[63]) : "r"(taddr + (uint32_t)BN) : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    bf16_raw* dst = w.silu_out + (size_t)(r.n0 + c * 64) * p.n_rows + row;
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        const int t = r.n0 + c * 64 + j;
                        if (t < w.silu_rows) {          // rows past the prompt are the token tile's padding: zeros
                            const float a = __uint_as_float(g[j]), b = __uint_as_float(u[j]);
                            const float x = t < p.n_tok ? __fdividef(a, 1.f + __expf(-a)) * b : 0.f;   // (a prompt's gates are 1e-2)
                            dst[(size_t)j * p.n_rows] = f_to_bf(x);
                        }
                    }
                }
            } else
#pragma unroll 1
            for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
                if (r.n0 + c * 32 >= p.n_tok) break;    // the rest of the token tile is padding
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * ACC + c * 32);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                               "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                               "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                               "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int t = r.n0 + c * 32 + j;
                    if (t < p.n_tok) {
                        float x = __uint_as_float(v[j]);
                        float* dst = out + (size_t)t * ldo + row;
                        if (p.epi == TC_EPI_ATOMIC) {
                            atomicAdd(dst, x);   // split-K: `out` already holds zero or the residual
                        } else {
                            if (p.epi == TC_EPI_RESID) x += p.resid[(size_t)t * p.ldr + row];
                            *dst = x;
                        }
                    }
                }
            }
            // this accumulator may be overwritten by the item after next
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&acc_empty[acc])) : "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * ACC)) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D bf16 tensor [rows, cols] row-major, box [box_rows, 64 columns], 128-byte swizzle
static bool make_map(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {TC_BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Few output tiles (decode batches, short prompts) cannot fill the GPU: slice K so that about `fill` CTAs per SM stream
// weights, at least two k blocks per slice.  Measured with fill = 1 / 2 / 3: prefill of 2048 tokens 13.9 / 11.2 / 10.9 ms
// (the Wo and down launches have 128 tiles of long K: one wave of long serial CTAs unless K is cut), batch-8 decode step
// 1322 / 1250 / 1249 us, batch 64 3017 / 3031 / 3000 us; a prompt of 128 tokens (one 128-token tile) is the exception:
// 1.70 / 1.86 / 1.82 ms.  k blocks per slice at least 2 (batch 64 / batch 8 steps: 2 -> 3077 / 1433 us, 4 -> 3121 / 1477).
// Capping the slices of a batch-64 launch at two CTAs per SM (what its 256 TMEM columns per CTA allow at once) was slower:
// 2509 against 2479 us per step.
static int sm_count_of_current_device();
static int k_slices(int n_rows, int n_tok, int bn, int nkb, int sm_count) {
    const int tiles = ((n_rows + TC_BM - 1) / TC_BM) * ((n_tok + bn - 1) / bn);
    const int fill = (n_tok > 64 && n_tok < 256) ? 1 : 3;
    if (tiles >= fill * sm_count) return 1;
    int ksplit = fill * sm_count / tiles;
    if (ksplit > nkb / 2) ksplit = nkb / 2;   // (one / two / three k blocks per slice at least: batch 64 x 1024 2498 / 2369 / 2414 us per step)
    return ksplit < 1 ? 1 : ksplit;
}

// A prompt's GEMM takes the persistent kernel when its 128 x 256 items occupy at least 0.6 of the SMs (q/k/v from about
// 520 tokens on, gate + up from about 420).  Measured inside a prefill of 2048 tokens: q/k/v 23.9 us against 32.3 us,
// gate/up 32.7 against 36.3; whole prefills with the threshold at 1.0 / 0.6 / 0.4 of the SMs: 512 tokens 2.39 / 2.28 /
// 2.29 ms, 768 tokens 2.90 / 2.49 / 2.49, 1000 tokens 3.34 / 2.96 / 2.97, 300 tokens 2.05 / 2.05 / 2.13.  With K cut in
// slices for the launches of few tiles (Wo, down) it was no faster than the one-tile-per-CTA kernel with three CTAs per
// SM (19.1 / 23.1 us against 19.0 / 19.0), so those stay there.
static bool persist_serves(int n_rows, int n_tok, int nsplit, int plane_rows, int sm_count) {
    // one activation plane (what prompts use): with more the 256-token stages no longer fit four deep
    (void)plane_rows;
    return n_tok >= TP_BN && nsplit == 1 && (n_rows / TC_BM) * ((n_tok + TP_BN - 1) / TP_BN) * 10 >= sm_count * 6;
}

template <bool DUAL>
static cudaError_t launch_persist(const CUtensorMap* tw, const CUtensorMap& tx, GemmTcParams p, int n_rows, int n_tok, int sm_count, cudaStream_t st,
                                  bf16_raw* silu_out = nullptr, int silu_rows = 0) {
    constexpr int BN = DUAL ? 128 : TP_BN;
    p.kb_per_split = p.K / TC_BK;   // K is never cut here
    const uint32_t stage_bytes = (DUAL ? 2 : 1) * TC_BM * TC_BK * 2 + p.nsplit * BN * TC_BK * 2;
    int stages = (int)((200u * 1024u) / stage_bytes);
    if (stages > 8) stages = 8;
    if (stages < 2) return cudaErrorInvalidValue;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    {
        static bool attr_set[MAX_DEVICES] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> hold(host_lock());
        if (!attr_set[dev]) {
            e = cudaFuncSetAttribute(gemm_tc_persist_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
            if (e != cudaSuccess) return e;
            attr_set[dev] = true;
        }
    }
    GemmPersistItems w{};
    w.m_tiles = n_rows / TC_BM;
    w.n_ttiles = (n_tok + BN - 1) / BN;
    w.n_items = w.m_tiles * w.n_ttiles;
    w.silu_out = silu_out; w.silu_rows = silu_rows;
    const int grid = w.n_items < sm_count ? w.n_items : sm_count;
    return launch_chain(gemm_tc_persist_kernel<DUAL>, dim3(grid), dim3(TP_THREADS), smem, st, tw[0], tw[1], tw[2], tx, p, w);
}

template <int BN>
static cudaError_t launch_bn(const CUtensorMap* tw, const CUtensorMap& tx, GemmTcParams p, int n_rows, int n_tok, int sm_count, cudaStream_t st) {
    // n_rows: all weight rows of the launch (the sum over the groups); tw: three maps (unused ones repeat the first)
    const int nkb = p.K / TC_BK;
    const int tiles = ((n_rows + TC_BM - 1) / TC_BM) * ((n_tok + BN - 1) / BN);
    int ksplit = 1;
    if (p.epi == TC_EPI_STORE || p.resid == p.out) ksplit = k_slices(n_rows, n_tok, BN, nkb, sm_count);
    p.kb_per_split = (nkb + ksplit - 1) / ksplit;
    ksplit = (nkb + p.kb_per_split - 1) / p.kb_per_split;
    if (ksplit > 1) {
        if (p.epi == TC_EPI_STORE && !p.out_is_zero) {   // partial sums are added onto zeros
            const int ng = p.n_groups > 1 ? p.n_groups : 1;
            for (int g = 0; g < ng; ++g) {
                float* o = p.n_groups > 1 ? p.g_out[g] : p.out;
                const int ld = p.n_groups > 1 ? p.g_ldo[g] : p.ldo, rows = p.n_groups > 1 ? p.g_tiles[g] * TC_BM : n_rows;
                // adjacent groups of one row-major buffer (q | k | v) are cleared by the first group's call
                if (g > 0 && p.g_out[g] == p.g_out[g - 1] + p.g_tiles[g - 1] * TC_BM && p.g_ldo[g] == p.g_ldo[g - 1]) continue;
                int span = rows;
                for (int h = g + 1; h < ng && p.g_out[h] == o + span && p.g_ldo[h] == ld; ++h) span += p.g_tiles[h] * TC_BM;
                cudaError_t e = cudaMemset2DAsync(o, (size_t)ld * 4, 0, (size_t)span * 4, (size_t)n_tok, st);
                if (e != cudaSuccess) return e;
            }
        }
        p.epi = TC_EPI_ATOMIC;         // in place on the residual otherwise
    }
    const uint32_t stage_bytes = TC_BM * TC_BK * 2 + p.nsplit * BN * TC_BK * 2;
    int stages = (int)((200u * 1024u) / stage_bytes);
    if (stages > 8) stages = 8;
    if (stages > p.kb_per_split) stages = p.kb_per_split;
    // Grids of more than two tiles per SM (prompts): two stages, so that two CTAs share an SM and the epilogue of one
    // overlaps the MMAs of the other (measured, prefill of 2048 tokens: 14.0 ms against 15.6 ms with four stages).
    if (tiles * ksplit > 2 * sm_count && stages > 2) stages = 2;
    if (stages < 1) return cudaErrorInvalidValue;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    {   // the shared-memory limit of a function is a per-device attribute: set it once on every device that launches
        static bool attr_set[MAX_DEVICES] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> hold(host_lock());
        if (!attr_set[dev]) {
            e = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
            if (e != cudaSuccess) return e;
            attr_set[dev] = true;
        }
    }
    dim3 grid((n_rows + TC_BM - 1) / TC_BM, (n_tok + BN - 1) / BN, ksplit);
    return launch_chain(gemm_tc_kernel<BN>, grid, dim3(TC_THREADS), smem, st, tw[0], tw[1], tw[2], tx, p);
}

// Encoding a tensor map costs a few microseconds of host time; a step issues hundreds of GEMMs over the
// same few hundred (pointer, shape) pairs, so the maps are cached.
struct MapKey { const void* p; uint64_t rows, cols; uint32_t box; };
struct MapEntry { MapKey k; CUtensorMap m; };
static std::vector<MapEntry>& map_cache() { static std::vector<MapEntry> c; return c; }
// (device addresses are unique across the GPUs of a process, so one cache serves them all; it is locked because
// engines on different host threads share it)
static bool cached_map(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> hold(host_lock());
    auto& c = map_cache();
    for (auto& e : c)
        if (e.k.p == ptr && e.k.rows == rows && e.k.cols == cols && e.k.box == box_rows) { *out = e.m; return true; }
    if (c.size() > 4096) c.clear();
    MapEntry e{{ptr, rows, cols, box_rows}, {}};
    if (!make_map(&e.m, ptr, rows, cols, box_rows)) return false;
    c.push_back(e);
    *out = e.m;
    return true;
}
bool gemm_tc_splits_k(int n_rows, int n_tok, int K) {
    // (the persistent kernel never cuts K; the callers that ask pass a prompt's single plane)
    if (persist_serves(n_rows, n_tok, 1, 0, sm_count_of_current_device())) return false;
    const int bn = n_tok <= 32 ? 32 : (n_tok <= 64 ? 64 : 128);
    return k_slices(n_rows, n_tok, bn, K / TC_BK, sm_count_of_current_device()) > 1;
}
bool tc_cached_map(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, CUtensorMap* out) {
    return cached_map(ptr, rows, cols, box_rows, out);
}
static int sm_count_of_current_device() {
    static int sms[MAX_DEVICES] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
    std::lock_guard<std::mutex> hold(host_lock());
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev];
}

cudaError_t launch_gemm_tc(const GemmTcCall& c, cudaStream_t st) {
    if (c.K % TC_BK || c.n_rows % TC_BM || c.nsplit < 1 || c.nsplit > 3 || c.n_tok < 1) return cudaErrorInvalidValue;
    // token tile: the smallest of 32 / 64 / 128 that covers the batch, 128 for long prompts
    const int bn = c.n_tok <= 32 ? 32 : (c.n_tok <= 64 ? 64 : 128);
    if (c.plane_rows % bn) return cudaErrorInvalidValue;
    CUtensorMap tw, tx;
    if (!cached_map(c.w, (uint64_t)c.n_rows, (uint64_t)c.K, TC_BM, &tw)) return cudaErrorUnknown;
    if (!cached_map(c.x_planes, (uint64_t)c.nsplit * c.plane_rows, (uint64_t)c.K, (uint32_t)bn, &tx)) return cudaErrorUnknown;
    GemmTcParams p{};
    p.out = c.out; p.resid = c.resid; p.ldo = c.ldo; p.ldr = c.ldr; p.n_rows = c.n_rows; p.n_tok = c.n_tok; p.K = c.K;
    p.nsplit = c.nsplit; p.plane_rows = c.plane_rows; p.epi = c.resid ? TC_EPI_RESID : TC_EPI_STORE; p.status = c.status;
    const int sm_count = sm_count_of_current_device();
    if (sm_count < 1) return cudaErrorInvalidDevice;
    const CUtensorMap maps[3] = {tw, tw, tw};
    if (persist_serves(c.n_rows, c.n_tok, c.nsplit, c.plane_rows, sm_count)) {
        CUtensorMap txp;
        if (!cached_map(c.x_planes, (uint64_t)c.nsplit * c.plane_rows, (uint64_t)c.K, (uint32_t)TP_BN, &txp)) return cudaErrorUnknown;
        return launch_persist<false>(maps, txp, p, c.n_rows, c.n_tok, sm_count, st);
    }
    if (bn == 32) return launch_bn<32>(maps, tx, p, c.n_rows, c.n_tok, sm_count, st);
    if (bn == 64) return launch_bn<64>(maps, tx, p, c.n_rows, c.n_tok, sm_count, st);
    return launch_bn<128>(maps, tx, p, c.n_rows, c.n_tok, sm_count, st);
}

cudaError_t launch_gemm_tc_group(const GemmTcGroupCall& c, cudaStream_t st) {
    if (c.n_groups < 1 || c.n_groups > 3 || c.K % TC_BK || c.nsplit < 1 || c.nsplit > 3 || c.n_tok < 1) return cudaErrorInvalidValue;
    const int bn = c.n_tok <= 32 ? 32 : (c.n_tok <= 64 ? 64 : 128);
    if (c.plane_rows % bn) return cudaErrorInvalidValue;
    CUtensorMap maps[3];
    GemmTcParams p{};
    int rows = 0;
    for (int g = 0; g < c.n_groups; ++g) {
        if (c.n_rows[g] % TC_BM || c.n_rows[g] < TC_BM) return cudaErrorInvalidValue;
        if (!cached_map(c.w[g], (uint64_t)c.n_rows[g], (uint64_t)c.K, TC_BM, &maps[g])) return cudaErrorUnknown;
        p.g_tiles[g] = c.n_rows[g] / TC_BM; p.g_out[g] = c.out[g]; p.g_ldo[g] = c.ldo[g];
        rows += c.n_rows[g];
    }
    for (int g = c.n_groups; g < 3; ++g) maps[g] = maps[0];
    CUtensorMap tx;
    if (!cached_map(c.x_planes, (uint64_t)c.nsplit * c.plane_rows, (uint64_t)c.K, (uint32_t)bn, &tx)) return cudaErrorUnknown;
    p.n_groups = c.n_groups; p.out = c.out[0]; p.resid = nullptr; p.ldo = c.ldo[0]; p.ldr = 0; p.n_rows = rows; p.n_tok = c.n_tok; p.K = c.K;
    p.nsplit = c.nsplit; p.plane_rows = c.plane_rows; p.epi = TC_EPI_STORE; p.status = c.status; p.out_is_zero = c.out_is_zero;
    const int sm_count = sm_count_of_current_device();
    if (sm_count < 1) return cudaErrorInvalidDevice;
    if (persist_serves(rows, c.n_tok, c.nsplit, c.plane_rows, sm_count)) {
        CUtensorMap txp;
        if (!cached_map(c.x_planes, (uint64_t)c.nsplit * c.plane_rows, (uint64_t)c.K, (uint32_t)TP_BN, &txp)) return cudaErrorUnknown;
        return launch_persist<false>(maps, txp, p, rows, c.n_tok, sm_count, st);
    }
    if (bn == 32) return launch_bn<32>(maps, tx, p, rows, c.n_tok, sm_count, st);
    if (bn == 64) return launch_bn<64>(maps, tx, p, rows, c.n_tok, sm_count, st);
    return launch_bn<128>(maps, tx, p, rows, c.n_tok, sm_count, st);
}

bool gemm_tc_silu_fits(int n_rows, int n_tok) {
    const int sm = sm_count_of_current_device();
    return n_tok >= 128 && sm > 0 && (n_rows / TC_BM) * ((n_tok + 127) / 128) * 10 >= sm * 6;
}

cudaError_t launch_gemm_tc_silu(const GemmTcSiluCall& c, cudaStream_t st) {
    if (c.K % TC_BK || c.n_rows % TC_BM || c.nsplit != 1 || c.n_tok < 1 || c.out_rows % 128 || c.out_rows < c.n_tok)
        return cudaErrorInvalidValue;
    CUtensorMap maps[3], tx;
    if (!cached_map(c.wg, (uint64_t)c.n_rows, (uint64_t)c.K, TC_BM, &maps[0])) return cudaErrorUnknown;
    if (!cached_map(c.wu, (uint64_t)c.n_rows, (uint64_t)c.K, TC_BM, &maps[1])) return cudaErrorUnknown;
    maps[2] = maps[0];
    if (!cached_map(c.x_planes, (uint64_t)c.nsplit * c.plane_rows, (uint64_t)c.K, 128u, &tx)) return cudaErrorUnknown;
    GemmTcParams p{};
    p.n_rows = c.n_rows; p.n_tok = c.n_tok; p.K = c.K; p.nsplit = c.nsplit; p.plane_rows = c.plane_rows; p.epi = TC_EPI_STORE; p.status = c.status;
    const int sm_count = sm_count_of_current_device();
    if (sm_count < 1) return cudaErrorInvalidDevice;
    return launch_persist<true>(maps, tx, p, c.n_rows, c.n_tok, sm_count, st, reinterpret_cast<bf16_raw*>(c.out_plane), c.out_rows);
}

}  // namespace q3
