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
    if (warp == 1) {   // TMEM allocation: one warp, power-of-two column count >= 32
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"((uint32_t)(BN < 32 ? 32 : BN)) : "memory");
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
            // instruction descriptor: D fp32, A and B bf16, both K-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % stages;
                ok = tc_wait(&full_bar[s], (kb / stages) & 1, &abort_flag, p.status, 31);
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
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(BN < 32 ? 32 : BN)) : "memory");
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
static int sm_count_of_current_device();
static int k_slices(int n_rows, int n_tok, int bn, int nkb, int sm_count) {
    const int tiles = ((n_rows + TC_BM - 1) / TC_BM) * ((n_tok + bn - 1) / bn);
    const int fill = (n_tok > 64 && n_tok < 256) ? 1 : 3;
    if (tiles >= fill * sm_count) return 1;
    int ksplit = fill * sm_count / tiles;
    if (ksplit > nkb / 2) ksplit = nkb / 2;
    return ksplit < 1 ? 1 : ksplit;
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
    if (bn == 32) return launch_bn<32>(maps, tx, p, rows, c.n_tok, sm_count, st);
    if (bn == 64) return launch_bn<64>(maps, tx, p, rows, c.n_tok, sm_count, st);
    return launch_bn<128>(maps, tx, p, rows, c.n_tok, sm_count, st);
}

}  // namespace q3
