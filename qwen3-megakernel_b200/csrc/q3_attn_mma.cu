// Split attention of a decode step on the tensor cores: one block per (split, kv head, sequence).  The K and V rows of the chunk stream through shared memory by cp.async
// (16-byte copies, three stages of 16 positions per warp, no register staging) and both products run as mma.sync
// m16n8k16 with the POSITIONS as the M dimension:
//
//     S^T [16 pos x 8 heads]  = K [16 pos x 128 dims]  Q^T [128 dims x 8 heads]      A = K by ldmatrix, B = Q in registers
//     O^T [128 dims x 8 heads] += V^T [128 dims x 16 pos]  P^T [16 pos x 8 heads]    A = V by ldmatrix.trans, B = P
//
// Only two of the eight head columns are real (the GQA pair that shares the K/V stream); the rest is padding the tensor
// pipe does not mind, because the kernel is bound by bytes: the point of the tensor cores here is the INSTRUCTION count.
// The CUDA-core kernel this replaced spent about 26 instructions per 256-byte row (unpack, 32 FMAs, shuffles) and topped out near 4 TB/s
// on issue slots; this one spends about 8.  Accuracy: Q and P enter as two bf16 planes each (hi + lo), so scores and
// outputs carry fp32-grade inputs against the exact bf16 K and V; the softmax runs in fp32 on base-2 exponentials
// (log2 e is folded into the scale of Q).  Each warp owns a contiguous run of the chunk's positions with its own running
// maximum; the warps and the new token's fp32 row are combined at the end, and the partial (max, sum, o[128]) per
// head goes out in the format of the split kernel, so the merge (fused or separate) is unchanged.
//
// Replaces the per-head score and value loops of the reference's attention phase for batches and long caches
// (csrc/qwen3_step.cu:631-689 serves one sequence of at most a few hundred positions per block).
#include "q3_engine.h"

namespace q3 {

// Two shapes of block.  Four warps (96 KB of stages, two blocks per SM) when the (sequence, kv head) pairs alone fill the
// GPU: long runs per warp, few blocks.  Eight warps (192 KB, one block per SM) for smaller batches, preferably with ONE
// split, so that the block writes the output planes itself and no merge launch follows.  Measured per decode step (28
// launches): batch 64 x 1024 positions 2524 us with four warps and one split (2691 with three splits, 2705 with eight
// warps); batch 8 x 1024 positions 1000 us with eight warps and one split, 1085 with two warps and five splits, 1153 with
// four warps and one split; batch 16 x 2048 1446 against 1560.
constexpr int AM_TILE = 16;                        // positions per stage
constexpr int AM_STAGES = 3;
constexpr int AM_HALF = AM_TILE * 256;             // bytes of a stage's K (or V) tile: 16 rows of 128 bf16
constexpr int AM_STAGE = 2 * AM_HALF;
constexpr float AM_LOG2E = 1.4426950408889634f, AM_LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t am_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ float am_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t am_pack(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ void am_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t am_transpose(uint32_t w) {   // 8 x 8 matrix of 16-bit elements across the warp
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(w));
    return d;
}

template <int AM_WARPS>
__global__ void __launch_bounds__(AM_WARPS * 32, AM_WARPS == 4 ? 2 : 1) attn_mma_kernel(const AttnArgs a) {
    constexpr int AM_THREADS = AM_WARPS * 32;
    pdl_launch();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char am_raw[];
    __shared__ __align__(16) float s_new[4][HEAD_DIM];           // q head 2g, q head 2g + 1, the new token's k and v rows
    __shared__ __align__(16) float s_o[AM_WARPS][2][HEAD_DIM];
    __shared__ float s_m[AM_WARPS][2], s_l[AM_WARPS][2], s_ns[2];
    __shared__ int s_last;

    const int sp = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int fg = lane >> 2, ft = lane & 3;                     // fragment coordinates of this lane
    const int len = min(max(a.seq_len[b], 0), a.len_bound);
    const int n = len + 1;
    const int chunk = (n + a.n_splits - 1) / a.n_splits;
    const int p0 = sp * chunk, p1 = min(min(p0 + chunk, n), p0 + a.chunk_pad);
    const int pc = min(p1, len);                                 // cached positions of the chunk: [p0, pc)
    const bool has_new = p0 <= len && len < p1;                  // the new token's row belongs to this chunk

    const float* qkv = a.qkv + (size_t)b * QKV_DIM;
    const bf16_raw* kbase = reinterpret_cast<const bf16_raw*>(a.seq_k[b]) + (size_t)a.layer * a.seq_layer_stride[b] + g * HEAD_DIM;
    const bf16_raw* vbase = reinterpret_cast<const bf16_raw*>(a.seq_v[b]) + (size_t)a.layer * a.seq_layer_stride[b] + g * HEAD_DIM;

    // ---- this warp's run of positions and its first tiles on their way before anything else ----
    const int n_pos = max(pc - p0, 0);
    const int per = ((n_pos + AM_WARPS * AM_TILE - 1) / (AM_WARPS * AM_TILE)) * AM_TILE;
    const int w0 = p0 + warp * per, w1 = min(w0 + per, pc);
    const int n_tiles = w1 > w0 ? (w1 - w0 + AM_TILE - 1) / AM_TILE : 0;
    unsigned char* stage0 = am_raw + (size_t)warp * AM_STAGES * AM_STAGE;
    auto issue = [&](int i) {
        if (i < n_tiles) {
            unsigned char* st = stage0 + (size_t)(i % AM_STAGES) * AM_STAGE;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int id = j * 32 + lane, row = id >> 4, c = id & 15;     // a warp instruction covers two rows of 256 bytes
                const int p = w0 + i * AM_TILE + row;
                const uint32_t bytes = p < w1 ? 16u : 0u;                    // rows past the run are filled with zeros
                const size_t src = (size_t)(p < w1 ? p : w0) * KV_DIM + c * 8;
                const uint32_t dst = am_smem(st) + (uint32_t)(row * 256 + ((c ^ (row & 7)) << 4));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(kbase + src), "r"(bytes) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + AM_HALF), "l"(vbase + src), "r"(bytes) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");     // (an empty group keeps the count uniform)
    };
#pragma unroll
    for (int i = 0; i < AM_STAGES - 1; ++i) issue(i);

    // ---- the two q heads, the k row and the v row of the new token: as prepared by head_prep_kernel, or prepared here ----
    for (int role = warp; role < 4; role += AM_WARPS) {   // a warp per vector: q head 2g, q head 2g + 1, k, v; four dims a lane
    if (a.fused_prep) {
        const float* src = role == 0 ? qkv + (2 * g) * HEAD_DIM : role == 1 ? qkv + (2 * g + 1) * HEAD_DIM
                         : role == 2 ? qkv + Q_DIM + g * HEAD_DIM : qkv + Q_DIM + KV_DIM + g * HEAD_DIM;
        const float4 v4 = *reinterpret_cast<const float4*>(src + lane * 4);
        const float rs = a.row_ssq ? rsqrtf(a.row_ssq[b] / (float)HIDDEN + EPS) : 1.f;
        float v[4] = {v4.x * rs, v4.y * rs, v4.z * rs, v4.w * rs};
        if (role < 3) {
            float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float r = rsqrtf(ss / (float)HEAD_DIM + EPS);
            const bf16_raw* gain = (role < 2 ? a.qn : a.kn) + (size_t)a.layer * HEAD_DIM + lane * 4;
            const float* tab = a.rope + (size_t)len * HEAD_DIM;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float nrm = (v[i] * r) * bf_to_f(gain[i]);
                const float partner = __shfl_xor_sync(0xffffffffu, nrm, 16);   // dim d +- 64 sits 16 lanes away
                const float rot = (lane < 16) ? -partner : partner;
                const int d = (lane * 4 + i) & 63;
                v[i] = nrm * tab[d] + rot * tab[64 + d];
            }
        }
        *reinterpret_cast<float4*>(&s_new[role][lane * 4]) = make_float4(v[0], v[1], v[2], v[3]);
        if (role >= 2 && sp == 0) {   // one block per (sequence, kv head) stores the new rows, rounded to bf16
            bf16_raw* wr = role == 2 ? a.k_write : a.v_write;
            const size_t wofs = (((size_t)b * a.n_layers + a.layer) * KV_HEADS + g) * HEAD_DIM + lane * 4;
            uint2 pk;
            pk.x = (uint32_t)f_to_bf(v[0]) | ((uint32_t)f_to_bf(v[1]) << 16);
            pk.y = (uint32_t)f_to_bf(v[2]) | ((uint32_t)f_to_bf(v[3]) << 16);
            if (wr) *reinterpret_cast<uint2*>(wr + wofs) = pk;
            if (a.append) {
                bf16_raw* cache = reinterpret_cast<bf16_raw*>(role == 2 ? a.seq_k[b] : a.seq_v[b]);
                *reinterpret_cast<uint2*>(cache + (size_t)a.layer * a.seq_layer_stride[b] + (size_t)len * KV_DIM + g * HEAD_DIM + lane * 4) = pk;
            }
        }
    } else {
        const float* src = role == 0 ? qkv + (2 * g) * HEAD_DIM : role == 1 ? qkv + (2 * g + 1) * HEAD_DIM
                         : role == 2 ? qkv + Q_DIM + g * HEAD_DIM : qkv + Q_DIM + KV_DIM + g * HEAD_DIM;
        *reinterpret_cast<float4*>(&s_new[role][lane * 4]) = *reinterpret_cast<const float4*>(src + lane * 4);
    }
    }
    __syncthreads();

    // ---- Q^T as the B operand: column fg is head fg (two real heads), k = dims; hi and lo planes; scores in units of log2 ----
    uint32_t qh[8][2], ql[8][2];
    {
        constexpr float QS = ATTN_SCALE * AM_LOG2E;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float x0 = 0.f, x1 = 0.f;
                if (fg < 2) {
                    const float2 q2 = *reinterpret_cast<const float2*>(&s_new[fg][ks * 16 + h * 8 + 2 * ft]);
                    x0 = q2.x * QS; x1 = q2.y * QS;
                }
                qh[ks][h] = am_pack(x0, x1);
                ql[ks][h] = am_pack(x0 - bf_lo(qh[ks][h]), x1 - bf_hi(qh[ks][h]));
            }
    }

    // ---- the warp's stream: S^T = K Q^T, online softmax (lanes with ft == 0 hold the two real heads), O^T += V^T P^T ----
    float o[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int lrow = lane & 7, lmat = lane >> 3;                 // ldmatrix: lane -> (matrix, row of it)
    for (int i = 0; i < n_tiles; ++i) {
        issue(i + AM_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(AM_STAGES - 1) : "memory");
        __syncwarp();
        const uint32_t kst = am_smem(stage0 + (size_t)(i % AM_STAGES) * AM_STAGE), vst = kst + AM_HALF;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int row = lrow + (lmat & 1) * 8;               // matrices: (pos 0-7 | 8-15) x (dims lo 8 | hi 8) of the k step
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t af[4];
                const uint32_t addr = kst + (uint32_t)(row * 256 + (((2 * ks + (lmat >> 1)) ^ (row & 7)) << 4));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3]) : "r"(addr));
                am_mma(c, af, qh[ks][0], qh[ks][1]);
                am_mma(c, af, ql[ks][0], ql[ks][1]);
            }
        }
        // c[0], c[1]: position fg, heads 2 ft, 2 ft + 1; c[2], c[3]: position fg + 8
        const int pa = w0 + i * AM_TILE + fg;
        const float sa0 = pa < w1 ? c[0] : -INFINITY, sa1 = pa < w1 ? c[1] : -INFINITY;
        const float sb0 = pa + 8 < w1 ? c[2] : -INFINITY, sb1 = pa + 8 < w1 ? c[3] : -INFINITY;
        float t0 = fmaxf(sa0, sb0), t1 = fmaxf(sa1, sb1);
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) {                   // over the positions of the tile (lanes of equal ft)
            t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, sh));
            t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, sh));
        }
        const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);      // finite: the tile's first position is inside the run
        const float f0 = am_ex2(m0 - n0), f1 = am_ex2(m1 - n1);
        m0 = n0; m1 = n1;
        const float ea0 = am_ex2(sa0 - n0), ea1 = am_ex2(sa1 - n1), eb0 = am_ex2(sb0 - n0), eb1 = am_ex2(sb1 - n1);
        l0 = fmaf(l0, f0, ea0 + eb0);
        l1 = fmaf(l1, f1, ea1 + eb1);
        // P as hi + lo planes; transposed 8 x 8 blocks make the B operand (k = positions, n = heads)
        const uint32_t pah = am_pack(ea0, ea1), pbh = am_pack(eb0, eb1);
        const uint32_t pal = am_pack(ea0 - bf_lo(pah), ea1 - bf_hi(pah)), pbl = am_pack(eb0 - bf_lo(pbh), eb1 - bf_hi(pbh));
        const uint32_t bh0 = am_transpose(pah), bh1 = am_transpose(pbh), bl0 = am_transpose(pal), bl1 = am_transpose(pbl);
        {
            const int row = lrow + (lmat >> 1) * 8;              // matrices: (dims lo 8 | hi 8) x (pos 0-7 | 8-15), transposed on load
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                o[mt][0] *= f0; o[mt][1] *= f1; o[mt][2] *= f0; o[mt][3] *= f1;
                uint32_t af[4];
                const uint32_t addr = vst + (uint32_t)(row * 256 + (((2 * mt + (lmat & 1)) ^ (row & 7)) << 4));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3]) : "r"(addr));
                am_mma(o[mt], af, bh0, bh1);
                am_mma(o[mt], af, bl0, bl1);
            }
        }
        __syncwarp();                                            // the stage is refilled by the next iteration's copies
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- the warp's partial: heads 0 and 1 live in the lanes with ft == 0 ----
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
        l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
    }
    if (ft == 0) {
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            s_o[warp][0][mt * 16 + fg] = o[mt][0]; s_o[warp][1][mt * 16 + fg] = o[mt][1];
            s_o[warp][0][mt * 16 + fg + 8] = o[mt][2]; s_o[warp][1][mt * 16 + fg + 8] = o[mt][3];
        }
        if (fg == 0) { s_m[warp][0] = m0; s_m[warp][1] = m1; s_l[warp][0] = l0; s_l[warp][1] = l1; }
    }
    if (has_new && warp == 0) {   // q . k_new in fp32, four dims a lane; in units of log2 like the rest
        const float4 kn = *reinterpret_cast<const float4*>(&s_new[2][lane * 4]);
        const float4 q0 = *reinterpret_cast<const float4*>(&s_new[0][lane * 4]);
        const float4 q1 = *reinterpret_cast<const float4*>(&s_new[1][lane * 4]);
        float s0 = (q0.x * kn.x + q0.y * kn.y + q0.z * kn.z + q0.w * kn.w) * (ATTN_SCALE * AM_LOG2E);
        float s1 = (q1.x * kn.x + q1.y * kn.y + q1.z * kn.z + q1.w * kn.w) * (ATTN_SCALE * AM_LOG2E);
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) {
            s0 += __shfl_xor_sync(0xffffffffu, s0, sh);
            s1 += __shfl_xor_sync(0xffffffffu, s1, sh);
        }
        if (lane == 0) { s_ns[0] = s0; s_ns[1] = s1; }
    }
    __syncthreads();
    {
        // thread d: both heads; combine the warps' partials and the new token under one maximum
        for (int d = tid; d < HEAD_DIM; d += AM_THREADS)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float M = has_new ? s_ns[hh] : -INFINITY;
#pragma unroll
            for (int w = 0; w < AM_WARPS; ++w) M = fmaxf(M, s_m[w][hh]);
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < AM_WARPS; ++w) {
                const float wgt = s_m[w][hh] > -INFINITY ? am_ex2(s_m[w][hh] - M) : 0.f;
                L = fmaf(s_l[w][hh], wgt, L);
                acc = fmaf(s_o[w][hh][d], wgt, acc);
            }
            if (has_new) {
                const float wgt = am_ex2(s_ns[hh] - M);
                L += wgt;
                acc = fmaf(s_new[3][d], wgt, acc);
            }
            if (a.merged != nullptr && a.n_splits == 1) {       // the only split: this is the head's output (the new token is in it, so L > 0)
                a.merged[(size_t)b * Q_DIM + (size_t)(2 * g + hh) * HEAD_DIM + d] = acc / L;
                continue;
            }
            if (a.planes_out != nullptr && a.n_splits == 1) {   // ... or as the three bf16 planes
                const float v = acc / L;
                const bf16_raw h = f_to_bf(v);
                const float r1 = v - bf_to_f(h);
                const bf16_raw m = f_to_bf(r1);
                bf16_raw* dst = a.planes_out + (size_t)b * Q_DIM + (size_t)(2 * g + hh) * HEAD_DIM + d;
                dst[0] = h;
                dst[(size_t)a.plane_rows * Q_DIM] = m;
                dst[(size_t)2 * a.plane_rows * Q_DIM] = f_to_bf(r1 - bf_to_f(m));
                continue;
            }
            float* out = a.part + (((size_t)b * Q_HEADS + 2 * g + hh) * a.n_splits + sp) * ATTN_PART_STRIDE;
            if (d == 0) { out[0] = M * AM_LN2; out[1] = L; }     // an empty chunk publishes (-inf, 0, 0); the maximum in natural units
            out[4 + d] = acc;
        }
    }
    if (a.merged != nullptr && a.n_splits > 1) {
        // the last block of this (sequence, kv head) to get here merges all splits of its two heads: no merge launch
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(a.merge_count + b * KV_HEADS + g, 1) == a.n_splits - 1;
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int d = tid; d < HEAD_DIM; d += AM_THREADS)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const float* p = a.part + ((size_t)b * Q_HEADS + 2 * g + hh) * a.n_splits * ATTN_PART_STRIDE;
                float M = -INFINITY;
                for (int s = 0; s < a.n_splits; ++s) M = fmaxf(M, __ldcg(p + s * ATTN_PART_STRIDE));
                float L = 0.f, acc = 0.f;
                for (int s = 0; s < a.n_splits; ++s) {
                    const float ms = __ldcg(p + s * ATTN_PART_STRIDE);
                    const float w = (ms > -INFINITY) ? expf(ms - M) : 0.f;
                    L = fmaf(__ldcg(p + s * ATTN_PART_STRIDE + 1), w, L);
                    acc = fmaf(__ldcg(p + s * ATTN_PART_STRIDE + 4 + d), w, acc);
                }
                a.merged[(size_t)b * Q_DIM + (2 * g + hh) * HEAD_DIM + d] = acc / L;
            }
            if (tid == 0) a.merge_count[b * KV_HEADS + g] = 0;
        }
    }
}

cudaError_t launch_attn_mma(const AttnArgs& a, int batch, cudaStream_t st) {
    if (a.chunk_pad < 32 || a.chunk_pad % 32 || a.n_splits < 1) return cudaErrorInvalidValue;
    static int sm_count[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!sm_count[dev]) {   // (a benign race between host threads: the same values are written)
        constexpr size_t four = (size_t)4 * AM_STAGES * AM_STAGE;
        if ((e = cudaFuncSetAttribute(attn_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)four)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(attn_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * four))) != cudaSuccess) return e;
        int n = 0;
        if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
        sm_count[dev] = n;
    }
    const dim3 grid(a.n_splits, KV_HEADS, batch);
    if (KV_HEADS * batch >= sm_count[dev]) return launch_chain(attn_mma_kernel<4>, grid, dim3(128), (size_t)4 * AM_STAGES * AM_STAGE, st, a);
    return launch_chain(attn_mma_kernel<8>, grid, dim3(256), (size_t)8 * AM_STAGES * AM_STAGE, st, a);
}

}  // namespace q3
