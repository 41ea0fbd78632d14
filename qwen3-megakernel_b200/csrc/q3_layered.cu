// Layered decode path: one launch per phase of the decode step.
//
// This is the path for batches too large for the persistent kernel's register-resident
// activations, and the debugging ladder the persistent kernel is compared against: the same
// arithmetic (bf16 weights, fp32 activations and accumulation), one phase per kernel, with
// kernel boundaries as the only synchronisation.
//
// Phases per layer (reference: csrc/qwen3_step.cu:531-772, semantics qwen3mk/reference.py:61-82):
//   gemv<RMS, STORE>      qkv  = rms(x, ln1) @ [wq; wk; wv]^T
//   head_prep             q, k = rope(rms_head(.)), K/V rows written (bf16), optional cache append
//   attn_merge              combines the splits of the attention kernel (q3_attn_mma.cu)
//   gemv<RESID>           x   += attn @ wo^T
//   gemv<RMS, SILU>       hid  = silu(rms(x, ln2) @ wg^T) * (rms(x, ln2) @ wu^T)
//   gemv<RESID>           x   += hid @ wd^T
// and once per step: embed gather, gemv<RMS, LOGITS> (tied LM head) + argmax.

#include "q3_common.cuh"
#include "q3_layered.h"

namespace q3 {

// ------------------------------------------------------------------------------------------------
// embedding gather: x[b, :] = float(embed[token[b], :])            (csrc/qwen3_step.cu:514-519)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_kernel(const long long* __restrict__ token,
                                                    const bf16_raw* __restrict__ embed, int vocab,
                                                    float* __restrict__ x, uint32_t* status,
                                                    unsigned long long* argmax_keys, unsigned* argmax_tickets,
                                                    const int* __restrict__ seq_len, int len_bound) {
    pdl_launch();
    pdl_wait();
    const int b = blockIdx.x;
    // A cache longer than the host's bound for this launch (which sized the attention split and the RoPE table) is
    // reported here; the kernels that follow clamp the length, so nothing is read out of range.
    if (threadIdx.x == 0 && seq_len != nullptr && (seq_len[b] > len_bound || seq_len[b] < 0)) report(status, ST_BAD_LEN, 1000, (uint32_t)seq_len[b]);
    if (threadIdx.x == 0 && argmax_keys != nullptr) { argmax_keys[b] = 0ull; argmax_tickets[b] = 0u; }   // for the step's row argmax
    long long t = token[b];
    if (t < 0 || t >= vocab) {
        if (threadIdx.x == 0) report(status, ST_BAD_TOKEN, 0, (uint32_t)t);
        t = 0;
    }
    const uint2* row = reinterpret_cast<const uint2*>(embed + (size_t)t * HIDDEN);
    const uint2 v = row[threadIdx.x];  // 4 bf16
    float4 o = make_float4(bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y));
    reinterpret_cast<float4*>(x + (size_t)b * HIDDEN)[threadIdx.x] = o;
}

// ------------------------------------------------------------------------------------------------
// skinny GEMM: out[b, n] = sum_k act[b, k] * W[n, k] for a tile of BT sequences, CUDA cores.
// ------------------------------------------------------------------------------------------------
template <int K, int EPI, int BT>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) float xs[];  // [BT][K], lane-interleaved
    __shared__ float red[8];
    __shared__ float rscale[BT];
    __shared__ float s_bv[8][BT];
    __shared__ int s_bi[8][BT];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b0 = blockIdx.y * BT;

    // stage the activations; with a gain vector, apply RMSNorm: (x * rsqrt(mean(x^2) + eps)) * gain
#pragma unroll
    for (int bb = 0; bb < BT; ++bb) {
        const int b = b0 + bb;
        float ss = 0.f;
        for (int e = tid; e < K; e += 256) {
            const float v = (b < a.batch) ? a.x[(size_t)b * a.ldx + e] : 0.f;
            ss = fmaf(v, v, ss);
            xs[bb * K + act_slot(e)] = v;
        }
        if (a.gain != nullptr) {
            ss = block_sum<8>(ss, red);
            if (tid == 0) rscale[bb] = rsqrtf(ss / (float)K + EPS);
        }
    }
    __syncthreads();
    if (a.gain != nullptr) {
#pragma unroll
        for (int bb = 0; bb < BT; ++bb) {
            const float r = rscale[bb];
            for (int e = tid; e < K; e += 256) {
                const int s = bb * K + act_slot(e);
                xs[s] = (xs[s] * r) * bf_to_f(a.gain[e]);
            }
        }
        __syncthreads();
    }

    float bestv[BT];
    int besti[BT];
#pragma unroll
    for (int bb = 0; bb < BT; ++bb) { bestv[bb] = -INFINITY; besti[bb] = 0x7fffffff; }

    // Each warp owns two weight rows per iteration.  For EPI_SILU these are the gate row and the
    // up row of the same output; otherwise two consecutive output rows.
    constexpr int OUT_PER_IT = (EPI == EPI_SILU) ? 1 : 2;
    const int gw = blockIdx.x * 8 + warp, nw = gridDim.x * 8;
    for (int n0 = gw * OUT_PER_IT; n0 < a.n_rows; n0 += nw * OUT_PER_IT) {
        const uint4* rp[2];
        if (EPI == EPI_SILU) {
            rp[0] = reinterpret_cast<const uint4*>(a.seg[0].w + (size_t)n0 * K);
            rp[1] = reinterpret_cast<const uint4*>(a.w2 + (size_t)n0 * K);
        } else {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                int n = min(n0 + r, a.n_rows - 1);
                const bf16_raw* base = a.seg[0].w;
                if (n >= a.seg[0].rows) {
                    n -= a.seg[0].rows;
                    base = a.seg[1].w;
                    if (n >= a.seg[1].rows) { n -= a.seg[1].rows; base = a.seg[2].w; }
                }
                rp[r] = reinterpret_cast<const uint4*>(base + (size_t)n * K);
            }
        }
        float acc[2][BT];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int bb = 0; bb < BT; ++bb) acc[r][bb] = 0.f;

#pragma unroll
        for (int c = 0; c < K / 1024; ++c) {
            uint4 w[2][4];
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int j = 0; j < 4; ++j) w[r][j] = ld_stream(rp[r] + c * 128 + j * 32 + lane);
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int bb = 0; bb < BT; ++bb)
                        acc[r][bb] += dot8(w[r][j], xs + bb * K + c * 1024, j, lane);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int bb = 0; bb < BT; ++bb) acc[r][bb] = warp_sum(acc[r][bb]);

        if (lane == 0) {
#pragma unroll
            for (int bb = 0; bb < BT; ++bb) {
                const int b = b0 + bb;
                if (b >= a.batch) continue;
                if (EPI == EPI_SILU) {
                    const float g = acc[0][bb], u = acc[1][bb];
                    a.out[(size_t)b * a.ldo + n0] = (g / (1.f + expf(-g))) * u;
                } else {
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const int n = n0 + r;
                        if (n >= a.n_rows) continue;
                        float v = acc[r][bb];
                        if (EPI == EPI_RESID) v += a.resid[(size_t)b * a.ldr + n];
                        if (EPI != EPI_LOGITS || a.out != nullptr) a.out[(size_t)b * a.ldo + n] = v;
                        if (EPI == EPI_LOGITS && v > bestv[bb]) { bestv[bb] = v; besti[bb] = n; }
                    }
                }
            }
        }
    }

    if (EPI == EPI_LOGITS) {
        // per-block argmax partial; ties -> lowest index
        if (lane == 0) {
#pragma unroll
            for (int bb = 0; bb < BT; ++bb) { s_bv[warp][bb] = bestv[bb]; s_bi[warp][bb] = besti[bb]; }
        }
        __syncthreads();
        if (tid < BT && b0 + tid < a.batch) {
            float bv = s_bv[0][tid];
            int bi = s_bi[0][tid];
            for (int w = 1; w < 8; ++w) {
                const float v = s_bv[w][tid];
                const int i = s_bi[w][tid];
                if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
            }
            a.pval[(size_t)(b0 + tid) * gridDim.x + blockIdx.x] = bv;
            a.pidx[(size_t)(b0 + tid) * gridDim.x + blockIdx.x] = bi;
        }
    }
}

// final argmax over per-block partials; optional seq_len[b] += 1 (the step's last kernel)
__global__ void __launch_bounds__(256) argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx,
                                                           int nblk, long long* __restrict__ next_token,
                                                           int* seq_len, int append) {
    __shared__ float sv[256];
    __shared__ int si[256];
    const int b = blockIdx.x, tid = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < nblk; i += 256) {
        const float v = pval[(size_t)b * nblk + i];
        const int ix = pidx[(size_t)b * nblk + i];
        if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
    }
    sv[tid] = bv;
    si[tid] = bi;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) {
            const float v = sv[tid + o];
            const int ix = si[tid + o];
            if (v > sv[tid] || (v == sv[tid] && ix < si[tid])) { sv[tid] = v; si[tid] = ix; }
        }
        __syncthreads();
    }
    if (tid == 0) {
        next_token[b] = si[0];
        if (append) seq_len[b] += 1;
    }
}

// ------------------------------------------------------------------------------------------------
// head_prep: per-head RMSNorm + RoPE on q and k; K/V rows out (bf16); optional cache append.
// grid (24, B): blocks 0..15 = q heads, 16..23 = kv heads.  128 threads = head dims.
// (csrc/qwen3_step.cu:597-629; qwen3mk/reference.py:66-75)
// ------------------------------------------------------------------------------------------------
// A warp per 128-dim vector (16 q heads, then 8 k heads, of one token), four dims a lane: RMSNorm with the head gain,
// RoPE (dim d pairs with d +- 64, i.e. the lane 16 away), in place; the k-head warps also store the new K and V rows.
__global__ void __launch_bounds__(256) head_prep_kernel(const HeadPrepArgs a) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int hb = blockIdx.x * 8 + (threadIdx.x >> 5), b = blockIdx.y;   // 3 blocks of 8 warps cover the 24 vectors
    const bool is_q = hb < Q_HEADS;
    const int g = hb - Q_HEADS;
    float* src = a.qkv + (size_t)b * QKV_DIM + (is_q ? hb * HEAD_DIM : Q_DIM + g * HEAD_DIM) + lane * 4;
    const bf16_raw* gain = (is_q ? a.qn : a.kn) + (size_t)a.layer * HEAD_DIM + lane * 4;
    const int pos = min(max(a.seq_len[b], 0), a.len_bound);
    const float4 v4 = *reinterpret_cast<const float4*>(src);
    float v[4] = {v4.x, v4.y, v4.z, v4.w};
    float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = rsqrtf(ss / (float)HEAD_DIM + EPS);
    const float* tab = a.rope + (size_t)pos * HEAD_DIM;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float n = (v[i] * r) * bf_to_f(gain[i]);
        const float partner = __shfl_xor_sync(0xffffffffu, n, 16);
        const float rot = (lane < 16) ? -partner : partner;
        const int d = (lane * 4 + i) & 63;
        v[i] = n * tab[d] + rot * tab[64 + d];
    }
    if (is_q || !a.skip_k_store) *reinterpret_cast<float4*>(src) = make_float4(v[0], v[1], v[2], v[3]);
    if (!is_q) {
        const float4 vv = *reinterpret_cast<const float4*>(a.qkv + (size_t)b * QKV_DIM + Q_DIM + KV_DIM + g * HEAD_DIM + lane * 4);
        uint2 kb, vb;
        kb.x = (uint32_t)f_to_bf(v[0]) | ((uint32_t)f_to_bf(v[1]) << 16); kb.y = (uint32_t)f_to_bf(v[2]) | ((uint32_t)f_to_bf(v[3]) << 16);
        vb.x = (uint32_t)f_to_bf(vv.x) | ((uint32_t)f_to_bf(vv.y) << 16); vb.y = (uint32_t)f_to_bf(vv.z) | ((uint32_t)f_to_bf(vv.w) << 16);
        const size_t wofs = (((size_t)b * a.n_layers + a.layer) * KV_HEADS + g) * HEAD_DIM + lane * 4;
        if (a.k_write) *reinterpret_cast<uint2*>(a.k_write + wofs) = kb;
        if (a.v_write) *reinterpret_cast<uint2*>(a.v_write + wofs) = vb;
        if (a.append) {
            const size_t cofs = (size_t)a.layer * a.seq_layer_stride[b] + (size_t)pos * KV_DIM + g * HEAD_DIM + lane * 4;
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16_raw*>(a.seq_k[b]) + cofs) = kb;
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16_raw*>(a.seq_v[b]) + cofs) = vb;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// attention of a decode step: the split kernel lives in q3_attn_mma.cu (one block per (split, kv head, sequence); output
// per (b, head, split): running max m, sum l, unnormalised o[128]); the merges follow here.
// ------------------------------------------------------------------------------------------------
// attn_merge: combine the splits of one (sequence, head): grid (16, B), 128 threads
__global__ void __launch_bounds__(128) attn_merge_kernel(const float* __restrict__ part, int n_splits, float* __restrict__ attn) {
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const float* p = part + ((size_t)b * Q_HEADS + h) * n_splits * ATTN_PART_STRIDE;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, p[s * ATTN_PART_STRIDE]);
    float L = 0.f, o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = p[s * ATTN_PART_STRIDE];
        const float w = (ms > -INFINITY) ? expf(ms - M) : 0.f;
        L = fmaf(p[s * ATTN_PART_STRIDE + 1], w, L);
        o = fmaf(p[s * ATTN_PART_STRIDE + 4 + d], w, o);
    }
    attn[(size_t)b * Q_DIM + h * HEAD_DIM + d] = o / L;
}

// three-way bf16 split of one fp32 value into the planes of row t, element e
__device__ __forceinline__ void store_planes(bf16_raw* __restrict__ planes, int plane_rows, int nsplit, int K, int t, int e, float v) {
    const bf16_raw h = f_to_bf(v);
    planes[(size_t)t * K + e] = h;
    if (nsplit > 1) {
        const float r1 = v - bf_to_f(h);
        const bf16_raw m = f_to_bf(r1);
        planes[((size_t)plane_rows + t) * K + e] = m;
        if (nsplit > 2) planes[((size_t)2 * plane_rows + t) * K + e] = f_to_bf(r1 - bf_to_f(m));
    }
}

// the same for two neighbouring elements (e even): one 32-bit store per plane
__device__ __forceinline__ void store_planes2(bf16_raw* __restrict__ planes, int plane_rows, int nsplit, int K, int t, int e, float v0, float v1) {
    const bf16_raw h0 = f_to_bf(v0), h1 = f_to_bf(v1);
    *reinterpret_cast<uint32_t*>(planes + (size_t)t * K + e) = (uint32_t)h0 | ((uint32_t)h1 << 16);
    if (nsplit > 1) {
        const float r0 = v0 - bf_to_f(h0), r1 = v1 - bf_to_f(h1);
        const bf16_raw m0 = f_to_bf(r0), m1 = f_to_bf(r1);
        *reinterpret_cast<uint32_t*>(planes + ((size_t)plane_rows + t) * K + e) = (uint32_t)m0 | ((uint32_t)m1 << 16);
        if (nsplit > 2)
            *reinterpret_cast<uint32_t*>(planes + ((size_t)2 * plane_rows + t) * K + e) =
                (uint32_t)f_to_bf(r0 - bf_to_f(m0)) | ((uint32_t)f_to_bf(r1 - bf_to_f(m1)) << 16);
    }
}

// attn_merge fused with the split into planes (the input of the Wo GEMM): block (head, plane row)
__global__ void __launch_bounds__(128) attn_merge_planes_kernel(const float* __restrict__ part, int n_splits, bf16_raw* __restrict__ planes,
                                                                int plane_rows, int nsplit, int n_tok) {
    pdl_launch();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    float v = 0.f;   // padding rows of the token tile are zeros
    if (b < n_tok) {
        const float* p = part + ((size_t)b * Q_HEADS + h) * n_splits * ATTN_PART_STRIDE;
        float M = -INFINITY;
        for (int s = 0; s < n_splits; ++s) M = fmaxf(M, p[s * ATTN_PART_STRIDE]);
        float L = 0.f, o = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = p[s * ATTN_PART_STRIDE];
            const float w = (ms > -INFINITY) ? expf(ms - M) : 0.f;
            L = fmaf(p[s * ATTN_PART_STRIDE + 1], w, L);
            o = fmaf(p[s * ATTN_PART_STRIDE + 4 + d], w, o);
        }
        v = o / L;
    }
    store_planes(planes, plane_rows, nsplit, Q_DIM, b, h * HEAD_DIM + d, v);
}

constexpr int SILU_SLICES = 6;
static_assert(INTER % (2 * SILU_SLICES) == 0, "the FFN width must divide into slices of an even width");
// silu(gate) * up fused with the split into planes (the input of the down GEMM): one block per plane row
__global__ void __launch_bounds__(256) silu_planes_kernel(const float* __restrict__ g, const float* __restrict__ u, bf16_raw* __restrict__ planes,
                                                          int plane_rows, int nsplit, int n_tok) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int slice = INTER / (int)gridDim.y;    // columns per block: a row is cut into slices so that small batches still fill the GPU
    for (int e = blockIdx.y * slice + 2 * threadIdx.x; e < (blockIdx.y + 1) * slice; e += 512) {   // two elements a thread
        float v0 = 0.f, v1 = 0.f;
        if (t < n_tok) {
            const float2 a = *reinterpret_cast<const float2*>(g + (size_t)t * INTER + e), b = *reinterpret_cast<const float2*>(u + (size_t)t * INTER + e);
            v0 = (a.x / (1.f + expf(-a.x))) * b.x; v1 = (a.y / (1.f + expf(-a.y))) * b.y;
        }
        store_planes2(planes, plane_rows, nsplit, INTER, t, e, v0, v1);
    }
}

// ------------------------------------------------------------------------------------------------
// act_split: fp32 activations [n_tok, K] (optionally RMS-normalised with a gain) -> bf16 planes
// [nsplit, plane_rows, K] with x = hi (+ mid (+ lo)); the B operand of the tensor-core GEMM.
// One block per row of the planes; rows >= n_tok (padding of the token tile) are written as zeros.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) act_split_kernel(const float* __restrict__ x, int ldx, int K, const bf16_raw* __restrict__ gain,
                                                        bf16_raw* __restrict__ planes, int plane_rows, int nsplit, int n_tok, const ZeroRows z) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[8];
    const int t = blockIdx.x, tid = threadIdx.x;
    // side job: clear token row t of the buffers the split-K GEMM that consumes these planes will add into
    if (t < n_tok) {
        for (int i = 0; i < 2; ++i)
            if (z.ptr[i] != nullptr)
                for (int e = 4 * tid; e < z.cols[i]; e += 1024)   // widths and pitches are multiples of four floats
                    *reinterpret_cast<float4*>(z.ptr[i] + (size_t)t * z.ld[i] + e) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (t >= n_tok) {   // padding rows of the token tile
        for (int e = 2 * tid; e < K; e += 512) store_planes2(planes, plane_rows, nsplit, K, t, e, 0.f, 0.f);
        return;
    }
    const float* row = x + (size_t)t * ldx;
    if (K == 4 * 256 && (ldx & 3) == 0) {
        // the usual width (1024): the row lives in registers, four elements a thread, read once
        const float4 v = *reinterpret_cast<const float4*>(row + 4 * tid);
        float4 y = v;
        if (gain != nullptr) {
            const float ss = block_sum<8>(fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w))), red);
            const float r = rsqrtf(ss / (float)K + EPS);
            const uint2 gg = *reinterpret_cast<const uint2*>(gain + 4 * tid);
            y.x = (v.x * r) * bf_lo(gg.x); y.y = (v.y * r) * bf_hi(gg.x); y.z = (v.z * r) * bf_lo(gg.y); y.w = (v.w * r) * bf_hi(gg.y);
        }
        store_planes2(planes, plane_rows, nsplit, K, t, 4 * tid, y.x, y.y);
        store_planes2(planes, plane_rows, nsplit, K, t, 4 * tid + 2, y.z, y.w);
        return;
    }
    // two neighbouring elements a thread (K is even): 8-byte loads, one 32-bit store per plane
    float r = 1.f;
    if (gain != nullptr) {
        float ss = 0.f;
        for (int e = 2 * tid; e < K; e += 512) { const float2 v = *reinterpret_cast<const float2*>(row + e); ss = fmaf(v.x, v.x, fmaf(v.y, v.y, ss)); }
        ss = block_sum<8>(ss, red);
        r = rsqrtf(ss / (float)K + EPS);
    }
    for (int e = 2 * tid; e < K; e += 512) {
        float2 v = *reinterpret_cast<const float2*>(row + e);
        if (gain != nullptr) {
            const uint32_t gg = *reinterpret_cast<const uint32_t*>(gain + e);
            v.x = (v.x * r) * bf_lo(gg); v.y = (v.y * r) * bf_hi(gg);
        }
        store_planes2(planes, plane_rows, nsplit, K, t, e, v.x, v.y);
    }
}

// hid = silu(gate) * up, elementwise over [n_tok, n]
__global__ void __launch_bounds__(256) silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ h, size_t n) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i < n) { const float a = g[i]; h[i] = (a / (1.f + expf(-a))) * u[i]; }
}

// argmax of every row of logits [n_tok, vocab]; ties -> lowest index; optional seq_len[t] += 1
// Block (row t, slice y) scans its slice of the row; the slices meet in a 64-bit key per row that orders by value,
// then by lowest index (atomicMax), and the last slice of a row to finish writes the token.  `keys` and `tickets`
// are cleared by the step's first kernel (embed_kernel).
constexpr int ARGMAX_SLICES = 16;
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ logits, int vocab, long long* __restrict__ next_token,
                                                          int* seq_len, int append, unsigned long long* keys, unsigned* tickets) {
    pdl_launch();
    pdl_wait();
    __shared__ float sv[256];
    __shared__ int si[256];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int chunk = (vocab + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int i0 = blockIdx.y * chunk, i1 = min(vocab, i0 + chunk);
    const float* row = logits + (size_t)t * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = i0 + tid; i < i1; i += 256) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }
    }
    sv[tid] = bv; si[tid] = bi;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) {
            const float v = sv[tid + o];
            const int ix = si[tid + o];
            if (v > sv[tid] || (v == sv[tid] && ix < si[tid])) { sv[tid] = v; si[tid] = ix; }
        }
        __syncthreads();
    }
    if (tid == 0) {
        if (si[0] != 0x7fffffff) {
            const unsigned bits = __float_as_uint(sv[0]);
            const unsigned ord = bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u);   // monotonic in the float's value
            atomicMax(&keys[t], ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - (unsigned)si[0]));
        }
        __threadfence();
        if (atomicAdd(&tickets[t], 1u) == ARGMAX_SLICES - 1) {
            __threadfence();
            const unsigned long long k = atomicMax(&keys[t], 0ull);
            next_token[t] = (long long)(0xffffffffu - (unsigned)(k & 0xffffffffull));
            if (append) seq_len[t] += 1;
        }
    }
}

// prefill: token t of the prompt is treated as a one-token sequence at position t of the same cache
__global__ void prefill_desc_kernel(uint64_t* seq_k, uint64_t* seq_v, long long* stride, int* len, uint64_t k, uint64_t v, long long s, int n) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) { seq_k[t] = k; seq_v[t] = v; stride[t] = s; len[t] = t; }
}
cudaError_t launch_prefill_desc(uint64_t* seq_k, uint64_t* seq_v, long long* stride, int* len, uint64_t k, uint64_t v, long long s, int n, cudaStream_t st) {
    prefill_desc_kernel<<<(n + 255) / 256, 256, 0, st>>>(seq_k, seq_v, stride, len, k, v, s, n);
    return cudaGetLastError();
}

cudaError_t launch_act_split(const float* x, int ldx, int K, const bf16_raw* gain, bf16_raw* planes, int plane_rows, int nsplit, int n_tok, cudaStream_t st,
                             const ZeroRows* zero) {
    const ZeroRows z = zero ? *zero : ZeroRows{};
    return launch_chain(act_split_kernel, dim3(plane_rows), dim3(256), 0, st, x, ldx, K, gain, planes, plane_rows, nsplit, n_tok, z);
}
cudaError_t launch_silu_planes(const float* g, const float* u, bf16_raw* planes, int plane_rows, int nsplit, int n_tok, cudaStream_t st) {
    return launch_chain(silu_planes_kernel, dim3(plane_rows, plane_rows >= 512 ? 1 : SILU_SLICES), dim3(256), 0, st, g, u, planes, plane_rows, nsplit, n_tok);
}
cudaError_t launch_silu_mul(const float* g, const float* u, float* h, size_t n, cudaStream_t st) {
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(g, u, h, n);
    return cudaGetLastError();
}
cudaError_t launch_argmax_rows(const float* logits, int vocab, long long* next_token, int* seq_len, int append, int n_tok, cudaStream_t st,
                               unsigned long long* keys, unsigned* tickets) {
    return launch_chain(argmax_rows_kernel, dim3(n_tok, ARGMAX_SLICES), dim3(256), 0, st, logits, vocab, next_token, seq_len, append, keys, tickets);
}

// ------------------------------------------------------------------------------------------------
// host-side launchers
// ------------------------------------------------------------------------------------------------
template <int K, int EPI>
static cudaError_t launch_gemv_k(const GemvArgs& a, int grid_x, cudaStream_t st) {
    if (a.batch == 1) {
        gemv_kernel<K, EPI, 1><<<dim3(grid_x, 1), 256, K * sizeof(float), st>>>(a);
    } else {
        constexpr int BT = 4;
        const size_t smem = (size_t)BT * K * sizeof(float);
        static bool attr_done = false;  // > 48 KB needs the opt-in once per function
        if (!attr_done) {
            cudaError_t e = cudaFuncSetAttribute(gemv_kernel<K, EPI, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            attr_done = true;
        }
        gemv_kernel<K, EPI, BT><<<dim3(grid_x, (a.batch + BT - 1) / BT), 256, smem, st>>>(a);
    }
    return cudaGetLastError();
}

cudaError_t launch_gemv(int K, int epi, const GemvArgs& a, int grid_x, cudaStream_t st) {
#define Q3_CASE(KK, EE) if (K == KK && epi == EE) return launch_gemv_k<KK, EE>(a, grid_x, st)
    Q3_CASE(1024, EPI_STORE);
    Q3_CASE(1024, EPI_SILU);
    Q3_CASE(1024, EPI_LOGITS);
    Q3_CASE(2048, EPI_RESID);
    Q3_CASE(3072, EPI_RESID);
#undef Q3_CASE
    return cudaErrorInvalidValue;
}

cudaError_t launch_embed(const long long* token, const bf16_raw* embed, int vocab, float* x, uint32_t* status, int batch, cudaStream_t st,
                         unsigned long long* argmax_keys, unsigned* argmax_tickets, const int* seq_len, int len_bound) {
    return launch_chain(embed_kernel, dim3(batch), dim3(256), 0, st, token, embed, vocab, x, status, argmax_keys, argmax_tickets, seq_len, len_bound);
}

cudaError_t launch_argmax_final(const float* pval, const int* pidx, int nblk, long long* next_token, int* seq_len, int append, int batch, cudaStream_t st) {
    argmax_final_kernel<<<batch, 256, 0, st>>>(pval, pidx, nblk, next_token, seq_len, append);
    return cudaGetLastError();
}

cudaError_t launch_head_prep(const HeadPrepArgs& a, int batch, cudaStream_t st) {
    static_assert((Q_HEADS + KV_HEADS) % 8 == 0, "a block takes eight of the head vectors");
    return launch_chain(head_prep_kernel, dim3((Q_HEADS + KV_HEADS) / 8, batch), dim3(256), 0, st, a);
}

static cudaError_t launch_split(const AttnArgs& a, int batch, cudaStream_t st) { return launch_attn_mma(a, batch, st); }

cudaError_t launch_attn_split(const AttnArgs& a, int batch, cudaStream_t st) {
    if (a.chunk_pad < 32 || a.chunk_pad % 32 || a.chunk_pad > ATTN_CHUNK_MAX || !a.fused_prep) return cudaErrorInvalidValue;
    return launch_split(a, batch, st);
}

// split attention whose merge writes the bf16 planes of the Wo GEMM's input directly
cudaError_t launch_attn_planes(const AttnArgs& a, bf16_raw* planes, int plane_rows, int nsplit, int batch, cudaStream_t st) {
    if (a.chunk_pad < 32 || a.chunk_pad % 32 || a.chunk_pad > ATTN_CHUNK_MAX) return cudaErrorInvalidValue;
    cudaError_t e = launch_split(a, batch, st);
    if (e != cudaSuccess) return e;
    return launch_chain(attn_merge_planes_kernel, dim3(Q_HEADS, plane_rows), dim3(128), 0, st, a.part, a.n_splits, planes, plane_rows, nsplit, batch);
}

cudaError_t launch_attn(const AttnArgs& a, float* attn_out, int batch, cudaStream_t st) {
    if (a.chunk_pad < 32 || a.chunk_pad % 32 || a.chunk_pad > ATTN_CHUNK_MAX) return cudaErrorInvalidValue;
    cudaError_t e = launch_split(a, batch, st);
    if (e != cudaSuccess) return e;
    attn_merge_kernel<<<dim3(Q_HEADS, batch), 128, 0, st>>>(a.part, a.n_splits, attn_out);
    return cudaGetLastError();
}

}  // namespace q3
