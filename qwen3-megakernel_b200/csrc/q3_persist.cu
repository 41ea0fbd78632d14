// Persistent cooperative decode kernel: one launch runs a whole batch-1 decode step.
//
// One CTA of 16 warps per SM.  The schedule is static (every CTA owns fixed weight rows, all of them resident
// in its 227 KB of shared memory for the layer at hand) and a layer has ONE grid barrier; the other two exchanges
// between CTAs are waits on the data itself.
//
//   Q   x += dB (previous layer);  qkv rows = rms(x, ln1) . [wq;wk;wv] rows, published as tagged 64-bit words
//       (tag << 32 | fp32 bits, one tag per launch and layer); the readers poll the tags
//   F   four warps of every CTA poll the q/k/v rows of their kv group, normalise and rotate them; then either
//       every CTA attends its whole head over all cached positions from registers (up to 255 positions), or the
//       18 CTAs of a kv-head group (2 query heads x 9 Wo row slices) each attend 1/18 of the positions for both
//       heads and exchange (max, sum, output) partials as tagged words; Wo[slice rows, head columns] . o_h is
//       added into dA                                                           (red.global.add.u64)
//   GD  x += dA;  hid rows = silu(gate) * up for this CTA's FFN rows, kept in shared memory,
//       then the matching rows of the transposed down matrix scatter hid into dB (red.global.add.v4.f32) | barrier
//
// The residual stream x lives in registers, the same copy in every CTA (two elements per thread).  The attention
// delta (16 contributions an element) is summed in "counted accumulators": one 64-bit word per element holding the
// number of contributions in its top 8 bits and their sum as a 2^-32 fixed-point number below (red.global.add.u64
// adds both at once).  A reader polls its own two words until the count is complete, which makes the wait and the
// load one L2 round trip and needs no release fence on the writers' side.  The FFN delta has one contribution per
// CTA and element: there 64-bit atomics are too slow (measured on B200: 36 G scalar 64-bit reds per second against
// 600 G elements per second through red.v4.f32), so it stays on fp32 vector reds followed by a grid barrier:
// an arrive (red.release) and a bounded wait (relaxed poll + acquire fence).
//
// Weights never wait for a barrier, and a barrier never waits behind weights.  Each CTA's rows of the seven
// matrices of a layer are packed once (pack_weights_kernel) in the order and with the row padding of four
// shared-memory slots; one thread fetches a whole slot with TMA bulk copies at the START of the phase before the
// one that reads it, so that the copies have landed when the phase's barrier is polled.  The matrix-vector
// products run on the tensor cores (mma.sync m16n8k16) with the fp32 activation vector split into three bf16
// columns, which is exact to fp32 and needs no warp-shuffle reductions.
//
// Every wait is bounded: a wait that gives up records a status word and turns the remaining waits of the CTA into
// no-ops, so a launch always terminates and the host reads the error.
//
// What the reference does for the same step: csrc/qwen3_step.cu:382-818 (four barriers per layer,
// attention recomputed by every slice CTA, fixed position 128).
#include <cstring>

#include "q3_engine.h"

namespace q3 {

constexpr int CW = 16;                        // warps per CTA
constexpr int CT = CW * 32;                   // threads per CTA
constexpr int PT = CT;                        // threads per CTA
#ifndef Q3_LM_KEEP_PCT
#define Q3_LM_KEEP_PCT 15
#endif
constexpr int LM_KEEP_PCT = Q3_LM_KEEP_PCT;   // share of the LM head asked to stay in L2 from one step to the next (15 % = 47 MB; measured: 0 % 354 us, 15 % 350, 28 % 351, 40 % 358)
#ifndef Q3_PUMP_CHUNK
#define Q3_PUMP_CHUNK 131072
#endif
constexpr int PUMP_CHUNK = Q3_PUMP_CHUNK;     // largest single bulk copy of the weight stream (a multiple of 16)
constexpr int WO_SLICES = 9;                  // row slices of Wo; CTA c < 144 owns head c % 16, slice c / 16
constexpr int F_CTAS = Q_HEADS * WO_SLICES;   // 144
constexpr int GROUP_CTAS = 2 * WO_SLICES;     // CTAs sharing one kv head
constexpr int WO_ROWS_MAX = 116;              // largest slice: 4 * ceil(256 / 9)
constexpr int PERSIST_MAX_BATCH = 3;          // sequences served by back-to-back launches
constexpr int MIN_GRID = 147;                 // row shares must fit the shared-memory slots
constexpr int SC_HALF = 128;                  // the score buffer holds 3 * SC_HALF floats
constexpr int SPLIT_SC = 3 * SC_HALF / 2;     // split attention: scores kept per head = the most positions a CTA takes (192)
constexpr int PERSIST_MAX_LEN = GROUP_CTAS * SPLIT_SC - GROUP_CTAS;   // 3438 cached positions
constexpr int WROW = 1032;                    // elements between weight rows in shared memory: 1024 + 8 of padding, so that
                                              // the eight row addresses of an ldmatrix fall into different banks
constexpr int WOROW = 136;                    // the same for the 128-column Wo slice rows
constexpr int ATT_WARPS = 8;                  // split attention: warps that attend positions (32 positions per pass)
// Local attention (every CTA attends its whole head over all cached positions) serves up to 255 positions; measured,
// splitting the positions over the 18 CTAs of a kv group wins beyond that.
#ifndef Q3_N_ACC
#define Q3_N_ACC 2
#endif
constexpr int N_ACC = Q3_N_ACC;               // accumulators for the FFN delta (fewer same-address atomics each)
constexpr int EV_PER_LAYER = 12;              // trace stamps per layer
constexpr unsigned long long WAIT_NS = 200ull * 1000 * 1000;   // default patience of every device-side wait: 200 ms
constexpr int MAX_TP = 8;                     // tensor-parallel ranks: 1, 2, 4 or 8 (at least one kv head each)
constexpr int MAX_LAYERS = 63;                // the q/k/v tags of a launch are epoch * 64 + layer + 1
// Counted accumulators: word = (contributions << 56) + sum of round(v * 2^32) as a 56-bit two's complement number.
// A contribution is clamped to +-ACC_CLAMP so that MAX_GRID of them cannot reach the count field (2^55 / 2^32 = 8.4e6).
constexpr float ACC_SCALE = 4294967296.f;     // 2^32: resolution 2.3e-10, finer than fp32 for every |x| above 4e-3
constexpr float ACC_CLAMP = 50000.f;
constexpr int MAX_GRID = 160;                 // 160 * ACC_CLAMP < 2^23
constexpr unsigned long long ACC_ONE = 1ull << 56, ACC_HALF = 1ull << 55;
// fp32 tail of shared memory: 8 KB union | q_s[2][128] k_s v_s | o split [3][128] bf16 | hid split [3][32] bf16 | red lw misc | scores
constexpr int FBUF_FLOATS = 2048 + 4 * 128 + 192 + 48 + 32 + 16 + 16 + 3 * SC_HALF;
constexpr int TAIL_BYTES = FBUF_FLOATS * 4 + 8 * 8 + 16;

struct PersistParams {
    const bf16_raw *ln1, *qn, *kn, *ln2, *fnorm, *embed;
    const bf16_raw* packed;   // [L][grid][share_elems(grid)]: every CTA's rows of the seven layer matrices, padded, in consumption order
    const long long* token;
    const uint64_t* seq_k;
    const uint64_t* seq_v;
    const long long* seq_layer_stride;
    int* seq_len;
    float* logits;
    long long* next_token;
    bf16_raw* k_write;
    bf16_raw* v_write;
    unsigned long long* dA;   // [2][1024] counted accumulators: attention delta of layer l in buffer l & 1 (16 contributions an element)
    float* dB;        // [3][N_ACC][1024] FFN delta of layer l in buffer l % 3 (fp32 accumulators, one contribution per CTA and element)
    unsigned long long* xq;   // [4096] q | k | v rows of the current layer, each a (tag << 32 | fp32 bits) word
    const unsigned* epoch;    // launches completed on this state; gives every (launch, layer) its own tag
    unsigned long long* xp;   // [8 groups][2 heads][18 CTAs][XP_STRIDE] split-attention partials (max, sum, -, -, o[128]), tagged like xq
    const float* rope;
    unsigned* sync;   // [0] grid barrier counter, [2] end-of-step ticket
    unsigned long long wait_ns;   // patience of every device-side wait
    // Tensor parallelism over tp_size GPUs (1 = off).  Entry r of every array is rank r's buffer (this rank's own at
    // r = tp_rank): the attention delta, the FFN delta, the grid-barrier counter and the end-of-step mailbox
    // (two words per sender).  Peers' buffers are their memory, mapped into this process: they are only ever the
    // target of red / st instructions, never read.
    int tp_rank, tp_size;
    unsigned long long* tp_dA[MAX_TP];
    float* tp_dB[MAX_TP];
    unsigned* tp_bar[MAX_TP];
    unsigned long long* tp_mail[MAX_TP];
    uint32_t* status;
    float* pval;
    int* pidx;
    unsigned long long* trace;   // optional [grid][4 + 12 * n_layers] %globaltimer stamps of thread 0, or nullptr
    int n_layers, vocab, append;
};

struct PersistState {
    bf16_raw* packed;       // the layer matrices re-laid per CTA (see pack_weights_kernel)
    const void* src[7];     // the seven pointers `packed` was built from
    int tp_rank, tp_size;   // tensor-parallel position (0, 1 when off)
    float* peer_X[MAX_TP];  // the state allocations of all ranks as mapped here (own at tp_rank)
    float* X;               // dA[2] (64-bit words) | dB[3][N_ACC] (fp32) | xq[4096] (64-bit words) | epoch | xp
    int grid, smem;
};

// Which rows of which matrix CTA c of a grid of G owns, and how many elements its packed share of
// one layer takes.  Used by the decode kernel and by the kernel that packs the weights.
constexpr int XP_STRIDE = 132;                // 64-bit words per published partial
constexpr size_t XP_WORDS = (size_t)KV_HEADS * 2 * GROUP_CTAS * XP_STRIDE;
constexpr size_t ACC_FLOATS = (size_t)(4 + 3 * N_ACC) * HIDDEN;   // two vectors of 64-bit words, 3 * N_ACC of floats
constexpr size_t TP_OFFSET = ACC_FLOATS + 2 * QKV_DIM + 64 + 2 * XP_WORDS;   // [0] barrier counter of the tensor-parallel mode; mailbox at + 64 floats
constexpr size_t X_FLOATS = TP_OFFSET + 128;
struct Share {
    int q0, nq, qmax;       // rows [q0, q0 + nq) of this rank's [wq; wk; wv] rows, slot rows qmax
    int i0, ni, imax;       // FFN rows [i0, i0 + ni) of gate, up and down^T (global row numbers), slot rows imax
    int fh, fhl, fs, fr0, fn;   // F: query head (global, local), Wo row slice index, slice rows [fr0, fr0 + fn)
    int slices;             // Wo row slices per head
    bool has_f;
};
// With T tensor-parallel ranks, rank r owns query heads [r 16/T, (r+1) 16/T), kv heads [r 8/T, (r+1) 8/T), FFN rows
// [r 3072/T, (r+1) 3072/T) and, for the LM head, words [r V/T, (r+1) V/T); its 144 F CTAs are its 16/T heads times
// 9 T row slices of Wo.
__host__ __device__ inline Share share_of(int c, int G, int T = 1, int rank = 0) {
    Share s;
    const int QL = QKV_DIM / T, IL = INTER / T, HL = Q_HEADS / T;
    s.q0 = (int)((long long)c * QL / G); s.nq = (int)((long long)(c + 1) * QL / G) - s.q0; s.qmax = (QL + G - 1) / G;
    s.i0 = (int)((long long)c * IL / G); s.ni = (int)((long long)(c + 1) * IL / G) - s.i0; s.imax = (IL + G - 1) / G;
    s.i0 += rank * IL;
    s.has_f = c < F_CTAS;
    s.slices = F_CTAS / HL;
    s.fhl = c % HL; s.fs = c / HL; s.fh = rank * HL + s.fhl;
    s.fr0 = (s.fs * 256 / s.slices) * 4; s.fn = ((s.fs + 1) * 256 / s.slices) * 4 - s.fr0;
    return s;
}
// packed share of one (layer, CTA): A [qmax][WROW] | B [116][WOROW] | C [2 imax][WROW] | D [imax][WROW]
__host__ __device__ inline size_t share_elems(int G, int T = 1) {
    const int qmax = (QKV_DIM / T + G - 1) / G, imax = (INTER / T + G - 1) / G;
    return (size_t)(qmax + 3 * imax) * WROW + (size_t)WO_ROWS_MAX * WOROW;
}

// ---- PTX helpers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// SYS = true: system scope, for buffers that other GPUs add to as well (tensor parallelism)
template <bool SYS>
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    if (SYS) asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
    else asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float2 ldcg2(const float* p) { return __ldcg(reinterpret_cast<const float2*>(p)); }
// ---- counted accumulators ----------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long acc_word(float v) {
    v = fminf(fmaxf(v, -ACC_CLAMP), ACC_CLAMP);
    return ACC_ONE + (unsigned long long)__float2ll_rn(v * ACC_SCALE);
}
template <bool SYS>
__device__ __forceinline__ void acc_add(unsigned long long* addr, unsigned long long w) {
    if (SYS) asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(addr), "l"(w) : "memory");
    else asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(addr), "l"(w) : "memory");
}
template <bool SYS>
__device__ __forceinline__ void acc_load2(const unsigned long long* src, unsigned long long& w0, unsigned long long& w1) {
    if (SYS) asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(src) : "memory");
    else asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(src) : "memory");
}
__device__ __forceinline__ unsigned acc_count(unsigned long long w) { return (unsigned)((w + ACC_HALF) >> 56); }
__device__ __forceinline__ float acc_value(unsigned long long w) {
    const long long s = (long long)((w + ACC_HALF) & (ACC_ONE - 1)) - (long long)ACC_HALF;
    return __ll2float_rn(s) * (1.f / ACC_SCALE);
}
// barrier of the whole CTA (512 threads)
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// ---- counters in global memory: arrive and bounded wait ---------------------------------------------
__device__ __forceinline__ void counter_arrive(unsigned* cnt) {   // one thread, after a cta_sync
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
}
// the same on the counters of all `n` tensor-parallel ranks: one system-scope release fence, then one arrival each
__device__ __forceinline__ void counter_arrive_all(unsigned* const* cnt, int n) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int r = 0; r < n; ++r) asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(cnt[r]) : "memory");
}
// thread 0 polls until *cnt has reached `target` (wrap-safe), then every thread passes a cta_sync
template <bool SYS>
__device__ __forceinline__ void counter_wait(const unsigned* cnt, unsigned target, volatile int* abort_flag,
                                             uint32_t* status, uint32_t site, unsigned long long wait_ns) {
    if (threadIdx.x == 0 && !*abort_flag) {
        unsigned v;
        unsigned long long t0 = 0;
        unsigned it = 0;
        for (;;) {
            if (SYS) asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
            else asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
            if ((int)(v - target) >= 0) break;
            if ((++it & 255u) == 0) {
                const unsigned long long t = global_ns();
                if (t0 == 0) t0 = t;
                else if (t - t0 > wait_ns) {
                    report(status, ST_BARRIER_TIMEOUT, site, v);
                    *abort_flag = 1;
                    break;
                }
            }
        }
        if (SYS) asm volatile("fence.acq_rel.sys;" ::: "memory");
        else asm volatile("fence.acquire.gpu;" ::: "memory");
    }
    cta_sync();
}
// bounded wait on a shared-memory mbarrier; returns false when it gave up
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag, uint32_t* status, uint32_t site,
                                          unsigned long long wait_ns) {
    unsigned it = 0;
    unsigned long long t0 = 0;
    while (!mbar_try_wait(b, parity)) {
        if ((++it & 255u) == 0) {
            const unsigned long long t = global_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > wait_ns) {
                if ((threadIdx.x & 31) == 0) { report(status, ST_MBAR_TIMEOUT, site, parity); *abort_flag = 1; }
                return false;
            }
        }
    }
    return true;
}

// a single non-blocking test when the slot is already full (the normal case: the copies were issued a
// phase or more ahead); a late slot is polled by one lane per warp
__device__ __forceinline__ void slot_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag, uint32_t* status, uint32_t site,
                                          unsigned long long wait_ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    if (__all_sync(0xffffffffu, ok != 0)) return;
    if ((threadIdx.x & 31) == 0) mbar_wait(b, parity, abort_flag, status, site, wait_ns);
    __syncwarp();
}

// sum of the sixteen per-warp partial sums, read by one thread (four broadcast 16-byte loads)
__device__ __forceinline__ float sum16(const float* red) {
    const float4 a = *reinterpret_cast<const float4*>(red), b = *reinterpret_cast<const float4*>(red + 4);
    const float4 c = *reinterpret_cast<const float4*>(red + 8), d = *reinterpret_cast<const float4*>(red + 12);
    return ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w)) + (((c.x + c.y) + (c.z + c.w)) + ((d.x + d.y) + (d.z + d.w)));
}

__device__ __forceinline__ void unpack8f(const uint4& u, float* f) {
    f[0] = bf_lo(u.x); f[1] = bf_hi(u.x); f[2] = bf_lo(u.y); f[3] = bf_hi(u.y);
    f[4] = bf_lo(u.z); f[5] = bf_hi(u.z); f[6] = bf_lo(u.w); f[7] = bf_hi(u.w);
}
// ---- tensor-core GEMV pieces ------------------------------------------------------------------------
// y = W x with bf16 W and fp32 x runs on mma.sync.m16n8k16: W tiles are the A operand (ldmatrix from
// the padded shared-memory rows), and x enters as THREE bf16 columns of the B operand, x = hi + mid +
// lo (each the bf16 rounding of what the previous ones left), so that the products are exact and the
// fp32 accumulators hold W.hi, W.mid and W.lo; their sum is the fp32 dot product.  The other five
// B columns are zero.  No warp shuffles, a handful of instructions per 16 x 16 tile.
__device__ __forceinline__ void split3(float x, bf16_raw& h, bf16_raw& m, bf16_raw& l) {
    h = f_to_bf(x);
    const float r1 = x - bf_to_f(h);
    m = f_to_bf(r1);
    l = f_to_bf(r1 - bf_to_f(m));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&a)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&a)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// After the k loop: lanes with (lane & 3) == 0 hold columns 0, 1 (hi, mid) of rows g and g + 8, the
// next lane holds column 2 (lo).  Returns the two row sums in the (lane & 3) == 0 lanes.
__device__ __forceinline__ void fold_cols(const float (&c)[4], float& row_lo, float& row_hi) {
    const float l0 = __shfl_down_sync(0xffffffffu, c[0], 1);
    const float l1 = __shfl_down_sync(0xffffffffu, c[2], 1);
    row_lo = (c[0] + c[1]) + l0;
    row_hi = (c[2] + c[3]) + l1;
}


// Local attention keeps its K rows in a ring of four register buffers (a quarter-warp per position,
// 64 positions per pass): pass i lives in buffer i & 3 and the load of pass i + 4 is issued the moment
// pass i has been consumed.  The V rows are read dim-major instead (one warp per position, four dims
// per lane), so P.V needs no shuffles: the first eight positions of every warp are fetched before the
// barrier wait, the rest inside the loop.
__device__ __forceinline__ void ring_load(uint4 (&buf)[2], int pass, int npl, int len, int att_slot, int sub, const bf16_raw* kl) {
    const int pos = pass * 64 + att_slot;
    const bool live = pass < npl && pos < len;
    const uint4* row = reinterpret_cast<const uint4*>(kl + (size_t)(live ? pos : 0) * KV_DIM);
    ld_row16(buf[0], row + sub, live);
    ld_row16(buf[1], row + 8 + sub, live);
}
__device__ __forceinline__ uint2 ld_stream8(const void* ptr) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
    return v;
}
constexpr int LOCAL_V_PRE = 8;   // V positions per warp fetched ahead of the barrier wait
// Local attention: the i-th position whose V row warp w weighs.
__device__ __forceinline__ int local_v_pos(int w, int i) { return w + CW * i; }

// ====================================================================================================
// MODE picks the attention scheme at compile time, so that each variant carries only its own code and registers:
//   0  local attention, up to 128 cached positions (everything prefetched into 32 registers)
//   1  local attention, up to 191 cached positions (a third K pass and four more V rows in 16 more registers)
//   2  local attention, up to 255 cached positions (a fourth K pass and another four V rows)
//   3  split attention, up to PERSIST_MAX_LEN cached positions
// (measured per step at 192 / 255 / 319 / 383 positions: local 392 / 417 / 475 / 511 us, split 450 us throughout).
// The host picks the variant from its upper bound of the length; a cache longer than the variant serves is reported.
constexpr int N_MODES = 4;
__host__ __device__ constexpr int mode_max_len(int mode) { return mode == 0 ? 128 : mode < N_MODES - 1 ? 127 + 64 * mode : PERSIST_MAX_LEN; }
// TP: tensor-parallel build of the same kernel (system-scope atomics on the deltas, every rank's CTAs arrive at every
// rank's barrier, the arg-max is settled through the mailboxes); local attention only.
template <int MODE, bool TP>
__global__ void __launch_bounds__(PT, 1) q3_persist_decode(const PersistParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x, G = gridDim.x;
    const int L = p.n_layers;
    const unsigned long long wait_ns = p.wait_ns;
    if (p.seq_len[0] > mode_max_len(MODE) || p.seq_len[0] < 0) {   // the same for every CTA: nothing has been started yet
        if (tid == 0) report(p.status, ST_BAD_LEN, (uint32_t)MODE, (uint32_t)p.seq_len[0]);
        return;
    }

    // ---- static ownership ----
    static_assert(!TP || MODE < N_MODES - 1, "tensor parallelism serves the local-attention variants only");
    const int T = TP ? p.tp_size : 1, rank = TP ? p.tp_rank : 0;
    const Share sh = share_of(c, G, T, rank);
    const int q0 = sh.q0, nq = sh.nq, i0 = sh.i0, ni = sh.ni, qmax = sh.qmax, imax = sh.imax;
    const bool has_f = sh.has_f;
    const int fh = sh.fh, fs = sh.fs, fg = fh >> 1, fhh = fh & 1;   // fg: the (global) kv head of this CTA's query head
    const int fgl = sh.fhl >> 1;                                  // ... and its number among this rank's kv heads
    const int qrows = Q_DIM / T, kvrows = KV_DIM / T;             // this rank's q rows and k (= v) rows
    const int fj = fhh * sh.slices + fs;                          // index inside the kv-head group, 0..17 (without tensor parallelism)
    const int fr0 = sh.fr0, fn = sh.fn;
    (void)i0;
    const bool kv_writer = has_f && fj == 0;                      // one CTA per kv head stores the new K/V rows

    // ---- shared memory carve-up ----
    bf16_raw* sA = reinterpret_cast<bf16_raw*>(smem);                       // qkv rows        [qmax][WROW]
    bf16_raw* sB = sA + (size_t)qmax * WROW;                                // Wo slice        [116][WOROW]
    bf16_raw* sC = sB + WO_ROWS_MAX * WOROW;                                // gate | up rows  [2][imax][WROW]
    bf16_raw* sD = sC + (size_t)2 * imax * WROW;                            // down^T rows     [imax][WROW]
    float* fbuf = reinterpret_cast<float*>(sD + (size_t)imax * WROW);
    // one 8 KB region with a different tenant per phase
    uint32_t* xsp = reinterpret_cast<uint32_t*>(fbuf);   // Q, GD: activations split in three bf16 parts, [3][512] pairs (6 KB)
    float* part = fbuf + 1536;                           // Q: per-warp partial row sums [16][32] (2 KB)
    float* gpart = fbuf + 1536;                          // GD: per-warp partial sums of the 48 gate/up tile rows [16][48] (3 KB: runs into q_s, idle in GD)
    float* om = fbuf;                                    // F: [8 warps][2 heads][128] attention partials
    float* wo_part = fbuf;                               // F: [2 k-halves][128] Wo slice partial sums (after the partials are published)
    float* dout = fbuf;                                  // GD: [1024] down-projection outputs of this CTA (after the gate/up rows)
    float* xs = fbuf;                                    // LM head: [1024] fp32 activations
    float* q_s = fbuf + 2048;    // [2][128] both query heads of the group, scaled by 1/sqrt(128)
    float* k_s = q_s + 256;      // [128] the new K row (after norm + RoPE), fp32
    float* v_s = k_s + 128;      // [128] the new V row, fp32
    uint32_t* osp = reinterpret_cast<uint32_t*>(v_s + 128);   // [3][64] pairs: attention output of this CTA's head, split
    uint32_t* hsp = osp + 192;   // [3][16] pairs: this CTA's hid values, split
    float* red = reinterpret_cast<float*>(hsp + 48);          // [32]
    float* lw = red + 32;        // [16] per-warp probability sums, [w][head]
    float* misc = lw + 16;       // [16]: [0] score of the new row for this CTA's head
    float* sc = misc + 16;       // split attention: [2][SPLIT_SC] scores of this CTA's positions; local: [3 * SC_HALF] scores of all positions
    uint64_t* full = reinterpret_cast<uint64_t*>(sc + 3 * SC_HALF);   // [4] slot filled
    volatile int* abort_flag = reinterpret_cast<volatile int*>(full + 8);

    const int n_ev = 4 + EV_PER_LAYER * L;
#define Q3_TRACE(ev) do { if (p.trace != nullptr && tid == 0) p.trace[(size_t)c * n_ev + (ev)] = global_ns(); } while (0)
    Q3_TRACE(0);
    if (tid == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(&full[i], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // LM head rows of this CTA, four rows in flight per warp; every warp of the CTA (producers included)
    // takes part once the layer loop is over.  Keeps the warp's best (value, row); ties -> lowest row.
    // L2 residency: the layer matrices and most of the LM head pass through the 126 MB L2 once per step and are
    // fetched with an evict-first hint; the first LM_KEEP_PCT percent of every CTA's LM-head rows are fetched with an
    // evict-last hint instead, so that they are still in L2 when the next step of a decode loop comes for them.
    uint64_t pol_stream, pol_keep;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol_stream));
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol_keep));
    auto lm_stream = [&](int wi, int nw, float& bestv, int& besti) {
        const int vlo = (int)((long long)rank * p.vocab / T), V = (int)((long long)(rank + 1) * p.vocab / T) - vlo;   // this rank's words
        const int v0 = vlo + (int)((long long)c * V / G), v1 = vlo + (int)((long long)(c + 1) * V / G);
        const int vkeep = v0 + (int)((long long)(v1 - v0) * LM_KEEP_PCT / 100);
        for (int base = v0 + wi * 4; base < v1; base += nw * 4) {
            uint4 w[4][4];
            const uint64_t pol = (base < vkeep) ? pol_keep : pol_stream;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int row = min(base + k, v1 - 1);
                const uint4* rp = reinterpret_cast<const uint4*>(p.embed + (size_t)row * HIDDEN);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                                 : "=r"(w[k][j].x), "=r"(w[k][j].y), "=r"(w[k][j].z), "=r"(w[k][j].w) : "l"(rp + j * 32 + lane), "l"(pol));
            }
            float acc[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc[k] = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[k] += dot8(w[k][j], xs, j, lane);
                acc[k] = warp_sum(acc[k]);
            }
            if (lane == 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int row = base + k;
                    if (row < v1) {
                        if (p.logits) p.logits[row] = acc[k];
                        if (acc[k] > bestv) { bestv = acc[k]; besti = row; }
                    }
                }
            }
        }
    };
    float* const lm_bv = q_s;                               // [CW + NPW] per-warp best values
    int* const lm_bi = reinterpret_cast<int*>(k_s);         // [CW + NPW] and their rows

    // ================================================================================ weight delivery
    // There are no producer warps.  One thread (lane 0 of warp 1) moves the CTA's packed rows into the four slots
    // with TMA bulk copies, a whole slot at a time, at the START of a phase, so that the copies have landed before
    // the phase ends and nothing is in flight while a grid barrier is polled: measured on B200, a barrier polled
    // while 64 KB per SM of bulk copies are in flight takes 2.1 to 2.6 us instead of 1.55 us (the poll's answer
    // queues behind the copies), and cp.async (LDGSTS) copies in flight slow the other warps' own accesses.
    //   start of Q  (layer l): down rows of layer l         (43 KB, read in GD)
    //   start of F  (layer l): gate/up rows of layer l      (87 KB, read in GD)
    //   start of GD (layer l): q/k/v rows and Wo slice of layer l + 1   (58 + 31 KB)
    // The first chunk of a slot arms the slot's mbarrier with the slot's byte count; every warp waits on it before it reads the slot.
    const int bytesA = qmax * WROW * 2, bytesB = WO_ROWS_MAX * WOROW * 2, bytesC = 2 * imax * WROW * 2, bytesD = imax * WROW * 2;
    const bool pumper = tid == 32;
    int pump_armed = 0, pump_parity = 0;                // per slot: armed at all, and the parity of its last armed phase
    auto fetch_slot = [&](int slot, int layer) {
        if (!pumper || layer >= L || (slot == 1 && !has_f)) return;
        const int bytes = slot == 0 ? bytesA : slot == 1 ? bytesB : slot == 2 ? bytesC : bytesD;
        const int off = slot == 0 ? 0 : slot == 1 ? bytesA : slot == 2 ? bytesA + bytesB : bytesA + bytesB + bytesC;
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.packed + ((size_t)layer * G + c) * share_elems(G, T)) + off;
        unsigned char* dst = reinterpret_cast<unsigned char*>(slot == 0 ? sA : slot == 1 ? sB : slot == 2 ? sC : sD);
        fence_proxy_async();   // the slot's last readers used ordinary loads; they are behind a CTA barrier
        mbar_expect_tx(&full[slot], (uint32_t)bytes);
        pump_armed |= 1 << slot;
        pump_parity = (pump_parity & ~(1 << slot)) | ((layer & 1) << slot);
        for (int o = 0; o < bytes; o += PUMP_CHUNK)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                         ::"r"(smem_u32(dst + o)), "l"(src + o), "r"((uint32_t)min(PUMP_CHUNK, bytes - o)), "r"(smem_u32(&full[slot])), "l"(pol_stream) : "memory");
    };
    fetch_slot(0, 0);
    fetch_slot(1, 0);

    // ================================================================================ the step
    long long tok = p.token[0];
    if (tok < 0 || tok >= p.vocab) {
        if (tid == 0) report(p.status, ST_BAD_TOKEN, 0, (uint32_t)tok);
        tok = 0;
    }
    const int len = p.seq_len[0];
    const bf16_raw* kcache = reinterpret_cast<const bf16_raw*>(p.seq_k[0]);
    const bf16_raw* vcache = reinterpret_cast<const bf16_raw*>(p.seq_v[0]);
    const long long lstride = p.seq_layer_stride[0];
    const float* rope_row = p.rope + (size_t)len * HEAD_DIM;
    // The residual stream: elements 2 tid and 2 tid + 1 of x, the same values in every CTA.
    float x0, x1;
    {
        const uint32_t e = *reinterpret_cast<const uint32_t*>(p.embed + (size_t)tok * HIDDEN + 2 * tid);
        x0 = bf_lo(e); x1 = bf_hi(e);
    }
    // x += the attention delta, once all 16 contributions to this thread's two words have arrived (bounded).  The wait IS
    // the load: no counter, no fence; a word that is complete cannot change any more until the buffer is cleared.
    // Thread 0 first polls one sentinel word until it is nearly complete, so that the grid does not hammer lines that
    // are still being added to (measured: 0.5 us faster per wait than every thread polling from the start).
    auto acc_wait = [&](const unsigned long long* vec, unsigned expect, uint32_t site) {
        if (tid == 0 && !*abort_flag) {
            unsigned long long ws;
            unsigned it = 0;
            unsigned long long t0 = 0;
            for (;;) {
                if (TP) asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(ws) : "l"(vec + HIDDEN - 1) : "memory");
                else asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(ws) : "l"(vec + HIDDEN - 1) : "memory");
                if (acc_count(ws) + 2u >= expect) break;
                if ((++it & 63u) == 0) {
                    const unsigned long long t = global_ns();
                    if (t0 == 0) t0 = t;
                    else if (t - t0 > wait_ns) { report(p.status, ST_BARRIER_TIMEOUT, site, acc_count(ws)); *abort_flag = 1; break; }
                }
            }
        }
        cta_sync();
        unsigned long long w0 = 0, w1 = 0;
        if (!*abort_flag) {
            const unsigned long long* src = vec + 2 * tid;
            unsigned it = 0;
            unsigned long long t0 = 0;
            for (;;) {
                acc_load2<TP>(src, w0, w1);
                if (acc_count(w0) == expect && acc_count(w1) == expect) break;
                if ((++it & 63u) == 0) {
                    if (*abort_flag) break;
                    const unsigned long long t = global_ns();
                    if (t0 == 0) t0 = t;
                    else if (t - t0 > wait_ns) {
                        report(p.status, ST_BARRIER_TIMEOUT, site, acc_count(w0));
                        *abort_flag = 1;
                        break;
                    }
                }
            }
            if (*abort_flag) { w0 = 0; w1 = 0; }
        }
        x0 += acc_value(w0); x1 += acc_value(w1);
    };
    // x += the FFN delta: the sum of its fp32 accumulators (after the layer's grid barrier)
    auto add_ffn_delta = [&](const float* dBl) {
        float2 d[N_ACC];
#pragma unroll
        for (int i = 0; i < N_ACC; ++i) d[i] = ldcg2(dBl + (size_t)i * HIDDEN + 2 * tid);
        float s0 = d[0].x, s1 = d[0].y;
#pragma unroll
        for (int i = 1; i < N_ACC; ++i) { s0 += d[i].x; s1 += d[i].y; }
        x0 += s0; x1 += s1;
    };
    unsigned* bar = TP ? p.tp_bar[rank] : p.sync;
    unsigned target = 0;
    // Every (launch, layer) tags its q/k/v words differently, so a reader can tell a fresh word from an old one.
    const unsigned tag_base = __ldcg(p.epoch) * 64u;
    const int quarter = lane >> 3, sub = lane & 7;
    // ldmatrix.x4 row addresses of a 16 x 16 A tile: lanes 0-7 rows 0-7, 8-15 rows 8-15 (k 0-7); 16-31 the same rows at k 8-15
    const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8, lm_k = (lane >> 4) * 8;
    const int fr_n = lane >> 2, fr_k = (lane & 3) * 2;   // B fragment: column n, k pair; C fragment: rows fr_n, fr_n + 8

    // this CTA's share of the cached positions of kv head fg: [cp0, cp1)
    const int chunk = (len + GROUP_CTAS - 1) / GROUP_CTAS;
    const int cp0 = min(len, fj * chunk), cp1 = min(len, cp0 + chunk);
    const int npass = (cp1 - cp0 + 31) >> 5;                  // 32 positions per pass (warps 0..7, a quarter-warp each)
    const int att_slot = warp * 4 + quarter;                  // < 32 for the attending warps
    // Short caches: every CTA recomputes the attention of its own head over all positions (no exchange between
    // CTAs; the K/V rows come from L2).  Longer caches: the 18 CTAs of a kv group split the positions.
    constexpr bool local_attn = MODE < N_MODES - 1;
    constexpr int XPASS = local_attn ? MODE : 0;   // K passes (and groups of four V rows) beyond the first two
    const int npl = (len + 63) >> 6;                          // local attention: passes of 64 positions (16 warps x 4 quarter-warps)

    // gains of the next GEMV phase, fetched ahead of the barrier wait
    uint32_t gain2 = *reinterpret_cast<const uint32_t*>(p.ln1 + 2 * tid);

    uint4 ring[4][2];
    uint4 ring3[XPASS > 0 ? XPASS : 1][2];    // passes 2..: K row of position 64 pass + slot
    uint4 vext[XPASS > 0 ? 2 * XPASS : 1];    // ... and V[warp + 16 i][4 lane ..] for i = 8 .., two rows per uint4
    for (int l = 0; l < L; ++l) {
        const int ev = 1 + EV_PER_LAYER * l;
        // The attention delta alternates between two buffers, the FFN delta goes round three.  The last CTA clears, at the
        // start of GD of layer l, the attention buffer of layer l - 1 (next written in F of layer l + 1) and the FFN buffer
        // of layer l - 2 (next written in GD of layer l + 1): it has passed the grid barrier of layer l - 1, which every CTA
        // reaches after its last read of both, and its arrival at the barrier of layer l releases the stores to every
        // later writer.
        unsigned long long* dAl = p.dA + (size_t)(l & 1) * HIDDEN;
        float* dBl = p.dB + (size_t)(l % 3) * N_ACC * HIDDEN;
        const unsigned tag = tag_base + (unsigned)l + 1u;
        // K and V rows of the cached positions, fetched at the very start of the layer (they depend on nothing of this
        // step), so that they have arrived, and the SM's input path is quiet, when the q/k/v exchange starts polling.
        // Split attention: [0], [1] = K passes, [2], [3] = V passes of the CTA's positions.  Local attention:
        // [0], [1] = K passes 0, 1 (a quarter-warp per position) and [2], [3] = V[warp + 16 i][4 lane .. 4 lane + 3]
        // for i < 8, two positions per uint4.
        const bf16_raw* kl = kcache + (size_t)l * lstride + fg * HEAD_DIM;
        const bf16_raw* vl = vcache + (size_t)l * lstride + fg * HEAD_DIM;
        auto kv_prefetch = [&](int ll) {
            const bf16_raw* kl = kcache + (size_t)ll * lstride + fg * HEAD_DIM;
            const bf16_raw* vl = vcache + (size_t)ll * lstride + fg * HEAD_DIM;
            if (has_f && ll < L) {
                if (local_attn) {
#pragma unroll
                    for (int i = 0; i < 2; ++i) ring_load(ring[i], i, npl, len, att_slot, sub, kl);
                    if constexpr (XPASS > 0) {
#pragma unroll
                        for (int x = 0; x < XPASS; ++x) ring_load(ring3[x], 2 + x, npl, len, att_slot, sub, kl);
#pragma unroll
                        for (int i = 0; i < 4 * XPASS; ++i) {
                            const int pos = local_v_pos(warp, LOCAL_V_PRE + i);
                            const bool live = pos < len;
                            const bf16_raw* vp = vl + (size_t)(live ? pos : 0) * KV_DIM + lane * 4;
                            uint4& dst = vext[i >> 1];
                            if (i & 1) ld_row8(dst.z, dst.w, vp, live); else ld_row8(dst.x, dst.y, vp, live);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < LOCAL_V_PRE; ++i) {
                        const int pos = local_v_pos(warp, i);
                        const bool live = pos < len;
                        const bf16_raw* vp = vl + (size_t)(live ? pos : 0) * KV_DIM + lane * 4;
                        uint4& dst = ring[2 + (i >> 2)][(i >> 1) & 1];
                        if (i & 1) ld_row8(dst.z, dst.w, vp, live); else ld_row8(dst.x, dst.y, vp, live);
                    }
                } else if (warp < ATT_WARPS) {
#pragma unroll
                    for (int ps = 0; ps < 2; ++ps) {   // K: a quarter-warp per position
                        const int pos = cp0 + ps * 32 + att_slot;
                        const bool live = pos < cp1;
                        const uint4* kr = reinterpret_cast<const uint4*>(kl + (size_t)(live ? pos : 0) * KV_DIM);
                        ld_row16(ring[ps][0], kr + sub, live);
                        ld_row16(ring[ps][1], kr + 8 + sub, live);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {      // V: a warp per position, four dims per lane
                        const int pos = cp0 + warp + ATT_WARPS * i;
                        const bool live = pos < cp1;
                        const bf16_raw* vp = vl + (size_t)(live ? pos : 0) * KV_DIM + lane * 4;
                        uint4& dst = ring[2 + (i >> 2)][(i >> 1) & 1];
                        if (i & 1) ld_row8(dst.z, dst.w, vp, live); else ld_row8(dst.x, dst.y, vp, live);
                    }
                }
            }
        };
        // ==================================================================== Q
        {
            if (l > 0) add_ffn_delta(p.dB + (size_t)((l - 1) % 3) * N_ACC * HIDDEN);
            fetch_slot(3, l);   // down rows of this layer: landed before the q/k/v exchange starts polling
            {   // stage x * gain split in three bf16 parts (the 1/rms factor is applied to the row sums)
                bf16_raw h0, m0, l0, h1, m1, l1;
                split3(x0 * bf_lo(gain2), h0, m0, l0);
                split3(x1 * bf_hi(gain2), h1, m1, l1);
                xsp[tid] = (uint32_t)h0 | ((uint32_t)h1 << 16);
                xsp[512 + tid] = (uint32_t)m0 | ((uint32_t)m1 << 16);
                xsp[1024 + tid] = (uint32_t)l0 | ((uint32_t)l1 << 16);
            }
            const float ss = warp_sum(x0 * x0 + x1 * x1);
            if (lane == 0) red[warp] = ss;
            // the warps that will poll the q/k/v exchange request their K/V rows now (x is staged: nothing queues behind
            // these loads), the others while they wait for the exchange
            if (warp >= 8 && warp < 12) kv_prefetch(l);
            cta_sync();
            Q3_TRACE(ev + 0);
            // warp w: k range [64 w, 64 w + 64) of both 16-row tiles of this CTA's rows
            uint32_t bq[4][2];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int kp = (64 * warp + 16 * t + fr_k) >> 1;
                bq[t][0] = (fr_n < 3) ? xsp[fr_n * 512 + kp] : 0u;
                bq[t][1] = (fr_n < 3) ? xsp[fr_n * 512 + kp + 4] : 0u;
            }
            slot_wait(&full[0], l & 1, abort_flag, p.status, 10, wait_ns);
            {
                uint32_t af[2][4][4];
#pragma unroll
                for (int rt = 0; rt < 2; ++rt) {
                    const uint32_t abase = smem_u32(sA + (size_t)(16 * rt + lm_row) * WROW + 64 * warp + lm_k);
#pragma unroll
                    for (int t = 0; t < 4; ++t) ldsm_x4(af[rt][t], abase + 32 * t);
                }
                float cc[2][2][4];
#pragma unroll
                for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < 4; ++i) cc[rt][h][i] = 0.f;
#pragma unroll
                for (int t = 0; t < 4; ++t)
#pragma unroll
                    for (int rt = 0; rt < 2; ++rt) mma_bf16(cc[rt][t & 1], af[rt][t], bq[t][0], bq[t][1]);
#pragma unroll
                for (int rt = 0; rt < 2; ++rt) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) cc[rt][0][i] += cc[rt][1][i];
                    float r0, r1;
                    fold_cols(cc[rt][0], r0, r1);
                    if ((lane & 3) == 0) { part[warp * 32 + 16 * rt + fr_n] = r0; part[warp * 32 + 16 * rt + fr_n + 8] = r1; }
                }
            }
            cta_sync();
            if (warp == 0) {   // nq <= 28: the row sums and the 1/rms factor sit in warp 0
                if (tid < nq) {
                    const float r = rsqrtf(sum16(red) / (float)HIDDEN + EPS);
                    float v0 = 0.f, v1 = 0.f;
#pragma unroll
                    for (int w = 0; w < CW; w += 2) { v0 += part[w * 32 + tid]; v1 += part[w * 32 + 32 + tid]; }
                    // value and tag travel in one 64-bit word: no barrier between Q and F, the readers poll the tags
                    const unsigned long long word = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint((v0 + v1) * r);
                    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p.xq + q0 + tid), "l"(word) : "memory");
                }
                Q3_TRACE(ev + 1);
            }
            if (warp < 8 || warp >= 12) kv_prefetch(l);   // after the rows are published: nothing waits for these warps now
        }

        // ---- what the F phase needs that no other CTA produces: norm gains and the RoPE row ----
        float gq[4] = {0.f, 0.f, 0.f, 0.f}, cs[4] = {0.f, 0.f, 0.f, 0.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
        if (has_f) {
            if (warp >= 8 && warp < 11) {   // warps 8, 9 normalise the two q heads, warp 10 normalises k: dims 4*lane..
                const bf16_raw* gsrc = (warp < 10 ? p.qn : p.kn) + (size_t)l * HEAD_DIM + lane * 4;
                const uint2 gg = *reinterpret_cast<const uint2*>(gsrc);
                gq[0] = bf_lo(gg.x); gq[1] = bf_hi(gg.x); gq[2] = bf_lo(gg.y); gq[3] = bf_hi(gg.y);
                const float4 cc = *reinterpret_cast<const float4*>(rope_row + ((lane * 4) & 63));
                const float4 sv = *reinterpret_cast<const float4*>(rope_row + 64 + ((lane * 4) & 63));
                cs[0] = cc.x; cs[1] = cc.y; cs[2] = cc.z; cs[3] = cc.w;
                sn[0] = sv.x; sn[1] = sv.y; sn[2] = sv.z; sn[3] = sv.w;
            }
        }
        fetch_slot(2, l);       // gate/up rows of this layer: in flight during F, landed before its barrier is polled
        Q3_TRACE(ev + 2);

        // ==================================================================== F
        if (has_f) {
            // ---- q (both heads of the group), k, v of the new position: warps 8..11 ----
            if (warp >= 8 && warp < 12) {
                const int role = warp - 8;   // 0, 1: q heads 2g, 2g+1;  2: k;  3: v
                const unsigned long long* src = p.xq + (role < 2 ? (2 * fgl + role) * HEAD_DIM : (role == 2 ? qrows + fgl * HEAD_DIM : qrows + kvrows + fgl * HEAD_DIM)) + lane * 4;
                unsigned long long w0, w1, w2, w3;
                {   // bounded poll: the four words of this lane must all carry this layer's tag
                    unsigned it = 0;
                    unsigned long long t0 = 0;
                    for (;;) {
                        asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(src) : "memory");
                        asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(w2), "=l"(w3) : "l"(src + 2) : "memory");
                        const bool fresh = (unsigned)(w0 >> 32) == tag && (unsigned)(w1 >> 32) == tag && (unsigned)(w2 >> 32) == tag && (unsigned)(w3 >> 32) == tag;
                        if (__all_sync(0xffffffffu, fresh)) break;
                        if (*abort_flag) break;
                        if ((++it & 127u) == 0) {
                            const unsigned long long t = global_ns();
                            if (t0 == 0) t0 = t;
                            else if (t - t0 > wait_ns) {
                                if (lane == 0) { report(p.status, ST_BARRIER_TIMEOUT, 100 + l, (uint32_t)(w0 >> 32)); *abort_flag = 1; }
                                break;
                            }
                        }
                    }
                }
                const float4 v4 = make_float4(__uint_as_float((unsigned)w0), __uint_as_float((unsigned)w1), __uint_as_float((unsigned)w2), __uint_as_float((unsigned)w3));
                float v[4] = {v4.x, v4.y, v4.z, v4.w};
                float* dst = (role < 2) ? q_s + role * 128 : (role == 2 ? k_s : v_s);
                if (role < 3) {
                    const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
                    const float r = rsqrtf(ss / (float)HEAD_DIM + EPS);
                    const float post = (role < 2) ? ATTN_SCALE : 1.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float n = (v[i] * r) * gq[i];
                        const float partner = __shfl_xor_sync(0xffffffffu, n, 16);
                        const float rot = (lane < 16) ? -partner : partner;
                        v[i] = n * cs[i] + rot * sn[i];
                    }
                    *reinterpret_cast<float4*>(dst + lane * 4) = make_float4(v[0] * post, v[1] * post, v[2] * post, v[3] * post);
                } else {
                    *reinterpret_cast<float4*>(dst + lane * 4) = v4;
                }
                if (role >= 2 && kv_writer) {   // the new K (after norm + RoPE) and V rows, rounded to bf16
                    uint2 pk;
                    pk.x = (uint32_t)f_to_bf(v[0]) | ((uint32_t)f_to_bf(v[1]) << 16);
                    pk.y = (uint32_t)f_to_bf(v[2]) | ((uint32_t)f_to_bf(v[3]) << 16);
                    bf16_raw* wr = (role == 2) ? p.k_write : p.v_write;
                    if (wr) *reinterpret_cast<uint2*>(wr + ((size_t)l * KV_HEADS + fg) * HEAD_DIM + lane * 4) = pk;
                    if (p.append) {
                        bf16_raw* cb = const_cast<bf16_raw*>(role == 2 ? kcache : vcache);
                        *reinterpret_cast<uint2*>(cb + (size_t)l * lstride + (size_t)len * KV_DIM + fg * HEAD_DIM + lane * 4) = pk;
                    }
                }
            }
            cta_sync();
            Q3_TRACE(ev + 3);

            if (local_attn) {
                // ---- local attention of head fh over all cached positions ----
                float qa[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) { qa[i] = q_s[fhh * 128 + sub * 8 + i]; qa[8 + i] = q_s[fhh * 128 + 64 + sub * 8 + i]; }
                float tmax = -INFINITY;
                auto score_pass = [&](const uint4& k0, const uint4& k1, int ps) {
                    const int pos = ps * 64 + att_slot;
                    float kf[16];
                    unpack8f(k0, kf); unpack8f(k1, kf + 8);
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) { s0 = fmaf(qa[i], kf[i], s0); s1 = fmaf(qa[8 + i], kf[8 + i], s1); }
                    s0 += s1;
                    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
                    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
                    s0 += __shfl_xor_sync(0xffffffffu, s0, 4);
                    if (pos < len) { tmax = fmaxf(tmax, s0); if (sub == 0) sc[pos] = s0; }
                };
                score_pass(ring[0][0], ring[0][1], 0);
                score_pass(ring[1][0], ring[1][1], 1);   // all zero (and masked) when there is one pass
                if constexpr (XPASS > 0) {
#pragma unroll
                    for (int x = 0; x < XPASS; ++x)
                        if (npl > 2 + x) score_pass(ring3[x][0], ring3[x][1], 2 + x);
                }
                if (warp == 12) {   // the new row's score: q . k_new in fp32, unrounded
                    const float4 a = *reinterpret_cast<const float4*>(q_s + fhh * 128 + lane * 4);
                    const float4 b = *reinterpret_cast<const float4*>(k_s + lane * 4);
                    const float sn_ = warp_sum(a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w);
                    if (lane == 0) misc[0] = sn_;
                    tmax = fmaxf(tmax, sn_);
                }
                tmax = warp_max(tmax);
                if (lane == 0) red[warp] = tmax;
                cta_sync();
                float M = (lane < CW) ? red[lane] : -INFINITY;
                M = warp_max(M);

                // P.V with a warp per position and four dims per lane: every lane of the warp forms the same
                // probability from the shared score, so nothing crosses lanes
                float lsum = 0.f, acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int i = 0; i < LOCAL_V_PRE; ++i) {
                    const int pos = warp + CW * i;
                    const float pr = (pos < len) ? __expf(sc[min(pos, 3 * SC_HALF - 1)] - M) : 0.f;   // the rows past the cache were fetched as zeros
                    lsum += pr;
                    const uint4& src = ring[2 + (i >> 2)][(i >> 1) & 1];
                    const uint32_t vx = (i & 1) ? src.z : src.x, vy = (i & 1) ? src.w : src.y;
                    acc[i & 1][0] = fmaf(pr, bf_lo(vx), acc[i & 1][0]); acc[i & 1][1] = fmaf(pr, bf_hi(vx), acc[i & 1][1]);
                    acc[i & 1][2] = fmaf(pr, bf_lo(vy), acc[i & 1][2]); acc[i & 1][3] = fmaf(pr, bf_hi(vy), acc[i & 1][3]);
                }
                if constexpr (XPASS > 0) {
#pragma unroll
                    for (int i = 0; i < 4 * XPASS; ++i) {
                        const int pos = warp + CW * (LOCAL_V_PRE + i);
                        const float pr = (pos < len) ? __expf(sc[min(pos, 3 * SC_HALF - 1)] - M) : 0.f;
                        lsum += pr;
                        const uint4& src = vext[i >> 1];
                        const uint32_t vx = (i & 1) ? src.z : src.x, vy = (i & 1) ? src.w : src.y;
                        acc[i & 1][0] = fmaf(pr, bf_lo(vx), acc[i & 1][0]); acc[i & 1][1] = fmaf(pr, bf_hi(vx), acc[i & 1][1]);
                        acc[i & 1][2] = fmaf(pr, bf_lo(vy), acc[i & 1][2]); acc[i & 1][3] = fmaf(pr, bf_hi(vy), acc[i & 1][3]);
                    }
                }
                *reinterpret_cast<float4*>(om + warp * 128 + lane * 4) =
                    make_float4(acc[0][0] + acc[1][0], acc[0][1] + acc[1][1], acc[0][2] + acc[1][2], acc[0][3] + acc[1][3]);
                if (lane == 0) lw[warp] = lsum;
                cta_sync();
                Q3_TRACE(ev + 4);
                Q3_TRACE(ev + 5);
                if (tid < HEAD_DIM) {
                    const float pn = __expf(misc[0] - M);
                    float Ls = pn, o = pn * v_s[tid];
#pragma unroll
                    for (int w = 0; w < CW; ++w) { Ls += lw[w]; o += om[w * 128 + tid]; }
                    bf16_raw h, m, lo_;
                    split3(o / Ls, h, m, lo_);
                    reinterpret_cast<bf16_raw*>(osp)[tid] = h;
                    reinterpret_cast<bf16_raw*>(osp + 64)[tid] = m;
                    reinterpret_cast<bf16_raw*>(osp + 128)[tid] = lo_;
                }
                cta_sync();
            } else {
            // ---- scores of this CTA's cached positions, both heads: a quarter-warp per position ----
                float tmax0 = -INFINITY, tmax1 = -INFINITY;
                if (warp < ATT_WARPS) {
                    float qa[2][16];
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int i = 0; i < 8; ++i) { qa[hh][i] = q_s[hh * 128 + sub * 8 + i]; qa[hh][8 + i] = q_s[hh * 128 + 64 + sub * 8 + i]; }
                    for (int ps = 0; ps < npass; ++ps) {
                        const int idx = ps * 32 + att_slot, pos = cp0 + idx;
                        uint4 k0 = make_uint4(0, 0, 0, 0), k1 = k0;
                        if (ps == 0) { k0 = ring[0][0]; k1 = ring[0][1]; }
                        else if (ps == 1) { k0 = ring[1][0]; k1 = ring[1][1]; }
                        else if (pos < cp1) {
                            const uint4* kr = reinterpret_cast<const uint4*>(kl + (size_t)pos * KV_DIM);
                            k0 = ld_stream(kr + sub); k1 = ld_stream(kr + 8 + sub);
                        }
                        float kf[16];
                        unpack8f(k0, kf); unpack8f(k1, kf + 8);
                        float s0 = 0.f, s1 = 0.f;
#pragma unroll
                        for (int i = 0; i < 16; ++i) { s0 = fmaf(qa[0][i], kf[i], s0); s1 = fmaf(qa[1][i], kf[i], s1); }
#pragma unroll
                        for (int o = 1; o <= 4; o <<= 1) {
                            s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                            s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                        }
                        if (pos < cp1) {
                            tmax0 = fmaxf(tmax0, s0); tmax1 = fmaxf(tmax1, s1);
                            if (sub == 0) { sc[idx] = s0; sc[SPLIT_SC + idx] = s1; }
                        }
                    }
                    tmax0 = warp_max(tmax0); tmax1 = warp_max(tmax1);
                    if (lane == 0) { red[warp] = tmax0; red[8 + warp] = tmax1; }
                } else if (warp == 12) {   // the new row's score for this CTA's own head: q . k_new in fp32, unrounded
                    const float4 a = *reinterpret_cast<const float4*>(q_s + fhh * 128 + lane * 4);
                    const float4 b = *reinterpret_cast<const float4*>(k_s + lane * 4);
                    const float sn_ = warp_sum(a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w);
                    if (lane == 0) misc[0] = sn_;
                }
                cta_sync();
                float M0 = (lane < ATT_WARPS) ? red[lane] : -INFINITY, M1 = (lane < ATT_WARPS) ? red[8 + lane] : -INFINITY;
                M0 = warp_max(M0); M1 = warp_max(M1);

                // ---- probabilities and P.V against the CTA-wide maxima: the partial sums just add.  A warp per position
                //      and four dims per lane: every lane forms the same two probabilities, nothing crosses lanes ----
                if (warp < ATT_WARPS) {
                    float l0 = 0.f, l1 = 0.f, acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int idx = warp + ATT_WARPS * i;
                        const bool live = cp0 + idx < cp1;
                        const float p0 = live ? __expf(sc[idx] - M0) : 0.f, p1 = live ? __expf(sc[SPLIT_SC + idx] - M1) : 0.f;
                        l0 += p0; l1 += p1;
                        const uint4& src = ring[2 + (i >> 2)][(i >> 1) & 1];
                        const uint32_t vx = (i & 1) ? src.z : src.x, vy = (i & 1) ? src.w : src.y;
                        const float f0 = bf_lo(vx), f1 = bf_hi(vx), f2 = bf_lo(vy), f3 = bf_hi(vy);
                        acc[0][0] = fmaf(p0, f0, acc[0][0]); acc[0][1] = fmaf(p0, f1, acc[0][1]); acc[0][2] = fmaf(p0, f2, acc[0][2]); acc[0][3] = fmaf(p0, f3, acc[0][3]);
                        acc[1][0] = fmaf(p1, f0, acc[1][0]); acc[1][1] = fmaf(p1, f1, acc[1][1]); acc[1][2] = fmaf(p1, f2, acc[1][2]); acc[1][3] = fmaf(p1, f3, acc[1][3]);
                    }
#pragma unroll 2
                    for (int idx = warp + ATT_WARPS * 8; cp0 + idx < cp1; idx += ATT_WARPS) {
                        const uint2 v = ld_stream8(vl + (size_t)(cp0 + idx) * KV_DIM + lane * 4);
                        const float p0 = __expf(sc[idx] - M0), p1 = __expf(sc[SPLIT_SC + idx] - M1);
                        l0 += p0; l1 += p1;
                        const float f0 = bf_lo(v.x), f1 = bf_hi(v.x), f2 = bf_lo(v.y), f3 = bf_hi(v.y);
                        acc[0][0] = fmaf(p0, f0, acc[0][0]); acc[0][1] = fmaf(p0, f1, acc[0][1]); acc[0][2] = fmaf(p0, f2, acc[0][2]); acc[0][3] = fmaf(p0, f3, acc[0][3]);
                        acc[1][0] = fmaf(p1, f0, acc[1][0]); acc[1][1] = fmaf(p1, f1, acc[1][1]); acc[1][2] = fmaf(p1, f2, acc[1][2]); acc[1][3] = fmaf(p1, f3, acc[1][3]);
                    }
                    *reinterpret_cast<float4*>(om + (warp * 2) * 128 + lane * 4) = make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]);
                    *reinterpret_cast<float4*>(om + (warp * 2 + 1) * 128 + lane * 4) = make_float4(acc[1][0], acc[1][1], acc[1][2], acc[1][3]);
                    if (lane == 0) { lw[warp * 2] = l0; lw[warp * 2 + 1] = l1; }
                }
                cta_sync();
                // ---- publish the CTA's partial of both heads: (max, sum, unnormalised output), every word tagged ----
                if (tid < 256) {
                    const int hh = tid >> 7, d = tid & 127;
                    float o = 0.f, Ls = 0.f;
#pragma unroll
                    for (int w = 0; w < ATT_WARPS; ++w) { o += om[(w * 2 + hh) * 128 + d]; Ls += lw[w * 2 + hh]; }
                    const unsigned long long t64 = (unsigned long long)tag << 32;
                    unsigned long long* dst = p.xp + (size_t)((fg * 2 + hh) * GROUP_CTAS + fj) * XP_STRIDE;
                    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(dst + 4 + d), "l"(t64 | __float_as_uint(o)) : "memory");
                    __syncwarp();
                    if (d == 127) {   // the (max, sum) pair goes last: it is what the readers poll
                        asm volatile("st.relaxed.gpu.global.v2.b64 [%0], {%1, %2};" ::"l"(dst), "l"(t64 | __float_as_uint(hh ? M1 : M0)), "l"(t64 | __float_as_uint(Ls)) : "memory");
                    }
                }
                Q3_TRACE(ev + 4);

                // ---- merge the 18 partials of this CTA's head with the new row.  Step 1: one warp polls the 18
                //      (max, sum) pairs, which their writers store last, so that the polling stays light; step 2:
                //      eight warps read the outputs, half h = tid / 128 merging partials [9 h, 9 h + 9) for dim
                //      tid % 128, and go round again in the rare case that a word does not carry the tag yet.
                constexpr int HALF = GROUP_CTAS / 2;
                const unsigned long long* xsrc = p.xp + (size_t)((fg * 2 + fhh) * GROUP_CTAS) * XP_STRIDE;
                float* pm_s = misc + 8;          // [18] maxima   (misc[8..25] runs into sc, which is dead by now)
                float* pl_s = sc + 32;           // [18] sums
                unsigned long long wc[HALF];   // warps 0..7: this thread's nine output words
                const int mhalf = tid >> 7, md = tid & 127;
                const unsigned long long* msrc = xsrc + (size_t)(mhalf * HALF) * XP_STRIDE + 4 + md;
                auto load_outputs = [&]() {
#pragma unroll
                    for (int j = 0; j < HALF; ++j)
                        asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(wc[j]) : "l"(msrc + (size_t)j * XP_STRIDE) : "memory");
                };
                if (warp < 8) load_outputs();   // speculative: usually fresh by the time the pairs are, which saves a round trip
                if (warp == 8) {
                    unsigned long long wa = (unsigned long long)tag << 32, wb = wa;
                    unsigned it = 0;
                    unsigned long long t0 = 0;
                    for (;;) {
                        if (lane < GROUP_CTAS)
                            asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(wa), "=l"(wb) : "l"(xsrc + (size_t)lane * XP_STRIDE) : "memory");
                        const bool fresh = (unsigned)(wa >> 32) == tag && (unsigned)(wb >> 32) == tag;
                        if (__all_sync(0xffffffffu, fresh)) break;
                        if (*abort_flag) break;
                        if ((++it & 255u) == 0) {
                            const unsigned long long t = global_ns();
                            if (t0 == 0) t0 = t;
                            else if (t - t0 > wait_ns) {
                                if (lane == 0) { report(p.status, ST_BARRIER_TIMEOUT, 400 + l, 0); *abort_flag = 1; }
                                break;
                            }
                        }
                    }
                    if (lane < GROUP_CTAS) { pm_s[lane] = __uint_as_float((unsigned)wa); pl_s[lane] = __uint_as_float((unsigned)wb); }
                }
                cta_sync();
                if (tid < 2 * HEAD_DIM) {
                    const int half = mhalf, d = md;
                    float M, Ls, o;
                    unsigned it = 0;
                    unsigned long long t0 = 0;
                    for (;;) {
                        bool fresh = true;
                        M = -INFINITY; Ls = 0.f; o = 0.f;
#pragma unroll
                        for (int j = 0; j < HALF; ++j) {
                            fresh = fresh && (unsigned)(wc[j] >> 32) == tag;
                            const float mj = pm_s[half * HALF + j];   // -inf for a CTA that had no positions
                            const float Mn = fmaxf(M, mj);
                            const float keep = (M == -INFINITY) ? 0.f : __expf(M - Mn), wgt = (mj == -INFINITY) ? 0.f : __expf(mj - Mn);
                            Ls = fmaf(pl_s[half * HALF + j], wgt, Ls * keep);
                            o = fmaf(__uint_as_float((unsigned)wc[j]), wgt, o * keep);
                            M = Mn;
                        }
                        if (__all_sync(0xffffffffu, fresh)) break;
                        if (*abort_flag) break;
                        if ((++it & 63u) == 0) {
                            const unsigned long long t = global_ns();
                            if (t0 == 0) t0 = t;
                            else if (t - t0 > wait_ns) {
                                if (lane == 0) { report(p.status, ST_BARRIER_TIMEOUT, 450 + l, 0); *abort_flag = 1; }
                                break;
                            }
                        }
                        load_outputs();
                    }
                    q_s[half * 128 + d] = o;                       // the queries are dead by now
                    if (d == 0) { misc[4 + 2 * half] = M; misc[5 + 2 * half] = Ls; }
                }
                cta_sync();
                if (tid < HEAD_DIM) {
                    const float s_new = misc[0], m0 = misc[4], m1 = misc[6];
                    const float M = fmaxf(s_new, fmaxf(m0, m1));
                    const float pn = __expf(s_new - M);
                    const float w0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - M), w1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - M);
                    const float Ls = pn + misc[5] * w0 + misc[7] * w1;
                    const float o = pn * v_s[tid] + q_s[tid] * w0 + q_s[128 + tid] * w1;
                    bf16_raw h, m, lo_;
                    split3(o / Ls, h, m, lo_);
                    reinterpret_cast<bf16_raw*>(osp)[tid] = h;
                    reinterpret_cast<bf16_raw*>(osp + 64)[tid] = m;
                    reinterpret_cast<bf16_raw*>(osp + 128)[tid] = lo_;
                }
                Q3_TRACE(ev + 5);
                cta_sync();

            }

            // ---- Wo slice on the tensor cores: warp (rt, kh) = 16 rows x 64 head dims ----
            slot_wait(&full[1], l & 1, abort_flag, p.status, 11, wait_ns);
            {
                const int rt = warp >> 1, kh = warp & 1;
                float cc[4] = {0.f, 0.f, 0.f, 0.f};
                const uint32_t abase = smem_u32(sB + (size_t)(16 * rt + lm_row) * WOROW + 64 * kh + lm_k);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int kp = (64 * kh + 16 * t + fr_k) >> 1;
                    const uint32_t b0 = (fr_n < 3) ? osp[fr_n * 64 + kp] : 0u;
                    const uint32_t b1 = (fr_n < 3) ? osp[fr_n * 64 + kp + 4] : 0u;
                    uint32_t af[4];
                    ldsm_x4(af, abase + 32 * t);
                    mma_bf16(cc, af, b0, b1);
                }
                float r0, r1;
                fold_cols(cc, r0, r1);
                if ((lane & 3) == 0) { wo_part[kh * 128 + 16 * rt + fr_n] = r0; wo_part[kh * 128 + 16 * rt + fr_n + 8] = r1; }
            }
            cta_sync();
            if (tid < fn) {   // fn <= 116: the slice joins the attention delta (of every rank)
                const unsigned long long w = acc_word(wo_part[tid] + wo_part[128 + tid]);
                if (TP) { for (int r = 0; r < T; ++r) acc_add<true>(p.tp_dA[r] + (size_t)(l & 1) * HIDDEN + fr0 + tid, w); }
                else acc_add<false>(dAl + fr0 + tid, w);
            }
        }   // (wo_part is the next phase's staging area: the wait below passes a CTA barrier before anything is staged)
        Q3_TRACE(ev + 6);
        gain2 = *reinterpret_cast<const uint32_t*>(p.ln2 + (size_t)l * HIDDEN + 2 * tid);

        // ==================================================================== GD
        {
            acc_wait(dAl, (unsigned)Q_HEADS, 200 + l);   // every row of the attention delta receives one slice per query head
            Q3_TRACE(ev + 7);
            fetch_slot(0, l + 1);   // q/k/v rows and Wo slice of the next layer: landed before this phase's barrier is polled
            fetch_slot(1, l + 1);
            if (c == G - 1) {   // recycle the delta buffers (see the top of the loop): 8 KB each, 16 bytes a thread
                static_assert(N_ACC == 2, "both buffers are cleared as 8 KB");
                __stcg(reinterpret_cast<float4*>(p.dA + (size_t)((l + 1) & 1) * HIDDEN) + tid, make_float4(0.f, 0.f, 0.f, 0.f));
                __stcg(reinterpret_cast<float4*>(p.dB + (size_t)((l + 1) % 3) * N_ACC * HIDDEN) + tid, make_float4(0.f, 0.f, 0.f, 0.f));
            }
            {
                bf16_raw h0, m0, l0, h1, m1, l1;
                split3(x0 * bf_lo(gain2), h0, m0, l0);
                split3(x1 * bf_hi(gain2), h1, m1, l1);
                xsp[tid] = (uint32_t)h0 | ((uint32_t)h1 << 16);
                xsp[512 + tid] = (uint32_t)m0 | ((uint32_t)m1 << 16);
                xsp[1024 + tid] = (uint32_t)l0 | ((uint32_t)l1 << 16);
            }
            const float ss = warp_sum(x0 * x0 + x1 * x1);
            if (lane == 0) red[warp] = ss;
            cta_sync();
            Q3_TRACE(ev + 8);
            {
                // The slot holds one matrix of 2 * imax = 42 rows (gate rows, then up rows): three 16-row tiles cover it
                // (the last six rows of the third tile belong to the next slot and are never used).  Warp w takes
                // the k range [64 w, 64 w + 64) of all three tiles.
                uint32_t bx[4][2];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int kp = (64 * warp + 16 * t + fr_k) >> 1;
                    bx[t][0] = (fr_n < 3) ? xsp[fr_n * 512 + kp] : 0u;
                    bx[t][1] = (fr_n < 3) ? xsp[fr_n * 512 + kp + 4] : 0u;
                }
                slot_wait(&full[2], l & 1, abort_flag, p.status, 12, wait_ns);
                uint32_t af[3][4][4];
#pragma unroll
                for (int rt = 0; rt < 3; ++rt) {
                    const uint32_t abase = smem_u32(sC + (size_t)(16 * rt + lm_row) * WROW + 64 * warp + lm_k);
#pragma unroll
                    for (int t = 0; t < 4; ++t) ldsm_x4(af[rt][t], abase + 32 * t);
                }
                float cg[3][2][4];
#pragma unroll
                for (int rt = 0; rt < 3; ++rt)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < 4; ++i) cg[rt][h][i] = 0.f;
#pragma unroll
                for (int t = 0; t < 4; ++t)
#pragma unroll
                    for (int rt = 0; rt < 3; ++rt) mma_bf16(cg[rt][t & 1], af[rt][t], bx[t][0], bx[t][1]);
#pragma unroll
                for (int rt = 0; rt < 3; ++rt) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) cg[rt][0][i] += cg[rt][1][i];
                    float r0, r1;
                    fold_cols(cg[rt][0], r0, r1);
                    if ((lane & 3) == 0) { gpart[warp * 48 + 16 * rt + fr_n] = r0; gpart[warp * 48 + 16 * rt + fr_n + 8] = r1; }
                }
                cta_sync();
                if (tid < 32) {   // hid of this CTA's rows, split for the down projection; rows past the share are zero
                    float hv = 0.f;
                    if (tid < ni) {
                        const float r = rsqrtf(sum16(red) / (float)HIDDEN + EPS);
                        float g = 0.f, u = 0.f;
#pragma unroll
                        for (int w = 0; w < CW; ++w) { g += gpart[w * 48 + tid]; u += gpart[w * 48 + imax + tid]; }
                        g *= r; u *= r;
                        hv = (g / (1.f + expf(-g))) * u;
                    }
                    bf16_raw h, m, lo_;
                    split3(hv, h, m, lo_);
                    reinterpret_cast<bf16_raw*>(hsp)[tid] = h;
                    reinterpret_cast<bf16_raw*>(hsp + 16)[tid] = m;
                    reinterpret_cast<bf16_raw*>(hsp + 32)[tid] = lo_;
                }
            }
            cta_sync();   // hid ready; the activations and the gate/up slot are no longer needed
            Q3_TRACE(ev + 9);

            slot_wait(&full[3], l & 1, abort_flag, p.status, 13, wait_ns);
            {   // out[n] = sum_i wdT[i][n] * hid[i]: A = transposed tiles of the slot, k = this CTA's (<= 32) rows
                uint32_t bh[2][2];
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const int kp = (16 * t + fr_k) >> 1;
                    bh[t][0] = (fr_n < 3) ? hsp[fr_n * 16 + kp] : 0u;
                    bh[t][1] = (fr_n < 3) ? hsp[fr_n * 16 + kp + 4] : 0u;
                }
                // transposed ldmatrix: lanes 0-7 / 8-15 / 16-23 / 24-31 address rows i of the blocks (n 0-7, i 0-7), (n 8-15, i 0-7), (n 0-7, i 8-15), (n 8-15, i 8-15)
                const int ti = (lane & 7) + ((lane >> 4) & 1) * 8, tn = ((lane >> 3) & 1) * 8;
                uint32_t af[4][2][4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        int i = 16 * t + ti;
                        if (i >= ni) i = 0;   // hid is zero there; any finite row will do
                        ldsm_x4_trans(af[nt][t], smem_u32(sD + (size_t)i * WROW + 64 * warp + 16 * nt + tn));
                    }
                float cc[4][4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) cc[nt][i] = 0.f;
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) mma_bf16(cc[nt], af[nt][t], bh[t][0], bh[t][1]);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int n0 = 64 * warp + 16 * nt;
                    float r0, r1;
                    fold_cols(cc[nt], r0, r1);
                    if ((lane & 3) == 0) { dout[n0 + fr_n] = r0; dout[n0 + fr_n + 8] = r1; }
                }
            }
            cta_sync();
            if (tid < 256) {
                const float4 t = *reinterpret_cast<const float4*>(dout + tid * 4);
                const size_t off = (size_t)(l % 3) * N_ACC * HIDDEN + (size_t)(c & (N_ACC - 1)) * HIDDEN + tid * 4;
                if (TP) { for (int r = 0; r < T; ++r) red_add_v4<true>(p.tp_dB[r] + off, t.x, t.y, t.z, t.w); }
                else red_add_v4<false>(p.dB + off, t.x, t.y, t.z, t.w);
            }
            cta_sync();
            Q3_TRACE(ev + 10);
            if (tid == 0) {
                if (TP) counter_arrive_all(p.tp_bar, T);
                else counter_arrive(bar);
            }
        }
        target += (unsigned)(T * G);
        gain2 = (l + 1 < L) ? *reinterpret_cast<const uint32_t*>(p.ln1 + (size_t)(l + 1) * HIDDEN + 2 * tid)
                            : *reinterpret_cast<const uint32_t*>(p.fnorm + 2 * tid);
        counter_wait<TP>(bar, target, abort_flag, p.status, 300 + l, wait_ns);
        Q3_TRACE(ev + 11);
    }

    // ======================================================================== LM head + argmax
    {
        add_ffn_delta(p.dB + (size_t)((L - 1) % 3) * N_ACC * HIDDEN);
        const float ss = warp_sum(x0 * x0 + x1 * x1);
        if (lane == 0) red[warp] = ss;
        cta_sync();
        float tot = (lane < CW) ? red[lane] : 0.f;
        tot = warp_sum(tot);
        const float r = rsqrtf(tot / (float)HIDDEN + EPS);
        xs[act_slot(2 * tid)] = (x0 * r) * bf_lo(gain2);
        xs[act_slot(2 * tid + 1)] = (x1 * r) * bf_hi(gain2);
        cta_sync();

        float bestv = -INFINITY;
        int besti = 0x7fffffff;
        lm_stream(warp, CW, bestv, besti);
        Q3_TRACE(1 + EV_PER_LAYER * L);
        // CTA argmax (ties -> lowest index), then the last CTA to finish reduces over CTAs
        float* bv_s = lm_bv;
        int* bi_s = lm_bi;
        if (lane == 0) { bv_s[warp] = bestv; bi_s[warp] = besti; }
        cta_sync();
        int* last_flag = reinterpret_cast<int*>(v_s);
        if (tid == 0) {
            float bv = bv_s[0];
            int bi = bi_s[0];
            for (int w = 1; w < CW; ++w)
                if (bv_s[w] > bv || (bv_s[w] == bv && bi_s[w] < bi)) { bv = bv_s[w]; bi = bi_s[w]; }
            __stcg(p.pval + c, bv);
            __stcg(p.pidx + c, bi);
            __threadfence();
            const unsigned prev = atomicAdd(p.sync + 2, 1u);
            *last_flag = (prev == (unsigned)G - 1u);
            __threadfence();
        }
        cta_sync();
        if (*last_flag) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int i = tid; i < G; i += CT) {
                const float v = __ldcg(p.pval + i);
                const int ix = __ldcg(p.pidx + i);
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            cta_sync();
            if (lane == 0) { bv_s[warp] = bv; bi_s[warp] = bi; }
            cta_sync();
            // every CTA has read its last delta: the next launch starts from clean accumulators (dA and dB are adjacent)
            for (int i = tid; i < (int)(ACC_FLOATS / 4); i += CT) __stcg(reinterpret_cast<float4*>(p.dA) + i, make_float4(0.f, 0.f, 0.f, 0.f));
            cta_sync();
            if (tid == 0) {
                for (int w = 1; w < CW; ++w)
                    if (bv_s[w] > bv || (bv_s[w] == bv && bi_s[w] < bi)) { bv = bv_s[w]; bi = bi_s[w]; }
                if (TP) {
                    // This rank's best word goes to every rank's mailbox; the best of all ranks is the token.  The mail is
                    // also the hand-over to the next launch: a peer that holds it may start adding to this rank's deltas
                    // and arriving at its barrier, so the accumulators are clean and the counter is rearmed before it leaves.
                    *bar = 0u;
                    asm volatile("fence.acq_rel.sys;" ::: "memory");
                    const unsigned long long mtag = (unsigned long long)(tag_base / 64u + 1u) << 32;
                    for (int r = 0; r < T; ++r)
                        asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p.tp_mail[r] + 2 * rank),
                                     "l"(mtag | __float_as_uint(bv)), "l"(mtag | (unsigned)bi) : "memory");
                    for (int r = 0; r < T && !*abort_flag; ++r) {
                        unsigned long long m0, m1;
                        unsigned it = 0;
                        unsigned long long t0 = 0;
                        for (;;) {
                            asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(m0), "=l"(m1) : "l"(p.tp_mail[rank] + 2 * r) : "memory");
                            if ((m0 >> 32) == (mtag >> 32) && (m1 >> 32) == (mtag >> 32)) break;
                            if ((++it & 63u) == 0) {
                                const unsigned long long t = global_ns();
                                if (t0 == 0) t0 = t;
                                else if (t - t0 > wait_ns) { report(p.status, ST_PEER_TIMEOUT, 500 + r, (uint32_t)(m0 >> 32)); *abort_flag = 1; break; }
                            }
                        }
                        if (*abort_flag) break;
                        const float ov = __uint_as_float((unsigned)m0);
                        const int oi = (int)(unsigned)m1;
                        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                    }
                } else {
                    p.sync[0] = 0;   // every CTA has passed every barrier: rearm the counter for the next launch
                }
                p.next_token[0] = bi;
                if (p.append) p.seq_len[0] = len + 1;
                p.sync[2] = 0;
                *const_cast<unsigned*>(p.epoch) = tag_base / 64u + 1u;
            }
        }
        Q3_TRACE(2 + EV_PER_LAYER * L);
    }
    // The issuing thread makes sure (bounded) that every slot it armed has landed before the CTA gives its
    // shared memory back; after a clean step these four tests succeed at once.
    if (pumper) {
        for (int slot = 0; slot < 4; ++slot)
            if (pump_armed & (1 << slot)) mbar_wait(&full[slot], (uint32_t)((pump_parity >> slot) & 1), abort_flag, p.status, 30 + slot, wait_ns);
    }
#undef Q3_TRACE
}


// ---- weight packing ----------------------------------------------------------------------------------
// packed[l][c] = everything CTA c streams for layer l, in the order and with the row padding of its
// shared-memory slots: its rows of [wq; wk; wv], its Wo slice (the 128 columns of its head), its
// gate and up rows, and its rows of the transposed down matrix.  Rows beyond a share are zero.
struct PackArgs {
    const bf16_raw *wq, *wk, *wv, *wo, *wg, *wu, *wd;
    bf16_raw* packed;
    int tp_size, tp_rank;   // the rank's share of the heads and FFN rows is what gets packed
};
__global__ void __launch_bounds__(256) pack_weights_kernel(const PackArgs a) {
    const int c = blockIdx.x, G = gridDim.x, l = blockIdx.y;
    const int T = a.tp_size, rank = a.tp_rank;
    const Share sh = share_of(c, G, T, rank);
    const int qrows = Q_DIM / T, kvrows = KV_DIM / T;
    bf16_raw* dst = a.packed + ((size_t)l * G + c) * share_elems(G, T);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // A: 129 16-byte units per row (128 of data, 1 of padding)
    for (int u = threadIdx.x; u < sh.qmax * 129; u += 256) {
        const int j = u / 129, k = u % 129;
        uint4 v = zero;
        if (j < sh.nq && k < 128) {
            const int r = sh.q0 + j;   // row of this rank's [q rows; k rows; v rows]
            const bf16_raw* src = r < qrows ? a.wq + ((size_t)l * Q_DIM + rank * qrows + r) * HIDDEN
                                : r < qrows + kvrows ? a.wk + ((size_t)l * KV_DIM + rank * kvrows + (r - qrows)) * HIDDEN
                                                     : a.wv + ((size_t)l * KV_DIM + rank * kvrows + (r - qrows - kvrows)) * HIDDEN;
            v = reinterpret_cast<const uint4*>(src)[k];
        }
        reinterpret_cast<uint4*>(dst)[u] = v;
    }
    dst += (size_t)sh.qmax * WROW;
    // B: 17 units per row
    for (int u = threadIdx.x; u < WO_ROWS_MAX * 17; u += 256) {
        const int j = u / 17, k = u % 17;
        uint4 v = zero;
        if (sh.has_f && j < sh.fn && k < 16)
            v = reinterpret_cast<const uint4*>(a.wo + ((size_t)l * HIDDEN + sh.fr0 + j) * Q_DIM + sh.fh * HEAD_DIM)[k];
        reinterpret_cast<uint4*>(dst)[u] = v;
    }
    dst += (size_t)WO_ROWS_MAX * WOROW;
    // C: gate rows, then up rows
    for (int u = threadIdx.x; u < 2 * sh.imax * 129; u += 256) {
        const int jj = u / 129, k = u % 129;
        const bool up = jj >= sh.imax;
        const int j = up ? jj - sh.imax : jj;
        uint4 v = zero;
        if (j < sh.ni && k < 128) v = reinterpret_cast<const uint4*>((up ? a.wu : a.wg) + ((size_t)l * INTER + sh.i0 + j) * HIDDEN)[k];
        reinterpret_cast<uint4*>(dst)[u] = v;
    }
    dst += (size_t)2 * sh.imax * WROW;
    // D: row j holds wd[l][n][i0 + j] for n = 0..1023 (the down matrix transposed)
    for (int e = threadIdx.x; e < sh.imax * WROW; e += 256) {
        const int j = e / WROW, n = e % WROW;
        bf16_raw v = 0;
        if (j < sh.ni && n < HIDDEN) v = a.wd[((size_t)l * HIDDEN + n) * INTER + sh.i0 + j];
        dst[e] = v;
    }
}

// ====================================================================================================
// host side
// ====================================================================================================
static int smem_bytes_for(int grid) {
    const int qmax = (QKV_DIM + grid - 1) / grid, imax = (INTER + grid - 1) / grid;
    return (qmax + 3 * imax) * WROW * 2 + WO_ROWS_MAX * WOROW * 2 + TAIL_BYTES;
}

static const void* persist_kernel(int mode, bool tp = false) {
    if (tp) {
        switch (mode) {
            case 0: return reinterpret_cast<const void*>(q3_persist_decode<0, true>);
            case 1: return reinterpret_cast<const void*>(q3_persist_decode<1, true>);
            default: return reinterpret_cast<const void*>(q3_persist_decode<2, true>);
        }
    }
    switch (mode) {
        case 0: return reinterpret_cast<const void*>(q3_persist_decode<0, false>);
        case 1: return reinterpret_cast<const void*>(q3_persist_decode<1, false>);
        case 2: return reinterpret_cast<const void*>(q3_persist_decode<2, false>);
        default: return reinterpret_cast<const void*>(q3_persist_decode<3, false>);
    }
}

int persist_setup(q3_engine* e) {
    e->p_grid = 0; e->p_threads = PT; e->p_smem = 0; e->p_state = nullptr;
    int grid = e->sm_count;
    if (e->cfg.grid_limit > 0 && e->cfg.grid_limit < grid) grid = e->cfg.grid_limit;
    // too few CTAs for the slot sizes, too many for the accumulators' count field, or more layers than a launch has
    // tags for: the layered path serves everything
    if (grid < MIN_GRID || grid > MAX_GRID || e->cfg.n_layers > MAX_LAYERS) return Q3_OK;
    static_assert(2 * ((INTER + MIN_GRID - 1) / MIN_GRID) <= 48, "the gate/up rows of a CTA must fit three 16-row tiles");
    const int smem = smem_bytes_for(grid);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, e->device) != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "cudaGetDeviceProperties failed");
    if ((size_t)smem > prop.sharedMemPerBlockOptin) return Q3_OK;
    for (int variant = 0; variant < 2 * N_MODES - 1; ++variant) {   // the four attention variants, then the three tensor-parallel ones
        const void* fn = variant < N_MODES ? persist_kernel(variant) : persist_kernel(variant - N_MODES, true);
        cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "persist: set smem attribute (%d B): %s", smem, cudaGetErrorString(err));
        int per_sm = 0;
        err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, PT, smem);
        if (err != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "persist: occupancy query: %s", cudaGetErrorString(err));
        if (per_sm < 1 || per_sm * e->sm_count < grid || !prop.cooperativeLaunch)
            return engine_fail(e, Q3_ERR_NOT_RESIDENT, "persist: %d CTAs of %d threads and %d B shared memory cannot be co-resident", grid, PT, smem);
    }
    PersistState* s = new PersistState();
    s->packed = nullptr; s->X = nullptr; s->grid = grid; s->smem = smem;
    s->tp_rank = 0; s->tp_size = 1;
    for (int i = 0; i < MAX_TP; ++i) s->peer_X[i] = nullptr;
    for (int i = 0; i < 7; ++i) s->src[i] = nullptr;
    if (cudaMalloc(&s->X, X_FLOATS * sizeof(float)) != cudaSuccess ||
        cudaMemset(s->X, 0, X_FLOATS * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&s->packed, (size_t)e->cfg.n_layers * grid * share_elems(grid) * sizeof(bf16_raw)) != cudaSuccess) {
        if (s->X) cudaFree(s->X);
        delete s;
        return engine_fail(e, Q3_ERR_CUDA, "persist: scratch allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    e->p_state = s;
    e->p_grid = grid; e->p_smem = smem;
    return Q3_OK;
}

void persist_teardown(q3_engine* e) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    if (!s) return;
    for (int r = 0; r < MAX_TP; ++r)
        if (s->peer_X[r] && s->peer_X[r] != s->X) cudaIpcCloseMemHandle(s->peer_X[r]);
    if (s->packed) cudaFree(s->packed);
    if (s->X) cudaFree(s->X);
    delete s;
    e->p_state = nullptr;
}

// Batches of up to PERSIST_MAX_BATCH sequences are served as one launch per sequence (measured at 1024 cached
// positions: 2 sequences 2 x 0.47 ms against 1.60 ms on the layered path; from 4 sequences on the layered path's
// tensor-core projections win).
bool persist_supports(const q3_engine* e, const q3_decode_args* a) {
    const PersistState* s = static_cast<const PersistState*>(e->p_state);
    if (s == nullptr || a->batch < 1) return false;
    if (s->tp_size > 1) return a->batch == 1 && a->max_len <= mode_max_len(N_MODES - 2);   // one sequence, local attention
    return a->batch <= PERSIST_MAX_BATCH && a->max_len <= PERSIST_MAX_LEN;
}

// (Re)pack the layer matrices when one of the caller's pointers changes.  Runs on the legacy default
// stream and synchronises: weights change rarely, and later launches may use any stream.  The pack
// is keyed on the pointers: a caller that rewrites weights in place must call q3_set_weights with
// `Q3_W_REPACK` semantics, i.e. after q3_invalidate_weights.
int persist_weights_changed(q3_engine* e) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    if (!s) return Q3_OK;
    const void* now[7] = {e->w.wq, e->w.wk, e->w.wv, e->w.wo, e->w.wg, e->w.wu, e->w.wd};
    bool same = true;
    for (int i = 0; i < 7; ++i) same = same && (s->src[i] == now[i]);
    if (same) return Q3_OK;
    auto bf = [](const void* p) { return reinterpret_cast<const bf16_raw*>(p); };
    PackArgs a{bf(now[0]), bf(now[1]), bf(now[2]), bf(now[3]), bf(now[4]), bf(now[5]), bf(now[6]), s->packed, s->tp_size, s->tp_rank};
    pack_weights_kernel<<<dim3(s->grid, e->cfg.n_layers), 256>>>(a);
    ++e->launches;
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "persist: packing the weights failed: %s", cudaGetErrorString(err));
    for (int i = 0; i < 7; ++i) s->src[i] = now[i];
    return Q3_OK;
}

// A step that gave up half-way leaves partial sums in the delta accumulators and stale tags behind: start over.
int persist_recover(q3_engine* e) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    if (!s) return Q3_OK;
    if (cudaMemset(s->X, 0, X_FLOATS * sizeof(float)) != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "persist: clearing the scratch state failed");
    return Q3_OK;
}

void* persist_accumulators(const q3_engine* e, int64_t* bytes) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    if (!s) return nullptr;
    *bytes = (int64_t)(ACC_FLOATS * sizeof(float));
    return s->X;
}

// ---- tensor parallelism: the ranks' state allocations are mapped into one another with CUDA IPC ----
int persist_tp_export(q3_engine* e, void* handle64) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    if (!s) return engine_fail(e, Q3_ERR_UNSUPPORTED, "tensor parallelism needs the persistent kernel, which this engine does not have");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI hands IPC handles over as 64 bytes");
    cudaIpcMemHandle_t h;
    const cudaError_t err = cudaIpcGetMemHandle(&h, s->X);
    if (err != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(err));
    memcpy(handle64, &h, 64);
    return Q3_OK;
}

int persist_tp_attach(q3_engine* e, int rank, int size, const void* handles) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    if (!s) return engine_fail(e, Q3_ERR_UNSUPPORTED, "tensor parallelism needs the persistent kernel, which this engine does not have");
    if (!(size == 1 || size == 2 || size == 4 || size == 8) || rank < 0 || rank >= size)
        return engine_fail(e, Q3_ERR_INVALID, "q3_tp_attach: rank %d of %d (sizes 1, 2, 4, 8)", rank, size);
    if (e->cfg.vocab % size) return engine_fail(e, Q3_ERR_INVALID, "q3_tp_attach: vocabulary %d does not divide over %d ranks", e->cfg.vocab, size);
    for (int r = 0; r < MAX_TP; ++r) {   // drop earlier mappings
        if (s->peer_X[r] && s->peer_X[r] != s->X) cudaIpcCloseMemHandle(s->peer_X[r]);
        s->peer_X[r] = nullptr;
    }
    s->tp_rank = 0; s->tp_size = 1;
    persist_invalidate_weights(e);       // the packed copy depends on the rank's share
    if (size == 1) return Q3_OK;
    if (!handles) return engine_fail(e, Q3_ERR_INVALID, "q3_tp_attach: handles are required");
    for (int r = 0; r < size; ++r) {
        if (r == rank) { s->peer_X[r] = s->X; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(handles) + 64 * r, 64);
        void* ptr = nullptr;
        const cudaError_t err = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (err != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "cudaIpcOpenMemHandle (rank %d): %s", r, cudaGetErrorString(err));
        s->peer_X[r] = static_cast<float*>(ptr);
    }
    s->tp_rank = rank; s->tp_size = size;
    if (cudaMemset(s->X, 0, X_FLOATS * sizeof(float)) != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "q3_tp_attach: clearing the state failed");
    return Q3_OK;
}

void persist_invalidate_weights(q3_engine* e) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    if (s) for (int i = 0; i < 7; ++i) s->src[i] = nullptr;
}

int persist_decode(q3_engine* e, const q3_decode_args* a, cudaStream_t st) {
    PersistState* s = static_cast<PersistState*>(e->p_state);
    auto bf = [](const void* p) { return reinterpret_cast<const bf16_raw*>(p); };
    PersistParams p{};
    const q3_weights& w = e->w;
    p.ln1 = bf(w.ln1); p.qn = bf(w.qn); p.kn = bf(w.kn); p.ln2 = bf(w.ln2); p.fnorm = bf(w.fnorm); p.embed = bf(w.embed);
    p.packed = s->packed;
    p.token = reinterpret_cast<const long long*>(a->token);
    p.seq_k = a->seq_k; p.seq_v = a->seq_v; p.seq_layer_stride = reinterpret_cast<const long long*>(a->seq_layer_stride);
    p.seq_len = a->seq_len; p.logits = a->logits; p.next_token = reinterpret_cast<long long*>(a->next_token);
    p.k_write = reinterpret_cast<bf16_raw*>(a->k_write); p.v_write = reinterpret_cast<bf16_raw*>(a->v_write);
    p.dA = reinterpret_cast<unsigned long long*>(s->X); p.dB = s->X + 4 * HIDDEN;
    p.xq = reinterpret_cast<unsigned long long*>(s->X + ACC_FLOATS);
    p.epoch = reinterpret_cast<const unsigned*>(s->X + ACC_FLOATS + 2 * QKV_DIM);
    p.xp = reinterpret_cast<unsigned long long*>(s->X + ACC_FLOATS + 2 * QKV_DIM + 64);
    p.wait_ns = e->cfg.wait_limit_us > 0 ? (unsigned long long)e->cfg.wait_limit_us * 1000ull : WAIT_NS;
    const bool tp = s->tp_size > 1;
    p.tp_rank = s->tp_rank; p.tp_size = s->tp_size;
    for (int r = 0; r < s->tp_size; ++r) {
        float* X = s->peer_X[r] ? s->peer_X[r] : s->X;
        p.tp_dA[r] = reinterpret_cast<unsigned long long*>(X);
        p.tp_dB[r] = X + 4 * HIDDEN;
        p.tp_bar[r] = reinterpret_cast<unsigned*>(X + TP_OFFSET);
        p.tp_mail[r] = reinterpret_cast<unsigned long long*>(X + TP_OFFSET + 64);
    }
    p.rope = e->rope; p.sync = e->sync; p.status = e->status; p.pval = e->pval; p.pidx = e->pidx;
    p.trace = (e->trace && e->trace_words >= (int64_t)s->grid * (4 + EV_PER_LAYER * e->cfg.n_layers)) ? e->trace : nullptr;
    p.n_layers = e->cfg.n_layers; p.vocab = e->cfg.vocab; p.append = (a->flags & Q3_F_APPEND_KV) ? 1 : 0;
    int mode = 0;
    while (mode + 1 < N_MODES && a->max_len > mode_max_len(mode)) ++mode;
    // A small batch is one launch per sequence, back to back on the stream: the kernel reads entry 0 of every
    // per-sequence array, so the arrays are simply offset (outputs are [batch][...] with the batch axis leading).
    const size_t kv_row = (size_t)e->cfg.n_layers * KV_DIM;
    for (int b = 0; b < a->batch; ++b) {
        PersistParams q = p;
        q.token = p.token + b; q.seq_k = p.seq_k + b; q.seq_v = p.seq_v + b; q.seq_layer_stride = p.seq_layer_stride + b;
        q.seq_len = p.seq_len + b; q.next_token = p.next_token + b;
        q.logits = p.logits ? p.logits + (size_t)b * e->cfg.vocab : nullptr;
        q.k_write = p.k_write ? p.k_write + b * kv_row : nullptr;
        q.v_write = p.v_write ? p.v_write + b * kv_row : nullptr;
        void* args[] = {&q};
        cudaError_t err = cudaLaunchCooperativeKernel(persist_kernel(mode, tp), dim3(s->grid), dim3(PT), args, (size_t)s->smem, st);
        ++e->launches;
        if (err != cudaSuccess) return engine_fail(e, Q3_ERR_CUDA, "persist: cooperative launch failed: %s", cudaGetErrorString(err));
    }
    return Q3_OK;
}

}  // namespace q3
