/*
 * q3mk.h — C ABI of the B200 (sm_100a) Qwen3-0.6B decode / prefill engine.
 *
 * This is the boundary a host language binds.  Plain pointers and sizes only; no C++ or
 * torch types.  Every function returns Q3_OK (0) or a negative error code and never throws.
 * All pointers named "device" are CUDA device addresses on the engine's GPU; the caller owns
 * every input and output buffer, the engine owns only its scratch (allocated in q3_create).
 *
 * It replaces the reference project's host->device boundary, which is a Python class driving
 * one NVRTC-compiled kernel through the CUDA driver API:
 *     qwen3mk/kernel.py:109-233   class Megakernel (step / bind / launch / _launch)
 *     csrc/qwen3_step.cu:382-394  extern "C" __global__ qwen3_step(25 pointers)
 * Tensor layouts are the reference's (qwen3mk/kernel.py:27-50): bf16 weights in Hugging Face
 * [out, in] row-major order stacked over layers, fp32 logits, int64 tokens, bf16 K/V rows.
 *
 * Model geometry is fixed to Qwen3-0.6B per head/row: hidden 1024, 16 query heads, 8 KV heads,
 * head dim 128, FFN 3072, RoPE theta 1e6, eps 1e-6.  The layer count and vocabulary size are
 * run-time values (28 and 151936 for the real model) so that small models can be tested.
 */
#ifndef Q3MK_H
#define Q3MK_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q3_OK                 0
#define Q3_ERR_INVALID       (-1)  /* bad argument (message in q3_last_error)               */
#define Q3_ERR_CUDA          (-2)  /* a CUDA runtime call failed                            */
#define Q3_ERR_NOT_RESIDENT  (-3)  /* the persistent grid cannot be co-resident on the GPU  */
#define Q3_ERR_DEVICE_WAIT   (-4)  /* a bounded device-side wait gave up (see q3_status)    */
#define Q3_ERR_UNSUPPORTED   (-5)  /* valid request this build cannot serve on that path    */

/* q3_decode_args.flags */
#define Q3_F_APPEND_KV    0x1u  /* write the new K/V rows into cache slot seq_len[b], then seq_len[b] += 1 */
#define Q3_F_PATH_AUTO    0x0u  /* engine picks: persistent kernel for small batches, layered otherwise    */
#define Q3_F_PATH_LAYERED 0x10u /* one launch per phase (debug ladder, large batches)                      */
#define Q3_F_PATH_FUSED   0x30u /* layered, but batches of 4..64 run two launches per layer: split attention + one persistent
                                   kernel for Wo, norm, gate/up, SiLU, down, norm and the next layer's q/k/v (opt-in: measured
                                   slower than the launch chain so far) */
#define Q3_F_PATH_PERSIST 0x20u /* one persistent cooperative launch per step                              */
#define Q3_F_PATH_MASK    0xf0u
#define Q3_F_GRAPH        0x100u /* layered path: capture the step's launches into a CUDA graph and replay it on later calls with the same arguments */

typedef struct q3_engine q3_engine; /* opaque */

typedef struct q3_config {
    int32_t n_layers;       /* 28 for Qwen3-0.6B                                                 */
    int32_t vocab;          /* 151936 for Qwen3-0.6B; must be >= 1                               */
    int32_t max_batch;      /* largest q3_decode_args.batch the scratch is sized for (>= 1)      */
    int32_t max_tokens;     /* largest q3_prefill_args.n_tokens the scratch is sized for (0: no prefill) */
    int32_t grid_limit;     /* 0 = one CTA per SM; otherwise cap the persistent grid (tests)     */
    int32_t wait_limit_us;  /* patience of every device-side wait in microseconds; 0 = the default (200 ms).  Tests set it low to see a wait give up */
} q3_config;

/* The 13 weight tensors, device pointers to bf16.  Replaces slots 1..13 of the reference's
 * kernel argument list (qwen3mk/kernel.py:23-24, csrc/qwen3_step.cu:383-391). */
typedef struct q3_weights {
    const void* ln1;    /* [L, 1024]          */
    const void* wq;     /* [L, 2048, 1024]    */
    const void* wk;     /* [L, 1024, 1024]    */
    const void* wv;     /* [L, 1024, 1024]    */
    const void* qn;     /* [L, 128]           */
    const void* kn;     /* [L, 128]           */
    const void* wo;     /* [L, 1024, 2048]    */
    const void* ln2;    /* [L, 1024]          */
    const void* wg;     /* [L, 3072, 1024]    */
    const void* wu;     /* [L, 3072, 1024]    */
    const void* wd;     /* [L, 1024, 3072]    */
    const void* fnorm;  /* [1024]             */
    const void* embed;  /* [vocab, 1024], also the (tied) LM head */
} q3_weights;

/* One decode step for `batch` independent sequences.  Generalises the reference's fixed
 * batch-1 / position-128 launch (qwen3mk/kernel.py:180-191): sequence b decodes position
 * seq_len[b] against seq_len[b] cached positions.  The per-sequence descriptors live in device
 * memory so that back-to-back launches need no host work. */
typedef struct q3_decode_args {
    int32_t batch;                   /* 1..max_batch                                                   */
    int32_t max_len;                 /* host-side upper bound of seq_len[b] for this call (work split) */
    uint32_t flags;                  /* Q3_F_*                                                         */
    uint32_t reserved;
    const int64_t* token;            /* device [batch]  input token ids                                */
    const uint64_t* seq_k;           /* device [batch]  address of sequence b's K cache, bf16 [L][cap_b][8][128] */
    const uint64_t* seq_v;           /* device [batch]  same for V                                     */
    const int64_t* seq_layer_stride; /* device [batch]  elements between consecutive layers (cap_b * 1024) */
    int32_t* seq_len;                /* device [batch]  cached positions = position of this token; written only with Q3_F_APPEND_KV */
    float* logits;                   /* device [batch, vocab] fp32, or NULL                            */
    int64_t* next_token;             /* device [batch]  argmax, ties -> lowest index                   */
    void* k_write;                   /* device bf16 [batch, L, 8, 128] or NULL (K after head norm + RoPE) */
    void* v_write;                   /* device bf16 [batch, L, 8, 128] or NULL                         */
} q3_decode_args;

/* Causal prefill of one prompt: replaces qwen3mk/prefill.py:46-81 (fp32 torch loop) by GPU kernels. */
typedef struct q3_prefill_args {
    int32_t n_tokens;        /* 1..max_tokens                                        */
    int32_t cache_capacity;  /* positions per layer in kcache/vcache (>= n_tokens)   */
    const int64_t* ids;      /* device [n_tokens]                                    */
    void* kcache;            /* device bf16 [L, cache_capacity, 8, 128], slots [0, n_tokens) written */
    void* vcache;            /* device bf16 [L, cache_capacity, 8, 128]              */
    float* last_logits;      /* device [vocab] fp32, logits of the last position, or NULL */
    int64_t* next_token;     /* device [1] argmax of last_logits, or NULL            */
} q3_prefill_args;

/* Create an engine on CUDA device `device` (makes it current).  Replaces Megakernel.__init__
 * (qwen3mk/kernel.py:120-162): occupancy check, scratch, sync words. */
int q3_create(int device, const q3_config* cfg, q3_engine** out);

/* Free the engine's scratch.  Safe on NULL. */
void q3_destroy(q3_engine* e);

/* Record the weight pointers used by later calls (borrowed, never written).  Replaces the
 * pointer marshalling of Megakernel.step / bind (qwen3mk/kernel.py:185-188,203-206).  When a pointer of the seven
 * layer matrices differs from the last call's, the persistent kernel's packed copy is rebuilt: a kernel on the legacy
 * default stream followed by cudaDeviceSynchronize (a device-wide wait, once per weight set). */
int q3_set_weights(q3_engine* e, const q3_weights* w);

/* The persistent kernel streams an engine-owned re-layout of the seven layer matrices (built by
 * q3_set_weights, about 0.9 GB for the full model) and rebuilds it only when a weight POINTER
 * changes.  A caller that rewrites weights in place calls this before the next q3_set_weights.
 * No counterpart in the reference, which reads the caller's tensors directly. */
int q3_invalidate_weights(q3_engine* e);

/* Tensor parallelism over 2, 4 or 8 GPUs of one node, one process and one engine per GPU.  Rank r then owns query
 * heads [r 16/size, ..), kv heads [r 8/size, ..), FFN rows [r 3072/size, ..) and, for the LM head, words
 * [r vocab/size, ..); every rank keeps the whole residual stream.  The two per-layer sums over ranks (after the output
 * projection and after the down projection) are red instructions from every rank's CTAs straight into every rank's
 * accumulators over NVLink, fused into the phases that produce the partial sums; the grid barrier spans all ranks; the
 * arg-max is settled through per-rank mailboxes.  Peer memory is only ever written (red / st), never read.
 *   q3_tp_export: 64 bytes identifying this engine's state allocation (a CUDA IPC handle); the host exchanges them.
 *   q3_tp_attach: map the `size` handles (64 bytes each, in rank order; this rank's own entry is ignored) and switch
 *                 the engine to its share.  Call q3_set_weights afterwards (the FULL tensors: the engine packs its
 *                 share).  size = 1 switches tensor parallelism off again.
 * While attached, q3_decode serves batch 1 with up to 255 cached positions on the persistent path; every rank must
 * enqueue the same step (the kernels wait for one another, bounded by the wait limit).  Outputs: next_token on every
 * rank; logits only for the rank's words; k_write / v_write (and the appended cache rows) only for the rank's kv heads.
 * The reference is single-GPU (qwen3mk/kernel.py:120-131); no counterpart. */
int q3_tp_export(q3_engine* e, void* handle);
int q3_tp_attach(q3_engine* e, int32_t rank, int32_t size, const void* handles);

/* RoPE table: device fp32 [n_positions][128], row p = cos(p * f_0..f_63) then sin(p * f_0..f_63),
 * f_i = 1e6^(-2i/128).  Generalises the reference's single-position table
 * (qwen3mk/kernel.py:102-106).  Borrowed. */
int q3_set_rope(q3_engine* e, const float* table, int32_t n_positions);

/* Enqueue one decode step on `stream` (a cudaStream_t; NULL = default stream).  No host sync.
 * Replaces Megakernel._launch (qwen3mk/kernel.py:231-233). */
int q3_decode(q3_engine* e, const q3_decode_args* a, void* stream);

/* Enqueue a causal prefill on `stream`. */
int q3_prefill(q3_engine* e, const q3_prefill_args* a, void* stream);

/* One layered decode step WITHOUT an engine and without any device allocation, for callers that may
 * not call cudaMalloc where they decode (a plugin inside another runtime's memory budget, a process
 * whose device memory is fully pre-carved).  It has no counterpart in the reference.  The scratch is a
 * device array inside the library (about 0.4 MB per GPU, held until the process exits), which limits a
 * call to Q3_NOALLOC_MAX_BATCH sequences; larger batches are rejected with Q3_ERR_INVALID.  The first
 * call on a device looks up the array's address (make it before any stream capture).  All calls share
 * the array: do not let two calls overlap on the GPU, from one host thread or from several (the address
 * look-up itself is locked; the array is not).  `w`, `rope` and `a` are as for q3_set_weights,
 * q3_set_rope and q3_decode; only the layered path is available. */
#define Q3_NOALLOC_MAX_BATCH 2
int q3_decode_noalloc(const q3_weights* w, const float* rope, int32_t rope_positions, int32_t n_layers, int32_t vocab,
                      const q3_decode_args* a, void* stream);

/* Status of the last q3_decode_noalloc on the current device: synchronises `stream`, copies the status words
 * of the static array to `words` (up to `n`, may be NULL; same layout as q3_status) and returns Q3_OK or
 * Q3_ERR_DEVICE_WAIT (for example code 3: a token outside the vocabulary was replaced by token 0; code 5: a
 * cache longer than max_len).  Every q3_decode_noalloc clears the words when it starts, so read them before
 * the next call.  Allocates nothing.  No counterpart in the reference. */
int q3_noalloc_status(void* stream, uint32_t* words, int32_t n);

/* out[t, n] = (resid[t, n] +) sum_k w[n, k] * x[t, k] on the tensor cores (tcgen05 / TMEM / TMA): w bf16
 * [n_rows, K] row-major (n_rows a multiple of 128, K of 64), x fp32 [n_tok, K], out and resid fp32
 * [n_tok, n_rows] (resid may be NULL or alias out).  x is split into `nsplit` bf16 planes (1: rounded to
 * bf16, 3: exact to fp32) in the caller's `planes` buffer of at least nsplit * round_up(n_tok, tile) * K * 2
 * bytes, tile = 32 / 64 / 128 for n_tok <= 32 / <= 64 / more.  This is the dense product the reference's
 * prefill writes as `xn @ w.T` (qwen3mk/prefill.py:61-80); the engine uses it for prefill and for decode
 * batches too large for the persistent kernel.  Allocates nothing. */
int q3_linear_tc(const void* w, const float* x, float* out, const float* resid, int32_t n_rows, int32_t n_tok, int32_t K,
                 int32_t nsplit, void* planes, int64_t planes_bytes, void* stream);

/* Sample one token per row from fp32 logits [batch, vocab] on the device: keep the `top_k` largest logits of a row
 * (0 = all; ties at the k-th value are all kept), weigh them by exp((logit - max) / temperature) and return the first
 * index whose cumulative weight exceeds uniform[row] * total, in index order.  `uniform` is a device array of `batch`
 * numbers in [0, 1) drawn by the caller (so that a seed reproduces a run); temperature <= 0 or top_k == 1 returns the
 * arg-max (ties -> lowest index) and ignores `uniform`.  `out_tokens` (device int64 [batch]) may be the token buffer
 * of the next q3_decode, so that a sampled stream needs no host round trip.  Allocates nothing, no host sync.
 * The reference stops at greedy decoding and hands the fp32 logits to the caller for this step
 * (csrc/qwen3_step.cu:175, qwen3mk/kernel.py:44-50). */
int q3_sample(const float* logits, int32_t batch, int32_t vocab, float temperature, int32_t top_k,
              const float* uniform, int64_t* out_tokens, void* stream);

/* Synchronise `stream`, read the device status words and clear them.  Returns Q3_OK or
 * Q3_ERR_DEVICE_WAIT; `words` (may be NULL) receives up to `n` raw status words:
 * [0] error code, [1] where (phase id), [2] CTA index, [3] observed counter value. */
int q3_status(q3_engine* e, void* stream, uint32_t* words, int32_t n);

/* Phase tracing of the persistent kernel (the reference's trace came from an external tool:
 * README.md:174-239).  `buf` is a device buffer of n_words 64-bit words, or NULL to switch tracing
 * off.  While set and large enough (grid * (4 + 12 * n_layers) words), every persistent launch makes
 * thread 0 of CTA c store %globaltimer (ns) at buf[c * (4 + 12 L) + ev].  ev 0 = start; for layer l,
 * base = 1 + 12 l: +0 Q activations staged, +1 Q done, +2 K/V rows requested, +3 F q/k/v prepared,
 * +4 F scores done, +5 F head output ready, +6 F done (attention delta sent), +7 attention delta complete,
 * +8 GD activations staged, +9 GD hid ready, +10 GD done (FFN delta sent), +11 FFN delta complete; then
 * 1 + 12 L = LM-head rows done, 2 + 12 L = end.
 * Borrowed. */
int q3_set_trace(q3_engine* e, uint64_t* buf, int64_t n_words);

/* Number of kernel launches this engine has enqueued since creation. */
int64_t q3_launch_count(const q3_engine* e);

/* Persistent-grid geometry chosen at creation: CTAs, threads per CTA, dynamic smem bytes. */
int q3_grid_info(const q3_engine* e, int32_t* ctas, int32_t* threads, int32_t* smem_bytes);

/* Engine-owned scratch for tools and tests: name in {"x","qkv","attn","hid","status","persist_acc"}; returns a
 * device pointer and its size in bytes, or Q3_ERR_INVALID.  "persist_acc" is the persistent kernel's four delta
 * accumulators (64-bit words: contributions << 56 | fixed-point sum), all zero between launches. */
int q3_scratch(const q3_engine* e, const char* name, void** ptr, int64_t* bytes);

/* Message of the last error on this engine (or of the last failed q3_create when e == NULL). */
const char* q3_last_error(const q3_engine* e);

/* Library version string, e.g. "q3mk-b200 0.1 sm_100a". */
const char* q3_version(void);

#ifdef __cplusplus
}
#endif
#endif /* Q3MK_H */
