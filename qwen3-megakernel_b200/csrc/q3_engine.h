// Engine state shared by the translation units behind the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/q3mk.h"
#include "q3_common.cuh"
#include "q3_layered.h"

#define Q3_STATUS_WORDS 8
#define Q3_SYNC_WORDS 64
#define Q3_MAX_SPLITS 64
#ifndef Q3_TC_MIN_BATCH
#define Q3_TC_MIN_BATCH 4   // from this many tokens on the projections run as tensor-core GEMMs (measured at 1024 cached positions: batch 4 1804 vs 1882 us, batch 8 1959 vs 2420 us, batch 2 1740 vs 1598 us)
#endif

struct q3_engine {
    int device;
    q3_config cfg;
    q3_weights w;
    int have_weights;
    const float* rope;  // [rope_n, 128]
    int rope_n;
    int sm_count;
    int max_splits;     // attention splits the partial buffer is sized for
    int lm_grid;        // LM-head blocks the argmax partial buffers are sized for
    // scratch (device)
    float* x;       // [max_batch, 1024]  residual stream
    float* qkv;     // [max_batch, 4096]
    float* attn;    // [max_batch, 2048]
    float* hid;     // [max_batch, 3072]
    float* part;    // [max_batch, 16, max_splits, ATTN_PART_STRIDE]
    float* pval;    // [max_batch, lm_grid]
    int* pidx;      // [max_batch, lm_grid]
    uint32_t* status;
    uint32_t* sync;
    void* pf_desc;  // prefill: per-token sequence descriptors (4 arrays of `cap` entries) + a token slot
    // tensor-core path (batches of Q3_TC_MIN_BATCH or more tokens, prefill)
    int cap;            // tokens the scratch is sized for: max(max_batch, max_tokens)
    int part_slots;     // (token, split) slots in `part`
    void* planes;       // bf16 [3][cap rounded up to 128][3072] activation planes
    float* gate;        // [cap, 3072]
    float* up;          // [cap, 3072]
    float* logits_tc;   // [max_batch, vocab] when the caller passes no logits buffer
    void* lk_state;     // the layer kernel's row sums of squares and barrier words (q3_layer_tc.h)
    // persistent kernel geometry
    int p_grid, p_threads, p_smem;
    void* p_state;  // owned by q3_persist.cu
    int64_t launches;
    void* graphs;       // cache of captured layered steps (owned by q3_api.cu)
    void* capture_stream;  // cudaStream_t the steps are captured on
    unsigned long long* trace;  // caller-owned device buffer for phase time stamps, or nullptr
    int64_t trace_words;
    char err[512];
};

namespace q3 {
int persist_setup(q3_engine* e);
void persist_teardown(q3_engine* e);
bool persist_supports(const q3_engine* e, const q3_decode_args* a);
int persist_decode(q3_engine* e, const q3_decode_args* a, cudaStream_t st);
int persist_weights_changed(q3_engine* e);
void persist_invalidate_weights(q3_engine* e);
void* persist_accumulators(const q3_engine* e, int64_t* bytes);   // the four counted accumulator vectors (tests), or nullptr
int persist_tp_export(q3_engine* e, void* handle64);
int persist_tp_attach(q3_engine* e, int rank, int size, const void* handles);
int persist_recover(q3_engine* e);   // after a device-side wait gave up: clear the exchange buffers and accumulators
int engine_fail(q3_engine* e, int code, const char* fmt, ...);
// the layered decode step on engine `e` (one launch per phase); `e` supplies weights, RoPE table and scratch
// prompt-mode extras of the layered step: one sequence, tokens at positions 0..T-1 of this cache
struct PrefillCtx {
    const void* kcache;   // bf16 [L, capacity, 8, 128]
    const void* vcache;
    long long layer_stride;
};
// layer_kernel: decode batches the persistent layer kernel serves take it (two launches per layer); false keeps one
// launch per phase
int decode_layered(q3_engine* e, const q3_decode_args* a, cudaStream_t st, int tc_planes = 3, const PrefillCtx* prompt = nullptr,
                   bool layer_kernel = false);
cudaError_t launch_prefill_attn_tc(const float* qkv, const void* kcache_layer, const void* vcache_layer, int cap_rows, void* planes,
                                   int plane_rows, int nsplit, int T, uint32_t* status, cudaStream_t st);
}  // namespace q3
