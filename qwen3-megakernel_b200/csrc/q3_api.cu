// C ABI of the engine (declared in include/q3mk.h): engine life cycle, argument checks, path
// selection and the per-step launch sequence of the layered path.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "q3_engine.h"
#include "q3_gemm_tc.h"
#include "q3_layer_tc.h"

using namespace q3;

static char g_create_error[512] = "";

int q3::engine_fail(q3_engine* e, int code, const char* fmt, ...) {
    char* dst = e ? e->err : g_create_error;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(dst, 512, fmt, ap);
    va_end(ap);
    return code;
}
#define fail q3::engine_fail

#define CU(e, call)                                                                                  \
    do {                                                                                             \
        cudaError_t err__ = (call);                                                                  \
        if (err__ != cudaSuccess)                                                                    \
            return fail(e, Q3_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(err__), __FILE__, __LINE__); \
    } while (0)

static int alloc(q3_engine* e, void** p, size_t bytes) {
    CU(e, cudaMalloc(p, bytes));
    CU(e, cudaMemset(*p, 0, bytes));
    return Q3_OK;
}

// ------------------------------------------------------------------------------------------------
// CUDA graphs for the layered step: a step is hundreds of small launches whose arguments all live in
// device memory, so a call with the same argument block can replay a captured graph instead of
// re-issuing them.  A key is seen uncaptured once (which also performs one-time function attribute
// set-up), captured on its second use, and replayed afterwards.  Weights, RoPE table or trace changes
// drop the cache.
// ------------------------------------------------------------------------------------------------
struct GraphEntry {
    q3_decode_args key;
    int n_splits;
    int chunk_pad;         // the attention kernel's padded chunk length is baked into the captured arguments
    int seen;
    int64_t launches;      // kernels inside the graph
    cudaGraphExec_t exec;
};
static std::vector<GraphEntry>* graph_cache(q3_engine* e) {
    if (!e->graphs) e->graphs = new std::vector<GraphEntry>();
    return static_cast<std::vector<GraphEntry>*>(e->graphs);
}
static void drop_graphs(q3_engine* e) {
    if (!e->graphs) return;
    auto* v = static_cast<std::vector<GraphEntry>*>(e->graphs);
    for (auto& g : *v)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    v->clear();
}

extern "C" const char* q3_version(void) { return "q3mk-b200 0.1 sm_100a"; }

extern "C" const char* q3_last_error(const q3_engine* e) { return e ? e->err : g_create_error; }

extern "C" int q3_create(int device, const q3_config* cfg, q3_engine** out) {
    if (!cfg || !out) return fail(nullptr, Q3_ERR_INVALID, "q3_create: null argument");
    *out = nullptr;
    if (cfg->n_layers < 1 || cfg->vocab < 1 || cfg->max_batch < 1 || cfg->max_tokens < 0 || cfg->grid_limit < 0 || cfg->wait_limit_us < 0)
        return fail(nullptr, Q3_ERR_INVALID, "q3_create: n_layers=%d vocab=%d max_batch=%d max_tokens=%d grid_limit=%d out of range",
                    cfg->n_layers, cfg->vocab, cfg->max_batch, cfg->max_tokens, cfg->grid_limit);
    CU(nullptr, cudaSetDevice(device));
    cudaDeviceProp prop;
    CU(nullptr, cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(nullptr, Q3_ERR_UNSUPPORTED, "q3_create: device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);

    q3_engine* e = new (std::nothrow) q3_engine();
    if (!e) return fail(nullptr, Q3_ERR_INVALID, "q3_create: out of host memory");
    memset(e, 0, sizeof(*e));
    e->device = device;
    e->cfg = *cfg;
    e->sm_count = prop.multiProcessorCount;
    e->max_splits = Q3_MAX_SPLITS;
    e->lm_grid = e->sm_count * 8;
    e->cap = cfg->max_batch > cfg->max_tokens ? cfg->max_batch : cfg->max_tokens;
    const size_t B = (size_t)e->cap;
    // attention partials: up to 64 splits for small batches, at least 2 per token for large ones
    e->part_slots = (int)((B < 16 ? B : 16) * Q3_MAX_SPLITS > 2 * B ? (B < 16 ? B : 16) * Q3_MAX_SPLITS : 2 * B);
    const bool tc = e->cap >= Q3_TC_MIN_BATCH;
    const size_t cap_pad = (B + 127) / 128 * 128;
    int rc;
    if ((rc = alloc(e, (void**)&e->x, B * HIDDEN * 4)) ||
        (rc = alloc(e, (void**)&e->qkv, B * QKV_DIM * 4)) ||
        (rc = alloc(e, (void**)&e->attn, B * Q_DIM * 4)) ||
        (rc = alloc(e, (void**)&e->hid, B * INTER * 4)) ||
        (rc = alloc(e, (void**)&e->part, (size_t)e->part_slots * Q_HEADS * ATTN_PART_STRIDE * 4)) ||
        (rc = alloc(e, (void**)&e->pval, (size_t)cfg->max_batch * e->lm_grid * 4)) ||
        (rc = alloc(e, (void**)&e->pidx, (size_t)cfg->max_batch * e->lm_grid * 4)) ||
        (rc = alloc(e, (void**)&e->status, Q3_STATUS_WORDS * 4)) ||
        (rc = alloc(e, (void**)&e->sync, Q3_SYNC_WORDS * 4)) ||
        (rc = alloc(e, (void**)&e->pf_desc, 64 + B * 32)) ||
        (tc && ((rc = alloc(e, &e->planes, 3 * cap_pad * INTER * 2)) ||
                (rc = alloc(e, (void**)&e->gate, B * INTER * 4)) ||
                (rc = alloc(e, (void**)&e->up, B * INTER * 4)) ||
                (rc = alloc(e, &e->lk_state, LK_STATE_BYTES)) ||
                (cfg->max_batch >= Q3_TC_MIN_BATCH && (rc = alloc(e, (void**)&e->logits_tc, (size_t)cfg->max_batch * cfg->vocab * 4)))))) {
        strncpy(g_create_error, e->err, sizeof(g_create_error) - 1);
        q3_destroy(e);
        return rc;
    }
    {
        cudaStream_t cs = nullptr;
        if (cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking) != cudaSuccess) {
            fail(nullptr, Q3_ERR_CUDA, "q3_create: cudaStreamCreateWithFlags failed");
            q3_destroy(e);
            return Q3_ERR_CUDA;
        }
        e->capture_stream = cs;
    }
    rc = persist_setup(e);
    if (rc != Q3_OK) {
        strncpy(g_create_error, e->err, sizeof(g_create_error) - 1);
        q3_destroy(e);
        return rc;
    }
    *out = e;
    return Q3_OK;
}

extern "C" void q3_destroy(q3_engine* e) {
    if (!e) return;
    cudaSetDevice(e->device);
    drop_graphs(e);
    delete static_cast<std::vector<GraphEntry>*>(e->graphs);
    if (e->capture_stream) cudaStreamDestroy(static_cast<cudaStream_t>(e->capture_stream));
    persist_teardown(e);
    void* bufs[] = {e->x, e->qkv, e->attn, e->hid, e->part, e->pval, e->pidx, e->status, e->sync, e->pf_desc, e->planes, e->gate, e->up, e->logits_tc, e->lk_state};
    for (void* p : bufs)
        if (p) cudaFree(p);
    delete e;
}

extern "C" int q3_set_weights(q3_engine* e, const q3_weights* w) {
    if (!e || !w) return fail(e, Q3_ERR_INVALID, "q3_set_weights: null argument");
    const void* const* p = reinterpret_cast<const void* const*>(w);
    static const char* names[13] = {"ln1", "wq", "wk", "wv", "qn", "kn", "wo", "ln2", "wg", "wu", "wd", "fnorm", "embed"};
    for (int i = 0; i < 13; ++i) {
        if (!p[i]) return fail(e, Q3_ERR_INVALID, "q3_set_weights: %s is null", names[i]);
        if (reinterpret_cast<uintptr_t>(p[i]) & 15) return fail(e, Q3_ERR_INVALID, "q3_set_weights: %s is not 16-byte aligned", names[i]);
    }
    drop_graphs(e);
    e->w = *w;
    e->have_weights = 1;
    CU(e, cudaSetDevice(e->device));
    return persist_weights_changed(e);
}

extern "C" int q3_invalidate_weights(q3_engine* e) {
    if (!e) return Q3_ERR_INVALID;
    persist_invalidate_weights(e);
    return Q3_OK;
}

extern "C" int q3_tp_export(q3_engine* e, void* handle) {
    if (!e || !handle) return fail(e, Q3_ERR_INVALID, "q3_tp_export: null argument");
    CU(e, cudaSetDevice(e->device));
    return persist_tp_export(e, handle);
}

extern "C" int q3_tp_attach(q3_engine* e, int32_t rank, int32_t size, const void* handles) {
    if (!e) return fail(e, Q3_ERR_INVALID, "q3_tp_attach: null argument");
    CU(e, cudaSetDevice(e->device));
    drop_graphs(e);
    return persist_tp_attach(e, rank, size, handles);
}

extern "C" int q3_set_rope(q3_engine* e, const float* table, int32_t n_positions) {
    if (!e || !table || n_positions < 1) return fail(e, Q3_ERR_INVALID, "q3_set_rope: bad argument");
    drop_graphs(e);
    e->rope = table;
    e->rope_n = n_positions;
    return Q3_OK;
}

extern "C" int q3_set_trace(q3_engine* e, uint64_t* buf, int64_t n_words) {
    if (!e || n_words < 0) return fail(e, Q3_ERR_INVALID, "q3_set_trace: bad argument");
    e->trace = reinterpret_cast<unsigned long long*>(buf);
    e->trace_words = buf ? n_words : 0;
    return Q3_OK;
}

extern "C" int64_t q3_launch_count(const q3_engine* e) { return e ? e->launches : 0; }

extern "C" int q3_grid_info(const q3_engine* e, int32_t* ctas, int32_t* threads, int32_t* smem_bytes) {
    if (!e) return Q3_ERR_INVALID;
    if (ctas) *ctas = e->p_grid;
    if (threads) *threads = e->p_threads;
    if (smem_bytes) *smem_bytes = e->p_smem;
    return Q3_OK;
}

extern "C" int q3_scratch(const q3_engine* e, const char* name, void** ptr, int64_t* bytes) {
    if (!e || !name || !ptr || !bytes) return Q3_ERR_INVALID;
    const int64_t B = e->cap;
    if (!strcmp(name, "x")) { *ptr = e->x; *bytes = B * HIDDEN * 4; }
    else if (!strcmp(name, "qkv")) { *ptr = e->qkv; *bytes = B * QKV_DIM * 4; }
    else if (!strcmp(name, "attn")) { *ptr = e->attn; *bytes = B * Q_DIM * 4; }
    else if (!strcmp(name, "hid")) { *ptr = e->hid; *bytes = B * INTER * 4; }
    else if (!strcmp(name, "status")) { *ptr = e->status; *bytes = Q3_STATUS_WORDS * 4; }
    else if (!strcmp(name, "persist_acc")) { *ptr = persist_accumulators(e, bytes); if (!*ptr) return Q3_ERR_UNSUPPORTED; }
    else return Q3_ERR_INVALID;
    return Q3_OK;
}

extern "C" int q3_status(q3_engine* e, void* stream, uint32_t* words, int32_t n) {
    if (!e) return Q3_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t h[Q3_STATUS_WORDS];
    CU(e, cudaStreamSynchronize(st));
    CU(e, cudaMemcpy(h, e->status, sizeof(h), cudaMemcpyDeviceToHost));
    for (int i = 0; words && i < n && i < Q3_STATUS_WORDS; ++i) words[i] = h[i];
    if (h[0] == 0) return Q3_OK;
    // leave the engine reusable: clear the status and the barrier words
    CU(e, cudaMemset(e->status, 0, Q3_STATUS_WORDS * 4));
    CU(e, cudaMemset(e->sync, 0, Q3_SYNC_WORDS * 4));
    if (e->lk_state) CU(e, cudaMemset(e->lk_state, 0, LK_STATE_BYTES));
    if (persist_recover(e) != Q3_OK) return Q3_ERR_CUDA;
    return fail(e, Q3_ERR_DEVICE_WAIT, "device status: code %u at site %u, CTA %u, value %u", h[0], h[1], h[2], h[3]);
}

// ------------------------------------------------------------------------------------------------
// layered decode step
// ------------------------------------------------------------------------------------------------
// positions a split's block may take, rounded up to 32: with the split count it fixes the attention launch
static int chunk_pad_for(int max_len, int ns) { return (((max_len + 1 + ns - 1) / ns) + 31) / 32 * 32; }

static int splits_for(const q3_engine* e, int batch, int max_len) {
    const int n = max_len + 1;
    int by_len = (n + 31) / 32;                                   // at least 32 positions per split
    // The split count with the shortest estimated launch.  A launch takes `waves` rounds of blocks; a block costs a fixed
    // 4 us (prologue with the head preparation, combine) plus its positions at the block's share of an SM's part of the copy
    // bandwidth; more than one split adds the merge launch (5 us), one split writes the output planes itself.
    //   Batches whose (sequence, kv head) pairs fill the GPU: four-warp blocks, two per SM, 23 ns per position.  Fitted to,
    //   per step: batch 64 x 1024, 1 / 2 / 3 / 4 splits: 2524 / 2623 / 2691 / 2716 us; batch 32 x 2048, 1 / 2: 2057 / 2149;
    //   batch 24 x 1024, 1 / 3: 1336 / 1463; batch 48 x 1024, 1 / 2: 2235 / 2214; batch 20 x 4096, 2 / 3: 2814 / 2415.
    //   Smaller batches: eight-warp blocks, one per SM, 6 ns per position.  Batch 8 x 1024, 1 / 2 splits: 1000 / 1035 us;
    //   batch 4 x 512: 882 / 920; batch 16 x 2048: 1446 / 1597.
    const bool big = KV_HEADS * batch >= e->sm_count;
    const int slots = (big ? 2 : 1) * e->sm_count, pairs = KV_HEADS * batch;
    const double per_pos = big ? 0.023 : 0.006;
    double best = 1e30;
    int s = 1;
    for (int c = 1; c <= 16 && c <= by_len; ++c) {
        const int waves = (pairs * c + slots - 1) / slots, per = (n + c - 1) / c;
        const double t = waves * (4.0 + per_pos * per) + (c > 1 ? 5.0 : 0.0);
        if (t < best - 1e-9) { best = t; s = c; }
    }
    if (s < 1) s = 1;
    const int by_chunk = (n + ATTN_CHUNK_MAX - 1) / ATTN_CHUNK_MAX;   // a split takes at most ATTN_CHUNK_MAX positions (the launchers check it)
    if (s < by_chunk) s = by_chunk;
    if (s > e->max_splits) s = e->max_splits;
    if (e->part_slots > 0 && s * batch > e->part_slots) s = e->part_slots / batch;
    if (s < 1) s = 1;
    return s;
}

int q3::decode_layered(q3_engine* e, const q3_decode_args* a, cudaStream_t st, int tc_planes, const PrefillCtx* prompt, bool layer_kernel) {
    const bool last_token_only = prompt != nullptr;
    const int B = a->batch, L = e->cfg.n_layers, V = e->cfg.vocab;
    const q3_weights& w = e->w;
    const int append = (a->flags & Q3_F_APPEND_KV) ? 1 : 0;
    const int ns = splits_for(e, B, a->max_len);
    // From Q3_TC_MIN_BATCH tokens on, the projections are tensor-core GEMMs over bf16 planes of the
    // activations (tc_planes = 3: exact to fp32); below that, CUDA-core matrix-vector kernels.
    const bool tc = B >= Q3_TC_MIN_BATCH && e->planes != nullptr;
    const int tile = B <= 32 ? 32 : (B <= 64 ? 64 : 128);
    const int prow = (B + tile - 1) / tile * tile;
    bf16_raw* planes = reinterpret_cast<bf16_raw*>(e->planes);
    auto bf = [](const void* p) { return reinterpret_cast<const bf16_raw*>(p); };
#define LAUNCH(call)                                                                                   \
    do {                                                                                               \
        cudaError_t err__ = (call);                                                                    \
        ++e->launches;                                                                                 \
        if (err__ != cudaSuccess) return fail(e, Q3_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(err__)); \
    } while (0)
    // out[:, col0 : col0 + rows] (+)= planes @ wmat^T
    auto gemm = [&](const bf16_raw* wmat, int rows, int K, float* out, int ldo, const float* resid, int ldr) -> cudaError_t {
        GemmTcCall c{wmat, planes, out, resid, ldo, ldr, rows, B, K, tc_planes, prow, e->status};
        return launch_gemm_tc(c, st);
    };

    // the row argmax of the tensor-core LM head meets in e->pval (64-bit keys) and e->pidx (tickets): both are scratch
    // of the matrix-vector LM head otherwise, and at least 8 bytes a sequence
    // (only a decode step of at most max_batch sequences uses them: a prompt's tokens would overrun the buffers)
    const bool row_argmax = !last_token_only && B <= e->cfg.max_batch;
    unsigned long long* arg_keys = row_argmax ? reinterpret_cast<unsigned long long*>(e->pval) : nullptr;
    unsigned* arg_tickets = row_argmax ? reinterpret_cast<unsigned*>(e->pidx) : nullptr;
    // what the launches of this step can serve: the attention split covers n_splits * chunk_pad positions (the new one
    // included) and the RoPE table has rope_n rows; both are fixed by (n_splits, chunk_pad), like a captured graph
    const int pad = chunk_pad_for(a->max_len, ns);
    long long cover = (long long)ns * pad - 1;
    if (cover > e->rope_n - 1) cover = e->rope_n - 1;
    const int len_bound = (int)cover;
    LAUNCH(launch_embed(reinterpret_cast<const long long*>(a->token), bf(w.embed), V, e->x, e->status, B, st, arg_keys, arg_tickets, a->seq_len, len_bound));
    // Decode batches of 4..64 sequences: two launches per layer, the split attention and the persistent layer kernel
    // (everything between two attentions: merge, Wo, norm, gate/up, SiLU, down, norm, q/k/v of the next layer).
    const bool lk = layer_kernel && tc && prompt == nullptr && tc_planes == 3 && layer_tc_supports(e, B);
    if (lk) LAUNCH(launch_layer_tc(e, LK_MODE_FIRST, 0, B, st));
    for (int l = 0; lk && l < L; ++l) {
        AttnArgs t{};
        t.qkv = e->qkv; t.seq_k = a->seq_k; t.seq_v = a->seq_v;
        t.seq_layer_stride = reinterpret_cast<const long long*>(a->seq_layer_stride);
        t.seq_len = a->seq_len; t.part = e->part; t.layer = l; t.n_splits = ns;
        t.chunk_pad = pad; t.len_bound = len_bound;
        t.fused_prep = 1; t.qn = bf(w.qn); t.kn = bf(w.kn); t.rope = e->rope;
        t.k_write = reinterpret_cast<bf16_raw*>(a->k_write); t.v_write = reinterpret_cast<bf16_raw*>(a->v_write);
        t.n_layers = L; t.append = append;
        t.row_ssq = reinterpret_cast<const float*>(e->lk_state);   // the q/k/v rows still lack their norm's scale
        t.merged = e->attn;                                        // the last block of a (sequence, kv head) merges its splits
        t.merge_count = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(e->lk_state) + LK_STATE_MERGE_OFFSET);
        LAUNCH(launch_attn_split(t, B, st));
        LAUNCH(launch_layer_tc(e, l + 1 < L ? LK_MODE_MID : LK_MODE_LAST, l, B, st));
    }
    for (int l = 0; !lk && l < L; ++l) {
        GemvArgs g{};
        // qkv = rms(x, ln1) @ [wq; wk; wv]^T
        if (tc) {
            // a split-K launch adds its partial tiles onto zeros, which the producer of its input planes writes on the side
            const ZeroRows zq{{e->qkv, nullptr}, {QKV_DIM, 0}, {QKV_DIM, 0}};
            LAUNCH(launch_act_split(e->x, HIDDEN, HIDDEN, bf(w.ln1) + (size_t)l * HIDDEN, planes, prow, tc_planes, B, st,
                                    gemm_tc_splits_k(QKV_DIM, B, HIDDEN) ? &zq : nullptr));
            {   // the three projections in one launch: 32 weight tiles instead of 16 + 8 + 8
                GemmTcGroupCall c{};
                c.n_groups = 3;
                c.w[0] = bf(w.wq) + (size_t)l * Q_DIM * HIDDEN; c.n_rows[0] = Q_DIM; c.out[0] = e->qkv; c.ldo[0] = QKV_DIM;
                c.w[1] = bf(w.wk) + (size_t)l * KV_DIM * HIDDEN; c.n_rows[1] = KV_DIM; c.out[1] = e->qkv + Q_DIM; c.ldo[1] = QKV_DIM;
                c.w[2] = bf(w.wv) + (size_t)l * KV_DIM * HIDDEN; c.n_rows[2] = KV_DIM; c.out[2] = e->qkv + Q_DIM + KV_DIM; c.ldo[2] = QKV_DIM;
                c.x_planes = planes; c.n_tok = B; c.K = HIDDEN; c.nsplit = tc_planes; c.plane_rows = prow; c.status = e->status;
                c.out_is_zero = 1;   // act_split has cleared the rows
                LAUNCH(launch_gemm_tc_group(c, st));
            }
        } else {
            g.seg[0] = {bf(w.wq) + (size_t)l * Q_DIM * HIDDEN, Q_DIM};
            g.seg[1] = {bf(w.wk) + (size_t)l * KV_DIM * HIDDEN, KV_DIM};
            g.seg[2] = {bf(w.wv) + (size_t)l * KV_DIM * HIDDEN, KV_DIM};
            g.x = e->x; g.ldx = HIDDEN; g.gain = bf(w.ln1) + (size_t)l * HIDDEN;
            g.out = e->qkv; g.ldo = QKV_DIM; g.n_rows = QKV_DIM; g.batch = B;
            LAUNCH(launch_gemv(1024, EPI_STORE, g, QKV_DIM / 16, st));
        }

        HeadPrepArgs h{};
        h.qkv = e->qkv; h.qn = bf(w.qn); h.kn = bf(w.kn); h.rope = e->rope; h.seq_len = a->seq_len;
        h.k_write = reinterpret_cast<bf16_raw*>(a->k_write); h.v_write = reinterpret_cast<bf16_raw*>(a->v_write);
        h.seq_k = a->seq_k; h.seq_v = a->seq_v; h.seq_layer_stride = reinterpret_cast<const long long*>(a->seq_layer_stride);
        h.layer = l; h.n_layers = L; h.append = append; h.len_bound = len_bound;
        // A prompt's tokens attend rows that earlier tokens of the same launch append: those need the separate kernel.
        // A decode step prepares the heads inside the attention kernel (one launch less per layer).
        const bool fused_prep = prompt == nullptr;
        h.skip_k_store = (prompt != nullptr && B >= 64) ? 1 : 0;   // the tcgen05 attention of a long prompt reads K from the cache
        if (!fused_prep) LAUNCH(launch_head_prep(h, B, st));

        AttnArgs t{};
        t.qkv = e->qkv; t.seq_k = a->seq_k; t.seq_v = a->seq_v;
        t.seq_layer_stride = reinterpret_cast<const long long*>(a->seq_layer_stride);
        t.seq_len = a->seq_len; t.part = e->part; t.layer = l; t.n_splits = ns;
        t.chunk_pad = pad; t.len_bound = len_bound;
        t.fused_prep = fused_prep ? 1 : 0; t.qn = h.qn; t.kn = h.kn; t.rope = h.rope; t.k_write = h.k_write; t.v_write = h.v_write;
        t.n_layers = L; t.append = append;
        if (prompt != nullptr && B >= 64) {
            // a prompt: tiled causal attention over the rows head_prep has just written into the cache
            const bf16_raw* kc = bf(prompt->kcache) + (size_t)l * prompt->layer_stride;
            const bf16_raw* vc = bf(prompt->vcache) + (size_t)l * prompt->layer_stride;
            // tcgen05 attention; it writes the Wo GEMM's input planes itself
            LAUNCH(launch_prefill_attn_tc(e->qkv, kc, vc, (int)(prompt->layer_stride / KV_DIM), planes, prow, tc_planes, B, e->status, st));
        } else if (tc && ns == 1 && fused_prep && tc_planes == 3) {
            // one split: the attention blocks write the Wo GEMM's input planes themselves, no merge launch (the padding rows of the
            // token tile keep whatever they held: their columns of the product are never stored)
            t.planes_out = planes; t.plane_rows = prow;
            LAUNCH(launch_attn_split(t, B, st));
        } else if (tc) {
            LAUNCH(launch_attn_planes(t, planes, prow, tc_planes, B, st));   // the merge writes the Wo GEMM's input planes
            ++e->launches;  // two kernels
        } else {
            LAUNCH(launch_attn(t, e->attn, B, st));
            ++e->launches;  // launch_attn is two kernels
        }

        if (tc) {
            // x += attn @ wo^T
            LAUNCH(gemm(bf(w.wo) + (size_t)l * HIDDEN * Q_DIM, HIDDEN, Q_DIM, e->x, HIDDEN, e->x, HIDDEN));
            // hid = silu(rms(x, ln2) @ wg^T) * (rms(x, ln2) @ wu^T)
            // A long prompt: gate and up in one work item of the persistent GEMM, SiLU in its epilogue, the product written as
            // the down GEMM's input plane into the second third of the plane buffer (one plane in use, so that third is free).
            if (prompt != nullptr && tc_planes == 1 && gemm_tc_silu_fits(INTER, B)) {
                LAUNCH(launch_act_split(e->x, HIDDEN, HIDDEN, bf(w.ln2) + (size_t)l * HIDDEN, planes, prow, tc_planes, B, st, nullptr));
                bf16_raw* hplane = planes + (size_t)((e->cap + 127) / 128 * 128) * INTER;
                GemmTcSiluCall c{bf(w.wg) + (size_t)l * INTER * HIDDEN, bf(w.wu) + (size_t)l * INTER * HIDDEN, planes, hplane,
                                 INTER, B, HIDDEN, tc_planes, prow, prow, e->status};
                LAUNCH(launch_gemm_tc_silu(c, st));
                GemmTcCall d{bf(w.wd) + (size_t)l * HIDDEN * INTER, hplane, e->x, e->x, HIDDEN, HIDDEN, HIDDEN, B, INTER, 1, prow, e->status};
                LAUNCH(launch_gemm_tc(d, st));
                continue;
            }
            // hid = silu(rms(x, ln2) @ wg^T) * (rms(x, ln2) @ wu^T)
            const ZeroRows zf{{e->gate, e->up}, {INTER, INTER}, {INTER, INTER}};
            LAUNCH(launch_act_split(e->x, HIDDEN, HIDDEN, bf(w.ln2) + (size_t)l * HIDDEN, planes, prow, tc_planes, B, st,
                                    gemm_tc_splits_k(2 * INTER, B, HIDDEN) ? &zf : nullptr));
            {   // gate and up in one launch
                GemmTcGroupCall c{};
                c.n_groups = 2;
                c.w[0] = bf(w.wg) + (size_t)l * INTER * HIDDEN; c.n_rows[0] = INTER; c.out[0] = e->gate; c.ldo[0] = INTER;
                c.w[1] = bf(w.wu) + (size_t)l * INTER * HIDDEN; c.n_rows[1] = INTER; c.out[1] = e->up; c.ldo[1] = INTER;
                c.x_planes = planes; c.n_tok = B; c.K = HIDDEN; c.nsplit = tc_planes; c.plane_rows = prow; c.status = e->status;
                c.out_is_zero = 1;   // act_split has cleared the rows
                LAUNCH(launch_gemm_tc_group(c, st));
            }
            // x += (silu(gate) * up) @ wd^T
            LAUNCH(launch_silu_planes(e->gate, e->up, planes, prow, tc_planes, B, st));
            LAUNCH(gemm(bf(w.wd) + (size_t)l * HIDDEN * INTER, HIDDEN, INTER, e->x, HIDDEN, e->x, HIDDEN));
        } else {
            // x += attn @ wo^T
            g = GemvArgs{};
            g.seg[0] = {bf(w.wo) + (size_t)l * HIDDEN * Q_DIM, HIDDEN};
            g.x = e->attn; g.ldx = Q_DIM; g.out = e->x; g.ldo = HIDDEN; g.resid = e->x; g.ldr = HIDDEN;
            g.n_rows = HIDDEN; g.batch = B;
            LAUNCH(launch_gemv(2048, EPI_RESID, g, HIDDEN / 16, st));

            // hid = silu(rms(x, ln2) @ wg^T) * (rms(x, ln2) @ wu^T)
            g = GemvArgs{};
            g.seg[0] = {bf(w.wg) + (size_t)l * INTER * HIDDEN, INTER};
            g.w2 = bf(w.wu) + (size_t)l * INTER * HIDDEN;
            g.x = e->x; g.ldx = HIDDEN; g.gain = bf(w.ln2) + (size_t)l * HIDDEN;
            g.out = e->hid; g.ldo = INTER; g.n_rows = INTER; g.batch = B;
            LAUNCH(launch_gemv(1024, EPI_SILU, g, INTER / 8, st));

            // x += hid @ wd^T
            g = GemvArgs{};
            g.seg[0] = {bf(w.wd) + (size_t)l * HIDDEN * INTER, HIDDEN};
            g.x = e->hid; g.ldx = INTER; g.out = e->x; g.ldo = HIDDEN; g.resid = e->x; g.ldr = HIDDEN;
            g.n_rows = HIDDEN; g.batch = B;
            LAUNCH(launch_gemv(3072, EPI_RESID, g, HIDDEN / 16, st));
        }
    }
    // logits = rms(x, fnorm) @ embed^T ; next_token = argmax
    if (tc && row_argmax && V % 128 == 0 && (a->logits != nullptr || e->logits_tc != nullptr)) {
        float* logits = a->logits ? a->logits : e->logits_tc;
        LAUNCH(launch_act_split(e->x, HIDDEN, HIDDEN, bf(w.fnorm), planes, prow, tc_planes, B, st));
        LAUNCH(gemm(bf(w.embed), V, HIDDEN, logits, V, nullptr, 0));
        LAUNCH(launch_argmax_rows(logits, V, reinterpret_cast<long long*>(a->next_token), a->seq_len, append, B, st, arg_keys, arg_tickets));
    } else {
        // matrix-vector LM head: every sequence, or only the last token of a prompt
        const int nb = last_token_only ? 1 : B;
        if (nb > e->cfg.max_batch) return fail(e, Q3_ERR_INVALID, "decode: %d sequences exceed max_batch %d", nb, e->cfg.max_batch);
        GemvArgs g{};
        g.seg[0] = {bf(w.embed), V};
        g.x = e->x + (last_token_only ? (size_t)(B - 1) * HIDDEN : 0); g.ldx = HIDDEN; g.gain = bf(w.fnorm);
        g.out = a->logits; g.ldo = V; g.n_rows = V; g.batch = nb; g.pval = e->pval; g.pidx = e->pidx;
        int lm_grid = (V + 15) / 16;
        if (lm_grid > e->lm_grid) lm_grid = e->lm_grid;
        LAUNCH(launch_gemv(1024, EPI_LOGITS, g, lm_grid, st));
        LAUNCH(launch_argmax_final(e->pval, e->pidx, lm_grid, reinterpret_cast<long long*>(a->next_token), a->seq_len,
                                   last_token_only ? 0 : append, nb, st));
    }
#undef LAUNCH
    return Q3_OK;
}

extern "C" int q3_decode(q3_engine* e, const q3_decode_args* a, void* stream) {
    if (!e || !a) return fail(e, Q3_ERR_INVALID, "q3_decode: null argument");
    if (!e->have_weights) return fail(e, Q3_ERR_INVALID, "q3_decode: call q3_set_weights first");
    if (!e->rope) return fail(e, Q3_ERR_INVALID, "q3_decode: call q3_set_rope first");
    if (a->batch < 1 || a->batch > e->cfg.max_batch)
        return fail(e, Q3_ERR_INVALID, "q3_decode: batch %d outside 1..%d", a->batch, e->cfg.max_batch);
    if (a->max_len < 0 || a->max_len >= e->rope_n)
        return fail(e, Q3_ERR_INVALID, "q3_decode: max_len %d needs a RoPE table of more than %d rows (have %d)", a->max_len, a->max_len, e->rope_n);
    if (!a->token || !a->seq_k || !a->seq_v || !a->seq_layer_stride || !a->seq_len || !a->next_token)
        return fail(e, Q3_ERR_INVALID, "q3_decode: token, seq_k, seq_v, seq_layer_stride, seq_len and next_token are required");
    CU(e, cudaSetDevice(e->device));
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t path = a->flags & Q3_F_PATH_MASK;
    if (path == Q3_F_PATH_AUTO) path = persist_supports(e, a) ? Q3_F_PATH_PERSIST : Q3_F_PATH_LAYERED;
    if (path == Q3_F_PATH_PERSIST) {
        if (!persist_supports(e, a))
            return fail(e, Q3_ERR_UNSUPPORTED, "q3_decode: the persistent kernel does not serve batch %d at length %d", a->batch, a->max_len);
        return persist_decode(e, a, st);
    }
    if (path != Q3_F_PATH_LAYERED && path != Q3_F_PATH_FUSED) return fail(e, Q3_ERR_INVALID, "q3_decode: unknown path flag 0x%x", path);
    const bool layer_kernel = path == Q3_F_PATH_FUSED;
    if (!(a->flags & Q3_F_GRAPH)) return decode_layered(e, a, st, 3, nullptr, layer_kernel);

    // graph replay: the key is the argument block with max_len replaced by what it determines in the captured
    // launches: the split count and the padded chunk length (which also sizes the attention kernel's shared memory)
    q3_decode_args key = *a;
    key.max_len = 0;
    key.reserved = 0;
    const int ns = splits_for(e, a->batch, a->max_len);
    const int pad = chunk_pad_for(a->max_len, ns);
    auto* cache = graph_cache(e);
    GraphEntry* hit = nullptr;
    for (auto& g : *cache)
        if (g.n_splits == ns && g.chunk_pad == pad && !memcmp(&g.key, &key, sizeof(key))) { hit = &g; break; }
    if (!hit) {
        if (cache->size() >= 64) drop_graphs(e);
        cache->push_back(GraphEntry{key, ns, pad, 0, 0, nullptr});
        hit = &cache->back();
    }
    if (hit->exec) {
        CU(e, cudaGraphLaunch(hit->exec, st));
        e->launches += hit->launches;
        return Q3_OK;
    }
    if (hit->seen++ == 0) return decode_layered(e, a, st, 3, nullptr, layer_kernel);   // first use: plain launches
    const int64_t before = e->launches;
    // capture on the engine's own stream (the legacy default stream cannot be captured); nothing runs during capture
    cudaStream_t cs = static_cast<cudaStream_t>(e->capture_stream);
    CU(e, cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal));
    const int rc = decode_layered(e, a, cs, 3, nullptr, layer_kernel);
    cudaGraph_t graph = nullptr;
    const cudaError_t end = cudaStreamEndCapture(cs, &graph);
    if (rc != Q3_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (end != cudaSuccess || !graph) return fail(e, Q3_ERR_CUDA, "q3_decode: stream capture failed: %s", cudaGetErrorString(end));
    hit->launches = e->launches - before;
    e->launches = before;
    const cudaError_t inst = cudaGraphInstantiate(&hit->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (inst != cudaSuccess) { hit->exec = nullptr; return fail(e, Q3_ERR_CUDA, "q3_decode: cudaGraphInstantiate: %s", cudaGetErrorString(inst)); }
    CU(e, cudaGraphLaunch(hit->exec, st));
    e->launches += hit->launches;
    return Q3_OK;
}

// Activation planes of a prompt's GEMMs.  One: the activations enter the tensor cores rounded to bf16, like the weights and
// like the cached K/V rows that the prompt's later positions attend anyway.  Measured at 2048 tokens, full model, against
// the fp32 CPU checker: K/V rows rel-L2 6.6e-3 and logits 5.6e-3 with one plane, 4.0e-3 and 3.2e-3 with two (the cache
// rounding dominates both; the gates are 1e-2 and 2e-2); 5.6 ms against 7.3 ms.
constexpr int PREFILL_PLANES = 1;

// Prefill: the T prompt tokens run through the layered path as T one-token "sequences" of the same
// cache, token t at position t.  head_prep writes every K/V row into the cache before the attention
// kernels run, so token t attends rows [0, t) from the cache (rounded to bf16, as a later decode step
// will see them) and its own row in fp32: causal attention, the numerics of token-by-token decode.
// The projections are tensor-core GEMMs over PREFILL_PLANES bf16 planes of the activations.
static int prefill_batched(q3_engine* e, const q3_prefill_args* a, cudaStream_t st) {
    const int T = a->n_tokens;
    char* d = reinterpret_cast<char*>(e->pf_desc);
    uint64_t* seq_k = reinterpret_cast<uint64_t*>(d + 64);
    uint64_t* seq_v = seq_k + e->cap;
    long long* stride = reinterpret_cast<long long*>(seq_v + e->cap);
    int* len = reinterpret_cast<int*>(stride + e->cap);
    cudaError_t err = launch_prefill_desc(seq_k, seq_v, stride, len, reinterpret_cast<uint64_t>(a->kcache), reinterpret_cast<uint64_t>(a->vcache),
                                          (long long)a->cache_capacity * KV_DIM, T, st);
    ++e->launches;
    if (err != cudaSuccess) return fail(e, Q3_ERR_CUDA, "prefill descriptors: %s", cudaGetErrorString(err));
    q3_decode_args s{};
    s.batch = T; s.max_len = T - 1; s.flags = Q3_F_APPEND_KV | Q3_F_PATH_LAYERED;
    s.token = a->ids;
    s.seq_k = seq_k; s.seq_v = seq_v; s.seq_layer_stride = reinterpret_cast<const int64_t*>(stride); s.seq_len = len;
    s.logits = a->last_logits;
    s.next_token = a->next_token ? a->next_token : reinterpret_cast<int64_t*>(d + 32);
    const PrefillCtx ctx{a->kcache, a->vcache, (long long)a->cache_capacity * KV_DIM};
    return decode_layered(e, &s, st, PREFILL_PLANES, &ctx);
}

extern "C" int q3_linear_tc(const void* w, const float* x, float* out, const float* resid, int32_t n_rows, int32_t n_tok, int32_t K,
                            int32_t nsplit, void* planes, int64_t planes_bytes, void* stream) {
    if (!w || !x || !out || !planes) return fail(nullptr, Q3_ERR_INVALID, "q3_linear_tc: null argument");
    if (n_rows < 128 || n_rows % 128 || K < 128 || K % 64 || n_tok < 1 || nsplit < 1 || nsplit > 3)
        return fail(nullptr, Q3_ERR_INVALID, "q3_linear_tc: n_rows=%d (multiple of 128) n_tok=%d K=%d (multiple of 64) nsplit=%d (1..3)", n_rows, n_tok, K, nsplit);
    const int tile = n_tok <= 32 ? 32 : (n_tok <= 64 ? 64 : 128);
    const int plane_rows = (n_tok + tile - 1) / tile * tile;
    const int64_t need = (int64_t)nsplit * plane_rows * K * 2;
    if (planes_bytes < need) return fail(nullptr, Q3_ERR_INVALID, "q3_linear_tc: planes buffer holds %lld bytes, %lld needed", (long long)planes_bytes, (long long)need);
    cudaStream_t st = (cudaStream_t)stream;
    CU(nullptr, launch_act_split(x, K, K, nullptr, reinterpret_cast<bf16_raw*>(planes), plane_rows, nsplit, n_tok, st));
    GemmTcCall c{w, planes, out, resid, n_rows, n_rows, n_rows, n_tok, K, nsplit, plane_rows, nullptr};
    cudaError_t err = launch_gemm_tc(c, st);
    if (err != cudaSuccess) return fail(nullptr, Q3_ERR_CUDA, "q3_linear_tc: %s", cudaGetErrorString(err));
    return Q3_OK;
}

extern "C" int q3_prefill(q3_engine* e, const q3_prefill_args* a, void* stream) {
    if (!e || !a) return fail(e, Q3_ERR_INVALID, "q3_prefill: null argument");
    if (!e->have_weights) return fail(e, Q3_ERR_INVALID, "q3_prefill: call q3_set_weights first");
    if (!e->rope) return fail(e, Q3_ERR_INVALID, "q3_prefill: call q3_set_rope first");
    if (a->n_tokens < 1 || a->n_tokens > e->cfg.max_tokens)
        return fail(e, Q3_ERR_INVALID, "q3_prefill: n_tokens %d outside 1..max_tokens (%d)", a->n_tokens, e->cfg.max_tokens);
    if (a->cache_capacity < a->n_tokens) return fail(e, Q3_ERR_INVALID, "q3_prefill: cache_capacity %d < n_tokens %d", a->cache_capacity, a->n_tokens);
    if (a->n_tokens > e->rope_n) return fail(e, Q3_ERR_INVALID, "q3_prefill: RoPE table has %d rows, need %d", e->rope_n, a->n_tokens);
    if (!a->ids || !a->kcache || !a->vcache) return fail(e, Q3_ERR_INVALID, "q3_prefill: ids, kcache and vcache are required");
    CU(e, cudaSetDevice(e->device));
    return prefill_batched(e, a, (cudaStream_t)stream);
}
