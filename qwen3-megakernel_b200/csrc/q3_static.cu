// q3_decode_noalloc: a decode step for callers that are not allowed to allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a decode step: a
// plugin running inside another runtime's memory budget, a process whose device memory is fully
// pre-carved by a serving framework, or code between the begin and end of work that forbids
// allocation calls.  q3_create allocates the engine's scratch, so those callers cannot use an engine.
// This entry point needs none: the scratch of the layered decode path lives in a file-scope device
// array, sized for at most Q3_NOALLOC_MAX_BATCH sequences, and every GPU that loads the library
// holds those bytes until the process exits.
//
// The step itself is the layered path of q3_decode, kernel for kernel; only where the scratch comes
// from differs.  All calls share the one array: it keeps the previous call's contents (every buffer is
// fully rewritten before it is read, the status words are cleared on the stream at the start of each
// call), and two calls that overlap on the GPU would race on it.
#include <cstring>
#include <mutex>

#include "q3_engine.h"

using namespace q3;

namespace {

constexpr int NA_BATCH = 2;        // sequences per call
constexpr int NA_SPLITS = 16;      // attention splits the partial buffer holds
constexpr int NA_LM_GRID = 148 * 8;

struct Scratch {
    float x[NA_BATCH * HIDDEN];
    float qkv[NA_BATCH * QKV_DIM];
    float attn[NA_BATCH * Q_DIM];
    float hid[NA_BATCH * INTER];
    float part[NA_BATCH * Q_HEADS * NA_SPLITS * ATTN_PART_STRIDE];
    float pval[NA_BATCH * NA_LM_GRID];
    int pidx[NA_BATCH * NA_LM_GRID];
    uint32_t status[Q3_STATUS_WORDS];
};

// About 0.4 MB.  In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(Scratch)];

constexpr int MAX_DEVICES = 64;
Scratch* g_device_ptr[MAX_DEVICES] = {};
int g_sm_count[MAX_DEVICES] = {};
std::mutex g_setup_lock;   // the per-device set-up may be reached from several host threads at once

// Resolve (once per device, with that device current) the device address of the array.  Returns Q3_OK or an
// error code with its message recorded.
int scratch_of_current_device(int* dev_out, Scratch** out) {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return engine_fail(nullptr, Q3_ERR_CUDA, "q3_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(err));
    *dev_out = dev;
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_device_ptr[dev]) {
        int major = 0, sms = 0;
        err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return engine_fail(nullptr, Q3_ERR_CUDA, "q3_decode_noalloc: cudaDeviceGetAttribute: %s", cudaGetErrorString(err));
        if (major != 10) return engine_fail(nullptr, Q3_ERR_UNSUPPORTED, "q3_decode_noalloc: device %d is sm_%dx; this library holds sm_100a code only", dev, major);
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess || !ptr) return engine_fail(nullptr, Q3_ERR_CUDA, "q3_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
        g_sm_count[dev] = sms;
        g_device_ptr[dev] = static_cast<Scratch*>(ptr);
    }
    *out = g_device_ptr[dev];
    return Q3_OK;
}

}  // namespace

extern "C" int q3_noalloc_status(void* stream, uint32_t* words, int32_t n) {
    int dev = -1;
    Scratch* s = nullptr;
    const int rc = scratch_of_current_device(&dev, &s);
    if (rc != Q3_OK) return rc;
    uint32_t h[Q3_STATUS_WORDS];
    cudaError_t err = cudaStreamSynchronize((cudaStream_t)stream);
    if (err == cudaSuccess) err = cudaMemcpy(h, s->status, sizeof(h), cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) return engine_fail(nullptr, Q3_ERR_CUDA, "q3_noalloc_status: %s", cudaGetErrorString(err));
    for (int i = 0; words && i < n && i < Q3_STATUS_WORDS; ++i) words[i] = h[i];
    if (h[0] == 0) return Q3_OK;
    return engine_fail(nullptr, Q3_ERR_DEVICE_WAIT, "device status: code %u at site %u, block %u, value %u", h[0], h[1], h[2], h[3]);
}

extern "C" int q3_decode_noalloc(const q3_weights* w, const float* rope, int32_t rope_positions, int32_t n_layers, int32_t vocab,
                                 const q3_decode_args* a, void* stream) {
    if (!w || !rope || !a) return engine_fail(nullptr, Q3_ERR_INVALID, "q3_decode_noalloc: null argument");
    if (n_layers < 1 || vocab < 1 || rope_positions < 1)
        return engine_fail(nullptr, Q3_ERR_INVALID, "q3_decode_noalloc: n_layers=%d vocab=%d rope_positions=%d out of range", n_layers, vocab, rope_positions);
    if (a->batch < 1 || a->batch > NA_BATCH)
        return engine_fail(nullptr, Q3_ERR_INVALID, "q3_decode_noalloc: batch %d exceeds the static scratch (at most %d sequences per call)", a->batch, NA_BATCH);
    if (a->max_len < 0 || a->max_len >= rope_positions)
        return engine_fail(nullptr, Q3_ERR_INVALID, "q3_decode_noalloc: max_len %d needs a RoPE table of more than %d rows (have %d)", a->max_len, a->max_len, rope_positions);
    if ((a->flags & Q3_F_PATH_MASK) == Q3_F_PATH_PERSIST)
        return engine_fail(nullptr, Q3_ERR_UNSUPPORTED, "q3_decode_noalloc: only the layered path runs without an engine");
    if (!a->token || !a->seq_k || !a->seq_v || !a->seq_layer_stride || !a->seq_len || !a->next_token)
        return engine_fail(nullptr, Q3_ERR_INVALID, "q3_decode_noalloc: token, seq_k, seq_v, seq_layer_stride, seq_len and next_token are required");
    const void* const* wp = reinterpret_cast<const void* const*>(w);
    for (int i = 0; i < 13; ++i)
        if (!wp[i] || (reinterpret_cast<uintptr_t>(wp[i]) & 15))
            return engine_fail(nullptr, Q3_ERR_INVALID, "q3_decode_noalloc: weight %d is null or not 16-byte aligned", i);

    int dev = -1;
    Scratch* s = nullptr;
    const int rc0 = scratch_of_current_device(&dev, &s);   // the first call on a device resolves the array's address
    if (rc0 != Q3_OK) return rc0;
    cudaError_t err;

    // A host-side engine record that points into the static array; nothing is allocated.
    q3_engine e;
    memset(&e, 0, sizeof(e));
    e.device = dev;
    e.cfg.n_layers = n_layers; e.cfg.vocab = vocab; e.cfg.max_batch = NA_BATCH;
    e.w = *w; e.have_weights = 1;
    e.rope = rope; e.rope_n = rope_positions;
    e.sm_count = g_sm_count[dev];
    e.max_splits = NA_SPLITS;
    e.lm_grid = NA_LM_GRID;
    e.x = s->x; e.qkv = s->qkv; e.attn = s->attn; e.hid = s->hid; e.part = s->part; e.pval = s->pval; e.pidx = s->pidx;
    e.status = s->status;
    cudaStream_t st = (cudaStream_t)stream;
    err = cudaMemsetAsync(s->status, 0, sizeof(s->status), st);   // must start at zero
    if (err != cudaSuccess) return engine_fail(nullptr, Q3_ERR_CUDA, "q3_decode_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(err));
    const int rc = decode_layered(&e, a, st);
    if (rc != Q3_OK) engine_fail(nullptr, rc, "q3_decode_noalloc: %s", e.err);
    return rc;
}
