// Argument blocks and launchers of the layered (one launch per phase) decode path.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace q3 {

typedef unsigned short bf16_raw;

enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SILU = 2, EPI_LOGITS = 3 };

// floats per (sequence, head, split) attention partial: [0] max, [1] sum, [4..132) unnormalised output
constexpr int ATTN_PART_STRIDE = 132;
constexpr int ATTN_CHUNK_MAX = 4096;          // positions one block of the split-attention kernel takes (its scores live in shared memory)

struct GemvSeg {
    const bf16_raw* w;  // [rows, K] row-major bf16
    int rows;
};

struct GemvArgs {
    GemvSeg seg[3];        // weight rows: seg[0] rows first, then seg[1], then seg[2]
    const bf16_raw* w2;    // EPI_SILU: the "up" matrix paired row-by-row with seg[0] ("gate")
    const float* x;        // activations [batch, K], row stride ldx
    int ldx;
    const bf16_raw* gain;  // RMSNorm gain [K], or nullptr for no normalisation
    float* out;            // [batch, ldo]
    int ldo;
    const float* resid;    // EPI_RESID: out = resid + acc
    int ldr;
    int n_rows;
    int batch;
    float* pval;           // EPI_LOGITS: per-block argmax partials [batch, gridDim.x]
    int* pidx;
};

struct HeadPrepArgs {
    float* qkv;                       // [batch, 4096] fp32: q | k | v, q and k rewritten in place
    const bf16_raw* qn;               // [L, 128]
    const bf16_raw* kn;               // [L, 128]
    const float* rope;                // [positions, 128]: cos(64) | sin(64)
    const int* seq_len;               // [batch]
    bf16_raw* k_write;                // [batch, L, 8, 128] or nullptr
    bf16_raw* v_write;
    const uint64_t* seq_k;            // cache addresses, used when append != 0
    const uint64_t* seq_v;
    const long long* seq_layer_stride;
    int layer, n_layers, append;
    int len_bound;                    // lengths are clamped to [0, len_bound] (the embed kernel reports a longer cache)
    int skip_k_store;                 // the prepared k rows are only needed as bf16 cache rows (a long prompt's attention reads the cache): leave qkv's k as it is
};

struct AttnArgs {
    const float* qkv;                 // [batch, 4096] after head_prep
    const uint64_t* seq_k;
    const uint64_t* seq_v;
    const long long* seq_layer_stride;
    const int* seq_len;
    float* part;                      // [batch, 16, n_splits, ATTN_PART_STRIDE]
    int layer, n_splits;
    int chunk_pad;                    // positions per split, rounded up to 32: what the host's length bound allows (<= ATTN_CHUNK_MAX)
    // fused head preparation (decode steps): `qkv` holds the raw projections and every block normalises and rotates the
    // q heads and the k row of its (sequence, kv head) itself; the block of split 0 stores the new K/V rows
    int fused_prep;                   // 0: qkv was prepared by head_prep_kernel
    const bf16_raw* qn;
    const bf16_raw* kn;
    const float* rope;
    bf16_raw* k_write;
    bf16_raw* v_write;
    int n_layers, append;
    int len_bound;                    // n_splits * chunk_pad - 1 and the RoPE table's last row, whichever is smaller
    // fused_prep only: per-sequence sums of squares of the vector the q/k/v projections were taken of, when the producer
    // left the RMS norm's scale rsqrt(ssq / 1024 + eps) to this kernel (the layer kernel does); nullptr: already applied
    const float* row_ssq;
    // the block that finishes a (sequence, kv head) last merges its splits into merged[b, 2048] (nullptr: a separate
    // merge kernel follows); merge_count[b * 8 + g] counts the arrivals and is left at zero
    float* merged;
    int* merge_count;
    // a launch of ONE split needs no merge: its blocks write the normalised output as the three bf16 planes (hi, mid, lo)
    // [3][plane_rows][2048] the Wo GEMM reads
    bf16_raw* planes_out;
    int plane_rows;
};

cudaError_t launch_gemv(int K, int epi, const GemvArgs& a, int grid_x, cudaStream_t st);
cudaError_t launch_embed(const long long* token, const bf16_raw* embed, int vocab, float* x, uint32_t* status, int batch, cudaStream_t st,
                         unsigned long long* argmax_keys = nullptr, unsigned* argmax_tickets = nullptr,
                         const int* seq_len = nullptr, int len_bound = 0);
cudaError_t launch_argmax_final(const float* pval, const int* pidx, int nblk, long long* next_token, int* seq_len, int append, int batch, cudaStream_t st);
cudaError_t launch_head_prep(const HeadPrepArgs& a, int batch, cudaStream_t st);
cudaError_t launch_attn(const AttnArgs& a, float* attn_out, int batch, cudaStream_t st);
cudaError_t launch_attn_split(const AttnArgs& a, int batch, cudaStream_t st);   // the split kernel alone: partials only
cudaError_t launch_attn_mma(const AttnArgs& a, int batch, cudaStream_t st);     // q3_attn_mma.cu: the split kernel on mma.sync + cp.async
cudaError_t launch_attn_planes(const AttnArgs& a, bf16_raw* planes, int plane_rows, int nsplit, int batch, cudaStream_t st);
cudaError_t launch_silu_planes(const float* g, const float* u, bf16_raw* planes, int plane_rows, int nsplit, int n_tok, cudaStream_t st);
// up to two fp32 buffers whose first n_tok rows act_split clears on the side (the outputs of the split-K GEMM that follows)
struct ZeroRows {
    float* ptr[2];
    int ld[2], cols[2];
};
cudaError_t launch_act_split(const float* x, int ldx, int K, const bf16_raw* gain, bf16_raw* planes, int plane_rows, int nsplit, int n_tok, cudaStream_t st,
                             const ZeroRows* zero = nullptr);
cudaError_t launch_prefill_desc(uint64_t* seq_k, uint64_t* seq_v, long long* stride, int* len, uint64_t k, uint64_t v, long long s, int n, cudaStream_t st);
cudaError_t launch_silu_mul(const float* g, const float* u, float* h, size_t n, cudaStream_t st);
cudaError_t launch_argmax_rows(const float* logits, int vocab, long long* next_token, int* seq_len, int append, int n_tok, cudaStream_t st,
                               unsigned long long* keys, unsigned* tickets);

}  // namespace q3
