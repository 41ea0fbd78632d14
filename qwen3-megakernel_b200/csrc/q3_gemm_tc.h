// Tensor-core GEMM (tcgen05 + TMEM + TMA) used by prefill and large-batch decode.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

struct CUtensorMap_st;   // <cuda.h>'s tensor map

namespace q3 {

enum { TC_EPI_STORE = 0, TC_EPI_RESID = 1, TC_EPI_ATOMIC = 2 };

// device-side parameters
struct GemmTcParams {
    float* out;            // [n_tok, ldo] fp32; element (t, n) at out[t * ldo + n]
    const float* resid;    // TC_EPI_RESID: out = resid + acc (may alias out)
    int ldo, ldr;
    int n_rows;            // weight rows (multiple of 128)
    int n_tok;             // valid tokens
    int K;                 // multiple of 64
    int nsplit;            // activation planes (1..3)
    int plane_rows;        // rows per plane in the activation tensor (multiple of the token tile)
    int stages;
    int kb_per_split;      // k blocks (of 64) each grid.z slice covers
    int epi;
    uint32_t* status;
    // grouped launches: grid.x tiles [0, g_tiles[0]) belong to matrix 0, the next g_tiles[1] to matrix 1, ...
    int out_is_zero;       // host side only: skip the memset before a split-K launch
    int n_groups;          // 0 or 1: a single matrix (tm_w0, `out`, `ldo`)
    int g_tiles[3];
    float* g_out[3];
    int g_ldo[3];
};

// host-side call
struct GemmTcCall {
    const void* w;         // bf16 [n_rows, K] row-major
    const void* x_planes;  // bf16 [nsplit, plane_rows, K]: fp32 activations split as hi (+ mid (+ lo)); rows >= n_tok may hold anything (their columns of the product are never stored)
    float* out;
    const float* resid;    // nullptr: plain store
    int ldo, ldr;
    int n_rows, n_tok, K, nsplit, plane_rows;
    uint32_t* status;
};

cudaError_t launch_gemm_tc(const GemmTcCall& c, cudaStream_t st);

// Up to three weight matrices with the same K against the same activation planes in ONE launch (q/k/v, gate/up):
// group g writes out[g][t * ldo[g] + n] for its own rows n.  Plain stores or split-K atomics onto zeros; no residual.
struct GemmTcGroupCall {
    int n_groups;          // 1..3
    const void* w[3];      // bf16 [n_rows[g], K] row-major
    int n_rows[3];         // multiples of 128
    float* out[3];
    int ldo[3];
    const void* x_planes;
    int n_tok, K, nsplit, plane_rows;
    uint32_t* status;
    int out_is_zero;       // the caller has cleared the outputs: a split-K launch adds into them without a memset
};
cudaError_t launch_gemm_tc_group(const GemmTcGroupCall& c, cudaStream_t st);

// Prompts: out_plane = the bf16 plane of silu(x wg^T) * (x wu^T), both products in one work item of the persistent kernel,
// for the down GEMM to read; no fp32 gate / up matrices.  gemm_tc_silu_fits: the items occupy at least 0.6 of the SMs.
struct GemmTcSiluCall {
    const void* wg;        // bf16 [n_rows, K]
    const void* wu;        // bf16 [n_rows, K]
    const void* x_planes;  // bf16 [nsplit, plane_rows, K]
    void* out_plane;       // bf16 [out_rows, n_rows]; must not overlap x_planes; rows n_tok.. are written as zeros
    int n_rows, n_tok, K, nsplit, plane_rows, out_rows;
    uint32_t* status;
};
bool gemm_tc_silu_fits(int n_rows, int n_tok);
cudaError_t launch_gemm_tc_silu(const GemmTcSiluCall& c, cudaStream_t st);

// Whether a launch of n_rows weight rows (all groups together) against n_tok tokens will slice K, i.e. add partial tiles
// into an output that must hold zeros (or the residual) beforehand.
bool gemm_tc_splits_k(int n_rows, int n_tok, int K);

// A cached tensor map of a row-major bf16 matrix [rows, cols]: boxes of 64 columns x box_rows rows, 128-byte swizzle,
// out-of-range rows read as zeros.  (CUtensorMap is declared by <cuda.h>, which the caller includes.)
bool tc_cached_map(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, ::CUtensorMap_st* out);

}  // namespace q3
