// The persistent per-layer kernel of the batched decode path (tcgen05 GEMM phases with the element-wise work between
// them fused into the operand staging); see q3_layer_tc.cu.
#pragma once
#include <cuda_runtime.h>

struct q3_engine;

namespace q3 {

// FIRST: clear the accumulated outputs, then q/k/v of layer 0 from the embedded tokens.
// MID:   Wo + residual, gate/up, down + residual of `layer`, then q/k/v of `layer + 1`.
// LAST:  the same without a next layer.
enum { LK_MODE_FIRST = 0, LK_MODE_MID = 1, LK_MODE_LAST = 2 };

// [2][64] fp32 row sums of squares; at byte 512 two 64-bit barrier words; at byte 1024 [64][8] arrival counters of the
// attention splits of a (sequence, kv head)
constexpr int LK_STATE_BYTES = 1024 + 64 * 8 * 4;
constexpr int LK_STATE_MERGE_OFFSET = 1024;

// whether the engine's batched decode step of `batch` sequences can run on the layer kernel
bool layer_tc_supports(const q3_engine* e, int batch);
cudaError_t launch_layer_tc(q3_engine* e, int mode, int layer, int n_tok, cudaStream_t st);

}  // namespace q3
