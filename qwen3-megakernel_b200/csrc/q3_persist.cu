// Persistent cooperative decode kernel (placeholder until the kernel lands).
#include "q3_engine.h"

namespace q3 {
int persist_setup(q3_engine* e) { e->p_grid = 0; e->p_threads = 0; e->p_smem = 0; return Q3_OK; }
void persist_teardown(q3_engine*) {}
bool persist_supports(const q3_engine*, const q3_decode_args*) { return false; }
int persist_decode(q3_engine* e, const q3_decode_args*, cudaStream_t) { return engine_fail(e, Q3_ERR_UNSUPPORTED, "persistent kernel not built"); }
}  // namespace q3
