// Tensor-core (tcgen05 / TMEM / TMA) chunked prefill. Placeholder translation unit until the kernel lands: reports
// "not supported" so the C ABI routes nothing here.
#include "common.cuh"

namespace pgb {

bool prefill_tc_supported(int, int, bool) { return false; }

int prefill_tc_launch(const PrefillArgs &, int, int, cudaStream_t) { return PGB_ERR_UNSUPPORTED_DIM; }

}  // namespace pgb
