// Chunked prefill (placeholder until the tensor-core kernel lands): refuses loudly.
#include "common.cuh"

extern "C" __attribute__((visibility("default"))) int crit_b200_prefill(const crit_b200_prefill_params* params, void* stream) {
    (void)params;
    (void)stream;
    return CRIT_B200_EUNSUPPORTED;
}
