// Housekeeping entry points of the C ABI.
#include "common.cuh"

extern "C" __attribute__((visibility("default"))) int crit_b200_abi_version(void) { return CRIT_B200_ABI_VERSION; }

extern "C" __attribute__((visibility("default"))) int crit_b200_params_size(int32_t which) {
    switch (which) {
        case 0: return (int)sizeof(crit_b200_append_params);
        case 1: return (int)sizeof(crit_b200_gather_params);
        case 2: return (int)sizeof(crit_b200_slots_params);
        case 3: return (int)sizeof(crit_b200_attend_params);
        case 4: return (int)sizeof(crit_b200_merge_shards_params);
        case 5: return (int)sizeof(crit_b200_prefill_params);
        case 6: return (int)sizeof(crit_b200_exchange_params);
        case 7: return (int)sizeof(crit_b200_move_params);
        case 8: return (int)sizeof(crit_b200_compact_params);
        default: return CRIT_B200_EINVAL;
    }
}

extern "C" __attribute__((visibility("default"))) const char* crit_b200_error(int32_t code) {
    switch (code) {
        case 0: return "success";
        case CRIT_B200_EINVAL: return "crit_b200: a size, stride or pointer the call cannot take";
        case CRIT_B200_EUNSUPPORTED: return "crit_b200: no kernel was built for this geometry (head widths 64, 128 or 256 with keys and values of one width, pages of a multiple of 16 positions, page kinds bf16, fp16, fp8, fp8:row, int8, fp8:page)";
        case CRIT_B200_EWORKSPACE: return "crit_b200: the workspace is smaller than partial_rows * q_heads * max_splits * (value_dim + 2) floats";
        case CRIT_B200_EALIGN: return "crit_b200: q and pages are read in 16-byte vectors and outputs written in 8-byte ones: a pointer or stride is not aligned for that";
        case CRIT_B200_ESTATIC: return "crit_b200: crit_b200_attend_static holds 4,194,304 floats (16 MiB) of partials; this launch needs more (partial_rows * q_heads * max_splits * (value_dim + 2)): raise chunk or attend fewer rows a call";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "crit_b200: unknown error";
    }
}

extern "C" __attribute__((visibility("default"))) int crit_b200_device_sms(void) {
    int device = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return e == cudaSuccess ? sms : -(int)e - 100;
}
