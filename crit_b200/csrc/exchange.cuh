// The layout of a rank's exchange buffer and the two memory operations the peer exchange stands on (exchange.cu has the
// protocol).  In 4-byte words:
//   [0, 32)                              flags: flag[r] = the last step whose message from rank r has landed here
//   [32]                                 the ticket the blocks of a multi-block push count themselves on (own buffer only)
//   [64, 64 + 2 * world * stride)        messages: slot [step & 1][r] of `stride` floats (the message padded to 16 bytes)
#pragma once

#include "common.cuh"

namespace crit_b200 {

constexpr int EX_FLAG_WORDS = 64;
constexpr int EX_TICKET = 32;
constexpr int EX_MAX_WORLD = 32;
constexpr int EX_HEADER = 3;            // words after a fused message's payload: rank, step, rows (int32 bits)

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__host__ __device__ __forceinline__ int64_t ex_stride(int64_t floats) { return (floats + 3) / 4 * 4; }

// The fused exchange sends every float with its step beside it, as one 8-byte store: {value, step}.  An 8-byte store
// reaches a peer's memory whole, so a reader that finds the step it waits for has the value too: no fence orders data
// before a flag, and nothing waits for a write to be acknowledged across NVLink (a system-scope fence behind peer stores
// waits for exactly that, for microseconds).  A slot of the fused exchange is therefore twice a message's floats; the flags and headers of the plain
// exchange are not used by it.
__device__ __forceinline__ void ll_store(float* slot, int64_t idx, float v, int32_t step) {
    asm volatile("st.volatile.global.v2.b32 [%0], {%1, %2};" ::"l"(slot + 2 * idx), "r"(__float_as_uint(v)), "r"(step) : "memory");
}
__device__ __forceinline__ bool ll_load(const float* slot, int64_t idx, int32_t step, float& v) {
    uint32_t value, stamp;
    asm volatile("ld.volatile.global.v2.b32 {%0, %1}, [%2];" : "=r"(value), "=r"(stamp) : "l"(slot + 2 * idx) : "memory");
    v = __uint_as_float(value);
    return (int32_t)stamp == step;
}
// Element idx of every rank's message of `step` in this rank's own buffer (slot0: rank 0's slot, `stride` floats a
// slot), into v[0 .. world): false when one of them had not arrived after wait_ns.
__device__ __forceinline__ bool ll_gather(const float* slot0, int64_t stride, int world, int64_t idx, int32_t step, uint64_t wait_ns,
                                          float* v) {
    uint32_t missing = world >= 32 ? 0xffffffffu : ((1u << world) - 1u);
    uint64_t t0 = 0;
    while (true) {
        for (int r = 0; r < world; ++r)
            if ((missing >> r) & 1u) {
                float got;
                if (ll_load(slot0 + r * stride, idx, step, got)) v[r] = got, missing &= ~(1u << r);
            }
        if (!missing) return true;
        if (!t0) t0 = global_ns();
        else if (global_ns() - t0 > wait_ns) return false;
    }
}
// Slot [step & 1][rank] of the buffer at `buffer`.
__device__ __forceinline__ float* ex_slot(uint64_t buffer, int32_t step, int world, int rank, int64_t stride) {
    return reinterpret_cast<float*>(buffer) + EX_FLAG_WORDS + ((int64_t)(step & 1) * world + rank) * stride;
}
__device__ __forceinline__ int32_t ld_relaxed_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Waits (at most wait_ns) until ONE rank's flag is at `step`, then fences (acquire, system scope): the threads of a block
// each wait for one rank, so the flags are polled side by side (acquire loads one after another, by one thread, cost a
// memory round trip per rank).
__device__ __forceinline__ bool ex_wait_flag(const int32_t* flag, int32_t step, uint64_t wait_ns) {
    const uint64_t t0 = global_ns();
    bool ok = ld_relaxed_sys(flag) - step >= 0;
    while (!ok && global_ns() - t0 < wait_ns) ok = ld_relaxed_sys(flag) - step >= 0;
    __threadfence_system();
    return ok;
}

}  // namespace crit_b200
