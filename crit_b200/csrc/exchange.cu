// The exchange of the shards' partials over NVLink peer memory, without a collective library on the path.
//
// Every rank owns one exchange buffer that every other rank of the node has mapped (symmetric memory: the caller makes
// and maps the buffers and passes this GPU's view of all of them).  Layout of a buffer, in 4-byte words:
//   [0, 64)                              flags: flag[r] = the last step whose message from rank r has landed here
//   [64, 64 + 2 * world * stride)        messages: slot [step & 1][r] of `stride` floats (the message padded to 16 bytes)
// A step is two launches on every rank, in stream order:
//   push   one more on this rank's step counter (a device word: the step is captured in a CUDA graph), then this rank's
//          message is STORED into slot [step & 1][rank] of every rank's buffer (plain peer stores: posted writes over
//          NVLink, 16 bytes a thread), a system-scope fence, and flag[rank] = step in every buffer;
//   wait   waits (bounded in time) until all `world` flags of this rank's OWN buffer are at the step, then copies the
//          `world` messages of slot [step & 1] into a fixed local array for the merge-of-shards kernel.
// A push never waits, so no rank's progress depends on another rank's kernel having started; a wait that runs out sets the
// status word and copies nothing (the host reads the status and does not publish).  Slot [step & 1] of rank y is written
// again at step + 2, which rank x starts only after its own wait of step + 1, which needed y's push of step + 1, which y
// launched after its wait of `step` had read the slot: no message is overwritten before it was read.
// Loads never touch a peer's memory here: a rank reads only what the others stored into its own buffer.
// Reference: the reference states the technique on the host only (inference/partitioned-attention/README.md, "all-gather
// normalizers"); its merge is inference/partitioned-attention/plugin.py:52-64.
#include "common.cuh"

namespace crit_b200 {

constexpr int EX_FLAG_WORDS = 64;

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(1024) shard_push_kernel(const crit_b200_exchange_params p) {
    __shared__ int32_t step_now;
    if (threadIdx.x == 0) step_now = ++*p.step;
    __syncthreads();
    const int32_t step = step_now;
    const int64_t stride = (p.floats + 3) / 4 * 4;
    const int64_t vec = stride / 4;
    const float4* src = reinterpret_cast<const float4*>(p.mine);
    for (int r = 0; r < p.world; ++r) {
        float* base = reinterpret_cast<float*>(p.peers[r]) + EX_FLAG_WORDS + ((int64_t)(step & 1) * p.world + p.rank) * stride;
        float4* dst = reinterpret_cast<float4*>(base);
        for (int64_t i = threadIdx.x; i < vec; i += blockDim.x) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (4 * i + 3 < p.floats) {
                v = src[i];
            } else {
                float t[4] = {0.f, 0.f, 0.f, 0.f};
                for (int e = 0; e < 4; ++e)
                    if (4 * i + e < p.floats) t[e] = p.mine[4 * i + e];
                v = make_float4(t[0], t[1], t[2], t[3]);
            }
            dst[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.world) st_release_sys(reinterpret_cast<int32_t*>(p.peers[threadIdx.x]) + p.rank, step);
}

__global__ void __launch_bounds__(256) shard_wait_kernel(const crit_b200_exchange_params p) {
    __shared__ int landed;
    const int32_t step = *p.step;
    const int32_t* flags = reinterpret_cast<const int32_t*>(p.peers[p.rank]);
    if (threadIdx.x == 0) {
        const uint64_t t0 = global_ns();
        int ok = 0;
        do {
            ok = 1;
            for (int r = 0; r < p.world; ++r)
                if (ld_acquire_sys(flags + r) - step < 0) ok = 0;
        } while (!ok && global_ns() - t0 < (uint64_t)p.wait_ns);
        landed = ok;
        if (!ok && p.status) atomicExch(p.status, 0x800 + p.rank);
    }
    __syncthreads();
    if (!landed) return;
    const int64_t stride = (p.floats + 3) / 4 * 4;
    const float* slot = reinterpret_cast<const float*>(p.peers[p.rank]) + EX_FLAG_WORDS + (int64_t)(step & 1) * p.world * stride;
    const int64_t total = (int64_t)p.world * p.floats;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / p.floats, at = i - r * p.floats;
        p.gathered[i] = slot[r * stride + at];
    }
}

}  // namespace crit_b200

using namespace crit_b200;

static int check_exchange(const crit_b200_exchange_params& p) {
    if (!p.mine || !p.peers || !p.step || !p.gathered) return CRIT_B200_EINVAL;
    if (p.floats < 1 || p.world < 1 || p.world > 32 || p.rank < 0 || p.rank >= p.world || p.wait_ns < 1) return CRIT_B200_EINVAL;
    if (!aligned(p.mine, 16)) return CRIT_B200_EALIGN;
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_shard_push(const crit_b200_exchange_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_exchange_params p = *params;
    if (int e = check_exchange(p)) return e;
    shard_push_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(p);
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_shard_wait(const crit_b200_exchange_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_exchange_params p = *params;
    if (int e = check_exchange(p)) return e;
    const int64_t total = (int64_t)p.world * p.floats;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 64 ? (total + 255) / 256 : 64);
    shard_wait_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p);
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int64_t crit_b200_exchange_bytes(int32_t world, int64_t floats) {
    if (world < 1 || floats < 1) return CRIT_B200_EINVAL;
    return (EX_FLAG_WORDS + 2 * (int64_t)world * ((floats + 3) / 4 * 4)) * 4;
}
