// The exchange of the shards' partials over NVLink peer memory, without a collective library on the path.
//
// Every rank owns one exchange buffer that every other rank of the node has mapped (symmetric memory: the caller makes
// and maps the buffers and passes this GPU's view of all of them); exchange.cuh has its layout.  A step is two launches
// on every rank, in stream order:
//   push   one more on this rank's step counter (a device word: the step is captured in a CUDA graph), then this rank's
//          message is STORED into slot [step & 1][rank] of every rank's buffer (plain peer stores: posted writes over
//          NVLink, 16 bytes a thread), a system-scope fence, and flag[rank] = step in every buffer;
//   wait   waits (bounded in time) until all `world` flags of this rank's OWN buffer are at the step, then reads the
//          `world` messages of slot [step & 1].
// Two forms of each.  The plain pair moves a message the caller packed (crit_b200_shard_push) and copies the messages
// to a fixed local array for a later merge (crit_b200_shard_wait).  The fused pair does the arithmetic either side of
// the wire in the same launches: crit_b200_merge_push (decode.cu) folds this rank's split-K partials and stores each
// (token, head)'s result straight into the peers' slots, and crit_b200_wait_merge here merges the ranks' partials out
// of this rank's own buffer into the step's output as soon as the flags are up.
// The fused pair stores every float with its step beside it in one 8-byte store (exchange.cuh): a float is valid when its
// step is the reader's, so its exchange needs no flag, no fence and no header, and costs one NVLink write.
// A push never waits, so no rank's progress depends on another rank's kernel having started; a wait that runs out sets
// the status word (0x800 + rank) and writes nothing of the pair concerned (the plain wait also refuses a message whose
// header is not the step's: 0x900 + the sender): the host reads the status and does not publish.  After either, the exchange is out of step: the buffers are
// zeroed and the ranks synchronised again before the next step (slot [step & 1] of rank y is written again at step + 2,
// which rank x starts only after its own wait of step + 1 saw y's push of step + 1, which y launched after its wait of
// `step` had read the slot; that chain holds only while every wait succeeds).
// Loads never touch a peer's memory here: a rank reads only what the others stored into its own buffer.
// Reference: the reference states the technique on the host only (inference/partitioned-attention/README.md, "all-gather
// normalizers"); its merge is inference/partitioned-attention/plugin.py:52-64.
#include "exchange.cuh"

namespace crit_b200 {

__global__ void __launch_bounds__(1024) shard_push_kernel(const crit_b200_exchange_params p) {
    __shared__ int32_t step_now;
    if (threadIdx.x == 0) step_now = ++*p.step;
    __syncthreads();
    const int32_t step = step_now;
    const int64_t stride = ex_stride(p.floats);
    const int64_t vec = stride / 4;
    const float4* src = reinterpret_cast<const float4*>(p.mine);
    for (int r = 0; r < p.world; ++r) {
        float4* dst = reinterpret_cast<float4*>(ex_slot(p.peers[r], step, p.world, p.rank, stride));
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

// One block: its first `world` threads wait, one rank each, then every thread copies.  (Several blocks, each with its own
// wait, could disagree near the limit and leave `gathered` half written beside the status word.)
__global__ void __launch_bounds__(1024) shard_wait_kernel(const crit_b200_exchange_params p) {
    const int32_t step = *p.step;
    const uint64_t own = p.peers[p.rank];
    bool ok = true;
    if (threadIdx.x < p.world) {            // thread r waits for rank r
        ok = ex_wait_flag(reinterpret_cast<const int32_t*>(own) + threadIdx.x, step, (uint64_t)p.wait_ns);
        if (!ok && p.status) atomicExch(p.status, 0x800 + p.rank);
    }
    if (!__syncthreads_and(ok ? 1 : 0)) return;
    const int64_t stride = ex_stride(p.floats);
    const float* slot = ex_slot(own, step, p.world, 0, stride);
    const int64_t total = (int64_t)p.world * p.floats;
    for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
        const int64_t r = i / p.floats, at = i - r * p.floats;
        p.gathered[i] = slot[r * stride + at];
    }
}

// The merge of the ranks' partials, read where the peers stored them (the second launch of the fused exchange where one
// launch does not hold the step: crit_b200_exchange_merge).  A message is [n][dim] outputs then [n] log-sum-exps, every
// float with its step beside it (exchange.cuh).  Block = one (token, head): thread 0 gathers the ranks' log-sum-exps
// (a bounded wait per float), thread c column c of every rank: top = max lse over the ranks, w = exp(lse - top) (0 for
// -inf), out = sum w o / sum w in rank order, lse = top + log(sum w); a (token, head) no rank saw gets zeros and -inf.
// A float that never arrives: the status word (0x800 + rank), and nothing of its pair is written.
// Reference: inference/partitioned-attention/plugin.py:52-64.
template <typename TOUT>
__global__ void __launch_bounds__(256) wait_merge_kernel(const crit_b200_exchange_params p, const crit_b200_merge_shards_params m) {
    __shared__ float parts_lse[EX_MAX_WORLD];
    const int32_t step = *p.step;
    const int64_t stride = 2 * ex_stride(p.floats);
    const float* own = ex_slot(p.peers[p.rank], step, p.world, 0, stride);
    const int64_t n = m.n, entry = blockIdx.x;
    const int dim = m.dim;
    bool ok = true;
    if (threadIdx.x == 0) {
        float found[EX_MAX_WORLD];
        ok = ll_gather(own, stride, p.world, n * dim + entry, step, (uint64_t)p.wait_ns, found);
        for (int r = 0; r < p.world; ++r) parts_lse[r] = ok ? found[r] : -INFINITY;
    }
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    float mine[4] = {0.f, 0.f, 0.f, 0.f}, total = 0.f, sub = 0.f, denom = 1.f;
    if (ok) {
        float top = -INFINITY;
        for (int r = 0; r < p.world; ++r) top = fmaxf(top, parts_lse[r]);
        sub = top == -INFINITY ? 0.f : top;
        for (int r = 0; r < p.world; ++r) total += parts_lse[r] == -INFINITY ? 0.f : expf(parts_lse[r] - sub);
        denom = fmaxf(total, 1e-30f);
        const float inv = total > 0.f ? 1.f / denom : 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = threadIdx.x + 256 * k;
            if (c < dim) {
                float found[EX_MAX_WORLD];
                ok = ll_gather(own, stride, p.world, entry * dim + c, step, (uint64_t)p.wait_ns, found) && ok;
                float sum = 0.f;
                for (int r = 0; r < p.world; ++r) sum += (parts_lse[r] == -INFINITY ? 0.f : expf(parts_lse[r] - sub)) * (ok ? found[r] : 0.f);
                mine[k] = sum * inv;
            }
        }
    }
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (ok) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = threadIdx.x + 256 * k;
            if (c < dim) ((TOUT*)m.out)[entry * dim + c] = from_float<TOUT>(mine[k]);
        }
        if (threadIdx.x == 0 && m.lse) m.lse[entry] = total > 0.f ? sub + logf(denom) : -INFINITY;
    } else if (threadIdx.x == 0 && p.status) {
        atomicExch(p.status, 0x800 + p.rank);
    }
}

}  // namespace crit_b200

using namespace crit_b200;

namespace crit_b200 {
int check_exchange(const crit_b200_exchange_params& p, bool with_message) {
    if (!p.peers || !p.step) return CRIT_B200_EINVAL;
    if (with_message && (!p.mine || !p.gathered)) return CRIT_B200_EINVAL;
    if (p.floats < 1 || p.world < 1 || p.world > EX_MAX_WORLD || p.rank < 0 || p.rank >= p.world || p.wait_ns < 1) return CRIT_B200_EINVAL;
    if (with_message && !aligned(p.mine, 16)) return CRIT_B200_EALIGN;
    return 0;
}
}  // namespace crit_b200

extern "C" __attribute__((visibility("default"))) int crit_b200_shard_push(const crit_b200_exchange_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_exchange_params p = *params;
    if (int e = check_exchange(p, true)) return e;
    shard_push_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(p);
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_shard_wait(const crit_b200_exchange_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_exchange_params p = *params;
    if (int e = check_exchange(p, true)) return e;
    shard_wait_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(p);
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_wait_merge(const crit_b200_exchange_params* exchange,
                                                                           const crit_b200_merge_shards_params* merge, void* stream) {
    if (!exchange || !merge) return CRIT_B200_EINVAL;
    const crit_b200_exchange_params p = *exchange;
    const crit_b200_merge_shards_params m = *merge;
    if (int e = check_exchange(p, false)) return e;
    if (m.n < 1 || m.n > 0x7fffffff || m.dim < 1 || m.dim > 1024 || !m.out || m.parts != p.world) return CRIT_B200_EINVAL;
    if (p.floats != m.n * (m.dim + 1) + EX_HEADER) return CRIT_B200_EINVAL;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)m.n;
    switch (m.out_dtype) {
        case CRIT_B200_DTYPE_BF16: wait_merge_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p, m); break;
        case CRIT_B200_DTYPE_FP16: wait_merge_kernel<__half><<<blocks, 256, 0, s>>>(p, m); break;
        case CRIT_B200_DTYPE_FP32: wait_merge_kernel<float><<<blocks, 256, 0, s>>>(p, m); break;
        default: return CRIT_B200_EINVAL;
    }
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int64_t crit_b200_exchange_bytes(int32_t world, int64_t floats) {
    if (world < 1 || floats < 1) return CRIT_B200_EINVAL;
    // two alternating slots a rank, each wide enough for the fused exchange's {value, step} pairs (twice the floats)
    return (EX_FLAG_WORDS + 2 * (int64_t)world * 2 * ex_stride(floats)) * 4;
}
