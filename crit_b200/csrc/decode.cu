// Split-K decode / speculative-verify attention over paged KV: the fold of a row's splits and the host side of the
// launches (variant choice, TMA tensor maps).  The decode kernel itself is decode_kernel.cuh.
// Reference: paged_kv_attention/_kernels.py:558-604 (_merge_kernel), cuda_window.cu:1071-1286 (cw_merge, cw_merge2),
// :1482-1535 (the C ABI this one mirrors).
#include <mutex>

#include "decode_kernel.cuh"
#include "decode_tc.cuh"
#include "decode_sw.cuh"
#include "decode_ph.cuh"
#include "exchange.cuh"
#include "tensor_map.cuh"

namespace crit_b200 {

constexpr int MERGE_WARPS = 8;

// States a row of L positions has in the workspace: one a split, or two (a split's head and tail; m = -inf marks one
// that holds nothing, and the folds pass it over) after a launch that deals tiles out evenly.
// A sink logit (natural units of the scaled scores) joins a folded state (top in base-2 units, total relative to it):
// the maximum and the sum take it, the outputs shrink by 2^(old top - new top).
__device__ __forceinline__ void sink_fold(float sink, float& top, float& total, float& shrink) {
    const float s2 = sink * LOG2E;
    const float up = fmaxf(top, s2);
    if (up == -INFINITY) return;
    shrink = top == -INFINITY ? 0.f : ex2(top - up);
    total = total * shrink + ex2(s2 - up);
    top = up;
}

__device__ __forceinline__ int states_of(const crit_b200_attend_params& p, int64_t L) {
    const int n = (int)((L + p.chunk - 1) / p.chunk);
    return (p.flags & CRIT_B200_ATTEND_TCGEN05P) ? 2 * n : n;
}

// The fold of a row's many splits.  Block = (window token, query head).  First every split's maximum (one load a
// thread, the block's maximum through shared memory), then warp w sums splits w, w + 8, ... with weights that are fixed
// by then, so its loads do not wait for one another (a hundred splits cost a few round trips, not a dozen dependent
// ones), and the eight warps' sums are added in warp order.  m is in base-2 units, o and l are relative to it.
__global__ void __launch_bounds__(MERGE_WARPS * 32) merge_kernel(const crit_b200_attend_params p) {
    __shared__ float sm[MERGE_WARPS], sl[MERGE_WARPS];
    __shared__ float so[MERGE_WARPS][256];
    const int head = blockIdx.x;
    const int r = blockIdx.y / p.columns, col = blockIdx.y - r * p.columns;
    // the row's facts in one round trip (the loads do not wait for one another's branches)
    int count = p.counts ? p.counts[r] : p.columns;
    const int64_t first = p.firsts[r];
    const int offset = p.offsets ? p.offsets[r] - p.offsets[0] : r * p.columns;
    const int start = p.starts[r];
    count = count > p.columns ? p.columns : count;
    if (col >= count) return;
    const int64_t L = first + ((p.flags & CRIT_B200_ATTEND_CONTEXT) ? 0 : count);
    const int nsplit = states_of(p, L);
    if (nsplit < 1 || (nsplit == 1 && !(p.flags & CRIT_B200_ATTEND_PARTIALS) && !p.sinks)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int DV = p.value_dim, per = DV >> 5;
    const int prow = offset + col;
    if (nsplit > p.max_splits || prow < 0 || prow >= p.partial_rows) {      // a plan too small for this row: nothing is read
        if (p.status && threadIdx.x == 0) atomicExch(p.status, CRIT_B200_STATUS_PLAN);
        return;
    }
    const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
    const int64_t base = ((int64_t)prow * p.q_heads + head) * p.max_splits;
    const float* pm = p.workspace + states * DV;
    const float* pl = p.workspace + states * (DV + 1);
    float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int s = threadIdx.x; s < nsplit; s += MERGE_WARPS * 32) m = fmaxf(m, pm[base + s]);
    m = warp_max(m);
    if (lane == 0) sm[warp] = m;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < MERGE_WARPS; ++w) m = fmaxf(m, sm[w]);
    __syncthreads();                        // (sm is written again below)
    const float sub0 = m == -INFINITY ? 0.f : m;
#pragma unroll 4
    for (int s = warp; s < nsplit; s += MERGE_WARPS) {
        const float ms = pm[base + s], ls = pl[base + s];
        if (ms == -INFINITY && ls == 0.f) continue;         // a state that holds nothing (a NaN row's sum is not 0)
        const float* o = p.workspace + (base + s) * DV + lane * per;
        const float take = ex2(ms - sub0);
        l += ls * take;
        if (per == 8) {                     // (a lane's values are 16-byte aligned: DV is a multiple of 32 floats)
            const float4 v = *reinterpret_cast<const float4*>(o), u = *reinterpret_cast<const float4*>(o + 4);
            acc[0] += v.x * take, acc[1] += v.y * take, acc[2] += v.z * take, acc[3] += v.w * take;
            acc[4] += u.x * take, acc[5] += u.y * take, acc[6] += u.z * take, acc[7] += u.w * take;
        } else if (per == 4) {
            const float4 v = *reinterpret_cast<const float4*>(o);
            acc[0] += v.x * take, acc[1] += v.y * take, acc[2] += v.z * take, acc[3] += v.w * take;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < per) acc[i] += o[i] * take;
        }
    }
    if (lane == 0) sm[warp] = m, sl[warp] = l;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < per) so[warp][lane * per + i] = acc[i];
    __syncthreads();
    const int token = start + col;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < MERGE_WARPS; ++w) top = fmaxf(top, sm[w]);
    const float sub = top == -INFINITY ? 0.f : top;
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < MERGE_WARPS; ++w) total += sl[w] * ex2(sm[w] - sub);
    float shrink = 1.f;                     // the head's sink, last: one position more without a value
    if (p.sinks) sink_fold(p.sinks[head], top, total, shrink);
    const float inv = total > 0.f ? shrink / total : 0.f;
    for (int c = threadIdx.x; c < DV; c += MERGE_WARPS * 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < MERGE_WARPS; ++w) o += so[w][c] * ex2(sm[w] - sub);
        o *= inv;
        const int64_t at = (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head + c;
        if (p.q_dtype == CRIT_B200_DTYPE_BF16) ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(o);
        else ((__half*)p.out)[at] = __float2half_rn(o);
    }
    if (p.lse && threadIdx.x == 0)
        p.lse[(int64_t)token * p.q_heads + head] = total > 0.f ? top * LN2 + logf(total) : -INFINITY;
}


// The same fold for rows of few splits: one warp per (window token, query head), the splits in order.
template <int DV>
__global__ void __launch_bounds__(128) merge_warp_kernel(const crit_b200_attend_params p) {
    constexpr int PER = DV / 32;
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int64_t items = (int64_t)p.n_rows * p.columns * p.q_heads;
    if (item >= items) return;
    const int head = (int)(item % p.q_heads);
    const int rc = (int)(item / p.q_heads);
    const int r = rc / p.columns, col = rc - r * p.columns;
    // the row's facts in one round trip (the loads do not wait for one another's branches)
    int count = p.counts ? p.counts[r] : p.columns;
    const int64_t first = p.firsts[r];
    const int offset = p.offsets ? p.offsets[r] - p.offsets[0] : r * p.columns;
    const int start = p.starts[r];
    count = count > p.columns ? p.columns : count;
    if (col >= count) return;
    const int64_t L = first + ((p.flags & CRIT_B200_ATTEND_CONTEXT) ? 0 : count);
    const int nsplit = states_of(p, L);
    if (nsplit < 1 || (nsplit == 1 && !(p.flags & CRIT_B200_ATTEND_PARTIALS) && !p.sinks)) return;
    const int prow = offset + col;
    if (nsplit > p.max_splits || prow < 0 || prow >= p.partial_rows) {      // a plan too small for this row: nothing is read
        if (p.status && lane == 0) atomicExch(p.status, CRIT_B200_STATUS_PLAN);
        return;
    }
    const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
    const int64_t base = ((int64_t)prow * p.q_heads + head) * p.max_splits;
    const float* pm = p.workspace + states * DV;
    const float* pl = p.workspace + states * (DV + 1);
    // every split's maximum first (one load a lane), then one pass over the outputs with fixed weights
    float top = -INFINITY;
    for (int s = lane; s < nsplit; s += 32) top = fmaxf(top, pm[base + s]);
    top = warp_max(top);
    const float sub = top == -INFINITY ? 0.f : top;
    float total = 0.f, acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
#pragma unroll 4
    for (int s = 0; s < nsplit; ++s) {
        if (pm[base + s] == -INFINITY && pl[base + s] == 0.f) continue;         // a state that holds nothing
        const float w = ex2(pm[base + s] - sub);
        total += pl[base + s] * w;
        const float* o = p.workspace + (base + s) * DV + lane * PER;
        if constexpr (PER == 4) {
            const float4 v = *reinterpret_cast<const float4*>(o);
            acc[0] += v.x * w, acc[1] += v.y * w, acc[2] += v.z * w, acc[3] += v.w * w;
        } else if constexpr (PER == 8) {
            const float4 v = *reinterpret_cast<const float4*>(o), u = *reinterpret_cast<const float4*>(o + 4);
            acc[0] += v.x * w, acc[1] += v.y * w, acc[2] += v.z * w, acc[3] += v.w * w;
            acc[4] += u.x * w, acc[5] += u.y * w, acc[6] += u.z * w, acc[7] += u.w * w;
        } else {
            const float2 v = *reinterpret_cast<const float2*>(o);
            acc[0] += v.x * w, acc[1] += v.y * w;
        }
    }
    float shrink = 1.f;                     // the head's sink, last: one position more without a value
    if (p.sinks) sink_fold(p.sinks[head], top, total, shrink);
    const float inv = total > 0.f ? shrink / total : 0.f;
    const int token = start + col;
    const int64_t at = (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; i += 2) {
        const uint32_t packed = p.q_dtype == CRIT_B200_DTYPE_BF16 ? pack2<true>(acc[i] * inv, acc[i + 1] * inv)
                                                                   : pack2<false>(acc[i] * inv, acc[i + 1] * inv);
        *reinterpret_cast<uint32_t*>((char*)p.out + (at + i) * 2) = packed;
    }
    if (p.lse && lane == 0) p.lse[(int64_t)token * p.q_heads + head] = total > 0.f ? top * LN2 + logf(total) : -INFINITY;
}


// The fold of a rank's splits, sent: what merge_kernel computes for a (token, head), normalised, goes as FP32 into slot
// [step & 1][rank] of EVERY rank's exchange buffer (peer stores over NVLink; this rank's own buffer too) instead of into
// `out`: a message is [tokens x heads][DV] outputs then [tokens x heads] log-sum-exps (natural log), every float stored
// with the step beside it (exchange.cuh).  Block = (window token, query head); warp w folds splits w, w + 8, ... and the
// eight warps' states are folded in warp order, so a row of a hundred splits costs a dozen dependent loads, not a
// hundred.  A column past its row's count, and a row that holds no position, send zeros and -inf.  Nothing waits for a
// peer here.  FUSED: the same block then gathers its own (token, head) from every rank's message in this rank's own buffer
// (a bounded wait per float) and writes the merge of shards: the whole exchange in one launch, its latency one NVLink
// write.  The blocks count themselves out on a ticket in this rank's buffer; the last one moves the step counter on.
template <int DV, bool FUSED>
__global__ void __launch_bounds__(MERGE_WARPS * 32) merge_push_kernel(const crit_b200_attend_params p, const crit_b200_exchange_params x,
                                                                      const crit_b200_merge_shards_params shards) {
    constexpr int PER = DV / 32;
    __shared__ float sm[MERGE_WARPS], sl[MERGE_WARPS];
    __shared__ float so[MERGE_WARPS][DV];
    __shared__ float* slots[EX_MAX_WORLD];          // this rank's slot of the step in every rank's buffer
    __shared__ float parts_lse[EX_MAX_WORLD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int32_t step = *x.step + 1;
    const int64_t stride = 2 * ex_stride(x.floats);
    const uint64_t own_base = x.peers[x.rank];
    if (threadIdx.x < x.world) slots[threadIdx.x] = ex_slot(x.peers[threadIdx.x], step, x.world, x.rank, stride);
    const int64_t n = (x.floats - EX_HEADER) / (DV + 1);           // (token, head) pairs of a message
    const int head = blockIdx.x;
    const int r = blockIdx.y / p.columns, col = blockIdx.y - r * p.columns;
    int count = p.counts ? p.counts[r] : p.columns;
    count = count > p.columns ? p.columns : count;
    const int64_t L = p.firsts[r] + (count > 0 ? count : 0);
    const int nsplit = count > 0 ? states_of(p, L) : 0;
    const int prow = (p.offsets ? p.offsets[r] - p.offsets[0] : r * p.columns) + col;
    const int64_t entry = (int64_t)(p.starts[r] + col) * p.q_heads + head;
    const bool listed = entry >= 0 && entry < n;
    const bool fits = nsplit <= p.max_splits && prow >= 0 && prow < p.partial_rows;
    float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    if (listed && fits && col < count) {
        const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
        const int64_t base = ((int64_t)prow * p.q_heads + head) * p.max_splits;
        const float* pm = p.workspace + states * DV;
        const float* pl = p.workspace + states * (DV + 1);
#pragma unroll 4
        for (int s = warp; s < nsplit; s += MERGE_WARPS) {
            const float ms = pm[base + s], ls = pl[base + s];
            if (ms == -INFINITY && ls == 0.f) continue;         // a state that holds nothing (a NaN row's sum is not 0)
            const float* o = p.workspace + (base + s) * DV + lane * PER;
            float v[PER];
#pragma unroll
            for (int i = 0; i < PER; i += 2) {
                const float2 pair = *reinterpret_cast<const float2*>(o + i);
                v[i] = pair.x, v[i + 1] = pair.y;
            }
            const float top = fmaxf(m, ms);
            const float sub = top == -INFINITY ? 0.f : top;
            const float keep = ex2(m - sub), take = ex2(ms - sub);
            l = l * keep + ls * take;
#pragma unroll
            for (int i = 0; i < PER; ++i) acc[i] = acc[i] * keep + v[i] * take;
            m = top;
        }
    }
    if (listed && !fits && col < count && threadIdx.x == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_PLAN);
    if (lane == 0) sm[warp] = m, sl[warp] = l;
#pragma unroll
    for (int i = 0; i < PER; ++i) so[warp][lane * PER + i] = acc[i];
    __syncthreads();
    if (listed) {
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < MERGE_WARPS; ++w) top = fmaxf(top, sm[w]);
        const float sub = top == -INFINITY ? 0.f : top;
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < MERGE_WARPS; ++w) total += sl[w] * ex2(sm[w] - sub);
        const float inv = total > 0.f ? 1.f / total : 0.f;
        for (int c = threadIdx.x; c < DV; c += MERGE_WARPS * 32) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < MERGE_WARPS; ++w) o += so[w][c] * ex2(sm[w] - sub);
            o *= inv;
            for (int peer = 0; peer < x.world; ++peer) ll_store(slots[peer], entry * DV + c, o, step);
        }
        if (threadIdx.x == 0) {
            const float lse = total > 0.f ? top * LN2 + logf(total) : -INFINITY;
            for (int peer = 0; peer < x.world; ++peer) ll_store(slots[peer], n * DV + entry, lse, step);
        }
    }
    if constexpr (FUSED) {
        // this block's (token, head) out of every rank's message in this rank's own buffer: the log-sum-exps first (one
        // thread), then thread c takes column c of every rank; nothing of the pair is written unless all of it arrived
        constexpr int MINE = (DV + MERGE_WARPS * 32 - 1) / (MERGE_WARPS * 32);
        const float* own = ex_slot(own_base, step, x.world, 0, stride);
        bool ok = true;
        if (listed && threadIdx.x == 0) {
            float found[EX_MAX_WORLD];
            ok = ll_gather(own, stride, x.world, n * DV + entry, step, (uint64_t)x.wait_ns, found);
            for (int rr = 0; rr < x.world; ++rr) parts_lse[rr] = ok ? found[rr] : -INFINITY;
        }
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
        float mine[MINE], total = 0.f, sub = 0.f, denom = 1.f;
        if (ok && listed) {
            float top = -INFINITY;
            for (int rr = 0; rr < x.world; ++rr) top = fmaxf(top, parts_lse[rr]);
            sub = top == -INFINITY ? 0.f : top;
            for (int rr = 0; rr < x.world; ++rr) total += parts_lse[rr] == -INFINITY ? 0.f : expf(parts_lse[rr] - sub);
            denom = fmaxf(total, 1e-30f);
            const float inv = total > 0.f ? 1.f / denom : 0.f;
#pragma unroll
            for (int k = 0; k < MINE; ++k) {
                const int c = threadIdx.x + k * MERGE_WARPS * 32;
                mine[k] = 0.f;
                if (c < DV) {
                    float found[EX_MAX_WORLD];
                    ok = ll_gather(own, stride, x.world, entry * DV + c, step, (uint64_t)x.wait_ns, found) && ok;
                    float sum = 0.f;
                    for (int rr = 0; rr < x.world; ++rr)
                        sum += (parts_lse[rr] == -INFINITY ? 0.f : expf(parts_lse[rr] - sub)) * (ok ? found[rr] : 0.f);
                    mine[k] = sum * inv;
                }
            }
        }
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
        if (ok && listed) {
#pragma unroll
            for (int k = 0; k < MINE; ++k) {
                const int c = threadIdx.x + k * MERGE_WARPS * 32;
                if (c >= DV) continue;
                if (shards.out_dtype == CRIT_B200_DTYPE_BF16) ((__nv_bfloat16*)shards.out)[entry * DV + c] = __float2bfloat16_rn(mine[k]);
                else if (shards.out_dtype == CRIT_B200_DTYPE_FP16) ((__half*)shards.out)[entry * DV + c] = __float2half_rn(mine[k]);
                else ((float*)shards.out)[entry * DV + c] = mine[k];
            }
            if (threadIdx.x == 0 && shards.lse) shards.lse[entry] = total > 0.f ? sub + logf(denom) : -INFINITY;
        }
        if (!ok && threadIdx.x == 0 && x.status) atomicExch(x.status, 0x800 + x.rank);
    }
    // the step counter moves on when every block has read it: the last block out does it
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t* ticket = reinterpret_cast<int32_t*>(own_base) + EX_TICKET;
        if (atomicAdd(ticket, 1) == (int)(gridDim.x * gridDim.y) - 1) {
            *ticket = 0;
            *x.step = step;
        }
    }
}

// -- host side --------------------------------------------------------------------------------------------------------
typedef void (*decode_fn)(const crit_b200_attend_params, const int, const int, const int, const int, const CUtensorMap,
                          const CUtensorMap);
typedef int (*smem_fn)(int);

struct Variant {
    decode_fn fn;
    smem_fn smem;
    bool tma;
    int es;
};

template <int D, int DV, int PK, int NT, bool TMA>
static Variant variant() {
    return Variant{decode_kernel<D, DV, PK, NT, TMA>, DecodeCfg<D, DV, PK, NT, TMA>::smem_bytes, TMA, PK < 2 ? 2 : 1};
}

template <int PK, int NT, bool TMA>
static int pick_width(int d, int dv, Variant* out) {
    if (d == 64 && dv == 64) {
        if constexpr (!TMA) *out = variant<64, 64, PK, NT, false>();
        else return CRIT_B200_EUNSUPPORTED;
    } else if (d == 128 && dv == 128) {
        *out = variant<128, 128, PK, NT, TMA>();
    } else if (d == 256 && dv == 256) {
        if constexpr (NT <= 2) *out = variant<256, 256, PK, NT, TMA>();
        else return CRIT_B200_EUNSUPPORTED;
    } else {
        return CRIT_B200_EUNSUPPORTED;
    }
    return 0;
}

static int page_class(int kind, int page_dtype) {
    if (kind == CRIT_B200_KIND_16BIT) return page_dtype == CRIT_B200_DTYPE_BF16 ? 0 : (page_dtype == CRIT_B200_DTYPE_FP16 ? 1 : -1);
    if (kind == CRIT_B200_KIND_INT8) return 3;
    if (kind == CRIT_B200_KIND_FP8 || kind == CRIT_B200_KIND_FP8_ROW || kind == CRIT_B200_KIND_FP8_PAGE) return 2;
    return -1;
}

// 8-row tiles of query rows a block holds: as many as a row's columns times the group's heads need, up to 4 (32 rows),
// 2 where the value accumulators of more would not fit the registers (256-wide values).
static int row_tiles(int rows, int dv) {
    const int most = dv <= 128 ? 4 : 2;
    const int need = rows <= 8 ? 1 : (rows <= 16 ? 2 : 4);
    return need < most ? need : most;
}

template <int PK, bool TMA>
static int pick_rows(int d, int dv, int nt, Variant* out) {
    if (nt == 1) return pick_width<PK, 1, TMA>(d, dv, out);
    if (nt == 2) return pick_width<PK, 2, TMA>(d, dv, out);
    return pick_width<PK, 4, TMA>(d, dv, out);
}

static int pick(int kind, int page_dtype, int d, int dv, int nt, bool tma, Variant* out) {
    const int pk = page_class(kind, page_dtype);
    if (pk < 0) return CRIT_B200_EUNSUPPORTED;
#define CRIT_PICK(PK) return tma ? pick_rows<PK, true>(d, dv, nt, out) : pick_rows<PK, false>(d, dv, nt, out)
    switch (pk) {
        case 0: CRIT_PICK(0);
        case 1: CRIT_PICK(1);
        case 2: CRIT_PICK(2);
        default: CRIT_PICK(3);
    }
#undef CRIT_PICK
}

static int scale_mode(int kind) {
    return kind == CRIT_B200_KIND_FP8_ROW || kind == CRIT_B200_KIND_INT8 ? 1 : (kind == CRIT_B200_KIND_FP8_PAGE ? 2 : 0);
}

// Whether the TMA staging serves a launch: heads of 128 or 256 values, the pool's size known, and scale rows the bulk
// copies can take (a multiple of 16 bytes, 16-byte aligned, up to 1 KB a tile).
static bool tma_serves(const crit_b200_attend_params& p) {
    if (p.flags & CRIT_B200_ATTEND_NO_TMA) return false;
    if (!(p.flags & CRIT_B200_ATTEND_TMA) && p.kind != CRIT_B200_KIND_16BIT) return false;
    if (p.slots < 16 || p.slots > 0x7fffffffLL) return false;
    if (!(p.head_dim == p.value_dim && (p.head_dim == 128 || p.head_dim == 256))) return false;
    const int sm = scale_mode(p.kind);
    if (sm) {
        if (p.kv_heads % 4 || !aligned(p.key_scales, 16) || !aligned(p.value_scales, 16)) return false;
        if (sm == 1 && p.kv_heads > 8) return false;
        if (sm == 2 && p.kv_heads > 128) return false;
    }
    return true;
}

// Bytes of one stage's scales in shared memory (keys in the first half, values in the second).
static int scale_stage_bytes(const crit_b200_attend_params& p, bool tma) {
    const int sm = scale_mode(p.kind);
    if (!tma) return 128;
    if (sm == 2) return 2 * ((p.kv_heads * 4 + 15) / 16 * 16);
    if (sm == 1) return 2 * p.kv_heads * 64;
    return 0;
}

// Blocks of a kernel the current device holds at once (SMs x blocks per SM), remembered per kernel, shared-memory size
// and device.
static int resident_blocks(const void* fn, int smem) {
    struct Entry { const void* fn; int smem, device, blocks; };
    static Entry seen[256];
    static int n = 0;
    static std::mutex guard;            // calls may come from several host threads (one per device or engine)
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    std::lock_guard<std::mutex> lock(guard);
    for (int i = 0; i < n; ++i)
        if (seen[i].fn == fn && seen[i].smem == smem && seen[i].device == device) return seen[i].blocks;
    int sms = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, DECODE_THREADS, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    const int blocks = sms * per_sm;
    if (n < 256) seen[n++] = Entry{fn, smem, device, blocks};
    return blocks;
}

static int check(const crit_b200_attend_params& p) {
    if (!p.q || !p.out || !p.key_pages || !p.value_pages || !p.tables || !p.rows || !p.starts || !p.firsts)
        return CRIT_B200_EINVAL;
    if (p.n_rows < 1 || p.columns < 1 || p.columns > 64 || p.q_heads < 1 || p.kv_heads < 1 || p.q_heads % p.kv_heads)
        return CRIT_B200_EINVAL;
    if (p.page < 16 || p.page % 16) return CRIT_B200_EUNSUPPORTED;
    if (p.chunk < 16 || p.chunk % 16 || p.max_splits < 1) return CRIT_B200_EINVAL;
    if (scale_mode(p.kind) && (!p.key_scales || !p.value_scales)) return CRIT_B200_EINVAL;
    if (p.q_dtype != CRIT_B200_DTYPE_BF16 && p.q_dtype != CRIT_B200_DTYPE_FP16) return CRIT_B200_EUNSUPPORTED;
    if (p.kind == CRIT_B200_KIND_16BIT && p.page_dtype != p.q_dtype) return CRIT_B200_EUNSUPPORTED;
    if (!aligned(p.q, 16) || p.q_stride_token % 8 || p.q_stride_head % 8 || !aligned(p.key_pages, 16) ||
        !aligned(p.value_pages, 16) || !aligned(p.out, 8) || p.out_stride_token % 4 || p.out_stride_head % 4)
        return CRIT_B200_EALIGN;
    if (p.head_dim < 1 || p.value_dim < 1 || p.head_dim > 1024 || p.value_dim > 1024) return CRIT_B200_EUNSUPPORTED;
    if (p.sliding < 0 || (p.blocks && (p.blocks_k < 1 || p.block_size < 1))) return CRIT_B200_EINVAL;
    if (p.max_splits > 1 || (p.flags & CRIT_B200_ATTEND_PARTIALS) || p.sinks) {
        // partial_rows <= 2^31, q_heads and max_splits below 2^31, value_dim + 2 <= 1026: compared by division, so that no
        // product of the four can wrap
        if (p.partial_rows < 1 || (!p.offsets && (int64_t)p.partial_rows < (int64_t)p.n_rows * p.columns)) return CRIT_B200_EINVAL;
        if (!p.workspace || p.workspace_floats < 1) return CRIT_B200_EWORKSPACE;
        const int64_t per_row = (int64_t)p.q_heads * (p.value_dim + 2);              // < 2^31 * 1026
        if (per_row > p.workspace_floats / p.max_splits) return CRIT_B200_EWORKSPACE;
        if ((int64_t)p.partial_rows > p.workspace_floats / (per_row * p.max_splits)) return CRIT_B200_EWORKSPACE;
        if (!aligned(p.workspace, 16)) return CRIT_B200_EALIGN;
    }
    return 0;
}

// Whether the tcgen05 kernel serves a launch: E4M3 pages of 128-wide heads, at most 32 query rows a unit (columns x
// heads of a group), splits that are whole tiles of 128 positions, the pool's size known for the tensor maps.
static bool tc_serves(const crit_b200_attend_params& p) {
    if (page_class(p.kind, p.page_dtype) != 2) return false;
    if (p.head_dim != DT_D || p.value_dim != DT_D) return false;
    if (p.columns * (p.q_heads / p.kv_heads) > 32) return false;
    if (p.chunk % DT_N || p.chunk > DT_MAX_CHUNK) return false;
    if (p.slots < 16 || p.slots > 0x7fffffffLL) return false;
    if (p.n_rows > DT_MAX_LIST) return false;
    return true;
}

static int launch_decode_tc(const crit_b200_attend_params& p, cudaStream_t s) {
    CUtensorMap kmap, vmap;
    if (!page_map(&kmap, p.key_pages, 2, p.head_dim, p.kv_heads, p.slots) ||
        !page_map(&vmap, p.value_pages, 2, p.value_dim, p.kv_heads, p.slots))
        return CRIT_B200_EUNSUPPORTED;
    const int rows = p.columns * (p.q_heads / p.kv_heads);
    typedef void (*tc_fn)(const crit_b200_attend_params, const CUtensorMap, const CUtensorMap);
    const int nrg = rows <= 8 ? 0 : (rows <= 16 ? 1 : 2);
    static const tc_fn fns[3][3] = {
        {decode_tc_kernel<1, 0>, decode_tc_kernel<1, 1>, decode_tc_kernel<1, 2>},
        {decode_tc_kernel<2, 0>, decode_tc_kernel<2, 1>, decode_tc_kernel<2, 2>},
        {decode_tc_kernel<4, 0>, decode_tc_kernel<4, 1>, decode_tc_kernel<4, 2>}};
    const tc_fn fn = fns[nrg][scale_mode(p.kind)];
    cudaError_t ce = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, DT_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
        return CRIT_B200_EUNSUPPORTED;
    const int64_t most = (int64_t)p.max_splits * p.kv_heads * p.n_rows;        // units the launch can have
    const unsigned blocks = (unsigned)(most < 2 * sms ? most : 2 * sms);       // two persistent blocks per SM
    fn<<<blocks, DT_THREADS, DT_SMEM, s>>>(p, kmap, vmap);
    CRIT_CHECK_LAUNCH();
    return 0;
}

static int launch_decode_sw(const crit_b200_attend_params& p, cudaStream_t s) {
    CUtensorMap kmap, vmap;
    if (!page_map(&kmap, p.key_pages, 2, p.head_dim, p.kv_heads, p.slots) ||
        !page_map(&vmap, p.value_pages, 2, p.value_dim, p.kv_heads, p.slots))
        return CRIT_B200_EUNSUPPORTED;
    const int rows = p.columns * (p.q_heads / p.kv_heads);
    typedef void (*sw_fn)(const crit_b200_attend_params, const CUtensorMap, const CUtensorMap);
    const int nrg = rows <= 8 ? 0 : (rows <= 16 ? 1 : 2);
    static const sw_fn fns[3][3] = {
        {decode_sw_kernel<8, 0>, decode_sw_kernel<8, 1>, decode_sw_kernel<8, 2>},
        {decode_sw_kernel<16, 0>, decode_sw_kernel<16, 1>, decode_sw_kernel<16, 2>},
        {decode_sw_kernel<32, 0>, decode_sw_kernel<32, 1>, decode_sw_kernel<32, 2>}};
    const sw_fn fn = fns[nrg][scale_mode(p.kind)];
    const int smem = nrg == 0 ? SwCfg<8>::SMEM : (nrg == 1 ? SwCfg<16>::SMEM : SwCfg<32>::SMEM);
    cudaError_t ce = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (ce != cudaSuccess) return (int)ce;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
        return CRIT_B200_EUNSUPPORTED;
    const int64_t most = (int64_t)p.max_splits * p.kv_heads * p.n_rows;        // units the launch can have
    const unsigned blocks = (unsigned)(most < 2 * sms ? most : 2 * sms);       // two persistent blocks per SM
    fn<<<blocks, SW_THREADS, smem, s>>>(p, kmap, vmap);
    CRIT_CHECK_LAUNCH();
    return 0;
}

// Whether the whole-page-rows tcgen05 kernel serves a launch: E4M3 pages of 128-wide heads, 8 kv heads, at most 8 query
// rows a kv head (columns x heads of a group), splits of whole 16-position tiles, scales the bulk copies can take.
static bool ph_serves(const crit_b200_attend_params& p) {
    if (page_class(p.kind, p.page_dtype) != 2) return false;
    if (p.head_dim != DT_D || p.value_dim != DT_D || p.kv_heads != PH_HEADS) return false;
    if (p.columns * (p.q_heads / p.kv_heads) > 8) return false;
    if (p.chunk % PH_TILE || p.chunk > DT_MAX_CHUNK) return false;
    if (p.slots < 16 || p.slots > 0x7fffffffLL) return false;
    if (p.n_rows > PH_MAX_LIST || !p.workspace || p.max_splits < 2) return false;
    if (scale_mode(p.kind) != 0 && (!aligned(p.key_scales, 16) || !aligned(p.value_scales, 16))) return false;
    return true;
}

static int launch_decode_ph(const crit_b200_attend_params& p, cudaStream_t s) {
    CUtensorMap kmap, vmap;
    if (!page_rows_map(&kmap, p.key_pages, p.head_dim, p.kv_heads, p.slots) ||
        !page_rows_map(&vmap, p.value_pages, p.value_dim, p.kv_heads, p.slots))
        return CRIT_B200_EUNSUPPORTED;
    typedef void (*ph_fn)(const crit_b200_attend_params, const CUtensorMap, const CUtensorMap);
    static const ph_fn fns[2][3] = {{decode_ph_kernel<0, 1>, decode_ph_kernel<1, 1>, decode_ph_kernel<2, 1>},
                                    {decode_ph_kernel<0, 2>, decode_ph_kernel<1, 2>, decode_ph_kernel<2, 2>}};
    const int per_sm = (p.flags & CRIT_B200_ATTEND_PERSISTENT) ? 1 : 2;        // (a measurement's switch)
    const ph_fn fn = fns[per_sm - 1][scale_mode(p.kind)];
    const int PH_SMEM = per_sm == 1 ? PhCfg<1>::SMEM : PhCfg<2>::SMEM;
    cudaError_t ce = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, PH_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
        return CRIT_B200_EUNSUPPORTED;
    const int64_t most = (int64_t)((p.max_splits + 1) / 2) * p.n_rows;         // splits the launch can have: a block holds one at least
    const unsigned blocks = (unsigned)(most < per_sm * sms ? most : per_sm * sms);
    fn<<<blocks, PH_THREADS, PH_SMEM, s>>>(p, kmap, vmap);
    CRIT_CHECK_LAUNCH();
    return 0;
}

static int launch_decode(const crit_b200_attend_params& p, cudaStream_t s) {
    // draft trees (parents), sliding windows, sinks and block lists are the m16n8k16 kernel's only
    if ((p.parents || p.sinks || p.sliding > 0 || p.blocks || (p.flags & CRIT_B200_ATTEND_CONTEXT)) && (p.flags & (CRIT_B200_ATTEND_TCGEN05P | CRIT_B200_ATTEND_TCGEN05T | CRIT_B200_ATTEND_TCGEN05))) return CRIT_B200_EUNSUPPORTED;
    if (p.flags & CRIT_B200_ATTEND_TCGEN05P) return ph_serves(p) ? launch_decode_ph(p, s) : CRIT_B200_EUNSUPPORTED;
    if (p.flags & CRIT_B200_ATTEND_TCGEN05T) return tc_serves(p) && p.n_rows <= SW_MAX_LIST ? launch_decode_sw(p, s) : CRIT_B200_EUNSUPPORTED;
    if (p.flags & CRIT_B200_ATTEND_TCGEN05) return tc_serves(p) ? launch_decode_tc(p, s) : CRIT_B200_EUNSUPPORTED;
    // The library's choice: windows of several columns over E4M3 pages go to the tcgen05 kernel where it serves them
    // (the page bytes feed the tensor cores as they are; the m16n8k16 kernel converts every byte in registers and holds
    // 32 query rows of accumulators a warp, which makes it issue-bound there), everything else, single-column decode
    // rows above all, to the m16n8k16 kernel.  A column's bits then depend on whether it is read alone or in a window;
    // CRIT_B200_ATTEND_MMA_SYNC keeps every launch on the m16n8k16 kernel, whose bits do not.
    if (!(p.flags & CRIT_B200_ATTEND_MMA_SYNC) && p.columns > 1 && !p.parents && !p.sinks && p.sliding <= 0 && !p.blocks && !(p.flags & CRIT_B200_ATTEND_CONTEXT) && tc_serves(p))
        return launch_decode_tc(p, s);
    const int G = p.q_heads / p.kv_heads;
    const int rows = p.columns * G;
    const int nt = row_tiles(rows, p.value_dim);
    const int pk = page_class(p.kind, p.page_dtype);
    CUtensorMap kmap, vmap;
    memset(&kmap, 0, sizeof kmap);
    memset(&vmap, 0, sizeof vmap);
    bool tma = tma_serves(p) && pk >= 0 && page_map(&kmap, p.key_pages, pk, p.head_dim, p.kv_heads, p.slots) &&
               page_map(&vmap, p.value_pages, pk, p.value_dim, p.kv_heads, p.slots);
    Variant v;
    int e = pick(p.kind, p.page_dtype, p.head_dim, p.value_dim, nt, tma, &v);
    if (e) return e;
    const int scb = scale_stage_bytes(p, tma);
    const int smem = v.smem(scb);
    // Set at every launch: the attribute belongs to the function on the current device, and a process may drive several.
    cudaError_t ce = cudaFuncSetAttribute((const void*)v.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (ce != cudaSuccess) return (int)ce;
    const int ctiles = (rows + 8 * nt - 1) / (8 * nt);
    const int64_t most = (int64_t)p.max_splits * p.kv_heads * ctiles * p.n_rows;      // units the launch can have
    if (p.n_rows <= DECODE_MAX_LIST && (p.flags & CRIT_B200_ATTEND_PERSISTENT)) {
        // persistent: a fixed number of blocks (what the SMs hold at once) walk the launch's work list
        const int slots = resident_blocks((const void*)v.fn, smem);
        if (slots > 0) {
            const unsigned blocks = (unsigned)(most < slots ? most : slots);
            v.fn<<<blocks, DECODE_THREADS, smem, s>>>(p, ctiles, scale_mode(p.kind), scb, 1, kmap, vmap);
            CRIT_CHECK_LAUNCH();
            return 0;
        }
    }
    dim3 grid((unsigned)p.max_splits, (unsigned)(p.kv_heads * ctiles), (unsigned)p.n_rows);
    v.fn<<<grid, DECODE_THREADS, smem, s>>>(p, ctiles, scale_mode(p.kind), scb, 0, kmap, vmap);
    CRIT_CHECK_LAUNCH();
    return 0;
}

static int launch_merge(const crit_b200_attend_params& p, cudaStream_t s) {
    if (p.max_splits <= 1 && !(p.flags & CRIT_B200_ATTEND_PARTIALS) && !p.sinks) return 0;
    if (p.value_dim > 256 || p.value_dim % 32) return CRIT_B200_EUNSUPPORTED;
    if (p.max_splits <= 32) {
        const int64_t items = (int64_t)p.n_rows * p.columns * p.q_heads;
        const unsigned blocks = (unsigned)((items + 3) / 4);
        if (p.value_dim == 128) merge_warp_kernel<128><<<blocks, 128, 0, s>>>(p);
        else if (p.value_dim == 256) merge_warp_kernel<256><<<blocks, 128, 0, s>>>(p);
        else if (p.value_dim == 64) merge_warp_kernel<64><<<blocks, 128, 0, s>>>(p);
        else return CRIT_B200_EUNSUPPORTED;
    } else {
        dim3 grid((unsigned)p.q_heads, (unsigned)(p.n_rows * p.columns));
        merge_kernel<<<grid, MERGE_WARPS * 32, 0, s>>>(p);
    }
    CRIT_CHECK_LAUNCH();
    return 0;
}

// -- partials without an allocator ------------------------------------------------------------------------------------
// The scratch of crit_b200_attend_static: part of the library's image on every GPU that loads it.  In host code this
// name only stands for the array (it is not a device address): the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static __device__ __align__(256) float static_scratch[CRIT_B200_STATIC_SCRATCH_FLOATS];

static int static_scratch_address(float** out) {
    constexpr int MOST = 64;
    static float* found[MOST];
    static std::mutex guard;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MOST) return CRIT_B200_EUNSUPPORTED;
    std::lock_guard<std::mutex> lock(guard);
    if (!found[device]) {
        void* address = nullptr;
        e = cudaGetSymbolAddress(&address, static_scratch);
        if (e != cudaSuccess) return (int)e;
        found[device] = static_cast<float*>(address);
    }
    *out = found[device];
    return 0;
}

}  // namespace crit_b200

using namespace crit_b200;

extern "C" __attribute__((visibility("default"))) int crit_b200_attend_static(const crit_b200_attend_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    crit_b200_attend_params p = *params;
    float* scratch = nullptr;
    int e = static_scratch_address(&scratch);
    if (e) return e;
    p.workspace = scratch;
    p.workspace_floats = CRIT_B200_STATIC_SCRATCH_FLOATS;
    // check() validates every field first and compares the partials with the scratch by division (no product of the
    // caller's integers is formed): a launch that does not fit is refused with the entry point's own code
    e = check(p);
    if (e == CRIT_B200_EWORKSPACE) return CRIT_B200_ESTATIC;
    if (e) return e;
    e = launch_decode(p, (cudaStream_t)stream);
    return e ? e : launch_merge(p, (cudaStream_t)stream);
}

namespace crit_b200 {
int check_exchange(const crit_b200_exchange_params& p, bool with_message);      // exchange.cu
}

template <bool FUSED>
static int launch_merge_push(const crit_b200_attend_params& p, const crit_b200_exchange_params& x, const crit_b200_merge_shards_params& m,
                             cudaStream_t s) {
    const dim3 blocks((unsigned)p.q_heads, (unsigned)(p.n_rows * p.columns));
    if (p.value_dim == 128) merge_push_kernel<128, FUSED><<<blocks, MERGE_WARPS * 32, 0, s>>>(p, x, m);
    else if (p.value_dim == 256) merge_push_kernel<256, FUSED><<<blocks, MERGE_WARPS * 32, 0, s>>>(p, x, m);
    else if (p.value_dim == 64) merge_push_kernel<64, FUSED><<<blocks, MERGE_WARPS * 32, 0, s>>>(p, x, m);
    else return CRIT_B200_EUNSUPPORTED;
    CRIT_CHECK_LAUNCH();
    return 0;
}

static int check_merge_push(const crit_b200_attend_params& p, const crit_b200_exchange_params& x) {
    if (!(p.flags & CRIT_B200_ATTEND_PARTIALS)) return CRIT_B200_EINVAL;
    int e = check(p);
    if (!e) e = check_exchange(x, false);
    if (e) return e;
    if (x.floats < EX_HEADER + p.value_dim + 1 || (x.floats - EX_HEADER) % (p.value_dim + 1)) return CRIT_B200_EINVAL;
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_merge_push(const crit_b200_attend_params* attend,
                                                                           const crit_b200_exchange_params* exchange, void* stream) {
    if (!attend || !exchange) return CRIT_B200_EINVAL;
    const crit_b200_attend_params p = *attend;
    const crit_b200_exchange_params x = *exchange;
    if (int e = check_merge_push(p, x)) return e;
    crit_b200_merge_shards_params none;
    memset(&none, 0, sizeof none);
    return launch_merge_push<false>(p, x, none, (cudaStream_t)stream);
}

extern "C" __attribute__((visibility("default"))) int crit_b200_wait_merge(const crit_b200_exchange_params* exchange,
                                                                           const crit_b200_merge_shards_params* merge, void* stream);

// Fold + push and wait + merge of shards: one launch where every block of it is resident at once (a block per (token,
// head) of the step, up to the device's SM count: a block waits for the flag this rank's last block raises), else the two
// launches crit_b200_merge_push and crit_b200_wait_merge.
extern "C" __attribute__((visibility("default"))) int crit_b200_exchange_merge(const crit_b200_attend_params* attend,
                                                                               const crit_b200_exchange_params* exchange,
                                                                               const crit_b200_merge_shards_params* merge, void* stream) {
    if (!attend || !exchange || !merge) return CRIT_B200_EINVAL;
    const crit_b200_attend_params p = *attend;
    const crit_b200_exchange_params x = *exchange;
    const crit_b200_merge_shards_params m = *merge;
    if (int e = check_merge_push(p, x)) return e;
    if (m.n < 1 || m.dim != p.value_dim || !m.out || m.parts != x.world || x.floats != m.n * (m.dim + 1) + EX_HEADER) return CRIT_B200_EINVAL;
    if (m.out_dtype != CRIT_B200_DTYPE_BF16 && m.out_dtype != CRIT_B200_DTYPE_FP16 && m.out_dtype != CRIT_B200_DTYPE_FP32) return CRIT_B200_EINVAL;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 0;
    // one launch while every block of it is resident at once (4 blocks of 256 threads an SM at the least): a block
    // waits for the same block of the other ranks, which must not sit behind blocks that wait themselves
    const int64_t blocks = (int64_t)p.q_heads * p.n_rows * p.columns;
    if (blocks <= 4 * (int64_t)sms) return launch_merge_push<true>(p, x, m, (cudaStream_t)stream);
    crit_b200_merge_shards_params none;
    memset(&none, 0, sizeof none);
    if (int e = launch_merge_push<false>(p, x, none, (cudaStream_t)stream)) return e;
    return crit_b200_wait_merge(exchange, merge, stream);
}

extern "C" __attribute__((visibility("default"))) int crit_b200_attend_plan(int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                                                            int32_t value_dim, int32_t page, int32_t kind,
                                                                            int32_t page_dtype, int32_t columns, int32_t* out5) {
    if (!out5 || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads || columns < 1) return CRIT_B200_EINVAL;
    if (page < 16 || page % 16) return CRIT_B200_EUNSUPPORTED;
    const int rows = columns * (q_heads / kv_heads);
    const int nt = row_tiles(rows, value_dim);
    Variant v;
    int e = pick(kind, page_dtype, head_dim, value_dim, nt, false, &v);
    if (e) return e;
    const int smem = v.smem(128);
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) == cudaSuccess) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (cudaFuncSetAttribute((const void*)v.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess)
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)v.fn, DECODE_THREADS, smem);
    }
    cudaGetLastError();
    out5[0] = 1024;
    out5[1] = smem;
    out5[2] = 8 * nt;
    out5[3] = per_sm;
    out5[4] = sms;
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_decode(const crit_b200_attend_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    int e = check(*params);
    return e ? e : launch_decode(*params, (cudaStream_t)stream);
}

extern "C" __attribute__((visibility("default"))) int crit_b200_merge(const crit_b200_attend_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    int e = check(*params);
    return e ? e : launch_merge(*params, (cudaStream_t)stream);
}

extern "C" __attribute__((visibility("default"))) int crit_b200_attend(const crit_b200_attend_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    int e = check(*params);
    if (e) return e;
    e = launch_decode(*params, (cudaStream_t)stream);
    return e ? e : launch_merge(*params, (cudaStream_t)stream);
}
