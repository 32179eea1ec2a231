// Block-table page gather with dequantisation, slot mapping on the device, and the merge of shards' partials.
#include "common.cuh"

namespace crit_b200 {

// One warp per (position, kv head): out = code * scale in FP32, rounded to TOUT.
// Reference: inference/attention-state/code/pages.py:455-493 (gather, rows_at).
template <typename TOUT>
__global__ void __launch_bounds__(128) gather_kernel(const crit_b200_gather_params p) {
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= p.count * p.kv_heads) return;
    const int64_t n = item / p.kv_heads;
    const int h = (int)(item % p.kv_heads);
    int64_t slot;
    if (p.slots) slot = p.slots[n];
    else slot = (int64_t)p.table[n / p.page] * p.page + n % p.page;
    TOUT* dst = (TOUT*)p.out + item * p.dim;
    if (p.slots_total && (slot < 0 || slot >= p.slots_total)) {      // outside the page tensor: zeros, and reported
        if (lane == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_BOUNDS);
        for (int i = lane; i < p.dim; i += 32) dst[i] = from_float<TOUT>(0.f);
        return;
    }
    const int64_t row = slot * p.kv_heads + h;
    float scale = p.multiplier;
    if (p.kind == CRIT_B200_KIND_FP8_ROW || p.kind == CRIT_B200_KIND_INT8) scale = p.scales[row];
    else if (p.kind == CRIT_B200_KIND_FP8_PAGE) scale = p.scales[(slot / p.page) * p.kv_heads + h];
    for (int i = lane; i < p.dim; i += 32) {
        float v;
        if (p.kind == CRIT_B200_KIND_16BIT) {
            if (p.page_dtype == CRIT_B200_DTYPE_BF16) v = __bfloat162float(((const __nv_bfloat16*)p.pages)[row * p.dim + i]);
            else if (p.page_dtype == CRIT_B200_DTYPE_FP16) v = __half2float(((const __half*)p.pages)[row * p.dim + i]);
            else v = ((const float*)p.pages)[row * p.dim + i];
        } else if (p.kind == CRIT_B200_KIND_INT8) {
            v = __fmul_rn((float)((const int8_t*)p.pages)[row * p.dim + i], scale);
        } else {
            v = __fmul_rn(e4m3_to_float(((const uint8_t*)p.pages)[row * p.dim + i]), scale);
        }
        dst[i] = from_float<TOUT>(v);
    }
}

// Reference: pages.py:653-660 (_slots_at) and :721-722 (_slot).
__global__ void slots_kernel(const crit_b200_slots_params p) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    const int64_t pos = p.positions[i], row = p.rows[i];
    int64_t col = pos >= 0 ? pos / p.page : -((-pos + p.page - 1) / p.page);
    col = col < 0 ? 0 : (col > p.table_width - 1 ? p.table_width - 1 : col);
    const int64_t rem = ((pos % p.page) + p.page) % p.page;
    const bool inside = p.capacity ? (pos >= 0 && pos < p.capacity[row]) : true;
    p.slots[i] = inside ? (int64_t)p.tables[row * p.table_stride + col] * p.page + rem : (int64_t)p.dump * p.page;
}

// One warp per (token, head) row: top = max lse; w = exp(lse - top), 0 for -inf; out = sum w o / sum w;
// lse = top + log(sum w).  Reference: inference/partitioned-attention/plugin.py:52-64.
template <typename TIN, typename TOUT>
__global__ void __launch_bounds__(128) merge_shards_kernel(const crit_b200_merge_shards_params p) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (i >= p.n) return;
    float top = -INFINITY;
    for (int s = 0; s < p.parts; ++s) top = fmaxf(top, p.lses[(int64_t)s * p.n + i]);
    const float sub = top == -INFINITY ? 0.f : top;
    float total = 0.f;
    for (int s = 0; s < p.parts; ++s) {
        float l = p.lses[(int64_t)s * p.n + i];
        total += l == -INFINITY ? 0.f : expf(l - sub);
    }
    const float denom = fmaxf(total, 1e-30f);
    for (int c = lane; c < p.dim; c += 32) {
        float acc = 0.f;
        for (int s = 0; s < p.parts; ++s) {
            float l = p.lses[(int64_t)s * p.n + i];
            float w = l == -INFINITY ? 0.f : expf(l - sub);
            acc += w * to_float<TIN>(((const TIN*)p.outs)[((int64_t)s * p.n + i) * p.dim + c]);
        }
        ((TOUT*)p.out)[i * p.dim + c] = from_float<TOUT>(total > 0.f ? acc / denom : 0.f);
    }
    if (lane == 0 && p.lse) p.lse[i] = total > 0.f ? sub + logf(denom) : -INFINITY;
}

}  // namespace crit_b200

using namespace crit_b200;

extern "C" __attribute__((visibility("default"))) int crit_b200_gather(const crit_b200_gather_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_gather_params p = *params;
    if (p.count == 0) return 0;
    if (p.count < 0 || !p.pages || !p.out || (!p.table && !p.slots) || p.kv_heads < 1 || p.dim < 1 || p.page < 1)
        return CRIT_B200_EINVAL;
    if (p.kind >= CRIT_B200_KIND_FP8_ROW && !p.scales) return CRIT_B200_EINVAL;
    const unsigned grid = (unsigned)((p.count * p.kv_heads + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    switch (p.out_dtype) {
        case CRIT_B200_DTYPE_BF16: gather_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(p); break;
        case CRIT_B200_DTYPE_FP16: gather_kernel<__half><<<grid, 128, 0, s>>>(p); break;
        case CRIT_B200_DTYPE_FP32: gather_kernel<float><<<grid, 128, 0, s>>>(p); break;
        default: return CRIT_B200_EINVAL;
    }
    CRIT_CHECK_LAUNCH();
    return 0;
}

namespace crit_b200 {

// Block = (list, layer): the list's moves in order, each a copy of row_bytes bytes by the block's threads.
__global__ void __launch_bounds__(128) move_rows_kernel(const crit_b200_move_params p) {
    const int64_t list = blockIdx.x;
    const int layer = blockIdx.y;
    uint32_t* base = reinterpret_cast<uint32_t*>((char*)p.store + (int64_t)layer * p.slots * p.row_bytes);
    const int64_t words = p.row_bytes >> 2;
    for (int64_t j = 0; j < p.width; ++j) {
        const int64_t from = p.source[list * p.width + j], to = p.target[list * p.width + j];
        if (from == to) continue;                           // (block-uniform)
        if (from < 0 || from >= p.slots || to < 0 || to >= p.slots) {
            if (threadIdx.x == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_BOUNDS);
            continue;
        }
        const uint32_t* src = base + from * words;
        uint32_t* dst = base + to * words;
        for (int64_t w = threadIdx.x; w < words; w += blockDim.x) dst[w] = src[w];
        __syncthreads();                                     // the next move of the list may read this one's target
    }
}

}  // namespace crit_b200

namespace crit_b200 {

// Thread = (window row, column): the token's listed blocks as a page table of its own (see crit_b200_compact_params).
__global__ void __launch_bounds__(128) compact_blocks_kernel(const crit_b200_compact_params p) {
    const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= p.n_rows * p.columns) return;
    const int64_t r = item / p.columns;
    const int c = (int)(item - r * p.columns);
    int count = p.counts ? p.counts[r] : p.columns;
    count = count > p.columns ? p.columns : count;
    const int per = p.block_size / p.page;                       // pages a block holds
    int32_t* table = p.out_tables + item * ((int64_t)p.blocks_k * per);
    p.out_counts[item] = 0, p.out_firsts[item] = 0;
    if (c >= count) return;
    const int64_t token = p.starts[r] + c, pos = p.firsts[r] + c;
    const int32_t* from = p.tables + (int64_t)p.rows[r] * p.table_stride;
    const int32_t* listed = p.blocks + token * p.blocks_k;
    const int64_t own = pos / p.block_size;
    int placed = 0;
    bool has_own = false;
    for (int j = 0; j < p.blocks_k; ++j) {
        const int64_t b = listed[j];
        if (b < 0 || b > own) continue;                          // none, or wholly after the token's position
        bool twice = false;
        for (int i = 0; i < j; ++i) twice |= listed[i] == b;
        if (twice) continue;
        if (b == own) {                                          // goes last
            has_own = true;
            continue;
        }
        for (int i = 0; i < per; ++i) {
            const int64_t at = b * per + i;
            table[placed * per + i] = at < p.table_width ? from[at] : p.dump;
        }
        ++placed;
    }
    int64_t length = (int64_t)placed * p.block_size;
    if (has_own) {
        for (int i = 0; i < per; ++i) {
            const int64_t at = own * per + i;
            table[placed * per + i] = at < p.table_width ? from[at] : p.dump;
        }
        ++placed;
        length += pos - own * p.block_size + 1;
    }
    for (int i = placed * per; i < p.blocks_k * per; ++i) table[i] = p.dump;
    if (length > 0) {
        p.out_counts[item] = 1, p.out_firsts[item] = length - 1;
        return;
    }
    // the token sees nothing: zeros and -inf, as the fold of no state gives
    if (p.out) {
        for (int h = 0; h < p.q_heads; ++h)
            for (int d = 0; d < p.value_dim; ++d) {
                const int64_t at = token * p.out_stride_token + (int64_t)h * p.out_stride_head + d;
                if (p.out_dtype == CRIT_B200_DTYPE_BF16) ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(0.f);
                else ((__half*)p.out)[at] = __float2half_rn(0.f);
            }
    }
    if (p.lse)
        for (int h = 0; h < p.q_heads; ++h) p.lse[token * p.q_heads + h] = -INFINITY;
}

}  // namespace crit_b200

extern "C" __attribute__((visibility("default"))) int crit_b200_compact_blocks(const crit_b200_compact_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_compact_params p = *params;
    if (p.n_rows == 0) return 0;
    if (!p.tables || !p.rows || !p.starts || !p.firsts || !p.blocks || !p.out_tables || !p.out_counts || !p.out_firsts ||
        p.n_rows < 0 || p.columns < 1 || p.blocks_k < 1 || p.page < 1 || p.block_size < p.page || p.block_size % p.page ||
        p.table_width < 1)
        return CRIT_B200_EINVAL;
    if (p.out && p.out_dtype != CRIT_B200_DTYPE_BF16 && p.out_dtype != CRIT_B200_DTYPE_FP16) return CRIT_B200_EUNSUPPORTED;
    const int64_t items = p.n_rows * p.columns;
    crit_b200::compact_blocks_kernel<<<(unsigned)((items + 127) / 128), 128, 0, (cudaStream_t)stream>>>(p);
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_move_rows(const crit_b200_move_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_move_params p = *params;
    if (p.lists == 0 || p.width == 0) return 0;
    if (!p.store || !p.source || !p.target || p.lists < 0 || p.width < 0 || p.slots < 1 || p.layers < 1 || p.row_bytes < 4 ||
        p.row_bytes % 4 || p.lists > 0x7fffffffLL || p.layers > 65535)
        return CRIT_B200_EINVAL;
    dim3 grid((unsigned)p.lists, (unsigned)p.layers);
    crit_b200::move_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(p);
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_slots(const crit_b200_slots_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_slots_params p = *params;
    if (p.n == 0) return 0;
    if (p.n < 0 || !p.tables || !p.rows || !p.positions || !p.slots || p.page < 1 || p.table_width < 1)
        return CRIT_B200_EINVAL;
    slots_kernel<<<(unsigned)((p.n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p);
    CRIT_CHECK_LAUNCH();
    return 0;
}

extern "C" __attribute__((visibility("default"))) int crit_b200_merge_shards(const crit_b200_merge_shards_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_merge_shards_params p = *params;
    if (p.n == 0) return 0;
    if (p.n < 0 || p.parts < 1 || p.dim < 1 || !p.outs || !p.lses || !p.out) return CRIT_B200_EINVAL;
    const unsigned grid = (unsigned)((p.n + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
#define CRIT_MS(TI, TO) merge_shards_kernel<TI, TO><<<grid, 128, 0, s>>>(p)
    const int key = p.in_dtype * 3 + p.out_dtype;
    switch (key) {
        case 0: CRIT_MS(__nv_bfloat16, __nv_bfloat16); break;
        case 1: CRIT_MS(__nv_bfloat16, __half); break;
        case 2: CRIT_MS(__nv_bfloat16, float); break;
        case 3: CRIT_MS(__half, __nv_bfloat16); break;
        case 4: CRIT_MS(__half, __half); break;
        case 5: CRIT_MS(__half, float); break;
        case 6: CRIT_MS(float, __nv_bfloat16); break;
        case 7: CRIT_MS(float, __half); break;
        case 8: CRIT_MS(float, float); break;
        default: return CRIT_B200_EINVAL;
    }
#undef CRIT_MS
    CRIT_CHECK_LAUNCH();
    return 0;
}
