// KV append into pages: one warp per (token, kv head) of the keys, then of the values; a slot below 0 is skipped.
// The codes and scales equal the reference's rules bit for bit: every division is an IEEE division (__fdiv_rn), the
// E4M3 conversion is the hardware's round-to-nearest-even with saturation, and nothing here is compiled with
// fast-math.  Reference: paged_kv_attention/_kernels.py:112-150 (_write_kernel) and
// inference/attention-state/code/pages.py:420-453, :872-895.
#include <type_traits>

#include "common.cuh"

namespace crit_b200 {

constexpr int APPEND_WARPS = 4;

template <typename TIN>
__device__ __forceinline__ void load_row(const TIN* src, int dim, int lane, float (&x)[8]) {
    // dim <= 256: lane holds elements lane*per .. lane*per+per-1, per = dim / 32 (contiguous, vectorisable)
    const int per = dim >> 5;
    if constexpr (sizeof(TIN) == 2) {
        if ((per == 4 || per == 8) && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            // 16-bit rows of 128 or 256 elements: the lane's elements in one 8- or 16-byte load, unpacked in registers
            uint32_t w[4] = {0u, 0u, 0u, 0u};
            if (per == 4) {
                const uint2 v = *reinterpret_cast<const uint2*>(src + lane * 4);
                w[0] = v.x, w[1] = v.y;
            } else {
                const uint4 v = *reinterpret_cast<const uint4*>(src + lane * 8);
                w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 f;
                if constexpr (std::is_same<TIN, __nv_bfloat16>::value) f = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
                else f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                x[2 * i] = 2 * i < per ? f.x : 0.f, x[2 * i + 1] = 2 * i + 1 < per ? f.y : 0.f;
            }
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = i < per ? to_float<TIN>(src[lane * per + i]) : 0.f;
}

__device__ __forceinline__ float row_amax(const float (&x)[8], int per, bool& nan) {
    float a = 0.f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < per) {
            float v = fabsf(x[i]);
            bad |= (v != v);
            a = fmaxf(a, v);
        }
    a = warp_max(a);
    nan = __any_sync(0xffffffffu, bad);
    return a;
}

__device__ __forceinline__ float floor_scale(float amax, float top, bool nan) {
    float s = __fdiv_rn(amax, top);
    if (nan) return __int_as_float(0x7fc00000);
    return fmaxf(s, 1e-30f);
}

template <typename TPAGE>
__device__ __forceinline__ void store_16bit(TPAGE* dst, const float (&x)[8], int per, int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < per) dst[lane * per + i] = from_float<TPAGE>(x[i]);
}

// A lane's `per` consecutive codes as one store where they fill a word or two (heads of 128 or 256), else byte by byte.
__device__ __forceinline__ void store_codes(uint8_t* dst, const uint8_t (&c)[8], int per, int lane) {
    if (per == 4) {
        *reinterpret_cast<uint32_t*>(dst + lane * 4) = (uint32_t)c[0] | ((uint32_t)c[1] << 8) | ((uint32_t)c[2] << 16) | ((uint32_t)c[3] << 24);
    } else if (per == 8) {
        *reinterpret_cast<uint2*>(dst + lane * 8) =
            make_uint2((uint32_t)c[0] | ((uint32_t)c[1] << 8) | ((uint32_t)c[2] << 16) | ((uint32_t)c[3] << 24),
                       (uint32_t)c[4] | ((uint32_t)c[5] << 8) | ((uint32_t)c[6] << 16) | ((uint32_t)c[7] << 24));
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < per) dst[lane * per + i] = c[i];
    }
}

__device__ __forceinline__ void store_e4m3(uint8_t* dst, const float (&x)[8], float div, int per, int lane) {
    uint8_t c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = i < per ? float_to_e4m3(__fdiv_rn(x[i], div)) : (uint8_t)0;
    store_codes(dst, c, per, lane);
}

__device__ __forceinline__ void store_int8(int8_t* dst, const float (&x)[8], float div, int per, int lane) {
    uint8_t c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float y = rintf(__fdiv_rn(x[i], div));
        y = fminf(fmaxf(y, -127.f), 127.f);
        c[i] = i < per ? (uint8_t)(int8_t)y : (uint8_t)0;
    }
    store_codes(reinterpret_cast<uint8_t*>(dst), c, per, lane);
}

template <typename TIN>
__global__ void __launch_bounds__(APPEND_WARPS * 32) append_kernel(const crit_b200_append_params p, int heads_total) {
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * APPEND_WARPS + (threadIdx.x >> 5);
    if (item >= p.tokens * heads_total) return;
    const int64_t t = item / heads_total;
    const int hh = (int)(item % heads_total);
    const bool is_v = hh >= p.kv_heads;
    const int h = is_v ? hh - p.kv_heads : hh;
    const int64_t slot = p.slots[t];
    if (slot < 0) return;
    if (p.slots_total && slot >= p.slots_total) {         // outside the page tensor: skipped and reported, never written
        if (lane == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_BOUNDS);
        return;
    }
    const int dim = is_v ? p.value_dim : p.head_dim;
    const int per = dim >> 5;
    const TIN* src = is_v ? (const TIN*)p.values + t * p.value_stride_token + (int64_t)h * p.value_stride_head
                          : (const TIN*)p.keys + t * p.key_stride_token + (int64_t)h * p.key_stride_head;
    char* pages = (char*)(is_v ? p.value_pages : p.key_pages);
    float* scales = is_v ? p.value_scales : p.key_scales;
    const int64_t row = slot * p.kv_heads + h;

    if (p.kind == CRIT_B200_KIND_FP8_PAGE) {
        // One warp serves a run: consecutive tokens whose slots ascend by one inside one page.  The run's first token
        // leads; the others leave.
        const int64_t pg = slot / p.page;
        if (t > 0) {
            int64_t before = p.slots[t - 1];
            if (before >= 0 && before + 1 == slot && before / p.page == pg) return;
        }
        int64_t end = t + 1;
        while (end < p.tokens && end - t < p.page) {
            int64_t s = p.slots[end];
            if (s != p.slots[end - 1] + 1 || s / p.page != pg) break;
            ++end;
        }
        const int64_t stride_t = is_v ? p.value_stride_token : p.key_stride_token;
        float amax = 0.f;
        bool nan = false;
        for (int64_t r = t; r < end; ++r) {
            float x[8];
            load_row<TIN>(src + (r - t) * stride_t, dim, lane, x);
            bool bad;
            amax = fmaxf(amax, row_amax(x, per, bad));
            nan |= bad;
        }
        float scale = floor_scale(amax, 448.f, nan);
        const int first = (int)(slot % p.page);
        float* sdst = scales + pg * p.kv_heads + h;
        if (first > 0) {
            const float old = *sdst;
            scale = (scale > old || nan) ? scale : old;
            if (scale != old) {
                for (int o = 0; o < first; ++o) {
                    uint8_t* codes = (uint8_t*)pages + ((pg * p.page + o) * p.kv_heads + h) * dim;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (i < per) {
                            float v = __fdiv_rn(__fmul_rn(e4m3_to_float(codes[lane * per + i]), old), scale);
                            codes[lane * per + i] = float_to_e4m3(v);
                        }
                }
            }
        }
        __syncwarp();
        if (lane == 0) *sdst = scale;
        for (int64_t r = t; r < end; ++r) {
            float x[8];
            load_row<TIN>(src + (r - t) * stride_t, dim, lane, x);
            store_e4m3((uint8_t*)pages + ((slot + (r - t)) * p.kv_heads + h) * dim, x, scale, per, lane);
        }
        return;
    }

    float x[8];
    load_row<TIN>(src, dim, lane, x);
    if (p.kind == CRIT_B200_KIND_16BIT) {
        if (p.page_dtype == CRIT_B200_DTYPE_BF16) store_16bit((__nv_bfloat16*)pages + row * dim, x, per, lane);
        else if (p.page_dtype == CRIT_B200_DTYPE_FP16) store_16bit((__half*)pages + row * dim, x, per, lane);
        else store_16bit((float*)pages + row * dim, x, per, lane);
    } else if (p.kind == CRIT_B200_KIND_FP8) {
        store_e4m3((uint8_t*)pages + row * dim, x, is_v ? p.value_multiplier : p.key_multiplier, per, lane);
    } else {
        bool nan;
        const float top = p.kind == CRIT_B200_KIND_FP8_ROW ? 448.f : 127.f;
        const float scale = floor_scale(row_amax(x, per, nan), top, nan);
        if (p.kind == CRIT_B200_KIND_FP8_ROW) store_e4m3((uint8_t*)pages + row * dim, x, scale, per, lane);
        else store_int8((int8_t*)pages + row * dim, x, scale, per, lane);
        if (lane == 0) scales[row] = scale;
    }
}

}  // namespace crit_b200

using namespace crit_b200;

extern "C" __attribute__((visibility("default"))) int crit_b200_append(const crit_b200_append_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_append_params p = *params;
    if (p.tokens == 0) return 0;
    if (p.tokens < 0 || !p.keys || !p.slots || !p.key_pages || p.kv_heads < 1 || p.page < 1) return CRIT_B200_EINVAL;
    if (p.values && !p.value_pages) return CRIT_B200_EINVAL;
    auto width_ok = [](int d) { return d >= 32 && d <= 256 && d % 32 == 0; };
    if (!width_ok(p.head_dim) || (p.values && !width_ok(p.value_dim))) return CRIT_B200_EUNSUPPORTED;
    if (p.kind < 0 || p.kind > CRIT_B200_KIND_FP8_PAGE) return CRIT_B200_EUNSUPPORTED;
    if (p.kind >= CRIT_B200_KIND_FP8_ROW && (!p.key_scales || (p.values && !p.value_scales))) return CRIT_B200_EINVAL;
    if (p.kind == CRIT_B200_KIND_16BIT && p.page_dtype == CRIT_B200_DTYPE_FP32 && p.in_dtype != CRIT_B200_DTYPE_FP32)
        ;   // widening into FP32 pages is served too
    const int heads_total = p.values ? 2 * p.kv_heads : p.kv_heads;
    const int64_t items = p.tokens * heads_total;
    const unsigned grid = (unsigned)((items + APPEND_WARPS - 1) / APPEND_WARPS);
    cudaStream_t s = (cudaStream_t)stream;
    switch (p.in_dtype) {
        case CRIT_B200_DTYPE_BF16: append_kernel<__nv_bfloat16><<<grid, APPEND_WARPS * 32, 0, s>>>(p, heads_total); break;
        case CRIT_B200_DTYPE_FP16: append_kernel<__half><<<grid, APPEND_WARPS * 32, 0, s>>>(p, heads_total); break;
        case CRIT_B200_DTYPE_FP32: append_kernel<float><<<grid, APPEND_WARPS * 32, 0, s>>>(p, heads_total); break;
        default: return CRIT_B200_EINVAL;
    }
    CRIT_CHECK_LAUNCH();
    return 0;
}
