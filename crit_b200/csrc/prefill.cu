// Chunked prefill: one sequence's chunk of queries at positions position.. over its paged keys and values, causal.
//
// A block holds a tile of 64 query rows (a query row is one (token, query head of a kv head's group) pair, token-major,
// so a GQA group shares every key and value byte) and walks the sequence's positions in tiles of 64 (four pages of
// 16), staged by all four warps with cp.async into a two-stage ring; each warp owns 16 query rows (m16n8k16 MMAs, FP32
// accumulators, the online softmax of its rows in registers, one update per 64 positions).  8-bit pages are converted
// to FP16 in registers (the permuted orders of decode_kernel.cuh).  Only the tiles that straddle a row's own position
// are masked; tiles past the block's last visible position are never read.
// Reference: paged_kv_attention/_kernels.py:610-726 (_prefill_kernel), __init__.py:1245-1332 (prefill); the reference
// runs one program per (64 queries, query head), re-reading a kv head's pages once per query head of its group.
#include "decode_kernel.cuh"
#include "prefill_pair.cuh"
#include "prefill_tc.cuh"
#include "tensor_map.cuh"

namespace crit_b200 {

constexpr int PF_WARPS = 4;
constexpr int PF_THREADS = PF_WARPS * 32;
constexpr int PF_ROWS = 64;        // query rows a block holds
constexpr int PF_BN = 64;          // positions a stage holds

template <int D, int PK>
struct PrefillCfg {
    static constexpr int ES = PK < 2 ? 2 : 1;
    static constexpr int ROWB = D * ES;                 // bytes of a key or value row
    static constexpr int TILE = PF_BN * ROWB;
    static constexpr int STAGE = 2 * TILE + 2 * PF_BN * 4;      // keys, values, key scales, value scales
    static constexpr int QROW = D * 2 + (ES == 1 ? 16 : 0);
    static constexpr int QBYTES = PF_ROWS * QROW;
    static constexpr int SMEM = QBYTES + 2 * STAGE;
};

template <int D, int PK>
__global__ void __launch_bounds__(PF_THREADS) prefill_kernel(const crit_b200_prefill_params p, const int smode) {
    using C = PrefillCfg<D, PK>;
    constexpr int ES = C::ES;
    constexpr bool BF16 = PK == 0;
    constexpr int CH = C::ROWB / 16;                    // 16-byte chunks of a row
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* qs = smem;
    unsigned char* ring = smem + C::QBYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int h = blockIdx.y;
    const int G = p.q_heads / p.kv_heads;
    const int row0 = blockIdx.x * PF_ROWS;              // first query row (token * G + head in group) of the block
    const int seq = blockIdx.z;                         // one sequence of the launch
    const int tok0 = p.starts ? p.starts[seq] : seq * p.tokens;
    const int rows_total = (p.starts ? p.starts[seq + 1] - tok0 : p.tokens) * G;
    if (row0 >= rows_total) return;                     // a shorter sequence of a ragged launch
    const int32_t* table = p.table + (int64_t)seq * p.table_stride;
    const int64_t position = p.positions ? p.positions[seq] : (p.position_ptr ? *p.position_ptr : p.position);
    const int pos32 = (int)position;

    // -- queries into shared memory ----------------------------------------------------------------------------------
    {
        constexpr int CPR = D / 8;
        for (int idx = tid; idx < PF_ROWS * CPR; idx += PF_THREADS) {
            const int rr = idx / CPR, c = idx - rr * CPR;
            const int flat = row0 + rr;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (flat < rows_total) {
                const int tok = flat / G, gq = flat - tok * G;
                const char* src = (const char*)p.q + ((int64_t)(tok0 + tok) * p.q_stride_token + (int64_t)(h * G + gq) * p.q_stride_head + c * 8) * 2;
                v = *reinterpret_cast<const uint4*>(src);
            }
            if constexpr (ES == 2) {
                *reinterpret_cast<uint4*>(qs + rr * C::QROW + swz16(c, rr) * 16) = v;
            } else {
                if (p.q_dtype == CRIT_B200_DTYPE_BF16) {
                    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[i]));
                        f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
                        f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
                        __half2 hh = __floats2half2_rn(f.x, f.y);
                        w[i] = *reinterpret_cast<uint32_t*>(&hh);
                    }
                    v = make_uint4(w[0], w[1], w[2], w[3]);
                }
                *reinterpret_cast<uint4*>(qs + rr * C::QROW + c * 16) = v;
            }
        }
    }
    __syncthreads();

    // this warp's 16 query rows: fragments of Q (A operand), the last position each of the thread's two rows sees
    uint32_t qa[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        if constexpr (ES == 2) {
            const int j = lane >> 3, row = warp * 16 + (lane & 7) + 8 * (j & 1), chunk = 2 * ks + (j >> 1);
            ldmatrix_x4(qa[ks], smem_addr(qs + row * C::QROW + swz16(chunk, row) * 16));
        } else {
            const int row = warp * 16 + g;
            const uint2 lo = *reinterpret_cast<const uint2*>(qs + row * C::QROW + (t * (D / 4) + 4 * ks) * 2);
            const uint2 hi = *reinterpret_cast<const uint2*>(qs + (row + 8) * C::QROW + (t * (D / 4) + 4 * ks) * 2);
            qa[ks][0] = lo.x, qa[ks][1] = hi.x, qa[ks][2] = lo.y, qa[ks][3] = hi.y;
        }
    }
    int lastpos[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        const int flat = row0 + warp * 16 + g + 8 * hf;
        lastpos[hf] = flat < rows_total ? pos32 + flat / G : -1;
    }
    // the block reads positions up to its last row's own; tiles wholly at or before its first row's position need no mask
    const int last_row = (row0 + PF_ROWS < rows_total ? row0 + PF_ROWS : rows_total) - 1;
    const int end = pos32 + last_row / G + 1;
    const int clear = pos32 + row0 / G;                 // positions <= clear are seen by every row of the block
    const int ntiles = (end + PF_BN - 1) / PF_BN;

    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float kmul = (PK == 2 && smode == 0) ? p.key_multiplier : 1.f;
    const float sl2 = p.scale * LOG2E * kmul;
    const char* kbase = (const char*)p.key_pages + (int64_t)h * C::ROWB;
    const char* vbase = (const char*)p.value_pages + (int64_t)h * C::ROWB;
    const int64_t row_stride = (int64_t)p.kv_heads * C::ROWB;
    const int pages_per_tile = PF_BN / 16;
    const uint32_t tiles_per_page = (uint32_t)p.page >> 4;

    auto issue = [&](int i) {
        if (i < ntiles) {
            unsigned char* st = ring + (i & 1) * C::STAGE;
            const uint32_t ks = smem_addr(st), vs = ks + C::TILE, sc = vs + C::TILE;
            // 64 rows x CH chunks for keys and as many for values: each thread's rows come from one 16-position group
#pragma unroll
            for (int u = 0; u < PF_BN * CH / PF_THREADS; ++u) {
                const int id = tid + PF_THREADS * u, row = id / CH, c = id - row * CH;
                const uint32_t tile16 = (uint32_t)(i * pages_per_tile + (row >> 4));
                const uint32_t pidx = tile16 / tiles_per_page;
                const int pos = i * PF_BN + row;
                const bool ok = pos < end;
                const int64_t slot = ok ? (int64_t)table[pidx] * p.page + ((tile16 - pidx * tiles_per_page) << 4) + (row & 15) : 0;
                const int kc = ES == 2 ? swz16(c, row) : kswz8<D>(row, c);
                const int vc = ES == 2 ? swz16(c, row) : vswz8<D>(row, c);
                cp_async16(ks + row * C::ROWB + kc * 16, kbase + slot * row_stride + c * 16, ok);
                cp_async16(vs + row * C::ROWB + vc * 16, vbase + slot * row_stride + c * 16, ok);
            }
            if (PK >= 2 && smode) {
                const int row = tid & 63;
                const uint32_t tile16 = (uint32_t)(i * pages_per_tile + (row >> 4));
                const uint32_t pidx = tile16 / tiles_per_page;
                const bool ok = i * PF_BN + row < end;
                const int64_t pg = ok ? table[pidx] : 0;
                const int64_t slot = pg * p.page + ((tile16 - pidx * tiles_per_page) << 4) + (row & 15);
                const float* src = tid < 64 ? p.key_scales : p.value_scales;
                cp_async4(sc + tid * 4, src + (smode == 2 ? pg * p.kv_heads + h : slot * p.kv_heads + h), ok);
            }
        }
        cp_async_commit();
    };

    issue(0);
    for (int i = 0; i < ntiles; ++i) {
        issue(i + 1);
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* kst = ring + (i & 1) * C::STAGE;
        const unsigned char* vst = kst + C::TILE;
        const float* scales = reinterpret_cast<const float*>(vst + C::TILE);
        const int tile_pos = i * PF_BN;

        // scores: S[16 rows x 64 positions] = Q K^T
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
        if constexpr (ES == 2) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t kb[4];
                    const int j = lane >> 3, tok = np * 16 + (lane & 7) + 8 * (j >> 1), chunk = 2 * ks + (j & 1);
                    ldmatrix_x4(kb, smem_addr(kst + tok * C::ROWB + swz16(chunk, tok) * 16));
                    mma16816<BF16>(s[2 * np], qa[ks], kb[0], kb[1]);
                    mma16816<BF16>(s[2 * np + 1], qa[ks], kb[2], kb[3]);
                }
        } else {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t kw[2][D / 16];
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    const int row = np * 16 + g + 8 * n;
#pragma unroll
                    for (int qd = 0; qd < D / 64; ++qd) {
                        const int c = t * (D / 64) + qd;
                        const uint4 v = *reinterpret_cast<const uint4*>(kst + row * C::ROWB + kswz8<D>(row, c) * 16);
                        kw[n][qd * 4 + 0] = v.x, kw[n][qd * 4 + 1] = v.y, kw[n][qd * 4 + 2] = v.z, kw[n][qd * 4 + 3] = v.w;
                    }
                }
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t kb[4];
                    code4_to_f16x2x2<PK == 3>(kw[0][ks], kb[0], kb[1]);
                    code4_to_f16x2x2<PK == 3>(kw[1][ks], kb[2], kb[3]);
                    mma16816<BF16>(s[2 * np], qa[ks], kb[0], kb[1]);
                    mma16816<BF16>(s[2 * np + 1], qa[ks], kb[2], kb[3]);
                }
            }
        }

        // scale, mask, online softmax (base 2), one update per 64 positions
        const bool masked = tile_pos + PF_BN - 1 > clear;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int col = n * 8 + 2 * t + (e & 1);
                float x = s[n][e] * sl2;
                if (PK >= 2 && smode) x *= scales[col];
                if (masked && tile_pos + col > lastpos[e >> 1]) x = -INFINITY;
                s[n][e] = x;
                mx[e >> 1] = fmaxf(mx[e >> 1], x);
            }
        float alpha[2];
        bool rescale = false;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
            mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
            const bool moved = mx[hf] > m_run[hf] + LAZY || m_run[hf] == -INFINITY;
            const float top = moved ? mx[hf] : m_run[hf];
            const float sub = top == -INFINITY ? 0.f : top;
            alpha[hf] = moved ? ex2(m_run[hf] - sub) : 1.f;
            rescale |= moved && top != m_run[hf];
            m_run[hf] = top;
            mx[hf] = sub;
        }
        float sum[2] = {0.f, 0.f};
        uint32_t pa[4][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            float pr[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = ex2(s[n][e] - mx[e >> 1]);
                sum[e >> 1] += pv;
                float scaled = pv;
                if (PK >= 2 && smode) {
                    scaled = pv * scales[PF_BN + n * 8 + 2 * t + (e & 1)];
                    if (masked && s[n][e] == -INFINITY) scaled = 0.f;
                }
                pr[e] = scaled;
            }
            pa[n >> 1][(n & 1) * 2 + 0] = pack2<BF16>(pr[0], pr[1]);
            pa[n >> 1][(n & 1) * 2 + 1] = pack2<BF16>(pr[2], pr[3]);
        }
        l_run[0] = l_run[0] * alpha[0] + sum[0];
        l_run[1] = l_run[1] * alpha[1] + sum[1];
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                acc[n][0] *= alpha[0], acc[n][1] *= alpha[0];
                acc[n][2] *= alpha[1], acc[n][3] *= alpha[1];
            }
        }

        // outputs: O[16 rows x D] += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            if constexpr (ES == 2) {
#pragma unroll
                for (int np = 0; np < D / 16; ++np) {
                    uint32_t vb[4];
                    const int j = lane >> 3, tok = kk * 16 + (lane & 7) + 8 * (j & 1), chunk = 2 * np + (j >> 1);
                    ldmatrix_x4_trans(vb, smem_addr(vst + tok * C::ROWB + swz16(chunk, tok) * 16));
                    mma16816<BF16>(acc[2 * np], pa[kk], vb[0], vb[1]);
                    mma16816<BF16>(acc[2 * np + 1], pa[kk], vb[2], vb[3]);
                }
            } else {
                constexpr int VW = D / 32;
                uint32_t vw[4][VW];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int row = kk * 16 + 2 * t + (q4 & 1) + 8 * (q4 >> 1);
                    if constexpr (D == 64) {
                        const uint2 v = *reinterpret_cast<const uint2*>(vst + row * C::ROWB + vswz8<D>(row, g >> 1) * 16 + (g & 1) * 8);
                        vw[q4][0] = v.x, vw[q4][1] = v.y;
                    } else {
#pragma unroll
                        for (int qd = 0; qd < D / 128; ++qd) {
                            const int c = g * (D / 128) + qd;
                            const uint4 v = *reinterpret_cast<const uint4*>(vst + row * C::ROWB + vswz8<D>(row, c) * 16);
                            vw[q4][qd * 4 + 0] = v.x, vw[q4][qd * 4 + 1] = v.y, vw[q4][qd * 4 + 2] = v.z, vw[q4][qd * 4 + 3] = v.w;
                        }
                    }
                }
#pragma unroll
                for (int np = 0; np < D / 16; ++np) {
                    const int w = np >> 1;
                    const uint32_t sel = (np & 1) ? 0x7362u : 0x5140u;
                    uint32_t b00, b01, b10, b11;
                    code4_to_f16x2x2<PK == 3>(__byte_perm(vw[0][w], vw[1][w], sel), b00, b10);
                    code4_to_f16x2x2<PK == 3>(__byte_perm(vw[2][w], vw[3][w], sel), b01, b11);
                    mma16816<BF16>(acc[2 * np], pa[kk], b00, b01);
                    mma16816<BF16>(acc[2 * np + 1], pa[kk], b10, b11);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    // -- write the rows out ------------------------------------------------------------------------------------------
    const float vmul = (PK == 2 && smode == 0) ? p.value_multiplier : 1.f;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        float l = l_run[hf];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int flat = row0 + warp * 16 + g + 8 * hf;
        if (flat >= rows_total) continue;
        const int tok = flat / G, gq = flat - tok * G, head = h * G + gq;
        const float inv = l > 0.f ? vmul / l : 0.f;
        char* dst = (char*)p.out + ((int64_t)(tok0 + tok) * p.out_stride_token + (int64_t)head * p.out_stride_head) * 2;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const float a = acc[n][2 * hf] * inv, b = acc[n][2 * hf + 1] * inv;
            if constexpr (ES == 2) {
                *reinterpret_cast<uint32_t*>(dst + (n * 8 + 2 * t) * 2) =
                    p.q_dtype == CRIT_B200_DTYPE_BF16 ? pack2<true>(a, b) : pack2<false>(a, b);
            } else {
                const int c0 = (2 * t) * (D / 8) + n, c1 = (2 * t + 1) * (D / 8) + n;
                if (p.q_dtype == CRIT_B200_DTYPE_BF16) {
                    reinterpret_cast<__nv_bfloat16*>(dst)[c0] = __float2bfloat16_rn(a);
                    reinterpret_cast<__nv_bfloat16*>(dst)[c1] = __float2bfloat16_rn(b);
                } else {
                    reinterpret_cast<__half*>(dst)[c0] = __float2half_rn(a);
                    reinterpret_cast<__half*>(dst)[c1] = __float2half_rn(b);
                }
            }
        }
        if (p.lse && t == 0) p.lse[(int64_t)(tok0 + tok) * p.q_heads + head] = l > 0.f ? m_run[hf] * LN2 + logf(l) : -INFINITY;
    }
}

typedef void (*prefill_fn)(const crit_b200_prefill_params, const int);

template <int PK>
static int prefill_pick(int d, prefill_fn* fn, int* smem) {
    if (d == 64) *fn = prefill_kernel<64, PK>, *smem = PrefillCfg<64, PK>::SMEM;
    else if (d == 128) *fn = prefill_kernel<128, PK>, *smem = PrefillCfg<128, PK>::SMEM;
    else if (d == 256 && PK < 2) *fn = prefill_kernel<256, PK < 2 ? PK : 0>, *smem = PrefillCfg<256, PK < 2 ? PK : 0>::SMEM;   // 16-bit pages
    else return CRIT_B200_EUNSUPPORTED;
    return 0;
}

}  // namespace crit_b200

using namespace crit_b200;

extern "C" __attribute__((visibility("default"))) int crit_b200_prefill(const crit_b200_prefill_params* params, void* stream) {
    if (!params) return CRIT_B200_EINVAL;
    const crit_b200_prefill_params p = *params;
    if (p.tokens == 0) return 0;
    if (!p.q || !p.out || !p.key_pages || !p.value_pages || !p.table || p.tokens < 0 || p.q_heads < 1 || p.kv_heads < 1 ||
        p.q_heads % p.kv_heads)
        return CRIT_B200_EINVAL;
    if (p.sequences < 0 || (p.sequences > 1 && (!p.positions || p.table_stride < 0 || p.sequences > 65535))) return CRIT_B200_EINVAL;
    const unsigned nseq = p.sequences > 1 ? (unsigned)p.sequences : 1u;
    if (p.page < 16 || p.page % 16 || p.head_dim != p.value_dim) return CRIT_B200_EUNSUPPORTED;
    if (p.q_dtype != CRIT_B200_DTYPE_BF16 && p.q_dtype != CRIT_B200_DTYPE_FP16) return CRIT_B200_EUNSUPPORTED;
    if (p.kind == CRIT_B200_KIND_16BIT && p.page_dtype != p.q_dtype) return CRIT_B200_EUNSUPPORTED;
    const int smode = p.kind == CRIT_B200_KIND_FP8_ROW || p.kind == CRIT_B200_KIND_INT8 ? 1 : (p.kind == CRIT_B200_KIND_FP8_PAGE ? 2 : 0);
    if (smode && (!p.key_scales || !p.value_scales)) return CRIT_B200_EINVAL;
    if (!aligned(p.q, 16) || p.q_stride_token % 8 || p.q_stride_head % 8 || !aligned(p.key_pages, 16) ||
        !aligned(p.value_pages, 16) || !aligned(p.out, 4) || p.out_stride_token % 2 || p.out_stride_head % 2)
        return CRIT_B200_EALIGN;
    const int G = p.q_heads / p.kv_heads;
    // tcgen05 tiles: 16-bit pages of 128-wide heads, with the pool's size known for the tensor maps
    const bool tc_serves = p.kind == CRIT_B200_KIND_16BIT && p.head_dim == TC_D && p.value_dim == TC_D && p.slots >= 16 && p.slots <= 0x7fffffffLL;
    if ((p.flags & CRIT_B200_PREFILL_TCGEN05) && !tc_serves) return CRIT_B200_EUNSUPPORTED;
    if (tc_serves && !(p.flags & CRIT_B200_PREFILL_MMA_SYNC)) {
        const bool bf16 = p.page_dtype == CRIT_B200_DTYPE_BF16;
        CUtensorMap kmap, vmap;
        if (page_map(&kmap, p.key_pages, bf16 ? 0 : 1, p.head_dim, p.kv_heads, p.slots) &&
            page_map(&vmap, p.value_pages, bf16 ? 0 : 1, p.value_dim, p.kv_heads, p.slots)) {
            // blocks of 256 rows (one an SM) once the launch has one for every SM; below that the blocks of 128 fill more SMs
            const int64_t pairs = (int64_t)((p.tokens * G + TP_ROWS - 1) / TP_ROWS) * p.kv_heads * nseq;
            int device = 0, sms = 0;
            if (cudaGetDevice(&device) != cudaSuccess ||
                cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
                sms = 0;
            const bool pair = !(p.flags & CRIT_B200_PREFILL_SINGLE) && ((p.flags & CRIT_B200_PREFILL_PAIR) || (sms > 0 && pairs >= sms));
            if (pair) {
                auto tp = bf16 ? prefill_pair_kernel<true> : prefill_pair_kernel<false>;
                cudaError_t ce = cudaFuncSetAttribute((const void*)tp, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM);
                if (ce != cudaSuccess) return (int)ce;
                dim3 grid((unsigned)((p.tokens * G + TP_ROWS - 1) / TP_ROWS), (unsigned)p.kv_heads, nseq);
                tp<<<grid, TP_THREADS, TP_SMEM, (cudaStream_t)stream>>>(p, kmap, vmap, p.status);
                CRIT_CHECK_LAUNCH();
                return 0;
            }
            auto tc = bf16 ? prefill_tc_kernel<true> : prefill_tc_kernel<false>;
            cudaError_t ce = cudaFuncSetAttribute((const void*)tc, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
            if (ce != cudaSuccess) return (int)ce;
            dim3 grid((unsigned)((p.tokens * G + TC_ROWS - 1) / TC_ROWS), (unsigned)p.kv_heads, nseq);
            tc<<<grid, TC_THREADS, TC_SMEM, (cudaStream_t)stream>>>(p, kmap, vmap, p.status);
            CRIT_CHECK_LAUNCH();
            return 0;
        }
        if (p.flags & CRIT_B200_PREFILL_TCGEN05) return CRIT_B200_EUNSUPPORTED;
    }
    prefill_fn fn = nullptr;
    int smem = 0, e;
    if (p.kind == CRIT_B200_KIND_16BIT) e = p.page_dtype == CRIT_B200_DTYPE_BF16 ? prefill_pick<0>(p.head_dim, &fn, &smem) : prefill_pick<1>(p.head_dim, &fn, &smem);
    else if (p.kind == CRIT_B200_KIND_INT8) e = prefill_pick<3>(p.head_dim, &fn, &smem);
    else if (p.kind >= CRIT_B200_KIND_FP8 && p.kind <= CRIT_B200_KIND_FP8_PAGE) e = prefill_pick<2>(p.head_dim, &fn, &smem);
    else e = CRIT_B200_EUNSUPPORTED;
    if (e) return e;
    cudaError_t ce = cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (ce != cudaSuccess) return (int)ce;
    dim3 grid((unsigned)((p.tokens * G + PF_ROWS - 1) / PF_ROWS), (unsigned)p.kv_heads, nseq);
    fn<<<grid, PF_THREADS, smem, (cudaStream_t)stream>>>(p, smode);
    CRIT_CHECK_LAUNCH();
    return 0;
}
