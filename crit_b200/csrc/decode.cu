// Split-K decode / speculative-verify attention over paged KV, and the fold of a row's splits.
//
// One block serves (window row, kv head, split of `chunk` positions, tile of 16*MT query rows); a query row is one
// (column, query head of the kv head's group) pair, so a GQA group's heads and a verify window's columns share every
// key and value byte the block reads.  The block's four warps each stream their own 16-position tiles of the split
// (tile i of the split belongs to warp i mod 4) through a private ring of cp.async stages in shared memory: a warp
// never waits for another inside the loop.  Scores and outputs are m16n8k16 tensor-core products with FP32
// accumulators; the online softmax lives in registers (quad shuffles for the row maxima).  8-bit pages (E4M3, INT8)
// are converted to FP16 in registers on the way from shared memory to the tensor cores: the head dimension is
// consumed in a permuted order (each thread reads 16 contiguous bytes of a key row) and the value columns are
// produced in a permuted order (each thread owns 16 contiguous output columns), which needs no transposing load.
// The warps' states are folded through shared memory at the end; a row that fits one split is written out directly,
// else the split's state goes to the workspace for merge_kernel.
//
// HBM traffic per block: its split's keys and values once (the algorithmic bytes), the queries, and one partial state.
// Reference: paged_kv_attention/_kernels.py:263-478 (_partition, _window_kernel), :558-604 (_merge_kernel),
// cuda_window.cu:284-1286 (the CUDA flash tile and its merges).
#include "common.cuh"

namespace crit_b200 {

constexpr int DECODE_WARPS = 4;
constexpr int DECODE_THREADS = DECODE_WARPS * 32;
constexpr int MERGE_WARPS = 8;

// Page element classes: 0 bf16, 1 fp16, 2 E4M3 bytes, 3 INT8 bytes.
template <int D, int DV, int PK, int MT>
struct DecodeCfg {
    static constexpr int ES = PK < 2 ? 2 : 1;
    static constexpr bool BF16 = PK == 0;
    static constexpr int KROW = D * ES, VROW = DV * ES;
    static constexpr int KTILE = 16 * KROW, VTILE = 16 * VROW;
    static constexpr int STAGE = KTILE + VTILE + 128;
    static constexpr int STAGES = STAGE <= 4608 ? 4 : 3;
    static constexpr int QROW = D * 2 + (ES == 1 ? 16 : 0);
    static constexpr int QBYTES = 16 * MT * QROW;
    static constexpr int RING = DECODE_WARPS * STAGES * STAGE;
    static constexpr int FOLD = DECODE_WARPS * 16 * MT * (DV + 2) * 4;
    static constexpr int SMEM = QBYTES + (RING > FOLD ? RING : FOLD);
    static constexpr bool QREG = MT == 1 && D <= 128;
};

__device__ __forceinline__ int swz16(int c, int row) { return (c & ~7) | ((c ^ row) & 7); }

template <int D>
__device__ __forceinline__ int kswz8(int row, int c) {
    if constexpr (D == 128) return c ^ (row & 1);
    else if constexpr (D == 256) return c ^ (((row & 1) << 1) | ((c >> 3) & 1));
    else return c;
}
template <int DV>
__device__ __forceinline__ int vswz8(int row, int c) {
    if constexpr (DV == 128) return c ^ (((row >> 1) & 3) << 1);
    else if constexpr (DV == 256) return c ^ ((row >> 1) & 1) ^ (((row >> 2) & 1) << 2);
    else return c ^ ((row >> 1) & 3);
}

template <int D, int DV, int PK, int MT>
__global__ void __launch_bounds__(DECODE_THREADS) decode_kernel(const crit_b200_attend_params p, const int ctiles,
                                                               const int smode) {
    using C = DecodeCfg<D, DV, PK, MT>;
    constexpr bool BF16 = C::BF16;
    constexpr int ES = C::ES;
    constexpr int ROWS = 16 * MT;
    extern __shared__ __align__(128) unsigned char smem[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x;
    const int h = blockIdx.y / ctiles, ct = blockIdx.y - h * ctiles;
    const int r = blockIdx.z;
    const int G = p.q_heads / p.kv_heads;

    int count = p.counts ? p.counts[r] : p.columns;
    count = count > p.columns ? p.columns : count;
    if (count <= 0) return;
    if (ct * ROWS >= count * G) return;
    const int64_t first = p.firsts[r];
    const int64_t L = first + count;
    const int64_t begin = (int64_t)split * p.chunk;
    if (begin >= L) return;
    const int64_t end = begin + p.chunk < L ? begin + p.chunk : L;
    const int nsplit = (int)((L + p.chunk - 1) / p.chunk);
    const int32_t* table = p.tables + (int64_t)p.rows[r] * p.table_stride;
    const int start = p.starts[r];

    unsigned char* qs = smem;
    unsigned char* ring = smem + C::QBYTES + warp * (C::STAGES * C::STAGE);

    // -- the query tile into shared memory ---------------------------------------------------------------------------
    {
        constexpr int CPR = D / 8;
        for (int idx = tid; idx < ROWS * CPR; idx += DECODE_THREADS) {
            const int rr = idx / CPR, c = idx - rr * CPR;
            const int flat = ct * ROWS + rr;
            const int col = flat / G, gq = flat - col * G;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (col < count) {
                const char* src = (const char*)p.q +
                                  ((int64_t)(start + col) * p.q_stride_token + (int64_t)(h * G + gq) * p.q_stride_head + c * 8) * 2;
                v = *reinterpret_cast<const uint4*>(src);
            }
            if constexpr (ES == 2) {
                *reinterpret_cast<uint4*>(qs + rr * C::QROW + swz16(c, rr) * 16) = v;
            } else {
                if (p.q_dtype == CRIT_B200_DTYPE_BF16) {
                    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&w[i]);
                        float2 f = __bfloat1622float2(b);
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

    // The last position each of this thread's query rows sees (-1: a padding row).
    int64_t lastpos[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int flat = ct * ROWS + mt * 16 + g + 8 * hf;
            const int col = flat / G;
            lastpos[mt][hf] = col < count ? first + col : -1;
        }

    uint32_t qa[C::QREG ? D / 16 : 1][4];
    if constexpr (C::QREG) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            if constexpr (ES == 2) {
                const int j = lane >> 3, row = (lane & 7) + 8 * (j & 1), chunk = 2 * ks + (j >> 1);
                ldmatrix_x4(qa[ks], smem_addr(qs + row * C::QROW + swz16(chunk, row) * 16));
            } else {
                const uint2 lo = *reinterpret_cast<const uint2*>(qs + g * C::QROW + (t * (D / 4) + 4 * ks) * 2);
                const uint2 hi = *reinterpret_cast<const uint2*>(qs + (g + 8) * C::QROW + (t * (D / 4) + 4 * ks) * 2);
                qa[ks][0] = lo.x, qa[ks][1] = hi.x, qa[ks][2] = lo.y, qa[ks][3] = hi.y;
            }
        }
    }

    float acc[MT][DV / 8][4];
    float m_run[MT][2], l_run[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int n = 0; n < DV / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][n][i] = 0.f;
        m_run[mt][0] = m_run[mt][1] = -INFINITY;
        l_run[mt][0] = l_run[mt][1] = 0.f;
    }

    const float kmul = (PK == 2 && smode == 0) ? p.key_multiplier : 1.f;
    const float sl2 = p.scale * LOG2E * kmul;

    // -- this warp's tiles ---------------------------------------------------------------------------------------------
    const int tile0 = (int)(begin >> 4);
    const int tiles = (int)((end - begin + 15) >> 4);
    const int mine = tiles > warp ? (tiles - warp + DECODE_WARPS - 1) / DECODE_WARPS : 0;
    const char* kbase = (const char*)p.key_pages + (int64_t)h * C::KROW;
    const char* vbase = (const char*)p.value_pages + (int64_t)h * C::VROW;
    const int64_t krow_stride = (int64_t)p.kv_heads * C::KROW, vrow_stride = (int64_t)p.kv_heads * C::VROW;

    auto issue = [&](int i) {
        if (i < mine) {
            const int64_t pos0 = (int64_t)(tile0 + warp + i * DECODE_WARPS) << 4;
            const int pidx = (int)(pos0 / p.page);
            const int off = (int)(pos0 - (int64_t)pidx * p.page);
            const int pg = table[pidx];
            const int64_t slot0 = (int64_t)pg * p.page + off;
            const int live = (int)(L - pos0 < 16 ? L - pos0 : 16);
            unsigned char* st = ring + (i % C::STAGES) * C::STAGE;
            const uint32_t ks = smem_addr(st), vs = ks + C::KTILE;
            constexpr int KC = C::KROW / 16, VC = C::VROW / 16;
#pragma unroll
            for (int u = 0; u < 16 * KC / 32; ++u) {
                const int id = lane + 32 * u, row = id / KC, c = id - row * KC;
                const int pc = ES == 2 ? swz16(c, row) : kswz8<D>(row, c);
                const bool ok = row < live;
                cp_async16(ks + row * C::KROW + pc * 16, kbase + (slot0 + (ok ? row : 0)) * krow_stride + c * 16, ok);
            }
#pragma unroll
            for (int u = 0; u < 16 * VC / 32; ++u) {
                const int id = lane + 32 * u, row = id / VC, c = id - row * VC;
                const int pc = ES == 2 ? swz16(c, row) : vswz8<DV>(row, c);
                const bool ok = row < live;
                cp_async16(vs + row * C::VROW + pc * 16, vbase + (slot0 + (ok ? row : 0)) * vrow_stride + c * 16, ok);
            }
            if (PK >= 2 && smode) {
                const int row = lane & 15;
                const bool ok = row < live;
                const float* sc = lane < 16 ? p.key_scales : p.value_scales;
                const int64_t at = smode == 2 ? (int64_t)pg * p.kv_heads + h : (slot0 + (ok ? row : 0)) * p.kv_heads + h;
                cp_async4(vs + C::VTILE + lane * 4, sc + at, ok);
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int i = 0; i < C::STAGES - 1; ++i) issue(i);

    for (int i = 0; i < mine; ++i) {
        issue(i + C::STAGES - 1);
        cp_async_wait<C::STAGES - 1>();
        __syncwarp();
        const int64_t pos0 = (int64_t)(tile0 + warp + i * DECODE_WARPS) << 4;
        const unsigned char* kst = ring + (i % C::STAGES) * C::STAGE;
        const unsigned char* vst = kst + C::KTILE;
        const float* scales = reinterpret_cast<const float*>(vst + C::VTILE);

        // scores: S[16*MT x 16] = Q K^T
        float s[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[mt][n][e] = 0.f;

        uint32_t kw[2][ES == 1 ? D / 16 : 1];
        if constexpr (ES == 1) {
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int row = g + 8 * n;
#pragma unroll
                for (int qd = 0; qd < D / 64; ++qd) {
                    const int c = t * (D / 64) + qd;
                    const uint4 v = *reinterpret_cast<const uint4*>(kst + row * C::KROW + kswz8<D>(row, c) * 16);
                    kw[n][qd * 4 + 0] = v.x, kw[n][qd * 4 + 1] = v.y, kw[n][qd * 4 + 2] = v.z, kw[n][qd * 4 + 3] = v.w;
                }
            }
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t kb[4];
            if constexpr (ES == 2) {
                const int j = lane >> 3, tok = (lane & 7) + 8 * (j >> 1), chunk = 2 * ks + (j & 1);
                ldmatrix_x4(kb, smem_addr(kst + tok * C::KROW + swz16(chunk, tok) * 16));
            } else {
                kb[0] = code2_to_f16x2<PK == 3>(kw[0][ks]);
                kb[1] = code2_to_f16x2<PK == 3>(kw[0][ks] >> 16);
                kb[2] = code2_to_f16x2<PK == 3>(kw[1][ks]);
                kb[3] = code2_to_f16x2<PK == 3>(kw[1][ks] >> 16);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t a[4];
                if constexpr (C::QREG) {
                    a[0] = qa[ks][0], a[1] = qa[ks][1], a[2] = qa[ks][2], a[3] = qa[ks][3];
                } else if constexpr (ES == 2) {
                    const int j = lane >> 3, row = mt * 16 + (lane & 7) + 8 * (j & 1), chunk = 2 * ks + (j >> 1);
                    ldmatrix_x4(a, smem_addr(qs + row * C::QROW + swz16(chunk, row) * 16));
                } else {
                    const int row = mt * 16 + g;
                    const uint2 lo = *reinterpret_cast<const uint2*>(qs + row * C::QROW + (t * (D / 4) + 4 * ks) * 2);
                    const uint2 hi = *reinterpret_cast<const uint2*>(qs + (row + 8) * C::QROW + (t * (D / 4) + 4 * ks) * 2);
                    a[0] = lo.x, a[1] = hi.x, a[2] = lo.y, a[3] = hi.y;
                }
                mma16816<BF16>(s[mt][0], a, kb[0], kb[1]);
                mma16816<BF16>(s[mt][1], a, kb[2], kb[3]);
            }
        }

        // scale, mask, online softmax (base 2)
        float ksc[4] = {1.f, 1.f, 1.f, 1.f}, vsc[4] = {1.f, 1.f, 1.f, 1.f};
        if (PK >= 2 && smode) {
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const float2 a = *reinterpret_cast<const float2*>(scales + n * 8 + 2 * t);
                const float2 b = *reinterpret_cast<const float2*>(scales + 16 + n * 8 + 2 * t);
                ksc[2 * n] = a.x, ksc[2 * n + 1] = a.y, vsc[2 * n] = b.x, vsc[2 * n + 1] = b.y;
            }
        }
        const bool masked = pos0 + 16 > first;
        uint32_t pa[MT][4];
        bool rescale = false;
        float alpha[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float x = s[mt][n][e] * (sl2 * ksc[2 * n + (e & 1)]);
                    if (masked) {
                        const int64_t pos = pos0 + n * 8 + 2 * t + (e & 1);
                        if (pos > lastpos[mt][e >> 1]) x = -INFINITY;
                    }
                    s[mt][n][e] = x;
                    mx[e >> 1] = fmaxf(mx[e >> 1], x);
                }
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
                mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
                const float top = fmaxf(m_run[mt][hf], mx[hf]);
                const float sub = top == -INFINITY ? 0.f : top;
                alpha[mt][hf] = ex2(m_run[mt][hf] - sub);
                rescale |= top != m_run[mt][hf];
                m_run[mt][hf] = top;
                mx[hf] = sub;
            }
            float sum[2] = {0.f, 0.f};
            float pr[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = ex2(s[mt][n][e] - mx[e >> 1]);
                    sum[e >> 1] += pv;
                    pr[n][e] = pv * vsc[2 * n + (e & 1)];
                }
            l_run[mt][0] = l_run[mt][0] * alpha[mt][0] + sum[0];
            l_run[mt][1] = l_run[mt][1] * alpha[mt][1] + sum[1];
            pa[mt][0] = pack2<BF16>(pr[0][0], pr[0][1]);
            pa[mt][1] = pack2<BF16>(pr[0][2], pr[0][3]);
            pa[mt][2] = pack2<BF16>(pr[1][0], pr[1][1]);
            pa[mt][3] = pack2<BF16>(pr[1][2], pr[1][3]);
        }
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < DV / 8; ++n) {
                    acc[mt][n][0] *= alpha[mt][0], acc[mt][n][1] *= alpha[mt][0];
                    acc[mt][n][2] *= alpha[mt][1], acc[mt][n][3] *= alpha[mt][1];
                }
        }

        // outputs: O[16*MT x DV] += P V
        if constexpr (ES == 2) {
#pragma unroll
            for (int np = 0; np < DV / 16; ++np) {
                uint32_t vb[4];
                const int j = lane >> 3, tok = (lane & 7) + 8 * (j & 1), chunk = 2 * np + (j >> 1);
                ldmatrix_x4_trans(vb, smem_addr(vst + tok * C::VROW + swz16(chunk, tok) * 16));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma16816<BF16>(acc[mt][2 * np], pa[mt], vb[0], vb[1]);
                    mma16816<BF16>(acc[mt][2 * np + 1], pa[mt], vb[2], vb[3]);
                }
            }
        } else {
            constexpr int VW = DV / 32;            // 32-bit words of a value row this thread owns
            uint32_t vw[4][VW];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int row = 2 * t + (q4 & 1) + 8 * (q4 >> 1);
                if constexpr (DV == 64) {
                    const uint2 v = *reinterpret_cast<const uint2*>(vst + row * C::VROW + vswz8<DV>(row, g >> 1) * 16 + (g & 1) * 8);
                    vw[q4][0] = v.x, vw[q4][1] = v.y;
                } else {
#pragma unroll
                    for (int qd = 0; qd < DV / 128; ++qd) {
                        const int c = g * (DV / 128) + qd;
                        const uint4 v = *reinterpret_cast<const uint4*>(vst + row * C::VROW + vswz8<DV>(row, c) * 16);
                        vw[q4][qd * 4 + 0] = v.x, vw[q4][qd * 4 + 1] = v.y, vw[q4][qd * 4 + 2] = v.z, vw[q4][qd * 4 + 3] = v.w;
                    }
                }
            }
#pragma unroll
            for (int np = 0; np < DV / 16; ++np) {
                const int w = np >> 1;
                const uint32_t sel = (np & 1) ? 0x7362u : 0x5140u;
                const uint32_t x01 = __byte_perm(vw[0][w], vw[1][w], sel);
                const uint32_t x23 = __byte_perm(vw[2][w], vw[3][w], sel);
                const uint32_t b00 = code2_to_f16x2<PK == 3>(x01), b01 = code2_to_f16x2<PK == 3>(x23);
                const uint32_t b10 = code2_to_f16x2<PK == 3>(x01 >> 16), b11 = code2_to_f16x2<PK == 3>(x23 >> 16);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma16816<BF16>(acc[mt][2 * np], pa[mt], b00, b01);
                    mma16816<BF16>(acc[mt][2 * np + 1], pa[mt], b10, b11);
                }
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();

    // -- fold the four warps' states ---------------------------------------------------------------------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            l_run[mt][hf] += __shfl_xor_sync(0xffffffffu, l_run[mt][hf], 1);
            l_run[mt][hf] += __shfl_xor_sync(0xffffffffu, l_run[mt][hf], 2);
        }
    __syncthreads();
    float* fold = reinterpret_cast<float*>(smem + C::QBYTES);
    float* fm = fold;                                   // [warps][ROWS]
    float* fl = fold + DECODE_WARPS * ROWS;             // [warps][ROWS]
    float* fo = fold + 2 * DECODE_WARPS * ROWS;         // [warps][ROWS][DV]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int rr = mt * 16 + g + 8 * hf;
            if (t == 0) {
                fm[warp * ROWS + rr] = m_run[mt][hf];
                fl[warp * ROWS + rr] = l_run[mt][hf];
            }
            float* dst = fo + (warp * ROWS + rr) * DV;
#pragma unroll
            for (int n = 0; n < DV / 8; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = ES == 2 ? n * 8 + 2 * t + e : (2 * t + e) * (DV / 8) + n;
                    dst[col] = acc[mt][n][2 * hf + e];
                }
        }
    __syncthreads();

    const float vmul = (PK == 2 && smode == 0) ? p.value_multiplier : 1.f;
    const bool whole = nsplit == 1;
    const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
    for (int idx = tid; idx < ROWS * (DV / 4); idx += DECODE_THREADS) {
        const int rr = idx / (DV / 4), c4 = idx - rr * (DV / 4);
        const int flat = ct * ROWS + rr;
        const int col = flat / G, gq = flat - col * G;
        if (col >= count) continue;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < DECODE_WARPS; ++w) top = fmaxf(top, fm[w * ROWS + rr]);
        const float sub = top == -INFINITY ? 0.f : top;
        float l = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < DECODE_WARPS; ++w) {
            const float f = ex2(fm[w * ROWS + rr] - sub);
            l += fl[w * ROWS + rr] * f;
            const float4 v = *reinterpret_cast<const float4*>(fo + (w * ROWS + rr) * DV + c4 * 4);
            o.x += v.x * f, o.y += v.y * f, o.z += v.z * f, o.w += v.w * f;
        }
        o.x *= vmul, o.y *= vmul, o.z *= vmul, o.w *= vmul;
        const int token = start + col, head = h * G + gq;
        if (whole) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            char* dst = (char*)p.out + ((int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head + c4 * 4) * 2;
            uint2 packed;
            if (p.q_dtype == CRIT_B200_DTYPE_BF16) {
                packed.x = pack2<true>(o.x * inv, o.y * inv), packed.y = pack2<true>(o.z * inv, o.w * inv);
            } else {
                packed.x = pack2<false>(o.x * inv, o.y * inv), packed.y = pack2<false>(o.z * inv, o.w * inv);
            }
            *reinterpret_cast<uint2*>(dst) = packed;
            if (p.lse && c4 == 0) p.lse[(int64_t)token * p.q_heads + head] = l > 0.f ? top * LN2 + logf(l) : -INFINITY;
        } else {
            const int prow = (p.offsets ? p.offsets[r] - p.offsets[0] : r * p.columns) + col;
            const int64_t at = ((int64_t)prow * p.q_heads + head) * p.max_splits + split;
            *reinterpret_cast<float4*>(p.workspace + at * DV + c4 * 4) = o;
            if (c4 == 0) {
                p.workspace[states * DV + at] = top;
                p.workspace[states * (DV + 1) + at] = l;
            }
        }
    }
}

// The fold of a row's splits in split order (warp w takes splits w, w + 8, ...; the eight warps' states are folded in
// warp order).  Block = (window token, query head).  m is in base-2 units, o and l are relative to it.
__global__ void __launch_bounds__(MERGE_WARPS * 32) merge_kernel(const crit_b200_attend_params p) {
    __shared__ float sm[MERGE_WARPS], sl[MERGE_WARPS];
    __shared__ float so[MERGE_WARPS][256];
    const int head = blockIdx.x;
    const int r = blockIdx.y / p.columns, col = blockIdx.y - r * p.columns;
    int count = p.counts ? p.counts[r] : p.columns;
    count = count > p.columns ? p.columns : count;
    if (col >= count) return;
    const int64_t L = p.firsts[r] + count;
    const int nsplit = (int)((L + p.chunk - 1) / p.chunk);
    if (nsplit <= 1) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int DV = p.value_dim, per = DV >> 5;
    const int prow = (p.offsets ? p.offsets[r] - p.offsets[0] : r * p.columns) + col;
    const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
    const int64_t base = ((int64_t)prow * p.q_heads + head) * p.max_splits;
    const float* pm = p.workspace + states * DV;
    const float* pl = p.workspace + states * (DV + 1);
    float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int s = warp; s < nsplit; s += MERGE_WARPS) {
        const float ms = pm[base + s], ls = pl[base + s];
        const float* o = p.workspace + (base + s) * DV + lane * per;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = i < per ? o[i] : 0.f;
        const float top = fmaxf(m, ms);
        const float sub = top == -INFINITY ? 0.f : top;
        const float keep = ex2(m - sub), take = ex2(ms - sub);
        l = l * keep + ls * take;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = acc[i] * keep + v[i] * take;
        m = top;
    }
    if (lane == 0) sm[warp] = m, sl[warp] = l;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < per) so[warp][lane * per + i] = acc[i];
    __syncthreads();
    const int token = p.starts[r] + col;
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
    int count = p.counts ? p.counts[r] : p.columns;
    count = count > p.columns ? p.columns : count;
    if (col >= count) return;
    const int64_t L = p.firsts[r] + count;
    const int nsplit = (int)((L + p.chunk - 1) / p.chunk);
    if (nsplit <= 1) return;
    const int prow = (p.offsets ? p.offsets[r] - p.offsets[0] : r * p.columns) + col;
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
    const float inv = total > 0.f ? 1.f / total : 0.f;
    const int token = p.starts[r] + col;
    const int64_t at = (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; i += 2) {
        const uint32_t packed = p.q_dtype == CRIT_B200_DTYPE_BF16 ? pack2<true>(acc[i] * inv, acc[i + 1] * inv)
                                                                   : pack2<false>(acc[i] * inv, acc[i + 1] * inv);
        *reinterpret_cast<uint32_t*>((char*)p.out + (at + i) * 2) = packed;
    }
    if (p.lse && lane == 0) p.lse[(int64_t)token * p.q_heads + head] = total > 0.f ? top * LN2 + logf(total) : -INFINITY;
}

// -- host side --------------------------------------------------------------------------------------------------------
typedef void (*decode_fn)(const crit_b200_attend_params, const int, const int);

struct Variant {
    decode_fn fn;
    int smem;
};

template <int D, int DV, int PK, int MT>
static Variant variant() {
    return Variant{decode_kernel<D, DV, PK, MT>, DecodeCfg<D, DV, PK, MT>::SMEM};
}

template <int PK, int MT>
static int pick_width(int d, int dv, Variant* out) {
    if (d == 64 && dv == 64) *out = variant<64, 64, PK, MT>();
    else if (d == 128 && dv == 128) *out = variant<128, 128, PK, MT>();
    else if (d == 256 && dv == 256) {
        if constexpr (MT == 1) *out = variant<256, 256, PK, 1>();
        else return CRIT_B200_EUNSUPPORTED;
    } else return CRIT_B200_EUNSUPPORTED;
    return 0;
}

static int page_class(int kind, int page_dtype) {
    if (kind == CRIT_B200_KIND_16BIT) return page_dtype == CRIT_B200_DTYPE_BF16 ? 0 : (page_dtype == CRIT_B200_DTYPE_FP16 ? 1 : -1);
    if (kind == CRIT_B200_KIND_INT8) return 3;
    if (kind == CRIT_B200_KIND_FP8 || kind == CRIT_B200_KIND_FP8_ROW || kind == CRIT_B200_KIND_FP8_PAGE) return 2;
    return -1;
}

// Query rows a block's tile holds: 16, or 32 where a row's columns times the group's heads pass 16 and the value
// accumulators of two row tiles still fit the registers.
static int row_tiles(int rows, int dv) { return rows > 16 && dv <= 128 ? 2 : 1; }

static int pick(int kind, int page_dtype, int d, int dv, int mt, Variant* out) {
    const int pk = page_class(kind, page_dtype);
    if (pk < 0) return CRIT_B200_EUNSUPPORTED;
#define CRIT_PICK(PK)                                             \
    return mt == 2 ? pick_width<PK, 2>(d, dv, out) : pick_width<PK, 1>(d, dv, out)
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
    if (p.max_splits > 1) {
        const int64_t need = (int64_t)p.partial_rows * p.q_heads * p.max_splits * (p.value_dim + 2);
        if (!p.workspace || p.workspace_floats < need || p.partial_rows < 1) return CRIT_B200_EWORKSPACE;
        if (!aligned(p.workspace, 16)) return CRIT_B200_EALIGN;
    }
    return 0;
}

static int launch_decode(const crit_b200_attend_params& p, cudaStream_t s) {
    const int G = p.q_heads / p.kv_heads;
    const int rows = p.columns * G;
    const int mt = row_tiles(rows, p.value_dim);
    Variant v;
    int e = pick(p.kind, p.page_dtype, p.head_dim, p.value_dim, mt, &v);
    if (e) return e;
    // Set at every launch: the attribute belongs to the function on the current device, and a process may drive several.
    cudaError_t ce = cudaFuncSetAttribute((const void*)v.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, v.smem);
    if (ce != cudaSuccess) return (int)ce;
    const int ctiles = (rows + 16 * mt - 1) / (16 * mt);
    dim3 grid((unsigned)p.max_splits, (unsigned)(p.kv_heads * ctiles), (unsigned)p.n_rows);
    v.fn<<<grid, DECODE_THREADS, v.smem, s>>>(p, ctiles, scale_mode(p.kind));
    CRIT_CHECK_LAUNCH();
    return 0;
}

static int launch_merge(const crit_b200_attend_params& p, cudaStream_t s) {
    if (p.max_splits <= 1) return 0;
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

}  // namespace crit_b200

using namespace crit_b200;

extern "C" __attribute__((visibility("default"))) int crit_b200_attend_plan(int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t value_dim,
                                     int32_t page, int32_t kind, int32_t page_dtype, int32_t columns, int32_t* out5) {
    if (!out5 || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads || columns < 1) return CRIT_B200_EINVAL;
    if (page < 16 || page % 16) return CRIT_B200_EUNSUPPORTED;
    const int rows = columns * (q_heads / kv_heads);
    const int mt = row_tiles(rows, value_dim);
    Variant v;
    int e = pick(kind, page_dtype, head_dim, value_dim, mt, &v);
    if (e) return e;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) == cudaSuccess) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (cudaFuncSetAttribute((const void*)v.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, v.smem) == cudaSuccess)
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)v.fn, DECODE_THREADS, v.smem);
    }
    cudaGetLastError();
    out5[0] = 1024;
    out5[1] = v.smem;
    out5[2] = 16 * mt;
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
