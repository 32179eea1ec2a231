// Split-K decode / speculative-verify attention over paged KV: the device kernel.
//
// One block serves (window row, kv head, split of `chunk` positions, tile of 16*MT query rows); a query row is one
// (column, query head of the kv head's group) pair, so a GQA group's heads and a verify window's columns share every
// key and value byte the block reads.  The block's four warps each stream their own 16-position tiles of the split
// (tile i of the split belongs to warp i mod 4) through a private ring of stages in shared memory: a warp never waits
// for another inside the loop.
//
// Staging (template TMA):
//   true   one elected lane issues TMA tiled loads (cp.async.bulk.tensor, boxes of [16 positions][1 kv head][128 bytes]
//          with the 128-byte swizzle, from a 3-D tensor map over [slots][kv_heads][dim]) and bulk copies of the tile's
//          scales; their bytes are counted on the stage's mbarrier, which the warp's lanes then wait on (bounded);
//   false  every lane issues 16-byte cp.async copies (zero-filled past the row's last position) in commit groups.
// Scores and outputs are m16n8k16 tensor-core products with FP32 accumulators, with the POSITIONS on the instruction's
// 16-row axis and the query rows on its 8-column axis: S^T[16 positions x 8 query rows] = K Q^T and
// O^T[16 value columns x 8 query rows] += V^T P^T.  A decode step of a GQA group of up to 8 heads therefore fills the
// tile exactly (no padding rows), a verify window takes NT = 2 or 4 such column tiles, and the keys and values, which
// are the bytes streamed from HBM, are the A operands converted once per tile.  The probabilities cross from the
// accumulator layout to the B-operand layout with movmatrix (an 8x8 transpose inside the warp).  The online softmax
// lives in registers (shuffles over the lanes that share a query row).  8-bit pages (E4M3, INT8) are converted to
// FP16 in registers on the way from shared memory to the tensor cores: the head dimension is consumed in a permuted
// order (each thread reads 16 contiguous bytes of a key row) and the value columns are produced in a permuted order
// (each thread owns contiguous output columns), which needs no transposing load.  Where a tile is small (8-bit pages
// of heads up to 128 wide) an iteration takes two tiles (32 positions): two independent accumulator chains, and one
// softmax update for both.  The warps' states are folded through shared memory at the end; a row that fits one split
// is written out directly, else the split's state goes to the workspace for the merge.
//
// HBM traffic per block: its split's keys and values once (the algorithmic bytes), the queries, one partial state.
// Reference: paged_kv_attention/_kernels.py:263-478 (_partition, _window_kernel), cuda_window.cu:284-1065 (cw_tile).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace crit_b200 {

#ifndef CRIT_DECODE_STAGES_SMALL
#define CRIT_DECODE_STAGES_SMALL 4          // stages of a warp's ring where an iteration takes two tiles
#endif
#ifndef CRIT_DECODE_MIN_BLOCKS
#define CRIT_DECODE_MIN_BLOCKS 0            // blocks an SM the registers are budgeted for (0: what the shared memory allows)
#endif

constexpr int DECODE_WARPS = 4;
constexpr int DECODE_THREADS = DECODE_WARPS * 32;
constexpr float LAZY = 8.f;
constexpr int DECODE_MAX_LIST = 256;       // rows a persistent launch lists its work for

// Page element classes (PK): 0 bf16, 1 fp16, 2 E4M3 bytes, 3 INT8 bytes.
// NT: 8-row tiles of query rows a block holds (1, 2 or 4).
template <int D, int DV, int PK, int NT, bool TMA>
struct DecodeCfg {
    static constexpr int ES = PK < 2 ? 2 : 1;
    static constexpr bool BF16 = PK == 0;
    static constexpr int KROW = D * ES, VROW = DV * ES;
    static constexpr int KTILE = 16 * KROW, VTILE = 16 * VROW;
    static constexpr int TILES = KTILE + VTILE;
    static constexpr int TPI = TILES <= 4096 ? 2 : 1;          // tiles an iteration consumes
    static constexpr int STAGES = TPI == 2 ? CRIT_DECODE_STAGES_SMALL : 3;
    static constexpr int ROWS = 8 * NT;
    static constexpr int QROW = D * 2 + 16;                    // padded: rows 8 apart fall in different banks
    static constexpr int QBYTES = ROWS * QROW;
    static constexpr int FOLD = DECODE_WARPS * ROWS * (DV + 2) * 4;
    static constexpr bool QREG = NT * D <= 256;                // the query fragments stay in registers
    // dynamic shared memory: [1 KB of alignment slack][tiles | scales (or the fold)][queries][mbarriers]
    __host__ __device__ static constexpr int ring_bytes(int scb) { return DECODE_WARPS * STAGES * (TILES + scb); }
    __host__ __device__ static constexpr int region(int scb) { return ((ring_bytes(scb) > FOLD ? ring_bytes(scb) : FOLD) + 127) / 128 * 128; }
    __host__ __device__ static constexpr int smem_bytes(int scb) { return 1024 + region(scb) + QBYTES + DECODE_WARPS * STAGES * 8; }
    // blocks an SM holds by its 227 KB of shared memory (the scales' stage at its cp.async size).  A decode tile (8 query
    // rows) budgets its registers for as many, up to 3, so the compiler never trades a resident block for registers;
    // the wider tiles hold 2 or 4 times the accumulators and take what they need
    static constexpr int BY_SMEM = 232448 / (smem_bytes(128) + 1024);
    static constexpr int MIN_BLOCKS = CRIT_DECODE_MIN_BLOCKS ? CRIT_DECODE_MIN_BLOCKS
                                                             : (NT > 1 || BY_SMEM < 1 ? 1 : (BY_SMEM > 3 ? 3 : BY_SMEM));
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

// Byte offset of 16-byte chunk c of row `row` inside a 16-row tile.
//   TMA:      the tile is boxes of [16 rows][128 bytes] (2 KB each), chunk index xor'ed with row & 7 (128-byte swizzle);
//   cp.async: rows of ROWB bytes with a swizzle chosen for the reads each element size makes.
template <bool TMA, int ROWB, int ES, int DIM, bool IS_V>
__device__ __forceinline__ int tile_off(int row, int c) {
    if constexpr (TMA) {
        return ((c >> 3) << 11) + (row << 7) + (((c & 7) ^ (row & 7)) << 4);
    } else if constexpr (ES == 2) {
        return row * ROWB + (swz16(c, row) << 4);
    } else if constexpr (IS_V) {
        return row * ROWB + (vswz8<DIM>(row, c) << 4);
    } else {
        return row * ROWB + (kswz8<DIM>(row, c) << 4);
    }
}

template <int D, int DV, int PK, int NT, bool TMA>
__global__ void __launch_bounds__(DECODE_THREADS, DecodeCfg<D, DV, PK, NT, TMA>::MIN_BLOCKS)
decode_kernel(const crit_b200_attend_params p, const int ctiles, const int smode, const int scb, const int persistent,
              const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    using C = DecodeCfg<D, DV, PK, NT, TMA>;
    constexpr bool BF16 = C::BF16;
    constexpr int ES = C::ES;
    constexpr int ROWS = C::ROWS;
    constexpr int TPI = C::TPI;
    constexpr int KC = C::KROW / 16, VC = C::VROW / 16;      // 16-byte chunks of a key row, of a value row
    extern __shared__ unsigned char smem_raw[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = p.q_heads / p.kv_heads;

    // shared memory, its base rounded up to 1 KB (the 128-byte swizzle's period is 8 rows of 128 bytes)
    unsigned char* smem = smem_raw + ((1024 - (smem_addr(smem_raw) & 1023)) & 1023);
    const int region = C::region(scb);
    unsigned char* tiles = smem + warp * (C::STAGES * C::TILES);
    unsigned char* scales_ring = smem + DECODE_WARPS * C::STAGES * C::TILES + warp * (C::STAGES * scb);
    unsigned char* qs = smem + region;
    const uint32_t bars = smem_addr(qs + C::QBYTES) + warp * (C::STAGES * 8);

    if constexpr (TMA) {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < C::STAGES; ++s) mbar_init(bars + s * 8, 1);
            mbar_init_fence();
        }
    }

    // -- the work list -------------------------------------------------------------------------------------------------
    // persistent: the grid is a fixed number of blocks (a few per SM); every block lists the launch's work units
    // (row, kv head, query-row tile, split), counted from the rows' lengths read here on the device, and takes units
    // block, block + grid, ...  So a launch over rows of very different lengths starts no block that has nothing to
    // do, and the last wave is short.  Otherwise one unit per block, named by the block's place in a 3-D grid.
    __shared__ int unit_first[DECODE_MAX_LIST + 1];
    int units = 1;
    if (persistent) {
        if (warp == 0) {
            int carry = 0;
            for (int base = 0; base < p.n_rows; base += 32) {
                const int rr = base + lane;
                int mine_units = 0;
                if (rr < p.n_rows) {
                    int cnt = p.counts ? p.counts[rr] : p.columns;
                    cnt = cnt > p.columns ? p.columns : cnt;
                    if (cnt > 0) {
                        const int64_t len = p.firsts[rr] + ((p.flags & CRIT_B200_ATTEND_CONTEXT) ? 0 : cnt);
                        mine_units = (int)((len + p.chunk - 1) / p.chunk) * ((cnt * G + ROWS - 1) / ROWS) * p.kv_heads;
                    }
                }
                int scan = mine_units;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, scan, o);
                    if (lane >= o) scan += up;
                }
                if (rr < p.n_rows) unit_first[rr + 1] = carry + scan;
                carry += __shfl_sync(0xffffffffu, scan, 31);
            }
            if (lane == 0) unit_first[0] = 0;
        }
        __syncthreads();
        units = unit_first[p.n_rows];
    }
    int tbase = 0;              // tiles this warp has staged in earlier units (the stages' and mbarriers' running count)

    for (int unit = persistent ? (int)blockIdx.x : 0; unit < units; unit += persistent ? (int)gridDim.x : 1) {
    int split, h, ct, r;
    if (persistent) {
        int lo = 0, hi = p.n_rows;              // the row whose units hold this one
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (unit_first[mid] <= unit) lo = mid;
            else hi = mid;
        }
        r = lo;
    } else {
        r = blockIdx.z;
    }
    int count = p.counts ? p.counts[r] : p.columns;
    count = count > p.columns ? p.columns : count;
    if (count <= 0) continue;
    const int64_t first = p.firsts[r];
    const bool context = (p.flags & CRIT_B200_ATTEND_CONTEXT) != 0;       // the positions before `first` only
    const int64_t L = context ? first : first + count;
    const int nsplit = (int)((L + p.chunk - 1) / p.chunk);
    if (persistent) {
        const int local = unit - unit_first[r];
        const int row_tiles = (count * G + ROWS - 1) / ROWS;
        split = local % nsplit;
        ct = (local / nsplit) % row_tiles;
        h = local / (nsplit * row_tiles);
    } else {
        split = blockIdx.x;
        h = blockIdx.y / ctiles;
        ct = blockIdx.y - h * ctiles;
    }
    if (ct * ROWS >= count * G) continue;
    const int64_t begin = (int64_t)split * p.chunk;
    if (begin >= L) continue;
    const int64_t end = begin + p.chunk < L ? begin + p.chunk : L;
    const int32_t* table = p.tables + (int64_t)p.rows[r] * p.table_stride;
    const int start = p.starts[r];

    // -- the query tile into shared memory: ROWS rows of D 16-bit values (FP16 where the pages are 8-bit) -------------
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
            if (ES == 1 && p.q_dtype == CRIT_B200_DTYPE_BF16) {
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
    __syncthreads();

    // The last position each of this thread's query rows sees (-1: a padding row).  A thread's query rows are
    // nt * 8 + 2 * t + {0, 1}.
    int lastpos[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int flat = ct * ROWS + nt * 8 + 2 * t + e;
            const int col = flat / G;
            lastpos[nt][e] = col < count ? (int)(context ? first - 1 : first + col) : -1;
        }
    // A draft tree (p.parents): of the window's own positions a query row sees its column and the column's ancestors, bit
    // j of `seen` for column j (the chain of parents, at most `count` hops); the context before the window as ever.
    const bool tree = p.parents != nullptr;
    unsigned long long seen[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            seen[nt][e] = 0ull;
            if (tree && lastpos[nt][e] >= 0) {
                const int32_t* par = p.parents + p.starts[r];
                int at = (ct * ROWS + nt * 8 + 2 * t + e) / G;
                for (int hops = 0; at >= 0 && at < count && hops <= count; ++hops) {
                    seen[nt][e] |= 1ull << at;
                    at = par[at];
                }
            }
        }

    // The B operand of the scores: Q^T, k16 x n8 per step; b0 holds k = 2t, 2t+1 and b1 k = 2t+8, 2t+9 of query row g.
    auto q_frag = [&](int nt, int ks, uint32_t& b0, uint32_t& b1) {
        const unsigned char* row = qs + (nt * 8 + g) * C::QROW;
        if constexpr (ES == 1) {
            const uint2 v = *reinterpret_cast<const uint2*>(row + (t * (D / 4) + 4 * ks) * 2);
            b0 = v.x, b1 = v.y;
        } else {
            b0 = *reinterpret_cast<const uint32_t*>(row + (16 * ks + 2 * t) * 2);
            b1 = *reinterpret_cast<const uint32_t*>(row + (16 * ks + 8 + 2 * t) * 2);
        }
    };
    uint32_t qb[C::QREG ? NT : 1][C::QREG ? D / 16 : 1][2];
    if constexpr (C::QREG) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) q_frag(nt, ks, qb[nt][ks][0], qb[nt][ks][1]);
    }

    float acc[DV / 16][NT][4];
    float m_run[NT][2], l_run[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int mt = 0; mt < DV / 16; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
        m_run[nt][0] = m_run[nt][1] = -INFINITY;
        l_run[nt][0] = l_run[nt][1] = 0.f;
    }

    const float kmul = (PK == 2 && smode == 0) ? p.key_multiplier : 1.f;
    const float sl2 = p.scale * LOG2E * kmul;

    // -- this warp's tiles ---------------------------------------------------------------------------------------------
    const int tile0 = (int)(begin >> 4);
    const int ntiles = (int)((end - begin + 15) >> 4);
    const int mine = ntiles > warp ? (ntiles - warp + DECODE_WARPS - 1) / DECODE_WARPS : 0;
    const char* kbase = (const char*)p.key_pages + (int64_t)h * C::KROW;
    const char* vbase = (const char*)p.value_pages + (int64_t)h * C::VROW;
    const int64_t krow_stride = (int64_t)p.kv_heads * C::KROW, vrow_stride = (int64_t)p.kv_heads * C::VROW;
    const uint32_t scale_bytes = smode == 2 ? (uint32_t)p.kv_heads * 4u : (smode == 1 ? (uint32_t)p.kv_heads * 64u : 0u);
    const uint32_t tiles_per_page = (uint32_t)p.page >> 4;
    // a page id at or past this lies outside the page tensor (the tensor's size unknown: no page id does)
    const uint32_t pages_total = p.slots > 0 ? (uint32_t)(p.slots / p.page) : 0x7fffffffu;
    const int tshift = (tiles_per_page & (tiles_per_page - 1)) == 0 ? __ffs((int)tiles_per_page) - 1 : -1;
    const int Lr = (int)L;

    // The page ids of this warp's tiles, 32 tiles at a time: lane j holds the page of tile i0 + j of the warp's tiles (one
    // load a lane per 32 tiles, made 32 tiles ahead), and a tile's id reaches every lane by a shuffle.  So no tile waits
    // for a table read on its way to the copies.
    auto page_ids = [&](int i0) {
        const int k = i0 + lane;
        if (k >= mine) return 0;
        const uint32_t tile = (uint32_t)(tile0 + warp + k * DECODE_WARPS);
        return table[tshift >= 0 ? tile >> tshift : tile / tiles_per_page];
    };
    int pgs = 0, pgs_next = page_ids(0);
    bool outside = false;

    // cp.async staging of small tiles (four copies a lane for the keys, four for the values): each lane's source and
    // destination offsets inside a tile are fixed, so they are made once
    constexpr bool FIXED = !TMA && 16 * KC / 32 <= 4 && 16 * VC / 32 <= 4;
    constexpr int KU = FIXED ? 16 * KC / 32 : 1, VU = FIXED ? 16 * VC / 32 : 1;
    int ksrc[KU], kdst[KU], vsrc[VU], vdst[VU];
    if constexpr (FIXED) {
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int id = lane + 32 * u, row = id / KC, c = id - row * KC;
            ksrc[u] = row * (int)krow_stride + c * 16;
            kdst[u] = tile_off<false, C::KROW, ES, D, false>(row, c);
        }
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            const int id = lane + 32 * u, row = id / VC, c = id - row * VC;
            vsrc[u] = row * (int)vrow_stride + c * 16;
            vdst[u] = C::KTILE + tile_off<false, C::VROW, ES, DV, true>(row, c);
        }
    }

    auto issue = [&](int i) {
        if ((i & 31) == 0) {
            pgs = pgs_next;
            pgs_next = page_ids(i + 32);
        }
        if (i < mine) {
            const uint32_t tile = (uint32_t)(tile0 + warp + i * DECODE_WARPS);
            const uint32_t pidx = tshift >= 0 ? tile >> tshift : tile / tiles_per_page;
            const int off = (int)(tile - pidx * tiles_per_page) << 4;
            const uint32_t listed = (uint32_t)__shfl_sync(0xffffffffu, pgs, i & 31);
            outside |= listed >= pages_total;           // read the tensor's last page instead; reported at the unit's end
            const int pg = (int)(listed < pages_total ? listed : pages_total - 1);
            const int64_t slot0 = (int64_t)pg * p.page + off;
            const int stage = (tbase + i) % C::STAGES;
            const uint32_t ks = smem_addr(tiles + stage * C::TILES), vs = ks + C::KTILE;
            const uint32_t sc = smem_addr(scales_ring + stage * scb);
            if constexpr (TMA) {
                if (lane == 0) {
                    const uint32_t bar = bars + stage * 8;
                    fence_proxy_async();
                    mbar_expect_tx(bar, (uint32_t)C::TILES + (PK >= 2 ? 2u * scale_bytes : 0u));
#pragma unroll
                    for (int b = 0; b < C::KROW / 128; ++b) tma_load_3d(ks + b * 2048, &kmap, b * (128 / ES), h, (int)slot0, bar);
#pragma unroll
                    for (int b = 0; b < C::VROW / 128; ++b) tma_load_3d(vs + b * 2048, &vmap, b * (128 / ES), h, (int)slot0, bar);
                    if (PK >= 2 && smode) {
                        const int64_t at = smode == 2 ? (int64_t)pg * p.kv_heads : slot0 * p.kv_heads;
                        bulk_load(sc, p.key_scales + at, scale_bytes, bar);
                        bulk_load(sc + (scb >> 1), p.value_scales + at, scale_bytes, bar);
                    }
                }
            } else {
                const int live = Lr - (int)(tile << 4);          // rows past it are zero-filled
                if (FIXED && live >= 16) {
                    const char* ksrc0 = kbase + slot0 * krow_stride;
                    const char* vsrc0 = vbase + slot0 * vrow_stride;
#pragma unroll
                    for (int u = 0; u < KU; ++u) cp_async16(ks + kdst[u], ksrc0 + ksrc[u], true);
#pragma unroll
                    for (int u = 0; u < VU; ++u) cp_async16(ks + vdst[u], vsrc0 + vsrc[u], true);
                } else {
#pragma unroll
                    for (int u = 0; u < 16 * KC / 32; ++u) {
                        const int id = lane + 32 * u, row = id / KC, c = id - row * KC;
                        const bool ok = row < live;
                        cp_async16(ks + tile_off<false, C::KROW, ES, D, false>(row, c),
                                   kbase + (slot0 + (ok ? row : 0)) * krow_stride + c * 16, ok);
                    }
#pragma unroll
                    for (int u = 0; u < 16 * VC / 32; ++u) {
                        const int id = lane + 32 * u, row = id / VC, c = id - row * VC;
                        const bool ok = row < live;
                        cp_async16(vs + tile_off<false, C::VROW, ES, DV, true>(row, c),
                                   vbase + (slot0 + (ok ? row : 0)) * vrow_stride + c * 16, ok);
                    }
                }
                if (PK >= 2 && smode) {
                    const int row = lane & 15;
                    const bool ok = row < live;
                    const float* src = lane < 16 ? p.key_scales : p.value_scales;
                    const int64_t at = smode == 2 ? (int64_t)pg * p.kv_heads + h : (slot0 + (ok ? row : 0)) * p.kv_heads + h;
                    cp_async4(sc + lane * 4, src + at, ok);
                }
            }
        }
        if constexpr (!TMA) cp_async_commit();
    };

#pragma unroll
    for (int i = 0; i < C::STAGES - TPI; ++i) issue(i);

    bool dead = false;
    const int first32 = first > 0x7fffffffLL ? 0x7fffffff : (int)first;
    for (int i = 0; i < mine; i += TPI) {
#pragma unroll
        for (int u = 0; u < TPI; ++u) issue(i + C::STAGES - TPI + u);
        const int have = mine - i < TPI ? mine - i : TPI;          // tiles of this iteration (warp-uniform)
        if constexpr (TMA) {
            bool ok = true;
#pragma unroll
            for (int u = 0; u < TPI; ++u)
                if (u < have) ok &= mbar_wait(bars + ((tbase + i + u) % C::STAGES) * 8, (uint32_t)((tbase + i + u) / C::STAGES) & 1u);
            if (!__all_sync(0xffffffffu, ok)) {
                dead = true;                // a copy never landed: record it and leave, nothing is written
                break;
            }
        } else {
            cp_async_wait<C::STAGES - TPI>();
            __syncwarp();
        }

        float s[TPI][NT][4];
        float ksc[TPI][2], vsc[TPI][2];
        int pos0[TPI];
        bool masked = false;
#pragma unroll
        for (int u = 0; u < TPI; ++u) {
            pos0[u] = (tile0 + warp + (i + u) * DECODE_WARPS) << 4;
            ksc[u][0] = ksc[u][1] = vsc[u][0] = vsc[u][1] = 1.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[u][nt][e] = u < have ? 0.f : -INFINITY;
            if (u >= have) continue;
            masked |= pos0[u] + 16 > first32 || p.sliding > 0 || p.blocks != nullptr;
            const int stage = (tbase + i + u) % C::STAGES;
            unsigned char* kst = tiles + stage * C::TILES;
            const float* scales = reinterpret_cast<const float*>(scales_ring + stage * scb);
            if constexpr (TMA) {
                // A tiled load brings all 16 rows: the value rows past the row's last position become zeros, as the
                // zero-filling cp.async leaves them (a probability of 0 times a stale NaN would poison the output).
                const int live = Lr - pos0[u];
                if (live < 16) {
                    unsigned char* vst = kst + C::KTILE;
                    for (int id = lane; id < 16 * VC; id += 32) {
                        const int row = id / VC, c = id - row * VC;
                        if (row >= live)
                            *reinterpret_cast<uint4*>(vst + tile_off<true, C::VROW, ES, DV, true>(row, c)) = make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
            }
            // the tile's scales: ksc/vsc[u][hf] belong to position g + 8 * hf of the tile
            if (PK >= 2 && smode) {
                if constexpr (TMA) {
                    const float* vscales = scales + (scb >> 3);
                    if (smode == 2) {
                        ksc[u][0] = ksc[u][1] = scales[h];
                        vsc[u][0] = vsc[u][1] = vscales[h];
                    } else {
                        ksc[u][0] = scales[g * p.kv_heads + h], ksc[u][1] = scales[(g + 8) * p.kv_heads + h];
                        vsc[u][0] = vscales[g * p.kv_heads + h], vsc[u][1] = vscales[(g + 8) * p.kv_heads + h];
                    }
                } else {
                    ksc[u][0] = scales[g], ksc[u][1] = scales[g + 8];
                    vsc[u][0] = scales[16 + g], vsc[u][1] = scales[24 + g];
                }
            }

            // scores: S^T[16 positions x 8*NT query rows] = K Q^T
            uint32_t kw[2][ES == 1 ? D / 16 : 1];
            if constexpr (ES == 1) {
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    const int row = g + 8 * n;
#pragma unroll
                    for (int qd = 0; qd < D / 64; ++qd) {
                        const int c = t * (D / 64) + qd;
                        const uint4 v = *reinterpret_cast<const uint4*>(kst + tile_off<TMA, C::KROW, ES, D, false>(row, c));
                        kw[n][qd * 4 + 0] = v.x, kw[n][qd * 4 + 1] = v.y, kw[n][qd * 4 + 2] = v.z, kw[n][qd * 4 + 3] = v.w;
                    }
                }
            }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a[4];
                if constexpr (ES == 2) {
                    const int j = lane >> 3, row = (lane & 7) + 8 * (j & 1), chunk = 2 * ks + (j >> 1);
                    ldmatrix_x4(a, smem_addr(kst + tile_off<TMA, C::KROW, ES, D, false>(row, chunk)));
                } else {
                    code4_to_f16x2x2<PK == 3>(kw[0][ks], a[0], a[2]);
                    code4_to_f16x2x2<PK == 3>(kw[1][ks], a[1], a[3]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    uint32_t b0, b1;
                    if constexpr (C::QREG) b0 = qb[nt][ks][0], b1 = qb[nt][ks][1];
                    else q_frag(nt, ks, b0, b1);
                    mma16816<BF16>(s[u][nt], a, b0, b1);
                }
            }
        }

        // scale, mask, online softmax (base 2) over the iteration's positions
        uint32_t pb[TPI][NT][2];
        bool rescale = false;
        float alpha[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int u = 0; u < TPI; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float x = s[u][nt][e] * (sl2 * ksc[u][e >> 1]);
                    if (masked) {
                        const int pos = pos0[u] + g + 8 * (e >> 1);
                        if (p.sliding > 0 && pos <= lastpos[nt][e & 1] - p.sliding) x = -INFINITY;    // below the row's window
                        if (p.blocks && lastpos[nt][e & 1] >= 0) {      // block lists: only the positions of the token's blocks
                            const int32_t* listed = p.blocks + (int64_t)(p.starts[r] + (lastpos[nt][e & 1] - first32)) * p.blocks_k;
                            const int at = pos / p.block_size;
                            bool member = false;
                            for (int j = 0; j < p.blocks_k; ++j) member |= listed[j] == at;
                            if (!member) x = -INFINITY;
                        }
                        if (!tree) {
                            if (pos > lastpos[nt][e & 1]) x = -INFINITY;
                        } else if (lastpos[nt][e & 1] < 0 || (pos >= first32 && (pos - first32 >= count ||
                                                                                  !((seen[nt][e & 1] >> (pos - first32)) & 1ull)))) {
                            x = -INFINITY;
                        }
                    }
                    s[u][nt][e] = x;
                    mx[e & 1] = fmaxf(mx[e & 1], x);
                }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 4));
                mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 8));
                mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 16));
                // The running maximum moves only when the iteration's passes it by more than LAZY (2^8 in the
                // probabilities, well inside FP16 and FP32): most iterations then rescale nothing.
                const bool moved = mx[j] > m_run[nt][j] + LAZY || m_run[nt][j] == -INFINITY;
                const float top = moved ? mx[j] : m_run[nt][j];
                const float sub = top == -INFINITY ? 0.f : top;
                alpha[nt][j] = moved ? ex2(m_run[nt][j] - sub) : 1.f;
                rescale |= moved && top != m_run[nt][j];
                m_run[nt][j] = top;
                mx[j] = sub;
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int u = 0; u < TPI; ++u) {
                float pr[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = ex2(s[u][nt][e] - mx[e & 1]);
                    sum[e & 1] += pv;
                    float scaled = pv * vsc[u][e >> 1];
                    if (masked && s[u][nt][e] == -INFINITY) scaled = 0.f;     // a stale scale past the row's end
                    pr[e] = scaled;
                }
                // accumulator layout [position g (+8)][query rows 2t, 2t+1] -> B operand [positions 2t, 2t+1 (+8)][row g]
                pb[u][nt][0] = movmatrix_trans(pack2<BF16>(pr[0], pr[1]));
                pb[u][nt][1] = movmatrix_trans(pack2<BF16>(pr[2], pr[3]));
            }
            l_run[nt][0] = l_run[nt][0] * alpha[nt][0] + sum[0];
            l_run[nt][1] = l_run[nt][1] * alpha[nt][1] + sum[1];
        }
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int mt = 0; mt < DV / 16; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    acc[mt][nt][0] *= alpha[nt][0], acc[mt][nt][1] *= alpha[nt][1];
                    acc[mt][nt][2] *= alpha[nt][0], acc[mt][nt][3] *= alpha[nt][1];
                }
        }

        // outputs: O^T[DV value columns x 8*NT query rows] += V^T P^T
#pragma unroll
        for (int u = 0; u < TPI; ++u) {
            if (u >= have) continue;
            unsigned char* vst = tiles + ((tbase + i + u) % C::STAGES) * C::TILES + C::KTILE;
            if constexpr (ES == 2) {
#pragma unroll
                for (int mt = 0; mt < DV / 16; ++mt) {
                    uint32_t a[4];
                    const int j = lane >> 3, tok = (lane & 7) + 8 * (j >> 1), chunk = 2 * mt + (j & 1);
                    ldmatrix_x4_trans(a, smem_addr(vst + tile_off<TMA, C::VROW, ES, DV, true>(tok, chunk)));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma16816<BF16>(acc[mt][nt], a, pb[u][nt][0], pb[u][nt][1]);
                }
            } else {
                constexpr int VW = DV / 32;            // 32-bit words of a value row this thread owns
                uint32_t vw[4][VW];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int row = 2 * t + (q4 & 1) + 8 * (q4 >> 1);
                    if constexpr (DV == 64) {
                        const uint2 v = *reinterpret_cast<const uint2*>(vst + tile_off<false, C::VROW, ES, DV, true>(row, g >> 1) + (g & 1) * 8);
                        vw[q4][0] = v.x, vw[q4][1] = v.y;
                    } else {
#pragma unroll
                        for (int qd = 0; qd < DV / 128; ++qd) {
                            const int c = g * (DV / 128) + qd;
                            const uint4 v = *reinterpret_cast<const uint4*>(vst + tile_off<TMA, C::VROW, ES, DV, true>(row, c));
                            vw[q4][qd * 4 + 0] = v.x, vw[q4][qd * 4 + 1] = v.y, vw[q4][qd * 4 + 2] = v.z, vw[q4][qd * 4 + 3] = v.w;
                        }
                    }
                }
#pragma unroll
                for (int mt = 0; mt < DV / 16; ++mt) {
                    // bytes 2*mt and 2*mt+1 of this thread's value bytes are rows g and g+8 of the m-tile
                    const int w = mt >> 1;
                    const uint32_t sel = (mt & 1) ? 0x7362u : 0x5140u;
                    uint32_t a[4];
                    code4_to_f16x2x2<PK == 3>(__byte_perm(vw[0][w], vw[1][w], sel), a[0], a[1]);
                    code4_to_f16x2x2<PK == 3>(__byte_perm(vw[2][w], vw[3][w], sel), a[2], a[3]);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma16816<BF16>(acc[mt][nt], a, pb[u][nt][0], pb[u][nt][1]);
                }
            }
        }
        __syncwarp();
    }
    if (__any_sync(0xffffffffu, outside) && lane == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_BOUNDS);
    if constexpr (TMA) {
        if (__any_sync(0xffffffffu, dead)) {
            // Give every copy this warp still has in flight a last bounded chance to land before the block leaves.
            for (int s = 0; s < C::STAGES; ++s) mbar_wait(bars + s * 8, 0, 1000000ull);
            if (lane == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_TMA);
            dead = true;
        }
    } else {
        cp_async_wait<0>();
    }

    // -- fold the four warps' states ---------------------------------------------------------------------------------
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            l_run[nt][j] += __shfl_xor_sync(0xffffffffu, l_run[nt][j], 4);
            l_run[nt][j] += __shfl_xor_sync(0xffffffffu, l_run[nt][j], 8);
            l_run[nt][j] += __shfl_xor_sync(0xffffffffu, l_run[nt][j], 16);
        }
    const int any_dead = __syncthreads_or(dead ? 1 : 0);
    if (any_dead) return;
    float* fold = reinterpret_cast<float*>(smem);
    float* fm = fold;                                   // [warps][ROWS]
    float* fl = fold + DECODE_WARPS * ROWS;             // [warps][ROWS]
    float* fo = fold + 2 * DECODE_WARPS * ROWS;         // [warps][ROWS][DV]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int rr = nt * 8 + 2 * t + j;
            if (g == 0) {
                fm[warp * ROWS + rr] = m_run[nt][j];
                fl[warp * ROWS + rr] = l_run[nt][j];
            }
            float* dst = fo + (warp * ROWS + rr) * DV;
#pragma unroll
            for (int mt = 0; mt < DV / 16; ++mt)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const int col = ES == 2 ? mt * 16 + g + 8 * hf : g * (DV / 8) + 2 * mt + hf;
                    dst[col] = acc[mt][nt][2 * hf + j];
                }
        }
    __syncthreads();

    const float vmul = (PK == 2 && smode == 0) ? p.value_multiplier : 1.f;
    const bool whole = nsplit == 1 && !(p.flags & CRIT_B200_ATTEND_PARTIALS) && !p.sinks;     // (sinks join in the fold)
    const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
    const int prow0 = p.offsets ? p.offsets[r] - p.offsets[0] : r * p.columns;
    // a plan too small for this unit (more splits or partial rows than the workspace was sized for): the unit's state
    // is dropped and the status word says so, rather than written past the partials
    const bool fits = whole || (p.workspace && split < p.max_splits && prow0 >= 0 && prow0 + count <= p.partial_rows);
    if (!fits && tid == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_PLAN);
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
        } else if (fits) {
            const int prow = prow0 + col;
            const int64_t at = ((int64_t)prow * p.q_heads + head) * p.max_splits + split;
            *reinterpret_cast<float4*>(p.workspace + at * DV + c4 * 4) = o;
            if (c4 == 0) {
                p.workspace[states * DV + at] = top;
                p.workspace[states * (DV + 1) + at] = l;
            }
        }
    }
    tbase += mine;
    __syncthreads();            // the fold and the queries are read to the end before the next unit stages over them
    }
}

}  // namespace crit_b200
