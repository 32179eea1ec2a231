// Split-K decode attention over E4M3 pages on the fifth-generation tensor cores, one unit for ALL kv heads of a window
// row: the bytes a block asks HBM for are whole page rows, 16 slots x 8 kv heads x 128 bytes = 16 KB in one piece.
//
// decode_tc.cuh gives a unit one kv head, so its TMA boxes are 16 rows of 128 bytes that lie 1 KB apart, and eight blocks
// on eight SMs fetch the eight interleaved parts of a page at different times; streamed that way, even with nothing
// computed, the pages arrive clearly below the copy bandwidth, as whole 16 KB pieces close to it.  Here a tile is 16
// positions of all 8 kv heads, loaded by ONE box of a tensor map whose dimensions are permuted, [128 bytes][slots][kv
// heads]: the box lands head-major, row 16 * head + slot of the operand, although its source is one contiguous piece.
//
//     S [128 lanes x 128 columns]  = Q [128 x 128 bytes] . Ktile^T      lane 16 * head + j (hi) / + 8 + j (lo): query row j
//                                                                      of the head's group; column 16 * head' + slot
//     O [128 lanes x 128 values]  += P [128 x 128 bytes] . Vtile        P's row of a lane: zeros but for the 16 bytes of
//                                                                      its own head's columns
//
// Seven eighths of both products are between a head's queries and another head's keys: computed and never read (the
// tensor pipe has the time: 8 MMAs of M128 N128 K32 a tile, a third of what the tile's bytes take to arrive).  What it
// buys: every lane has work without any replica to fold, a lane's 16 columns are one page of one head (the page's two
// scales are scalars of the thread), the two lanes of a row halve them (8 probabilities a thread and tile), and the
// unit's result leaves the registers straight for the partials.
//
// Persistent blocks, two an SM, each with the same number of tiles: the launch's tiles (the rows' positions in order, 16
// a tile) are dealt out as contiguous runs of T / blocks tiles, never fewer than a split holds.  A run is cut into units
// where a row or a split of `chunk` positions ends, so a split belongs to one block or to two; its partial state goes
// to slot 2 s of the row's states (its head) or 2 s + 1 (its tail), and a block that holds a whole split marks slot
// 2 s + 1 empty (m = -inf, l = 0; the fold passes such states over).  A block's consecutive units mostly belong to one
// row, whose queries are split into the A operand once.  Roles: warps 0-3 softmax (thread = TMEM lane), warp 4
// producer (TMA; a tile's scales come by a bulk copy onto the same mbarrier as its keys), warp 5 the rows' queries and
// the first products, warp 6 the second products.  Every wait is bounded in time and polls the block's abort flag.
//
// Serves: E4M3 pages of 128-wide heads, 8 kv heads, columns x heads-per-group <= 8, chunks of whole 16-position tiles
// up to 2,048 positions.  HBM traffic per unit: its keys and values once, the pages' scales, one partial state.
// Reference: paged_kv_attention/_kernels.py:263-478 (_partition, _window_kernel), cuda_window.cu:284-1065 (cw_tile).
#pragma once

#include "decode_tc.cuh"

namespace crit_b200 {

constexpr int PH_TILE = 16;               // positions a tile holds
constexpr int PH_HEADS = 8;               // kv heads: 16 x 8 = the 128 rows of an operand
constexpr int PH_THREADS = 224;            // 4 softmax warps, a producer warp, a warp for each product's MMAs
constexpr int PH_MAX_LIST = 256;          // window rows a launch lists its work for

// PER_SM blocks an SM.  One: all 512 TMEM columns (scores of the even and of the odd tiles at 0 and 128, outputs at 256),
// probabilities of the even and of the odd tiles, 5 stages.  Two: 256 columns each (scores at 0, outputs at 128), one tile
// of probabilities, 2 stages.  Shared memory (after the 1 KB alignment): Q | P x NBUF | stages (keys 16 KB | values
// 16 KB) | the tiles' scales (1 KB a tile, SCALE_SLOTS tiles in turn) | small.
template <int PER_SM>
struct PhCfg {
    static constexpr int STAGES = PER_SM == 1 ? 5 : 2;
    static constexpr int NBUF = PER_SM == 1 ? 2 : 1;            // tiles of scores (TMEM) and of probabilities (shared memory) in turn
    static constexpr int SCALE_SLOTS = PER_SM == 1 ? 8 : 4;
    static constexpr uint32_t COLUMNS = PER_SM == 1 ? 512 : 256, O = 128 * NBUF;
    static constexpr int OFF_P = DT_OPER;
    static constexpr int OFF_STAGES = (1 + NBUF) * DT_OPER;
    static constexpr int OFF_SCALES = OFF_STAGES + STAGES * 2 * DT_KV_BYTES;
    static constexpr int OFF_SMALL = OFF_SCALES + SCALE_SLOTS * 1024;
    // mbarriers: stage s of keys / values full and empty; the scores' buffers full and read; the probabilities' buffers
    // written and their second product done; the queries
    static constexpr int KFULL = 0, VFULL = STAGES, KEMPTY = 2 * STAGES, VEMPTY = 3 * STAGES, SFULL = 4 * STAGES, SFREE = SFULL + NBUF,
                         PFULL = SFREE + NBUF, PVDONE = PFULL + NBUF, QFULL = PVDONE + NBUF, BARS = QFULL + 1;
    static constexpr int SMALL_QFAC = 0;                          // [2][64] floats: the rows' score factors, by the parity of the queries
    static constexpr int SMALL_BARS = 512;                        // up to 29 mbarriers
    static constexpr int SMALL_TMEM = SMALL_BARS + 29 * 8;
    static constexpr int SMALL_ABORT = SMALL_TMEM + 4;
    static constexpr int SMALL_LIST = 768;                        // unit_first [PH_MAX_LIST + 1] ints (padded)
    static constexpr int SMALL_COUNT = SMALL_LIST + (PH_MAX_LIST + 4) * 4;
    static constexpr int SMALL_START = SMALL_COUNT + PH_MAX_LIST * 4;
    static constexpr int SMALL_ROW = SMALL_START + PH_MAX_LIST * 4;
    static constexpr int SMALL_SPLITS = SMALL_ROW + PH_MAX_LIST * 4;
    static constexpr int SMALL_FIRST = SMALL_SPLITS + PH_MAX_LIST * 4;
    static constexpr int SMEM = 1024 + OFF_SMALL + SMALL_FIRST + PH_MAX_LIST * 8;
};
constexpr int PH_STAGE = 2 * DT_KV_BYTES;

struct PhUnit {
    int r, split, slot, count, ntiles, start;
    bool alone;                 // the unit is a whole split: its sibling slot holds nothing
    int64_t first, L, begin;
    const int32_t* table;
};
// This block's run of the launch's tiles, [g, g1) of rows.units, as units in order, each unit's tiles 0..ntiles-1.
// rows.unit_first[r] is row r's first tile in the launch, rows.splits[r] the number of its tiles.
struct PhWalk {
    int g, g1, i, cursor;
    bool live;
    PhUnit u;
    __device__ __forceinline__ void find(const crit_b200_attend_params& p, const DtRows& rows) {
        int lo = cursor;
        while (rows.unit_first[lo + 1] <= g) ++lo;
        cursor = lo;
        u.r = lo;
        u.count = rows.count[lo];
        u.first = rows.first[lo];
        u.L = u.first + u.count;
        const int per = p.chunk / PH_TILE;              // tiles a split holds
        const int j = g - rows.unit_first[lo];          // the unit's first tile in its row
        u.split = j / per;
        const int within = j - u.split * per;
        int split_end = (u.split + 1) * per;
        split_end = split_end < rows.splits[lo] ? split_end : rows.splits[lo];
        const int jend = split_end - j < g1 - g ? split_end : j + (g1 - g);
        u.begin = (int64_t)j * PH_TILE;
        u.ntiles = jend - j;
        u.slot = 2 * u.split + (within ? 1 : 0);
        u.alone = within == 0 && jend == split_end;
        u.table = p.tables + (int64_t)rows.row[lo] * p.table_stride;
        u.start = rows.start[lo];
    }
    __device__ __forceinline__ void begin(const crit_b200_attend_params& p, const DtRows& rows) {
        const int per = p.chunk / PH_TILE;
        int share = (rows.units + (int)gridDim.x - 1) / (int)gridDim.x;
        share = share > per ? share : per;
        const int64_t at = (int64_t)blockIdx.x * share;
        g = at < rows.units ? (int)at : rows.units;
        g1 = at + share < rows.units ? (int)(at + share) : rows.units;
        i = 0, cursor = 0;
        live = g < g1;
        if (live) find(p, rows);
    }
    __device__ __forceinline__ void next_unit(const crit_b200_attend_params& p, const DtRows& rows) {
        g += u.ntiles, i = 0;
        live = live && g < g1;
        if (live) find(p, rows);
    }
    __device__ __forceinline__ void next(const crit_b200_attend_params& p, const DtRows& rows) {
        if (!live) return;
        if (++i < u.ntiles) return;
        next_unit(p, rows);
    }
};

// SMODE as in decode_tc.cuh: 0 static multipliers, 1 a scale per (slot, kv head), 2 a scale per (page, kv head).
template <int SMODE, int PER_SM>
__global__ void __launch_bounds__(PH_THREADS, PER_SM)
decode_ph_kernel(const crit_b200_attend_params p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    using C = PhCfg<PER_SM>;
    constexpr int smode = SMODE;
    constexpr int PH_STAGES = C::STAGES, NBUF = C::NBUF, PH_SCALE_SLOTS = C::SCALE_SLOTS;
    constexpr int PH_KFULL = C::KFULL, PH_VFULL = C::VFULL, PH_KEMPTY = C::KEMPTY, PH_VEMPTY = C::VEMPTY, PH_SFULL = C::SFULL,
                  PH_SFREE = C::SFREE, PH_PFULL = C::PFULL, PH_PVDONE = C::PVDONE, PH_QFULL = C::QFULL;
    constexpr uint32_t PH_O = C::O, PH_COLUMNS = C::COLUMNS;
    constexpr uint32_t FULLMASK = 0xffffffffu;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024 - (smem_addr(smem_raw) & 1023)) & 1023);
    unsigned char* qbuf = smem;
    unsigned char* pbufs = smem + C::OFF_P;
    unsigned char* stages = smem + C::OFF_STAGES;
    float* scales = reinterpret_cast<float*>(smem + C::OFF_SCALES);
    unsigned char* small = smem + C::OFF_SMALL;
    float* qfac = reinterpret_cast<float*>(small + C::SMALL_QFAC);
    const uint32_t bars = smem_addr(small + C::SMALL_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(small + C::SMALL_TMEM);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(small + C::SMALL_ABORT);
    int* unit_first = reinterpret_cast<int*>(small + C::SMALL_LIST);
    int* m_count = reinterpret_cast<int*>(small + C::SMALL_COUNT);
    int* m_start = reinterpret_cast<int*>(small + C::SMALL_START);
    int* m_row = reinterpret_cast<int*>(small + C::SMALL_ROW);
    int* m_splits = reinterpret_cast<int*>(small + C::SMALL_SPLITS);
    int64_t* m_first = reinterpret_cast<int64_t*>(small + C::SMALL_FIRST);
    auto bar = [&](int which) { return bars + (uint32_t)which * 8u; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.q_heads / p.kv_heads;

    // -- setup ---------------------------------------------------------------------------------------------------------
    if (warp == 0) tmem_alloc(smem_addr(tmem_slot), PH_COLUMNS);
    if (tid == 32) {
        for (int s = 0; s < PH_STAGES; ++s) {
            mbar_init(bar(PH_KFULL + s), 1), mbar_init(bar(PH_KEMPTY + s), 1);
            mbar_init(bar(PH_VFULL + s), 1), mbar_init(bar(PH_VEMPTY + s), 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(bar(PH_SFULL + b), 1), mbar_init(bar(PH_SFREE + b), 128);
            mbar_init(bar(PH_PFULL + b), 128), mbar_init(bar(PH_PVDONE + b), 1);
        }
        mbar_init(bar(PH_QFULL), 32);
        *abort_flag = 0;
        mbar_init_fence();
    }
    for (int idx = tid; idx < (1 + NBUF) * DT_OPER / 16; idx += PH_THREADS) reinterpret_cast<uint4*>(qbuf)[idx] = make_uint4(0, 0, 0, 0);
    for (int rr = tid; rr < p.n_rows; rr += PH_THREADS) {
        int cnt = p.counts ? p.counts[rr] : p.columns;
        cnt = cnt > p.columns ? p.columns : (cnt < 0 ? 0 : cnt);
        const int64_t first = p.firsts[rr];
        m_count[rr] = cnt, m_start[rr] = p.starts[rr], m_row[rr] = p.rows[rr], m_first[rr] = first;
        m_splits[rr] = cnt > 0 ? (int)((first + cnt + PH_TILE - 1) / PH_TILE) : 0;          // the row's tiles
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {            // the rows' first tiles in the launch
        int carry = 0;
        for (int base = 0; base < p.n_rows; base += 32) {
            const int rr = base + lane;
            int scan = rr < p.n_rows ? m_splits[rr] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(FULLMASK, scan, o);
                if (lane >= o) scan += up;
            }
            if (rr < p.n_rows) unit_first[rr + 1] = carry + scan;
            carry += __shfl_sync(FULLMASK, scan, 31);
        }
        if (lane == 0) unit_first[0] = 0;
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    DtRows rows;
    rows.unit_first = unit_first, rows.count = m_count, rows.start = m_start, rows.row = m_row, rows.splits = m_splits;
    rows.first = m_first;
    rows.units = unit_first[p.n_rows];
    const uint32_t tpp = (uint32_t)p.page >> 4;
    const uint32_t pages_total = (uint32_t)(p.slots / p.page);
    int where = 0;              // which role's wait gave up

    if (warp == 4) {
        // -- producer: the unit's page ids in registers (tile 32 * j + lane of the unit in slot j of lane `lane`), loaded a
        //    unit ahead; lane 0 issues a tile's two boxes and the bulk copies of its scales ----------------------------------
        PhWalk w0, w1;
        w0.begin(p, rows);
        w1 = w0, w1.next_unit(p, rows);
        auto fetch_pages = [&](const PhWalk& w, int (&pg)[DT_NB]) {
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) pg[j] = -1;
            if (!w.live) return;
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) {
                const int64_t pos0 = w.u.begin + (int64_t)(lane + 32 * j) * 16;
                if (lane + 32 * j < w.u.ntiles) {
                    pg[j] = w.u.table[(uint32_t)(pos0 >> 4) / tpp];
                    if ((uint32_t)pg[j] >= pages_total) {       // outside the page tensor: read as past the end (zeros), reported
                        pg[j] = -1;
                        if (p.status) atomicExch(p.status, CRIT_B200_STATUS_BOUNDS);
                    }
                }
            }
        };
        // A tile's keys are asked for one tile before the values of the tile before it: the keys' place frees early (after
        // the first product), the values' late (after the second), and neither request waits behind the other's place.
        // The tile's scales travel with its keys (the softmax needs them with the scores), into one of eight places in
        // turn: the place of tile t is written again for tile t + 8, whose keys are asked for after the scores of tile
        // t + 3 are complete, which were issued after every softmax thread had read the scores of tile t + 1.
        int pg0[DT_NB], pg1[DT_NB];
        fetch_pages(w0, pg0);
        int t = 0, v_slot = 0;
        bool ok = true;
        auto ask_values = [&](int tv, int slot0) {
            const int stage = tv % PH_STAGES;
            ok = dt_wait<100>(bar(PH_VEMPTY + stage), (uint32_t)((tv / PH_STAGES) & 1) ^ 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) return;
            if (lane == 0) {
                mbar_expect_tx(bar(PH_VFULL + stage), (uint32_t)DT_KV_BYTES);
                tma_load_3d(smem_addr(stages + stage * PH_STAGE) + DT_KV_BYTES, &vmap, 0, slot0, 0, bar(PH_VFULL + stage));
            }
            __syncwarp();
        };
        while (w0.live && ok) {
            fetch_pages(w1, pg1);
            for (int i = 0; i < w0.u.ntiles; ++i, ++t) {
                int pgs = pg0[0];
#pragma unroll
                for (int j = 1; j < DT_NB; ++j)
                    if ((i >> 5) == j) pgs = pg0[j];
                const int pgb = __shfl_sync(FULLMASK, pgs, i & 31);
                const uint32_t tile16 = (uint32_t)(w0.u.begin >> 4) + (uint32_t)i;
                const int slot0 = pgb >= 0 ? (int)((int64_t)pgb * p.page + ((tile16 % tpp) << 4)) : (int)p.slots;
                const int stage = t % PH_STAGES;
                ok = dt_wait<100>(bar(PH_KEMPTY + stage), (uint32_t)((t / PH_STAGES) & 1) ^ 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                float* scs = scales + (t % PH_SCALE_SLOTS) * 256;
                if (smode != 0 && pgb < 0) {
                    for (int c = lane; c < 256; c += 32) scs[c] = 1.f;
                    __syncwarp();
                }
                if (lane == 0) {
                    const uint32_t full = bar(PH_KFULL + stage);
                    if (smode == 2 && pgb >= 0) {
                        mbar_expect_tx(full, (uint32_t)DT_KV_BYTES + 64u);
                        bulk_load(smem_addr(scs), p.key_scales + (int64_t)pgb * PH_HEADS, 32u, full);
                        bulk_load(smem_addr(scs + 8), p.value_scales + (int64_t)pgb * PH_HEADS, 32u, full);
                    } else if (smode == 1 && pgb >= 0) {
                        mbar_expect_tx(full, (uint32_t)DT_KV_BYTES + 1024u);
                        bulk_load(smem_addr(scs), p.key_scales + (int64_t)slot0 * PH_HEADS, 512u, full);
                        bulk_load(smem_addr(scs + 128), p.value_scales + (int64_t)slot0 * PH_HEADS, 512u, full);
                    } else {
                        mbar_expect_tx(full, (uint32_t)DT_KV_BYTES);
                    }
                    tma_load_3d(smem_addr(stages + stage * PH_STAGE), &kmap, 0, slot0, 0, full);
                }
                __syncwarp();
                if (t > 0) {
                    ask_values(t - 1, v_slot);
                    if (!ok) break;
                }
                v_slot = slot0;
            }
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) pg0[j] = pg1[j];
            w0 = w1, w1.next_unit(p, rows);
        }
        if (ok && t > 0) ask_values(t - 1, v_slot);
        if (!ok) {              // leaving early: the copies in flight land first (bounded)
            where = 0x610;
            for (int tt = t > PH_STAGES ? t - PH_STAGES : 0; tt <= t; ++tt) {
                mbar_wait(bar(PH_KFULL + tt % PH_STAGES), (uint32_t)(tt / PH_STAGES) & 1u, 20000000ull);
                if (tt + 1 < t) mbar_wait(bar(PH_VFULL + tt % PH_STAGES), (uint32_t)(tt / PH_STAGES) & 1u, 20000000ull);
            }
        }
    } else if (warp == 5) {
        // -- the rows' queries and the first products, S = Q K^T of every tile in order -----------------------------------------
        const uint32_t idesc_s = idesc_f8(false, 128, 128);
        const float sl2 = p.scale * LOG2E * (smode == 0 ? p.key_multiplier : 1.f);
        const int qt = lane & 3, jr = lane >> 2;
        bool ok = true;
        // A window row's queries as the A operand: row j of kv head h's group (column j / G, head h G + j % G) goes to
        // lanes 16 h + j (hi term) and 16 h + 8 + j (lo term); 4 lanes a row, one kv head a pass.
        auto store_q = [&](const PhUnit& u, int qn) {
            const int col = jr / G, gq = jr - col * G;
            const bool live_row = jr < p.columns * G && col < u.count;
#pragma unroll 2
            for (int h = 0; h < PH_HEADS; ++h) {
                uint4 raw[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) raw[c] = make_uint4(0, 0, 0, 0);
                if (live_row) {
                    const char* src = (const char*)p.q + ((int64_t)(u.start + col) * p.q_stride_token +
                                                          (int64_t)(h * G + gq) * p.q_stride_head + qt * 32) * 2;
#pragma unroll
                    for (int c = 0; c < 4; ++c) raw[c] = *reinterpret_cast<const uint4*>(src + c * 16);
                }
                float x[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t wds[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float2 f;
                        if (p.q_dtype == CRIT_B200_DTYPE_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wds[e]));
                        else f = __half22float2(*reinterpret_cast<const __half2*>(&wds[e]));
                        x[c * 8 + 2 * e] = f.x, x[c * 8 + 2 * e + 1] = f.y;
                    }
                }
                float amax = 0.f;
#pragma unroll
                for (int c = 0; c < 32; ++c) amax = fmaxf(amax, fabsf(x[c]));
                amax = fmaxf(amax, __shfl_xor_sync(FULLMASK, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(FULLMASK, amax, 2));
                int e = 0;                  // 2^e puts the row's largest magnitude in [128, 256)
                if (amax > 0.f) {
                    e = 7 - (int)(((__float_as_uint(amax) >> 23) & 0xffu) - 127u);
                    e = e > 100 ? 100 : (e < -100 ? -100 : e);
                }
                const float up = __uint_as_float((uint32_t)(e + 127) << 23), down = __uint_as_float((uint32_t)(127 - e) << 23);
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t h0, l0, h1, l1;
                    split_e4m3x2<1>(x[4 * c] * up, x[4 * c + 1] * up, h0, l0);
                    split_e4m3x2<1>(x[4 * c + 2] * up, x[4 * c + 3] * up, h1, l1);
                    hi[c] = h0 | (h1 << 16), lo[c] = l0 | (l1 << 16);
                }
                const int row_hi = 16 * h + jr, row_lo = row_hi + 8;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int chunk = 2 * qt + c;
                    *reinterpret_cast<uint4*>(qbuf + row_hi * 128 + ((chunk ^ (row_hi & 7)) << 4)) =
                        make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
                    *reinterpret_cast<uint4*>(qbuf + row_lo * 128 + ((chunk ^ (row_lo & 7)) << 4)) =
                        make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
                }
                if (qt == 0) qfac[(qn & 1) * 64 + h * 8 + jr] = down * sl2;
            }
            fence_proxy_async();
            mbar_arrive(bar(PH_QFULL));
            __syncwarp();
        };
        PhWalk w;
        w.begin(p, rows);
        int t = 0, qn = 0, q_row = -1;
        while (w.live && ok) {
            const int stage = t % PH_STAGES, sb = t % NBUF;
            if (w.i == 0 && w.u.r != q_row) {
                // Another window row: once the last tile's probabilities are written, every first product that read the old
                // queries has completed and every softmax thread has passed its wait for them (the queries' barrier never
                // runs two phases ahead of a waiter): the row's queries go over the last row's.
                if (t > 0) {
                    ok = dt_wait<32>(bar(PH_PFULL + (t - 1) % NBUF), (uint32_t)((t - 1) / NBUF) & 1u, abort_flag);
                    ok = __all_sync(FULLMASK, ok);
                    if (!ok) break;
                }
                store_q(w.u, qn);
                ++qn, q_row = w.u.r;
            }
            ok = dt_wait<32>(bar(PH_KFULL + stage), (uint32_t)(t / PH_STAGES) & 1u, abort_flag) &&
                 dt_wait<32>(bar(PH_SFREE + sb), (uint32_t)((t / NBUF) & 1) ^ 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t qa = smem_addr(qbuf), ka = smem_addr(stages + stage * PH_STAGE);
#pragma unroll
                for (int kk = 0; kk < DT_D / 32; ++kk)
                    umma_f8(tmem + 128u * sb, smem_desc_sw128(qa + kk * 32, 0, 1024), smem_desc_sw128(ka + kk * 32, 0, 1024),
                            idesc_s, kk > 0);
                umma_commit(bar(PH_SFULL + sb));
                umma_commit(bar(PH_KEMPTY + stage));
            }
            __syncwarp();
            w.next(p, rows);
            ++t;
        }
        if (!ok) where = 0x620;
    } else if (warp == 6) {
        // -- the second products, O (+)= P V of every tile in order, from a warp of their own: issuing a tile's eight MMAs
        //    and four commits from one thread took longer than the tile's softmax -------------------------------------------
        const uint32_t idesc_o = idesc_f8(true, 128, DT_D);
        bool ok = true;
        PhWalk w;
        w.begin(p, rows);
        int t = 0;
        while (w.live && ok) {
            const int pstage = t % PH_STAGES, pb = t % NBUF;
            ok = dt_wait<32>(bar(PH_PFULL + pb), (uint32_t)(t / NBUF) & 1u, abort_flag) &&
                 dt_wait<32>(bar(PH_VFULL + pstage), (uint32_t)(t / PH_STAGES) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t pa = smem_addr(pbufs + pb * DT_OPER), va = smem_addr(stages + pstage * PH_STAGE + DT_KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_f8(tmem + PH_O, smem_desc_sw128(pa + kk * 32, 0, 1024), smem_desc_sw128(va + kk * 4096, 16, 1024),
                            idesc_o, w.i > 0 || kk > 0);
                umma_commit(bar(PH_VEMPTY + pstage));
                umma_commit(bar(PH_PVDONE + pb));
            }
            __syncwarp();
            w.next(p, rows);
            ++t;
        }
        if (!ok) where = 0x630;
    } else {
        // -- softmax: thread = TMEM lane 32 * warp + lane.  Lane group lg (16 lanes) is kv head lg: lanes 0-7 hold the hi
        //    terms of its 8 query rows, lanes 8-15 their lo terms, and its columns of a tile are [16 lg, 16 lg + 16), the
        //    tile's 16 positions under that head.  The two lanes of a row share them: the hi lane takes positions 0-7, the
        //    lo lane 8-15, after one exchange of scores ---------------------------------------------------------------------
        const int lg = warp * 2 + (lane >> 4);
        const int jr = lane & 7;
        const bool second = (lane & 8) != 0;
        const int col = jr / G, gq = jr - col * G;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int prow = warp * 32 + lane;
        const int row_hi = prow & ~8, row_lo = row_hi | 8;
        const int cofs = second ? 8 : 0;                          // this thread's first position of a tile
        const float vmul = smode == 0 ? p.value_multiplier : 1.f;
        const float lo_unscale = second ? 1.f / 16.f : 1.f;     // this lane's outputs: the lo probabilities were stored times 16
        const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
        const int pb_hi = row_hi * 128 + ((lg ^ (row_hi & 7)) << 4) + cofs;       // this thread's bytes of a P tile
        const int pb_lo = row_lo * 128 + ((lg ^ (row_lo & 7)) << 4) + cofs;
        bool ok = true;
        PhWalk w;
        w.begin(p, rows);
        int t = 0, qn = 0, q_row = -1;
        float a_r = 0.f;
        while (w.live && ok) {
            PhWalk after = w;                   // the unit after this one, found while this one's first scores are on their way
            after.next_unit(p, rows);
            const int prow_first = p.offsets ? p.offsets[w.u.r] - p.offsets[0] : w.u.r * p.columns;
            if (w.u.r != q_row) {
                ok = dt_wait(bar(PH_QFULL), (uint32_t)qn & 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                a_r = qfac[(qn & 1) * 64 + lg * 8 + jr];
                ++qn, q_row = w.u.r;
            }
            const bool valid = jr < p.columns * G && col < w.u.count;
            const int lastpos = valid ? (int)(w.u.first + col) : -1;
            const int first32 = w.u.first > 0x7fffffffLL ? 0x7fffffff : (int)w.u.first;
            float m_run = -INFINITY, l_run = 0.f;
            for (int i = 0; i < w.u.ntiles; ++i, ++t) {
                const int stage = t % PH_STAGES, sb = t % NBUF;
                const int tile_pos = (int)w.u.begin + i * PH_TILE;
                ok = dt_wait(bar(PH_SFULL + sb), (uint32_t)(t / NBUF) & 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                tc_fence_after();
                if (tile_pos + PH_TILE > w.u.L) {
                    ok = dt_wait(bar(PH_VFULL + stage), (uint32_t)(t / PH_STAGES) & 1u, abort_flag);
                    ok = __all_sync(FULLMASK, ok);
                    if (!ok) break;
                    // the row's last page is partly filled: its value rows past the last position hold whatever the
                    // page held before, and a probability of 0 times a NaN code would not be 0.  Zeros instead (the
                    // second product reads them after this thread's arrival on the P barrier, behind the proxy fence).
                    unsigned char* vst = stages + stage * PH_STAGE + DT_KV_BYTES;
                    const int from = (int)(w.u.L - tile_pos);
                    for (int idx = tid; idx < 128 * 8; idx += 128)
                        if (((idx >> 3) & 15) >= from) *reinterpret_cast<uint4*>(vst + idx * 16) = make_uint4(0, 0, 0, 0);
                }
                // this lane's scores under its own head, then the exchange: each lane of a row ends with the sums hi + lo
                // of its own 8 positions.  (tcgen05.ld wants its first column on a multiple of 32 here: the head's 16
                // columns are read as the half of 32.)
                float s[8];
                {
                    float both[32];
                    tmem_ld32(tmem + lane_base + 128u * sb + (uint32_t)((lg >> 1) * 32), both);
                    tc_fence_before();
                    mbar_arrive(bar(PH_SFREE + sb));
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const float m0 = (lg & 1) ? both[16 + c] : both[c], m1 = (lg & 1) ? both[24 + c] : both[8 + c];
                        const float give = second ? m0 : m1, keep = second ? m1 : m0;
                        s[c] = keep + __shfl_xor_sync(FULLMASK, give, 8);
                    }
                }
                const float* scs = scales + (t % PH_SCALE_SLOTS) * 256;
                const bool mask = !valid || tile_pos + PH_TILE - 1 > first32;
                float kf = a_r, lv = 0.f, rv = 1.f;
                if (smode == 2) {
                    const float vs = scs[8 + lg];
                    kf = a_r * scs[lg], lv = __log2f(vs), rv = __fdividef(1.f, vs);
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    if (smode == 1) {
                        kf = a_r, lv = 0.f;
                        if (tile_pos + cofs + c < w.u.L) {
                            kf = a_r * scs[(cofs + c) * PH_HEADS + lg];
                            lv = __log2f(scs[128 + (cofs + c) * PH_HEADS + lg]);
                        }
                    }
                    float x = s[c] * kf + lv;
                    if (mask && tile_pos + cofs + c > lastpos) x = -INFINITY;
                    s[c] = x;
                    if (c & 1) mx1 = fmaxf(mx1, x);
                    else mx0 = fmaxf(mx0, x);
                }
                float mx = fmaxf(mx0, mx1);
                mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 8));           // the row's other half
                const bool moved = mx > m_run + DT_LAZY || m_run == -INFINITY;
                const float top = moved ? mx : m_run;
                const float sub = top == -INFINITY ? 0.f : top;
                const float alpha = moved ? ex2(m_run - sub) : 1.f;
                const bool rescale = moved && top != m_run && i > 0;
                m_run = top;

                // this tile's P tile is free once the second product that read it last (NBUF tiles before) has landed
                ok = dt_wait(bar(PH_PVDONE + sb), (uint32_t)((t / NBUF) & 1) ^ 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                float psum = 0.f;
                uint32_t wh[2], wl[2];
#pragma unroll
                for (int c2 = 0; c2 < 4; ++c2) {
                    const float pa = ex2(s[2 * c2] - sub), pb = ex2(s[2 * c2 + 1] - sub);
                    if (smode == 1) {
                        float va = 1.f, vb = 1.f;
                        if (tile_pos + cofs + 2 * c2 < w.u.L) va = scs[128 + (cofs + 2 * c2) * PH_HEADS + lg];
                        if (tile_pos + cofs + 2 * c2 + 1 < w.u.L) vb = scs[128 + (cofs + 2 * c2 + 1) * PH_HEADS + lg];
                        psum += __fdividef(pa, va) + __fdividef(pb, vb);
                    } else {
                        psum += pa + pb;
                    }
                    uint32_t h2, l2;
                    split_e4m3x2<16>(pa, pb, h2, l2);
                    if (c2 & 1) wh[c2 >> 1] |= h2 << 16, wl[c2 >> 1] |= l2 << 16;
                    else wh[c2 >> 1] = h2, wl[c2 >> 1] = l2;
                }
                *reinterpret_cast<uint2*>(pbufs + sb * DT_OPER + pb_hi) = make_uint2(wh[0], wh[1]);
                *reinterpret_cast<uint2*>(pbufs + sb * DT_OPER + pb_lo) = make_uint2(wl[0], wl[1]);
                l_run = l_run * alpha + psum * rv;

                if (__any_sync(FULLMASK, rescale)) {
                    // a maximum moved: the warp brings its output lanes to the new reference, once the second product of
                    // the tile before has landed (the products complete in order: the outputs are settled then)
                    ok = dt_wait(bar(PH_PVDONE + (t - 1) % NBUF), (uint32_t)((t - 1) / NBUF) & 1u, abort_flag);
                    ok = __all_sync(FULLMASK, ok);
                    if (!ok) break;
                    tc_fence_after();
                    dt_rescale(tmem + lane_base + PH_O, alpha);
                }
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(bar(PH_PFULL + sb));
            }
            if (!ok) break;

            // -- the unit's result: its last second product, hi + lo of the outputs, one row a pair of lanes ------------------
            const int tl = t - 1;
            ok = dt_wait(bar(PH_PVDONE + tl % NBUF), (uint32_t)(tl / NBUF) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            const float l_row = l_run + __shfl_xor_sync(FULLMASK, l_run, 8);
            const bool fits = p.workspace && 2 * w.u.split + 1 < p.max_splits && prow_first >= 0 && prow_first + w.u.count <= p.partial_rows;
            if (!fits && tid == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_PLAN);
            const int head = lg * G + gq;
            const int64_t at = ((int64_t)(prow_first + col) * p.q_heads + head) * p.max_splits + w.u.slot;
            // the hi lane keeps value columns 0..63, the lo lane 64..127, 32 at a time
#pragma unroll
            for (int c4 = 0; c4 < 2; ++c4) {
                float oa[32], ob[32];
                tmem_ld32(tmem + lane_base + PH_O + 32u * c4, oa);
                tmem_ld32(tmem + lane_base + PH_O + 64u + 32u * c4, ob);
                float keep[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float give = (second ? oa[j] : ob[j]) * lo_unscale;
                    const float mine = (second ? ob[j] : oa[j]) * lo_unscale;
                    keep[j] = (mine + __shfl_xor_sync(FULLMASK, give, 8)) * vmul;
                }
                const int dv = (second ? 64 : 0) + 32 * c4;
                if (valid && fits) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(p.workspace + at * DT_D + dv + 4 * j) =
                            make_float4(keep[4 * j], keep[4 * j + 1], keep[4 * j + 2], keep[4 * j + 3]);
                }
            }
            tc_fence_before();
            if (valid && fits && !second) {
                p.workspace[states * DT_D + at] = m_run;
                p.workspace[states * (DT_D + 1) + at] = l_row;
                if (w.u.alone) {                // nobody holds the split's tail: its slot reads as empty
                    p.workspace[states * DT_D + at + 1] = -INFINITY;
                    p.workspace[states * (DT_D + 1) + at + 1] = 0.f;
                }
            }
            w = after;
        }
        if (!ok) where = 0x640;
    }

    if (where && p.status) atomicExch(p.status, where);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, PH_COLUMNS);
}

}  // namespace crit_b200
