// Split-K decode / speculative-verify attention over E4M3 pages on the fifth-generation tensor cores: the page bytes go
// from HBM to shared memory by TMA and from there straight into tcgen05.mma (kind::f8f6f4); no thread ever converts a
// key or a value.
//
// Two persistent blocks per SM (192 threads, 256 TMEM columns and about 105 KB of shared memory each) walk a work list
// of units (window row, split of `chunk` positions, kv head), built on the device from the rows' lengths: block b takes
// units b, b + grid, ...  A unit's positions stream through a ring of DT_STAGES stages as tiles of 128 positions (eight
// TMA boxes of [16 positions][1 kv head][128 bytes] for the keys, eight for the values, 128-byte swizzle: the K-major /
// MN-major operand layouts of the MMA); a stage's keys and values land and free on separate mbarriers (the keys are free
// once the first product has read them), and the ring runs on across units, so HBM never waits for a unit's epilogue.
// One block's chain of dependent steps per tile (scores -> softmax -> probabilities -> outputs) is long; the SM's other
// block fills its gaps.  Warp roles:
//   warps 0-3  softmax: thread = one TMEM lane.  Reads its scores (tcgen05.ld), applies the row's and the pages' scales,
//              keeps the running maximum (lazily) and sum, writes its probabilities as E4M3 into the A-operand tile of the
//              second product, rescales its output lane in TMEM when the maximum moved, and folds / writes the unit's
//              result;
//   warp 4     producer: a unit's page ids and page scales in registers, loaded one and two units ahead; TMA loads;
//   warp 5     MMA issue (one lane): S = Q K^T (4 MMAs of M128 N128 K32 per tile), O += P V (4 MMAs) one tile behind; at a
//              unit's start it first issues the last unit's final second product, then splits the unit's queries (whose
//              global loads it started a unit earlier) into the A operand.
// The MMA multiplies E4M3 by E4M3, so the 16-bit queries and the probabilities are each split in two E4M3 terms:
// x * 2^e = hi + lo, hi = e4m3(x * 2^e), lo = e4m3(x * 2^e - hi), 2^e a per-row power of two that puts the row's largest
// magnitude in [128, 256): exact for bf16 queries (8 significant bits = 4 + 4), to 2^-9 of the value for FP16 queries
// and for the probabilities.  hi and lo are separate rows of the M = 128 operand (TMEM lanes j and j + 8 of a group of
// 16), so one MMA computes both terms and their sum is one shuffle.  A unit has at most 32 query rows (columns x heads
// of the group) in NRG groups of 8; a group's 16 lanes are replicated 8 / NRG times over the 128 lanes, each replica
// owning 16 * NRG columns of a tile (its probabilities elsewhere are zeros), and the two lanes of a row share those
// columns, so every lane does distinct softmax work.
// The page codes enter the products exactly; the scales of the keys multiply the scores' columns, those of the values
// are folded into the probabilities as an exponent offset (p' = 2^(s + log2 vs - m)), so the accumulators need no
// per-page pass.  Every wait is bounded in time and polls a block-wide abort flag; a wait that runs out sets the status
// word, the block frees its TMEM and leaves without hanging.
//
// HBM traffic per unit: its keys and values once (the algorithmic bytes), 8 scale floats per page, the queries, one
// partial state.  Reference: paged_kv_attention/_kernels.py:263-478 (_partition, _window_kernel),
// cuda_window.cu:284-1065 (cw_tile); the partial states and their merge are those of decode_kernel.cuh.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "tcgen05.cuh"

namespace crit_b200 {

constexpr int DT_N = 128;                 // positions a tile holds
constexpr int DT_D = 128;                 // head width (keys and values)
constexpr int DT_STAGES = 2;
constexpr int DT_THREADS = 192;
constexpr int DT_MAX_LIST = 256;          // window rows a launch lists its work for
constexpr int DT_MAX_CHUNK = 2048;        // positions of a split: the producer holds a unit's page ids in registers
constexpr int DT_NB = DT_MAX_CHUNK / 512; // ... boxes of 16 positions per lane
constexpr int DT_KV_BYTES = DT_N * 128;   // one tile of keys (or values): 16 KB
constexpr int DT_STAGE = 2 * DT_KV_BYTES + 1024;     // keys | values | 128 key scales, 128 value scales
constexpr int DT_OPER = 128 * 128;        // an A operand: 128 rows of 128 bytes
constexpr float DT_LAZY = 8.f;            // the running maximum moves only when a tile beats it by 2^8: a probability is
                                          // at most 2^8, inside E4M3's range, and the largest of a row is at least 1
constexpr uint32_t DT_COLUMNS = 256;      // TMEM: scores 0..127, outputs 128..255
constexpr uint32_t DT_O = 128;
constexpr uint64_t DT_WAIT_NS = 250000000ull;

// shared memory (after the 1 KB alignment): Q | P (the unit fold's scratch too) | stages | small
constexpr int DT_OFF_Q = 0;
constexpr int DT_OFF_P = DT_OPER;
constexpr int DT_OFF_STAGES = 2 * DT_OPER;
constexpr int DT_OFF_SMALL = DT_OFF_STAGES + DT_STAGES * DT_STAGE;
constexpr int DT_SMALL_QFAC = 0;                              // [2][32] floats: the rows' score factors, by the unit's parity
constexpr int DT_SMALL_FM = 256;                              // [64] floats
constexpr int DT_SMALL_FL = 512;                              // [64] floats
constexpr int DT_SMALL_BARS = 768;                            // 16 mbarriers
constexpr int DT_SMALL_TMEM = 768 + 16 * 8;                   // the TMEM address
constexpr int DT_SMALL_ABORT = DT_SMALL_TMEM + 4;
constexpr int DT_SMALL_LIST = 1024;                           // unit_first [DT_MAX_LIST + 1] ints (padded to 16 bytes)
constexpr int DT_LIST_BYTES = (DT_MAX_LIST + 4) * 4;
constexpr int DT_SMALL_COUNT = DT_SMALL_LIST + DT_LIST_BYTES; // the rows' counts, starts, table rows, splits: ints each
constexpr int DT_SMALL_START = DT_SMALL_COUNT + DT_MAX_LIST * 4;
constexpr int DT_SMALL_ROW = DT_SMALL_START + DT_MAX_LIST * 4;
constexpr int DT_SMALL_SPLITS = DT_SMALL_ROW + DT_MAX_LIST * 4;
constexpr int DT_SMALL_FIRST = DT_SMALL_SPLITS + DT_MAX_LIST * 4;   // the rows' first positions [DT_MAX_LIST] int64
constexpr int DT_SMEM = 1024 + DT_OFF_SMALL + DT_SMALL_FIRST + DT_MAX_LIST * 8;

// mbarriers: a stage's keys and values land and are released separately (the keys are free once the first product
// has read them, long before the values), so the next keys stream in while a tile's softmax runs
enum { DT_KFULL = 0, DT_VFULL = 2, DT_KEMPTY = 4, DT_VEMPTY = 6, DT_SFULL = 8, DT_SFREE = 9, DT_PFULL = 10, DT_PVDONE = 11,
       DT_QFULL = 12, DT_FOLD_A = 13, DT_FOLD_B = 14 };

__device__ __forceinline__ uint32_t idesc_f8(bool b_mn_major, int M, int N) {
    uint32_t d = 0;
    d |= 1u << 4;                                  // D format: F32; A and B formats 0: E4M3
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Two FP16 values -> two E4M3 bytes (the low half in the low byte), round to nearest, saturating.
__device__ __forceinline__ uint32_t f16x2_to_e4m3x2(uint32_t h2) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(h2));
    return r;
}
// hi + lo / LOSCALE = the pair to within 2^-8 of each value (two E4M3 bytes each, the first value in the low byte).
// LOSCALE 16 (the probabilities): the lo term is stored times 16, which keeps the small ones out of E4M3's subnormals
// (a probability down to 2^-13 of the row's reference survives); the lo rows' outputs are divided by 16 at the end.
template <int LOSCALE>
__device__ __forceinline__ void split_e4m3x2(float a, float b, uint32_t& hi, uint32_t& lo) {
    __half2 h = __floats2half2_rn(a, b);
    const uint32_t hw = *reinterpret_cast<uint32_t*>(&h);
    hi = f16x2_to_e4m3x2(hw);
    const uint32_t back = e4m3x2_to_f16x2(hi);
    __half2 rest = __hsub2(h, *reinterpret_cast<const __half2*>(&back));
    if (LOSCALE != 1) rest = __hmul2(rest, __float2half2_rn((float)LOSCALE));
    lo = f16x2_to_e4m3x2(*reinterpret_cast<uint32_t*>(&rest));
}

// A bounded wait that also gives up when another thread of the block already did.  BACKOFF: nanoseconds to sleep
// between polls (the roles that wait long share their issue slots with the softmax warps; those poll without a pause).
// The polling loop is one out-of-line function: the kernel has some thirty waits, and their loops inline would be a
// good part of its instruction footprint.
__device__ __noinline__ bool dt_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned backoff) {
    const uint64_t t0 = global_ns();
    do {
        if (backoff) __nanosleep(backoff);
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    } while (global_ns() - t0 < DT_WAIT_NS);
    *abort_flag = 1;
    return false;
}
template <int BACKOFF = 0>
__device__ __forceinline__ bool dt_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    return dt_wait_slow(bar, parity, abort_flag, BACKOFF);
}
// A warp's output lanes times a factor per lane (the rare move of a running maximum), out of line for the same reason.
__device__ __noinline__ void dt_rescale(uint32_t taddr, float alpha) {
#pragma unroll
    for (int c4 = 0; c4 < DT_D / 32; ++c4) {
        float o[32];
        tmem_ld32(taddr + 32u * c4, o);
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] *= alpha;
        tmem_st32(taddr + 32u * c4, o);
    }
}

// The launch's rows, copied to shared memory once: no role reads global memory to find its next unit.
struct DtRows {
    const int* unit_first;
    const int* count;
    const int* start;
    const int* row;
    const int* splits;
    const int64_t* first;
    int units;
};

// One unit of the work list.
struct DtUnit {
    int r, h, split, count, nsplit, ntiles, start;
    int64_t first, L, begin;
    const int32_t* table;
};
// `cursor`: a row at or before the unit's (a block's units come in rising order, so the search is a short walk).
__device__ __forceinline__ void dt_unit(const crit_b200_attend_params& p, const DtRows& rows, int unit, int& cursor, DtUnit& u) {
    int lo = cursor;
    while (rows.unit_first[lo + 1] <= unit) ++lo;
    cursor = lo;
    u.r = lo;
    u.count = rows.count[lo];
    u.first = rows.first[lo];
    u.L = u.first + u.count;
    u.nsplit = rows.splits[lo];
    const unsigned local = (unsigned)(unit - rows.unit_first[lo]);
    u.split = (int)(local / (unsigned)p.kv_heads);
    u.h = (int)(local - (unsigned)u.split * (unsigned)p.kv_heads);
    u.begin = (int64_t)u.split * p.chunk;
    const int span = (int)(u.begin + p.chunk < u.L ? p.chunk : u.L - u.begin);
    u.ntiles = (span + DT_N - 1) / DT_N;
    u.table = p.tables + (int64_t)rows.row[lo] * p.table_stride;
    u.start = rows.start[lo];
}

// A walk over this block's tiles in order: units block, block + grid, ..., each unit's tiles 0..ntiles-1.
struct DtWalk {
    int unit, k, i, cursor;
    bool live;
    DtUnit u;
    __device__ __forceinline__ void begin(const crit_b200_attend_params& p, const DtRows& rows) {
        unit = blockIdx.x, k = 0, i = 0, cursor = 0;
        live = unit < rows.units;
        if (live) dt_unit(p, rows, unit, cursor, u);
    }
    __device__ __forceinline__ void next(const crit_b200_attend_params& p, const DtRows& rows) {
        if (!live) return;
        if (++i < u.ntiles) return;
        next_unit(p, rows);
    }
    __device__ __forceinline__ void next_unit(const crit_b200_attend_params& p, const DtRows& rows) {
        i = 0, ++k, unit += gridDim.x;
        live = unit < rows.units;
        if (live) dt_unit(p, rows, unit, cursor, u);
    }
};

// NRG: groups of 8 query rows a unit holds (1, 2 or 4: up to 8, 16 or 32 rows).  A group takes 16 TMEM lanes (hi and lo
// terms), so the 128 lanes hold 8 / NRG replicas of the unit's rows, each owning 16 * NRG columns of a tile.
// SMODE: 0 static multipliers, 1 a scale per (slot, kv head), 2 a scale per (page, kv head): a template parameter, so
// the loops hold one rule's code only (the kernel's instruction footprint is what its warps wait for most: taking the
// other rules' code out of the loops shortened a tile's softmax by a third).
template <int NRG, int SMODE>
__global__ void __launch_bounds__(DT_THREADS, 2)
decode_tc_kernel(const crit_b200_attend_params p, const __grid_constant__ CUtensorMap kmap,
                 const __grid_constant__ CUtensorMap vmap) {
    constexpr int smode = SMODE;
    constexpr int REPL = 8 / NRG;         // replicas of the unit's rows
    constexpr int R = 8 * NRG;            // query rows a unit holds (padded)
    constexpr int W = DT_N / REPL;        // columns of a tile one replica owns
    constexpr int CT = W / 2;             // ... and one thread: the two lanes of a row halve them
    constexpr int GC = CT < 16 ? CT : 16; // a thread's columns come in groups inside one box of 16 positions
    constexpr int NGC = CT / GC;
    constexpr uint32_t FULLMASK = 0xffffffffu;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024 - (smem_addr(smem_raw) & 1023)) & 1023);
    unsigned char* qbuf = smem + DT_OFF_Q;
    unsigned char* pbuf = smem + DT_OFF_P;
    unsigned char* stages = smem + DT_OFF_STAGES;
    unsigned char* small = smem + DT_OFF_SMALL;
    float* qfac = reinterpret_cast<float*>(small + DT_SMALL_QFAC);
    float* fm = reinterpret_cast<float*>(small + DT_SMALL_FM);
    float* fl = reinterpret_cast<float*>(small + DT_SMALL_FL);
    const uint32_t bars = smem_addr(small + DT_SMALL_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(small + DT_SMALL_TMEM);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(small + DT_SMALL_ABORT);
    int* unit_first = reinterpret_cast<int*>(small + DT_SMALL_LIST);
    int* m_count = reinterpret_cast<int*>(small + DT_SMALL_COUNT);
    int* m_start = reinterpret_cast<int*>(small + DT_SMALL_START);
    int* m_row = reinterpret_cast<int*>(small + DT_SMALL_ROW);
    int* m_splits = reinterpret_cast<int*>(small + DT_SMALL_SPLITS);
    int64_t* m_first = reinterpret_cast<int64_t*>(small + DT_SMALL_FIRST);
    auto bar = [&](int which) { return bars + (uint32_t)which * 8u; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.q_heads / p.kv_heads;

    // -- setup ---------------------------------------------------------------------------------------------------------
    if (warp == 0) tmem_alloc(smem_addr(tmem_slot), DT_COLUMNS);
    if (tid == 32) {
        for (int s = 0; s < DT_STAGES; ++s) {
            mbar_init(bar(DT_KFULL + s), 1), mbar_init(bar(DT_KEMPTY + s), 1);
            mbar_init(bar(DT_VFULL + s), 1), mbar_init(bar(DT_VEMPTY + s), 1);
        }
        mbar_init(bar(DT_SFULL), 1), mbar_init(bar(DT_SFREE), 128);
        mbar_init(bar(DT_PFULL), 128), mbar_init(bar(DT_PVDONE), 1);
        mbar_init(bar(DT_QFULL), 32);
        mbar_init(bar(DT_FOLD_A), 128), mbar_init(bar(DT_FOLD_B), 128);
        *abort_flag = 0;
        mbar_init_fence();
    }
    for (int idx = tid; idx < DT_OPER / 16; idx += DT_THREADS) reinterpret_cast<uint4*>(pbuf)[idx] = make_uint4(0, 0, 0, 0);
    for (int rr = tid; rr < p.n_rows; rr += DT_THREADS) {
        int cnt = p.counts ? p.counts[rr] : p.columns;
        cnt = cnt > p.columns ? p.columns : (cnt < 0 ? 0 : cnt);
        const int64_t first = p.firsts[rr];
        m_count[rr] = cnt, m_start[rr] = p.starts[rr], m_row[rr] = p.rows[rr], m_first[rr] = first;
        m_splits[rr] = cnt > 0 ? (int)((first + cnt + p.chunk - 1) / p.chunk) : 0;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {            // the work list: a row has splits x kv heads units
        int carry = 0;
        for (int base = 0; base < p.n_rows; base += 32) {
            const int rr = base + lane;
            int scan = rr < p.n_rows ? m_splits[rr] * p.kv_heads : 0;
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
        // -- producer -------------------------------------------------------------------------------------------------
        // A unit's page ids (and its pages' scales) sit in registers, box 32 * j + lane of the unit in slot j of lane
        // `lane`; they are loaded one unit (the scales) and two units (the page ids) ahead, so no tile waits for a
        // lookup.  Lane b < 8 issues box b (16 positions) of a tile; a box past the row's end reads out of the tensor's
        // range, which the TMA fills with zeros.
        DtWalk w0, w1, w2;
        w0.begin(p, rows);
        w1 = w0, w1.next_unit(p, rows);
        w2 = w1, w2.next_unit(p, rows);
        auto fetch_pages = [&](const DtWalk& w, int (&pg)[DT_NB]) {
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) pg[j] = -1;
            if (!w.live) return;
            const int64_t end = w.u.begin + p.chunk < w.u.L ? w.u.begin + p.chunk : w.u.L;
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) {
                const int64_t pos0 = w.u.begin + (int64_t)(lane + 32 * j) * 16;
                if (pos0 < end) {
                    pg[j] = w.u.table[(uint32_t)(pos0 >> 4) / tpp];
                    if ((uint32_t)pg[j] >= pages_total) {       // outside the page tensor: read as past the end (zeros), reported
                        pg[j] = -1;
                        if (p.status) atomicExch(p.status, CRIT_B200_STATUS_BOUNDS);
                    }
                }
            }
        };
        auto fetch_scales = [&](const DtWalk& w, const int (&pg)[DT_NB], float (&ks)[DT_NB], float (&vs)[DT_NB]) {
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) {
                ks[j] = vs[j] = 1.f;
                if (smode == 2 && w.live && pg[j] >= 0) {
                    ks[j] = p.key_scales[(int64_t)pg[j] * p.kv_heads + w.u.h];
                    vs[j] = p.value_scales[(int64_t)pg[j] * p.kv_heads + w.u.h];
                }
            }
        };
        int pg0[DT_NB], pg1[DT_NB], pg2[DT_NB];
        float ks0[DT_NB], vs0[DT_NB], ks1[DT_NB], vs1[DT_NB];
        fetch_pages(w0, pg0);
        fetch_scales(w0, pg0, ks0, vs0);
        fetch_pages(w1, pg1);
        int t = 0;
        bool ok = true;
        while (w0.live && ok) {
            fetch_scales(w1, pg1, ks1, vs1);
            fetch_pages(w2, pg2);
            for (int i = 0; i < w0.u.ntiles; ++i, ++t) {
                int pgs = pg0[0];
                float kss = ks0[0], vss = vs0[0];
#pragma unroll
                for (int j = 1; j < DT_NB; ++j)
                    if ((i >> 2) == j) pgs = pg0[j], kss = ks0[j], vss = vs0[j];
                const int src = ((i & 3) << 3) + (lane & 7);
                const int pgb = __shfl_sync(FULLMASK, pgs, src);
                const float ksb = __shfl_sync(FULLMASK, kss, src), vsb = __shfl_sync(FULLMASK, vss, src);
                const uint32_t tile16 = (uint32_t)(w0.u.begin >> 4) + (uint32_t)(i * 8 + (lane & 7));
                const int slot0 = pgb >= 0 ? (int)((int64_t)pgb * p.page + ((tile16 % tpp) << 4)) : (int)p.slots;
                const int stage = t % DT_STAGES;
                const uint32_t free_parity = (uint32_t)((t / DT_STAGES) & 1) ^ 1u;
                unsigned char* st = stages + stage * DT_STAGE;
                ok = (dt_wait<100>(bar(DT_KEMPTY + stage), free_parity, abort_flag));
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(bar(DT_KFULL + stage), (uint32_t)DT_KV_BYTES);
                __syncwarp();
                if (lane < 8) tma_load_3d(smem_addr(st) + lane * 2048, &kmap, 0, w0.u.h, slot0, bar(DT_KFULL + stage));
                // the values, and with them the tile's scales (read by the softmax, which ends before the values are free)
                ok = (dt_wait<100>(bar(DT_VEMPTY + stage), free_parity, abort_flag));
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                float* scs = reinterpret_cast<float*>(st + 2 * DT_KV_BYTES);
                if (lane < 8) {
                    if (smode == 2) scs[lane] = ksb, scs[128 + lane] = vsb;
                    else if (smode == 1) reinterpret_cast<int*>(scs)[lane] = pgb >= 0 ? slot0 : -1;
                }
                __syncwarp();
                if (lane == 0) mbar_expect_tx(bar(DT_VFULL + stage), (uint32_t)DT_KV_BYTES);
                __syncwarp();
                if (lane < 8) tma_load_3d(smem_addr(st) + DT_KV_BYTES + lane * 2048, &vmap, 0, w0.u.h, slot0, bar(DT_VFULL + stage));
            }
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) pg0[j] = pg1[j], ks0[j] = ks1[j], vs0[j] = vs1[j], pg1[j] = pg2[j];
            w0 = w1, w1 = w2, w2.next_unit(p, rows);
        }
        if (!ok) {              // leaving early: the copies in flight land first (bounded)
            where = 0x410;
            for (int tt = t > DT_STAGES ? t - DT_STAGES : 0; tt <= t; ++tt) {
                mbar_wait(bar(DT_KFULL + tt % DT_STAGES), (uint32_t)(tt / DT_STAGES) & 1u, 20000000ull);
                if (tt < t) mbar_wait(bar(DT_VFULL + tt % DT_STAGES), (uint32_t)(tt / DT_STAGES) & 1u, 20000000ull);
            }
        }
    } else if (warp == 5) {
        // -- query preparation and MMA issue ------------------------------------------------------------------------------
        const uint32_t idesc_s = idesc_f8(false, 128, DT_N);
        const uint32_t idesc_o = idesc_f8(true, 128, DT_D);
        const float sl2 = p.scale * LOG2E * (smode == 0 ? p.key_multiplier : 1.f);
        const int qt = lane & 3;
        bool ok = true, have_prev = false, prev_acc = false;
        int prev_t = 0;
        auto issue_pv = [&]() {             // O (+)= P V of tile prev_t
            const int pstage = prev_t % DT_STAGES;
            ok = (dt_wait<32>(bar(DT_PFULL), (uint32_t)prev_t & 1u, abort_flag)) &&
                 dt_wait<32>(bar(DT_VFULL + pstage), (uint32_t)(prev_t / DT_STAGES) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) return;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t pa = smem_addr(pbuf), va = smem_addr(stages + pstage * DT_STAGE + DT_KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < DT_N / 32; ++kk)
                    umma_f8(tmem + DT_O, smem_desc_sw128(pa + kk * 32, 0, 1024), smem_desc_sw128(va + kk * 4096, 16, 1024),
                            idesc_o, prev_acc || kk > 0);
                umma_commit(bar(DT_VEMPTY + pstage));
                umma_commit(bar(DT_PVDONE));
            }
            __syncwarp();
        };
        // The unit's queries as the A operand: 4 lanes a row, 8 rows a pass.  Row r of the unit goes to TMEM lanes
        // 16 * lg + (r & 7) (hi) and + 8 (lo) of every lane group lg that serves its row group.  The global loads are
        // issued a unit ahead (load_q), the split and the stores happen at the unit's start (store_q).
        uint4 raw[NRG][4];
        auto load_q = [&](const DtWalk& wq) {
#pragma unroll
            for (int ps = 0; ps < NRG; ++ps) {
                const int r = ps * 8 + (lane >> 2);
                const int col = r / G, gq = r - col * G;
#pragma unroll
                for (int c = 0; c < 4; ++c) raw[ps][c] = make_uint4(0, 0, 0, 0);
                if (wq.live && col < wq.u.count) {
                    const char* src = (const char*)p.q + ((int64_t)(wq.u.start + col) * p.q_stride_token +
                                                          (int64_t)(wq.u.h * G + gq) * p.q_stride_head + qt * 32) * 2;
#pragma unroll
                    for (int c = 0; c < 4; ++c) raw[ps][c] = *reinterpret_cast<const uint4*>(src + c * 16);
                }
            }
        };
        auto store_q = [&](int k) {
#pragma unroll
            for (int ps = 0; ps < NRG; ++ps) {
                const int r = ps * 8 + (lane >> 2);
                float x[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t wds[4] = {raw[ps][c].x, raw[ps][c].y, raw[ps][c].z, raw[ps][c].w};
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
                // 2^e puts the row's largest magnitude in [128, 256)
                int e = 0;
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
#pragma unroll
                for (int rep = 0; rep < REPL; ++rep) {
                    const int row_hi = 16 * (rep * NRG + ps) + (r & 7), row_lo = row_hi + 8;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int chunk = 2 * qt + c;
                        *reinterpret_cast<uint4*>(qbuf + row_hi * 128 + ((chunk ^ (row_hi & 7)) << 4)) =
                            make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
                        *reinterpret_cast<uint4*>(qbuf + row_lo * 128 + ((chunk ^ (row_lo & 7)) << 4)) =
                            make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
                    }
                }
                if (qt == 0) qfac[(k & 1) * 32 + r] = down * sl2;
            }
            fence_proxy_async();
            mbar_arrive(bar(DT_QFULL));
            __syncwarp();
        };
        DtWalk w;
        w.begin(p, rows);
        load_q(w);
        int t = 0;
        while (w.live && ok) {
            const int stage = t % DT_STAGES;
            if (w.i == 0) {
                // A new unit.  The last unit's final second product goes first (its epilogue waits for it: by then every
                // softmax thread has read the last scores and has passed the wait for the last unit's queries, so the
                // barrier of the queries never runs two phases ahead of a waiter); then this unit's queries go over the
                // last one's, while the softmax warps are busy with that epilogue.
                if (have_prev) {
                    issue_pv();
                    have_prev = false;
                    if (!ok) break;
                }
                if (t > 0) {
                    ok = (dt_wait<32>(bar(DT_SFULL), (uint32_t)(t - 1) & 1u, abort_flag) &&
                                         dt_wait<32>(bar(DT_SFREE), (uint32_t)(t & 1) ^ 1u, abort_flag));
                    ok = __all_sync(FULLMASK, ok);
                    if (!ok) break;
                }
                store_q(w.k);
                {
                    DtWalk after = w;           // the next unit's queries start their way from global memory now
                    after.next_unit(p, rows);
                    load_q(after);
                }
            }
            ok = (dt_wait<32>(bar(DT_KFULL + stage), (uint32_t)(t / DT_STAGES) & 1u, abort_flag));
            ok = ok && (dt_wait<32>(bar(DT_SFREE), (uint32_t)(t & 1) ^ 1u, abort_flag));
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t qa = smem_addr(qbuf), ka = smem_addr(stages + stage * DT_STAGE);
#pragma unroll
                for (int kk = 0; kk < DT_D / 32; ++kk)
                    umma_f8(tmem, smem_desc_sw128(qa + kk * 32, 0, 1024), smem_desc_sw128(ka + kk * 32, 0, 1024), idesc_s, kk > 0);
                umma_commit(bar(DT_SFULL));
                umma_commit(bar(DT_KEMPTY + stage));
            }
            __syncwarp();
            if (have_prev) issue_pv();
            have_prev = true, prev_t = t, prev_acc = w.i > 0;
            w.next(p, rows);
            ++t;
        }
        if (ok && have_prev) issue_pv();
        if (!ok) where = 0x420;
    } else {
        // -- softmax: thread = TMEM lane 32 * warp + lane.  A lane group is 16 lanes: lanes 0-7 hold the hi terms of 8
        //    query rows, lanes 8-15 their lo terms; group lg serves query rows 8 * (lg % NRG) .. + 7 and owns columns
        //    [W * (lg / NRG), + W) of every tile.  The two lanes of a row share its columns: the hi lane takes the
        //    first half, the lo lane the second, after one exchange of scores ------------------------------------------
        const int lg = warp * 2 + (lane >> 4), rgi = lg % NRG, part = lg / NRG;
        const int jr = lane & 7;
        const bool second = (lane & 8) != 0;
        const int r = rgi * 8 + jr;
        const int col = r / G;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int prow = warp * 32 + lane;
        const int row_hi = prow & ~8, row_lo = row_hi | 8;
        const int cmine = part * W + (second ? CT : 0);           // this thread's first column of a tile
        const float vmul = smode == 0 ? p.value_multiplier : 1.f;
        const float lo_unscale = second ? 1.f / 16.f : 1.f;     // this lane's outputs: the lo probabilities were stored times 16
        const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
        float* fo = reinterpret_cast<float*>(pbuf);         // the unit's fold: [64 (lane group, row) entries][64] floats
        unsigned char* pb_hi = pbuf + row_hi * 128;
        unsigned char* pb_lo = pbuf + row_lo * 128;
        bool ok = true;
        DtWalk w;
        w.begin(p, rows);
        int t = 0;
        while (w.live && ok) {
            const int k = w.k;
            DtWalk after = w;                   // the unit after this one, found while this one's first scores are on their way
            after.next_unit(p, rows);
            ok = (dt_wait(bar(DT_QFULL), (uint32_t)k & 1u, abort_flag));
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            const float a_r = qfac[(k & 1) * 32 + r];
            const bool valid = col < w.u.count;
            const int lastpos = valid ? (int)(w.u.first + col) : -1;
            const int first32 = w.u.first > 0x7fffffffLL ? 0x7fffffff : (int)w.u.first;
            float m_run = -INFINITY, l_run = 0.f;
            for (int i = 0; i < w.u.ntiles; ++i, ++t) {
                const int stage = t % DT_STAGES;
                const int tile_pos = (int)w.u.begin + i * DT_N;
                ok = (dt_wait(bar(DT_SFULL), (uint32_t)t & 1u, abort_flag) &&
                                     dt_wait(bar(DT_VFULL + stage), (uint32_t)(t / DT_STAGES) & 1u, abort_flag));
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                tc_fence_after();
                if (tile_pos + DT_N > w.u.L && (w.u.L & 15)) {
                    // the row's last page is partly filled: its value rows past the last position hold whatever the
                    // page held before, and a probability of 0 times a NaN code would not be 0.  Zeros instead (the
                    // second product reads them after this thread's arrival on the P barrier, behind the proxy fence).
                    unsigned char* vst = stages + stage * DT_STAGE + DT_KV_BYTES;
                    const int from = (int)(w.u.L - tile_pos), to = (from + 15) & ~15;
                    for (int idx = tid; idx < (to - from) * 8; idx += 128)
                        *reinterpret_cast<uint4*>(vst + (from + (idx >> 3)) * 128 + ((idx & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                // this lane's scores of the group's W columns, then the exchange: each lane of a row ends with the sums
                // hi + lo of its own CT columns.  (tcgen05.ld wants its first column on a multiple of 32 here: 16 columns
                // are read as the half of 32.)
                float s[CT];
                {
                    float mine[W];
                    if constexpr (W == 16) {
                        float both[32];
                        tmem_ld32(tmem + lane_base + (uint32_t)((part >> 1) * 32), both);
#pragma unroll
                        for (int c = 0; c < 16; ++c) mine[c] = (part & 1) ? both[16 + c] : both[c];
                    } else {
#pragma unroll
                        for (int q = 0; q < W / 32; ++q) {
                            float part32[32];
                            tmem_ld32(tmem + lane_base + (uint32_t)(part * W + 32 * q), part32);
#pragma unroll
                            for (int c = 0; c < 32; ++c) mine[32 * q + c] = part32[c];
                        }
                    }
                    tc_fence_before();
                    mbar_arrive(bar(DT_SFREE));
#pragma unroll
                    for (int c = 0; c < CT; ++c) {
                        const float give = second ? mine[c] : mine[c + CT];
                        const float keep = second ? mine[c + CT] : mine[c];
                        s[c] = keep + __shfl_xor_sync(FULLMASK, give, 8);
                    }
                }
                const float* scs = reinterpret_cast<const float*>(stages + stage * DT_STAGE + 2 * DT_KV_BYTES);
                const bool mask = !valid || tile_pos + DT_N - 1 > first32;
                float mx0 = -INFINITY, mx1 = -INFINITY;
                float rvg[NGC];
#pragma unroll
                for (int g = 0; g < NGC; ++g) {
                    const int cb = cmine + g * GC;
                    float kf = a_r, lv = 0.f;
                    rvg[g] = 1.f;
                    if (smode == 2) {
                        const float vs = scs[128 + (cb >> 4)];
                        kf = a_r * scs[cb >> 4], lv = __log2f(vs), rvg[g] = __fdividef(1.f, vs);
                    }
                    // a scale per slot: read here from global memory, at the box's first slot the producer left
                    const int slot0 = smode == 1 ? reinterpret_cast<const int*>(scs)[cb >> 4] : -1;
#pragma unroll
                    for (int c = 0; c < GC; ++c) {
                        if (smode == 1) {
                            kf = a_r, lv = 0.f;
                            if (slot0 >= 0 && tile_pos + cb + c < w.u.L) {
                                const int64_t at = ((int64_t)slot0 + ((cb + c) & 15)) * p.kv_heads + w.u.h;
                                kf = a_r * p.key_scales[at], lv = __log2f(p.value_scales[at]);
                            }
                        }
                        float x = s[g * GC + c] * kf + lv;
                        if (mask && tile_pos + cb + c > lastpos) x = -INFINITY;
                        s[g * GC + c] = x;
                        if (c & 1) mx1 = fmaxf(mx1, x);
                        else mx0 = fmaxf(mx0, x);
                    }
                }
                float mx = fmaxf(mx0, mx1);
                mx = fmaxf(mx, __shfl_xor_sync(FULLMASK, mx, 8));           // the row's other half
                const bool moved = mx > m_run + DT_LAZY || m_run == -INFINITY;
                const float top = moved ? mx : m_run;
                const float sub = top == -INFINITY ? 0.f : top;
                const float alpha = moved ? ex2(m_run - sub) : 1.f;
                const bool rescale = moved && top != m_run && i > 0;
                m_run = top;

                // the P tile is free (and the outputs settled) once the second product of the tile before has landed
                ok = (dt_wait(bar(DT_PVDONE), (uint32_t)(t & 1) ^ 1u, abort_flag));
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                float l_tile = 0.f;
#pragma unroll
                for (int g = 0; g < NGC; ++g) {
                    const int cb = cmine + g * GC;
                    float psum = 0.f;
                    uint32_t wh[GC / 4], wl[GC / 4];
                    const int slot0 = smode == 1 ? reinterpret_cast<const int*>(scs)[cb >> 4] : -1;
#pragma unroll
                    for (int c2 = 0; c2 < GC / 2; ++c2) {
                        const float pa = ex2(s[g * GC + 2 * c2] - sub), pb = ex2(s[g * GC + 2 * c2 + 1] - sub);
                        if (smode == 1) {
                            float va = 1.f, vb = 1.f;
                            if (slot0 >= 0) {
                                const int64_t at = ((int64_t)slot0 + ((cb + 2 * c2) & 15)) * p.kv_heads + w.u.h;
                                if (tile_pos + cb + 2 * c2 < w.u.L) va = p.value_scales[at];
                                if (tile_pos + cb + 2 * c2 + 1 < w.u.L) vb = p.value_scales[at + p.kv_heads];
                            }
                            psum += __fdividef(pa, va) + __fdividef(pb, vb);
                        } else {
                            psum += pa + pb;
                        }
                        uint32_t h2, l2;
                        split_e4m3x2<16>(pa, pb, h2, l2);
                        if (c2 & 1) wh[c2 >> 1] |= h2 << 16, wl[c2 >> 1] |= l2 << 16;
                        else wh[c2 >> 1] = h2, wl[c2 >> 1] = l2;
                    }
                    l_tile += psum * rvg[g];
                    const int chunk = cb >> 4, within = cb & 15;
                    if constexpr (GC == 8) {
                        *reinterpret_cast<uint2*>(pb_hi + ((chunk ^ (row_hi & 7)) << 4) + within) = make_uint2(wh[0], wh[1]);
                        *reinterpret_cast<uint2*>(pb_lo + ((chunk ^ (row_lo & 7)) << 4) + within) = make_uint2(wl[0], wl[1]);
                    } else {
                        *reinterpret_cast<uint4*>(pb_hi + ((chunk ^ (row_hi & 7)) << 4)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                        *reinterpret_cast<uint4*>(pb_lo + ((chunk ^ (row_lo & 7)) << 4)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                    }
                }
                l_run = l_run * alpha + l_tile;

                if (__any_sync(FULLMASK, rescale)) {
                    // a maximum moved: the warp brings its output lanes to the new reference
                    tc_fence_after();
                    dt_rescale(tmem + lane_base + DT_O, alpha);
                }
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(bar(DT_PFULL));
            }
            if (!ok) break;

            // -- the unit's result: wait for its last second product, fold the replicas, write ------------------------------
            const int tl = t - 1;
            ok = (dt_wait(bar(DT_PVDONE), (uint32_t)tl & 1u, abort_flag));
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            // hi + lo of the outputs: the hi lane keeps value columns 0..63, the lo lane 64..127
            float keep[64];
#pragma unroll
            for (int c4 = 0; c4 < 2; ++c4) {
                float oa[32], ob[32];
                tmem_ld32(tmem + lane_base + DT_O + 32u * c4, oa);
                tmem_ld32(tmem + lane_base + DT_O + 64u + 32u * c4, ob);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float give = (second ? oa[j] : ob[j]) * lo_unscale;
                    const float mine = (second ? ob[j] : oa[j]) * lo_unscale;
                    keep[32 * c4 + j] = mine + __shfl_xor_sync(FULLMASK, give, 8);
                }
            }
            tc_fence_before();
            const int entry = lg * 8 + jr, swz = entry & 15;
            {
                const float l_row = l_run + __shfl_xor_sync(FULLMASK, l_run, 8);
                if (!second) fm[entry] = m_run, fl[entry] = l_row;
            }
            const bool whole = w.u.nsplit == 1 && !(p.flags & CRIT_B200_ATTEND_PARTIALS);
            const int prow_first = p.offsets ? p.offsets[w.u.r] - p.offsets[0] : w.u.r * p.columns;
            const bool fits = whole || (p.workspace && w.u.split < p.max_splits && prow_first >= 0 && prow_first + w.u.count <= p.partial_rows);
            if (!fits && tid == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_PLAN);
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {          // value columns 0..63, then 64..127
                if ((int)second == pass) {
#pragma unroll
                    for (int f4 = 0; f4 < 16; ++f4)
                        *reinterpret_cast<float4*>(fo + entry * 64 + ((f4 ^ swz) << 2)) =
                            make_float4(keep[4 * f4], keep[4 * f4 + 1], keep[4 * f4 + 2], keep[4 * f4 + 3]);
                }
                mbar_arrive(bar(DT_FOLD_A));
                ok = (dt_wait(bar(DT_FOLD_A), (uint32_t)pass, abort_flag));
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
#pragma unroll
                for (int it = 0; it < R / 8; ++it) {
                    const int idx = tid + 128 * it;
                    const int rr = idx >> 4, f = idx & 15;
                    const int rgx = rr >> 3, jx = rr & 7;
                    const int colx = rr / G, gqx = rr - colx * G;
                    if (colx < w.u.count) {
                        float top = -INFINITY;
#pragma unroll
                        for (int pt = 0; pt < REPL; ++pt) top = fmaxf(top, fm[(pt * NRG + rgx) * 8 + jx]);
                        const float sub = top == -INFINITY ? 0.f : top;
                        float l = 0.f;
                        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int pt = 0; pt < REPL; ++pt) {
                            const int e = (pt * NRG + rgx) * 8 + jx;
                            const float fac = ex2(fm[e] - sub);
                            l += fl[e] * fac;
                            const float4 v = *reinterpret_cast<const float4*>(fo + e * 64 + ((f ^ (e & 15)) << 2));
                            o.x += v.x * fac, o.y += v.y * fac, o.z += v.z * fac, o.w += v.w * fac;
                        }
                        o.x *= vmul, o.y *= vmul, o.z *= vmul, o.w *= vmul;
                        const int token = w.u.start + colx, head = w.u.h * G + gqx, dv = pass * 64 + f * 4;
                        if (whole) {
                            const float inv = l > 0.f ? 1.f / l : 0.f;
                            char* dst = (char*)p.out + ((int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head + dv) * 2;
                            uint2 packed;
                            if (p.q_dtype == CRIT_B200_DTYPE_BF16) {
                                packed.x = pack2<true>(o.x * inv, o.y * inv), packed.y = pack2<true>(o.z * inv, o.w * inv);
                            } else {
                                packed.x = pack2<false>(o.x * inv, o.y * inv), packed.y = pack2<false>(o.z * inv, o.w * inv);
                            }
                            *reinterpret_cast<uint2*>(dst) = packed;
                            if (p.lse && dv == 0) p.lse[(int64_t)token * p.q_heads + head] = l > 0.f ? top * LN2 + logf(l) : -INFINITY;
                        } else if (fits) {
                            const int prow_ws = prow_first + colx;
                            const int64_t at = ((int64_t)prow_ws * p.q_heads + head) * p.max_splits + w.u.split;
                            *reinterpret_cast<float4*>(p.workspace + at * DT_D + dv) = o;
                            if (dv == 0) {
                                p.workspace[states * DT_D + at] = top;
                                p.workspace[states * (DT_D + 1) + at] = l;
                            }
                        }
                    }
                }
                mbar_arrive(bar(DT_FOLD_B));
                ok = (dt_wait(bar(DT_FOLD_B), (uint32_t)pass, abort_flag));
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
            }
            if (!ok) break;
            // the fold used the P tile: this thread's row back to zeros (the columns it never writes stay zero)
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(pbuf + prow * 128 + c * 16) = make_uint4(0, 0, 0, 0);
            __syncwarp();               // a row's other lane writes into this row too
            w = after;
        }
        if (!ok) where = 0x440;
    }

    if (where && p.status) atomicExch(p.status, where);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, DT_COLUMNS);
}

}  // namespace crit_b200
