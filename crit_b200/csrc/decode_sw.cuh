// Split-K decode / speculative-verify attention over E4M3 pages on the fifth-generation tensor cores, with the operands
// swapped so that the bytes streamed from HBM fill the MMA's 128 rows:
//
//     S^T [128 positions x N]  = K [128 positions x 128]  . Q^T [128 x N]         (A = the key tile as TMA left it)
//     O^T [128 values    x N] += V^T [128 values x 128 positions] . P^T [128 positions x N]   (A = the value tile, MN-major)
//
// N = 2 x the unit's query rows (a row's 16-bit query, and later its probabilities, enter as two E4M3 terms hi + lo, in
// columns r and NR + r; NR = 8, 16 or 32 rows: columns x heads of a kv head's group).  Against decode_tc.cuh, which puts
// the few query rows on the 128-row side and fills it with replicas, this form has no replica to fold and no padding to
// multiply: a tile costs 8 MMAs of N = 16..64 instead of N = 128, and the softmax threads each own one POSITION of the
// tile (a TMEM lane), so a thread's page scale, value scale and causal mask are scalars.
//
// A softmax thread never reduces across positions inside the loop.  The row maxima are references, equal in all 128
// threads, that move lazily: a tile's scores are compared with reference + 8 and the 128 threads vote (one barrier with an
// OR, bounded like every wait here); only when some score passes (the unit's first tile, and rarely later) the block takes the row maxima exactly
// (redux over the warps, shared memory across them) and rescales.  The row sums stay per thread until the unit's end.
// Probabilities go to shared memory as E4M3 bytes, one byte a (row, position), into the K-major B operand of the second
// product; the values' scales enter the scores as an exponent offset, as in decode_tc.cuh.
//
// Block: 4 softmax warps (thread = TMEM lane = position of the tile, later = value column of the output), a producer warp
// (TMA boxes of [16 positions][1 kv head][128 bytes], the unit's page ids and scales in registers a unit ahead) and a warp
// that prepares the unit's queries and issues the MMAs.  Two persistent blocks an SM walk the work list of
// decode_tc.cuh (unit = window row, split, kv head).  Every wait is bounded and polls the block's abort flag.
//
// HBM traffic per unit: its keys and values once, 8 scale floats per page, the queries, one partial state.
// Reference: paged_kv_attention/_kernels.py:263-478 (_partition, _window_kernel), cuda_window.cu:284-1065 (cw_tile).
#pragma once

#include "decode_tc.cuh"

namespace crit_b200 {

constexpr int SW_THREADS = 192;
constexpr int SW_MAX_LIST = 128;            // window rows a launch lists its work for
constexpr uint32_t SW_COLUMNS = 256;        // TMEM: scores buffer 0 at 0, buffer 1 at 64, outputs at 128 (up to 64 each)
constexpr uint32_t SW_S1 = 64, SW_O = 128;

// shared memory (after the 1 KB alignment): Q^T x 2 (N rows of 128 bytes, by the unit's parity) | P^T x 2 (the same, by the
// tile's parity) | stages | small.
// A decode unit (8 rows) has small operands and takes three stages; the wider ones two: two blocks an SM either way.
template <int NR>
struct SwCfg {
    static constexpr int N = 2 * NR;
    static constexpr int OPER = N * 128;
    static constexpr int STAGES = NR == 8 ? 3 : 2;
    static constexpr int OFF_Q = 0, OFF_P = 2 * OPER, OFF_STAGES = 4 * OPER;
    static constexpr int OFF_SMALL = OFF_STAGES + STAGES * DT_STAGE;
    static constexpr int SMALL_QFAC = 0;                             // [2][32] floats: the rows' score factors, by the unit's parity
    static constexpr int SMALL_MREF = 256;                           // [2][32] floats: the rows' references, current and last
    static constexpr int SMALL_ROWMAX = 512;                         // [4 warps][32] floats: a tile's row maxima; the unit's row sums
    static constexpr int SMALL_BARS = 1024;                          // 24 mbarriers
    static constexpr int SMALL_TMEM = SMALL_BARS + 24 * 8;
    static constexpr int SMALL_ABORT = SMALL_TMEM + 4;
    static constexpr int SMALL_VOTES = SMALL_ABORT + 4;              // three ints: the softmax threads' votes, by the tile modulo 3
    static constexpr int SMALL_LIST = 1280;                          // unit_first [SW_MAX_LIST + 1] ints (padded)
    static constexpr int SMALL_COUNT = SMALL_LIST + (SW_MAX_LIST + 4) * 4;
    static constexpr int SMALL_START = SMALL_COUNT + SW_MAX_LIST * 4;
    static constexpr int SMALL_ROW = SMALL_START + SW_MAX_LIST * 4;
    static constexpr int SMALL_SPLITS = SMALL_ROW + SW_MAX_LIST * 4;
    static constexpr int SMALL_FIRST = SMALL_SPLITS + SW_MAX_LIST * 4;
    static constexpr int SMEM = 1024 + OFF_SMALL + SMALL_FIRST + SW_MAX_LIST * 8;
};

// mbarriers: stage s of keys / values full and empty; scores buffer b full / free; P^T buffer b full / its second product
// done; the queries of an even / odd unit; the softmax threads' vote and meeting
enum { SW_KFULL = 0, SW_VFULL = 3, SW_KEMPTY = 6, SW_VEMPTY = 9, SW_SFULL = 12, SW_SFREE = 14, SW_PFULL = 16, SW_PVDONE = 18,
       SW_QFULL = 20, SW_VOTE = 22, SW_MEET = 23 };

// kind::f8f6f4 instruction descriptor, E4M3 x E4M3 -> F32, with either operand K-major (0) or MN-major (1).
__device__ __forceinline__ uint32_t idesc_f8_majors(bool a_mn_major, bool b_mn_major, int M, int N) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= (a_mn_major ? 1u : 0u) << 15;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}

// 16 consecutive FP32 columns of this thread's TMEM lane (taddr on a multiple of 32 columns, or 16 past one).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// N consecutive columns (N = 16, 32 or 64) of this thread's lane.
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, float (&v)[N]) {
    if constexpr (N == 16) {
        tmem_ld16(taddr, v);
    } else {
#pragma unroll
        for (int q = 0; q < N / 32; ++q) {
            float part[32];
            tmem_ld32(taddr + 32u * q, part);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[32 * q + i] = part[i];
        }
    }
}

// The largest of a float over the warp, in one redux (on an order-preserving integer image of the float).
__device__ __forceinline__ float warp_max_redux(float x) {
    int key = __float_as_int(x);
    key = key >= 0 ? key : key ^ 0x7fffffff;
    int top;
    asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(top) : "r"(key));
    top = top >= 0 ? top : top ^ 0x7fffffff;
    return __int_as_float(top);
}

// NR: query rows a unit holds (8, 16 or 32).  SMODE as in decode_tc.cuh (0 static multipliers, 1 a scale per (slot, kv
// head), 2 a scale per (page, kv head)).
template <int NR, int SMODE>
__global__ void __launch_bounds__(SW_THREADS, 2)
decode_sw_kernel(const crit_b200_attend_params p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    using C = SwCfg<NR>;
    constexpr int smode = SMODE;
    constexpr int N = C::N;                   // MMA columns: the hi terms of the rows, then the lo terms
    constexpr int SW_STAGES = C::STAGES;
    constexpr uint32_t FULLMASK = 0xffffffffu;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024 - (smem_addr(smem_raw) & 1023)) & 1023);
    unsigned char* qbuf = smem + C::OFF_Q;
    unsigned char* pbufs = smem + C::OFF_P;
    unsigned char* stages = smem + C::OFF_STAGES;
    unsigned char* small = smem + C::OFF_SMALL;
    float* qfac = reinterpret_cast<float*>(small + C::SMALL_QFAC);
    float* mref = reinterpret_cast<float*>(small + C::SMALL_MREF);
    float* rowmax = reinterpret_cast<float*>(small + C::SMALL_ROWMAX);
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
    if (warp == 0) tmem_alloc(smem_addr(tmem_slot), SW_COLUMNS);
    if (tid == 32) {
        for (int s = 0; s < SW_STAGES; ++s) {
            mbar_init(bar(SW_KFULL + s), 1), mbar_init(bar(SW_KEMPTY + s), 1);
            mbar_init(bar(SW_VFULL + s), 1), mbar_init(bar(SW_VEMPTY + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(SW_SFULL + b), 1), mbar_init(bar(SW_SFREE + b), 128);
            mbar_init(bar(SW_PFULL + b), 128), mbar_init(bar(SW_PVDONE + b), 1);
        }
        mbar_init(bar(SW_QFULL), 32), mbar_init(bar(SW_QFULL + 1), 32);
        mbar_init(bar(SW_VOTE), 128), mbar_init(bar(SW_MEET), 128);
        *abort_flag = 0;
        for (int v = 0; v < 3; ++v) reinterpret_cast<volatile int*>(small + C::SMALL_VOTES)[v] = 0;
        mbar_init_fence();
    }
    if (tid < 32) mref[tid] = -INFINITY;
    for (int idx = tid; idx < 4 * C::OPER / 16; idx += SW_THREADS) reinterpret_cast<uint4*>(qbuf)[idx] = make_uint4(0, 0, 0, 0);
    for (int rr = tid; rr < p.n_rows; rr += SW_THREADS) {
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
        // -- producer: as decode_tc.cuh's (a unit's page ids and page scales in registers, a unit and two ahead) ----------
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
                const int stage = t % SW_STAGES;
                const uint32_t free_parity = (uint32_t)((t / SW_STAGES) & 1) ^ 1u;
                unsigned char* st = stages + stage * DT_STAGE;
                ok = dt_wait<100>(bar(SW_KEMPTY + stage), free_parity, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(bar(SW_KFULL + stage), (uint32_t)DT_KV_BYTES);
                __syncwarp();
                if (lane < 8) tma_load_3d(smem_addr(st) + lane * 2048, &kmap, 0, w0.u.h, slot0, bar(SW_KFULL + stage));
                ok = dt_wait<100>(bar(SW_VEMPTY + stage), free_parity, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                float* scs = reinterpret_cast<float*>(st + 2 * DT_KV_BYTES);
                if (lane < 8) {
                    if (smode == 2) scs[lane] = ksb, scs[128 + lane] = vsb;
                    else if (smode == 1) reinterpret_cast<int*>(scs)[lane] = pgb >= 0 ? slot0 : -1;
                }
                __syncwarp();
                if (lane == 0) mbar_expect_tx(bar(SW_VFULL + stage), (uint32_t)DT_KV_BYTES);
                __syncwarp();
                if (lane < 8) tma_load_3d(smem_addr(st) + DT_KV_BYTES + lane * 2048, &vmap, 0, w0.u.h, slot0, bar(SW_VFULL + stage));
            }
#pragma unroll
            for (int j = 0; j < DT_NB; ++j) pg0[j] = pg1[j], ks0[j] = ks1[j], vs0[j] = vs1[j], pg1[j] = pg2[j];
            w0 = w1, w1 = w2, w2.next_unit(p, rows);
        }
        if (!ok) {              // leaving early: the copies in flight land first (bounded)
            where = 0x510;
            for (int tt = t > SW_STAGES ? t - SW_STAGES : 0; tt <= t; ++tt) {
                mbar_wait(bar(SW_KFULL + tt % SW_STAGES), (uint32_t)(tt / SW_STAGES) & 1u, 20000000ull);
                if (tt < t) mbar_wait(bar(SW_VFULL + tt % SW_STAGES), (uint32_t)(tt / SW_STAGES) & 1u, 20000000ull);
            }
        }
    } else if (warp == 5) {
        // -- query preparation and MMA issue ------------------------------------------------------------------------------
        const uint32_t idesc_s = idesc_f8_majors(false, false, 128, N);       // S^T = K Q^T: both K-major
        const uint32_t idesc_o = idesc_f8_majors(true, false, 128, N);        // O^T += V^T P^T: the values MN-major
        const float sl2 = p.scale * LOG2E * (smode == 0 ? p.key_multiplier : 1.f);
        const int qt = lane & 3;
        bool ok = true, have_prev = false, prev_acc = false;
        int prev_t = 0;
        auto issue_pv = [&]() {             // O^T (+)= V^T P^T of tile prev_t
            const int pstage = prev_t % SW_STAGES, pb = prev_t & 1;
            ok = dt_wait<32>(bar(SW_PFULL + pb), (uint32_t)(prev_t >> 1) & 1u, abort_flag) &&
                 dt_wait<32>(bar(SW_VFULL + pstage), (uint32_t)(prev_t / SW_STAGES) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) return;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t pa = smem_addr(pbufs + pb * C::OPER), va = smem_addr(stages + pstage * DT_STAGE + DT_KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < DT_N / 32; ++kk)
                    umma_f8(tmem + SW_O, smem_desc_sw128(va + kk * 4096, 16, 1024), smem_desc_sw128(pa + kk * 32, 0, 1024), idesc_o,
                            prev_acc || kk > 0);
                umma_commit(bar(SW_VEMPTY + pstage));
                umma_commit(bar(SW_PVDONE + pb));
            }
            __syncwarp();
        };
        // The unit's queries as the B operand Q^T: row r of the unit's NR rows gives tile row r (hi) and NR + r (lo),
        // 128 bytes each with the 128-byte swizzle; 4 lanes a row, 8 rows a pass.  Loaded a unit ahead.
        uint4 raw[NR / 8][4];
        auto load_q = [&](const DtWalk& wq) {
#pragma unroll
            for (int ps = 0; ps < NR / 8; ++ps) {
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
            unsigned char* qdst = qbuf + (k & 1) * C::OPER;
#pragma unroll
            for (int ps = 0; ps < NR / 8; ++ps) {
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
                const int row_hi = r, row_lo = NR + r;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int chunk = 2 * qt + c;
                    *reinterpret_cast<uint4*>(qdst + row_hi * 128 + ((chunk ^ (row_hi & 7)) << 4)) =
                        make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
                    *reinterpret_cast<uint4*>(qdst + row_lo * 128 + ((chunk ^ (row_lo & 7)) << 4)) =
                        make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
                }
                if (qt == 0) qfac[(k & 1) * 32 + r] = down * sl2;
            }
            fence_proxy_async();
            mbar_arrive(bar(SW_QFULL + (k & 1)));
            __syncwarp();
        };
        // The queries run a unit ahead of the products: unit k's sit in buffer k & 1 when its first product is issued, and
        // unit k + 1's are written over unit k - 1's right after unit k's first tile is under way (by then the second
        // product of unit k - 1's last tile has been issued, which waited for its probabilities: every product that read
        // that buffer has completed and the softmax threads are done with its factors); unit k + 2's leave global memory.
        DtWalk w, ahead;
        w.begin(p, rows);
        load_q(w);
        if (w.live) store_q(0);
        ahead = w, ahead.next_unit(p, rows);
        load_q(ahead);
        int t = 0;
        while (w.live && ok) {
            const int stage = t % SW_STAGES, sb = t & 1;
            ok = dt_wait<32>(bar(SW_KFULL + stage), (uint32_t)(t / SW_STAGES) & 1u, abort_flag) &&
                 dt_wait<32>(bar(SW_SFREE + sb), (uint32_t)((t >> 1) & 1) ^ 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t qa = smem_addr(qbuf + (w.k & 1) * C::OPER), ka = smem_addr(stages + stage * DT_STAGE);
#pragma unroll
                for (int kk = 0; kk < DT_D / 32; ++kk)
                    umma_f8(tmem + (sb ? SW_S1 : 0u), smem_desc_sw128(ka + kk * 32, 0, 1024), smem_desc_sw128(qa + kk * 32, 0, 1024),
                            idesc_s, kk > 0);
                umma_commit(bar(SW_SFULL + sb));
                umma_commit(bar(SW_KEMPTY + stage));
            }
            __syncwarp();
            if (have_prev) issue_pv();
            if (!ok) break;
            if (w.i == 0) {
                if (ahead.live) store_q(ahead.k);
                ahead.next_unit(p, rows);
                load_q(ahead);
            }
            have_prev = true, prev_t = t, prev_acc = w.i > 0;
            w.next(p, rows);
            ++t;
        }
        if (ok && have_prev) issue_pv();
        if (!ok) where = 0x520;
    } else {
        // -- softmax: thread = position 32 * warp + lane of the tile (a TMEM lane of the scores), later value column
        //    32 * warp + lane of the outputs ---------------------------------------------------------------------------
        const int pos_in_tile = warp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float vmul = smode == 0 ? p.value_multiplier : 1.f;
        const int64_t states = (int64_t)p.partial_rows * p.q_heads * p.max_splits;
        const int box = pos_in_tile >> 4;
        // this thread's byte of row n of a P^T tile: rows of 128 bytes, the 16-byte chunks swizzled by the row
        const int pchunk = pos_in_tile >> 4, pwithin = pos_in_tile & 15;
        bool ok = true;
        // The 128 softmax threads meet on mbarriers (every wait bounded, as all waits here): vote() ORs a predicate over
        // them through a flag in shared memory (three flags in turn: the one of tile t + 2 is cleared after tile t's
        // meeting, which nobody can have passed twice over), meet() is a plain meeting.
        volatile int* votes = reinterpret_cast<volatile int*>(small + C::SMALL_VOTES);
        uint32_t n_vote = 0, n_meet = 0;
        auto vote = [&](bool mine, int tile) -> int {
            if (mine) votes[tile % 3] = 1;
            mbar_arrive(bar(SW_VOTE));
            if (!dt_wait(bar(SW_VOTE), n_vote++ & 1u, abort_flag)) return -1;
            const int any = votes[tile % 3];
            if (tid == 0) votes[(tile + 2) % 3] = 0;
            return any;
        };
        auto meet = [&]() -> bool {
            mbar_arrive(bar(SW_MEET));
            return dt_wait(bar(SW_MEET), n_meet++ & 1u, abort_flag);
        };
        // the scores of this thread's position: the queries' hi and lo terms added, N / 2 rows at a time
        auto load_scores = [&](uint32_t taddr, float (&s)[NR]) {
            if constexpr (NR == 8) {
                float raw[16];
                tmem_ld16(taddr, raw);
#pragma unroll
                for (int r = 0; r < 8; ++r) s[r] = raw[r] + raw[8 + r];
            } else if constexpr (NR == 16) {
                float raw[32];
                tmem_ld32(taddr, raw);
#pragma unroll
                for (int r = 0; r < 16; ++r) s[r] = raw[r] + raw[16 + r];
            } else {
                tmem_ld32(taddr, s);
                float lo[32];
                tmem_ld32(taddr + 32u, lo);
#pragma unroll
                for (int r = 0; r < 32; ++r) s[r] += lo[r];
            }
        };
        DtWalk w;
        w.begin(p, rows);
        int t = 0;
        int mb = 0;             // which of the two reference arrays is current (every thread toggles it at the same points)
        while (w.live && ok) {
            const int k = w.k;
            DtWalk after = w;
            after.next_unit(p, rows);
            const int prow_first = p.offsets ? p.offsets[w.u.r] - p.offsets[0] : w.u.r * p.columns;
            ok = dt_wait(bar(SW_QFULL + (k & 1)), (uint32_t)(k >> 1) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            const int rows_live = w.u.count * G;                 // the unit's query rows (row r: column r / G)
            const int first32 = w.u.first > 0x7fffffffLL ? 0x7fffffff : (int)w.u.first;
            const float* a_r = qfac + (k & 1) * 32;              // the rows' score factors (the same for every thread)
            float l_part[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) l_part[r] = 0.f;
            // (the rows' references are -inf here: every thread wrote them so itself, at the launch's or the last unit's end)
            for (int i = 0; i < w.u.ntiles; ++i, ++t) {
                const int stage = t % SW_STAGES, sb = t & 1, pb = t & 1;
                const int tile_pos = (int)w.u.begin + i * DT_N;
                const int pos = tile_pos + pos_in_tile;
                ok = dt_wait(bar(SW_SFULL + sb), (uint32_t)(t >> 1) & 1u, abort_flag) &&
                     dt_wait(bar(SW_VFULL + stage), (uint32_t)(t / SW_STAGES) & 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                tc_fence_after();
                unsigned char* st = stages + stage * DT_STAGE;
                if (tile_pos + DT_N > w.u.L && (w.u.L & 15)) {
                    // the row's last page is partly filled: value rows past the last position become zeros (a probability
                    // of 0 times a stale NaN code would not be 0); read by the second product behind the proxy fence below
                    unsigned char* vst = st + DT_KV_BYTES;
                    const int from = (int)(w.u.L - tile_pos), to = (from + 15) & ~15;
                    for (int idx = tid; idx < (to - from) * 8; idx += 128)
                        *reinterpret_cast<uint4*>(vst + (from + (idx >> 3)) * 128 + ((idx & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                float s[NR];
                load_scores(tmem + lane_base + (sb ? SW_S1 : 0u), s);
                tc_fence_before();
                mbar_arrive(bar(SW_SFREE + sb));
                // this position's scales: the scores' factor, the values' exponent offset and its inverse for the row sums
                const float* scs = reinterpret_cast<const float*>(st + 2 * DT_KV_BYTES);
                float kf = 1.f, lv = 0.f, rv = 1.f;
                if (smode == 2) {
                    const float vs = scs[128 + box];
                    kf = scs[box], lv = __log2f(vs), rv = __fdividef(1.f, vs);
                } else if (smode == 1) {
                    const int slot0 = reinterpret_cast<const int*>(scs)[box];
                    if (slot0 >= 0 && pos < w.u.L) {
                        const int64_t at = ((int64_t)slot0 + (pos_in_tile & 15)) * p.kv_heads + w.u.h;
                        const float vs = p.value_scales[at];
                        kf = p.key_scales[at], lv = __log2f(vs), rv = __fdividef(1.f, vs);
                    }
                }
                const bool edge = tile_pos + DT_N - 1 > first32 || rows_live < NR;
                bool passes = false;
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    float x = s[r] * (a_r[r] * kf) + lv;
                    if (edge && (r >= rows_live || pos > first32 + r / G)) x = -INFINITY;
                    s[r] = x;
                    passes |= x > mref[mb * 32 + r] + DT_LAZY;
                }
                const int voted = vote(passes, t);
                ok = __all_sync(FULLMASK, voted >= 0);
                if (!ok) break;
                if (voted) {
                    // some score passed its row's reference by 2^8 (or the unit starts): the rows' maxima exactly, over the
                    // block; the references, the sums and the outputs follow the rows that moved.  Every thread works the
                    // new references out itself and writes them, all the same, to the array that is not current (last read
                    // before the vote above), so one meeting serves
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        const float top = warp_max_redux(s[r]);
                        if (lane == 0) rowmax[warp * 32 + r] = top;
                    }
                    ok = __all_sync(FULLMASK, meet());
                    if (!ok) break;
                    bool moved = false;
                    float alpha[NR];
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        const float old = mref[mb * 32 + r];
                        const float top = fmaxf(fmaxf(rowmax[r], rowmax[32 + r]), fmaxf(rowmax[64 + r], rowmax[96 + r]));
                        const bool go = top > old + DT_LAZY || (old == -INFINITY && top > -INFINITY);
                        alpha[r] = go && old > -INFINITY ? ex2(old - top) : 1.f;
                        moved |= alpha[r] != 1.f;
                        l_part[r] *= alpha[r];
                        mref[(mb ^ 1) * 32 + r] = go ? top : old;
                    }
                    mb ^= 1;
                    if (moved && i > 0) {
                        // every second product so far has landed; O^T: lane = value column, column j = row j (hi) or j - NR (lo)
                        ok = dt_wait(bar(SW_PVDONE + ((t - 1) & 1)), (uint32_t)((t - 1) >> 1) & 1u, abort_flag);
                        ok = __all_sync(FULLMASK, ok);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            if constexpr (NR == 8) {
                                if (half == 1) break;
                                float o[16];
                                tmem_ld16(tmem + lane_base + SW_O, o);
#pragma unroll
                                for (int r = 0; r < 8; ++r) o[r] *= alpha[r], o[8 + r] *= alpha[r];
                                tmem_st16(tmem + lane_base + SW_O, o);
                            } else if constexpr (NR == 16) {
                                if (half == 1) break;
                                float o[32];
                                tmem_ld32(tmem + lane_base + SW_O, o);
#pragma unroll
                                for (int r = 0; r < 16; ++r) o[r] *= alpha[r], o[16 + r] *= alpha[r];
                                tmem_st32(tmem + lane_base + SW_O, o);
                            } else {
                                float o[32];
                                tmem_ld32(tmem + lane_base + SW_O + 32u * half, o);
#pragma unroll
                                for (int r = 0; r < 32; ++r) o[r] *= alpha[r];
                                tmem_st32(tmem + lane_base + SW_O + 32u * half, o);
                            }
                        }
                        tc_fence_before();
                    }
                }
                // this tile's P^T buffer is free once the second product of the tile two before has landed
                ok = dt_wait(bar(SW_PVDONE + pb), (uint32_t)((t >> 1) & 1) ^ 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                // probabilities: p' = 2^(x - reference) <= 2^8, two E4M3 terms (the lo term times 16), one byte a (row,
                // position) into the P^T tile; the row sums take p' / vs
                unsigned char* pbuf = pbufs + pb * C::OPER;
#pragma unroll
                for (int r2 = 0; r2 < NR / 2; ++r2) {
                    const int ra = 2 * r2, rb = ra + 1;
                    const float ma = mref[mb * 32 + ra], mbr = mref[mb * 32 + rb];
                    const float pa = ex2(s[ra] - (ma == -INFINITY ? 0.f : ma));
                    const float pbv = ex2(s[rb] - (mbr == -INFINITY ? 0.f : mbr));
                    l_part[ra] += pa * rv, l_part[rb] += pbv * rv;
                    uint32_t h2, l2;
                    split_e4m3x2<16>(pa, pbv, h2, l2);
                    pbuf[ra * 128 + ((pchunk ^ (ra & 7)) << 4) + pwithin] = (unsigned char)(h2 & 0xffu);
                    pbuf[rb * 128 + ((pchunk ^ (rb & 7)) << 4) + pwithin] = (unsigned char)(h2 >> 8);
                    pbuf[(NR + ra) * 128 + ((pchunk ^ ((NR + ra) & 7)) << 4) + pwithin] = (unsigned char)(l2 & 0xffu);
                    pbuf[(NR + rb) * 128 + ((pchunk ^ ((NR + rb) & 7)) << 4) + pwithin] = (unsigned char)(l2 >> 8);
                }
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(bar(SW_PFULL + pb));
            }
            if (!ok) break;

            // -- the unit's result: its last second product, the row sums over the block, one store a (row, value column) ---
            const int tl = t - 1;
            ok = dt_wait(bar(SW_PVDONE + (tl & 1)), (uint32_t)(tl >> 1) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                float v = l_part[r];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(FULLMASK, v, off);
                if (lane == 0) rowmax[warp * 32 + r] = v;
            }
            ok = __all_sync(FULLMASK, meet());
            if (!ok) break;
            const bool whole = w.u.nsplit == 1 && !(p.flags & CRIT_B200_ATTEND_PARTIALS);
            const bool fits = whole || (p.workspace && w.u.split < p.max_splits && prow_first >= 0 && prow_first + w.u.count <= p.partial_rows);
            if (!fits && tid == 0 && p.status) atomicExch(p.status, CRIT_B200_STATUS_PLAN);
            const int dv = pos_in_tile;             // this thread's value column
            tc_fence_after();
            {
                // hi and lo terms of NR rows: loaded 32 columns at a time at the most
                constexpr int STEP = NR < 16 ? NR : 16;             // rows a pass
#pragma unroll
                for (int r0 = 0; r0 < NR; r0 += STEP) {
                    float hi[STEP], lo[STEP];
                    if constexpr (STEP == 8) {
                        float both[16];
                        tmem_ld16(tmem + lane_base + SW_O, both);
#pragma unroll
                        for (int r = 0; r < 8; ++r) hi[r] = both[r], lo[r] = both[8 + r];
                    } else {
                        tmem_ld16(tmem + lane_base + SW_O + (uint32_t)r0, hi);
                        tmem_ld16(tmem + lane_base + SW_O + (uint32_t)(NR + r0), lo);
                    }
#pragma unroll
                    for (int rr = 0; rr < STEP; ++rr) {
                        const int r = r0 + rr;
                        if (r >= rows_live) continue;
                        const int colx = r / G, gqx = r - colx * G;
                        const int token = w.u.start + colx, head = w.u.h * G + gqx;
                        const float value = (hi[rr] + lo[rr] * (1.f / 16.f)) * vmul;
                        const float l = (rowmax[r] + rowmax[32 + r]) + (rowmax[64 + r] + rowmax[96 + r]);
                        const float top = mref[mb * 32 + r];
                        if (whole) {
                            const float inv = l > 0.f ? 1.f / l : 0.f;
                            const int64_t at = (int64_t)token * p.out_stride_token + (int64_t)head * p.out_stride_head + dv;
                            if (p.q_dtype == CRIT_B200_DTYPE_BF16) ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(value * inv);
                            else ((__half*)p.out)[at] = __float2half_rn(value * inv);
                            if (p.lse && dv == 0) p.lse[(int64_t)token * p.q_heads + head] = l > 0.f ? top * LN2 + logf(l) : -INFINITY;
                        } else if (fits) {
                            const int64_t at = ((int64_t)(prow_first + colx) * p.q_heads + head) * p.max_splits + w.u.split;
                            p.workspace[at * DT_D + dv] = value;
                            if (dv == 0) {
                                p.workspace[states * DT_D + at] = top;
                                p.workspace[states * (DT_D + 1) + at] = l;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            // the next unit's references: -inf in the array that is not current (last read before the meeting above), which
            // every thread writes for itself and then takes as current
#pragma unroll
            for (int r = 0; r < NR; ++r) mref[(mb ^ 1) * 32 + r] = -INFINITY;
            mb ^= 1;
            w = after;
        }
        if (!ok) where = 0x540;
    }

    if (where && p.status) atomicExch(p.status, where);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, SW_COLUMNS);
}

}  // namespace crit_b200
