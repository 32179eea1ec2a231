// Chunked prefill on the fifth-generation tensor cores: tcgen05.mma with the accumulators in tensor memory, in a
// warp-specialised pipeline.
//
// A block holds 128 query rows (token-major (token, head of the kv head's group) pairs: a GQA group shares the keys and
// values it reads) and walks the sequence's positions in tiles of 64 (four pages of 16).  Warp roles:
//   warps 0-3  softmax: thread = one query row = one TMEM lane.  It reads its 64 scores of a tile (tcgen05.ld), masks the
//              tile that straddles its own position, updates its running maximum (lazily: when beaten by 2^8) and sum,
//              writes its probabilities as bf16/fp16 back into tensor memory, over its own scores (tcgen05.st: the
//              second product takes its A operand from TMEM, so the probabilities never cross shared memory), and
//              rescales its output lane in TMEM when its maximum moved;
//   warp 4     producer: the next 32 boxes' page ids in registers, a batch ahead; TMA tiled loads (boxes of
//              [16 positions][1 head][64 values], 128-byte swizzle: exactly the K-major / MN-major operand layouts the
//              MMA reads) into a ring of two stages whose keys and values land and free separately (the keys are
//              free once the first product has read them, so the next keys stream in during a tile's softmax);
//   warp 5     MMA issue (one lane): S = Q K^T as eight tcgen05.mma (M 128, N 64, K 16) into one of TWO score buffers
//              (TMEM columns 0..63 and 64..127), O += P V as four (M 128, N 128, K 16, V as the MN-major B operand) into
//              columns 128..255, one tile behind: a tile's softmax overlaps the next tile's first product.
// Two blocks share an SM (96 KB of shared memory, 256 TMEM columns each).  Every wait is bounded in time and polls a
// block-wide abort flag; a wait that runs out sets the status word, and the block frees its TMEM and leaves without
// writing.  tcgen05.ld / tcgen05.st are warp-collective: every lane of a warp issues them, whether its row exists or not.
// Reference: paged_kv_attention/_kernels.py:610-726 (_prefill_kernel); the reference's sm_100 wrappers were never run
// (kernels/core/include/crit_kcore/mma.cuh:349-354).
#pragma once

#include <cuda.h>

#include "tcgen05.cuh"

namespace crit_b200 {

constexpr int TC_ROWS = 128;       // query rows a block holds
constexpr int TC_BN = 64;          // positions a tile holds
constexpr int TC_D = 128;          // head width
constexpr int TC_THREADS = 224;     // 4 softmax warps, a producer warp, a warp for each product's MMAs
constexpr int TC_Q_BYTES = 2 * TC_ROWS * 128;               // two 64-value halves of [128 rows][128 bytes]
constexpr int TC_K_BYTES = 2 * TC_BN * 128;                 // two halves of [64 positions][128 bytes]
constexpr int TC_STAGE = 2 * TC_K_BYTES;                    // keys, values
constexpr int TC_SMEM = TC_Q_BYTES + 2 * TC_STAGE + 256;     // 16 mbarriers, the TMEM address, the abort flag
constexpr uint32_t TC_COLUMNS = 256;                        // TMEM: scores at 0..63 and 64..127, outputs at 128..255
constexpr uint32_t TC_O = 128;
constexpr float TC_LAZY = 8.f;

enum { TC_KFULL = 0, TC_VFULL = 2, TC_KEMPTY = 4, TC_VEMPTY = 6, TC_SFULL = 8, TC_SFREE = 10, TC_PFULL = 12, TC_PVDONE = 13, TC_PFREE = 14 };

__device__ __forceinline__ void tc_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// A bounded wait that also gives up when another thread of the block already did.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    do {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    } while (global_ns() - t0 < 250000000ull);
    *abort_flag = 1;
    return false;
}

template <bool BF16>
__global__ void __launch_bounds__(TC_THREADS, 2) prefill_tc_kernel(const crit_b200_prefill_params p,
                                                                   const __grid_constant__ CUtensorMap kmap,
                                                                   const __grid_constant__ CUtensorMap vmap, int32_t* status) {
    constexpr uint32_t FULLMASK = 0xffffffffu;
    extern __shared__ __align__(1024) unsigned char smem[];        // the 128-byte swizzle wants 1 KB alignment (checked below)
    unsigned char* qs = smem;
    unsigned char* stages = smem + TC_Q_BYTES;
    unsigned char* small = stages + 2 * TC_STAGE;
    const uint32_t bars = smem_addr(small);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(small + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(small + 132);
    auto bar = [&](int which) { return bars + (uint32_t)which * 8u; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    const int G = p.q_heads / p.kv_heads;
    const int row0 = blockIdx.x * TC_ROWS;
    const int seq = blockIdx.z;                 // one sequence of the launch
    const int tok0 = p.starts ? p.starts[seq] : seq * p.tokens;
    const int rows_total = (p.starts ? p.starts[seq + 1] - tok0 : p.tokens) * G;
    if (row0 >= rows_total) return;             // a shorter sequence of a ragged launch (the whole block leaves, before any allocation)
    const int32_t* table = p.table + (int64_t)seq * p.table_stride;
    const int pos32 = (int)(p.positions ? p.positions[seq] : (p.position_ptr ? *p.position_ptr : p.position));

    if (smem_addr(smem) & 1023u) {              // never seen; the operand layouts would be wrong: say so and leave
        if (tid == 0 && status) atomicExch(status, 0x1ff);
        return;
    }
    if (warp == 0) tmem_alloc(smem_addr(tmem_slot), TC_COLUMNS);
    if (tid == 32) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(TC_KFULL + b), 1), mbar_init(bar(TC_KEMPTY + b), 1);
            mbar_init(bar(TC_VFULL + b), 1), mbar_init(bar(TC_VEMPTY + b), 1);
            mbar_init(bar(TC_SFULL + b), 1), mbar_init(bar(TC_SFREE + b), 128);
        }
        mbar_init(bar(TC_PFULL), 128), mbar_init(bar(TC_PVDONE), 1);
        mbar_init(bar(TC_PFREE), 1), mbar_init(bar(TC_PFREE + 1), 1);
        *abort_flag = 0;
        mbar_init_fence();
    }

    // -- queries into shared memory, K-major with the 128-byte swizzle ---------------------------------------------------
    for (int idx = tid; idx < TC_ROWS * 16; idx += TC_THREADS) {
        const int rr = idx >> 4, c = idx & 15;
        const int flat = row0 + rr;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (flat < rows_total) {
            const int tok = flat / G, gq = flat - tok * G;
            const char* src = (const char*)p.q + ((int64_t)(tok0 + tok) * p.q_stride_token + (int64_t)(h * G + gq) * p.q_stride_head + c * 8) * 2;
            v = *reinterpret_cast<const uint4*>(src);
        }
        *reinterpret_cast<uint4*>(qs + (c >> 3) * (TC_ROWS * 128) + rr * 128 + (((c & 7) ^ (rr & 7)) << 4)) = v;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int last_row = (row0 + TC_ROWS < rows_total ? row0 + TC_ROWS : rows_total) - 1;
    const int end = pos32 + last_row / G + 1;               // the block reads positions [0, end)
    const int clear = pos32 + row0 / G;                     // positions <= clear are seen by every row of the block
    const int ntiles = (end + TC_BN - 1) / TC_BN;
    const uint32_t tiles_per_page = (uint32_t)p.page >> 4;
    int where = 0;                 // which role's wait gave up

    if (warp == 4) {
        // -- producer: lane l holds the page id of box 32 * batch + l (a box is 16 positions), a batch ahead ---------------
        const int nboxes = (end + 15) >> 4;
        auto fetch = [&](int batch) {
            const int box = batch * 32 + lane;
            return box < nboxes ? table[(uint32_t)box / tiles_per_page] : 0;
        };
        int cur = fetch(0), nxt = fetch(1);
        bool ok = true;
        // The keys of tile i are asked for before the values of tile i - 1: a key buffer is free after the first
        // product of the tile two back, long before the value buffer of the tile before is (after ITS second product),
        // and the first products are what the softmax warps wait for.
        int v_slot0 = 0, v_boxes = 0;
        auto values = [&](int t) {          // the values of tile t (its slot and boxes kept from the keys' turn)
            const int s = t & 1;
            const uint32_t vs = smem_addr(stages + s * TC_STAGE) + TC_K_BYTES;
            ok = tc_wait(bar(TC_VEMPTY + s), (uint32_t)((t >> 1) & 1) ^ 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) return;
            if (lane == 0) mbar_expect_tx(bar(TC_VFULL + s), (uint32_t)v_boxes * 2u * 2048u);
            __syncwarp();
            if (lane < v_boxes) {
#pragma unroll
                for (int half = 0; half < 2; ++half)
                    tma_load_3d(vs + half * (TC_BN * 128) + lane * 2048, &vmap, half * 64, h, v_slot0, bar(TC_VFULL + s));
            }
        };
        for (int i = 0; i < ntiles; ++i) {
            if (i > 0 && (i & 7) == 0) cur = nxt, nxt = fetch((i >> 3) + 1);
            const int s = i & 1;
            const int live = end - i * TC_BN < TC_BN ? end - i * TC_BN : TC_BN;
            const int boxes = (live + 15) >> 4;
            const int pg = __shfl_sync(FULLMASK, cur, ((i & 7) << 2) + (lane & 3));
            const uint32_t tile16 = (uint32_t)(i * (TC_BN / 16) + (lane & 3));
            const int slot0 = (int)((int64_t)pg * p.page + ((tile16 % tiles_per_page) << 4));
            const uint32_t ks = smem_addr(stages + s * TC_STAGE);
            ok = tc_wait(bar(TC_KEMPTY + s), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(bar(TC_KFULL + s), (uint32_t)boxes * 2u * 2048u);
            __syncwarp();
            if (lane < boxes) {
#pragma unroll
                for (int half = 0; half < 2; ++half)
                    tma_load_3d(ks + half * (TC_BN * 128) + lane * 2048, &kmap, half * 64, h, slot0, bar(TC_KFULL + s));
            }
            if (i > 0) {
                values(i - 1);
                if (!ok) break;
            }
            v_slot0 = slot0, v_boxes = boxes;
        }
        if (ok && ntiles > 0) values(ntiles - 1);
        if (!ok) where = 0x110;
    } else if (warp == 5) {
        // -- the first products, S = Q K^T of every tile ------------------------------------------------------------------------
        const uint32_t idesc_s = idesc_f16(BF16, false, TC_ROWS, TC_BN);
        // The operands' descriptors are made once: a step of 16 bytes in the address is a step of 1 in the descriptor, so a
        // tile's MMAs take theirs with one addition each (the issue of the twelve MMAs of a tile is what bounds the block).
        const uint64_t q_desc = smem_desc_sw128(smem_addr(qs), 0, 1024);
        const uint64_t k_desc0 = smem_desc_sw128(smem_addr(stages), 0, 1024);
        bool ok = true;
        for (int i = 0; i < ntiles && ok; ++i) {
            const int s = i & 1;
            // (a tile's probabilities sit over its scores: the buffer is free for the scores of tile i once the second
            // product of tile i - 2 has read them; the two products are issued by different warps)
            ok = tc_wait(bar(TC_KFULL + s), (uint32_t)(i >> 1) & 1u, abort_flag) &&
                 tc_wait(bar(TC_SFREE + s), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag) &&
                 tc_wait(bar(TC_PFREE + s), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint64_t kd = k_desc0 + (uint64_t)((s * TC_STAGE) >> 4);
#pragma unroll
                for (int ks = 0; ks < TC_D / 16; ++ks)
                    umma_f16(tmem + (uint32_t)(s * TC_BN), q_desc + (uint64_t)(((ks >> 2) * (TC_ROWS * 128) + (ks & 3) * 32) >> 4),
                             kd + (uint64_t)(((ks >> 2) * (TC_BN * 128) + (ks & 3) * 32) >> 4), idesc_s, ks > 0);
                umma_commit(bar(TC_SFULL + s));
                umma_commit(bar(TC_KEMPTY + s));
            }
            __syncwarp();
        }
        if (!ok) where = 0x120;
    } else if (warp == 6) {
        // -- the second products, O (+)= P V of every tile, from a warp of their own (one thread issuing a tile's twelve MMAs
        //    was what bounded the block) -----------------------------------------------------------------------------------
        const uint32_t idesc_o = idesc_f16(BF16, true, TC_ROWS, TC_D);
        const uint64_t v_desc0 = smem_desc_sw128(smem_addr(stages) + TC_K_BYTES, TC_BN * 128, 1024);
        bool ok = true;
        auto issue_pv = [&](int t) {        // O (+)= P V of tile t
            ok = tc_wait(bar(TC_PFULL), (uint32_t)t & 1u, abort_flag) &&
                 tc_wait(bar(TC_VFULL + (t & 1)), (uint32_t)(t >> 1) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) return;
            tc_fence_after();
            if (lane == 0) {
                // the probabilities of tile t sit over its scores: 16 of them (8 columns) a K step
                const uint32_t pa = tmem + (uint32_t)((t & 1) * TC_BN);
                const uint64_t vd = v_desc0 + (uint64_t)(((t & 1) * TC_STAGE) >> 4);
                if (t > 0) umma_f16_ts(tmem + TC_O, pa, vd, idesc_o, true);
                else umma_f16_ts(tmem + TC_O, pa, vd, idesc_o, false);
#pragma unroll
                for (int kk = 1; kk < TC_BN / 16; ++kk) umma_f16_ts(tmem + TC_O, pa + kk * 8, vd + (uint64_t)(kk * 2048 >> 4), idesc_o, true);
                umma_commit(bar(TC_VEMPTY + (t & 1)));
                umma_commit(bar(TC_PVDONE));
                umma_commit(bar(TC_PFREE + (t & 1)));
            }
            __syncwarp();
        };
        for (int i = 0; i < ntiles && ok; ++i) issue_pv(i);
        if (!ok) where = 0x130;
    } else {
        // -- softmax: thread = query row row0 + tid = TMEM lane tid -------------------------------------------------------------
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int flat = row0 + tid;
        const bool has_row = flat < rows_total;
        const int lastpos = has_row ? pos32 + flat / G : -1;
        const float sl2 = p.scale * LOG2E;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int i = 0; i < ntiles; ++i) {
            const int s = i & 1;
            const int tile_pos = i * TC_BN;
            unsigned char* vst = stages + s * TC_STAGE + TC_K_BYTES;
            ok = tc_wait(bar(TC_SFULL + s), (uint32_t)(i >> 1) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
            if (!ok) break;
            tc_fence_after();
            float sc[TC_BN];
            {
                float half[32];
                tmem_ld32(tmem + lane_base + (uint32_t)(s * TC_BN), half);
#pragma unroll
                for (int j = 0; j < 32; ++j) sc[j] = half[j];
                tmem_ld32(tmem + lane_base + (uint32_t)(s * TC_BN + 32), half);
#pragma unroll
                for (int j = 0; j < 32; ++j) sc[32 + j] = half[j];
            }
            tc_fence_before();
            tc_arrive(bar(TC_SFREE + s));
            const int live = end - tile_pos;
            if (live < TC_BN) {
                // value rows past the block's last position: zeros (a probability of 0 times stale bytes must stay 0),
                // written once the tile's values have landed
                ok = tc_wait(bar(TC_VFULL + s), (uint32_t)(i >> 1) & 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                for (int idx = tid; idx < TC_BN * 16; idx += 128) {
                    const int rr = idx >> 4, c = idx & 15;
                    if (rr >= live)
                        *reinterpret_cast<uint4*>(vst + (c >> 3) * (TC_BN * 128) + rr * 128 + (((c & 7) ^ (rr & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                }
            }
            // The maximum is taken over the raw scores (the scale is positive), and a probability is one FFMA and one
            // exp2: 2^(score * scale * log2 e - reference).  Only the tiles that straddle a row's own position mask.
            const bool masked = tile_pos + TC_BN - 1 > clear;
            if (masked) {
#pragma unroll
                for (int j = 0; j < TC_BN; ++j)
                    if (tile_pos + j > lastpos) sc[j] = -INFINITY;
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int j = 0; j < TC_BN; j += 4) {
                mx0 = fmaxf(mx0, sc[j]), mx1 = fmaxf(mx1, sc[j + 1]);
                mx2 = fmaxf(mx2, sc[j + 2]), mx3 = fmaxf(mx3, sc[j + 3]);
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
            const bool moved = mx > m_run + TC_LAZY || m_run == -INFINITY;
            const float top = moved ? mx : m_run;
            const float sub = top == -INFINITY ? 0.f : top;
            const float alpha = moved ? ex2(m_run - sub) : 1.f;
            const bool rescale = moved && top != m_run && i > 0;
            m_run = top;
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t pw[32];
            const float nsub = -sub;
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const float a = ex2(fmaf(sc[2 * e], sl2, nsub)), b = ex2(fmaf(sc[2 * e + 1], sl2, nsub));
                sum0 += a, sum1 += b;
                pw[e] = pack2<BF16>(a, b);
            }
            l_run = l_run * alpha + (sum0 + sum1);
            // over this row's own scores (read above, and the buffer's next scores come after the second product that
            // reads these probabilities: the MMA warp issues them in that order)
            tmem_st32u(tmem + lane_base + (uint32_t)(s * TC_BN), pw);
            if (__any_sync(FULLMASK, rescale)) {
                // a maximum of the warp's rows moved: their partial outputs go to the new reference, once the second
                // product of the tile before has landed
                ok = tc_wait(bar(TC_PVDONE), (uint32_t)(i - 1) & 1u, abort_flag);
                ok = __all_sync(FULLMASK, ok);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < TC_D / 32; ++c) {
                    float o[32];
                    tmem_ld32(tmem + lane_base + TC_O + c * 32, o);
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] *= alpha;
                    tmem_st32(tmem + lane_base + TC_O + c * 32, o);
                }
            }
            if (live < TC_BN) fence_proxy_async();          // the zeros written over the last tile's values
            tc_fence_before();
            tc_arrive(bar(TC_PFULL));
        }
        // -- this thread's row out ---------------------------------------------------------------------------------------
        if (ok && ntiles > 0) {
            ok = tc_wait(bar(TC_PVDONE), (uint32_t)(ntiles - 1) & 1u, abort_flag);
            ok = __all_sync(FULLMASK, ok);
        }
        if (ok) {
            tc_fence_after();
            const int tok = flat / G, gq = flat - tok * G, head = h * G + gq;
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            char* dst = (char*)p.out + ((int64_t)(tok0 + tok) * p.out_stride_token + (int64_t)head * p.out_stride_head) * 2;
#pragma unroll
            for (int c = 0; c < TC_D / 32; ++c) {
                float o[32];
                tmem_ld32(tmem + lane_base + TC_O + c * 32, o);
                if (has_row) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 v;
                        v.x = pack2<BF16>(o[j] * inv, o[j + 1] * inv), v.y = pack2<BF16>(o[j + 2] * inv, o[j + 3] * inv);
                        v.z = pack2<BF16>(o[j + 4] * inv, o[j + 5] * inv), v.w = pack2<BF16>(o[j + 6] * inv, o[j + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + (c * 32 + j) * 2) = v;
                    }
                }
            }
            if (has_row && p.lse) p.lse[(int64_t)(tok0 + tok) * p.q_heads + head] = l_run > 0.f ? m_run * LN2 + logf(l_run) : -INFINITY;
        } else {
            where = 0x140;
        }
    }
    if (where && status) atomicExch(status, where);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TC_COLUMNS);
}

}  // namespace crit_b200
