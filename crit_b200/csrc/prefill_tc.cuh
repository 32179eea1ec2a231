// Chunked prefill on the fifth-generation tensor cores: tcgen05.mma with the accumulators in tensor memory.
//
// A block holds 128 query rows (token-major (token, head of the kv head's group) pairs: a GQA group shares the keys and
// values it reads) and walks the sequence's positions in tiles of 64 (four pages of 16).  Per tile:
//   1. one thread issues the TMA tiled loads of the NEXT tile's pages (boxes of [16 positions][1 head][64 values],
//      128-byte swizzle: exactly the K-major / MN-major operand layouts the MMA reads) into the other stage;
//   2. one thread issues S = Q K^T: eight tcgen05.mma (M 128, N 64, K 16) from shared-memory descriptors into TMEM
//      columns 0..63, and commits to an mbarrier;
//   3. every thread owns one query row (= one TMEM lane): it reads its 64 scores with tcgen05.ld, masks the tile that
//      straddles its own position, updates its running maximum and sum, and writes its probabilities as bf16/fp16 into
//      shared memory in the A-operand layout (over the key tile, which is dead by then);
//   4. when a row's maximum moved (lazily: by more than 2^8), the rows' partial outputs in TMEM columns 64..191 are
//      rescaled with tcgen05.ld / tcgen05.st;
//   5. one thread issues O += P V: four tcgen05.mma (M 128, N 128, K 16), V as the MN-major B operand, and commits.
// Two blocks share an SM (99 KB of shared memory, 256 TMEM columns each), so one block's softmax overlaps the other's
// MMAs.  Every wait is bounded; a wait that runs out sets the status word, and the block frees its TMEM and leaves
// without writing.
// Reference: paged_kv_attention/_kernels.py:610-726 (_prefill_kernel); the reference's sm_100 wrappers were never run
// (kernels/core/include/crit_kcore/mma.cuh:349-354).
#pragma once

#include <cuda.h>

#include "tcgen05.cuh"

namespace crit_b200 {

constexpr int TC_ROWS = 128;       // query rows a block holds
constexpr int TC_BN = 64;          // positions a tile holds
constexpr int TC_D = 128;          // head width
constexpr int TC_Q_BYTES = 2 * TC_ROWS * 128;               // two 64-value halves of [128 rows][128 bytes]
constexpr int TC_K_BYTES = 2 * TC_BN * 128;                 // two halves of [64 positions][128 bytes]
constexpr int TC_STAGE = 2 * TC_K_BYTES;                    // keys, values
constexpr int TC_SMEM = 1024 + TC_Q_BYTES + 2 * TC_STAGE + 64;
constexpr uint32_t TC_COLUMNS = 256;                        // TMEM: scores at 0..63, outputs at 64..191

template <bool BF16>
__global__ void __launch_bounds__(TC_ROWS) prefill_tc_kernel(const crit_b200_prefill_params p,
                                                             const __grid_constant__ CUtensorMap kmap,
                                                             const __grid_constant__ CUtensorMap vmap, int32_t* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024 - (smem_addr(smem_raw) & 1023)) & 1023);
    unsigned char* qs = smem;
    unsigned char* stages = smem + TC_Q_BYTES;
    const uint32_t bars = smem_addr(stages + 2 * TC_STAGE);   // [0], [1]: a stage's loads; [2]: scores; [3]: outputs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stages + 2 * TC_STAGE + 32);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int h = blockIdx.y;
    const int G = p.q_heads / p.kv_heads;
    const int row0 = blockIdx.x * TC_ROWS;
    const int rows_total = p.tokens * G;
    const int pos32 = (int)(p.position_ptr ? *p.position_ptr : p.position);

    if (warp == 0) tmem_alloc(smem_addr(tmem_slot), TC_COLUMNS);
    if (tid == 0) {
        for (int b = 0; b < 4; ++b) mbar_init(bars + b * 8, 1);
        mbar_init_fence();
    }

    // -- queries into shared memory, K-major with the 128-byte swizzle ---------------------------------------------------
    for (int idx = tid; idx < TC_ROWS * 16; idx += TC_ROWS) {
        const int rr = idx >> 4, c = idx & 15;
        const int flat = row0 + rr;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (flat < rows_total) {
            const int tok = flat / G, gq = flat - tok * G;
            const char* src = (const char*)p.q + ((int64_t)tok * p.q_stride_token + (int64_t)(h * G + gq) * p.q_stride_head + c * 8) * 2;
            v = *reinterpret_cast<const uint4*>(src);
        }
        *reinterpret_cast<uint4*>(qs + (c >> 3) * (TC_ROWS * 128) + rr * 128 + (((c & 7) ^ (rr & 7)) << 4)) = v;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_s = tmem + ((uint32_t)(warp * 32) << 16);          // this warp's lanes, scores
    const uint32_t t_o = t_s + 64;                                      // outputs

    const int flat = row0 + tid;
    const int lastpos = flat < rows_total ? pos32 + flat / G : -1;
    const int last_row = (row0 + TC_ROWS < rows_total ? row0 + TC_ROWS : rows_total) - 1;
    const int end = pos32 + last_row / G + 1;               // the block reads positions [0, end)
    const int clear = pos32 + row0 / G;                     // positions <= clear are seen by every row of the block
    const int ntiles = (end + TC_BN - 1) / TC_BN;
    const uint32_t tiles_per_page = (uint32_t)p.page >> 4;
    const float sl2 = p.scale * LOG2E;
    const uint32_t idesc_s = idesc_f16(BF16, false, TC_ROWS, TC_BN);
    const uint32_t idesc_o = idesc_f16(BF16, true, TC_ROWS, TC_D);

    auto load_tile = [&](int i) {           // one thread: the tile's live pages into stage i & 1
        const int tile_pos = i * TC_BN;
        const int live = end - tile_pos < TC_BN ? end - tile_pos : TC_BN;
        const int boxes = (live + 15) >> 4;
        const uint32_t ks = smem_addr(stages + (i & 1) * TC_STAGE), vs = ks + TC_K_BYTES;
        const uint32_t bar = bars + (i & 1) * 8;
        fence_proxy_async();
        mbar_expect_tx(bar, (uint32_t)boxes * 4u * 2048u);
        for (int b = 0; b < boxes; ++b) {
            const uint32_t tile16 = (uint32_t)(i * (TC_BN / 16) + b);
            const uint32_t pidx = tile16 / tiles_per_page;
            const int slot0 = (int)((int64_t)p.table[pidx] * p.page + ((tile16 - pidx * tiles_per_page) << 4));
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                tma_load_3d(ks + half * (TC_BN * 128) + b * 2048, &kmap, half * 64, h, slot0, bar);
                tma_load_3d(vs + half * (TC_BN * 128) + b * 2048, &vmap, half * 64, h, slot0, bar);
            }
        }
    };

    float m_run = -INFINITY, l_run = 0.f;
    bool dead = false;
    int where = 0;                 // which wait gave up (0x100 loads, 0x200 scores, 0x300 outputs) + the tile
    if (tid == 0 && ntiles > 0) load_tile(0);
    for (int i = 0; i < ntiles && !dead; ++i) {
        const int tile_pos = i * TC_BN;
        unsigned char* kst = stages + (i & 1) * TC_STAGE;
        unsigned char* vst = kst + TC_K_BYTES;
        if (tid == 0 && i + 1 < ntiles) load_tile(i + 1);
        dead = !mbar_wait(bars + (i & 1) * 8, (uint32_t)(i >> 1) & 1u);
        if (dead) where = 0x100 + i;
        const int live = end - tile_pos;
        if (live < TC_BN) {
            // value rows past the block's last position: zeros (a probability of 0 times stale bytes must stay 0)
            for (int idx = tid; idx < TC_BN * 16; idx += TC_ROWS) {
                const int rr = idx >> 4, c = idx & 15;
                if (rr >= live)
                    *reinterpret_cast<uint4*>(vst + (c >> 3) * (TC_BN * 128) + rr * 128 + (((c & 7) ^ (rr & 7)) << 4)) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async();
        }
        tc_fence_before();
        dead = __syncthreads_or(dead);
        if (dead) break;
        tc_fence_after();

        // scores
        if (tid == 0) {
#pragma unroll
            for (int ks = 0; ks < TC_D / 16; ++ks) {
                const uint64_t a = smem_desc_sw128(smem_addr(qs) + (ks >> 2) * (TC_ROWS * 128) + (ks & 3) * 32, 0, 1024);
                const uint64_t b = smem_desc_sw128(smem_addr(kst) + (ks >> 2) * (TC_BN * 128) + (ks & 3) * 32, 0, 1024);
                umma_f16(tmem, a, b, idesc_s, ks > 0);
            }
            umma_commit(bars + 2 * 8);
        }
        dead = !mbar_wait(bars + 2 * 8, (uint32_t)i & 1u);
        if (dead) where = 0x200 + i;
        dead = __syncthreads_or(dead);
        if (dead) break;
        tc_fence_after();

        // this thread's row of the tile: scale, mask, running maximum (lazy), probabilities
        float s[TC_BN];
        {
            float half[32];
            tmem_ld32(t_s, half);
#pragma unroll
            for (int j = 0; j < 32; ++j) s[j] = half[j];
            tmem_ld32(t_s + 32, half);
#pragma unroll
            for (int j = 0; j < 32; ++j) s[32 + j] = half[j];
        }
        const bool masked = tile_pos + TC_BN - 1 > clear;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < TC_BN; ++j) {
            float x = s[j] * sl2;
            if (masked && tile_pos + j > lastpos) x = -INFINITY;
            s[j] = x;
            mx = fmaxf(mx, x);
        }
        const bool moved = mx > m_run + LAZY || m_run == -INFINITY;
        const float top = moved ? mx : m_run;
        const float sub = top == -INFINITY ? 0.f : top;
        const float alpha = moved ? ex2(m_run - sub) : 1.f;
        const bool rescale = moved && top != m_run && i > 0;
        m_run = top;
        float sum = 0.f;
        unsigned char* prow = kst + tid * 128;              // the probabilities go over the key tile's first 16 KB
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float a = ex2(s[c * 8 + 2 * e] - sub), b = ex2(s[c * 8 + 2 * e + 1] - sub);
                sum += a + b;
                w[e] = pack2<BF16>(a, b);
            }
            *reinterpret_cast<uint4*>(prow + ((c ^ (tid & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        l_run = l_run * alpha + sum;
        if (__syncthreads_or(rescale ? 1 : 0)) {
            // the rows whose maximum moved bring their partial outputs to the new reference
#pragma unroll
            for (int c = 0; c < TC_D / 32; ++c) {
                float o[32];
                tmem_ld32(t_o + c * 32, o);
#pragma unroll
                for (int j = 0; j < 32; ++j) o[j] *= alpha;
                tmem_st32(t_o + c * 32, o);
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        // outputs
        if (tid == 0) {
#pragma unroll
            for (int kk = 0; kk < TC_BN / 16; ++kk) {
                const uint64_t a = smem_desc_sw128(smem_addr(kst) + kk * 32, 0, 1024);
                const uint64_t b = smem_desc_sw128(smem_addr(vst) + kk * 2048, TC_BN * 128, 1024);
                umma_f16(tmem + 64, a, b, idesc_o, i > 0 || kk > 0);
            }
            umma_commit(bars + 3 * 8);
        }
        dead = !mbar_wait(bars + 3 * 8, (uint32_t)i & 1u);
        if (dead) where = 0x300 + i;
        dead = __syncthreads_or(dead);
        tc_fence_after();
    }

    // -- this thread's row out ---------------------------------------------------------------------------------------
    // tcgen05.ld is warp-collective: every lane of a warp issues it, the lanes without a row only skip the stores.
    if (!dead) {
        const bool has_row = flat < rows_total;
        const int tok = flat / G, gq = flat - tok * G, head = h * G + gq;
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        char* dst = (char*)p.out + ((int64_t)tok * p.out_stride_token + (int64_t)head * p.out_stride_head) * 2;
#pragma unroll
        for (int c = 0; c < TC_D / 32; ++c) {
            float o[32];
            tmem_ld32(t_o + c * 32, o);
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
        if (has_row && p.lse) p.lse[(int64_t)tok * p.q_heads + head] = l_run > 0.f ? m_run * LN2 + logf(l_run) : -INFINITY;
    }
    if (dead && where && status) atomicExch(status, where);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TC_COLUMNS);
}

}  // namespace crit_b200
