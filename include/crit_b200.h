/* crit_b200: C ABI of the B200-native paged KV-cache hot path (KV append into pages, block-table gather, split-K
 * decode / speculative-verify attention with its log-sum-exp merge, chunked prefill).
 *
 * Conventions (they mirror the reference's one native boundary on this path, crit's CUDA flash tile:
 * kernels/techniques/attention/paged-kv-attention/torch-ext/paged_kv_attention/cuda_window.cu:1482-1535, bound by
 * ctypes in paged_kv_attention/__init__.py:807-883):
 *   - plain pointers and sizes, parameter blocks are POD structs passed by address and copied by the call;
 *   - every pointer is DEVICE memory of the thread's current device unless its comment says "host";
 *   - the caller owns every buffer; a call allocates nothing and never waits for the host;
 *   - work is queued on `stream` (a cudaStream_t as void*; NULL is the legacy default stream) and may be captured
 *     in a CUDA graph;
 *   - the return value is 0 on success, a cudaError_t (> 0) when the runtime refused a launch, or a negative
 *     CRIT_B200_E* code when the parameters describe something the kernels do not serve; crit_b200_error() names it.
 */
#ifndef CRIT_B200_H
#define CRIT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CRIT_B200_ABI_VERSION 3

/* Page kinds (the reference's KINDS, paged_kv_attention/__init__.py:78, plus the per-page FP8 scale). */
#define CRIT_B200_KIND_16BIT    0   /* bf16 or fp16 pages (page_dtype says which) */
#define CRIT_B200_KIND_FP8      1   /* E4M3 codes, one multiplier per layer for keys and one for values */
#define CRIT_B200_KIND_FP8_ROW  2   /* E4M3 codes, FP32 scale per (slot, kv head): scales [slots][kv_heads] */
#define CRIT_B200_KIND_INT8     3   /* INT8 codes, FP32 scale per (slot, kv head) */
#define CRIT_B200_KIND_FP8_PAGE 4   /* E4M3 codes, FP32 scale per (page, kv head): scales [pages][kv_heads] */

#define CRIT_B200_DTYPE_BF16 0
#define CRIT_B200_DTYPE_FP16 1
#define CRIT_B200_DTYPE_FP32 2

#define CRIT_B200_EINVAL      (-1)  /* a size, stride or pointer the call cannot take */
#define CRIT_B200_EUNSUPPORTED (-2) /* a geometry no kernel was built for (head widths, page size, page kind) */
#define CRIT_B200_EWORKSPACE  (-3)  /* the workspace is smaller than crit_b200_attend_plan said */
#define CRIT_B200_EALIGN      (-4)  /* a pointer or stride is not aligned as the kernels read it */
#define CRIT_B200_ESTATIC     (-5)  /* the launch needs more partials than crit_b200_attend_static's built-in scratch holds */

/* What a kernel leaves in a `status` word (it sets, never clears): a launch whose word is not 0 afterwards has skipped
 * the work concerned and written nothing for it. */
#define CRIT_B200_STATUS_TMA    1      /* a TMA copy of the m16n8k16 decode kernel never landed (bounded wait) */
#define CRIT_B200_STATUS_PLAN   2      /* a row took more splits or partial rows than max_splits / partial_rows allow */
#define CRIT_B200_STATUS_BOUNDS 3      /* a slot or page id lay outside the page tensor (slots_total / slots given) */
                                       /* 0x110..0x1ff: the tcgen05 prefill kernel's waits; 0x410..0x440: the tcgen05 decode
                                          kernel's; 0x800 + rank: the peer exchange waited in vain; 0x900 + rank: that
                                          rank's message carried another step's or shape's header */

/* -- KV append ---------------------------------------------------------------------------------------------------
 * Replaces paged_kv_attention.write (paged_kv_attention/__init__.py:289-324, kernel _kernels.py:112-150) and the torch
 * path of KVPool.write (inference/attention-state/code/pages.py:420-453 with fp8_rows/int8_rows :872-895).
 * keys [tokens][kv_heads][head_dim] and values [tokens][kv_heads][value_dim] (strides in elements, last dimension
 * contiguous) go to slots[t] of pages laid out [slots][kv_heads][dim]; a slot below 0 is skipped.  values NULL: keys
 * only.  Codes and scales are bit-exact with the reference's rules. */
typedef struct crit_b200_append_params {
    const void* keys;
    const void* values;
    const int64_t* slots;
    void* key_pages;
    void* value_pages;
    float* key_scales;           /* kinds 2, 3: [slots][kv_heads]; kind 4: [pages][kv_heads]; else NULL */
    float* value_scales;
    int32_t* status;             /* or NULL: set to CRIT_B200_STATUS_BOUNDS when a slot lay outside [0, slots_total) */
    int64_t tokens;
    int64_t slots_total;         /* slots each page tensor stores; a slot at or past it is skipped and reported.  0: unknown,
                                    nothing is checked */
    int64_t key_stride_token, key_stride_head, value_stride_token, value_stride_head;
    int32_t kv_heads, head_dim, value_dim, page;
    int32_t kind, in_dtype, page_dtype;
    float key_multiplier, value_multiplier;     /* kind 1: codes = x / multiplier */
} crit_b200_append_params;

int crit_b200_append(const crit_b200_append_params* params, void* stream);

/* -- block-table page gather -------------------------------------------------------------------------------------
 * Replaces KVPool.gather / rows_at (pages.py:455-493): rows of one page tensor, dequantised (code * scale in FP32,
 * then rounded to out_dtype), read through a page table (slots NULL: positions 0..count-1 of `table`) or at explicit
 * slots (table NULL).  out [count][kv_heads][dim] contiguous. */
typedef struct crit_b200_gather_params {
    const void* pages;
    const float* scales;
    const int32_t* table;
    const int64_t* slots;
    void* out;
    int32_t* status;             /* or NULL: set to CRIT_B200_STATUS_BOUNDS when a slot lay outside [0, slots_total) */
    int64_t count;
    int64_t slots_total;         /* slots the page tensor stores; a row whose slot is outside reads as zeros.  0: unchecked */
    int32_t kv_heads, dim, page;
    int32_t kind, page_dtype, out_dtype;
    float multiplier;
} crit_b200_gather_params;

int crit_b200_gather(const crit_b200_gather_params* params, void* stream);

/* -- slot mapping on the device ----------------------------------------------------------------------------------
 * Replaces KVPool._slots_at (pages.py:653-660) and the per-token host arithmetic of KVPool.reserve (:347, :721-722):
 * slot = tables[row[i]][clamp(p / page)] * page + p % page; with `capacity` (one per table row) a position outside
 * [0, capacity[row]) gets dump * page. */
typedef struct crit_b200_slots_params {
    const int32_t* tables;
    const int64_t* rows;         /* [n] table row of each position */
    const int64_t* positions;    /* [n] */
    const int64_t* capacity;     /* [table rows] or NULL */
    int64_t* slots;              /* [n] out */
    int64_t n, table_stride;
    int32_t table_width, page, dump;
} crit_b200_slots_params;

int crit_b200_slots(const crit_b200_slots_params* params, void* stream);

/* Rows of one store (keys, values or their row scales, all layers) moved between slots: for every list r, in order
 * j = 0 .. width - 1, the `row_bytes` bytes at slot source[r][j] of every layer go to slot target[r][j] (nothing where
 * the two are equal).  A list's moves happen one after another, so a later move may read what an earlier one of the
 * same list wrote over only if the lists say so; the accepted path of a draft tree (node path[j] -> position j, path[j]
 * >= j) never does.  Lists are independent (their slots are disjoint).  The pool's commit_round uses it to bring an
 * accepted path's KV to consecutive positions (inference/attention-state/code/pages.py:662-684). */
typedef struct crit_b200_move_params {
    void* store;                 /* [layers][slots] rows of row_bytes bytes */
    const int64_t* source;       /* [lists][width] slots */
    const int64_t* target;       /* [lists][width] slots */
    int64_t lists, width, slots; /* slots: rows a layer holds (a slot outside [0, slots) is skipped and reported) */
    int64_t row_bytes;           /* a multiple of 4 */
    int32_t layers;
    int32_t* status;             /* optional device word: CRIT_B200_STATUS_BOUNDS */
} crit_b200_move_params;

int crit_b200_move_rows(const crit_b200_move_params* params, void* stream);

/* Block lists turned into page tables of their own (the block-sparse reader's gather, paged_kv_attention/_kernels.py:
 * 481-555): every token of the launch's window rows (row r, column c: token starts[r] + c at position firsts[r] + c)
 * becomes a row of ONE column whose table holds the pages of the token's listed KV blocks only (block_size a multiple of
 * page; ids below 0, above the token's position, or listed twice are left out; the block holding the token's own position
 * goes last and counts up to that position).  Attending the compact rows (rows = 0 .. n - 1, columns = 1, counts and
 * firsts as written here) reads the listed blocks and nothing else.  A column past its row's count gets count 0; a token
 * that sees no position gets count 0 and, when `out` is given, zeros there (and -inf in `lse`). */
typedef struct crit_b200_compact_params {
    const int32_t* tables;       /* [table rows][table_stride] page ids */
    const int32_t* rows;         /* [n_rows] table row of each window row */
    const int32_t* starts;       /* [n_rows] */
    const int32_t* counts;       /* [n_rows] or NULL: `columns` each */
    const int64_t* firsts;       /* [n_rows] */
    const int32_t* blocks;       /* [tokens][blocks_k] */
    int32_t* out_tables;         /* [n_rows * columns][blocks_k * block_size / page] */
    int32_t* out_counts;         /* [n_rows * columns] 1 or 0 */
    int64_t* out_firsts;         /* [n_rows * columns] the compact row's last position */
    void* out;                   /* optional: the attention's out, for the tokens that see nothing */
    float* lse;                  /* optional */
    int64_t n_rows, table_stride, out_stride_token, out_stride_head;
    int32_t table_width, columns, blocks_k, block_size, page, dump, q_heads, value_dim, out_dtype;
} crit_b200_compact_params;

int crit_b200_compact_blocks(const crit_b200_compact_params* params, void* stream);

#define CRIT_B200_ATTEND_NO_TMA 1   /* stage pages with cp.async even where the TMA path serves the geometry */
#define CRIT_B200_ATTEND_TMA    2   /* stage pages with TMA wherever it serves the geometry (default: 16-bit pages only,
                                       where it measured faster; 8-bit pages measured faster with cp.async) */

#define CRIT_B200_ATTEND_PERSISTENT 4 /* a fixed number of blocks (what the SMs hold at once) walk a work list built on the
                                        device from the rows' lengths, instead of one block per (split, kv head, row)
                                        slot of a 3-D grid; the same bits; at most 256 rows, else the 3-D grid */

#define CRIT_B200_ATTEND_TCGEN05 8   /* the tcgen05 kernel (E4M3 page bytes straight into kind::f8f6f4 MMAs, queries and
                                       probabilities as two E4M3 terms each) or CRIT_B200_EUNSUPPORTED: E4M3 pages of
                                       128-wide heads, columns x group heads <= 32, chunk a multiple of 128, slots set */
#define CRIT_B200_ATTEND_MMA_SYNC 16 /* the m16n8k16 kernel even where the tcgen05 kernel serves the launch */
#define CRIT_B200_ATTEND_TCGEN05T 64 /* the tcgen05 kernel with the operands swapped (the key and value tiles on the MMA's 128
                                        rows, the query rows on its columns) or CRIT_B200_EUNSUPPORTED: the same launches
                                        CRIT_B200_ATTEND_TCGEN05 takes */
#define CRIT_B200_ATTEND_TCGEN05P 128 /* the tcgen05 kernel over whole page rows (a unit reads all kv heads of its positions: one
                                         contiguous piece of HBM a tile; the launch's tiles are dealt out evenly, so a split
                                         may be shared by two blocks) or CRIT_B200_EUNSUPPORTED: E4M3 pages of 128-wide heads,
                                         8 kv heads, columns x group heads <= 8, chunk a multiple of 16 up to 2,048, a workspace
                                         with max_splits >= 2 x the splits of the longest row: a split has two states there,
                                         and both launches (decode and merge) carry the flag */
#define CRIT_B200_ATTEND_CONTEXT 256 /* every column of a row sees the positions BEFORE firsts[r] and none from there on (the
                                        part of a prompt chunk's attention that reads the pages, when the chunk's own keys
                                        and values are read fresh from elsewhere and the two parts merged by their lse);
                                        the m16n8k16 kernel's; both launches (decode and merge) carry the flag */
#define CRIT_B200_ATTEND_PARTIALS 32 /* every row's split states go to the workspace, a row of one split too (the first launch
                                        writes nothing to out / lse): what crit_b200_merge_push sends, or what
                                        crit_b200_merge folds */

/* -- split-K decode / speculative-verify attention ------------------------------------------------------------------
 * Replaces paged_kv_attention.attend (paged_kv_attention/__init__.py:396-576; kernels _kernels.py:263-478 and :558-604,
 * cuda_window.cu:284-1286) behind DeviceAttention._windows (inference/attention-state/code/device_attention.py:659-704).
 * R window rows; row r is counts[r] (NULL: `columns`; more than `columns` reads as `columns`) tokens starts[r].. of q
 * over the page table tables[rows[r]]; column c sits at position firsts[r] + c and sees positions 0..firsts[r] + c.
 * A row's positions are cut into contiguous splits of `chunk` positions; each split writes one partial state per
 * (token, query head) into `workspace`, and crit_b200_merge folds a row's splits in split order.  A row that fits one
 * split is written to out / lse by the first launch.  crit_b200_attend runs both launches. */
typedef struct crit_b200_attend_params {
    const void* q;               /* [tokens][q_heads][head_dim], bf16 or fp16 (q_dtype) */
    void* out;                   /* [tokens][q_heads][value_dim], q_dtype */
    float* lse;                  /* [tokens][q_heads] natural-log sum of exp of the scaled scores, or NULL */
    const void* key_pages;       /* [slots][kv_heads][head_dim] */
    const void* value_pages;     /* [slots][kv_heads][value_dim] */
    const float* key_scales;
    const float* value_scales;
    const int32_t* tables;       /* [S][table_stride] page ids */
    const int32_t* rows;         /* [R] */
    const int32_t* starts;       /* [R] */
    const int32_t* counts;       /* [R] or NULL */
    const int64_t* firsts;       /* [R] */
    const int32_t* offsets;      /* [R] first partial row of each row, counted from offsets[0]; or NULL (r * columns) */
    float* workspace;            /* crit_b200_attend_plan's floats, or NULL when max_splits is 1 */
    int32_t* status;             /* or NULL: a device word a kernel sets (never clears) when a bounded wait gave up */
    int64_t workspace_floats;
    int64_t slots;               /* slots each page tensor stores ((pages + 1) * page): the bound of the TMA tensor maps;
                                    0: unknown, pages are staged with cp.async and page ids are not range-checked */
    int64_t q_stride_token, q_stride_head, out_stride_token, out_stride_head, table_stride;
    int32_t n_rows, columns, partial_rows;
    int32_t q_heads, kv_heads, head_dim, value_dim, page;
    int32_t kind, page_dtype, q_dtype;
    int32_t chunk;               /* positions per split: a multiple of 16 */
    int32_t max_splits;          /* splits a partial row has room for: ceil(positions a row may reach / chunk) */
    int32_t flags;               /* CRIT_B200_ATTEND_* */
    float scale, key_multiplier, value_multiplier;
    const int32_t* parents;      /* NULL, or [tokens of q]: each token's parent COLUMN in its row, -1 for none (a draft tree,
                                    the columns in topological order): a column then sees the positions before its row's
                                    first and, of the window, itself and its ancestors instead of the columns before it
                                    (paged_kv_attention/_kernels.py:154-165, :325-329).  Served by the m16n8k16 kernel; a
                                    launch that names a tcgen05 kernel with parents is CRIT_B200_EUNSUPPORTED */
    const float* sinks;          /* NULL, or [q_heads] FP32: a sink logit a query head (in the units of the scaled scores), a
                                    position more without a value: the fold of a row's splits adds it to the maximum and the
                                    sum (and the lse), last.  The launch then takes the workspace whatever the splits
                                    (device_attention.py:1301-1335, _kernels.py:597-598); m16n8k16 kernel only */
    int32_t sliding;             /* 0, or the positions a column sees up to its own (a sliding window): positions at or
                                    below its own minus `sliding` are masked (_kernels.py:332-333); m16n8k16 kernel only */
    int32_t blocks_k, block_size;/* with `blocks`: ids a token lists, positions a block holds */
    const int32_t* blocks;       /* NULL, or [tokens of q][blocks_k] KV block ids, -1 for none: of what the other rules
                                    leave, a token sees only the positions of its listed blocks (block-sparse lists,
                                    _kernels.py:481-555; here as a mask: every position is still read); m16n8k16 kernel only */
} crit_b200_attend_params;

/* out[0] positions per split this library would choose (a multiple of 16), out[1] bytes of dynamic shared memory a
 * block takes, out[2] query rows a block's tile holds, out[3] blocks resident per SM, out[4] SMs of the device.
 * The partials of a launch take partial_rows * q_heads * max_splits * (value_dim + 2) floats, the reference's
 * workspace_floats (paged_kv_attention/__init__.py:359-362).  Returns 0, or CRIT_B200_EUNSUPPORTED. */
int crit_b200_attend_plan(int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t value_dim, int32_t page,
                          int32_t kind, int32_t page_dtype, int32_t columns, int32_t* out5);

int crit_b200_decode(const crit_b200_attend_params* params, void* stream);   /* the splits' partials */
int crit_b200_merge(const crit_b200_attend_params* params, void* stream);    /* the fold in split order */
int crit_b200_attend(const crit_b200_attend_params* params, void* stream);   /* both */

/* crit_b200_attend for callers that may not allocate device memory.  It has no counterpart in the reference (whose
 * launches always take their partials from a torch workspace or the engine's scratch).
 *
 * Some hosts of this library cannot call cudaMalloc on the path that runs attention: an engine that plans every device
 * byte at load and refuses allocation afterwards, a plugin sandbox that is given buffers but no allocator, a request
 * path that cannot afford the device-wide synchronisation an allocation implies.  For them the split-K partials live
 * in an array compiled into the library: CRIT_B200_STATIC_SCRATCH_FLOATS FP32 values (16 MiB) in every GPU's memory
 * from the moment the library is loaded there until the process exits.  params->workspace and workspace_floats are
 * ignored; every other field means what it means for crit_b200_attend, and the results are the same bits.
 *
 * Limit: partial_rows * q_heads * max_splits * (value_dim + 2) must not pass CRIT_B200_STATIC_SCRATCH_FLOATS, else the
 * call returns CRIT_B200_ESTATIC and launches nothing (raise `chunk` so rows take fewer splits, or attend fewer rows a
 * call).  The call itself allocates and frees nothing, on the device or through any library.
 * The first call on each device looks the array's device address up (with that device current) and keeps it; make that
 * first call before any stream capture begins.  All calls on a device share the one array and it keeps the previous
 * call's partials: nothing in it needs clearing, because a launch writes every partial it later reads, but two calls
 * that run on the GPU at the same time (different streams, threads or engines) race on it: run them one after another. */
#define CRIT_B200_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
int crit_b200_attend_static(const crit_b200_attend_params* params, void* stream);

/* -- merge of shards --------------------------------------------------------------------------------------------
 * Replaces PartitionedAttention.merge (inference/partitioned-attention/plugin.py:52-64; host form merge_partials,
 * code/implementation.py:119-138): parts partials of the same n (token, head) rows over disjoint keys,
 * outs [parts][n][dim] (FP32, or the in_dtype), lses [parts][n] FP32 (-inf: a part that saw no key) ->
 * out [n][dim] (out_dtype) and lse [n]; a row no part saw gets zeros and -inf. */
typedef struct crit_b200_merge_shards_params {
    const void* outs;
    const float* lses;
    void* out;
    float* lse;
    int64_t n;
    int32_t parts, dim, in_dtype, out_dtype;
} crit_b200_merge_shards_params;

int crit_b200_merge_shards(const crit_b200_merge_shards_params* params, void* stream);

/* -- the exchange of the shards' partials over peer memory ---------------------------------------------------------------
 * What an engine with one process per GPU runs between its ranks' partial attention and crit_b200_merge_shards, in place
 * of a collective library's all-gather (the reference leaves "partitioning and collectives" to the engine:
 * inference/partitioned-attention/README.md; its merge is plugin.py:52-64).  Every rank owns one exchange buffer of
 * crit_b200_exchange_bytes(world, floats) bytes, zeroed before the first step, that every rank has mapped; `peers` is a
 * DEVICE array of this GPU's addresses of all `world` buffers.  crit_b200_shard_push adds one to *step (a device
 * counter, so the pair is capturable in a CUDA graph), stores `mine` into every rank's buffer and raises this rank's flag
 * there; it never waits.  crit_b200_shard_wait waits at most wait_ns nanoseconds for the `world` messages of the step to
 * land in this rank's own buffer and copies them to gathered [world][floats] (the layout crit_b200_merge_shards reads);
 * when the wait runs out it copies nothing and sets *status (0x800 + rank).  Only stores cross NVLink. */
typedef struct crit_b200_exchange_params {
    const float* mine;           /* this rank's message, 16-byte aligned */
    const uint64_t* peers;       /* [world] device array of buffer addresses */
    int32_t* step;               /* device counter of steps, the same on every rank */
    float* gathered;             /* [world][floats] */
    int32_t* status;             /* or NULL */
    int64_t floats;
    int64_t wait_ns;
    int32_t world, rank;
} crit_b200_exchange_params;

int crit_b200_shard_push(const crit_b200_exchange_params* params, void* stream);
int crit_b200_shard_wait(const crit_b200_exchange_params* params, void* stream);
int64_t crit_b200_exchange_bytes(int32_t world, int64_t floats);

/* The same exchange with the arithmetic either side of it (what one decode step of a context sharded by KV range runs
 * after crit_b200_decode with CRIT_B200_ATTEND_PARTIALS): crit_b200_merge_push folds this rank's splits (the fold of
 * crit_b200_merge) and stores each (token, head)'s normalised output and log-sum-exp as FP32 straight into every rank's
 * buffer, every float in one 8-byte store with the step beside it, so a reader that finds its step has the value: no
 * flag, fence or header is involved and the exchange costs one NVLink write.  crit_b200_wait_merge gathers, for every
 * (token, head), the `world` ranks' floats from this rank's own buffer (a wait of at most wait_ns per float) and writes
 * the merge of shards to merge->out / merge->lse (merge->outs and ->lses are not read; parts = world).  A message is
 * tokens x q_heads x (value_dim + 1) floats + 3: exchange->floats says so, and the attend rows' tokens cover
 * 0 .. tokens - 1.  exchange->mine and ->gathered are not used; the buffers are crit_b200_exchange_bytes(world, floats)
 * bytes as for the plain pair.  A float that never arrives (a rank that stayed away, or one that ran a step ahead and
 * stored over the slot) sets the status word (0x800 + rank) and nothing of its (token, head) is written: the step's
 * output is then not published. */
int crit_b200_merge_push(const crit_b200_attend_params* attend, const crit_b200_exchange_params* exchange, void* stream);
int crit_b200_wait_merge(const crit_b200_exchange_params* exchange, const crit_b200_merge_shards_params* merge, void* stream);
/* Both in one launch where the step is small enough that every block of the launch is resident at once (a block per
 * (token, head), up to the device's SM count: each block folds and pushes its own pair, waits for the ranks' flags and
 * merges its own pair out of this rank's buffer), else the two launches above, one after the other. */
int crit_b200_exchange_merge(const crit_b200_attend_params* attend, const crit_b200_exchange_params* exchange,
                             const crit_b200_merge_shards_params* merge, void* stream);

/* -- chunked prefill ---------------------------------------------------------------------------------------------
 * Replaces paged_kv_attention.prefill (paged_kv_attention/__init__.py:1245-1332; kernel _kernels.py:610-726) behind
 * DeviceAttention._prefill_rows (device_attention.py:901-916): one sequence's chunk of `tokens` queries at positions
 * position.. (position_ptr, a device int64, wins over position when not NULL) over its page table, causal; the
 * chunk's keys and values are in the pages already.  16-bit pages of 128-wide heads run on tcgen05 tensor-core tiles
 * with TMEM accumulators (TMA-staged pages); every other geometry on m16n8k16 tiles. */
#define CRIT_B200_PREFILL_MMA_SYNC 1   /* the m16n8k16 kernel even where the tcgen05 kernel serves the geometry (0: tcgen05
                                          tiles for 16-bit pages of 128-wide heads, m16n8k16 tiles otherwise) */
#define CRIT_B200_PREFILL_TCGEN05  2   /* the tcgen05 kernel or CRIT_B200_EUNSUPPORTED */
#define CRIT_B200_PREFILL_SINGLE   4   /* with tcgen05 tiles: blocks of 128 query rows, two an SM, even for a launch large
                                          enough for the blocks of 256 rows (two halves over one ring of key and value
                                          tiles, one block an SM), which are the default from one such block an SM on */
#define CRIT_B200_PREFILL_PAIR     8   /* with tcgen05 tiles: the blocks of 256 rows however small the launch */

typedef struct crit_b200_prefill_params {
    const void* q;
    void* out;
    float* lse;                  /* or NULL */
    const void* key_pages;
    const void* value_pages;
    const float* key_scales;
    const float* value_scales;
    const int32_t* table;        /* [pages of the sequence] */
    const int64_t* position_ptr; /* or NULL */
    int32_t* status;             /* or NULL: set (never cleared) when a bounded wait of the tcgen05 kernel gave up */
    int64_t position;
    int64_t slots;               /* slots each page tensor stores ((pages + 1) * page), 0: unknown (no TMA, no tcgen05 path) */
    int64_t q_stride_token, q_stride_head, out_stride_token, out_stride_head;
    int32_t tokens, q_heads, kv_heads, head_dim, value_dim, page;
    int32_t kind, page_dtype, q_dtype;
    int32_t flags;               /* CRIT_B200_PREFILL_* */
    float scale, key_multiplier, value_multiplier;
    /* several sequences' chunks in one launch (sequences > 1): table is [sequences][table_stride], positions holds
     * each sequence's first new position, tokens is the most tokens a sequence brings, and lse is indexed like out */
    const int32_t* starts;       /* or NULL. [sequences + 1] on the device: sequence s's tokens are rows
                                    starts[s] .. starts[s + 1] of q and out (NULL: rows s * tokens .. of each) */
    const int64_t* positions;    /* [sequences] on the device; required when sequences > 1; when not NULL it wins over
                                    position_ptr and position for one sequence too */
    int32_t sequences;           /* 0 or 1: one sequence */
    int32_t table_stride;        /* ints between two sequences' tables */
} crit_b200_prefill_params;

int crit_b200_prefill(const crit_b200_prefill_params* params, void* stream);

/* -- the pool's page allocator (host code: no stream, no device memory) ------------------------------------------- */
/* A min-heap of the free page ids (the lowest free page is the next one taken: the order crit's pool keeps,
 * inference/attention-state/code/pages.py:721-741), a reference count per page (forks share pages until one writes)
 * and the floor (one past the highest page in use).  Not thread-safe: one pool, one caller at a time. */
void* crit_b200_pager_create(int32_t pages);                 /* NULL when pages < 1 or out of memory */
void crit_b200_pager_destroy(void* pager);
int32_t crit_b200_pager_take(void* pager);                   /* the lowest free page, its count 1; -1 when none is free */
int32_t crit_b200_pager_drop(void* pager, int32_t page);     /* one holder less: the count left (0: free again), -1 if not held */
int32_t crit_b200_pager_share(void* pager, int32_t page);    /* one holder more: the count, -1 if not held */
int32_t crit_b200_pager_refs(void* pager, int32_t page);
int32_t crit_b200_pager_free(void* pager);                   /* free pages */
int32_t crit_b200_pager_floor(void* pager);
int32_t crit_b200_pager_shared(void* pager);                 /* pages held more than once */
/* A step's rows grown at once: row i holds have[i] pages and needs need[i]; its new pages are taken in row order, lowest
 * free page first, into out (capacity entries).  Returns how many; -(taken + 1) when the pool ran out (the pages taken
 * so far stay taken and are in out). */
int64_t crit_b200_pager_grow(void* pager, int32_t rows, const int32_t* have, const int32_t* need, int32_t* out, int64_t capacity);

/* -- housekeeping ------------------------------------------------------------------------------------------------ */
int crit_b200_abi_version(void);
/* sizeof of each parameter block, in the order append, gather, slots, attend, merge_shards, prefill: a binding checks
 * its own struct layout against it (the reference's crit_cw_params_size, cuda_window.cu:1495-1497); 6 exchange, 7 move, 8 compact. */
int crit_b200_params_size(int32_t which);
const char* crit_b200_error(int32_t code);       /* host string; cudaGetErrorString for codes above 0 */
int crit_b200_device_sms(void);                  /* SMs of the current device, or a negative error */

#ifdef __cplusplus
}
#endif
#endif
