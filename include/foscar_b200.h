/* C ABI of libfoscar_b200: paged GQA decode attention over packed INT2/INT4 KV caches on
 * B200 (sm_100a). Plain pointers and sizes only; every launch is asynchronous on the given
 * CUDA stream (a cudaStream_t passed as void*). Return value: 0 on success, a negative
 * FQ_ERR_* for a refused argument, or a positive cudaError_t from the launch.
 *
 * The reference has no C ABI: its device entry points are TVM-FFI callables compiled from
 * CuTe-DSL. Each entry point below names the reference call it stands in for.
 *
 * Device-side faults never trap: a kernel that meets an out-of-range slot, page id, output row
 * or length, or a wait that ran out, skips the access and ORs a FQ_STATUS_* bit into the
 * caller's int32 status word (may be NULL).
 */
#ifndef FOSCAR_B200_H
#define FOSCAR_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FQ_PAGE_SIZE 64
#define FQ_VMAX_BINS 256

/* host-side refusals */
#define FQ_ERR_BAD_ARG (-1)
#define FQ_ERR_UNSUPPORTED (-2)
#define FQ_ERR_TOO_LARGE (-3)
#define FQ_ERR_SCRATCH_TOO_SMALL (-4) /* fq_decode_split_static: needs more than its static scratch */

/* device status bits */
#define FQ_STATUS_BAD_SLOT 0x1      /* append: slot >= num_pages * 64 (skipped) */
#define FQ_STATUS_BAD_PAGE 0x2      /* dequantize/decode: page id outside the pool (skipped) */
#define FQ_STATUS_BAD_ROW 0x4       /* dequantize: output row outside k_out/v_out (skipped) */
#define FQ_STATUS_BAD_LENGTH 0x8    /* negative length, or longer than the request's pages */
#define FQ_STATUS_TIMEOUT 0x10      /* a bounded device wait ran out; output is invalid */

/* One layer's pools (reference: QuantKVCache, src/foscar/kv_cache.py:477-533).
 * k_codes, v_codes: uint8 [num_pages, num_kv_heads, 64, head_dim*bits/8].
 * scales: [num_pages, num_kv_heads, 64, 4] (s_k,z_k,s_v,z_v) when k_groups == 1, else the
 *   sectioned block [num_pages, num_kv_heads, 2*k_groups*64 + 128]; f32 or bf16. With
 *   k_channel_group == 64 (k_groups 1) the block is [128 + 2*head_dim]: token t's (s_v, z_v) at
 *   2t, then the page's K channel rows s_d and z_d (src/foscar/quant_layout.py:9-21, 57-85).
 * v_page_max: uint32 [num_pages, num_kv_heads]; v_max_hist: uint32 [256]. */
typedef struct fq_pools {
  int32_t bits;          /* 2 or 4 */
  int32_t head_dim;      /* 64, 128 or 256 */
  int32_t num_kv_heads;
  int32_t k_groups;      /* head_dim / K token-wise group: 1, 2 or 4 */
  int32_t scale_bf16;    /* 0: f32 records, 1: bf16 records */
  int32_t num_pages;
  int32_t k_channel_group; /* 0: K per token; 64: K per channel over the 64 tokens of a page */
  int32_t reserved;
  uint8_t* k_codes;
  uint8_t* v_codes;
  void* scales;
  uint32_t* v_page_max;
  uint32_t* v_max_hist;
} fq_pools;

const char* fq_version(void);
const char* fq_error_string(int code);

/* Quantize bf16 K,V [T, HKV, D] (token strides in elements) and write them at slot_mapping
 * (int64 [T]; negative = skipped). k_clip/v_clip: order-statistic index of the per-row clip,
 * -1 for none. Stands in for QuantKVCache.append -> launch_writer
 * (src/foscar/kv_cache.py:618-687, src/foscar/_append_core.py:1320-1332). */
int fq_append(const fq_pools* pools, const void* k, const void* v, int64_t k_token_stride,
              int64_t v_token_stride, const int64_t* slot_mapping, int32_t num_tokens,
              int32_t k_clip, int32_t v_clip, int32_t* status, void* stream);

/* Layout-only write of engine-quantized tokens: codes uint8 [T, HKV, D] one value per byte,
 * f32 scales/zeros [T, HKV(, k_groups)]; the code pointers 4-byte aligned. Stands in for
 * QuantKVCache.append_quantized (src/foscar/kv_cache.py:689-767). */
int fq_append_quantized(const fq_pools* pools, const uint8_t* k_codes, const float* k_scale,
                        const float* k_zero, const uint8_t* v_codes, const float* v_scale,
                        const float* v_zero, const int64_t* slot_mapping, int32_t num_tokens,
                        int32_t* status, void* stream);

/* Quantize and write whole page groups of a cache whose K is quantized per channel over the 64
 * tokens of a page (k_channel_group == 64) and whose V is per token: k, v bf16, page i's tokens
 * being rows [64 i, 64 i + valid[i]) (token strides in elements); page_ids int32 [P]; valid
 * int32 [P] or NULL (all 64). K statistics run over a page's valid tokens only; code rows past
 * them are not written and their V records are cleared. A page that gains tokens is written
 * again with all of them. The reference has no counterpart: its append refuses these layouts
 * (src/foscar/kv_cache.py:643-644) although its decode reads them
 * (src/foscar/_sm100/int_fold_decode.py:5012-5036). */
int fq_append_page_groups(const fq_pools* pools, const void* k, const void* v,
                          int64_t k_token_stride, int64_t v_token_stride,
                          const int32_t* page_ids, const int32_t* valid, int32_t num_page_groups,
                          int32_t* status, void* stream);

/* The same page groups from an engine that quantized them itself (layout-only, the channel-wise
 * counterpart of fq_append_quantized): k_codes, v_codes uint8 [P * 64, HKV, D] one value per
 * byte, contiguous, 4-byte aligned; k_scale, k_zero f32 [P, HKV, D] (per page and channel);
 * v_scale, v_zero f32 [P * 64, HKV]; page_ids, valid as above. Codes are masked to the stored
 * width and records saturated like fq_append_quantized's. No reference counterpart
 * (QuantKVCache.append_quantized refuses these layouts, src/foscar/kv_cache.py:769-774). */
int fq_append_quantized_page_groups(const fq_pools* pools, const uint8_t* k_codes,
                                    const float* k_scale, const float* k_zero,
                                    const uint8_t* v_codes, const float* v_scale,
                                    const float* v_zero, const int32_t* page_ids,
                                    const int32_t* valid, int32_t num_page_groups,
                                    int32_t* status, void* stream);

/* Read K,V of a batch back into bf16 rows [N, HKV, D]: out[out_indptr[b]+t] =
 * bf16(fma(s, q, z)) for t < seq_lens[b]. Stands in for QuantKVCache.dequantize
 * (src/foscar/kv_cache.py:792-877). out_indptr is int32 or int64 (out_indptr_64). k_out and
 * v_out are 16-byte aligned and the row strides (in elements) multiples of 8. */
int fq_dequantize(const fq_pools* pools, void* k_out, void* v_out, int64_t k_row_stride,
                  int64_t v_row_stride, int64_t num_out_rows, const int32_t* page_indptr,
                  const int32_t* page_indices, int32_t num_entries, const int32_t* seq_lens,
                  const void* out_indptr, int32_t out_indptr_64, int32_t batch,
                  int32_t* status, void* stream);

/* Clear the sign bit of every v_page_max cell and rebuild v_max_hist from the cells. Stands
 * in for QuantKVCache.recount_v_max (src/foscar/kv_cache.py:595-616). */
int fq_recount_vmax(const fq_pools* pools, void* stream);

/* One decode step. Stands in for launch_fold / launch_fold_graph
 * (src/foscar/_sm100/fold_runtime.py:680-779).
 * A work item is (request, KV head, head tile, chunk of 128-token tiles). With worklist ==
 * NULL the items are implicit: every request is cut into `kv_splits` contiguous chunks by the
 * kernel from seq_lens. Otherwise worklist is the int32 list fq_plan_worklist writes: a header
 * {pieces, units, ctas, rows' word offset, rows carry their request (0/1), 0...},
 * cta_start[ctas + 1] (padded to 8 words), then one row per piece
 *   {request, kv_head, head_tile, tile_begin, tile_end, partial_slot, 0, 0}
 * (the last two words: the request's length and table offset once
 * fq_worklist_attach_requests has filled them in)
 * with partial_slot -1 = write the final output. CTA c runs rows [cta_start[c], cta_start[c+1]).
 * The header is read on the device, so a captured launch follows a list rewritten between
 * replays; launch with max_ctas = the plan's ctas.
 * Items with a partial slot write unnormalised f32 o_partial [max_splits, B, HQ, D] and
 * l_partial / m_partial [max_splits, B, HQ] (m in the log2 domain); fq_merge combines them. */
typedef struct fq_decode_args {
  int32_t batch;
  int32_t num_qo_heads;
  int32_t out_dtype;            /* 0 bf16, 1 f16, 2 f32 */
  int32_t kv_splits;            /* implicit mode: chunks per request, >= 1 */
  int32_t max_splits;           /* leading extent of the partial buffers */
  int32_t num_work;             /* explicit mode: most rows the list may hold */
  int32_t max_ctas;             /* grid cap; 0 = one CTA per SM */
  int32_t flags;                /* bit 0: launch with programmatic stream serialization (PDL): the
                                 * kernel's on-chip set-up overlaps the tail of the launch before it
                                 * in the stream; it waits for that launch before its first global
                                 * access (the reference's enable_pdl, wrapper.py:1111-1117) */
  float sm_scale;
  float o_scale;
  const int32_t* worklist;      /* NULL = implicit mode */
  const int32_t* seq_lens;      /* int32 [B] */
  const int32_t* page_table;    /* int32 flat page ids */
  const int32_t* table_offsets; /* int32 [B]: first entry of request b in page_table */
  int64_t table_len;            /* entries in page_table (bounds check) */
  const void* q;                /* fp8 e4m3 [B, HQ, D] */
  const float* q_descale;       /* NULL or f32, element (b,h) at b*stride_b + h*stride_h */
  int64_t q_descale_stride_b;
  int64_t q_descale_stride_h;
  void* out;                    /* [B, HQ, D] in out_dtype */
  float* lse;                   /* NULL or f32 [B, HQ], natural log */
  float* o_partial;
  float* l_partial;
  float* m_partial;
  int32_t* status;
  /* In-kernel merge of split units (optional). unit_counters: int32 [B * HKV * head_tiles],
   * zero before the first launch; each piece of a unit bumps its counter after writing its
   * partials, and the CTA that brings it to the unit's piece count merges the unit's partials
   * in slot order (the arithmetic of fq_merge), writes out/lse and sets the counter back to 0,
   * so no merge launch follows and the counters need no clearing between launches.
   * split_counts: int32 per unit, pieces of each unit in an explicit list (NULL: kv_splits). */
  int32_t* unit_counters;
  const int32_t* split_counts;
  /* Cycle budget of one device wait; 0 = the default (about a second). When a wait runs out the
   * CTA gives up, FQ_STATUS_TIMEOUT is set and the output is invalid; unit_counters may then be
   * left non-zero and must be cleared before the next launch. */
  int64_t wait_budget_cycles;
  /* Query tokens per request (speculative / multi-token decode); 0 or 1 = one. With q_len = L > 1
   * q and out are [B, L, HQ, D], lse is [B, L, HQ], q_descale element (b, l, h) sits at
   * (b*L + l)*stride_b + h*stride_h, seq_lens counts the L new tokens (already appended), and
   * query token l attends to positions < seq_lens[b] - (L - 1 - l). The L tokens of a KV head's
   * query heads share that head's KV stream as L * HQ/HKV columns of one unit, so head_tiles =
   * ceil(L * HQ/HKV / 8) for unit_counters, split_counts and the planners. Split units need
   * unit_counters (the in-kernel merge); fq_merge does not know this row order. The reference
   * refuses q_len_per_req != 1 (src/foscar/wrapper.py:756-761). */
  int32_t q_len;
  int32_t reserved;
} fq_decode_args;

int fq_decode(const fq_pools* pools, const fq_decode_args* args, void* stream);

/* Split decode plus merge for callers that cannot allocate device memory. It has no counterpart
 * in the reference, whose wrapper always takes the partial buffers from a caller-allocated
 * workspace. Some hosts of this library have no workspace to give: a plugin running inside an
 * engine that owns the CUDA allocator and forbids cudaMalloc from extensions, or a call site
 * inside a region where allocation is illegal (a stream capture, a real-time loop). For them the
 * unnormalised partials (o, l, m) of a uniform split (worklist == NULL, kv_splits >= 1) go into a
 * buffer of FQ_STATIC_SCRATCH_BYTES that is part of the library image itself, so every GPU that
 * loads the library carries those bytes until the process exits. The caller passes inputs and
 * outputs exactly as to fq_decode; o_partial/l_partial/m_partial/max_splits are ignored.
 *   - Limit: kv_splits * batch * num_qo_heads * (head_dim + 2) * 4 bytes must fit the buffer,
 *     else FQ_ERR_SCRATCH_TOO_SMALL is returned and nothing is launched.
 *   - The first call on each device looks the buffer's device address up; make that first call
 *     (with the device current) before any stream capture.
 *   - Calls no cudaMalloc, cudaFree or allocating library routine.
 *   - All calls share the one buffer, which keeps the previous call's partials. Nothing needs
 *     clearing (each call writes every slot it later reads), but two calls that overlap on the GPU
 *     (different streams, or graphs replayed concurrently) race on it: order them. */
#define FQ_STATIC_SCRATCH_BYTES (8u << 20)
int fq_decode_split_static(const fq_pools* pools, const fq_decode_args* args, void* stream);

/* Merge split partials in fixed slot order. split_counts NULL: every row combines slots
 * [0, kv_splits). Otherwise split_counts is int32 [B * HKV * head_tiles], the piece count of
 * each unit (request, KV head, tile of eight query heads): a unit with one piece wrote its final
 * output itself and is left alone. Stands in for launch_reduction
 * (src/foscar/_sm100/gqa_decode.py:377-456). */
int fq_merge(const float* o_partial, const float* l_partial, const float* m_partial,
             const int32_t* split_counts, int32_t kv_splits, int32_t max_splits, int32_t batch,
             int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim, float o_scale,
             void* out, int32_t out_dtype, float* lse, void* stream);

/* Merge attention states from several sequence shards: out = sum_r exp(lse_r - L) o_r,
 * L = logsumexp_r lse_r, o f32 [R, B, HQ, D], lse f32 [R, B, HQ] (natural log). The reference
 * has no counterpart (single-GPU library); this is the local half of the cross-GPU
 * sequence split. o_row_stride / lse_stride: elements between consecutive rows of o and of lse
 * (0: dense, D and 1), so that one gathered buffer of [R, B, HQ, D + 1] rows (o, then lse) can
 * be merged in place. */
int fq_merge_states(const float* o_shards, const float* lse_shards, int32_t num_shards,
                    int32_t batch, int32_t num_qo_heads, int32_t head_dim, void* out,
                    int32_t out_dtype, float* lse, int64_t o_row_stride, int64_t lse_stride,
                    void* stream);

/* The cross-GPU step of a sequence-split decode in one launch per rank: this rank's attention
 * state (o f32 [B, HQ, D] normalised, lse f32 [B, HQ] natural log) is written into a staging slot
 * in every rank's memory through peer-mapped pointers (plain stores), the step is posted on a flag
 * there, the peers' flags are waited for in this rank's own memory (bounded by
 * wait_budget_cycles, 0 = default; FQ_STATUS_TIMEOUT and an untouched output when a peer never
 * posts) and the gathered rows are merged locally as fq_merge_states merges them.
 * staging: host array of `world` device pointers, entry r being rank r's staging buffer of
 * fq_exchange_bytes bytes as mapped in this process (zeroed before the first step); step: 1, 2,
 * 3, ... the same on every rank, or 0 to count the steps on the device (every rank launching
 * the same number of times), which makes the launch replayable from a CUDA graph. The reference
 * has no counterpart (single-GPU library). */
int64_t fq_exchange_bytes(int32_t world, int32_t batch, int32_t num_qo_heads, int32_t head_dim);
int fq_exchange_merge(void* const* staging, int32_t rank, int32_t world, const float* o_local,
                      const float* lse_local, int32_t batch, int32_t num_qo_heads,
                      int32_t head_dim, int64_t step, void* out, int32_t out_dtype,
                      float* lse_out, int64_t wait_budget_cycles, int32_t* status, void* stream);

/* Host-only planning. fq_plan_splits: uniform split count for the longest request (closed-form
 * cost model; stands in for plan_splits_sm100, src/foscar/_sm100/scheduler.py:129-160).
 * fq_plan_worklist: balanced pieces from host seq_lens: writes the list (at most max_words int32
 * words; fq_worklist_words gives the size that always suffices) and the piece count of each
 * unit into split_counts [B * HKV * head_tiles]; returns the number of pieces, or a negative
 * FQ_ERR_* (FQ_ERR_TOO_LARGE when a unit would need more than max_splits pieces). `bits` (2 or
 * 4) and `head_dim` set the tokens of a tile (fq_tile_tokens) and the cost of a tile against the
 * fixed cost of a piece (fq_piece_overhead, in tiles). No unit gets more than max_splits pieces:
 * the planner raises every CTA's share until the longest unit fits. fq_tile_tokens has no
 * reference counterpart (the reference's tile is fixed per build,
 * src/foscar/_sm100/int_fold_decode.py:1509-1530). */
int fq_plan_splits(int32_t batch, int32_t num_kv_heads, int32_t head_tiles, int32_t max_kv_len,
                   int32_t bits, int32_t head_dim, int32_t sm_count);
int fq_plan_worklist(const int32_t* seq_lens, int32_t batch, int32_t num_kv_heads,
                     int32_t head_tiles, int32_t num_ctas, int32_t max_splits,
                     int32_t* worklist, int32_t max_words, int32_t* split_counts,
                     int32_t bits, int32_t head_dim);
int64_t fq_worklist_words(int32_t batch, int32_t num_kv_heads, int32_t head_tiles,
                          int32_t num_ctas);
/* Host-only, optional: write every row's request length and page-table offset into the row's
 * two spare words (from host copies of seq_lens and table_offsets, [batch] each) and set header
 * word 4, so that the kernel takes them from the row instead of from fq_decode_args.seq_lens /
 * table_offsets: one dependent global round trip less before a CTA's first tile (about a
 * microsecond of a launch that starts with a cold L2). The lengths given here then count, not
 * the device array's; a list without the mark is read as before. No reference counterpart. */
int fq_worklist_attach_requests(int32_t* worklist, int64_t words, const int32_t* seq_lens,
                                const int32_t* table_offsets, int32_t batch);
int fq_tile_tokens(int32_t bits, int32_t head_dim);
/* CTAs of the decode kernel that share an SM in this build of the library (1 or 2): a planner
 * gives fq_plan_worklist / fq_plan_splits that many times the device's SM count. */
int fq_ctas_per_sm(int32_t bits, int32_t head_dim);
int fq_piece_overhead(int32_t bits, int32_t head_dim);
int64_t fq_workspace_bytes(int32_t max_splits, int32_t batch, int32_t num_qo_heads,
                           int32_t head_dim);

/* Tensor-core self test: runs one 128-token tile of both contractions on known operands and
 * writes the raw accumulators (f32 [128][16] each) for the host to compare. mode 0: K operand
 * from tensor memory; mode 1: K operand from shared memory. */
int fq_umma_selftest(int32_t mode, const uint8_t* k_bytes, const uint8_t* q_bytes,
                     const uint8_t* v_bytes, const uint8_t* p_bytes, float* s_out, float* o_out,
                     int32_t* status, void* stream);

/* Wait self test: one small kernel whose threads wait, with the given cycle budget, for a
 * barrier phase that nothing completes. The wait runs out, the kernel sets FQ_STATUS_TIMEOUT in
 * *status and 1 in *gave_up and returns; the context stays usable. It exercises the give-up path
 * every bounded device wait of this library shares (the reference traps instead,
 * src/foscar/_sm100/int_fold_decode.py:131-175). */
int fq_wait_selftest(int64_t budget_cycles, int32_t* status, int32_t* gave_up, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FOSCAR_B200_H */
