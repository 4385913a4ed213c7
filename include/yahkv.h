/* yahkv: the paged, quantized KV-cache path of yet-another-halo-engine for NVIDIA B200 (sm_100a), as a C ABI.
 *
 * The reference engine has no FFI for this path: its "operator API" is a struct of buffer views plus kernel launches
 * by name with an ordered binding list. Each entry point below names the reference interface it stands in for
 * (paths relative to the reference project's root). One context serves one GPU and, like the reference engine
 * (engine/model/generator.hpp:56), is not reentrant: callers serialise calls on a context. Every call returns 0 or a
 * negative YAHKV_ERR_* code; nothing throws across this boundary and nothing is launched after a failed check
 * (the reference validates before launching, engine/model/loom_decoder.hpp:186-209, :230-234).
 *
 * Geometry is the engine's: 24 query heads, 4 KV heads (GQA 6), head_dim 256 (engine/model/loom_decoder.hpp:55-57),
 * score scale 1/16, optional sigmoid output gate. Pages hold 64 tokens. Cache formats are GGUF q8_0 / q4_0 blocks of
 * 32 elements with fp16 scales (engine/core/gguf_quant.cpp:310-320, :72-75, :48-51).
 *
 * Pool layout (per layer, per side K|V; all layers of a side live in one allocation):
 *   codes  [num_pages][4 kv heads][64 tokens][256 B (q8_0) | 128 B (q4_0)]
 *   scales [num_pages][4 kv heads][64 tokens][8] fp16
 * In device memory the q8_0 K codes are GGUF's int8 bytes as they are (the attention kernel feeds them to the integer
 * tensor-core MMA untouched); a q8_0 V code byte is held with its sign bit flipped (u = code + 128), which saves the
 * attention kernels an instruction per four codes. yahkv_read_page / yahkv_write_page / yahkv_export_token and the
 * snapshot files translate, so everything outside the device sees GGUF's int8 codes. Only
 * yahkv_attend_decode_noalloc, which is handed device pools directly, sees the device form. q4_0 bytes are GGUF's as
 * they are.
 * slot(pos) = table[pos / 64] * 64 + pos % 64 (the reference's rule with 256 -> 64,
 * engine/gpu/loom/tools/gen_decode_attn.py:5, :64-72). One block table per sequence is shared by all layers
 * (docs/architecture.md:212).
 */
#ifndef YAHKV_H_
#define YAHKV_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define YAHKV_FMT_Q8_0 0
#define YAHKV_FMT_Q4_0 1
/* The reference's own kv8a16 cache format (engine/gpu/loom/tools/gen_kvq.py:166-285, :474-660;
 * docs/architecture.md:210-230), on 64-token pages of four 16-key tiles (the reference uses 256-token pages):
 *   K  per token, minus a per-channel mean fixed per (sequence, layer): per (head, 128-dim half) an int8 scale,
 *      codes u = roundeven((k - mean) / s) + 128, dwords of four dims in byte slots (d0, d2, d1, d3), fp16 pair
 *      (256 s, -384 s);  pools: codes [page][4][64][256 B], pairs [page][4][64][2][2] fp16.
 *   V  per (16-key tile, channel): centre and scale over the tile's keys, codes in four dwords per channel
 *      (dword w byte p = key 4w + (0, 2, 1, 3)[p]), fp16 pair (256 sf, cf - 384 sf);
 *      pools: codes [page][4][4 tiles][256][16 B], pairs [page][4][4][256][2] fp16.
 *   The tile of a sequence's newest key stays in fp16 (the "open tile", engine/gpu/loom/tools/gen_decode_attn.py:426-427)
 *   and attention reads it from there; a tile is quantized when its 16th key arrives.
 * 2336 B per token per layer. Supported with this format: yahkv_append, yahkv_attend_decode, yahkv_attend_prefill
 * (its dequantize pass reads the tile of each sequence's newest key from the open buffer, the others from the pools),
 * the host-buffer decode steps, yahkv_read_page / yahkv_write_page, yahkv_seq_set_kmean, yahkv_read_open_tile,
 * yahkv_snapshot_save / yahkv_snapshot_load (pages plus, per layer, the mean and the open tile), decode batches
 * (yahkv_batch_*; the layers of a sequence must have been appended with the same calls), yahkv_rope_append (the RoPE
 * kernel leaves fp16 rows for the format's own append kernels). Not supported (refused with YAHKV_ERR_INVALID):
 * yahkv_export_token, yahkv_append_slots, head-sharded contexts, and yahkv_seq_set_len to anything but 0. */
#define YAHKV_FMT_KV8A16 2
/* Its 4-bit sibling kv4a16 (engine/gpu/loom/tools/gen_kvq.py:288-463, :474-660 with 4-bit V), same pages, tiles, open
 * tile, mean and supported calls as YAHKV_FMT_KV8A16:
 *   K  (k - mean) per head through the orthonormal Walsh-Hadamard transform H256 / 16 (in f32: butterflies 1, 2, 4 dims
 *      apart, then 8 .. 128), per 32-dim group of the rotated row lo = min, s = (max - lo) / 15,
 *      u = clamp(roundeven((r - lo) / s), 0, 15); a dword holds 8 dims, dim 2j at bits 4j, dim 2j + 1 at bits 16 + 4j;
 *      fp16 pair (16 s, lo - 16 s);  pools: codes [page][4][64][128 B], pairs [page][4][64][8][2] fp16. Attention rotates
 *      the query the same way (prefill attention rotates the cached rows back instead), so q.k is unchanged.
 *   V  per (16-key tile, channel) 15 levels: u = clamp(roundeven((v - cf) / sf) + 7, 0, 14), two dwords per channel
 *      (nibble p of dword w = key 8w + 2p for p < 4, 8w + 2(p - 4) + 1 otherwise), fp16 pair (16 sf, cf - 23 sf);
 *      pools: codes [page][4][4 tiles][256][8 B], pairs [page][4][4][256][2] fp16.
 * 1408 B per token per layer. */
#define YAHKV_FMT_KV4A16 3
/* Unquantized fp16 pages, the reference's fp16 cache mode (dattn_kvappend / dattn_part,
 * engine/gpu/loom/tools/gen_decode_attn.py:30-94, :97-335): K and V rows as they arrive, token-major on both sides
 * (the reference keeps V transposed in 16-key tiles; here V is token-major like the GGUF formats), no scale pools.
 * pools: [page][4][64 tokens][512 B] per side; 4096 B per token per layer. Every call of the GGUF formats works except
 * yahkv_export_token (there is no block form: use yahkv_read_page; its scales argument receives nothing). */
#define YAHKV_FMT_F16 4

#define YAHKV_SIDE_K 0
#define YAHKV_SIDE_V 1

#define YAHKV_OUT_F16 0
#define YAHKV_OUT_F32 1

#define YAHKV_OK 0
#define YAHKV_ERR_INVALID (-1)   /* bad argument, id, size or table entry */
#define YAHKV_ERR_NO_PAGES (-2)  /* the page pool is exhausted */
#define YAHKV_ERR_CUDA (-3)      /* a CUDA call failed; the message carries its text */
#define YAHKV_ERR_NO_DEVICE (-4) /* a hot-path call on a host-only context, or no usable GPU */
#define YAHKV_ERR_ORDER (-5)     /* positions appended out of order, or attend before any append */
#define YAHKV_ERR_CAPACITY (-6)  /* more sequences, pages per sequence, tokens or splits than configured */

typedef struct yahkv_ctx yahkv_ctx;

typedef struct yahkv_config {
  int32_t device;            /* CUDA ordinal; -1 = host-only context: allocator and tables work, hot calls fail */
  int32_t n_layers;          /* full-attention layers sharing the block tables */
  int32_t n_q_heads;         /* 24 */
  int32_t n_kv_heads;        /* 4 */
  int32_t head_dim;          /* 256 */
  int32_t page_tokens;       /* 64 */
  int32_t num_pages;         /* physical pages per layer */
  int32_t fmt;               /* YAHKV_FMT_* */
  int32_t max_seqs;          /* live sequences */
  int32_t max_pages_per_seq; /* block table width */
  int32_t max_splits;        /* split-K units per (sequence, kv head); 0 = 64 */
  int32_t max_batch_tokens;  /* tokens per append call and query rows per prefill call; 0 = 8192 */
  float softmax_scale;       /* 0 = 1/16 */
  /* Head-sharded layout (benchmark only): the context serves KV heads [kv_head_begin, kv_head_begin + kv_head_count)
   * and their query heads (6 per KV head); count 0 = all four. Appends skip the other heads' K/V, decode and prefill
   * attention write only the owned query heads' rows of `out` and leave the rest untouched, so ranks holding
   * disjoint head ranges of the same sequences produce disjoint slices of one output. Decode batches
   * (yahkv_batch_*) need all four heads. */
  int32_t kv_head_begin;
  int32_t kv_head_count;
  /* Cached keys (chunk included, summed over the sequences of one call, each rounded up to whole pages) that one
   * yahkv_attend_prefill call may cover. > 0: the fp16 scratch of the prefill dequantize pass (4 KB per key) is
   * allocated once at yahkv_create and a larger call is refused with YAHKV_ERR_CAPACITY, so the call never
   * allocates or synchronises. 0: the scratch grows to the largest call seen, which costs a device synchronisation
   * and a reallocation whenever the high-water mark rises. */
  int32_t max_prefill_keys;
} yahkv_config;

/* Replaces LoomDecoder::OwnState / LoomPrefill's pool allocation (engine/model/loom_decoder.hpp:159-183,
 * engine/model/loom_prefill.hpp:1306-1318): allocates the pools, the device block tables and the split-K workspace
 * once, zero-filled. On failure *out is NULL and yahkv_last_error(NULL) holds the reason. */
int yahkv_create(const yahkv_config* cfg, yahkv_ctx** out);
void yahkv_destroy(yahkv_ctx* ctx);
/* Message of the last failed call on ctx (ctx == NULL: of the last failed yahkv_create). Never NULL. */
const char* yahkv_last_error(const yahkv_ctx* ctx);
const char* yahkv_error_name(int code);

/* ---- host page allocator and block tables ------------------------------------------------------------------
 * The reference has one sequence and an identity table (engine/model/loom_decoder.hpp:175-179); its checkers
 * scramble the table (engine/gpu/loom/tools/dattn_q_check.py:151). Here a LIFO free list hands out pages; the host
 * copy of every table is the truth and changed rows reach the device as async copies ahead of the next hot call. */
int yahkv_seq_create(yahkv_ctx* ctx, int32_t* seq);
/* Returns the sequence's pages to the pool. Work already queued for it must have been ordered before (same stream). */
int yahkv_seq_free(yahkv_ctx* ctx, int32_t seq);
/* Grows the table so positions < n_tokens have a page. YAHKV_ERR_NO_PAGES leaves the sequence unchanged. */
int yahkv_seq_reserve(yahkv_ctx* ctx, int32_t seq, int64_t n_tokens);
/* Tests and imports: replace the table with caller-chosen pages (each in [0, num_pages), none owned by another
 * sequence; the reference's check is engine/model/loom_prefill.hpp:1314-1316). Pages the sequence held are freed. */
int yahkv_seq_set_table(yahkv_ctx* ctx, int32_t seq, const int32_t* pages, int32_t n);
int yahkv_seq_table(const yahkv_ctx* ctx, int32_t seq, const int32_t** pages, int32_t* n);
/* Appended length of a sequence in one layer (= highest appended position + 1). */
int yahkv_seq_len(const yahkv_ctx* ctx, int32_t seq, int32_t layer, int64_t* len);
/* Declare the length (after yahkv_append_slots, or to roll a sequence back to a prefix). layer -1 = all layers. */
int yahkv_seq_set_len(yahkv_ctx* ctx, int32_t seq, int32_t layer, int64_t len);
int yahkv_pages_free(const yahkv_ctx* ctx, int32_t* n);
/* YAHKV_FMT_KV8A16 only. Sets the per-channel K mean of a sequence in one layer (layer -1 = all): mean_host [4][256]
 * f32, subtracted from every K row before it is quantized. Replaces the reference's yah_kmean dispatch
 * (engine/gpu/loom/tools/gen_kvq.py:99-163, computed there from the first prefill chunk; zeros when the decoder owns
 * the state, engine/model/loom_decoder.hpp:46): here the caller supplies it, before the sequence's first append;
 * a fresh sequence has mean 0. Blocks. */
int yahkv_seq_set_kmean(yahkv_ctx* ctx, int32_t seq, int32_t layer, const float* mean_host);
/* YAHKV_FMT_KV8A16 only (inspection): the current open tile of (seq, layer) as [4][256][16] fp16; key j of the tile
 * that holds the newest position is column j, columns past the sequence's length are stale. Blocks. */
int yahkv_read_open_tile(yahkv_ctx* ctx, int32_t seq, int32_t layer, void* tile_host);

/* ---- hot path (asynchronous on `stream`, a cudaStream_t; NULL = the context's own stream) -------------------- */

/* Replaces dattn_kvappend / dattn_kappend_q + dattn_vappend_q (engine/model/loom_decoder.hpp:254-264) and the chunk
 * writers yah_kq8 / yah_vq8 (engine/model/loom_prefill.hpp:3346-3366): quantizes n_tokens fp16 K and V rows
 * ([n_tokens][4][256], device) and scatters them through the block tables. seq_ids / positions are host arrays; each
 * sequence's positions must continue its length in this layer (the q8_0 analogue of the reference's contiguity rule,
 * engine/model/loom_decoder.hpp:233-234) and be covered by yahkv_seq_reserve. */
int yahkv_append(yahkv_ctx* ctx, int32_t layer, int32_t n_tokens, const int32_t* seq_ids, const int64_t* positions,
                 const void* k_dev, const void* v_dev, void* stream);
/* Replaces the reference's "rope" kernel together with the appends that follow it (QK RMSNorm + NeoX RoPE on 64 of
 * 256 dims, theta 1e7, then dattn_kappend_q / dattn_vappend_q: engine/gpu/loom/yah_fused_qk_rope_f32.loom:1-9, :32,
 * engine/model/loom_decoder.hpp:250-261) in one launch. q_dev [n][24][256], k_dev, v_dev [n][4][256] f32 as the
 * projections produce them; q_weight_dev, k_weight_dev [256] f32 norm weights; eps the norm epsilon.
 *   K: normed, rotated, rounded to fp16, quantized and scattered exactly as yahkv_append would store that fp16 row;
 *   V: rounded to fp16, quantized and scattered;  q_out_dev [n][24][256] fp16: normed, rotated q for yahkv_attend_*
 *   (NULL: no q output, for callers that hand the raw q to yahkv_attend_prefill_qraw).
 * seq_ids / positions and the order rule as in yahkv_append. */
int yahkv_rope_append(yahkv_ctx* ctx, int32_t layer, int32_t n_tokens, const int32_t* seq_ids, const int64_t* positions,
                      const float* q_dev, const float* k_dev, const float* v_dev, const float* q_weight_dev,
                      const float* k_weight_dev, float eps, void* q_out_dev, void* stream);

/* The same with a device-resident slot mapping (slot = page * 64 + token in page; negative = skip the token).
 * Lengths are not tracked by this call: declare them with yahkv_seq_set_len. */
int yahkv_append_slots(yahkv_ctx* ctx, int32_t layer, int32_t n_tokens, const int64_t* slot_mapping_dev,
                       const void* k_dev, const void* v_dev, void* stream);

/* Replaces dattn_part(_q) + dattn_reduce (engine/model/loom_decoder.hpp:259-268): one query token per sequence over
 * keys 0 .. len-1 of that sequence in `layer` (append first, then attend: engine/gpu/loom/tools/gen_decode_attn.py:7).
 * q_dev [n_seqs][24][256] fp16; gate_dev [n_seqs][24][256] f32 or NULL (out *= sigmoid(gate), gen_decode_attn.py:402-407);
 * out_dev [n_seqs][24][256] fp16 or f32 by out_dtype. n_splits: split-K units per (sequence, kv head), 0 = automatic. */
int yahkv_attend_decode(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const void* q_dev,
                        const float* gate_dev, void* out_dev, int32_t out_dtype, int32_t n_splits, void* stream);

/* The same on the raw f32 q projection (q_raw_dev [n_seqs][24][256] f32): the attention kernel's prologue norms every
 * head row (RMS over its 256 dims, x q_weight_dev [256] f32, epsilon eps), rotates it at the position of the
 * sequence's newest key (len - 1: append first) and rounds it to fp16 with the arithmetic of yahkv_rope_append, so the
 * result has the bits of yahkv_rope_append's q_out_dev followed by yahkv_attend_decode. The attend-side half of the
 * reference's norm + RoPE fusion (engine/gpu/loom/yah_fused_qk_rope_f32.loom:1-9; gen_attn_fa.py:56-61 for prefill).
 * q_raw_dev and q_weight_dev 16-byte aligned. */
int yahkv_attend_decode_qraw(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const float* q_raw_dev,
                             const float* q_weight_dev, float eps, const float* gate_dev, void* out_dev,
                             int32_t out_dtype, int32_t n_splits, void* stream);

/* Replaces yah_attn_wmma (engine/model/loom_prefill.hpp:3393-3447): causal attention of one chunk per sequence over
 * the cache, which already holds the chunk (append first). Sequence i contributes chunk_lens[i] query rows, packed in
 * order: q_dev [sum chunk_lens][24][256] fp16; row j of sequence i sits at position len_i - chunk_lens[i] + j and sees
 * keys <= that position (engine/gpu/loom/tools/gen_attn_fa.py:2897-2904). gate / out as above, same packing. */
int yahkv_attend_prefill(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids,
                         const int32_t* chunk_lens, const void* q_dev, const float* gate_dev, void* out_dev,
                         int32_t out_dtype, void* stream);

/* The same with the query side of the fused norm + RoPE done in the attention kernel's prologue, as the reference's
 * prefill kernel does with its QNORM option (engine/gpu/loom/tools/gen_attn_fa.py:56-61): q_raw_dev
 * [sum chunk_lens][24][256] f32 is the raw q projection; every row is normed (RMS over its 256 dims, x q_weight_dev
 * [256] f32, epsilon eps), rotated at its position (len_i - chunk_lens[i] + j) and rounded to fp16 with the
 * arithmetic of yahkv_rope_append, so the result has the bits of yahkv_rope_append's q_out_dev followed by
 * yahkv_attend_prefill. Call yahkv_rope_append first for K and V (its q_out_dev may then be NULL). */
int yahkv_attend_prefill_qraw(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids,
                              const int32_t* chunk_lens, const float* q_raw_dev, const float* q_weight_dev, float eps,
                              const float* gate_dev, void* out_dev, int32_t out_dtype, void* stream);

/* One decode step of one layer with HOST buffers (what an engine without device-resident activations calls):
 * copies k/v/q (and gate) in, appends one token per sequence at its current length, attends, copies out back and
 * waits for it. k_host, v_host [n_seqs][4][256] fp16; q_host [n_seqs][24][256] fp16; out_host by out_dtype. */
int yahkv_decode_step_host(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const void* k_host,
                           const void* v_host, const void* q_host, const float* gate_host, void* out_host,
                           int32_t out_dtype);
/* The same step queued without waiting, so that a host which already holds the next layer's (or step's) inputs can
 * queue it while this one runs: the copies go on the context's own copy-in and copy-out streams around the kernels,
 * over two sets of staging buffers used in turn (the engine queues work the same way and waits only on the events it
 * needs, engine/model/engine.hpp:210-225). The host buffers must be page-locked and stay untouched until
 * yahkv_decode_step_host_wait returns, which waits for every queued read-back and reports a kernel that gave up. */
int yahkv_decode_step_host_async(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids,
                                 const void* k_host, const void* v_host, const void* q_host, const float* gate_host,
                                 void* out_host, int32_t out_dtype);
int yahkv_decode_step_host_wait(yahkv_ctx* ctx);

/* ---- inspection (parity tests, checkpoints); these block until the context's queued work is done ------------- */

/* One page record of one layer and side: codes [4][64][256|128] bytes to codes_host, scales [4][64][8] fp16 to
 * scales_host (either may be NULL). YAHKV_FMT_KV8A16: K codes [4][64][256], K pairs [4][64][2][2] fp16; V codes
 * [4][4][256][16], V pairs [4][4][256][2] fp16. The reference's checkers read whole pools back the same way
 * (engine/gpu/loom/tools/dattn_q_check.py:219-220). */
int yahkv_read_page(yahkv_ctx* ctx, int32_t layer, int32_t side, int32_t page, void* codes_host, void* scales_host);
int yahkv_write_page(yahkv_ctx* ctx, int32_t layer, int32_t side, int32_t page, const void* codes_host,
                     const void* scales_host);
/* The token at (seq, pos) as GGUF blocks, 4 heads x 8 blocks of [fp16 d][codes] (34 or 18 bytes each), the form
 * QuantizeQ8_0 writes (engine/core/gguf_quant.cpp:310-320). k_blocks / v_blocks may be NULL. */
int yahkv_export_token(yahkv_ctx* ctx, int32_t layer, int32_t seq, int64_t pos, void* k_blocks, void* v_blocks);
int yahkv_sync(yahkv_ctx* ctx);

/* ---- device-resident decode batches (CUDA-graph friendly) -----------------------------------------------------
 * The reference queues decode steps back to back with no host round trip: positions come from a device array
 * (engine/model/loom_decoder.hpp:131-133, :239; docs/architecture.md:171). A yahkv_batch is the batched analogue: the
 * lengths of a fixed set of sequences live on the device, and small kernels derive each step's slots and split-K
 * units from them, so plan / decode_layer / advance touch no host state and can be stream-captured into a CUDA graph
 * once and replayed.
 *   batch_create        the sequences must have equal lengths in all layers; allocates the batch's device arrays.
 *   batch_prepare       NOT capturable. Reserves pages for the next horizon_steps positions, uploads block tables and
 *                       lengths, and fixes the pages per split-K unit and the units per sequence for that horizon.
 *                       *layout_changed = 1 when either changed, i.e. a captured graph must be captured again.
 *   batch_plan          capturable; once per step: slots of the new tokens and the step's units from the lengths.
 *   batch_decode_layer  capturable; per layer: append k/v [n][4][256] fp16 at the planned slots, then attend with
 *                       q [n][24][256] over lengths + 1 keys (rows in batch_create's order).
 *   batch_advance       capturable; once per step: lengths += 1 on the device.
 *   batch_commit        host side: tells the context that `steps` steps have been queued (eagerly or by replaying a
 *                       graph), so sequence lengths and later non-batch calls see them. At most the prepared horizon. */
typedef struct yahkv_batch yahkv_batch;
int yahkv_batch_create(yahkv_ctx* ctx, int32_t n_seqs, const int32_t* seq_ids, yahkv_batch** out);
void yahkv_batch_destroy(yahkv_batch* batch);
/* Split-K units per (sequence, kv head) for the batch's longest sequence, as n_splits of yahkv_attend_decode (0 =
 * automatic, the default); shorter sequences get units of the same page count. Takes effect at the next batch_prepare. */
int yahkv_batch_set_splits(yahkv_batch* batch, int32_t n_splits);
int yahkv_batch_prepare(yahkv_batch* batch, int32_t horizon_steps, int32_t* layout_changed, void* stream);
int yahkv_batch_plan(yahkv_batch* batch, void* stream);
int yahkv_batch_decode_layer(yahkv_batch* batch, int32_t layer, const void* k_dev, const void* v_dev, const void* q_dev,
                             const float* gate_dev, void* out_dev, int32_t out_dtype, void* stream);
/* batch_decode_layer on the raw f32 projections (capturable; q_dev [n][24][256], k_dev, v_dev [n][4][256] f32, norm
 * weights [256] f32, epsilon eps): the reference's whole per-layer attention section in the engine's own terms
 * (rope, append, part, reduce with the position on the device: engine/model/loom_decoder.hpp:250-268, :131-133).
 * K is normed, rotated at the sequences' device-resident positions and appended with V as yahkv_rope_append does; the
 * query side is done in the part kernel's prologue as in yahkv_attend_decode_qraw. The cos / sin table is built by the
 * first call that needs it, which therefore cannot be inside a capture: run one step eagerly (or any
 * yahkv_rope_append) first. q_dev and q_weight_dev 16-byte aligned. */
int yahkv_batch_decode_layer_raw(yahkv_batch* batch, int32_t layer, const float* q_dev, const float* k_dev,
                                 const float* v_dev, const float* q_weight_dev, const float* k_weight_dev, float eps,
                                 const float* gate_dev, void* out_dev, int32_t out_dtype, void* stream);
int yahkv_batch_advance(yahkv_batch* batch, void* stream);
int yahkv_batch_commit(yahkv_batch* batch, int32_t steps);

/* Cache snapshots (the reference's LoomPrefill::SaveState / LoadState, engine/model/loom_prefill.hpp:973-1024, for
 * this path's state): the listed sequences with their per-layer lengths and every page they reference, stored in
 * logical page order, so a load takes fresh pages from the free list and may land anywhere in the pool. A snapshot
 * loads only into a context of the same format, layer count and geometry. Both calls block. On load, seq_ids_out
 * receives the new sequence ids in the saved order; *n_inout is the array's capacity on entry, the count on return;
 * a failed load leaves no sequence behind. */
int yahkv_snapshot_save(yahkv_ctx* ctx, int32_t n_seqs, const int32_t* seq_ids, const char* path);
int yahkv_snapshot_load(yahkv_ctx* ctx, const char* path, int32_t* seq_ids_out, int32_t* n_inout);

/* Bytes of device memory the context holds, and kernels it has launched since creation (for benchmarks). */
int yahkv_device_bytes(const yahkv_ctx* ctx, int64_t* bytes);
int yahkv_launch_count(const yahkv_ctx* ctx, int64_t* launches);

/* ---- test hooks ------------------------------------------------------------------------------------------------
 * yahkv_debug_wait_timeout runs the give-up path of the library's bounded device waits on purpose: one small kernel
 * waits at most limit_us microseconds (1 .. 1,000,000) on a barrier nobody arrives at, stops waiting, records the
 * sticky status word and returns, so the next yahkv_sync fails with YAHKV_ERR_CUDA and clears it. The reference bounds
 * its device-side polls the same way and leaves a sticky status (engine/gpu/loom/tools/gen_chain.py:12-19). Nothing
 * traps or faults, the context stays usable.
 * yahkv_debug_set_prefill_sms sets the number of SMs whose last partly filled wave the prefill planner splits along
 * the keys (0 = never split, at most the device's count; the default is twice the number of CTA pairs the device
 * runs at once). The kernel runs CTA pairs, so the wave is n_sm / 2 pairs. A small test reaches the split and merge
 * path this way. */
int yahkv_debug_wait_timeout(yahkv_ctx* ctx, int64_t limit_us, void* stream);
int yahkv_debug_set_prefill_sms(yahkv_ctx* ctx, int32_t n_sm);

/* Per-kernel device time for benchmarks: while enabled, every launch is bracketed by a CUDA event pair on its own
 * stream (the reference's counterpart is its per-dispatch timer, engine/run/hal_run.cc:124-135). Enabling or
 * disabling clears the record. _read waits for the device and sums the pairs of one kernel. */
#define YAHKV_KERNEL_APPEND 0
#define YAHKV_KERNEL_DECODE_PART 1
#define YAHKV_KERNEL_DECODE_COMBINE 2
#define YAHKV_KERNEL_PREFILL 3
#define YAHKV_KERNEL_PREFILL_DEQUANT 4
#define YAHKV_KERNEL_COUNT 5
int yahkv_kernel_timing(yahkv_ctx* ctx, int32_t enable);
int yahkv_kernel_timing_read(yahkv_ctx* ctx, int32_t kernel, double* total_ms, int64_t* launches);

/* ---- decode attention without any allocation ---------------------------------------------------------------
 * No counterpart in the reference (its decoder allocates its acc/ml workspace itself, loom_decoder.hpp:125-126).
 * For hosts that may not allocate GPU memory (a server whose own allocator holds the whole device, a plugin in a
 * process that forbids cudaMalloc after start-up, a latency-critical loop that cannot afford an allocation's
 * implicit synchronisation). Such a host cannot even create a yahkv_ctx, so this call takes no context: the caller
 * owns and passes every input and output, and the split-K work list, partial results and status word live in a
 * static device array inside the library (YAHKV_NOALLOC_SCRATCH_BYTES, held by every GPU that loads the library
 * until the process exits). It calls no cudaMalloc / cudaFree / pinned allocation / stream or event creation.
 *
 * Pools use the layout at the top of this file, q8_0 codes in their device form. Row b of tables_dev belongs to sequence b of the call; lens_dev[b]
 * is its number of visible keys (clamped to [1, table_stride * 64] on the device). n_splits is the fixed number of
 * split-K units per (sequence, kv head). Refused with YAHKV_ERR_CAPACITY beyond YAHKV_NOALLOC_MAX_SEQS sequences or
 * YAHKV_NOALLOC_MAX_UNITS = n_seqs * 4 * n_splits units. Results equal yahkv_attend_decode's with the same n_splits.
 *
 * All calls on a device share the static array, which keeps the previous call's contents (each call rewrites what
 * it reads): calls whose kernels could overlap on the GPU race, so issue them on one stream or order them yourself.
 * The first call on each device resolves the array's device address and sets kernel attributes; make that call
 * before starting any stream capture. err (may be NULL) receives the message of a refused call. */
#define YAHKV_NOALLOC_MAX_SEQS 256
#define YAHKV_NOALLOC_MAX_UNITS 1024
#define YAHKV_NOALLOC_SCRATCH_BYTES 6381824
typedef struct yahkv_noalloc_args {
  int32_t fmt;          /* YAHKV_FMT_* */
  int32_t n_layers;     /* layers in the pools */
  int32_t num_pages;    /* pages per layer */
  int32_t layer;
  const void* kcodes;   /* device, 16-byte aligned */
  const void* vcodes;
  const void* kscales;
  const void* vscales;
  const int32_t* tables_dev; /* [n_seqs][table_stride] */
  int32_t table_stride;
  int32_t n_seqs;
  const int32_t* lens_dev;   /* [n_seqs] */
  const void* q_dev;         /* [n_seqs][24][256] fp16 */
  const float* gate_dev;     /* [n_seqs][24][256] f32 or NULL */
  void* out_dev;             /* [n_seqs][24][256] by out_dtype */
  int32_t out_dtype;
  int32_t n_splits;
  float softmax_scale;       /* 0 = 1/16 */
  void* stream;              /* cudaStream_t; NULL = the default stream */
} yahkv_noalloc_args;
int yahkv_attend_decode_noalloc(const yahkv_noalloc_args* args, char* err, int32_t err_cap);
/* The error channel of the call above, equally allocation-free (no counterpart in the reference): queues on `stream`
 * an asynchronous copy of the static array's status word into *status_host, which the caller owns (page-locked memory
 * if the copy is to be truly asynchronous). Once the stream has reached the copy, 0 means every yahkv_attend_decode_noalloc
 * ordered before it on this device ran to completion; non-zero means a kernel gave up a bounded wait and the outputs
 * of the last call are invalid. The next call clears the word. Fails with YAHKV_ERR_ORDER before the first
 * yahkv_attend_decode_noalloc on the device (the array's address is resolved there). */
int yahkv_noalloc_status(int32_t* status_host, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* YAHKV_H_ */
