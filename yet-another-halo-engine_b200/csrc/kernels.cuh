// Device-side contracts shared by the kernels and the host library: geometry constants, the work descriptors the host
// plans per call, and one launch function per kernel. Launchers enqueue on the given stream and return the CUDA error.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace yahkv {

constexpr int kQHeads = 24;
constexpr int kKvHeads = 4;
constexpr int kGroup = 6;        // query heads per kv head
constexpr int kHeadDim = 256;
constexpr int kPageTokens = 64;
constexpr int kBlocksPerRow = 8; // 32-element blocks per head row

constexpr int kFmtQ8 = 0;
constexpr int kFmtQ4 = 1;
// The reference's own kv8a16 format (engine/gpu/loom/tools/gen_kvq.py:166-285, :474-660): K codes per token with a
// scale pair per 128-dim half; V codes per (16-key tile, channel) with a statistic pair per channel, four tiles to a
// page; the tile of the newest key stays open in fp16 (kv8a16.cu).
constexpr int kFmtKv8 = 2;
// Its 4-bit sibling kv4a16 (gen_kvq.py:288-463): K rotated by the Walsh-Hadamard transform H256 / 16, 16 levels per
// 32-dim group with an (16 s, lo - 16 s) pair; V 15 levels per (tile, channel) with a (16 sf, cf - 23 sf) pair
// (kv4a16.cu).
constexpr int kFmtKv4 = 3;
// Unquantized fp16 pages, the reference's fp16 cache mode (engine/gpu/loom/tools/gen_decode_attn.py:30-94, :97-335):
// K and V rows as they arrive, token-major on both sides, no scale pools (decode_f16.cu).
constexpr int kFmtF16 = 4;
constexpr int kTileKeys = 16;
constexpr int kTilesPerPage = kPageTokens / kTileKeys;
// The reference's own formats: V in 16-key tiles, an open fp16 tile and a K mean per (sequence, layer).
__host__ __device__ constexpr bool IsTileFmt(int fmt) { return fmt == kFmtKv8 || fmt == kFmtKv4; }

// Bytes of one token row of one kv head on the K side (the rows of the K tensor map). The V side of a page record has
// the same total size in every format (a tile format stores it as [tile][channel][16 or 8 bytes]).
__host__ __device__ constexpr int CodeBytes(int fmt) {
  return fmt == kFmtF16 ? 512 : (fmt == kFmtQ4 || fmt == kFmtKv4 ? 128 : 256);
}
// One page record of one kv head: codes then (in a separate pool) scales.
__host__ __device__ constexpr int RecordCodeBytes(int fmt) { return kPageTokens * CodeBytes(fmt); }
constexpr int kRecordScaleBytes = kPageTokens * kBlocksPerRow * 2;   // q8_0 / q4_0: 8 fp16 block scales per token
// Scale (q8_0, q4_0) or statistic (tile formats) bytes of one page record of one kv head, by side (0 = K, 1 = V):
// kv8a16 K holds 2 halves x an fp16 pair per token, kv4a16 K 8 groups x a pair; the V side of both holds an fp16 pair
// per (tile, channel).
__host__ __device__ constexpr int RecordScaleBytes(int fmt, int side) {
  return fmt == kFmtF16  ? 0
         : !IsTileFmt(fmt) ? kRecordScaleBytes
         : side == 1     ? kTilesPerPage * kHeadDim * 2 * 2
                         : kPageTokens * (fmt == kFmtKv8 ? 2 : 8) * 2 * 2;
}

// The pools of one context. Codes are addressed both by pointer (append, inspection) and through 2-D tensor maps
// whose rows are token rows of CodeBytes(fmt) bytes (attention's gathers).
// Device representation of q8_0 codes. K codes are GGUF's int8 bytes as they are: the attention kernel feeds them
// to the integer MMA without touching them. V codes are stored with the sign bit flipped, u = code + 128 (offset
// binary), so that the attention kernel turns a byte into the fp16 integer with one byte-permute and one subtract
// instead of three instructions. Everything that leaves the device (yahkv_read_page, yahkv_export_token,
// snapshots) or enters it (yahkv_write_page, snapshot load) flips the V bytes back, so hosts and files see GGUF's
// int8 codes on both sides. q4_0 nibbles are unsigned already and are stored as GGUF has them.
constexpr std::uint32_t kQ8FlipWord = 0x80808080U;
constexpr int kQ8FlipByte = 0x80;
// The flip of one side (0 = K, 1 = V) of a q8_0 pool, as a byte and as a word of four codes.
__host__ __device__ constexpr int Q8FlipByte(int side) { return side == 0 ? 0 : kQ8FlipByte; }
__host__ __device__ constexpr std::uint32_t Q8FlipWord(int side) { return side == 0 ? 0U : kQ8FlipWord; }

struct PoolView {
  std::uint8_t* kcodes;
  std::uint8_t* vcodes;
  std::uint16_t* kscales;
  std::uint16_t* vscales;
  int fmt;
  int num_pages;
  int n_layers;
  int kv_head_begin;   // the context's KV heads: [kv_head_begin, kv_head_begin + kv_head_count)
  int kv_head_count;
  __host__ __device__ bool OwnsKvHead(int h) const { return h >= kv_head_begin && h < kv_head_begin + kv_head_count; }
};

// One split-K unit of decode attention: pages [page_begin, page_end) of one sequence for one kv head.
struct DecodeUnit {
  std::int32_t batch;       // row of q / out
  std::int32_t seq;         // block-table row
  std::int32_t kvh;
  std::int32_t page_begin;
  std::int32_t page_end;
  std::int32_t n_keys;      // visible keys of the sequence (its length)
  std::int32_t partial;     // row of the partial workspace this unit writes
  std::int32_t pad;
};
// Where the partials of one (batch row, kv head) lie, for the combine pass.
struct CombineItem {
  std::int32_t first_partial;
  std::int32_t n_partials;
};

// One row of a device-resident decode batch: its block-table row and the split-K units reserved for it per kv head
// (units [first_unit + kvh * n_units, + n_units) belong to kv head kvh).
struct BatchSeq {
  std::int32_t seq_row;
  std::int32_t first_unit;
  std::int32_t n_units;
  std::int32_t open_cur;    // tile formats: the sequence's current open-tile buffer (the same in every layer)
};
struct VTileWork;
// vwork_dev / state_rows_dev: tile formats only (else null): per batch row the V tile work item of this step's token and
// the row of the sequence's layer-0 state (the kernels add the layer).
cudaError_t LaunchBatchPlan(const std::int32_t* lens_dev, const BatchSeq* seqs_dev, int n_seqs,
                            const std::int32_t* tables_dev, int table_stride, int unit_pages, int num_pages,
                            DecodeUnit* units_dev, CombineItem* items_dev, std::int64_t* slots_dev,
                            VTileWork* vwork_dev, std::int32_t* state_rows_dev, int n_layers, cudaStream_t stream);
cudaError_t LaunchBatchAdvance(std::int32_t* lens_dev, int n_seqs, int by, cudaStream_t stream);

// Prefill attention reads a dequantized fp16 copy of the sequences' K and V (the reference's yah_kdeq / yah_vdeq
// pre-pass, engine/gpu/loom/tools/gen_attn_fa.py:4648-4860): rows [kv_row0 + kvh * kv_rows, ...) of the scratch hold
// kv head kvh of the sequence, token-major, 256 fp16 each, kv_rows = the length rounded up to whole pages.
struct PrefillSeq {
  std::int32_t seq;         // block-table row
  std::int32_t n_pages;     // pages holding keys 0 .. kv_len - 1
  std::int32_t kv_len;      // keys in the cache, the chunk included
  std::int32_t kv_rows;     // n_pages * 64
  std::int32_t kv_row0;     // first scratch row of the sequence
  std::int32_t pad[3];      // pad[0]: kv8a16 only, which of the sequence's two open-tile buffers is current
};
// What an attention kernel needs to norm and rotate raw f32 query rows itself (the query side of the fused norm + RoPE
// kernel, done in the attention kernel's prologue).
struct QueryRaw {
  const float* q;           // [rows][24][256] f32, the raw q projection
  const float* weight;      // [256] f32 norm weights
  const float2* rope_tab;   // (cos, sin) [rope_rows][32]
  float eps;
  int rope_rows;
};
// One tile of prefill attention: 128 query rows of one sequence for one query head.
constexpr int kPrefillTileRows = 128;
struct PrefillTile {
  std::int32_t kv_row0;     // first scratch row of (sequence, kv head of this query head)
  std::int32_t head;        // query head
  std::int32_t q_row0;      // first packed query row of the tile
  std::int32_t n_rows;      // valid query rows in the tile (<= 128)
  std::int32_t pos0;        // position of the tile's first query row; row r sees keys 0 .. pos0 + r
  std::int32_t jt_begin;    // 64-key tiles [jt_begin, jt_end) of the keys the rows can see: all of them for a whole
  std::int32_t jt_end;      // tile, a slice of them for a part of a split tile
  std::int32_t part;        // -1: the CTA finishes the rows itself; >= 0: slot of its unnormalised partial result
};
static_assert(sizeof(PrefillTile) == 32, "uploaded as an array");

// A tile of the call's last, partly filled wave that was split along the keys into n_parts CTAs (every second entry
// of the tile list from tile_index on, every second part slot, because tiles come as pairs of heads): the merge
// kernel joins their partial results.
struct PrefillMerge {
  std::int32_t tile_index;
  std::int32_t n_parts;
};
constexpr int kPrefillMaxParts = 4;   // key ranges a tile is split into at most
// Partial result of one part: O [128 rows][256] f32 unnormalised, then (max in log2 units, sum) per row.
constexpr int kPrefillPartAccFloats = kPrefillTileRows * kHeadDim;
constexpr int kPrefillPartMlFloats = kPrefillTileRows * 2;

// Partial workspace per unit: acc [6][256] f32 (unnormalised), then ml [6][2] f32 (max in log2 units, sum).
constexpr int kPartialAccFloats = kGroup * kHeadDim;
constexpr int kPartialMlFloats = kGroup * 2;
// Split-K units one (batch row, kv head) may have: the combine kernel keeps one weight per unit in shared memory.
// Every planner stays below it (yahkv_config.max_splits is refused above it).
constexpr int kCombineMaxUnits = 1024;

// Launch with programmatic stream serialization allowed: see ChainedKernelEntry in ptx.cuh.
template <class... Params, class... Args>
cudaError_t LaunchChained(void (*kernel)(Params...), dim3 grid, dim3 block, std::size_t smem, cudaStream_t stream,
                          Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

cudaError_t LaunchAppend(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                         const void* k_dev, const void* v_dev, cudaStream_t stream);
cudaError_t LaunchRopeAppend(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                             const std::int32_t* positions_dev, const float* q_dev, const float* k_dev,
                             const float* v_dev, const float* q_weight_dev, const float* k_weight_dev, float eps,
                             const float2* rope_tab_dev, int rope_rows, void* q_out_dev, void* kv16_out_dev,
                             cudaStream_t stream);

struct DecodeLaunch {
  const CUtensorMap* kmap;  // host pointers to the encoded maps (passed by value to the kernel)
  const CUtensorMap* vmap;
  PoolView pool;
  int layer;
  const std::int32_t* tables_dev;
  int table_stride;
  const DecodeUnit* units_dev;
  int n_units;
  const CombineItem* items_dev;
  int n_seqs;
  const void* q_dev;        // [n_seqs][24][256] fp16, or f32 when q_raw is set
  bool q_raw;               // the query is the raw f32 projection: the part kernel's prologue norms and rotates it
  const float* q_weight_dev;   // q_raw: [256] f32 norm weights
  float q_eps;
  const float2* rope_tab_dev;  // q_raw: (cos, sin) [rope_rows][32]
  int rope_rows;
  const float* gate_dev;
  void* out_dev;
  int out_f32;
  float scale_log2;         // softmax scale * log2(e)
  float* partial_acc;
  float* partial_ml;
  int* status_dev;          // sticky error word, 0 = ok
};
cudaError_t LaunchDecodePart(const DecodeLaunch& a, cudaStream_t stream);
// fp16 pages (decode_f16.cu)
cudaError_t LaunchF16DecodePart(const DecodeLaunch& a, cudaStream_t stream);
cudaError_t ConfigureF16Kernels();

// ---- kv8a16 (kv8a16.cu) ----
// Per-sequence state of the format beyond the pools, per layer: two open-tile buffers [2][4 heads][256][16] fp16 (the
// tile of the newest key in fp16; which of the two is current is host state) and the K channel mean [4][256] f32.
constexpr int kOpenTileHalfs = kKvHeads * kHeadDim * kTileKeys;   // one buffer, in fp16 elements
// One 16-key V tile touched by an append call.
struct VTileWork {
  std::int32_t state_row;   // (sequence * n_layers + layer): index of the open-tile pair (+ the launch's state_row_add)
  std::int32_t phys_tile;   // page * 4 + tile in page: the pool slot of the tile
  std::int32_t n_old;       // keys 0 .. n_old - 1 were appended earlier and come from open buffer read_buf
  std::int32_t n_keys;      // keys of the tile after this call
  std::int32_t read_buf;    // 0 | 1
  std::int32_t write_buf;   // open buffer that receives the tile's keys (-1: the tile is not the newest, keep none)
  std::int32_t complete;    // n_keys == 16: quantize and store the tile
  std::int32_t pad;
  std::int32_t src[kTileKeys];   // input token index of key j for j >= n_old
};
static_assert(sizeof(VTileWork) == 96, "uploaded as an array");
// state_row_add is added to every state row of the call: 0 when the host listed (sequence * n_layers + layer) rows,
// the layer when a decode batch's plan kernel listed layer-0 rows once for all layers of a step.
cudaError_t LaunchKv8AppendK(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                             const std::int32_t* state_rows_dev, int state_row_add, const float* kmean_dev,
                             const void* k_dev, cudaStream_t stream);
cudaError_t LaunchKv8AppendV(const PoolView& pool, int layer, int n_work, const VTileWork* work_dev, int state_row_add,
                             void* open_tiles_dev, const void* v_dev, cudaStream_t stream);
// Decode attention over kv8a16 pools. DecodeUnit::pad carries the sequence's current open buffer (0 | 1);
// state_stride = n_layers (the open-tile pair of (sequence, layer) is row seq * n_layers + layer).
cudaError_t LaunchKv8DecodePart(const DecodeLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream);
cudaError_t ConfigureKv8Kernels();
// kv4a16 (kv4a16.cu): the K append (rotation + 4-bit groups) and decode attention; the V append and the prefill
// dequantize pass are the kv8a16 launchers above and below, which switch on pool.fmt.
cudaError_t LaunchKv4AppendK(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                             const std::int32_t* state_rows_dev, int state_row_add, const float* kmean_dev,
                             const void* k_dev, cudaStream_t stream);
cudaError_t LaunchKv4DecodePart(const DecodeLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream);
cudaError_t ConfigureKv4Kernels();
cudaError_t LaunchDecodeCombine(const DecodeLaunch& a, cudaStream_t stream);
// Shared-memory bytes the decode kernel asks for (for the one-time attribute set-up).
cudaError_t ConfigureDecodeKernels();

struct PrefillLaunch {
  PoolView pool;
  int layer;
  const std::int32_t* tables_dev;
  int table_stride;
  const PrefillSeq* seqs_dev;
  int n_seqs;
  int max_pages;            // largest n_pages of the call (grid of the dequantize pass)
  void* k16_dev;            // fp16 scratch [rows][256], K and V
  void* v16_dev;
  const void* q_dev;        // [rows][24][256] fp16, or f32 when q_raw is set
  bool q_raw;               // the query is the raw f32 projection: the kernel's prologue norms and rotates its rows
  const float* q_weight_dev;   // q_raw: [256] f32 norm weights
  float q_eps;              // q_raw: norm epsilon
  const float2* rope_tab_dev;  // q_raw: (cos, sin) [rope_rows][32]
  int rope_rows;
  const CUtensorMap* k16map;  // scratch as [rows][256] fp16, 128-byte swizzle; boxes K 64 dims x 32 keys, V 64 x 64
  const CUtensorMap* v16map;
  const PrefillTile* tiles_dev;
  int n_tiles;
  const PrefillMerge* merges_dev;   // split tiles of this call (may be empty)
  int n_merges;
  float* part_acc;                  // [parts][128][256] f32
  float* part_ml;                   // [parts][128][2] f32
  const float* gate_dev;
  void* out_dev;
  int out_f32;
  float scale_log2;
  int* status_dev;
};
cudaError_t LaunchPrefillDequant(const PrefillLaunch& a, cudaStream_t stream);
// kv8a16: the same pass for that format (kv8a16.cu); PrefillSeq::pad[0] names each sequence's current open buffer.
cudaError_t LaunchKv8PrefillDequant(const PrefillLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream);
// kv4a16 (kv4a16.cu): K rows are rotated back (the transform is its own inverse) so the chunk's q needs no rotation.
cudaError_t LaunchKv4PrefillDequant(const PrefillLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream);
cudaError_t LaunchPrefill(const PrefillLaunch& a, cudaStream_t stream);
cudaError_t ConfigurePrefillKernels(int* max_active_pairs);   // also: how many CTA pairs the device runs at once
// Encodes a 2-D tiled tensor map (row-major, `inner` elements of `elem_bytes` per row, 128-byte swizzle). Host only.
bool EncodeTensorMap2D(CUtensorMap* map, int elem_bytes, void* base, std::uint64_t inner, std::uint64_t rows,
                       std::uint32_t box_inner, std::uint32_t box_rows);

// Status codes the kernels write into the sticky status word.
constexpr int kStatusWaitTimeout = 1;
// One CTA waits at most limit_ns on an mbarrier nobody arrives at, gives up, records kStatusWaitTimeout and returns:
// the give-up path of every bounded wait in this library, run on purpose (yahkv_debug_wait_timeout).
cudaError_t LaunchWaitProbe(int* status_dev, std::uint64_t limit_ns, cudaStream_t stream);

}  // namespace yahkv
