// The C ABI of the library (include/yahkv.h): context and device resources, stream-ordered uploads of block tables
// and work lists, and the entry points that validate, plan and launch. There is no CPU fallback: a hot-path call on
// a context without a GPU fails with YAHKV_ERR_NO_DEVICE.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/yahkv.h"
#include "kernels.cuh"
#include "kv_host.hpp"

using namespace yahkv;

namespace {

std::mutex g_create_mu;
std::string g_create_error;

// A small set of pinned staging buffers handed out round-robin. A buffer is reused only after the copies that read it
// have completed (its event), so host-side state can change right after a call returns.
class Staging {
 public:
  static constexpr int kSlots = 8;
  ~Staging() {
    for (auto& s : slots_) {
      if (s.host != nullptr) cudaFreeHost(s.host);
      if (s.ev != nullptr) cudaEventDestroy(s.ev);
    }
  }
  cudaError_t Acquire(std::size_t bytes, char** out) {
    Slot& s = slots_[next_];
    cur_ = next_;
    next_ = (next_ + 1) % kSlots;
    if (s.ev == nullptr) {
      cudaError_t e = cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming);
      if (e != cudaSuccess) return e;
    }
    if (s.in_flight) {
      cudaError_t e = cudaEventSynchronize(s.ev);
      if (e != cudaSuccess) return e;
      s.in_flight = false;
    }
    if (s.cap < bytes) {
      if (s.host != nullptr) cudaFreeHost(s.host);
      s.host = nullptr, s.cap = 0;
      const std::size_t cap = std::max<std::size_t>(bytes, 1 << 16);
      cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&s.host), cap, cudaHostAllocDefault);
      if (e != cudaSuccess) return e;
      s.cap = cap;
    }
    *out = s.host;
    return cudaSuccess;
  }
  // Marks the buffer handed out last as busy until everything queued on `stream` so far has run.
  cudaError_t Release(cudaStream_t stream) {
    Slot& s = slots_[cur_];
    s.in_flight = true;
    return cudaEventRecord(s.ev, stream);
  }

 private:
  struct Slot {
    char* host = nullptr;
    std::size_t cap = 0;
    cudaEvent_t ev = nullptr;
    bool in_flight = false;
  };
  Slot slots_[kSlots];
  int next_ = 0, cur_ = 0;
};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

struct yahkv_ctx {
  explicit yahkv_ctx(const yahkv_config& c) : cfg(c), host(c) {}
  yahkv_config cfg;
  KvHost host;
  mutable std::string err;
  bool has_device = false;
  PoolView pool{};
  CUtensorMap kmap{}, vmap{};
  std::int32_t* tables_dev = nullptr;
  DecodeUnit* units_dev = nullptr;
  CombineItem* items_dev = nullptr;
  PrefillTile* tiles_dev = nullptr;
  int max_tiles = 0;
  std::int64_t* slots_dev = nullptr;
  float* partial_acc = nullptr;
  float* partial_ml = nullptr;
  int max_units = 0;
  int* status_dev = nullptr;
  cudaStream_t stream = nullptr;
  Staging staging;
  // Device-side staging of the host-buffer entry points: two sets used in turn, so the copies of one layer-step (on
  // their own streams) overlap the kernels of the previous one (on the context's stream).
  struct HostStage {
    void *k = nullptr, *v = nullptr, *q = nullptr, *out = nullptr;
    float* gate = nullptr;
    cudaEvent_t in_ready = nullptr, compute_done = nullptr, out_done = nullptr;
    bool used = false;
  };
  HostStage hst[2];
  // fused RoPE + append: cos / sin of every position the block tables can hold, and the call's positions
  float2* rope_tab_dev = nullptr;
  int rope_rows = 0;
  std::int32_t* rope_pos_dev = nullptr;
  std::uint16_t* rope_kv16_dev = nullptr;   // tile formats: fp16 [2 sides][tokens][4][256] out of the RoPE kernel
  std::vector<std::int32_t> rope_pos_scratch;
  int hst_next = 0;
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
  std::int64_t launches = 0;
  std::int64_t device_bytes = 0;
  // optional per-kernel timing: event pairs around each launch, summed on read
  bool timing = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timing_events[YAHKV_KERNEL_COUNT];
  std::vector<cudaEvent_t> event_pool;
  std::vector<std::int64_t> slot_scratch;
  std::vector<std::int64_t> pos_scratch;
  std::vector<PrefillTile> tile_scratch;
  std::vector<PrefillMerge> merge_scratch;
  PrefillMerge* merges_dev = nullptr;
  float* part_acc_dev = nullptr;   // partial results of split prefill tiles
  float* part_ml_dev = nullptr;
  int n_sm = 0;                    // SMs the prefill planner fills waves of
  int n_sm_device = 0;             // SMs of the device (the planner's default and upper bound)
  std::vector<PrefillSeq> pseq_scratch;
  PrefillSeq* pseqs_dev = nullptr;
  void *k16_dev = nullptr, *v16_dev = nullptr;   // fp16 scratch of the prefill dequantize pass, grown on demand
  std::int64_t p16_rows = 0;
  CUtensorMap k16map{}, v16map{};
  float scale_log2 = 0.0F;
  // kv8a16: per (sequence, layer) two open fp16 V tiles and the K channel mean; per-call work lists
  void* open_tiles_dev = nullptr;
  float* kmean_dev = nullptr;
  std::int32_t* state_rows_dev = nullptr;
  VTileWork* vwork_dev = nullptr;
  std::vector<VTileWork> vwork_scratch;
  std::vector<std::int32_t> state_row_scratch;
  std::vector<DecodeUnit> unit_scratch;
};

namespace {

int Fail(const yahkv_ctx* ctx, int code, std::string msg) {
  ctx->err = std::move(msg);
  return code;
}
int FailHost(const yahkv_ctx* ctx, HostError e) { return Fail(ctx, e.code, std::move(e.message)); }
int FailCuda(const yahkv_ctx* ctx, const char* what, cudaError_t e) {
  return Fail(ctx, YAHKV_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

#define YAHKV_CUDA(ctx, call)                                     \
  do {                                                            \
    const cudaError_t e_ = (call);                                \
    if (e_ != cudaSuccess) return FailCuda((ctx), #call, e_);     \
  } while (0)

template <class T>
cudaError_t DevAlloc(yahkv_ctx* ctx, T** p, std::size_t count, bool zero) {
  const std::size_t bytes = std::max<std::size_t>(count * sizeof(T), 256);
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(p), bytes);
  if (e != cudaSuccess) return e;
  ctx->device_bytes += static_cast<std::int64_t>(bytes);
  if (zero) e = cudaMemset(*p, 0, bytes);
  return e;
}

EncodeTiledFn g_encode = nullptr;   // cuTensorMapEncodeTiled, fetched once per process
int ResizePrefillScratch(yahkv_ctx* ctx, std::int64_t rows);

int EncodeMap(yahkv_ctx* ctx, EncodeTiledFn encode, CUtensorMap* map, void* base) {
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(CodeBytes(ctx->cfg.fmt));
  const cuuint64_t rows = static_cast<cuuint64_t>(ctx->cfg.n_layers) * ctx->cfg.num_pages * kKvHeads * kPageTokens;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, kPageTokens};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Fail(ctx, YAHKV_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(r));
  return YAHKV_OK;
}

int InitDevice(yahkv_ctx* ctx) {
  const yahkv_config& c = ctx->cfg;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || c.device >= count)
    return Fail(ctx, YAHKV_ERR_NO_DEVICE, "no CUDA device " + std::to_string(c.device));
  YAHKV_CUDA(ctx, cudaSetDevice(c.device));
  cudaDeviceProp prop{};
  YAHKV_CUDA(ctx, cudaGetDeviceProperties(&prop, c.device));
  if (prop.major != 10)
    return Fail(ctx, YAHKV_ERR_NO_DEVICE, std::string("this library is built for sm_100a only; device is ") + prop.name);
  // A blocking stream: it orders itself against the legacy default stream, so a caller that prepares buffers on the
  // default stream (and passes no stream) needs no extra synchronisation.
  YAHKV_CUDA(ctx, cudaStreamCreate(&ctx->stream));

  const std::size_t recs = static_cast<std::size_t>(c.n_layers) * c.num_pages * kKvHeads;
  ctx->pool.fmt = c.fmt, ctx->pool.num_pages = c.num_pages, ctx->pool.n_layers = c.n_layers;
  ctx->pool.kv_head_begin = ctx->host.kv_head_begin(), ctx->pool.kv_head_count = ctx->host.kv_head_count();
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->pool.kcodes, recs * RecordCodeBytes(c.fmt), true));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->pool.vcodes, recs * RecordCodeBytes(c.fmt), true));
  if (c.fmt == YAHKV_FMT_Q8_0)   // code 0 in the V side's device representation (sign bit flipped)
    YAHKV_CUDA(ctx, cudaMemset(ctx->pool.vcodes, kQ8FlipByte, recs * RecordCodeBytes(c.fmt)));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->pool.kscales, recs * (RecordScaleBytes(c.fmt, 0) / 2), true));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->pool.vscales, recs * (RecordScaleBytes(c.fmt, 1) / 2), true));
  if (IsTileFmt(c.fmt)) {
    const std::size_t states = static_cast<std::size_t>(c.max_seqs) * c.n_layers;
    YAHKV_CUDA(ctx, DevAlloc(ctx, reinterpret_cast<std::uint16_t**>(&ctx->open_tiles_dev), states * 2 * kOpenTileHalfs, true));
    YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->kmean_dev, states * kKvHeads * kHeadDim, true));
    YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->state_rows_dev, static_cast<std::size_t>(c.max_batch_tokens), false));
    YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->vwork_dev, static_cast<std::size_t>(c.max_batch_tokens) + 2 * c.max_seqs, false));
    YAHKV_CUDA(ctx, ConfigureKv8Kernels());
    YAHKV_CUDA(ctx, ConfigureKv4Kernels());
  }
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->tables_dev, static_cast<std::size_t>(c.max_seqs) * c.max_pages_per_seq, true));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->slots_dev, static_cast<std::size_t>(c.max_batch_tokens), false));
  ctx->max_units = c.max_seqs * kKvHeads * c.max_splits;
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->units_dev, static_cast<std::size_t>(ctx->max_units), false));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->items_dev, static_cast<std::size_t>(c.max_seqs) * kKvHeads, false));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->partial_acc, static_cast<std::size_t>(ctx->max_units) * kPartialAccFloats, false));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->partial_ml, static_cast<std::size_t>(ctx->max_units) * kPartialMlFloats, false));
  YAHKV_CUDA(ctx, cudaDeviceGetAttribute(&ctx->n_sm, cudaDevAttrMultiProcessorCount, c.device));
  ctx->n_sm_device = ctx->n_sm;
  ctx->max_tiles = (c.max_batch_tokens / kPrefillTileRows + c.max_seqs) * kQHeads + kPrefillMaxParts * ctx->n_sm;
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->tiles_dev, static_cast<std::size_t>(ctx->max_tiles), false));
  if (ctx->n_sm > 0) {
    YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->merges_dev, static_cast<std::size_t>(ctx->n_sm), false));
    // a tail of up to n_sm - 1 tiles, each in up to kPrefillMaxParts parts (78 MB on 148 SMs)
    const std::size_t parts = static_cast<std::size_t>(ctx->n_sm) * kPrefillMaxParts;
    YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->part_acc_dev, parts * kPrefillPartAccFloats, false));
    YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->part_ml_dev, parts * kPrefillPartMlFloats, false));
  }
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->pseqs_dev, static_cast<std::size_t>(c.max_seqs), false));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->status_dev, 1, true));
  const std::size_t ns = static_cast<std::size_t>(c.max_seqs);
  for (auto& h : ctx->hst) {
    YAHKV_CUDA(ctx, DevAlloc(ctx, reinterpret_cast<char**>(&h.k), ns * kKvHeads * kHeadDim * 2, false));
    YAHKV_CUDA(ctx, DevAlloc(ctx, reinterpret_cast<char**>(&h.v), ns * kKvHeads * kHeadDim * 2, false));
    YAHKV_CUDA(ctx, DevAlloc(ctx, reinterpret_cast<char**>(&h.q), ns * kQHeads * kHeadDim * 2, false));
    YAHKV_CUDA(ctx, DevAlloc(ctx, reinterpret_cast<char**>(&h.out), ns * kQHeads * kHeadDim * 4, false));
    YAHKV_CUDA(ctx, DevAlloc(ctx, &h.gate, ns * kQHeads * kHeadDim, false));
    YAHKV_CUDA(ctx, cudaEventCreateWithFlags(&h.in_ready, cudaEventDisableTiming));
    YAHKV_CUDA(ctx, cudaEventCreateWithFlags(&h.compute_done, cudaEventDisableTiming));
    YAHKV_CUDA(ctx, cudaEventCreateWithFlags(&h.out_done, cudaEventDisableTiming));
  }
  YAHKV_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
  YAHKV_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));

  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres{};
  YAHKV_CUDA(ctx, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
    return Fail(ctx, YAHKV_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled");
  const auto encode = reinterpret_cast<EncodeTiledFn>(fn);
  g_encode = encode;
  if (int r = EncodeMap(ctx, encode, &ctx->kmap, ctx->pool.kcodes); r != YAHKV_OK) return r;
  if (int r = EncodeMap(ctx, encode, &ctx->vmap, ctx->pool.vcodes); r != YAHKV_OK) return r;
  if (c.max_prefill_keys > 0)
    if (int r = ResizePrefillScratch(ctx, static_cast<std::int64_t>(c.max_prefill_keys) * kKvHeads); r != YAHKV_OK) return r;
  YAHKV_CUDA(ctx, ConfigureDecodeKernels());
  if (c.fmt == YAHKV_FMT_F16) YAHKV_CUDA(ctx, ConfigureF16Kernels());
  {
    int pairs = 0;   // CTA pairs of the prefill kernel that run at the same time: the planner's wave
    YAHKV_CUDA(ctx, ConfigurePrefillKernels(&pairs));
    if (pairs > 0) ctx->n_sm = std::min(ctx->n_sm, 2 * pairs);
  }
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  ctx->has_device = true;
  return YAHKV_OK;
}

void FreeDevice(yahkv_ctx* ctx) {
  if (ctx->cfg.device < 0) return;
  cudaSetDevice(ctx->cfg.device);
  if (ctx->stream != nullptr) cudaStreamSynchronize(ctx->stream);
  void* ptrs[] = {ctx->pool.kcodes, ctx->pool.vcodes, ctx->pool.kscales, ctx->pool.vscales, ctx->tables_dev,
                  ctx->slots_dev,   ctx->units_dev,   ctx->items_dev,    ctx->partial_acc,  ctx->partial_ml,
                  ctx->tiles_dev,   ctx->status_dev,  ctx->pseqs_dev, ctx->k16_dev, ctx->v16_dev,
                  ctx->merges_dev, ctx->part_acc_dev, ctx->part_ml_dev,
                  ctx->rope_tab_dev, ctx->rope_pos_dev, ctx->open_tiles_dev, ctx->kmean_dev, ctx->state_rows_dev,
                  ctx->vwork_dev,   ctx->rope_kv16_dev};
  for (void* p : ptrs)
    if (p != nullptr) cudaFree(p);
  for (cudaStream_t st : {ctx->h2d_stream, ctx->d2h_stream})
    if (st != nullptr) cudaStreamSynchronize(st), cudaStreamDestroy(st);
  for (auto& h : ctx->hst) {
    for (void* p : {h.k, h.v, h.q, h.out, static_cast<void*>(h.gate)})
      if (p != nullptr) cudaFree(p);
    for (cudaEvent_t e : {h.in_ready, h.compute_done, h.out_done})
      if (e != nullptr) cudaEventDestroy(e);
  }
  if (ctx->stream != nullptr) cudaStreamDestroy(ctx->stream);
  for (auto& list : ctx->timing_events)
    for (auto& pr : list) cudaEventDestroy(pr.first), cudaEventDestroy(pr.second);
  for (cudaEvent_t e : ctx->event_pool) cudaEventDestroy(e);
}

// Event pair around one kernel launch while timing is on: Begin before the launch, End right after it.
struct TimedLaunch {
  TimedLaunch(yahkv_ctx* c, int kernel, cudaStream_t st) : ctx(c), id(kernel), stream(st) {
    if (!ctx->timing) return;
    a = Take(), b = Take();
    if (a != nullptr && b != nullptr) cudaEventRecord(a, stream);
  }
  void End() {
    if (!ctx->timing || a == nullptr || b == nullptr) return;
    cudaEventRecord(b, stream);
    ctx->timing_events[id].emplace_back(a, b);
  }
  cudaEvent_t Take() {
    if (!ctx->event_pool.empty()) {
      cudaEvent_t e = ctx->event_pool.back();
      ctx->event_pool.pop_back();
      return e;
    }
    cudaEvent_t e = nullptr;
    return cudaEventCreate(&e) == cudaSuccess ? e : nullptr;
  }
  yahkv_ctx* ctx;
  int id;
  cudaStream_t stream;
  cudaEvent_t a = nullptr, b = nullptr;
};

cudaStream_t StreamOf(yahkv_ctx* ctx, void* stream) {
  return stream != nullptr ? static_cast<cudaStream_t>(stream) : ctx->stream;
}

int RequireDevice(yahkv_ctx* ctx, const char* what) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  if (!ctx->has_device)
    return Fail(ctx, YAHKV_ERR_NO_DEVICE, std::string(what) + ": host-only context (no GPU, no CPU fallback)");
  if (cudaSetDevice(ctx->cfg.device) != cudaSuccess) return Fail(ctx, YAHKV_ERR_CUDA, "cudaSetDevice failed");
  return YAHKV_OK;
}

// Copies `bytes` at `src` (host) to `dst` (device) on `stream` through a pinned staging buffer.
int StagedUpload(yahkv_ctx* ctx, void* dst, const void* src, std::size_t bytes, cudaStream_t stream) {
  char* buf = nullptr;
  YAHKV_CUDA(ctx, ctx->staging.Acquire(bytes, &buf));
  std::memcpy(buf, src, bytes);
  YAHKV_CUDA(ctx, cudaMemcpyAsync(dst, buf, bytes, cudaMemcpyHostToDevice, stream));
  YAHKV_CUDA(ctx, ctx->staging.Release(stream));
  return YAHKV_OK;
}

// Block-table rows changed on the host since the last hot call go to the device ahead of the kernels that read them.
int FlushTables(yahkv_ctx* ctx, cudaStream_t stream) {
  struct Range {
    int seq, lo, hi;
  };
  std::vector<Range> ranges;
  std::size_t total = 0;
  ctx->host.ForEachDirty([&](int s, int lo, int hi) {
    ranges.push_back({s, lo, hi});
    total += static_cast<std::size_t>(hi - lo) * 4;
  });
  if (ranges.empty()) return YAHKV_OK;
  // A flush that fails part-way marks every range dirty again, so the rows go up with the next hot call instead of
  // being lost.
  auto fail = [&](const char* what, cudaError_t e) {
    for (const Range& r : ranges) ctx->host.MarkDirtyAgain(r.seq, r.lo, r.hi);
    return FailCuda(ctx, what, e);
  };
  char* buf = nullptr;
  if (cudaError_t e = ctx->staging.Acquire(total, &buf); e != cudaSuccess) return fail("table staging", e);
  std::size_t off = 0;
  for (const Range& r : ranges) {
    const std::size_t bytes = static_cast<std::size_t>(r.hi - r.lo) * 4;
    if (bytes == 0) continue;
    std::memcpy(buf + off, ctx->host.table_row(r.seq) + r.lo, bytes);
    if (cudaError_t e = cudaMemcpyAsync(ctx->tables_dev + static_cast<std::size_t>(r.seq) * ctx->cfg.max_pages_per_seq + r.lo,
                                        buf + off, bytes, cudaMemcpyHostToDevice, stream);
        e != cudaSuccess)
      return fail("table upload", e);
    off += bytes;
  }
  if (cudaError_t e = ctx->staging.Release(stream); e != cudaSuccess) return fail("table staging event", e);
  return YAHKV_OK;
}

// (Re)allocates the fp16 K and V scratch of the prefill dequantize pass for `rows` token rows and encodes its maps.
int ResizePrefillScratch(yahkv_ctx* ctx, std::int64_t rows) {
  if (ctx->k16_dev != nullptr) cudaFree(ctx->k16_dev), ctx->device_bytes -= ctx->p16_rows * kHeadDim * 2;
  if (ctx->v16_dev != nullptr) cudaFree(ctx->v16_dev), ctx->device_bytes -= ctx->p16_rows * kHeadDim * 2;
  ctx->k16_dev = ctx->v16_dev = nullptr, ctx->p16_rows = 0;
  const std::size_t bytes = static_cast<std::size_t>(rows) * kHeadDim * 2;
  YAHKV_CUDA(ctx, cudaMalloc(&ctx->k16_dev, bytes));
  YAHKV_CUDA(ctx, cudaMalloc(&ctx->v16_dev, bytes));
  ctx->device_bytes += 2 * static_cast<std::int64_t>(bytes);
  ctx->p16_rows = rows;
  // boxes: K [32 keys][64 dims] (each CTA of a pair loads half of a tile's keys), V [64 keys][64 dims]
  if (!EncodeTensorMap2D(&ctx->k16map, 2, ctx->k16_dev, kHeadDim, static_cast<std::uint64_t>(rows), 64, 32) ||
      !EncodeTensorMap2D(&ctx->v16map, 2, ctx->v16_dev, kHeadDim, static_cast<std::uint64_t>(rows), 64, 64))
    return Fail(ctx, YAHKV_ERR_CUDA, "tensor map encode failed for the prefill scratch");
  return YAHKV_OK;
}

int CheckStatus(yahkv_ctx* ctx) {
  int st = 0;
  YAHKV_CUDA(ctx, cudaMemcpy(&st, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemset(ctx->status_dev, 0, sizeof(int));
    return Fail(ctx, YAHKV_ERR_CUDA, "a kernel gave up a bounded wait (status " + std::to_string(st) + "); results of the call are invalid");
  }
  return YAHKV_OK;
}

}  // namespace

namespace yahkv {
bool EncodeTensorMap2D(CUtensorMap* map, int elem_bytes, void* base, std::uint64_t inner, std::uint64_t rows,
                       std::uint32_t box_inner, std::uint32_t box_rows) {
  if (g_encode == nullptr || rows == 0) return false;
  const CUtensorMapDataType type = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {inner * static_cast<cuuint64_t>(elem_bytes)};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return g_encode(map, type, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace yahkv

extern "C" {

const char* yahkv_error_name(int code) {
  switch (code) {
    case YAHKV_OK: return "YAHKV_OK";
    case YAHKV_ERR_INVALID: return "YAHKV_ERR_INVALID";
    case YAHKV_ERR_NO_PAGES: return "YAHKV_ERR_NO_PAGES";
    case YAHKV_ERR_CUDA: return "YAHKV_ERR_CUDA";
    case YAHKV_ERR_NO_DEVICE: return "YAHKV_ERR_NO_DEVICE";
    case YAHKV_ERR_ORDER: return "YAHKV_ERR_ORDER";
    case YAHKV_ERR_CAPACITY: return "YAHKV_ERR_CAPACITY";
    default: return "YAHKV_ERR_UNKNOWN";
  }
}

const char* yahkv_last_error(const yahkv_ctx* ctx) {
  if (ctx != nullptr) return ctx->err.c_str();
  std::lock_guard<std::mutex> lock(g_create_mu);
  static thread_local std::string copy;
  copy = g_create_error;
  return copy.c_str();
}

int yahkv_create(const yahkv_config* cfg, yahkv_ctx** out) {
  auto fail = [&](int code, const std::string& msg) {
    std::lock_guard<std::mutex> lock(g_create_mu);
    g_create_error = msg;
    return code;
  };
  if (out == nullptr) return fail(YAHKV_ERR_INVALID, "yahkv_create: null out pointer");
  *out = nullptr;
  if (cfg == nullptr) return fail(YAHKV_ERR_INVALID, "yahkv_create: null config");
  yahkv_config c = *cfg;
  if (c.max_splits == 0) c.max_splits = 64;
  if (c.max_batch_tokens == 0) c.max_batch_tokens = 8192;
  if (c.softmax_scale == 0.0F) c.softmax_scale = 1.0F / 16.0F;
  std::string why;
  if (int r = KvHost::ValidateConfig(c, &why); r != YAHKV_OK) return fail(r, "yahkv_create: " + why);
  if (c.max_batch_tokens < c.max_seqs) c.max_batch_tokens = c.max_seqs;
  yahkv_ctx* ctx = new (std::nothrow) yahkv_ctx(c);
  if (ctx == nullptr) return fail(YAHKV_ERR_INVALID, "yahkv_create: out of host memory");
  ctx->scale_log2 = c.softmax_scale * 1.4426950408889634F;
  ctx->slot_scratch.resize(static_cast<std::size_t>(c.max_batch_tokens));
  if (c.device >= 0) {
    if (int r = InitDevice(ctx); r != YAHKV_OK) {
      const std::string msg = ctx->err;
      FreeDevice(ctx);
      delete ctx;
      return fail(r, "yahkv_create: " + msg);
    }
  }
  *out = ctx;
  return YAHKV_OK;
}

void yahkv_destroy(yahkv_ctx* ctx) {
  if (ctx == nullptr) return;
  FreeDevice(ctx);
  delete ctx;
}

int yahkv_seq_create(yahkv_ctx* ctx, int32_t* seq) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  if (seq == nullptr) return Fail(ctx, YAHKV_ERR_INVALID, "seq_create: null out pointer");
  HostError e = ctx->host.SeqCreate(seq);
  if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  if (ctx->has_device && IsTileFmt(ctx->cfg.fmt)) {   // a fresh sequence: mean 0, first open buffer
    ctx->host.ResetOpenState(*seq);
    if (cudaSetDevice(ctx->cfg.device) != cudaSuccess) return Fail(ctx, YAHKV_ERR_CUDA, "cudaSetDevice failed");
    YAHKV_CUDA(ctx, cudaDeviceSynchronize());
    YAHKV_CUDA(ctx, cudaMemset(ctx->kmean_dev + static_cast<std::size_t>(*seq) * ctx->cfg.n_layers * kKvHeads * kHeadDim, 0,
                               static_cast<std::size_t>(ctx->cfg.n_layers) * kKvHeads * kHeadDim * sizeof(float)));
  }
  return YAHKV_OK;
}

int yahkv_seq_free(yahkv_ctx* ctx, int32_t seq) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  HostError e = ctx->host.SeqFree(seq);
  return e.code == YAHKV_OK ? YAHKV_OK : FailHost(ctx, std::move(e));
}

int yahkv_seq_reserve(yahkv_ctx* ctx, int32_t seq, int64_t n_tokens) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  HostError e = ctx->host.SeqReserve(seq, n_tokens);
  return e.code == YAHKV_OK ? YAHKV_OK : FailHost(ctx, std::move(e));
}

int yahkv_seq_set_table(yahkv_ctx* ctx, int32_t seq, const int32_t* pages, int32_t n) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  HostError e = ctx->host.SeqSetTable(seq, pages, n);
  return e.code == YAHKV_OK ? YAHKV_OK : FailHost(ctx, std::move(e));
}

int yahkv_seq_table(const yahkv_ctx* ctx, int32_t seq, const int32_t** pages, int32_t* n) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  if (!ctx->host.live(seq)) return Fail(ctx, YAHKV_ERR_INVALID, "seq_table: not a live sequence: " + std::to_string(seq));
  if (pages != nullptr) *pages = ctx->host.table_row(seq);
  if (n != nullptr) *n = ctx->host.n_pages(seq);
  return YAHKV_OK;
}

int yahkv_seq_len(const yahkv_ctx* ctx, int32_t seq, int32_t layer, int64_t* len) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  if (!ctx->host.live(seq)) return Fail(ctx, YAHKV_ERR_INVALID, "seq_len: not a live sequence: " + std::to_string(seq));
  if (layer < 0 || layer >= ctx->cfg.n_layers || len == nullptr) return Fail(ctx, YAHKV_ERR_INVALID, "seq_len: bad layer or null pointer");
  *len = ctx->host.len(seq, layer);
  return YAHKV_OK;
}

int yahkv_seq_set_len(yahkv_ctx* ctx, int32_t seq, int32_t layer, int64_t len) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  if (IsTileFmt(ctx->cfg.fmt) && len != 0)
    return Fail(ctx, YAHKV_ERR_INVALID, "seq_set_len: a YAHKV_FMT_KV8A16 / YAHKV_FMT_KV4A16 sequence can only be reset to length 0 (its open tile holds the newest keys)");
  HostError e = ctx->host.SeqSetLen(seq, layer, len);
  if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  if (IsTileFmt(ctx->cfg.fmt) && layer == -1) ctx->host.ResetOpenState(seq);
  return YAHKV_OK;
}

int yahkv_seq_set_kmean(yahkv_ctx* ctx, int32_t seq, int32_t layer, const float* mean_host) {
  if (int r = RequireDevice(ctx, "seq_set_kmean"); r != YAHKV_OK) return r;
  if (!IsTileFmt(ctx->cfg.fmt)) return Fail(ctx, YAHKV_ERR_INVALID, "seq_set_kmean: only for YAHKV_FMT_KV8A16 / YAHKV_FMT_KV4A16");
  if (!ctx->host.live(seq) || mean_host == nullptr || layer < -1 || layer >= ctx->cfg.n_layers)
    return Fail(ctx, YAHKV_ERR_INVALID, "seq_set_kmean: bad sequence, layer or null pointer");
  for (int l = 0; l < ctx->cfg.n_layers; ++l)
    if ((layer == -1 || layer == l) && ctx->host.len(seq, l) != 0)
      return Fail(ctx, YAHKV_ERR_ORDER, "seq_set_kmean: the mean is fixed once a key has been appended");
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  for (int l = 0; l < ctx->cfg.n_layers; ++l)
    if (layer == -1 || layer == l)
      YAHKV_CUDA(ctx, cudaMemcpy(ctx->kmean_dev + (static_cast<std::size_t>(seq) * ctx->cfg.n_layers + l) * kKvHeads * kHeadDim,
                                 mean_host, static_cast<std::size_t>(kKvHeads) * kHeadDim * sizeof(float), cudaMemcpyHostToDevice));
  return YAHKV_OK;
}

int yahkv_read_open_tile(yahkv_ctx* ctx, int32_t seq, int32_t layer, void* tile_host) {
  if (int r = RequireDevice(ctx, "read_open_tile"); r != YAHKV_OK) return r;
  if (!IsTileFmt(ctx->cfg.fmt)) return Fail(ctx, YAHKV_ERR_INVALID, "read_open_tile: only for YAHKV_FMT_KV8A16 / YAHKV_FMT_KV4A16");
  if (!ctx->host.live(seq) || tile_host == nullptr || layer < 0 || layer >= ctx->cfg.n_layers)
    return Fail(ctx, YAHKV_ERR_INVALID, "read_open_tile: bad sequence, layer or null pointer");
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  const std::size_t row = (static_cast<std::size_t>(seq) * ctx->cfg.n_layers + layer) * 2 + ctx->host.open_cur(seq, layer);
  YAHKV_CUDA(ctx, cudaMemcpy(tile_host, static_cast<const std::uint16_t*>(ctx->open_tiles_dev) + row * kOpenTileHalfs,
                             static_cast<std::size_t>(kOpenTileHalfs) * 2, cudaMemcpyDeviceToHost));
  return YAHKV_OK;
}

int yahkv_pages_free(const yahkv_ctx* ctx, int32_t* n) {
  if (ctx == nullptr || n == nullptr) return YAHKV_ERR_INVALID;
  *n = ctx->host.pages_free();
  return YAHKV_OK;
}

// The append of the tile formats once the slots are planned and uploaded. K: one row per token against its sequence's
// mean. V: one work item per 16-key tile the call touches; the tile of each sequence's newest key also stays in fp16
// (engine/gpu/loom/tools/gen_decode_attn.py:436-573). k_dev / v_dev: fp16 [n_tokens][4][256].
static int TileAppend(yahkv_ctx* ctx, int layer, int n_tokens, const int32_t* seq_ids, const int64_t* positions,
                      const void* k_dev, const void* v_dev, cudaStream_t st) {
  ctx->host.PlanKv8Tiles(layer, n_tokens, seq_ids, positions, &ctx->vwork_scratch);
  ctx->state_row_scratch.resize(static_cast<std::size_t>(n_tokens));
  for (int i = 0; i < n_tokens; ++i)
    ctx->state_row_scratch[static_cast<std::size_t>(i)] = seq_ids[i] * ctx->cfg.n_layers + layer;
  if (int r = StagedUpload(ctx, ctx->state_rows_dev, ctx->state_row_scratch.data(), static_cast<std::size_t>(n_tokens) * 4, st); r != YAHKV_OK)
    return r;
  if (int r = StagedUpload(ctx, ctx->vwork_dev, ctx->vwork_scratch.data(), ctx->vwork_scratch.size() * sizeof(VTileWork), st);
      r != YAHKV_OK)
    return r;
  TimedLaunch tl(ctx, YAHKV_KERNEL_APPEND, st);
  YAHKV_CUDA(ctx, (ctx->cfg.fmt == YAHKV_FMT_KV4A16 ? LaunchKv4AppendK : LaunchKv8AppendK)(
                      ctx->pool, layer, n_tokens, ctx->slots_dev, ctx->state_rows_dev, 0, ctx->kmean_dev, k_dev, st));
  YAHKV_CUDA(ctx, LaunchKv8AppendV(ctx->pool, layer, static_cast<int>(ctx->vwork_scratch.size()), ctx->vwork_dev, 0,
                                   ctx->open_tiles_dev, v_dev, st));
  tl.End();
  ctx->launches += 2;
  return YAHKV_OK;
}

int yahkv_append(yahkv_ctx* ctx, int32_t layer, int32_t n_tokens, const int32_t* seq_ids, const int64_t* positions,
                 const void* k_dev, const void* v_dev, void* stream) {
  if (int r = RequireDevice(ctx, "append"); r != YAHKV_OK) return r;
  if (n_tokens > ctx->cfg.max_batch_tokens) return Fail(ctx, YAHKV_ERR_CAPACITY, "append: more tokens than max_batch_tokens");
  if (n_tokens > 0 && (k_dev == nullptr || v_dev == nullptr)) return Fail(ctx, YAHKV_ERR_INVALID, "append: null K or V pointer");
  HostError e = ctx->host.PlanAppend(layer, n_tokens, seq_ids, positions, ctx->slot_scratch.data());
  if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  if (n_tokens == 0) return YAHKV_OK;
  cudaStream_t st = StreamOf(ctx, stream);
  if (int r = FlushTables(ctx, st); r != YAHKV_OK) return r;
  if (int r = StagedUpload(ctx, ctx->slots_dev, ctx->slot_scratch.data(), static_cast<std::size_t>(n_tokens) * 8, st); r != YAHKV_OK)
    return r;
  if (IsTileFmt(ctx->cfg.fmt)) return TileAppend(ctx, layer, n_tokens, seq_ids, positions, k_dev, v_dev, st);
  TimedLaunch tl(ctx, YAHKV_KERNEL_APPEND, st);
  YAHKV_CUDA(ctx, LaunchAppend(ctx->pool, layer, n_tokens, ctx->slots_dev, k_dev, v_dev, st));
  tl.End();
  ctx->launches += 1;
  return YAHKV_OK;
}

// cos / sin table of the fused RoPE: angle = pos / theta^(2 p / 64), p < 32, evaluated in double precision on the
// host and rounded to f32 once (engine/gpu/loom/yah_fused_qk_rope_f32.loom:5, :32 for the formula and theta).
static int EnsureRopeTable(yahkv_ctx* ctx) {
  if (ctx->rope_tab_dev != nullptr) return YAHKV_OK;
  const int rows = ctx->cfg.max_pages_per_seq * kPageTokens;
  std::vector<float2> tab(static_cast<std::size_t>(rows) * 32);
  double inv_freq[32];
  for (int p = 0; p < 32; ++p) inv_freq[p] = std::pow(1.0e7, -2.0 * p / 64.0);
  for (int pos = 0; pos < rows; ++pos)
    for (int p = 0; p < 32; ++p) {
      const double a = static_cast<double>(pos) * inv_freq[p];
      tab[static_cast<std::size_t>(pos) * 32 + p] = make_float2(static_cast<float>(std::cos(a)), static_cast<float>(std::sin(a)));
    }
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->rope_tab_dev, tab.size(), false));
  YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->rope_pos_dev, static_cast<std::size_t>(ctx->cfg.max_batch_tokens), false));
  if (IsTileFmt(ctx->cfg.fmt))   // fp16 K and V rows between the RoPE kernel and the tile appends
    YAHKV_CUDA(ctx, DevAlloc(ctx, &ctx->rope_kv16_dev, static_cast<std::size_t>(ctx->cfg.max_batch_tokens) * 2 * kKvHeads * kHeadDim, false));
  YAHKV_CUDA(ctx, cudaMemcpy(ctx->rope_tab_dev, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice));
  ctx->rope_rows = rows;
  return YAHKV_OK;
}

int yahkv_rope_append(yahkv_ctx* ctx, int32_t layer, int32_t n_tokens, const int32_t* seq_ids, const int64_t* positions,
                      const float* q_dev, const float* k_dev, const float* v_dev, const float* q_weight_dev,
                      const float* k_weight_dev, float eps, void* q_out_dev, void* stream) {
  if (int r = RequireDevice(ctx, "rope_append"); r != YAHKV_OK) return r;
  if (n_tokens > ctx->cfg.max_batch_tokens) return Fail(ctx, YAHKV_ERR_CAPACITY, "rope_append: more tokens than max_batch_tokens");
  if (n_tokens > 0 && (q_dev == nullptr || k_dev == nullptr || v_dev == nullptr || q_weight_dev == nullptr ||
                       k_weight_dev == nullptr))   // q_out_dev may be null: the query side is then left to the caller
    return Fail(ctx, YAHKV_ERR_INVALID, "rope_append: null pointer");
  if (!(eps >= 0.0F)) return Fail(ctx, YAHKV_ERR_INVALID, "rope_append: eps must be non-negative");
  if (int r = EnsureRopeTable(ctx); r != YAHKV_OK) return r;   // before the plan: a failure here changes no state
  HostError e = ctx->host.PlanAppend(layer, n_tokens, seq_ids, positions, ctx->slot_scratch.data());
  if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  if (n_tokens == 0) return YAHKV_OK;
  ctx->rope_pos_scratch.resize(static_cast<std::size_t>(n_tokens));
  for (int i = 0; i < n_tokens; ++i) ctx->rope_pos_scratch[static_cast<std::size_t>(i)] = static_cast<std::int32_t>(positions[i]);
  cudaStream_t st = StreamOf(ctx, stream);
  if (int r = FlushTables(ctx, st); r != YAHKV_OK) return r;
  if (int r = StagedUpload(ctx, ctx->slots_dev, ctx->slot_scratch.data(), static_cast<std::size_t>(n_tokens) * 8, st); r != YAHKV_OK)
    return r;
  if (int r = StagedUpload(ctx, ctx->rope_pos_dev, ctx->rope_pos_scratch.data(), static_cast<std::size_t>(n_tokens) * 4, st);
      r != YAHKV_OK)
    return r;
  TimedLaunch tl(ctx, YAHKV_KERNEL_APPEND, st);
  YAHKV_CUDA(ctx, LaunchRopeAppend(ctx->pool, layer, n_tokens, ctx->slots_dev, ctx->rope_pos_dev, q_dev, k_dev, v_dev,
                                   q_weight_dev, k_weight_dev, eps, ctx->rope_tab_dev, ctx->rope_rows, q_out_dev,
                                   ctx->rope_kv16_dev, st));
  tl.End();
  ctx->launches += 1;
  if (IsTileFmt(ctx->cfg.fmt)) {   // the kernel left fp16 rows (K after norm and RoPE): the format's own appends take them
    const std::uint16_t* k16 = ctx->rope_kv16_dev;
    const std::uint16_t* v16 = k16 + static_cast<std::size_t>(n_tokens) * kKvHeads * kHeadDim;
    return TileAppend(ctx, layer, n_tokens, seq_ids, positions, k16, v16, st);
  }
  return YAHKV_OK;
}

int yahkv_append_slots(yahkv_ctx* ctx, int32_t layer, int32_t n_tokens, const int64_t* slot_mapping_dev,
                       const void* k_dev, const void* v_dev, void* stream) {
  if (int r = RequireDevice(ctx, "append_slots"); r != YAHKV_OK) return r;
  if (IsTileFmt(ctx->cfg.fmt))
    return Fail(ctx, YAHKV_ERR_INVALID, "append_slots: YAHKV_FMT_KV8A16 / YAHKV_FMT_KV4A16 need the sequence of every token (use yahkv_append)");
  if (layer < 0 || layer >= ctx->cfg.n_layers) return Fail(ctx, YAHKV_ERR_INVALID, "append_slots: layer out of range");
  if (n_tokens < 0) return Fail(ctx, YAHKV_ERR_INVALID, "append_slots: negative token count");
  if (n_tokens == 0) return YAHKV_OK;
  if (slot_mapping_dev == nullptr || k_dev == nullptr || v_dev == nullptr)
    return Fail(ctx, YAHKV_ERR_INVALID, "append_slots: null pointer");
  cudaStream_t st = StreamOf(ctx, stream);
  if (int r = FlushTables(ctx, st); r != YAHKV_OK) return r;
  TimedLaunch tl(ctx, YAHKV_KERNEL_APPEND, st);
  YAHKV_CUDA(ctx, LaunchAppend(ctx->pool, layer, n_tokens, slot_mapping_dev, k_dev, v_dev, st));
  tl.End();
  ctx->launches += 1;
  return YAHKV_OK;
}

static int AttendDecode(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const void* q_dev, bool q_raw,
                        const float* q_weight_dev, float eps, const float* gate_dev, void* out_dev, int32_t out_dtype,
                        int32_t n_splits, void* stream);

int yahkv_attend_decode(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const void* q_dev,
                        const float* gate_dev, void* out_dev, int32_t out_dtype, int32_t n_splits, void* stream) {
  return AttendDecode(ctx, layer, n_seqs, seq_ids, q_dev, false, nullptr, 0.0F, gate_dev, out_dev, out_dtype, n_splits,
                      stream);
}

int yahkv_attend_decode_qraw(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const float* q_raw_dev,
                             const float* q_weight_dev, float eps, const float* gate_dev, void* out_dev,
                             int32_t out_dtype, int32_t n_splits, void* stream) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  if (n_seqs > 0 && q_weight_dev == nullptr) return Fail(ctx, YAHKV_ERR_INVALID, "attend_decode_qraw: null norm weights");
  if (!(eps >= 0.0F)) return Fail(ctx, YAHKV_ERR_INVALID, "attend_decode_qraw: eps must be non-negative");
  if ((reinterpret_cast<std::uintptr_t>(q_raw_dev) & 15) != 0 || (reinterpret_cast<std::uintptr_t>(q_weight_dev) & 15) != 0)
    return Fail(ctx, YAHKV_ERR_INVALID, "attend_decode_qraw: q and the norm weights must be 16-byte aligned");
  return AttendDecode(ctx, layer, n_seqs, seq_ids, q_raw_dev, true, q_weight_dev, eps, gate_dev, out_dev, out_dtype,
                      n_splits, stream);
}

static int AttendDecode(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const void* q_dev, bool q_raw,
                        const float* q_weight_dev, float eps, const float* gate_dev, void* out_dev, int32_t out_dtype,
                        int32_t n_splits, void* stream) {
  if (int r = RequireDevice(ctx, "attend_decode"); r != YAHKV_OK) return r;
  if (q_raw)
    if (int r = EnsureRopeTable(ctx); r != YAHKV_OK) return r;   // before the plan: a failure here changes no state
  if (out_dtype != YAHKV_OUT_F16 && out_dtype != YAHKV_OUT_F32) return Fail(ctx, YAHKV_ERR_INVALID, "attend_decode: bad out_dtype");
  if (n_seqs > 0 && (q_dev == nullptr || out_dev == nullptr)) return Fail(ctx, YAHKV_ERR_INVALID, "attend_decode: null q or out pointer");
  bool changed = false;
  HostError e = ctx->host.PlanDecode(layer, n_seqs, seq_ids, n_splits, ctx->cfg.max_splits, ctx->max_units, &changed);
  if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  if (n_seqs == 0) return YAHKV_OK;
  // The plan is cached on the host from here on; anything that fails before both kernels are queued drops it, so the
  // next identical call plans and uploads again instead of launching on a unit list that never reached the device.
  struct PlanGuard {
    KvHost* host;
    bool keep = false;
    ~PlanGuard() {
      if (!keep) host->InvalidateDecodePlan();
    }
  } guard{&ctx->host};
  cudaStream_t st = StreamOf(ctx, stream);
  if (int r = FlushTables(ctx, st); r != YAHKV_OK) return r;
  const bool kv8 = IsTileFmt(ctx->cfg.fmt);
  if (kv8) {
    // Every unit carries its sequence's current open-tile buffer of THIS layer. The layers of a step usually agree on
    // it, so the list is uploaded again only when the plan or one of those indices differs from what the device holds.
    const auto& planned = ctx->host.units();
    bool same = !changed && ctx->unit_scratch.size() == planned.size();
    if (!same) ctx->unit_scratch = planned;
    for (DecodeUnit& u : ctx->unit_scratch) {
      const std::int32_t cur = ctx->host.open_cur(u.seq, layer);
      if (u.pad != cur) u.pad = cur, same = false;
    }
    changed = !same;
  }
  const auto& units = kv8 ? ctx->unit_scratch : ctx->host.units();
  const auto& items = ctx->host.items();
  if (changed) {
    // One staging buffer holds both lists so they share a completion event.
    const std::size_t ub = units.size() * sizeof(DecodeUnit), ib = items.size() * sizeof(CombineItem);
    char* buf = nullptr;
    YAHKV_CUDA(ctx, ctx->staging.Acquire(ub + ib, &buf));
    std::memcpy(buf, units.data(), ub);
    std::memcpy(buf + ub, items.data(), ib);
    YAHKV_CUDA(ctx, cudaMemcpyAsync(ctx->units_dev, buf, ub, cudaMemcpyHostToDevice, st));
    YAHKV_CUDA(ctx, cudaMemcpyAsync(ctx->items_dev, buf + ub, ib, cudaMemcpyHostToDevice, st));
    YAHKV_CUDA(ctx, ctx->staging.Release(st));
  }
  DecodeLaunch a{};
  a.kmap = &ctx->kmap, a.vmap = &ctx->vmap, a.pool = ctx->pool, a.layer = layer;
  a.tables_dev = ctx->tables_dev, a.table_stride = ctx->cfg.max_pages_per_seq;
  a.units_dev = ctx->units_dev, a.n_units = static_cast<int>(units.size());
  a.items_dev = ctx->items_dev, a.n_seqs = n_seqs;
  a.q_dev = q_dev, a.gate_dev = gate_dev, a.out_dev = out_dev, a.out_f32 = out_dtype == YAHKV_OUT_F32;
  a.q_raw = q_raw, a.q_weight_dev = q_weight_dev, a.q_eps = eps, a.rope_tab_dev = ctx->rope_tab_dev, a.rope_rows = ctx->rope_rows;
  a.scale_log2 = ctx->scale_log2;
  a.partial_acc = ctx->partial_acc, a.partial_ml = ctx->partial_ml, a.status_dev = ctx->status_dev;
  // The merge runs as its own small launch: letting the last-arriving unit merge inside the part kernel was measured
  // 1% slower end to end (every CTA then pays a fence and an atomic on exit).
  TimedLaunch tp(ctx, YAHKV_KERNEL_DECODE_PART, st);
  cudaError_t le = ctx->cfg.fmt == YAHKV_FMT_KV4A16 ? LaunchKv4DecodePart(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                   : kv8                            ? LaunchKv8DecodePart(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                   : ctx->cfg.fmt == YAHKV_FMT_F16  ? LaunchF16DecodePart(a, st)
                                                    : LaunchDecodePart(a, st);
  tp.End();
  if (le == cudaSuccess) {
    TimedLaunch tc(ctx, YAHKV_KERNEL_DECODE_COMBINE, st);
    le = LaunchDecodeCombine(a, st);
    tc.End();
  }
  if (le != cudaSuccess) return FailCuda(ctx, "decode attention launch", le);
  guard.keep = true;
  ctx->launches += 2;
  return YAHKV_OK;
}

static int AttendPrefill(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const int32_t* chunk_lens,
                         const void* q_dev, bool q_raw, const float* q_weight_dev, float eps, const float* gate_dev,
                         void* out_dev, int32_t out_dtype, void* stream);

int yahkv_attend_prefill(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids,
                         const int32_t* chunk_lens, const void* q_dev, const float* gate_dev, void* out_dev,
                         int32_t out_dtype, void* stream) {
  return AttendPrefill(ctx, layer, n_seqs, seq_ids, chunk_lens, q_dev, false, nullptr, 0.0F, gate_dev, out_dev, out_dtype,
                       stream);
}

int yahkv_attend_prefill_qraw(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids,
                              const int32_t* chunk_lens, const float* q_raw_dev, const float* q_weight_dev, float eps,
                              const float* gate_dev, void* out_dev, int32_t out_dtype, void* stream) {
  if (ctx == nullptr) return YAHKV_ERR_INVALID;
  if (n_seqs > 0 && q_weight_dev == nullptr) return Fail(ctx, YAHKV_ERR_INVALID, "attend_prefill_qraw: null norm weights");
  if (!(eps >= 0.0F)) return Fail(ctx, YAHKV_ERR_INVALID, "attend_prefill_qraw: eps must be non-negative");
  if ((reinterpret_cast<std::uintptr_t>(q_weight_dev) & 7) != 0)
    return Fail(ctx, YAHKV_ERR_INVALID, "attend_prefill_qraw: the norm weights must be 8-byte aligned");
  return AttendPrefill(ctx, layer, n_seqs, seq_ids, chunk_lens, q_raw_dev, true, q_weight_dev, eps, gate_dev, out_dev,
                       out_dtype, stream);
}

static int AttendPrefill(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const int32_t* chunk_lens,
                         const void* q_dev, bool q_raw, const float* q_weight_dev, float eps, const float* gate_dev,
                         void* out_dev, int32_t out_dtype, void* stream) {
  if (int r = RequireDevice(ctx, "attend_prefill"); r != YAHKV_OK) return r;
  if (q_raw)
    if (int r = EnsureRopeTable(ctx); r != YAHKV_OK) return r;
  if (out_dtype != YAHKV_OUT_F16 && out_dtype != YAHKV_OUT_F32) return Fail(ctx, YAHKV_ERR_INVALID, "attend_prefill: bad out_dtype");
  if (n_seqs > 0 && (q_dev == nullptr || out_dev == nullptr)) return Fail(ctx, YAHKV_ERR_INVALID, "attend_prefill: null q or out pointer");
  if ((reinterpret_cast<std::uintptr_t>(q_dev) & 15) != 0 || (reinterpret_cast<std::uintptr_t>(out_dev) & 15) != 0)
    return Fail(ctx, YAHKV_ERR_INVALID, "attend_prefill: q and out must be 16-byte aligned");
  std::int64_t rows = 0, scratch_rows = 0;
  int max_pages = 0;
  int n_parts = 0;
  HostError e = ctx->host.PlanPrefill(layer, n_seqs, seq_ids, chunk_lens, ctx->cfg.max_batch_tokens, ctx->n_sm,
                                      &ctx->pseq_scratch, &ctx->tile_scratch, &ctx->merge_scratch, &n_parts, &rows,
                                      &scratch_rows, &max_pages);
  if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  if (ctx->tile_scratch.empty()) return YAHKV_OK;
  if (static_cast<int>(ctx->tile_scratch.size()) > ctx->max_tiles) return Fail(ctx, YAHKV_ERR_CAPACITY, "attend_prefill: too many tiles");
  const bool kv8 = IsTileFmt(ctx->cfg.fmt);
  if (kv8)   // the tile of each sequence's newest key is read from its current open buffer
    for (PrefillSeq& ps : ctx->pseq_scratch) ps.pad[0] = ctx->host.open_cur(ps.seq, layer);
  cudaStream_t st = StreamOf(ctx, stream);
  // The fp16 scratch of the dequantize pass: fixed at create when the configuration sizes it, else grown to the
  // largest call seen (a one-time cost per high-water mark, with a device synchronisation).
  if (scratch_rows > ctx->p16_rows) {
    if (ctx->cfg.max_prefill_keys > 0)
      return Fail(ctx, YAHKV_ERR_CAPACITY, "attend_prefill: the call covers " + std::to_string(scratch_rows / kKvHeads) +
                                               " cached keys, max_prefill_keys is " + std::to_string(ctx->cfg.max_prefill_keys));
    YAHKV_CUDA(ctx, cudaDeviceSynchronize());
    if (int r = ResizePrefillScratch(ctx, scratch_rows); r != YAHKV_OK) return r;
  }
  if (int r = FlushTables(ctx, st); r != YAHKV_OK) return r;
  {
    const std::size_t sb = ctx->pseq_scratch.size() * sizeof(PrefillSeq), tb = ctx->tile_scratch.size() * sizeof(PrefillTile);
    const std::size_t mb = ctx->merge_scratch.size() * sizeof(PrefillMerge);
    char* buf = nullptr;
    YAHKV_CUDA(ctx, ctx->staging.Acquire(sb + tb + mb, &buf));
    std::memcpy(buf, ctx->pseq_scratch.data(), sb);
    std::memcpy(buf + sb, ctx->tile_scratch.data(), tb);
    if (mb > 0) std::memcpy(buf + sb + tb, ctx->merge_scratch.data(), mb);
    YAHKV_CUDA(ctx, cudaMemcpyAsync(ctx->pseqs_dev, buf, sb, cudaMemcpyHostToDevice, st));
    YAHKV_CUDA(ctx, cudaMemcpyAsync(ctx->tiles_dev, buf + sb, tb, cudaMemcpyHostToDevice, st));
    if (mb > 0) YAHKV_CUDA(ctx, cudaMemcpyAsync(ctx->merges_dev, buf + sb + tb, mb, cudaMemcpyHostToDevice, st));
    YAHKV_CUDA(ctx, ctx->staging.Release(st));
  }
  PrefillLaunch a{};
  a.pool = ctx->pool, a.layer = layer;
  a.tables_dev = ctx->tables_dev, a.table_stride = ctx->cfg.max_pages_per_seq;
  a.seqs_dev = ctx->pseqs_dev, a.n_seqs = n_seqs, a.max_pages = max_pages;
  a.k16_dev = ctx->k16_dev, a.v16_dev = ctx->v16_dev;
  a.q_dev = q_dev, a.k16map = &ctx->k16map, a.v16map = &ctx->v16map;
  a.q_raw = q_raw, a.q_weight_dev = q_weight_dev, a.q_eps = eps, a.rope_tab_dev = ctx->rope_tab_dev, a.rope_rows = ctx->rope_rows;
  a.tiles_dev = ctx->tiles_dev, a.n_tiles = static_cast<int>(ctx->tile_scratch.size());
  a.merges_dev = ctx->merges_dev, a.n_merges = static_cast<int>(ctx->merge_scratch.size());
  a.part_acc = ctx->part_acc_dev, a.part_ml = ctx->part_ml_dev;
  a.gate_dev = gate_dev, a.out_dev = out_dev, a.out_f32 = out_dtype == YAHKV_OUT_F32;
  a.scale_log2 = ctx->scale_log2, a.status_dev = ctx->status_dev;
  {
    TimedLaunch tl(ctx, YAHKV_KERNEL_PREFILL_DEQUANT, st);
    YAHKV_CUDA(ctx, ctx->cfg.fmt == YAHKV_FMT_KV4A16 ? LaunchKv4PrefillDequant(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                    : kv8                            ? LaunchKv8PrefillDequant(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                                                     : LaunchPrefillDequant(a, st));
    tl.End();
  }
  TimedLaunch tl(ctx, YAHKV_KERNEL_PREFILL, st);
  YAHKV_CUDA(ctx, LaunchPrefill(a, st));
  tl.End();
  ctx->launches += a.n_merges > 0 ? 3 : 2;
  return YAHKV_OK;
}

int yahkv_decode_step_host_async(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids,
                                 const void* k_host, const void* v_host, const void* q_host, const float* gate_host,
                                 void* out_host, int32_t out_dtype) {
  if (int r = RequireDevice(ctx, "decode_step_host"); r != YAHKV_OK) return r;
  if (n_seqs <= 0 || n_seqs > ctx->cfg.max_seqs) return Fail(ctx, YAHKV_ERR_INVALID, "decode_step_host: bad n_seqs");
  if (seq_ids == nullptr || k_host == nullptr || v_host == nullptr || q_host == nullptr || out_host == nullptr)
    return Fail(ctx, YAHKV_ERR_INVALID, "decode_step_host: null pointer");
  if (layer < 0 || layer >= ctx->cfg.n_layers) return Fail(ctx, YAHKV_ERR_INVALID, "decode_step_host: layer out of range");
  if (out_dtype != YAHKV_OUT_F16 && out_dtype != YAHKV_OUT_F32) return Fail(ctx, YAHKV_ERR_INVALID, "decode_step_host: bad out_dtype");
  ctx->pos_scratch.resize(static_cast<std::size_t>(n_seqs));
  for (int b = 0; b < n_seqs; ++b) {
    if (!ctx->host.live(seq_ids[b])) return Fail(ctx, YAHKV_ERR_INVALID, "decode_step_host: not a live sequence");
    const std::int64_t pos = ctx->host.len(seq_ids[b], layer);
    ctx->pos_scratch[static_cast<std::size_t>(b)] = pos;
    HostError e = ctx->host.SeqReserve(seq_ids[b], pos + 1);
    if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  }
  yahkv_ctx::HostStage& h = ctx->hst[ctx->hst_next];
  cudaStream_t st = ctx->stream, in = ctx->h2d_stream, back = ctx->d2h_stream;
  const std::size_t kvb = static_cast<std::size_t>(n_seqs) * kKvHeads * kHeadDim * 2;
  const std::size_t qb = static_cast<std::size_t>(n_seqs) * kQHeads * kHeadDim * 2;
  const std::size_t ob = static_cast<std::size_t>(n_seqs) * kQHeads * kHeadDim * (out_dtype == YAHKV_OUT_F32 ? 4 : 2);
  // inputs: behind the kernels that last read this set, on the copy-in stream
  if (h.used) YAHKV_CUDA(ctx, cudaStreamWaitEvent(in, h.compute_done, 0));
  YAHKV_CUDA(ctx, cudaMemcpyAsync(h.k, k_host, kvb, cudaMemcpyHostToDevice, in));
  YAHKV_CUDA(ctx, cudaMemcpyAsync(h.v, v_host, kvb, cudaMemcpyHostToDevice, in));
  YAHKV_CUDA(ctx, cudaMemcpyAsync(h.q, q_host, qb, cudaMemcpyHostToDevice, in));
  if (gate_host != nullptr)
    YAHKV_CUDA(ctx, cudaMemcpyAsync(h.gate, gate_host, static_cast<std::size_t>(n_seqs) * kQHeads * kHeadDim * 4,
                                    cudaMemcpyHostToDevice, in));
  YAHKV_CUDA(ctx, cudaEventRecord(h.in_ready, in));
  // kernels: behind the inputs and behind the read-back that last used this set's output buffer
  YAHKV_CUDA(ctx, cudaStreamWaitEvent(st, h.in_ready, 0));
  if (h.used) YAHKV_CUDA(ctx, cudaStreamWaitEvent(st, h.out_done, 0));
  h.used = true;
  ctx->hst_next ^= 1;
  if (int r = yahkv_append(ctx, layer, n_seqs, seq_ids, ctx->pos_scratch.data(), h.k, h.v, st); r != YAHKV_OK) return r;
  if (int r = yahkv_attend_decode(ctx, layer, n_seqs, seq_ids, h.q, gate_host != nullptr ? h.gate : nullptr, h.out,
                                  out_dtype, 0, st);
      r != YAHKV_OK)
    return r;
  YAHKV_CUDA(ctx, cudaEventRecord(h.compute_done, st));
  // output: behind the kernels, on the copy-out stream
  YAHKV_CUDA(ctx, cudaStreamWaitEvent(back, h.compute_done, 0));
  YAHKV_CUDA(ctx, cudaMemcpyAsync(out_host, h.out, ob, cudaMemcpyDeviceToHost, back));
  YAHKV_CUDA(ctx, cudaEventRecord(h.out_done, back));
  return YAHKV_OK;
}

int yahkv_decode_step_host_wait(yahkv_ctx* ctx) {
  if (int r = RequireDevice(ctx, "decode_step_host_wait"); r != YAHKV_OK) return r;
  YAHKV_CUDA(ctx, cudaStreamSynchronize(ctx->d2h_stream));   // every read-back follows its kernels
  return CheckStatus(ctx);
}

int yahkv_decode_step_host(yahkv_ctx* ctx, int32_t layer, int32_t n_seqs, const int32_t* seq_ids, const void* k_host,
                           const void* v_host, const void* q_host, const float* gate_host, void* out_host,
                           int32_t out_dtype) {
  if (int r = yahkv_decode_step_host_async(ctx, layer, n_seqs, seq_ids, k_host, v_host, q_host, gate_host, out_host,
                                           out_dtype);
      r != YAHKV_OK)
    return r;
  YAHKV_CUDA(ctx, cudaStreamSynchronize(ctx->d2h_stream));
  return CheckStatus(ctx);
}

int yahkv_sync(yahkv_ctx* ctx) {
  if (int r = RequireDevice(ctx, "sync"); r != YAHKV_OK) return r;
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  return CheckStatus(ctx);
}

// GGUF int8 codes <-> the pools' device representation (kernels.cuh): V bytes flip, the same way in both
// directions; K bytes and q4_0 are untouched.
static void FlipQ8(int fmt, int side, std::uint8_t* codes, std::size_t n) {
  if (fmt != YAHKV_FMT_Q8_0 || Q8FlipByte(side) == 0) return;
  for (std::size_t i = 0; i < n; ++i) codes[i] ^= static_cast<std::uint8_t>(Q8FlipByte(side));
}

static int PageAccess(yahkv_ctx* ctx, int32_t layer, int32_t side, int32_t page, void* codes_host, void* scales_host,
                      bool write) {
  if (int r = RequireDevice(ctx, write ? "write_page" : "read_page"); r != YAHKV_OK) return r;
  if (layer < 0 || layer >= ctx->cfg.n_layers || page < 0 || page >= ctx->cfg.num_pages ||
      (side != YAHKV_SIDE_K && side != YAHKV_SIDE_V))
    return Fail(ctx, YAHKV_ERR_INVALID, "page access: layer, side or page out of range");
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  const std::size_t rec = (static_cast<std::size_t>(layer) * ctx->cfg.num_pages + page) * kKvHeads;
  std::uint8_t* codes = (side == YAHKV_SIDE_K ? ctx->pool.kcodes : ctx->pool.vcodes) + rec * RecordCodeBytes(ctx->cfg.fmt);
  const std::size_t rsb = static_cast<std::size_t>(RecordScaleBytes(ctx->cfg.fmt, side));
  std::uint16_t* scales = (side == YAHKV_SIDE_K ? ctx->pool.kscales : ctx->pool.vscales) + rec * (rsb / 2);
  const std::size_t cb = static_cast<std::size_t>(kKvHeads) * RecordCodeBytes(ctx->cfg.fmt);
  const std::size_t sb = static_cast<std::size_t>(kKvHeads) * rsb;
  if (codes_host != nullptr) {   // q8_0 codes cross the boundary as GGUF int8, the V pool holds them sign-flipped
    if (write) {
      std::vector<std::uint8_t> tmp(static_cast<const std::uint8_t*>(codes_host), static_cast<const std::uint8_t*>(codes_host) + cb);
      FlipQ8(ctx->cfg.fmt, side, tmp.data(), cb);
      YAHKV_CUDA(ctx, cudaMemcpy(codes, tmp.data(), cb, cudaMemcpyHostToDevice));
    } else {
      YAHKV_CUDA(ctx, cudaMemcpy(codes_host, codes, cb, cudaMemcpyDeviceToHost));
      FlipQ8(ctx->cfg.fmt, side, static_cast<std::uint8_t*>(codes_host), cb);
    }
  }
  if (scales_host != nullptr)
    YAHKV_CUDA(ctx, write ? cudaMemcpy(scales, scales_host, sb, cudaMemcpyHostToDevice)
                          : cudaMemcpy(scales_host, scales, sb, cudaMemcpyDeviceToHost));
  return YAHKV_OK;
}

int yahkv_read_page(yahkv_ctx* ctx, int32_t layer, int32_t side, int32_t page, void* codes_host, void* scales_host) {
  return PageAccess(ctx, layer, side, page, codes_host, scales_host, false);
}

int yahkv_write_page(yahkv_ctx* ctx, int32_t layer, int32_t side, int32_t page, const void* codes_host,
                     const void* scales_host) {
  return PageAccess(ctx, layer, side, page, const_cast<void*>(codes_host), const_cast<void*>(scales_host), true);
}

int yahkv_export_token(yahkv_ctx* ctx, int32_t layer, int32_t seq, int64_t pos, void* k_blocks, void* v_blocks) {
  if (int r = RequireDevice(ctx, "export_token"); r != YAHKV_OK) return r;
  if (IsTileFmt(ctx->cfg.fmt) || ctx->cfg.fmt == YAHKV_FMT_F16)
    return Fail(ctx, YAHKV_ERR_INVALID, "export_token: only the GGUF formats have a block form (use yahkv_read_page)");
  if (layer < 0 || layer >= ctx->cfg.n_layers) return Fail(ctx, YAHKV_ERR_INVALID, "export_token: layer out of range");
  if (!ctx->host.live(seq)) return Fail(ctx, YAHKV_ERR_INVALID, "export_token: not a live sequence");
  if (pos < 0 || pos >= static_cast<std::int64_t>(ctx->host.n_pages(seq)) * kPageTokens)
    return Fail(ctx, YAHKV_ERR_INVALID, "export_token: position outside the reserved pages");
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  const int page = ctx->host.table_row(seq)[pos / kPageTokens];
  const int tok = static_cast<int>(pos % kPageTokens);
  const int cbytes = CodeBytes(ctx->cfg.fmt), bcodes = cbytes / kBlocksPerRow;
  for (int side = 0; side < 2; ++side) {
    auto* dst = static_cast<std::uint8_t*>(side == 0 ? k_blocks : v_blocks);
    if (dst == nullptr) continue;
    for (int h = 0; h < kKvHeads; ++h) {
      const std::size_t rec = (static_cast<std::size_t>(layer) * ctx->cfg.num_pages + page) * kKvHeads + h;
      std::uint8_t codes[256];
      std::uint16_t scales[kBlocksPerRow];
      const std::uint8_t* cs = (side == 0 ? ctx->pool.kcodes : ctx->pool.vcodes) + rec * RecordCodeBytes(ctx->cfg.fmt) +
                               static_cast<std::size_t>(tok) * cbytes;
      const std::uint16_t* ss = (side == 0 ? ctx->pool.kscales : ctx->pool.vscales) + rec * kPageTokens * kBlocksPerRow +
                                static_cast<std::size_t>(tok) * kBlocksPerRow;
      YAHKV_CUDA(ctx, cudaMemcpy(codes, cs, static_cast<std::size_t>(cbytes), cudaMemcpyDeviceToHost));
      FlipQ8(ctx->cfg.fmt, side, codes, static_cast<std::size_t>(cbytes));
      YAHKV_CUDA(ctx, cudaMemcpy(scales, ss, sizeof(scales), cudaMemcpyDeviceToHost));
      for (int b = 0; b < kBlocksPerRow; ++b) {
        std::memcpy(dst, &scales[b], 2);
        std::memcpy(dst + 2, codes + b * bcodes, static_cast<std::size_t>(bcodes));
        dst += 2 + bcodes;
      }
    }
  }
  return YAHKV_OK;
}

int yahkv_kernel_timing(yahkv_ctx* ctx, int32_t enable) {
  if (int r = RequireDevice(ctx, "kernel_timing"); r != YAHKV_OK) return r;
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  for (auto& list : ctx->timing_events) {
    for (auto& pr : list) ctx->event_pool.push_back(pr.first), ctx->event_pool.push_back(pr.second);
    list.clear();
  }
  ctx->timing = enable != 0;
  return YAHKV_OK;
}

int yahkv_kernel_timing_read(yahkv_ctx* ctx, int32_t kernel, double* total_ms, int64_t* launches) {
  if (int r = RequireDevice(ctx, "kernel_timing_read"); r != YAHKV_OK) return r;
  if (kernel < 0 || kernel >= YAHKV_KERNEL_COUNT || total_ms == nullptr || launches == nullptr)
    return Fail(ctx, YAHKV_ERR_INVALID, "kernel_timing_read: bad kernel id or null pointer");
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  double sum = 0;
  for (auto& pr : ctx->timing_events[kernel]) {
    float ms = 0;
    YAHKV_CUDA(ctx, cudaEventElapsedTime(&ms, pr.first, pr.second));
    sum += ms;
  }
  *total_ms = sum;
  *launches = static_cast<std::int64_t>(ctx->timing_events[kernel].size());
  return YAHKV_OK;
}

// ---- device-resident decode batches ------------------------------------------------------------------------
struct yahkv_batch {
  yahkv_ctx* ctx = nullptr;
  std::vector<std::int32_t> seqs;
  std::vector<std::int32_t> lens;       // host mirror of lens_dev (committed steps only)
  std::vector<BatchSeq> rows;
  int total_units = 0;
  int horizon = 0;
  std::int32_t* lens_dev = nullptr;
  BatchSeq* rows_dev = nullptr;
  DecodeUnit* units_dev = nullptr;
  CombineItem* items_dev = nullptr;
  std::int64_t* slots_dev = nullptr;
  VTileWork* vwork_dev = nullptr;          // tile formats: the step's V tile work item per row
  std::int32_t* state_rows_dev = nullptr;  // tile formats: layer-0 state row per row
  int units_cap = 0;
  int n_splits = 0;      // units per (sequence, kv head) asked for with yahkv_batch_set_splits; 0 = automatic
  int unit_pages = 0;    // pages per unit of the prepared horizon (a parameter of the plan kernel)
};
namespace {
constexpr int kBatchUnitPages = 24;   // the automatic planner's unit size on large batches (kv_host.hpp)
void BatchFree(yahkv_batch* b) {
  for (void* p : {static_cast<void*>(b->lens_dev), static_cast<void*>(b->rows_dev), static_cast<void*>(b->units_dev),
                  static_cast<void*>(b->items_dev), static_cast<void*>(b->slots_dev), static_cast<void*>(b->vwork_dev),
                  static_cast<void*>(b->state_rows_dev)})
    if (p != nullptr) cudaFree(p);
  delete b;
}
}  // namespace

int yahkv_batch_create(yahkv_ctx* ctx, int32_t n_seqs, const int32_t* seq_ids, yahkv_batch** out) {
  if (int r = RequireDevice(ctx, "batch_create"); r != YAHKV_OK) return r;
  if (out == nullptr) return Fail(ctx, YAHKV_ERR_INVALID, "batch_create: null out pointer");
  *out = nullptr;
  if (n_seqs <= 0 || n_seqs > ctx->cfg.max_seqs || seq_ids == nullptr) return Fail(ctx, YAHKV_ERR_INVALID, "batch_create: bad sequence list");
  if (ctx->host.kv_head_count() != kKvHeads) return Fail(ctx, YAHKV_ERR_INVALID, "batch_create: decode batches need a context that holds all four kv heads");
  auto* b = new (std::nothrow) yahkv_batch();
  if (b == nullptr) return Fail(ctx, YAHKV_ERR_INVALID, "batch_create: out of host memory");
  b->ctx = ctx;
  for (int i = 0; i < n_seqs; ++i) {
    const int s = seq_ids[i];
    if (!ctx->host.live(s)) {
      delete b;
      return Fail(ctx, YAHKV_ERR_INVALID, "batch_create: not a live sequence: " + std::to_string(s));
    }
    const std::int64_t n = ctx->host.len(s, 0);
    for (int l = 1; l < ctx->cfg.n_layers; ++l)
      if (ctx->host.len(s, l) != n) {
        delete b;
        return Fail(ctx, YAHKV_ERR_ORDER, "batch_create: sequence " + std::to_string(s) + " has different lengths in its layers");
      }
    b->seqs.push_back(s);
    b->lens.push_back(static_cast<std::int32_t>(n));
  }
  b->units_cap = ctx->max_units;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&b->lens_dev), sizeof(std::int32_t) * n_seqs);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b->rows_dev), sizeof(BatchSeq) * n_seqs);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b->units_dev), sizeof(DecodeUnit) * b->units_cap);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b->items_dev), sizeof(CombineItem) * n_seqs * kKvHeads);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&b->slots_dev), sizeof(std::int64_t) * n_seqs);
  if (e == cudaSuccess && IsTileFmt(ctx->cfg.fmt)) e = cudaMalloc(reinterpret_cast<void**>(&b->vwork_dev), sizeof(VTileWork) * n_seqs);
  if (e == cudaSuccess && IsTileFmt(ctx->cfg.fmt)) e = cudaMalloc(reinterpret_cast<void**>(&b->state_rows_dev), sizeof(std::int32_t) * n_seqs);
  if (e != cudaSuccess) {
    BatchFree(b);
    return FailCuda(ctx, "batch_create", e);
  }
  *out = b;
  return YAHKV_OK;
}

void yahkv_batch_destroy(yahkv_batch* b) {
  if (b == nullptr) return;
  cudaSetDevice(b->ctx->cfg.device);
  cudaDeviceSynchronize();
  BatchFree(b);
}

int yahkv_batch_set_splits(yahkv_batch* b, int32_t n_splits) {
  if (b == nullptr) return YAHKV_ERR_INVALID;
  yahkv_ctx* ctx = b->ctx;
  if (n_splits < 0) return Fail(ctx, YAHKV_ERR_INVALID, "batch_set_splits: negative n_splits");
  if (n_splits > ctx->cfg.max_splits) return Fail(ctx, YAHKV_ERR_CAPACITY, "batch_set_splits: n_splits above max_splits");
  b->n_splits = n_splits;   // takes effect at the next batch_prepare
  return YAHKV_OK;
}

int yahkv_batch_prepare(yahkv_batch* b, int32_t horizon_steps, int32_t* layout_changed, void* stream) {
  if (b == nullptr) return YAHKV_ERR_INVALID;
  yahkv_ctx* ctx = b->ctx;
  if (int r = RequireDevice(ctx, "batch_prepare"); r != YAHKV_OK) return r;
  if (horizon_steps < 1) return Fail(ctx, YAHKV_ERR_INVALID, "batch_prepare: horizon must be at least one step");
  const int n = static_cast<int>(b->seqs.size());
  // pages for every position the next `horizon_steps` steps will append: the table widths and the pool's free pages
  // are checked for the whole batch first, so a refusal changes nothing
  std::int64_t new_pages = 0;
  for (int i = 0; i < n; ++i) {
    if (!ctx->host.live(b->seqs[i]) || ctx->host.len(b->seqs[i], 0) != b->lens[i])
      return Fail(ctx, YAHKV_ERR_ORDER, "batch_prepare: a sequence of the batch was freed or changed outside the batch");
    // Tile formats: the layers of a sequence share one plan per step, so they must agree on the open-tile buffer
    // (they do whenever every layer was appended with the same calls).
    for (int l = 1; IsTileFmt(ctx->cfg.fmt) && l < ctx->cfg.n_layers; ++l)
      if (ctx->host.open_cur(b->seqs[i], l) != ctx->host.open_cur(b->seqs[i], 0))
        return Fail(ctx, YAHKV_ERR_ORDER, "batch_prepare: the layers of sequence " + std::to_string(b->seqs[i]) +
                                              " were appended with different chunkings (their open tiles differ)");
    const std::int64_t need = (static_cast<std::int64_t>(b->lens[i]) + horizon_steps + kPageTokens - 1) / kPageTokens;
    if (need > ctx->cfg.max_pages_per_seq) return Fail(ctx, YAHKV_ERR_CAPACITY, "batch_prepare: horizon exceeds max_pages_per_seq");
    new_pages += std::max<std::int64_t>(need - ctx->host.n_pages(b->seqs[i]), 0);
  }
  if (new_pages > ctx->host.pages_free())
    return Fail(ctx, YAHKV_ERR_NO_PAGES, "batch_prepare: the horizon needs " + std::to_string(new_pages) +
                                             " new pages, " + std::to_string(ctx->host.pages_free()) + " are free");
  for (int i = 0; i < n; ++i) {
    HostError e = ctx->host.SeqReserve(b->seqs[i], static_cast<std::int64_t>(b->lens[i]) + horizon_steps);
    if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  }
  // Pages per unit, the same for every sequence of the batch (the plan kernel cuts every sequence at multiples of it):
  // the automatic size, or what the asked-for split count gives on the longest sequence; never so small that a
  // sequence would need more than max_splits units (its last unit would otherwise take all the rest). Even, because
  // the part kernels' two page sets take alternate pages.
  int unit_pages = b->n_splits > 0 ? 1 : kBatchUnitPages;
  for (int i = 0; i < n; ++i) {
    const int pages = (b->lens[i] + horizon_steps + kPageTokens - 1) / kPageTokens;
    const int cap = b->n_splits > 0 ? b->n_splits : ctx->cfg.max_splits;
    unit_pages = std::max(unit_pages, (pages + cap - 1) / cap);
  }
  if (unit_pages > 1) unit_pages += unit_pages & 1;
  // units reserved per sequence, the longest sequences first (CTAs are handed out in index order)
  std::vector<int> order(static_cast<std::size_t>(n));
  for (int i = 0; i < n; ++i) order[static_cast<std::size_t>(i)] = i;
  std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return b->lens[x] > b->lens[y]; });
  std::vector<BatchSeq> rows(static_cast<std::size_t>(n));
  int total = 0;
  for (int i : order) {
    const int pages = (b->lens[i] + horizon_steps + kPageTokens - 1) / kPageTokens;
    BatchSeq r{};
    r.seq_row = b->seqs[i];
    r.open_cur = IsTileFmt(ctx->cfg.fmt) ? ctx->host.open_cur(b->seqs[i], 0) : 0;
    r.n_units = std::min(std::max((pages + unit_pages - 1) / unit_pages, 1), ctx->cfg.max_splits);
    r.first_unit = total;
    total += r.n_units * kKvHeads;
    rows[static_cast<std::size_t>(i)] = r;
  }
  if (total > b->units_cap) return Fail(ctx, YAHKV_ERR_CAPACITY, "batch_prepare: more split-K units than the workspace holds");
  bool changed = rows.size() != b->rows.size() || total != b->total_units || unit_pages != b->unit_pages;
  for (std::size_t i = 0; !changed && i < rows.size(); ++i)
    changed = rows[i].n_units != b->rows[i].n_units || rows[i].first_unit != b->rows[i].first_unit;
  if (layout_changed != nullptr) *layout_changed = changed ? 1 : 0;
  cudaStream_t st = StreamOf(ctx, stream);
  if (int r = FlushTables(ctx, st); r != YAHKV_OK) return r;
  {
    const std::size_t lb = sizeof(std::int32_t) * static_cast<std::size_t>(n), rb = sizeof(BatchSeq) * static_cast<std::size_t>(n);
    char* buf = nullptr;
    YAHKV_CUDA(ctx, ctx->staging.Acquire(lb + rb, &buf));
    std::memcpy(buf, b->lens.data(), lb);
    std::memcpy(buf + lb, rows.data(), rb);
    YAHKV_CUDA(ctx, cudaMemcpyAsync(b->lens_dev, buf, lb, cudaMemcpyHostToDevice, st));
    YAHKV_CUDA(ctx, cudaMemcpyAsync(b->rows_dev, buf + lb, rb, cudaMemcpyHostToDevice, st));
    YAHKV_CUDA(ctx, ctx->staging.Release(st));
  }
  b->rows = std::move(rows);
  b->total_units = total;
  b->unit_pages = unit_pages;
  b->horizon = horizon_steps;
  return YAHKV_OK;
}

int yahkv_batch_plan(yahkv_batch* b, void* stream) {
  if (b == nullptr) return YAHKV_ERR_INVALID;
  yahkv_ctx* ctx = b->ctx;
  if (int r = RequireDevice(ctx, "batch_plan"); r != YAHKV_OK) return r;
  if (b->total_units == 0) return Fail(ctx, YAHKV_ERR_ORDER, "batch_plan: call batch_prepare first");
  YAHKV_CUDA(ctx, LaunchBatchPlan(b->lens_dev, b->rows_dev, static_cast<int>(b->seqs.size()), ctx->tables_dev,
                                  ctx->cfg.max_pages_per_seq, b->unit_pages, ctx->cfg.num_pages, b->units_dev,
                                  b->items_dev, b->slots_dev, b->vwork_dev, b->state_rows_dev, ctx->cfg.n_layers,
                                  StreamOf(ctx, stream)));
  ctx->launches += 1;
  return YAHKV_OK;
}

int yahkv_batch_decode_layer(yahkv_batch* b, int32_t layer, const void* k_dev, const void* v_dev, const void* q_dev,
                             const float* gate_dev, void* out_dev, int32_t out_dtype, void* stream) {
  if (b == nullptr) return YAHKV_ERR_INVALID;
  yahkv_ctx* ctx = b->ctx;
  if (int r = RequireDevice(ctx, "batch_decode_layer"); r != YAHKV_OK) return r;
  if (layer < 0 || layer >= ctx->cfg.n_layers) return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer: layer out of range");
  if (out_dtype != YAHKV_OUT_F16 && out_dtype != YAHKV_OUT_F32) return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer: bad out_dtype");
  if (k_dev == nullptr || v_dev == nullptr || q_dev == nullptr || out_dev == nullptr)
    return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer: null device pointer");
  if (b->total_units == 0) return Fail(ctx, YAHKV_ERR_ORDER, "batch_decode_layer: call batch_prepare first");
  cudaStream_t st = StreamOf(ctx, stream);
  const int n = static_cast<int>(b->seqs.size());
  const bool tile_fmt = IsTileFmt(ctx->cfg.fmt);
  if (tile_fmt) {
    YAHKV_CUDA(ctx, (ctx->cfg.fmt == YAHKV_FMT_KV4A16 ? LaunchKv4AppendK : LaunchKv8AppendK)(
                        ctx->pool, layer, n, b->slots_dev, b->state_rows_dev, layer, ctx->kmean_dev, k_dev, st));
    YAHKV_CUDA(ctx, LaunchKv8AppendV(ctx->pool, layer, n, b->vwork_dev, layer, ctx->open_tiles_dev, v_dev, st));
  } else {
    YAHKV_CUDA(ctx, LaunchAppend(ctx->pool, layer, n, b->slots_dev, k_dev, v_dev, st));
  }
  DecodeLaunch a{};
  a.kmap = &ctx->kmap, a.vmap = &ctx->vmap, a.pool = ctx->pool, a.layer = layer;
  a.tables_dev = ctx->tables_dev, a.table_stride = ctx->cfg.max_pages_per_seq;
  a.units_dev = b->units_dev, a.n_units = b->total_units;
  a.items_dev = b->items_dev, a.n_seqs = n;
  a.q_dev = q_dev, a.gate_dev = gate_dev, a.out_dev = out_dev, a.out_f32 = out_dtype == YAHKV_OUT_F32;
  a.scale_log2 = ctx->scale_log2;
  a.partial_acc = ctx->partial_acc, a.partial_ml = ctx->partial_ml, a.status_dev = ctx->status_dev;
  YAHKV_CUDA(ctx, ctx->cfg.fmt == YAHKV_FMT_KV4A16   ? LaunchKv4DecodePart(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                  : ctx->cfg.fmt == YAHKV_FMT_KV8A16 ? LaunchKv8DecodePart(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                  : ctx->cfg.fmt == YAHKV_FMT_F16    ? LaunchF16DecodePart(a, st)
                                                     : LaunchDecodePart(a, st));
  YAHKV_CUDA(ctx, LaunchDecodeCombine(a, st));
  ctx->launches += tile_fmt ? 4 : 3;
  return YAHKV_OK;
}

int yahkv_batch_decode_layer_raw(yahkv_batch* b, int32_t layer, const float* q_dev, const float* k_dev, const float* v_dev,
                                 const float* q_weight_dev, const float* k_weight_dev, float eps, const float* gate_dev,
                                 void* out_dev, int32_t out_dtype, void* stream) {
  if (b == nullptr) return YAHKV_ERR_INVALID;
  yahkv_ctx* ctx = b->ctx;
  if (int r = RequireDevice(ctx, "batch_decode_layer_raw"); r != YAHKV_OK) return r;
  if (layer < 0 || layer >= ctx->cfg.n_layers) return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer_raw: layer out of range");
  if (out_dtype != YAHKV_OUT_F16 && out_dtype != YAHKV_OUT_F32) return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer_raw: bad out_dtype");
  if (k_dev == nullptr || v_dev == nullptr || q_dev == nullptr || out_dev == nullptr || q_weight_dev == nullptr ||
      k_weight_dev == nullptr)
    return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer_raw: null device pointer");
  if (!(eps >= 0.0F)) return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer_raw: eps must be non-negative");
  if ((reinterpret_cast<std::uintptr_t>(q_dev) & 15) != 0 || (reinterpret_cast<std::uintptr_t>(q_weight_dev) & 15) != 0)
    return Fail(ctx, YAHKV_ERR_INVALID, "batch_decode_layer_raw: q and the norm weights must be 16-byte aligned");
  if (b->total_units == 0) return Fail(ctx, YAHKV_ERR_ORDER, "batch_decode_layer_raw: call batch_prepare first");
  cudaStream_t st = StreamOf(ctx, stream);
  if (ctx->rope_tab_dev == nullptr) {   // the cos / sin table is built once, with an allocation and a blocking copy
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    YAHKV_CUDA(ctx, cudaStreamIsCapturing(st, &cs));
    if (cs != cudaStreamCaptureStatusNone)
      return Fail(ctx, YAHKV_ERR_ORDER, "batch_decode_layer_raw: the RoPE table does not exist yet; run one step eagerly (or yahkv_rope_append) before capturing");
    if (int r = EnsureRopeTable(ctx); r != YAHKV_OK) return r;
  }
  const int n = static_cast<int>(b->seqs.size());
  const bool tile_fmt = IsTileFmt(ctx->cfg.fmt);
  // K and V: norm + RoPE + append at the planned slots, positions = the device-resident lengths; no q output (the part
  // kernel's prologue does the query side)
  YAHKV_CUDA(ctx, LaunchRopeAppend(ctx->pool, layer, n, b->slots_dev, b->lens_dev, q_dev, k_dev, v_dev, q_weight_dev,
                                   k_weight_dev, eps, ctx->rope_tab_dev, ctx->rope_rows, nullptr, ctx->rope_kv16_dev, st));
  if (tile_fmt) {   // the kernel left fp16 rows: the format's own appends take them
    const std::uint16_t* k16 = ctx->rope_kv16_dev;
    const std::uint16_t* v16 = k16 + static_cast<std::size_t>(n) * kKvHeads * kHeadDim;
    YAHKV_CUDA(ctx, (ctx->cfg.fmt == YAHKV_FMT_KV4A16 ? LaunchKv4AppendK : LaunchKv8AppendK)(
                        ctx->pool, layer, n, b->slots_dev, b->state_rows_dev, layer, ctx->kmean_dev, k16, st));
    YAHKV_CUDA(ctx, LaunchKv8AppendV(ctx->pool, layer, n, b->vwork_dev, layer, ctx->open_tiles_dev, v16, st));
  }
  DecodeLaunch a{};
  a.kmap = &ctx->kmap, a.vmap = &ctx->vmap, a.pool = ctx->pool, a.layer = layer;
  a.tables_dev = ctx->tables_dev, a.table_stride = ctx->cfg.max_pages_per_seq;
  a.units_dev = b->units_dev, a.n_units = b->total_units;
  a.items_dev = b->items_dev, a.n_seqs = n;
  a.q_dev = q_dev, a.gate_dev = gate_dev, a.out_dev = out_dev, a.out_f32 = out_dtype == YAHKV_OUT_F32;
  a.q_raw = true, a.q_weight_dev = q_weight_dev, a.q_eps = eps, a.rope_tab_dev = ctx->rope_tab_dev, a.rope_rows = ctx->rope_rows;
  a.scale_log2 = ctx->scale_log2;
  a.partial_acc = ctx->partial_acc, a.partial_ml = ctx->partial_ml, a.status_dev = ctx->status_dev;
  YAHKV_CUDA(ctx, ctx->cfg.fmt == YAHKV_FMT_KV4A16   ? LaunchKv4DecodePart(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                  : ctx->cfg.fmt == YAHKV_FMT_KV8A16 ? LaunchKv8DecodePart(a, ctx->open_tiles_dev, ctx->cfg.n_layers, st)
                  : ctx->cfg.fmt == YAHKV_FMT_F16    ? LaunchF16DecodePart(a, st)
                                                     : LaunchDecodePart(a, st));
  YAHKV_CUDA(ctx, LaunchDecodeCombine(a, st));
  ctx->launches += tile_fmt ? 5 : 3;
  return YAHKV_OK;
}

int yahkv_batch_advance(yahkv_batch* b, void* stream) {
  if (b == nullptr) return YAHKV_ERR_INVALID;
  yahkv_ctx* ctx = b->ctx;
  if (int r = RequireDevice(ctx, "batch_advance"); r != YAHKV_OK) return r;
  YAHKV_CUDA(ctx, LaunchBatchAdvance(b->lens_dev, static_cast<int>(b->seqs.size()), 1, StreamOf(ctx, stream)));
  ctx->launches += 1;
  return YAHKV_OK;
}

int yahkv_batch_commit(yahkv_batch* b, int32_t steps) {
  if (b == nullptr) return YAHKV_ERR_INVALID;
  yahkv_ctx* ctx = b->ctx;
  if (steps < 0 || steps > b->horizon) return Fail(ctx, YAHKV_ERR_ORDER, "batch_commit: more steps than the prepared horizon");
  for (std::size_t i = 0; i < b->seqs.size(); ++i) {
    HostError e = ctx->host.SeqSetLen(b->seqs[i], -1, static_cast<std::int64_t>(b->lens[i]) + steps);
    if (e.code != YAHKV_OK) return FailHost(ctx, std::move(e));
  }
  for (auto& n : b->lens) n += steps;
  b->horizon -= steps;
  ctx->host.InvalidateDecodePlan();
  return YAHKV_OK;
}

// ---- snapshots: sequences with their pages, in logical page order, so a load may place them anywhere ----------
namespace {
struct SnapshotHeader {
  char magic[8];            // "YAHKVSN1"
  std::int32_t fmt, n_layers, n_q_heads, n_kv_heads, head_dim, page_tokens, n_seqs, reserved;
};
struct FileCloser {
  void operator()(std::FILE* f) const {
    if (f != nullptr) std::fclose(f);
  }
};
}  // namespace

int yahkv_snapshot_save(yahkv_ctx* ctx, int32_t n_seqs, const int32_t* seq_ids, const char* path) {
  if (int r = RequireDevice(ctx, "snapshot_save"); r != YAHKV_OK) return r;
  if (n_seqs < 0 || (n_seqs > 0 && seq_ids == nullptr) || path == nullptr)
    return Fail(ctx, YAHKV_ERR_INVALID, "snapshot_save: bad sequence list or path");
  for (int i = 0; i < n_seqs; ++i)
    if (!ctx->host.live(seq_ids[i])) return Fail(ctx, YAHKV_ERR_INVALID, "snapshot_save: not a live sequence");
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  std::unique_ptr<std::FILE, FileCloser> f(std::fopen(path, "wb"));
  if (!f) return Fail(ctx, YAHKV_ERR_INVALID, std::string("snapshot_save: cannot open ") + path);
  const yahkv_config& c = ctx->cfg;
  SnapshotHeader h{};
  std::memcpy(h.magic, "YAHKVSN1", 8);
  h.fmt = c.fmt, h.n_layers = c.n_layers, h.n_q_heads = c.n_q_heads, h.n_kv_heads = c.n_kv_heads;
  h.head_dim = c.head_dim, h.page_tokens = c.page_tokens, h.n_seqs = n_seqs;
  bool ok = std::fwrite(&h, sizeof(h), 1, f.get()) == 1;
  // Per page record: K codes, K scales (or pairs), V codes, V scales (or statistic pairs), each for the four kv heads.
  const std::size_t cb = static_cast<std::size_t>(kKvHeads) * RecordCodeBytes(c.fmt);
  const std::size_t sbk = static_cast<std::size_t>(kKvHeads) * RecordScaleBytes(c.fmt, 0);
  const std::size_t sbv = static_cast<std::size_t>(kKvHeads) * RecordScaleBytes(c.fmt, 1);
  std::vector<std::uint8_t> buf(2 * cb + sbk + sbv);
  std::vector<std::uint8_t> state(static_cast<std::size_t>(kKvHeads) * kHeadDim * 4 + static_cast<std::size_t>(kOpenTileHalfs) * 2);
  for (int i = 0; i < n_seqs && ok; ++i) {
    const int s = seq_ids[i];
    const std::int32_t np = ctx->host.n_pages(s);
    ok = std::fwrite(&np, 4, 1, f.get()) == 1;
    for (int l = 0; l < c.n_layers && ok; ++l) {
      const std::int64_t len = ctx->host.len(s, l);
      ok = std::fwrite(&len, 8, 1, f.get()) == 1;
    }
    for (int l = 0; l < c.n_layers && ok; ++l)
      for (int p = 0; p < np && ok; ++p) {
        const std::size_t rec = (static_cast<std::size_t>(l) * c.num_pages + ctx->host.table_row(s)[p]) * kKvHeads;
        YAHKV_CUDA(ctx, cudaMemcpy(buf.data(), ctx->pool.kcodes + rec * RecordCodeBytes(c.fmt), cb, cudaMemcpyDeviceToHost));
        YAHKV_CUDA(ctx, cudaMemcpy(buf.data() + cb, ctx->pool.kscales + rec * (RecordScaleBytes(c.fmt, 0) / 2), sbk, cudaMemcpyDeviceToHost));
        YAHKV_CUDA(ctx, cudaMemcpy(buf.data() + cb + sbk, ctx->pool.vcodes + rec * RecordCodeBytes(c.fmt), cb, cudaMemcpyDeviceToHost));
        YAHKV_CUDA(ctx, cudaMemcpy(buf.data() + 2 * cb + sbk, ctx->pool.vscales + rec * (RecordScaleBytes(c.fmt, 1) / 2), sbv, cudaMemcpyDeviceToHost));
        FlipQ8(c.fmt, YAHKV_SIDE_K, buf.data(), cb);                 // the file holds GGUF int8 codes
        FlipQ8(c.fmt, YAHKV_SIDE_V, buf.data() + cb + sbk, cb);
        ok = std::fwrite(buf.data(), buf.size(), 1, f.get()) == 1;
      }
    // The tile formats keep state beyond the pages: per layer the K channel mean and the open fp16 tile.
    for (int l = 0; IsTileFmt(c.fmt) && l < c.n_layers && ok; ++l) {
      const std::size_t srow = static_cast<std::size_t>(s) * c.n_layers + l;
      YAHKV_CUDA(ctx, cudaMemcpy(state.data(), ctx->kmean_dev + srow * kKvHeads * kHeadDim,
                                 static_cast<std::size_t>(kKvHeads) * kHeadDim * 4, cudaMemcpyDeviceToHost));
      YAHKV_CUDA(ctx, cudaMemcpy(state.data() + static_cast<std::size_t>(kKvHeads) * kHeadDim * 4,
                                 static_cast<const std::uint16_t*>(ctx->open_tiles_dev) + (srow * 2 + ctx->host.open_cur(s, l)) * kOpenTileHalfs,
                                 static_cast<std::size_t>(kOpenTileHalfs) * 2, cudaMemcpyDeviceToHost));
      ok = std::fwrite(state.data(), state.size(), 1, f.get()) == 1;
    }
  }
  if (!ok) return Fail(ctx, YAHKV_ERR_INVALID, std::string("snapshot_save: write failed on ") + path);
  return YAHKV_OK;
}

int yahkv_snapshot_load(yahkv_ctx* ctx, const char* path, int32_t* seq_ids_out, int32_t* n_inout) {
  if (int r = RequireDevice(ctx, "snapshot_load"); r != YAHKV_OK) return r;
  if (path == nullptr || seq_ids_out == nullptr || n_inout == nullptr)
    return Fail(ctx, YAHKV_ERR_INVALID, "snapshot_load: null argument");
  std::unique_ptr<std::FILE, FileCloser> f(std::fopen(path, "rb"));
  if (!f) return Fail(ctx, YAHKV_ERR_INVALID, std::string("snapshot_load: cannot open ") + path);
  const yahkv_config& c = ctx->cfg;
  SnapshotHeader h{};
  if (std::fread(&h, sizeof(h), 1, f.get()) != 1 || std::memcmp(h.magic, "YAHKVSN1", 8) != 0)
    return Fail(ctx, YAHKV_ERR_INVALID, "snapshot_load: not a yahkv snapshot");
  // Only into an identical set, as the reference's LoadState (engine/model/loom_prefill.hpp:973-1024).
  if (h.fmt != c.fmt || h.n_layers != c.n_layers || h.n_q_heads != c.n_q_heads || h.n_kv_heads != c.n_kv_heads ||
      h.head_dim != c.head_dim || h.page_tokens != c.page_tokens)
    return Fail(ctx, YAHKV_ERR_INVALID, "snapshot_load: format, layer count or geometry differ from this context");
  if (h.n_seqs < 0 || h.n_seqs > *n_inout) return Fail(ctx, YAHKV_ERR_CAPACITY, "snapshot_load: more sequences than the caller's array holds");
  YAHKV_CUDA(ctx, cudaDeviceSynchronize());
  const std::size_t cb = static_cast<std::size_t>(kKvHeads) * RecordCodeBytes(c.fmt);
  const std::size_t sbk = static_cast<std::size_t>(kKvHeads) * RecordScaleBytes(c.fmt, 0);
  const std::size_t sbv = static_cast<std::size_t>(kKvHeads) * RecordScaleBytes(c.fmt, 1);
  std::vector<std::uint8_t> buf(2 * cb + sbk + sbv);
  std::vector<std::uint8_t> state(static_cast<std::size_t>(kKvHeads) * kHeadDim * 4 + static_cast<std::size_t>(kOpenTileHalfs) * 2);
  std::vector<std::int32_t> made;
  auto undo = [&](int code, const std::string& msg) {   // a failed load leaves no half-made sequences behind
    for (auto it = made.rbegin(); it != made.rend(); ++it) ctx->host.SeqFree(*it);   // restores the free lists' order
    return Fail(ctx, code, msg);
  };
  for (int i = 0; i < h.n_seqs; ++i) {
    std::int32_t np = 0;
    if (std::fread(&np, 4, 1, f.get()) != 1 || np < 0) return undo(YAHKV_ERR_INVALID, "snapshot_load: truncated file");
    std::vector<std::int64_t> lens(static_cast<std::size_t>(c.n_layers));
    if (std::fread(lens.data(), 8, lens.size(), f.get()) != lens.size()) return undo(YAHKV_ERR_INVALID, "snapshot_load: truncated file");
    std::int32_t s = -1;
    HostError e = ctx->host.SeqCreate(&s);
    if (e.code != YAHKV_OK) return undo(e.code, e.message);
    made.push_back(s);
    e = ctx->host.SeqReserve(s, static_cast<std::int64_t>(np) * kPageTokens);
    if (e.code != YAHKV_OK) return undo(e.code, e.message);
    for (int l = 0; l < c.n_layers; ++l) {
      e = ctx->host.SeqSetLen(s, l, lens[static_cast<std::size_t>(l)]);
      if (e.code != YAHKV_OK) return undo(e.code, "snapshot_load: " + e.message);
    }
    for (int l = 0; l < c.n_layers; ++l)
      for (int p = 0; p < np; ++p) {
        if (std::fread(buf.data(), buf.size(), 1, f.get()) != 1) return undo(YAHKV_ERR_INVALID, "snapshot_load: truncated file");
        FlipQ8(c.fmt, YAHKV_SIDE_K, buf.data(), cb);
        FlipQ8(c.fmt, YAHKV_SIDE_V, buf.data() + cb + sbk, cb);
        const std::size_t rec = (static_cast<std::size_t>(l) * c.num_pages + ctx->host.table_row(s)[p]) * kKvHeads;
        cudaError_t ce = cudaMemcpy(ctx->pool.kcodes + rec * RecordCodeBytes(c.fmt), buf.data(), cb, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(ctx->pool.kscales + rec * (RecordScaleBytes(c.fmt, 0) / 2), buf.data() + cb, sbk, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(ctx->pool.vcodes + rec * RecordCodeBytes(c.fmt), buf.data() + cb + sbk, cb, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(ctx->pool.vscales + rec * (RecordScaleBytes(c.fmt, 1) / 2), buf.data() + 2 * cb + sbk, sbv, cudaMemcpyHostToDevice);
        if (ce != cudaSuccess) return undo(YAHKV_ERR_CUDA, std::string("snapshot_load: ") + cudaGetErrorString(ce));
      }
    if (IsTileFmt(c.fmt)) {   // the mean and the open tile of every layer; the tile lands in the first buffer
      ctx->host.ResetOpenState(s);
      for (int l = 0; l < c.n_layers; ++l) {
        if (std::fread(state.data(), state.size(), 1, f.get()) != 1) return undo(YAHKV_ERR_INVALID, "snapshot_load: truncated file");
        const std::size_t srow = static_cast<std::size_t>(s) * c.n_layers + l;
        cudaError_t ce = cudaMemcpy(ctx->kmean_dev + srow * kKvHeads * kHeadDim, state.data(),
                                    static_cast<std::size_t>(kKvHeads) * kHeadDim * 4, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess)
          ce = cudaMemcpy(static_cast<std::uint16_t*>(ctx->open_tiles_dev) + srow * 2 * kOpenTileHalfs,
                          state.data() + static_cast<std::size_t>(kKvHeads) * kHeadDim * 4,
                          static_cast<std::size_t>(kOpenTileHalfs) * 2, cudaMemcpyHostToDevice);
        if (ce != cudaSuccess) return undo(YAHKV_ERR_CUDA, std::string("snapshot_load: ") + cudaGetErrorString(ce));
      }
    }
    seq_ids_out[i] = s;
  }
  *n_inout = h.n_seqs;
  return YAHKV_OK;
}

int yahkv_debug_wait_timeout(yahkv_ctx* ctx, int64_t limit_us, void* stream) {
  if (int r = RequireDevice(ctx, "debug_wait_timeout"); r != YAHKV_OK) return r;
  if (limit_us < 1 || limit_us > 1000000) return Fail(ctx, YAHKV_ERR_INVALID, "debug_wait_timeout: limit must be 1 us .. 1 s");
  YAHKV_CUDA(ctx, LaunchWaitProbe(ctx->status_dev, static_cast<std::uint64_t>(limit_us) * 1000ULL, StreamOf(ctx, stream)));
  ctx->launches += 1;
  return YAHKV_OK;
}

int yahkv_debug_set_prefill_sms(yahkv_ctx* ctx, int32_t n_sm) {
  if (int r = RequireDevice(ctx, "debug_set_prefill_sms"); r != YAHKV_OK) return r;
  if (n_sm < 0 || n_sm > ctx->n_sm_device) return Fail(ctx, YAHKV_ERR_INVALID, "debug_set_prefill_sms: 0 .. the device's SM count");
  ctx->n_sm = n_sm;
  return YAHKV_OK;
}

int yahkv_device_bytes(const yahkv_ctx* ctx, int64_t* bytes) {
  if (ctx == nullptr || bytes == nullptr) return YAHKV_ERR_INVALID;
  *bytes = ctx->device_bytes;
  return YAHKV_OK;
}

int yahkv_launch_count(const yahkv_ctx* ctx, int64_t* launches) {
  if (ctx == nullptr || launches == nullptr) return YAHKV_ERR_INVALID;
  *launches = ctx->launches;
  return YAHKV_OK;
}

}  // extern "C"
