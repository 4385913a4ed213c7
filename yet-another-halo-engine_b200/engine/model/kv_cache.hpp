// C++ face of the yahkv C ABI for the engine's own code: the calls LoomDecoder::Step and LoomPrefill::RunAttention
// make on this path become one-liners, and errors surface as exceptions thrown before anything is launched, the
// engine's convention (LoomError, engine/model/loom_runtime.hpp:44-60; checks before dispatch,
// engine/model/loom_decoder.hpp:186-209, :230-234).
//
//   reference                                               here
//   LoomDecoder::OwnState() / LoomPrefill pools             KvCache::OwnState(cfg)   (one object, shared by both)
//   LoomDecoder::Bind(LoomPrefill::DecoderState())          nothing to do: prefill and decode use the same KvCache
//   dattn_kappend_q + dattn_vappend_q | dattn_kvappend      Append(layer, seqs, positions, k, v, stream)
//   dattn_part(_q) + dattn_reduce                           AttendDecode(layer, seqs, q, gate, out, ...)
//   yah_kq8 | yah_vq8 ... + yah_attn_wmma                   Append(...) then AttendPrefill(...)
// Header-only; link with libyahkv.so. Not reentrant, like the engine (engine/model/generator.hpp:56).
#ifndef YAH_MODEL_KV_CACHE_HPP_
#define YAH_MODEL_KV_CACHE_HPP_

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "yahkv.h"

namespace yah::model {

class KvError : public std::runtime_error {
 public:
  KvError(int code, const std::string& what) : std::runtime_error(what), code_(code) {}
  [[nodiscard]] int code() const { return code_; }

 private:
  int code_;
};

class KvCache {
 public:
  // The engine's geometry (engine/model/loom_decoder.hpp:55-57) with 64-token pages.
  static yahkv_config Config(int device, int n_layers, int num_pages, int max_seqs, int max_pages_per_seq,
                             int fmt = YAHKV_FMT_Q8_0) {
    yahkv_config c{};
    c.device = device, c.n_layers = n_layers, c.n_q_heads = 24, c.n_kv_heads = 4, c.head_dim = 256;
    c.page_tokens = 64, c.num_pages = num_pages, c.fmt = fmt, c.max_seqs = max_seqs;
    c.max_pages_per_seq = max_pages_per_seq;
    return c;
  }

  // Allocates the pools, tables and workspaces (LoomDecoder::OwnState, engine/model/loom_decoder.hpp:159-183).
  static KvCache OwnState(const yahkv_config& cfg) {
    yahkv_ctx* ctx = nullptr;
    const int rc = yahkv_create(&cfg, &ctx);
    if (rc != YAHKV_OK) throw KvError(rc, std::string("kv cache: ") + yahkv_last_error(nullptr));
    return KvCache(ctx);
  }

  KvCache(KvCache&& o) noexcept : ctx_(std::exchange(o.ctx_, nullptr)) {}
  KvCache& operator=(KvCache&& o) noexcept {
    if (this != &o) {
      yahkv_destroy(ctx_);
      ctx_ = std::exchange(o.ctx_, nullptr);
    }
    return *this;
  }
  KvCache(const KvCache&) = delete;
  KvCache& operator=(const KvCache&) = delete;
  ~KvCache() { yahkv_destroy(ctx_); }

  [[nodiscard]] yahkv_ctx* handle() const { return ctx_; }

  // ---- sequences and pages ----
  [[nodiscard]] std::int32_t NewSequence() {
    std::int32_t s = -1;
    Check(yahkv_seq_create(ctx_, &s));
    return s;
  }
  void FreeSequence(std::int32_t seq) { Check(yahkv_seq_free(ctx_, seq)); }
  void Reserve(std::int32_t seq, std::int64_t n_tokens) { Check(yahkv_seq_reserve(ctx_, seq, n_tokens)); }
  void SetTable(std::int32_t seq, const std::vector<std::int32_t>& pages) {
    Check(yahkv_seq_set_table(ctx_, seq, pages.data(), static_cast<std::int32_t>(pages.size())));
  }
  [[nodiscard]] std::vector<std::int32_t> Table(std::int32_t seq) const {
    const std::int32_t* p = nullptr;
    std::int32_t n = 0;
    Check(yahkv_seq_table(ctx_, seq, &p, &n));
    return std::vector<std::int32_t>(p, p + n);
  }
  [[nodiscard]] std::int64_t Length(std::int32_t seq, std::int32_t layer) const {
    std::int64_t n = 0;
    Check(yahkv_seq_len(ctx_, seq, layer, &n));
    return n;
  }
  void SetLength(std::int32_t seq, std::int64_t len, std::int32_t layer = -1) {
    Check(yahkv_seq_set_len(ctx_, seq, layer, len));
  }
  [[nodiscard]] std::int32_t PagesFree() const {
    std::int32_t n = 0;
    Check(yahkv_pages_free(ctx_, &n));
    return n;
  }

  // ---- the hot path (device pointers, asynchronous on `stream`) ----
  void Append(std::int32_t layer, const std::vector<std::int32_t>& seqs, const std::vector<std::int64_t>& positions,
              const void* k_dev, const void* v_dev, void* stream = nullptr) {
    if (seqs.size() != positions.size()) throw KvError(YAHKV_ERR_INVALID, "kv cache: one position per token expected");
    Check(yahkv_append(ctx_, layer, static_cast<std::int32_t>(seqs.size()), seqs.data(), positions.data(), k_dev, v_dev,
                       stream));
  }
  // The reference's "rope" dispatch and the appends behind it (loom_decoder.hpp:250-261) as one call: f32 q / k / v as
  // the projections leave them, fp16 q for the attention out.
  void RopeAppend(std::int32_t layer, const std::vector<std::int32_t>& seqs, const std::vector<std::int64_t>& positions,
                  const float* q_dev, const float* k_dev, const float* v_dev, const float* q_weight_dev,
                  const float* k_weight_dev, float eps, void* q_out_dev, void* stream = nullptr) {
    if (seqs.size() != positions.size()) throw KvError(YAHKV_ERR_INVALID, "kv cache: one position per token expected");
    Check(yahkv_rope_append(ctx_, layer, static_cast<std::int32_t>(seqs.size()), seqs.data(), positions.data(), q_dev,
                            k_dev, v_dev, q_weight_dev, k_weight_dev, eps, q_out_dev, stream));
  }
  void AttendDecode(std::int32_t layer, const std::vector<std::int32_t>& seqs, const void* q_dev, const float* gate_dev,
                    void* out_dev, std::int32_t out_dtype = YAHKV_OUT_F16, std::int32_t n_splits = 0,
                    void* stream = nullptr) {
    Check(yahkv_attend_decode(ctx_, layer, static_cast<std::int32_t>(seqs.size()), seqs.data(), q_dev, gate_dev, out_dev,
                              out_dtype, n_splits, stream));
  }
  void AttendPrefill(std::int32_t layer, const std::vector<std::int32_t>& seqs, const std::vector<std::int32_t>& chunks,
                     const void* q_dev, const float* gate_dev, void* out_dev, std::int32_t out_dtype = YAHKV_OUT_F16,
                     void* stream = nullptr) {
    if (seqs.size() != chunks.size()) throw KvError(YAHKV_ERR_INVALID, "kv cache: one chunk length per sequence expected");
    Check(yahkv_attend_prefill(ctx_, layer, static_cast<std::int32_t>(seqs.size()), seqs.data(), chunks.data(), q_dev,
                               gate_dev, out_dev, out_dtype, stream));
  }
  // AttendDecode on the raw f32 q projection: the part kernel's prologue norms and rotates each head row at the
  // position of the sequence's newest key; RopeAppend may then get a null q_out_dev.
  void AttendDecodeRawQ(std::int32_t layer, const std::vector<std::int32_t>& seqs, const float* q_raw_dev,
                        const float* q_weight_dev, float eps, const float* gate_dev, void* out_dev,
                        std::int32_t out_dtype = YAHKV_OUT_F16, std::int32_t n_splits = 0, void* stream = nullptr) {
    Check(yahkv_attend_decode_qraw(ctx_, layer, static_cast<std::int32_t>(seqs.size()), seqs.data(), q_raw_dev,
                                   q_weight_dev, eps, gate_dev, out_dev, out_dtype, n_splits, stream));
  }
  // AttendPrefill on the raw f32 q projection: the attention kernel's prologue norms and rotates its rows (the
  // reference's QNORM option, engine/gpu/loom/tools/gen_attn_fa.py:56-61); RopeAppend may then get a null q_out_dev.
  void AttendPrefillRawQ(std::int32_t layer, const std::vector<std::int32_t>& seqs, const std::vector<std::int32_t>& chunks,
                         const float* q_raw_dev, const float* q_weight_dev, float eps, const float* gate_dev,
                         void* out_dev, std::int32_t out_dtype = YAHKV_OUT_F16, void* stream = nullptr) {
    if (seqs.size() != chunks.size()) throw KvError(YAHKV_ERR_INVALID, "kv cache: one chunk length per sequence expected");
    Check(yahkv_attend_prefill_qraw(ctx_, layer, static_cast<std::int32_t>(seqs.size()), seqs.data(), chunks.data(),
                                    q_raw_dev, q_weight_dev, eps, gate_dev, out_dev, out_dtype, stream));
  }
  // One layer of a decode step with page-locked HOST buffers, queued without waiting; WaitHostSteps() collects them.
  void DecodeStepHostAsync(std::int32_t layer, const std::vector<std::int32_t>& seqs, const void* k_host,
                           const void* v_host, const void* q_host, const float* gate_host, void* out_host,
                           std::int32_t out_dtype = YAHKV_OUT_F16) {
    Check(yahkv_decode_step_host_async(ctx_, layer, static_cast<std::int32_t>(seqs.size()), seqs.data(), k_host, v_host,
                                       q_host, gate_host, out_host, out_dtype));
  }
  void WaitHostSteps() { Check(yahkv_decode_step_host_wait(ctx_)); }
  void Synchronize() { Check(yahkv_sync(ctx_)); }

  // ---- snapshots (LoomPrefill::SaveState / LoadState, engine/model/loom_prefill.hpp:973-1024) ----
  void SaveState(const std::vector<std::int32_t>& seqs, const std::string& path) {
    Check(yahkv_snapshot_save(ctx_, static_cast<std::int32_t>(seqs.size()), seqs.data(), path.c_str()));
  }
  // The sequences of the file, on fresh pages and under fresh ids (at most `max_seqs` of them).
  [[nodiscard]] std::vector<std::int32_t> LoadState(const std::string& path, std::int32_t max_seqs) {
    std::vector<std::int32_t> ids(static_cast<std::size_t>(max_seqs > 0 ? max_seqs : 0));
    std::int32_t n = max_seqs;
    Check(yahkv_snapshot_load(ctx_, path.c_str(), ids.data(), &n));
    ids.resize(static_cast<std::size_t>(n));
    return ids;
  }

  // ---- decode steps with no host work in between (engine/model/loom_decoder.hpp:131-133: the position lives on the
  // device). Prepare is host work; Plan / DecodeLayer / DecodeLayerRaw / Advance are plain launches and may be
  // captured into a CUDA graph; Commit tells the cache how many steps were queued. ----
  class DecodeBatch {
   public:
    DecodeBatch(KvCache& cache, const std::vector<std::int32_t>& seqs) : cache_(&cache) {
      cache.Check(yahkv_batch_create(cache.ctx_, static_cast<std::int32_t>(seqs.size()), seqs.data(), &b_));
    }
    DecodeBatch(const DecodeBatch&) = delete;
    DecodeBatch& operator=(const DecodeBatch&) = delete;
    ~DecodeBatch() { yahkv_batch_destroy(b_); }
    // Reserves pages for `horizon_steps` more positions; true when the unit layout changed (capture again).
    bool Prepare(std::int32_t horizon_steps, void* stream = nullptr) {
      std::int32_t changed = 0;
      cache_->Check(yahkv_batch_prepare(b_, horizon_steps, &changed, stream));
      return changed != 0;
    }
    void Plan(void* stream = nullptr) { cache_->Check(yahkv_batch_plan(b_, stream)); }
    void DecodeLayer(std::int32_t layer, const void* k_dev, const void* v_dev, const void* q_dev, const float* gate_dev,
                     void* out_dev, std::int32_t out_dtype = YAHKV_OUT_F16, void* stream = nullptr) {
      cache_->Check(yahkv_batch_decode_layer(b_, layer, k_dev, v_dev, q_dev, gate_dev, out_dev, out_dtype, stream));
    }
    // The layer on the raw f32 projections: the reference's rope, append, part, reduce sequence
    // (engine/model/loom_decoder.hpp:250-268).
    void DecodeLayerRaw(std::int32_t layer, const float* q_dev, const float* k_dev, const float* v_dev,
                        const float* q_weight_dev, const float* k_weight_dev, float eps, const float* gate_dev,
                        void* out_dev, std::int32_t out_dtype = YAHKV_OUT_F16, void* stream = nullptr) {
      cache_->Check(yahkv_batch_decode_layer_raw(b_, layer, q_dev, k_dev, v_dev, q_weight_dev, k_weight_dev, eps, gate_dev,
                                                 out_dev, out_dtype, stream));
    }
    void Advance(void* stream = nullptr) { cache_->Check(yahkv_batch_advance(b_, stream)); }
    void Commit(std::int32_t steps) { cache_->Check(yahkv_batch_commit(b_, steps)); }

   private:
    KvCache* cache_;
    yahkv_batch* b_ = nullptr;
  };

 private:
  explicit KvCache(yahkv_ctx* ctx) : ctx_(ctx) {}
  void Check(int rc) const {
    if (rc != YAHKV_OK) throw KvError(rc, std::string("kv cache: ") + yahkv_last_error(ctx_));
  }
  yahkv_ctx* ctx_ = nullptr;
};

}  // namespace yah::model

#endif  // YAH_MODEL_KV_CACHE_HPP_
