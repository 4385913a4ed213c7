// Host side of the cache: the page allocator, the per-sequence block tables, per-layer lengths, validation, and the
// planners that turn a batch of sequences into the work lists the kernels read. No CUDA in this header.
//
// The reference keeps one sequence with an identity page table (engine/model/loom_decoder.hpp:175-179) and validates
// every table entry before upload (engine/model/loom_prefill.hpp:1314-1316); batching, the free list and the split-K
// planner are this library's own. Errors are reported as codes plus a message, never thrown across the C ABI, and
// every check runs before anything is queued (engine/model/loom_decoder.hpp:186-209).
#pragma once

#include <algorithm>
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "../../include/yahkv.h"
#include "kernels.cuh"

namespace yahkv {

struct HostError {
  int code = YAHKV_OK;
  std::string message;
};

class KvHost {
 public:
  explicit KvHost(const yahkv_config& cfg) : cfg_(cfg) {
    const std::size_t ns = static_cast<std::size_t>(cfg.max_seqs);
    table_.assign(ns * static_cast<std::size_t>(cfg.max_pages_per_seq), 0);
    n_pages_.assign(ns, 0);
    live_.assign(ns, 0);
    len_.assign(ns * static_cast<std::size_t>(cfg.n_layers), 0);
    dirty_lo_.assign(ns, 0);
    dirty_hi_.assign(ns, 0);
    owner_.assign(static_cast<std::size_t>(cfg.num_pages), -1);
    // LIFO free list: page 0 is handed out first.
    free_pages_.reserve(static_cast<std::size_t>(cfg.num_pages));
    for (int p = cfg.num_pages - 1; p >= 0; --p) free_pages_.push_back(p);
    free_seqs_.reserve(ns);
    for (int s = cfg.max_seqs - 1; s >= 0; --s) free_seqs_.push_back(s);
  }

  static int ValidateConfig(const yahkv_config& c, std::string* why) {
    auto bad = [&](const char* m) {
      *why = m;
      return YAHKV_ERR_INVALID;
    };
    if (c.n_q_heads != kQHeads || c.n_kv_heads != kKvHeads || c.head_dim != kHeadDim)
      return bad("geometry must be 24 query heads, 4 kv heads, head_dim 256");
    if (c.page_tokens != kPageTokens) return bad("page_tokens must be 64");
    if (c.fmt != YAHKV_FMT_Q8_0 && c.fmt != YAHKV_FMT_Q4_0 && c.fmt != YAHKV_FMT_KV8A16 && c.fmt != YAHKV_FMT_KV4A16 &&
        c.fmt != YAHKV_FMT_F16)
      return bad("fmt must be YAHKV_FMT_Q8_0, YAHKV_FMT_Q4_0, YAHKV_FMT_KV8A16, YAHKV_FMT_KV4A16 or YAHKV_FMT_F16");
    if ((c.fmt == YAHKV_FMT_KV8A16 || c.fmt == YAHKV_FMT_KV4A16) && c.kv_head_count != 0 && c.kv_head_count != kKvHeads)
      return bad("YAHKV_FMT_KV8A16 / YAHKV_FMT_KV4A16 contexts hold all four kv heads");
    if (c.n_layers < 1 || c.n_layers > 1024) return bad("n_layers out of range");
    if (c.num_pages < 1) return bad("num_pages must be positive");
    if (c.max_seqs < 1 || c.max_pages_per_seq < 1) return bad("max_seqs and max_pages_per_seq must be positive");
    if (c.max_splits < 0 || c.max_batch_tokens < 0) return bad("max_splits and max_batch_tokens must not be negative");
    static_assert(kCombineMaxUnits == 1024, "the message below names the limit");
    if (c.max_prefill_keys < 0 || 1LL * c.max_prefill_keys * kKvHeads >= (1LL << 31))
      return bad("max_prefill_keys out of range");
    if (c.max_splits > kCombineMaxUnits) return bad("max_splits must not exceed 1024 (the combine kernel's unit limit)");
    if (c.kv_head_begin < 0 || c.kv_head_count < 0 || c.kv_head_begin + c.kv_head_count > kKvHeads ||
        (c.kv_head_count == 0 && c.kv_head_begin != 0))
      return bad("kv_head_begin / kv_head_count must describe a range inside the 4 kv heads (count 0 = all)");
    // Token rows of all layers are addressed by a signed 32-bit tensor-map coordinate.
    const long long rows = 1LL * c.n_layers * c.num_pages * kKvHeads * kPageTokens;
    if (rows >= (1LL << 31)) return bad("n_layers * num_pages too large for the pool's row index");
    return YAHKV_OK;
  }

  const yahkv_config& cfg() const { return cfg_; }
  int kv_head_begin() const { return cfg_.kv_head_begin; }
  int kv_head_count() const { return cfg_.kv_head_count == 0 ? kKvHeads : cfg_.kv_head_count; }
  int pages_free() const { return static_cast<int>(free_pages_.size()); }
  bool live(int seq) const { return seq >= 0 && seq < cfg_.max_seqs && live_[static_cast<std::size_t>(seq)] != 0; }
  int n_pages(int seq) const { return n_pages_[static_cast<std::size_t>(seq)]; }
  const std::int32_t* table_row(int seq) const {
    return table_.data() + static_cast<std::size_t>(seq) * static_cast<std::size_t>(cfg_.max_pages_per_seq);
  }
  std::int64_t len(int seq, int layer) const {
    return len_[static_cast<std::size_t>(seq) * static_cast<std::size_t>(cfg_.n_layers) + static_cast<std::size_t>(layer)];
  }

  HostError SeqCreate(std::int32_t* seq) {
    if (free_seqs_.empty()) return {YAHKV_ERR_CAPACITY, "no free sequence slot (max_seqs reached)"};
    const int s = free_seqs_.back();
    free_seqs_.pop_back();
    live_[static_cast<std::size_t>(s)] = 1;
    n_pages_[static_cast<std::size_t>(s)] = 0;
    SetLenAll(s, 0);
    *seq = s;
    return {};
  }

  HostError SeqFree(int seq) {
    if (!live(seq)) return {YAHKV_ERR_INVALID, "seq_free: not a live sequence: " + std::to_string(seq)};
    ReleasePages(seq);
    live_[static_cast<std::size_t>(seq)] = 0;
    SetLenAll(seq, 0);
    free_seqs_.push_back(seq);
    return {};
  }

  HostError SeqReserve(int seq, std::int64_t n_tokens) {
    if (!live(seq)) return {YAHKV_ERR_INVALID, "seq_reserve: not a live sequence: " + std::to_string(seq)};
    if (n_tokens < 0) return {YAHKV_ERR_INVALID, "seq_reserve: negative token count"};
    const std::int64_t need = (n_tokens + kPageTokens - 1) / kPageTokens;
    const int have = n_pages_[static_cast<std::size_t>(seq)];
    if (need <= have) return {};
    if (need > cfg_.max_pages_per_seq)
      return {YAHKV_ERR_CAPACITY, "seq_reserve: " + std::to_string(n_tokens) + " tokens need more than max_pages_per_seq pages"};
    if (need - have > static_cast<std::int64_t>(free_pages_.size()))
      return {YAHKV_ERR_NO_PAGES, "seq_reserve: page pool exhausted (" + std::to_string(free_pages_.size()) +
                                      " free, " + std::to_string(need - have) + " needed)"};
    std::int32_t* row = mutable_row(seq);
    for (int i = have; i < need; ++i) {
      const std::int32_t p = free_pages_.back();
      free_pages_.pop_back();
      owner_[static_cast<std::size_t>(p)] = seq;
      row[i] = p;
    }
    n_pages_[static_cast<std::size_t>(seq)] = static_cast<int>(need);
    MarkDirty(seq, have, static_cast<int>(need));
    return {};
  }

  HostError SeqSetTable(int seq, const std::int32_t* pages, int n) {
    if (!live(seq)) return {YAHKV_ERR_INVALID, "seq_set_table: not a live sequence: " + std::to_string(seq)};
    if (n < 0 || (n > 0 && pages == nullptr)) return {YAHKV_ERR_INVALID, "seq_set_table: bad page list"};
    if (n > cfg_.max_pages_per_seq) return {YAHKV_ERR_CAPACITY, "seq_set_table: more pages than max_pages_per_seq"};
    // Validate everything before changing anything.
    std::vector<std::int32_t> sorted(pages, pages + n);
    std::sort(sorted.begin(), sorted.end());
    for (int i = 0; i < n; ++i) {
      const std::int32_t p = sorted[static_cast<std::size_t>(i)];
      if (p < 0 || p >= cfg_.num_pages)
        return {YAHKV_ERR_INVALID, "page table entry out of range: " + std::to_string(p)};
      if (i > 0 && sorted[static_cast<std::size_t>(i - 1)] == p)
        return {YAHKV_ERR_INVALID, "page table names page " + std::to_string(p) + " twice"};
      const int own = owner_[static_cast<std::size_t>(p)];
      if (own != -1 && own != seq)
        return {YAHKV_ERR_INVALID, "page " + std::to_string(p) + " belongs to sequence " + std::to_string(own)};
    }
    ReleasePages(seq);
    // Take the named pages out of the free list.
    std::vector<char> take(static_cast<std::size_t>(cfg_.num_pages), 0);
    for (int i = 0; i < n; ++i) take[static_cast<std::size_t>(pages[i])] = 1;
    free_pages_.erase(std::remove_if(free_pages_.begin(), free_pages_.end(),
                                     [&](std::int32_t p) { return take[static_cast<std::size_t>(p)] != 0; }),
                      free_pages_.end());
    std::int32_t* row = mutable_row(seq);
    for (int i = 0; i < n; ++i) {
      row[i] = pages[i];
      owner_[static_cast<std::size_t>(pages[i])] = seq;
    }
    n_pages_[static_cast<std::size_t>(seq)] = n;
    MarkDirty(seq, 0, n);
    return {};
  }

  HostError SeqSetLen(int seq, int layer, std::int64_t len) {
    if (!live(seq)) return {YAHKV_ERR_INVALID, "seq_set_len: not a live sequence: " + std::to_string(seq)};
    if (layer < -1 || layer >= cfg_.n_layers) return {YAHKV_ERR_INVALID, "seq_set_len: layer out of range"};
    if (len < 0 || len > static_cast<std::int64_t>(n_pages_[static_cast<std::size_t>(seq)]) * kPageTokens)
      return {YAHKV_ERR_INVALID, "seq_set_len: length beyond the reserved pages"};
    if (layer == -1)
      SetLenAll(seq, len);
    else
      len_ref(seq, layer) = len;
    return {};
  }

  // Checks one append call and computes its slots; on success also advances the lengths. Nothing changes on error.
  HostError PlanAppend(int layer, int n_tokens, const std::int32_t* seq_ids, const std::int64_t* positions,
                       std::int64_t* slots_out) {
    if (layer < 0 || layer >= cfg_.n_layers) return {YAHKV_ERR_INVALID, "append: layer out of range"};
    if (n_tokens < 0) return {YAHKV_ERR_INVALID, "append: negative token count"};
    if (n_tokens > 0 && (seq_ids == nullptr || positions == nullptr)) return {YAHKV_ERR_INVALID, "append: null id or position array"};
    scratch_len_.clear();
    for (int t = 0; t < n_tokens; ++t) {
      const int s = seq_ids[t];
      if (!live(s)) return {YAHKV_ERR_INVALID, "append: not a live sequence: " + std::to_string(s)};
      std::int64_t cur = -1;
      for (auto& e : scratch_len_)
        if (e.first == s) cur = e.second;
      if (cur < 0) cur = len(s, layer);
      const std::int64_t pos = positions[t];
      if (pos != cur)
        return {YAHKV_ERR_ORDER, "append: sequence " + std::to_string(s) + " layer " + std::to_string(layer) +
                                     " expects position " + std::to_string(cur) + ", got " + std::to_string(pos)};
      if (pos >= static_cast<std::int64_t>(n_pages_[static_cast<std::size_t>(s)]) * kPageTokens)
        return {YAHKV_ERR_INVALID, "append: position " + std::to_string(pos) + " of sequence " + std::to_string(s) +
                                       " is past its reserved pages"};
      slots_out[t] = static_cast<std::int64_t>(table_row(s)[pos / kPageTokens]) * kPageTokens + pos % kPageTokens;
      bool found = false;
      for (auto& e : scratch_len_)
        if (e.first == s) e.second = pos + 1, found = true;
      if (!found) scratch_len_.emplace_back(s, pos + 1);
    }
    for (auto& e : scratch_len_) len_ref(e.first, layer) = e.second;
    return {};
  }

  // Split-K plan of one decode call. units / items are rebuilt only when the (sequence, length) list or the split
  // request differs from the cached one; *changed says whether they must be uploaded again.
  HostError PlanDecode(int layer, int n_seqs, const std::int32_t* seq_ids, int n_splits, int max_splits,
                       int max_units, bool* changed) {
    if (layer < 0 || layer >= cfg_.n_layers) return {YAHKV_ERR_INVALID, "attend_decode: layer out of range"};
    if (n_seqs < 0 || (n_seqs > 0 && seq_ids == nullptr)) return {YAHKV_ERR_INVALID, "attend_decode: bad sequence list"};
    if (n_seqs > cfg_.max_seqs) return {YAHKV_ERR_CAPACITY, "attend_decode: more rows than max_seqs"};
    if (n_splits < 0) return {YAHKV_ERR_INVALID, "attend_decode: negative n_splits"};
    if (n_splits > max_splits) return {YAHKV_ERR_CAPACITY, "attend_decode: n_splits above max_splits"};
    key_scratch_.clear();
    key_scratch_.push_back(n_splits);
    long long total_pages = 0;
    for (int b = 0; b < n_seqs; ++b) {
      const int s = seq_ids[b];
      if (!live(s)) return {YAHKV_ERR_INVALID, "attend_decode: not a live sequence: " + std::to_string(s)};
      const std::int64_t n = len(s, layer);
      if (n <= 0)
        return {YAHKV_ERR_ORDER, "attend_decode: sequence " + std::to_string(s) + " has no keys in layer " +
                                     std::to_string(layer) + " (append first)"};
      key_scratch_.push_back(s);
      key_scratch_.push_back(n);
      total_pages += (n + kPageTokens - 1) / kPageTokens;
    }
    if (key_scratch_ == plan_key_) {
      *changed = false;
      return {};
    }
    // Automatic unit size: about five units per resident CTA slot (148 SMs x 2), at most 24 pages each. Measured on
    // the batch-32 benchmark: 10 pages 237 us, 16: 226, 24: 222, 32: 224, 48: 227 per layer; smaller units pay the
    // per-CTA prologue and partial write-back more often, larger ones leave a longer tail.
    const int hb = kv_head_begin(), hc = kv_head_count();
    int auto_pages = static_cast<int>((total_pages * hc + 1479) / 1480);
    auto_pages = std::min(std::max(auto_pages, 1), 24);
    std::vector<DecodeUnit> units;
    std::vector<CombineItem> items(static_cast<std::size_t>(n_seqs) * kKvHeads);
    for (int b = 0; b < n_seqs; ++b) {
      const int s = seq_ids[b];
      const std::int64_t n = len(s, layer);
      const int pages = static_cast<int>((n + kPageTokens - 1) / kPageTokens);
      int per = n_splits > 0 ? (pages + n_splits - 1) / n_splits : auto_pages;
      per = std::max(per, (pages + max_splits - 1) / max_splits);
      // The part kernel's two page sets take alternate pages of a unit: an odd count leaves one set idle for a page,
      // so a unit costs as much as the next even count. Rounding up never raises the number of units.
      if (per > 1) per += per & 1;
      int nu = (pages + per - 1) / per;
      // Graded sizes: with eight or more units the last quarter of them is half as long (and the others a little
      // longer, the count stays). CTAs take units longest first, so the short ones of all sequences run last and fill
      // the gaps of the final wave: equal units on a grid that is not a multiple of the resident CTAs leave a last
      // wave that is mostly idle (8 x 131072 tokens in 64 splits: 1952 equal units on 592 CTA slots).
      bounds_.clear();
      if (nu >= 8) {
        const int n_small = nu / 4, n_big = nu - n_small;
        int big = (2 * pages + 2 * n_big + n_small - 1) / (2 * n_big + n_small);
        big += big & 1;
        const int small = std::max(((big / 2) + 1) & ~1, 2);
        int p = 0;
        for (int k = 0; k < n_big && p < pages; ++k) bounds_.push_back(p = std::min(p + big, pages));
        while (p < pages) bounds_.push_back(p = std::min(p + small, pages));
      } else {
        for (int k = 0; k < nu; ++k) bounds_.push_back(std::min(pages, (k + 1) * per));
      }
      nu = static_cast<int>(bounds_.size());
      for (int h = hb; h < hb + hc; ++h) {   // heads outside the context's range keep n_partials = 0
        items[static_cast<std::size_t>(b) * kKvHeads + h] = {static_cast<std::int32_t>(units.size()), nu};
        for (int k = 0; k < nu; ++k) {
          DecodeUnit u{};
          u.batch = b, u.seq = s, u.kvh = h;
          u.page_begin = k == 0 ? 0 : bounds_[static_cast<std::size_t>(k) - 1], u.page_end = bounds_[static_cast<std::size_t>(k)];
          u.n_keys = static_cast<std::int32_t>(n);
          u.partial = static_cast<std::int32_t>(units.size());
          units.push_back(u);
        }
      }
    }
    if (static_cast<long long>(units.size()) > max_units)
      return {YAHKV_ERR_CAPACITY, "attend_decode: split-K plan needs " + std::to_string(units.size()) +
                                      " units, workspace holds " + std::to_string(max_units)};
    // Longest units first: CTAs are handed out in index order, so the short tail units fill the last wave.
    std::stable_sort(units.begin(), units.end(), [](const DecodeUnit& a, const DecodeUnit& b) {
      return a.page_end - a.page_begin > b.page_end - b.page_begin;
    });
    units_ = std::move(units);
    items_ = std::move(items);
    plan_key_ = key_scratch_;
    *changed = true;
    return {};
  }
  void InvalidateDecodePlan() { plan_key_.clear(); }

  // ---- kv8a16: which of a (sequence, layer)'s two open-tile buffers is current, and the V tile work of an append --
  int open_cur(int seq, int layer) const {
    return open_cur_.empty() ? 0 : open_cur_[static_cast<std::size_t>(seq) * static_cast<std::size_t>(cfg_.n_layers) + static_cast<std::size_t>(layer)];
  }
  // Called after a successful PlanAppend of the same call: the tokens of every sequence are consecutive positions
  // starting at its previous length, so the first position seen is that length. Builds one work item per 16-key tile
  // the call touches and flips the open buffer of sequences whose newest tile changed.
  void PlanKv8Tiles(int layer, int n_tokens, const std::int32_t* seq_ids, const std::int64_t* positions,
                    std::vector<VTileWork>* work) {
    if (open_cur_.empty()) open_cur_.assign(static_cast<std::size_t>(cfg_.max_seqs) * static_cast<std::size_t>(cfg_.n_layers), 0);
    work->clear();
    struct Span {
      int seq;
      std::int64_t p0, p1;
    };
    std::vector<Span> spans;
    for (int t = 0; t < n_tokens; ++t) {
      bool found = false;
      for (auto& sp : spans)
        if (sp.seq == seq_ids[t]) sp.p1 = positions[t] + 1, found = true;
      if (!found) spans.push_back({seq_ids[t], positions[t], positions[t] + 1});
    }
    for (const Span& sp : spans) {
      const std::size_t si = static_cast<std::size_t>(sp.seq) * static_cast<std::size_t>(cfg_.n_layers) + static_cast<std::size_t>(layer);
      const int cur = open_cur_[si];
      const std::int64_t t0 = sp.p0 / kTileKeys, t1 = (sp.p1 - 1) / kTileKeys;
      for (std::int64_t tile = t0; tile <= t1; ++tile) {
        VTileWork w{};
        w.state_row = static_cast<std::int32_t>(si);
        w.phys_tile = table_row(sp.seq)[tile * kTileKeys / kPageTokens] * kTilesPerPage + static_cast<std::int32_t>(tile % kTilesPerPage);
        w.n_old = tile == t0 ? static_cast<std::int32_t>(sp.p0 - tile * kTileKeys) : 0;
        w.n_keys = static_cast<std::int32_t>(std::min<std::int64_t>(kTileKeys, sp.p1 - tile * kTileKeys));
        w.read_buf = cur;
        w.write_buf = tile != t1 ? -1 : (t0 == t1 ? cur : cur ^ 1);
        w.complete = w.n_keys == kTileKeys ? 1 : 0;
        for (int j = 0; j < kTileKeys; ++j) w.src[j] = -1;
        work->push_back(w);
      }
      if (t0 != t1) open_cur_[si] = cur ^ 1;
    }
    // input token index of every new key
    for (int t = 0; t < n_tokens; ++t) {
      const std::int64_t tile = positions[t] / kTileKeys;
      std::size_t base = 0;
      for (const Span& sp : spans) {
        const std::int64_t t0 = sp.p0 / kTileKeys, t1 = (sp.p1 - 1) / kTileKeys;
        if (sp.seq == seq_ids[t]) {
          (*work)[base + static_cast<std::size_t>(tile - t0)].src[positions[t] % kTileKeys] = t;
          break;
        }
        base += static_cast<std::size_t>(t1 - t0 + 1);
      }
    }
  }
  void ResetOpenState(int seq) {
    if (open_cur_.empty()) return;
    for (int l = 0; l < cfg_.n_layers; ++l) open_cur_[static_cast<std::size_t>(seq) * static_cast<std::size_t>(cfg_.n_layers) + static_cast<std::size_t>(l)] = 0;
  }
  const std::vector<DecodeUnit>& units() const { return units_; }
  const std::vector<CombineItem>& items() const { return items_; }

  // Work lists of one prefill call: per sequence the span of the fp16 scratch it is dequantized into, and tiles of
  // 128 query rows x one query head, the ones with the most keys first so that the short ones fill the tail.
  // n_sm > 0: the tiles of the last, partly filled wave (one CTA per SM and wave, all tiles cost about the same) are
  // split along their keys into parts that fill the wave's idle SMs; `merges` lists them for the merge kernel, one
  // entry per head.
  HostError PlanPrefill(int layer, int n_seqs, const std::int32_t* seq_ids, const std::int32_t* chunk_lens,
                        int max_rows, int n_sm, std::vector<PrefillSeq>* seqs, std::vector<PrefillTile>* tiles,
                        std::vector<PrefillMerge>* merges, int* n_parts, std::int64_t* total_rows,
                        std::int64_t* scratch_rows, int* max_pages) {
    if (layer < 0 || layer >= cfg_.n_layers) return {YAHKV_ERR_INVALID, "attend_prefill: layer out of range"};
    if (n_seqs < 0 || (n_seqs > 0 && (seq_ids == nullptr || chunk_lens == nullptr)))
      return {YAHKV_ERR_INVALID, "attend_prefill: bad sequence list"};
    seqs->clear();
    tiles->clear();
    std::int64_t row = 0, kv_row = 0;
    *max_pages = 0;
    for (int i = 0; i < n_seqs; ++i) {
      const int s = seq_ids[i];
      if (!live(s)) return {YAHKV_ERR_INVALID, "attend_prefill: not a live sequence: " + std::to_string(s)};
      const std::int64_t n = len(s, layer);
      const int c = chunk_lens[i];
      if (c <= 0) return {YAHKV_ERR_INVALID, "attend_prefill: chunk length must be positive"};
      if (c > n)
        return {YAHKV_ERR_ORDER, "attend_prefill: chunk of " + std::to_string(c) + " rows but sequence " +
                                     std::to_string(s) + " holds " + std::to_string(n) + " keys (append first)"};
      PrefillSeq ps{};
      ps.seq = s;
      ps.n_pages = static_cast<std::int32_t>((n + kPageTokens - 1) / kPageTokens);
      ps.kv_len = static_cast<std::int32_t>(n);
      ps.kv_rows = ps.n_pages * kPageTokens;
      ps.kv_row0 = static_cast<std::int32_t>(kv_row);
      seqs->push_back(ps);
      *max_pages = std::max(*max_pages, static_cast<int>(ps.n_pages));
      for (int r = 0; r < c; r += kPrefillTileRows)
        for (int h = kv_head_begin() * kGroup; h < (kv_head_begin() + kv_head_count()) * kGroup; ++h) {
          PrefillTile t{};
          t.kv_row0 = static_cast<std::int32_t>(kv_row + static_cast<std::int64_t>(h / kGroup) * ps.kv_rows);
          t.head = h;
          t.q_row0 = static_cast<std::int32_t>(row + r);
          t.n_rows = std::min(kPrefillTileRows, c - r);
          t.pos0 = static_cast<std::int32_t>(n - c + r);
          t.jt_begin = 0, t.jt_end = (t.pos0 + t.n_rows + 63) / 64, t.part = -1;
          tiles->push_back(t);
        }
      row += c;
      kv_row += static_cast<std::int64_t>(kKvHeads) * ps.kv_rows;
      if (kv_row >= (1LL << 31)) return {YAHKV_ERR_CAPACITY, "attend_prefill: too many cached keys in one call"};
    }
    if (row > max_rows) return {YAHKV_ERR_CAPACITY, "attend_prefill: more query rows than max_batch_tokens"};
    std::stable_sort(tiles->begin(), tiles->end(),
                     [](const PrefillTile& a, const PrefillTile& b) { return a.pos0 + a.n_rows > b.pos0 + b.n_rows; });
    merges->clear();
    *n_parts = 0;
    // The kernel runs the two heads of a pair (entries 2 i and 2 i + 1: equal sort keys keep the neighbours of the loop
    // above together) as one CTA pair on two SMs, so the wave is counted in pairs.
    const int n_pairs = static_cast<int>(tiles->size()) / 2;
    const int wave = n_sm / 2;
    const int tail = wave > 0 ? n_pairs % wave : 0;   // a call of fewer pairs than the wave is all tail
    // Split factor: the tail's pairs cut into f key ranges take ceil(tail f / wave) waves of 1 / f tile time each.
    int f = 1;
    double best = 1.0;
    for (int c = 2; c <= kPrefillMaxParts && tail > 0; ++c) {
      const double cost = static_cast<double>((tail * c + wave - 1) / wave) / c;
      if (cost < best - 1e-9) best = cost, f = c;
    }
    if (f > 1) {
      const std::vector<PrefillTile> last(tiles->end() - 2 * tail, tiles->end());
      tiles->resize(static_cast<std::size_t>(2 * (n_pairs - tail)));
      for (std::size_t i = 0; i + 1 < last.size(); i += 2) {
        const PrefillTile& t = last[i];
        const int ff = std::min(f, t.jt_end / 2);   // a part covers at least two key tiles
        if (ff < 2) {
          tiles->push_back(last[i]);
          tiles->push_back(last[i + 1]);
          continue;
        }
        // part k of the two heads sits at entries first + 2 k, first + 2 k + 1 and takes the part slots of the same
        // parity: the merge kernel steps by two
        merges->push_back({static_cast<std::int32_t>(tiles->size()), ff});
        merges->push_back({static_cast<std::int32_t>(tiles->size()) + 1, ff});
        for (int k = 0; k < ff; ++k)
          for (int h = 0; h < 2; ++h) {
            PrefillTile p = last[i + static_cast<std::size_t>(h)];
            p.jt_begin = t.jt_end * k / ff, p.jt_end = t.jt_end * (k + 1) / ff, p.part = (*n_parts)++;
            tiles->push_back(p);
          }
      }
    }
    *total_rows = row;
    *scratch_rows = kv_row;
    return {};
  }

  // Puts a range back that ForEachDirty handed out but the caller could not upload.
  void MarkDirtyAgain(int seq, int lo, int hi) { MarkDirty(seq, lo, hi); }

  // Rows of the block table changed since the last call: [lo, hi) per sequence. The caller uploads and clears.
  template <class F>
  void ForEachDirty(F&& fn) {
    for (int s : dirty_list_) {
      const std::size_t i = static_cast<std::size_t>(s);
      if (dirty_hi_[i] > dirty_lo_[i]) fn(s, dirty_lo_[i], dirty_hi_[i]);
      dirty_lo_[i] = dirty_hi_[i] = 0;
    }
    dirty_list_.clear();
  }

 private:
  std::int32_t* mutable_row(int seq) {
    return table_.data() + static_cast<std::size_t>(seq) * static_cast<std::size_t>(cfg_.max_pages_per_seq);
  }
  std::int64_t& len_ref(int seq, int layer) {
    return len_[static_cast<std::size_t>(seq) * static_cast<std::size_t>(cfg_.n_layers) + static_cast<std::size_t>(layer)];
  }
  void SetLenAll(int seq, std::int64_t v) {
    for (int l = 0; l < cfg_.n_layers; ++l) len_ref(seq, l) = v;
  }
  void ReleasePages(int seq) {
    const std::int32_t* row = table_row(seq);
    // Pushed in table order, so the most recently added page is reused first.
    for (int i = 0; i < n_pages_[static_cast<std::size_t>(seq)]; ++i) {
      owner_[static_cast<std::size_t>(row[i])] = -1;
      free_pages_.push_back(row[i]);
    }
    n_pages_[static_cast<std::size_t>(seq)] = 0;
  }
  void MarkDirty(int seq, int lo, int hi) {
    const std::size_t i = static_cast<std::size_t>(seq);
    if (dirty_hi_[i] == dirty_lo_[i]) {
      dirty_lo_[i] = lo, dirty_hi_[i] = hi;
      dirty_list_.push_back(seq);
    } else {
      dirty_lo_[i] = std::min(dirty_lo_[i], lo), dirty_hi_[i] = std::max(dirty_hi_[i], hi);
    }
  }

  yahkv_config cfg_;
  std::vector<std::int32_t> table_;
  std::vector<int> n_pages_;
  std::vector<char> live_;
  std::vector<std::int64_t> len_;
  std::vector<int> dirty_lo_, dirty_hi_, dirty_list_;
  std::vector<int> owner_;
  std::vector<std::int32_t> free_pages_;
  std::vector<int> free_seqs_;
  std::vector<std::pair<int, std::int64_t>> scratch_len_;
  std::vector<std::int64_t> key_scratch_, plan_key_;
  std::vector<DecodeUnit> units_;
  std::vector<CombineItem> items_;
  std::vector<int> open_cur_;   // kv8a16: current open-tile buffer per (sequence, layer)
  std::vector<int> bounds_;     // PlanDecode: page boundaries of one sequence's units
};

}  // namespace yahkv
