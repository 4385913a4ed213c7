// CPU oracle for the paged quantized KV-cache path. TEST INFRASTRUCTURE ONLY: the shipped library never links,
// loads or calls anything in this file; only the parity tests, the smoke check and the CPU-baseline leg of the
// benchmark do, as the checker or as the timed CPU arm.
//
// What it restates (paths are relative to the reference project's root):
//   block quantize q8_0          engine/core/gguf_quant.cpp:310-320  (QuantizeQ8_0)
//   block decode q8_0 / q4_0     engine/core/gguf_quant.cpp:72-75 / :48-51
//   block quantize q4_0          NOT in the reference (its only quantizer is Q8_0). Restated from the published ggml
//                                algorithm (ggml-quants.c quantize_row_q4_0_ref, ggml pinned by the reference only
//                                as "pip install gguf", engine/tests/gguf_check.py:5). The reference pins the q4_0
//                                DECODE side only, so q4_0 quantize parity is "unpinned" by the reference; the CPU
//                                tests check this restatement against the installed gguf package instead.
//   page mapping + clamps        engine/gpu/loom/tools/gen_decode_attn.py:59-72 (256-token pages there, 64 here)
//   table validation             engine/model/loom_prefill.hpp:1314-1316
//   decode attention, float64    engine/gpu/loom/tools/dattn_q_check.py:193-201 (scores K.q/16, exp(s-max), normalise,
//                                @V, optional sigmoid gate), keys 0..pos visible (gen_decode_attn.py:7, :145)
//   decode attention, f32 2-level  gen_decode_attn.py:205-275 (per-page max/sum) and :373-408 (merge in page order)
//   prefill attention, float64   causal rule key <= start + i (engine/gpu/loom/tools/gen_attn_fa.py:2897-2904), same
//                                scale, normalisation and gate (gen_attn_fa.py:67-71)
// Pinning: the q8_0 quantizer and both decoders are checked bit-for-bit against the reference's own C++ compiled from
// its sources (oracle/_ref, built by oracle/Makefile) and against committed golden vectors made with it.
//
// Pool layout modelled here (the library's canonical layout): per layer and per side (K or V)
//   codes  [num_pages][n_kv_heads][page_tokens][code_bytes]   code_bytes = 256 (q8_0, int8) or 128 (q4_0, packed)
//   scales [num_pages][n_kv_heads][page_tokens][8]            fp16, one per 32-element block
// q4_0 packing inside a block's 16 bytes follows the reference decoder: byte j = element j (low nibble) and
// element j + 16 (high nibble), value = d * (nibble - 8).
#include <algorithm>
#include <atomic>
#include <bit>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int kHeadDim = 256;
constexpr int kBlocks = 8;      // 32-element blocks per head row
constexpr int kQHeads = 24;
constexpr int kKvHeads = 4;
constexpr int kGroup = kQHeads / kKvHeads;

inline float HalfBitsToFloat(std::uint16_t h) { return static_cast<float>(std::bit_cast<_Float16>(h)); }
inline std::uint16_t FloatToHalfBits(float f) { return std::bit_cast<std::uint16_t>(static_cast<_Float16>(f)); }

struct Geometry {
  int fmt;          // 0 = q8_0, 1 = q4_0, 4 = fp16 pages (rows as they are, no scales)
  int page_tokens;  // 64
  int num_pages;
  int code_bytes() const { return fmt == 4 ? 512 : (fmt == 0 ? 256 : 128); }
  std::size_t record_codes() const { return static_cast<std::size_t>(page_tokens) * code_bytes(); }
  std::size_t record_scales() const { return fmt == 4 ? 0 : static_cast<std::size_t>(page_tokens) * kBlocks; }
};

// One 32-value block -> int8 codes + fp16 scale, exactly as QuantizeQ8_0: d = amax / 127 (f32 divide),
// inv = 1 / d (f32), code = lround(x * inv) (ties away from zero), stored scale = half(d), round to nearest even.
void BlockQ8(const float* x, std::int8_t* codes, std::uint16_t* scale) {
  float amax = 0.0F;
  for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[i]));
  const float d = amax / 127.0F;
  const float inv = d > 0.0F ? 1.0F / d : 0.0F;
  *scale = FloatToHalfBits(d);
  for (int i = 0; i < 32; ++i) codes[i] = static_cast<std::int8_t>(std::lround(x[i] * inv));
}

// One 32-value block -> 16 packed bytes + fp16 scale (ggml's q4_0): the value of largest magnitude (first one on
// ties) maps to -8, d = max / -8, id = 1 / d, nibble = min(15, trunc(x * id + 8.5)).
void BlockQ4(const float* x, std::uint8_t* packed, std::uint16_t* scale) {
  float amax = 0.0F, mx = 0.0F;
  for (int i = 0; i < 32; ++i) {
    const float a = std::fabs(x[i]);
    if (a > amax) amax = a, mx = x[i];
  }
  const float d = mx / -8.0F;
  const float id = d != 0.0F ? 1.0F / d : 0.0F;
  *scale = FloatToHalfBits(d);
  for (int j = 0; j < 16; ++j) {
    const float x0 = x[j] * id, x1 = x[j + 16] * id;
    const int q0 = std::min(15, static_cast<int>(static_cast<std::int8_t>(x0 + 8.5F)));
    const int q1 = std::min(15, static_cast<int>(static_cast<std::int8_t>(x1 + 8.5F)));
    packed[j] = static_cast<std::uint8_t>(q0 | (q1 << 4));
  }
}

// Logical position -> physical token row of the pool, with the writers' clamps (position into the table's span,
// page id into the pool).
inline std::int64_t SlotOf(const Geometry& g, const std::int32_t* table, int table_len, std::int64_t pos) {
  const std::int64_t span = static_cast<std::int64_t>(table_len) * g.page_tokens;
  pos = std::min<std::int64_t>(std::max<std::int64_t>(pos, 0), span - 1);
  const std::int64_t lp = std::min<std::int64_t>(pos / g.page_tokens, table_len - 1);
  std::int64_t pg = table[lp];
  pg = std::min<std::int64_t>(std::max<std::int64_t>(pg, 0), g.num_pages - 1);
  return pg * g.page_tokens + pos % g.page_tokens;
}

// Dequantized head row (256 floats) of physical token row `slot`, kv head h.
void DecodeRow(const Geometry& g, const std::uint8_t* codes, const std::uint16_t* scales, std::int64_t slot, int h,
               float* y) {
  const std::int64_t page = slot / g.page_tokens, tok = slot % g.page_tokens;
  const std::size_t rec = static_cast<std::size_t>(page) * kKvHeads + h;
  const std::uint8_t* c = codes + rec * g.record_codes() + static_cast<std::size_t>(tok) * g.code_bytes();
  if (g.fmt == 4) {   // fp16 pages (the reference's fp16 pools, gen_decode_attn.py:4-6, :296-303: f16 widened to f32)
    std::uint16_t hbits[kHeadDim];
    std::memcpy(hbits, c, sizeof(hbits));
    for (int i = 0; i < kHeadDim; ++i) y[i] = HalfBitsToFloat(hbits[i]);
    return;
  }
  const std::uint16_t* s = scales + rec * g.record_scales() + static_cast<std::size_t>(tok) * kBlocks;
  for (int b = 0; b < kBlocks; ++b) {
    const float d = HalfBitsToFloat(s[b]);
    if (g.fmt == 0) {
      for (int j = 0; j < 32; ++j) y[b * 32 + j] = d * static_cast<std::int8_t>(c[b * 32 + j]);
    } else {
      for (int j = 0; j < 16; ++j) {
        y[b * 32 + j] = d * ((c[b * 16 + j] & 0xF) - 8);
        y[b * 32 + j + 16] = d * ((c[b * 16 + j] >> 4) - 8);
      }
    }
  }
}

template <class F>
void ParallelFor(int n, int threads, F&& fn) {
  threads = std::max(1, std::min(threads, n));
  if (threads == 1) {
    for (int i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<int> next{0};
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&] {
      for (int i = next.fetch_add(1); i < n; i = next.fetch_add(1)) fn(i);
    });
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

int yahkv_oracle_hardware_threads() { return static_cast<int>(std::max(1U, std::thread::hardware_concurrency())); }

// n floats (a multiple of 32) -> n/32 GGUF q8_0 blocks of 34 bytes [half d][32 x int8].
void yahkv_oracle_quantize_q8_0(const float* x, std::uint64_t n, std::uint8_t* dst) {
  for (std::uint64_t b = 0; b < n / 32; ++b, x += 32, dst += 34) {
    std::uint16_t hd;
    BlockQ8(x, reinterpret_cast<std::int8_t*>(dst + 2), &hd);
    std::memcpy(dst, &hd, 2);
  }
}

// n floats (a multiple of 32) -> n/32 GGUF q4_0 blocks of 18 bytes [half d][16 packed bytes].
void yahkv_oracle_quantize_q4_0(const float* x, std::uint64_t n, std::uint8_t* dst) {
  for (std::uint64_t b = 0; b < n / 32; ++b, x += 32, dst += 18) {
    std::uint16_t hd;
    BlockQ4(x, dst + 2, &hd);
    std::memcpy(dst, &hd, 2);
  }
}

void yahkv_oracle_dequantize_q8_0(const std::uint8_t* src, std::uint64_t n, float* y) {
  for (std::uint64_t b = 0; b < n / 32; ++b, src += 34, y += 32) {
    std::uint16_t hd;
    std::memcpy(&hd, src, 2);
    const float d = HalfBitsToFloat(hd);
    for (int j = 0; j < 32; ++j) y[j] = d * static_cast<std::int8_t>(src[2 + j]);
  }
}

void yahkv_oracle_dequantize_q4_0(const std::uint8_t* src, std::uint64_t n, float* y) {
  for (std::uint64_t b = 0; b < n / 32; ++b, src += 18, y += 32) {
    std::uint16_t hd;
    std::memcpy(&hd, src, 2);
    const float d = HalfBitsToFloat(hd);
    for (int j = 0; j < 16; ++j) y[j] = d * ((src[2 + j] & 0xF) - 8), y[j + 16] = d * ((src[2 + j] >> 4) - 8);
  }
}

// Every table entry must name a page of the pool. Returns the index of the first bad entry, or -1.
// Head-row RMSNorm + NeoX RoPE as the reference's "rope" kernel states it
// (engine/gpu/loom/yah_fused_qk_rope_f32.loom:4-6: inv_rms = rsqrt(sum x^2 / head_dim + eps), normed = (x * inv_rms) *
// weight, out[p] = normed[p] cos - normed[p + half] sin, out[p + half] = normed[p] sin + normed[p + half] cos,
// angle = pos / theta^(2 p / rotary_dim); :32 theta = 1e7; rotary_dim 64 of head_dim 256 at the engine's geometry),
// with the operation order pinned so that a GPU kernel can reproduce the bits: the sum of squares is 32 chains of
// eight fused multiply-adds (elements 8 l .. 8 l + 7) joined by a butterfly over distances 16, 8, 4, 2, 1; every
// other operation is one IEEE f32 operation; cos and sin are evaluated in double precision and rounded to f32.
// Rows are [256] f32; the result is rounded to fp16 (the append's input format). The reference has no CPU model of
// this kernel, so this restatement is pinned by the formula only.
void yahkv_oracle_rope_rows(const float* x, std::int64_t rows, const float* weight, float eps, const std::int32_t* pos,
                            std::uint16_t* out_half) {
  for (std::int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * 256;
    float part[32];
    for (int l = 0; l < 32; ++l) {
      float acc = 0.0F;
      for (int j = 0; j < 8; ++j) acc = std::fmaf(xr[8 * l + j], xr[8 * l + j], acc);
      part[l] = acc;
    }
    for (int m = 16; m >= 1; m >>= 1) {
      float next[32];
      for (int l = 0; l < 32; ++l) next[l] = part[l] + part[l ^ m];
      for (int l = 0; l < 32; ++l) part[l] = next[l];
    }
    const float mean = part[0] * (1.0F / 256.0F);
    const float inv = 1.0F / std::sqrt(mean + eps);
    float n[256];
    for (int i = 0; i < 256; ++i) {
      const float t = xr[i] * inv;
      n[i] = t * weight[i];
    }
    for (int p = 0; p < 32; ++p) {
      const double angle = static_cast<double>(pos[r]) * std::pow(1.0e7, -2.0 * p / 64.0);
      const float c = static_cast<float>(std::cos(angle)), sn = static_cast<float>(std::sin(angle));
      const float a = n[p], b = n[p + 32];
      const float ac = a * c, bs = b * sn, as = a * sn, bc = b * c;
      n[p] = ac - bs;
      n[p + 32] = as + bc;
    }
    for (int i = 0; i < 256; ++i) out_half[r * 256 + i] = FloatToHalfBits(n[i]);
  }
}

int yahkv_oracle_validate_table(const std::int32_t* table, int n, int num_pages) {
  for (int i = 0; i < n; ++i)
    if (table[i] < 0 || table[i] >= num_pages) return i;
  return -1;
}

std::int64_t yahkv_oracle_slot(int page_tokens, int num_pages, const std::int32_t* table, int table_len,
                               std::int64_t pos) {
  const Geometry g{0, page_tokens, num_pages};
  return SlotOf(g, table, table_len, pos);
}

// Appends n_tokens rows (fp16 bits, [n_tokens][4][256]) of one side (K or V) at the given physical token rows.
void yahkv_oracle_append_slots(int fmt, int page_tokens, int num_pages, std::uint8_t* codes, std::uint16_t* scales,
                               const std::int64_t* slots, int n_tokens, const std::uint16_t* x, int threads) {
  const Geometry g{fmt, page_tokens, num_pages};
  ParallelFor(n_tokens, threads, [&](int t) {
    const std::int64_t slot = slots[t];
    if (slot < 0) return;  // padding token
    const std::int64_t page = slot / g.page_tokens, tok = slot % g.page_tokens;
    float row[kHeadDim];
    for (int h = 0; h < kKvHeads; ++h) {
      const std::uint16_t* src = x + (static_cast<std::size_t>(t) * kKvHeads + h) * kHeadDim;
      for (int i = 0; i < kHeadDim; ++i) row[i] = HalfBitsToFloat(src[i]);  // exact widening
      const std::size_t rec = static_cast<std::size_t>(page) * kKvHeads + h;
      std::uint8_t* c = codes + rec * g.record_codes() + static_cast<std::size_t>(tok) * g.code_bytes();
      if (fmt == 4) {   // fp16 pages: the row as it came
        std::memcpy(c, src, kHeadDim * 2);
        continue;
      }
      std::uint16_t* s = scales + rec * g.record_scales() + static_cast<std::size_t>(tok) * kBlocks;
      for (int b = 0; b < kBlocks; ++b) {
        if (fmt == 0)
          BlockQ8(row + b * 32, reinterpret_cast<std::int8_t*>(c + b * 32), s + b);
        else
          BlockQ4(row + b * 32, c + b * 16, s + b);
      }
    }
  });
}

// One sequence's tokens at logical positions pos0 .. pos0 + n_tokens - 1 through its block table.
void yahkv_oracle_append_seq(int fmt, int page_tokens, int num_pages, std::uint8_t* codes, std::uint16_t* scales,
                             const std::int32_t* table, int table_len, std::int64_t pos0, int n_tokens,
                             const std::uint16_t* x, int threads) {
  const Geometry g{fmt, page_tokens, num_pages};
  std::vector<std::int64_t> slots(static_cast<std::size_t>(n_tokens));
  for (int t = 0; t < n_tokens; ++t) slots[static_cast<std::size_t>(t)] = SlotOf(g, table, table_len, pos0 + t);
  yahkv_oracle_append_slots(fmt, page_tokens, num_pages, codes, scales, slots.data(), n_tokens, x, threads);
}

// GGUF blocks of the token at physical row `slot`: 4 heads x 8 blocks of [half d][codes], 34 or 18 bytes each.
void yahkv_oracle_export_row(int fmt, int page_tokens, int num_pages, const std::uint8_t* codes,
                             const std::uint16_t* scales, std::int64_t slot, std::uint8_t* blocks) {
  const Geometry g{fmt, page_tokens, num_pages};
  const std::int64_t page = slot / g.page_tokens, tok = slot % g.page_tokens;
  const int cb = fmt == 0 ? 32 : 16;
  for (int h = 0; h < kKvHeads; ++h) {
    const std::size_t rec = static_cast<std::size_t>(page) * kKvHeads + h;
    const std::uint8_t* c = codes + rec * g.record_codes() + static_cast<std::size_t>(tok) * g.code_bytes();
    const std::uint16_t* s = scales + rec * g.record_scales() + static_cast<std::size_t>(tok) * kBlocks;
    for (int b = 0; b < kBlocks; ++b, blocks += 2 + cb) {
      std::memcpy(blocks, s + b, 2);
      std::memcpy(blocks + 2, c + b * cb, static_cast<std::size_t>(cb));
    }
  }
}

// Decode attention of one sequence, float64: n_keys = pos + 1 visible keys, q fp16 bits [24][256], gate f32 [24][256]
// or null, out double [24][256].
void yahkv_oracle_attend_decode_f64(int fmt, int page_tokens, int num_pages, const std::uint8_t* kcodes,
                                    const std::uint16_t* kscales, const std::uint8_t* vcodes,
                                    const std::uint16_t* vscales, const std::int32_t* table, int table_len,
                                    std::int64_t n_keys, const std::uint16_t* q, const float* gate, double scale,
                                    double* out, int threads) {
  const Geometry g{fmt, page_tokens, num_pages};
  ParallelFor(kKvHeads, threads, [&](int h) {
    std::vector<float> kd(static_cast<std::size_t>(n_keys) * kHeadDim), vd(kd.size());
    for (std::int64_t p = 0; p < n_keys; ++p) {
      const std::int64_t slot = SlotOf(g, table, table_len, p);
      DecodeRow(g, kcodes, kscales, slot, h, kd.data() + p * kHeadDim);
      DecodeRow(g, vcodes, vscales, slot, h, vd.data() + p * kHeadDim);
    }
    std::vector<double> s(static_cast<std::size_t>(n_keys));
    for (int j = 0; j < kGroup; ++j) {
      const int hh = h * kGroup + j;
      double qd[kHeadDim];
      for (int i = 0; i < kHeadDim; ++i) qd[i] = HalfBitsToFloat(q[hh * kHeadDim + i]);
      double mx = -INFINITY;
      for (std::int64_t p = 0; p < n_keys; ++p) {
        double a = 0;
        const float* kr = kd.data() + p * kHeadDim;
        for (int i = 0; i < kHeadDim; ++i) a += static_cast<double>(kr[i]) * qd[i];
        s[static_cast<std::size_t>(p)] = a * scale;
        mx = std::max(mx, a * scale);
      }
      double sum = 0;
      for (auto& v : s) v = std::exp(v - mx), sum += v;
      double acc[kHeadDim] = {};
      for (std::int64_t p = 0; p < n_keys; ++p) {
        const double w = s[static_cast<std::size_t>(p)] / sum;
        const float* vr = vd.data() + p * kHeadDim;
        for (int i = 0; i < kHeadDim; ++i) acc[i] += w * vr[i];
      }
      for (int i = 0; i < kHeadDim; ++i) {
        double o = acc[i];
        if (gate) o /= 1.0 + std::exp(-static_cast<double>(gate[hh * kHeadDim + i]));
        out[hh * kHeadDim + i] = o;
      }
    }
  });
}

// The same attention in f32 with the reference kernels' two-level softmax: per page max / sum / P.V, then a merge in
// page order. Batched over sequences; this is the timed CPU arm. tables is [n_seqs][table_stride].
void yahkv_oracle_attend_decode_f32(int fmt, int page_tokens, int num_pages, const std::uint8_t* kcodes,
                                    const std::uint16_t* kscales, const std::uint8_t* vcodes,
                                    const std::uint16_t* vscales, const std::int32_t* tables, int table_stride,
                                    const std::int32_t* n_keys, int n_seqs, const std::uint16_t* q, const float* gate,
                                    float scale, float* out, int threads) {
  const Geometry g{fmt, page_tokens, num_pages};
  ParallelFor(n_seqs * kKvHeads, threads, [&](int item) {
    const int sq = item / kKvHeads, h = item % kKvHeads;
    const std::int32_t* table = tables + static_cast<std::size_t>(sq) * table_stride;
    const std::int64_t n = n_keys[sq];
    const int pages = static_cast<int>((n + page_tokens - 1) / page_tokens);
    float qf[kGroup][kHeadDim];
    for (int j = 0; j < kGroup; ++j)
      for (int i = 0; i < kHeadDim; ++i)
        qf[j][i] = HalfBitsToFloat(q[(static_cast<std::size_t>(sq) * kQHeads + h * kGroup + j) * kHeadDim + i]);
    std::vector<float> acc(static_cast<std::size_t>(pages) * kGroup * kHeadDim, 0.0F);
    std::vector<float> ms(static_cast<std::size_t>(pages) * kGroup), ls(ms.size());
    std::vector<float> kr(static_cast<std::size_t>(page_tokens) * kHeadDim), vr(kr.size());
    std::vector<float> sc(static_cast<std::size_t>(page_tokens));
    for (int pg = 0; pg < pages; ++pg) {
      const std::int64_t base = static_cast<std::int64_t>(pg) * page_tokens;
      const int cnt = static_cast<int>(std::min<std::int64_t>(page_tokens, n - base));
      for (int t = 0; t < cnt; ++t) {
        const std::int64_t slot = SlotOf(g, table, table_stride, base + t);
        DecodeRow(g, kcodes, kscales, slot, h, kr.data() + t * kHeadDim);
        DecodeRow(g, vcodes, vscales, slot, h, vr.data() + t * kHeadDim);
      }
      for (int j = 0; j < kGroup; ++j) {
        float mx = -INFINITY;
        for (int t = 0; t < cnt; ++t) {
          float a = 0;
          for (int i = 0; i < kHeadDim; ++i) a += kr[t * kHeadDim + i] * qf[j][i];
          sc[static_cast<std::size_t>(t)] = a * scale;
          mx = std::max(mx, a * scale);
        }
        float l = 0;
        float* ap = acc.data() + (static_cast<std::size_t>(pg) * kGroup + j) * kHeadDim;
        for (int t = 0; t < cnt; ++t) {
          const float p = std::exp(sc[static_cast<std::size_t>(t)] - mx);
          l += p;
          for (int i = 0; i < kHeadDim; ++i) ap[i] += p * vr[t * kHeadDim + i];
        }
        ms[static_cast<std::size_t>(pg) * kGroup + j] = mx;
        ls[static_cast<std::size_t>(pg) * kGroup + j] = l;
      }
    }
    for (int j = 0; j < kGroup; ++j) {
      const int hh = h * kGroup + j;
      float M = -INFINITY;
      for (int pg = 0; pg < pages; ++pg) M = std::max(M, ms[static_cast<std::size_t>(pg) * kGroup + j]);
      float L = 0;
      float A[kHeadDim] = {};
      for (int pg = 0; pg < pages; ++pg) {
        const float w = std::exp(ms[static_cast<std::size_t>(pg) * kGroup + j] - M);
        L += w * ls[static_cast<std::size_t>(pg) * kGroup + j];
        const float* ap = acc.data() + (static_cast<std::size_t>(pg) * kGroup + j) * kHeadDim;
        for (int i = 0; i < kHeadDim; ++i) A[i] += w * ap[i];
      }
      const float inv = 1.0F / L;
      float* o = out + (static_cast<std::size_t>(sq) * kQHeads + hh) * kHeadDim;
      for (int i = 0; i < kHeadDim; ++i) {
        float v = A[i] * inv;
        if (gate) v *= 1.0F / (1.0F + std::exp(-gate[(static_cast<std::size_t>(sq) * kQHeads + hh) * kHeadDim + i]));
        o[i] = v;
      }
    }
  });
}

// Causal chunk attention of one sequence, float64. The cache already holds start + n_q tokens (the chunk was
// appended first). Query i of the chunk sits at position start + i and sees keys 0 .. start + i. Only the query rows
// q_begin .. q_end - 1 are computed; q [n_q][24][256] fp16 bits, out [q_end - q_begin][24][256] double.
void yahkv_oracle_attend_prefill_f64(int fmt, int page_tokens, int num_pages, const std::uint8_t* kcodes,
                                     const std::uint16_t* kscales, const std::uint8_t* vcodes,
                                     const std::uint16_t* vscales, const std::int32_t* table, int table_len,
                                     std::int64_t start, int n_q, int q_begin, int q_end, const std::uint16_t* q,
                                     const float* gate, double scale, double* out, int threads) {
  const Geometry g{fmt, page_tokens, num_pages};
  const std::int64_t total = start + n_q;
  std::vector<float> kd(static_cast<std::size_t>(total) * kKvHeads * kHeadDim), vd(kd.size());
  ParallelFor(static_cast<int>(total), threads, [&](int p) {
    const std::int64_t slot = SlotOf(g, table, table_len, p);
    for (int h = 0; h < kKvHeads; ++h) {
      DecodeRow(g, kcodes, kscales, slot, h, kd.data() + (static_cast<std::size_t>(p) * kKvHeads + h) * kHeadDim);
      DecodeRow(g, vcodes, vscales, slot, h, vd.data() + (static_cast<std::size_t>(p) * kKvHeads + h) * kHeadDim);
    }
  });
  ParallelFor((q_end - q_begin) * kQHeads, threads, [&](int item) {
    const int i = q_begin + item / kQHeads, hh = item % kQHeads, h = hh / kGroup;
    const std::int64_t n = start + i + 1;
    const std::uint16_t* qr = q + (static_cast<std::size_t>(i) * kQHeads + hh) * kHeadDim;
    double qd[kHeadDim];
    for (int d = 0; d < kHeadDim; ++d) qd[d] = HalfBitsToFloat(qr[d]);
    std::vector<double> s(static_cast<std::size_t>(n));
    double mx = -INFINITY;
    for (std::int64_t p = 0; p < n; ++p) {
      const float* kr = kd.data() + (static_cast<std::size_t>(p) * kKvHeads + h) * kHeadDim;
      double a = 0;
      for (int d = 0; d < kHeadDim; ++d) a += static_cast<double>(kr[d]) * qd[d];
      s[static_cast<std::size_t>(p)] = a * scale;
      mx = std::max(mx, a * scale);
    }
    double sum = 0;
    for (auto& v : s) v = std::exp(v - mx), sum += v;
    double acc[kHeadDim] = {};
    for (std::int64_t p = 0; p < n; ++p) {
      const double w = s[static_cast<std::size_t>(p)] / sum;
      const float* vr = vd.data() + (static_cast<std::size_t>(p) * kKvHeads + h) * kHeadDim;
      for (int d = 0; d < kHeadDim; ++d) acc[d] += w * vr[d];
    }
    double* o = out + (static_cast<std::size_t>(i - q_begin) * kQHeads + hh) * kHeadDim;
    for (int d = 0; d < kHeadDim; ++d) {
      double v = acc[d];
      if (gate) v /= 1.0 + std::exp(-static_cast<double>(gate[(static_cast<std::size_t>(i) * kQHeads + hh) * kHeadDim + d]));
      o[d] = v;
    }
  });
}

}  // extern "C"
