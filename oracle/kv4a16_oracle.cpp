// CPU oracle for the reference's own kv4a16 cache format. TEST INFRASTRUCTURE ONLY, like yahkv_oracle.cpp.
//
// What it restates (paths relative to the reference project's root):
//   K quantizer   engine/gpu/loom/tools/gen_kvq.py:288-463, model engine/gpu/loom/tools/dattn_q_check.py:74-84:
//                 x = f32(f16(k)) - mean per head through the orthonormal Walsh-Hadamard transform H256 (Sylvester
//                 order, x 1/16); per 32-dim group of rotated dims lo = min, hi = max, s = (hi - lo) / 15 (1 when 0),
//                 u = clamp(roundeven((x - lo) * (1 / s)), 0, 15); a dword holds 8 dims, dim 2j at bits 4j and dim
//                 2j + 1 at bits 16 + 4j; scale pair f16 (16 s, lo - 16 s).
//                 The transform here runs in f32 as the reference's kernel does (butterflies 1, 2, 4 dims apart inside
//                 an 8-dim chunk, then chunks 1, 2, 4, 8, 16 apart: gen_kvq.py:344-378), not in float64 as its numpy
//                 model does, so a code can differ from the model's by one level where a value sits on a rounding
//                 boundary; the reference's own checker accepts that (it fails a K row only when the dequantized
//                 values differ by 1e-2 or more, dattn_q_check.py:231-236), and tests/test_kv4a16_oracle_cpu.py holds
//                 this file to the same bar against golden vectors made with the model.
//   K decoder     dattn_q_check.py:95-98: rotated (k - mean) = u * (S / 16) + (C' + S). The attention rotates q by the
//                 same transform, so q.k is unchanged (gen_decode_attn.py:655-717).
//   V quantizer   gen_kvq.py:474-660, model dattn_q_check.py:101-122 with bits = 4: per (16-key tile, channel)
//                 cen = (max + min) / 2, s = (max - min) / 14 (1 when 0), both rounded to f16 first,
//                 u = clamp(roundeven((v - cf) * (1 / sf)) + 7, 0, 14); two dwords per channel, nibble p of dword w =
//                 key 8w + 2p (p < 4) or 8w + 2(p - 4) + 1; pair f16 (16 sf, cf - 23 sf). Pinned bit for bit.
//   V decoder     dattn_q_check.py:125-137: v = u * (S / 16) + S + C'.
//   open tile, attention: as for kv8a16 (kv8a16_oracle.cpp), with q rotated in float64 (dattn_q_check.py:203).
//
// Pool layout modelled (this library's, 64-token pages = 4 tiles):
//   kcodes [pages][4 heads][64 tokens][128]      bytes of the head's 32 dwords
//   kscales [pages][4][64][8 groups][2]          f16 pairs
//   vcodes [pages][4][4 tiles][256 channels][8]  bytes of the channel's 2 dwords
//   vstats [pages][4][4][256][2]                 f16 pairs
#include <algorithm>
#include <atomic>
#include <bit>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int kHeadDim = 256, kKvHeads = 4, kQHeads = 24, kGroup = 6, kTile = 16;
constexpr int kKBytes = 128, kKGroups = 8, kVBytes = 8;

inline float H2F(std::uint16_t h) { return static_cast<float>(std::bit_cast<_Float16>(h)); }
inline std::uint16_t F2H(float f) { return std::bit_cast<std::uint16_t>(static_cast<_Float16>(f)); }

// H256 x / 16 in f32, in the order of a 32-lane warp that holds 8 consecutive dims per lane.
void Hadamard256(float* x) {
  for (int h = 1; h < 8; h <<= 1)
    for (int base = 0; base < kHeadDim; base += 8)
      for (int i = 0; i < 8; ++i)
        if ((i & h) == 0) {
          const float a = x[base + i], b = x[base + i + h];
          x[base + i] = a + b, x[base + i + h] = a - b;
        }
  for (int o = 1; o < 32; o <<= 1)
    for (int lane = 0; lane < 32; ++lane)
      if ((lane & o) == 0)
        for (int i = 0; i < 8; ++i) {
          const float a = x[lane * 8 + i], b = x[(lane ^ o) * 8 + i];
          x[lane * 8 + i] = a + b, x[(lane ^ o) * 8 + i] = a - b;
        }
  for (int d = 0; d < kHeadDim; ++d) x[d] *= 0.0625F;
}
void Hadamard256(double* x) {
  for (int h = 1; h < kHeadDim; h <<= 1)
    for (int i = 0; i < kHeadDim; ++i)
      if ((i & h) == 0) {
        const double a = x[i], b = x[i + h];
        x[i] = a + b, x[i + h] = a - b;
      }
  for (int d = 0; d < kHeadDim; ++d) x[d] *= 0.0625;
}

inline int NibbleShift(int i) { return 4 * (i / 2) + ((i & 1) ? 16 : 0); }   // dim i of a dword's 8

// k [4][256] f16, mean [4][256] f32 -> codes [4][128] bytes, scales [4][8][2] f16
void QuantK(const std::uint16_t* k, const float* mean, std::uint8_t* codes, std::uint16_t* scales) {
  for (int h = 0; h < kKvHeads; ++h) {
    float x[kHeadDim];
    for (int d = 0; d < kHeadDim; ++d) x[d] = H2F(k[h * kHeadDim + d]) - mean[h * kHeadDim + d];
    Hadamard256(x);
    std::uint32_t dw[32] = {};
    for (int g = 0; g < kKGroups; ++g) {
      float lo = INFINITY, hi = -INFINITY;
      for (int d = 0; d < 32; ++d) lo = std::min(lo, x[32 * g + d]), hi = std::max(hi, x[32 * g + d]);
      const float s0 = (hi - lo) / 15.0F;
      const float s = s0 > 0.0F ? s0 : 1.0F;
      const float inv = 1.0F / s;
      for (int d = 0; d < 32; ++d) {
        float u = std::nearbyint((x[32 * g + d] - lo) * inv);
        u = std::min(std::max(u, 0.0F), 15.0F);
        const int dim = 32 * g + d;
        dw[dim / 8] |= static_cast<std::uint32_t>(u) << NibbleShift(dim % 8);
      }
      const float S0 = s * 16.0F;
      scales[(h * kKGroups + g) * 2 + 0] = F2H(S0);
      scales[(h * kKGroups + g) * 2 + 1] = F2H(lo - S0);
    }
    std::memcpy(codes + h * kKBytes, dw, kKBytes);
  }
}

// -> the rotated (k - mean) as attention sees it, [4][256] f32
void DeqK(const std::uint8_t* codes, const std::uint16_t* scales, float* out) {
  for (int h = 0; h < kKvHeads; ++h) {
    std::uint32_t dw[32];
    std::memcpy(dw, codes + h * kKBytes, kKBytes);
    for (int dim = 0; dim < kHeadDim; ++dim) {
      const float u = static_cast<float>((dw[dim / 8] >> NibbleShift(dim % 8)) & 15U);
      const float S = H2F(scales[(h * kKGroups + dim / 32) * 2]), Cp = H2F(scales[(h * kKGroups + dim / 32) * 2 + 1]);
      out[h * kHeadDim + dim] = u * (S / 16.0F) + (Cp + S);
    }
  }
}

inline int VKey(int w, int p) { return 8 * w + (p < 4 ? 2 * p : 2 * (p - 4) + 1); }

// v: [16 keys][4][256] f16 -> codes [4][256][8], stats [4][256][2]
void QuantVTile(const std::uint16_t* v, std::uint8_t* codes, std::uint16_t* stats) {
  for (int c = 0; c < kKvHeads * kHeadDim; ++c) {
    float x[kTile], mx = -INFINITY, mn = INFINITY;
    for (int key = 0; key < kTile; ++key) {
      x[key] = H2F(v[key * kKvHeads * kHeadDim + c]);
      mx = std::max(mx, x[key]), mn = std::min(mn, x[key]);
    }
    const float cen = (mx + mn) * 0.5F;
    const float s0 = (mx - mn) / 14.0F;
    const float s = s0 > 0.0F ? s0 : 1.0F;
    const float sf = H2F(F2H(s)), cf = H2F(F2H(cen));
    const float inv = 1.0F / sf;
    std::uint32_t dw[2] = {0, 0};
    for (int w = 0; w < 2; ++w)
      for (int p = 0; p < 8; ++p) {
        float u = std::nearbyint((x[VKey(w, p)] - cf) * inv) + 7.0F;
        u = std::min(std::max(u, 0.0F), 14.0F);
        dw[w] |= static_cast<std::uint32_t>(u) << (4 * p);
      }
    std::memcpy(codes + c * kVBytes, dw, kVBytes);
    stats[c * 2 + 0] = F2H(sf * 16.0F);
    const float t = sf * -23.0F;
    stats[c * 2 + 1] = F2H(cf + t);
  }
}

// codes [4][256][8], stats [4][256][2] -> out [16 keys][4][256]
void DeqVTile(const std::uint8_t* codes, const std::uint16_t* stats, float* out) {
  for (int c = 0; c < kKvHeads * kHeadDim; ++c) {
    const float S = H2F(stats[c * 2]), Cp = H2F(stats[c * 2 + 1]);
    std::uint32_t dw[2];
    std::memcpy(dw, codes + c * kVBytes, kVBytes);
    for (int w = 0; w < 2; ++w)
      for (int p = 0; p < 8; ++p) {
        const float u = static_cast<float>((dw[w] >> (4 * p)) & 15U);
        const float a = u * (S / 16.0F);
        const float b = a + S;
        out[VKey(w, p) * kKvHeads * kHeadDim + c] = b + Cp;
      }
  }
}

struct Pools {
  int page_tokens, num_pages;
  std::uint8_t* kcodes;
  std::uint16_t* kscales;
  std::uint8_t* vcodes;
  std::uint16_t* vstats;
};
inline std::int64_t PageOf(const Pools& g, const std::int32_t* table, int table_len, std::int64_t pos) {
  const std::int64_t lp = std::min<std::int64_t>(std::max<std::int64_t>(pos / g.page_tokens, 0), table_len - 1);
  return std::min<std::int64_t>(std::max<std::int64_t>(table[lp], 0), g.num_pages - 1);
}

template <class F>
void ParallelFor(int n, int threads, F&& fn) {
  threads = std::max(1, std::min(threads, n));
  std::atomic<int> next{0};
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&] {
      for (int i = next.fetch_add(1); i < n; i = next.fetch_add(1)) fn(i);
    });
  for (auto& th : pool) th.join();
}

// The rotated K rows and the V rows of keys 0 .. n - 1 as attention sees them, [n][4][256] each.
void DequantizeSequence(const Pools& g, const std::uint16_t* open_tile, const std::int32_t* table, int table_len,
                        std::int64_t n, int threads, std::vector<float>* kd, std::vector<float>* vd) {
  const int tiles_per_page = g.page_tokens / kTile;
  const std::int64_t n_tiles = (n + kTile - 1) / kTile, cur = (n - 1) / kTile;
  kd->assign(static_cast<std::size_t>(n_tiles) * kTile * kKvHeads * kHeadDim, 0.0F);
  vd->assign(kd->size(), 0.0F);
  ParallelFor(static_cast<int>(n_tiles), threads, [&](int t) {
    for (int key = 0; key < kTile; ++key) {
      const std::int64_t pos = static_cast<std::int64_t>(t) * kTile + key;
      if (pos >= n) break;
      const std::int64_t page = PageOf(g, table, table_len, pos);
      const int tok = static_cast<int>(pos % g.page_tokens);
      std::uint8_t codes[kKvHeads * kKBytes];
      std::uint16_t scales[kKvHeads * kKGroups * 2];
      for (int h = 0; h < kKvHeads; ++h) {
        const std::size_t rec = static_cast<std::size_t>(page) * kKvHeads + h;
        std::memcpy(codes + h * kKBytes, g.kcodes + (rec * g.page_tokens + tok) * kKBytes, kKBytes);
        std::memcpy(scales + h * kKGroups * 2, g.kscales + (rec * g.page_tokens + tok) * kKGroups * 2, kKGroups * 4);
      }
      DeqK(codes, scales, kd->data() + static_cast<std::size_t>(pos) * kKvHeads * kHeadDim);
    }
    float* vt = vd->data() + static_cast<std::size_t>(t) * kTile * kKvHeads * kHeadDim;
    if (t == cur) {
      for (int key = 0; key < kTile; ++key)
        for (int c = 0; c < kKvHeads * kHeadDim; ++c) vt[key * kKvHeads * kHeadDim + c] = H2F(open_tile[c * kTile + key]);
    } else {
      const std::int64_t pos = static_cast<std::int64_t>(t) * kTile;
      const std::int64_t page = PageOf(g, table, table_len, pos);
      const int t_in_page = static_cast<int>(pos % g.page_tokens) / kTile;
      std::vector<std::uint8_t> codes(static_cast<std::size_t>(kKvHeads) * kHeadDim * kVBytes);
      std::vector<std::uint16_t> stats(static_cast<std::size_t>(kKvHeads) * kHeadDim * 2);
      for (int h = 0; h < kKvHeads; ++h) {
        const std::size_t rec = (static_cast<std::size_t>(page) * kKvHeads + h) * tiles_per_page + t_in_page;
        std::memcpy(codes.data() + static_cast<std::size_t>(h) * kHeadDim * kVBytes, g.vcodes + rec * kHeadDim * kVBytes, kHeadDim * kVBytes);
        std::memcpy(stats.data() + static_cast<std::size_t>(h) * kHeadDim * 2, g.vstats + rec * kHeadDim * 2, kHeadDim * 4);
      }
      DeqVTile(codes.data(), stats.data(), vt);
    }
  });
}

}  // namespace

extern "C" {

void yahkv_oracle_kv4_quant_k(const std::uint16_t* k, const float* mean, std::uint8_t* codes, std::uint16_t* scales) {
  QuantK(k, mean, codes, scales);
}
void yahkv_oracle_kv4_deq_k(const std::uint8_t* codes, const std::uint16_t* scales, float* out) { DeqK(codes, scales, out); }
void yahkv_oracle_kv4_quant_vtile(const std::uint16_t* v, std::uint8_t* codes, std::uint16_t* stats) {
  QuantVTile(v, codes, stats);
}
void yahkv_oracle_kv4_deq_vtile(const std::uint8_t* codes, const std::uint16_t* stats, float* out) {
  DeqVTile(codes, stats, out);
}
// x [n_rows][256] f64, in place: H256 x / 16 (self-inverse).
void yahkv_oracle_hadamard256_f64(double* x, int n_rows) {
  for (int r = 0; r < n_rows; ++r) Hadamard256(x + static_cast<std::size_t>(r) * kHeadDim);
}

// Appends n tokens at positions pos0 .. pos0 + n - 1 of a sequence (same contract as the kv8a16 form).
void yahkv_oracle_kv4_append_seq(int page_tokens, int num_pages, std::uint8_t* kcodes, std::uint16_t* kscales,
                                 std::uint8_t* vcodes, std::uint16_t* vstats, std::uint16_t* open_tile,
                                 const float* mean, const std::int32_t* table, int table_len, std::int64_t pos0, int n,
                                 const std::uint16_t* k, const std::uint16_t* v) {
  const Pools g{page_tokens, num_pages, kcodes, kscales, vcodes, vstats};
  const int tiles_per_page = page_tokens / kTile;
  for (int i = 0; i < n; ++i) {
    const std::int64_t pos = pos0 + i;
    const std::int64_t page = PageOf(g, table, table_len, pos);
    const int tok = static_cast<int>(pos % page_tokens);
    std::uint8_t codes[kKvHeads * kKBytes];
    std::uint16_t scales[kKvHeads * kKGroups * 2];
    QuantK(k + static_cast<std::size_t>(i) * kKvHeads * kHeadDim, mean, codes, scales);
    for (int h = 0; h < kKvHeads; ++h) {
      const std::size_t rec = static_cast<std::size_t>(page) * kKvHeads + h;
      std::memcpy(kcodes + (rec * page_tokens + tok) * kKBytes, codes + h * kKBytes, kKBytes);
      std::memcpy(kscales + (rec * page_tokens + tok) * kKGroups * 2, scales + h * kKGroups * 2, kKGroups * 4);
    }
    const int col = static_cast<int>(pos % kTile);
    for (int c = 0; c < kKvHeads * kHeadDim; ++c)
      open_tile[c * kTile + col] = v[static_cast<std::size_t>(i) * kKvHeads * kHeadDim + c];
    if (col == kTile - 1) {   // the tile's 16th key: quantize it (the open tile keeps its fp16 values)
      std::vector<std::uint16_t> tile(static_cast<std::size_t>(kTile) * kKvHeads * kHeadDim);
      for (int key = 0; key < kTile; ++key)
        for (int c = 0; c < kKvHeads * kHeadDim; ++c) tile[static_cast<std::size_t>(key) * kKvHeads * kHeadDim + c] = open_tile[c * kTile + key];
      std::vector<std::uint8_t> vc(static_cast<std::size_t>(kKvHeads) * kHeadDim * kVBytes);
      std::vector<std::uint16_t> stats(static_cast<std::size_t>(kKvHeads) * kHeadDim * 2);
      QuantVTile(tile.data(), vc.data(), stats.data());
      const int t_in_page = tok / kTile;
      for (int h = 0; h < kKvHeads; ++h) {
        const std::size_t rec = (static_cast<std::size_t>(page) * kKvHeads + h) * tiles_per_page + t_in_page;
        std::memcpy(vcodes + rec * kHeadDim * kVBytes, vc.data() + static_cast<std::size_t>(h) * kHeadDim * kVBytes, kHeadDim * kVBytes);
        std::memcpy(vstats + rec * kHeadDim * 2, stats.data() + static_cast<std::size_t>(h) * kHeadDim * 2, kHeadDim * 4);
      }
    }
  }
}

// kd, vd [n][4][256] f32 out: what attention sees (K rotated), for the numpy prefill model.
void yahkv_oracle_kv4_dequantize(int page_tokens, int num_pages, const std::uint8_t* kcodes, const std::uint16_t* kscales,
                                 const std::uint8_t* vcodes, const std::uint16_t* vstats, const std::uint16_t* open_tile,
                                 const std::int32_t* table, int table_len, std::int64_t n_keys, float* kd_out,
                                 float* vd_out, int threads) {
  const Pools g{page_tokens, num_pages, const_cast<std::uint8_t*>(kcodes), const_cast<std::uint16_t*>(kscales),
                const_cast<std::uint8_t*>(vcodes), const_cast<std::uint16_t*>(vstats)};
  std::vector<float> kd, vd;
  DequantizeSequence(g, open_tile, table, table_len, n_keys, threads, &kd, &vd);
  const std::size_t n = static_cast<std::size_t>(n_keys) * kKvHeads * kHeadDim;
  std::memcpy(kd_out, kd.data(), n * sizeof(float));
  std::memcpy(vd_out, vd.data(), n * sizeof(float));
}

// q [24][256] f16, gate [24][256] f32 or null -> out [24][256] f64. Keys 0 .. n_keys - 1; the keys of tile
// (n_keys - 1) / 16 are read from the open tile in fp16, all earlier tiles dequantized; q rotated in float64.
void yahkv_oracle_kv4_attend_decode_f64(int page_tokens, int num_pages, const std::uint8_t* kcodes,
                                        const std::uint16_t* kscales, const std::uint8_t* vcodes,
                                        const std::uint16_t* vstats, const std::uint16_t* open_tile,
                                        const std::int32_t* table, int table_len, std::int64_t n_keys,
                                        const std::uint16_t* q, const float* gate, double scale, double* out,
                                        int threads) {
  const Pools g{page_tokens, num_pages, const_cast<std::uint8_t*>(kcodes), const_cast<std::uint16_t*>(kscales),
                const_cast<std::uint8_t*>(vcodes), const_cast<std::uint16_t*>(vstats)};
  const std::int64_t n = n_keys;
  std::vector<float> kd, vd;
  DequantizeSequence(g, open_tile, table, table_len, n, threads, &kd, &vd);
  ParallelFor(kQHeads, threads, [&](int hh) {
    const int h = hh / kGroup;
    double qd[kHeadDim];
    for (int d = 0; d < kHeadDim; ++d) qd[d] = H2F(q[hh * kHeadDim + d]);
    Hadamard256(qd);
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
    for (int d = 0; d < kHeadDim; ++d) {
      double v = acc[d];
      if (gate != nullptr) v /= 1.0 + std::exp(-static_cast<double>(gate[hh * kHeadDim + d]));
      out[hh * kHeadDim + d] = v;
    }
  });
}

}  // extern "C"
