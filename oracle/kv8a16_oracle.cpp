// CPU oracle for the reference's own kv8a16 cache format. TEST INFRASTRUCTURE ONLY, like yahkv_oracle.cpp.
//
// What it restates (paths relative to the reference project's root); every function is pinned bit for bit against
// golden vectors made with the reference's numpy models (tests/golden/make_golden_kv8a16.py):
//   K quantizer   engine/gpu/loom/tools/gen_kvq.py:166-285, model engine/gpu/loom/tools/dattn_q_check.py:61-73:
//                 x = f32(f16(k)) - mean; per (head, 128-dim half) s = amax / 127 (1 when 0),
//                 u = roundeven(x * (1 / s)) + 128; a dword holds dims 4i .. 4i+3 in byte slots (d0, d2, d1, d3);
//                 scale pair f16 (256 s, -384 s).
//   K decoder     dattn_q_check.py:87-98: k - mean = (u - 128) * (S / 256), S the pair's first value. The mean is never
//                 added back: it shifts every score of a head by the same amount (docs/architecture.md:206).
//   V quantizer   gen_kvq.py:474-660, model dattn_q_check.py:101-122: per (16-key tile, channel) cen = (max + min) / 2,
//                 s = (max - min) / 254 (1 when 0), both rounded to f16 first, u = clamp(roundeven((v - cf) * (1 / sf))
//                 + 128, 0, 255); dword w byte p = key 4w + (0, 2, 1, 3)[p]; pair f16 (256 sf, cf - 384 sf).
//   V decoder     dattn_q_check.py:125-137: v = u * (S / 256) + S + C'.
//   open tile     the tile that holds the newest key stays in fp16 and attention reads it from there
//                 (engine/gpu/loom/tools/gen_decode_attn.py:426-427, :995-1028; checker dattn_q_check.py:166-170).
//   attention     the checker's float64 model (dattn_q_check.py:193-201) over the dequantized K - mean and V.
//
// Pool layout modelled (this library's, 64-token pages = 4 tiles; the reference uses 256-token pages):
//   kcodes [pages][4 heads][64 tokens][256]     bytes of the head's 64 dwords
//   kscales [pages][4][64][2 halves][2]         f16 pairs
//   vcodes [pages][4][4 tiles][256 channels][16] bytes of the channel's 4 dwords
//   vstats [pages][4][4][256][2]                f16 pairs
//   open tile per sequence [4][256][16] f16: keys 16 t .. 16 t + 15 of the tile t = (len - 1) / 16
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
constexpr int kPerm4[4] = {0, 2, 1, 3};

inline float H2F(std::uint16_t h) { return static_cast<float>(std::bit_cast<_Float16>(h)); }
inline std::uint16_t F2H(float f) { return std::bit_cast<std::uint16_t>(static_cast<_Float16>(f)); }

void QuantK(const std::uint16_t* k, const float* mean, std::uint8_t* codes, std::uint16_t* scales) {
  for (int h = 0; h < kKvHeads; ++h)
    for (int half = 0; half < 2; ++half) {
      float x[128], amax = 0.0F;
      for (int d = 0; d < 128; ++d) {
        x[d] = H2F(k[h * kHeadDim + half * 128 + d]) - mean[h * kHeadDim + half * 128 + d];
        amax = std::max(amax, std::fabs(x[d]));
      }
      const float s0 = amax / 127.0F;
      const float s = s0 > 0.0F ? s0 : 1.0F;
      const float inv = 1.0F / s;
      for (int d = 0; d < 128; ++d) {
        const int dim = half * 128 + d;
        const auto u = static_cast<std::uint32_t>(std::nearbyint(x[d] * inv) + 128.0F);
        // dword dim / 4 holds dim 4i + perm[b] in byte slot b
        int slot = 0;
        for (int b = 0; b < 4; ++b)
          if (kPerm4[b] == dim % 4) slot = b;
        codes[h * kHeadDim + (dim / 4) * 4 + slot] = static_cast<std::uint8_t>(u);
      }
      scales[(h * 2 + half) * 2 + 0] = F2H(s * 256.0F);
      scales[(h * 2 + half) * 2 + 1] = F2H(s * -384.0F);
    }
}

void DeqK(const std::uint8_t* codes, const std::uint16_t* scales, float* out) {
  for (int h = 0; h < kKvHeads; ++h)
    for (int dim = 0; dim < kHeadDim; ++dim) {
      int slot = 0;
      for (int b = 0; b < 4; ++b)
        if (kPerm4[b] == dim % 4) slot = b;
      const float u = codes[h * kHeadDim + (dim / 4) * 4 + slot];
      const float S = H2F(scales[(h * 2 + dim / 128) * 2]);
      out[h * kHeadDim + dim] = (u - 128.0F) * (S / 256.0F);
    }
}

// v: [16 keys][4][256] f16 -> codes [4][256][16], stats [4][256][2]
void QuantVTile(const std::uint16_t* v, std::uint8_t* codes, std::uint16_t* stats) {
  for (int c = 0; c < kKvHeads * kHeadDim; ++c) {
    float x[kTile], mx = -INFINITY, mn = INFINITY;
    for (int key = 0; key < kTile; ++key) {
      x[key] = H2F(v[key * kKvHeads * kHeadDim + c]);
      mx = std::max(mx, x[key]), mn = std::min(mn, x[key]);
    }
    const float cen = (mx + mn) * 0.5F;
    const float s0 = (mx - mn) / 254.0F;
    const float s = s0 > 0.0F ? s0 : 1.0F;
    const float sf = H2F(F2H(s)), cf = H2F(F2H(cen));
    const float inv = 1.0F / sf;
    for (int w = 0; w < 4; ++w)
      for (int p = 0; p < 4; ++p) {
        const int key = 4 * w + kPerm4[p];
        float u = std::nearbyint((x[key] - cf) * inv) + 128.0F;
        u = std::min(std::max(u, 0.0F), 255.0F);
        codes[c * 16 + 4 * w + p] = static_cast<std::uint8_t>(static_cast<std::uint32_t>(u));
      }
    stats[c * 2 + 0] = F2H(sf * 256.0F);
    const float t = sf * -384.0F;
    stats[c * 2 + 1] = F2H(cf + t);
  }
}

// codes [4][256][16], stats [4][256][2] -> out [16 keys][4][256]
void DeqVTile(const std::uint8_t* codes, const std::uint16_t* stats, float* out) {
  for (int c = 0; c < kKvHeads * kHeadDim; ++c) {
    const float S = H2F(stats[c * 2]), Cp = H2F(stats[c * 2 + 1]);
    for (int w = 0; w < 4; ++w)
      for (int p = 0; p < 4; ++p) {
        const int key = 4 * w + kPerm4[p];
        const float u = codes[c * 16 + 4 * w + p];
        const float a = u * (S / 256.0F);
        const float b = a + S;
        out[key * kKvHeads * kHeadDim + c] = b + Cp;
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

}  // namespace

extern "C" {

void yahkv_oracle_kv8_quant_k(const std::uint16_t* k, const float* mean, std::uint8_t* codes, std::uint16_t* scales) {
  QuantK(k, mean, codes, scales);
}
void yahkv_oracle_kv8_deq_k(const std::uint8_t* codes, const std::uint16_t* scales, float* out) { DeqK(codes, scales, out); }
void yahkv_oracle_kv8_quant_vtile(const std::uint16_t* v, std::uint8_t* codes, std::uint16_t* stats) {
  QuantVTile(v, codes, stats);
}
void yahkv_oracle_kv8_deq_vtile(const std::uint8_t* codes, const std::uint16_t* stats, float* out) {
  DeqVTile(codes, stats, out);
}

// Appends n tokens at positions pos0 .. pos0 + n - 1 of a sequence: K rows quantized and placed; V keys written into
// the open tile (which always holds the fp16 keys of the tile of the newest position), every tile that the call
// completes quantized and placed. k, v: [n][4][256] f16; open_tile [4][256][16] f16; mean [4][256] f32.
void yahkv_oracle_kv8_append_seq(int page_tokens, int num_pages, std::uint8_t* kcodes, std::uint16_t* kscales,
                                 std::uint8_t* vcodes, std::uint16_t* vstats, std::uint16_t* open_tile,
                                 const float* mean, const std::int32_t* table, int table_len, std::int64_t pos0, int n,
                                 const std::uint16_t* k, const std::uint16_t* v) {
  const Pools g{page_tokens, num_pages, kcodes, kscales, vcodes, vstats};
  const int tiles_per_page = page_tokens / kTile;
  for (int i = 0; i < n; ++i) {
    const std::int64_t pos = pos0 + i;
    const std::int64_t page = PageOf(g, table, table_len, pos);
    const int tok = static_cast<int>(pos % page_tokens);
    std::uint8_t codes[kKvHeads * kHeadDim];
    std::uint16_t scales[kKvHeads * 4];
    QuantK(k + static_cast<std::size_t>(i) * kKvHeads * kHeadDim, mean, codes, scales);
    for (int h = 0; h < kKvHeads; ++h) {
      const std::size_t rec = static_cast<std::size_t>(page) * kKvHeads + h;
      std::memcpy(kcodes + (rec * page_tokens + tok) * kHeadDim, codes + h * kHeadDim, kHeadDim);
      std::memcpy(kscales + (rec * page_tokens + tok) * 4, scales + h * 4, 8);
    }
    const int col = static_cast<int>(pos % kTile);
    for (int c = 0; c < kKvHeads * kHeadDim; ++c)
      open_tile[c * kTile + col] = v[static_cast<std::size_t>(i) * kKvHeads * kHeadDim + c];
    if (col == kTile - 1) {   // the tile's 16th key: quantize it (the open tile keeps its fp16 values)
      std::vector<std::uint16_t> tile(static_cast<std::size_t>(kTile) * kKvHeads * kHeadDim);
      for (int key = 0; key < kTile; ++key)
        for (int c = 0; c < kKvHeads * kHeadDim; ++c) tile[static_cast<std::size_t>(key) * kKvHeads * kHeadDim + c] = open_tile[c * kTile + key];
      std::vector<std::uint8_t> codes(static_cast<std::size_t>(kKvHeads) * kHeadDim * 16);
      std::vector<std::uint16_t> stats(static_cast<std::size_t>(kKvHeads) * kHeadDim * 2);
      QuantVTile(tile.data(), codes.data(), stats.data());
      const int t_in_page = tok / kTile;
      for (int h = 0; h < kKvHeads; ++h) {
        const std::size_t rec = (static_cast<std::size_t>(page) * kKvHeads + h) * tiles_per_page + t_in_page;
        std::memcpy(vcodes + rec * kHeadDim * 16, codes.data() + static_cast<std::size_t>(h) * kHeadDim * 16, kHeadDim * 16);
        std::memcpy(vstats + rec * kHeadDim * 2, stats.data() + static_cast<std::size_t>(h) * kHeadDim * 2, kHeadDim * 4);
      }
    }
  }
}

// q [24][256] f16, gate [24][256] f32 or null -> out [24][256] f64. Keys 0 .. n_keys - 1; the keys of tile
// (n_keys - 1) / 16 are read from the open tile in fp16, all earlier tiles dequantized.
void yahkv_oracle_kv8_attend_decode_f64(int page_tokens, int num_pages, const std::uint8_t* kcodes,
                                        const std::uint16_t* kscales, const std::uint8_t* vcodes,
                                        const std::uint16_t* vstats, const std::uint16_t* open_tile,
                                        const std::int32_t* table, int table_len, std::int64_t n_keys,
                                        const std::uint16_t* q, const float* gate, double scale, double* out,
                                        int threads) {
  const Pools g{page_tokens, num_pages, const_cast<std::uint8_t*>(kcodes), const_cast<std::uint16_t*>(kscales),
                const_cast<std::uint8_t*>(vcodes), const_cast<std::uint16_t*>(vstats)};
  const int tiles_per_page = page_tokens / kTile;
  const std::int64_t n = n_keys;
  const std::int64_t n_tiles = (n + kTile - 1) / kTile, cur = (n - 1) / kTile;
  std::vector<float> kd(static_cast<std::size_t>(n_tiles) * kTile * kKvHeads * kHeadDim), vd(kd.size());
  ParallelFor(static_cast<int>(n_tiles), threads, [&](int t) {
    for (int key = 0; key < kTile; ++key) {
      const std::int64_t pos = static_cast<std::int64_t>(t) * kTile + key;
      if (pos >= n) break;
      const std::int64_t page = PageOf(g, table, table_len, pos);
      const int tok = static_cast<int>(pos % page_tokens);
      std::uint8_t codes[kKvHeads * kHeadDim];
      std::uint16_t scales[kKvHeads * 4];
      for (int h = 0; h < kKvHeads; ++h) {
        const std::size_t rec = static_cast<std::size_t>(page) * kKvHeads + h;
        std::memcpy(codes + h * kHeadDim, kcodes + (rec * page_tokens + tok) * kHeadDim, kHeadDim);
        std::memcpy(scales + h * 4, kscales + (rec * page_tokens + tok) * 4, 8);
      }
      DeqK(codes, scales, kd.data() + static_cast<std::size_t>(pos) * kKvHeads * kHeadDim);
    }
    float* vt = vd.data() + static_cast<std::size_t>(t) * kTile * kKvHeads * kHeadDim;
    if (t == cur) {
      for (int key = 0; key < kTile; ++key)
        for (int c = 0; c < kKvHeads * kHeadDim; ++c) vt[key * kKvHeads * kHeadDim + c] = H2F(open_tile[c * kTile + key]);
    } else {
      const std::int64_t pos = static_cast<std::int64_t>(t) * kTile;
      const std::int64_t page = PageOf(g, table, table_len, pos);
      const int t_in_page = static_cast<int>(pos % page_tokens) / kTile;
      std::vector<std::uint8_t> codes(static_cast<std::size_t>(kKvHeads) * kHeadDim * 16);
      std::vector<std::uint16_t> stats(static_cast<std::size_t>(kKvHeads) * kHeadDim * 2);
      for (int h = 0; h < kKvHeads; ++h) {
        const std::size_t rec = (static_cast<std::size_t>(page) * kKvHeads + h) * tiles_per_page + t_in_page;
        std::memcpy(codes.data() + static_cast<std::size_t>(h) * kHeadDim * 16, vcodes + rec * kHeadDim * 16, kHeadDim * 16);
        std::memcpy(stats.data() + static_cast<std::size_t>(h) * kHeadDim * 2, vstats + rec * kHeadDim * 2, kHeadDim * 4);
      }
      DeqVTile(codes.data(), stats.data(), vt);
    }
  });
  ParallelFor(kQHeads, threads, [&](int hh) {
    const int h = hh / kGroup;
    double qd[kHeadDim];
    for (int d = 0; d < kHeadDim; ++d) qd[d] = H2F(q[hh * kHeadDim + d]);
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
