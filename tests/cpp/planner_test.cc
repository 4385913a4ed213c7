// Host-only checks of the two work planners in csrc/kv_host.hpp (no GPU, no library: the header has no CUDA calls).
//   PlanDecode: every page of every (sequence, kv head) lies in exactly one split-K unit, in order; units of more
//   than one page have an even page count except a sequence's last; a sequence of eight or more long units gets
//   graded sizes (its last units about half as long); the list is sorted longest first; partial slots are the combine items'.
//   PlanPrefill: tiles come as neighbouring pairs of query heads of one kv head with equal rows and key ranges; the
//   pairs of the last, partly filled wave are split along the keys into parts whose ranges tile the whole range, the
//   parts of one head every second entry and every second part slot, one merge entry per head.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <set>
#include <vector>

#include "csrc/kv_host.hpp"

#define EXPECT(c)                                                         \
  do {                                                                    \
    if (!(c)) {                                                           \
      std::fprintf(stderr, "%s:%d: EXPECT(%s) failed\n", __FILE__, __LINE__, #c); \
      std::exit(1);                                                       \
    }                                                                     \
  } while (0)

using namespace yahkv;

static yahkv_config Config(int max_seqs, int max_pages, int n_layers) {
  yahkv_config c{};
  c.n_layers = n_layers;
  c.num_pages = max_seqs * max_pages;
  c.fmt = YAHKV_FMT_Q8_0;
  c.max_seqs = max_seqs;
  c.max_pages_per_seq = max_pages;
  c.max_batch_tokens = 8192;
  c.max_splits = 64;
  return c;
}

static void CheckDecodePlan(const std::vector<int>& lens, int n_splits) {
  const int n = static_cast<int>(lens.size());
  KvHost host(Config(n, 2048, 1));
  std::vector<std::int32_t> ids;
  for (int len : lens) {
    std::int32_t s = -1;
    EXPECT(host.SeqCreate(&s).code == YAHKV_OK);
    EXPECT(host.SeqReserve(s, len).code == YAHKV_OK);
    EXPECT(host.SeqSetLen(s, 0, len).code == YAHKV_OK);
    ids.push_back(s);
  }
  bool changed = false;
  EXPECT(host.PlanDecode(0, n, ids.data(), n_splits, 64, n * kKvHeads * 64, &changed).code == YAHKV_OK);
  EXPECT(changed);
  const auto& units = host.units();
  const auto& items = host.items();
  EXPECT(static_cast<int>(items.size()) == n * kKvHeads);
  // coverage per (batch row, kv head), in partial order
  std::map<std::pair<int, int>, std::vector<DecodeUnit>> by_row;
  std::set<int> partials;
  for (std::size_t i = 0; i < units.size(); ++i) {
    const DecodeUnit& u = units[i];
    EXPECT(u.page_end > u.page_begin);
    EXPECT(partials.insert(u.partial).second);
    by_row[{u.batch, u.kvh}].push_back(u);
    if (i > 0)   // longest first
      EXPECT(units[i - 1].page_end - units[i - 1].page_begin >= u.page_end - u.page_begin);
  }
  for (int b = 0; b < n; ++b)
    for (int h = 0; h < kKvHeads; ++h) {
      auto row = by_row[{b, h}];
      std::sort(row.begin(), row.end(), [](const DecodeUnit& a, const DecodeUnit& c) { return a.partial < c.partial; });
      const CombineItem it = items[static_cast<std::size_t>(b) * kKvHeads + h];
      const int pages = (lens[static_cast<std::size_t>(b)] + kPageTokens - 1) / kPageTokens;
      EXPECT(it.n_partials == static_cast<int>(row.size()));
      int at = 0;
      for (std::size_t k = 0; k < row.size(); ++k) {
        EXPECT(row[k].partial == it.first_partial + static_cast<int>(k));
        EXPECT(row[k].page_begin == at);
        EXPECT(row[k].n_keys == lens[static_cast<std::size_t>(b)] && row[k].seq == ids[static_cast<std::size_t>(b)]);
        const int np = row[k].page_end - row[k].page_begin;
        if (k + 1 < row.size()) EXPECT(np == 1 || np % 2 == 0);   // the two page sets of a CTA alternate pages
        at = row[k].page_end;
      }
      EXPECT(at == pages);
      if (n_splits > 0) EXPECT(static_cast<int>(row.size()) <= n_splits);
      const int first = row.front().page_end - row.front().page_begin;
      for (const DecodeUnit& u : row) EXPECT(u.page_end - u.page_begin <= first);
      if (row.size() >= 8 && first >= 16) {   // graded: the last whole unit is about half of the first (short units
        // are rounded to even page counts, which can use up the pages before the graded ones are reached)
        const int last_full = row[row.size() - 2].page_end - row[row.size() - 2].page_begin;
        EXPECT(2 * last_full <= first + 4);
      }
    }
  // the same call again: nothing to upload
  EXPECT(host.PlanDecode(0, n, ids.data(), n_splits, 64, n * kKvHeads * 64, &changed).code == YAHKV_OK);
  EXPECT(!changed);
}

static void CheckPrefillPlan(const std::vector<int>& cached, const std::vector<int>& chunks, int n_sm) {
  const int n = static_cast<int>(cached.size());
  KvHost host(Config(n, 1024, 1));
  std::vector<std::int32_t> ids, cl;
  for (int i = 0; i < n; ++i) {
    std::int32_t s = -1;
    EXPECT(host.SeqCreate(&s).code == YAHKV_OK);
    EXPECT(host.SeqReserve(s, cached[static_cast<std::size_t>(i)] + chunks[static_cast<std::size_t>(i)]).code == YAHKV_OK);
    EXPECT(host.SeqSetLen(s, 0, cached[static_cast<std::size_t>(i)] + chunks[static_cast<std::size_t>(i)]).code == YAHKV_OK);
    ids.push_back(s);
    cl.push_back(chunks[static_cast<std::size_t>(i)]);
  }
  std::vector<PrefillSeq> seqs;
  std::vector<PrefillTile> tiles;
  std::vector<PrefillMerge> merges;
  int n_parts = 0, max_pages = 0;
  std::int64_t rows = 0, scratch_rows = 0;
  EXPECT(host.PlanPrefill(0, n, ids.data(), cl.data(), 8192, n_sm, &seqs, &tiles, &merges, &n_parts, &rows, &scratch_rows,
                          &max_pages).code == YAHKV_OK);
  EXPECT(tiles.size() % 2 == 0);
  std::int64_t want_rows = 0;
  for (int c : chunks) want_rows += c;
  EXPECT(rows == want_rows);
  // pairs: two heads of one kv head, everything else equal; part slots of a pair are neighbours
  std::set<int> slots;
  for (std::size_t i = 0; i < tiles.size(); i += 2) {
    const PrefillTile &a = tiles[i], &b = tiles[i + 1];
    EXPECT(a.head % 2 == 0 && b.head == a.head + 1 && a.head / kGroup == b.head / kGroup);
    EXPECT(a.kv_row0 == b.kv_row0 && a.q_row0 == b.q_row0 && a.n_rows == b.n_rows && a.pos0 == b.pos0);
    EXPECT(a.jt_begin == b.jt_begin && a.jt_end == b.jt_end && a.jt_end > a.jt_begin);
    EXPECT((a.part < 0) == (b.part < 0));
    if (a.part >= 0) {
      EXPECT(b.part == a.part + 1);
      EXPECT(slots.insert(a.part).second && slots.insert(b.part).second);
    }
  }
  EXPECT(static_cast<int>(slots.size()) == n_parts);
  // merges: one per head; the parts of a head every second entry, every second slot, their key ranges tiling the whole
  EXPECT(merges.size() % 2 == 0);
  std::size_t split_tiles = 0;
  for (const PrefillMerge& m : merges) {
    const PrefillTile& first = tiles[static_cast<std::size_t>(m.tile_index)];
    EXPECT(m.n_parts >= 2 && m.n_parts <= kPrefillMaxParts && first.part >= 0 && first.jt_begin == 0);
    int at = 0;
    for (int k = 0; k < m.n_parts; ++k) {
      const PrefillTile& t = tiles[static_cast<std::size_t>(m.tile_index + 2 * k)];
      EXPECT(t.head == first.head && t.q_row0 == first.q_row0 && t.part == first.part + 2 * k);
      EXPECT(t.jt_begin == at && t.jt_end - t.jt_begin >= 2);
      at = t.jt_end;
    }
    EXPECT(at == (first.pos0 + first.n_rows + 63) / 64);
    split_tiles += static_cast<std::size_t>(m.n_parts);
  }
  // every (query tile, head) once: whole tiles plus one merge per split tile
  std::size_t whole = 0;
  for (const PrefillTile& t : tiles) whole += t.part < 0 ? 1 : 0;
  std::size_t want_tiles = 0;
  for (int c : chunks) want_tiles += static_cast<std::size_t>((c + kPrefillTileRows - 1) / kPrefillTileRows) * kQHeads;
  EXPECT(whole + merges.size() == want_tiles);
  EXPECT(whole + split_tiles == tiles.size());
  if (n_sm >= 2) {   // what is left whole fills whole waves of n_sm / 2 pairs, or the tail could not be split
    const std::size_t wave = static_cast<std::size_t>(n_sm / 2);
    if (!merges.empty()) EXPECT((whole / 2) % wave == 0 || merges.size() / 2 < (want_tiles / 2) % wave);
  } else {
    EXPECT(merges.empty());
  }
}

int main() {
  CheckDecodePlan({1, 63, 64, 65, 4096}, 0);
  CheckDecodePlan({32768, 1024, 20000, 777}, 0);
  CheckDecodePlan({131072, 131072}, 64);
  CheckDecodePlan({131072}, 7);
  CheckDecodePlan({5000, 300}, 1);
  CheckPrefillPlan({30720, 30720, 30720, 30720}, {2048, 2048, 2048, 2048}, 148);
  CheckPrefillPlan({500}, {129}, 20);
  CheckPrefillPlan({500}, {129}, 0);
  CheckPrefillPlan({0, 63, 500, 1000, 64}, {100, 1, 129, 300, 128}, 14);
  CheckPrefillPlan({0}, {1}, 148);
  std::printf("planner_test: ok\n");
  return 0;
}
