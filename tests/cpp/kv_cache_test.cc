// The C++ adapter over the C ABI on a host-only context (no GPU): allocator behaviour and the engine's error
// convention (exceptions before any launch). Built and run by tests/test_cpp_adapter_cpu.py.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "engine/model/kv_cache.hpp"

using yah::model::KvCache;
using yah::model::KvError;

#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) {                                                            \
      std::fprintf(stderr, "%s:%d: EXPECT(%s) failed\n", __FILE__, __LINE__, #cond); \
      std::exit(1);                                                           \
    }                                                                         \
  } while (0)

template <class F>
int CodeOf(F&& f) {
  try {
    f();
  } catch (const KvError& e) {
    return e.code();
  }
  return YAHKV_OK;
}

int main() {
  KvCache kv = KvCache::OwnState(KvCache::Config(/*device=*/-1, /*n_layers=*/2, /*num_pages=*/6, /*max_seqs=*/3,
                                                 /*max_pages_per_seq=*/4));
  const int a = kv.NewSequence(), b = kv.NewSequence();
  kv.Reserve(a, 130);
  EXPECT((kv.Table(a) == std::vector<std::int32_t>{0, 1, 2}));
  EXPECT(kv.PagesFree() == 3);
  kv.SetLength(a, 130);
  EXPECT(kv.Length(a, 0) == 130 && kv.Length(a, 1) == 130);
  EXPECT(CodeOf([&] { kv.Reserve(b, 64 * 4); }) == YAHKV_ERR_NO_PAGES);   // 4 needed, 3 free: nothing changes
  EXPECT(kv.PagesFree() == 3 && kv.Table(b).empty());
  EXPECT(CodeOf([&] { kv.Reserve(a, 64 * 5); }) == YAHKV_ERR_CAPACITY);
  EXPECT(CodeOf([&] { kv.SetTable(b, {1}); }) == YAHKV_ERR_INVALID);      // page 1 belongs to a
  EXPECT(CodeOf([&] { kv.SetTable(b, {6}); }) == YAHKV_ERR_INVALID);      // out of range
  kv.FreeSequence(a);
  EXPECT(kv.PagesFree() == 6);
  kv.Reserve(b, 65);
  EXPECT((kv.Table(b) == std::vector<std::int32_t>{2, 1}));               // last freed, first reused
  // the hot path refuses to run without a GPU: there is no CPU fallback
  const std::vector<std::int32_t> seqs{b};
  const std::vector<std::int64_t> pos{0};
  char dummy[16] = {};
  EXPECT(CodeOf([&] { kv.Append(0, seqs, pos, dummy, dummy); }) == YAHKV_ERR_NO_DEVICE);
  EXPECT(CodeOf([&] { kv.AttendDecode(0, seqs, dummy, nullptr, dummy); }) == YAHKV_ERR_NO_DEVICE);
  const float* fdummy = reinterpret_cast<const float*>(dummy);
  EXPECT(CodeOf([&] { kv.RopeAppend(0, seqs, pos, fdummy, fdummy, fdummy, fdummy, fdummy, 1e-6F, dummy); }) == YAHKV_ERR_NO_DEVICE);
  EXPECT(CodeOf([&] { kv.DecodeStepHostAsync(0, seqs, dummy, dummy, dummy, nullptr, dummy); }) == YAHKV_ERR_NO_DEVICE);
  EXPECT(CodeOf([&] { kv.WaitHostSteps(); }) == YAHKV_ERR_NO_DEVICE);
  EXPECT(CodeOf([&] { kv.AttendPrefill(0, seqs, {1}, dummy, nullptr, dummy); }) == YAHKV_ERR_NO_DEVICE);
  alignas(16) float fal[4] = {};
  EXPECT(CodeOf([&] { kv.AttendDecodeRawQ(0, seqs, fal, fal, 1e-6F, nullptr, dummy); }) == YAHKV_ERR_NO_DEVICE);
  EXPECT(CodeOf([&] { kv.AttendPrefillRawQ(0, seqs, {1}, fal, fal, 1e-6F, nullptr, dummy); }) == YAHKV_ERR_NO_DEVICE);
  EXPECT(CodeOf([&] { kv.SaveState(seqs, "/nonexistent-dir/x.yahkv"); }) != YAHKV_OK);
  EXPECT(CodeOf([&] { (void)kv.LoadState("/nonexistent-dir/x.yahkv", 1); }) != YAHKV_OK);
  EXPECT(CodeOf([&] {   // a batch needs the device too
           KvCache::DecodeBatch batch(kv, seqs);
           batch.Prepare(1);
           batch.Plan();
           batch.DecodeLayerRaw(0, fal, fal, fal, fal, fal, 1e-6F, nullptr, dummy);
           batch.Advance();
           batch.Commit(1);
         }) != YAHKV_OK);
  EXPECT(kv.Length(b, 0) == 0);
  // a bad geometry is refused at creation
  yahkv_config bad = KvCache::Config(-1, 1, 4, 1, 1);
  bad.head_dim = 128;
  EXPECT(CodeOf([&] { (void)KvCache::OwnState(bad); }) == YAHKV_ERR_INVALID);
  KvCache moved = std::move(kv);
  EXPECT(moved.PagesFree() == 4);
  std::puts("kv_cache_test: ok");
  return 0;
}
