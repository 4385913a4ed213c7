// The C++ adapter (engine/model/kv_cache.hpp) driving the GPU path the way the engine's drivers would: one sequence,
// a prompt appended as one chunk and attended with AttendPrefill, then decode steps (Append + AttendDecode, then a
// DecodeBatch), a snapshot saved and loaded back, all with
// device buffers this program owns. Inputs come from raw files written by tests/test_cpp_adapter_gpu.py, outputs go
// back to raw files that the test compares with the CPU oracle.
//   usage: kv_cache_gpu_test <dir> <n_prompt> <n_decode> <fmt>
//   reads  <dir>/k.f16 v.f16 [n][4][256], q.f16 [n][24][256], table.i32   (n = n_prompt + n_decode)
//   writes <dir>/prefill.f32 [n_prompt][24][256], decode.f32 [n_decode][24][256], loaded.f32 [24][256]
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "engine/model/kv_cache.hpp"

using yah::model::KvCache;

static std::vector<char> ReadFile(const std::string& path) {
  std::FILE* f = std::fopen(path.c_str(), "rb");
  if (f == nullptr) std::exit(2);
  std::fseek(f, 0, SEEK_END);
  const long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<char> buf(static_cast<std::size_t>(n));
  if (std::fread(buf.data(), 1, buf.size(), f) != buf.size()) std::exit(2);
  std::fclose(f);
  return buf;
}
static void WriteFile(const std::string& path, const void* p, std::size_t bytes) {
  std::FILE* f = std::fopen(path.c_str(), "wb");
  if (f == nullptr || std::fwrite(p, 1, bytes, f) != bytes) std::exit(2);
  std::fclose(f);
}
#define CUDA_OK(call)                                                       \
  do {                                                                      \
    if ((call) != cudaSuccess) {                                            \
      std::fprintf(stderr, "%s:%d: %s failed\n", __FILE__, __LINE__, #call); \
      std::exit(3);                                                         \
    }                                                                       \
  } while (0)

int main(int argc, char** argv) {
  if (argc != 5) return 2;
  const std::string dir = argv[1];
  const int n_prompt = std::atoi(argv[2]), n_decode = std::atoi(argv[3]), fmt = std::atoi(argv[4]);
  const int n = n_prompt + n_decode;
  const auto k = ReadFile(dir + "/k.f16"), v = ReadFile(dir + "/v.f16"), q = ReadFile(dir + "/q.f16");
  const auto tab = ReadFile(dir + "/table.i32");
  const std::vector<std::int32_t> table(reinterpret_cast<const std::int32_t*>(tab.data()),
                                        reinterpret_cast<const std::int32_t*>(tab.data() + tab.size()));
  const std::size_t kv_row = 4 * 256 * 2, q_row = 24 * 256 * 2, o_row = 24 * 256 * 4;
  void *kd = nullptr, *vd = nullptr, *qd = nullptr, *od = nullptr;
  CUDA_OK(cudaMalloc(&kd, k.size()));
  CUDA_OK(cudaMalloc(&vd, v.size()));
  CUDA_OK(cudaMalloc(&qd, q.size()));
  CUDA_OK(cudaMalloc(&od, static_cast<std::size_t>(n) * o_row));
  void* ld = nullptr;   // output of the sequence loaded back from a snapshot
  CUDA_OK(cudaMalloc(&ld, o_row));
  CUDA_OK(cudaMemcpy(kd, k.data(), k.size(), cudaMemcpyHostToDevice));
  CUDA_OK(cudaMemcpy(vd, v.data(), v.size(), cudaMemcpyHostToDevice));
  CUDA_OK(cudaMemcpy(qd, q.data(), q.size(), cudaMemcpyHostToDevice));

  try {
    KvCache kv = KvCache::OwnState(KvCache::Config(/*device=*/0, /*n_layers=*/1, /*num_pages=*/64, /*max_seqs=*/2,
                                                   /*max_pages_per_seq=*/static_cast<int>(table.size()), fmt));
    const std::int32_t seq = kv.NewSequence();
    kv.SetTable(seq, table);
    // the prompt as one chunk: append, then causal attention over it (LoomPrefill::RunAttention's KV section)
    std::vector<std::int32_t> ids(static_cast<std::size_t>(n_prompt), seq);
    std::vector<std::int64_t> pos(static_cast<std::size_t>(n_prompt));
    for (int i = 0; i < n_prompt; ++i) pos[static_cast<std::size_t>(i)] = i;
    kv.Append(0, ids, pos, kd, vd);
    kv.AttendPrefill(0, {seq}, {n_prompt}, qd, nullptr, od, YAHKV_OUT_F32);
    // decode steps: append position p, attend over 0 .. p (LoomDecoder::Step's attention section)
    const int n_eager = n_decode / 2;
    for (int s = 0; s < n_eager; ++s) {
      const int p = n_prompt + s;
      kv.Append(0, {seq}, {p}, static_cast<const char*>(kd) + p * kv_row, static_cast<const char*>(vd) + p * kv_row);
      kv.AttendDecode(0, {seq}, static_cast<const char*>(qd) + p * q_row, nullptr, static_cast<char*>(od) + p * o_row,
                      YAHKV_OUT_F32);
    }
    // the remaining steps as a device-resident batch: the position lives on the device, the host only queues launches
    {
      KvCache::DecodeBatch batch(kv, {seq});
      batch.Prepare(n_decode - n_eager);
      for (int s = n_eager; s < n_decode; ++s) {
        const int p = n_prompt + s;
        batch.Plan();
        batch.DecodeLayer(0, static_cast<const char*>(kd) + p * kv_row, static_cast<const char*>(vd) + p * kv_row,
                          static_cast<const char*>(qd) + p * q_row, nullptr, static_cast<char*>(od) + p * o_row, YAHKV_OUT_F32);
        batch.Advance();
      }
      batch.Commit(n_decode - n_eager);
    }
    kv.Synchronize();
    if (kv.Length(seq, 0) != n) return 4;
    // snapshot round trip: the sequence comes back on other pages under another id and attends to the same result
    kv.SaveState({seq}, dir + "/state.yahkv");
    const std::vector<std::int32_t> loaded = kv.LoadState(dir + "/state.yahkv", 1);
    if (loaded.size() != 1 || loaded[0] == seq || kv.Length(loaded[0], 0) != n) return 7;
    kv.AttendDecode(0, loaded, static_cast<const char*>(qd) + (n - 1) * q_row, nullptr, ld, YAHKV_OUT_F32);
    kv.Synchronize();
    // an order error is thrown before anything is launched and leaves the cache as it was
    bool thrown = false;
    try {
      kv.Append(0, {seq}, {n + 5}, kd, vd);
    } catch (const yah::model::KvError& e) {
      thrown = e.code() == YAHKV_ERR_ORDER;
    }
    if (!thrown || kv.Length(seq, 0) != n) return 5;
  } catch (const yah::model::KvError& e) {
    std::fprintf(stderr, "KvError %d: %s\n", e.code(), e.what());
    return 6;
  }
  std::vector<char> out(static_cast<std::size_t>(n) * o_row);
  CUDA_OK(cudaMemcpy(out.data(), od, out.size(), cudaMemcpyDeviceToHost));
  WriteFile(dir + "/prefill.f32", out.data(), static_cast<std::size_t>(n_prompt) * o_row);
  WriteFile(dir + "/decode.f32", out.data() + static_cast<std::size_t>(n_prompt) * o_row,
            static_cast<std::size_t>(n_decode) * o_row);
  std::vector<char> lout(o_row);
  CUDA_OK(cudaMemcpy(lout.data(), ld, lout.size(), cudaMemcpyDeviceToHost));
  WriteFile(dir + "/loaded.f32", lout.data(), lout.size());
  std::puts("kv_cache_gpu_test: ok");
  return 0;
}
