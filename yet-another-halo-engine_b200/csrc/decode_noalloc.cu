// yahkv_attend_decode_noalloc: decode attention for callers that must not allocate GPU memory.
//
// Who needs this. A host that runs inside someone else's memory budget: an inference server whose allocator has
// already claimed the whole device, a plugin loaded into a process that forbids cudaMalloc after start-up, or a
// real-time loop where an allocation's implicit device synchronisation is not acceptable. Such a caller owns every
// buffer itself (pools, block tables, lengths, queries, outputs) and cannot create a yahkv context, because
// yahkv_create allocates.
//
// What it is. The same split-K attention kernel and combine kernel as yahkv_attend_decode, launched through the same
// launchers, but everything they use beyond the caller's inputs and outputs (the list of split-K units, the per-unit
// partial results, the status word) lives in one file-scope __device__ array below instead of a cudaMalloc'ed
// workspace. A small planning kernel writes the unit list into that array from the caller's device-resident lengths,
// so no host-to-device copy and no pinned staging is needed either. The call uses no cudaMalloc, cudaFree, pinned
// allocation or stream/event creation.
//
// Limits and sharing. The array is YAHKV_NOALLOC_SCRATCH_BYTES (about 6.4 MB) and every GPU that loads the library
// holds it until the process exits. It bounds a call to n_seqs <= 256 and n_seqs * 4 * n_splits <= 1024 units; larger
// requests are refused. All calls on a device share the array: two calls whose kernels overlap on the GPU (different
// streams, or different host threads) race on it, so callers serialise them on one stream. The array keeps the last
// call's contents; everything a call reads it first rewrites (the planner rewrites the units and combine items, each
// unit rewrites its partial), and the status word is cleared by the planner.
//
// Errors. A kernel that gives up a bounded wait records it in the array's status word; yahkv_noalloc_status copies
// that word into the caller's host memory with one asynchronous copy on the caller's stream (no allocation either).
//
// First call on a device. The array's name in host code is only a handle, not a device address, so the first call on
// each device resolves its address with cudaGetSymbolAddress (and raises the kernels' shared-memory limit). That
// set-up call should happen before any stream capture begins.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/yahkv.h"
#include "kernels.cuh"

namespace yahkv {
namespace {

constexpr int kMaxUnits = YAHKV_NOALLOC_MAX_UNITS;
constexpr int kMaxSeqs = YAHKV_NOALLOC_MAX_SEQS;

// Layout of the scratch array (byte offsets, each a multiple of 256).
constexpr std::size_t kUnitsOff = 0;
constexpr std::size_t kItemsOff = kUnitsOff + sizeof(DecodeUnit) * kMaxUnits;
constexpr std::size_t kMlOff = kItemsOff + sizeof(CombineItem) * kMaxSeqs * kKvHeads;
constexpr std::size_t kStatusOff = kMlOff + sizeof(float) * kPartialMlFloats * kMaxUnits;
constexpr std::size_t kAccOff = kStatusOff + 256;
constexpr std::size_t kScratchBytes = kAccOff + sizeof(float) * kPartialAccFloats * kMaxUnits;
static_assert(kScratchBytes <= YAHKV_NOALLOC_SCRATCH_BYTES, "scratch layout exceeds the documented size");
static_assert(kItemsOff % 256 == 0 && kMlOff % 256 == 0 && kStatusOff % 256 == 0 && kAccOff % 256 == 0, "alignment");

static __device__ __align__(256) unsigned char g_noalloc_scratch[YAHKV_NOALLOC_SCRATCH_BYTES];

// One thread per (sequence, kv head): writes that pair's units and its combine item. Device code may name the array
// directly; the host passes the resolved address anyway so both sides agree on one pointer.
__global__ void NoAllocPlanKernel(unsigned char* scratch, const std::int32_t* __restrict__ lens, int n_seqs,
                                  int n_splits, int max_keys) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx == 0) *reinterpret_cast<int*>(scratch + kStatusOff) = 0;
  if (idx >= n_seqs * kKvHeads) return;
  const int b = idx / kKvHeads, h = idx % kKvHeads;
  const int n = min(max(lens[b], 1), max_keys);      // lengths come from device memory: clamp, never trust
  const int pages = (n + kPageTokens - 1) / kPageTokens;
  const int per = (pages + n_splits - 1) / n_splits;
  const int nu = (pages + per - 1) / per;            // <= n_splits
  auto* units = reinterpret_cast<DecodeUnit*>(scratch + kUnitsOff);
  auto* items = reinterpret_cast<CombineItem*>(scratch + kItemsOff);
  const int first = idx * n_splits;
  items[idx] = {first, nu};
  for (int k = 0; k < n_splits; ++k) {
    DecodeUnit u;
    u.batch = b, u.seq = b, u.kvh = h;
    u.page_begin = min(k * per, pages);
    u.page_end = min((k + 1) * per, pages);          // empty past nu: such a unit exits without writing anything,
                                                     // and the combine item above (n_partials = nu) never reads it
    u.n_keys = n;
    u.partial = first + k;
    u.pad = 0;
    units[first + k] = u;
  }
}

struct DeviceSetup {
  bool done = false;
  unsigned char* scratch = nullptr;
};
std::mutex g_mu;
DeviceSetup g_setup[64];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int Refuse(char* err, int cap, int code, const char* msg) {
  if (err != nullptr && cap > 0) std::snprintf(err, static_cast<std::size_t>(cap), "%s", msg);
  return code;
}

}  // namespace
}  // namespace yahkv

using namespace yahkv;

extern "C" int yahkv_attend_decode_noalloc(const yahkv_noalloc_args* a, char* err, int32_t err_cap) {
  if (a == nullptr) return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: null argument block");
  if (a->fmt != YAHKV_FMT_Q8_0 && a->fmt != YAHKV_FMT_Q4_0)
    return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: fmt must be YAHKV_FMT_Q8_0 or YAHKV_FMT_Q4_0");
  if (a->n_layers < 1 || a->layer < 0 || a->layer >= a->n_layers || a->num_pages < 1 || a->table_stride < 1)
    return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: layer, n_layers, num_pages or table_stride out of range");
  if (1LL * a->n_layers * a->num_pages * kKvHeads * kPageTokens >= (1LL << 31))
    return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: pool too large for the row index");
  if (a->n_seqs < 1 || a->n_splits < 1)
    return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: n_seqs and n_splits must be positive");
  if (a->n_seqs > kMaxSeqs || 1LL * a->n_seqs * kKvHeads * a->n_splits > kMaxUnits)
    return Refuse(err, err_cap, YAHKV_ERR_CAPACITY,
                  "attend_decode_noalloc: request exceeds the static scratch (n_seqs <= 256 and "
                  "n_seqs * 4 * n_splits <= 1024)");
  if (a->out_dtype != YAHKV_OUT_F16 && a->out_dtype != YAHKV_OUT_F32)
    return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: bad out_dtype");
  if (a->kcodes == nullptr || a->vcodes == nullptr || a->kscales == nullptr || a->vscales == nullptr ||
      a->tables_dev == nullptr || a->lens_dev == nullptr || a->q_dev == nullptr || a->out_dev == nullptr)
    return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: null device pointer");
  if ((reinterpret_cast<std::uintptr_t>(a->kcodes) | reinterpret_cast<std::uintptr_t>(a->vcodes) |
       reinterpret_cast<std::uintptr_t>(a->kscales) | reinterpret_cast<std::uintptr_t>(a->vscales)) & 15)
    return Refuse(err, err_cap, YAHKV_ERR_INVALID, "attend_decode_noalloc: pool pointers must be 16-byte aligned");

  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return Refuse(err, err_cap, YAHKV_ERR_NO_DEVICE, "attend_decode_noalloc: no current CUDA device");
  unsigned char* scratch = nullptr;
  {
    // Once per device, with that device current: resolve the array's device address (its host-side name is not one)
    // and raise the attention kernels' dynamic shared-memory limit. Neither allocates.
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceSetup& s = g_setup[dev];
    if (!s.done) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess) return Refuse(err, err_cap, YAHKV_ERR_CUDA, cudaGetErrorString(e));
      e = ConfigureDecodeKernels();
      if (e != cudaSuccess) return Refuse(err, err_cap, YAHKV_ERR_CUDA, cudaGetErrorString(e));
      if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q{};
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
          return Refuse(err, err_cap, YAHKV_ERR_CUDA, "attend_decode_noalloc: cuTensorMapEncodeTiled not available");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
      }
      s.scratch = static_cast<unsigned char*>(p);
      s.done = true;
    }
    scratch = s.scratch;
  }

  // Tensor maps over the caller's code pools (a host-side encode into a struct on this stack; nothing is allocated).
  CUtensorMap kmap, vmap;
  {
    const cuuint64_t row_bytes = static_cast<cuuint64_t>(CodeBytes(a->fmt));
    const cuuint64_t rows = static_cast<cuuint64_t>(a->n_layers) * a->num_pages * kKvHeads * kPageTokens;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {128, kPageTokens};
    const cuuint32_t elem[2] = {1, 1};
    for (int side = 0; side < 2; ++side) {
      const CUresult r = g_encode(side == 0 ? &kmap : &vmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                                  const_cast<void*>(side == 0 ? a->kcodes : a->vcodes), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return Refuse(err, err_cap, YAHKV_ERR_CUDA, "attend_decode_noalloc: tensor map encode failed");
    }
  }

  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  const int pairs = a->n_seqs * kKvHeads;
  NoAllocPlanKernel<<<(pairs + 127) / 128, 128, 0, stream>>>(scratch, a->lens_dev, a->n_seqs, a->n_splits,
                                                             a->table_stride * kPageTokens);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return Refuse(err, err_cap, YAHKV_ERR_CUDA, cudaGetErrorString(e));

  DecodeLaunch l{};
  l.kmap = &kmap, l.vmap = &vmap;
  l.pool.kcodes = static_cast<std::uint8_t*>(const_cast<void*>(a->kcodes));
  l.pool.vcodes = static_cast<std::uint8_t*>(const_cast<void*>(a->vcodes));
  l.pool.kscales = static_cast<std::uint16_t*>(const_cast<void*>(a->kscales));
  l.pool.vscales = static_cast<std::uint16_t*>(const_cast<void*>(a->vscales));
  l.pool.fmt = a->fmt, l.pool.num_pages = a->num_pages, l.pool.n_layers = a->n_layers;
  l.pool.kv_head_begin = 0, l.pool.kv_head_count = kKvHeads;
  l.layer = a->layer;
  l.tables_dev = a->tables_dev, l.table_stride = a->table_stride;
  l.units_dev = reinterpret_cast<const DecodeUnit*>(scratch + kUnitsOff);
  l.n_units = pairs * a->n_splits;
  l.items_dev = reinterpret_cast<const CombineItem*>(scratch + kItemsOff);
  l.n_seqs = a->n_seqs;
  l.q_dev = a->q_dev, l.gate_dev = a->gate_dev, l.out_dev = a->out_dev, l.out_f32 = a->out_dtype == YAHKV_OUT_F32;
  l.scale_log2 = (a->softmax_scale == 0.0F ? 1.0F / 16.0F : a->softmax_scale) * 1.4426950408889634F;
  l.partial_acc = reinterpret_cast<float*>(scratch + kAccOff);
  l.partial_ml = reinterpret_cast<float*>(scratch + kMlOff);
  l.status_dev = reinterpret_cast<int*>(scratch + kStatusOff);
  e = LaunchDecodePart(l, stream);
  if (e == cudaSuccess) e = LaunchDecodeCombine(l, stream);
  if (e != cudaSuccess) return Refuse(err, err_cap, YAHKV_ERR_CUDA, cudaGetErrorString(e));
  return YAHKV_OK;
}

extern "C" int yahkv_noalloc_status(int32_t* status_host, void* stream) {
  if (status_host == nullptr) return YAHKV_ERR_INVALID;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return YAHKV_ERR_NO_DEVICE;
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_setup[dev].done) return YAHKV_ERR_ORDER;   // the address is resolved by the first attend call
    scratch = g_setup[dev].scratch;
  }
  const cudaError_t e = cudaMemcpyAsync(status_host, scratch + kStatusOff, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                        static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? YAHKV_OK : YAHKV_ERR_CUDA;
}
