// Device-resident decode stepping: the per-step bookkeeping of a fixed batch of sequences done by small kernels from
// device-resident lengths, so that a whole multi-layer decode step (plan, then per layer append + attend, then
// advance) touches no host state and can be captured once into a CUDA graph and replayed.
//
// The reference engine works the same way: positions come from a device array and steps are queued back to back
// with no host round trip (engine/model/loom_decoder.hpp:131-133, :239; docs/architecture.md:171). Its single
// sequence becomes a batch here, and its fixed one-workgroup-per-page grid becomes a fixed number of split-K units
// per sequence, reserved for the growth the caller announced; units that hold no page yet exit at once.
#include "kernels.cuh"
#include "ptx.cuh"

namespace yahkv {
namespace {

// One thread per (batch row, kv head): this step appends position lens[b] and attends over lens[b] + 1 keys.
__global__ void BatchPlanKernel(const std::int32_t* __restrict__ lens, const BatchSeq* __restrict__ seqs, int n_seqs,
                                const std::int32_t* __restrict__ tables, int table_stride, int unit_pages,
                                int num_pages, DecodeUnit* __restrict__ units, CombineItem* __restrict__ items,
                                std::int64_t* __restrict__ slots, VTileWork* __restrict__ vwork,
                                std::int32_t* __restrict__ state_rows, int n_layers) {
  ChainedKernelEntry();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_seqs * kKvHeads) return;
  const int b = idx / kKvHeads, h = idx % kKvHeads;
  const BatchSeq bs = seqs[b];
  const int pos = max(lens[b], 0);
  const int n = pos + 1;
  const int pages = min((n + kPageTokens - 1) / kPageTokens, table_stride);
  const int used = min((pages + unit_pages - 1) / unit_pages, bs.n_units);
  const int first = bs.first_unit + h * bs.n_units;
  items[idx] = {first, used};
  for (int k = 0; k < bs.n_units; ++k) {
    DecodeUnit u;
    u.batch = b, u.seq = bs.seq_row, u.kvh = h;
    u.page_begin = min(k * unit_pages, pages);
    // the last reserved unit takes whatever is left, so an under-reserved batch degrades to longer units, never to
    // missing keys
    u.page_end = k == bs.n_units - 1 ? pages : min((k + 1) * unit_pages, pages);
    u.n_keys = n;
    u.partial = first + k;
    u.pad = bs.open_cur;
    units[first + k] = u;
  }
  if (h == 0) {
    std::int32_t page = tables[static_cast<std::size_t>(bs.seq_row) * table_stride + min(pos / kPageTokens, table_stride - 1)];
    page = min(max(page, 0), num_pages - 1);
    slots[b] = static_cast<std::int64_t>(page) * kPageTokens + pos % kPageTokens;
    if (vwork != nullptr) {
      // Tile formats: the step's token is key pos % 16 of tile pos / 16. A single-token append stays in the
      // sequence's current open buffer (the host planner's rule for a call that touches one tile), and the tile is
      // quantized when this is its 16th key.
      VTileWork w;
      w.state_row = bs.seq_row * n_layers;
      w.phys_tile = page * kTilesPerPage + (pos % kPageTokens) / kTileKeys;
      w.n_old = pos % kTileKeys;
      w.n_keys = w.n_old + 1;
      w.read_buf = bs.open_cur;
      w.write_buf = bs.open_cur;
      w.complete = w.n_keys == kTileKeys ? 1 : 0;
      w.pad = 0;
      for (int j = 0; j < kTileKeys; ++j) w.src[j] = j == w.n_old ? b : -1;
      vwork[b] = w;
      state_rows[b] = bs.seq_row * n_layers;
    }
  }
}

__global__ void BatchAdvanceKernel(std::int32_t* __restrict__ lens, int n_seqs, int by) {
  ChainedKernelEntry();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < n_seqs) lens[b] += by;
}

// A wait that cannot succeed: the barrier expects one arrival and nobody arrives. The kernel leaves by the same path
// a real kernel takes when a copy never lands: it stops waiting at the limit, sets the sticky status word, returns.
__global__ void WaitProbeKernel(int* status, std::uint64_t limit_ns) {
  __shared__ std::uint64_t bar;
  if (threadIdx.x == 0) {
    MbarInit(&bar, 1);
    FenceBarrierInit();
  }
  __syncthreads();
  const bool ok = MbarWait(&bar, 0, limit_ns);
  if (!ok && threadIdx.x == 0) atomicExch(status, kStatusWaitTimeout);
}

}  // namespace

cudaError_t LaunchWaitProbe(int* status_dev, std::uint64_t limit_ns, cudaStream_t stream) {
  WaitProbeKernel<<<1, 32, 0, stream>>>(status_dev, limit_ns);
  return cudaGetLastError();
}

cudaError_t LaunchBatchPlan(const std::int32_t* lens_dev, const BatchSeq* seqs_dev, int n_seqs,
                            const std::int32_t* tables_dev, int table_stride, int unit_pages, int num_pages,
                            DecodeUnit* units_dev, CombineItem* items_dev, std::int64_t* slots_dev,
                            VTileWork* vwork_dev, std::int32_t* state_rows_dev, int n_layers, cudaStream_t stream) {
  if (n_seqs <= 0) return cudaSuccess;
  const int threads = n_seqs * kKvHeads;
  return LaunchChained(BatchPlanKernel, (threads + 127) / 128, 128, 0, stream, lens_dev, seqs_dev, n_seqs, tables_dev,
                       table_stride, unit_pages, num_pages, units_dev, items_dev, slots_dev, vwork_dev, state_rows_dev,
                       n_layers);
}

cudaError_t LaunchBatchAdvance(std::int32_t* lens_dev, int n_seqs, int by, cudaStream_t stream) {
  if (n_seqs <= 0) return cudaSuccess;
  return LaunchChained(BatchAdvanceKernel, (n_seqs + 127) / 128, 128, 0, stream, lens_dev, n_seqs, by);
}

}  // namespace yahkv
