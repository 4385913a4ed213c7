// Pieces shared by the split-K decode kernels of all cache formats (decode_attn.cu, kv8a16.cu, kv4a16.cu,
// decode_f16.cu): the wait for a ring stage, its release by the last of a page's warps, and the merge of a unit's
// eight warps into one partial. The kernels differ in what a stage holds and in the arithmetic between these calls.
#pragma once

#include <cmath>

#include "kernels.cuh"
#include "ptx.cuh"

namespace yahkv {

// Cross-warp merge scratch at the end of a unit: per warp acc [6][kDecodeMergeStride] f32 and (m, l) [8][2].
constexpr int kDecodeMergeStride = kHeadDim + 8;
constexpr int kDecodeMergeWarpFloats = kGroup * kDecodeMergeStride + 16;

// Waits until fill number `gen` of a stage has landed. The mbarrier wait names its phase by parity only, so it is safe
// only for a warp that is not a whole phase ahead of the barrier; a stage is refilled by the OTHER page set, whose
// progress this warp does not otherwise depend on, so the warp first makes sure (a bounded poll of the stage's fill
// counter, almost always true at once) that the fill it wants has at least been issued. A wait that gives up does not
// stop the warp half-way through a unit: it raises the CTA's abort flag so that nothing more is fetched and every
// other warp stops waiting, the warp finishes on whatever the ring holds, and the status word the kernel sets at its
// end marks the call's results invalid. Called by a whole converged warp; returns the warp's new `alive`.
__device__ __forceinline__ bool RingWait(bool alive, int* fill_cnt_s, std::uint64_t* full_bar_s, int gen,
                                         volatile int* abort_flag) {
  if (!alive) return false;
  const int need = gen + 1;
  volatile int* fills = fill_cnt_s;
  bool ok = *abort_flag == 0;
  if (ok && *fills < need) {
    const std::uint64_t t0 = GlobalTimerNs();
    while (*fills < need) {
      if (*abort_flag != 0 || GlobalTimerNs() - t0 > kWaitLimitNs) {
        ok = false;
        break;
      }
    }
  }
  if (!ok || !__all_sync(0xFFFFFFFFU, MbarWait(full_bar_s, static_cast<std::uint32_t>(gen) & 1U))) {
    *abort_flag = 1;
    return false;
  }
  return true;
}

// This warp is done reading a stage (every shared-memory read of it has been consumed by an MMA or sits in a
// register). True in every lane of the last of the page's `n_warps` warps, which then refills the stage.
__device__ __forceinline__ bool RingRelease(int* done_cnt_s, int lane, int n_warps) {
  __syncwarp();
  int last = 0;
  if (lane == 0) {
    __threadfence_block();
    last = atomicAdd(done_cnt_s, 1) == n_warps - 1;
    if (last) {
      *done_cnt_s = 0;
      __threadfence_block();
    }
  }
  return __shfl_sync(0xFFFFFFFFU, last, 0) != 0;
}

// After the page loop and a __syncthreads: when a wait gave up, the copies the CTA still has in flight get one more
// bounded wait each (the fill counters say which phase of which stage is outstanding), so that none lands in shared
// memory that is about to be reused. Every thread calls it; ends with a barrier of its own when it had work.
__device__ __forceinline__ void RingDrainAfterAbort(volatile int* abort_flag, const int* fill_cnt,
                                                    std::uint64_t* full_bar, int n_bars) {
  if (*abort_flag == 0) return;   // the same value in every thread
  if (threadIdx.x == 0)
    for (int x = 0; x < n_bars; ++x)
      if (fill_cnt[x] > 0) MbarWait(&full_bar[x], static_cast<std::uint32_t>(fill_cnt[x] - 1) & 1U, 20000000ULL);
  __syncthreads();
}

// Merge of the unit's warps into one partial (max, sum, unnormalised acc[6][256]) and its store. `merge` is shared
// memory of kWarps * kDecodeMergeWarpFloats floats (the ring, free by now); o_acc[c][0..3] of lane (g, t) holds heads
// 2t, 2t+1 of two output dims of tile c: dims 16c + g and 16c + g + 8 (kInterleaved = false) or 16c + 2g and
// 16c + 2g + 1 (true, the order the q8_0 / q4_0 kernel's transposed byte loads produce). A warp that saw no page has
// max -inf and weight 0. Called by all kWarps * 32 threads.
template <int kWarps, bool kInterleaved>
__device__ __forceinline__ void MergeUnitAndStore(float* merge, const float (&o_acc)[16][4], float m_run, float l_run,
                                                  int warp, int lane, float* __restrict__ acc_out,
                                                  float* __restrict__ ml_out) {
  const int g = lane >> 2, t = lane & 3;
  {
    float* mine = merge + warp * kDecodeMergeWarpFloats;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      if (2 * t < kGroup) {   // lanes with t = 3 hold the two padding heads
        if constexpr (kInterleaved) {
          *reinterpret_cast<float2*>(mine + (2 * t) * kDecodeMergeStride + 16 * c + 2 * g) = make_float2(o_acc[c][0], o_acc[c][2]);
          *reinterpret_cast<float2*>(mine + (2 * t + 1) * kDecodeMergeStride + 16 * c + 2 * g) = make_float2(o_acc[c][1], o_acc[c][3]);
        } else {
          mine[(2 * t) * kDecodeMergeStride + 16 * c + g] = o_acc[c][0];
          mine[(2 * t + 1) * kDecodeMergeStride + 16 * c + g] = o_acc[c][1];
          mine[(2 * t) * kDecodeMergeStride + 16 * c + g + 8] = o_acc[c][2];
          mine[(2 * t + 1) * kDecodeMergeStride + 16 * c + g + 8] = o_acc[c][3];
        }
      }
    }
    if (t == 0 && g < kGroup) {
      float* ml = mine + kGroup * kDecodeMergeStride;
      ml[2 * g] = m_run;
      ml[2 * g + 1] = l_run;
    }
  }
  __syncthreads();
  // one output dim per thread and head (a CTA of fewer than 256 threads takes several dims per thread)
#pragma unroll
  for (int h = 0; h < kGroup; ++h) {
    float mw[kWarps], M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      mw[w] = merge[w * kDecodeMergeWarpFloats + kGroup * kDecodeMergeStride + 2 * h];
      M = fmaxf(M, mw[w]);
    }
    float wgt[kWarps], lsum = 0.0F;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      wgt[w] = mw[w] == -INFINITY ? 0.0F : exp2f(mw[w] - M);
      lsum = fmaf(wgt[w], merge[w * kDecodeMergeWarpFloats + kGroup * kDecodeMergeStride + 2 * h + 1], lsum);
    }
    for (int dim = threadIdx.x; dim < kHeadDim; dim += kWarps * 32) {
      float a = 0.0F;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) a = fmaf(wgt[w], merge[w * kDecodeMergeWarpFloats + h * kDecodeMergeStride + dim], a);
      acc_out[h * kHeadDim + dim] = a;
    }
    if (threadIdx.x == 0) ml_out[2 * h] = M, ml_out[2 * h + 1] = lsum;
  }
}

}  // namespace yahkv
