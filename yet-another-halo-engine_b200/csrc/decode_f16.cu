// Split-K decode attention over unquantized fp16 pages (YAHKV_FMT_F16), the reference's fp16 cache mode.
//
// Stands in for dattn_part (engine/gpu/loom/tools/gen_decode_attn.py:97-335) over fp16 pools; the combine pass is the
// one of the other formats. Numeric contract as there: keys 0 .. len-1 visible, score = q.k * scale, fp32 softmax
// statistics, partials (max, sum, unnormalised acc) merged in unit order.
//
// The shape of the quantized formats' kernel: one CTA per split-K unit, a ring of page stages filled by non-multicast
// TMA on one mbarrier each (K and V of a page as four swizzled 64 x 128 B boxes per side: 64 KB per stage, three
// stages, one CTA per SM), eight warps on two pages at a time, warp = 16 keys with all 256 dims, last-arriver refill,
// fill-generation guard, bounded waits with the abort drain. What differs is that nothing is decoded: S^T = Q K^T runs
// on the f16 MMA with the fp16 query as the A operand (rows 0-5 = the six heads) and the K rows as ldmatrix delivers
// them, accumulating over the sixteen 16-dim steps in the instruction's accumulator; O^T += V^T P^T takes V through
// ldmatrix.trans and the weights as an fp16 high part plus residual. 4096 B per token per layer, HBM-bound.
#include <cuda_fp16.h>

#include <cmath>

#include "decode_ring.cuh"
#include "qrope.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

namespace yahkv {
namespace {

constexpr int kStages = 3;
constexpr int kKeyGroups = 4;
constexpr int kPageSets = 2;
constexpr int kWarps = kKeyGroups * kPageSets;
constexpr int kThreads = kWarps * 32;
constexpr int kBoxBytes = 64 * 128;                       // 64 token rows x 64 dims of fp16
constexpr int kBoxesPerSide = kHeadDim * 2 / 128;         // 4
constexpr int kSideBytes = kBoxesPerSide * kBoxBytes;     // 32768
static_assert(kSideBytes == RecordCodeBytes(kFmtF16), "record size");
constexpr int kStageBytes = 2 * kSideBytes;
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kQLanes = 24;
constexpr int kQSteps = kHeadDim / 16;                    // k-steps of the score product
constexpr int kQfragOff = kRingBytes;                     // [16 steps][24 lanes][2] u32
constexpr int kBarOff = kQfragOff + kQSteps * kQLanes * 8;
constexpr int kDoneOff = kBarOff + 8 * kStages;
constexpr int kFillOff = kDoneOff + 4 * kStages;
constexpr int kAbortOff = kFillOff + 4 * kStages;
constexpr int kSmemBytes = (kAbortOff + 4 + 127) / 128 * 128;
static_assert(kSmemBytes + 1024 <= 228 * 1024, "one CTA per SM");
static_assert(kWarps * kDecodeMergeWarpFloats * 4 <= kRingBytes, "the merge scratch aliases the ring");
constexpr float kLazyRescale = 4.0F;
constexpr int kStatusSmemMisaligned = 2;

template <bool kQRaw>   // kQRaw: the raw f32 query, normed and rotated in the prologue (qrope.cuh)
__global__ void __launch_bounds__(kThreads, 1)
    F16DecodePartKernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                        PoolView pool, int layer, const std::int32_t* __restrict__ tables, int table_stride,
                        const DecodeUnit* __restrict__ units, const __half* __restrict__ q, const QueryRaw qraw,
                        float scale_log2,
                        float* __restrict__ partial_acc, float* __restrict__ partial_ml, int* status) {
  ChainedKernelEntry();
  extern __shared__ __align__(1024) std::uint8_t smem[];
  std::uint32_t* qfrag = reinterpret_cast<std::uint32_t*>(smem + kQfragOff);
  std::uint64_t* full_bar = reinterpret_cast<std::uint64_t*>(smem + kBarOff);
  int* done_cnt = reinterpret_cast<int*>(smem + kDoneOff);
  int* fill_cnt = reinterpret_cast<int*>(smem + kFillOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kAbortOff);
  if ((SmemAddr(smem) & 1023U) != 0) {   // never seen; a misaligned swizzle would corrupt results
    if (threadIdx.x == 0) atomicExch(status, kStatusSmemMisaligned);
    return;
  }

  const DecodeUnit u = units[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kw = warp & (kKeyGroups - 1);   // keys 16 kw .. 16 kw + 15 of a page
  const int par = warp / kKeyGroups;        // this warp's pages: index par, par + 2, ... of the unit
  const int t = lane & 3;
  const int n_pages = u.page_end - u.page_begin;
  if (n_pages <= 0) return;
  const std::int32_t* row = tables + static_cast<std::size_t>(u.seq) * table_stride + u.page_begin;

  // Gather of one page into a ring stage; a whole converged warp calls it, one elected lane issues. Once a wait has
  // given up nothing more is fetched: the CTA is on its way out and must not leave copies in flight behind it.
  auto issue = [&](int s, std::int32_t page) {
    if (*abort_flag != 0) return;
    page = min(max(page, 0), pool.num_pages - 1);   // never trust a table entry read from memory
    const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + page) * kKvHeads + u.kvh;
    const int y = static_cast<int>(rec * kPageTokens);
    std::uint8_t* st = smem + s * kStageBytes;
    if (ElectOne()) {
      fill_cnt[s] += 1;
      MbarArriveExpectTx(&full_bar[s], kStageBytes);
#pragma unroll
      for (int b = 0; b < kBoxesPerSide; ++b) {
        TmaLoad2D(st + b * kBoxBytes, &kmap, b * 128, y, &full_bar[s]);
        TmaLoad2D(st + kSideBytes + b * kBoxBytes, &vmap, b * 128, y, &full_bar[s]);
      }
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      PrefetchTensorMap(&kmap);
      PrefetchTensorMap(&vmap);
      for (int s = 0; s < kStages; ++s) {
        MbarInit(&full_bar[s], 1);
        done_cnt[s] = 0;
        fill_cnt[s] = 0;
      }
      *abort_flag = 0;
      FenceBarrierInit();
    }
    __syncwarp();
    for (int i = 0; i < kStages && i < n_pages; ++i) issue(i, __ldg(row + i));
  }

  // Query operands: warp h < 6 lays out head h. For k-step ks (dims 16 ks .. 16 ks + 15) the A registers of lane
  // (g = head, t) are a0 = dims 16 ks + 2t, + 1 and a2 = dims 16 ks + 8 + 2t, + 1 (rows 8-15 of the MMA stay zero).
  // Lane l of the warp holds dims 8 l .. 8 l + 7 = step l / 2, half l % 2: its four dword pairs go to t = 0 .. 3.
  if (warp < kGroup) {
    const uint4 raw = LoadQueryLane8<kQRaw>(q, qraw, static_cast<std::size_t>(u.batch) * kQHeads + u.kvh * kGroup + warp,
                                            u.n_keys - 1, lane);
    const std::uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    const int ks = lane >> 1, half = lane & 1;
#pragma unroll
    for (int tt = 0; tt < 4; ++tt) qfrag[((ks * kQLanes + warp * 4 + tt) << 1) + half] = w[tt];
  }
  __syncthreads();   // barriers initialised, query operands visible
  const int qlane = lane < kQLanes ? lane : lane - 8;   // the two padding rows of the MMA reuse heads 4, 5
  const std::uint32_t qa_addr = SmemAddr(qfrag + (qlane << 1));

  float o_acc[16][4];   // [c][0..3] = (dim 16c + g, head 2t), (16c + g, 2t+1), (16c + g + 8, 2t), (16c + g + 8, 2t+1)
#pragma unroll
  for (int c = 0; c < 16; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[c][i] = 0.0F;
  float m_run = -INFINITY, l_run = 0.0F;
  bool alive = true;

  // ldmatrix row addresses inside a 64 x 128 B box (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
  //   K (plain): matrices = (keys 0-7 | 8-15) x (chunk 2x | 2x + 1): lane -> key (lane & 7) + 8 ((lane >> 3) & 1), chunk half lane >> 4
  //   V (transposed): matrices = (chunk 2x | 2x + 1) x (keys 0-7 | 8-15): lane -> key (lane & 7) + 8 (lane >> 4), chunk half (lane >> 3) & 1
  const int k_key = kw * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const std::uint32_t lm_k = k_key * 128 + (((lane >> 4) ^ (k_key & 7)) << 4);
  const int v_key = kw * 16 + (lane & 7) + (lane >> 4) * 8;
  const std::uint32_t lm_v = v_key * 128 + ((((lane >> 3) & 1) ^ (v_key & 7)) << 4);
  const int my_key0 = kw * 16 + 2 * t;   // keys whose scores this thread holds: kt * 8 + 2t + j of the group's 16

  for (int i = par; i < n_pages; i += kPageSets) {
    const int s = i % kStages;
    const int gen = i / kStages;
    std::int32_t refill_page = 0;
    if (lane == 0 && i + kStages < n_pages) refill_page = __ldg(row + i + kStages);
    alive = RingWait(alive, fill_cnt + s, &full_bar[s], gen, abort_flag);
    const std::uint32_t k_base = SmemAddr(smem + s * kStageBytes), v_base = k_base + kSideBytes;

    // ---- S^T = Q K^T: sixteen 16-dim steps accumulate in the MMA; rows 0-5 of the result are the six heads ----
    float acc[2][4] = {{0.0F, 0.0F, 0.0F, 0.0F}, {0.0F, 0.0F, 0.0F, 0.0F}};
#pragma unroll
    for (int ks = 0; ks < kQSteps; ++ks) {
      std::uint32_t w[4], a0, a2;
      LdMatrixX4(k_base + (ks >> 2) * kBoxBytes + (lm_k ^ (static_cast<std::uint32_t>(ks & 3) << 5)), w);
      asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(a0), "=r"(a2) : "r"(qa_addr + ks * (kQLanes * 8)));
      MmaF16(acc[0], a0, 0U, a2, 0U, w[0], w[2]);
      MmaF16(acc[1], a0, 0U, a2, 0U, w[1], w[3]);
    }
    float sc[2][2];
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) sc[kt][0] = acc[kt][0] * scale_log2, sc[kt][1] = acc[kt][1] * scale_log2;
    if ((u.page_begin + i + 1) * kPageTokens > u.n_keys) {   // only ever true on a sequence's last page
      const int key_pos0 = (u.page_begin + i) * kPageTokens + my_key0;
#pragma unroll
      for (int kt = 0; kt < 2; ++kt)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (key_pos0 + kt * 8 + j >= u.n_keys) sc[kt][j] = -INFINITY;
    }

    // ---- softmax statistics (per head g, the 16 keys spread over the four lanes of a quad) ----
    float tmax = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFU, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFU, tmax, 2));
    if (__any_sync(0xFFFFFFFFU, lane < kQLanes && tmax > m_run + kLazyRescale)) {
      const float m_new = fmaxf(m_run, tmax);
      const float alpha = m_new == -INFINITY ? 1.0F : Exp2Fast(m_run - m_new);
      m_run = m_new;
      l_run *= alpha;
      const float al0 = __shfl_sync(0xFFFFFFFFU, alpha, (2 * t) * 4);
      const float al1 = __shfl_sync(0xFFFFFFFFU, alpha, (2 * t + 1) * 4);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        o_acc[c][0] *= al0, o_acc[c][2] *= al0;
        o_acc[c][1] *= al1, o_acc[c][3] *= al1;
      }
    }
    const float m_use = m_run == -INFINITY ? 0.0F : m_run;
    std::uint32_t p_hi[2], p_lo[2];
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) {
      const float p0 = Exp2Fast(sc[kt][0] - m_use), p1 = Exp2Fast(sc[kt][1] - m_use);
      l_run += p0 + p1;
      const __half2 h2 = __floats2half2_rn(p0, p1);
      const float2 hf = __half22float2(h2);
      const __half2 l2 = __floats2half2_rn(p0 - hf.x, p1 - hf.y);
      p_hi[kt] = *reinterpret_cast<const std::uint32_t*>(&h2);
      p_lo[kt] = *reinterpret_cast<const std::uint32_t*>(&l2);
    }

    // ---- O^T += V^T P^T: ldmatrix.trans hands over 16 dims x 16 keys of V as the A operand ----
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      std::uint32_t w[4];
      LdMatrixX4Trans(v_base + (c >> 2) * kBoxBytes + (lm_v ^ (static_cast<std::uint32_t>(c & 3) << 5)), w);
      MmaF16(o_acc[c], w[0], w[1], w[2], w[3], p_hi[0], p_hi[1]);
      MmaF16(o_acc[c], w[0], w[1], w[2], w[3], p_lo[0], p_lo[1]);
    }

    // The last of the page's four warps to finish with the stage refills it. The MMAs above consumed every ldmatrix
    // result, so this warp's reads of the stage are complete.
    const bool last = RingRelease(&done_cnt[s], lane, kKeyGroups);
    if (last && i + kStages < n_pages) issue(s, __shfl_sync(0xFFFFFFFFU, refill_page, 0));
  }
  if (!alive && lane == 0) atomicExch(status, kStatusWaitTimeout);
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 1);
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 2);

  // Every stage has been consumed (or a wait gave up): the ring is free to hold the merge scratch.
  __syncthreads();
  RingDrainAfterAbort(abort_flag, fill_cnt, full_bar, kStages);
  MergeUnitAndStore<kWarps, false>(reinterpret_cast<float*>(smem), o_acc, m_run, l_run, warp, lane,
                                     partial_acc + static_cast<std::size_t>(u.partial) * kPartialAccFloats,
                                     partial_ml + static_cast<std::size_t>(u.partial) * kPartialMlFloats);
}

}  // namespace

cudaError_t ConfigureF16Kernels() {
  cudaError_t e = cudaFuncSetAttribute(F16DecodePartKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(F16DecodePartKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

cudaError_t LaunchF16DecodePart(const DecodeLaunch& a, cudaStream_t stream) {
  if (a.n_units <= 0 || a.n_seqs <= 0) return cudaSuccess;
  if (a.q_raw) {
    const QueryRaw qr{static_cast<const float*>(a.q_dev), a.q_weight_dev, a.rope_tab_dev, a.q_eps, a.rope_rows};
    return LaunchChained(F16DecodePartKernel<true>, a.n_units, kThreads, kSmemBytes, stream, *a.kmap, *a.vmap, a.pool,
                         a.layer, a.tables_dev, a.table_stride, a.units_dev, static_cast<const __half*>(nullptr), qr,
                         a.scale_log2, a.partial_acc, a.partial_ml, a.status_dev);
  }
  return LaunchChained(F16DecodePartKernel<false>, a.n_units, kThreads, kSmemBytes, stream, *a.kmap, *a.vmap, a.pool,
                       a.layer, a.tables_dev, a.table_stride, a.units_dev, static_cast<const __half*>(a.q_dev), QueryRaw{},
                       a.scale_log2, a.partial_acc, a.partial_ml, a.status_dev);
}

}  // namespace yahkv
