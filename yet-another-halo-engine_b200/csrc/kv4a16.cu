// The reference's 4-bit cache format kv4a16 on B200: K append (Walsh-Hadamard rotation + 16 levels per 32-dim group),
// split-K decode attention over the rotated codes, and the dequantize pass of prefill attention. The V append is the
// tile kernel of kv8a16.cu at 4 bits; the open fp16 tile, the K mean and the page / tile bookkeeping are shared with
// kv8a16.
//
// Stands in for yah_kq4 / dattn_kappend_q (4-bit) and dattn_part_q with 4-bit K and V:
// engine/gpu/loom/tools/gen_kvq.py:288-463, engine/gpu/loom/tools/gen_decode_attn.py:576-1040 (:655-717 for the rotated
// query). Arithmetic of the quantizer, operation for operation (numpy model engine/gpu/loom/tools/dattn_q_check.py:74-84):
//   x = f32(f16(k)) - mean;  r = H256 x / 16 per head, in f32: a lane of the warp holds 8 consecutive dims, butterflies
//   1, 2, 4 dims apart inside the lane, then lanes 1, 2, 4, 8, 16 apart (gen_kvq.py:344-378);
//   per 32-dim group of r: lo = min, hi = max, s = (hi - lo) / 15 (1 when 0), u = clamp(roundeven((r - lo) * (1 / s)), 0, 15);
//   a dword holds 8 dims, dim 2j at bits 4j and dim 2j + 1 at bits 16 + 4j;  pair = f16 (16 s, lo - 16 s).
// Attention sees r = (1 + u / 16) S + C' = u S / 16 + (S + C') and rotates the query the same way, so q.k is unchanged.
//
// Pools (per layer): kcodes [page][4][64 tokens][128 B], kscales [page][4][64][8 groups][2] f16,
// vcodes [page][4][4 tiles][256 channels][8 B], vscales [page][4][4][256][2] f16. 1408 B per token per layer.
#include <cuda_fp16.h>

#include <cmath>

#include "decode_ring.cuh"
#include "qrope.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

namespace yahkv {
namespace {

// r = H256 x / 16 over the 256 values a warp holds (8 consecutive dims per lane). Every sum and difference is a single
// rounded f32 operation in a fixed order: the CPU restatement does the same ones, so codes agree bit for bit.
__device__ __forceinline__ void Hadamard256(float (&x)[8], int lane) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1)
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if ((i & h) == 0) {
        const float a = x[i], b = x[i + h];
        x[i] = __fadd_rn(a, b), x[i + h] = __fsub_rn(a, b);
      }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const bool upper = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float other = __shfl_xor_sync(0xFFFFFFFFU, x[i], o);
      x[i] = upper ? __fsub_rn(other, x[i]) : __fadd_rn(x[i], other);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] *= 0.0625F;
}
__device__ __forceinline__ int NibbleShift(int i) { return 4 * (i >> 1) + ((i & 1) ? 16 : 0); }

// ---------------------------------------------------------------------------------------------------------------
// Append, K side: one warp per (token, kv head); lane l holds dims 8 l .. 8 l + 7, a 32-dim group is 4 lanes.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) Kv4AppendKKernel(PoolView pool, int layer, const std::int64_t* __restrict__ slots,
                                                        const std::int32_t* __restrict__ state_rows, int state_row_add,
                                                        const float* __restrict__ kmean,
                                                        const __half* __restrict__ k_in) {
  ChainedKernelEntry();
  const int token = blockIdx.x, h = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const std::int64_t slot = slots[token];
  if (slot < 0 || !pool.OwnsKvHead(h)) return;   // warp-uniform
  std::int64_t page = slot / kPageTokens;
  const int tok = static_cast<int>(slot % kPageTokens);
  page = min(max(page, static_cast<std::int64_t>(0)), static_cast<std::int64_t>(pool.num_pages - 1));
  const uint4 raw = *reinterpret_cast<const uint4*>(k_in + (static_cast<std::size_t>(token) * kKvHeads + h) * kHeadDim + lane * 8);
  const float* mean = kmean + (static_cast<std::size_t>(state_rows[token] + state_row_add) * kKvHeads + h) * kHeadDim + lane * 8;
  const float4 m0 = *reinterpret_cast<const float4*>(mean), m1 = *reinterpret_cast<const float4*>(mean + 4);
  const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
  const __half2* hp = reinterpret_cast<const __half2*>(&raw);
  float x[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(hp[i]);
    x[2 * i] = __fsub_rn(f.x, mm[2 * i]), x[2 * i + 1] = __fsub_rn(f.y, mm[2 * i + 1]);
  }
  Hadamard256(x, lane);
  float lo = x[0], hi = x[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) lo = fminf(lo, x[i]), hi = fmaxf(hi, x[i]);
#pragma unroll
  for (int o = 1; o <= 2; o <<= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xFFFFFFFFU, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFU, hi, o));
  }
  const float s0 = __fdiv_rn(__fsub_rn(hi, lo), 15.0F);
  const float s = s0 > 0.0F ? s0 : 1.0F;
  const float inv = __fdiv_rn(1.0F, s);
  std::uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float u = rintf(__fmul_rn(__fsub_rn(x[i], lo), inv));
    u = fminf(fmaxf(u, 0.0F), 15.0F);
    w |= static_cast<std::uint32_t>(u) << NibbleShift(i);
  }
  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + static_cast<std::size_t>(page)) * kKvHeads + h;
  *reinterpret_cast<std::uint32_t*>(pool.kcodes + rec * RecordCodeBytes(kFmtKv4) + static_cast<std::size_t>(tok) * 128 + lane * 4) = w;
  if ((lane & 3) == 0) {
    std::uint16_t* sc = pool.kscales + rec * (RecordScaleBytes(kFmtKv4, 0) / 2) + static_cast<std::size_t>(tok) * 16 + (lane >> 2) * 2;
    const float S0 = __fmul_rn(s, 16.0F);
    *reinterpret_cast<__half2*>(sc) = __halves2half2(__float2half_rn(S0), __float2half_rn(__fsub_rn(lo, S0)));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Decode attention: one CTA per split-K unit; the shape of the other formats' kernel (a ring of page stages filled by
// non-multicast TMA on one mbarrier each, warp = one 16-key tile with all 256 dims, four warps per page in work,
// last-arriver refill, fill-generation guard, bounded waits with the abort drain).
//
// A stage: the page's K codes as one swizzled 64 x 128 B box, its K pairs (2 KB), its four V tiles as stored (8 KB)
// and the V pairs (4 KB): 22,528 B. The kernel is bound by instruction latency, not by memory, and runs best as many
// small CTAs whose prologues and merges overlap: one set of four warps on a two-stage ring, four CTAs per SM (242 us
// per layer on the batch-32 workload against 251 as two sets on four stages with two CTAs per SM).
//
// Scores. With the query rotated and quantized to two int8 planes (q = step (256 hi + lo)):
//   q.r = sum_g [ (S_g / 16) sum_{d in g} q_d u_d  +  (S_g + C'_g) sum_{d in g} q_d ].
// The first sum is exact on the integer MMA (s8 planes x the nibbles as unsigned bytes 0 .. 15: a 16-byte ldmatrix row
// is one group of a key, `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are the two halves of the k dimension, and the
// query bytes are laid out in that order once per CTA). The second is a small matrix product of its own: the key's 32 B
// pair row [S_0, C'_0, S_1, C'_1, ...] is the B operand of one f16 MMA as it lies in shared memory, against the
// per-group query sums (f16 hi part in rows 0-5, residual in rows 8-13, each value in both the S and the C' slot).
// The ldmatrix rows follow the key order of the V tile's dwords (as in the kv8a16 kernel), so the weights need no
// shuffle before the second product.
// Values. v = u S / 16 + (S + C') per (tile, channel). A thread's dword holds eight keys of a channel; rotated so that
// a key pair's nibbles sit at bits 4-7 / 20-23 and or-ed into 0x5400 they are the f16 pair 64 + u (a rotate and one
// logic instruction per MMA register, no subtract), so o += (S / 16) sum p (64 + u) + (C' - 3 S) sum p.
// ---------------------------------------------------------------------------------------------------------------
#ifndef YAHKV_KV4_STAGES
#define YAHKV_KV4_STAGES 2
#endif
#ifndef YAHKV_KV4_PAGE_SETS
#define YAHKV_KV4_PAGE_SETS 1
#endif
#ifndef YAHKV_KV4_CTAS
#define YAHKV_KV4_CTAS 4
#endif
constexpr int kStages = YAHKV_KV4_STAGES;
constexpr int kKeyGroups = 4;
constexpr int kPageSets = YAHKV_KV4_PAGE_SETS;
constexpr int kCtas = YAHKV_KV4_CTAS;
constexpr int kWarps = kKeyGroups * kPageSets;
constexpr int kThreads = kWarps * 32;
constexpr int kKBytes = RecordCodeBytes(kFmtKv4);           // 8192: one 64 x 128 B box
constexpr int kVBytes = RecordCodeBytes(kFmtKv4);           // 8192: [4 tiles][256 channels][8 B]
constexpr int kVsBytes = RecordScaleBytes(kFmtKv4, 1);      // 4096
constexpr int kKsBytes = RecordScaleBytes(kFmtKv4, 0);      // 2048: [64 tokens][8 groups][2] f16
constexpr int kTxBytes = kKBytes + kVBytes + kVsBytes + kKsBytes;
constexpr int kKOff = 0;
constexpr int kVOff = kKOff + kStages * kKBytes;
constexpr int kVsOff = kVOff + kStages * kVBytes;
constexpr int kKsOff = kVsOff + kStages * kVsBytes;
constexpr int kRingBytes = kKsOff + kStages * kKsBytes;
constexpr int kQLanes = 24;
constexpr int kQfragOff = kRingBytes;                              // [8 groups][24 lanes][4] u32
constexpr int kBarOff = kQfragOff + kBlocksPerRow * kQLanes * 16;
constexpr int kDoneOff = kBarOff + 8 * kStages;
constexpr int kFillOff = kDoneOff + 4 * kStages;
constexpr int kQStepOff = kFillOff + 4 * kStages;                  // [8] f32
constexpr int kQSumOff = kQStepOff + 32;                           // [8 heads][8 groups] u32: f16 hi | f16 residual << 16
constexpr int kAbortOff = kQSumOff + 8 * 8 * 4;
constexpr int kSmemBytes = (kAbortOff + 4 + 127) / 128 * 128;
static_assert(kCtas * (kSmemBytes + 1024) <= 228 * 1024, "the resident CTAs of an SM");
static_assert(kWarps * kDecodeMergeWarpFloats * 4 <= kRingBytes, "the merge scratch aliases the ring");
constexpr float kLazyRescale = 4.0F;
constexpr float kQSteps = 32000.0F;
constexpr int kStatusSmemMisaligned = 2;

__device__ __forceinline__ void MmaS8U8(int (&d)[4], const std::uint32_t (&a)[4], std::uint32_t b0, std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void MmaF16Zero(float (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                           std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0F));
}
__device__ __forceinline__ void LoadQ4(std::uint32_t (&a)[4], std::uint32_t addr) {
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
}
__device__ __forceinline__ std::uint32_t PackBytes(int b0, int b1, int b2, int b3) {
  return (static_cast<std::uint32_t>(b0) & 255U) | ((static_cast<std::uint32_t>(b1) & 255U) << 8) |
         ((static_cast<std::uint32_t>(b2) & 255U) << 16) | ((static_cast<std::uint32_t>(b3) & 255U) << 24);
}

template <bool kQRaw>   // kQRaw: the raw f32 query, normed and rotated in the prologue (qrope.cuh)
__global__ void __launch_bounds__(kThreads, kCtas)
    Kv4DecodePartKernel(const __grid_constant__ CUtensorMap kmap, PoolView pool, int layer,
                        const std::int32_t* __restrict__ tables, int table_stride, const DecodeUnit* __restrict__ units,
                        const __half* __restrict__ q, const QueryRaw qraw, float scale_log2,
                        const __half* __restrict__ open_tiles,
                        int n_layers, float* __restrict__ partial_acc, float* __restrict__ partial_ml, int* status) {
  ChainedKernelEntry();
  extern __shared__ __align__(1024) std::uint8_t smem[];
  std::uint32_t* qfrag = reinterpret_cast<std::uint32_t*>(smem + kQfragOff);
  std::uint64_t* full_bar = reinterpret_cast<std::uint64_t*>(smem + kBarOff);
  int* done_cnt = reinterpret_cast<int*>(smem + kDoneOff);
  int* fill_cnt = reinterpret_cast<int*>(smem + kFillOff);
  float* q_step = reinterpret_cast<float*>(smem + kQStepOff);
  std::uint32_t* q_sum = reinterpret_cast<std::uint32_t*>(smem + kQSumOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kAbortOff);
  if ((SmemAddr(smem) & 1023U) != 0) {   // never seen; a misaligned swizzle would corrupt results
    if (threadIdx.x == 0) atomicExch(status, kStatusSmemMisaligned);
    return;
  }

  const DecodeUnit u = units[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kw = warp & (kKeyGroups - 1);   // tile kw of a page
  const int par = warp / kKeyGroups;        // this warp's pages: index par, par + 2, ... of the unit
  const int g = lane >> 2, t = lane & 3;
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
    if (ElectOne()) {
      fill_cnt[s] += 1;
      MbarArriveExpectTx(&full_bar[s], kTxBytes);
      TmaLoad2D(smem + kKOff + s * kKBytes, &kmap, 0, y, &full_bar[s]);
      BulkLoad(smem + kVOff + s * kVBytes, pool.vcodes + rec * kVBytes, kVBytes, &full_bar[s]);
      BulkLoad(smem + kVsOff + s * kVsBytes, pool.vscales + rec * (kVsBytes / 2), kVsBytes, &full_bar[s]);
      BulkLoad(smem + kKsOff + s * kKsBytes, pool.kscales + rec * (kKsBytes / 2), kKsBytes, &full_bar[s]);
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      PrefetchTensorMap(&kmap);
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

  // Query: warp h < 6 rotates head h (lane l holds dims 8 l .. 8 l + 7), quantizes it to 16 bits against the rotated
  // row's largest magnitude (q16 = rint(r * 32000 / amax), hi = (q16 + 128) >> 8, lo = q16 - 256 hi) and leaves, per
  // group (4 lanes) and lane, the A operand of the integer MMA: bytes in the order the code nibbles unpack
  // (dims 0, 4, 1, 5 of the lane's 8, then 2, 6, 3, 7), hi plane in rows 0-5, lo plane in rows 8-13.
  for (int hq = warp; hq < kGroup; hq += kWarps) {   // one head per warp and pass
    const uint4 raw = LoadQueryLane8<kQRaw>(q, qraw, static_cast<std::size_t>(u.batch) * kQHeads + u.kvh * kGroup + hq,
                                            u.n_keys - 1, lane);
    const __half2* hp = reinterpret_cast<const __half2*>(&raw);
    float x[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(hp[i]);
      x[2 * i] = f.x, x[2 * i + 1] = f.y;
    }
    Hadamard256(x, lane);
    float amax = 0.0F;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFU, amax, o));
    const float inv = amax > 0.0F ? kQSteps / amax : 0.0F;
    const float step = amax / kQSteps;
    int hi[8], lo[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q16 = __float2int_rn(x[i] * inv);
      hi[i] = (q16 + 128) >> 8;
      lo[i] = q16 - hi[i] * 256;
      sum += q16;
    }
    const uint4 frag = make_uint4(PackBytes(hi[0], hi[4], hi[1], hi[5]), PackBytes(lo[0], lo[4], lo[1], lo[5]),
                                  PackBytes(hi[2], hi[6], hi[3], hi[7]), PackBytes(lo[2], lo[6], lo[3], lo[7]));
    *reinterpret_cast<uint4*>(qfrag + (((lane >> 2) * kQLanes + hq * 4 + (lane & 3)) << 2)) = frag;
    sum += __shfl_xor_sync(0xFFFFFFFFU, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFU, sum, 2);   // the group's sum of the quantized query, exact
    if ((lane & 3) == 0) {
      const float qf = static_cast<float>(sum) * step;
      const __half h16 = __float2half_rn(qf);
      const __half l16 = __float2half_rn(qf - __half2float(h16));
      q_sum[hq * 8 + (lane >> 2)] = static_cast<std::uint32_t>(__half_as_ushort(h16)) |
                                      (static_cast<std::uint32_t>(__half_as_ushort(l16)) << 16);
    }
    if (lane == 0) q_step[hq] = step;
  }
  __syncthreads();   // barriers initialised, query operands visible
  const int qlane = lane < kQLanes ? lane : lane - 8;   // the two padding rows of the MMA reuse heads 4, 5
  const int head = qlane >> 2;
  const std::uint32_t qa_addr = SmemAddr(qfrag + (qlane << 2));
  const float c1 = scale_log2 * q_step[head] * 0.0625F;   // softmax scale x log2(e) x query step x 1 / 16
  // A operand of the pair-row product: k = 2t, 2t+1 (S_t, C'_t) and 2t+8, 2t+9 (S_t+4, C'_t+4) all take the group's
  // query sum; rows 0-5 its f16 hi part, rows 8-13 the residual.
  std::uint32_t qs_a0, qs_a1, qs_a2, qs_a3;
  {
    const std::uint32_t s0 = q_sum[head * 8 + t], s1 = q_sum[head * 8 + t + 4];
    qs_a0 = __byte_perm(s0, s0, 0x1010), qs_a1 = __byte_perm(s0, s0, 0x3232);
    qs_a2 = __byte_perm(s1, s1, 0x1010), qs_a3 = __byte_perm(s1, s1, 0x3232);
  }

  float o_acc[16][4];   // [c][0..3] = (channel 16c + g, head 2t), (16c + g, 2t+1), (16c + g + 8, 2t), (16c + g + 8, 2t+1)
#pragma unroll
  for (int c = 0; c < 16; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[c][i] = 0.0F;
  float m_run = -INFINITY, l_run = 0.0F;
  bool alive = true;

  // ldmatrix row of this lane in the K box: matrix (lane >> 3) & 1 is key tile kt, row lane & 7 its column c, which is
  // key 4 (c / 2) + 2 kt + c % 2 of the 16; 16-byte chunk (= group) 2x + (lane >> 4) of the 128-byte row, swizzled.
  const int lm_key = kw * kTileKeys + 4 * ((lane & 7) >> 1) + 2 * ((lane >> 3) & 1) + (lane & 1);
  const std::uint32_t lm0 = lm_key * 128 + (((lane >> 4) ^ (lm_key & 7)) << 4);
  const int cur_tile = (u.n_keys - 1) / kTileKeys;
  const __half* open_buf = open_tiles + ((static_cast<std::size_t>(u.seq) * n_layers + layer) * 2 + (u.pad & 1)) * kOpenTileHalfs +
                           static_cast<std::size_t>(u.kvh) * kHeadDim * kTileKeys;
  NibConsts nib{};
  nib.Load();
  // Rotations that bring this thread's four keys of a V dword to bits 4-7 / 20-23: the pair (4t, 4t+1) sits at bits
  // 8 (t & 1) + (0, 16), the pair (4t+2, 4t+3) four bits higher; what else rotates in is masked away.
  const int v_rot_lo = (8 * (t & 1) + 28) & 31, v_rot_hi = 8 * (t & 1);

  for (int i = par; i < n_pages; i += kPageSets) {
    const int s = i % kStages;
    const int gen = i / kStages;
    std::int32_t refill_page = 0;
    if (lane == 0 && i + kStages < n_pages) refill_page = __ldg(row + i + kStages);
    alive = RingWait(alive, fill_cnt + s, &full_bar[s], gen, abort_flag);
    const int tile = (u.page_begin + i) * kTilesPerPage + kw;
    if (tile <= cur_tile) {   // warp-uniform: tiles past the newest key hold nothing
      const std::uint32_t k_base = SmemAddr(smem + kKOff + s * kKBytes);
      const std::uint8_t* ks_stage = smem + kKsOff + s * kKsBytes;

      // ---- scores ----
      float s1[2][2] = {{0.0F, 0.0F}, {0.0F, 0.0F}};   // sum_g S_g x (integer sum of q u) per (key tile, column)
#pragma unroll
      for (int x = 0; x < 4; ++x) {   // groups 2x, 2x + 1
        std::uint32_t w[4];
        LdMatrixX4(k_base + (lm0 ^ (static_cast<std::uint32_t>(x) << 5)), w);
        // pairs of groups 2x, 2x + 1 of this thread's four keys 4t .. 4t+3 of the tile (key 4t + 2 kt + j)
        uint2 pr[4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          pr[kk] = *reinterpret_cast<const uint2*>(ks_stage + (kw * kTileKeys + 4 * t + kk) * 32 + 8 * x);
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          std::uint32_t qa[4];
          LoadQ4(qa, qa_addr + (2 * x + hb) * (kQLanes * 16));
#pragma unroll
          for (int kt = 0; kt < 2; ++kt) {
            const std::uint32_t cw = w[2 * hb + kt];
            int acc[4];
            MmaS8U8(acc, qa, cw & 0x0F0F0F0FU, (cw >> 4) & 0x0F0F0F0FU);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const std::uint32_t pair = hb == 0 ? pr[2 * kt + j].x : pr[2 * kt + j].y;
              const float S = __low2float(*reinterpret_cast<const __half2*>(&pair));
              s1[kt][j] = fmaf(S, static_cast<float>(acc[j] * 256 + acc[2 + j]), s1[kt][j]);
            }
          }
        }
      }
      float sc[2][2];
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {   // sum_g (S_g + C'_g) x (group sum of q): the key's pair row is the B operand as it lies
        const int key = kw * kTileKeys + 4 * (g >> 1) + 2 * kt + (g & 1);
        const std::uint32_t* prow = reinterpret_cast<const std::uint32_t*>(ks_stage + key * 32);
        float d[4];
        MmaF16Zero(d, qs_a0, qs_a1, qs_a2, qs_a3, prow[t], prow[t + 4]);
        sc[kt][0] = fmaf(s1[kt][0], c1, (d[0] + d[2]) * scale_log2);
        sc[kt][1] = fmaf(s1[kt][1], c1, (d[1] + d[3]) * scale_log2);
      }
      if (tile == cur_tile) {   // keys past the sequence's length
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (tile * kTileKeys + 4 * t + 2 * kt + j >= u.n_keys) sc[kt][j] = -INFINITY;
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
      float psum = 0.0F;
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        const float p0 = Exp2Fast(sc[kt][0] - m_use), p1 = Exp2Fast(sc[kt][1] - m_use);
        psum += p0 + p1;
        const __half2 h2 = __floats2half2_rn(p0, p1);
        const float2 hf = __half22float2(h2);
        const __half2 l2 = __floats2half2_rn(p0 - hf.x, p1 - hf.y);
        p_hi[kt] = *reinterpret_cast<const std::uint32_t*>(&h2);
        p_lo[kt] = *reinterpret_cast<const std::uint32_t*>(&l2);
      }
      l_run += psum;

      // ---- O^T += V^T P^T: k-slots (2t, 2t+1) = keys 4t, 4t+1 and (2t+8, 2t+9) = keys 4t+2, 4t+3 ----
      if (tile == cur_tile) {   // the open tile, fp16 [channel][16 keys]
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const uint2 r0 = *reinterpret_cast<const uint2*>(open_buf + (16 * c + g) * kTileKeys + 4 * t);
          const uint2 r1 = *reinterpret_cast<const uint2*>(open_buf + (16 * c + g + 8) * kTileKeys + 4 * t);
          MmaF16(o_acc[c], r0.x, r1.x, r0.y, r1.y, p_hi[0], p_hi[1]);
          MmaF16(o_acc[c], r0.x, r1.x, r0.y, r1.y, p_lo[0], p_lo[1]);
        }
      } else {
        psum += __shfl_xor_sync(0xFFFFFFFFU, psum, 1);
        psum += __shfl_xor_sync(0xFFFFFFFFU, psum, 2);   // the tile's sum of weights of head g
        const float ps0 = __shfl_sync(0xFFFFFFFFU, psum, (2 * t) * 4), ps1 = __shfl_sync(0xFFFFFFFFU, psum, (2 * t + 1) * 4);
        // dword t / 2 of a channel holds its keys 8 (t / 2) .. + 7; this thread's four are the nibbles at bits
        // 8 (t & 1) + (0, 16, 4, 20)
        const std::uint32_t* vc = reinterpret_cast<const std::uint32_t*>(smem + kVOff + s * kVBytes + kw * (kHeadDim * 8)) + 2 * g + (t >> 1);
        const std::uint32_t* vs = reinterpret_cast<const std::uint32_t*>(smem + kVsOff + s * kVsBytes + kw * (kHeadDim * 4)) + g;
        constexpr std::uint32_t kMagic64 = 0x54005400U;   // f16 64.0 twice: a nibble at bits 4-7 adds its value
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const std::uint32_t x0 = vc[32 * c], x1 = vc[32 * c + 16];
          const std::uint32_t a0 = AndOr(__funnelshift_r(x0, x0, v_rot_lo), nib.hi_mask, kMagic64);
          const std::uint32_t a2 = AndOr(__funnelshift_r(x0, x0, v_rot_hi), nib.hi_mask, kMagic64);
          const std::uint32_t a1 = AndOr(__funnelshift_r(x1, x1, v_rot_lo), nib.hi_mask, kMagic64);
          const std::uint32_t a3 = AndOr(__funnelshift_r(x1, x1, v_rot_hi), nib.hi_mask, kMagic64);
          float d[4];
          MmaF16Zero(d, a0, a1, a2, a3, p_hi[0], p_hi[1]);
          MmaF16(d, a0, a1, a2, a3, p_lo[0], p_lo[1]);
          const std::uint32_t s0 = vs[16 * c], s1w = vs[16 * c + 8];
          const float2 st0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
          const float2 st1 = __half22float2(*reinterpret_cast<const __half2*>(&s1w));
          const float sa0 = st0.x * 0.0625F, sb0 = fmaf(-3.0F, st0.x, st0.y);   // S / 16;  S + C' - 64 S / 16
          const float sa1 = st1.x * 0.0625F, sb1 = fmaf(-3.0F, st1.x, st1.y);
          o_acc[c][0] = fmaf(sa0, d[0], fmaf(sb0, ps0, o_acc[c][0]));
          o_acc[c][1] = fmaf(sa0, d[1], fmaf(sb0, ps1, o_acc[c][1]));
          o_acc[c][2] = fmaf(sa1, d[2], fmaf(sb1, ps0, o_acc[c][2]));
          o_acc[c][3] = fmaf(sa1, d[3], fmaf(sb1, ps1, o_acc[c][3]));
        }
      }
    }

    // The last of the page's four warps to finish with the stage refills it. The MMAs above consumed every shared
    // memory read of the stage, so this warp's reads are complete.
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

// ---------------------------------------------------------------------------------------------------------------
// Prefill attention's dequantize pass: K rows decoded and rotated back (H256 / 16 is its own inverse), so the chunk's
// query needs no rotation and the tensor-core kernel of the other formats runs unchanged; V tiles transposed to
// token-major with the per-channel affine applied, the tile of the newest key from the open fp16 buffer.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kDequantThreads = 256;
__global__ void __launch_bounds__(kDequantThreads)
    Kv4DequantPagesKernel(PoolView pool, int layer, int n_layers, const std::int32_t* __restrict__ tables,
                          int table_stride, const PrefillSeq* __restrict__ seqs, const __half* __restrict__ open_tiles,
                          __half* __restrict__ k16, __half* __restrict__ v16) {
  const PrefillSeq ps = seqs[blockIdx.z];
  const int p = blockIdx.x, kvh = blockIdx.y;
  if (p >= ps.n_pages || !pool.OwnsKvHead(kvh)) return;
  std::int32_t page = __ldg(tables + static_cast<std::size_t>(ps.seq) * table_stride + p);
  page = min(max(page, 0), pool.num_pages - 1);
  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + page) * kKvHeads + kvh;
  const std::size_t out_row0 = static_cast<std::size_t>(ps.kv_row0) + static_cast<std::size_t>(kvh) * ps.kv_rows +
                               static_cast<std::size_t>(p) * kPageTokens;
  {   // K: a warp per token row; lane l holds dword l = dims 8 l .. 8 l + 7 of the rotated row
    const std::uint8_t* codes = pool.kcodes + rec * RecordCodeBytes(kFmtKv4);
    const std::uint16_t* scales = pool.kscales + rec * (RecordScaleBytes(kFmtKv4, 0) / 2);
    __half* out = k16 + out_row0 * kHeadDim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int tok = warp; tok < kPageTokens; tok += kDequantThreads / 32) {
      const std::uint32_t w = *reinterpret_cast<const std::uint32_t*>(codes + tok * 128 + lane * 4);
      const std::uint32_t pw = *reinterpret_cast<const std::uint32_t*>(scales + tok * 16 + (lane >> 2) * 2);
      const float2 pr = __half22float2(*reinterpret_cast<const __half2*>(&pw));
      const float a = pr.x * 0.0625F, b = pr.y + pr.x;
      float x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = fmaf(static_cast<float>((w >> NibbleShift(i)) & 15U), a, b);
      Hadamard256(x, lane);
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
      *reinterpret_cast<uint4*>(out + static_cast<std::size_t>(tok) * kHeadDim + lane * 8) = o;
    }
  }
  {   // V: thread -> two neighbouring channels of one tile (16 keys each), written as one half2 per key
    const std::uint8_t* codes = pool.vcodes + rec * RecordCodeBytes(kFmtKv4);
    const std::uint16_t* stats = pool.vscales + rec * (RecordScaleBytes(kFmtKv4, 1) / 2);
    const int open_tile = (ps.kv_len - 1) / kTileKeys;
    const __half* open_buf = open_tiles + ((static_cast<std::size_t>(ps.seq) * n_layers + layer) * 2 + (ps.pad[0] & 1)) * kOpenTileHalfs +
                             static_cast<std::size_t>(kvh) * kHeadDim * kTileKeys;
    __half* out = v16 + out_row0 * kHeadDim;
    for (int w = threadIdx.x; w < kTilesPerPage * (kHeadDim / 2); w += kDequantThreads) {
      const int tl = w / (kHeadDim / 2), ch = (w % (kHeadDim / 2)) * 2;
      const int tile = p * kTilesPerPage + tl;
      float val[2][kTileKeys];
      if (tile == open_tile) {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const uint4* src = reinterpret_cast<const uint4*>(open_buf + (ch + x) * kTileKeys);
          const uint4 a = src[0], b = src[1];
          const __half2* ha = reinterpret_cast<const __half2*>(&a);
          const __half2* hb = reinterpret_cast<const __half2*>(&b);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 fa = __half22float2(ha[i]), fb = __half22float2(hb[i]);
            val[x][2 * i] = fa.x, val[x][2 * i + 1] = fa.y;
            val[x][8 + 2 * i] = fb.x, val[x][8 + 2 * i + 1] = fb.y;
          }
        }
      } else {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const uint2 c = *reinterpret_cast<const uint2*>(codes + (static_cast<std::size_t>(tl) * kHeadDim + ch + x) * 8);
          const std::uint32_t st = *reinterpret_cast<const std::uint32_t*>(stats + (static_cast<std::size_t>(tl) * kHeadDim + ch + x) * 2);
          const float2 pr = __half22float2(*reinterpret_cast<const __half2*>(&st));
          const float a = pr.x * 0.0625F, b = pr.x + pr.y;
          const std::uint32_t cw[2] = {c.x, c.y};
#pragma unroll
          for (int d = 0; d < 2; ++d)
#pragma unroll
            for (int n = 0; n < 8; ++n) {   // nibble n of dword d = key 8d + 2n (n < 4) or 8d + 2(n - 4) + 1
              const int key = 8 * d + (n < 4 ? 2 * n : 2 * (n - 4) + 1);
              val[x][key] = fmaf(a, static_cast<float>((cw[d] >> (4 * n)) & 15U), b);
            }
        }
      }
#pragma unroll
      for (int k = 0; k < kTileKeys; ++k)
        *reinterpret_cast<__half2*>(out + static_cast<std::size_t>(tl * kTileKeys + k) * kHeadDim + ch) =
            __floats2half2_rn(val[0][k], val[1][k]);
    }
  }
}

}  // namespace

cudaError_t ConfigureKv4Kernels() {
  cudaError_t e = cudaFuncSetAttribute(Kv4DecodePartKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(Kv4DecodePartKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

cudaError_t LaunchKv4AppendK(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                             const std::int32_t* state_rows_dev, int state_row_add, const float* kmean_dev,
                             const void* k_dev, cudaStream_t stream) {
  if (n_tokens <= 0) return cudaSuccess;
  return LaunchChained(Kv4AppendKKernel, n_tokens, 128, 0, stream, pool, layer, slots_dev, state_rows_dev, state_row_add,
                       kmean_dev, static_cast<const __half*>(k_dev));
}

cudaError_t LaunchKv4DecodePart(const DecodeLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream) {
  if (a.n_units <= 0 || a.n_seqs <= 0) return cudaSuccess;
  const auto* open16 = static_cast<const __half*>(open_tiles_dev);
  if (a.q_raw) {
    const QueryRaw qr{static_cast<const float*>(a.q_dev), a.q_weight_dev, a.rope_tab_dev, a.q_eps, a.rope_rows};
    return LaunchChained(Kv4DecodePartKernel<true>, a.n_units, kThreads, kSmemBytes, stream, *a.kmap, a.pool, a.layer,
                         a.tables_dev, a.table_stride, a.units_dev, static_cast<const __half*>(nullptr), qr, a.scale_log2,
                         open16, n_layers, a.partial_acc, a.partial_ml, a.status_dev);
  }
  return LaunchChained(Kv4DecodePartKernel<false>, a.n_units, kThreads, kSmemBytes, stream, *a.kmap, a.pool, a.layer,
                       a.tables_dev, a.table_stride, a.units_dev, static_cast<const __half*>(a.q_dev), QueryRaw{},
                       a.scale_log2, open16, n_layers, a.partial_acc, a.partial_ml, a.status_dev);
}

cudaError_t LaunchKv4PrefillDequant(const PrefillLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream) {
  if (a.n_seqs <= 0 || a.max_pages <= 0) return cudaSuccess;
  const dim3 grid(static_cast<unsigned>(a.max_pages), kKvHeads, static_cast<unsigned>(a.n_seqs));
  Kv4DequantPagesKernel<<<grid, kDequantThreads, 0, stream>>>(a.pool, a.layer, n_layers, a.tables_dev, a.table_stride,
                                                             a.seqs_dev, static_cast<const __half*>(open_tiles_dev),
                                                             static_cast<__half*>(a.k16_dev), static_cast<__half*>(a.v16_dev));
  return cudaGetLastError();
}

}  // namespace yahkv
