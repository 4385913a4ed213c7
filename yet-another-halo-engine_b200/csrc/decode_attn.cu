// Paged split-K decode attention over the quantized cache, and its combine pass.
//
// Stands in for the reference's dattn_part / dattn_part_q (one workgroup per kv head and page, partial softmax and
// P.V) and dattn_reduce (merge, divide, sigmoid gate): engine/gpu/loom/tools/gen_decode_attn.py:97-335, :576-1040,
// :338-411. Numeric contract kept from there: keys 0 .. len-1 visible, invalid keys get weight 0, score = q.k * scale,
// fp32 softmax statistics, partials (max, sum, unnormalised acc) merged in unit order, out = A / L * sigmoid(gate).
//
// Shape of the work. One CTA processes one split-K unit: a run of pages of one sequence for one kv head, all six query
// heads of the GQA group at once, so every cache byte is read from HBM exactly once per call. Each page's K and V
// records are gathered through the block table with non-multicast TMA: two 2-D tiled copies per side (64 token rows
// x 128 B, 128-byte swizzle, so the ldmatrix reads below are bank-conflict free) plus one bulk copy per side for the
// 64 x 8 fp16 scales, all completing on one mbarrier per ring stage. There is no producer warp: whichever warp
// finishes a stage last refills it, so no warp waits for another.
//
// Eight warps work on two pages at a time: warp w owns key group w % 4 (16 keys) of the pages whose index in the unit
// has parity w / 4, and for those keys it does everything: scores over all 256 dims, softmax, and all 256 output
// dims (64 accumulator registers). No warp ever exchanges anything with another one inside the page loop: per page
// there is one wait, one softmax per key group and no barrier, which is what keeps the number of instructions issued
// per cached byte low enough for q4_0 as well (an earlier layout split the head dimension over warp pairs: half the
// accumulators per thread, but two barriers, an exchange through shared memory and a duplicated softmax per page).
//
// The path is HBM-bound (2176 B per token per layer in q8_0), but at GQA 6 it needs 5.6 multiply-adds per byte, more
// than the fp32 pipes can give at HBM rate, so the dot products run on the warp-level tensor-core MMA with register
// operands, and what limits the kernel next is the number of instructions issued per byte. The two products are
// treated differently for that reason:
//   Q.K^T runs on the integer MMA (m16n8k32, s8 x s8 -> s32) straight on the cached codes: a 32-element block is
//   exactly one k-step, ldmatrix delivers the code bytes in the B operand's register layout, and nothing is converted
//   (q4_0: three logic instructions turn eight nibbles into the signed bytes 16 (n - 8): the nibble moved to the top of
//   its byte and the byte's sign bit flipped, so the format's offset costs nothing). The query row is quantized
//   once per CTA to 16 bits against its head's largest magnitude and split into two int8 planes, hi and lo
//   (q = s (256 hi + lo), |error| <= s / 2 = amax / 64000 per element, far below the fp16 query's own spacing).
//   Both planes ride in one MMA as rows 0-5 and 8-13 of the 16-row A operand, so one instruction gives the exact
//   block sums of both; they are joined in integers, converted once, and multiplied by the block's fp16 scale in
//   fp32.
//   P.V stays on the f16 MMA: V codes become exact f16 integers by a byte permute and a magic-number subtract, and
//   the per-(key, block) V scale is folded into the weights, which are split into an f16 high and low part (two
//   MMAs) so the weights keep ~22 bits: a single f16 weight would cost up to 3e-3 absolute error on outlier channels.
//
// MMA orientation. S^T[head][key] = Q[head][dim] . K[key][dim]: A = Q (hi and lo planes of the six heads), B = K^T
// read with ldmatrix straight from the token-major page. O^T[dim][head] = V^T[dim][key] . P^T[key][head]: A = V^T read
// with ldmatrix.trans from the same token-major layout, B = the weights, which the first MMA left in exactly the
// register layout the second one wants. The dims inside a 16-wide step of the second MMA are a fixed permutation of
// the page's dims, undone when the accumulators are written out.
#include <cuda_fp16.h>

#include <cmath>

#include "decode_ring.cuh"
#include "qrope.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

namespace yahkv {
namespace {

// The shape of a CTA per format: page sets (pages in work at a time; warp w takes the pages i with
// i % kPageSets = w / 4), ring stages (a stage = one page of one kv head: 34 KB q8_0, 18 KB q4_0) and resident CTAs per
// SM. q8_0 is bound by memory: two sets of four warps on a three-stage ring, two CTAs per SM. q4_0 is bound by
// instruction latency, and more, smaller CTAs overlap their prologues and merges better: one set of four warps on a
// two-stage ring, four CTAs per SM (measured on 8 x 131072 tokens: 275 us per layer against 295 with the q8_0 shape;
// three CTAs with three stages 283, three CTAs with four stages 342).
#ifndef YAHKV_Q8_PAGE_SETS
#define YAHKV_Q8_PAGE_SETS 2
#endif
#ifndef YAHKV_Q8_STAGES
#define YAHKV_Q8_STAGES 3
#endif
#ifndef YAHKV_Q8_CTAS
#define YAHKV_Q8_CTAS 2
#endif
#ifndef YAHKV_Q4_PAGE_SETS
#define YAHKV_Q4_PAGE_SETS 1
#endif
#ifndef YAHKV_Q4_STAGES
#define YAHKV_Q4_STAGES 2
#endif
#ifndef YAHKV_Q4_CTAS
#define YAHKV_Q4_CTAS 4
#endif
constexpr int kKeyGroups = 4;              // 16 keys of a page each
template <int kFmt>
struct Shape {
  static constexpr int kPageSets = kFmt == kFmtQ8 ? YAHKV_Q8_PAGE_SETS : YAHKV_Q4_PAGE_SETS;
  static constexpr int kCtas = kFmt == kFmtQ8 ? YAHKV_Q8_CTAS : YAHKV_Q4_CTAS;
  static constexpr int kWarps = kPageSets * kKeyGroups;
  static constexpr int kThreads = kWarps * 32;
};
constexpr int kBoxBytes = 64 * 128;        // one swizzled TMA box: 64 token rows x 128 B

template <int kFmt>
struct StageLayout {
  static constexpr int kBoxesPerSide = kFmt == kFmtQ8 ? 2 : 1;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kBoxesPerSide * kBoxBytes;
  static constexpr int kKsOff = 2 * kBoxesPerSide * kBoxBytes;
  static constexpr int kVsOff = kKsOff + kRecordScaleBytes;
  static constexpr int kBytes = kVsOff + kRecordScaleBytes;  // 34816 (q8_0) or 18432 (q4_0), a multiple of 1024
  static constexpr int kStages = kFmt == kFmtQ8 ? YAHKV_Q8_STAGES : YAHKV_Q4_STAGES;
};

// fp16 number i (0..3) of four packed in a uint2, widened to f32. i is a compile-time constant after unrolling.
__device__ __forceinline__ float ScaleOf(const uint2& v, int i) {
  const std::uint32_t w = i < 2 ? v.x : v.y;
  const __half2 h = *reinterpret_cast<const __half2*>(&w);
  return (i & 1) ? __high2float(h) : __low2float(h);
}

// One S^T step on the integer tensor pipe: D(16 x 8, s32) = A(16 x 32, s8) . B(32 x 8, s8), accumulator input zero.
// A = the query planes of one 32-element block (LoadQ: one 16-byte load from shared memory at use, shared by the two
// key tiles of the block); B = the code bytes of eight keys as ldmatrix left them.
__device__ __forceinline__ void LoadQ(std::uint32_t (&a)[4], std::uint32_t q_addr) {
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(q_addr));
}
__device__ __forceinline__ void MmaQK(int (&d)[4], const std::uint32_t (&a)[4], std::uint32_t b0, std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
// The block sum of one (head, key): the hi plane's sum times 256 plus the lo plane's, exact in 32 bits
// (|sum| <= 32 x 128 x 32768), as a float.
__device__ __forceinline__ float JoinPlanes(int hi, int lo) { return static_cast<float>(hi * 256 + lo); }

// Query quantization: 16 bits against the head's largest magnitude. 32000 keeps the hi plane inside [-125, 125].
constexpr float kQSteps = 32000.0F;

// Shared memory of a CTA, all dynamic so that the ring starts at the window's 1024-byte aligned base (the swizzled
// TMA boxes need that alignment): ring | Q operands | mbarriers | stage counters | query steps | abort flag.
// Lanes 24-31 of a warp hold the two padding heads of the 8-wide MMA; they reuse the Q operands of lanes 16-23
// (duplicates of heads 4, 5 whose results are never stored), so the Q array is 24 lanes wide.
constexpr int kQLanes = 24;
constexpr int kQfragBytes = kBlocksPerRow * kQLanes * 16;   // per 32-element block the A operand's four registers
template <int kFmt>
struct SmemLayout {
  static constexpr int kRing = StageLayout<kFmt>::kStages * StageLayout<kFmt>::kBytes;
  static_assert(kRing >= Shape<kFmt>::kWarps * kDecodeMergeWarpFloats * 4, "the merge scratch of a unit's end aliases the ring");
  static constexpr int kQfragOff = kRing;
  static constexpr int kBarOff = kQfragOff + kQfragBytes;
  static constexpr int kCntOff = kBarOff + 8 * StageLayout<kFmt>::kStages;
  static constexpr int kFillOff = kCntOff + 4 * StageLayout<kFmt>::kStages;     // fills issued per stage
  static constexpr int kQScaleOff = kFillOff + 4 * StageLayout<kFmt>::kStages;  // [8] f32, one per head (6 used)
  static constexpr int kAbortOff = kQScaleOff + 4 * 8;
  static constexpr int kBytes = kAbortOff + 4;
};
template <int kFmt>
constexpr int DecodeSmemBytes() {
  return (SmemLayout<kFmt>::kBytes + 127) / 128 * 128;
}
constexpr int kStatusSmemMisaligned = 2;

// Running max may lag the true max by this much (log2 units) before the accumulators are rescaled; weights stay
// <= 2^4, so weight x scale fits fp16 for every representable fp16 input.
constexpr float kLazyRescale = 4.0F;

// kQRaw: the query is the raw f32 projection (qraw) and the prologue norms and rotates the unit's six head rows itself,
// at the position of the sequence's newest key (qrope.cuh).
template <int kFmt, bool kQRaw>
__global__ void __launch_bounds__(Shape<kFmt>::kThreads, Shape<kFmt>::kCtas)
    DecodePartKernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                     PoolView pool, int layer, const std::int32_t* __restrict__ tables, int table_stride,
                     const DecodeUnit* __restrict__ units, const __half* __restrict__ q, const QueryRaw qraw,
                     float scale_log2, float* __restrict__ partial_acc, float* __restrict__ partial_ml, int* status) {
  ChainedKernelEntry();
  using L = StageLayout<kFmt>;
  using S = SmemLayout<kFmt>;
  constexpr int kPageSets = Shape<kFmt>::kPageSets, kWarps = Shape<kFmt>::kWarps;
  extern __shared__ __align__(1024) std::uint8_t smem_raw[];
  std::uint8_t* ring = smem_raw;
  std::uint32_t* qfrag = reinterpret_cast<std::uint32_t*>(smem_raw + S::kQfragOff);   // [8 blocks][24 lanes][4]
  std::uint64_t* full_bar = reinterpret_cast<std::uint64_t*>(smem_raw + S::kBarOff);
  int* done_cnt = reinterpret_cast<int*>(smem_raw + S::kCntOff);        // warps done reading a stage's page
  int* fill_cnt = reinterpret_cast<int*>(smem_raw + S::kFillOff);       // fills issued to a stage so far
  float* q_scale = reinterpret_cast<float*>(smem_raw + S::kQScaleOff);  // query quantization step per head
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + S::kAbortOff);   // a wait gave up
  if ((SmemAddr(smem_raw) & 1023U) != 0) {   // never seen; checked because a misaligned swizzle would corrupt results
    if (threadIdx.x == 0) atomicExch(status, kStatusSmemMisaligned);
    return;
  }

  const DecodeUnit u = units[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kw = warp & (kKeyGroups - 1);   // key group: keys 16 kw .. 16 kw + 15 of a page
  const int par = warp / kKeyGroups;        // this warp's pages: index par, par + 2, ... of the unit
  const int n_pages = u.page_end - u.page_begin;
  if (n_pages <= 0) return;   // a unit reserved for growth that holds no page yet: the merge does not count it
  const std::int32_t* row = tables + static_cast<std::size_t>(u.seq) * table_stride + u.page_begin;

  // Gather of one page into a ring stage: 2 TMA boxes per side (q8_0; 1 for q4_0) + the two scale records, all
  // completing on the stage's mbarrier. Called by a whole converged warp with warp-uniform arguments; one elected
  // lane issues (asynchronous copies issued from inside a single-lane branch cost several times more issue time).
  // Once any warp has given up a wait nothing more is fetched: the CTA is on its way out and must not leave copies
  // in flight behind it.
  auto issue = [&](int s, std::int32_t page) {
    if (*abort_flag != 0) return;
    page = min(max(page, 0), pool.num_pages - 1);   // never trust a table entry read from memory
    const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + page) * kKvHeads + u.kvh;
    const int y = static_cast<int>(rec * kPageTokens);
    std::uint8_t* st = ring + s * L::kBytes;
    if (ElectOne()) {
      fill_cnt[s] += 1;
      MbarArriveExpectTx(&full_bar[s], L::kBytes);
#pragma unroll
      for (int b = 0; b < L::kBoxesPerSide; ++b) {
        TmaLoad2D(st + L::kKOff + b * kBoxBytes, &kmap, b * 128, y, &full_bar[s]);
        TmaLoad2D(st + L::kVOff + b * kBoxBytes, &vmap, b * 128, y, &full_bar[s]);
      }
      BulkLoad(st + L::kKsOff, pool.kscales + rec * (kPageTokens * kBlocksPerRow), kRecordScaleBytes, &full_bar[s]);
      BulkLoad(st + L::kVsOff, pool.vscales + rec * (kPageTokens * kBlocksPerRow), kRecordScaleBytes, &full_bar[s]);
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      PrefetchTensorMap(&kmap);
      PrefetchTensorMap(&vmap);
      for (int s = 0; s < L::kStages; ++s) {
        MbarInit(&full_bar[s], 1);
        done_cnt[s] = 0;
        fill_cnt[s] = 0;
      }
      *abort_flag = 0;
      FenceBarrierInit();
    }
    __syncwarp();
    for (int i = 0; i < L::kStages && i < n_pages; ++i) issue(i, __ldg(row + i));
  }

  const int t = lane & 3;
  // Query planes through shared memory. Warp h < 6 quantizes head h of the group: lane l holds dims 8 l .. 8 l + 7
  // (block l / 4, elements 8 (l % 4) .. + 7 of it). q16 = rint(q * 32000 / amax), hi = (q16 + 128) >> 8,
  // lo = q16 - 256 hi in [-128, 127]. The A operand of block b for lane (g = head, t) is four registers:
  //   a0 = hi of elements 4t .. 4t+3, a1 = lo of the same, a2 = hi of elements 16+4t .. 16+4t+3, a3 = lo of those,
  // so that rows 0-5 of the MMA are the hi plane and rows 8-13 the lo plane of the six heads.
  for (int hq = warp; hq < kGroup; hq += kWarps) {   // one head per warp (per pass, in a CTA of fewer than six warps)
    const uint4 raw = LoadQueryLane8<kQRaw>(q, qraw, static_cast<std::size_t>(u.batch) * kQHeads + u.kvh * kGroup + hq,
                                            u.n_keys - 1, lane);
    const __half2* hp = reinterpret_cast<const __half2*>(&raw);
    float x[8];
    float amax = 0.0F;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(hp[i]);
      x[2 * i] = f.x, x[2 * i + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFU, amax, o));
    const float inv = amax > 0.0F ? kQSteps / amax : 0.0F;
    std::uint32_t hi_w[2] = {0, 0}, lo_w[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q16 = __float2int_rn(x[i] * inv);
      const int hi = (q16 + 128) >> 8;
      const int lo = q16 - hi * 256;
      hi_w[i >> 2] |= (static_cast<std::uint32_t>(hi) & 0xFFU) << (8 * (i & 3));
      lo_w[i >> 2] |= (static_cast<std::uint32_t>(lo) & 0xFFU) << (8 * (i & 3));
    }
    const int blk = lane >> 2, e0 = (lane & 3) * 8;
    const int reg = e0 < 16 ? 0 : 2, t0 = (e0 & 15) >> 2;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      std::uint32_t* dst = qfrag + ((blk * kQLanes + hq * 4 + t0 + j) << 2) + reg;
      dst[0] = hi_w[j];
      dst[1] = lo_w[j];
    }
    // q = step (256 hi + lo); q4_0 codes enter the MMA as 16 (n - 8), which the step absorbs
    if (lane == 0) q_scale[hq] = (amax / kQSteps) * (kFmt == kFmtQ8 ? 1.0F : 0.0625F);
  }
  __syncthreads();   // barriers initialised, query planes visible
  const int qlane = lane < kQLanes ? lane : lane - 8;
  const std::uint32_t qa_addr = SmemAddr(qfrag + (qlane << 2));   // block b: + b * kQLanes * 16 bytes
  const float score_scale = scale_log2 * q_scale[qlane >> 2];     // softmax scale x log2(e) x the head's query step

  float o_acc[16][4];   // tile c = dims 16 c .. 16 c + 15 (in the MMA's permuted order)
#pragma unroll
  for (int c = 0; c < 16; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[c][i] = 0.0F;
  float m_run = -INFINITY, l_run = 0.0F;
  bool alive = true;

  // ldmatrix row addresses: lane supplies row (lane & 7) + 8 * ((lane >> 3) & 1) of the key group's 16 keys and the
  // 16-byte chunk 2x + (lane >> 4) of its 128-byte row, swizzled: physical chunk = chunk ^ (row & 7).
  // Chunk pair x differs from pair 0 in address bits 5-6 only, and the swizzle is an xor, so pair x's offset is pair
  // 0's xor (x << 5). q8_0 keeps one register and pays the xor at each use; q4_0, whose page loop has no slack on the
  // logic pipe or on the address path of its ldmatrix reads, keeps the four offsets in registers (measured: 391 us per
  // launch of the long-context workload with the xor, 323 us with the registers; q8_0 201 against 204 us).
  const int lm_key = kw * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const std::uint32_t lm0 = lm_key * 128 + (((lane >> 4) ^ (lm_key & 7)) << 4);
  std::uint32_t lm_arr[4];
#pragma unroll
  for (int x = 0; x < 4; ++x) lm_arr[x] = lm_key * 128 + ((((2 * x) | (lane >> 4)) ^ (lm_key & 7)) << 4);
  auto lm_off = [&](int x) -> std::uint32_t {
    if constexpr (kFmt == kFmtQ4) {
      return lm_arr[x];
    } else {
      return lm0 ^ (static_cast<std::uint32_t>(x) << 5);
    }
  };
  // Keys whose scores this thread holds: kt * 8 + 2t + j of the group's 16.
  const int my_key0 = kw * 16 + 2 * t;

  NibConsts nib{};
  if constexpr (kFmt == kFmtQ4) nib.Load();
  static_assert(kPageSets <= L::kStages, "the stage counter below wraps at most once per step");
  for (int i = par; i < n_pages; i += kPageSets) {
    const int s = i % L::kStages;    // ring stage of page i
    const int gen = i / L::kStages;  // fills of that stage before this page's
    // Table entry of the page that will take this stage next, fetched a whole iteration before it is needed.
    std::int32_t refill_page = 0;
    if (lane == 0 && i + L::kStages < n_pages) refill_page = __ldg(row + i + L::kStages);
    alive = RingWait(alive, fill_cnt + s, &full_bar[s], gen, abort_flag);
    const std::uint8_t* st = ring + s * L::kBytes;
    const std::uint32_t k_base = SmemAddr(st + L::kKOff), v_base = SmemAddr(st + L::kVOff);

    // ---- S^T = Q K^T: per 32-element block the exact integer sums of the two query planes, joined, converted once,
    // times the block's fp16 scale ----
    float sc[2][2] = {{0.0F, 0.0F}, {0.0F, 0.0F}};
#pragma unroll
    for (int dh = 0; dh < 2; ++dh) {   // blocks 4 dh .. 4 dh + 3 (scales fetched per half to keep registers low)
      uint2 ks_raw[2][2];
#pragma unroll
      for (int kt = 0; kt < 2; ++kt)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          ks_raw[kt][j] = *reinterpret_cast<const uint2*>(st + L::kKsOff + (my_key0 + kt * 8 + j) * 16 + dh * 8);
      if constexpr (kFmt == kFmtQ8) {
        // One ldmatrix.x4 = one block of 16 keys: registers 0 / 2 are the two 16-byte halves of keys 0-7 (the B
        // operand's k 0-15 and 16-31), registers 1 / 3 those of keys 8-15. Dim half dh is TMA box dh.
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          std::uint32_t w[4], qa[4];
          LdMatrixX4(k_base + dh * kBoxBytes + lm_off(b), w);
          LoadQ(qa, qa_addr + (4 * dh + b) * (kQLanes * 16));
          int a0[4], a1[4];
          MmaQK(a0, qa, w[0], w[2]);
          MmaQK(a1, qa, w[1], w[3]);
          sc[0][0] = fmaf(ScaleOf(ks_raw[0][0], b), JoinPlanes(a0[0], a0[2]), sc[0][0]);
          sc[0][1] = fmaf(ScaleOf(ks_raw[0][1], b), JoinPlanes(a0[1], a0[3]), sc[0][1]);
          sc[1][0] = fmaf(ScaleOf(ks_raw[1][0], b), JoinPlanes(a1[0], a1[2]), sc[1][0]);
          sc[1][1] = fmaf(ScaleOf(ks_raw[1][1], b), JoinPlanes(a1[1], a1[3]), sc[1][1]);
        }
      } else {
        // One ldmatrix.x4 covers two 16-byte blocks of 16 keys; a thread's word is bytes 4t .. 4t+3 of a block, i.e.
        // elements 4t .. 4t+3 in the low nibbles (k 4t ..) and 16+4t .. in the high ones (k 16+4t ..).
#pragma unroll
        for (int bp = 0; bp < 2; ++bp) {
          std::uint32_t w[4];
          LdMatrixX4(k_base + lm_off(2 * dh + bp), w);
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const int b = 2 * bp + hb;   // block 4 dh + b
            std::uint32_t qa[4];
            LoadQ(qa, qa_addr + (4 * dh + b) * (kQLanes * 16));
            int a0[4], a1[4];
            std::uint32_t lo, hi;
            Nib8ToS8(nib.top_mask, nib.sign_flip, w[2 * hb], lo, hi);
            MmaQK(a0, qa, lo, hi);
            Nib8ToS8(nib.top_mask, nib.sign_flip, w[2 * hb + 1], lo, hi);
            MmaQK(a1, qa, lo, hi);
            sc[0][0] = fmaf(ScaleOf(ks_raw[0][0], b), JoinPlanes(a0[0], a0[2]), sc[0][0]);
            sc[0][1] = fmaf(ScaleOf(ks_raw[0][1], b), JoinPlanes(a0[1], a0[3]), sc[0][1]);
            sc[1][0] = fmaf(ScaleOf(ks_raw[1][0], b), JoinPlanes(a1[0], a1[2]), sc[1][0]);
            sc[1][1] = fmaf(ScaleOf(ks_raw[1][1], b), JoinPlanes(a1[1], a1[3]), sc[1][1]);
          }
        }
      }
    }

    // ---- softmax statistics (per head g, the 16 keys spread over the four lanes of a quad) ----
    float tmax = -INFINITY;
#pragma unroll
    for (int kt = 0; kt < 2; ++kt)
#pragma unroll
      for (int j = 0; j < 2; ++j) sc[kt][j] *= score_scale;
    if ((u.page_begin + i + 1) * kPageTokens > u.n_keys) {   // only ever true on a sequence's last page
      const int key_pos0 = (u.page_begin + i) * kPageTokens + my_key0;
#pragma unroll
      for (int kt = 0; kt < 2; ++kt)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (key_pos0 + kt * 8 + j >= u.n_keys) sc[kt][j] = -INFINITY;
    }
    tmax = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFU, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFU, tmax, 2));
    // Only the six real heads vote: the padding lanes hold duplicates.
    if (__any_sync(0xFFFFFFFFU, lane < kQLanes && tmax > m_run + kLazyRescale)) {
      const float m_new = fmaxf(m_run, tmax);
      const float alpha = m_new == -INFINITY ? 1.0F : Exp2Fast(m_run - m_new);  // m_run = -inf gives 0
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
    // Weights as an fp16 high part plus an fp16 residual (22 bits together), one half2 per key pair.
    __half2 p_hi[2], p_lo[2];
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) {
      const float p0 = Exp2Fast(sc[kt][0] - m_use), p1 = Exp2Fast(sc[kt][1] - m_use);
      l_run += p0 + p1;
      p_hi[kt] = __floats2half2_rn(p0, p1);
      const float2 hf = __half22float2(p_hi[kt]);
      p_lo[kt] = __floats2half2_rn(p0 - hf.x, p1 - hf.y);
    }

    // ---- O^T += V^T P^T, the V scale of (key, block) folded into the weights ----
#pragma unroll
    for (int dh = 0; dh < 2; ++dh) {
      uint2 vs_raw[2][2];
#pragma unroll
      for (int kt = 0; kt < 2; ++kt)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          vs_raw[kt][j] = *reinterpret_cast<const uint2*>(st + L::kVsOff + (my_key0 + kt * 8 + j) * 16 + dh * 8);
      // weight x scale without leaving fp16: hi = round(p_hi d); the rounding error of that product is recovered
      // exactly by an fma and joins the low part: lo = p_lo d + (p_hi d - hi).
      auto weights = [&](int b, std::uint32_t (&hi)[2], std::uint32_t (&lo)[2]) {
#pragma unroll
        for (int kt = 0; kt < 2; ++kt) {
          const std::uint32_t w0 = b < 2 ? vs_raw[kt][0].x : vs_raw[kt][0].y;
          const std::uint32_t w1 = b < 2 ? vs_raw[kt][1].x : vs_raw[kt][1].y;
          const std::uint32_t dw = __byte_perm(w0, w1, (b & 1) ? 0x7632 : 0x5410);
          const __half2 d2 = *reinterpret_cast<const __half2*>(&dw);
          const __half2 h = __hmul2(p_hi[kt], d2);
          const __half2 r = __hfma2(p_hi[kt], d2, __hneg2(h));
          const __half2 l = __hfma2(p_lo[kt], d2, r);
          hi[kt] = *reinterpret_cast<const std::uint32_t*>(&h);
          lo[kt] = *reinterpret_cast<const std::uint32_t*>(&l);
        }
      };
      if constexpr (kFmt == kFmtQ8) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          std::uint32_t hi[2], lo[2];
          weights(b, hi, lo);
          std::uint32_t w[4];
          LdMatrixX4Trans(v_base + dh * kBoxBytes + lm_off(b), w);
          std::uint32_t a0, a1, a2, a3;
          Offset8x4ToHalf2(w[0], a0, a1);
          Offset8x4ToHalf2(w[1], a2, a3);
          MmaF16(o_acc[8 * dh + 2 * b], a0, a1, a2, a3, hi[0], hi[1]);
          MmaF16(o_acc[8 * dh + 2 * b], a0, a1, a2, a3, lo[0], lo[1]);
          Offset8x4ToHalf2(w[2], a0, a1);
          Offset8x4ToHalf2(w[3], a2, a3);
          MmaF16(o_acc[8 * dh + 2 * b + 1], a0, a1, a2, a3, hi[0], hi[1]);
          MmaF16(o_acc[8 * dh + 2 * b + 1], a0, a1, a2, a3, lo[0], lo[1]);
        }
      } else {
#pragma unroll
        for (int bp = 0; bp < 2; ++bp) {
          std::uint32_t w[4];
          LdMatrixX4Trans(v_base + lm_off(2 * dh + bp), w);
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const int b = 2 * bp + hb;
            std::uint32_t hi[2], lo[2];
            weights(b, hi, lo);
            std::uint32_t la0, la1, ha0, ha1, la2, la3, ha2, ha3;
            Nib4x4ToHalf2(nib, w[2 * hb], la0, la1, ha0, ha1);      // keys 0-7 of the group's 16
            Nib4x4ToHalf2(nib, w[2 * hb + 1], la2, la3, ha2, ha3);  // keys 8-15
            MmaF16(o_acc[8 * dh + 2 * b], la0, la1, la2, la3, hi[0], hi[1]);
            MmaF16(o_acc[8 * dh + 2 * b], la0, la1, la2, la3, lo[0], lo[1]);
            MmaF16(o_acc[8 * dh + 2 * b + 1], ha0, ha1, ha2, ha3, hi[0], hi[1]);
            MmaF16(o_acc[8 * dh + 2 * b + 1], ha0, ha1, ha2, ha3, lo[0], lo[1]);
          }
        }
      }
    }

    // The last of the page's four warps to finish with the stage refills it (no warp ever waits for another one).
    const bool last = RingRelease(&done_cnt[s], lane, kKeyGroups);
    if (last && i + L::kStages < n_pages) issue(s, __shfl_sync(0xFFFFFFFFU, refill_page, 0));
  }
  if (!alive && lane == 0) atomicExch(status, kStatusWaitTimeout);
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 1);
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 2);

  // Every stage has been consumed (or a wait gave up): the ring is free to hold the merge scratch.
  __syncthreads();
  RingDrainAfterAbort(abort_flag, fill_cnt, full_bar, L::kStages);
  MergeUnitAndStore<kWarps, true>(reinterpret_cast<float*>(ring), o_acc, m_run, l_run, warp, lane,
                                  partial_acc + static_cast<std::size_t>(u.partial) * kPartialAccFloats,
                                  partial_ml + static_cast<std::size_t>(u.partial) * kPartialMlFloats);
}

// Merge the units of one (batch row, query head): out = (sum w_i acc_i) / (sum w_i l_i) * sigmoid(gate) with
// w_i = 2^(m_i - M), accumulated in unit order (engine/gpu/loom/tools/gen_decode_attn.py:373-408). One CTA per head,
// thread = output dim. The merge is latency-bound, so the weights are prepared in shared memory first and the loads
// of the weighted sum are all independent of each other.
constexpr int kCombineEarly = 32;   // partial rows fetched before their weights are known
__global__ void __launch_bounds__(kHeadDim)
    DecodeCombineKernel(const CombineItem* __restrict__ items, const float* __restrict__ partial_acc,
                        const float* __restrict__ partial_ml, const float* __restrict__ gate, void* out, int out_f32) {
  __shared__ float m_s[kCombineMaxUnits], w_s[kCombineMaxUnits], l_s[kCombineMaxUnits];
  __shared__ float red_s[kHeadDim / 32];
  __shared__ float inv_l;
  ChainedKernelEntry();
  const int b = blockIdx.x / kQHeads, hh = blockIdx.x % kQHeads;
  const int kvh = hh / kGroup, j = hh % kGroup;
  const CombineItem it = items[b * kKvHeads + kvh];
  const int n = min(it.n_partials, kCombineMaxUnits);   // the planner never exceeds it
  if (n <= 0) return;   // a kv head outside the context's range: its query heads' rows belong to another context
  const float* ml_g = partial_ml + static_cast<std::size_t>(it.first_partial) * kPartialMlFloats + 2 * j;
  const float* acc_g = partial_acc + static_cast<std::size_t>(it.first_partial) * kPartialAccFloats + j * kHeadDim + threadIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // The merge is a chain of dependent global loads (max, weights, weighted sum), so the first rows of the weighted
  // sum are fetched up front, together with the (max, sum) pairs, and only multiplied once the weights exist.
  float early[kCombineEarly];
#pragma unroll
  for (int i = 0; i < kCombineEarly; ++i)
    early[i] = i < n ? acc_g[static_cast<std::size_t>(i) * kPartialAccFloats] : 0.0F;
  float mx = -INFINITY;
  for (int i = tid; i < n; i += kHeadDim) {
    const float2 ml = *reinterpret_cast<const float2*>(ml_g + static_cast<std::size_t>(i) * kPartialMlFloats);
    m_s[i] = ml.x, l_s[i] = ml.y;
    mx = fmaxf(mx, ml.x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFU, mx, o));
  if (lane == 0) red_s[warp] = mx;
  __syncthreads();
  float M = red_s[0];
#pragma unroll
  for (int w = 1; w < kHeadDim / 32; ++w) M = fmaxf(M, red_s[w]);
  for (int i = tid; i < n; i += kHeadDim) w_s[i] = m_s[i] == -INFINITY ? 0.0F : Exp2Fast(m_s[i] - M);
  __syncthreads();
  if (tid == 0) {   // the sum of the units' sums in unit order (few terms, kept sequential so the result is reproducible)
    float Lsum = 0.0F;
    for (int i = 0; i < n; ++i) Lsum = fmaf(w_s[i], l_s[i], Lsum);
    inv_l = 1.0F / Lsum;
  }
  float A = 0.0F;
#pragma unroll
  for (int i = 0; i < kCombineEarly; ++i) A = fmaf(i < n ? w_s[i] : 0.0F, early[i], A);   // unit order
#pragma unroll 8
  for (int i = kCombineEarly; i < n; ++i) A = fmaf(w_s[i], acc_g[static_cast<std::size_t>(i) * kPartialAccFloats], A);
  __syncthreads();
  float o = A * inv_l;
  const std::size_t oi = (static_cast<std::size_t>(b) * kQHeads + hh) * kHeadDim + tid;
  if (gate != nullptr) o *= 1.0F / (1.0F + expf(-gate[oi]));
  if (out_f32)
    static_cast<float*>(out)[oi] = o;
  else
    static_cast<__half*>(out)[oi] = __float2half_rn(o);
}

}  // namespace

cudaError_t ConfigureDecodeKernels() {
  cudaError_t e = cudaFuncSetAttribute(DecodePartKernel<kFmtQ8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       DecodeSmemBytes<kFmtQ8>());
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(DecodePartKernel<kFmtQ8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeSmemBytes<kFmtQ8>());
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(DecodePartKernel<kFmtQ4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeSmemBytes<kFmtQ4>());
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(DecodePartKernel<kFmtQ4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeSmemBytes<kFmtQ4>());
  return e;
}

template <int kFmt, bool kQRaw>
static cudaError_t LaunchPart(const DecodeLaunch& a, cudaStream_t stream) {
  const QueryRaw qr{kQRaw ? static_cast<const float*>(a.q_dev) : nullptr, a.q_weight_dev, a.rope_tab_dev, a.q_eps, a.rope_rows};
  return LaunchChained(DecodePartKernel<kFmt, kQRaw>, a.n_units, Shape<kFmt>::kThreads, DecodeSmemBytes<kFmt>(), stream,
                       *a.kmap, *a.vmap, a.pool, a.layer, a.tables_dev, a.table_stride, a.units_dev,
                       kQRaw ? nullptr : static_cast<const __half*>(a.q_dev), qr, a.scale_log2, a.partial_acc,
                       a.partial_ml, a.status_dev);
}

cudaError_t LaunchDecodePart(const DecodeLaunch& a, cudaStream_t stream) {
  if (a.n_units <= 0 || a.n_seqs <= 0) return cudaSuccess;
  if (a.pool.fmt == kFmtQ8) return a.q_raw ? LaunchPart<kFmtQ8, true>(a, stream) : LaunchPart<kFmtQ8, false>(a, stream);
  return a.q_raw ? LaunchPart<kFmtQ4, true>(a, stream) : LaunchPart<kFmtQ4, false>(a, stream);
}

cudaError_t LaunchDecodeCombine(const DecodeLaunch& a, cudaStream_t stream) {
  if (a.n_units <= 0 || a.n_seqs <= 0) return cudaSuccess;
  return LaunchChained(DecodeCombineKernel, a.n_seqs * kQHeads, kHeadDim, 0, stream, a.items_dev, a.partial_acc,
                       a.partial_ml, a.gate_dev, a.out_dev, a.out_f32);
}

}  // namespace yahkv
