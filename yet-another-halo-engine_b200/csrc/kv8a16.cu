// The reference's own kv8a16 cache format on B200: append (K per token, V per 16-key tile with an open fp16 tile) and
// split-K decode attention, on 64-token pages of four tiles (the reference uses 256-token pages).
//
// Stands in for dattn_kappend_q / dattn_vappend_q / dattn_part_q in their kv8a16 form and for the chunk writers yah_kq8 /
// yah_vq8 / yah_vseed: engine/gpu/loom/tools/gen_decode_attn.py:1043-1107, :436-573, :576-1040 and
// engine/gpu/loom/tools/gen_kvq.py:166-285, :474-660, :676-730. The arithmetic is the reference's, operation for
// operation, so that codes, scale pairs and statistic pairs are bit-identical to its numpy models
// (engine/gpu/loom/tools/dattn_q_check.py:61-73, :101-122):
//   K  x = f32(f16(k)) - mean;  per (head, 128-dim half): s = amax / 127 (1 when 0),  u = roundeven(x * (1 / s)) + 128,
//      a dword holds dims 4i .. 4i+3 in byte slots (d0, d2, d1, d3);  pair = f16 (256 s, -384 s).
//   V  per (16-key tile, channel): cen = (max + min) / 2, s = (max - min) / 254 (1 when 0), both rounded to f16,
//      u = clamp(roundeven((v - cf) * (1 / sf)) + 128, 0, 255), dword w byte p = key 4w + (0, 2, 1, 3)[p];
//      pair = f16 (256 sf, cf - 384 sf).
// The tile that holds a sequence's newest key stays in fp16 in an "open tile" buffer and attention reads it from
// there, also right after its 16th key has quantized it (gen_decode_attn.py:426-427, :995-1028). The K mean is
// never added back: it moves every score of a head by the same amount (docs/architecture.md:206).
//
// Pools (per layer, all in the context's four allocations):
//   kcodes [page][4][64 tokens][256 B]   kscales [page][4][64][2 halves][2] f16
//   vcodes [page][4][4 tiles][256 channels][16 B]   vscales [page][4][4][256][2] f16
// Per (sequence, layer): two open-tile buffers [4][256][16] f16 and the mean [4][256] f32. An append that moves on to
// a new tile writes that tile into the OTHER buffer, so the kernel's blocks never write what another block still
// reads; which buffer is current is host state, handed to the kernels per call.
//
// Decode attention has the shape of the q8_0 / q4_0 kernel (a TMA-filled ring of page stages, whole-tile warps); see
// the comment above it. Prefill attention uses the tensor-core kernel of the other formats behind a dequantize pass of
// its own (Kv8DequantPagesKernel).
#include <cuda_fp16.h>

#include <cmath>

#include "decode_ring.cuh"
#include "qrope.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

namespace yahkv {
namespace {

// ---------------------------------------------------------------------------------------------------------------
// Append, K side: one warp per (token, kv head); lane l holds dims 8 l .. 8 l + 7, a 128-dim half is 16 lanes.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) Kv8AppendKKernel(PoolView pool, int layer, const std::int64_t* __restrict__ slots,
                                                        const std::int32_t* __restrict__ state_rows, int state_row_add,
                                                        const float* __restrict__ kmean,
                                                        const __half* __restrict__ k_in) {
  ChainedKernelEntry();
  const int token = blockIdx.x, h = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const std::int64_t slot = slots[token];
  if (slot < 0 || !pool.OwnsKvHead(h)) return;
  std::int64_t page = slot / kPageTokens;
  const int tok = static_cast<int>(slot % kPageTokens);
  page = min(max(page, static_cast<std::int64_t>(0)), static_cast<std::int64_t>(pool.num_pages - 1));
  const uint4 raw = *reinterpret_cast<const uint4*>(k_in + (static_cast<std::size_t>(token) * kKvHeads + h) * kHeadDim + lane * 8);
  const float* mean = kmean + (static_cast<std::size_t>(state_rows[token] + state_row_add) * kKvHeads + h) * kHeadDim + lane * 8;
  const float4 m0 = *reinterpret_cast<const float4*>(mean), m1 = *reinterpret_cast<const float4*>(mean + 4);
  const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
  const __half2* hp = reinterpret_cast<const __half2*>(&raw);
  float x[8], amax = 0.0F;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(hp[i]);
    x[2 * i] = __fsub_rn(f.x, mm[2 * i]), x[2 * i + 1] = __fsub_rn(f.y, mm[2 * i + 1]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
  for (int o = 1; o <= 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFU, amax, o));   // over the half's 16 lanes
  const float s0 = __fdiv_rn(amax, 127.0F);
  const float s = s0 > 0.0F ? s0 : 1.0F;
  const float inv = __fdiv_rn(1.0F, s);
  std::uint32_t w[2];
#pragma unroll
  for (int d = 0; d < 2; ++d) {   // dword 2 lane + d holds dims 4i .. 4i+3 in byte slots (d0, d2, d1, d3)
    const float* xx = x + 4 * d;
    const std::uint32_t u0 = static_cast<std::uint32_t>(rintf(__fmul_rn(xx[0], inv)) + 128.0F);
    const std::uint32_t u1 = static_cast<std::uint32_t>(rintf(__fmul_rn(xx[1], inv)) + 128.0F);
    const std::uint32_t u2 = static_cast<std::uint32_t>(rintf(__fmul_rn(xx[2], inv)) + 128.0F);
    const std::uint32_t u3 = static_cast<std::uint32_t>(rintf(__fmul_rn(xx[3], inv)) + 128.0F);
    w[d] = (u0 & 255U) | ((u2 & 255U) << 8) | ((u1 & 255U) << 16) | ((u3 & 255U) << 24);
  }
  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + static_cast<std::size_t>(page)) * kKvHeads + h;
  std::uint8_t* codes = pool.kcodes + rec * RecordCodeBytes(kFmtKv8) + static_cast<std::size_t>(tok) * 256;
  *reinterpret_cast<uint2*>(codes + lane * 8) = make_uint2(w[0], w[1]);
  if ((lane & 15) == 0) {
    std::uint16_t* sc = pool.kscales + rec * (RecordScaleBytes(kFmtKv8, 0) / 2) + static_cast<std::size_t>(tok) * 4 + (lane >> 4) * 2;
    const __half2 pr = __halves2half2(__float2half_rn(__fmul_rn(s, 256.0F)), __float2half_rn(__fmul_rn(s, -384.0F)));
    *reinterpret_cast<__half2*>(sc) = pr;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Append, V side: one CTA per (tile touched by the call, kv head), thread = channel.
// ---------------------------------------------------------------------------------------------------------------
// kBits = 8: 255 levels around the centre, four dwords per channel. kBits = 4 (kv4a16, dattn_q_check.py:101-122 with
// bits = 4): 15 levels, u = clamp(roundeven((v - cf) / sf) + 7, 0, 14), two dwords per channel with nibble p of dword w =
// key 8w + 2p (p < 4) or 8w + 2(p - 4) + 1, pair (16 sf, cf - 23 sf).
template <int kBits>
__global__ void __launch_bounds__(kHeadDim) Kv8AppendVKernel(PoolView pool, int layer, const VTileWork* __restrict__ work,
                                                             int state_row_add, __half* __restrict__ open_tiles,
                                                             const __half* __restrict__ v_in) {
  ChainedKernelEntry();
  const VTileWork wk = work[blockIdx.x];
  const int h = blockIdx.y, ch = threadIdx.x;
  if (!pool.OwnsKvHead(h)) return;
  __half* open_pair = open_tiles + static_cast<std::size_t>(wk.state_row + state_row_add) * 2 * kOpenTileHalfs;
  const std::size_t ch_off = (static_cast<std::size_t>(h) * kHeadDim + ch) * kTileKeys;
  __align__(16) __half v[kTileKeys];
  {
    const uint4* src = reinterpret_cast<const uint4*>(open_pair + static_cast<std::size_t>(wk.read_buf) * kOpenTileHalfs + ch_off);
    const uint4 a = src[0], b = src[1];
    *reinterpret_cast<uint4*>(v) = a;
    *reinterpret_cast<uint4*>(v + 8) = b;
  }
#pragma unroll
  for (int j = 0; j < kTileKeys; ++j)
    if (j >= wk.n_old && j < wk.n_keys)
      v[j] = v_in[(static_cast<std::size_t>(wk.src[j]) * kKvHeads + h) * kHeadDim + ch];
  if (wk.write_buf >= 0) {   // the sequence's newest tile: its keys stay available in fp16 (stale columns are masked)
    uint4* dst = reinterpret_cast<uint4*>(open_pair + static_cast<std::size_t>(wk.write_buf) * kOpenTileHalfs + ch_off);
    dst[0] = *reinterpret_cast<const uint4*>(v);
    dst[1] = *reinterpret_cast<const uint4*>(v + 8);
  }
  if (wk.complete == 0) return;
  float x[kTileKeys], mx = -INFINITY, mn = INFINITY;
#pragma unroll
  for (int j = 0; j < kTileKeys; ++j) {
    x[j] = __half2float(v[j]);
    mx = fmaxf(mx, x[j]), mn = fminf(mn, x[j]);
  }
  constexpr float kLevels = kBits == 8 ? 254.0F : 14.0F, kOff = kBits == 8 ? 128.0F : 7.0F, kMax = kBits == 8 ? 255.0F : 14.0F;
  constexpr float kSMul = kBits == 8 ? 256.0F : 16.0F, kCMul = kBits == 8 ? -384.0F : -23.0F;
  const float cen = __fmul_rn(__fadd_rn(mx, mn), 0.5F);
  const float s0 = __fdiv_rn(__fsub_rn(mx, mn), kLevels);
  const float s = s0 > 0.0F ? s0 : 1.0F;
  const float sf = __half2float(__float2half_rn(s)), cf = __half2float(__float2half_rn(cen));
  const float inv = __fdiv_rn(1.0F, sf);
  std::uint32_t u[kTileKeys];
#pragma unroll
  for (int k = 0; k < kTileKeys; ++k) {
    float q = __fadd_rn(rintf(__fmul_rn(__fsub_rn(x[k], cf), inv)), kOff);
    q = fminf(fmaxf(q, 0.0F), kMax);
    u[k] = static_cast<std::uint32_t>(q);
  }
  std::int64_t page = wk.phys_tile / kTilesPerPage;
  page = min(max(page, static_cast<std::int64_t>(0)), static_cast<std::int64_t>(pool.num_pages - 1));
  const int t_in_page = wk.phys_tile % kTilesPerPage;
  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + static_cast<std::size_t>(page)) * kKvHeads + h;
  constexpr int kChBytes = kBits * 2;   // 16 codes of a channel
  std::uint8_t* codes = pool.vcodes + rec * RecordCodeBytes(kBits == 8 ? kFmtKv8 : kFmtKv4) + (static_cast<std::size_t>(t_in_page) * kHeadDim + ch) * kChBytes;
  if constexpr (kBits == 8) {   // dword d byte p = key 4d + (0, 2, 1, 3)[p]
    std::uint32_t w[4];
#pragma unroll
    for (int d = 0; d < 4; ++d) w[d] = u[4 * d] | (u[4 * d + 2] << 8) | (u[4 * d + 1] << 16) | (u[4 * d + 3] << 24);
    *reinterpret_cast<uint4*>(codes) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {                      // dword d: keys 8d + (0, 2, 4, 6) in the low 16 bits, 8d + (1, 3, 5, 7) in the high ones
    std::uint32_t w[2];
#pragma unroll
    for (int d = 0; d < 2; ++d) {
      w[d] = 0;
#pragma unroll
      for (int p = 0; p < 8; ++p) w[d] |= u[8 * d + (p < 4 ? 2 * p : 2 * (p - 4) + 1)] << (4 * p);
    }
    *reinterpret_cast<uint2*>(codes) = make_uint2(w[0], w[1]);
  }
  std::uint16_t* st = pool.vscales + rec * (RecordScaleBytes(kFmtKv8, 1) / 2) + (static_cast<std::size_t>(t_in_page) * kHeadDim + ch) * 2;
  *reinterpret_cast<__half2*>(st) =
      __halves2half2(__float2half_rn(__fmul_rn(sf, kSMul)), __float2half_rn(__fadd_rn(cf, __fmul_rn(sf, kCMul))));
}

// ---------------------------------------------------------------------------------------------------------------
// Decode attention: one CTA per split-K unit (a run of pages of one sequence for one kv head, all six query heads).
//
// The same shape as the q8_0 / q4_0 kernel: a ring of page-sized stages filled by non-multicast TMA on one mbarrier
// per stage, eight warps on two pages at a time (warp w owns 16-key tile w % 4 of the pages of parity w / 4 and does
// everything for it: scores over 256 dims, softmax, 256 output channels), the last of a page's four warps refills its
// stage, no barrier and no exchange inside the page loop. A stage holds the page's K codes as two swizzled 64 x 128 B
// boxes (box = one 128-dim half), its four V tiles as stored (one linear 16 KB copy), the V statistic pairs (4 KB) and
// the K scale pairs (512 B): 37,376 B, three stages per CTA, two CTAs per SM.
//
// Scores: the integer MMA on the unsigned codes, the four 32-byte blocks of a half accumulating in the instruction's
// accumulator, which starts at -128 x the plane sums of the query half (u = value + 128). The ldmatrix rows are given
// in the order the V tile packs its keys, so that score column c of key tile kt is key 4 (c / 2) + 2 kt + c % 2 and
// the weights land in the second MMA's operand layout with no shuffle; a thread's four scores are then four
// consecutive keys, and their scale pairs two 16-byte loads.
// Values: v = a (u - 128) + b per (tile, channel), a = S / 256, b = 1.5 S + C'. u - 128 enters the f16 MMA as exact
// integers against the weights' hi and lo parts (both into one fresh accumulator); a and b are applied in fp32 to
// the tile's sums: o += a d + b sum(p) (with the codes entering as 1024 + u and b shifted to match). The tile that holds the newest key is read in fp16 from the sequence's open
// buffer (in the same key order), by plain loads: one tile per sequence and kv head.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kKv8Stages = 3;
constexpr int kKv8KeyGroups = 4;
constexpr int kKv8PageSets = 2;
constexpr int kKv8Warps = kKv8KeyGroups * kKv8PageSets;
constexpr int kKv8Threads = kKv8Warps * 32;
constexpr int kKv8BoxBytes = 64 * 128;
constexpr int kKv8KBytes = 2 * kKv8BoxBytes;                          // K codes of a page of one kv head
constexpr int kKv8VBytes = kTilesPerPage * kHeadDim * kTileKeys;      // V codes
constexpr int kKv8VsBytes = kTilesPerPage * kHeadDim * 4;             // V statistic pairs
constexpr int kKv8KsBytes = kPageTokens * 2 * 4;                      // K scale pairs
static_assert(kKv8KBytes == RecordCodeBytes(kFmtKv8) && kKv8VBytes == RecordCodeBytes(kFmtKv8), "record sizes");
static_assert(kKv8KsBytes == RecordScaleBytes(kFmtKv8, 0) && kKv8VsBytes == RecordScaleBytes(kFmtKv8, 1), "record sizes");
constexpr int kKv8TxBytes = kKv8KBytes + kKv8VBytes + kKv8VsBytes + kKv8KsBytes;
// Shared memory (dynamic, 1024-byte aligned base): the four parts of the ring each as [stage][...] so that every K box
// starts on a 1024-byte boundary without padding; then the query operands and the bookkeeping words. Two CTAs and
// their 1 KB reservations fill an SM's 228 KB to within 512 bytes.
constexpr int kKv8KOff = 0;
constexpr int kKv8VOff = kKv8KOff + kKv8Stages * kKv8KBytes;
constexpr int kKv8VsOff = kKv8VOff + kKv8Stages * kKv8VBytes;
constexpr int kKv8KsOff = kKv8VsOff + kKv8Stages * kKv8VsBytes;
constexpr int kKv8RingBytes = kKv8KsOff + kKv8Stages * kKv8KsBytes;
constexpr int kKv8QLanes = 24;
constexpr int kKv8QfragOff = kKv8RingBytes;                           // [8 blocks][24 lanes][4] u32
constexpr int kKv8BarOff = kKv8QfragOff + kBlocksPerRow * kKv8QLanes * 16;
constexpr int kKv8DoneOff = kKv8BarOff + 8 * kKv8Stages;
constexpr int kKv8FillOff = kKv8DoneOff + 4 * kKv8Stages;
constexpr int kKv8QStepOff = kKv8FillOff + 4 * kKv8Stages;            // [8] f32
constexpr int kKv8QCorrOff = (kKv8QStepOff + 32 + 7) / 8 * 8;         // [2 halves][8 heads] int2
constexpr int kKv8AbortOff = kKv8QCorrOff + 2 * 8 * 8;
constexpr int kKv8SmemBytes = (kKv8AbortOff + 4 + 127) / 128 * 128;
static_assert(2 * (kKv8SmemBytes + 1024) <= 228 * 1024, "two CTAs per SM");
static_assert(kKv8Warps * kDecodeMergeWarpFloats * 4 <= kKv8RingBytes, "the merge scratch aliases the ring");
constexpr float kLazyRescale = 4.0F;
constexpr float kQSteps = 32000.0F;
constexpr int kStatusSmemMisaligned = 2;

__device__ __forceinline__ void MmaS8U8Acc(int (&d)[4], const std::uint32_t (&a)[4], std::uint32_t b0, std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

template <bool kQRaw>   // kQRaw: the raw f32 query, normed and rotated in the prologue (qrope.cuh)
__global__ void __launch_bounds__(kKv8Threads, 2)
    Kv8DecodePartKernel(const __grid_constant__ CUtensorMap kmap, PoolView pool, int layer,
                        const std::int32_t* __restrict__ tables, int table_stride, const DecodeUnit* __restrict__ units,
                        const __half* __restrict__ q, const QueryRaw qraw, float scale_log2,
                        const __half* __restrict__ open_tiles,
                        int n_layers, float* __restrict__ partial_acc, float* __restrict__ partial_ml, int* status) {
  ChainedKernelEntry();
  extern __shared__ __align__(1024) std::uint8_t smem[];
  std::uint32_t* qfrag = reinterpret_cast<std::uint32_t*>(smem + kKv8QfragOff);
  std::uint64_t* full_bar = reinterpret_cast<std::uint64_t*>(smem + kKv8BarOff);
  int* done_cnt = reinterpret_cast<int*>(smem + kKv8DoneOff);     // warps done reading a stage's page
  int* fill_cnt = reinterpret_cast<int*>(smem + kKv8FillOff);     // fills issued to a stage so far
  float* q_step = reinterpret_cast<float*>(smem + kKv8QStepOff);
  int2* q_corr = reinterpret_cast<int2*>(smem + kKv8QCorrOff);    // -128 x the plane sums of each query half
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kKv8AbortOff);
  if ((SmemAddr(smem) & 1023U) != 0) {   // never seen; a misaligned swizzle would corrupt results
    if (threadIdx.x == 0) atomicExch(status, kStatusSmemMisaligned);
    return;
  }

  const DecodeUnit u = units[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kw = warp & (kKv8KeyGroups - 1);   // tile kw of a page
  const int par = warp / kKv8KeyGroups;        // this warp's pages: index par, par + 2, ... of the unit
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
      MbarArriveExpectTx(&full_bar[s], kKv8TxBytes);
      TmaLoad2D(smem + kKv8KOff + s * kKv8KBytes, &kmap, 0, y, &full_bar[s]);
      TmaLoad2D(smem + kKv8KOff + s * kKv8KBytes + kKv8BoxBytes, &kmap, 128, y, &full_bar[s]);
      BulkLoad(smem + kKv8VOff + s * kKv8VBytes, pool.vcodes + rec * kKv8VBytes, kKv8VBytes, &full_bar[s]);
      BulkLoad(smem + kKv8VsOff + s * kKv8VsBytes, pool.vscales + rec * (kKv8VsBytes / 2), kKv8VsBytes, &full_bar[s]);
      BulkLoad(smem + kKv8KsOff + s * kKv8KsBytes, pool.kscales + rec * (kKv8KsBytes / 2), kKv8KsBytes, &full_bar[s]);
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      PrefetchTensorMap(&kmap);
      for (int s = 0; s < kKv8Stages; ++s) {
        MbarInit(&full_bar[s], 1);
        done_cnt[s] = 0;
        fill_cnt[s] = 0;
      }
      *abort_flag = 0;
      FenceBarrierInit();
    }
    __syncwarp();
    for (int i = 0; i < kKv8Stages && i < n_pages; ++i) issue(i, __ldg(row + i));
  }

  // Query planes through shared memory. Warp h < 6 quantizes head h: lane l holds dims 8 l .. 8 l + 7, bytes in the
  // pool's order (a dword's dims in slots d0, d2, d1, d3). q16 = rint(q * 32000 / amax), hi = (q16 + 128) >> 8,
  // lo = q16 - 256 hi. The A operand of 32-byte block b for lane (g = head, t): a0 = hi bytes 4t .. 4t+3, a1 = lo of the
  // same, a2 = hi bytes 16+4t .., a3 = lo of those: rows 0-5 of the MMA are the hi plane, rows 8-13 the lo plane.
  if (warp < kGroup) {
    const uint4 raw = LoadQueryLane8<kQRaw>(q, qraw, static_cast<std::size_t>(u.batch) * kQHeads + u.kvh * kGroup + warp,
                                            u.n_keys - 1, lane);
    const __half2* hp = reinterpret_cast<const __half2*>(&raw);
    float x[8], amax = 0.0F;
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
    int sum_hi = 0, sum_lo = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q16 = __float2int_rn(x[i] * inv);
      const int hi = (q16 + 128) >> 8;
      const int lo = q16 - hi * 256;
      sum_hi += hi, sum_lo += lo;
      const int slot = (i & 3) == 1 ? 2 : (i & 3) == 2 ? 1 : (i & 3);
      hi_w[i >> 2] |= (static_cast<std::uint32_t>(hi) & 0xFFU) << (8 * slot);
      lo_w[i >> 2] |= (static_cast<std::uint32_t>(lo) & 0xFFU) << (8 * slot);
    }
#pragma unroll
    for (int o = 1; o <= 8; o <<= 1) {   // plane sums over the 128-dim half (16 lanes)
      sum_hi += __shfl_xor_sync(0xFFFFFFFFU, sum_hi, o);
      sum_lo += __shfl_xor_sync(0xFFFFFFFFU, sum_lo, o);
    }
    if ((lane & 15) == 0) q_corr[(lane >> 4) * 8 + warp] = make_int2(-128 * sum_hi, -128 * sum_lo);
    const int blk = lane >> 2, e0 = (lane & 3) * 8;
    const int reg = e0 < 16 ? 0 : 2, t0 = (e0 & 15) >> 2;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      std::uint32_t* dst = qfrag + ((blk * kKv8QLanes + warp * 4 + t0 + j) << 2) + reg;
      dst[0] = hi_w[j];
      dst[1] = lo_w[j];
    }
    if (lane == 0) q_step[warp] = amax / kQSteps;
  }
  __syncthreads();   // barriers initialised, query planes visible
  const int qlane = lane < kKv8QLanes ? lane : lane - 8;   // the two padding rows of the MMA reuse heads 4, 5
  const std::uint32_t qa_addr = SmemAddr(qfrag + (qlane << 2));
  // softmax scale x log2(e) x the head's query step x 1 / 256 (the K pair's first value is 256 s)
  const float score_scale = scale_log2 * q_step[qlane >> 2] * (1.0F / 256.0F);
  const int2* my_corr = q_corr + (qlane >> 2);   // [half][head]: loaded at use, the loop has no registers to spare

  float o_acc[16][4];   // [c][0..3] = (channel 16c + g, head 2t), (16c + g, 2t+1), (16c + g + 8, 2t), (16c + g + 8, 2t+1)
#pragma unroll
  for (int c = 0; c < 16; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[c][i] = 0.0F;
  float m_run = -INFINITY, l_run = 0.0F;
  bool alive = true;

  // ldmatrix row of this lane in a K box: matrix (lane >> 3) & 1 is key tile kt, row lane & 7 its column c, which is
  // key 4 (c / 2) + 2 kt + c % 2 of the 16; 16-byte chunk 2x + (lane >> 4) of the 128-byte row, swizzled.
  const int lm_key = kw * kTileKeys + 4 * ((lane & 7) >> 1) + 2 * ((lane >> 3) & 1) + (lane & 1);
  const std::uint32_t lm0 = lm_key * 128 + (((lane >> 4) ^ (lm_key & 7)) << 4);
  const int cur_tile = (u.n_keys - 1) / kTileKeys;

  for (int i = par; i < n_pages; i += kKv8PageSets) {
    const int s = i % kKv8Stages;
    const int gen = i / kKv8Stages;
    std::int32_t refill_page = 0;
    if (lane == 0 && i + kKv8Stages < n_pages) refill_page = __ldg(row + i + kKv8Stages);
    alive = RingWait(alive, fill_cnt + s, &full_bar[s], gen, abort_flag);
    const int tile = (u.page_begin + i) * kTilesPerPage + kw;
    if (tile <= cur_tile) {   // warp-uniform: tiles past the newest key hold nothing
      const std::uint32_t k_base = SmemAddr(smem + kKv8KOff + s * kKv8KBytes);

      // ---- scores ----
      int acc[2][2][4];   // [key tile][half][hi col 2t, hi col 2t+1, lo col 2t, lo col 2t+1]
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int2 cr = my_corr[8 * hf];
#pragma unroll
        for (int kt = 0; kt < 2; ++kt) acc[kt][hf][0] = cr.x, acc[kt][hf][1] = cr.x, acc[kt][hf][2] = cr.y, acc[kt][hf][3] = cr.y;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          std::uint32_t w[4], qa[4];
          LdMatrixX4(k_base + hf * kKv8BoxBytes + (lm0 ^ (static_cast<std::uint32_t>(b) << 5)), w);
          LoadQ4(qa, qa_addr + (4 * hf + b) * (kKv8QLanes * 16));
          MmaS8U8Acc(acc[0][hf], qa, w[0], w[2]);
          MmaS8U8Acc(acc[1][hf], qa, w[1], w[3]);
        }
      }
      // This thread's four columns are keys 4t .. 4t+3 of the tile (key 4t + 2 kt + j): their scale pairs are 32
      // consecutive bytes, per key (half 0: 256 s, -384 s; half 1: the same).
      float sc[2][2];
      {
        const uint4* ks = reinterpret_cast<const uint4*>(smem + kKv8KsOff + s * kKv8KsBytes + (kw * kTileKeys + 4 * t) * 8);
        const uint4 ka = ks[0], kb = ks[1];
        const std::uint32_t pr[4][2] = {{ka.x, ka.y}, {ka.z, ka.w}, {kb.x, kb.y}, {kb.z, kb.w}};
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float s0 = __low2float(*reinterpret_cast<const __half2*>(&pr[2 * kt + j][0]));
            const float s1 = __low2float(*reinterpret_cast<const __half2*>(&pr[2 * kt + j][1]));
            const float v0 = static_cast<float>(acc[kt][0][j] * 256 + acc[kt][0][2 + j]);
            const float v1 = static_cast<float>(acc[kt][1][j] * 256 + acc[kt][1][2 + j]);
            sc[kt][j] = fmaf(s0, v0, s1 * v1) * score_scale;
          }
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
      if (__any_sync(0xFFFFFFFFU, lane < kKv8QLanes && tmax > m_run + kLazyRescale)) {
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
        const __half* open_buf = open_tiles + ((static_cast<std::size_t>(u.seq) * n_layers + layer) * 2 + (u.pad & 1)) * kOpenTileHalfs +
            static_cast<std::size_t>(u.kvh) * kHeadDim * kTileKeys;
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
        // One ldmatrix.x4 = the dwords of 32 channels (row = a channel's 16 bytes): matrices 0 / 1 are channels
        // 16c + r and 16c + 8 + r of c = 2 cp, matrices 2 / 3 those of c = 2 cp + 1; the thread's word is keys 4t .. 4t+3
        // in byte slots (0, 2, 1, 3).
        const std::uint32_t v_addr = SmemAddr(smem + kKv8VOff + s * kKv8VBytes + kw * (kHeadDim * kTileKeys)) + lane * 16;
        const std::uint32_t* vs = reinterpret_cast<const std::uint32_t*>(smem + kKv8VsOff + s * kKv8VsBytes + kw * (kHeadDim * 4)) + g;
#pragma unroll
        for (int cp = 0; cp < 8; ++cp) {
          std::uint32_t w[4];
          LdMatrixX4(v_addr + cp * 512, w);
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int c = 2 * cp + x;
            // bytes (0, 2) = keys 4t, 4t+1; bytes (1, 3) = keys 4t+2, 4t+3. A byte permuted under 0x64 is the f16
            // 1024 + u: the offset is not subtracted here but joins the per-channel affine below
            // (v = a (u - 128) + b = a (1024 + u) + (b - 1152 a), and b - 1152 a = C' - 3 S).
            const std::uint32_t a0 = __byte_perm(w[2 * x], 0x64646464U, 0x4240), a2 = __byte_perm(w[2 * x], 0x64646464U, 0x4341);
            const std::uint32_t a1 = __byte_perm(w[2 * x + 1], 0x64646464U, 0x4240), a3 = __byte_perm(w[2 * x + 1], 0x64646464U, 0x4341);
            float d[4];
            MmaF16Zero(d, a0, a1, a2, a3, p_hi[0], p_hi[1]);
            MmaF16(d, a0, a1, a2, a3, p_lo[0], p_lo[1]);
            const std::uint32_t s0 = vs[16 * c], s1 = vs[16 * c + 8];
            const float2 st0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
            const float2 st1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));
            const float sa0 = st0.x * (1.0F / 256.0F), sb0 = fmaf(-3.0F, st0.x, st0.y);
            const float sa1 = st1.x * (1.0F / 256.0F), sb1 = fmaf(-3.0F, st1.x, st1.y);
            o_acc[c][0] = fmaf(sa0, d[0], fmaf(sb0, ps0, o_acc[c][0]));
            o_acc[c][1] = fmaf(sa0, d[1], fmaf(sb0, ps1, o_acc[c][1]));
            o_acc[c][2] = fmaf(sa1, d[2], fmaf(sb1, ps0, o_acc[c][2]));
            o_acc[c][3] = fmaf(sa1, d[3], fmaf(sb1, ps1, o_acc[c][3]));
          }
        }
      }
    }

    // The last of the page's four warps to finish with the stage refills it. The MMAs above consumed every shared
    // memory read of the stage, so this warp's reads are complete.
    const bool last = RingRelease(&done_cnt[s], lane, kKv8KeyGroups);
    if (last && i + kKv8Stages < n_pages) issue(s, __shfl_sync(0xFFFFFFFFU, refill_page, 0));
  }
  if (!alive && lane == 0) atomicExch(status, kStatusWaitTimeout);
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 1);
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 2);

  // Every stage has been consumed (or a wait gave up): the ring is free to hold the merge scratch.
  __syncthreads();
  RingDrainAfterAbort(abort_flag, fill_cnt, full_bar, kKv8Stages);
  MergeUnitAndStore<kKv8Warps, false>(reinterpret_cast<float*>(smem), o_acc, m_run, l_run, warp, lane,
                                      partial_acc + static_cast<std::size_t>(u.partial) * kPartialAccFloats,
                                      partial_ml + static_cast<std::size_t>(u.partial) * kPartialMlFloats);
}

// ---------------------------------------------------------------------------------------------------------------
// Prefill attention's dequantize pass for this format: every page of every sequence of the call, through the block
// table, to the token-major fp16 scratch the tensor-core kernel reads (the reference's yah_kdeq* / yah_vdeq* pre-pass,
// engine/gpu/loom/tools/gen_attn_fa.py:4648-4860). K = fp16((u - 128) s) per 128-dim half, bytes back in dim order;
// the mean stays out (it moves every score of a head by the same amount). V = fp16((u - 128) a + b) per (tile,
// channel), transposed from [channel][16 keys] to [key][channel]; the tile that holds the sequence's newest key comes
// from the open fp16 buffer, as in decode attention.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kKv8DequantThreads = 256;
__global__ void __launch_bounds__(kKv8DequantThreads)
    Kv8DequantPagesKernel(PoolView pool, int layer, int n_layers, const std::int32_t* __restrict__ tables,
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
  {   // K: thread -> 8 bytes of a token row = dims 8 grp .. 8 grp + 7 with the middle two of each dword swapped
    const std::uint8_t* codes = pool.kcodes + rec * RecordCodeBytes(kFmtKv8);
    const std::uint16_t* scales = pool.kscales + rec * (RecordScaleBytes(kFmtKv8, 0) / 2);
    __half* out = k16 + out_row0 * kHeadDim;
    for (int gidx = threadIdx.x; gidx < kPageTokens * (kHeadDim / 8); gidx += kKv8DequantThreads) {
      const int tok = gidx >> 5, grp = gidx & 31;
      const float s = __half2float(__ushort_as_half(scales[tok * 4 + (grp >> 4) * 2])) * (1.0F / 256.0F);
      const uint2 c = *reinterpret_cast<const uint2*>(codes + tok * 256 + grp * 8);
      const std::uint8_t* cb = reinterpret_cast<const std::uint8_t*>(&c);
      float v[8];
#pragma unroll
      for (int d = 0; d < 2; ++d) {
        v[4 * d + 0] = s * static_cast<float>(static_cast<int>(cb[4 * d + 0]) - 128);
        v[4 * d + 1] = s * static_cast<float>(static_cast<int>(cb[4 * d + 2]) - 128);
        v[4 * d + 2] = s * static_cast<float>(static_cast<int>(cb[4 * d + 1]) - 128);
        v[4 * d + 3] = s * static_cast<float>(static_cast<int>(cb[4 * d + 3]) - 128);
      }
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      *reinterpret_cast<uint4*>(out + static_cast<std::size_t>(tok) * kHeadDim + grp * 8) = o;
    }
  }
  {   // V: thread -> two neighbouring channels of one tile (16 keys each), written as one half2 per key
    const std::uint8_t* codes = pool.vcodes + rec * RecordCodeBytes(kFmtKv8);
    const std::uint16_t* stats = pool.vscales + rec * (RecordScaleBytes(kFmtKv8, 1) / 2);
    const int open_tile = (ps.kv_len - 1) / kTileKeys;
    const __half* open_buf = open_tiles + ((static_cast<std::size_t>(ps.seq) * n_layers + layer) * 2 + (ps.pad[0] & 1)) * kOpenTileHalfs +
                             static_cast<std::size_t>(kvh) * kHeadDim * kTileKeys;
    __half* out = v16 + out_row0 * kHeadDim;
    for (int w = threadIdx.x; w < kTilesPerPage * (kHeadDim / 2); w += kKv8DequantThreads) {
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
          const uint4 c = *reinterpret_cast<const uint4*>(codes + (static_cast<std::size_t>(tl) * kHeadDim + ch + x) * 16);
          const std::uint32_t st = *reinterpret_cast<const std::uint32_t*>(stats + (static_cast<std::size_t>(tl) * kHeadDim + ch + x) * 2);
          const float2 pr = __half22float2(*reinterpret_cast<const __half2*>(&st));
          const float a = pr.x * (1.0F / 256.0F), b = fmaf(1.5F, pr.x, pr.y);
          const std::uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
          for (int d = 0; d < 4; ++d) {   // dword d byte slot (0, 1, 2, 3) = key 4d + (0, 2, 1, 3)
            val[x][4 * d + 0] = fmaf(a, static_cast<float>(static_cast<int>(cw[d] & 255U) - 128), b);
            val[x][4 * d + 2] = fmaf(a, static_cast<float>(static_cast<int>((cw[d] >> 8) & 255U) - 128), b);
            val[x][4 * d + 1] = fmaf(a, static_cast<float>(static_cast<int>((cw[d] >> 16) & 255U) - 128), b);
            val[x][4 * d + 3] = fmaf(a, static_cast<float>(static_cast<int>(cw[d] >> 24) - 128), b);
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

cudaError_t ConfigureKv8Kernels() {
  cudaError_t e = cudaFuncSetAttribute(Kv8DecodePartKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kKv8SmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(Kv8DecodePartKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kKv8SmemBytes);
}

cudaError_t LaunchKv8AppendK(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                             const std::int32_t* state_rows_dev, int state_row_add, const float* kmean_dev,
                             const void* k_dev, cudaStream_t stream) {
  if (n_tokens <= 0) return cudaSuccess;
  return LaunchChained(Kv8AppendKKernel, n_tokens, 128, 0, stream, pool, layer, slots_dev, state_rows_dev, state_row_add,
                       kmean_dev, static_cast<const __half*>(k_dev));
}

cudaError_t LaunchKv8AppendV(const PoolView& pool, int layer, int n_work, const VTileWork* work_dev, int state_row_add,
                             void* open_tiles_dev, const void* v_dev, cudaStream_t stream) {
  if (n_work <= 0) return cudaSuccess;
  if (pool.fmt == kFmtKv4)
    return LaunchChained(Kv8AppendVKernel<4>, dim3(n_work, kKvHeads), kHeadDim, 0, stream, pool, layer, work_dev,
                         state_row_add, static_cast<__half*>(open_tiles_dev), static_cast<const __half*>(v_dev));
  return LaunchChained(Kv8AppendVKernel<8>, dim3(n_work, kKvHeads), kHeadDim, 0, stream, pool, layer, work_dev,
                       state_row_add, static_cast<__half*>(open_tiles_dev), static_cast<const __half*>(v_dev));
}

cudaError_t LaunchKv8DecodePart(const DecodeLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream) {
  if (a.n_units <= 0 || a.n_seqs <= 0) return cudaSuccess;
  const auto* open16 = static_cast<const __half*>(open_tiles_dev);
  if (a.q_raw) {
    const QueryRaw qr{static_cast<const float*>(a.q_dev), a.q_weight_dev, a.rope_tab_dev, a.q_eps, a.rope_rows};
    return LaunchChained(Kv8DecodePartKernel<true>, a.n_units, kKv8Threads, kKv8SmemBytes, stream, *a.kmap, a.pool, a.layer,
                         a.tables_dev, a.table_stride, a.units_dev, static_cast<const __half*>(nullptr), qr, a.scale_log2,
                         open16, n_layers, a.partial_acc, a.partial_ml, a.status_dev);
  }
  return LaunchChained(Kv8DecodePartKernel<false>, a.n_units, kKv8Threads, kKv8SmemBytes, stream, *a.kmap, a.pool, a.layer,
                       a.tables_dev, a.table_stride, a.units_dev, static_cast<const __half*>(a.q_dev), QueryRaw{},
                       a.scale_log2, open16, n_layers, a.partial_acc, a.partial_ml, a.status_dev);
}

cudaError_t LaunchKv8PrefillDequant(const PrefillLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream) {
  if (a.n_seqs <= 0 || a.max_pages <= 0) return cudaSuccess;
  const dim3 grid(static_cast<unsigned>(a.max_pages), kKvHeads, static_cast<unsigned>(a.n_seqs));
  Kv8DequantPagesKernel<<<grid, kKv8DequantThreads, 0, stream>>>(a.pool, a.layer, n_layers, a.tables_dev, a.table_stride,
                                                                a.seqs_dev, static_cast<const __half*>(open_tiles_dev),
                                                                static_cast<__half*>(a.k16_dev), static_cast<__half*>(a.v16_dev));
  return cudaGetLastError();
}

}  // namespace yahkv
