// Chunked-prefill attention over the quantized cache: the one dense contraction of the path, on tcgen05 tensor cores
// with TMEM accumulators, fed by TMA.
//
// Stands in for the reference's yah_attn_wmma (causal FlashAttention over the paged cache, f16 MMA with f32
// accumulate, online softmax with exp2, f16 P, o / sum * sigmoid(gate): engine/gpu/loom/tools/gen_attn_fa.py:1-22,
// :67-71, :2897-2904, :3005-3042) together with its dequantize pre-pass yah_kdeq* / yah_vdeq* (:4648-4860), which
// the reference measured as a win over decoding at staging (docs/results.md:206). Like the reference's kernel it is
// not bit-identical to any ordering; the parity bar is 2e-3 max-abs against the float64 oracle.
//
// Pass 1, DequantPagesKernel (HBM-bound): every page of every sequence of the call, through the block table, to a
// token-major fp16 scratch (K and V), value = fp16(code * scale). 34.8 KB read and 64 KB written per page and kv head.
//
// Pass 2, PrefillKernel (tensor-bound): one CTA pair (a cluster of two CTAs on the two SMs of a TPC, cta_group::2)
// per tile of 128 query rows of two query heads of one KV head; head_dim 256. The pair shares every K and V tile:
// each CTA loads half of it, so a 64-key tile costs each SM 32 KB of L2 reads instead of 64 KB.
//   S = Q K^T   tcgen05.mma kind::f16, M 256 over the pair (128 rows = one head per CTA), N 64 (one 64-key tile), K 256
//               in 16 steps; A = Q held in each CTA's tensor memory for the whole CTA, B = the K tile in shared
//               memory (K-major, 128-byte swizzle), keys 0-31 in the leader, 32-63 in the peer; D = S in TMEM.
//   softmax     per CTA, two warpgroups of one thread per query row; tiles alternate between them. tcgen05.ld of the
//               64 scores (which frees the S buffer), causal mask, reference max with a lazy rescale of O (threshold
//               2^8) handed from the group of tile j to the group of tile j + 1 through shared memory, P = 2^(s - m)
//               as fp16 into a swizzled shared-memory tile. Each group keeps a partial row sum; the epilogue joins them.
//   O += P V    tcgen05.mma M 256, N 256, K 64 in 4 steps; A = P from each CTA's shared memory, B = the V tile as
//               loaded (token-major = MN-major B operand, 128-byte swizzle), dims 0-127 in the leader, 128-255 in the
//               peer; D = O in TMEM (256 columns).
// Q lives in tensor memory because with it in shared memory the kernel was bound by shared-memory bandwidth (the
// 64 KB Q tile re-read for every key tile). P goes through shared memory (16 KB per tile) so that the S buffer is
// free as soon as it has been read: S then runs two tiles ahead of P.V and the softmax of a tile, with its signals
// across the pair, has two tile periods before the tensor pipe waits for it.
// TMEM columns (all 512): S double-buffered 2 x 64, O 256, Q 128. Shared memory per CTA: YAHKV_PREFILL_STAGES stages
// of half a K tile + half a V tile (32 KB each), two P tiles, the barriers.
// Warp roles: 0-7 softmax / correction / epilogue, 8 TMA producer, 9 MMA issuer (leader CTA only) and TMEM owner; the
// producer and the issuer run their loops as converged warps and predicate only the asynchronous instructions on an
// elected lane. The TMA loads of both CTAs count their bytes on the leader's barrier (cta_group::2 loads, no
// multicast); the leader's commits arrive on the barriers of both CTAs; the peer's softmax warps arrive on the
// leader's barriers with plain (CTA-scope) remote arrivals. Every mbarrier wait is bounded and abortable: a wait that
// gives up raises a CTA-wide abort flag, every role leaves its loop, both CTAs meet at the cluster barrier, TMEM is
// freed, and the status word tells the host the call's results are invalid.
//
// Tiles of a call's last, partly filled wave arrive split along the keys (PrefillTile::jt_begin / jt_end / part): such
// a CTA leaves its unnormalised accumulator and the rows' (max, sum) in a workspace and PrefillMergeKernel joins the
// parts.
//
// What bounds it: the tensor pipe needs 1,024 clocks per 64-key tile (16 x 32 + 4 x 128). One CTA per (tile, head)
// with the whole K / V tile in each SM ran at ~1,430: every CTA pulled its own 64 KB per tile from L2, 45 B/clock/SM
// or about 10.5 TB/s over the chip. The pair halves that traffic.
#include <cuda_fp16.h>

#include <cmath>

#include "kernels.cuh"
#include "ptx.cuh"

#ifndef YAHKV_PREFILL_STAGES
#define YAHKV_PREFILL_STAGES 5   // K / V half tiles in flight per CTA (at least 3: S runs two tiles ahead of P.V)
#endif

namespace yahkv {
namespace {

// ----------------------------------------------------------------------------------------------------------------
// Pass 1: dequantize pages to fp16
// ----------------------------------------------------------------------------------------------------------------
constexpr int kDequantThreads = 256;

template <int kFmt>
__global__ void __launch_bounds__(kDequantThreads)
    DequantPagesKernel(PoolView pool, int layer, const std::int32_t* __restrict__ tables, int table_stride,
                       const PrefillSeq* __restrict__ seqs, __half* __restrict__ k16, __half* __restrict__ v16) {
  const PrefillSeq ps = seqs[blockIdx.z];
  const int p = blockIdx.x, kvh = blockIdx.y;
  if (p >= ps.n_pages || !pool.OwnsKvHead(kvh)) return;
  std::int32_t page = __ldg(tables + static_cast<std::size_t>(ps.seq) * table_stride + p);
  page = min(max(page, 0), pool.num_pages - 1);
  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + page) * kKvHeads + kvh;
  const std::size_t out_row0 = static_cast<std::size_t>(ps.kv_row0) + static_cast<std::size_t>(kvh) * ps.kv_rows +
                               static_cast<std::size_t>(p) * kPageTokens;
#pragma unroll
  for (int side = 0; side < 2; ++side) {
    const std::uint8_t* codes = (side == 0 ? pool.kcodes : pool.vcodes) + rec * RecordCodeBytes(kFmt);
    const std::uint16_t* scales = (side == 0 ? pool.kscales : pool.vscales) + rec * (kPageTokens * kBlocksPerRow);
    __half* out = (side == 0 ? k16 : v16) + out_row0 * kHeadDim;
    if constexpr (kFmt == kFmtF16) {   // fp16 pages: a gather of the rows as they are
      for (int gidx = threadIdx.x; gidx < kPageTokens * (kHeadDim / 8); gidx += kDequantThreads)
        *reinterpret_cast<uint4*>(out + static_cast<std::size_t>(gidx >> 5) * kHeadDim + (gidx & 31) * 8) =
            *reinterpret_cast<const uint4*>(codes + static_cast<std::size_t>(gidx) * 16);
      continue;
    }
    // thread -> 8 consecutive elements of a token row; 64 tokens x 32 groups = 2048 groups, 8 per thread
    for (int gidx = threadIdx.x; gidx < kPageTokens * (kHeadDim / 8); gidx += kDequantThreads) {
      const int tok = gidx >> 5, grp = gidx & 31;   // grp: elements 8 grp .. 8 grp + 7, block grp / 4
      const float d = __half2float(__ushort_as_half(scales[tok * kBlocksPerRow + (grp >> 2)]));
      float v[8];
      if constexpr (kFmt == kFmtQ8) {
        const uint2 c = *reinterpret_cast<const uint2*>(codes + tok * 256 + grp * 8);
        const std::uint8_t* cb = reinterpret_cast<const std::uint8_t*>(&c);   // K: int8; V: u = code + 128
#pragma unroll
        for (int i = 0; i < 8; ++i)
          v[i] = d * static_cast<float>(side == 0 ? static_cast<int>(static_cast<std::int8_t>(cb[i]))
                                                  : static_cast<int>(cb[i]) - kQ8FlipByte);
      } else {
        // block b = grp / 4 occupies bytes 16 b .. 16 b + 15; element e of the block is the low (e < 16) or high
        // nibble of byte e % 16. This group holds elements 8 (grp % 4) .. + 7 of its block.
        const int e0 = (grp & 3) * 8;
        const uint2 c = *reinterpret_cast<const uint2*>(codes + tok * 128 + (grp >> 2) * 16 + (e0 & 15));
        const std::uint8_t* cb = reinterpret_cast<const std::uint8_t*>(&c);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d * static_cast<float>(static_cast<int>(e0 < 16 ? (cb[i] & 0xF) : (cb[i] >> 4)) - 8);
      }
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      *reinterpret_cast<uint4*>(out + static_cast<std::size_t>(tok) * kHeadDim + grp * 8) = o;
    }
  }
}

// ----------------------------------------------------------------------------------------------------------------
// Pass 2: tcgen05 flash attention, one CTA pair (cta_group::2) per two query heads of a KV head
// ----------------------------------------------------------------------------------------------------------------
constexpr int kTileM = kPrefillTileRows;   // 128 query rows per CTA, 256 per pair
constexpr int kTileN = 64;                 // keys per KV tile
constexpr int kSoftmaxThreads = 256;       // warps 0-7: two warpgroups of one thread per query row
constexpr int kPrefillThreads = 320;       // + warp 8 TMA producer, warp 9 MMA issuer (leader CTA) and TMEM owner
constexpr int kWarpTma = 8, kWarpMma = 9;
// Each CTA of a pair holds half of every B operand: K rows (keys) 32 rank .. + 31 of the tile as four [32 keys][64 dims]
// boxes, V columns (dims) 128 rank .. + 127 as two [64 keys][64 dims] boxes. 16 KB each per tile.
constexpr int kKHalfBytes = (kTileN / 2) * kHeadDim * 2;
constexpr int kVHalfBytes = kTileN * (kHeadDim / 2) * 2;
constexpr int kKBlockBytes = (kTileN / 2) * 128;   // one [32 keys][64 dims] box
constexpr int kVBlockBytes = kTileN * 128;         // one [64 keys][64 dims] box
constexpr int kPBytes = kTileM * kTileN * 2;       // P of one tile: [128 rows][64 fp16], K-major, 128-byte swizzle
constexpr int kKvStages = YAHKV_PREFILL_STAGES;
static_assert(kKvStages >= 3, "S(j + 2) is issued before P(j) V(j): the loads of tile j + 2 must not wait for the stage of tile j");
constexpr int kSmemK = 0;
constexpr int kSmemV = kSmemK + kKvStages * kKHalfBytes;
constexpr int kSmemP = kSmemV + kKvStages * kVHalfBytes;
constexpr int kSmemBars = kSmemP + 2 * kPBytes;
constexpr int kBarBytes = 256;
constexpr int kPrefillSmemBytes = kSmemBars + kBarBytes + 4 * kTileM * 4;   // barriers, then the max / sum exchange
static_assert(kPrefillSmemBytes <= 232448, "shared memory of one CTA");
// TMEM columns (512 in all, the same in both CTAs): S double-buffered, O, and Q as the A operand of S = Q K^T.
constexpr int kTmemCols = 512;
constexpr int kColS = 0;      // two buffers of 64 fp32 columns
constexpr int kColO = 128;    // 256 fp32 columns
constexpr int kColQ = 384;    // 128 columns = 256 fp16 per row
constexpr float kPrefillLazyRescale = 8.0F;
constexpr int kStatusPrefillAbort = 3;

// Shared-memory matrix descriptors, 128-byte swizzle (layout type 2), descriptor version 1: bits 0-13 start address
// >> 4, 16-29 leading byte offset >> 4, 32-45 stride byte offset >> 4, bit 46 version, 61-63 layout.
//   K-major operand  [rows][64 fp16]: rows 128 B apart, groups of 8 rows 1024 B apart (stride byte offset).
//   MN-major operand [keys][64 fp16] x blocks: 8-key groups 1024 B apart (stride), 64-element blocks `lbo` apart.
// The high word is the same for every operand of this kernel.
constexpr std::uint32_t kDescHi = (1024U >> 4) | (1U << 14) | (2U << 29);
__device__ __forceinline__ std::uint32_t DescLo(std::uint32_t addr, std::uint32_t lbo_bytes) {
  return ((addr >> 4) & 0x3FFFU) | (((lbo_bytes >> 4) & 0x3FFFU) << 16);
}
// Instruction descriptor of kind::f16: fp16 A and B, fp32 accumulate, A K-major.
__host__ __device__ constexpr std::uint32_t InstrDesc(int m, int n, bool b_mn_major) {
  return (1U << 4) | (0U << 7) | (0U << 10) | (0U << 15) | ((b_mn_major ? 1U : 0U) << 16) |
         (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}

// D(tmem) (+)= A * B over the CTA pair: M = 256 (128 rows in each CTA's tensor memory, the same columns in both), the
// B half of each CTA from its shared memory at the same offset. Issued by one thread of the leader CTA.
//   Ts: A from each CTA's own tensor memory (two fp16 per 32-bit column). Q is held there for the whole CTA: with it
//       in shared memory the kernel was bound by shared-memory bandwidth (the 64 KB tile re-read for every key tile).
//   Ss: A from each CTA's own shared memory (descriptor), used for P.
__device__ __forceinline__ void UmmaF16Ts2(std::uint32_t d_tmem, std::uint32_t a_tmem, std::uint32_t b_desc_lo,
                                           std::uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 bd;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 bd, {%2, %3};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], bd, %4, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_desc_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate ? 1U : 0U)
      : "memory");
}
__device__ __forceinline__ void UmmaF16Ss2(std::uint32_t d_tmem, std::uint32_t a_desc_lo, std::uint32_t b_desc_lo,
                                           std::uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 ad, bd;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 ad, {%1, %3};\n"
      "mov.b64 bd, {%2, %3};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], ad, bd, %4, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_desc_lo), "r"(b_desc_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate ? 1U : 0U)
      : "memory");
}
// Arrives, once every tcgen05 operation this thread issued before has completed, on the barrier at this shared-memory
// offset in both CTAs of the pair (one commit per CTA).
__device__ __forceinline__ void UmmaCommitPair(std::uint64_t* bar) {
  const std::uint32_t a = SmemAddr(bar);
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(MapToCta(a, 0))
               : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(MapToCta(a, 1))
               : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TmemLd32(std::uint32_t addr, std::uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr));
}
__device__ __forceinline__ void TmemSt32(std::uint32_t addr, const std::uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
      "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void TmemWaitLd() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemWaitSt() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Bounded, abortable wait: gives up after ~2 s or as soon as another role of this CTA has raised the abort flag.
// kCluster: the barrier is arrived on from the other CTA of the pair (acquire at cluster scope).
template <bool kCluster = false>
__device__ __forceinline__ bool WaitOrAbort(std::uint64_t* bar, std::uint32_t parity, volatile int* abort_flag) {
  auto poll = [&]() { return kCluster ? MbarTryWaitCluster(bar, parity) : MbarTryWait(bar, parity); };
  if (poll()) return true;
  const std::uint64_t t0 = GlobalTimerNs();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (poll()) return true;
    if (*abort_flag != 0) return false;
    if (GlobalTimerNs() - t0 > 2000000000ULL) {
      *abort_flag = 1;
      return false;
    }
  }
}

// The barriers sit at the same shared-memory offsets in both CTAs of a pair. "leader": only the leader's copy is
// used (the peer arrives on it remotely). "both": the leader's MMA warp commits to the copy of each CTA, and each
// CTA waits on its own. "local": used inside one CTA only.
struct PrefillBars {
  std::uint64_t q_full;                // leader: softmax warps of both CTAs -> MMA: Q is in tensor memory
  std::uint64_t kv_full[kKvStages];    // leader: TMA of both CTAs -> MMA: both halves of K(j) and V(j) have landed
  std::uint64_t kv_empty[kKvStages];   // both: MMA -> TMA: P(j) V(j), the last reader of the stage, is complete
  std::uint64_t s_full[2];             // both: MMA -> softmax: S(j) is in its buffer
  std::uint64_t s_free[2];             // leader: softmax warps of both CTAs -> MMA: S(j) has been read into registers
  std::uint64_t p_full[2];             // leader: softmax warps of both CTAs -> MMA: P(j) is in shared memory, O rescaled
  std::uint64_t m_posted[2];           // local: softmax group of tile j -> group of tile j + 1: m(j) is in shared memory
  std::uint64_t pv_done[2];            // both: MMA -> softmax: O += P(j) V(j) complete, one barrier per tile parity
  std::uint64_t o_done;                // both: the last P.V is complete
  std::uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(PrefillBars) <= kBarBytes, "the max / sum exchange follows the barriers");

// kQRaw: the query arrives as the raw f32 projection (qraw) and the prologue does the query side of the fused norm +
// RoPE kernel for its rows, to the same bits: head RMS norm with that kernel's summation order (32 chains of 8
// consecutive dims, joined as a balanced tree), x inv x weight, NeoX RoPE on dims < 64 (pairs p, p + 32) at position
// pos0 + row, rounded to fp16. Stands in for the reference's QNORM prologue (engine/gpu/loom/tools/gen_attn_fa.py:56-61).
template <bool kQRaw>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPrefillThreads, 1)
    PrefillKernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const PrefillTile* __restrict__ tiles, const __half* __restrict__ q, const QueryRaw qraw,
                  const float* __restrict__ gate, void* out, int out_f32, float scale_log2,
                  float* __restrict__ part_acc, float* __restrict__ part_ml, int* status) {
  extern __shared__ __align__(1024) std::uint8_t smem[];
  PrefillBars* bars = reinterpret_cast<PrefillBars*>(smem + kSmemBars);
  volatile int* abort_flag = &bars->abort_flag;
  // Blocks 2 i and 2 i + 1 hold the tiles of two query heads of one KV head over the same query rows: the same key
  // range, the same K and V tiles, the same number of tiles (the planner emits them as neighbours).
  const PrefillTile tile = tiles[blockIdx.x];
  const std::uint32_t rank = ClusterCtaRank();   // 0 = leader: its MMA warp issues for the pair
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Key tiles jt0 .. jt0 + n_tiles - 1 of the keys the tile's rows can see: all of them, or one slice of a tile
  // that the planner split along the keys. Every loop below runs on the local index j; only the load coordinate and
  // the causal mask use the absolute tile jt0 + j.
  const int jt0 = tile.jt_begin;
  const int n_tiles = tile.jt_end - tile.jt_begin;

  // The swizzled operands need the 1024-byte aligned base. The dynamic shared memory starts at the same offset in
  // both CTAs, so either both leave here or neither does.
  if ((SmemAddr(smem) & 1023U) != 0) {
    if (threadIdx.x == 0) atomicExch(status, kStatusPrefillAbort);
    return;
  }
  if (threadIdx.x == 0) {
    MbarInit(&bars->q_full, 2 * kSoftmaxThreads / 32);   // one arrival per softmax warp of the pair
    for (int s = 0; s < kKvStages; ++s) {
      MbarInit(&bars->kv_full[s], 1);                     // the leader's expect_tx; both CTAs' copies count bytes on it
      MbarInit(&bars->kv_empty[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      MbarInit(&bars->s_full[g], 1);
      MbarInit(&bars->s_free[g], 2 * kSoftmaxThreads / 64);   // one arrival per warp of the tile's group, both CTAs
      MbarInit(&bars->p_full[g], 2 * kSoftmaxThreads / 64);
      MbarInit(&bars->m_posted[g], kSoftmaxThreads / 64);
      MbarInit(&bars->pv_done[g], 1);
    }
    MbarInit(&bars->o_done, 1);
    bars->abort_flag = 0;
    FenceBarrierInit();
  }
  if (warp == kWarpMma) {   // TMEM: the same warp of both CTAs allocates for the pair, and frees at the end
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&bars->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  TcFenceBefore();
  ClusterSync();   // both CTAs' barriers are initialised before either arrives on the other's
  TcFenceAfter();
  const std::uint32_t tmem = bars->tmem_base;

  if (warp == kWarpTma) {
    // ------------------------------ TMA producer: this CTA's halves of the K and V tiles ------------------------------
    // The warp stays converged; one elected lane issues the copies. All bytes of a stage, from both CTAs, are counted
    // on the leader's barrier, whose one arrival is the leader's expect_tx.
    const bool elected = ElectOne();
    if (elected) {
      PrefetchTensorMap(&kmap);
      PrefetchTensorMap(&vmap);
    }
    bool ok = true;
    int s = 0;
    std::uint32_t ph = 1;   // parity of the "empty" phase to wait for: 0 on the ring's second round, then alternating
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int y = tile.kv_row0 + (jt0 + j) * kTileN;
      if (j >= kKvStages) ok = WaitOrAbort(&bars->kv_empty[s], ph, abort_flag);
      if (!ok) break;
      if (elected) {
        const std::uint32_t full = MapToCta(SmemAddr(&bars->kv_full[s]), 0);
        if (rank == 0) MbarArriveExpectTx(&bars->kv_full[s], 2 * (kKHalfBytes + kVHalfBytes));
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)   // keys 32 rank .. + 31 of the tile, 64 dims per box
          TmaLoad2DPair(smem + kSmemK + s * kKHalfBytes + kb * kKBlockBytes, &kmap, kb * 64,
                        y + static_cast<int>(rank) * (kTileN / 2), full);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)   // all 64 keys, dims 128 rank + 64 kb .. + 63
          TmaLoad2DPair(smem + kSmemV + s * kVHalfBytes + kb * kVBlockBytes, &vmap,
                        (static_cast<int>(rank) * 2 + kb) * 64, y, full);
      }
      if (++s == kKvStages) s = 0, ph ^= 1U;
    }
  } else if (warp == kWarpMma) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    // Issue order: S(0), S(1), then for every tile j: S(j + 2), P(j) V(j). The tensor pipe executes one thread's
    // instructions in that order, so between the end of S(j) and the start of P(j) V(j) it has two tiles of other
    // work (P(j-2) V(j-2), S(j+1), P(j-1) V(j-1), S(j+2)): the softmax of tile j, with its two signals across the
    // pair, may take two tile periods before the pipe waits for it. S(j + 2) reuses the buffer of S(j), which is
    // free as soon as the softmax threads have read it into registers (s_free), because P goes to shared memory.
    // The whole warp runs the loop converged and only the tcgen05 instructions are predicated on the elected lane:
    // operands that are uniform across a converged warp reach the instruction without per-lane register traffic.
    if (rank == 0) {
      const bool elected = ElectOne();
      constexpr std::uint32_t idesc_s = InstrDesc(2 * kTileM, kTileN, false);
      constexpr std::uint32_t idesc_o = InstrDesc(2 * kTileM, kHeadDim, true);
      const std::uint32_t k_lo0 = DescLo(SmemAddr(smem + kSmemK), 16);             // K-major: lbo unused (16 B)
      const std::uint32_t v_lo0 = DescLo(SmemAddr(smem + kSmemV), kVBlockBytes);   // MN-major: lbo = 64-dim block pitch
      const std::uint32_t p_lo0 = DescLo(SmemAddr(smem + kSmemP), 16);             // K-major A operand
      const std::uint32_t q_col = tmem + kColQ, o_col = tmem + kColO;
      int ks = 0;                        // ring stage of the next S tile
      std::uint32_t kph = 0;
      int pv_s = 0;                      // ring stage of the next P.V tile (its V arrived with the K of S(j))
      auto issue_s = [&](int j) -> bool {   // S(j) = Q K(j)^T, A = Q from tensor memory, 16 dims (8 columns) per step
        if (!WaitOrAbort<true>(&bars->kv_full[ks], kph, abort_flag)) return false;
        if (j >= 2 && !WaitOrAbort<true>(&bars->s_free[j & 1], static_cast<std::uint32_t>((j - 2) >> 1) & 1U, abort_flag))
          return false;
        TcFenceAfter();
        const std::uint32_t lo = k_lo0 + ks * (kKHalfBytes >> 4);
        const std::uint32_t s_col = tmem + kColS + (j & 1) * kTileN;
        if (elected) {   // one divergent region per batch of instructions, not one per instruction
#pragma unroll
          for (int i = 0; i < 16; ++i)   // 64-dim blocks 4 KB apart, 16 dims = 32 B inside a block
            UmmaF16Ts2(s_col, q_col + i * 8, lo + (((i >> 2) * kKBlockBytes + (i & 3) * 32) >> 4), idesc_s, i > 0);
          UmmaCommitPair(&bars->s_full[j & 1]);
        }
        if (++ks == kKvStages) ks = 0, kph ^= 1U;
        return true;
      };
      auto issue_pv = [&](int j) -> bool {   // O += P(j) V(j), A = P from shared memory, 16 keys (32 B of a row) per step
        if (!WaitOrAbort<true>(&bars->p_full[j & 1], static_cast<std::uint32_t>(j >> 1) & 1U, abort_flag)) return false;
        TcFenceAfter();
        const std::uint32_t plo = p_lo0 + (j & 1) * (kPBytes >> 4);
        const std::uint32_t lo = v_lo0 + pv_s * (kVHalfBytes >> 4);
        if (elected) {
#pragma unroll
          for (int k16 = 0; k16 < kTileN / 16; ++k16)
            UmmaF16Ss2(o_col, plo + k16 * (32 >> 4), lo + k16 * ((16 * 128) >> 4), idesc_o, j > 0 || k16 > 0);
          UmmaCommitPair(&bars->kv_empty[pv_s]);
          UmmaCommitPair(&bars->pv_done[j & 1]);
        }
        if (++pv_s == kKvStages) pv_s = 0;
        return true;
      };
      bool ok = WaitOrAbort<true>(&bars->q_full, 0, abort_flag);
      if (ok && n_tiles > 0) ok = issue_s(0);
      if (ok && n_tiles > 1) ok = issue_s(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 2 < n_tiles) ok = issue_s(j + 2);
        if (ok) ok = issue_pv(j);
      }
      if (ok && elected) UmmaCommitPair(&bars->o_done);
    }
  } else {
    // ------------------ softmax, correction, epilogue: two warpgroups of one thread per query row ------------------
    // Warp w and w + 4 hold the same 32 rows (a warp reaches TMEM lanes 32 (w % 4) .. + 31). Group hc = 0 is warps
    // 0-3, group 1 warps 4-7; for the Q load and the epilogue a group takes half of the head dimension.
    const int r = threadIdx.x & (kTileM - 1);                    // query row 0..127
    const int hc = threadIdx.x >> 7;                             // warpgroup
    const std::uint32_t lane_addr = tmem + (static_cast<std::uint32_t>((warp & 3) * 32) << 16);
    // Q row -> tensor memory: this thread's 128 dims (256 B) as 64 columns of fp16 pairs. Rows past the chunk are zero.
    if constexpr (kQRaw) {
      const bool valid = r < tile.n_rows;
      const float* row = qraw.q + (static_cast<std::size_t>(tile.q_row0 + (valid ? r : 0)) * kQHeads + tile.head) * kHeadDim;
      // sum of squares over the whole row: chain l covers dims 8 l .. 8 l + 7; the tree joins chain l with l + 16,
      // then + 8, + 4, + 2, + 1 (the order of a butterfly over 32 lanes of 8 dims each)
      float ss[32];
#pragma unroll
      for (int l = 0; l < 32; ++l) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(row + l * 8));
        const float4 b = __ldg(reinterpret_cast<const float4*>(row + l * 8 + 4));
        float acc = 0.0F;
        acc = fmaf(a.x, a.x, acc), acc = fmaf(a.y, a.y, acc), acc = fmaf(a.z, a.z, acc), acc = fmaf(a.w, a.w, acc);
        acc = fmaf(b.x, b.x, acc), acc = fmaf(b.y, b.y, acc), acc = fmaf(b.z, b.z, acc), acc = fmaf(b.w, b.w, acc);
        ss[l] = acc;
      }
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1)
#pragma unroll
        for (int l = 0; l < m; ++l) ss[l] = __fadd_rn(ss[l], ss[l + m]);
      const float inv = __fdiv_rn(1.0F, __fsqrt_rn(__fadd_rn(__fmul_rn(ss[0], 1.0F / kHeadDim), qraw.eps)));
      const int pos = min(max(tile.pos0 + r, 0), qraw.rope_rows - 1);
      const float2* cs_row = qraw.rope_tab + static_cast<std::size_t>(pos) * 32;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const int d0 = hc * (kHeadDim / 2) + part * 64;   // this thread's 64 dims of the part
        std::uint32_t qr[32];
        if (d0 == 0) {   // the rotary dims: pairs (p, p + 32)
#pragma unroll
          for (int p = 0; p < 32; p += 2) {
            float lo[2], hi[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float xl = __fmul_rn(__fmul_rn(__ldg(row + p + e), inv), __ldg(qraw.weight + p + e));
              const float xh = __fmul_rn(__fmul_rn(__ldg(row + p + e + 32), inv), __ldg(qraw.weight + p + e + 32));
              const float2 cs = __ldg(cs_row + p + e);
              lo[e] = __fsub_rn(__fmul_rn(xl, cs.x), __fmul_rn(xh, cs.y));
              hi[e] = __fadd_rn(__fmul_rn(xl, cs.y), __fmul_rn(xh, cs.x));
            }
            const __half2 hl = __floats2half2_rn(lo[0], lo[1]), hh = __floats2half2_rn(hi[0], hi[1]);
            qr[p / 2] = *reinterpret_cast<const std::uint32_t*>(&hl);
            qr[16 + p / 2] = *reinterpret_cast<const std::uint32_t*>(&hh);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float2 x = __ldg(reinterpret_cast<const float2*>(row + d0 + 2 * i));
            const float2 w = __ldg(reinterpret_cast<const float2*>(qraw.weight + d0 + 2 * i));
            const __half2 h = __floats2half2_rn(__fmul_rn(__fmul_rn(x.x, inv), w.x), __fmul_rn(__fmul_rn(x.y, inv), w.y));
            qr[i] = *reinterpret_cast<const std::uint32_t*>(&h);
          }
        }
        if (!valid) {
#pragma unroll
          for (int i = 0; i < 32; ++i) qr[i] = 0U;
        }
        TmemSt32(lane_addr + kColQ + hc * 64 + part * 32, qr);
      }
      TmemWaitSt();
      TcFenceBefore();
      __syncwarp();
      if (lane == 0) MbarArriveCluster(MapToCta(SmemAddr(&bars->q_full), 0));
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(
          q + (static_cast<std::size_t>(tile.q_row0 + r) * kQHeads + tile.head) * kHeadDim + hc * (kHeadDim / 2));
      const bool valid = r < tile.n_rows;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        std::uint32_t qr[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v = valid ? __ldg(src + part * 8 + i) : make_uint4(0, 0, 0, 0);
          qr[4 * i] = v.x, qr[4 * i + 1] = v.y, qr[4 * i + 2] = v.z, qr[4 * i + 3] = v.w;
        }
        TmemSt32(lane_addr + kColQ + hc * 64 + part * 32, qr);
      }
      TmemWaitSt();
      TcFenceBefore();
      __syncwarp();
      if (lane == 0) MbarArriveCluster(MapToCta(SmemAddr(&bars->q_full), 0));
    }
    // Tiles alternate between the two warpgroups: group g = hc runs the softmax of tiles j = g, g + 2, ..., one
    // thread per query row with all 64 columns, so a tile's softmax may take up to two tile periods before it holds
    // the tensor pipe back. The rows' reference maximum travels between the groups through shared memory: the
    // group of tile j posts m(j) as soon as it has decided it (before its exponentials), the group of tile j + 1
    // picks it up. Each group keeps its own partial row sum, relative to the reference it last saw.
    const int my_last_key = tile.pos0 + r;                       // row r sees keys 0 .. pos0 + r
    float m_mine = -INFINITY, l_mine = 0.0F;
    float* mref = reinterpret_cast<float*>(smem + kSmemBars + kBarBytes);   // [128 rows]
    bool ok = true;
    for (int j = hc; j < n_tiles; j += 2) {
      const std::uint32_t ph = static_cast<std::uint32_t>(j >> 1) & 1U;
      ok = WaitOrAbort(&bars->s_full[hc], ph, abort_flag);
      ok = __all_sync(0xFFFFFFFFU, ok);
      if (!ok) break;
      TcFenceAfter();
      std::uint32_t sraw[64];
      TmemLd32(lane_addr + kColS + hc * kTileN, *reinterpret_cast<std::uint32_t(*)[32]>(&sraw[0]));
      TmemLd32(lane_addr + kColS + hc * kTileN + 32, *reinterpret_cast<std::uint32_t(*)[32]>(&sraw[32]));
      TmemWaitLd();
      TcFenceBefore();
      __syncwarp();   // every lane holds its row of S: the buffer may take S(j + 2)
      if (lane == 0) MbarArriveCluster(MapToCta(SmemAddr(&bars->s_free[hc]), 0));
      // Row max on the raw scores (the scale is positive); the causal mask only on tiles that reach past the tile's
      // first row (a warp-uniform test), where a masked score becomes -inf.
      const int key0 = (jt0 + j) * kTileN;
      if (key0 + kTileN - 1 > tile.pos0) {
#pragma unroll
        for (int c = 0; c < kTileN; ++c)
          if (key0 + c > my_last_key) sraw[c] = 0xFF800000U;   // -inf
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < kTileN; ++c) mx[c & 3] = fmaxf(mx[c & 3], __uint_as_float(sraw[c]));
      const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;   // log2 units from here on
      float m_ref = -INFINITY;
      if (j >= 1) {   // m(j-1), posted by the other group
        ok = WaitOrAbort(&bars->m_posted[hc ^ 1], static_cast<std::uint32_t>((j - 1) >> 1) & 1U, abort_flag);
        ok = __all_sync(0xFFFFFFFFU, ok);
        if (!ok) break;
        m_ref = mref[r];
      }
      if (m_mine != m_ref) {   // the other group moved the reference: bring this group's partial sum along
        l_mine *= Exp2Fast(m_mine - m_ref);   // m_mine = -inf only while l_mine = 0
        m_mine = m_ref;
      }
      const bool need = tmax > m_ref + kPrefillLazyRescale;
      if (__any_sync(0xFFFFFFFFU, need)) {   // warp-uniform (TMEM accesses are warp-wide)
        // O may only be rescaled once P(j-1) V(j-1) has completed, which also means the other group has finished
        // tile j - 1 (rare path: the reference settles after the first few tiles)
        if (j >= 1) {
          ok = WaitOrAbort(&bars->pv_done[hc ^ 1], static_cast<std::uint32_t>((j - 1) >> 1) & 1U, abort_flag);
          ok = __all_sync(0xFFFFFFFFU, ok);
          if (!ok) break;
          TcFenceAfter();
        }
        const float m_new = need ? tmax : m_ref;
        const float alpha = m_new == -INFINITY ? 1.0F : Exp2Fast(m_ref - m_new);
        m_mine = m_ref = m_new;
        l_mine *= alpha;
        if (j >= 1) {
#pragma unroll 1
          for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
            std::uint32_t o[32];
            TmemLd32(lane_addr + kColO + c0, o);
            TmemWaitLd();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            TmemSt32(lane_addr + kColO + c0, o);
          }
          TmemWaitSt();
        }
      }
      mref[r] = m_ref;
      __syncwarp();
      if (lane == 0) MbarArrive(&bars->m_posted[hc]);   // release: the warp's 32 rows of m(j) are posted
      const float neg_m = m_ref == -INFINITY ? 0.0F : -m_ref;
      // p = 2^(s * scale - m): one fma + one ex2 per element; the row sum in fp32 before the fp16 rounding. P goes
      // to shared memory as the A operand of P.V: this thread's row of 64 fp16 = one 128-byte row of the K-major,
      // 128-byte swizzled tile (16-byte chunk c of row r sits at chunk c ^ (r % 8)).
      float ls[4] = {0.0F, 0.0F, 0.0F, 0.0F};
      std::uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0 = Exp2Fast(fmaf(__uint_as_float(sraw[2 * i]), scale_log2, neg_m));
        const float p1 = Exp2Fast(fmaf(__uint_as_float(sraw[2 * i + 1]), scale_log2, neg_m));
        ls[i & 3] += p0 + p1;
        const __half2 h = __floats2half2_rn(p0, p1);
        pk[i] = *reinterpret_cast<const std::uint32_t*>(&h);
      }
      l_mine += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      if (j >= 2) {   // this group's P buffer was last read by P(j-2) V(j-2)
        ok = WaitOrAbort(&bars->pv_done[hc], static_cast<std::uint32_t>((j - 2) >> 1) & 1U, abort_flag);
        ok = __all_sync(0xFFFFFFFFU, ok);
        if (!ok) break;
      }
      {
        std::uint8_t* prow = smem + kSmemP + hc * kPBytes + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      FenceProxyAsync();   // the tensor core reads the tile through the async proxy
      TcFenceBefore();     // orders a rescale of O (tcgen05.st) before the arrival
      __syncwarp();        // every lane's row is written: one arrival stands for the warp
      if (lane == 0) MbarArriveCluster(MapToCta(SmemAddr(&bars->p_full[hc]), 0));
    }
    // ---- epilogue: O / l * sigmoid(gate); the two groups bring their partial sums to the final reference ----
    if (ok && n_tiles > 0) {
      ok = WaitOrAbort(&bars->o_done, 0, abort_flag);
      ok = __all_sync(0xFFFFFFFFU, ok);
    }
    float* xsum = mref + kTileM;   // [2 groups][128 rows]
    NamedBarrierSync(1, kSoftmaxThreads);   // the last m posted is visible to both groups
    if (n_tiles > 0) {
      const float m_fin = mref[r];
      if (m_mine != m_fin) l_mine *= Exp2Fast(m_mine - m_fin);
    }
    xsum[hc * kTileM + r] = l_mine;
    NamedBarrierSync(1, kSoftmaxThreads);
    if (ok && n_tiles > 0 && tile.part >= 0) {
      // A part of a split tile: the unnormalised accumulator and the row's (reference max, sum) go to the part's slot
      // of the workspace; the merge kernel joins the parts.
      TcFenceAfter();
      float* acc = part_acc + (static_cast<std::size_t>(tile.part) * kTileM + r) * kHeadDim + hc * (kHeadDim / 2);
      if (hc == 0) {
        float* ml = part_ml + (static_cast<std::size_t>(tile.part) * kTileM + r) * 2;
        ml[0] = mref[r];
        ml[1] = l_mine + xsum[kTileM + r];
      }
#pragma unroll 1
      for (int c0 = 0; c0 < kHeadDim / 2; c0 += 32) {
        std::uint32_t o[32];
        TmemLd32(lane_addr + kColO + hc * (kHeadDim / 2) + c0, o);
        TmemWaitLd();
        uint4* dst = reinterpret_cast<uint4*>(acc + c0);
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
      }
    } else if (ok && n_tiles > 0) {
      TcFenceAfter();
      const float inv = 1.0F / (l_mine + xsum[(hc ^ 1) * kTileM + r]);
      const bool valid = r < tile.n_rows;
      const std::size_t oi = (static_cast<std::size_t>(tile.q_row0 + r) * kQHeads + tile.head) * kHeadDim + hc * (kHeadDim / 2);
#pragma unroll 1
      for (int c0 = 0; c0 < kHeadDim / 2; c0 += 32) {
        std::uint32_t o[32];
        TmemLd32(lane_addr + kColO + hc * (kHeadDim / 2) + c0, o);
        TmemWaitLd();
        if (valid) {
          float v[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            v[c] = __uint_as_float(o[c]) * inv;
            if (gate != nullptr) v[c] *= 1.0F / (1.0F + expf(-gate[oi + c0 + c]));
          }
          if (out_f32) {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out) + oi + c0);
#pragma unroll
            for (int c = 0; c < 8; ++c) dst[c] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
          } else {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(out) + oi + c0);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 pk;
              __half2* ph = reinterpret_cast<__half2*>(&pk);
#pragma unroll
              for (int i = 0; i < 4; ++i) ph[i] = __floats2half2_rn(v[8 * c + 2 * i], v[8 * c + 2 * i + 1]);
              dst[c] = pk;
            }
          }
        }
      }
    }
  }
  // ---- teardown: every role of both CTAs arrives here, also after an abort. Past the cluster barrier neither CTA
  // issues tensor work on, nor arrives on barriers of, the other; then the pair's tensor memory is freed. ----
  TcFenceBefore();
  ClusterSync();
  if (threadIdx.x == 0 && bars->abort_flag != 0) atomicExch(status, kStatusPrefillAbort);
  if (warp == kWarpMma) {
    TcFenceAfter();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// Joins the parts of a split tile: out = (sum_i 2^(m_i - M) O_i) / (sum_i 2^(m_i - M) l_i) * sigmoid(gate), parts in
// order. Tiles come as pairs of heads, so the part slots of one head are two apart. One CTA per (split tile, group of 4 rows), thread = output dim; the rows of a group are independent, so their
// loads overlap (one CTA walking all 128 rows one after the other spent ~2 us of load latency per row).
constexpr int kMergeRows = 4;
constexpr int kMergeMaxParts = kPrefillMaxParts;
__global__ void __launch_bounds__(kHeadDim)
    PrefillMergeKernel(const PrefillMerge* __restrict__ merges, const PrefillTile* __restrict__ tiles,
                       const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                       const float* __restrict__ gate, void* out, int out_f32) {
  const PrefillMerge mg = merges[blockIdx.x];
  const PrefillTile t = tiles[mg.tile_index];
  const int d = threadIdx.x;
  const int np = min(mg.n_parts, kMergeMaxParts);
  float acc[kMergeRows][kMergeMaxParts], m[kMergeRows][kMergeMaxParts], l[kMergeRows][kMergeMaxParts];
#pragma unroll
  for (int rr = 0; rr < kMergeRows; ++rr) {
    const int r = blockIdx.y * kMergeRows + rr;
#pragma unroll
    for (int i = 0; i < kMergeMaxParts; ++i) {
      const bool on = i < np && r < t.n_rows;
      const std::size_t row = static_cast<std::size_t>(t.part + (on ? 2 * i : 0)) * kTileM + (on ? r : 0);
      acc[rr][i] = on ? part_acc[row * kHeadDim + d] : 0.0F;
      m[rr][i] = on ? part_ml[row * 2] : -INFINITY;
      l[rr][i] = on ? part_ml[row * 2 + 1] : 0.0F;
    }
  }
#pragma unroll
  for (int rr = 0; rr < kMergeRows; ++rr) {
    const int r = blockIdx.y * kMergeRows + rr;
    if (r >= t.n_rows) break;
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMergeMaxParts; ++i) M = fmaxf(M, m[rr][i]);
    float a = 0.0F, ls = 0.0F;
#pragma unroll
    for (int i = 0; i < kMergeMaxParts; ++i) {
      const float w = m[rr][i] == -INFINITY ? 0.0F : Exp2Fast(m[rr][i] - M);
      a = fmaf(w, acc[rr][i], a);
      ls = fmaf(w, l[rr][i], ls);
    }
    float o = a / ls;
    const std::size_t oi = (static_cast<std::size_t>(t.q_row0 + r) * kQHeads + t.head) * kHeadDim + d;
    if (gate != nullptr) o *= 1.0F / (1.0F + expf(-gate[oi]));
    if (out_f32)
      static_cast<float*>(out)[oi] = o;
    else
      static_cast<__half*>(out)[oi] = __float2half_rn(o);
  }
}

}  // namespace

cudaError_t ConfigurePrefillKernels(int* max_active_pairs) {
  cudaError_t e = cudaFuncSetAttribute(PrefillKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmemBytes);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(PrefillKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmemBytes);
  if (e != cudaSuccess) return e;
  // A pair needs two SMs of one GPC; a GPC with an odd number of usable SMs leaves one idle.
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2, 1, 1), cfg.blockDim = dim3(kPrefillThreads, 1, 1), cfg.dynamicSmemBytes = kPrefillSmemBytes;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, PrefillKernel<false>, &cfg);
  if (e != cudaSuccess) return e;
  *max_active_pairs = n;
  return cudaSuccess;
}

cudaError_t LaunchPrefillDequant(const PrefillLaunch& a, cudaStream_t stream) {
  if (a.n_seqs <= 0 || a.max_pages <= 0) return cudaSuccess;
  const dim3 grid(static_cast<unsigned>(a.max_pages), kKvHeads, static_cast<unsigned>(a.n_seqs));
  auto* k16 = static_cast<__half*>(a.k16_dev);
  auto* v16 = static_cast<__half*>(a.v16_dev);
  if (a.pool.fmt == kFmtQ8)
    DequantPagesKernel<kFmtQ8><<<grid, kDequantThreads, 0, stream>>>(a.pool, a.layer, a.tables_dev, a.table_stride,
                                                                     a.seqs_dev, k16, v16);
  else if (a.pool.fmt == kFmtF16)
    DequantPagesKernel<kFmtF16><<<grid, kDequantThreads, 0, stream>>>(a.pool, a.layer, a.tables_dev, a.table_stride,
                                                                      a.seqs_dev, k16, v16);
  else
    DequantPagesKernel<kFmtQ4><<<grid, kDequantThreads, 0, stream>>>(a.pool, a.layer, a.tables_dev, a.table_stride,
                                                                     a.seqs_dev, k16, v16);
  return cudaGetLastError();
}

cudaError_t LaunchPrefill(const PrefillLaunch& a, cudaStream_t stream) {
  if (a.n_tiles <= 0) return cudaSuccess;
  if ((a.n_tiles & 1) != 0) return cudaErrorInvalidValue;   // tiles come as pairs of query heads, one cluster each
  if (a.q_raw) {
    const QueryRaw qr{static_cast<const float*>(a.q_dev), a.q_weight_dev, a.rope_tab_dev, a.q_eps, a.rope_rows};
    PrefillKernel<true><<<a.n_tiles, kPrefillThreads, kPrefillSmemBytes, stream>>>(
        *a.k16map, *a.v16map, a.tiles_dev, nullptr, qr, a.gate_dev, a.out_dev, a.out_f32, a.scale_log2, a.part_acc,
        a.part_ml, a.status_dev);
  } else {
    PrefillKernel<false><<<a.n_tiles, kPrefillThreads, kPrefillSmemBytes, stream>>>(
        *a.k16map, *a.v16map, a.tiles_dev, static_cast<const __half*>(a.q_dev), QueryRaw{}, a.gate_dev, a.out_dev,
        a.out_f32, a.scale_log2, a.part_acc, a.part_ml, a.status_dev);
  }
  if (a.n_merges > 0)
    PrefillMergeKernel<<<dim3(a.n_merges, kTileM / kMergeRows), kHeadDim, 0, stream>>>(a.merges_dev, a.tiles_dev, a.part_acc, a.part_ml, a.gate_dev,
                                                          a.out_dev, a.out_f32);
  return cudaGetLastError();
}

}  // namespace yahkv
