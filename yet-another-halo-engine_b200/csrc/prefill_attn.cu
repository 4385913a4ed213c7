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
// Pass 2, PrefillKernel (tensor-bound): one CTA per tile of 128 query rows of one query head; head_dim 256.
//   S = Q K^T   tcgen05.mma kind::f16, M 128, N 64 (one 64-key tile), K 256 in 16 steps; A = Q held in tensor memory
//               for the whole CTA, B = the K tile in shared memory (K-major, 128-byte swizzle, four 64-dim TMA
//               boxes), D = S in TMEM.
//   softmax     two warpgroups of one thread per query row; tiles alternate between them. tcgen05.ld of the 64
//               scores, causal mask, reference max with a lazy rescale of O (threshold 2^8) handed from the group of
//               tile j to the group of tile j + 1 through shared memory, P = 2^(s - m) as fp16 written back over S
//               with tcgen05.st. Each group keeps a partial row sum; the epilogue joins them.
//   O += P V    tcgen05.mma M 128, N 256, K 64 in 4 steps; A = P from tensor memory, B = the V tile as loaded
//               (token-major = MN-major B operand, 128-byte swizzle), D = O in TMEM (256 columns).
// Both A operands live in tensor memory because with them in shared memory the kernel was bound by shared-memory
// bandwidth (the 64 KB Q tile re-read for every key tile).
// TMEM columns (all 512): S / P double-buffered 2 x 64, O 256, Q 128. Shared memory: three stages of K tile + V tile
// (64 KB each), one full / empty barrier pair per stage.
// Warp roles: 0-7 softmax / correction / epilogue, 8 TMA producer, 9 MMA issuer and TMEM owner; the producer and the
// issuer run their loops as converged warps and predicate only the asynchronous instructions on an elected lane
// (issued from inside a lane-0 branch a tcgen05.mma cost ~67 clocks of issue, from a converged warp ~27). No
// multicast, no cluster. Every mbarrier wait is bounded and abortable: a wait that gives up raises a CTA-wide abort
// flag, every role leaves its loop, TMEM is freed, and the status word tells the host the call's results are invalid.
//
// Tiles of a call's last, partly filled wave arrive split along the keys (PrefillTile::jt_begin / jt_end / part): such
// a CTA leaves its unnormalised accumulator and the rows' (max, sum) in a workspace and PrefillMergeKernel joins the
// parts.
//
// What bounds it: the tensor pipe needs 1,024 clocks per 64-key tile (16 x 32 + 4 x 128) and the measured steady
// state is ~1,430. The six query heads of a GQA group times the query tiles are separate CTAs, so every CTA pulls
// its own 64 KB per tile from L2: 45 B/clock/SM, about 10.5 TB/s over the chip, which is where the MMA warp's waits
// for loads come from (~125 clocks per tile). A CTA pair per two heads (cta_group::2, half of each B operand per
// CTA) removes those waits but puts two cross-CTA signals into the S -> softmax -> P.V chain, and with only two S
// buffers in TMEM that chain then bounds the tile at ~1,700 clocks; it needs a third S buffer (Q out of TMEM) to pay.
#include <cuda_fp16.h>

#include <cmath>

#include "kernels.cuh"
#include "ptx.cuh"

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
// Pass 2: tcgen05 flash attention
// ----------------------------------------------------------------------------------------------------------------
constexpr int kTileM = kPrefillTileRows;   // 128 query rows
constexpr int kTileN = 64;                 // keys per KV tile
constexpr int kSoftmaxThreads = 256;       // warps 0-7: two threads per query row, 32 of a tile's 64 columns each
constexpr int kPrefillThreads = 320;       // + warp 8 TMA producer, warp 9 MMA issuer
constexpr int kWarpTma = 8, kWarpMma = 9;
constexpr int kKvTileBytes = kTileN * kHeadDim * 2;  // 32768: four [64 keys][64 dims] boxes
constexpr int kKvStages = 3;
constexpr int kSmemK = 0;
constexpr int kSmemV = kSmemK + kKvStages * kKvTileBytes;
constexpr int kSmemBars = kSmemV + kKvStages * kKvTileBytes;
constexpr int kBarBytes = 256;
constexpr int kPrefillSmemBytes = kSmemBars + kBarBytes + 4 * kTileM * 4;   // barriers, then the max / sum exchange
// TMEM columns (512 in all): S / P double-buffered, O, and Q as the A operand of S = Q K^T.
constexpr int kTmemCols = 512;
constexpr int kColS = 0;      // two buffers of 64 fp32 columns; P (fp16 pairs) overwrites the first 32 of its buffer
constexpr int kColO = 128;    // 256 fp32 columns
constexpr int kColQ = 384;    // 128 columns = 256 fp16 per row
constexpr float kPrefillLazyRescale = 8.0F;
constexpr int kStatusPrefillAbort = 3;

// Shared-memory matrix descriptors, 128-byte swizzle (layout type 2), descriptor version 1: bits 0-13 start address
// >> 4, 16-29 leading byte offset >> 4, 32-45 stride byte offset >> 4, bit 46 version, 61-63 layout.
//   K-major operand  [rows][64 fp16]: rows 128 B apart, groups of 8 rows 1024 B apart (stride byte offset).
//   MN-major operand [keys][64 fp16] x blocks: 8-key groups 1024 B apart (stride), 64-element blocks `lbo` apart.
// Instruction descriptor of kind::f16: fp16 A and B, fp32 accumulate, A K-major.
__host__ __device__ constexpr std::uint32_t InstrDesc(int m, int n, bool b_mn_major) {
  return (1U << 4) | (0U << 7) | (0U << 10) | (0U << 15) | ((b_mn_major ? 1U : 0U) << 16) |
         (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}

// D(tmem) (+)= A(tmem) * B(smem). The A operand sits in tensor memory (row = lane, two fp16 per 32-bit column), so an
// MMA step reads only its B slice from shared memory: with both operands in shared memory this kernel was bound by
// shared-memory bandwidth (the 64 KB Q tile was re-read for every 64-key tile).
__device__ __forceinline__ void UmmaF16Ts(std::uint32_t d_tmem, std::uint32_t a_tmem, std::uint32_t b_desc_lo,
                                          std::uint32_t b_desc_hi, std::uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 bd;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 bd, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_desc_lo), "r"(b_desc_hi), "r"(idesc), "r"(accumulate ? 1U : 0U)
      : "memory");
}
__device__ __forceinline__ void UmmaCommit(std::uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar))
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

// Bounded, abortable wait: gives up after ~2 s or as soon as another role has raised the abort flag.
__device__ __forceinline__ bool WaitOrAbort(std::uint64_t* bar, std::uint32_t parity, volatile int* abort_flag) {
  if (MbarTryWait(bar, parity)) return true;
  const std::uint64_t t0 = GlobalTimerNs();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (MbarTryWait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (GlobalTimerNs() - t0 > 2000000000ULL) {
      *abort_flag = 1;
      return false;
    }
  }
}

struct PrefillBars {
  std::uint64_t q_full;    // softmax threads -> MMA: Q is in tensor memory
  std::uint64_t kv_full[kKvStages];    // TMA -> MMA: K(j) and V(j) have landed (one wait per tile for both)
  std::uint64_t kv_empty[kKvStages];   // MMA -> TMA: P(j) V(j), the last reader of the stage, is complete
  std::uint64_t s_full[2]; // MMA -> softmax: S(j) is in its buffer
  std::uint64_t p_full[2]; // softmax -> MMA: P(j) written over S(j), O rescaled; one per tile parity
  std::uint64_t m_posted[2];   // softmax group of tile j -> group of tile j + 1: m(j) is in shared memory
  std::uint64_t pv_done;   // MMA -> softmax: O += P(j) V(j) complete
  std::uint64_t o_done;    // MMA -> softmax: the last P.V is complete (a parity wait on pv_done may lag at most one phase,
                           // which the epilogue cannot guarantee)
  std::uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(PrefillBars) <= kBarBytes, "the max / sum exchange follows the barriers");

__global__ void __launch_bounds__(kPrefillThreads, 1)
    PrefillKernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const PrefillTile* __restrict__ tiles, const __half* __restrict__ q, const float* __restrict__ gate,
                  void* out, int out_f32, float scale_log2, float* __restrict__ part_acc, float* __restrict__ part_ml,
                  int* status) {
  extern __shared__ __align__(1024) std::uint8_t smem[];
  PrefillBars* bars = reinterpret_cast<PrefillBars*>(smem + kSmemBars);
  volatile int* abort_flag = &bars->abort_flag;
  const PrefillTile tile = tiles[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Key tiles jt0 .. jt0 + n_tiles - 1 of the keys the tile's rows can see: all of them, or one slice of a tile
  // that the planner split along the keys. Every loop below runs on the local index j; only the load coordinate and
  // the causal mask use the absolute tile jt0 + j.
  const int jt0 = tile.jt_begin;
  const int n_tiles = tile.jt_end - tile.jt_begin;

  if ((SmemAddr(smem) & 1023U) != 0) {   // the swizzled operands need the 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(status, kStatusPrefillAbort);
    return;
  }
  if (threadIdx.x == 0) {
    MbarInit(&bars->q_full, kSoftmaxThreads / 32);   // one arrival per softmax warp
    for (int s = 0; s < kKvStages; ++s) {
      MbarInit(&bars->kv_full[s], 1);
      MbarInit(&bars->kv_empty[s], 1);
    }
    MbarInit(&bars->s_full[0], 1);
    MbarInit(&bars->s_full[1], 1);
    for (int g = 0; g < 2; ++g) {
      MbarInit(&bars->p_full[g], kSoftmaxThreads / 64);   // one arrival per warp of the tile's group
      MbarInit(&bars->m_posted[g], kSoftmaxThreads / 64);
    }
    MbarInit(&bars->pv_done, 1);
    MbarInit(&bars->o_done, 1);
    bars->abort_flag = 0;
    FenceBarrierInit();
  }
  if (warp == kWarpMma) {   // TMEM: one warp allocates, the same warp frees
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&bars->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const std::uint32_t tmem = bars->tmem_base;

  if (warp == kWarpTma) {
    // ------------------------------ TMA producer: K and V tiles into their rings ------------------------------
    {   // the warp stays converged; one elected lane issues the copies
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
          MbarArriveExpectTx(&bars->kv_full[s], 2 * kKvTileBytes);
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            TmaLoad2D(smem + kSmemK + s * kKvTileBytes + kb * (kTileN * 128), &kmap, kb * 64, y, &bars->kv_full[s]);
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            TmaLoad2D(smem + kSmemV + s * kKvTileBytes + kb * (kTileN * 128), &vmap, kb * 64, y, &bars->kv_full[s]);
        }
        if (++s == kKvStages) s = 0, ph ^= 1U;
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------ MMA issuer ------------------------------
    // The tensor pipe executes in issue order, which is what makes the buffer reuse safe without further barriers:
    // S(j+2) is issued after P(j) V(j), the last reader of that S / P buffer.
    // Issue cost is what bounds this kernel, so the whole warp runs the loop converged and only the tcgen05.mma /
    // tcgen05.commit instructions are predicated on the elected lane: operands that are uniform across a converged
    // warp reach the instruction without per-lane register traffic (measured: ~67 clocks per MMA issued from inside
    // a lane-0 branch, under 40 from a converged warp). Descriptors are a constant high word and a low word = stage
    // base + compile-time offset; ring positions are running counters.
    {
      const bool elected = ElectOne();
      constexpr std::uint32_t idesc_s = InstrDesc(kTileM, kTileN, false);
      constexpr std::uint32_t idesc_o = InstrDesc(kTileM, kHeadDim, true);
      // descriptor words: K-major operand lbo 16 B, sbo 1024 B; MN-major V lbo = 64-dim block pitch
      constexpr std::uint32_t desc_hi = (1024U >> 4) | (1U << 14) | (2U << 29);
      std::uint32_t k_lo[kKvStages], v_lo[kKvStages];
#pragma unroll
      for (int s = 0; s < kKvStages; ++s) {
        k_lo[s] = ((SmemAddr(smem + kSmemK + s * kKvTileBytes) >> 4) & 0x3FFFU) | ((16U >> 4) << 16);
        v_lo[s] = ((SmemAddr(smem + kSmemV + s * kKvTileBytes) >> 4) & 0x3FFFU) |
                  ((static_cast<std::uint32_t>(kTileN * 128) >> 4) << 16);
      }
      const std::uint32_t q_col = tmem + kColQ, o_col = tmem + kColO;
      int pv_s = 0;                      // ring stage of the next P.V tile (its V arrived with the K of S(j))
      auto issue_pv = [&](int j) -> bool {   // O += P(j) V(j), A = P from its S buffer, 16 keys (8 columns) per step
        if (!WaitOrAbort(&bars->p_full[j & 1], static_cast<std::uint32_t>(j >> 1) & 1U, abort_flag)) return false;
        TcFenceAfter();
        const std::uint32_t p_col = tmem + kColS + (j & 1) * kTileN;
        const std::uint32_t lo = pv_s == 0 ? v_lo[0] : pv_s == 1 ? v_lo[1] : v_lo[2];
        if (elected) UmmaF16Ts(o_col, p_col, lo, desc_hi, idesc_o, j > 0);
#pragma unroll
        for (int k16 = 1; k16 < kTileN / 16; ++k16)
          if (elected) UmmaF16Ts(o_col, p_col + k16 * 8, lo + k16 * ((16 * 128) >> 4), desc_hi, idesc_o, true);
        if (elected) UmmaCommit(&bars->kv_empty[pv_s]);
        if (elected) UmmaCommit(&bars->pv_done);
        if (++pv_s == kKvStages) pv_s = 0;
        return true;
      };
      static_assert(kKvStages == 3, "the stage selects above are written for three stages");
      bool ok = WaitOrAbort(&bars->q_full, 0, abort_flag);
      int s = 0;
      std::uint32_t ph = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = j & 1;
        ok = WaitOrAbort(&bars->kv_full[s], ph, abort_flag);
        if (!ok) break;
        TcFenceAfter();
        const std::uint32_t lo = s == 0 ? k_lo[0] : s == 1 ? k_lo[1] : k_lo[2];
        const std::uint32_t s_col = tmem + kColS + b * kTileN;
#pragma unroll
        for (int i = 0; i < 16; ++i)   // A = Q from tensor memory, 16 dims (8 columns) per step; 64-dim blocks 8 KB apart
          if (elected) UmmaF16Ts(s_col, q_col + i * 8, lo + (((i >> 2) * (kTileN * 128) + (i & 3) * 32) >> 4), desc_hi, idesc_s, i > 0);
        if (elected) UmmaCommit(&bars->s_full[b]);
        if (++s == kKvStages) s = 0, ph ^= 1U;
        // the previous tile's P.V goes behind this tile's S, so the tensor pipe has work while softmax(j) runs
        if (j >= 1) ok = issue_pv(j - 1);
      }
      if (ok && n_tiles > 0) ok = issue_pv(n_tiles - 1);
      if (ok && elected) UmmaCommit(&bars->o_done);
    }
  } else {
    // ------------------ softmax, correction, epilogue: two warpgroups of one thread per query row ------------------
    // Warp w and w + 4 hold the same 32 rows (a warp reaches TMEM lanes 32 (w % 4) .. + 31). Group hc = 0 is warps
    // 0-3, group 1 warps 4-7; for the Q load and the epilogue a group takes half of the head dimension.
    const int r = threadIdx.x & (kTileM - 1);                    // query row 0..127
    const int hc = threadIdx.x >> 7;                             // warpgroup
    const std::uint32_t lane_addr = tmem + (static_cast<std::uint32_t>((warp & 3) * 32) << 16);
    // Q row -> tensor memory: this thread's 128 dims (256 B) as 64 columns of fp16 pairs. Rows past the chunk are zero.
    {
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
      if (lane == 0) MbarArrive(&bars->q_full);
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
          ok = WaitOrAbort(&bars->pv_done, static_cast<std::uint32_t>(j - 1) & 1U, abort_flag);
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
      // back into tensor memory as the A operand of P.V: 64 fp16 = the first 32 columns of this S buffer.
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
      TmemSt32(lane_addr + kColS + hc * kTileN, pk);
      TmemWaitSt();
      TcFenceBefore();
      __syncwarp();   // every lane's P columns are in tensor memory: one arrival stands for the warp
      if (lane == 0) MbarArrive(&bars->p_full[hc]);
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
  // ---- teardown: every role arrives here, also after an abort ----
  TcFenceBefore();
  __syncthreads();
  if (threadIdx.x == 0 && bars->abort_flag != 0) atomicExch(status, kStatusPrefillAbort);
  if (warp == kWarpMma) {
    TcFenceAfter();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// Joins the parts of a split tile: out = (sum_i 2^(m_i - M) O_i) / (sum_i 2^(m_i - M) l_i) * sigmoid(gate), parts in
// order. One CTA per (split tile, group of 4 rows), thread = output dim; the rows of a group are independent, so their
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
      const std::size_t row = static_cast<std::size_t>(t.part + (on ? i : 0)) * kTileM + (on ? r : 0);
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

cudaError_t ConfigurePrefillKernels() {
  return cudaFuncSetAttribute(PrefillKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmemBytes);
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
  PrefillKernel<<<a.n_tiles, kPrefillThreads, kPrefillSmemBytes, stream>>>(
      *a.k16map, *a.v16map, a.tiles_dev, static_cast<const __half*>(a.q_dev), a.gate_dev, a.out_dev, a.out_f32,
      a.scale_log2, a.part_acc, a.part_ml, a.status_dev);
  if (a.n_merges > 0)
    PrefillMergeKernel<<<dim3(a.n_merges, kTileM / kMergeRows), kHeadDim, 0, stream>>>(a.merges_dev, a.tiles_dev, a.part_acc, a.part_ml, a.gate_dev,
                                                          a.out_dev, a.out_f32);
  return cudaGetLastError();
}

}  // namespace yahkv
