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
// Decode attention here uses plain global loads (every warp takes whole 16-key tiles: K rows as 16-byte loads that
// land in the integer MMA's operand layout, V tiles a dword per (channel, lane)); it is the straightforward form, not
// yet the TMA-ring form of the q8_0 / q4_0 kernel.
#include <cuda_fp16.h>

#include <cmath>

#include "kernels.cuh"
#include "ptx.cuh"

namespace yahkv {
namespace {

// ---------------------------------------------------------------------------------------------------------------
// Append, K side: one warp per (token, kv head); lane l holds dims 8 l .. 8 l + 7, a 128-dim half is 16 lanes.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) Kv8AppendKKernel(PoolView pool, int layer, const std::int64_t* __restrict__ slots,
                                                        const std::int32_t* __restrict__ state_rows,
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
  const float* mean = kmean + (static_cast<std::size_t>(state_rows[token]) * kKvHeads + h) * kHeadDim + lane * 8;
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
__global__ void __launch_bounds__(kHeadDim) Kv8AppendVKernel(PoolView pool, int layer, const VTileWork* __restrict__ work,
                                                             __half* __restrict__ open_tiles,
                                                             const __half* __restrict__ v_in) {
  ChainedKernelEntry();
  const VTileWork wk = work[blockIdx.x];
  const int h = blockIdx.y, ch = threadIdx.x;
  if (!pool.OwnsKvHead(h)) return;
  __half* open_pair = open_tiles + static_cast<std::size_t>(wk.state_row) * 2 * kOpenTileHalfs;
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
  const float cen = __fmul_rn(__fadd_rn(mx, mn), 0.5F);
  const float s0 = __fdiv_rn(__fsub_rn(mx, mn), 254.0F);
  const float s = s0 > 0.0F ? s0 : 1.0F;
  const float sf = __half2float(__float2half_rn(s)), cf = __half2float(__float2half_rn(cen));
  const float inv = __fdiv_rn(1.0F, sf);
  std::uint32_t w[4];
#pragma unroll
  for (int d = 0; d < 4; ++d) {   // dword d byte p = key 4d + (0, 2, 1, 3)[p]
    std::uint32_t u[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float q = __fadd_rn(rintf(__fmul_rn(__fsub_rn(x[4 * d + k], cf), inv)), 128.0F);
      q = fminf(fmaxf(q, 0.0F), 255.0F);
      u[k] = static_cast<std::uint32_t>(q);
    }
    w[d] = u[0] | (u[2] << 8) | (u[1] << 16) | (u[3] << 24);
  }
  std::int64_t page = wk.phys_tile / kTilesPerPage;
  page = min(max(page, static_cast<std::int64_t>(0)), static_cast<std::int64_t>(pool.num_pages - 1));
  const int t_in_page = wk.phys_tile % kTilesPerPage;
  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + static_cast<std::size_t>(page)) * kKvHeads + h;
  std::uint8_t* codes = pool.vcodes + rec * RecordCodeBytes(kFmtKv8) + (static_cast<std::size_t>(t_in_page) * kHeadDim + ch) * 16;
  *reinterpret_cast<uint4*>(codes) = make_uint4(w[0], w[1], w[2], w[3]);
  std::uint16_t* st = pool.vscales + rec * (RecordScaleBytes(kFmtKv8, 1) / 2) + (static_cast<std::size_t>(t_in_page) * kHeadDim + ch) * 2;
  *reinterpret_cast<__half2*>(st) =
      __halves2half2(__float2half_rn(__fmul_rn(sf, 256.0F)), __float2half_rn(__fadd_rn(cf, __fmul_rn(sf, -384.0F))));
}

// ---------------------------------------------------------------------------------------------------------------
// Decode attention: one CTA per split-K unit, a warp per 16-key tile (round robin), all 256 dims per warp.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kKv8Warps = 8;
constexpr int kKv8Threads = kKv8Warps * 32;
constexpr int kMergeStride = kHeadDim + 8;
constexpr int kMergeWarpFloats = kGroup * kMergeStride + 16;
constexpr int kKv8SmemBytes = kKv8Warps * kMergeWarpFloats * 4;   // merge scratch; the query planes alias its start
constexpr float kLazyRescale = 4.0F;
constexpr float kQSteps = 32000.0F;

__device__ __forceinline__ void MmaS8U8Acc(int (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                           std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void MmaF16Zero(float (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                           std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0F));
}

__global__ void __launch_bounds__(kKv8Threads, 2)
    Kv8DecodePartKernel(PoolView pool, int layer, const std::int32_t* __restrict__ tables, int table_stride,
                        const DecodeUnit* __restrict__ units, const __half* __restrict__ q, float scale_log2,
                        const __half* __restrict__ open_tiles, int n_layers, float* __restrict__ partial_acc,
                        float* __restrict__ partial_ml) {
  ChainedKernelEntry();
  extern __shared__ __align__(16) std::uint8_t smem[];
  // Query planes in the pool's byte order: [6 heads][hi | lo][256 B], then per (head, half) -128 x the plane sums and
  // the head's quantization step. They live at the start of the merge scratch, which is only used after the loop.
  std::uint8_t* planes = smem;                                        // 6 * 2 * 256
  int* corr = reinterpret_cast<int*>(smem + 6 * 2 * 256);             // [6][2 halves][2 planes]
  float* q_step = reinterpret_cast<float*>(smem + 6 * 2 * 256 + 96);  // [8]

  const DecodeUnit u = units[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_pages = u.page_end - u.page_begin;
  if (n_pages <= 0) return;

  if (warp < kGroup) {   // quantize head `warp` to two int8 planes, bytes in the order the K pool holds a dword
    const __half* qrow = q + (static_cast<std::size_t>(u.batch) * kQHeads + u.kvh * kGroup + warp) * kHeadDim;
    const uint4 raw = *reinterpret_cast<const uint4*>(qrow + 8 * lane);
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
    int hi[8], lo[8], sum_hi = 0, sum_lo = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q16 = __float2int_rn(x[i] * inv);
      hi[i] = (q16 + 128) >> 8;
      lo[i] = q16 - hi[i] * 256;
      sum_hi += hi[i], sum_lo += lo[i];
    }
    auto pack = [](const int* v) {   // byte slots (d0, d2, d1, d3)
      return (static_cast<std::uint32_t>(v[0]) & 255U) | ((static_cast<std::uint32_t>(v[2]) & 255U) << 8) |
             ((static_cast<std::uint32_t>(v[1]) & 255U) << 16) | ((static_cast<std::uint32_t>(v[3]) & 255U) << 24);
    };
    *reinterpret_cast<uint2*>(planes + (warp * 2 + 0) * 256 + lane * 8) = make_uint2(pack(hi), pack(hi + 4));
    *reinterpret_cast<uint2*>(planes + (warp * 2 + 1) * 256 + lane * 8) = make_uint2(pack(lo), pack(lo + 4));
#pragma unroll
    for (int o = 1; o <= 8; o <<= 1) {   // plane sums over the 128-dim half (16 lanes)
      sum_hi += __shfl_xor_sync(0xFFFFFFFFU, sum_hi, o);
      sum_lo += __shfl_xor_sync(0xFFFFFFFFU, sum_lo, o);
    }
    if ((lane & 15) == 0) {
      corr[(warp * 2 + (lane >> 4)) * 2 + 0] = -128 * sum_hi;
      corr[(warp * 2 + (lane >> 4)) * 2 + 1] = -128 * sum_lo;
    }
    if (lane == 0) q_step[warp] = amax / kQSteps;
  }
  __syncthreads();
  const int gq = g < kGroup ? g : g - 2;   // the two padding rows of the MMA reuse heads 4, 5
  const std::uint8_t* my_hi = planes + (gq * 2 + 0) * 256 + 32 * t;
  const std::uint8_t* my_lo = planes + (gq * 2 + 1) * 256 + 32 * t;
  int c_hi[2], c_lo[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) c_hi[hf] = corr[(gq * 2 + hf) * 2], c_lo[hf] = corr[(gq * 2 + hf) * 2 + 1];
  const float score_scale = scale_log2 * q_step[gq];

  float o_acc[16][4];
#pragma unroll
  for (int c = 0; c < 16; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[c][i] = 0.0F;
  float m_run = -INFINITY, l_run = 0.0F;

  const std::int32_t* row = tables + static_cast<std::size_t>(u.seq) * table_stride;
  const int cur_tile = (u.n_keys - 1) / kTileKeys;
  const int tile_begin = u.page_begin * kTilesPerPage;
  const int tile_end = min(u.page_end * kTilesPerPage, cur_tile + 1);
  const __half* open_buf = open_tiles + ((static_cast<std::size_t>(u.seq) * n_layers + layer) * 2 + (u.pad & 1)) * kOpenTileHalfs +
                           static_cast<std::size_t>(u.kvh) * kHeadDim * kTileKeys;

  for (int tile = tile_begin + warp; tile < tile_end; tile += kKv8Warps) {
    const bool open = tile == cur_tile;
    std::int32_t page = __ldg(row + tile / kTilesPerPage);
    page = min(max(page, 0), pool.num_pages - 1);
    const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + page) * kKvHeads + u.kvh;
    const int t_in_page = tile % kTilesPerPage;
    // Which key of the tile sits in column c of key tile kt: quantized tiles pack keys so that the V dwords unpack
    // straight into the second MMA's operand (column 2t, 2t+1 of tile 0 = keys 4t, 4t+1; of tile 1 = keys 4t+2, 4t+3);
    // the open tile is in natural order.
    auto key_of = [&](int kt, int c) { return open ? kt * 8 + c : 4 * (c >> 1) + 2 * kt + (c & 1); };
    const std::uint8_t* kbase = pool.kcodes + rec * RecordCodeBytes(kFmtKv8) + static_cast<std::size_t>(t_in_page) * kTileKeys * 256;
    const std::uint16_t* ksc = pool.kscales + rec * (RecordScaleBytes(kFmtKv8, 0) / 2) + static_cast<std::size_t>(t_in_page) * kTileKeys * 4;

    // ---- scores: per 128-dim half the integer sums of the two query planes over the unsigned codes ----
    float sc[2][2];
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) {
      const std::uint8_t* krow = kbase + key_of(kt, g) * 256 + 32 * t;   // this lane's 32 bytes of each half
      float part[2] = {0.0F, 0.0F};
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const uint4 ka = *reinterpret_cast<const uint4*>(krow + hf * 128), kb = *reinterpret_cast<const uint4*>(krow + hf * 128 + 16);
        const std::uint32_t kw[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
        int acc[4] = {c_hi[hf], c_hi[hf], c_lo[hf], c_lo[hf]};
#pragma unroll
        for (int j = 0; j < 4; ++j) {   // k-step j: this lane's bytes 8j .. 8j+7 of the half, query bytes likewise
          const uint2 qh = *reinterpret_cast<const uint2*>(my_hi + hf * 128 + 8 * j);
          const uint2 ql = *reinterpret_cast<const uint2*>(my_lo + hf * 128 + 8 * j);
          MmaS8U8Acc(acc, qh.x, ql.x, qh.y, ql.y, kw[2 * j], kw[2 * j + 1]);
        }
        // columns 2t, 2t+1 of this key tile: scale pair of their keys, first value = 256 s
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const std::uint16_t sbits = __ldg(ksc + key_of(kt, 2 * t + j) * 4 + hf * 2);
          const float sdeq = __half2float(__ushort_as_half(sbits)) * (1.0F / 256.0F);
          part[j] = fmaf(sdeq, static_cast<float>(acc[j] * 256 + acc[2 + j]), part[j]);
        }
      }
      sc[kt][0] = part[0] * score_scale, sc[kt][1] = part[1] * score_scale;
    }
    // keys past the sequence's length (only in its newest tile)
    if ((tile + 1) * kTileKeys > u.n_keys) {
#pragma unroll
      for (int kt = 0; kt < 2; ++kt)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (tile * kTileKeys + key_of(kt, 2 * t + j) >= u.n_keys) sc[kt][j] = -INFINITY;
    }
    float tmax = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFU, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFU, tmax, 2));
    if (__any_sync(0xFFFFFFFFU, g < kGroup && tmax > m_run + kLazyRescale)) {
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
    psum += __shfl_xor_sync(0xFFFFFFFFU, psum, 1);
    psum += __shfl_xor_sync(0xFFFFFFFFU, psum, 2);   // the tile's sum of weights of head g
    const float ps0 = __shfl_sync(0xFFFFFFFFU, psum, (2 * t) * 4), ps1 = __shfl_sync(0xFFFFFFFFU, psum, (2 * t + 1) * 4);

    // ---- O^T += V^T P^T ----
    if (open) {   // fp16 keys in natural order: k-slots (2t, 2t+1) = keys 2t, 2t+1; (2t+8, 2t+9) = keys 2t+8, 2t+9
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const __half* r0 = open_buf + (16 * c + g) * kTileKeys + 2 * t;
        const __half* r1 = r0 + 8 * kTileKeys;
        const std::uint32_t a0 = *reinterpret_cast<const std::uint32_t*>(r0), a1 = *reinterpret_cast<const std::uint32_t*>(r1);
        const std::uint32_t a2 = *reinterpret_cast<const std::uint32_t*>(r0 + 8), a3 = *reinterpret_cast<const std::uint32_t*>(r1 + 8);
        MmaF16(o_acc[c], a0, a1, a2, a3, p_hi[0], p_hi[1]);
        MmaF16(o_acc[c], a0, a1, a2, a3, p_lo[0], p_lo[1]);
      }
    } else {      // v = (u - 128) a + b with a = S / 256, b = 1.5 S + C' (= the tile's centre), per channel
      const std::uint8_t* vbase = pool.vcodes + rec * RecordCodeBytes(kFmtKv8) + static_cast<std::size_t>(t_in_page) * kHeadDim * 16;
      const std::uint16_t* vst = pool.vscales + rec * (RecordScaleBytes(kFmtKv8, 1) / 2) + static_cast<std::size_t>(t_in_page) * kHeadDim * 2;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const int ch0 = 16 * c + g, ch1 = ch0 + 8;
        const std::uint32_t w0 = __ldg(reinterpret_cast<const std::uint32_t*>(vbase + ch0 * 16 + 4 * t));
        const std::uint32_t w1 = __ldg(reinterpret_cast<const std::uint32_t*>(vbase + ch1 * 16 + 4 * t));
        const std::uint32_t s0 = __ldg(reinterpret_cast<const std::uint32_t*>(vst + ch0 * 2));
        const std::uint32_t s1 = __ldg(reinterpret_cast<const std::uint32_t*>(vst + ch1 * 2));
        std::uint32_t a0, a1, a2, a3;
        Offset8x4ToHalf2(w0, a0, a2);   // bytes (0, 2) = keys 4t, 4t+1;  bytes (1, 3) = keys 4t+2, 4t+3
        Offset8x4ToHalf2(w1, a1, a3);
        float d[4], e[4];
        MmaF16Zero(d, a0, a1, a2, a3, p_hi[0], p_hi[1]);
        MmaF16Zero(e, a0, a1, a2, a3, p_lo[0], p_lo[1]);
        const float2 st0 = __half22float2(*reinterpret_cast<const __half2*>(&s0));
        const float2 st1 = __half22float2(*reinterpret_cast<const __half2*>(&s1));
        const float sa0 = st0.x * (1.0F / 256.0F), sb0 = fmaf(1.5F, st0.x, st0.y);
        const float sa1 = st1.x * (1.0F / 256.0F), sb1 = fmaf(1.5F, st1.x, st1.y);
        o_acc[c][0] = fmaf(sa0, d[0] + e[0], fmaf(sb0, ps0, o_acc[c][0]));
        o_acc[c][1] = fmaf(sa0, d[1] + e[1], fmaf(sb0, ps1, o_acc[c][1]));
        o_acc[c][2] = fmaf(sa1, d[2] + e[2], fmaf(sb1, ps0, o_acc[c][2]));
        o_acc[c][3] = fmaf(sa1, d[3] + e[3], fmaf(sb1, ps1, o_acc[c][3]));
      }
    }
  }
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 1);
  l_run += __shfl_xor_sync(0xFFFFFFFFU, l_run, 2);

  __syncthreads();   // the query planes are dead: the scratch now holds the warps' results
  float* merge = reinterpret_cast<float*>(smem);
  {
    float* mine = merge + warp * kMergeWarpFloats;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      // o_acc[c][0..3] = (channel 16c + g, head 2t), (16c + g, 2t+1), (16c + g + 8, 2t), (16c + g + 8, 2t+1)
      if (2 * t < kGroup) {
        mine[(2 * t) * kMergeStride + 16 * c + g] = o_acc[c][0];
        mine[(2 * t + 1) * kMergeStride + 16 * c + g] = o_acc[c][1];
        mine[(2 * t) * kMergeStride + 16 * c + g + 8] = o_acc[c][2];
        mine[(2 * t + 1) * kMergeStride + 16 * c + g + 8] = o_acc[c][3];
      }
    }
    if (t == 0 && g < kGroup) {
      float* ml = mine + kGroup * kMergeStride;
      ml[2 * g] = m_run;
      ml[2 * g + 1] = l_run;
    }
  }
  __syncthreads();
  {
    const int tid = threadIdx.x;
    float* acc_out = partial_acc + static_cast<std::size_t>(u.partial) * kPartialAccFloats;
    float* ml_out = partial_ml + static_cast<std::size_t>(u.partial) * kPartialMlFloats;
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
      float mw[kKv8Warps], M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kKv8Warps; ++w) {
        mw[w] = merge[w * kMergeWarpFloats + kGroup * kMergeStride + 2 * h];
        M = fmaxf(M, mw[w]);
      }
      float a = 0.0F, lsum = 0.0F;
#pragma unroll
      for (int w = 0; w < kKv8Warps; ++w) {
        const float wgt = mw[w] == -INFINITY ? 0.0F : exp2f(mw[w] - M);
        const float* src = merge + w * kMergeWarpFloats;
        a = fmaf(wgt, src[h * kMergeStride + tid], a);
        lsum = fmaf(wgt, src[kGroup * kMergeStride + 2 * h + 1], lsum);
      }
      acc_out[h * kHeadDim + tid] = a;
      if (tid == 0) ml_out[2 * h] = M, ml_out[2 * h + 1] = lsum;
    }
  }
}

}  // namespace

cudaError_t ConfigureKv8Kernels() {
  return cudaFuncSetAttribute(Kv8DecodePartKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kKv8SmemBytes);
}

cudaError_t LaunchKv8AppendK(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                             const std::int32_t* state_rows_dev, const float* kmean_dev, const void* k_dev,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return cudaSuccess;
  return LaunchChained(Kv8AppendKKernel, n_tokens, 128, 0, stream, pool, layer, slots_dev, state_rows_dev, kmean_dev,
                       static_cast<const __half*>(k_dev));
}

cudaError_t LaunchKv8AppendV(const PoolView& pool, int layer, int n_work, const VTileWork* work_dev, void* open_tiles_dev,
                             const void* v_dev, cudaStream_t stream) {
  if (n_work <= 0) return cudaSuccess;
  return LaunchChained(Kv8AppendVKernel, dim3(n_work, kKvHeads), kHeadDim, 0, stream, pool, layer, work_dev,
                       static_cast<__half*>(open_tiles_dev), static_cast<const __half*>(v_dev));
}

cudaError_t LaunchKv8DecodePart(const DecodeLaunch& a, const void* open_tiles_dev, int n_layers, cudaStream_t stream) {
  if (a.n_units <= 0 || a.n_seqs <= 0) return cudaSuccess;
  return LaunchChained(Kv8DecodePartKernel, a.n_units, kKv8Threads, kKv8SmemBytes, stream, a.pool, a.layer, a.tables_dev,
                       a.table_stride, a.units_dev, static_cast<const __half*>(a.q_dev), a.scale_log2,
                       static_cast<const __half*>(open_tiles_dev), n_layers, a.partial_acc, a.partial_ml);
}

}  // namespace yahkv
