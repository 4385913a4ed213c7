// KV append: quantize fp16 K/V token rows into GGUF-style 32-element blocks and scatter them into the paged pools.
//
// Stands in for the reference's dattn_kvappend / dattn_kappend_q / dattn_vappend_q (decode, one token) and
// yah_kq8 / yah_vq8 (prefill chunk): engine/gpu/loom/tools/gen_decode_attn.py:30-94, :1043-1107, :436-573 and
// engine/gpu/loom/tools/gen_kvq.py:166-285, :474-581. The block arithmetic is the reference's CPU codec,
// engine/core/gguf_quant.cpp:310-320 (QuantizeQ8_0), reproduced bit for bit:
//   d = amax / 127 (IEEE f32 divide), inv = 1 / d (0 when d == 0), code = lround(x * inv) (ties away from zero),
//   stored scale = half(d) rounded to nearest even; codes come from the f32 inv, not from the rounded scale.
// q4_0 follows ggml's quantizer (the reference only decodes q4_0, engine/core/gguf_quant.cpp:48-51): the value of
// largest magnitude (first on ties) maps to -8, d = max / -8, nibble = min(15, trunc(x / d + 8.5)), byte j of a block
// = element j (low nibble) | element j + 16 (high nibble).
//
// One warp handles one (token, side, kv head) row of 256 values: lane l holds elements 8l .. 8l+7, so a block is four
// neighbouring lanes. Loads are 16 B per lane (512 B per warp, coalesced), code stores 8 B per lane (q8_0) and the
// row's eight scales are written by the first lane of each block. HBM-bound: 4096 B read + 2176 B (q8_0) or 1152 B
// (q4_0) written per token per layer.
#include <cuda_fp16.h>

#include "kernels.cuh"
#include "ptx.cuh"
#include "qrope.cuh"

namespace yahkv {
namespace {

constexpr int kAppendThreads = 256;  // 8 warps = 2 sides x 4 kv heads of one token

// Quantizes one (token, side, kv head) row held by a warp (lane l: elements 8l .. 8l+7, already exact fp16 values
// widened to f32) and stores codes and scales at the token's place in its page record.
template <int kFmt>
__device__ __forceinline__ void QuantizeStoreRow(const PoolView& pool, int layer, std::int64_t page, int tok, int side,
                                                 int h, int lane, const float (&x)[8]) {
  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + static_cast<std::size_t>(page)) * kKvHeads + h;
  std::uint8_t* codes = (side == 0 ? pool.kcodes : pool.vcodes) + rec * RecordCodeBytes(kFmt) +
                        static_cast<std::size_t>(tok) * CodeBytes(kFmt);
  std::uint16_t* scales = (side == 0 ? pool.kscales : pool.vscales) + rec * (kPageTokens * kBlocksPerRow) +
                          static_cast<std::size_t>(tok) * kBlocksPerRow;
  const int blk = lane >> 2, sub = lane & 3;

  if constexpr (kFmt == kFmtF16) {   // fp16 pages: the row as it came (x holds fp16 values exactly)
    __half2 hx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) hx[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
    *reinterpret_cast<uint4*>(codes + lane * 16) = *reinterpret_cast<const uint4*>(hx);
    (void)scales, (void)blk, (void)sub;
  } else if constexpr (kFmt == kFmtQ8) {
    float amax = 0.0F;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFU, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFU, amax, 2));
    const float d = __fdiv_rn(amax, 127.0F);
    const float inv = d > 0.0F ? __fdiv_rn(1.0F, d) : 0.0F;
    std::uint32_t w[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = static_cast<int>(roundf(__fmul_rn(x[i], inv)));  // roundf: halfway cases away from zero = lround
      w[i >> 2] |= (static_cast<std::uint32_t>(q) & 0xFFU) << (8 * (i & 3));
    }
    // the pools' device representation of q8_0 codes: K as it is, V with the sign bits flipped
    const std::uint32_t flip = Q8FlipWord(side);
    *reinterpret_cast<uint2*>(codes + lane * 8) = make_uint2(w[0] ^ flip, w[1] ^ flip);
    if (sub == 0) scales[blk] = __half_as_ushort(__float2half_rn(d));
  } else {
    // Largest magnitude of the block with its sign, first occurrence on ties.
    float amax = 0.0F, mx = 0.0F;
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = fabsf(x[i]);
      if (a > amax) amax = a, mx = x[i], idx = sub * 8 + i;
    }
#pragma unroll
    for (int off = 1; off <= 2; off <<= 1) {
      const float a2 = __shfl_xor_sync(0xFFFFFFFFU, amax, off);
      const float m2 = __shfl_xor_sync(0xFFFFFFFFU, mx, off);
      const int i2 = __shfl_xor_sync(0xFFFFFFFFU, idx, off);
      if (a2 > amax || (a2 == amax && a2 > 0.0F && i2 < idx)) amax = a2, mx = m2, idx = i2;
    }
    const float d = __fdiv_rn(mx, -8.0F);
    const float id = d != 0.0F ? __fdiv_rn(1.0F, d) : 0.0F;
    std::uint32_t nib = 0;  // nibble i of this lane's eight elements at bits 4i
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = min(15, static_cast<int>(__fadd_rn(__fmul_rn(x[i], id), 8.5F)));
      nib |= static_cast<std::uint32_t>(q) << (4 * i);
    }
    // Elements j and j + 16 share a byte: lanes sub 0 / 1 pair with lanes sub 2 / 3.
    const std::uint32_t hi = __shfl_down_sync(0xFFFFFFFFU, nib, 2);
    if (sub < 2) {
      std::uint32_t w[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const std::uint32_t b = ((nib >> (4 * i)) & 0xFU) | (((hi >> (4 * i)) & 0xFU) << 4);
        w[i >> 2] |= b << (8 * (i & 3));
      }
      *reinterpret_cast<uint2*>(codes + blk * 16 + sub * 8) = make_uint2(w[0], w[1]);
    }
    if (sub == 0) scales[blk] = __half_as_ushort(__float2half_rn(d));
  }
}

template <int kFmt>
__global__ void __launch_bounds__(kAppendThreads) AppendKernel(PoolView pool, int layer,
                                                               const std::int64_t* __restrict__ slots,
                                                               const __half* __restrict__ k_in,
                                                               const __half* __restrict__ v_in) {
  ChainedKernelEntry();
  const int token = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int side = warp >> 2, h = warp & 3;
  const std::int64_t slot = slots[token];
  if (slot < 0 || !pool.OwnsKvHead(h)) return;  // padding token, or a head another context holds
  // Writers clamp the page into the pool instead of trusting the mapping (gen_decode_attn.py:59-69).
  std::int64_t page = slot / kPageTokens;
  const int tok = static_cast<int>(slot % kPageTokens);
  page = min(max(page, static_cast<std::int64_t>(0)), static_cast<std::int64_t>(pool.num_pages - 1));

  const __half* src = (side == 0 ? k_in : v_in) + (static_cast<std::size_t>(token) * kKvHeads + h) * kHeadDim;
  const uint4 raw = *reinterpret_cast<const uint4*>(src + lane * 8);
  const __half2* hp = reinterpret_cast<const __half2*>(&raw);
  float x[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(hp[i]);
    x[2 * i] = f.x, x[2 * i + 1] = f.y;
  }

  QuantizeStoreRow<kFmt>(pool, layer, page, tok, side, h, lane, x);
}


// ----------------------------------------------------------------------------------------------------------------
// Fused QK RMSNorm + NeoX RoPE + append: the reference's "rope" kernel followed by its K and V appends
// (engine/gpu/loom/yah_fused_qk_rope_f32.loom:1-9, engine/model/loom_decoder.hpp:250-261) in one launch.
//   inv_rms = 1 / sqrt(sum_i x[i]^2 / 256 + eps);  normed[i] = (x[i] * inv_rms) * weight[i]
//   p < 32: out[p] = normed[p] cos - normed[p + 32] sin;  out[p + 32] = normed[p] sin + normed[p + 32] cos
//   with angle = pos / theta^(2 p / 64), theta = 1e7; dims 64 .. 255 pass through.
// One warp per head of one token: 24 query heads (written as fp16 for the attention), 4 K heads (normed, rotated,
// rounded to fp16, quantized, scattered) and 4 V heads (rounded to fp16, quantized, scattered). Every f32 operation
// is a single IEEE operation in a fixed order (no contraction, sum of squares as a per-lane fma chain followed by a
// butterfly), and cos / sin come from a table computed on the host in double precision, so the CPU restatement
// reproduces the bits.
// ----------------------------------------------------------------------------------------------------------------
constexpr int kRopeThreads = 32 * (kQHeads + 2 * kKvHeads);

template <int kFmt>
__global__ void __launch_bounds__(kRopeThreads)
    RopeAppendKernel(PoolView pool, int layer, const std::int64_t* __restrict__ slots,
                     const std::int32_t* __restrict__ positions, const float* __restrict__ q_in,
                     const float* __restrict__ k_in, const float* __restrict__ v_in, const float* __restrict__ q_weight,
                     const float* __restrict__ k_weight, float eps, const float2* __restrict__ rope_tab, int rope_rows,
                     __half* __restrict__ q_out, __half* __restrict__ kv16_out) {
  const int token = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool is_q = warp < kQHeads, is_v = warp >= kQHeads + kKvHeads;
  const int h = is_q ? warp : (warp - kQHeads) & (kKvHeads - 1);
  const float* src = is_q ? q_in + (static_cast<std::size_t>(token) * kQHeads + h) * kHeadDim
                          : (is_v ? v_in : k_in) + (static_cast<std::size_t>(token) * kKvHeads + h) * kHeadDim;
  float x[8];
  {
    const float4 a = *reinterpret_cast<const float4*>(src + lane * 8);
    const float4 b = *reinterpret_cast<const float4*>(src + lane * 8 + 4);
    x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
  }
  if (!is_v) NormRopeLane8(x, is_q ? q_weight : k_weight, eps, rope_tab, rope_rows, positions[token], lane);
  __half2 hx[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) hx[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
  if (is_q) {
    if (q_out == nullptr || !pool.OwnsKvHead(h / kGroup)) return;   // no q output asked for; heads of another context
    *reinterpret_cast<uint4*>(q_out + (static_cast<std::size_t>(token) * kQHeads + h) * kHeadDim + lane * 8) =
        *reinterpret_cast<const uint4*>(hx);
    return;
  }
  if constexpr (kFmt == kFmtKv8) {
    // The tile formats quantize K against a mean and V per 16-key tile: this kernel leaves the fp16 rows (K after
    // norm and RoPE) in a scratch, [2 sides][tokens][4][256], and the format's own append kernels take them from there.
    __half* dst = kv16_out + ((static_cast<std::size_t>(is_v ? gridDim.x : 0) + token) * kKvHeads + h) * kHeadDim + lane * 8;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(hx);
    return;
  } else {
    const std::int64_t slot = slots[token];
    if (slot < 0 || !pool.OwnsKvHead(h)) return;  // padding token, or a head another context holds
    std::int64_t page = slot / kPageTokens;
    const int tok = static_cast<int>(slot % kPageTokens);
    page = min(max(page, static_cast<std::int64_t>(0)), static_cast<std::int64_t>(pool.num_pages - 1));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(hx[i]);
      x[2 * i] = f.x, x[2 * i + 1] = f.y;
    }
    QuantizeStoreRow<kFmt>(pool, layer, page, tok, is_v ? 1 : 0, h, lane, x);
  }
}

}  // namespace

cudaError_t LaunchAppend(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                         const void* k_dev, const void* v_dev, cudaStream_t stream) {
  if (n_tokens <= 0) return cudaSuccess;
  const auto* k = static_cast<const __half*>(k_dev);
  const auto* v = static_cast<const __half*>(v_dev);
  if (pool.fmt == kFmtQ8)
    return LaunchChained(AppendKernel<kFmtQ8>, n_tokens, kAppendThreads, 0, stream, pool, layer, slots_dev, k, v);
  if (pool.fmt == kFmtF16)
    return LaunchChained(AppendKernel<kFmtF16>, n_tokens, kAppendThreads, 0, stream, pool, layer, slots_dev, k, v);
  return LaunchChained(AppendKernel<kFmtQ4>, n_tokens, kAppendThreads, 0, stream, pool, layer, slots_dev, k, v);
}

cudaError_t LaunchRopeAppend(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                             const std::int32_t* positions_dev, const float* q_dev, const float* k_dev,
                             const float* v_dev, const float* q_weight_dev, const float* k_weight_dev, float eps,
                             const float2* rope_tab_dev, int rope_rows, void* q_out_dev, void* kv16_out_dev,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return cudaSuccess;
  auto* qo = static_cast<__half*>(q_out_dev);
  auto* kv = static_cast<__half*>(kv16_out_dev);
  if (IsTileFmt(pool.fmt))
    RopeAppendKernel<kFmtKv8><<<n_tokens, kRopeThreads, 0, stream>>>(pool, layer, slots_dev, positions_dev, q_dev, k_dev,
                                                                     v_dev, q_weight_dev, k_weight_dev, eps, rope_tab_dev,
                                                                     rope_rows, qo, kv);
  else if (pool.fmt == kFmtF16)
    RopeAppendKernel<kFmtF16><<<n_tokens, kRopeThreads, 0, stream>>>(pool, layer, slots_dev, positions_dev, q_dev, k_dev,
                                                                     v_dev, q_weight_dev, k_weight_dev, eps, rope_tab_dev,
                                                                     rope_rows, qo, kv);
  else if (pool.fmt == kFmtQ8)
    RopeAppendKernel<kFmtQ8><<<n_tokens, kRopeThreads, 0, stream>>>(pool, layer, slots_dev, positions_dev, q_dev, k_dev,
                                                                    v_dev, q_weight_dev, k_weight_dev, eps, rope_tab_dev,
                                                                    rope_rows, qo, kv);
  else
    RopeAppendKernel<kFmtQ4><<<n_tokens, kRopeThreads, 0, stream>>>(pool, layer, slots_dev, positions_dev, q_dev, k_dev,
                                                                    v_dev, q_weight_dev, k_weight_dev, eps, rope_tab_dev,
                                                                    rope_rows, qo, kv);
  return cudaGetLastError();
}

}  // namespace yahkv
