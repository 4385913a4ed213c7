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

namespace yahkv {
namespace {

constexpr int kAppendThreads = 256;  // 8 warps = 2 sides x 4 kv heads of one token

template <int kFmt>
__global__ void __launch_bounds__(kAppendThreads) AppendKernel(PoolView pool, int layer,
                                                               const std::int64_t* __restrict__ slots,
                                                               const __half* __restrict__ k_in,
                                                               const __half* __restrict__ v_in) {
  const int token = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int side = warp >> 2, h = warp & 3;
  const std::int64_t slot = slots[token];
  if (slot < 0) return;  // padding token
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

  const std::size_t rec = (static_cast<std::size_t>(layer) * pool.num_pages + static_cast<std::size_t>(page)) * kKvHeads + h;
  std::uint8_t* codes = (side == 0 ? pool.kcodes : pool.vcodes) + rec * RecordCodeBytes(kFmt) +
                        static_cast<std::size_t>(tok) * CodeBytes(kFmt);
  std::uint16_t* scales = (side == 0 ? pool.kscales : pool.vscales) + rec * (kPageTokens * kBlocksPerRow) +
                          static_cast<std::size_t>(tok) * kBlocksPerRow;
  const int blk = lane >> 2, sub = lane & 3;

  if constexpr (kFmt == kFmtQ8) {
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
    *reinterpret_cast<uint2*>(codes + lane * 8) = make_uint2(w[0], w[1]);
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

}  // namespace

cudaError_t LaunchAppend(const PoolView& pool, int layer, int n_tokens, const std::int64_t* slots_dev,
                         const void* k_dev, const void* v_dev, cudaStream_t stream) {
  if (n_tokens <= 0) return cudaSuccess;
  const auto* k = static_cast<const __half*>(k_dev);
  const auto* v = static_cast<const __half*>(v_dev);
  if (pool.fmt == kFmtQ8)
    AppendKernel<kFmtQ8><<<n_tokens, kAppendThreads, 0, stream>>>(pool, layer, slots_dev, k, v);
  else
    AppendKernel<kFmtQ4><<<n_tokens, kAppendThreads, 0, stream>>>(pool, layer, slots_dev, k, v);
  return cudaGetLastError();
}

}  // namespace yahkv
