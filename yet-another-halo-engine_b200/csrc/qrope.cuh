// The head RMS norm + NeoX RoPE of the reference's "rope" kernel (QK RMSNorm, rotary on 64 of 256 dims, theta 1e7:
// engine/gpu/loom/yah_fused_qk_rope_f32.loom:1-9, :32) as a warp-level function, shared by the fused append kernel
// (kv_append.cu) and by the decode kernels that take the raw f32 query (the attend-side half of that fusion).
#pragma once

#include <cuda_fp16.h>

#include "kernels.cuh"

namespace yahkv {

constexpr int kHalfRot = 32;   // rotary_dim 64: dim p pairs with p + 32

// One head row [256] f32 over a converged warp, lane l holding dims 8 l .. 8 l + 7 in x: x <- norm(x) * weight, then
// rotated at `pos`. The sum of squares is a chain of eight fmas per lane joined by an xor butterfly (16, 8, 4, 2, 1);
// every product and sum is rounded on its own (no contraction), so the result does not depend on the compiler.
// rope_tab holds (cos, sin) [rope_rows][32]; pos is clamped to the table.
__device__ __forceinline__ void NormRopeLane8(float (&x)[8], const float* __restrict__ weight, float eps,
                                              const float2* __restrict__ rope_tab, int rope_rows, int pos, int lane) {
  float acc = 0.0F;
#pragma unroll
  for (int j = 0; j < 8; ++j) acc = fmaf(x[j], x[j], acc);
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFU, acc, m));
  const float inv = __fdiv_rn(1.0F, __fsqrt_rn(__fadd_rn(__fmul_rn(acc, 1.0F / kHeadDim), eps)));
  const float* wp = weight + lane * 8;
  const float4 wa = *reinterpret_cast<const float4*>(wp), wb = *reinterpret_cast<const float4*>(wp + 4);
  const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = __fmul_rn(__fmul_rn(x[j], inv), w[j]);
  // dims 0 .. 63 sit in lanes 0 .. 7; dim p pairs with p + 32, i.e. lane l with lane l ^ 4, same j
  pos = min(max(pos, 0), rope_rows - 1);
  const float2* cs_row = rope_tab + static_cast<std::size_t>(pos) * kHalfRot + (lane & 3) * 8;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float other = __shfl_xor_sync(0xFFFFFFFFU, x[j], 4);
    if (lane < 8) {
      const float2 cs = cs_row[j];
      x[j] = lane < 4 ? __fsub_rn(__fmul_rn(x[j], cs.x), __fmul_rn(other, cs.y))
                      : __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(x[j], cs.x));
    }
  }
}

// This lane's eight dims (8 lane .. 8 lane + 7) of one query head as fp16, the form every decode kernel's prologue
// starts from: read from the fp16 query tensor, or (kQRaw) made from the raw f32 row at position `pos` with the bits
// the fused append kernel writes to its q output. Whole converged warp.
template <bool kQRaw>
__device__ __forceinline__ uint4 LoadQueryLane8(const __half* __restrict__ q16, const QueryRaw& qr, std::size_t head_row,
                                                int pos, int lane) {
  if constexpr (kQRaw) {
    const float* src = qr.q + head_row * kHeadDim + lane * 8;
    const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
    float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    NormRopeLane8(x, qr.weight, qr.eps, qr.rope_tab, qr.rope_rows, pos, lane);
    __half2 hx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) hx[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
    return *reinterpret_cast<const uint4*>(hx);
  } else {
    return *reinterpret_cast<const uint4*>(q16 + head_row * kHeadDim + 8 * lane);
  }
}

}  // namespace yahkv
