// Thin wrappers over the sm_100a PTX this library uses: mbarriers, bulk-async (TMA) copies, ldmatrix and the
// register-operand f16 MMA. Every wait is bounded: a wait that gives up returns false and the caller records an error
// status instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace yahkv {

__device__ __forceinline__ std::uint32_t SmemAddr(const void* p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void MbarInit(std::uint64_t* bar, std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void FenceBarrierInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void MbarArrive(std::uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ void MbarArriveExpectTx(std::uint64_t* bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(std::uint64_t* bar, std::uint32_t parity) {
  std::uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(SmemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ std::uint64_t GlobalTimerNs() {
  std::uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the barrier's phase `parity` to complete, for at most `limit_ns` (about two seconds unless the caller
// says otherwise). The reference bounds its device-side polls the same way and leaves a sticky status behind
// (engine/gpu/loom/tools/gen_chain.py:12-19).
constexpr std::uint64_t kWaitLimitNs = 2000000000ULL;
__device__ __forceinline__ bool MbarWait(std::uint64_t* bar, std::uint32_t parity,
                                         std::uint64_t limit_ns = kWaitLimitNs) {
  if (MbarTryWait(bar, parity)) return true;
  const std::uint64_t t0 = GlobalTimerNs();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (MbarTryWait(bar, parity)) return true;
    if (GlobalTimerNs() - t0 > limit_ns) return false;
  }
}

// Programmatic dependent launch. A kernel launched with LaunchChained (kernels.cuh) may start while the kernel before
// it in the stream is still running; ChainedKernelEntry, first thing in the kernel, lets the NEXT kernel be scheduled
// as soon as every CTA of this one has started, then waits until the kernels before have completed and their writes
// are visible. Nothing is read or written before it, so the result is that of a plain stream; what overlaps is the
// launch latency and block scheduling of consecutive small kernels. After a plain launch both are no-ops.
__device__ __forceinline__ void ChainedKernelEntry() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// True in exactly one lane of a fully converged warp (all 32 lanes must execute it).
__device__ __forceinline__ bool ElectOne() {
  std::uint32_t e;
  asm volatile("{ .reg .pred P; elect.sync _|P, 0xffffffff; selp.u32 %0, 1, 0, P; }" : "=r"(e));
  return e != 0;
}

// 2-D tiled TMA load (no multicast): box at (x, y) of the tensor map into this CTA's shared memory.
__device__ __forceinline__ void TmaLoad2D(void* smem_dst, const CUtensorMap* map, int x, int y, std::uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          SmemAddr(smem_dst)),
      "l"(reinterpret_cast<std::uint64_t>(map)), "r"(x), "r"(y), "r"(SmemAddr(bar))
      : "memory");
}
// ---- CTA pairs (thread-block clusters of two) ----
__device__ __forceinline__ std::uint32_t ClusterCtaRank() {
  std::uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of the same shared-memory location in the CTA of rank `cta_rank` of this cluster.
__device__ __forceinline__ std::uint32_t MapToCta(std::uint32_t smem_addr, std::uint32_t cta_rank) {
  std::uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
// Cluster-wide barrier of all threads of all CTAs, with release / acquire ordering of shared memory across the CTAs.
__device__ __forceinline__ void ClusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier given by its shared::cluster address (this CTA's or the peer's). Default semantics (release
// at CTA scope): a release at cluster scope cost ~1,300 clocks per arrival here. What the arrivals of this library
// order across the pair is tensor-memory and async-proxy traffic, which tcgen05.fence / fence.proxy.async before the
// arrival order; no generic-proxy data crosses between the CTAs.
__device__ __forceinline__ void MbarArriveCluster(std::uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// try_wait on a barrier of this CTA that the peer arrives on: acquires at cluster scope.
__device__ __forceinline__ bool MbarTryWaitCluster(std::uint64_t* bar, std::uint32_t parity) {
  std::uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(SmemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// 2-D tiled TMA load (no multicast) for a CTA pair: the box lands in this CTA's shared memory, the bytes are counted
// on the barrier at `bar_cluster_addr`, which may belong to the other CTA of the pair.
__device__ __forceinline__ void TmaLoad2DPair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                              std::uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];" ::"r"(SmemAddr(smem_dst)),
      "l"(reinterpret_cast<std::uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void BulkLoad(void* smem_dst, const void* gsrc, std::uint32_t bytes, std::uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   SmemAddr(smem_dst)),
               "l"(reinterpret_cast<std::uint64_t>(gsrc)), "r"(bytes), "r"(SmemAddr(bar))
               : "memory");
}
__device__ __forceinline__ void PrefetchTensorMap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<std::uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void LdMatrixX4(std::uint32_t addr, std::uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void LdMatrixX4Trans(std::uint32_t addr, std::uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void MmaF16(float (&d)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                       std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void NamedBarrierSync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// 2^x on the special-function unit, one instruction (flush-to-zero; exact powers of two for integer x, -inf -> 0).
__device__ __forceinline__ float Exp2Fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Four q8_0 codes as the pools hold them (u = code + 128 per byte) -> two half2 of exact integers: bytes (0, 2) and
// bytes (1, 3). 0x6400 | u is the fp16 value 1024 + u, so the code is that minus 1152.
__device__ __forceinline__ void Offset8x4ToHalf2(std::uint32_t u, std::uint32_t& h02, std::uint32_t& h13) {
  const std::uint32_t lo = __byte_perm(u, 0x64646464U, 0x4240);
  const std::uint32_t hi = __byte_perm(u, 0x64646464U, 0x4341);
  const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
  const __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias);
  const __half2 b = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
  h02 = *reinterpret_cast<const std::uint32_t*>(&a);
  h13 = *reinterpret_cast<const std::uint32_t*>(&b);
}
// Four packed q4_0 bytes -> the unsigned bytes 16 n of their low nibbles (byte order kept) and of their high
// nibbles: a nibble moved to the top of its byte. Three instructions, each with one immediate.
__device__ __forceinline__ void Nib8ToU8(std::uint32_t w, std::uint32_t& lo, std::uint32_t& hi) {
  lo = (w << 4) & 0xF0F0F0F0U;
  hi = w & 0xF0F0F0F0U;
}
// d = (a & b) ^ c as one logic instruction with all three inputs in registers.
__device__ __forceinline__ std::uint32_t AndXor(std::uint32_t a, std::uint32_t b, std::uint32_t c) {
  std::uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// The same nibbles as the SIGNED bytes 16 (n - 8): the nibble at the top of its byte with the byte's sign bit
// flipped, so that the q4_0 offset costs nothing and the codes enter the s8 x s8 MMA with a zero accumulator.
// Three instructions (a shift and two and-xor) given the mask 0xF0F0F0F0 and the flip 0x80808080 in registers.
__device__ __forceinline__ void Nib8ToS8(std::uint32_t mask, std::uint32_t flip, std::uint32_t w, std::uint32_t& lo,
                                         std::uint32_t& hi) {
  lo = AndXor(w << 4, mask, flip);
  hi = AndXor(w, mask, flip);
}
// d = (a & b) | c as ONE logic instruction with all three inputs in registers. Written as a & imm | imm the compiler
// must split it (an instruction carries one immediate), which doubles the cost of every nibble conversion.
__device__ __forceinline__ std::uint32_t AndOr(std::uint32_t a, std::uint32_t b, std::uint32_t c) {
  std::uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// The three constants of the nibble conversion, held in registers the compiler cannot turn back into immediates.
struct NibConsts {
  std::uint32_t lo_mask, hi_mask, magic, top_mask, sign_flip;
  __device__ __forceinline__ void Load() {
    asm volatile("mov.u32 %0, 0x000F000F;" : "=r"(lo_mask));
    asm volatile("mov.u32 %0, 0x00F000F0;" : "=r"(hi_mask));
    asm volatile("mov.u32 %0, 0x64006400;" : "=r"(magic));
    asm volatile("mov.u32 %0, 0xF0F0F0F0;" : "=r"(top_mask));
    asm volatile("mov.u32 %0, 0x80808080;" : "=r"(sign_flip));
  }
};
// Four packed q4_0 bytes -> low nibbles of bytes (0,2), (1,3) and high nibbles of bytes (0,2), (1,3), each minus 8.
__device__ __forceinline__ void Nib4x4ToHalf2(const NibConsts& k, std::uint32_t w, std::uint32_t& l02,
                                              std::uint32_t& l13, std::uint32_t& h02, std::uint32_t& h13) {
  // Low nibbles: 0x6400 | n is the fp16 1024 + n, minus 1032. High nibbles stay where they are: 0x6400 | (n << 4) is
  // 1024 + 16 n, and (1024 + 16 n) / 16 - 72 = n - 8 in one exact fma, which saves the two shifts by 4.
  const __half2 bias = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));  // 1032
  const __half2 sixteenth = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));  // 1 / 16
  const __half2 bias_hi = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));    // -72
  const std::uint32_t w8 = w >> 8;
  const std::uint32_t a = AndOr(w, k.lo_mask, k.magic);
  const std::uint32_t b = AndOr(w8, k.lo_mask, k.magic);
  const std::uint32_t c = AndOr(w, k.hi_mask, k.magic);
  const std::uint32_t d = AndOr(w8, k.hi_mask, k.magic);
  const __half2 ra = __hsub2(*reinterpret_cast<const __half2*>(&a), bias);
  const __half2 rb = __hsub2(*reinterpret_cast<const __half2*>(&b), bias);
  const __half2 rc = __hfma2(*reinterpret_cast<const __half2*>(&c), sixteenth, bias_hi);
  const __half2 rd = __hfma2(*reinterpret_cast<const __half2*>(&d), sixteenth, bias_hi);
  l02 = *reinterpret_cast<const std::uint32_t*>(&ra);
  l13 = *reinterpret_cast<const std::uint32_t*>(&rb);
  h02 = *reinterpret_cast<const std::uint32_t*>(&rc);
  h13 = *reinterpret_cast<const std::uint32_t*>(&rd);
}

}  // namespace yahkv
