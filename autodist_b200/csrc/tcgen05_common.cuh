// Device helpers shared by the tcgen05 kernels (GEMM, convolution): mbarrier waits with a limit, TMA tile loads,
// shared-memory matrix descriptors, tcgen05.mma / commit / ld wrappers and the small vector load/store helpers.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace adb200 {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr long long kWaitLimitCycles = 100000000LL;    // ~50 ms at 1.9 GHz: no legitimate wait is longer


__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the limit ran out or another role of this CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Shared-memory matrix descriptor (sm_100 form, 128-byte swizzle).
//   K-major : rows of 128 bytes, groups of 8 rows 1024 bytes apart (SBO); LBO unused.
//   MN-major: chunks of 64 elements along M/N; inside a chunk 8-row groups along K are 1024 bytes apart (SBO),
//             chunks are BK*128 bytes apart (LBO).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;    // descriptor version of sm_100
  d |= (uint64_t)2 << 61;    // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ uint32_t make_idesc(int n, bool a_mn, bool b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;                       // D format: f32
  d |= 1u << 7;                       // A format: bf16
  d |= 1u << 10;                      // B format: bf16
  d |= (a_mn ? 1u : 0u) << 15;        // A major
  d |= (b_mn ? 1u : 0u) << 16;        // B major
  d |= (uint32_t)(n >> 3) << 17;      // N / 8
  d |= (uint32_t)(BM >> 4) << 24;     // M / 16
  return d;
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Dropout decisions: the same counter-based function as the layernorm / softmax kernels (elementwise.cu), so a mask
// drawn in a fused epilogue is reproduced by any other kernel from (seed, element offset).
__device__ __forceinline__ uint64_t mix64(uint64_t seed, uint64_t idx) {
  uint64_t x = seed + idx * 0x9E3779B97F4A7C15ull;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}
__device__ __forceinline__ void keep_scale8(uint64_t seed, uint64_t base, uint32_t thresh16, float inv_keep, float* out) {
  const uint64_t h0 = mix64(seed, base >> 2), h1 = mix64(seed, (base >> 2) + 1);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    out[j] = (((uint32_t)(h0 >> (16 * j)) & 0xFFFFu) >= thresh16) ? inv_keep : 0.0f;
    out[4 + j] = (((uint32_t)(h1 >> (16 * j)) & 0xFFFFu) >= thresh16) ? inv_keep : 0.0f;
  }
}
__device__ __forceinline__ void store8_bf16(__nv_bfloat16* dst, const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void unpack8_bf16(const uint4& u, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
}
__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* src, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
}

// tanh on the special-function unit (one instruction, relative error about 2^-11: below the rounding of the bf16 values
// the epilogues produce). The epilogue threads are the scarce resource of a GEMM with a fused activation: 128 threads
// per tile of 32768 outputs.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  const float t = tanh_fast(k * fmaf(0.044715f * x * x, x, x));
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float x2 = x * x;
  const float t = tanh_fast(k * fmaf(0.044715f * x2, x, x));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k * fmaf(3.0f * 0.044715f, x2, 1.0f);
}

}  // namespace tc
}  // namespace adb200
