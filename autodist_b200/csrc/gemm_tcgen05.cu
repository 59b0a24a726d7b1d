// Batched bf16 GEMM on the 5th-generation tensor cores (sm_100a): D[b][M,N] = A[b][M,K] * B[b][N,K]^T.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0    TMA producer   cp.async.bulk.tensor (4-D tiled maps, 128-byte swizzle) into a ring of smem stages
//   warp 1    MMA issuer     one lane issues tcgen05.mma (cta_group::1, kind::f16, 128 x BN x 16), accumulators in TMEM
//   warps 2-5 epilogue       tcgen05.ld of the accumulator (two TMEM buffers, so tile i+1 is multiplied while tile i
//                            is written), fused bias / GELU / GELU-derivative / scale, direct 32-byte row stores
//
// Either operand may be K-major (contraction dimension contiguous in memory) or MN-major (the M or N dimension
// contiguous): the backward GEMMs of a linear layer (dX = dY W, dW = dY^T X) and of attention read the same
// tensors as the forward pass without a transpose kernel.
//
// Every mbarrier wait is bounded: when a wait gives up the CTA records an error code in `error_flag`, lets its own
// TMA copies land, frees its TMEM and returns, so a bad launch cannot hang the device.
//
// The reference has no counterpart: its matmuls are TensorFlow/cuBLAS library calls
// (examples/benchmark/utils/modeling/layers/dense_einsum.py:185-191).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_tcgen05.h"
#include "pdl.cuh"
#include "gemm_epilogue.cuh"
#include "tcgen05_common.cuh"

namespace adb200 {
namespace {

using namespace tc;

template <int BN> struct Cfg {
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGES = (BN == 256) ? 3 : (BN == 128 ? 6 : 8);
  // Epilogue warps: four cover the TMEM lane quarters; the widest tile has eight, two per quarter with half of the
  // columns each, because 128 threads cannot apply a bias or an activation to 32768 outputs in the time of one tile.
  static constexpr int EPI_WARPS = (BN == 256) ? 8 : 4;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int CW = BN / (EPI_WARPS / 4);          // columns per epilogue warp
  static constexpr int TMEM_COLS = 2 * BN;              // double-buffered fp32 accumulator
  // TMA-store staging (widest tile only): one 4 KB buffer per epilogue warp. The whole CTA stays near 208 KB so that the
  // blocks of a small kernel launched behind it (programmatic dependent launch) still fit beside it on the SM.
  static constexpr int STAGING = (BN == 256) ? EPI_WARPS * 4096 : 0;
  static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + STAGING + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(Cfg<BN>::THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ TmapArray tmBs, const __grid_constant__ CUtensorMap tmC,
            const __grid_constant__ CUtensorMap tmC2, const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + C::STAGES * A_BYTES;
  uint8_t* staging = smem + C::STAGES * (A_BYTES + C::B_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::STAGING);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull[s], 1); mbar_init(&tempty[s], 32 * C::EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync();       // everything above touched only this CTA's shared and tensor memory; global memory is read from here on

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int per_batch = tiles_m * tiles_n;
  const long long total = (long long)per_batch * p.batch_lo * p.batch_hi;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (long long t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int b = (int)(t / per_batch), rem = (int)(t % per_batch);
        const int tn = rem / tiles_m, tm = rem % tiles_m;
        const int b_lo = b % p.batch_lo, b_hi = b / p.batch_lo;
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[stage], A_BYTES + C::B_BYTES);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * C::B_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_4d(a_dst + j * (BK * 128), &tmA, &full[stage], m0 + 64 * j, k0, b_lo, b_hi);
          } else {
            tma_load_4d(a_dst, &tmA, &full[stage], k0, m0, b_lo, b_hi);
          }
          // Row-sharded B: the rows of the stored matrix live in their owners' memories; each shard's map addresses that peer
          // directly. K-major B stores [N, K] (a tile's N rows come from one owner), MN-major B stores [K, N] (a K block's
          // 64 rows come from one owner).
          if (B_MN) {
            const int shard = p.b_shard_rows > 0 ? k0 / p.b_shard_rows : 0;
            const int kl = k0 - shard * p.b_shard_rows;
            const CUtensorMap* tmB = &tmBs.m[shard];
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_4d(b_dst + j * (BK * 128), tmB, &full[stage], n0 + 64 * j, kl, b_lo, b_hi);
          } else {
            const int shard = p.b_shard_rows > 0 ? n0 / p.b_shard_rows : 0;
            const int nb = n0 - shard * p.b_shard_rows;
            tma_load_4d(b_dst, &tmBs.m[shard], &full[stage], k0, nb, b_lo, b_hi);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.error_flag) atomicExch(p.error_flag, 1);
      }
      // Let copies that are still in flight land before the CTA goes away (the consumer may have given up).
      if (*abort_flag) {
        for (int s = 0; s < C::STAGES; ++s) {
          const long long t0 = clock64();
          while (!mbar_try(&full[s], 0) && !mbar_try(&full[s], 1) && clock64() - t0 < 20000000LL) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BN, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0; int as = 0; uint32_t aphase = 0; bool ok = true;
      for (long long t = blockIdx.x; t < total && ok; t += gridDim.x) {
        if (!mbar_wait(&tempty[as], aphase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * C::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_desc(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
            umma(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);          // frees the smem stage once these MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[as]);               // accumulator complete -> epilogue
        if (++as == 2) { as = 0; aphase ^= 1; }
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.error_flag) atomicExch(p.error_flag, 2);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 -> TMEM lane quarter warp % 4)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;                  // 0, or 1 for the second warp of a lane quarter
    int as = 0; uint32_t aphase = 0; bool ok = true;
    const bool vec_ok = (p.ldc % 8 == 0);
    EpiStage est{&tmC, &tmC2, smem_u32(staging) + (uint32_t)(warp - 2) * 4096u, 0, 1};
    for (long long t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const int b = (int)(t / per_batch), rem = (int)(t % per_batch);
      const int tn = rem / tiles_m, tm = rem % tiles_m;
      const int b_lo = b % p.batch_lo, b_hi = b / p.batch_lo;
      const int row = tm * BM + q * 32 + lane;
      const int n0 = tn * BN;
      if (!mbar_wait(&tfull[as], aphase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const long long coff = (long long)b_hi * p.strideC_hi + (long long)b_lo * p.strideC_lo + (long long)row * p.ldc;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN);
      bool handled = false;
      if constexpr (BN == 128) {
        if (p.epilogue == EPI_SOFTMAX || p.epilogue == EPI_SOFTMAX_GRAD) {
          // One thread holds its whole row (128 columns): the row reduction needs no communication.
          handled = true;
          float x[128];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            __syncwarp();
            tmem_ld16(t_row + c * 16, x + c * 16);
          }
          const uint32_t thresh = (uint32_t)(p.drop_p * 65536.0f);
          const float inv_keep = p.drop_p > 0.f ? 1.0f / (1.0f - p.drop_p) : 1.0f;
          const uint64_t sd = p.drop_seed + (p.drop_step ? (uint64_t)(*p.drop_step) * 0x100000001B3ull : 0ull);
          if (row < p.M) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + coff;
            if (p.epilogue == EPI_SOFTMAX) {
              float mx = -INFINITY;
#pragma unroll
              for (int j = 0; j < 128; ++j) {
                x[j] = x[j] * p.alpha + (p.mask ? __ldg(p.mask + (long long)b_hi * 128 + j) : 0.f);
                mx = fmaxf(mx, x[j]);
              }
              float sum = 0.f;
#pragma unroll
              for (int j = 0; j < 128; ++j) { x[j] = __expf(x[j] - mx); sum += x[j]; }
              const float inv = 1.0f / sum;
#pragma unroll
              for (int c = 0; c < 16; ++c) {
#pragma unroll
                for (int j = 0; j < 8; ++j) x[c * 8 + j] *= inv;
                store8_bf16(out + c * 8, x + c * 8);
                if (p.C2 != nullptr && p.drop_p > 0.f) {
                  float ks[8], y[8];
                  keep_scale8(sd, (uint64_t)(coff + c * 8), thresh, inv_keep, ks);
#pragma unroll
                  for (int j = 0; j < 8; ++j) y[j] = x[c * 8 + j] * ks[j];
                  store8_bf16(p.C2 + coff + c * 8, y);
                }
              }
            } else {
              float s = 0.f;
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                float pr[8];
                load8_bf16(p.aux + coff + c * 8, pr);
                if (p.drop_p > 0.f) {
                  float ks[8];
                  keep_scale8(sd, (uint64_t)(coff + c * 8), thresh, inv_keep, ks);
#pragma unroll
                  for (int j = 0; j < 8; ++j) x[c * 8 + j] *= ks[j];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) s += x[c * 8 + j] * pr[j];
              }
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                float pr[8], y[8];
                load8_bf16(p.aux + coff + c * 8, pr);
#pragma unroll
                for (int j = 0; j < 8; ++j) y[j] = p.alpha * pr[j] * (x[c * 8 + j] - s);
                store8_bf16(out + c * 8, y);
              }
            }
          }
        }
      }
      if (!handled) {
        const uint32_t t_w = t_row + (uint32_t)(half * C::CW);
        const int n_w = n0 + half * C::CW;
        if (BN == 256 && p.tma_store) gemm_epilogue_row_tma<C::CW>(p, est, t_w, row, tm * BM + q * 32, n_w, b_lo, b_hi, coff, vec_ok, lane);
        else gemm_epilogue_row<C::CW>(p, t_w, row, n_w, coff, vec_ok);
      }
      __syncwarp();
      tc_fence_before();
      mbar_arrive(&tempty[as]);
      if (++as == 2) { as = 0; aphase ^= 1; }
    }
    if (BN == 256 && p.tma_store && lane == 0) bulk_wait_all();       // this warp's output copies have landed
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (p.error_flag) atomicExch(p.error_flag, 3);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

template <int BN, bool A_MN, bool B_MN>
cudaError_t launch_one(const CUtensorMap& tmA, const TmapArray& tmB, const GemmParams& p, int num_sms, cudaStream_t stream,
                       const CUtensorMap& tmC, const CUtensorMap& tmC2) {
  using C = Cfg<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch_lo * p.batch_hi;
  const int grid = (int)(tiles < num_sms ? tiles : num_sms);
  launch_pdl(kern, dim3(grid), dim3(C::THREADS), C::SMEM, stream, tmA, tmB, tmC, tmC2, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm(const CUtensorMap& tmA, const TmapArray& tmB, const GemmParams& p, int bn, bool a_mn, bool b_mn,
                        int num_sms, cudaStream_t stream, const CUtensorMap* tmC_, const CUtensorMap* tmC2_) {
  if (p.tma_store && tmC_ == nullptr) return cudaErrorInvalidValue;
  // unused maps still travel as kernel parameters: any valid descriptor will do
  const CUtensorMap& tmC = tmC_ != nullptr ? *tmC_ : tmA;
  const CUtensorMap& tmC2 = tmC2_ != nullptr ? *tmC2_ : tmC;
#define ADB_DISPATCH(BN_)                                                                      \
  if (bn == BN_) {                                                                             \
    if (!a_mn && !b_mn) return launch_one<BN_, false, false>(tmA, tmB, p, num_sms, stream, tmC, tmC2);    \
    if (!a_mn && b_mn) return launch_one<BN_, false, true>(tmA, tmB, p, num_sms, stream, tmC, tmC2);      \
    if (a_mn && !b_mn) return launch_one<BN_, true, false>(tmA, tmB, p, num_sms, stream, tmC, tmC2);      \
    return launch_one<BN_, true, true>(tmA, tmB, p, num_sms, stream, tmC, tmC2);                          \
  }
  ADB_DISPATCH(256)
  ADB_DISPATCH(128)
  ADB_DISPATCH(64)
#undef ADB_DISPATCH
  return cudaErrorInvalidValue;
}

}  // namespace adb200
