// The tcgen05 GEMM with two SMs on one 256 x 256 tile (tcgen05.mma.cta_group::2): D[b][M,N] = A[b][M,K] * B[b][N,K]^T.
//
// A cluster of two CTAs owns a tile. Each CTA stages its own half of both operands - 128 rows of A (its half of the
// tile's M extent) and 128 rows of B (its half of the N extent) - with ordinary, non-multicast TMA loads, so a K block
// costs each SM 32 KB of shared-memory fill instead of the 48 KB of the one-CTA 128 x 256 tile. One thread of the
// leader CTA (cluster rank 0) issues the MMAs; the hardware reads A and B from both CTAs' shared memory and writes each
// CTA's 128 accumulator rows into that CTA's own TMEM, which its own epilogue warps drain.
//
// Synchronisation (every barrier at the same shared-memory offset in both CTAs):
//   full[s]    leader only. The leader's producer posts the byte count of both CTAs' loads; both CTAs' TMA loads
//              complete on it (cp.async.bulk.tensor ... cta_group::2 lets a load signal the peer CTA's barrier).
//   empty[s]   one per CTA: the leader's MMA thread commits to both (two tcgen05.commit, the second to the peer's
//              address), releasing the stage in each CTA for that CTA's producer.
//   tfull[a]   one per CTA, committed to in the same way when an accumulator is complete.
//   tempty[a]  leader only: the eight epilogue warps of both CTAs arrive on it (remote mbarrier.arrive for the peer).
// TMEM is allocated and freed by warp 1 of both CTAs with the cta_group::2 forms; a cluster barrier after the barrier
// initialisation and another before the deallocation keep either CTA from touching the other too early or leaving
// while the other still reads its shared memory. Every mbarrier wait is bounded as in the one-CTA kernel; both CTAs
// always reach the final cluster barrier.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_epilogue.cuh"
#include "gemm_tcgen05.h"
#include "pdl.cuh"
#include "tcgen05_common.cuh"

namespace adb200 {
namespace {

using namespace tc;

constexpr int BN2 = 256;                 // tile width; each CTA stages BN2 / 2 rows of B
constexpr int B2_BYTES = (BN2 / 2) * BK * 2;
constexpr int STAGES2 = 5;              // 5 x 32 KB + 32 KB of output staging: the CTA stays at 193 KB (room for a dependent kernel's blocks)
constexpr int TMEM_COLS2 = 2 * BN2;
constexpr int EPI_WARPS2 = 8;            // two per TMEM lane quarter, half of the tile's columns each
constexpr int kThreads2 = 64 + 32 * EPI_WARPS2;
constexpr int STAGING2 = EPI_WARPS2 * 4096;   // TMA-store staging: one 4 KB buffer per epilogue warp
constexpr int SMEM2 = STAGES2 * (A_BYTES + B2_BYTES) + STAGING2 + 1024 /*align*/ + 256 /*barriers*/;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of `local` (an address of this CTA's shared memory) in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion is counted on `bar_cluster_addr`, a barrier of this CTA or of its pair partner.
__device__ __forceinline__ void tma_load_4d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void umma2(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Arrives on the barrier at `cluster_addr` (any CTA of the cluster) once the MMAs issued so far have completed.
__device__ __forceinline__ void umma2_commit(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return (long long)t;
}
__device__ __forceinline__ uint32_t make_idesc2(bool a_mn, bool b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;                       // D format: f32
  d |= 1u << 7;                       // A format: bf16
  d |= 1u << 10;                      // B format: bf16
  d |= (a_mn ? 1u : 0u) << 15;        // A major
  d |= (b_mn ? 1u : 0u) << 16;        // B major
  d |= (uint32_t)(BN2 >> 3) << 17;    // N / 8 of the pair's tile
  d |= (uint32_t)(256 >> 4) << 24;    // M / 16 of the pair's tile
  return d;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads2, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
             const __grid_constant__ CUtensorMap tmC2, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory starts at the same offset in both CTAs, so the aligned layouts coincide
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES2 * A_BYTES;
  uint8_t* staging = smem + STAGES2 * (A_BYTES + B2_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + STAGING2);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES2;
  uint64_t* tfull = bars + 2 * STAGES2;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // trace (when given): 0 entry, 1 set-up done, 2 first stage full, 3 last MMA committed, 4 ns the MMA thread waited for
  // full stages, 5 ns it waited for a free accumulator, 6 ns the first epilogue warp spent draining, 7 end
  long long* trace = p.trace != nullptr ? p.trace + (long long)blockIdx.x * 8 : nullptr;
  if (trace != nullptr && threadIdx.x == 0) trace[0] = now_ns();
  const uint32_t rank = cluster_ctarank();            // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull[s], 1); mbar_init(&tempty[s], 2 * EPI_WARPS2); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS2) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // both CTAs' barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_sync();       // everything above touched only shared and tensor memory; global memory is read from here on
  if (trace != nullptr && threadIdx.x == 0) trace[1] = now_ns();

  const int tiles_m = (p.M + 255) / 256;
  const int tiles_n = (p.N + BN2 - 1) / BN2;
  const int per_batch = tiles_m * tiles_n;
  const long long total = (long long)per_batch * p.batch_lo * p.batch_hi;
  const int num_kb = (p.K + BK - 1) / BK;
  const long long pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (each CTA: its halves of A and B)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (long long t = pair; t < total && ok; t += pairs) {
        const int b = (int)(t / per_batch), rem = (int)(t % per_batch);
        const int tn = rem / tiles_m, tm = rem % tiles_m;
        const int b_lo = b % p.batch_lo, b_hi = b / p.batch_lo;
        const int m0 = tm * 256 + (int)rank * 128, n0 = tn * BN2 + (int)rank * (BN2 / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          if (leader) mbar_expect_tx(&full[stage], 2 * (A_BYTES + B2_BYTES));
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B2_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_4d_pair(a_dst + j * (BK * 128), &tmA, bar, m0 + 64 * j, k0, b_lo, b_hi);
          } else {
            tma_load_4d_pair(a_dst, &tmA, bar, k0, m0, b_lo, b_hi);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_4d_pair(b_dst + j * (BK * 128), &tmB, bar, n0 + 64 * j, k0, b_lo, b_hi);
          } else {
            tma_load_4d_pair(b_dst, &tmB, bar, k0, n0, b_lo, b_hi);
          }
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.error_flag) atomicExch(p.error_flag, 41);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc2(A_MN, B_MN);
      int stage = 0; uint32_t phase = 0; int as = 0; uint32_t aphase = 0; bool ok = true;
      for (long long t = pair; t < total && ok; t += pairs) {
        const long long w0 = trace != nullptr ? now_ns() : 0;
        if (!mbar_wait(&tempty[as], aphase ^ 1, abort_flag)) { ok = false; break; }
        if (trace != nullptr) trace[5] += now_ns() - w0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN2);
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long w1 = trace != nullptr ? now_ns() : 0;
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          if (trace != nullptr) { const long long w2 = now_ns(); trace[4] += w2 - w1; if (trace[2] == 0) trace[2] = w2; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B2_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_desc(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
            umma2(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma2_commit(smem_u32(&empty[stage]));
          umma2_commit(map_to_cta(smem_u32(&empty[stage]), 1));
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma2_commit(smem_u32(&tfull[as]));            // accumulator complete -> both CTAs' epilogues
        umma2_commit(map_to_cta(smem_u32(&tfull[as]), 1));
        if (trace != nullptr) trace[3] = now_ns();
        if (++as == 2) { as = 0; aphase ^= 1; }
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.error_flag) atomicExch(p.error_flag, 42);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 -> TMEM lane quarter warp % 4)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;                  // which half of the tile's columns this warp drains
    int as = 0; uint32_t aphase = 0; bool ok = true;
    const bool vec_ok = (p.ldc % 8 == 0);
    EpiStage est{&tmC, &tmC2, smem_u32(staging) + (uint32_t)(warp - 2) * 4096u, 0, 1};
    for (long long t = pair; t < total && ok; t += pairs) {
      const int b = (int)(t / per_batch), rem = (int)(t % per_batch);
      const int tn = rem / tiles_m, tm = rem % tiles_m;
      const int b_lo = b % p.batch_lo, b_hi = b / p.batch_lo;
      const int row = tm * 256 + (int)rank * 128 + q * 32 + lane;
      const int n0 = tn * BN2;
      if (!mbar_wait(&tfull[as], aphase, abort_flag)) { ok = false; break; }
      const long long e0 = trace != nullptr ? now_ns() : 0;
      tc_fence_after();
      const long long coff = (long long)b_hi * p.strideC_hi + (long long)b_lo * p.strideC_lo + (long long)row * p.ldc;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN2);
      const uint32_t t_w = t_row + (uint32_t)(half * (BN2 / 2));
      const int n_w = n0 + half * (BN2 / 2);
      if (p.tma_store) gemm_epilogue_row_tma<BN2 / 2>(p, est, t_w, row, tm * 256 + (int)rank * 128 + q * 32, n_w, b_lo, b_hi, coff, vec_ok, lane);
      else gemm_epilogue_row<BN2 / 2>(p, t_w, row, n_w, coff, vec_ok);
      __syncwarp();
      tc_fence_before();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[as]), 0));
      if (trace != nullptr && threadIdx.x == 64) trace[6] += now_ns() - e0;
      if (++as == 2) { as = 0; aphase ^= 1; }
    }
    if (p.tma_store && lane == 0) bulk_wait_all();       // this warp's output copies have landed
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (p.error_flag) atomicExch(p.error_flag, 43);
    }
  }

  if (trace != nullptr && threadIdx.x == 0) trace[7] = now_ns();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // neither CTA leaves, or frees TMEM, while the other still works
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS2) : "memory");
  }
}

template <bool A_MN, bool B_MN>
cudaError_t launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int num_sms, cudaStream_t stream,
                        const CUtensorMap& tmC, const CUtensorMap& tmC2) {
  auto kern = gemm2_kernel<A_MN, B_MN>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2);
    if (e != cudaSuccess) return e;
    // how many pairs the GPU holds at once: SM pairs of one cluster sit in one GPC, so it can be fewer than SMs / 2
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(num_sms & ~1);
    q.blockDim = dim3(kThreads2);
    q.dynamicSmemBytes = SMEM2;
    cudaLaunchAttribute a[1];
    a[0].id = cudaLaunchAttributeClusterDimension;
    a[0].val.clusterDim.x = 2; a[0].val.clusterDim.y = 1; a[0].val.clusterDim.z = 1;
    q.attrs = a; q.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &q);
    if (e != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = num_sms / 2; }
    max_pairs = n < num_sms / 2 ? n : num_sms / 2;
  }
  const long long tiles = (long long)((p.M + 255) / 256) * ((p.N + BN2 - 1) / BN2) * p.batch_lo * p.batch_hi;
  const int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
  if (pairs <= 0) return cudaSuccess;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads2);
  cfg.dynamicSmemBytes = SMEM2;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr; cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmC2, p);
}

}  // namespace

// The pair kernel: `tmA` / `tmB` are the maps of launch_gemm with boxes of 128 rows for a K-major operand (64 x 64
// for an MN-major one). No fused softmax and no row-sharded B here.
cudaError_t launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, bool a_mn, bool b_mn, int num_sms,
                             cudaStream_t stream, const CUtensorMap* tmC_, const CUtensorMap* tmC2_) {
  if (p.tma_store && tmC_ == nullptr) return cudaErrorInvalidValue;
  const CUtensorMap& tmC = tmC_ != nullptr ? *tmC_ : tmA;
  const CUtensorMap& tmC2 = tmC2_ != nullptr ? *tmC2_ : tmC;
  if (p.b_shard_rows > 0 || p.epilogue == EPI_SOFTMAX || p.epilogue == EPI_SOFTMAX_GRAD) return cudaErrorInvalidValue;
  if (!a_mn && !b_mn) return launch_pair<false, false>(tmA, tmB, p, num_sms, stream, tmC, tmC2);
  if (!a_mn && b_mn) return launch_pair<false, true>(tmA, tmB, p, num_sms, stream, tmC, tmC2);
  if (a_mn && !b_mn) return launch_pair<true, false>(tmA, tmB, p, num_sms, stream, tmC, tmC2);
  return launch_pair<true, true>(tmA, tmB, p, num_sms, stream, tmC, tmC2);
}

}  // namespace adb200
