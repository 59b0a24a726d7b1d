// 2-D convolution as an implicit GEMM on the 5th-generation tensor cores (sm_100a): forward, input gradient and
// weight gradient over channels-last bf16 activations, no im2col matrix in memory.
//
// Same persistent, warp-specialised shape as the GEMM (gemm_tcgen05.cu):
//   warp 0    TMA producer   per K block one box of the activation patch shifted by the filter tap (zero fill outside
//                            the image = the padding) and one box of the weight, 128-byte swizzle, ring of stages
//   warp 1    MMA issuer     tcgen05.mma 128 x BN x 16, bf16 -> fp32 in TMEM, two accumulator buffers
//   warps 2-5 epilogue       tcgen05.ld, then
//                              forward:         + bias, ReLU, per-channel sum / sum of squares (batch-norm statistics,
//                                               reduced in shared memory across the CTA's tiles), bf16 store
//                              input gradient:  bf16 store (strided positions for a strided convolution)
//                              weight gradient: fp32 store or vector atomic add (split-K)
//
// M rows of a forward / input-gradient tile are a patch of pixels (tw x th x tn <= 128) so that one 4-D box covers all of
// them for any tap; the weight gradient contracts over 64-pixel patches with both operands MN-major.
//
// Every mbarrier wait is bounded; a wait that gives up sets `error_flag`, the CTA lets its copies land, frees its
// TMEM and returns.
//
// The reference's convolutions are tf.keras layers running in cuDNN (examples/benchmark/imagenet.py:232-249).
#include "conv_tcgen05.h"
#include "pdl.cuh"
#include "tcgen05_common.cuh"

namespace adb200 {
namespace {

using namespace tc;

template <int BN, int MODE> struct ConvCfg {
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int TMEM_COLS = 2 * BN;
  // Eight epilogue warps: two per TMEM lane quarter, half of the tile's columns each. Layers with a short contraction
  // (1 x 1 convolutions) spend longer draining a tile than multiplying it, and four warps could not keep up.
  static constexpr int EPI_WARPS = 8;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int CHUNKS = BN / 16 / (EPI_WARPS / 4);      // 16-column chunks per epilogue warp
  static constexpr int STAT_BYTES = (MODE == CONV_FPROP) ? 2 * kMaxStatChannels * 4 : 0;
  static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/ + STAT_BYTES;
};

struct TileCoord {
  int w0, h0, n0;       // patch origin in the pixel grid
  int c0;               // first column of the GEMM N extent
  int m0;               // weight gradient: first output channel
  int tap;              // weight gradient: tap of this tile
  int kbeg, kend;       // weight gradient: patch range of this tile
};

template <int BN, int MODE>
__device__ __forceinline__ TileCoord decode_tile(const ConvParams& p, long long t) {
  TileCoord c;
  if (MODE != CONV_WGRAD) {
    const int m_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    const int ct = (int)(t / m_tiles), m = (int)(t % m_tiles);
    c.w0 = (m % p.tiles_w) * p.tw;
    c.h0 = ((m / p.tiles_w) % p.tiles_h) * p.th;
    c.n0 = (m / (p.tiles_w * p.tiles_h)) * p.tn;
    c.c0 = ct * BN;
    c.m0 = 0; c.tap = 0; c.kbeg = 0; c.kend = 0;
  } else {
    const int m_tiles = (p.Mc + BM - 1) / BM, c_tiles = (p.Nc + BN - 1) / BN;
    long long r = t;
    c.m0 = (int)(r % m_tiles) * BM; r /= m_tiles;
    c.c0 = (int)(r % c_tiles) * BN; r /= c_tiles;
    c.tap = (int)(r % p.ntaps);
    const int ks = (int)(r / p.ntaps);
    const long long P = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
    c.kbeg = (int)(P * ks / p.ksplit);
    c.kend = (int)(P * (ks + 1) / p.ksplit);
    c.w0 = c.h0 = c.n0 = 0;
  }
  return c;
}

__device__ __forceinline__ long long total_tiles(const ConvParams& p, int bn, int mode) {
  const int c_tiles = (p.Nc + bn - 1) / bn;
  if (mode != CONV_WGRAD) return (long long)p.tiles_w * p.tiles_h * p.tiles_n * c_tiles;
  return (long long)((p.Mc + BM - 1) / BM) * c_tiles * p.ntaps * p.ksplit;
}

// Sum of v[0..15] over the 32 lanes of a warp, column j ends up in the lanes whose bits 4..1 spell j (both lanes of a
// pair hold it). 16 shuffles instead of 80: every step halves the columns a lane is responsible for.
__device__ __forceinline__ float warp_column_sums16(float* v, int lane) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int half = 8 >> s;
    const bool upper = (lane & (16 >> s)) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16 >> s);
    }
  }
  return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}

template <int BN, int MODE>
__global__ void __launch_bounds__(ConvCfg<BN, MODE>::THREADS, 1)
conv_kernel(const __grid_constant__ ConvMaps maps, const __grid_constant__ ConvParams p) {
  using C = ConvCfg<BN, MODE>;
  constexpr bool A_MN = MODE == CONV_WGRAD;
  constexpr bool B_MN = MODE != CONV_FPROP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + C::STAGES * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * (A_BYTES + C::B_BYTES));
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_stat = reinterpret_cast<float*>(smem + C::STAGES * (A_BYTES + C::B_BYTES) + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool do_stats = (MODE == CONV_FPROP) && p.stats != nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull[s], 1); mbar_init(&tempty[s], 32 * C::EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (MODE == CONV_FPROP) {
    if (do_stats) for (int i = threadIdx.x; i < 2 * p.Nc; i += C::THREADS) s_stat[i] = 0.f;
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

  // trace (when given): 0 start, 1 first load issued, 2 last load issued, 3 first stage full, 4 last MMA committed,
  // 5 cycles the first epilogue warp spent between "accumulator full" and "accumulator released" (summed over tiles),
  // 6 cycles it waited for full accumulators, 7 end
  long long* trace = p.trace != nullptr ? p.trace + (long long)blockIdx.x * 8 : nullptr;
  if (trace != nullptr && threadIdx.x == 0) trace[0] = clock64();
  const long long total = total_tiles(p, BN, MODE);
  const int kcb = (p.Kc + BK - 1) / BK;
  const int rows = p.tw * p.th * p.tn;
  const int col_rows = p.th * p.tn;                 // rows of one patch column (wsplit boxes)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      if (trace != nullptr) trace[1] = clock64();
      for (long long t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const TileCoord tc_ = decode_tile<BN, MODE>(p, t);
        if (MODE != CONV_WGRAD) {
          const uint32_t a_bytes = (uint32_t)rows * 128u;
          for (int tp = 0; tp < p.ntaps && ok; ++tp) {
            const ConvTap tap = p.taps[tp];
            const CUtensorMap* mapA = &maps.act[tap.amap];
            for (int cb = 0; cb < kcb; ++cb) {
              if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
              mbar_expect_tx(&full[stage], a_bytes + C::B_BYTES);
              uint8_t* a_dst = sA + stage * A_BYTES;
              uint8_t* b_dst = sB + stage * C::B_BYTES;
              if (!p.wsplit) {
                tma_load_4d(a_dst, mapA, &full[stage], cb * BK, tc_.w0 + tap.dw, tc_.h0 + tap.dh, tc_.n0);
              } else {
                for (int j = 0; j < p.tw; ++j)
                  tma_load_4d(a_dst + j * col_rows * 128, mapA, &full[stage], (tc_.w0 + j) * p.xstep, tc_.h0 + tap.dh, tc_.n0, 0);
              }
              if (MODE == CONV_FPROP) {
                tma_load_4d(b_dst, &maps.w, &full[stage], cb * BK, tap.wtap, tc_.c0, 0);
              } else {
#pragma unroll
                for (int j = 0; j < BN / 64; ++j)
                  tma_load_4d(b_dst + j * (BK * 128), &maps.w, &full[stage], tc_.c0 + 64 * j, tap.wtap, cb * BK, 0);
              }
              if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
          }
        } else {
          const ConvTap tap = p.taps[tc_.tap];
          const CUtensorMap* mapX = &maps.act[tap.amap];
          for (int pi = tc_.kbeg; pi < tc_.kend; ++pi) {
            const int w0 = (pi % p.tiles_w) * p.tw;
            const int h0 = ((pi / p.tiles_w) % p.tiles_h) * p.th;
            const int n0 = (pi / (p.tiles_w * p.tiles_h)) * p.tn;
            if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
            // output channels beyond Cout need no load: those accumulator rows are never stored
            const int a_chunks = (tc_.m0 + 64 < p.Mc) ? 2 : 1;
            mbar_expect_tx(&full[stage], a_chunks * (BK * 128) + C::B_BYTES);
            uint8_t* a_dst = sA + stage * A_BYTES;
            uint8_t* b_dst = sB + stage * C::B_BYTES;
            if (!p.wsplit) {
              for (int j = 0; j < a_chunks; ++j) tma_load_4d(a_dst + j * (BK * 128), &maps.dy, &full[stage], tc_.m0 + 64 * j, w0, h0, n0);
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_4d(b_dst + j * (BK * 128), mapX, &full[stage], tc_.c0 + 64 * j, w0 + tap.dw, h0 + tap.dh, n0);
            } else {
              for (int jw = 0; jw < p.tw; ++jw) {
                for (int j = 0; j < a_chunks; ++j)
                  tma_load_4d(a_dst + j * (BK * 128) + jw * col_rows * 128, &maps.dy, &full[stage], tc_.m0 + 64 * j, w0 + jw, h0, n0);
                tma_load_4d(b_dst + jw * col_rows * 128, mapX, &full[stage], (w0 + jw) * p.xstep, h0 + tap.dh, n0, 0);
              }
            }
            if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
      if (trace != nullptr) trace[2] = clock64();
      if (!ok) {
        *abort_flag = 1;
        if (p.error_flag) atomicExch(p.error_flag, 11);
      }
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
        int num_kb;
        if (MODE != CONV_WGRAD) {
          num_kb = p.ntaps * kcb;
        } else {
          const TileCoord tc_ = decode_tile<BN, MODE>(p, t);
          num_kb = tc_.kend - tc_.kbeg;
        }
        if (num_kb <= 0) continue;
        if (!mbar_wait(&tempty[as], aphase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          if (trace != nullptr && t == blockIdx.x && kb == 0) trace[3] = clock64();
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
          umma_commit(&empty[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[as]);
        if (trace != nullptr) trace[4] = clock64();
        if (++as == 2) { as = 0; aphase ^= 1; }
      }
      if (!ok) {
        *abort_flag = 1;
        if (p.error_flag) atomicExch(p.error_flag, 12);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 -> TMEM lane quarter warp % 4)
    const int q = warp & 3;
    const int c_lo = ((warp - 2) >> 2) * C::CHUNKS;      // first 16-column chunk of this warp's share of the tile
    int as = 0; uint32_t aphase = 0; bool ok = true;
    const int r = q * 32 + lane;
    for (long long t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const TileCoord tc_ = decode_tile<BN, MODE>(p, t);
      if (MODE == CONV_WGRAD && tc_.kend <= tc_.kbeg) continue;
      bool valid;
      long long off;
      if (MODE != CONV_WGRAD) {
        int j, i, nn;
        if (!p.wsplit) { j = r % p.tw; i = (r / p.tw) % p.th; nn = r / (p.tw * p.th); }
        else { j = r / col_rows; const int rem = r % col_rows; i = rem % p.th; nn = rem / p.th; }
        const int gw = tc_.w0 + j, gh = tc_.h0 + i, gn = tc_.n0 + nn;
        valid = r < rows && gw < p.GW && gh < p.GH && gn < p.GN;
        off = (((long long)gn * p.OH + (long long)gh * p.os + p.oh0) * p.OW + (long long)gw * p.os + p.ow0) * p.ldc;
      } else {
        const int row = tc_.m0 + r;
        valid = row < p.Mc;
        off = (long long)row * p.ldc + (long long)p.taps[tc_.tap].wtap * p.wtap_stride;
      }
      const long long tw0 = trace != nullptr ? clock64() : 0;
      if (MODE == CONV_DGRAD) {
        if (p.addend != nullptr) {
          // The gradient another consumer of the same tensor produced (a residual fork) is added to this tile. Its whole
          // row segment is requested before the wait for the accumulator, so the loads overlap the tile's MMAs, and
          // the chunk loop below is unrolled so that the prefetched vectors stay in registers.
          uint4 pre[2 * C::CHUNKS];
          const int cw0 = tc_.c0 + c_lo * 16;
          const __nv_bfloat16* src = p.addend + off + cw0;
#pragma unroll
          for (int h = 0; h < 2 * C::CHUNKS; ++h) {
            pre[h] = make_uint4(0, 0, 0, 0);
            if (valid && cw0 + h * 8 < p.Nc) pre[h] = *reinterpret_cast<const uint4*>(src + h * 8);
          }
          if (!mbar_wait(&tfull[as], aphase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN);
#pragma unroll
          for (int c = 0; c < C::CHUNKS; ++c) {
            const int col0 = cw0 + c * 16;
            if (col0 < p.Nc) {                     // uniform over the warp
              float v[16], a[16];
              __syncwarp();
              tmem_ld16(t_row + (c_lo + c) * 16, v);
              unpack8_bf16(pre[2 * c], a);
              unpack8_bf16(pre[2 * c + 1], a + 8);
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) v[jj] += a[jj];
              if (valid) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + off + col0;
                store8_bf16(dst, v);                                  // Nc is a multiple of 8: a chunk holds 8 or 16 columns
                if (col0 + 8 < p.Nc) store8_bf16(dst + 8, v + 8);
              }
            }
          }
          __syncwarp();
          tc_fence_before();
          mbar_arrive(&tempty[as]);
          if (++as == 2) { as = 0; aphase ^= 1; }
          continue;
        }
      }
      if (!mbar_wait(&tfull[as], aphase, abort_flag)) { ok = false; break; }
      const long long tw1 = trace != nullptr ? clock64() : 0;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN);
#pragma unroll 1
      for (int c = c_lo; c < c_lo + C::CHUNKS; ++c) {
        const int col0 = tc_.c0 + c * 16;
        if (col0 >= p.Nc) break;                 // uniform over the warp
        float v[16];
        __syncwarp();
        tmem_ld16(t_row + c * 16, v);
        const int ncols = valid ? min(16, p.Nc - col0) : 0;
        if (MODE == CONV_WGRAD) {
          if (ncols > 0) {
            float* dst = reinterpret_cast<float*>(p.out) + off + col0;
            const bool vec = ncols == 16 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
            if (p.accumulate) {
              if (vec) {
#pragma unroll
                for (int jj = 0; jj < 16; jj += 4) atomicAdd(reinterpret_cast<float4*>(dst + jj), make_float4(v[jj], v[jj + 1], v[jj + 2], v[jj + 3]));
              } else {
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) if (jj < ncols) atomicAdd(dst + jj, v[jj]);
              }
            } else if (vec) {
#pragma unroll
              for (int jj = 0; jj < 16; jj += 4) *reinterpret_cast<float4*>(dst + jj) = make_float4(v[jj], v[jj + 1], v[jj + 2], v[jj + 3]);
            } else {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) if (jj < ncols) dst[jj] = v[jj];
            }
          }
        } else {
          if (MODE == CONV_FPROP) {
            if (p.bias != nullptr) {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) if (col0 + jj < p.Nc) v[jj] += __ldg(p.bias + col0 + jj);
            }
            if (p.relu) {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) v[jj] = fmaxf(v[jj], 0.f);
            }
          }
          if (ncols > 0) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + off + col0;
            if (ncols == 16 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
              store8_bf16(dst, v);
              store8_bf16(dst + 8, v + 8);
            } else {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) if (jj < ncols) dst[jj] = __float2bfloat16(v[jj]);
            }
          }
          if (MODE == CONV_FPROP) {
            if (do_stats) {
              // statistics of what the next layer will read: the values as rounded to bf16
              float s1[16], s2[16];
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) {
                const float x = (jj < ncols) ? __bfloat162float(__float2bfloat16(v[jj])) : 0.f;
                s1[jj] = x; s2[jj] = x * x;
              }
              const float a = warp_column_sums16(s1, lane);
              const float b = warp_column_sums16(s2, lane);
              // both lanes of a pair hold one column: bits 4..1 of the lane, most significant first
              const int colm = col0 + (((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1));
              if ((lane & 1) == 0 && colm < p.Nc) {
                atomicAdd(&s_stat[colm], a);
                atomicAdd(&s_stat[p.Nc + colm], b);
              }
            }
          }
        }
      }
      __syncwarp();
      tc_fence_before();
      mbar_arrive(&tempty[as]);
      if (trace != nullptr && threadIdx.x == 64) { trace[5] += clock64() - tw1; trace[6] += tw1 - tw0; }
      if (++as == 2) { as = 0; aphase ^= 1; }
    }
    if (trace != nullptr && threadIdx.x == 64) trace[7] = clock64();
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (p.error_flag) atomicExch(p.error_flag, 13);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
  if (MODE == CONV_FPROP) {
    if (do_stats) {
      for (int i = threadIdx.x; i < 2 * p.Nc; i += C::THREADS) {
        const float x = s_stat[i];
        if (x != 0.f) atomicAdd(p.stats + i, x);
      }
    }
  }
}

template <int BN, int MODE>
cudaError_t launch_one(const ConvMaps& maps, const ConvParams& p, int num_sms, cudaStream_t stream) {
  using C = ConvCfg<BN, MODE>;
  auto kern = conv_kernel<BN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int c_tiles = (p.Nc + BN - 1) / BN;
  long long tiles;
  if (MODE != CONV_WGRAD) tiles = (long long)p.tiles_w * p.tiles_h * p.tiles_n * c_tiles;
  else tiles = (long long)((p.Mc + BM - 1) / BM) * c_tiles * p.ntaps * p.ksplit;
  if (tiles <= 0) return cudaSuccess;
  const int grid = (int)(tiles < num_sms ? tiles : num_sms);
  launch_pdl(kern, dim3(grid), dim3(C::THREADS), C::SMEM, stream, maps, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_conv(const ConvMaps& maps, const ConvParams& p, int bn, int num_sms, cudaStream_t stream) {
  if (p.tw * p.th * p.tn > BM || p.ntaps < 1 || p.ntaps > kMaxConvTaps) return cudaErrorInvalidValue;
  if (p.mode == CONV_WGRAD && (p.tw * p.th * p.tn != BK || p.ksplit < 1)) return cudaErrorInvalidValue;
  if (p.mode == CONV_FPROP && p.stats != nullptr && p.Nc > kMaxStatChannels) return cudaErrorInvalidValue;
#define ADB_CONV_DISPATCH(BN_)                                                                      \
  if (bn == BN_) {                                                                                  \
    if (p.mode == CONV_FPROP) return launch_one<BN_, CONV_FPROP>(maps, p, num_sms, stream);          \
    if (p.mode == CONV_DGRAD) return launch_one<BN_, CONV_DGRAD>(maps, p, num_sms, stream);          \
    if (p.mode == CONV_WGRAD) return launch_one<BN_, CONV_WGRAD>(maps, p, num_sms, stream);          \
  }
  ADB_CONV_DISPATCH(256)
  ADB_CONV_DISPATCH(128)
  ADB_CONV_DISPATCH(64)
#undef ADB_CONV_DISPATCH
  return cudaErrorInvalidValue;
}

}  // namespace adb200
