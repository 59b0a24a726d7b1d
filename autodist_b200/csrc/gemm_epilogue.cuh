// The generic epilogue of the tcgen05 GEMM kernels: one thread owns one accumulator row (TMEM lane) and walks it in
// chunks of 16 columns - scale, bias / GELU / tanh / addend, then bf16 or fp32 row stores (see GemmParams).
#pragma once
#include "gemm_tcgen05.h"
#include "tcgen05_common.cuh"

namespace adb200 {
namespace tc {

// t_row: TMEM address of this thread's lane at the first column of the accumulator; row: output row (may be >= M);
// n0: first output column of the tile; coff: element offset of (row, 0) in C.
template <int BN>
__device__ __forceinline__ void gemm_epilogue_row(const GemmParams& p, uint32_t t_row, int row, int n0, long long coff, bool vec_ok) {
#pragma unroll 1
  for (int c = 0; c < BN / 16; ++c) {
    float v[16];
    __syncwarp();                          // tcgen05.ld is warp-collective: reconverge after predicated stores
    tmem_ld16(t_row + c * 16, v);
    const int col0 = n0 + c * 16;
    const int ncols = (row < p.M) ? min(16, p.N - col0) : 0;
    if (ncols > 0) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] *= p.alpha;
    if (p.epilogue == EPI_BIAS || p.epilogue == EPI_BIAS_GELU || p.epilogue == EPI_BIAS_TANH) {
#pragma unroll
      for (int j = 0; j < 16; ++j) if (j < ncols) v[j] += __ldg(p.bias + col0 + j);
      if (p.epilogue == EPI_BIAS_TANH) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = tanhf(v[j]);
      }
    } else if (p.epilogue == EPI_ADD || p.epilogue == EPI_MUL_GELU_GRAD) {
      const __nv_bfloat16* aux = p.aux + coff + col0;
      float x[16];
      if (ncols == 16 && vec_ok) {
        const uint4 u0 = *reinterpret_cast<const uint4*>(aux), u1 = *reinterpret_cast<const uint4*>(aux + 8);
        const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
        const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f0 = __bfloat1622float2(h0[j]), f1 = __bfloat1622float2(h1[j]);
          x[2 * j] = f0.x; x[2 * j + 1] = f0.y; x[8 + 2 * j] = f1.x; x[8 + 2 * j + 1] = f1.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = (j < ncols) ? __bfloat162float(aux[j]) : 0.f;
      }
      if (p.epilogue == EPI_ADD) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] += x[j];
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= gelu_tanh_grad(x[j]);
      }
    }
    if (p.c_is_fp32) {
      float* dst = reinterpret_cast<float*>(p.C) + coff + col0;
      if (p.beta != 0.0f) {
        if (ncols == 16 && (p.ldc % 4 == 0)) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            float4 o = *reinterpret_cast<float4*>(dst + j);
            o.x += v[j]; o.y += v[j + 1]; o.z += v[j + 2]; o.w += v[j + 3];
            *reinterpret_cast<float4*>(dst + j) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (j < ncols) dst[j] += v[j];
        }
      } else if (ncols == 16 && (p.ldc % 4 == 0)) {
#pragma unroll
        for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) if (j < ncols) dst[j] = v[j];
      }
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + coff + col0;
      if (ncols == 16 && vec_ok) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
          w[j] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) if (j < ncols) dst[j] = __float2bfloat16(v[j]);
      }
      if (p.epilogue == EPI_BIAS_GELU) {
        __nv_bfloat16* dst2 = p.C2 + coff + col0;
        if (ncols == 16 && vec_ok) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(gelu_tanh(v[2 * j]), gelu_tanh(v[2 * j + 1]));
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst2) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst2 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (j < ncols) dst2[j] = __float2bfloat16(gelu_tanh(v[j]));
        }
      }
    }
    }  // ncols > 0
  }
}

}  // namespace tc
}  // namespace adb200
