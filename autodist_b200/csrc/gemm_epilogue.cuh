// The generic epilogue of the tcgen05 GEMM kernels: one thread owns one accumulator row (TMEM lane) and walks it in
// chunks of 16 columns - scale, bias / GELU / tanh / addend, then bf16 or fp32 row stores (see GemmParams).
#pragma once
#include "gemm_tcgen05.h"
#include "tcgen05_common.cuh"

namespace adb200 {
namespace tc {

// The arithmetic of the epilogue on 16 accumulator values of one row, in place: scale, then bias (+ tanh), addend or
// GELU derivative. `ncols` of the 16 columns starting at `col0` exist (0: nothing is read from memory).
__device__ __forceinline__ void gemm_epilogue_math16(const GemmParams& p, float* v, int col0, int ncols, long long coff, bool vec_ok) {
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] *= p.alpha;
  if (p.epilogue == EPI_BIAS || p.epilogue == EPI_BIAS_GELU || p.epilogue == EPI_BIAS_TANH) {
    if (ncols == 16 && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 16; j += 4) {                      // col0 is a multiple of 16: four aligned 16-byte loads
        const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + j));
        v[j] += b4.x; v[j + 1] += b4.y; v[j + 2] += b4.z; v[j + 3] += b4.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) if (j < ncols) v[j] += __ldg(p.bias + col0 + j);
    }
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
}

// ---------------------------------------------------------------------------------------------------------------------
// Output through shared memory and TMA. A thread owns one row, so direct stores leave a warp writing 32 different rows in
// 16-byte pieces - partial sectors that cost the L2 as much as full ones and compete with the operand loads. Here each
// epilogue warp stages 32 rows x 128 bytes (64 bf16 or 32 fp32 columns) in the 128-byte-swizzled layout and one lane hands
// the box to the TMA unit, which writes whole lines (or adds them into an fp32 output: beta = 1). Rows and columns
// past the matrix are clipped by the copy itself. Two 4 KB buffers per warp alternate, so staging overlaps the copy.
struct EpiStage {
  const CUtensorMap* tmC;      // output map, box (128 bytes of columns, 32 rows, 1, 1), 128-byte swizzle
  const CUtensorMap* tmC2;     // second output of EPI_BIAS_GELU
  uint32_t smem;               // shared address of this warp's 4 KB staging buffers (1024-byte aligned)
  int units;                   // copies issued so far by this warp (picks the buffer)
  int bufs;                    // 2: staging of one box overlaps the copy of the one before; 1: they alternate
};

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// box_row: first output row of this warp's 32 rows; lane = row inside the box. Other arguments as gemm_epilogue_row.
// BNW: columns this warp drains (the tile's width, or half of it when two warps share a TMEM lane quarter).
template <int BNW>
__device__ __forceinline__ void gemm_epilogue_row_tma(const GemmParams& p, EpiStage& st, uint32_t t_row, int row, int box_row, int n0, int b_lo,
                                                      int b_hi, long long coff, bool vec_ok, int lane) {
  const bool f32 = p.c_is_fp32 != 0;
  const int gcols = f32 ? 32 : 64;                   // columns in one 128-byte staging row
  const bool two = p.epilogue == EPI_BIAS_GELU;      // two outputs (bf16): the pre-activation, then its GELU
  const uint32_t swz = (uint32_t)(lane & 7);
#pragma unroll 1
  for (int g = 0; g * gcols < BNW; ++g) {
    const int gcol0 = n0 + g * gcols;
    if (gcol0 >= p.N) break;                          // uniform over the CTA
    if (lane == 0) {                                  // the buffer about to be written is no longer being read
      if (st.bufs < 2) bulk_wait_read<0>(); else bulk_wait_read<1>();
    }
    __syncwarp();
    const uint32_t base = st.smem + (st.bufs < 2 ? 0u : (uint32_t)(st.units & 1)) * 4096u;
    const uint32_t buf = base + (uint32_t)lane * 128u;
    uint32_t act[32];                                 // packed GELU values of the group (two outputs only)
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      if (f32 && cc >= 2) break;
      float v[16];
      __syncwarp();                                   // tcgen05.ld is warp-collective
      tmem_ld16(t_row + g * gcols + cc * 16, v);
      const int col0 = gcol0 + cc * 16;
      const int ncols = (row < p.M) ? max(0, min(16, p.N - col0)) : 0;
      gemm_epilogue_math16(p, v, col0, ncols, coff, vec_ok);
      if (f32) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          st_shared_v4(buf + (((uint32_t)(cc * 4 + i) ^ swz) << 4), __float_as_uint(v[4 * i]), __float_as_uint(v[4 * i + 1]),
                       __float_as_uint(v[4 * i + 2]), __float_as_uint(v[4 * i + 3]));
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
          st_shared_v4(buf + (((uint32_t)(cc * 2 + h) ^ swz) << 4), pack_bf16x2(v[8 * h], v[8 * h + 1]), pack_bf16x2(v[8 * h + 2], v[8 * h + 3]),
                       pack_bf16x2(v[8 * h + 4], v[8 * h + 5]), pack_bf16x2(v[8 * h + 6], v[8 * h + 7]));
        if (two) {
#pragma unroll
          for (int j = 0; j < 8; ++j) act[cc * 8 + j] = pack_bf16x2(gelu_tanh(v[2 * j]), gelu_tanh(v[2 * j + 1]));
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the staged rows are visible to the TMA unit
    __syncwarp();
    if (lane == 0) {
      if (f32 && p.beta != 0.0f) tma_reduce_add_4d(st.tmC, base, gcol0, box_row, b_lo, b_hi);
      else tma_store_4d(st.tmC, base, gcol0, box_row, b_lo, b_hi);
      bulk_commit();
    }
    st.units += 1;
    if (two) {
      // second output from the values kept in registers, through the other buffer (or the same one once it has been read)
      if (lane == 0) {
        if (st.bufs < 2) bulk_wait_read<0>(); else bulk_wait_read<1>();
      }
      __syncwarp();
      const uint32_t base2 = st.smem + (st.bufs < 2 ? 0u : (uint32_t)(st.units & 1)) * 4096u;
      const uint32_t buf2 = base2 + (uint32_t)lane * 128u;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        st_shared_v4(buf2 + (((uint32_t)j ^ swz) << 4), act[4 * j], act[4 * j + 1], act[4 * j + 2], act[4 * j + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        tma_store_4d(st.tmC2, base2, gcol0, box_row, b_lo, b_hi);
        bulk_commit();
      }
      st.units += 1;
    }
  }
}

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
    gemm_epilogue_math16(p, v, col0, ncols, coff, vec_ok);
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
