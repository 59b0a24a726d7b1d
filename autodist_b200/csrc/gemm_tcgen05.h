// Host-side interface of the tcgen05 GEMM (see gemm_tcgen05.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace adb200 {

enum GemmEpilogue { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_GELU = 2, EPI_MUL_GELU_GRAD = 3, EPI_ADD = 4, EPI_BIAS_TANH = 5,
                    EPI_SOFTMAX = 6, EPI_SOFTMAX_GRAD = 7 };

struct GemmParams {
  int M, N, K;                 // per batch entry
  int batch_lo, batch_hi;      // two batch dimensions (1 when unused)
  void* C;                     // output, bf16 or fp32, row-major with leading dimension ldc (elements)
  long long ldc, strideC_lo, strideC_hi;
  int c_is_fp32;
  __nv_bfloat16* C2;           // EPI_BIAS_GELU: gelu(C) goes here (same strides as C)
  const float* bias;           // EPI_BIAS*: one value per output column
  const __nv_bfloat16* aux;    // EPI_MUL_GELU_GRAD: pre-activation; EPI_ADD: addend (may alias C); same strides as C
  int epilogue;
  float alpha;                 // scale applied to the accumulator first
  float beta;                  // fp32 output only: 0 = overwrite, otherwise C += result
  int* error_flag;             // device int, set non-zero when a bounded wait gave up
  // Row softmax fused into the epilogue (attention, N == 128 == tile width; one thread owns one row):
  //   EPI_SOFTMAX      C = softmax(alpha * acc + mask[b_hi][col]); C2 (optional) = dropout(C)
  //   EPI_SOFTMAX_GRAD C = alpha * P * (d - sum(d * P)), d = acc * dropout mask, P read from aux
  const float* mask;           // additive fp32 mask [batch_hi, N] or null
  float drop_p;                // dropout probability of the attention probabilities (0 = off)
  unsigned long long drop_seed;
  const long long* drop_step;  // device step counter mixed into the seed (null = none)
  int b_shard_rows;            // > 0: B is split by rows into shards of this many rows, shard s read through tmB.m[s]
  int tma_store;               // 1: the output goes through shared memory and TMA (maps tmC / tmC2 of the launch are valid)
  long long* trace;            // optional tuning aid of the two-CTA kernel: [grid, 8] nanosecond marks per CTA, or null
};

// B operand maps: one for an ordinary GEMM; one per owner rank when the rows of B (a weight matrix sharded along
// axis 0) live in the owners' memories and are fetched tile by tile over NVLink by (non-multicast) TMA loads.
struct TmapArray {
  CUtensorMap m[8];
};

// `bn` is the N extent of the tile (64, 128 or 256). The tensor maps must be 4-D bf16 maps with 128-byte swizzle:
//   K-major operand : dims (K, rows, batch_lo, batch_hi), box (64, 128 for A / bn for B, 1, 1)
//   MN-major operand: dims (rows, K, batch_lo, batch_hi), box (64, 64, 1, 1)
// With p.tma_store, `tmC` (and `tmC2` for EPI_BIAS_GELU) map the output: same element type as C, box (128 bytes of columns,
// 32 rows, 1, 1), 128-byte swizzle; fp32 outputs need beta 0 or 1. Otherwise both may be null.
cudaError_t launch_gemm(const CUtensorMap& tmA, const TmapArray& tmB, const GemmParams& p, int bn, bool a_mn,
                        bool b_mn, int num_sms, cudaStream_t stream, const CUtensorMap* tmC = nullptr, const CUtensorMap* tmC2 = nullptr);

// The same product on pairs of SMs (tcgen05.mma.cta_group::2, 256 x 256 tiles; gemm_tcgen05_2cta.cu). Maps as above
// with boxes of 128 rows for a K-major operand. No fused softmax, no row-sharded B.
cudaError_t launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, bool a_mn, bool b_mn, int num_sms,
                             cudaStream_t stream, const CUtensorMap* tmC = nullptr, const CUtensorMap* tmC2 = nullptr);

}  // namespace adb200
