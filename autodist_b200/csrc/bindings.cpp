// Python bindings of the sm_100a kernels: tensor-map construction, argument checks, launches on the current stream.
#include <cstdlib>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <mutex>
#include <unordered_map>
#include <vector>

#include "comm.h"
#include "elementwise.h"
#include "gemm_tcgen05.h"

void register_conv(pybind11::module& m);

namespace {

using at::Tensor;
using c10::optional;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    TORCH_CHECK(e == cudaSuccess && p != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

Tensor as4d(const Tensor& t) {
  TORCH_CHECK(t.dim() >= 2 && t.dim() <= 4, "operand must have 2 to 4 dimensions");
  Tensor v = t;
  while (v.dim() < 4) v = v.unsqueeze(0);
  return v;
}

// 4-D bf16 tiled map over a strided view [b_hi, b_lo, outer, inner] (inner stride 1), 128-byte swizzle.
CUtensorMap make_map(const Tensor& v, int box_outer) {
  TORCH_CHECK(v.scalar_type() == at::kBFloat16, "GEMM operands must be bf16");
  TORCH_CHECK(v.stride(3) == 1, "innermost dimension must be contiguous");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(v.data_ptr()) % 16 == 0, "operand base must be 16-byte aligned");
  cuuint64_t dims[4] = {(cuuint64_t)v.size(3), (cuuint64_t)v.size(2), (cuuint64_t)v.size(1), (cuuint64_t)v.size(0)};
  cuuint64_t strides[3];
  int64_t prev = v.size(3);
  for (int i = 0; i < 3; ++i) {
    const int d = 2 - i;   // tensor dim of map dim i+1
    int64_t s = v.size(d) > 1 ? v.stride(d) : prev;
    TORCH_CHECK((s * 2) % 16 == 0 && s > 0, "operand strides must be positive multiples of 8 elements, got ", s);
    strides[i] = (cuuint64_t)s * 2;
    prev = s * v.size(d);
  }
  cuuint32_t box[4] = {64, (cuuint32_t)box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, v.data_ptr(), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

// 4-D map over an output view [b_hi, b_lo, rows, cols] (bf16 or fp32, inner stride 1) for the TMA-store epilogue: boxes of
// 128 bytes of columns x 32 rows, 128-byte swizzle. Returns false when the view cannot be described (a base or a stride
// that is not a multiple of 16 bytes): the caller then keeps the direct stores.
bool make_store_map(const Tensor& v, CUtensorMap* out) {
  const bool f32 = v.scalar_type() == at::kFloat;
  const int64_t esz = f32 ? 4 : 2;
  if (v.stride(3) != 1 || reinterpret_cast<uintptr_t>(v.data_ptr()) % 16 != 0) return false;
  cuuint64_t dims[4] = {(cuuint64_t)v.size(3), (cuuint64_t)v.size(2), (cuuint64_t)v.size(1), (cuuint64_t)v.size(0)};
  cuuint64_t strides[3];
  int64_t prev = v.size(3);
  for (int i = 0; i < 3; ++i) {
    const int d = 2 - i;
    const int64_t s = v.size(d) > 1 ? v.stride(d) : prev;
    if (s <= 0 || (s * esz) % 16 != 0) return false;
    strides[i] = (cuuint64_t)(s * esz);
    prev = s * v.size(d);
  }
  cuuint32_t box[4] = {(cuuint32_t)(128 / esz), 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_fn()(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, v.data_ptr(), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tuning aid: when set (int64 CUDA tensor of at least 8 x SM-count words, zeroed by the caller), launches of the two-CTA
// GEMM record nanosecond marks per CTA into it (see gemm_tcgen05_2cta.cu).
long long* g_gemm_trace = nullptr;
void gemm_set_trace(const optional<Tensor>& t) {
  if (t.has_value()) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong && t->is_contiguous() && t->numel() >= 8LL * num_sms(), "int64 [SMs, 8] needed");
    g_gemm_trace = reinterpret_cast<long long*>(t->data_ptr<int64_t>());
  } else {
    g_gemm_trace = nullptr;
  }
}

// D = alpha * A.B^T (+ epilogue). a: [.., M, K] (K-major) or [.., K, M] (a_mn); b: [.., N, K] or [.., K, N] (b_mn);
// c: [.., M, N] bf16 or fp32 view with unit inner stride.
void gemm_impl(const Tensor& a_, const Tensor& b_, Tensor c_, bool a_mn, bool b_mn, int64_t epilogue, const optional<Tensor>& bias,
               const optional<Tensor>& c2, const optional<Tensor>& aux, double alpha, double beta, Tensor error_flag, int64_t bn,
               const optional<Tensor>& mask, double drop_p, int64_t drop_seed, const optional<Tensor>& drop_step) {
  const c10::cuda::CUDAGuard guard(a_.device());
  Tensor a = as4d(a_), b = as4d(b_), c = as4d(c_);
  const int M = a_mn ? a.size(3) : a.size(2), K = a_mn ? a.size(2) : a.size(3);
  const int N = b_mn ? b.size(3) : b.size(2), Kb = b_mn ? b.size(2) : b.size(3);
  TORCH_CHECK(K == Kb, "contraction extents differ: ", K, " vs ", Kb);
  TORCH_CHECK(a.size(0) == b.size(0) && a.size(1) == b.size(1), "batch dimensions of A and B differ");
  TORCH_CHECK(c.size(0) == a.size(0) && c.size(1) == a.size(1) && c.size(2) == M && c.size(3) == N, "output shape mismatch");
  TORCH_CHECK(c.stride(3) == 1, "output inner stride must be 1");
  // bn: tile width 64 / 128 / 256 of the one-CTA kernel, or 512 = the 256 x 256 tile of the two-CTA kernel; 0 picks one
  // (two CTAs when both extents fill a pair's tile and AUTODIST_GEMM_PAIR is not 0)
  const bool softmax_epi = epilogue == adb200::EPI_SOFTMAX || epilogue == adb200::EPI_SOFTMAX_GRAD;
  static bool pair_unavailable = false;        // set when a cluster launch was refused once (see below)
  const bool auto_bn = bn <= 0;
  if (bn <= 0) {
    static const bool pair_default = [] { const char* e = std::getenv("AUTODIST_GEMM_PAIR"); return e == nullptr || e[0] != '0'; }();
    bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
    // pairs pay off once their 256 x 256 tiles fill the SM pairs, or when a long contraction makes the shared-memory
    // fill per FLOP (what the pair halves for B) the limit
    const int64_t pair_tiles = (int64_t)((M + 255) / 256) * ((N + 255) / 256) * a.size(0) * a.size(1);
    static const int64_t pair_min_k = [] { const char* e = std::getenv("AUTODIST_GEMM_PAIR_MIN_K"); return e != nullptr ? std::atoll(e) : 2048LL; }();
    if (pair_default && !pair_unavailable && bn == 256 && M >= 256 && !softmax_epi && (pair_tiles >= num_sms() / 2 || K >= pair_min_k))
      bn = 512;
  }
  TORCH_CHECK(bn == 64 || bn == 128 || bn == 256 || bn == 512, "bn must be 64, 128, 256 or 512 (two-CTA tile)");
  const bool pair = bn == 512;
  CUtensorMap tmA = make_map(a, a_mn ? 64 : 128);
  adb200::TmapArray tmB;
  tmB.m[0] = make_map(b, b_mn ? 64 : (pair ? 128 : (int)bn));
  for (int i = 1; i < 8; ++i) tmB.m[i] = tmB.m[0];
  adb200::GemmParams p{};
  p.b_shard_rows = 0;
  p.trace = g_gemm_trace;
  p.M = M; p.N = N; p.K = K;
  p.batch_lo = a.size(1); p.batch_hi = a.size(0);
  p.C = c.data_ptr();
  p.ldc = c.stride(2);
  p.strideC_lo = c.size(1) > 1 ? c.stride(1) : 0;
  p.strideC_hi = c.size(0) > 1 ? c.stride(0) : 0;
  TORCH_CHECK(c.scalar_type() == at::kFloat || c.scalar_type() == at::kBFloat16, "output must be fp32 or bf16");
  p.c_is_fp32 = c.scalar_type() == at::kFloat;
  p.epilogue = (int)epilogue;
  p.alpha = (float)alpha;
  p.beta = (float)beta;
  p.bias = nullptr; p.C2 = nullptr; p.aux = nullptr;
  if (epilogue == adb200::EPI_BIAS || epilogue == adb200::EPI_BIAS_GELU || epilogue == adb200::EPI_BIAS_TANH) {
    TORCH_CHECK(bias.has_value() && bias->scalar_type() == at::kFloat && bias->numel() >= N, "fp32 bias of N entries needed");
    p.bias = bias->data_ptr<float>();
  }
  if (epilogue == adb200::EPI_BIAS_GELU) {
    TORCH_CHECK(c2.has_value() && c2->scalar_type() == at::kBFloat16 && !p.c_is_fp32, "bf16 second output needed");
    Tensor c2v = as4d(*c2);
    TORCH_CHECK(c2v.strides() == c.strides(), "second output must share the strides of the first");
    p.C2 = reinterpret_cast<__nv_bfloat16*>(c2v.data_ptr());
  }
  if (epilogue == adb200::EPI_MUL_GELU_GRAD || epilogue == adb200::EPI_ADD) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16 && !p.c_is_fp32, "bf16 auxiliary operand and bf16 output needed");
    Tensor av = as4d(*aux);
    TORCH_CHECK(av.strides() == c.strides(), "pre-activation must share the strides of the output");
    p.aux = reinterpret_cast<const __nv_bfloat16*>(av.data_ptr());
  }
  p.mask = nullptr; p.drop_p = 0.f; p.drop_seed = 0; p.drop_step = nullptr;
  if (epilogue == adb200::EPI_SOFTMAX || epilogue == adb200::EPI_SOFTMAX_GRAD) {
    TORCH_CHECK(bn == 128 && N == 128 && !p.c_is_fp32 && c.stride(2) == 128, "the softmax epilogues need N == 128 and a contiguous bf16 output row");
    if (mask.has_value()) {
      TORCH_CHECK(mask->scalar_type() == at::kFloat && mask->numel() == a.size(0) * 128, "fp32 mask [batch_hi, 128] needed");
      p.mask = mask->data_ptr<float>();
    }
    p.drop_p = (float)drop_p;
    p.drop_seed = (unsigned long long)drop_seed;
    p.drop_step = drop_step.has_value() ? reinterpret_cast<const long long*>(drop_step->data_ptr<int64_t>()) : nullptr;
    if (epilogue == adb200::EPI_SOFTMAX && c2.has_value()) {
      Tensor c2v = as4d(*c2);
      TORCH_CHECK(c2v.scalar_type() == at::kBFloat16 && c2v.strides() == c.strides(), "dropped copy must share the strides of the output");
      p.C2 = reinterpret_cast<__nv_bfloat16*>(c2v.data_ptr());
    }
    if (epilogue == adb200::EPI_SOFTMAX_GRAD) {
      TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16, "probabilities needed");
      Tensor av = as4d(*aux);
      TORCH_CHECK(av.strides() == c.strides(), "probabilities must share the strides of the output");
      p.aux = reinterpret_cast<const __nv_bfloat16*>(av.data_ptr());
    }
  }
  p.error_flag = error_flag.data_ptr<int>();
  // Output through shared memory and TMA (whole lines instead of 16-byte pieces of 32 rows per store instruction) for
  // products large enough to care; AUTODIST_GEMM_TMA_STORE=0 keeps direct stores everywhere.
  static const bool tma_store_default = [] { const char* e = std::getenv("AUTODIST_GEMM_TMA_STORE"); return e == nullptr || e[0] != '0'; }();
  CUtensorMap tmC, tmC2;
  p.tma_store = 0;
  if (tma_store_default && !softmax_epi && bn >= 256 && (!p.c_is_fp32 || p.beta == 0.0f || p.beta == 1.0f) && make_store_map(c, &tmC)) {
    p.tma_store = 1;
    tmC2 = tmC;
    if (epilogue == adb200::EPI_BIAS_GELU && !make_store_map(as4d(*c2), &tmC2)) p.tma_store = 0;
  }
  cudaError_t e = pair ? adb200::launch_gemm_pair(tmA, tmB.m[0], p, a_mn, b_mn, num_sms(), at::cuda::getCurrentCUDAStream(),
                                                  p.tma_store ? &tmC : nullptr, p.tma_store ? &tmC2 : nullptr)
                       : adb200::launch_gemm(tmA, tmB, p, (int)bn, a_mn, b_mn, num_sms(), at::cuda::getCurrentCUDAStream(),
                                             p.tma_store ? &tmC : nullptr, p.tma_store ? &tmC2 : nullptr);
  if (pair && auto_bn && e != cudaSuccess) {
    // A device (or partition of one) that cannot schedule clusters of two refuses the launch: remember it and run this and
    // every later product on the one-CTA kernel.
    (void)cudaGetLastError();
    pair_unavailable = true;
    tmB.m[0] = make_map(b, b_mn ? 64 : 256);
    for (int i = 1; i < 8; ++i) tmB.m[i] = tmB.m[0];
    e = adb200::launch_gemm(tmA, tmB, p, 256, a_mn, b_mn, num_sms(), at::cuda::getCurrentCUDAStream(), p.tma_store ? &tmC : nullptr,
                            p.tma_store ? &tmC2 : nullptr);
  }
  TORCH_CHECK(e == cudaSuccess, "GEMM launch failed: ", cudaGetErrorString(e));
}

void gemm(const Tensor& a, const Tensor& b, Tensor c, bool a_mn, bool b_mn, int64_t epilogue, const optional<Tensor>& bias,
          const optional<Tensor>& c2, const optional<Tensor>& aux, double alpha, double beta, Tensor error_flag, int64_t bn) {
  TORCH_CHECK(epilogue <= adb200::EPI_BIAS_TANH, "use gemm_softmax for the softmax epilogues");
  gemm_impl(a, b, c, a_mn, b_mn, epilogue, bias, c2, aux, alpha, beta, error_flag, bn, c10::nullopt, 0.0, 0, c10::nullopt);
}

// Attention products with the row softmax in the epilogue (rows of 128):
//   grad == false: c = softmax(alpha * a.b^T + mask), c2 (optional) = dropout(c)
//   grad == true : c = alpha * P * (d - sum(d * P)) with d = (a.b^T) * dropout mask and P = aux
void gemm_softmax(const Tensor& a, const Tensor& b, Tensor c, const optional<Tensor>& c2, const optional<Tensor>& mask,
                  const optional<Tensor>& aux, bool grad, double alpha, double drop_p, int64_t seed, const optional<Tensor>& step,
                  Tensor error_flag) {
  gemm_impl(a, b, c, false, false, grad ? adb200::EPI_SOFTMAX_GRAD : adb200::EPI_SOFTMAX, c10::nullopt, c2, aux, alpha, 0.0, error_flag,
            128, mask, drop_p, seed, step);
}

// Y = A . W^T (+ bias) where W [N, K] is split by rows into `world` equal shards that live in the owners' symmetric
// memory: every B tile is fetched from its owner by a TMA load over NVLink inside the GEMM (no gathered copy of W).
// shard_ptrs: one device address per owner (host list), each a contiguous bf16 [N / world, K] block.
void gemm_gathered_b(const Tensor& a_, const std::vector<int64_t>& shard_ptrs, int64_t rows_per_shard, Tensor c_, int64_t epilogue,
                     const optional<Tensor>& bias, Tensor error_flag, int64_t bn) {
  const c10::cuda::CUDAGuard guard(a_.device());
  Tensor a = as4d(a_), c = as4d(c_);
  const int world = (int)shard_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8, "1 to 8 shards");
  const int M = a.size(2), K = a.size(3);
  const int N = (int)rows_per_shard * world;
  TORCH_CHECK(a.size(0) == 1 && a.size(1) == 1, "the gathered-weight GEMM is not batched");
  TORCH_CHECK(c.size(2) == M && c.size(3) == N && c.stride(3) == 1, "output shape mismatch");
  if (bn <= 0) bn = rows_per_shard % 256 == 0 ? 256 : (rows_per_shard % 128 == 0 ? 128 : 64);
  TORCH_CHECK(rows_per_shard % bn == 0, "rows per shard must be a multiple of the tile width ", bn);
  TORCH_CHECK(K % 8 == 0, "K must be a multiple of 8");
  CUtensorMap tmA = make_map(a, 128);
  adb200::TmapArray tmB;
  for (int s = 0; s < 8; ++s) {
    const int src = s < world ? s : 0;
    cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)rows_per_shard, 1, 1};
    cuuint64_t strides[3] = {(cuuint64_t)K * 2, (cuuint64_t)K * 2 * rows_per_shard, (cuuint64_t)K * 2 * rows_per_shard};
    cuuint32_t box[4] = {64, (cuuint32_t)bn, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode_fn()(&tmB.m[s], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, reinterpret_cast<void*>(shard_ptrs[src]), dims, strides, box,
                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for shard ", s, " with code ", (int)r);
  }
  adb200::GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.batch_lo = 1; p.batch_hi = 1;
  p.C = c.data_ptr(); p.ldc = c.stride(2); p.strideC_lo = 0; p.strideC_hi = 0;
  p.c_is_fp32 = c.scalar_type() == at::kFloat;
  p.epilogue = (int)epilogue; p.alpha = 1.0f; p.beta = 0.0f;
  p.bias = nullptr; p.C2 = nullptr; p.aux = nullptr;
  if (epilogue == adb200::EPI_BIAS) {
    TORCH_CHECK(bias.has_value() && bias->scalar_type() == at::kFloat && bias->numel() >= N, "fp32 bias of N entries needed");
    p.bias = bias->data_ptr<float>();
  } else {
    TORCH_CHECK(epilogue == adb200::EPI_NONE, "only the plain and bias epilogues are offered here");
  }
  p.error_flag = error_flag.data_ptr<int>();
  p.b_shard_rows = (int)rows_per_shard;
  cudaError_t e = adb200::launch_gemm(tmA, tmB, p, (int)bn, false, false, num_sms(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "GEMM launch failed: ", cudaGetErrorString(e));
}

// dX = dY . W where W [N_out, K_in] is split by rows into `world` equal shards in the owners' memories (the input gradient of
// gemm_gathered_b's layer): W is the MN-major B operand and every 64-row K block is fetched from the owner of those rows.
void gemm_gathered_bt(const Tensor& a_, const std::vector<int64_t>& shard_ptrs, int64_t rows_per_shard, int64_t cols, Tensor c_, Tensor error_flag) {
  const c10::cuda::CUDAGuard guard(a_.device());
  Tensor a = as4d(a_), c = as4d(c_);
  const int world = (int)shard_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8, "1 to 8 shards");
  const int M = a.size(2), K = a.size(3);
  TORCH_CHECK(K == rows_per_shard * world, "dY width must equal the number of weight rows");
  TORCH_CHECK(a.size(0) == 1 && a.size(1) == 1, "the gathered-weight GEMM is not batched");
  TORCH_CHECK(c.size(2) == M && c.size(3) == cols && c.stride(3) == 1, "output shape mismatch");
  TORCH_CHECK(rows_per_shard % 64 == 0 && cols % 8 == 0, "rows per shard must be a multiple of 64 and the width a multiple of 8");
  const int64_t bn = cols >= 256 ? 256 : (cols > 64 ? 128 : 64);
  CUtensorMap tmA = make_map(a, 128);
  adb200::TmapArray tmB;
  for (int s = 0; s < 8; ++s) {
    const int src = s < world ? s : 0;
    cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows_per_shard, 1, 1};
    cuuint64_t strides[3] = {(cuuint64_t)cols * 2, (cuuint64_t)cols * 2 * rows_per_shard, (cuuint64_t)cols * 2 * rows_per_shard};
    cuuint32_t box[4] = {64, 64, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode_fn()(&tmB.m[s], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, reinterpret_cast<void*>(shard_ptrs[src]), dims, strides, box,
                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed for shard ", s, " with code ", (int)r);
  }
  adb200::GemmParams p{};
  p.M = M; p.N = (int)cols; p.K = K; p.batch_lo = 1; p.batch_hi = 1;
  p.C = c.data_ptr(); p.ldc = c.stride(2); p.strideC_lo = 0; p.strideC_hi = 0;
  p.c_is_fp32 = c.scalar_type() == at::kFloat;
  p.epilogue = adb200::EPI_NONE; p.alpha = 1.0f; p.beta = 0.0f;
  p.error_flag = error_flag.data_ptr<int>();
  p.b_shard_rows = (int)rows_per_shard;
  cudaError_t e = adb200::launch_gemm(tmA, tmB, p, (int)bn, false, true, num_sms(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "GEMM launch failed: ", cudaGetErrorString(e));
}

#define BF(t) reinterpret_cast<__nv_bfloat16*>((t).data_ptr())
#define CBF(t) reinterpret_cast<const __nv_bfloat16*>((t).data_ptr())
#define OPT_BF(t) ((t).has_value() ? reinterpret_cast<__nv_bfloat16*>((t)->data_ptr()) : nullptr)
#define OPT_F(t) ((t).has_value() ? (t)->data_ptr<float>() : nullptr)
#define OPT_I64(t) ((t).has_value() ? (t)->data_ptr<int64_t>() : nullptr)
#define OPT_LL(t) ((t).has_value() ? reinterpret_cast<const long long*>((t)->data_ptr<int64_t>()) : nullptr)
#define STREAM at::cuda::getCurrentCUDAStream()

void ln_fwd(const Tensor& x, const optional<Tensor>& res, const Tensor& gamma, const Tensor& beta, const optional<Tensor>& z, Tensor y,
            Tensor mean, Tensor rstd, double eps, double p_drop, int64_t seed, const optional<Tensor>& step) {
  const int H = x.size(-1), rows = x.numel() / H;
  TORCH_CHECK(H % 8 == 0 && H <= 1024, "layernorm width must be a multiple of 8 and at most 1024");
  adb200::ln_fwd(CBF(x), OPT_BF(res), gamma.data_ptr<float>(), beta.data_ptr<float>(), OPT_BF(z), BF(y), mean.data_ptr<float>(),
                 rstd.data_ptr<float>(), rows, H, (float)eps, (float)p_drop, (uint64_t)seed, OPT_LL(step), STREAM);
}
// part: fp32 scratch of ln_bwd_part_floats(H) elements that must be ZERO on entry (allocate it with zeros once); it is zero again on
// return. dsum (optional, fp32 [H]): column sums of the tensor handed to the layer in front of the residual connection (dx when the dropout
// copy is written, else dz) - the bias gradient of that layer, produced without another pass over the tensor.
void ln_bwd(const Tensor& dy, const Tensor& z, const Tensor& mean, const Tensor& rstd, const Tensor& gamma, const optional<Tensor>& dz_add,
            Tensor dz, const optional<Tensor>& dx, Tensor part, Tensor dgamma, Tensor dbeta, double p_drop, int64_t seed,
            const optional<Tensor>& step, bool accumulate, const optional<Tensor>& dsum) {
  const int H = dy.size(-1), rows = dy.numel() / H;
  TORCH_CHECK(H % 8 == 0 && H <= 1024, "layernorm width must be a multiple of 8 and at most 1024");
  TORCH_CHECK(part.numel() >= adb200::ln_bwd_part_floats(H), "partial buffer too small (ln_bwd_part_floats(H) floats, zero-filled)");
  if (dsum.has_value()) TORCH_CHECK(dsum->scalar_type() == at::kFloat && dsum->numel() >= H, "dsum must be fp32 [H]");
  adb200::ln_bwd(CBF(dy), CBF(z), mean.data_ptr<float>(), rstd.data_ptr<float>(), gamma.data_ptr<float>(), OPT_BF(dz_add), BF(dz),
                 OPT_BF(dx), part.data_ptr<float>(), dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), OPT_F(dsum), rows, H, (float)p_drop,
                 (uint64_t)seed, OPT_LL(step), accumulate ? 1 : 0, STREAM);
}
void embed_sum(const Tensor& word, const Tensor& pos, const Tensor& type, const Tensor& ids, const optional<Tensor>& tt, Tensor z, int64_t S,
               const optional<Tensor>& error_flag) {
  const int H = word.size(1), rows = ids.numel();
  TORCH_CHECK(pos.size(0) >= S, "position table shorter than the sequence");
  adb200::embed_sum(CBF(word), CBF(pos), CBF(type), ids.data_ptr<int64_t>(), OPT_I64(tt), BF(z), rows, (int)S, H, word.size(0), type.size(0),
                    error_flag.has_value() ? error_flag->data_ptr<int>() : nullptr, STREAM);
}
void scatter_add_rows(Tensor dst, const Tensor& idx, const Tensor& src, double scale) {
  adb200::scatter_add_rows(dst.data_ptr<float>(), idx.data_ptr<int64_t>(), CBF(src), idx.numel(), src.size(-1), (float)scale, STREAM);
}
void strided_rowsum(const Tensor& x, Tensor out, int64_t keys, int64_t stride, int64_t count) {
  adb200::strided_rowsum(CBF(x), out.data_ptr<float>(), keys, stride, count, x.size(-1), STREAM);
}
void keyed_colsum(const Tensor& x, const optional<Tensor>& key, Tensor part, Tensor out, int64_t keys, bool accumulate) {
  const int H = x.size(-1), rows = x.numel() / H;
  TORCH_CHECK(H % 8 == 0, "width must be a multiple of 8");
  TORCH_CHECK(part.numel() >= (long long)adb200::colsum_parts(rows) * keys * H, "partial buffer too small");
  adb200::keyed_colsum(CBF(x), OPT_I64(key), part.data_ptr<float>(), out.data_ptr<float>(), rows, H, keys, accumulate ? 1 : 0, STREAM);
}
void gather_rows(const Tensor& src, const Tensor& idx, Tensor out) {
  adb200::gather_rows(CBF(src), idx.data_ptr<int64_t>(), BF(out), idx.numel(), src.size(-1), STREAM);
}
void gather_rows_f32(const Tensor& src, const Tensor& idx, Tensor out) {
  TORCH_CHECK(src.scalar_type() == at::kFloat && src.is_contiguous() && src.size(-1) % 8 == 0, "fp32 contiguous table, width a multiple of 8");
  adb200::gather_rows_f32(src.data_ptr<float>(), idx.data_ptr<int64_t>(), BF(out), idx.numel(), src.size(-1), STREAM);
}
void scatter_add_rows_bf16(Tensor dst, const Tensor& idx, const Tensor& src) {
  adb200::scatter_add_rows_bf16(BF(dst), idx.data_ptr<int64_t>(), CBF(src), idx.numel(), src.size(-1), STREAM);
}
void softmax_fwd(const Tensor& x, const optional<Tensor>& mask, Tensor p, const optional<Tensor>& p_drop, double scale, double pd,
                 int64_t seed, const optional<Tensor>& step) {
  const int S = x.size(-1);
  TORCH_CHECK(adb200::softmax_supported(S) && x.dim() == 4, "scores must be [B, heads, S, S] with S in {64, 128, 256, 512, 1024}");
  const long long rows = x.numel() / S;
  adb200::softmax_fwd(CBF(x), OPT_F(mask), BF(p), OPT_BF(p_drop), rows, S, (int)(x.size(1) * x.size(2)), (float)scale, (float)pd,
                      (uint64_t)seed, OPT_LL(step), STREAM);
}
void softmax_bwd(Tensor dp, const Tensor& p, double scale, double pd, int64_t seed, const optional<Tensor>& step) {
  const int S = p.size(-1);
  adb200::softmax_bwd(BF(dp), CBF(p), p.numel() / S, S, (float)scale, (float)pd, (uint64_t)seed, OPT_LL(step), STREAM);
}
void xent(Tensor logits, const Tensor& labels, const optional<Tensor>& weights, Tensor denom, Tensor loss_sum, int64_t V, double loss_scale,
          bool compute_denom, double eps) {
  const int ld = logits.size(-1), rows = logits.numel() / ld;
  if (compute_denom) {
    TORCH_CHECK(weights.has_value(), "weights needed to compute the denominator");
    adb200::weight_sum(weights->data_ptr<float>(), rows, denom.data_ptr<float>(), (float)eps, STREAM);
  }
  adb200::xent(BF(logits), labels.data_ptr<int64_t>(), OPT_F(weights), denom.data_ptr<float>(), loss_sum.data_ptr<float>(), rows, (int)V, ld,
               (float)loss_scale, STREAM);
}
void gelu_bwd(const Tensor& dy, const Tensor& u, Tensor dx) { adb200::gelu_bwd(CBF(dy), CBF(u), BF(dx), u.numel(), STREAM); }
void tanh_bwd(const Tensor& dy, const Tensor& y, Tensor dx) { adb200::tanh_bwd(CBF(dy), CBF(y), BF(dx), y.numel(), STREAM); }
void add_bf16(const Tensor& a, const Tensor& b, Tensor out) {
  TORCH_CHECK(a.numel() % 8 == 0, "length must be a multiple of 8");
  adb200::add_bf16(CBF(a), CBF(b), BF(out), a.numel(), STREAM);
}
void adam_update(Tensor p, const Tensor& g, Tensor m, Tensor v, const optional<Tensor>& p16, const Tensor& lr, double b1, double b2, double eps,
                 double wd, bool decoupled, const Tensor& step, double grad_scale) {
  adb200::adam_update(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), OPT_BF(p16), p.numel(),
                      lr.data_ptr<float>(), (float)b1, (float)b2, (float)eps, (float)wd, decoupled ? 1 : 0,
                      reinterpret_cast<const long long*>(step.data_ptr<int64_t>()), (float)grad_scale, STREAM);
}
void sgd_update(Tensor p, const Tensor& g, const optional<Tensor>& mom, const optional<Tensor>& p16, const Tensor& lr, double momentum,
                double dampening, double wd, bool nesterov, const Tensor& step, double grad_scale) {
  adb200::sgd_update(p.data_ptr<float>(), g.data_ptr<float>(), OPT_F(mom), OPT_BF(p16), p.numel(), lr.data_ptr<float>(), (float)momentum,
                     (float)dampening, (float)wd, nesterov ? 1 : 0, reinterpret_cast<const long long*>(step.data_ptr<int64_t>()),
                     (float)grad_scale, STREAM);
}
void adagrad_update(Tensor p, const Tensor& g, Tensor acc, const optional<Tensor>& p16, const Tensor& lr, double eps, double wd, double grad_scale) {
  adb200::adagrad_update(p.data_ptr<float>(), g.data_ptr<float>(), acc.data_ptr<float>(), OPT_BF(p16), p.numel(), lr.data_ptr<float>(),
                         (float)eps, (float)wd, (float)grad_scale, STREAM);
}
void sparse_rows_update(Tensor p, const optional<Tensor>& s1, const optional<Tensor>& s2, const optional<Tensor>& p16, const Tensor& rows,
                        const Tensor& g, int64_t kind, const Tensor& lr, double b1, double b2, double eps, const optional<Tensor>& step,
                        double grad_scale) {
  TORCH_CHECK(p.dim() == 2 && p.is_contiguous() && p.scalar_type() == at::kFloat, "parameter must be a contiguous fp32 [V, H] table");
  TORCH_CHECK(g.scalar_type() == at::kFloat && g.is_contiguous() && g.dim() == 2 && g.size(0) == rows.numel() && g.size(1) == p.size(1),
              "gradient rows must be fp32 [n, H]");
  TORCH_CHECK(rows.scalar_type() == at::kLong && rows.is_contiguous(), "row ids must be int64");
  TORCH_CHECK(kind == 0 || (s1.has_value() && s1->sizes() == p.sizes()), "state 1 must match the table");
  TORCH_CHECK(kind != 1 || (s2.has_value() && s2->sizes() == p.sizes() && step.has_value()), "lazy Adam needs both moments and the step");
  adb200::sparse_rows_update(p.data_ptr<float>(), OPT_F(s1), OPT_F(s2), OPT_BF(p16), rows.data_ptr<int64_t>(), g.data_ptr<float>(),
                             (int)rows.numel(), (int)p.size(1), p.size(0), (int)kind, lr.data_ptr<float>(), (float)b1, (float)b2,
                             (float)eps, OPT_LL(step), (float)grad_scale, STREAM);
}
// Owner-side update of the flagged rows of a shard (p, g, s1, s2: fp32 [rows, H]; flags: uint8 [rows]); clears what it used.
void flagged_rows_update(Tensor p, const optional<Tensor>& s1, const optional<Tensor>& s2, const optional<Tensor>& p16, Tensor g, Tensor flags,
                         int64_t rows, int64_t H, int64_t kind, const Tensor& lr, double b1, double b2, double eps, const optional<Tensor>& step) {
  TORCH_CHECK(p.scalar_type() == at::kFloat && g.scalar_type() == at::kFloat && flags.scalar_type() == at::kByte, "fp32 table / gradient, uint8 flags");
  TORCH_CHECK(p.numel() >= rows * H && g.numel() >= rows * H && flags.numel() >= rows, "buffers smaller than rows x H");
  TORCH_CHECK(kind == 0 || s1.has_value(), "state 1 needed");
  TORCH_CHECK(kind != 1 || (s2.has_value() && step.has_value()), "Adam needs both moments and the step");
  adb200::flagged_rows_update(p.data_ptr<float>(), OPT_F(s1), OPT_F(s2), OPT_BF(p16), g.data_ptr<float>(), flags.data_ptr<uint8_t>(), rows, (int)H,
                              (int)kind, lr.data_ptr<float>(), (float)b1, (float)b2, (float)eps, OPT_LL(step), STREAM);
}
void lstm_cell_fwd(const Tensor& gates, const Tensor& c_prev, Tensor c, Tensor h, double forget_bias) {
  const int B = c_prev.size(0), S = c_prev.size(1);
  TORCH_CHECK(gates.scalar_type() == at::kFloat && gates.size(1) == 4 * S && gates.is_contiguous(), "gates must be fp32 [B, 4S]");
  adb200::lstm_cell_fwd(gates.data_ptr<float>(), c_prev.data_ptr<float>(), c.data_ptr<float>(), BF(h), B, S, (float)forget_bias, STREAM);
}
void lstm_cell_bwd(const Tensor& gates, const Tensor& c_prev, const Tensor& c, const Tensor& dh, const optional<Tensor>& dc_next,
                   Tensor dgates, Tensor dc_prev, double forget_bias) {
  const int B = c_prev.size(0), S = c_prev.size(1);
  adb200::lstm_cell_bwd(gates.data_ptr<float>(), c_prev.data_ptr<float>(), c.data_ptr<float>(), dh.data_ptr<float>(), OPT_F(dc_next),
                        dgates.data_ptr<float>(), dc_prev.data_ptr<float>(), B, S, (float)forget_bias, STREAM);
}
void sumsq(const Tensor& x, Tensor acc, double weight) { adb200::sumsq(x.data_ptr<float>(), x.numel(), acc.data_ptr<float>(), (float)weight, STREAM); }
void clip_scale(Tensor x, const Tensor& acc, double max_norm) { adb200::clip_scale(x.data_ptr<float>(), x.numel(), acc.data_ptr<float>(), (float)max_norm, STREAM); }
// Batch-norm over a channels-last matrix x [rows, C] (training mode statistics), optional residual addend and fused ReLU:
// y = relu?(bn(x) + res). `sums` (optional, fp32 [2, C]) holds sum x and sum x^2 already (from the convolution's epilogue).
void bn_fwd(const Tensor& x, const Tensor& gamma, const Tensor& beta, const optional<Tensor>& res, Tensor y, Tensor mean, Tensor rstd,
            double eps, bool relu, const optional<Tensor>& sums_in, const optional<Tensor>& run_mean, const optional<Tensor>& run_var,
            const optional<Tensor>& batches, double momentum) {
  const int C = x.size(-1), rows = x.numel() / C;
  float* rm = nullptr; float* rv = nullptr; long long* nb = nullptr;
  if (run_mean.has_value()) {
    TORCH_CHECK(run_var.has_value() && run_mean->scalar_type() == at::kFloat && run_var->scalar_type() == at::kFloat && run_mean->numel() == C &&
                run_var->numel() == C && run_mean->is_contiguous() && run_var->is_contiguous(), "running statistics must be fp32 [C]");
    rm = run_mean->data_ptr<float>(); rv = run_var->data_ptr<float>();
  }
  if (batches.has_value()) nb = reinterpret_cast<long long*>(batches->data_ptr<int64_t>());
  TORCH_CHECK(C % 8 == 0 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "x must be contiguous bf16 [.., C], C % 8 == 0");
  TORCH_CHECK(y.is_contiguous() && y.numel() == x.numel() && mean.numel() == C && rstd.numel() == C && gamma.numel() == C && beta.numel() == C,
              "output and per-channel tensors must match x");
  if (res.has_value()) TORCH_CHECK(res->is_contiguous() && res->numel() == x.numel() && res->scalar_type() == at::kBFloat16, "residual must match x");
  if (sums_in.has_value()) {
    TORCH_CHECK(sums_in->scalar_type() == at::kFloat && sums_in->numel() == 2 * C && sums_in->is_contiguous(), "sums must be fp32 [2, C]");
    adb200::bn_fwd(CBF(x), gamma.data_ptr<float>(), beta.data_ptr<float>(), OPT_BF(res), BF(y), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                   nullptr, sums_in->data_ptr<float>(), nullptr, rows, C, (float)eps, relu ? 1 : 0, 1, rm, rv, nb, (float)momentum, STREAM);
    return;
  }
  Tensor part = at::empty({(int64_t)adb200::bn_parts(rows, C) * 2 * C}, x.options().dtype(at::kFloat));
  Tensor sums = at::empty({2 * C}, x.options().dtype(at::kFloat));
  adb200::bn_fwd(CBF(x), gamma.data_ptr<float>(), beta.data_ptr<float>(), OPT_BF(res), BF(y), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                 part.data_ptr<float>(), sums.data_ptr<float>(), nullptr, rows, C, (float)eps, relu ? 1 : 0, 0, rm, rv, nb, (float)momentum,
                 STREAM);
}
// Returns [dbeta, dgamma] stacked as a [2, C] fp32 tensor; writes dx and (optional) dres = dy masked by the ReLU.
// dgamma_acc / dbeta_acc (optional, fp32 [C]): the batch-norm parameters' gradient buffers; the sums are added into them.
Tensor bn_bwd(const Tensor& dy, const Tensor& x, const Tensor& y, const Tensor& mean, const Tensor& rstd, const Tensor& gamma, Tensor dx,
              const optional<Tensor>& dres, bool relu, const optional<Tensor>& dgamma_acc, const optional<Tensor>& dbeta_acc) {
  const int C = x.size(-1), rows = x.numel() / C;
  TORCH_CHECK(C % 8 == 0 && C <= 16384 && x.is_contiguous() && dy.is_contiguous() && dx.is_contiguous() && dy.numel() == x.numel() && dx.numel() == x.numel(),
              "dy, x, dx must be contiguous bf16 [.., C] of one shape, C % 8 == 0");
  if (dres.has_value()) TORCH_CHECK(dres->is_contiguous() && dres->numel() == x.numel() && dres->scalar_type() == at::kBFloat16, "dres must match x");
  // partial sums: a per-device scratch that the kernels keep zero between calls (they add into it and clear what they read);
  // batch-norm backward calls of one device are issued on one stream
  static std::unordered_map<int, Tensor> scratch;
  Tensor& part = scratch[x.get_device()];
  if (!part.defined() || part.numel() < adb200::bn_bwd_part_floats(C))
    part = at::zeros({(int64_t)adb200::bn_bwd_part_floats(std::max(C, 4096))}, x.options().dtype(at::kFloat));
  Tensor sums = at::empty({5, C}, x.options().dtype(at::kFloat));              // [dbeta, dgamma, A, B, K]
  adb200::bn_bwd(CBF(dy), CBF(x), CBF(y), mean.data_ptr<float>(), rstd.data_ptr<float>(), gamma.data_ptr<float>(), BF(dx), OPT_BF(dres),
                 part.data_ptr<float>(), sums.data_ptr<float>(), sums.data_ptr<float>() + 2 * C, rows, C, relu ? 1 : 0, OPT_F(dgamma_acc),
                 OPT_F(dbeta_acc), STREAM);
  return sums.narrow(0, 0, 2);
}
// code: uint8 [N, Ho, Wo, C], the window position of each output's first maximum
void maxpool_fwd(const Tensor& x, Tensor y, Tensor code, int64_t k, int64_t stride, int64_t pad) {
  TORCH_CHECK(x.dim() == 4 && x.is_contiguous() && x.size(3) % 8 == 0 && x.scalar_type() == at::kBFloat16, "x must be contiguous bf16 [N, H, W, C]");
  TORCH_CHECK(y.is_contiguous() && code.is_contiguous() && code.scalar_type() == at::kByte && code.numel() == y.numel() && k * k < 255 &&
              y.size(0) == x.size(0) && y.size(3) == x.size(3), "y / code must be [N, Ho, Wo, C]");
  adb200::maxpool_fwd(CBF(x), BF(y), code.data_ptr<uint8_t>(), x.size(0), x.size(1), x.size(2), x.size(3), k, stride, pad, y.size(1),
                      y.size(2), STREAM);
}
void maxpool_bwd(const Tensor& code, const Tensor& dy, Tensor dx, int64_t k, int64_t stride, int64_t pad) {
  TORCH_CHECK(dx.dim() == 4 && dx.is_contiguous() && dy.is_contiguous() && code.is_contiguous() && code.numel() == dy.numel() &&
              dx.size(3) % 8 == 0, "dx [N, H, W, C], dy / code [N, Ho, Wo, C], contiguous");
  adb200::maxpool_bwd(code.data_ptr<uint8_t>(), CBF(dy), BF(dx), dx.size(0), dx.size(1), dx.size(2), dx.size(3), k, stride, pad, dy.size(1),
                      dy.size(2), STREAM);
}
void im2col(const Tensor& x, Tensor cols, int64_t KH, int64_t KW, int64_t stride, int64_t pad) {
  TORCH_CHECK(x.dim() == 4 && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && x.size(3) % 8 == 0, "x must be contiguous bf16 [N, H, W, C], C % 8 == 0");
  const int N = x.size(0), H = x.size(1), W = x.size(2), C = x.size(3);
  const int Ho = (H + 2 * pad - KH) / stride + 1, Wo = (W + 2 * pad - KW) / stride + 1;
  TORCH_CHECK(cols.numel() == (int64_t)N * Ho * Wo * KH * KW * C, "cols has the wrong size");
  adb200::im2col(CBF(x), BF(cols), N, H, W, C, KH, KW, stride, pad, Ho, Wo, STREAM);
}
void col2im(const Tensor& dcols, Tensor dx, int64_t KH, int64_t KW, int64_t stride, int64_t pad) {
  TORCH_CHECK(dx.dim() == 4 && dx.is_contiguous() && dx.scalar_type() == at::kBFloat16 && dx.size(3) % 8 == 0, "dx must be contiguous bf16 [N, H, W, C]");
  const int N = dx.size(0), H = dx.size(1), W = dx.size(2), C = dx.size(3);
  const int Ho = (H + 2 * pad - KH) / stride + 1, Wo = (W + 2 * pad - KW) / stride + 1;
  TORCH_CHECK(dcols.numel() == (int64_t)N * Ho * Wo * KH * KW * C, "dcols has the wrong size");
  adb200::col2im(CBF(dcols), BF(dx), N, H, W, C, KH, KW, stride, pad, Ho, Wo, STREAM);
}
// Image [N, C, H, W] (any strides, fp32 or bf16, C <= 8) -> bf16 [N, Hp, Wp, 8] with the pixels at offset (pad, pad) and zeros elsewhere.
void pad_image8(const Tensor& x, Tensor xp, int64_t pad) {
  TORCH_CHECK(x.dim() == 4 && x.size(1) <= 8 && (x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16), "x must be [N, C<=8, H, W] fp32 or bf16");
  TORCH_CHECK(xp.dim() == 4 && xp.size(3) == 8 && xp.is_contiguous() && xp.scalar_type() == at::kBFloat16 && xp.size(0) == x.size(0) &&
              xp.size(1) >= x.size(2) + pad && xp.size(2) >= x.size(3) + pad, "xp must be contiguous bf16 [N, Hp, Wp, 8]");
  adb200::pad_image8(x.data_ptr(), x.scalar_type() == at::kFloat ? 1 : 0, x.stride(0), x.stride(1), x.stride(2), x.stride(3), x.size(0),
                     x.size(1), x.size(2), x.size(3), BF(xp), xp.size(1), xp.size(2), (int)pad, STREAM);
}
// Bias gradient of a convolution over channels-last dy [.., C]: out (fp32 [C]) = column sums of dy, or of dy masked by y > 0
// when the convolution had a fused ReLU, in which case the masked gradient is also written to dx. accumulate: out += sums.
void relu_bwd_colsum(const Tensor& dy, const optional<Tensor>& y, const optional<Tensor>& dx, Tensor out, bool accumulate) {
  const int C = dy.size(-1), rows = dy.numel() / C;
  TORCH_CHECK(C % 8 == 0 && dy.is_contiguous() && dy.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kFloat && out.numel() == C &&
              out.is_contiguous(), "dy must be contiguous bf16 [.., C] (C % 8 == 0), out fp32 [C]");
  TORCH_CHECK(y.has_value() == dx.has_value(), "y and dx come together");
  if (y.has_value()) TORCH_CHECK(y->is_contiguous() && dx->is_contiguous() && y->numel() == dy.numel() && dx->numel() == dy.numel(), "y, dx must match dy");
  Tensor part = at::empty({(int64_t)adb200::bn_parts(rows, C) * C}, dy.options().dtype(at::kFloat));
  adb200::relu_bwd_colsum(CBF(dy), y.has_value() ? CBF(*y) : nullptr, dx.has_value() ? BF(*dx) : nullptr, part.data_ptr<float>(),
                          out.data_ptr<float>(), rows, C, accumulate ? 1 : 0, STREAM);
}
void relu_bwd(const Tensor& dy, const Tensor& y, Tensor dx) {
  TORCH_CHECK(dy.is_contiguous() && y.is_contiguous() && dx.is_contiguous() && dy.numel() == y.numel() && dx.numel() == y.numel() && y.numel() % 8 == 0,
              "contiguous bf16 tensors of one size (a multiple of 8)");
  adb200::relu_bwd(CBF(dy), CBF(y), BF(dx), y.numel(), STREAM);
}
void psgd_p(Tensor M, const optional<Tensor>& err, const Tensor& Q, Tensor P) {
  const int m = M.size(0), n = M.size(1), r = Q.size(1);
  TORCH_CHECK(r >= 1 && r <= 4 && M.is_contiguous() && Q.is_contiguous() && P.is_contiguous(), "rank 1..4, contiguous fp32 operands");
  adb200::psgd_p(M.data_ptr<float>(), OPT_F(err), Q.data_ptr<float>(), P.data_ptr<float>(), m, n, r, STREAM);
}
void psgd_q(const Tensor& M, const Tensor& P, Tensor Qn) {
  const int m = M.size(0), n = M.size(1), r = P.size(1);
  TORCH_CHECK(r >= 1 && r <= 4 && M.is_contiguous() && P.is_contiguous() && Qn.is_contiguous(), "rank 1..4, contiguous fp32 operands");
  adb200::psgd_q(M.data_ptr<float>(), P.data_ptr<float>(), Qn.data_ptr<float>(), m, n, r, STREAM);
}
void psgd_d(Tensor M, Tensor err, const Tensor& P, const Tensor& Q) {
  const int m = M.size(0), n = M.size(1), r = P.size(1);
  adb200::psgd_d(M.data_ptr<float>(), err.data_ptr<float>(), P.data_ptr<float>(), Q.data_ptr<float>(), m, n, r, STREAM);
}
// One pass of PowerSGD over every matrix of the step (see elementwise.cu). off / p_off / q_off / *_prefix: int64 device tensors,
// m / n: int32 device tensors; phase 0 = P = (grad + err) Q, 1 = orthogonalise P, 2 = Q = grad^T P, 3 = err = grad - P Q^T, grad = P Q^T.
void psgd_batched(int64_t phase, Tensor grad, Tensor err, Tensor P, Tensor Q, const Tensor& off, const Tensor& m, const Tensor& n,
                  const Tensor& p_off, const Tensor& q_off, const Tensor& row_prefix, const Tensor& blk_prefix, const Tensor& elem_prefix,
                  int64_t rank, int64_t rows, int64_t blocks, int64_t elems) {
  const int nmat = m.numel();
  TORCH_CHECK(rank >= 1 && rank <= 4 && grad.scalar_type() == at::kFloat && err.scalar_type() == at::kFloat && P.scalar_type() == at::kFloat &&
              Q.scalar_type() == at::kFloat, "fp32 buffers, rank 1..4");
  TORCH_CHECK(off.numel() == nmat && n.numel() == nmat && p_off.numel() == nmat && q_off.numel() == nmat && row_prefix.numel() == nmat + 1 &&
              blk_prefix.numel() == nmat + 1 && elem_prefix.numel() == nmat + 1 && m.scalar_type() == at::kInt && n.scalar_type() == at::kInt,
              "table arrays of the wrong length or type");
  auto ll = [](const Tensor& t) { return reinterpret_cast<const long long*>(t.data_ptr<int64_t>()); };
  adb200::psgd_batched((int)phase, grad.data_ptr<float>(), err.data_ptr<float>(), P.data_ptr<float>(), Q.data_ptr<float>(), ll(off),
                       m.data_ptr<int>(), n.data_ptr<int>(), ll(p_off), ll(q_off), ll(row_prefix), ll(blk_prefix), ll(elem_prefix), nmat, (int)rank,
                       rows, blocks, elems, STREAM);
}
void cast_f32_bf16(const Tensor& x, Tensor y) { adb200::cast_f32_bf16(x.data_ptr<float>(), BF(y), x.numel(), STREAM); }
void increment(Tensor c) { adb200::increment(reinterpret_cast<long long*>(c.data_ptr<int64_t>()), STREAM); }

// ---------------------------------------------------------------------------------------------- communication
adb200::SymCtx make_ctx(const Tensor& flag_ptrs, Tensor epochs, Tensor error, int64_t rank, int64_t world, double timeout_s) {
  adb200::SymCtx c;
  c.flags = reinterpret_cast<uint32_t* const*>(flag_ptrs.data_ptr<int64_t>());
  c.epochs = reinterpret_cast<uint32_t*>(epochs.data_ptr<int32_t>());
  c.error = error.data_ptr<int32_t>();
  c.rank = (int)rank;
  c.world = (int)world;
  c.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  TORCH_CHECK(world >= 1 && world <= 8, "1 to 8 ranks supported");
  TORCH_CHECK(epochs.numel() >= adb200::kMaxCommBlocks + 2, "epoch array too small (blocks + 2 words)");
  return c;
}

// buf_ptrs: int64 device tensor with every rank's wire-buffer address; mc_ptr: multicast address or 0.
void allreduce(const Tensor& flag_ptrs, Tensor epochs, Tensor error, int64_t rank, int64_t world, double timeout_s, const Tensor& buf_ptrs,
               int64_t mc_ptr, int64_t wire, int64_t n, const optional<Tensor>& src32, const optional<Tensor>& residual,
               const optional<Tensor>& dst32, double scale, int64_t blocks) {
  adb200::SymCtx c = make_ctx(flag_ptrs, epochs, error, rank, world, timeout_s);
  const int vec = wire == adb200::WIRE_F32 ? 4 : 8;
  TORCH_CHECK(n % vec == 0, "bucket length must be a multiple of ", vec);
  if (blocks <= 0) blocks = adb200::comm_grid(n / vec / world, adb200::kMaxCommBlocks);
  TORCH_CHECK(blocks <= adb200::kMaxCommBlocks, "too many blocks");
  adb200::launch_allreduce(c, reinterpret_cast<void* const*>(buf_ptrs.data_ptr<int64_t>()), reinterpret_cast<void*>(mc_ptr), (int)wire, n,
                           OPT_F(src32), OPT_F(residual), OPT_F(dst32), (float)scale, (int)blocks, STREAM);
}

void reduce_scatter_update(const Tensor& flag_ptrs, Tensor epochs, Tensor error, int64_t rank, int64_t world, double timeout_s,
                           const Tensor& grad_ptrs, const Tensor& p16_ptrs, const optional<Tensor>& p32_ptrs, int64_t mc_grad, int64_t mc_p16,
                           int64_t mc_p32, Tensor master,
                           const optional<Tensor>& s1, const optional<Tensor>& s2, const Tensor& seg_start, const Tensor& seg_len,
                           const Tensor& seg_state, const optional<Tensor>& seg_flags, const Tensor& owned_prefix, int64_t kind, const Tensor& lr, const Tensor& step, double b1,
                           double b2, double eps, double wd, double momentum, double grad_scale, bool decoupled, bool nesterov, double scale,
                           int64_t blocks) {
  adb200::SymCtx c = make_ctx(flag_ptrs, epochs, error, rank, world, timeout_s);
  const int nseg = seg_start.numel();
  TORCH_CHECK(owned_prefix.numel() == nseg + 1, "owned_prefix must have nseg + 1 entries");
  TORCH_CHECK(blocks > 0 && blocks <= adb200::kMaxCommBlocks, "bad block count");
  adb200::launch_reduce_scatter_update(
      c, reinterpret_cast<float* const*>(grad_ptrs.data_ptr<int64_t>()), reinterpret_cast<__nv_bfloat16* const*>(p16_ptrs.data_ptr<int64_t>()),
      p32_ptrs.has_value() ? reinterpret_cast<float* const*>(p32_ptrs->data_ptr<int64_t>()) : nullptr, reinterpret_cast<float*>(mc_grad),
      reinterpret_cast<__nv_bfloat16*>(mc_p16), reinterpret_cast<float*>(mc_p32), master.data_ptr<float>(), OPT_F(s1),
      OPT_F(s2), reinterpret_cast<const long long*>(seg_start.data_ptr<int64_t>()), reinterpret_cast<const long long*>(seg_len.data_ptr<int64_t>()),
      reinterpret_cast<const long long*>(seg_state.data_ptr<int64_t>()),
      seg_flags.has_value() ? reinterpret_cast<const long long*>(seg_flags->data_ptr<int64_t>()) : nullptr,
      reinterpret_cast<const long long*>(owned_prefix.data_ptr<int64_t>()), nseg,
      (int)kind, lr.data_ptr<float>(), reinterpret_cast<const long long*>(step.data_ptr<int64_t>()), (float)b1, (float)b2, (float)eps, (float)wd,
      (float)momentum, (float)grad_scale, decoupled ? 1 : 0, nesterov ? 1 : 0, (float)scale, (int)blocks, STREAM);
}

void sparse_scatter_add(const Tensor& flag_ptrs, Tensor epochs, Tensor error, int64_t rank, int64_t world, double timeout_s,
                        const Tensor& shard_ptrs, const optional<Tensor>& touched_ptrs, const Tensor& ids, const Tensor& vals, int64_t V,
                        double scale, int64_t barriers, int64_t blocks) {
  adb200::SymCtx c = make_ctx(flag_ptrs, epochs, error, rank, world, timeout_s);
  const int H = vals.size(-1);
  TORCH_CHECK(H % 4 == 0, "row width must be a multiple of 4");
  TORCH_CHECK(blocks > 0 && blocks <= adb200::kMaxCommBlocks, "bad block count");
  adb200::launch_sparse_scatter_add(c, reinterpret_cast<float* const*>(shard_ptrs.data_ptr<int64_t>()),
                                    touched_ptrs.has_value() ? reinterpret_cast<uint8_t* const*>(touched_ptrs->data_ptr<int64_t>()) : nullptr,
                                    ids.data_ptr<int64_t>(), vals.data_ptr(),
                                    vals.scalar_type() == at::kBFloat16 ? 1 : 0, ids.numel(), H, V, (float)scale, (int)barriers, (int)blocks, STREAM);
}

void embedding_gather_peers(const Tensor& flag_ptrs, Tensor epochs, Tensor error, int64_t rank, int64_t world, double timeout_s,
                            const Tensor& shard_ptrs, const Tensor& ids, Tensor out, int64_t V, int64_t barriers, int64_t blocks) {
  adb200::SymCtx c = make_ctx(flag_ptrs, epochs, error, rank, world, timeout_s);
  TORCH_CHECK(out.size(-1) % 8 == 0, "row width must be a multiple of 8");
  TORCH_CHECK(blocks > 0 && blocks <= adb200::kMaxCommBlocks, "bad block count");
  adb200::launch_embedding_gather_peers(c, reinterpret_cast<__nv_bfloat16* const*>(shard_ptrs.data_ptr<int64_t>()), ids.data_ptr<int64_t>(),
                                        BF(out), ids.numel(), out.size(-1), V, (int)barriers, (int)blocks, STREAM);
}

void sym_barrier(const Tensor& flag_ptrs, Tensor epochs, Tensor error, int64_t rank, int64_t world, double timeout_s, int64_t blocks) {
  adb200::SymCtx c = make_ctx(flag_ptrs, epochs, error, rank, world, timeout_s);
  TORCH_CHECK(blocks > 0 && blocks <= adb200::kMaxCommBlocks, "block count must be in [1, ", adb200::kMaxCommBlocks, "]");
  adb200::launch_barrier(c, (int)blocks, STREAM);
}

// step (optional int64 device scalar) overrides my_step; staleness < 0 publishes the step without waiting; max_lead (optional int32
// device scalar) keeps the largest lead this rank had when it passed the gate.
void staleness_gate(const Tensor& flag_ptrs, Tensor epochs, Tensor error, int64_t rank, int64_t world, double timeout_s,
                    const Tensor& clock_ptrs, int64_t my_step, int64_t staleness, const optional<Tensor>& step, const optional<Tensor>& max_lead) {
  adb200::SymCtx c = make_ctx(flag_ptrs, epochs, error, rank, world, timeout_s);
  adb200::launch_staleness_gate(c, reinterpret_cast<uint32_t* const*>(clock_ptrs.data_ptr<int64_t>()), (uint32_t)my_step, OPT_LL(step),
                                (int)staleness, max_lead.has_value() ? max_lead->data_ptr<int>() : nullptr, STREAM);
}

// Relaxed parameter server with GPU owners (plain SGD): p32_owner[segment] -= lr * grad_scale * grad[segment], as vector reductions on
// the owners' fp32 copies. Segment tables: int64 device tensors; prefix has nseg + 1 entries; every start / length a multiple of 4.
void relaxed_push_sgd(const Tensor& p32_ptrs, const Tensor& grad, const Tensor& seg_start, const Tensor& seg_len, const Tensor& seg_owner,
                      const Tensor& prefix, const Tensor& lr, double grad_scale, int64_t blocks) {
  const int nseg = seg_start.numel();
  TORCH_CHECK(prefix.numel() == nseg + 1 && seg_owner.numel() == nseg && grad.scalar_type() == at::kFloat, "bad segment tables");
  auto ll = [](const Tensor& t) { return reinterpret_cast<const long long*>(t.data_ptr<int64_t>()); };
  adb200::launch_relaxed_push_sgd(reinterpret_cast<float* const*>(p32_ptrs.data_ptr<int64_t>()), grad.data_ptr<float>(), ll(seg_start), ll(seg_len),
                                  ll(seg_owner), ll(prefix), nseg, lr.data_ptr<float>(), (float)grad_scale, (int)blocks, STREAM);
}
// Refresh this rank's fp32 and bf16 copies of every segment from the segment's owner.
void relaxed_pull(const Tensor& p32_ptrs, Tensor master, Tensor p16, const Tensor& seg_start, const Tensor& seg_len, const Tensor& seg_owner,
                  const Tensor& prefix, int64_t rank, int64_t blocks) {
  const int nseg = seg_start.numel();
  TORCH_CHECK(prefix.numel() == nseg + 1 && seg_owner.numel() == nseg, "bad segment tables");
  auto ll = [](const Tensor& t) { return reinterpret_cast<const long long*>(t.data_ptr<int64_t>()); };
  adb200::launch_relaxed_pull(reinterpret_cast<float* const*>(p32_ptrs.data_ptr<int64_t>()), master.data_ptr<float>(), BF(p16), ll(seg_start),
                              ll(seg_len), ll(seg_owner), ll(prefix), nseg, (int)rank, (int)blocks, STREAM);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm_set_trace", &gemm_set_trace);
  m.def("gemm", &gemm);
  m.def("gemm_softmax", &gemm_softmax);
  m.def("gemm_gathered_b", &gemm_gathered_b);
  m.def("gemm_gathered_bt", &gemm_gathered_bt);
  m.def("ln_fwd", &ln_fwd);
  m.def("ln_bwd", &ln_bwd);
  m.def("ln_bwd_blocks", &adb200::ln_bwd_blocks);
  m.def("ln_bwd_part_floats", &adb200::ln_bwd_part_floats);
  m.def("colsum_parts", &adb200::colsum_parts);
  m.def("embed_sum", &embed_sum);
  m.def("scatter_add_rows", &scatter_add_rows);
  m.def("strided_rowsum", &strided_rowsum);
  m.def("keyed_colsum", &keyed_colsum);
  m.def("gather_rows", &gather_rows);
  m.def("gather_rows_f32", &gather_rows_f32);
  m.def("scatter_add_rows_bf16", &scatter_add_rows_bf16);
  m.def("softmax_fwd", &softmax_fwd);
  m.def("softmax_bwd", &softmax_bwd);
  m.def("xent", &xent);
  m.def("tanh_bwd", &tanh_bwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("add_bf16", &add_bf16);
  m.def("adam_update", &adam_update);
  m.def("sgd_update", &sgd_update);
  m.def("adagrad_update", &adagrad_update);
  m.def("sparse_rows_update", &sparse_rows_update);
  m.def("flagged_rows_update", &flagged_rows_update);
  m.def("cast_f32_bf16", &cast_f32_bf16);
  m.def("bn_fwd", &bn_fwd);
  m.def("bn_bwd", &bn_bwd);
  m.def("maxpool_fwd", &maxpool_fwd);
  m.def("maxpool_bwd", &maxpool_bwd);
  m.def("im2col", &im2col);
  m.def("col2im", &col2im);
  m.def("pad_image8", &pad_image8);
  m.def("relu_bwd", &relu_bwd);
  m.def("relu_bwd_colsum", &relu_bwd_colsum);
  m.def("psgd_batched", &psgd_batched);
  m.def("psgd_p", &psgd_p);
  m.def("psgd_q", &psgd_q);
  m.def("psgd_d", &psgd_d);
  m.def("lstm_cell_fwd", &lstm_cell_fwd);
  m.def("lstm_cell_bwd", &lstm_cell_bwd);
  m.def("sumsq", &sumsq);
  m.def("clip_scale", &clip_scale);
  m.def("increment", &increment);
  m.def("allreduce", &allreduce);
  m.def("reduce_scatter_update", &reduce_scatter_update);
  m.def("sparse_scatter_add", &sparse_scatter_add);
  m.def("embedding_gather_peers", &embedding_gather_peers);
  m.def("sym_barrier", &sym_barrier);
  m.def("staleness_gate", &staleness_gate);
  m.def("relaxed_push_sgd", &relaxed_push_sgd);
  m.def("relaxed_pull", &relaxed_pull);
  m.attr("MAX_COMM_BLOCKS") = adb200::kMaxCommBlocks;
  register_conv(m);
}
