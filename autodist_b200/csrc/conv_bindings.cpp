// Python bindings of the implicit-GEMM convolution: geometry -> patch shape, filter-tap table and tensor maps.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <mutex>

#include "conv_tcgen05.h"

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

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// 4-D bf16 map, 128-byte swizzle, zero fill outside. dims / strides in elements, innermost stride 1.
CUtensorMap map4(const void* base, int64_t d0, int64_t d1, int64_t d2, int64_t d3, int64_t s1, int64_t s2, int64_t s3, int b0, int b1,
                 int b2, int b3, bool* ok = nullptr) {
  TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "tensor base must be 16-byte aligned");
  TORCH_CHECK(d0 > 0 && d1 > 0 && d2 > 0 && d3 > 0, "empty tensor");
  TORCH_CHECK(s1 % 8 == 0 && s2 % 8 == 0 && s3 % 8 == 0 && s1 > 0 && s2 > 0 && s3 > 0, "strides must be positive multiples of 8 elements");
  TORCH_CHECK(b0 == 64 && b1 >= 1 && b1 <= 256 && b2 >= 1 && b2 <= 256 && b3 >= 1 && b3 <= 256, "bad box");
  cuuint64_t dims[4] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2, (cuuint64_t)d3};
  cuuint64_t strides[3] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2, (cuuint64_t)s3 * 2};
  cuuint32_t box[4] = {(cuuint32_t)b0, (cuuint32_t)b1, (cuuint32_t)b2, (cuuint32_t)b3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (ok != nullptr) *ok = r == CUDA_SUCCESS;
  else TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

struct Patch { int tw, th, tn; };

int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Patch of at most `limit` pixels (exactly `limit` when `exact`) that wastes the fewest rows over the grid.
Patch choose_patch(int GW, int GH, int GN, int limit, bool exact, bool wsplit) {
  Patch best{1, 1, 1};
  double best_eff = -1.0;
  long long best_area = 0;
  for (int tw = 1; tw <= limit; ++tw) {
    if (!exact && tw > GW) break;
    if (wsplit && tw > 16) break;
    for (int th = 1; tw * th <= limit; ++th) {
      if (!exact && th > GH) break;
      int tn = limit / (tw * th);
      if (exact) {
        if (tw * th * tn != limit) continue;
      } else {
        tn = std::min(tn, GN);
      }
      if (tn < 1 || tn > 256 || tw > 256 || th > 256) continue;
      if (wsplit && (th * tn) % 8 != 0) continue;
      const double tiles = (double)ceil_div(GW, tw) * ceil_div(GH, th) * ceil_div(GN, tn);
      const double eff = (double)GW * GH * GN / (tiles * limit);
      const long long area = (long long)tw * th;
      if (eff > best_eff + 1e-9 || (eff > best_eff - 1e-9 && (area > best_area || (area == best_area && tw > best.tw)))) {
        best_eff = eff; best_area = area; best = Patch{tw, th, tn};
      }
    }
  }
  TORCH_CHECK(best_eff > 0, "no patch shape fits this convolution");
  return best;
}

int pick_bn(int n) { return n >= 256 ? 256 : (n > 64 ? 128 : 64); }

void check_act(const Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 4 && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), what,
              " must be a contiguous bf16 [N, H, W, C] CUDA tensor");
  TORCH_CHECK(t.size(3) % 8 == 0, what, ": channel count must be a multiple of 8");
}

struct Geometry {
  int N, H, W, Cin, OH, OW, Cout, KH, KW, stride, pad;
  bool pointwise;      // 1x1, stride 1, no padding: pixels flatten into one dimension
};

Geometry geometry(const Tensor& x, const Tensor& w, const Tensor& y, int64_t stride, int64_t pad) {
  Geometry g;
  g.N = x.size(0); g.H = x.size(1); g.W = x.size(2); g.Cin = x.size(3);
  g.Cout = w.size(0); g.KH = w.size(1); g.KW = w.size(2);
  TORCH_CHECK(w.dim() == 4 && w.size(3) == g.Cin && w.is_contiguous() && w.scalar_type() == at::kBFloat16,
              "weight must be contiguous bf16 [Cout, KH, KW, Cin]");
  TORCH_CHECK(stride == 1 || stride == 2, "stride 1 or 2");
  TORCH_CHECK(g.KH * g.KW <= adb200::kMaxConvTaps, "filter too large");
  g.stride = stride; g.pad = pad;
  g.OH = (g.H + 2 * pad - g.KH) / stride + 1;
  g.OW = (g.W + 2 * pad - g.KW) / stride + 1;
  TORCH_CHECK(y.size(0) == g.N && y.size(1) == g.OH && y.size(2) == g.OW && y.size(3) == g.Cout, "output shape mismatch");
  g.pointwise = g.KH == 1 && g.KW == 1 && stride == 1 && pad == 0;
  return g;
}

// Maps of the input as the forward pass reads it: one per parity class for stride 2. Box = (64, bw, bh, bn).
void input_maps(adb200::ConvMaps& maps, const Tensor& x, const Geometry& g, int bw, int bh, int bn) {
  const char* base = reinterpret_cast<const char*>(x.data_ptr());
  const int64_t C = g.Cin, W = g.W, H = g.H;
  if (g.pointwise) {
    maps.act[0] = map4(base, C, (int64_t)g.N * H * W, 1, 1, C, C * g.N * H * W, C * g.N * H * W, 64, bw, bh, bn);
    for (int i = 1; i < 4; ++i) maps.act[i] = maps.act[0];
    return;
  }
  if (g.stride == 1) {
    maps.act[0] = map4(base, C, W, H, g.N, C, W * C, H * W * C, 64, bw, bh, bn);
    for (int i = 1; i < 4; ++i) maps.act[i] = maps.act[0];
    return;
  }
  TORCH_CHECK(H >= 2 && W >= 2, "strided convolution of a 1-pixel image");
  for (int ph = 0; ph < 2; ++ph)
    for (int pw = 0; pw < 2; ++pw)
      maps.act[ph * 2 + pw] = map4(base + ((int64_t)ph * W + pw) * C * 2, C, (W - pw + 1) / 2, (H - ph + 1) / 2, g.N, 2 * C, 2 * W * C,
                                   H * W * C, 64, bw, bh, bn);
}

// Taps as the forward pass (and the weight gradient) sees them: output pixel (oh, ow) reads input (oh*s + r - pad, ..).
int forward_taps(adb200::ConvTap* taps, const Geometry& g) {
  int n = 0;
  for (int r = 0; r < g.KH; ++r)
    for (int s = 0; s < g.KW; ++s) {
      const int a = r - g.pad, b = s - g.pad;
      adb200::ConvTap t;
      t.wtap = (short)(r * g.KW + s);
      if (g.stride == 1) {
        t.dh = (short)a; t.dw = (short)b; t.amap = 0;
      } else {
        const int ph = ((a % 2) + 2) % 2, pw = ((b % 2) + 2) % 2;
        t.dh = (short)((a - ph) / 2); t.dw = (short)((b - pw) / 2); t.amap = (short)(ph * 2 + pw);
      }
      taps[n++] = t;
    }
  return n;
}

void set_grid(adb200::ConvParams& p, int GW, int GH, int GN, Patch pt) {
  p.tw = pt.tw; p.th = pt.th; p.tn = pt.tn;
  p.GW = GW; p.GH = GH; p.GN = GN;
  p.tiles_w = ceil_div(GW, pt.tw); p.tiles_h = ceil_div(GH, pt.th); p.tiles_n = ceil_div(GN, pt.tn);
}

// Tuning aid: when set (int64 CUDA tensor of at least 8 x SM-count words, zeroed by the caller), the next launches record
// clock64 marks per CTA into it.
long long* g_trace = nullptr;
void conv_set_trace(const optional<Tensor>& t) {
  if (t.has_value()) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong && t->is_contiguous() && t->numel() >= 8LL * sm_count(), "int64 [SMs, 8] needed");
    g_trace = reinterpret_cast<long long*>(t->data_ptr<int64_t>());
  } else {
    g_trace = nullptr;
  }
}

void launch(const adb200::ConvMaps& maps, const adb200::ConvParams& p_, int bn) {
  adb200::ConvParams p = p_;
  p.trace = g_trace;
  cudaError_t e = adb200::launch_conv(maps, p, bn, sm_count(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "convolution launch failed: ", cudaGetErrorString(e));
}

// CTAs per output tile of the weight gradient: as many as fit in one wave, each with at least four K blocks.
int split_k(int base_tiles, long long patches) {
  int ks = std::max(1, sm_count() / base_tiles);
  ks = (int)std::min<long long>(ks, std::max<long long>(1, patches / 4));
  return ks;
}

// y = conv(x, w) (+ bias) (ReLU); stats (optional, fp32 [2, Cout], zeroed by the caller) receives per-channel sum / sum of squares of y.
void conv_fprop(const Tensor& x, const Tensor& w, Tensor y, const optional<Tensor>& bias, bool relu, const optional<Tensor>& stats,
                int64_t stride, int64_t pad, Tensor error_flag) {
  const c10::cuda::CUDAGuard guard(x.device());
  check_act(x, "x"); check_act(y, "y");
  const Geometry g = geometry(x, w, y, stride, pad);
  adb200::ConvParams p{};
  adb200::ConvMaps maps{};
  p.mode = adb200::CONV_FPROP;
  const int GW = g.pointwise ? g.N * g.OH * g.OW : g.OW, GH = g.pointwise ? 1 : g.OH, GN = g.pointwise ? 1 : g.N;
  const Patch pt = choose_patch(GW, GH, GN, 128, false, false);
  set_grid(p, GW, GH, GN, pt);
  input_maps(maps, x, g, pt.tw, pt.th, pt.tn);
  const int bn = pick_bn(g.Cout);
  maps.w = map4(w.data_ptr(), g.Cin, g.KH * g.KW, g.Cout, 1, g.Cin, (int64_t)g.Cin * g.KH * g.KW, (int64_t)g.Cin * g.KH * g.KW * g.Cout, 64, 1,
                bn, 1);
  maps.dy = maps.w;
  p.ntaps = forward_taps(p.taps, g);
  p.Nc = g.Cout; p.Kc = g.Cin; p.Mc = 0; p.ksplit = 1;
  p.out = y.data_ptr(); p.ldc = g.Cout;
  p.OH = GH; p.OW = GW; p.os = 1; p.oh0 = 0; p.ow0 = 0;
  p.bias = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->numel() == g.Cout && bias->is_contiguous(), "fp32 bias of Cout entries needed");
    p.bias = bias->data_ptr<float>();
  }
  p.relu = relu ? 1 : 0;
  p.stats = nullptr;
  if (stats.has_value()) {
    TORCH_CHECK(stats->scalar_type() == at::kFloat && stats->numel() == 2 * g.Cout && stats->is_contiguous() && g.Cout <= adb200::kMaxStatChannels,
                "stats must be fp32 [2, Cout] with Cout <= 2048");
    p.stats = stats->data_ptr<float>();
  }
  p.error_flag = error_flag.data_ptr<int>();
  launch(maps, p, bn);
}

// dx = the input gradient of conv(x, w) given dy. Every element of dx is written.
void conv_dgrad(const Tensor& dy, const Tensor& w, Tensor dx, int64_t stride, int64_t pad, Tensor error_flag,
                const c10::optional<Tensor>& addend) {
  const c10::cuda::CUDAGuard guard(dy.device());
  check_act(dy, "dy"); check_act(dx, "dx");
  if (addend.has_value()) {
    check_act(*addend, "addend");
    TORCH_CHECK(addend->sizes() == dx.sizes() && addend->data_ptr() != dx.data_ptr(), "addend must have dx's shape and its own storage");
  }
  const Geometry g = geometry(dx, w, dy, stride, pad);
  const int bn = pick_bn(g.Cin);
  adb200::ConvMaps maps{};
  maps.w = map4(w.data_ptr(), g.Cin, g.KH * g.KW, g.Cout, 1, g.Cin, (int64_t)g.Cin * g.KH * g.KW, (int64_t)g.Cin * g.KH * g.KW * g.Cout, 64, 1,
                64, 1);
  maps.dy = maps.w;
  const char* base = reinterpret_cast<const char*>(dy.data_ptr());
  const int64_t C = g.Cout;
  const int classes = g.stride;      // parity classes per dimension
  auto class_taps = [&](int ph, int pw, adb200::ConvTap* taps) {
    int n = 0;
    for (int r = 0; r < g.KH; ++r)
      for (int s = 0; s < g.KW; ++s) {
        const int a = ph + g.pad - r, b = pw + g.pad - s;
        if (g.stride == 2 && ((a & 1) || (b & 1))) continue;
        adb200::ConvTap t;
        t.dh = (short)(a / g.stride); t.dw = (short)(b / g.stride);
        t.wtap = (short)(r * g.KW + s); t.amap = 0;
        if (taps != nullptr) taps[n] = t;
        ++n;
      }
    return n;
  };
  // positions of dx that no output pixel reads (e.g. the odd pixels of a 1x1 stride-2 convolution) get no launch: clear first
  bool uncovered = false;
  for (int ph = 0; ph < classes; ++ph)
    for (int pw = 0; pw < classes; ++pw) uncovered |= class_taps(ph, pw, nullptr) == 0;
  if (uncovered) {
    if (addend.has_value()) dx.copy_(*addend); else dx.zero_();
  }
  for (int ph = 0; ph < classes; ++ph)
    for (int pw = 0; pw < classes; ++pw) {
      adb200::ConvParams p{};
      p.mode = adb200::CONV_DGRAD;
      const int n = class_taps(ph, pw, p.taps);
      const int GH = (g.H - ph + classes - 1) / classes, GW = (g.W - pw + classes - 1) / classes;
      if (GH <= 0 || GW <= 0 || n == 0) continue;
      p.ntaps = n;
      Patch pt;
      if (g.pointwise) {
        const int G = g.N * g.H * g.W;
        pt = choose_patch(G, 1, 1, 128, false, false);
        set_grid(p, G, 1, 1, pt);
        maps.act[0] = map4(base, C, G, 1, 1, C, C * G, C * G, 64, pt.tw, pt.th, pt.tn);
        p.OH = 1; p.OW = G;
      } else {
        pt = choose_patch(GW, GH, g.N, 128, false, false);
        set_grid(p, GW, GH, g.N, pt);
        maps.act[0] = map4(base, C, g.OW, g.OH, g.N, C, (int64_t)g.OW * C, (int64_t)g.OH * g.OW * C, 64, pt.tw, pt.th, pt.tn);
        p.OH = g.H; p.OW = g.W;
      }
      for (int i = 1; i < 4; ++i) maps.act[i] = maps.act[0];
      p.Nc = g.Cin; p.Kc = g.Cout; p.Mc = 0; p.ksplit = 1;
      p.out = dx.data_ptr(); p.ldc = g.Cin;
      p.addend = addend.has_value() ? reinterpret_cast<const __nv_bfloat16*>(addend->data_ptr()) : nullptr;
      p.os = classes; p.oh0 = ph; p.ow0 = pw;
      p.error_flag = error_flag.data_ptr<int>();
      launch(maps, p, bn);
    }
}

// dw (fp32 [Cout, KH, KW, Cin]) = the weight gradient of conv(x, w) given dy: overwritten, or added to with `accumulate`
// (the parameter's gradient buffer, cleared once per step by its owner).
void conv_wgrad(const Tensor& dy, const Tensor& x, Tensor dw, int64_t stride, int64_t pad, Tensor error_flag, bool accumulate) {
  const c10::cuda::CUDAGuard guard(dy.device());
  check_act(dy, "dy"); check_act(x, "x");
  TORCH_CHECK(dw.dim() == 4 && dw.scalar_type() == at::kFloat && dw.is_contiguous(), "dw must be contiguous fp32 [Cout, KH, KW, Cin]");
  Geometry g;
  g.N = x.size(0); g.H = x.size(1); g.W = x.size(2); g.Cin = x.size(3);
  g.Cout = dw.size(0); g.KH = dw.size(1); g.KW = dw.size(2);
  TORCH_CHECK(dw.size(3) == g.Cin && (stride == 1 || stride == 2) && g.KH * g.KW <= adb200::kMaxConvTaps, "bad weight-gradient shape");
  g.stride = stride; g.pad = pad;
  g.OH = (g.H + 2 * pad - g.KH) / stride + 1;
  g.OW = (g.W + 2 * pad - g.KW) / stride + 1;
  TORCH_CHECK(dy.size(0) == g.N && dy.size(1) == g.OH && dy.size(2) == g.OW && dy.size(3) == g.Cout, "dy shape mismatch");
  g.pointwise = g.KH == 1 && g.KW == 1 && stride == 1 && pad == 0;
  adb200::ConvParams p{};
  adb200::ConvMaps maps{};
  p.mode = adb200::CONV_WGRAD;
  const int GW = g.pointwise ? g.N * g.OH * g.OW : g.OW, GH = g.pointwise ? 1 : g.OH, GN = g.pointwise ? 1 : g.N;
  const Patch pt = choose_patch(GW, GH, GN, 64, true, false);
  set_grid(p, GW, GH, GN, pt);
  input_maps(maps, x, g, pt.tw, pt.th, pt.tn);
  const int64_t C = g.Cout;
  if (g.pointwise) maps.dy = map4(dy.data_ptr(), C, GW, 1, 1, C, C * GW, C * GW, 64, pt.tw, pt.th, pt.tn);
  else maps.dy = map4(dy.data_ptr(), C, g.OW, g.OH, g.N, C, (int64_t)g.OW * C, (int64_t)g.OH * g.OW * C, 64, pt.tw, pt.th, pt.tn);
  maps.w = maps.dy;
  p.ntaps = forward_taps(p.taps, g);
  const int bn = pick_bn(g.Cin);
  p.Nc = g.Cin; p.Kc = 0; p.Mc = g.Cout;
  const long long patches = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
  const int base_tiles = ceil_div(g.Cout, 128) * ceil_div(g.Cin, bn) * p.ntaps;
  p.ksplit = split_k(base_tiles, patches);
  p.accumulate = (p.ksplit > 1 || accumulate) ? 1 : 0;
  if (p.accumulate && !accumulate) dw.zero_();
  p.out = dw.data_ptr(); p.ldc = (long long)g.KH * g.KW * g.Cin; p.wtap_stride = g.Cin;
  p.error_flag = error_flag.data_ptr<int>();
  launch(maps, p, bn);
}

// ---- first layer of an image network: 3 (<= 8) input channels ------------------------------------------------------------------
// xp is the image padded to 8 channels with its spatial halo written out: [N, Hp, Wp, 8] bf16, Hp >= (OH-1)*stride + KH,
// Wp*8 >= ((OW-1)*stride)*8 + 64. A filter row (KW taps x 8 channels <= 64 elements) of one output pixel is contiguous in
// memory, so the contraction runs over KH "row taps" of 64 elements each; wr is the weight as [Cout, KH, 64] (zero beyond KW*8).
// Preferred form: one 4-D map whose second dimension steps by one output column (8 or 16 elements) while the box is 64
// elements wide, i.e. neighbouring rows of the map overlap in memory; then a whole patch is one box. Should the driver
// refuse such a map, the caller falls back to one box per patch column (`wsplit`).
bool rowtap_maps(adb200::ConvMaps& maps, const Tensor& xp, int64_t stride, int OW, Patch pt, bool allow_overlap) {
  const int64_t N = xp.size(0), Hp = xp.size(1), Wp = xp.size(2);
  const char* base = reinterpret_cast<const char*>(xp.data_ptr());
  const int64_t row = Wp * 8;
  if (allow_overlap) {
    bool ok = true;
    for (int ph = 0; ph < (int)stride && ok; ++ph)
      maps.act[ph] = map4(base + ph * row * 2, 64, OW, (Hp - ph + stride - 1) / stride, N, stride * 8, stride * row, Hp * row, 64, pt.tw, pt.th,
                          pt.tn, &ok);
    if (ok) {
      for (int i = (int)stride; i < 4; ++i) maps.act[i] = maps.act[0];
      return true;
    }
    return false;
  }
  for (int ph = 0; ph < (int)stride; ++ph)
    maps.act[ph] = map4(base + ph * row * 2, row, (Hp - ph + stride - 1) / stride, N, 1, stride * row, Hp * row, N * Hp * row, 64, pt.th, pt.tn, 1);
  for (int i = (int)stride; i < 4; ++i) maps.act[i] = maps.act[0];
  return true;
}

int rowtap_taps(adb200::ConvTap* taps, int KH, int stride) {
  for (int r = 0; r < KH; ++r) {
    adb200::ConvTap t;
    t.dw = 0; t.wtap = (short)r;
    t.amap = (short)(r % stride); t.dh = (short)(r / stride);
    taps[r] = t;
  }
  return KH;
}

void check_rowtap(const Tensor& xp, int64_t KH, int64_t stride, int OH, int OW) {
  TORCH_CHECK(xp.is_cuda() && xp.dim() == 4 && xp.size(3) == 8 && xp.scalar_type() == at::kBFloat16 && xp.is_contiguous(),
              "xp must be contiguous bf16 [N, Hp, Wp, 8]");
  TORCH_CHECK(stride == 1 || stride == 2, "stride 1 or 2");
  TORCH_CHECK(xp.size(1) >= (OH - 1) * stride + KH && xp.size(2) * 8 >= (int64_t)(OW - 1) * stride * 8 + 64 && xp.size(2) % 2 == 0,
              "padded image too small for this output size");
}

void conv_rowtap_fprop(const Tensor& xp, const Tensor& wr, Tensor y, const optional<Tensor>& bias, bool relu, const optional<Tensor>& stats,
                       int64_t stride, Tensor error_flag) {
  const c10::cuda::CUDAGuard guard(xp.device());
  check_act(y, "y");
  const int N = y.size(0), OH = y.size(1), OW = y.size(2), Cout = y.size(3);
  TORCH_CHECK(wr.dim() == 3 && wr.size(0) == Cout && wr.size(2) == 64 && wr.scalar_type() == at::kBFloat16 && wr.is_contiguous(),
              "wr must be contiguous bf16 [Cout, KH, 64]");
  const int KH = wr.size(1);
  check_rowtap(xp, KH, stride, OH, OW);
  TORCH_CHECK(xp.size(0) == N, "batch mismatch");
  adb200::ConvParams p{};
  adb200::ConvMaps maps{};
  p.mode = adb200::CONV_FPROP;
  Patch pt = choose_patch(OW, OH, N, 128, false, false);
  if (rowtap_maps(maps, xp, stride, OW, pt, true)) {
    p.wsplit = 0;
  } else {
    pt = choose_patch(OW, OH, N, 128, false, true);
    rowtap_maps(maps, xp, stride, OW, pt, false);
    p.wsplit = 1; p.xstep = (int)stride * 8;
  }
  set_grid(p, OW, OH, N, pt);
  const int bn = pick_bn(Cout);
  maps.w = map4(wr.data_ptr(), 64, KH, Cout, 1, 64, 64 * KH, (int64_t)64 * KH * Cout, 64, 1, bn, 1);
  maps.dy = maps.w;
  p.ntaps = rowtap_taps(p.taps, KH, stride);
  p.Nc = Cout; p.Kc = 64; p.ksplit = 1;
  p.out = y.data_ptr(); p.ldc = Cout; p.OH = OH; p.OW = OW; p.os = 1;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->numel() == Cout && bias->is_contiguous(), "fp32 bias of Cout entries needed");
    p.bias = bias->data_ptr<float>();
  }
  p.relu = relu ? 1 : 0;
  if (stats.has_value()) {
    TORCH_CHECK(stats->scalar_type() == at::kFloat && stats->numel() == 2 * Cout && stats->is_contiguous(), "stats must be fp32 [2, Cout]");
    p.stats = stats->data_ptr<float>();
  }
  p.error_flag = error_flag.data_ptr<int>();
  launch(maps, p, bn);
}

void conv_rowtap_wgrad(const Tensor& dy, const Tensor& xp, Tensor dwr, int64_t stride, Tensor error_flag) {
  const c10::cuda::CUDAGuard guard(dy.device());
  check_act(dy, "dy");
  const int N = dy.size(0), OH = dy.size(1), OW = dy.size(2), Cout = dy.size(3);
  TORCH_CHECK(dwr.dim() == 3 && dwr.size(0) == Cout && dwr.size(2) == 64 && dwr.scalar_type() == at::kFloat && dwr.is_contiguous(),
              "dwr must be contiguous fp32 [Cout, KH, 64]");
  const int KH = dwr.size(1);
  check_rowtap(xp, KH, stride, OH, OW);
  adb200::ConvParams p{};
  adb200::ConvMaps maps{};
  p.mode = adb200::CONV_WGRAD;
  Patch pt = choose_patch(OW, OH, N, 64, true, false);
  if (rowtap_maps(maps, xp, stride, OW, pt, true)) {
    p.wsplit = 0;
  } else {
    pt = choose_patch(OW, OH, N, 64, true, true);
    rowtap_maps(maps, xp, stride, OW, pt, false);
    p.wsplit = 1; p.xstep = (int)stride * 8;
  }
  set_grid(p, OW, OH, N, pt);
  const int64_t C = Cout;
  maps.dy = map4(dy.data_ptr(), C, OW, OH, N, C, (int64_t)OW * C, (int64_t)OH * OW * C, 64, p.wsplit ? 1 : pt.tw, pt.th, pt.tn);
  maps.w = maps.dy;
  p.ntaps = rowtap_taps(p.taps, KH, stride);
  p.Nc = 64; p.Mc = Cout;
  const long long patches = (long long)p.tiles_w * p.tiles_h * p.tiles_n;
  p.ksplit = split_k(ceil_div(Cout, 128) * KH, patches);
  p.accumulate = p.ksplit > 1 ? 1 : 0;
  if (p.accumulate) dwr.zero_();
  p.out = dwr.data_ptr(); p.ldc = (long long)KH * 64; p.wtap_stride = 64;
  p.error_flag = error_flag.data_ptr<int>();
  launch(maps, p, 64);
}

}  // namespace

void register_conv(pybind11::module& m) {
  m.def("conv_set_trace", &conv_set_trace);
  m.def("conv_fprop", &conv_fprop);
  namespace py = pybind11;
  m.def("conv_dgrad", &conv_dgrad, py::arg("dy"), py::arg("w"), py::arg("dx"), py::arg("stride"), py::arg("pad"), py::arg("error_flag"),
        py::arg("addend") = py::none());
  m.def("conv_wgrad", &conv_wgrad);
  m.def("conv_rowtap_fprop", &conv_rowtap_fprop);
  m.def("conv_rowtap_wgrad", &conv_rowtap_wgrad);
}
