// Allocation-free column sums (see no_alloc.h for who needs this and the rules of use).
//
// Two kernels, same arithmetic as the column-sum pair in elementwise.cu: the first writes per-row-chunk partial sums
// into scratch, the second adds the partials. The scratch is the file-scope array below instead of a caller tensor.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "no_alloc.h"

namespace {

constexpr int kMaxParts = 16;
constexpr int kMaxDevices = 64;

// Device-resident scratch: partial sums [part][col]. In host code this name is only a handle for the runtime (its
// host-side value is not a device address); the launch code below obtains the real address once per device.
static __device__ __align__(256) float g_scratch[kMaxParts * ADB200_NOALLOC_MAX_COLS];

thread_local char t_error[256] = "";
float* g_scratch_addr[kMaxDevices] = {nullptr};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}

// part[y][c] = sum over rows of chunk y of x[row][c]; a block covers 64 columns with 32 row lanes per 8-column vector.
__global__ void partial_colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ part, int rows, int cols,
                                      int rows_per_block) {
  __shared__ float sm[32][65];
  const int vec = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * 64 + vec * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < cols)
    for (int r = r0 + rl; r < r1; r += 32) {
      float v[8];
      load8(x + (long long)r * cols + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] += v[i];
    }
#pragma unroll
  for (int i = 0; i < 8; ++i) sm[rl][vec * 8 + i] = a[i];
  __syncthreads();
  if (threadIdx.x < 64 && blockIdx.x * 64 + threadIdx.x < cols) {
    float t = 0.f;
#pragma unroll 8
    for (int i = 0; i < 32; ++i) t += sm[i][threadIdx.x];
    part[(long long)blockIdx.y * cols + blockIdx.x * 64 + threadIdx.x] = t;
  }
}

__global__ void final_colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int parts, int cols) {
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + (threadIdx.x & 31), w = threadIdx.x >> 5;
  float a = 0.f;
  if (c < cols)
    for (int r = w; r < parts; r += 8) a += part[(long long)r * cols + c];
  sm[w][threadIdx.x & 31] = a;
  __syncthreads();
  if (w == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][threadIdx.x];
    out[c] = t;
  }
}

int refuse(int code, const char* msg) {
  snprintf(t_error, sizeof(t_error), "%s", msg);
  return code;
}

}  // namespace

extern "C" const char* adb200_noalloc_last_error(void) { return t_error; }

extern "C" int adb200_colsum_bf16_noalloc(const void* x_bf16, float* out, int rows, int cols, cudaStream_t stream) {
  t_error[0] = 0;
  if (rows < 1 || cols < 8 || cols % 8 != 0) return refuse(ADB200_NOALLOC_BAD_SHAPE, "rows must be >= 1 and cols a positive multiple of 8");
  if (cols > ADB200_NOALLOC_MAX_COLS) {
    snprintf(t_error, sizeof(t_error), "cols = %d exceeds the built-in scratch (at most %d columns)", cols, ADB200_NOALLOC_MAX_COLS);
    return ADB200_NOALLOC_TOO_WIDE;
  }
  if (x_bf16 == nullptr || out == nullptr || reinterpret_cast<uintptr_t>(x_bf16) % 16 != 0)
    return refuse(ADB200_NOALLOC_BAD_POINTER, "x and out must be non-null and x 16-byte aligned");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return refuse((int)e, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return refuse(ADB200_NOALLOC_BAD_SHAPE, "device ordinal out of range");
  if (g_scratch_addr[dev] == nullptr) {
    // Set-up, once per device, with that device current: turn the symbol into this device's address.
    float* addr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_scratch);
    if (e != cudaSuccess || addr == nullptr) return refuse((int)e, cudaGetErrorString(e));
    g_scratch_addr[dev] = addr;
  }
  float* scratch = g_scratch_addr[dev];
  const int parts = rows >= 2048 ? kMaxParts : (rows >= 256 ? 4 : 1);
  const int rows_per_block = (rows + parts - 1) / parts;
  dim3 grid((cols + 63) / 64, parts);
  partial_colsum_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x_bf16), scratch, rows, cols, rows_per_block);
  final_colsum_kernel<<<(cols + 31) / 32, 256, 0, stream>>>(scratch, out, parts, cols);
  e = cudaGetLastError();
  if (e != cudaSuccess) return refuse((int)e, cudaGetErrorString(e));
  return 0;
}
