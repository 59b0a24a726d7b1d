// Bandwidth-bound kernels of the transformer / optimizer path, written for sm_100a (HBM3e-bound: 16-byte
// vector accesses, one pass over the data, reductions in registers + warp shuffles, statistics in fp32).
//
//   layernorm (+ residual add + dropout) forward / backward, embedding sum + layernorm, masked softmax (+dropout)
//   forward / backward, log-softmax cross-entropy forward+backward in one pass, row gather / scatter-add,
//   column sums (bias gradients), fused Adam / SGD-momentum / Adagrad updates that also emit the bf16 compute copy.
//
// In the reference all of these are TensorFlow library ops (LayerNormalization, softmax, sparse CE, ResourceApply*:
// examples/benchmark/utils/modeling/layers/transformer.py:133-164, masked_softmax.py:37-56,
// autodist/kernel/common/op_info.py:24-68).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "elementwise.h"
#include "pdl.cuh"

namespace adb200 {
namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Counter-based dropout mask: the same (seed, index) gives the same decision in forward and backward. One 64-bit
// hash decides four neighbouring elements (16 bits each), so a vector of eight costs two hashes.
__device__ __forceinline__ uint64_t mix(uint64_t seed, uint64_t idx) {
  uint64_t x = seed + idx * 0x9E3779B97F4A7C15ull;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}
// Scales (0 or 1 / keep probability) of the eight elements starting at `base` (a multiple of 8).
__device__ __forceinline__ void keep_scale8(uint64_t seed, uint64_t base, uint32_t thresh16, float inv_keep, float* out) {
  const uint64_t h0 = mix(seed, base >> 2), h1 = mix(seed, (base >> 2) + 1);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    out[j] = (((uint32_t)(h0 >> (16 * j)) & 0xFFFFu) >= thresh16) ? inv_keep : 0.0f;
    out[4 + j] = (((uint32_t)(h1 >> (16 * j)) & 0xFFFFu) >= thresh16) ? inv_keep : 0.0f;
  }
}
__device__ __forceinline__ uint64_t step_seed(uint64_t seed, const long long* step) {
  return seed + (step ? (uint64_t)(*step) * 0x100000001B3ull : 0ull);
}

__device__ __forceinline__ void load8(const bf16* p, float* v) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void unpack8(const uint4& u, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void store8(bf16* p, const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------------------------------------ LayerNorm
// One warp per row, H a multiple of 8 and at most 8 * 32 * MAXV. z = dropout(x) + residual is written back (it is
// what the backward pass needs), y = LN(z) * gamma + beta.
constexpr int MAXV = 4;   // 8-element vectors per lane -> H <= 1024

// Sum of `v` over the block (at most 4 warps); every thread gets the result. `red` holds one float per warp.
__device__ __forceinline__ float ln_block_sum(float v, float* red, int lane, int wib, int nw) {
  v = warp_sum(v);
  if (nw == 1) return v;
  __syncthreads();                       // the previous use of `red` has been read
  if (lane == 0) red[wib] = v;
  __syncthreads();
  float s = red[0];
  for (int w = 1; w < nw; ++w) s += red[w];
  return s;
}

// One thread per 8 columns (H / 8 threads, rounded up to whole warps): every access is one 16-byte vector per thread and
// registers stay few. A block walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and requests the next row's vectors before
// it reduces the current one.
__global__ void ln_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, const float* __restrict__ gamma,
                              const float* __restrict__ beta, bf16* __restrict__ z, bf16* __restrict__ y,
                              float* __restrict__ mean, float* __restrict__ rstd, int rows, int H, float eps,
                              float p_drop, uint64_t seed, const long long* step) {
  pdl_sync();
  __shared__ float red[4];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int col = threadIdx.x * 8;
  const bool active = col < H;
  const uint32_t thresh = (uint32_t)(p_drop * 65536.0f);
  const float inv_keep = p_drop > 0.f ? 1.0f / (1.0f - p_drop) : 1.0f;
  const uint64_t sd = step_seed(seed, step);
  float gg[8] = {0, 0, 0, 0, 0, 0, 0, 0}, bb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (active) {
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + col), g1 = *reinterpret_cast<const float4*>(gamma + col + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(beta + col), b1 = *reinterpret_cast<const float4*>(beta + col + 4);
    gg[0] = g0.x; gg[1] = g0.y; gg[2] = g0.z; gg[3] = g0.w; gg[4] = g1.x; gg[5] = g1.y; gg[6] = g1.z; gg[7] = g1.w;
    bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w; bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
  }
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0}, r[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int row = blockIdx.x;
  if (row < rows && active) {
    load8(x + (long long)row * H + col, v);
    if (res) load8(res + (long long)row * H + col, r);
  }
  for (; row < rows; row += gridDim.x) {
    const long long off = (long long)row * H + col;
    float vn[8] = {0, 0, 0, 0, 0, 0, 0, 0}, rn[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int next = row + gridDim.x;
    if (next < rows && active) {
      load8(x + (long long)next * H + col, vn);
      if (res) load8(res + (long long)next * H + col, rn);
    }
    if (active) {
      if (p_drop > 0.f) {
        float ks[8];
        keep_scale8(sd, (uint64_t)off, thresh, inv_keep, ks);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= ks[j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += r[j];
    }
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j];
    const float mu = ln_block_sum(s, red, lane, wib, nw) / H;
    float q = 0.f;
    if (active) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float dd = v[j] - mu; q += dd * dd; }
    }
    const float rs = rsqrtf(ln_block_sum(q, red, lane, wib, nw) / H + eps);
    if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
    if (active) {
      if (z) store8(z + off, v);
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mu) * rs * gg[j] + bb[j];
      store8(y + off, o);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[j] = vn[j]; r[j] = rn[j]; }
  }
}

// dz = rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat)); dx = dz * dropout mask (only written when p_drop > 0).
// `dz_add` (optional) is added to dz before it is stored: the gradient arriving over the residual connection.
// One thread per 8 columns, a block walks rows blockIdx.x, blockIdx.x + gridDim.x, ... with the next row's loads issued
// before the current row's reductions; its per-column sums (dgamma, dbeta and, when asked, the sum of what it writes to
// dx - the bias gradient of the linear layer in front of the residual) stay in registers and are written once per block
// into part[k][slot][H], k = 0 (dgamma), 1 (dbeta), 2 (sum of the output), slot = block % kLnSlots. `part` must be zero on
// entry; the reduction kernel that follows clears what it reads, so the buffer is zero again afterwards.
constexpr int kLnSlots = 16;

__global__ void ln_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ z, const float* __restrict__ mean,
                              const float* __restrict__ rstd, const float* __restrict__ gamma, const bf16* __restrict__ dz_add,
                              bf16* __restrict__ dz, bf16* __restrict__ dx, float* __restrict__ part, int rows, int H, float p_drop,
                              uint64_t seed, const long long* step, int want_out_sum) {
  pdl_sync();
  __shared__ float red[2][4];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int col = threadIdx.x * 8;
  const bool active = col < H;
  const uint32_t thresh = (uint32_t)(p_drop * 65536.0f);
  const float inv_keep = p_drop > 0.f ? 1.0f / (1.0f - p_drop) : 1.0f;
  const uint64_t sd = step_seed(seed, step);
  float gam[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (active) {
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + col), g1 = *reinterpret_cast<const float4*>(gamma + col + 4);
    gam[0] = g0.x; gam[1] = g0.y; gam[2] = g0.z; gam[3] = g0.w; gam[4] = g1.x; gam[5] = g1.y; gam[6] = g1.z; gam[7] = g1.w;
  }
  float ag[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ab[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ax[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float d[8] = {0, 0, 0, 0, 0, 0, 0, 0}, zz[8] = {0, 0, 0, 0, 0, 0, 0, 0}, add[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int row = blockIdx.x;
  float mu = 0.f, rs = 0.f;
  if (row < rows) {
    mu = mean[row]; rs = rstd[row];
    if (active) {
      const long long off = (long long)row * H + col;
      load8(dy + off, d);
      load8(z + off, zz);
      if (dz_add) load8(dz_add + off, add);
    }
  }
  for (; row < rows; row += gridDim.x) {
    const long long off = (long long)row * H + col;
    // the next row's vectors are requested now and consumed in the next iteration
    float dn[8] = {0, 0, 0, 0, 0, 0, 0, 0}, zn[8] = {0, 0, 0, 0, 0, 0, 0, 0}, an[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int next = row + gridDim.x;
    float mun = 0.f, rsn = 0.f;
    if (next < rows) {
      mun = mean[next]; rsn = rstd[next];
      if (active) {
        const long long noff = (long long)next * H + col;
        load8(dy + noff, dn);
        load8(z + noff, zn);
        if (dz_add) load8(dz_add + noff, an);
      }
    }
    float xh[8], g[8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      xh[j] = (zz[j] - mu) * rs;
      ag[j] += d[j] * xh[j];
      ab[j] += d[j];
      g[j] = d[j] * gam[j];
      s1 += g[j];
      s2 += g[j] * xh[j];
    }
    if (!active) { s1 = 0.f; s2 = 0.f; }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (nw > 1) {
      __syncthreads();
      if (lane == 0) { red[0][wib] = s1; red[1][wib] = s2; }
      __syncthreads();
      s1 = red[0][0]; s2 = red[1][0];
      for (int w = 1; w < nw; ++w) { s1 += red[0][w]; s2 += red[1][w]; }
    }
    s1 /= H; s2 /= H;
    if (active) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (g[j] - s1 - xh[j] * s2) + add[j];
      store8(dz + off, o);
      if (p_drop > 0.f && dx) {
        float ks[8];
        keep_scale8(sd, (uint64_t)off, thresh, inv_keep, ks);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= ks[j];
        store8(dx + off, o);
      }
      if (want_out_sum) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ax[j] += __bfloat162float(__float2bfloat16(o[j]));     // what the next kernel reads
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { d[j] = dn[j]; zz[j] = zn[j]; add[j] = an[j]; }
    mu = mun; rs = rsn;
  }
  if (active) {
    // The blocks add their sums into kLnSlots shared rows (vector reductions, a few dozen blocks per address) instead of
    // writing one row each: the follow-up kernel then reads 16 rows per output instead of hundreds.
    const long long stride = (long long)kLnSlots * H;
    float* p0 = part + (long long)(blockIdx.x % kLnSlots) * H + col;
    atomicAdd(reinterpret_cast<float4*>(p0), make_float4(ag[0], ag[1], ag[2], ag[3]));
    atomicAdd(reinterpret_cast<float4*>(p0 + 4), make_float4(ag[4], ag[5], ag[6], ag[7]));
    atomicAdd(reinterpret_cast<float4*>(p0 + stride), make_float4(ab[0], ab[1], ab[2], ab[3]));
    atomicAdd(reinterpret_cast<float4*>(p0 + stride + 4), make_float4(ab[4], ab[5], ab[6], ab[7]));
    if (want_out_sum) {
      atomicAdd(reinterpret_cast<float4*>(p0 + 2 * stride), make_float4(ax[0], ax[1], ax[2], ax[3]));
      atomicAdd(reinterpret_cast<float4*>(p0 + 2 * stride + 4), make_float4(ax[4], ax[5], ax[6], ax[7]));
    }
  }
}

// Up to three column sums over partials laid out [k][parts][H] in one launch: blockIdx.y = k, out = outs[k]. The partials are
// cleared as they are read (the producer adds into them again next time).
__global__ void colsum3_f32_kernel(float* __restrict__ part, float* __restrict__ out0, float* __restrict__ out1,
                                   float* __restrict__ out2, int parts, int H, int accumulate) {
  pdl_sync();
  __shared__ float sm[8][33];
  float* src = part + (long long)blockIdx.y * parts * H;
  float* out = blockIdx.y == 0 ? out0 : (blockIdx.y == 1 ? out1 : out2);
  const int c = blockIdx.x * 32 + (threadIdx.x & 31), w = threadIdx.x >> 5;
  float a = 0.f;
  if (c < H)
    for (int r = w; r < parts; r += 8) { a += src[(long long)r * H + c]; src[(long long)r * H + c] = 0.f; }
  sm[w][threadIdx.x & 31] = a;
  __syncthreads();
  if (w == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][threadIdx.x];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// out[c] (+)= sum over `parts` rows of part[r][c]. A block covers 32 columns; its 8 warps split the partial rows.
__global__ void colsum_f32_kernel(const float* __restrict__ part, float* __restrict__ out, int parts, int H, int accumulate) {
  pdl_sync();
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + (threadIdx.x & 31), w = threadIdx.x >> 5;
  float a = 0.f;
  if (c < H)
    for (int r = w; r < parts; r += 8) a += part[(long long)r * H + c];
  sm[w][threadIdx.x & 31] = a;
  __syncthreads();
  if (w == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][threadIdx.x];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// Two reductions in one launch (layernorm's dgamma and dbeta): blockIdx.y picks the pair.
__global__ void colsum2_f32_kernel(const float* __restrict__ part_a, float* __restrict__ out_a, const float* __restrict__ part_b,
                                   float* __restrict__ out_b, int parts, int H, int accumulate) {
  pdl_sync();
  __shared__ float sm[8][33];
  const float* part = blockIdx.y ? part_b : part_a;
  float* out = blockIdx.y ? out_b : out_a;
  const int c = blockIdx.x * 32 + (threadIdx.x & 31), w = threadIdx.x >> 5;
  float a = 0.f;
  if (c < H)
    for (int r = w; r < parts; r += 8) a += part[(long long)r * H + c];
  sm[w][threadIdx.x & 31] = a;
  __syncthreads();
  if (w == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sm[i][threadIdx.x];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// ------------------------------------------------------------------------------------------------ embeddings
// z[row] = word[ids[row]] + pos[row % S] + type[tt[row]]  (bf16 tables), then the layernorm kernel runs on z.
__global__ void embed_sum_kernel(const bf16* __restrict__ word, const bf16* __restrict__ pos, const bf16* __restrict__ type,
                                 const int64_t* __restrict__ ids, const int64_t* __restrict__ tt, bf16* __restrict__ z,
                                 int rows, int S, int H, long long V, long long types, int* __restrict__ error) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  long long w = ids[warp], t = tt ? tt[warp] : 0;
  if ((unsigned long long)w >= (unsigned long long)V || (unsigned long long)t >= (unsigned long long)types) {
    // ids outside the tables read row 0 instead of foreign memory; the step is reported as failed
    if (lane == 0 && error != nullptr) atomicExch(error, 21);
    w = 0; t = 0;
  }
  const int s = warp % S;
  for (int vec = lane; vec < H / 8; vec += 32) {
    float a[8], b[8], c[8];
    load8(word + w * H + vec * 8, a);
    load8(pos + (long long)s * H + vec * 8, b);
    load8(type + t * H + vec * 8, c);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += b[j] + c[j];
    store8(z + (long long)warp * H + vec * 8, a);
  }
}

// dst[idx[r]] += src[r] (fp32 destination, bf16 source rows): dense embedding gradient by vector atomics.
__global__ void scatter_add_rows_kernel(float* __restrict__ dst, const int64_t* __restrict__ idx, const bf16* __restrict__ src,
                                        int rows, int H, float scale) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const long long r = idx[warp];
  for (int vec = lane; vec < H / 8; vec += 32) {
    float a[8];
    load8(src + (long long)warp * H + vec * 8, a);
    float* d = dst + r * H + vec * 8;
    atomicAdd(reinterpret_cast<float4*>(d), make_float4(a[0] * scale, a[1] * scale, a[2] * scale, a[3] * scale));
    atomicAdd(reinterpret_cast<float4*>(d + 4), make_float4(a[4] * scale, a[5] * scale, a[6] * scale, a[7] * scale));
  }
}

// out[k][c] = sum over rows r = k + j*stride (j < count) of x[r][c]: position-embedding gradient (k = position).
__global__ void strided_rowsum_kernel(const bf16* __restrict__ x, float* __restrict__ out, int keys, int stride, int count, int H) {
  pdl_sync();
  const int k = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H || k >= keys) return;
  float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < count; ++j) {
    float v[8];
    load8(x + ((long long)k + (long long)j * stride) * H + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] += v[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) out[(long long)k * H + c + i] = a[i];
}

// part[y][k][c] = sum over row chunk y of the rows with key[row]==k of x[row][c]   (keys small: token-type gradient).
// With key == nullptr every row has key 0: plain column sums (bias gradients). A block covers 64 columns (8 vectors)
// with 32 row lanes per vector; the lanes' sums meet in shared memory.
__global__ void keyed_colsum_kernel(const bf16* __restrict__ x, const int64_t* __restrict__ key, float* __restrict__ part,
                                    int rows, int H, int keys, int rows_per_block) {
  pdl_sync();
  __shared__ float sm[32][65];
  const int vec = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * 64 + vec * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  for (int k = 0; k < keys; ++k) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (c < H)
      for (int r = r0 + rl; r < r1; r += 32) {
        if (key && key[r] != k) continue;
        float v[8];
        load8(x + (long long)r * H + c, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += v[i];
      }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm[rl][vec * 8 + i] = a[i];
    __syncthreads();
    if (threadIdx.x < 64 && blockIdx.x * 64 + threadIdx.x < H) {
      float t = 0.f;
#pragma unroll 8
      for (int i = 0; i < 32; ++i) t += sm[i][threadIdx.x];
      part[((long long)blockIdx.y * keys + k) * H + blockIdx.x * 64 + threadIdx.x] = t;
    }
    __syncthreads();
  }
}

// out[r] = src[idx[r]] (bf16 rows)
__global__ void gather_rows_kernel(const bf16* __restrict__ src, const int64_t* __restrict__ idx, bf16* __restrict__ out, int rows, int H) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const long long r = idx[warp];
  for (int vec = lane; vec < H / 8; vec += 32)
    *reinterpret_cast<uint4*>(out + (long long)warp * H + vec * 8) = *reinterpret_cast<const uint4*>(src + r * H + vec * 8);
}

// Row gather from an fp32 table with the bf16 cast fused (sampled-softmax / embedding lookups of master weights).
__global__ void gather_rows_f32_kernel(const float* __restrict__ src, const int64_t* __restrict__ idx, bf16* __restrict__ out, int rows, int H) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const long long r = idx[warp];
  for (int vec = lane; vec < H / 8; vec += 32) {
    const float4 a = *reinterpret_cast<const float4*>(src + r * H + vec * 8);
    const float4 b = *reinterpret_cast<const float4*>(src + r * H + vec * 8 + 4);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    store8(out + (long long)warp * H + vec * 8, v);
  }
}

// dst[idx[r]] += src[r] for bf16 rows whose indices are unique (MLM positions of one sequence never repeat)
__global__ void scatter_add_rows_bf16_kernel(bf16* __restrict__ dst, const int64_t* __restrict__ idx, const bf16* __restrict__ src, int rows, int H) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const long long r = idx[warp];
  for (int vec = lane; vec < H / 8; vec += 32) {
    float a[8], b[8];
    load8(src + (long long)warp * H + vec * 8, a);
    load8(dst + r * H + vec * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] += a[j];
    store8(dst + r * H + vec * 8, b);
  }
}

// ------------------------------------------------------------------------------------------------ softmax
// Rows of length S (<= 1024, multiple of 8) of a [B, heads, S, S] tensor; one warp per row. p = softmax(scale*x + mask[b]);
// writes p (needed by the backward pass) and, when dropout is on, p_drop = dropout(p) for the P.V product.
template <int TPR> __device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <int TPR> __device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// TPR threads per row, VPT 8-element vectors per thread: S = 8 * TPR * VPT. (S = 128 -> 16 threads, two rows per warp.)
template <int TPR, int VPT>
__global__ void softmax_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ mask, bf16* __restrict__ p,
                                   bf16* __restrict__ p_drop, long long rows, int S, int rows_per_batch, float scale,
                                   float pd, uint64_t seed, const long long* step) {
  pdl_sync();
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gt / TPR;
  const int t = (int)(gt % TPR);
  const bool live = row < rows;
  const long long rr = live ? row : rows - 1;
  const int b = (int)(rr / rows_per_batch);
  float v[VPT][8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (t + TPR * i) * 8;
    load8(x + rr * S + col, v[i]);
    float mk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (mask) {
      const float4 m0 = *reinterpret_cast<const float4*>(mask + (long long)b * S + col);
      const float4 m1 = *reinterpret_cast<const float4*>(mask + (long long)b * S + col + 4);
      mk[0] = m0.x; mk[1] = m0.y; mk[2] = m0.z; mk[3] = m0.w; mk[4] = m1.x; mk[5] = m1.y; mk[6] = m1.z; mk[7] = m1.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[i][j] = v[i][j] * scale + mk[j]; mx = fmaxf(mx, v[i][j]); }
  }
  mx = group_max<TPR>(mx);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[i][j] = __expf(v[i][j] - mx); s += v[i][j]; }
  const float inv = 1.0f / group_sum<TPR>(s);
  if (!live) return;
  const uint32_t thresh = (uint32_t)(pd * 65536.0f);
  const float inv_keep = pd > 0.f ? 1.0f / (1.0f - pd) : 1.0f;
  const uint64_t sd = step_seed(seed, step);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const long long off = row * S + (t + TPR * i) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[i][j] *= inv;
    store8(p + off, v[i]);
    if (pd > 0.f && p_drop) {
      float ks[8];
      keep_scale8(sd, (uint64_t)off, thresh, inv_keep, ks);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] *= ks[j];
      store8(p_drop + off, v[i]);
    }
  }
}

// ds = scale * p * (dp' - sum(dp' * p)) with dp' = dp * dropout mask; written over dp.
template <int TPR, int VPT>
__global__ void softmax_bwd_kernel(bf16* __restrict__ dp, const bf16* __restrict__ p, long long rows, int S, float scale,
                                   float pd, uint64_t seed, const long long* step) {
  pdl_sync();
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gt / TPR;
  const int t = (int)(gt % TPR);
  const bool live = row < rows;
  const long long rr = live ? row : rows - 1;
  const uint32_t thresh = (uint32_t)(pd * 65536.0f);
  const float inv_keep = pd > 0.f ? 1.0f / (1.0f - pd) : 1.0f;
  const uint64_t sd = step_seed(seed, step);
  float d[VPT][8], pr[VPT][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const long long off = rr * S + (t + TPR * i) * 8;
    load8(dp + off, d[i]);
    load8(p + off, pr[i]);
    if (pd > 0.f) {
      float ks[8];
      keep_scale8(sd, (uint64_t)off, thresh, inv_keep, ks);
#pragma unroll
      for (int j = 0; j < 8; ++j) d[i][j] *= ks[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += d[i][j] * pr[i][j];
  }
  s = group_sum<TPR>(s);
  if (!live) return;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) d[i][j] = scale * pr[i][j] * (d[i][j] - s);
    store8(dp + row * S + (t + TPR * i) * 8, d[i]);
  }
}

// ------------------------------------------------------------------------------------------------ cross-entropy
// One block per row of logits [rows, ld] (first V columns valid). loss_sum += w * (lse - x[label]); the logits are
// overwritten by d loss / d logits = w / denom * (softmax - onehot) (zero in the padding columns). denom is read
// from device memory (sum of weights, computed by weight_sum_kernel) so that the whole step stays on the device.
__global__ void weight_sum_kernel(const float* __restrict__ w, int n, float* __restrict__ out, float eps) {
  pdl_sync();
  float a = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) a += w[i];
  a = warp_sum(a);
  __shared__ float s[32];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += s[i];
    *out = t + eps;
  }
}

__global__ void xent_kernel(bf16* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ weights,
                            const float* __restrict__ denom, float* __restrict__ loss_sum, int V, int ld, float loss_scale) {
  pdl_sync();
  const int row = blockIdx.x;
  bf16* x = logits + (long long)row * ld;
  __shared__ float red[32];
  __shared__ float bc;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, __bfloat162float(x[c]));
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) { float m = red[0]; for (int i = 1; i < (blockDim.x >> 5); ++i) m = fmaxf(m, red[i]); bc = m; }
  __syncthreads();
  mx = bc;
  float s = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) s += __expf(__bfloat162float(x[c]) - mx);
  s = warp_sum(s);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.f; for (int i = 0; i < (blockDim.x >> 5); ++i) t += red[i]; bc = t; }
  __syncthreads();
  const float sum = bc;
  const float w = weights ? weights[row] : 1.0f;
  const float dn = *denom;
  const long long label = labels[row];
  if (threadIdx.x == 0) atomicAdd(loss_sum, loss_scale * w * (logf(sum) + mx - __bfloat162float(x[label])) / dn);
  const float g = loss_scale * w / dn;
  const float inv = 1.0f / sum;
  for (int c = threadIdx.x; c < ld; c += blockDim.x) {
    float v = 0.f;
    if (c < V) v = g * (__expf(__bfloat162float(x[c]) - mx) * inv - (c == label ? 1.0f : 0.0f));
    x[c] = __float2bfloat16(v);
  }
}

// Image with at most 8 channels (any strides) -> bf16 [N, Hp, Wp, 8]: pixels at (pad, pad), zeros in the halo and the spare channels.
template <typename T>
__global__ void pad_image8_kernel(const T* __restrict__ x, long long sn, long long sc, long long sh, long long sw, int C, int H, int W,
                                  bf16* __restrict__ xp, int Hp, int Wp, int pad, long long total) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int wp = (int)(i % Wp), hp = (int)((i / Wp) % Hp);
  const long long n = i / ((long long)Wp * Hp);
  const int h = hp - pad, w = wp - pad;
  float v[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) v[c] = 0.f;
  if (h >= 0 && h < H && w >= 0 && w < W) {
    const T* src = x + n * sn + h * sh + w * sw;
#pragma unroll
    for (int c = 0; c < 8; ++c) if (c < C) v[c] = (float)src[c * sc];
  }
  uint32_t o[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    __nv_bfloat162 hh = __floats2bfloat162_rn(v[2 * c], v[2 * c + 1]);
    o[c] = *reinterpret_cast<uint32_t*>(&hh);
  }
  *reinterpret_cast<uint4*>(xp + i * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void relu_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ y, uint4* __restrict__ dx, long long n8) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  uint4 d = dy[i];
  const uint4 yy = y[i];
  uint32_t* dw = reinterpret_cast<uint32_t*>(&d);
  const uint32_t* yw = reinterpret_cast<const uint32_t*>(&yy);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    // a bf16 is positive when it is neither zero nor has its sign bit set
    const uint32_t lo = yw[k] & 0xFFFFu, hi = yw[k] >> 16;
    const uint32_t keep_lo = (lo != 0u && lo < 0x8000u) ? 0xFFFFu : 0u;
    const uint32_t keep_hi = (hi != 0u && hi < 0x8000u) ? 0xFFFF0000u : 0u;
    dw[k] &= (keep_lo | keep_hi);
  }
  dx[i] = d;
}

__global__ void tanh_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y, bf16* __restrict__ dx, long long n) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { float t = __bfloat162float(y[i]); dx[i] = __float2bfloat16(__bfloat162float(dy[i]) * (1.0f - t * t)); }
}

__global__ void gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ u, bf16* __restrict__ dx, long long n) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = __bfloat162float(u[i]);
  const float k = 0.7978845608028654f;
  const float t = tanhf(k * (x + 0.044715f * x * x * x));
  const float d = 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k * (1.0f + 3.0f * 0.044715f * x * x);
  dx[i] = __float2bfloat16(__bfloat162float(dy[i]) * d);
}

__global__ void add_bf16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ out, long long n8) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float x[8], y[8];
  load8(a + i * 8, x);
  load8(b + i * 8, y);
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] += y[j];
  store8(out + i * 8, x);
}

// ------------------------------------------------------------------------------------------------ optimizers
// Flat multi-tensor updates over [n] fp32 master weights; each also writes the bf16 copy the next forward reads.
// lr and the step counter live in device memory so that a captured CUDA graph follows schedules.
__global__ void adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                            bf16* __restrict__ p16, long long n, const float* __restrict__ lr_ptr, float b1, float b2, float eps,
                            float wd, int decoupled, const long long* __restrict__ step_ptr, float grad_scale) {
  pdl_sync();
  const float lr = *lr_ptr;
  const float t = (float)(*step_ptr);
  const float c1 = 1.0f - powf(b1, t), c2 = 1.0f - powf(b2, t);
  const float inv_c1 = 1.0f / c1, inv_c2 = 1.0f / c2;
  const long long nvec = n / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  // two independent 16-byte groups per iteration keep eight loads in flight per thread
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < nvec; q += 2 * stride) {
    float4 P[2], G[2], M[2], V[2];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const long long i = (q + u * stride) * 4;
      live[u] = (q + u * stride) < nvec;
      if (live[u]) {
        P[u] = *reinterpret_cast<const float4*>(p + i);
        G[u] = __ldcs(reinterpret_cast<const float4*>(g + i));
        M[u] = *reinterpret_cast<const float4*>(m + i);
        V[u] = *reinterpret_cast<const float4*>(v + i);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (!live[u]) continue;
      const long long i = (q + u * stride) * 4;
      float pp[4] = {P[u].x, P[u].y, P[u].z, P[u].w}, gg[4] = {G[u].x, G[u].y, G[u].z, G[u].w};
      float mm[4] = {M[u].x, M[u].y, M[u].z, M[u].w}, vv[4] = {V[u].x, V[u].y, V[u].z, V[u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float gr = gg[j] * grad_scale;
        if (wd != 0.f) { if (decoupled) pp[j] *= 1.0f - lr * wd; else gr += wd * pp[j]; }
        mm[j] = b1 * mm[j] + (1.0f - b1) * gr;
        vv[j] = b2 * vv[j] + (1.0f - b2) * gr * gr;
        pp[j] -= lr * (mm[j] * inv_c1) / (sqrtf(vv[j] * inv_c2) + eps);
      }
      *reinterpret_cast<float4*>(p + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (p16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
        *reinterpret_cast<uint2*>(p16 + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      }
    }
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = nvec * 4 + threadIdx.x;
    float gr = g[i] * grad_scale, pp = p[i];
    if (wd != 0.f) { if (decoupled) pp *= 1.0f - lr * wd; else gr += wd * pp; }
    const float mm = b1 * m[i] + (1.0f - b1) * gr, vv = b2 * v[i] + (1.0f - b2) * gr * gr;
    pp -= lr * (mm * inv_c1) / (sqrtf(vv * inv_c2) + eps);
    p[i] = pp; m[i] = mm; v[i] = vv;
    if (p16) p16[i] = __float2bfloat16(pp);
  }
}

__global__ void sgd_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ mom, bf16* __restrict__ p16,
                           long long n, const float* __restrict__ lr_ptr, float momentum, float dampening, float wd, int nesterov,
                           const long long* __restrict__ step_ptr, float grad_scale) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float lr = *lr_ptr;
  float gr = g[i] * grad_scale + wd * p[i];
  if (momentum != 0.f) {
    const float b = (*step_ptr <= 1) ? gr : momentum * mom[i] + (1.0f - dampening) * gr;
    mom[i] = b;
    gr = nesterov ? gr + momentum * b : b;
  }
  const float np = p[i] - lr * gr;
  p[i] = np;
  if (p16) p16[i] = __float2bfloat16(np);
}

__global__ void adagrad_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ acc, bf16* __restrict__ p16,
                               long long n, const float* __restrict__ lr_ptr, float eps, float wd, float grad_scale) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float gr = g[i] * grad_scale + wd * p[i];
  const float a = acc[i] + gr * gr;
  acc[i] = a;
  const float np = p[i] - *lr_ptr * gr / (sqrtf(a) + eps);
  p[i] = np;
  if (p16) p16[i] = __float2bfloat16(np);
}

// Row-sparse updates: only the rows that received a gradient are touched (rows must be unique, i.e. a coalesced
// gradient). kind 0 = SGD, 1 = lazy Adam (moments of untouched rows do not decay), 2 = Adagrad. One warp per row.
__global__ void sparse_rows_update_kernel(float* __restrict__ p, float* __restrict__ s1, float* __restrict__ s2,
                                          bf16* __restrict__ p16, const int64_t* __restrict__ rows, const float* __restrict__ g,
                                          int n, int H, long long V, int kind, const float* __restrict__ lr_ptr, float b1, float b2,
                                          float eps, const long long* __restrict__ step_ptr, float grad_scale) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n) return;
  const long long r = rows[warp];
  if (r < 0 || r >= V) return;                       // out-of-range ids are ignored, never written
  const float lr = *lr_ptr;
  float inv_c1 = 1.f, inv_c2 = 1.f;
  if (kind == 1) {
    const float t = (float)(*step_ptr);
    inv_c1 = 1.0f / (1.0f - powf(b1, t));
    inv_c2 = 1.0f / (1.0f - powf(b2, t));
  }
  for (int c = lane; c < H; c += 32) {
    const long long i = r * H + c;
    const float gr = g[(long long)warp * H + c] * grad_scale;
    float np;
    if (kind == 0) {
      np = p[i] - lr * gr;
    } else if (kind == 1) {
      const float m = b1 * s1[i] + (1.0f - b1) * gr, v = b2 * s2[i] + (1.0f - b2) * gr * gr;
      s1[i] = m;
      s2[i] = v;
      np = p[i] - lr * (m * inv_c1) / (sqrtf(v * inv_c2) + eps);
    } else {
      const float a = s1[i] + gr * gr;
      s1[i] = a;
      np = p[i] - lr * gr / (sqrtf(a) + eps);
    }
    p[i] = np;
    if (p16) p16[i] = __float2bfloat16(np);
  }
}

// Owner-side update of a row-sharded table: only rows whose flag was raised by the scatter-add of this step are touched.
// Their gradient row (already the mean over replicas) is applied, written back as bf16, cleared, and the flag is lowered, so
// that update and clearing cost what the touched rows cost, not what the shard costs. kind as in sparse_rows_update_kernel.
__global__ void flagged_rows_update_kernel(float* __restrict__ p, float* __restrict__ s1, float* __restrict__ s2, bf16* __restrict__ p16,
                                           float* __restrict__ g, uint8_t* __restrict__ flags, long long rows, int H, int kind,
                                           const float* __restrict__ lr_ptr, float b1, float b2, float eps,
                                           const long long* __restrict__ step_ptr) {
  pdl_sync();
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const float lr = *lr_ptr;
  float inv_c1 = 1.f, inv_c2 = 1.f;
  if (kind == 1) {
    const float t = (float)(*step_ptr);
    inv_c1 = 1.0f / (1.0f - powf(b1, t));
    inv_c2 = 1.0f / (1.0f - powf(b2, t));
  }
  for (long long r = warp0; r < rows; r += nwarp) {
    if (flags[r] == 0) continue;
    for (int c = lane; c < H; c += 32) {
      const long long i = r * H + c;
      const float gr = g[i];
      g[i] = 0.f;
      float np;
      if (kind == 0) {
        np = p[i] - lr * gr;
      } else if (kind == 1) {
        const float m = b1 * s1[i] + (1.0f - b1) * gr, v = b2 * s2[i] + (1.0f - b2) * gr * gr;
        s1[i] = m;
        s2[i] = v;
        np = p[i] - lr * (m * inv_c1) / (sqrtf(v * inv_c2) + eps);
      } else {
        const float a = s1[i] + gr * gr;
        s1[i] = a;
        np = p[i] - lr * gr / (sqrtf(a) + eps);
      }
      p[i] = np;
      if (p16) p16[i] = __float2bfloat16(np);
    }
    __syncwarp();
    if (lane == 0) flags[r] = 0;
  }
}

// ------------------------------------------------------------------------------------------------ LSTM cell (K17)
// gates [B, 4S] in the order i, j, f, o (fp32); c = sigmoid(f + fb) * c_prev + sigmoid(i) * tanh(j); h = sigmoid(o) * tanh(c)
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

__global__ void lstm_cell_fwd_kernel(const float* __restrict__ gates, const float* __restrict__ c_prev, float* __restrict__ c,
                                     bf16* __restrict__ h, int B, int S, float forget_bias) {
  pdl_sync();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * S) return;
  const int b = (int)(idx / S), s = (int)(idx % S);
  const float* g = gates + (long long)b * 4 * S;
  const float i = g[s], j = g[S + s], f = g[2 * S + s], o = g[3 * S + s];
  const float cn = sigmoidf_(f + forget_bias) * c_prev[idx] + sigmoidf_(i) * tanhf(j);
  c[idx] = cn;
  h[idx] = __float2bfloat16(sigmoidf_(o) * tanhf(cn));
}

__global__ void lstm_cell_bwd_kernel(const float* __restrict__ gates, const float* __restrict__ c_prev, const float* __restrict__ c,
                                     const float* __restrict__ dh, const float* __restrict__ dc_next, float* __restrict__ dgates,
                                     float* __restrict__ dc_prev, int B, int S, float forget_bias) {
  pdl_sync();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * S) return;
  const int b = (int)(idx / S), s = (int)(idx % S);
  const float* g = gates + (long long)b * 4 * S;
  float* dg = dgates + (long long)b * 4 * S;
  const float si = sigmoidf_(g[s]), tj = tanhf(g[S + s]), sf = sigmoidf_(g[2 * S + s] + forget_bias), so = sigmoidf_(g[3 * S + s]);
  const float tc = tanhf(c[idx]);
  const float d_h = dh[idx];
  const float dct = (dc_next ? dc_next[idx] : 0.f) + d_h * so * (1.0f - tc * tc);
  dg[s] = dct * tj * si * (1.0f - si);
  dg[S + s] = dct * si * (1.0f - tj * tj);
  dg[2 * S + s] = dct * c_prev[idx] * sf * (1.0f - sf);
  dg[3 * S + s] = d_h * tc * so * (1.0f - so);
  dc_prev[idx] = dct * sf;
}

// ------------------------------------------------------------------------------------------------ global-norm clip (K19)
// acc += weight * sum(x^2); later x *= min(1, max_norm / (sqrt(acc) + 1e-6)). The norm never visits the host.
__global__ void sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ acc, float weight) {
  pdl_sync();
  float a = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) a += x[i] * x[i];
  a = warp_sum(a);
  __shared__ float sm[32];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += sm[i];
    atomicAdd(acc, t * weight);
  }
}
__global__ void clip_scale_kernel(float* __restrict__ x, long long n, const float* __restrict__ acc, float max_norm) {
  pdl_sync();
  const float norm = sqrtf(*acc);
  if (norm <= max_norm) return;
  const float sc = max_norm / (norm + 1e-6f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= sc;
}

// ------------------------------------------------------------------------------------------------ convolution as GEMM (K10)
// Channels-last activations x [N, H, W, C] (C a multiple of 8). im2col lays the receptive fields out as the rows of the
// GEMM operand cols [N*Ho*Wo, KH*KW*C] (tap-major, channel-minor, matching a weight reshaped to [Cout, KH, KW, C]);
// col2im is its adjoint in gather form: every input pixel sums the taps that read it, so no atomics are needed.
__global__ void im2col_kernel(const bf16* __restrict__ x, bf16* __restrict__ cols, int N, int H, int W, int C, int KH, int KW,
                              int stride, int pad, int Ho, int Wo) {
  pdl_sync();
  const int c8 = C / 8;
  const long long total = (long long)N * Ho * Wo * KH * KW * c8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int cv = (int)(idx % c8);
  long long r = idx / c8;
  const int tap = (int)(r % (KH * KW));
  r /= (KH * KW);
  const int wo = (int)(r % Wo), ho = (int)((r / Wo) % Ho), n = (int)(r / ((long long)Wo * Ho));
  const int hi = ho * stride - pad + tap / KW, wi = wo * stride - pad + tap % KW;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (hi >= 0 && hi < H && wi >= 0 && wi < W)
    v = *reinterpret_cast<const uint4*>(x + (((long long)n * H + hi) * W + wi) * C + cv * 8);
  *reinterpret_cast<uint4*>(cols + idx * 8) = v;
}

__global__ void col2im_kernel(const bf16* __restrict__ dcols, bf16* __restrict__ dx, int N, int H, int W, int C, int KH, int KW,
                              int stride, int pad, int Ho, int Wo) {
  pdl_sync();
  const int c8 = C / 8;
  const long long total = (long long)N * H * W * c8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int cv = (int)(idx % c8);
  long long r = idx / c8;
  const int wi = (int)(r % W), hi = (int)((r / W) % H), n = (int)(r / ((long long)W * H));
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int kh = 0; kh < KH; ++kh) {
    const int hn = hi + pad - kh;
    if (hn < 0 || hn % stride) continue;
    const int ho = hn / stride;
    if (ho >= Ho) continue;
    for (int kw = 0; kw < KW; ++kw) {
      const int wn = wi + pad - kw;
      if (wn < 0 || wn % stride) continue;
      const int wo = wn / stride;
      if (wo >= Wo) continue;
      float v[8];
      load8(dcols + ((((long long)n * Ho + ho) * Wo + wo) * (KH * KW) + kh * KW + kw) * C + cv * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
  store8(dx + idx * 8, acc);
}

// ------------------------------------------------------------------------------------------------ batch-norm (K14), pooling (K15)
// Channels-last activations seen as a matrix [rows = N*H*W, C] (C a multiple of 8).
// Statistics: part[y][0][c] = sum x, part[y][1][c] = sum x^2 over row chunk y (then colsum_f32 over the chunks).
// Each thread keeps four independent 16-byte loads in flight.
__global__ void bn_stats_kernel(const bf16* __restrict__ x, float* __restrict__ part, int rows, int C, int rows_per_block) {
  pdl_sync();
  __shared__ float s1[32][65], s2[32][65];
  const int vec = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * 64 + vec * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < C)
    for (int r = r0 + rl; r < r1; r += 128) {
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + 32 * u;
        if (rr < r1) {
          load8(x + (long long)rr * C + c, v[u]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) { a[i] += v[u][i]; b[i] += v[u][i] * v[u][i]; }
    }
#pragma unroll
  for (int i = 0; i < 8; ++i) { s1[rl][vec * 8 + i] = a[i]; s2[rl][vec * 8 + i] = b[i]; }
  __syncthreads();
  if (threadIdx.x < 64 && blockIdx.x * 64 + threadIdx.x < C) {
    float t1 = 0.f, t2 = 0.f;
    for (int i = 0; i < 32; ++i) { t1 += s1[i][threadIdx.x]; t2 += s2[i][threadIdx.x]; }
    part[((long long)blockIdx.y * 2 + 0) * C + blockIdx.x * 64 + threadIdx.x] = t1;
    part[((long long)blockIdx.y * 2 + 1) * C + blockIdx.x * 64 + threadIdx.x] = t2;
  }
}

// Bias gradient of a convolution (+ ReLU backward): dx = dy masked by y > 0 (when y is given), part[chunk][c] = sum of dx over
// the chunk's rows. Channels-last matrix [rows, C]; 64 channels per block column, four 16-byte loads in flight per thread.
__global__ void relu_bwd_colsum_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y, bf16* __restrict__ dx, float* __restrict__ part,
                                       int rows, int C, int rows_per_block) {
  pdl_sync();
  __shared__ float s1[32][65];
  const int vec = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * 64 + vec * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < C)
    for (int r = r0 + rl; r < r1; r += 128) {
      float v[4][8], m[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + 32 * u;
        if (rr < r1) {
          load8(dy + (long long)rr * C + c, v[u]);
          if (y != nullptr) load8(y + (long long)rr * C + c, m[u]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) { v[u][i] = 0.f; m[u][i] = 1.f; }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + 32 * u;
        if (y != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[u][i] = m[u][i] > 0.f ? v[u][i] : 0.f;
          if (rr < r1) store8(dx + (long long)rr * C + c, v[u]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += v[u][i];
      }
    }
#pragma unroll
  for (int i = 0; i < 8; ++i) s1[rl][vec * 8 + i] = a[i];
  __syncthreads();
  if (threadIdx.x < 64 && blockIdx.x * 64 + threadIdx.x < C) {
    float t1 = 0.f;
    for (int i = 0; i < 32; ++i) t1 += s1[i][threadIdx.x];
    part[(long long)blockIdx.y * C + blockIdx.x * 64 + threadIdx.x] = t1;
  }
}

// y = relu?(x * scale + shift (+ res)) with scale / shift derived from the per-channel sums (sum x, sum x^2): every block
// first builds the table for all C channels in shared memory (C rsqrt per block instead of one per element), block 0 also
// records mean / rstd and folds the batch statistics into the running ones - one launch for the whole normalisation.
// Dynamic shared memory: 2 * C floats.
__global__ void __launch_bounds__(256, 6) bn_apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, bf16* __restrict__ y, long long total8, int C,
                                int relu, const float* __restrict__ sums, const float* __restrict__ gamma, const float* __restrict__ beta,
                                float inv_rows, float eps, float* __restrict__ mean, float* __restrict__ rstd, float* __restrict__ run_mean,
                                float* __restrict__ run_var, long long* __restrict__ batches, float momentum, float unbias) {
  pdl_sync();
  extern __shared__ float s_coef[];                 // [scale (C), shift (C)]
  // the first elements are requested before the table is built, so that the table's latency hides under them
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  uint4 xq = make_uint4(0, 0, 0, 0), rq = make_uint4(0, 0, 0, 0);
  if (idx < total8) {
    xq = *reinterpret_cast<const uint4*>(x + idx * 8);
    if (res != nullptr) rq = *reinterpret_cast<const uint4*>(res + idx * 8);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && batches != nullptr) *batches += 1;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float mu = sums[c] * inv_rows;
    const float var = fmaxf(sums[C + c] * inv_rows - mu * mu, 0.f);
    const float rs = rsqrtf(var + eps);
    const float sc = gamma[c] * rs;
    s_coef[c] = sc;
    s_coef[C + c] = beta[c] - mu * sc;
    if (blockIdx.x == 0) {
      mean[c] = mu;
      rstd[c] = rs;
      if (run_mean != nullptr) {
        run_mean[c] = (1.0f - momentum) * run_mean[c] + momentum * mu;
        run_var[c] = (1.0f - momentum) * run_var[c] + momentum * var * unbias;
      }
    }
  }
  __syncthreads();
  while (idx < total8) {
    const long long next = idx + stride;
    uint4 xn = make_uint4(0, 0, 0, 0), rn = make_uint4(0, 0, 0, 0);
    if (next < total8) {
      xn = *reinterpret_cast<const uint4*>(x + next * 8);
      if (res != nullptr) rn = *reinterpret_cast<const uint4*>(res + next * 8);
    }
    const int c = (int)(idx % (C / 8)) * 8;
    float v[8], rv[8];
    unpack8(xq, v);
    unpack8(rq, rv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float o = fmaf(v[j], s_coef[c + j], s_coef[C + c + j]) + rv[j];
      v[j] = relu ? fmaxf(o, 0.f) : o;
    }
    store8(y + idx * 8, v);
    idx = next; xq = xn; rq = rn;
  }
}

// Backward statistics and coefficients in one launch. Each block adds its sums over a chunk of rows into one of kBnSlots
// shared rows of partials: part[y % kBnSlots][0][c] += sum dy', part[..][1][c] += sum dy' * xhat, dy' = dy masked by the
// ReLU (y > 0). The last block of a 64-channel group to finish (a ticket counter per group) adds the slots up, clears them
// and its counter, and writes what the second pass needs:
//   dx = gamma * rstd * (dy' - dbeta / M - xhat * dgamma / M) = A * dy' + B * x + K per channel; coef = [A (C), B (C), K (C)]
// together with sums = [dbeta (C), dgamma (C)], which are also added into dbeta_acc / dgamma_acc (the parameters'
// gradient buffers) when those are given. `counters` ([C / 64]) and `part` ([kBnSlots, 2, C]) must be zero on entry and
// are zero again on exit.
constexpr int kBnSlots = 16;
constexpr int kBnCounterFloats = 256;          // ticket counters in front of the slots: one per 64 channels, C <= 16384

__global__ void __launch_bounds__(256, 4) bn_bwd_stats_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ y,
                                    const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ gamma,
                                    unsigned int* __restrict__ counters, float* __restrict__ part, float* __restrict__ sums,
                                    float* __restrict__ coef, float* __restrict__ dgamma_acc, float* __restrict__ dbeta_acc,
                                    int rows, int C, int rows_per_block, int relu, float inv_rows) {
  pdl_sync();
  __shared__ float s1[32][65], s2[32][65];
  __shared__ int s_last;
  const int vec = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * 64 + vec * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  // a = sum dy', b = sum dy' * x; sum dy' * xhat = rstd * (b - mean * a) is formed once per block from the totals
  float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < C) {
    for (int r = r0 + rl; r < r1; r += 64) {
      uint4 dq[2], xq[2], yq[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int rr = r + 32 * u;
        dq[u] = xq[u] = make_uint4(0, 0, 0, 0);
        yq[u] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);      // bf16 ones: keeps the gradient
        if (rr < r1) {
          dq[u] = *reinterpret_cast<const uint4*>(dy + (long long)rr * C + c);
          xq[u] = *reinterpret_cast<const uint4*>(x + (long long)rr * C + c);
          if (relu) yq[u] = *reinterpret_cast<const uint4*>(y + (long long)rr * C + c);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        float d[8], xv[8], yv[8];
        unpack8(dq[u], d);
        unpack8(xq[u], xv);
        unpack8(yq[u], yv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float g = yv[i] <= 0.f ? 0.f : d[i];
          a[i] += g;
          b[i] = fmaf(g, xv[i], b[i]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) { s1[rl][vec * 8 + i] = a[i]; s2[rl][vec * 8 + i] = b[i]; }
  __syncthreads();
  const int cc = blockIdx.x * 64 + threadIdx.x;              // the channel thread < 64 owns from here on
  if (threadIdx.x < 64 && cc < C) {
    float t1 = 0.f, t2 = 0.f;
    for (int i = 0; i < 32; ++i) { t1 += s1[i][threadIdx.x]; t2 += s2[i][threadIdx.x]; }
    t2 = rstd[cc] * (t2 - mean[cc] * t1);
    atomicAdd(&part[((long long)(blockIdx.y % kBnSlots) * 2 + 0) * C + cc], t1);
    atomicAdd(&part[((long long)(blockIdx.y % kBnSlots) * 2 + 1) * C + cc], t2);
    __threadfence();                                         // the sums are visible before the ticket is taken
  }
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&counters[blockIdx.x], 1u) == gridDim.y - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x < 64 && cc < C) {
    const int slots = gridDim.y < kBnSlots ? gridDim.y : kBnSlots;
    float s0 = 0.f, sx = 0.f;
    for (int r = 0; r < slots; ++r) {
      float* p0 = &part[((long long)r * 2 + 0) * C + cc];
      float* p1 = &part[((long long)r * 2 + 1) * C + cc];
      s0 += __ldcg(p0);                                      // written by atomics in L2: read there, not through L1
      sx += __ldcg(p1);
      *p0 = 0.f;
      *p1 = 0.f;
    }
    sums[cc] = s0;
    sums[C + cc] = sx;
    if (dbeta_acc != nullptr) dbeta_acc[cc] += s0;
    if (dgamma_acc != nullptr) dgamma_acc[cc] += sx;
    const float rsd = rstd[cc];
    const float ga = gamma[cc] * rsd;
    const float k0 = s0 * inv_rows, k1 = sx * inv_rows;
    const float bx = -ga * rsd * k1;
    coef[cc] = ga;
    coef[C + cc] = bx;
    coef[2 * C + cc] = -bx * mean[cc] - ga * k0;
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0u;
}

__global__ void bn_bwd_apply_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ y,
                                    const float* __restrict__ coef, bf16* __restrict__ dx, bf16* __restrict__ dres, long long total8, int C,
                                    int relu) {
  pdl_sync();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int c = (int)(idx % (C / 8)) * 8;
  float d[8], xv[8], yv[8];
  load8(dy + idx * 8, d);
  load8(x + idx * 8, xv);
  if (relu) load8(y + idx * 8, yv);
  float ca[8], cb[8], ck[8];                          // per-channel coefficients, six 16-byte loads
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float4 a4 = *reinterpret_cast<const float4*>(coef + c + 4 * h);
    const float4 b4 = *reinterpret_cast<const float4*>(coef + C + c + 4 * h);
    const float4 k4 = *reinterpret_cast<const float4*>(coef + 2 * C + c + 4 * h);
    ca[4 * h] = a4.x; ca[4 * h + 1] = a4.y; ca[4 * h + 2] = a4.z; ca[4 * h + 3] = a4.w;
    cb[4 * h] = b4.x; cb[4 * h + 1] = b4.y; cb[4 * h + 2] = b4.z; cb[4 * h + 3] = b4.w;
    ck[4 * h] = k4.x; ck[4 * h + 1] = k4.y; ck[4 * h + 2] = k4.z; ck[4 * h + 3] = k4.w;
  }
  float gm[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float g = (relu && yv[j] <= 0.f) ? 0.f : d[j];
    gm[j] = g;
    d[j] = fmaf(ca[j], g, fmaf(cb[j], xv[j], ck[j]));
  }
  store8(dx + idx * 8, d);
  if (dres != nullptr) store8(dres + idx * 8, gm);      // gradient of the residual branch: dy masked by the ReLU
}

// Max pooling over [N, H, W, C] windows (k x k, stride, pad). The forward pass records, per output element, which
// window position held the first maximum (kh * k + kw, 255 = empty window); the backward pass routes the gradient
// with that code, so ties (common after a ReLU) go to exactly one input as in the library.
__global__ void maxpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, uint8_t* __restrict__ code, int N, int H, int W,
                                   int C, int k, int stride, int pad, int Ho, int Wo) {
  pdl_sync();
  const int c8 = C / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)N * Ho * Wo * c8) return;
  const int cv = (int)(idx % c8);
  long long r = idx / c8;
  const int wo = (int)(r % Wo), ho = (int)((r / Wo) % Ho), n = (int)(r / ((long long)Wo * Ho));
  float m[8];
  uint32_t pos[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { m[j] = -INFINITY; pos[j] = 255u; }
  for (int kh = 0; kh < k; ++kh)
    for (int kw = 0; kw < k; ++kw) {
      const int hi = ho * stride - pad + kh, wi = wo * stride - pad + kw;
      if (hi < 0 || hi >= H || wi < 0 || wi >= W) continue;
      float v[8];
      load8(x + (((long long)n * H + hi) * W + wi) * C + cv * 8, v);
      const uint32_t t = (uint32_t)(kh * k + kw);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (pos[j] == 255u || v[j] > m[j]) { m[j] = v[j]; pos[j] = t; }
    }
  store8(y + idx * 8, m);
  const uint32_t lo = pos[0] | (pos[1] << 8) | (pos[2] << 16) | (pos[3] << 24);
  const uint32_t hi4 = pos[4] | (pos[5] << 8) | (pos[6] << 16) | (pos[7] << 24);
  *reinterpret_cast<uint2*>(code + idx * 8) = make_uint2(lo, hi4);
}

// KT / ST: window and stride as compile-time constants for the common poolings (3x3 stride 2, 2x2 stride 2), so that the
// divisions and the tap loop cost nothing; 0 = take them from the arguments.
template <int KT, int ST>
__global__ void maxpool_bwd_kernel(const uint8_t* __restrict__ code, const bf16* __restrict__ dy, bf16* __restrict__ dx, int N, int H,
                                   int W, int C, int k_arg, int stride_arg, int pad, int Ho, int Wo) {
  pdl_sync();
  const int k = KT > 0 ? KT : k_arg, stride = ST > 0 ? ST : stride_arg;
  const int c8 = C / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)N * H * W * c8) return;
  const int cv = (int)(idx % c8);
  long long r = idx / c8;
  const int wi = (int)(r % W), hi = (int)((r / W) % H), n = (int)(r / ((long long)W * H));
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int kh = 0; kh < k; ++kh) {
    const int hn = hi + pad - kh;
    if (hn < 0 || hn % stride) continue;
    const int ho = hn / stride;
    if (ho >= Ho) continue;
#pragma unroll
    for (int kw = 0; kw < k; ++kw) {
      const int wn = wi + pad - kw;
      if (wn < 0 || wn % stride) continue;
      const int wo = wn / stride;
      if (wo >= Wo) continue;
      const long long o = ((((long long)n * Ho + ho) * Wo + wo) * C) + cv * 8;
      const uint2 packed = *reinterpret_cast<const uint2*>(code + o);
      const uint32_t t = (uint32_t)(kh * k + kw);
      float dv[8];
      load8(dy + o, dv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t p = ((j < 4 ? packed.x : packed.y) >> (8 * (j & 3))) & 0xffu;
        if (p == t) acc[j] += dv[j];
      }
    }
  }
  store8(dx + idx * 8, acc);
}

// ------------------------------------------------------------------------------------------------ PowerSGD (K8)
// Rank-r (r <= 4) factors of an fp32 matrix M [m, n]; all three kernels are bandwidth-bound passes over M.
//   psgd_p : M += err (in place); P[i, :] = M[i, :] . Q          one warp per row
//   psgd_q : Qn[j, :] = sum_i M[i, j] * P[i, :]                  blocks own 32 columns, their warps split the rows
//   psgd_d : err = M - P Q^T;  M = P Q^T                          elementwise
constexpr int PSGD_MAXR = 4;

__global__ void psgd_p_kernel(float* __restrict__ M, const float* __restrict__ err, const float* __restrict__ Q, float* __restrict__ P,
                              int m, int n, int r) {
  pdl_sync();
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= m) return;
  float acc[PSGD_MAXR] = {0.f, 0.f, 0.f, 0.f};
  for (int j = lane; j < n; j += 32) {
    const long long idx = (long long)row * n + j;
    float v = M[idx];
    if (err) { v += err[idx]; M[idx] = v; }
    for (int k = 0; k < r; ++k) acc[k] += v * Q[(long long)j * r + k];
  }
  for (int k = 0; k < r; ++k) {
    const float t = warp_sum(acc[k]);
    if (lane == 0) P[(long long)row * r + k] = t;
  }
}

__global__ void psgd_q_kernel(const float* __restrict__ M, const float* __restrict__ P, float* __restrict__ Qn, int m, int n, int r) {
  pdl_sync();
  __shared__ float sm[8][32][PSGD_MAXR];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  float acc[PSGD_MAXR] = {0.f, 0.f, 0.f, 0.f};
  if (col < n)
    for (int i = w; i < m; i += 8) {
      const float v = M[(long long)i * n + col];
      for (int k = 0; k < r; ++k) acc[k] += v * P[(long long)i * r + k];
    }
  for (int k = 0; k < PSGD_MAXR; ++k) sm[w][lane][k] = acc[k];
  __syncthreads();
  if (w == 0 && col < n)
    for (int k = 0; k < r; ++k) {
      float t = 0.f;
      for (int i = 0; i < 8; ++i) t += sm[i][lane][k];
      Qn[(long long)col * r + k] = t;
    }
}

__global__ void psgd_d_kernel(float* __restrict__ M, float* __restrict__ err, const float* __restrict__ P, const float* __restrict__ Q,
                              int m, int n, int r) {
  pdl_sync();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)m * n) return;
  const int i = (int)(idx / n), j = (int)(idx % n);
  float a = 0.f;
  for (int k = 0; k < r; ++k) a += P[(long long)i * r + k] * Q[(long long)j * r + k];
  err[idx] = M[idx] - a;
  M[idx] = a;
}

// ---- PowerSGD over all matrices of a step at once ------------------------------------------------------------------------------
// Each gradient matrix i is M_i = grad[off_i : off_i + m_i * n_i] seen as [m_i, n_i]; its factors live at P[p_off_i] ([m_i, r]) and
// Q[q_off_i] ([n_i, r]) in two flat buffers that are all-reduced as one message each. The three passes run once per step for all
// matrices (a table lookup finds the matrix of a row / column block / element) instead of three launches per variable.
struct PsgdTable {
  const long long* off;         // [nmat] start of M_i in the flat gradient / residual buffers
  const int* m;                 // [nmat]
  const int* n;                 // [nmat]
  const long long* p_off;       // [nmat]
  const long long* q_off;       // [nmat]
  const long long* row_prefix;  // [nmat + 1] rows before matrix i
  const long long* blk_prefix;  // [nmat + 1] 32-column blocks before matrix i
  const long long* elem_prefix; // [nmat + 1] elements before matrix i
  int nmat;
};

__device__ __forceinline__ int psgd_find(const long long* prefix, int nmat, long long x) {
  int lo = 0, hi = nmat - 1;                      // last i with prefix[i] <= x
  while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (prefix[mid] <= x) lo = mid; else hi = mid - 1; }
  return lo;
}

// M += err (written back), P = M Q: one warp per matrix row.
__global__ void psgd_p_batched_kernel(float* __restrict__ grad, const float* __restrict__ err, const float* __restrict__ Q,
                                      float* __restrict__ P, PsgdTable t, int r, long long rows) {
  pdl_sync();
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int i = psgd_find(t.row_prefix, t.nmat, row);
  const int n = t.n[i];
  const long long local = row - t.row_prefix[i];
  float* M = grad + t.off[i] + local * n;
  const float* e = err + t.off[i] + local * n;
  const float* q = Q + t.q_off[i];
  float acc[PSGD_MAXR] = {0.f, 0.f, 0.f, 0.f};
  for (int j = lane; j < n; j += 32) {
    const float v = M[j] + e[j];
    M[j] = v;
    for (int k = 0; k < r; ++k) acc[k] += v * q[(long long)j * r + k];
  }
  for (int k = 0; k < r; ++k) {
    const float s = warp_sum(acc[k]);
    if (lane == 0) P[t.p_off[i] + local * r + k] = s;
  }
}

// Modified Gram-Schmidt on the columns of every P_i (one block per matrix), as orthogonalize_ of the Python compressor.
__global__ void psgd_orth_batched_kernel(float* __restrict__ P, PsgdTable t, int r) {
  pdl_sync();
  __shared__ float red[32];
  __shared__ float bcast;
  const int i = blockIdx.x;
  const int m = t.m[i];
  float* p = P + t.p_off[i];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  auto block_sum = [&](float v) {
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (threadIdx.x == 0) { float s = 0.f; for (int x = 0; x < nw; ++x) s += red[x]; bcast = s; }
    __syncthreads();
    return bcast;
  };
  for (int k = 0; k < r; ++k) {
    float a = 0.f;
    for (int row = threadIdx.x; row < m; row += blockDim.x) { const float v = p[(long long)row * r + k]; a += v * v; }
    const float inv = 1.0f / (sqrtf(block_sum(a)) + 1e-8f);
    for (int row = threadIdx.x; row < m; row += blockDim.x) p[(long long)row * r + k] *= inv;
    __syncthreads();
    for (int j = k + 1; j < r; ++j) {
      float d = 0.f;
      for (int row = threadIdx.x; row < m; row += blockDim.x) d += p[(long long)row * r + k] * p[(long long)row * r + j];
      const float dot = block_sum(d);
      for (int row = threadIdx.x; row < m; row += blockDim.x) p[(long long)row * r + j] -= dot * p[(long long)row * r + k];
      __syncthreads();
    }
  }
}

// Q = M^T P: one block (8 warps) per 32 columns of one matrix.
__global__ void psgd_q_batched_kernel(const float* __restrict__ grad, const float* __restrict__ P, float* __restrict__ Q, PsgdTable t, int r) {
  pdl_sync();
  __shared__ float sm[8][32][PSGD_MAXR];
  const int i = psgd_find(t.blk_prefix, t.nmat, blockIdx.x);
  const int m = t.m[i], n = t.n[i];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int col = (int)(blockIdx.x - t.blk_prefix[i]) * 32 + lane;
  const float* M = grad + t.off[i];
  const float* p = P + t.p_off[i];
  float acc[PSGD_MAXR] = {0.f, 0.f, 0.f, 0.f};
  if (col < n)
    for (int row = w; row < m; row += 8) {
      const float v = M[(long long)row * n + col];
      for (int k = 0; k < r; ++k) acc[k] += v * p[(long long)row * r + k];
    }
  for (int k = 0; k < PSGD_MAXR; ++k) sm[w][lane][k] = acc[k];
  __syncthreads();
  if (w == 0 && col < n)
    for (int k = 0; k < r; ++k) {
      float s = 0.f;
      for (int x = 0; x < 8; ++x) s += sm[x][lane][k];
      Q[t.q_off[i] + (long long)col * r + k] = s;
    }
}

// err = M - P Q^T; M = P Q^T: one thread per element of all matrices.
__global__ void psgd_d_batched_kernel(float* __restrict__ grad, float* __restrict__ err, const float* __restrict__ P, const float* __restrict__ Q,
                                      PsgdTable t, int r, long long total) {
  pdl_sync();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int i = psgd_find(t.elem_prefix, t.nmat, idx);
  const long long local = idx - t.elem_prefix[i];
  const int n = t.n[i];
  const long long row = local / n, col = local % n;
  float a = 0.f;
  for (int k = 0; k < r; ++k) a += P[t.p_off[i] + row * r + k] * Q[t.q_off[i] + col * r + k];
  const long long g = t.off[i] + local;
  err[g] = grad[g] - a;
  grad[g] = a;
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, bf16* __restrict__ y, long long n) {
  pdl_sync();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2bfloat16(x[i]);
}

__global__ void increment_kernel(long long* c) {
  pdl_sync(); *c += 1; }

inline int blocks_for(long long n, int per) { return (int)((n + per - 1) / per); }

}  // namespace

// ---------------------------------------------------------------------------------------------- launchers
void ln_fwd(const bf16* x, const bf16* res, const float* gamma, const float* beta, bf16* z, bf16* y, float* mean, float* rstd,
            int rows, int H, float eps, float p_drop, uint64_t seed, const long long* step, cudaStream_t st) {
  if (rows <= 0) return;
  const int threads = ((H / 8 + 31) / 32) * 32;
  launch_pdl(ln_fwd_kernel, dim3(rows < 1184 ? rows : 1184), dim3(threads), 0, st, x, res, gamma, beta, z, y, mean, rstd, rows, H, eps, p_drop, seed, step);
}
// Blocks of the backward kernel: four per SM when there are rows enough, so that a block keeps several rows (its
// per-column partial sums are written once per block).
int ln_bwd_blocks(int rows) { return rows < 592 ? (rows < 1 ? 1 : rows) : 592; }
int ln_bwd_part_floats(int H) { return 3 * kLnSlots * H; }
// part: 3 * 16 * H floats, zero on entry and zero again on return. dsum (optional): column sums of the tensor the kernel hands to the layer in
// front of the residual connection (dx when the dropout copy is written, else dz).
void ln_bwd(const bf16* dy, const bf16* z, const float* mean, const float* rstd, const float* gamma, const bf16* dz_add, bf16* dz,
            bf16* dx, float* part, float* dgamma, float* dbeta, float* dsum, int rows, int H, float p_drop, uint64_t seed,
            const long long* step, int accumulate, cudaStream_t st) {
  const int blocks = ln_bwd_blocks(rows);
  const int threads = ((H / 8 + 31) / 32) * 32;
  launch_pdl(ln_bwd_kernel, dim3(blocks), dim3(threads), 0, st, dy, z, mean, rstd, gamma, dz_add, dz, dx, part, rows, H, p_drop, seed, step, dsum != nullptr);
  launch_pdl(colsum3_f32_kernel, dim3(dim3(blocks_for(H, 32), dsum != nullptr ? 3 : 2)), dim3(256), 0, st, part, dgamma, dbeta, dsum, kLnSlots, H, accumulate);
}
void embed_sum(const bf16* word, const bf16* pos, const bf16* type, const int64_t* ids, const int64_t* tt, bf16* z, int rows, int S,
               int H, long long V, long long types, int* error, cudaStream_t st) {
  launch_pdl(embed_sum_kernel, dim3(blocks_for(rows, 4)), dim3(128), 0, st, word, pos, type, ids, tt, z, rows, S, H, V, types, error);
}
void scatter_add_rows(float* dst, const int64_t* idx, const bf16* src, int rows, int H, float scale, cudaStream_t st) {
  launch_pdl(scatter_add_rows_kernel, dim3(blocks_for(rows, 4)), dim3(128), 0, st, dst, idx, src, rows, H, scale);
}
void strided_rowsum(const bf16* x, float* out, int keys, int stride, int count, int H, cudaStream_t st) {
  dim3 grid(blocks_for(H / 8, 128), keys);
  launch_pdl(strided_rowsum_kernel, dim3(grid), dim3(128), 0, st, x, out, keys, stride, count, H);
}
int colsum_parts(int rows) { return rows >= 2048 ? 16 : (rows >= 256 ? 4 : 1); }
void keyed_colsum(const bf16* x, const int64_t* key, float* part, float* out, int rows, int H, int keys, int accumulate, cudaStream_t st) {
  const int parts = colsum_parts(rows);
  const int rpb = (rows + parts - 1) / parts;
  dim3 grid(blocks_for(H, 64), parts);
  launch_pdl(keyed_colsum_kernel, dim3(grid), dim3(256), 0, st, x, key, part, rows, H, keys, rpb);
  launch_pdl(colsum_f32_kernel, dim3(blocks_for(keys * H, 32)), dim3(256), 0, st, part, out, parts, keys * H, accumulate);
}
void gather_rows(const bf16* src, const int64_t* idx, bf16* out, int rows, int H, cudaStream_t st) {
  launch_pdl(gather_rows_kernel, dim3(blocks_for(rows, 4)), dim3(128), 0, st, src, idx, out, rows, H);
}
void gather_rows_f32(const float* src, const int64_t* idx, bf16* out, int rows, int H, cudaStream_t st) {
  launch_pdl(gather_rows_f32_kernel, dim3(blocks_for(rows, 4)), dim3(128), 0, st, src, idx, out, rows, H);
}
void scatter_add_rows_bf16(bf16* dst, const int64_t* idx, const bf16* src, int rows, int H, cudaStream_t st) {
  launch_pdl(scatter_add_rows_bf16_kernel, dim3(blocks_for(rows, 4)), dim3(128), 0, st, dst, idx, src, rows, H);
}
#define ADB_SOFTMAX_DISPATCH(KERNEL, ...)                                                              \
  do {                                                                                                 \
    const int threads = S / 8;                                                                         \
    if (threads == 8) launch_pdl(KERNEL<8, 1>, dim3(blocks_for(rows * 8, 256)), dim3(256), 0, st, __VA_ARGS__);            \
    else if (threads == 16) launch_pdl(KERNEL<16, 1>, dim3(blocks_for(rows * 16, 256)), dim3(256), 0, st, __VA_ARGS__);    \
    else if (threads == 32) launch_pdl(KERNEL<32, 1>, dim3(blocks_for(rows * 32, 256)), dim3(256), 0, st, __VA_ARGS__);    \
    else if (threads == 64) launch_pdl(KERNEL<32, 2>, dim3(blocks_for(rows * 32, 256)), dim3(256), 0, st, __VA_ARGS__);    \
    else if (threads == 128) launch_pdl(KERNEL<32, 4>, dim3(blocks_for(rows * 32, 256)), dim3(256), 0, st, __VA_ARGS__);   \
  } while (0)
bool softmax_supported(int S) { return S == 64 || S == 128 || S == 256 || S == 512 || S == 1024; }
void softmax_fwd(const bf16* x, const float* mask, bf16* p, bf16* p_drop, long long rows, int S, int rows_per_batch, float scale,
                 float pd, uint64_t seed, const long long* step, cudaStream_t st) {
  ADB_SOFTMAX_DISPATCH(softmax_fwd_kernel, x, mask, p, p_drop, rows, S, rows_per_batch, scale, pd, seed, step);
}
void softmax_bwd(bf16* dp, const bf16* p, long long rows, int S, float scale, float pd, uint64_t seed, const long long* step,
                 cudaStream_t st) {
  ADB_SOFTMAX_DISPATCH(softmax_bwd_kernel, dp, p, rows, S, scale, pd, seed, step);
}
void weight_sum(const float* w, int n, float* out, float eps, cudaStream_t st) { launch_pdl(weight_sum_kernel, dim3(1), dim3(256), 0, st, w, n, out, eps); }
void xent(bf16* logits, const int64_t* labels, const float* weights, const float* denom, float* loss_sum, int rows, int V, int ld,
          float loss_scale, cudaStream_t st) {
  launch_pdl(xent_kernel, dim3(rows), dim3(V >= 4096 ? 1024 : 128), 0, st, logits, labels, weights, denom, loss_sum, V, ld, loss_scale);
}
void gelu_bwd(const bf16* dy, const bf16* u, bf16* dx, long long n, cudaStream_t st) {
  launch_pdl(gelu_bwd_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, st, dy, u, dx, n);
}
void pad_image8(const void* x, int is_fp32, long long sn, long long sc, long long sh, long long sw, int N, int C, int H, int W, bf16* xp,
                int Hp, int Wp, int pad, cudaStream_t st) {
  const long long total = (long long)N * Hp * Wp;
  if (is_fp32) launch_pdl(pad_image8_kernel<float>, dim3(blocks_for(total, 256)), dim3(256), 0, st, reinterpret_cast<const float*>(x), sn, sc, sh, sw, C, H, W, xp, Hp, Wp, pad, total);
  else launch_pdl(pad_image8_kernel<bf16>, dim3(blocks_for(total, 256)), dim3(256), 0, st, reinterpret_cast<const bf16*>(x), sn, sc, sh, sw, C, H, W, xp, Hp, Wp, pad, total);
}
void relu_bwd(const bf16* dy, const bf16* y, bf16* dx, long long n, cudaStream_t st) {
  launch_pdl(relu_bwd_kernel, dim3(blocks_for(n / 8, 256)), dim3(256), 0, st, reinterpret_cast<const uint4*>(dy), reinterpret_cast<const uint4*>(y),
                                                          reinterpret_cast<uint4*>(dx), n / 8);
}
void tanh_bwd(const bf16* dy, const bf16* y, bf16* dx, long long n, cudaStream_t st) {
  launch_pdl(tanh_bwd_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, st, dy, y, dx, n);
}
void add_bf16(const bf16* a, const bf16* b, bf16* out, long long n, cudaStream_t st) {
  launch_pdl(add_bf16_kernel, dim3(blocks_for(n / 8, 256)), dim3(256), 0, st, a, b, out, n / 8);
}
void adam_update(float* p, const float* g, float* m, float* v, bf16* p16, long long n, const float* lr, float b1, float b2,
                 float eps, float wd, int decoupled, const long long* step, float grad_scale, cudaStream_t st) {
  const long long groups = (n / 4 + 1) / 2 + 1;
  const int blocks = (int)((groups + 255) / 256 < 148 * 16 ? (groups + 255) / 256 : 148 * 16);
  launch_pdl(adam_kernel, dim3(blocks < 1 ? 1 : blocks), dim3(256), 0, st, p, g, m, v, p16, n, lr, b1, b2, eps, wd, decoupled, step, grad_scale);
}
void sgd_update(float* p, const float* g, float* mom, bf16* p16, long long n, const float* lr, float momentum, float dampening,
                float wd, int nesterov, const long long* step, float grad_scale, cudaStream_t st) {
  launch_pdl(sgd_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, st, p, g, mom, p16, n, lr, momentum, dampening, wd, nesterov, step, grad_scale);
}
void adagrad_update(float* p, const float* g, float* acc, bf16* p16, long long n, const float* lr, float eps, float wd,
                    float grad_scale, cudaStream_t st) {
  launch_pdl(adagrad_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, st, p, g, acc, p16, n, lr, eps, wd, grad_scale);
}
void sparse_rows_update(float* p, float* s1, float* s2, bf16* p16, const int64_t* rows, const float* g, int n, int H, long long V,
                        int kind, const float* lr, float b1, float b2, float eps, const long long* step, float grad_scale,
                        cudaStream_t st) {
  if (n <= 0) return;
  launch_pdl(sparse_rows_update_kernel, dim3(blocks_for(n, 8)), dim3(256), 0, st, p, s1, s2, p16, rows, g, n, H, V, kind, lr, b1, b2, eps, step, grad_scale);
}
void flagged_rows_update(float* p, float* s1, float* s2, bf16* p16, float* g, uint8_t* flags, long long rows, int H, int kind,
                         const float* lr, float b1, float b2, float eps, const long long* step, cudaStream_t st) {
  if (rows <= 0) return;
  long long blocks = (rows + 7) / 8;
  if (blocks > 148 * 32) blocks = 148 * 32;
  launch_pdl(flagged_rows_update_kernel, dim3((int)blocks), dim3(256), 0, st, p, s1, s2, p16, g, flags, rows, H, kind, lr, b1, b2, eps, step);
}
void lstm_cell_fwd(const float* gates, const float* c_prev, float* c, bf16* h, int B, int S, float fb, cudaStream_t st) {
  launch_pdl(lstm_cell_fwd_kernel, dim3(blocks_for((long long)B * S, 256)), dim3(256), 0, st, gates, c_prev, c, h, B, S, fb);
}
void lstm_cell_bwd(const float* gates, const float* c_prev, const float* c, const float* dh, const float* dc_next, float* dgates,
                   float* dc_prev, int B, int S, float fb, cudaStream_t st) {
  launch_pdl(lstm_cell_bwd_kernel, dim3(blocks_for((long long)B * S, 256)), dim3(256), 0, st, gates, c_prev, c, dh, dc_next, dgates, dc_prev, B, S, fb);
}
void sumsq(const float* x, long long n, float* acc, float weight, cudaStream_t st) {
  const int blocks = (int)(n / 1024 + 1 < 592 ? n / 1024 + 1 : 592);
  launch_pdl(sumsq_kernel, dim3(blocks), dim3(256), 0, st, x, n, acc, weight);
}
void clip_scale(float* x, long long n, const float* acc, float max_norm, cudaStream_t st) {
  const int blocks = (int)(n / 1024 + 1 < 592 ? n / 1024 + 1 : 592);
  launch_pdl(clip_scale_kernel, dim3(blocks), dim3(256), 0, st, x, n, acc, max_norm);
}
// Row chunks per channel block: enough blocks to fill the SMs (~8 per SM) while each chunk keeps >= 128 rows.
int bn_bwd_part_floats(int C) { return kBnCounterFloats + kBnSlots * 2 * C; }
int bn_parts(int rows, int C) {
  const int cb = (C + 63) / 64;
  int parts = (592 + cb - 1) / cb;
  if (parts > rows / 128) parts = rows / 128;
  if (parts > 512) parts = 512;
  return parts < 1 ? 1 : parts;
}
// part: [bn_parts, 2, C]; sums: [2, C]; coef: [2, C] (forward) or [3, C] (backward)
// sums_given: `sums` already holds the per-channel sum and sum of squares (the convolution's epilogue produced them); the
// whole normalisation is then one launch.
void bn_fwd(const bf16* x, const float* gamma, const float* beta, const bf16* res, bf16* y, float* mean, float* rstd, float* part, float* sums,
            float* coef, int rows, int C, float eps, int relu, int sums_given, float* run_mean, float* run_var, long long* batches,
            float momentum, cudaStream_t st) {
  const long long total8 = (long long)rows * (C / 8);
  const float unbias = rows > 1 ? (float)rows / (float)(rows - 1) : 1.0f;
  if (!sums_given) {
    const int parts = bn_parts(rows, C), rpb = (rows + parts - 1) / parts;
    launch_pdl(bn_stats_kernel, dim3(dim3(blocks_for(C, 64), parts)), dim3(256), 0, st, x, part, rows, C, rpb);
    launch_pdl(colsum_f32_kernel, dim3(blocks_for(2 * C, 32)), dim3(256), 0, st, part, sums, parts, 2 * C, 0);
  }
  // a few elements per thread: the per-block table of 2 * C coefficients is amortised over at least 4 x 2048 elements
  long long blocks = (total8 + 256 * 4 - 1) / (256 * 4);
  if (blocks > 148 * 6) blocks = 148 * 6;          // one resident wave (6 blocks of 256 threads per SM)
  launch_pdl(bn_apply_kernel, dim3((int)(blocks < 1 ? 1 : blocks)), dim3(256), 2 * C * sizeof(float), st, x, res, y, total8, C, relu, sums, gamma, beta, 1.0f / rows,
                                                                                      eps, mean, rstd, run_mean, run_var, batches, momentum, unbias);
  (void)coef;
}
void bn_bwd(const bf16* dy, const bf16* x, const bf16* y, const float* mean, const float* rstd, const float* gamma, bf16* dx, bf16* dres,
            float* part, float* sums, float* coef, int rows, int C, int relu, float* dgamma_acc, float* dbeta_acc, cudaStream_t st) {
  const int parts = bn_parts(rows, C), rpb = (rows + parts - 1) / parts;
  launch_pdl(bn_bwd_stats_kernel, dim3(dim3(blocks_for(C, 64), parts)), dim3(256), 0, st, dy, x, y, mean, rstd, gamma, reinterpret_cast<unsigned int*>(part),
                                                                      part + kBnCounterFloats, sums, coef, dgamma_acc, dbeta_acc, rows, C, rpb,
                                                                      relu, 1.0f / rows);
  const long long total8 = (long long)rows * (C / 8);
  launch_pdl(bn_bwd_apply_kernel, dim3(blocks_for(total8, 256)), dim3(256), 0, st, dy, x, y, coef, dx, dres, total8, C, relu);
}
// dx = relu'(y) * dy (skipped when y is null) and out[c] (+)= column sums of dx. part: [bn_parts(rows, C), C] floats.
void relu_bwd_colsum(const bf16* dy, const bf16* y, bf16* dx, float* part, float* out, int rows, int C, int accumulate, cudaStream_t st) {
  const int parts = bn_parts(rows, C), rpb = (rows + parts - 1) / parts;
  launch_pdl(relu_bwd_colsum_kernel, dim3(dim3(blocks_for(C, 64), parts)), dim3(256), 0, st, dy, y, dx, part, rows, C, rpb);
  launch_pdl(colsum_f32_kernel, dim3(blocks_for(C, 32)), dim3(256), 0, st, part, out, parts, C, accumulate);
}
void maxpool_fwd(const bf16* x, bf16* y, uint8_t* code, int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo,
                 cudaStream_t st) {
  launch_pdl(maxpool_fwd_kernel, dim3(blocks_for((long long)N * Ho * Wo * (C / 8), 256)), dim3(256), 0, st, x, y, code, N, H, W, C, k, stride, pad, Ho, Wo);
}
void maxpool_bwd(const uint8_t* code, const bf16* dy, bf16* dx, int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo,
                 cudaStream_t st) {
  const int blocks = blocks_for((long long)N * H * W * (C / 8), 256);
  if (k == 3 && stride == 2) launch_pdl(maxpool_bwd_kernel<3, 2>, dim3(blocks), dim3(256), 0, st, code, dy, dx, N, H, W, C, k, stride, pad, Ho, Wo);
  else if (k == 2 && stride == 2) launch_pdl(maxpool_bwd_kernel<2, 2>, dim3(blocks), dim3(256), 0, st, code, dy, dx, N, H, W, C, k, stride, pad, Ho, Wo);
  else launch_pdl(maxpool_bwd_kernel<0, 0>, dim3(blocks), dim3(256), 0, st, code, dy, dx, N, H, W, C, k, stride, pad, Ho, Wo);
}
void im2col(const bf16* x, bf16* cols, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Ho, int Wo, cudaStream_t st) {
  const long long total = (long long)N * Ho * Wo * KH * KW * (C / 8);
  launch_pdl(im2col_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, st, x, cols, N, H, W, C, KH, KW, stride, pad, Ho, Wo);
}
void col2im(const bf16* dcols, bf16* dx, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Ho, int Wo, cudaStream_t st) {
  const long long total = (long long)N * H * W * (C / 8);
  launch_pdl(col2im_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, st, dcols, dx, N, H, W, C, KH, KW, stride, pad, Ho, Wo);
}
void psgd_p(float* M, const float* err, const float* Q, float* P, int m, int n, int r, cudaStream_t st) {
  launch_pdl(psgd_p_kernel, dim3(blocks_for(m, 4)), dim3(128), 0, st, M, err, Q, P, m, n, r);
}
void psgd_q(const float* M, const float* P, float* Qn, int m, int n, int r, cudaStream_t st) {
  launch_pdl(psgd_q_kernel, dim3(blocks_for(n, 32)), dim3(256), 0, st, M, P, Qn, m, n, r);
}
void psgd_d(float* M, float* err, const float* P, const float* Q, int m, int n, int r, cudaStream_t st) {
  launch_pdl(psgd_d_kernel, dim3(blocks_for((long long)m * n, 256)), dim3(256), 0, st, M, err, P, Q, m, n, r);
}
// tab: int64 [8 arrays] laid out by the caller as device pointers; phase 0 = P pass, 1 = orthogonalise, 2 = Q pass, 3 = decompress.
void psgd_batched(int phase, float* grad, float* err, float* P, float* Q, const long long* off, const int* m, const int* n,
                  const long long* p_off, const long long* q_off, const long long* row_prefix, const long long* blk_prefix,
                  const long long* elem_prefix, int nmat, int r, long long rows, long long blocks, long long elems, cudaStream_t st) {
  if (nmat <= 0) return;
  PsgdTable t{off, m, n, p_off, q_off, row_prefix, blk_prefix, elem_prefix, nmat};
  if (phase == 0) launch_pdl(psgd_p_batched_kernel, dim3(blocks_for(rows, 4)), dim3(128), 0, st, grad, err, Q, P, t, r, rows);
  else if (phase == 1) launch_pdl(psgd_orth_batched_kernel, dim3(nmat), dim3(256), 0, st, P, t, r);
  else if (phase == 2) launch_pdl(psgd_q_batched_kernel, dim3((unsigned)blocks), dim3(256), 0, st, grad, P, Q, t, r);
  else launch_pdl(psgd_d_batched_kernel, dim3(blocks_for(elems, 256)), dim3(256), 0, st, grad, err, P, Q, t, r, elems);
}
void cast_f32_bf16(const float* x, bf16* y, long long n, cudaStream_t st) {
  launch_pdl(cast_f32_bf16_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, st, x, y, n);
}
void increment(long long* c, cudaStream_t st) { launch_pdl(increment_kernel, dim3(1), dim3(1), 0, st, c); }

}  // namespace adb200
