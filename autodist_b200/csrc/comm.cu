// Gradient synchronisation kernels over NVSwitch peer memory (sm_100a, one process per GPU).
//
// Every rank allocates the same symmetric buffers and maps its peers' copies (plain peer pointers, and an NVLS
// multicast address when the fabric offers one). The kernels below read and write those buffers directly, so the
// collective and the arithmetic around it are one launch:
//
//   allreduce_kernel        K1/K6/K7  compress (fp32 -> fp16/bf16 with error-feedback residual) + two-shot mean
//                                     all-reduce (each rank reduces its slice from all peers and writes the result to
//                                     all peers; `multimem.ld_reduce` / `multimem.st` through the switch when a
//                                     multicast address is given) + widening of the result
//   reduce_scatter_update   K2        reduce the owned segments of a gradient bucket from all peers, apply the
//                                     optimizer (Adam / SGD-momentum / Adagrad) to the owner's fp32 state and write
//                                     the new bf16 (and fp32) parameters into every peer's parameter buffer
//   sparse_scatter_add      K4        row-sparse gradients: each row is added into its owner's shard with
//                                     red.global.add over the peer pointer (row -> shard by the uneven-split rule)
//   embedding_gather_peers  K5        partitioned embedding lookup: rows are read from the shard that owns them
//   barrier_kernel          K20       stand-alone bounded barrier / staleness gate
//
// Cross-GPU ordering uses one flag word per (block, peer) written with st.release.sys and polled with
// ld.acquire.sys; flags carry an epoch that the kernel keeps in device memory, so launches can be replayed from a
// CUDA graph. Every wait is bounded by `timeout_ns` (globaltimer): on expiry the kernel stores an error code and
// returns without touching peer memory again.
//
// These replace the reference's TensorFlow collectives and parameter-server accumulators
// (autodist/kernel/synchronization/compressor.py:84-96, ps_synchronizer.py:460-633,
// all_reduce_synchronizer.py:132-173); the reference itself contains no device code.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.h"

namespace adb200 {
namespace {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block-level barrier across ranks. Block b of every rank meets block b of every other rank.
// flags[r] points at rank r's flag array laid out [block][sender]. Returns false on timeout.
__device__ bool sym_barrier(const SymCtx& c) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_epoch = c.epochs[blockIdx.x] + 1;
    c.epochs[blockIdx.x] = s_epoch;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  if (threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(c.flags[peer] + (size_t)blockIdx.x * c.world + c.rank, e);
    const uint32_t* mine = c.flags[c.rank] + (size_t)blockIdx.x * c.world + peer;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    while ((int32_t)(ld_acquire_sys(mine) - e) < 0) {
      if (((++it) & 63u) == 0 && globaltimer_ns() - t0 > c.timeout_ns) {
        s_ok = 0;
        atomicExch(c.error, 100 + peer);
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// Grid-wide barrier among the blocks of this launch on this GPU (arrival count + generation word in device memory).
// The cross-GPU barrier above pairs block b with the peers' block b only; where a phase reads data that *any* block
// of a rank produced (the packed wire buffer, the reduced result), the blocks of that rank meet here first.
// The launcher cuts the grid to the number of blocks the GPU holds at once (occupancy calculator), so all of them are
// resident; the wait is bounded.
__device__ bool grid_barrier(const SymCtx& c) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok = 1;
    uint32_t* count = c.epochs + kMaxCommBlocks;
    volatile uint32_t* gen_p = c.epochs + kMaxCommBlocks + 1;
    __threadfence();
    const uint32_t gen = *gen_p;
    if (atomicAdd(count, 1u) == gridDim.x - 1) {
      atomicExch(count, 0u);
      __threadfence();
      atomicAdd(const_cast<uint32_t*>(gen_p), 1u);
    } else {
      const unsigned long long t0 = globaltimer_ns();
      uint32_t it = 0;
      while (*gen_p == gen) {
        if (((++it) & 63u) == 0 && globaltimer_ns() - t0 > c.timeout_ns) {
          s_ok = 0;
          atomicExch(c.error, 300);
          break;
        }
      }
    }
    __threadfence();
  }
  __syncthreads();
  return s_ok != 0;
}

template <typename T> struct Wire;
template <> struct Wire<float> {
  static constexpr int VEC = 4;
  __device__ static void load(const float* p, float* v) { float4 a = *reinterpret_cast<const float4*>(p); v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; }
  __device__ static void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
  __device__ static float to(float x) { return x; }
  __device__ static float from(float x) { return x; }
  __device__ static void mc_reduce(const float* p, float* v) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "l"(p) : "memory");
  }
  __device__ static void mc_store(float* p, const float* v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
  }
};
template <> struct Wire<__nv_bfloat16> {
  static constexpr int VEC = 8;
  __device__ static void load(const __nv_bfloat16* p, float* v) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__nv_bfloat16* p, const float* v) {
    uint4 u; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  __device__ static __nv_bfloat16 to(float x) { return __float2bfloat16(x); }
  __device__ static float from(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static void mc_reduce(const __nv_bfloat16* p, float* v) {
    uint32_t r[4];
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(p) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&r[i])); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void mc_store(__nv_bfloat16* p, const float* v) {
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]); r[i] = *reinterpret_cast<uint32_t*>(&h); }
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(__uint_as_float(r[0])), "f"(__uint_as_float(r[1])),
                 "f"(__uint_as_float(r[2])), "f"(__uint_as_float(r[3])) : "memory");
  }
};
template <> struct Wire<__half> {
  static constexpr int VEC = 8;
  __device__ static void load(const __half* p, float* v) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__half* p, const float* v) {
    uint4 u; __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  __device__ static __half to(float x) { return __float2half_rn(x); }
  __device__ static float from(__half x) { return __half2float(x); }
  __device__ static void mc_reduce(const __half* p, float* v) {
    uint32_t r[4];
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(p) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(*reinterpret_cast<__half2*>(&r[i])); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void mc_store(__half* p, const float* v) {
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]); r[i] = *reinterpret_cast<uint32_t*>(&h); }
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(__uint_as_float(r[0])), "f"(__uint_as_float(r[1])),
                 "f"(__uint_as_float(r[2])), "f"(__uint_as_float(r[3])) : "memory");
  }
};

// ------------------------------------------------------------------------------------------------ K1 (+K6, K7)
// n must be a multiple of Wire<T>::VEC (the host pads buckets). bufs[r] = rank r's wire buffer (T), mc = multicast
// address of the same buffer or null. src32/residual/dst32 are local fp32 arrays (null to skip a phase):
//   phase A  wire[i] = T(src32[i] + residual[i]); residual[i] = that sum - float(wire[i])
//   phase B  my slice: wire_all_peers[i] = T(scale * sum_r wire_r[i])
//   phase C  dst32[i] = float(wire[i])
template <typename T>
__global__ void __launch_bounds__(512) allreduce_kernel(SymCtx c, T* const* bufs, T* mc, long long n, const float* src32,
                                                        float* residual, float* dst32, float scale) {
  constexpr int VEC = Wire<T>::VEC;
  const long long nvec = n / VEC;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
  T* mine = bufs[c.rank];
  if (src32) {
    for (long long i = tid; i < nvec; i += nthr) {
      float v[VEC], w[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        float t = src32[i * VEC + j] + (residual ? residual[i * VEC + j] : 0.f);
        T q = Wire<T>::to(t);
        w[j] = Wire<T>::from(q);
        v[j] = t;
      }
      if (residual) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) residual[i * VEC + j] = v[j] - w[j];
      }
      Wire<T>::store(mine + i * VEC, w);
    }
    if (!grid_barrier(c)) return;      // every block of this rank has packed before any block tells the peers
  }
  if (!sym_barrier(c)) return;
  const long long chunk = (nvec + c.world - 1) / c.world;
  const long long lo = chunk * c.rank, hi = min(nvec, lo + chunk);
  if (mc) {
    for (long long i = lo + tid; i < hi; i += nthr) {
      float a[VEC];
      Wire<T>::mc_reduce(mc + i * VEC, a);
#pragma unroll
      for (int j = 0; j < VEC; ++j) a[j] *= scale;
      Wire<T>::mc_store(mc + i * VEC, a);
    }
  } else {
    for (long long i = lo + tid; i < hi; i += nthr) {
      float a[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) a[j] = 0.f;
      float v[8][VEC];
#pragma unroll
      for (int r = 0; r < 8; ++r) if (r < c.world) Wire<T>::load(bufs[r] + i * VEC, v[r]);
#pragma unroll
      for (int r = 0; r < 8; ++r) if (r < c.world) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) a[j] += v[r][j];
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) a[j] *= scale;
#pragma unroll
      for (int r = 0; r < 8; ++r) if (r < c.world) Wire<T>::store(bufs[r] + i * VEC, a);
    }
  }
  if (!sym_barrier(c)) return;
  if (dst32) {
    if (!grid_barrier(c)) return;      // every peer block has delivered its slice (all local blocks passed their barrier)
    for (long long i = tid; i < nvec; i += nthr) {
      float w[VEC];
      Wire<T>::load(mine + i * VEC, w);
#pragma unroll
      for (int j = 0; j < VEC; ++j) dst32[i * VEC + j] = w[j];
    }
  }
}

// ------------------------------------------------------------------------------------------------ K2
// Segment table: seg_start[s], seg_len[s] (elements of the flat bucket, both multiples of 4), seg_state[s] = offset of
// the segment inside this rank's compact optimizer state, for the segments this rank owns; owned_prefix[s] = number
// of owned elements before segment s (owned_prefix[nseg] = total). grads[r] = rank r's fp32 gradient bucket,
// p16[r] / p32[r] = rank r's bf16 / fp32 parameter buckets (p32 may be null: fp32 master only at the owner).
struct OptArgs {
  int kind;              // 0 sgd(momentum), 1 adam, 2 adagrad
  const float* lr;       // device scalar
  const long long* step; // device scalar (already incremented for this step)
  float b1, b2, eps, wd, momentum, grad_scale;
  int decoupled, nesterov;
};

// mc_grad / mc_p16 / mc_p32: multicast addresses of the gradient buffer and of the two parameter copies (null = none).
// With them the owner's reduction is one `multimem.ld_reduce` per vector (the switch adds the ranks' values) and the
// write-back one `multimem.st` per copy (the switch replicates it) instead of one peer load / store per rank.
__global__ void __launch_bounds__(512) reduce_scatter_update_kernel(SymCtx c, float* const* grads, __nv_bfloat16* const* p16,
                                                                    float* const* p32, float* mc_grad, __nv_bfloat16* mc_p16,
                                                                    float* mc_p32, float* master, float* s1, float* s2,
                                                                    const long long* seg_start, const long long* seg_len,
                                                                    const long long* seg_state, const long long* seg_flags,
                                                                    const long long* owned_prefix, int nseg, OptArgs o, float scale) {
  if (!sym_barrier(c)) return;
  const long long total4 = owned_prefix[nseg] / 4;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
  const float lr = *o.lr;
  const float t = (float)(*o.step);
  const float c1 = 1.0f - powf(o.b1, t), c2 = 1.0f - powf(o.b2, t);
  for (long long q = tid; q < total4; q += nthr) {
    const long long e = q * 4;
    int lo = 0, hi = nseg - 1;                       // last segment whose prefix <= e
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (owned_prefix[mid] <= e) lo = mid; else hi = mid - 1; }
    const long long within = e - owned_prefix[lo];
    const long long gi = seg_start[lo] + within;     // index in the flat bucket
    const long long si = seg_state[lo] + within;     // index in the owner's compact state
    // bit 0 of the segment's flags: the consumers fetch this segment from its owner inside their GEMMs (gemm_gathered_b),
    // so the updated values are written to the owner's own copies only
    const bool local_only = seg_flags != nullptr && (seg_flags[lo] & 1);
    float g[4] = {0.f, 0.f, 0.f, 0.f};
    if (mc_grad != nullptr) {
      Wire<float>::mc_reduce(mc_grad + gi, g);
    } else {
      float4 v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) if (r < c.world) v[r] = *reinterpret_cast<const float4*>(grads[r] + gi);
#pragma unroll
      for (int r = 0; r < 8; ++r) if (r < c.world) { g[0] += v[r].x; g[1] += v[r].y; g[2] += v[r].z; g[3] += v[r].w; }
    }
    float4 pm = *reinterpret_cast<float4*>(master + si);
    float p[4] = {pm.x, pm.y, pm.z, pm.w};
    float a[4], b[4];
    if (s1) { float4 x = *reinterpret_cast<float4*>(s1 + si); a[0] = x.x; a[1] = x.y; a[2] = x.z; a[3] = x.w; }
    if (s2) { float4 x = *reinterpret_cast<float4*>(s2 + si); b[0] = x.x; b[1] = x.y; b[2] = x.z; b[3] = x.w; }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gr = g[j] * scale * o.grad_scale;
      if (o.kind == 1) {
        if (o.wd != 0.f) { if (o.decoupled) p[j] *= 1.0f - lr * o.wd; else gr += o.wd * p[j]; }
        a[j] = o.b1 * a[j] + (1.0f - o.b1) * gr;
        b[j] = o.b2 * b[j] + (1.0f - o.b2) * gr * gr;
        p[j] -= lr * (a[j] / c1) / (sqrtf(b[j] / c2) + o.eps);
      } else if (o.kind == 0) {
        gr += o.wd * p[j];
        if (o.momentum != 0.f) {
          a[j] = (*o.step <= 1) ? gr : o.momentum * a[j] + gr;
          gr = o.nesterov ? gr + o.momentum * a[j] : a[j];
        }
        p[j] -= lr * gr;
      } else {
        gr += o.wd * p[j];
        a[j] += gr * gr;
        p[j] -= lr * gr / (sqrtf(a[j]) + o.eps);
      }
    }
    *reinterpret_cast<float4*>(master + si) = make_float4(p[0], p[1], p[2], p[3]);
    if (s1) *reinterpret_cast<float4*>(s1 + si) = make_float4(a[0], a[1], a[2], a[3]);
    if (s2) *reinterpret_cast<float4*>(s2 + si) = make_float4(b[0], b[1], b[2], b[3]);
    __nv_bfloat162 h0 = __floats2bfloat162_rn(p[0], p[1]), h1 = __floats2bfloat162_rn(p[2], p[3]);
    const uint2 w = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
    if (local_only) {
      *reinterpret_cast<uint2*>(p16[c.rank] + gi) = w;
      if (p32) *reinterpret_cast<float4*>(p32[c.rank] + gi) = make_float4(p[0], p[1], p[2], p[3]);
      continue;
    }
    if (mc_p16 != nullptr) {
      asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc_p16 + gi), "f"(__uint_as_float(w.x)), "f"(__uint_as_float(w.y))
                   : "memory");
    } else {
#pragma unroll
      for (int r = 0; r < 8; ++r) if (r < c.world) *reinterpret_cast<uint2*>(p16[r] + gi) = w;
    }
    if (p32) {
      if (mc_p32 != nullptr) {
        Wire<float>::mc_store(mc_p32 + gi, p);
      } else {
#pragma unroll
        for (int r = 0; r < 8; ++r) if (r < c.world) *reinterpret_cast<float4*>(p32[r] + gi) = make_float4(p[0], p[1], p[2], p[3]);
      }
    }
  }
  sym_barrier(c);
}

// ------------------------------------------------------------------------------------------------ K4 / K5
// Rows of a [V, H] table split along axis 0 into `world` shards with sizes V/world (+1 for the first V%world);
// shard s lives on rank s at shard[s] with its rows re-based to 0.
__device__ __forceinline__ void owner_of(long long id, long long V, int world, int& owner, long long& local) {
  const long long qn = V / world, rn = V % world;
  long long a = id / (qn + 1), b = qn > 0 ? (id - rn) / qn : 0;
  owner = (int)(a > b ? a : b);
  local = id - (owner * qn + (owner < rn ? owner : rn));
}

// barriers: bit 0 = meet the peers before the first access (the owners' shards are ready), bit 1 = after the last one
// (every rank's rows have landed). A step with several lookups / pushes brackets the whole group instead of each call.
// touched (optional): per-owner byte flags, one per shard row; the flag of every row that receives a gradient is raised so
// that the owner's update can skip the rest of its shard.
__global__ void sparse_scatter_add_kernel(SymCtx c, float* const* shard, uint8_t* const* touched, const int64_t* ids,
                                          const __nv_bfloat16* vals32_or_16, int vals_are_bf16, long long nrows, int H, long long V,
                                          float scale, int barriers) {
  if ((barriers & 1) && !sym_barrier(c)) return;    // owners have zeroed their shards
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long long r = warp; r < nrows; r += nwarp) {
    const long long id = ids[r];
    if ((unsigned long long)id >= (unsigned long long)V) {       // a bad id must not become a write into a peer's memory
      if (lane == 0) atomicExch(c.error, 301);
      continue;
    }
    int owner; long long local;
    owner_of(id, V, c.world, owner, local);
    float* dst = shard[owner] + local * H;
    if (touched != nullptr && lane == 0) touched[owner][local] = 1;
    for (int col = lane * 4; col < H; col += 128) {
      float4 v;
      if (vals_are_bf16) {
        const __nv_bfloat16* s = vals32_or_16 + r * H + col;
        v = make_float4(__bfloat162float(s[0]), __bfloat162float(s[1]), __bfloat162float(s[2]), __bfloat162float(s[3]));
      } else {
        v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(vals32_or_16) + r * H + col);
      }
      v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
      atomicAdd(reinterpret_cast<float4*>(dst + col), v);   // red.global.add.v4.f32 on the owner's memory
    }
  }
  if (barriers & 2) sym_barrier(c);
}

__global__ void embedding_gather_peers_kernel(SymCtx c, __nv_bfloat16* const* shard, const int64_t* ids, __nv_bfloat16* out,
                                              long long nrows, int H, long long V, int barriers) {
  if ((barriers & 1) && !sym_barrier(c)) return;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarp = ((long long)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long long r = warp; r < nrows; r += nwarp) {
    const long long id = ids[r];
    if ((unsigned long long)id >= (unsigned long long)V) {       // a bad id reads nothing: its row is zero and the error is recorded
      if (lane == 0) atomicExch(c.error, 302);
      for (int col = lane * 8; col < H; col += 256) *reinterpret_cast<uint4*>(out + r * H + col) = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    int owner; long long local;
    owner_of(id, V, c.world, owner, local);
    const __nv_bfloat16* src = shard[owner] + local * H;
    for (int col = lane * 8; col < H; col += 256)
      *reinterpret_cast<uint4*>(out + r * H + col) = *reinterpret_cast<const uint4*>(src + col);
  }
  if (barriers & 2) sym_barrier(c);
}

// ------------------------------------------------------------------------------------------------ K20
// Staleness gate: publishes this rank's step to every peer and waits until step - min(peer steps) <= staleness.
__global__ void barrier_kernel(SymCtx c) { sym_barrier(c); }

// step_ptr (optional): the step is read from device memory (a counter the step's kernels increment), so that the launch can
// be replayed from a CUDA graph. staleness < 0: publish the step only (no wait). max_lead (optional): the largest lead over
// the slowest peer this rank ever had when it passed the gate.
__global__ void staleness_gate_kernel(SymCtx c, uint32_t* const* clocks, uint32_t my_step, const long long* step_ptr, int staleness,
                                      int* max_lead) {
  if (step_ptr != nullptr) my_step = (uint32_t)(*step_ptr);
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(clocks[threadIdx.x] + c.rank, my_step);
    if (staleness < 0) return;
    const uint32_t* theirs = clocks[c.rank] + threadIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    int32_t lead;
    while ((lead = (int32_t)(my_step - ld_acquire_sys(theirs))) > (int32_t)staleness) {
      if (((++it) & 63u) == 0 && globaltimer_ns() - t0 > c.timeout_ns) { atomicExch(c.error, 200 + threadIdx.x); break; }
    }
    if (max_lead != nullptr && lead > 0) atomicMax(max_lead, (int)lead);
  }
}

// ------------------------------------------------------------------------------------------------ relaxed parameter server
// Bounded-staleness / asynchronous modes with GPU owners and plain SGD: a worker applies its own gradient to the owner's fp32
// copy as soon as it has it - p_owner -= lr * g as a vector reduction over NVLink, which commutes with every other worker's, so
// no lock and no barrier is needed - and later refreshes its local copies from the owners. seg_owner[s] names the rank whose
// copy of segment s is the authoritative one.
__global__ void relaxed_push_sgd_kernel(float* const* p32, const float* __restrict__ grad, const long long* seg_start,
                                        const long long* seg_len, const long long* seg_owner, const long long* prefix, int nseg,
                                        const float* lr_ptr, float grad_scale) {
  const long long total4 = prefix[nseg] / 4;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
  const float step = -(*lr_ptr) * grad_scale;
  for (long long q = tid; q < total4; q += nthr) {
    const long long e = q * 4;
    int lo = 0, hi = nseg - 1;
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (prefix[mid] <= e) lo = mid; else hi = mid - 1; }
    const long long gi = seg_start[lo] + (e - prefix[lo]);
    const float4 g = *reinterpret_cast<const float4*>(grad + gi);
    atomicAdd(reinterpret_cast<float4*>(p32[seg_owner[lo]] + gi), make_float4(step * g.x, step * g.y, step * g.z, step * g.w));
  }
}

__global__ void relaxed_pull_kernel(float* const* p32, float* __restrict__ master, __nv_bfloat16* __restrict__ p16, const long long* seg_start,
                                    const long long* seg_len, const long long* seg_owner, const long long* prefix, int nseg, int rank) {
  const long long total4 = prefix[nseg] / 4;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
  for (long long q = tid; q < total4; q += nthr) {
    const long long e = q * 4;
    int lo = 0, hi = nseg - 1;
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (prefix[mid] <= e) lo = mid; else hi = mid - 1; }
    const long long gi = seg_start[lo] + (e - prefix[lo]);
    const int owner = (int)seg_owner[lo];
    const float4 v = *reinterpret_cast<const float4*>(p32[owner] + gi);
    if (owner != rank) *reinterpret_cast<float4*>(master + gi) = v;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p16 + gi) = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
  }
}

}  // namespace

int comm_grid(long long n_vec, int max_blocks) {
  long long b = (n_vec + 511) / 512;
  if (b < 1) b = 1;
  return (int)(b > max_blocks ? max_blocks : b);
}

// The grid barrier inside allreduce_kernel needs every block of the launch on an SM at the same time. The launch is an
// ordinary one, so the grid is cut to what the occupancy calculator says one GPU holds at once (SMs x blocks per SM for
// this kernel's registers and 512 threads); every rank runs the same kernel on the same part and gets the same number.
// Blocks of other streams' kernels only delay the arrival of a block: they never wait on this launch, and the wait is
// bounded by the context's timeout.
template <typename T>
static int resident_blocks(int blocks) {
  static int limit = 0;
  if (limit == 0) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_kernel<T>, 512, 0);
    limit = sms * per_sm > 0 ? sms * per_sm : 1;
  }
  return blocks < limit ? blocks : limit;
}

void launch_allreduce(const SymCtx& c, void* const* bufs, void* mc, int wire, long long n, const float* src32, float* residual,
                      float* dst32, float scale, int blocks, cudaStream_t st) {
  if (wire == WIRE_F32)
    allreduce_kernel<float><<<resident_blocks<float>(blocks), 512, 0, st>>>(c, reinterpret_cast<float* const*>(bufs), reinterpret_cast<float*>(mc), n, src32, residual, dst32, scale);
  else if (wire == WIRE_BF16)
    allreduce_kernel<__nv_bfloat16><<<resident_blocks<__nv_bfloat16>(blocks), 512, 0, st>>>(c, reinterpret_cast<__nv_bfloat16* const*>(bufs), reinterpret_cast<__nv_bfloat16*>(mc), n, src32, residual, dst32, scale);
  else
    allreduce_kernel<__half><<<resident_blocks<__half>(blocks), 512, 0, st>>>(c, reinterpret_cast<__half* const*>(bufs), reinterpret_cast<__half*>(mc), n, src32, residual, dst32, scale);
}

void launch_reduce_scatter_update(const SymCtx& c, float* const* grads, __nv_bfloat16* const* p16, float* const* p32, float* mc_grad,
                                  __nv_bfloat16* mc_p16, float* mc_p32, float* master,
                                  float* s1, float* s2, const long long* seg_start, const long long* seg_len, const long long* seg_state,
                                  const long long* seg_flags, const long long* owned_prefix, int nseg, int kind, const float* lr, const long long* step, float b1,
                                  float b2, float eps, float wd, float momentum, float grad_scale, int decoupled, int nesterov,
                                  float scale, int blocks, cudaStream_t st) {
  OptArgs o{kind, lr, step, b1, b2, eps, wd, momentum, grad_scale, decoupled, nesterov};
  reduce_scatter_update_kernel<<<blocks, 512, 0, st>>>(c, grads, p16, p32, mc_grad, mc_p16, mc_p32, master, s1, s2, seg_start, seg_len, seg_state, seg_flags,
                                                       owned_prefix, nseg, o, scale);
}

void launch_sparse_scatter_add(const SymCtx& c, float* const* shard, uint8_t* const* touched, const int64_t* ids, const void* vals,
                               int vals_are_bf16, long long nrows, int H, long long V, float scale, int barriers, int blocks, cudaStream_t st) {
  sparse_scatter_add_kernel<<<blocks, 256, 0, st>>>(c, shard, touched, ids, reinterpret_cast<const __nv_bfloat16*>(vals), vals_are_bf16, nrows, H, V,
                                                    scale, barriers);
}

void launch_embedding_gather_peers(const SymCtx& c, __nv_bfloat16* const* shard, const int64_t* ids, __nv_bfloat16* out, long long nrows,
                                   int H, long long V, int barriers, int blocks, cudaStream_t st) {
  embedding_gather_peers_kernel<<<blocks, 256, 0, st>>>(c, shard, ids, out, nrows, H, V, barriers);
}

void launch_barrier(const SymCtx& c, int blocks, cudaStream_t st) { barrier_kernel<<<blocks, 32, 0, st>>>(c); }

void launch_staleness_gate(const SymCtx& c, uint32_t* const* clocks, uint32_t my_step, const long long* step_ptr, int staleness, int* max_lead,
                           cudaStream_t st) {
  staleness_gate_kernel<<<1, 32, 0, st>>>(c, clocks, my_step, step_ptr, staleness, max_lead);
}

void launch_relaxed_push_sgd(float* const* p32, const float* grad, const long long* seg_start, const long long* seg_len,
                             const long long* seg_owner, const long long* prefix, int nseg, const float* lr, float grad_scale, int blocks,
                             cudaStream_t st) {
  relaxed_push_sgd_kernel<<<blocks, 512, 0, st>>>(p32, grad, seg_start, seg_len, seg_owner, prefix, nseg, lr, grad_scale);
}

void launch_relaxed_pull(float* const* p32, float* master, __nv_bfloat16* p16, const long long* seg_start, const long long* seg_len,
                         const long long* seg_owner, const long long* prefix, int nseg, int rank, int blocks, cudaStream_t st) {
  relaxed_pull_kernel<<<blocks, 512, 0, st>>>(p32, master, p16, seg_start, seg_len, seg_owner, prefix, nseg, rank);
}

}  // namespace adb200
