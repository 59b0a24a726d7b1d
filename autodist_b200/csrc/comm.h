// Host-side interface of the symmetric-memory communication kernels (see comm.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace adb200 {

enum WireType { WIRE_F32 = 0, WIRE_BF16 = 1, WIRE_F16 = 2 };
constexpr int kMaxCommBlocks = 128;

struct SymCtx {
  uint32_t* const* flags;      // device array [world]: rank r's flag words, laid out [block][sender]
  uint32_t* epochs;            // local device array [kMaxCommBlocks + 2]: barriers each block index has passed, then the
                               // two words (arrival count, generation) of the local grid-wide barrier
  int* error;                  // local device int: 0 = fine, 100+peer / 200+peer = a bounded wait gave up
  int rank, world;
  unsigned long long timeout_ns;
};

int comm_grid(long long n_vec, int max_blocks);
void launch_allreduce(const SymCtx& c, void* const* bufs, void* mc, int wire, long long n, const float* src32, float* residual,
                      float* dst32, float scale, int blocks, cudaStream_t st);
void launch_reduce_scatter_update(const SymCtx& c, float* const* grads, __nv_bfloat16* const* p16, float* const* p32, float* mc_grad,
                                  __nv_bfloat16* mc_p16, float* mc_p32, float* master,
                                  float* s1, float* s2, const long long* seg_start, const long long* seg_len, const long long* seg_state,
                                  const long long* seg_flags, const long long* owned_prefix, int nseg, int kind, const float* lr, const long long* step, float b1,
                                  float b2, float eps, float wd, float momentum, float grad_scale, int decoupled, int nesterov,
                                  float scale, int blocks, cudaStream_t st);
void launch_sparse_scatter_add(const SymCtx& c, float* const* shard, uint8_t* const* touched, const int64_t* ids, const void* vals,
                               int vals_are_bf16, long long nrows, int H, long long V, float scale, int barriers, int blocks, cudaStream_t st);
void launch_embedding_gather_peers(const SymCtx& c, __nv_bfloat16* const* shard, const int64_t* ids, __nv_bfloat16* out, long long nrows,
                                   int H, long long V, int barriers, int blocks, cudaStream_t st);
void launch_barrier(const SymCtx& c, int blocks, cudaStream_t st);
void launch_staleness_gate(const SymCtx& c, uint32_t* const* clocks, uint32_t my_step, const long long* step_ptr, int staleness, int* max_lead,
                           cudaStream_t st);
void launch_relaxed_push_sgd(float* const* p32, const float* grad, const long long* seg_start, const long long* seg_len,
                             const long long* seg_owner, const long long* prefix, int nseg, const float* lr, float grad_scale, int blocks,
                             cudaStream_t st);
void launch_relaxed_pull(float* const* p32, float* master, __nv_bfloat16* p16, const long long* seg_start, const long long* seg_len,
                         const long long* seg_owner, const long long* prefix, int nseg, int rank, int blocks, cudaStream_t st);

}  // namespace adb200
