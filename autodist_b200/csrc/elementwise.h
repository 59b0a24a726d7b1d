// Host-side interface of the bandwidth-bound kernels (see elementwise.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace adb200 {
typedef __nv_bfloat16 bf16_t;
void ln_fwd(const bf16_t* x, const bf16_t* res, const float* gamma, const float* beta, bf16_t* z, bf16_t* y, float* mean, float* rstd,
            int rows, int H, float eps, float p_drop, uint64_t seed, const long long* step, cudaStream_t st);
int ln_bwd_blocks(int rows);
int ln_bwd_part_floats(int H);
void ln_bwd(const bf16_t* dy, const bf16_t* z, const float* mean, const float* rstd, const float* gamma, const bf16_t* dz_add, bf16_t* dz,
            bf16_t* dx, float* part, float* dgamma, float* dbeta, float* dsum, int rows, int H, float p_drop, uint64_t seed,
            const long long* step, int accumulate, cudaStream_t st);
void embed_sum(const bf16_t* word, const bf16_t* pos, const bf16_t* type, const int64_t* ids, const int64_t* tt, bf16_t* z, int rows, int S,
               int H, long long V, long long types, int* error, cudaStream_t st);
void scatter_add_rows(float* dst, const int64_t* idx, const bf16_t* src, int rows, int H, float scale, cudaStream_t st);
void strided_rowsum(const bf16_t* x, float* out, int keys, int stride, int count, int H, cudaStream_t st);
int colsum_parts(int rows);
void keyed_colsum(const bf16_t* x, const int64_t* key, float* part, float* out, int rows, int H, int keys, int accumulate, cudaStream_t st);
void gather_rows(const bf16_t* src, const int64_t* idx, bf16_t* out, int rows, int H, cudaStream_t st);
void gather_rows_f32(const float* src, const int64_t* idx, bf16_t* out, int rows, int H, cudaStream_t st);
void scatter_add_rows_bf16(bf16_t* dst, const int64_t* idx, const bf16_t* src, int rows, int H, cudaStream_t st);
bool softmax_supported(int S);
void softmax_fwd(const bf16_t* x, const float* mask, bf16_t* p, bf16_t* p_drop, long long rows, int S, int rows_per_batch, float scale,
                 float pd, uint64_t seed, const long long* step, cudaStream_t st);
void softmax_bwd(bf16_t* dp, const bf16_t* p, long long rows, int S, float scale, float pd, uint64_t seed, const long long* step,
                 cudaStream_t st);
void weight_sum(const float* w, int n, float* out, float eps, cudaStream_t st);
void xent(bf16_t* logits, const int64_t* labels, const float* weights, const float* denom, float* loss_sum, int rows, int V, int ld,
          float loss_scale, cudaStream_t st);
void gelu_bwd(const bf16_t* dy, const bf16_t* u, bf16_t* dx, long long n, cudaStream_t st);
void tanh_bwd(const bf16_t* dy, const bf16_t* y, bf16_t* dx, long long n, cudaStream_t st);
void add_bf16(const bf16_t* a, const bf16_t* b, bf16_t* out, long long n, cudaStream_t st);
void adam_update(float* p, const float* g, float* m, float* v, bf16_t* p16, long long n, const float* lr, float b1, float b2,
                 float eps, float wd, int decoupled, const long long* step, float grad_scale, cudaStream_t st);
void sgd_update(float* p, const float* g, float* mom, bf16_t* p16, long long n, const float* lr, float momentum, float dampening,
                float wd, int nesterov, const long long* step, float grad_scale, cudaStream_t st);
void sparse_rows_update(float* p, float* s1, float* s2, bf16_t* p16, const int64_t* rows, const float* g, int n, int H, long long V,
                        int kind, const float* lr, float b1, float b2, float eps, const long long* step, float grad_scale,
                        cudaStream_t st);
void flagged_rows_update(float* p, float* s1, float* s2, bf16_t* p16, float* g, uint8_t* flags, long long rows, int H, int kind,
                         const float* lr, float b1, float b2, float eps, const long long* step, cudaStream_t st);
void adagrad_update(float* p, const float* g, float* acc, bf16_t* p16, long long n, const float* lr, float eps, float wd,
                    float grad_scale, cudaStream_t st);
void lstm_cell_fwd(const float* gates, const float* c_prev, float* c, bf16_t* h, int B, int S, float fb, cudaStream_t st);
void lstm_cell_bwd(const float* gates, const float* c_prev, const float* c, const float* dh, const float* dc_next, float* dgates,
                   float* dc_prev, int B, int S, float fb, cudaStream_t st);
void sumsq(const float* x, long long n, float* acc, float weight, cudaStream_t st);
void clip_scale(float* x, long long n, const float* acc, float max_norm, cudaStream_t st);
int bn_parts(int rows, int C);
int bn_bwd_part_floats(int C);
void bn_fwd(const bf16_t* x, const float* gamma, const float* beta, const bf16_t* res, bf16_t* y, float* mean, float* rstd, float* part,
            float* sums, float* coef, int rows, int C, float eps, int relu, int sums_given, float* run_mean, float* run_var,
            long long* batches, float momentum, cudaStream_t st);
void bn_bwd(const bf16_t* dy, const bf16_t* x, const bf16_t* y, const float* mean, const float* rstd, const float* gamma, bf16_t* dx,
            bf16_t* dres, float* part, float* sums, float* coef, int rows, int C, int relu, float* dgamma_acc, float* dbeta_acc, cudaStream_t st);
void maxpool_fwd(const bf16_t* x, bf16_t* y, uint8_t* code, int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo,
                 cudaStream_t st);
void maxpool_bwd(const uint8_t* code, const bf16_t* dy, bf16_t* dx, int N, int H, int W, int C, int k, int stride, int pad, int Ho,
                 int Wo, cudaStream_t st);
void im2col(const bf16_t* x, bf16_t* cols, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Ho, int Wo, cudaStream_t st);
void col2im(const bf16_t* dcols, bf16_t* dx, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Ho, int Wo, cudaStream_t st);
void pad_image8(const void* x, int is_fp32, long long sn, long long sc, long long sh, long long sw, int N, int C, int H, int W, bf16_t* xp,
                int Hp, int Wp, int pad, cudaStream_t st);
void relu_bwd_colsum(const bf16_t* dy, const bf16_t* y, bf16_t* dx, float* part, float* out, int rows, int C, int accumulate,
                     cudaStream_t st);
void relu_bwd(const bf16_t* dy, const bf16_t* y, bf16_t* dx, long long n, cudaStream_t st);
void psgd_p(float* M, const float* err, const float* Q, float* P, int m, int n, int r, cudaStream_t st);
void psgd_q(const float* M, const float* P, float* Qn, int m, int n, int r, cudaStream_t st);
void psgd_d(float* M, float* err, const float* P, const float* Q, int m, int n, int r, cudaStream_t st);
void psgd_batched(int phase, float* grad, float* err, float* P, float* Q, const long long* off, const int* m, const int* n,
                  const long long* p_off, const long long* q_off, const long long* row_prefix, const long long* blk_prefix,
                  const long long* elem_prefix, int nmat, int r, long long rows, long long blocks, long long elems, cudaStream_t st);
void cast_f32_bf16(const float* x, bf16_t* y, long long n, cudaStream_t st);
void increment(long long* c, cudaStream_t st);
}  // namespace adb200
