// Host-side launchers of the memory-bound kernels in elementwise.cu.  Every
// function enqueues on `st`, allocates nothing, and returns 0 on success,
// -1 for an unsupported shape and -3 for a launch error.  bf16 tensors are
// passed as void*.
#pragma once
#include <cuda_runtime.h>

namespace piper {

// y = rmsnorm(x (+ res)) * w; when res != nullptr the sum is also written to
// h_out (the new residual stream).  rstd[T] is saved for backward.
int rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                long long T, int D, float eps, cudaStream_t st);

// Number of row-strips (and rows of dw_partial) rmsnorm_bwd uses for T rows.
int rmsnorm_bwd_num_partials(long long T);

// dx = d rmsnorm / dx (+ dres); dw goes to dw_f32 and/or dw_bf16 (either may
// be null), added to the existing value when accumulate != 0.  dw_partial is
// caller-provided scratch of rmsnorm_bwd_num_partials(T) * D floats.
int rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                void* dx, float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate, long long T,
                int D, cudaStream_t st);

// Packed qkv [T, (Hq+2Hkv)*hd] -> same layout with optional per-head RMSNorm
// (qw/kw, may be null) and rotary embedding applied to the q and k heads.
int qk_rope_fwd(const void* in, void* out, const float* cosp, const float* sinp, const void* qw,
                const void* kw, long long T, int S, int Hq, int Hkv, int hd, int interleaved, float eps,
                cudaStream_t st);
int qk_rope_bwd(const void* dout, const void* in, void* din, const float* cosp, const float* sinp,
                const void* qw, const void* kw, float* dqw, float* dkw, long long T, int S, int Hq,
                int Hkv, int hd, int interleaved, float eps, cudaStream_t st);

int swiglu_fwd(const void* h13, void* act, long long T, int F, cudaStream_t st);
int swiglu_bwd(const void* h13, const void* dact, void* dh13, long long T, int F, cudaStream_t st);

int embedding_fwd(const long long* tokens, const void* table, void* out, long long T, int D, int V,
                  int* status, cudaStream_t st);
int embedding_bwd(const long long* tokens, const void* dout, float* dtable, long long T, int D, int V,
                  cudaStream_t st);

// Per-row loss and log-sum-exp of bf16 logits [T, V] with row stride ld.
int ce_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long T, int V,
           long long ld, long long ignore_index, cudaStream_t st);
// out = (softmax - onehot) * gscale[0] * row_scale; out may alias logits.
int ce_bwd(const void* logits, const long long* labels, const float* lse, const float* gscale,
           float row_scale, void* out, long long T, int V, long long ld, long long ignore_index,
           cudaStream_t st);

int adam_flat(float* master, float* m, float* v, const float* grad, void* param_bf16, long long n,
              float lr, float b1, float b2, float eps, float wd, int step, float grad_scale, int decoupled,
              cudaStream_t st);
int cast_f32_to_bf16(const float* in, void* out, long long n, float scale, cudaStream_t st);
int add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t st);
int accum_bf16_into_f32(const void* g, float* acc, long long n, cudaStream_t st);

}  // namespace piper
