// Data-parallel gradient reduction fused with the sharded optimizer step, and the ZeRO-3 parameter gather, as
// kernels over NVLink peer memory (zero_fused.cu).
//
// Sharding is by parameter rows: parameter i of a bucket, seen as [N_i, K_i], is cut into dp pieces of R_i rows
// (R_i = ceil(N_i / dp) rounded up to 64), rank p owning piece p.  A rank's shard buffers (bf16 parameters, fp32
// master weights, Adam moments, gradient accumulator) are the concatenation of its pieces; piece p of parameter i
// starts at shard_off[i] in every rank's shard and at full_base[i] + p * stride[i] in the full, unsharded layout
// (stride[i] = R_i * K_i elements).  Row pieces are what the all-gather GEMM (ag_gemm_sm100.cu) consumes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace piper {

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale;
  int decoupled_decay;           // 1: AdamW (w -= lr*wd*w); 0: Adam with L2 decay folded into the gradient
};

// Device arrays of length n (one entry per parameter of the bucket), all in elements.
struct ZeroTable {
  const long long* full_base;    // offset of the parameter in the full layout (a multiple of 64)
  const long long* shard_off;    // offset of a rank's piece in its shard buffers
  const long long* stride;       // elements per piece (a multiple of 64)
  const long long* padded;       // parameter size rounded up to 64 (the full layout keeps that padding)
  int n;
};

struct ZeroReduceArgs {
  const float* const* peer_grads;   // [dp] full fp32 gradient buffers (symmetric memory)
  float* shard_grads;               // [S] gradient accumulator of this rank's shard, or null
  float* master;                    // [S] fp32 master weights, Adam moments
  float* m;
  float* v;
  void* shard_params;               // [S] bf16 parameters of this rank's shard
  void* const* peer_params;         // [dp] full bf16 parameter buffers to store the update into, or null
  ZeroTable t;
  int my_rank, dp;
  int accumulate;                   // add the reduced gradients to shard_grads (read-modify-write)
  int final_step;                   // apply Adam with the accumulated gradients and clear the accumulator
  AdamHyper h;
  uint64_t* const* peer_flags;      // [dp] flag arrays; DONE block of dp words at done_off
  int done_off;
  unsigned long long use;
  unsigned int* cta_counter;
  const int* abort;                 // set by the wait kernel in front: skip everything
  int num_ctas;
};

// shard_grads (+)= sum over ranks of their gradients for this rank's pieces; clears this rank's own copy of those
// pieces; with final_step also Adam, the new bf16 shard, and (peer_params given) the new parameters stored into
// every rank's full buffer.  The last CTA publishes `use` in the DONE block of every rank.
int zero_reduce(const ZeroReduceArgs& a, cudaStream_t st);

// Clears every piece of the full gradient buffer that another rank owns (after all ranks have read them).
int zero_clear_others(float* grads, const ZeroTable& t, int my_rank, int dp, int num_ctas, cudaStream_t st);

// full[piece p of parameter i] = shard of rank p, for every rank p and every parameter except skip_slot
// (only parameter only_slot when that is >= 0).
int zero_gather(const void* const* peer_shards, void* full, const ZeroTable& t, int dp, int skip_slot, int only_slot,
                const int* abort, int num_ctas, cudaStream_t st);

}  // namespace piper
