// Host-side launchers of the kernels that fuse a collective with the compute
// next to it over NVLink peer memory (fused_collectives.cu), and of the
// symmetric-memory helpers they need (symm.cpp).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace piper {

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale;
};

// Data-parallel bucket update in one kernel: reduce-scatter of the fp32
// gradient bucket over peer memory, Adam on this rank's shard, and all-gather
// of the updated bf16 parameters by storing them into every peer's buffer.
//   peer_grads[p], peer_params[p], peer_flags[p]: device arrays (length dp) of
//   pointers into rank p's symmetric buffers; flags block = 2*dp uint64
//   (ready[dp], done[dp]).  master/m/v: this rank's fp32 shard (shard_numel).
//   epoch must increase by one per launch on every rank.  timeout_ns bounds
//   every wait on a peer; on expiry status is set to kStatusPeerTimeout.
int f1_rs_adam_ag(const float* const* peer_grads, void* const* peer_params, uint64_t* const* peer_flags,
                  float* master, float* m, float* v, int my_rank, int dp, long long shard_numel,
                  unsigned long long epoch, AdamHyper h, unsigned int* cta_counter, int* status,
                  unsigned long long timeout_ns, int num_ctas, cudaStream_t st);

// Expert-parallel dispatch: writes every (token, choice) row of x [T, D] into the region that the owner of
// its expert keeps for this source rank (peer stores), publishes the per-expert counts and a completion flag.
// pos[t*k+j] = owner * (ep*cap) + row inside the owner's buffer.  cursor [ep*experts_local] must be zero and
// seg_off is scratch of the same size.  Flag block layout per rank: dispatch_ready[ep], out_ready[ep].
int ep_dispatch_push(const void* x, const int* idx, const int* counts, int* seg_off, int* cursor, int* pos,
                     void* const* peer_recv, int* const* peer_meta, uint64_t* const* peer_flags,
                     unsigned int* cta_counter, int my_rank, int ep, int experts_local, long long T, int D, int k,
                     int cap, unsigned long long epoch, int num_ctas, cudaStream_t st);

// Owner side: wait (bounded) for all sources, then build the group table of the regions and the flat
// count vector [ep * experts_local].
int ep_wait_table(const uint64_t* flags, const int* meta, int* g_start, int* g_len, int* counts_out, int ep,
                  int experts_local, int cap, unsigned long long epoch, unsigned long long timeout_ns, int* status,
                  cudaStream_t st);

// Publishes `epoch` into slot (slot0 + my_rank) of every peer's flag block.
int ep_signal(uint64_t* const* peer_flags, int slot0, int my_rank, int ep, unsigned long long epoch, cudaStream_t st);

// Token side: out[t] = sum_j weights[t,j] * (row pos[t*k+j] of the owner's output buffer), after waiting
// (bounded) for every owner's "outputs ready" flag.
int ep_combine_pull(const void* const* peer_out, const int* pos, const float* weights, void* out,
                    const uint64_t* out_flags, long long T, int D, int k, int ep, int cap, unsigned long long epoch,
                    unsigned long long timeout_ns, int* status, int num_ctas, cudaStream_t st);

}  // namespace piper
