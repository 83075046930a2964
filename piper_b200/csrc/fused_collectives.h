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

}  // namespace piper
