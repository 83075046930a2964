// Fused compute + collective kernels over NVLink peer memory.
//
// f1: data-parallel gradient bucket -> updated parameters, one kernel.
//   1. every CTA publishes "my gradients are final" (epoch) into each peer's
//      flag block and waits, bounded, for the same flag from every peer;
//   2. for the elements of this rank's shard it sums the fp32 gradients of
//      all ranks with 16-byte peer loads, applies Adam to the fp32 master
//      weights and moments, and stores the new bf16 parameters into every
//      rank's parameter buffer (peer stores) - reduce-scatter, optimizer and
//      all-gather without touching HBM in between;
//   3. the last CTA to finish publishes "done"; every CTA waits for "done"
//      from all peers (so the local parameter buffer is complete and nobody
//      reads the local gradients any more) and zeroes its slice of the local
//      gradient bucket for the next step.
// Plain ld/st over peer mappings only: no TMA, no multicast.
#include "fused_collectives.h"

#include <cuda_bf16.h>

#include "ptx.cuh"

namespace piper {
namespace {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const uint64_t* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint64_t* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Waits until flags[0..n) are all >= epoch.  Bounded by a wall-clock deadline
// and by the shared status word (another CTA or kernel already failed).
__device__ bool wait_flags(const uint64_t* flags, int n, unsigned long long epoch,
                           unsigned long long timeout_ns, int* status) {
  const unsigned long long t0 = globaltimer_ns();
  for (int p = 0; p < n; ++p) {
    unsigned spins = 0;
    while (ld_acquire_sys(flags + p) < epoch) {
      if ((++spins & 255u) == 0) {
        if (*reinterpret_cast<volatile int*>(status) != 0) return false;
        if (globaltimer_ns() - t0 > timeout_ns) {
          atomicCAS(status, 0, kStatusPeerTimeout);
          return false;
        }
      }
      __nanosleep(64);
    }
  }
  return true;
}

constexpr int F1_THREADS = 256;

__global__ void __launch_bounds__(F1_THREADS)
f1_kernel(const float* const* __restrict__ peer_grads, __nv_bfloat16* const* __restrict__ peer_params,
          uint64_t* const* __restrict__ peer_flags, float* __restrict__ master, float* __restrict__ m,
          float* __restrict__ v, int my_rank, int dp, long long shard_numel, unsigned long long epoch,
          AdamHyper h, unsigned int* cta_counter, int* status, unsigned long long timeout_ns) {
  __shared__ int ok_s;
  uint64_t* local_flags = peer_flags[my_rank];
  // ---- 1. publish "gradients final", wait for the peers
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int p = 0; p < dp; ++p) st_release_sys(peer_flags[p] + my_rank, epoch);
    ok_s = wait_flags(local_flags, dp, epoch, timeout_ns, status) ? 1 : 0;
  }
  __syncthreads();
  if (!ok_s) return;

  // ---- 2. reduce + Adam + parameter broadcast over this rank's shard
  const long long base = static_cast<long long>(my_rank) * shard_numel;
  const long long nvec = shard_numel / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * F1_THREADS + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * F1_THREADS) {
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < dp; ++p) {
      const float4 t = reinterpret_cast<const float4*>(peer_grads[p] + base)[i];
      g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
    }
    float4 w = reinterpret_cast<float4*>(master)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* gp = reinterpret_cast<float*>(&g);
    float* wp = reinterpret_cast<float*>(&w);
    float* mp = reinterpret_cast<float*>(&mm);
    float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gr = gp[k] * h.grad_scale;
      mp[k] = h.beta1 * mp[k] + (1.f - h.beta1) * gr;
      vp[k] = h.beta2 * vp[k] + (1.f - h.beta2) * gr * gr;
      const float denom = sqrtf(vp[k] / h.bias_corr2) + h.eps;
      wp[k] = wp[k] - h.lr * (mp[k] / h.bias_corr1) / denom - h.lr * h.weight_decay * wp[k];
    }
    reinterpret_cast<float4*>(master)[i] = w;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    uint2 packed;
    packed.x = pack_bf16x2(wp[0], wp[1]);
    packed.y = pack_bf16x2(wp[2], wp[3]);
    for (int p = 0; p < dp; ++p) reinterpret_cast<uint2*>(peer_params[p] + base)[i] = packed;
  }

  // ---- 3. last CTA publishes "done"; everyone waits for the peers' "done"
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < dp; ++p) st_release_sys(peer_flags[p] + dp + my_rank, epoch);
    }
    ok_s = wait_flags(local_flags + dp, dp, epoch, timeout_ns, status) ? 1 : 0;
  }
  __syncthreads();
  if (!ok_s) return;
  // nobody reads the local gradients any more: clear them for the next step
  float4* lg = reinterpret_cast<float4*>(const_cast<float*>(peer_grads[my_rank]));
  const long long total_vec = shard_numel * dp / 4;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i = static_cast<long long>(blockIdx.x) * F1_THREADS + threadIdx.x; i < total_vec;
       i += static_cast<long long>(gridDim.x) * F1_THREADS)
    lg[i] = z;
}

}  // namespace

int f1_rs_adam_ag(const float* const* peer_grads, void* const* peer_params, uint64_t* const* peer_flags,
                  float* master, float* m, float* v, int my_rank, int dp, long long shard_numel,
                  unsigned long long epoch, AdamHyper h, unsigned int* cta_counter, int* status,
                  unsigned long long timeout_ns, int num_ctas, cudaStream_t st) {
  if (shard_numel % 4 != 0 || dp < 1) return -1;
  if (shard_numel == 0) return 0;
  f1_kernel<<<num_ctas, F1_THREADS, 0, st>>>(peer_grads, reinterpret_cast<__nv_bfloat16* const*>(peer_params),
                                            peer_flags, master, m, v, my_rank, dp, shard_numel, epoch, h,
                                            cta_counter, status, timeout_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper
