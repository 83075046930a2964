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

#include <cstdlib>

#include "peer_sync.cuh"
#include "ptx.cuh"

namespace piper {
namespace {

constexpr int F1_THREADS = 256;
// float4 vectors per thread per trip (all loads are issued before any use); fewer for large groups, whose
// per-vector peer loads already keep enough bytes in flight
__host__ __device__ constexpr int f1_unroll(int dp) { return dp <= 2 ? 4 : (dp <= 4 ? 2 : 1); }

__device__ __forceinline__ float4 ld_stream_f4(const float* p) {
  float4 r;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void adam_vec(float4& g, float4& w, float4& mm, float4& vv, const AdamHyper& h) {
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
}

// DP > 0: group size known at compile time (peer loops fully unrolled); DP == 0: any size.
template <int DP>
__global__ void __launch_bounds__(F1_THREADS)
f1_kernel(const float* const* __restrict__ peer_grads, __nv_bfloat16* const* __restrict__ peer_params,
          uint64_t* const* __restrict__ peer_flags, float* __restrict__ master, float* __restrict__ m,
          float* __restrict__ v, int my_rank, int dp_rt, long long shard_numel, unsigned long long epoch,
          AdamHyper h, unsigned int* cta_counter, int* status, unsigned long long timeout_ns) {
  __shared__ int ok_s;
  const int dp = DP > 0 ? DP : dp_rt;
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
  const long long stride = static_cast<long long>(gridDim.x) * F1_THREADS;
  const long long first = static_cast<long long>(blockIdx.x) * F1_THREADS + threadIdx.x;
  if (DP > 0) {
    constexpr int NP = DP > 0 ? DP : 1;
    constexpr int F1_UNROLL = f1_unroll(NP);
    const float* gsrc[NP];
    __nv_bfloat16* pdst[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      // start with the next rank's copy so that the ranks of a group do not all read the same peer at once
      const int q = (my_rank + 1 + p) % NP;
      gsrc[p] = peer_grads[q] + base;
      pdst[p] = peer_params[q] + base;
    }
    for (long long i0 = first; i0 < nvec; i0 += stride * F1_UNROLL) {
      float4 g[F1_UNROLL][NP], w[F1_UNROLL], mm[F1_UNROLL], vv[F1_UNROLL];
#pragma unroll
      for (int u = 0; u < F1_UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) {
#pragma unroll
          for (int p = 0; p < NP; ++p) g[u][p] = ld_stream_f4(gsrc[p] + 4 * i);
          w[u] = ld_stream_f4(master + 4 * i);
          mm[u] = ld_stream_f4(m + 4 * i);
          vv[u] = ld_stream_f4(v + 4 * i);
        }
      }
#pragma unroll
      for (int u = 0; u < F1_UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) {
          float4 s = g[u][0];
#pragma unroll
          for (int p = 1; p < NP; ++p) {
            s.x += g[u][p].x; s.y += g[u][p].y; s.z += g[u][p].z; s.w += g[u][p].w;
          }
          adam_vec(s, w[u], mm[u], vv[u], h);
          // this rank's own copy of the slice is read by nobody else: clear it for the next step right away
          reinterpret_cast<float4*>(const_cast<float*>(gsrc[NP - 1]))[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          reinterpret_cast<float4*>(master)[i] = w[u];
          reinterpret_cast<float4*>(m)[i] = mm[u];
          reinterpret_cast<float4*>(v)[i] = vv[u];
          uint2 packed;
          packed.x = pack_bf16x2(w[u].x, w[u].y);
          packed.y = pack_bf16x2(w[u].z, w[u].w);
#pragma unroll
          for (int p = 0; p < NP; ++p) reinterpret_cast<uint2*>(pdst[p])[i] = packed;
        }
      }
    }
  } else {
    for (long long i = first; i < nvec; i += stride) {
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < dp; ++p) {
        const float4 t = ld_stream_f4(peer_grads[p] + base + 4 * i);
        g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
      }
      float4 w = reinterpret_cast<float4*>(master)[i];
      float4 mm = reinterpret_cast<float4*>(m)[i];
      float4 vv = reinterpret_cast<float4*>(v)[i];
      adam_vec(g, w, mm, vv, h);
      reinterpret_cast<float4*>(master)[i] = w;
      reinterpret_cast<float4*>(m)[i] = mm;
      reinterpret_cast<float4*>(v)[i] = vv;
      uint2 packed;
      packed.x = pack_bf16x2(w.x, w.y);
      packed.y = pack_bf16x2(w.z, w.w);
      for (int p = 0; p < dp; ++p) reinterpret_cast<uint2*>(peer_params[p] + base)[i] = packed;
    }
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
  // nobody reads the local gradients any more: clear the slices the peers have read (the fixed-size path has
  // already cleared this rank's own slice)
  float4* lg = reinterpret_cast<float4*>(const_cast<float*>(peer_grads[my_rank]));
  const long long total_vec = shard_numel * dp / 4;
  const long long own_lo = DP > 0 ? base / 4 : -1, own_hi = DP > 0 ? base / 4 + nvec : -1;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (long long i = first; i < total_vec; i += stride)
    if (i < own_lo || i >= own_hi) lg[i] = z;
}

}  // namespace

int f1_rs_adam_ag(const float* const* peer_grads, void* const* peer_params, uint64_t* const* peer_flags,
                  float* master, float* m, float* v, int my_rank, int dp, long long shard_numel,
                  unsigned long long epoch, AdamHyper h, unsigned int* cta_counter, int* status,
                  unsigned long long timeout_ns, int num_ctas, cudaStream_t st) {
  if (shard_numel % 4 != 0 || dp < 1) return -1;
  if (shard_numel == 0) return 0;
  auto pp = reinterpret_cast<__nv_bfloat16* const*>(peer_params);
  // Every CTA waits inside the kernel for the last CTA of each rank, so the whole grid has to be resident at
  // once: never launch more CTAs than fit on the device.
#define PIPER_F1_LAUNCH(DPV)                                                                                   \
  {                                                                                                            \
    static int capacity = 0;                                                                                   \
    if (capacity == 0) {                                                                                       \
      int per_sm = 0, dev = 0, sms = 0;                                                                        \
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, f1_kernel<DPV>, F1_THREADS, 0) !=             \
              cudaSuccess ||                                                                                   \
          cudaGetDevice(&dev) != cudaSuccess ||                                                                \
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || per_sm < 1)      \
        return -2;                                                                                             \
      capacity = per_sm * sms;                                                                                 \
    }                                                                                                          \
    if (num_ctas > capacity) num_ctas = capacity;                                                              \
    if (num_ctas < 1) num_ctas = 1;                                                                            \
    f1_kernel<DPV><<<num_ctas, F1_THREADS, 0, st>>>(peer_grads, pp, peer_flags, master, m, v, my_rank, dp,      \
                                                    shard_numel, epoch, h, cta_counter, status, timeout_ns);   \
  }
  switch (dp) {
    case 1: PIPER_F1_LAUNCH(1); break;
    case 2: PIPER_F1_LAUNCH(2); break;
    case 4: PIPER_F1_LAUNCH(4); break;
    case 8: PIPER_F1_LAUNCH(8); break;
    default: PIPER_F1_LAUNCH(0); break;
  }
#undef PIPER_F1_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper

