// Gradient reduce-scatter + Adam (+ parameter all-gather) and the ZeRO-3 parameter gather over peer memory.
// Plain 16-byte loads and stores on peer mappings; no TMA, no multicast.  Neither kernel waits for anything:
// the launcher brackets them with one-thread kernels that publish and wait for flag words (ep_exchange.cu), so a
// grid never holds SMs while it waits for a peer.
#include "zero_fused.h"

#include <cuda_bf16.h>

#include "peer_sync.cuh"
#include "ptx.cuh"

namespace piper {
namespace {

constexpr int kThreads = 256;

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
    float gr = gp[k] * h.grad_scale;
    if (!h.decoupled_decay) gr += h.weight_decay * wp[k];
    mp[k] = h.beta1 * mp[k] + (1.f - h.beta1) * gr;
    vp[k] = h.beta2 * vp[k] + (1.f - h.beta2) * gr * gr;
    const float denom = sqrtf(vp[k] / h.bias_corr2) + h.eps;
    float w = wp[k] - h.lr * (mp[k] / h.bias_corr1) / denom;
    if (h.decoupled_decay) w -= h.lr * h.weight_decay * wp[k];
    wp[k] = w;
  }
}

// vectors per thread per trip; every load of a trip (peer gradients, accumulator, optimizer state) is issued
// before the first use, so one trip costs one round of memory latency, remote and local overlapped
__host__ __device__ constexpr int unroll_for(int dp, bool acc, bool fin) {
  return dp <= 2 ? (fin ? (acc ? 2 : 4) : 4) : (dp <= 4 ? ((acc && fin) ? 1 : 2) : 1);
}

__device__ __forceinline__ void store_update(const float4& w, const float4& mm, const float4& vv, float* master,
                                             float* m, float* v, float* shard_grads, __nv_bfloat16* shard_params,
                                             __nv_bfloat16* const* peer_params, int dp, long long so, long long fo,
                                             long long i) {
  reinterpret_cast<float4*>(master + so)[i] = w;
  reinterpret_cast<float4*>(m + so)[i] = mm;
  reinterpret_cast<float4*>(v + so)[i] = vv;
  if (shard_grads != nullptr) reinterpret_cast<float4*>(shard_grads + so)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  uint2 packed;
  packed.x = pack_bf16x2(w.x, w.y);
  packed.y = pack_bf16x2(w.z, w.w);
  reinterpret_cast<uint2*>(shard_params + so)[i] = packed;
  if (peer_params != nullptr)
    for (int p = 0; p < dp; ++p) reinterpret_cast<uint2*>(peer_params[p] + fo)[i] = packed;
}

// DP > 0: group size known at compile time (peer loops fully unrolled); DP == 0: any size.  ACC / FIN mirror the
// run-time flags `accumulate` / `final_step` for DP > 0 (the DP == 0 kernel reads the flags).
template <int DP, bool ACC, bool FIN>
__global__ void __launch_bounds__(kThreads, 2)
zero_reduce_kernel(const float* const* __restrict__ peer_grads, float* __restrict__ shard_grads,
                   float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                   __nv_bfloat16* __restrict__ shard_params, __nv_bfloat16* const* __restrict__ peer_params,
                   ZeroTable t, int my_rank, int dp_rt, int accumulate, int final_step, AdamHyper h,
                   uint64_t* const* __restrict__ peer_flags, int done_off, unsigned long long use,
                   unsigned int* cta_counter, const int* __restrict__ abort) {
  if (abort[0] != 0) return;
  const int dp = DP > 0 ? DP : dp_rt;
  constexpr int NP = DP > 0 ? DP : 1;
  constexpr int U = unroll_for(NP, ACC, FIN);
  const long long stride_thr = static_cast<long long>(gridDim.x) * kThreads;
  const long long first = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  for (int s = 0; s < t.n; ++s) {
    const long long piece = t.stride[s];
    long long len = t.padded[s] - static_cast<long long>(my_rank) * piece;
    len = len < 0 ? 0 : (len > piece ? piece : len);
    const long long nvec = len / 4;
    const long long fo = t.full_base[s] + static_cast<long long>(my_rank) * piece;
    const long long so = t.shard_off[s];
    if (DP > 0) {
      // per-slot base pointers in registers; a parameter has fewer than 2^31 vectors, so the trip index is 32-bit
      const float4* gsrc[NP];
      uint2* pdst[NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        gsrc[p] = reinterpret_cast<const float4*>(peer_grads[(my_rank + 1 + p) % NP] + fo);   // own copy last
        pdst[p] = (FIN && peer_params != nullptr) ? reinterpret_cast<uint2*>(peer_params[(my_rank + 1 + p) % NP] + fo)
                                                  : nullptr;
      }
      float4* own = const_cast<float4*>(gsrc[NP - 1]);
      float4* sg4 = (ACC || !FIN) ? reinterpret_cast<float4*>(shard_grads + so) : nullptr;
      float4* w4 = reinterpret_cast<float4*>(master + so);
      float4* m4 = reinterpret_cast<float4*>(m + so);
      float4* v4 = reinterpret_cast<float4*>(v + so);
      uint2* sp2 = reinterpret_cast<uint2*>(shard_params + so);
      const unsigned n32 = static_cast<unsigned>(nvec);
      const unsigned step32 = static_cast<unsigned>(stride_thr);
      for (unsigned i0 = static_cast<unsigned>(first); i0 < n32; i0 += step32 * U) {
        float4 g[U][NP], acc[ACC ? U : 1], w[FIN ? U : 1], mm[FIN ? U : 1], vv[FIN ? U : 1];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const unsigned i = i0 + u * step32;
          if (i < n32) {
#pragma unroll
            for (int p = 0; p < NP; ++p) g[u][p] = ld_stream_f4(reinterpret_cast<const float*>(gsrc[p] + i));
            if (ACC) acc[ACC ? u : 0] = ld_stream_f4(reinterpret_cast<const float*>(sg4 + i));
            if (FIN) {
              w[FIN ? u : 0] = ld_stream_f4(reinterpret_cast<const float*>(w4 + i));
              mm[FIN ? u : 0] = ld_stream_f4(reinterpret_cast<const float*>(m4 + i));
              vv[FIN ? u : 0] = ld_stream_f4(reinterpret_cast<const float*>(v4 + i));
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const unsigned i = i0 + u * step32;
          if (i >= n32) continue;
          float4 sum = g[u][0];
#pragma unroll
          for (int p = 1; p < NP; ++p) {
            sum.x += g[u][p].x; sum.y += g[u][p].y; sum.z += g[u][p].z; sum.w += g[u][p].w;
          }
          if (ACC) {
            const float4 a = acc[ACC ? u : 0];
            sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
          }
          // this rank's own copy of the piece is read by nobody else: clear it for the next accumulation
          own[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (!FIN) {
            sg4[i] = sum;
          } else {
            float4& wu = w[FIN ? u : 0];
            float4& mu = mm[FIN ? u : 0];
            float4& vu = vv[FIN ? u : 0];
            adam_vec(sum, wu, mu, vu, h);
            w4[i] = wu;
            m4[i] = mu;
            v4[i] = vu;
            if (ACC) sg4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            uint2 packed;
            packed.x = pack_bf16x2(wu.x, wu.y);
            packed.y = pack_bf16x2(wu.z, wu.w);
            sp2[i] = packed;
            if (peer_params != nullptr) {
#pragma unroll
              for (int p = 0; p < NP; ++p) pdst[p][i] = packed;
            }
          }
        }
      }
    } else {
      for (long long i = first; i < nvec; i += stride_thr) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < dp; ++p) {
          const float4 x = ld_stream_f4(peer_grads[p] + fo + 4 * i);
          sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
        }
        if (accumulate) {
          const float4 a = reinterpret_cast<const float4*>(shard_grads + so)[i];
          sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
        }
        reinterpret_cast<float4*>(const_cast<float*>(peer_grads[my_rank]) + fo)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!final_step) {
          reinterpret_cast<float4*>(shard_grads + so)[i] = sum;
          continue;
        }
        float4 w = reinterpret_cast<const float4*>(master + so)[i];
        float4 mm = reinterpret_cast<const float4*>(m + so)[i];
        float4 vv = reinterpret_cast<const float4*>(v + so)[i];
        adam_vec(sum, w, mm, vv, h);
        store_update(w, mm, vv, master, m, v, shard_grads, shard_params, peer_params, dp, so, fo, i);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < dp; ++p) st_release_sys(peer_flags[p] + done_off + my_rank, use);
    }
  }
}

// Clears the pieces of the full gradient buffer that the peers own (they have read them; this rank's own pieces
// were cleared by the reduction).  blockIdx.y = owner rank.
__global__ void __launch_bounds__(kThreads)
zero_clear_others_kernel(float* __restrict__ grads, ZeroTable t, int my_rank) {
  const int p = blockIdx.y;
  if (p == my_rank) return;
  const long long stride_thr = static_cast<long long>(gridDim.x) * kThreads;
  const long long first = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < t.n; ++s) {
    const long long piece = t.stride[s];
    long long len = t.padded[s] - static_cast<long long>(p) * piece;
    len = len < 0 ? 0 : (len > piece ? piece : len);
    float4* dst = reinterpret_cast<float4*>(grads + t.full_base[s] + static_cast<long long>(p) * piece);
#pragma unroll 4
    for (long long i = first; i < len / 4; i += stride_thr) dst[i] = z;
  }
}

// blockIdx.y = source rank.
__global__ void __launch_bounds__(kThreads)
zero_gather_kernel(const __nv_bfloat16* const* __restrict__ peer_shards, __nv_bfloat16* __restrict__ full, ZeroTable t,
                   int skip_slot, int only_slot, const int* __restrict__ abort) {
  if (abort != nullptr && abort[0] != 0) return;
  const int p = blockIdx.y;
  const __nv_bfloat16* shard = peer_shards[p];
  const long long stride_thr = static_cast<long long>(gridDim.x) * kThreads;
  const long long first = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  for (int s = 0; s < t.n; ++s) {
    if (s == skip_slot || (only_slot >= 0 && s != only_slot)) continue;
    const long long piece = t.stride[s];
    long long len = t.padded[s] - static_cast<long long>(p) * piece;
    len = len < 0 ? 0 : (len > piece ? piece : len);
    const long long nvec = len / 8;                    // 16-byte vectors of bf16
    const uint4* src = reinterpret_cast<const uint4*>(shard + t.shard_off[s]);
    uint4* dst = reinterpret_cast<uint4*>(full + t.full_base[s] + static_cast<long long>(p) * piece);
    for (long long i0 = first; i0 < nvec; i0 += stride_thr * 4) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride_thr < nvec) x[u] = src[i0 + u * stride_thr];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride_thr < nvec) dst[i0 + u * stride_thr] = x[u];
    }
  }
}

}  // namespace

int zero_reduce(const ZeroReduceArgs& a, cudaStream_t st) {
  if (a.dp < 1 || a.t.n < 0 || a.num_ctas < 1 || a.abort == nullptr) return -1;
  if (a.accumulate && a.shard_grads == nullptr) return -1;
  if (!a.final_step && a.shard_grads == nullptr) return -1;
  auto sp = static_cast<__nv_bfloat16*>(a.shard_params);
  auto pp = reinterpret_cast<__nv_bfloat16* const*>(a.peer_params);
#define PIPER_ZERO_LAUNCH_AF(DPV, ACC, FIN)                                                                      \
  zero_reduce_kernel<DPV, ACC, FIN><<<a.num_ctas, kThreads, 0, st>>>(                                            \
      a.peer_grads, a.shard_grads, a.master, a.m, a.v, sp, pp, a.t, a.my_rank, a.dp, a.accumulate, a.final_step, \
      a.h, a.peer_flags, a.done_off, a.use, a.cta_counter, a.abort)
#define PIPER_ZERO_LAUNCH(DPV)                                        \
  do {                                                                \
    if (a.accumulate && a.final_step) PIPER_ZERO_LAUNCH_AF(DPV, true, true);        \
    else if (a.accumulate) PIPER_ZERO_LAUNCH_AF(DPV, true, false);    \
    else if (a.final_step) PIPER_ZERO_LAUNCH_AF(DPV, false, true);    \
    else PIPER_ZERO_LAUNCH_AF(DPV, false, false);                     \
  } while (0)
  switch (a.dp) {
    case 1: PIPER_ZERO_LAUNCH(1); break;
    case 2: PIPER_ZERO_LAUNCH(2); break;
    case 4: PIPER_ZERO_LAUNCH(4); break;
    case 8: PIPER_ZERO_LAUNCH(8); break;
    default: PIPER_ZERO_LAUNCH_AF(0, false, false); break;
  }
#undef PIPER_ZERO_LAUNCH_AF
#undef PIPER_ZERO_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int zero_clear_others(float* grads, const ZeroTable& t, int my_rank, int dp, int num_ctas, cudaStream_t st) {
  if (dp < 1 || t.n < 0 || num_ctas < 1 || my_rank < 0 || my_rank >= dp) return -1;
  if (t.n == 0 || dp == 1) return 0;
  zero_clear_others_kernel<<<dim3(num_ctas, dp), kThreads, 0, st>>>(grads, t, my_rank);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int zero_gather(const void* const* peer_shards, void* full, const ZeroTable& t, int dp, int skip_slot, int only_slot,
                const int* abort, int num_ctas, cudaStream_t st) {
  if (dp < 1 || t.n < 0 || num_ctas < 1) return -1;
  if (t.n == 0) return 0;
  const dim3 grid(num_ctas, dp);
  zero_gather_kernel<<<grid, kThreads, 0, st>>>(reinterpret_cast<const __nv_bfloat16* const*>(peer_shards),
                                                static_cast<__nv_bfloat16*>(full), t, skip_slot, only_slot, abort);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper
