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

// ===================================================================== F3
// Expert-parallel dispatch and combine over peer memory.
//
// Every rank owns a receive buffer of ep regions (one per source rank, `cap`
// rows each).  A token's row is written straight into the region that the
// owner of its expert reserves for this source - the permutation into
// expert order and the all-to-all are one pass of peer stores, with the
// per-expert row counts and a "region complete" flag sent the same way.  The
// owner then runs its grouped GEMMs over the regions (the group table is
// built on the device from the received counts), publishes "outputs ready",
// and the token's rank gathers its k expert outputs with peer loads while
// applying the router weights: combine all-to-all and weighted sum in one
// kernel.  No host synchronisation anywhere in the exchange.

// seg_off[e]: first row of expert e inside the region this rank fills on the
// owner of e (padded prefix over that owner's experts).  Also publishes this
// rank's counts into every owner's metadata block.
__global__ void ep_prepare_kernel(const int* __restrict__ counts, int* __restrict__ seg_off,
                                  int* const* __restrict__ peer_meta, int my_rank, int ep, int experts_local) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  for (int d = 0; d < ep; ++d) {
    int run = 0;
    for (int l = 0; l < experts_local; ++l) {
      const int e = d * experts_local + l;
      seg_off[e] = run;
      run += (counts[e] + 127) / 128 * 128;
      peer_meta[d][my_rank * experts_local + l] = counts[e];
    }
  }
}

__global__ void ep_dispatch_push_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                        const int* __restrict__ counts, const int* __restrict__ seg_off,
                                        int* __restrict__ cursor, int* __restrict__ pos,
                                        __nv_bfloat16* const* __restrict__ peer_recv,
                                        uint64_t* const* __restrict__ peer_flags, unsigned int* cta_counter,
                                        int my_rank, int ep, int experts_local, long long T, int D, int k, int cap,
                                        unsigned long long epoch) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long w0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int vecs = D / 8;                      // 16-byte vectors per row
  for (long long t = w0; t < T; t += warps) {
    // lanes 0..k-1 each reserve the destination row of one of the token's k copies
    int d_l = 0, row_l = 0;
    if (lane < k) {
      const int e = idx[t * k + lane];
      d_l = e / experts_local;
      row_l = my_rank * cap + seg_off[e] + atomicAdd(cursor + e, 1);
      pos[t * k + lane] = d_l * (ep * cap) + row_l;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + t * D);
    // the row is read once (four vectors per lane per trip) and stored k times
    for (int i0 = lane; i0 < vecs; i0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + 32 * u < vecs) v[u] = src[i0 + 32 * u];
      for (int j = 0; j < k; ++j) {
        const int d = __shfl_sync(0xffffffffu, d_l, j);
        const int row = __shfl_sync(0xffffffffu, row_l, j);
        uint4* dst = reinterpret_cast<uint4*>(peer_recv[d] + static_cast<long long>(row) * D);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i0 + 32 * u < vecs) dst[i0 + 32 * u] = v[u];
      }
    }
  }
  // zero the padding rows of every segment this rank owns in the peers' regions
  const int E = ep * experts_local;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int e = blockIdx.x; e < E; e += gridDim.x) {
    const int d = e / experts_local;
    const int first = my_rank * cap + seg_off[e] + counts[e];
    const int last = my_rank * cap + seg_off[e] + (counts[e] + 127) / 128 * 128;
    uint4* base = reinterpret_cast<uint4*>(peer_recv[d] + static_cast<long long>(first) * D);
    const long long nvec = static_cast<long long>(last - first) * (D / 8);
    for (long long i = threadIdx.x; i < nvec; i += blockDim.x) base[i] = z;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < ep; ++p) st_release_sys(peer_flags[p] + my_rank, epoch);
    }
  }
}

// The same dispatch with the rows leaving through the bulk-copy engine: a warp stages a token's row in shared
// memory once and issues one bulk store (shared -> global, to local or peer memory) per destination row, two
// tokens in flight per warp.  Large stores keep the NVLink packets full and leave the SM's load/store units
// free.  Dynamic shared memory: warps_per_CTA * 2 * D * 2 bytes.
__global__ void ep_dispatch_push_bulk_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                             const int* __restrict__ counts, const int* __restrict__ seg_off,
                                             int* __restrict__ cursor, int* __restrict__ pos,
                                             __nv_bfloat16* const* __restrict__ peer_recv,
                                             uint64_t* const* __restrict__ peer_flags, unsigned int* cta_counter,
                                             int my_rank, int ep, int experts_local, long long T, int D, int k,
                                             int cap, unsigned long long epoch) {
  extern __shared__ __align__(128) uint8_t stage[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long w0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int vecs = D / 8;
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2;
  uint8_t* wbuf = stage + static_cast<size_t>(warp) * 2 * row_bytes;
  int n = 0;
  for (long long t = w0; t < T; t += warps, ++n) {
    int d_l = 0, row_l = 0;
    if (lane < k) {
      const int e = idx[t * k + lane];
      d_l = e / experts_local;
      row_l = my_rank * cap + seg_off[e] + atomicAdd(cursor + e, 1);
      pos[t * k + lane] = d_l * (ep * cap) + row_l;
    }
    uint8_t* buf = wbuf + (n & 1) * row_bytes;
    if (lane == 0) bulk_wait_group_read<1>();      // the stores of two tokens ago have read this buffer
    __syncwarp();
    const uint4* src = reinterpret_cast<const uint4*>(x + t * D);
    for (int i = lane; i < vecs; i += 32) reinterpret_cast<uint4*>(buf)[i] = src[i];
    fence_proxy_async_smem();
    __syncwarp();
    for (int j = 0; j < k; ++j) {
      const int d = __shfl_sync(0xffffffffu, d_l, j);
      const int row = __shfl_sync(0xffffffffu, row_l, j);
      if (lane == 0) {
        __nv_bfloat16* dst = peer_recv[d] + static_cast<long long>(row) * D;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                     "r"(smem_u32(buf)), "r"(row_bytes)
                     : "memory");
      }
    }
    if (lane == 0) bulk_commit_group();
  }
  if (lane == 0) {
    bulk_wait_group<0>();                          // every row has been written
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  __syncwarp();
  // zero the padding rows of every segment this rank owns in the peers' regions
  const int E = ep * experts_local;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int e = blockIdx.x; e < E; e += gridDim.x) {
    const int d = e / experts_local;
    const int first = my_rank * cap + seg_off[e] + counts[e];
    const int last = my_rank * cap + seg_off[e] + (counts[e] + 127) / 128 * 128;
    uint4* base = reinterpret_cast<uint4*>(peer_recv[d] + static_cast<long long>(first) * D);
    const long long nvec = static_cast<long long>(last - first) * (D / 8);
    for (long long i = threadIdx.x; i < nvec; i += blockDim.x) base[i] = z;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < ep; ++p) st_release_sys(peer_flags[p] + my_rank, epoch);
    }
  }
}

// Waits for every source's "region complete" flag, then builds the group
// table of the regions: group (src, l) starts at src*cap + padded prefix.
__global__ void ep_wait_table_kernel(const uint64_t* __restrict__ flags, const int* __restrict__ meta,
                                     int* __restrict__ g_start, int* __restrict__ g_len, int* __restrict__ counts_out,
                                     int ep, int experts_local, int cap, unsigned long long epoch,
                                     unsigned long long timeout_ns, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (!wait_flags(flags, ep, epoch, timeout_ns, status)) return;
  for (int s = 0; s < ep; ++s) {
    int run = s * cap;
    for (int l = 0; l < experts_local; ++l) {
      const int g = s * experts_local + l;
      const int c = meta[g];
      const int len = (c + 127) / 128 * 128;
      g_start[g] = run;
      g_len[g] = len;
      counts_out[g] = c;
      run += len;
    }
  }
}

__global__ void ep_signal_kernel(uint64_t* const* __restrict__ peer_flags, int slot0, int my_rank, int ep,
                                 unsigned long long epoch) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  __threadfence_system();
  for (int p = 0; p < ep; ++p) st_release_sys(peer_flags[p] + slot0 + my_rank, epoch);
}

// out[t] = sum_j weights[t, j] * peer_out[owner(t, j)][row(t, j)].
__global__ void ep_combine_pull_kernel(const __nv_bfloat16* const* __restrict__ peer_out, const int* __restrict__ pos,
                                       const float* __restrict__ weights, __nv_bfloat16* __restrict__ out,
                                       const uint64_t* __restrict__ out_flags, long long T, int D, int k, int ep,
                                       int cap, unsigned long long epoch, unsigned long long timeout_ns,
                                       int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = wait_flags(out_flags, ep, epoch, timeout_ns, status) ? 1 : 0;
  __syncthreads();
  if (!ok_s) return;
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long region = static_cast<long long>(ep) * cap;
  const int vecs = D / 8;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    // lanes 0..k-1 hold the location and the router weight of one expert output each
    const __nv_bfloat16* src_l = nullptr;
    float w_l = 0.f;
    if (lane < k) {
      const int p = pos[t * k + lane];
      src_l = peer_out[static_cast<int>(p / region)] + (p % region) * D;
      w_l = weights[t * k + lane];
    }
    for (int i0 = lane; i0 < vecs; i0 += 64) {
      const bool two = i0 + 32 < vecs;
      float acc[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[u][c] = 0.f;
      // four expert outputs at a time: eight 16-byte peer loads in flight per lane before the first use
      for (int j0 = 0; j0 < k; j0 += 4) {
        uint4 q[4][2];
        float w[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = j0 + jj < k ? j0 + jj : k - 1;
          const uint4* row = reinterpret_cast<const uint4*>(
              __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(src_l), j));
          w[jj] = __shfl_sync(0xffffffffu, w_l, j);
          if (j0 + jj >= k) w[jj] = 0.f;           // past the last expert: the clamped row is read but not used
          q[jj][0] = row[i0];
          q[jj][1] = two ? row[i0 + 32] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[jj][u]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float2 f = __bfloat1622float2(h[c]);
              acc[u][2 * c] += w[jj] * f.x;
              acc[u][2 * c + 1] += w[jj] * f.y;
            }
          }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && !two) break;
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int c = 0; c < 4; ++c) oh[c] = __floats2bfloat162_rn(acc[u][2 * c], acc[u][2 * c + 1]);
        reinterpret_cast<uint4*>(out + t * D)[i0 + 32 * u] = o;
      }
    }
  }
}

// The same combine with the expert outputs arriving through the bulk-copy engine: per token a warp walks the row
// in pieces of CHUNK bytes; for each piece lane 0 requests the k source pieces (from local or peer memory) into
// shared memory with k bulk loads on one mbarrier, one piece ahead of the arithmetic, and the lanes then add the
// k pieces with their router weights.  Dynamic shared memory: warps_per_CTA * 2 * k * CHUNK bytes + barriers.
constexpr int kPullChunk = 1024;      // bytes of one row piece: 16 bf16 per lane

__global__ void ep_combine_pull_bulk_kernel(const __nv_bfloat16* const* __restrict__ peer_out,
                                            const int* __restrict__ pos, const float* __restrict__ weights,
                                            __nv_bfloat16* __restrict__ out, const uint64_t* __restrict__ out_flags,
                                            long long T, int D, int k, int ep, int cap, unsigned long long epoch,
                                            unsigned long long timeout_ns, int* status) {
  extern __shared__ __align__(128) uint8_t stage[];
  __shared__ int ok_s;
  __shared__ __align__(8) uint64_t bars[16];       // two per warp (up to 8 warps)
  if (threadIdx.x == 0) ok_s = wait_flags(out_flags, ep, epoch, timeout_ns, status) ? 1 : 0;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  if (lane == 0) {
    mbar_init(&bars[2 * warp], 1);
    mbar_init(&bars[2 * warp + 1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (!ok_s) return;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long region = static_cast<long long>(ep) * cap;
  const int pieces = (D * 2 + kPullChunk - 1) / kPullChunk;        // per row
  uint8_t* wbuf = stage + static_cast<size_t>(warp) * 2 * k * kPullChunk;
  const long long w0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  // flat sequence of (token, piece) items of this warp; item i uses buffer and barrier i & 1
  long long n_items = 0;
  for (long long t = w0; t < T; t += warps) n_items += pieces;
  const __nv_bfloat16* src_l = nullptr;      // lanes 0..k-1: source row of the token being requested
  long long req_tok = -1;
  auto request = [&](long long item) {       // all lanes call; lane j < k issues the load of source j
    const long long t = w0 + (item / pieces) * warps;
    const int piece = static_cast<int>(item % pieces);
    if (t != req_tok) {
      req_tok = t;
      if (lane < k) {
        const int p = pos[t * k + lane];
        src_l = peer_out[static_cast<int>(p / region)] + (p % region) * D;
      }
    }
    const int bytes = (piece + 1) * kPullChunk <= D * 2 ? kPullChunk : D * 2 - piece * kPullChunk;
    uint64_t* bar = &bars[2 * warp + (item & 1)];
    uint8_t* buf = wbuf + (item & 1) * k * kPullChunk;
    if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(bytes) * k);
    __syncwarp();
    if (lane < k) {
      const uint8_t* src = reinterpret_cast<const uint8_t*>(src_l) + piece * kPullChunk;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(buf + lane * kPullChunk)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                   : "memory");
    }
  };
  __shared__ float wts[8][32];               // router weights of the token being summed, per warp
  long long requested = 0, done = 0;
  if (n_items > 0) { request(0); requested = 1; }
  bool ok = true;
  long long sum_tok = -1;
  for (long long item = 0; item < n_items; ++item) {
    const long long t = w0 + (item / pieces) * warps;
    const int piece = static_cast<int>(item % pieces);
    if (item + 1 < n_items) { request(item + 1); requested = item + 2; }   // one piece ahead
    if (t != sum_tok) {
      sum_tok = t;
      __syncwarp();
      if (lane < k) wts[warp][lane] = weights[t * k + lane];
      __syncwarp();
    }
    ok = __all_sync(0xffffffffu, mbar_wait(&bars[2 * warp + (item & 1)], (item >> 1) & 1, status));
    if (!ok) break;
    done = item + 1;
    const uint8_t* buf = wbuf + (item & 1) * k * kPullChunk;
    const int col = piece * (kPullChunk / 2) + lane * 16;          // first of this lane's 16 columns
    if (col < D) {
      float acc[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) acc[c] = 0.f;
      for (int j = 0; j < k; ++j) {
        const float w = wts[warp][j];
        const uint4* q = reinterpret_cast<const uint4*>(buf + j * kPullChunk + lane * 32);
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const uint4 v = q[h2];
          const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float2 f = __bfloat1622float2(hh[c]);
            acc[h2 * 8 + 2 * c] += w * f.x;
            acc[h2 * 8 + 2 * c + 1] += w * f.y;
          }
        }
      }
      uint4 o[2];
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
      for (int c = 0; c < 8; ++c) oh[c] = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
      uint4* dst = reinterpret_cast<uint4*>(out + t * D + col);
      dst[0] = o[0];
      dst[1] = o[1];
    }
    __syncwarp();      // everyone has read the buffer before it is requested again (two items later)
  }
  // after a failed wait: let the pieces that are still on their way land before the shared memory goes away
  for (long long i = done; i < requested; ++i) mbar_wait(&bars[2 * warp + (i & 1)], (i >> 1) & 1, nullptr);
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

namespace piper {

int ep_dispatch_push(const void* x, const int* idx, const int* counts, int* seg_off, int* cursor, int* pos,
                     void* const* peer_recv, int* const* peer_meta, uint64_t* const* peer_flags,
                     unsigned int* cta_counter, int my_rank, int ep, int experts_local, long long T, int D, int k,
                     int cap, unsigned long long epoch, int num_ctas, cudaStream_t st) {
  if (D % 8 != 0 || ep < 1 || experts_local < 1 || k < 1 || k > 32) return -1;
  ep_prepare_kernel<<<1, 32, 0, st>>>(counts, seg_off, peer_meta, my_rank, ep, experts_local);
  // Rows can also leave through the bulk-copy engine (PIPER_F3_BULK_PUSH=1).  Measured on a B200 pair the
  // plain-store kernel is slightly faster (peer writes top out near 400-430 GB/s either way), so it is the default.
  static int use_bulk = -1;
  if (use_bulk < 0) {
    const char* env = getenv("PIPER_F3_BULK_PUSH");
    use_bulk = (env != nullptr && env[0] == '1') ? 1 : 0;
  }
  const size_t smem = static_cast<size_t>(256 / 32) * 2 * D * 2;
  if (use_bulk && smem <= 200 * 1024) {
    static size_t configured = 0;
    if (smem > configured) {
      if (cudaFuncSetAttribute(ep_dispatch_push_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem)) != cudaSuccess)
        return -2;
      configured = smem;
    }
    ep_dispatch_push_bulk_kernel<<<num_ctas, 256, smem, st>>>(
        static_cast<const __nv_bfloat16*>(x), idx, counts, seg_off, cursor, pos,
        reinterpret_cast<__nv_bfloat16* const*>(peer_recv), peer_flags, cta_counter, my_rank, ep, experts_local, T, D,
        k, cap, epoch);
  } else {
    ep_dispatch_push_kernel<<<num_ctas, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), idx, counts, seg_off,
                                                      cursor, pos, reinterpret_cast<__nv_bfloat16* const*>(peer_recv),
                                                      peer_flags, cta_counter, my_rank, ep, experts_local, T, D, k, cap,
                                                      epoch);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ep_wait_table(const uint64_t* flags, const int* meta, int* g_start, int* g_len, int* counts_out, int ep,
                  int experts_local, int cap, unsigned long long epoch, unsigned long long timeout_ns, int* status,
                  cudaStream_t st) {
  ep_wait_table_kernel<<<1, 32, 0, st>>>(flags, meta, g_start, g_len, counts_out, ep, experts_local, cap, epoch,
                                         timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ep_signal(uint64_t* const* peer_flags, int slot0, int my_rank, int ep, unsigned long long epoch, cudaStream_t st) {
  ep_signal_kernel<<<1, 32, 0, st>>>(peer_flags, slot0, my_rank, ep, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ep_combine_pull(const void* const* peer_out, const int* pos, const float* weights, void* out,
                    const uint64_t* out_flags, long long T, int D, int k, int ep, int cap, unsigned long long epoch,
                    unsigned long long timeout_ns, int* status, int num_ctas, cudaStream_t st) {
  if (D % 8 != 0 || k < 1 || k > 32) return -1;
  // Bulk loads into shared memory are the default: on a B200 pair they pull 530 GB/s against 485 GB/s for plain
  // peer loads (PIPER_F3_BULK_PULL=0 selects the plain-load kernel).
  static int use_bulk = -1;
  if (use_bulk < 0) {
    const char* env = getenv("PIPER_F3_BULK_PULL");
    use_bulk = (env != nullptr && env[0] == '0') ? 0 : 1;
  }
  const size_t smem = static_cast<size_t>(256 / 32) * 2 * k * kPullChunk;
  if (use_bulk && smem <= 200 * 1024) {
    static size_t configured = 0;
    if (smem > configured) {
      if (cudaFuncSetAttribute(ep_combine_pull_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem)) != cudaSuccess)
        return -2;
      configured = smem;
    }
    ep_combine_pull_bulk_kernel<<<num_ctas, 256, smem, st>>>(
        reinterpret_cast<const __nv_bfloat16* const*>(peer_out), pos, weights, static_cast<__nv_bfloat16*>(out),
        out_flags, T, D, k, ep, cap, epoch, timeout_ns, status);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  }
  ep_combine_pull_kernel<<<num_ctas, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16* const*>(peer_out), pos,
                                                   weights, static_cast<__nv_bfloat16*>(out), out_flags, T, D, k, ep,
                                                   cap, epoch, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper
