// Expert-parallel token exchange over NVLink peer memory, forward and backward.
//
// Every rank of an expert-parallel group owns, per exchange slot, a receive
// buffer of `ep` regions (one per source rank, `cap_src` rows each).  The four
// transfers of one mixture-of-experts layer and microbatch are
//
//   dispatch      token owner  -> expert owner   ep_dispatch_push (gather by router index + peer stores)
//   return        expert owner -> token owner    ep_block_push    (contiguous expert segments, peer stores)
//   grad dispatch token owner  -> expert owner   ep_block_push
//   grad return   expert owner -> token owner    ep_block_push
//
// The permutation into expert order and the all-to-all are one pass of peer
// stores; the per-expert row counts travel the same way, so the host never
// learns (or waits for) a count.  The grouped GEMMs of the experts read the
// receive regions in place (the group table is built on the device by
// ep_wait_table).
//
// Synchronisation is by two kinds of flag words per buffer and peer, both
// carrying the buffer's use number:
//   READY (writer -> reader): "my rows of use u are in your buffer";
//   FREE  (reader -> writer): "I have finished reading use u of my buffer".
// A writer waits for FREE >= (use that last occupied the buffer) before its
// first store, a reader waits for READY >= u before its first load.  All
// waits are bounded (peer_sync.cuh); nothing here uses TMA or multicast.
#include "ep_exchange.h"

#include <cuda_bf16.h>

#include "peer_sync.cuh"
#include "ptx.cuh"

namespace piper {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxSegments = 2048;

// One thread: wait for the owners' FREE flags, lay out this rank's segments inside each owner's region, check the
// region capacity, publish counts and local segment starts to the owners.
//   seg_off[e]   first row of expert e inside the region this rank fills on the owner of e
//   ctl[0]       1 if the dispatch must not run (a wait ran out)
//   ctl[1 + d]   1 if the rows for owner d do not fit its region (they are not sent; status = bad argument)
__global__ void ep_prepare_kernel(const int* __restrict__ counts, const int* __restrict__ g_start_loc,
                                  int* __restrict__ seg_off, int* __restrict__ ctl, int* const* __restrict__ peer_meta,
                                  const uint64_t* __restrict__ free_flags, unsigned long long free_needed, int my_rank,
                                  int ep, int experts_local, int cap_src, unsigned long long timeout_ns, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  ctl[0] = 0;
  if (!wait_flags(free_flags, ep, free_needed, timeout_ns, status, /*tag=*/1)) {
    ctl[0] = 1;
    return;
  }
  const int G = ep * experts_local;
  for (int d = 0; d < ep; ++d) {
    int run = 0;
    for (int l = 0; l < experts_local; ++l) {
      const int e = d * experts_local + l;
      const int c = counts[e];
      seg_off[e] = run;
      if (c < 0) run = cap_src + 1; else run += (c + 127) / 128 * 128;
    }
    const bool over = run > cap_src;
    ctl[1 + d] = over ? 1 : 0;
    if (over) report_bad_argument(status, 21, d, run);
    // meta block of a slot: counts [ep * El] followed by the senders' local segment starts [ep * El]
    for (int l = 0; l < experts_local; ++l) {
      const int e = d * experts_local + l;
      peer_meta[d][my_rank * experts_local + l] = over ? 0 : counts[e];
      peer_meta[d][G + my_rank * experts_local + l] = g_start_loc[e];
    }
  }
}

__global__ void __launch_bounds__(kThreads)
ep_dispatch_push_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                        const int* __restrict__ counts, const int* __restrict__ g_start_loc,
                        const int* __restrict__ seg_off, const int* __restrict__ ctl, int* __restrict__ cursor,
                        int* __restrict__ pos_loc, __nv_bfloat16* const* __restrict__ peer_recv,
                        uint64_t* const* __restrict__ peer_flags, int ready_off, unsigned long long use,
                        unsigned int* cta_counter, int my_rank, int ep, int experts_local, long long T, int D, int k,
                        int cap_src, int* status) {
  if (ctl[0] != 0) return;
  const int E = ep * experts_local;
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long w0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int vecs = D / 8;                      // 16-byte vectors per row
  for (long long t = w0; t < T; t += warps) {
    // lanes 0..k-1 each reserve the destination row of one of the token's k copies
    int d_l = -1, row_l = 0;
    if (lane < k) {
      const int e = idx[t * k + lane];
      int p = -1;
      if (e >= 0 && e < E) {
        const int c = atomicAdd(cursor + e, 1);
        const int d = e / experts_local;
        if (c < counts[e] && ctl[1 + d] == 0) {
          d_l = d;
          row_l = my_rank * cap_src + seg_off[e] + c;
          p = g_start_loc[e] + c;
        } else if (ctl[1 + d] == 0) {
          report_bad_argument(status, 23, e, c);         // more rows for e than its count announced
        }
      } else {
        report_bad_argument(status, 22, e, t);           // expert index out of range
      }
      pos_loc[t * k + lane] = p < 0 ? 0 : p;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + t * D);
    // the row is read once (four vectors per lane per trip) and stored k times; every lane makes the same number
    // of trips, because the shuffles below need the whole warp
    for (int base = 0; base < vecs; base += 128) {
      const int i0 = base + lane;
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + 32 * u < vecs) v[u] = src[i0 + 32 * u];
      for (int j = 0; j < k; ++j) {
        const int d = __shfl_sync(0xffffffffu, d_l, j);
        const int row = __shfl_sync(0xffffffffu, row_l, j);
        if (d < 0) continue;
        uint4* dst = reinterpret_cast<uint4*>(peer_recv[d] + static_cast<long long>(row) * D);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i0 + 32 * u < vecs) dst[i0 + 32 * u] = v[u];
      }
    }
  }
  // zero the padding rows of every segment this rank owns in the peers' regions
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int e = blockIdx.x; e < E; e += gridDim.x) {
    const int d = e / experts_local;
    if (ctl[1 + d] != 0) continue;
    const int first = my_rank * cap_src + seg_off[e] + counts[e];
    const int last = my_rank * cap_src + seg_off[e] + (counts[e] + 127) / 128 * 128;
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
      for (int p = 0; p < ep; ++p) st_release_sys(peer_flags[p] + ready_off + my_rank, use);
    }
  }
}

// Owner side: wait (bounded) for every source's READY flag, then build the group table of the regions:
// group (src, l) starts at src * cap_src + padded prefix over that source's local experts.
__global__ void ep_wait_table_kernel(const uint64_t* __restrict__ ready_flags, const int* __restrict__ meta,
                                     int* __restrict__ g_start, int* __restrict__ g_len, int* __restrict__ counts_out,
                                     int ep, int experts_local, int cap_src, unsigned long long use,
                                     unsigned long long timeout_ns, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const bool ok = wait_flags(ready_flags, ep, use, timeout_ns, status, /*tag=*/2);
  for (int s = 0; s < ep; ++s) {
    int run = s * cap_src;
    for (int l = 0; l < experts_local; ++l) {
      const int g = s * experts_local + l;
      int c = ok ? meta[g] : 0;                // after a failed wait the table is empty: nothing is computed
      if (c < 0 || run + (c + 127) / 128 * 128 > (s + 1) * cap_src) c = 0;
      const int len = (c + 127) / 128 * 128;
      g_start[g] = run;
      g_len[g] = len;
      counts_out[g] = c;
      run += len;
    }
  }
}

// Copies whole segments of rows into peers' buffers.  Segment g: rows [seg_src[g], seg_src[g] + seg_len[g]) of
// `src` go to rank g / group_div, rows [seg_dst[g] + dst_bias, ...).  The launcher puts a one-thread kernel that
// waits for the destinations' FREE flags in front of this one (a grid of spinning CTAs would hold SMs that the
// kernel it is waiting for may need); abort[0] != 0 means that wait ran out.  The last CTA to finish publishes
// READY to every rank.
__global__ void __launch_bounds__(kThreads)
ep_block_push_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ seg_src,
                     const int* __restrict__ seg_len, const int* __restrict__ seg_dst, int num_segments, int group_div,
                     int dst_bias, long long src_rows, long long dst_rows, __nv_bfloat16* const* __restrict__ peer_dst,
                     uint64_t* const* __restrict__ peer_flags, const int* __restrict__ abort, int ready_off,
                     unsigned long long use, unsigned int* cta_counter, int my_rank, int ep, int D, int* status) {
  __shared__ int prefix[kMaxSegments + 1];     // chunks (of 32 rows) before segment g
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    ok_s = abort[0] == 0 ? 1 : 0;
    int run = 0;
    for (int g = 0; g < num_segments; ++g) {
      prefix[g] = run;
      int len = seg_len[g];
      const long long s0 = seg_src[g], d0 = static_cast<long long>(seg_dst[g]) + dst_bias;
      if (len < 0 || s0 < 0 || s0 + len > src_rows || d0 < 0 || d0 + len > dst_rows) {
        report_bad_argument(status, 24, g, d0 + len);   // a segment outside its buffer is not copied
        len = 0;
      }
      run += (len + 31) / 32;
    }
    prefix[num_segments] = run;
  }
  __syncthreads();
  if (!ok_s) return;
  const int total = prefix[num_segments];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = D / 8;
  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    int lo = 0, hi = num_segments;             // last g with prefix[g] <= item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= item) lo = mid; else hi = mid;
    }
    const int g = lo;
    const int r0 = (item - prefix[g]) * 32;
    const int len = min(32, seg_len[g] - r0);
    const __nv_bfloat16* s = src + (static_cast<long long>(seg_src[g]) + r0) * D;
    __nv_bfloat16* d = peer_dst[g / group_div] + (static_cast<long long>(seg_dst[g]) + dst_bias + r0) * D;
    for (int r = warp; r < len; r += kThreads / 32) {
      const uint4* sr = reinterpret_cast<const uint4*>(s + static_cast<long long>(r) * D);
      uint4* dr = reinterpret_cast<uint4*>(d + static_cast<long long>(r) * D);
      for (int i0 = lane; i0 < vecs; i0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i0 + 32 * u < vecs) v[u] = sr[i0 + 32 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i0 + 32 * u < vecs) dr[i0 + 32 * u] = v[u];
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
      for (int p = 0; p < ep; ++p) st_release_sys(peer_flags[p] + ready_off + my_rank, use);
    }
  }
}

__global__ void ep_wait_kernel(const uint64_t* __restrict__ flags, int n, unsigned long long value,
                               unsigned long long timeout_ns, int* status, int tag, int* abort) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const bool ok = wait_flags(flags, n, value, timeout_ns, status, tag);
  if (abort != nullptr) abort[0] = ok ? 0 : 1;
}

__global__ void ep_signal_kernel(uint64_t* const* __restrict__ peer_flags, int off, int my_rank, int ep,
                                 unsigned long long value) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  __threadfence_system();
  for (int p = 0; p < ep; ++p) st_release_sys(peer_flags[p] + off + my_rank, value);
}

}  // namespace

int ep_dispatch_push(const EpDispatchArgs& a, cudaStream_t st) {
  if (a.D % 8 != 0 || a.ep < 1 || a.experts_local < 1 || a.k < 1 || a.k > 32 || a.cap_src % 128 != 0) return -1;
  if (a.num_ctas < 1) return -1;
  ep_prepare_kernel<<<1, 32, 0, st>>>(a.counts, a.g_start_loc, a.seg_off, a.ctl, a.peer_meta, a.free_flags,
                                      a.free_needed, a.my_rank, a.ep, a.experts_local, a.cap_src, a.timeout_ns,
                                      a.status);
  ep_dispatch_push_kernel<<<a.num_ctas, kThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(a.x), a.idx, a.counts, a.g_start_loc, a.seg_off, a.ctl, a.cursor, a.pos_loc,
      reinterpret_cast<__nv_bfloat16* const*>(a.peer_recv), a.peer_flags, a.ready_off, a.use, a.cta_counter, a.my_rank,
      a.ep, a.experts_local, a.T, a.D, a.k, a.cap_src, a.status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ep_wait_table(const uint64_t* ready_flags, const int* meta, int* g_start, int* g_len, int* counts_out, int ep,
                  int experts_local, int cap_src, unsigned long long use, unsigned long long timeout_ns, int* status,
                  cudaStream_t st) {
  ep_wait_table_kernel<<<1, 32, 0, st>>>(ready_flags, meta, g_start, g_len, counts_out, ep, experts_local, cap_src, use,
                                         timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ep_block_push(const EpBlockPushArgs& a, cudaStream_t st) {
  if (a.D % 8 != 0 || a.ep < 1 || a.group_div < 1 || a.num_segments < 1 || a.num_segments > kMaxSegments) return -1;
  if (a.num_ctas < 1 || a.abort == nullptr) return -1;
  ep_wait_kernel<<<1, 32, 0, st>>>(a.free_flags, a.ep, a.free_needed, a.timeout_ns, a.status, /*tag=*/3, a.abort);
  ep_block_push_kernel<<<a.num_ctas, kThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(a.src), a.seg_src, a.seg_len, a.seg_dst, a.num_segments, a.group_div,
      a.dst_bias, a.src_rows, a.dst_rows, reinterpret_cast<__nv_bfloat16* const*>(a.peer_dst), a.peer_flags,
      a.abort, a.ready_off, a.use, a.cta_counter, a.my_rank, a.ep, a.D, a.status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ep_wait(const uint64_t* flags, int n, unsigned long long value, unsigned long long timeout_ns, int* status,
            int tag, int* abort, cudaStream_t st) {
  ep_wait_kernel<<<1, 32, 0, st>>>(flags, n, value, timeout_ns, status, tag, abort);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ep_signal(uint64_t* const* peer_flags, int off, int my_rank, int ep, unsigned long long value, cudaStream_t st) {
  ep_signal_kernel<<<1, 32, 0, st>>>(peer_flags, off, my_rank, ep, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper
