// Mixture-of-experts routing kernels for sm_100a: softmax + top-k router,
// scatter of token rows into zero-padded per-expert segments, weighted
// combine, and the backward passes.  One warp handles one token.
#include "moe.h"

#include "ptx.cuh"

#include <cuda_bf16.h>
#include <stdint.h>

namespace piper {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

constexpr int MAX_PER_LANE = 8;   // E <= 256
constexpr int MAX_K = 8;

// Softmax probabilities of one token, E/32 values per lane (expert e lives in
// lane e % 32, slot e / 32).
__device__ __forceinline__ void token_softmax(const __nv_bfloat16* row, int E, int lane, float (&p)[MAX_PER_LANE]) {
  float mx = -INFINITY;
#pragma unroll
  for (int s = 0; s < MAX_PER_LANE; ++s) {
    const int e = s * 32 + lane;
    p[s] = (e < E) ? __bfloat162float(row[e]) : -INFINITY;
    mx = fmaxf(mx, p[s]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int s = 0; s < MAX_PER_LANE; ++s) {
    p[s] = (s * 32 + lane < E) ? __expf(p[s] - mx) : 0.f;
    sum += p[s];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int s = 0; s < MAX_PER_LANE; ++s) p[s] *= inv;
}

__global__ void route_kernel(const __nv_bfloat16* __restrict__ logits, float* __restrict__ weights,
                             int* __restrict__ idx, int* __restrict__ counts, long long T, int E, int k,
                             int renorm) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float p[MAX_PER_LANE];
  token_softmax(logits + t * E, E, lane, p);
  float sel_w[MAX_K];
  int sel_e[MAX_K];
  float total = 0.f;
  for (int j = 0; j < k; ++j) {
    // arg-max over the remaining probabilities; ties go to the lower expert index
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int s = 0; s < MAX_PER_LANE; ++s) {
      const int e = s * 32 + lane;
      if (e < E && (p[s] > best || (p[s] == best && e < best_e))) { best = p[s]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    sel_w[j] = best;
    sel_e[j] = best_e;
    total += best;
    if ((best_e & 31) == lane) p[best_e >> 5] = -1.f;   // remove from further rounds
  }
  if (lane == 0) {
    const float scale = renorm ? 1.f / total : 1.f;
    for (int j = 0; j < k; ++j) {
      weights[t * k + j] = sel_w[j] * scale;
      idx[t * k + j] = sel_e[j];
      atomicAdd(counts + sel_e[j], 1);
    }
  }
}

// w_j = p_j / S (renorm) or p_j; dp_i for selected i, then dlogits = p * (dp - <dp, p>).
__global__ void route_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ idx,
                                 const float* __restrict__ weights, const float* __restrict__ dweights,
                                 __nv_bfloat16* __restrict__ dlogits, long long T, int E, int k, int renorm) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float p[MAX_PER_LANE], dp[MAX_PER_LANE];
  token_softmax(logits + t * E, E, lane, p);
#pragma unroll
  for (int s = 0; s < MAX_PER_LANE; ++s) dp[s] = 0.f;
  float S = 1.f, dot_w = 0.f;
  if (renorm) {
    S = 0.f;
    for (int j = 0; j < k; ++j) {
      const int e = idx[t * k + j];
      const float pe = __shfl_sync(0xffffffffu, p[e >> 5], e & 31);
      S += pe;
      dot_w += dweights[t * k + j] * weights[t * k + j];
    }
  }
  for (int j = 0; j < k; ++j) {
    const int e = idx[t * k + j];
    const float g = renorm ? (dweights[t * k + j] - dot_w) / S : dweights[t * k + j];
    if ((e & 31) == lane) dp[e >> 5] = g;
  }
  float inner = 0.f;
#pragma unroll
  for (int s = 0; s < MAX_PER_LANE; ++s) inner += dp[s] * p[s];
  inner = warp_sum(inner);
#pragma unroll
  for (int s = 0; s < MAX_PER_LANE; ++s) {
    const int e = s * 32 + lane;
    if (e < E) dlogits[t * E + e] = __float2bfloat16(p[s] * (dp[s] - inner));
  }
}

__global__ void group_table_kernel(const int* __restrict__ counts, int num_groups, int experts,
                                   const int* __restrict__ row_base, int* __restrict__ g_start,
                                   int* __restrict__ g_len, int* __restrict__ total) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int run = 0, last = 0;
  for (int g = 0; g < num_groups; ++g) {
    if (row_base != nullptr && g % experts == 0) run = row_base[g / experts];
    const int len = (counts[g] + 127) / 128 * 128;
    g_start[g] = run;
    g_len[g] = len;
    run += len;
    if (run > last) last = run;
  }
  total[0] = last;
}

struct alignas(16) vec16 { uint4 v; };

// One warp per token: claims a row per entry, copies the token row there.
__global__ void permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                               const int* __restrict__ g_start, int* __restrict__ cursor, int* __restrict__ pos,
                               __nv_bfloat16* __restrict__ rows, long long T, int D, int k, int E, long long rows_cap,
                               int* status) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + t * D);
  for (int j = 0; j < k; ++j) {
    int r = -1;
    if (lane == 0) {
      const int e = idx[t * k + j];
      if (e >= 0 && e < E) r = g_start[e] + atomicAdd(cursor + e, 1);
      if (r < 0 || r >= rows_cap) {             // rejected: recorded, the copy is skipped
        report_bad_argument(status, 31, e, r);
        r = -1;
      }
      pos[t * k + j] = r < 0 ? 0 : r;
    }
    r = __shfl_sync(0xffffffffu, r, 0);
    if (r < 0) continue;
    uint4* dst = reinterpret_cast<uint4*>(rows + static_cast<long long>(r) * D);
    for (int i = lane; i < D / 8; i += 32) dst[i] = src[i];
  }
}

// Zeroes rows [g_start + counts, g_start + g_len) of every group.
__global__ void zero_padding_kernel(__nv_bfloat16* __restrict__ rows, const int* __restrict__ g_start,
                                    const int* __restrict__ g_len, const int* __restrict__ counts, int D,
                                    long long rows_cap, int* status) {
  const int g = blockIdx.x;
  const int first = g_start[g] + counts[g];
  const int last = g_start[g] + g_len[g];
  if (counts[g] < 0 || g_start[g] < 0 || last < first || last > rows_cap) {
    if (threadIdx.x == 0) report_bad_argument(status, 35, g, last);
    return;                                   // a segment outside the buffer is left alone
  }
  const uint4 z = make_uint4(0, 0, 0, 0);
  const long long nvec = static_cast<long long>(last - first) * (D / 8);
  uint4* base = reinterpret_cast<uint4*>(rows + static_cast<long long>(first) * D);
  for (long long i = threadIdx.x; i < nvec; i += blockDim.x) base[i] = z;
}

__global__ void permute_bwd_kernel(const __nv_bfloat16* __restrict__ drows, const int* __restrict__ pos,
                                   __nv_bfloat16* __restrict__ dx, long long T, int D, int k, long long rows_cap,
                                   int* status) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const long long r = pos[t * k + j];
      if (r < 0 || r >= rows_cap) {             // a row outside the buffer contributes nothing
        report_bad_argument(status, 32, t, r);
        continue;
      }
      const uint4 q = reinterpret_cast<const uint4*>(drows + r * D)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 f = __bfloat1622float2(h[c]);
        acc[2 * c] += f.x;
        acc[2 * c + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int c = 0; c < 4; ++c) oh[c] = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
    reinterpret_cast<uint4*>(dx + t * D)[i] = o;
  }
}

__global__ void combine_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ pos,
                               const float* __restrict__ weights, __nv_bfloat16* __restrict__ out, long long T,
                               int D, int k, long long rows_cap, int* status) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const float w = weights[t * k + j];
      const long long r = pos[t * k + j];
      if (r < 0 || r >= rows_cap) {
        report_bad_argument(status, 33, t, r);
        continue;
      }
      const uint4 q = reinterpret_cast<const uint4*>(rows + r * D)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 f = __bfloat1622float2(h[c]);
        acc[2 * c] += w * f.x;
        acc[2 * c + 1] += w * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int c = 0; c < 4; ++c) oh[c] = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
    reinterpret_cast<uint4*>(out + t * D)[i] = o;
  }
}

__global__ void combine_bwd_kernel(const __nv_bfloat16* __restrict__ rows, const __nv_bfloat16* __restrict__ dout,
                                   const int* __restrict__ pos, const float* __restrict__ weights,
                                   __nv_bfloat16* __restrict__ drows, float* __restrict__ dweights, long long T,
                                   int D, int k, long long rows_cap, int* status) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int j = 0; j < k; ++j) {
    const float w = weights[t * k + j];
    const long long r = pos[t * k + j];
    if (r < 0 || r >= rows_cap) {
      if (lane == 0) {
        report_bad_argument(status, 34, t, r);
        dweights[t * k + j] = 0.f;
      }
      continue;
    }
    float dot = 0.f;
    for (int i = lane; i < D / 8; i += 32) {
      const uint4 g = reinterpret_cast<const uint4*>(dout + t * D)[i];
      const uint4 q = reinterpret_cast<const uint4*>(rows + r * D)[i];
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
      const __nv_bfloat162* qh = reinterpret_cast<const __nv_bfloat162*>(&q);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 gf = __bfloat1622float2(gh[c]);
        const float2 qf = __bfloat1622float2(qh[c]);
        dot += gf.x * qf.x + gf.y * qf.y;
        oh[c] = __floats2bfloat162_rn(w * gf.x, w * gf.y);
      }
      reinterpret_cast<uint4*>(drows + r * D)[i] = o;
    }
    dot = warp_sum(dot);
    if (lane == 0) dweights[t * k + j] = dot;
  }
}

inline unsigned warps_grid(long long warps, int threads) {
  return static_cast<unsigned>((warps * 32 + threads - 1) / threads);
}

}  // namespace

#define PIPER_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -3)

int moe_route(const void* logits, float* weights, int* idx, int* counts, long long T, int E, int k, int renorm,
              cudaStream_t st) {
  if (E > 32 * MAX_PER_LANE || k > MAX_K || k > E || k < 1) return -1;
  if (T == 0) return 0;
  route_kernel<<<warps_grid(T, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), weights, idx, counts,
                                                   T, E, k, renorm);
  return PIPER_LAUNCH_OK();
}

int moe_route_bwd(const void* logits, const int* idx, const float* weights, const float* dweights, void* dlogits,
                  long long T, int E, int k, int renorm, cudaStream_t st) {
  if (E > 32 * MAX_PER_LANE || k > MAX_K) return -1;
  if (T == 0) return 0;
  route_bwd_kernel<<<warps_grid(T, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), idx, weights,
                                                       dweights, static_cast<__nv_bfloat16*>(dlogits), T, E, k,
                                                       renorm);
  return PIPER_LAUNCH_OK();
}

int moe_group_table(const int* counts, int num_groups, int experts, const int* row_base, int* g_start, int* g_len,
                    int* total, cudaStream_t st) {
  if (num_groups <= 0 || experts <= 0) return -1;
  group_table_kernel<<<1, 32, 0, st>>>(counts, num_groups, experts, row_base, g_start, g_len, total);
  return PIPER_LAUNCH_OK();
}

int moe_permute(const void* x, const int* idx, const int* g_start, const int* g_len, const int* counts, int* cursor,
                int* pos, void* rows, long long T, int D, int E, int k, long long rows_cap, int* status,
                cudaStream_t st) {
  if (D % 8 != 0) return -1;
  if (T > 0)
    permute_kernel<<<warps_grid(T, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), idx, g_start, cursor,
                                                       pos, static_cast<__nv_bfloat16*>(rows), T, D, k, E, rows_cap,
                                                       status);
  zero_padding_kernel<<<E, 256, 0, st>>>(static_cast<__nv_bfloat16*>(rows), g_start, g_len, counts, D, rows_cap, status);
  return PIPER_LAUNCH_OK();
}

int moe_permute_bwd(const void* drows, const int* pos, void* dx, long long T, int D, int k, long long rows_cap,
                    int* status, cudaStream_t st) {
  if (D % 8 != 0) return -1;
  if (T == 0) return 0;
  permute_bwd_kernel<<<warps_grid(T, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(drows), pos,
                                                         static_cast<__nv_bfloat16*>(dx), T, D, k, rows_cap, status);
  return PIPER_LAUNCH_OK();
}

int moe_combine(const void* rows, const int* pos, const float* weights, void* out, long long T, int D, int k,
                long long rows_cap, int* status, cudaStream_t st) {
  if (D % 8 != 0) return -1;
  if (T == 0) return 0;
  combine_kernel<<<warps_grid(T, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows), pos, weights,
                                                     static_cast<__nv_bfloat16*>(out), T, D, k, rows_cap, status);
  return PIPER_LAUNCH_OK();
}

int moe_combine_bwd(const void* rows, const void* dout, const int* pos, const float* weights, void* drows,
                    float* dweights, const int* g_start, const int* g_len, const int* counts, int num_groups,
                    long long T, int D, int k, long long rows_cap, int* status, cudaStream_t st) {
  if (D % 8 != 0) return -1;
  if (T > 0)
    combine_bwd_kernel<<<warps_grid(T, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows),
                                                           static_cast<const __nv_bfloat16*>(dout), pos, weights,
                                                           static_cast<__nv_bfloat16*>(drows), dweights, T, D, k,
                                                           rows_cap, status);
  zero_padding_kernel<<<num_groups, 256, 0, st>>>(static_cast<__nv_bfloat16*>(drows), g_start, g_len, counts, D,
                                                  rows_cap, status);
  return PIPER_LAUNCH_OK();
}

}  // namespace piper
