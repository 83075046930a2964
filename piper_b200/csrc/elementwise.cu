// Memory-bound kernels of the transformer block for sm_100a: RMSNorm
// (optionally fused with the residual add), QK-norm + RoPE on the packed QKV
// projection, SwiGLU, embedding gather / scatter-add, row-wise cross-entropy
// with in-place gradient, and the flat-buffer Adam update.  All of them move
// 16-byte vectors and keep fp32 math in registers; none allocates.
#include "elementwise.h"

#include "ptx.cuh"

#include <cuda_bf16.h>
#include <stdint.h>

namespace piper {
namespace {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

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

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) scratch[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? scratch[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* scratch) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) scratch[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? scratch[threadIdx.x] : -INFINITY;
  if (w == 0) {
    t = warp_max(t);
    if (l == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

// ------------------------------------------------------------------ RMSNorm
// One CTA per row.  Optional residual: h = x + res is written to h_out and
// normalised, so the block's "x = x + f(norm(x))" costs one pass.
constexpr int NORM_THREADS = 256;

__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd, int D, float eps) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
  const bf16x8* rr = res ? reinterpret_cast<const bf16x8*>(res + row * D) : nullptr;
  bf16x8* hr = h_out ? reinterpret_cast<bf16x8*>(h_out + row * D) : nullptr;
  const int nvec = D / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += NORM_THREADS) {
    float f[8];
    unpack8(xr[i], f);
    if (rr) {
      float g[8];
      unpack8(rr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      // Round the residual stream to bf16 before it is normalised, so that
      // forward and backward see the same values.
      const bf16x8 hp = pack8(f);
      hr[i] = hp;
      unpack8(hp, f);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum<NORM_THREADS>(ss, scratch);
  const float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0) rstd[row] = r;
  const bf16x8* src = rr ? reinterpret_cast<const bf16x8*>(h_out + row * D) : xr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * D);
  for (int i = threadIdx.x; i < nvec; i += NORM_THREADS) {
    float f[8], g[8];
    unpack8(src[i], f);
    unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * r * g[j];
    yr[i] = pack8(f);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)), plus an optional pass-through
// gradient dres added to dx (the residual branch).  Column sums of dy*xhat
// go to dw_partial[blockIdx.x][D]; a second kernel reduces them in a fixed
// order, so the weight gradient is reproducible.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int D) {
  extern __shared__ float dw_acc[];   // D floats
  __shared__ float scratch[32];
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) dw_acc[i] = 0.f;
  __syncthreads();
  const int nvec = D / 8;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * D);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = threadIdx.x; i < nvec; i += NORM_THREADS) {
      float a[8], b[8], g[8];
      unpack8(dyr[i], a);
      unpack8(xr[i], b);
      unpack8(wr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * g[j] * b[j] * r;
    }
    dot = block_sum<NORM_THREADS>(dot, scratch) / D;
    const bf16x8* drr = dres ? reinterpret_cast<const bf16x8*>(dres + row * D) : nullptr;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * D);
    for (int i = threadIdx.x; i < nvec; i += NORM_THREADS) {
      float a[8], b[8], g[8], o[8];
      unpack8(dyr[i], a);
      unpack8(xr[i], b);
      unpack8(wr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = b[j] * r;
        o[j] = r * (a[j] * g[j] - xhat * dot);
        dw_acc[i * 8 + j] += a[j] * xhat;   // column owned by this thread
      }
      if (drr) {
        float e[8];
        unpack8(drr[i], e);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += e[j];
      }
      dxr[i] = pack8(o);
    }
  }
  __syncthreads();
  float* out = dw_partial + static_cast<long long>(blockIdx.x) * D;
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) out[i] = dw_acc[i];
}

// Register-resident variants for D == VPT * 8 * NORM_THREADS (2048, 4096, 8192): every thread owns VPT
// 8-element vectors of the row, so the row is read from memory exactly once and the block reduction needs a
// single barrier (the per-warp sums alternate between two scratch rows; a thread can only reach the write of
// row k+2 after every thread has passed the barrier of row k+1, i.e. after all reads of row k).
__device__ __forceinline__ float block_sum_once(float v, float (*scratch)[NORM_THREADS / 32], int parity) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) scratch[parity][threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; ++i) t += scratch[parity][i];
  return t;
}

template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                       __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd, float eps) {
  constexpr int D = VPT * 8 * NORM_THREADS;
  __shared__ float scratch[2][NORM_THREADS / 32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * D);
  bf16x8 xv[VPT], rv[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) xv[v] = xr[threadIdx.x + v * NORM_THREADS];
  if (res) {
    const bf16x8* rr = reinterpret_cast<const bf16x8*>(res + row * D);
#pragma unroll
    for (int v = 0; v < VPT; ++v) rv[v] = rr[threadIdx.x + v * NORM_THREADS];
  }
  float f[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    unpack8(xv[v], f[v]);
    if (res) {
      float g[8];
      unpack8(rv[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[v][j] += g[j];
      const bf16x8 hp = pack8(f[v]);   // the residual stream is bf16: normalise what is stored
      reinterpret_cast<bf16x8*>(h_out + row * D)[threadIdx.x + v * NORM_THREADS] = hp;
      unpack8(hp, f[v]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[v][j] * f[v][j];
  }
  ss = block_sum_once(ss, scratch, 0);
  const float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0) rstd[row] = r;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * D);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    float g[8];
    unpack8(wr[threadIdx.x + v * NORM_THREADS], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[v][j] = f[v][j] * r * g[j];
    yr[threadIdx.x + v * NORM_THREADS] = pack8(f[v]);
  }
}

// Two CTAs per SM (one for 8192-wide rows): the row vectors stay packed (bf16) in registers and are unpacked where they are used, which
// keeps the kernel under 128 registers with the next row's loads in flight.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS, VPT <= 2 ? 2 : 1)
rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, int T) {
  constexpr int D = VPT * 8 * NORM_THREADS;
  __shared__ float scratch[2][NORM_THREADS / 32];
  bf16x8 gw[VPT];
  float dw[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    gw[v] = reinterpret_cast<const bf16x8*>(w)[threadIdx.x + v * NORM_THREADS];
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[v][j] = 0.f;
  }
  // The next row's vectors are fetched before the current row is reduced, so the loads overlap the barrier.
  bf16x8 na[VPT], nb[VPT], ne[VPT];
  float nr = 0.f;
  long long row = blockIdx.x;
  auto fetch = [&](long long rw) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + rw * D);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + rw * D);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      na[v] = dyr[threadIdx.x + v * NORM_THREADS];
      nb[v] = xr[threadIdx.x + v * NORM_THREADS];
    }
    if (dres) {
      const bf16x8* er = reinterpret_cast<const bf16x8*>(dres + rw * D);
#pragma unroll
      for (int v = 0; v < VPT; ++v) ne[v] = er[threadIdx.x + v * NORM_THREADS];
    }
    nr = rstd[rw];
  };
  if (row < T) fetch(row);
  int parity = 0;
  for (; row < T; row += gridDim.x, parity ^= 1) {
    bf16x8 ca[VPT], cb[VPT], ce[VPT];
    const float r = nr;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      ca[v] = na[v];
      cb[v] = nb[v];
      if (dres) ce[v] = ne[v];
    }
    if (row + gridDim.x < T) fetch(row + gridDim.x);
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float a[8], b[8], g[8];
      unpack8(ca[v], a);
      unpack8(cb[v], b);
      unpack8(gw[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * g[j] * (b[j] * r);
    }
    dot = block_sum_once(dot, scratch, parity) / D;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * D);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float a[8], b[8], g[8], o[8];
      unpack8(ca[v], a);
      unpack8(cb[v], b);
      unpack8(gw[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = b[j] * r;
        o[j] = r * (a[j] * g[j] - xhat * dot);
        dw[v][j] += a[j] * xhat;
      }
      if (dres) {
        float e[8];
        unpack8(ce[v], e);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += e[j];
      }
      dxr[threadIdx.x + v * NORM_THREADS] = pack8(o);
    }
  }
  float* out = dw_partial + static_cast<long long>(blockIdx.x) * D;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    float4* o4 = reinterpret_cast<float4*>(out + (threadIdx.x + v * NORM_THREADS) * 8);
    o4[0] = make_float4(dw[v][0], dw[v][1], dw[v][2], dw[v][3]);
    o4[1] = make_float4(dw[v][4], dw[v][5], dw[v][6], dw[v][7]);
  }
}

// dw[c] (+)= sum_b partial[b][c]; fp32 output (the flat gradient bucket) or
// bf16 when dw_bf16 is given.  A block owns 32 columns; its 32 thread rows each
// sum a contiguous slice of the partials and the slices are added in a fixed
// order, so the result does not depend on timing.
constexpr int RED_SLICES = 32;
__global__ void __launch_bounds__(32 * RED_SLICES)
reduce_partials_kernel(const float* __restrict__ partial, int nblocks, int D,
                       float* __restrict__ dw_f32, __nv_bfloat16* __restrict__ dw_bf16,
                       int accumulate) {
  __shared__ float part[RED_SLICES][32];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int per = (nblocks + RED_SLICES - 1) / RED_SLICES;
  const int b0 = threadIdx.y * per;
  const int b1 = min(nblocks, b0 + per);
  float s = 0.f;
  if (c < D) {
#pragma unroll 4
    for (int b = b0; b < b1; ++b) s += partial[static_cast<long long>(b) * D + c];
  }
  part[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y != 0 || c >= D) return;
  s = 0.f;
#pragma unroll
  for (int i = 0; i < RED_SLICES; ++i) s += part[i][threadIdx.x];
  if (dw_f32) dw_f32[c] = accumulate ? dw_f32[c] + s : s;
  if (dw_bf16) dw_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(dw_bf16[c]) + s : s);
}

// --------------------------------------------------------- QK-norm + RoPE
// qkv is the packed projection [T, (Hq + 2*Hkv) * hd], hd = 128 or 64; v heads are copied.
// rope pairs: interleaved (x[2i], x[2i+1]) or half-split (x[i], x[i+hd/2]).
// cos/sin are fp32 [S, hd/2]; position of token t is t % S.
//
// A group of hd/16 lanes handles one (token, head) vector.  Every lane owns two 16-byte vectors chosen so
// that both members of each of its eight rope pairs are its own: elements [16l, 16l+16) in the interleaved
// form, [8l, 8l+8) and [hd/2 + 8l, hd/2 + 8l + 8) in the half-split form.  In both forms the lane's pairs use
// cos/sin entries [8l, 8l+8).
// A lane group walks this many consecutive heads of one token, so the token's cos/sin entries are loaded once.
constexpr int ROPE_HEADS_PER_GROUP = 8;

template <int HD>
struct RopeGroup {
  static constexpr int LANES = HD / 16;
  int lane, off0, off1;
  unsigned mask;
  __device__ __forceinline__ RopeGroup(int interleaved) {
    const int wl = threadIdx.x & 31;
    lane = wl & (LANES - 1);
    mask = ((LANES == 32 ? 0u : (1u << LANES)) - 1u) << (wl & ~(LANES - 1));
    off0 = interleaved ? 16 * lane : 8 * lane;
    off1 = interleaved ? 16 * lane + 8 : HD / 2 + 8 * lane;
  }
  __device__ __forceinline__ float sum(float v) const {
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
    return v;
  }
};

// (a, b) -> (a*c - b*s, a*s + b*c) on the lane's eight pairs.
__device__ __forceinline__ void rope_rotate(float (&v0)[8], float (&v1)[8], const float (&c)[8], const float (&s)[8],
                                            int interleaved) {
  if (interleaved) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float a0 = v0[2 * p], b0 = v0[2 * p + 1], a1 = v1[2 * p], b1 = v1[2 * p + 1];
      v0[2 * p] = a0 * c[p] - b0 * s[p];
      v0[2 * p + 1] = a0 * s[p] + b0 * c[p];
      v1[2 * p] = a1 * c[4 + p] - b1 * s[4 + p];
      v1[2 * p + 1] = a1 * s[4 + p] + b1 * c[4 + p];
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = v0[j], b = v1[j];
      v0[j] = a * c[j] - b * s[j];
      v1[j] = a * s[j] + b * c[j];
    }
  }
}

__device__ __forceinline__ void load8f(const float* p, float (&f)[8], float scale) {
  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
  f[0] = lo.x * scale; f[1] = lo.y * scale; f[2] = lo.z * scale; f[3] = lo.w * scale;
  f[4] = hi.x * scale; f[5] = hi.y * scale; f[6] = hi.z * scale; f[7] = hi.w * scale;
}

template <int HD>
__global__ void __launch_bounds__(256)
qk_rope_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
               const float* __restrict__ cosp, const float* __restrict__ sinp,
               const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
               float* __restrict__ rstd_out, long long T, int S, int Hq, int Hkv,
               int interleaved, float eps, float sin_sign) {
  const RopeGroup<HD> g(interleaved);
  constexpr int LANES = RopeGroup<HD>::LANES;
  const int heads = Hq + 2 * Hkv;
  const int chunks = (heads + ROPE_HEADS_PER_GROUP - 1) / ROPE_HEADS_PER_GROUP;
  const unsigned total = static_cast<unsigned>(T) * chunks;   // the launcher keeps this below 2^31
  const unsigned stride = gridDim.x * (blockDim.x / LANES);
  for (unsigned gi = blockIdx.x * (blockDim.x / LANES) + threadIdx.x / LANES; gi < total; gi += stride) {
    const long long t = gi / static_cast<unsigned>(chunks);
    const int h0 = static_cast<int>(gi - static_cast<unsigned>(t) * chunks) * ROPE_HEADS_PER_GROUP;
    const int h1 = min(heads, h0 + ROPE_HEADS_PER_GROUP);
    float c[8], s[8];
    const int cs = static_cast<int>(static_cast<unsigned>(t) % static_cast<unsigned>(S)) * (HD / 2) + 8 * g.lane;
    load8f(cosp + cs, c, 1.f);
    load8f(sinp + cs, s, sin_sign);
#pragma unroll 4
    for (int h = h0; h < h1; ++h) {
      const __nv_bfloat16* src = in + (t * heads + h) * HD;
      __nv_bfloat16* dst = out + (t * heads + h) * HD;
      const bf16x8 p0 = *reinterpret_cast<const bf16x8*>(src + g.off0);
      const bf16x8 p1 = *reinterpret_cast<const bf16x8*>(src + g.off1);
      if (h >= Hq + Hkv) {   // value head: plain copy
        *reinterpret_cast<bf16x8*>(dst + g.off0) = p0;
        *reinterpret_cast<bf16x8*>(dst + g.off1) = p1;
        continue;
      }
      float v0[8], v1[8];
      unpack8(p0, v0);
      unpack8(p1, v1);
      const __nv_bfloat16* nw = (h < Hq) ? qw : kw;
      if (nw != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v0[j] * v0[j] + v1[j] * v1[j];
        ss = g.sum(ss);
        const float r = rsqrtf(ss / HD + eps);
        if (rstd_out != nullptr && g.lane == 0) rstd_out[t * (Hq + Hkv) + h] = r;
        float w0[8], w1[8];
        unpack8(*reinterpret_cast<const bf16x8*>(nw + g.off0), w0);
        unpack8(*reinterpret_cast<const bf16x8*>(nw + g.off1), w1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v0[j] = v0[j] * r * w0[j];
          v1[j] = v1[j] * r * w1[j];
        }
      }
      rope_rotate(v0, v1, c, s, interleaved);
      *reinterpret_cast<bf16x8*>(dst + g.off0) = pack8(v0);
      *reinterpret_cast<bf16x8*>(dst + g.off1) = pack8(v1);
    }
  }
}

// Backward of QK-norm + RoPE: un-rotate the incoming gradient (RoPE is an
// orthogonal map, so its transpose is the rotation by -theta), then apply the
// RMSNorm backward per head.  Weight-gradient contributions are summed in
// shared memory per CTA and added to fp32 dqw/dkw with one atomic per element
// and CTA.
template <int HD>
__global__ void __launch_bounds__(256)
qk_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ in /*pre-norm qkv*/,
                   __nv_bfloat16* __restrict__ din, const float* __restrict__ cosp,
                   const float* __restrict__ sinp, const __nv_bfloat16* __restrict__ qw,
                   const __nv_bfloat16* __restrict__ kw, float* __restrict__ dqw,
                   float* __restrict__ dkw, long long T, int S, int Hq, int Hkv,
                   int interleaved, float eps) {
  __shared__ float sdw[2][HD];
  const bool want_dw = dqw != nullptr || dkw != nullptr;
  if (want_dw) {
    for (int i = threadIdx.x; i < 2 * HD; i += blockDim.x) (&sdw[0][0])[i] = 0.f;
    __syncthreads();
  }
  const RopeGroup<HD> g(interleaved);
  constexpr int LANES = RopeGroup<HD>::LANES;
  const int heads = Hq + 2 * Hkv;
  const int chunks = (heads + ROPE_HEADS_PER_GROUP - 1) / ROPE_HEADS_PER_GROUP;
  const unsigned total = static_cast<unsigned>(T) * chunks;   // the launcher keeps this below 2^31
  const unsigned stride = gridDim.x * (blockDim.x / LANES);
  for (unsigned gi = blockIdx.x * (blockDim.x / LANES) + threadIdx.x / LANES; gi < total; gi += stride) {
    const long long t = gi / static_cast<unsigned>(chunks);
    const int h0 = static_cast<int>(gi - static_cast<unsigned>(t) * chunks) * ROPE_HEADS_PER_GROUP;
    const int h1 = min(heads, h0 + ROPE_HEADS_PER_GROUP);
    float c[8], s[8];
    const int cs = static_cast<int>(static_cast<unsigned>(t) % static_cast<unsigned>(S)) * (HD / 2) + 8 * g.lane;
    load8f(cosp + cs, c, 1.f);
    load8f(sinp + cs, s, -1.f);
#pragma unroll 4
    for (int h = h0; h < h1; ++h) {
      const __nv_bfloat16* gp = dout + (t * heads + h) * HD;
      __nv_bfloat16* dst = din + (t * heads + h) * HD;
      const bf16x8 p0 = *reinterpret_cast<const bf16x8*>(gp + g.off0);
      const bf16x8 p1 = *reinterpret_cast<const bf16x8*>(gp + g.off1);
      if (h >= Hq + Hkv) {
        *reinterpret_cast<bf16x8*>(dst + g.off0) = p0;
        *reinterpret_cast<bf16x8*>(dst + g.off1) = p1;
        continue;
      }
      float d0[8], d1[8];
      unpack8(p0, d0);
      unpack8(p1, d1);
      rope_rotate(d0, d1, c, s, interleaved);
      const __nv_bfloat16* nw = (h < Hq) ? qw : kw;
      if (nw != nullptr) {
        const __nv_bfloat16* src = in + (t * heads + h) * HD;
        float x0[8], x1[8], w0[8], w1[8];
        unpack8(*reinterpret_cast<const bf16x8*>(src + g.off0), x0);
        unpack8(*reinterpret_cast<const bf16x8*>(src + g.off1), x1);
        unpack8(*reinterpret_cast<const bf16x8*>(nw + g.off0), w0);
        unpack8(*reinterpret_cast<const bf16x8*>(nw + g.off1), w1);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x0[j] * x0[j] + x1[j] * x1[j];
        ss = g.sum(ss);
        const float r = rsqrtf(ss / HD + eps);
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += (d0[j] * w0[j] * x0[j] + d1[j] * w1[j] * x1[j]) * r;
        dot = g.sum(dot) / HD;
        float* acc = sdw[h < Hq ? 0 : 1];
        const bool add = (h < Hq ? dqw : dkw) != nullptr;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh0 = x0[j] * r, xh1 = x1[j] * r;
          if (add) {
            atomicAdd(acc + g.off0 + j, d0[j] * xh0);
            atomicAdd(acc + g.off1 + j, d1[j] * xh1);
          }
          d0[j] = r * (d0[j] * w0[j] - xh0 * dot);
          d1[j] = r * (d1[j] * w1[j] - xh1 * dot);
        }
      }
      *reinterpret_cast<bf16x8*>(dst + g.off0) = pack8(d0);
      *reinterpret_cast<bf16x8*>(dst + g.off1) = pack8(d1);
    }
  }
  if (want_dw) {
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * HD; i += blockDim.x) {
      float* dwp = i < HD ? dqw : dkw;
      const float v = (&sdw[0][0])[i];
      if (dwp != nullptr && v != 0.f) atomicAdd(dwp + (i < HD ? i : i - HD), v);
    }
  }
}

// ------------------------------------------------------------------- SwiGLU
// h13 = [gate | up] of width 2F per row; act = silu(gate) * up.
// Threads walk the flattened [T][F/8] vector index with a grid stride; row and column advance incrementally
// (stride_rows, stride_cols = stride / (F/8), stride % (F/8) come from the host), so the loop has no division.
struct VecWalk {
  long long row;
  int c;
  __device__ __forceinline__ VecWalk(int vecs) {
    const long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    row = i0 / vecs;
    c = static_cast<int>(i0 - row * vecs);
  }
  __device__ __forceinline__ void next(int vecs, int stride_rows, int stride_cols) {
    row += stride_rows;
    c += stride_cols;
    if (c >= vecs) {
      c -= vecs;
      ++row;
    }
  }
};

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ h13, __nv_bfloat16* __restrict__ act, long long T, int F,
                  int stride_rows, int stride_cols) {
  const int vecs = F / 8;
  for (VecWalk w(vecs); w.row < T; w.next(vecs, stride_rows, stride_cols)) {
    const bf16x8* base = reinterpret_cast<const bf16x8*>(h13 + w.row * 2 * F);
    float g[8], u[8], o[8];
    unpack8(base[w.c], g);
    unpack8(base[vecs + w.c], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<bf16x8*>(act + w.row * F)[w.c] = pack8(o);
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ h13, const __nv_bfloat16* __restrict__ dact,
                  __nv_bfloat16* __restrict__ dh13, long long T, int F, int stride_rows, int stride_cols) {
  const int vecs = F / 8;
  for (VecWalk w(vecs); w.row < T; w.next(vecs, stride_rows, stride_cols)) {
    const bf16x8* base = reinterpret_cast<const bf16x8*>(h13 + w.row * 2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(base[w.c], g);
    unpack8(base[vecs + w.c], u);
    unpack8(reinterpret_cast<const bf16x8*>(dact + w.row * F)[w.c], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
    }
    bf16x8* ob = reinterpret_cast<bf16x8*>(dh13 + w.row * 2 * F);
    ob[w.c] = pack8(dg);
    ob[vecs + w.c] = pack8(du);
  }
}

// ---------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ tokens,
                                     const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ out,
                                     long long T, int D, int V, int* status) {
  const long long row = blockIdx.x;
  long long tok = tokens[row];
  if (tok < 0 || tok >= V) {   // recorded, not trapped
    if (threadIdx.x == 0) report_bad_argument(status, 41, row, tok);
    tok = 0;
  }
  const bf16x8* src = reinterpret_cast<const bf16x8*>(table + tok * D);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + row * D);
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
}

// dtable[tok] += dout[row]; fp32 atomics straight into the gradient bucket.
__global__ void embedding_bwd_kernel(const long long* __restrict__ tokens,
                                     const __nv_bfloat16* __restrict__ dout, float* __restrict__ dtable,
                                     long long T, int D, int V) {
  const long long row = blockIdx.x;
  const long long tok = tokens[row];
  if (tok < 0 || tok >= V) return;
  const __nv_bfloat16* src = dout + row * D;
  float* dst = dtable + tok * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(dst + i, __bfloat162float(src[i]));
}

// ------------------------------------------------------------ cross-entropy
// One CTA per row of bf16 logits [T, V]: online max / sum-exp, per-token loss
// and log-sum-exp.  ignore_index rows produce loss 0.
constexpr int CE_THREADS = 512;

__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
              float* __restrict__ loss, float* __restrict__ lse, int V, long long ld,
              long long ignore_index) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(lr)[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    const float f = __bfloat162float(lr[i]);
    if (f > m) {
      s *= __expf(m - f);
      m = f;
    }
    s += __expf(f - m);
  }
  const float gm = block_max<CE_THREADS>(m, scratch);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<CE_THREADS>(s, scratch);
  if (threadIdx.x == 0) {
    const float l = gm + logf(gs);
    lse[row] = l;
    const long long y = labels[row];
    loss[row] = (y == ignore_index || y < 0 || y >= V) ? 0.f : l - __bfloat162float(lr[y]);
  }
}

// dlogits = (softmax - onehot) * gscale[0] * row_scale, written to `out`
// (may alias logits).
__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
              const float* __restrict__ lse, const float* __restrict__ gscale, float row_scale,
              __nv_bfloat16* __restrict__ out, int V, long long ld, long long ignore_index) {
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  __nv_bfloat16* orow = out + row * ld;
  const long long y = labels[row];
  const bool ignored = (y == ignore_index || y < 0 || y >= V);
  const float sc = ignored ? 0.f : gscale[0] * row_scale;
  const float l = lse[row];
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(lr)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = __expf(f[j] - l);
      f[j] = (p - ((i * 8 + j) == y ? 1.f : 0.f)) * sc;
    }
    reinterpret_cast<bf16x8*>(orow)[i] = pack8(f);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    const float p = __expf(__bfloat162float(lr[i]) - l);
    orow[i] = __float2bfloat16((p - (i == y ? 1.f : 0.f)) * sc);
  }
}

// --------------------------------------------------------------------- Adam
// Flat-buffer Adam / AdamW: fp32 master / m / v, fp32 gradient (scaled by
// grad_scale), bf16 parameter copy written in the same pass.  decoupled != 0
// is AdamW (the decay shrinks the weight directly); otherwise the decay is
// the L2 term of torch.optim.Adam, added to the gradient before the moments.
__global__ void adam_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                 const float* __restrict__ grad, __nv_bfloat16* __restrict__ param,
                                 long long n, float lr, float b1, float b2, float eps, float wd,
                                 float bc1, float bc2, float grad_scale, int decoupled) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p = master[i];
    float g = grad[i] * grad_scale;
    if (!decoupled) g += wd * p;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi / bc2) + eps;
    p = p - lr * (mi / bc1) / denom - (decoupled ? lr * wd * p : 0.f);
    master[i] = p;
    if (param) param[i] = __float2bfloat16(p);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                        long long n, float scale) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16(in[i] * scale);
}

// acc (fp32) += g (bf16): gradient accumulation into the flat bucket for
// parameters whose gradient comes from autograd as a bf16 tensor.
__global__ void accum_bf16_into_f32_kernel(const __nv_bfloat16* __restrict__ g, float* __restrict__ acc,
                                           long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    acc[i] += __bfloat162float(g[i]);
}

// out = a + b over n bf16 elements (n % 8 == 0): the residual add at a stage boundary.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    unpack8(reinterpret_cast<const bf16x8*>(a)[i], x);
    unpack8(reinterpret_cast<const bf16x8*>(b)[i], y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    reinterpret_cast<bf16x8*>(out)[i] = pack8(x);
  }
}

// True when every non-null pointer is 16-byte aligned (the kernels use 16-byte vector accesses).
template <typename... P>
inline bool aligned16(P... ptrs) {
  return ((reinterpret_cast<uintptr_t>(static_cast<const void*>(ptrs)) | ...) & 15u) == 0;
}

inline int grid_for(long long work, int threads, int max_blocks = 148 * 16) {
  long long b = (work + threads - 1) / threads;
  if (b > max_blocks) b = max_blocks;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

#define PIPER_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -3)

int rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                long long T, int D, float eps, cudaStream_t st) {
  if (D % 8 != 0) return -1;
  if (T == 0) return 0;
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* rp = static_cast<const __nv_bfloat16*>(res);
  const auto* wp = static_cast<const __nv_bfloat16*>(w);
  auto* yp = static_cast<__nv_bfloat16*>(y);
  auto* hp = static_cast<__nv_bfloat16*>(h_out);
  const unsigned grid = static_cast<unsigned>(T);
  switch (D) {
    case 2048: rmsnorm_fwd_reg_kernel<1><<<grid, NORM_THREADS, 0, st>>>(xp, rp, wp, yp, hp, rstd, eps); return PIPER_LAUNCH_OK();
    case 4096: rmsnorm_fwd_reg_kernel<2><<<grid, NORM_THREADS, 0, st>>>(xp, rp, wp, yp, hp, rstd, eps); return PIPER_LAUNCH_OK();
    case 8192: rmsnorm_fwd_reg_kernel<4><<<grid, NORM_THREADS, 0, st>>>(xp, rp, wp, yp, hp, rstd, eps); return PIPER_LAUNCH_OK();
    default: break;
  }
  rmsnorm_fwd_kernel<<<static_cast<unsigned>(T), NORM_THREADS, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
      static_cast<__nv_bfloat16*>(h_out), rstd, D, eps);
  return PIPER_LAUNCH_OK();
}

// Two strips per SM of a 148-SM part, whatever the device: the allocation-free entry point sizes its built-in
// scratch array (PIPER_NOALLOC_MAX_STRIPS) from this fixed bound.
int rmsnorm_bwd_num_partials(long long T) {
  const int cap = 148 * 2;
  return static_cast<int>(T < cap ? (T > 0 ? T : 1) : cap);
}

int rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                void* dx, float* dw_partial, float* dw_f32, void* dw_bf16, int accumulate, long long T,
                int D, cudaStream_t st) {
  if (D % 8 != 0 || D * sizeof(float) > 160 * 1024) return -1;
  if (T < 0 || T > 2147483647LL) return -1;      // the kernels index rows with a 32-bit int
  if (T == 0) return 0;
  const int nb = rmsnorm_bwd_num_partials(T);
  const dim3 red_grid((D + 31) / 32), red_block(32, RED_SLICES);
  if (D == 2048 || D == 4096 || D == 8192) {
    const auto* dyp = static_cast<const __nv_bfloat16*>(dy);
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    const auto* wp = static_cast<const __nv_bfloat16*>(w);
    const auto* ep = static_cast<const __nv_bfloat16*>(dres);
    auto* dxp = static_cast<__nv_bfloat16*>(dx);
    const int Ti = static_cast<int>(T);
    if (D == 2048) rmsnorm_bwd_reg_kernel<1><<<nb, NORM_THREADS, 0, st>>>(dyp, xp, wp, rstd, ep, dxp, dw_partial, Ti);
    else if (D == 4096) rmsnorm_bwd_reg_kernel<2><<<nb, NORM_THREADS, 0, st>>>(dyp, xp, wp, rstd, ep, dxp, dw_partial, Ti);
    else rmsnorm_bwd_reg_kernel<4><<<nb, NORM_THREADS, 0, st>>>(dyp, xp, wp, rstd, ep, dxp, dw_partial, Ti);
    reduce_partials_kernel<<<red_grid, red_block, 0, st>>>(dw_partial, nb, D, dw_f32,
                                                           static_cast<__nv_bfloat16*>(dw_bf16), accumulate);
    return PIPER_LAUNCH_OK();
  }
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    configured = true;
  }
  rmsnorm_bwd_kernel<<<nb, NORM_THREADS, D * sizeof(float), st>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),
      static_cast<__nv_bfloat16*>(dx), dw_partial, static_cast<int>(T), D);
  reduce_partials_kernel<<<red_grid, red_block, 0, st>>>(dw_partial, nb, D, dw_f32,
                                                         static_cast<__nv_bfloat16*>(dw_bf16), accumulate);
  return PIPER_LAUNCH_OK();
}

int qk_rope_fwd(const void* in, void* out, const float* cosp, const float* sinp, const void* qw,
                const void* kw, long long T, int S, int Hq, int Hkv, int hd, int interleaved, float eps,
                cudaStream_t st) {
  const long long groups = T * ((Hq + 2 * Hkv + ROPE_HEADS_PER_GROUP - 1) / ROPE_HEADS_PER_GROUP);
  if (groups == 0) return 0;
  if (hd != 128 && hd != 64) return -1;
  if (groups >= (1ll << 31) || static_cast<long long>(S) * (hd / 2) >= (1ll << 31)) return -1;
  if (!aligned16(in, out, cosp, sinp, qw, kw)) return -4;
  const int threads = 256;
  const int blocks = grid_for(groups * (hd / 16), threads);
  auto a = static_cast<const __nv_bfloat16*>(in);
  auto o = static_cast<__nv_bfloat16*>(out);
  auto q = static_cast<const __nv_bfloat16*>(qw);
  auto k = static_cast<const __nv_bfloat16*>(kw);
  if (hd == 128)
    qk_rope_kernel<128><<<blocks, threads, 0, st>>>(a, o, cosp, sinp, q, k, nullptr, T, S, Hq, Hkv,
                                                    interleaved, eps, 1.f);
  else if (hd == 64)
    qk_rope_kernel<64><<<blocks, threads, 0, st>>>(a, o, cosp, sinp, q, k, nullptr, T, S, Hq, Hkv,
                                                   interleaved, eps, 1.f);
  else
    return -1;
  return PIPER_LAUNCH_OK();
}

int qk_rope_bwd(const void* dout, const void* in, void* din, const float* cosp, const float* sinp,
                const void* qw, const void* kw, float* dqw, float* dkw, long long T, int S, int Hq,
                int Hkv, int hd, int interleaved, float eps, cudaStream_t st) {
  const long long groups = T * ((Hq + 2 * Hkv + ROPE_HEADS_PER_GROUP - 1) / ROPE_HEADS_PER_GROUP);
  if (groups == 0) return 0;
  if (hd != 128 && hd != 64) return -1;
  if (groups >= (1ll << 31) || static_cast<long long>(S) * (hd / 2) >= (1ll << 31)) return -1;
  if (!aligned16(dout, in, din, cosp, sinp, qw, kw)) return -4;
  const int threads = 256;
  const int blocks = grid_for(groups * (hd / 16), threads);
  auto g = static_cast<const __nv_bfloat16*>(dout);
  auto a = static_cast<const __nv_bfloat16*>(in);
  auto o = static_cast<__nv_bfloat16*>(din);
  auto q = static_cast<const __nv_bfloat16*>(qw);
  auto k = static_cast<const __nv_bfloat16*>(kw);
  if (hd == 128)
    qk_rope_bwd_kernel<128><<<blocks, threads, 0, st>>>(g, a, o, cosp, sinp, q, k, dqw, dkw, T, S, Hq,
                                                        Hkv, interleaved, eps);
  else if (hd == 64)
    qk_rope_bwd_kernel<64><<<blocks, threads, 0, st>>>(g, a, o, cosp, sinp, q, k, dqw, dkw, T, S, Hq,
                                                       Hkv, interleaved, eps);
  else
    return -1;
  return PIPER_LAUNCH_OK();
}

int swiglu_fwd(const void* h13, void* act, long long T, int F, cudaStream_t st) {
  if (F % 8 != 0) return -1;
  if (T == 0) return 0;
  const int vecs = F / 8;
  const int blocks = grid_for(T * vecs, 256);
  const long long stride = static_cast<long long>(blocks) * 256;
  swiglu_fwd_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h13), static_cast<__nv_bfloat16*>(act), T,
                                            F, static_cast<int>(stride / vecs), static_cast<int>(stride % vecs));
  return PIPER_LAUNCH_OK();
}

int swiglu_bwd(const void* h13, const void* dact, void* dh13, long long T, int F, cudaStream_t st) {
  if (F % 8 != 0) return -1;
  if (T == 0) return 0;
  const int vecs = F / 8;
  const int blocks = grid_for(T * vecs, 256);
  const long long stride = static_cast<long long>(blocks) * 256;
  swiglu_bwd_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h13),
                                            static_cast<const __nv_bfloat16*>(dact), static_cast<__nv_bfloat16*>(dh13),
                                            T, F, static_cast<int>(stride / vecs), static_cast<int>(stride % vecs));
  return PIPER_LAUNCH_OK();
}

int embedding_fwd(const long long* tokens, const void* table, void* out, long long T, int D, int V,
                  int* status, cudaStream_t st) {
  if (D % 8 != 0) return -1;
  if (T == 0) return 0;
  embedding_fwd_kernel<<<static_cast<unsigned>(T), 128, 0, st>>>(
      tokens, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), T, D, V, status);
  return PIPER_LAUNCH_OK();
}

int embedding_bwd(const long long* tokens, const void* dout, float* dtable, long long T, int D, int V,
                  cudaStream_t st) {
  if (T == 0) return 0;
  embedding_bwd_kernel<<<static_cast<unsigned>(T), 256, 0, st>>>(
      tokens, static_cast<const __nv_bfloat16*>(dout), dtable, T, D, V);
  return PIPER_LAUNCH_OK();
}

int ce_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long T, int V,
           long long ld, long long ignore_index, cudaStream_t st) {
  if (ld % 8 != 0) return -1;
  if (T == 0) return 0;
  ce_fwd_kernel<<<static_cast<unsigned>(T), CE_THREADS, 0, st>>>(
      static_cast<const __nv_bfloat16*>(logits), labels, loss, lse, V, ld, ignore_index);
  return PIPER_LAUNCH_OK();
}

int ce_bwd(const void* logits, const long long* labels, const float* lse, const float* gscale,
           float row_scale, void* out, long long T, int V, long long ld, long long ignore_index,
           cudaStream_t st) {
  if (ld % 8 != 0) return -1;
  if (T == 0) return 0;
  ce_bwd_kernel<<<static_cast<unsigned>(T), CE_THREADS, 0, st>>>(
      static_cast<const __nv_bfloat16*>(logits), labels, lse, gscale, row_scale,
      static_cast<__nv_bfloat16*>(out), V, ld, ignore_index);
  return PIPER_LAUNCH_OK();
}

int adam_flat(float* master, float* m, float* v, const float* grad, void* param_bf16, long long n,
              float lr, float b1, float b2, float eps, float wd, int step, float grad_scale, int decoupled,
              cudaStream_t st) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, static_cast<float>(step));
  const float bc2 = 1.f - powf(b2, static_cast<float>(step));
  adam_flat_kernel<<<grid_for(n, 256), 256, 0, st>>>(master, m, v, grad,
                                                    static_cast<__nv_bfloat16*>(param_bf16), n, lr, b1, b2,
                                                    eps, wd, bc1, bc2, grad_scale, decoupled);
  return PIPER_LAUNCH_OK();
}

int cast_f32_to_bf16(const float* in, void* out, long long n, float scale, cudaStream_t st) {
  if (n == 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, st>>>(in, static_cast<__nv_bfloat16*>(out), n, scale);
  return PIPER_LAUNCH_OK();
}

int add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t st) {
  if (n % 8 != 0) return -1;
  if (n == 0) return 0;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a),
                                                       static_cast<const __nv_bfloat16*>(b),
                                                       static_cast<__nv_bfloat16*>(out), n / 8);
  return PIPER_LAUNCH_OK();
}

int accum_bf16_into_f32(const void* g, float* acc, long long n, cudaStream_t st) {
  if (n == 0) return 0;
  accum_bf16_into_f32_kernel<<<grid_for(n, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(g), acc, n);
  return PIPER_LAUNCH_OK();
}

}  // namespace piper
