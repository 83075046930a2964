// Causal grouped-query flash attention for sm_100a, forward and backward,
// on the packed projection qkv[T, (Hq + 2*Hkv) * hd] (T = B*S tokens, each
// sequence a multiple of 128 long).  All matrix products run on tcgen05 with
// accumulators in tensor memory; operands arrive by TMA (no multicast) in
// 128-byte-swizzled tiles, and the probability / score-gradient tiles the
// threads produce are written to shared memory in the same swizzled layout so
// that they can feed the next tcgen05.mma directly.
//
// Forward (attn_fwd_kernel): one CTA per (128 query rows, head).  Warps 0-3
// own one query row per thread (row == TMEM lane), warp 4 issues TMA, warp 5
// issues MMAs.  S = Q K^T is double-buffered in TMEM so the next block's
// scores are computed while the threads run the online softmax; each P V
// product lands in a fresh TMEM buffer and is folded into fp32 registers with
// the running rescale factor, so TMEM is never rewritten by threads.
//
// Backward (attn_bwd_kernel<MODE>): one template for both passes.
//   MODE 0 (dQ):  stationary tile = 128 query rows of one head (Q, dO);
//                 streams 64-row K/V tiles; accumulates dQ.
//   MODE 1 (dKV): stationary tile = 128 key rows of one kv head (K, V);
//                 streams 64-row Q/dO tiles of every query head in the group;
//                 accumulates dK and dV.
// In both, S' = X1 Y1^T and dP' = X2 Y2^T are recomputed into double-buffered
// TMEM, threads form P' = exp(S' - lse) and dS' = P' (dP' - delta) as bf16
// tiles in shared memory, and acc1 += dS' Y1 (acc2 += P' Y2 in MODE 1) reuses
// the streamed tiles as MN-major operands.  Nothing is reduced with atomics,
// so gradients are reproducible.
//
// Every mbarrier wait is bounded (see ptx.cuh); on expiry a status code is
// recorded and the CTA unwinds and frees its TMEM.
#include "attention_sm100.h"

#include <cstdlib>
#include <map>
#include <mutex>

#include "ptx.cuh"

namespace piper {
namespace {

// Bounded wait on an mbarrier phase (see mbar_wait in ptx.cuh).
__device__ __forceinline__ bool await(uint64_t* bar, uint32_t parity, int* status) {
  return mbar_wait(bar, parity, status);
}

// The same for a whole warp, with one outcome for all its lanes: a lane that gave up while its neighbours saw
// the phase complete must not leave them alone at the next warp-wide synchronisation.
__device__ __forceinline__ bool await_all(uint64_t* bar, uint32_t parity, int* status) {
  return __all_sync(0xffffffffu, await(bar, parity, status));
}

// One arrival per warp: the lanes converge first, so whatever each of them wrote (and fenced) before the call
// is ordered before the arrival that lane 0 performs for all of them.  256 threads arriving one by one on the
// same barrier word would serialise in the shared-memory atomic unit several times per tile.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Writes 32 consecutive bf16 values (given as 16 packed words) of row `row`,
// starting at 16-byte chunk index `chunk0` (multiple of 4) of a 128-byte
// swizzled row.  `tile` is the 1024-byte-aligned base of a [rows][128 B] tile.
__device__ __forceinline__ void store_row_chunk_sw128(uint8_t* tile, int row, int chunk0,
                                                      const uint32_t (&w)[16]) {
  uint8_t* rbase = tile + row * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int phys = (chunk0 + q) ^ (row & 7);
    *reinterpret_cast<uint4*>(rbase + phys * 16) =
        make_uint4(w[4 * q + 0], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
  }
}

// ================================================================= forward
// warps 0-3 and 6-9: two softmax groups of 128 threads (each takes half the key columns of every score
// tile and half the head dimension of the output); warp 4: TMA; warp 5: MMA
constexpr int FWD_THREADS = 320;

template <int HD>
struct FwdSmem {
  static constexpr int HALVES = HD / 64;
  static constexpr int TILE = 128 * HD * 2;     // Q, K or V tile
  static constexpr int P_BYTES = 128 * 128 * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;            // 2 stages
  static constexpr int V_OFF = 3 * TILE;        // 2 stages
  static constexpr int P_OFF = 5 * TILE;
  static constexpr int X_OFF = P_OFF + P_BYTES;   // row-max exchange [2 tiles][2 groups][128] + row-sum [2][128]
  static constexpr int BAR_OFF = X_OFF + 6 * 128 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

struct FwdBars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];     // K is free again once S = Q K^T of its block has been computed ...
  uint64_t v_full[2], v_empty[2];     // ... V only after P V, so the two rings run at different distances
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, p_empty;
  uint64_t o_full[2], o_empty[2];
  uint64_t mx_full[2], l_full;        // the two softmax groups exchange row maxima / row sums
  uint32_t tmem_base;
};

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap, __nv_bfloat16* __restrict__ out,
                float* __restrict__ lse, int S, int Hq, int Hkv, float scale_log2, int* status) {
  using L = FwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  FwdBars* bars = reinterpret_cast<FwdBars*>(smem + L::BAR_OFF);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;   // longest rows first
  const int head = blockIdx.y;
  const int b = blockIdx.z;
  const int g = head / (Hq / Hkv);
  const int n_blocks = qblk + 1;
  const long long tok0 = static_cast<long long>(b) * S;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 8);        // one arrival per softmax warp
      mbar_init(&bars->o_full[i], 1);
      mbar_init(&bars->o_empty[i], 8);
      mbar_init(&bars->mx_full[i], 8);
    }
    mbar_init(&bars->p_full, 8);
    mbar_init(&bars->p_empty, 1);
    mbar_init(&bars->l_full, 8);
    fence_mbar_init();
    tma_prefetch_desc(&tmap);
  }
  if (warp == 5) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const uint32_t tmem_s = tmem_base;          // 2 x 128 columns
  const uint32_t tmem_o = tmem_base + 256;    // 2 x HD columns

  if (warp == 4) {
    // ------------------------------------------------------------- TMA
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars->q_full, L::TILE);
      for (int h = 0; h < L::HALVES; ++h)
        tma_load_2d(smem + L::Q_OFF + h * 16384, &tmap, &bars->q_full, head * HD + 64 * h,
                    static_cast<int>(tok0) + qblk * 128);
      // K and V blocks are loaded as soon as their own stage is free, whichever comes first
      int kj = 0, vj = 0;
      uint32_t idle = 0;
      bool ok = true;
      while ((kj < n_blocks || vj < n_blocks) && ok) {
        bool progressed = false;
        if (kj < n_blocks && mbar_test_wait(&bars->k_empty[kj & 1], ((kj >> 1) & 1) ^ 1)) {
          const int s = kj & 1;
          mbar_arrive_expect_tx(&bars->k_full[s], L::TILE);
          for (int h = 0; h < L::HALVES; ++h)
            tma_load_2d(smem + L::K_OFF + s * L::TILE + h * 16384, &tmap, &bars->k_full[s],
                        (Hq + g) * HD + 64 * h, static_cast<int>(tok0) + kj * 128);
          ++kj;
          progressed = true;
        }
        if (vj < n_blocks && mbar_test_wait(&bars->v_empty[vj & 1], ((vj >> 1) & 1) ^ 1)) {
          const int s = vj & 1;
          mbar_arrive_expect_tx(&bars->v_full[s], L::TILE);
          for (int h = 0; h < L::HALVES; ++h)
            tma_load_2d(smem + L::V_OFF + s * L::TILE + h * 16384, &tmap, &bars->v_full[s],
                        (Hq + Hkv + g) * HD + 64 * h, static_cast<int>(tok0) + vj * 128);
          ++vj;
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > kMaxMbarPolls) {
          atomicCAS(status, 0, kStatusMbarTimeout);
          ok = false;
        } else if ((idle & 1023u) == 0 && *reinterpret_cast<volatile int*>(status) != 0) {
          ok = false;
        }
      }
      if (!ok) {
        // Unwinding after a failed wait: let the copies already issued land
        // before the CTA and its shared memory go away.
        await(&bars->q_full, 0, nullptr);
        for (int jj = kj - 1; jj >= 0 && jj >= kj - 2; --jj)
          await(&bars->k_full[jj & 1], (jj >> 1) & 1, nullptr);
        for (int jj = vj - 1; jj >= 0 && jj >= vj - 2; --jj)
          await(&bars->v_full[jj & 1], (jj >> 1) & 1, nullptr);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------- MMA
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, HD, false, true);
      const uint32_t q_addr = smem_u32(smem + L::Q_OFF);
      const uint32_t p_addr = smem_u32(smem + L::P_OFF);
      // descriptors of the operands that never move (Q, the probability tile), one per k-step: the issuing
      // thread's instruction count per MMA is what bounds the loops below
      uint64_t dq[HD / 16], dp[8];
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        dq[ks] = umma_desc_sw128(q_addr + (ks / 4) * 16384 + (ks % 4) * 32, 16, 1024);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        dp[ks] = umma_desc_sw128(p_addr + (ks / 4) * 16384 + (ks % 4) * 32, 16, 1024);
      bool ok = await(&bars->q_full, 0, status);
      // Two queues served in whatever order their inputs arrive: S of block s_next (needs K and a free TMEM
      // stage) and P V of block p_next (needs the probabilities, V and a free output stage).
      int s_next = 0, p_next = 0;
      uint32_t idle = 0;
      while (p_next < n_blocks && ok) {
        bool progressed = false;
        if (p_next < s_next) {
          const int jj = p_next;
          const int sb = jj & 1;
          if (mbar_test_wait(&bars->p_full, jj & 1) && mbar_test_wait(&bars->v_full[sb], (jj >> 1) & 1) &&
              mbar_test_wait(&bars->o_empty[sb], ((jj >> 1) & 1) ^ 1)) {
            tc_fence_after();
            const uint64_t dv0 = umma_desc_sw128(smem_u32(smem + L::V_OFF + sb * L::TILE), 16384, 1024);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_bf16_ss(tmem_o + sb * HD, dp[ks], dv0 + (ks * 2048 >> 4), idesc_pv, ks > 0 ? 1u : 0u);
            umma_commit(&bars->p_empty);
            umma_commit(&bars->o_full[sb]);
            umma_commit(&bars->v_empty[sb]);
            ++p_next;
            progressed = true;
          }
        }
        if (s_next < n_blocks) {
          const int j = s_next;
          const int s = j & 1;
          if (mbar_test_wait(&bars->k_full[s], (j >> 1) & 1) &&
              mbar_test_wait(&bars->s_empty[s], ((j >> 1) & 1) ^ 1)) {
            tc_fence_after();
            const uint64_t dk0 = umma_desc_sw128(smem_u32(smem + L::K_OFF + s * L::TILE), 16, 1024);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
              umma_bf16_ss(tmem_s + s * 128, dq[ks], dk0 + (off >> 4), idesc_qk, ks > 0 ? 1u : 0u);
            }
            umma_commit(&bars->s_full[s]);
            umma_commit(&bars->k_empty[s]);
            ++s_next;
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > kMaxMbarPolls) {
          atomicCAS(status, 0, kStatusMbarTimeout);
          ok = false;
        } else if ((idle & 1023u) == 0 && *reinterpret_cast<volatile int*>(status) != 0) {
          ok = false;
        }
      }
    }
  } else {
    // --------------------------------------------------- softmax + output
    // A warp reaches the TMEM lanes 32*(warp % 4)..+31.  Group wg owns key columns [64*wg, 64*wg + 64) of every
    // score tile and output columns [wg*HD/2, (wg+1)*HD/2); per tile the groups exchange their row maxima.
    constexpr int HH = HD / 2;
    const int wg = warp >= 6 ? 1 : 0;
    const int row = (warp & 3) * 32 + lane;      // query row == TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float* xbuf = reinterpret_cast<float*>(smem + L::X_OFF);
    float o_acc[HH];
#pragma unroll
    for (int i = 0; i < HH; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int s = j & 1;
      const bool diag = (j == qblk);
      if (!await_all(&bars->s_full[s], (j >> 1) & 1, status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_s + lane_sel + s * 128 + wg * 64;
      uint32_t sv[64];
      {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(ts, r0);
        tmem_ld_32x32(ts + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sv[i] = r0[i]; sv[32 + i] = r1[i]; }
      }
      tc_fence_before();
      warp_arrive(&bars->s_empty[s], lane);            // the scores live in registers from here on
      if (diag) {
        // causal mask, applied once to the registers of the only tile that needs it: a score of -inf then
        // drops out of the maximum and turns into a probability of exactly zero below
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (wg * 64 + i > row) sv[i] = 0xff800000u;
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; i += 2)
        mx = fmaxf(mx, fmaxf(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])));
      xbuf[(s * 2 + wg) * 128 + row] = mx;
      warp_arrive(&bars->mx_full[s], lane);
      if (!await_all(&bars->mx_full[s], (j >> 1) & 1, status)) { ok = false; break; }
      mx = fmaxf(mx, xbuf[(s * 2 + (wg ^ 1)) * 128 + row]);
      const float m_new = fmaxf(m_run, mx);
      const float alpha = fast_exp2((m_run - m_new) * scale_log2);
      const float msc = m_new * scale_log2;
      if (j > 0 && !await_all(&bars->p_empty, (j - 1) & 1, status)) { ok = false; break; }
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = fast_exp2(__uint_as_float(sv[c * 32 + 2 * i]) * scale_log2 - msc);
          const float p1 = fast_exp2(__uint_as_float(sv[c * 32 + 2 * i + 1]) * scale_log2 - msc);
          rs += p0 + p1;
          w[i] = pack_bf16x2(p0, p1);
        }
        store_row_chunk_sw128(smem + L::P_OFF + wg * 16384, row, c * 4, w);
      }
      fence_proxy_async_smem();
      warp_arrive(&bars->p_full, lane);
      if (j > 0) {
        const int sb = (j - 1) & 1;
        if (!await_all(&bars->o_full[sb], ((j - 1) >> 1) & 1, status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t to = tmem_o + lane_sel + sb * HD + wg * HH;
#pragma unroll
        for (int c = 0; c < HH / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(to + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha_prev + __uint_as_float(r[i]);
        }
        tc_fence_before();
        warp_arrive(&bars->o_empty[sb], lane);
      }
      l_run = l_run * alpha + rs;
      m_run = m_new;
      alpha_prev = alpha;
    }
    if (ok) {
      // total row sum = this group's partial + the other group's
      xbuf[(4 + wg) * 128 + row] = l_run;
      warp_arrive(&bars->l_full, lane);
      ok = await_all(&bars->l_full, 0, status);
    }
    if (ok) {
      const float l_tot = l_run + xbuf[(4 + (wg ^ 1)) * 128 + row];
      const int jj = n_blocks - 1;
      const int sb = jj & 1;
      if (await_all(&bars->o_full[sb], (jj >> 1) & 1, status)) {
        tc_fence_after();
        const uint32_t to = tmem_o + lane_sel + sb * HD + wg * HH;
        const float inv = 1.f / l_tot;
        const long long tok = tok0 + static_cast<long long>(qblk) * 128 + row;
        __nv_bfloat16* orow = out + tok * (static_cast<long long>(Hq) * HD) + head * HD + wg * HH;
#pragma unroll
        for (int c = 0; c < HH / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(to + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = v * 8 + 2 * i;
              const float a = (o_acc[c * 32 + e] * alpha_prev + __uint_as_float(r[e])) * inv;
              const float bb = (o_acc[c * 32 + e + 1] * alpha_prev + __uint_as_float(r[e + 1])) * inv;
              ow[i] = pack_bf16x2(a, bb);
            }
            reinterpret_cast<uint4*>(orow + c * 32)[v] = o;
          }
        }
        if (wg == 0)
          lse[(static_cast<long long>(b) * Hq + head) * S + qblk * 128 + row] =
              m_run * (scale_log2 * 0.6931471805599453f) + logf(l_tot);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ================================================================ backward
// delta[b, h, s] = sum_d dO[t, h, d] * O[t, h, d]; HD/8 lanes per (t, h), one 16-byte vector of each per lane.
template <int HD>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                  float* __restrict__ delta, long long T, int S, int Hq) {
  constexpr int LANES = HD / 8;
  const int wl = threadIdx.x & 31;
  const int lane = wl & (LANES - 1);
  const unsigned mask = ((1u << LANES) - 1u) << (wl & ~(LANES - 1));
  const unsigned total = static_cast<unsigned>(T * Hq);   // the launcher keeps T * Hq below 2^31
  const unsigned stride = gridDim.x * (256 / LANES);
  for (unsigned gi = blockIdx.x * (256 / LANES) + threadIdx.x / LANES; gi < total; gi += stride) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + static_cast<long long>(gi) * HD + 8 * lane);
    const uint4 b = *reinterpret_cast<const uint4*>(d_o + static_cast<long long>(gi) * HD + 8 * lane);
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ap[i]), y = __bfloat1622float2(bp[i]);
      s += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int off = LANES / 2; off > 0; off >>= 1) s += __shfl_xor_sync(mask, s, off);
    const unsigned t = gi / static_cast<unsigned>(Hq), h = gi - t * Hq;
    const unsigned bi = t / static_cast<unsigned>(S), si = t - bi * S;
    if (lane == 0) delta[(static_cast<long long>(bi) * Hq + h) * S + si] = s;
  }
}

// warps 0-3 and 6-9: two groups of 128 threads that split the columns of every S'/dP' tile; warp 4: TMA;
// warp 5: MMA
constexpr int BWD_THREADS = 320;

template <int HD>
struct BwdSmem {
  static constexpr int HALVES = HD / 64;
  static constexpr int X_TILE = 128 * HD * 2;      // stationary tile
  static constexpr int Y_TILE = 64 * HD * 2;       // streamed tile
  static constexpr int Y_HALF = 64 * 128;          // one 64x64 box
  static constexpr int PT_BYTES = 128 * 64 * 2;    // P' or dS' tile (one swizzle row per row)
  static constexpr int X1_OFF = 0;
  static constexpr int X2_OFF = X_TILE;
  static constexpr int Y_STAGES = 4;
  static constexpr int Y_OFF = 2 * X_TILE;         // Y_STAGES x (Y1, Y2), see y_off
  // Streamed stages are laid out in pairs: the same 64-column half of the same operand of stages 2p and 2p+1
  // is one contiguous 128-row tile.  (Issuing S' and dP' of two consecutive tiles as one N = 128 MMA each was
  // tried on this layout: every MMA costs the issuing thread about 110 cycles whatever its width, but the two
  // TMEM stages are never free at the same moment in steady state, so the pairs did not form.)
  static constexpr int HALF_STRIDE = 2 * Y_HALF;   // between the 64-column halves of one stage's operand
  __host__ __device__ static constexpr int y_off(int st, int operand, int half) {
    return (st >> 1) * (4 * Y_TILE) + operand * (2 * Y_TILE) + half * HALF_STRIDE + (st & 1) * Y_HALF;
  }
  static constexpr int P_OFF = Y_OFF + Y_STAGES * 2 * Y_TILE;
  static constexpr int DS_OFF = P_OFF + PT_BYTES;
  static constexpr int VEC_OFF = DS_OFF + PT_BYTES;              // 3 stages x (lse[64], delta[64]) floats
  static constexpr int BAR_OFF = VEC_OFF + 3 * 2 * 64 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

struct BwdBars {
  uint64_t x_full;
  uint64_t y_full[4], y_empty[4];     // streamed tiles (BwdSmem::Y_STAGES)
  uint64_t s_full[2], s_empty[2];     // S' and dP' pair
  uint64_t t_full, t_empty;           // P'/dS' shared-memory tiles
  uint64_t v_full[2];                 // per-column lse/delta vectors (MODE 1)
  uint64_t acc_full;
  uint32_t tmem_base;
};

// MODE 0: dQ.  MODE 1: dK, dV.
template <int HD, int MODE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv_x,   // box {64, 128} over packed qkv
                const __grid_constant__ CUtensorMap tmap_qkv_y,   // box {64, 64}  over packed qkv
                const __grid_constant__ CUtensorMap tmap_do_x,    // box {64, 128} over dO [T, Hq*hd]
                const __grid_constant__ CUtensorMap tmap_do_y,    // box {64, 64}  over dO
                const float* __restrict__ lse, const float* __restrict__ delta,
                __nv_bfloat16* __restrict__ d_qkv, int S, int Hq, int Hkv, float scale,
                float scale_log2, int* status) {
  using L = BwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  BwdBars* bars = reinterpret_cast<BwdBars*>(smem + L::BAR_OFF);
  float* vec = reinterpret_cast<float*>(smem + L::VEC_OFF);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = Hq / Hkv;
  const int b = blockIdx.z;
  const long long tok0 = static_cast<long long>(b) * S;
  const int W = (Hq + 2 * Hkv) * HD;   // packed row width

  // Stationary block index and iteration space.
  //   MODE 0: blockIdx.y = query head; streams kv tiles i in [0, 2*xb + 1].
  //   MODE 1: blockIdx.y = kv head; for each query head of the group streams
  //           q tiles i in [2*xb, S/64 - 1].
  const int xb = (MODE == 0) ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int hy = blockIdx.y;
  const int g = (MODE == 0) ? hy / group : hy;
  const int tiles_per_head = (MODE == 0) ? (2 * xb + 2) : (S / 64 - 2 * xb);
  const int n_iter = (MODE == 0) ? tiles_per_head : tiles_per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(&bars->x_full, 1);
    for (int i = 0; i < L::Y_STAGES; ++i) {
      mbar_init(&bars->y_full[i], 1);
      mbar_init(&bars->y_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 8);        // one arrival per softmax warp
      mbar_init(&bars->v_full[i], 2);        // warps 0 and 1 write the vectors
    }
    mbar_init(&bars->t_full, 8);
    mbar_init(&bars->t_empty, 1);
    mbar_init(&bars->acc_full, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_qkv_x);
    tma_prefetch_desc(&tmap_qkv_y);
    tma_prefetch_desc(&tmap_do_x);
    tma_prefetch_desc(&tmap_do_y);
  }
  if (warp == 5) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  // columns: [0,64) S'0  [64,128) S'1  [128,192) dP'0  [192,256) dP'1
  //          [256,256+HD) acc1   [384,384+HD) acc2
  const uint32_t tmem_acc1 = tmem_base + 256;
  const uint32_t tmem_acc2 = tmem_base + 384;

  if (warp == 4) {
    // ------------------------------------------------------------- TMA
    if (lane == 0) {
      const int xrow = static_cast<int>(tok0) + xb * 128;
      mbar_arrive_expect_tx(&bars->x_full, 2 * L::X_TILE);
      for (int h = 0; h < L::HALVES; ++h) {
        if (MODE == 0) {
          tma_load_2d(smem + L::X1_OFF + h * 16384, &tmap_qkv_x, &bars->x_full, hy * HD + 64 * h, xrow);
          tma_load_2d(smem + L::X2_OFF + h * 16384, &tmap_do_x, &bars->x_full, hy * HD + 64 * h, xrow);
        } else {
          tma_load_2d(smem + L::X1_OFF + h * 16384, &tmap_qkv_x, &bars->x_full,
                      (Hq + g) * HD + 64 * h, xrow);
          tma_load_2d(smem + L::X2_OFF + h * 16384, &tmap_qkv_x, &bars->x_full,
                      (Hq + Hkv + g) * HD + 64 * h, xrow);
        }
      }
      int it = 0;
      for (; it < n_iter; ++it) {
        const int st = it % L::Y_STAGES;
        if (!await(&bars->y_empty[st], ((it / L::Y_STAGES) & 1) ^ 1, status)) break;
        const int hh = (MODE == 0) ? hy : g * group + it / tiles_per_head;   // query head
        const int ti = (MODE == 0) ? it : 2 * xb + it % tiles_per_head;      // streamed tile index
        const int yrow = static_cast<int>(tok0) + ti * 64;
        uint8_t* yb = smem + L::Y_OFF;
        mbar_arrive_expect_tx(&bars->y_full[st], 2 * L::Y_TILE);
        for (int h = 0; h < L::HALVES; ++h) {
          uint8_t* y1 = yb + L::y_off(st, 0, h);
          uint8_t* y2 = yb + L::y_off(st, 1, h);
          if (MODE == 0) {
            tma_load_2d(y1, &tmap_qkv_y, &bars->y_full[st], (Hq + g) * HD + 64 * h, yrow);
            tma_load_2d(y2, &tmap_qkv_y, &bars->y_full[st], (Hq + Hkv + g) * HD + 64 * h, yrow);
          } else {
            tma_load_2d(y1, &tmap_qkv_y, &bars->y_full[st], hh * HD + 64 * h, yrow);
            tma_load_2d(y2, &tmap_do_y, &bars->y_full[st], hh * HD + 64 * h, yrow);
          }
        }
      }
      if (it < n_iter) {
        // Unwinding: wait (bounded) for the copies in flight.
        await(&bars->x_full, 0, nullptr);
        for (int jj = it - 1; jj >= 0 && jj > it - 1 - L::Y_STAGES; --jj)
          await(&bars->y_full[jj % L::Y_STAGES], (jj / L::Y_STAGES) & 1, nullptr);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------- MMA
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, false, true);
      const uint32_t x1 = smem_u32(smem + L::X1_OFF);
      const uint32_t x2 = smem_u32(smem + L::X2_OFF);
      const uint32_t p_addr = smem_u32(smem + L::P_OFF);
      const uint32_t ds_addr = smem_u32(smem + L::DS_OFF);
      uint64_t dx1[HD / 16], dx2[HD / 16];       // descriptors of the stationary operands, fixed for the kernel
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const uint32_t xo = (ks / 4) * 16384 + (ks % 4) * 32;
        dx1[ks] = umma_desc_sw128(x1 + xo, 16, 1024);
        dx2[ks] = umma_desc_sw128(x2 + xo, 16, 1024);
      }
      const uint64_t d_ds = umma_desc_sw128(ds_addr, 16, 1024);
      const uint64_t d_p = umma_desc_sw128(p_addr, 16, 1024);
      bool ok = await(&bars->x_full, 0, status);
      // Two queues served in whatever order their inputs arrive: S'/dP' of tile s_next needs its streamed tile
      // and a free TMEM stage; the accumulation of tile a_next needs the P'/dS' tiles the threads wrote.  A fixed
      // order would let a streamed tile that is still in flight hold back the accumulation that frees the
      // shared-memory stage the next load is waiting for.
      int s_next = 0, a_next = 0;
      uint32_t idle = 0;
      while (a_next < n_iter && ok) {
        bool progressed = false;
        if (a_next < s_next && mbar_test_wait(&bars->t_full, a_next & 1)) {
          const int jt = a_next;
          const int st = jt % L::Y_STAGES;
          tc_fence_after();
          const uint64_t dy1 = umma_desc_sw128(smem_u32(smem + L::Y_OFF + L::y_off(st, 0, 0)), L::HALF_STRIDE, 1024);
          const uint64_t dy2 = umma_desc_sw128(smem_u32(smem + L::Y_OFF + L::y_off(st, 1, 0)), L::HALF_STRIDE, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {   // contraction over the 64 streamed rows
            umma_bf16_ss(tmem_acc1, d_ds + (ks * 32 >> 4), dy1 + (ks * 2048 >> 4), idesc_acc,
                         (jt > 0 || ks > 0) ? 1u : 0u);
          }
          if (MODE == 1) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              umma_bf16_ss(tmem_acc2, d_p + (ks * 32 >> 4), dy2 + (ks * 2048 >> 4), idesc_acc,
                           (jt > 0 || ks > 0) ? 1u : 0u);
            }
          }
          umma_commit(&bars->t_empty);
          umma_commit(&bars->y_empty[st]);
          if (jt == n_iter - 1) umma_commit(&bars->acc_full);
          ++a_next;
          progressed = true;
        }
        if (s_next < n_iter) {
          const int it = s_next;
          const int st = it % L::Y_STAGES;
          const int ss = it & 1;
          if (mbar_test_wait(&bars->y_full[st], (it / L::Y_STAGES) & 1) &&
              mbar_test_wait(&bars->s_empty[ss], ((it >> 1) & 1) ^ 1)) {
            tc_fence_after();
            const uint32_t y1 = smem_u32(smem + L::Y_OFF + L::y_off(st, 0, 0));
            const uint32_t y2 = smem_u32(smem + L::Y_OFF + L::y_off(st, 1, 0));
            constexpr uint32_t idesc = idesc_s;
            // one descriptor per operand and tile; the k-steps only add a constant to its address field (the
            // issuing thread's instruction count per MMA is what bounds this loop)
            const uint64_t dy1 = umma_desc_sw128(y1, 16, 1024);
            const uint64_t dy2 = umma_desc_sw128(y2, 16, 1024);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              const uint32_t yo = (ks / 4) * L::HALF_STRIDE + (ks % 4) * 32;
              umma_bf16_ss(tmem_base + ss * 64, dx1[ks], dy1 + (yo >> 4), idesc, ks > 0 ? 1u : 0u);
            }
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              const uint32_t yo = (ks / 4) * L::HALF_STRIDE + (ks % 4) * 32;
              umma_bf16_ss(tmem_base + 128 + ss * 64, dx2[ks], dy2 + (yo >> 4), idesc, ks > 0 ? 1u : 0u);
            }
            umma_commit(&bars->s_full[ss]);
            ++s_next;
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > kMaxMbarPolls) {
          atomicCAS(status, 0, kStatusMbarTimeout);
          ok = false;
        } else if ((idle & 1023u) == 0 && *reinterpret_cast<volatile int*>(status) != 0) {
          ok = false;
        }
      }
    }
  } else {
    // ------------------------------------------- P' / dS' tiles + epilogue
    // A warp reaches the TMEM lanes 32*(warp % 4)..+31; the two groups take columns [0,32) and [32,64).
    const int wg = warp >= 6 ? 1 : 0;
    const int row = (warp & 3) * 32 + lane;   // stationary row == TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int xpos = xb * 128 + row;   // position of this row inside the sequence
    float row_lse = 0.f, row_delta = 0.f;
    if (MODE == 0) {
      const long long idx = (static_cast<long long>(b) * Hq + hy) * S + xpos;
      row_lse = lse[idx] * 1.4426950408889634f;
      row_delta = delta[idx];
    }
    float pre_lse = 0.f, pre_delta = 0.f;      // MODE 1: this thread's lse/delta entries of the next streamed tile
    if (MODE == 1 && wg == 0 && row < 64 && n_iter > 0) {
      const long long idx = (static_cast<long long>(b) * Hq + g * group) * S + 2 * xb * 64 + row;
      pre_lse = lse[idx];
      pre_delta = delta[idx];
    }
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it & 1;
      // lse/delta vectors: three stages, so a stage is rewritten only after every thread has left the
      // iteration that read it (a thread enters iteration it only after the MMAs of it - 2 have retired)
      const int vs = it % 3;
      const int ti = (MODE == 0) ? it : 2 * xb + it % tiles_per_head;
      if (MODE == 1) {
        // Per-column lse/delta of the streamed query tile -> shared memory.  The values of the next tile are
        // requested right away and stay in flight while this tile is processed.
        if (wg == 0 && row < 64) {
          vec[vs * 128 + row] = pre_lse * 1.4426950408889634f;
          vec[vs * 128 + 64 + row] = pre_delta;
          warp_arrive(&bars->v_full[st], lane);
          if (it + 1 < n_iter) {
            const int hn = g * group + (it + 1) / tiles_per_head;
            const int tn = 2 * xb + (it + 1) % tiles_per_head;
            const long long idx = (static_cast<long long>(b) * Hq + hn) * S + tn * 64 + row;
            pre_lse = lse[idx];            // no arithmetic on these until the next iteration: a dependent
            pre_delta = delta[idx];        // instruction here would stall this warp on the loads right away
          }
        }
        // Bounded wait instead of a named barrier: a thread that gave up on
        // an earlier wait must not strand the others here.
        if (!await_all(&bars->v_full[st], (it >> 1) & 1, status)) { ok = false; break; }
      }
      if (!await_all(&bars->s_full[st], (it >> 1) & 1, status)) { ok = false; break; }
      tc_fence_after();
      // Causal mask is needed only where the streamed tile overlaps the
      // stationary rows: element (x row, y col) is kept iff key <= query.
      const int ypos0 = ti * 64;
      const bool need_mask = (MODE == 0) ? (ypos0 + 63 > xb * 128) : (ypos0 < xb * 128 + 127);
      const uint32_t ts = tmem_base + lane_sel + st * 64;
      {
        const int c = wg;
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(ts + c * 32, sv);
        tmem_ld_32x32(ts + 128 + c * 32, dv);
        tmem_ld_wait();
        tc_fence_before();
        warp_arrive(&bars->s_empty[st], lane);   // S'/dP' of this stage now live in registers
        if (need_mask) {
          // causal mask, applied once to the registers of the tiles that cross the diagonal: a score of -inf
          // turns into a probability (and a score gradient) of exactly zero below
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            const int qpos = (MODE == 0) ? xpos : ypos0 + col;
            const int kpos = (MODE == 0) ? ypos0 + col : xpos;
            if (kpos > qpos) sv[i] = 0xff800000u;
          }
        }
        uint32_t pw[16], dw[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p[2], d[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = c * 32 + 2 * i + e;
            const float l2 = (MODE == 0) ? row_lse : vec[vs * 128 + col];
            const float dl = (MODE == 0) ? row_delta : vec[vs * 128 + 64 + col];
            const float pv = fast_exp2(__uint_as_float(sv[2 * i + e]) * scale_log2 - l2);
            p[e] = pv;
            d[e] = pv * (__uint_as_float(dv[2 * i + e]) - dl);
          }
          pw[i] = pack_bf16x2(p[0], p[1]);
          dw[i] = pack_bf16x2(d[0], d[1]);
        }
        // the tiles were last read by the MMAs of the previous iteration
        if (it >= 1 && !await_all(&bars->t_empty, (it - 1) & 1, status)) { ok = false; break; }
        if (MODE == 1) store_row_chunk_sw128(smem + L::P_OFF, row, c * 4, pw);
        store_row_chunk_sw128(smem + L::DS_OFF, row, c * 4, dw);
      }
      fence_proxy_async_smem();
      warp_arrive(&bars->t_full, lane);
    }
    if (ok && await_all(&bars->acc_full, 0, status)) {
      tc_fence_after();
      const long long tok = tok0 + xpos;
      // MODE 0 writes dQ of head hy; MODE 1 writes dK and dV of kv head g.
      __nv_bfloat16* o1 = d_qkv + tok * W + ((MODE == 0) ? hy * HD : (Hq + g) * HD);
      __nv_bfloat16* o2 = d_qkv + tok * W + (Hq + Hkv + g) * HD;
#pragma unroll 1
      for (int a = 0; a < (MODE == 0 ? 1 : 2); ++a) {
        const uint32_t ta = (a == 0 ? tmem_acc1 : tmem_acc2) + lane_sel;
        __nv_bfloat16* orow = (a == 0) ? o1 : o2;
        const float sc = (a == 0) ? scale : 1.f;
#pragma unroll 1
        for (int c = wg; c < HD / 32; c += 2) {
          uint32_t r[32];
          tmem_ld_32x32(ta + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              ow[i] = pack_bf16x2(__uint_as_float(r[v * 8 + 2 * i]) * sc,
                                  __uint_as_float(r[v * 8 + 2 * i + 1]) * sc);
            reinterpret_cast<uint4*>(orow + c * 32)[v] = o;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename K>
int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess
             ? 0
             : -2;
}

}  // namespace

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

int attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int Hq, int Hkv, int hd,
             float softmax_scale, int* status, cudaStream_t st) {
  if (S % 128 != 0 || Hq % Hkv != 0 || (hd != 64 && hd != 128)) return -1;
  if (B == 0) return 0;
  const long long T = static_cast<long long>(B) * S;
  const uint64_t W = static_cast<uint64_t>(Hq + 2 * Hkv) * hd;
  CUtensorMap tm;
  int rc = make_tmap_2d_bf16(&tm, qkv, W, T, W * 2, 64, 128);
  if (rc != 0) return rc;
  const float scale_log2 = softmax_scale * 1.4426950408889634f;
  dim3 grid(S / 128, Hq, B);
  if (hd == 128) {
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_kernel<128>, FwdSmem<128>::TOTAL)) return -2; cfg = true; }
    attn_fwd_kernel<128><<<grid, FWD_THREADS, FwdSmem<128>::TOTAL, st>>>(
        tm, static_cast<__nv_bfloat16*>(out), lse, S, Hq, Hkv, scale_log2, status);
  } else {
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_kernel<64>, FwdSmem<64>::TOTAL)) return -2; cfg = true; }
    attn_fwd_kernel<64><<<grid, FWD_THREADS, FwdSmem<64>::TOTAL, st>>>(
        tm, static_cast<__nv_bfloat16*>(out), lse, S, Hq, Hkv, scale_log2, status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Side stream and the two events that fork the dK/dV kernel off a caller's stream and join it again; one set
// per (device, caller stream), created on first use and kept for the life of the process.
struct BwdFork {
  cudaStream_t side = nullptr;
  cudaEvent_t ready = nullptr, done = nullptr;
};

static bool bwd_fork(cudaStream_t st, BwdFork* out) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, BwdFork> forks;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(mu);
  auto it = forks.find({dev, st});
  if (it == forks.end()) {
    BwdFork f;
    int least = 0, greatest = 0;   // the long dK/dV CTAs should win SMs over the dQ CTAs queued behind them
    if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) return false;
    if (cudaStreamCreateWithPriority(&f.side, cudaStreamNonBlocking, greatest) != cudaSuccess) return false;
    if (cudaEventCreateWithFlags(&f.ready, cudaEventDisableTiming) != cudaSuccess) return false;
    if (cudaEventCreateWithFlags(&f.done, cudaEventDisableTiming) != cudaSuccess) return false;
    it = forks.emplace(std::make_pair(dev, st), f).first;
  }
  *out = it->second;
  return true;
}

template <int HD>
static int attn_bwd_impl(const void* qkv, const void* out, const void* d_out, const float* lse,
                         float* delta, void* d_qkv, int B, int S, int Hq, int Hkv, float softmax_scale,
                         int* status, cudaStream_t st) {
  const long long T = static_cast<long long>(B) * S;
  const uint64_t W = static_cast<uint64_t>(Hq + 2 * Hkv) * HD;
  const uint64_t Wo = static_cast<uint64_t>(Hq) * HD;
  CUtensorMap tqx, tqy, tdx, tdy;
  int rc;
  if ((rc = make_tmap_2d_bf16(&tqx, qkv, W, T, W * 2, 64, 128)) != 0) return rc;
  if ((rc = make_tmap_2d_bf16(&tqy, qkv, W, T, W * 2, 64, 64)) != 0) return rc;
  if ((rc = make_tmap_2d_bf16(&tdx, d_out, Wo, T, Wo * 2, 64, 128)) != 0) return rc;
  if ((rc = make_tmap_2d_bf16(&tdy, d_out, Wo, T, Wo * 2, 64, 64)) != 0) return rc;
  static bool cfg = false;
  if (!cfg) {
    if (set_smem(attn_bwd_kernel<HD, 0>, BwdSmem<HD>::TOTAL)) return -2;
    if (set_smem(attn_bwd_kernel<HD, 1>, BwdSmem<HD>::TOTAL)) return -2;
    cfg = true;
  }
  if (((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(d_out)) & 15u) != 0) return -1;
  if (T * Hq >= (1ll << 31)) return -1;
  const long long delta_blocks = (T * Hq * (HD / 8) + 255) / 256;
  attn_delta_kernel<HD><<<static_cast<unsigned>(delta_blocks < 148 * 16 ? delta_blocks : 148 * 16), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out), delta, T, S, Hq);
  const float scale_log2 = softmax_scale * 1.4426950408889634f;
  // The two gradient kernels are independent (dK/dV and dQ go to different columns of d_qkv) and each holds a
  // whole SM per CTA.  The dK/dV grid is small (S/128 x Hkv CTAs, under two waves for eight KV heads), so its last
  // wave leaves SMs idle and its longest CTA (the first key tile, visited by every query tile of its head group)
  // sets its duration.  It is launched first on a high-priority side stream and the dQ CTAs fill the idle SMs
  // (measured: 0.995 -> 0.751 ms for 32 q / 8 kv heads at S = 4096).  PIPER_ATTN_FORK=0 runs both kernels one
  // after the other on the caller's stream.
  static int use_fork = -1;
  if (use_fork < 0) {
    const char* env = getenv("PIPER_ATTN_FORK");
    use_fork = (env != nullptr && env[0] == '0') ? 0 : 1;
  }
  BwdFork fork;
  cudaStream_t kv_stream = st;
  if (use_fork) {
    if (!bwd_fork(st, &fork)) return -3;
    if (cudaEventRecord(fork.ready, st) != cudaSuccess || cudaStreamWaitEvent(fork.side, fork.ready, 0) != cudaSuccess)
      return -3;
    kv_stream = fork.side;
  }
  attn_bwd_kernel<HD, 1><<<dim3(S / 128, Hkv, B), BWD_THREADS, BwdSmem<HD>::TOTAL, kv_stream>>>(
      tqx, tqy, tdx, tdy, lse, delta, static_cast<__nv_bfloat16*>(d_qkv), S, Hq, Hkv, softmax_scale,
      scale_log2, status);
  const bool kv_ok = cudaGetLastError() == cudaSuccess;
  if (use_fork && cudaEventRecord(fork.done, fork.side) != cudaSuccess) return -3;
  attn_bwd_kernel<HD, 0><<<dim3(S / 128, Hq, B), BWD_THREADS, BwdSmem<HD>::TOTAL, st>>>(
      tqx, tqy, tdx, tdy, lse, delta, static_cast<__nv_bfloat16*>(d_qkv), S, Hq, Hkv, softmax_scale,
      scale_log2, status);
  const bool q_ok = cudaGetLastError() == cudaSuccess;
  if (use_fork && cudaStreamWaitEvent(st, fork.done, 0) != cudaSuccess) return -3;   // the caller's stream owns both
  return kv_ok && q_ok ? 0 : -3;
}

int attn_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta,
             void* d_qkv, int B, int S, int Hq, int Hkv, int hd, float softmax_scale, int* status,
             cudaStream_t st) {
  if (S % 128 != 0 || Hq % Hkv != 0 || (hd != 64 && hd != 128)) return -1;
  if (B == 0) return 0;
  if (hd == 128)
    return attn_bwd_impl<128>(qkv, out, d_out, lse, delta, d_qkv, B, S, Hq, Hkv, softmax_scale, status, st);
  return attn_bwd_impl<64>(qkv, out, d_out, lse, delta, d_qkv, B, S, Hq, Hkv, softmax_scale, status, st);
}

}  // namespace piper
