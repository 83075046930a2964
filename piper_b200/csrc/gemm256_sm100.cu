// Dense bf16 GEMM for sm_100a with 256x256 output tiles per CTA:
// C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation in tensor memory.
//
// Why a second tile shape: an SM reads shared-memory fills from L2 at a fixed
// width, and a 128x256 tile needs 48 KiB of operands per 64-deep k-block for
// 512 tensor-core cycles of work, which leaves the kernel bound by that port.
// A 256x256 tile needs 64 KiB per k-block for 1024 cycles of work: a third
// fewer operand bytes per flop, the ratio a two-SM tile pair would reach,
// without pairing SMs.
//
// The price is tensor memory: two 128x256 fp32 accumulators (rows 0-127 and
// 128-255 of the tile) fill all 512 columns, so there is no second
// accumulator set to run ahead into.  Instead the epilogue drains the two
// halves one after the other and frees each as soon as it is read, and the
// MMA warp starts the next tile's first half while the second half is still
// being drained; only the drain of one half (eight warps, 128 columns each)
// is exposed per tile.
//
// Roles by warp: 0 TMA producer (3-stage ring, non-multicast loads), 1 MMA
// issuer, 2 TMEM allocator, 4-11 epilogue (warp w reads TMEM lanes
// 32*(w%4)..+31, columns 128*((w-4)/4)..+127 of each half).  Tiles are handed
// out dynamically.  Operand layouts and epilogues are those of the 128x256
// kernel (gemm_sm100.cu).  All waits are bounded.
#include "gemm_sm100.h"
#include "ptx.cuh"

namespace piper {
namespace {

constexpr int BM = 256;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 32 KiB: two 128-row halves (K-major) or four 64-wide boxes (MN-major)
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int A_HALF_BYTES = 128 * BK * 2;
constexpr int MN_BOX_BYTES = 64 * BK * 2;
constexpr int NUM_THREADS = 384;
constexpr int EPI_WARPS = 8;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int C_STAGE_BYTES = 32 * 32 * 4;   // fp32 epilogue: one 32x32 block per epilogue warp
constexpr int SMEM_BYTES_F32 = STAGES * STAGE_BYTES + 1024 /*align*/ + 1024 /*barriers, padded*/ + EPI_WARPS * C_STAGE_BYTES;

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full;
  uint64_t acc_empty[2];     // one per accumulator half
  uint32_t tmem_base;
  int tile_ring[8];          // producer -> MMA warp: tile of the n-th local tile (-1: no more)
  int acc_tile[2];           // MMA warp -> epilogue, by parity of the local tile number
};

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm256_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, void* __restrict__ c_ptr, long long ldc, int M, int N,
               int K, int accumulate, int* status, int* sched) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;
  // Tiles that run at the same time should share operands: walk the dimension with fewer tiles fastest, so a
  // wave of CTAs covers all of it and the operand of the long dimension streams through L2 once.
  const bool n_fast = tiles_n < tiles_m;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->acc_full, 2);               // tcgen05.commit + the MMA thread's arrive (publishes acc_tile)
    mbar_init(&bars->acc_empty[0], EPI_WARPS);
    mbar_init(&bars->acc_empty[1], EPI_WARPS);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0, n_local = 0;
      bool ok = true;
      while (ok) {
        const int tile = sched != nullptr ? atomicAdd(&sched[0], 1)
                                          : static_cast<int>(blockIdx.x + n_local * gridDim.x);
        const bool none_left = tile >= num_tiles;
        bars->tile_ring[n_local & 7] = none_left ? -1 : tile;
        if (none_left) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (mbar_wait(&bars->empty[s], ph ^ 1, status)) mbar_arrive(&bars->full[s]);   // end marker, no bytes
          break;
        }
        const int m0 = (n_fast ? tile / tiles_n : tile % tiles_m) * BM;
        const int n0 = (n_fast ? tile % tiles_n : tile / tiles_m) * BN;
        ++n_local;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, status)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_arrive_expect_tx(&bars->full[s], STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * MN_BOX_BYTES, &tmap_a, &bars->full[s], m0 + 64 * j, k0);
          } else {
            tma_load_2d(sa, &tmap_a, &bars->full[s], k0, m0);
            tma_load_2d(sa + A_HALF_BYTES, &tmap_a, &bars->full[s], k0, m0 + 128);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * MN_BOX_BYTES, &tmap_b, &bars->full[s], n0 + 64 * j, k0);
          } else {
            tma_load_2d(sb, &tmap_b, &bars->full[s], k0, n0);
          }
        }
      }
      if (!ok) {
        for (int s = 0; s < STAGES; ++s) {       // let the copies already issued land
          if (it <= static_cast<uint32_t>(s)) continue;
          const uint32_t fills = (it - 1 - s) / STAGES + 1;
          mbar_wait(&bars->full[s], (fills - 1) & 1, nullptr);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, BN, A_MN, B_MN);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      while (ok) {
        {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, status)) { ok = false; break; }
        }
        const int tile = *reinterpret_cast<volatile int*>(&bars->tile_ring[local_tile & 7]);
        const uint32_t acc_ph = local_tile & 1;     // each half is filled once per tile
        if (tile < 0) {
          // no more tiles: wait until the last tile is drained, then release the epilogue warps
          if (!mbar_wait(&bars->acc_empty[0], acc_ph ^ 1, status)) break;
          if (!mbar_wait(&bars->acc_empty[1], acc_ph ^ 1, status)) break;
          bars->acc_tile[local_tile & 1] = -1;
          mbar_arrive(&bars->acc_full);
          mbar_arrive(&bars->acc_full);
          break;
        }
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (kb > 0 && !mbar_wait(&bars->full[s], ph, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (kb == 0) {
              // this half of the previous tile must have been read out
              if (!mbar_wait(&bars->acc_empty[h], acc_ph ^ 1, status)) { ok = false; break; }
              tc_fence_after();
            }
            const uint32_t tmem_d = tmem_base + h * BN;
            const uint32_t sah = A_MN ? sa + h * 2 * MN_BOX_BYTES : sa + h * A_HALF_BYTES;
            // one descriptor per operand; a k-step only adds a constant to its address field
            const uint64_t da0 = A_MN ? umma_desc_sw128(sah, MN_BOX_BYTES, 1024) : umma_desc_sw128(sah, 16, 1024);
            const uint64_t db0 = B_MN ? umma_desc_sw128(sb, MN_BOX_BYTES, 1024) : umma_desc_sw128(sb, 16, 1024);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t da = da0 + ((A_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2)) >> 4);
              const uint64_t db = db0 + ((B_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2)) >> 4);
              umma_bf16_ss(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          if (ok) umma_commit(&bars->empty[s]);
        }
        if (ok) {
          bars->acc_tile[local_tile & 1] = tile;
          mbar_arrive(&bars->acc_full);      // publishes acc_tile
          umma_commit(&bars->acc_full);      // arrives when both halves are complete
        }
        ++local_tile;
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------- epilogue
    const int q = warp & 3;                     // TMEM lanes [32q, 32q + 32)
    const int ch = (warp - 4) >> 2;             // columns [128ch, 128ch + 128) of each half
    uint32_t local_tile = 0;
    for (;; ++local_tile) {
      if (!mbar_wait(&bars->acc_full, local_tile & 1, status)) break;
      const int tile = *reinterpret_cast<volatile int*>(&bars->acc_tile[local_tile & 1]);
      if (tile < 0) break;
      const int m0 = (n_fast ? tile / tiles_n : tile % tiles_m) * BM;
      const int n0 = (n_fast ? tile % tiles_n : tile / tiles_m) * BN;
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int row = m0 + h * 128 + q * 32 + lane;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * BN + ch * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col0 = n0 + ch * 128 + c * 32;
          if (row < M && col0 < N) {
            if (EPI == kEpiStoreBf16) {
              __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(c_ptr) + row * ldc + col0;
              if (col0 + 32 <= N) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  uint4 o;
                  o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                  o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                  o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                  o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                  reinterpret_cast<uint4*>(crow)[v] = o;
                }
              } else {
                #pragma unroll
                for (int j = 0; j < 32; ++j)   // constant indices keep r[] in registers
                  if (col0 + j < N) crow[j] = __float2bfloat16(__uint_as_float(r[j]));
              }
            }
          }
          if (EPI == kEpiAccumF32 && m0 + h * 128 + q * 32 < M && col0 < N) {
            // fp32 output: stage the warp's 32x32 block in shared memory (16-byte chunks XOR-swizzled by row) and
            // send it as one TMA store, or one TMA reduce-add when accumulating (see gemm_sm100.cu)
            float* cbuf = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 1024 + (warp - 4) * C_STAGE_BYTES);
            bulk_wait_group_read<0>();               // the previous block has left the buffer
            __syncwarp();
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              const float4 o = make_float4(__uint_as_float(r[4 * v + 0]), __uint_as_float(r[4 * v + 1]),
                                           __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
              reinterpret_cast<float4*>(cbuf + lane * 32)[v ^ (lane & 7)] = o;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (accumulate) tma_reduce_add_2d_bulk(&tmap_c, cbuf, col0, m0 + h * 128 + q * 32);
              else tma_store_2d_bulk(&tmap_c, cbuf, col0, m0 + h * 128 + q * 32);
              bulk_commit_group();
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->acc_empty[h]);   // the next tile may overwrite this half
      }
    }
    if (EPI == kEpiAccumF32 && lane == 0) bulk_wait_group<0>();   // staged blocks must leave before the CTA does
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (sched != nullptr && threadIdx.x == 0) {
    if (atomicAdd(&sched[1], 1) == static_cast<int>(gridDim.x) - 1) {   // last CTA rearms the scheduler slot
      sched[0] = 0;
      sched[1] = 0;
      __threadfence();
    }
  }
}

template <bool A_MN, bool B_MN, int EPI>
int launch256(const GemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb, int num_sms, int* sched,
              cudaStream_t stream) {
  auto kern = gemm256_kernel<A_MN, B_MN, EPI>;
  constexpr int smem_bytes = EPI == kEpiAccumF32 ? SMEM_BYTES_F32 : SMEM_BYTES;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -2;
    configured = true;
  }
  CUtensorMap tc = ta;      // unused by the bf16 epilogue
  if (EPI == kEpiAccumF32) {
    const int rc = make_tmap_c_f32(&tc, g.c, g.N, g.M, static_cast<uint64_t>(g.ldc) * 4);
    if (rc != 0) return rc;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(ta, tb, tc, g.c, g.ldc, g.M, g.N, g.K, g.accumulate, g.status,
                                                  sched);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

int gemm256_bf16_launch(const GemmArgs& g, int num_sms, int* sched, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return 0;
  CUtensorMap ta, tb;
  int rc;
  // K-major operand: dims {K, rows}, box {64, 128 or 256 rows}; MN-major operand: dims {rows, K}, box {64, 64}.
  rc = g.a_mn_major ? make_tmap_2d_bf16(&ta, g.a, g.M, g.K, g.lda * 2, 64, BK)
                    : make_tmap_2d_bf16(&ta, g.a, g.K, g.M, g.lda * 2, BK, 128);
  if (rc != 0) return rc;
  rc = g.b_mn_major ? make_tmap_2d_bf16(&tb, g.b, g.N, g.K, g.ldb * 2, 64, BK)
                    : make_tmap_2d_bf16(&tb, g.b, g.K, g.N, g.ldb * 2, BK, BN);
  if (rc != 0) return rc;
  const int key = (g.a_mn_major ? 4 : 0) | (g.b_mn_major ? 2 : 0) | (g.epilogue == kEpiAccumF32 ? 1 : 0);
  switch (key) {
    case 0: return launch256<false, false, kEpiStoreBf16>(g, ta, tb, num_sms, sched, stream);
    case 1: return launch256<false, false, kEpiAccumF32>(g, ta, tb, num_sms, sched, stream);
    case 2: return launch256<false, true, kEpiStoreBf16>(g, ta, tb, num_sms, sched, stream);
    case 3: return launch256<false, true, kEpiAccumF32>(g, ta, tb, num_sms, sched, stream);
    case 4: return launch256<true, false, kEpiStoreBf16>(g, ta, tb, num_sms, sched, stream);
    case 5: return launch256<true, false, kEpiAccumF32>(g, ta, tb, num_sms, sched, stream);
    case 6: return launch256<true, true, kEpiStoreBf16>(g, ta, tb, num_sms, sched, stream);
    default: return launch256<true, true, kEpiAccumF32>(g, ta, tb, num_sms, sched, stream);
  }
}

}  // namespace piper
