// ZeRO-3 all-gather fused into the GEMM that consumes the gathered weight
// (sm_100a): Y[M, N] = X[M, K] * W[N, K]^T where W is sharded by rows over
// the data-parallel group, rank p holding rows [p*R, (p+1)*R) in symmetric
// memory (R a multiple of 64).
//
// Same pipeline as the dense kernel (persistent CTAs, TMA producer warp,
// single-thread tcgen05.mma issuer, two TMEM accumulators, four epilogue
// warps).  The difference is the B operand: every 256-row weight tile is
// fetched as four 64-row TMA boxes, each straight from the shard of the rank
// that owns those rows - the local shard or a peer's over NVLink - through
// one tensor map per rank.  The loads are ordinary (non-multicast) TMA
// loads, so a remote tile crosses NVLink once per CTA that needs it while the
// tensor cores work on the previous stage.  The CTAs of the first M tile
// also store each weight box to the local full-size buffer (TMA store from
// shared memory), so the backward GEMMs of the same bucket read local HBM.
#include "gemm_sm100.h"
#include "ptx.cuh"

namespace piper {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int BOX_BYTES = 64 * BK * 2;
constexpr int NUM_THREADS = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
};

struct PeerMaps {
  CUtensorMap m[kMaxPeers];
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ PeerMaps peers,
               const __grid_constant__ CUtensorMap tmap_full, __nv_bfloat16* __restrict__ c, long long ldc, int M,
               int N, int K, int rows_per_shard, int num_peers, int write_through, int* status) {
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->acc_full[a], 1);
      mbar_init(&bars->acc_empty[a], 4);
    }
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM;
        const int n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, status)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_arrive_expect_tx(&bars->full[s], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &bars->full[s], kb * BK, m0);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) {
            const int row = n0 + 64 * j;
            int p = row / rows_per_shard;
            int local = row - p * rows_per_shard;
            if (p >= num_peers) {          // past the last weight row: an out-of-range box reads zeros
              p = num_peers - 1;
              local = rows_per_shard + (row - num_peers * rows_per_shard);
            }
            tma_load_2d(sb + j * BOX_BYTES, &peers.m[p], &bars->full[s], kb * BK, local);
          }
        }
      }
      if (!ok) {
        for (int s = 0; s < STAGES; ++s) {
          if (it <= static_cast<uint32_t>(s)) continue;
          const uint32_t fills = (it - 1 - s) / STAGES + 1;
          mbar_wait(&bars->full[s], (fills - 1) & 1, nullptr);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, false, false);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int m_tile = tile % tiles_m;
        const int n0 = (tile / tiles_m) * BN;
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_ph ^ 1, status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, status)) { ok = false; break; }
          tc_fence_after();
          uint8_t* sbp = smem + s * STAGE_BYTES + A_STAGE_BYTES;
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // four 64-row boxes stacked: rows of box j start 8192 B after box j-1, i.e. 8-row groups stay
            // 1024 B apart across the whole 256-row tile
            umma_bf16_ss(tmem_d, umma_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024),
                         umma_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          if (write_through && m_tile == 0) {
            // keep a local copy of the gathered weight for the backward GEMMs
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              if (n0 + 64 * j < N) tma_store_2d(&tmap_full, sbp + j * BOX_BYTES, kb * BK, n0 + 64 * j);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
      if (write_through) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else if (warp >= 4) {
    const int ew = warp - 4;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const int m0 = (tile % tiles_m) * BM;
      const int n0 = (tile / tiles_m) * BN;
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, status)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + ew * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + cc * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + cc * 32;
        if (row < M && col0 < N) {
          __nv_bfloat16* crow = c + row * ldc + col0;
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
            for (int j = 0; j < 32 && col0 + j < N; ++j) crow[j] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace

int ag_gemm_launch(const AgGemmArgs& g, int num_sms, cudaStream_t st) {
  if (g.num_peers < 1 || g.num_peers > kMaxPeers || g.rows_per_shard % 64 != 0 || g.K % 8 != 0) return -1;
  if (g.M <= 0 || g.N <= 0) return 0;
  CUtensorMap ta, tfull;
  PeerMaps pm;
  int rc;
  if ((rc = make_tmap_2d_bf16(&ta, g.x, g.K, g.M, static_cast<uint64_t>(g.K) * 2, BK, BM)) != 0) return rc;
  for (int p = 0; p < g.num_peers; ++p) {
    // the last shard may hold fewer valid rows (N not a multiple of the shard size)
    long long rows = g.N - static_cast<long long>(p) * g.rows_per_shard;
    if (rows > g.rows_per_shard) rows = g.rows_per_shard;
    if (rows < 1) rows = 1;
    if ((rc = make_tmap_2d_bf16(&pm.m[p], g.w_shards[p], g.K, rows, static_cast<uint64_t>(g.K) * 2, BK, 64)) != 0)
      return rc;
  }
  for (int p = g.num_peers; p < kMaxPeers; ++p) pm.m[p] = pm.m[0];
  const void* full = g.w_full != nullptr ? g.w_full : g.w_shards[0];
  const long long full_rows = g.w_full != nullptr ? g.N : 1;
  if ((rc = make_tmap_2d_bf16(&tfull, full, g.K, full_rows, static_cast<uint64_t>(g.K) * 2, BK, 64)) != 0) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -2;
    configured = true;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  ag_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, pm, tfull, static_cast<__nv_bfloat16*>(g.y), g.N, g.M,
                                                        g.N, g.K, g.rows_per_shard, g.num_peers,
                                                        g.w_full != nullptr ? 1 : 0, g.status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper
