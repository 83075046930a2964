// ZeRO-3 all-gather fused into the GEMM that consumes the gathered weight
// (sm_100a): Y[M, N] = X[M, K] * W[N, K]^T where W is sharded by rows over
// the data-parallel group, rank p holding rows [p*R, (p+1)*R) in symmetric
// memory (R a multiple of 64).
//
// Same pipeline as the dense kernel (persistent CTAs, TMA producer warp,
// single-thread tcgen05.mma issuer, two TMEM accumulators, four epilogue
// warps) plus a gather warp per CTA.
//
// Gathered mode (a local full-size buffer is given): the gather warps of all
// CTAs together pull every remote 64-row x 64-column weight box exactly once
// over NVLink - a TMA load from the owner's shard into shared memory and a
// TMA store into the local full buffer, several boxes in flight per CTA - and
// count finished boxes per 256-row weight block in global memory.  Boxes are
// handed out through one atomic counter in the order the GEMM needs them.
// The GEMM walks weight blocks starting with the ones this rank owns (read
// straight from its shard), so the tensor cores are busy while the first
// remote blocks arrive; before it loads a block with remote rows the
// producer waits, bounded, for that block's counter.  After all remote boxes
// the gather warps copy the local shard into the full buffer as well, which
// the backward GEMMs then read from local HBM.
//
// Direct mode (no full buffer): every weight box is loaded by TMA from the
// shard of its owner by each CTA that needs it.
//
// All TMA loads are ordinary (non-multicast) loads.
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
constexpr int GATHER_BUFS = 4;                 // 8 KiB boxes staged per CTA; GATHER_BUFS - 1 loads in flight
constexpr int GATHER_AHEAD = GATHER_BUFS - 1;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + GATHER_BUFS * BOX_BYTES + 1024 + 256;
constexpr uint32_t kMaxReadyPolls = 1u << 20;  // x (100 ns sleep + one load): gives up after about a second

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t g_full[GATHER_BUFS];
  uint32_t tmem_base;
  int g_block[16];           // weight block of the gather chunk in flight (-1: local copy, not counted)
};

// Geometry shared by the producer and the gather warp.
struct Geo {
  int N, rows_per_shard, num_peers, me, tiles_n, k_blocks, first_block;
  __device__ int owner(int row) const {
    const int p = row / rows_per_shard;
    return p < num_peers ? p : num_peers - 1;
  }
  // position in the walk over weight blocks (own blocks first) -> block index
  __device__ int block_at(int pos) const { return (first_block + pos) % tiles_n; }
  // number of gather chunks the producer has to wait for before it may read this block from the full buffer
  __device__ int needed(int nb) const {
    int boxes = 0;
    for (int j = 0; j < BN / 64; ++j) {
      const int row = nb * BN + 64 * j;
      if (row < N && owner(row) != me) ++boxes;
    }
    return boxes * k_blocks;
  }
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

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ PeerMaps peers,
               const __grid_constant__ CUtensorMap tmap_full, __nv_bfloat16* __restrict__ c, long long ldc, int M,
               int N, int K, int rows_per_shard, int num_peers, int me, int gathered, int* scratch, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES + GATHER_BUFS * BOX_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;
  uint8_t* gbuf = smem + STAGES * STAGE_BYTES;             // gather staging boxes (1024-byte aligned)
  Geo geo;
  geo.N = N; geo.rows_per_shard = rows_per_shard; geo.num_peers = num_peers; geo.me = me;
  geo.tiles_n = tiles_n; geo.k_blocks = k_blocks;
  geo.first_block = gathered ? (me * rows_per_shard) / BN % tiles_n : 0;
  int* gather_next = scratch;            // [0]: next gather chunk
  int* ready = scratch + 2;              // [2 + block]: gathered chunks of that weight block

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < GATHER_BUFS; ++b) mbar_init(&bars->g_full[b], 1);
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
        const int nb = geo.block_at(tile / tiles_m);
        const int n0 = nb * BN;
        if (gathered) {
          // rows of other ranks are read from the local full buffer once the gather warps have delivered them
          const int need = geo.needed(nb);
          if (need > 0) {
            uint32_t polls = 0;
            while (ld_acquire_gpu(ready + nb) < need) {
              if (++polls > kMaxReadyPolls || ((polls & 255u) == 0 && *reinterpret_cast<volatile int*>(status) != 0)) {
                atomicCAS(status, 0, kStatusPeerTimeout);
                ok = false;
                break;
              }
              __nanosleep(100);
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy flag read -> async-proxy tile loads
          }
        }
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
            if (gathered && (p != me || row >= N))
              tma_load_2d(sb + j * BOX_BYTES, &tmap_full, &bars->full[s], kb * BK, row);
            else
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
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // four 64-row boxes stacked: rows of box j start 8192 B after box j-1, i.e. 8-row groups stay
            // 1024 B apart across the whole 256-row tile
            umma_bf16_ss(tmem_d, umma_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024),
                         umma_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------ gather warp
    if (lane == 0 && gathered) {
      // Chunk c = (64-row box, k-block).  Boxes of other ranks come first, in the order the GEMM reaches them
      // (the circular range that starts right after this rank's rows), then this rank's own boxes.
      const int total_boxes = (N + 63) / 64;
      int my_first = me * rows_per_shard / 64;
      if (my_first > total_boxes) my_first = total_boxes;
      int my_last = ((me + 1) * rows_per_shard < N ? (me + 1) * rows_per_shard : N);
      my_last = (my_last + 63) / 64;
      const int my_count = my_last > my_first ? my_last - my_first : 0;
      const int remote_boxes = total_boxes - my_count;
      const int total = total_boxes * k_blocks;
      constexpr int PENDING = 3;             // stores that may still be in flight when the next one is issued
      uint32_t n = 0;                        // chunks whose load has been issued
      uint32_t stored = 0, counted = 0;      // chunks whose store has been issued / whose arrival has been counted
      int src_x[GATHER_BUFS] = {0, 0, 0, 0}, src_row[GATHER_BUFS] = {0, 0, 0, 0};
      bool ok = true;
      auto store_chunk = [&](uint32_t i) -> bool {
        const int b = i % GATHER_BUFS;
        if (!mbar_wait(&bars->g_full[b], (i / GATHER_BUFS) & 1, status)) return false;
        tma_store_2d(&tmap_full, gbuf + b * BOX_BYTES, src_x[b], src_row[b]);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        return true;
      };
      auto count_upto = [&](uint32_t end) {   // stores [counted, end) are complete: publish them
        if (end <= counted) return;
        asm volatile("fence.proxy.async;" ::: "memory");       // async-proxy stores -> generic-proxy counters
        __threadfence();
        for (; counted < end; ++counted) {
          const int nb = bars->g_block[counted & 15];
          if (nb >= 0) atomicAdd(ready + nb, 1);
        }
      };
      int c = atomicAdd(gather_next, 1);
      while (ok && c < total) {
        if (*reinterpret_cast<volatile int*>(status) != 0) { ok = false; break; }
        const int next_c = atomicAdd(gather_next, 1);   // claimed now, used next trip: its latency is hidden
        const int bi = c / k_blocks;
        const int kb = c - bi * k_blocks;
        const bool remote = bi < remote_boxes;
        const int box = remote ? (my_first + my_count + bi) % total_boxes : my_first + (bi - remote_boxes);
        const int row = box * 64;
        const int p = geo.owner(row);
        const int b = n % GATHER_BUFS;
        // the store that last used this buffer (issued one trip ago) must have read it before it is overwritten
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        src_x[b] = kb * BK;
        src_row[b] = row;
        bars->g_block[n & 15] = remote ? row / BN : -1;
        mbar_arrive_expect_tx(&bars->g_full[b], BOX_BYTES);
        tma_load_2d(gbuf + b * BOX_BYTES, &peers.m[p], &bars->g_full[b], kb * BK, row - p * rows_per_shard);
        ++n;
        if (n > GATHER_AHEAD) {
          if (!store_chunk(stored)) { ok = false; break; }
          ++stored;
          if (stored > PENDING) {
            asm volatile("cp.async.bulk.wait_group %0;" ::"n"(PENDING) : "memory");
            count_upto(stored - PENDING);
          }
        }
        c = next_c;
      }
      // drain: chunks [stored, n) still sit in shared memory (or are on their way into it)
      for (uint32_t i = stored; i < n; ++i) {
        if (ok && store_chunk(i)) {
          stored = i + 1;
        } else {
          ok = false;
          mbar_wait(&bars->g_full[i % GATHER_BUFS], (i / GATHER_BUFS) & 1, nullptr);   // let the load land
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (ok) count_upto(stored);
    }
  } else if (warp >= 4) {
    const int ew = warp - 4;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const int m0 = (tile % tiles_m) * BM;
      const int n0 = geo.block_at(tile / tiles_m) * BN;
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
            #pragma unroll
                for (int j = 0; j < 32; ++j)   // constant indices keep r[] in registers
                  if (col0 + j < N) crow[j] = __float2bfloat16(__uint_as_float(r[j]));
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
  if (g.my_index < 0 || g.my_index >= g.num_peers) return -1;
  if (static_cast<long long>(g.num_peers) * g.rows_per_shard < g.N) return -1;
  if (g.M <= 0 || g.N <= 0) return 0;
  const int tiles_n = (g.N + BN - 1) / BN;
  const bool gathered = g.w_full != nullptr;
  if (gathered && (g.scratch == nullptr || g.scratch_ints < tiles_n + 2)) return -1;
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
  const void* full = gathered ? g.w_full : g.w_shards[g.my_index];
  const long long full_rows = gathered ? g.N : 1;
  if ((rc = make_tmap_2d_bf16(&tfull, full, g.K, full_rows, static_cast<uint64_t>(g.K) * 2, BK, 64)) != 0) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -2;
    configured = true;
  }
  if (gathered && cudaMemsetAsync(g.scratch, 0, sizeof(int) * (tiles_n + 2), st) != cudaSuccess) return -3;
  const int tiles = ((g.M + BM - 1) / BM) * tiles_n;
  const int grid = tiles < num_sms ? tiles : num_sms;
  ag_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, pm, tfull, static_cast<__nv_bfloat16*>(g.y), g.N, g.M,
                                                        g.N, g.K, g.rows_per_shard, g.num_peers, g.my_index,
                                                        gathered ? 1 : 0, g.scratch, g.status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper
