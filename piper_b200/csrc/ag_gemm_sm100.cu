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
// CTAs together copy every remote weight byte exactly once over NVLink - the
// shards and the gathered weight are contiguous, so this is a flat copy in
// pieces of up to 8 KiB: a bulk load from the owner's shard into shared
// memory and a bulk store into the local full buffer, several pieces in
// flight per CTA - and count finished pieces per 256-row weight block in
// global memory.  Pieces are handed out through one atomic counter in the
// order the GEMM needs them.
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

// Geometry shared by the producer and the gather warp.  The gathered weight and every shard are contiguous
// row-major memory, so the gather is a flat copy in pieces of `piece` bytes (a power of two that divides both a
// shard and a 256-row weight block, so no piece straddles either).
struct Geo {
  int N, rows_per_shard, num_peers, me, tiles_n, k_blocks, first_block;
  long long total_bytes, shard_bytes, block_bytes, my_lo, my_hi;   // byte ranges inside the gathered weight
  int piece;
  // position in the walk over weight blocks (own blocks first) -> block index
  __device__ int block_at(int pos) const { return (first_block + pos) % tiles_n; }
  __device__ long long pieces_in(long long lo, long long hi) const { return hi > lo ? (hi - lo + piece - 1) / piece : 0; }
  // number of gathered pieces the producer has to wait for before it may read this block from the full buffer
  __device__ int needed(int nb) const {
    const long long lo = nb * block_bytes;
    const long long hi = lo + block_bytes < total_bytes ? lo + block_bytes : total_bytes;
    const long long before_hi = hi < my_lo ? hi : my_lo;      // part of the block below this rank's rows
    const long long after_lo = lo > my_hi ? lo : my_hi;       // part of the block above this rank's rows
    return static_cast<int>(pieces_in(lo, before_hi) + pieces_in(after_lo, hi));
  }
};

struct ShardPtrs {
  const uint8_t* p[kMaxPeers];
};

struct PeerMaps {
  CUtensorMap m[kMaxPeers];
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ PeerMaps peers,
               const __grid_constant__ CUtensorMap tmap_full, __nv_bfloat16* __restrict__ c, long long ldc, int M,
               int N, int K, int rows_per_shard, int num_peers, int me, int gathered, int* scratch, int* status,
               const __grid_constant__ ShardPtrs shards, uint8_t* __restrict__ w_full, int piece) {
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
  geo.total_bytes = static_cast<long long>(N) * K * 2;
  geo.shard_bytes = static_cast<long long>(rows_per_shard) * K * 2;
  geo.block_bytes = static_cast<long long>(BN) * K * 2;
  geo.my_lo = geo.shard_bytes * me < geo.total_bytes ? geo.shard_bytes * me : geo.total_bytes;
  geo.my_hi = geo.shard_bytes * (me + 1) < geo.total_bytes ? geo.shard_bytes * (me + 1) : geo.total_bytes;
  geo.piece = piece;
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
        // where each of the tile's four 64-row weight boxes comes from (worked out once per tile: the k loop
        // below has to issue a stage every few hundred cycles)
        const CUtensorMap* bmap[BN / 64];
        int brow[BN / 64];
#pragma unroll
        for (int j = 0; j < BN / 64; ++j) {
          const int row = n0 + 64 * j;
          int p = row / rows_per_shard;
          int local = row - p * rows_per_shard;
          if (p >= num_peers) {          // past the last weight row: an out-of-range box reads zeros
            p = num_peers - 1;
            local = rows_per_shard + (row - num_peers * rows_per_shard);
          }
          const bool from_full = gathered && (p != me || row >= N);
          bmap[j] = from_full ? &tmap_full : &peers.m[p];
          brow[j] = from_full ? row : local;
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
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(sb + j * BOX_BYTES, bmap[j], &bars->full[s], kb * BK, brow[j]);
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
      // Piece c of the flat copy: first the bytes above this rank's rows, then the bytes below them (the order in
      // which the GEMM reaches the blocks), last this rank's own rows.  Large contiguous bulk copies keep the
      // NVLink requests long.
      // remote bytes in the circular order that starts at the GEMM's first block: [start, my_lo) (non-empty
      // only when that block straddles the start of this rank's rows), [my_hi, end), [0, start); then own rows
      const long long start = geo.first_block * geo.block_bytes < geo.my_lo ? geo.first_block * geo.block_bytes : geo.my_lo;
      const long long seg_lo[4] = {start, geo.my_hi, 0, geo.my_lo};
      const long long seg_hi[4] = {geo.my_lo, geo.total_bytes, start, geo.my_hi};
      long long seg_first[5];
      seg_first[0] = 0;
      for (int i = 0; i < 4; ++i) seg_first[i + 1] = seg_first[i] + geo.pieces_in(seg_lo[i], seg_hi[i]);
      const long long total = seg_first[4];
      constexpr int PENDING = 3;             // stores that may still be in flight when the next one is issued
      uint32_t n = 0;                        // pieces whose load has been issued
      uint32_t stored = 0, counted = 0;      // pieces whose store has been issued / whose arrival has been counted
      long long dst_off[GATHER_BUFS] = {0, 0, 0, 0};
      uint32_t len[GATHER_BUFS] = {0, 0, 0, 0};
      bool ok = true;
      auto store_piece = [&](uint32_t i) -> bool {
        const int b = i % GATHER_BUFS;
        if (!mbar_wait(&bars->g_full[b], (i / GATHER_BUFS) & 1, status)) return false;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(w_full + dst_off[b]),
                     "r"(smem_u32(gbuf + b * BOX_BYTES)), "r"(len[b])
                     : "memory");
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
      long long c = atomicAdd(gather_next, 1);
      while (ok && c < total) {
        if (*reinterpret_cast<volatile int*>(status) != 0) { ok = false; break; }
        const long long next_c = atomicAdd(gather_next, 1);   // claimed now, used next trip: its latency is hidden
        int seg = 0;
        while (seg < 3 && c >= seg_first[seg + 1]) ++seg;
        const long long off = seg_lo[seg] + (c - seg_first[seg]) * piece;
        const long long end = seg_hi[seg];
        const bool remote = seg < 3;
        const uint32_t bytes = static_cast<uint32_t>(end - off < piece ? end - off : piece);
        const int p = static_cast<int>(off / geo.shard_bytes);
        const int b = n % GATHER_BUFS;
        // the store that last used this buffer (issued one trip ago) must have read it before it is overwritten
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        dst_off[b] = off;
        len[b] = bytes;
        bars->g_block[n & 15] = remote ? static_cast<int>(off / geo.block_bytes) : -1;
        mbar_arrive_expect_tx(&bars->g_full[b], bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(gbuf + b * BOX_BYTES)), "l"(shards.p[p] + (off - p * geo.shard_bytes)), "r"(bytes),
                     "r"(smem_u32(&bars->g_full[b]))
                     : "memory");
        ++n;
        if (n > GATHER_AHEAD) {
          if (!store_piece(stored)) { ok = false; break; }
          ++stored;
          if (stored > PENDING) {
            asm volatile("cp.async.bulk.wait_group %0;" ::"n"(PENDING) : "memory");
            count_upto(stored - PENDING);
          }
        }
        c = next_c;
      }
      // drain: pieces [stored, n) still sit in shared memory (or are on their way into it)
      for (uint32_t i = stored; i < n; ++i) {
        if (ok && store_piece(i)) {
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
  // gather piece: the largest power of two up to 8 KiB that divides a shard and a 256-row block
  const long long shard_bytes = static_cast<long long>(g.rows_per_shard) * g.K * 2;
  const long long block_bytes = static_cast<long long>(BN) * g.K * 2;
  int piece = BOX_BYTES;
  while (piece > 16 && (shard_bytes % piece != 0 || block_bytes % piece != 0)) piece >>= 1;
  ShardPtrs sp;
  for (int p = 0; p < kMaxPeers; ++p)
    sp.p[p] = static_cast<const uint8_t*>(g.w_shards[p < g.num_peers ? p : 0]);
  const int tiles = ((g.M + BM - 1) / BM) * tiles_n;
  const int grid = tiles < num_sms ? tiles : num_sms;
  ag_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, pm, tfull, static_cast<__nv_bfloat16*>(g.y), g.N, g.M,
                                                        g.N, g.K, g.rows_per_shard, g.num_peers, g.my_index,
                                                        gathered ? 1 : 0, g.scratch, g.status, sp,
                                                        static_cast<uint8_t*>(g.w_full), piece);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace piper
