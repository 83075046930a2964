// Dense bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T with fp32
// accumulation in tensor memory.
//
// One persistent CTA per SM walks 128x256 output tiles.  Roles by warp:
//   warp 0      TMA producer: fills a 4-stage shared-memory ring with
//               128-byte-swizzled operand tiles (cp.async.bulk.tensor, no
//               multicast).
//   warp 1      MMA issuer: one lane issues tcgen05.mma (128x256x16) into one
//               of two 256-column TMEM accumulators and commits to mbarriers.
//   warp 2      TMEM allocator / deallocator.
//   warps 4-7   epilogue: tcgen05.ld the finished accumulator (32 lanes per
//               warp), convert and store, while the MMA warp already works on
//               the next tile in the other accumulator.
//
// Each operand can be K-major (contraction index contiguous in memory) or
// MN-major (row index contiguous), which covers forward (X W^T), input
// gradient (dY W) and weight gradient (dY^T X) of a linear layer without any
// transposed copy.  The epilogue either stores bf16 or adds into an fp32
// buffer (gradient accumulation into the flat fp32 bucket).
//
// All mbarrier waits are bounded; on expiry the kernel records a status code,
// drains its TMA copies, frees TMEM and returns.
#include "gemm_sm100.h"

#include <cstdlib>

#include "ptx.cuh"

namespace piper {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int ACC_BUFS = 2;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int MN_BOX_BYTES = 64 * BK * 2;    // one MN-major TMA box: 64 k-rows x 128 B
constexpr int NUM_THREADS = 256;
constexpr int C_STAGE_BYTES = 32 * 32 * 4;   // fp32 epilogue: one 32x32 block per warp, two buffers per warp
constexpr int C_STAGING_BYTES = 4 * 2 * C_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int SMEM_BYTES_F32 = STAGES * STAGE_BYTES + 1024 /*align*/ + 1024 /*barriers, padded*/ + C_STAGING_BYTES;

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[ACC_BUFS];
  uint64_t acc_empty[ACC_BUFS];
  uint32_t tmem_base;
  int tile_ring[8];          // producer -> MMA warp: tile index of the n-th local tile (-1 = no more tiles)
  int acc_tile[ACC_BUFS];    // MMA warp -> epilogue: tile index held by each accumulator (-1 = no more tiles)
};

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
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
    for (int a = 0; a < ACC_BUFS; ++a) {
      mbar_init(&bars->acc_full[a], 2);    // tcgen05.commit + the MMA thread's own arrive (publishes acc_tile)
      mbar_init(&bars->acc_empty[a], 4);   // one arrive per epilogue warp
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, ACC_BUFS * BN);
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
        // Tiles are handed out dynamically (one atomic per tile) so that a CTA that reaches the SM late,
        // or shares the GPU with communication kernels, simply processes fewer tiles.
        const int tile = sched != nullptr ? atomicAdd(&sched[0], 1)
                                          : static_cast<int>(blockIdx.x + n_local * gridDim.x);
        const bool none_left = tile >= num_tiles;
        bars->tile_ring[n_local & 7] = none_left ? -1 : tile;
        if (none_left) {
          // pass the end marker to the MMA warp through the next stage's barrier (no bytes expected)
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (mbar_wait(&bars->empty[s], ph ^ 1, status)) mbar_arrive(&bars->full[s]);
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
        // Unwinding: let the copies already issued land before the CTA (and
        // its shared memory) goes away.  Stage s was last filled by iteration
        // it_s = largest value < it congruent to s.
        for (int s = 0; s < STAGES; ++s) {
          if (it <= static_cast<uint32_t>(s)) continue;
          const uint32_t fills = (it - 1 - s) / STAGES + 1;
          mbar_wait(&bars->full[s], (fills - 1) & 1, nullptr);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      while (ok) {
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        // the first stage of a tile also tells which tile it is
        {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, status)) { ok = false; break; }
        }
        const int tile = *reinterpret_cast<volatile int*>(&bars->tile_ring[local_tile & 7]);
        if (!mbar_wait(&bars->acc_empty[acc], acc_ph ^ 1, status)) { ok = false; break; }
        if (tile < 0) {
          // no more tiles: release the epilogue warps (both arrivals of the accumulator barrier)
          bars->acc_tile[acc] = -1;
          mbar_arrive(&bars->acc_full[acc]);
          mbar_arrive(&bars->acc_full[acc]);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (kb > 0 && !mbar_wait(&bars->full[s], ph, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          // one descriptor per operand and stage; a k-step only adds a constant to its address field, which
          // keeps the issuing thread's instruction count per MMA low
          const uint64_t da0 = A_MN ? umma_desc_sw128(sa, MN_BOX_BYTES, 1024) : umma_desc_sw128(sa, 16, 1024);
          const uint64_t db0 = B_MN ? umma_desc_sw128(sb, MN_BOX_BYTES, 1024) : umma_desc_sw128(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = da0 + ((A_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2)) >> 4);
            const uint64_t db = db0 + ((B_MN ? k * (UMMA_K * 128) : k * (UMMA_K * 2)) >> 4);
            umma_bf16_ss(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);       // frees the smem stage when the MMAs retire
        }
        if (ok) {
          bars->acc_tile[acc] = tile;
          mbar_arrive(&bars->acc_full[acc]);  // publishes acc_tile
          umma_commit(&bars->acc_full[acc]);  // arrives when the accumulator is complete
        }
        ++local_tile;
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------- epilogue
    const int ew = warp - 4;                  // == warp % 4: TMEM lanes [32*ew, 32*ew+32)
    uint32_t local_tile = 0;
    bool ok = true;
    for (;; ++local_tile) {
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, status)) { ok = false; break; }
      const int tile = *reinterpret_cast<volatile int*>(&bars->acc_tile[acc]);
      if (tile < 0) break;
      const int m0 = (n_fast ? tile / tiles_n : tile % tiles_m) * BM;
      const int n0 = (n_fast ? tile % tiles_n : tile / tiles_m) * BN;
      tc_fence_after();
      const int row = m0 + ew * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
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
        if (EPI == kEpiAccumF32 && m0 + ew * 32 < M && col0 < N) {
          // fp32 output: the warp's 32x32 block goes through shared memory (128-byte rows, 16-byte chunks
          // XOR-swizzled by row so that the 32 row-writes of one instruction spread over all banks) and leaves
          // as one TMA store, or one TMA reduce-add when accumulating: C is never read into the SM, the stores
          // are full lines, and the tensor map clips ragged edges.
          float* cbuf = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 1024 +
                                                 (ew * 2 + (c & 1)) * C_STAGE_BYTES);
          bulk_wait_group_read<1>();               // the store that last used this buffer has read it
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
            if (accumulate) tma_reduce_add_2d_bulk(&tmap_c, cbuf, col0, m0 + ew * 32);
            else tma_store_2d_bulk(&tmap_c, cbuf, col0, m0 + ew * 32);
            bulk_commit_group();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
    }
    if (EPI == kEpiAccumF32 && lane == 0) bulk_wait_group<0>();   // staged blocks must leave before the CTA does
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, ACC_BUFS * BN);
  }
  if (sched != nullptr && threadIdx.x == 0) {
    // the last CTA to leave rearms the scheduler slot for its next use
    if (atomicAdd(&sched[1], 1) == static_cast<int>(gridDim.x) - 1) {
      sched[0] = 0;
      sched[1] = 0;
      __threadfence();
    }
  }
}

// Pool of tile-scheduler slots (next tile, finished CTAs), one slot per launch in rotation.  It is the only
// device memory this library allocates by itself: 32 KiB, once per process.
constexpr int kSchedSlots = 4096;

int* next_sched_slot() {
  static int* pool = nullptr;
  static unsigned long long counter = 0;
  static bool disabled = false;
  if (disabled) return nullptr;
  if (pool == nullptr) {
    const char* env = getenv("PIPER_GEMM_STATIC_TILES");
    if (env != nullptr && env[0] == '1') {
      disabled = true;
      return nullptr;
    }
    if (cudaMalloc(&pool, kSchedSlots * 2 * sizeof(int)) != cudaSuccess ||
        cudaMemset(pool, 0, kSchedSlots * 2 * sizeof(int)) != cudaSuccess) {
      pool = nullptr;
      disabled = true;
      return nullptr;
    }
  }
  return pool + 2 * (counter++ % kSchedSlots);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point, so the
// library does not link against libcuda directly.
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

}  // namespace

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  EncodeFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  // The driver entry point needs a current context on the calling thread;
  // autograd's backward threads have only used the runtime API lazily.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// fp32 tensor map of C with 32x32 boxes and 128-byte swizzle (epilogue staging layout).
int make_tmap_c_f32(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes) {
  EncodeFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

template <bool A_MN, bool B_MN, int EPI>
static int launch(const GemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb, int num_sms,
                  cudaStream_t stream) {
  auto kern = gemm_kernel<A_MN, B_MN, EPI>;
  constexpr int smem_bytes = EPI == kEpiAccumF32 ? SMEM_BYTES_F32 : SMEM_BYTES;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess)
      return -2;
    configured = true;
  }
  CUtensorMap tc = ta;      // unused by the bf16 epilogue
  if (EPI == kEpiAccumF32) {
    const int rc = make_tmap_c_f32(&tc, g.c, g.N, g.M, static_cast<uint64_t>(g.ldc) * 4);
    if (rc != 0) return rc;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(ta, tb, tc, g.c, g.ldc, g.M, g.N, g.K, g.accumulate,
                                                  g.status, next_sched_slot());
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// 0: choose by shape, 128 / 256: forced by PIPER_GEMM_TILE
static int forced_tile() {
  static int v = -1;
  if (v < 0) {
    const char* env = getenv("PIPER_GEMM_TILE");
    v = env == nullptr ? 0 : atoi(env);
    if (v != 128 && v != 256) v = 0;
  }
  return v;
}

int gemm_bf16_launch(const GemmArgs& g, int num_sms, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return 0;
  {
    // 256x256 tiles move a third fewer operand bytes per flop.  Measured on B200: they win for bf16 outputs once
    // there is at least one tile per SM, and for fp32 (weight-gradient) outputs that are at least as tall as
    // wide; wide fp32 outputs do a little better with 128x256 tiles and their double-buffered accumulators.
    const int tile = g.tile != 0 ? g.tile : forced_tile();
    const long long tiles256 = static_cast<long long>((g.M + 255) / 256) * ((g.N + 255) / 256);
    const bool fits = g.M >= 256 && g.N >= 256 && tiles256 >= num_sms;
    const bool pays = g.epilogue == kEpiStoreBf16 || g.M >= g.N;
    if (tile == 256 || (tile == 0 && fits && pays))
      return gemm256_bf16_launch(g, num_sms, next_sched_slot(), stream);
  }
  CUtensorMap ta, tb;
  int rc;
  // K-major operand: dims {K, rows}, box {64, tile rows}.
  // MN-major operand: dims {rows, K}, box {64, 64}.
  rc = g.a_mn_major ? make_tmap_2d_bf16(&ta, g.a, g.M, g.K, g.lda * 2, 64, BK)
                    : make_tmap_2d_bf16(&ta, g.a, g.K, g.M, g.lda * 2, BK, BM);
  if (rc != 0) return rc;
  rc = g.b_mn_major ? make_tmap_2d_bf16(&tb, g.b, g.N, g.K, g.ldb * 2, 64, BK)
                    : make_tmap_2d_bf16(&tb, g.b, g.K, g.N, g.ldb * 2, BK, BN);
  if (rc != 0) return rc;
  const int key = (g.a_mn_major ? 4 : 0) | (g.b_mn_major ? 2 : 0) | (g.epilogue == kEpiAccumF32 ? 1 : 0);
  switch (key) {
    case 0: return launch<false, false, kEpiStoreBf16>(g, ta, tb, num_sms, stream);
    case 1: return launch<false, false, kEpiAccumF32>(g, ta, tb, num_sms, stream);
    case 2: return launch<false, true, kEpiStoreBf16>(g, ta, tb, num_sms, stream);
    case 3: return launch<false, true, kEpiAccumF32>(g, ta, tb, num_sms, stream);
    case 4: return launch<true, false, kEpiStoreBf16>(g, ta, tb, num_sms, stream);
    case 5: return launch<true, false, kEpiAccumF32>(g, ta, tb, num_sms, stream);
    case 6: return launch<true, true, kEpiStoreBf16>(g, ta, tb, num_sms, stream);
    default: return launch<true, true, kEpiAccumF32>(g, ta, tb, num_sms, stream);
  }
}

}  // namespace piper
