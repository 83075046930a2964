// Grouped bf16 GEMMs of the mixture-of-experts MLP for sm_100a.
//
// Token rows arrive grouped by (source rank, local expert); group g occupies
// rows [g_start[g], g_start[g] + g_len[g]) of a row buffer, with g_len a
// multiple of 128 (segments are padded with zero rows) and expert(g) =
// g % experts.  Three products share one kernel template:
//
//   kGroupedFwd    Y[rows, N]  = X[rows, K]  * W[e][N, K]^T      (forward)
//   kGroupedDgrad  dX[rows, K] = dY[rows, N] * W[e][N, K]        (input gradient)
//   kGroupedWgrad  dW[e][N, K] += dY[rows_e, N]^T * X[rows_e, K] (weight gradient,
//                  contraction over all row segments of expert e)
//
// The structure is that of the dense kernel (gemm_sm100.cu): persistent
// CTAs, TMA producer warp, single-thread tcgen05.mma issuer, two TMEM
// accumulators, eight epilogue warps; only the tile -> coordinate mapping
// differs and is computed on the device from the group table, because the
// row counts are produced by the router on the GPU.  Expert weights are read
// through a 3-D tensor map (k, n, expert).  No multicast; bounded waits.
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
constexpr int MN_BOX_BYTES = 64 * BK * 2;
constexpr int NUM_THREADS = 384;     // TMA, MMA, TMEM-allocation and one idle warp, then eight epilogue warps
constexpr int MAX_GROUPS = 1024;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + (MAX_GROUPS + 1) * 4;

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
};

struct GroupedParams {
  const int* g_start;    // [G] first row of each group
  const int* g_len;      // [G] padded row count (multiple of 128)
  int num_groups;        // G = sources * experts
  int experts;           // local experts
  int N, K;              // weight shape per expert [N, K]
  void* c;               // output
  long long ldc;
  int accumulate;
  int* status;
};

// Tile descriptor resolved from a linear tile index.
struct Tile {
  int m0, n0;       // output coordinates (rows / weight-N for wgrad, cols)
  int expert;
  int group;        // row group (fwd/dgrad)
  bool valid;
};

template <int MODE>
__device__ __forceinline__ Tile resolve_tile(int t, const int* tile_prefix, const GroupedParams& p,
                                             int total_m_tiles, int tiles_n) {
  Tile r;
  r.valid = true;
  if (MODE == kGroupedWgrad) {
    const int tiles_m = (p.N + BM - 1) / BM;
    const int per_expert = tiles_m * tiles_n;
    r.expert = t / per_expert;
    const int rem = t % per_expert;
    r.m0 = (rem % tiles_m) * BM;
    r.n0 = (rem / tiles_m) * BN;
    r.group = 0;
    return r;
  }
  // Column tiles of one row tile are consecutive, and row tiles are walked expert by expert (all sources of an
  // expert together): the CTAs of a wave share their A tiles and a few experts' weights through L2, so both
  // operands stream from DRAM once.  (Row tiles fastest re-read every row once per column tile.)
  (void)total_m_tiles;
  const int mt = t / tiles_n;
  r.n0 = (t % tiles_n) * BN;
  int lo = 0, hi = p.num_groups;          // largest q with tile_prefix[q] <= mt
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_prefix[mid] <= mt) lo = mid; else hi = mid;
  }
  const int sources = p.num_groups / p.experts;
  r.expert = lo / sources;                 // tile_prefix is ordered (expert, source)
  r.group = (lo % sources) * p.experts + r.expert;
  r.m0 = p.g_start[r.group] + (mt - tile_prefix[lo]) * BM;
  return r;
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  int* tile_prefix = reinterpret_cast<int*>(smem + STAGES * STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr bool A_MN = (MODE == kGroupedWgrad);
  constexpr bool B_MN = (MODE != kGroupedFwd);
  const int out_cols = (MODE == kGroupedFwd) ? p.N : p.K;       // columns of the output matrix
  const int contract = (MODE == kGroupedFwd) ? p.K : p.N;       // contraction length (fwd / dgrad)
  const int tiles_n = (out_cols + BN - 1) / BN;
  const int sources = p.num_groups / p.experts;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->acc_full[a], 1);
      mbar_init(&bars->acc_empty[a], 8);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    int acc = 0;
    for (int q = 0; q < p.num_groups; ++q) {           // q = expert * sources + source; group = source * experts + expert
      tile_prefix[q] = acc;
      acc += p.g_len[(q % sources) * p.experts + q / sources] / BM;
    }
    tile_prefix[p.num_groups] = acc;
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const int total_m_tiles = tile_prefix[p.num_groups];
  const int num_tiles = (MODE == kGroupedWgrad) ? p.experts * ((p.N + BM - 1) / BM) * tiles_n
                                                : total_m_tiles * tiles_n;

  // Number of 64-deep k-blocks of a tile.
  auto k_blocks_of = [&](const Tile& t) -> int {
    if (MODE != kGroupedWgrad) return (contract + BK - 1) / BK;
    int n = 0;
    for (int s = 0; s < sources; ++s) n += p.g_len[s * p.experts + t.expert] / BK;
    return n;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int ti = blockIdx.x; ti < num_tiles && ok; ti += gridDim.x) {
        const Tile t = resolve_tile<MODE>(ti, tile_prefix, p, total_m_tiles, tiles_n);
        auto issue = [&](int a_x, int a_y, int b_x, int b_y) -> bool {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, p.status)) return false;
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_arrive_expect_tx(&bars->full[s], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * MN_BOX_BYTES, &tmap_a, &bars->full[s], a_x + 64 * j, a_y);
          } else {
            tma_load_2d(sa, &tmap_a, &bars->full[s], a_x, a_y);
          }
          if (MODE == kGroupedFwd) {
            tma_load_3d(sb, &tmap_b, &bars->full[s], b_x, b_y, t.expert);
          } else if (MODE == kGroupedDgrad) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * MN_BOX_BYTES, &tmap_b, &bars->full[s], b_x + 64 * j, b_y, t.expert);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * MN_BOX_BYTES, &tmap_b, &bars->full[s], b_x + 64 * j, b_y);
          }
          ++it;
          return true;
        };
        if (MODE == kGroupedWgrad) {
          for (int s = 0; s < sources && ok; ++s) {
            const int g = s * p.experts + t.expert;
            const int r0 = p.g_start[g], len = p.g_len[g];
            for (int r = 0; r < len && ok; r += BK) ok = issue(t.m0, r0 + r, t.n0, r0 + r);
          }
        } else {
          const int kb = (contract + BK - 1) / BK;
          for (int k = 0; k < kb && ok; ++k) {
            // fwd:   A[x=k, y=row], B[x=k, y=n, z=e]
            // dgrad: A[x=k(contraction over N), y=row], B[x=out col, y=k, z=e]
            ok = (MODE == kGroupedFwd) ? issue(k * BK, t.m0, k * BK, t.n0) : issue(k * BK, t.m0, t.n0, k * BK);
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
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int ti = blockIdx.x; ti < num_tiles && ok; ti += gridDim.x) {
        const Tile t = resolve_tile<MODE>(ti, tile_prefix, p, total_m_tiles, tiles_n);
        const int kb_total = k_blocks_of(t);
        if (kb_total == 0) continue;
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        ++local_tile;
        if (!mbar_wait(&bars->acc_empty[acc], acc_ph ^ 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(sa + k * (UMMA_K * 128), MN_BOX_BYTES, 1024)
                                     : umma_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(sb + k * (UMMA_K * 128), MN_BOX_BYTES, 1024)
                                     : umma_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3;                     // TMEM lanes [32q, 32q + 32)
    const int ch = (warp - 4) >> 2;             // columns [128ch, 128ch + 128) of the tile
    uint32_t local_tile = 0;
    bool ok = true;
    for (int ti = blockIdx.x; ti < num_tiles && ok; ti += gridDim.x) {
      const Tile t = resolve_tile<MODE>(ti, tile_prefix, p, total_m_tiles, tiles_n);
      const int kb_total = k_blocks_of(t);
      const int row_limit = (MODE == kGroupedWgrad) ? p.N : 0x7fffffff;
      const int row = t.m0 + q * 32 + lane;
      const long long c_off = (MODE == kGroupedWgrad) ? static_cast<long long>(t.expert) * p.N * p.K : 0;
      if (kb_total == 0) {
        // expert without rows: nothing to add; a non-accumulating output tile is zero
        if (!p.accumulate && row < row_limit) {
          for (int j = ch * 128; j < ch * 128 + 128 && t.n0 + j < out_cols; ++j) {
            if (MODE == kGroupedWgrad) reinterpret_cast<float*>(p.c)[c_off + row * p.ldc + t.n0 + j] = 0.f;
          }
        }
        continue;
      }
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      ++local_tile;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, p.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + ch * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = t.n0 + ch * 128 + c * 32;
        if (row < row_limit && col0 < out_cols) {
          if (MODE == kGroupedWgrad) {
            float* crow = reinterpret_cast<float*>(p.c) + c_off + row * p.ldc + col0;
            if (col0 + 32 <= out_cols) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v + 0]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if (p.accumulate) {
                  const float4 q = reinterpret_cast<const float4*>(crow)[v];
                  o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w;
                }
                reinterpret_cast<float4*>(crow)[v] = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {      // constant indices keep r[] in registers
                if (col0 + j < out_cols) {
                  const float x = __uint_as_float(r[j]);
                  crow[j] = p.accumulate ? crow[j] + x : x;
                }
              }
            }
          } else {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.c) + row * p.ldc + col0;
            if (col0 + 32 <= out_cols) {
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
              for (int j = 0; j < 32; ++j)        // constant indices keep r[] in registers
                if (col0 + j < out_cols) crow[j] = __float2bfloat16(__uint_as_float(r[j]));
            }
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

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1) {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  const cuuint32_t box[3] = {b0, b1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r =
      fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

template <int MODE>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GroupedParams& p, int num_sms, cudaStream_t st) {
  auto kern = grouped_gemm_kernel<MODE>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -2;
    configured = true;
  }
  kern<<<num_sms, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

int grouped_gemm_launch(const GroupedGemmArgs& g, int num_sms, cudaStream_t st) {
  if (g.num_groups <= 0 || g.num_groups > MAX_GROUPS || g.experts <= 0 || g.num_groups % g.experts != 0) return -11;
  if (g.N % 8 != 0 || g.K % 8 != 0 || g.rows_capacity < 0) return -12;
  if (g.rows_capacity == 0) {
    // A rank can receive no rows at all (every token routed to experts of other ranks): nothing to multiply.
    // The weight gradient of such a step is zero.
    if (g.mode == kGroupedWgrad && !g.accumulate) {
      const size_t bytes = static_cast<size_t>(g.experts) * g.N * g.K * sizeof(float);
      if (cudaMemsetAsync(g.out, 0, bytes, st) != cudaSuccess) return -3;
    }
    return 0;
  }
  GroupedParams p;
  p.g_start = g.g_start;
  p.g_len = g.g_len;
  p.num_groups = g.num_groups;
  p.experts = g.experts;
  p.N = g.N;
  p.K = g.K;
  p.c = g.out;
  p.accumulate = g.accumulate;
  p.status = g.status;
  CUtensorMap ta, tb;
  int rc;
  const uint64_t R = static_cast<uint64_t>(g.rows_capacity);
  const uint64_t N = g.N, K = g.K, E = g.experts;
  if (g.mode == kGroupedFwd) {
    // A = X [R, K] K-major; B = W [E, N, K] K-major; C = Y [R, N]
    if ((rc = make_tmap_2d_bf16(&ta, g.x, K, R, K * 2, BK, BM)) != 0) return rc;
    if ((rc = make_tmap_3d_bf16(&tb, g.w, K, N, E, K * 2, N * K * 2, BK, BN)) != 0) return rc;
    p.ldc = g.N;
    return launch<kGroupedFwd>(ta, tb, p, num_sms, st);
  }
  if (g.mode == kGroupedDgrad) {
    // A = dY [R, N] K-major (contraction N); B = W [E, N, K] read MN-major; C = dX [R, K]
    if ((rc = make_tmap_2d_bf16(&ta, g.dy, N, R, N * 2, BK, BM)) != 0) return rc;
    if ((rc = make_tmap_3d_bf16(&tb, g.w, K, N, E, K * 2, N * K * 2, 64, BK)) != 0) return rc;
    p.ldc = g.K;
    return launch<kGroupedDgrad>(ta, tb, p, num_sms, st);
  }
  // wgrad: A = dY [R, N] MN-major, B = X [R, K] MN-major, C = dW [E, N, K] fp32
  if ((rc = make_tmap_2d_bf16(&ta, g.dy, N, R, N * 2, 64, BK)) != 0) return rc;
  if ((rc = make_tmap_2d_bf16(&tb, g.x, K, R, K * 2, 64, BK)) != 0) return rc;
  p.ldc = g.K;
  return launch<kGroupedWgrad>(ta, tb, p, num_sms, st);
}

}  // namespace piper
