// Host-side interface of the tcgen05 GEMM family (gemm_sm100.cu,
// grouped_gemm_sm100.cu).  Plain C++ / CUDA runtime types only, so the
// kernels build without any framework headers.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace piper {

enum : int {
  kEpiStoreBf16 = 0,   // C (bf16) = acc
  kEpiAccumF32 = 1,    // C (fp32) = acc, or C += acc when accumulate != 0
};

// C[M,N] = A[M,K] * B[N,K]^T.
//   a_mn_major == 0: A is stored row-major [M, K] with row stride lda (elements).
//   a_mn_major == 1: A is stored row-major [K, M] with row stride lda.
//   b_mn_major == 0: B is stored row-major [N, K] with row stride ldb.
//   b_mn_major == 1: B is stored row-major [K, N] with row stride ldb.
// Base pointers must be 16-byte aligned and lda/ldb multiples of 8 elements
// (TMA global-stride rule); ldc is in elements of the output type.
struct GemmArgs {
  const void* a;
  const void* b;
  void* c;
  long long lda, ldb, ldc;
  int M, N, K;
  int a_mn_major, b_mn_major;
  int epilogue;     // kEpi*
  int accumulate;   // only for kEpiAccumF32
  int* status;      // device int, 0 = ok (see ptx.cuh)
  int tile = 0;     // 0: chosen by shape (or PIPER_GEMM_TILE); 128 / 256: that CTA tile height
};

// Returns 0 on success, a negative code for a launch/set-up failure, or the
// CUresult of a failed tensor-map encode.
int gemm_bf16_launch(const GemmArgs& args, int num_sms, cudaStream_t stream);

// Same contract with 256x256 tiles per CTA (gemm256_sm100.cu).  sched: two zeroed ints of device memory for the
// dynamic tile scheduler (rearmed by the kernel), or null for static tile striding.  gemm_bf16_launch picks
// between the two tile shapes; PIPER_GEMM_TILE=128 or 256 forces one.
int gemm256_bf16_launch(const GemmArgs& args, int num_sms, int* sched, cudaStream_t stream);

enum : int {
  kGroupedFwd = 0,     // Y[rows, N]  = X[rows, K] * W[e]^T
  kGroupedDgrad = 1,   // dX[rows, K] = dY[rows, N] * W[e]
  kGroupedWgrad = 2,   // dW[e][N, K] (+)= dY[rows_e]^T * X[rows_e]   (fp32 output)
};

// Grouped GEMMs of the expert MLP.  Rows of x / dy / out are grouped: group g
// owns rows [g_start[g], g_start[g] + g_len[g]), g_len a multiple of 128 with
// zero padding rows, and uses expert g % experts of w [experts, N, K].
// g_start / g_len live on the device.  rows_capacity is the row count of the
// row buffers.  out is bf16 [rows_capacity, N] (fwd), bf16 [rows_capacity, K]
// (dgrad) or fp32 [experts, N, K] (wgrad; accumulate selects += or =).
struct GroupedGemmArgs {
  int mode;
  const void* x;        // [rows_capacity, K]   (fwd, wgrad)
  const void* dy;       // [rows_capacity, N]   (dgrad, wgrad)
  const void* w;        // [experts, N, K]      (fwd, dgrad)
  void* out;
  const int* g_start;
  const int* g_len;
  int num_groups, experts;
  int N, K;
  long long rows_capacity;
  int accumulate;
  int* status;
};

int grouped_gemm_launch(const GroupedGemmArgs& args, int num_sms, cudaStream_t stream);

constexpr int kMaxPeers = 8;

// Y[M, N] = X[M, K] * W[N, K]^T with W sharded by rows: w_shards[p] points at
// rank p's rows [p*rows_per_shard, (p+1)*rows_per_shard) (local or peer-mapped
// memory, rows_per_shard a multiple of 64); shard my_index is this rank's own.
// When w_full is not null every remote row crosses NVLink once, into w_full
// ([N, K], local memory, complete when the kernel ends), and scratch must
// point at scratch_ints >= ceil(N / 256) + 2 ints of device memory that no
// other launch in flight uses.  When w_full is null each CTA loads the weight
// boxes it needs straight from their owners.
struct AgGemmArgs {
  const void* x;
  const void* w_shards[kMaxPeers];
  void* w_full;
  void* y;
  int M, N, K;
  int rows_per_shard, num_peers, my_index;
  int* scratch;
  int scratch_ints;
  int* status;
};

int ag_gemm_launch(const AgGemmArgs& args, int num_sms, cudaStream_t stream);

// fp32 tensor map of an output matrix with 32x32 boxes and 128-byte swizzle (layout of the fp32 epilogue staging).
int make_tmap_c_f32(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes);

// Encodes a 2-D bf16 tensor map with 128-byte swizzle.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

}  // namespace piper
