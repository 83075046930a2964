// Implementation of the allocation-free RMSNorm backward entry point; see
// no_alloc.h for the contract.
#include "no_alloc.h"

#include <cstdio>

#include "elementwise.h"

namespace {

// Scratch for the per-strip partial sums of the weight gradient.  In host
// code this name is only a handle for cudaGetSymbolAddress, never an address
// a kernel may be given.
static __device__ __align__(256) float g_dw_partial_scratch[PIPER_NOALLOC_MAX_STRIPS * PIPER_NOALLOC_MAX_D];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};   // device address of the array, per device ordinal
thread_local char g_error[256] = "";

int fail(int code, const char* fmt, long long a = 0, long long b = 0) {
  std::snprintf(g_error, sizeof(g_error), fmt, a, b);
  return code;
}

// Device address of the scratch array on the current device, resolved once
// per device while that device is current.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(-2, "cannot identify the current CUDA device (ordinal %lld)", dev);
    return nullptr;
  }
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dw_partial_scratch);
    if (e != cudaSuccess || p == nullptr) {
      std::snprintf(g_error, sizeof(g_error), "cudaGetSymbolAddress failed on device %d: %s", dev,
                    cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch_addr[dev] = p;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int piper_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                         void* dx, float* dw, int accumulate, long long T, int D,
                                         cudaStream_t stream) {
  g_error[0] = '\0';
  if (T < 0) return fail(-1, "T must be non-negative, got %lld", T);
  if (T > 2147483647LL) return fail(-1, "T = %lld exceeds the 32-bit row index of the kernels (max %lld)", T, 2147483647LL);
  if (D <= 0 || D % 8 != 0) return fail(-1, "D must be a positive multiple of 8, got %lld", D);
  if (D > PIPER_NOALLOC_MAX_D)
    return fail(-1, "D = %lld exceeds the built-in scratch size (PIPER_NOALLOC_MAX_D = %lld)", D,
                PIPER_NOALLOC_MAX_D);
  if (piper::rmsnorm_bwd_num_partials(T) > PIPER_NOALLOC_MAX_STRIPS)
    return fail(-1, "T = %lld needs more strips than the scratch array holds (%lld)", T,
                PIPER_NOALLOC_MAX_STRIPS);
  if (T == 0) return 0;
  float* scratch = scratch_for_current_device();
  if (scratch == nullptr) return -2;
  const int rc = piper::rmsnorm_bwd(dy, x, w, rstd, /*dres=*/nullptr, dx, scratch, dw, /*dw_bf16=*/nullptr,
                                    accumulate, T, D, stream);
  if (rc != 0) return fail(-3, "kernel launch failed with code %lld", rc);
  return 0;
}

extern "C" const char* piper_noalloc_last_error(void) { return g_error; }
