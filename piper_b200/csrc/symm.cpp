// Symmetric memory for the fused collective kernels: device allocations that
// every rank of a group maps into its own address space.
//
// A buffer is a plain cudaMalloc allocation (one allocation per buffer, so
// its IPC handle has offset zero), exported with cudaIpcGetMemHandle; the
// 64-byte handles travel through the job's torch.distributed store and each
// peer maps them with cudaIpcOpenMemHandle, which also enables NVLink peer
// access.  Kernels then use ordinary loads and stores on the peer pointers.
#include <ATen/ATen.h>
#include <cuda_runtime.h>
#include <torch/library.h>

#include <cstring>

namespace {

using at::Tensor;

void cuda_check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "symmetric memory: ", what, " failed: ", cudaGetErrorString(e));
}

// Zero-initialised device buffer of nbytes, owned by the returned uint8 tensor.
Tensor symm_alloc(int64_t nbytes) {
  int dev = 0;
  cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
  void* p = nullptr;
  const size_t n = nbytes > 0 ? static_cast<size_t>(nbytes) : 1;
  cuda_check(cudaMalloc(&p, n), "cudaMalloc");
  cuda_check(cudaMemset(p, 0, n), "cudaMemset");
  cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  auto opts = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev);
  return at::from_blob(p, {nbytes}, [](void* q) { cudaFree(q); }, opts);
}

// 64-byte IPC handle of a buffer returned by symm_alloc, as a CPU uint8 tensor.
Tensor symm_export(const Tensor& buf) {
  cudaIpcMemHandle_t h;
  cuda_check(cudaIpcGetMemHandle(&h, buf.data_ptr()), "cudaIpcGetMemHandle");
  Tensor out = at::empty({static_cast<int64_t>(sizeof(h))}, at::kByte);
  std::memcpy(out.data_ptr(), &h, sizeof(h));
  return out;
}

// Maps a peer's buffer; returns the device address in this process.
int64_t symm_import(const Tensor& handle) {
  TORCH_CHECK(handle.numel() == static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* p = nullptr;
  cuda_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<int64_t>(p);
}

void symm_release(int64_t ptr) {
  if (ptr != 0) cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
}

}  // namespace

void register_symm_ops(torch::Library& m) {
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_export", &symm_export);
  m.def("symm_import", &symm_import);
  m.def("symm_release", &symm_release);
}
