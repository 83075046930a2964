// Symmetric memory for the fused collective kernels: device allocations that
// every rank of a group maps into its own address space.
//
// A buffer is a plain cudaMalloc allocation exported with cudaIpcGetMemHandle.
// The runtime may carve several small allocations out of one underlying
// block, and an IPC handle always names the whole block, so an exported
// record is (64-byte handle, offset of the buffer inside its block), and the
// importing side opens each block once per process (reference-counted) and
// adds the offset.  The records travel through the job's torch.distributed
// store; cudaIpcOpenMemHandle also enables NVLink peer access.  Kernels then
// use ordinary loads and stores on the peer pointers.
#include <ATen/ATen.h>
#include <cuda_runtime.h>
#include <torch/library.h>

#include <cuda.h>

#include <cstring>
#include <map>
#include <mutex>
#include <string>

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

using AddressRangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);

AddressRangeFn address_range_fn() {
  static AddressRangeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cuda_check(cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q), "cudaGetDriverEntryPoint");
    TORCH_CHECK(q == cudaDriverEntryPointSuccess && p != nullptr, "symmetric memory: cuMemGetAddressRange unavailable");
    fn = reinterpret_cast<AddressRangeFn>(p);
  }
  return fn;
}

constexpr int64_t kRecordBytes = static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)) + 8;

// Export record of a buffer returned by symm_alloc: IPC handle of its block + offset inside the block,
// as a CPU uint8 tensor.
Tensor symm_export(const Tensor& buf) {
  cudaIpcMemHandle_t h;
  cuda_check(cudaIpcGetMemHandle(&h, buf.data_ptr()), "cudaIpcGetMemHandle");
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUdeviceptr ptr = reinterpret_cast<CUdeviceptr>(buf.data_ptr());
  TORCH_CHECK(address_range_fn()(&base, &size, ptr) == CUDA_SUCCESS, "symmetric memory: cuMemGetAddressRange failed");
  const uint64_t offset = static_cast<uint64_t>(ptr - base);
  Tensor out = at::empty({kRecordBytes}, at::kByte);
  std::memcpy(out.data_ptr(), &h, sizeof(h));
  std::memcpy(static_cast<uint8_t*>(out.data_ptr()) + sizeof(h), &offset, 8);
  return out;
}

struct OpenedBlock {
  void* base = nullptr;
  int refs = 0;
};
std::mutex g_mu;
std::map<std::string, OpenedBlock> g_blocks;          // handle bytes -> mapping of that block in this process
std::multimap<int64_t, std::string> g_ptr_block;      // address handed out -> its block

// Maps a peer's buffer; returns the device address in this process.
int64_t symm_import(const Tensor& record) {
  TORCH_CHECK(record.numel() == kRecordBytes, "bad symmetric-memory export record");
  cudaIpcMemHandle_t h;
  uint64_t offset = 0;
  std::memcpy(&h, record.data_ptr(), sizeof(h));
  std::memcpy(&offset, static_cast<const uint8_t*>(record.data_ptr()) + sizeof(h), 8);
  const std::string key(reinterpret_cast<const char*>(&h), sizeof(h));
  std::lock_guard<std::mutex> lock(g_mu);
  OpenedBlock& blk = g_blocks[key];
  if (blk.refs == 0) {
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      g_blocks.erase(key);
      cuda_check(e, "cudaIpcOpenMemHandle");
    }
    blk.base = p;
  }
  ++blk.refs;
  const int64_t addr = reinterpret_cast<int64_t>(static_cast<uint8_t*>(blk.base) + offset);
  g_ptr_block.emplace(addr, key);
  return addr;
}

void symm_release(int64_t ptr) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_ptr_block.find(ptr);
  if (it == g_ptr_block.end()) return;
  auto blk = g_blocks.find(it->second);
  g_ptr_block.erase(it);
  if (blk == g_blocks.end()) return;
  if (--blk->second.refs == 0) {
    cudaIpcCloseMemHandle(blk->second.base);
    g_blocks.erase(blk);
  }
}

// A tensor over memory the caller owns (a range of a symm_alloc buffer): not a view of another tensor, so it
// can be returned from a custom op and saved by autograd like any freshly allocated tensor.
Tensor symm_tensor_bf16(int64_t ptr, int64_t rows, int64_t cols) {
  int dev = 0;
  cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
  TORCH_CHECK(ptr != 0 && ptr % 16 == 0 && rows >= 0 && cols > 0, "symm_tensor_bf16: bad address or shape");
  auto opts = at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, dev);
  return at::from_blob(reinterpret_cast<void*>(ptr), {rows, cols}, opts);
}

}  // namespace

void register_symm_ops(torch::Library& m) {
  m.def("symm_tensor_bf16", &symm_tensor_bf16);
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_export", &symm_export);
  m.def("symm_import", &symm_import);
  m.def("symm_release", &symm_release);
}
