// Symmetric-memory runtime: raw device allocations that can be shared between the
// processes of one node through CUDA IPC handles, so kernels can load/store peer
// memory over NVLink.  (Allocations of PyTorch's caching allocator cannot be shared
// when it uses virtual-memory segments, hence the explicit cudaMalloc here.)
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>
#include <string>

namespace {

void throw_if(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    char buf[200];
    snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
    throw std::runtime_error(buf);
  }
}

int64_t symm_alloc(int64_t nbytes, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  void* p = nullptr;
  throw_if(cudaMalloc(&p, (size_t)nbytes), "cudaMalloc (symmetric buffer)");
  throw_if(cudaMemset(p, 0, (size_t)nbytes), "cudaMemset (symmetric buffer)");
  return reinterpret_cast<int64_t>(p);
}
void symm_free(int64_t ptr, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  cudaFree(reinterpret_cast<void*>(ptr));
}
pybind11::bytes ipc_get_handle(int64_t ptr) {
  cudaIpcMemHandle_t h;
  throw_if(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr)), "cudaIpcGetMemHandle");
  return pybind11::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}
int64_t ipc_open_handle(const std::string& bytes, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  if (bytes.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, bytes.data(), sizeof(h));
  void* p = nullptr;
  throw_if(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<int64_t>(p);
}
void ipc_close(int64_t ptr, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
}
torch::Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, torch::ScalarType dtype, int64_t device) {
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, (c10::DeviceIndex)device);
  return torch::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts);
}
bool can_access_peer(int64_t dev, int64_t peer) {
  int ok = 0;
  cudaDeviceCanAccessPeer(&ok, (int)dev, (int)peer);
  return ok != 0;
}

}  // namespace

void register_symm(pybind11::module_& m) {
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_free", &symm_free);
  m.def("ipc_get_handle", &ipc_get_handle);
  m.def("ipc_open_handle", &ipc_open_handle);
  m.def("ipc_close", &ipc_close);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("can_access_peer", &can_access_peer);
}
