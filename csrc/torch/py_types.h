// Python-side handle types shared by the binding translation units.
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <memory>

#include "kernels/api.h"
#include "runtime/symm_heap.h"

namespace fastb_py {
namespace py = pybind11;
using namespace fastb;

inline void cuda_check(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }
inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// ---- symmetric heap -----------------------------------------------------------------------------
struct HeapPy {
  std::shared_ptr<SymmHeap> h;
  int device;
  torch::Tensor tensor(int64_t offset, std::vector<int64_t> shape, py::object dtype) const {
    auto dt = torch::python::detail::py_object_to_dtype(dtype);
    auto opts = torch::TensorOptions().dtype(dt).device(torch::kCUDA, device);
    // The deleter holds a reference to the heap: the slab outlives every tensor carved from it.
    auto keep = h;
    return torch::from_blob(static_cast<char*>(h->local_base()) + offset, shape, [keep](void*) {}, opts);
  }
};

// ---- status block -------------------------------------------------------------------------------
struct StatusPy {
  DeviceStatus* d = nullptr;
  StatusPy() {
    cuda_check(cudaMalloc(reinterpret_cast<void**>(&d), sizeof(DeviceStatus)), "cudaMalloc status");
    cuda_check(cudaMemset(d, 0, sizeof(DeviceStatus)), "clear status");
  }
  ~StatusPy() { if (d) cudaFree(d); }
  // Synchronises the current stream, then returns (code, site, detail, seen, want).
  py::tuple read() const {
    DeviceStatus s;
    cuda_check(cudaStreamSynchronize(cur_stream()), "sync before status read");
    cuda_check(cudaMemcpy(&s, d, sizeof(s), cudaMemcpyDeviceToHost), "read status");
    return py::make_tuple(s.code, s.site, s.detail, s.seen, s.want);
  }
  void clear() { cuda_check(cudaMemsetAsync(d, 0, sizeof(DeviceStatus), cur_stream()), "clear status"); }
};


}  // namespace fastb_py
