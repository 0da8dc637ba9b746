// Bindings of the MoE kernels (routing, split scan, dispatch, grouped GEMM, combine).
#include <ATen/cuda/CUDAContext.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include "kernels/api.h"

namespace py = pybind11;
using namespace fastb;

namespace {

void cu_check(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }
cudaStream_t stream_now() { return at::cuda::getCurrentCUDAStream().stream(); }

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cu_check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q), "cudaGetDriverEntryPoint");
    TORCH_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available in this driver");
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// A 2-D bf16 row-major matrix [rows, cols] (row pitch in elements) tiled in boxes of
// {box_cols, box_rows} with the 128-byte swizzle. box_cols must be 64 (one 128-byte line).
struct TensorMap2D {
  alignas(64) CUtensorMap map;
  TensorMap2D(int64_t ptr, int64_t rows, int64_t cols, int64_t pitch_elems, int box_cols, int box_rows) {
    TORCH_CHECK(box_cols == 64, "128-byte swizzle wants boxes of 64 bf16 in the contiguous dimension");
    TORCH_CHECK(box_rows >= 1 && box_rows <= 256, "box rows out of range");
    TORCH_CHECK(ptr % 16 == 0 && (pitch_elems * 2) % 16 == 0, "tensor map base and pitch must be 16-byte aligned");
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * 2};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, reinterpret_cast<void*>(ptr), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", static_cast<int>(r));
  }
};

void grouped_gemm(int mode, int epilogue, const TensorMap2D& a, const TensorMap2D& b, torch::Tensor group_off, int tiles_n, int fixed_m_tiles,
                  int red_len, int b_rows_per_group, int c_rows_per_group, torch::Tensor c, c10::optional<torch::Tensor> c2, int64_t status_ptr,
                  uint64_t timeout_ns, int ctas) {
  TORCH_CHECK(group_off.is_cuda() && group_off.dtype() == torch::kInt32 && group_off.is_contiguous() && group_off.numel() >= 2, "group_off: cuda int32[G+1]");
  TORCH_CHECK(c.is_cuda() && c.dtype() == torch::kBFloat16 && c.dim() == 2 && c.stride(1) == 1, "c: cuda bf16 [rows, cols]");
  TORCH_CHECK(red_len % 64 == 0 && tiles_n >= 1, "reduction length must be a multiple of 64");
  GemmArgs g{};
  g.group_off = group_off.data_ptr<int>();
  g.num_groups = static_cast<int>(group_off.numel()) - 1;
  g.tiles_n = tiles_n; g.fixed_m_tiles = fixed_m_tiles; g.red_len = red_len;
  g.b_rows_per_group = b_rows_per_group; g.c_rows_per_group = c_rows_per_group;
  g.c = reinterpret_cast<__nv_bfloat16*>(c.data_ptr()); g.ldc = c.stride(0);
  if (c2.has_value()) {
    TORCH_CHECK(c2->is_cuda() && c2->dtype() == torch::kBFloat16 && c2->dim() == 2 && c2->stride(1) == 1, "c2: cuda bf16 [rows, cols]");
    g.c2 = reinterpret_cast<__nv_bfloat16*>(c2->data_ptr()); g.ldc2 = c2->stride(0);
  }
  g.status = reinterpret_cast<DeviceStatus*>(status_ptr);
  g.timeout_ns = timeout_ns;
  cu_check(launch_grouped_gemm(static_cast<GemmMode>(mode), static_cast<GemmEpilogue>(epilogue), a.map, b.map, g, ctas, stream_now()), "grouped_gemm launch");
}

}  // namespace

void bind_moe(py::module_& m) {
  py::class_<TensorMap2D>(m, "TensorMap2D").def(py::init<int64_t, int64_t, int64_t, int64_t, int, int>());
  m.def("grouped_gemm", &grouped_gemm);
  m.def("grouped_gemm_smem_bytes", &grouped_gemm_smem_bytes);
}
