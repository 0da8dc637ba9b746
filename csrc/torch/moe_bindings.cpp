// Bindings of the MoE kernels (routing, split scan, dispatch, grouped GEMM, combine).
#include <cuda.h>
#include <cuda_runtime.h>

#include "py_types.h"

namespace py = pybind11;
using namespace fastb;
using namespace fastb_py;

namespace {

void cu_check(cudaError_t e, const char* what) { cuda_check(e, what); }
cudaStream_t stream_now() { return cur_stream(); }

template <class T> T* ptr_or_null(const c10::optional<torch::Tensor>& t) { return t.has_value() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr; }
void want(const torch::Tensor& t, c10::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == dt, name, ": expected a contiguous CUDA tensor of the right dtype");
}

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
  TensorMap2D() = default;
  // A 2-D byte matrix (e4m3 rows) tiled in boxes of {64 bytes, box_rows}, no swizzle: the ring the converter
  // warps of the e4m3-operand GEMM read from.
  static TensorMap2D bytes(int64_t ptr, int64_t rows, int64_t cols, int64_t pitch_bytes, int box_rows) {
    TORCH_CHECK(box_rows >= 1 && box_rows <= 256 && ptr % 16 == 0 && pitch_bytes % 16 == 0 && cols % 64 == 0, "byte tensor map: 16-byte aligned base and pitch, columns a multiple of 64");
    TensorMap2D t;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
    cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled()(&t.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (bytes) failed with code ", static_cast<int>(r));
    return t;
  }
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
                  uint64_t timeout_ns, int ctas, int64_t gate_counter_ptr, c10::optional<torch::Tensor> gate_target, bool pair, int band_rows,
                  const TensorMap2D* map_c, const TensorMap2D* map_c2, bool direct_epilogue, c10::optional<torch::Tensor> a_scales,
                  c10::optional<torch::Tensor> group_rows, int gate_tile_rows) {
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
  g.band_rows = band_rows;
  g.direct_epilogue = direct_epilogue ? 1 : 0;
  g.gate_tile_rows = gate_tile_rows;
  if (a_scales.has_value()) {
    want(*a_scales, torch::kFloat32, "a_scales");
    TORCH_CHECK(pair && red_len % 128 == 0 && a_scales->dim() == 2 && a_scales->size(1) == red_len / 128, "a_scales: float [rows, red_len / 128], CTA-pair kernel");
    g.a_scales = a_scales->data_ptr<float>();
  }
  if (group_rows.has_value()) {
    want(*group_rows, torch::kInt32, "group_rows");
    TORCH_CHECK(group_rows->numel() >= g.num_groups, "group_rows: int32 [G]");
    g.group_rows = group_rows->data_ptr<int>();
  }
  if (gate_counter_ptr != 0) {
    TORCH_CHECK(gate_target.has_value() && gate_target->is_cuda() && gate_target->scalar_type() == torch::kInt64 &&
                gate_target->numel() >= (gate_tile_rows > 0 ? 1 : g.num_groups), "gate_target: cuda int64[G], or one entry per tile with gate_tile_rows");
    g.gate_slots = static_cast<int>(gate_target->numel());
    g.gate_counter = reinterpret_cast<const unsigned long long*>(gate_counter_ptr);
    g.gate_target = reinterpret_cast<const unsigned long long*>(gate_target->data_ptr());
  }
  if (pair) {
    TORCH_CHECK(map_c != nullptr && (map_c2 != nullptr) == c2.has_value(), "the CTA-pair kernel stores through tensor maps: give one for c, and one for c2 when c2 is given");
    cu_check(launch_grouped_gemm_pair(static_cast<GemmMode>(mode), static_cast<GemmEpilogue>(epilogue), a.map, b.map, map_c->map, map_c2 ? &map_c2->map : nullptr, g,
                                      ctas, stream_now()), "grouped_gemm pair launch");
  } else
    cu_check(launch_grouped_gemm(static_cast<GemmMode>(mode), static_cast<GemmEpilogue>(epilogue), a.map, b.map, g, ctas, stream_now()), "grouped_gemm launch");
}

void route_topk(torch::Tensor logits, c10::optional<torch::Tensor> bias, int K, torch::Tensor topk_idx, torch::Tensor topk_w,
                torch::Tensor slot_in_block, torch::Tensor block_cnt) {
  want(logits, torch::kFloat32, "logits"); want(topk_idx, torch::kInt32, "topk_idx"); want(topk_w, torch::kFloat32, "topk_w");
  want(slot_in_block, torch::kInt32, "slot_in_block"); want(block_cnt, torch::kInt32, "block_cnt");
  const int T = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
  const int blocks = (T + kRouteTokensPerBlock - 1) / kRouteTokensPerBlock;
  TORCH_CHECK(topk_idx.numel() == static_cast<int64_t>(T) * K && slot_in_block.numel() >= static_cast<int64_t>(blocks) * kRouteTokensPerBlock * K &&
              block_cnt.numel() == static_cast<int64_t>(blocks) * E, "route_topk: output shapes");
  cu_check(launch_route_topk(logits.data_ptr<float>(), ptr_or_null<const float>(bias), T, E, K, topk_idx.data_ptr<int>(), topk_w.data_ptr<float>(),
                             slot_in_block.data_ptr<int>(), block_cnt.data_ptr<int>(), stream_now()), "route_topk");
}

void splits_scan(const HeapPy& heap, int64_t counts_off, int64_t flags_off, uint64_t epoch, torch::Tensor block_cnt, torch::Tensor block_base,
                 torch::Tensor send_base, torch::Tensor send_cnt, torch::Tensor group_off, torch::Tensor group_rows, torch::Tensor arrive_target,
                 c10::optional<torch::Tensor> traffic, int num_channels, int row_align, int cap_rows, const StatusPy& st, uint64_t timeout_ns,
                 c10::optional<torch::Tensor> send_pos, int64_t epoch_dev_ptr, c10::optional<torch::Tensor> tile_target, int tile_rows) {
  SplitsArgs a{};
  if (tile_target.has_value()) {
    want(*tile_target, torch::kInt64, "tile_target");
    TORCH_CHECK(tile_target->dim() == 2 && tile_target->size(0) == num_channels && tile_rows > 0, "tile_target: int64 [channels, tiles]");
    a.tile_target = reinterpret_cast<unsigned long long*>(tile_target->data_ptr());
    a.tile_rows = tile_rows;
    a.num_tiles = static_cast<int>(tile_target->size(1));
  }
  a.row_align = row_align;
  a.cap_rows = cap_rows;
  a.peer_table = heap.h->device_peer_table(); a.rank = heap.h->rank(); a.world = heap.h->world();
  a.num_experts = static_cast<int>(send_base.numel()); a.num_blocks = static_cast<int>(block_cnt.numel() / a.num_experts); a.num_channels = num_channels;
  a.counts_heap_off = counts_off; a.flags_heap_off = flags_off; a.epoch = epoch;
  want(block_cnt, torch::kInt32, "block_cnt"); want(block_base, torch::kInt32, "block_base"); want(send_base, torch::kInt32, "send_base");
  want(send_cnt, torch::kInt32, "send_cnt"); want(group_off, torch::kInt32, "group_off"); want(group_rows, torch::kInt32, "group_rows");
  want(arrive_target, torch::kInt64, "arrive_target");
  const int El = a.num_experts / a.world;
  TORCH_CHECK(group_off.numel() == El + 1 && group_rows.numel() == El && arrive_target.numel() == static_cast<int64_t>(num_channels) * El, "splits_scan: shapes");
  a.block_cnt = block_cnt.data_ptr<int>(); a.block_base = block_base.data_ptr<int>(); a.send_base = send_base.data_ptr<int>();
  a.send_cnt = send_cnt.data_ptr<int>(); a.group_off = group_off.data_ptr<int>(); a.group_rows = group_rows.data_ptr<int>();
  a.arrive_target = reinterpret_cast<unsigned long long*>(arrive_target.data_ptr());
  a.traffic_matrix = ptr_or_null<int>(traffic);
  a.send_pos = ptr_or_null<int>(send_pos);
  a.epoch_dev = reinterpret_cast<unsigned long long*>(epoch_dev_ptr);
  a.status = st.d; a.timeout_ns = timeout_ns;
  cu_check(launch_splits_scan(a, stream_now()), "splits_scan");
}

void zero_pad_rows(torch::Tensor buf, torch::Tensor group_off, torch::Tensor group_rows) {
  TORCH_CHECK(buf.is_cuda() && buf.dim() == 2 && buf.is_contiguous(), "buf: contiguous CUDA matrix");
  cu_check(launch_zero_pad_rows(buf.data_ptr(), buf.size(1) * buf.element_size(), group_off.data_ptr<int>(), group_rows.data_ptr<int>(),
                                static_cast<int>(group_rows.numel()), stream_now()), "zero_pad_rows");
}

void dispatch_push(const HeapPy& heap, torch::Tensor x, torch::Tensor topk_idx, c10::optional<torch::Tensor> row_scale, torch::Tensor slot_in_block,
                   torch::Tensor block_base, torch::Tensor send_base, torch::Tensor dest_row, bool compute_rows, bool fp8, int64_t recv_off,
                   int64_t scale_off, int64_t arrive_off, int64_t entry_flags_off, uint64_t entry_epoch, const StatusPy& st, uint64_t timeout_ns, int ctas,
                   c10::optional<torch::Tensor> send_list, int tile_rows, int num_tiles, c10::optional<torch::Tensor> xq,
                   c10::optional<torch::Tensor> xq_scales) {
  want(x, torch::kBFloat16, "x"); want(topk_idx, torch::kInt32, "topk_idx"); want(dest_row, torch::kInt32, "dest_row");
  DispatchArgs a{};
  a.peer_table = heap.h->device_peer_table(); a.rank = heap.h->rank(); a.world = heap.h->world();
  a.num_experts = static_cast<int>(send_base.numel()); a.T = static_cast<int>(x.size(0)); a.H = static_cast<int>(x.size(1));
  a.K = static_cast<int>(topk_idx.size(1));
  a.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()); a.topk_idx = topk_idx.data_ptr<int>(); a.row_scale = ptr_or_null<const float>(row_scale);
  a.slot_in_block = slot_in_block.data_ptr<int>(); a.block_base = block_base.data_ptr<int>(); a.send_base = send_base.data_ptr<int>();
  a.dest_row = dest_row.data_ptr<int>(); a.compute_rows = compute_rows; a.fp8 = fp8;
  a.send_list = ptr_or_null<const int>(send_list);
  a.tile_rows = tile_rows; a.num_tiles = num_tiles;
  if (xq.has_value()) {
    TORCH_CHECK(fp8 && xq_scales.has_value(), "dispatch_push: xq needs fp8 and xq_scales");
    want(*xq, torch::kUInt8, "xq"); want(*xq_scales, torch::kFloat32, "xq_scales");
    TORCH_CHECK(xq->numel() >= x.numel() && xq_scales->numel() >= x.numel() / 128, "dispatch_push: xq / xq_scales too small");
    a.xq = xq->data_ptr<uint8_t>(); a.xq_scales = xq_scales->data_ptr<float>();
  }
  a.recv_heap_off = recv_off; a.scale_heap_off = scale_off; a.arrive_heap_off = arrive_off;
  a.entry_flags_heap_off = entry_flags_off; a.entry_epoch = entry_epoch; a.status = st.d; a.timeout_ns = timeout_ns;
  cu_check(launch_dispatch_push(a, ctas, stream_now()), "dispatch_push");
}

void combine_pull(const HeapPy& heap, int num_experts, torch::Tensor topk_idx, torch::Tensor dest_row, c10::optional<torch::Tensor> weights, int64_t src_off,
                  int64_t ready_off, uint64_t ready_epoch, c10::optional<torch::Tensor> out, c10::optional<torch::Tensor> dot_with,
                  c10::optional<torch::Tensor> dot_out, int H, const StatusPy& st, uint64_t timeout_ns, int ctas, int64_t epoch_dev_ptr) {
  CombineArgs a{};
  a.peer_table = heap.h->device_peer_table(); a.rank = heap.h->rank(); a.world = heap.h->world(); a.num_experts = num_experts;
  a.T = static_cast<int>(topk_idx.size(0)); a.K = static_cast<int>(topk_idx.size(1)); a.H = H;
  a.topk_idx = topk_idx.data_ptr<int>(); a.dest_row = dest_row.data_ptr<int>(); a.weights = ptr_or_null<const float>(weights);
  a.src_heap_off = src_off; a.ready_flags_heap_off = ready_off; a.ready_epoch = ready_epoch;
  a.epoch_dev = reinterpret_cast<const unsigned long long*>(epoch_dev_ptr);
  a.out = ptr_or_null<__nv_bfloat16>(out); a.dot_with = ptr_or_null<const __nv_bfloat16>(dot_with); a.dot_out = ptr_or_null<float>(dot_out);
  TORCH_CHECK((a.out != nullptr) != (a.dot_out != nullptr), "combine_pull: give either out or dot_out");
  a.status = st.d; a.timeout_ns = timeout_ns;
  cu_check(launch_combine_pull(a, ctas, stream_now()), "combine_pull");
}

}  // namespace

void bind_moe(py::module_& m) {
  py::class_<TensorMap2D>(m, "TensorMap2D").def(py::init<int64_t, int64_t, int64_t, int64_t, int, int>()).def_static("bytes", &TensorMap2D::bytes);
  m.def("grouped_gemm", &grouped_gemm, py::arg("mode"), py::arg("epilogue"), py::arg("a"), py::arg("b"), py::arg("group_off"), py::arg("tiles_n"),
        py::arg("fixed_m_tiles"), py::arg("red_len"), py::arg("b_rows_per_group"), py::arg("c_rows_per_group"), py::arg("c"), py::arg("c2"),
        py::arg("status_ptr"), py::arg("timeout_ns"), py::arg("ctas"), py::arg("gate_counter_ptr"), py::arg("gate_target"), py::arg("pair"),
        py::arg("band_rows"), py::arg("map_c") = nullptr, py::arg("map_c2") = nullptr, py::arg("direct_epilogue") = false, py::arg("a_scales") = py::none(),
        py::arg("group_rows") = py::none(), py::arg("gate_tile_rows") = 0);
  m.def("grouped_gemm_smem_bytes", &grouped_gemm_smem_bytes);
  m.attr("ROUTE_TOKENS_PER_BLOCK") = kRouteTokensPerBlock;
  m.def("route_topk", &route_topk);
  m.def("splits_scan", &splits_scan, py::arg("heap"), py::arg("counts_off"), py::arg("flags_off"), py::arg("epoch"), py::arg("block_cnt"), py::arg("block_base"),
        py::arg("send_base"), py::arg("send_cnt"), py::arg("group_off"), py::arg("group_rows"), py::arg("arrive_target"), py::arg("traffic"),
        py::arg("num_channels"), py::arg("row_align"), py::arg("cap_rows"), py::arg("status"), py::arg("timeout_ns"), py::arg("send_pos"),
        py::arg("epoch_dev_ptr"), py::arg("tile_target") = py::none(), py::arg("tile_rows") = 0);
  m.def("zero_pad_rows", &zero_pad_rows);
  m.def("build_send_list", [](torch::Tensor topk_idx, torch::Tensor slot_in_block, torch::Tensor block_base, torch::Tensor send_pos, torch::Tensor list, const StatusPy& st) {
    want(topk_idx, torch::kInt32, "topk_idx"); want(send_pos, torch::kInt32, "send_pos"); want(list, torch::kInt32, "list");
    TORCH_CHECK(list.numel() >= topk_idx.numel(), "build_send_list: list too short");
    cu_check(launch_build_send_list(topk_idx.data_ptr<int>(), slot_in_block.data_ptr<int>(), block_base.data_ptr<int>(), send_pos.data_ptr<int>(),
                                    static_cast<int>(topk_idx.size(0)), static_cast<int>(topk_idx.size(1)), static_cast<int>(send_pos.numel()),
                                    list.data_ptr<int>(), st.d, stream_now()), "build_send_list");
  });
  m.def("norm_gate_smem_bytes", [](int E, int H, int K, bool backward) { return static_cast<int64_t>(norm_gate_smem_bytes(E, H, K, backward)); });
  m.def("norm_gate_route", [](torch::Tensor h, torch::Tensor norm_w, torch::Tensor gate, c10::optional<torch::Tensor> bias, int K, double eps, torch::Tensor hn,
                              torch::Tensor rstd, torch::Tensor logits, torch::Tensor topk_idx, torch::Tensor topk_w, torch::Tensor slot_in_block,
                              torch::Tensor block_cnt) {
    want(h, torch::kBFloat16, "h"); want(norm_w, torch::kBFloat16, "norm_w"); want(gate, torch::kBFloat16, "gate"); want(hn, torch::kBFloat16, "hn");
    want(rstd, torch::kFloat32, "rstd"); want(logits, torch::kFloat32, "logits"); want(topk_idx, torch::kInt32, "topk_idx"); want(topk_w, torch::kFloat32, "topk_w");
    want(slot_in_block, torch::kInt32, "slot_in_block"); want(block_cnt, torch::kInt32, "block_cnt");
    NormGateArgs a{};
    a.T = static_cast<int>(h.size(0)); a.H = static_cast<int>(h.size(1)); a.num_experts = static_cast<int>(gate.size(0)); a.K = K; a.eps = static_cast<float>(eps);
    const int blocks = (a.T + kRouteTokensPerBlock - 1) / kRouteTokensPerBlock;
    TORCH_CHECK(gate.size(1) == a.H && norm_w.numel() == a.H && hn.sizes() == h.sizes() && rstd.numel() >= a.T && logits.numel() == static_cast<int64_t>(a.T) * a.num_experts &&
                topk_idx.numel() == static_cast<int64_t>(a.T) * K && topk_w.numel() == topk_idx.numel() &&
                slot_in_block.numel() >= static_cast<int64_t>(blocks) * kRouteTokensPerBlock * K && block_cnt.numel() >= static_cast<int64_t>(blocks) * a.num_experts,
                "norm_gate_route: shapes");
    a.h = reinterpret_cast<const __nv_bfloat16*>(h.data_ptr()); a.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w.data_ptr());
    a.gate = reinterpret_cast<const __nv_bfloat16*>(gate.data_ptr()); a.bias = ptr_or_null<const float>(bias);
    a.hn = reinterpret_cast<__nv_bfloat16*>(hn.data_ptr()); a.rstd = rstd.data_ptr<float>(); a.logits = logits.data_ptr<float>();
    a.topk_idx = topk_idx.data_ptr<int>(); a.topk_w = topk_w.data_ptr<float>(); a.slot_in_block = slot_in_block.data_ptr<int>(); a.block_cnt = block_cnt.data_ptr<int>();
    cu_check(launch_norm_gate_route(a, stream_now()), "norm_gate_route");
  });
  m.def("norm_gate_bwd", [](torch::Tensor h, torch::Tensor norm_w, torch::Tensor gate, torch::Tensor rstd, torch::Tensor topk_idx, torch::Tensor topk_w,
                            torch::Tensor grad_w, torch::Tensor grad_hn, torch::Tensor grad_h, torch::Tensor d_gate, torch::Tensor d_norm_w) {
    want(h, torch::kBFloat16, "h"); want(norm_w, torch::kBFloat16, "norm_w"); want(gate, torch::kBFloat16, "gate"); want(rstd, torch::kFloat32, "rstd");
    want(topk_idx, torch::kInt32, "topk_idx"); want(topk_w, torch::kFloat32, "topk_w"); want(grad_w, torch::kFloat32, "grad_w");
    want(grad_hn, torch::kBFloat16, "grad_hn"); want(grad_h, torch::kBFloat16, "grad_h"); want(d_gate, torch::kFloat32, "d_gate"); want(d_norm_w, torch::kFloat32, "d_norm_w");
    NormGateBwdArgs a{};
    a.T = static_cast<int>(h.size(0)); a.H = static_cast<int>(h.size(1)); a.num_experts = static_cast<int>(gate.size(0)); a.K = static_cast<int>(topk_idx.size(1));
    TORCH_CHECK(gate.size(1) == a.H && grad_hn.sizes() == h.sizes() && grad_h.sizes() == h.sizes() && d_gate.numel() == gate.numel() && d_norm_w.numel() == a.H &&
                grad_w.sizes() == topk_idx.sizes() && topk_w.sizes() == topk_idx.sizes() && rstd.numel() >= a.T, "norm_gate_bwd: shapes");
    a.h = reinterpret_cast<const __nv_bfloat16*>(h.data_ptr()); a.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w.data_ptr());
    a.gate = reinterpret_cast<const __nv_bfloat16*>(gate.data_ptr()); a.rstd = rstd.data_ptr<float>(); a.topk_idx = topk_idx.data_ptr<int>();
    a.topk_w = topk_w.data_ptr<float>(); a.grad_w = grad_w.data_ptr<float>(); a.grad_hn = reinterpret_cast<const __nv_bfloat16*>(grad_hn.data_ptr());
    a.grad_h = reinterpret_cast<__nv_bfloat16*>(grad_h.data_ptr()); a.d_gate = d_gate.data_ptr<float>(); a.d_norm_w = d_norm_w.data_ptr<float>();
    cu_check(launch_norm_gate_bwd(a, stream_now()), "norm_gate_bwd");
  });
  m.def("dispatch_push", &dispatch_push, py::arg("heap"), py::arg("x"), py::arg("topk_idx"), py::arg("row_scale"), py::arg("slot_in_block"), py::arg("block_base"),
        py::arg("send_base"), py::arg("dest_row"), py::arg("compute_rows"), py::arg("fp8"), py::arg("recv_off"), py::arg("scale_off"), py::arg("arrive_off"),
        py::arg("entry_flags_off"), py::arg("entry_epoch"), py::arg("status"), py::arg("timeout_ns"), py::arg("ctas"), py::arg("send_list"),
        py::arg("tile_rows") = 0, py::arg("num_tiles") = 0, py::arg("xq") = py::none(), py::arg("xq_scales") = py::none());
  m.def("quantise_rows", [](torch::Tensor x, torch::Tensor q, torch::Tensor scales, int ctas) {
    want(x, torch::kBFloat16, "x"); want(q, torch::kUInt8, "q"); want(scales, torch::kFloat32, "scales");
    TORCH_CHECK(x.dim() == 2 && q.numel() >= x.numel() && scales.numel() >= x.numel() / 128, "quantise_rows: q / scales too small");
    cu_check(launch_quantise_rows(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)),
                                  q.data_ptr<uint8_t>(), scales.data_ptr<float>(), ctas, stream_now()), "quantise_rows");
  });
  m.def("combine_pull", &combine_pull);
  m.def("peer_signal", [](const HeapPy& heap, int64_t flags_off, uint64_t epoch, int64_t epoch_dev_ptr) {
    cu_check(launch_peer_signal(heap.h->device_peer_table(), heap.h->rank(), heap.h->world(), flags_off, epoch,
                                reinterpret_cast<const unsigned long long*>(epoch_dev_ptr), stream_now()), "peer_signal");
  });
  m.def("wait_counters", [](int64_t counter_ptr, torch::Tensor target, const StatusPy& st, uint64_t timeout_ns) {
    cu_check(launch_wait_counters(reinterpret_cast<const unsigned long long*>(counter_ptr), reinterpret_cast<const unsigned long long*>(target.data_ptr()),
                                  static_cast<int>(target.numel()), st.d, timeout_ns, stream_now()), "wait_counters");
  });
  m.def("swiglu_fwd", [](torch::Tensor gu, torch::Tensor act) {
    want(gu, torch::kBFloat16, "gate_up"); want(act, torch::kBFloat16, "act");
    cu_check(launch_swiglu_fwd(reinterpret_cast<const __nv_bfloat16*>(gu.data_ptr()), reinterpret_cast<__nv_bfloat16*>(act.data_ptr()), gu.size(0),
                               static_cast<int>(act.size(1)), stream_now()), "swiglu_fwd");
  });
  m.def("swiglu_bwd", [](torch::Tensor gu, torch::Tensor dact, torch::Tensor dgu, int64_t rows_dev_ptr) {
    want(gu, torch::kBFloat16, "gate_up"); want(dact, torch::kBFloat16, "d_act"); want(dgu, torch::kBFloat16, "d_gate_up");
    cu_check(launch_swiglu_bwd(reinterpret_cast<const __nv_bfloat16*>(gu.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(dact.data_ptr()),
                               reinterpret_cast<__nv_bfloat16*>(dgu.data_ptr()), gu.size(0), static_cast<int>(dact.size(1)), reinterpret_cast<const int*>(rows_dev_ptr),
                               stream_now()), "swiglu_bwd");
  });
  m.def("dequant_fp8", [](torch::Tensor q, torch::Tensor scales, torch::Tensor out, int64_t rows_dev_ptr) {
    want(q, torch::kUInt8, "q"); want(scales, torch::kFloat32, "scales"); want(out, torch::kBFloat16, "out");
    cu_check(launch_dequant_fp8(q.data_ptr<uint8_t>(), scales.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), q.size(0),
                                static_cast<int>(q.size(1)), reinterpret_cast<const int*>(rows_dev_ptr), stream_now()), "dequant_fp8");
  });
  m.def("sumsq_add", [](torch::Tensor a, torch::Tensor b, double scale, torch::Tensor partial, torch::Tensor out) {
    want(a, torch::kBFloat16, "a"); want(b, torch::kBFloat16, "b"); want(partial, torch::kFloat32, "partial"); want(out, torch::kFloat32, "out");
    TORCH_CHECK(a.numel() == b.numel(), "sumsq_add: shapes");
    cu_check(launch_sumsq_add(reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()), a.numel(),
                              static_cast<float>(scale), partial.data_ptr<float>(), static_cast<int>(partial.numel()), out.data_ptr<float>(), stream_now()), "sumsq_add");
  });
  m.def("scaled_sum", [](torch::Tensor a, torch::Tensor b, torch::Tensor gscale, double factor, torch::Tensor out) {
    want(a, torch::kBFloat16, "a"); want(b, torch::kBFloat16, "b"); want(gscale, torch::kFloat32, "gscale"); want(out, torch::kBFloat16, "out");
    cu_check(launch_scaled_sum(reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()), a.numel(),
                               gscale.data_ptr<float>(), static_cast<float>(factor), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), stream_now()), "scaled_sum");
  });
  m.def("embedding_bwd", [](torch::Tensor sorted_ids, torch::Tensor perm, torch::Tensor grad_out, torch::Tensor grad_table) {
    want(sorted_ids, torch::kInt64, "sorted_ids"); want(perm, torch::kInt64, "perm"); want(grad_out, torch::kBFloat16, "grad_out");
    want(grad_table, torch::kBFloat16, "grad_table");
    cu_check(launch_embedding_bwd(reinterpret_cast<const long long*>(sorted_ids.data_ptr()), reinterpret_cast<const long long*>(perm.data_ptr()),
                                  reinterpret_cast<const __nv_bfloat16*>(grad_out.data_ptr()), reinterpret_cast<__nv_bfloat16*>(grad_table.data_ptr()),
                                  sorted_ids.numel(), static_cast<int>(grad_out.size(1)), stream_now()), "embedding_bwd");
  });
  m.def("embedding_index", [](torch::Tensor ids, int V) {
    want(ids, torch::kInt64, "ids");
    const int64_t T = ids.numel();
    const int64_t blocks = (T + embedding_index_block() - 1) / embedding_index_block();
    auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(ids.device());
    auto hist = torch::empty({blocks, V}, i32), rank = torch::empty({T}, i32), total = torch::empty({V}, i32), start = torch::empty({V + 1}, i32);
    auto sorted_ids = torch::empty({T}, ids.options()), perm = torch::empty({T}, ids.options());
    cu_check(launch_embedding_index(reinterpret_cast<const long long*>(ids.data_ptr()), T, V, hist.data_ptr<int>(), rank.data_ptr<int>(), total.data_ptr<int>(),
                                    start.data_ptr<int>(), reinterpret_cast<long long*>(sorted_ids.data_ptr()), reinterpret_cast<long long*>(perm.data_ptr()), stream_now()),
             "embedding_index");
    return std::make_tuple(sorted_ids, perm);
  });
  m.def("adamw", [](torch::Tensor param, torch::Tensor master, torch::Tensor m1, torch::Tensor v, torch::Tensor grad, double lr, double b1, double b2,
                    double eps, double wd, int64_t step, double grad_scale) {
    want(param, torch::kBFloat16, "param"); want(master, torch::kFloat32, "master"); want(m1, torch::kFloat32, "m"); want(v, torch::kFloat32, "v");
    want(grad, torch::kBFloat16, "grad");
    const double c1 = 1.0 / (1.0 - std::pow(b1, static_cast<double>(step))), c2 = 1.0 / (1.0 - std::pow(b2, static_cast<double>(step)));
    cu_check(launch_adamw(reinterpret_cast<__nv_bfloat16*>(param.data_ptr()), master.data_ptr<float>(), m1.data_ptr<float>(), v.data_ptr<float>(),
                          reinterpret_cast<const __nv_bfloat16*>(grad.data_ptr()), param.numel(), static_cast<float>(lr), static_cast<float>(b1),
                          static_cast<float>(b2), static_cast<float>(eps), static_cast<float>(wd), static_cast<float>(c1), static_cast<float>(c2),
                          static_cast<float>(grad_scale), stream_now()), "adamw");
  });
}
