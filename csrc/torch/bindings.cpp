// Python bindings (torch extension module fast_b200._C): symmetric heap, status blocks, and the
// launchers of every sm_100a kernel. Takes the place of the reference's TORCH_LIBRARY class
// flash_comm_t (nvidia/alltoall_nvshmem.cpp:390-662) and pybind module flash_t
// (amd/flash.cpp:650-666); the user-facing API built on top lives in fast_b200/parallel.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <memory>

#include "py_types.h"

namespace py = pybind11;
using namespace fastb;
using namespace fastb_py;

namespace {


// ---- a2a program ----------------------------------------------------------------------------------
struct A2AProgramPy {
  torch::Tensor items_dev, expect_rail_dev;
  int n_items = 0, num_stages = 0;
  bool has_waits = false;  // some item waits for bytes another item of a peer's (or this) launch forwards
  unsigned long long expect_output = 0, expect_balance = 0;
  int64_t total_bytes = 0;

  // items: int64[k, 10] as produced by Plan.lower(); expect_rail: list of bytes per stage.
  A2AProgramPy(torch::Tensor items, std::vector<int64_t> expect_rail, int64_t exp_out, int64_t exp_bal, int device) {
    TORCH_CHECK(items.dim() == 2 && items.size(1) == 10 && items.dtype() == torch::kInt64 && items.is_cpu(), "items must be CPU int64[k, 10]");
    TORCH_CHECK(static_cast<int>(expect_rail.size()) <= kSigMaxStages, "too many stages for the signal block");
    n_items = static_cast<int>(items.size(0));
    num_stages = static_cast<int>(expect_rail.size());
    expect_output = static_cast<unsigned long long>(exp_out);
    expect_balance = static_cast<unsigned long long>(exp_bal);
    auto host = torch::empty({std::max(n_items, 1), static_cast<int64_t>(sizeof(A2AWork))}, torch::kUInt8);
    A2AWork* w = reinterpret_cast<A2AWork*>(host.data_ptr());
    auto it = items.contiguous();
    const int64_t* q = it.data_ptr<int64_t>();
    for (int i = 0; i < n_items; ++i, q += 10) {
      w[i].src_off = q[0]; w[i].dst_off = q[1]; w[i].bytes = q[2]; w[i].dst_rank = static_cast<int>(q[3]);
      w[i].src_buf = static_cast<unsigned char>(q[4]); w[i].dst_buf = static_cast<unsigned char>(q[5]);
      w[i].wait_kind = static_cast<unsigned char>(q[6]); w[i].signal_kind = static_cast<unsigned char>(q[7]);
      w[i].stage = static_cast<int>(q[8]); w[i].wait_stage = static_cast<int>(q[9]); w[i].pad_ = 0;
      total_bytes += q[2];
      if (q[6] != 0) has_waits = true;
    }
    auto dev = torch::Device(torch::kCUDA, device);
    items_dev = host.to(dev);
    auto er = torch::empty({std::max(num_stages, 1)}, torch::kInt64);
    for (int k = 0; k < num_stages; ++k) er[k] = expect_rail[k];
    expect_rail_dev = er.to(dev);
  }

  A2ARankArgs args(const HeapPy& heap, std::array<int64_t, 4> src_ptrs, std::array<int64_t, 4> dst_offs, int64_t sig_off,
                   uint64_t epoch, const StatusPy& st, uint64_t timeout_ns, int64_t stamps_ptr = 0) const {
    A2ARankArgs a{};
    a.items = reinterpret_cast<const A2AWork*>(items_dev.data_ptr());
    a.n_items = n_items; a.rank = heap.h->rank(); a.world = heap.h->world(); a.num_stages = num_stages;
    a.peer_table = heap.h->device_peer_table();
    for (int i = 0; i < 4; ++i) { a.src_base[i] = reinterpret_cast<const unsigned char*>(src_ptrs[i]); a.dst_heap_off[i] = dst_offs[i]; }
    a.sig_heap_off = sig_off; a.epoch = epoch; a.expect_output = expect_output; a.expect_balance = expect_balance;
    a.expect_rail = reinterpret_cast<const unsigned long long*>(expect_rail_dev.data_ptr());
    a.status = st.d; a.timeout_ns = timeout_ns;
    a.phase_stamps = reinterpret_cast<unsigned long long*>(stamps_ptr);
    return a;
  }
};

void a2a_launch(const A2AProgramPy& p, const HeapPy& heap, std::array<int64_t, 4> src_ptrs, std::array<int64_t, 4> dst_offs,
                int64_t sig_off, uint64_t epoch, const StatusPy& st, uint64_t timeout_ns, int ctas, int threads, int64_t stamps_ptr, bool bulk) {
  TORCH_CHECK(heap.h->world() <= kSigMaxWorld, "world larger than the signal block supports");
  A2ARankArgs a = p.args(heap, src_ptrs, dst_offs, sig_off, epoch, st, timeout_ns, stamps_ptr);
  a.bulk = bulk ? 1 : 0;
  cuda_check(launch_a2a_push(&a, nullptr, 1, ctas, threads, cur_stream(), p.has_waits), "a2a_push launch");
}

// One cooperative launch that runs every virtual rank of an in-process group.
void a2a_launch_group(std::vector<const A2AProgramPy*> progs, std::vector<const HeapPy*> heaps,
                      std::vector<std::array<int64_t, 4>> src_ptrs, std::array<int64_t, 4> dst_offs, int64_t sig_off, uint64_t epoch,
                      std::vector<const StatusPy*> sts, uint64_t timeout_ns, int ctas, int threads) {
  const int n = static_cast<int>(progs.size());
  TORCH_CHECK(n >= 1 && static_cast<int>(heaps.size()) == n && static_cast<int>(src_ptrs.size()) == n && static_cast<int>(sts.size()) == n, "one entry per virtual rank");
  std::vector<A2ARankArgs> host(n);
  for (int r = 0; r < n; ++r) host[r] = progs[r]->args(*heaps[r], src_ptrs[r], dst_offs, sig_off, epoch, *sts[r], timeout_ns);
  auto dev = torch::empty({static_cast<int64_t>(n * sizeof(A2ARankArgs))}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, heaps[0]->device));
  cuda_check(cudaMemcpyAsync(dev.data_ptr(), host.data(), n * sizeof(A2ARankArgs), cudaMemcpyHostToDevice, cur_stream()), "upload group args");
  cuda_check(launch_a2a_push(nullptr, reinterpret_cast<const A2ARankArgs*>(dev.data_ptr()), n, ctas, threads, cur_stream()), "a2a_push group launch");
  cuda_check(cudaStreamSynchronize(cur_stream()), "a2a_push group sync");  // args buffer must outlive the launch
}

}  // namespace

void bind_moe(py::module_& m);  // defined in moe_bindings.cpp

PYBIND11_MODULE(_C, m) {
  m.doc() = "fast_b200 native runtime and sm_100a kernels";
  m.attr("SIG_WORDS") = kSigWords;

  py::class_<HeapPy>(m, "SymmHeap")
      .def(py::init([](int rank, int world, int64_t bytes, int device) {
        c10::cuda::CUDAGuard g(device);
        return HeapPy{std::make_shared<SymmHeap>(rank, world, static_cast<size_t>(bytes)), device};
      }))
      .def_static("create_local_group", [](int world, int64_t bytes, int device) {
        c10::cuda::CUDAGuard g(device);
        std::vector<HeapPy> out;
        for (SymmHeap* h : SymmHeap::create_local_group(world, static_cast<size_t>(bytes))) out.push_back(HeapPy{std::shared_ptr<SymmHeap>(h), device});
        return out;
      })
      .def_static("create_device_group", [](std::vector<int> devices, int64_t bytes) {
        std::vector<HeapPy> out;
        auto hs = SymmHeap::create_device_group(devices, static_cast<size_t>(bytes));
        for (size_t r = 0; r < hs.size(); ++r) out.push_back(HeapPy{std::shared_ptr<SymmHeap>(hs[r]), devices[r]});
        return out;
      })
      .def("ipc_handle", [](const HeapPy& h) { return py::bytes(h.h->ipc_handle()); })
      .def("open_peers", [](HeapPy& h, std::vector<std::string> handles) { c10::cuda::CUDAGuard g(h.device); h.h->open_peers(handles); })
      .def("close_peers", [](HeapPy& h) { c10::cuda::CUDAGuard g(h.device); h.h->close_peers(); })
      .def("alloc", [](HeapPy& h, int64_t bytes) { return static_cast<int64_t>(h.h->alloc(static_cast<size_t>(bytes))); })
      .def("free", [](HeapPy& h, int64_t off) { h.h->free(static_cast<size_t>(off)); })
      .def("tensor", &HeapPy::tensor)
      .def("base_ptr", [](const HeapPy& h, int r) { return reinterpret_cast<int64_t>(h.h->peer_base(r)); })
      .def("table_ptr", [](const HeapPy& h) { return reinterpret_cast<int64_t>(h.h->device_peer_table()); })
      .def_property_readonly("rank", [](const HeapPy& h) { return h.h->rank(); })
      .def_property_readonly("world", [](const HeapPy& h) { return h.h->world(); })
      .def_property_readonly("bytes", [](const HeapPy& h) { return static_cast<int64_t>(h.h->bytes()); })
      .def_property_readonly("in_use", [](const HeapPy& h) { return static_cast<int64_t>(h.h->in_use()); });

  py::class_<StatusPy>(m, "StatusBlock")
      .def(py::init<>())
      .def("read", &StatusPy::read)
      .def("clear", &StatusPy::clear)
      .def("ptr", [](const StatusPy& s) { return reinterpret_cast<int64_t>(s.d); });

  py::class_<A2AProgramPy>(m, "A2AProgram")
      .def(py::init<torch::Tensor, std::vector<int64_t>, int64_t, int64_t, int>())
      .def_readonly("n_items", &A2AProgramPy::n_items)
      .def_readonly("num_stages", &A2AProgramPy::num_stages)
      .def_readonly("has_waits", &A2AProgramPy::has_waits)
      .def_readonly("total_bytes", &A2AProgramPy::total_bytes);

  m.def("a2a_launch", &a2a_launch, py::arg("program"), py::arg("heap"), py::arg("src_ptrs"), py::arg("dst_offs"), py::arg("sig_off"), py::arg("epoch"),
        py::arg("status"), py::arg("timeout_ns"), py::arg("ctas"), py::arg("threads"), py::arg("stamps_ptr") = 0, py::arg("bulk") = false);
  m.attr("PHASE_STAMP_WORDS") = kPhaseStampWords;
  m.attr("SIG_MAX_WORLD") = kSigMaxWorld;
  m.def("a2a_launch_group", &a2a_launch_group);
  m.def("wait_probe", [](int64_t flag_ptr, uint64_t want, const StatusPy& st, uint64_t timeout_ns) {
    cuda_check(launch_wait_probe(reinterpret_cast<const unsigned long long*>(flag_ptr), want, st.d, timeout_ns, cur_stream()), "wait_probe");
  });
  m.def("launch_count", &launch_count);
  bind_moe(m);
}
