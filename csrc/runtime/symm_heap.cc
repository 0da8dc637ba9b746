#include "symm_heap.h"

#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>

namespace fastb {

namespace {
void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("SymmHeap: ") + what + ": " + cudaGetErrorString(e));
}
}  // namespace

SymmHeap::SymmHeap(int rank, int world, size_t bytes) : rank_(rank), world_(world), bytes_(bytes) {
  if (rank < 0 || rank >= world) throw std::invalid_argument("SymmHeap: rank out of range");
  peer_base_.assign(world, nullptr);
  void* p = nullptr;
  check(cudaMalloc(&p, bytes), "cudaMalloc slab");
  check(cudaMemset(p, 0, bytes), "cudaMemset slab");
  peer_base_[rank] = p;
  ranges_ = RangeAllocator(bytes);
  if (world == 1) { opened_ = true; upload_table(); }
}

std::vector<SymmHeap*> SymmHeap::create_local_group(int world, size_t bytes) {
  std::vector<SymmHeap*> hs;
  std::vector<void*> slabs(world, nullptr);
  for (int r = 0; r < world; ++r) {
    check(cudaMalloc(&slabs[r], bytes), "cudaMalloc slab");
    check(cudaMemset(slabs[r], 0, bytes), "cudaMemset slab");
  }
  for (int r = 0; r < world; ++r) {
    SymmHeap* h = new SymmHeap();
    h->rank_ = r; h->world_ = world; h->bytes_ = bytes;
    h->peer_base_ = slabs;
    h->ranges_ = RangeAllocator(bytes);
    h->opened_ = true;
    h->upload_table();
    hs.push_back(h);
  }
  return hs;
}

std::vector<SymmHeap*> SymmHeap::create_device_group(const std::vector<int>& devices, size_t bytes) {
  const int world = static_cast<int>(devices.size());
  if (world < 1) throw std::invalid_argument("SymmHeap: need at least one device");
  int before = 0;
  check(cudaGetDevice(&before), "cudaGetDevice");
  std::vector<void*> slabs(world, nullptr);
  for (int r = 0; r < world; ++r) {
    check(cudaSetDevice(devices[r]), "cudaSetDevice");
    for (int q = 0; q < world; ++q) {
      if (devices[q] == devices[r]) continue;
      const cudaError_t e = cudaDeviceEnablePeerAccess(devices[q], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();  // clears the sticky-free error
      else check(e, "cudaDeviceEnablePeerAccess");
    }
    check(cudaMalloc(&slabs[r], bytes), "cudaMalloc slab");
    check(cudaMemset(slabs[r], 0, bytes), "cudaMemset slab");
  }
  std::vector<SymmHeap*> hs;
  for (int r = 0; r < world; ++r) {
    check(cudaSetDevice(devices[r]), "cudaSetDevice");
    SymmHeap* h = new SymmHeap();
    h->rank_ = r; h->world_ = world; h->bytes_ = bytes;
    h->peer_base_ = slabs;
    h->ranges_ = RangeAllocator(bytes);
    h->opened_ = true;
    h->upload_table();  // the table lives on this rank's device
    hs.push_back(h);
  }
  check(cudaSetDevice(before), "cudaSetDevice");
  return hs;
}

void SymmHeap::close_peers() {
  for (int r = 0; r < world_; ++r) {
    if (r == rank_ || !peer_base_[r]) continue;
    if (r < static_cast<int>(ipc_opened_.size()) && ipc_opened_[r]) {
      cudaIpcCloseMemHandle(peer_base_[r]);
      ipc_opened_[r] = 0;
      peer_base_[r] = nullptr;
    }
  }
  ipc_opened_.clear();
}

void SymmHeap::free_local() {
  if (owns_slab_ && peer_base_[rank_]) cudaFree(peer_base_[rank_]);
  peer_base_[rank_] = nullptr;
  if (d_table_) { cudaFree(d_table_); d_table_ = nullptr; }
}

// Peers are unmapped before the local slab goes. Ranks that want the defined order across
// processes call close_peers(), meet in a barrier, and then drop the heap.
SymmHeap::~SymmHeap() {
  close_peers();
  free_local();
}

std::string SymmHeap::ipc_handle() const {
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, peer_base_[rank_]), "cudaIpcGetMemHandle");
  static_assert(sizeof(h) == kIpcHandleBytes, "unexpected IPC handle size");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void SymmHeap::open_peers(const std::vector<std::string>& handles) {
  if (static_cast<int>(handles.size()) != world_) throw std::invalid_argument("SymmHeap: need one handle per rank");
  ipc_opened_.assign(world_, 0);
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    if (handles[r].size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("SymmHeap: bad handle size");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handles[r].data(), sizeof(h));
    void* p = nullptr;
    check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    peer_base_[r] = p;
    ipc_opened_[r] = 1;
  }
  opened_ = true;
  upload_table();
}

void SymmHeap::upload_table() {
  if (!d_table_) check(cudaMalloc(reinterpret_cast<void**>(&d_table_), sizeof(void*) * world_), "cudaMalloc table");
  check(cudaMemcpy(d_table_, peer_base_.data(), sizeof(void*) * world_, cudaMemcpyHostToDevice), "upload table");
}

}  // namespace fastb
