// Symmetric heap: one device slab per rank, mapped into every peer, carved by an allocator whose
// decisions are identical on all ranks (same call sequence -> same offsets), so a buffer is
// addressed on any peer as peer_base[r] + offset.
//
// Replaces the reference's NVSHMEM symmetric heap + CUDA-IPC "shared_memory_t" mapping
// (nvidia/src/fast_alltoall/flash_alltoall_nvshmem.cu:68-91, :1411-1640;
//  nvidia/alltoall_nvshmem.cpp:476-506). Handles are exchanged by the caller (torch.distributed).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "range_allocator.h"

namespace fastb {

constexpr int kIpcHandleBytes = 64;

class SymmHeap {
 public:
  // Real multi-process rank: allocates the local slab on the current device.
  SymmHeap(int rank, int world, size_t bytes);
  // In-process group of `world` virtual ranks on the current device (single-GPU emulation and
  // tests): returns heaps that already see each other.
  static std::vector<SymmHeap*> create_local_group(int world, size_t bytes);
  // In-process group with rank r on CUDA device devices[r] (peer access is enabled between them): one process
  // driving several GPUs, e.g. to profile one rank's kernel while it writes real peer memory over NVLink.
  static std::vector<SymmHeap*> create_device_group(const std::vector<int>& devices, size_t bytes);
  ~SymmHeap();

  std::string ipc_handle() const;                          // 64 raw bytes
  void open_peers(const std::vector<std::string>& handles);  // handles[r] from rank r

  // Two-phase teardown. CUDA leaves freeing an exported allocation undefined while an importer
  // still has it mapped, so every rank first unmaps its peers (close_peers), the ranks meet in a
  // host barrier, and only then does anybody free its own slab (free_local, or the destructor).
  // Both are idempotent; after close_peers the heap can no longer reach a peer.
  void close_peers();
  void free_local();
  bool peers_open() const { return opened_ && world_ > 1 && !ipc_opened_.empty(); }

  int rank() const { return rank_; }
  int world() const { return world_; }
  size_t bytes() const { return bytes_; }
  void* local_base() const { return peer_base_[rank_]; }
  void* peer_base(int r) const { return peer_base_[r]; }
  void* const* device_peer_table() const { return d_table_; }  // device array [world] of slab bases

  // Offsets are multiples of 256 B. Throws std::runtime_error when full.
  size_t alloc(size_t bytes) { return ranges_.alloc(bytes); }
  void free(size_t offset) { ranges_.free(offset); }
  size_t in_use() const { return ranges_.in_use(); }

 private:
  SymmHeap() = default;
  void upload_table();
  int rank_ = 0, world_ = 1;
  size_t bytes_ = 0;
  bool opened_ = false;
  bool owns_slab_ = true;
  std::vector<char> ipc_opened_;  // peers mapped through an IPC handle (closed in the destructor)
  std::vector<void*> peer_base_;
  void** d_table_ = nullptr;
  RangeAllocator ranges_;
};

}  // namespace fastb
