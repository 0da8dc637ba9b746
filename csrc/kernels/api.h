// C launch surface of the sm_100a kernels (no torch types; raw pointers + stream).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../runtime/device_sync.cuh"

namespace fastb {

// ---------------------------------------------------------------------------------------------
// a2a_push: executes one rank's work list of a staged / fan-out all-to-all(v) plan.
// ---------------------------------------------------------------------------------------------
struct A2AWork {
  long long src_off, dst_off, bytes;
  int dst_rank;
  unsigned char src_buf, dst_buf, wait_kind, signal_kind;
  int stage, wait_stage;
  int pad_;
};
static_assert(sizeof(A2AWork) == 48, "A2AWork layout is shared with the host packer");

constexpr int kSigReadyOff = 0;      // u64 ready[world]   (written by peers: their current epoch)
constexpr int kSigMaxWorld = 64;
constexpr int kSigCounterOff = kSigMaxWorld;  // u64 counters: [0] balance, [1] output, [2+k] rail stage k
constexpr int kSigMaxStages = 4096;
constexpr int kSigTicketOff = kSigCounterOff + 2 + kSigMaxStages;  // u64 CTA exit ticket
constexpr int kSigWords = kSigTicketOff + 2;

struct A2ARankArgs {
  const A2AWork* items;
  int n_items, rank, world, num_stages;
  void* const* peer_table;               // [world] slab bases (device array)
  const unsigned char* src_base[4];      // local bases of input / output / balance / rail
  long long dst_heap_off[4];             // slab offsets of the same four buffers on every rank
  long long sig_heap_off;                // slab offset of the signal block (kSigWords u64)
  unsigned long long epoch;              // 1, 2, 3, ... per collective on this communicator
  unsigned long long expect_output, expect_balance;
  const unsigned long long* expect_rail; // [num_stages] bytes landing in my rail staging
  DeviceStatus* status;
  unsigned long long timeout_ns;
};

// device_args == nullptr: one real rank, `host_args` is passed by value. Otherwise one cooperative
// launch with gridDim.y = virtual_ranks runs every rank of an in-process group (single-GPU
// emulation); `device_args` points to an array of virtual_ranks structs in device memory.
cudaError_t launch_a2a_push(const A2ARankArgs* host_args, const A2ARankArgs* device_args, int virtual_ranks, int ctas,
                            int threads, cudaStream_t stream);

// Waits (bounded) on a flag nothing sets; used to test the timeout path without any peer.
cudaError_t launch_wait_probe(const unsigned long long* flag, unsigned long long want, DeviceStatus* status,
                              unsigned long long timeout_ns, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// grouped_gemm: tcgen05 / TMEM grouped bf16 GEMM (forward, dgrad, wgrad) with optional SwiGLU.
// ---------------------------------------------------------------------------------------------
enum class GemmMode : int { kForward = 0, kDgrad = 1, kWgrad = 2 };
enum class GemmEpilogue : int { kStore = 0, kSwiGLU = 1 };

struct GemmArgs {
  const int* group_off;    // [num_groups + 1] row offsets of the groups, multiples of 128 (device)
  int num_groups;
  int tiles_n;             // tiles along the output columns (columns / 256)
  int fixed_m_tiles;       // wgrad only: tiles along the output rows of one group (rows / 128)
  int red_len;             // forward / dgrad: reduction length (multiple of 64)
  int b_rows_per_group;    // rows of one group's slice in operand B's matrix (forward: N, dgrad: N)
  int c_rows_per_group;    // wgrad only: output rows per group
  __nv_bfloat16* c;        // output; SwiGLU: activations [rows, columns / 2]
  long long ldc;
  __nv_bfloat16* c2;       // SwiGLU only, optional: raw gate|up tile output [rows, columns]
  long long ldc2;
  DeviceStatus* status;
  unsigned long long timeout_ns;
};

int grouped_gemm_smem_bytes();
// Tensor maps (bf16, 128-byte swizzle) must use these boxes: forward A {64,128} B {64,256};
// dgrad A {64,128} B {64,64}; wgrad A {64,64} B {64,64}  ({inner, outer} elements).
cudaError_t launch_grouped_gemm(GemmMode mode, GemmEpilogue epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& args,
                                int ctas, cudaStream_t stream);

}  // namespace fastb
