// a2a_push: one persistent launch per rank that pushes every byte of an all-to-all(v) plan
// straight into peers' memory with 16-byte stores over NVLink, ordered by byte counters.
//
// Roles folded into this one kernel (reference kernels in
// nvidia/src/fast_alltoall/flash_alltoall_nvshmem.cu): balance all-to-all + completion flags
// (:2099-2238, :2459-2470), intrinsic all-to-all (:2240-2370), per-stage put (:1691-1737),
// credit / stage-ready waits (:1645-1689, :2451-2457), redistribute (:1881-2013) and the
// spread-out baseline (:674-822). Differences by design: data lands in its final slot whenever
// the rail GPU is the destination, staging regions are never reused inside a collective (no
// ping-pong credits), counters only grow inside a collective and are cleared by the last CTA
// after every wait has been satisfied, and each wait is bounded.
#include <atomic>

#include "api.h"

namespace fastb {

namespace {

__device__ __forceinline__ void copy_bytes(unsigned char* __restrict__ dst, const unsigned char* __restrict__ src, long long bytes) {
  const int tid = threadIdx.x, nt = blockDim.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | static_cast<uintptr_t>(bytes)) & 15u) == 0) {
    const int4* s = reinterpret_cast<const int4*>(src);
    int4* d = reinterpret_cast<int4*>(dst);
    const long long n = bytes >> 4;
    constexpr int U = 8;
    long long i = tid;
    for (; i + static_cast<long long>(U - 1) * nt < n; i += static_cast<long long>(U) * nt) {
      int4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = __ldcg(s + i + static_cast<long long>(u) * nt);
#pragma unroll
      for (int u = 0; u < U; ++u) __stcg(d + i + static_cast<long long>(u) * nt, v[u]);
    }
    for (; i < n; i += nt) __stcg(d + i, __ldcg(s + i));
    return;
  }
  // Unaligned ends: bytes until dst is 16-aligned, then 16-byte stores if src happens to agree,
  // else a plain byte loop (correct for any offsets; only tiny or odd-sized pieces land here).
  if ((reinterpret_cast<uintptr_t>(dst) & 15u) == (reinterpret_cast<uintptr_t>(src) & 15u) && bytes >= 32) {
    const long long head = (16 - (reinterpret_cast<uintptr_t>(dst) & 15u)) & 15u;
    const long long body = (bytes - head) & ~15ll;
    for (long long i = tid; i < head; i += nt) dst[i] = src[i];
    const int4* s = reinterpret_cast<const int4*>(src + head);
    int4* d = reinterpret_cast<int4*>(dst + head);
    for (long long i = tid; i < (body >> 4); i += nt) __stcg(d + i, __ldcg(s + i));
    for (long long i = head + body + tid; i < bytes; i += nt) dst[i] = src[i];
    return;
  }
  for (long long i = tid; i < bytes; i += nt) dst[i] = src[i];
}

// Phase of a work item for the optional time stamps: 0 balance, 1 rail (inter-server stage),
// 2 redistribute (forward of staged data), 3 direct (intrinsic traffic and flat plans).
__device__ __forceinline__ int phase_of(const A2AWork& w) {
  if (w.signal_kind == 1) return 0;
  if (w.signal_kind == 2) return 1;
  return w.wait_kind == 2 ? 2 : 3;
}

__device__ __forceinline__ void run_rank(const A2ARankArgs& a) {
  __shared__ int s_ok;
  // Bytes this CTA has stored into each peer's OUTPUT and not yet announced. Output arrivals are
  // only consumed at the end of the collective, so they are announced once per CTA (one fence for
  // the whole list instead of one per work item); staged data is announced item by item because a
  // forwarder is waiting for it.
  __shared__ unsigned long long s_pending[kSigMaxWorld];
  // Peers whose entry flag this CTA has already seen for this epoch: the flag is polled once per
  // CTA and peer, not once per work item.
  __shared__ unsigned char s_peer_ready[kSigMaxWorld];
  const int tid = threadIdx.x;
  for (int i = tid; i < kSigMaxWorld; i += blockDim.x) { s_pending[i] = 0ull; s_peer_ready[i] = 0; }
  if (tid == 0) s_ok = 1;
  __syncthreads();
  unsigned char* my_slab = static_cast<unsigned char*>(a.peer_table[a.rank]);
  unsigned long long* my_sig = reinterpret_cast<unsigned long long*>(my_slab + a.sig_heap_off);
  unsigned long long* my_cnt = my_sig + kSigCounterOff;
  // Optional per-phase stamps (globaltimer ns of this GPU): [0] first CTA in, [1 + 2 p] / [2 + 2 p]
  // first start / last end of a work item of phase p, [9] last CTA out. The host clears them (start
  // slots to ~0) before the launch.
  unsigned long long* stamps = a.phase_stamps;
  if (stamps && tid == 0) atomicMin(stamps + 0, global_timer_ns());

  // Tell every peer that this rank's buffers may be written for this epoch.
  if (blockIdx.x == 0 && tid < a.world) {
    unsigned long long* peer_sig = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[tid]) + a.sig_heap_off);
    st_release_sys(peer_sig + kSigReadyOff + a.rank, a.epoch);
  }
  bool alive = true;
  for (int it = blockIdx.x; it < a.n_items && alive; it += gridDim.x) {
    const A2AWork w = a.items[it];
    // Every thread evaluates the same condition (shared memory is only written by thread 0 between
    // barriers), so the barriers below are taken by all threads or by none.
    const bool must_wait = !s_peer_ready[w.dst_rank] || w.wait_kind != 0;
    if (must_wait) {
      if (tid == 0) {
        bool ok = s_peer_ready[w.dst_rank] || wait_ge_bounded(my_sig + kSigReadyOff + w.dst_rank, a.epoch, a.status, kSiteEntryReady, w.dst_rank, a.timeout_ns);
        if (ok && w.wait_kind == 1)
          ok = wait_ge_bounded(my_cnt + 0, a.expect_balance, a.status, kSiteBalanceArrive, it, a.timeout_ns);
        if (ok && w.wait_kind == 2)
          ok = wait_ge_bounded(my_cnt + 2 + w.wait_stage, a.expect_rail[w.wait_stage], a.status, kSiteRailArrive, w.wait_stage, a.timeout_ns);
        s_ok = ok ? 1 : 0;
      }
      __syncthreads();
      alive = s_ok != 0;
      if (!alive) break;
      if (tid == 0) s_peer_ready[w.dst_rank] = 1;  // read again only after the next barrier every thread takes
    }
    if (stamps && tid == 0) atomicMin(stamps + 1 + 2 * phase_of(w), global_timer_ns());
    unsigned char* dst_slab = static_cast<unsigned char*>(a.peer_table[w.dst_rank]);
    copy_bytes(dst_slab + a.dst_heap_off[w.dst_buf] + w.dst_off, a.src_base[w.src_buf] + w.src_off, w.bytes);
    if (w.signal_kind == 3) {
      // Output bytes are announced once, after the whole list (one barrier below covers them all).
      if (tid == 0) s_pending[w.dst_rank] += static_cast<unsigned long long>(w.bytes);
      if (must_wait) __syncthreads();  // publishes s_peer_ready to the other threads
    } else {
      __syncthreads();  // every thread's stores precede thread 0's release below
      if (tid == 0) {
        unsigned long long* dst_cnt = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[w.dst_rank]) + a.sig_heap_off) + kSigCounterOff;
        const int slot = w.signal_kind == 1 ? 0 : 2 + w.stage;
        fence_sys();
        red_add_release_sys(dst_cnt + slot, static_cast<unsigned long long>(w.bytes));
      }
    }
    if (stamps && tid == 0) atomicMax(stamps + 2 + 2 * phase_of(w), global_timer_ns());
  }
  __syncthreads();  // all copies of this CTA are issued; announce the output bytes, one peer per thread
  if (tid < a.world && s_pending[tid] != 0ull) {
    unsigned long long* dst_cnt = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[tid]) + a.sig_heap_off) + kSigCounterOff;
    fence_sys();
    red_add_release_sys(dst_cnt + 1, s_pending[tid]);
  }
  // The collective is over for this rank once everything addressed to its output has landed. Only
  // the last CTA to finish its pushes waits for that (the others leave their SM at once); it then
  // clears the counters: all local waits are done by then and no peer can signal the next epoch
  // before this rank publishes `ready` again.
  if (tid == 0) {
    __threadfence();
    const unsigned long long ticket = atomicAdd(my_sig + kSigTicketOff, 1ull);
    if (ticket == gridDim.x - 1) {
      const bool aborted = *reinterpret_cast<volatile unsigned long long*>(&a.status->abort) != 0ull;
      const bool ok = !aborted && wait_ge_bounded(my_cnt + 1, a.expect_output, a.status, kSiteOutputArrive, 0, a.timeout_ns);
      if (ok) {
        my_cnt[0] = 0; my_cnt[1] = 0;
        for (int k = 0; k < a.num_stages; ++k) my_cnt[2 + k] = 0;
      }
      my_sig[kSigTicketOff] = 0;
      __threadfence_system();
      if (stamps) atomicMax(stamps + 9, global_timer_ns());
    }
  }
}

__global__ void __launch_bounds__(1024) a2a_push_kernel(const A2ARankArgs a) { run_rank(a); }
__global__ void __launch_bounds__(1024) a2a_push_group_kernel(const A2ARankArgs* __restrict__ all) { run_rank(all[blockIdx.y]); }

__global__ void wait_probe_kernel(const unsigned long long* flag, unsigned long long want, DeviceStatus* st, unsigned long long timeout_ns) {
  if (threadIdx.x == 0) wait_ge_bounded(flag, want, st, kSiteTest, 0, timeout_ns);
}

}  // namespace

namespace { std::atomic<unsigned long long> g_launches{0}; }
unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
void note_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

cudaError_t launch_a2a_push(const A2ARankArgs* host_args, const A2ARankArgs* device_args, int virtual_ranks, int ctas, int threads,
                            cudaStream_t stream) {
  if (ctas < 1 || threads < 32 || threads > 1024 || virtual_ranks < 1) return cudaErrorInvalidValue;
  if (device_args == nullptr) {
    if (host_args == nullptr || virtual_ranks != 1) return cudaErrorInvalidValue;
    a2a_push_kernel<<<ctas, threads, 0, stream>>>(*host_args);
    note_launch();
  return cudaGetLastError();
  }
  // All virtual ranks wait on one another, so they must be co-resident: cooperative launch.
  void* params[] = {const_cast<A2ARankArgs**>(&device_args)};
  note_launch();
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(a2a_push_group_kernel), dim3(ctas, virtual_ranks), dim3(threads), params, 0, stream);
}

cudaError_t launch_wait_probe(const unsigned long long* flag, unsigned long long want, DeviceStatus* status,
                              unsigned long long timeout_ns, cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(flag, want, status, timeout_ns);
  note_launch();
  return cudaGetLastError();
}

}  // namespace fastb
