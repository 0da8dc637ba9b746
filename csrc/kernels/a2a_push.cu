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
#include <algorithm>
#include <atomic>

#include "api.h"
#include "sm100_ptx.cuh"

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

// ---- bulk-copy variant of copy_bytes ---------------------------------------------------------------
// One elected thread moves the bytes with the bulk-copy engine instead of every thread with loads and
// stores: local global memory -> a ring of shared-memory buffers (cp.async.bulk with mbarrier
// completion), then shared memory -> the peer's global memory (cp.async.bulk store, bulk-group
// completion). Both legs are plain bulk copies; the load side only ever reads this GPU's own memory.
// Needs 16-byte aligned pointers and size; other pieces take the load/store loop above.
constexpr int kBulkBufs = 4;
constexpr int kBulkChunk = 32 * 1024;
constexpr int kBulkSmemBytes = kBulkBufs * kBulkChunk;

struct BulkState {
  unsigned char* ring;       // kBulkBufs x kBulkChunk bytes of dynamic shared memory, 128-byte aligned
  uint64_t* full;            // kBulkBufs mbarriers (count 1)
  volatile int* abort_flag;  // CTA-shared give-up word of the bounded mbarrier wait
  uint32_t loads;            // loads issued so far by this CTA's elected thread (buffer = loads % kBulkBufs)
  uint32_t stores;           // stores issued so far
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
// Called by ONE thread. Returns false if a load never completed (bounded wait).
__device__ __forceinline__ bool copy_bytes_bulk(BulkState& b, unsigned char* dst, const unsigned char* src, long long bytes, DeviceStatus* st,
                                                unsigned long long timeout_ns) {
  const int n = static_cast<int>((bytes + kBulkChunk - 1) / kBulkChunk);
  auto size_of = [&](int c) { return static_cast<uint32_t>(c + 1 < n ? kBulkChunk : bytes - static_cast<long long>(c) * kBulkChunk); };
  auto issue_load = [&](int c) {
    const uint32_t buf = b.loads % kBulkBufs;
    const uint32_t bar = smem_addr(b.full + buf), sz = size_of(c);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(sz) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(b.ring + buf * kBulkChunk)), "l"(src + static_cast<long long>(c) * kBulkChunk), "r"(sz), "r"(bar) : "memory");
    ++b.loads;
  };
  // Buffers are taken in ring order by loads and stores alike. Stores of earlier pieces have long been issued:
  // make sure they are done reading their buffers, then keep kBulkBufs - 1 loads ahead of the stores.
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  int loaded = 0;
  for (; loaded < n && loaded < kBulkBufs - 1; ++loaded) issue_load(loaded);
  for (int c = 0; c < n; ++c) {
    const uint32_t buf = b.stores % kBulkBufs;
    if (!ptx::mbar_wait_bounded(b.full + buf, (b.stores / kBulkBufs) & 1u, b.abort_flag, st, 900, timeout_ns)) return false;
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst + static_cast<long long>(c) * kBulkChunk), "r"(smem_addr(b.ring + buf * kBulkChunk)), "r"(size_of(c)) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    ++b.stores;
    if (loaded < n) {
      // The next load takes the buffer that store c - 1 read: every store but the one just issued must be done reading.
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      issue_load(loaded++);
    }
  }
  return true;
}
// All bulk stores of this thread have completed and are ordered before what follows in the generic proxy.
__device__ __forceinline__ void bulk_drain() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  asm volatile("fence.proxy.async.global;" ::: "memory");
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
  __shared__ __align__(8) uint64_t s_bulk_full[kBulkBufs];
  extern __shared__ __align__(128) unsigned char s_bulk_ring[];  // kBulkSmemBytes when a.bulk, else nothing
  const int tid = threadIdx.x;
  for (int i = tid; i < kSigMaxWorld; i += blockDim.x) { s_pending[i] = 0ull; s_peer_ready[i] = 0; }
  if (tid == 0) {
    s_ok = 1;
    if (a.bulk) {
      for (int i = 0; i < kBulkBufs; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&s_bulk_full[i])) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
  }
  __shared__ int s_bulk_abort;
  if (tid == 0) s_bulk_abort = 0;
  BulkState bulk{s_bulk_ring, s_bulk_full, &s_bulk_abort, 0u, 0u};  // used by thread 0 only
  bool bulk_ok = true;
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
    unsigned char* dst_ptr = dst_slab + a.dst_heap_off[w.dst_buf] + w.dst_off;
    const unsigned char* src_ptr = a.src_base[w.src_buf] + w.src_off;
    const bool by_engine = a.bulk && ((reinterpret_cast<uintptr_t>(dst_ptr) | reinterpret_cast<uintptr_t>(src_ptr) | static_cast<uintptr_t>(w.bytes)) & 15u) == 0;
    if (by_engine) {
      if (tid == 0 && bulk_ok) {
        if (w.wait_kind != 0) asm volatile("fence.proxy.async.global;" ::: "memory");  // staged bytes were written by peers: order them before the engine's reads
        bulk_ok = copy_bytes_bulk(bulk, dst_ptr, src_ptr, w.bytes, a.status, a.timeout_ns);
        if (bulk_ok && w.signal_kind != 3) bulk_drain();  // a forwarder waits for this piece: its stores must have landed before the counter moves
      }
    } else {
      copy_bytes(dst_ptr, src_ptr, w.bytes);
    }
    if (w.signal_kind == 3) {
      // Output bytes are announced once, after the whole list (one barrier below covers them all).
      if (tid == 0 && bulk_ok) s_pending[w.dst_rank] += static_cast<unsigned long long>(w.bytes);
      if (must_wait) __syncthreads();  // publishes s_peer_ready to the other threads
    } else {
      __syncthreads();  // every thread's stores precede thread 0's release below
      if (tid == 0 && bulk_ok) {
        unsigned long long* dst_cnt = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[w.dst_rank]) + a.sig_heap_off) + kSigCounterOff;
        const int slot = w.signal_kind == 1 ? 0 : 2 + w.stage;
        fence_sys();
        red_add_release_sys(dst_cnt + slot, static_cast<unsigned long long>(w.bytes));
      }
    }
    if (stamps && tid == 0) atomicMax(stamps + 2 + 2 * phase_of(w), global_timer_ns());
  }
  if (a.bulk && tid == 0) {
    bulk_drain();  // every engine store of this CTA has landed before anything is announced
    if (!bulk_ok)  // a load never completed (already reported): announce nothing, the peers' bounded waits will say so
      for (int i = 0; i < kSigMaxWorld; ++i) s_pending[i] = 0ull;
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
                            cudaStream_t stream, bool needs_coresidency) {
  if (ctas < 1 || threads < 32 || threads > 1024 || virtual_ranks < 1) return cudaErrorInvalidValue;
  if (device_args == nullptr) {
    if (host_args == nullptr || virtual_ranks != 1) return cudaErrorInvalidValue;
    const int smem = host_args->bulk ? kBulkSmemBytes : 0;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(a2a_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return e;
    }
    // The grid never exceeds what one GPU can hold at once. A plan with waiting work items (two-tier plans: forwarders
    // wait for balance / rail arrivals that peers push, while peers' forwarders wait for what this rank pushes) is
    // launched cooperatively: the driver then starts it only when the whole grid can be resident, so a waiting CTA
    // can never keep a pushing one of the same launch off the GPU.
    int dev = 0, sms = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, a2a_push_kernel, threads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    ctas = std::min(ctas, sms * per_sm);
    if (needs_coresidency) {
      A2ARankArgs args = *host_args;
      void* params[] = {&args};
      e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(a2a_push_kernel), dim3(ctas), dim3(threads), params, smem, stream);
      if (e == cudaSuccess) note_launch();
      return e;
    }
    a2a_push_kernel<<<ctas, threads, smem, stream>>>(*host_args);
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
