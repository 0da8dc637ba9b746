// MoE routing on the device, with no host round trip between the gate and the expert GEMMs:
//   route_topk   : softmax(+bias) top-k per token, per-block expert histogram and the stable rank
//                  of every (token, slot) inside its block;
//   splits_scan  : prefix sums over blocks -> per-expert send counts, all-gather of the counts by
//                  direct stores into every peer's symmetric pad, then receive offsets, padded
//                  group offsets for the grouped GEMM and cumulative arrival targets.
// The reference has no router; its counterpart of the count exchange is the host-side workload
// broadcast (nvidia/alltoall_nvshmem.cpp:452-472), which this replaces with ~1 KB of NVLink stores.
#include "api.h"

namespace fastb {

namespace {

constexpr int kTokensPerBlock = kRouteTokensPerBlock;
constexpr int kRouteThreads = 256;

// One warp per token at a time. E <= 256 (8 values per lane).
template <int MAX_PER_LANE>
__global__ void __launch_bounds__(kRouteThreads) route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E,
                                                                   int K, int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                                   int* __restrict__ slot_in_block, int* __restrict__ block_cnt) {
  extern __shared__ int s_eid[];  // [kTokensPerBlock * K]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kRouteThreads / 32;
  const int t0 = blockIdx.x * kTokensPerBlock;
  const int nt = min(kTokensPerBlock, T - t0);
  for (int lt = warp; lt < kTokensPerBlock; lt += nwarps) {
    const int t = t0 + lt;
    if (lt >= nt) {
      for (int j = lane; j < K; j += 32) s_eid[lt * K + j] = -1;
      continue;
    }
    float sel[MAX_PER_LANE], raw[MAX_PER_LANE];
    unsigned taken = 0u;  // bit i: candidate lane + 32 i is chosen already, or past the last expert
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      // NaN logits count as -inf: the selection below stays total and the weights stay finite.
      float r = e < E ? logits[static_cast<long long>(t) * E + e] : -INFINITY;
      if (r != r) r = -INFINITY;
      float s = e < E ? r + (bias ? bias[e] : 0.0f) : -INFINITY;
      if (s != s) s = -INFINITY;
      raw[i] = r;
      sel[i] = s;
      if (e >= E) taken |= 1u << i;
      mx = fmaxf(mx, r);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // Selection uses logits + bias; the weights are the softmax of the raw logits over the
    // chosen experts (renormalised), which for bias == 0 is Mixtral's softmax-over-top-k.
    // A token with fewer than K selectable values (-inf / NaN rows, masked experts) still gets K
    // distinct expert ids in range: the lowest unchosen ids, with weight 0.
    float wsum = 0.0f;
    float my_w = 0.0f;
    int my_e = -1;
    for (int j = 0; j < K; ++j) {
      float best = -INFINITY;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i)
        if (!((taken >> i) & 1u) && (best_e == 0x7fffffff || sel[i] > best)) { best = sel[i]; best_e = lane + 32 * i; }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; }
      }
      float r = -INFINITY;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i)
        if (lane + 32 * i == best_e) { r = raw[i]; taken |= 1u << i; }
      r = __shfl_sync(0xffffffffu, r, best_e & 31);
      const float p = r > -INFINITY ? __expf(r - mx) : 0.0f;
      wsum += p;
      if (lane == j) { my_w = p; my_e = best_e; }
    }
    if (lane < K) {
      topk_idx[static_cast<long long>(t) * K + lane] = my_e;
      topk_w[static_cast<long long>(t) * K + lane] = wsum > 0.0f ? my_w / wsum : 0.0f;
      s_eid[lt * K + lane] = my_e;
    }
  }
  __syncthreads();
  // Stable rank of every entry among the entries of the same expert in this block: thread e walks
  // the block's entries in (token, slot) order.
  const int n = kTokensPerBlock * K;
  for (int e = threadIdx.x; e < E; e += kRouteThreads) {
    int c = 0;
    for (int i = 0; i < n; ++i)
      if (s_eid[i] == e) {
        slot_in_block[static_cast<long long>(t0) * K + i] = c;
        ++c;
      }
    block_cnt[static_cast<long long>(blockIdx.x) * E + e] = c;
  }
}

// Single CTA. Thread e owns expert e (E <= 1024).
__global__ void __launch_bounds__(1024) splits_scan_kernel(const SplitsArgs a) {
  extern __shared__ int s_tot[];  // [E] padded totals per expert, then [world] scratch
  const int e = threadIdx.x;
  const int E = a.num_experts, W = a.world, El = E / W;
  unsigned char* my_slab = static_cast<unsigned char*>(a.peer_table[a.rank]);
  int* my_counts = reinterpret_cast<int*>(my_slab + a.counts_heap_off);                       // [W][E]
  unsigned long long* my_flags = reinterpret_cast<unsigned long long*>(my_slab + a.flags_heap_off);  // [W]
  __shared__ unsigned long long s_epoch;
  if (e == 0) s_epoch = a.epoch_dev ? (*a.epoch_dev = *a.epoch_dev + 1ull) : a.epoch;
  __syncthreads();
  const unsigned long long epoch = s_epoch;
  int mine = 0;
  if (e < E) {
    // Eight independent loads in flight per round (the running sum is the only serial part).
    for (int b0 = 0; b0 < a.num_blocks; b0 += 8) {
      int c[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) c[u] = b0 + u < a.num_blocks ? __ldg(a.block_cnt + static_cast<long long>(b0 + u) * E + e) : 0;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (b0 + u < a.num_blocks) { a.block_base[static_cast<long long>(b0 + u) * E + e] = mine; mine += c[u]; }
    }
    // All-gather by stores: my row of the count matrix goes to every rank (myself included).
    for (int r = 0; r < W; ++r) {
      int* dst = reinterpret_cast<int*>(static_cast<unsigned char*>(a.peer_table[r]) + a.counts_heap_off);
      dst[a.rank * E + e] = mine;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (e < W) {
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[e]) + a.flags_heap_off);
    st_release_sys(dst + a.rank, epoch);
  }
  __shared__ int s_ok;
  if (e == 0) s_ok = 1;
  __syncthreads();
  if (e < W) {
    if (!wait_ge_bounded(my_flags + e, epoch, a.status, kSiteCountsArrive, e, a.timeout_ns)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  // The count matrix is read once (coalesced, W independent loads per thread) and kept in shared
  // memory when it fits; every later loop reads the copy.
  int* s_cnt = s_tot + E;  // [W][E] when a.counts_in_smem
  int tot = 0, before_me = 0;
  if (e < E) {
    for (int s = 0; s < W; ++s) {
      const int c = *reinterpret_cast<volatile int*>(my_counts + s * E + e);
      if (a.counts_in_smem) s_cnt[s * E + e] = c;
      tot += c;
      if (s < a.rank) before_me += c;
    }
    s_tot[e] = (tot + a.row_align - 1) / a.row_align * a.row_align;
  }
  auto count_at = [&](int s, int q) { return a.counts_in_smem ? s_cnt[s * E + q] : *reinterpret_cast<volatile int*>(my_counts + s * E + q); };
  __shared__ int s_over;
  if (e == 0) s_over = 0;
  __syncthreads();
  // Every rank sees the same count matrix, so every rank reaches the same verdict: if any rank's
  // padded rows exceed the receive capacity, the step is refused everywhere (no rows are sent, the
  // GEMMs get empty groups) and the status block says how many rows were needed.
  if (e < W) {
    int need = 0;
    for (int q = 0; q < El; ++q) need += s_tot[e * El + q];
    if (need > a.cap_rows) { atomicMax(&s_over, need); }
  }
  __syncthreads();
  if (s_over) {
    if (e == 0) report_failure(a.status, kStatusBadArg, kSiteCapacity, a.rank, static_cast<unsigned long long>(s_over), static_cast<unsigned long long>(a.cap_rows));
    if (e < E) { a.send_base[e] = 0; a.send_cnt[e] = 0; }
    if (e <= El) a.group_off[e] = 0;
    if (e < El) a.group_rows[e] = 0;
    return;
  }
  if (e < E) {
    // Row where my first token for expert e lands on its owner: padded sizes of the owner's
    // earlier experts plus the rows of lower-ranked sources for e.
    const int d = e / El, le = e % El;
    int base = 0;
    for (int q = 0; q < le; ++q) base += s_tot[d * El + q];
    a.send_base[e] = base + before_me;
    a.send_cnt[e] = mine;
    if (a.send_pos) {
      // Entries are sent expert-slot by expert-slot: all ranks' local expert 0, then 1, ... Within a
      // slot every sender starts with itself and walks the ranks upwards, so that at any moment the
      // senders aim at different receivers.
      int pos = 0;
      for (int q = 0; q < E; ++q) {
        const int key_q = (q % El) * W + (q / El - a.rank + W) % W, key_e = le * W + (d - a.rank + W) % W;
        if (key_q < key_e) pos += count_at(a.rank, q);
      }
      a.send_pos[e] = pos;
    }
    if (d == a.rank) {
      a.group_off[le] = base;
      a.group_rows[le] = tot;
      if (le == El - 1) a.group_off[El] = base + s_tot[e];
      // Monotone arrival targets, one per channel (forward dispatch, backward dispatch).
      for (int ch = 0; ch < a.num_channels; ++ch) a.arrive_target[ch * El + le] += static_cast<unsigned long long>(tot);
      if (a.tile_target != nullptr) {
        // The same per tile of the receive buffer: this expert's rows fill its tiles from `base` on.
        for (int r0 = 0; r0 < tot; r0 += a.tile_rows) {
          const int t = (base + r0) / a.tile_rows;
          if (t >= a.num_tiles) break;
          const unsigned long long rows = static_cast<unsigned long long>(min(a.tile_rows, tot - r0));
          for (int ch = 0; ch < a.num_channels; ++ch) a.tile_target[static_cast<long long>(ch) * a.num_tiles + t] += rows;
        }
      }
    }
  }
  // Token traffic matrix of this step, [src][dst], for the scheduler / observability.
  if (a.traffic_matrix)
    for (int i = threadIdx.x; i < W * W; i += blockDim.x) {
      const int s = i / W, d = i % W;
      int sent = 0;
      for (int q = 0; q < El; ++q) sent += count_at(s, d * El + q);
      a.traffic_matrix[i] = sent;
    }
}

__global__ void build_send_list_kernel(const int* __restrict__ topk_idx, const int* __restrict__ slot_in_block, const int* __restrict__ block_base,
                                       const int* __restrict__ send_pos, int T, int K, int E, int* __restrict__ list, DeviceStatus* status) {
  const long long tj = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (tj >= static_cast<long long>(T) * K) return;
  const int e = topk_idx[tj];
  if (e < 0 || e >= E) {  // an id no router of this library produces: skip the entry, say so, touch nothing
    if (status) report_failure(status, kStatusBadArg, kSiteExpertId, static_cast<unsigned long long>(tj), static_cast<unsigned long long>(static_cast<unsigned int>(e)), static_cast<unsigned long long>(E));
    return;
  }
  const int t = static_cast<int>(tj / K);
  list[send_pos[e] + block_base[static_cast<long long>(t / kTokensPerBlock) * E + e] + slot_in_block[tj]] = static_cast<int>(tj);
}

// Zeroes the rows between each group's real end and its padded end.
__global__ void zero_pad_rows_kernel(unsigned char* buf, long long row_bytes, const int* __restrict__ group_off, const int* __restrict__ group_rows, int groups) {
  const int g = blockIdx.y;
  if (g >= groups) return;
  const long long begin = (static_cast<long long>(group_off[g]) + group_rows[g]) * row_bytes;
  const long long end = static_cast<long long>(group_off[g + 1]) * row_bytes;
  uint4* p = reinterpret_cast<uint4*>(buf + begin);
  const long long n = (end - begin) / 16;
  for (long long i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
}

}  // namespace

cudaError_t launch_route_topk(const float* logits, const float* bias, int T, int E, int K, int* topk_idx, float* topk_w, int* slot_in_block,
                              int* block_cnt, cudaStream_t stream) {
  if (E < 1 || E > 256 || K < 1 || K > 32 || K > E) return cudaErrorInvalidValue;
  const int blocks = (T + kTokensPerBlock - 1) / kTokensPerBlock;
  if (blocks == 0) return cudaSuccess;
  const size_t smem = sizeof(int) * kTokensPerBlock * K;
  if (E <= 32) route_topk_kernel<1><<<blocks, kRouteThreads, smem, stream>>>(logits, bias, T, E, K, topk_idx, topk_w, slot_in_block, block_cnt);
  else if (E <= 64) route_topk_kernel<2><<<blocks, kRouteThreads, smem, stream>>>(logits, bias, T, E, K, topk_idx, topk_w, slot_in_block, block_cnt);
  else if (E <= 128) route_topk_kernel<4><<<blocks, kRouteThreads, smem, stream>>>(logits, bias, T, E, K, topk_idx, topk_w, slot_in_block, block_cnt);
  else route_topk_kernel<8><<<blocks, kRouteThreads, smem, stream>>>(logits, bias, T, E, K, topk_idx, topk_w, slot_in_block, block_cnt);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_splits_scan(const SplitsArgs& a, cudaStream_t stream) {
  if (a.tile_target != nullptr && (a.tile_rows < 1 || a.row_align % a.tile_rows || a.num_tiles < 1)) return cudaErrorInvalidValue;
  if ((a.row_align != 128 && a.row_align != 256) || a.num_experts < 1 || a.num_experts > 1024 || a.world < 1 || a.world > a.num_experts || a.num_experts % a.world) return cudaErrorInvalidValue;
  int threads = (std::max(a.num_experts, a.world) + 31) / 32 * 32;
  SplitsArgs b = a;
  b.counts_in_smem = static_cast<long long>(a.world) * a.num_experts <= 8192 ? 1 : 0;  // 32 KiB of the 48 KiB default
  const size_t smem = sizeof(int) * (a.num_experts + a.world + (b.counts_in_smem ? a.world * a.num_experts : 0));
  splits_scan_kernel<<<1, threads, smem, stream>>>(b);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_build_send_list(const int* topk_idx, const int* slot_in_block, const int* block_base, const int* send_pos, int T, int K, int E,
                                   int* list, DeviceStatus* status, cudaStream_t stream) {
  const long long n = static_cast<long long>(T) * K;
  if (n == 0) return cudaSuccess;
  build_send_list_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(topk_idx, slot_in_block, block_base, send_pos, T, K, E, list, status);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_zero_pad_rows(void* buf, long long row_bytes, const int* group_off, const int* group_rows, int groups, cudaStream_t stream) {
  if (row_bytes % 16) return cudaErrorInvalidValue;
  if (groups == 0) return cudaSuccess;
  zero_pad_rows_kernel<<<dim3(8, groups), 256, 0, stream>>>(static_cast<unsigned char*>(buf), row_bytes, group_off, group_rows, groups);
  note_launch();
  return cudaGetLastError();
}

}  // namespace fastb

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in route_noalloc.h).
// ---------------------------------------------------------------------------------------------
#include <atomic>
#include <cstdio>

#include "route_noalloc.h"

namespace fastb {
namespace {

constexpr int kNoAllocMaxTokens = 16384, kNoAllocMaxExperts = 256, kNoAllocMaxTopK = 8;
constexpr int kNoAllocMaxBlocks = kNoAllocMaxTokens / kRouteTokensPerBlock;
constexpr size_t kNoAllocCntBytes = sizeof(int) * kNoAllocMaxBlocks * kNoAllocMaxExperts;    // per-block histograms
constexpr size_t kNoAllocSlotBytes = sizeof(int) * kNoAllocMaxTokens * kNoAllocMaxTopK;       // in-block ranks
constexpr size_t kNoAllocBytes = kNoAllocCntBytes + kNoAllocSlotBytes;                        // 640 KiB

// Scratch of the allocation-free entry point. In host code this name is only a handle for
// cudaGetSymbolAddress; kernels receive the device address obtained from it.
static __device__ __align__(256) unsigned char g_route_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
// One address per device, filled by the first call on that device. Atomic: several host threads
// may make that first call at once (they would all store the same value).
std::atomic<void*> g_scratch_addr[kMaxDevices] = {};
thread_local char g_noalloc_error[256] = "";

__global__ void sum_block_counts_kernel(const int* __restrict__ block_cnt, int blocks, int E, int* __restrict__ expert_counts) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  int s = 0;
  for (int b = 0; b < blocks; ++b) s += block_cnt[static_cast<long long>(b) * E + e];
  expert_counts[e] = s;
}

int refuse(cudaError_t code, const char* fmt, int a = 0, int b = 0) {
  snprintf(g_noalloc_error, sizeof(g_noalloc_error), fmt, a, b);
  return static_cast<int>(code);
}

}  // namespace
}  // namespace fastb

extern "C" void fastb_route_topk_noalloc_limits(int* max_tokens, int* max_experts, int* max_top_k) {
  if (max_tokens) *max_tokens = fastb::kNoAllocMaxTokens;
  if (max_experts) *max_experts = fastb::kNoAllocMaxExperts;
  if (max_top_k) *max_top_k = fastb::kNoAllocMaxTopK;
}

extern "C" const char* fastb_noalloc_last_error(void) { return fastb::g_noalloc_error; }

extern "C" int fastb_route_topk_noalloc(const float* logits, const float* bias, int T, int E, int K, int* topk_idx, float* topk_w,
                                        int* expert_counts, void* stream_v) {
  using namespace fastb;
  g_noalloc_error[0] = '\0';
  if (!logits || !topk_idx || !topk_w || !expert_counts) return refuse(cudaErrorInvalidValue, "fastb_route_topk_noalloc: null buffer");
  if (T < 0 || T > kNoAllocMaxTokens) return refuse(cudaErrorInvalidValue, "fastb_route_topk_noalloc: %d tokens exceed the fixed scratch (max %d)", T, kNoAllocMaxTokens);
  if (E < 1 || E > kNoAllocMaxExperts) return refuse(cudaErrorInvalidValue, "fastb_route_topk_noalloc: %d experts exceed the fixed scratch (max %d)", E, kNoAllocMaxExperts);
  if (K < 1 || K > kNoAllocMaxTopK || K > E) return refuse(cudaErrorInvalidValue, "fastb_route_topk_noalloc: top-%d is outside 1..min(%d, experts)", K, kNoAllocMaxTopK);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return refuse(e, "fastb_route_topk_noalloc: cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices) return refuse(cudaErrorInvalidDevice, "fastb_route_topk_noalloc: device index %d not supported (max %d)", dev, kMaxDevices - 1);
  void* scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // Once per device, with that device current: translate the symbol into its device address.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_route_scratch);
    if (e != cudaSuccess || p == nullptr) return refuse(e != cudaSuccess ? e : cudaErrorInvalidSymbol, "fastb_route_topk_noalloc: cudaGetSymbolAddress failed");
    g_scratch_addr[dev].store(p, std::memory_order_release);
    scratch = p;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int blocks = (T + kRouteTokensPerBlock - 1) / kRouteTokensPerBlock;
  int* block_cnt = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch));
  int* slot_in_block = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + kNoAllocCntBytes);
  if (blocks > 0) {
    e = launch_route_topk(logits, bias, T, E, K, topk_idx, topk_w, slot_in_block, block_cnt, stream);
    if (e != cudaSuccess) return refuse(e, "fastb_route_topk_noalloc: routing kernel launch failed");
  }
  sum_block_counts_kernel<<<(E + 127) / 128, 128, 0, stream>>>(block_cnt, blocks, E, expert_counts);
  e = cudaGetLastError();
  if (e != cudaSuccess) return refuse(e, "fastb_route_topk_noalloc: count kernel launch failed");
  note_launch();
  return 0;
}
