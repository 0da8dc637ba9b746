// Fused MoE transport kernels over peer memory (NVLink P2P loads/stores issued inside the kernel):
//   dispatch_push : gather token rows by routing index, optional per-row scale, optional e4m3
//                   quantisation with 1x128 block scales, and store them straight into the final
//                   row of the owning expert's receive buffer on the peer; per-expert arrival
//                   counters are bumped with release semantics once a CTA's rows are out.
//   combine_pull  : un-permute + top-k weighted reduction: every token pulls its k expert rows
//                   from the peers and accumulates them in fp32 (fixed slot order => reproducible),
//                   or, in dot mode, produces <grad_out[t], row_j> for the router gradient.
// In FAST's terms these are the all-to-all of the forward pass and its transpose
// (amd/flash.cpp:400-408 `backward` flag) with the permute / reduce fused in; the reference moves
// opaque bytes with ncclSend/ncclRecv groups or NVSHMEM puts and leaves the packing to the caller.
#include <cuda_fp8.h>

#include "api.h"

namespace fastb {

namespace {

constexpr int kCommThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

constexpr int kMaxK = 8;
constexpr int kMaxScaleGroups = 128;  // fp8 dispatch: rows of up to 128 x 128 = 16384 elements

// 16 bf16 elements of a lane -> 16 e4m3 bytes; 8 consecutive lanes (128 elements) share one scale.
// Every lane of the warp calls this together (lanes past the row's end pass zeros).
// The scale is amax / 448 rounded UP to the next value a bf16 can hold: quantised values still fit
// e4m3, and a receiver that multiplies in bf16 (the expert GEMM's converter warps) reproduces
// value x scale without a second rounding. The abs / max run on bf16 pairs, the conversion on float pairs.
__device__ __forceinline__ uint4 quantise16(const uint4 (&raw)[2], float& sc) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[0]);  // 8 pairs = my 16 elements
  __nv_bfloat162 m2 = __habs2(h[0]);
#pragma unroll
  for (int i = 1; i < 8; ++i) m2 = __hmax2(m2, __habs2(h[i]));
  float amax = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
  for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  sc = __uint_as_float((__float_as_uint(fmaxf(amax, 1e-12f) * (1.0f / 448.0f)) + 0xFFFFu) & 0xFFFF0000u);
  const float inv = 1.0f / sc;
  uint4 q;
  unsigned short* qs = reinterpret_cast<unsigned short*>(&q);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    qs[i] = __nv_cvt_float2_to_fp8x2(make_float2(f.x * inv, f.y * inv), __NV_SATFINITE, __NV_E4M3);
  }
  return q;
}

// One warp per row: x [T, H] bf16 -> q [T, H] e4m3 bytes + scales [T, H / 128], in this GPU's own memory.
// The sorted dispatch sends every (token, slot) entry from a warp of its own; with the rows quantised
// here first, a token's K entries copy bytes instead of each repeating the reduction and the conversions.
__global__ void __launch_bounds__(kCommThreads) quantise_rows_kernel(const __nv_bfloat16* __restrict__ x, int T, int H, unsigned char* __restrict__ q,
                                                                      float* __restrict__ scales) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int chunks16 = H / 16, sgroups = H / 128;
  for (long long t = blockIdx.x * wpb + warp; t < T; t += static_cast<long long>(gridDim.x) * wpb) {
    const uint4* src = reinterpret_cast<const uint4*>(x + t * H);
    uint4* out = reinterpret_cast<uint4*>(q + t * H);
    constexpr int U = 2;
    for (int c0 = 0; c0 < chunks16; c0 += 32 * U) {
      uint4 raw[U][2];
      bool active[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + 32 * u + lane;
        active[u] = c < chunks16;
        raw[u][0] = active[u] ? __ldg(src + 2 * c) : make_uint4(0, 0, 0, 0);
        raw[u][1] = active[u] ? __ldg(src + 2 * c + 1) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (c0 + 32 * u >= chunks16) break;  // warp-uniform
        const int c = c0 + 32 * u + lane;
        float sc;
        const uint4 v = quantise16(raw[u], sc);
        if (active[u]) {
          out[c] = v;
          if ((lane & 7) == 0) scales[t * sgroups + c / 8] = sc;
        }
      }
    }
  }
}

// FP8: rows leave as e4m3 + scales; SORTED: one warp per (token, slot) entry of send_list (one destination per warp, so the
// per-slot arrays shrink to one element); SCALED: bf16 rows are multiplied by row_scale on the way. The variants exist for
// their register counts: the copy loops are bound by the stores a SM keeps in flight, i.e. by resident warps.
template <bool FP8, bool SORTED, bool SCALED>
__global__ void __launch_bounds__(kCommThreads, SORTED ? 4 : 3) dispatch_push_kernel(const DispatchArgs a) {
  extern __shared__ int s_cnt[];  // rows this CTA sent: [E] per expert, or [world][num_tiles] per destination tile
  __shared__ int s_ok;
  __shared__ __align__(16) float s_scales[(kCommThreads / 32) * kMaxScaleGroups];  // fp8 mode: the 1x128 scales of the row each warp is sending
  const int E = a.num_experts, El = E / a.world;
  const int n_cnt = a.tile_rows > 0 ? a.world * a.num_tiles : E;
  for (int e = threadIdx.x; e < n_cnt; e += blockDim.x) s_cnt[e] = 0;
  if (threadIdx.x == 0) s_ok = 1;
  if (*reinterpret_cast<volatile unsigned long long*>(&a.status->abort) != 0ull) return;  // an earlier kernel of this rank refused the step
  __syncthreads();
  if (a.entry_epoch != 0) {
    // Entry handshake: publish that my receive buffers may be written, then wait for the peers.
    unsigned long long* my_flags = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[a.rank]) + a.entry_flags_heap_off);
    if (blockIdx.x == 0 && threadIdx.x < a.world) {
      unsigned long long* dst = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[threadIdx.x]) + a.entry_flags_heap_off);
      st_release_sys(dst + a.rank, a.entry_epoch);
    }
    if (threadIdx.x < a.world && !wait_ge_bounded(my_flags + threadIdx.x, a.entry_epoch, a.status, kSiteEntryReady, threadIdx.x, a.timeout_ns)) s_ok = 0;
    __syncthreads();
    if (!s_ok) return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  constexpr int tpb = kRouteTokensPerBlock;
  const int chunks = a.H / 8;  // 16-byte chunks per row
  // Unsorted mode: one warp per token, the row is read once and stored to its K destinations.
  // Sorted mode (send_list != null): one warp per (token, slot) entry, entries ordered by
  // (local expert index, destination rank counted from the sender upwards), so that every rank's expert 0 fills first, then
  // expert 1, ... and the gated GEMM of the receivers can start while later experts still arrive.
  constexpr int NJ = SORTED ? 1 : kMaxK;  // destinations one warp serves
  const long long n_work = SORTED ? static_cast<long long>(a.T) * a.K : a.T;
  // Adds this CTA's row counts to the receivers' arrival counters (release: the rows are stored before the counters move)
  // and clears them. Called by every thread of the CTA.
  auto publish_counts = [&]() {
    __syncthreads();  // every row of this CTA so far is stored
    for (int e = threadIdx.x; e < n_cnt; e += blockDim.x) {
      const int n = s_cnt[e];
      if (n == 0) continue;
      s_cnt[e] = 0;
      const int peer = a.tile_rows > 0 ? e / a.num_tiles : e / El;
      const int slot = a.tile_rows > 0 ? e % a.num_tiles : e % El;
      unsigned long long* cnt = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a.peer_table[peer]) + a.arrive_heap_off);
      fence_sys();
      red_add_release_sys(cnt + slot, static_cast<unsigned long long>(n));
    }
    __syncthreads();  // cleared before the next rows are counted
  };
  // Every warp of a CTA makes the same number of rounds (a round = one entry per warp), so the CTA can meet at a barrier
  // between rounds. In sorted order the counts are published every kPublishRounds rounds instead of once at the end:
  // the CTAs walk the send list together, so a receiver's tiles complete in list order while the dispatch is still
  // running, which is what lets its gated GEMM start early.
  constexpr int kPublishRounds = 8;
  const long long round_stride = static_cast<long long>(gridDim.x) * wpb;
  int round = 0;
  for (long long base = static_cast<long long>(blockIdx.x) * wpb; base < n_work; base += round_stride) {
    const long long wi = base + warp;
    if (wi < n_work) {
      int t, jbeg, nj;
      if (SORTED) { const int tj = a.send_list[wi]; t = tj / a.K; jbeg = tj % a.K; nj = 1; }
      else { t = static_cast<int>(wi); jbeg = 0; nj = a.K; }
      unsigned char* out_row[NJ];  // where each slot's row starts on its receiver (null: nothing to send for the slot)
      float scale[NJ];
      int row_of[NJ];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        out_row[j] = nullptr; scale[j] = 1.0f; row_of[j] = 0;
        if (j < nj) {
          const long long tj = static_cast<long long>(t) * a.K + jbeg + j;
          const int e = a.topk_idx[tj];
          if (e < 0 || e >= E) {  // not an expert: nothing is indexed with it; the step is flagged and the entry skipped
            if (lane == 0) report_failure(a.status, kStatusBadArg, kSiteExpertId, static_cast<unsigned long long>(tj), static_cast<unsigned long long>(static_cast<unsigned int>(e)), static_cast<unsigned long long>(E));
            continue;
          }
          int row;
          if (a.compute_rows) {
            row = a.send_base[e] + a.block_base[static_cast<long long>(t / tpb) * E + e] + a.slot_in_block[tj];
            if (lane == 0) a.dest_row[tj] = row;
          } else {
            row = a.dest_row[tj];
          }
          row_of[j] = row;
          out_row[j] = static_cast<unsigned char*>(a.peer_table[e / El]) + a.recv_heap_off + static_cast<long long>(row) * a.H * (FP8 ? 1 : 2);
          if (SCALED) scale[j] = a.row_scale[tj];
          if (lane == 0) atomicAdd(&s_cnt[a.tile_rows > 0 ? (e / El) * a.num_tiles + min(row / a.tile_rows, a.num_tiles - 1) : e], 1);
        }
      }
      const uint4* src = reinterpret_cast<const uint4*>(a.x + static_cast<long long>(t) * a.H);
      if constexpr (!FP8) {
        // Four 16-byte chunks per lane in flight before the first store: the loop is bound by the
        // latency of the local loads otherwise.
        constexpr int U = 4;
        for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
          uint4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (c0 + 32 * u < chunks) v[u] = __ldg(src + c0 + 32 * u);
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int c = c0 + 32 * u;
            if (c >= chunks) break;
            float f[8];
            if (SCALED) unpack8(v[u], f);
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
              if (j >= nj || out_row[j] == nullptr) continue;
              uint4* out = reinterpret_cast<uint4*>(out_row[j]) + c;
              if (SCALED) {
                float g[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) g[i] = f[i] * scale[j];
                *out = pack8(g);
              } else {
                *out = v[u];
              }
            }
          }
        }
      } else {
        // 16 elements per lane (one 16-byte store of e4m3); 8 consecutive lanes = 128 elements share
        // one scale (amax / 448). The row's scales leave as 16-byte stores after the payload: 4-byte
        // remote stores would each cost a packet of their own.
        const int sgroups = a.H / 128;
        const int chunks16 = a.H / 16;
        float* my_scales = s_scales + warp * kMaxScaleGroups;
        if (a.xq != nullptr) {
          // Rows were quantised once by quantise_rows_kernel: this entry copies bytes.
          const uint4* qsrc = reinterpret_cast<const uint4*>(a.xq + static_cast<long long>(t) * a.H);
          constexpr int U = 4;
          for (int c0 = lane; c0 < chunks16; c0 += 32 * U) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
              if (c0 + 32 * u < chunks16) v[u] = __ldg(qsrc + c0 + 32 * u);
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int c = c0 + 32 * u;
              if (c >= chunks16) break;
#pragma unroll
              for (int j = 0; j < NJ; ++j) {
                if (j >= nj || out_row[j] == nullptr) continue;
                *(reinterpret_cast<uint4*>(out_row[j]) + c) = v[u];
              }
            }
          }
          for (int g = lane; g < sgroups; g += 32) my_scales[g] = __ldg(a.xq_scales + static_cast<long long>(t) * sgroups + g);
        } else {
          // The whole warp walks the row together (the shuffles in quantise16 need every lane); lanes past
          // the end of a short row carry zeros and store nothing. Two blocks of 512 elements are in flight
          // per pass (their loads are issued before either is reduced). Measured: neither more resident warps
          // (8, 16 or 24 per SM), nor requesting the next pass before reducing this one, nor packed arithmetic
          // moves this path off about 600 GB/s to one peer; a plain copy of already quantised rows reaches 624.
          constexpr int U = 2;
          for (int c0 = 0; c0 < chunks16; c0 += 32 * U) {
            uint4 raw[U][2];
            bool active[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int c = c0 + 32 * u + lane;
              active[u] = c < chunks16;
              raw[u][0] = active[u] ? __ldg(src + 2 * c) : make_uint4(0, 0, 0, 0);
              raw[u][1] = active[u] ? __ldg(src + 2 * c + 1) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              if (c0 + 32 * u >= chunks16) break;  // warp-uniform: the second block of the last pass may not exist
              const int c = c0 + 32 * u + lane;
              float sc;
              const uint4 q = quantise16(raw[u], sc);
              if (active[u] && (lane & 7) == 0) my_scales[c / 8] = sc;
#pragma unroll
              for (int j = 0; j < NJ; ++j) {
                if (j >= nj || !active[u] || out_row[j] == nullptr) continue;
                *(reinterpret_cast<uint4*>(out_row[j]) + c) = q;
              }
            }
          }
        }
        __syncwarp();
        // sgroups is a multiple of 2 (H % 256 == 0): pairs of scales always; quads when the row's scale block is 16-byte aligned.
        const bool quad = (sgroups & 3) == 0;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          if (j >= nj || out_row[j] == nullptr) continue;
          // the receiver's slab base is the row pointer minus the row's offset in the receive buffer
          float* srow = reinterpret_cast<float*>(out_row[j] - a.recv_heap_off - static_cast<long long>(row_of[j]) * a.H + a.scale_heap_off) + static_cast<long long>(row_of[j]) * sgroups;
          if (quad) {
            for (int g = lane * 4; g < sgroups; g += 128) *reinterpret_cast<float4*>(srow + g) = *reinterpret_cast<const float4*>(my_scales + g);
          } else {
            for (int g = lane * 2; g < sgroups; g += 64) *reinterpret_cast<float2*>(srow + g) = *reinterpret_cast<const float2*>(my_scales + g);
          }
        }
        __syncwarp();  // the next row reuses my_scales
      }
    }  // wi < n_work
    if (SORTED && (++round % kPublishRounds) == 0 && base + round_stride < n_work) publish_counts();
  }
  publish_counts();
}

__global__ void __launch_bounds__(kCommThreads) combine_pull_kernel(const CombineArgs a) {
  __shared__ int s_ok;
  const int El = a.num_experts / a.world;
  if (threadIdx.x == 0) s_ok = 1;
  if (*reinterpret_cast<volatile unsigned long long*>(&a.status->abort) != 0ull) return;
  __syncthreads();
  const unsigned long long ready_epoch = a.epoch_dev ? *a.epoch_dev : a.ready_epoch;
  if (ready_epoch != 0) {
    const unsigned long long* flags = reinterpret_cast<const unsigned long long*>(static_cast<unsigned char*>(a.peer_table[a.rank]) + a.ready_flags_heap_off);
    if (threadIdx.x < a.world && !wait_ge_bounded(flags + threadIdx.x, ready_epoch, a.status, kSiteCombineReady, threadIdx.x, a.timeout_ns)) s_ok = 0;
    __syncthreads();
    if (!s_ok) return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int chunks = a.H / 8;
  for (int t = blockIdx.x * wpb + warp; t < a.T; t += gridDim.x * wpb) {
    const uint4* rows[kMaxK];
    float w[kMaxK];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) {
      rows[j] = nullptr; w[j] = 0.0f;
      if (j < a.K) {
        const long long tj = static_cast<long long>(t) * a.K + j;
        const int e = a.topk_idx[tj];
        if (e < 0 || e >= a.num_experts) {  // flagged and left out of the sum (rows[j] stays null)
          if (lane == 0) report_failure(a.status, kStatusBadArg, kSiteExpertId, static_cast<unsigned long long>(tj), static_cast<unsigned long long>(static_cast<unsigned int>(e)), static_cast<unsigned long long>(a.num_experts));
          continue;
        }
        rows[j] = reinterpret_cast<const uint4*>(static_cast<unsigned char*>(a.peer_table[e / El]) + a.src_heap_off +
                                                 static_cast<long long>(a.dest_row[tj]) * a.H * 2);
        w[j] = a.weights ? a.weights[tj] : 1.0f;
      }
    }
    if (a.dot_out == nullptr) {
      uint4* out = reinterpret_cast<uint4*>(a.out + static_cast<long long>(t) * a.H);
      constexpr int U = 2;  // two chunks x K rows of peer loads in flight per lane
      for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
        uint4 v[U][kMaxK];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int j = 0; j < kMaxK; ++j)
            if (j < a.K && c0 + 32 * u < chunks) v[u][j] = rows[j] ? __ldcg(rows[j] + c0 + 32 * u) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + 32 * u;
          if (c >= chunks) break;
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
          for (int j = 0; j < kMaxK; ++j) {
            if (j >= a.K) break;
            float f[8];
            unpack8(v[u][j], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[j], f[i], acc[i]);
          }
          out[c] = pack8(acc);
        }
      }
    } else {
      const uint4* g = reinterpret_cast<const uint4*>(a.dot_with + static_cast<long long>(t) * a.H);
      float dots[kMaxK];
#pragma unroll
      for (int j = 0; j < kMaxK; ++j) dots[j] = 0.0f;
      for (int c = lane; c < chunks; c += 32) {
        float gf[8];
        unpack8(__ldg(g + c), gf);
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
          if (j >= a.K) break;
          float f[8];
          unpack8(rows[j] ? __ldcg(rows[j] + c) : make_uint4(0, 0, 0, 0), f);
#pragma unroll
          for (int i = 0; i < 8; ++i) dots[j] = fmaf(gf[i], f[i], dots[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxK; ++j) {
        if (j >= a.K) break;
        float d = dots[j];
#pragma unroll
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) a.dot_out[static_cast<long long>(t) * a.K + j] = d;
      }
    }
  }
}

__global__ void peer_signal_kernel(void* const* peer_table, int rank, int world, long long flags_heap_off, unsigned long long epoch,
                                   const unsigned long long* epoch_dev) {
  if (epoch_dev) epoch = *epoch_dev;
  if (threadIdx.x < world) {
    __threadfence_system();
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(peer_table[threadIdx.x]) + flags_heap_off);
    st_release_sys(dst + rank, epoch);
  }
}

__global__ void wait_counters_kernel(const unsigned long long* counter, const unsigned long long* target, int n, DeviceStatus* st,
                                     unsigned long long timeout_ns) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) wait_ge_bounded(counter + i, target[i], st, kSiteRailArrive, i, timeout_ns);
}

}  // namespace

cudaError_t launch_dispatch_push(const DispatchArgs& a, int ctas, cudaStream_t stream) {
  if (a.K < 1 || a.K > kMaxK || a.H % 256 || a.world < 1 || a.num_experts % a.world || ctas < 1) return cudaErrorInvalidValue;
  if (a.fp8 && a.H / 128 > kMaxScaleGroups) return cudaErrorInvalidValue;
  if ((a.xq != nullptr) != (a.xq_scales != nullptr) || (a.xq != nullptr && !a.fp8)) return cudaErrorInvalidValue;
  if (a.T == 0) return cudaSuccess;
  if (a.tile_rows < 0 || (a.tile_rows > 0 && a.num_tiles < 1)) return cudaErrorInvalidValue;
  const size_t smem = sizeof(int) * (a.tile_rows > 0 ? static_cast<size_t>(a.world) * a.num_tiles : static_cast<size_t>(a.num_experts));
  if (smem > 200 * 1024) return cudaErrorInvalidValue;  // per-CTA histogram of destination tiles must fit in shared memory
  auto go = [&](auto kern) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return e;
    }
    kern<<<ctas, kCommThreads, smem, stream>>>(a);
    note_launch();
    return cudaGetLastError();
  };
  const bool sorted = a.send_list != nullptr, scaled = a.row_scale != nullptr;
  if (a.fp8) return sorted ? go(dispatch_push_kernel<true, true, false>) : go(dispatch_push_kernel<true, false, false>);
  if (sorted) return scaled ? go(dispatch_push_kernel<false, true, true>) : go(dispatch_push_kernel<false, true, false>);
  return scaled ? go(dispatch_push_kernel<false, false, true>) : go(dispatch_push_kernel<false, false, false>);
}

cudaError_t launch_quantise_rows(const __nv_bfloat16* x, int T, int H, unsigned char* q, float* scales, int ctas, cudaStream_t stream) {
  if (H % 256 || H / 128 > kMaxScaleGroups || ctas < 1 || T < 0) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  quantise_rows_kernel<<<ctas, kCommThreads, 0, stream>>>(x, T, H, q, scales);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_combine_pull(const CombineArgs& a, int ctas, cudaStream_t stream) {
  if (a.K < 1 || a.K > kMaxK || a.H % 256 || a.world < 1 || a.num_experts % a.world || ctas < 1) return cudaErrorInvalidValue;
  if (a.T == 0) return cudaSuccess;
  combine_pull_kernel<<<ctas, kCommThreads, 0, stream>>>(a);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_peer_signal(void* const* peer_table, int rank, int world, long long flags_heap_off, unsigned long long epoch,
                               const unsigned long long* epoch_dev, cudaStream_t stream) {
  peer_signal_kernel<<<1, 64, 0, stream>>>(peer_table, rank, world, flags_heap_off, epoch, epoch_dev);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_wait_counters(const unsigned long long* counter, const unsigned long long* target, int n, DeviceStatus* status,
                                 unsigned long long timeout_ns, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  wait_counters_kernel<<<(n + 63) / 64, 64, 0, stream>>>(counter, target, n, status, timeout_ns);
  note_launch();
  return cudaGetLastError();
}

}  // namespace fastb
