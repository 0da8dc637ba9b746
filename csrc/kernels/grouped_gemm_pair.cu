// Grouped bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 over a 256 x 256 tile.
//
// Two CTAs of a cluster share one output tile. CTA r of the pair loads its 128 rows of A and its
// 128 columns of B (half of each operand, plain TMA loads, no multicast), the leader (cluster
// rank 0) issues one M=256 MMA per 16-wide k step, and each CTA keeps its 128 x 256 fp32
// accumulator half in its own tensor memory and runs its own epilogue. Halving the B traffic per
// SM leaves room for six smem stages of 32 KiB instead of four of 48 KiB.
//
// Barrier map (same smem offsets in both CTAs):
//   full[s]      leader only: one arrive.expect_tx by the leader's producer for the bytes of BOTH
//                CTAs; the peer's TMA loads count onto it through the pair-wide load form.
//   empty[s]     each CTA: released by the leader's commit, multicast to both CTAs.
//   acc_full[a]  each CTA: leader's commit after the last k step, multicast to both.
//   acc_empty[a] leader only: 8 arrivals (4 epilogue warps of each CTA; the peer's arrive remotely).
//   epi_load     each CTA: bytes of the saved gate|up tiles the fused SwiGLU-backward epilogue loads.
// Same modes, arrival gate and bounded waits as the one-CTA kernel; group offsets must be multiples
// of 256. The epilogues leave through a two-buffer shared-memory ring and TMA stores
// (gemm_epilogue_tma.cuh): output matrices are described by tensor maps of 64 x 128 boxes.
#include <cuda_fp8.h>

#include "gemm_epilogue_tma.cuh"

namespace fastb {

namespace {

using namespace ptx;
using namespace gemm;

constexpr int PM = 128;            // rows per CTA
constexpr int TILE_M = 2 * PM;     // rows per pair
constexpr int PN = BN / 2;         // B columns loaded per CTA
constexpr int kStages = 6;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kABytes = PM * BK * 2;  // 16 KiB
constexpr int kBBytes = PN * BK * 2;  // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
// e4m3 A operand (forward only): rows arrive as e4m3 bytes with one fp32 scale per 128 elements.
// The producer TMA-loads each 128 x 64-byte block into a small ring; converter warps (one ring slot
// each) turn it into the bf16 swizzled A tile of the stage (value x scale, rounded to bf16) and
// arrive on the stage's full barrier beside the bytes of B. One smem stage less pays for the ring.
constexpr int kStagesFp8 = 5;
constexpr int kQStages = 4;
constexpr int kQBytes = PM * BK;      // 8 KiB of e4m3
constexpr int kCvtWarps = 4;
constexpr int kThreadsFp8 = kThreads + 32 * kCvtWarps;

struct __align__(8) SmemCtl {
  uint64_t full[kStages], empty[kStages], acc_full[kAccStages], acc_empty[kAccStages], epi_load, q_full[kQStages], q_empty[kQStages];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 + sizeof(SmemCtl);
constexpr int kSmemBytesFp8 = kStagesFp8 * kStageBytes + kQStages * kQBytes + kEpiBytes + 1024 + sizeof(SmemCtl);
static_assert(kSmemBytes <= 227 * 1024 && kSmemBytesFp8 <= 227 * 1024, "dynamic shared memory of one CTA on sm_100a");
static_assert(kStagesFp8 <= kStages, "barrier arrays are sized for the larger stage count");
static_assert(kABytes % 1024 == 0 && kBBytes % 1024 == 0, "operand tiles start on 1024-byte boundaries (128-byte swizzle atoms)");
static_assert(kAccStages * BN <= kTmemCols && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "tensor memory columns: power of two, at most 512");
static_assert(BK * 2 == 128, "one k block is one 128-byte swizzle row of bf16");
static_assert(kThreads == 32 * (2 + kEpiWarps) && kEpiWarps == 4, "warp roles: producer, MMA issuer, four epilogue warps (one per TMEM lane quarter)");

// Packed bf16 helpers of the e4m3 converters (bf16 arithmetic keeps subnormal inputs).
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16_pair_of(float x) {  // x is bf16-representable by construction; truncation is exact then
  const uint32_t h = __float_as_uint(x) >> 16;
  return h | (h << 16);
}

// TMA_EPI: outputs leave through the shared-memory ring and TMA stores; otherwise every epilogue
// thread writes (and, for the fused SwiGLU backward, reads) its own row in global memory.
// A_FP8 (forward only): map_a describes e4m3 bytes (boxes of 64 bytes x 128 rows, no swizzle) and
// p.a_scales their 1x128 scales; see kStagesFp8 above.
template <GemmMode MODE, GemmEpilogue EPI, bool TMA_EPI, bool A_FP8>
__global__ void __launch_bounds__(A_FP8 ? kThreadsFp8 : kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                         const __grid_constant__ CUtensorMap map_c2, const GemmArgs p) {
  static_assert(!A_FP8 || MODE == GemmMode::kForward, "the e4m3 operand feeds the forward contraction only");
  constexpr int NS = A_FP8 ? kStagesFp8 : kStages;  // operand stages in use
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_ring = tiles + NS * kStageBytes;                                 // A_FP8 only: kQStages x 8 KiB of e4m3
  uint8_t* epi_stage = q_ring + (A_FP8 ? kQStages * kQBytes : 0);            // two 16 KiB buffers, 1024-byte aligned like the operand tiles
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(epi_stage + kEpiBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_cta_rank();  // 0 = leader
  const bool leader = cta == 0;
  constexpr bool A_MN = MODE == GemmMode::kWgrad;
  constexpr bool B_MN = MODE != GemmMode::kForward;

  if (threadIdx.x == 0) {
    // full[s] (leader's copy is the one in use): the producer's expect_tx arrival, plus one arrival from
    // each CTA's converter warp when the A tile is written by them instead of by TMA.
    for (int s = 0; s < NS; ++s) { mbar_init(&ctl->full[s], A_FP8 ? 1 + 2 : 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < kAccStages; ++a) { mbar_init(&ctl->acc_full[a], 1); mbar_init(&ctl->acc_empty[a], 2 * kEpiWarps); }
    mbar_init(&ctl->epi_load, 1);
    for (int q = 0; q < kQStages; ++q) { mbar_init(&ctl->q_full[q], 1); mbar_init(&ctl->q_empty[q], 1); }
    ctl->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    prefetch_tmap(&map_c);
    if (EPI != GemmEpilogue::kStore) prefetch_tmap(&map_c2);
  }
  if (warp == 1) { tmem_alloc_pair(&ctl->tmem_base, kTmemCols); tmem_relinquish_pair(); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  TileWalker<TILE_M> walk{p.group_off, p.num_groups, p.tiles_n, p.fixed_m_tiles, p.red_len, MODE == GemmMode::kWgrad, p.band_rows};
  TileCoord tc;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs, each for its own halves) ----------------
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      int gated = -1;
      for (int tile = pair; ok && walk.locate(tile, tc); tile += pairs) {
        if (p.gate_counter != nullptr) {
          // Arrival gate: per group, or (gate_tile_rows > 0) per tile of that many rows of the grouped matrix.
          const int slot = min(p.gate_tile_rows > 0 ? (tc.row0 + tc.m_idx * TILE_M) / p.gate_tile_rows : tc.g, p.gate_slots - 1);
          if (slot != gated) {
            if (!(ok = wait_ge_bounded(p.gate_counter + slot, p.gate_target[slot], p.status, kSiteRailArrive, slot, p.timeout_ns))) { *abort_flag = 1; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");
            gated = slot;
          }
        }
        for (int kb = 0; kb < tc.red_blocks; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!(ok = mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 100 + s, p.timeout_ns))) break;
          uint8_t* sa = tiles + s * kStageBytes;
          uint8_t* sb = sa + kABytes;
          const uint32_t full_leader = map_to_cta(smem_u32(&ctl->full[s]), 0);
          const int m0 = tc.m_idx * TILE_M + static_cast<int>(cta) * PM;  // first row of my A half inside the group / fixed dim
          const int n0 = tc.n_idx * BN + static_cast<int>(cta) * PN;      // first column of my B half
          if (A_FP8) {  // e4m3 block into the ring (its converter warp writes the A half of the stage), B by TMA as usual
            const int q = it % kQStages;
            const uint32_t qph = (it / kQStages) & 1;
            if (!(ok = mbar_wait_bounded(&ctl->q_empty[q], qph ^ 1, abort_flag, p.status, 600 + q, p.timeout_ns))) break;
            mbar_arrive_expect_tx(&ctl->q_full[q], kQBytes);
            tma_load_2d(q_ring + q * kQBytes, &map_a, kb * BK, tc.row0 + m0, &ctl->q_full[q]);
            if (leader) mbar_arrive_expect_tx(&ctl->full[s], 2 * kBBytes);
            tma_load_2d_pair(sb, &map_b, kb * BK, tc.g * p.b_rows_per_group + n0, full_leader);
            continue;
          }
          if (leader) mbar_arrive_expect_tx(&ctl->full[s], 2 * kStageBytes);
          if (MODE == GemmMode::kForward) {
            tma_load_2d_pair(sa, &map_a, kb * BK, tc.row0 + m0, full_leader);
            tma_load_2d_pair(sb, &map_b, kb * BK, tc.g * p.b_rows_per_group + n0, full_leader);
          } else if (MODE == GemmMode::kDgrad) {
            tma_load_2d_pair(sa, &map_a, kb * BK, tc.row0 + m0, full_leader);
#pragma unroll
            for (int j = 0; j < PN / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), &map_b, n0 + j * 64, tc.g * p.b_rows_per_group + kb * BK, full_leader);
          } else {
#pragma unroll
            for (int j = 0; j < PM / 64; ++j)
              tma_load_2d_pair(sa + j * (BK * 128), &map_a, m0 + j * 64, tc.row0 + kb * BK, full_leader);
#pragma unroll
            for (int j = 0; j < PN / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), &map_b, n0 + j * 64, tc.row0 + kb * BK, full_leader);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, BN, A_MN, B_MN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = pair; ok && walk.locate(tile, tc); tile += pairs) {
        if (tc.red_blocks == 0) continue;
        const int a = acc_it % kAccStages;
        const uint32_t aph = (acc_it / kAccStages) & 1;
        ++acc_it;
        if (!(ok = mbar_wait_bounded(&ctl->acc_empty[a], aph ^ 1, abort_flag, p.status, 200 + a, p.timeout_ns))) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = 0; kb < tc.red_blocks; ++kb, ++it) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!(ok = mbar_wait_bounded(&ctl->full[s], ph, abort_flag, p.status, 300 + s, p.timeout_ns))) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + s * kStageBytes), sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            mma_bf16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          mma_commit_pair(&ctl->empty[s], 0x3);
        }
        if (ok) mma_commit_pair(&ctl->acc_full[a], 0x3);
      }
    }
  } else if (A_FP8 && warp >= 2 + kEpiWarps) {
    // ---------------- e4m3 -> bf16 converters (both CTAs, each for its 128 rows of A) ----------------
    // Converter warp w owns every k block with index = w (mod kCvtWarps), i.e. ring slot w: it converts the
    // whole 128 x 64 block alone, so that the proxy fence each block needs (generic-proxy writes before the
    // tensor core's async-proxy reads, several hundred cycles) overlaps with the other warps' conversions.
    // Lane l owns the 16-byte piece (l & 3) of rows (l >> 2) + 8 i: a pass reads 512 contiguous bytes of the
    // ring and writes eight full 128-byte rows of the swizzled tile.
    static_assert(kQStages == kCvtWarps, "one ring slot per converter warp");
    const int cw = warp - (2 + kEpiWarps);
    const int sub = lane & 3, r8 = lane >> 2;
    const int sgroups = p.red_len / 128;
    const uint32_t two60 = 0x5D805D80u;  // bf16 pair (2^60, 2^60)
    uint32_t it = 0;
    bool ok = true;
    for (int tile = pair; ok && walk.locate(tile, tc); tile += pairs) {
      const int m0 = tc.m_idx * TILE_M + static_cast<int>(cta) * PM;
      const int real_rows = p.group_rows ? min(p.group_rows[tc.g], 1 << 30) : 1 << 30;
      const float* srow = p.a_scales + static_cast<long long>(tc.row0 + m0 + r8) * sgroups;
      for (int kb = 0; kb < tc.red_blocks; ++kb, ++it) {
        if (static_cast<int>(it % kCvtWarps) != cw) continue;
        const int s = it % NS;
        // This block's scales (one per row; two k blocks share a scale group). Requested before the wait for the
        // block itself, whose latency they hide behind. Rows past the group's real end become zeros, whatever the
        // buffers hold there.
        uint32_t s2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int row = r8 + 8 * i;
          const float sc = m0 + row < real_rows ? __ldg(srow + static_cast<long long>(8 * i) * sgroups + (kb >> 1)) : 0.0f;
          s2[i] = bf16_pair_of(sc * 1.152921504606846976e18f);  // (scale x 2^60) twice
        }
        if (!(ok = mbar_wait_bounded(&ctl->q_full[cw], (it / kQStages) & 1, abort_flag, p.status, 700 + cw, p.timeout_ns))) break;
        const uint8_t* qb = q_ring + cw * kQBytes;
        uint8_t* sa = tiles + s * kStageBytes;
        // No conversion instruction is used. An e4m3 byte (sign s, magnitude g = eeeemmm) read as the bf16 bit
        // pattern (s << 15) | (g << 4) is exactly the value x 2^-120, subnormals included (both formats then sit at
        // exponent field 0). Two exact multiplications of the bf16 pair bring it back: by 2^60, then by scale x 2^60;
        // senders make their scales bf16-representable, so the second product is value x scale rounded once to bf16
        // (other scales are used truncated to bf16 precision). A scale of zero (dead row) gives zeros.
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int row = r8 + 8 * i;
          const uint4 v = *reinterpret_cast<const uint4*>(qb + row * BK + sub * 16);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t lo = __byte_perm(w[e], 0u, 0x4140), hi = __byte_perm(w[e], 0u, 0x4342);  // bytes spread to 16-bit lanes
            const uint32_t blo = ((lo & 0x007f007fu) << 4) | ((lo & 0x00800080u) << 8);
            const uint32_t bhi = ((hi & 0x007f007fu) << 4) | ((hi & 0x00800080u) << 8);
            o[2 * e] = mul_bf16x2(mul_bf16x2(blo, two60), s2[i]);
            o[2 * e + 1] = mul_bf16x2(mul_bf16x2(bhi, two60), s2[i]);
          }
          *reinterpret_cast<uint4*>(sa + row * 128 + (((2 * sub) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(sa + row * 128 + (((2 * sub + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        fence_proxy_async_smem();  // the tensor core reads these bytes through the async proxy
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&ctl->q_empty[cw]);
          mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->full[s]), 0));
        }
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, each for its 128 rows) ----------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // my accumulator row inside this CTA's half
    EpiRing ring{epi_stage, threadIdx.x == 64, 0u};
    uint32_t acc_it = 0, load_phase = 0;
    bool ok = true;
    for (int tile = pair; ok && walk.locate(tile, tc); tile += pairs) {
      const int a = acc_it % kAccStages;
      const uint32_t aph = (acc_it / kAccStages) & 1;
      const bool empty_reduction = tc.red_blocks == 0;
      if (!empty_reduction) {
        ++acc_it;
        if (!(ok = mbar_wait_bounded(&ctl->acc_full[a], aph, abort_flag, p.status, 400 + a, p.timeout_ns))) break;
        tc_fence_after_sync();
      }
      // first output row of this CTA's half (TMA store coordinate)
      const int c_row0 = (MODE == GemmMode::kWgrad ? tc.g * p.c_rows_per_group : tc.row0) + tc.m_idx * TILE_M + static_cast<int>(cta) * PM;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN;
      if (!TMA_EPI) {
        const long long c_row = static_cast<long long>(c_row0) + r;
        if (EPI == GemmEpilogue::kStore) {
          epilogue_store_row(p.c + c_row * p.ldc + static_cast<long long>(tc.n_idx) * BN, t_row, empty_reduction);
        } else if (EPI == GemmEpilogue::kSwiGLUBwd) {
          epilogue_swiglu_bwd_row(p.c + c_row * p.ldc + static_cast<long long>(tc.n_idx) * (2 * BN),
                                  p.c2 + c_row * p.ldc2 + static_cast<long long>(tc.n_idx) * (2 * BN), t_row);
        } else {
          epilogue_swiglu_row(p.c + c_row * p.ldc + static_cast<long long>(tc.n_idx) * (BN / 2),
                              p.c2 ? p.c2 + c_row * p.ldc2 + static_cast<long long>(tc.n_idx) * BN : nullptr, t_row);
        }
      } else if (EPI == GemmEpilogue::kStore) {
        epilogue_store_tma(ring, &map_c, tc.n_idx * BN, c_row0, r, t_row, empty_reduction);
      } else if (EPI == GemmEpilogue::kSwiGLUBwd) {
        ok = epilogue_swiglu_bwd_tma(ring, &map_c, &map_c2, tc.n_idx * (2 * BN), c_row0, r, t_row, &ctl->epi_load, load_phase, abort_flag, p.status, p.timeout_ns);
      } else {
        epilogue_swiglu_tma(ring, &map_c, tc.n_idx * (BN / 2), p.c2 ? &map_c2 : nullptr, tc.n_idx * BN, c_row0, r, t_row);
      }
      if (!empty_reduction) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->acc_empty[a]), 0));
      }
    }
    ring.drain();  // every bulk store of this CTA has landed before anything is torn down
  }
  // ---------------- teardown: nobody frees tensor memory while the pair still uses it ----------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc_pair(tmem_base, kTmemCols); }
}

template <class Kernel>
cudaError_t launch_kernel(Kernel kern, int threads, int smem, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const CUtensorMap& c2,
                          const GemmArgs& args, int ctas, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(ctas & ~1);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, a, b, c, c2, args);
  if (e == cudaSuccess) note_launch();
  return e;
}

template <GemmMode MODE, GemmEpilogue EPI>
cudaError_t launch_one(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const CUtensorMap& c2, const GemmArgs& args, int ctas,
                       cudaStream_t stream) {
  if (args.direct_epilogue) return launch_kernel(grouped_gemm_pair_kernel<MODE, EPI, false, false>, kThreads, kSmemBytes, a, b, c, c2, args, ctas, stream);
  return launch_kernel(grouped_gemm_pair_kernel<MODE, EPI, true, false>, kThreads, kSmemBytes, a, b, c, c2, args, ctas, stream);
}

}  // namespace

cudaError_t launch_grouped_gemm_pair(GemmMode mode, GemmEpilogue epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c,
                                     const CUtensorMap* map_c2, const GemmArgs& args, int ctas, cudaStream_t stream) {
  if (ctas < 2) return cudaErrorInvalidValue;
  if ((args.c2 != nullptr) != (map_c2 != nullptr)) return cudaErrorInvalidValue;
  const CUtensorMap& c2 = map_c2 ? *map_c2 : map_c;  // unused by the kernel when args.c2 is null
  if (args.a_scales != nullptr) {
    // e4m3 rows with 1x128 scales as operand A: forward contractions, TMA-store epilogues only.
    if (mode != GemmMode::kForward || args.direct_epilogue || args.red_len % 128 != 0 || epi == GemmEpilogue::kSwiGLUBwd) return cudaErrorInvalidValue;
    if (epi == GemmEpilogue::kSwiGLU)
      return launch_kernel(grouped_gemm_pair_kernel<GemmMode::kForward, GemmEpilogue::kSwiGLU, true, true>, kThreadsFp8, kSmemBytesFp8, map_a, map_b, map_c, c2, args, ctas, stream);
    return launch_kernel(grouped_gemm_pair_kernel<GemmMode::kForward, GemmEpilogue::kStore, true, true>, kThreadsFp8, kSmemBytesFp8, map_a, map_b, map_c, c2, args, ctas, stream);
  }
  if (epi == GemmEpilogue::kSwiGLU) {
    if (mode != GemmMode::kForward) return cudaErrorInvalidValue;
    return launch_one<GemmMode::kForward, GemmEpilogue::kSwiGLU>(map_a, map_b, map_c, c2, args, ctas, stream);
  }
  if (epi == GemmEpilogue::kSwiGLUBwd) {
    if (mode != GemmMode::kDgrad || args.c2 == nullptr) return cudaErrorInvalidValue;
    return launch_one<GemmMode::kDgrad, GemmEpilogue::kSwiGLUBwd>(map_a, map_b, map_c, c2, args, ctas, stream);
  }
  switch (mode) {
    case GemmMode::kForward: return launch_one<GemmMode::kForward, GemmEpilogue::kStore>(map_a, map_b, map_c, c2, args, ctas, stream);
    case GemmMode::kDgrad: return launch_one<GemmMode::kDgrad, GemmEpilogue::kStore>(map_a, map_b, map_c, c2, args, ctas, stream);
    default: return launch_one<GemmMode::kWgrad, GemmEpilogue::kStore>(map_a, map_b, map_c, c2, args, ctas, stream);
  }
}

}  // namespace fastb
