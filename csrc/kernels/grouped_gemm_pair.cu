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

struct __align__(8) SmemCtl {
  uint64_t full[kStages], empty[kStages], acc_full[kAccStages], acc_empty[kAccStages], epi_load;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 + sizeof(SmemCtl);
static_assert(kSmemBytes <= 227 * 1024, "dynamic shared memory of one CTA on sm_100a");
static_assert(kABytes % 1024 == 0 && kBBytes % 1024 == 0, "operand tiles start on 1024-byte boundaries (128-byte swizzle atoms)");
static_assert(kAccStages * BN <= kTmemCols && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "tensor memory columns: power of two, at most 512");
static_assert(BK * 2 == 128, "one k block is one 128-byte swizzle row of bf16");
static_assert(kThreads == 32 * (2 + kEpiWarps) && kEpiWarps == 4, "warp roles: producer, MMA issuer, four epilogue warps (one per TMEM lane quarter)");

// TMA_EPI: outputs leave through the shared-memory ring and TMA stores; otherwise every epilogue
// thread writes (and, for the fused SwiGLU backward, reads) its own row in global memory.
template <GemmMode MODE, GemmEpilogue EPI, bool TMA_EPI>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                         const __grid_constant__ CUtensorMap map_c2, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* epi_stage = tiles + kStages * kStageBytes;  // two 16 KiB buffers, 1024-byte aligned like the operand tiles
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(epi_stage + kEpiBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_cta_rank();  // 0 = leader
  const bool leader = cta == 0;
  constexpr bool A_MN = MODE == GemmMode::kWgrad;
  constexpr bool B_MN = MODE != GemmMode::kForward;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < kAccStages; ++a) { mbar_init(&ctl->acc_full[a], 1); mbar_init(&ctl->acc_empty[a], 2 * kEpiWarps); }
    mbar_init(&ctl->epi_load, 1);
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
      int gated_group = -1;
      for (int tile = pair; ok && walk.locate(tile, tc); tile += pairs) {
        if (p.gate_counter != nullptr && tc.g != gated_group) {
          if (!(ok = wait_ge_bounded(p.gate_counter + tc.g, p.gate_target[tc.g], p.status, kSiteRailArrive, tc.g, p.timeout_ns))) { *abort_flag = 1; break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");
          gated_group = tc.g;
        }
        for (int kb = 0; kb < tc.red_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 100 + s, p.timeout_ns))) break;
          uint8_t* sa = tiles + s * kStageBytes;
          uint8_t* sb = sa + kABytes;
          const uint32_t full_leader = map_to_cta(smem_u32(&ctl->full[s]), 0);
          if (leader) mbar_arrive_expect_tx(&ctl->full[s], 2 * kStageBytes);
          const int m0 = tc.m_idx * TILE_M + static_cast<int>(cta) * PM;  // first row of my A half inside the group / fixed dim
          const int n0 = tc.n_idx * BN + static_cast<int>(cta) * PN;      // first column of my B half
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
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
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

template <GemmMode MODE, GemmEpilogue EPI>
cudaError_t launch_one(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const CUtensorMap& c2, const GemmArgs& args, int ctas,
                       cudaStream_t stream) {
  auto kern = args.direct_epilogue ? grouped_gemm_pair_kernel<MODE, EPI, false> : grouped_gemm_pair_kernel<MODE, EPI, true>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(ctas & ~1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
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

}  // namespace

cudaError_t launch_grouped_gemm_pair(GemmMode mode, GemmEpilogue epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c,
                                     const CUtensorMap* map_c2, const GemmArgs& args, int ctas, cudaStream_t stream) {
  if (ctas < 2) return cudaErrorInvalidValue;
  if ((args.c2 != nullptr) != (map_c2 != nullptr)) return cudaErrorInvalidValue;
  const CUtensorMap& c2 = map_c2 ? *map_c2 : map_c;  // unused by the kernel when args.c2 is null
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
