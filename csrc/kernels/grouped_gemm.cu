// Grouped bf16 GEMM on tcgen05 tensor cores with TMEM accumulators, fed by TMA.
//
// One persistent, warp-specialised kernel covers the three contractions of an expert MLP:
//   kForward : C[rows of g, N]  = A[rows of g, K]   * W_g[N, K]^T      (A, W K-major)
//   kDgrad   : dX[rows of g, K] = dY[rows of g, N]  * W_g[N, K]        (dY K-major, W MN-major)
//   kWgrad   : dW_g[N, K]       = dY[rows of g, N]^T * X[rows of g, K] (both MN-major, group = reduction range)
// Row ranges of the groups come from a device array of offsets (multiples of 128, produced on the
// device by the routing kernels), so no host round trip sits between routing and the GEMM.
// Roles: warp 0 = TMA producer (one elected lane), warp 1 = MMA issuer (one elected lane, owns
// the TMEM allocation), warps 2-5 = epilogue (tcgen05.ld -> bf16 -> global). Two accumulator
// stages of 256 TMEM columns let the epilogue of tile i overlap the main loop of tile i+1.
// Every mbarrier wait is bounded; on give-up the CTA unwinds, frees its TMEM and returns.
//
// The reference has no GEMM of any kind; this is part of the fused MoE path layered on its
// all-to-all (see SwiGLU epilogue below).
#include "gemm_common.cuh"

namespace fastb {

namespace {

using namespace ptx;
using namespace gemm;

constexpr int BM = 128;
constexpr int kStages = 4;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kABytes = BM * BK * 2;   // 16 KiB
constexpr int kBBytes = BN * BK * 2;   // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;

struct __align__(8) SmemCtl {
  uint64_t full[kStages], empty[kStages], acc_full[kAccStages], acc_empty[kAccStages];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + sizeof(SmemCtl);
static_assert(kSmemBytes <= 227 * 1024, "dynamic shared memory of one CTA on sm_100a");
static_assert(kABytes % 1024 == 0 && kBBytes % 1024 == 0, "operand tiles start on 1024-byte boundaries (128-byte swizzle atoms)");
static_assert(kAccStages * BN <= kTmemCols && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "tensor memory columns: power of two, at most 512");
static_assert(BK * 2 == 128, "one k block is one 128-byte swizzle row of bf16");
static_assert(kThreads == 32 * (2 + kEpiWarps) && kEpiWarps == 4, "warp roles: producer, MMA issuer, four epilogue warps (one per TMEM lane quarter)");

template <GemmMode MODE, GemmEpilogue EPI>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment.
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(tiles + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr bool A_MN = MODE == GemmMode::kWgrad;
  constexpr bool B_MN = MODE != GemmMode::kForward;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < kAccStages; ++a) { mbar_init(&ctl->acc_full[a], 1); mbar_init(&ctl->acc_empty[a], kEpiWarps); }
    ctl->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
  }
  if (warp == 1) { tmem_alloc(&ctl->tmem_base, kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  TileWalker<BM> walk{p.group_off, p.num_groups, p.tiles_n, p.fixed_m_tiles, p.red_len, MODE == GemmMode::kWgrad, p.band_rows};
  TileCoord tc;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      int gated = -1;
      for (int tile = blockIdx.x; ok && walk.locate(tile, tc); tile += gridDim.x) {
        if (p.gate_counter != nullptr) {
          // Arrival gate: rows are pushed by peers; start as soon as the group (or, with gate_tile_rows > 0,
          // the tile of that many rows of the grouped matrix) is all in.
          const int slot = min(p.gate_tile_rows > 0 ? (tc.row0 + tc.m_idx * BM) / p.gate_tile_rows : tc.g, p.gate_slots - 1);
          if (slot != gated) {
            if (!(ok = wait_ge_bounded(p.gate_counter + slot, p.gate_target[slot], p.status, kSiteRailArrive, slot, p.timeout_ns))) { *abort_flag = 1; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");  // peer (generic-proxy) writes before TMA (async-proxy) reads
            gated = slot;
          }
        }
        for (int kb = 0; kb < tc.red_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 100 + s, p.timeout_ns))) break;
          uint8_t* sa = tiles + s * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_arrive_expect_tx(&ctl->full[s], kStageBytes);
          if (MODE == GemmMode::kForward) {
            tma_load_2d(sa, &map_a, kb * BK, tc.row0 + tc.m_idx * BM, &ctl->full[s]);
            tma_load_2d(sb, &map_b, kb * BK, tc.g * p.b_rows_per_group + tc.n_idx * BN, &ctl->full[s]);
          } else if (MODE == GemmMode::kDgrad) {
            tma_load_2d(sa, &map_a, kb * BK, tc.row0 + tc.m_idx * BM, &ctl->full[s]);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)  // B[n_out, red] read from W_g[red][n_out]: boxes of 64 n_out x BK red
              tma_load_2d(sb + j * (BK * 128), &map_b, tc.n_idx * BN + j * 64, tc.g * p.b_rows_per_group + kb * BK, &ctl->full[s]);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &map_a, tc.m_idx * BM + j * 64, tc.row0 + kb * BK, &ctl->full[s]);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &map_b, tc.n_idx * BN + j * 64, tc.row0 + kb * BK, &ctl->full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && walk.locate(tile, tc); tile += gridDim.x) {
        if (tc.red_blocks == 0) continue;  // nothing to accumulate: the epilogue writes zeros on its own
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
            // K-major: 16 bf16 of k are 32 B further inside the 128 B swizzled line.
            // MN-major: 16 k lines are two 8-line atoms = 2048 B further.
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            mma_bf16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          mma_commit(&ctl->empty[s]);  // frees the smem stage once these MMAs have read it
        }
        if (ok) mma_commit(&ctl->acc_full[a]);
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> bf16 -> global ----------------
    const int quarter = warp & 3;  // a warp may only touch TMEM lanes 32*(warp%4) .. +31
    uint32_t acc_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && walk.locate(tile, tc); tile += gridDim.x) {
      const int a = acc_it % kAccStages;
      const uint32_t aph = (acc_it / kAccStages) & 1;
      const bool empty_reduction = tc.red_blocks == 0;  // wgrad of an expert that got no tokens
      if (!empty_reduction) {
        ++acc_it;
        if (!(ok = mbar_wait_bounded(&ctl->acc_full[a], aph, abort_flag, p.status, 400 + a, p.timeout_ns))) break;
        tc_fence_after_sync();
      }
      const int row_in_tile = quarter * 32 + lane;
      const long long c_row = MODE == GemmMode::kWgrad ? static_cast<long long>(tc.g) * p.c_rows_per_group + tc.m_idx * BM + row_in_tile
                                                        : static_cast<long long>(tc.row0) + tc.m_idx * BM + row_in_tile;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN;
      if (EPI == GemmEpilogue::kStore) {
        epilogue_store_row(p.c + c_row * p.ldc + static_cast<long long>(tc.n_idx) * BN, t_row, empty_reduction);
      } else {
        epilogue_swiglu_row(p.c + c_row * p.ldc + static_cast<long long>(tc.n_idx) * (BN / 2),
                            p.c2 ? p.c2 + c_row * p.ldc2 + static_cast<long long>(tc.n_idx) * BN : nullptr, t_row);
      }
      if (!empty_reduction) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);
      }
    }
  }
  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, kTmemCols); }
}

}  // namespace

int grouped_gemm_smem_bytes() { return kSmemBytes; }

template <GemmMode MODE, GemmEpilogue EPI>
static cudaError_t launch_one(const CUtensorMap& a, const CUtensorMap& b, const GemmArgs& args, int ctas, cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<MODE, EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<ctas, kThreads, kSmemBytes, stream>>>(a, b, args);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_grouped_gemm(GemmMode mode, GemmEpilogue epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& args,
                                int ctas, cudaStream_t stream) {
  if (ctas < 1) return cudaErrorInvalidValue;
  if (epi == GemmEpilogue::kSwiGLUBwd || args.a_scales != nullptr) return cudaErrorInvalidValue;  // only the CTA-pair kernel carries these
  if (epi == GemmEpilogue::kSwiGLU) {
    if (mode != GemmMode::kForward) return cudaErrorInvalidValue;
    return launch_one<GemmMode::kForward, GemmEpilogue::kSwiGLU>(map_a, map_b, args, ctas, stream);
  }
  switch (mode) {
    case GemmMode::kForward: return launch_one<GemmMode::kForward, GemmEpilogue::kStore>(map_a, map_b, args, ctas, stream);
    case GemmMode::kDgrad: return launch_one<GemmMode::kDgrad, GemmEpilogue::kStore>(map_a, map_b, args, ctas, stream);
    default: return launch_one<GemmMode::kWgrad, GemmEpilogue::kStore>(map_a, map_b, args, ctas, stream);
  }
}

}  // namespace fastb
