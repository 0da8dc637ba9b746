// Epilogues of the CTA-pair grouped GEMM that leave through shared memory and TMA stores.
//
// Each of the 128 epilogue threads owns one accumulator row in tensor memory. Writing that row
// straight to global memory makes every warp-wide 16-byte store touch 32 different 128-byte lines.
// Here a thread converts 64 columns at a time and drops them into a 128-row x 128-byte staging
// buffer laid out with the 128-byte swizzle (16-byte chunk j of row r sits at chunk j ^ (r & 7)),
// which is free of bank conflicts for this access pattern, and one elected thread hands the
// buffer to the TMA unit (cp.async.bulk.tensor store, bulk-group completion). Two buffers form a
// ring, so that converting chunk n overlaps the store of chunk n - 1. The fused SwiGLU backward
// also reads its saved gate|up tile through TMA loads into the same two buffers and transforms
// it in place.
//
// All TMA loads here are plain loads of this GPU's own memory.
#pragma once
#include "gemm_common.cuh"

namespace fastb {
namespace gemm {

constexpr int kEpiChunkCols = 64;                 // bf16 columns per staged chunk = one 128-byte swizzle row
constexpr int kEpiRows = 128;                     // rows of one CTA's accumulator half
constexpr int kEpiBufBytes = kEpiRows * 128;      // 16 KiB
constexpr int kEpiBytes = 2 * kEpiBufBytes;
constexpr int kEpiThreads = 128;

// Named barrier 1: the four epilogue warps only (barrier 0 is __syncthreads of the whole CTA).
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(ptx::smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most N of this thread's bulk groups still have to READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// Until every bulk group of this thread is complete (its global writes are done).
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint4* chunk_ptr(uint8_t* buf, int r, int j) {
  return reinterpret_cast<uint4*>(buf + r * 128 + ((j ^ (r & 7)) << 4));
}
// 32 fp32 values (bit patterns in v) of row r -> bf16 columns [32 h, 32 h + 32) of the chunk in buf.
__device__ __forceinline__ void stage_half(uint8_t* buf, int r, int h, const uint32_t (&v)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) *chunk_ptr(buf, r, 4 * h + q) = pack8(v + 8 * q);
}

// Ring of two staging buffers. Every epilogue thread calls acquire / release in the same order;
// `issuer` is true for the single thread that issues (and therefore tracks) the bulk stores.
struct EpiRing {
  uint8_t* base;
  bool issuer;
  uint32_t n;
  __device__ __forceinline__ uint8_t* acquire() {
    if (issuer) bulk_wait_read<1>();  // the store that read this buffer two chunks ago is done with it
    epi_bar();
    return base + (n & 1u) * kEpiBufBytes;
  }
  __device__ __forceinline__ void release(const CUtensorMap* map, int x, int y) {
    ptx::fence_proxy_async_smem();    // my generic-proxy writes are visible to the TMA unit
    epi_bar();
    if (issuer) { tma_store_2d(map, base + (n & 1u) * kEpiBufBytes, x, y); bulk_commit(); }
    ++n;
  }
  // Before the CTA exits (or frees anything): all stores have landed.
  __device__ __forceinline__ void drain() { if (issuer) bulk_wait_all(); }
};

// Plain store of the CTA's 128 x 256 accumulator half: four chunks of 64 columns.
__device__ __forceinline__ void epilogue_store_tma(EpiRing& ring, const CUtensorMap* map_c, int col0, int row0, int r, uint32_t t_row, bool zero) {
#pragma unroll 1
  for (int c = 0; c < BN / kEpiChunkCols; ++c) {
    uint32_t lo[32], hi[32];
    if (!zero) {
      ptx::tmem_ld_32x32(t_row + c * kEpiChunkCols, lo);
      ptx::tmem_ld_32x32(t_row + c * kEpiChunkCols + 32, hi);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) { lo[i] = 0; hi[i] = 0; }
    }
    uint8_t* buf = ring.acquire();
    if (!zero) ptx::tmem_wait_ld();
    stage_half(buf, r, 0, lo);
    stage_half(buf, r, 1, hi);
    ring.release(map_c, col0 + c * kEpiChunkCols, row0);
  }
}

// SwiGLU forward: the 256 accumulator columns are [128 gate | 128 up] of the same 128 features.
// act (map_act, 128 columns per tile) = silu(gate) * up; with map_gu the raw tile is kept too.
__device__ __forceinline__ void epilogue_swiglu_tma(EpiRing& ring, const CUtensorMap* map_act, int act_col0, const CUtensorMap* map_gu, int gu_col0,
                                                    int row0, int r, uint32_t t_row) {
#pragma unroll 1
  for (int c = 0; c < (BN / 2) / kEpiChunkCols; ++c) {
    uint32_t o[2][32];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t g[32], u[32];
      ptx::tmem_ld_32x32(t_row + c * kEpiChunkCols + h * 32, g);
      ptx::tmem_ld_32x32(t_row + BN / 2 + c * kEpiChunkCols + h * 32, u);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[h][i] = __float_as_uint(silu(__uint_as_float(g[i])) * __uint_as_float(u[i]));
    }
    uint8_t* buf = ring.acquire();
    stage_half(buf, r, 0, o[0]);
    stage_half(buf, r, 1, o[1]);
    ring.release(map_act, act_col0 + c * kEpiChunkCols, row0);
  }
  if (map_gu != nullptr) epilogue_store_tma(ring, map_gu, gu_col0, row0, r, t_row, false);
}

// SwiGLU backward fused into the dgrad that produces d(act): the tile's 256 accumulator columns
// are d(act) of 256 consecutive features = two blocks of 128; block b sits in the gate|up layout
// at columns [256 b, 256 b + 128) (gate) and [256 b + 128, 256 b + 256) (up) of the tile's
// 512-column span that starts at gu_col0. Per chunk of 64 features the saved gate and up tiles
// are TMA-loaded into the two staging buffers, every thread turns its own row into d(gate) and
// d(up) in place, and both buffers are stored to map_dgu at the same coordinates.
// `load_bar` is an mbarrier (count 1) of this CTA; `load_phase` carries its parity across calls.
// Returns false if the wait for a load gave up.
__device__ __forceinline__ bool epilogue_swiglu_bwd_tma(EpiRing& ring, const CUtensorMap* map_dgu, const CUtensorMap* map_gu, int gu_col0, int row0,
                                                        int r, uint32_t t_row, uint64_t* load_bar, uint32_t& load_phase, volatile int* abort_flag,
                                                        DeviceStatus* st, unsigned long long timeout_ns) {
  uint8_t* gbuf = ring.base;
  uint8_t* ubuf = ring.base + kEpiBufBytes;
#pragma unroll 1
  for (int c = 0; c < BN / kEpiChunkCols; ++c) {
    const int col = gu_col0 + (c >> 1) * 256 + (c & 1) * kEpiChunkCols;
    if (ring.issuer) {
      bulk_wait_read<0>();  // the previous chunk's stores have read both buffers
      ptx::mbar_arrive_expect_tx(load_bar, 2 * kEpiBufBytes);
      ptx::tma_load_2d(gbuf, map_gu, col, row0, load_bar);
      ptx::tma_load_2d(ubuf, map_gu, col + 128, row0, load_bar);
    }
    uint32_t d[2][32];
    ptx::tmem_ld_32x32(t_row + c * kEpiChunkCols, d[0]);
    ptx::tmem_ld_32x32(t_row + c * kEpiChunkCols + 32, d[1]);
    if (!ptx::mbar_wait_bounded(load_bar, load_phase, abort_flag, st, 500, timeout_ns)) { ptx::tmem_wait_ld(); return false; }
    load_phase ^= 1u;
    ptx::tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4* gp = chunk_ptr(gbuf, r, j);
      uint4* up = chunk_ptr(ubuf, r, j);
      float g[8], u[8], og[8], ou[8];
      unpack8_bf16(*gp, g);
      unpack8_bf16(*up, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // d(act) is rounded to bf16 first, as the unfused path stores it before the element-wise kernel
        const float da = __bfloat162float(__float2bfloat16_rn(__uint_as_float(d[j >> 2][(j & 3) * 8 + i])));
        const float s = 1.0f / (1.0f + __expf(-g[i]));
        const float sl = g[i] * s;
        ou[i] = da * sl;
        og[i] = da * u[i] * (s + sl * (1.0f - s));
      }
      *gp = make_uint4(pack_bf16(og[0], og[1]), pack_bf16(og[2], og[3]), pack_bf16(og[4], og[5]), pack_bf16(og[6], og[7]));
      *up = make_uint4(pack_bf16(ou[0], ou[1]), pack_bf16(ou[2], ou[3]), pack_bf16(ou[4], ou[5]), pack_bf16(ou[6], ou[7]));
    }
    ptx::fence_proxy_async_smem();
    epi_bar();
    if (ring.issuer) {
      tma_store_2d(map_dgu, gbuf, col, row0);
      tma_store_2d(map_dgu, ubuf, col + 128, row0);
      bulk_commit();
    }
  }
  return true;
}

}  // namespace gemm
}  // namespace fastb
