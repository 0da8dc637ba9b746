// Pieces shared by the one-CTA and the CTA-pair grouped GEMM kernels: tile walk and epilogues.
#pragma once
#include "api.h"
#include "sm100_ptx.cuh"
#include "tile_walker.h"

namespace fastb {
namespace gemm {

constexpr int BN = 256, BK = 64, UMMA_K = 16;

static_assert(BK == kWalkBK, "the tile walker counts reduction steps of BK");

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ uint4 pack8(const uint32_t* r) {
  return make_uint4(pack_bf16(__uint_as_float(r[0]), __uint_as_float(r[1])), pack_bf16(__uint_as_float(r[2]), __uint_as_float(r[3])),
                    pack_bf16(__uint_as_float(r[4]), __uint_as_float(r[5])), pack_bf16(__uint_as_float(r[6]), __uint_as_float(r[7])));
}

// One thread = one output row: reads its 256 fp32 accumulators from TMEM (t_row = TMEM address of
// the row's first column) and writes bf16 to global. `zero` writes zeros without touching TMEM.
__device__ __forceinline__ void epilogue_store_row(__nv_bfloat16* crow, uint32_t t_row, bool zero) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    if (!zero) { ptx::tmem_ld_32x32(t_row + c * 32, r); ptx::tmem_wait_ld(); }
    else {
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = 0;
    }
    uint4* dst = reinterpret_cast<uint4*>(crow + c * 32);
#pragma unroll
    for (int q = 0; q < 4; ++q) dst[q] = pack8(r + 8 * q);
  }
}

// SwiGLU: the 256 columns of a tile are [128 gate | 128 up] of the same 128 features.
__device__ __forceinline__ void epilogue_swiglu_row(__nv_bfloat16* arow, __nv_bfloat16* gurow, uint32_t t_row) {
#pragma unroll 1
  for (int c = 0; c < BN / 64; ++c) {
    uint32_t g[32], u[32];
    ptx::tmem_ld_32x32(t_row + c * 32, g);
    ptx::tmem_ld_32x32(t_row + BN / 2 + c * 32, u);
    ptx::tmem_wait_ld();
    uint4* dst = reinterpret_cast<uint4*>(arow + c * 32);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = silu(__uint_as_float(g[8 * q + i])) * __uint_as_float(u[8 * q + i]);
      dst[q] = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
    }
    if (gurow) {
      uint4* dg = reinterpret_cast<uint4*>(gurow + c * 32);
      uint4* du = reinterpret_cast<uint4*>(gurow + BN / 2 + c * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q) { dg[q] = pack8(g + 8 * q); du[q] = pack8(u + 8 * q); }
    }
  }
}

__device__ __forceinline__ void unpack8_bf16(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// SwiGLU backward fused into the dgrad that produces d(act): the 256 accumulator columns of the
// tile are d(act) for 256 consecutive features = two blocks of 128; block b sits in the gate|up
// layout at columns [256 b, 256 b + 128) (gate) and [256 b + 128, 256 b + 256) (up). gu_row and
// dgu_row point at the row's first column of this tile's 512-column span.
__device__ __forceinline__ void epilogue_swiglu_bwd_row(__nv_bfloat16* dgu_row, const __nv_bfloat16* gu_row, uint32_t t_row) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t d[32];
    ptx::tmem_ld_32x32(t_row + c * 32, d);
    const int col = (c / 4) * 256 + (c % 4) * 32;
    const uint4* gp = reinterpret_cast<const uint4*>(gu_row + col);
    const uint4* up = reinterpret_cast<const uint4*>(gu_row + col + 128);
    uint4 gv[4], uv[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) { gv[q] = __ldg(gp + q); uv[q] = __ldg(up + q); }
    ptx::tmem_wait_ld();
    uint4* dg = reinterpret_cast<uint4*>(dgu_row + col);
    uint4* du = reinterpret_cast<uint4*>(dgu_row + col + 128);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float g[8], u[8], og[8], ou[8];
      unpack8_bf16(gv[q], g);
      unpack8_bf16(uv[q], u);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // d(act) is rounded to bf16 first, as the unfused path stores it before the element-wise kernel
        const float da = __bfloat162float(__float2bfloat16_rn(__uint_as_float(d[8 * q + i])));
        const float s = 1.0f / (1.0f + __expf(-g[i]));
        const float sl = g[i] * s;
        ou[i] = da * sl;
        og[i] = da * u[i] * (s + sl * (1.0f - s));
      }
      dg[q] = make_uint4(pack_bf16(og[0], og[1]), pack_bf16(og[2], og[3]), pack_bf16(og[4], og[5]), pack_bf16(og[6], og[7]));
      du[q] = make_uint4(pack_bf16(ou[0], ou[1]), pack_bf16(ou[2], ou[3]), pack_bf16(ou[4], ou[5]), pack_bf16(ou[6], ou[7]));
    }
  }
}

}  // namespace gemm
}  // namespace fastb
