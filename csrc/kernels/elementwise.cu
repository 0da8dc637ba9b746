// Element-wise kernels of the expert MLP and the optimizer (memory-bound; 16-byte accesses).
#include <cuda_fp8.h>

#include "api.h"

namespace fastb {

namespace {

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

// gate_up rows are tiles of [128 gate | 128 up]; chunk c (8 features) of tile n sits at
// 256 n + 8 (c % 16) for the gate and 128 further for the up projection.
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ gu, uint4* __restrict__ act, long long rows, int inter) {
  const int cpr = inter / 8;  // output chunks per row
  const long long total = rows * cpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cpr;
    const int c = static_cast<int>(i % cpr);
    const long long base = r * (2 * cpr) + (c / 16) * 32 + (c % 16);
    float g[8], u[8], o[8];
    unpack8(gu[base], g);
    unpack8(gu[base + 16], u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.0f + __expf(-g[k])) * u[k];
    act[i] = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const uint4* __restrict__ gu, const uint4* __restrict__ dact, uint4* __restrict__ dgu, long long rows, int inter,
                                  const int* __restrict__ rows_dev) {
  if (rows_dev) rows = min(rows, static_cast<long long>(*rows_dev));  // rows in use this step (device-side count)
  const int cpr = inter / 8;
  const long long total = rows * cpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cpr;
    const int c = static_cast<int>(i % cpr);
    const long long base = r * (2 * cpr) + (c / 16) * 32 + (c % 16);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(gu[base], g);
    unpack8(gu[base + 16], u);
    unpack8(dact[i], d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.0f / (1.0f + __expf(-g[k]));
      const float silu = g[k] * s;
      du[k] = d[k] * silu;
      dg[k] = d[k] * u[k] * (s + silu * (1.0f - s));
    }
    dgu[base] = pack8(dg);
    dgu[base + 16] = pack8(du);
  }
}

__global__ void dequant_fp8_kernel(const uint2* __restrict__ q, const float* __restrict__ scales, uint4* __restrict__ out, long long rows, int H,
                                   const int* __restrict__ rows_dev) {
  if (rows_dev) rows = min(rows, static_cast<long long>(*rows_dev));
  const int cpr = H / 8;
  const long long total = rows * cpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cpr;
    const int c = static_cast<int>(i % cpr);
    const float sc = scales[r * (H / 128) + c / 16];
    const uint2 v = q[i];
    const unsigned char* b = reinterpret_cast<const unsigned char*>(&v);
    float f[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const __half_raw h = __nv_cvt_fp8_to_halfraw(b[k], __NV_E4M3);
      f[k] = __half2float(*reinterpret_cast<const __half*>(&h)) * sc;
    }
    out[i] = pack8(f);
  }
}

// One thread owns groups of 4 consecutive parameters: its fp32 accesses are 16 bytes, contiguous across the warp
// (512 bytes per instruction), its bf16 accesses 8 bytes. Two groups are in flight per iteration. Nothing is read
// twice, so every access is marked streaming (evict first).
__global__ void adamw_kernel(uint2* __restrict__ param, float4* __restrict__ master, float4* __restrict__ m, float4* __restrict__ v,
                             const uint2* __restrict__ grad, long long n4, float lr, float b1, float b2, float eps, float wd, float c1, float c2,
                             float gscale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int U = 2;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < n4; i0 += U * stride) {
    float4 w[U], mm[U], vv[U];
    uint2 g[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < n4) { g[u] = __ldcs(grad + i); w[u] = __ldcs(master + i); mm[u] = __ldcs(m + i); vv[u] = __ldcs(v + i); }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n4) break;
      const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g[u].x));
      const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g[u].y));
      const float gk[4] = {g01.x * gscale, g01.y * gscale, g23.x * gscale, g23.y * gscale};
      float* wp = reinterpret_cast<float*>(&w[u]);
      float* mp = reinterpret_cast<float*>(&mm[u]);
      float* vp = reinterpret_cast<float*>(&vv[u]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        mp[k] = b1 * mp[k] + (1.0f - b1) * gk[k];
        vp[k] = b2 * vp[k] + (1.0f - b2) * gk[k] * gk[k];
        const float upd = (mp[k] * c1) / (sqrtf(vp[k] * c2) + eps);
        wp[k] = wp[k] - lr * (upd + wd * wp[k]);
      }
      __stcs(master + i, w[u]);
      __stcs(m + i, mm[u]);
      __stcs(v + i, vv[u]);
      uint2 pb;
      *reinterpret_cast<__nv_bfloat162*>(&pb.x) = __floats2bfloat162_rn(wp[0], wp[1]);
      *reinterpret_cast<__nv_bfloat162*>(&pb.y) = __floats2bfloat162_rn(wp[2], wp[3]);
      __stcs(param + i, pb);
    }
  }
}

// sum((a + b)^2) over n8 chunks of 8 bf16: per-block partial sums, then one block folds them in a
// fixed order (deterministic).
__global__ void sumsq_add_partial_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, long long n8, float* __restrict__ partial) {
  float acc = 0.0f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    unpack8(a[i], x);
    unpack8(b[i], y);
#pragma unroll
    for (int k = 0; k < 8; ++k) { const float o = __bfloat162float(__float2bfloat16_rn(x[k] + y[k])); acc = fmaf(o, o, acc); }
  }
  __shared__ float s[32];
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) partial[blockIdx.x] = v;
  }
}
__global__ void fold_partials_kernel(const float* __restrict__ partial, int n, float scale, float* __restrict__ out) {
  __shared__ float s[32];
  float acc = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) *out = v * scale;
  }
}
// grad = (a + b) * (*gscale) * factor, as bf16.
__global__ void scaled_sum_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, long long n8, const float* __restrict__ gscale, float factor,
                                  uint4* __restrict__ out) {
  const float g = (*gscale) * factor;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8], y[8], o[8];
    unpack8(a[i], x);
    unpack8(b[i], y);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = __bfloat162float(__float2bfloat16_rn(x[k] + y[k])) * g;
    out[i] = pack8(o);
  }
}

// Embedding gradient: ids sorted ascending with their original positions; the warp that sits on the
// first entry of a run of equal ids sums the run's rows in fp32 (in position order) and writes one
// bf16 row of the table gradient.
__global__ void embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ perm, const uint4* __restrict__ grad_out,
                                     uint4* __restrict__ grad_table, long long T, int H) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= T) return;
  const long long id = sorted_ids[i];
  if (id < 0) return;  // slots no valid id was sorted into
  if (i > 0 && sorted_ids[i - 1] == id) return;
  long long end = i + 1;
  while (end < T && sorted_ids[end] == id) ++end;
  const int chunks = H / 8;
  for (int c = lane; c < chunks; c += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long j = i; j < end; ++j) {
      float f[8];
      unpack8(grad_out[perm[j] * chunks + c], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f[k];
    }
    grad_table[id * chunks + c] = pack8(acc);
  }
}

// ---- ids grouped by value, positions in order: a counting sort the embedding gradient is fed from -----------
// Work is independent of the data (heavy duplicates cost the same as none). Blocks of kIdxBlock tokens:
//   1. per-block histogram of the ids (counts) and, per token, its rank among the block's earlier tokens with
//      the same id (position order, so the grouping is stable and the later summation order is fixed);
//   2. per id, the running sum over blocks (where a block's tokens of that id start inside the id's run);
//   3. exclusive scan over the ids (where each id's run starts);
//   4. scatter: sorted_ids / perm, the arrays embedding_bwd_kernel consumes.
constexpr int kIdxBlock = 256;

__global__ void __launch_bounds__(kIdxBlock) emb_block_hist_kernel(const long long* __restrict__ ids, long long T, int V, int* __restrict__ hist,
                                                                   int* __restrict__ rank_in_block) {
  __shared__ long long s_id[kIdxBlock];
  const long long p = blockIdx.x * static_cast<long long>(kIdxBlock) + threadIdx.x;
  long long id = -1;
  if (p < T) { id = ids[p]; if (id < 0 || id >= V) id = -1; }  // out-of-range ids take no part (F.embedding would have refused them)
  s_id[threadIdx.x] = id;
  __syncthreads();
  if (id < 0) { if (p < T) rank_in_block[p] = -1; return; }
  int r = 0;
  for (int j = 0; j < static_cast<int>(threadIdx.x); ++j) r += s_id[j] == id ? 1 : 0;
  rank_in_block[p] = r;
  atomicAdd(hist + static_cast<long long>(blockIdx.x) * V + id, 1);
}

__global__ void emb_scan_blocks_kernel(int* __restrict__ hist, int blocks, int V, int* __restrict__ total) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= V) return;
  int run = 0;
  // Eight independent loads in flight per round (the running sum is the only serial part).
  for (int b0 = 0; b0 < blocks; b0 += 8) {
    int c[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) c[u] = b0 + u < blocks ? hist[static_cast<long long>(b0 + u) * V + v] : 0;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (b0 + u < blocks) { hist[static_cast<long long>(b0 + u) * V + v] = run; run += c[u]; }  // counts become offsets inside the id's run
  }
  total[v] = run;
}

// Single block: start[v] = sum of total[< v]; start[V] = number of tokens that took part. Four ids per thread and pass.
__global__ void __launch_bounds__(1024) emb_scan_ids_kernel(const int* __restrict__ total, int V, int* __restrict__ start) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int v0 = 0; v0 < V; v0 += 4096) {
    const int v = v0 + 4 * threadIdx.x;
    int x[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) x[u] = v + u < V ? total[v + u] : 0;
    const int mine = x[0] + x[1] + x[2] + x[3];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += y; }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += y; }
      s_warp[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    int before = s_carry + (warp ? s_warp[warp - 1] : 0) + incl - mine;
#pragma unroll
    for (int u = 0; u < 4; ++u) { if (v + u < V) start[v + u] = before; before += x[u]; }
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = before;
    __syncthreads();
  }
  if (threadIdx.x == 0) start[V] = s_carry;
}

__global__ void emb_scatter_kernel(const long long* __restrict__ ids, const int* __restrict__ rank_in_block, const int* __restrict__ hist,
                                   const int* __restrict__ start, long long T, int V, long long* __restrict__ sorted_ids, long long* __restrict__ perm) {
  const long long p = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (p >= T) return;
  const int r = rank_in_block[p];
  if (r < 0) return;
  const long long id = ids[p];
  const long long slot = start[id] + hist[(p / kIdxBlock) * V + id] + r;
  sorted_ids[slot] = id;
  perm[slot] = p;
}

int grid_for(long long items) { return static_cast<int>(std::min<long long>((items + 255) / 256, 148 * 8)); }

}  // namespace

cudaError_t launch_swiglu_fwd(const __nv_bfloat16* gate_up, __nv_bfloat16* act, long long rows, int inter, cudaStream_t stream) {
  if (inter % 128) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  swiglu_fwd_kernel<<<grid_for(rows * inter / 8), 256, 0, stream>>>(reinterpret_cast<const uint4*>(gate_up), reinterpret_cast<uint4*>(act), rows, inter);
  note_launch();
  return cudaGetLastError();
}
cudaError_t launch_swiglu_bwd(const __nv_bfloat16* gate_up, const __nv_bfloat16* d_act, __nv_bfloat16* d_gate_up, long long rows, int inter,
                              const int* rows_dev, cudaStream_t stream) {
  if (inter % 128) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  swiglu_bwd_kernel<<<grid_for(rows * inter / 8), 256, 0, stream>>>(reinterpret_cast<const uint4*>(gate_up), reinterpret_cast<const uint4*>(d_act),
                                                                  reinterpret_cast<uint4*>(d_gate_up), rows, inter, rows_dev);
  note_launch();
  return cudaGetLastError();
}
cudaError_t launch_sumsq_add(const __nv_bfloat16* a, const __nv_bfloat16* b, long long n, float scale, float* partial, int partial_len, float* out,
                             cudaStream_t stream) {
  if (n % 8 || partial_len < 1) return cudaErrorInvalidValue;
  const int blocks = std::min(partial_len, grid_for(n / 8));
  sumsq_add_partial_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(a), reinterpret_cast<const uint4*>(b), n / 8, partial);
  fold_partials_kernel<<<1, 1024, 0, stream>>>(partial, blocks, scale, out);
  note_launch(2);
  return cudaGetLastError();
}
cudaError_t launch_scaled_sum(const __nv_bfloat16* a, const __nv_bfloat16* b, long long n, const float* gscale, float factor, __nv_bfloat16* out,
                              cudaStream_t stream) {
  if (n % 8) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  scaled_sum_kernel<<<grid_for(n / 8), 256, 0, stream>>>(reinterpret_cast<const uint4*>(a), reinterpret_cast<const uint4*>(b), n / 8, gscale, factor,
                                                       reinterpret_cast<uint4*>(out));
  note_launch();
  return cudaGetLastError();
}
cudaError_t launch_embedding_bwd(const long long* sorted_ids, const long long* perm, const __nv_bfloat16* grad_out, __nv_bfloat16* grad_table, long long T,
                                 int H, cudaStream_t stream) {
  if (H % 8) return cudaErrorInvalidValue;
  if (T == 0) return cudaSuccess;
  const long long threads = T * 32;
  embedding_bwd_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(sorted_ids, perm, reinterpret_cast<const uint4*>(grad_out),
                                                                                      reinterpret_cast<uint4*>(grad_table), T, H);
  note_launch();
  return cudaGetLastError();
}
cudaError_t launch_embedding_index(const long long* ids, long long T, int V, int* hist, int* rank_in_block, int* total, int* start, long long* sorted_ids,
                                   long long* perm, cudaStream_t stream) {
  if (T <= 0 || V <= 0) return cudaErrorInvalidValue;
  const int blocks = static_cast<int>((T + kIdxBlock - 1) / kIdxBlock);
  cudaError_t e = cudaMemsetAsync(hist, 0, sizeof(int) * static_cast<size_t>(blocks) * V, stream);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(sorted_ids, 0xFF, sizeof(long long) * static_cast<size_t>(T), stream);  // -1: slots that stay unused are skipped downstream
  if (e != cudaSuccess) return e;
  emb_block_hist_kernel<<<blocks, kIdxBlock, 0, stream>>>(ids, T, V, hist, rank_in_block);
  emb_scan_blocks_kernel<<<(V + 255) / 256, 256, 0, stream>>>(hist, blocks, V, total);
  emb_scan_ids_kernel<<<1, 1024, 0, stream>>>(total, V, start);
  emb_scatter_kernel<<<blocks, kIdxBlock, 0, stream>>>(ids, rank_in_block, hist, start, T, V, sorted_ids, perm);
  note_launch(4);
  return cudaGetLastError();
}
int embedding_index_block() { return kIdxBlock; }
cudaError_t launch_dequant_fp8(const unsigned char* q, const float* scales, __nv_bfloat16* out, long long rows, int H, const int* rows_dev,
                               cudaStream_t stream) {
  if (H % 128) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  dequant_fp8_kernel<<<grid_for(rows * H / 8), 256, 0, stream>>>(reinterpret_cast<const uint2*>(q), scales, reinterpret_cast<uint4*>(out), rows, H, rows_dev);
  note_launch();
  return cudaGetLastError();
}
cudaError_t launch_adamw(__nv_bfloat16* param, float* master, float* m, float* v, const __nv_bfloat16* grad, long long n, float lr, float beta1,
                         float beta2, float eps, float weight_decay, float bias_c1, float bias_c2, float grad_scale, cudaStream_t stream) {
  if (n % 8) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  adamw_kernel<<<grid_for(n / 8), 256, 0, stream>>>(reinterpret_cast<uint2*>(param), reinterpret_cast<float4*>(master), reinterpret_cast<float4*>(m),
                                                    reinterpret_cast<float4*>(v), reinterpret_cast<const uint2*>(grad), n / 4, lr, beta1, beta2, eps,
                                                    weight_decay, bias_c1, bias_c2, grad_scale);
  note_launch();
  return cudaGetLastError();
}

}  // namespace fastb
