// Router front end fused into one pass over the activations:
//   norm_gate_route : RMSNorm(h) -> hn, router logits hn . gate^T, softmax-over-top-k weights, the
//                     expert choice and the per-block histogram / stable ranks that the split scan
//                     consumes (what route_topk produces from ready-made logits);
//   norm_gate_bwd   : the matching backward: gradients of the selected logits from the weight
//                     gradients, d(hn) = grad of the MoE input + sum_j dlogit_j * gate[e_j], the gate
//                     and norm-weight gradients (block partials in shared memory, then fp32 atomics)
//                     and the RMSNorm backward to d(h).
// The reference has no router; in a stock stack these are a layer-norm kernel, a small library
// GEMM, top-k, gather, softmax and their backward kernels with the activations re-read each time.
// Limits: num_experts <= 32 (one logit per lane), hidden % 256 == 0, and the gate matrix (forward)
// or the gate matrix plus the fp32 gradient accumulators (backward) must fit in shared memory.
#include "api.h"

namespace fastb {

namespace {

constexpr int kTokensPerBlock = kRouteTokensPerBlock;
constexpr int kGateThreads = 512;  // forward: 16 warps per block, two tokens per warp and pass
constexpr int kGateBwdThreads = 512;            // backward: 16 warps hide the shared-memory and reduction latency of the per-token chain
constexpr int kGateBwdMaxChunksPerThread = 2;  // backward: hidden <= 2 * 512 * 8 = 8192

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
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Dynamic shared memory: gate [E][H] bf16, norm weight [H] bf16, then int s_eid[kTokensPerBlock * K].
// A warp takes two tokens per pass: every gate chunk is read and unpacked once for both rows.
template <int EMAX>
__global__ void __launch_bounds__(kGateThreads) norm_gate_route_kernel(const NormGateArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int E = a.num_experts, H = a.H, K = a.K;
  uint4* s_gate = reinterpret_cast<uint4*>(smem);                            // [E][H / 8]
  uint4* s_nw = s_gate + static_cast<size_t>(E) * (H / 8);                  // [H / 8]
  int* s_eid = reinterpret_cast<int*>(s_nw + H / 8);                        // [kTokensPerBlock * K]
  const int chunks = H / 8;
  for (int i = threadIdx.x; i < E * chunks; i += blockDim.x) s_gate[i] = __ldg(reinterpret_cast<const uint4*>(a.gate) + i);
  for (int i = threadIdx.x; i < chunks; i += blockDim.x) s_nw[i] = __ldg(reinterpret_cast<const uint4*>(a.norm_w) + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kGateThreads / 32;
  const int t0 = blockIdx.x * kTokensPerBlock;
  const int nt = min(kTokensPerBlock, a.T - t0);
  // Logits of one token are spread over the lanes' partial sums: reduce, publish, choose the top k.
  auto finish = [&](int lt, const float (&acc)[EMAX]) {
    const int t = t0 + lt;
    float raw = -INFINITY;  // lane e ends up with logit e
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      if (e >= E) break;
      const float v = warp_sum(acc[e]);
      if (lane == e) raw = v;
    }
    if (lane < E) a.logits[static_cast<long long>(t) * E + lane] = raw;
    if (raw != raw) raw = -INFINITY;  // NaN counts as -inf: the selection stays total
    float sel = lane < E ? raw + (a.bias ? a.bias[lane] : 0.0f) : -INFINITY;
    if (sel != sel) sel = -INFINITY;
    float mx = raw;
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    bool taken = lane >= E;
    float wsum = 0.0f, my_w = 0.0f;
    int my_e = -1;
    for (int j = 0; j < K; ++j) {
      float best = taken ? -INFINITY : sel;
      int best_e = taken ? 0x7fffffff : lane;
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; }
      }
      if (lane == best_e) taken = true;
      const float r = __shfl_sync(0xffffffffu, raw, best_e & 31);
      const float pw = r > -INFINITY ? __expf(r - mx) : 0.0f;
      wsum += pw;
      if (lane == j) { my_w = pw; my_e = best_e; }
    }
    if (lane < K) {
      a.topk_idx[static_cast<long long>(t) * K + lane] = my_e;
      a.topk_w[static_cast<long long>(t) * K + lane] = wsum > 0.0f ? my_w / wsum : 0.0f;
      s_eid[lt * K + lane] = my_e;
    }
  };
  for (int lt = warp; lt < kTokensPerBlock; lt += 2 * nwarps) {
    const int ltb = lt + nwarps;
    const bool va = lt < nt, vb = ltb < nt;   // vb implies va
    if (!vb)
      for (int j = lane; j < K; j += 32) s_eid[ltb * K + j] = -1;
    if (!va) {
      for (int j = lane; j < K; j += 32) s_eid[lt * K + j] = -1;
      continue;
    }
    const uint4* ha = reinterpret_cast<const uint4*>(a.h + static_cast<long long>(t0 + lt) * H);
    const uint4* hb = reinterpret_cast<const uint4*>(a.h + static_cast<long long>(t0 + (vb ? ltb : lt)) * H);  // a dead second token re-reads the first
    float ssa = 0.0f, ssb = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      float fa[8], fb[8];
      unpack8(__ldg(ha + c), fa);
      unpack8(__ldg(hb + c), fb);
#pragma unroll
      for (int i = 0; i < 8; ++i) { ssa = fmaf(fa[i], fa[i], ssa); ssb = fmaf(fb[i], fb[i], ssb); }
    }
    ssa = warp_sum(ssa);
    ssb = warp_sum(ssb);
    const float ra = rsqrtf(ssa / static_cast<float>(H) + a.eps), rb = rsqrtf(ssb / static_cast<float>(H) + a.eps);
    if (lane == 0) { a.rstd[t0 + lt] = ra; if (vb) a.rstd[t0 + ltb] = rb; }
    // second pass over the rows (still in L1): normalised rows out, logits accumulated against the gate rows
    float acca[EMAX], accb[EMAX];
#pragma unroll
    for (int e = 0; e < EMAX; ++e) { acca[e] = 0.0f; accb[e] = 0.0f; }
    uint4* oa = reinterpret_cast<uint4*>(a.hn + static_cast<long long>(t0 + lt) * H);
    uint4* ob = reinterpret_cast<uint4*>(a.hn + static_cast<long long>(t0 + ltb) * H);
    for (int c = lane; c < chunks; c += 32) {
      float fa[8], fb[8], w[8], ya[8], yb[8];
      unpack8(__ldg(ha + c), fa);
      unpack8(__ldg(hb + c), fb);
      unpack8(s_nw[c], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) { ya[i] = bf16_round(fa[i] * ra * w[i]); yb[i] = bf16_round(fb[i] * rb * w[i]); }  // normalised and scaled in fp32, rounded once
      oa[c] = pack8(ya);
      if (vb) ob[c] = pack8(yb);
#pragma unroll
      for (int e = 0; e < EMAX; ++e) {
        if (e >= E) break;
        float g[8];
        unpack8(s_gate[static_cast<size_t>(e) * chunks + c], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) { acca[e] = fmaf(ya[i], g[i], acca[e]); accb[e] = fmaf(yb[i], g[i], accb[e]); }
      }
    }
    finish(lt, acca);
    if (vb) finish(ltb, accb);
  }
  __syncthreads();
  const int n = kTokensPerBlock * K;
  for (int e = threadIdx.x; e < E; e += kGateThreads) {
    int c = 0;
    for (int i = 0; i < n; ++i)
      if (s_eid[i] == e) {
        a.slot_in_block[static_cast<long long>(t0) * K + i] = c;
        ++c;
      }
    a.block_cnt[static_cast<long long>(blockIdx.x) * E + e] = c;
  }
}

// Dynamic shared memory: gate [E][H] bf16, norm weight [H] bf16, then fp32 accumulators d_gate [E][H], d_nw [H].
// The block walks its tokens one after another and every thread owns the same 16-byte column chunks for all
// of them, so the gradient partials in shared memory are updated with plain read-modify-writes (no two
// threads ever touch the same word); the row-wide sum the RMSNorm backward needs is one block reduction per
// token.
__global__ void __launch_bounds__(kGateBwdThreads) norm_gate_bwd_kernel(const NormGateBwdArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float s_part[2][kGateBwdThreads / 32];
  const int E = a.num_experts, H = a.H, K = a.K;
  const int chunks = H / 8;
  uint4* s_gate = reinterpret_cast<uint4*>(smem);
  uint4* s_nw = s_gate + static_cast<size_t>(E) * chunks;
  float* s_dgate = reinterpret_cast<float*>(s_nw + chunks);  // [E][H]
  float* s_dnw = s_dgate + static_cast<size_t>(E) * H;       // [H]
  for (int i = threadIdx.x; i < E * chunks; i += blockDim.x) s_gate[i] = __ldg(reinterpret_cast<const uint4*>(a.gate) + i);
  for (int i = threadIdx.x; i < chunks; i += blockDim.x) s_nw[i] = __ldg(reinterpret_cast<const uint4*>(a.norm_w) + i);
  for (int i = threadIdx.x; i < (E + 1) * H; i += blockDim.x) s_dgate[i] = 0.0f;  // d_gate and d_nw are contiguous
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One block per SM, each with an equal share of the tokens (no second, partly filled wave).
  const int per = (a.T + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int t0 = blockIdx.x * per;
  const int nt = max(0, min(per, a.T - t0));
  constexpr int kMaxK = 8;
  constexpr int kMaxC = kGateBwdMaxChunksPerThread;  // my chunks are threadIdx.x + kGateBwdThreads * i, i < nc <= kMaxC
  const int nc = (chunks - static_cast<int>(threadIdx.x) + kGateBwdThreads - 1) / kGateBwdThreads;
  // The next token's rows are requested before the current token is worked on, and a token's rows stay in
  // registers for both passes: no global-memory latency sits between two block reductions.
  uint4 nx[kMaxC], ng[kMaxC];
  auto request = [&](int lt) {
    const uint4* hrow = reinterpret_cast<const uint4*>(a.h + static_cast<long long>(t0 + lt) * H);
    const uint4* grow = reinterpret_cast<const uint4*>(a.grad_hn + static_cast<long long>(t0 + lt) * H);
#pragma unroll
    for (int i = 0; i < kMaxC; ++i)
      if (i < nc) { nx[i] = __ldg(hrow + threadIdx.x + kGateBwdThreads * i); ng[i] = __ldg(grow + threadIdx.x + kGateBwdThreads * i); }
  };
  if (nt > 0) request(0);
  for (int lt = 0; lt < nt; ++lt) {
    const int t = t0 + lt;
    uint4 cx[kMaxC], cg[kMaxC];
#pragma unroll
    for (int i = 0; i < kMaxC; ++i) { cx[i] = nx[i]; cg[i] = ng[i]; }
    if (lt + 1 < nt) request(lt + 1);
    // gradients of the selected logits: w = softmax(l_sel)  =>  dl_j = w_j (gw_j - sum_i w_i gw_i)
    float dl[kMaxK];
    int ex[kMaxK];
    float dotw = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) {
      dl[j] = 0.0f; ex[j] = 0;
      if (j < K) {
        const long long tj = static_cast<long long>(t) * K + j;
        ex[j] = __ldg(a.topk_idx + tj);
        dotw = fmaf(__ldg(a.topk_w + tj), __ldg(a.grad_w + tj), dotw);
      }
    }
#pragma unroll
    for (int j = 0; j < kMaxK; ++j)
      if (j < K) {
        const long long tj = static_cast<long long>(t) * K + j;
        const bool in_range = ex[j] >= 0 && ex[j] < E;
        dl[j] = in_range ? __ldg(a.topk_w + tj) * (__ldg(a.grad_w + tj) - dotw) : 0.0f;
        if (!in_range) ex[j] = 0;
      }
    const float rstd = __ldg(a.rstd + t);
    // pass 1 over my chunks: s = sum(dxhat * xhat), the gate / norm-weight gradient partials; keeps xhat and
    // dxhat = d(hn) * w of my chunks for pass 2
    float s = 0.0f;
    float kxh[kMaxC][8], kdx[kMaxC][8];
#pragma unroll
    for (int ci = 0; ci < kMaxC; ++ci) {
      if (ci >= nc) break;
      const int c = threadIdx.x + kGateBwdThreads * ci;
      float x[8], w[8], g[8], hn[8];
      unpack8(cx[ci], x);
      unpack8(s_nw[c], w);
      unpack8(cg[ci], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) { kxh[ci][i] = x[i] * rstd; hn[i] = bf16_round(kxh[ci][i] * w[i]); }  // hn as the forward pass rounded it
#pragma unroll
      for (int j = 0; j < kMaxK; ++j)
        if (j < K) {
          float q[8];
          unpack8(s_gate[static_cast<size_t>(ex[j]) * chunks + c], q);
          // a chunk's first four accumulators sit in the row's first half, the other four in its second
          // half: a warp's 16-byte accesses are then contiguous (no two-way bank conflict)
          float4* dg = reinterpret_cast<float4*>(s_dgate + static_cast<size_t>(ex[j]) * H) + c;
          float4 d0 = dg[0], d1 = dg[chunks];
          d0.x = fmaf(dl[j], hn[0], d0.x); d0.y = fmaf(dl[j], hn[1], d0.y); d0.z = fmaf(dl[j], hn[2], d0.z); d0.w = fmaf(dl[j], hn[3], d0.w);
          d1.x = fmaf(dl[j], hn[4], d1.x); d1.y = fmaf(dl[j], hn[5], d1.y); d1.z = fmaf(dl[j], hn[6], d1.z); d1.w = fmaf(dl[j], hn[7], d1.w);
          dg[0] = d0; dg[chunks] = d1;
#pragma unroll
          for (int i = 0; i < 8; ++i) g[i] = fmaf(dl[j], q[i], g[i]);
        }
      float4* dn = reinterpret_cast<float4*>(s_dnw) + c;
      float4 n0 = dn[0], n1 = dn[chunks];
      n0.x = fmaf(g[0], kxh[ci][0], n0.x); n0.y = fmaf(g[1], kxh[ci][1], n0.y); n0.z = fmaf(g[2], kxh[ci][2], n0.z); n0.w = fmaf(g[3], kxh[ci][3], n0.w);
      n1.x = fmaf(g[4], kxh[ci][4], n1.x); n1.y = fmaf(g[5], kxh[ci][5], n1.y); n1.z = fmaf(g[6], kxh[ci][6], n1.z); n1.w = fmaf(g[7], kxh[ci][7], n1.w);
      dn[0] = n0; dn[chunks] = n1;
#pragma unroll
      for (int i = 0; i < 8; ++i) { kdx[ci][i] = g[i] * w[i]; s = fmaf(kdx[ci][i], kxh[ci][i], s); }
    }
    s = warp_sum(s);
    if (lane == 0) s_part[lt & 1][warp] = s;   // two buffers: the next token's partials never overwrite sums still being read
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kGateBwdThreads / 32; ++i) tot += s_part[lt & 1][i];
    tot /= static_cast<float>(H);
    // pass 2, from registers: d(h) = rstd * (dxhat - xhat * s)
    uint4* orow = reinterpret_cast<uint4*>(a.grad_h + static_cast<long long>(t) * H);
#pragma unroll
    for (int ci = 0; ci < kMaxC; ++ci) {
      if (ci >= nc) break;
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rstd * (kdx[ci][i] - kxh[ci][i] * tot);
      orow[threadIdx.x + kGateBwdThreads * ci] = pack8(o);
    }
  }
  __syncthreads();
  // rows of d_gate and d_nw are contiguous ((E + 1) rows of H); undo the half-row split on the way out
  for (int i = threadIdx.x; i < (E + 1) * H; i += blockDim.x) {
    const int row = i / H, p = i % H;                      // p: position in shared memory
    const int half = p / (H / 2), q = p % (H / 2);          // accumulator (q % 4) + 4 * half of chunk q / 4
    const int col = (q / 4) * 8 + half * 4 + (q % 4);
    const float v = s_dgate[i];
    if (v != 0.0f) atomicAdd((row < E ? a.d_gate + static_cast<size_t>(row) * H : a.d_norm_w) + col, v);
  }
}

}  // namespace

size_t norm_gate_smem_bytes(int E, int H, int K, bool backward) {
  const size_t base = (static_cast<size_t>(E) + 1) * H * 2;
  return backward ? base + (static_cast<size_t>(E) + 1) * H * 4 : base + sizeof(int) * kTokensPerBlock * K;
}

cudaError_t launch_norm_gate_route(const NormGateArgs& a, cudaStream_t stream) {
  if (a.num_experts < 1 || a.num_experts > 32 || a.K < 1 || a.K > a.num_experts || a.K > 32 || a.H % 256) return cudaErrorInvalidValue;
  const size_t smem = norm_gate_smem_bytes(a.num_experts, a.H, a.K, false);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  const int blocks = (a.T + kTokensPerBlock - 1) / kTokensPerBlock;
  if (blocks == 0) return cudaSuccess;
  auto go = [&](auto kern) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    kern<<<blocks, kGateThreads, smem, stream>>>(a);
    note_launch();
    return cudaGetLastError();
  };
  if (a.num_experts <= 8) return go(norm_gate_route_kernel<8>);
  if (a.num_experts <= 16) return go(norm_gate_route_kernel<16>);
  return go(norm_gate_route_kernel<32>);
}

cudaError_t launch_norm_gate_bwd(const NormGateBwdArgs& a, cudaStream_t stream) {
  if (a.num_experts < 1 || a.num_experts > 32 || a.K < 1 || a.K > 8 || a.H % 256 || a.H > kGateBwdMaxChunksPerThread * kGateBwdThreads * 8) return cudaErrorInvalidValue;
  const size_t smem = norm_gate_smem_bytes(a.num_experts, a.H, a.K, true);
  if (smem > 220 * 1024) return cudaErrorInvalidValue;
  if (a.T <= 0) return cudaSuccess;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  const int blocks = std::max(1, std::min(sms, (a.T + 31) / 32));  // at least 32 tokens per block: each block adds its partial sums to global memory once
  e = cudaFuncSetAttribute(norm_gate_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  norm_gate_bwd_kernel<<<blocks, kGateBwdThreads, smem, stream>>>(a);
  note_launch();
  return cudaGetLastError();
}

}  // namespace fastb
