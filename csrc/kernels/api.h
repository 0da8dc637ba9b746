// C launch surface of the sm_100a kernels (no torch types; raw pointers + stream).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../runtime/device_sync.cuh"

namespace fastb {

// Number of kernels this library has launched in this process (for bench accounting).
unsigned long long launch_count();
void note_launch(int n = 1);

// ---------------------------------------------------------------------------------------------
// a2a_push: executes one rank's work list of a staged / fan-out all-to-all(v) plan.
// ---------------------------------------------------------------------------------------------
struct A2AWork {
  long long src_off, dst_off, bytes;
  int dst_rank;
  unsigned char src_buf, dst_buf, wait_kind, signal_kind;
  int stage, wait_stage;
  int pad_;
};
static_assert(sizeof(A2AWork) == 48, "A2AWork layout is shared with the host packer");

constexpr int kSigReadyOff = 0;      // u64 ready[world]   (written by peers: their current epoch)
// Peers one signal block has room for. A launch on a larger world is refused by the binding; planning, lowering and
// the host executors have no such limit (beyond 64 ranks a communicator plans one-rank views of a plan).
constexpr int kSigMaxWorld = 64;
constexpr int kSigCounterOff = kSigMaxWorld;  // u64 counters: [0] balance, [1] output, [2+k] rail stage k
constexpr int kSigMaxStages = 4096;
constexpr int kSigTicketOff = kSigCounterOff + 2 + kSigMaxStages;  // u64 CTA exit ticket
constexpr int kSigWords = kSigTicketOff + 2;

struct A2ARankArgs {
  const A2AWork* items;
  int n_items, rank, world, num_stages;
  void* const* peer_table;               // [world] slab bases (device array)
  const unsigned char* src_base[4];      // local bases of input / output / balance / rail
  long long dst_heap_off[4];             // slab offsets of the same four buffers on every rank
  long long sig_heap_off;                // slab offset of the signal block (kSigWords u64)
  unsigned long long epoch;              // 1, 2, 3, ... per collective on this communicator
  unsigned long long expect_output, expect_balance;
  const unsigned long long* expect_rail; // [num_stages] bytes landing in my rail staging
  DeviceStatus* status;
  unsigned long long timeout_ns;
  // Optional, device u64[10] of globaltimer stamps: [0] kernel start, [1 + 2 p] / [2 + 2 p] first start /
  // last end of the work items of phase p (0 balance, 1 rail, 2 redistribute, 3 direct), [9] end. The caller
  // presets start slots ([0] and odd slots) to all ones and the others to zero.
  unsigned long long* phase_stamps;
  // 1: pieces whose pointers and size are multiples of 16 bytes are moved by one thread per CTA with bulk
  // copies through shared memory (local load, then store to the peer) instead of by every thread with
  // loads and stores. Real ranks only (the in-process group launch keeps the load/store loop).
  int bulk;
};
constexpr int kPhaseStampWords = 10;

// device_args == nullptr: one real rank, `host_args` is passed by value. Otherwise one cooperative
// launch with gridDim.y = virtual_ranks runs every rank of an in-process group (single-GPU
// emulation); `device_args` points to an array of virtual_ranks structs in device memory.
// needs_coresidency (real ranks): the work list has items that wait for other items of the same launch; the kernel is
// then launched cooperatively so that its whole grid is resident at once.
cudaError_t launch_a2a_push(const A2ARankArgs* host_args, const A2ARankArgs* device_args, int virtual_ranks, int ctas,
                            int threads, cudaStream_t stream, bool needs_coresidency = false);

// Waits (bounded) on a flag nothing sets; used to test the timeout path without any peer.
cudaError_t launch_wait_probe(const unsigned long long* flag, unsigned long long want, DeviceStatus* status,
                              unsigned long long timeout_ns, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// grouped_gemm: tcgen05 / TMEM grouped bf16 GEMM (forward, dgrad, wgrad) with optional SwiGLU.
// ---------------------------------------------------------------------------------------------
enum class GemmMode : int { kForward = 0, kDgrad = 1, kWgrad = 2 };
enum class GemmEpilogue : int {
  kStore = 0,
  kSwiGLU = 1,     // forward: out = silu(gate) * up (+ optional raw gate|up tile)
  kSwiGLUBwd = 2,  // dgrad of the second projection: the tile is d(act); c2 holds the saved gate|up tiles and c
                   // receives d(gate|up) in the same layout (CTA-pair kernel only)
};

struct GemmArgs {
  const int* group_off;    // [num_groups + 1] row offsets of the groups, multiples of 128 (device)
  int num_groups;
  int tiles_n;             // tiles along the output columns (columns / 256)
  int fixed_m_tiles;       // wgrad only: tiles along the output rows of one group (rows / 128)
  int red_len;             // forward / dgrad: reduction length (multiple of 64)
  int b_rows_per_group;    // rows of one group's slice in operand B's matrix (forward: N, dgrad: N)
  int c_rows_per_group;    // wgrad only: output rows per group
  __nv_bfloat16* c;        // output; SwiGLU: activations [rows, columns / 2]
  long long ldc;
  __nv_bfloat16* c2;       // SwiGLU only, optional: raw gate|up tile output [rows, columns]
  long long ldc2;
  DeviceStatus* status;
  unsigned long long timeout_ns;
  // Optional arrival gate: before the first load of group g the TMA producer waits until
  // gate_counter[g] >= gate_target[g] (rows pushed by peers have landed). Null = no gate.
  const unsigned long long* gate_counter;
  const unsigned long long* gate_target;
  int band_rows;           // rows of a raster band (0 = default 4096): tiles are visited band by band, all columns per band
  int direct_epilogue;     // CTA-pair kernel: 1 = epilogue threads access global memory row by row instead of staging tiles for TMA
  // CTA-pair kernel, forward only: operand A is e4m3 (map_a: u8 matrix, boxes {64,128}, no swizzle) with one fp32 scale per
  // 128 elements of a row in a_scales [rows, red_len / 128]; null = bf16 operand.
  const float* a_scales;
  const int* group_rows;   // optional [num_groups]: real rows of each group; the e4m3 feed turns rows past them into zeros
  int gate_tile_rows;      // 0: gate_counter / gate_target are indexed by group; > 0: by (row of the grouped matrix) / gate_tile_rows
  int gate_slots;          // entries of gate_counter / gate_target (indices are clamped to the last one)
};

int grouped_gemm_smem_bytes();
// Tensor maps (bf16, 128-byte swizzle) must use these boxes: forward A {64,128} B {64,256};
// dgrad A {64,128} B {64,64}; wgrad A {64,64} B {64,64}  ({inner, outer} elements).
cudaError_t launch_grouped_gemm(GemmMode mode, GemmEpilogue epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& args,
                                int ctas, cudaStream_t stream);
// CTA-pair variant (256 x 256 tiles, cta_group::2). Group offsets must be multiples of 256,
// fixed_m_tiles counts 256-row tiles, and operand B's boxes are forward {64,128}; dgrad / wgrad
// boxes are as above. Outputs leave through TMA stores: map_c describes args.c and map_c2
// (null exactly when args.c2 is null) describes args.c2, both with boxes {64,128}; for the fused
// SwiGLU backward map_c2 is the saved gate|up matrix, which the epilogue TMA-loads.
cudaError_t launch_grouped_gemm_pair(GemmMode mode, GemmEpilogue epi, const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c,
                                     const CUtensorMap* map_c2, const GemmArgs& args, int ctas, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// MoE routing / dispatch / combine
// ---------------------------------------------------------------------------------------------
cudaError_t launch_route_topk(const float* logits, const float* bias, int T, int E, int K, int* topk_idx, float* topk_w, int* slot_in_block,
                              int* block_cnt, cudaStream_t stream);
constexpr int kRouteTokensPerBlock = 128;  // tokens per routing block (block_cnt / block_base granularity)

struct SplitsArgs {
  void* const* peer_table;
  int rank, world, num_experts, num_blocks, num_channels;
  int row_align;               // group row ranges are padded to this many rows (128 or 256)
  int cap_rows;                // rows of the receive buffers; a step that needs more is refused on every rank
  int counts_in_smem;          // set by the launcher: the [world][E] count matrix fits in shared memory
  long long counts_heap_off;   // int [world][E] on every rank
  long long flags_heap_off;    // u64 [world] on every rank: epoch of the last counts row received from each rank
  unsigned long long epoch;
  // Graph-replayable epochs: when non-null, the kernel increments *epoch_dev and uses the new value
  // instead of `epoch` (a value baked into a captured launch would repeat on every replay).
  unsigned long long* epoch_dev;
  const int* block_cnt;        // [num_blocks][E]
  int* block_base;             // [num_blocks][E] out
  int* send_base;              // [E] out: destination row of my first token for expert e
  int* send_cnt;               // [E] out: tokens I send to expert e
  int* send_pos;               // [E] out (may be null): first index of expert e's entries in the sorted send list,
                               // experts ordered by (local expert index, owner rank)
  int* group_off;              // [E/world + 1] out: padded row offsets of my experts
  int* group_rows;             // [E/world] out: real rows of my experts
  unsigned long long* arrive_target;  // [num_channels][E/world] in/out: cumulative rows expected
  // Optional tile-granular targets: tile_target [num_channels][num_tiles] in/out, cumulative real rows expected in
  // every tile_rows-row tile of this rank's receive buffer (tile_rows divides row_align). Null = not kept.
  unsigned long long* tile_target;
  int tile_rows, num_tiles;
  int* traffic_matrix;         // [world][world] out (tokens), may be null
  DeviceStatus* status;
  unsigned long long timeout_ns;
};
cudaError_t launch_splits_scan(const SplitsArgs& a, cudaStream_t stream);
// list[send_pos[e] + rank of (t, j) among my entries for e] = t*K + j  (see SplitsArgs::send_pos).
// Entries whose expert id is outside [0, E) are skipped and reported in `status` (kSiteExpertId).
cudaError_t launch_build_send_list(const int* topk_idx, const int* slot_in_block, const int* block_base, const int* send_pos, int T, int K, int E,
                                   int* list, DeviceStatus* status, cudaStream_t stream);
cudaError_t launch_zero_pad_rows(void* buf, long long row_bytes, const int* group_off, const int* group_rows, int groups, cudaStream_t stream);

// Router front end in one pass (moe_gate.cu): RMSNorm, router logits, top-k, softmax-over-top-k weights and the
// per-block histogram / ranks of route_topk. num_experts <= 32, H % 256 == 0, (num_experts + 1) * H * 2 bytes of
// shared memory (+ 4 bytes per accumulator in the backward pass).
struct NormGateArgs {
  const __nv_bfloat16* h;       // [T, H]
  const __nv_bfloat16* norm_w;  // [H]
  const __nv_bfloat16* gate;    // [E, H]
  const float* bias;            // [E] or null: added for the expert choice only
  int T, H, num_experts, K;
  float eps;
  __nv_bfloat16* hn;            // [T, H] out: h * rstd * norm_w
  float* rstd;                  // [T] out
  float* logits;                // [T, E] out: hn . gate^T (fp32 accumulation of the bf16 values)
  int* topk_idx;                // [T, K] out
  float* topk_w;                // [T, K] out
  int* slot_in_block;           // as launch_route_topk
  int* block_cnt;
};
cudaError_t launch_norm_gate_route(const NormGateArgs& a, cudaStream_t stream);
struct NormGateBwdArgs {
  const __nv_bfloat16* h;       // [T, H] input of the forward pass
  const __nv_bfloat16* norm_w;  // [H]
  const __nv_bfloat16* gate;    // [E, H]
  const float* rstd;            // [T]
  const int* topk_idx;          // [T, K]
  const float* topk_w;          // [T, K]
  const float* grad_w;          // [T, K] gradient of the routing weights
  const __nv_bfloat16* grad_hn; // [T, H] gradient of hn from its other consumer (the MoE input)
  int T, H, num_experts, K;
  __nv_bfloat16* grad_h;        // [T, H] out
  float* d_gate;                // [E, H] fp32, accumulated into (zero it first)
  float* d_norm_w;              // [H] fp32, accumulated into
};
cudaError_t launch_norm_gate_bwd(const NormGateBwdArgs& a, cudaStream_t stream);
size_t norm_gate_smem_bytes(int E, int H, int K, bool backward);

struct DispatchArgs {
  void* const* peer_table;
  int rank, world, num_experts, T, K, H;
  const __nv_bfloat16* x;      // [T, H]
  const int* topk_idx;         // [T, K]
  const float* row_scale;      // [T, K] or null: scale applied to the row sent for slot j
  const int* slot_in_block;    // [T, K]
  const int* block_base;       // [blocks][E]
  const int* send_base;        // [E]
  const int* send_list;        // [T*K] or null: (token*K + slot) entries in sending order (sorted mode)
  int* dest_row;               // [T, K]: written when compute_rows != 0, else read
  int compute_rows;
  int fp8;                     // 1: send e4m3 bytes + one fp32 scale per 128 elements
  const unsigned char* xq;     // fp8 only, optional: rows already quantised by launch_quantise_rows ([T, H] e4m3); x is then not read
  const float* xq_scales;      // their scales [T, H/128]
  long long recv_heap_off;     // destination rows: bf16 [cap, H] (or u8 [cap, H] when fp8)
  long long scale_heap_off;    // fp8 only: float [cap, H/128]
  long long arrive_heap_off;   // u64 arrival counters of this channel: [E/world] per expert, or [num_tiles] per tile
  int tile_rows, num_tiles;    // tile_rows > 0: arrivals are counted per tile of that many destination rows (num_tiles per rank)
  long long entry_flags_heap_off;  // u64 [world]; used when entry_epoch != 0
  unsigned long long entry_epoch;
  DeviceStatus* status;
  unsigned long long timeout_ns;
};
cudaError_t launch_dispatch_push(const DispatchArgs& a, int ctas, cudaStream_t stream);
// x [T, H] bf16 -> q [T, H] e4m3 + scales [T, H/128] (1 x 128 blocks, bf16-exact scales), all local: the
// quantisation the fp8 dispatch otherwise does per entry, done once per row.
cudaError_t launch_quantise_rows(const __nv_bfloat16* x, int T, int H, unsigned char* q, float* scales, int ctas, cudaStream_t stream);

struct CombineArgs {
  void* const* peer_table;
  int rank, world, num_experts, T, K, H;
  const int* topk_idx;         // [T, K]
  const int* dest_row;         // [T, K]
  const float* weights;        // [T, K] or null (= 1)
  long long src_heap_off;      // bf16 [cap, H] on every rank
  long long ready_flags_heap_off;  // u64 [world] in my slab: peer d's rows are final once flags[d] >= ready_epoch
  unsigned long long ready_epoch;
  const unsigned long long* epoch_dev;  // when non-null, *epoch_dev replaces ready_epoch (see SplitsArgs)
  __nv_bfloat16* out;          // [T, H] sum_j w * row_j (null in dot mode)
  const __nv_bfloat16* dot_with;  // dot mode: [T, H]
  float* dot_out;              // dot mode: [T, K] = <dot_with[t], row_j>
  DeviceStatus* status;
  unsigned long long timeout_ns;
};
cudaError_t launch_combine_pull(const CombineArgs& a, int ctas, cudaStream_t stream);

// Writes `epoch` (release, system scope) into slot `rank` of the flag array of every rank.
cudaError_t launch_peer_signal(void* const* peer_table, int rank, int world, long long flags_heap_off, unsigned long long epoch,
                               const unsigned long long* epoch_dev, cudaStream_t stream);
// Bounded wait until counter[i] >= target[i] for all i < n (one thread each).
cudaError_t launch_wait_counters(const unsigned long long* counter, const unsigned long long* target, int n, DeviceStatus* status,
                                 unsigned long long timeout_ns, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// element-wise
// ---------------------------------------------------------------------------------------------
// gate_up: [rows, 2I] in tiles of [128 gate | 128 up]; act: [rows, I].
cudaError_t launch_swiglu_fwd(const __nv_bfloat16* gate_up, __nv_bfloat16* act, long long rows, int inter, cudaStream_t stream);
// d_gate_up = d(silu(g) * u) given d_act. rows_dev (optional, device) caps the rows processed.
cudaError_t launch_swiglu_bwd(const __nv_bfloat16* gate_up, const __nv_bfloat16* d_act, __nv_bfloat16* d_gate_up, long long rows, int inter,
                              const int* rows_dev, cudaStream_t stream);
// Dequantises e4m3 rows with one fp32 scale per 128 elements to bf16. rows_dev (optional, device) caps the rows processed.
cudaError_t launch_dequant_fp8(const unsigned char* q, const float* scales, __nv_bfloat16* out, long long rows, int H, const int* rows_dev,
                               cudaStream_t stream);
// out = scale * sum((a + b)^2) with (a + b) rounded to bf16 first (loss of a residual sum); partial is scratch of partial_len floats.
cudaError_t launch_sumsq_add(const __nv_bfloat16* a, const __nv_bfloat16* b, long long n, float scale, float* partial, int partial_len, float* out,
                             cudaStream_t stream);
// out = bf16(a + b) * (*gscale) * factor (gradient of the above).
cudaError_t launch_scaled_sum(const __nv_bfloat16* a, const __nv_bfloat16* b, long long n, const float* gscale, float factor, __nv_bfloat16* out,
                              cudaStream_t stream);
// Table gradient of an embedding lookup from ids sorted ascending (with their positions); rows of grad_table not named by any id are left as they are.
cudaError_t launch_embedding_bwd(const long long* sorted_ids, const long long* perm, const __nv_bfloat16* grad_out, __nv_bfloat16* grad_table, long long T,
                                 int H, cudaStream_t stream);
// Groups token positions by id with a counting sort (stable: positions ascending inside an id): sorted_ids / perm [T] as
// launch_embedding_bwd takes them; entries past start[V] (ids outside [0, V)) are left as they were. Scratch: hist
// [ceil(T / embedding_index_block())][V] ints (cleared here), rank_in_block [T], total [V], start [V + 1].
cudaError_t launch_embedding_index(const long long* ids, long long T, int V, int* hist, int* rank_in_block, int* total, int* start, long long* sorted_ids,
                                   long long* perm, cudaStream_t stream);
int embedding_index_block();
// AdamW on bf16 parameters with fp32 master weights and moments.
cudaError_t launch_adamw(__nv_bfloat16* param, float* master, float* m, float* v, const __nv_bfloat16* grad, long long n, float lr, float beta1,
                         float beta2, float eps, float weight_decay, float bias_c1, float bias_c2, float grad_scale, cudaStream_t stream);

}  // namespace fastb
