// Internal interface between the C ABI (woq_capi.cu) and the kernel translation units.
#pragma once
#include <cuda.h>

#include "woq_common.cuh"

namespace woq {

// ---- tensor-parallel exchange fused into the decode kernel's epilogue ---------------------
// Every rank of one node owns a "symmetric" buffer with the same layout and maps all peers'
// buffers (CUDA IPC).  Layout of one buffer:
//   [0, 4096)               control words: epoch (u32 @0), finished CTAs of the running grid (u32 @4)
//   [4096, +slot_n*2048)    exchange words {2 x bf16, stamp}, 8 bytes each:
//                           [epoch & 3][source rank][tile][token][lane]
//   [gather_off, ..)        gather area (the caller places gathered tensors here)
// A launch with a comm mode is one "epoch" (the same number on every rank, because all ranks
// issue the same sequence of launches); its stamp is epoch + 1.  The warp that finishes a
// tile stores each lane's two results and the stamp as one 8-byte word into every other
// rank's slot (data and mark arrive together, no fence).
//   all-reduce: the same warp then reads its own slots for the other ranks' words of the same
//     tile (all ranks' loads in flight together) and adds them in rank order;
//   all-gather: nobody waits.  The NEXT launch on the comm (or comm_fence) copies the words of
//     the other ranks into this rank's gathered tensor with its otherwise idle epilogue warps,
//     while its own weights stream: the gathered tensor is complete when that launch ends.
// Four slot sets, indexed by epoch & 3: finishing the launch of epoch X takes every peer's
// words of epoch X - 1 at least, so a rank that writes set E & 3 knows every peer has finished
// the launches up to E - 3, and with them the reading of epoch E - 4.
constexpr int kCommMaxRanks = 8;
constexpr int kCommMaxTiles = 1024;
constexpr int kCommCtlBytes = 4096;
constexpr int kCommSets = 4;
enum CommMode { kCommNone = 0, kCommAllReduce = 1, kCommAllGather = 2 };

// The all-gather of the previous launch on the comm, still to be received on this rank.
struct CommPending {
  __nv_bfloat16* dst;  // this rank's gathered tensor [m][world * n_out]; null: nothing pending
  int m, n, n_out, tiles, gate_up, pair;  // of the launch that sent it (pair: two values per word)
};

struct CommParams {
  uint8_t* peer[kCommMaxRanks];  // base of every rank's buffer as mapped here (peer[rank]: own)
  int mode, world, rank;
  int64_t ar_n;        // 64 x the tiles a slot set holds
  CommPending pend;
};

// ---- INT4 decode (M <= 16) -----------------------------------------------------------
struct DecodeParams {
  const uint8_t* wq;       // tiled nibbles [tiles][kb_per_tile][2048]
  const uint32_t* sz;      // [tiles][groups][64] {bf16 scale, bf16 128+zp}
  const float* bias;       // [n] or null
  const __nv_bfloat16* x;  // [m][ldx]
  __nv_bfloat16* y;        // [m][ldy]  (scatter: [*][ldy])
  const __nv_bfloat16* other0;
  const __nv_bfloat16* other1;
  const int32_t* row_idx;       // scatter epilogue
  const __nv_bfloat16* row_w;   // scatter epilogue
  float* partials;         // [2 * grid][16][64]
  uint32_t* counters;      // [tiles], zero between calls
  int* status;             // 0, or the code of the wait that gave up
  int64_t ldx, ldy;
  int64_t ldo;  // row length of other0 / other1
  int m, n, n_out, k;
  int tiles, kb_per_tile, kbpg_shift, groups, gps;  // gps = groups a full stage can touch
  int fusion, gate_up, stages;
  int exact;  // 0: scale after the sum; 1, 2: per-weight bf16 rounding (2: shift-free high nibbles)
  int unit;   // CTA shares are multiples of this many k-blocks
  int x_rows, red_tok;  // shared-memory rows for x per stage / tokens in the reduction buffer
#ifdef WOQ_B200_TIMELINE
  unsigned long long* stamps;  // measuring build only: [8 launches][1024 CTAs][8] global-timer stamps
  int launch_seq;
#endif
  CommParams comm;
};

// How a launch cuts the weight: `cluster` == 0 is the stream-K grid (equal contiguous shares of
// the k-block sequence, split tiles reduced through the workspace); `cluster` == C >= 1 is
// tiles x C CTAs in thread-block clusters of C that reduce through distributed shared memory.
struct DecodePlan {
  int grid, cluster, kpw, unit, smem_budget;
};

template <class P>
__device__ __forceinline__ int decode_row_to_n(const P& p, int tile, int row) {
  if (p.gate_up) return row < 32 ? tile * 32 + row : p.n / 2 + tile * 32 + (row - 32);
  return tile * kTileN + row;
}

// 0 per-layer choice, 1 always stream-K, 2 cluster grid whenever the tiles fit (see DecodePlan)
void decode_int4_set_split(int mode);
DecodePlan decode_int4_plan(int m, int tiles, int kb_per_tile, int kb_per_group, int num_sms);
size_t decode_int4_partial_bytes(int grid);
cudaError_t launch_decode_int4(DecodeParams p, const DecodePlan& plan, cudaStream_t stream);
// Receives a pending all-gather without running a linear (status: the workspace-style status word).
cudaError_t launch_comm_fence(const CommParams& c, int* status, int num_sms, cudaStream_t stream);

// ---- INT4 tensor-core path (any M up to 256 per launch) --------------------------------
// Row layout: tiles of 128 output rows x 64 k, 4096 bytes each, [tile][k-block][half][row][16 B].
// Word j' = 4 * half + j of a row holds k = 8 j' + 2 s in nibble s (bits 4s..4s+3) and
// k = 8 j' + 2 s + 1 in nibble s + 4, so (w >> 4s) & 0x000f000f is the bf16x2 pair (k, k+1).
// Scales: [tile][group][128] words, same {bf16 scale, bf16 128 + zp} format.
constexpr int kTcTileN = 128;
constexpr int kTcBlockBytes = kTcTileN * kBlockK / 2;  // 4096

struct TcParams {
  const uint8_t* wq;
  const uint32_t* sz;
  const float* bias;
  __nv_bfloat16* y;
  const __nv_bfloat16* other0;
  const __nv_bfloat16* other1;
  const int32_t* row_idx;
  const __nv_bfloat16* row_w;
  float* partials;     // [2 * grid][n_tok][128]
  uint32_t* counters;  // [tiles]
  int* status;
  int64_t ldy;
  int m, n, n_out, k;
  int m0;              // first token row of this launch inside the x tensor map
  int n_tok;           // token columns of the MMA (multiple of 16, <= 256)
  int tiles, kb_per_tile, kbpg_shift, groups;
  int kbs, stages;     // k-blocks per stage; slots of the A-group / activation ring
  int w_ring, a_col0;  // slots of the packed-weight ring (a multiple of four); first TMEM column of the A groups
  int fusion, gate_up;
};

// the M <= 16 kernel's launches opt into programmatic dependent launch unless WOQ_B200_PDL=0 was
// set before first use (the tcgen05 kernels launch plainly)
bool dependent_launch_enabled();
int tc_pick_grid(int tiles, int kb_per_tile, int num_sms);
size_t tc_partial_bytes(int grid, int n_tok);
size_t tc_plan(TcParams& p);  // fills a_col0, kbs, stages, w_ring from n_tok; returns the dynamic shared memory (0: none)
cudaError_t launch_int4_tc(TcParams p, const CUtensorMap& xmap, int grid, cudaStream_t stream);

__host__ __device__ inline int tc_tile_row_to_n(int n_total, int gate_up, int tile, int row) {
  if (gate_up) return row < 64 ? tile * 64 + row : n_total / 2 + tile * 64 + (row - 64);
  return tile * kTcTileN + row;
}

// ---- INT8 compute path ----------------------------------------------------------------------
struct I8Params {
  const int8_t* wq;     // operand images [tiles64][kc_per_tile][8192]
  const float* sw;      // per-channel weight scales [n_pad]
  const float* sa;      // per-token activation scales [m]
  const int32_t* zpa;   // per-token activation zero points [m] (asymmetric codes are u8), or null
  const int32_t* comp;  // with zpa: per-row sums of the weight codes [n_pad]
  const float* bias;
  __nv_bfloat16* y;     // may be null when only the accumulators are wanted
  const __nv_bfloat16* other0;
  const __nv_bfloat16* other1;
  int* acc_out;         // optional [m][n] int32 accumulators
  void* partials;       // int32 [2 * grid][n_tok][128]
  uint32_t* counters;
  int* status;
  int64_t ldy;
  int m, n, n_out;
  int m0, n_tok;
  int tiles, kc_per_tile;  // 128-row tiles, 128-k chunks
  int stages, fusion, gate_up;
};
cudaError_t launch_pack_int8(const int8_t* plain, int8_t* tiled, int n, int k, int tiles64,
                             int gate_up, cudaStream_t stream);
cudaError_t launch_unpack_int8(const int8_t* tiled, int8_t* plain, int n, int k, int gate_up,
                               cudaStream_t stream);
cudaError_t launch_pad_scale(const void* src, float* dst, int n, int n_pad, int dtype,
                             cudaStream_t stream);
cudaError_t launch_quant_act(const __nv_bfloat16* x, int64_t ldx, int m, int k, int asym, int per_tensor,
                             int8_t* qa, float* sa, int32_t* zpa, float* range, cudaStream_t stream);
cudaError_t launch_rmsnorm_quant(const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* gamma, float eps, int m,
                                 int k, int asym, __nv_bfloat16* y, int64_t ldy, int8_t* qa, float* sa, int32_t* zpa,
                                 cudaStream_t stream);
cudaError_t launch_weight_row_sum(const int8_t* plain, int n, int k, int32_t* comp, cudaStream_t stream);
size_t int8_partial_bytes(int grid, int n_tok);
cudaError_t launch_int8_tc(I8Params p, const CUtensorMap& qamap, int grid, cudaStream_t stream);

// ---- INT8 compute with K-block scaling (woq_int8_block.cu) --------------------------------
struct I8BlockParams {
  const uint8_t* w;      // plain [n][k/2] nibbles (w4) or [n][k] s8
  const float* sw;       // [n][groups] weight scales
  const float* zpw;      // [n][groups] weight zero points or null (default_zp)
  const int32_t* comp;   // [n][kc] sums of (qw - zp_w) per K block (asymmetric activations)
  const uint8_t* qa;     // [m][k] activation codes (w4: even / odd interleaved inside every 8)
  const float* sa;       // [m][kc]
  const int32_t* zpa;    // [m][kc]
  const int32_t* sumqa;  // [m][kc] sums of the activation codes per K block
  const float* bias;
  __nv_bfloat16* y;      // may be null when only the accumulators are wanted
  const __nv_bfloat16* other0;
  const __nv_bfloat16* other1;
  int32_t* acc_out;      // optional [kc][m][n] block accumulators after the compensation
  int64_t ldy;
  int m, n, k, kb, kc, group, groups, fusion, w4, asym;
  float default_zp;
};
cudaError_t launch_act_block_quant(const __nv_bfloat16* x, int64_t ldx, int m, int k, int kb, int act_mode,
                                   int interleave, uint8_t* qa, float* sa, int32_t* zpa, int32_t* sumqa,
                                   float* range, float* folded, cudaStream_t stream);
cudaError_t launch_weight_block_sum(const uint8_t* w, const float* zpw, int n, int k, int kb, int group, int groups,
                                    float default_zp, int w4, int32_t* comp, cudaStream_t stream);
cudaError_t launch_i8_block(const I8BlockParams& p, cudaStream_t stream);

// ---- general route: any weight dtype, fp32 / fp16 / bf16 compute, plain layout -----------
struct GenericParams {
  const uint8_t* w;     // plain [n][row_bytes]: nibbles (even k low) or bytes
  const float* scales;  // [n][groups] fp32 as given (rounded to the compute dtype in the kernel)
  const float* zps;     // [n][groups] or null (then default_zp)
  const float* bias;    // [n] or null
  const void* x;        // [m][ldx] of io_dtype
  void* y;              // [m][ldy] of io_dtype
  const void* other0;
  const void* other1;
  int64_t ldx, ldy;
  int m, n, k, group, groups, row_bytes;
  int weight_dtype, compute_dtype, io_dtype, fusion;  // WOQ_B200_DTYPE_* / WOQ_B200_T_*
  float default_zp;
};
cudaError_t launch_generic(const GenericParams& p, cudaStream_t stream);
cudaError_t launch_dump_generic(const GenericParams& p, float* out, cudaStream_t stream);

// ---- pack / unpack / dump ------------------------------------------------------------
struct PackInt4Args {
  const uint8_t* plain;  // [n][ceil(k/2)]
  uint8_t* tiled;
  int n, k, tiles, kb_per_tile, gate_up;
  int tc;  // 0: 64-row fragment layout, 1: 128-row row layout
};
cudaError_t launch_pack_int4(const PackInt4Args& a, cudaStream_t stream);
cudaError_t launch_unpack_int4(const uint8_t* tiled, uint8_t* plain, int n, int k, int tiles,
                               int kb_per_tile, int gate_up, cudaStream_t stream);

struct PackScaleArgs {
  const void* scales;  // [n][groups] (or transposed [groups][n])
  const void* zps;     // same shape or null
  uint32_t* sz;        // [tiles][groups][64]
  int* bad_zp;         // bit 0: a zero point is not an integer in 0..127; bit 1: see pack_scales_kernel
  int n, tiles, groups, gate_up;
  int transposed;     // scales are [groups][n]
  int zp_transposed;  // zero points are [groups][n]
  int scale_dtype, zp_dtype, default_zp;
  int tc;  // 0: [tiles64][groups][64] fragment order, 1: [tiles128][groups][128] row order
};
cudaError_t launch_pack_scales(const PackScaleArgs& a, cudaStream_t stream);

cudaError_t launch_dump_dequant_int4(const uint8_t* tiled, const uint32_t* sz, __nv_bfloat16* w,
                                     int n, int k, int tiles, int kb_per_tile, int kb_per_group,
                                     int groups, int gate_up, cudaStream_t stream);
cudaError_t launch_dump_dequant_int4_tc(const uint8_t* tiled, const uint32_t* sz, __nv_bfloat16* w,
                                        int n, int k, int tiles, int kb_per_tile, int kbpg_shift,
                                        int groups, int gate_up, cudaStream_t stream);

cudaError_t launch_gather_rows(const __nv_bfloat16* x, int64_t ldx, const int32_t* idx,
                               __nv_bfloat16* out, int64_t rows, int k, cudaStream_t stream);

// AWQ / GPTQ int32 checkpoints -> plain nibble layout [n][k/2]
cudaError_t launch_awq_to_plain(const int32_t* qweight_kn8, uint8_t* plain, int n, int k,
                                cudaStream_t stream);
cudaError_t launch_gptq_to_plain(const int32_t* qweight_k8n, uint8_t* plain, int n, int k,
                                 cudaStream_t stream);
// packed int32 zero points [groups][n/8] -> u8 [n][groups]; gptq_plus_one adds 1 (GPTQ v1)
cudaError_t launch_unpack_qzeros(const int32_t* qzeros, uint8_t* zps, int n, int groups, int awq,
                                 int plus_one, cudaStream_t stream);

__host__ __device__ inline int tile_row_to_n(int n_total, int gate_up, int tile, int row) {
  if (gate_up) return row < 32 ? tile * 32 + row : n_total / 2 + tile * 32 + (row - 32);
  return tile * kTileN + row;
}

void count_launch();

}  // namespace woq
