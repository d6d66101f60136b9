// INT4 weight-only-quantised GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for
// any token count up to 256 per launch.
//
// Orientation: the weight is the A operand (128 output rows = the 128 TMEM lanes), the
// activations are the B operand (N = tokens, 16..256), so one CTA tile is y^T[128 rows x
// tokens] accumulated in fp32 in TMEM over the whole K of its share.
//
//   warp 8      producer: bulk copies of packed nibbles + group scales, TMA tile loads of x
//               (128-byte swizzled K-major rows) - all completing on mbarriers;
//   warps 0-7   dequantise: thread = output row.  Two 128-bit shared loads give the row's 64
//               nibbles of a k-block; each becomes bf16((q - zp) * bf16(scale)) exactly (the
//               reference's tile dequantiser) and the 32 packed registers go straight to
//               TMEM with one tcgen05.st - the dequantised tile never touches shared memory.
//               Even / odd k-blocks alternate between the two warpgroups;
//   warp 9      one thread issues tcgen05.mma (A from TMEM, B from shared memory) and
//               releases A slots / x stages / the accumulator with tcgen05.commit;
//   warps 0-7   epilogue at the end of a tile segment: tcgen05.ld the accumulators, then
//               either the fused post-op and store, or - when the CTA saw only part of K -
//               a partial tile in the workspace that the last contributor sums in a fixed
//               order.
// Work split: the (tile, k-block) sequence is cut into equal contiguous shares, one per SM.
#include <cstdlib>

#include "woq_kernels.h"
#include "woq_tc_common.cuh"

namespace woq {

namespace {

constexpr int kDequantWarps = 8;
constexpr int kTcThreads = (kDequantWarps + 2) * 32;
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kASlots = 8;           // 32 TMEM columns each (one k-block of bf16 A)
constexpr int kDCol0 = 0;            // accumulator columns [0, 256)
constexpr int kACol0 = 256;          // A slots in columns [256, 512)
constexpr int kTmemCols = 512;
constexpr int kMaxTcStages = 8;
constexpr int kTcHeaderBytes = 1024;

struct TcHeader {
  uint64_t w_full[kMaxTcStages], w_empty[kMaxTcStages];
  uint64_t x_full[kMaxTcStages], x_empty[kMaxTcStages];
  uint64_t a_full[kASlots], a_empty[kASlots];
  uint64_t d_full, d_empty;
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};
static_assert(sizeof(TcHeader) <= kTcHeaderBytes, "header too large");

__device__ __forceinline__ int tc_owner_of(int64_t b, int64_t total, int64_t ctas) {
  return static_cast<int>(((b + 1) * ctas - 1) / total);
}

__device__ __forceinline__ int tc_row_to_n(const TcParams& p, int tile, int row) {
  if (p.gate_up) return row < 64 ? tile * 64 + row : p.n / 2 + tile * 64 + (row - 64);
  return tile * kTcTileN + row;
}

// One (row, token) result through bias, rounding and the fused post-op.
__device__ __forceinline__ void tc_store(const TcParams& p, int tile, int row, int tok, float v) {
  const int n = tc_row_to_n(p, tile, row);
  if (tok >= p.m || n >= p.n) return;
  if (p.bias) v += p.bias[n];
  float r = bf16_round(v);
  if (p.fusion == FUSE_SCALED_SCATTER_ADD) {
    const size_t o = static_cast<size_t>(p.row_idx[tok]) * p.ldy + n;
    const float w = __bfloat162float(p.row_w[tok]);
    p.y[o] = __float2bfloat16_rn(__bfloat162float(p.y[o]) + r * w);
    return;
  }
  const size_t o = static_cast<size_t>(tok) * p.ldy + n;
  if (p.fusion == FUSE_ADD || p.fusion == FUSE_ADD_ADD) {
    r = bf16_round(r + __bfloat162float(p.other0[o]));
    if (p.fusion == FUSE_ADD_ADD) r = bf16_round(r + __bfloat162float(p.other1[o]));
  } else if (p.fusion == FUSE_MUL) {
    r = bf16_round(r * __bfloat162float(p.other0[o]));
  } else {
    r = unary_post_op(r, p.fusion);
  }
  p.y[o] = __float2bfloat16_rn(r);
}

__global__ void __launch_bounds__(kTcThreads, 1)
    woq_int4_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap xmap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  TcHeader* hdr = reinterpret_cast<TcHeader*>(smem);
  const int x_stage_bytes = p.kbs * p.n_tok * 128;
  const int w_stage_bytes = p.kbs * kTcBlockBytes + (p.kbs + 1) * 512;
  uint8_t* x_stages = smem + kTcHeaderBytes;
  uint8_t* w_stages = x_stages + static_cast<size_t>(p.stages) * x_stage_bytes;
  float* fin = reinterpret_cast<float*>(w_stages + static_cast<size_t>(p.stages) * w_stage_bytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned base
    if (tid == 0) atomicCAS(p.status, 0, 99);
    return;
  }
  const int64_t total = static_cast<int64_t>(p.tiles) * p.kb_per_tile;
  const int64_t b_begin = (static_cast<int64_t>(blockIdx.x) * total) / gridDim.x;
  const int64_t b_end = (static_cast<int64_t>(blockIdx.x + 1) * total) / gridDim.x;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&hdr->w_full[s], 1);
      mbar_init(&hdr->w_empty[s], kDequantWarps);
      mbar_init(&hdr->x_full[s], 1);
      mbar_init(&hdr->x_empty[s], 1);
    }
    for (int s = 0; s < kASlots; ++s) {
      mbar_init(&hdr->a_full[s], 4);
      mbar_init(&hdr->a_empty[s], 1);
    }
    mbar_init(&hdr->d_full, 1);
    mbar_init(&hdr->d_empty, kDequantWarps);
    hdr->abort_flag = 0;
    hdr->is_last = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&hdr->tmem_base, kTmemCols);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = hdr->tmem_base;
  volatile int* abort_flag = &hdr->abort_flag;

  // every role walks the same sequence of stages
  int tile = static_cast<int>(b_begin / p.kb_per_tile);
  int kb0 = static_cast<int>(b_begin % p.kb_per_tile);
  int64_t b = b_begin;
  auto stage_len = [&]() {
    int nkb = p.kb_per_tile - kb0;
    if (nkb > p.kbs) nkb = p.kbs;
    if (nkb > b_end - b) nkb = static_cast<int>(b_end - b);
    return nkb;
  };
  auto advance = [&](int nkb) {
    b += nkb;
    kb0 += nkb;
    if (kb0 == p.kb_per_tile) {
      kb0 = 0;
      ++tile;
    }
  };

  if (warp == kProducerWarp) {
    if (lane == 0) {
      for (int it = 0; b < b_end; ++it) {
        const int nkb = stage_len();
        const int slot = it % p.stages;
        const uint32_t phase = (it / p.stages) & 1;
        uint8_t* ws = w_stages + static_cast<size_t>(slot) * w_stage_bytes;
        uint8_t* xs = x_stages + static_cast<size_t>(slot) * x_stage_bytes;
        const int g0 = kb0 >> p.kbpg_shift;
        const int ng = ((kb0 + nkb - 1) >> p.kbpg_shift) - g0 + 1;
        mbar_wait(&hdr->w_empty[slot], phase ^ 1, abort_flag, p.status, 11);
        mbar_arrive_expect_tx(&hdr->w_full[slot], nkb * kTcBlockBytes + ng * 512);
        bulk_g2s(ws, p.wq + (static_cast<size_t>(tile) * p.kb_per_tile + kb0) * kTcBlockBytes,
                 nkb * kTcBlockBytes, &hdr->w_full[slot]);
        bulk_g2s(ws + p.kbs * kTcBlockBytes,
                 p.sz + (static_cast<size_t>(tile) * p.groups + g0) * kTcTileN, ng * 512,
                 &hdr->w_full[slot]);
        mbar_wait(&hdr->x_empty[slot], phase ^ 1, abort_flag, p.status, 12);
        mbar_arrive_expect_tx(&hdr->x_full[slot], nkb * p.n_tok * 128);
        for (int j = 0; j < nkb; ++j)
          tma_load_2d(xs + j * p.n_tok * 128, &xmap, (kb0 + j) * kBlockK, p.m0, &hdr->x_full[slot]);
        advance(nkb);
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(p.n_tok, /*bf16*/ 1, /*f32*/ 1);
      int kbc = 0, seg = 0;
      bool seg_start = true;
      for (int it = 0; b < b_end; ++it) {
        const int nkb = stage_len();
        const int slot = it % p.stages;
        const uint32_t phase = (it / p.stages) & 1;
        const uint8_t* xs = x_stages + static_cast<size_t>(slot) * x_stage_bytes;
        const bool seg_end = (kb0 + nkb == p.kb_per_tile) || (b + nkb == b_end);
        mbar_wait(&hdr->x_full[slot], phase, abort_flag, p.status, 13);
        for (int j = 0; j < nkb; ++j) {
          const int i = kbc + j, aslot = i % kASlots;
          mbar_wait(&hdr->a_full[aslot], (i / kASlots) & 1, abort_flag, p.status, 14);
          if (seg_start && j == 0)
            mbar_wait(&hdr->d_empty, (seg & 1) ^ 1, abort_flag, p.status, 15);
          tc_fence_after_sync();
          const uint64_t bdesc = umma_desc_k128(smem_u32(xs + j * p.n_tok * 128));
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ts(tmem_base + kDCol0, tmem_base + kACol0 + aslot * 32 + ks * 8,
                        bdesc + ks * 2, idesc, (seg_start && j == 0 && ks == 0) ? 0u : 1u);
          tc_commit(&hdr->a_empty[aslot]);
        }
        tc_commit(&hdr->x_empty[slot]);
        if (seg_end) {
          tc_commit(&hdr->d_full);
          ++seg;
        }
        seg_start = seg_end;
        kbc += nkb;
        advance(nkb);
      }
    }
  } else {
    // --------------------------- dequantise + epilogue warps -----------------------------
    const int wg = warp >> 2, q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    int kbc = 0, seg = 0, seg_kb0 = kb0;
    bool first_segment = true;
    for (int it = 0; b < b_end; ++it) {
      const int nkb = stage_len();
      const int slot = it % p.stages;
      const uint32_t phase = (it / p.stages) & 1;
      const uint8_t* ws = w_stages + static_cast<size_t>(slot) * w_stage_bytes;
      const bool seg_end = (kb0 + nkb == p.kb_per_tile) || (b + nkb == b_end);
      mbar_wait(&hdr->w_full[slot], phase, abort_flag, p.status, 16);
      const int g0 = kb0 >> p.kbpg_shift;
      for (int j = 0; j < nkb; ++j) {
        const int i = kbc + j;
        if ((i & 1) != wg) continue;
        const int aslot = i % kASlots;
        const uint4* wp = reinterpret_cast<const uint4*>(ws + j * kTcBlockBytes);
        const uint4 v0 = wp[row], v1 = wp[kTcTileN + row];
        const uint32_t szw = reinterpret_cast<const uint32_t*>(
            ws + p.kbs * kTcBlockBytes)[(((kb0 + j) >> p.kbpg_shift) - g0) * kTcTileN + row];
        const uint32_t z2 = __byte_perm(szw, 0, 0x1010), s2 = __byte_perm(szw, 0, 0x3232);
        const uint32_t words[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        uint32_t r[32];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
#pragma unroll
          for (int s = 0; s < 4; ++s)
            r[jj * 4 + s] = bf16x2_mul(
                bf16x2_sub(lop3_and_or(words[jj] >> (4 * s), 0x000f000fu, kBf16Magic), z2), s2);
        }
        mbar_wait(&hdr->a_empty[aslot], ((i / kASlots) & 1) ^ 1, abort_flag, p.status, 17);
        tc_fence_after_sync();
        tmem_st_x32(lane_addr + kACol0 + aslot * 32, r);
        tc_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->a_full[aslot]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->w_empty[slot]);
      kbc += nkb;

      if (seg_end) {
        const int seg_kb1 = kb0 + nkb;
        const bool whole = (seg_kb0 == 0 && seg_kb1 == p.kb_per_tile);
        const int half_tok = p.n_tok / 2;  // this warpgroup's token columns
        const int tok0 = wg * half_tok;
        mbar_wait(&hdr->d_full, seg & 1, abort_flag, p.status, 18);
        tc_fence_after_sync();
        if (whole && p.fusion != FUSE_SILU_MUL) {
          for (int c = 0; c < half_tok; c += 8) {
            uint32_t v[8];
            tmem_ld_x8(lane_addr + kDCol0 + tok0 + c, v);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e) tc_store(p, tile, row, tok0 + c + e, __uint_as_float(v[e]));
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->d_empty);
        } else {
          // park this CTA's contribution in the workspace (also used to pair gate/up rows)
          const int my_slot = blockIdx.x * 2 + (first_segment ? 0 : 1);
          float* dst = p.partials + static_cast<size_t>(my_slot) * p.n_tok * kTcTileN;
          for (int c = 0; c < half_tok; c += 8) {
            uint32_t v[8];
            tmem_ld_x8(lane_addr + kDCol0 + tok0 + c, v);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (tok0 + c + e < p.m)
                __stcg(dst + static_cast<size_t>(tok0 + c + e) * kTcTileN + row, __uint_as_float(v[e]));
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->d_empty);
          const int64_t tb0 = static_cast<int64_t>(tile) * p.kb_per_tile;
          const int c_first = tc_owner_of(tb0, total, gridDim.x);
          const int c_last = tc_owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
          __threadfence();
          named_bar_sync(1, kDequantWarps * 32);
          if (tid == 0) {
            int last = 1;
            if (!whole) {
              const unsigned old = atomicAdd(p.counters + tile, 1u);
              last = (old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
            }
            hdr->is_last = last;
          }
          named_bar_sync(1, kDequantWarps * 32);
          if (hdr->is_last) {
            __threadfence();
            for (int c = 0; c < half_tok; ++c) {
              const int tok = tok0 + c;
              if (tok >= p.m) break;
              float v = 0.f;
              float v_up = 0.f;
              for (int cc = c_first; cc <= c_last; ++cc) {
                const int64_t cb = (static_cast<int64_t>(cc) * total) / gridDim.x;
                const int slot2 = whole ? my_slot : cc * 2 + (cb >= tb0 ? 0 : 1);
                const float* src = p.partials + static_cast<size_t>(slot2) * p.n_tok * kTcTileN +
                                   static_cast<size_t>(tok) * kTcTileN;
                v += __ldcg(src + row);
                if (p.fusion == FUSE_SILU_MUL && row < 64) v_up += __ldcg(src + row + 64);
              }
              if (p.fusion == FUSE_SILU_MUL) {
                if (row < 64) {
                  const int ng_ = tile * 64 + row;       // gate row
                  const int nu_ = p.n / 2 + ng_;         // matching up row
                  if (p.bias) {
                    v += p.bias[ng_];
                    v_up += p.bias[nu_];
                  }
                  const float gate = bf16_round(v), up = bf16_round(v_up);
                  if (ng_ < p.n_out)
                    p.y[static_cast<size_t>(tok) * p.ldy + ng_] =
                        __float2bfloat16_rn(up * silu_bf16(gate));
                }
              } else {
                tc_store(p, tile, row, tok, v);
              }
            }
            if (tid == 0 && !whole) p.counters[tile] = 0;
          }
          named_bar_sync(1, kDequantWarps * 32);
        }
        ++seg;
        first_segment = false;
      }
      advance(nkb);
      if (seg_end) seg_kb0 = kb0;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  (void)fin;
}

}  // namespace

size_t tc_partial_bytes(int grid, int n_tok) {
  return static_cast<size_t>(grid) * 2 * n_tok * kTcTileN * sizeof(float);
}

int tc_pick_grid(int tiles, int kb_per_tile, int num_sms) {
  const int64_t total = static_cast<int64_t>(tiles) * kb_per_tile;
  int64_t grid = num_sms;
  if (grid > total) grid = total;
  return static_cast<int>(grid < 1 ? 1 : grid);
}

cudaError_t launch_int4_tc(TcParams p, const CUtensorMap& xmap, int grid, cudaStream_t stream) {
  // k-blocks per stage: enough bytes in flight for small token counts, one x tile otherwise
  p.kbs = p.n_tok <= 32 ? 4 : (p.n_tok <= 64 ? 2 : 1);
  const int x_stage = p.kbs * p.n_tok * 128;
  const int w_stage = p.kbs * kTcBlockBytes + (p.kbs + 1) * 512;
  const int budget = 200 * 1024;
  int stages = (budget - kTcHeaderBytes) / (x_stage + w_stage);
  if (stages > kMaxTcStages) stages = kMaxTcStages;
  if (const char* e = getenv("WOQ_B200_TC_STAGES")) {
    const int want = atoi(e);
    if (want >= 2 && want <= stages) stages = want;
  }
  if (stages < 2) return cudaErrorInvalidConfiguration;
  p.stages = stages;
  const size_t smem = kTcHeaderBytes + static_cast<size_t>(stages) * (x_stage + w_stage);
  cudaError_t e = cudaFuncSetAttribute(woq_int4_tc_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  woq_int4_tc_kernel<<<grid, kTcThreads, smem, stream>>>(p, xmap);
  return cudaGetLastError();
}

}  // namespace woq
