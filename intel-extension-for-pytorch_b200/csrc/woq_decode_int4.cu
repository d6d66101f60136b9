// INT4 weight-only-quantised skinny GEMM for M <= 16 tokens ("decode"): an HBM-bound stream
// of packed weights.
//
// Persistent kernel, two CTAs per SM.  The weight is a linear sequence of k-blocks
// (64 rows x 64 k, 2 KB each, tile-major); CTA c owns an equal contiguous share of it.
// One producer warp moves up to eight k-blocks of one tile per pipeline stage (weights,
// their group scales and the matching slice of x) with bulk asynchronous copies that
// complete on an mbarrier; eight consumer warps take one k-block each:
//   * nibbles become bf16 "128 + q" A-fragments with one lop3 per register (no subtract, no
//     multiply): the tensor core accumulates sum_k x*(128+q) per k-block in fp32, a fifth
//     MMA with an all-ones A-fragment gives sum_k x, and the group's scale and zero point
//     are applied once per k-block:  acc += s * (sum - (128 + zp) * sum_x);
//   * at a tile boundary the eight warps' partial sums are added in shared memory; a CTA
//     that saw the whole K of the tile writes y directly, otherwise the partial goes to the
//     workspace and the last contributor to arrive sums all partials in a fixed order
//     (results do not depend on timing) and runs the fused epilogue.
#include <cstdlib>

#include "woq_kernels.h"

namespace woq {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kStageKBlocks = kConsumerWarps;               // k-blocks per stage
constexpr int kXRowBytes = kStageKBlocks * kBlockK * 2 + 16;  // +16: bank spread between tokens
constexpr int kRedTokStride = 68;                             // floats; conflict-free scatter
constexpr int kHeaderBytes = 1024;
constexpr int kMaxStages = 8;

struct SmemHeader {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  int abort_flag;
  int is_last;
};

__device__ __forceinline__ int owner_of(int64_t b, int64_t total, int64_t ctas) {
  // CTA c owns k-blocks [c*total/ctas, (c+1)*total/ctas)
  return static_cast<int>(((b + 1) * ctas - 1) / total);
}

template <int TB>
__global__ void __launch_bounds__(kThreads, TB == 1 ? 2 : 1)
    woq_int4_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(smem);
  constexpr int NTOK = 8 * TB;
  const int sz_stage_bytes = (p.gps + 1) * 256;
  const int stage_bytes = kStageKBlocks * kBlockBytes + sz_stage_bytes + NTOK * kXRowBytes;
  uint8_t* stages = smem + kHeaderBytes;
  float* red = reinterpret_cast<float*>(stages + static_cast<size_t>(p.stages) * stage_bytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t total = static_cast<int64_t>(p.tiles) * p.kb_per_tile;
  const int64_t b_begin = (static_cast<int64_t>(blockIdx.x) * total) / gridDim.x;
  const int64_t b_end = (static_cast<int64_t>(blockIdx.x + 1) * total) / gridDim.x;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], kConsumerWarps);
    }
    hdr->abort_flag = 0;
    hdr->is_last = 0;
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* abort_flag = &hdr->abort_flag;

  if (warp == kConsumerWarps) {
    // ------------------------------ producer warp ------------------------------------
    int it = 0;
    for (int64_t b = b_begin; b < b_end; ++it) {
      const int tile = static_cast<int>(b / p.kb_per_tile);
      const int kb0 = static_cast<int>(b % p.kb_per_tile);
      int nkb = p.kb_per_tile - kb0;
      if (nkb > kStageKBlocks) nkb = kStageKBlocks;
      if (nkb > b_end - b) nkb = static_cast<int>(b_end - b);
      const int slot = it % p.stages;
      const uint32_t phase = (it / p.stages) & 1;
      uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
      if (lane == 0) {
        mbar_wait(&hdr->empty[slot], phase ^ 1, abort_flag, p.status, 1);
        const int g0 = kb0 / p.kb_per_group;
        const int ng = (kb0 + nkb - 1) / p.kb_per_group - g0 + 1;
        uint32_t bytes = nkb * kBlockBytes;
        if (!(p.debug & 4)) bytes += ng * 256;
        if (!(p.debug & 2)) bytes += p.m * nkb * (kBlockK * 2);
        mbar_arrive_expect_tx(&hdr->full[slot], bytes);
        bulk_g2s(st, p.wq + (static_cast<size_t>(tile) * p.kb_per_tile + kb0) * kBlockBytes,
                 nkb * kBlockBytes, &hdr->full[slot]);
        if (!(p.debug & 4))
          bulk_g2s(st + kStageKBlocks * kBlockBytes,
                   p.sz + (static_cast<size_t>(tile) * p.groups + g0) * 64, ng * 256,
                   &hdr->full[slot]);
      }
      __syncwarp();
      if (lane < p.m && !(p.debug & 2)) {
        bulk_g2s(st + kStageKBlocks * kBlockBytes + sz_stage_bytes + lane * kXRowBytes,
                 p.x + static_cast<size_t>(lane) * p.ldx + static_cast<size_t>(kb0) * kBlockK,
                 nkb * (kBlockK * 2), &hdr->full[slot]);
      }
      b += nkb;
    }
    return;
  }

  // -------------------------------- consumer warps ---------------------------------------
  const int g = lane >> 2, t = lane & 3;
  float acc[4][TB][4];
#pragma unroll
  for (int rt = 0; rt < 4; ++rt)
#pragma unroll
    for (int tb = 0; tb < TB; ++tb)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[rt][tb][i] = 0.f;

  int cur_tile = -1, seg_kb0 = 0, seg_kb1 = 0;
  bool first_segment = true;

  auto flush = [&]() {
    // 1. this warp's partial sums -> red[warp][tok][row]
    float* my = red + warp * (NTOK * kRedTokStride);
#pragma unroll
    for (int rt = 0; rt < 4; ++rt)
#pragma unroll
      for (int tb = 0; tb < TB; ++tb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = rt * 16 + (i >> 1) * 8 + g;
          const int tok = tb * 8 + 2 * t + (i & 1);
          my[tok * kRedTokStride + row] = acc[rt][tb][i];
          acc[rt][tb][i] = 0.f;
        }
    named_bar_sync(1, kConsumerWarps * 32);
    // 2. thread -> (row, tokens q*4 + tid/64)
    const int row = tid & 63;
    float v[NTOK / 4];
#pragma unroll
    for (int q = 0; q < NTOK / 4; ++q) {
      const int tok = q * 4 + (tid >> 6);
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w)
        s += red[w * (NTOK * kRedTokStride) + tok * kRedTokStride + row];
      v[q] = s;
    }
    const bool whole = (seg_kb0 == 0 && seg_kb1 == p.kb_per_tile);
    bool do_epilogue = whole;
    if (!whole) {
      // partial: park it in the workspace, the last contributor reduces
      const int my_slot = blockIdx.x * 2 + (first_segment ? 0 : 1);
      float* dst = p.partials + static_cast<size_t>(my_slot) * (16 * kTileN);
#pragma unroll
      for (int q = 0; q < NTOK / 4; ++q) {
        const int tok = q * 4 + (tid >> 6);
        if (tok < p.m) __stcg(dst + tok * kTileN + row, v[q]);
      }
      __threadfence();
      named_bar_sync(1, kConsumerWarps * 32);
      const int64_t tb0 = static_cast<int64_t>(cur_tile) * p.kb_per_tile;
      const int c_first = owner_of(tb0, total, gridDim.x);
      const int c_last = owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
      if (tid == 0) {
        const unsigned old = atomicAdd(p.counters + cur_tile, 1u);
        hdr->is_last = (old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
      }
      named_bar_sync(1, kConsumerWarps * 32);
      if (hdr->is_last) {
        __threadfence();
#pragma unroll
        for (int q = 0; q < NTOK / 4; ++q) v[q] = 0.f;
        for (int c = c_first; c <= c_last; ++c) {
          const int64_t cb = (static_cast<int64_t>(c) * total) / gridDim.x;
          const int slot = c * 2 + (cb >= tb0 ? 0 : 1);
          const float* src = p.partials + static_cast<size_t>(slot) * (16 * kTileN);
#pragma unroll
          for (int q = 0; q < NTOK / 4; ++q) {
            const int tok = q * 4 + (tid >> 6);
            if (tok < p.m) v[q] += __ldcg(src + tok * kTileN + row);
          }
        }
        if (tid == 0) p.counters[cur_tile] = 0;
        do_epilogue = true;
      }
    }
    if (do_epilogue) {
      if (p.fusion == FUSE_SILU_MUL) {
        // rows 0..31 of the tile are gate rows, rows 32..63 the matching up rows
        named_bar_sync(1, kConsumerWarps * 32);
        float* fin = red;
#pragma unroll
        for (int q = 0; q < NTOK / 4; ++q) {
          const int tok = q * 4 + (tid >> 6);
          const int n = decode_row_to_n(p, cur_tile, row);
          float r = v[q];
          if (n < p.n && p.bias) r += p.bias[n];
          fin[tok * kRedTokStride + row] = bf16_round(r);
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (row < 32) {
          const int col = cur_tile * 32 + row;
#pragma unroll
          for (int q = 0; q < NTOK / 4; ++q) {
            const int tok = q * 4 + (tid >> 6);
            if (tok < p.m && col < p.n_out) {
              const float gate = fin[tok * kRedTokStride + row];
              const float up = fin[tok * kRedTokStride + row + 32];
              p.y[static_cast<size_t>(tok) * p.ldy + col] =
                  __float2bfloat16_rn(up * silu_bf16(gate));
            }
          }
        }
      } else {
        const int n = decode_row_to_n(p, cur_tile, row);
#pragma unroll
        for (int q = 0; q < NTOK / 4; ++q) {
          const int tok = q * 4 + (tid >> 6);
          if (tok < p.m && n < p.n) {
            float r = v[q];
            if (p.bias) r += p.bias[n];
            r = bf16_round(r);
            if (p.fusion == FUSE_SCALED_SCATTER_ADD) {
              const size_t o = static_cast<size_t>(p.row_idx[tok]) * p.ldy + n;
              const float w = __bfloat162float(p.row_w[tok]);
              p.y[o] = __float2bfloat16_rn(__bfloat162float(p.y[o]) + r * w);
            } else {
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
          }
        }
      }
    }
    named_bar_sync(1, kConsumerWarps * 32);  // red is free again
    first_segment = false;
  };

  int it = 0;
  for (int64_t b = b_begin; b < b_end; ++it) {
    const int tile = static_cast<int>(b / p.kb_per_tile);
    const int kb0 = static_cast<int>(b % p.kb_per_tile);
    int nkb = p.kb_per_tile - kb0;
    if (nkb > kStageKBlocks) nkb = kStageKBlocks;
    if (nkb > b_end - b) nkb = static_cast<int>(b_end - b);
    if (tile != cur_tile) {
      if (cur_tile >= 0) flush();
      cur_tile = tile;
      seg_kb0 = kb0;
    }
    seg_kb1 = kb0 + nkb;
    const int slot = it % p.stages;
    const uint32_t phase = (it / p.stages) & 1;
    const uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
    mbar_wait(&hdr->full[slot], phase, abort_flag, p.status, 2);

    if (warp < nkb && !(p.debug & 1)) {
      const int kb = kb0 + warp;
      // packed weights: four row-tiles x four k-steps
      const uint4* wp = reinterpret_cast<const uint4*>(st + warp * kBlockBytes) + lane;
      uint4 wv[4];
#pragma unroll
      for (int rt = 0; rt < 4; ++rt) wv[rt] = wp[rt * 32];
      // activations: this lane's 16 k of token g (+8)
      uint32_t xb[TB][8];
      const uint8_t* xs = st + kStageKBlocks * kBlockBytes + sz_stage_bytes;
#pragma unroll
      for (int tb = 0; tb < TB; ++tb) {
        const int tok = tb * 8 + g;
        if (tok < p.m) {
          const uint4* xp =
              reinterpret_cast<const uint4*>(xs + tok * kXRowBytes + warp * (kBlockK * 2) + t * 32);
          const uint4 a = xp[0], c = xp[1];
          xb[tb][0] = a.x; xb[tb][1] = a.y; xb[tb][2] = a.z; xb[tb][3] = a.w;
          xb[tb][4] = c.x; xb[tb][5] = c.y; xb[tb][6] = c.z; xb[tb][7] = c.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) xb[tb][i] = 0u;
        }
      }
      // scales of this k-block's group for rows g, g+8 of each row-tile
      const int gl = kb / p.kb_per_group - kb0 / p.kb_per_group;
      const uint4* sp =
          reinterpret_cast<const uint4*>(st + kStageKBlocks * kBlockBytes + gl * 256 + g * 32);
      const uint4 s_lo = sp[0], s_hi = sp[1];
      const uint32_t szw[8] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w, s_hi.x, s_hi.y, s_hi.z, s_hi.w};

      float accg[4][TB][4];
      float sx[TB][4];
#pragma unroll
      for (int tb = 0; tb < TB; ++tb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sx[tb][i] = 0.f;
#pragma unroll
        for (int rt = 0; rt < 4; ++rt)
#pragma unroll
          for (int i = 0; i < 4; ++i) accg[rt][tb][i] = 0.f;
      }
      const uint32_t ones[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int tb = 0; tb < TB; ++tb) mma_bf16_16816(sx[tb], ones, xb[tb][2 * j], xb[tb][2 * j + 1]);
#pragma unroll
        for (int rt = 0; rt < 4; ++rt) {
          const uint32_t w = (j == 0) ? wv[rt].x : (j == 1) ? wv[rt].y : (j == 2) ? wv[rt].z : wv[rt].w;
          uint32_t a[4];
          a[0] = lop3_and_or(w, 0x000f000fu, kBf16Magic);
          a[1] = lop3_and_or(w >> 4, 0x000f000fu, kBf16Magic);
          a[2] = lop3_and_or(w >> 8, 0x000f000fu, kBf16Magic);
          a[3] = lop3_and_or(w >> 12, 0x000f000fu, kBf16Magic);
#pragma unroll
          for (int tb = 0; tb < TB; ++tb)
            mma_bf16_16816(accg[rt][tb], a, xb[tb][2 * j], xb[tb][2 * j + 1]);
        }
      }
#pragma unroll
      for (int rt = 0; rt < 4; ++rt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t word = szw[rt * 2 + h];
          const float s = __uint_as_float(word & 0xffff0000u);
          const float nz = -__uint_as_float(word << 16);
#pragma unroll
          for (int tb = 0; tb < TB; ++tb)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const float d = fmaf(nz, sx[tb][c], accg[rt][tb][h * 2 + c]);
              acc[rt][tb][h * 2 + c] = fmaf(s, d, acc[rt][tb][h * 2 + c]);
            }
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&hdr->empty[slot]);
    b += nkb;
  }
  if (cur_tile >= 0) flush();
}

}  // namespace

size_t decode_int4_partial_bytes(int grid) { return static_cast<size_t>(grid) * 2 * 16 * kTileN * 4; }

int decode_int4_pick_grid(const DecodeShape& s, int num_sms) {
  const int64_t total = static_cast<int64_t>(s.tiles) * s.kb_per_tile;
  int per_sm = s.m <= 8 ? 2 : 1;
  if (const char* e = getenv("WOQ_B200_GRID_PER_SM")) per_sm = atoi(e) > 1 && s.m <= 8 ? 2 : 1;
  int64_t grid = static_cast<int64_t>(num_sms) * per_sm;
  if (grid > total) grid = total;
  return static_cast<int>(grid < 1 ? 1 : grid);
}

cudaError_t launch_decode_int4(DecodeParams p, int grid, cudaStream_t stream) {
  const int tb = p.m <= 8 ? 1 : 2;
  const int ntok = 8 * tb;
  const int stage_bytes = kStageKBlocks * kBlockBytes + (p.gps + 1) * 256 + ntok * kXRowBytes;
  const int red_bytes = kConsumerWarps * ntok * kRedTokStride * 4;
  const int budget = (tb == 1 ? 110 : 220) * 1024;
  int stages = (budget - kHeaderBytes - red_bytes) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (const char* e = getenv("WOQ_B200_STAGES")) {
    const int want = atoi(e);
    if (want >= 2 && want <= stages) stages = want;
  }
  if (const char* e = getenv("WOQ_B200_DEBUG")) p.debug = atoi(e);
  if (stages < 2) return cudaErrorInvalidConfiguration;
  p.stages = stages;
  const size_t smem = kHeaderBytes + static_cast<size_t>(stages) * stage_bytes + red_bytes;
  cudaError_t e;
  if (tb == 1) {
    e = cudaFuncSetAttribute(woq_int4_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    woq_int4_decode_kernel<1><<<grid, kThreads, smem, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(woq_int4_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    woq_int4_decode_kernel<2><<<grid, kThreads, smem, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace woq
