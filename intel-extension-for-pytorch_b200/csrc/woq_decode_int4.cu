// INT4 weight-only-quantised skinny GEMM for M <= 16 tokens ("decode"): an HBM-bound stream
// of packed weights.
//
// Persistent kernel, two CTAs per SM (one for 9..16 tokens).  The weight is a linear sequence
// of k-blocks (64 rows x 64 k, 2 KB each, tile-major); CTA c owns an equal contiguous share.
// One producer warp moves up to eight k-blocks of one tile per pipeline stage (weights, their
// group scales and the matching slice of x) with bulk asynchronous copies that complete on
// an mbarrier; eight consumer warps take one k-block each:
//   * nibbles become bf16 "128 + q" A-fragments with one lop3 per register (no subtract, no
//     multiply): the tensor core accumulates sum_k x*(128+q) per k-block in fp32, a fifth
//     MMA with an all-ones A-fragment gives sum_k x, and the group's scale and zero point
//     are applied once per k-block:  acc += s * (sum - (128 + zp) * sum_x);
//   * at a tile boundary the eight warps' partial sums are added in shared memory; a CTA
//     that saw the whole K of the tile writes y directly, otherwise the partial goes to the
//     workspace and the last contributor to arrive sums all partials in a fixed order
//     (results do not depend on timing) and runs the fused epilogue.  A CTA that still has
//     tiles to stream does not wait for the arrival count: it looks at it after its last
//     tile.
// The memory system needs about 2.5 us x 44 GB/s = 110+ KB in flight per SM to stay busy,
// which sets the number of pipeline stages.
#include <cstdlib>

#include "woq_kernels.h"

namespace woq {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kStageKBlocks = kConsumerWarps;                 // k-blocks per stage
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

template <int TB, bool EXACT>
__global__ void __launch_bounds__(kThreads, TB == 1 ? 2 : 1)
    woq_int4_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(smem);
  constexpr int NTOK = 8 * TB;
  const int sz_stage_bytes = (p.gps + 1) * 256;
  const int stage_bytes = kStageKBlocks * kBlockBytes + sz_stage_bytes + p.x_rows * kXRowBytes;
  const int red_tok = p.red_tok;  // tokens kept in the cross-warp reduction buffer
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

  // producer and consumers walk the same sequence of stages (never across a tile boundary)
  int tile = static_cast<int>(b_begin / p.kb_per_tile);
  int kb0 = static_cast<int>(b_begin % p.kb_per_tile);
  int64_t b = b_begin;
  int slot = 0;
  uint32_t phase = 0;
  auto stage_len = [&]() {
    int nkb = p.kb_per_tile - kb0;
    if (nkb > kStageKBlocks) nkb = kStageKBlocks;
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
    if (++slot == p.stages) {
      slot = 0;
      phase ^= 1;
    }
  };

  if (warp == kConsumerWarps) {
    // ------------------------------ producer warp ------------------------------------
    while (b < b_end) {
      const int nkb = stage_len();
      uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
      if (lane == 0) {
        mbar_wait(&hdr->empty[slot], phase ^ 1, abort_flag, p.status, 1);
        const int g0 = kb0 >> p.kbpg_shift;
        const int ng = ((kb0 + nkb - 1) >> p.kbpg_shift) - g0 + 1;
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
      advance(nkb);
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

  int seg_kb0 = kb0;
  bool first_segment = true;
  int pend_tile = -1;     // first partial segment whose arrival count is looked at at the end
  unsigned pend_old = 0;  // (thread 0) what the arrival atomic returned

  // bias, rounding and the fused post-op for one (row, token) of tile `tl`
  auto epilogue = [&](int tl, int row, int tok, float r) {
    const int n = decode_row_to_n(p, tl, row);
    if (tok >= p.m || n >= p.n) return;
    if (p.bias) r += p.bias[n];
    r = bf16_round(r);
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
  };

  // thread -> (row, tokens q*4 + tid/64): finish tile `tl` from the values v[] (or, for a
  // split tile, from the contributors' partial tiles summed in CTA order)
  auto finish_tile = [&](int tl, bool from_partials, float (&v)[NTOK / 4]) {
    const int row = tid & 63;
    if (from_partials) {
      const int64_t tb0 = static_cast<int64_t>(tl) * p.kb_per_tile;
      const int c_first = owner_of(tb0, total, gridDim.x);
      const int c_last = owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
#pragma unroll
      for (int q = 0; q < NTOK / 4; ++q) v[q] = 0.f;
      for (int c = c_first; c <= c_last; ++c) {
        const int64_t cb = (static_cast<int64_t>(c) * total) / gridDim.x;
        const float* src =
            p.partials + static_cast<size_t>(c * 2 + (cb >= tb0 ? 0 : 1)) * (16 * kTileN);
#pragma unroll
        for (int q = 0; q < NTOK / 4; ++q) {
          const int tok = q * 4 + (tid >> 6);
          if (tok < p.m) v[q] += __ldcg(src + tok * kTileN + row);
        }
      }
    }
    if (p.fusion == FUSE_SILU_MUL) {
      // rows 0..31 of the tile are gate rows, rows 32..63 the matching up rows
      float* fin = red;
#pragma unroll
      for (int q = 0; q < NTOK / 4; ++q) {
        const int tok = q * 4 + (tid >> 6);
        if (tok < red_tok) {
          const int n = decode_row_to_n(p, tl, row);
          float r = v[q];
          if (n < p.n && p.bias) r += p.bias[n];
          fin[tok * kRedTokStride + row] = bf16_round(r);
        }
      }
      named_bar_sync(1, kConsumerThreads);
      if (row < 32) {
        const int col = tl * 32 + row;
#pragma unroll
        for (int q = 0; q < NTOK / 4; ++q) {
          const int tok = q * 4 + (tid >> 6);
          if (tok < p.m && col < p.n_out) {
            const float gate = fin[tok * kRedTokStride + row];
            const float up = fin[tok * kRedTokStride + row + 32];
            p.y[static_cast<size_t>(tok) * p.ldy + col] = __float2bfloat16_rn(up * silu_bf16(gate));
          }
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < NTOK / 4; ++q) epilogue(tl, row, q * 4 + (tid >> 6), v[q]);
    }
  };

  // end of a tile segment [seg_kb0, seg_kb1) of tile `tl`; `more` = this CTA has more work
  auto flush = [&](int tl, int seg_kb1, bool more) {
    // 1. this warp's partial sums -> red[warp][tok][row]
    float* my = red + warp * (red_tok * kRedTokStride);
#pragma unroll
    for (int rt = 0; rt < 4; ++rt)
#pragma unroll
      for (int tb = 0; tb < TB; ++tb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = rt * 16 + (i >> 1) * 8 + g;
          const int tok = tb * 8 + 2 * t + (i & 1);
          if (tok < red_tok) my[tok * kRedTokStride + row] = acc[rt][tb][i];
          acc[rt][tb][i] = 0.f;
        }
    named_bar_sync(1, kConsumerThreads);
    // 2. sum over the warps
    const int row = tid & 63;
    float v[NTOK / 4];
#pragma unroll
    for (int q = 0; q < NTOK / 4; ++q) {
      const int tok = q * 4 + (tid >> 6);
      float s = 0.f;
      if (tok < red_tok) {
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w)
          s += red[w * (red_tok * kRedTokStride) + tok * kRedTokStride + row];
      }
      v[q] = s;
    }
    const bool whole = (seg_kb0 == 0 && seg_kb1 == p.kb_per_tile);
    if (whole) {
      if (p.fusion == FUSE_SILU_MUL) named_bar_sync(1, kConsumerThreads);  // red is reused
      finish_tile(tl, false, v);
    } else {
      // partial: park it in the workspace, the last contributor to arrive reduces
      const int my_slot = blockIdx.x * 2 + (first_segment ? 0 : 1);
      float* dst = p.partials + static_cast<size_t>(my_slot) * (16 * kTileN);
#pragma unroll
      for (int q = 0; q < NTOK / 4; ++q) {
        const int tok = q * 4 + (tid >> 6);
        if (tok < p.m) __stcg(dst + tok * kTileN + row, v[q]);
      }
      named_bar_sync(1, kConsumerThreads);
      if (first_segment && more) {
        if (tid == 0) {
          __threadfence();
          pend_old = atomicAdd(p.counters + tl, 1u);
        }
        pend_tile = tl;
      } else {
        if (tid == 0) {
          const int64_t tb0 = static_cast<int64_t>(tl) * p.kb_per_tile;
          const int c_first = owner_of(tb0, total, gridDim.x);
          const int c_last = owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
          __threadfence();
          const unsigned old = atomicAdd(p.counters + tl, 1u);
          const int last = (old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
          if (last) p.counters[tl] = 0;
          hdr->is_last = last;
        }
        named_bar_sync(1, kConsumerThreads);
        if (hdr->is_last) {
          __threadfence();
          finish_tile(tl, true, v);
        }
      }
    }
    named_bar_sync(1, kConsumerThreads);  // red and is_last are free again
    first_segment = false;
  };

  while (b < b_end) {
    const int nkb = stage_len();
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
      const int gl = (kb >> p.kbpg_shift) - (kb0 >> p.kbpg_shift);
      const uint4* sp =
          reinterpret_cast<const uint4*>(st + kStageKBlocks * kBlockBytes + gl * 256 + g * 32);
      const uint4 s_lo = sp[0], s_hi = sp[1];
      const uint32_t szw[8] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w, s_hi.x, s_hi.y, s_hi.z, s_hi.w};

      if constexpr (EXACT) {
        // bf16((q - zp) * bf16 scale) per weight, exactly the reference's tile dequantiser;
        // the MMAs accumulate straight into the running sums
        uint32_t zz[8], ss[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          zz[i] = __byte_perm(szw[i], 0, 0x1010);
          ss[i] = __byte_perm(szw[i], 0, 0x3232);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int rt = 0; rt < 4; ++rt) {
            const uint32_t w = (j == 0) ? wv[rt].x : (j == 1) ? wv[rt].y : (j == 2) ? wv[rt].z : wv[rt].w;
            uint32_t a[4];
            a[0] = bf16x2_mul(bf16x2_sub(lop3_and_or(w, 0x000f000fu, kBf16Magic), zz[rt * 2]), ss[rt * 2]);
            a[1] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 4, 0x000f000fu, kBf16Magic), zz[rt * 2 + 1]), ss[rt * 2 + 1]);
            a[2] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 8, 0x000f000fu, kBf16Magic), zz[rt * 2]), ss[rt * 2]);
            a[3] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 12, 0x000f000fu, kBf16Magic), zz[rt * 2 + 1]), ss[rt * 2 + 1]);
#pragma unroll
            for (int tb = 0; tb < TB; ++tb)
              mma_bf16_16816(acc[rt][tb], a, xb[tb][2 * j], xb[tb][2 * j + 1]);
          }
        }
      } else {
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
          for (int tb = 0; tb < TB; ++tb)
            mma_bf16_16816(sx[tb], ones, xb[tb][2 * j], xb[tb][2 * j + 1]);
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
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&hdr->empty[slot]);
    const bool seg_end = (kb0 + nkb == p.kb_per_tile) || (b + nkb == b_end);
    if (seg_end) flush(tile, kb0 + nkb, b + nkb < b_end);
    advance(nkb);
    if (seg_end) seg_kb0 = kb0;
  }
  if (pend_tile >= 0) {
    if (tid == 0) {
      const int64_t tb0 = static_cast<int64_t>(pend_tile) * p.kb_per_tile;
      const int c_first = owner_of(tb0, total, gridDim.x);
      const int c_last = owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
      const int last = (pend_old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
      if (last) p.counters[pend_tile] = 0;
      hdr->is_last = last;
    }
    named_bar_sync(1, kConsumerThreads);
    if (hdr->is_last) {
      __threadfence();
      float v[NTOK / 4];
      finish_tile(pend_tile, true, v);
    }
  }
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
  p.x_rows = p.m;
  p.red_tok = (p.m + 1) & ~1;
  const int stage_bytes = kStageKBlocks * kBlockBytes + (p.gps + 1) * 256 + p.x_rows * kXRowBytes;
  const int red_bytes = kConsumerWarps * p.red_tok * kRedTokStride * 4;
  const int budget = (tb == 1 ? 112 : 224) * 1024;
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
  void (*kern)(const DecodeParams) =
      tb == 1 ? (p.exact ? woq_int4_decode_kernel<1, true> : woq_int4_decode_kernel<1, false>)
              : (p.exact ? woq_int4_decode_kernel<2, true> : woq_int4_decode_kernel<2, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  kern<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace woq
