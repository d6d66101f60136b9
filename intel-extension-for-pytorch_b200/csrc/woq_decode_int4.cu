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
constexpr int kProducerWarp = kConsumerWarps, kFirstEpilogueWarp = kConsumerWarps + 1;
// Epilogue warps take tile segments round-robin, so the global-memory round trips of one
// segment's partial-tile protocol overlap the next segment's.
__host__ __device__ constexpr int epilogue_warps(int tb) { return tb == 1 ? 3 : 4; }
__host__ __device__ constexpr int block_threads(int tb) {
  return (kConsumerWarps + 1 + epilogue_warps(tb)) * 32;
}
// named barriers: 1 + e "segment for epilogue warp e is in shared memory", 5 + e "... is drained"
constexpr int kBarRedFull = 1, kBarRedFree = 5;
constexpr int kStageKBlocks = kConsumerWarps;                 // k-blocks per stage
constexpr int kXRowBytes = kStageKBlocks * kBlockK * 2 + 16;  // +16: bank spread between tokens
constexpr int kRedTokStride = 68;                             // floats; conflict-free scatter
constexpr int kHeaderBytes = 1024;
constexpr int kMaxStages = 8;

struct SmemHeader {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  int abort_flag;
};

__device__ __forceinline__ int owner_of(int64_t b, int64_t total, int64_t ctas) {
  // CTA c owns k-blocks [c*total/ctas, (c+1)*total/ctas)
  return static_cast<int>(((b + 1) * ctas - 1) / total);
}

// bias, rounding and the fused post-op for one (row, token) of tile `tl`
__device__ __forceinline__ void decode_epilogue(const DecodeParams& p, int tl, int row, int tok, float r) {
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
}

// The stages a CTA walks: its share [b_begin, b_end) of the k-block sequence cut at tile
// boundaries ("segments") and then into runs of up to kStageKBlocks k-blocks.  Producer and
// consumers step through the same sequence.
struct StageIter {
  int tile, kb, k1, left, kbpt;  // current tile, next k-block, segment end, k-blocks left
  __device__ StageIter(int tile0, int kb0, int left0, int kbpt0)
      : tile(tile0), kb(kb0), k1(min(kbpt0, kb0 + left0)), left(left0), kbpt(kbpt0) {}
  __device__ bool done() const { return left <= 0; }
  __device__ int nkb() const { return min(kStageKBlocks, k1 - kb); }
  __device__ void next(int n) {
    kb += n;
    left -= n;
    if (kb == k1) {
      if (kb == kbpt) {
        kb = 0;
        ++tile;
      }
      k1 = min(kbpt, kb + left);
    }
  }
};

template <int TB, bool EXACT>
__global__ void __launch_bounds__(block_threads(TB), TB == 1 ? 2 : 1)
    woq_int4_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(smem);
  constexpr int NTOK = 8 * TB;
  constexpr int E = epilogue_warps(TB);
  const int sz_stage_bytes = (p.gps + 1) * 256;
  const int stage_bytes = kStageKBlocks * kBlockBytes + sz_stage_bytes + p.x_rows * kXRowBytes;
  const int red_tok = p.red_tok;  // tokens kept in the cross-warp reduction buffer
  uint8_t* stages = smem + kHeaderBytes;
  float* red = reinterpret_cast<float*>(stages + static_cast<size_t>(p.stages) * stage_bytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t total = static_cast<int64_t>(p.tiles) * p.kb_per_tile;
  const int64_t b_begin = (static_cast<int64_t>(blockIdx.x) * total) / gridDim.x;
  const int64_t b_end = (static_cast<int64_t>(blockIdx.x + 1) * total) / gridDim.x;
  const int tile0 = static_cast<int>(b_begin / p.kb_per_tile);
  const int kb00 = static_cast<int>(b_begin - static_cast<int64_t>(tile0) * p.kb_per_tile);
  const int share = static_cast<int>(b_end - b_begin);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], kConsumerWarps);
    }
    hdr->abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  // A following launch that opted into programmatic dependent launch may start its weight
  // stream while this grid is still running.
  grid_launch_dependents();
  volatile int* abort_flag = &hdr->abort_flag;

  if (warp == kProducerWarp) {
    // ------------------------------ producer warp ------------------------------------
    // Weights and scales never depend on the previous kernel in the stream, x does: the
    // first pipeline fill issues the weight copies, then waits for the previous grid, then
    // issues the x copies.
    auto issue_weights = [&](const StageIter& it, int slot) {
      const int nkb = it.nkb();
      uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
      const int g0 = it.kb >> p.kbpg_shift;
      const int ng = ((it.kb + nkb - 1) >> p.kbpg_shift) - g0 + 1;
      uint32_t bytes = nkb * kBlockBytes;
      if (!(p.debug & 4)) bytes += ng * 256;
      if (!(p.debug & 2)) bytes += p.m * nkb * (kBlockK * 2);
      mbar_arrive_expect_tx(&hdr->full[slot], bytes);
      bulk_g2s(st, p.wq + (static_cast<size_t>(it.tile) * p.kb_per_tile + it.kb) * kBlockBytes,
               nkb * kBlockBytes, &hdr->full[slot]);
      if (!(p.debug & 4))
        bulk_g2s(st + kStageKBlocks * kBlockBytes,
                 p.sz + (static_cast<size_t>(it.tile) * p.groups + g0) * 64, ng * 256,
                 &hdr->full[slot]);
    };
    auto issue_x = [&](const StageIter& it, int slot) {  // lane = token
      if (lane < p.m && !(p.debug & 2)) {
        uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
        bulk_g2s(st + kStageKBlocks * kBlockBytes + sz_stage_bytes + lane * kXRowBytes,
                 p.x + static_cast<size_t>(lane) * p.ldx + static_cast<size_t>(it.kb) * kBlockK,
                 it.nkb() * (kBlockK * 2), &hdr->full[slot]);
      }
    };
    StageIter it(tile0, kb00, share, p.kb_per_tile);
    {
      StageIter fill = it;
      if (lane == 0)
        for (int s = 0; s < p.stages && !fill.done(); ++s) {
          issue_weights(fill, s);
          fill.next(fill.nkb());
        }
      grid_dependency_wait();
      __syncwarp();
      for (int s = 0; s < p.stages && !it.done(); ++s) {
        issue_x(it, s);
        it.next(it.nkb());
      }
    }
    int slot = 0;
    uint32_t phase = 1;  // the slots are on their second use from here on
    while (!it.done()) {
      if (lane == 0) {
        mbar_wait(&hdr->empty[slot], phase ^ 1, abort_flag, p.status, 1);
        if (p.debug & 8)
          mbar_arrive(&hdr->full[slot]);  // experiment: consumers re-read the stale stage
        else
          issue_weights(it, slot);
      }
      __syncwarp();
      if (!(p.debug & 8)) issue_x(it, slot);
      it.next(it.nkb());
      if (++slot == p.stages) {
        slot = 0;
        phase ^= 1;
      }
    }
    return;
  }

  if (warp >= kFirstEpilogueWarp) {
    // ------------------------------ epilogue warps -------------------------------------
    // Take the eight consumer warps' partial sums of a finished tile segment out of shared
    // memory, so the consumers go straight on to the next tile; then either run the fused
    // epilogue or park a partial tile and, if this CTA is the last contributor to arrive,
    // reduce the tile in a fixed order.  Segments go round-robin over the epilogue warps.
    const int me = warp - kFirstEpilogueWarp;
    int turn = 0;
    int tl = tile0, k0 = kb00, left = share;
    bool first_segment = true;
    bool waited = false;
    for (; left > 0; first_segment = false, turn = (turn + 1 == E) ? 0 : turn + 1) {
      const int k1 = min(p.kb_per_tile, k0 + left);
      const bool whole = (k0 == 0 && k1 == p.kb_per_tile);
      const int seg_tile = tl;
      left -= k1 - k0;
      k0 = 0;
      ++tl;
      if (turn != me) continue;
      named_bar_sync(kBarRedFull + me, kConsumerThreads + 32);
      // lane -> rows lane and lane + 32 (in the gate/up layout: a gate row and its up row)
      float v0[NTOK], v1[NTOK];
#pragma unroll
      for (int tok = 0; tok < NTOK; ++tok) {
        float s0 = 0.f, s1 = 0.f;
        if (tok < red_tok) {
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) {
            const float* r = red + w * (red_tok * kRedTokStride) + tok * kRedTokStride;
            s0 += r[lane];
            s1 += r[lane + 32];
          }
        }
        v0[tok] = s0;
        v1[tok] = s1;
      }
      __threadfence_block();
      named_bar_arrive(kBarRedFree + me, kConsumerThreads + 32);
      if (!waited) {
        grid_dependency_wait();  // y, the fused operands and the workspace belong to this grid now
        waited = true;
      }
      bool do_epilogue = whole;
      if (!whole) {
        const int my_slot = blockIdx.x * 2 + (first_segment ? 0 : 1);
        float* dst = p.partials + static_cast<size_t>(my_slot) * (16 * kTileN);
#pragma unroll
        for (int tok = 0; tok < NTOK; ++tok)
          if (tok < p.m) {
            __stcg(dst + tok * kTileN + lane, v0[tok]);
            __stcg(dst + tok * kTileN + lane + 32, v1[tok]);
          }
        __threadfence();
        __syncwarp();
        const int64_t tb0 = static_cast<int64_t>(seg_tile) * p.kb_per_tile;
        const int c_first = owner_of(tb0, total, gridDim.x);
        const int c_last = owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
        unsigned old = 0;
        if (lane == 0) old = atomicAdd(p.counters + seg_tile, 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == static_cast<unsigned>(c_last - c_first)) {
          __threadfence();
#pragma unroll
          for (int tok = 0; tok < NTOK; ++tok) v0[tok] = v1[tok] = 0.f;
          for (int c = c_first; c <= c_last; ++c) {
            const int64_t cb = (static_cast<int64_t>(c) * total) / gridDim.x;
            const float* src =
                p.partials + static_cast<size_t>(c * 2 + (cb >= tb0 ? 0 : 1)) * (16 * kTileN);
#pragma unroll
            for (int tok = 0; tok < NTOK; ++tok)
              if (tok < p.m) {
                v0[tok] += __ldcg(src + tok * kTileN + lane);
                v1[tok] += __ldcg(src + tok * kTileN + lane + 32);
              }
          }
          if (lane == 0) p.counters[seg_tile] = 0;
          do_epilogue = true;
        }
      }
      if (do_epilogue) {
        if (p.fusion == FUSE_SILU_MUL) {
          const int col = seg_tile * 32 + lane;
          const int n_gate = decode_row_to_n(p, seg_tile, lane);
          const int n_up = decode_row_to_n(p, seg_tile, lane + 32);
#pragma unroll
          for (int tok = 0; tok < NTOK; ++tok)
            if (tok < p.m && col < p.n_out) {
              float gate = v0[tok], up = v1[tok];
              if (p.bias) {
                gate += p.bias[n_gate];
                up += p.bias[n_up];
              }
              p.y[static_cast<size_t>(tok) * p.ldy + col] =
                  __float2bfloat16_rn(bf16_round(up) * silu_bf16(bf16_round(gate)));
            }
        } else {
#pragma unroll
          for (int tok = 0; tok < NTOK; ++tok) {
            decode_epilogue(p, seg_tile, lane, tok, v0[tok]);
            decode_epilogue(p, seg_tile, lane + 32, tok, v1[tok]);
          }
        }
      }
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
  int seg = 0;  // segment number modulo E

  // end of a tile segment: hand this warp's partial sums to an epilogue warp and go on
  auto flush = [&](bool first) {
    // the buffer is free once the previous segment's epilogue warp has read it
    if (!first) named_bar_sync(kBarRedFree + (seg == 0 ? E - 1 : seg - 1), kConsumerThreads + 32);
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
    __threadfence_block();
    named_bar_arrive(kBarRedFull + seg, kConsumerThreads + 32);
    seg = (seg + 1 == E) ? 0 : seg + 1;
  };

  StageIter it(tile0, kb00, share, p.kb_per_tile);
  int slot = 0;
  uint32_t phase = 0;
  bool first_flush = true;
  while (!it.done()) {
    const int nkb = it.nkb();
    const int kb0 = it.kb;
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
    if (kb0 + nkb == it.k1) {
      flush(first_flush);
      first_flush = false;
    }
    it.next(nkb);
    if (++slot == p.stages) {
      slot = 0;
      phase ^= 1;
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
  // Programmatic dependent launch: this grid may start streaming weights while the previous
  // kernel in the stream drains (it waits for that kernel before it touches x, y or the
  // workspace).  After a kernel that never signals, or after a copy, this is ordinary ordering.
  static const bool pdl = [] {
    const char* e = getenv("WOQ_B200_PDL");
    return !(e && atoi(e) == 0);
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block_threads(tb));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace woq
