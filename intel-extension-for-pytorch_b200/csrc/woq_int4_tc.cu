// INT4 weight-only-quantised GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for
// any token count up to 256 per launch.
//
// Orientation: the weight is the A operand (128 output rows = the 128 TMEM lanes), the
// activations are the B operand (N = tokens, 16..256), so one CTA tile is y^T[128 rows x
// tokens] accumulated in fp32 in TMEM over the whole K of its share.
//
//   warp 16     producer: bulk copies of packed nibbles + group scales;
//   warp 17     producer: TMA tile loads of x (128-byte swizzled K-major rows) - all copies
//               complete on mbarriers;
//   warps 0-15  dequantise: thread = output row.  Two 128-bit shared loads give the row's 64
//               nibbles of a k-block; each becomes bf16((q - zp) * bf16(scale)) exactly (the
//               reference's tile dequantiser) and the 32 packed registers go straight to
//               TMEM with one tcgen05.st - the dequantised tile never touches shared memory.
//               Consecutive stages go round-robin to the four warpgroups;
//   warps 18,19 one thread each issues tcgen05.mma (A from TMEM, B from shared memory) for
//               alternate stages: per stage one wait (the A group is written and the x
//               tiles have landed) and one tcgen05.commit that frees the stage's buffers and
//               its A group together;
//   warps 0-15  epilogue at the end of a tile segment: tcgen05.ld the accumulators, then
//               either the fused post-op and store, or - when the CTA saw only part of K -
//               a partial tile in the workspace that the last contributor sums in a fixed
//               order.
// Scalar bookkeeping is what the single-thread roles and the stage hand-overs are made of, and a
// lone thread gets through only one dependent instruction every 10-15 cycles beside sixteen busy
// warps.  So every role keeps its own few 32-bit counters (k-blocks left in the tile and in the
// CTA's share, ring slot and parity), and a dequantising warpgroup steps from one of its stages
// straight to the next one, four stages on, instead of walking the stages between.
// Two rings.  The packed weights travel through a shared-memory ring of up to 32 slots that
// the dequantising warps free as soon as they have the nibbles in registers; the dequantised
// A groups (TMEM) and the activation tiles form a second, shorter ring freed by the MMAs'
// commit.  The accumulator takes as many TMEM columns as there are token columns (rounded to
// 32), the A groups all the others: 8 groups beside a 256-column accumulator, 14 beside a
// 64-column one.  Weight bytes in flight per SM are bounded by shared memory (about 100 KB
// and more for up to 128 tokens), not by TMEM.
// Work split: the (tile, k-block) sequence is cut into equal contiguous shares, one per SM.
#include "woq_kernels.h"
#include "woq_tc_common.cuh"

namespace woq {

namespace {

constexpr int kDequantWarps = 16;
constexpr int kWarpGroups = kDequantWarps / 4;
constexpr int kIssuers = 2;  // threads that issue MMAs, each in a warp of its own
constexpr int kTcThreads = (kDequantWarps + 2 + kIssuers) * 32;
constexpr int kProducerWarp = kDequantWarps, kXProducerWarp = kDequantWarps + 1, kMmaWarp = kDequantWarps + 2;
constexpr int kDCol0 = 0;            // accumulator columns [0, a_col0)
constexpr int kTmemCols = 512;       // A groups (32 columns = one k-block of bf16 A) fill the rest
constexpr int kMaxTcStages = 16;     // A-group / activation ring
constexpr int kMaxWRing = 32;        // packed-weight ring
constexpr int kTcHeaderBytes = 1024;

struct TcHeader {
  uint64_t w_full[kMaxWRing];     // packed weights + scales of the weight-ring slot have landed
  uint64_t w_free[kMaxWRing];     // the four dequantising warps have read the slot
  uint64_t full[kMaxTcStages];    // A group written (4 warps) and x tiles landed (1 + bytes)
  uint64_t free_[kMaxTcStages];   // the stage's MMAs have completed: A group and x tiles may be reused
  uint64_t issued[kIssuers];      // MMA thread t has issued the MMAs of its latest stage
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

// Eight tokens (chunk ch) of one row: the fused operands of all eight are loaded before the
// first is used (raw bits, converted at use), so the chunk costs one global round trip, not
// one per token.  The scatter epilogue keeps the per-token routine (its rows come from a table).
__device__ __forceinline__ void tc_store8(const TcParams& p, int tile, int row, int ch, const float* v) {
  const bool binary = p.fusion == FUSE_ADD || p.fusion == FUSE_ADD_ADD || p.fusion == FUSE_MUL;
  const int n = tc_row_to_n(p, tile, row);
  if (!binary || n >= p.n) {
#pragma unroll
    for (int e = 0; e < 8; ++e) tc_store(p, tile, row, ch * 8 + e, v[e]);
    return;
  }
  const unsigned short* o0 = reinterpret_cast<const unsigned short*>(p.other0);
  const unsigned short* o1 = reinterpret_cast<const unsigned short*>(p.other1);
  uint32_t f[8], g[8];
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (ch * 8 + e < p.m) {
      const size_t o = static_cast<size_t>(ch * 8 + e) * p.ldy + n;
      f[e] = o0[o];
      if (p.fusion == FUSE_ADD_ADD) g[e] = o1[o];
    }
  const float b = p.bias ? p.bias[n] : 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (ch * 8 + e < p.m) {
      float r = v[e];
      if (p.bias) r += b;
      r = bf16_round(r);
      const float a = __uint_as_float(f[e] << 16);
      if (p.fusion == FUSE_MUL) {
        r = bf16_round(r * a);
      } else {
        r = bf16_round(r + a);
        if (p.fusion == FUSE_ADD_ADD) r = bf16_round(r + __uint_as_float(g[e] << 16));
      }
      p.y[static_cast<size_t>(ch * 8 + e) * p.ldy + n] = __float2bfloat16_rn(r);
    }
}

__global__ void __launch_bounds__(kTcThreads, 1)
    woq_int4_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap xmap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  TcHeader* hdr = reinterpret_cast<TcHeader*>(smem);
  const int x_stage_bytes = p.kbs * p.n_tok * 128;
  const int w_stage_bytes = p.kbs * kTcBlockBytes + (p.kbs + 1) * 512;
  uint8_t* x_stages = smem + kTcHeaderBytes;
  uint8_t* w_stages = x_stages + static_cast<size_t>(p.stages) * x_stage_bytes;

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
      mbar_init(&hdr->full[s], 5);
      mbar_init(&hdr->free_[s], 1);
    }
    for (int s = 0; s < p.w_ring; ++s) {
      mbar_init(&hdr->w_full[s], 1);
      mbar_init(&hdr->w_free[s], 4);
    }
    for (int t = 0; t < kIssuers; ++t) mbar_init(&hdr->issued[t], 1);
    mbar_init(&hdr->d_full, kIssuers);
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
  // No programmatic dependent launch for this kernel (measured: 2-3 us per launch from the weights
  // prefetched and TMEM allocated while the previous kernel drained; not kept).
  const uint32_t tmem_base = hdr->tmem_base;
  volatile int* abort_flag = &hdr->abort_flag;

  // Every role walks the same sequence of stages; a stage is up to `kbs` k-blocks of one tile and
  // never crosses a tile end or the end of the CTA's share.  Stage number s uses slot s % stages
  // of the A-group / activation ring (shared-memory tiles and kbs * 32 TMEM columns) and slot
  // s % w_ring of the packed-weight ring.
  const int kbpt = p.kb_per_tile, kbs = p.kbs, n_stages = p.stages, n_wring = p.w_ring;
  const int tile0 = static_cast<int>(b_begin / kbpt);
  const int kb00 = static_cast<int>(b_begin % kbpt);
  const int rem0 = static_cast<int>(b_end - b_begin);

  if (warp == kProducerWarp) {
    // packed weights and their group scales
    if (lane == 0) {
      int tile = tile0, kb0 = kb00, rem = rem0, wslot = 0;
      uint32_t wphase = 0;
      while (rem > 0) {
        int nkb = kbpt - kb0;
        if (nkb > kbs) nkb = kbs;
        if (nkb > rem) nkb = rem;
        uint8_t* ws = w_stages + static_cast<size_t>(wslot) * w_stage_bytes;
        const int g0 = kb0 >> p.kbpg_shift;
        const int ng = ((kb0 + nkb - 1) >> p.kbpg_shift) - g0 + 1;
        mbar_wait(&hdr->w_free[wslot], wphase ^ 1, abort_flag, p.status, 11);
        mbar_arrive_expect_tx(&hdr->w_full[wslot], nkb * kTcBlockBytes + ng * 512);
        bulk_g2s(ws, p.wq + (static_cast<size_t>(tile) * kbpt + kb0) * kTcBlockBytes,
                 nkb * kTcBlockBytes, &hdr->w_full[wslot]);
        bulk_g2s(ws + kbs * kTcBlockBytes,
                 p.sz + (static_cast<size_t>(tile) * p.groups + g0) * kTcTileN, ng * 512,
                 &hdr->w_full[wslot]);
        kb0 += nkb;
        rem -= nkb;
        if (kb0 == kbpt) {
          kb0 = 0;
          ++tile;
        }
        if (++wslot == n_wring) {
          wslot = 0;
          wphase ^= 1;
        }
      }
    }
  } else if (warp == kXProducerWarp) {
    // activation tiles (TMA, 128-byte swizzle), one per k-block
    if (lane == 0) {
      int kb0 = kb00, rem = rem0, slot = 0;
      uint32_t phase = 0;
      while (rem > 0) {
        int nkb = kbpt - kb0;
        if (nkb > kbs) nkb = kbs;
        if (nkb > rem) nkb = rem;
        uint8_t* xs = x_stages + static_cast<size_t>(slot) * x_stage_bytes;
        mbar_wait(&hdr->free_[slot], phase ^ 1, abort_flag, p.status, 12);
        mbar_arrive_expect_tx(&hdr->full[slot], nkb * p.n_tok * 128);
        for (int j = 0; j < nkb; ++j)
          tma_load_2d(xs + j * p.n_tok * 128, &xmap, (kb0 + j) * kBlockK, p.m0, &hdr->full[slot]);
        kb0 += nkb;
        rem -= nkb;
        if (kb0 == kbpt) kb0 = 0;
        if (++slot == n_stages) {
          slot = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp >= kMmaWarp) {
    if (lane == 0) {
      // The issuing threads take the stages in turn.  Issuing an MMA blocks the thread while the
      // tensor core is busy, and the waits, the commit and the bookkeeping around a stage cost
      // about as much again; with two threads one of them has finished its wait when the other
      // has issued its last MMA (one thread alone: 5-25 % slower at every token count).  A token
      // (`issued`) keeps the stages in order, so the MMA that starts a tile's accumulator runs
      // before any that adds to it.
      const int me = warp - kMmaWarp;
      const int before_me = (me + kIssuers - 1) % kIssuers;
      int turn = 0;  // whose stage the current one is
      int mst = 0;   // stage number within this CTA
      const uint32_t idesc = umma_idesc(p.n_tok, /*bf16*/ 1, /*bf16*/ 1, /*f32*/ 1);
      const uint64_t desc_hi = umma_desc_k128(0) & 0xffffffff00000000ull;
      const uint32_t x_base_lo = (smem_u32(x_stages) & 0x3FFFFu) >> 4;
      const uint32_t x_stage_lo = static_cast<uint32_t>(x_stage_bytes) >> 4;
      const uint32_t x_blk_lo = static_cast<uint32_t>(p.n_tok * 128) >> 4;
      const uint32_t d_addr = tmem_base + kDCol0;
      const uint32_t a_base = tmem_base + p.a_col0;
      const uint32_t a_stage = static_cast<uint32_t>(kbs * 32);
      uint32_t seg = 0;
      bool first_of_segment = true;
      int kb0 = kb00, rem = rem0, slot = 0;
      uint32_t phase = 0;
      uint32_t a_addr = a_base, b_lo = x_base_lo;  // of the current slot
      while (rem > 0) {
        int nkb = kbpt - kb0;
        if (nkb > kbs) nkb = kbs;
        if (nkb > rem) nkb = rem;
        if (turn == me) {
          mbar_wait(&hdr->full[slot], phase, abort_flag, p.status, 13);
          if (first_of_segment) mbar_wait(&hdr->d_empty, (seg & 1) ^ 1, abort_flag, p.status, 15);
          // the previous stage's MMAs have been issued (by the thread before this one)
          if (mst > 0) mbar_wait(&hdr->issued[before_me], ((mst - 1) / kIssuers) & 1, abort_flag, p.status, 14);
          tc_fence_after_sync();
          uint32_t accumulate = first_of_segment ? 0u : 1u;
          uint32_t a = a_addr, bl = b_lo;
          for (int j = 0; j < nkb; ++j) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              umma_f16_ts(d_addr, a + ks * 8, desc_hi | (bl + ks * 2), idesc, accumulate);
              accumulate = 1;
            }
            a += 32;
            bl += x_blk_lo;
          }
          mbar_arrive(&hdr->issued[me]);
          tc_commit(&hdr->free_[slot]);
        }
        kb0 += nkb;
        rem -= nkb;
        first_of_segment = false;
        if (kb0 == kbpt || rem == 0) {
          // Segment end, every issuing thread: what this thread issued for the segment is
          // tracked.  A thread that does not own the segment's last stage first waits until that
          // stage has been issued: otherwise it could run on through a following short segment
          // and arrive on d_full a second time before the owner's arrival for this one.
          if (turn != me) mbar_wait(&hdr->issued[turn], (mst / kIssuers) & 1, abort_flag, p.status, 14);
          tc_commit(&hdr->d_full);
          ++seg;
          first_of_segment = true;
          if (kb0 == kbpt) kb0 = 0;
        }
        ++mst;
        if (++turn == kIssuers) turn = 0;
        a_addr += a_stage;
        b_lo += x_stage_lo;
        if (++slot == n_stages) {
          slot = 0;
          phase ^= 1;
          a_addr = a_base;
          b_lo = x_base_lo;
        }
      }
    }
  } else {
    // --------------------------- dequantise + epilogue warps -----------------------------
    const int wg = warp >> 2, q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int n_chunks = p.n_tok / 8;  // 8-token column chunks, dealt round-robin to warpgroups
    // accumulators of this segment summed in a fixed order
    auto load_acc = [&](int ch, int n_used, float (&v)[8]) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
      for (int a = 0; a < n_used; ++a) {
        uint32_t t[8];
        tmem_ld_x8(lane_addr + kDCol0 + a * p.n_tok + ch * 8, t);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += __uint_as_float(t[e]);
      }
    };
    int seg = 0;
    bool first_segment = true;
    // a first segment that is partial is reduced at the very end if this CTA turns out to be
    // the last contributor; `pend_old` (thread 0) is the arrival count the atomic returned
    int pend_tile = -1;
    unsigned pend_old = 0;

    // sum the contributors' partial tiles of `t` in CTA order and run the epilogue
    auto reduce_and_store = [&](int t, bool whole, int own_slot) {
      const int64_t tb0 = static_cast<int64_t>(t) * p.kb_per_tile;
      const int c_first = tc_owner_of(tb0, total, gridDim.x);
      const int c_last = tc_owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
      for (int ch = wg; ch < n_chunks; ch += kWarpGroups) {
        if (ch * 8 >= p.m) break;
        // eight tokens at a time, all their loads in flight together
        float v[8], v_up[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v_up[e] = 0.f;
        for (int cc = c_first; cc <= c_last; ++cc) {
          const int64_t cb = (static_cast<int64_t>(cc) * total) / gridDim.x;
          const int slot2 = whole ? own_slot : cc * 2 + (cb >= tb0 ? 0 : 1);
          const float* src = p.partials + static_cast<size_t>(slot2) * p.n_tok * kTcTileN +
                             static_cast<size_t>(ch * 8) * kTcTileN + row;
          float part[8], part_up[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            part[e] = __ldcg(src + e * kTcTileN);
            part_up[e] = (p.fusion == FUSE_SILU_MUL && row < 64) ? __ldcg(src + e * kTcTileN + 64) : 0.f;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            v[e] += part[e];
            v_up[e] += part_up[e];
          }
        }
        if (p.fusion != FUSE_SILU_MUL) {
          tc_store8(p, t, row, ch, v);
          continue;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int tok = ch * 8 + e;
          if (tok >= p.m) break;
          {
            if (row < 64) {
              const int n_gate = t * 64 + row, n_up = p.n / 2 + n_gate;
              float g = v[e], u = v_up[e];
              if (p.bias) {
                g += p.bias[n_gate];
                u += p.bias[n_up];
              }
              const float gate = bf16_round(g), up = bf16_round(u);
              if (n_gate < p.n_out)
                p.y[static_cast<size_t>(tok) * p.ldy + n_gate] =
                    __float2bfloat16_rn(up * silu_bf16(gate));
            }
          }
        }
      }
    };

    // Segment by segment (a segment = the CTA's k-blocks of one tile).  The segment's stages
    // have the global numbers st .. st + ns - 1; this warpgroup takes those equal to wg modulo
    // four and keeps the ring positions of its next stage (both rings have at least four
    // slots, so a step of four wraps at most once).
    int tile = tile0, seg_kb0 = kb00, rem = rem0;
    int st = 0, own = wg;
    int slot = wg, wslot = wg;
    uint32_t phase = 0, wphase = 0;
    while (rem > 0) {
      int seg_len = kbpt - seg_kb0;
      if (seg_len > rem) seg_len = rem;
      const int ns = (seg_len + kbs - 1) / kbs;
      const int seg_kb1 = seg_kb0 + seg_len;
      for (; own < st + ns; own += kWarpGroups) {
        const int kb0 = seg_kb0 + (own - st) * kbs;
        int nkb = seg_kb1 - kb0;
        if (nkb > kbs) nkb = kbs;
        const uint8_t* ws = w_stages + static_cast<size_t>(wslot) * w_stage_bytes;
        mbar_wait(&hdr->w_full[wslot], wphase, abort_flag, p.status, 16);
        const int g0 = kb0 >> p.kbpg_shift;
        for (int j = 0; j < nkb; ++j) {
          const uint4* wp = reinterpret_cast<const uint4*>(ws + j * kTcBlockBytes);
          const uint4 v0 = wp[row], v1 = wp[kTcTileN + row];
          const uint32_t szw = reinterpret_cast<const uint32_t*>(
              ws + kbs * kTcBlockBytes)[(((kb0 + j) >> p.kbpg_shift) - g0) * kTcTileN + row];
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
          if (j == nkb - 1) {
            // the values of the weight slot's last k-block have been used: the slot is free
            __syncwarp();
            if (lane == 0) mbar_arrive(&hdr->w_free[wslot]);
          }
          if (j == 0) {
            mbar_wait(&hdr->free_[slot], phase ^ 1, abort_flag, p.status, 17);
            tc_fence_after_sync();
          }
          // the lanes may leave a wait loop or the one-lane arrive above apart; the TMEM store is
          // a warp-wide instruction
          __syncwarp();
          tmem_st_x32(lane_addr + p.a_col0 + slot * (kbs * 32) + j * 32, r);
        }
        tc_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->full[slot]);
        slot += kWarpGroups;
        if (slot >= n_stages) {
          slot -= n_stages;
          phase ^= 1;
        }
        wslot += kWarpGroups;
        if (wslot >= n_wring) {
          wslot -= n_wring;
          wphase ^= 1;
        }
      }
      st += ns;

      {
        const bool whole = (seg_kb0 == 0 && seg_len == kbpt);
        const bool more = rem > seg_len;  // this CTA goes on to another tile
        const int n_used = 1;
        mbar_wait(&hdr->d_full, seg & 1, abort_flag, p.status, 18);
        tc_fence_after_sync();
        __syncwarp();  // the TMEM loads below are warp-wide instructions
        if (whole && p.fusion != FUSE_SILU_MUL) {
          for (int ch = wg; ch < n_chunks; ch += kWarpGroups) {
            float v[8];
            load_acc(ch, n_used, v);
            tc_store8(p, tile, row, ch, v);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->d_empty);
        } else {
          // park this CTA's contribution in the workspace (also pairs gate / up rows)
          const int my_slot = blockIdx.x * 2 + (first_segment ? 0 : 1);
          float* dst = p.partials + static_cast<size_t>(my_slot) * p.n_tok * kTcTileN;
          for (int ch = wg; ch < n_chunks; ch += kWarpGroups) {
            float v[8];
            load_acc(ch, n_used, v);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (ch * 8 + e < p.m)
                __stcg(dst + static_cast<size_t>(ch * 8 + e) * kTcTileN + row, v[e]);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->d_empty);
          named_bar_sync(1, kDequantWarps * 32);
          const bool defer = !whole && first_segment && more;
          if (defer) {
            // more tiles follow: count the arrival now, look at the answer when all work is done
            if (tid == 0) {
              __threadfence();
              pend_old = atomicAdd(p.counters + tile, 1u);
            }
            pend_tile = tile;
          } else {
            if (tid == 0) {
              int last = 1;
              if (!whole) {
                const int64_t tb0 = static_cast<int64_t>(tile) * p.kb_per_tile;
                const int c_first = tc_owner_of(tb0, total, gridDim.x);
                const int c_last = tc_owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
                __threadfence();
                const unsigned old = atomicAdd(p.counters + tile, 1u);
                last = (old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
                if (last) p.counters[tile] = 0;
              }
              hdr->is_last = last;
            }
            named_bar_sync(1, kDequantWarps * 32);
            if (hdr->is_last) {
              __threadfence();
              reduce_and_store(tile, whole, my_slot);
            }
            named_bar_sync(1, kDequantWarps * 32);
          }
        }
        ++seg;
        first_segment = false;
      }
      rem -= seg_len;
      seg_kb0 = seg_kb1;
      if (seg_kb0 == kbpt) {
        seg_kb0 = 0;
        ++tile;
      }
    }
    if (pend_tile >= 0) {
      if (tid == 0) {
        const int64_t tb0 = static_cast<int64_t>(pend_tile) * p.kb_per_tile;
        const int c_first = tc_owner_of(tb0, total, gridDim.x);
        const int c_last = tc_owner_of(tb0 + p.kb_per_tile - 1, total, gridDim.x);
        const int last = (pend_old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
        if (last) p.counters[pend_tile] = 0;
        hdr->is_last = last;
      }
      named_bar_sync(1, kDequantWarps * 32);
      if (hdr->is_last) {
        __threadfence();
        reduce_and_store(pend_tile, false, 0);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    __syncwarp();  // lane 0 comes from the issuing loop
    tmem_dealloc(tmem_base, kTmemCols);
  }
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

// Pipeline shape of a launch with `n_tok` token columns (a multiple of 16, at most 256): fills
// a_col0, kbs, stages and w_ring of `p` and returns the dynamic shared memory in bytes, or 0 when
// no valid shape exists.
size_t tc_plan(TcParams& p) {
  // TMEM: the accumulator takes the token columns (rounded to 32), the A groups the rest.
  p.a_col0 = (p.n_tok + 31) & ~31;
  const int a_groups = (kTmemCols - p.a_col0) / 32;
  // k-blocks per stage.  Every stage costs each role a fixed amount of scalar bookkeeping and
  // barrier traffic, whatever the stage holds, so up to 128 tokens, where the MMAs of one k-block
  // are short, a stage takes as many k-blocks as the rings allow: three up to 64 tokens (four or
  // five A groups of three), two up to 128 (four activation slots of 32 KB).
  p.kbs = p.n_tok <= 64 ? 3 : p.n_tok <= 128 ? 2 : 1;
  const int x_stage = p.kbs * p.n_tok * 128;
  const int w_stage = p.kbs * kTcBlockBytes + (p.kbs + 1) * 512;
  const int budget = 224 * 1024 - kTcHeaderBytes;
  int stages, w_ring;
  if (p.n_tok > 128) {
    // a launch this wide is bound by the dequantising warps and the tensor core, not by bytes
    // in flight: one ring length for both
    stages = budget / (x_stage + w_stage);
    if (stages > a_groups / p.kbs) stages = a_groups / p.kbs;
    w_ring = stages;
  } else {
    // A-group ring as long as TMEM allows within half of the shared memory; the packed weights
    // get what is left
    stages = a_groups / p.kbs;
    if (stages > kMaxTcStages) stages = kMaxTcStages;
    while (stages > 4 && stages * x_stage > budget / 2) --stages;
    w_ring = (budget - stages * x_stage) / w_stage;
    if (w_ring > kMaxWRing) w_ring = kMaxWRing;
  }
  // A parity wait cannot tell a barrier that is one completion short from one that is three
  // short, so whoever waits for use u of a slot must know that use u - 1 has completed.
  //  - A group / activation ring: a warpgroup works on every fourth stage and reaches stage s only
  //    after stage s - 4, whose wait covered the MMAs of stage s - 4 - stages; the MMAs complete in
  //    order, so with at least four slots the previous use (stage s - stages) has completed.
  //  - packed-weight ring: nothing orders the landing of one stage's weights against a warpgroup
  //    that works on other stages, so its length is a multiple of four: every slot then belongs to
  //    one warpgroup, which has itself waited for the slot's previous use.  (A ring of six beside
  //    four warpgroups let a warpgroup find, about once in a thousand 256-token launches, a slot
  //    whose previous load had not landed yet: it read the use before that, released the slot
  //    early, and the launch ended in a time-out or a launch failure.)
  w_ring &= ~3;
  if (stages < 4 || w_ring < 4) return 0;
  p.w_ring = w_ring;
  p.stages = stages;
  return kTcHeaderBytes + static_cast<size_t>(stages) * x_stage + static_cast<size_t>(w_ring) * w_stage;
}

cudaError_t launch_int4_tc(TcParams p, const CUtensorMap& xmap, int grid, cudaStream_t stream) {
  const size_t smem = tc_plan(p);
  if (smem == 0) return cudaErrorInvalidConfiguration;
  cudaError_t e = cudaFuncSetAttribute(woq_int4_tc_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  woq_int4_tc_kernel<<<grid, kTcThreads, smem, stream>>>(p, xmap);
  return cudaGetLastError();
}

}  // namespace woq
