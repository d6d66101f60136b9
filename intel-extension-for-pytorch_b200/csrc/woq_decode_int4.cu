// INT4 weight-only-quantised skinny GEMM for M <= 16 tokens ("decode"): an HBM-bound stream
// of packed weights.
//
// Persistent kernel, two CTAs per SM, ten warps each.  The weight is a
// linear sequence of k-blocks (64 rows x 64 k, 2 KB each, tile-major); CTA c owns an equal
// contiguous share, cut at tile boundaries into "segments".
//   * The producer warp moves 8 or 16 k-blocks of one tile per pipeline stage (weights, their
//     group scales and the matching slice of x) with bulk asynchronous copies that complete
//     on an mbarrier.  Under programmatic dependent launch the first pipeline fill of
//     weights is issued before the previous kernel in the stream has finished; x is not
//     touched until it has.
//   * Eight consumer warps take one or two k-blocks of a stage each.  Default dequantiser:
//     bf16((q - zp) * bf16 scale) per weight, bit for bit the reference's tile dequantiser,
//     as bf16x2 A-fragments of mma.m16n8k16 (x is the B operand, fp32 accumulation).
//     Nibbles at bits 0..3 of a half-word are OR-ed into the mantissa of 128.0 (one lop3);
//     nibbles at bits 4..7 are used in place: masked, the half-word read as bf16 is
//     16 q * 2^-133 exactly, and the scale for those rows is pre-multiplied by 2^129.
//     Fast variant (hint STREAM_FAST): no subtract or multiply per weight.  The tensor core
//     accumulates sum_k x * (128 + q) per k-block for the rows whose nibbles sit at bits 0..3
//     and sum_k x * 16 q 2^-133 for the rows used in place (x enters multiplied by 2^64 so
//     that these products stay normal fp32 numbers); an MMA with an all-ones A-fragment gives
//     sum_k x, and scale and zero point are applied to the sums per k-block.  Five integer
//     instructions per eight weights instead of thirteen integer and bf16 ones.
//   * At the end of a segment the consumers drop their partial sums in shared memory and go
//     on; the epilogue warp adds them.  A CTA that saw the whole K of the tile writes y
//     (bias, rounding, fused post-op); otherwise the partial goes to the workspace and the
//     last contributor to arrive sums all partials in CTA order (results do not depend on
//     timing) and runs the epilogue.  Nobody waits for an arrival count.  The CTA's last
//     segment is taken by the producer warp, idle by then.
// The memory system needs about 2.5 us x 44 GB/s = 110+ KB in flight per SM to stay busy,
// which sets the number of pipeline stages.
//
// Cluster variant (layers with at most two tiles' worth of CTAs per SM): the grid is
// tiles x C CTAs in thread-block clusters of C; the C CTAs of a cluster split the K range of
// one tile, one segment each.  Ranks 1..C-1 push their partial tile into the shared memory
// of rank 0 (st.shared::cluster), one cluster barrier orders the pushes, and rank 0 adds the
// partials in rank order and runs the epilogue: no global partial tiles, no atomics, no
// fences, and nothing to clear in the workspace.
#include <cstdlib>

#include "woq_kernels.h"

namespace woq {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarp = kConsumerWarps, kEpilogueWarp = kConsumerWarps + 1;
constexpr int kThreads = (kConsumerWarps + 2) * 32;
// named barriers: "a segment's partial sums are in shared memory" for the epilogue warp and,
// for a CTA's last segment, for the producer warp; "the buffer has been read"
constexpr int kBarRedFull = 1, kBarRedFullLast = 2, kBarRedFree = 3;
// k-blocks per pipeline stage: each consumer warp takes KPW (1 or 2) adjacent k-blocks
__host__ __device__ constexpr int stage_kblocks(int kpw) { return kConsumerWarps * kpw; }
// bytes of one token's x slice in a stage; +16: bank spread between tokens
__host__ __device__ constexpr int x_row_bytes(int kpw) { return stage_kblocks(kpw) * kBlockK * 2 + 16; }
// how the weights become bf16
enum DequantMode {
  kScaleAfterSum = 0,  // approximate: scale and zero point applied to fp32 sums per k-block
  kExactShift = 1,     // bf16((q - zp) * s) per weight, every nibble shifted down to bit 0
  kExactInPlace = 2    // the same values; nibbles at bits 4..7 are used where they are
};
constexpr int kRedTokStride = 68;                             // floats; conflict-free scatter
constexpr int kHeaderBytes = 1024;
constexpr int kMaxStages = 8;

// What the tile epilogue reads of the launch parameters, copied into shared memory when the
// CTA starts.  The epilogue is a function of its own; handed the kernel parameter by
// reference it would fetch every field through a generic pointer into the parameter bank,
// and the first touch of those lines costs a round trip to device memory (about 2 us per
// epilogue call when measured), on the serial tail of every launch.
struct EpiParams {
  const float* bias;
  __nv_bfloat16* y;
  const __nv_bfloat16* other0;
  const __nv_bfloat16* other1;
  const int32_t* row_idx;
  const __nv_bfloat16* row_w;
  int* status;
  int64_t ldy, ldo;
  int m, n, n_out, fusion, gate_up;
  CommParams comm;
};

struct SmemHeader {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  int abort_flag;
  int finished_warps;  // of the two warps that run epilogues
  EpiParams epi;
};
static_assert(sizeof(SmemHeader) <= kHeaderBytes, "shared-memory header");

// The k-block sequence is dealt out in units of `unit` k-blocks: CTA c owns units
// [c*units/ctas, (c+1)*units/ctas).
__device__ __forceinline__ int owner_of(int64_t b, int unit, int64_t units, int64_t ctas) {
  return static_cast<int>(((b / unit + 1) * ctas - 1) / units);
}

// ---- thread-block cluster helpers (plain distributed-shared-memory stores, no multicast) ----
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_num_ctas() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Hardware barrier over all threads of the cluster (threads that have exited count as
// arrived); release / acquire makes shared-memory stores of any CTA visible to the others.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Store into the shared memory of CTA `rank` of this cluster at the offset `local` has here.
__device__ __forceinline__ void st_cluster_f32(float* local, uint32_t rank, float v) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}

__device__ __forceinline__ uint32_t* comm_ctl(uint8_t* base) { return reinterpret_cast<uint32_t*>(base); }
// Exchange slots carry their own arrival mark: every 8-byte word is {two bf16 values, stamp},
// written with one store, so data and mark arrive together and no fence is needed.
// [epoch & 3][source rank][tile][token][lane] words.
__device__ __forceinline__ uint2* comm_ar_word(const CommParams& c, uint8_t* base, int parity, int src,
                                               int tile, int tok, int lane) {
  const size_t tiles = static_cast<size_t>(c.ar_n / kTileN);
  return reinterpret_cast<uint2*>(base + kCommCtlBytes) +
         (((static_cast<size_t>(parity) * kCommMaxRanks + src) * tiles + tile) * 16 + tok) * 32 + lane;
}
__device__ __forceinline__ void st_relaxed_sys_v2(uint2* p, uint2 v) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
// Polls (bounded) until the word carries `stamp`; returns its data half.
__device__ __forceinline__ uint32_t comm_wait_word(const uint2* w, uint32_t stamp, int* status) {
  uint2 v = ld_relaxed_sys_v2(w);
  if (v.y == stamp) return v.x;
  if (*reinterpret_cast<volatile int*>(status) != 0) return 0u;
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    v = ld_relaxed_sys_v2(w);
    if (v.y == stamp) return v.x;
    if ((++spins & 255u) == 0) {
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitLimitCycles) {
        atomicCAS(status, 0, 3);
        return 0u;
      }
    }
  }
}

// Timeline probe, compiled in only with -DWOQ_B200_TIMELINE (a measuring build, never the
// shipped library): CTA c of launch q writes global-timer stamps to p.stamps[q % 8][c][idx].
#ifdef WOQ_B200_TIMELINE
__device__ __forceinline__ uint32_t tl_smid() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void decode_stamp(const DecodeParams& p, int idx) {
  if (p.stamps) p.stamps[(static_cast<size_t>(p.launch_seq & 7) * 1024 + blockIdx.x) * 8 + idx] = global_timer_ns();
}
#else
__device__ __forceinline__ void decode_stamp(const DecodeParams&, int) {}
#endif

// The stages a CTA walks: its share [b_begin, b_end) of the k-block sequence cut at tile
// boundaries ("segments") and then into runs of up to kStageKBlocks k-blocks.  Producer and
// consumers step through the same sequence.
struct StageIter {
  int tile, kb, k1, left, kbpt, skb;  // tile, next k-block, segment end, k-blocks left, ...
  __device__ StageIter(int tile0, int kb0, int left0, int kbpt0, int skb0)
      : tile(tile0), kb(kb0), k1(min(kbpt0, kb0 + left0)), left(left0), kbpt(kbpt0), skb(skb0) {}
  __device__ bool done() const { return left <= 0; }
  __device__ int nkb() const { return min(skb, k1 - kb); }
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

// Bias, rounding, fused post-op and store of one finished 64-row tile, by one warp: a0 / a1
// hold rows lane and lane + 32 for every token.  A function of its own (not inlined) so that
// its registers are allocated apart from the main loop's; with the tensor-parallel exchange
// compiled in (COMM) it also swaps the tile with the other ranks.
template <int NTOK, bool COMM>
__device__ __noinline__ void decode_tile_epilogue(const EpiParams& p, int tl, int lane, uint32_t epoch,
                                                  float* a0, float* a1) {
  if (COMM && p.comm.mode == kCommAllReduce) {
    // Row-parallel linear: every rank's bf16 partial of this tile goes to every rank; each
    // rank then adds them in rank order (fp32) and rounds once, so all ranks hold the same
    // bits; bias and post-op follow the reduction.
    const CommParams& c = p.comm;
    const uint32_t stamp = epoch + 1;
    const int parity = epoch & (kCommSets - 1);
    uint32_t mine[NTOK];
#pragma unroll
    for (int tok = 0; tok < NTOK; ++tok)
      if (tok < p.m) {
        mine[tok] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(a0[tok]))) |
                    (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(a1[tok]))) << 16);
        for (int q = 0; q < c.world; ++q)
          if (q != c.rank)
            st_relaxed_sys_v2(comm_ar_word(c, c.peer[q], parity, c.rank, tl, tok, lane),
                              make_uint2(mine[tok], stamp));
      }
    // Two tokens at a time: the words of every source rank are requested together (one round
    // trip to the local L2 for all of them, not one per rank), then added in rank order; only a
    // word that had not arrived yet is polled for.
#pragma unroll
    for (int h = 0; h < NTOK; h += 2) {
      if (h >= p.m) continue;
      uint2 v[kCommMaxRanks][2];
#pragma unroll
      for (int r = 0; r < kCommMaxRanks; ++r)
        if (r < c.world && r != c.rank) {
#pragma unroll
          for (int i = 0; i < 2; ++i)
            if (h + i < p.m) v[r][i] = ld_relaxed_sys_v2(comm_ar_word(c, c.peer[c.rank], parity, r, tl, h + i, lane));
        }
      float s0[2] = {0.f, 0.f}, s1[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kCommMaxRanks; ++r)
        if (r < c.world) {
#pragma unroll
          for (int i = 0; i < 2; ++i)
            if (h + i < p.m) {
              uint32_t w;
              if (r == c.rank)
                w = mine[h + i];
              else if (v[r][i].y == stamp)
                w = v[r][i].x;
              else
                w = comm_wait_word(comm_ar_word(c, c.peer[c.rank], parity, r, tl, h + i, lane), stamp, p.status);
              s0[i] += __uint_as_float(w << 16);
              s1[i] += __uint_as_float(w & 0xffff0000u);
            }
        }
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (h + i < p.m) {
          a0[h + i] = bf16_round(s0[i]);
          a1[h + i] = bf16_round(s1[i]);
        }
    }
  }
  // Words for the gather: the two results of this lane per token.  Everything the epilogue
  // reads from global memory (bias, fused operands, scatter rows) is loaded for up to eight
  // tokens before the first value is used: one round trip instead of one per token.
  uint32_t out[NTOK];
  if (p.fusion == FUSE_SILU_MUL) {
    // gate/up layout: row lane is a gate row, row lane + 32 its up row
    const int col = tl * 32 + lane;
    const bool ok = col < p.n_out;
    float b_gate = 0.f, b_up = 0.f;
    if (p.bias && ok) {
      b_gate = p.bias[decode_row_to_n(p, tl, lane)];
      b_up = p.bias[decode_row_to_n(p, tl, lane + 32)];
    }
#pragma unroll
    for (int tok = 0; tok < NTOK; ++tok) {
      out[tok] = 0u;
      if (tok < p.m && ok) {
        float gate = a0[tok], up = a1[tok];
        if (p.bias) {
          gate += b_gate;
          up += b_up;
        }
        const __nv_bfloat16 v = __float2bfloat16_rn(bf16_round(up) * silu_bf16(bf16_round(gate)));
        p.y[static_cast<size_t>(tok) * p.ldy + col] = v;
        out[tok] = __bfloat16_as_ushort(v);
      }
    }
  } else {
    const int n0 = decode_row_to_n(p, tl, lane), n1 = decode_row_to_n(p, tl, lane + 32);
    const bool ok0 = n0 < p.n, ok1 = n1 < p.n;
    const int c0 = ok0 ? n0 : 0, c1 = ok1 ? n1 : 0;  // columns that always exist
    float b0 = 0.f, b1 = 0.f;
    if (p.bias) {
      b0 = p.bias[c0];
      b1 = p.bias[c1];
    }
    // Eight tokens at a time (register budget).  Loads sit in loops of their own, guarded per
    // token, so that those of all existing tokens are in flight together; the arithmetic
    // follows in guarded loops.  Raw bf16 bits here, converted where they are used: a
    // conversion inside the guarded load loop would wait for its load before the next one is
    // issued.
    const auto bf = [](uint32_t b) { return __uint_as_float(b << 16); };
#pragma unroll
    for (int h = 0; h < NTOK; h += 8) {
      if (h >= p.m) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[h + i] = 0u;
        continue;
      }
      uint32_t f0[8], f1[8], wr[8];  // one register each: packed halves would tie a load to its neighbour
      int rows[8];
      auto load_rows = [&](const __nv_bfloat16* src, int64_t ld) {
        const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (h + i < p.m) {
            const size_t o = static_cast<size_t>(h + i) * ld;
            f0[i] = s16[o + c0];
            f1[i] = s16[o + c1];
          }
      };
      if (p.fusion == FUSE_SCALED_SCATTER_ADD) {
        // y[row_idx[tok]] += result * row_w[tok]; the rows of one call are distinct
        const unsigned short* y16 = reinterpret_cast<const unsigned short*>(p.y);
        const unsigned short* w16 = reinterpret_cast<const unsigned short*>(p.row_w);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (h + i < p.m) {
            rows[i] = p.row_idx[h + i];
            wr[i] = w16[h + i];
          }
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (h + i < p.m) {
            const size_t o = static_cast<size_t>(rows[i]) * p.ldy;
            f0[i] = y16[o + c0];
            f1[i] = y16[o + c1];
          }
      } else if (p.fusion == FUSE_ADD || p.fusion == FUSE_ADD_ADD || p.fusion == FUSE_MUL) {
        load_rows(p.other0, p.ldo);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (h + i < p.m) {
          float v0 = a0[h + i], v1 = a1[h + i];
          if (p.bias) {
            v0 += b0;
            v1 += b1;
          }
          v0 = bf16_round(v0);
          v1 = bf16_round(v1);
          if (p.fusion == FUSE_SCALED_SCATTER_ADD) {
            v0 = bf(f0[i]) + v0 * bf(wr[i]);
            v1 = bf(f1[i]) + v1 * bf(wr[i]);
          } else if (p.fusion == FUSE_ADD || p.fusion == FUSE_ADD_ADD) {
            v0 = bf16_round(v0 + bf(f0[i]));
            v1 = bf16_round(v1 + bf(f1[i]));
          } else if (p.fusion == FUSE_MUL) {
            v0 = bf16_round(v0 * bf(f0[i]));
            v1 = bf16_round(v1 * bf(f1[i]));
          } else {
            v0 = unary_post_op(v0, p.fusion);
            v1 = unary_post_op(v1, p.fusion);
          }
          a0[h + i] = v0;
          a1[h + i] = v1;
        }
      if (p.fusion == FUSE_ADD_ADD) {
        load_rows(p.other1, p.ldo);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (h + i < p.m) {
            a0[h + i] = bf16_round(a0[h + i] + bf(f0[i]));
            a1[h + i] = bf16_round(a1[h + i] + bf(f1[i]));
          }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        out[h + i] = 0u;
        if (h + i < p.m) {
          const __nv_bfloat16 v0 = __float2bfloat16_rn(a0[h + i]), v1 = __float2bfloat16_rn(a1[h + i]);
          const size_t o = static_cast<size_t>(p.fusion == FUSE_SCALED_SCATTER_ADD ? rows[i] : h + i) * p.ldy;
          if (ok0) p.y[o + n0] = v0;
          if (ok1) p.y[o + n1] = v1;
          if (p.fusion != FUSE_SCALED_SCATTER_ADD)
            out[h + i] = (ok0 ? __bfloat16_as_ushort(v0) : 0u) |
                         (ok1 ? static_cast<uint32_t>(__bfloat16_as_ushort(v1)) << 16 : 0u);
        }
      }
    }
  }
  if (COMM && p.comm.mode == kCommAllGather) {
    // Column-parallel linear: p.y is this rank's column block of the gathered tensor.  The
    // tile also goes to every other rank's slots; nobody waits here.  The other ranks' tiles
    // are copied into this rank's gathered tensor by the next launch on the comm
    // (comm_receive_pending), off the critical path of this one.
    const CommParams& c = p.comm;
    const uint32_t stamp = epoch + 1;
    const int parity = epoch & (kCommSets - 1);
#pragma unroll
    for (int tok = 0; tok < NTOK; ++tok)
      if (tok < p.m)
        for (int q = 0; q < c.world; ++q)
          if (q != c.rank)
            st_relaxed_sys_v2(comm_ar_word(c, c.peer[q], parity, c.rank, tl, tok, lane),
                              make_uint2(out[tok], stamp));
  }
}

// Receives the previous launch's all-gather (see CommPending): the (tile, source rank) pairs
// are dealt round-robin to the CTAs, one warp each; lane l copies its word of every token into
// this rank's gathered tensor.  `epoch` is the running launch's, the words carry the stamp of
// the launch before it.
__device__ __noinline__ void comm_receive_pending(const CommParams& c, uint32_t epoch, int* status, int lane,
                                                  int worker, int workers) {
  const CommPending& g = c.pend;
  const uint32_t stamp = epoch;  // (epoch - 1) + 1
  const int set = (epoch - 1u) & (kCommSets - 1);
  const int items = g.tiles * (c.world - 1);
  for (int item = worker; item < items; item += workers) {
    const int tl = item / (c.world - 1);
    int r = item - tl * (c.world - 1);
    if (r >= c.rank) ++r;
    int c0, c1;
    if (g.gate_up) {
      c0 = tl * 32 + lane;
      c1 = g.n / 2 + tl * 32 + lane;
    } else {
      c0 = tl * kTileN + lane;
      c1 = tl * kTileN + lane + 32;
    }
    __nv_bfloat16* dst = g.dst + static_cast<int64_t>(r) * g.n_out;
    const int64_t ld = static_cast<int64_t>(g.n_out) * c.world;
    for (int h = 0; h < g.m; h += 4) {
      uint2 v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (h + i < g.m) v[i] = ld_relaxed_sys_v2(comm_ar_word(c, c.peer[c.rank], set, r, tl, h + i, lane));
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (h + i < g.m) {
          const uint32_t w = v[i].y == stamp
                                 ? v[i].x
                                 : comm_wait_word(comm_ar_word(c, c.peer[c.rank], set, r, tl, h + i, lane), stamp, status);
          const int64_t o = static_cast<int64_t>(h + i) * ld;
          if (c0 < g.n_out) dst[o + c0] = __ushort_as_bfloat16(static_cast<unsigned short>(w & 0xffffu));
          if (g.pair && c1 < g.n_out) dst[o + c1] = __ushort_as_bfloat16(static_cast<unsigned short>(w >> 16));
        }
    }
  }
}

__global__ void __launch_bounds__(32) comm_fence_kernel(const __grid_constant__ CommParams c, int* status) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(comm_ctl(c.peer[c.rank]));
  comm_receive_pending(c, epoch, status, threadIdx.x, blockIdx.x, gridDim.x);
}

// COMM: compiled with the tensor-parallel exchange in the epilogue (the plain variant carries
// none of its code or registers).
template <int TB, int MODE, int KPW, bool COMM, bool CLUSTER>
__global__ void __launch_bounds__(kThreads, 2)
    woq_int4_decode_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(smem);
  constexpr int NTOK = 8 * TB;
  constexpr int kStageKBlocks = stage_kblocks(KPW);
  constexpr int kXRowBytes = x_row_bytes(KPW);
  const int sz_stage_bytes = (p.gps + 1) * 256;
  const int stage_bytes = kStageKBlocks * kBlockBytes + sz_stage_bytes + p.x_rows * kXRowBytes;
  const int red_tok = p.red_tok;  // tokens kept in the cross-warp reduction buffer
  uint8_t* stages = smem + kHeaderBytes;
  float* red = reinterpret_cast<float*>(stages + static_cast<size_t>(p.stages) * stage_bytes);
  // cluster variant, rank 0: the partial tiles pushed by ranks 1 .. C-1, [rank][token][row]
  float* parts = red + kConsumerWarps * red_tok * kRedTokStride;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t units = static_cast<int64_t>(p.tiles) * p.kb_per_tile / p.unit;
  int64_t b_begin, b_end;
  uint32_t crank = 0, csize = 1;
  if constexpr (CLUSTER) {
    // CTA r of a cluster owns units [r * u / C, (r + 1) * u / C) of its tile's u units
    csize = cluster_num_ctas();
    crank = cluster_cta_rank();
    const int64_t tile = blockIdx.x / csize;
    const int units_t = p.kb_per_tile / p.unit;
    b_begin = tile * p.kb_per_tile + static_cast<int64_t>(crank * units_t / csize) * p.unit;
    b_end = tile * p.kb_per_tile + static_cast<int64_t>((crank + 1) * units_t / csize) * p.unit;
  } else {
    b_begin = (static_cast<int64_t>(blockIdx.x) * units) / gridDim.x * p.unit;
    b_end = (static_cast<int64_t>(blockIdx.x + 1) * units) / gridDim.x * p.unit;
  }
  const int tile0 = static_cast<int>(b_begin / p.kb_per_tile);
  const int kb00 = static_cast<int>(b_begin - static_cast<int64_t>(tile0) * p.kb_per_tile);
  const int share = static_cast<int>(b_end - b_begin);

  if (tid == 0) {
    decode_stamp(p, 0);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], kConsumerWarps);
    }
    hdr->abort_flag = 0;
    hdr->finished_warps = 0;
    EpiParams& e = hdr->epi;
    e.bias = p.bias;
    e.y = p.y;
    e.other0 = p.other0;
    e.other1 = p.other1;
    e.row_idx = p.row_idx;
    e.row_w = p.row_w;
    e.status = p.status;
    e.ldy = p.ldy;
    e.ldo = p.ldo;
    e.m = p.m;
    e.n = p.n;
    e.n_out = p.n_out;
    e.fusion = p.fusion;
    e.gate_up = p.gate_up;
    if constexpr (COMM) e.comm = p.comm;
    mbar_fence_init();
  }
  __syncthreads();
  // A following launch that opted into programmatic dependent launch may start its weight
  // stream while this grid is still running.
  grid_launch_dependents();
  volatile int* abort_flag = &hdr->abort_flag;

  // Segments of this CTA's share: [kb00, ...) of tile0, then whole tiles, the last maybe short.
  const int seg0_len = min(share, p.kb_per_tile - kb00);
  const int nseg = share <= 0 ? 0 : 1 + (share - seg0_len + p.kb_per_tile - 1) / p.kb_per_tile;

  // ---- end-of-segment work, done by the epilogue warp; the CTA's last segment goes to the
  // producer warp (idle by then), so that the global-memory round trips of a short CTA's two
  // partial tiles overlap.  The warp takes the eight consumer warps' partial sums out of
  // shared memory, so the consumers go straight on to the next tile; then it either runs the
  // fused epilogue or parks a partial tile and, if this CTA is the last contributor to
  // arrive, reduces the tile in a fixed order.
  uint32_t epoch = 0;  // read by the warps that run epilogues, once the previous grid is done
  // The three epilogues decode steps use most (plain, residual add, silu(gate) * up; no
  // exchange) are written out here: a handful of instructions per token on the serial tail of
  // the launch, the partial sums stay in registers.  Everything else goes through the general
  // routine, on copies of the sums so that the arrays here never have their address taken.
  auto run_epilogue = [&](int tl, float* a0, float* a1) {
    const int fusion = p.fusion;
    const bool plain = (!COMM || p.comm.mode == kCommNone) &&
                       (fusion == FUSE_NONE || fusion == FUSE_ADD || fusion == FUSE_SILU_MUL);
    if (!plain) {
      float w0[NTOK], w1[NTOK];
#pragma unroll
      for (int tok = 0; tok < NTOK; ++tok) {
        w0[tok] = a0[tok];
        w1[tok] = a1[tok];
      }
      decode_tile_epilogue<NTOK, COMM>(hdr->epi, tl, lane, epoch, w0, w1);
      return;
    }
    const int n0 = decode_row_to_n(p, tl, lane), n1 = decode_row_to_n(p, tl, lane + 32);
    const int m = p.m;
    const int64_t ldy = p.ldy;
    float b0 = 0.f, b1 = 0.f;
    if (fusion == FUSE_SILU_MUL) {
      // gate/up layout: row lane is a gate row, row lane + 32 its up row
      const int col = tl * 32 + lane;
      if (col >= p.n_out) return;
      if (p.bias) {
        b0 = p.bias[n0];
        b1 = p.bias[n1];
      }
      __nv_bfloat16* yc = p.y + col;
#pragma unroll
      for (int tok = 0; tok < NTOK; ++tok)
        if (tok < m) {
          float gate = a0[tok], up = a1[tok];
          if (p.bias) {
            gate += b0;
            up += b1;
          }
          yc[tok * ldy] = __float2bfloat16_rn(bf16_round(up) * silu_bf16(bf16_round(gate)));
        }
      return;
    }
    const bool ok0 = n0 < p.n, ok1 = n1 < p.n;
    const int c0 = ok0 ? n0 : 0, c1 = ok1 ? n1 : 0;  // columns that always exist
    if (p.bias) {
      b0 = p.bias[c0];
      b1 = p.bias[c1];
    }
    uint32_t f0[NTOK], f1[NTOK];
    if (fusion == FUSE_ADD) {
      // all loads first (raw bf16 bits, converted where they are used): one round trip
      const unsigned short* o16 = reinterpret_cast<const unsigned short*>(p.other0);
      const int64_t ldo = p.ldo;
#pragma unroll
      for (int tok = 0; tok < NTOK; ++tok)
        if (tok < m) {
          f0[tok] = o16[tok * ldo + c0];
          f1[tok] = o16[tok * ldo + c1];
        }
    }
#pragma unroll
    for (int tok = 0; tok < NTOK; ++tok)
      if (tok < m) {
        float v0 = a0[tok], v1 = a1[tok];
        if (p.bias) {
          v0 += b0;
          v1 += b1;
        }
        v0 = bf16_round(v0);
        v1 = bf16_round(v1);
        if (fusion == FUSE_ADD) {
          v0 = bf16_round(v0 + __uint_as_float(f0[tok] << 16));
          v1 = bf16_round(v1 + __uint_as_float(f1[tok] << 16));
        }
        if (ok0) p.y[tok * ldy + n0] = __float2bfloat16_rn(v0);
        if (ok1) p.y[tok * ldy + n1] = __float2bfloat16_rn(v1);
      }
  };
  // Both epilogue-running warps call this when they are done; the second one of the last CTA
  // of the grid closes the epoch.
  auto finish_comm = [&]() {
    if (!COMM || p.comm.mode == kCommNone) return;
    int second = 0;
    if (lane == 0) second = atomicAdd(&hdr->finished_warps, 1);
    if (!__shfl_sync(0xffffffffu, second, 0)) return;
    if (lane == 0) {
      // the end of the grid orders these stores before anything the next launch reads
      uint32_t* ctl = comm_ctl(p.comm.peer[p.comm.rank]);
      if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {
        ctl[1] = 0;
        *reinterpret_cast<volatile uint32_t*>(ctl) = epoch + 1;
      }
    }
  };
  // `old` (lane 0) is what the arrival counter of tile tl held before this CTA counted in:
  // the last contributor adds all partials in CTA order and runs the epilogue
  auto resolve = [&](int tl, unsigned old, float* a0, float* a1) {
    old = __shfl_sync(0xffffffffu, old, 0);
    const int64_t tb0 = static_cast<int64_t>(tl) * p.kb_per_tile;
    const int c_first = owner_of(tb0, p.unit, units, gridDim.x);
    const int c_last = owner_of(tb0 + p.kb_per_tile - 1, p.unit, units, gridDim.x);
    if (old != static_cast<unsigned>(c_last - c_first)) return;
    __threadfence();
#pragma unroll
    for (int tok = 0; tok < NTOK; ++tok) a0[tok] = a1[tok] = 0.f;
    // The first contributor's share began before this tile unless it begins exactly with it
    // (its partial is then its first segment's); every later contributor begins inside the
    // tile, so this is its first segment.  Two contributors and eight tokens at a time; the
    // loads sit in a loop of their own so that all of them are in flight together, the adds
    // follow in CTA order.
    const int64_t cb_first = (static_cast<int64_t>(c_first) * units) / gridDim.x * p.unit;
    const float* slot0 = p.partials + static_cast<size_t>(c_first * 2 + (cb_first >= tb0 ? 0 : 1)) * (16 * kTileN) + lane;
    for (int c = c_first; c <= c_last; c += 2) {
      const float* src0 = c == c_first ? slot0 : p.partials + static_cast<size_t>(c * 2) * (16 * kTileN) + lane;
      const bool two = c + 1 <= c_last;
      const float* src1 = p.partials + static_cast<size_t>((two ? c + 1 : c) * 2) * (16 * kTileN) + lane;
#pragma unroll
      for (int h = 0; h < NTOK; h += 8) {
        if (h >= p.m) continue;
        float t0[8], t1[8], u0[8], u1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (h + i < p.m) {
            t0[i] = __ldcg(src0 + (h + i) * kTileN);
            t1[i] = __ldcg(src0 + (h + i) * kTileN + 32);
            u0[i] = __ldcg(src1 + (h + i) * kTileN);
            u1[i] = __ldcg(src1 + (h + i) * kTileN + 32);
          }
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (h + i < p.m) {
            a0[h + i] += t0[i];
            a1[h + i] += t1[i];
            if (two) {
              a0[h + i] += u0[i];
              a1[h + i] += u1[i];
            }
          }
      }
    }
    if (lane == 0) p.counters[tl] = 0;
    run_epilogue(tl, a0, a1);
  };
  // v0/v1: lane -> rows lane and lane + 32 of the tile, all tokens
  auto take_segment = [&](int bar_full, bool signal_free, int seg_tile, bool whole, bool first_segment,
                          float* v0, float* v1, int& pend_tile, unsigned& pend_old) {
    named_bar_sync(bar_full, kConsumerThreads + 32);
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
    // (a named barrier orders the shared-memory accesses made before it among its
    // participants; a fence on top of it cost about 0.6 us per call when measured)
    if (signal_free) named_bar_arrive(kBarRedFree, kConsumerThreads + 32);
    if (whole) {
      run_epilogue(seg_tile, v0, v1);
      return;
    }
    // Park the partial tile and count this CTA in.  Whether it was the last contributor is
    // looked at after the next partial segment (or at the end): the atomic's round trip then
    // overlaps other work instead of stalling this warp.
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
    unsigned old = 0;
    if (lane == 0) old = atomicAdd(p.counters + seg_tile, 1u);
    if (pend_tile >= 0) resolve(pend_tile, pend_old, v0, v1);
    pend_tile = seg_tile;
    pend_old = old;
  };

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
      const uint32_t bytes = nkb * kBlockBytes + ng * 256 + p.m * nkb * (kBlockK * 2);
      mbar_arrive_expect_tx(&hdr->full[slot], bytes);
      bulk_g2s(st, p.wq + (static_cast<size_t>(it.tile) * p.kb_per_tile + it.kb) * kBlockBytes,
               nkb * kBlockBytes, &hdr->full[slot]);
      bulk_g2s(st + kStageKBlocks * kBlockBytes,
               p.sz + (static_cast<size_t>(it.tile) * p.groups + g0) * 64, ng * 256,
               &hdr->full[slot]);
    };
    auto issue_x = [&](const StageIter& it, int slot) {  // lane = token
      if (lane < p.m) {
        uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
        bulk_g2s(st + kStageKBlocks * kBlockBytes + sz_stage_bytes + lane * kXRowBytes,
                 p.x + static_cast<size_t>(lane) * p.ldx + static_cast<size_t>(it.kb) * kBlockK,
                 it.nkb() * (kBlockK * 2), &hdr->full[slot]);
      }
    };
    StageIter it(tile0, kb00, share, p.kb_per_tile, kStageKBlocks);
    {
      StageIter fill = it;
      if (lane == 0)
        for (int s = 0; s < p.stages && !fill.done(); ++s) {
          issue_weights(fill, s);
          fill.next(fill.nkb());
        }
      if (lane == 0) decode_stamp(p, 1);
      grid_dependency_wait();
      if (lane == 0) decode_stamp(p, 2);
      if (COMM && p.comm.mode != kCommNone)
        epoch = *reinterpret_cast<volatile uint32_t*>(comm_ctl(p.comm.peer[p.comm.rank]));
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
        issue_weights(it, slot);
      }
      __syncwarp();
      issue_x(it, slot);
      it.next(it.nkb());
      if (++slot == p.stages) {
        slot = 0;
        phase ^= 1;
      }
    }
    if constexpr (CLUSTER) {
      // The CTA's only segment.  Ranks 1 .. C-1 push their partial tile into rank 0's shared
      // memory; after the cluster barrier rank 0 adds them in rank order and finishes the tile.
      float v0[NTOK], v1[NTOK];
      if (nseg > 0) {
        named_bar_sync(kBarRedFullLast, kConsumerThreads + 32);
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
      } else {
#pragma unroll
        for (int tok = 0; tok < NTOK; ++tok) v0[tok] = v1[tok] = 0.f;
      }
      if (lane == 0) decode_stamp(p, 5);
      if (csize > 1) {
        if (crank != 0) {
          float* mine = parts + crank * (red_tok * kRedTokStride);
#pragma unroll
          for (int tok = 0; tok < NTOK; ++tok)
            if (tok < p.m) {
              st_cluster_f32(mine + tok * kRedTokStride + lane, 0, v0[tok]);
              st_cluster_f32(mine + tok * kRedTokStride + lane + 32, 0, v1[tok]);
            }
        }
        __syncwarp();
        cluster_sync_all();
        if (crank == 0) {
          for (uint32_t c = 1; c < csize; ++c) {
            const float* src = parts + c * (red_tok * kRedTokStride);
#pragma unroll
            for (int tok = 0; tok < NTOK; ++tok)
              if (tok < p.m) {
                v0[tok] += src[tok * kRedTokStride + lane];
                v1[tok] += src[tok * kRedTokStride + lane + 32];
              }
          }
        }
      }
      if (lane == 0) decode_stamp(p, 6);
      if (crank == 0) run_epilogue(tile0, v0, v1);
      if (lane == 0) decode_stamp(p, 7);
    } else if (nseg > 0) {
      // the CTA's last segment
      float v0[NTOK], v1[NTOK];
      int pend_tile = -1;
      unsigned pend_old = 0;
      const int k0 = nseg == 1 ? kb00 : 0;
      const int len = nseg == 1 ? share : share - seg0_len - (nseg - 2) * p.kb_per_tile;
      take_segment(kBarRedFullLast, false, tile0 + nseg - 1, k0 == 0 && len == p.kb_per_tile,
                   nseg == 1, v0, v1, pend_tile, pend_old);
      if (pend_tile >= 0) resolve(pend_tile, pend_old, v0, v1);
      if (lane == 0) decode_stamp(p, 7);
    }
    finish_comm();
    return;
  }

  if (warp == kEpilogueWarp) {
    // ------------------------------ epilogue warp --------------------------------------
    float v0[NTOK], v1[NTOK];
    int pend_tile = -1;
    unsigned pend_old = 0;
    grid_dependency_wait();  // y, the fused operands and the workspace belong to this grid now
    if (COMM && p.comm.mode != kCommNone) {
      epoch = *reinterpret_cast<volatile uint32_t*>(comm_ctl(p.comm.peer[p.comm.rank]));
      // the previous launch's all-gather, received while this launch's weights stream
      if (p.comm.pend.dst && p.comm.world > 1)
        comm_receive_pending(hdr->epi.comm, epoch, p.status, lane, blockIdx.x, gridDim.x);
    }
    if constexpr (!CLUSTER) {
      for (int sg = 0; sg + 1 < nseg; ++sg) {
        take_segment(kBarRedFull, true, tile0 + sg, sg > 0 || kb00 == 0, sg == 0, v0, v1, pend_tile,
                     pend_old);
      }
      if (pend_tile >= 0) resolve(pend_tile, pend_old, v0, v1);
    }
    finish_comm();
    if (CLUSTER && csize > 1) cluster_sync_all();
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
  int seg = 0;  // segments flushed so far

  // end of a tile segment: hand this warp's partial sums over and go on
  auto flush = [&]() {
    // the buffer is free once the epilogue warp has read the previous segment
    if (seg > 0) named_bar_sync(kBarRedFree, kConsumerThreads + 32);
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
    ++seg;
    named_bar_arrive(seg == nseg ? kBarRedFullLast : kBarRedFull, kConsumerThreads + 32);
  };

  StageIter it(tile0, kb00, share, p.kb_per_tile, kStageKBlocks);
  int slot = 0;
  uint32_t phase = 0;
#ifdef WOQ_B200_TIMELINE
  long long tl_wait = 0, tl_begin = 0;
#endif
  // per-row constants of the current group, rows g, g+8 of each row-tile
  uint32_t cz[8], cs[8];
  // per-lane offsets inside a stage.  A lane whose token does not exist reads the last real
  // token's x instead: its MMA columns are never written out, and columns do not mix.
  const int w_off = lane * 16;
  const int s_off = kStageKBlocks * kBlockBytes + g * 32;
  int x_off[TB];
#pragma unroll
  for (int tb = 0; tb < TB; ++tb)
    x_off[tb] = kStageKBlocks * kBlockBytes + sz_stage_bytes + min(tb * 8 + g, p.m - 1) * kXRowBytes + t * 32;
  while (!it.done()) {
    const int nkb = it.nkb();
    const int kb0 = it.kb;
    const uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
#ifdef WOQ_B200_TIMELINE
    const long long tl_c0 = clock64();
#endif
    mbar_wait(&hdr->full[slot], phase, abort_flag, p.status, 2);
#ifdef WOQ_B200_TIMELINE
    tl_wait += clock64() - tl_c0;
    if (tl_begin == 0) tl_begin = clock64();
#endif
    if (warp == 0 && lane == 0 && kb0 == kb00) decode_stamp(p, 3);

    // one k-block (64 rows x 64 k) of the stage: index idx, constants reloaded if `prep`
    auto do_kblock = [&](const int idx, const bool prep) {
      const int kb = kb0 + idx;
      // packed weights: one 128-bit load per k-step covers the four row-tiles
      const uint4* wp = reinterpret_cast<const uint4*>(st + idx * kBlockBytes + w_off);
      uint4 wv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = wp[j * 32];
      // activations: this lane's 16 k of token g (+8)
      uint32_t xb[TB][8];
#pragma unroll
      for (int tb = 0; tb < TB; ++tb) {
        const uint4* xp = reinterpret_cast<const uint4*>(st + x_off[tb] + idx * (kBlockK * 2));
        const uint4 a = xp[0], c = xp[1];
        xb[tb][0] = a.x; xb[tb][1] = a.y; xb[tb][2] = a.z; xb[tb][3] = a.w;
        xb[tb][4] = c.x; xb[tb][5] = c.y; xb[tb][6] = c.z; xb[tb][7] = c.w;
      }
      // {bf16 scale, bf16 128 + zp} of this k-block's group for rows g, g+8 of each row-tile
      if (prep) {
        const int gl = (kb >> p.kbpg_shift) - (kb0 >> p.kbpg_shift);
        const uint4* sp = reinterpret_cast<const uint4*>(st + s_off + gl * 256);
        const uint4 s_lo = sp[0], s_hi = sp[1];
        const uint32_t szw[8] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w, s_hi.x, s_hi.y, s_hi.z, s_hi.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if constexpr (MODE == kScaleAfterSum) {
            // x enters the MMAs multiplied by 2^64 (see below).  Row g (even i): the A operand
            // is 128 + q, so sum = 2^64 sum_k x (128 + q): subtract (128 + zp) sum_k x, scale by
            // s 2^-64.  Row g+8 (odd i): the A operand is the nibble in place, 16 q 2^-133 as a
            // subnormal bf16, so sum = 2^-65 sum_k x q: subtract zp 2^-129 sum_k x, scale by s 2^65.
            const float sf = __uint_as_float(szw[i] & 0xffff0000u);
            const float zf = __uint_as_float(szw[i] << 16);  // 128 + zp
            if (i & 1) {
              cs[i] = __float_as_uint(sf * 36893488147419103232.f);                           // 2^65
              cz[i] = __float_as_uint((zf - 128.f) * 1.4693679385278594e-39f);                // 2^-129
            } else {
              cs[i] = __float_as_uint(sf * 5.421010862427522e-20f);                           // 2^-64
              cz[i] = __float_as_uint(zf);
            }
          } else if (MODE == kExactInPlace && (i & 1)) {
            // row g+8 takes its nibbles from bits 4..7 / 20..23 without a shift: read as bf16
            // the masked half-word is 16 q * 2^-133 exactly (the encoding is linear below
            // 2^-125), so subtract 16 zp * 2^-133 and multiply by scale * 2^129
            cz[i] = (szw[i] & 0xfu) * 0x00100010u;
            cs[i] = __byte_perm(szw[i], 0, 0x3232) + 0x40804080u;
          } else {
            cz[i] = __byte_perm(szw[i], 0, 0x1010);
            cs[i] = __byte_perm(szw[i], 0, 0x3232);
          }
        }
      }

      if constexpr (MODE != kScaleAfterSum) {
        // bf16((q - zp) * bf16 scale) per weight, exactly the reference's tile dequantiser;
        // the MMAs accumulate straight into the running sums
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int rt = 0; rt < 4; ++rt) {
            const uint32_t w = (rt == 0) ? wv[j].x : (rt == 1) ? wv[j].y : (rt == 2) ? wv[j].z : wv[j].w;
            const uint32_t z0 = cz[rt * 2], z1 = cz[rt * 2 + 1], s0 = cs[rt * 2], s1 = cs[rt * 2 + 1];
            uint32_t a[4];
            if constexpr (MODE == kExactInPlace) {
              const uint32_t u = w >> 8;
              a[0] = bf16x2_mul(bf16x2_sub(lop3_and_or(w, 0x000f000fu, kBf16Magic), z0), s0);
              a[1] = bf16x2_mul(bf16x2_sub(w & 0x00f000f0u, z1), s1);
              a[2] = bf16x2_mul(bf16x2_sub(lop3_and_or(u, 0x000f000fu, kBf16Magic), z0), s0);
              a[3] = bf16x2_mul(bf16x2_sub(u & 0x00f000f0u, z1), s1);
            } else {
              a[0] = bf16x2_mul(bf16x2_sub(lop3_and_or(w, 0x000f000fu, kBf16Magic), z0), s0);
              a[1] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 4, 0x000f000fu, kBf16Magic), z1), s1);
              a[2] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 8, 0x000f000fu, kBf16Magic), z0), s0);
              a[3] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 12, 0x000f000fu, kBf16Magic), z1), s1);
            }
#pragma unroll
            for (int tb = 0; tb < TB; ++tb)
              mma_bf16_16816(acc[rt][tb], a, xb[tb][2 * j], xb[tb][2 * j + 1]);
          }
        }
      } else {
        // Activations times 2^64 (exact unless |x| >= 2^63): the in-place rows multiply x by
        // numbers near 2^-129, and the products must stay in fp32's normal range.
#pragma unroll
        for (int tb = 0; tb < TB; ++tb)
#pragma unroll
          for (int i = 0; i < 8; ++i) xb[tb][i] = bf16x2_mul(xb[tb][i], 0x5f805f80u);
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
            const uint32_t w = (rt == 0) ? wv[j].x : (rt == 1) ? wv[j].y : (rt == 2) ? wv[j].z : wv[j].w;
            const uint32_t u = w >> 8;
            uint32_t a[4];
            a[0] = lop3_and_or(w, 0x000f000fu, kBf16Magic);
            a[1] = w & 0x00f000f0u;
            a[2] = lop3_and_or(u, 0x000f000fu, kBf16Magic);
            a[3] = u & 0x00f000f0u;
#pragma unroll
            for (int tb = 0; tb < TB; ++tb)
              mma_bf16_16816(accg[rt][tb], a, xb[tb][2 * j], xb[tb][2 * j + 1]);
          }
        }
#pragma unroll
        for (int rt = 0; rt < 4; ++rt)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float s = __uint_as_float(cs[rt * 2 + h]);
            const float nz = -__uint_as_float(cz[rt * 2 + h]);
#pragma unroll
            for (int tb = 0; tb < TB; ++tb)
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                const float d = fmaf(nz, sx[tb][c], accg[rt][tb][h * 2 + c]);
                acc[rt][tb][h * 2 + c] = fmaf(s, d, acc[rt][tb][h * 2 + c]);
              }
          }
      }
    };
    if (nkb == kStageKBlocks) {
      // full stage: straight-line code, the second k-block's loads overlap the first's math
      // (a warp's two k-blocks share their group unless a group is a single k-block)
#pragma unroll
      for (int kk = 0; kk < KPW; ++kk) do_kblock(KPW * warp + kk, kk == 0 || p.kbpg_shift == 0);
    } else {
#pragma unroll 1
      for (int kk = 0; kk < KPW; ++kk)
        if (KPW * warp + kk < nkb) do_kblock(KPW * warp + kk, true);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&hdr->empty[slot]);
    if (kb0 + nkb == it.k1) {
      if (warp == 0 && lane == 0) decode_stamp(p, 4);
      flush();
    }
    it.next(nkb);
    if (++slot == p.stages) {
      slot = 0;
      phase ^= 1;
    }
  }
#ifdef WOQ_B200_TIMELINE
  if (warp == 3 && lane == 0 && p.stamps)
    p.stamps[(static_cast<size_t>(p.launch_seq & 7) * 1024 + blockIdx.x) * 8 + 6] =
        (static_cast<long long>(tl_smid()) << 56) | ((tl_wait & 0xffffffll) << 32) | ((clock64() - tl_begin) & 0xffffffffll);
#endif
  if (CLUSTER && csize > 1) {
    __syncwarp();
    cluster_sync_all();
  }
}

}  // namespace

size_t decode_int4_partial_bytes(int grid) { return static_cast<size_t>(grid) * 2 * 16 * kTileN * 4; }

namespace {

// Tuning variables, read once when the library is first used (never per launch):
//   WOQ_B200_DECODE_SPLIT  0 choose per layer (default), 1 always the stream-K grid,
//                          2 the cluster grid whenever the layer has few enough tiles
//   WOQ_B200_PDL           0 switches programmatic dependent launch off
struct DecodeTuning {
  int split, pdl;
};
DecodeTuning& tuning() {
  static DecodeTuning t = [] {
    auto env_int = [](const char* name, int fallback) {
      const char* e = getenv(name);
      return e ? atoi(e) : fallback;
    };
    DecodeTuning v;
    v.split = env_int("WOQ_B200_DECODE_SPLIT", 0);
    v.pdl = env_int("WOQ_B200_PDL", 1);
    return v;
  }();
  return t;
}

// bytes of one pipeline stage / of the cross-warp reduction buffer
int stage_bytes_for(int m, int kpw, int kbpg_shift) {
  const int gps = (stage_kblocks(kpw) >> kbpg_shift) + 1;
  return stage_kblocks(kpw) * kBlockBytes + (gps + 1) * 256 + m * x_row_bytes(kpw);
}
int red_tok_for(int m) { return (m + 1) & ~1; }
int red_bytes_for(int m) { return kConsumerWarps * red_tok_for(m) * kRedTokStride * 4; }
constexpr int kBudgetTwoCtas = 112 * 1024;  // shared memory of one CTA

// two k-blocks per warp and stage while two such stages fit beside the x rows (1..6 tokens)
int pick_kpw(int m, int kbpg_shift) {
  if (m > 8) return 1;
  const int fits = (kBudgetTwoCtas - kHeaderBytes - red_bytes_for(m)) / stage_bytes_for(m, 2, kbpg_shift) >= 2;
  return fits ? 2 : 1;
}

template <int TB, int KPW, bool COMM, bool CLUSTER>
void (*pick_kernel_mode(int mode))(const DecodeParams) {
  switch (mode) {
    case kScaleAfterSum: return woq_int4_decode_kernel<TB, kScaleAfterSum, KPW, COMM, CLUSTER>;
    case kExactShift: return woq_int4_decode_kernel<TB, kExactShift, KPW, COMM, CLUSTER>;
    default: return woq_int4_decode_kernel<TB, kExactInPlace, KPW, COMM, CLUSTER>;
  }
}
template <int TB, int KPW>
void (*pick_kernel(int mode, bool comm, bool cluster))(const DecodeParams) {
  if (cluster) return comm ? pick_kernel_mode<TB, KPW, true, true>(mode) : pick_kernel_mode<TB, KPW, false, true>(mode);
  return comm ? pick_kernel_mode<TB, KPW, true, false>(mode) : pick_kernel_mode<TB, KPW, false, false>(mode);
}

}  // namespace

void decode_int4_set_split(int mode) { tuning().split = mode; }
bool dependent_launch_enabled() { return tuning().pdl != 0; }

namespace {

// How many clusters of c CTAs the device keeps resident at once (thread-block clusters never
// span GPCs, so this is less than slots / c), asked of the runtime once per cluster size for a
// CTA that takes half an SM's shared memory [0] and for one that takes nearly all of it [1].
struct ClusterCapacity {
  int cap[2][9];
};
const ClusterCapacity& cluster_capacity(int num_sms) {
  static ClusterCapacity cc = [num_sms] {
    ClusterCapacity v{};
    void (*kern)(const DecodeParams) = woq_int4_decode_kernel<1, kExactInPlace, 1, false, true>;
    for (int big = 0; big < 2; ++big) {
      const int smem = big ? 2 * kBudgetTwoCtas - 8 * 1024 : kBudgetTwoCtas;
      const bool attr_ok =
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess;
      for (int c = 1; c <= 8; ++c) {
        int n = 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(c * 8);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = c;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (!attr_ok || cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
          cudaGetLastError();
          n = (big ? 1 : 2) * num_sms / c * 7 / 8;  // conservative guess
        }
        v.cap[big][c] = n;
      }
    }
    return v;
  }();
  return cc;
}

}  // namespace

DecodePlan decode_int4_plan(int m, int tiles, int kb_per_tile, int kb_per_group, int num_sms) {
  int shift = 0;
  while ((1 << (shift + 1)) <= kb_per_group && shift < 30) ++shift;
  DecodePlan pl{};
  const int slots = 2 * num_sms;  // CTAs resident at once
  const int64_t total_kb = static_cast<int64_t>(tiles) * kb_per_tile;

  // stream-K: 2 CTAs per SM, equal contiguous shares of the k-block sequence; shares are dealt
  // in pairs of k-blocks when a warp takes two, so that a pair never straddles two groups
  pl.kpw = pick_kpw(m, shift);
  pl.unit = pl.kpw == 2 && kb_per_group % 2 == 0 ? 2 : 1;
  pl.cluster = 0;
  pl.smem_budget = kBudgetTwoCtas;
  const int64_t units = total_kb / pl.unit;
  pl.grid = static_cast<int>(units < slots ? (units < 1 ? 1 : units) : slots);
  if (tuning().split == 1 || tiles > slots) return pl;

  // cluster grid: tiles x C CTAs, all resident at once.  Work of the busiest SM against the
  // even share gives the efficiency of a split, with a penalty for a single CTA per SM: the
  // dequantising warps of one CTA alone do not keep an SM's issue slots busy.
  const ClusterCapacity& cc = cluster_capacity(num_sms);
  int best_c = 0;
  double best_eff = 0.0;
  for (int c = 1; c <= 8 && tiles * c <= slots; ++c) {
    if (c > 1 && kb_per_tile / c < kConsumerWarps) break;
    if (tiles > cc.cap[0][c]) continue;  // would need a second wave
    const int slice = (kb_per_tile + c - 1) / c;
    const int per_sm = (tiles * c + num_sms - 1) / num_sms;
    double eff = static_cast<double>(total_kb) / (static_cast<double>(num_sms) * per_sm * slice);
    if (per_sm < 2) eff *= 0.9;
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best_c = c;
    }
  }
  if (best_c == 0) return pl;
  // time estimates in microseconds: a stream-K launch pays about 9 us of dependency, fill and
  // split-K fix-up round trips, a cluster launch about 5; streaming at about 4.5 TB/s
  const double stream_us = static_cast<double>(total_kb) * kBlockBytes / 4.5e6;
  if (tuning().split != 2 && stream_us / best_eff + 5.0 >= stream_us + 9.0) return pl;
  pl.cluster = best_c;
  pl.grid = tiles * best_c;
  const int slice = kb_per_tile / best_c;
  pl.kpw = m <= 8 && slice >= 2 * kConsumerWarps && kb_per_group % 2 == 0 && pick_kpw(m, shift) == 2 ? 2 : 1;
  pl.unit = pl.kpw;
  // a grid with at most one CTA per SM may use the shared memory two CTAs would share
  if (pl.grid <= num_sms && tiles <= cc.cap[1][best_c]) pl.smem_budget = 2 * kBudgetTwoCtas - 8 * 1024;
  return pl;
}

cudaError_t launch_comm_fence(const CommParams& c, int* status, int num_sms, cudaStream_t stream) {
  comm_fence_kernel<<<num_sms, 32, 0, stream>>>(c, status);
  return cudaGetLastError();
}

cudaError_t launch_decode_int4(DecodeParams p, const DecodePlan& plan, cudaStream_t stream) {
  const int tb = p.m <= 8 ? 1 : 2;
  const int kpw = plan.kpw;
  p.unit = plan.unit;
  p.x_rows = p.m;
  p.red_tok = red_tok_for(p.m);
  const int skb = stage_kblocks(kpw);
  p.gps = (skb >> p.kbpg_shift) + 1;  // groups a stage can touch
  const int stage_bytes = skb * kBlockBytes + (p.gps + 1) * 256 + p.x_rows * x_row_bytes(kpw);
  const int red_bytes = red_bytes_for(p.m);
  const int parts_bytes = plan.cluster > 1 ? plan.cluster * p.red_tok * kRedTokStride * 4 : 0;
  int stages = (plan.smem_budget - kHeaderBytes - red_bytes - parts_bytes) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (plan.cluster) {
    // one segment per CTA: no more stages than the longest slice needs
    const int units_t = p.kb_per_tile / plan.unit;
    const int slice = (units_t + plan.cluster - 1) / plan.cluster * plan.unit;
    const int need = (slice + skb - 1) / skb;
    if (stages > need) stages = need;
    if (stages < 1) return cudaErrorInvalidConfiguration;
  } else if (stages < 2) {
    return cudaErrorInvalidConfiguration;
  }
  p.stages = stages;
#ifdef WOQ_B200_TIMELINE
  static int launch_seq = 0;
  p.launch_seq = launch_seq++;
#endif
  const size_t smem = kHeaderBytes + static_cast<size_t>(stages) * stage_bytes + red_bytes + parts_bytes;
  const bool comm = p.comm.mode != kCommNone;
  const bool cl = plan.cluster > 0;
  void (*kern)(const DecodeParams) = tb == 2     ? pick_kernel<2, 1>(p.exact, comm, cl)
                                     : kpw == 2 ? pick_kernel<1, 2>(p.exact, comm, cl)
                                                : pick_kernel<1, 1>(p.exact, comm, cl);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  // Programmatic dependent launch: this grid may start streaming weights while the previous
  // kernel in the stream drains (it waits for that kernel before it touches x, y or the
  // workspace).  After a kernel that never signals, or after a copy, this is ordinary ordering.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan.grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (tuning().pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  if (cl) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = plan.cluster;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace woq
