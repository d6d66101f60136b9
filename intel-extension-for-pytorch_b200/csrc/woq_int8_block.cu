// INT8 compute with K-block scaling: INT4 or INT8 weights, every activation quantisation mode
// of the reference (csrc/cpu/aten/utils/woq_defines.h:11-19), on the plain weight layout.
//
// Per K block of kb = min(group, 128) elements (csrc/cpu/aten/Linear.cpp:362-376):
//     qC[m,n] = sum_k qa[m,k] * (qw[n,k] - zp_w[n,g])                     int32, exact
//     qC     -= comp[n,block] * zp_a[m,block]                              (asymmetric activations)
//     C[m,n] += (float(qC) * scale_a[m,block]) * scale_w[n,g]              fp32
// (csrc/cpu/aten/utils/woq.h:962-1126 for 4-bit weights, :2231-2354 for INT8 weights).  The
// integer part runs on the tensor cores (mma.sync m16n8k32, s32 accumulate) with the weight
// codes as they are stored (u8 nibbles 0..15 or s8 bytes): sum qa * (qw - zp_w) is taken as
// sum qa * qw - zp_w * sum qa, with the block sums of the activation codes made by the
// quantiser; both are exact integer identities.
//
// Activation quantisation (woq_dynamic_quant.h:1526-1750): one range per tensor (modes 0 / 4), per
// K block over all tokens (1 / 5), per token (2 / 6), per token and K block (3 / 7); symmetric
// (+4): scale = max|x| / 127, s8 codes; asymmetric: scale = (max - min) / 255,
// zp = -nearbyint(min / scale), u8 codes nearbyint(x / scale + zp).  Three small kernels: ranges
// per (token, block), the fold over what shares a range, the codes.
//
// A CTA owns 16 output rows and 8 tokens; its four warps take every fourth K block and their
// fp32 sums are added in warp order at the end (nothing depends on timing).  Larger token counts
// are further CTAs that read the weights again (from L2): this route is built for decode-sized
// batches; the tcgen05 kernel of woq_int8.cu keeps INT8 weights with whole-K activation ranges.
#include "woq_kernels.h"

namespace woq {

namespace {

// ---- activation quantisation --------------------------------------------------------------
// one warp per (token, block): range of the block
__global__ void __launch_bounds__(256) act_block_range_kernel(const __nv_bfloat16* x, int64_t ldx, int m, int k,
                                                              int kb, int kc, float* range) {
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= m * kc) return;
  const int tok = item / kc, c = item - tok * kc;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(tok) * ldx + c * kb;
  const int len = min(kb, k - c * kb);
  float lo = INFINITY, hi = -INFINITY;
  for (int i = lane; i < len; i += 32) {
    const float v = __bfloat162float(xr[i]);
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if (lane == 0) {
    range[2 * item] = lo;
    range[2 * item + 1] = hi;
  }
}

// Folds the (token, block) ranges over what shares one: base 0 everything (1 output), base 1 the
// tokens of a block (kc outputs), base 2 the blocks of a token (m outputs).  One CTA per output.
__global__ void __launch_bounds__(256) act_fold_range_kernel(const float* range, int m, int kc, int base,
                                                             float* folded) {
  __shared__ float red[16];
  const int out = blockIdx.x, tid = threadIdx.x;
  float lo = INFINITY, hi = -INFINITY;
  const int count = base == 0 ? m * kc : base == 1 ? m : kc;
  for (int i = tid; i < count; i += 256) {
    const int item = base == 0 ? i : base == 1 ? i * kc + out : out * kc + i;
    lo = fminf(lo, range[2 * item]);
    hi = fmaxf(hi, range[2 * item + 1]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if ((tid & 31) == 0) {
    red[tid >> 5] = lo;
    red[8 + (tid >> 5)] = hi;
  }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < 8; ++i) {
      lo = fminf(lo, red[i]);
      hi = fmaxf(hi, red[8 + i]);
    }
    folded[2 * out] = fminf(lo, red[0]);
    folded[2 * out + 1] = fmaxf(hi, red[8]);
  }
}

// one warp per (token, block): scale, zero point, codes and their sum.  `interleave`: inside
// every 8 elements the even ones first, then the odd ones (the order the INT4 weight words
// give their nibbles in).
template <bool ASYM>
__global__ void __launch_bounds__(256) act_block_quant_kernel(const __nv_bfloat16* x, int64_t ldx, int m, int k,
                                                              int kb, int kc, int base, const float* range,
                                                              const float* folded, int interleave, uint8_t* qa,
                                                              float* sa, int32_t* zpa, int32_t* sumqa) {
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= m * kc) return;
  const int tok = item / kc, c = item - tok * kc;
  const float* r = base == 3 ? range + 2 * item : base == 0 ? folded : base == 1 ? folded + 2 * c : folded + 2 * tok;
  const float lo = r[0], hi = r[1];
  float scale, zp = 0.f;
  if (ASYM) {
    scale = __fdiv_rn(hi - lo, 255.0f);
    zp = scale > 0.f ? -rintf(__fdiv_rn(lo, scale)) : 0.f;
  } else {
    scale = __fdiv_rn(fmaxf(fabsf(hi), fabsf(lo)), 127.0f);
  }
  const float q_lo = ASYM ? 0.f : -128.f, q_hi = ASYM ? 255.f : 127.f;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(tok) * ldx + c * kb;
  uint8_t* qr = qa + static_cast<int64_t>(tok) * k + c * kb;
  const int len = min(kb, k - c * kb);
  int sum = 0;
  for (int i = lane; i < len; i += 32) {
    float q = 0.f;
    if (scale > 0.f) q = fminf(fmaxf(rintf(__fdiv_rn(__bfloat162float(xr[i]), scale) + zp), q_lo), q_hi);
    const int qi = static_cast<int>(q);
    sum += qi;
    const int pos = interleave ? (i & ~7) + ((i & 1) ? 4 : 0) + ((i & 7) >> 1) : i;
    qr[pos] = static_cast<uint8_t>(qi & 0xff);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) {
    sa[item] = scale;
    zpa[item] = static_cast<int32_t>(zp);
    sumqa[item] = sum;
  }
}

// ---- weight side: per (row, block) sum of (qw - zp_w), for asymmetric activations ----------
template <bool W4>
__global__ void __launch_bounds__(256) weight_block_sum_kernel(const uint8_t* w, const float* zpw, int n, int k,
                                                               int kb, int kc, int group, int groups,
                                                               float default_zp, int32_t* comp) {
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n * kc) return;
  const int row = item / kc, c = item - row * kc;
  const int g = group >= k ? 0 : (c * kb) / group;
  const int z = static_cast<int>(zpw ? zpw[static_cast<size_t>(row) * groups + g] : default_zp);
  int sum = 0;
  for (int i = lane; i < kb; i += 32) {
    const int kk = c * kb + i;
    int q;
    if (W4) {
      const uint8_t b = w[static_cast<size_t>(row) * (k / 2) + (kk >> 1)];
      q = (kk & 1) ? (b >> 4) : (b & 15);
    } else {
      q = static_cast<int8_t>(w[static_cast<size_t>(row) * k + kk]);
    }
    sum += q - z;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) comp[item] = sum;
}

// ---- the GEMM -----------------------------------------------------------------------------------
template <bool AU8, bool BU8>
__device__ __forceinline__ void mma_i8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  if (AU8 && BU8)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else if (AU8)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else if (BU8)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kI8Warps = 4;

template <bool W4, bool ASYM>
__global__ void __launch_bounds__(kI8Warps * 32) woq_i8_block_kernel(const I8BlockParams p) {
  __shared__ float red[kI8Warps][16][9];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row_lo = blockIdx.x * 16 + g, row_hi = row_lo + 8;
  const int tok0 = blockIdx.y * 8;
  // rows / tokens outside the problem read row / token 0 and are never written
  const int r0 = row_lo < p.n ? row_lo : 0, r1 = row_hi < p.n ? row_hi : 0;
  const int tok_b = tok0 + g < p.m ? tok0 + g : 0;           // the token whose codes this lane feeds (B column g)
  const int tc0 = tok0 + 2 * t, tc1 = tc0 + 1;               // the tokens of this lane's accumulator columns
  const int ta = tc0 < p.m ? tc0 : 0, tb = tc1 < p.m ? tc1 : 0;
  const size_t row_bytes = W4 ? p.k / 2 : p.k;
  const uint8_t* w0 = p.w + r0 * row_bytes;
  const uint8_t* w1 = p.w + r1 * row_bytes;
  const uint8_t* qb = p.qa + static_cast<size_t>(tok_b) * p.k;
  float c[4] = {0.f, 0.f, 0.f, 0.f};  // (row_lo, tc0) (row_lo, tc1) (row_hi, tc0) (row_hi, tc1)

  for (int blk = warp; blk < p.kc; blk += kI8Warps) {
    int acc[4] = {0, 0, 0, 0};
    const int k0 = blk * p.kb;
    for (int kk = 0; kk < p.kb; kk += 64) {
      const int kq = k0 + kk + 16 * t;  // this lane's 16 k of the 64
      const uint4 bv = *reinterpret_cast<const uint4*>(qb + kq);
      if (W4) {
        const uint2 a = *reinterpret_cast<const uint2*>(w0 + (kq >> 1));
        const uint2 b = *reinterpret_cast<const uint2*>(w1 + (kq >> 1));
        mma_i8<true, ASYM>(acc, a.x & 0x0f0f0f0fu, b.x & 0x0f0f0f0fu, (a.x >> 4) & 0x0f0f0f0fu,
                           (b.x >> 4) & 0x0f0f0f0fu, bv.x, bv.y);
        mma_i8<true, ASYM>(acc, a.y & 0x0f0f0f0fu, b.y & 0x0f0f0f0fu, (a.y >> 4) & 0x0f0f0f0fu,
                           (b.y >> 4) & 0x0f0f0f0fu, bv.z, bv.w);
      } else {
        const uint4 a = *reinterpret_cast<const uint4*>(w0 + kq);
        const uint4 b = *reinterpret_cast<const uint4*>(w1 + kq);
        mma_i8<false, ASYM>(acc, a.x, b.x, a.y, b.y, bv.x, bv.y);
        mma_i8<false, ASYM>(acc, a.z, b.z, a.w, b.w, bv.z, bv.w);
      }
    }
    // the block's part of C
    const int grp = p.group >= p.k ? 0 : k0 / p.group;
    const float s0 = p.sw[static_cast<size_t>(r0) * p.groups + grp], s1 = p.sw[static_cast<size_t>(r1) * p.groups + grp];
    const int z0 = static_cast<int>(p.zpw ? p.zpw[static_cast<size_t>(r0) * p.groups + grp] : p.default_zp);
    const int z1 = static_cast<int>(p.zpw ? p.zpw[static_cast<size_t>(r1) * p.groups + grp] : p.default_zp);
    const int ia = ta * p.kc + blk, ib = tb * p.kc + blk;
    const int sqa = p.sumqa[ia], sqb = p.sumqa[ib];
    int v[4] = {acc[0] - z0 * sqa, acc[1] - z0 * sqb, acc[2] - z1 * sqa, acc[3] - z1 * sqb};
    if (ASYM) {
      const int c0 = p.comp[static_cast<size_t>(r0) * p.kc + blk], c1 = p.comp[static_cast<size_t>(r1) * p.kc + blk];
      const int za = p.zpa[ia], zb = p.zpa[ib];
      v[0] -= c0 * za;
      v[1] -= c0 * zb;
      v[2] -= c1 * za;
      v[3] -= c1 * zb;
    }
    if (p.acc_out) {
      int32_t* ao = p.acc_out + static_cast<size_t>(blk) * p.m * p.n;
      if (row_lo < p.n && tc0 < p.m) ao[static_cast<size_t>(tc0) * p.n + row_lo] = v[0];
      if (row_lo < p.n && tc1 < p.m) ao[static_cast<size_t>(tc1) * p.n + row_lo] = v[1];
      if (row_hi < p.n && tc0 < p.m) ao[static_cast<size_t>(tc0) * p.n + row_hi] = v[2];
      if (row_hi < p.n && tc1 < p.m) ao[static_cast<size_t>(tc1) * p.n + row_hi] = v[3];
    }
    const float sa_a = p.sa[ia], sa_b = p.sa[ib];
    c[0] += (static_cast<float>(v[0]) * sa_a) * s0;
    c[1] += (static_cast<float>(v[1]) * sa_b) * s0;
    c[2] += (static_cast<float>(v[2]) * sa_a) * s1;
    c[3] += (static_cast<float>(v[3]) * sa_b) * s1;
  }
  red[warp][g][2 * t] = c[0];
  red[warp][g][2 * t + 1] = c[1];
  red[warp][g + 8][2 * t] = c[2];
  red[warp][g + 8][2 * t + 1] = c[3];
  __syncthreads();
  // 128 threads, 128 results: thread -> (row, token)
  const int rr = threadIdx.x >> 3, tt = threadIdx.x & 7;
  const int row = blockIdx.x * 16 + rr, tok = tok0 + tt;
  if (!p.y || row >= p.n || tok >= p.m) return;
  float v = p.bias ? p.bias[row] : 0.f;
#pragma unroll
  for (int w = 0; w < kI8Warps; ++w) v += red[w][rr][tt];
  float r = bf16_round(v);
  const size_t o = static_cast<size_t>(tok) * p.ldy + row;
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

// Many tokens: a CTA owns 64 rows x 64 tokens and walks the whole K.  Warp w keeps the weights of
// its 16 rows of a k-step in registers and runs them against eight 8-token column blocks (the
// four warps read the same activation codes, so three of the four reads hit L1); every warp sees
// every K block, so there is nothing to add across warps.  Against the 16 x 8 kernel above this
// reads the weights 8 times and the activation codes 4 times less often.
constexpr int kWideTokBlocks = 8;
constexpr int kWideTok = 8 * kWideTokBlocks;
constexpr int kWideChunk = 16;             // K blocks whose per-token figures are staged at a time
constexpr int kWideStages = 4;             // k-steps in flight (cp.async ring)
constexpr int kWideStride = kWideTok + 2;  // even (64-bit loads stay aligned), not a multiple of 32

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <bool W4, bool ASYM>
__global__ void __launch_bounds__(kI8Warps * 32) woq_i8_block_wide_kernel(const I8BlockParams p) {
  // A ring of four stages of one 64-wide k-step each: the CTA's 64 weight rows (64 B each, 32 B for 4-bit
  // weights) and the codes of its 64 tokens (64 B each), copied with 16-byte cp.async by all
  // threads (four consecutive threads cover one row's chunk) and read back as MMA fragments.
  // Rows are 64 B apart in shared memory: the two rows a quarter-warp reads together with one
  // 128-bit load are 128 contiguous bytes, so the fragment loads have no bank conflicts.
  constexpr int kWRow = W4 ? 32 : 64;
  __shared__ __align__(16) uint8_t s_w[kWideStages][64 * kWRow];
  __shared__ __align__(16) uint8_t s_a[kWideStages][kWideTok * 64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row_lo = blockIdx.x * 64 + warp * 16 + g, row_hi = row_lo + 8;
  const int tok0 = blockIdx.y * kWideTok;
  const int r0 = row_lo < p.n ? row_lo : 0, r1 = row_hi < p.n ? row_hi : 0;
  const size_t row_bytes = W4 ? p.k / 2 : p.k;
  // column block nt: this lane feeds the codes of token tok0 + 8 nt + g and owns the accumulator
  // columns of tokens tok0 + 8 nt + 2t, + 1; rows and tokens outside the problem read row / token 0
  // this thread's 16-byte pieces of a stage: piece c -> (row or token c / 4 (c / 2 for 4-bit
  // weights), 16-byte part c % 4 (c % 2))
  constexpr int kWParts = kWRow / 16, kWPieces = 64 * kWParts / (kI8Warps * 32);
  const uint8_t* src_w[kWPieces > 0 ? kWPieces : 1];
  int dst_w[kWPieces > 0 ? kWPieces : 1];
#pragma unroll
  for (int j = 0; j < kWPieces; ++j) {
    const int cidx = threadIdx.x + j * kI8Warps * 32, r = cidx / kWParts, part = cidx % kWParts;
    const int gr = blockIdx.x * 64 + r;
    src_w[j] = p.w + static_cast<size_t>(gr < p.n ? gr : 0) * row_bytes + part * 16;
    dst_w[j] = r * kWRow + part * 16;
  }
  const uint8_t* src_a[2];
  int dst_a[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int cidx = threadIdx.x + j * kI8Warps * 32, tk = cidx / 4, part = cidx % 4;
    const int gt = tok0 + tk;
    src_a[j] = p.qa + static_cast<size_t>(gt < p.m ? gt : 0) * p.k + part * 16;
    dst_a[j] = tk * 64 + part * 16;
  }
  const int steps = p.k / 64;  // k-steps over the whole K (a K block is kb / 64 of them)
  // one commit group per k-step, empty beyond the last, so that "all but the newest
  // kWideStages - 2 groups have landed" always means "this iteration's step has landed"
  auto issue = [&](int step) {
    if (step < steps) {
      const int koff = step * 64, stage = step % kWideStages;
#pragma unroll
      for (int j = 0; j < kWPieces; ++j) cp_async16(&s_w[stage][dst_w[j]], src_w[j] + (W4 ? koff / 2 : koff));
#pragma unroll
      for (int j = 0; j < 2; ++j) cp_async16(&s_a[stage][dst_a[j]], src_a[j] + koff);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int st = 0; st < kWideStages - 1; ++st) issue(st);
  // C starts from the fp32 bias and takes the K blocks in order, as the reference does
  const float b_lo = p.bias ? p.bias[r0] : 0.f, b_hi = p.bias ? p.bias[r1] : 0.f;
  float c[kWideTokBlocks][4];
#pragma unroll
  for (int nt = 0; nt < kWideTokBlocks; ++nt) {
    c[nt][0] = c[nt][1] = b_lo;
    c[nt][2] = c[nt][3] = b_hi;
  }

  // scales, code sums and zero points of the CTA's 64 tokens for 32 K blocks at a time,
  // transposed to [block][token]: the drain of a block reads them with two or three shared loads
  // per column block instead of four to six global ones
  __shared__ __align__(8) float s_sa[kWideChunk][kWideStride];
  __shared__ __align__(8) int s_sq[kWideChunk][kWideStride];
  __shared__ __align__(8) int s_zp[ASYM ? kWideChunk : 1][kWideStride];
  for (int blk = 0; blk < p.kc; ++blk) {
    if ((blk % kWideChunk) == 0) {
      __syncthreads();  // everyone is done with the previous chunk
      for (int i = threadIdx.x; i < kWideTok * kWideChunk; i += kI8Warps * 32) {
        const int tok = i / kWideChunk, b = i % kWideChunk;
        const int gt = tok0 + tok < p.m ? tok0 + tok : 0;
        if (blk + b < p.kc) {
          const size_t src = static_cast<size_t>(gt) * p.kc + blk + b;
          s_sa[b][tok] = p.sa[src];
          s_sq[b][tok] = p.sumqa[src];
          if (ASYM) s_zp[b][tok] = p.zpa[src];
        }
      }
      __syncthreads();
    }
    const int bl = blk % kWideChunk;
    int acc[kWideTokBlocks][4];
#pragma unroll
    for (int nt = 0; nt < kWideTokBlocks; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0;
    const int k0 = blk * p.kb;
    for (int kk = 0; kk < p.kb; kk += 64) {
      const int step = (k0 + kk) / 64, stage = step % kWideStages;
      cp_async_wait<kWideStages - 2>();  // this step's copies of this thread have landed
      __syncthreads();                   // ... everyone's have, and everyone has left the previous step's buffer
      issue(step + kWideStages - 1);     // which is the buffer this copy goes to
      uint32_t a[8];  // A fragments of the two k32 MMAs: rows g and g + 8 of this warp's 16
      const int wr = warp * 16 + g;
      if (W4) {
        const uint2 u = *reinterpret_cast<const uint2*>(&s_w[stage][wr * kWRow + 8 * t]);
        const uint2 v = *reinterpret_cast<const uint2*>(&s_w[stage][(wr + 8) * kWRow + 8 * t]);
        a[0] = u.x & 0x0f0f0f0fu; a[1] = v.x & 0x0f0f0f0fu; a[2] = (u.x >> 4) & 0x0f0f0f0fu; a[3] = (v.x >> 4) & 0x0f0f0f0fu;
        a[4] = u.y & 0x0f0f0f0fu; a[5] = v.y & 0x0f0f0f0fu; a[6] = (u.y >> 4) & 0x0f0f0f0fu; a[7] = (v.y >> 4) & 0x0f0f0f0fu;
      } else {
        const uint4 u = *reinterpret_cast<const uint4*>(&s_w[stage][wr * kWRow + 16 * t]);
        const uint4 v = *reinterpret_cast<const uint4*>(&s_w[stage][(wr + 8) * kWRow + 16 * t]);
        a[0] = u.x; a[1] = v.x; a[2] = u.y; a[3] = v.y;
        a[4] = u.z; a[5] = v.z; a[6] = u.w; a[7] = v.w;
      }
#pragma unroll
      for (int nt = 0; nt < kWideTokBlocks; ++nt) {
        const uint4 bv = *reinterpret_cast<const uint4*>(&s_a[stage][(8 * nt + g) * 64 + 16 * t]);
        mma_i8<W4, ASYM>(acc[nt], a[0], a[1], a[2], a[3], bv.x, bv.y);
        mma_i8<W4, ASYM>(acc[nt], a[4], a[5], a[6], a[7], bv.z, bv.w);
      }
    }
    // the block's part of C, as in the 16 x 8 kernel
    const int grp = p.group >= p.k ? 0 : k0 / p.group;
    const float s0 = p.sw[static_cast<size_t>(r0) * p.groups + grp], s1 = p.sw[static_cast<size_t>(r1) * p.groups + grp];
    const int z0 = static_cast<int>(p.zpw ? p.zpw[static_cast<size_t>(r0) * p.groups + grp] : p.default_zp);
    const int z1 = static_cast<int>(p.zpw ? p.zpw[static_cast<size_t>(r1) * p.groups + grp] : p.default_zp);
    int c0 = 0, c1 = 0;
    if (ASYM) {
      c0 = p.comp[static_cast<size_t>(r0) * p.kc + blk];
      c1 = p.comp[static_cast<size_t>(r1) * p.kc + blk];
    }
#pragma unroll
    for (int nt = 0; nt < kWideTokBlocks; ++nt) {
      // tokens 8 nt + 2t and + 1 of the CTA (a token outside the problem holds token 0's figures)
      const int2 sq = *reinterpret_cast<const int2*>(&s_sq[bl][8 * nt + 2 * t]);
      const float2 sav = *reinterpret_cast<const float2*>(&s_sa[bl][8 * nt + 2 * t]);
      const int sqa = sq.x, sqb = sq.y;
      int v[4] = {acc[nt][0] - z0 * sqa, acc[nt][1] - z0 * sqb, acc[nt][2] - z1 * sqa, acc[nt][3] - z1 * sqb};
      if (ASYM) {
        const int2 zz = *reinterpret_cast<const int2*>(&s_zp[bl][8 * nt + 2 * t]);
        const int za = zz.x, zb = zz.y;
        v[0] -= c0 * za;
        v[1] -= c0 * zb;
        v[2] -= c1 * za;
        v[3] -= c1 * zb;
      }
      if (p.acc_out) {
        const int tc0 = tok0 + 8 * nt + 2 * t, tc1 = tc0 + 1;
        int32_t* ao = p.acc_out + static_cast<size_t>(blk) * p.m * p.n;
        if (row_lo < p.n && tc0 < p.m) ao[static_cast<size_t>(tc0) * p.n + row_lo] = v[0];
        if (row_lo < p.n && tc1 < p.m) ao[static_cast<size_t>(tc1) * p.n + row_lo] = v[1];
        if (row_hi < p.n && tc0 < p.m) ao[static_cast<size_t>(tc0) * p.n + row_hi] = v[2];
        if (row_hi < p.n && tc1 < p.m) ao[static_cast<size_t>(tc1) * p.n + row_hi] = v[3];
      }
      const float sa_a = sav.x, sa_b = sav.y;
      c[nt][0] += (static_cast<float>(v[0]) * sa_a) * s0;
      c[nt][1] += (static_cast<float>(v[1]) * sa_b) * s0;
      c[nt][2] += (static_cast<float>(v[2]) * sa_a) * s1;
      c[nt][3] += (static_cast<float>(v[3]) * sa_b) * s1;
    }
  }
  if (!p.y) return;
#pragma unroll
  for (int nt = 0; nt < kWideTokBlocks; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (i & 2) ? row_hi : row_lo;
      const int tok = tok0 + 8 * nt + 2 * t + (i & 1);
      if (row >= p.n || tok >= p.m) continue;
      float r = bf16_round(c[nt][i]);
      const size_t o = static_cast<size_t>(tok) * p.ldy + row;
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

}  // namespace

cudaError_t launch_act_block_quant(const __nv_bfloat16* x, int64_t ldx, int m, int k, int kb, int act_mode,
                                   int interleave, uint8_t* qa, float* sa, int32_t* zpa, int32_t* sumqa,
                                   float* range, float* folded, cudaStream_t stream) {
  const int kc = (k + kb - 1) / kb, base = act_mode & 3;
  const unsigned blocks = static_cast<unsigned>((static_cast<int64_t>(m) * kc + 7) / 8);
  act_block_range_kernel<<<blocks, 256, 0, stream>>>(x, ldx, m, k, kb, kc, range);
  if (base != 3) {
    const int outs = base == 0 ? 1 : base == 1 ? kc : m;
    act_fold_range_kernel<<<outs, 256, 0, stream>>>(range, m, kc, base, folded);
  }
  if (act_mode >= 4)
    act_block_quant_kernel<false><<<blocks, 256, 0, stream>>>(x, ldx, m, k, kb, kc, base, range, folded, interleave,
                                                              qa, sa, zpa, sumqa);
  else
    act_block_quant_kernel<true><<<blocks, 256, 0, stream>>>(x, ldx, m, k, kb, kc, base, range, folded, interleave,
                                                             qa, sa, zpa, sumqa);
  return cudaGetLastError();
}

cudaError_t launch_weight_block_sum(const uint8_t* w, const float* zpw, int n, int k, int kb, int group, int groups,
                                    float default_zp, int w4, int32_t* comp, cudaStream_t stream) {
  const int kc = k / kb;
  const unsigned blocks = static_cast<unsigned>((static_cast<int64_t>(n) * kc + 7) / 8);
  if (w4)
    weight_block_sum_kernel<true><<<blocks, 256, 0, stream>>>(w, zpw, n, k, kb, kc, group, groups, default_zp, comp);
  else
    weight_block_sum_kernel<false><<<blocks, 256, 0, stream>>>(w, zpw, n, k, kb, kc, group, groups, default_zp, comp);
  return cudaGetLastError();
}

cudaError_t launch_i8_block(const I8BlockParams& p, cudaStream_t stream) {
  if (p.m > 16) {
    // 64 rows x 64 tokens per CTA
    const dim3 wgrid(static_cast<unsigned>((p.n + 63) / 64), static_cast<unsigned>((p.m + kWideTok - 1) / kWideTok));
    if (wgrid.y > 65535) return cudaErrorInvalidConfiguration;
    if (p.w4) {
      if (p.asym)
        woq_i8_block_wide_kernel<true, true><<<wgrid, kI8Warps * 32, 0, stream>>>(p);
      else
        woq_i8_block_wide_kernel<true, false><<<wgrid, kI8Warps * 32, 0, stream>>>(p);
    } else {
      if (p.asym)
        woq_i8_block_wide_kernel<false, true><<<wgrid, kI8Warps * 32, 0, stream>>>(p);
      else
        woq_i8_block_wide_kernel<false, false><<<wgrid, kI8Warps * 32, 0, stream>>>(p);
    }
    return cudaGetLastError();
  }
  const dim3 grid(static_cast<unsigned>((p.n + 15) / 16), static_cast<unsigned>((p.m + 7) / 8));
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  if (p.w4) {
    if (p.asym)
      woq_i8_block_kernel<true, true><<<grid, kI8Warps * 32, 0, stream>>>(p);
    else
      woq_i8_block_kernel<true, false><<<grid, kI8Warps * 32, 0, stream>>>(p);
  } else {
    if (p.asym)
      woq_i8_block_kernel<false, true><<<grid, kI8Warps * 32, 0, stream>>>(p);
    else
      woq_i8_block_kernel<false, false><<<grid, kI8Warps * 32, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace woq
