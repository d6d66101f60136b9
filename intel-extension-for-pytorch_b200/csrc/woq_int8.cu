// INT8-compute path (WoqLowpMode.INT8 with INT8 symmetric per-channel weights):
//   * prepack of the plain [N, K] int8 weight into "operand images": tiles of 64 rows x 128 k,
//     8 KB each, stored exactly as the tensor core wants a K-major 128-byte-swizzled operand
//     (row r of an 8-row group at r*128 bytes, its 16-byte chunk c at position c ^ r), so a
//     bulk copy of two consecutive images is a ready 128-row A operand - no tensor map needed;
//   * dynamic per-token symmetric quantisation of the bf16 activations (true division, round
//     half to even): the reference's dynamic_quantize_per_block for QUANT_A_PER_M_SYM;
//   * one tcgen05 kernel (kind::i8, int32 accumulators in TMEM) for every token count: weights
//     need no dequantisation, so even for one token an MMA covers 4 KB of weights and the
//     kernel stays memory-bound.  Stream-K over (tile, k-chunk) with int32 partial tiles:
//     the accumulators do not depend on how K was split.
#include <cuda_fp16.h>

#include <cstdlib>

#include "woq_kernels.h"
#include "woq_tc_common.cuh"

namespace woq {

namespace {

// ---- operand image layout -------------------------------------------------------------
__host__ __device__ inline int image_offset(int r /*0..63*/, int kbyte /*0..127*/) {
  return (r >> 3) * 1024 + (r & 7) * 128 + ((((kbyte >> 4) ^ (r & 7))) << 4) + (kbyte & 15);
}

__global__ void pack_int8_kernel(const int8_t* plain, int8_t* tiled, int n, int k, int tiles64,
                                 int kc_per_tile, int gate_up) {
  // one thread per 16 bytes of the image
  const int64_t total = static_cast<int64_t>(tiles64) * kc_per_tile * 512;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int chunk = i & 7, r = (i >> 3) & 63;
  const int64_t blk = i >> 9;
  const int kc = static_cast<int>(blk % kc_per_tile), t64 = static_cast<int>(blk / kc_per_tile);
  const int row128 = (t64 & 1) * 64 + r;
  const int nn = tc_tile_row_to_n(n, gate_up, t64 >> 1, row128);
  uint4 v = make_uint4(0, 0, 0, 0);
  if (nn < n) v = *reinterpret_cast<const uint4*>(plain + static_cast<int64_t>(nn) * k + kc * 128 + chunk * 16);
  *reinterpret_cast<uint4*>(tiled + blk * 8192 + image_offset(r, chunk * 16)) = v;
}

__global__ void unpack_int8_kernel(const int8_t* tiled, int8_t* plain, int n, int k, int kc_per_tile,
                                   int gate_up) {
  const int64_t chunks_per_row = k / 16;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(n) * chunks_per_row) return;
  const int nn = static_cast<int>(i / chunks_per_row), ch = static_cast<int>(i % chunks_per_row);
  int tile128, row128;
  if (gate_up) {
    const int half = n / 2, idx = nn < half ? nn : nn - half;
    tile128 = idx / 64;
    row128 = (idx % 64) + (nn < half ? 0 : 64);
  } else {
    tile128 = nn / 128;
    row128 = nn % 128;
  }
  const int t64 = tile128 * 2 + (row128 >> 6), r = row128 & 63;
  const int kc = ch / 8, chunk = ch % 8;
  const int64_t blk = static_cast<int64_t>(t64) * kc_per_tile + kc;
  *reinterpret_cast<uint4*>(plain + static_cast<int64_t>(nn) * k + ch * 16) =
      *reinterpret_cast<const uint4*>(tiled + blk * 8192 + image_offset(r, chunk * 16));
}

__global__ void pad_scale_kernel(const void* src, float* dst, int n, int n_pad, int dtype) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pad) return;
  float v = 0.f;
  if (i < n) {
    if (dtype == 1) v = reinterpret_cast<const float*>(src)[i];
    else if (dtype == 2) v = __half2float(reinterpret_cast<const __half*>(src)[i]);
    else v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i]);
  }
  dst[i] = v;
}

// ---- dynamic activation quantisation ------------------------------------------------------
// Follows dynamic_quantize_per_block (csrc/cpu/aten/utils/woq_dynamic_quant.h:1526-1750).
// Symmetric: scale = max(|max|, |min|) / 127, q = clamp(nearbyint(x / scale), -128, 127) as s8.
// Asymmetric: scale = (max - min) / 255, zp = -nearbyint(min / scale),
// q = clamp(nearbyint(x / scale + zp), 0, 255) as u8.  True division, round-half-even; no
// clamping of the range to zero and no epsilon; a constant row of zeros gets codes 0.
// Per token: one range per row.  Per tensor: one range over all rows (act_row_range_kernel
// first, then every CTA folds the row ranges).  One CTA per token row.
__device__ __forceinline__ void block_min_max(float& lo, float& hi, float* red) {
  const int tid = threadIdx.x;
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
  lo = red[0];
  hi = red[8];
#pragma unroll
  for (int i = 1; i < 8; ++i) {
    lo = fminf(lo, red[i]);
    hi = fmaxf(hi, red[8 + i]);
  }
  __syncthreads();
}

__device__ __forceinline__ void row_min_max(const __nv_bfloat16* xr, int k, float& lo, float& hi) {
  lo = INFINITY;
  hi = -INFINITY;
  for (int i = threadIdx.x * 8; i < k; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __uint_as_float(w[j] << 16), b = __uint_as_float(w[j] & 0xffff0000u);
      lo = fminf(lo, fminf(a, b));
      hi = fmaxf(hi, fmaxf(a, b));
    }
  }
}

__global__ void __launch_bounds__(256) act_row_range_kernel(const __nv_bfloat16* x, int64_t ldx, int k,
                                                            float* range) {
  __shared__ float red[16];
  float lo, hi;
  row_min_max(x + static_cast<int64_t>(blockIdx.x) * ldx, k, lo, hi);
  block_min_max(lo, hi, red);
  if (threadIdx.x == 0) {
    range[2 * blockIdx.x] = lo;
    range[2 * blockIdx.x + 1] = hi;
  }
}

// range: null (per token) or the [m_total][2] row ranges of the whole tensor (per tensor)
template <bool ASYM>
__global__ void __launch_bounds__(256) quant_act_kernel(const __nv_bfloat16* x, int64_t ldx, int k,
                                                        int8_t* qa, float* sa, int32_t* zpa,
                                                        const float* range, int m_total) {
  __shared__ float red[16];
  const int m = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(m) * ldx;
  float lo, hi;
  if (range) {
    lo = INFINITY;
    hi = -INFINITY;
    for (int i = tid; i < m_total; i += 256) {
      lo = fminf(lo, range[2 * i]);
      hi = fmaxf(hi, range[2 * i + 1]);
    }
  } else {
    row_min_max(xr, k, lo, hi);
  }
  block_min_max(lo, hi, red);
  float scale, zp = 0.f;
  if (ASYM) {
    scale = __fdiv_rn(hi - lo, 255.0f);
    const float z = -rintf(__fdiv_rn(lo, scale));
    zp = z;
    if (tid == 0) zpa[m] = scale > 0.f ? static_cast<int32_t>(z) : 0;
  } else {
    scale = __fdiv_rn(fmaxf(fabsf(hi), fabsf(lo)), 127.0f);
  }
  if (tid == 0) sa[m] = scale;
  const float q_lo = ASYM ? 0.f : -128.f, q_hi = ASYM ? 255.f : 127.f;
  int8_t* qr = qa + static_cast<int64_t>(m) * k;
  for (int i = tid * 8; i < k; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __uint_as_float(w[j] << 16), b = __uint_as_float(w[j] & 0xffff0000u);
      float ql = 0.f, qh = 0.f;
      if (scale > 0.f) {
        ql = fminf(fmaxf(rintf(__fdiv_rn(a, scale) + zp), q_lo), q_hi);
        qh = fminf(fmaxf(rintf(__fdiv_rn(b, scale) + zp), q_lo), q_hi);
      }
      const uint32_t c = (static_cast<uint32_t>(static_cast<int>(ql)) & 0xffu) |
                         ((static_cast<uint32_t>(static_cast<int>(qh)) & 0xffu) << 8);
      out[j >> 1] |= c << ((j & 1) * 16);
    }
    *reinterpret_cast<uint2*>(qr + i) = make_uint2(out[0], out[1]);
  }
}

// RMSNorm fused with the per-token quantiser: one CTA per token row.
//   y = bf16(x * rsqrt(mean(x^2) + eps) * gamma)   (fp32 arithmetic, one rounding)
// and then exactly what quant_act_kernel does on y, without y making a round trip through
// memory (it is written only when the caller wants it).  Three passes over the row, which
// stays in L1 after the first.
template <bool ASYM>
__global__ void __launch_bounds__(256) rmsnorm_quant_kernel(const __nv_bfloat16* x, int64_t ldx,
                                                            const __nv_bfloat16* gamma, float eps, int k,
                                                            __nv_bfloat16* y, int64_t ldy, int8_t* qa, float* sa,
                                                            int32_t* zpa) {
  __shared__ float red[16];
  const int m = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(m) * ldx;
  // pass 1: sum of squares
  float ss = 0.f;
  for (int i = tid * 8; i < k; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __uint_as_float(w[j] << 16), b = __uint_as_float(w[j] & 0xffff0000u);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  ss = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) ss += red[i];
  __syncthreads();
  const float inv = rsqrtf(__fdiv_rn(ss, static_cast<float>(k)) + eps);
  auto normed = [&](uint32_t xw, uint32_t gw, float& a, float& b) {
    a = bf16_round(__uint_as_float(xw << 16) * inv * __uint_as_float(gw << 16));
    b = bf16_round(__uint_as_float(xw & 0xffff0000u) * inv * __uint_as_float(gw & 0xffff0000u));
  };
  // pass 2: range of the normalised row (and y itself, if wanted)
  float lo = INFINITY, hi = -INFINITY;
  for (int i = tid * 8; i < k; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint4 g = *reinterpret_cast<const uint4*>(gamma + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w}, gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a, b;
      normed(w[j], gw[j], a, b);
      lo = fminf(lo, fminf(a, b));
      hi = fmaxf(hi, fmaxf(a, b));
      out[j] = (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xffff0000u);
    }
    if (y) *reinterpret_cast<uint4*>(y + static_cast<int64_t>(m) * ldy + i) = make_uint4(out[0], out[1], out[2], out[3]);
  }
  block_min_max(lo, hi, red);
  float scale, zp = 0.f;
  if (ASYM) {
    scale = __fdiv_rn(hi - lo, 255.0f);
    const float z = -rintf(__fdiv_rn(lo, scale));
    zp = z;
    if (tid == 0) zpa[m] = scale > 0.f ? static_cast<int32_t>(z) : 0;
  } else {
    scale = __fdiv_rn(fmaxf(fabsf(hi), fabsf(lo)), 127.0f);
  }
  if (tid == 0) sa[m] = scale;
  const float q_lo = ASYM ? 0.f : -128.f, q_hi = ASYM ? 255.f : 127.f;
  int8_t* qr = qa + static_cast<int64_t>(m) * k;
  // pass 3: codes
  for (int i = tid * 8; i < k; i += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const uint4 g = *reinterpret_cast<const uint4*>(gamma + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w}, gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a, b;
      normed(w[j], gw[j], a, b);
      float ql = 0.f, qh = 0.f;
      if (scale > 0.f) {
        ql = fminf(fmaxf(rintf(__fdiv_rn(a, scale) + zp), q_lo), q_hi);
        qh = fminf(fmaxf(rintf(__fdiv_rn(b, scale) + zp), q_lo), q_hi);
      }
      const uint32_t c = (static_cast<uint32_t>(static_cast<int>(ql)) & 0xffu) |
                         ((static_cast<uint32_t>(static_cast<int>(qh)) & 0xffu) << 8);
      out[j >> 1] |= c << ((j & 1) * 16);
    }
    *reinterpret_cast<uint2*>(qr + i) = make_uint2(out[0], out[1]);
  }
}

// compensation[n] = sum over k of the weight codes of row n (plain [n][k] int8): what an
// activation zero point contributes to every accumulator of that row.  One warp per row.
__global__ void __launch_bounds__(256) weight_row_sum_kernel(const int8_t* w, int n, int k, int32_t* comp) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const int8_t* wr = w + static_cast<int64_t>(row) * k;
  int sum = 0;
  for (int i = lane * 16; i < k; i += 32 * 16) {
    const uint4 v = *reinterpret_cast<const uint4*>(wr + i);
    const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) sum = __dp4a(static_cast<int>(q[j]), 0x01010101, sum);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) comp[row] = sum;
}

// ---- tcgen05 int8 GEMM -------------------------------------------------------------------
constexpr int kEpiWarps = 16;  // four warpgroups; warp w reads TMEM lanes 32 * (w % 4) ...
constexpr int kI8Threads = (kEpiWarps + 3) * 32;
constexpr int kI8Producer = kEpiWarps, kI8Mma = kEpiWarps + 1, kI8Mma2 = kEpiWarps + 2;
constexpr int kI8MaxStages = 8;
constexpr int kI8HeaderBytes = 1024;
constexpr int kI8TmemCols = 256;
constexpr int kChunkBytes = 16384;  // 128 rows x 128 k

struct I8Header {
  uint64_t full[kI8MaxStages], empty[kI8MaxStages];
  uint64_t issued[2];  // MMA warp t has issued the MMAs of its latest k-chunk
  uint64_t d_full, d_empty;
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

__device__ __forceinline__ int i8_owner_of(int64_t b, int64_t total, int64_t ctas) {
  return static_cast<int>(((b + 1) * ctas - 1) / total);
}

// (acc - compensation[n] * zp_a[tok]) * scale_a[tok] * scale_w[n]: the integer part is exact
// (csrc/cpu/aten/utils/woq.h:2310-2321)
__device__ __forceinline__ float i8_scaled(const I8Params& p, int acc, int tok, int n) {
  if (p.zpa) acc -= p.comp[n] * p.zpa[tok];
  return (static_cast<float>(acc) * p.sa[tok]) * p.sw[n];
}

__device__ __forceinline__ void i8_store(const I8Params& p, int tile, int row, int tok, int acc) {
  const int n = tc_tile_row_to_n(p.n, p.gate_up, tile, row);
  if (tok >= p.m || n >= p.n) return;
  // C = bias + (float(acc) * scale_a) * scale_w   (fp32), then bf16 and the post-op
  float v = i8_scaled(p, acc, tok, n);
  if (p.bias) v = p.bias[n] + v;
  float r = bf16_round(v);
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

// Eight tokens (chunk ch) of one row, four at a time: the fused operands of four tokens are
// loaded before the first is used (raw bits, converted at use), so they cost one global round
// trip, not one per token (four, not eight: the kernel has no registers to spare).
__device__ __forceinline__ void i8_store8(const I8Params& p, int tile, int row, int ch, const int* acc) {
  const bool binary = p.fusion == FUSE_ADD || p.fusion == FUSE_ADD_ADD || p.fusion == FUSE_MUL;
  const int n = tc_tile_row_to_n(p.n, p.gate_up, tile, row);
  if (!binary || n >= p.n || p.m <= 16) {  // few tokens: the plain routine is as fast
#pragma unroll
    for (int e = 0; e < 8; ++e) i8_store(p, tile, row, ch * 8 + e, acc[e]);
    return;
  }
  const unsigned short* o0 = reinterpret_cast<const unsigned short*>(p.other0);
  const unsigned short* o1 = reinterpret_cast<const unsigned short*>(p.other1);
#pragma unroll
  for (int h = 0; h < 8; h += 4) {
    uint32_t f[4];
    float r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (ch * 8 + h + e < p.m) f[e] = o0[static_cast<size_t>(ch * 8 + h + e) * p.ldy + n];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (ch * 8 + h + e < p.m) {
        float v = i8_scaled(p, acc[h + e], ch * 8 + h + e, n);
        if (p.bias) v = p.bias[n] + v;
        const float a = __uint_as_float(f[e] << 16);
        r[e] = p.fusion == FUSE_MUL ? bf16_round(bf16_round(v) * a) : bf16_round(bf16_round(v) + a);
      }
    if (p.fusion == FUSE_ADD_ADD) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (ch * 8 + h + e < p.m) f[e] = o1[static_cast<size_t>(ch * 8 + h + e) * p.ldy + n];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (ch * 8 + h + e < p.m) r[e] = bf16_round(r[e] + __uint_as_float(f[e] << 16));
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (ch * 8 + h + e < p.m)
        p.y[static_cast<size_t>(ch * 8 + h + e) * p.ldy + n] = __float2bfloat16_rn(r[e]);
  }
}

__global__ void __launch_bounds__(kI8Threads, 1)
    woq_int8_tc_kernel(const I8Params p, const __grid_constant__ CUtensorMap qamap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  I8Header* hdr = reinterpret_cast<I8Header*>(smem);
  const int b_stage_bytes = p.n_tok * 128;
  const int stage_bytes = kChunkBytes + b_stage_bytes;
  uint8_t* stages = smem + kI8HeaderBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (smem_u32(smem) & 1023u) {
    if (tid == 0) atomicCAS(p.status, 0, 99);
    return;
  }
  const int64_t total = static_cast<int64_t>(p.tiles) * p.kc_per_tile;
  const int64_t b_begin = (static_cast<int64_t>(blockIdx.x) * total) / gridDim.x;
  const int64_t b_end = (static_cast<int64_t>(blockIdx.x + 1) * total) / gridDim.x;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], 1);
    }
    mbar_init(&hdr->issued[0], 1);
    mbar_init(&hdr->issued[1], 1);
    mbar_init(&hdr->d_full, 2);
    mbar_init(&hdr->d_empty, kEpiWarps);
    hdr->abort_flag = 0;
    hdr->is_last = 0;
    mbar_fence_init();
  }
  if (warp == kI8Mma) {
    tmem_alloc(&hdr->tmem_base, kI8TmemCols);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = hdr->tmem_base;
  volatile int* abort_flag = &hdr->abort_flag;

  // all roles walk the same sequence of k-chunks: chunk index b -> (tile, kc)
  int tile = static_cast<int>(b_begin / p.kc_per_tile);
  int kc = static_cast<int>(b_begin % p.kc_per_tile);
  int64_t b = b_begin;
  int slot = 0;
  uint32_t phase = 0;
  auto advance = [&]() {
    ++b;
    if (++kc == p.kc_per_tile) {
      kc = 0;
      ++tile;
    }
    if (++slot == p.stages) {
      slot = 0;
      phase ^= 1;
    }
  };

  if (warp == kI8Producer) {
    if (lane == 0) {
      while (b < b_end) {
        uint8_t* st = stages + static_cast<size_t>(slot) * stage_bytes;
        mbar_wait(&hdr->empty[slot], phase ^ 1, abort_flag, p.status, 21);
        mbar_arrive_expect_tx(&hdr->full[slot], kChunkBytes + b_stage_bytes);
        const int8_t* src0 = p.wq + (static_cast<size_t>(2 * tile) * p.kc_per_tile + kc) * 8192;
        const int8_t* src1 = p.wq + (static_cast<size_t>(2 * tile + 1) * p.kc_per_tile + kc) * 8192;
        bulk_g2s(st, src0, 8192, &hdr->full[slot]);
        bulk_g2s(st + 8192, src1, 8192, &hdr->full[slot]);
        tma_load_2d(st + kChunkBytes, &qamap, kc * 128, p.m0, &hdr->full[slot]);
        advance();
      }
    }
  } else if (warp == kI8Mma || warp == kI8Mma2) {
    if (lane == 0) {
      // Two threads issue the MMAs of alternate k-chunks: issuing blocks a thread while the
      // tensor core is busy, and the wait and commit around a chunk cost about as much again.
      // A token (`issued`) keeps the chunks in order, so the MMA that starts a tile's
      // accumulator runs before any that adds to it.
      const int me = warp == kI8Mma ? 0 : 1;
      // A = weights (s8), B = activations (s8, or u8 when quantised asymmetrically)
      const uint32_t idesc = umma_idesc(p.n_tok, /*s8*/ 1, p.zpa ? /*u8*/ 0 : /*s8*/ 1, /*s32*/ 2);
      const uint64_t desc_hi = umma_desc_k128(0) & 0xffffffff00000000ull;
      const uint32_t base_lo = (smem_u32(stages) & 0x3FFFFu) >> 4;
      const uint32_t stage_lo = static_cast<uint32_t>(stage_bytes) >> 4;
      uint32_t seg = 0;
      bool first_of_segment = true;
      int n = 0;  // chunk number within this CTA
      while (b < b_end) {
        const bool seg_end = (kc + 1 == p.kc_per_tile) || (b + 1 == b_end);
        if ((n & 1) == me) {
          mbar_wait(&hdr->full[slot], phase, abort_flag, p.status, 22);
          if (first_of_segment) mbar_wait(&hdr->d_empty, (seg & 1) ^ 1, abort_flag, p.status, 23);
          if (n > 0) mbar_wait(&hdr->issued[me ^ 1], ((n - 1) >> 1) & 1, abort_flag, p.status, 25);
          tc_fence_after_sync();
          uint32_t accumulate = first_of_segment ? 0u : 1u;
          const uint32_t a_lo = base_lo + slot * stage_lo;
          const uint32_t b_lo = a_lo + (kChunkBytes >> 4);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            umma_i8_ss(tmem_base, desc_hi | (a_lo + ks * 2), desc_hi | (b_lo + ks * 2), idesc, accumulate);
            accumulate = 1;
          }
          mbar_arrive(&hdr->issued[me]);
          tc_commit(&hdr->empty[slot]);
        }
        first_of_segment = false;
        if (seg_end) {
          tc_commit(&hdr->d_full);  // both threads: all this thread issued for the segment
          ++seg;
          first_of_segment = true;
        }
        ++n;
        advance();
      }
    }
  } else {
    // ------------------------------- epilogue warps ----------------------------------------
    const int wg = warp >> 2, q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int n_chunks = p.n_tok / 8;  // 8-token column chunks, dealt round-robin to warpgroups
    constexpr int kGroups = kEpiWarps / 4;
    int seg = 0, seg_kc0 = kc;
    bool first_segment = true;
    int pend_tile = -1;
    unsigned pend_old = 0;
    int* partials = reinterpret_cast<int*>(p.partials);

    auto reduce_and_store = [&](int t, bool whole, int own_slot) {
      const int64_t tb0 = static_cast<int64_t>(t) * p.kc_per_tile;
      const int c_first = i8_owner_of(tb0, total, gridDim.x);
      const int c_last = i8_owner_of(tb0 + p.kc_per_tile - 1, total, gridDim.x);
      for (int ch = wg; ch < n_chunks && ch * 8 < p.m; ch += kGroups) {
        // eight tokens at a time, all their loads in flight together
        int v[8], v_up[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v_up[e] = 0;
        for (int cc = c_first; cc <= c_last; ++cc) {
          const int64_t cb = (static_cast<int64_t>(cc) * total) / gridDim.x;
          const int slot2 = whole ? own_slot : cc * 2 + (cb >= tb0 ? 0 : 1);
          const int* src = partials + static_cast<size_t>(slot2) * p.n_tok * kTcTileN +
                           static_cast<size_t>(ch * 8) * kTcTileN + row;
          int part[8], part_up[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            part[e] = __ldcg(src + e * kTcTileN);
            part_up[e] = (p.fusion == FUSE_SILU_MUL && row < 64) ? __ldcg(src + e * kTcTileN + 64) : 0;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            v[e] += part[e];
            v_up[e] += part_up[e];
          }
        }
        if (p.fusion != FUSE_SILU_MUL) {
          i8_store8(p, t, row, ch, v);
          continue;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int tok = ch * 8 + e;
          if (tok >= p.m) break;
          {
            if (row < 64) {
              const int n_gate = t * 64 + row, n_up = p.n / 2 + n_gate;
              if (n_gate < p.n_out) {
                float g = i8_scaled(p, static_cast<int>(v[e]), tok, n_gate);
                float u = i8_scaled(p, static_cast<int>(v_up[e]), tok, n_up);
                if (p.bias) {
                  g = p.bias[n_gate] + g;
                  u = p.bias[n_up] + u;
                }
                p.y[static_cast<size_t>(tok) * p.ldy + n_gate] =
                    __float2bfloat16_rn(bf16_round(u) * silu_bf16(bf16_round(g)));
              }
            }
          }
        }
      }
    };

    while (b < b_end) {
      const bool seg_end = (kc + 1 == p.kc_per_tile) || (b + 1 == b_end);
      if (seg_end) {
        const bool whole = (seg_kc0 == 0 && kc + 1 == p.kc_per_tile);
        mbar_wait(&hdr->d_full, seg & 1, abort_flag, p.status, 24);
        tc_fence_after_sync();
        if (whole && p.fusion != FUSE_SILU_MUL) {
          for (int ch = wg; ch < n_chunks; ch += kGroups) {
            uint32_t v[8];
            tmem_ld_x8(lane_addr + ch * 8, v);
            tc_wait_ld();
            if (p.acc_out) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const int tok = ch * 8 + e, n = tc_tile_row_to_n(p.n, p.gate_up, tile, row);
                if (tok < p.m && n < p.n) p.acc_out[static_cast<size_t>(tok) * p.n + n] = static_cast<int>(v[e]);
              }
            }
            if (p.y) {
              i8_store8(p, tile, row, ch, reinterpret_cast<const int*>(v));
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->d_empty);
        } else {
          const int my_slot = blockIdx.x * 2 + (first_segment ? 0 : 1);
          int* dst = partials + static_cast<size_t>(my_slot) * p.n_tok * kTcTileN;
          for (int ch = wg; ch < n_chunks; ch += kGroups) {
            uint32_t v[8];
            tmem_ld_x8(lane_addr + ch * 8, v);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (ch * 8 + e < p.m)
                __stcg(dst + static_cast<size_t>(ch * 8 + e) * kTcTileN + row, static_cast<int>(v[e]));
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->d_empty);
          named_bar_sync(1, kEpiWarps * 32);
          const bool defer = !whole && first_segment && (b + 1 < b_end);
          if (defer) {
            if (tid == 0) {
              __threadfence();
              pend_old = atomicAdd(p.counters + tile, 1u);
            }
            pend_tile = tile;
          } else {
            if (tid == 0) {
              int last = 1;
              if (!whole) {
                const int64_t tb0 = static_cast<int64_t>(tile) * p.kc_per_tile;
                const int c_first = i8_owner_of(tb0, total, gridDim.x);
                const int c_last = i8_owner_of(tb0 + p.kc_per_tile - 1, total, gridDim.x);
                __threadfence();
                const unsigned old = atomicAdd(p.counters + tile, 1u);
                last = (old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
                if (last) p.counters[tile] = 0;
              }
              hdr->is_last = last;
            }
            named_bar_sync(1, kEpiWarps * 32);
            if (hdr->is_last) {
              __threadfence();
              if (p.acc_out) {
                // accumulators of a split tile: sum of the partial tiles
                const int64_t tb0 = static_cast<int64_t>(tile) * p.kc_per_tile;
                const int c_first = i8_owner_of(tb0, total, gridDim.x);
                const int c_last = i8_owner_of(tb0 + p.kc_per_tile - 1, total, gridDim.x);
                const int n = tc_tile_row_to_n(p.n, p.gate_up, tile, row);
                for (int tok = wg; tok < p.m && n < p.n; tok += kGroups) {
                  int v = 0;
                  for (int cc = c_first; cc <= c_last; ++cc) {
                    const int64_t cb = (static_cast<int64_t>(cc) * total) / gridDim.x;
                    const int slot2 = whole ? my_slot : cc * 2 + (cb >= tb0 ? 0 : 1);
                    v += __ldcg(partials + static_cast<size_t>(slot2) * p.n_tok * kTcTileN +
                                static_cast<size_t>(tok) * kTcTileN + row);
                  }
                  p.acc_out[static_cast<size_t>(tok) * p.n + n] = v;
                }
              }
              if (p.y) reduce_and_store(tile, whole, my_slot);
            }
            named_bar_sync(1, kEpiWarps * 32);
          }
        }
        ++seg;
        first_segment = false;
      }
      advance();
      if (seg_end) seg_kc0 = kc;
    }
    if (pend_tile >= 0) {
      if (tid == 0) {
        const int64_t tb0 = static_cast<int64_t>(pend_tile) * p.kc_per_tile;
        const int c_first = i8_owner_of(tb0, total, gridDim.x);
        const int c_last = i8_owner_of(tb0 + p.kc_per_tile - 1, total, gridDim.x);
        const int last = (pend_old == static_cast<unsigned>(c_last - c_first)) ? 1 : 0;
        if (last) p.counters[pend_tile] = 0;
        hdr->is_last = last;
      }
      named_bar_sync(1, kEpiWarps * 32);
      if (hdr->is_last) {
        __threadfence();
        if (p.acc_out) {
          const int64_t tb0 = static_cast<int64_t>(pend_tile) * p.kc_per_tile;
          const int c_first = i8_owner_of(tb0, total, gridDim.x);
          const int c_last = i8_owner_of(tb0 + p.kc_per_tile - 1, total, gridDim.x);
          const int n = tc_tile_row_to_n(p.n, p.gate_up, pend_tile, row);
          for (int tok = wg; tok < p.m && n < p.n; tok += kGroups) {
            int v = 0;
            for (int cc = c_first; cc <= c_last; ++cc) {
              const int64_t cb = (static_cast<int64_t>(cc) * total) / gridDim.x;
              v += __ldcg(partials + static_cast<size_t>(cc * 2 + (cb >= tb0 ? 0 : 1)) * p.n_tok * kTcTileN +
                          static_cast<size_t>(tok) * kTcTileN + row);
            }
            p.acc_out[static_cast<size_t>(tok) * p.n + n] = v;
          }
        }
        if (p.y) reduce_and_store(pend_tile, false, 0);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kI8Mma) {
    tc_fence_after_sync();
    __syncwarp();  // lane 0 comes from the issuing loop
    tmem_dealloc(tmem_base, kI8TmemCols);
  }
}

inline unsigned blocks_for(int64_t n, int threads) {
  return static_cast<unsigned>((n + threads - 1) / threads);
}

}  // namespace

cudaError_t launch_pack_int8(const int8_t* plain, int8_t* tiled, int n, int k, int tiles64,
                             int gate_up, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(tiles64) * (k / 128) * 512;
  pack_int8_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(plain, tiled, n, k, tiles64, k / 128,
                                                               gate_up);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_unpack_int8(const int8_t* tiled, int8_t* plain, int n, int k, int gate_up,
                               cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(n) * (k / 16);
  unpack_int8_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(tiled, plain, n, k, k / 128, gate_up);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_pad_scale(const void* src, float* dst, int n, int n_pad, int dtype,
                             cudaStream_t stream) {
  pad_scale_kernel<<<blocks_for(n_pad, 256), 256, 0, stream>>>(src, dst, n, n_pad, dtype);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_quant_act(const __nv_bfloat16* x, int64_t ldx, int m, int k, int asym, int per_tensor,
                             int8_t* qa, float* sa, int32_t* zpa, float* range, cudaStream_t stream) {
  if (per_tensor) {
    act_row_range_kernel<<<m, 256, 0, stream>>>(x, ldx, k, range);
    count_launch();
  }
  const float* r = per_tensor ? range : nullptr;
  if (asym)
    quant_act_kernel<true><<<m, 256, 0, stream>>>(x, ldx, k, qa, sa, zpa, r, m);
  else
    quant_act_kernel<false><<<m, 256, 0, stream>>>(x, ldx, k, qa, sa, zpa, r, m);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_rmsnorm_quant(const __nv_bfloat16* x, int64_t ldx, const __nv_bfloat16* gamma, float eps, int m,
                                 int k, int asym, __nv_bfloat16* y, int64_t ldy, int8_t* qa, float* sa, int32_t* zpa,
                                 cudaStream_t stream) {
  if (asym)
    rmsnorm_quant_kernel<true><<<m, 256, 0, stream>>>(x, ldx, gamma, eps, k, y, ldy, qa, sa, zpa);
  else
    rmsnorm_quant_kernel<false><<<m, 256, 0, stream>>>(x, ldx, gamma, eps, k, y, ldy, qa, sa, zpa);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_weight_row_sum(const int8_t* plain, int n, int k, int32_t* comp, cudaStream_t stream) {
  weight_row_sum_kernel<<<(n + 7) / 8, 256, 0, stream>>>(plain, n, k, comp);
  count_launch();
  return cudaGetLastError();
}

size_t int8_partial_bytes(int grid, int n_tok) {
  return static_cast<size_t>(grid) * 2 * n_tok * kTcTileN * sizeof(int);
}

cudaError_t launch_int8_tc(I8Params p, const CUtensorMap& qamap, int grid, cudaStream_t stream) {
  const int stage_bytes = kChunkBytes + p.n_tok * 128;
  int stages = (200 * 1024 - kI8HeaderBytes) / stage_bytes;
  if (stages > kI8MaxStages) stages = kI8MaxStages;
  if (stages < 2) return cudaErrorInvalidConfiguration;
  p.stages = stages;
  const size_t smem = kI8HeaderBytes + static_cast<size_t>(stages) * stage_bytes;
  cudaError_t e = cudaFuncSetAttribute(woq_int8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  woq_int8_tc_kernel<<<grid, kI8Threads, smem, stream>>>(p, qamap);
  count_launch();
  return cudaGetLastError();
}

}  // namespace woq
