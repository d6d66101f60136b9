// General WOQ linear: every weight dtype (INT4, NF4, INT8, FP8 e4m3), every compute dtype the
// reference routes to (fp32, fp16, bf16: csrc/cpu/aten/kernels/WoqLinearKrnl.cpp:75-165), any
// K and any group size that is a multiple of 8, on the plain weight layout the reference's
// Python side hands over ([N, ceil(K/2)] nibbles, even k low, or [N, K] bytes).
//
// It is the route for what the tuned kernels do not take (they cover INT4 with bf16 compute on
// 64-aligned shapes and INT8 with INT8 compute): a functional kernel on the CUDA cores, not a
// tuned one.  A warp owns four output rows and walks the whole K for eight tokens at a time;
// a lane dequantises eight consecutive weights of each row per step,
//     w = round_c((code - zp) * round_c(scale)),   round_c = rounding to the compute dtype,
// multiplies them with the activations (rounded to the compute dtype) and accumulates in fp32;
// the lanes' sums meet in a shuffle tree.  Nothing is split along K, so results do not depend
// on the launch shape.  Larger token counts run as several passes over the weights.
#include <cuda_fp16.h>

#include "../../include/woq_b200.h"
#include "woq_kernels.h"

namespace woq {

namespace {

constexpr int kRows = 4;    // output rows per warp
constexpr int kTok = 8;     // tokens per pass
constexpr int kWarps = 4;   // warps per CTA

// NF4 code -> value (reference: csrc/cpu/aten/utils/woq_utils.h:34-51)
__constant__ float kNf4[16] = {-1.0f,
                               -0.6961928009986877f,
                               -0.5250730514526367f,
                               -0.39491748809814453f,
                               -0.28444138169288635f,
                               -0.18477343022823334f,
                               -0.09105003625154495f,
                               0.0f,
                               0.07958029955625534f,
                               0.16093020141124725f,
                               0.24611230194568634f,
                               0.33791524171829224f,
                               0.44070982933044434f,
                               0.5626170039176941f,
                               0.7229568362236023f,
                               1.0f};

// FP8 e4m3 byte -> fp32, bit for bit the reference's conversion
// (csrc/cpu/aten/utils/woq.h:465-483): exponent rebias by 120, three mantissa bits, zero when
// the low seven bits are zero; no special case for NaN or subnormal codes.
__device__ __forceinline__ float fp8_e4m3_to_f32(uint32_t x) {
  if ((x & 127u) == 0u) return __uint_as_float((x & 128u) << 24);
  const uint32_t bits = ((x & 7u) << 20) | ((((x >> 3) & 15u) + 120u) << 23) | ((x & 128u) << 24);
  return __uint_as_float(bits);
}

template <int C>
__device__ __forceinline__ float round_c(float v) {
  if (C == WOQ_B200_T_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (C == WOQ_B200_T_F16) return __half2float(__float2half_rn(v));
  return v;
}
__device__ __forceinline__ float round_io(float v, int io) {
  if (io == WOQ_B200_T_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (io == WOQ_B200_T_F16) return __half2float(__float2half_rn(v));
  return v;
}
__device__ __forceinline__ float load_io(const void* p, size_t i, int io) {
  if (io == WOQ_B200_T_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (io == WOQ_B200_T_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return static_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_io(void* p, size_t i, float v, int io) {
  if (io == WOQ_B200_T_BF16)
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else if (io == WOQ_B200_T_F16)
    static_cast<__half*>(p)[i] = __float2half_rn(v);
  else
    static_cast<float*>(p)[i] = v;
}

// post-ops on data of the io dtype: fp32 arithmetic inside, one rounding to the io dtype per
// op (silu rounds the sigmoid as well), as the reference's epilogue does on its output type
__device__ __forceinline__ float post_op_io(float y, const GenericParams& p, size_t o) {
  const int io = p.io_dtype;
  switch (p.fusion) {
    case FUSE_GELU_ERF: return round_io(0.5f * y * (1.0f + erff(y * 0.70710678118654752f)), io);
    case FUSE_GELU_TANH: {
      const float inner = 0.7978845608028654f * (y + 0.044715f * y * y * y);
      return round_io(0.5f * y * (1.0f + tanhf(inner)), io);
    }
    case FUSE_RELU: return fmaxf(y, 0.0f);
    case FUSE_SILU: {
      const float sig = round_io(1.0f / (1.0f + expf(-y)), io);
      return round_io(y * sig, io);
    }
    case FUSE_ADD: return round_io(y + load_io(p.other0, o, io), io);
    case FUSE_ADD_ADD: return round_io(round_io(y + load_io(p.other0, o, io), io) + load_io(p.other1, o, io), io);
    case FUSE_MUL: return round_io(y * load_io(p.other0, o, io), io);
    default: return y;
  }
}

// the eight codes of one 8-k chunk of row `row` as floats (before zero point and scale)
template <int WD>
__device__ __forceinline__ void load_codes(const GenericParams& p, int row, int k0, float (&c)[8]) {
  if (WD == WOQ_B200_DTYPE_INT4 || WD == WOQ_B200_DTYPE_NF4) {
    const uint8_t* src = p.w + static_cast<size_t>(row) * p.row_bytes + (k0 >> 1);
    uint32_t word;
    if ((p.row_bytes & 3) == 0 && k0 + 8 <= ((p.k + 1) & ~1)) {
      word = *reinterpret_cast<const uint32_t*>(src);
    } else {
      word = 0;
      for (int b = 0; b < 4; ++b)
        if ((k0 >> 1) + b < p.row_bytes) word |= static_cast<uint32_t>(src[b]) << (8 * b);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t q = (word >> (4 * i)) & 15u;
      c[i] = WD == WOQ_B200_DTYPE_NF4 ? kNf4[q] : static_cast<float>(q);
    }
  } else {
    const uint8_t* src = p.w + static_cast<size_t>(row) * p.row_bytes + k0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t b = k0 + i < p.k ? src[i] : 0u;
      c[i] = WD == WOQ_B200_DTYPE_FP8 ? fp8_e4m3_to_f32(b) : static_cast<float>(static_cast<int8_t>(b));
    }
  }
}

template <int WD, int C>
__global__ void __launch_bounds__(kWarps * 32) woq_generic_kernel(const GenericParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * kWarps + warp) * kRows;
  const int tok0 = blockIdx.y * kTok;
  if (row0 >= p.n) return;
  float acc[kRows][kTok];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < kTok; ++t) acc[r][t] = 0.f;
  const int ntok = min(kTok, p.m - tok0);

  for (int k0 = lane * 8; k0 < p.k; k0 += 32 * 8) {
    // activations of this chunk, rounded to the compute dtype
    float xv[kTok][8];
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = 0.f;
        if (t < ntok && k0 + i < p.k) v = load_io(p.x, static_cast<size_t>(tok0 + t) * p.ldx + k0 + i, p.io_dtype);
        xv[t][i] = round_c<C>(v);
      }
    }
    const int g = p.group >= p.k ? 0 : k0 / p.group;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int row = row0 + r;
      if (row >= p.n) break;
      float c[8];
      load_codes<WD>(p, row, k0, c);
      const float s = round_c<C>(p.scales[static_cast<size_t>(row) * p.groups + g]);
      const float z = p.zps ? p.zps[static_cast<size_t>(row) * p.groups + g] : p.default_zp;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float w = round_c<C>((c[i] - z) * s);
#pragma unroll
        for (int t = 0; t < kTok; ++t) acc[r][t] = fmaf(xv[t][i], w, acc[r][t]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      float v = acc[r][t];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
      acc[r][t] = v;
    }
  // lane (r, t) of the first 32 results writes one of them
  const int r = lane / kTok, t = lane % kTok;
  float v = 0.f;
#pragma unroll
  for (int rr = 0; rr < kRows; ++rr)
#pragma unroll
    for (int tt = 0; tt < kTok; ++tt)
      if (rr == r && tt == t) v = acc[rr][tt];
  const int row = row0 + r;
  if (row < p.n && t < ntok) {
    if (p.bias) v += p.bias[row];
    const size_t o = static_cast<size_t>(tok0 + t) * p.ldy + row;
    v = round_io(v, p.io_dtype);
    v = post_op_io(v, p, o);
    store_io(p.y, o, v, p.io_dtype);
  }
}

template <int WD>
cudaError_t launch_wd(const GenericParams& p, dim3 grid, cudaStream_t stream) {
  switch (p.compute_dtype) {
    case WOQ_B200_T_BF16: woq_generic_kernel<WD, WOQ_B200_T_BF16><<<grid, kWarps * 32, 0, stream>>>(p); break;
    case WOQ_B200_T_F16: woq_generic_kernel<WD, WOQ_B200_T_F16><<<grid, kWarps * 32, 0, stream>>>(p); break;
    case WOQ_B200_T_F32: woq_generic_kernel<WD, WOQ_B200_T_F32><<<grid, kWarps * 32, 0, stream>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// dequantised weight [n][k] in the compute dtype's values, stored as fp32 (parity hook)
template <int WD>
__global__ void dump_generic_kernel(const GenericParams p, float* out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t chunks = (p.k + 7) / 8;
  if (i >= static_cast<int64_t>(p.n) * chunks) return;
  const int row = static_cast<int>(i / chunks), k0 = static_cast<int>(i % chunks) * 8;
  float c[8];
  load_codes<WD>(p, row, k0, c);
  const int g = p.group >= p.k ? 0 : k0 / p.group;
  float s = p.scales[static_cast<size_t>(row) * p.groups + g];
  const float z = p.zps ? p.zps[static_cast<size_t>(row) * p.groups + g] : p.default_zp;
  for (int j = 0; j < 8 && k0 + j < p.k; ++j) {
    float w;
    if (p.compute_dtype == WOQ_B200_T_BF16)
      w = round_c<WOQ_B200_T_BF16>((c[j] - z) * round_c<WOQ_B200_T_BF16>(s));
    else if (p.compute_dtype == WOQ_B200_T_F16)
      w = round_c<WOQ_B200_T_F16>((c[j] - z) * round_c<WOQ_B200_T_F16>(s));
    else
      w = (c[j] - z) * s;
    out[static_cast<size_t>(row) * p.k + k0 + j] = w;
  }
}

}  // namespace

cudaError_t launch_generic(const GenericParams& p, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>(ceil_div(p.n, kWarps * kRows)), static_cast<unsigned>(ceil_div(p.m, kTok)));
  switch (p.weight_dtype) {
    case WOQ_B200_DTYPE_INT4: return launch_wd<WOQ_B200_DTYPE_INT4>(p, grid, stream);
    case WOQ_B200_DTYPE_NF4: return launch_wd<WOQ_B200_DTYPE_NF4>(p, grid, stream);
    case WOQ_B200_DTYPE_INT8: return launch_wd<WOQ_B200_DTYPE_INT8>(p, grid, stream);
    case WOQ_B200_DTYPE_FP8: return launch_wd<WOQ_B200_DTYPE_FP8>(p, grid, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_dump_generic(const GenericParams& p, float* out, cudaStream_t stream) {
  const int64_t items = static_cast<int64_t>(p.n) * ((p.k + 7) / 8);
  const unsigned blocks = static_cast<unsigned>(ceil_div(items, 256));
  switch (p.weight_dtype) {
    case WOQ_B200_DTYPE_INT4: dump_generic_kernel<WOQ_B200_DTYPE_INT4><<<blocks, 256, 0, stream>>>(p, out); break;
    case WOQ_B200_DTYPE_NF4: dump_generic_kernel<WOQ_B200_DTYPE_NF4><<<blocks, 256, 0, stream>>>(p, out); break;
    case WOQ_B200_DTYPE_INT8: dump_generic_kernel<WOQ_B200_DTYPE_INT8><<<blocks, 256, 0, stream>>>(p, out); break;
    case WOQ_B200_DTYPE_FP8: dump_generic_kernel<WOQ_B200_DTYPE_FP8><<<blocks, 256, 0, stream>>>(p, out); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace woq
