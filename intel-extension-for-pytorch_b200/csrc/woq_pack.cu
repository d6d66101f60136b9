// Prepack (plain -> tiled), its bit-exact inverse, scale / zero-point re-layout, the exact
// bf16 dequantised-weight dump, and AWQ / GPTQ int32 checkpoint unpacking.  One-off work at
// model load: simple one-thread-per-word kernels.
#include <cuda_fp16.h>

#include "woq_kernels.h"

namespace woq {

namespace {

__device__ __forceinline__ uint32_t plain_nibble(const uint8_t* plain, int n_rows, int k_cols,
                                                 int64_t row_bytes, int n, int k) {
  if (n >= n_rows || k >= k_cols) return 0u;
  const uint8_t b = plain[static_cast<int64_t>(n) * row_bytes + (k >> 1)];
  return (k & 1) ? (b >> 4) : (b & 0xF);
}

__global__ void pack_int4_kernel(PackInt4Args a) {
  const int64_t total_words = static_cast<int64_t>(a.tiles) * a.kb_per_tile * 512;
  const int64_t wi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (wi >= total_words) return;
  const int rt = wi & 3, lane = (wi >> 2) & 31, j = (wi >> 7) & 3;
  const int64_t blk = wi >> 9;
  const int kb = static_cast<int>(blk % a.kb_per_tile), tile = static_cast<int>(blk / a.kb_per_tile);
  const int g = lane >> 2, t = lane & 3;
  const int r0 = rt * 16 + g, r1 = r0 + 8;
  const int n0 = tile_row_to_n(a.n, a.gate_up, tile, r0), n1 = tile_row_to_n(a.n, a.gate_up, tile, r1);
  const int k0 = kb * kBlockK + 16 * t + 4 * j;
  const int64_t row_bytes = (a.k + 1) / 2;
  uint32_t w = 0;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n0, k0 + 0) << 0;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n1, k0 + 0) << 4;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n0, k0 + 2) << 8;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n1, k0 + 2) << 12;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n0, k0 + 1) << 16;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n1, k0 + 1) << 20;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n0, k0 + 3) << 24;
  w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n1, k0 + 3) << 28;
  reinterpret_cast<uint32_t*>(a.tiled)[wi] = w;
}

// 128-row layout: word index inside a 4096-byte block and the nibble's bit position
__host__ __device__ inline void tc_slot(int row, int k, int& word, int& shift) {
  const int jp = k >> 3, kk = k & 7, s = kk >> 1, odd = kk & 1;
  const int half = jp >> 2, j = jp & 3;
  word = (half * kTcTileN + row) * 4 + j;
  shift = 4 * s + 16 * odd;
}

__global__ void pack_int4_tc_kernel(PackInt4Args a) {
  const int64_t total_words = static_cast<int64_t>(a.tiles) * a.kb_per_tile * 1024;
  const int64_t wi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (wi >= total_words) return;
  const int j = wi & 3, row = (wi >> 2) & 127, half = (wi >> 9) & 1;
  const int64_t blk = wi >> 10;
  const int kb = static_cast<int>(blk % a.kb_per_tile), tile = static_cast<int>(blk / a.kb_per_tile);
  const int n = tc_tile_row_to_n(a.n, a.gate_up, tile, row);
  const int k0 = kb * kBlockK + 8 * (4 * half + j);
  const int64_t row_bytes = (a.k + 1) / 2;
  uint32_t w = 0;
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n, k0 + 2 * s) << (4 * s);
    w |= plain_nibble(a.plain, a.n, a.k, row_bytes, n, k0 + 2 * s + 1) << (4 * s + 16);
  }
  reinterpret_cast<uint32_t*>(a.tiled)[wi] = w;
}

__global__ void dump_dequant_int4_tc_kernel(const uint32_t* tiled, const uint32_t* sz,
                                            __nv_bfloat16* w, int n, int k, int tiles,
                                            int kb_per_tile, int kbpg_shift, int groups, int gate_up) {
  const int64_t total_words = static_cast<int64_t>(tiles) * kb_per_tile * 1024;
  const int64_t wi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (wi >= total_words) return;
  const int j = wi & 3, row = (wi >> 2) & 127, half = (wi >> 9) & 1;
  const int64_t blk = wi >> 10;
  const int kb = static_cast<int>(blk % kb_per_tile), tile = static_cast<int>(blk / kb_per_tile);
  const int nn = tc_tile_row_to_n(n, gate_up, tile, row);
  if (nn >= n) return;
  const uint32_t szw = sz[(static_cast<int64_t>(tile) * groups + (kb >> kbpg_shift)) * kTcTileN + row];
  const uint32_t z2 = __byte_perm(szw, 0, 0x1010), s2 = __byte_perm(szw, 0, 0x3232);
  const uint32_t word = tiled[wi];
  const int k0 = kb * kBlockK + 8 * (4 * half + j);
  uint32_t* w32 = reinterpret_cast<uint32_t*>(w);
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const uint32_t v =
        bf16x2_mul(bf16x2_sub(lop3_and_or(word >> (4 * s), 0x000f000fu, kBf16Magic), z2), s2);
    if (k0 + 2 * s + 1 < k) w32[(static_cast<int64_t>(nn) * k + k0 + 2 * s) >> 1] = v;
  }
}

__device__ __forceinline__ uint32_t tiled_nibble(const uint32_t* tiled, int n_total, int gate_up,
                                                 int kb_per_tile, int n, int k) {
  int tile, row;
  if (gate_up) {
    const int half = n_total / 2;
    const int nn = n < half ? n : n - half;
    tile = nn / 32;
    row = (nn % 32) + (n < half ? 0 : 32);
  } else {
    tile = n / kTileN;
    row = n % kTileN;
  }
  int word, shift;
  int4_slot(row, k % kBlockK, word, shift);
  const int64_t blk = static_cast<int64_t>(tile) * kb_per_tile + k / kBlockK;
  return (tiled[blk * 512 + word] >> shift) & 0xF;
}

__global__ void unpack_int4_kernel(const uint32_t* tiled, uint8_t* plain, int n, int k, int tiles,
                                   int kb_per_tile, int gate_up) {
  const int64_t row_bytes = (k + 1) / 2;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(n) * row_bytes) return;
  const int row = static_cast<int>(i / row_bytes), kk = static_cast<int>(i % row_bytes) * 2;
  uint32_t lo = tiled_nibble(tiled, n, gate_up, kb_per_tile, row, kk);
  uint32_t hi = (kk + 1 < k) ? tiled_nibble(tiled, n, gate_up, kb_per_tile, row, kk + 1) : 0u;
  plain[i] = static_cast<uint8_t>(lo | (hi << 4));
}

__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dtype) {
  switch (dtype) {
    case 1: return reinterpret_cast<const float*>(p)[i];
    case 2: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case 3: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case 4: return static_cast<float>(reinterpret_cast<const uint8_t*>(p)[i]);
    case 5: return static_cast<float>(reinterpret_cast<const int8_t*>(p)[i]);
    default: return 0.f;
  }
}

__global__ void pack_scales_kernel(PackScaleArgs a) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(a.tiles) * a.groups * (a.tc ? kTcTileN : kTileN);
  if (i >= total) return;
  const int tn = a.tc ? kTcTileN : kTileN;
  const int row = static_cast<int>(i % tn);
  const int grp = static_cast<int>((i / tn) % a.groups);
  const int tile = static_cast<int>(i / (static_cast<int64_t>(tn) * a.groups));
  const int n = a.tc ? tc_tile_row_to_n(a.n, a.gate_up, tile, row)
                     : tile_row_to_n(a.n, a.gate_up, tile, row);
  float s = 0.f, z = static_cast<float>(a.default_zp);
  if (n < a.n) {
    const int64_t src = a.transposed ? static_cast<int64_t>(grp) * a.n + n
                                     : static_cast<int64_t>(n) * a.groups + grp;
    s = load_as_float(a.scales, src, a.scale_dtype);
    if (a.zps) {
      const int64_t zsrc = a.zp_transposed ? static_cast<int64_t>(grp) * a.n + n
                                           : static_cast<int64_t>(n) * a.groups + grp;
      z = load_as_float(a.zps, zsrc, a.zp_dtype);
      if (!(z >= 0.f && z <= 127.f && z == rintf(z))) {
        atomicOr(a.bad_zp, 1);
        z = 0.f;
      }
    }
  }
  // The bf16 compute path multiplies by the bf16-rounded scale (round to nearest even of the
  // fp32 value); 128 + zp is exact in bf16.
  const uint32_t sb = __bfloat16_as_ushort(__float2bfloat16_rn(s));
  const uint32_t zb = __bfloat16_as_ushort(__float2bfloat16_rn(128.f + z));
  // The decode kernel's shift-free dequantiser multiplies by scale * 2^129 and keeps 16 * zp in
  // eight bits: it needs a normal scale below 0.5 and a zero point below 16.
  const uint32_t sexp = (sb >> 7) & 0xffu;
  if (n < a.n && (sexp < 1u || sexp > 125u || z > 15.f)) atomicOr(a.bad_zp, 2);
  a.sz[(static_cast<int64_t>(tile) * a.groups + grp) * tn + (a.tc ? row : scale_slot(row))] =
      (sb << 16) | zb;
}

__global__ void dump_dequant_int4_kernel(const uint32_t* tiled, const uint32_t* sz,
                                         __nv_bfloat16* w, int n, int k, int tiles, int kb_per_tile,
                                         int kb_per_group, int groups, int gate_up) {
  const int64_t total_words = static_cast<int64_t>(tiles) * kb_per_tile * 512;
  const int64_t wi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (wi >= total_words) return;
  const int rt = wi & 3, lane = (wi >> 2) & 31, j = (wi >> 7) & 3;
  const int64_t blk = wi >> 9;
  const int kb = static_cast<int>(blk % kb_per_tile), tile = static_cast<int>(blk / kb_per_tile);
  const int g = lane >> 2, t = lane & 3;
  const int r0 = rt * 16 + g, r1 = r0 + 8;
  const int grp = kb / kb_per_group;
  const uint32_t* szt = sz + (static_cast<int64_t>(tile) * groups + grp) * kTileN;
  uint32_t out[4];
  dequant_word_exact(tiled[wi], szt[scale_slot(r0)], szt[scale_slot(r1)], out);
  const int n0 = tile_row_to_n(n, gate_up, tile, r0), n1 = tile_row_to_n(n, gate_up, tile, r1);
  const int k0 = kb * kBlockK + 16 * t + 4 * j;
  uint32_t* w32 = reinterpret_cast<uint32_t*>(w);
  if (k0 + 3 < k || k0 + 1 < k) {
    if (n0 < n) {
      if (k0 + 1 < k) w32[(static_cast<int64_t>(n0) * k + k0) >> 1] = out[0];
      if (k0 + 3 < k) w32[(static_cast<int64_t>(n0) * k + k0 + 2) >> 1] = out[2];
    }
    if (n1 < n) {
      if (k0 + 1 < k) w32[(static_cast<int64_t>(n1) * k + k0) >> 1] = out[1];
      if (k0 + 3 < k) w32[(static_cast<int64_t>(n1) * k + k0 + 2) >> 1] = out[3];
    }
  }
}

// AWQ: qweight [K][N/8] int32, nibble j of a word is column 8*c + order[j]
__global__ void awq_to_plain_kernel(const int32_t* q, uint8_t* plain, int n, int k) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row_bytes = k / 2;
  if (i >= static_cast<int64_t>(n) * row_bytes) return;
  const int row = static_cast<int>(i / row_bytes), kk = static_cast<int>(i % row_bytes) * 2;
  // inverse of order {0,2,4,6,1,3,5,7}: column c (0..7) sits in nibble inv[c]
  const int inv[8] = {0, 4, 1, 5, 2, 6, 3, 7};
  const int word = row >> 3, sh = 4 * inv[row & 7];
  const uint32_t lo = (static_cast<uint32_t>(q[static_cast<int64_t>(kk) * (n / 8) + word]) >> sh) & 0xF;
  const uint32_t hi =
      (static_cast<uint32_t>(q[static_cast<int64_t>(kk + 1) * (n / 8) + word]) >> sh) & 0xF;
  plain[i] = static_cast<uint8_t>(lo | (hi << 4));
}

// GPTQ: qweight [K/8][N] int32, nibble j of word r is k = 8*r + j
__global__ void gptq_to_plain_kernel(const int32_t* q, uint8_t* plain, int n, int k) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row_bytes = k / 2;
  if (i >= static_cast<int64_t>(n) * row_bytes) return;
  const int row = static_cast<int>(i / row_bytes), kk = static_cast<int>(i % row_bytes) * 2;
  const uint32_t wv = static_cast<uint32_t>(q[static_cast<int64_t>(kk >> 3) * n + row]);
  plain[i] = static_cast<uint8_t>((wv >> (4 * (kk & 7))) & 0xFF);
}

__global__ void unpack_qzeros_kernel(const int32_t* qz, uint8_t* zps, int n, int groups, int awq,
                                     int plus_one) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(n) * groups) return;
  const int row = static_cast<int>(i / groups), grp = static_cast<int>(i % groups);
  const int inv[8] = {0, 4, 1, 5, 2, 6, 3, 7};
  const int sh = 4 * (awq ? inv[row & 7] : (row & 7));
  const uint32_t v = (static_cast<uint32_t>(qz[static_cast<int64_t>(grp) * (n / 8) + (row >> 3)]) >> sh) & 0xF;
  zps[i] = static_cast<uint8_t>((v + (plus_one ? 1u : 0u)) & 0xF);
}

// out[i, :] = x[idx[i], :] for bf16 rows of k elements (k % 8 == 0): the token gather of an
// expert (reference: fuse_index_unsqueeze, csrc/cpu/aten/kernels/MoEKrnl.cpp:123-160)
__global__ void gather_rows_kernel(const __nv_bfloat16* x, int64_t ldx, const int32_t* idx,
                                   __nv_bfloat16* out, int64_t rows, int k) {
  const int chunks = k / 8;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * chunks) return;
  const int64_t r = i / chunks;
  const int c = static_cast<int>(i % chunks);
  reinterpret_cast<uint4*>(out + r * k)[c] =
      reinterpret_cast<const uint4*>(x + static_cast<int64_t>(idx[r]) * ldx)[c];
}

inline unsigned blocks_for(int64_t n, int threads) {
  return static_cast<unsigned>((n + threads - 1) / threads);
}

}  // namespace

cudaError_t launch_pack_int4(const PackInt4Args& a, cudaStream_t stream) {
  const int64_t words = static_cast<int64_t>(a.tiles) * a.kb_per_tile * (a.tc ? 1024 : 512);
  if (a.tc)
    pack_int4_tc_kernel<<<blocks_for(words, 256), 256, 0, stream>>>(a);
  else
    pack_int4_kernel<<<blocks_for(words, 256), 256, 0, stream>>>(a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_unpack_int4(const uint8_t* tiled, uint8_t* plain, int n, int k, int tiles,
                               int kb_per_tile, int gate_up, cudaStream_t stream) {
  const int64_t bytes = static_cast<int64_t>(n) * ((k + 1) / 2);
  unpack_int4_kernel<<<blocks_for(bytes, 256), 256, 0, stream>>>(
      reinterpret_cast<const uint32_t*>(tiled), plain, n, k, tiles, kb_per_tile, gate_up);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_pack_scales(const PackScaleArgs& a, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(a.tiles) * a.groups * (a.tc ? kTcTileN : kTileN);
  pack_scales_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_dump_dequant_int4(const uint8_t* tiled, const uint32_t* sz, __nv_bfloat16* w,
                                     int n, int k, int tiles, int kb_per_tile, int kb_per_group,
                                     int groups, int gate_up, cudaStream_t stream) {
  const int64_t words = static_cast<int64_t>(tiles) * kb_per_tile * 512;
  dump_dequant_int4_kernel<<<blocks_for(words, 256), 256, 0, stream>>>(
      reinterpret_cast<const uint32_t*>(tiled), sz, w, n, k, tiles, kb_per_tile, kb_per_group,
      groups, gate_up);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_dump_dequant_int4_tc(const uint8_t* tiled, const uint32_t* sz, __nv_bfloat16* w,
                                        int n, int k, int tiles, int kb_per_tile, int kbpg_shift,
                                        int groups, int gate_up, cudaStream_t stream) {
  const int64_t words = static_cast<int64_t>(tiles) * kb_per_tile * 1024;
  dump_dequant_int4_tc_kernel<<<blocks_for(words, 256), 256, 0, stream>>>(
      reinterpret_cast<const uint32_t*>(tiled), sz, w, n, k, tiles, kb_per_tile, kbpg_shift, groups,
      gate_up);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const __nv_bfloat16* x, int64_t ldx, const int32_t* idx,
                               __nv_bfloat16* out, int64_t rows, int k, cudaStream_t stream) {
  gather_rows_kernel<<<blocks_for(rows * (k / 8), 256), 256, 0, stream>>>(x, ldx, idx, out, rows, k);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_awq_to_plain(const int32_t* q, uint8_t* plain, int n, int k,
                                cudaStream_t stream) {
  const int64_t bytes = static_cast<int64_t>(n) * (k / 2);
  awq_to_plain_kernel<<<blocks_for(bytes, 256), 256, 0, stream>>>(q, plain, n, k);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_gptq_to_plain(const int32_t* q, uint8_t* plain, int n, int k,
                                 cudaStream_t stream) {
  const int64_t bytes = static_cast<int64_t>(n) * (k / 2);
  gptq_to_plain_kernel<<<blocks_for(bytes, 256), 256, 0, stream>>>(q, plain, n, k);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_unpack_qzeros(const int32_t* qzeros, uint8_t* zps, int n, int groups, int awq,
                                 int plus_one, cudaStream_t stream) {
  unpack_qzeros_kernel<<<blocks_for(static_cast<int64_t>(n) * groups, 256), 256, 0, stream>>>(
      qzeros, zps, n, groups, awq, plus_one);
  count_launch();
  return cudaGetLastError();
}

}  // namespace woq
