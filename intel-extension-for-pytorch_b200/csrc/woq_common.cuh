// Shared device helpers for the WOQ kernels: tiled weight layout, bf16 nibble dequantisation,
// mbarrier / bulk-copy / mma PTX wrappers with bounded waits.  sm_100a only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace woq {

// ---------------------------------------------------------------------------------------
// INT4 tiled layout.
//
// The weight [N, K] is cut into tiles of 64 output rows x 64 k ("k-block").  A k-block of a
// tile is 2048 bytes: 4 k-steps j, each 32 lanes x 16 bytes, so that lane l of a warp fetches
// what it needs for one m16n8k16 step of all four 16-row row-tiles with a single 128-bit
// shared-memory load.  With g = l / 4 and t = l % 4, word rt (0..3) of lane l in k-step j
// holds, for rows r0 = 16*rt + g and r1 = r0 + 8 and k0 = 64*kb + 16*t + 4*j:
//   bits  3: 0  q[r0][k0+0]     bits 19:16  q[r0][k0+1]
//   bits  7: 4  q[r1][k0+0]     bits 23:20  q[r1][k0+1]
//   bits 11: 8  q[r0][k0+2]     bits 27:24  q[r0][k0+3]
//   bits 15:12  q[r1][k0+2]     bits 31:28  q[r1][k0+3]
// (w >> 4i) & 0x000f000f | 0x43004300 is then a bf16x2 register holding 128 + q for one
// A-fragment register of mma.m16n8k16 (k order inside a k-block is permuted consistently
// for A and B).  Tiles are stored [tile][k-block], so any run of k-blocks of one tile is
// one contiguous range for a bulk copy.
//
// Scales: [tile][group][64] 32-bit words; slot p = 8*g + 2*rt + h holds row 16*rt + 8*h + g:
// high half = bf16(scale), low half = bf16(128 + zero_point) (exact: zero points are
// integers in 0..127).  A lane reads its 8 rows with two 128-bit loads.
// ---------------------------------------------------------------------------------------
constexpr int kTileN = 64;
constexpr int kBlockK = 64;
constexpr int kBlockBytes = kTileN * kBlockK / 2;  // 2048
constexpr uint32_t kBf16Magic = 0x43004300u;       // two bf16 128.0

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Position of nibble (row r in tile, k in k-block) inside the 2048-byte block:
// returns word index (0..511) and bit shift.
__host__ __device__ inline void int4_slot(int r, int k, int& word, int& shift) {
  const int rt = r >> 4, rr = r & 15, g = rr & 7, h = rr >> 3;
  const int t = k >> 4, kk = k & 15, j = kk >> 2, c = kk & 3;
  word = ((j * 32) + (g * 4 + t)) * 4 + rt;
  // c: 0 -> bits 3:0 (+4 if h), 1 -> bits 19:16, 2 -> bits 11:8, 3 -> bits 27:24
  shift = ((c & 1) ? 16 : 0) + ((c & 2) ? 8 : 0) + (h ? 4 : 0);
}

__host__ __device__ inline int scale_slot(int r) {
  const int rt = r >> 4, rr = r & 15, g = rr & 7, h = rr >> 3;
  return 8 * g + 2 * rt + h;
}

// ---------------------------------------------------------------------------------------
// bf16x2 arithmetic used by the exact tile dequantiser
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a&b)|c
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Exact dequantisation of one packed word: out[i] (i = 0..3) is a bf16x2 register with
// bf16((q - zp) * s) for the two nibbles selected by shift 4*i.  `sz_r0` / `sz_r1` are the
// scale words of rows r0 / r1.  (q - zp) is exact in bf16; the product of two bf16 numbers
// is exact in fp32, so one mul.rn.bf16x2 equals "multiply in fp32, round to nearest even".
__device__ __forceinline__ void dequant_word_exact(uint32_t w, uint32_t sz_r0, uint32_t sz_r1,
                                                   uint32_t out[4]) {
  const uint32_t z0 = __byte_perm(sz_r0, 0, 0x1010), s0 = __byte_perm(sz_r0, 0, 0x3232);
  const uint32_t z1 = __byte_perm(sz_r1, 0, 0x1010), s1 = __byte_perm(sz_r1, 0, 0x3232);
  out[0] = bf16x2_mul(bf16x2_sub(lop3_and_or(w, 0x000f000fu, kBf16Magic), z0), s0);
  out[1] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 4, 0x000f000fu, kBf16Magic), z1), s1);
  out[2] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 8, 0x000f000fu, kBf16Magic), z0), s0);
  out[3] = bf16x2_mul(bf16x2_sub(lop3_and_or(w >> 12, 0x000f000fu, kBf16Magic), z1), s1);
}

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
#ifdef WOQ_USE_TEST_WAIT
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#else
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#endif
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Upper bound for any in-kernel wait.  A wait that runs out records `code` in *status,
// raises the block-wide abort flag, and returns false; from then on every wait in the
// block returns immediately so that all threads still reach the end of the kernel.
// Time is taken from the SM cycle counter and only looked at every 1024 polls: the common
// case (the barrier flips within a few polls) costs nothing beyond the polls themselves.
constexpr long long kWaitLimitCycles = 4000000000ll;  // about 2 s

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
  if (mbar_test(bar, parity)) return true;
  uint32_t spins = 0;
  long long t0 = 0;
  while (!mbar_test(bar, parity)) {
    if ((++spins & 1023u) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// Bulk asynchronous copy global -> this CTA's shared memory, completion on an mbarrier.
// Addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// system-scope flag traffic between GPUs
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Programmatic dependent launch (no-ops for a grid launched without the attribute)
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void named_bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// D += A(16x16, row) * B(16x8, col), bf16 inputs, fp32 accumulate
__device__ __forceinline__ void mma_bf16_16816(float d[4], const uint32_t a[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D += A(16x32, row) * B(32x8, col), s8 inputs, s32 accumulate
__device__ __forceinline__ void mma_s8_16832(int d[4], const uint32_t a[4], uint32_t b0,
                                             uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Post-ops on the bf16-rounded result, mirroring the reference's epilogue on bf16 data:
// fp32 arithmetic inside, one rounding to bf16 per op (silu rounds sigmoid as well).
__device__ __forceinline__ float silu_bf16(float y) {
  const float sig = bf16_round(1.0f / (1.0f + expf(-y)));
  return bf16_round(y * sig);
}

constexpr int FUSE_NONE = 0x0, FUSE_GELU_ERF = 0x1, FUSE_GELU_TANH = 0x2, FUSE_RELU = 0x3,
              FUSE_SILU = 0x4, FUSE_ADD = 0x10, FUSE_ADD_ADD = 0x20, FUSE_MUL = 0x30,
              FUSE_SILU_MUL = 0x100, FUSE_SCALED_SCATTER_ADD = 0x200;

__device__ __forceinline__ float unary_post_op(float y, int fusion) {
  switch (fusion) {
    case FUSE_GELU_ERF:
      return bf16_round(0.5f * y * (1.0f + erff(y * 0.70710678118654752f)));
    case FUSE_GELU_TANH: {
      const float inner = 0.7978845608028654f * (y + 0.044715f * y * y * y);
      return bf16_round(0.5f * y * (1.0f + tanhf(inner)));
    }
    case FUSE_RELU:
      return fmaxf(y, 0.0f);
    case FUSE_SILU:
      return silu_bf16(y);
    default:
      return y;
  }
}

}  // namespace woq
