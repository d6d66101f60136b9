/*
 * woq_oracle_c.c -- C restatement of the reference's CPU WOQ linear kernels.
 *
 * TEST INFRASTRUCTURE ONLY: this is the CPU checker and the timed CPU baseline.  The shipped
 * CUDA path never links or calls it.
 *
 * What it follows (paths inside intel/intel-extension-for-pytorch):
 *   - blocked weight layout, block_n = 32, block_k = 64 (128 for int8 compute): INT4 byte
 *     [kb][i] = q[n0+i][k] | q[n0+i+16][k] << 4          csrc/cpu/aten/kernels/WoqUtilKrnl.cpp:32-249
 *     (block_k rule: csrc/cpu/aten/Linear.cpp:362-376)
 *   - scales / zero points re-laid out per 32-column block with bf16 copies made by rounding
 *     the fp32 values                                   csrc/cpu/jit/cpu/kernels/ContextLinearWoq.h:60-128
 *   - bf16 tile dequantisation w = bf16((q - zp) * scale_bf16) followed by a bf16 x bf16 ->
 *     fp32 block GEMM accumulated over all k blocks, bias preloaded in fp32, fp32 -> bf16 at
 *     the end, post-op on the bf16 data                  csrc/cpu/aten/utils/woq.h:1223-1325,
 *                                                        1501-1581, 1801-1964, 2924-2945, 3285-3462
 *   - OpenMP over (n block, m block)                     csrc/cpu/aten/utils/woq.h:3267-3275
 *   - per-token symmetric int8 activation quantisation   csrc/cpu/aten/utils/woq_dynamic_quant.h:1526-1750
 *   - int8 x int8 -> int32 per 128-k block, C += float(acc) * scale_a * scale_w
 *                                                        csrc/cpu/aten/utils/woq.h:2231-2354
 *   - small-M (M < 5) fp16 microkernel: per 32-column block and 64-k block
 *     acc[m][n] = sum_k x_fp16[m][k] * (LUT[q[k][n]] - zp[n]) with fp16 fused multiply-adds,
 *     then C[m][n] += scale_fp16[n] * acc[m][n]; fp16 bias preloaded, fp16 -> bf16 at the end
 *                                                        csrc/cpu/aten/utils/woq.h:784-951,1862-1920
 *     (what qlinear_woq_affine runs for lowp BF16 and M < 5, kernels/WoqLinearKrnl.cpp:75-106)
 * The reference reaches its block GEMMs through libxsmm (BRGEMM), which is not part of the
 * reference tree; here they are plain loops the compiler vectorises (AVX-512 / AVX2 clones
 * picked at run time).  The small-M microkernel is written with AVX512-FP16 intrinsics like
 * the reference's own (csrc/cpu/tpp/woq/vec.h) and is only offered where the CPU has them.  Parity of this file is pinned by tests that compare it with the
 * numpy oracle (oracle/woq_oracle.py), which in turn is pinned by the golden fixtures.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__x86_64__) && defined(__GNUC__)
#include <immintrin.h>
#define WOQ_HAVE_FP16_KERNEL 1
#endif

#define NB 32 /* WOQ_N_BLOCK_SIZE, csrc/cpu/aten/utils/woq_defines.h:46 */

#if defined(__x86_64__) && defined(__GNUC__) && !defined(WOQ_ORACLE_NO_CLONES)
#define HOT __attribute__((target_clones("avx512f", "avx2", "default")))
#else
#define HOT
#endif

#define EXPORT __attribute__((visibility("default")))

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16_rne(f)); }

enum { FUSE_NONE = 0, FUSE_GELU_ERF = 1, FUSE_GELU_TANH = 2, FUSE_RELU = 3, FUSE_SILU = 4,
       FUSE_ADD = 0x10, FUSE_ADD_ADD = 0x20, FUSE_MUL = 0x30, FUSE_SILU_MUL = 0x100 };

typedef struct {
  int n, k, npad, nc, kc, kb, group, ngroups, is_int8;
  uint8_t* packed;   /* INT4: [nc][kc][kb][16]; INT8: [nc][kc][kb][32] */
  float* scale;      /* [nc][ngroups][32]: bf16-rounded for INT4, fp32 for int8 compute */
  float* scale32;    /* [nc][ngroups][32]: the fp32 scales as given (the fp16 kernel rounds them to fp16) */
  float* zp;         /* [nc][ngroups][32] */
  float* bias;       /* [npad] or NULL */
} woq_layer;

static int pick_block_k(int k, int group, int base) {
  /* get_block_k: min(group, base), halved until it divides K */
  int kb = (group > 0 && group < base) ? group : base;
  while (k % kb) kb /= 2;
  return kb;
}

EXPORT void woq_oracle_layer_free(woq_layer* L) {
  if (!L) return;
  free(L->packed); free(L->scale); free(L->scale32); free(L->zp); free(L->bias); free(L);
}

/* scales: [n][ngroups] fp32 (already widened from fp16 if the checkpoint had fp16);
 * zps: [n][ngroups] fp32 or NULL (symmetric storage: 8 for INT4, 0 for INT8). */
EXPORT woq_layer* woq_oracle_layer_create(const uint8_t* qweight, int n, int k, int is_int8,
                                          const float* scales, const float* zps,
                                          const float* bias, int group, int int8_compute) {
  woq_layer* L = (woq_layer*)calloc(1, sizeof(woq_layer));
  L->n = n; L->k = k; L->is_int8 = is_int8;
  L->group = group > 0 ? group : k;
  L->ngroups = (k + L->group - 1) / L->group;
  L->npad = (n + NB - 1) / NB * NB;
  L->nc = L->npad / NB;
  L->kb = pick_block_k(k, group, int8_compute ? 128 : 64);
  L->kc = k / L->kb;
  const size_t per_block = (size_t)L->kb * (is_int8 ? NB : NB / 2);
  L->packed = (uint8_t*)calloc((size_t)L->nc * L->kc, per_block);
  L->scale = (float*)calloc((size_t)L->nc * L->ngroups * NB, sizeof(float));
  L->zp = (float*)calloc((size_t)L->nc * L->ngroups * NB, sizeof(float));
  L->scale32 = (float*)calloc((size_t)L->nc * L->ngroups * NB, sizeof(float));
  const int row_bytes = is_int8 ? k : (k + 1) / 2;
  for (int nc = 0; nc < L->nc; ++nc) {
    for (int kc = 0; kc < L->kc; ++kc) {
      uint8_t* dst = L->packed + ((size_t)nc * L->kc + kc) * per_block;
      for (int kk = 0; kk < L->kb; ++kk) {
        const int kidx = kc * L->kb + kk;
        if (is_int8) {
          for (int i = 0; i < NB; ++i) {
            const int row = nc * NB + i;
            dst[kk * NB + i] = row < n ? qweight[(size_t)row * row_bytes + kidx] : 0;
          }
        } else {
          for (int i = 0; i < NB / 2; ++i) {
            const int r0 = nc * NB + i, r1 = r0 + NB / 2;
            uint8_t lo = 0, hi = 0;
            if (r0 < n) { uint8_t b = qweight[(size_t)r0 * row_bytes + kidx / 2]; lo = (kidx & 1) ? b >> 4 : b & 0xF; }
            if (r1 < n) { uint8_t b = qweight[(size_t)r1 * row_bytes + kidx / 2]; hi = (kidx & 1) ? b >> 4 : b & 0xF; }
            dst[kk * (NB / 2) + i] = (uint8_t)(lo | (hi << 4));
          }
        }
      }
    }
    for (int g = 0; g < L->ngroups; ++g)
      for (int i = 0; i < NB; ++i) {
        const int row = nc * NB + i;
        const size_t o = ((size_t)nc * L->ngroups + g) * NB + i;
        /* padded rows: scale 1, zero point 0 (LinearWoqPacked.cpp:344-361); weights are 0 */
        float s = row < n ? scales[(size_t)row * L->ngroups + g] : 1.0f;
        float z = row < n ? (zps ? zps[(size_t)row * L->ngroups + g] : (is_int8 ? 0.f : 8.f)) : 0.f;
        L->scale[o] = int8_compute ? s : round_bf16(s);
        L->scale32[o] = s;
        L->zp[o] = z;
      }
  }
  if (bias) {
    L->bias = (float*)calloc(L->npad, sizeof(float));
    memcpy(L->bias, bias, (size_t)n * sizeof(float));
  }
  return L;
}

/* Dequantise one [kb][32] tile to bf16 values (held as float). */
HOT static void dequant_tile_int4(const uint8_t* blk, int kb, const float* scale, const float* zp,
                                  float* tile) {
  for (int kk = 0; kk < kb; ++kk) {
    const uint8_t* b = blk + kk * (NB / 2);
    float* t = tile + kk * NB;
    for (int i = 0; i < NB / 2; ++i) {
      const float lo = (float)(b[i] & 0xF), hi = (float)(b[i] >> 4);
      t[i] = (lo - zp[i]) * scale[i];
      t[i + NB / 2] = (hi - zp[i + NB / 2]) * scale[i + NB / 2];
    }
    for (int i = 0; i < NB; ++i) { /* round to nearest even bf16 */
      uint32_t u;
      memcpy(&u, &t[i], 4);
      u += 0x7fffu + ((u >> 16) & 1u);
      u &= 0xffff0000u;
      memcpy(&t[i], &u, 4);
    }
  }
}

HOT static void dequant_tile_int8(const uint8_t* blk, int kb, const float* scale, const float* zp,
                                  float* tile) {
  for (int kk = 0; kk < kb; ++kk) {
    const int8_t* b = (const int8_t*)blk + kk * NB;
    float* t = tile + kk * NB;
    for (int i = 0; i < NB; ++i) {
      t[i] = ((float)b[i] - zp[i]) * scale[i];
      uint32_t u;
      memcpy(&u, &t[i], 4);
      u += 0x7fffu + ((u >> 16) & 1u);
      u &= 0xffff0000u;
      memcpy(&t[i], &u, 4);
    }
  }
}

/* acc[m][32] += x[m][k0 .. k0+kb) * tile[kb][32]; products of bf16 values are exact in fp32 */
HOT static void block_gemm(const float* x, int ldx, int mrows, int kb, const float* tile,
                           float* acc) {
  for (int m = 0; m < mrows; ++m) {
    float a[NB];
    for (int i = 0; i < NB; ++i) a[i] = acc[m * NB + i];
    const float* xr = x + (size_t)m * ldx;
    for (int kk = 0; kk < kb; ++kk) {
      const float xv = xr[kk];
      const float* t = tile + kk * NB;
      for (int i = 0; i < NB; ++i) a[i] += xv * t[i];
    }
    for (int i = 0; i < NB; ++i) acc[m * NB + i] = a[i];
  }
}

static float silu_bf16(float y) {
  const float sig = round_bf16((float)(1.0 / (1.0 + exp(-(double)y))));
  return round_bf16(y * sig);
}

static float post_op(float y, int fusion, float o0, float o1) {
  switch (fusion) {
    case FUSE_GELU_ERF: return round_bf16((float)(0.5 * y * (1.0 + erf((double)y / sqrt(2.0)))));
    case FUSE_GELU_TANH: {
      const double v = y, inner = sqrt(2.0 / M_PI) * (v + 0.044715 * v * v * v);
      return round_bf16((float)(0.5 * v * (1.0 + tanh(inner))));
    }
    case FUSE_RELU: return y > 0.f ? y : 0.f;
    case FUSE_SILU: return silu_bf16(y);
    case FUSE_ADD: return round_bf16(y + o0);
    case FUSE_ADD_ADD: return round_bf16(round_bf16(y + o0) + o1);
    case FUSE_MUL: return round_bf16(y * o0);
    default: return y;
  }
}

#define BLOCK_M 32

/* bf16-compute linear: x [m][k] bf16 bits, y [m][n_out] bf16 bits. */
EXPORT int woq_oracle_linear_bf16(const woq_layer* L, const uint16_t* x, int m, int fusion,
                                  const uint16_t* other0, const uint16_t* other1, uint16_t* y,
                                  int threads) {
  const int k = L->k, n = L->n;
  float* xf = (float*)malloc((size_t)m * k * sizeof(float));
  for (size_t i = 0; i < (size_t)m * k; ++i) xf[i] = bf16_to_f32(x[i]);
  const int mblocks = (m + BLOCK_M - 1) / BLOCK_M;
  const int kb_per_group = L->group / L->kb > 0 ? L->group / L->kb : 1;
  uint16_t* ytmp = NULL;
  if (fusion == FUSE_SILU_MUL) ytmp = (uint16_t*)malloc((size_t)m * n * sizeof(uint16_t));
  uint16_t* yo = ytmp ? ytmp : y;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel
  {
    float* tile = (float*)malloc((size_t)L->kb * NB * sizeof(float));
    float* acc = (float*)malloc((size_t)BLOCK_M * NB * sizeof(float));
#pragma omp for collapse(2) schedule(static)
    for (int nc = 0; nc < L->nc; ++nc) {
      for (int mb = 0; mb < mblocks; ++mb) {
        const int m0 = mb * BLOCK_M, mrows = (m - m0) < BLOCK_M ? (m - m0) : BLOCK_M;
        for (int mm = 0; mm < mrows; ++mm)
          for (int i = 0; i < NB; ++i) acc[mm * NB + i] = L->bias ? L->bias[nc * NB + i] : 0.f;
        for (int kc = 0; kc < L->kc; ++kc) {
          const int g = kc / kb_per_group < L->ngroups ? kc / kb_per_group : L->ngroups - 1;
          const float* sc = L->scale + ((size_t)nc * L->ngroups + g) * NB;
          const float* zp = L->zp + ((size_t)nc * L->ngroups + g) * NB;
          if (L->is_int8)
            dequant_tile_int8(L->packed + ((size_t)nc * L->kc + kc) * L->kb * NB, L->kb, sc, zp, tile);
          else
            dequant_tile_int4(L->packed + ((size_t)nc * L->kc + kc) * L->kb * (NB / 2), L->kb, sc, zp, tile);
          block_gemm(xf + (size_t)m0 * k + (size_t)kc * L->kb, k, mrows, L->kb, tile, acc);
        }
        for (int mm = 0; mm < mrows; ++mm)
          for (int i = 0; i < NB; ++i) {
            const int col = nc * NB + i;
            if (col >= n) continue;
            const size_t o = (size_t)(m0 + mm) * n + col;
            float v = round_bf16(acc[mm * NB + i]);
            if (fusion != FUSE_SILU_MUL)
              v = post_op(v, fusion, other0 ? bf16_to_f32(other0[o]) : 0.f,
                          other1 ? bf16_to_f32(other1[o]) : 0.f);
            yo[o] = f32_to_bf16_rne(v);
          }
      }
    }
    free(tile);
    free(acc);
  }
  if (fusion == FUSE_SILU_MUL) {
    const int half = n / 2;
    for (int mm = 0; mm < m; ++mm)
      for (int c = 0; c < half; ++c) {
        const float gate = bf16_to_f32(ytmp[(size_t)mm * n + c]);
        const float up = bf16_to_f32(ytmp[(size_t)mm * n + half + c]);
        y[(size_t)mm * half + c] = f32_to_bf16_rne(up * silu_bf16(gate));
      }
    free(ytmp);
  }
  free(xf);
  return 0;
}

/* ---- small-M fp16 microkernel (woq.h:784-951) ------------------------------------------- */
EXPORT int woq_oracle_has_fp16_kernel(void) {
#ifdef WOQ_HAVE_FP16_KERNEL
  return __builtin_cpu_supports("avx512fp16") && __builtin_cpu_supports("avx512bw");
#else
  return 0;
#endif
}

#ifdef WOQ_HAVE_FP16_KERNEL
#define FP16_TARGET __attribute__((target("avx512fp16,avx512bw,avx512vl,avx512dq,avx512f")))

/* 32 floats -> 32 fp16 lanes (round to nearest even) */
FP16_TARGET static inline __m512h load32_f32_as_ph(const float* p) {
  const __m256h lo = _mm512_cvtxps_ph(_mm512_loadu_ps(p));
  const __m256h hi = _mm512_cvtxps_ph(_mm512_loadu_ps(p + 16));
  return _mm512_castsi512_ph(_mm512_inserti64x4(_mm512_castsi256_si512(_mm256_castph_si256(lo)),
                                                _mm256_castph_si256(hi), 1));
}

/* One 32-column block, all K, M <= 4 token rows.  c[m] leaves as 32 fp16 lanes. */
FP16_TARGET static void small_m_block_fp16(const woq_layer* L, int nc, const _Float16* xh, int m,
                                           int kb_per_group, __m512h* c) {
  /* LUT {0, ..., 15} as fp16 (asymmetric INT4; symmetric storage is q + 8 with zero point 8) */
  __m512h lut;
  {
    _Float16 t[32];
    for (int i = 0; i < 32; ++i) t[i] = (_Float16)(i & 15);
    lut = _mm512_loadu_ph(t);
  }
  const __m128i nib = _mm_set1_epi8(0x0F);
  for (int kc = 0; kc < L->kc; ++kc) {
    const int g = kc / kb_per_group < L->ngroups ? kc / kb_per_group : L->ngroups - 1;
    const size_t so = ((size_t)nc * L->ngroups + g) * NB;
    const __m512h vs = load32_f32_as_ph(L->scale32 + so);
    const __m512h vz = load32_f32_as_ph(L->zp + so);
    const uint8_t* blk = L->packed + ((size_t)nc * L->kc + kc) * L->kb * (NB / 2);
    __m512h acc[4];
    for (int mm = 0; mm < m; ++mm) acc[mm] = _mm512_setzero_ph();
    for (int kk = 0; kk < L->kb; ++kk) {
      const __m128i b = _mm_loadu_si128((const __m128i*)(blk + kk * (NB / 2)));
      _mm_prefetch((const char*)(blk + (kk + 64) * (NB / 2)), _MM_HINT_T0);
      const __m256i lo = _mm256_cvtepu8_epi16(_mm_and_si128(b, nib));
      const __m256i hi = _mm256_cvtepu8_epi16(_mm_and_si128(_mm_srli_epi16(b, 4), nib));
      const __m512i idx = _mm512_inserti64x4(_mm512_castsi256_si512(lo), hi, 1);
      const __m512h w = _mm512_sub_ph(_mm512_castsi512_ph(_mm512_permutexvar_epi16(idx, _mm512_castph_si512(lut))), vz);
      const int kidx = kc * L->kb + kk;
      for (int mm = 0; mm < m; ++mm)
        acc[mm] = _mm512_fmadd_ph(_mm512_set1_ph(xh[(size_t)mm * L->k + kidx]), w, acc[mm]);
    }
    for (int mm = 0; mm < m; ++mm) c[mm] = _mm512_fmadd_ph(vs, acc[mm], c[mm]);
  }
}

FP16_TARGET static int linear_fp16_small_m(const woq_layer* L, const uint16_t* x, int m, int fusion,
                                           const uint16_t* other0, const uint16_t* other1, uint16_t* y,
                                           int threads) {
  const int k = L->k, n = L->n;
  _Float16* xh = (_Float16*)malloc((size_t)m * k * sizeof(_Float16));
  for (size_t i = 0; i < (size_t)m * k; ++i) xh[i] = (_Float16)bf16_to_f32(x[i]);
  const int kb_per_group = L->group / L->kb > 0 ? L->group / L->kb : 1;
  uint16_t* ytmp = NULL;
  if (fusion == FUSE_SILU_MUL) ytmp = (uint16_t*)malloc((size_t)m * n * sizeof(uint16_t));
  uint16_t* yo = ytmp ? ytmp : y;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(static)
  for (int nc = 0; nc < L->nc; ++nc) {
    __m512h c[4];
    for (int mm = 0; mm < m; ++mm)
      c[mm] = L->bias ? load32_f32_as_ph(L->bias + nc * NB) : _mm512_setzero_ph();
    small_m_block_fp16(L, nc, xh, m, kb_per_group, c);
    for (int mm = 0; mm < m; ++mm) {
      _Float16 t[NB];
      _mm512_storeu_ph(t, c[mm]);
      for (int i = 0; i < NB; ++i) {
        const int col = nc * NB + i;
        if (col >= n) continue;
        const size_t o = (size_t)mm * n + col;
        float v = round_bf16((float)t[i]);
        if (fusion != FUSE_SILU_MUL)
          v = post_op(v, fusion, other0 ? bf16_to_f32(other0[o]) : 0.f, other1 ? bf16_to_f32(other1[o]) : 0.f);
        yo[o] = f32_to_bf16_rne(v);
      }
    }
  }
  if (fusion == FUSE_SILU_MUL) {
    const int half = n / 2;
    for (int mm = 0; mm < m; ++mm)
      for (int cc = 0; cc < half; ++cc) {
        const float gate = bf16_to_f32(ytmp[(size_t)mm * n + cc]);
        const float up = bf16_to_f32(ytmp[(size_t)mm * n + half + cc]);
        y[(size_t)mm * half + cc] = f32_to_bf16_rne(up * silu_bf16(gate));
      }
    free(ytmp);
  }
  free(xh);
  return 0;
}
#endif

/* The reference's kernel for lowp BF16 and fewer than 5 tokens: INT4 weights, fp16 arithmetic.
 * Returns -2 where the CPU lacks AVX512-FP16 (the caller then times the bf16 tile kernel). */
EXPORT int woq_oracle_linear_fp16_small_m(const woq_layer* L, const uint16_t* x, int m, int fusion,
                                          const uint16_t* other0, const uint16_t* other1, uint16_t* y,
                                          int threads) {
  if (L->is_int8 || m < 1 || m > 4) return -1;
#ifdef WOQ_HAVE_FP16_KERNEL
  if (woq_oracle_has_fp16_kernel()) return linear_fp16_small_m(L, x, m, fusion, other0, other1, y, threads);
#endif
  return -2;
}

/* Per-token symmetric activation quantisation; a row of zeros gets codes 0. */
EXPORT void woq_oracle_quant_act_sym(const uint16_t* x, int m, int k, int8_t* qa, float* sa) {
#pragma omp parallel for schedule(static)
  for (int mm = 0; mm < m; ++mm) {
    const uint16_t* xr = x + (size_t)mm * k;
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < k; ++i) {
      const float v = bf16_to_f32(xr[i]);
      mn = v < mn ? v : mn;
      mx = v > mx ? v : mx;
    }
    const float s = fmaxf(fabsf(mx), fabsf(mn)) / 127.0f;
    sa[mm] = s;
    for (int i = 0; i < k; ++i) {
      float q = s > 0.f ? nearbyintf(bf16_to_f32(xr[i]) / s) : 0.f;
      q = q < -128.f ? -128.f : (q > 127.f ? 127.f : q);
      qa[(size_t)mm * k + i] = (int8_t)q;
    }
  }
}

HOT static void block_gemm_s8(const int8_t* qa, int lda, int mrows, int kb, const int8_t* blk,
                              int32_t* qc) {
  for (int m = 0; m < mrows; ++m) {
    int32_t a[NB];
    for (int i = 0; i < NB; ++i) a[i] = 0;
    const int8_t* ar = qa + (size_t)m * lda;
    for (int kk = 0; kk < kb; ++kk) {
      const int32_t av = ar[kk];
      const int8_t* b = blk + kk * NB;
      for (int i = 0; i < NB; ++i) a[i] += av * (int32_t)b[i];
    }
    for (int i = 0; i < NB; ++i) qc[m * NB + i] = a[i];
  }
}

/* int8-compute linear for INT8 symmetric per-channel weights.  acc32 (optional) receives the
 * int32 accumulators summed over the whole K. */
EXPORT int woq_oracle_linear_int8(const woq_layer* L, const uint16_t* x, int m, int fusion,
                                  const uint16_t* other0, const uint16_t* other1, uint16_t* y,
                                  int32_t* acc32, int threads) {
  if (!L->is_int8) return -1;
  const int k = L->k, n = L->n;
  int8_t* qa = (int8_t*)malloc((size_t)m * k);
  float* sa = (float*)malloc((size_t)m * sizeof(float));
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
  woq_oracle_quant_act_sym(x, m, k, qa, sa);
  const int mblocks = (m + BLOCK_M - 1) / BLOCK_M;
  uint16_t* ytmp = NULL;
  if (fusion == FUSE_SILU_MUL) ytmp = (uint16_t*)malloc((size_t)m * n * sizeof(uint16_t));
  uint16_t* yo = ytmp ? ytmp : y;
#pragma omp parallel
  {
    int32_t* qc = (int32_t*)malloc((size_t)BLOCK_M * NB * sizeof(int32_t));
    int32_t* tot = (int32_t*)malloc((size_t)BLOCK_M * NB * sizeof(int32_t));
    float* c = (float*)malloc((size_t)BLOCK_M * NB * sizeof(float));
#pragma omp for collapse(2) schedule(static)
    for (int nc = 0; nc < L->nc; ++nc) {
      for (int mb = 0; mb < mblocks; ++mb) {
        const int m0 = mb * BLOCK_M, mrows = (m - m0) < BLOCK_M ? (m - m0) : BLOCK_M;
        const float* sw = L->scale + (size_t)nc * L->ngroups * NB; /* per channel: group 0 */
        for (int mm = 0; mm < mrows; ++mm)
          for (int i = 0; i < NB; ++i) {
            c[mm * NB + i] = L->bias ? L->bias[nc * NB + i] : 0.f;
            tot[mm * NB + i] = 0;
          }
        for (int kc = 0; kc < L->kc; ++kc) {
          block_gemm_s8(qa + (size_t)m0 * k + (size_t)kc * L->kb, k, mrows, L->kb,
                        (const int8_t*)L->packed + ((size_t)nc * L->kc + kc) * L->kb * NB, qc);
          for (int mm = 0; mm < mrows; ++mm)
            for (int i = 0; i < NB; ++i) {
              const float v = ((float)qc[mm * NB + i] * sa[m0 + mm]) * sw[i];
              c[mm * NB + i] = c[mm * NB + i] + v;
              tot[mm * NB + i] += qc[mm * NB + i];
            }
        }
        for (int mm = 0; mm < mrows; ++mm)
          for (int i = 0; i < NB; ++i) {
            const int col = nc * NB + i;
            if (col >= n) continue;
            const size_t o = (size_t)(m0 + mm) * n + col;
            if (acc32) acc32[o] = tot[mm * NB + i];
            float v = round_bf16(c[mm * NB + i]);
            if (fusion != FUSE_SILU_MUL)
              v = post_op(v, fusion, other0 ? bf16_to_f32(other0[o]) : 0.f,
                          other1 ? bf16_to_f32(other1[o]) : 0.f);
            yo[o] = f32_to_bf16_rne(v);
          }
      }
    }
    free(qc); free(tot); free(c);
  }
  if (fusion == FUSE_SILU_MUL) {
    const int half = n / 2;
    for (int mm = 0; mm < m; ++mm)
      for (int cc = 0; cc < half; ++cc) {
        const float gate = bf16_to_f32(ytmp[(size_t)mm * n + cc]);
        const float up = bf16_to_f32(ytmp[(size_t)mm * n + half + cc]);
        y[(size_t)mm * half + cc] = f32_to_bf16_rne(up * silu_bf16(gate));
      }
    free(ytmp);
  }
  free(qa);
  free(sa);
  return 0;
}

EXPORT int woq_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
