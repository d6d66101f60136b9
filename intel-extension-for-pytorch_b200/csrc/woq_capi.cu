// C ABI of libwoq_b200.so (declared in include/woq_b200.h): contexts, argument checks and
// kernel selection.  No kernel code lives here.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include <cuda_fp16.h>

#include "../../include/woq_b200.h"
#include "woq_internal.h"
#include "woq_kernels.h"

namespace woq {
static std::atomic<int64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace woq

namespace {

constexpr uint64_t kMagic = 0x574f5142323030ull;  // "WOQB200"
constexpr size_t kWsHeaderBytes = 64 * 1024;      // status word + per-tile arrival counters
constexpr int kMaxCounterTiles = (kWsHeaderBytes - 256) / 4;

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace

namespace woq {
int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace woq

namespace {

#define CUDA_TRY(expr)                                                                     \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return fail(WOQ_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));     \
  } while (0)

}  // namespace

struct woq_b200_ctx {
  uint64_t magic;
  woq_b200_desc desc;
  int device;
  int num_sms;
  // derived
  int tiles;         // ceil(N / 64) (gate/up layout: N / 64)
  int kb_per_tile;   // K / 64
  int kb_per_group;  // group size / 64 (per-channel: kb_per_tile)
  int groups;        // groups along K
  int gate_up;
  // device buffers
  uint8_t* wq;       // INT4: tiled nibbles; INT8: plain [n_pad][k]
  uint32_t* sz;      // INT4 group scales + zero points
  uint8_t* wq_tc;    // INT4: 128-row layout for the tensor-core kernel
  uint32_t* sz_tc;
  int tiles_tc, kbpg_shift;
  size_t wq_tc_bytes, sz_tc_bytes;
  float* scale_f32;  // INT8: per-channel fp32 scales [n_pad]
  int32_t* comp;     // INT8 with asymmetric activations: per-row sums of the weight codes [n_pad]
  int is_int8;       // INT8 weights with INT8 compute
  int plain_scales;  // INT4: every scale is normal and below 0.5, every zero point below 16
  int kc_per_tile;   // INT8: K / 128
  float* bias;       // fp32 [n] or null
  size_t wq_bytes, sz_bytes;
  // Prepack check result (bit 0: a zero point is not an integer in 0..127, bit 1: scales or zero
  // points outside the range of the shift-free dequantiser).  With WOQ_B200_LAYOUT_DEFER_CHECK
  // the flag travels to pinned host memory asynchronously and is looked at by the first call
  // that needs it, so that loading many layers does not synchronise once per layer.
  // general route (woq_generic.cu): plain weight bytes, fp32 scales / zero points [n][groups]
  int is_generic;
  uint8_t* g_w;
  float* g_scales;
  float* g_zps;
  int g_row_bytes, g_group, g_groups;
  // INT8 compute with K-block scaling (woq_int8_block.cu): the buffers above plus comp
  int is_i8block, kb, kc;
  int* d_flag;
  int* h_flag;
  cudaEvent_t flag_ready;
  int flag_pending;  // 1 until the flag has been looked at
  int flag_bad;
};

namespace woq {
int ctx_device(const woq_b200_ctx* c) { return c && c->magic == kMagic ? c->device : -1; }
}  // namespace woq

namespace {

// The buffers of a context (and the kernels' launch configuration) belong to one device: a
// call made with another device current would hand this device's pointers to that one.
int check_current_device(const woq_b200_ctx* c) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != c->device)
    return fail(WOQ_B200_ERR_INVALID_ARG, "the context lives on device %d but device %d is current", c->device, dev);
  return WOQ_B200_OK;
}

int check_ctx(const woq_b200_ctx* c) {
  if (!c) return fail(WOQ_B200_ERR_INVALID_ARG, "context is null");
  if (c->magic != kMagic) return fail(WOQ_B200_ERR_BAD_HANDLE, "context magic mismatch");
  return WOQ_B200_OK;
}

// Looks at a deferred prepack check result once (see woq_b200_ctx::d_flag).
int settle_prepack_flag(const woq_b200_ctx* cc) {
  woq_b200_ctx* c = const_cast<woq_b200_ctx*>(cc);
  if (c->flag_pending) {
    CUDA_TRY(cudaEventSynchronize(c->flag_ready));
    c->flag_bad = (*c->h_flag & 1) ? 1 : 0;
    c->plain_scales = (*c->h_flag & 2) ? 0 : 1;
    c->flag_pending = 0;
  }
  if (c->flag_bad) return fail(WOQ_B200_ERR_INVALID_ARG, "zero points must be integers in [0, 127]");
  return WOQ_B200_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__global__ void convert_bias_kernel(const void* src, float* dst, int n, int dtype) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  dst[i] = dtype == WOQ_B200_T_F32 ? reinterpret_cast<const float*>(src)[i]
                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i]);
}

}  // namespace

namespace {

// INT8 symmetric per-channel weights, INT8 compute with per-token symmetric activations
int create_int8(const woq_b200_desc* d, const void* qweight, const void* scales,
                const void* zero_points, const void* bias, cudaStream_t stream, woq_b200_ctx** out) {
  if (d->lowp_mode != WOQ_B200_LOWP_INT8)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "INT8 weights are built for lowp_mode INT8 only (got %d)", d->lowp_mode);
  if (d->act_quant_mode != WOQ_B200_ACT_PER_M_SYM && d->act_quant_mode != WOQ_B200_ACT_PER_M &&
      d->act_quant_mode != WOQ_B200_ACT_PER_TENSOR_SYM && d->act_quant_mode != WOQ_B200_ACT_PER_TENSOR)
    return fail(WOQ_B200_ERR_UNSUPPORTED,
                "activation quantisation mode %d is not built (per tensor 0 / 4 and per token 2 / 6 are; the "
                "per-K-block modes 1, 3, 5, 7 are not)", d->act_quant_mode);
  if (zero_points) return fail(WOQ_B200_ERR_INVALID_ARG, "INT8 weights with INT8 compute are symmetric: no zero points");
  if (d->group_size > 0 && d->group_size < d->k)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "INT8 compute path takes per-channel weight scales (group_size -1)");
  if (d->weight_format != WOQ_B200_FMT_PLAIN) return fail(WOQ_B200_ERR_INVALID_ARG, "INT8 weights come in plain format");
  if (d->k % 128 != 0) return fail(WOQ_B200_ERR_UNSUPPORTED, "INT8 path needs K %% 128 == 0 (K=%lld)", (long long)d->k);
  const int gate_up = (d->layout_flags & WOQ_B200_LAYOUT_GATE_UP) ? 1 : 0;
  if (gate_up && (d->n % 128 != 0)) return fail(WOQ_B200_ERR_INVALID_ARG, "gate/up layout needs N %% 128 == 0");
  woq_b200_ctx* c = new (std::nothrow) woq_b200_ctx();
  if (!c) return fail(WOQ_B200_ERR_CUDA, "out of host memory");
  memset(c, 0, sizeof(*c));
  c->desc = *d;
  c->gate_up = gate_up;
  c->is_int8 = 1;
  auto bail = [&](int rc) {
    if (c->wq) cudaFree(c->wq);
    if (c->scale_f32) cudaFree(c->scale_f32);
    if (c->bias) cudaFree(c->bias);
    if (c->comp) cudaFree(c->comp);
    delete c;
    return rc;
  };
#define CUDA_TRY_I(expr)                                                                    \
  do {                                                                                      \
    cudaError_t e__ = (expr);                                                               \
    if (e__ != cudaSuccess)                                                                 \
      return bail(fail(WOQ_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__))); \
  } while (0)
  CUDA_TRY_I(cudaGetDevice(&c->device));
  CUDA_TRY_I(cudaDeviceGetAttribute(&c->num_sms, cudaDevAttrMultiProcessorCount, c->device));
  c->tiles_tc = static_cast<int>((d->n + 127) / 128);
  c->kc_per_tile = static_cast<int>(d->k / 128);
  c->wq_bytes = static_cast<size_t>(c->tiles_tc) * 2 * c->kc_per_tile * 8192;
  c->sz_bytes = static_cast<size_t>(c->tiles_tc) * 128 * sizeof(float);
  CUDA_TRY_I(cudaMalloc(&c->wq, c->wq_bytes));
  CUDA_TRY_I(cudaMalloc(&c->scale_f32, c->sz_bytes));
  CUDA_TRY_I(woq::launch_pack_int8(static_cast<const int8_t*>(qweight), reinterpret_cast<int8_t*>(c->wq),
                                   (int)d->n, (int)d->k, c->tiles_tc * 2, gate_up, stream));
  CUDA_TRY_I(woq::launch_pad_scale(scales, c->scale_f32, (int)d->n, c->tiles_tc * 128, d->scale_dtype, stream));
  if (d->act_quant_mode == WOQ_B200_ACT_PER_M || d->act_quant_mode == WOQ_B200_ACT_PER_TENSOR) {
    // asymmetric activations: the zero point's share of every accumulator is taken out with
    // the per-row sums of the weight codes (the reference's cached compensation)
    const size_t comp_bytes = static_cast<size_t>(c->tiles_tc) * 128 * sizeof(int32_t);
    CUDA_TRY_I(cudaMalloc(&c->comp, comp_bytes));
    CUDA_TRY_I(cudaMemsetAsync(c->comp, 0, comp_bytes, stream));
    CUDA_TRY_I(woq::launch_weight_row_sum(static_cast<const int8_t*>(qweight), (int)d->n, (int)d->k, c->comp, stream));
  }
  if (bias) {
    CUDA_TRY_I(cudaMalloc(&c->bias, static_cast<size_t>(d->n) * sizeof(float)));
    convert_bias_kernel<<<(unsigned)((d->n + 255) / 256), 256, 0, stream>>>(bias, c->bias, (int)d->n, d->bias_dtype);
    woq::count_launch();
    CUDA_TRY_I(cudaGetLastError());
  }
  CUDA_TRY_I(cudaStreamSynchronize(stream));
#undef CUDA_TRY_I
  c->magic = kMagic;
  *out = c;
  return WOQ_B200_OK;
}

struct Int8Workspace {
  size_t partial_off, sa_off, zpa_off, range_off, qa_off, total;
};
Int8Workspace int8_ws_layout(const woq_b200_ctx* c, int64_t m) {
  Int8Workspace w;
  int n_tok = static_cast<int>(m < 256 ? m : 256);
  n_tok = (n_tok + 15) / 16 * 16;
  if (n_tok < 16) n_tok = 16;
  w.partial_off = kWsHeaderBytes;
  size_t off = w.partial_off + woq::int8_partial_bytes(c->num_sms, n_tok);
  w.sa_off = (off + 255) / 256 * 256;
  const size_t m_pad = static_cast<size_t>((m + 63) / 64 * 64);
  w.zpa_off = w.sa_off + m_pad * sizeof(float);
  w.range_off = w.zpa_off + m_pad * sizeof(int32_t);
  off = w.range_off + 2 * m_pad * sizeof(float);
  w.qa_off = (off + 1023) / 1024 * 1024;
  w.total = w.qa_off + static_cast<size_t>(m) * c->desc.k;
  return w;
}

}  // namespace

namespace {

__global__ void to_f32_kernel(const void* src, float* dst, int64_t count, int dtype) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float v;
  switch (dtype) {
    case WOQ_B200_T_F32: v = static_cast<const float*>(src)[i]; break;
    case WOQ_B200_T_F16: v = __half2float(static_cast<const __half*>(src)[i]); break;
    case WOQ_B200_T_BF16: v = __bfloat162float(static_cast<const __nv_bfloat16*>(src)[i]); break;
    case WOQ_B200_T_U8: v = static_cast<float>(static_cast<const uint8_t*>(src)[i]); break;
    default: v = static_cast<float>(static_cast<const int8_t*>(src)[i]); break;
  }
  dst[i] = v;
}

// Does a description need the general route (woq_generic.cu)?  The tuned kernels take INT4 with
// bf16 compute on 64-aligned shapes and INT8 with INT8 compute.
bool wants_generic(const woq_b200_desc* d) {
  if (d->layout_flags & WOQ_B200_LAYOUT_GENERIC) return true;
  if (d->weight_dtype == WOQ_B200_DTYPE_NF4 || d->weight_dtype == WOQ_B200_DTYPE_FP8) return true;
  if (d->lowp_mode == WOQ_B200_LOWP_INT8) return false;
  if (d->weight_dtype == WOQ_B200_DTYPE_INT8) return true;
  if (d->lowp_mode == WOQ_B200_LOWP_FP16) return true;
  if (d->k % 64 != 0) return true;
  const int64_t g_eff = d->group_size > 0 ? d->group_size : d->k;
  if (g_eff < d->k && (g_eff % 64 != 0 || (g_eff & (g_eff - 1)) != 0)) return true;
  return false;
}

// lowp INT8 descriptions the tcgen05 INT8 kernel does not take: INT4 weights, grouped weight
// scales, or an activation range per K block (modes 1, 3, 5, 7)
bool wants_i8block(const woq_b200_desc* d) {
  if (d->lowp_mode != WOQ_B200_LOWP_INT8) return false;
  if (d->weight_dtype == WOQ_B200_DTYPE_INT4) return true;
  if (d->weight_dtype != WOQ_B200_DTYPE_INT8) return false;
  if (d->group_size > 0 && d->group_size < d->k) return true;
  return (d->act_quant_mode & 1) != 0;
}

struct I8BlockWs {
  size_t qa, sa, zpa, sumqa, range, folded, total;
};
I8BlockWs i8block_ws(const woq_b200_ctx* c, int64_t m) {
  I8BlockWs w;
  const size_t mk = static_cast<size_t>(m) * c->kc;
  size_t off = kWsHeaderBytes;
  w.sa = off;      off += (mk * 4 + 255) / 256 * 256;
  w.zpa = off;     off += (mk * 4 + 255) / 256 * 256;
  w.sumqa = off;   off += (mk * 4 + 255) / 256 * 256;
  w.range = off;   off += (mk * 8 + 255) / 256 * 256;
  w.folded = off;  off += (static_cast<size_t>(m > c->kc ? m : c->kc) * 8 + 255) / 256 * 256;
  w.qa = off;      off += (static_cast<size_t>(m) * c->desc.k + 255) / 256 * 256;
  w.total = off;
  return w;
}

int create_generic(const woq_b200_desc* d, const void* qweight, const void* scales, const void* zero_points,
                   const void* bias, cudaStream_t stream, woq_b200_ctx** out);

int create_i8block(const woq_b200_desc* d, const void* qweight, const void* scales, const void* zero_points,
                   const void* bias, cudaStream_t stream, woq_b200_ctx** out) {
  if (d->act_quant_mode < 0 || d->act_quant_mode > 7)
    return fail(WOQ_B200_ERR_INVALID_ARG, "activation quantisation mode must be 0..7 for lowp INT8, got %d", d->act_quant_mode);
  if (d->layout_flags & WOQ_B200_LAYOUT_GATE_UP)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "no fused silu*mul on the K-block INT8 route (use silu, then mul)");
  int kb = d->group_size > 0 && d->group_size < 128 ? d->group_size : 128;
  while (d->k % kb) kb /= 2;
  if (kb < 64)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "INT8 compute needs a K block of 64 or 128 (K=%lld, group %d give %d)",
                (long long)d->k, d->group_size, kb);
  // storage: the plain weight and fp32 scales / zero points of the general route
  woq_b200_desc g = *d;
  g.lowp_mode = WOQ_B200_LOWP_BF16;
  g.layout_flags |= WOQ_B200_LAYOUT_GENERIC;
  woq_b200_ctx* c = nullptr;
  if (int rc = create_generic(&g, qweight, scales, zero_points, bias, stream, &c)) return rc;
  c->desc = *d;
  c->is_generic = 0;
  c->is_i8block = 1;
  c->kb = kb;
  c->kc = static_cast<int>(d->k / kb);
  if (!(d->act_quant_mode & 4)) {
    cudaError_t e = cudaMalloc(&c->comp, static_cast<size_t>(d->n) * c->kc * sizeof(int32_t));
    if (e == cudaSuccess)
      e = woq::launch_weight_block_sum(c->g_w, c->g_zps, (int)d->n, (int)d->k, kb, c->g_group, c->g_groups,
                                       d->weight_dtype == WOQ_B200_DTYPE_INT4 ? 8.f : 0.f,
                                       d->weight_dtype == WOQ_B200_DTYPE_INT4, c->comp, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) {
      woq_b200_ctx_destroy(c);
      return fail(WOQ_B200_ERR_CUDA, "block sums of the weight: %s", cudaGetErrorString(e));
    }
    woq::count_launch();
  }
  *out = c;
  return WOQ_B200_OK;
}

int run_i8block(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx, int32_t fusion, const void* o0,
                const void* o1, void* y, int64_t ldy, uint8_t* qa_natural, float* sa_out, int32_t* zpa_out,
                int32_t* acc_out, void* ws, size_t ws_bytes, cudaStream_t stream) {
  const I8BlockWs L = i8block_ws(c, m);
  if (ws_bytes < L.total) return fail(WOQ_B200_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", ws_bytes, L.total);
  if (fusion == WOQ_B200_FUSE_SILU_MUL)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "no fused silu*mul on the K-block INT8 route (use silu, then mul)");
  uint8_t* w8 = static_cast<uint8_t*>(ws);
  const int mode = c->desc.act_quant_mode;
  const int w4 = c->desc.weight_dtype == WOQ_B200_DTYPE_INT4;
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  float* sa = reinterpret_cast<float*>(w8 + L.sa);
  int32_t* zpa = reinterpret_cast<int32_t*>(w8 + L.zpa);
  int32_t* sumqa = reinterpret_cast<int32_t*>(w8 + L.sumqa);
  float* range = reinterpret_cast<float*>(w8 + L.range);
  float* folded = reinterpret_cast<float*>(w8 + L.folded);
  if (qa_natural) {  // parity hook: the codes in natural order
    CUDA_TRY(woq::launch_act_block_quant(xb, ldx, (int)m, (int)c->desc.k, c->kb, mode, 0, qa_natural, sa, zpa, sumqa,
                                         range, folded, stream));
    woq::count_launch();
  }
  CUDA_TRY(woq::launch_act_block_quant(xb, ldx, (int)m, (int)c->desc.k, c->kb, mode, w4, w8 + L.qa, sa, zpa, sumqa,
                                       range, folded, stream));
  woq::count_launch();
  const size_t mk = static_cast<size_t>(m) * c->kc;
  if (sa_out) CUDA_TRY(cudaMemcpyAsync(sa_out, sa, mk * 4, cudaMemcpyDeviceToDevice, stream));
  if (zpa_out) CUDA_TRY(cudaMemcpyAsync(zpa_out, zpa, mk * 4, cudaMemcpyDeviceToDevice, stream));
  if (!y && !acc_out) return WOQ_B200_OK;
  woq::I8BlockParams p{};
  p.w = c->g_w;
  p.sw = c->g_scales;
  p.zpw = c->g_zps;
  p.comp = c->comp;
  p.qa = w8 + L.qa;
  p.sa = sa;
  p.zpa = zpa;
  p.sumqa = sumqa;
  p.bias = c->bias;
  p.y = static_cast<__nv_bfloat16*>(y);
  p.other0 = static_cast<const __nv_bfloat16*>(o0);
  p.other1 = static_cast<const __nv_bfloat16*>(o1);
  p.acc_out = acc_out;
  p.ldy = ldy;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(c->desc.n);
  p.k = static_cast<int>(c->desc.k);
  p.kb = c->kb;
  p.kc = c->kc;
  p.group = c->g_group;
  p.groups = c->g_groups;
  p.fusion = fusion;
  p.w4 = w4;
  p.asym = (mode & 4) ? 0 : 1;
  p.default_zp = w4 ? 8.f : 0.f;
  CUDA_TRY(woq::launch_i8_block(p, stream));
  woq::count_launch();
  return WOQ_B200_OK;
}

int create_generic(const woq_b200_desc* d, const void* qweight, const void* scales, const void* zero_points,
                   const void* bias, cudaStream_t stream, woq_b200_ctx** out) {
  if (d->lowp_mode == WOQ_B200_LOWP_INT8)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "the general route computes in fp32 / fp16 / bf16, not INT8");
  if (d->weight_format != WOQ_B200_FMT_PLAIN)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "the general route takes plain-format weights (GPTQ / AWQ layouts go "
                "through the INT4 bf16 route: K %% 64 == 0, power-of-two group size >= 64)");
  if (d->layout_flags & WOQ_B200_LAYOUT_GATE_UP)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "the gate/up layout belongs to the INT4 bf16 and INT8 routes");
  const int64_t g_eff = d->group_size > 0 && d->group_size < d->k ? d->group_size : d->k;
  if (g_eff < d->k && g_eff % 8 != 0)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "group size must be a multiple of 8 (got %d)", d->group_size);
  const bool four_bit = d->weight_dtype == WOQ_B200_DTYPE_INT4 || d->weight_dtype == WOQ_B200_DTYPE_NF4;
  if ((d->weight_dtype == WOQ_B200_DTYPE_NF4 || d->weight_dtype == WOQ_B200_DTYPE_FP8) && zero_points)
    return fail(WOQ_B200_ERR_INVALID_ARG, "NF4 / FP8 weights are symmetric: no zero points");
  woq_b200_ctx* c = new (std::nothrow) woq_b200_ctx();
  if (!c) return fail(WOQ_B200_ERR_CUDA, "out of host memory");
  memset(c, 0, sizeof(*c));
  c->desc = *d;
  c->is_generic = 1;
  c->g_row_bytes = static_cast<int>(four_bit ? (d->k + 1) / 2 : d->k);
  c->g_group = static_cast<int>(g_eff);
  c->g_groups = static_cast<int>((d->k + g_eff - 1) / g_eff);
  auto bail = [&](int rc) {
    cudaFree(c->g_w);
    cudaFree(c->g_scales);
    cudaFree(c->g_zps);
    cudaFree(c->bias);
    delete c;
    return rc;
  };
#define CUDA_TRY_G(expr)                                                                    \
  do {                                                                                      \
    cudaError_t e__ = (expr);                                                               \
    if (e__ != cudaSuccess)                                                                 \
      return bail(fail(WOQ_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__))); \
  } while (0)
  CUDA_TRY_G(cudaGetDevice(&c->device));
  CUDA_TRY_G(cudaDeviceGetAttribute(&c->num_sms, cudaDevAttrMultiProcessorCount, c->device));
  c->wq_bytes = static_cast<size_t>(d->n) * c->g_row_bytes;
  const int64_t sg = d->n * c->g_groups;
  c->sz_bytes = static_cast<size_t>(sg) * sizeof(float) * (zero_points ? 2 : 1);
  CUDA_TRY_G(cudaMalloc(&c->g_w, c->wq_bytes));
  CUDA_TRY_G(cudaMalloc(&c->g_scales, sg * sizeof(float)));
  CUDA_TRY_G(cudaMemcpyAsync(c->g_w, qweight, c->wq_bytes, cudaMemcpyDeviceToDevice, stream));
  to_f32_kernel<<<static_cast<unsigned>((sg + 255) / 256), 256, 0, stream>>>(scales, c->g_scales, sg, d->scale_dtype);
  woq::count_launch();
  if (zero_points) {
    if (d->zp_dtype != WOQ_B200_T_F32 && d->zp_dtype != WOQ_B200_T_U8 && d->zp_dtype != WOQ_B200_T_S8)
      return bail(fail(WOQ_B200_ERR_INVALID_ARG, "zero points must be fp32, u8 or s8 here"));
    CUDA_TRY_G(cudaMalloc(&c->g_zps, sg * sizeof(float)));
    to_f32_kernel<<<static_cast<unsigned>((sg + 255) / 256), 256, 0, stream>>>(zero_points, c->g_zps, sg, d->zp_dtype);
    woq::count_launch();
  }
  if (bias) {
    CUDA_TRY_G(cudaMalloc(&c->bias, static_cast<size_t>(d->n) * sizeof(float)));
    to_f32_kernel<<<static_cast<unsigned>((d->n + 255) / 256), 256, 0, stream>>>(bias, c->bias, d->n, d->bias_dtype);
    woq::count_launch();
  }
  CUDA_TRY_G(cudaGetLastError());
  CUDA_TRY_G(cudaStreamSynchronize(stream));
#undef CUDA_TRY_G
  c->magic = kMagic;
  *out = c;
  return WOQ_B200_OK;
}

// compute dtype of a call on a general-route context
int generic_compute_dtype(const woq_b200_ctx* c, int io_dtype) {
  if (c->desc.lowp_mode == WOQ_B200_LOWP_BF16) return WOQ_B200_T_BF16;
  if (c->desc.lowp_mode == WOQ_B200_LOWP_FP16) return WOQ_B200_T_F16;
  return io_dtype;  // lowp NONE: the activation's dtype (WoqLinearKrnl.cpp:75-106)
}

void fill_generic(const woq_b200_ctx* c, woq::GenericParams* p) {
  p->w = c->g_w;
  p->scales = c->g_scales;
  p->zps = c->g_zps;
  p->bias = c->bias;
  p->n = static_cast<int>(c->desc.n);
  p->k = static_cast<int>(c->desc.k);
  p->group = c->g_group;
  p->groups = c->g_groups;
  p->row_bytes = c->g_row_bytes;
  p->weight_dtype = c->desc.weight_dtype;
  p->default_zp = c->desc.weight_dtype == WOQ_B200_DTYPE_INT4 ? 8.f : 0.f;
}

}  // namespace

extern "C" {

int woq_b200_version(void) { return 100; }

const char* woq_b200_last_error(void) { return g_err; }

int64_t woq_b200_kernel_launches(void) { return woq::g_launches.load(); }

size_t woq_b200_workspace_header_bytes(void) { return kWsHeaderBytes; }

int woq_b200_set_option(int32_t option, int32_t value) {
  if (option == WOQ_B200_OPT_DECODE_SPLIT) {
    if (value < 0 || value > 2) return fail(WOQ_B200_ERR_INVALID_ARG, "decode split must be 0, 1 or 2, got %d", value);
    woq::decode_int4_set_split(value);
    return WOQ_B200_OK;
  }
  return fail(WOQ_B200_ERR_INVALID_ARG, "unknown option %d", option);
}

int woq_b200_ctx_create(const woq_b200_desc* d, const void* qweight, const void* scales,
                        const void* zero_points, const void* bias, void* stream_,
                        woq_b200_ctx** out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!d || !qweight || !scales || !out)
    return fail(WOQ_B200_ERR_INVALID_ARG, "desc, qweight, scales and out must be non-null");
  *out = nullptr;
  if (d->n <= 0 || d->k <= 0 || d->n > (1 << 24) || d->k > (1 << 24))
    return fail(WOQ_B200_ERR_INVALID_ARG, "bad shape N=%lld K=%lld", (long long)d->n, (long long)d->k);
  if (d->weight_dtype < WOQ_B200_DTYPE_INT8 || d->weight_dtype > WOQ_B200_DTYPE_FP8)
    return fail(WOQ_B200_ERR_INVALID_ARG, "unknown weight dtype %d", d->weight_dtype);
  if (d->lowp_mode < WOQ_B200_LOWP_NONE || d->lowp_mode > WOQ_B200_LOWP_INT8)
    return fail(WOQ_B200_ERR_INVALID_ARG, "unknown lowp_mode %d", d->lowp_mode);
  if (d->group_size == 0 || d->group_size < -1)
    return fail(WOQ_B200_ERR_INVALID_ARG, "group_size must be -1 or positive, got %d", d->group_size);
  if ((zero_points == nullptr) != (d->zp_dtype == WOQ_B200_T_NONE))
    return fail(WOQ_B200_ERR_INVALID_ARG, "zero_points pointer and zp_dtype disagree");
  if ((bias == nullptr) != (d->bias_dtype == WOQ_B200_T_NONE))
    return fail(WOQ_B200_ERR_INVALID_ARG, "bias pointer and bias_dtype disagree");
  if (d->bias_dtype != WOQ_B200_T_NONE && d->bias_dtype != WOQ_B200_T_F32 &&
      d->bias_dtype != WOQ_B200_T_BF16)
    return fail(WOQ_B200_ERR_INVALID_ARG, "bias must be fp32 or bf16");
  if (d->scale_dtype != WOQ_B200_T_F32 && d->scale_dtype != WOQ_B200_T_F16 &&
      d->scale_dtype != WOQ_B200_T_BF16)
    return fail(WOQ_B200_ERR_INVALID_ARG, "scales must be fp32, fp16 or bf16");

  if (wants_i8block(d)) return create_i8block(d, qweight, scales, zero_points, bias, stream, out);
  if (wants_generic(d)) return create_generic(d, qweight, scales, zero_points, bias, stream, out);
  if (d->weight_dtype == WOQ_B200_DTYPE_INT8) return create_int8(d, qweight, scales, zero_points, bias, stream, out);
  // ---- INT4 ----
  if (d->k % 64 != 0)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "INT4 path needs K %% 64 == 0 (K=%lld)", (long long)d->k);
  const int64_t g_eff = d->group_size > 0 ? d->group_size : d->k;
  if (g_eff % 64 != 0 || (g_eff < d->k && (g_eff & (g_eff - 1)) != 0))
    return fail(WOQ_B200_ERR_UNSUPPORTED,
                "INT4 path needs a power-of-two group size >= 64 or per-channel (got %d)",
                d->group_size);
  const int gate_up = (d->layout_flags & WOQ_B200_LAYOUT_GATE_UP) ? 1 : 0;
  if (gate_up && (d->n % 128 != 0))
    return fail(WOQ_B200_ERR_INVALID_ARG, "gate/up layout needs N %% 128 == 0");
  if (d->weight_format != WOQ_B200_FMT_PLAIN && (d->n % 8 != 0))
    return fail(WOQ_B200_ERR_INVALID_ARG, "GPTQ/AWQ formats need N %% 8 == 0");

  woq_b200_ctx* c = new (std::nothrow) woq_b200_ctx();
  if (!c) return fail(WOQ_B200_ERR_CUDA, "out of host memory");
  memset(c, 0, sizeof(*c));
  c->desc = *d;
  c->gate_up = gate_up;
  CUDA_TRY(cudaGetDevice(&c->device));
  CUDA_TRY(cudaDeviceGetAttribute(&c->num_sms, cudaDevAttrMultiProcessorCount, c->device));
  c->tiles = static_cast<int>((d->n + 63) / 64);
  c->kb_per_tile = static_cast<int>(d->k / 64);
  c->kb_per_group = static_cast<int>(g_eff >= d->k ? c->kb_per_tile : g_eff / 64);
  c->groups = static_cast<int>((d->k + g_eff - 1) / g_eff);
  c->wq_bytes = static_cast<size_t>(c->tiles) * c->kb_per_tile * woq::kBlockBytes;
  c->sz_bytes = static_cast<size_t>(c->tiles) * c->groups * 64 * 4;
  c->tiles_tc = static_cast<int>((d->n + 127) / 128);
  c->kbpg_shift = 30;  // per-channel: every k-block maps to group 0
  if (g_eff < d->k) {
    c->kbpg_shift = 0;
    while ((1 << c->kbpg_shift) < c->kb_per_group) ++c->kbpg_shift;
  }
  c->wq_tc_bytes = static_cast<size_t>(c->tiles_tc) * c->kb_per_tile * woq::kTcBlockBytes;
  c->sz_tc_bytes = static_cast<size_t>(c->tiles_tc) * c->groups * 128 * 4;

  int* d_flag = nullptr;
  uint8_t* tmp_plain = nullptr;
  uint8_t* tmp_zp = nullptr;
  auto cleanup = [&](int rc) {
    if (tmp_plain) cudaFree(tmp_plain);
    if (tmp_zp) cudaFree(tmp_zp);
    if (rc != WOQ_B200_OK) {
      if (c->d_flag) cudaFree(c->d_flag);
      if (c->h_flag) cudaFreeHost(c->h_flag);
      if (c->flag_ready) cudaEventDestroy(c->flag_ready);
      if (c->wq) cudaFree(c->wq);
      if (c->sz) cudaFree(c->sz);
      if (c->wq_tc) cudaFree(c->wq_tc);
      if (c->sz_tc) cudaFree(c->sz_tc);
      if (c->bias) cudaFree(c->bias);
      delete c;
    }
    return rc;
  };
#define CUDA_TRY_C(expr)                                                                       \
  do {                                                                                         \
    cudaError_t e__ = (expr);                                                                  \
    if (e__ != cudaSuccess)                                                                    \
      return cleanup(fail(WOQ_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__))); \
  } while (0)

  const bool want_stream = !(d->layout_flags & WOQ_B200_LAYOUT_TC_ONLY);
  const bool want_tc = !(d->layout_flags & WOQ_B200_LAYOUT_STREAM_ONLY);
  if (!want_stream) c->wq_bytes = c->sz_bytes = 0;
  if (!want_tc) c->wq_tc_bytes = c->sz_tc_bytes = 0;
  if (want_stream) {
    CUDA_TRY_C(cudaMalloc(&c->wq, c->wq_bytes));
    CUDA_TRY_C(cudaMalloc(&c->sz, c->sz_bytes));
  }
  if (want_tc) {
    CUDA_TRY_C(cudaMalloc(&c->wq_tc, c->wq_tc_bytes));
    CUDA_TRY_C(cudaMalloc(&c->sz_tc, c->sz_tc_bytes));
  }
  CUDA_TRY_C(cudaMalloc(&c->d_flag, sizeof(int)));
  CUDA_TRY_C(cudaMallocHost(&c->h_flag, sizeof(int)));
  CUDA_TRY_C(cudaEventCreateWithFlags(&c->flag_ready, cudaEventDisableTiming));
  d_flag = c->d_flag;
  *c->h_flag = 0;
  CUDA_TRY_C(cudaMemsetAsync(d_flag, 0, sizeof(int), stream));

  const uint8_t* plain = static_cast<const uint8_t*>(qweight);
  const void* zps = zero_points;
  int zp_dtype = d->zp_dtype;
  int transposed = 0;
  if (d->weight_format != WOQ_B200_FMT_PLAIN) {
    // int32 checkpoint layouts: scales / zero points are [groups][N]
    CUDA_TRY_C(cudaMalloc(&tmp_plain, static_cast<size_t>(d->n) * (d->k / 2)));
    if (d->weight_format == WOQ_B200_FMT_AWQ)
      CUDA_TRY_C(woq::launch_awq_to_plain(static_cast<const int32_t*>(qweight), tmp_plain,
                                          (int)d->n, (int)d->k, stream));
    else
      CUDA_TRY_C(woq::launch_gptq_to_plain(static_cast<const int32_t*>(qweight), tmp_plain,
                                           (int)d->n, (int)d->k, stream));
    plain = tmp_plain;
    transposed = (d->layout_flags & WOQ_B200_LAYOUT_SCALES_NK) ? 0 : 1;
    if (zero_points && d->zp_dtype != WOQ_B200_T_F32 && d->zp_dtype != WOQ_B200_T_U8) {
      // packed int32 zero points [groups][N/8]
      CUDA_TRY_C(cudaMalloc(&tmp_zp, static_cast<size_t>(d->n) * c->groups));
      CUDA_TRY_C(woq::launch_unpack_qzeros(static_cast<const int32_t*>(zero_points), tmp_zp,
                                           (int)d->n, c->groups,
                                           d->weight_format == WOQ_B200_FMT_AWQ, 0, stream));
      zps = tmp_zp;
      zp_dtype = WOQ_B200_T_U8;
      // tmp_zp is [N][groups]; scales stay transposed -> handled by two passes below
    }
  }
  if (want_stream) {
    woq::PackInt4Args pa{plain, c->wq, (int)d->n, (int)d->k, c->tiles, c->kb_per_tile, gate_up, 0};
    CUDA_TRY_C(woq::launch_pack_int4(pa, stream));
  }
  if (want_tc) {
    woq::PackInt4Args pt{plain, c->wq_tc, (int)d->n, (int)d->k, c->tiles_tc, c->kb_per_tile, gate_up, 1};
    CUDA_TRY_C(woq::launch_pack_int4(pt, stream));
  }

  woq::PackScaleArgs sa{};
  sa.scales = scales;
  sa.zps = zps;
  sa.sz = c->sz;
  sa.bad_zp = d_flag;
  sa.n = (int)d->n;
  sa.tiles = c->tiles;
  sa.groups = c->groups;
  sa.gate_up = gate_up;
  sa.transposed = transposed;
  sa.zp_transposed = (tmp_zp != nullptr) ? 0 : transposed;
  sa.scale_dtype = d->scale_dtype;
  sa.zp_dtype = zp_dtype;
  sa.default_zp = 8;  // symmetric INT4 is stored as q + 8
  sa.tc = 0;
  if (want_stream) CUDA_TRY_C(woq::launch_pack_scales(sa, stream));
  sa.sz = c->sz_tc;
  sa.tiles = c->tiles_tc;
  sa.tc = 1;
  if (want_tc) CUDA_TRY_C(woq::launch_pack_scales(sa, stream));

  if (bias) {
    CUDA_TRY_C(cudaMalloc(&c->bias, static_cast<size_t>(d->n) * sizeof(float)));
    convert_bias_kernel<<<(unsigned)((d->n + 255) / 256), 256, 0, stream>>>(bias, c->bias, (int)d->n,
                                                                          d->bias_dtype);
    woq::count_launch();
    CUDA_TRY_C(cudaGetLastError());
  }
  CUDA_TRY_C(cudaMemcpyAsync(c->h_flag, d_flag, sizeof(int), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY_C(cudaEventRecord(c->flag_ready, stream));
  c->flag_pending = 1;
  c->plain_scales = 0;
  if (!(d->layout_flags & WOQ_B200_LAYOUT_DEFER_CHECK) || tmp_plain || tmp_zp) {
    // look at the result now (the temporaries of a checkpoint format are freed below, which
    // waits for the device anyway)
    if (int rc = settle_prepack_flag(c)) return cleanup(rc);
  }
#undef CUDA_TRY_C
  c->magic = kMagic;
  *out = c;
  return cleanup(WOQ_B200_OK);
}

int woq_b200_ctx_destroy(woq_b200_ctx* c) {
  if (int rc = check_ctx(c)) return rc;
  c->magic = 0;
  if (c->d_flag) cudaFree(c->d_flag);
  if (c->h_flag) cudaFreeHost(c->h_flag);
  if (c->flag_ready) cudaEventDestroy(c->flag_ready);
  cudaFree(c->g_w);
  cudaFree(c->g_scales);
  cudaFree(c->g_zps);
  cudaFree(c->wq);
  cudaFree(c->sz);
  cudaFree(c->wq_tc);
  cudaFree(c->sz_tc);
  cudaFree(c->scale_f32);
  cudaFree(c->comp);
  cudaFree(c->bias);
  delete c;
  return WOQ_B200_OK;
}

int woq_b200_ctx_desc(const woq_b200_ctx* c, woq_b200_desc* out) {
  if (int rc = check_ctx(c)) return rc;
  if (!out) return fail(WOQ_B200_ERR_INVALID_ARG, "out is null");
  *out = c->desc;
  return WOQ_B200_OK;
}

size_t woq_b200_ctx_device_bytes(const woq_b200_ctx* c) {
  if (check_ctx(c)) return 0;
  return c->wq_bytes + c->sz_bytes + c->wq_tc_bytes + c->sz_tc_bytes;
}

int woq_b200_ctx_unpack(const woq_b200_ctx* c, void* qweight_plain, void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (!qweight_plain) return fail(WOQ_B200_ERR_INVALID_ARG, "output is null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (c->is_generic || c->is_i8block) {
    CUDA_TRY(cudaMemcpyAsync(qweight_plain, c->g_w, c->wq_bytes, cudaMemcpyDeviceToDevice, stream));
    return WOQ_B200_OK;
  }
  if (c->is_int8) {
    CUDA_TRY(woq::launch_unpack_int8(reinterpret_cast<const int8_t*>(c->wq), static_cast<int8_t*>(qweight_plain),
                                     (int)c->desc.n, (int)c->desc.k, c->gate_up, stream));
    return WOQ_B200_OK;
  }
  if (!c->wq)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "unpack needs the streaming layout (context was packed tensor-core only)");
  CUDA_TRY(woq::launch_unpack_int4(c->wq, static_cast<uint8_t*>(qweight_plain), (int)c->desc.n,
                                   (int)c->desc.k, c->tiles, c->kb_per_tile, c->gate_up, stream));
  return WOQ_B200_OK;
}

size_t woq_b200_workspace_bytes(const woq_b200_ctx* c, int64_t m) {
  if (check_ctx(c)) return 0;
  if (c->is_generic) return kWsHeaderBytes;  // the general route needs no scratch
  if (c->is_i8block) return i8block_ws(c, m < 1 ? 1 : m).total;
  if (c->is_int8) return int8_ws_layout(c, m < 1 ? 1 : m).total;
  // header + one pair of partial tiles per CTA of the largest grid
  size_t decode = woq::decode_int4_partial_bytes(2 * c->num_sms);
  int n_tok = static_cast<int>(m < 256 ? m : 256);
  n_tok = (n_tok + 15) / 16 * 16;
  if (n_tok < 16) n_tok = 16;
  size_t tc = woq::tc_partial_bytes(c->num_sms, n_tok);
  return kWsHeaderBytes + (decode > tc ? decode : tc);
}

static int run_decode(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx, int32_t fusion,
                      const void* o0, const void* o1, const int32_t* row_idx, const void* row_w,
                      void* y, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t stream,
                      const woq::CommParams* comm = nullptr, const float* bias_override = nullptr,
                      int64_t ldo_override = 0) {
  if (ws_bytes < woq_b200_workspace_bytes(c, m))
    return fail(WOQ_B200_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", ws_bytes,
                woq_b200_workspace_bytes(c, m));
  if (c->tiles > kMaxCounterTiles)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "N too large for the workspace header");
  if (int rc = settle_prepack_flag(c)) return rc;
  woq::DecodeParams p{};
  p.wq = c->wq;
  p.sz = c->sz;
  p.bias = c->bias;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.other0 = static_cast<const __nv_bfloat16*>(o0);
  p.other1 = static_cast<const __nv_bfloat16*>(o1);
  p.row_idx = row_idx;
  p.row_w = static_cast<const __nv_bfloat16*>(row_w);
  uint8_t* w8 = static_cast<uint8_t*>(ws);
  p.status = reinterpret_cast<int*>(w8);
  p.counters = reinterpret_cast<uint32_t*>(w8 + 256);
  p.partials = reinterpret_cast<float*>(w8 + kWsHeaderBytes);
  p.ldx = ldx;
  p.ldy = ldy;
  p.ldo = ldy;
  p.m = (int)m;
  p.n = (int)c->desc.n;
  p.n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? (int)(c->desc.n / 2) : (int)c->desc.n;
  p.k = (int)c->desc.k;
  p.tiles = c->tiles;
  p.kb_per_tile = c->kb_per_tile;
  p.kbpg_shift = c->kbpg_shift;
  p.groups = c->groups;
  p.fusion = fusion;
  p.gate_up = c->gate_up;
  // The scale-after-sum form only on request: it stays within the output tolerance for one
  // linear (mean relative deviation 1.2e-3 .. 1.7e-3 from the per-weight form, bar 2e-3) but
  // a product of two such linears (gate/up, woq_linear_silu followed by woq_linear_mul) does not.
  const bool after_sum = c->desc.kernel_hint == WOQ_B200_HINT_STREAM_FAST;
  p.exact = after_sum ? 0 : c->plain_scales ? 2 : 1;
#ifdef WOQ_B200_TIMELINE
  {
    const size_t need = woq_b200_workspace_bytes(c, m), extra = 8 * 1024 * 8 * sizeof(unsigned long long);
    p.stamps = ws_bytes >= need + extra ? reinterpret_cast<unsigned long long*>(w8 + (need + 255) / 256 * 256) : nullptr;
  }
#endif
  if (comm) p.comm = *comm;
  if (ldo_override) p.ldo = ldo_override;
  if (bias_override) p.bias = bias_override;
  const woq::DecodePlan plan = woq::decode_int4_plan((int)m, c->tiles, c->kb_per_tile, c->kb_per_group, c->num_sms);
  CUDA_TRY(woq::launch_decode_int4(p, plan, stream));
  woq::count_launch();
  return WOQ_B200_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// K-major tile map over a row-major [rows][ld] matrix of `elt_bytes`-byte elements:
// box = 128 bytes along K x `box_rows` rows, 128-byte swizzle, zero fill outside.
static int make_kmajor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols,
                           int64_t ld, int elt_bytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(WOQ_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elt_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elt_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elt_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(WOQ_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return WOQ_B200_OK;
}

static int run_tc(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx, int32_t fusion,
                  const void* o0, const void* o1, const int32_t* row_idx, const void* row_w,
                  void* y, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (ws_bytes < woq_b200_workspace_bytes(c, m))
    return fail(WOQ_B200_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", ws_bytes,
                woq_b200_workspace_bytes(c, m));
  if (c->tiles_tc > kMaxCounterTiles)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "N too large for the workspace header");
  if (int rc = settle_prepack_flag(c)) return rc;
  CUtensorMap xmap;
  const int64_t mt = m < 256 ? m : 256;
  int n_tok = static_cast<int>((mt + 15) / 16 * 16);
  if (int rc = make_kmajor_map(&xmap, x, m, c->desc.k, ldx, 2, n_tok)) return rc;
  uint8_t* w8 = static_cast<uint8_t*>(ws);
  const bool scatter = fusion == WOQ_B200_FUSE_SCALED_SCATTER_ADD;
  for (int64_t m0 = 0; m0 < m; m0 += 256) {
    const int64_t mm = m - m0 < 256 ? m - m0 : 256;
    woq::TcParams p{};
    p.wq = c->wq_tc;
    p.sz = c->sz_tc;
    p.bias = c->bias;
    p.y = scatter ? static_cast<__nv_bfloat16*>(y) : static_cast<__nv_bfloat16*>(y) + m0 * ldy;
    p.other0 = o0 ? static_cast<const __nv_bfloat16*>(o0) + m0 * ldy : nullptr;
    p.other1 = o1 ? static_cast<const __nv_bfloat16*>(o1) + m0 * ldy : nullptr;
    p.row_idx = row_idx ? row_idx + m0 : nullptr;
    p.row_w = row_w ? static_cast<const __nv_bfloat16*>(row_w) + m0 : nullptr;
    p.status = reinterpret_cast<int*>(w8);
    p.counters = reinterpret_cast<uint32_t*>(w8 + 256);
    p.partials = reinterpret_cast<float*>(w8 + kWsHeaderBytes);
    p.ldy = ldy;
    p.m = (int)mm;
    p.n = (int)c->desc.n;
    p.n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? (int)(c->desc.n / 2) : (int)c->desc.n;
    p.k = (int)c->desc.k;
    p.m0 = (int)m0;
    p.n_tok = n_tok;
    p.tiles = c->tiles_tc;
    p.kb_per_tile = c->kb_per_tile;
    p.kbpg_shift = c->kbpg_shift;
    p.groups = c->groups;
    p.fusion = fusion;
    p.gate_up = c->gate_up;
    const int grid = woq::tc_pick_grid(c->tiles_tc, c->kb_per_tile, c->num_sms);
    CUDA_TRY(woq::launch_int4_tc(p, xmap, grid, stream));
    woq::count_launch();
  }
  return WOQ_B200_OK;
}

// The tcgen05 int8 kernel, 256 tokens per launch, on activations that are already quantised:
// codes qa [m, K], scales sa [m], zero points zpa [m] (null for the symmetric modes).
static int run_int8_gemm(const woq_b200_ctx* c, const int8_t* qa, const float* sa, const int32_t* zpa, int64_t m,
                         int32_t fusion, const void* o0, const void* o1, void* y, int64_t ldy, int32_t* acc_out,
                         uint8_t* w8, size_t partial_off, cudaStream_t stream) {
  const int64_t k = c->desc.k;
  const int64_t mt = m < 256 ? m : 256;
  const int n_tok = static_cast<int>((mt + 15) / 16 * 16);
  CUtensorMap qamap;
  if (int rc = make_kmajor_map(&qamap, qa, m, k, k, 1, n_tok)) return rc;
  for (int64_t m0 = 0; m0 < m; m0 += 256) {
    const int64_t mm = m - m0 < 256 ? m - m0 : 256;
    woq::I8Params p{};
    p.wq = reinterpret_cast<const int8_t*>(c->wq);
    p.sw = c->scale_f32;
    p.sa = sa + m0;
    p.zpa = zpa ? zpa + m0 : nullptr;
    p.comp = c->comp;
    p.bias = c->bias;
    p.y = y ? static_cast<__nv_bfloat16*>(y) + m0 * ldy : nullptr;
    p.other0 = o0 ? static_cast<const __nv_bfloat16*>(o0) + m0 * ldy : nullptr;
    p.other1 = o1 ? static_cast<const __nv_bfloat16*>(o1) + m0 * ldy : nullptr;
    p.acc_out = acc_out ? acc_out + m0 * c->desc.n : nullptr;
    p.status = reinterpret_cast<int*>(w8);
    p.counters = reinterpret_cast<uint32_t*>(w8 + 256);
    p.partials = w8 + partial_off;
    p.ldy = ldy;
    p.m = (int)mm;
    p.n = (int)c->desc.n;
    p.n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? (int)(c->desc.n / 2) : (int)c->desc.n;
    p.m0 = (int)m0;
    p.n_tok = n_tok;
    p.tiles = c->tiles_tc;
    p.kc_per_tile = c->kc_per_tile;
    p.fusion = fusion;
    p.gate_up = c->gate_up;
    const int64_t total = static_cast<int64_t>(c->tiles_tc) * c->kc_per_tile;
    const int grid = static_cast<int>(total < c->num_sms ? total : c->num_sms);
    CUDA_TRY(woq::launch_int8_tc(p, qamap, grid, stream));
  }
  return WOQ_B200_OK;
}

// INT8 compute: quantise the activations per token, then the tcgen05 int8 kernel per 256 tokens
static int run_int8(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx, int32_t fusion,
                    const void* o0, const void* o1, void* y, int64_t ldy, int8_t* qa_out, float* sa_out,
                    int32_t* acc_out, void* ws, size_t ws_bytes, cudaStream_t stream) {
  const Int8Workspace L = int8_ws_layout(c, m);
  if (ws_bytes < L.total)
    return fail(WOQ_B200_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", ws_bytes, L.total);
  if (c->tiles_tc > kMaxCounterTiles)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "N too large for the workspace header");
  uint8_t* w8 = static_cast<uint8_t*>(ws);
  float* sa = reinterpret_cast<float*>(w8 + L.sa_off);
  int8_t* qa = reinterpret_cast<int8_t*>(w8 + L.qa_off);
  const int64_t k = c->desc.k;
  int32_t* zpa = reinterpret_cast<int32_t*>(w8 + L.zpa_off);
  const int mode = c->desc.act_quant_mode;
  const int asym = mode == WOQ_B200_ACT_PER_M || mode == WOQ_B200_ACT_PER_TENSOR;
  const int per_tensor = mode == WOQ_B200_ACT_PER_TENSOR || mode == WOQ_B200_ACT_PER_TENSOR_SYM;
  CUDA_TRY(woq::launch_quant_act(static_cast<const __nv_bfloat16*>(x), ldx, (int)m, (int)k, asym, per_tensor, qa, sa,
                                 zpa, reinterpret_cast<float*>(w8 + L.range_off), stream));
  if (qa_out) CUDA_TRY(cudaMemcpyAsync(qa_out, qa, static_cast<size_t>(m) * k, cudaMemcpyDeviceToDevice, stream));
  if (sa_out) CUDA_TRY(cudaMemcpyAsync(sa_out, sa, static_cast<size_t>(m) * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  if (!y && !acc_out) return WOQ_B200_OK;
  return run_int8_gemm(c, qa, sa, asym ? zpa : nullptr, m, fusion, o0, o1, y, ldy, acc_out, w8, L.partial_off, stream);
}

static bool use_tc_path(const woq_b200_ctx* c, int64_t m) {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("WOQ_B200_KERNEL_HINT");
    env = e ? atoi(e) : 0;
  }
  if (!c->wq_tc) return false;  // context packed for the streaming kernel only
  if (!c->wq) return true;      // context packed for the tensor-core kernel only
  const int hint = c->desc.kernel_hint ? c->desc.kernel_hint : env;
  if (hint == WOQ_B200_HINT_TENSOR_CORE) return true;
  if (hint == WOQ_B200_HINT_STREAM || hint == WOQ_B200_HINT_STREAM_FAST) return false;
  return m > 16;
}

int woq_b200_linear_any(const woq_b200_ctx* c, const void* x, int32_t io_dtype, int64_t m, int64_t ldx,
                        int32_t fusion, const void* const* others, int32_t n_others, void* y, int64_t ldy,
                        void* workspace, size_t workspace_bytes, void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (!c->is_generic) {
    if (io_dtype != WOQ_B200_T_BF16)
      return fail(WOQ_B200_ERR_UNSUPPORTED, "this context was packed for bf16 activations; create it with "
                  "WOQ_B200_LAYOUT_GENERIC to run it on fp32 or fp16 ones");
    return woq_b200_linear(c, x, m, ldx, fusion, others, n_others, y, ldy, workspace, workspace_bytes, stream_);
  }
  if (io_dtype != WOQ_B200_T_BF16 && io_dtype != WOQ_B200_T_F16 && io_dtype != WOQ_B200_T_F32)
    return fail(WOQ_B200_ERR_INVALID_ARG, "activations must be bf16, fp16 or fp32");
  if (m == 0) return WOQ_B200_OK;
  if (!x || !y || m < 0) return fail(WOQ_B200_ERR_INVALID_ARG, "x and y must be non-null, M non-negative");
  if (int rc = check_current_device(c)) return rc;
  if (ldx < c->desc.k || ldy < c->desc.n) return fail(WOQ_B200_ERR_INVALID_ARG, "ldx / ldy smaller than K / N");
  int need = 0;
  switch (fusion) {
    case WOQ_B200_FUSE_NONE: case WOQ_B200_FUSE_GELU_ERF: case WOQ_B200_FUSE_GELU_TANH:
    case WOQ_B200_FUSE_RELU: case WOQ_B200_FUSE_SILU: need = 0; break;
    case WOQ_B200_FUSE_ADD: case WOQ_B200_FUSE_MUL: need = 1; break;
    case WOQ_B200_FUSE_ADD_ADD: need = 2; break;
    case WOQ_B200_FUSE_SILU_MUL:
      return fail(WOQ_B200_ERR_UNSUPPORTED, "the general route has no fused silu*mul (use silu, then mul)");
    default: return fail(WOQ_B200_ERR_INVALID_ARG, "unexpected fusion type %#x", fusion);
  }
  if (n_others != need || (need > 0 && (!others || !others[0])) || (need > 1 && !others[1]))
    return fail(WOQ_B200_ERR_INVALID_ARG, "fusion %#x takes %d extra tensors, got %d", fusion, need, n_others);
  woq::GenericParams p{};
  fill_generic(c, &p);
  p.x = x;
  p.y = y;
  p.other0 = need > 0 ? others[0] : nullptr;
  p.other1 = need > 1 ? others[1] : nullptr;
  p.ldx = ldx;
  p.ldy = ldy;
  p.m = static_cast<int>(m);
  p.io_dtype = io_dtype;
  p.compute_dtype = generic_compute_dtype(c, io_dtype);
  p.fusion = fusion;
  // tokens in slabs that keep the grid's y dimension in range
  for (int64_t m0 = 0; m0 < m; m0 += 65535 * 8) {
    woq::GenericParams q = p;
    const size_t esz = io_dtype == WOQ_B200_T_F32 ? 4 : 2;
    q.m = static_cast<int>(m - m0 < 65535 * 8 ? m - m0 : 65535 * 8);
    q.x = static_cast<const uint8_t*>(x) + m0 * ldx * esz;
    q.y = static_cast<uint8_t*>(y) + m0 * ldy * esz;
    if (q.other0) q.other0 = static_cast<const uint8_t*>(p.other0) + m0 * ldy * esz;
    if (q.other1) q.other1 = static_cast<const uint8_t*>(p.other1) + m0 * ldy * esz;
    CUDA_TRY(woq::launch_generic(q, static_cast<cudaStream_t>(stream_)));
    woq::count_launch();
  }
  (void)workspace;
  (void)workspace_bytes;
  return WOQ_B200_OK;
}

int woq_b200_dump_dequant_f32(const woq_b200_ctx* c, int32_t compute_dtype, float* w_f32, void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (!c->is_generic) return fail(WOQ_B200_ERR_UNSUPPORTED, "general-route contexts only (see woq_b200_dump_dequant)");
  if (!w_f32) return fail(WOQ_B200_ERR_INVALID_ARG, "output is null");
  if (compute_dtype != WOQ_B200_T_BF16 && compute_dtype != WOQ_B200_T_F16 && compute_dtype != WOQ_B200_T_F32)
    return fail(WOQ_B200_ERR_INVALID_ARG, "compute dtype must be bf16, fp16 or fp32");
  woq::GenericParams p{};
  fill_generic(c, &p);
  p.compute_dtype = compute_dtype;
  CUDA_TRY(woq::launch_dump_generic(p, w_f32, static_cast<cudaStream_t>(stream_)));
  woq::count_launch();
  return WOQ_B200_OK;
}

int woq_b200_linear(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx, int32_t fusion,
                    const void* const* others, int32_t n_others, void* y, int64_t ldy,
                    void* workspace, size_t workspace_bytes, void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (c->is_generic)
    return woq_b200_linear_any(c, x, WOQ_B200_T_BF16, m, ldx, fusion, others, n_others, y, ldy, workspace,
                               workspace_bytes, stream_);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (m == 0) return WOQ_B200_OK;
  if (!x || !y || !workspace) return fail(WOQ_B200_ERR_INVALID_ARG, "x, y and workspace must be non-null");
  if (m < 0) return fail(WOQ_B200_ERR_INVALID_ARG, "negative M");
  if (int rc = check_current_device(c)) return rc;
  if (ldx < c->desc.k || (ldx % 8) != 0 || !aligned16(x))
    return fail(WOQ_B200_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx >= K and ldx %% 8 == 0");
  int need = 0;
  switch (fusion) {
    case WOQ_B200_FUSE_NONE: case WOQ_B200_FUSE_GELU_ERF: case WOQ_B200_FUSE_GELU_TANH:
    case WOQ_B200_FUSE_RELU: case WOQ_B200_FUSE_SILU: need = 0; break;
    case WOQ_B200_FUSE_ADD: case WOQ_B200_FUSE_MUL: need = 1; break;
    case WOQ_B200_FUSE_ADD_ADD: need = 2; break;
    case WOQ_B200_FUSE_SILU_MUL:
      if (!c->gate_up)
        return fail(WOQ_B200_ERR_INVALID_ARG, "silu_mul needs a context created with the gate/up layout");
      need = 0;
      break;
    default: return fail(WOQ_B200_ERR_INVALID_ARG, "unexpected fusion type %#x", fusion);
  }
  if (n_others != need || (need > 0 && !others))
    return fail(WOQ_B200_ERR_INVALID_ARG, "fusion %#x takes %d extra tensors, got %d", fusion, need, n_others);
  const void* o0 = need > 0 ? others[0] : nullptr;
  const void* o1 = need > 1 ? others[1] : nullptr;
  if ((need > 0 && !o0) || (need > 1 && !o1)) return fail(WOQ_B200_ERR_INVALID_ARG, "null extra tensor");
  const int64_t n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? c->desc.n / 2 : c->desc.n;
  if (ldy < n_out) return fail(WOQ_B200_ERR_INVALID_ARG, "ldy smaller than the output width");
  if (c->is_i8block)
    return run_i8block(c, x, m, ldx, fusion, o0, o1, y, ldy, nullptr, nullptr, nullptr, nullptr, workspace,
                       workspace_bytes, stream);
  if (c->is_int8)
    return run_int8(c, x, m, ldx, fusion, o0, o1, y, ldy, nullptr, nullptr, nullptr, workspace,
                    workspace_bytes, stream);
  if (use_tc_path(c, m))
    return run_tc(c, x, m, ldx, fusion, o0, o1, nullptr, nullptr, y, ldy, workspace, workspace_bytes,
                  stream);
  // tokens in slabs of 16 through the decode kernel
  for (int64_t m0 = 0; m0 < m; m0 += 16) {
    const int64_t mm = m - m0 < 16 ? m - m0 : 16;
    const __nv_bfloat16* xs = static_cast<const __nv_bfloat16*>(x) + m0 * ldx;
    __nv_bfloat16* ys = static_cast<__nv_bfloat16*>(y) + m0 * ldy;
    const void* s0 = o0 ? static_cast<const __nv_bfloat16*>(o0) + m0 * ldy : nullptr;
    const void* s1 = o1 ? static_cast<const __nv_bfloat16*>(o1) + m0 * ldy : nullptr;
    if (int rc = run_decode(c, xs, mm, ldx, fusion, s0, s1, nullptr, nullptr, ys, ldy, workspace,
                            workspace_bytes, stream))
      return rc;
  }
  return WOQ_B200_OK;
}

// ---- RMSNorm fused with the activation quantiser, and the linear on quantised activations ---
int woq_b200_rmsnorm_quant(const void* x, int64_t ldx, const void* gamma, float eps, int64_t m, int64_t k,
                           int32_t act_quant_mode, void* y, int64_t ldy, void* qa, void* sa, void* zpa,
                           void* stream_) {
  if (m == 0) return WOQ_B200_OK;
  if (!x || !gamma || !qa || !sa) return fail(WOQ_B200_ERR_INVALID_ARG, "x, gamma, qa and sa must be non-null");
  if (m < 0 || k <= 0 || (k % 16) != 0)
    return fail(WOQ_B200_ERR_INVALID_ARG, "woq_b200_rmsnorm_quant needs M >= 0 and K a positive multiple of 16");
  if (act_quant_mode != WOQ_B200_ACT_PER_M && act_quant_mode != WOQ_B200_ACT_PER_M_SYM)
    return fail(WOQ_B200_ERR_UNSUPPORTED,
                "woq_b200_rmsnorm_quant quantises per token (WOQ_B200_ACT_PER_M or _PER_M_SYM), got mode %d",
                act_quant_mode);
  const int asym = act_quant_mode == WOQ_B200_ACT_PER_M;
  if (asym && !zpa) return fail(WOQ_B200_ERR_INVALID_ARG, "the asymmetric mode writes zero points: zpa is null");
  if (ldx < k || (ldx % 8) != 0 || !aligned16(x) || !aligned16(gamma) || !aligned16(qa))
    return fail(WOQ_B200_ERR_INVALID_ARG, "x, gamma and qa must be 16-byte aligned, ldx >= K and ldx %% 8 == 0");
  if (y && (ldy < k || (ldy % 8) != 0 || !aligned16(y)))
    return fail(WOQ_B200_ERR_INVALID_ARG, "y must be 16-byte aligned with ldy >= K and ldy %% 8 == 0");
  CUDA_TRY(woq::launch_rmsnorm_quant(static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(gamma),
                                     eps, (int)m, (int)k, asym, static_cast<__nv_bfloat16*>(y), ldy,
                                     static_cast<int8_t*>(qa), static_cast<float*>(sa), static_cast<int32_t*>(zpa),
                                     static_cast<cudaStream_t>(stream_)));
  return WOQ_B200_OK;
}

int woq_b200_linear_prequant(const woq_b200_ctx* c, const void* qa, const void* sa, const void* zpa, int64_t m,
                             int32_t fusion, const void* const* others, int32_t n_others, void* y, int64_t ldy,
                             void* workspace, size_t workspace_bytes, void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (m == 0) return WOQ_B200_OK;
  if (!c->is_int8 || c->is_i8block || c->is_generic)
    return fail(WOQ_B200_ERR_UNSUPPORTED,
                "woq_b200_linear_prequant takes contexts on the tcgen05 INT8 route (INT8 weights, lowp INT8, "
                "one activation scale per token)");
  const int mode = c->desc.act_quant_mode;
  if (mode != WOQ_B200_ACT_PER_M && mode != WOQ_B200_ACT_PER_M_SYM)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "the context quantises activations in mode %d, not per token", mode);
  const bool asym = mode == WOQ_B200_ACT_PER_M;
  if (!qa || !sa || !y || !workspace || m < 0 || (asym && !zpa))
    return fail(WOQ_B200_ERR_INVALID_ARG, "qa, sa, y and workspace must be non-null (zpa too for the asymmetric mode)");
  if (!asym && zpa) return fail(WOQ_B200_ERR_INVALID_ARG, "the context's mode is symmetric: zpa must be null");
  if (!aligned16(qa)) return fail(WOQ_B200_ERR_INVALID_ARG, "qa must be 16-byte aligned");
  if (int rc = check_current_device(c)) return rc;
  int need = 0;
  switch (fusion) {
    case WOQ_B200_FUSE_NONE: case WOQ_B200_FUSE_GELU_ERF: case WOQ_B200_FUSE_GELU_TANH:
    case WOQ_B200_FUSE_RELU: case WOQ_B200_FUSE_SILU: need = 0; break;
    case WOQ_B200_FUSE_ADD: case WOQ_B200_FUSE_MUL: need = 1; break;
    case WOQ_B200_FUSE_ADD_ADD: need = 2; break;
    case WOQ_B200_FUSE_SILU_MUL:
      if (!c->gate_up)
        return fail(WOQ_B200_ERR_INVALID_ARG, "silu_mul needs a context created with the gate/up layout");
      break;
    default: return fail(WOQ_B200_ERR_INVALID_ARG, "unexpected fusion type %#x", fusion);
  }
  if (n_others != need || (need > 0 && !others))
    return fail(WOQ_B200_ERR_INVALID_ARG, "fusion %#x takes %d extra tensors, got %d", fusion, need, n_others);
  const void* o0 = need > 0 ? others[0] : nullptr;
  const void* o1 = need > 1 ? others[1] : nullptr;
  if ((need > 0 && !o0) || (need > 1 && !o1)) return fail(WOQ_B200_ERR_INVALID_ARG, "null extra tensor");
  const int64_t n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? c->desc.n / 2 : c->desc.n;
  if (ldy < n_out) return fail(WOQ_B200_ERR_INVALID_ARG, "ldy smaller than the output width");
  const Int8Workspace L = int8_ws_layout(c, m);
  if (workspace_bytes < L.total)
    return fail(WOQ_B200_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", workspace_bytes, L.total);
  if (c->tiles_tc > kMaxCounterTiles)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "N too large for the workspace header");
  return run_int8_gemm(c, static_cast<const int8_t*>(qa), static_cast<const float*>(sa),
                       static_cast<const int32_t*>(zpa), m, fusion, o0, o1, y, ldy, nullptr,
                       static_cast<uint8_t*>(workspace), L.partial_off, static_cast<cudaStream_t>(stream_));
}

// ---- tensor-parallel exchange (one node, CUDA IPC) ---------------------------------------
struct woq_b200_comm {
  uint64_t magic;
  int rank, world, device;
  int64_t ar_n;         // row length of an all-reduce slot (multiple of 64)
  size_t gather_off, gather_bytes, total_bytes;
  uint8_t* local;       // this rank's buffer (cudaMalloc)
  uint8_t* peer[woq::kCommMaxRanks];
  bool connected;
  int num_sms;
  int* status;          // status word of the fence kernel (inside `local`)
  woq::CommPending pending;  // the all-gather of the latest launch, if it was one
};

static int check_comm(const woq_b200_comm* cm) {
  if (!cm) return fail(WOQ_B200_ERR_INVALID_ARG, "comm is null");
  if (cm->magic != kMagic + 1) return fail(WOQ_B200_ERR_BAD_HANDLE, "comm magic mismatch");
  return WOQ_B200_OK;
}

int woq_b200_comm_create(int32_t rank, int32_t world, int64_t max_n, size_t gather_bytes,
                         woq_b200_comm** out) {
  if (!out) return fail(WOQ_B200_ERR_INVALID_ARG, "out is null");
  if (world < 1 || world > woq::kCommMaxRanks || rank < 0 || rank >= world)
    return fail(WOQ_B200_ERR_INVALID_ARG, "rank %d of %d: at most %d ranks", rank, world, woq::kCommMaxRanks);
  if (max_n < 1 || max_n > static_cast<int64_t>(woq::kCommMaxTiles) * woq::kTileN)
    return fail(WOQ_B200_ERR_INVALID_ARG, "max_n out of range");
  woq_b200_comm* cm = new woq_b200_comm();
  cm->rank = rank;
  cm->world = world;
  cm->ar_n = (max_n + woq::kTileN - 1) / woq::kTileN * woq::kTileN;
  // {2 x bf16, stamp} words: [4 sets][8 sources][ar_n / 64 tiles][16 tokens][32 lanes] x 8 B
  const size_t ar_bytes = static_cast<size_t>(cm->ar_n) * 512 * woq::kCommSets;
  cm->gather_off = (woq::kCommCtlBytes + ar_bytes + 255) / 256 * 256;
  cm->gather_bytes = (gather_bytes + 255) / 256 * 256;
  cm->total_bytes = cm->gather_off + cm->gather_bytes;
  cm->connected = false;
  for (auto& q : cm->peer) q = nullptr;
  cm->pending = woq::CommPending{};
  cudaError_t e = cudaGetDevice(&cm->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&cm->num_sms, cudaDevAttrMultiProcessorCount, cm->device);
  if (e == cudaSuccess) e = cudaMalloc(&cm->local, cm->total_bytes);
  if (e == cudaSuccess) e = cudaMemset(cm->local, 0, cm->total_bytes);
  if (e != cudaSuccess) {
    delete cm;
    return fail(WOQ_B200_ERR_CUDA, "comm buffer: %s", cudaGetErrorString(e));
  }
  cm->peer[rank] = cm->local;
  cm->status = reinterpret_cast<int*>(cm->local + 2048);  // inside the control block, never a control word
  cm->magic = kMagic + 1;
  *out = cm;
  return WOQ_B200_OK;
}

int woq_b200_comm_export(const woq_b200_comm* cm, void* handle) {
  if (int rc = check_comm(cm)) return rc;
  static_assert(sizeof(cudaIpcMemHandle_t) == WOQ_B200_COMM_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  CUDA_TRY(cudaIpcGetMemHandle(&h, cm->local));
  memcpy(handle, &h, sizeof(h));
  return WOQ_B200_OK;
}

int woq_b200_comm_connect(woq_b200_comm* cm, const void* handles) {
  if (int rc = check_comm(cm)) return rc;
  if (cm->connected) return fail(WOQ_B200_ERR_INVALID_ARG, "comm is already connected");
  for (int q = 0; q < cm->world; ++q) {
    if (q == cm->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + q * sizeof(h), sizeof(h));
    void* ptr = nullptr;
    CUDA_TRY(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    cm->peer[q] = static_cast<uint8_t*>(ptr);
  }
  cm->connected = true;
  return WOQ_B200_OK;
}

void* woq_b200_comm_gather_ptr(const woq_b200_comm* cm) {
  if (check_comm(cm)) return nullptr;
  return cm->local + cm->gather_off;
}

int woq_b200_comm_destroy(woq_b200_comm* cm) {
  if (int rc = check_comm(cm)) return rc;
  cm->magic = 0;
  for (int q = 0; q < cm->world; ++q)
    if (q != cm->rank && cm->peer[q]) cudaIpcCloseMemHandle(cm->peer[q]);
  cudaFree(cm->local);
  delete cm;
  return WOQ_B200_OK;
}

static int comm_params(const woq_b200_ctx* c, const woq_b200_comm* cm, int64_t m, woq::CommParams* cp) {
  if (int rc = check_ctx(c)) return rc;
  if (int rc = check_comm(cm)) return rc;
  if (!cm->connected && cm->world > 1) return fail(WOQ_B200_ERR_INVALID_ARG, "comm is not connected");
  if (c->is_int8 || c->is_generic || c->is_i8block || m > 16 || m < 1)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "the fused exchange covers INT4 weights with bf16 compute and 1..16 tokens");
  if (!c->wq) return fail(WOQ_B200_ERR_UNSUPPORTED, "context was packed without the streaming layout");
  if (c->tiles > woq::kCommMaxTiles) return fail(WOQ_B200_ERR_UNSUPPORTED, "N too large for the stamp table");
  for (int q = 0; q < woq::kCommMaxRanks; ++q) cp->peer[q] = cm->peer[q];
  cp->world = cm->world;
  cp->rank = cm->rank;
  cp->ar_n = cm->ar_n;
  cp->pend = cm->pending;  // this launch receives it; the caller records its own afterwards
  return WOQ_B200_OK;
}

int woq_b200_linear_allreduce(const woq_b200_ctx* c, const woq_b200_comm* cm, const void* x, int64_t m,
                              int64_t ldx, int32_t fusion, const void* const* others,
                              int32_t n_others, const float* bias, void* y, int64_t ldy,
                              void* workspace, size_t workspace_bytes, void* stream_) {
  woq::CommParams cp{};
  if (m == 0) return WOQ_B200_OK;
  if (int rc = comm_params(c, cm, m, &cp)) return rc;
  cp.mode = woq::kCommAllReduce;
  if (c->bias) return fail(WOQ_B200_ERR_INVALID_ARG, "a row-parallel context must be packed without bias (it is added after the reduction)");
  if (c->desc.n > cm->ar_n) return fail(WOQ_B200_ERR_INVALID_ARG, "N exceeds the comm's max_n");
  int need = fusion == WOQ_B200_FUSE_ADD || fusion == WOQ_B200_FUSE_MUL ? 1 : fusion == WOQ_B200_FUSE_ADD_ADD ? 2 : 0;
  if (fusion == WOQ_B200_FUSE_SILU_MUL || fusion == WOQ_B200_FUSE_SCALED_SCATTER_ADD)
    return fail(WOQ_B200_ERR_INVALID_ARG, "fusion %#x cannot follow a reduction over K shards", fusion);
  if (n_others != need || (need > 0 && !others)) return fail(WOQ_B200_ERR_INVALID_ARG, "fusion %#x takes %d extra tensors", fusion, need);
  if (!x || !y || !workspace) return fail(WOQ_B200_ERR_INVALID_ARG, "x, y and workspace must be non-null");
  if (ldx < c->desc.k || (ldx % 8) != 0 || !aligned16(x))
    return fail(WOQ_B200_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx >= K and ldx %% 8 == 0");
  if (ldy < c->desc.n) return fail(WOQ_B200_ERR_INVALID_ARG, "ldy smaller than the output width");
  const int rc = run_decode(c, x, m, ldx, fusion, need > 0 ? others[0] : nullptr, need > 1 ? others[1] : nullptr,
                            nullptr, nullptr, y, ldy, workspace, workspace_bytes, static_cast<cudaStream_t>(stream_),
                            &cp, bias);
  if (rc == WOQ_B200_OK) const_cast<woq_b200_comm*>(cm)->pending = woq::CommPending{};  // received by this launch
  return rc;
}

int woq_b200_linear_allgather(const woq_b200_ctx* c, const woq_b200_comm* cm, const void* x, int64_t m,
                              int64_t ldx, int32_t fusion, const void* const* others,
                              int32_t n_others, size_t gather_offset, void* workspace,
                              size_t workspace_bytes, void* stream_) {
  woq::CommParams cp{};
  if (m == 0) return WOQ_B200_OK;
  if (int rc = comm_params(c, cm, m, &cp)) return rc;
  cp.mode = woq::kCommAllGather;
  if (fusion == WOQ_B200_FUSE_SCALED_SCATTER_ADD) return fail(WOQ_B200_ERR_INVALID_ARG, "scatter cannot be gathered");
  if (fusion == WOQ_B200_FUSE_SILU_MUL && !c->gate_up)
    return fail(WOQ_B200_ERR_INVALID_ARG, "silu_mul needs a context created with the gate/up layout");
  int need = fusion == WOQ_B200_FUSE_ADD || fusion == WOQ_B200_FUSE_MUL ? 1 : fusion == WOQ_B200_FUSE_ADD_ADD ? 2 : 0;
  if (n_others != need || (need > 0 && !others)) return fail(WOQ_B200_ERR_INVALID_ARG, "fusion %#x takes %d extra tensors", fusion, need);
  const int64_t n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? c->desc.n / 2 : c->desc.n;
  const size_t bytes = static_cast<size_t>(m) * n_out * cm->world * 2;
  if ((gather_offset % 16) != 0 || gather_offset + bytes > cm->gather_bytes)
    return fail(WOQ_B200_ERR_INVALID_ARG, "gathered tensor [%lld, %lld] at offset %zu does not fit the gather area (%zu bytes)",
                (long long)m, (long long)(n_out * cm->world), gather_offset, cm->gather_bytes);
  if (!x || !workspace) return fail(WOQ_B200_ERR_INVALID_ARG, "x and workspace must be non-null");
  if (ldx < c->desc.k || (ldx % 8) != 0 || !aligned16(x))
    return fail(WOQ_B200_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx >= K and ldx %% 8 == 0");
  if (c->desc.n > cm->ar_n) return fail(WOQ_B200_ERR_INVALID_ARG, "N exceeds the comm's max_n");
  // y = this rank's column block of the gathered tensor; `others` are local [M, N_out] tensors
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(cm->local + cm->gather_off + gather_offset) +
                     static_cast<int64_t>(cm->rank) * n_out;
  const int rc = run_decode(c, x, m, ldx, fusion, need > 0 ? others[0] : nullptr, need > 1 ? others[1] : nullptr,
                            nullptr, nullptr, y, n_out * cm->world, workspace, workspace_bytes,
                            static_cast<cudaStream_t>(stream_), &cp, nullptr, n_out);
  if (rc == WOQ_B200_OK) {
    // the other ranks' column blocks are received by the next launch on this comm
    woq::CommPending g{};
    g.dst = reinterpret_cast<__nv_bfloat16*>(cm->local + cm->gather_off + gather_offset);
    g.m = static_cast<int>(m);
    g.n = static_cast<int>(c->desc.n);
    g.n_out = static_cast<int>(n_out);
    g.tiles = c->tiles;
    g.gate_up = c->gate_up;
    g.pair = fusion != WOQ_B200_FUSE_SILU_MUL;
    const_cast<woq_b200_comm*>(cm)->pending = cm->world > 1 ? g : woq::CommPending{};
  }
  return rc;
}

int woq_b200_comm_fence(woq_b200_comm* cm, void* stream_) {
  if (int rc = check_comm(cm)) return rc;
  if (!cm->pending.dst || cm->world == 1) {
    cm->pending = woq::CommPending{};
    return WOQ_B200_OK;
  }
  woq::CommParams cp{};
  for (int q = 0; q < woq::kCommMaxRanks; ++q) cp.peer[q] = cm->peer[q];
  cp.world = cm->world;
  cp.rank = cm->rank;
  cp.ar_n = cm->ar_n;
  cp.pend = cm->pending;
  CUDA_TRY(woq::launch_comm_fence(cp, cm->status, cm->num_sms, static_cast<cudaStream_t>(stream_)));
  woq::count_launch();
  cm->pending = woq::CommPending{};
  return WOQ_B200_OK;
}

int woq_b200_comm_status(woq_b200_comm* cm, void* stream_) {
  if (int rc = check_comm(cm)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int h = 0;
  CUDA_TRY(cudaMemcpyAsync(&h, cm->status, sizeof(int), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  if (h != 0) {
    CUDA_TRY(cudaMemsetAsync(cm->status, 0, sizeof(int), stream));
    return fail(WOQ_B200_ERR_DEVICE_WAIT, "woq_b200_comm_fence gave up waiting for a peer (code %d)", h);
  }
  return WOQ_B200_OK;
}

int woq_b200_linear_scatter(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx,
                            const int32_t* row_idx, const void* row_weight, void* out,
                            int64_t ld_out, void* workspace, size_t workspace_bytes,
                            void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (m == 0) return WOQ_B200_OK;
  if (!x || !out || !workspace || !row_idx || !row_weight)
    return fail(WOQ_B200_ERR_INVALID_ARG, "null argument");
  if (ldx < c->desc.k || (ldx % 8) != 0 || !aligned16(x))
    return fail(WOQ_B200_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx >= K and ldx %% 8 == 0");
  if (ld_out < c->desc.n) return fail(WOQ_B200_ERR_INVALID_ARG, "ld_out smaller than N");
  if (c->is_int8 || c->is_generic || c->is_i8block)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "scatter epilogue is built for INT4 bf16 contexts");
  if (use_tc_path(c, m))
    return run_tc(c, x, m, ldx, WOQ_B200_FUSE_SCALED_SCATTER_ADD, nullptr, nullptr, row_idx, row_weight,
                  out, ld_out, workspace, workspace_bytes, stream);
  for (int64_t m0 = 0; m0 < m; m0 += 16) {
    const int64_t mm = m - m0 < 16 ? m - m0 : 16;
    const __nv_bfloat16* xs = static_cast<const __nv_bfloat16*>(x) + m0 * ldx;
    if (int rc = run_decode(c, xs, mm, ldx, WOQ_B200_FUSE_SCALED_SCATTER_ADD, nullptr, nullptr,
                            row_idx + m0, static_cast<const __nv_bfloat16*>(row_weight) + m0, out,
                            ld_out, workspace, workspace_bytes, stream))
      return rc;
  }
  return WOQ_B200_OK;
}

size_t woq_b200_moe_workspace_bytes(const woq_b200_ctx* w13, const woq_b200_ctx* w2, int64_t tokens) {
  if (check_ctx(w13) || check_ctx(w2) || tokens < 0) return 0;
  size_t a = woq_b200_workspace_bytes(w13, tokens), b = woq_b200_workspace_bytes(w2, tokens);
  size_t lin = ((a > b ? a : b) + 1023) / 1024 * 1024;
  return lin + static_cast<size_t>(tokens) * (w13->desc.k + w13->desc.n / 2) * 2 + 2048;
}

int woq_b200_moe_expert(const woq_b200_ctx* w13, const woq_b200_ctx* w2, const void* hidden, int64_t ldh,
                        const int32_t* token_idx, const void* token_weight, int64_t tokens, void* out,
                        int64_t ld_out, void* workspace, size_t workspace_bytes, void* stream_) {
  if (int rc = check_ctx(w13)) return rc;
  if (int rc = check_ctx(w2)) return rc;
  if (tokens == 0) return WOQ_B200_OK;
  if (!hidden || !token_idx || !token_weight || !out || !workspace || tokens < 0)
    return fail(WOQ_B200_ERR_INVALID_ARG, "null or negative argument");
  if (!w13->gate_up) return fail(WOQ_B200_ERR_INVALID_ARG, "w13 must be packed with the gate/up layout");
  if (w13->desc.n / 2 != w2->desc.k || w2->desc.n > ld_out || (w13->desc.k % 8) != 0)
    return fail(WOQ_B200_ERR_INVALID_ARG, "expert shapes do not chain (w13 %lldx%lld, w2 %lldx%lld)",
                (long long)w13->desc.n, (long long)w13->desc.k, (long long)w2->desc.n, (long long)w2->desc.k);
  const size_t need = woq_b200_moe_workspace_bytes(w13, w2, tokens);
  if (workspace_bytes < need)
    return fail(WOQ_B200_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", workspace_bytes, need);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  size_t a = woq_b200_workspace_bytes(w13, tokens), b = woq_b200_workspace_bytes(w2, tokens);
  const size_t lin = ((a > b ? a : b) + 1023) / 1024 * 1024;
  uint8_t* w8 = static_cast<uint8_t*>(workspace);
  __nv_bfloat16* xg = reinterpret_cast<__nv_bfloat16*>(w8 + lin);
  __nv_bfloat16* act = xg + tokens * w13->desc.k;
  act = reinterpret_cast<__nv_bfloat16*>((reinterpret_cast<uintptr_t>(act) + 1023) / 1024 * 1024);
  CUDA_TRY(woq::launch_gather_rows(static_cast<const __nv_bfloat16*>(hidden), ldh, token_idx, xg, tokens,
                                   (int)w13->desc.k, stream));
  if (int rc = woq_b200_linear(w13, xg, tokens, w13->desc.k, WOQ_B200_FUSE_SILU_MUL, nullptr, 0, act,
                               w13->desc.n / 2, workspace, lin, stream_))
    return rc;
  return woq_b200_linear_scatter(w2, act, tokens, w2->desc.k, token_idx, token_weight, out, ld_out, workspace,
                                 lin, stream_);
}

int woq_b200_dump_dequant(const woq_b200_ctx* c, void* w_bf16, void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (!w_bf16) return fail(WOQ_B200_ERR_INVALID_ARG, "output is null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (c->is_int8 || c->is_i8block)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "the INT8 compute path never dequantises its weights");
  if (c->is_generic)
    return fail(WOQ_B200_ERR_UNSUPPORTED, "general-route context: use woq_b200_dump_dequant_f32");
  if (c->wq_tc) {
    // the routine the tensor-core kernel uses for its tiles
    CUDA_TRY(woq::launch_dump_dequant_int4_tc(c->wq_tc, c->sz_tc, static_cast<__nv_bfloat16*>(w_bf16),
                                              (int)c->desc.n, (int)c->desc.k, c->tiles_tc,
                                              c->kb_per_tile, c->kbpg_shift, c->groups, c->gate_up,
                                              stream));
  } else {
    CUDA_TRY(woq::launch_dump_dequant_int4(c->wq, c->sz, static_cast<__nv_bfloat16*>(w_bf16),
                                           (int)c->desc.n, (int)c->desc.k, c->tiles, c->kb_per_tile,
                                           c->kb_per_group, c->groups, c->gate_up, stream));
  }
  return WOQ_B200_OK;
}

int woq_b200_int8_internals(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx, int8_t* qa,
                            float* sa, int32_t* acc, void* workspace, size_t workspace_bytes,
                            void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (!c->is_int8) return fail(WOQ_B200_ERR_INVALID_ARG, "context does not use INT8 compute");
  if (m <= 0 || !x || !workspace) return fail(WOQ_B200_ERR_INVALID_ARG, "bad arguments");
  if (ldx < c->desc.k || (ldx % 8) != 0 || !aligned16(x))
    return fail(WOQ_B200_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx >= K and ldx %% 8 == 0");
  return run_int8(c, x, m, ldx, WOQ_B200_FUSE_NONE, nullptr, nullptr, nullptr, c->desc.n, qa, sa, acc,
                  workspace, workspace_bytes, static_cast<cudaStream_t>(stream_));
}

int woq_b200_int8_block_internals(const woq_b200_ctx* c, const void* x, int64_t m, int64_t ldx, uint8_t* qa,
                                  float* sa, int32_t* zpa, int32_t* acc, void* workspace, size_t workspace_bytes,
                                  void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (!c->is_i8block) return fail(WOQ_B200_ERR_INVALID_ARG, "context does not use INT8 compute with K blocks");
  if (m <= 0 || !x || !workspace) return fail(WOQ_B200_ERR_INVALID_ARG, "bad arguments");
  if (ldx < c->desc.k || (ldx % 8) != 0 || !aligned16(x))
    return fail(WOQ_B200_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx >= K and ldx %% 8 == 0");
  return run_i8block(c, x, m, ldx, WOQ_B200_FUSE_NONE, nullptr, nullptr, nullptr, c->desc.n, qa, sa, zpa, acc,
                     workspace, workspace_bytes, static_cast<cudaStream_t>(stream_));
}

int woq_b200_ctx_route(const woq_b200_ctx* c) {
  if (check_ctx(c)) return -1;
  if (c->is_i8block) return WOQ_B200_ROUTE_INT8_BLOCK;
  if (c->is_generic) return WOQ_B200_ROUTE_GENERAL;
  if (c->is_int8) return WOQ_B200_ROUTE_INT8;
  return WOQ_B200_ROUTE_INT4_BF16;
}

int woq_b200_int8_block_size(const woq_b200_ctx* c) {
  if (check_ctx(c) || !c->is_i8block) return 0;
  return c->kb;
}

int woq_b200_int8_zero_points(const woq_b200_ctx* c, int64_t m, int32_t* zp, const void* workspace,
                              size_t workspace_bytes, void* stream_) {
  if (int rc = check_ctx(c)) return rc;
  if (!c->is_int8) return fail(WOQ_B200_ERR_INVALID_ARG, "context does not use INT8 compute");
  if (!zp || !workspace || m < 1) return fail(WOQ_B200_ERR_INVALID_ARG, "null pointer or no tokens");
  const Int8Workspace L = int8_ws_layout(c, m);
  if (workspace_bytes < L.total)
    return fail(WOQ_B200_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", workspace_bytes, L.total);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int mode = c->desc.act_quant_mode;
  if (mode == WOQ_B200_ACT_PER_M || mode == WOQ_B200_ACT_PER_TENSOR) {
    CUDA_TRY(cudaMemcpyAsync(zp, static_cast<const uint8_t*>(workspace) + L.zpa_off,
                             static_cast<size_t>(m) * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream));
  } else {
    CUDA_TRY(cudaMemsetAsync(zp, 0, static_cast<size_t>(m) * sizeof(int32_t), stream));
  }
  return WOQ_B200_OK;
}

int woq_b200_decode_plan(const woq_b200_ctx* c, int64_t m, int32_t* out) {
  if (int rc = check_ctx(c)) return rc;
  if (!out || m < 1 || m > 16 || c->is_int8 || c->is_generic || c->is_i8block || !c->wq)
    return fail(WOQ_B200_ERR_INVALID_ARG, "decode plan: INT4 context with the streaming layout, 1..16 tokens");
  const woq::DecodePlan plan = woq::decode_int4_plan((int)m, c->tiles, c->kb_per_tile, c->kb_per_group, c->num_sms);
  out[0] = plan.grid;
  out[1] = plan.cluster;
  out[2] = plan.kpw;
  out[3] = plan.smem_budget;
  return WOQ_B200_OK;
}

int woq_b200_tc_plan(int32_t n_tok, int32_t* out) {
  if (!out || n_tok < 16 || n_tok > 256 || (n_tok & 15))
    return fail(WOQ_B200_ERR_INVALID_ARG, "tensor-core plan: token columns 16..256, a multiple of 16");
  woq::TcParams p{};
  p.n_tok = n_tok;
  const size_t smem = woq::tc_plan(p);
  if (smem == 0) return fail(WOQ_B200_ERR_UNSUPPORTED, "no pipeline shape for %d token columns", (int)n_tok);
  out[0] = p.kbs;
  out[1] = p.stages;
  out[2] = p.w_ring;
  out[3] = p.a_col0;
  out[4] = static_cast<int32_t>(smem);
  return WOQ_B200_OK;
}

int woq_b200_workspace_status(void* workspace, void* stream_) {
  if (!workspace) return fail(WOQ_B200_ERR_INVALID_ARG, "workspace is null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int h = 0;
  CUDA_TRY(cudaMemcpyAsync(&h, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  if (h != 0) {
    // a kernel that gave up may have left arrival counters behind: the whole header starts over
    CUDA_TRY(cudaMemsetAsync(workspace, 0, kWsHeaderBytes, stream));
    return fail(WOQ_B200_ERR_DEVICE_WAIT, "a bounded in-kernel wait gave up (code %d)", h);
  }
  return WOQ_B200_OK;
}

}  // extern "C"
