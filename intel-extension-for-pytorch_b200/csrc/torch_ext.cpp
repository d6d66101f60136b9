// PyTorch operator registration for the WOQ linear path, CUDA dispatch key.
//
// Mirrors the reference's op surface for this path so that its Python modules work unchanged:
//   torch_ipex::{ipex_woq_linear, woq_linear_gelu, woq_linear_new_gelu, woq_linear_relu,
//                woq_linear_silu, woq_linear_add, woq_linear_add_add, woq_linear_mul, woq_linear}
//       (reference: csrc/cpu/aten/Linear.cpp:1025-1108)
//   ipex_prepack::{weight_only_qlinear_prepack, weight_only_qlinear_prepack_int4,
//                  woq_linear_pack_weight, woq_linear_unpack_weight} and the class ipex_prepack.WoqLinearOpContext
//       (reference: csrc/cpu/jit/cpu/kernels/RegisterOpContextClass.cpp:127-222)
// plus torch_ipex::woq_linear_silu_mul (the reference's two-op gate/up composition as one op).
// Everything numeric happens behind the C ABI of libwoq_b200.so; this file only converts
// between tensors and pointers.  A missing CUDA device or library is an error, never a
// fallback.
#include <ATen/ATen.h>
#include <ATen/autocast_mode.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/custom_class.h>
#include <torch/library.h>

#include <map>
#include <mutex>

#include "../../include/woq_b200.h"

namespace {

constexpr int64_t kHandleMagic = 0x574f5148414e444cll;  // "WOQHANDL"
constexpr int64_t kGateUpStateBit = 0x100;                // pickled weight_dtype of a gate/up context

int dtype_code(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return WOQ_B200_T_F32;
    case at::kHalf: return WOQ_B200_T_F16;
    case at::kBFloat16: return WOQ_B200_T_BF16;
    case at::kByte: return WOQ_B200_T_U8;
    case at::kChar: return WOQ_B200_T_S8;
    default: TORCH_CHECK(false, "WOQ: unsupported tensor dtype ", t.scalar_type());
  }
}

#define WOQ_CHECK(expr)                                                       \
  do {                                                                        \
    int rc__ = (expr);                                                        \
    TORCH_CHECK(rc__ == WOQ_B200_OK, "WOQ: ", woq_b200_last_error(), " (status ", rc__, ")"); \
  } while (0)

// One zeroed workspace per (device, stream); grows on demand.  Calls on one stream are ordered,
// which is what a shared workspace needs.
std::mutex g_ws_mu;
std::map<std::pair<int, cudaStream_t>, at::Tensor> g_ws_pool;

at::Tensor& workspace_for(c10::DeviceIndex dev, cudaStream_t stream, size_t bytes) {
  // the same (device, stream) as the previous call of this thread: no lock, no look-up
  thread_local int last_dev = -1;
  thread_local cudaStream_t last_stream = nullptr;
  thread_local at::Tensor* last = nullptr;
  if (last && last_dev == dev && last_stream == stream && static_cast<size_t>(last->numel()) >= bytes) return *last;
  std::lock_guard<std::mutex> lock(g_ws_mu);
  auto& t = g_ws_pool[{dev, stream}];
  if (!t.defined() || static_cast<size_t>(t.numel()) < bytes) {
    t = at::zeros({static_cast<int64_t>(bytes)},
                  at::TensorOptions().dtype(at::kByte).device(at::Device(at::kCUDA, dev)));
  }
  last_dev = dev;
  last_stream = stream;
  last = &t;  // std::map never moves its elements
  return t;
}

// Synchronises every stream that has run a WOQ op and raises if a kernel gave up one of its
// bounded waits (its output is then not valid).  The ops themselves never synchronise.
void woq_check_status() {
  std::lock_guard<std::mutex> lock(g_ws_mu);
  for (auto& kv : g_ws_pool) {
    if (!kv.second.defined()) continue;
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(kv.first.first));
    WOQ_CHECK(woq_b200_workspace_status(kv.second.data_ptr(), kv.first.second));
  }
}

// plain INT4 weight [N, K/2] (k even in the low nibble) with its input channels re-ordered
at::Tensor shuffle_int4_columns(const at::Tensor& w, const at::Tensor& order) {
  auto q = at::stack({w.bitwise_and(15), w.bitwise_right_shift(4)}, 2).reshape({w.size(0), -1});
  q = q.index_select(1, order);
  auto pairs = q.reshape({w.size(0), -1, 2});
  return pairs.select(2, 0).bitwise_or(pairs.select(2, 1).bitwise_left_shift(4)).contiguous();
}

struct WoqLinearOpContext : torch::CustomClassHolder {
  int64_t magic = kHandleMagic;
  woq_b200_ctx* ctx = nullptr;
  // INT4: `ctx` keeps the streaming tiling only (M <= 16); the tensor-core tiling is packed into
  // a second context the first time a call brings more than 16 tokens, so that a model that only
  // decodes holds one copy of its weights.
  woq_b200_ctx* ctx_tc = nullptr;
  // lowp NONE computes in the activation's dtype: fp32 / fp16 activations run on a general-route
  // copy of the layer, packed the first time such a call arrives
  woq_b200_ctx* ctx_gen = nullptr;
  std::mutex tc_mu;
  // constructor arguments, kept so that the context can be pickled in a layout-independent way
  int64_t weight_dtype, group_size, lowp_mode, act_quant_mode;
  bool cache_weight_for_large_batch;
  std::vector<int64_t> weight_shape;  // [N, K]
  at::Tensor scales, zero_points, bias, g_idx;
  at::Tensor perm, inv_perm;  // act-order: input channels sorted by group / back (int64 on the device)
  c10::optional<int64_t> batch_size;
  c10::DeviceIndex device = 0;
  int layout_flags = 0;

  ~WoqLinearOpContext() override {
    if (ctx) woq_b200_ctx_destroy(ctx);
    if (ctx_tc) woq_b200_ctx_destroy(ctx_tc);
    if (ctx_gen) woq_b200_ctx_destroy(ctx_gen);
  }

  // the general-route context for activations that are not bf16 (lowp NONE on a tuned INT4 layer)
  woq_b200_ctx* ctx_general() {
    if (woq_b200_ctx_route(ctx) == WOQ_B200_ROUTE_GENERAL) return ctx;
    std::lock_guard<std::mutex> lock(tc_mu);
    if (!ctx_gen) {
      woq_b200_desc d{};
      WOQ_CHECK(woq_b200_ctx_desc(ctx, &d));
      TORCH_CHECK(!(d.layout_flags & WOQ_B200_LAYOUT_GATE_UP), "WOQ: a gate/up layer takes bf16 activations only");
      d.weight_format = WOQ_B200_FMT_PLAIN;
      d.layout_flags = WOQ_B200_LAYOUT_GENERIC | WOQ_B200_LAYOUT_SCALES_NK;
      auto stream = at::cuda::getCurrentCUDAStream(device);
      auto plain = at::empty({weight_shape[0], (weight_shape[1] + 1) / 2},
                             at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
      WOQ_CHECK(woq_b200_ctx_unpack(ctx, plain.data_ptr(), stream.stream()));
      WOQ_CHECK(woq_b200_ctx_create(&d, plain.data_ptr(), scales.data_ptr(),
                                    zero_points.defined() ? zero_points.data_ptr() : nullptr,
                                    bias.defined() ? bias.data_ptr() : nullptr, stream.stream(), &ctx_gen));
    }
    return ctx_gen;
  }

  // the context a call with M tokens runs on
  woq_b200_ctx* ctx_for(int64_t M) {
    if (M <= 16 || weight_dtype != WOQ_B200_DTYPE_INT4 || (layout_flags & WOQ_B200_LAYOUT_TC_ONLY) ||
        woq_b200_ctx_route(ctx) != WOQ_B200_ROUTE_INT4_BF16)
      return ctx;
    std::lock_guard<std::mutex> lock(tc_mu);
    if (!ctx_tc) {
      woq_b200_desc d{};
      WOQ_CHECK(woq_b200_ctx_desc(ctx, &d));
      d.weight_format = WOQ_B200_FMT_PLAIN;  // the plain weight comes out of the first context
      d.layout_flags = (d.layout_flags & ~WOQ_B200_LAYOUT_STREAM_ONLY) | WOQ_B200_LAYOUT_TC_ONLY | WOQ_B200_LAYOUT_SCALES_NK;
      auto stream = at::cuda::getCurrentCUDAStream(device);
      auto plain = at::empty({weight_shape[0], (weight_shape[1] + 1) / 2},
                             at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
      WOQ_CHECK(woq_b200_ctx_unpack(ctx, plain.data_ptr(), stream.stream()));
      WOQ_CHECK(woq_b200_ctx_create(&d, plain.data_ptr(), scales.data_ptr(),
                                    zero_points.defined() ? zero_points.data_ptr() : nullptr,
                                    bias.defined() ? bias.data_ptr() : nullptr, stream.stream(), &ctx_tc));
    }
    return ctx_tc;
  }

  static c10::intrusive_ptr<WoqLinearOpContext> create(
      at::Tensor weight, int64_t weight_dtype, std::vector<int64_t> weight_shape, at::Tensor scales,
      c10::optional<at::Tensor> zero_points, c10::optional<at::Tensor> bias,
      c10::optional<at::Tensor> g_idx, c10::optional<int64_t> batch_size, int64_t group_size,
      int64_t lowp_mode, int64_t act_quant_mode, bool cache_weight_for_large_batch,
      int64_t weight_format, int64_t layout_flags) {
    TORCH_CHECK(weight_shape.size() == 2, "WOQ: weight_shape must be [N, K]");
    const bool act_order = g_idx.has_value() && g_idx->defined();
    auto self = c10::make_intrusive<WoqLinearOpContext>();
    // everything lives on the weight's CUDA device (CPU tensors are moved to the current one)
    at::Device dev = weight.is_cuda() ? weight.device()
                                      : at::Device(at::kCUDA, at::cuda::current_device());
    c10::cuda::CUDAGuard guard(dev);
    auto to_dev = [&](const at::Tensor& t) { return t.to(dev).contiguous(); };
    at::Tensor w = to_dev(weight);
    at::Tensor perm, inv_perm, gi;
    if (act_order) {
      // GPTQ act-order: g_idx[k] is the group of input channel k.  As in the reference
      // (csrc/cpu/jit/cpu/kernels/LinearWoqPacked.cpp:755-870) the weight's input channels are
      // shuffled once so that every group is contiguous, and the activations are shuffled the
      // same way at run time.
      TORCH_CHECK(weight_dtype == WOQ_B200_DTYPE_INT4 && weight_format == WOQ_B200_FMT_PLAIN && group_size > 0,
                  "WOQ: g_idx needs a plain INT4 weight with a group size");
      gi = g_idx->to(dev).to(at::kLong).contiguous();
      TORCH_CHECK(gi.dim() == 1 && gi.numel() == weight_shape[1], "WOQ: g_idx size and weight shape mismatch");
      perm = at::argsort(gi, /*stable=*/true, /*dim=*/0, /*descending=*/false);
      auto sorted = gi.index_select(0, perm);
      auto want = at::arange(weight_shape[1], sorted.options()).floor_divide(group_size);
      TORCH_CHECK(at::equal(sorted, want), "WOQ: g_idx must assign exactly group_size input channels to every group");
      inv_perm = at::empty_like(perm);
      inv_perm.index_put_({perm}, at::arange(weight_shape[1], perm.options()));
      w = shuffle_int4_columns(w, perm);
    }
    at::Tensor s = to_dev(scales.dim() > 2 ? scales.squeeze() : scales);
    if (s.scalar_type() == at::kDouble) s = s.to(at::kFloat);
    at::Tensor z, b;
    if (zero_points.has_value() && zero_points->defined()) {
      z = to_dev(zero_points->dim() > 2 ? zero_points->squeeze() : *zero_points);
      if (z.scalar_type() != at::kFloat && z.scalar_type() != at::kByte) z = z.to(at::kFloat);
    }
    if (bias.has_value() && bias->defined()) {
      b = to_dev(*bias);
      if (b.scalar_type() != at::kFloat && b.scalar_type() != at::kBFloat16) b = b.to(at::kFloat);
    }
    woq_b200_desc d{};
    d.n = weight_shape[0];
    d.k = weight_shape[1];
    d.weight_dtype = static_cast<int32_t>(weight_dtype);
    d.group_size = static_cast<int32_t>(group_size);
    d.lowp_mode = static_cast<int32_t>(lowp_mode);
    d.act_quant_mode = static_cast<int32_t>(act_quant_mode);
    d.weight_format = static_cast<int32_t>(weight_format);
    d.scale_dtype = dtype_code(s);
    d.zp_dtype = z.defined() ? dtype_code(z) : WOQ_B200_T_NONE;
    d.bias_dtype = b.defined() ? dtype_code(b) : WOQ_B200_T_NONE;
    d.layout_flags = static_cast<int32_t>(layout_flags) | WOQ_B200_LAYOUT_SCALES_NK;
    if (weight_dtype == WOQ_B200_DTYPE_INT4 && !(layout_flags & (WOQ_B200_LAYOUT_STREAM_ONLY | WOQ_B200_LAYOUT_TC_ONLY)))
      d.layout_flags |= WOQ_B200_LAYOUT_STREAM_ONLY;
    d.kernel_hint = WOQ_B200_HINT_AUTO;
    auto stream = at::cuda::getCurrentCUDAStream(dev.index());
    WOQ_CHECK(woq_b200_ctx_create(&d, w.data_ptr(), s.data_ptr(), z.defined() ? z.data_ptr() : nullptr,
                                  b.defined() ? b.data_ptr() : nullptr, stream.stream(), &self->ctx));
    self->weight_dtype = weight_dtype;
    self->group_size = group_size;
    self->lowp_mode = lowp_mode;
    self->act_quant_mode = act_quant_mode;
    self->cache_weight_for_large_batch = cache_weight_for_large_batch;
    self->weight_shape = weight_shape;
    self->scales = s;
    self->zero_points = z;
    self->bias = b;
    if (act_order) {
      self->g_idx = gi;
      self->perm = perm;
      self->inv_perm = inv_perm;
    }
    self->batch_size = batch_size;
    self->device = dev.index();
    self->layout_flags = static_cast<int>(layout_flags);
    return self;
  }

  // plain [N, K/2] u8 (INT4) or [N, K] s8 (INT8): the reference's to_public(get_weight())
  at::Tensor get_weight() {
    c10::cuda::CUDAGuard guard(device);
    const bool int4 = weight_dtype == WOQ_B200_DTYPE_INT4 || weight_dtype == WOQ_B200_DTYPE_NF4;
    const bool bytes_u8 = int4 || weight_dtype == WOQ_B200_DTYPE_FP8;
    auto out = at::empty({weight_shape[0], int4 ? (weight_shape[1] + 1) / 2 : weight_shape[1]},
                         at::TensorOptions().dtype(bytes_u8 ? at::kByte : at::kChar).device(at::kCUDA, device));
    WOQ_CHECK(woq_b200_ctx_unpack(ctx, out.data_ptr(), at::cuda::getCurrentCUDAStream(device).stream()));
    return inv_perm.defined() ? shuffle_int4_columns(out, inv_perm) : out;
  }
  at::Tensor to_public(const at::Tensor& w) { return w; }
  c10::optional<at::Tensor> get_bias() { return bias.defined() ? c10::make_optional(bias) : c10::nullopt; }
  at::Tensor get_scales() { return scales; }
  c10::optional<at::Tensor> get_zero_points() {
    return zero_points.defined() ? c10::make_optional(zero_points) : c10::nullopt;
  }
  std::vector<int64_t> get_weight_shape() { return weight_shape; }
  c10::optional<at::Tensor> get_g_idx() { return g_idx.defined() ? c10::make_optional(g_idx) : c10::nullopt; }
  c10::optional<at::Tensor> get_cached_weight() { return c10::nullopt; }
  c10::optional<at::Tensor> get_cached_compensation() { return c10::nullopt; }
  at::Tensor pack(const at::Tensor& w) { return w; }
  // reference: WoqLinearOpContext::load_from_ctx (csrc/cpu/jit/cpu/kernels/OpContext.cpp) takes
  // over the packed weight and metadata of another context; here the other context's plain
  // weight is packed anew on this context's device
  void load_from_ctx(c10::intrusive_ptr<WoqLinearOpContext> other) {
    TORCH_CHECK(other && other->ctx, "WOQ: load_from_ctx needs a live context");
    if (other.get() == this) return;
    auto fresh = create(other->get_weight(), other->weight_dtype, other->weight_shape, other->scales,
                        other->zero_points.defined() ? c10::make_optional(other->zero_points) : c10::nullopt,
                        other->bias.defined() ? c10::make_optional(other->bias) : c10::nullopt,
                        other->g_idx.defined() ? c10::make_optional(other->g_idx) : c10::nullopt, other->batch_size,
                        other->group_size, other->lowp_mode, other->act_quant_mode,
                        other->cache_weight_for_large_batch, WOQ_B200_FMT_PLAIN,
                        other->layout_flags & WOQ_B200_LAYOUT_GATE_UP);
    std::lock_guard<std::mutex> lock(tc_mu);
    std::swap(ctx, fresh->ctx);
    std::swap(ctx_tc, fresh->ctx_tc);
    std::swap(ctx_gen, fresh->ctx_gen);
    weight_dtype = fresh->weight_dtype;
    group_size = fresh->group_size;
    lowp_mode = fresh->lowp_mode;
    act_quant_mode = fresh->act_quant_mode;
    cache_weight_for_large_batch = fresh->cache_weight_for_large_batch;
    weight_shape = fresh->weight_shape;
    scales = fresh->scales;
    zero_points = fresh->zero_points;
    bias = fresh->bias;
    g_idx = fresh->g_idx;
    perm = fresh->perm;
    inv_perm = fresh->inv_perm;
    batch_size = fresh->batch_size;
    device = fresh->device;
    layout_flags = fresh->layout_flags;
  }
  // CPU int64 tensor holding the raw pointer to this object (non-owning), as in the reference
  at::Tensor get_data_handle() {
    auto t = at::empty({1}, at::TensorOptions().dtype(at::kLong));
    t.data_ptr<int64_t>()[0] = reinterpret_cast<int64_t>(this);
    return t;
  }
};

WoqLinearOpContext* from_handle(const at::Tensor& handle) {
  TORCH_CHECK(handle.device().is_cpu() && handle.scalar_type() == at::kLong && handle.numel() == 1,
              "WOQ: W_prepack must be the 1-element CPU int64 handle of a WoqLinearOpContext");
  auto* c = reinterpret_cast<WoqLinearOpContext*>(handle.data_ptr<int64_t>()[0]);
  TORCH_CHECK(c != nullptr && c->magic == kHandleMagic, "WOQ: stale or foreign op-context handle");
  return c;
}

at::Tensor run(WoqLinearOpContext* c, const at::Tensor& input, int32_t fusion,
               const std::vector<at::Tensor>& others) {
  TORCH_CHECK(input.is_cuda(), "WOQ: input must be a CUDA tensor");
  TORCH_CHECK(input.get_device() == c->device, "WOQ: input is on cuda:", input.get_device(),
              " but the weights are on cuda:", static_cast<int>(c->device));
  const int64_t K = c->weight_shape[1], N = c->weight_shape[0];
  TORCH_CHECK(input.size(-1) == K, "WOQ: the last dimension of input (", input.size(-1),
              ") does not match the weight's in_features (", K, ")");
  c10::cuda::CUDAGuard guard(c->device);
  at::Tensor x = input.reshape({-1, K});
  if (c->perm.defined()) x = x.index_select(1, c->perm);  // act-order: channels in group order
  const auto in_dtype = x.scalar_type();
  TORCH_CHECK(in_dtype == at::kBFloat16 || in_dtype == at::kHalf || in_dtype == at::kFloat,
              "WOQ: activations must be bfloat16, float16 or float32, got ", in_dtype);
  // Compute dtype as the reference routes it (WoqLinearKrnl.cpp:75-165): lowp BF16 / INT8 convert
  // the activation themselves, so any floating input is cast to bf16 for the tuned kernels; lowp
  // NONE computes in the activation's dtype and lowp FP16 in fp16, which the general kernel does
  // (on the layer's general-route context) with the activation left as it is.
  const int route = woq_b200_ctx_route(c->ctx);
  const bool general = route == WOQ_B200_ROUTE_GENERAL ||
                       (route == WOQ_B200_ROUTE_INT4_BF16 && c->lowp_mode == WOQ_B200_LOWP_NONE &&
                        in_dtype != at::kBFloat16);
  if (!general && in_dtype != at::kBFloat16) x = x.to(at::kBFloat16);
  const int64_t esz = static_cast<int64_t>(x.element_size());
  if (x.stride(-1) != 1 || (x.stride(0) * esz % 16) != 0 || (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15))
    x = x.contiguous();
  const int64_t M = x.size(0);
  const int64_t n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? N / 2 : N;
  at::Tensor y = at::empty({M, n_out}, x.options());
  std::vector<at::Tensor> oth;
  std::vector<const void*> optr;
  for (auto& o : others) {
    at::Tensor t = o.reshape({-1, n_out});
    TORCH_CHECK(t.size(0) == M, "WOQ: extra operand has ", t.size(0), " rows, expected ", M);
    if (t.scalar_type() != x.scalar_type()) t = t.to(x.scalar_type());
    oth.push_back(t.contiguous());
    optr.push_back(oth.back().data_ptr());
  }
  auto stream = at::cuda::getCurrentCUDAStream(c->device);
  if (M > 0) {
    woq_b200_ctx* k = general ? c->ctx_general() : c->ctx_for(M);
    const size_t need = woq_b200_workspace_bytes(k, M);
    at::Tensor& ws = workspace_for(c->device, stream.stream(), need);
    if (general) {
      const int io = x.scalar_type() == at::kBFloat16 ? WOQ_B200_T_BF16
                     : x.scalar_type() == at::kHalf   ? WOQ_B200_T_F16
                                                      : WOQ_B200_T_F32;
      WOQ_CHECK(woq_b200_linear_any(k, x.data_ptr(), io, M, x.stride(0), fusion,
                                    optr.empty() ? nullptr : optr.data(), static_cast<int32_t>(optr.size()),
                                    y.data_ptr(), y.stride(0), ws.data_ptr(), ws.numel(), stream.stream()));
    } else {
      WOQ_CHECK(woq_b200_linear(k, x.data_ptr(), M, x.stride(0), fusion,
                                optr.empty() ? nullptr : optr.data(), static_cast<int32_t>(optr.size()),
                                y.data_ptr(), y.stride(0), ws.data_ptr(), ws.numel(), stream.stream()));
    }
  }
  auto sizes = input.sizes().vec();
  sizes.back() = n_out;
  y = y.view(sizes);
  return y.scalar_type() == in_dtype ? y : y.to(in_dtype);
}

at::Tensor woq_unary(const at::Tensor& input, const at::Tensor& handle, int32_t fusion) {
  return run(from_handle(handle), input, fusion, {});
}

at::Tensor ipex_woq_linear(const at::Tensor& i, const at::Tensor& h) { return woq_unary(i, h, WOQ_B200_FUSE_NONE); }
at::Tensor woq_linear_gelu(const at::Tensor& i, const at::Tensor& h) { return woq_unary(i, h, WOQ_B200_FUSE_GELU_ERF); }
at::Tensor woq_linear_new_gelu(const at::Tensor& i, const at::Tensor& h) { return woq_unary(i, h, WOQ_B200_FUSE_GELU_TANH); }
at::Tensor woq_linear_relu(const at::Tensor& i, const at::Tensor& h) { return woq_unary(i, h, WOQ_B200_FUSE_RELU); }
at::Tensor woq_linear_silu(const at::Tensor& i, const at::Tensor& h) { return woq_unary(i, h, WOQ_B200_FUSE_SILU); }
at::Tensor woq_linear_silu_mul(const at::Tensor& i, const at::Tensor& h) { return woq_unary(i, h, WOQ_B200_FUSE_SILU_MUL); }
at::Tensor woq_linear_add(const at::Tensor& i, const at::Tensor& h, const std::vector<at::Tensor>& o) {
  TORCH_CHECK(o.size() >= 1, "WOQ: woq_linear_add takes one extra tensor");
  return run(from_handle(h), i, WOQ_B200_FUSE_ADD, {o[0]});
}
at::Tensor woq_linear_add_add(const at::Tensor& i, const at::Tensor& h, const std::vector<at::Tensor>& o) {
  TORCH_CHECK(o.size() >= 2, "WOQ: woq_linear_add_add takes two extra tensors");
  return run(from_handle(h), i, WOQ_B200_FUSE_ADD_ADD, {o[0], o[1]});
}
at::Tensor woq_linear_mul(const at::Tensor& i, const at::Tensor& h, const std::vector<at::Tensor>& o) {
  TORCH_CHECK(o.size() >= 1, "WOQ: woq_linear_mul takes one extra tensor");
  return run(from_handle(h), i, WOQ_B200_FUSE_MUL, {o[0]});
}

// B200-side fusion (the reference runs the norm and the activation quantiser as separate steps):
// RMSNorm and the per-token INT8 quantiser in one kernel, so that the linears that read the same
// normalised activations (q / k / v, gate / up) share one quantisation.  Returns (codes int8
// [.., K], scales f32 [rows], zero points int32 [rows] - empty for the symmetric mode).
std::tuple<at::Tensor, at::Tensor, at::Tensor> woq_rmsnorm_quant(const at::Tensor& input, const at::Tensor& weight,
                                                                 double eps, int64_t act_quant_mode) {
  TORCH_CHECK(input.is_cuda() && input.scalar_type() == at::kBFloat16, "WOQ: rmsnorm_quant takes bf16 CUDA input");
  const int64_t K = input.size(-1);
  TORCH_CHECK(weight.numel() == K, "WOQ: the norm weight has ", weight.numel(), " elements, expected ", K);
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor x = input.reshape({-1, K});
  if (x.stride(-1) != 1 || (x.stride(0) % 8) != 0 || (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15)) x = x.contiguous();
  at::Tensor g = weight.to(input.device(), at::kBFloat16).contiguous();
  const int64_t M = x.size(0);
  auto sizes = input.sizes().vec();
  at::Tensor qa = at::empty(sizes, x.options().dtype(at::kChar));
  at::Tensor sa = at::empty({M}, x.options().dtype(at::kFloat));
  const bool asym = act_quant_mode == WOQ_B200_ACT_PER_M;
  at::Tensor zpa = at::empty({asym ? M : 0}, x.options().dtype(at::kInt));
  auto stream = at::cuda::getCurrentCUDAStream(input.get_device());
  WOQ_CHECK(woq_b200_rmsnorm_quant(x.data_ptr(), x.stride(0), g.data_ptr(), static_cast<float>(eps), M, K,
                                   static_cast<int32_t>(act_quant_mode), nullptr, 0, qa.data_ptr(), sa.data_ptr(),
                                   asym ? zpa.data_ptr() : nullptr, stream.stream()));
  return std::make_tuple(qa, sa, zpa);
}

// The linear on activations quantised by woq_rmsnorm_quant; `fusion` as in the C ABI (0 none,
// 0x100 silu*mul on a gate/up context, ...), `others` the extra operands of the binary post-ops.
at::Tensor woq_linear_prequant(const at::Tensor& qa, const at::Tensor& sa, const at::Tensor& zpa,
                               const at::Tensor& handle, int64_t fusion, const std::vector<at::Tensor>& others) {
  WoqLinearOpContext* c = from_handle(handle);
  TORCH_CHECK(qa.is_cuda() && qa.scalar_type() == at::kChar && qa.get_device() == c->device,
              "WOQ: qa must be an int8 tensor on the weights' device");
  const int64_t K = c->weight_shape[1], N = c->weight_shape[0];
  TORCH_CHECK(qa.size(-1) == K, "WOQ: the last dimension of qa (", qa.size(-1), ") does not match in_features (", K, ")");
  c10::cuda::CUDAGuard guard(c->device);
  at::Tensor q2 = qa.reshape({-1, K}).contiguous();
  const int64_t M = q2.size(0);
  const int64_t n_out = fusion == WOQ_B200_FUSE_SILU_MUL ? N / 2 : N;
  at::Tensor y = at::empty({M, n_out}, qa.options().dtype(at::kBFloat16));
  std::vector<at::Tensor> oth;
  std::vector<const void*> optr;
  for (auto& o : others) {
    at::Tensor t = o.reshape({-1, n_out});
    TORCH_CHECK(t.size(0) == M, "WOQ: extra operand has ", t.size(0), " rows, expected ", M);
    oth.push_back(t.to(at::kBFloat16).contiguous());
    optr.push_back(oth.back().data_ptr());
  }
  auto stream = at::cuda::getCurrentCUDAStream(c->device);
  if (M > 0) {
    woq_b200_ctx* k = c->ctx_for(M);
    at::Tensor& ws = workspace_for(c->device, stream.stream(), woq_b200_workspace_bytes(k, M));
    WOQ_CHECK(woq_b200_linear_prequant(k, q2.data_ptr(), sa.data_ptr(), zpa.numel() ? zpa.data_ptr() : nullptr, M,
                                       static_cast<int32_t>(fusion), optr.empty() ? nullptr : optr.data(),
                                       static_cast<int32_t>(optr.size()), y.data_ptr(), y.stride(0), ws.data_ptr(),
                                       ws.numel(), stream.stream()));
  }
  auto sizes = qa.sizes().vec();
  sizes.back() = n_out;
  return y.view(sizes);
}

// reference: csrc/cpu/aten/MoE.cpp:260-288 + kernels/MoEKrnl.cpp:254-285.  top_x = the tokens routed to
// this expert, idx = which of their top-k slots; the three handles are the expert's w1 / w3 / w2.
at::Tensor mixtral_moe_woq(const at::Tensor& hidden_states, const at::Tensor& top_x, const at::Tensor& idx,
                           const at::Tensor& gate_wei, const at::Tensor& up_wei, const at::Tensor& down_wei,
                           const at::Tensor& routing_weights, at::Tensor output, bool is_distributed) {
  if (top_x.size(0) == 0) return output;
  TORCH_CHECK(!is_distributed, "WOQ: the distributed MoE all-reduce is done by the caller in this build");
  TORCH_CHECK(output.is_cuda() && output.scalar_type() == at::kBFloat16 && output.is_contiguous(),
              "WOQ: MoE output must be a contiguous bf16 CUDA tensor");
  auto* g = from_handle(gate_wei);
  auto* u = from_handle(up_wei);
  auto* d = from_handle(down_wei);
  c10::cuda::CUDAGuard guard(d->device);
  at::Tensor tx = top_x.to(hidden_states.device());
  at::Tensor x = hidden_states.index_select(0, tx);
  at::Tensor a = run(u, x, WOQ_B200_FUSE_MUL, {run(g, x, WOQ_B200_FUSE_SILU, {})});
  at::Tensor w = routing_weights.index({tx, idx.to(hidden_states.device())}).to(at::kBFloat16).contiguous();
  at::Tensor ti = tx.to(at::kInt).contiguous();
  if (a.scalar_type() != at::kBFloat16) a = a.to(at::kBFloat16);
  a = a.contiguous();
  const int64_t M = a.size(0);
  auto stream = at::cuda::getCurrentCUDAStream(d->device);
  woq_b200_ctx* dk = d->ctx_for(M);
  at::Tensor& ws = workspace_for(d->device, stream.stream(), woq_b200_workspace_bytes(dk, M));
  WOQ_CHECK(woq_b200_linear_scatter(dk, a.data_ptr(), M, a.stride(0), ti.data_ptr<int32_t>(), w.data_ptr(),
                                    output.data_ptr(), output.stride(0), ws.data_ptr(), ws.numel(),
                                    stream.stream()));
  return output;
}

// reference: csrc/cpu/aten/MoE.cpp:290-330.  topk_ids [tokens, top_k] names each token's experts; every
// selected expert runs the per-expert routine above on its tokens.  The (token, slot) pairs of all
// experts come from one stable sort on the device and one copy of the per-expert counts to the host.
at::Tensor deepseek_moe_woq(const at::Tensor& hidden_states, const at::Tensor& topk_ids,
                            const std::vector<c10::intrusive_ptr<WoqLinearOpContext>>& gate_ctx,
                            const std::vector<c10::intrusive_ptr<WoqLinearOpContext>>& up_ctx,
                            const std::vector<c10::intrusive_ptr<WoqLinearOpContext>>& down_ctx,
                            const at::Tensor& routing_weights, bool is_distributed) {
  const int64_t experts = static_cast<int64_t>(gate_ctx.size());
  TORCH_CHECK(static_cast<int64_t>(up_ctx.size()) == experts && static_cast<int64_t>(down_ctx.size()) == experts,
              "WOQ: deepseek_moe_woq takes one gate, up and down context per expert");
  TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.size(0) == hidden_states.size(0),
              "WOQ: topk_ids must be [tokens, top_k]");
  at::Tensor output = at::zeros_like(hidden_states);
  if (experts == 0 || topk_ids.numel() == 0) return output;
  const int64_t top_k = topk_ids.size(1);
  at::Tensor flat = topk_ids.to(hidden_states.device()).reshape({-1}).to(at::kLong);
  at::Tensor order = at::argsort(flat, /*stable=*/true, /*dim=*/0, /*descending=*/false);
  at::Tensor counts = at::bincount(flat, {}, experts).cpu();
  TORCH_CHECK(counts.size(0) == experts, "WOQ: topk_ids names an expert beyond the contexts given");
  const int64_t* cnt = counts.data_ptr<int64_t>();
  int64_t off = 0;
  for (int64_t e = 0; e < experts; ++e) {
    if (cnt[e] == 0) continue;
    at::Tensor pairs = order.narrow(0, off, cnt[e]);
    off += cnt[e];
    at::Tensor top_x = at::floor_divide(pairs, top_k);
    at::Tensor idx = at::remainder(pairs, top_k);
    output = mixtral_moe_woq(hidden_states, top_x, idx, gate_ctx[e]->get_data_handle(),
                             up_ctx[e]->get_data_handle(), down_ctx[e]->get_data_handle(), routing_weights,
                             output, is_distributed);
  }
  return output;
}

int64_t dtype_from_str(const std::string& s) {
  if (s == "int8") return WOQ_B200_DTYPE_INT8;
  if (s == "int4") return WOQ_B200_DTYPE_INT4;
  if (s == "nf4") return WOQ_B200_DTYPE_NF4;
  if (s == "fp8") return WOQ_B200_DTYPE_FP8;
  TORCH_CHECK(false, "WOQ: Unexpected weight dtype: ", s);
}

// context-free form: packs, runs, and drops the context (reference: Linear.cpp:556-617)
at::Tensor woq_linear(const at::Tensor& input, const at::Tensor& qweight, const std::string& weight_dtype,
                      const std::vector<int64_t>& weight_shape, const std::vector<at::Tensor>& weight_scales,
                      const c10::optional<std::vector<at::Tensor>>& weight_zeros,
                      const c10::optional<std::vector<at::Tensor>>& bias,
                      const c10::optional<at::Tensor>& g_idx, int64_t group_size, int64_t lowp_mode,
                      int64_t act_quant_mode, const c10::optional<at::Tensor>& compensation) {
  TORCH_CHECK(!weight_scales.empty(), "WOQ: weight_scales is empty");
  c10::optional<at::Tensor> z, b;
  if (weight_zeros.has_value() && !weight_zeros->empty()) z = (*weight_zeros)[0];
  if (bias.has_value() && !bias->empty() && (*bias)[0].defined()) b = (*bias)[0];
  auto ctx = WoqLinearOpContext::create(qweight, dtype_from_str(weight_dtype), weight_shape, weight_scales[0],
                                        z, b, g_idx, c10::nullopt, group_size, lowp_mode, act_quant_mode,
                                        false, WOQ_B200_FMT_PLAIN, 0);
  return run(ctx.get(), input, WOQ_B200_FUSE_NONE, {});
}

c10::intrusive_ptr<WoqLinearOpContext> prepack(
    at::Tensor W, int64_t W_dtype, std::vector<int64_t> W_shape, at::Tensor scales,
    c10::optional<at::Tensor> zero_points, c10::optional<at::Tensor> B, c10::optional<at::Tensor> g_idx,
    c10::optional<int64_t> batch_size, int64_t group_size, int64_t lowp_mode, int64_t act_quant_mode,
    bool cache_weight_for_large_batch) {
  return WoqLinearOpContext::create(W, W_dtype, W_shape, scales, zero_points, B, g_idx, batch_size,
                                    group_size, lowp_mode, act_quant_mode, cache_weight_for_large_batch,
                                    WOQ_B200_FMT_PLAIN, 0);
}

c10::intrusive_ptr<WoqLinearOpContext> prepack_int4(
    at::Tensor W, at::Tensor scales, c10::optional<at::Tensor> zeros, c10::optional<at::Tensor> B,
    c10::optional<at::Tensor> g_idx, c10::optional<int64_t> batch_size, int64_t group_size,
    int64_t lowp_mode, int64_t act_quant_mode, bool cache_weight_for_large_batch, int64_t weight_format) {
  // scales / zeros arrive as [N, groups] (the Python side has converted checkpoint layouts)
  int64_t N, K;
  if (weight_format == WOQ_B200_FMT_GPTQ) {
    N = W.size(1);
    K = W.size(0) * 8;
  } else if (weight_format == WOQ_B200_FMT_AWQ) {
    N = W.size(1) * 8;
    K = W.size(0);
  } else {
    N = W.size(0);
    K = W.size(1) * (W.scalar_type() == at::kInt ? 8 : 2);
    if (W.scalar_type() == at::kInt) W = W.contiguous().view(at::kByte);  // 8 nibbles, low first
  }
  c10::optional<at::Tensor> z;
  if (zeros.has_value() && zeros->defined()) z = zeros->to(at::kFloat);
  return WoqLinearOpContext::create(W, WOQ_B200_DTYPE_INT4, {N, K}, scales, z, B, g_idx, batch_size,
                                    group_size, lowp_mode, act_quant_mode, cache_weight_for_large_batch,
                                    weight_format, 0);
}

c10::intrusive_ptr<WoqLinearOpContext> prepack_gate_up(
    at::Tensor W, int64_t W_dtype, std::vector<int64_t> W_shape, at::Tensor scales,
    c10::optional<at::Tensor> zero_points, c10::optional<at::Tensor> B, int64_t group_size,
    int64_t lowp_mode, int64_t act_quant_mode) {
  return WoqLinearOpContext::create(W, W_dtype, W_shape, scales, zero_points, B, c10::nullopt, c10::nullopt,
                                    group_size, lowp_mode, act_quant_mode, false, WOQ_B200_FMT_PLAIN,
                                    WOQ_B200_LAYOUT_GATE_UP);
}

// woq_linear_pack_weight of the reference returns the blocked weight and the {fp32, fp16, bf16}
// copies of scales / zero points / bias for the context-free woq_linear op
// (csrc/cpu/jit/cpu/kernels/OpContext.cpp packWoqLinearWeight, ContextLinearWoq.h:60-128).
// Here the device repack belongs to a context, so the weight is handed on in its public plain
// format (which woq_linear accepts) together with the same dtype copies.
std::tuple<at::Tensor, std::vector<at::Tensor>, c10::optional<std::vector<at::Tensor>>,
           c10::optional<std::vector<at::Tensor>>, c10::optional<at::Tensor>>
pack_weight(const at::Tensor& W, const std::string& W_dtype, const std::vector<int64_t>& W_shape,
            const at::Tensor& scales, const c10::optional<at::Tensor>& zero_points,
            const c10::optional<at::Tensor>& B, const c10::optional<at::Tensor>& g_idx, int64_t group_size,
            int64_t lowp_mode) {
  (void)dtype_from_str(W_dtype);  // rejects unknown dtype names
  (void)W_shape;
  (void)group_size;
  (void)lowp_mode;
  auto copies = [](const at::Tensor& t) {
    auto f = t.to(at::kFloat);
    return std::vector<at::Tensor>{f, f.to(at::kHalf), f.to(at::kBFloat16)};
  };
  c10::optional<std::vector<at::Tensor>> z, b;
  if (zero_points.has_value() && zero_points->defined()) z = copies(*zero_points);
  if (B.has_value() && B->defined()) b = copies(*B);
  return std::make_tuple(W.contiguous(), copies(scales), z, b, g_idx);
}

at::Tensor unpack_weight(const at::Tensor& weight, const std::string&, const std::vector<int64_t>&, int64_t) {
  return weight;  // weights handed out by get_weight() are already in the public plain format
}

// AutocastCUDA: cast the activation to the autocast dtype, like the reference's AutocastCPU
// wrappers (csrc/cpu/aten/Linear.cpp:874-1005)
at::Tensor autocast_input(const at::Tensor& x) {
  return x.is_floating_point() ? x.to(at::autocast::get_autocast_dtype(at::kCUDA)) : x;
}
#define AUTOCAST_UNARY(name)                                                          \
  at::Tensor name##_autocast(const at::Tensor& i, const at::Tensor& h) {              \
    c10::impl::ExcludeDispatchKeyGuard no_autocast(c10::DispatchKey::AutocastCUDA);   \
    return name(autocast_input(i), h);                                                \
  }
AUTOCAST_UNARY(ipex_woq_linear)
AUTOCAST_UNARY(woq_linear_gelu)
AUTOCAST_UNARY(woq_linear_new_gelu)
AUTOCAST_UNARY(woq_linear_relu)
AUTOCAST_UNARY(woq_linear_silu)
AUTOCAST_UNARY(woq_linear_silu_mul)
#define AUTOCAST_BINARY(name)                                                                        \
  at::Tensor name##_autocast(const at::Tensor& i, const at::Tensor& h, const std::vector<at::Tensor>& o) { \
    c10::impl::ExcludeDispatchKeyGuard no_autocast(c10::DispatchKey::AutocastCUDA);                  \
    return name(autocast_input(i), h, o);                                                            \
  }
AUTOCAST_BINARY(woq_linear_add)
AUTOCAST_BINARY(woq_linear_add_add)
AUTOCAST_BINARY(woq_linear_mul)

}  // namespace

TORCH_LIBRARY(ipex_prepack, m) {
  m.class_<WoqLinearOpContext>("WoqLinearOpContext")
      .def("get_weight", &WoqLinearOpContext::get_weight)
      .def("get_bias", &WoqLinearOpContext::get_bias)
      .def("get_scales", &WoqLinearOpContext::get_scales)
      .def("get_zero_points", &WoqLinearOpContext::get_zero_points)
      .def("get_weight_shape", &WoqLinearOpContext::get_weight_shape)
      .def("get_g_idx", &WoqLinearOpContext::get_g_idx)
      .def("get_cached_weight", &WoqLinearOpContext::get_cached_weight)
      .def("get_cached_compensation", &WoqLinearOpContext::get_cached_compensation)
      .def("pack", &WoqLinearOpContext::pack)
      .def("to_public", &WoqLinearOpContext::to_public)
      .def("get_data_handle", &WoqLinearOpContext::get_data_handle)
      .def("load_from_ctx", &WoqLinearOpContext::load_from_ctx)
      .def_pickle(
          // state: the reference's 12-tuple (csrc/cpu/jit/cpu/kernels/OpContext.h:363-375) with the
          // weight in its plain format; a gate/up-interleaved context marks itself with one
          // extra bit in the weight dtype
          [](const c10::intrusive_ptr<WoqLinearOpContext>& self) {
            return std::make_tuple(self->get_weight().cpu(),
                                   self->weight_dtype | ((self->layout_flags & WOQ_B200_LAYOUT_GATE_UP) ? kGateUpStateBit : 0),
                                   self->weight_shape,
                                   self->scales.cpu(),
                                   self->zero_points.defined() ? c10::make_optional(self->zero_points.cpu()) : c10::nullopt,
                                   self->bias.defined() ? c10::make_optional(self->bias.cpu()) : c10::nullopt,
                                   self->g_idx.defined() ? c10::make_optional(self->g_idx.cpu()) : c10::nullopt,
                                   self->batch_size, self->group_size,
                                   self->lowp_mode, self->act_quant_mode, self->cache_weight_for_large_batch);
          },
          [](std::tuple<at::Tensor, int64_t, std::vector<int64_t>, at::Tensor, c10::optional<at::Tensor>,
                        c10::optional<at::Tensor>, c10::optional<at::Tensor>, c10::optional<int64_t>, int64_t,
                        int64_t, int64_t, bool> st) {
            const int64_t wd = std::get<1>(st);
            return WoqLinearOpContext::create(std::get<0>(st), wd & ~kGateUpStateBit, std::get<2>(st), std::get<3>(st),
                                              std::get<4>(st), std::get<5>(st), std::get<6>(st), std::get<7>(st),
                                              std::get<8>(st), std::get<9>(st), std::get<10>(st), std::get<11>(st),
                                              WOQ_B200_FMT_PLAIN, (wd & kGateUpStateBit) ? WOQ_B200_LAYOUT_GATE_UP : 0);
          });
  m.def("weight_only_qlinear_prepack(Tensor W, int W_dtype, int[] W_shape, Tensor scales, Tensor? zero_points, "
        "Tensor? B, Tensor? g_idx, int? batch_size, int group_size, int lowp_mode, int act_quant_mode, "
        "bool cache_weight_for_large_batch=False) -> __torch__.torch.classes.ipex_prepack.WoqLinearOpContext",
        prepack);
  m.def("weight_only_qlinear_prepack_int4(Tensor W, Tensor scales, Tensor? zeros, Tensor? B, Tensor? g_idx, "
        "int? batch_size, int group_size, int lowp_mode, int act_quant_mode, "
        "bool cache_weight_for_large_batch=False, int weight_format=0) -> "
        "__torch__.torch.classes.ipex_prepack.WoqLinearOpContext",
        prepack_int4);
  m.def("weight_only_qlinear_prepack_gate_up(Tensor W, int W_dtype, int[] W_shape, Tensor scales, "
        "Tensor? zero_points, Tensor? B, int group_size, int lowp_mode, int act_quant_mode) -> "
        "__torch__.torch.classes.ipex_prepack.WoqLinearOpContext",
        prepack_gate_up);
  m.def("woq_linear_pack_weight(Tensor W, str W_dtype, int[] W_shape, Tensor scales, Tensor? zero_points, "
        "Tensor? B, Tensor? g_idx, int group_size, int lowp_mode) -> "
        "(Tensor, Tensor[], Tensor[]?, Tensor[]?, Tensor?)",
        pack_weight);
  m.def("woq_linear_unpack_weight(Tensor W, str W_dtype, int[] W_shape, int lowp_mode) -> Tensor", unpack_weight);
}

TORCH_LIBRARY(torch_ipex, m) {
  m.def("ipex_woq_linear(Tensor input, Tensor W_prepack) -> Tensor");
  m.def("woq_linear_gelu(Tensor input, Tensor W_prepack) -> Tensor");
  m.def("woq_linear_new_gelu(Tensor input, Tensor W_prepack) -> Tensor");
  m.def("woq_linear_relu(Tensor input, Tensor W_prepack) -> Tensor");
  m.def("woq_linear_silu(Tensor input, Tensor W_prepack) -> Tensor");
  m.def("woq_linear_silu_mul(Tensor input, Tensor W_prepack) -> Tensor");
  m.def("woq_linear_add(Tensor input, Tensor W_prepack, Tensor[] others) -> Tensor");
  m.def("woq_linear_add_add(Tensor input, Tensor W_prepack, Tensor[] others) -> Tensor");
  m.def("woq_linear_mul(Tensor input, Tensor W_prepack, Tensor[] others) -> Tensor");
  m.def("mixtral_moe_woq(Tensor hidden_states, Tensor top_x, Tensor idx, Tensor gate_wei, Tensor up_wei, "
        "Tensor down_wei, Tensor routing_weights, Tensor output, bool is_distributed) -> Tensor");
  m.def("deepseek_moe_woq(Tensor hidden_states, Tensor topk_ids, "
        "__torch__.torch.classes.ipex_prepack.WoqLinearOpContext[] gate_ctx, "
        "__torch__.torch.classes.ipex_prepack.WoqLinearOpContext[] up_ctx, "
        "__torch__.torch.classes.ipex_prepack.WoqLinearOpContext[] down_ctx, "
        "Tensor routing_weights, bool is_distributed) -> Tensor");
  m.def("woq_rmsnorm_quant(Tensor input, Tensor weight, float eps, int act_quant_mode) -> (Tensor, Tensor, Tensor)");
  m.def("woq_linear_prequant(Tensor qa, Tensor sa, Tensor zpa, Tensor W_prepack, int fusion, Tensor[] others) -> Tensor");
  m.def("woq_check_status() -> ()", woq_check_status);
  m.def("woq_linear(Tensor input, Tensor qweight, str weight_dtype, int[] weight_shape, Tensor[] weight_scales, "
        "Tensor[]? weight_zeros, Tensor[]? bias, Tensor? g_idx, int group_size, int lowp_mode, "
        "int act_quant_mode, Tensor? compensation) -> Tensor");
}

TORCH_LIBRARY_IMPL(torch_ipex, CUDA, m) {
  m.impl("ipex_woq_linear", ipex_woq_linear);
  m.impl("woq_linear_gelu", woq_linear_gelu);
  m.impl("woq_linear_new_gelu", woq_linear_new_gelu);
  m.impl("woq_linear_relu", woq_linear_relu);
  m.impl("woq_linear_silu", woq_linear_silu);
  m.impl("woq_linear_silu_mul", woq_linear_silu_mul);
  m.impl("woq_linear_add", woq_linear_add);
  m.impl("woq_linear_add_add", woq_linear_add_add);
  m.impl("woq_linear_mul", woq_linear_mul);
  m.impl("woq_linear", woq_linear);
  m.impl("mixtral_moe_woq", mixtral_moe_woq);
  m.impl("deepseek_moe_woq", deepseek_moe_woq);
  m.impl("woq_rmsnorm_quant", woq_rmsnorm_quant);
  m.impl("woq_linear_prequant", woq_linear_prequant);
}

TORCH_LIBRARY_IMPL(torch_ipex, AutocastCUDA, m) {
  m.impl("ipex_woq_linear", ipex_woq_linear_autocast);
  m.impl("woq_linear_gelu", woq_linear_gelu_autocast);
  m.impl("woq_linear_new_gelu", woq_linear_new_gelu_autocast);
  m.impl("woq_linear_relu", woq_linear_relu_autocast);
  m.impl("woq_linear_silu", woq_linear_silu_autocast);
  m.impl("woq_linear_silu_mul", woq_linear_silu_mul_autocast);
  m.impl("woq_linear_add", woq_linear_add_autocast);
  m.impl("woq_linear_add_add", woq_linear_add_add_autocast);
  m.impl("woq_linear_mul", woq_linear_mul_autocast);
}
