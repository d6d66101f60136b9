"""Fused-epilogue wrappers around WOQ linears: same classes and forward signatures as the
reference's _IPEXlinear*CPU modules (transformers/models/cpu/fusions/linear_fusion.py:21-492).
Each forward is one operator call with the epilogue fused into the kernel."""
import torch
from torch import nn


class _IPEXlinearFusion(nn.Module):
    def __init__(self, linear, tpp=False, woq=True):
        super().__init__()
        self.tpp = tpp
        self.woq = woq
        self.linear = linear

    def _handle(self):
        assert self.woq and getattr(self.linear, "_op_context", None) is not None, (
            "this build fuses epilogues for weight-only-quantised linears only")
        return self.linear._op_context.get_data_handle()


class _IPEXlinearSilu(_IPEXlinearFusion):
    def forward(self, x):
        return torch.ops.torch_ipex.woq_linear_silu(x, self._handle())


class _IPEXlinearRelu(_IPEXlinearFusion):
    def forward(self, x):
        return torch.ops.torch_ipex.woq_linear_relu(x, self._handle())


class _IPEXlinearMul(_IPEXlinearFusion):
    def forward(self, x, y):
        return torch.ops.torch_ipex.woq_linear_mul(x, self._handle(), [y])


class _IPEXlinearAdd(_IPEXlinearFusion):
    def forward(self, x, y):
        return torch.ops.torch_ipex.woq_linear_add(x, self._handle(), [y])


class _IPEXlinearAddAdd(_IPEXlinearFusion):
    def forward(self, x, y, z):
        return torch.ops.torch_ipex.woq_linear_add_add(x, self._handle(), [y, z])


class _IPEXlinearNewGelu(_IPEXlinearFusion):
    def forward(self, x):
        return torch.ops.torch_ipex.woq_linear_new_gelu(x, self._handle())


class _IPEXlinearGelu(_IPEXlinearFusion):
    def forward(self, x):
        return torch.ops.torch_ipex.woq_linear_gelu(x, self._handle())


class _IPEXlinearSiluMul(nn.Module):
    """silu(linear_s(x)) * linear_m(x): woq_linear_silu then woq_linear_mul, exactly the
    reference's composition (linear_fusion.py:482-490)."""

    def __init__(self, module_s, module_m, tpp=False, woq=True):
        super().__init__()
        self.tpp = tpp
        self.woq = woq
        self.linear_s = module_s
        self.linear_m = module_m

    def forward(self, x):
        y = torch.ops.torch_ipex.woq_linear_silu(x, self.linear_s._op_context.get_data_handle())
        return torch.ops.torch_ipex.woq_linear_mul(x, self.linear_m._op_context.get_data_handle(), [y])


class _IPEXlinearFusedGateUp(nn.Module):
    """One kernel for a stacked gate/up weight: y = silu(gate(x)) * up(x).  Not in the reference;
    numerically the same composition as _IPEXlinearSiluMul."""

    is_gate_up = True

    def __init__(self, op_context, out_features, lowp_mode=-1, act_quant_mode=-1):
        super().__init__()
        self._op_context = op_context
        self.out_features = out_features
        self._lowp_mode = int(lowp_mode)
        self._act_quant_mode = int(act_quant_mode)

    @classmethod
    def from_quantized(cls, qweight, dtype, shape, scales, zero_points, group_size, lowp_mode, act_quant_mode=-1):
        from ..._ops import load_ops

        load_ops()
        ctx = torch.ops.ipex_prepack.weight_only_qlinear_prepack_gate_up(
            qweight, int(dtype), list(shape), scales, zero_points, None, group_size, int(lowp_mode),
            int(act_quant_mode))
        return cls(ctx, shape[0] // 2, lowp_mode, act_quant_mode)

    def forward(self, x):
        return torch.ops.torch_ipex.woq_linear_silu_mul(x, self._op_context.get_data_handle())


    @classmethod
    def from_linears(cls, gate, up):
        """Stack two WeightOnlyQuantizedLinear modules (gate over up) into one gate/up context.
        Quantisation is per output row, so stacking the codes, scales and zero points is exact:
        the fused layer multiplies by the same dequantised weights as the two it came from."""
        from ...nn.modules.weight_only_quantization import WeightOnlyQuantizedLinear

        assert isinstance(gate, WeightOnlyQuantizedLinear) and isinstance(up, WeightOnlyQuantizedLinear)
        qw, s, z, b, meta = _stack_quantized([gate, up])
        assert b is None, "the fused gate/up layer is built for projections without bias"
        return cls.from_quantized(qw, meta["dtype"], [qw.shape[0], meta["k"]], s, z, meta["group_size"],
                                  meta["lowp_mode"], meta["act_quant_mode"])


def _stack_quantized(linears):
    """Codes, scales, zero points and bias of several WOQ linears with the same K and recipe,
    concatenated along N."""
    ctxs = [m._op_context for m in linears]
    first = linears[0]
    k = ctxs[0].get_weight_shape()[1]
    for m, c in zip(linears, ctxs):
        assert c.get_weight_shape()[1] == k, "concatenated linears must share in_features"
        assert c.get_g_idx() is None, "act-order layers are not concatenated (reference: linear_fusion.py:313-321)"
        assert (m.dtype, m._group_size, m._lowp_mode, m._act_quant_mode) == (
            first.dtype, first._group_size, first._lowp_mode, first._act_quant_mode), "mixed recipes"
    qw = torch.cat([c.get_weight() for c in ctxs], 0)
    scales = torch.cat([c.get_scales().reshape(c.get_weight_shape()[0], -1) for c in ctxs], 0)
    zps = [c.get_zero_points() for c in ctxs]
    zero_points = None if zps[0] is None else torch.cat(
        [z.reshape(c.get_weight_shape()[0], -1) for z, c in zip(zps, ctxs)], 0)
    biases = [c.get_bias() for c in ctxs]
    bias = torch.cat(biases, 0) if all(b is not None for b in biases) else None
    if first._group_size <= 0:
        scales = scales.reshape(-1)
        zero_points = None if zero_points is None else zero_points.reshape(-1)
    meta = dict(dtype=first.dtype, k=k, group_size=first._group_size, lowp_mode=first._lowp_mode,
                act_quant_mode=first._act_quant_mode)
    return qw, scales, zero_points, bias, meta


class _IPEXConcatLinear(nn.Module):
    """Several linears that read the same input (q / k / v projections) as one: the reference's
    _IPEXConcatLinearCPU (transformers/models/cpu/fusions/linear_fusion.py:296-434).  `module`
    carries linear_0 .. linear_{num_concat-1}.  For WOQ linears without act-order the reference
    dequantises, concatenates and quantises again with the concatenated scales and zero points;
    as every row keeps its own scale and zero point that gives back the same codes, so here the
    codes, scales and zero points are concatenated directly.  forward(x) returns the
    concatenated output [.., sum of out_features]; otherwise (act-order, or linears that are not
    WOQ) a tuple of the separate outputs, as the reference does."""

    def __init__(self, module, tpp=False, woq=True):
        super().__init__()
        from ...nn.modules.weight_only_quantization import WeightOnlyQuantizedLinear

        assert hasattr(module, "linear_0") and hasattr(module, "num_concat")
        self.num_concat = module.num_concat
        self.tpp, self.woq = tpp, woq
        linears = [getattr(module, f"linear_{i}") for i in range(self.num_concat)]
        self.concat_linear = None
        fusable = woq and all(isinstance(m, WeightOnlyQuantizedLinear) for m in linears) and all(
            m._op_context.get_g_idx() is None for m in linears)
        if fusable:
            qw, s, z, b, meta = _stack_quantized(linears)
            first = linears[0]
            shell = nn.Module()
            shell.in_features, shell.out_features, shell.bias = meta["k"], qw.shape[0], None
            self.concat_linear = WeightOnlyQuantizedLinear._init_cls(
                shell, meta["dtype"], qw, s, z, b, None, meta["group_size"], meta["lowp_mode"],
                meta["act_quant_mode"], first._cache_weight_for_large_batch, False)
            self.out_features = [m.out_features for m in linears]
        else:
            for i, m in enumerate(linears):
                setattr(self, f"linear_{i}", m)

    def forward(self, x):
        if self.concat_linear is not None:
            return self.concat_linear(x)
        return tuple(getattr(self, f"linear_{i}")(x) for i in range(self.num_concat))


# reference names
_IPEXConcatLinearCPU = _IPEXConcatLinear
_IPEXlinearSiluCPU = _IPEXlinearSilu
_IPEXlinearReluCPU = _IPEXlinearRelu
_IPEXlinearMulCPU = _IPEXlinearMul
_IPEXlinearAddCPU = _IPEXlinearAdd
_IPEXlinearAddAddCPU = _IPEXlinearAddAdd
_IPEXlinearNewGeluCPU = _IPEXlinearNewGelu
_IPEXlinearGeluCPU = _IPEXlinearGelu
_IPEXlinearSiluMulCPU = _IPEXlinearSiluMul
