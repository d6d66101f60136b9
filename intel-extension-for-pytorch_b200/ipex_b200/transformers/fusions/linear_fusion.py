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

    def __init__(self, op_context, out_features):
        super().__init__()
        self._op_context = op_context
        self.out_features = out_features

    @classmethod
    def from_quantized(cls, qweight, dtype, shape, scales, zero_points, group_size, lowp_mode, act_quant_mode=-1):
        from ..._ops import load_ops

        load_ops()
        ctx = torch.ops.ipex_prepack.weight_only_qlinear_prepack_gate_up(
            qweight, int(dtype), list(shape), scales, zero_points, None, group_size, int(lowp_mode),
            int(act_quant_mode))
        return cls(ctx, shape[0] // 2)

    def forward(self, x):
        return torch.ops.torch_ipex.woq_linear_silu_mul(x, self._op_context.get_data_handle())


# reference names
_IPEXlinearSiluCPU = _IPEXlinearSilu
_IPEXlinearReluCPU = _IPEXlinearRelu
_IPEXlinearMulCPU = _IPEXlinearMul
_IPEXlinearAddCPU = _IPEXlinearAdd
_IPEXlinearAddAddCPU = _IPEXlinearAddAdd
_IPEXlinearNewGeluCPU = _IPEXlinearNewGelu
_IPEXlinearGeluCPU = _IPEXlinearGelu
_IPEXlinearSiluMulCPU = _IPEXlinearSiluMul
