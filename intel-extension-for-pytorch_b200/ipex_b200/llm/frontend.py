"""ipex.llm.optimize for the WOQ path.

The weight-only-quantisation branch of the reference's optimize()
(intel_extension_for_pytorch/transformers/optimize.py:2074-2295): every nn.Linear except the
language-model head becomes a WeightOnlyQuantizedLinear, either by quantising its floating
weight (quantization/_quantize.py:436-467 convert()) or from a low-precision checkpoint
(utils/weight_only_quantization.py:224-375), and the linears of Llama-style blocks are fused the
way the reference's model rewrites do it (models/reference/modules/decoder.py:18-66,
cpu/fusions/linear_fusion.py:296-492): q / k / v projections into one concatenated linear, gate
and up projections into one kernel with the silu*mul epilogue, residual adds into the o / down
projections where the block exposes them."""
import copy
import types

import torch
from torch import nn

from ..nn.modules.weight_only_quantization import WeightOnlyQuantizedLinear
from ..quantization import QConfigWoq


def convert(model: nn.Module, qconfig, skip=("lm_head",)):
    """Replace every nn.Linear (except names in `skip`) by its weight-only-quantised version."""
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear) and name not in skip:
            child.qconfig = qconfig
            setattr(model, name, WeightOnlyQuantizedLinear.from_float(child))
        else:
            convert(child, qconfig, skip)
    return model


class _ConcatSlice(nn.Module):
    """Stands where one of several concatenated projections stood (q_proj / k_proj / v_proj of an
    attention block whose forward calls them one after the other on the same tensor): the first
    call on a new input runs the concatenated linear once, the others return their columns of
    that result."""

    def __init__(self, owner, index):
        super().__init__()
        object.__setattr__(self, "_owner", owner)  # not a sub-module: the owner holds the weights
        self.index = index
        self.in_features = owner.concat.concat_linear.in_features
        self.out_features = owner.concat.out_features[index]

    def forward(self, x):
        return self._owner.column_block(x, self.index)


class _ConcatOwner(nn.Module):
    def __init__(self, concat):
        super().__init__()
        self.concat = concat
        bounds = [0]
        for n in concat.out_features:
            bounds.append(bounds[-1] + n)
        self.bounds = bounds
        self._x = None  # the input the cached output belongs to, held so its storage cannot be reused
        self._version = -1
        self._out = None
        self._served = 0

    def column_block(self, x, index):
        fresh = (self._x is None or x.data_ptr() != self._x.data_ptr() or x._version != self._version
                 or x.shape != self._x.shape or x.dtype != self._x.dtype or (self._served >> index) & 1)
        if fresh:
            self._out = self.concat(x)
            self._x, self._version, self._served = x, x._version, 0
        self._served |= 1 << index
        out = self._out[..., self.bounds[index]:self.bounds[index + 1]]
        if self._served == (1 << len(self.concat.out_features)) - 1:
            self._x, self._out = None, None  # every projection has been handed out
        return out


def _is_woq(m):
    return isinstance(m, WeightOnlyQuantizedLinear)


def fuse_llama_style_blocks(model: nn.Module):
    """In place.  A module with WOQ `q_proj`, `k_proj`, `v_proj` gets them served by one
    concatenated linear; a module with WOQ `gate_proj`, `up_proj`, `down_proj` and a SiLU `act_fn`
    (the Llama / Mistral / Qwen MLP) computes down_proj(silu(gate) * up) with gate and up in one
    kernel.  Modules that do not match are left alone."""
    from ..transformers.fusions.linear_fusion import _IPEXConcatLinear, _IPEXlinearFusedGateUp

    for mod in list(model.modules()):
        q, k, v = (getattr(mod, n, None) for n in ("q_proj", "k_proj", "v_proj"))
        if _is_woq(q) and _is_woq(k) and _is_woq(v) and q._op_context.get_g_idx() is None and not q.bias:
            holder = nn.Module()
            holder.linear_0, holder.linear_1, holder.linear_2, holder.num_concat = q, k, v, 3
            concat = _IPEXConcatLinear(holder)
            if concat.concat_linear is not None:
                owner = _ConcatOwner(concat)
                mod.qkv_concat = owner
                mod.q_proj, mod.k_proj, mod.v_proj = (_ConcatSlice(owner, i) for i in range(3))
        g, u, d = (getattr(mod, n, None) for n in ("gate_proj", "up_proj", "down_proj"))
        act = getattr(mod, "act_fn", None)
        silu = isinstance(act, nn.SiLU) or getattr(act, "__name__", "") == "silu"
        if _is_woq(g) and _is_woq(u) and _is_woq(d) and silu and not g.bias and not u.bias and (
                g._lowp_mode == 2 or (g._lowp_mode == 3 and g._act_quant_mode in (0, 2, 4, 6) and g.dtype == 1)):
            mod.gate_up_fused = _IPEXlinearFusedGateUp.from_linears(g, u)
            del mod.gate_proj, mod.up_proj
            mod.forward = types.MethodType(lambda self, x: self.down_proj(self.gate_up_fused(x)), mod)
    from ..transformers.fusions.linear_fusion import _IPEXlinearAdd

    for mod in list(model.modules()):
        # a decoder layer in the Hugging Face layout: the residual adds after attention and after
        # the MLP can run in the epilogues of o_proj and down_proj.  The layer's own forward is
        # not replaced; a forward that knows these attributes (the reference's decoder-layer
        # rewrite names them the same way, models/reference/modules/decoder.py:18-66) uses them.
        attn, mlp = getattr(mod, "self_attn", None), getattr(mod, "mlp", None)
        if attn is not None and mlp is not None and _is_woq(getattr(attn, "o_proj", None)) and _is_woq(
                getattr(mlp, "down_proj", None)):
            mod.mha_linear_add = _IPEXlinearAdd(attn.o_proj)
            mod.mlp_linear_add = _IPEXlinearAdd(mlp.down_proj)
    return model


def optimize(model, dtype=torch.bfloat16, quantization_config=None, inplace=False, device="cuda",
             low_precision_checkpoint=None, fuse=True, **kwargs):
    """quantization_config: a mapping from get_weight_only_quant_qconfig_mapping().
    low_precision_checkpoint: (state_dict, quant_config) of a GPTQ / AWQ / FP8 checkpoint, as the
    reference takes it; the linears are then built from the checkpoint's tensors."""
    assert quantization_config is not None, "this build of llm.optimize covers weight-only quantisation"
    qconfig = getattr(quantization_config, "global_qconfig", quantization_config)
    assert isinstance(qconfig, QConfigWoq), "quantization_config must come from get_weight_only_quant_qconfig_mapping"
    if not inplace:
        model = copy.deepcopy(model)
    model = model.eval()
    if low_precision_checkpoint is not None:
        from ..utils.weight_only_quantization import _convert_woq_with_low_precision_checkpoint

        state_dict, quant_config = low_precision_checkpoint
        _convert_woq_with_low_precision_checkpoint(model, quantization_config, state_dict, quant_config, inplace=True)
    else:
        convert(model, qconfig)
    model = model.to(device=device, dtype=dtype)
    if fuse:
        fuse_llama_style_blocks(model)
    return model
