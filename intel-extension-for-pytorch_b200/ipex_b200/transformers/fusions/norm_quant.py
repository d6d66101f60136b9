"""RMSNorm fused with the activation quantiser of the INT8-compute WOQ linears behind it.

A B200-side fusion: in the reference the norm (stock RMSNorm of the model rewrites,
transformers/models/reference/modules/decoder.py) and the per-token activation quantiser (the
prologue of the INT8 kernel, csrc/cpu/aten/utils/woq_dynamic_quant.h:1526-1750) are separate steps,
and every linear that reads the normalised activations quantises them again.  Here one kernel
normalises and quantises a token row, and the q / k / v (or gate / up) linears all consume the
same codes: one pass over the activations instead of one per linear plus the norm's own."""
import torch
from torch import nn

FUSE_NONE, FUSE_SILU_MUL = 0x0, 0x100
_PER_TOKEN_MODES = (2, 6)  # WoqActQuantMode.PER_BATCH, PER_BATCH_SYM


class _IPEXRmsNormQuantLinears(nn.Module):
    """norm: a module with `weight` [K] and `eps` / `variance_epsilon` (nn.RMSNorm, LlamaRMSNorm).
    linears: WeightOnlyQuantizedLinear modules with INT8 weights, WoqLowpMode.INT8 and a per-token
    activation mode, all the same mode (_IPEXlinearFusedGateUp modules are accepted too: they
    apply silu * mul).  forward(x) returns the tuple of their outputs on rmsnorm(x)."""

    def __init__(self, norm, linears):
        super().__init__()
        self.weight = norm.weight
        eps = getattr(norm, "eps", None)
        self.eps = float(eps if eps is not None else getattr(norm, "variance_epsilon", 1e-6))
        self.linears = nn.ModuleList(linears)
        modes = {int(getattr(m, "_act_quant_mode", -1)) for m in linears}
        assert len(modes) == 1 and modes <= set(_PER_TOKEN_MODES), (
            f"the linears must share one per-token activation mode (2 or 6), got {sorted(modes)}")
        self.act_quant_mode = modes.pop()
        for m in linears:
            assert int(getattr(m, "_lowp_mode", -1)) == 3, "the fused quantiser feeds INT8-compute linears"

    def forward(self, x):
        qa, sa, zpa = torch.ops.torch_ipex.woq_rmsnorm_quant(x, self.weight, self.eps, self.act_quant_mode)
        outs = []
        for m in self.linears:
            fusion = FUSE_SILU_MUL if getattr(m, "is_gate_up", False) else FUSE_NONE
            outs.append(torch.ops.torch_ipex.woq_linear_prequant(qa, sa, zpa, m._op_context.get_data_handle(),
                                                                 fusion, []))
        return tuple(outs)
