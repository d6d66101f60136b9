"""Shared helpers of the tests: seeded synthetic layers quantised by the oracle's restatement
of the reference quantiser, and conversions between numpy and torch bf16."""
import numpy as np
import torch

from oracle import woq_oracle as O


def bf16_tensor(a: np.ndarray, device="cpu") -> torch.Tensor:
    """float32 array of bf16-representable values -> torch bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).to(device)


def bf16_numpy(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def make_int4_layer(n, k, group_size, seed, sym=False, std=0.02, bias=False):
    """W ~ N(0, std) quantised asymmetric INT4; scales handed on as fp16 (the canonical
    triple q, s16, zp)."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * std).astype(np.float32)
    if group_size > 0:
        qw, s, z = O.quantize_per_block(w, O.WOQ_DTYPE_INT4, group_size, sym)
    else:
        qw, s, z = O.quantize_per_channel(w, O.WOQ_DTYPE_INT4, sym)
        s = s[:, None]
        z = None if z is None else z[:, None]
    s16 = s.astype(np.float16)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32) if bias else None
    return dict(qw=qw, s16=s16, z=z, bias=b, n=n, k=k, g=group_size)


def make_acts(m, k, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return O.rne_bf16((rng.standard_normal((m, k)) * scale).astype(np.float32))


def to_device_layer(layer, device):
    qw = torch.from_numpy(layer["qw"]).to(device)
    s = torch.from_numpy(layer["s16"]).to(device)
    z = None if layer["z"] is None else torch.from_numpy(layer["z"]).to(device)
    b = None if layer["bias"] is None else torch.from_numpy(layer["bias"]).to(device)
    return qw, s, z, b
