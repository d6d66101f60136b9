"""CPU-only checks of the Python surface: the extension loads, the operators exist with the
reference's schemas, and the tensor-parallel helper reduces over a 2-rank gloo group."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


@pytest.fixture(scope="module")
def ipex():
    import importlib.util

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location(
        "build_ext", os.path.join(root, "intel-extension-for-pytorch_b200", "build_ext.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    import ipex_b200

    ipex_b200.load_ops()
    return ipex_b200


def test_operator_schemas(ipex):
    s = str(torch.ops.torch_ipex.ipex_woq_linear.default._schema)
    assert s == "torch_ipex::ipex_woq_linear(Tensor input, Tensor W_prepack) -> Tensor"
    for name in ("woq_linear_gelu", "woq_linear_new_gelu", "woq_linear_relu", "woq_linear_silu"):
        assert "(Tensor input, Tensor W_prepack) -> Tensor" in str(getattr(torch.ops.torch_ipex, name).default._schema)
    for name in ("woq_linear_add", "woq_linear_add_add", "woq_linear_mul"):
        assert "Tensor[] others" in str(getattr(torch.ops.torch_ipex, name).default._schema)
    s = str(torch.ops.torch_ipex.woq_linear.default._schema)
    assert "str weight_dtype, int[] weight_shape, Tensor[] weight_scales" in s
    s = str(torch.ops.ipex_prepack.weight_only_qlinear_prepack.default._schema)
    assert "int W_dtype, int[] W_shape, Tensor scales, Tensor? zero_points" in s
    assert "WoqLinearOpContext" in s
    s = str(torch.ops.ipex_prepack.woq_linear_pack_weight.default._schema)
    assert "-> (Tensor, Tensor[], Tensor[]?, Tensor[]?, Tensor?)" in s and "str W_dtype" in s
    s = str(torch.ops.ipex_prepack.weight_only_qlinear_prepack_int4.default._schema)
    assert "int weight_format=0" in s


def test_cpu_tensors_are_refused_not_computed(ipex):
    """There is no CPU kernel behind these operators."""
    x = torch.randn(2, 64).bfloat16()
    h = torch.zeros(1, dtype=torch.int64)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.torch_ipex.ipex_woq_linear(x, h)


def test_surface_names(ipex):
    q = ipex.quantization
    assert int(q.WoqWeightDtype.INT4) == 2 and int(q.WoqLowpMode.INT8) == 3
    assert int(q.WoqActQuantMode.PER_BATCH_SYM) == 6
    from ipex_b200.llm.quantization import IPEXWeightOnlyQuantizedLinear, QuantDtype, QuantMethod
    from ipex_b200.nn.modules import IpexWoqLinearAllreduce, WeightOnlyQuantizedLinear, WoqWeightFormat

    assert "cuda" in IPEXWeightOnlyQuantizedLinear.module_mapping
    assert int(WoqWeightFormat.AWQ_FORMAT) == 2 and int(QuantMethod.AWQ_GEMM) == 1 and int(QuantDtype.INT4) == 0
    assert issubclass(IpexWoqLinearAllreduce, WeightOnlyQuantizedLinear)


def _tp_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "intel-extension-for-pytorch_b200"))
    from ipex_b200.nn.modules.weight_only_quantization import all_reduce_and_bias_add

    torch.manual_seed(0)
    full = torch.randn(4, 8, 32)           # [rank, M, N] partial outputs of a row-parallel layer
    bias = torch.randn(32)
    out = all_reduce_and_bias_add(None, bias, full[rank].clone())
    expect = full[:world].sum(0) + bias
    ret[rank] = bool(torch.allclose(out, expect, atol=1e-6))
    dist.destroy_process_group()


def test_row_parallel_reduce_two_ranks_gloo(ipex):
    world = 2
    mgr = mp.get_context("spawn").Manager()  # no fork of this multi-threaded process
    ret = mgr.dict()
    with socket.socket() as sock:  # a free port, not a guessed one
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    mp.spawn(_tp_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world))


def test_checkpoint_tensor_conversions_on_cpu(ipex):
    """The low-precision checkpoint loader's tensor conversions (no GPU needed): a GPTQ layer
    with act-order comes out as plain nibbles with scales / zero points per output row, group
    sizes are read off the tensors, and a block-scaled FP8 layer gets one scale per row and K block."""
    import numpy as np

    from ipex_b200.nn.modules.weight_only_quantization import WoqWeightFormat
    from ipex_b200.utils.weight_only_quantization import _get_linear_parameters, _gptq_to_plain
    from oracle import woq_oracle as O

    n, k, g = 64, 256, 64
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, (n, k)).astype(np.uint32)
    qT = q.T.reshape(k // 8, 8, n)
    gq = np.zeros((k // 8, n), dtype=np.uint32)
    for j in range(8):
        gq |= qT[:, j, :] << (4 * j)
    z = rng.integers(1, 16, (n, k // g))
    zz = (z.T - 1) % 16
    gz = np.zeros((k // g, n // 8), dtype=np.uint32)
    for j in range(8):
        gz |= zz[:, j::8].astype(np.uint32) << (4 * j)
    s = (rng.random((k // g, n)) * 0.01 + 0.001).astype(np.float16)
    tq, ts, tz = (torch.from_numpy(gq.view(np.int32)), torch.from_numpy(s), torch.from_numpy(gz.view(np.int32)))
    # the oracle's reading of the same checkpoint words
    np.testing.assert_array_equal(O.gptq_unpack_int32_rows(gq).T, q.astype(np.uint8))
    plain, ps, pz = _gptq_to_plain(tq, ts.clone(), tz.clone())
    np.testing.assert_array_equal(plain.numpy(), O.pack_nibbles(q.astype(np.uint8)))
    np.testing.assert_array_equal(ps.float().numpy(), s.T.astype(np.float32))
    np.testing.assert_array_equal(pz.float().numpy(), z.astype(np.float32))

    g_idx = torch.from_numpy(rng.permutation(np.arange(k) // g).astype(np.int32))
    sd = {"fc.qweight": tq, "fc.scales": ts, "fc.qzeros": tz, "fc.g_idx": g_idx}
    w, sc, zp, b, group, gi, fmt = _get_linear_parameters("fc", sd, {"quant_method": "gptq"}, True)
    assert group == g and gi is not None and fmt == WoqWeightFormat.PLAIN_FORMAT and w.dtype == torch.uint8
    w, sc, zp, b, group, gi, fmt = _get_linear_parameters("fc", sd, {"quant_method": "gptq"}, False)
    assert group == g and gi is None and fmt == WoqWeightFormat.GPTQ_FORMAT and w.dtype == torch.int32
    natural = dict(sd, **{"fc.g_idx": torch.arange(k, dtype=torch.int32) // g})
    assert _get_linear_parameters("fc", natural, {"quant_method": "gptq"}, True)[5] is None

    w8 = torch.randn(200, 256).to(torch.float8_e4m3fn)
    sinv = torch.rand(2, 2) + 0.5
    w, sc, zp, b, group, gi, fmt = _get_linear_parameters(
        "fc", {"fc.weight": w8, "fc.weight_scale_inv": sinv}, {"quant_method": "fp8", "weight_block_size": [128, 128]}, None)
    assert w.dtype == torch.uint8 and sc.shape == (200, 2) and group == 128 and zp is None
    assert torch.equal(sc[:128], sinv[0].expand(128, 2)) and torch.equal(sc[128:], sinv[1].expand(72, 2))
    # a layer the checkpoint keeps in floating point
    assert _get_linear_parameters("head", {"head.weight": torch.ones(4, 4)}, {"quant_method": "awq"}, None)[1] is None
