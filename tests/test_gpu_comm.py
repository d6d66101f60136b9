"""The tensor-parallel exchange fused into the decode kernel (woq_b200_linear_allreduce /
woq_b200_linear_allgather), through the C ABI.

One GPU: a single-rank comm goes through the same epilogue code (stores, stamps, epochs) and
must reproduce the plain linear bit for bit.  An all-gather leaves the other ranks' columns to
the next fused call or to Comm.fence(); the workers read a gathered tensor only after one.  Two or more GPUs: one process per GPU
(tests/comm_worker.py); the row-parallel result is checked against the oracle's
row_parallel_linear and must be bit-identical on all ranks, the gathered column-parallel
result must be bit-identical to the unsharded linear.
"""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import woq_oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, make_acts, make_int4_layer, to_device_layer

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def capi():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ipex_b200 import _capi

    _capi.lib()
    return _capi


def test_single_rank_comm_reproduces_the_plain_linear(capi):
    n, k, g = 448, 1024, 128
    layer = make_int4_layer(n, k, g, seed=5)
    qw, s, z, _ = to_device_layer(layer, "cuda")
    ctx = capi.WoqContext(qw, s, z, None, n, k, capi.DTYPE_INT4, g, capi.LOWP_BF16)
    comm = capi.Comm(0, 1, n, 16 * n * 2, "cuda")
    bias = torch.linspace(-1, 1, n, device="cuda")
    for m in (1, 4, 9, 16):  # several epochs on one comm, both buffer parities
        x = bf16_tensor(make_acts(m, k, seed=m), "cuda")
        resid = bf16_tensor(make_acts(m, n, seed=50 + m), "cuda")
        plain = ctx.linear(x)
        # reduce of one partial = bf16 of it; then + bias, rounded again
        want = (plain.float() + bias).bfloat16()
        got = ctx.linear_allreduce(comm, x, bias=bias)
        assert torch.equal(got, want)
        got = ctx.linear_allreduce(comm, x, capi.FUSE_ADD, [resid])
        assert torch.equal(got, ctx.linear(x, capi.FUSE_ADD, [resid]))
        gathered = ctx.linear_allgather(comm, x, capi.FUSE_GELU_TANH)
        torch.cuda.synchronize()
        assert torch.equal(gathered, ctx.linear(x, capi.FUSE_GELU_TANH))
    ctx.workspace(16).status()
    comm.close()


def test_comm_argument_errors(capi):
    layer = make_int4_layer(128, 256, 128, seed=1, bias=True)
    qw, s, z, b = to_device_layer(layer, "cuda")
    with_bias = capi.WoqContext(qw, s, z, b, 128, 256, capi.DTYPE_INT4, 128, capi.LOWP_BF16)
    comm = capi.Comm(0, 1, 128, 4096, "cuda")
    x = bf16_tensor(make_acts(2, 256, seed=0), "cuda")
    with pytest.raises(capi.WoqError):   # bias belongs after the reduction
        with_bias.linear_allreduce(comm, x)
    with pytest.raises(capi.WoqError):   # more than 16 tokens
        with_bias.linear_allgather(comm, bf16_tensor(make_acts(17, 256, seed=0), "cuda"))
    with pytest.raises(capi.WoqError):   # gathered tensor larger than the gather area
        with_bias.linear_allgather(comm, bf16_tensor(make_acts(16, 256, seed=0), "cuda"), gather_offset=2048)
    comm.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_on_separate_gpus(capi, world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import tests.comm_worker as W

    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "comm_worker.py"), str(tmp_path)],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{outs[r][-3000:]}"
    ranks = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]

    # row-parallel: all ranks hold the same bits, and they are the oracle's
    layer = make_int4_layer(W.N_ROW, W.K_ROW, W.G, seed=77)
    ks, gs = W.K_ROW // world, W.K_ROW // world // W.G
    shards = [(layer["qw"][:, r * ks // 2:(r + 1) * ks // 2], layer["s16"][:, r * gs:(r + 1) * gs],
               layer["z"][:, r * gs:(r + 1) * gs]) for r in range(world)]
    bias = np.linspace(-1, 1, W.N_ROW).astype(np.float32)
    for m, seed in W.CASES_ROW:
        x = make_acts(m, W.K_ROW, seed=seed)
        for key in (f"row_m{m}", f"row_add_m{m}"):
            for r in range(1, world):
                np.testing.assert_array_equal(ranks[r][key], ranks[0][key])
        ref = O.row_parallel_linear(x, [s[0] for s in shards], [s[1] for s in shards], [s[2] for s in shards],
                                    bias, O.WOQ_DTYPE_INT4, W.G)
        mx, mr = O.parity_metrics(ranks[0][f"row_m{m}"], ref)
        assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)
        ref_nb = O.row_parallel_linear(x, [s[0] for s in shards], [s[1] for s in shards], [s[2] for s in shards],
                                       None, O.WOQ_DTYPE_INT4, W.G)
        ref_add = O.rne_bf16(ref_nb + make_acts(m, W.N_ROW, seed=100 + seed))
        mx, mr = O.parity_metrics(ranks[0][f"row_add_m{m}"], ref_add)
        assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)

    # column-parallel: the gathered tensor equals the unsharded linear on one GPU, bit for bit
    col = make_int4_layer(W.N_COL, W.K_COL, W.G, seed=78, bias=True)
    qw, s, z, b = to_device_layer(col, "cuda")
    whole = capi.WoqContext(qw, s, z, b, W.N_COL, W.K_COL, capi.DTYPE_INT4, W.G, capi.LOWP_BF16)
    gate_up = capi.WoqContext(qw, s, z, None, W.N_COL, W.K_COL, capi.DTYPE_INT4, W.G, capi.LOWP_BF16,
                              layout_flags=capi.LAYOUT_GATE_UP)
    for m, seed in [(1, 10), (7, 11), (16, 12)]:
        x = bf16_tensor(make_acts(m, W.K_COL, seed=seed), "cuda")
        want = bf16_numpy(whole.linear(x))
        want_act = bf16_numpy(gate_up.linear(x, capi.FUSE_SILU_MUL))
        for r in range(world):
            np.testing.assert_array_equal(ranks[r][f"col_m{m}"], want)
            np.testing.assert_array_equal(ranks[r][f"gateup_m{m}"], want_act)
