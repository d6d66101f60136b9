"""One rank of the fused tensor-parallel exchange test: run by tests/test_gpu_comm.py as
`python tests/comm_worker.py <out_dir>` with RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT set,
one process per GPU.  Writes this rank's outputs to <out_dir>/rank<r>.npz."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "intel-extension-for-pytorch_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

from tests.helpers import bf16_numpy, bf16_tensor, make_acts, make_int4_layer  # noqa: E402

CASES_ROW = [(1, 0), (5, 1), (16, 2), (3, 3)]      # (tokens, seed): several epochs on one comm
N_ROW, K_ROW, G = 320, 2048, 128                   # row-parallel: K sharded
N_COL, K_COL = 1024, 512                           # column-parallel: N sharded (gate/up: 2 x 512)


def main():
    out_dir = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    import datetime

    # only carries the 64-byte handles; a lost peer ends this rank instead of hanging it
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    from ipex_b200 import _capi as capi

    dev = torch.device("cuda", rank)
    comm = capi.Comm(rank, world, max(N_ROW, N_COL), 16 * N_COL * 2 * 2, dev)
    res = {}

    # ---- row-parallel + all-reduce (+ bias, + residual) ----
    layer = make_int4_layer(N_ROW, K_ROW, G, seed=77)
    ks = K_ROW // world
    gs = ks // G
    qw = torch.from_numpy(layer["qw"][:, rank * ks // 2:(rank + 1) * ks // 2].copy()).to(dev)
    s = torch.from_numpy(layer["s16"][:, rank * gs:(rank + 1) * gs].copy()).to(dev)
    z = torch.from_numpy(layer["z"][:, rank * gs:(rank + 1) * gs].copy()).to(dev)
    ctx = capi.WoqContext(qw, s, z, None, N_ROW, ks, capi.DTYPE_INT4, G, capi.LOWP_BF16)
    bias = torch.from_numpy(np.linspace(-1, 1, N_ROW).astype(np.float32)).to(dev)
    dist.barrier()  # the kernels wait about 2 s for a peer, not for its start-up
    for m, seed in CASES_ROW:
        x = make_acts(m, K_ROW, seed=seed)
        xs = bf16_tensor(x[:, rank * ks:(rank + 1) * ks].copy(), dev)
        y = ctx.linear_allreduce(comm, xs, bias=bias)
        res[f"row_m{m}"] = bf16_numpy(y)
        resid = bf16_tensor(make_acts(m, N_ROW, seed=100 + seed), dev)
        y2 = ctx.linear_allreduce(comm, xs, capi.FUSE_ADD, [resid])
        res[f"row_add_m{m}"] = bf16_numpy(y2)
    ctx.workspace(16).status()

    # ---- column-parallel + all-gather, plain and gate/up silu_mul ----
    col = make_int4_layer(N_COL, K_COL, G, seed=78, bias=True)
    ns = N_COL // world
    qw = torch.from_numpy(col["qw"][rank * ns:(rank + 1) * ns].copy()).to(dev)
    s = torch.from_numpy(col["s16"][rank * ns:(rank + 1) * ns].copy()).to(dev)
    z = torch.from_numpy(col["z"][rank * ns:(rank + 1) * ns].copy()).to(dev)
    b = torch.from_numpy(col["bias"][rank * ns:(rank + 1) * ns].copy()).to(dev)
    cctx = capi.WoqContext(qw, s, z, b, ns, K_COL, capi.DTYPE_INT4, G, capi.LOWP_BF16)
    # gate/up: this rank's gate rows then its up rows
    half = N_COL // 2
    hs = half // world
    rows = np.r_[rank * hs:(rank + 1) * hs, half + rank * hs:half + (rank + 1) * hs]
    gqw = torch.from_numpy(col["qw"][rows].copy()).to(dev)
    gsc = torch.from_numpy(col["s16"][rows].copy()).to(dev)
    gz = torch.from_numpy(col["z"][rows].copy()).to(dev)
    gctx = capi.WoqContext(gqw, gsc, gz, None, 2 * hs, K_COL, capi.DTYPE_INT4, G, capi.LOWP_BF16,
                           layout_flags=capi.LAYOUT_GATE_UP)
    off2 = 16 * N_COL * 2
    torch.cuda.synchronize()
    dist.barrier()
    for m, seed in [(1, 10), (7, 11), (16, 12)]:
        x = bf16_tensor(make_acts(m, K_COL, seed=seed), dev)
        full = cctx.linear_allgather(comm, x, gather_offset=0)
        act = gctx.linear_allgather(comm, x, capi.FUSE_SILU_MUL, gather_offset=off2)
        # the first gather was completed by the second call; the second one by the fence
        comm.fence()
        torch.cuda.synchronize()
        comm.status()
        res[f"col_m{m}"] = bf16_numpy(full)
        res[f"gateup_m{m}"] = bf16_numpy(act)
        # an exchange between two gathers into the same place, as the API asks
        ctx.linear_allreduce(comm, bf16_tensor(np.zeros((1, ks), np.float32), dev))
    cctx.workspace(16).status()
    torch.cuda.synchronize()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **res)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
