"""Host-side checks of bench.py that need no GPU: the byte accounting behind the reported
GB/s, the configuration table of `--configs`, and the reference arm's JSON line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_weight_bytes_match_the_algorithmic_figure():
    # INT4 g128: nibbles + fp16 scale + u8 zero point per group
    assert bench.weight_bytes(4096, 4096) == 8_388_608 + 262_144 + 131_072
    layer = bench.full_layer_weight_bytes()
    elts = 10240 * 8192 + 8192 * 8192 + 57344 * 8192 + 8192 * 28672
    assert layer == int(elts * 0.5234375)


def test_layer_shapes_shard_columns_and_rows():
    for p in (1, 2, 4, 8):
        shapes = {name: (n, k, kind) for name, n, k, kind in bench.layer_shapes(p)}
        assert shapes["qkv"] == (10240 // p, 8192, "col")
        assert shapes["o_proj"] == (8192, 8192 // p, "row")
        assert shapes["gate_up"] == (57344 // p, 8192, "col")
        assert shapes["down_proj"] == (8192, 28672 // p, "row")
        # a row-parallel shard keeps whole quantisation groups
        assert (8192 // p) % bench.GROUP == 0 and (28672 // p) % bench.GROUP == 0


def test_config_table_covers_every_benchmark_configuration():
    configs = {c[0].split("-")[0] for c in bench.CONFIG_CASES}
    assert configs == {"c1", "c2", "c3", "c5"}  # c4 (the MoE layer) is built apart from the table
    assert bench.MOE_TOKENS == (1, 16, 256, 4096)
    for config, name, n, k, kind, fusion, ms in bench.CONFIG_CASES:
        assert kind in ("int4", "int8") and fusion in ("none", "silu_mul", "add")
        assert k % 128 == 0 and n % 64 == 0 and len(ms) >= 3
        if fusion == "silu_mul":
            assert n % 128 == 0  # gate and up halves, 64-row tiles each
    c1 = [c for c in bench.CONFIG_CASES if c[0].startswith("c1")][0]
    assert c1[2:4] == (4096, 4096) and c1[6] == (1, 4, 32, 256)


def test_reference_arm_prints_one_json_line():
    env = dict(os.environ, OMP_NUM_THREADS="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
