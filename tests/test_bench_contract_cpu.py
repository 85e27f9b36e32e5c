"""CPU: the pieces of bench.py that decide what the JSON line says about the workload (no timing, no GPU)."""
import argparse
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _args(**kw):
    base = dict(path="auto", unfused=False, shard="batch", config=5)
    base.update(kw)
    return argparse.Namespace(**base)


def test_flops_per_cell_counts_the_necessary_contractions(bench):
    # forward: S for max/avg (+ S again for the compression when there are attention channels);
    # backward: S for the attention gradients, gF1, gF2 -- each 2*C flop per cell
    assert bench.flops_per_cell(dict(Kc=4, bwd=True)) == 5 * 2 * bench.C_FEAT
    assert bench.flops_per_cell(dict(Kc=4, bwd=False)) == 2 * 2 * bench.C_FEAT
    assert bench.flops_per_cell(dict(Kc=0, bwd=False)) == 1 * 2 * bench.C_FEAT


def test_workload_config_of_the_headline_configuration(bench):
    cfg = dict(bench.CONFIGS[5])
    c = bench.workload_config(_args(), cfg, 1)
    assert c["workload"] == cfg["name"] and c["path"] == "level"
    assert c["cells_per_step"] == 8 * (135 * 240) ** 2 == 8398080000
    assert c["flop_per_cell"] == 2560
    assert c["sharding"] == "batch x rows = 1 x 1" and c["l2"] == "inputs larger than L2"


@pytest.mark.parametrize("world, prefer, text", [(2, "batch", "2 x 1"), (8, "batch", "8 x 1"), (3, "batch", "1 x 3"),
                                                 (6, "batch", "2 x 3"), (4, "rows", "1 x 4")])
def test_workload_config_names_the_partition_the_sharding_module_makes(bench, world, prefer, text):
    from separableflowthesis_b200 import sharding
    cfg = dict(bench.CONFIGS[5])
    c = bench.workload_config(_args(shard=prefer), cfg, world)
    assert c["sharding"] == "batch x rows = " + text
    sh = sharding.make_shard(cfg["B"], cfg["H"], world, 0, prefer=prefer)
    assert c["sharding"] == f"batch x rows = {sh.g_batch} x {sh.g_rows}"
    # the shards' cells add up to the workload's
    cells = 0
    for r in range(world):
        s = sharding.make_shard(cfg["B"], cfg["H"], world, r, prefer=prefer)
        cells += (s.b1 - s.b0) * (s.r1 - s.r0) * cfg["W"] * cfg["H"] * cfg["W"]
    assert cells == c["cells_per_step"]


def test_path_resolution(bench):
    assert bench.resolve_path(_args(), dict(Kc=4)) == "level"
    assert bench.resolve_path(_args(unfused=True), dict(Kc=4)) == "ops"
    assert bench.resolve_path(_args(), dict(Kc=0)) == "ops"
    assert bench.resolve_path(_args(path="lookup"), dict(Kc=4)) == "lookup"
