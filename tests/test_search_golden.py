"""The product's generic rTile policy returns exactly what the reference's search returns.

Golden vectors: tests/golden/search_golden.json, recorded from the reference itself by
tests/golden/gen_search_golden.py (README shapes M0-M13, shard shapes, ragged, skinny, primes,
tiny shapes, other element widths, a modified device)."""
import os
import sys
import types
from pathlib import Path

import pytest

from conftest import hint_record
from mlir_roller_b200 import analyze, arch, utils

# a checkout of the reference next to this repository (or named by MLIR_ROLLER_REFERENCE)
REFERENCE_SRC = Path(os.environ.get("MLIR_ROLLER_REFERENCE",
                                    Path(__file__).resolve().parents[2] / "reference")) / "src"


def _cases(golden):
    return golden["searches"]


def test_every_golden_search_matches(golden_search):
    assert len(golden_search["searches"]) >= 100
    for s in _cases(golden_search):
        dev = arch.CUDA(**s.get("arch_overrides", {}))
        cfg = analyze.MatmulConfig(s["M"], s["N"], s["K"], s.get("el_bits", 32))
        hints = analyze.get_roller_hints(cfg, dev, topk=s["topk"])
        assert [hint_record(h) for h in hints] == s["hints"], (s["M"], s["N"], s["K"], s["topk"])


def test_readme_shapes_top_hint(golden_search):
    # every README shape ranks block [128,128] / thread [16,8] / rstep 32 first on the A100 model
    for s in _cases(golden_search)[: 14 * 3]:
        top = s["hints"][0]
        assert (top["block_tile"], top["thread_tile"], top["rstep"]) == ([128, 128], [16, 8], 32)


def test_helpers_match(golden_search):
    h = golden_search["helpers"]
    for n, v in h["get_all_factors"].items():
        assert utils.get_all_factors(int(n)) == v
    for n, v in h["factorize"].items():
        assert utils.factorize(int(n)) == v
    for c in h["coalesced_factor"]:
        assert utils.coalesced_factor(c["sub"], c["full"]) == c["out"]
    for c in h["coalesced_tensor_shape"]:
        assert utils.coalesced_tensor_shape(c["sub"], c["full"], c["txn"]) == c["out"]
    for c in h["get_block_dims"]:
        assert utils.get_block_dims(c["block"], c["reg"]) == c["out"]
    for c in h["compute_memory_traffic"]:
        cfg = analyze.MatmulConfig(*c["shape"], el_bits=32)
        assert analyze.compute_memory_traffic(c["tile"], cfg, arch.CUDA()) == c["out"]
    pol = analyze.Policy(analyze.MatmulConfig(2048, 2048, 2048, 32), arch.CUDA())
    for n, v in h["score_block_size"].items():
        assert list(pol.score_block_size(int(n))) == v
    for n, v in h["reduce_step_candidates"].items():
        assert pol.get_reduce_step_candidates(int(n)) == v
    dev = arch.CUDA()
    for name, v in h["CUDA"].items():
        assert getattr(dev, name) == v


def test_tiledict_surface():
    cfg = analyze.MatmulConfig(2048, 2048, 2048, 32)
    hints = analyze.get_roller_hints(cfg, arch.CUDA(), topk=20)
    assert len(hints) == 20
    h = hints[0]
    # attributes the reference's callers read (src/roller.py:363-366,385,531-543)
    assert h.matmul_config is cfg and h.smem_cost == 32768
    assert hash(h) == hash(tuple(h.block_tile + h.thread_tile))
    assert "block_tile=[128, 128]" in repr(h) and "32.0 KiB" in repr(h)
    assert len({id(x) for x in hints}) == 20  # independent objects
    hints[0].thread_tile.append(1)
    assert hints[1].thread_tile != hints[0].thread_tile
    assert cfg.el_bytes == 4 and cfg.get_output_shape() == (2048, 2048)
    a, b = cfg.get_input_shapes()
    assert a.to_list() == [2048, 2048] and b.to_list() == [2048, 2048]


def test_compat_aliases():
    from mlir_roller_b200 import compat
    compat.install()
    import analyze as flat_analyze  # noqa: F401
    from arch import CUDA as FlatCUDA
    assert FlatCUDA is arch.CUDA


@pytest.mark.skipif(not REFERENCE_SRC.exists(), reason="reference checkout not present")
def test_live_against_reference_checkout():
    """Where the reference is mounted, compare against it directly on extra random shapes."""
    import importlib.util
    import random
    stub = types.ModuleType("humanize")
    stub.naturalsize = lambda n, binary=False: str(n)
    saved = {k: sys.modules.get(k) for k in ("humanize", "arch", "utils", "analyze")}
    sys.modules["humanize"] = stub
    try:
        mods = {}
        for name in ("arch", "utils", "analyze"):
            spec = importlib.util.spec_from_file_location(name, REFERENCE_SRC / f"{name}.py")
            mods[name] = importlib.util.module_from_spec(spec)
            sys.modules[name] = mods[name]
            spec.loader.exec_module(mods[name])
        rng = random.Random(7)
        for _ in range(25):
            m, n, k = (rng.choice([rng.randint(1, 700), 2 ** rng.randint(0, 13)]) for _ in range(3))
            want = mods["analyze"].get_roller_hints(
                mods["analyze"].MatmulConfig(m, n, k, 32), mods["arch"].CUDA(), topk=12)
            got = analyze.get_roller_hints(analyze.MatmulConfig(m, n, k, 32), arch.CUDA(), topk=12)
            assert [hint_record(h) for h in got] == [hint_record(h) for h in want], (m, n, k)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
