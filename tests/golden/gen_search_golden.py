"""Generates tests/golden/search_golden.json by running the reference's own rTile search.

Run where a checkout of the reference is available (default: a directory named `reference`
next to this repository):

    python tests/golden/gen_search_golden.py [/path/to/reference]

The reference imports `humanize` at module scope but only uses it in TileDict.__repr__
(src/analyze.py:9,114-116); a stub module stands in for it. Nothing from the reference is
copied: only the values its functions return are recorded.
"""
from __future__ import annotations

import json
import sys
import types
from pathlib import Path

README_SHAPES = [
    (2048, 2048, 2048), (2048, 2048, 8192), (2048, 4096, 2048), (2048, 4096, 4096),
    (2048, 8192, 2048), (2048, 8192, 4096), (2048, 8192, 8192), (4096, 2048, 2048),
    (4096, 4096, 8192), (4096, 8192, 2048), (4096, 8192, 4096), (8192, 2048, 8192),
    (8192, 4096, 2048), (8192, 4096, 4096),
]
EXTRA_SHAPES = [
    (16384, 16384, 16384), (1024, 4096, 4096), (4096, 8192, 16384),
    (4097, 2049, 8193), (16, 8192, 8192),
    (64, 64, 64), (100, 60, 36), (7, 13, 17), (1024, 1024, 67), (1024, 768, 131),
    (1, 1, 1), (1, 4096, 4096), (96, 160, 224), (4096, 4096, 4096), (8192, 8192, 8192),
    (333, 777, 1000), (2, 3, 5), (640, 480, 360),
]
TOPKS = [1, 10, 20]


def hint_record(td) -> dict:
    return {
        "block_tile": list(td.block_tile), "thread_tile": list(td.thread_tile),
        "rstep": int(td.rstep), "traffic": int(td.traffic), "smem_cost": int(td.smem_cost),
        "block_per_SM": int(td.block_per_SM), "num_wave": int(td.num_wave),
        "grid_size": int(td.grid_size),
    }


def main() -> None:
    ref = Path(sys.argv[1]) if len(sys.argv) > 1 else \
        Path(__file__).resolve().parents[3] / "reference"
    stub = types.ModuleType("humanize")
    stub.naturalsize = lambda n, binary=False: str(n)
    sys.modules["humanize"] = stub
    sys.path.insert(0, str(ref / "src"))
    import analyze  # noqa: E402  (the reference's module)
    import arch     # noqa: E402
    import utils    # noqa: E402

    out: dict = {"source": "NaOHCC/mlir-roller src/analyze.py, src/arch.py, src/utils.py",
                 "arch": "CUDA()", "searches": [], "helpers": {}}

    for (m, n, k) in README_SHAPES + EXTRA_SHAPES:
        for topk in TOPKS:
            cfg = analyze.MatmulConfig(M=m, N=n, K=k, el_bits=32)
            rec = {"M": m, "N": n, "K": k, "topk": topk}
            try:
                hints = analyze.get_roller_hints(cfg, arch.CUDA(), topk=topk)
                rec["hints"] = [hint_record(h) for h in hints]
            except Exception as e:  # record how the reference fails, if it does
                rec["raises"] = type(e).__name__
            out["searches"].append(rec)

    # a different element width and a modified device, to pin the parametric parts
    for (m, n, k, bits) in [(2048, 2048, 2048, 16), (4096, 4096, 4096, 64), (512, 1024, 256, 8)]:
        cfg = analyze.MatmulConfig(M=m, N=n, K=k, el_bits=bits)
        hints = analyze.get_roller_hints(cfg, arch.CUDA(), topk=10)
        out["searches"].append({"M": m, "N": n, "K": k, "topk": 10, "el_bits": bits,
                                "hints": [hint_record(h) for h in hints]})
    dev = arch.CUDA(smem_cap=48 * 1024, compute_max_core=80)
    cfg = analyze.MatmulConfig(M=4096, N=4096, K=4096, el_bits=32)
    out["searches"].append({"M": 4096, "N": 4096, "K": 4096, "topk": 10,
                            "arch_overrides": {"smem_cap": 48 * 1024, "compute_max_core": 80},
                            "hints": [hint_record(h) for h in
                                      analyze.get_roller_hints(cfg, dev, topk=10)]})

    h = out["helpers"]
    h["get_all_factors"] = {str(n): utils.get_all_factors(n) for n in
                            [1, 2, 3, 4, 9, 16, 36, 67, 100, 2048, 2049, 4097, 8193, 16384, 16384 * 128]}
    h["factorize"] = {str(n): utils.factorize(n) for n in [1, 2, 12, 97, 360, 2048, 8193]}
    cf_cases = [([1, 32], [2048, 2048]), ([4, 2048], [2048, 2048]), ([128, 32], [2048, 4096]),
                ([16], [16]), ([8, 8192], [16, 8192]), ([3, 5], [7, 5])]
    h["coalesced_factor"] = [{"sub": s, "full": f, "out": int(utils.coalesced_factor(s, f))}
                             for s, f in cf_cases]
    cts_cases = [([128, 2048], [2048, 2048], 32), ([128, 128], [2048, 2048], 8),
                 ([0, 5], [10, 10], 8), ([241, 8193], [4097, 8193], 32), ([16, 32], [16, 8192], 8)]
    h["coalesced_tensor_shape"] = [{"sub": s, "full": f, "txn": t,
                                    "out": int(utils.coalesced_tensor_shape(s, f, t))}
                                   for s, f, t in cts_cases]
    h["get_block_dims"] = [{"block": b, "reg": r, "out": utils.get_block_dims(list(b), list(r))}
                           for b, r in [([128, 128, 0], [16, 8, 0]), ([64, 256], [16, 8]),
                                        ([16, 32], [2, 2])]]
    tr_cases = [([128, 128], (2048, 2048, 2048)), ([64, 256], (2048, 2048, 8192)),
                ([241, 32], (4097, 2049, 8193)), ([16, 32], (16, 8192, 8192))]
    h["compute_memory_traffic"] = [
        {"tile": t, "shape": list(s),
         "out": int(analyze.compute_memory_traffic(t, analyze.MatmulConfig(*s, el_bits=32), arch.CUDA()))}
        for t, s in tr_cases]
    cuda = arch.CUDA()
    h["CUDA"] = {f: getattr(cuda, f) for f in
                 ["reg_cap", "smem_cap", "compute_max_core", "warp_size", "sm_partition",
                  "max_smem_usage", "platform", "compute_capability", "l2_cache_size_bytes",
                  "transaction_size", "bandwidth"]}
    pol = analyze.Policy(analyze.MatmulConfig(2048, 2048, 2048, 32), arch.CUDA())
    h["score_block_size"] = {str(n): list(pol.score_block_size(n)) for n in [32, 64, 96, 128, 256, 1000, 1024]}
    h["reduce_step_candidates"] = {str(k): pol.get_reduce_step_candidates(k) for k in [2048, 67, 61, 8193, 131, 64]}

    dst = Path(__file__).resolve().parent / "search_golden.json"
    dst.write_text(json.dumps(out, separators=(",", ":")) + "\n")
    print(f"wrote {dst} ({dst.stat().st_size} bytes, {len(out['searches'])} searches)")


if __name__ == "__main__":
    main()
