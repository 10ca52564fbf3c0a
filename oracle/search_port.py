"""TEST INFRASTRUCTURE -- CPU restatement of the reference's Roller rTile search.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this
module; the product (mlir_roller_b200/) never does.

It re-states, as plain functions over dicts, what NaOHCC/mlir-roller computes in
src/analyze.py (Policy.emit_config and helpers), src/utils.py and the `CUDA` device model of
src/arch.py:40-61. It deliberately keeps the reference's cost structure (numpy divisor lists,
a deep copy per emitted hint) so that timing it stands in for timing the reference's search,
which cannot travel to the GPU box.

Pinned: tests/test_oracle_search.py checks it against tests/golden/search_golden.json, which
tests/golden/gen_search_golden.py produced by running the reference itself.
"""
from __future__ import annotations

import copy
import itertools
import math

import numpy as np

# The reference's device model, src/arch.py:47-61 (A100-class numbers).
A100_MODEL = {
    "reg_cap": 65536, "smem_cap": 64 * 1024, "compute_max_core": 108, "warp_size": 32,
    "sm_partition": 4, "max_smem_usage": 2 * 64 * 1024, "transaction_size": [32, 128],
    "bandwidth": [750, 12080],
}


def divisors(n):
    """src/utils.py:6-17: divisors below ceil(sqrt(n)), the root if n is a square, and the
    cofactors, via numpy."""
    root = int(np.ceil(np.sqrt(n)))
    low = np.where(n % np.arange(1, root) == 0)[0] + 1
    mid = [root] if root * root == n else np.array([], dtype=int)
    return [int(v) for v in np.concatenate([low, mid, n // low[::-1]])]


def contiguous_run(sub, full):
    """src/utils.py:34-40."""
    if len(sub) == 1 or sub[-1] != full[-1]:
        return sub[-1]
    return sub[-1] * contiguous_run(sub[:-1], full[:-1])


def moved_elems(sub, full, txn):
    """src/utils.py:44-57."""
    n = math.prod(sub)
    if n == 0:
        return 0
    return txn * n // min(txn, contiguous_run(sub, full))


def el_bytes(cfg):
    return (cfg["el_bits"] + 7) // 8


def tile_traffic(tile, cfg, dev):
    """src/analyze.py:62-81."""
    eb = el_bytes(cfg)
    rd = dev["transaction_size"][1] // eb
    wr = dev["transaction_size"][0] // eb
    total = moved_elems([tile[0], cfg["K"]], [cfg["M"], cfg["K"]], rd)
    total += moved_elems([tile[1], cfg["K"]], [cfg["N"], cfg["K"]], rd)
    total += moved_elems(list(tile), [cfg["M"], cfg["N"]], wr)
    return total * eb


def stage_bytes(tile, rstep, cfg):
    """src/analyze.py:120-123."""
    return (tile[0] + tile[1]) * rstep * el_bytes(cfg)


def analyse_tile(tile, rstep, cfg, dev):
    """src/analyze.py:125-168. Returns None for an infeasible tile."""
    smem = stage_bytes(tile, rstep, cfg)
    if smem > dev["smem_cap"]:
        return None
    regs = int(2 * tile[0] * tile[1] * el_bytes(cfg) / 32)
    if regs > dev["reg_cap"]:
        return None
    grid = ((cfg["M"] + tile[0] - 1) // tile[0]) * ((cfg["N"] + tile[1] - 1) // tile[1])
    per_sm = min(dev["max_smem_usage"] // max(smem, 1), dev["reg_cap"] // max(regs, 1),
                 dev["sm_partition"])
    waves = int(np.ceil(grid / int(per_sm * dev["compute_max_core"])))
    return {"block_tile": list(tile), "thread_tile": [], "rstep": rstep,
            "traffic": tile_traffic(tile, cfg, dev), "smem_cost": smem, "block_per_SM": per_sm,
            "num_wave": waves, "grid_size": grid}


def reduce_candidates(k):
    """src/analyze.py:203-215."""
    cands = divisors(k)
    if len(cands) == 2 and k > 64:
        cands = [1]
        while cands[-1] * 2 < k:
            cands.append(cands[-1] * 2)
    return cands


def run_scores(tile, rstep, cfg):
    return [contiguous_run([tile[0], rstep], [cfg["M"], cfg["K"]]),
            contiguous_run([tile[1], rstep], [cfg["N"], cfg["K"]])]


def base_reduce_step(cfg, dev):
    """src/analyze.py:181-201,217-221 ("sim" score against one read transaction)."""
    txn = dev["transaction_size"][1] // el_bytes(cfg)

    def score(step):
        total = 0.0
        for run in run_scores([1, 1], step, cfg):
            total += (2 * run * txn) / (run * run + txn * txn)
        return total

    return max(reduce_candidates(cfg["K"]), key=score)


def ranked_block_tiles(cfg, dev, rstep):
    """src/analyze.py:223-255."""
    axes = []
    for extent in (cfg["M"], cfg["N"]):
        sizes = set(f for f in divisors(extent) if f >= 1)
        sizes |= {p for p in (2, 4, 8, 16, 32) if 1 < p < extent}
        axes.append(sorted(sizes))
    found = []
    for m, n in itertools.product(axes[0], axes[1]):
        td = analyse_tile([m, n], rstep, cfg, dev)
        if td is not None:
            found.append(td)
    return sorted(found, key=lambda td: (td["traffic"] + 1) * td["num_wave"])


def widen_reduce_step(td, cfg, dev):
    """src/analyze.py:257-277."""
    limit = min(dev["max_smem_usage"] // td["block_per_SM"], dev["smem_cap"])
    ok = [s for s in reduce_candidates(cfg["K"])
          if s % td["rstep"] == 0 and stage_bytes(td["block_tile"], s, cfg) <= limit]
    if not ok:
        ok = [td["rstep"]]
    td["rstep"] = max(ok, key=lambda s: float(sum(run_scores(td["block_tile"], s, cfg))))
    td["smem_cost"] = stage_bytes(td["block_tile"], td["rstep"], cfg)


def thread_counts(td, dev):
    """src/analyze.py:279-308."""
    def score(n):
        warps = (n + dev["warp_size"] - 1) // dev["warp_size"]
        return (max(warps / dev["sm_partition"], dev["sm_partition"] / warps),
                (warps * dev["warp_size"] - n) / n)

    sizes = [f for f in divisors(int(math.prod(td["block_tile"]))) if f <= 1024]
    return sorted(sizes, key=score)


def thread_tile_for(td, threads, cfg, dev):
    """src/analyze.py:329-365. Returns None when the tile needs 256 registers or more."""
    per_thread = math.prod(td["block_tile"]) // threads
    pairs = [[per_thread // i, i] for i in range(1, int(math.sqrt(per_thread)) + 1)
             if per_thread % i == 0]

    def cost(tt):
        total = 0
        for extent in tt:
            total += (extent * cfg["K"]) / dev["bandwidth"][1]
        return total

    best = sorted(pairs, key=cost)[0]
    if int(math.prod(best) * el_bytes(cfg) / 4) >= 256:
        return None
    return best


def roller_hints(M, N, K, el_bits=32, topk=10, dev=None):
    """src/analyze.py:367-387: list of hint dicts, best first."""
    dev = A100_MODEL if dev is None else dev
    cfg = {"M": M, "N": N, "K": K, "el_bits": el_bits}
    out = []
    for td in ranked_block_tiles(cfg, dev, base_reduce_step(cfg, dev)):
        widen_reduce_step(td, cfg, dev)
        taken = 0
        for threads in thread_counts(td, dev):
            tt = thread_tile_for(td, threads, cfg, dev)
            if tt is None:
                break
            td["thread_tile"] = tt
            out.append(copy.deepcopy(td))
            taken += 1
            if taken == 2 or len(out) >= topk:
                break
        if len(out) >= topk:
            break
    return out
