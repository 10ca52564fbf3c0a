"""Integer helpers of the rTile search (same names and results as the reference's src/utils.py).

The reference builds divisor lists with numpy on every call (src/utils.py:6-17), which is a
visible share of its 2-5 ms per search; here they are plain-integer loops behind a cache.
"""
from __future__ import annotations

import math
from functools import lru_cache
from typing import List, Sequence


@lru_cache(maxsize=4096)
def _divisors(n: int) -> tuple:
    small, large = [], []
    d = 1
    while d * d <= n:
        if n % d == 0:
            small.append(d)
            if d * d != n:
                large.append(n // d)
        d += 1
    return tuple(small + large[::-1])


def get_all_factors(n: int) -> List[int]:
    """All divisors of n in ascending order (src/utils.py:6-17)."""
    return list(_divisors(int(n)))


def factorize(n: int) -> List[int]:
    """Prime factors of n with multiplicity, ascending (src/utils.py:20-31)."""
    out: List[int] = []
    p = 2
    while n > 1:
        while n % p == 0:
            out.append(p)
            n //= p
        p += 1
    return out


def coalesced_factor(subtensor: Sequence[int], tensor: Sequence[int]) -> int:
    """Length of the contiguous run a sub-tensor covers in its parent (src/utils.py:34-40).

    Walking from the innermost dimension outwards, the run keeps growing while the sub-tensor
    spans the parent's full extent.
    """
    run = 1
    for i in range(len(subtensor) - 1, -1, -1):
        run *= subtensor[i]
        if i == 0 or subtensor[i] != tensor[i]:
            break
    return run


def coalesced_tensor_shape(subtensor: Sequence[int], tensor: Sequence[int],
                           transaction_size: int) -> int:
    """Elements actually moved when a sub-tensor is fetched in whole memory transactions
    (src/utils.py:44-57)."""
    elems = math.prod(subtensor)
    if elems == 0:
        return 0
    run = coalesced_factor(subtensor, tensor)
    return transaction_size * elems // min(transaction_size, run)


def get_block_dims(block_tile: Sequence[int], reg_tile: Sequence[int]) -> List[int]:
    """Thread-block dimensions for a block tile split into per-thread tiles, x/y swapped so
    that x runs along N (src/utils.py:60-69)."""
    dims = [b // r if (b != 0 and r != 0) else 1 for b, r in zip(block_tile, reg_tile)]
    dims[0], dims[1] = dims[1], dims[0]
    return dims
