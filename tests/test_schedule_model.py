"""The work distribution of the GEMM kernels, restated on the host and checked for the
properties the device code relies on (csrc/gemm_tf32_sm100.cuh: Schedule, the partial-tile
exchange and the cooperative completion of shared tiles). The arithmetic is the kernel's: the
sk_tiles tiles cut along K are split over the rounds (round r owns tiles [tile_begin[r],
tile_begin[r + 1]), a geometric sequence of sizes made by the host, csrc/capi.cu:
plan_configure), a round's units = tiles * cpt are dealt in contiguous runs to the workers'
positions, worker w playing position (w + round * rot) mod workers, every worker consuming its
run from the end. Runs on the CPU; the GPU tests check the results, this checks the
bookkeeping."""
import itertools

import pytest


def round_tiles(sk_tiles, rounds, ratio_percent=100):
    """Boundaries of the rounds, as the library computes them."""
    ratio = ratio_percent / 100.0
    total = sum(ratio ** r for r in range(rounds))
    tb, cum = [0], 0.0
    for r in range(1, rounds + 1):
        cum += ratio ** (r - 1)
        b = int(cum / total * sk_tiles + 0.5)
        b = min(max(b, tb[-1] + 1), sk_tiles - (rounds - r))
        tb.append(sk_tiles if r == rounds else b)
    return tb


class Schedule:
    def __init__(self, num_tiles, workers, num_kb, chunk_kb, sk_tiles, rounds, ratio=100):
        self.num_tiles, self.workers, self.num_kb, self.chunk_kb = num_tiles, workers, num_kb, chunk_kb
        self.sk_tiles, self.rounds = sk_tiles, rounds
        self.cpt = -(-num_kb // chunk_kb)
        self.tile_begin = round_tiles(sk_tiles, rounds, ratio) if rounds > 1 else [0, sk_tiles]
        self.rot = (workers * 3) // 8 + 1 if rounds > 1 else 0

    def shape(self, r):
        t0, t1 = self.tile_begin[r], self.tile_begin[r + 1]
        units = (t1 - t0) * self.cpt
        return t0 * self.cpt, t1 - t0, units // self.workers, units % self.workers

    def unit_begin(self, r, p):
        base, _, q, rem = self.shape(r)
        return base + q * p + rem * p // self.workers

    def worker_at(self, p, r):
        return (p - r * self.rot) % self.workers

    def cooperative(self, r):
        """Whether round r's shared tiles are completed by all their workers together."""
        return self.workers >= 3 * self.shape(r)[1]

    def segments(self, worker):
        """(tile, kb0, kb1, final, round, pos) in the order the worker executes them."""
        out = []
        for r in range(self.rounds):
            pos = (worker + r * self.rot) % self.workers
            b, e = self.unit_begin(r, pos), self.unit_begin(r, pos + 1)
            while e > b:
                tile = (e - 1) // self.cpt
                t0 = tile * self.cpt
                sb = max(b, t0)
                out.append((tile, (sb - t0) * self.chunk_kb, min((e - t0) * self.chunk_kb, self.num_kb),
                            e - t0 == self.cpt, r, pos))
                e = sb
        t = self.sk_tiles + worker
        while t < self.num_tiles:
            out.append((t, 0, self.num_kb, True, 0, worker))
            t += self.workers
        return out

    def which_of(self, r, p, tile):
        return 0 if (self.unit_begin(r, p + 1) - 1) // self.cpt == tile else 1

    def participants(self, r, tile):
        u0, u1 = tile * self.cpt, (tile + 1) * self.cpt
        return [p for p in range(self.workers)
                if self.unit_begin(r, p) < u1 and self.unit_begin(r, p + 1) > u0
                and self.unit_begin(r, p + 1) != self.unit_begin(r, p)]


CASES = [
    # tiles, workers, num_kb, chunk_kb, sk_tiles, rounds[, ratio in percent]
    (64, 74, 128, 4, 64, 1), (64, 74, 128, 4, 64, 2), (64, 74, 128, 4, 64, 4), (64, 74, 128, 4, 64, 8),
    (512, 74, 512, 4, 512, 8), (128, 148, 48, 4, 128, 4), (32, 74, 48, 8, 32, 4), (35, 74, 49, 4, 35, 5),
    (300, 74, 64, 4, 4, 1), (256, 74, 64, 8, 34, 1), (117, 148, 49, 4, 117, 3),
    # rounds of unequal size, tile counts that no number of rounds divides
    (64, 74, 128, 4, 64, 4, 60), (64, 74, 128, 4, 64, 8, 125), (128, 74, 128, 4, 128, 4, 60),
    (67, 74, 128, 4, 67, 4, 100), (67, 74, 33, 4, 67, 16, 40), (16, 148, 128, 4, 16, 16, 400),
    (131, 148, 64, 8, 131, 5, 150), (256, 74, 128, 4, 256, 3, 25),
]


def test_round_boundaries():
    assert round_tiles(64, 4) == [0, 16, 32, 48, 64]
    assert round_tiles(64, 4, 60) == [0, 29, 47, 58, 64]
    assert round_tiles(64, 4, 125) == [0, 11, 25, 42, 64]
    for tiles, rounds, ratio in itertools.product((1, 2, 5, 16, 17, 64, 1000, 65536), (1, 2, 3, 7, 16),
                                                  (25, 60, 100, 150, 400)):
        if rounds > tiles:
            continue
        tb = round_tiles(tiles, rounds, ratio)
        assert tb[0] == 0 and tb[-1] == tiles and len(tb) == rounds + 1
        assert all(b > a for a, b in zip(tb, tb[1:]))        # every round owns a tile
        sizes = [b - a for a, b in zip(tb, tb[1:])]
        if tiles >= 64 * rounds and ratio != 100:
            assert sizes == sorted(sizes, reverse=ratio < 100)


@pytest.mark.parametrize("case", CASES)
def test_every_k_block_of_every_tile_is_computed_exactly_once(case):
    tiles, workers, num_kb, chunk_kb, sk_tiles, rounds = case[:6]
    s = Schedule(*case)
    covered = [[0] * num_kb for _ in range(tiles)]
    finals = [0] * tiles
    for w in range(workers):
        rounds_seen = []
        for tile, kb0, kb1, final, r, pos in s.segments(w):
            assert 0 <= kb0 < kb1 <= num_kb
            for kb in range(kb0, kb1):
                covered[tile][kb] += 1
            finals[tile] += final
            rounds_seen.append(r if tile < sk_tiles else rounds)
            assert final == (kb1 == num_kb)
        assert rounds_seen == sorted(rounds_seen)          # a worker moves through the rounds in order
    assert all(c == 1 for row in covered for c in row)
    assert finals == [1] * tiles                           # one worker holds the end of each tile


@pytest.mark.parametrize("case", [c for c in CASES if c[5] > 1])
def test_no_tile_straddles_two_rounds_and_positions_rotate(case):
    tiles, workers, num_kb, chunk_kb, sk_tiles, rounds = case[:6]
    s = Schedule(*case)
    round_of = {}
    for w in range(workers):
        for tile, kb0, kb1, final, r, pos in s.segments(w):
            assert round_of.setdefault(tile, r) == r
            assert s.worker_at(pos, r) == w
    finishing = [{w for w in range(workers) for (t, _, _, f, r, _) in s.segments(w) if f and r == rr}
                 for rr in range(rounds)]
    if rounds >= 2 and all(len(f) < workers for f in finishing):
        assert finishing[0] != finishing[1]                # not the same workers round after round


@pytest.mark.parametrize("case", CASES)
def test_partial_tiles_have_one_reader_in_the_plain_exchange(case):
    """The worker holding the end of a tile reads the partials of the positions before it, down
    to the one that started the tile; every published partial is read exactly once."""
    tiles, workers, num_kb, chunk_kb, sk_tiles, rounds = case[:6]
    s = Schedule(*case)
    published, read = set(), []
    for w in range(workers):
        for tile, kb0, kb1, final, r, pos in s.segments(w):
            if not final:
                key = (r, pos, tile)
                assert key not in published
                published.add(key)
            elif kb0 > 0:
                p = pos - 1
                while True:
                    if s.unit_begin(r, p + 1) != s.unit_begin(r, p):
                        read.append((r, p, tile))
                    if s.unit_begin(r, p) <= tile * s.cpt:
                        break
                    p -= 1
    assert sorted(read) == sorted(published)
    # a worker publishes at most once per round here (it alternates between two slots)
    per_round = {}
    for r, pos, tile in published:
        per_round[(r, pos)] = per_round.get((r, pos), 0) + 1
    assert all(n == 1 for n in per_round.values())


@pytest.mark.parametrize("case", [c for c in CASES if c[5] > 1])
@pytest.mark.parametrize("boxes", [4, 2, 1])
def test_cooperative_completion_covers_every_box_once(case, boxes):
    """Every worker holding part of a shared tile publishes (at most two partials per round,
    in different slots), the first min(P, boxes) of them each take boxes my_idx, my_idx + R, ...:
    each box of each shared tile is completed exactly once, and every slot has exactly R readers."""
    tiles, workers, num_kb, chunk_kb, sk_tiles, rounds = case[:6]
    s = Schedule(*case)
    done = {}
    readers = {}
    for w in range(workers):
        slots_used = {}
        for tile, kb0, kb1, final, r, pos in s.segments(w):
            if kb0 == 0 and final:
                done[(tile, "whole")] = done.get((tile, "whole"), 0) + 1
                continue
            which = s.which_of(r, pos, tile)
            assert (r, which) not in slots_used, "two partials of one round in one slot"
            slots_used[(r, which)] = tile
            parts = s.participants(r, tile)
            assert pos in parts and len(parts) >= 2
            R = min(len(parts), boxes)
            my_idx = parts.index(pos)
            if my_idx >= R:
                continue
            for c in range(my_idx, boxes, R):
                done[(tile, c)] = done.get((tile, c), 0) + 1
            for p in parts:
                key = (r, s.worker_at(p, r), s.which_of(r, p, tile))
                readers[key] = readers.get(key, 0) + 1
        assert all(sum(1 for (rr, _w) in slots_used if rr == r) <= 2 for r in range(rounds))
    for tile in range(sk_tiles):
        if (tile, "whole") in done:
            assert done[(tile, "whole")] == 1 and not any((tile, c) in done for c in range(boxes))
        else:
            assert [done.get((tile, c), 0) for c in range(boxes)] == [1] * boxes
    for (r, w, which), n in readers.items():
        # the slot (r, w, which) holds worker w's partial of one tile of round r
        seg = [(t, pos) for (t, kb0, kb1, f, rr, pos) in s.segments(w)
               if rr == r and t < sk_tiles and not (kb0 == 0 and f) and s.which_of(r, pos, t) == which]
        assert len(seg) == 1
        assert n == min(len(s.participants(r, seg[0][0])), boxes)


def test_the_arithmetic_stays_within_32_bits():
    # the kernel computes unit_begin with 32-bit products: base + q * p + rem * p / workers
    for tiles, workers, cpt, rounds in itertools.product((1, 64, 8192, 1 << 20), (1, 74, 148), (2, 128, 2048), (1, 8, 16)):
        if rounds > tiles:
            continue
        units = tiles * cpt
        if units >= 1 << 31:
            continue          # the host does not enable the split beyond this
        tb = round_tiles(tiles, rounds)
        for r in range(rounds):
            ur = (tb[r + 1] - tb[r]) * cpt
            q, rem = divmod(ur, workers)
            assert tb[r] * cpt + q * workers + rem == tb[r + 1] * cpt <= units
            assert rem * workers < 1 << 31 and q * workers < 1 << 31


@pytest.mark.parametrize("case", [c for c in CASES if c[5] > 1])
def test_rounds_of_either_kind_share_the_slots_safely(case):
    """Each round decides by itself whether shared tiles are completed cooperatively (a tile
    shared by three workers or more) or by the worker holding the end of the reduction. Both
    kinds number a worker's slots the same way -- (round & 1) * 2 + which, the plain exchange
    using which = 0 only -- so a slot is next used two rounds later by the same worker, whatever
    the kinds of the two rounds, and that worker waits for the slot's flag to be handed back."""
    s = Schedule(*case)
    kinds = {s.cooperative(r) for r in range(s.rounds)}
    used = {}
    for w in range(s.workers):
        for tile, kb0, kb1, final, r, pos in s.segments(w):
            if tile >= s.sk_tiles or (kb0 == 0 and final):
                continue
            if s.cooperative(r):
                which = s.which_of(r, pos, tile)
            elif final:
                continue                   # the plain exchange: the completing worker publishes nothing
            else:
                which = 0
            key = (w, (r & 1) * 2 + which)
            assert r not in used.setdefault(key, []), "one slot twice in a round"
            used[key].append(r)
    for (w, slot), rs in used.items():
        assert all(b - a >= 2 for a, b in zip(rs, rs[1:]))
        assert all((r & 1) == slot // 2 for r in rs)
    assert kinds  # (both kinds occur over the cases: see below)


def test_the_cases_cover_both_kinds_of_round_in_one_launch():
    mixed = [c for c in CASES if c[5] > 1 and len({Schedule(*c).cooperative(r) for r in range(c[5])}) == 2]
    assert mixed
