"""Pins the oracle's search restatement to the reference's recorded outputs."""
from oracle import search_port


def test_oracle_search_matches_golden(golden_search):
    checked = 0
    for s in golden_search["searches"]:
        if "arch_overrides" in s:
            dev = dict(search_port.A100_MODEL)
            dev.update(s["arch_overrides"])
            dev["max_smem_usage"] = 2 * dev["smem_cap"]
        else:
            dev = None
        got = search_port.roller_hints(s["M"], s["N"], s["K"], s.get("el_bits", 32), s["topk"], dev)
        assert got == s["hints"], (s["M"], s["N"], s["K"], s["topk"])
        checked += 1
    assert checked == len(golden_search["searches"])


def test_oracle_divisors(golden_search):
    for n, v in golden_search["helpers"]["get_all_factors"].items():
        assert search_port.divisors(int(n)) == v
