import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_search():
    import json
    return json.loads((ROOT / "tests" / "golden" / "search_golden.json").read_text())


def hint_record(td) -> dict:
    return {"block_tile": list(td.block_tile), "thread_tile": list(td.thread_tile),
            "rstep": td.rstep, "traffic": td.traffic, "smem_cost": td.smem_cost,
            "block_per_SM": td.block_per_SM, "num_wave": td.num_wave, "grid_size": td.grid_size}
