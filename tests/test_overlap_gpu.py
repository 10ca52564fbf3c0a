"""The exchange of C that runs underneath the computation (mgpu.OverlappedGemm) and the block
copy it is built on. The multi-rank check runs one process per visible GPU, two at most; with a
single GPU it still covers the banded computation, the symmetric allocation and the fence."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from mlir_roller_b200 import _lib

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def test_copy_block_between_strided_matrices():
    src = torch.rand(300, 520, device="cuda")
    dst = torch.zeros(400, 700, device="cuda")
    # block of 200 x 130 from src[50:, 64:] into dst[10:, 32:]
    _lib.copy_block_async(dst.data_ptr() + (10 * 700 + 32) * 4, 700,
                          src.data_ptr() + (50 * 520 + 64) * 4, 520, 200, 130)
    torch.cuda.synchronize()
    want = torch.zeros_like(dst)
    want[10:210, 32:162] = src[50:250, 64:194]
    assert torch.equal(dst, want)
    # contiguous form and the empty block
    a = torch.rand(64, 128, device="cuda")
    b = torch.empty_like(a)
    _lib.copy_block_async(b.data_ptr(), 128, a.data_ptr(), 128, 64, 128)
    _lib.copy_block_async(b.data_ptr(), 128, a.data_ptr(), 128, 0, 128)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    with pytest.raises(RuntimeError):
        _lib.copy_block_async(b.data_ptr(), 64, a.data_ptr(), 128, 4, 128)   # ld < cols


def test_overlapped_gemm_ranks():
    n = min(2, torch.cuda.device_count())
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(HERE / "overlap_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "FAIL" not in res.stdout
