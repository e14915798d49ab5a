"""Tensor-parallel path: the sharding rule on CPU ranks (gloo, world size 2), and on GPUs when at least two
are visible.  Every rendezvous uses 127.0.0.1."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

WORKER = str(Path(__file__).resolve().parent / "tp_worker.py")


def _launch(nproc, args, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + os.getpid() % 1000), WORKER] + args
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, f"worker failed:\n{r.stdout[-3000:]}\n{r.stderr[-6000:]}"
    return r.stdout


@pytest.mark.parametrize("nproc", [2, 4])
def test_sharding_rule_on_cpu_ranks(nproc):
    out = _launch(nproc, ["cpu"])
    assert f"tp_worker cpu ok on {nproc} ranks" in out


@pytest.mark.gpu
def test_tensor_parallel_engine_matches_oracle(built_lib, tmp_path):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    nproc = 4 if n >= 4 else 2
    out = _launch(nproc, ["gpu", str(tmp_path)])
    assert f"tp_worker gpu ok on {nproc} ranks" in out
