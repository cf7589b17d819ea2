"""Multi-GPU tests: peer-memory collectives against NCCL, sharded Parallel Muon and the replicated all-reduce path
against a single-GPU run of the same global batch. Run as child processes (one per GPU), NVLS off."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_workers(mode, nproc=2, port=29731):
    try:                                       # a port that is free now; the fixed numbers are the fallback
        from conftest import free_port
        port = free_port()
    except Exception:
        pass
    import tempfile
    result_dir = tempfile.mkdtemp(prefix="pgb_multi_")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, PGB_RESULT_DIR=result_dir)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "multi_worker.py"), mode]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-3000:])
    res = {}
    lines = out.stdout.splitlines()
    for name in sorted(os.listdir(result_dir)):               # the per-rank files first, stdout lines as the fallback
        with open(os.path.join(result_dir, name)) as fh:
            lines = fh.read().splitlines() + lines
    for line in lines:
        if line.startswith("RESULT"):
            try:
                _, rank, payload = line.split(" ", 2)
                res.setdefault(int(rank), json.loads(payload))
            except ValueError:                                # an interleaved stdout line; the rank's file has the clean copy
                pass
    assert len(res) == nproc
    return res


def _world_sizes():
    import torch
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n] or [2]


@pytest.mark.parametrize("nproc", _world_sizes())
def test_peer_collectives_match_nccl(nproc):
    res = run_workers("collectives", nproc=nproc, port=29731 + nproc)
    for r in res.values():
        assert r["allreduce_err"] < 1e-5 and r["twoshot_err"] < 1e-5 and r["sumsq_rel"] < 1e-5 and r["packaged_err"] < 1e-5, r


@pytest.mark.parametrize("nproc", _world_sizes())
@pytest.mark.parametrize("mode,port", [("sharded", 29750), ("replicated", 29770)])
def test_distributed_step_matches_single_gpu(mode, port, nproc):
    """Three optimizer steps (the last with fake-quant on) of the same global batch on `nproc` GPUs and on one: 4 and 8 ranks
    reach the 4- and 8-peer reduction kernels and shard maps in which some ranks own no slot of a bank."""
    res = run_workers(mode, nproc=nproc, port=port + nproc)
    assert res[0]["worst_rel_update_err"] < 0.05, res[0]
    for r in range(1, nproc):          # the all-reduced loss: equal up to the summation order of the library's all-reduce
        assert res[r]["mean_losses"] == pytest.approx(res[0]["mean_losses"], rel=1e-9)
