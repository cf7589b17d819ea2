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
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "multi_worker.py"), mode]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-3000:])
    res = {}
    for line in out.stdout.splitlines():
        if line.startswith("RESULT"):
            _, rank, payload = line.split(" ", 2)
            res[int(rank)] = json.loads(payload)
    assert len(res) == nproc
    return res


def test_peer_collectives_match_nccl():
    res = run_workers("collectives", port=29731)
    for r in res.values():
        assert r["allreduce_err"] < 1e-5 and r["twoshot_err"] < 1e-5 and r["sumsq_rel"] < 1e-5 and r["packaged_err"] < 1e-5, r


@pytest.mark.parametrize("mode,port", [("sharded", 29732), ("replicated", 29733)])
def test_distributed_step_matches_single_gpu(mode, port):
    res = run_workers(mode, port=port)
    assert res[0]["worst_rel_update_err"] < 0.05, res[0]
    assert res[0]["mean_losses"] == res[1]["mean_losses"]
