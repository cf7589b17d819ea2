"""Failure detection without touching a GPU: failures are made on the host (a rank that raises, never joins or exits;
a corrupted or missing file; a mismatched fingerprint) and, for multi-rank cases, among gloo ranks on CPU."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from parameter_golf_b200.data import shards as S
from parameter_golf_b200.spec import family_preset

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, body, nproc=2, port=None, timeout=120):
    from conftest import free_port
    port = free_port()
    script = tmp_path / "w.py"
    script.write_text("import os, sys, time, datetime\nsys.path.insert(0, %r)\nimport torch, torch.distributed as dist\n" % ROOT + textwrap.dedent(body))
    env = dict(os.environ, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
                           "--master-port", str(port), str(script)], capture_output=True, text=True, env=env, cwd=ROOT, timeout=timeout)


def test_rank_that_never_joins_is_detected_by_timeout(tmp_path):
    out = _run(tmp_path, """
        dist.init_process_group('gloo', timeout=datetime.timedelta(seconds=3))
        rank = dist.get_rank()
        t = torch.ones(1)
        if rank == 1:
            time.sleep(8)                      # misses the collective
            print('LATE', flush=True); sys.exit(0)
        try:
            dist.all_reduce(t)
            print('UNEXPECTED', flush=True)
        except Exception as e:
            print('DETECTED', type(e).__name__, flush=True)
        """, port=29691)
    assert "DETECTED" in out.stdout and "UNEXPECTED" not in out.stdout, (out.stdout, out.stderr[-1500:])


def test_rank_that_raises_is_reported_through_the_store(tmp_path):
    out = _run(tmp_path, """
        dist.init_process_group('gloo', timeout=datetime.timedelta(seconds=20))
        rank = dist.get_rank()
        store = dist.distributed_c10d._get_default_store()
        for step in range(3):
            if rank == 1 and step == 1:
                store.set('failed', 'rank1: injected exception at step 1')      # heartbeat-style report, between steps
                break
            if store.num_keys() and store.check(['failed']):
                print('PEER_FAILED', store.get('failed').decode(), flush=True); break
            time.sleep(0.3)
            if store.check(['failed']):
                print('PEER_FAILED', store.get('failed').decode(), flush=True); break
            dist.all_reduce(torch.ones(1))
        """, port=29692)
    assert "PEER_FAILED rank1: injected exception at step 1" in out.stdout, (out.stdout, out.stderr[-1500:])


def test_missing_and_corrupt_shards_fail_loudly(tmp_path):
    with pytest.raises(FileNotFoundError):
        S.DistributedTokenLoader(str(tmp_path / "nothing_*.bin"))
    p = tmp_path / "x_train_000000.bin"
    S.write_shard(str(p), np.arange(100))
    raw = bytearray(p.read_bytes())
    raw[8:12] = (5000).to_bytes(4, "little")                 # header now promises more tokens than the file holds
    p.write_bytes(raw)
    with pytest.raises(S.ShardError, match="does not match"):
        S.DistributedTokenLoader(str(tmp_path / "x_train_*.bin"))


def test_wallclock_and_eval_deadlines_end_runs_cleanly(tmp_path, monkeypatch):
    import math
    import numpy as np
    from parameter_golf_b200.data.bpb import BpbLuts
    from parameter_golf_b200.eval.ttt import eval_score_first_ttt
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.models.runner import OracleRunner
    s = family_preset("tiny_cpu")
    m = s.model
    m.vocab_size, m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads, m.eval_seq_len = 32, 1, 16, 2, 1, 16
    s.eval.stride, s.eval.chunk_tokens, s.eval.max_eval_seconds = 4, 32, 1e-9
    p = gpt.fill_deterministic(m)
    before = {k: v.clone() for k, v in p.items()}
    toks = np.random.default_rng(0).integers(0, 32, 16 * 6 + 1).astype(np.uint16)
    loss, bpb = eval_score_first_ttt(OracleRunner(m, p), toks, m, s.eval, BpbLuts.seeded(32))
    assert math.isfinite(loss) and all((p[k] == before[k]).all() for k in p)       # past the deadline: scoring only, no adaptation


def test_fingerprint_mismatch_blocks_resume_and_artifact_mismatch_blocks_load(tmp_path):
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.quant.container import ArtifactError
    from parameter_golf_b200.quant.export import export_model, load_artifact
    a, b = family_preset("tiny_cpu"), family_preset("tiny_cpu")
    b.model.num_heads = 2
    blob = export_model(a, gpt.init_params(a.model, 0))
    with pytest.raises(ArtifactError, match="num_heads"):
        load_artifact(blob, b.validate())


class _FakeStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_rank_health_reports_failures_and_silent_peers():
    from parameter_golf_b200.parallel.health import PeerFailure, RankHealth
    store, now = _FakeStore(), [1000.0]
    a = RankHealth(store, 0, 2, timeout_s=5.0, clock=lambda: now[0])
    b = RankHealth(store, 1, 2, timeout_s=5.0, clock=lambda: now[0])
    a.check()                                   # nobody has beaten yet: start-up is not policed
    a.beat(1)
    b.beat(1)
    now[0] += 4.0
    a.check()
    now[0] += 2.0                               # rank 1 silent for 6 s > 5 s
    with pytest.raises(PeerFailure, match="rank1 silent"):
        a.check()
    b.beat(2)
    a.check()
    with pytest.raises(ValueError):
        with b.guard():
            raise ValueError("shard 7 is truncated")
    with pytest.raises(PeerFailure, match="rank1: ValueError: shard 7 is truncated"):
        a.check()


def test_training_ranks_stop_on_the_host_when_a_peer_fails_between_steps(tmp_path):
    """Two gloo ranks run the real training loop on the CPU backend; rank 1's backend raises in its third step. Rank 0 must
    end with PeerFailure before its next step instead of waiting in a collective."""
    out = _run(tmp_path, """
        dist.init_process_group('gloo', timeout=datetime.timedelta(seconds=30))
        rank = dist.get_rank()
        from parameter_golf_b200.spec import family_preset
        from parameter_golf_b200.train import VariantRunner, OracleBackend
        from parameter_golf_b200.parallel.health import PeerFailure
        spec = family_preset('tiny_cpu')
        spec.train.world_size, spec.train.rank, spec.train.backend = 2, rank, 'cuda_distributed'   # the factory below supplies a CPU backend
        spec.train.total_iterations, spec.train.max_wallclock_seconds, spec.mode = 6, 0.0, 'proxy'

        class Flaky(OracleBackend):
            calls = 0
            def train_step(self, *a, **k):
                Flaky.calls += 1
                if rank == 1 and Flaky.calls == 3:
                    raise RuntimeError('injected: device lost')
                time.sleep(0.2)
                return super().train_step(*a, **k)

        try:
            VariantRunner(spec, backend_factory=lambda s, p: Flaky(s, p)).run('proxy')
            print('RANK', rank, 'FINISHED', flush=True)
        except PeerFailure as e:
            print('RANK', rank, 'PEER_FAILURE', e, 'after', Flaky.calls, 'steps', flush=True)
        except RuntimeError as e:
            print('RANK', rank, 'RAISED', e, flush=True)
        """, port=29695, timeout=240)
    assert "RANK 1 RAISED injected: device lost" in out.stdout, (out.stdout, out.stderr[-2000:])
    assert "RANK 0 PEER_FAILURE rank1: RuntimeError: injected: device lost" in out.stdout, (out.stdout, out.stderr[-2000:])
    assert "RANK 0 FINISHED" not in out.stdout


def test_wallclock_cap_is_agreed_across_ranks_when_one_clock_runs_ahead(tmp_path):
    """Two gloo ranks run the real training loop with a wall-clock cap; rank 1's clock jumps past the cap after a few
    steps. Both ranks must leave the loop on the same step (the decision is all-reduced), so neither is left waiting in
    the gradient all-reduce of a step its peer never starts."""
    out = _run(tmp_path, """
        dist.init_process_group('gloo', timeout=datetime.timedelta(seconds=20))
        rank = dist.get_rank()
        from parameter_golf_b200.spec import family_preset
        from parameter_golf_b200.train import VariantRunner
        spec = family_preset('tiny_cpu')
        spec.train.world_size, spec.train.rank = 2, rank
        spec.train.total_iterations, spec.train.max_wallclock_seconds, spec.mode = 30, 500.0, 'proxy'
        spec.train.wallclock_warmdown, spec.train.late_qat_threshold = True, 0.5
        spec.quant.scheme = 'none'
        spec.train.artifact_path = os.path.join(%r, 'a.pgrs')
        r = VariantRunner(spec)
        calls = [0]
        def clock():
            calls[0] += 1
            return time.perf_counter() + (1000.0 if rank == 1 and calls[0] > 9 else 0.0)
        r.clock = clock
        res = r.run('proxy')
        sys.stdout.write(chr(10) + f'RANK {rank} STEPS {res.steps} EARLY {res.stopped_early}' + chr(10)); sys.stdout.flush()      # one write per rank: the two ranks share a pipe
        """ % str(tmp_path), port=29697, timeout=240)
    lines = sorted(l for l in out.stdout.splitlines() if l.startswith("RANK"))
    assert len(lines) == 2, (out.stdout, out.stderr[-2000:])
    steps = [int(l.split()[3]) for l in lines]
    assert steps[0] == steps[1] and 0 < steps[0] < 30, lines
    assert all(l.endswith("EARLY True") for l in lines), lines
