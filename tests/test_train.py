import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from parameter_golf_b200.models import gpt
from parameter_golf_b200.quant.export import load_artifact
from parameter_golf_b200.spec import family_preset
from parameter_golf_b200.train import VariantRunner, mode_max_steps, record_gaps, split_param_groups, step_batch_plan
from parameter_golf_b200.utils.checkpoint import load_checkpoint, save_checkpoint
from parameter_golf_b200.utils.logging import RunLog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
from conftest import free_port  # noqa: E402


def quiet(spec):
    return VariantRunner(spec, RunLog(spec.name, console=False))


def test_tiny_config_end_to_end(tmp_path, monkeypatch):
    """2 layers, d128, 4/2 heads, vocab 1024, seq 256, 8x256 tokens, 20 Muon+Adam steps, int6 + zstd round trip."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "record_shaped_proxy"
    s.train.total_iterations = 20
    s.train.artifact_path = str(tmp_path / "tiny.pgrs")
    s.eval.max_tokens = 1024
    r = quiet(s)
    import parameter_golf_b200.train as tr
    monkeypatch.setattr(tr, "mode_max_steps", lambda spec, mode: 20)
    res = r.run()
    assert res.steps == 20 and res.tokens_per_step == 8 * 256
    assert res.train_loss_last < res.train_loss_first < 7.0
    assert os.path.getsize(s.train.artifact_path) == res.artifact_bytes and res.budget_ok
    assert np.isfinite(res.val_loss) and np.isfinite(res.val_bpb) and res.eval_kind == "sliding"
    back = load_artifact(open(s.train.artifact_path, "rb").read(), s)
    assert back["qo_bank"].shape == (4, 128, 128)
    lines = res.key_value_lines()
    assert any(l.startswith("step_avg_ms=") for l in lines) and any(l.startswith("fingerprint=") for l in lines)
    assert any(l.startswith("record_audit_json=") for l in r.log.lines)
    assert any(l.startswith("step:20/20 train_loss:") for l in r.log.lines)


def test_batch_plan_and_modes():
    s = family_preset("record_11l")
    s.train.world_size = 8
    assert step_batch_plan(s, "record") == (786432, 1)
    s.train.world_size = 2
    assert step_batch_plan(s, "record_shaped_proxy") == (786432, 4)
    assert step_batch_plan(s, "smoke") == (2 * 2048 * 2, 1)
    assert mode_max_steps(s, "smoke") == 4 and mode_max_steps(s, "proxy") == 32 and mode_max_steps(s, "record") == 9000
    assert step_batch_plan(family_preset("tiny_cpu"), "record") == (2048, 1)


def test_param_groups_follow_python_grouping():
    s = family_preset("record_11l")
    s.model.value_embedding.enabled = True
    shapes = gpt.param_shapes(s.model)
    banks, groups = split_param_groups(s, shapes)
    assert banks == ["qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank"]
    assert groups[0]["names"] == ["tok_emb", "bigram_embed", "ve_embed"] and groups[0]["lr"] == s.train.tied_embed_lr
    assert "bigram_proj" in groups[1]["names"] and "ve_proj" in groups[1]["names"] and "resid_mix" in groups[1]["names"]


def test_record_gate_fails_closed():
    s = family_preset("record_11l")
    gaps = record_gaps(s, "record")
    assert any("shards" in g for g in gaps) and any("8 GPUs" in g for g in gaps)
    assert record_gaps(s, "proxy") == []


def test_wallclock_cap_stops_cleanly(tmp_path, monkeypatch):
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "proxy"
    s.train.max_wallclock_seconds = 0.2
    s.train.total_iterations = 32
    s.train.artifact_path = str(tmp_path / "a.pgrs")
    res = quiet(s).run()
    assert res.stopped_early and 0 < res.steps < 32 and np.isfinite(res.val_bpb)


def test_checkpoint_resume_continues_the_trajectory(tmp_path, monkeypatch):
    """3 steps + checkpoint + resume for 3 more reproduces the loss trajectory of 6 straight steps
    (multi-threaded CPU reductions make bit equality of the weights too strict)."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))

    def run(iters, **kw):
        s = family_preset("tiny_cpu")
        s.mode = "proxy"
        s.train.total_iterations = iters
        s.train.train_log_every = 1
        s.train.artifact_path = str(tmp_path / f"a{iters}{len(kw)}.pgrs")
        for k, v in kw.items():
            setattr(s.train, k, v)
        r = quiet(s)
        res = r.run()
        losses = [float(l.split("train_loss:")[1].split()[0]) for l in r.log.lines if l.startswith("step:")]
        return losses, res

    ck = str(tmp_path / "ck.bin")
    full, res_full = run(6)
    run(3, checkpoint_every=3, checkpoint_path=ck)
    st = load_checkpoint(ck)
    assert st["step"] == 3 and "muon" in st["optim"] and st["loader"]["pos"] > 0
    resumed, res_resumed = run(6, resume_from=ck)
    assert len(resumed) == 3 and np.allclose(resumed, full[3:], atol=2e-3)
    assert abs(res_resumed.val_loss - res_full.val_loss) < 5e-3


def test_checkpoint_detects_corruption_and_fingerprint(tmp_path, monkeypatch):
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    ck = str(tmp_path / "c.bin")
    save_checkpoint(ck, "abc", 1, {"w": torch.ones(3)}, {}, {"file_idx": 0, "pos": 0})
    raw = bytearray(open(ck, "rb").read())
    raw[-1] ^= 1
    open(ck, "wb").write(raw)
    with pytest.raises(ValueError, match="corrupted"):
        load_checkpoint(ck)
    save_checkpoint(ck, "abc", 1, {"w": torch.ones(3)}, {}, {"file_idx": 0, "pos": 0})
    s = family_preset("tiny_cpu")
    s.mode, s.train.resume_from = "smoke", ck
    with pytest.raises(RuntimeError, match="fingerprint"):
        quiet(s).run()


def test_cli_prints_key_value_protocol(tmp_path):
    env = dict(os.environ, PGB_DATA_ROOT=str(tmp_path / "d"), PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "parameter_golf_b200.train", "run", "--family", "tiny_cpu", "--mode", "smoke",
                          "--artifact", str(tmp_path / "x.pgrs"), "train.seed=7"], capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    kv = dict(l.split("=", 1) for l in out.stdout.splitlines() if "=" in l and not l.startswith("record_audit_json"))
    assert kv["steps"] == "4" and kv["mode"] == "smoke" and float(kv["val_bpb"]) > 0


def test_two_cpu_ranks_stay_in_sync(tmp_path):
    """gloo ranks: each reads its own span, gradients are averaged, and both end with identical weights."""
    script = tmp_path / "w.py"
    script.write_text(f"""
import os, sys, hashlib, torch
sys.path.insert(0, {ROOT!r})
import torch.distributed as dist
from parameter_golf_b200.spec import family_preset
from parameter_golf_b200.train import VariantRunner
from parameter_golf_b200.utils.logging import RunLog
dist.init_process_group('gloo')
s = family_preset('tiny_cpu'); s.mode = 'smoke'
s.train.backend = 'cpu'; s.train.rank = dist.get_rank(); s.train.world_size = 2
s.allow_unsupported_variants = True
s.train.artifact_path = {str(tmp_path)!r} + f'/a{{dist.get_rank()}}.pgrs'
s.quant.compression = 'none'
import parameter_golf_b200.spec as sp
orig = sp.RunSpec.validate
sp.RunSpec.validate = lambda self: self
res = VariantRunner(s, RunLog('r', rank=dist.get_rank(), console=False)).run()
open({str(tmp_path)!r} + f'/ok{{dist.get_rank()}}.txt', 'w').write(f'{{res.steps}} {{res.val_bpb!r}}')     # a file per rank: stdout lines of two ranks can interleave
""")
    env = dict(os.environ, PGB_DATA_ROOT=str(tmp_path / "d"), PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", str(free_port()), str(script)], capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert out.returncode == 0, (out.stdout[-1000:], out.stderr[-3000:])
    oks = [open(tmp_path / f"ok{r}.txt").read().split() for r in range(2)]
    assert oks[0][0] == oks[1][0] == "4" and oks[0][1] == oks[1][1], (oks, out.stderr[-1000:])     # identical reduced val_bpb on both ranks


def test_optional_record_ideas_train_export_and_reload_on_the_cpu_backend(tmp_path, monkeypatch):
    """YaRN tables, the value residual and two multi-token-prediction heads through the trainer: the heads are trained but not
    exported, the learned lambdas are, and the artifact reloads into an evaluable model."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_overrides(["model.value_residual=true", "model.mtp_num_heads=2", "model.mtp_loss_weight=0.2", "model.rope.mode=yarn",
                       "model.rope.yarn_max_len=1024", "model.rope.yarn_train_len=256"])
    s.train.total_iterations = 6
    s.train.artifact_path = str(tmp_path / "ideas.pgrs")
    s.eval.max_tokens = 512
    r = quiet(s)
    import parameter_golf_b200.train as tr
    monkeypatch.setattr(tr, "mode_max_steps", lambda spec, mode: 6)
    res = r.run()
    assert res.steps == 6 and np.isfinite(res.val_loss) and np.isfinite(res.train_loss_last)
    # zero-initialised heads: the first training loss is the uniform one plus 0.2 times the heads' uniform loss
    assert abs(res.train_loss_first - 1.2 * np.log(s.model.vocab_size)) < 0.05
    back = load_artifact(open(s.train.artifact_path, "rb").read(), s)
    assert "mtp_heads" not in back and back["vr_lambda"].shape == (s.model.num_layers, 2)
    assert float((back["vr_lambda"] - 0.5).abs().max()) > 0          # the lambdas moved
    ids = torch.randint(0, s.model.vocab_size, (1, 32))
    assert torch.isfinite(gpt.gpt_forward(s.model, back, ids, ids))


def test_lawa_average_replaces_the_final_weights(tmp_path, monkeypatch):
    """train.lawa_enabled: the exported weights are the mean of the windowed snapshots, not the last iterate or the EMA."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_overrides(["train.lawa_enabled=true", "train.lawa_k=2", "train.lawa_freq=2"])
    s.train.total_iterations = 6
    s.train.artifact_path = str(tmp_path / "lawa.pgrs")
    s.eval.max_tokens = 512
    r = quiet(s)
    import parameter_golf_b200.train as tr
    monkeypatch.setattr(tr, "mode_max_steps", lambda spec, mode: 6)
    snaps = []
    real = tr.Lawa.collect

    def spy(self, params):
        real(self, params)
        snaps.append({k: v.detach().float().cpu().clone() for k, v in params.items()})
    monkeypatch.setattr(tr.Lawa, "collect", spy)
    exported = {}
    real_export = tr.export_model

    def grab(spec, params, *a, **k):
        exported.update({n: v.detach().float().cpu().clone() for n, v in params.items()})
        return real_export(spec, params, *a, **k)
    monkeypatch.setattr(tr, "export_model", grab)
    res = r.run()
    assert res.steps == 6 and len(snaps) == 3 and any("lawa:applying LAWA averaging k=2" in l for l in r.log.lines)
    for name in ("qo_bank", "tok_emb", "attn_scale"):
        want = (snaps[1][name] + snaps[2][name]) / 2
        assert torch.allclose(exported[name], want, atol=1e-6), name
    assert not torch.allclose(exported["qo_bank"], snaps[2]["qo_bank"], atol=1e-6)      # not simply the last iterate


def test_training_on_exported_text_shards_and_bpb_from_the_byte_sidecar(tmp_path, monkeypatch):
    """Local text -> tokenizer -> shards -> trainer -> evaluation: the bits-per-byte denominator read from the per-position
    byte sidecar equals the one derived from the tokenizer's piece table."""
    import json
    from parameter_golf_b200.data import text_shards as T
    rng = np.random.default_rng(0)
    words = ["alpha", "beta", "gamma", "delta", "tensor", "memory", "kernel", "golf", "parameter", "stream", "42", "the", "of", "and"]
    docs = [" ".join(rng.choice(words, size=int(rng.integers(20, 60)))) + "." for _ in range(500)]
    model = T.train_sentencepiece(iter(docs), 300, str(tmp_path / "tok" / "sp"))
    tok = T.load_sentencepiece(model)
    out = tmp_path / "shards"
    T.export_shards(iter(docs), tok, str(out), num_val_docs=60, shard_tokens=1 << 20)

    def run(extra):
        s = family_preset("tiny_cpu")
        s.mode = "smoke"
        s.apply_overrides([f"model.vocab_size={tok.vocab_size}", "train.seq_len=64", "model.train_seq_len=64", "model.eval_seq_len=64",
                           "train.batch_tokens=512", f"train.train_data_pattern={out}/fineweb_train_*.bin",
                           f"train.validation_data_pattern={out}/fineweb_val_*.bin", "eval.stride=64"] + extra)
        s.train.total_iterations = 3
        s.train.artifact_path = str(tmp_path / "a.pgrs")
        s.eval.max_tokens = 1024
        import parameter_golf_b200.train as tr
        monkeypatch.setattr(tr, "mode_max_steps", lambda spec, mode: 3)
        return quiet(s).run()

    a = run([f"eval.tokenizer_vocab_path={model}"])
    b = run([f"eval.caseops_byte_sidecar_pattern={out}/fineweb_val_bytes_*.bin"])
    # two runs of the same configuration agree only to the rounding of threaded CPU reductions (a few int6 codes flip), so the
    # losses are compared loosely and the byte counts, which are what this test is about, through the bpb / loss ratio
    assert np.isfinite(a.val_bpb) and a.val_loss == pytest.approx(b.val_loss, rel=1e-4)
    assert a.val_bpb / a.val_loss == pytest.approx(b.val_bpb / b.val_loss, rel=1e-9)
    assert abs(a.train_loss_first - np.log(tok.vocab_size)) < 0.2


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_parallel_muon_on_cpu_ranks_matches_the_replicated_optimizer(tmp_path, world):
    """gloo ranks with different data: three steps of the sharded optimizer (gradient slots reduced to their owners, momentum
    and Newton-Schulz on the owned slots only, all-gather of the new slots, clip factor from one scalar all-reduce) leave every
    rank with the parameters the replicated all-reduce path produces. With three ranks the two-slot MLP banks leave the last
    rank without a slot."""
    script = tmp_path / "w.py"
    script.write_text(f"""
import sys
sys.path.insert(0, {ROOT!r})
import torch, torch.distributed as dist
dist.init_process_group('gloo')
rank, world = dist.get_rank(), dist.get_world_size()
from parameter_golf_b200.models import gpt
from parameter_golf_b200.spec import family_preset
from parameter_golf_b200.train import OracleBackend
def backend(mode):
    s = family_preset('tiny_cpu')
    s.train.world_size, s.train.rank = world, rank
    s.train.distributed_optimizer_backend = mode
    s.train.grad_clip_norm = 0.05                      # small enough to bite, so the agreed norm matters
    s.validate()
    return OracleBackend(s, gpt.init_params(s.model, 11)), s
A, s = backend('all_reduce_replicated_muon')
B, _ = backend('sharded_parallel_muon')
assert B.sharded and not A.sharded
g = torch.Generator().manual_seed(100 + rank)
for step in range(3):
    ids = torch.randint(0, s.model.vocab_size, (2, 64), generator=g)
    tgt = torch.randint(0, s.model.vocab_size, (2, 64), generator=g)
    A.train_step([(ids, tgt)], 1.0, 0.95, False)
    B.train_step([(ids, tgt)], 1.0, 0.95, False)
worst = max(float((A.params[k] - B.params[k]).abs().max()) for k in A.params)
moved = float((A.params['qo_bank'] - gpt.init_params(s.model, 11)['qo_bank']).abs().max())
own = [tuple(b.shape) for b in B.muon.bufs]
full = B.muon.state_dict()['bufs']
mom = max(float((f - a).abs().max()) for f, a in zip(full, A.muon.bufs))
# every rank holds the same parameters
flat = torch.cat([B.params[k].reshape(-1) for k in sorted(B.params)])
ref = flat.clone()
dist.broadcast(ref, 0)
open({str(tmp_path)!r} + f'/res{{rank}}.txt', 'w').write(' '.join(str(x) for x in ('RES', rank, worst, moved, mom, float((flat - ref).abs().max()), own[2][0])))
""")
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                          "--master-port", str(free_port()), str(script)], capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    rows = [open(tmp_path / f"res{r}.txt").read().split() for r in range(world)]      # one file per rank: prints of several ranks interleave
    for _, rank, worst, moved, mom, spread, up_slots in rows:
        assert float(moved) > 1e-3                                   # the optimizer did something
        assert float(worst) < 2e-5 and float(mom) < 2e-5, (worst, mom)
        assert float(spread) == 0.0
        assert int(up_slots) == (1 if int(rank) < 2 else 0)         # tiny_cpu has two layers: two MLP slots


def test_cli_accepts_the_reference_trainer_flag_names(tmp_path):
    """pg-train/src/main.rs:58-122: --builtin, --seq-len, --batch-tokens, --max-steps, --eval-stride, --quant-scheme, ... map to
    spec keys; `plan` shows the result without running anything."""
    env = dict(os.environ, PGB_DATA_ROOT=str(tmp_path / "d"), PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "parameter_golf_b200.train", "run", "--builtin", "tiny_cpu", "--mode", "smoke", "--seq-len", "128",
                          "--batch-tokens", "1024", "--max-steps", "2", "--eval-stride", "32", "--eval-max-tokens", "512", "--quant-scheme",
                          "gptq_lite_int6", "--min-lr-scale", "0.1", "--attention-backend", "cudnn", "--fast-bank-updates",
                          "--artifact", str(tmp_path / "x.pgrs")], capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    kv = dict(l.split("=", 1) for l in out.stdout.splitlines() if "=" in l and not l.startswith("record_audit_json"))
    assert kv["steps"] == "2" and float(kv["val_bpb"]) > 0
    from parameter_golf_b200.train import REFERENCE_FLAGS
    s = family_preset("tiny_cpu")
    for key in REFERENCE_FLAGS.values():                   # every mapped key exists in the spec
        obj = s
        for part in key.split("."):
            assert hasattr(obj, part), key
            obj = getattr(obj, part)


def test_sharded_optimizer_state_survives_a_change_of_world_size(tmp_path):
    """Elastic restart: the checkpointed optimizer state is the full momentum (gathered from the owners), so a job resumed on a
    different number of ranks re-slices it; gathering it again gives back exactly what was saved."""
    def launch(world, body):
        script = tmp_path / f"w{world}.py"
        script.write_text(f"""
import sys
sys.path.insert(0, {ROOT!r})
import torch, torch.distributed as dist
dist.init_process_group('gloo')
rank, world = dist.get_rank(), dist.get_world_size()
from parameter_golf_b200.models import gpt
from parameter_golf_b200.spec import family_preset
from parameter_golf_b200.train import OracleBackend
s = family_preset('tiny_cpu')
s.train.world_size, s.train.rank = world, rank
s.train.distributed_optimizer_backend = 'sharded_parallel_muon'
s.validate()
path = {str(tmp_path / 'opt.pt')!r}
""" + body)
        env = dict(os.environ, PYTHONPATH=ROOT)
        out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                              "--master-port", str(free_port()), str(script)], capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
        assert out.returncode == 0, out.stderr[-3000:]

    launch(2, """
B = OracleBackend(s, gpt.init_params(s.model, 11))
g = torch.Generator().manual_seed(7 + rank)
for _ in range(2):
    ids = torch.randint(0, s.model.vocab_size, (2, 64), generator=g)
    B.train_step([(ids, ids)], 1.0, 0.95, False)
st = B.state_dict()                      # a collective
if rank == 0:
    torch.save({'opt': st, 'params': B.params}, path)
""")
    launch(3, """
ck = torch.load(path, weights_only=False)
B = OracleBackend(s, {k: v.clone() for k, v in ck['params'].items()})
B.load_state_dict(ck['opt'])
assert [tuple(b.shape)[0] for b in B.muon.bufs][:2] == ([2, 2] if rank < 2 else [0, 0])      # four attention slots over three ranks
again = B.state_dict()
for a, b in zip(again['muon']['bufs'], ck['opt']['muon']['bufs']):
    assert torch.equal(a, b)
assert float(ck['opt']['muon']['bufs'][0].abs().max()) > 0
ids = torch.randint(0, s.model.vocab_size, (2, 64), generator=torch.Generator().manual_seed(rank))
assert B.train_step([(ids, ids)], 1.0, 0.95, False) > 0
""")


def test_trainer_resumes_a_two_rank_sharded_run_on_four_ranks(tmp_path):
    """Elastic restart through the trainer: two gloo ranks with the sharded optimizer write a checkpoint (a collective: the
    owners' momentum is gathered, rank 0 writes, the others wait), four ranks resume it, continue from the saved step with the
    same global batches, and the run matches one that never stopped (the data stream position is global, the optimizer state is
    re-sliced, four ranks average the same eight sequences two ranks did)."""
    def launch(world, tag, extra):
        script = tmp_path / f"{tag}.py"
        script.write_text(f"""
import os, sys, json
sys.path.insert(0, {ROOT!r})
import torch.distributed as dist
from parameter_golf_b200.spec import family_preset
from parameter_golf_b200.train import VariantRunner
import parameter_golf_b200.train as tr
from parameter_golf_b200.utils.logging import RunLog
dist.init_process_group('gloo')
s = family_preset('tiny_cpu')
s.mode = 'smoke'
s.train.rank, s.train.world_size = dist.get_rank(), dist.get_world_size()
s.apply_overrides(['train.distributed_optimizer_backend=sharded_parallel_muon', 'train.batch_tokens=2048', 'train.grad_accum_steps=1'] + {extra!r})
s.train.artifact_path = {str(tmp_path)!r} + '/{tag}.pgrs'
s.eval.max_tokens = 512
tr.step_batch_plan = lambda spec, mode: (2048, 1)
tr.mode_max_steps = lambda spec, mode: spec.train.total_iterations
r = VariantRunner(s, RunLog('r', rank=dist.get_rank(), console=False))
res = r.run()
if dist.get_rank() == 0:
    losses = [float(l.split('train_loss:')[1].split()[0]) for l in r.log.lines if l.startswith('step:')]
    json.dump({{'losses': losses, 'val_loss': res.val_loss, 'steps': res.steps}}, open({str(tmp_path)!r} + '/{tag}.json', 'w'))
""")
        env = dict(os.environ, PGB_DATA_ROOT=str(tmp_path / "d"), PYTHONPATH=ROOT)
        out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                              "--master-port", str(free_port()), str(script)], capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
        assert out.returncode == 0, out.stderr[-3000:]
        import json
        return json.load(open(tmp_path / f"{tag}.json"))

    ck = str(tmp_path / "ck.bin")
    full = launch(2, "full", ["train.total_iterations=4"])
    launch(2, "first", ["train.total_iterations=2", "train.checkpoint_every=2", f"train.checkpoint_path={ck}"])
    resumed = launch(4, "resumed", ["train.total_iterations=4", f"train.resume_from={ck}"])
    assert full["steps"] == 4 and resumed["steps"] == 2
    # rank 0 logs the loss of its own share of the batch (four sequences of eight with two ranks, two with four), so the logged
    # training losses differ; the model does not: same global gradient and optimizer state, so the same validation loss up to
    # what the int6 export makes of last-bit differences in the weights (the single-process resume test allows the same)
    assert abs(resumed["val_loss"] - full["val_loss"]) < 1e-2, (resumed["val_loss"], full["val_loss"])


def test_ternary_family_trains_with_its_estimator_and_round_trips(tmp_path, monkeypatch):
    """Ternary QAT from the first step, ternary export with xz, FP8 storage of the small tensors, YaRN tables, three
    Newton-Schulz steps: the pieces of the ternary record's recipe through the trainer at a toy size."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_overrides(["model.qat_kind=ternary", "model.qat_ternary_group=64", "quant.ternary_group=64", "quant.scheme=ternary_b158",
                       "quant.compression=lzma9", "quant.float_storage=fp8", "quant.prune_to_target=false", "train.qat_enabled=true",
                       "train.muon_ns_steps=3", "model.rope.mode=yarn", "model.rope.dims=16", "model.rope.yarn_max_len=1024",
                       "model.rope.yarn_train_len=256", "model.bigram.enabled=true", "model.bigram.vocab_size=128", "model.bigram.dim=32",
                       "model.fp8_qat=true", "model.softcap_kind=poly5", "model.z_loss_weight=0.0001", "model.logit_softcap=10",
                       "model.embed_dim=48"])
    s.train.total_iterations = 4
    s.train.artifact_path = str(tmp_path / "t.pgrs")
    s.eval.max_tokens = 512
    import parameter_golf_b200.train as tr
    monkeypatch.setattr(tr, "mode_max_steps", lambda spec, mode: 4)
    r = quiet(s)
    res = r.run()
    assert res.steps == 4 and np.isfinite(res.val_loss) and res.budget_ok
    blob = open(s.train.artifact_path, "rb").read()
    assert blob[:6] == bytes([0xFD]) + b"7zXZ" + bytes([0])           # an xz stream
    back = load_artifact(blob, s)
    codes = (back["mlp_up_bank"].reshape(-1, 64) / back["mlp_up_bank"].reshape(-1, 64).abs().amax(-1, keepdim=True).clamp_min(1e-12)).round()
    assert set(codes.unique().tolist()) <= {-1.0, 0.0, 1.0}
    assert torch.equal(back["bigram_embed"], back["bigram_embed"].to(torch.float8_e4m3fn).float())      # stored as e4m3


def test_binary_family_recipe_trains_and_round_trips(tmp_path, monkeypatch):
    """The binary submission's recipe at a toy size through the trainer: 1-bit QAT from the first step with the matching export,
    xz, FP8 small tensors, normed output projections, the per-block smear, the vocabulary bias, the time-fraction warm-down."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_overrides(["model.qat_kind=binary", "model.qat_ternary_group=64", "quant.ternary_group=64", "quant.scheme=binary_b1",
                       "quant.compression=lzma9", "quant.float_storage=fp8", "quant.prune_to_target=false", "train.qat_enabled=true",
                       "train.muon_ns_steps=3", "model.normed_out_proj=true", "model.block_smear=true", "model.vocab_bias=true",
                       "model.softcap_kind=poly5", "model.logit_softcap=10", "model.embed_dim=48", "model.fp8_qat=true",
                       "train.warmdown_frac=0.5", "train.ema_decay=0", "train.swa_enabled=false"])
    s.train.total_iterations = 4
    s.train.artifact_path = str(tmp_path / "b.pgrs")
    s.eval.max_tokens = 512
    import parameter_golf_b200.train as tr
    monkeypatch.setattr(tr, "mode_max_steps", lambda spec, mode: 4)
    seen = []
    real = tr.OracleBackend.train_step

    def spy(self, batches, scale, mom, qat):
        seen.append((scale, qat))
        return real(self, batches, scale, mom, qat)
    monkeypatch.setattr(tr.OracleBackend, "train_step", spy)
    res = quiet(s).run()
    assert res.steps == 4 and np.isfinite(res.val_loss) and res.budget_ok
    assert [q for _, q in seen] == [True] * 4
    assert seen[0][0] == 1.0 and seen[-1][0] < 1.0                    # the second half of the run (by time or by steps) decays
    back = load_artifact(open(s.train.artifact_path, "rb").read(), s)
    grp = back["mlp_down_bank"].reshape(-1, 64).abs()
    assert torch.allclose(grp, grp[:, :1].expand_as(grp))             # sign codes: one magnitude per group
    assert back["block_smear_gate"].shape == (s.model.num_layers, s.model.model_dim) and back["vocab_bias"].shape == (s.model.vocab_size,)
    assert float(back["block_smear_gate"].abs().max()) > 0.0          # the gates moved off their zero start


def test_cycled_recurrent_model_trains_exports_and_reloads(tmp_path, monkeypatch):
    """The depth-recurrence submission's shape at a toy size: three unique blocks cycled to six virtual layers with per-depth
    adapters, noisy QAT on the shared blocks, 8-bit codes for the (all shared) banks; the artifact carries the adapters."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_env({"NUM_UNIQUE_BLOCKS": "3", "EFFECTIVE_DEPTH": "6", "DEPTH_LORA_RANK": "4", "XSA_LAST_N": "2"})
    s.apply_overrides(["model.qat_kind=noise", "train.qat_enabled=true", "quant.matrix_bits=8", "quant.prune_to_target=false"])
    s.train.total_iterations = 4
    s.train.artifact_path = str(tmp_path / "r.pgrs")
    s.eval.max_tokens = 512
    import parameter_golf_b200.train as tr
    monkeypatch.setattr(tr, "mode_max_steps", lambda spec, mode: 4)
    captured = {}
    real_export = tr.export_model

    def spy(spec, params, *a, **k):
        captured["p"] = {n: v.detach().clone() for n, v in params.items()}
        return real_export(spec, params, *a, **k)
    monkeypatch.setattr(tr, "export_model", spy)
    res = quiet(s).run()
    assert res.steps == 4 and np.isfinite(res.val_loss) and np.isfinite(res.train_loss_last)
    p = captured["p"]
    assert p["depth_lora_q_up"].shape == (6, s.model.model_dim, 4) and float(p["depth_lora_q_up"].abs().max()) > 0     # moved off zero
    back = load_artifact(open(s.train.artifact_path, "rb").read(), s)
    for k in ("depth_lora_q_down", "depth_lora_q_up", "depth_lora_v_down", "depth_lora_v_up", "skip_weights"):
        assert back[k].shape == p[k].shape and torch.allclose(back[k], p[k].half().float(), atol=0), k
    assert float((back["qo_bank"] - p["qo_bank"]).abs().max()) <= float(p["qo_bank"].abs().amax()) / 127


def test_sequence_and_batch_curriculum_switches_at_its_fractions(tmp_path, monkeypatch):
    """SEQ_LEN_START / BATCH_TOKENS_START of the ternary record: short sequences and a small batch first, the full shapes once the
    given fraction of the steps (no wall-clock cap here) has passed."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "record_shaped_proxy"
    s.apply_env({"SEQ_LEN_START": "64", "SEQ_SCHEDULE_FRACTION": "0.5", "BATCH_TOKENS_START": "512", "BATCH_SCHEDULE_FRACTION": "0.25"})
    s.train.batch_tokens, s.train.total_iterations = 1024, 8
    s.train.artifact_path = str(tmp_path / "c.pgrs")
    s.eval.max_tokens = 512
    s.validate()
    import parameter_golf_b200.train as tr
    shapes = []
    real = tr.OracleBackend.train_step

    def spy(self, batches, scale, mom, qat):
        shapes.append(tuple(batches[0][0].shape))
        return real(self, batches, scale, mom, qat)
    monkeypatch.setattr(tr.OracleBackend, "train_step", spy)
    res = quiet(s).run()
    assert res.steps == 8
    # steps 0-1: 512 tokens as rows of 64; steps 2-3: the full 1024 tokens, still rows of 64; from step 4: rows of 256
    assert shapes == [(8, 64)] * 2 + [(16, 64)] * 2 + [(4, 256)] * 4
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["train.seq_len_start=1024"]).validate()
    with pytest.raises(ValueError):
        family_preset("tiny_cpu").apply_overrides(["train.seq_len_start=100"]).validate()


def test_ema_starts_at_its_fraction_of_the_run(tmp_path, monkeypatch):
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_env({"EMA_DECAY": "0.9", "EMA_START_FRACTION": "0.5"})
    s.train.swa_enabled = False
    s.train.artifact_path = str(tmp_path / "e.pgrs")
    s.eval.max_tokens = 512
    import parameter_golf_b200.train as tr
    calls = []
    real = tr.Ema.update
    monkeypatch.setattr(tr.Ema, "update", lambda self, p: (calls.append(1), real(self, p))[1])
    res = quiet(s).run()
    assert res.steps == 4 and len(calls) == 2           # the steps that begin at progress 2/4 and 3/4
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["train.ema_start_fraction=0.5"]).validate()


def test_periodic_validation_logs_and_does_not_count_as_training_time(tmp_path, monkeypatch):
    """VAL_LOSS_EVERY of the baseline trainer (train_gpt.py:964-994): the current weights on the validation split every N steps
    and at the last step; the clock that drives the wall-clock cap and the step average is stopped meanwhile."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "record_shaped_proxy"
    s.apply_env({"VAL_LOSS_EVERY": "3"})
    s.train.total_iterations = 7
    s.train.artifact_path = str(tmp_path / "v.pgrs")
    s.eval.max_tokens = 1024
    r = quiet(s)
    lines = []
    real_info = r.log.info
    r.log.info = lambda msg: (lines.append(msg), real_info(msg))[1]
    now = [0.0]

    def clock():                     # one second per reading: validation would add readings if it ran on this clock
        now[0] += 1.0
        return now[0]
    r.clock = clock
    res = r.run()
    assert [h[0] for h in res.val_history] == [3, 6, 7]
    assert all(np.isfinite(h[1]) and h[2] > 0 for h in res.val_history)
    assert res.val_history[-1][1] < res.val_history[0][1]                          # it learns between the validations
    vals = [l for l in lines if " val_loss:" in l and l.startswith("step:")]
    assert len(vals) == 3 and "val_bpb:" in vals[0] and "train_time:" in vals[0]
    assert not any(k.startswith("val_history") for k in (l.split("=")[0] for l in res.key_value_lines()))
    # without the option nothing is evaluated during training
    s.train.val_loss_every = 0
    assert quiet(s).run().val_history == []


def test_qat_switches_on_for_the_last_fraction_of_the_run(tmp_path, monkeypatch):
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "record_shaped_proxy"
    s.apply_overrides(["train.qat_fraction=0.25", "train.late_qat_threshold=0", "train.total_iterations=8"])
    s.train.artifact_path = str(tmp_path / "q.pgrs")
    s.eval.max_tokens = 512
    import parameter_golf_b200.train as tr
    seen = []
    real = tr.OracleBackend.train_step
    monkeypatch.setattr(tr.OracleBackend, "train_step", lambda self, b, scale, mom, qat: (seen.append(qat), real(self, b, scale, mom, qat))[1])
    quiet(s).run()
    assert seen == [False] * 6 + [True] * 2


def test_record_gate_on_the_measured_step_time(tmp_path, monkeypatch):
    """Record mode fails closed when steps are slower than train.record_max_ms_per_step; the measurement leaves out the first
    train.timing_skip_steps steps (pg-train/src/lib.rs:1509-1521, :4129-4134)."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.train.timing_skip_steps = 1
    s.train.artifact_path = str(tmp_path / "g.pgrs")
    s.eval.max_tokens = 512
    r = quiet(s)
    now, calls = [0.0], []

    def clock():
        now[0] += 10.0 if len(calls) == 2 else 0.05           # the reading that ends the first step comes 10 s late
        calls.append(1)
        return now[0]
    r.clock = clock
    res = r.run()
    assert res.steps == 4 and res.step_avg_ms > 2000 and res.measured_ms_per_step < 500       # the slow first step is left out
    # the gate itself applies to record runs only
    import parameter_golf_b200.train as tr
    with pytest.raises(RuntimeError, match="too slow"):
        tr.check_record_step_time("record", 100, 131.0, 130.0)
    tr.check_record_step_time("record", 100, 129.0, 130.0)
    tr.check_record_step_time("record", 100, 500.0, 0.0)
    tr.check_record_step_time("record_shaped_proxy", 100, 500.0, 130.0)
    e = family_preset("record_11l").apply_env({"PG_RECORD_MAX_MS_PER_STEP": "90", "PG_RECORD_TIMING_SKIP_STEPS": "5"})
    assert e.train.record_max_ms_per_step == 90.0 and e.train.timing_skip_steps == 5


def test_result_lines_also_carry_the_reference_trainers_key_names(tmp_path, monkeypatch):
    """Scripts that parse the reference binary's ``key=value`` output (pg-train/src/main.rs:218-431) find the same names here."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.train.artifact_path = str(tmp_path / "k.pgrs")
    s.eval.max_tokens = 512
    res = quiet(s).run()
    kv = dict(l.split("=", 1) for l in res.key_value_lines())
    assert kv["run_name"] == "tiny_cpu" and kv["steps_completed"] == "4" and kv["train_backend"] == "cpu" and kv["world_size"] == "1"
    assert kv["variant_fingerprint"] == res.fingerprint and float(kv["ms_per_step"]) > 0 and kv["timing_steps"] == "4"
    assert int(kv["tokens_seen_global"]) == 4 * int(kv["global_batch_tokens"]) and kv["train_data_source"] == "synthetic_zipf_markov"
    assert kv["bpb_byte_source"] == "seeded_table" and kv["timing_backend"] == "host_perf_counter" and float(kv["timing_eval_ms"]) > 0
    assert kv["steps"] == "4" and "val_bpb" in kv                       # this framework's own names stay


def test_frontier_algorithm_notes_are_informational():
    from parameter_golf_b200.train import frontier_algorithm_notes
    f = family_preset("frontier_1855_like")
    f.quant.lqer.enabled, f.eval.caseops_byte_sidecar_pattern = True, "v_bytes_*.bin"
    assert frontier_algorithm_notes(f) == []
    r = frontier_algorithm_notes(family_preset("record_11l"))
    assert any("document boundaries" in n for n in r) and any("LQER" in n for n in r) and any("SparseAttnGate" in n for n in r)


def test_cli_log_file_starts_with_the_spec_and_the_environment(tmp_path):
    env = dict(os.environ, PGB_DATA_ROOT=str(tmp_path / "d"), PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-m", "parameter_golf_b200.train", "run", "--family", "tiny_cpu", "--mode", "smoke", "--log-dir", str(tmp_path / "logs"),
                          "--artifact", str(tmp_path / "x.pgrs")], capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    text = open(tmp_path / "logs" / "tiny_cpu.txt").read()
    assert text.startswith("=" * 100) and 'family = "tiny_cpu"' in text and "torch=" in text and "step:4/4 train_loss:" in text
    assert "record_audit_json=" in text and "\nval_bpb=" in text and "steps_completed=4" in text


def test_preflight_checks_a_planned_run_without_a_device(tmp_path, capsys):
    from parameter_golf_b200.data.shards import write_shard, write_synthetic_dataset
    from parameter_golf_b200.train import main, preflight
    root = str(tmp_path / "shards")
    write_synthetic_dataset(root, 1024, train_tokens=1 << 16, val_tokens=1 << 12, seed=1)
    s = family_preset("record_11l")
    s.mode = "record_shaped_proxy"
    s.train.world_size, s.train.artifact_path = 8, str(tmp_path / "out" / "a.pgrs")
    s.train.train_data_pattern, s.train.validation_data_pattern = root + "/fineweb_train_*.bin", root + "/fineweb_val_*.bin"
    lines, ok = preflight(s)
    kv = dict(l.split("=", 1) for l in lines)
    assert not ok and "one step needs 786440" in kv["preflight.problem"]            # 65,536 tokens cannot feed one record step
    assert kv["preflight.tokens_per_step"] == "786432" and kv["preflight.local_sequences_per_micro_batch"] == "48"
    s.train.batch_tokens = 8 * 2048
    lines, ok = preflight(s)
    kv = dict(l.split("=", 1) for l in lines)
    assert ok and kv["preflight.train_tokens"] == str(1 << 16) and float(kv["preflight.train_data_passes"]) == pytest.approx(8 * (8 * 2048 + 8) / 65536, abs=1e-3)
    assert float(kv["preflight.engine_memory_gib"]) > 0 and int(kv["preflight.artifact_budget_bytes"]) < 16_000_000
    # a damaged shard and a missing sidecar are both reported
    bad = tmp_path / "shards" / "fineweb_train_000009.bin"
    bad.write_bytes(b"\\0" * 100)
    s.eval.caseops_byte_sidecar_pattern = str(tmp_path / "nothing_*.bin")
    lines, ok = preflight(s)
    probs = [l for l in lines if l.startswith("preflight.problem=")]
    assert not ok and any("fineweb_train_000009.bin" in p for p in probs) and any("byte sidecar" in p for p in probs)
    assert main(["preflight", "--family", "tiny_cpu", "--mode", "smoke", "--artifact", str(tmp_path / "x.pgrs")]) == 0
    assert "preflight.ok=true" in capsys.readouterr().out


def test_priming_steps_leave_no_trace(tmp_path, monkeypatch):
    """WARMUP_STEPS of the Python trainers: steps that run and are then undone (weights, optimizer state, data position, random
    state), so a primed run equals an unprimed one (train_gpt.py:937-961)."""
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))

    def run(prime):
        s = family_preset("tiny_cpu")
        s.mode = "smoke"
        s.apply_env({"WARMUP_STEPS": str(prime)})
        assert s.train.prime_steps == prime and s.train.warmup_steps == 0
        s.train.artifact_path = str(tmp_path / f"p{prime}.pgrs")
        s.eval.max_tokens = 512
        r = quiet(s)
        lines = []
        real = r.log.info
        r.log.info = lambda msg: (lines.append(msg), real(msg))[1]
        res = r.run()
        return res, lines
    plain, _ = run(0)
    primed, lines = run(3)
    assert [l for l in lines if l.startswith("warmup_step:")] == ["warmup_step:1/3", "warmup_step:2/3", "warmup_step:3/3"]
    assert primed.train_loss_first == pytest.approx(plain.train_loss_first, rel=1e-6) and primed.train_loss_last == pytest.approx(plain.train_loss_last, rel=1e-5)
    # (two identical runs differ in the last digits of the round-tripped validation loss: threaded CPU reductions move a few
    # weights across an int6 rounding boundary)
    assert abs(primed.val_loss - plain.val_loss) < 1e-4
    family_preset("record_11l").apply_overrides(["train.prime_steps=2"]).validate()          # accepted; the CUDA backends skip it with a log line


def test_code_churn_is_logged_for_discrete_weight_training(tmp_path, monkeypatch):
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    from parameter_golf_b200.train import code_churn
    s = family_preset("tiny_cpu")
    p = gpt.init_params(s.model, 1)
    s.model.qat_kind, s.model.qat_ternary_group = "binary", 64
    frac, prev = code_churn(s.model, p, None)
    assert frac == 0.0
    p2 = {k: v.clone() for k, v in p.items()}
    p2["kv_bank"][0, 0, :8] *= -1                                    # eight signs flip
    frac, _ = code_churn(s.model, p2, prev)
    assert frac == pytest.approx(8 / sum(p[b].numel() for b in gpt.BANKS))
    s.mode = "smoke"
    s.apply_env({"CHURN_LOG_EVERY": "2"})
    s.apply_overrides(["quant.scheme=binary_b1", "quant.ternary_group=64", "quant.prune_to_target=false", "train.qat_enabled=true"])
    s.train.artifact_path = str(tmp_path / "c.pgrs")
    s.eval.max_tokens = 512
    res = quiet(s).run()
    assert [h[0] for h in res.churn_history] == [2, 4] and res.churn_history[0][1] == 0.0 and 0.0 < res.churn_history[1][1] < 1.0


def test_trainer_picks_the_evaluation_temperature_from_its_grid(tmp_path, monkeypatch):
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_env({"TEMP_SCALING": "1"})
    s.eval.temperature_grid = [0.5, 1.0, 2.0]
    s.train.artifact_path = str(tmp_path / "t.pgrs")
    s.eval.max_tokens = 512
    r = quiet(s)
    lines = []
    real = r.log.info
    r.log.info = lambda msg: (lines.append(msg), real(msg))[1]
    res = r.run()
    search = [l for l in lines if l.startswith("temperature_search:")]
    assert len(search) == 1 and f"optimal_T:{res.eval_temperature}" in search[0] and res.eval_temperature in (0.5, 1.0, 2.0)
    import json
    table = json.loads(search[0].split("temperature_search:")[1].split(" optimal_T")[0])
    assert min(table, key=table.get) == str(res.eval_temperature) and np.isfinite(res.val_loss)
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["eval.auto_temperature=true"]).validate()


def test_matrices_can_be_trained_with_adamw_instead_of_muon(tmp_path, monkeypatch):
    monkeypatch.setenv("PGB_DATA_ROOT", str(tmp_path / "data"))
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.apply_env({"MATRIX_OPTIMIZER": "adam", "ADAM_LR": "0.003"})
    from parameter_golf_b200.train import split_param_groups
    p = gpt.init_params(s.model, 1)
    banks, groups = split_param_groups(s, p)
    assert banks == [] and groups[-1] == {"names": list(gpt.BANKS), "lr": 0.003}
    s.train.artifact_path = str(tmp_path / "m.pgrs")
    s.eval.max_tokens = 512
    res = quiet(s).run()
    assert res.steps == 4 and np.isfinite(res.val_loss)
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["train.matrix_optimizer=adamw"]).validate()
