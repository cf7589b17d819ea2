import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from parameter_golf_b200.models import gpt
from parameter_golf_b200.spec import RunSpec, family_preset
from parameter_golf_b200.utils import interop as I

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_safetensors_roundtrip_and_layout(tmp_path):
    t = {"a": torch.randn(3, 4), "b": torch.randn(5).half(), "c": torch.randn(2, 2).bfloat16()}
    p = str(tmp_path / "x.safetensors")
    I.write_safetensors(p, t, {"k": "v"})
    raw = open(p, "rb").read()
    hl = int.from_bytes(raw[:8], "little")
    hdr = json.loads(raw[8:8 + hl])
    assert hdr["a"] == {"dtype": "F32", "shape": [3, 4], "data_offsets": [0, 48]} and hdr["__metadata__"] == {"k": "v"}
    back = I.read_safetensors(p)
    assert all(torch.equal(back[k], t[k]) for k in t)
    with pytest.raises(ValueError):
        open(p, "wb").write(raw[:4])
        I.read_safetensors(p)


def test_name_map_roundtrip():
    s = family_preset("record_11l")
    s.model.num_layers, s.model.model_dim, s.model.num_heads, s.model.num_kv_heads = 2, 64, 2, 1
    s.model.value_embedding.enabled, s.model.value_embedding.layers = True, [0, 1]
    p = gpt.fill_deterministic(s.model)
    sd = I.to_python_state_dict(s.model, p)
    assert "blocks.1.attn.q_gain" in sd and "bigram.proj.weight" in sd and "ve_layer_scales.1" in sd
    back = I.from_python_state_dict(s.model, sd)
    assert set(back) == set(p) and all(torch.equal(back[k], p[k]) for k in p)
    # the optional parameters of the record script keep its names: value-residual lambdas, the update gate, the extra heads
    m = s.model
    m.value_residual, m.dtg, m.mtp_num_heads, m.tie_embeddings = True, True, 2, False
    p = gpt.fill_deterministic(m)
    sd = I.to_python_state_dict(m, p)
    assert sd["blocks.1.attn.vr_lambda"].shape == (2,) and sd["blocks.0.dtg_gate.weight"].shape == (1, 64) and sd["blocks.0.dtg_gate.bias"].shape == (1,)
    assert sd["mtp_heads.1.weight"].shape == (m.vocab_size, 64) and "lm_head.weight" in sd
    back = I.from_python_state_dict(m, sd)
    assert set(back) == set(p) and all(torch.equal(back[k], p[k]) for k in p)
    del sd["qo_bank"]
    with pytest.raises(KeyError):
        I.from_python_state_dict(s.model, sd)


def test_parity_report_tolerances():
    a = {"loss": torch.tensor(1.0), "grad.w": torch.ones(4)}
    b = {"loss": torch.tensor(1.0005), "grad.w": torch.ones(4) * 1.01, "grad.v": torch.ones(2)}
    r = I.compare_step_dumps(a, b)
    assert r.missing == ["grad.v"] and not r.ok and r.worst_grad_rel < 0.02
    del b["grad.v"]
    assert I.compare_step_dumps(a, b).ok
    b["grad.w"] = torch.ones(4) * 1.5
    assert not I.compare_step_dumps(a, b).ok


def test_shipped_specs_load_and_validate():
    for name in ("record_profile", "baseline_9l", "tiny_cpu", "ternary_10l", "binary_15l"):
        s = RunSpec.load(os.path.join(ROOT, "specs", f"{name}.toml")).validate()
        assert s.fingerprint() == family_preset(s.model.family).fingerprint()


def test_eval_cli_and_leaderboard_gate(tmp_path):
    from parameter_golf_b200.data.shards import write_shard, generate_markov_tokens
    from parameter_golf_b200.quant.export import export_model
    s = family_preset("tiny_cpu")
    art = str(tmp_path / "a.pgrs")
    export_model(s, gpt.init_params(s.model, 1), art)
    write_shard(str(tmp_path / "v_val_000000.bin"), generate_markov_tokens(256 * 3 + 1, 1024, 5))
    env = dict(os.environ, PYTHONPATH=ROOT)
    base = [sys.executable, "-m", "parameter_golf_b200.evalcli", "--artifact", art, "--family", "tiny_cpu", "--val-pattern", str(tmp_path / "v_val_*.bin")]
    out = subprocess.run(base, capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    kv = dict(l.split("=", 1) for l in out.stdout.splitlines() if "=" in l and not l.startswith("eval_audit_json"))
    assert kv["eval_kind"] == "sliding" and float(kv["val_bpb"]) > 0 and "eval_audit_json=" in out.stdout
    # and under the reference evaluator's names (pg-eval/src/bin/run.rs)
    assert kv["eval_bpb"] == kv["val_bpb"] and kv["eval_status"] == "ok" and kv["eval_tokens"] == str(256 * 3) and kv["eval_stride"] == "64"
    assert int(kv["submission_total_bytes"]) == int(kv["artifact_bytes"]) + int(kv["code_bytes"])
    out = subprocess.run(base + ["--leaderboard", "--bytes", "placeholder", "--max-tokens", "300"], capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 2 and "placeholder" in out.stderr and "full validation set" in out.stderr


def test_eval_cli_accepts_the_reference_binary_flag_names(tmp_path):
    """``--builtin``, ``--val-data``, ``--stride``, ``--tokenizer-vocab``, ``--caseops-byte-sidecar`` (pg-eval/src/bin/run.rs:19-27)
    set the spec keys they name; with a byte sidecar the bits-per-byte denominator is the sidecar's sum."""
    import json
    from parameter_golf_b200.data.shards import write_shard, generate_markov_tokens
    from parameter_golf_b200.quant.export import export_model
    s = family_preset("tiny_cpu")
    art = str(tmp_path / "a.pgrs")
    export_model(s, gpt.init_params(s.model, 1), art)
    n = 256 * 2 + 1
    write_shard(str(tmp_path / "v_val_000000.bin"), generate_markov_tokens(n, 1024, 5))
    write_shard(str(tmp_path / "v_val_bytes_000000.bin"), np.full(n, 3, dtype=np.uint16))
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "parameter_golf_b200.evalcli", "--artifact", art, "--builtin", "tiny_cpu", "--val-data", str(tmp_path / "v_val_*.bin"),
           "--stride", "128", "--caseops-byte-sidecar", str(tmp_path / "v_val_bytes_*.bin")]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    kv = dict(l.split("=", 1) for l in out.stdout.splitlines() if "=" in l and not l.startswith("eval_audit_json"))
    audit = json.loads([l for l in out.stdout.splitlines() if l.startswith("eval_audit_json=")][0].split("=", 1)[1])
    assert audit["stride"] == 128
    # 3 bytes per token everywhere: bits per byte = loss / ln 2 / 3
    assert float(kv["val_bpb"]) == pytest.approx(float(kv["val_loss"]) / np.log(2) / 3, rel=1e-6)


def test_submission_manifest_counts_source_and_fails_closed(tmp_path):
    from parameter_golf_b200 import submission as Sub
    from parameter_golf_b200.quant.export import export_model
    s = family_preset("tiny_cpu")
    art = str(tmp_path / "a.pgrs")
    export_model(s, gpt.init_params(s.model, 1), art)
    code = tmp_path / "code"
    (code / "pkg" / "__pycache__").mkdir(parents=True)
    (code / "pkg" / "a.py").write_text("x = 1\n" * 100)
    (code / "pkg" / "k.cu").write_text("// kernel\n" * 50)
    (code / "pkg" / "lib.so").write_bytes(b"\0" * 5000)                 # build products are not source
    (code / "pkg" / "__pycache__" / "a.pyc").write_bytes(b"\0" * 999)
    man = Sub.build_manifest(art, [str(code)])
    assert man["code_file_count"] == 2 and man["code_bytes"] == 600 + 500 and man["code_bytes_by_type"] == {".cu": 500, ".py": 600}
    assert man["artifact"]["bytes"] == os.path.getsize(art) and man["artifact"]["tensors"] > 10
    assert man["artifact"]["variant_fingerprint"] == f"{s.fingerprint():016x}"
    assert man["under_budget"] and man["total_bytes"] == man["artifact"]["bytes"] + 1100
    out = tmp_path / "m" / "submission.json"
    assert Sub.main(["--artifact", art, "--code", str(code), "--out", str(out)]) == 0 and json.load(open(out))["code_bytes"] == 1100
    assert Sub.main(["--artifact", art, "--code", str(code), "--limit", str(man["total_bytes"])]) == 1      # the limit itself is over budget
    assert Sub.main(["--artifact", art, "--code", str(tmp_path / "missing")]) == 2
    assert Sub.main(["--artifact", str(tmp_path / "none.pgrs"), "--code", str(code)]) == 2


def test_eval_cli_temperature_search(tmp_path):
    from parameter_golf_b200.data.shards import write_shard, generate_markov_tokens
    from parameter_golf_b200.quant.export import export_model
    s = family_preset("tiny_cpu")
    art = str(tmp_path / "a.pgrs")
    export_model(s, gpt.init_params(s.model, 1), art)
    write_shard(str(tmp_path / "v_val_000000.bin"), generate_markov_tokens(256 * 2 + 1, 1024, 5))
    write_shard(str(tmp_path / "t_train_000000.bin"), generate_markov_tokens(256 * 4 + 1, 1024, 6))
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "parameter_golf_b200.evalcli", "--artifact", art, "--family", "tiny_cpu", "--val-pattern", str(tmp_path / "v_val_*.bin"),
           "--find-temperature", f"train.train_data_pattern={tmp_path}/t_train_*.bin", "eval.temperature_calibration_tokens=1024",
           "eval.temperature_grid=[0.9,1.0,1.1]"]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    kv = dict(l.split("=", 1) for l in out.stdout.splitlines() if "=" in l and not l.startswith("eval_audit_json"))
    assert float(kv["temperature"]) in (0.9, 1.0, 1.1) and len(json.loads(kv["temperature_search"])) == 3 and float(kv["val_bpb"]) > 0
    out = subprocess.run(cmd[:-3] + ["--device", "cuda"], capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode != 0


def test_eval_cli_runs_document_isolated_lora_ttt(tmp_path):
    """eval.adaptation_backend = doc_lora through the evaluation CLI on a stream of boundary-opened documents."""
    from parameter_golf_b200.data.shards import write_shard
    from parameter_golf_b200.quant.export import export_model
    s = family_preset("tiny_cpu")
    art = str(tmp_path / "a.pgrs")
    export_model(s, gpt.init_params(s.model, 1), art)
    rng = np.random.default_rng(0)
    docs = [np.concatenate([[1], rng.integers(2, 1024, size=int(rng.integers(40, 120)))]) for _ in range(5)]
    write_shard(str(tmp_path / "v_val_000000.bin"), np.concatenate(docs).astype(np.uint16))
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "parameter_golf_b200.evalcli", "--artifact", art, "--family", "tiny_cpu", "--val-pattern", str(tmp_path / "v_val_*.bin"),
           "eval.adaptation_backend=doc_lora", "eval.legal_score_first=true", "eval.doc_chunk_size=32", "eval.doc_lora_rank=4", "eval.doc_batch_size=4"]
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    kv = dict(l.split("=", 1) for l in out.stdout.splitlines() if "=" in l and not l.startswith("eval_audit_json"))
    assert kv["eval_kind"] == "doc_lora" and float(kv["val_bpb"]) > 0 and np.isfinite(float(kv["val_loss"]))


def test_eval_cli_document_lora_on_two_cpu_ranks_matches_one(tmp_path):
    """Documents are split over ranks in contiguous slices and the three sums reduced: without adapters (which are drawn from a
    per-rank generator) two ranks must print exactly the one-rank result."""
    from conftest import free_port
    from parameter_golf_b200.data.shards import write_shard
    from parameter_golf_b200.quant.export import export_model
    s = family_preset("tiny_cpu")
    art = str(tmp_path / "a.pgrs")
    export_model(s, gpt.init_params(s.model, 1), art)
    rng = np.random.default_rng(2)
    docs = [np.concatenate([[1], rng.integers(2, 1024, size=int(rng.integers(30, 90)))]) for _ in range(6)]
    write_shard(str(tmp_path / "v_val_000000.bin"), np.concatenate(docs).astype(np.uint16))
    env = dict(os.environ, PYTHONPATH=ROOT)
    tail = ["--artifact", art, "--family", "tiny_cpu", "--val-pattern", str(tmp_path / "v_val_*.bin"), "eval.adaptation_backend=doc_lora",
            "eval.legal_score_first=true", "eval.doc_chunk_size=32", "eval.doc_lora_rank=0", "eval.doc_batch_size=2"]
    one = subprocess.run([sys.executable, "-m", "parameter_golf_b200.evalcli"] + tail, capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", str(free_port()), "-m", "parameter_golf_b200.evalcli"] + tail,
                         capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert one.returncode == 0 and two.returncode == 0, (one.stderr[-800:], two.stderr[-1500:])
    get = lambda out: float([l for l in out.stdout.splitlines() if l.startswith("val_loss=")][0].split("=")[1])
    assert abs(get(one) - get(two)) < 1e-5            # the same tokens in differently shaped batches: equal up to float32 rounding


def test_leaderboard_rules_follow_the_reference_binary():
    """pg-eval/src/bin/run.rs:251-303: score-first, a boundary token for prefix-document TTT, the configured world size for the
    LoRA-phased evaluator, the byte sidecar when CaseOps is on."""
    import argparse
    from parameter_golf_b200.evalcli import leaderboard_violations
    args = argparse.Namespace(bytes="seeded", val_pattern="v_*.bin")
    s = family_preset("baseline_sp8192")
    assert leaderboard_violations(s, args) == []
    s.eval.legal_score_first = False
    assert any("legal_score_first" in b for b in leaderboard_violations(s, args))
    s = family_preset("baseline_sp8192")
    s.eval.adaptation_backend, s.model.smear_gate_boundary_token_id = "gpu_lora_phased", None
    assert any("boundary token" in b for b in leaderboard_violations(s, args))
    s.model.smear_gate_boundary_token_id, s.train.world_size = 1, 8
    assert any("world size" in b for b in leaderboard_violations(s, args))
    h = family_preset("hybrid_competitive_sp8192")
    assert any("caseops-byte-sidecar" in b for b in leaderboard_violations(h, args))
    h.eval.caseops_byte_sidecar_pattern = "x_bytes_*.bin"
    assert leaderboard_violations(h, args) == []
    args.bytes = "tokenizer"
    assert any("tokenizer-vocab" in b for b in leaderboard_violations(family_preset("baseline_sp8192"), args))


def test_interop_command_line_round_trip_and_parity_report(tmp_path, capsys):
    """state_dict (Python names) -> artifact -> state_dict; a step dump compared with itself passes, with a perturbed copy fails."""
    from parameter_golf_b200.data.shards import write_shard
    from parameter_golf_b200.utils import interop as I
    s = family_preset("tiny_cpu")
    p = gpt.init_params(s.model, 4)
    p["qo_bank"][s.model.num_layers:] = torch.randn_like(p["qo_bank"][s.model.num_layers:]) * 0.05
    p["mlp_down_bank"] = torch.randn_like(p["mlp_down_bank"]) * 0.05
    state = str(tmp_path / "model.safetensors")
    I.write_safetensors(state, {k: v.contiguous() for k, v in I.to_python_state_dict(s.model, p).items()})
    art, back = str(tmp_path / "m.pgrs"), str(tmp_path / "back.safetensors")
    assert I.main(["import", "--family", "tiny_cpu", "--state", state, "--artifact", art, "quant.prune_to_target=false"]) == 0
    assert I.main(["export", "--family", "tiny_cpu", "--artifact", art, "--state", back]) == 0
    rt = I.from_python_state_dict(s.model, I.read_safetensors(back))
    assert float((rt["kv_bank"] - p["kv_bank"]).abs().max()) < float(p["kv_bank"].abs().max()) / 20          # int6 round trip
    write_shard(str(tmp_path / "t.bin"), np.random.default_rng(0).integers(0, 1024, 2 * 64 + 1).astype(np.uint16))
    d1, d2 = str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors")
    args = ["dump-step", "--family", "tiny_cpu", "--state", state, "--tokens", str(tmp_path / "t.bin"), "--batch", "2", "--seq-len", "64", "--python-names"]
    assert I.main(args + ["--out", d1]) == 0 and I.main(args + ["--out", d2]) == 0
    dump = I.read_safetensors(d1)
    assert "grad.blocks.0.attn.q_gain" in dump and "grad.tok_emb.weight" in dump and float(dump["loss"]) > 0
    capsys.readouterr()
    assert I.main(["compare", d1, d2]) == 0 and "parity_ok=true" in capsys.readouterr().out
    dump["grad.qo_bank"] = dump["grad.qo_bank"] * 1.05
    I.write_safetensors(d2, dump)
    assert I.main(["compare", d1, d2]) == 1
    out = capsys.readouterr().out
    assert "parity_ok=false" in out and "worst_grad_name=grad.qo_bank" in out
