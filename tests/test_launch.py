"""The local launcher: command lines, metric parsing, result JSON of attached and detached runs, byte sidecars."""
import json
import os
import subprocess
import sys
import time

import numpy as np
import pytest

from parameter_golf_b200 import launch as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_metric_parsing_and_per_step_figures():
    text = "steps=4\nval_bpb=3.25\nbudget_ok=true\nmode=smoke\ntrain_ms=100.0\n[rank0] noise=1\nbad key=1\nrecord_audit_json={\"gaps\": []}\nnot a metric\n"
    m = L.parse_key_value_metrics(text)
    assert m["steps"] == 4 and m["val_bpb"] == 3.25 and m["budget_ok"] is True and m["mode"] == "smoke"
    assert m["train_ms_per_step"] == 25.0 and m["record_audit_json"] == {"gaps": []}
    assert "noise" not in m and "bad key" not in m
    assert L.coerce_metric("1e-3") == 1e-3 and L.coerce_metric("17") == 17 and L.coerce_metric("abc") == "abc"


def test_command_lines():
    one = L.build_command("run", 1, ["--family", "tiny_cpu"])
    assert one[:4] == [sys.executable, "-m", "parameter_golf_b200.train", "run"] and one[-2:] == ["--family", "tiny_cpu"]
    many = L.build_command("run", 4, ["--spec", "s.toml"], port=1234)
    assert many[1:3] == ["-m", "torch.distributed.run"] and "--nproc-per-node=4" in many and many[many.index("--master-addr") + 1] == "127.0.0.1"
    assert many[many.index("--master-port") + 1] == "1234" and many[-1] == "train.world_size=4"
    assert L.build_command("run", 2, ["train.world_size=2"], port=1)[-1] == "train.world_size=2"          # not added twice
    ev = L.build_command("eval", 2, ["--artifact", "a"], port=1)
    assert "parameter_golf_b200.evalcli" in ev and "train.world_size=2" not in ev
    assert L.build_command("bench", 1, ["bench/gemm_bench.py", "--m", "128"])[1:] == ["bench/gemm_bench.py", "--m", "128"]
    with pytest.raises(SystemExit):
        L.build_command("bench", 1, [])


def test_attached_run_writes_the_result_json(tmp_path):
    env = dict(os.environ, PGB_DATA_ROOT=str(tmp_path / "d"), PYTHONPATH=ROOT)
    rj = str(tmp_path / "out" / "run.json")
    out = subprocess.run([sys.executable, "-m", "parameter_golf_b200.launch", "run", "--label", "tiny", "--result-json", rj, "--",
                          "--family", "tiny_cpu", "--mode", "smoke", "--artifact", str(tmp_path / "a.pgrs")],
                         capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    assert "val_bpb=" in out.stdout                                     # attached: the command's output is echoed
    r = json.load(open(rj))
    assert r["status"] == "ok" and r["returncode"] == 0 and r["label"] == "tiny" and r["metrics"]["steps"] == 4
    assert r["metrics"]["val_bpb"] > 0 and r["metrics"]["record_audit_json"]["mode"] == "smoke" and os.path.exists(r["log"])
    st = subprocess.run([sys.executable, "-m", "parameter_golf_b200.launch", "status", rj], capture_output=True, text=True, env=env, cwd=ROOT)
    assert st.returncode == 0 and "status=ok" in st.stdout and "steps=4" in st.stdout
    # a failing command is recorded as such, with the end of its output
    bad = str(tmp_path / "bad.json")
    out = subprocess.run([sys.executable, "-m", "parameter_golf_b200.launch", "run", "--result-json", bad, "--", "--family", "no_such_family"],
                         capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    r = json.load(open(bad))
    assert out.returncode != 0 and r["status"] == "failed" and r["returncode"] == out.returncode and "no_such_family" in r["tail"]


def test_detached_run_finishes_on_its_own(tmp_path):
    env = dict(os.environ, PGB_DATA_ROOT=str(tmp_path / "d"), PYTHONPATH=ROOT)
    rj = str(tmp_path / "run.json")
    t0 = time.time()
    out = subprocess.run([sys.executable, "-m", "parameter_golf_b200.launch", "run", "--detach", "--result-json", rj, "--",
                          "--family", "tiny_cpu", "--mode", "smoke", "--artifact", str(tmp_path / "a.pgrs")],
                         capture_output=True, text=True, env=env, cwd=ROOT, timeout=120)
    assert out.returncode == 0 and "detached=true" in out.stdout, out.stderr[-1500:]
    w = subprocess.run([sys.executable, "-m", "parameter_golf_b200.launch", "wait", rj, "--timeout", "240"], capture_output=True, text=True, env=env,
                       cwd=ROOT, timeout=300)
    assert w.returncode == 0 and "status=ok" in w.stdout, (w.stdout, w.stderr[-500:], time.time() - t0)
    assert json.load(open(rj))["metrics"]["steps"] == 4
    none = subprocess.run([sys.executable, "-m", "parameter_golf_b200.launch", "run", "--detach", "--", "--family", "tiny_cpu"], capture_output=True, text=True,
                          env=env, cwd=ROOT)
    assert none.returncode != 0 and "--result-json" in none.stderr


def test_byte_sidecars_follow_the_tokenizer_table(tmp_path):
    spm = pytest.importorskip("sentencepiece")
    from parameter_golf_b200.data.bpb import BpbLuts
    from parameter_golf_b200.data.shards import load_validation_byte_sidecar, load_validation_tokens, open_shard, write_shard
    corpus = tmp_path / "c.txt"
    corpus.write_text("\n".join(f"the quick brown fox {i} jumps over the lazy dog" for i in range(400)))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "tok"), vocab_size=320, model_type="bpe", byte_fallback=True,
                                   bos_id=1, eos_id=2, unk_id=3, pad_id=0, minloglevel=2)
    sp = spm.SentencePieceProcessor(model_file=str(tmp_path / "tok.model"))
    ids = np.array([1] + sp.encode("the lazy dog jumps over the quick fox 17"), dtype=np.uint16)
    write_shard(str(tmp_path / "fineweb_val_000000.bin"), ids[:9])
    write_shard(str(tmp_path / "fineweb_val_000001.bin"), ids[9:])
    names = L.ensure_byte_sidecars(str(tmp_path / "fineweb_val_*.bin"), str(tmp_path / "tok.model"), 320)
    assert [os.path.basename(n) for n in names] == ["fineweb_val_bytes_000000.bin", "fineweb_val_bytes_000001.bin"]
    side = load_validation_byte_sidecar(str(tmp_path / "fineweb_val_bytes_*.bin"))
    luts = BpbLuts.from_sentencepiece(str(tmp_path / "tok.model"), 320)
    want = luts.token_bytes(np.concatenate([[0], ids[:-1].astype(np.int64)]), ids.astype(np.int64))
    assert np.array_equal(side, want.astype(np.float32))                 # the previous token carries over the shard boundary
    assert int(side[1:].sum()) == len("the lazy dog jumps over the quick fox 17".encode())
    # a second call keeps what is there; the validation loader skips the sidecars that its pattern also matches
    stamp = os.path.getmtime(names[0])
    L.ensure_byte_sidecars(str(tmp_path / "fineweb_val_*.bin"), str(tmp_path / "tok.model"), 320)
    assert os.path.getmtime(names[0]) == stamp
    assert np.array_equal(load_validation_tokens(str(tmp_path / "fineweb_val_*.bin"), 4)[: len(ids)], ids[: len(load_validation_tokens(str(tmp_path / "fineweb_val_*.bin"), 4))])


def test_doctor_reports_the_environment_without_a_gpu(capsys):
    from parameter_golf_b200 import doctor
    info = doctor.collect()
    assert info["torch"] and "gloo" in info["dist_backends"] and isinstance(info["gpus"], list) and info["sm100_gpus"] == len(
        [g for g in info["gpus"] if g["capability"].startswith("10.")])
    assert doctor.main(["--json"]) == 0
    assert json.loads(capsys.readouterr().out)["python"] == info["python"]
    if not info["cuda_available"]:
        assert doctor.main(["--require-gpu"]) == 1
