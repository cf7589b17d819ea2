"""Local launcher: run a training, evaluation or benchmark command on N GPUs of this node, attached or detached, and keep
its outcome as a result JSON.

Role of the reference's ``parameter-golf-rs/deploy/run_detached.py`` without the cloud service: that script wraps the train /
eval / bench binaries, writes a ``status: running`` record before the command starts (``:48-58``), parses the ``key=value``
lines the binaries print into typed metrics (``:61-87``), adds per-step timing figures (``:90-101``), writes the final record
atomically (``:34-45``) and can generate the validation byte sidecars a tokenizer implies (``:761-780``). Here the command is
``python -m torch.distributed.run`` on 127.0.0.1 (one process per GPU) or plain ``python`` for one process, and "detached" is
a supervisor process in its own session that outlives the caller.

    python -m parameter_golf_b200.launch run   --gpus 8 --result-json out/run.json -- --spec specs/record_profile.toml --mode record
    python -m parameter_golf_b200.launch eval  --gpus 8 --result-json out/eval.json -- --artifact a.pgrs --family record_11l --device cuda
    python -m parameter_golf_b200.launch bench --result-json out/gemm.json -- bench/gemm_bench.py
    python -m parameter_golf_b200.launch run   --detach --result-json out/run.json -- --family tiny_cpu --mode smoke
    python -m parameter_golf_b200.launch status out/run.json          # or: wait out/run.json --timeout 900
    python -m parameter_golf_b200.launch sidecar --val-pattern 'data/fineweb_val_[0-9]*.bin' --tokenizer-vocab tok.model
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import socket
import subprocess
import sys
import time
from typing import Dict, List, Optional

TAIL_LINES = 80
TARGETS = {"run": ["-m", "parameter_golf_b200.train", "run"], "eval": ["-m", "parameter_golf_b200.evalcli"], "bench": []}


def coerce_metric(raw: str):
    v = raw.strip()
    if v.lower() in ("true", "false"):
        return v.lower() == "true"
    try:
        return float(v) if any(c in v for c in ".eE") else int(v)
    except ValueError:
        return v


def parse_key_value_metrics(text: str) -> Dict[str, object]:
    """``key=value`` lines of the CLIs' stdout as typed metrics; ``*_json`` lines are decoded into nested objects."""
    out: Dict[str, object] = {}
    for line in text.splitlines():
        if "=" not in line or line.startswith("["):
            continue
        k, v = line.split("=", 1)
        k = k.strip()
        if not k or " " in k:
            continue
        if k.endswith("_json"):
            try:
                out[k] = json.loads(v)
            except ValueError:
                pass
            continue
        out[k] = coerce_metric(v)
    steps = out.get("steps")
    if isinstance(steps, int) and steps > 0:            # per-step figures for every *_ms total the trainer prints
        for k, v in list(out.items()):
            if k.endswith("_ms") and isinstance(v, (int, float)) and not isinstance(v, bool):
                out[f"{k}_per_step"] = float(v) / steps
    return out


def write_result(path: Optional[str], result: dict) -> None:
    if not path:
        return
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(result, f, indent=2, sort_keys=True)
        f.write("\n")
    os.replace(tmp, path)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def build_command(kind: str, gpus: int, rest: List[str], port: Optional[int] = None) -> List[str]:
    """The process line for ``kind`` in (run, eval, bench): one process, or one per GPU under ``torch.distributed.run``."""
    target = TARGETS[kind] + list(rest)
    if kind == "bench" and not rest:
        raise SystemExit("bench needs a script path after --")
    if kind == "run" and gpus > 1 and not any(a.startswith("train.world_size=") for a in rest):
        target.append(f"train.world_size={gpus}")
    if gpus <= 1:
        return [sys.executable] + target
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
            "--master-port", str(port or free_port())] + target


def supervise(cmd: List[str], label: str, result_json: Optional[str], log_path: Optional[str], echo: bool) -> int:
    """Run ``cmd`` to its end; stdout and stderr go to the log (and the terminal when attached), the result JSON is written before
    and after."""
    t0 = time.time()
    write_result(result_json, {"label": label, "command": cmd, "returncode": None, "status": "running", "pid": os.getpid(), "started": t0,
                               "log": log_path, "tail": ""})
    lines: List[str] = []
    log = open(log_path, "w", encoding="utf-8") if log_path else None
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, bufsize=1)
    try:
        for line in proc.stdout:
            lines.append(line)
            if log:
                log.write(line)
                log.flush()
            if echo:
                sys.stdout.write(line)
        rc = proc.wait()
    finally:
        if log:
            log.close()
    text = "".join(lines)
    write_result(result_json, {"label": label, "command": cmd, "returncode": rc, "status": "ok" if rc == 0 else "failed", "started": t0,
                               "seconds": round(time.time() - t0, 3), "log": log_path, "metrics": parse_key_value_metrics(text),
                               "tail": "".join(lines[-TAIL_LINES:])})
    return rc


def ensure_byte_sidecars(val_pattern: str, tokenizer_vocab: str, vocab_size: int) -> List[str]:
    """For every validation shard matched by ``val_pattern`` write the byte-count sidecar shard next to it
    (``fineweb_val_000000.bin`` -> ``fineweb_val_bytes_000000.bin``; existing ones are kept): entry ``i`` is the number of
    UTF-8 bytes token ``i`` stands for after token ``i - 1`` by the tokenizer's table rule, carried across shard boundaries."""
    import numpy as np
    from .data.bpb import BpbLuts
    from .data.shards import is_byte_sidecar_path, open_shard, write_shard
    luts = BpbLuts.from_sentencepiece(tokenizer_vocab, vocab_size)
    files = sorted(f for f in glob.glob(val_pattern) if not is_byte_sidecar_path(f))
    if not files:
        raise FileNotFoundError(f"no validation shard matches {val_pattern!r}")
    out, prev = [], 0
    for path in files:
        toks = np.asarray(open_shard(path)).astype(np.int64)
        name = os.path.join(os.path.dirname(path), os.path.basename(path).replace("_val_", "_val_bytes_", 1))
        if name == path:
            raise ValueError(f"cannot derive a sidecar name from {path!r} (no '_val_' in the file name)")
        if not os.path.exists(name):
            prevs = np.concatenate([[prev], toks[:-1]])
            write_shard(name, luts.token_bytes(prevs, toks).astype(np.uint16))
        prev = int(toks[-1]) if toks.size else prev
        out.append(name)
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.launch")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for kind in TARGETS:
        p = sub.add_parser(kind)
        p.add_argument("--gpus", type=int, default=1)
        p.add_argument("--label", default=kind)
        p.add_argument("--result-json")
        p.add_argument("--log")
        p.add_argument("--detach", action="store_true", help="return at once; a supervisor in its own session finishes the run")
        p.add_argument("--supervise", action="store_true", help=argparse.SUPPRESS)
        p.add_argument("--print-command", action="store_true", help="print the process line and exit")
    for name in ("status", "wait"):
        p = sub.add_parser(name)
        p.add_argument("result_json")
        p.add_argument("--timeout", type=float, default=0.0)
    p = sub.add_parser("sidecar")
    p.add_argument("--val-pattern", required=True)
    p.add_argument("--tokenizer-vocab", required=True)
    p.add_argument("--vocab-size", type=int, default=0)
    a = ap.parse_args(argv)

    if a.cmd == "sidecar":
        vocab = a.vocab_size
        if vocab <= 0:
            from .data.text_shards import load_sentencepiece
            vocab = int(load_sentencepiece(a.tokenizer_vocab).vocab_size)
        for name in ensure_byte_sidecars(a.val_pattern, a.tokenizer_vocab, vocab):
            print(f"sidecar={name}")
        return 0
    if a.cmd in ("status", "wait"):
        deadline = time.time() + a.timeout
        while True:
            try:
                with open(a.result_json, encoding="utf-8") as f:
                    r = json.load(f)
            except FileNotFoundError:
                r = {"status": "missing"}
            if a.cmd == "status" or r.get("status") in ("ok", "failed") or (a.timeout > 0 and time.time() >= deadline):
                break
            time.sleep(0.5)
        print(f"status={r.get('status')}\nreturncode={r.get('returncode')}")
        for k, v in sorted((r.get("metrics") or {}).items()):
            if not isinstance(v, (dict, list)):
                print(f"{k}={v}")
        return 0 if r.get("status") == "ok" else (3 if r.get("status") == "running" else 1)

    cmd = build_command(a.cmd, a.gpus, rest)
    if a.print_command:
        print(" ".join(cmd))
        return 0
    log_path = a.log or (os.path.splitext(a.result_json)[0] + ".log" if a.result_json else None)
    if a.detach and not a.supervise:
        if not a.result_json:
            raise SystemExit("--detach needs --result-json (the only way to learn the outcome)")
        again = [sys.executable, "-m", "parameter_golf_b200.launch", a.cmd, "--gpus", str(a.gpus), "--label", a.label, "--result-json", a.result_json,
                 "--log", log_path, "--supervise", "--"] + rest
        sup = subprocess.Popen(again, stdin=subprocess.DEVNULL, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, start_new_session=True,
                               env=dict(os.environ, PYTHONPATH=os.pathsep.join(filter(None, [os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                                                          os.environ.get("PYTHONPATH")]))))
        print(f"detached=true\nsupervisor_pid={sup.pid}\nresult_json={a.result_json}\nlog={log_path}")
        return 0
    return supervise(cmd, a.label, a.result_json, log_path, echo=not a.supervise)


if __name__ == "__main__":
    sys.exit(main())
