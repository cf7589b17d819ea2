"""Environment check: what the framework will find on this machine, read-only.

    python -m parameter_golf_b200.doctor [--require-gpu] [--json]

Prints ``key=value`` lines (or one JSON object): interpreter and torch versions, the CUDA toolkit torch was built with, ``nvcc``
if on the path, the in-tree extension (present, loadable), NCCL, and per GPU its name, compute capability, memory and which
peers it can address directly. It changes nothing on the device: no clocks, modes or limits are touched, only queried through
torch. Counterpart of the image checks the reference keeps beside its deploy scripts (parameter-golf-rs/deploy/check_cudnn.py,
Dockerfile:11-32: pinned CUDA / NCCL / cuDNN versions); exit code 1 when ``--require-gpu`` is given and no sm_100 device, or
not the built extension, is there.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import subprocess
import sys


def collect() -> dict:
    import torch
    info = {"python": sys.version.split()[0], "torch": torch.__version__, "torch_cuda": torch.version.cuda, "cuda_available": torch.cuda.is_available()}
    nvcc = shutil.which("nvcc")
    if nvcc:
        try:
            out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
            info["nvcc"] = next((l.split("release")[-1].strip() for l in out.splitlines() if "release" in l), "unknown")
        except Exception as exc:           # noqa: BLE001 - reported, not fatal
            info["nvcc"] = f"error: {exc}"
    else:
        info["nvcc"] = None
    here = os.path.dirname(os.path.abspath(__file__))
    built = sorted(glob.glob(os.path.join(here, "_C*.so")))
    info["extension_files"] = [os.path.basename(b) for b in built]
    try:
        info["nccl"] = ".".join(str(x) for x in torch.cuda.nccl.version()) if hasattr(torch.cuda, "nccl") else None
    except Exception:                      # noqa: BLE001
        info["nccl"] = None
    import torch.distributed as dist
    info["dist_backends"] = [b for b in ("nccl", "gloo") if getattr(dist, f"is_{b}_available")()]
    gpus = []
    if info["cuda_available"]:
        n = torch.cuda.device_count()
        for i in range(n):
            pr = torch.cuda.get_device_properties(i)
            gpus.append({"index": i, "name": pr.name, "capability": f"{pr.major}.{pr.minor}", "memory_gib": round(pr.total_memory / 2 ** 30, 1),
                         "sms": pr.multi_processor_count,
                         "peers": [j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j)]})
        if built:
            try:
                from .ops import native
                native.load()
                info["extension_loaded"] = True
            except Exception as exc:       # noqa: BLE001
                info["extension_loaded"] = f"error: {exc}"
    info["gpus"] = gpus
    info["sm100_gpus"] = sum(1 for g in gpus if g["capability"].startswith("10."))
    return info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.doctor")
    ap.add_argument("--require-gpu", action="store_true")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    info = collect()
    if a.json:
        print(json.dumps(info, sort_keys=True))
    else:
        for k, v in info.items():
            if k == "gpus":
                for g in v:
                    print(f"gpu{g['index']}={g['name']} sm_{g['capability'].replace('.', '')} {g['memory_gib']}GiB {g['sms']}SMs peers={g['peers']}")
            else:
                print(f"{k}={v}")
    ok = info["sm100_gpus"] > 0 and bool(info["extension_files"]) and info.get("extension_loaded") is True
    if a.require_gpu and not ok:
        print("doctor: no sm_100 GPU with a loadable in-tree extension", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
