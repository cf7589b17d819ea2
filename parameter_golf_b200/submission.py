"""Byte-budget manifest of a submission: the compressed model artifact plus every counted source file must stay below the
limit (decimal bytes, strict), and the manifest pins both by hash.

Counterpart of the reference's ``parameter-golf-rs/deploy/build_submission.py``; this one also opens the artifact, so the
manifest carries the container kind, the tensor count and the variant fingerprint stamped at export time, and it breaks the
counted code down by file type.

    python -m parameter_golf_b200.submission --artifact artifact.pgrs --code parameter_golf_b200 bench.py --out submission.json

Fails closed: a missing path, an unreadable artifact or a total at or above the limit all end with a non-zero exit code.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from typing import Dict, List

from .quant import container as C
from .quant.export import check_budget

LIMIT_BYTES = 16_000_000
SKIP_DIRS = {"__pycache__", "build", ".git"}
SKIP_SUFFIXES = (".so", ".o", ".pyc", ".hash", ".log")


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def counted_files(paths: List[str]) -> List[str]:
    """Every regular file under the given paths, sorted, without build products (shared objects, caches): what is counted is
    source. A path that does not exist is an error, never silently zero bytes."""
    out: List[str] = []
    for p in paths:
        if not os.path.exists(p):
            raise FileNotFoundError(f"counted code path does not exist: {p}")
        if os.path.isfile(p):
            out.append(p)
            continue
        for dp, dns, fns in os.walk(p):
            dns[:] = sorted(d for d in dns if d not in SKIP_DIRS)
            for fn in sorted(fns):
                if not fn.endswith(SKIP_SUFFIXES):
                    out.append(os.path.join(dp, fn))
    return out


def artifact_summary(path: str) -> Dict[str, object]:
    """Container kind, payload size, tensor count and the metadata stamped at export (fingerprint, scheme)."""
    blob = open(path, "rb").read()
    info: Dict[str, object] = {"bytes": len(blob), "sha256": hashlib.sha256(blob).hexdigest(), "container": blob[:4].decode("latin1")}
    try:
        raw = C.decompress_payload(blob)
        recs, meta = C.read_pgrs(raw)
        md = json.loads(meta) if meta else {}
        info.update(payload_bytes=len(raw), tensors=len(recs), variant_fingerprint=md.get("variant_fingerprint"), format=md.get("format"),
                    scheme=md.get("scheme"))
    except Exception as e:                       # other artifact families (the baseline's int8 + zlib) are counted but not opened
        info["unparsed"] = str(e)[:200]
    return info


def build_manifest(artifact: str, code: List[str], limit: int = LIMIT_BYTES) -> Dict[str, object]:
    files = counted_files(code)
    by_ext: Dict[str, int] = {}
    hashes = hashlib.sha256()
    total_code = 0
    for f in files:
        n = os.path.getsize(f)
        total_code += n
        ext = os.path.splitext(f)[1] or "(none)"
        by_ext[ext] = by_ext.get(ext, 0) + n
        hashes.update(sha256_file(f).encode("ascii"))
    art = artifact_summary(artifact)
    total = int(art["bytes"]) + total_code
    return {"event": "submission_byte_budget", "limit": limit, "model_artifact": artifact, "artifact": art, "code_paths": list(code),
            "code_file_count": len(files), "code_bytes": total_code, "code_bytes_by_type": dict(sorted(by_ext.items())),
            "code_sha256": hashes.hexdigest(), "total_bytes": total, "under_budget": check_budget(int(art["bytes"]), total_code, limit)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.submission")
    ap.add_argument("--artifact", "--model-artifact", dest="artifact", required=True)
    ap.add_argument("--code", nargs="+", required=True)
    ap.add_argument("--out")
    ap.add_argument("--limit", type=int, default=LIMIT_BYTES)
    a = ap.parse_args(argv)
    if not os.path.isfile(a.artifact):
        print(f"model artifact does not exist: {a.artifact}", file=sys.stderr)
        return 2
    try:
        man = build_manifest(a.artifact, a.code, a.limit)
    except FileNotFoundError as e:
        print(str(e), file=sys.stderr)
        return 2
    text = json.dumps(man, indent=2, sort_keys=True) + "\n"
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            f.write(text)
    print(json.dumps(man, sort_keys=True))
    if not man["under_budget"]:
        print(f"submission exceeds byte budget: {man['total_bytes']} >= {a.limit}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
