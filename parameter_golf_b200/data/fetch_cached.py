"""Manifest-driven materialisation of a tokenised dataset variant: the whole validation split, the first N training shards and
the tokenizer files of one variant (``sp1024``, ``sp8192``, ``byte260`` ...) are placed under a data directory.

Role of the reference's ``data/cached_challenge_fineweb.py`` (variant -> ``fineweb10B_<variant>``, shard counts read from
``manifest.json``, ``--train-shards``, ``--with-docs``, existing files kept, hard link before copy). That script fetches from a
hosted dataset repository; this one reads a *mirror* that is already reachable as a directory (``--source``: a root written by
`parameter_golf_b200.data.text_shards` ``--tokenizer-config``, or a copy of the hosted layout), because the machines this
framework is developed on have no network. With ``--repo-id`` and the ``huggingface_hub`` package installed the same manifest
logic pulls from the hosted repository instead (not exercised by the tests).

    python -m parameter_golf_b200.data.fetch_cached --source /mirror/root --dest data --variant sp1024 --train-shards 8
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
from typing import Callable, List, Optional

from .shards import read_shard_header


def dataset_dir_for_variant(name: str) -> str:
    if name == "byte260" or (name.startswith("sp") and name[2:].isdigit()):
        return f"fineweb10B_{name}"
    raise ValueError(f"unsupported variant {name!r}; expected byte260 or sp<VOCAB_SIZE>")


def _place(src: str, dst: str) -> bool:
    """Hard-link (else copy) ``src`` to ``dst`` unless it is there already; True when a file was written."""
    if os.path.exists(dst):
        return False
    if os.path.islink(dst):
        os.unlink(dst)                       # a dangling link from an earlier, interrupted run
    os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
    real = os.path.realpath(src)
    if not os.path.isfile(real):
        raise FileNotFoundError(f"the mirror lacks {src}")
    try:
        os.link(real, dst)
    except OSError:
        shutil.copy2(real, dst)
    return True


def local_getter(source: str) -> Callable[[str], str]:
    return lambda rel: os.path.join(source, rel)


def hub_getter(repo_id: str, prefix: str) -> Callable[[str], str]:
    from huggingface_hub import hf_hub_download           # optional dependency, needs network access

    def get(rel: str) -> str:
        rel = f"{prefix}/{rel}" if prefix else rel
        head, name = os.path.split(rel)
        return hf_hub_download(repo_id=repo_id, filename=name, subfolder=head or None, repo_type="dataset")
    return get


def fetch_variant(get: Callable[[str], str], dest: str, variant: str, train_shards: int = 80, with_docs: bool = False) -> dict:
    """Returns ``{"dataset_dir", "train", "val", "tokenizer", "written"}`` (paths under ``dest``)."""
    if train_shards < 0:
        raise ValueError("train_shards must be non-negative")
    name = dataset_dir_for_variant(variant)
    man_dst = os.path.join(dest, "manifest.json")
    _place(get("manifest.json"), man_dst)
    with open(man_dst, encoding="utf-8") as fh:
        manifest = json.load(fh)
    entry = next((d for d in manifest.get("datasets", []) if d.get("name") == name), None)
    if entry is None:
        raise ValueError(f"dataset {name} is not in the manifest (it lists {[d.get('name') for d in manifest.get('datasets', [])]})")
    stats = entry.get("stats") or {}
    have_train, have_val = int(stats.get("files_train", 0)), int(stats.get("files_val", 0))
    if train_shards > have_train:
        raise ValueError(f"{variant} has {have_train} training shards, {train_shards} were asked for")
    tok = next((t for t in manifest.get("tokenizers", []) if t.get("name") == entry.get("tokenizer_name")), None)
    if tok is None:
        raise ValueError(f"tokenizer {entry.get('tokenizer_name')} is not in the manifest")
    written: List[str] = []

    def take(rel: str) -> str:
        dst = os.path.join(dest, rel)
        if _place(get(rel), dst):
            written.append(rel)
        return dst
    out = {"dataset_dir": os.path.join(dest, "datasets", name), "train": [], "val": [], "tokenizer": [], "written": written}
    for i in range(have_val):
        out["val"].append(take(f"datasets/{name}/fineweb_val_{i:06d}.bin"))
        try:                                  # the byte-count sidecar travels with its validation shard when the mirror has one
            take(f"datasets/{name}/fineweb_val_bytes_{i:06d}.bin")
        except (FileNotFoundError, OSError):
            pass
    for i in range(train_shards):
        out["train"].append(take(f"datasets/{name}/fineweb_train_{i:06d}.bin"))
    for key in ("model_path", "vocab_path", "path"):
        if tok.get(key):
            out["tokenizer"].append(take(str(tok[key])))
    if with_docs:
        for rel in ("docs_selected.jsonl", "docs_selected.source_manifest.json"):
            take(rel)
    for path in out["train"] + out["val"]:
        read_shard_header(path)               # magic, version and size of every shard that was placed
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.data.fetch_cached")
    ap.add_argument("train_shards_positional", nargs="?", type=int, default=None, help=argparse.SUPPRESS)
    ap.add_argument("--train-shards", type=int, default=80)
    ap.add_argument("--variant", default="sp1024")
    ap.add_argument("--with-docs", action="store_true")
    ap.add_argument("--dest", default="data")
    ap.add_argument("--source", default=None, help="a directory holding manifest.json, datasets/ and tokenizers/")
    ap.add_argument("--repo-id", default=os.environ.get("MATCHED_FINEWEB_REPO_ID"), help="hosted dataset repository (needs huggingface_hub and a network)")
    ap.add_argument("--remote-prefix", default=os.environ.get("MATCHED_FINEWEB_REMOTE_ROOT_PREFIX", "datasets"))
    a = ap.parse_args(argv)
    if not a.source and not a.repo_id:
        ap.error("give --source (a local mirror) or --repo-id (a hosted dataset repository)")
    get = local_getter(a.source) if a.source else hub_getter(a.repo_id, a.remote_prefix)
    n = a.train_shards_positional if a.train_shards_positional is not None else a.train_shards
    out = fetch_variant(get, a.dest, a.variant, n, a.with_docs)
    print(json.dumps({"dataset_dir": out["dataset_dir"], "train_shards": len(out["train"]), "val_shards": len(out["val"]),
                      "tokenizer_files": len(out["tokenizer"]), "files_written": len(out["written"])}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
