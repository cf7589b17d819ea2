"""From local text to token shards: tokenizer training and shard export without a network.

The reference's data tooling downloads a document dump and tokenises it
(``data/download_hf_docs_and_tokenize.py``: SentencePiece BPE training ``:248-296``, streaming shard export with a BOS
token in front of every document and the first ``num_val_docs`` documents as the validation split ``:309-396``, pure-byte
tokenizer ``:36-70``). This module is the part of that which works on files that are already on disk:

* documents come from a ``.jsonl`` file (one object per line with a ``text`` field), a ``.txt`` file (one document per
  blank-line-separated block) or a directory of such files;
* `train_sentencepiece` trains a BPE model with the reference's trainer settings (byte fallback, split digits, NFKC, no
  dummy prefix, pad/bos/eos/unk = 0/1/2/3); `ByteTokenizer` is the 260-entry pure-byte vocabulary;
* `export_shards` streams ``[BOS] + tokens`` per document into ``fineweb_val_*.bin`` / ``fineweb_train_*.bin`` shards of
  the uint16 format `shards.write_shard` writes, refuses ids outside the declared vocabulary, and writes next to every
  validation shard a byte-count sidecar (``fineweb_val_bytes_*.bin``) holding the UTF-8 bytes each position stands for, so
  bits-per-byte can be computed from the stream itself.

    python -m parameter_golf_b200.data.text_shards --docs corpus.jsonl --out data/sp1024 --vocab 1024 --val-docs 500
    python -m parameter_golf_b200.data.text_shards --docs texts/ --out data/bytes --tokenizer bytes

A run then points at the result with ``train.train_data_pattern=data/sp1024/fineweb_train_*.bin``,
``train.validation_data_pattern=data/sp1024/fineweb_val_*.bin`` (byte sidecars matched by the pattern are skipped),
``model.vocab_size=1024`` and either ``eval.tokenizer_vocab_path=data/sp1024/tokenizers/fineweb_1024_bpe.model`` or
``eval.caseops_byte_sidecar_pattern=data/sp1024/fineweb_val_bytes_*.bin`` for the bits-per-byte denominator.
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np

from .bpb import BpbLuts
from .shards import write_shard

SP_TRAINER_DEFAULTS = dict(model_type="bpe", character_coverage=0.999, byte_fallback=True, split_digits=True,
                           normalization_rule_name="nmt_nfkc", add_dummy_prefix=False, pad_id=0, bos_id=1, eos_id=2, unk_id=3,
                           hard_vocab_limit=False)


# ---- documents ------------------------------------------------------------------------------------------------------

def iter_documents(path: str) -> Iterator[str]:
    """Documents of a ``.jsonl`` file (``text`` field), a text file (blank-line separated blocks) or, recursively in sorted
    order, of every such file in a directory. Empty documents are dropped."""
    if os.path.isdir(path):
        for f in sorted(glob.glob(os.path.join(path, "**", "*"), recursive=True)):
            if os.path.isfile(f) and f.endswith((".jsonl", ".txt", ".md")):
                yield from iter_documents(f)
        return
    if path.endswith(".jsonl"):
        with open(path, "r", encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if not line:
                    continue
                text = json.loads(line).get("text", "")
                if text:
                    yield text
        return
    with open(path, "r", encoding="utf-8") as fh:
        block: List[str] = []
        for line in fh:
            if line.strip():
                block.append(line.rstrip("\n"))
            elif block:
                yield "\n".join(block)
                block = []
        if block:
            yield "\n".join(block)


# ---- tokenizers -----------------------------------------------------------------------------------------------------

@dataclass
class Tokenizer:
    """What the exporter needs from a tokenizer: ids per document, the vocabulary size, the BOS id and the byte tables."""
    name: str
    vocab_size: int
    bos_id: int
    eos_id: int
    encode_batch: Callable[[Sequence[str]], List[np.ndarray]]
    decode: Callable[[Sequence[int]], str]
    luts: BpbLuts
    model_path: Optional[str] = None


class ByteTokenizer:
    """ids 0..3 = pad, bos, eos, unk; id 4 + b = byte b (``download_hf_docs_and_tokenize.py:36-70``)."""
    pad_id, bos_id, eos_id, unk_id, byte_offset = 0, 1, 2, 3, 4
    vocab_size = 260

    def encode(self, text: str) -> np.ndarray:
        return np.frombuffer(text.encode("utf-8", errors="replace"), dtype=np.uint8).astype(np.int32) + self.byte_offset

    def decode(self, ids: Sequence[int]) -> str:
        b = bytes(int(i) - self.byte_offset for i in ids if int(i) >= self.byte_offset)
        return b.decode("utf-8", errors="replace")

    def luts(self) -> BpbLuts:
        base = np.zeros(self.vocab_size, np.int16)
        base[self.byte_offset:] = 1
        bound = np.zeros(self.vocab_size, bool)
        bound[: self.byte_offset] = True
        return BpbLuts(base, np.zeros(self.vocab_size, bool), bound)

    def as_tokenizer(self) -> Tokenizer:
        return Tokenizer("pure_byte", self.vocab_size, self.bos_id, self.eos_id, lambda texts: [self.encode(t) for t in texts], self.decode,
                         self.luts())


def train_sentencepiece(docs: Iterable[str], vocab_size: int, model_prefix: str, max_docs: Optional[int] = None, **overrides) -> str:
    """Train a SentencePiece BPE model on ``docs`` with the reference's settings; returns the ``.model`` path."""
    import sentencepiece as spm

    def sentences():
        for i, d in enumerate(docs):
            if max_docs is not None and i >= max_docs:
                return
            # the trainer reads "sentences": long documents are cut at line breaks so that none exceeds its length limit
            for line in d.split("\n"):
                if line.strip():
                    yield line

    os.makedirs(os.path.dirname(os.path.abspath(model_prefix)), exist_ok=True)
    kwargs = dict(SP_TRAINER_DEFAULTS, sentence_iterator=sentences(), model_prefix=model_prefix, vocab_size=int(vocab_size))
    kwargs.update(overrides)
    spm.SentencePieceTrainer.train(**kwargs)
    return model_prefix + ".model"


def load_sentencepiece(model_path: str) -> Tokenizer:
    import sentencepiece as spm
    sp = spm.SentencePieceProcessor(model_file=model_path)
    v = int(sp.vocab_size())
    return Tokenizer(f"sp_bpe_{v}", v, int(sp.bos_id()), int(sp.eos_id()),
                     lambda texts: [np.asarray(ids, dtype=np.int32) for ids in sp.encode(list(texts), out_type=int)],
                     lambda ids: sp.decode([int(i) for i in ids]), BpbLuts.from_sentencepiece(model_path, v), model_path)


# ---- export ---------------------------------------------------------------------------------------------------------

class _ShardWriter:
    """Fills fixed-size shards of one split; the validation split also gets its byte-count sidecar shards."""

    def __init__(self, out_dir: str, split: str, shard_tokens: int, with_bytes: bool):
        self.out_dir, self.split, self.cap, self.with_bytes = out_dir, split, shard_tokens, with_bytes
        self.buf = np.empty(shard_tokens, dtype=np.uint16)
        self.bbuf = np.empty(shard_tokens, dtype=np.uint16) if with_bytes else None
        self.fill = 0
        self.files = 0
        self.tokens = 0

    def add(self, toks: np.ndarray, nbytes: Optional[np.ndarray]):
        pos = 0
        while pos < len(toks):
            take = min(self.cap - self.fill, len(toks) - pos)
            self.buf[self.fill:self.fill + take] = toks[pos:pos + take]
            if self.with_bytes:
                self.bbuf[self.fill:self.fill + take] = nbytes[pos:pos + take]
            self.fill += take
            pos += take
            if self.fill == self.cap:
                self.flush()
        self.tokens += len(toks)

    def flush(self):
        if self.fill == 0:
            return
        write_shard(os.path.join(self.out_dir, f"fineweb_{self.split}_{self.files:06d}.bin"), self.buf[:self.fill])
        if self.with_bytes:
            write_shard(os.path.join(self.out_dir, f"fineweb_{self.split}_bytes_{self.files:06d}.bin"), self.bbuf[:self.fill])
        self.files += 1
        self.fill = 0


def position_bytes(tok: Tokenizer, ids: np.ndarray) -> np.ndarray:
    """UTF-8 bytes each position of ``[BOS] + document`` stands for, by the table rule of `BpbLuts.token_bytes` (a leading
    ``▁`` counts one byte unless the previous token is a boundary such as BOS)."""
    prev = np.concatenate([[ids[0]], ids[:-1]])
    b = tok.luts.token_bytes(prev, ids)
    b[0] = 0                                        # the BOS position itself
    return b.astype(np.uint16)


def export_shards(docs: Iterable[str], tok: Tokenizer, out_dir: str, num_val_docs: int = 1000, shard_tokens: int = 10 ** 8, append_eos: bool = False,
                  batch_docs: int = 256, byte_sidecar: bool = True) -> Dict[str, int]:
    """Write the validation split (the first ``num_val_docs`` documents) and the training split. Every document becomes
    ``[BOS] + ids (+ [EOS])``. Returns counts of documents, tokens, files and validation bytes per split."""
    if tok.vocab_size > 1 << 16:
        raise ValueError(f"vocab_size={tok.vocab_size} is too large for uint16 shard storage")
    os.makedirs(out_dir, exist_ok=True)
    for stale in glob.glob(os.path.join(out_dir, "fineweb_train_*.bin")) + glob.glob(os.path.join(out_dir, "fineweb_val_*.bin")):
        os.remove(stale)
    writers = {"val": _ShardWriter(out_dir, "val", shard_tokens, byte_sidecar), "train": _ShardWriter(out_dir, "train", shard_tokens, False)}
    stats = {"docs_val": 0, "docs_train": 0, "bytes_val": 0}
    batch: List[str] = []

    def drain():
        for ids in tok.encode_batch(batch):
            ids = np.asarray(ids, dtype=np.int64)
            toks = np.empty(ids.size + 1 + int(append_eos), dtype=np.int64)
            toks[0] = tok.bos_id
            toks[1:1 + ids.size] = ids
            if append_eos:
                toks[-1] = tok.eos_id
            if toks.size and (toks.min() < 0 or toks.max() >= tok.vocab_size):
                bad = int(toks[(toks < 0) | (toks >= tok.vocab_size)][0])
                raise ValueError(f"token id {bad} outside declared vocab_size={tok.vocab_size}")
            split = "val" if stats["docs_val"] < num_val_docs else "train"
            nbytes = None
            if split == "val" and byte_sidecar:
                nbytes = position_bytes(tok, toks)
                stats["bytes_val"] += int(nbytes.sum())
            writers[split].add(toks.astype("<u2"), nbytes)
            stats[f"docs_{split}"] += 1
        batch.clear()

    for d in docs:
        batch.append(d)
        if len(batch) >= batch_docs or stats["docs_val"] + len(batch) == num_val_docs:
            drain()
    if batch:
        drain()
    for split, w in writers.items():
        w.flush()
        stats[f"tokens_{split}"] = w.tokens
        stats[f"files_{split}"] = w.files
    manifest = {"tokenizer": tok.name, "vocab_size": tok.vocab_size, "bos_id": tok.bos_id, "eos_id": tok.eos_id, "append_eos": append_eos,
                "tokenizer_model": os.path.basename(tok.model_path) if tok.model_path else None, "shard_tokens": shard_tokens, **stats,
                "train_pattern": "fineweb_train_*.bin", "val_pattern": "fineweb_val_[0-9]*.bin", "val_bytes_pattern": "fineweb_val_bytes_*.bin"}
    with open(os.path.join(out_dir, "manifest.json"), "w") as fh:
        json.dump(manifest, fh, indent=1, sort_keys=True)
    return stats


def tokenizer_kind(spec: dict) -> str:
    """``byte`` or ``sentencepiece_bpe`` for an entry of a tokenizer config (the rules of data/download_hf_docs_and_tokenize.py:192-214:
    an explicit ``kind``, the ``byte260`` dataset suffix, else a ``vocab_size`` means SentencePiece BPE)."""
    kind = spec.get("kind")
    if kind in ("byte", "pure_byte") or str(spec.get("builder", "")).endswith("build_pure_byte_tokenizer") or spec.get("dataset_suffix") == "byte260":
        return "byte"
    if kind in ("sentencepiece_bpe", "sentencepiece") or str(spec.get("builder", "")).endswith("build_sentencepiece_tokenizer") or "vocab_size" in spec:
        return "sentencepiece_bpe"
    raise ValueError(f"unsupported tokenizer spec {spec.get('name', '<unnamed>')!r}: expected a pure-byte or SentencePiece BPE entry")


def export_from_config(docs_path: str, output_root: str, config_path: str, val_docs: int = 1000, shard_tokens: int = 10 ** 8,
                       tokenizer_train_docs: Optional[int] = None, append_eos: bool = False) -> dict:
    """One dataset per entry of a tokenizer config file (``{"tokenizers": [{"name", "dataset_suffix", "vocab_size"}, ...]}``, the
    format of the reference's data/tokenizer_specs.json), in its directory layout: ``<root>/tokenizers/`` for the models,
    ``<root>/datasets/fineweb10B_<suffix>/`` for the shards, ``<root>/manifest.json`` listing both
    (data/download_hf_docs_and_tokenize.py:578-622)."""
    with open(config_path, encoding="utf-8") as fh:
        payload = json.load(fh)
    specs = payload.get("tokenizer_specs", payload.get("tokenizers")) if isinstance(payload, dict) else payload
    if not isinstance(specs, list) or not specs or not all(isinstance(x, dict) for x in specs):
        raise ValueError("the tokenizer config must hold a non-empty list of objects")
    manifest = {"version": 1, "num_val_docs": val_docs, "shard_size": shard_tokens, "append_eos": append_eos, "docs": os.path.basename(docs_path),
                "tokenizer_specs": specs, "tokenizers": [], "datasets": []}
    for spec in specs:
        kind = tokenizer_kind(spec)
        suffix = spec.get("dataset_suffix") or ("byte260" if kind == "byte" else f"sp{int(spec['vocab_size'])}")
        name = spec.get("name") or ("pure_byte_260" if kind == "byte" else f"sp_bpe_{int(spec['vocab_size'])}")
        if kind == "byte":
            tok = ByteTokenizer().as_tokenizer()
            tok_manifest = {"name": name, "kind": kind, "vocab_size": tok.vocab_size}
        else:
            vocab = int(spec["vocab_size"])
            model = train_sentencepiece(iter_documents(docs_path), vocab, os.path.join(output_root, "tokenizers", f"fineweb_{vocab}_bpe"),
                                        max_docs=spec.get("tokenizer_train_docs", tokenizer_train_docs))
            tok = load_sentencepiece(model)
            tok_manifest = {"name": name, "kind": kind, "vocab_size": vocab, "model_path": os.path.relpath(model, output_root),
                            "vocab_path": os.path.relpath(os.path.splitext(model)[0] + ".vocab", output_root)}
        out_dir = os.path.join(output_root, "datasets", f"fineweb10B_{suffix}")
        stats = export_shards(iter_documents(docs_path), tok, out_dir, val_docs, shard_tokens, append_eos)
        rel = os.path.relpath(out_dir, output_root)
        manifest["tokenizers"].append(tok_manifest)
        manifest["datasets"].append({"name": f"fineweb10B_{suffix}", "tokenizer_name": name, "tokenizer_kind": kind, "path": rel,
                                     "train_glob": os.path.join(rel, "fineweb_train_*.bin"), "val_glob": os.path.join(rel, "fineweb_val_[0-9]*.bin"),
                                     "val_bytes_glob": os.path.join(rel, "fineweb_val_bytes_*.bin"), "vocab_size": tok.vocab_size, "bos_id": tok.bos_id,
                                     "eos_id": tok.eos_id, "stats": stats})
    os.makedirs(output_root, exist_ok=True)
    with open(os.path.join(output_root, "manifest.json"), "w", encoding="utf-8") as fh:
        json.dump(manifest, fh, indent=2)
        fh.write("\n")
    with open(os.path.join(output_root, "tokenizer_config.export.json"), "w", encoding="utf-8") as fh:
        json.dump({"tokenizers": specs}, fh, indent=2)
        fh.write("\n")
    return manifest


def _main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.data.text_shards")
    ap.add_argument("--docs", required=True, help=".jsonl (text field), .txt (blank-line separated) or a directory of them")
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", default="train", help="'train' (SentencePiece BPE on --docs), 'bytes', or a .model file to reuse")
    ap.add_argument("--vocab", type=int, default=1024)
    ap.add_argument("--tokenizer-train-docs", type=int, default=None)
    ap.add_argument("--val-docs", type=int, default=1000)
    ap.add_argument("--shard-tokens", type=int, default=10 ** 8)
    ap.add_argument("--append-eos", action="store_true")
    ap.add_argument("--tokenizer-config", default=None,
                    help="JSON list of tokenizers ({'tokenizers': [{'name', 'dataset_suffix', 'vocab_size'}]}): one dataset per entry under "
                         "<out>/datasets/fineweb10B_<suffix>/, models under <out>/tokenizers/, <out>/manifest.json")
    a = ap.parse_args(argv)
    if a.tokenizer_config:
        man = export_from_config(a.docs, a.out, a.tokenizer_config, a.val_docs, a.shard_tokens, a.tokenizer_train_docs, a.append_eos)
        print(json.dumps({"datasets": [d["name"] for d in man["datasets"]], "manifest": os.path.join(a.out, "manifest.json")}))
        return 0
    if a.tokenizer == "bytes":
        tok = ByteTokenizer().as_tokenizer()
    else:
        model = a.tokenizer
        if model == "train":
            model = train_sentencepiece(iter_documents(a.docs), a.vocab, os.path.join(a.out, "tokenizers", f"fineweb_{a.vocab}_bpe"),
                                        max_docs=a.tokenizer_train_docs)
        tok = load_sentencepiece(model)
    stats = export_shards(iter_documents(a.docs), tok, a.out, a.val_docs, a.shard_tokens, a.append_eos)
    print(json.dumps({"tokenizer": tok.name, "vocab_size": tok.vocab_size, **stats}))
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
