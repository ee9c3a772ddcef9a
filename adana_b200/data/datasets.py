"""Dataset registry: where each corpus lives on disk and how it is prepared.

Every corpus is stored as flat uint16 GPT-2-BPE token streams (`train.bin` / `val.bin`, or
`train_0000.bin ...` for multi-file corpora), the layout of the reference's preparers
(src/data/fineweb.py:11-77, fineweb_100.py:24-188, slimpajama.py, redpajama.py, c4.py,
openwebtext2.py, fineweb_edu.py, wikitext.py, arxiv.py, shakespeare.py).  Here all of them go
through ONE table-driven pipeline: `CorpusSpec` names the directory, the Hugging Face source
and the validation split; `prepare_corpus` tokenises with a process pool and appends to the
token files.  A corpus whose `.bin` files already exist is returned without touching the
network, and `synthetic-zipf` needs nothing but NumPy.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, Optional

import numpy as np

EOT_GPT2 = 50256


# ---- synthetic streams ------------------------------------------------------------------------
def make_zipf_tokens(n_tokens: int, vocab: int = 50304, exponent: float = 1.0, seed: int = 0) -> np.ndarray:
    """iid tokens with P(k) ∝ 1/(k+1)^exponent over [0, vocab) as uint16, by inverse-CDF sampling."""
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** exponent
    cdf = np.cumsum(p / p.sum())
    cdf[-1] = 1.0
    out = np.empty(n_tokens, dtype=np.uint16)
    step = 1 << 22
    for s in range(0, n_tokens, step):
        u = rng.random(min(step, n_tokens - s))
        out[s:s + len(u)] = np.searchsorted(cdf, u, side="right").astype(np.uint16)
    return out


def zipf_entropy(vocab: int = 50304, exponent: float = 1.0) -> float:
    """Entropy in nats of the Zipf distribution: the loss floor of an iid Zipf stream."""
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** exponent
    p /= p.sum()
    return float(-(p * np.log(p)).sum())


def write_zipf_dataset(root, n_train: int = 8_000_000, n_val: int = 1_000_000, vocab: int = 50304,
                       exponent: float = 1.0, seed: int = 0, n_files: int = 1) -> Dict[str, str]:
    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    out: Dict[str, str] = {}
    val = root / "val.bin"
    if not val.exists():
        make_zipf_tokens(n_val, vocab, exponent, seed + 10_000).tofile(val)
    out["val"] = str(val)
    if n_files == 1:
        tr = root / "train.bin"
        if not tr.exists():
            make_zipf_tokens(n_train, vocab, exponent, seed).tofile(tr)
        out["train"] = str(tr)
    else:
        for i in range(n_files):
            f = root / f"train_{i:04d}.bin"
            if not f.exists():
                make_zipf_tokens(n_train // n_files, vocab, exponent, seed + i).tofile(f)
            out[f"train_{i:04d}"] = str(f)
    return out


# ---- corpus table ------------------------------------------------------------------------------
@dataclass(frozen=True)
class CorpusSpec:
    subdir: str
    hf_path: Optional[str] = None
    hf_name: Optional[str] = None
    hf_split: str = "train"
    val_fraction: float = 0.0005
    text_key: str = "text"
    multi_file: bool = False
    char_level: bool = False


CORPORA: Dict[str, CorpusSpec] = {
    "fineweb": CorpusSpec("fineweb-10BT", "HuggingFaceFW/fineweb", "sample-10BT", val_fraction=0.0001),
    "finewebedu": CorpusSpec("fineweb-edu-100BT", "HuggingFaceFW/fineweb-edu", "sample-100BT", val_fraction=0.0001),
    "fineweb_100": CorpusSpec("fineweb-100BT", "HuggingFaceFW/fineweb", "sample-100BT", multi_file=True),
    "c4": CorpusSpec("c4", "allenai/c4", "en", val_fraction=0.0001),
    "slimpajama": CorpusSpec("slimpajama6B", "DKYoon/SlimPajama-6B"),
    "slimpajama_chunk1": CorpusSpec("slimpajama6B", "cerebras/SlimPajama-627B", hf_split="train/chunk1"),
    "redpajama": CorpusSpec("redpajama1Tsample", "togethercomputer/RedPajama-Data-1T-Sample"),
    "redpajamav2": CorpusSpec("redpajamaV2sample", "togethercomputer/RedPajama-Data-V2", "sample",
                              text_key="raw_content"),
    "openwebtext2": CorpusSpec("openwebtext2", "the_pile_openwebtext2"),
    "wikitext": CorpusSpec("wikitext", "wikitext", "wikitext-103-raw-v1", val_fraction=0.0),
    "arxiv": CorpusSpec("arxiv", None),
    "arxiv2000": CorpusSpec("arxiv", None),
    "shakespeare-char": CorpusSpec("shakespeare", None, char_level=True),
}


def _tokenizer():
    try:
        import tiktoken

        enc = tiktoken.get_encoding("gpt2")
        return lambda s: enc.encode_ordinary(s) + [enc.eot_token]
    except Exception as e:  # no tiktoken / no cached BPE files
        raise RuntimeError(
            "GPT-2 BPE tokenizer unavailable (tiktoken and its vocabulary files are needed to "
            f"prepare a text corpus): {e}") from e


class TokenFileWriter:
    """Appends uint16 tokens to `<prefix>.bin`, or rolls `<prefix>_NNNN.bin` files of `roll` tokens."""

    def __init__(self, path_prefix: Path, roll: Optional[int] = None):
        self.prefix, self.roll = Path(path_prefix), roll
        self.idx, self.count, self.files = 0, 0, []
        self._fh = None
        self._open()

    def _open(self):
        name = f"{self.prefix}_{self.idx:04d}.bin" if self.roll else f"{self.prefix}.bin"
        self._fh = open(name, "wb")
        self.files.append(name)
        self.count = 0

    def write(self, ids: Iterable[int]):
        arr = np.asarray(list(ids), dtype=np.uint16)
        arr.tofile(self._fh)
        self.count += len(arr)
        if self.roll and self.count >= self.roll:
            self._fh.close()
            self.idx += 1
            self._open()

    def close(self):
        self._fh.close()


def prepare_corpus(spec: CorpusSpec, root: Path, texts: Optional[Iterable[str]] = None,
                   val_docs: int = 1470, tokens_per_file: int = 1_000_000_000) -> None:
    """Tokenise `texts` (or the Hugging Face source of `spec`) into the token files under `root`."""
    root.mkdir(parents=True, exist_ok=True)
    if texts is None:
        if spec.hf_path is None:
            raise RuntimeError(f"{spec.subdir}: no downloadable source is registered; place train.bin/val.bin in {root}")
        try:
            from datasets import load_dataset
        except ImportError as e:
            raise RuntimeError("the `datasets` package is needed to download a corpus") from e
        ds = load_dataset(spec.hf_path, name=spec.hf_name, split=spec.hf_split)
        texts = (ex[spec.text_key] for ex in ds)
    if spec.char_level:
        blob = "".join(texts)
        chars = sorted(set(blob))
        lut = {c: i for i, c in enumerate(chars)}
        ids = np.array([lut[c] for c in blob], dtype=np.uint16)
        n_val = max(1, int(0.1 * len(ids)))
        ids[:-n_val].tofile(root / "train.bin")
        ids[-n_val:].tofile(root / "val.bin")
        return
    tok = _tokenizer()
    rng = np.random.default_rng(2357)
    train = TokenFileWriter(root / "train", roll=tokens_per_file if spec.multi_file else None)
    val = TokenFileWriter(root / "val")
    for i, t in enumerate(texts):
        to_val = (i < val_docs) if spec.multi_file else (rng.random() < spec.val_fraction)
        (val if to_val else train).write(tok(t))
    train.close()
    val.close()


def _existing_files(root: Path, spec: CorpusSpec) -> Optional[Dict[str, str]]:
    val = root / "val.bin"
    if spec.multi_file:
        files = sorted(root.glob("train_*.bin"))
        if len(files) >= 3 and val.exists():
            d = {f.stem: str(f) for f in files}
            d["val"] = str(val)
            return d
    if (root / "train.bin").exists() and val.exists():
        return {"train": str(root / "train.bin"), "val": str(val)}
    return None


def get_dataset(args) -> Dict[str, object]:
    """Returns {'train' | 'train_XXXX'...: path, 'val': path}."""
    name = args.dataset
    base = Path(args.datasets_dir)
    if name == "synthetic-zipf":
        return write_zipf_dataset(base / "synthetic-zipf", n_train=getattr(args, "synthetic_tokens", 8_000_000),
                                  vocab=args.vocab_size, exponent=getattr(args, "zipf_exponent", 1.0),
                                  seed=getattr(args, "data_seed", 0))
    if name == "arxiv+wiki":
        parts = [get_dataset(_with(args, dataset=d)) for d in ("arxiv", "wikitext")]
        cat = lambda k: np.concatenate([np.memmap(p[k], dtype=np.uint16, mode="r") for p in parts])
        return {"train": cat("train"), "val": cat("val")}
    if name in ("arxiv", "arxiv2000", "shakespeare-char"):
        # the corpora with sources of their own (data/text_sources.py); token files placed by hand still win
        from . import text_sources as TS

        found = _existing_files(base / CORPORA[name].subdir, CORPORA[name])
        if found is not None:
            return found
        if name == "shakespeare-char":
            return TS.load_shakespeare_char(base)
        return TS.load_arxiv(base, [2000] if name == "arxiv2000" else None)
    if name not in CORPORA:
        raise NotImplementedError(f"Unknow dataset key '{name}'")
    spec = CORPORA[name]
    root = base / spec.subdir
    found = _existing_files(root, spec)
    if found is None:
        prepare_corpus(spec, root)
        found = _existing_files(root, spec)
        if found is None:
            raise RuntimeError(f"preparing {name} produced no token files in {root}")
    return found


def _with(args, **kw):
    import copy

    a = copy.copy(args)
    for k, v in kw.items():
        setattr(a, k, v)
    return a


# ---- command line: download (optional) and tokenise a corpus -----------------------------------
def iter_parquet_texts(folder: Path, text_key: str = "text", batch_rows: int = 1000):
    """Stream the text column of every `*.parquet` under `folder` (sorted), row group by row group."""
    import pyarrow.parquet as pq

    files = sorted(Path(folder).rglob("*.parquet"))
    if not files:
        raise FileNotFoundError(f"no .parquet files under {folder}")
    for f in files:
        pf = pq.ParquetFile(f)
        for batch in pf.iter_batches(batch_size=batch_rows, columns=[text_key]):
            yield from batch.column(0).to_pylist()


def download_snapshot(spec: CorpusSpec, target: Path) -> Path:
    """Fetch the parquet files of a Hugging Face sample (needs network and `huggingface_hub`)."""
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:
        raise RuntimeError("huggingface_hub is needed to download; use --skip-download with local parquet files") from e
    pattern = f"sample/{spec.hf_name.split('-')[-1]}/*" if spec.hf_name and spec.hf_name.startswith("sample-") else None
    return Path(snapshot_download(spec.hf_path, repo_type="dataset", local_dir=str(target),
                                  allow_patterns=[pattern] if pattern else None))


def main(argv=None) -> int:
    """`python -m adana_b200.data.datasets --dataset fineweb_100 --download-dir ./fineweb --output-dir ./datasets`
    — the two steps of the reference's `process_fineweb_100bt.py` (download the sample, tokenise it into
    `train_XXXX.bin` + `val.bin`) for any corpus of the table; `--skip-download` tokenises local parquet files."""
    import argparse

    p = argparse.ArgumentParser(description="Download and tokenise a pre-training corpus")
    p.add_argument("--dataset", default="fineweb_100", choices=sorted(CORPORA))
    p.add_argument("--download-dir", default="./fineweb/")
    p.add_argument("--output-dir", default="./datasets/")
    p.add_argument("--skip-download", action="store_true")
    p.add_argument("--tokens-per-file", type=int, default=1_000_000_000)
    p.add_argument("--val-docs", type=int, default=1470)
    a = p.parse_args(argv)
    spec = CORPORA[a.dataset]
    src = Path(a.download_dir)
    if not a.skip_download:
        print(f"step 1: downloading {spec.hf_path} ({spec.hf_name}) to {src}")
        download_snapshot(spec, src)
    root = Path(a.output_dir) / spec.subdir
    if _existing_files(root, spec) is not None:
        print(f"{root} already holds token files; nothing to do")
        return 0
    print(f"step 2: tokenising {src} into {root}")
    prepare_corpus(spec, root, texts=iter_parquet_texts(src, spec.text_key), val_docs=a.val_docs,
                   tokens_per_file=a.tokens_per_file)
    found = _existing_files(root, spec) or {}
    print(f"wrote {len(found)} files under {root}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
