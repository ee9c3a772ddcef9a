"""Preparers of the two corpora that do not come from the Hugging Face hub.

arXiv hep-th (`--dataset arxiv`, `arxiv2000`): one tar archive of LaTeX sources per year 1993-2003 from the KDD-cup
mirror; every paper is converted to Markdown with `pandoc` (one second per paper, papers that take longer are
dropped), tokenised with the GPT-2 BPE and dealt by position (i mod 10: 0-6 train, 7-8 validation, 9 test) into
`<root>/<year>/{train,val,test}.npy`; a dataset is the concatenation of its years (reference src/data/arxiv.py:16-116).
Shakespeare at character level (`--dataset shakespeare-char`): the "tiny Shakespeare" text, vocabulary = its sorted
distinct characters, the first 90 % of the lines for training and the rest for validation (src/data/shakespeare.py:1-52).

Without network access the same steps run from local files: put `hep-th-<year>.tar.gz` (or an unpacked
`tex/<year>/` directory) under `<datasets_dir>/arxiv/`, or `raw.txt` under `<datasets_dir>/shakespeare/`.  Without
`pandoc` a plain LaTeX stripper (comments, commands and environments' markers removed, text kept) stands in, so
the pipeline still produces a corpus, and says so.
"""
from __future__ import annotations

import re
import shutil
import subprocess
import tarfile
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional

import numpy as np

ARXIV_YEARS = list(range(1993, 2004))          # 1992 is left out, as in the reference
ARXIV_URL = "https://www.cs.cornell.edu/projects/kddcup/download/hep-th-{year}.tar.gz"
SHAKESPEARE_URL = "https://raw.githubusercontent.com/karpathy/char-rnn/master/data/tinyshakespeare/input.txt"


def _download(url: str, dest: Path, timeout: float = 60.0) -> None:
    import urllib.request

    dest.parent.mkdir(parents=True, exist_ok=True)
    tmp = dest.with_name(dest.name + ".part")
    with urllib.request.urlopen(url, timeout=timeout) as r, open(tmp, "wb") as f:
        shutil.copyfileobj(r, f)
    tmp.replace(dest)


# ---- LaTeX -> text ---------------------------------------------------------------------------------------------------
_COMMENT = re.compile(r"(?<!\\)%.*")
_ENV = re.compile(r"\\(begin|end)\{[^}]*\}")
_CMD_ARG = re.compile(r"\\(?:cite|ref|label|eqref|bibitem|include|input|usepackage|documentclass)\*?(?:\[[^\]]*\])?\{[^}]*\}")
_CMD = re.compile(r"\\[a-zA-Z@]+\*?(?:\[[^\]]*\])?")


def strip_latex(src: str) -> str:
    """A rough LaTeX-to-text pass for machines without pandoc: comments, referencing commands with their arguments,
    environment markers and command names go; braces are dropped and the text they hold stays."""
    s = _COMMENT.sub("", src)
    s = _CMD_ARG.sub("", s)
    s = _ENV.sub("", s)
    s = _CMD.sub("", s)
    s = s.replace("{", "").replace("}", "").replace("~", " ")
    return re.sub(r"\n{3,}", "\n\n", s).strip() + "\n"


def tex_to_markdown(texfile: Path, mdfile: Path, timeout: float = 1.0) -> bool:
    """pandoc with the reference's flags and time limit; the stripper when pandoc is not installed."""
    if shutil.which("pandoc"):
        try:
            subprocess.run(["pandoc", "--wrap=none", "--from", "latex", str(texfile), "--output", str(mdfile)],
                           stderr=subprocess.PIPE, timeout=timeout, check=False)
        except subprocess.TimeoutExpired:
            return False
        return mdfile.exists()
    mdfile.write_text(strip_latex(texfile.read_text(encoding="utf8", errors="ignore")), encoding="utf8")
    return True


# ---- arXiv -----------------------------------------------------------------------------------------------------------
def fetch_arxiv_year(root: Path, year: int) -> None:
    """`<root>/md/<year>/` from `<root>/tex/<year>/`, which comes from `<root>/hep-th-<year>.tar.gz`, which is
    downloaded when it is not there."""
    texdir = root / "tex" / str(year)
    if not texdir.exists():
        tar = root / f"hep-th-{year}.tar.gz"
        if not tar.exists():
            try:
                print(f"Downloading Arxiv year {year}")
                _download(ARXIV_URL.format(year=year), tar)
            except Exception as e:
                raise RuntimeError(f"arxiv {year}: cannot download {ARXIV_URL.format(year=year)} ({e}); place the archive "
                                   f"at {tar} or its unpacked papers under {texdir}") from e
        with tarfile.open(tar) as t:
            t.extractall(root / "tex", filter="data")
    mddir = root / "md" / str(year)
    mddir.mkdir(parents=True, exist_ok=True)
    if not shutil.which("pandoc"):
        print("pandoc is not installed: converting LaTeX with the built-in stripper")
    for tex in sorted(p for p in texdir.iterdir() if p.is_file()):
        tex_to_markdown(tex, mddir / f"{tex.name}.md")


def tokenize_arxiv_year(root: Path, year: int, encode: Callable[[str], List[int]]) -> None:
    splits: Dict[str, List[int]] = {"train": [], "val": [], "test": []}
    for i, md in enumerate(sorted((root / "md" / str(year)).iterdir())):
        text = md.read_text(encoding="utf8", errors="ignore")
        splits["train" if i % 10 <= 6 else "val" if i % 10 <= 8 else "test"].extend(encode(text))
    out = root / str(year)
    out.mkdir(parents=True, exist_ok=True)
    for name, ids in splits.items():
        np.asarray(ids, dtype=np.uint16).tofile(out / f"{name}.npy")


def load_arxiv(datasets_dir: Path, years: Optional[Iterable[int]] = None, encode: Optional[Callable] = None) -> Dict[str, np.ndarray]:
    """{'train', 'val'}: uint16 token arrays, the years concatenated (raw memmaps named .npy like the reference's)."""
    years = list(ARXIV_YEARS if years is None else years)
    if not set(years) <= set(ARXIV_YEARS):
        raise ValueError(f"arxiv years must lie in {ARXIV_YEARS[0]}..{ARXIV_YEARS[-1]}")
    root = Path(datasets_dir) / "arxiv"
    root.mkdir(parents=True, exist_ok=True)
    for y in years:
        if not (root / "md" / str(y)).exists():
            fetch_arxiv_year(root, y)
    for y in years:
        if not (root / str(y) / "train.npy").exists():
            if encode is None:
                from .datasets import _tokenizer

                tok = _tokenizer()
                encode = lambda s: tok(s)[:-1]          # the reference does not append the end-of-text token here
            tokenize_arxiv_year(root, y, encode)
    return {split: np.concatenate([np.memmap(root / str(y) / f"{split}.npy", dtype=np.uint16, mode="r") for y in years])
            for split in ("train", "val")}


# ---- Shakespeare, character level --------------------------------------------------------------------------------------
def load_shakespeare_char(datasets_dir: Path) -> Dict[str, np.ndarray]:
    """{'train', 'val'} as uint16 arrays plus `vocab.txt` (one character code per line) beside them."""
    root = Path(datasets_dir) / "shakespeare"
    root.mkdir(parents=True, exist_ok=True)
    raw = root / "raw.txt"
    if not (root / "train.npy").exists():
        if not raw.exists():
            try:
                print("Downloading raw Shakespeare texts")
                _download(SHAKESPEARE_URL, raw)
            except Exception as e:
                raise RuntimeError(f"shakespeare-char: cannot download {SHAKESPEARE_URL} ({e}); place the text at {raw}") from e
        lines = raw.read_text(encoding="utf8").splitlines(keepends=True)
        chars = sorted(set("".join(lines)))
        lut = {c: i for i, c in enumerate(chars)}
        cut = int(len(lines) * 0.9)
        for name, part in (("train", lines[:cut]), ("val", lines[cut:])):
            np.asarray([lut[c] for c in "".join(part)], dtype=np.uint16).tofile(root / f"{name}.npy")
        (root / "vocab.txt").write_text("\n".join(str(ord(c)) for c in chars))
    return {s: np.memmap(root / f"{s}.npy", dtype=np.uint16, mode="r") for s in ("train", "val")}
