import numpy as np
import pytest
import torch

from adana_b200.data import DataReader, MultiFileDataReader, PinnedBatchStager, make_zipf_tokens, write_zipf_dataset
from adana_b200.data.datasets import zipf_entropy


@pytest.fixture(scope="module")
def stream():
    return make_zipf_tokens(60_000, vocab=1000, exponent=1.0, seed=0)


def test_zipf_stream(stream):
    assert stream.dtype == np.uint16 and stream.max() < 1000
    counts = np.bincount(stream, minlength=1000)
    assert counts[0] > counts[9] > counts[99]
    assert counts[0] / counts[1] == pytest.approx(2.0, rel=0.15)
    assert 5.0 < zipf_entropy(1000) < 6.5
    assert zipf_entropy(50304) == pytest.approx(7.5664, abs=2e-3)


def test_reader_matches_the_documented_index_plan(stream):
    S, B = 64, 4
    r = DataReader(stream, B, S, seed=7, auto_shard=False)
    rng = np.random.default_rng(7)
    order = rng.permutation((len(stream) - S - 1) // S - 1)
    off = rng.integers(S)
    x, y = r.sample_batch()
    starts = order[:B] * S + off
    assert x.dtype == torch.int64 and x.shape == (B, S)
    for i, s in enumerate(starts):
        assert np.array_equal(x[i].numpy(), stream[s:s + S].astype(np.int64))
        assert np.array_equal(y[i].numpy(), stream[s + 1:s + S + 1].astype(np.int64))


def test_rank_sharding_is_disjoint_and_covers_global_batches(stream):
    S, B, N = 32, 4, 4
    single = DataReader(stream, B, S, seed=3, world_size=1, rank=0)
    ranks = [DataReader(stream, B, S, seed=3, world_size=N, rank=r) for r in range(N)]
    for step in range(3):
        per_rank = [r.sample_batch()[0] for r in ranks]
        for r in range(N):
            assert torch.equal(per_rank[r], single.sample_batch()[0])  # global batch N*step + r


def test_epoch_rollover_and_resume(stream):
    S, B = 128, 8
    r = DataReader(stream, B, S, seed=1, auto_shard=False)
    per_epoch = r.num_batches()
    for _ in range(per_epoch - 2):
        r.sample_batch()
    st = r.state_dict()
    nxt = [r.sample_batch()[0] for _ in range(5)]      # crosses into epoch 1
    assert r.last_epoch == 1
    r2 = DataReader(stream, B, S, seed=1, auto_shard=False)
    r2.load_state_dict(st)
    assert len(r2.preview_next_samples(2)) == 2 and r2.step == st["step"]  # peeking does not advance
    for t in nxt:
        assert torch.equal(r2.sample_batch()[0], t)


def test_with_replacement(stream):
    r = DataReader(stream, 4, 32, seed=5, with_replacement=True, world_size=2, rank=1)
    a = r.sample_batch()[0]
    r.set_step(0)
    assert torch.equal(a, r.sample_batch()[0])
    idx = np.random.default_rng(5 + 0 * 2 + 1).integers(len(stream) - 32 - 1, size=4)
    assert np.array_equal(a[0].numpy(), stream[idx[0]:idx[0] + 32].astype(np.int64))


def test_multi_file_reader_switches_and_resumes(tmp_path):
    files = write_zipf_dataset(tmp_path, n_train=60_000, n_val=5_000, vocab=500, n_files=3)
    train = {k: v for k, v in files.items() if k.startswith("train_")}
    r = MultiFileDataReader(train, 4, 64, seed=11, auto_shard=False)
    n = r.current_file_num_batches()
    seen = []
    for i in range(n + 3):
        if i == n - 1:
            st = r.state_dict()
        seen.append(r.sample_batch()[0])
    assert r.current_file_idx == 1 and r.step == 3
    r2 = MultiFileDataReader(train, 4, 64, seed=11, auto_shard=False)
    r2.load_state_dict(st)
    for t in seen[n - 1:]:
        assert torch.equal(r2.sample_batch()[0], t)
    single = DataReader(np.fromfile(train["train_0001"], dtype=np.uint16), 4, 64, seed=11 + 1000, auto_shard=False)
    assert torch.equal(seen[n], single.sample_batch()[0])


def test_pinned_stager_cpu_path(stream):
    r1 = DataReader(stream, 4, 32, seed=2, auto_shard=False)
    r2 = DataReader(stream, 4, 32, seed=2, auto_shard=False)
    for look in (True, False):
        r1.set_step(0)
        r2.set_step(0)
        st = PinnedBatchStager(r1, "cpu", lookahead=look)
        for _ in range(4):
            x, y = st.next_batch()
            xr, yr = r2.sample_batch()
            assert torch.equal(x, xr) and torch.equal(y, yr)
        assert st.bytes_per_batch == 2 * 4 * 32 * 8


def test_batch_order_equals_the_reference_reader(ref_src, monkeypatch):
    """Same seed, same token file: the reference's DataReader and this one deliver the same batches, step after
    step and after a jump with `set_step` (what lets a run be resumed, or compared, across the two code bases)."""
    import importlib
    import sys
    import types

    import numpy as np
    import tiktoken
    import torch

    from adana_b200.data.readers import DataReader

    monkeypatch.setattr(tiktoken, "get_encoding", lambda name: types.SimpleNamespace(name=name))
    if "adana_refdata" not in sys.modules:
        pkg = types.ModuleType("adana_refdata")
        pkg.__path__ = [str(ref_src / "data")]
        sys.modules["adana_refdata"] = pkg
    ref = importlib.import_module("adana_refdata.utils")
    toks = np.random.default_rng(0).integers(0, 50000, size=200000).astype(np.uint16)
    kw = dict(local_batch_size=4, sequence_length=64, seed=7, keep_in_ram=True, with_replacement=False, auto_shard=False)
    a, b = DataReader(toks, **kw), ref.DataReader(toks, **kw)
    assert a.num_batches() == b.num_batches()
    for start in (0, 333, 779):
        a.set_step(start)
        b.set_step(start)
        for _ in range(20):
            (xa, ya), (xb, yb) = a.sample_batch(), b.sample_batch()
            assert torch.equal(xa, xb) and torch.equal(ya, yb)


def test_multi_file_reader_equals_the_reference_reader(ref_src, monkeypatch, tmp_path, capsys):
    """Four token files, 400 batches (several file switches): the same batches as the reference's
    MultiFileDataReader, the same `state_dict()` keys, and each side resumes from the other's state."""
    import copy
    import importlib
    import sys
    import types

    import numpy as np
    import tiktoken
    import torch

    from adana_b200.data.readers import MultiFileDataReader

    monkeypatch.setattr(tiktoken, "get_encoding", lambda name: types.SimpleNamespace(name=name))
    if "adana_refdata" not in sys.modules:
        pkg = types.ModuleType("adana_refdata")
        pkg.__path__ = [str(ref_src / "data")]
        sys.modules["adana_refdata"] = pkg
    ref = importlib.import_module("adana_refdata.utils")
    rng = np.random.default_rng(0)
    files = {}
    for i in range(4):
        f = tmp_path / f"train_{i:04d}.bin"
        rng.integers(0, 50000, size=20000 + 1000 * i).astype(np.uint16).tofile(f)
        files[f"train_{i:04d}"] = str(f)
    kw = dict(local_batch_size=4, sequence_length=64, seed=11, with_replacement=False, auto_shard=False, keep_in_ram=True)
    a, b = MultiFileDataReader(data_files=files, **kw), ref.MultiFileDataReader(data_files=files, **kw)
    a.set_step(0)
    b.set_step(0)
    for _ in range(400):
        (xa, ya), (xb, yb) = a.sample_batch(), b.sample_batch()
        assert torch.equal(xa, xb) and torch.equal(ya, yb)
    sa, sb = a.state_dict(), b.state_dict()
    assert set(sa) == set(sb) and sa["step"] == sb["step"] and sa["current_file_idx"] == sb["current_file_idx"]
    a2, b2 = MultiFileDataReader(data_files=files, **kw), ref.MultiFileDataReader(data_files=files, **kw)
    a2.load_state_dict(copy.deepcopy(sb))
    b2.load_state_dict(copy.deepcopy(sa))
    for _ in range(50):
        x = a.sample_batch()[0]
        assert torch.equal(x, b.sample_batch()[0]) and torch.equal(x, a2.sample_batch()[0]) and torch.equal(x, b2.sample_batch()[0])
    capsys.readouterr()


def test_arxiv_and_shakespeare_preparers_run_from_local_sources(tmp_path):
    """The corpora with their own sources: a year's tar archive of LaTeX papers -> Markdown -> tokens dealt 7/2/1 by
    position, and the character-level Shakespeare split 90/10 by lines; offline they start from local files."""
    import io
    import tarfile
    import types

    from adana_b200.data import text_sources as TS
    from adana_b200.data.datasets import get_dataset

    root = tmp_path / "arxiv"
    root.mkdir()
    with tarfile.open(root / "hep-th-2000.tar.gz", "w:gz") as tar:
        for i in range(10):
            body = (f"% a comment\n\\documentclass{{article}}\\begin{{document}}\\section{{Paper {i}}} We study $x_{i}$ "
                    f"\\cite{{foo}} in detail.\\end{{document}}\n").encode()
            info = tarfile.TarInfo(f"2000/00010{i:02d}")
            info.size = len(body)
            tar.addfile(info, io.BytesIO(body))
    assert "comment" not in TS.strip_latex("text % comment\n\\cite{a} more") and "more" in TS.strip_latex("\\cite{a} more")
    out = TS.load_arxiv(tmp_path, [2000], encode=lambda s: [ord(c) % 251 for c in s])
    assert len(list((root / "md" / "2000").iterdir())) == 10
    n_train, n_val = len(out["train"]), len(out["val"])
    n_test = len(np.memmap(root / "2000" / "test.npy", dtype=np.uint16, mode="r"))
    assert n_train > n_val > n_test > 0 and abs(n_train / (n_val / 2) - 7) < 1.5      # 7 : 2 : 1 papers
    with pytest.raises(ValueError):
        TS.load_arxiv(tmp_path, [1992])

    sh = tmp_path / "shakespeare"
    sh.mkdir()
    (sh / "raw.txt").write_text("".join(f"line {i}: to be or not to be\n" for i in range(50)))
    args = types.SimpleNamespace(dataset="shakespeare-char", datasets_dir=str(tmp_path), vocab_size=50304)
    d = get_dataset(args)
    vocab = (sh / "vocab.txt").read_text().split()
    assert len(d["train"]) > 8 * len(d["val"]) > 0 and int(max(d["train"].max(), d["val"].max())) == len(vocab) - 1
    assert chr(int(vocab[int(d["train"][0])])) == "l"
