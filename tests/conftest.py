import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "slow: longer CPU test")


@pytest.fixture(scope="session")
def ref_src():
    """Path of an unmodified copy of the reference sources, when one is installed."""
    p = ROOT / "baseline" / "_ref" / "src"
    if not (p / "optim" / "adana.py").exists():
        pytest.skip("reference sources not installed under baseline/_ref")
    return p


def tiny_args(model="enoki", **kw):
    from adana_b200.config import flags

    a = flags.defaults()
    a.model, a.n_layer, a.n_head, a.n_embd, a.qkv_dim = model, 2, 2, 128, 64
    a.mlp_hidden_dim, a.sequence_length, a.vocab_size = 256, 32, 512
    a.dtype, a.device, a.weight_tying, a.init_scheme = "float32", "cpu", False, "ScaledGPT"
    a.z_loss_coeff, a.acc_steps, a.grad_clip, a.bias, a.dropout = 1e-3, 1, 0.5, False, 0.0
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def torchrun(nproc: int):
    """Command prefix that starts `nproc` ranks on this machine; torchrun picks a free rendezvous port itself
    (binding a port, closing it and handing the number on races with every other test that does the same)."""
    return [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
            "--nproc-per-node", str(nproc)]


@pytest.fixture(autouse=True)
def _checked_build_status_stays_clear(request):
    """Under the checked build (ADANA_DEBUG=1) every kernel compares the indices it computes with the extents it was
    given and reports a violation through the device status word: after each GPU test on valid inputs the word must
    still be 0 (tests of the bounded waits read and clear the word themselves)."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    from adana_b200.ops import _lib

    if not _lib.DEBUG_BUILD:
        return
    import torch

    if torch.cuda.is_available():
        buf = _lib.status_buffer()
        code = int(buf[0].item())
        buf.zero_()
        assert code == 0, f"checked build recorded status {_lib.STATUS_NAMES.get(code, code)}"
