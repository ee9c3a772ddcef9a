"""Inference CLI pieces: checkpoint discovery, prefix stripping, KV-cached decode == full re-forward."""
import json

import pytest
import torch

from conftest import tiny_args
from adana_b200 import inference as inf
from adana_b200.models.utils import get_model


@pytest.mark.parametrize("arch,extra", [("enoki", {}), ("qwen3", dict(n_kv_head=2, elementwise_attn_output_gate=True))])
def test_kv_cache_decode_matches_full_forward(arch, extra):
    a = tiny_args(arch, **extra)
    torch.manual_seed(0)
    m = get_model(a).eval()
    assert inf.KVDecoder.supported(m)
    idx = torch.randint(0, a.vocab_size, (2, 9))
    dec = inf.KVDecoder(m, batch=2)
    got = [dec.forward(idx[:, :5])]                 # prefill
    for t in range(5, 9):                           # token by token
        got.append(dec.forward(idx[:, t:t + 1]))
    def full_at(t):                                  # the model returns last-position logits only
        with torch.no_grad():
            return m(idx[:, :t + 1], get_logits=True)["logits"][:, -1]

    for j, t in enumerate(range(4, 9)):
        assert torch.allclose(got[j], full_at(t), atol=2e-4, rtol=1e-4), (arch, t)
    # second prefill chunk on top of a warm cache
    dec2 = inf.KVDecoder(m, batch=2)
    dec2.forward(idx[:, :3])
    assert torch.allclose(dec2.forward(idx[:, 3:8]), full_at(7), atol=2e-4, rtol=1e-4)


def test_greedy_generation_equals_model_generate():
    a = tiny_args("enoki")
    torch.manual_seed(1)
    m = get_model(a).eval()
    idx = torch.randint(0, a.vocab_size, (1, 4))
    new = torch.cat(list(inf.generate_tokens(m, idx, 6, temperature=0, top_k=None)), dim=1)
    cur = idx
    with torch.no_grad():
        for _ in range(6):
            nxt = m(cur, get_logits=True)["logits"][:, -1].argmax(-1, keepdim=True)
            cur = torch.cat((cur, nxt), 1)
    assert torch.equal(new, cur[:, 4:])


def test_checkpoint_discovery_and_load(tmp_path):
    a = tiny_args("enoki")
    torch.manual_seed(2)
    m = get_model(a)
    exp = tmp_path / "exp"
    (exp / "ckpts" / "latest").mkdir(parents=True)
    state = {"module._orig_mod." + k: v for k, v in m.state_dict().items()}
    torch.save({"model": state, "itr": 7}, exp / "ckpts" / "latest" / "main.pt")
    (exp / "summary.json").write_text(json.dumps({"args": {k: v for k, v in vars(a).items()
                                                          if isinstance(v, (int, float, str, bool, type(None)))}}))
    for given in (exp, exp / "ckpts", exp / "ckpts" / "latest", exp / "ckpts" / "latest" / "main.pt"):
        f, d = inf.find_checkpoint_file(given)
        assert f == exp / "ckpts" / "latest" / "main.pt" and d == exp
    with pytest.raises(FileNotFoundError):
        inf.find_checkpoint_file(tmp_path / "nothing")
    m2 = inf.load_model(exp, "cpu")
    for (k, v), (k2, v2) in zip(m.state_dict().items(), m2.state_dict().items()):
        assert k == k2 and torch.equal(v, v2)
