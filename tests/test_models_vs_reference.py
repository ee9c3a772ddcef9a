"""Every model family against the reference's own class: same parameter names, and with the reference's weights
loaded the same logits and loss (bit for bit on CPU fp32).  Needs the unmodified reference under baseline/_ref."""
import argparse
import sys
import types

import pytest
import torch

COMMON = ["--n_layer", "2", "--n_head", "2", "--n_embd", "128", "--sequence_length", "64", "--batch_size", "2",
          "--vocab_size", "512", "--dtype", "float32", "--device", "cpu", "--dropout", "0.0", "--z_loss_coeff", "1e-3"]
CASES = {
    "base": ["--model", "base"],
    "llama": ["--model", "llama", "--multiple_of", "32"],
    "enoki": ["--model", "enoki", "--qkv_dim", "64", "--mlp_hidden_dim", "256"],
    "qwen3": ["--model", "qwen3", "--qkv_dim", "64", "--mlp_hidden_dim", "256"],
    "qwen3next": ["--model", "qwen3next", "--qkv_dim", "64", "--mlp_hidden_dim", "256"],
    "qwen3-moe": ["--model", "qwen3", "--qkv_dim", "64", "--mlp_hidden_dim", "256", "--moe", "--moe_num_experts", "4",
                  "--moe_num_experts_per_tok", "2"],
    "base-moe": ["--model", "base", "--moe", "--moe_num_experts", "4", "--moe_num_experts_per_tok", "2"],
    "test": ["--model", "test"],
    "diloco": ["--model", "diloco", "--qkv_dim", "64", "--mlp_hidden_dim", "256"],
    "base-parallel-block": ["--model", "base", "--parallel_block"],
    "enoki-bias": ["--model", "enoki", "--qkv_dim", "64", "--mlp_hidden_dim", "256", "--bias", "True"],
    "qwen3-as-launched": ["--model", "qwen3", "--qkv_dim", "64", "--mlp_hidden_dim", "256", "--elementwise_attn_output_gate",
                          "--normalization_layer_type", "rmsnorm", "--weight_tying", "False"],
    "qwen3-moe-shared-expert": ["--model", "qwen3", "--qkv_dim", "64", "--mlp_hidden_dim", "256", "--moe", "--moe_num_experts", "4",
                                "--moe_num_experts_per_tok", "2", "--moe_num_shared_experts", "1"],
    "qwen3-moe-expert-choice": ["--model", "qwen3", "--qkv_dim", "64", "--mlp_hidden_dim", "256", "--moe", "--moe_num_experts", "4",
                                "--moe_routing", "expert_choice"],
    "qwen3next-moe": ["--model", "qwen3next", "--qkv_dim", "64", "--mlp_hidden_dim", "256", "--moe", "--moe_num_experts", "4",
                      "--moe_num_experts_per_tok", "2"],
    "llama-moe": ["--model", "llama", "--multiple_of", "32", "--moe", "--moe_num_experts", "4", "--moe_num_experts_per_tok", "2"],
}
_REF_TOP = ("config", "models", "optim", "data", "distributed", "logger")


def _forget_reference_modules():
    for k in [k for k in sys.modules if k.split(".")[0] in _REF_TOP]:
        del sys.modules[k]


def _reference_model(ref_src, argv, monkeypatch):
    import tiktoken

    monkeypatch.setattr(tiktoken, "get_encoding", lambda name: types.SimpleNamespace(name=name))   # no network here
    _forget_reference_modules()
    sys.path.insert(0, str(ref_src))
    try:
        import config as ref_config
        from models.utils import get_model as ref_get_model

        parser = argparse.ArgumentParser(allow_abbrev=False)
        parser.add_argument("--config_format", default="base")
        args = ref_config.parse_args_with_format(format="base", base_parser=parser, namespace=None, args=argv)
        torch.manual_seed(0)
        model = ref_get_model(args)
        model._group_specs = model.get_parameter_group_specs()     # imports its packages lazily: ask while they resolve
        return model
    finally:
        sys.path.remove(str(ref_src))
        _forget_reference_modules()


@pytest.mark.parametrize("name", sorted(CASES))
def test_model_equals_the_reference_class_on_the_reference_weights(ref_src, name, monkeypatch):
    from adana_b200.config import parse_args_with_format
    from adana_b200.models.utils import get_model

    torch.compiler.set_stance("force_eager")       # the reference decorates helpers with torch.compile
    argv = COMMON + CASES[name]
    ref = _reference_model(ref_src, argv, monkeypatch)
    parser = argparse.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base")
    torch.manual_seed(1)
    ours = get_model(parse_args_with_format(format="base", base_parser=parser, namespace=None, args=argv))
    ref_sd = ref.state_dict()
    assert set(ref_sd) == set(ours.state_dict())                      # checkpoint-compatible names
    for k, v in ours.state_dict().items():
        assert v.shape == ref_sd[k].shape, k
    # the same split into decayed and undecayed parameters (what weight decay is applied to)
    canon = lambda specs: sorted((tuple(sorted(g["params"])), repr({k: v for k, v in g.items() if k != "params"})) for g in specs)
    assert canon(ours.get_parameter_group_specs()) == canon(ref._group_specs)
    ours.load_state_dict(ref_sd)
    ref.eval()
    ours.eval()
    torch.manual_seed(5)
    idx, tgt = torch.randint(0, 512, (2, 64)), torch.randint(0, 512, (2, 64))
    with torch.no_grad():
        want = ref(idx, targets=tgt, get_logits=True)
        got = ours(idx, targets=tgt, get_logits=True)
    assert torch.allclose(got["logits"], want["logits"], atol=1e-6, rtol=0)
    assert abs(float(got["loss"]) - float(want["loss"])) < 1e-6


@pytest.mark.parametrize("name", ["enoki", "qwen3-moe", "qwen3next", "llama"])
def test_training_loss_and_gradients_equal_the_reference(ref_src, name, monkeypatch):
    """Train mode (z-loss and, for MoE, the router's auxiliary losses included): the same loss and the same
    gradient for every parameter."""
    from adana_b200.config import parse_args_with_format
    from adana_b200.models.utils import get_model

    torch.compiler.set_stance("force_eager")
    argv = COMMON + CASES[name]
    ref = _reference_model(ref_src, argv, monkeypatch)
    parser = argparse.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base")
    ours = get_model(parse_args_with_format(format="base", base_parser=parser, namespace=None, args=argv))
    ours.load_state_dict(ref.state_dict())
    ref.train()
    ours.train()
    torch.manual_seed(6)
    idx, tgt = torch.randint(0, 512, (2, 64)), torch.randint(0, 512, (2, 64))
    lw = ref(idx, targets=tgt)["loss"]
    lg = ours(idx, targets=tgt)["loss"]
    assert abs(lg.item() - lw.item()) < 1e-6
    lw.backward()
    lg.backward()
    ref_grads = {k: p.grad for k, p in ref.named_parameters()}
    for k, p in ours.named_parameters():
        if ref_grads[k] is None:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0, k
        else:
            assert torch.allclose(p.grad, ref_grads[k], atol=2e-6, rtol=1e-5), (k, float((p.grad - ref_grads[k]).abs().max()))


@pytest.mark.parametrize("name", ["enoki", "qwen3-moe"])
def test_evaluation_equals_the_reference_eval(ref_src, name, monkeypatch):
    """The evaluation loop (loss, accuracy, perplexity, auxiliary losses, router logits for MoE) against the
    reference's `eval` over the same validation batches."""
    import importlib

    import numpy as np

    from adana_b200.config import parse_args_with_format
    from adana_b200.data.readers import DataReader
    from adana_b200.models.utils import get_model
    from adana_b200.train.loop import evaluate

    torch.compiler.set_stance("force_eager")
    argv = COMMON + CASES[name]
    moe = "moe" in name
    toks = np.random.default_rng(2).integers(0, 512, size=20000).astype(np.uint16)
    kw = dict(local_batch_size=2, sequence_length=64, seed=3, keep_in_ram=True, with_replacement=False, auto_shard=False)
    ref = _reference_model(ref_src, argv, monkeypatch)
    if "wandb" not in sys.modules:
        try:
            import wandb  # noqa: F401
        except Exception:
            monkeypatch.setitem(sys.modules, "wandb", types.ModuleType("wandb"))
    sys.path.insert(0, str(ref_src))
    try:
        ref_eval = importlib.import_module("optim.utils").eval
        ref_reader = importlib.import_module("data.utils").DataReader(toks, **kw)
        ref_reader.set_step(0)
        ref.eval()
        want = ref_eval(ref, ref_reader, max_num_batches=5, moe=moe, get_router_logits=moe)
    finally:
        sys.path.remove(str(ref_src))
        _forget_reference_modules()
    parser = argparse.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base")
    ours = get_model(parse_args_with_format(format="base", base_parser=parser, namespace=None, args=argv))
    ours.load_state_dict(ref.state_dict())
    ours.eval()
    reader = DataReader(toks, **kw)
    reader.set_step(0)
    got = evaluate(ours, reader, max_num_batches=5, moe=moe, get_router_logits=moe)
    assert got[0] == pytest.approx(want[0], abs=1e-7) and got[1] == pytest.approx(want[1], abs=1e-6)
    assert got[2] == pytest.approx(want[2], rel=1e-6)
    assert set(got[3]) == set(want[3])
    for k in want[3]:
        assert got[3][k] == pytest.approx(want[3][k], abs=1e-6), k
    if moe:
        assert got[4].shape == want[4].shape and torch.allclose(got[4], want[4], atol=1e-5)


@pytest.mark.parametrize("name", ["base", "llama", "enoki", "qwen3"])
def test_tensor_parallel_plan_equals_the_reference(ref_src, name, monkeypatch):
    """Which projections are split by columns and which by rows under `--tp_size`."""
    from adana_b200.config import parse_args_with_format
    from adana_b200.models.utils import get_model

    torch.compiler.set_stance("force_eager")
    argv = COMMON + CASES[name]
    ref = _reference_model(ref_src, argv, monkeypatch)
    want = {path: type(style).__name__.replace("Parallel", "").lower() for path, style in type(ref).get_tp_plan().items()}
    parser = argparse.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base")
    ours = get_model(parse_args_with_format(format="base", base_parser=parser, namespace=None, args=argv))
    assert dict(type(ours).get_tp_plan()) == want


@pytest.mark.parametrize("name", ["base", "enoki", "qwen3"])
def test_sampling_equals_the_reference_generate(ref_src, name, monkeypatch):
    """`model.generate` with temperature and top-k from the same RNG seed: the same tokens as the reference's; and
    the KV-cached decoder of the inference tool continues the same sequence."""
    from adana_b200 import inference
    from adana_b200.config import parse_args_with_format
    from adana_b200.models.utils import get_model

    torch.compiler.set_stance("force_eager")
    argv = COMMON + CASES[name]
    ref = _reference_model(ref_src, argv, monkeypatch)
    parser = argparse.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base")
    ours = get_model(parse_args_with_format(format="base", base_parser=parser, namespace=None, args=argv))
    ours.load_state_dict(ref.state_dict())
    ref.eval()
    ours.eval()
    prompt = torch.tensor([[5, 17, 300, 2]])
    with torch.no_grad():
        torch.manual_seed(7)
        want = ref.generate(prompt.clone(), 12, temperature=0.8, top_k=20)
        torch.manual_seed(7)
        got = ours.generate(prompt.clone(), 12, temperature=0.8, top_k=20)
        assert torch.equal(got, want)
        torch.manual_seed(7)
        stream = torch.cat(list(inference.generate_tokens(ours, prompt.clone(), 12, temperature=0.8, top_k=20)), dim=1)
    assert torch.equal(stream, want[:, prompt.shape[1]:])
