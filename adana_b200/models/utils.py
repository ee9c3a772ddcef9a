"""Model factory keyed by `--model` (reference: src/models/utils.py:21-72)."""
from __future__ import annotations


def get_model(args):
    name = args.model
    if getattr(args, "init_compat", "none") == "reference" and name not in ("enoki", "diloco", "qwen3"):
        # asked-for bit-identical initial weights must not silently become different ones
        raise NotImplementedError(f"--init_compat reference covers --model enoki, diloco and qwen3, not {name}")
    if name in ("enoki", "diloco"):
        from .enoki import Enoki

        return Enoki(args)
    if name == "qwen3":
        from .qwen3 import Qwen3

        return Qwen3(args)
    if name == "qwen3next":
        from .qwen3next import Qwen3Next

        return Qwen3Next(args)
    if name == "base":
        from .gpt import GPTBase

        return GPTBase(args)
    if name == "llama":
        from .llama import Llama

        return Llama(args)
    if name == "test":
        from .test_model import Test

        return Test(args)
    raise KeyError(f"Unknown model '{name}'.")
