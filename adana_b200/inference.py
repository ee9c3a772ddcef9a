"""Text generation from a training checkpoint.

    python inference.py --checkpoint <exp_dir | ckpt dir | main.pt> [--prompt "..."] [--stream]
                        [--temperature 0.8] [--top_k 200] [--max_tokens 100] [--device cuda:0]

Same command line and checkpoint discovery as the reference's `inference.py` (1-463): the experiment
directory's `summary.json` supplies the model arguments, `ckpts/latest/main.pt` (or `main.pt` / `ckpt.pt`)
the weights, key prefixes from DDP (`module.`) and compiled models (`_orig_mod.`) are stripped, and
without `--prompt` the tool drops into an interactive loop.  A checkpoint of an FSDP run, which has no `main.pt`,
is read too: its `sharded/` directory (the `torch.distributed.checkpoint` layout, whether written here or by the
reference) is reassembled into full tensors without a process group (`train/checkpoint.py::full_state_from_sharded`);
the reference's tool reads DDP/single checkpoints only.

The decode loop is new: the reference re-runs the whole context through the network for every new token
(models/base.py generate: O(T²) per sequence).  `KVDecoder` keeps per-layer key/value caches for the RoPE
decoders (Enoki / DiLoCo, Qwen3 incl. GQA and the sigmoid output gate), so a token costs one row of every
GEMM plus one attention row; prefill is a single batched pass.  Other architectures, and contexts that
outgrow the trained sequence length (where the reference slides the window and re-bases the positions),
fall back to the model's own `generate`.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

from .models.enoki import apply_rotary_emb


def _sharded_marker(ckpt_dir: Path):
    """The index file of the `sharded/` directory of a checkpoint written by an FSDP run, or None (`.metadata` of a
    torch.distributed.checkpoint directory; `layout.json` of the flat-shard files earlier versions wrote)."""
    for name in (".metadata", "layout.json"):
        f = ckpt_dir / "sharded" / name
        if f.exists():
            return f
    return None


def find_checkpoint_file(path):
    """-> (checkpoint file, experiment directory) for a file, an exp dir, `ckpts/` or `ckpts/<name>/`.  For a
    checkpoint of an FSDP run (no `main.pt`) the file returned is the index file of its `sharded/` directory."""
    p = Path(path)
    if p.is_file() and p.suffix == ".pt":
        exp = p.parent.parent.parent if p.parent.parent.name == "ckpts" else p.parent
        return p, exp
    if p.is_dir():
        if p.parent.name == "ckpts" and (p / "main.pt").exists():
            return p / "main.pt", p.parent.parent
        if p.name == "ckpts" and (p / "latest" / "main.pt").exists():
            return p / "latest" / "main.pt", p.parent
        for cand in (p / "ckpts" / "latest" / "main.pt", p / "main.pt", p / "ckpt.pt"):
            if cand.exists():
                return cand, p
        for d, exp in ((p / "ckpts" / "latest", p), (p / "latest", p.parent), (p, p.parent.parent)):
            if _sharded_marker(d) is not None:
                return _sharded_marker(d), exp
    tried = [str(p / "ckpts" / "latest" / "main.pt"), str(p / "main.pt"), str(p / "ckpt.pt")]
    raise FileNotFoundError("could not find a checkpoint file; tried:\n  " + "\n  ".join(tried))


def load_config(path):
    ckpt, exp = find_checkpoint_file(path)
    summary = exp / "summary.json"
    if not summary.exists():
        raise FileNotFoundError(f"{summary} is required: it records the arguments the model was built with")
    args = json.loads(summary.read_text()).get("args")
    if args is None:
        raise ValueError("summary.json has no 'args' entry")
    return argparse.Namespace(**args), ckpt


def strip_prefixes(state):
    out = {}
    for k, v in state.items():
        while k.startswith(("_orig_mod.", "module.")):
            k = k.split(".", 1)[1]
        out[k.replace("._orig_mod.", ".")] = v
    return out


def load_model(path, device="cpu"):
    from .models.utils import get_model

    cfg, ckpt = load_config(path)
    cfg.device = device
    cfg.dropout = 0.0
    model = get_model(cfg)
    if ckpt.name in (".metadata", "layout.json"):      # sharded checkpoint of an FSDP run: reassemble the full tensors
        from .train.checkpoint import full_state_from_sharded

        blob = {"model": full_state_from_sharded(ckpt.parent)}
        meta = ckpt.parent.parent / "meta.pt"
        if meta.exists():
            blob["itr"] = torch.load(meta, map_location="cpu", weights_only=False).get("itr")
    else:
        blob = torch.load(ckpt, map_location="cpu", weights_only=False)
    state = strip_prefixes(blob["model"] if "model" in blob else blob)
    missing, unexpected = model.load_state_dict(state, strict=False)
    # a tied output head is the embedding tensor itself: a checkpoint that stores the tensor once is complete
    params = dict(model.named_parameters(remove_duplicate=False))
    stored = {id(params[k]) for k in state if k in params}
    missing = [k for k in missing if k not in params or id(params[k]) not in stored]
    if missing:
        print(f"warning: {len(missing)} parameters missing from the checkpoint (e.g. {missing[0]})", file=sys.stderr)
    if unexpected:
        print(f"warning: {len(unexpected)} unexpected entries (e.g. {unexpected[0]})", file=sys.stderr)
    itr = blob.get("itr")
    print(f"loaded {ckpt} (iteration {itr}) — {sum(p.numel() for p in model.parameters()) / 1e6:.1f}M parameters")
    return model.to(device).eval()


# ---- incremental decoding ----------------------------------------------------------------------------------------
class KVDecoder:
    """Key/value-cached forward for the RoPE decoders.  `supported(model)` tells whether it applies."""

    def __init__(self, model, max_len=None, batch=1, dtype=None):
        self.m = model
        self.arch = model.arch
        blocks = model.transformer.h
        a0 = blocks[0].attn
        self.hd = a0.qkv_dim
        self.n_kv = getattr(a0, "n_kv_head", a0.n_head)
        self.max_len = max_len or model.config.sequence_length
        dev = next(model.parameters()).device
        dtype = dtype or next(model.parameters()).dtype
        self.k = [torch.zeros(batch, self.n_kv, self.max_len, self.hd, device=dev, dtype=dtype) for _ in blocks]
        self.v = [torch.zeros_like(t) for t in self.k]
        self.pos = 0
        self.freqs = model.freqs_cis.to(dev)

    @staticmethod
    def supported(model) -> bool:
        arch = getattr(model, "arch", None)
        if arch not in ("enoki", "diloco", "qwen3") or not hasattr(model, "freqs_cis"):
            return False
        return not any(type(b.mlp).__name__ == "MoE" or "MoE" in type(b.mlp).__name__ for b in model.transformer.h)

    def _attn(self, li, attn, x):
        B, T, _ = x.shape
        gate = None
        if self.arch == "qwen3":
            q = attn.q_proj(x)
            k = attn.k_proj(x).view(B, T, -1, self.hd)
            v = attn.v_proj(x).view(B, T, -1, self.hd)
            if attn.gate:
                q, gate = q.view(B, T, -1, 2 * self.hd).split([self.hd, self.hd], dim=-1)
            else:
                q = q.view(B, T, -1, self.hd)
            if attn.use_qknorm:
                q, k = attn.q_norm(q), attn.k_norm(k)
            out_proj = attn.o_proj
        else:
            q, k, v = attn.c_attn(x).chunk(3, dim=-1)
            q, k, v = (t.view(B, T, -1, self.hd) for t in (q, k, v))
            if attn.use_qknorm:
                q, k = attn.q_layernorm(q), attn.k_layernorm(k)
            out_proj = attn.c_proj
        q, k = apply_rotary_emb(q, k, self.freqs[self.pos:self.pos + T])
        q, k = q.to(v.dtype).transpose(1, 2), k.to(v.dtype).transpose(1, 2)
        self.k[li][:, :, self.pos:self.pos + T] = k
        self.v[li][:, :, self.pos:self.pos + T] = v.transpose(1, 2)
        end = self.pos + T
        keys, vals = self.k[li][:, :, :end], self.v[li][:, :, :end]
        if T == 1:
            y = F.scaled_dot_product_attention(q, keys, vals, enable_gqa=self.n_kv != q.size(1))
        else:
            # prefill on top of an existing cache: row i of the new block sees cache + new tokens up to i
            mask = torch.ones(T, end, dtype=torch.bool, device=x.device).tril(diagonal=self.pos)
            y = F.scaled_dot_product_attention(q, keys, vals, attn_mask=mask, enable_gqa=self.n_kv != q.size(1))
        y = y.transpose(1, 2)
        if gate is not None:
            y = y * torch.sigmoid(gate)
        return out_proj(y.reshape(B, T, -1))

    @torch.no_grad()
    def forward(self, idx):
        """idx [B, T] new tokens -> logits of the last position [B, V]; advances the cache by T."""
        m = self.m
        T = idx.size(1)
        if self.pos + T > self.max_len:
            raise ValueError("context longer than the cache")
        x = m.transformer.wte(idx)
        for li, blk in enumerate(m.transformer.h):
            x = x + blk.scale * self._attn(li, blk.attn, blk.ln_1(x))
            y, _ = blk.mlp(blk.ln_2(x))
            x = x + blk.scale * y
        self.pos += T
        return m.lm_head(m.transformer.ln_f(x[:, -1:, :]))[:, 0, :]


def _sample(logits, temperature, top_k):
    if temperature == 0:
        return logits.argmax(-1, keepdim=True)
    logits = logits / temperature
    if top_k is not None:
        kth = torch.topk(logits, min(top_k, logits.size(-1))).values[:, [-1]]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    return torch.multinomial(F.softmax(logits.float(), dim=-1), 1)


@torch.no_grad()
def generate_tokens(model, idx, max_new_tokens, temperature=1.0, top_k=None):
    """Yields one [B,1] tensor of token ids at a time.  Cached decode when the architecture allows it."""
    S = model.config.sequence_length
    if KVDecoder.supported(model) and idx.size(1) + max_new_tokens <= S:
        dec = KVDecoder(model, batch=idx.size(0))
        logits = dec.forward(idx)
        for i in range(max_new_tokens):
            nxt = _sample(logits, temperature, top_k)
            yield nxt
            if i + 1 < max_new_tokens:
                logits = dec.forward(nxt)
        return
    for _ in range(max_new_tokens):
        ctx = idx if idx.size(1) <= S else idx[:, -S:]
        logits = model(ctx, get_logits=True)["logits"][:, -1, :]
        nxt = _sample(logits, temperature, top_k)
        idx = torch.cat((idx, nxt), dim=1)
        yield nxt


def _encode(model, text):
    dev = next(model.parameters()).device
    ids = model.tokenizer.encode(text, allowed_special={"<|endoftext|>"})
    return torch.tensor(ids, dtype=torch.long, device=dev).view(1, -1)


def generate_from_string(model, prompt, max_new_tokens, temperature=1.0, top_k=None):
    idx = _encode(model, prompt)
    new = [t for t in generate_tokens(model, idx, max_new_tokens, temperature, top_k)]
    return model.tokenizer.decode(torch.cat([idx] + new, dim=1)[0].tolist())


def stream_generate(model, prompt, max_new_tokens, temperature=1.0, top_k=None, out=sys.stdout):
    """Print text as tokens arrive.  Byte-level BPE pieces can end inside a UTF-8 sequence, so the whole
    continuation is re-decoded and only the stable new suffix is written."""
    idx = _encode(model, prompt)
    out.write(prompt)
    out.flush()
    ids, shown = [], ""
    for t in generate_tokens(model, idx, max_new_tokens, temperature, top_k):
        ids.append(int(t[0, 0]))
        text = model.tokenizer.decode(ids)
        if text.endswith("�"):
            continue
        out.write(text[len(shown):])
        out.flush()
        shown = text
    out.write("\n")
    return prompt + shown


def main(argv=None):
    p = argparse.ArgumentParser(description="Generate text from a checkpoint")
    p.add_argument("--checkpoint", type=str, default=None, help="experiment directory, checkpoint directory or .pt file")
    p.add_argument("--resume_from", type=str, default=None, help="alias for --checkpoint")
    p.add_argument("--device", type=str, default=None)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top_k", type=int, default=200, help="0 disables top-k")
    p.add_argument("--max_tokens", type=int, default=100)
    p.add_argument("--prompt", type=str, default=None, help="omit for interactive mode")
    p.add_argument("--stream", action="store_true")
    a = p.parse_args(argv)
    path = a.resume_from or a.checkpoint
    if path is None:
        p.error("--checkpoint is required")
    device = a.device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    print(f"Using device: {device}")
    model = load_model(path, device)
    top_k = None if a.top_k == 0 else a.top_k

    def run(prompt):
        if a.stream:
            stream_generate(model, prompt, a.max_tokens, a.temperature, top_k)
        else:
            print(generate_from_string(model, prompt, a.max_tokens, a.temperature, top_k))

    if a.prompt is not None:
        run(a.prompt)
        return 0
    print(f"temperature={a.temperature} top_k={a.top_k} max_tokens={a.max_tokens}; 'quit' to stop")
    while True:
        try:
            prompt = input("Enter prompt: ").strip()
        except (EOFError, KeyboardInterrupt):
            print()
            break
        if prompt.lower() in ("quit", "exit", "q"):
            break
        if prompt:
            run(prompt)
            print()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
