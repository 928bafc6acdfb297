"""Small Finezen configurations and the glue between model folders and the plain implementation."""

from __future__ import annotations

import json
from pathlib import Path

import torch

from plain import finezen_plain as plain


def attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        out["mask"] = {"size": window}
    if rot:
        out["rot"] = rot
    return {"type": "attention", "mixer": out}


def rot(dims, base, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def latent(heads, dim, vdim, kv_rank, q_rank, scale, window=None):
    out = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if window:
        out["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": out}


def moe(ff, experts, top, shared=0):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


def config(vocab, width, layers, scale=1.0, mult=1.0, loop=None, eps=1e-5):
    out = {"architecture": "Finezen", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
           "residual_mult": mult, "layers": layers}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Odd sizes: several kv heads, value heads smaller and larger than key heads, windows shorter and
# longer than a page, every band of the frequency ramp met within a few dozen positions, a layer
# without rotation, one without a window, one without a feed-forward, one without a shared expert,
# two and three chosen experts, a loop over the two middle layers run three times.
SMALL_A = config(211, 64, [
    layer(attention(4, 2, 12, 20, 0.3, window=7, rot=rot(8, 40.0, (3.0, 48, 6.0, 1.5))), moe(40, 6, 2, shared=24)),
    layer(latent(3, 8, 12, 20, 24, 0.35, window=21), moe(24, 5, 3)),
    layer(attention(6, 3, 10, 6, 0.32, rot=rot(10, 900.0)), None),
    layer(latent(2, 12, 6, 28, 80, 0.3), moe(56, 9, 1, shared=40)),
    layer(attention(2, 1, 16, 16, 0.25, window=33), moe(32, 4, 4, shared=8)),
], scale=2.5, mult=0.6, loop=(1, 3, 3))
# Sizes that the tensor-core kernels take; the loop starts at the first layer and ends at the last.
SMALL_B = config(257, 128, [
    layer(attention(4, 2, 64, 64, 0.125, window=40, rot=rot(32, 10000.0, (4.0, 64, 16.0, 2.0))), moe(64, 8, 2, shared=128)),
    layer(latent(4, 32, 32, 64, 48, 0.18, window=24), moe(128, 4, 2, shared=64)),
    layer(attention(2, 2, 128, 128, 0.09, window=16, rot=rot(128, 500000.0)), moe(64, 7, 3)),
], scale=1.0, mult=1.0, loop=(0, 3, 2), eps=1e-6)
# No loop; one head; a window of one (a token sees itself only) and of two; everything rotated; a
# width that is no multiple of 8 (no tensor-core product takes it).
NO_LOOP = config(97, 52, [
    layer(attention(1, 1, 8, 8, 0.4, window=1, rot=rot(8, 100.0)), moe(32, 3, 1, shared=16)),
    layer(latent(1, 8, 16, 24, 32, 0.3, window=2), moe(16, 2, 2)),
    layer(attention(3, 1, 8, 24, 0.35, window=50, rot=rot(4, 30.0, (2.0, 16, 4.0, 1.0))), None),
], scale=4.0, mult=1.3)
# A loop that is one layer run four times, a latent wider than 256 channels.
ONE_LAYER_LOOP = config(97, 48, [
    layer(latent(2, 8, 8, 288, 24, 0.3, window=19), moe(16, 16, 4, shared=32)),
    layer(attention(2, 2, 16, 8, 0.3, window=12, rot=rot(6, 1000.0, (8.0, 32, 8.0, 1.0))), moe(24, 3, 2)),
], scale=0.7, mult=0.5, loop=(1, 2, 4))
SMALL = {"small_a": (SMALL_A, 4, 41), "small_b": (SMALL_B, 16, 42), "no_loop": (NO_LOOP, 8, 43),
         "one_layer_loop": (ONE_LAYER_LOOP, 16, 44)}       # config, page size, seed


def write_model(folder: Path, raw: dict, seed: int, dtype=torch.bfloat16, sharpen: float = 4.0) -> Path:
    """A random model folder whose numbers make faults visible: query, key and value projections
    scaled up (one key's score stands out, so a wrong, missing or extra key shows), sinks, gates,
    norm weights, biases and slopes of a size that matters, router logits far enough apart that
    the choice is no close call."""
    from safetensors.torch import load_file, save_file

    from paged_attention_engine_b200.weights import write_random_model

    write_random_model(folder, raw, seed, dtype)
    path = str(Path(folder) / "model.safetensors")
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(seed + 1000)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith((".mix.q", ".mix.k", ".mix.v", ".mix.dq", ".mix.uq", ".mix.dkv", ".mix.uk", ".mix.uv", ".up", ".gate")):
            t = t * sharpen
        elif name.endswith(".mix.g"):
            t = t * 40.0
        elif name.endswith(".shared.sg"):
            t = t * 30.0
        elif name.endswith(".mix.sink"):
            t = torch.randn(t.shape, generator=gen) * 2.0
        elif name.endswith(".mlp.router"):
            t = t * 12.0
        elif name.endswith((".q.norm", ".k.norm", ".dq.norm", ".dkv.norm")):
            t = 1.0 + torch.rand(t.shape, generator=gen) * 1.5
        elif name.endswith(".alpha"):
            t = 0.3 + torch.rand(t.shape, generator=gen) * 0.9
        elif name.endswith(".b"):
            t = torch.randn(t.shape, generator=gen) * 0.2
        elif name.endswith(("norm1", "norm2", "norm1b", "norm2b", "final.norm")):
            t = (0.5 + torch.rand(t.shape, generator=gen)) * (torch.randint(0, 2, t.shape, generator=gen) * 2.0 - 1.0)
        elif name == "head":
            t = t * 12.0
        tensors[name] = t.to(tensors[name].dtype)
    save_file(tensors, path)
    return Path(folder)


def read_model(folder: Path):
    from safetensors.torch import load_file

    return json.loads((Path(folder) / "config.json").read_text()), load_file(str(Path(folder) / "model.safetensors"))


# A router's choice is a step function of its input: where two experts' logits are closer than
# rounding can move them, the engine may choose otherwise than the plain model, and rightly so.
# The tests' prompts avoid such tokens: a token whose choice is closer than this (in any routed
# layer run) is drawn again.
CLEAR_CHOICE = 0.03


def clear_requests(folder: Path, lengths, seed: int, margin: float = CLEAR_CHOICE):
    """(requests, logits): prompts of the given lengths for which no router's choice is a close
    call, drawn from `seed`, and the plain model's logits for them."""
    raw, tensors = read_model(folder)
    gen = torch.Generator().manual_seed(seed)
    requests, logits = {}, {}
    for i, n in enumerate(lengths):
        tokens = torch.randint(0, raw["vocab"], (n,), generator=gen).tolist()
        for _ in range(60 + 2 * n):
            margins = []
            out = plain.forward(raw, tensors, tokens, margins=margins)
            close = torch.stack(margins).min(dim=0).values < margin if margins else torch.zeros(n, dtype=torch.bool)
            if not bool(close.any()):
                break
            # a changed token changes what later tokens see: redraw the first close one and look again
            tokens[int(close.nonzero()[0])] = int(torch.randint(0, raw["vocab"], (1,), generator=gen))
        else:
            raise AssertionError(f"no prompt of {n} tokens with clear choices was found")
        requests[f"r{i}"], logits[f"r{i}"] = tokens, out.float()
    return requests, logits


FP32_RTOL = 5e-5
BF16_RTOL = 2.0 ** -5


def tolerance(dtype, reference: torch.Tensor) -> float:
    top = max(1.0, float(reference.abs().max()))
    return (FP32_RTOL if dtype in (torch.float32, "float32") else BF16_RTOL) * top


_rounding: dict = {}


def rounding_error(folder: Path, tokens) -> torch.Tensor:
    """Per position, how far the plain model's logits move when every sublayer's input is rounded
    to bfloat16 once, which is the least that a bfloat16 engine does. These models' weights are
    scaled up to make faults visible; the same scaling lets a position where two keys' scores nearly
    tie turn one rounding into a visible change of its logits."""
    key = (str(folder), tuple(tokens))
    if key not in _rounding:
        raw, tensors = read_model(folder)
        exact = plain.forward(raw, tensors, list(tokens))
        plain.narrow = lambda h: h.to(torch.bfloat16).to(h.dtype)
        try:
            rounded = plain.forward(raw, tensors, list(tokens))
        finally:
            plain.narrow = None
        _rounding[key] = (rounded - exact).abs().max(dim=1).values.float()
    return _rounding[key]


ROUNDINGS = 4.0


def row_tolerance(dtype, reference: torch.Tensor, folder: Path, tokens) -> torch.Tensor:
    """The tolerance per position: `tolerance`, and in bfloat16 at least ROUNDINGS times what one
    rounding of the sublayers' inputs does to that position in the plain model."""
    flat = torch.full((reference.shape[0],), tolerance(dtype, reference))
    if dtype in (torch.float32, "float32"):
        return flat
    return torch.maximum(flat, ROUNDINGS * rounding_error(folder, tokens))
