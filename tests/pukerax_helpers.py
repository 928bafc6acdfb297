"""Small Pukerax configurations and the glue between model folders and the plain implementation."""

from __future__ import annotations

import json
from pathlib import Path

import torch

from plain import pukerax_plain as plain


def mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, dims=None):
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
           "rot": {"base": base, "dims": dims or rot_dim}}
    if q_rank:
        out["q_rank"] = q_rank
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale, identity=0, groups=None, shared=0):
    router = {"experts": experts, "top": top, "scale": scale}
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mix, mlp):
    return {"type": "latent_attention", "mixer": mix, "mlp": mlp}


def config(vocab, width, layers, streams=None, eps=1e-5):
    out = {"architecture": "Pukerax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        out["streams"] = streams
    return out


# Odd head sizes, value heads smaller and larger than key heads, a query latent smaller and larger
# than the width, a layer without a feed-forward, routers with and without groups, identity
# experts and a shared expert, groups that close experts the choice would otherwise take (as many
# chosen experts as one kept group has), groups of one expert each, several kept groups, top 1.
SMALL_A = config(211, 64, [
    layer(mixer(3, 8, 4, 12, 20, 24, 0.35, base=50000.0), dense(96)),
    layer(mixer(2, 12, 6, 6, 28, 80, 0.3), moe(40, 6, 2, 2.2, identity=2, groups=(4, 1), shared=24)),
    layer(mixer(4, 6, 8, 10, 12, 16, 0.4, base=300.0), None),
    layer(mixer(1, 20, 4, 28, 24, 0, 0.25), moe(56, 5, 3, 1.0)),
    layer(mixer(3, 8, 4, 12, 20, 24, 0.35), moe(24, 9, 1, 0.7, identity=3, groups=(12, 5))),
], streams=4)
# Sizes that the tensor-core kernels take; two streams; groups of which one is kept.
SMALL_B = config(257, 128, [
    layer(mixer(4, 32, 32, 32, 64, 80, 0.125, base=500000.0), dense(256)),
    layer(mixer(2, 16, 32, 64, 64, 48, 0.2), moe(64, 7, 2, 2.0, identity=3, groups=(2, 1), shared=128)),
    layer(mixer(4, 32, 16, 16, 112, 64, 0.14), moe(128, 4, 2, 1.5, shared=64)),
], streams=2, eps=1e-6)
# One stream with hyper-connection tensors (a read weight, a 1 x 1 mix and an output weight all the same).
ONE_STREAM = config(97, 48, [
    layer(mixer(2, 8, 8, 16, 24, 32, 0.3), moe(32, 4, 2, 1.0, identity=1)),
    layer(mixer(2, 8, 8, 16, 24, 32, 0.3), dense(64)),
], streams=1)
# No streams at all: plain residual sums.
PLAIN_SUMS = config(97, 48, [
    layer(mixer(2, 8, 8, 16, 24, 32, 0.3), moe(32, 6, 2, 1.8, identity=2, groups=(2, 1), shared=16)),
    layer(mixer(3, 12, 4, 8, 40, 0, 0.28), None),
    layer(mixer(2, 8, 8, 16, 24, 32, 0.3, dims=4), dense(64)),
])
# A latent wider than 256 channels and many streams.
WIDE_LATENT = config(97, 48, [layer(mixer(2, 8, 16, 8, 288, 24, 0.3), dense(64)),
                              layer(mixer(3, 8, 16, 8, 288, 24, 0.3), moe(16, 16, 4, 3.0, groups=(4, 2)))], streams=8)
SMALL = {"small_a": (SMALL_A, 4, 31), "small_b": (SMALL_B, 16, 32), "one_stream": (ONE_STREAM, 8, 33),
         "plain_sums": (PLAIN_SUMS, 16, 34), "wide_latent": (WIDE_LATENT, 8, 35)}       # config, page size, seed


def write_model(folder: Path, raw: dict, seed: int, dtype=torch.bfloat16, sharpen: float = 4.0) -> Path:
    """A random model folder whose numbers make faults visible: query, key and value projections
    scaled up (one key's score stands out, so a wrong, missing or extra key shows), gates, read
    and write weights of the streams, mixing matrices and norm weights of a size that matters,
    router logits far enough apart that the choice is no close call, a correction large enough
    to change it."""
    from safetensors.torch import load_file, save_file

    from paged_attention_engine_b200.weights import write_random_model

    write_random_model(folder, raw, seed, dtype)
    path = str(Path(folder) / "model.safetensors")
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(seed + 1000)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith((".mix.q", ".mix.dq", ".mix.uq", ".mix.dkv", ".mix.uk", ".mix.uv", ".mlp.up", ".up")):
            t = t * sharpen
        elif name.endswith(".mix.g"):
            t = t * 40.0
        elif name.endswith(".mlp.router"):
            t = t * 12.0
        elif name.endswith(".mlp.correction"):
            # small shifts that reorder close scores, and a quarter of the experts so far down that
            # a negative choice score must still beat a closed group's
            t = torch.randn(t.shape, generator=gen) * 0.05 - 1.5 * (torch.rand(t.shape, generator=gen) < 0.25)
        elif name.endswith((".dq.norm", ".dkv.norm")):
            t = 1.0 + torch.rand(t.shape, generator=gen) * 1.5
        elif name.endswith((".norm1", ".norm2", "final.norm")):
            t = torch.randn(t.shape, generator=gen) * 0.4
        elif name.endswith(".in"):
            # positive: the streams are much alike, and a read with mixed signs would cancel them
            t = torch.rand(t.shape, generator=gen) + 0.3
        elif name.endswith(".out"):
            t = (torch.rand(t.shape, generator=gen) + 0.3) * (torch.randint(0, 2, t.shape, generator=gen) * 2.0 - 1.0)
        elif name.endswith(".mix") and t.dim() == 2 and ".hc" in name:
            t = torch.eye(t.shape[0]) * 0.7 + torch.randn(t.shape, generator=gen) * 0.25
        elif name == "head":
            t = t * 12.0
        tensors[name] = t.to(tensors[name].dtype)
    save_file(tensors, path)
    return Path(folder)


def read_model(folder: Path):
    from safetensors.torch import load_file

    return json.loads((Path(folder) / "config.json").read_text()), load_file(str(Path(folder) / "model.safetensors"))


def plain_logits(folder: Path, tokens) -> torch.Tensor:
    raw, tensors = read_model(folder)
    return plain.forward(raw, tensors, list(tokens)).float()


# A router's choice is a step function of its input: where two experts' choice scores are closer
# than rounding can move them, the engine may choose otherwise than the plain model, and rightly
# so. The tests' prompts avoid such tokens: a token whose choice is closer than this (in any
# routed layer) is drawn again.
CLEAR_CHOICE = 0.015


def clear_requests(folder: Path, lengths, seed: int, margin: float = CLEAR_CHOICE):
    """(requests, logits): prompts of the given lengths for which no router's choice is a close
    call, drawn from `seed`, and the plain model's logits for them."""
    raw, tensors = read_model(folder)
    gen = torch.Generator().manual_seed(seed)
    requests, logits = {}, {}
    for i, n in enumerate(lengths):
        tokens = torch.randint(0, raw["vocab"], (n,), generator=gen).tolist()
        for _ in range(40 + n):
            margins = []
            out = plain.forward(raw, tensors, tokens, margins=margins)
            close = torch.stack(margins).min(dim=0).values < margin if margins else torch.zeros(n, dtype=torch.bool)
            if not bool(close.any()):
                break
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
