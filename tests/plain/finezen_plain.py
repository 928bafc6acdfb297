"""A plain, slow Finezen: one function per mechanism, written from the design's equations.

Everything runs on the CPU in float64 over one whole sequence at a time. It shares no code with
the engine: it reads a dictionary of tensors by their checkpoint names and the config.json
dictionary. Latent attention is computed in its expanded form (every head's keys and values are
made from the latent), the routed feed-forward token by token.

Notation: T tokens, W model width, H query heads, G key/value heads, d query/key channels and dv
value channels per head, c the key/value latent, cq the query latent, E experts, positions
p = 0..T-1, m the residual multiplier.
"""

from __future__ import annotations

import math

import torch

F = torch.float64

# A function applied to every sublayer's input (the normed stream), or None. Tests set it to a
# rounding to bfloat16 to learn how far one rounding of an input moves a model's logits.
narrow = None


def _f(t):
    return t.to(F)


def _input(h):
    return narrow(h) if narrow is not None else h


def dynamic_tanh(x, tensors, name):
    """tanh(alpha x) * w + b: a norm without statistics. alpha is a scalar, w and b vectors."""
    return torch.tanh(_f(tensors[f"{name}.alpha"]) * x) * _f(tensors[name]) + _f(tensors[f"{name}.b"])


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * _f(weight)


def yarn_frequencies(dims, base, scaling):
    """(frequencies [dims / 2], amplitude). Without scaling f_i = base^(-2i / dims) and amplitude 1.
    With it, pair i is slowed down by `factor` to the degree ramp_i, a linear ramp between the pair
    that turns `fast` times within `original` positions and the one that turns `slow` times."""
    freqs = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return freqs, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, rot):
    """Turns the pairs (i, i + dims / 2), i < dims / 2, of the last axis of x [T, heads, n] by the
    angle p * f_i; channels from `dims` on pass."""
    dims = rot["dims"]
    freqs, amplitude = yarn_frequencies(dims, rot["base"], rot.get("scaling"))
    out = x.clone()
    where = torch.tensor(positions, dtype=F).view(-1, 1)
    for i in range(dims // 2):
        a = where * freqs[i]
        cos, sin = torch.cos(a) * amplitude, torch.sin(a) * amplitude
        u, v = x[..., i], x[..., i + dims // 2]
        out[..., i] = u * cos - v * sin
        out[..., i + dims // 2] = v * cos + u * sin
    return out


def windowed_softmax_attention(q, k, v, scale, window, sink=None):
    """q [T, H, n], k [T, G, n], v [T, G, dv]; query head h reads key/value head h // (H / G); query i
    sees keys j with 0 <= i - j < window (window 0 or None: every j <= i). `sink` [H]: one more term
    exp(sink_h) in the denominator, with no value."""
    T, H = q.shape[0], q.shape[1]
    per = H // k.shape[1]
    k, v = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)      # every query head's own copy
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for i in range(T):
        first = max(0, i - window + 1) if window else 0
        scores = torch.einsum("hn,jhn->hj", q[i], k[first: i + 1]) * scale
        top = scores.max(dim=1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[:, None])
        e = torch.exp(scores - top)
        denominator = e.sum(dim=1, keepdim=True)
        if sink is not None:
            denominator = denominator + torch.exp(sink[:, None] - top)
        out[i] = torch.einsum("hj,jhv->hv", e / denominator, v[first: i + 1])
    return out


def head_gates(h, gate_weight):
    """sigmoid(W_g h): one number per token and head, [T, H, 1]."""
    return torch.sigmoid(h @ _f(gate_weight).T)[:, :, None]


def attention(h, tensors, prefix, m, eps, positions):
    """Grouped-query attention: q and k normed over the whole projection, partly rotated, a window,
    a learned sink, a gate per head. h [T, W] -> [T, W]."""
    get = lambda name: _f(tensors[f"{prefix}.{name}"])
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ get("q").T, tensors[f"{prefix}.q.norm"], eps).view(T, H, d)
    k = rms_norm(h @ get("k").T, tensors[f"{prefix}.k.norm"], eps).view(T, G, d)
    v = (h @ get("v").T).view(T, G, dv)
    if m.get("rot"):
        q, k = rotate_half(q, positions, m["rot"]), rotate_half(k, positions, m["rot"])
    window = (m.get("mask") or {}).get("size") or 0
    out = windowed_softmax_attention(q, k, v, m["scale"], window, sink=get("sink"))
    out = out * head_gates(h, tensors[f"{prefix}.g"])
    return out.reshape(T, H * dv) @ get("o").T


def latent_attention(h, tensors, prefix, m, eps):
    """Attention without positions whose keys and values are expansions of one normed latent per
    token; the queries go through a normed latent of their own. h [T, W] -> [T, W]."""
    get = lambda name: _f(tensors[f"{prefix}.{name}"])
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (rms_norm(h @ get("dq").T, tensors[f"{prefix}.dq.norm"], eps) @ get("uq").T).view(T, H, d)
    latent = rms_norm(h @ get("dkv").T, tensors[f"{prefix}.dkv.norm"], eps)
    k = (latent @ get("uk").T).view(T, H, d)
    v = (latent @ get("uv").T).view(T, H, dv)
    window = (m.get("mask") or {}).get("size") or 0
    out = windowed_softmax_attention(q, k, v, m["scale"], window)
    out = out * head_gates(h, tensors[f"{prefix}.g"])
    return out.reshape(T, H * dv) @ get("o").T


def gated_expert(h, tensors, prefix):
    """W_down (silu(W_gate h) * (W_up h))."""
    gate = h @ _f(tensors[f"{prefix}.gate"]).T
    return (gate * torch.sigmoid(gate) * (h @ _f(tensors[f"{prefix}.up"]).T)) @ _f(tensors[f"{prefix}.down"]).T


def route(h, router, top, margins=None):
    """Per token the `top` experts with the largest sigmoid(W_router h) and those scores, which are
    the weights as they are. `margins`, a list, receives per token how far the last chosen expert's
    logit is from that of the first one not chosen."""
    logits = h @ _f(router).T
    best = logits.topk(min(top + 1, logits.shape[1]), dim=-1)
    if margins is not None:
        margins.append(best.values[:, top - 1] - best.values[:, top] if logits.shape[1] > top
                       else torch.full((h.shape[0],), math.inf, dtype=F))
    return best.indices[:, :top], torch.sigmoid(best.values[:, :top])


def mixture(h, tensors, prefix, mlp, margins=None):
    """sum over the chosen experts of expert(w h), the weight on the expert's INPUT, plus the shared
    expert times sigmoid(W_sg h)."""
    chosen, weights = route(h, tensors[f"{prefix}.router"], mlp["router"]["top"], margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            out[t] += gated_expert(w * h[t: t + 1], tensors, f"{prefix}.e{e}")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, tensors, f"{prefix}.shared") * torch.sigmoid(h @ _f(tensors[f"{prefix}.shared.sg"]).T)
    return out


def layer_runs(raw):
    """[(layer index, whether the embedding's output is added before it)] in running order: the
    layers start .. stop - 1 run `times` times in a row, each pass but the first after the
    embedding's output has been added once more."""
    n = len(raw["layers"])
    loop = raw.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(start)]
    for p in range(times):
        runs += [(i, p > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def forward(raw, tensors, tokens, margins=None, streams=None):
    """Logits [T, vocab] of one sequence. `streams`, a list, receives the residual stream after
    every layer run."""
    positions = list(range(len(tokens)))
    eps, m = raw["norm"]["eps"], raw["residual_mult"]
    embedded = _f(tensors["embed"])[torch.tensor(tokens)] * raw["embedding"]["scale"]
    x = embedded.clone()
    for i, add in layer_runs(raw):
        layer, p = raw["layers"][i], f"l{i}"
        if add:
            x = x + embedded
        h = _input(dynamic_tanh(x, tensors, f"{p}.norm1"))
        if layer["type"] == "attention":
            y = attention(h, tensors, f"{p}.mix", layer["mixer"], eps, positions)
        else:
            y = latent_attention(h, tensors, f"{p}.mix", layer["mixer"], eps)
        x = x + m * dynamic_tanh(y, tensors, f"{p}.norm1b")
        if layer.get("mlp"):
            h = _input(dynamic_tanh(x, tensors, f"{p}.norm2"))
            x = x + m * dynamic_tanh(mixture(h, tensors, f"{p}.mlp", layer["mlp"], margins), tensors, f"{p}.norm2b")
        if streams is not None:
            streams.append(x.clone())
    return dynamic_tanh(x, tensors, "final.norm") @ _f(tensors["head"]).T
