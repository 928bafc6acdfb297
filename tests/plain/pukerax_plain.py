"""A plain, slow Pukerax: one function per mechanism, written from the design's equations.

Everything runs on the CPU in float64 over one whole sequence at a time. It shares no code
with the engine: it reads a dictionary of tensors by their checkpoint names and the
config.json dictionary. Latent attention is computed in its expanded form (every head's keys
and values are made from the latent), the routed feed-forward token by token.

Notation: T tokens, W model width, S streams, H heads, d unrotated and r rotated query/key
channels per head, dv value channels, c the key/value latent, cq the query latent, E routed
experts, I identity experts, positions p = 0..T-1.
"""

from __future__ import annotations

import math

import torch

F = torch.float64

# A function applied to every sublayer's input (the normed read of the stream), or None. Tests set
# it to a rounding to bfloat16 to learn how far one rounding of an input moves a model's logits.
narrow = None


def _f(t):
    return t.to(F)


def _input(h):
    return narrow(h) if narrow is not None else h


def rms_norm(x, weight, eps, offset=0.0):
    """x / sqrt(mean(x^2) + eps) * (offset + w) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (offset + _f(weight))


def rotate_interleaved(x, positions, dims, base):
    """Turns the pairs (2i, 2i + 1), i < dims / 2, of the last axis of x [T, ..., n] by the angle
    p * base^(-2i / dims); channels from `dims` on pass."""
    out = x.clone()
    where = torch.tensor(positions, dtype=F).view(-1, *([1] * (x.dim() - 2)))
    for i in range(dims // 2):
        a = where * float(base) ** (-2.0 * i / dims)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * torch.cos(a) - v * torch.sin(a)
        out[..., 2 * i + 1] = v * torch.cos(a) + u * torch.sin(a)
    return out


def causal_softmax_attention(q, k, v, scale):
    """q, k [T, H, n], v [T, H, dv]: query i over keys j <= i, ordinary softmax."""
    T = q.shape[0]
    out = torch.zeros(T, q.shape[1], v.shape[2], dtype=F)
    for i in range(T):
        scores = torch.einsum("hn,jhn->hj", q[i], k[: i + 1]) * scale
        out[i] = torch.einsum("hj,jhv->hv", torch.softmax(scores, dim=-1), v[: i + 1])
    return out


def latent_attention(h, tensors, prefix, m, eps, positions):
    """h [T, W] -> [T, W]. The query goes through a normed latent when the mixer has `q_rank`."""
    get = lambda name: _f(tensors[f"{prefix}.{name}"])
    H, d, r, dv, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    if m.get("q_rank"):
        q = rms_norm(h @ get("dq").T, tensors[f"{prefix}.dq.norm"], eps) @ get("uq").T
    else:
        q = h @ get("q").T
    q = q.view(T, H, d + r)
    down = h @ get("dkv").T
    latent = rms_norm(down[:, :c], tensors[f"{prefix}.dkv.norm"], eps)
    shared = rotate_interleaved(down[:, c:], positions, m["rot"]["dims"], m["rot"]["base"])        # [T, r]
    q_rot = rotate_interleaved(q[:, :, d:], positions, m["rot"]["dims"], m["rot"]["base"])
    keys = torch.cat([(latent @ get("uk").T).view(T, H, d), shared[:, None, :].expand(T, H, r)], dim=-1)
    values = (latent @ get("uv").T).view(T, H, dv)
    out = causal_softmax_attention(torch.cat([q[:, :, :d], q_rot], dim=-1), keys, values, m["scale"])
    if f"{prefix}.g" in tensors:
        out = out * torch.sigmoid(h @ get("g").T)[:, :, None]
    return out.reshape(T, H * dv) @ get("o").T


def squared_relu_mlp(h, up, down):
    z = torch.relu(h @ _f(up).T)
    return (z * z) @ _f(down).T


def identity_expert(h):
    """An expert without tensors: its output is its input."""
    return h


def _gap(values, k):
    """Per row, how far the k-th largest value is from the next one (infinite when there is none)."""
    if k >= values.shape[-1]:
        return torch.full(values.shape[:-1], math.inf, dtype=F)
    top = values.topk(k + 1, dim=-1).values
    return top[..., k - 1] - top[..., k]


def route(h, router, correction, r, margins=None):
    """Per token the chosen experts and their weights: ([T, top] indices, [T, top] weights).
    `margins`, a list, receives per token how close the choice was: the smaller of the gaps
    between the last kept and the first dropped group, and the last chosen and the first
    unchosen expert."""
    total = router.shape[0]
    scores = torch.softmax(h @ _f(router).T, dim=-1)                    # [T, E + I]
    choice = scores + _f(correction)
    groups = r.get("groups")
    margin = torch.full((h.shape[0],), math.inf, dtype=F)
    if groups:
        size = total // groups["count"]
        best = choice.view(-1, groups["count"], size).max(dim=-1).values
        margin = _gap(best, groups["keep"])
        kept = best.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(size, dim=1), -math.inf)
    chosen = choice.topk(r["top"], dim=-1).indices
    if margins is not None:
        margins.append(torch.minimum(margin, _gap(choice, r["top"])))
    weights = scores.gather(1, chosen)
    weights = weights / (weights.sum(dim=-1, keepdim=True) + 1e-20) * r["scale"]
    return chosen, weights


def routed_feed_forward(h, tensors, prefix, mlp, margins=None):
    r = mlp["router"]
    identity = int(r.get("identity") or 0)
    real = r["experts"]
    correction = tensors.get(f"{prefix}.correction")
    if correction is None:
        correction = torch.zeros(real + identity)
    chosen, weights = route(h, tensors[f"{prefix}.router"], correction, r, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            if e >= real:
                out[t] += w * identity_expert(h[t])
            else:
                out[t] += w * squared_relu_mlp(h[t : t + 1], tensors[f"{prefix}.e{e}.up"], tensors[f"{prefix}.e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + squared_relu_mlp(h, tensors[f"{prefix}.shared.up"], tensors[f"{prefix}.shared.down"])
    return out


def feed_forward(h, tensors, prefix, mlp, margins=None):
    if mlp["kind"] == "dense":
        return squared_relu_mlp(h, tensors[f"{prefix}.up"], tensors[f"{prefix}.down"])
    return routed_feed_forward(h, tensors, prefix, mlp, margins)


def connect(streams, y, tensors, prefix):
    """streams [S, T, W], y [T, W]: new stream t = sum_s mix[s, t] old s + out[t] y."""
    mix, out = _f(tensors[f"{prefix}.mix"]), _f(tensors[f"{prefix}.out"])
    return torch.einsum("st,snw->tnw", mix, streams) + out[:, None, None] * y[None]


def forward(raw, tensors, tokens, layer_outputs=None, margins=None):
    """float64 logits [T, vocab] of one sequence; `layer_outputs`, a list, receives the residual
    stream (the sum of the streams) after every layer, `margins`, a list, per routed layer how
    close every token's choice of experts was."""
    eps = raw["norm"]["eps"]
    positions = list(range(len(tokens)))
    x = _f(tensors["embed"])[torch.tensor(tokens, dtype=torch.long)]
    S = raw.get("streams")
    streams = x[None].repeat(S, 1, 1) if S else None
    for i, layer in enumerate(raw["layers"]):
        branches = [(1, lambda h: latent_attention(h, tensors, f"l{i}.mix", layer["mixer"], eps, positions))]
        if layer.get("mlp"):
            branches.append((2, lambda h: feed_forward(h, tensors, f"l{i}.mlp", layer["mlp"], margins)))
        for q, branch in branches:
            if S:
                u = torch.einsum("s,snw->nw", _f(tensors[f"l{i}.hc{q}.in"]), streams)
                streams = connect(streams, branch(_input(rms_norm(u, tensors[f"l{i}.norm{q}"], eps, 1.0))), tensors, f"l{i}.hc{q}")
            else:
                x = x + branch(_input(rms_norm(x, tensors[f"l{i}.norm{q}"], eps, 1.0)))
        if layer_outputs is not None:
            layer_outputs.append(streams.sum(dim=0) if S else x)
    if S:
        x = streams.sum(dim=0)
    return rms_norm(x, tensors["final.norm"], eps, 1.0) @ _f(tensors["head"]).T
