"""Latent attention: keys and values of all heads are expansions of ONE small latent per token.

Per token the layer projects h down to kv_rank + rot_dim numbers: the first kv_rank, RMS-normed
with a weight, are the latent c; the last rot_dim, rotated (interleaved pairs), are a key part
that all heads share. Head n's key is [W_uk[n] c | shared part], its value W_uv[n] c; its query
is [dim unrotated | rot_dim rotated] channels of W_q h. Only c and the shared part are cached:
one key row of kv_rank + rot_dim channels per token, which is key and value at once.

The expansions are never made. With A_n = W_uk[n]^T q_unrotated[n] (kv_rank numbers),
q[n] . k[n] = A_n . c + q_rotated[n] . shared, so every head attends the same latent rows as
one key/value head whose key is [c | shared] and whose value is c; the value expansion W_uv[n]
is applied to the attention's output over the latent. A layer may read the latent of an
earlier layer (through the schedule's `cache_from`): it has no down projection and writes nothing.

With `rot_dim` 0 and no position encoding there is no shared part and nothing turns: the key row
is the latent alone. With a `window` a query sees that many keys, itself included.

Two options. The queries may go through a latent of their own: c_q = RMSnorm(W_dq h) with a
weight, q = W_uq c_q (`q_rank`). And every head's output may be multiplied by one sigmoid of a
projection of h (`head_gate`, a gate per head, not per channel) before the output projection.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, CacheNeed, Part, TensorSpec


@MIXERS.register("latent_attention")
class LatentAttention(Part):
    """params: hidden_size, num_heads, head_dim (unrotated channels), rot_dim, value_dim, kv_rank,
    scale, norm_eps, own_latent (False: the layer reads another entry's cache), window (0: causal),
    position_encoding (a dict with its `kind`; its `dims` are at most rot_dim: the leading channels
    of the rotated part turn), q_rank (0 or absent: no query latent), head_gate (False or absent: none).
    tensors: q [heads * (head_dim + rot_dim), hidden], or with a query latent dq [q_rank, hidden],
    dq.norm [q_rank] and uq [heads * (head_dim + rot_dim), q_rank]; g [heads, hidden] with a gate; dkv [kv_rank + rot_dim, hidden] and dkv.norm
    [kv_rank] with a latent of its own; uk [heads * head_dim, kv_rank]; uv [heads * value_dim, kv_rank];
    o [hidden, heads * value_dim]."""

    @classmethod
    def _sizes(cls, spec: PartSpec):
        p = spec.params
        return int(p["num_heads"]), int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"]), int(p["kv_rank"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden = int(spec.params["hidden_size"])
        heads, d, r, dv, c = cls._sizes(spec)
        name = spec.tensor_name
        q_rank = int(spec.params.get("q_rank") or 0)
        if q_rank:
            out = [TensorSpec(name("dq"), (q_rank, hidden), "matrix"), TensorSpec(name("dq.norm"), (q_rank,), "scale"),
                   TensorSpec(name("uq"), (heads * (d + r), q_rank), "matrix")]
        else:
            out = [TensorSpec(name("q"), (heads * (d + r), hidden), "matrix")]
        if spec.params.get("head_gate"):
            out.append(TensorSpec(name("g"), (heads, hidden), "matrix"))
        if spec.params.get("own_latent", True):
            out += [TensorSpec(name("dkv"), (c + r, hidden), "matrix"), TensorSpec(name("dkv.norm"), (c,), "scale")]
        return out + [TensorSpec(name("uk"), (heads * d, c), "matrix"), TensorSpec(name("uv"), (heads * dv, c), "matrix"),
                      TensorSpec(name("o"), (hidden, heads * dv), "matrix")]

    @classmethod
    def sub_parts(cls, spec: PartSpec) -> list[tuple[str, PartSpec]]:
        enc = spec.params.get("position_encoding")
        if enc is None:
            return []
        return [("position_encoding", PartSpec(enc["kind"], {k: v for k, v in enc.items() if k != "kind"}, spec.prefix))]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, _, r, _, c = cls._sizes(spec)
        return CacheNeed(1, c + r, int(spec.params.get("window") or 0), c, values_in_keys=True)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank = self._sizes(spec)
        heads, d, r, dv, c = self._sizes(spec)
        self.scale = float(p["scale"])
        self.window = int(p.get("window") or 0)
        self.norm_eps = float(p["norm_eps"])
        self.own_latent = bool(p.get("own_latent", True))
        name = spec.tensor_name
        self.q_rank = int(p.get("q_rank") or 0)
        self.head_gate = bool(p.get("head_gate"))
        # One projection for q (or the query latent) | gates | down: the columns of its output in that order.
        rows = [tensors.pop(name("dq" if self.q_rank else "q"))]
        self.q_cols = int(rows[0].shape[0])
        if self.head_gate:
            rows.append(tensors.pop(name("g")))
        self.latent_norm = self.query_norm = self.uq_weight = None
        if self.q_rank:
            self.query_norm, self.uq_weight = tensors.pop(name("dq.norm")), tensors.pop(name("uq"))
        if self.own_latent:
            rows.append(tensors.pop(name("dkv")))
            self.latent_norm = tensors.pop(name("dkv.norm"))
        self.in_weight = torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0]
        # [heads, kv_rank, head_dim]: head n's key expansion transposed, so that A_n is a product like any other.
        self.uk_t = tensors.pop(name("uk")).view(heads, d, c).transpose(1, 2).contiguous()
        self.uv = tensors.pop(name("uv")).view(heads, dv, c).contiguous()
        self.o_weight = tensors.pop(name("o"))
        built = self.build_sub_parts(tensors)
        self.position_encoding = built[0] if built else None
        if self.position_encoding is not None and self.position_encoding.dims > r:
            raise ValueError(f"latent_attention: {self.position_encoding.dims} rotated channels, rot_dim is {r}")

    def forward(self, ctx, x, residual, cache):
        ops = self.ops
        group = ctx.groups[cache.group]
        heads, d, r, dv, c = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank
        if cache.writes != self.own_latent:
            raise ValueError("latent_attention: a layer with a latent of its own writes its cache, one without reads another's")
        proj = ops.linear(x, self.in_weight, None, None, out_dtype=torch.float32)
        table = self.position_encoding.table(ctx) if self.position_encoding is not None else None
        gate_off = self.q_cols
        k_off = gate_off + (heads if self.head_gate else 0)
        prep = dict(q_dim=d + r, k_dim=c + r, value_dim=0, q_norm=None, k_norm=self.latent_norm, q_span=0, k_span=c,
                    eps=self.norm_eps, table=table, interleaved=True, q_rot0=d, k_rot0=c, keys=cache.keys, values=None,
                    page_size=cache.page_size, out_dtype=self.runtime.dtype)
        slots = group.slots if self.own_latent else None
        if self.q_rank:
            # the token's latent row into its page; then the queries from their own normed latent
            proj = ops.materialized(proj)
            if self.own_latent:
                ops.head_prep(proj, q_off=0, k_off=k_off, v_off=0, heads=0, kv_heads=1, slots=slots, **prep)
            query_latent = ops.rms_norm_columns(proj, 0, self.q_rank, self.query_norm, self.norm_eps, self.runtime.dtype)
            if table is None:
                # no channel turns: the queries leave their product in the engine's dtype
                q = ops.linear(query_latent, self.uq_weight, None, None, out_dtype=self.runtime.dtype)
            else:
                queries = ops.linear(query_latent, self.uq_weight, None, None, out_dtype=torch.float32)
                q = ops.head_prep(queries, q_off=0, k_off=0, v_off=0, heads=heads, kv_heads=0, slots=None, **prep)
        else:
            # queries [tokens, heads, d + r] with their rotated channels turned; the token's latent row into its page
            q = ops.head_prep(proj, q_off=0, k_off=k_off, v_off=0, heads=heads, kv_heads=1 if self.own_latent else 0,
                              slots=slots, **prep)
        # [A_n | rotated channels] per head: the query against the latent rows
        q = ops.linear_heads(q, self.uk_t, heads, in_stride=d + r, tail=r)
        over_latent = ops.paged_attention_scored(
            q, cache.keys, cache.keys, group.block_table, ctx.q_start, ctx.q_pos0, ctx.kv_len, heads, 1, c + r, c,
            cache.page_size, ctx.max_q_len, self.scale, window=self.window, max_kv_len=ctx.max_kv_len,
            num_single=ctx.num_single)
        out = ops.linear_heads(over_latent, self.uv, heads, in_stride=c, tail=0)
        if self.head_gate:
            out = ops.sigmoid_gate(out, proj, gate_off, group=dv)
        # without a residual (a caller that sums by itself) the output leaves in float32
        return ops.linear(out, self.o_weight, None, residual, out_dtype=residual.dtype if residual is not None else torch.float32)
