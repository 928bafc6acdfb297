"""Grouped-query attention with normed, partly rotated heads, a sink and an output gate.

q, k, v and the gate are one fused projection without bias (float32 out). Every query and key
head is RMS-normed over its channels with a weight that all heads share (or all query heads of a
token are normed at once, and all its key heads, with weights as long as those projections), then
a leading span of the head is rotated (pairs (i, i + span/2)) by the layer's position encoding;
keys and values go to their pages. Query i sees key j <= i with i - j < window (no window: every
earlier key). The softmax's denominator may hold one more term exp(s_h) without a value (a sink:
s_h = 0, or a learned number per head), and the concatenated heads may be multiplied by
sigmoid(W_g h), a gate per channel or one per head, before the output projection, which takes the
residual in its epilogue. Value heads may have another size than key heads.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, CacheNeed, Part, TensorSpec


@MIXERS.register("gated_window_attention")
class GatedWindowAttention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, scale, window (0: all
    keys), qk_norm_eps (None: q and k are not normed), qk_norm ("head", the default: per head with a
    weight [head_dim] that the heads share; "whole": over the whole projection with weights [heads *
    head_dim] and [kv_heads * head_dim]), unit_sink (bool), learned_sink (bool: a tensor `sink`
    [heads]), output_gate (False, True or "channel": g [heads * value_dim, hidden]; "head": g [heads,
    hidden]), position_encoding (a dict with its `kind` and `dims`, or None).
    tensors: q, k, v, o (and g) matrices; q.norm, k.norm; sink."""

    @classmethod
    def _sizes(cls, spec: PartSpec):
        p = spec.params
        heads, kv_heads, d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        return heads, kv_heads, d, int(p.get("value_dim") or d)

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        p = spec.params
        hidden = int(p["hidden_size"])
        heads, kv_heads, d, dv = cls._sizes(spec)
        rows = {"q": heads * d, "k": kv_heads * d, "v": kv_heads * dv}
        if p.get("output_gate"):
            rows["g"] = heads if p["output_gate"] == "head" else heads * dv
        out = [TensorSpec(spec.tensor_name(n), (r, hidden), "matrix") for n, r in rows.items()]
        if p.get("qk_norm_eps") is not None:
            whole = p.get("qk_norm", "head") == "whole"
            out += [TensorSpec(spec.tensor_name("q.norm"), (heads * d if whole else d,), "scale"),
                    TensorSpec(spec.tensor_name("k.norm"), (kv_heads * d if whole else d,), "scale")]
        if p.get("learned_sink"):
            out.append(TensorSpec(spec.tensor_name("sink"), (heads,), "vector"))
        out.append(TensorSpec(spec.tensor_name("o"), (hidden, heads * dv), "matrix"))
        return out

    @classmethod
    def sub_parts(cls, spec: PartSpec) -> list[tuple[str, PartSpec]]:
        enc = spec.params.get("position_encoding")
        if enc is None:
            return []
        return [("position_encoding", PartSpec(enc["kind"], {k: v for k, v in enc.items() if k != "kind"}, spec.prefix))]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, kv_heads, d, dv = cls._sizes(spec)
        return CacheNeed(kv_heads, d, int(spec.params.get("window") or 0), 0 if dv == d else dv)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim = self._sizes(spec)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"gated_window_attention: {self.num_heads} heads over {self.num_kv_heads} kv heads")
        self.scale = float(p["scale"])
        self.window = int(p.get("window") or 0)
        self.norm_eps = p.get("qk_norm_eps")
        self.gated = bool(p.get("output_gate"))
        self.gate_group = self.value_dim if p.get("output_gate") == "head" else 1
        if p.get("qk_norm", "head") not in ("head", "whole"):
            raise ValueError(f"gated_window_attention: qk_norm '{p.get('qk_norm')}' (head, whole)")
        self.whole_norm = p.get("qk_norm", "head") == "whole"
        names = ("q", "k", "v") + (("g",) if self.gated else ())
        # One projection for q | k | v | g: the columns of its output in that order.
        self.in_weight = torch.cat([tensors.pop(spec.tensor_name(n)) for n in names], dim=0).contiguous()
        self.q_norm = self.k_norm = None
        if self.norm_eps is not None:
            self.q_norm, self.k_norm = tensors.pop(spec.tensor_name("q.norm")), tensors.pop(spec.tensor_name("k.norm"))
        # A sink whose logit is 0: one more term exp(0) in every head's denominator.
        self.sink = torch.zeros(self.num_heads, dtype=torch.float32, device=runtime.device) if p.get("unit_sink") else None
        if p.get("learned_sink"):
            self.sink = tensors.pop(spec.tensor_name("sink"))
        self.o_weight = tensors.pop(spec.tensor_name("o"))
        built = self.build_sub_parts(tensors)
        self.position_encoding = built[0] if built else None
        self.rot_dims = self.position_encoding.dims if self.position_encoding is not None else 0
        if self.rot_dims > self.head_dim:
            raise ValueError(f"gated_window_attention: {self.rot_dims} rotated channels in heads of {self.head_dim}")

    def forward(self, ctx, x, residual, cache):
        ops = self.ops
        group = ctx.groups[cache.group]
        h, g, d, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        proj = ops.linear(x, self.in_weight, None, None, out_dtype=torch.float32)
        table = self.position_encoding.table(ctx) if self.position_encoding is not None else None
        q = ops.head_prep(
            proj, q_off=0, k_off=h * d, v_off=(h + g) * d, heads=h, kv_heads=g, q_dim=d, k_dim=d, value_dim=dv,
            q_norm=self.q_norm, k_norm=self.k_norm, q_span=d, k_span=d, eps=float(self.norm_eps or 0.0),
            table=table, interleaved=False, q_rot0=0, k_rot0=0, slots=group.slots if cache.writes else None,
            keys=cache.keys, values=cache.values, page_size=cache.page_size, out_dtype=self.runtime.dtype, whole=self.whole_norm)
        out = ops.paged_attention_scored(
            q, cache.keys, cache.values, group.block_table, ctx.q_start, ctx.q_pos0, ctx.kv_len, h, g, d, dv,
            cache.page_size, ctx.max_q_len, self.scale, sink=self.sink, window=self.window,
            max_kv_len=ctx.max_kv_len, num_single=ctx.num_single)
        if self.gated:
            out = ops.sigmoid_gate(out, proj, (h + g) * d + g * dv, group=self.gate_group)
        # without a residual (a caller that sums by itself) the output leaves in float32
        return ops.linear(out, self.o_weight, None, residual, out_dtype=residual.dtype if residual is not None else torch.float32)
