"""Feed-forwards. SwiGLU as in the reference (engine/model.py:317-320):
down(silu(gate(x)) * up(x)), no biases; gate and up are one product here, and the
down projection takes the residual in its epilogue."""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import FEED_FORWARDS, Part, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(Part):
    """params: hidden_size, intermediate_size. tensors: gate_proj/up_proj/down_proj .weight."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [
            TensorSpec(spec.tensor_name("gate_proj.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("up_proj.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("down_proj.weight"), (hidden, inter), "matrix"),
        ]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.intermediate_size = int(spec.params["intermediate_size"])
        gate = tensors.pop(spec.tensor_name("gate_proj.weight"))
        up = tensors.pop(spec.tensor_name("up_proj.weight"))
        # Gate and up are one product. Where the kernels offer it, their rows alternate in
        # blocks (16 gate rows, their 16 up rows, ...) so that SiLU x up runs inside the
        # product; else rows [0, I) are the gate and rows [I, 2I) the up projection.
        interleave = getattr(self.ops, "interleave_gate_up", None)
        self.gate_up_weight = interleave(gate, up) if interleave is not None else None
        self.interleaved = self.gate_up_weight is not None
        if not self.interleaved:
            self.gate_up_weight = torch.cat([gate, up], dim=0).contiguous()
        self.down_weight = tensors.pop(spec.tensor_name("down_proj.weight"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        if self.interleaved:
            hidden = ops.linear_swiglu(x, self.gate_up_weight)
        else:
            hidden = ops.silu_mul(ops.linear(x, self.gate_up_weight, None))
        return ops.linear(hidden, self.down_weight, None, residual)


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(Part):
    """down(act(up(x))) without biases. params: hidden_size, intermediate_size, activation
    ("gelu_erf": 0.5 z (1 + erf(z / sqrt 2)), "gelu_tanh", or "relu2": max(z, 0)^2). tensors:
    up.weight, down.weight. The residual may be float32 while x is in the engine's dtype: the down
    projection adds it in its epilogue and leaves the residual's dtype; without a residual (a
    caller that sums by itself) the output leaves in float32."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [
            TensorSpec(spec.tensor_name("up.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("down.weight"), (hidden, inter), "matrix"),
        ]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.activation = str(spec.params.get("activation", "gelu_erf"))
        self.up_weight = tensors.pop(spec.tensor_name("up.weight"))
        self.down_weight = tensors.pop(spec.tensor_name("down.weight"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        hidden = ops.linear(x, self.up_weight, None, activation=self.activation)     # the activation in the product's epilogue
        return ops.linear(hidden, self.down_weight, None, residual, out_dtype=residual.dtype if residual is not None else torch.float32)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(Part):
    """down(g * sigmoid(alpha * g) * (u + 1)) with g = min(gate(x), limit) and u = clamp(up(x),
    -limit, limit); all three projections have biases. params: hidden_size, intermediate_size,
    limit, alpha. tensors: gate, up [intermediate, hidden], down [hidden, intermediate] and
    gate.b, up.b, down.b. Gate and up are one product (float32 out: the clamps and the
    activation see unrounded sums); the down projection adds its bias and the residual in its
    epilogue and leaves the residual's dtype."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        name = spec.tensor_name
        return [TensorSpec(name("gate"), (inter, hidden), "matrix"), TensorSpec(name("gate.b"), (inter,), "vector"),
                TensorSpec(name("up"), (inter, hidden), "matrix"), TensorSpec(name("up.b"), (inter,), "vector"),
                TensorSpec(name("down"), (hidden, inter), "matrix"), TensorSpec(name("down.b"), (hidden,), "vector")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.limit, self.alpha = float(spec.params["limit"]), float(spec.params["alpha"])
        name = spec.tensor_name
        # rows [0, I) are the gate and rows [I, 2I) the up projection
        self.gate_up_weight = torch.cat([tensors.pop(name("gate")), tensors.pop(name("up"))], dim=0).contiguous()
        self.gate_up_bias = torch.cat([tensors.pop(name("gate.b")), tensors.pop(name("up.b"))], dim=0).contiguous()
        self.down_weight, self.down_bias = tensors.pop(name("down")), tensors.pop(name("down.b"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        gate_up = ops.linear(x, self.gate_up_weight, self.gate_up_bias, None, out_dtype=torch.float32)
        hidden = ops.clamped_glu(gate_up, self.limit, self.alpha, self.runtime.dtype)
        return ops.linear(hidden, self.down_weight, self.down_bias, residual, out_dtype=residual.dtype)


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(Part):
    """A mixture of experts without biases, of which each token uses `top`. An expert is
    down_e(act(up_e(x))), or, `gated`, down_e(silu(gate_e(x)) * up_e(x)).

    Router logits z = W_router x in float32; scores s = softmax(z) (or sigmoid) over all experts;
    the choice goes by s + correction (a stored vector) among the experts of the `group_keep` best of
    `group_count` groups of neighbours (a group's score is its largest choice score), the weights
    are the chosen s / (their sum + weight_eps) * weight_scale, or, not normalized, the chosen s *
    weight_scale. A weight multiplies its expert's output, or (`weight_on` "input") its input:
    the sum of expert(w x), which differs because an expert is not linear. The last
    `identity_experts` router outputs are experts without tensors that return x itself. A shared
    expert of its own size runs for every token, `shared_gate`: times sigmoid(W_sg x), one number
    per token.

    params: hidden_size, intermediate_size, activation, gated (bool), num_experts (with tensors),
    identity_experts, top, score ("softmax" or "sigmoid"), choice_correction (bool), group_count (0:
    none), group_keep, normalize_weights (default True), weight_eps, weight_scale, weight_on ("output",
    the default, or "input"), shared_size (0: none), shared_gate (bool).
    tensors: router [num_experts + identity_experts, hidden], correction (the same count),
    e<i>.up [intermediate, hidden] (and e<i>.gate), e<i>.down [hidden, intermediate], shared.up (and
    shared.gate), shared.down, shared.sg [1, hidden].

    Only the chosen (token, expert) pairs are computed: the pairs are sorted by expert into a
    staging matrix whose rows are padded to whole tiles per expert (and multiplied by their weights
    on the way, when the weights are on the input), a grouped product per projection
    walks the tiles with each tile's own expert's weights (the activation in the first one's epilogue, or
    gate and up as one product and SiLU x up after it; float32 out of the second), and one kernel
    adds every token's weighted rows, in the order of its choice, and its input times the weights of
    the experts that return their input, to what the shared expert's plain products left (which
    carries the residual, if there is one). The shared expert's gate is one more row of the router's
    product."""

    @classmethod
    def _sizes(cls, spec: PartSpec):
        p = spec.params
        return (int(p["hidden_size"]), int(p["intermediate_size"]), int(p["num_experts"]), int(p.get("identity_experts") or 0),
                int(p.get("shared_size") or 0))

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, ff, experts, identity, shared = cls._sizes(spec)
        name = spec.tensor_name
        gated = bool(spec.params.get("gated"))
        out = [TensorSpec(name("router"), (experts + identity, hidden), "matrix")]
        if spec.params.get("choice_correction"):
            out.append(TensorSpec(name("correction"), (experts + identity,), "vector"))
        for e in range(experts):
            if gated:
                out.append(TensorSpec(name(f"e{e}.gate"), (ff, hidden), "matrix"))
            out += [TensorSpec(name(f"e{e}.up"), (ff, hidden), "matrix"), TensorSpec(name(f"e{e}.down"), (hidden, ff), "matrix")]
        if shared:
            if gated:
                out.append(TensorSpec(name("shared.gate"), (shared, hidden), "matrix"))
            out += [TensorSpec(name("shared.up"), (shared, hidden), "matrix"), TensorSpec(name("shared.down"), (hidden, shared), "matrix")]
            if spec.params.get("shared_gate"):
                out.append(TensorSpec(name("shared.sg"), (1, hidden), "matrix"))
        return out

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden, self.ff, self.experts, self.identity, self.shared = self._sizes(spec)
        self.top = int(p["top"])
        self.score = str(p.get("score", "softmax"))
        self.group_count, self.group_keep = int(p.get("group_count") or 0), int(p.get("group_keep") or 0)
        self.weight_eps, self.weight_scale = float(p.get("weight_eps") or 0.0), float(p.get("weight_scale", 1.0))
        self.normalize = bool(p.get("normalize_weights", True))
        self.gated = bool(p.get("gated"))
        self.activation = None if self.gated else str(p.get("activation", "relu2"))
        self.weight_on_input = p.get("weight_on", "output") == "input"
        if p.get("weight_on", "output") not in ("output", "input"):
            raise ValueError(f"routed_experts: weight_on '{p.get('weight_on')}' (output, input)")
        if self.weight_on_input and self.identity:
            raise ValueError("routed_experts: experts that return their input take their weights on the output")
        self.shared_gate = bool(p.get("shared_gate")) and self.shared > 0
        name = spec.tensor_name
        self.router = tensors.pop(name("router"))
        self.router_rows = int(self.router.shape[0])
        if self.shared_gate:
            # the shared expert's gate is one more row of the router's product
            self.router = torch.cat([self.router, tensors.pop(name("shared.sg"))], dim=0).contiguous()
        self.correction = tensors.pop(name("correction")) if p.get("choice_correction") else None
        ups = [tensors.pop(name(f"e{e}.up")) for e in range(self.experts)]
        self.gate_up_block = 0
        if self.gated:
            # Gate and up are one grouped product. Where the kernels offer it, an expert's rows alternate
            # in blocks (16 gate rows, their 16 up rows, ...) so that SiLU x up runs inside the product;
            # else an expert's gate rows come first and its up rows after them.
            gates = [tensors.pop(name(f"e{e}.gate")) for e in range(self.experts)]
            interleave = getattr(self.ops, "interleave_gate_up", None)
            mixed = [interleave(g, u) for g, u in zip(gates, ups)] if interleave is not None else [None]
            if mixed[0] is not None:
                ups, self.gate_up_block = mixed, int(getattr(self.ops, "SWIGLU_BLOCK", 16))
            else:
                ups = [torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]
        downs = [tensors.pop(name(f"e{e}.down")) for e in range(self.experts)]
        self.up_weight = torch.stack(ups, dim=0).contiguous()            # [experts, ff or 2 ff, hidden]
        self.down_weight = torch.stack(downs, dim=0).contiguous()        # [experts, hidden, ff]
        self.shared_up = tensors.pop(name("shared.up")) if self.shared else None
        self.shared_down = tensors.pop(name("shared.down")) if self.shared else None
        self.shared_interleaved = False
        if self.shared and self.gated:
            gate = tensors.pop(name("shared.gate"))
            interleave = getattr(self.ops, "interleave_gate_up", None)
            both = interleave(gate, self.shared_up) if interleave is not None else None
            self.shared_interleaved = both is not None
            self.shared_up = both if both is not None else torch.cat([gate, self.shared_up], dim=0).contiguous()

    def step_weight_bytes(self, num_tokens: int) -> int:
        """What a step of `num_tokens` tokens reads: the router, the shared expert and the experts it
        can be expected to choose (every token draws `top` of all experts alike)."""
        size = self.up_weight.element_size()
        total = self.experts + self.identity
        matrices = 3 if self.gated else 2
        touched = self.experts * (1.0 - (1.0 - min(1.0, self.top / total)) ** max(1, num_tokens))
        bytes_ = self.router.numel() * self.router.element_size() + matrices * self.shared * self.hidden * size
        return int(bytes_ + touched * matrices * self.ff * self.hidden * size)

    def _shared_hidden(self, x):
        ops = self.ops
        if not self.gated:
            return ops.linear(x, self.shared_up, None, activation=self.activation)
        if self.shared_interleaved:
            return ops.linear_swiglu(x, self.shared_up)
        return ops.silu_mul(ops.linear(x, self.shared_up, None))

    def forward(self, ctx, x, residual):
        ops = self.ops
        x = ops.materialized(x)
        logits = ops.linear(x, self.router, None, None, out_dtype=torch.float32)
        chosen, weights, _ = ops.route(logits, self.correction, self.top, self.group_count, self.group_keep, self.score,
                                       self.weight_eps, self.weight_scale, dense=False, normalize=self.normalize,
                                       experts=self.router_rows)
        base = ops.materialized(residual)
        if base is not None and base.dtype != torch.float32:
            base = residual = base.float()
        if self.shared_gate and residual is not None:
            raise ValueError("routed_experts: a gated shared expert cannot carry the residual")
        if self.shared:
            base = ops.linear(self._shared_hidden(x), self.shared_down, None, residual, out_dtype=torch.float32)
        plan = ops.expert_plan(x, chosen, self.experts, weights if self.weight_on_input else None)
        if self.gated:
            hidden = ops.linear_grouped(plan.staged, self.up_weight, plan, swiglu_block=self.gate_up_block)
        else:
            hidden = ops.linear_grouped(plan.staged, self.up_weight, plan, activation=self.activation)
        y = ops.linear_grouped(hidden, self.down_weight, plan, out_dtype=torch.float32)
        return ops.expert_combine(y, plan, None if self.weight_on_input else weights, x, base,
                                  base_gate=(logits, self.router_rows) if self.shared_gate else None)
