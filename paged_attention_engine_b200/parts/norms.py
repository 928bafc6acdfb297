"""Norms. RMSNorm as the reference computes it (engine/model.py:117-123): the mean of the
squares and the scaling in 32-bit, no bias, no mean subtraction. The kernel multiplies
by the weight in 32-bit too and rounds once; the reference rounds before and after the
weight, which costs one more rounding in bfloat16 and nothing in float32."""

from __future__ import annotations

from ..config.model_spec import PartSpec
from .base import NORMS, Part, TensorSpec


def offset_weight(weight, offset):
    """The weight a norm multiplies by: what the checkpoint stores, plus `offset` (float32)."""
    return weight + float(offset) if offset else weight


@NORMS.register("rms_norm")
class RMSNorm(Part):
    """params: size, eps, out ("engine": the result is in the engine's dtype whatever x is, as a
    float32 residual stream needs; default: x's dtype), weight_offset (c: the checkpoint stores
    w - c, as a weight kept around zero does with c = 1; default 0). tensors: weight [size]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["size"]),), "vector" if spec.params.get("weight_offset") else "scale")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.eps = float(spec.params["eps"])
        self.weight = offset_weight(tensors[spec.tensor_name("weight")], spec.params.get("weight_offset"))
        self.out_dtype = runtime.dtype if spec.params.get("out") == "engine" else None

    def forward(self, ctx, x):
        if self.out_dtype is not None:
            return self.ops.rms_norm_cast(x, self.weight, self.eps, self.out_dtype)
        return self.ops.rms_norm(x, self.weight, self.eps)


@NORMS.register("layer_norm")
class LayerNorm(Part):
    """(x - mean) / sqrt(var + eps) * weight + bias, var the mean of the squared deviations;
    statistics in 32-bit. params: size, eps, bias (default True), out ("engine": the result is
    in the engine's dtype even when x, a float32 residual stream, is not; default: x's dtype).
    tensors: weight [size], bias [size]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        size = int(spec.params["size"])
        out = [TensorSpec(spec.tensor_name("weight"), (size,), "scale")]
        if spec.params.get("bias", True):
            out.append(TensorSpec(spec.tensor_name("bias"), (size,), "vector"))
        return out

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.eps = float(spec.params["eps"])
        self.weight = tensors[spec.tensor_name("weight")]
        self.bias = tensors[spec.tensor_name("bias")] if spec.params.get("bias", True) else None
        self.out_dtype = runtime.dtype if spec.params.get("out") == "engine" else None

    def forward(self, ctx, x):
        return self.ops.layer_norm(x, self.weight, self.bias, self.eps, self.out_dtype)


@NORMS.register("stream_rms_norm")
class StreamRMSNorm(Part):
    """The read of a decoder with several residual streams: u = sum_s read[s] x_s, then u /
    sqrt(mean(u^2) + eps) * weight in the engine's dtype. x is float32 [tokens, streams * size]
    (or [tokens, size]: streams that are all equal). params: size, streams, eps, weight_offset (as
    for rms_norm), weighted_read (False: the plain sum of the streams, no `read` tensor).
    tensors: weight [size], read [streams]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        out = [TensorSpec(spec.tensor_name("weight"), (int(spec.params["size"]),), "vector" if spec.params.get("weight_offset") else "scale")]
        if spec.params.get("weighted_read", True):
            out.append(TensorSpec(spec.tensor_name("read"), (int(spec.params["streams"]),), "scale"))
        return out

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.eps = float(spec.params["eps"])
        self.streams = int(spec.params["streams"])
        self.weight = offset_weight(tensors[spec.tensor_name("weight")], spec.params.get("weight_offset"))
        self.read = tensors[spec.tensor_name("read")] if spec.params.get("weighted_read", True) else None

    def forward(self, ctx, x):
        return self.ops.streams_read_norm(x, self.read, self.weight, self.eps, self.streams, self.runtime.dtype)


@NORMS.register("dynamic_tanh")
class DynamicTanh(Part):
    """A norm that computes no mean and no variance: tanh(alpha * x) * weight + bias, alpha one
    learned scalar. params: size. tensors: weight [size], alpha [], bias [size]. x is a float32
    stream (or a residual sum that is still pending: this norm's kernel makes it on the way); the
    result is in the engine's dtype. As the norm AFTER a sublayer it is not run by itself:
    `add_to` leaves x + mult * norm(y) pending, and the norm that reads the stream next makes
    that sum and its own read in one pass."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        size = int(spec.params["size"])
        return [TensorSpec(spec.tensor_name("weight"), (size,), "scale"), TensorSpec(spec.tensor_name("alpha"), (), "scale"),
                TensorSpec(spec.tensor_name("bias"), (size,), "vector")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors[spec.tensor_name("weight")]
        self.alpha = tensors[spec.tensor_name("alpha")].reshape(1)
        self.bias = tensors[spec.tensor_name("bias")]

    def forward(self, ctx, x):
        return self.ops.dyt_norm(x, self.alpha, self.weight, self.bias, self.runtime.dtype)

    def add_to(self, ctx, stream, y, mult: float):
        """stream + mult * norm(y): float32, pending until the next read."""
        return self.ops.residual_add(stream, y, mult, (self.alpha, self.weight, self.bias))
