"""Connections: how a sublayer's output goes back into the residual stream(s).

A hyper-connection keeps S streams per token. With the sublayer's output y, a matrix M indexed
[from, to] and a vector b, all streams are renewed at once from the old ones:
x'_t = sum_s M[s, t] x_s + b[t] y. (The read, a weighted sum of the streams, is the norm part
`stream_rms_norm`.) M and b are float32, as the streams are.
"""

from __future__ import annotations

from ..config.model_spec import PartSpec
from .base import CONNECTIONS, Part, TensorSpec


@CONNECTIONS.register("hyper_connection")
class HyperConnection(Part):
    """params: streams. tensors: mix [streams, streams], out [streams]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        s = int(spec.params["streams"])
        return [TensorSpec(spec.tensor_name("mix"), (s, s), "mixing"), TensorSpec(spec.tensor_name("out"), (s,), "scale")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.streams = int(spec.params["streams"])
        self.mix = tensors[spec.tensor_name("mix")]
        self.out = tensors[spec.tensor_name("out")]

    def forward(self, ctx, streams, y):
        """streams: float32 [tokens, S * width] (or [tokens, width]: S equal streams); y: the sublayer's
        output, float32 [tokens, width] or a product still to be summed. -> the new streams (pending)."""
        return self.ops.streams_write(streams, y, self.mix, self.out, self.streams)
