"""One registry from the architecture's name (config.json `architectures[0]`) to its model.

An entry holds the typed configuration class and the builder that turns a
configuration into a `ModelSpec`. The reference has a single hard-wired class
(engine/model.py:164, `Qwen2Engine`); here the name decides, everywhere: the
loader, the random-weights writer, generation and trace replay all go through
`resolve`.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .errors import ConfigError
from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .bidonex import BidonexConfig
from .finezen import FinezenConfig
from .qwen2 import Qwen2Config
from .pukerax import PukeraxConfig
from .zugarax import ZugaraxConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any
    build_spec: Callable[[Any], ModelSpec]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec) -> None:
    ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def resolve(raw: Mapping[str, Any]):
    """(typed configuration, ModelSpec) for the dictionary of a config.json."""
    # `architectures` is a list whose first name counts; a configuration may also name its one
    # architecture under `architecture`.
    names = raw.get("architectures") or ([raw["architecture"]] if raw.get("architecture") else None)
    if not names:
        raise ConfigError("config.json: key 'architectures' (or 'architecture') is missing; known: " + ", ".join(sorted(ARCHITECTURES)))
    arch = ARCHITECTURES.get(str(names[0]))
    if arch is None:
        raise ConfigError(
            f"config.json: architecture '{names[0]}' is not registered; known: " + ", ".join(sorted(ARCHITECTURES))
        )
    config = arch.config_class.from_dict(raw)
    return config, arch.build_spec(config)


def resolve_folder(folder: str | Path):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no such file")
    return resolve(json.loads(path.read_text()))


# --------------------------------------------------------------------------- #
# Qwen2 dense decoder (engine/model.py:322-351: per layer norm, attention, residual,
# norm, SwiGLU, residual; then the final norm and the head)
# --------------------------------------------------------------------------- #

def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    rotary = {"kind": "rotary", "head_dim": cfg.head_dim, "theta": cfg.rope_theta}
    layers = []
    for i in range(cfg.num_hidden_layers):
        prefix = f"model.layers.{i}"
        norm = {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
        layers.append(
            LayerSpec("pre_norm_residual", dict(
                mixer_norm=PartSpec("rms_norm", norm, f"{prefix}.input_layernorm"),
                mixer=PartSpec(
                    "gqa_attention",
                    {
                        "hidden_size": cfg.hidden_size,
                        "num_heads": cfg.num_attention_heads,
                        "num_kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                        "qkv_bias": True,  # always present in the reference (engine/model.py:87-92)
                        "scale": cfg.attention_scale,
                        "window": cfg.layer_window(i),
                        "position_encoding": rotary,
                    },
                    f"{prefix}.self_attn",
                ),
                feed_forward_norm=PartSpec("rms_norm", norm, f"{prefix}.post_attention_layernorm"),
                feed_forward=PartSpec(
                    "swiglu",
                    {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size},
                    f"{prefix}.mlp",
                ),
            ))
        )
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec(
            "token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, "model.embed_tokens"
        ),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm"),
        head=PartSpec(
            "lm_head",
            {
                "vocab_size": cfg.vocab_size,
                "hidden_size": cfg.hidden_size,
                "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
            },
            "lm_head",
        ),
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_spec)


# --------------------------------------------------------------------------- #
# Bidonex: token + learned position embedding into a float32 residual stream; per layer ONE
# LayerNorm whose output both branches read, x <- x + mixer(h) + ff(h); the mixer is a scored
# sliding-window attention (short convolutions on q, k, v; unit-RMS q and k; temperature, cap,
# log-distance bias, kept first keys, sink) or the generalized delta rule; the feed-forward is
# two matrices around the exact GELU, or absent; LayerNorm and an untied head at the end.
# --------------------------------------------------------------------------- #

# Fixed by the design: the decay is exp(-exp(-1/2) * sigmoid(.)), the unit key's epsilon 1e-6.
BIDONEX_DECAY_SCALE = 0.6065306597126334
BIDONEX_KEY_EPS = 1e-6


def bidonex_spec(cfg: BidonexConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        prefix = f"l{i}"
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec(
                "scored_window_attention",
                {
                    "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "scale": m.scale, "softcap": m.softcap, "conv_taps": m.conv,
                    "window": m.window, "keep_first": m.keep_first, "qk_norm_eps": cfg.norm_eps,
                    "head_temperature": True, "distance_bias": True, "sink": True,
                },
                f"{prefix}.mix",
            )
        else:
            mixer = PartSpec(
                "general_delta",
                {
                    "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "decay_rank": m.rank,
                    "decay_scale": BIDONEX_DECAY_SCALE, "key_eps": BIDONEX_KEY_EPS, "norm_eps": cfg.norm_eps,
                },
                f"{prefix}.mix",
            )
        parts = dict(
            norm=PartSpec("layer_norm", {"size": cfg.width, "eps": cfg.norm_eps, "out": "engine"},
                          names={"weight": f"{prefix}.norm1", "bias": f"{prefix}.norm1.b"}),
            mixer=mixer,
        )
        if layer.ff:
            parts["feed_forward"] = PartSpec(
                "dense_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.ff, "activation": "gelu_erf"},
                names={"up.weight": f"{prefix}.mlp.up", "down.weight": f"{prefix}.mlp.down"})
        layers.append(LayerSpec("parallel_residual" if layer.ff else "mixer_residual", parts))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding=PartSpec(
            "token_position_embedding",
            {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "max_positions": cfg.max_positions, "position_scale": 1.0},
            names={"weight": "embed", "positions": "pos"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(cfg.layers))),
        final_norm=PartSpec("layer_norm", {"size": cfg.width, "eps": cfg.norm_eps, "out": "engine"},
                            names={"weight": "final.norm", "bias": "final.norm.b"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None},
                      names={"weight": "head"}),
    )


register_architecture("Bidonex", BidonexConfig, bidonex_spec)


# --------------------------------------------------------------------------- #
# Zugarax: a scaled token embedding into a float32 residual stream; pre-norm layers (RMS norm,
# mixer, add; RMS norm, feed-forward, add; a layer may have no feed-forward); three mixers: a
# gated sliding-window attention with normed, partly rotated heads and one added to the softmax's
# denominator, a latent attention whose cache holds one normed latent and one rotated key part per
# token (a layer may read an earlier layer's), and the matrix memory of xLSTM; a feed-forward
# whose gate and up projections are clamped; RMS norm, an untied head and a tanh cap on the logits.
# --------------------------------------------------------------------------- #

# Fixed by the design: the gate's sigmoid is sharpened by 1.702; the sink's logit is 0.
ZUGARAX_GLU_ALPHA = 1.702
# The design has no longest sequence; positions are 32-bit integers.
ZUGARAX_MAX_POSITIONS = 1 << 30


def zugarax_spec(cfg: ZugaraxConfig) -> ModelSpec:
    layers = []
    schedule = []
    for i, layer in enumerate(cfg.layers):
        prefix = f"l{i}"
        m = layer.mixer
        cache_from = None
        if layer.type == "attention":
            encoding = None
            if m.rot is not None:
                scaling = dict(m.rot.scaling, kind="banded") if m.rot.scaling is not None else None
                encoding = {"kind": "scaled_rotary", "dims": m.rot.dims, "base": m.rot.base, "scaling": scaling}
            mixer = PartSpec(
                "gated_window_attention",
                {
                    "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "scale": m.scale, "window": m.window, "qk_norm_eps": cfg.norm_eps,
                    "unit_sink": True, "output_gate": True, "position_encoding": encoding,
                },
                f"{prefix}.mix",
            )
        elif layer.type == "latent_attention":
            scaling = dict(m.rot.scaling, kind="ramped") if m.rot.scaling is not None else None
            mixer = PartSpec(
                "latent_attention",
                {
                    "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
                    "value_dim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": cfg.norm_eps,
                    "own_latent": m.kv_from is None,
                    "position_encoding": {"kind": "scaled_rotary", "dims": m.rot.dims, "base": m.rot.base, "scaling": scaling},
                },
                f"{prefix}.mix",
            )
            cache_from = m.kv_from
        else:
            mixer = PartSpec(
                "matrix_memory",
                {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim,
                 "gate_cap": m.gate_cap, "norm_eps": cfg.norm_eps},
                f"{prefix}.mix",
            )
        norm = lambda name: PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "out": "engine"},
                                     names={"weight": f"{prefix}.{name}"})
        if layer.ff:
            parts = dict(
                mixer_norm=norm("norm1"), mixer=mixer, feed_forward_norm=norm("norm2"),
                feed_forward=PartSpec(
                    "clamped_glu", {"hidden_size": cfg.width, "intermediate_size": layer.ff, "limit": layer.limit,
                                    "alpha": ZUGARAX_GLU_ALPHA},
                    f"{prefix}.mlp"))
            layers.append(LayerSpec("pre_norm_residual", parts))
        else:
            layers.append(LayerSpec("mixer_residual", dict(norm=norm("norm1"), mixer=mixer)))
        schedule.append(ScheduleEntry(i, cache_from))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=ZUGARAX_MAX_POSITIONS,
        embedding=PartSpec("scaled_token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embedding_scale},
                           names={"weight": "embed"}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "out": "engine"}, names={"weight": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None, "softcap": cfg.logit_softcap},
                      names={"weight": "head"}),
    )


register_architecture("Zugarax", ZugaraxConfig, zugarax_spec)


# --------------------------------------------------------------------------- #
# Pukerax: a token embedding into float32; S residual streams joined by hyper-connections (each
# sublayer reads a weighted sum of the streams and its output is written back into all of them
# while a small matrix mixes them), or one stream with plain sums; RMS norms whose weights are
# stored around zero; latent attention whose queries go through a normed latent of their own and
# whose heads are gated by one sigmoid each; a feed-forward of squared ReLUs, dense or routed
# (softmax scores, a correction added for the choice only, groups of experts, experts that return
# their input, a shared expert); the streams' sum, RMS norm and an untied head at the end.
# --------------------------------------------------------------------------- #

# The design has no longest sequence; positions are 32-bit integers.
PUKERAX_MAX_POSITIONS = 1 << 30
# Fixed by the design: what is added to the sum of the chosen experts' scores before the division.
PUKERAX_WEIGHT_EPS = 1e-20


def pukerax_spec(cfg: PukeraxConfig) -> ModelSpec:
    layers = []
    streams = cfg.streams
    for i, layer in enumerate(cfg.layers):
        prefix = f"l{i}"
        m = layer.mixer
        mixer = PartSpec(
            "latent_attention",
            {
                "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
                "value_dim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "norm_eps": cfg.norm_eps,
                "head_gate": True,
                "position_encoding": {"kind": "scaled_rotary", "dims": m.rot_dims, "base": m.rot_base, "scaling": None},
            },
            f"{prefix}.mix",
        )
        feed_forward = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            feed_forward = PartSpec(
                "dense_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "relu2"},
                names={"up.weight": f"{prefix}.mlp.up", "down.weight": f"{prefix}.mlp.down"})
        elif layer.mlp is not None:
            r = layer.mlp.router
            feed_forward = PartSpec(
                "routed_experts",
                {
                    "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "relu2",
                    "num_experts": r.experts, "identity_experts": r.identity, "top": r.top, "score": "softmax",
                    "choice_correction": True, "group_count": r.group_count, "group_keep": r.group_keep,
                    "weight_eps": PUKERAX_WEIGHT_EPS, "weight_scale": r.scale, "shared_size": layer.mlp.shared_ff,
                },
                f"{prefix}.mlp",
            )

        def norm(name, q):
            if streams:
                return PartSpec("stream_rms_norm", {"size": cfg.width, "streams": streams, "eps": cfg.norm_eps, "weight_offset": 1.0,
                                                    "weighted_read": True},
                                names={"weight": f"{prefix}.{name}", "read": f"{prefix}.hc{q}.in"})
            return PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "out": "engine", "weight_offset": 1.0},
                            names={"weight": f"{prefix}.{name}"})

        parts = dict(mixer_norm=norm("norm1", 1), mixer=mixer)
        if feed_forward is not None:
            parts.update(feed_forward_norm=norm("norm2", 2), feed_forward=feed_forward)
        if streams:
            parts["mixer_merge"] = PartSpec("hyper_connection", {"streams": streams}, f"{prefix}.hc1")
            if feed_forward is not None:
                parts["feed_forward_merge"] = PartSpec("hyper_connection", {"streams": streams}, f"{prefix}.hc2")
            block = "hyper_connected" if feed_forward is not None else "hyper_connected_mixer"
        else:
            block = "pre_norm_residual" if feed_forward is not None else "mixer_residual"
            if feed_forward is None:
                parts = dict(norm=parts["mixer_norm"], mixer=mixer)
        layers.append(LayerSpec(block, parts))
    if streams:
        final_norm = PartSpec("stream_rms_norm", {"size": cfg.width, "streams": streams, "eps": cfg.norm_eps, "weight_offset": 1.0,
                                                  "weighted_read": False}, names={"weight": "final.norm"})
    else:
        final_norm = PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "out": "engine", "weight_offset": 1.0},
                              names={"weight": "final.norm"})
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=PUKERAX_MAX_POSITIONS,
        embedding=PartSpec("scaled_token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": 1.0},
                           names={"weight": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(cfg.layers))),
        final_norm=final_norm,
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None}, names={"weight": "head"}),
    )


register_architecture("Pukerax", PukeraxConfig, pukerax_spec)


# --------------------------------------------------------------------------- #
# Finezen: a scaled token embedding into a float32 residual stream; every sublayer between two
# norms without statistics, x <- x + m * dyt_b(f(dyt_a(x))) with dyt(v) = tanh(alpha v) w + b; the
# mixer a windowed grouped-query attention (q and k normed over the whole projection, a leading
# span of each head rotated with ramped frequencies, a learned sink per head, a gate per head) or a
# windowed latent attention without positions (a query latent, a gate per head); the feed-forward a
# mixture of gated experts (sigmoid scores taken as weights as they are, on the experts' inputs) with
# a shared expert behind a sigmoid of its own; a span of layers may run several times with the same
# weights, a cache per pass, the embedding's output joining the stream again before each further
# pass; the same norm and an untied head at the end.
# --------------------------------------------------------------------------- #

# The design has no longest sequence; positions are 32-bit integers.
FINEZEN_MAX_POSITIONS = 1 << 30


def finezen_spec(cfg: FinezenConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        prefix = f"l{i}"
        m = layer.mixer
        if layer.type == "attention":
            encoding = None
            if m.rot is not None:
                scaling = dict(m.rot.scaling, kind="ramped") if m.rot.scaling is not None else None
                encoding = {"kind": "scaled_rotary", "dims": m.rot.dims, "base": m.rot.base, "scaling": scaling}
            mixer = PartSpec(
                "gated_window_attention",
                {
                    "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "scale": m.scale, "window": m.window, "qk_norm_eps": cfg.norm_eps, "qk_norm": "whole",
                    "learned_sink": True, "output_gate": "head", "position_encoding": encoding,
                },
                f"{prefix}.mix",
            )
        else:
            mixer = PartSpec(
                "latent_attention",
                {
                    "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": 0, "value_dim": m.vdim,
                    "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "norm_eps": cfg.norm_eps, "window": m.window,
                    "head_gate": True, "position_encoding": None,
                },
                f"{prefix}.mix",
            )
        norm = lambda name: PartSpec("dynamic_tanh", {"size": cfg.width},
                                     names={"weight": f"{prefix}.{name}", "alpha": f"{prefix}.{name}.alpha", "bias": f"{prefix}.{name}.b"})
        parts = dict(mixer_norm=norm("norm1"), mixer=mixer, mixer_out_norm=norm("norm1b"))
        if layer.mlp is not None:
            parts.update(
                feed_forward_norm=norm("norm2"),
                feed_forward=PartSpec(
                    "routed_experts",
                    {
                        "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "gated": True, "num_experts": layer.mlp.experts,
                        "top": layer.mlp.top, "score": "sigmoid", "normalize_weights": False, "weight_scale": 1.0,
                        "weight_on": "input", "shared_size": layer.mlp.shared_ff, "shared_gate": bool(layer.mlp.shared_ff),
                    },
                    f"{prefix}.mlp",
                ),
                feed_forward_out_norm=norm("norm2b"))
        layers.append(LayerSpec("sandwich_residual" if layer.mlp is not None else "sandwich_residual_mixer", parts,
                                {"residual_mult": cfg.residual_mult}))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=FINEZEN_MAX_POSITIONS,
        embedding=PartSpec("scaled_token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embedding_scale},
                           names={"weight": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, None, add) for i, add in cfg.runs()),
        final_norm=PartSpec("dynamic_tanh", {"size": cfg.width},
                            names={"weight": "final.norm", "alpha": "final.norm.alpha", "bias": "final.norm.b"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None}, names={"weight": "head"}),
    )


register_architecture("Finezen", FinezenConfig, finezen_spec)
