"""Finezen on the host: configuration, registry, tensor list, schedule, cache plan, the plain mechanisms by hand."""

import json
import math

import pytest
import torch

import finezen_helpers as fh
from paged_attention_engine_b200.cache import plan_cache
from paged_attention_engine_b200.config import ConfigError, FinezenConfig, resolve
from paged_attention_engine_b200.weights import collect_tensor_specs
from plain import finezen_plain as plain


def test_configuration_round_trip_and_registry():
    for raw, _page, _seed in fh.SMALL.values():
        cfg, spec = resolve(raw)
        assert isinstance(cfg, FinezenConfig)
        assert FinezenConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.to_dict() == raw
        assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"]
        for layer, entry in zip(spec.layers, raw["layers"]):
            assert layer.block == ("sandwich_residual" if entry["mlp"] else "sandwich_residual_mixer")
            assert layer.params["residual_mult"] == raw["residual_mult"]
            assert layer.mixer_norm.kind == layer.mixer_out_norm.kind == "dynamic_tanh"
            if entry["type"] == "attention":
                p = layer.mixer.params
                assert layer.mixer.kind == "gated_window_attention"
                assert (p["qk_norm"], p["learned_sink"], p["output_gate"]) == ("whole", True, "head")
                assert p["window"] == (entry["mixer"].get("mask") or {}).get("size", 0)
            else:
                p = layer.mixer.params
                assert layer.mixer.kind == "latent_attention" and p["head_gate"] and p["rot_dim"] == 0 and p["position_encoding"] is None
            if entry["mlp"]:
                p = layer.feed_forward.params
                assert layer.feed_forward.kind == "routed_experts"
                assert (p["gated"], p["score"], p["normalize_weights"], p["weight_on"]) == (True, "sigmoid", False, "input")
                assert p["shared_gate"] == bool(entry["mlp"].get("shared"))
        assert spec.final_norm.kind == "dynamic_tanh"


def test_the_schedule_repeats_the_loop_with_the_embedding_joining_again():
    _, spec = resolve(fh.SMALL_A)            # layers 1, 2 three times
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == [
        (0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]
    assert plain.layer_runs(fh.SMALL_A) == [(e.layer, e.add_embedding) for e in spec.schedule]
    _, spec = resolve(fh.NO_LOOP)
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == [(0, False), (1, False), (2, False)]
    _, spec = resolve(fh.ONE_LAYER_LOOP)
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == [(0, False), (1, False), (1, True), (1, True), (1, True)]
    _, spec = resolve(fh.SMALL_B)            # the loop is the whole model
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == [(0, False), (1, False), (2, False), (0, True), (1, False), (2, False)]
    once = json.loads(json.dumps(fh.SMALL_B))
    once["loop"]["times"] = 1
    assert [(e.layer, e.add_embedding) for e in resolve(once)[1].schedule] == [(0, False), (1, False), (2, False)]


def test_absent_keys_mean_absent_mechanisms_and_tensor_shapes():
    cfg = FinezenConfig.from_dict(fh.SMALL_A)
    assert cfg.layers[2].mlp is None and cfg.layers[2].mixer.window == 0 and cfg.layers[2].mixer.rot.scaling is None
    assert cfg.layers[1].mlp.shared_ff == 0 and cfg.layers[3].mixer.window == 0 and cfg.layers[4].mixer.rot is None
    assert FinezenConfig.from_dict(fh.NO_LOOP).loop is None
    names = collect_tensor_specs(resolve(fh.SMALL_A)[1])
    assert names["l0.mix.q"].shape == (48, 64) and names["l0.mix.k"].shape == (24, 64) and names["l0.mix.v"].shape == (40, 64)
    assert names["l0.mix.q.norm"].shape == (48,) and names["l0.mix.k.norm"].shape == (24,)       # over the whole projection
    assert names["l0.mix.sink"].shape == (4,) and names["l0.mix.g"].shape == (4, 64) and names["l0.mix.o"].shape == (64, 80)
    assert names["l1.mix.dq"].shape == (24, 64) and names["l1.mix.uq"].shape == (24, 24) and names["l1.mix.dkv"].shape == (20, 64)
    assert names["l1.mix.uk"].shape == (24, 20) and names["l1.mix.uv"].shape == (36, 20) and names["l1.mix.g"].shape == (3, 64)
    assert names["l0.norm1.alpha"].shape == () and names["l0.norm1b.b"].shape == (64,) and names["final.norm.alpha"].shape == ()
    assert names["l0.mlp.router"].shape == (6, 64) and names["l0.mlp.e5.gate"].shape == (40, 64) and "l0.mlp.e6.up" not in names
    assert names["l0.mlp.shared.sg"].shape == (1, 64) and names["l0.mlp.shared.down"].shape == (64, 24)
    assert "l1.mlp.shared.up" not in names and "l1.mlp.shared.sg" not in names
    assert "l2.norm2" not in names and "l2.norm2b" not in names and "l2.mlp.router" not in names


@pytest.mark.parametrize("damage, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["embedding"].pop("scale"), "embedding.scale"),
    (lambda c: c["layers"][0].update(type="mlstm"), "layers[0].type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "layers[0].mixer.heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "layers[0].mixer.rot.scaling.fast"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "layers[1].mixer.q_rank"),
    (lambda c: c["layers"][1]["mixer"]["mask"].pop("size"), "layers[1].mixer.mask.size"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "layers[0].mlp.kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "router.top"),
    (lambda c: c["layers"][1]["mlp"].pop("expert"), "layers[1].mlp.expert.ff"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("ff"), "layers[0].mlp.shared.ff"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop.times"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(damage, text):
    raw = json.loads(json.dumps(fh.SMALL_A))
    damage(raw)
    with pytest.raises(ConfigError, match=text.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
        FinezenConfig.from_dict(raw)


def test_cache_plan_every_pass_has_pages_of_its_own_and_no_state():
    _, spec = resolve(fh.SMALL_A)
    plan = plan_cache(spec)
    assert not plan.state_needs
    assert sorted(plan.entry_group) == list(range(len(spec.schedule)))         # every run of a layer holds its own keys
    by_entry = {pos: plan.groups[g] for pos, (g, _i) in plan.entry_group.items()}
    first = by_entry[0]
    assert (first.num_kv_heads, first.head_dim, first.value_dim, first.window) == (2, 12, 20, 7)
    latent = by_entry[1]
    assert (latent.num_kv_heads, latent.head_dim, latent.value_dim, latent.values_in_keys, latent.window) == (1, 20, 20, True, 21)
    # the three passes over layer 1 share a group and have an index each within it
    assert plan.entry_group[1][0] == plan.entry_group[3][0] == plan.entry_group[5][0]
    assert len({plan.entry_group[p][1] for p in (1, 3, 5)}) == 3


def test_plain_mechanisms_on_cases_worked_by_hand():
    f64 = torch.float64
    # the norm without statistics
    tensors = {"n": torch.tensor([2.0, -1.0]), "n.alpha": torch.tensor(0.5), "n.b": torch.tensor([0.25, 0.0])}
    got = plain.dynamic_tanh(torch.tensor([[2.0, 4.0]], dtype=f64), tensors, "n")
    assert torch.allclose(got, torch.tensor([[2.0 * math.tanh(1.0) + 0.25, -math.tanh(2.0)]], dtype=f64))
    # pairs (i, i + dims/2): with dims 4 channel 0 pairs with 2; position 1, frequency 1: one radian; channel 4 passes
    x = torch.tensor([[[1.0, 5.0, 0.0, 0.0, 7.0]], [[1.0, 5.0, 0.0, 0.0, 7.0]]], dtype=f64)
    turned = plain.rotate_half(x, [0, 1], {"dims": 4, "base": 100.0})
    assert torch.allclose(turned[0], x[0])
    f1 = 100.0 ** -0.5
    want = torch.tensor([[math.cos(1.0), 5.0 * math.cos(f1), math.sin(1.0), 5.0 * math.sin(f1), 7.0]], dtype=f64)
    assert torch.allclose(turned[1], want)
    # the ramp: below `lo` a pair keeps its frequency, above `hi` it is divided by the factor
    freqs, amplitude = plain.yarn_frequencies(8, 40.0, {"factor": 3.0, "original": 48, "fast": 6.0, "slow": 1.5})
    plain_f = [40.0 ** (-2.0 * i / 8) for i in range(4)]
    assert freqs[0] == plain_f[0] and freqs[3] == pytest.approx(plain_f[3] / 3.0) and plain_f[1] / 3.0 < freqs[1] < plain_f[1]
    assert amplitude == pytest.approx(0.1 * math.log(3.0) + 1.0)
    # a window of 2: the third query does not see the first key; the sink takes weight and gives nothing
    q = torch.ones(3, 1, 1, dtype=f64)
    k = torch.zeros(3, 1, 1, dtype=f64)
    v = torch.tensor([[[100.0]], [[1.0]], [[3.0]]], dtype=f64)
    out = plain.windowed_softmax_attention(q, k, v, 1.0, 2)
    assert out.flatten().tolist() == pytest.approx([100.0, 50.5, 2.0])
    out = plain.windowed_softmax_attention(q, k, v, 1.0, 2, sink=torch.tensor([0.0], dtype=f64))
    assert out.flatten().tolist() == pytest.approx([50.0, 101.0 / 3.0, 4.0 / 3.0])
    # the weight is on the expert's input: expert(w h), not w expert(h)
    tensors = {"m.router": torch.tensor([[0.0, 0.0], [1.0, 0.0]]),
               "m.e0.gate": torch.ones(1, 2), "m.e0.up": torch.ones(1, 2), "m.e0.down": torch.ones(2, 1),
               "m.e1.gate": torch.tensor([[1.0, 0.0]]), "m.e1.up": torch.tensor([[0.0, 1.0]]), "m.e1.down": torch.tensor([[1.0], [0.0]]),
               "m.shared.gate": torch.tensor([[0.0, 1.0]]), "m.shared.up": torch.tensor([[1.0, 0.0]]), "m.shared.down": torch.tensor([[0.0], [1.0]]),
               "m.shared.sg": torch.tensor([[0.0, 2.0]])}
    mlp = {"kind": "moe", "expert": {"ff": 1}, "router": {"experts": 2, "top": 1}, "shared": {"ff": 1}}
    h = torch.tensor([[2.0, 3.0]], dtype=f64)
    w = 1.0 / (1.0 + math.exp(-2.0))                 # expert 1: logit 2 against 0; its score is the weight as it is
    silu = lambda z: z / (1.0 + math.exp(-z))
    routed = silu(w * 2.0) * (w * 3.0)               # gate reads channel 0, up channel 1, both of w h
    shared = silu(3.0) * 2.0 / (1.0 + math.exp(-6.0))
    out = plain.mixture(h, tensors, "m", mlp)
    assert out[0].tolist() == pytest.approx([routed, shared])
    assert routed != pytest.approx(w * silu(2.0) * 3.0)
    # two chosen experts: both scores as they are, no renormalisation
    chosen, weights = plain.route(torch.tensor([[1.0, -1.0, 3.0]], dtype=f64), torch.eye(3), 2)
    assert chosen.tolist() == [[2, 0]] and weights[0].tolist() == pytest.approx([1 / (1 + math.exp(-3.0)), 1 / (1 + math.exp(-1.0))])


def test_random_models_are_written_and_read_back(tmp_path):
    from paged_attention_engine_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "m", fh.NO_LOOP, 3)
    raw, tensors = fh.read_model(folder)
    assert raw["architecture"] == "Finezen" and "loop" not in raw
    assert tensors["l0.norm1.alpha"].shape == () and tensors["l0.mix.sink"].shape == (1,)
    logits = plain.forward(raw, tensors, [1, 2, 3])
    assert logits.shape == (3, 97) and bool(torch.isfinite(logits).all())
