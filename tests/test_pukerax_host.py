"""Pukerax on the host: configuration, registry, tensor list, cache plan, the plain mechanisms by hand."""

import json
import math

import pytest
import torch

import pukerax_helpers as ph
from paged_attention_engine_b200.cache import plan_cache
from paged_attention_engine_b200.config import ConfigError, PukeraxConfig, resolve
from paged_attention_engine_b200.weights import collect_tensor_specs
from plain import pukerax_plain as plain


def test_configuration_round_trip_and_registry():
    for raw, _page, _seed in ph.SMALL.values():
        cfg, spec = resolve(raw)
        assert isinstance(cfg, PukeraxConfig)
        assert PukeraxConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.to_dict() == raw
        assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"]
        for layer, entry in zip(spec.layers, raw["layers"]):
            if raw.get("streams"):
                assert layer.block == ("hyper_connected" if entry["mlp"] else "hyper_connected_mixer")
                assert layer.mixer_norm.kind == "stream_rms_norm" and layer.mixer_merge.kind == "hyper_connection"
            else:
                assert layer.block == ("pre_norm_residual" if entry["mlp"] else "mixer_residual")
            assert layer.mixer.kind == "latent_attention" and layer.mixer.params["head_gate"]
            if entry["mlp"]:
                assert layer.feed_forward.kind == ("dense_mlp" if entry["mlp"]["kind"] == "dense" else "routed_experts")
                assert layer.feed_forward.params["activation"] == "relu2"
        assert spec.final_norm.kind == ("stream_rms_norm" if raw.get("streams") else "rms_norm")


def test_absent_keys_mean_absent_mechanisms():
    cfg = PukeraxConfig.from_dict(ph.SMALL_A)
    assert cfg.streams == 4 and PukeraxConfig.from_dict(ph.PLAIN_SUMS).streams == 0
    assert cfg.layers[2].mlp is None and cfg.layers[3].mixer.q_rank == 0 and cfg.layers[1].mixer.q_rank == 80
    router = cfg.layers[3].mlp.router
    assert (router.identity, router.group_count, cfg.layers[3].mlp.shared_ff) == (0, 0, 0)
    router = cfg.layers[1].mlp.router
    assert (router.experts, router.identity, router.total, router.group_count, router.group_keep) == (6, 2, 8, 4, 1)
    assert PukeraxConfig.from_dict(ph.PLAIN_SUMS).layers[2].mixer.rot_dims == 4
    names = collect_tensor_specs(resolve(ph.SMALL_A)[1])
    assert names["l0.mix.dq"].shape == (24, 64) and names["l0.mix.uq"].shape == (3 * 12, 24) and names["l0.mix.dq.norm"].shape == (24,)
    assert names["l0.mix.dkv"].shape == (24, 64) and names["l0.mix.g"].shape == (3, 64) and names["l0.mix.o"].shape == (64, 36)
    assert "l3.mix.dq" not in names and names["l3.mix.q"].shape == (24, 64)
    assert names["l1.mlp.router"].shape == (8, 64) and names["l1.mlp.correction"].shape == (8,)
    assert "l1.mlp.e5.up" in names and "l1.mlp.e6.up" not in names and names["l1.mlp.shared.down"].shape == (64, 24)
    assert "l3.mlp.shared.up" not in names and "l2.norm2" not in names and "l2.hc2.mix" not in names
    assert names["l2.hc1.mix"].shape == (4, 4) and names["l2.hc1.in"].shape == (4,) and names["l0.hc2.out"].shape == (4,)
    assert names["l0.norm1"].kind == "vector" and names["final.norm"].kind == "vector"       # stored around zero
    plain_names = collect_tensor_specs(resolve(ph.PLAIN_SUMS)[1])
    assert not any(".hc" in n for n in plain_names) and "l0.norm2" in plain_names


@pytest.mark.parametrize("damage, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["layers"][0].update(type="attention"), "layers[0].type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "layers[0].mixer.kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].pop("base"), "layers[0].mixer.rot.base"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "layers[0].mlp.kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "layers[1].mlp.router.top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "router.groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "router.top"),
    (lambda c: c["layers"][1]["mlp"].pop("expert"), "layers[1].mlp.expert.ff"),
    (lambda c: c["layers"][1]["mlp"]["shared"].pop("ff"), "layers[1].mlp.shared.ff"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(damage, text):
    raw = json.loads(json.dumps(ph.SMALL_A))
    damage(raw)
    with pytest.raises(ConfigError, match=text.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
        PukeraxConfig.from_dict(raw)


def test_cache_plan_holds_one_latent_row_per_token_and_no_state():
    plan = plan_cache(resolve(ph.SMALL_A)[1])
    by_entry = {pos: plan.groups[g] for pos, (g, _i) in plan.entry_group.items()}
    first = by_entry[0]
    assert (first.num_kv_heads, first.head_dim, first.value_dim, first.values_in_keys, first.window) == (1, 24, 20, True, 0)
    assert first.stored_per_token == 24
    assert by_entry[1].head_dim == 34 and by_entry[2].head_dim == 20
    assert plan.entry_group[0][0] == plan.entry_group[4][0]          # equal sizes share a group
    assert not plan.state_needs


def test_plain_mechanisms_on_cases_worked_by_hand():
    # the norm's stored weight is an offset from one
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    rms = math.sqrt(12.5)
    assert torch.allclose(plain.rms_norm(x, torch.tensor([0.0, 1.0]), 0.0, 1.0), torch.tensor([[3.0 / rms, 8.0 / rms]], dtype=torch.float64))
    # a pair at position 1 with dims 2 turns by one radian; the channel after it passes
    v = torch.tensor([[1.0, 0.0, 7.0], [1.0, 0.0, 7.0]], dtype=torch.float64)
    turned = plain.rotate_interleaved(v, [0, 1], 2, 100.0)
    assert torch.allclose(turned[0], v[0]) and torch.allclose(turned[1], torch.tensor([math.cos(1.0), math.sin(1.0), 7.0], dtype=torch.float64))
    # streams: the mix matrix is indexed [from, to]
    streams = torch.tensor([[[1.0]], [[10.0]]], dtype=torch.float64)
    tensors = {"c.mix": torch.tensor([[1.0, 2.0], [0.0, 3.0]]), "c.out": torch.tensor([0.5, -1.0])}
    new = plain.connect(streams, torch.tensor([[4.0]], dtype=torch.float64), tensors, "c")
    assert new.flatten().tolist() == [1.0 + 2.0, 2.0 + 30.0 - 4.0]
    # routing: router rows that read one input each, so the logits are the input
    h = torch.tensor([[2.0, 1.0, 0.0, 1.5]], dtype=torch.float64)
    s = torch.softmax(h[0], dim=0)
    zero = torch.zeros(4)
    chosen, weights = plain.route(h, torch.eye(4), zero, {"top": 2, "scale": 3.0})
    assert chosen.tolist() == [[0, 3]]
    assert torch.allclose(weights[0], torch.stack([s[0], s[3]]) / (s[0] + s[3]) * 3.0)
    # the correction moves the choice, not the weights
    chosen, weights = plain.route(h, torch.eye(4), torch.tensor([-1.0, 0.0, 0.0, 0.0]), {"top": 2, "scale": 1.0})
    assert chosen.tolist() == [[3, 1]] and torch.allclose(weights[0], torch.stack([s[3], s[1]]) / (s[3] + s[1]))
    # groups {0, 1} and {2, 3}: the second group's best is below the first's, so expert 3 is closed
    # although its score is the second best, and expert 1 is chosen instead
    margins = []
    chosen, _ = plain.route(h, torch.eye(4), zero, {"top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}}, margins)
    assert sorted(chosen[0].tolist()) == [0, 1]
    assert margins[0][0] == pytest.approx(min(float(s[0] - s[3]), math.inf))      # the groups' gap; no third open expert
    # negative choice scores still beat a closed group
    chosen, _ = plain.route(h, torch.eye(4), torch.tensor([-5.0, -9.0, -7.0, -7.0]), {"top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}})
    assert sorted(chosen[0].tolist()) == [0, 1]
    # an identity expert returns the input times its weight; a shared expert is added for every token
    mlp = {"kind": "moe", "expert": {"ff": 1}, "router": {"experts": 1, "identity": 1, "top": 1, "scale": 2.0}, "shared": {"ff": 1}}
    tensors = {"m.router": torch.tensor([[0.0, 0.0], [1.0, 0.0]]), "m.correction": torch.zeros(2),
               "m.e0.up": torch.ones(1, 2), "m.e0.down": torch.ones(2, 1),
               "m.shared.up": torch.tensor([[1.0, 1.0]]), "m.shared.down": torch.tensor([[1.0], [0.0]])}
    h = torch.tensor([[1.0, 2.0], [-1.0, 0.5]], dtype=torch.float64)
    out = plain.routed_feed_forward(h, tensors, "m", mlp)
    # token 0 chooses the identity expert (logit 1 > 0) with weight 2; token 1 the real one: relu(-0.5)^2 = 0
    assert torch.allclose(out[0], 2.0 * h[0] + torch.tensor([9.0, 0.0], dtype=torch.float64))
    assert torch.allclose(out[1], torch.zeros(2, dtype=torch.float64))


def test_random_models_are_written_with_streams_that_start_near_the_identity(tmp_path):
    from paged_attention_engine_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "m", ph.ONE_STREAM, 3)
    raw, tensors = ph.read_model(folder)
    assert raw["streams"] == 1 and tensors["l0.hc1.mix"].shape == (1, 1)
    folder = write_random_model(tmp_path / "n", ph.SMALL_A, 3)
    _, tensors = ph.read_model(folder)
    assert float((tensors["l0.hc2.mix"].float() - torch.eye(4)).abs().max()) < 0.2
    assert float(tensors["l0.norm1"].float().abs().max()) < 0.2
