"""Pukerax on the GPU: every mechanism against the plain implementation, then whole models
through the step function under every kind of schedule, the scheduler and the trace program."""

import copy
import math

import pytest
import torch

import helpers
import pukerax_helpers as ph
from plain import pukerax_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
DEV = "cuda:0"


def _ops():
    from paged_attention_engine_b200.kernels import ops

    return ops


def _close(got, want, dtype, scale=1.0):
    tol = (2e-5 if dtype == torch.float32 else 2.0 ** -6) * scale * max(1.0, float(want.abs().max()))
    gap = float((got.double().cpu() - want.double()).abs().max())
    assert gap <= tol, f"max difference {gap} > {tol}"


# --------------------------------------------------------------------------- #
# Mechanisms alone
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams, width, splits", [(1, 48, 1), (2, 64, 3), (3, 257, 1), (4, 1024, 5), (8, 40, 2)])
def test_streams_read_write_and_both_in_one_kernel(dtype, streams, width, splits):
    """The read (weighted sum, norm), the write (mix and output weight), the write of one sublayer
    with the read of the next in one kernel, equal streams given as one, and a sublayer's output
    that is still the planes of a split product."""
    ops = _ops()
    T = 7
    x = torch.randn(T, streams, width) * 2.0
    planes = torch.randn(splits, T, width)
    y = planes.double().sum(0)
    mix, out_w = torch.randn(streams, streams), torch.randn(streams)
    in_w, norm_w = torch.randn(streams), torch.rand(width) + 0.5
    dev = lambda t: t.to(DEV).contiguous()
    tensors = {"c.mix": mix, "c.out": out_w}
    want_new = plain.connect(x.double().transpose(0, 1), y, tensors, "c")                    # [S, T, W]
    want_read = plain.rms_norm(torch.einsum("s,stw->tw", in_w.double(), want_new), norm_w, 1e-5)
    flat = dev(x.view(T, streams * width))
    sublayer = ops.PendingSum(dev(planes), None, None, torch.float32) if splits > 1 else dev(planes[0])
    # the write alone
    pending = ops.streams_write(flat, sublayer, dev(mix), dev(out_w), streams)
    new = ops.materialized(pending)
    _close(new.view(T, streams, width).transpose(0, 1), want_new, torch.float32)
    # the read alone, of those streams, with and without read weights
    _close(ops.streams_read_norm(new, dev(in_w), dev(norm_w), 1e-5, streams, dtype), want_read, dtype)
    _close(ops.streams_read_norm(new, None, dev(norm_w), 1e-5, streams, dtype), plain.rms_norm(want_new.sum(0), norm_w, 1e-5), dtype)
    # write and read in one kernel: the same bits as the two kernels
    sublayer = ops.PendingSum(dev(planes), None, None, torch.float32) if splits > 1 else dev(planes[0])
    pending = ops.streams_write(flat, sublayer, dev(mix), dev(out_w), streams)
    fused = ops.streams_read_norm(pending, dev(in_w), dev(norm_w), 1e-5, streams, dtype)
    assert pending.value is not None and torch.equal(pending.value, new)
    assert torch.equal(fused, ops.streams_read_norm(new, dev(in_w), dev(norm_w), 1e-5, streams, dtype))
    # equal streams given as one row
    one = torch.randn(T, width)
    spread = one[:, None, :].expand(T, streams, width).double().transpose(0, 1)
    _close(ops.streams_read_norm(dev(one), dev(in_w), dev(norm_w), 1e-5, streams, dtype),
           plain.rms_norm(torch.einsum("s,stw->tw", in_w.double(), spread), norm_w, 1e-5), dtype)
    got = ops.materialized(ops.streams_write(dev(one), dev(planes[0]), dev(mix), dev(out_w), streams))
    _close(got.view(T, streams, width).transpose(0, 1), plain.connect(spread, planes[0].double(), tensors, "c"), torch.float32)


@pytest.mark.parametrize("total, top, groups, keep, scale", [
    (4, 2, 0, 0, 1.0), (10, 3, 2, 1, 1.7), (8, 2, 4, 2, 1.0), (12, 1, 12, 5, 0.7), (16, 4, 4, 2, 3.0), (64, 6, 8, 3, 2.0),
    (40, 8, 0, 0, 1.0), (7, 7, 0, 0, 1.0), (96, 3, 3, 1, 1.0)])
def test_router_choice_groups_and_weights(total, top, groups, keep, scale):
    ops = _ops()
    gen = torch.Generator().manual_seed(total * 7 + top)
    T = 37
    logits = torch.randn(T, total, generator=gen) * 3.0
    # negative corrections: choice scores below zero must still beat a closed group's
    correction = torch.randn(total, generator=gen) * 0.1 - 1.25 - 1.25 * (torch.rand(total, generator=gen) < 0.2)
    r = {"top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    margins = []
    want_chosen, want_weights = plain.route(logits.double(), torch.eye(total), correction, r, margins)
    clear = margins[0] > 1e-5
    assert int(clear.sum()) > T // 2
    chosen, weights, dense = ops.route(logits.to(DEV), correction.to(DEV), top, groups, keep, "softmax", 1e-20, scale)
    chosen, weights, dense = chosen.cpu().long(), weights.cpu(), dense.cpu()
    assert torch.equal(chosen[clear], want_chosen[clear])                      # in the order of the choice, too
    assert torch.allclose(weights[clear].double(), want_weights[clear], rtol=2e-5, atol=1e-7)
    want_dense = torch.zeros(T, total, dtype=torch.float64).scatter_(1, want_chosen, want_weights)
    assert torch.allclose(dense[clear].double(), want_dense[clear], rtol=2e-5, atol=1e-7)
    assert torch.allclose(weights.sum(1), torch.full((T,), scale), rtol=1e-5)
    # logits that are still the planes of a split product: added in their order by the kernel itself
    planes = torch.randn(3, T, total, generator=gen)
    summed = (planes[0] + planes[1]) + planes[2]
    pending = ops.PendingSum(planes.to(DEV), None, None, torch.float32)
    one = ops.route(summed.to(DEV), correction.to(DEV), top, groups, keep, "softmax", 1e-20, scale)
    two = ops.route(pending, correction.to(DEV), top, groups, keep, "softmax", 1e-20, scale)
    assert pending.value is None and all(torch.equal(a, b) for a, b in zip(one, two))


def test_router_without_correction():
    ops = _ops()
    logits = torch.randn(9, 6) * 2.0
    want_chosen, want_weights = plain.route(logits.double(), torch.eye(6), torch.zeros(6), {"top": 3, "scale": 1.5})
    chosen, weights, dense = ops.route(logits.to(DEV), None, 3, 0, 0, "softmax", 0.0, 1.5, dense=False)
    assert dense is None
    assert torch.equal(chosen.cpu().long(), want_chosen) and torch.allclose(weights.cpu().double(), want_weights, rtol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, top, experts, identity, width, ff", [
    (1, 2, 4, 0, 64, 32), (7, 3, 5, 2, 48, 24), (300, 2, 6, 1, 128, 64), (1200, 2, 6, 1, 128, 64), (900, 4, 16, 0, 64, 200), (130, 1, 3, 3, 72, 40),
    (260, 2, 2, 0, 256, 96), (50, 2, 4, 1, 44, 20), (40, 2, 3, 0, 64, 20)])
def test_experts_over_the_chosen_pairs_only(dtype, tokens, top, experts, identity, width, ff):
    """The pairs sorted by expert, both grouped products and the weighted sum against a loop over
    tokens; an expert with hundreds of pairs (several tiles), experts with none, pairs of experts
    without tensors, one token; few pairs (one block sorts them) and thousands."""
    ops = _ops()
    gen = torch.Generator().manual_seed(tokens + top)
    total = experts + identity
    x = torch.randn(tokens, width, generator=gen).to(dtype)
    # uneven: the first expert gets most pairs, the last expert with tensors none
    favour = torch.rand(tokens, total, generator=gen)
    favour[:, 0] += 0.5
    if experts > 2:
        favour[:, experts - 1] = -1.0
    chosen = favour.topk(top, dim=1).indices.int()
    weights = torch.rand(tokens, top, generator=gen) + 0.1
    up = (torch.randn(experts, ff, width, generator=gen) * 0.2).to(dtype)
    down = (torch.randn(experts, width, ff, generator=gen) * 0.2).to(dtype)
    base = torch.randn(tokens, width, generator=gen)
    plan = ops.expert_plan(x.to(DEV), chosen.to(DEV), experts)
    rows, tiles = plan.rows.cpu(), plan.tiles.cpu()
    with_tensors = chosen < experts
    assert bool((rows[with_tensors] >= 0).all()) and bool((rows[~with_tensors] == -1).all())
    assert len(set(rows[with_tensors].tolist())) == int(with_tensors.sum())                     # every pair a row of its own
    for t, k in with_tensors.nonzero().tolist():
        row = int(rows[t, k])
        assert int(tiles[row // ops.EXPERT_TILE, 0]) == int(chosen[t, k]) and row % ops.EXPERT_TILE < int(tiles[row // ops.EXPERT_TILE, 1])
        assert torch.equal(plan.staged[row].cpu(), x[t])
    assert int(tiles[:-1][tiles[:-1, 0] >= 0, 1].sum()) == int(with_tensors.sum())
    used = int(tiles[-1, 0])                                             # the tiles in use are the first ones
    assert bool((tiles[:used, 0] >= 0).all()) and bool((tiles[used:-1, 0] == -1).all())
    hidden = ops.linear_grouped(plan.staged, up.to(DEV), plan, activation="relu2")
    y = ops.linear_grouped(hidden, down.to(DEV), plan, out_dtype=torch.float32)
    got = ops.expert_combine(y, plan, weights.to(DEV), x.to(DEV), base.to(DEV))
    bare = ops.expert_combine(y, plan, weights.to(DEV), x.to(DEV))
    want = base.double().clone()
    for t in range(tokens):
        for k in range(top):
            e = int(chosen[t, k])
            if e >= experts:
                want[t] += float(weights[t, k]) * x[t].double()
                continue
            z = torch.relu(x[t].double() @ up[e].double().T)
            if dtype == torch.bfloat16:
                z = z.to(dtype).double()
            z = z * z
            if dtype == torch.bfloat16:
                z = z.to(dtype).double()
            want[t] += float(weights[t, k]) * (z @ down[e].double().T)
    _close(got, want, dtype, scale=2.0)
    _close(bare, want - base.double(), dtype, scale=2.0)
    halves = torch.randn(2, tokens, width, generator=gen)
    pending = ops.PendingSum(halves.to(DEV), None, None, torch.float32)
    assert torch.equal(ops.expert_combine(y, plan, weights.to(DEV), x.to(DEV), pending),
                       ops.expert_combine(y, plan, weights.to(DEV), x.to(DEV), (halves[0] + halves[1]).to(DEV)))
    assert pending.value is None
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gates_norm_of_columns_and_the_squared_relu(dtype):
    ops = _ops()
    x = torch.randn(6, 4 * 10).to(dtype)
    proj = torch.randn(6, 50)
    want = x.double().view(6, 4, 10) * torch.sigmoid(proj[:, 7:11].double())[:, :, None]
    _close(ops.sigmoid_gate(x.to(DEV), proj.to(DEV), 7, group=10), want.reshape(6, 40), dtype)
    w = torch.rand(24) + 0.5
    _close(ops.rms_norm_columns(proj.to(DEV), 11, 24, w.to(DEV), 1e-6, dtype), plain.rms_norm(proj[:, 11:35].double(), w, 1e-6), dtype)
    for tokens, k, n in ((5, 64, 48), (70, 128, 256), (300, 64, 96)):
        a, b = (torch.randn(tokens, k) * 0.5).to(dtype), (torch.randn(n, k) * 0.3).to(dtype)
        got = ops.materialized(ops.linear(a.to(DEV), b.to(DEV), None, activation="relu2"))
        z = torch.relu(a.double() @ b.double().T)
        if dtype == torch.bfloat16:
            z = z.to(torch.bfloat16).double()            # the product is rounded before the activation
        _close(got, z * z, dtype, scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, index", [("small_a", 1), ("small_a", 4), ("small_b", 1), ("small_b", 2), ("plain_sums", 0)])
def test_routed_feed_forward_alone(folders, name, index, dtype):
    """One routed feed-forward of a model against the plain one, on inputs whose choices are clear."""
    from paged_attention_engine_b200.config import resolve
    from paged_attention_engine_b200.parts import FEED_FORWARDS, Runtime

    raw, tensors = ph.read_model(folders[name])
    spec = resolve(raw)[1].layers[index].feed_forward
    mlp = raw["layers"][index]["mlp"]
    gen = torch.Generator().manual_seed(index)
    h = torch.randn(90, raw["width"], generator=gen).to(dtype)
    margins = []
    want = plain.routed_feed_forward(h.double(), tensors, f"l{index}.mlp", mlp, margins)
    clear = margins[0] > ph.CLEAR_CHOICE
    assert int(clear.sum()) > 30
    runtime = Runtime(_ops(), dtype, torch.device(DEV))
    own = {k: (v.float() if v.dim() == 1 else v.to(dtype)).to(DEV) for k, v in tensors.items() if k.startswith(f"l{index}.mlp.")}
    part = FEED_FORWARDS.get(spec.kind)(spec, own, runtime)
    got = _ops().materialized(part.forward(None, h.to(DEV), None))
    assert got.dtype == torch.float32
    _close(got[clear.to(DEV)], want[clear], dtype, scale=2.0)
    residual = torch.randn(90, raw["width"], generator=gen)
    got = _ops().materialized(part.forward(None, h.to(DEV), residual.to(DEV)))
    _close(got[clear.to(DEV)], (want + residual.double())[clear], dtype, scale=2.0)


# --------------------------------------------------------------------------- #
# Whole models through the step function
# --------------------------------------------------------------------------- #

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("pukerax")
    return {name: ph.write_model(root / name, raw, seed) for name, (raw, _page, seed) in ph.SMALL.items()}


@pytest.fixture(scope="module")
def prompts(folders):
    """Per model: prompts whose routers' choices are clear, and the plain model's logits for them."""
    return {name: ph.clear_requests(folders[name], [53, 9, 38, 2, 27], seed) for name, (_raw, _page, seed) in ph.SMALL.items()}


def _check(folder, dtype, trace, requests, oracle, page, max_live=4, fragment=None):
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer

    engine = Engine.from_pretrained(folder, dtype)
    replayer = Replayer(engine, helpers.max_live_tokens(trace, page), page, max_live)
    if fragment is not None and replayer.manager.groups:
        helpers.fragment_pool(replayer.manager, fragment)
    outputs = {}
    for record in trace:
        logits = replayer.run(record)
        if logits is not None:
            outputs[record["step"]] = logits.float().cpu()
    engine.runtime.ops.check_device_errors()
    got = helpers.collect(trace, outputs, requests)
    for key, want in oracle.items():
        gap = (got[key] - want).abs().max(dim=1).values
        allowed = ph.row_tolerance(dtype, want, folder, requests[key])
        worst = int((gap - allowed).argmax())
        assert bool((gap <= allowed).all()), f"{key}: |dlogit| {float(gap[worst])} > {float(allowed[worst])} at position {worst}"
    assert not replayer.manager.live_requests()
    assert replayer.manager.num_free == replayer.manager.num_blocks
    return got


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ph.SMALL))
def test_schedules_agree_with_the_plain_model(folders, prompts, name, dtype):
    raw, page, seed = ph.SMALL[name]
    requests, oracle = prompts[name]
    whole = _check(folders[name], dtype, helpers.trace_whole(requests), requests, oracle, page)
    tail = _check(folders[name], dtype, helpers.trace_tail(requests, tail=30), requests, oracle, page)
    chunks = _check(folders[name], dtype, helpers.trace_chunks(requests, seed), requests, oracle, page, fragment=seed)
    mixed = _check(folders[name], dtype, helpers.trace_mixed(requests, seed, live_limit=3, decode_tail=10), requests, oracle,
                   page, max_live=3, fragment=seed + 1)
    # How the tokens were cut, what else was in the batch and which pages and slots were used
    # changes a logit by rounding only.
    cut = (2e-5 if dtype == torch.float32 else 2.0 ** -6)
    for key in requests:
        top = max(1.0, float(oracle[key].abs().max()))
        for other in (tail, chunks, mixed):
            assert float((other[key] - whole[key]).abs().max()) <= cut * top


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_many_pages(folders, dtype):
    raw, page, seed = ph.SMALL["small_b"]
    requests, oracle = ph.clear_requests(folders["small_b"], [150], seed + 50)
    _check(folders["small_b"], dtype, helpers.trace_tail(requests, tail=140), requests, oracle, page)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_that_stands_out_is_found(tmp_path, dtype):
    """One early token whose key stands out for every later query, hundreds of tokens back and
    across many pages. Only that token's embedding has channel 0; the latent's first channel reads
    channel 0 alone and its norm weight is large, so that token's key and value are many times any
    other's, and about half of the queries (those whose product with it is positive) put nearly all
    their weight on it. The logits follow the plain model, and are far from the plain model of the
    same prompt without that token."""
    from safetensors.torch import load_file, save_file

    raw = ph.config(61, 64, [ph.layer(ph.mixer(2, 16, 16, 16, 32, 24, 0.25, base=10000.0), ph.dense(64))], streams=2)
    folder = ph.write_model(tmp_path / "far", raw, 77)
    path = str(folder / "model.safetensors")
    tensors = load_file(path)
    for name, change in (("embed", lambda t: (t[:, 0].zero_(), t[60, 0].fill_(3.0))), ("l0.mix.dkv", lambda t: (t[0].zero_(), t[0, 0].fill_(4.0))),
                         ("l0.mix.dkv.norm", lambda t: t[0].fill_(40.0))):
        t = tensors[name].float()
        change(t)
        tensors[name] = t.to(torch.bfloat16)
    save_file(tensors, path)
    gen = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, 60, (420,), generator=gen).tolist()
    tokens[3] = 60                                       # the one token of its kind
    want = plain.forward(raw, tensors, tokens).float()
    without = plain.forward(raw, tensors, tokens[:3] + [7] + tokens[4:]).float()
    requests = {"r0": tokens}
    got = _check(folder, dtype, helpers.trace_tail(requests, tail=40), requests, {"r0": want}, 16)["r0"]
    missing = (without[300:] - got[300:]).abs().max(dim=1).values
    assert float(missing.median()) > 4.0 * ph.tolerance(torch.bfloat16, want)
    assert float(missing.max()) > 10.0 * float((want[300:] - got[300:]).abs().max())


def _plain_greedy(folder, prompt, count):
    raw, tensors = ph.read_model(folder)
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain.forward(raw, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small_b", "plain_sums"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from paged_attention_engine_b200 import LLM, Request

    raw, page, seed = ph.SMALL[name]
    llm = LLM.from_pretrained(folders[name], dtype=str(dtype).replace("torch.", ""), num_blocks=48, block_size=page,
                              max_num_seqs=4, max_num_batched_tokens=16, record_logits=True)
    prompts, _ = ph.clear_requests(folders[name], [5, 21, 12], seed + 20)
    for i, prompt in enumerate(prompts.values()):
        assert llm.add_request(Request(f"g{i}", tuple(prompt), 7))
    out = llm.run_to_completion()
    raw_config, tensors = ph.read_model(folders[name])
    for i, prompt in enumerate(prompts.values()):
        tokens = list(out[f"g{i}"])
        assert len(tokens) == 7
        margins = []
        want = plain.forward(raw_config, tensors, prompt + tokens, margins=margins).float()[len(prompt) - 1 : -1]
        got = torch.stack(llm.scheduler.finished[f"g{i}"].step_logits)
        # generated tokens were not drawn for clear choices: compare up to the first close call
        close = (torch.stack(margins).min(dim=0).values < ph.CLEAR_CHOICE).nonzero()
        clear_until = int(close[0]) if len(close) else len(prompt) + 7
        rows = max(0, min(7, clear_until - (len(prompt) - 1)))
        assert rows >= 1
        assert float((got[:rows] - want[:rows]).abs().max()) <= ph.tolerance(dtype, want)
        if dtype == torch.float32 and rows == 7:
            assert tokens == _plain_greedy(folders[name], prompt, 7)


def test_trace_program_on_a_random_model(folders, prompts, tmp_path):
    raw, page, seed = ph.SMALL["small_a"]
    requests, oracle = prompts["small_a"]
    requests = {k: requests[k] for k in ("r1", "r2", "r4")}
    trace = helpers.trace_mixed(requests, seed, live_limit=2, decode_tail=6)
    outputs = helpers.run_trace_program(folders["small_a"], "bfloat16", trace, helpers.max_live_tokens(trace, page),
                                        tmp_path / "out", raw["vocab"], block_size=page)
    got = helpers.collect(trace, outputs, requests)
    for key in requests:
        assert float((got[key] - oracle[key]).abs().max()) <= ph.tolerance(torch.bfloat16, oracle[key])


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_tolerance_notices_a_fault_in_any_mechanism(folders, prompts, dtype, monkeypatch):
    """The plain model with one mechanism changed (the mix matrix transposed, no gate, the other
    pairing, the correction in the weights, no groups, silent identity experts, ...) leaves the
    tolerance around the engine's logits: the comparisons above could tell."""
    raw, page, seed = ph.SMALL["small_a"]
    requests, oracle = prompts["small_a"]
    requests, oracle = {"r0": requests["r0"]}, {"r0": oracle["r0"]}
    got = _check(folders["small_a"], dtype, helpers.trace_whole(requests), requests, oracle, page)["r0"]
    config, tensors = ph.read_model(folders["small_a"])
    tol = ph.tolerance(dtype, oracle["r0"])

    def gap(changed_config=config, changed_tensors=tensors):
        return float((plain.forward(changed_config, changed_tensors, requests["r0"]).float() - got).abs().max())

    def changed(path, value):
        out = copy.deepcopy(config)
        node = out
        for key in path[:-1]:
            node = node[key]
        if value is None:
            node.pop(path[-1])
        else:
            node[path[-1]] = value
        return out

    def with_tensor(name, change):
        out = dict(tensors)
        out[name] = change(tensors[name].float()).to(tensors[name].dtype)
        return out

    faults = {
        "score scale": gap(changed(["layers", 0, "mixer", "scale"], 0.3)),
        "rotation base": gap(changed(["layers", 0, "mixer", "rot", "base"], 500.0)),
        "rotated channels": gap(changed(["layers", 2, "mixer", "rot", "dims"], 6)),
        "mix matrix transposed": gap(changed_tensors=with_tensor("l1.hc1.mix", lambda t: t.T.contiguous())),
        "read weights": gap(changed_tensors=with_tensor("l2.hc1.in", torch.ones_like)),
        "write weights": gap(changed_tensors=with_tensor("l3.hc2.out", torch.ones_like)),
        "query latent's norm weight": gap(changed_tensors=with_tensor("l0.mix.dq.norm", torch.ones_like)),
        "head gates": gap(changed_tensors={k: v for k, v in tensors.items() if not k.endswith(".mix.g")}),
        "router scale": gap(changed(["layers", 1, "mlp", "router", "scale"], 2.0)),
        "one expert more": gap(changed(["layers", 3, "mlp", "router", "top"], 4)),
        "no groups": gap(changed(["layers", 1, "mlp", "router", "groups"], None)),
        "other groups": gap(changed(["layers", 1, "mlp", "router", "groups"], {"count": 2, "keep": 1})),
        "no correction": gap(changed_tensors=with_tensor("l1.mlp.correction", torch.zeros_like)),
        "no shared expert": gap(changed(["layers", 1, "mlp", "shared"], None)),
        "streams": gap(changed(["streams"], None)),
    }
    monkeypatch.setattr(plain, "identity_expert", lambda h: torch.zeros_like(h))
    faults["silent identity experts"] = gap()
    monkeypatch.undo()
    plain_norm = plain.rms_norm
    monkeypatch.setattr(plain, "rms_norm", lambda x, w, eps, offset=0.0: plain_norm(x, w, eps, 0.0))
    faults["norm weights not around zero"] = gap()
    monkeypatch.undo()
    plain_rotate = plain.rotate_interleaved

    def halves(x, positions, dims, base):
        order = list(range(0, dims, 2)) + list(range(1, dims, 2)) + list(range(dims, x.shape[-1]))
        back = torch.tensor(order).argsort()
        return plain_rotate(x[..., back], positions, dims, base)[..., order]

    monkeypatch.setattr(plain, "rotate_interleaved", halves)
    faults["pairs (i, i + half)"] = gap()
    monkeypatch.undo()
    plain_softmax = torch.softmax

    def route_with_corrected_weights(h, router, correction, r, margins=None):
        chosen, _ = plain_route(h, router, correction, r)
        scores = plain_softmax(h @ router.double().T, dim=-1) + correction.double()
        weights = scores.gather(1, chosen)
        return chosen, weights / (weights.sum(dim=-1, keepdim=True) + 1e-20) * r["scale"]

    plain_route = plain.route
    monkeypatch.setattr(plain, "route", route_with_corrected_weights)
    faults["the correction in the weights"] = gap()
    monkeypatch.undo()
    assert gap() <= tol
    # bfloat16's tolerance is a thousand times wider: there the coarse faults must show, in float32 all of them
    coarse = ("mix matrix transposed", "head gates", "streams", "silent identity experts", "norm weights not around zero",
              "pairs (i, i + half)", "the correction in the weights")
    unseen = {what: value for what, value in faults.items() if (dtype == torch.float32 or what in coarse) and not value > 1.5 * tol}
    assert not unseen, f"the plain model with these faults is within 1.5 x the tolerance {tol}: {unseen}"
