"""Finezen on the GPU: every mechanism against the plain implementation, then whole models
through the step function under every kind of schedule, the scheduler and the trace program."""

import copy

import pytest
import torch

import finezen_helpers as fh
import helpers
from plain import finezen_plain as plain

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


dev = lambda t: t.to(DEV).contiguous()


# --------------------------------------------------------------------------- #
# Mechanisms alone
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, width, planes", [(1, 48, 1), (7, 64, 3), (5, 257, 1), (300, 1024, 2)])
def test_norm_without_statistics_alone_and_with_the_sum_before_it(dtype, tokens, width, planes):
    """The read alone; the write x + m * norm_b(y) alone; both in one kernel (the same bits); a
    sublayer's output that is still the planes of a split product; a second stream that joins."""
    ops = _ops()
    gen = torch.Generator().manual_seed(tokens + width)
    x = torch.randn(tokens, width, generator=gen) * 2.0
    parts = torch.randn(planes, tokens, width, generator=gen)
    extra = torch.randn(tokens, width, generator=gen)
    names = {}
    for n in ("a", "b"):
        names.update({n: torch.randn(width, generator=gen), f"{n}.alpha": torch.rand((), generator=gen) + 0.3,
                      f"{n}.b": torch.randn(width, generator=gen) * 0.3})
    norm = lambda n: (dev(names[f"{n}.alpha"].reshape(1)), dev(names[n]), dev(names[f"{n}.b"]))
    mult = 0.7
    y = parts.double().sum(0)
    want_new = x.double() + mult * plain.dynamic_tanh(y, names, "b")
    _close(ops.dyt_norm(dev(x), *norm("a"), dtype), plain.dynamic_tanh(x.double(), names, "a"), dtype)
    sublayer = lambda: ops.PendingSum(dev(parts), None, None, torch.float32) if planes > 1 else dev(parts[0])
    pending = ops.residual_add(dev(x), sublayer(), mult, norm("b"))
    new = ops.materialized(pending)
    _close(new, want_new, torch.float32)
    pending = ops.residual_add(dev(x), sublayer(), mult, norm("b"))
    fused = ops.dyt_norm(pending, *norm("a"), dtype)
    assert pending.value is not None and torch.equal(pending.value, new)
    assert torch.equal(fused, ops.dyt_norm(new, *norm("a"), dtype))
    _close(fused, plain.dynamic_tanh(want_new, names, "a"), dtype)
    # a stream that joins: alone, and taken along by a pending sum
    joined = ops.join_stream(dev(x), dev(extra))
    _close(ops.materialized(joined), x.double() + extra.double(), torch.float32)
    pending = ops.join_stream(ops.residual_add(dev(x), sublayer(), mult, norm("b")), dev(extra))
    got = ops.dyt_norm(pending, *norm("a"), dtype)
    _close(pending.value, want_new + extra.double(), torch.float32)
    _close(got, plain.dynamic_tanh(want_new + extra.double(), names, "a"), dtype)
    # without a norm after the sublayer the output is added as it is
    _close(ops.materialized(ops.residual_add(dev(x), dev(parts[0]), 2.0)), x.double() + 2.0 * parts[0].double(), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, d, dv, dims, tokens", [(4, 2, 12, 20, 8, 5), (6, 2, 128, 96, 64, 70), (3, 3, 10, 6, 10, 9), (1, 1, 8, 8, 0, 3)])
def test_query_and_key_norm_over_the_whole_projection(dtype, heads, kv_heads, d, dv, dims, tokens):
    """One RMS norm over all query heads of a token and one over all its key heads, weights as long
    as the projections, then the rotation of each head's leading span, against the plain functions."""
    ops = _ops()
    gen = torch.Generator().manual_seed(heads * d)
    width = (heads + kv_heads) * d + kv_heads * dv
    proj = torch.randn(tokens, width, generator=gen)
    proj[:, : heads * d] *= torch.linspace(0.2, 3.0, heads * d)          # heads of unequal size: a per-head norm would differ
    qw, kw = torch.rand(heads * d, generator=gen) + 0.5, torch.rand(kv_heads * d, generator=gen) + 0.5
    positions = list(range(3, 3 + tokens))
    rot = {"dims": dims, "base": 50.0, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}} if dims else None
    q = plain.rms_norm(proj[:, : heads * d].double(), qw, 1e-5).view(tokens, heads, d)
    k = plain.rms_norm(proj[:, heads * d: (heads + kv_heads) * d].double(), kw, 1e-5).view(tokens, kv_heads, d)
    table = None
    if rot:
        q, k = plain.rotate_half(q, positions, rot), plain.rotate_half(k, positions, rot)
        freqs, amplitude = plain.yarn_frequencies(dims, rot["base"], rot["scaling"])
        table = ops.rotary_table(dev(torch.tensor(positions, dtype=torch.int32)), dev(torch.tensor(freqs, dtype=torch.float64).float()), amplitude)
    page = 4
    keys = torch.zeros(tokens // page + 2, kv_heads, page, d, dtype=dtype, device=DEV)
    values = torch.zeros(tokens // page + 2, kv_heads, page, dv, dtype=dtype, device=DEV)
    slots = torch.arange(page, page + tokens, dtype=torch.int32, device=DEV)           # from the second page on
    got = ops.head_prep(dev(proj), q_off=0, k_off=heads * d, v_off=(heads + kv_heads) * d, heads=heads, kv_heads=kv_heads,
                        q_dim=d, k_dim=d, value_dim=dv, q_norm=dev(qw), k_norm=dev(kw), q_span=d, k_span=d, eps=1e-5, table=table,
                        interleaved=False, q_rot0=0, k_rot0=0, slots=slots, keys=keys, values=values, page_size=page,
                        out_dtype=dtype, whole=True)
    _close(got.view(tokens, heads, d), q, dtype)
    stored = keys.permute(0, 2, 1, 3).reshape(-1, kv_heads, d)[page: page + tokens]
    _close(stored, k, dtype)
    stored = values.permute(0, 2, 1, 3).reshape(-1, kv_heads, dv)[page: page + tokens]
    _close(stored, proj[:, (heads + kv_heads) * d:].view(tokens, kv_heads, dv), dtype)


@pytest.mark.parametrize("total, top, extra", [(4, 2, 0), (12, 1, 1), (7, 7, 3), (40, 8, 1), (96, 3, 0)])
def test_router_with_sigmoid_scores_taken_as_they_are(total, top, extra):
    """The chosen experts' sigmoids are the weights, not renormalized; the router's outputs may be the
    leading columns of wider rows; planes of a split product are added by the kernel."""
    ops = _ops()
    gen = torch.Generator().manual_seed(total * 7 + top)
    T = 33
    rows = torch.randn(T, total + extra, generator=gen) * 3.0
    margins = []
    want_chosen, want_weights = plain.route(rows[:, :total].double(), torch.eye(total), top, margins)
    clear = margins[0] > 1e-5
    chosen, weights, _ = ops.route(dev(rows), None, top, score="sigmoid", dense=False, normalize=False, experts=total)
    assert torch.equal(chosen.cpu().long()[clear], want_chosen[clear])
    assert torch.allclose(weights.cpu().double()[clear], want_weights[clear], rtol=2e-5, atol=1e-7)
    planes = torch.randn(3, T, total + extra, generator=gen)
    pending = ops.PendingSum(dev(planes), None, None, torch.float32)
    one = ops.route(dev((planes[0] + planes[1]) + planes[2]), None, top, score="sigmoid", dense=False, normalize=False, experts=total)
    two = ops.route(pending, None, top, score="sigmoid", dense=False, normalize=False, experts=total)
    assert pending.value is None and torch.equal(one[0], two[0]) and torch.equal(one[1], two[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, top, experts, width, ff", [(1, 2, 4, 64, 32), (7, 3, 5, 48, 24), (300, 2, 6, 128, 64), (2500, 1, 3, 64, 40),
                                                             (130, 4, 16, 72, 200), (50, 2, 4, 44, 20)])
def test_gated_experts_weighted_on_their_input(dtype, tokens, top, experts, width, ff):
    """Pairs sorted by expert with rows w * x, gate|up as one grouped product, SiLU x up, the down
    product, the sum without weights over a base behind a sigmoid, against a loop over tokens."""
    ops = _ops()
    gen = torch.Generator().manual_seed(tokens + top)
    x = torch.randn(tokens, width, generator=gen).to(dtype)
    favour = torch.rand(tokens, experts, generator=gen)
    favour[:, 0] += 0.5
    if experts > 2:
        favour[:, experts - 1] = -1.0                      # an expert without pairs
    chosen = favour.topk(top, dim=1).indices.int()
    weights = torch.rand(tokens, top, generator=gen) * 0.9 + 0.1
    gate = (torch.randn(experts, ff, width, generator=gen) * 0.2).to(dtype)
    up = (torch.randn(experts, ff, width, generator=gen) * 0.2).to(dtype)
    down = (torch.randn(experts, width, ff, generator=gen) * 0.2).to(dtype)
    base = torch.randn(tokens, width, generator=gen)
    gate_rows = torch.randn(tokens, experts + 1, generator=gen) * 2.0
    want = base.double() * torch.sigmoid(gate_rows[:, experts].double())[:, None]
    for t in range(min(tokens, 400)):
        for k in range(top):
            e = int(chosen[t, k])
            h = float(weights[t, k]) * x[t].double()
            if dtype == torch.bfloat16:
                h = h.to(torch.bfloat16).double()           # the staged row is rounded once
            g = gate[e].double() @ h
            want[t] += down[e].double() @ (g * torch.sigmoid(g) * (up[e].double() @ h))
    plan = ops.expert_plan(dev(x), dev(chosen), experts, dev(weights))
    hidden = ops.silu_mul(ops.linear_grouped(plan.staged, dev(torch.cat([gate, up], dim=1)), plan))
    y = ops.linear_grouped(hidden, dev(down), plan, out_dtype=torch.float32)
    got = ops.expert_combine(y, plan, None, dev(x), dev(base), base_gate=(dev(gate_rows), experts))
    n = min(tokens, 400)
    _close(got[:n], want[:n], dtype, scale=2.0)
    # gate and up rows in alternating blocks of 16: SiLU x up in the product's own epilogue where the
    # tensor-core kernel takes the shape, by the stand-alone kernel elsewhere; the same numbers
    if ff % 16 == 0:
        mixed = torch.stack([ops.interleave_gate_up(dev(gate[e]), dev(up[e])) for e in range(experts)])
        fused = ops.linear_grouped(plan.staged, mixed, plan, swiglu_block=ops.SWIGLU_BLOCK)
        pairs = plan.rows.flatten().long()
        _close(fused[pairs], hidden[pairs].double().cpu(), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, d, dv, window, page, requests", [
    (4, 64, 64, 24, 16, [(0, 70)]),                                   # a prompt from its first token, past the window
    (3, 32, 16, 100, 16, [(150, 1), (37, 40), (200, 1), (0, 1)]),     # single tokens far in, a portion, a first token
    (33, 48, 48, 1, 8, [(20, 3), (64, 1)]),                           # more heads than a block's rows; a window of one
    (2, 288, 288, 65, 32, [(130, 2), (63, 66)]),                      # a wide latent; windows that end at and beside tile borders
    (5, 20, 12, 30, 4, [(90, 1), (10, 50)]),                          # sizes that only the CUDA-core kernel takes
])
def test_windowed_attention_over_latent_rows(dtype, heads, d, dv, window, page, requests):
    """Many heads over ONE cached row per token whose leading channels are its value, with a
    window: prompts, portions and single tokens in one step, over a shuffled block table whose
    entries before every window are gone (-1) and whose pool holds NaN in every page that no request holds."""
    ops = _ops()
    gen = torch.Generator().manual_seed(heads * d + window)
    scale = 0.6 / d ** 0.5
    total_pages = sum(-(-(past + new) // page) for past, new in requests) + 3
    order = torch.randperm(total_pages, generator=gen).tolist()
    pool = torch.full((total_pages, 1, page, d), float("nan"))
    width = max(-(-(past + new) // page) for past, new in requests)
    table = torch.full((len(requests), width), -1, dtype=torch.int32)
    q_rows, want_rows, q_start, q_pos0, kv_len = [], [], [0], [], []
    for b, (past, new) in enumerate(requests):
        n = past + new
        rows = torch.randn(n, 1, d, generator=gen).to(dtype).double()
        q = torch.randn(n, heads, d, generator=gen).to(dtype).double()
        want_rows.append(plain.windowed_softmax_attention(q, rows, rows[:, :, :dv], scale, window)[past:])
        q_rows.append(q[past:])
        first_seen = max(0, past - window + 1)
        for index in range(first_seen // page, -(-n // page)):
            table[b, index] = order.pop()
        for pos in range(first_seen // page * page, n):  # pages that no query of the step sees stay NaN
            pool[table[b, pos // page], 0, pos % page] = rows[pos, 0].float()
        q_start.append(q_start[-1] + new)
        q_pos0.append(past)
        kv_len.append(n)
    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
    keys = dev(pool.to(dtype))
    singles = sum(1 for _, new in requests if new == 1)
    got = ops.paged_attention_scored(
        dev(torch.cat(q_rows).to(dtype).view(-1, heads * d)), keys, keys, dev(table), ints(q_start), ints(q_pos0), ints(kv_len), heads, 1,
        d, dv, page, max(new for _, new in requests), scale, window=window, max_kv_len=max(kv_len), num_single=singles)
    want = torch.cat(want_rows).view(-1, heads * dv)
    assert bool(torch.isfinite(got).all())
    _close(got, want, dtype)


# --------------------------------------------------------------------------- #
# Single parts of a model against the plain functions
# --------------------------------------------------------------------------- #

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("finezen")
    return {name: fh.write_model(root / name, raw, seed) for name, (raw, _page, seed) in fh.SMALL.items()}


@pytest.fixture(scope="module")
def prompts(folders):
    """Per model: prompts whose routers' choices are clear, and the plain model's logits for them."""
    return {name: fh.clear_requests(folders[name], [45, 9, 31, 2, 23], seed) for name, (_raw, _page, seed) in fh.SMALL.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, index", [("small_a", 0), ("small_a", 1), ("small_a", 3), ("small_a", 4), ("small_b", 0), ("small_b", 1), ("one_layer_loop", 0)])
def test_routed_feed_forward_alone(folders, name, index, dtype):
    from paged_attention_engine_b200.config import resolve
    from paged_attention_engine_b200.parts import FEED_FORWARDS, Runtime

    raw, tensors = fh.read_model(folders[name])
    spec = resolve(raw)[1].layers[index].feed_forward
    mlp = raw["layers"][index]["mlp"]
    gen = torch.Generator().manual_seed(index)
    h = torch.randn(90, raw["width"], generator=gen).to(dtype)
    margins = []
    want = plain.mixture(h.double(), tensors, f"l{index}.mlp", mlp, margins)
    clear = margins[0] > fh.CLEAR_CHOICE
    assert int(clear.sum()) > 30
    runtime = Runtime(_ops(), dtype, torch.device(DEV))
    own = {k: (v.float() if v.dim() == 1 else v.to(dtype)).to(DEV) for k, v in tensors.items() if k.startswith(f"l{index}.mlp.")}
    part = FEED_FORWARDS.get(spec.kind)(spec, own, runtime)
    got = _ops().materialized(part.forward(None, h.to(DEV), None))
    assert got.dtype == torch.float32
    _close(got[clear.to(DEV)], want[clear], dtype, scale=3.0)


# --------------------------------------------------------------------------- #
# Whole models through the step function
# --------------------------------------------------------------------------- #

def _check(folder, dtype, trace, requests, oracle, page, max_live=4, fragment=None, slack=1.0):
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
        allowed = slack * fh.row_tolerance(dtype, want, folder, requests[key])
        worst = int((gap - allowed).argmax())
        assert bool((gap <= allowed).all()), f"{key}: |dlogit| {float(gap[worst])} > {float(allowed[worst])} at position {worst}"
    assert not replayer.manager.live_requests()
    assert replayer.manager.num_free == replayer.manager.num_blocks
    return got


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(fh.SMALL))
def test_schedules_agree_with_the_plain_model(folders, prompts, name, dtype):
    raw, page, seed = fh.SMALL[name]
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
def test_long_decoding_past_every_window(folders, dtype):
    raw, page, seed = fh.SMALL["small_b"]
    requests, oracle = fh.clear_requests(folders["small_b"], [150], seed + 50)
    _check(folders["small_b"], dtype, helpers.trace_tail(requests, tail=140), requests, oracle, page)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_over_many_pages(tmp_path, dtype):
    """400 tokens over 25 pages, windows of 130 and 100 keys that pass over prompt and decoded
    tokens alike, both layers run twice; every expert is chosen, so no router's choice can be a
    close call. Head sizes that the tensor-core attention kernels take in bfloat16."""
    raw = fh.config(131, 64, [
        fh.layer(fh.attention(4, 2, 32, 32, 0.18, window=130, rot=fh.rot(16, 10000.0, (4.0, 64, 16.0, 1.0))), fh.moe(32, 3, 3, shared=48)),
        fh.layer(fh.latent(4, 16, 32, 48, 40, 0.25, window=100), fh.moe(48, 2, 2)),
    ], scale=1.5, mult=0.9, loop=(0, 2, 2))
    folder = fh.write_model(tmp_path / "long", raw, 61)
    gen = torch.Generator().manual_seed(8)
    requests = {"r0": torch.randint(0, 131, (400,), generator=gen).tolist()}
    config, tensors = fh.read_model(folder)
    oracle = {"r0": plain.forward(config, tensors, requests["r0"]).float()}
    whole = _check(folder, dtype, helpers.trace_whole(requests), requests, oracle, 16)
    tail = _check(folder, dtype, helpers.trace_tail(requests, tail=160), requests, oracle, 16)
    chunks = _check(folder, dtype, helpers.trace_chunks(requests, 4), requests, oracle, 16, fragment=9)
    cut = (2e-5 if dtype == torch.float32 else 2.0 ** -6) * max(1.0, float(oracle["r0"].abs().max()))
    for other in (tail, chunks):
        assert float((other["r0"] - whole["r0"]).abs().max()) <= cut


WINDOWS = (24, 19)          # of the attention layer and of the latent layer below


def _edge_model(tmp_path):
    """Two layers, one of each attention, without feed-forwards, and a prompt with ONE token that
    stands out in both. Only its embedding has channel 0, and channel 1 is 0 in every embedding, so
    that after the first norm (bias 0 on channel 0, 1 on channel 1) channel 0 is this token's alone
    and channel 1 is the same constant for all. In the attention layer an unrotated key channel
    reads channel 0 and the same channel of every query head reads channel 1, both with large norm
    weights: every query's score with this token's key is far above the others'. In the latent layer
    the latent's first channel reads channel 0 alone and its norm weight is large. The token's value
    is several times any other's, the output projections are scaled up, the gates are near one half.
    Every query that sees the token gives it most of its weight; the first query that does NOT see
    it, a window further on, differs visibly from a model whose window is one longer."""
    from safetensors.torch import load_file, save_file

    raw = fh.config(61, 64, [
        fh.layer(fh.attention(2, 1, 16, 16, 0.25, window=WINDOWS[0], rot=fh.rot(8, 10000.0)), None),
        fh.layer(fh.latent(2, 16, 16, 32, 24, 0.25, window=WINDOWS[1]), None)], scale=1.0, mult=1.0)
    folder = fh.write_model(tmp_path / "edge", raw, 77)
    path = str(folder / "model.safetensors")
    tensors = load_file(path)
    for name, change in (("embed", lambda t: (t[:, 0].zero_(), t[:, 1].zero_(), t[60].mul_(5.0), t[60, 0].fill_(3.0))),
                         ("l0.norm1", lambda t: t[0].fill_(1.0)),
                         ("l0.norm1.b", lambda t: (t[0].zero_(), t[1].fill_(1.0))),
                         ("l0.mix.k", lambda t: (t[8].zero_(), t[8, 0].fill_(4.0))),
                         ("l0.mix.q", lambda t: (t[8].zero_(), t[8, 1].fill_(2.0), t[24].zero_(), t[24, 1].fill_(2.0))),
                         ("l0.mix.k.norm", lambda t: t[8].fill_(3.0)),
                         ("l0.mix.q.norm", lambda t: (t[8].fill_(3.0), t[24].fill_(3.0))),
                         ("l0.mix.sink", lambda t: t.fill_(-2.0)),
                         ("l1.mix.dkv", lambda t: (t[0].zero_(), t[0, 0].fill_(4.0))),
                         ("l1.mix.dkv.norm", lambda t: t[0].fill_(30.0)),
                         ("l0.mix.o", lambda t: t.mul_(80.0)), ("l1.mix.o", lambda t: t.mul_(80.0)),
                         ("l0.mix.g", lambda t: t.mul_(0.05)), ("l1.mix.g", lambda t: t.mul_(0.05))):
        t = tensors[name].float()
        change(t)
        tensors[name] = t.to(torch.bfloat16)
    save_file(tensors, path)
    return raw, folder, tensors


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("at, decoded", [(5, False), (5, True), (40, True), (0, False)])
def test_keys_just_inside_and_just_outside_each_window(tmp_path, dtype, at, decoded):
    """The outstanding token stands at position `at` (the very first token; inside the first page;
    beyond a page border); the queries at the windows' edges come in a prompt's portion or one by
    one. The logits follow the plain model, and at the edges they are far from the plain model whose
    window is one token longer or shorter. (This model's output projections are scaled up eighty
    times to make one key's presence a matter of six tolerances; the bfloat16 engine's own rounding
    grows with them, to up to 1.4 tolerances here, so it is given two.)"""
    raw, folder, tensors = _edge_model(tmp_path)
    gen = torch.Generator().manual_seed(5 + at)
    tokens = torch.randint(0, 60, (90,), generator=gen).tolist()
    tokens[at] = 60
    want = plain.forward(raw, tensors, tokens).float()
    requests = {"r0": tokens}
    trace = helpers.trace_tail(requests, tail=90 - at - 10) if decoded else helpers.trace_chunks(requests, 3)
    slack = 1.0 if dtype == torch.float32 else 2.0
    got = _check(folder, dtype, trace, requests, {"r0": want}, 16, slack=slack)["r0"]
    tol = fh.tolerance(torch.bfloat16, want)
    for layer, window in enumerate(WINDOWS):
        for delta in (-1, 1):
            other = copy.deepcopy(raw)
            other["layers"][layer]["mixer"]["mask"]["size"] = window + delta
            wrong = plain.forward(other, tensors, tokens).float()
            edge = at + window - 1 + (1 if delta > 0 else 0)        # the last query that sees it; the first that does not
            assert float((wrong[edge] - got[edge]).abs().max()) > 4.0 * tol, (layer, delta)
            assert float((want[edge] - got[edge]).abs().max()) <= slack * tol


def _plain_greedy(folder, prompt, count):
    raw, tensors = fh.read_model(folder)
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain.forward(raw, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small_b", "no_loop"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from paged_attention_engine_b200 import LLM, Request

    raw, page, seed = fh.SMALL[name]
    llm = LLM.from_pretrained(folders[name], dtype=str(dtype).replace("torch.", ""), num_blocks=48, block_size=page,
                              max_num_seqs=4, max_num_batched_tokens=16, record_logits=True)
    prompts, _ = fh.clear_requests(folders[name], [5, 21, 12], seed + 20)
    for i, prompt in enumerate(prompts.values()):
        assert llm.add_request(Request(f"g{i}", tuple(prompt), 7))
    out = llm.run_to_completion()
    raw_config, tensors = fh.read_model(folders[name])
    for i, prompt in enumerate(prompts.values()):
        tokens = list(out[f"g{i}"])
        assert len(tokens) == 7
        margins = []
        want = plain.forward(raw_config, tensors, prompt + tokens, margins=margins).float()[len(prompt) - 1: -1]
        got = torch.stack(llm.scheduler.finished[f"g{i}"].step_logits)
        # generated tokens were not drawn for clear choices: compare up to the first close call
        close = (torch.stack(margins).min(dim=0).values < fh.CLEAR_CHOICE).nonzero() if margins else []
        clear_until = int(close[0]) if len(close) else len(prompt) + 7
        rows = max(0, min(7, clear_until - (len(prompt) - 1)))
        assert rows >= 1
        assert float((got[:rows] - want[:rows]).abs().max()) <= fh.tolerance(dtype, want)
        if dtype == torch.float32 and rows == 7:
            assert tokens == _plain_greedy(folders[name], prompt, 7)


def test_trace_program_on_a_random_model(folders, prompts, tmp_path):
    raw, page, seed = fh.SMALL["small_a"]
    requests, oracle = prompts["small_a"]
    requests = {k: requests[k] for k in ("r1", "r2", "r4")}
    trace = helpers.trace_mixed(requests, seed, live_limit=2, decode_tail=6)
    outputs = helpers.run_trace_program(folders["small_a"], "bfloat16", trace, helpers.max_live_tokens(trace, page),
                                        tmp_path / "out", raw["vocab"], block_size=page)
    got = helpers.collect(trace, outputs, requests)
    for key in requests:
        allowed = fh.row_tolerance(torch.bfloat16, oracle[key], folders["small_a"], requests[key])
        assert bool(((got[key] - oracle[key]).abs().max(dim=1).values <= allowed).all())


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_tolerance_notices_a_fault_in_any_mechanism(folders, prompts, dtype, monkeypatch):
    """The plain model with one mechanism changed leaves the tolerance around the engine's logits:
    the comparisons above could tell."""
    raw, page, seed = fh.SMALL["small_a"]
    requests, oracle = prompts["small_a"]
    requests, oracle = {"r0": requests["r0"]}, {"r0": oracle["r0"]}
    got = _check(folders["small_a"], dtype, helpers.trace_whole(requests), requests, oracle, page)["r0"]
    config, tensors = fh.read_model(folders["small_a"])
    tol = fh.tolerance(dtype, oracle["r0"])

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
        "score scale": gap(changed(["layers", 0, "mixer", "scale"], 0.2)),
        "rotation base": gap(changed(["layers", 0, "mixer", "rot", "base"], 500.0)),
        "rotated channels": gap(changed(["layers", 2, "mixer", "rot", "dims"], 6)),
        "no frequency scaling": gap(changed(["layers", 0, "mixer", "rot", "scaling"], None)),
        "window one longer": gap(changed(["layers", 0, "mixer", "mask", "size"], 8)),
        "window one shorter": gap(changed(["layers", 0, "mixer", "mask", "size"], 6)),
        "latent window one longer": gap(changed(["layers", 1, "mixer", "mask", "size"], 22)),
        "latent window one shorter": gap(changed(["layers", 1, "mixer", "mask", "size"], 20)),
        "no sink": gap(changed_tensors=with_tensor("l0.mix.sink", lambda t: t - 40.0)),
        "a sink of logit 0": gap(changed_tensors=with_tensor("l2.mix.sink", torch.zeros_like)),
        "query norm weight": gap(changed_tensors=with_tensor("l0.mix.q.norm", torch.ones_like)),
        "query latent's norm weight": gap(changed_tensors=with_tensor("l1.mix.dq.norm", torch.ones_like)),
        "norm slope": gap(changed_tensors=with_tensor("l1.norm1.alpha", lambda t: t * 1.5)),
        "norm bias": gap(changed_tensors=with_tensor("l3.norm2b.b", torch.zeros_like)),
        "residual multiplier": gap(changed(["residual_mult"], 1.0)),
        "embedding scale": gap(changed(["embedding", "scale"], 1.0)),
        "one pass fewer": gap(changed(["loop", "times"], 2)),
        "another span of the loop": gap(changed(["loop", "stop"], 4)),
        "one expert more": gap(changed(["layers", 1, "mlp", "router", "top"], 4)),
        "no shared expert": gap(changed(["layers", 0, "mlp", "shared"], None)),
        "shared gate": gap(changed_tensors=with_tensor("l3.mlp.shared.sg", torch.zeros_like)),
    }
    monkeypatch.setattr(plain, "head_gates", lambda h, w: torch.ones(h.shape[0], w.shape[0], 1, dtype=torch.float64))
    faults["head gates"] = gap()
    monkeypatch.undo()
    plain_norm = plain.rms_norm

    def per_head(x, weight, eps):
        # a norm per head instead of one over the whole projection, where the weight is as long as a projection
        if weight.numel() in (48, 24, 60, 30):
            size = {48: 12, 24: 12, 60: 10, 30: 10}[weight.numel()]
            return plain_norm(x.view(x.shape[0], -1, size), torch.ones(size), eps).reshape(x.shape) * weight.double()
        return plain_norm(x, weight, eps)

    monkeypatch.setattr(plain, "rms_norm", per_head)
    faults["a norm per head"] = gap()
    monkeypatch.undo()
    plain_rotate = plain.rotate_half

    def interleaved(x, positions, rot):
        dims = rot["dims"]
        order = list(range(0, dims, 2)) + list(range(1, dims, 2)) + list(range(dims, x.shape[-1]))
        back = torch.tensor(order).argsort()
        return plain_rotate(x[..., order], positions, rot)[..., back]

    monkeypatch.setattr(plain, "rotate_half", interleaved)
    faults["pairs (2i, 2i + 1)"] = gap()
    monkeypatch.undo()
    plain_expert = plain.gated_expert
    plain_route = plain.route

    def weight_on_output(h, tensors_, prefix, mlp, margins=None):
        chosen, weights = plain_route(h, tensors_[f"{prefix}.router"], mlp["router"]["top"])
        out = torch.zeros_like(h)
        for t in range(h.shape[0]):
            for e, w in zip(chosen[t].tolist(), weights[t]):
                out[t] += w * plain_expert(h[t: t + 1], tensors_, f"{prefix}.e{e}")[0]
        if mlp.get("shared"):
            out = out + plain_expert(h, tensors_, f"{prefix}.shared") * torch.sigmoid(h @ tensors_[f"{prefix}.shared.sg"].double().T)
        return out

    monkeypatch.setattr(plain, "mixture", weight_on_output)
    faults["weights on the experts' outputs"] = gap()
    monkeypatch.undo()

    def renormalized(h, router, top, margins=None):
        chosen, weights = plain_route(h, router, top)
        return chosen, weights / weights.sum(dim=-1, keepdim=True)

    monkeypatch.setattr(plain, "route", renormalized)
    faults["weights renormalized"] = gap()
    monkeypatch.undo()
    plain_runs = plain.layer_runs
    monkeypatch.setattr(plain, "layer_runs", lambda raw_: [(i, False) for i, _ in plain_runs(raw_)])
    faults["the embedding does not join again"] = gap()
    monkeypatch.undo()
    assert gap() <= tol
    # bfloat16's tolerance is a thousand times wider: there the coarse faults must show, in float32 all of them
    coarse = ("head gates", "residual multiplier", "embedding scale", "one pass fewer", "the embedding does not join again")
    unseen = {what: value for what, value in faults.items() if (dtype == torch.float32 or what in coarse) and not value > 1.5 * tol}
    assert not unseen, f"the plain model with these faults is within 1.5 x the tolerance {tol}: {unseen}"
