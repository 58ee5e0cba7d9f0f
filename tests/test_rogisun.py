"""The Rogisun decoder in the engine against the plain implementation of tests/plain/rogisun_plain.py.

Every test runs on the CPU over the torch stand-ins of the kernels (which checks the parts, the cache and state
manager, the step function and the scheduler) and, marked gpu, on the real kernels in float32 and bfloat16.
"""
import math

import pytest
import torch

from serve_b200.cache import CacheManager
from serve_b200.config import ConfigError, PartSpec, build_spec, config_from_dict
from serve_b200.engine.step import BatchShape, StepContext
from serve_b200.parts import build_part
from tests import helpers
from tests.plain import rogisun_plain as P
from tests.rogisun_cases import BACKENDS, CONFIGS, compare_rows, make_engine, make_weights, plain_logits, runtime_for, settled_weights, tolerance, write_model

LENGTHS = {"p": [1, 5, 23, 49, 75, 130], "q": [2, 9, 31, 64, 101], "o": [3, 40, 90]}
PAGE = {"p": 8, "q": 16, "o": 4}


# ---- configuration and description ----------------------------------------------------------------------------
def test_configuration_is_read_from_the_file_and_describes_every_layer():
    from serve_b200.weights.random_init import model_tensor_decls

    for name, raw in CONFIGS.items():
        cfg = config_from_dict(raw)
        assert type(cfg).__name__ == "RogisunConfig" and cfg.width == raw["width"] and cfg.canon_taps == raw["canon"]["taps"]
        spec = build_spec(cfg)
        assert [l.parts["mixer"].kind for l in spec.layers] == [l["type"] for l in raw["layers"]]
        assert [("feed_forward" in l.parts) for l in spec.layers] == [l["mlp"] is not None for l in raw["layers"]]
        decls = {n: tuple(d.shape) for n, d in model_tensor_decls(cfg).items()}
        assert decls == P.tensor_shapes(raw)
        assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("breaker", [
    lambda c: c["layers"][0].update(type="other"),
    lambda c: c["layers"][0]["mixer"].pop("heads"),
    lambda c: c.pop("canon"),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=99),
    lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3),
])
def test_configuration_refuses_what_it_cannot_run(breaker):
    import copy

    raw = copy.deepcopy(CONFIGS["p"])
    breaker(raw)
    with pytest.raises(ConfigError):
        config_from_dict(raw)


def test_a_file_decides_the_width_of_the_two_step_projections(tmp_path):
    """Without a rank in the configuration the delta-rule mixer takes it from the shapes in the file."""
    import copy

    raw = copy.deepcopy(CONFIGS["q"])
    w = make_weights(raw, 3)
    folder = write_model(str(tmp_path / "m"), raw, w)
    del raw["layers"][0]["mixer"]["right"]["rank"]
    import json, os

    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    eng = make_engine(folder, ("emu", "float32"), 16, 8)
    toks = helpers.random_tokens(raw["vocab"], 12, 1)
    got = helpers.replay(eng, helpers.trace_whole({"a": toks}))
    helpers.compare_with_plain(got, {"a": plain_logits(w, CONFIGS["q"], toks)}, atol=2e-4)


# ---- whole models under every way of cutting the work ------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{config name: {dtype: (weights, requests, plain logits, model folder)}}; the bfloat16 models have damped experts
    (rogisun_cases.settled_weights says why)."""
    out = {}
    for name in LENGTHS:
        cfg = CONFIGS[name]
        reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=20 + i) for i, n in enumerate(LENGTHS[name])}
        out[name] = {}
        for dt, gain in (("float32", 1.0), ("bfloat16", 0.1)):
            w, plain = settled_weights(cfg, reqs, min_margin=0.05 if gain == 1.0 else 0.0, expert_gain=gain)
            out[name][dt] = (w, reqs, plain, write_model(str(tmp_path_factory.mktemp(f"{name}-{dt}")), cfg, w, getattr(torch, dt)))
    return out


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["p", "q", "o"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "single_tokens"])
def test_cuts_match_plain(models, name, backend, cut):
    w, reqs, plain, folder = models[name][backend[1]]
    page = PAGE[name]
    eng = make_engine(folder, backend, page, num_pages=-(-160 // page) * 2, graphs=(cut == "tail_decode"))
    if cut == "single_tokens":
        steps = helpers.trace_tail_decode({k: v for k, v in reqs.items() if len(v) <= 50}, tail=10 ** 6)
    else:
        make = {"whole": helpers.trace_whole, "tail_decode": lambda r: helpers.trace_tail_decode(r, tail=40),
                "portions": lambda r: helpers.trace_portions(r, sizes=(7, 2, 19, 1, 3, 2, 33, 5, 2, 11))}[cut]
        steps = make(reqs)
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    compare_rows(got, plain, backend)
    eng.cache.check()
    assert eng.cache.live == 0


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["p", "q", "o"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, backend):
    """Unequal requests side by side, portions beside single tokens, fewer slots and pages than requests: every
    row must equal the request run alone. Pages and states are poisoned first, so that a page or a state that is
    read without having been written (or cleared) shows."""
    w, reqs, plain, folder = models[name][backend[1]]
    page = PAGE[name]
    steps = helpers.trace_mixed(reqs, live=3, seed=7)
    need = helpers.tokens_needed(steps, page) // page
    assert need < sum(-(-len(t) // page) for t in reqs.values())
    # behind the start of a query's block of positions no key is read again: the cache manager gives those pages back at
    # once, so three live requests get by with what a block and a portion span, far fewer pages than their tokens
    block = max(l["mixer"]["left"]["mask"]["size"] for l in CONFIGS[name]["layers"] if l["type"] == "parallel")
    pool = min(need, 3 * CacheManager.most_pages_of_a_request(None, page, 160, 21, block))
    assert pool < sum(-(-len(t) // page) for t in reqs.values())
    eng = make_engine(folder, backend, page, num_pages=pool, max_slots=3, context=160)
    for view in eng.stepper.views:
        if view.k is not None:
            view.k.fill_(float("nan"))
            view.v.fill_(float("nan"))
        for st in view.states.values():
            st.fill_(float("nan"))
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    compare_rows(got, plain, backend)
    eng.cache.check()
    assert eng.cache.live == 0 and eng.cache.free_slots == 3
    assert max(g.pool.high_water for g in eng.cache.groups) <= pool


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_side_by_side(models, backend):
    """Two requests decoded one token at a time for 120 steps after short prompts (from CUDA graphs on the GPU): the
    states are carried through every step, and the blocks of positions and the pages are crossed many times."""
    cfg = CONFIGS["q"]
    w, _, _, folder = models["q"][backend[1]]
    seqs = {f"d{i}": helpers.random_tokens(cfg["vocab"], 140 - 9 * i, seed=60 + i) for i in range(2)}
    plain = {rid: plain_logits(w, cfg, toks) for rid, toks in seqs.items()}
    eng = make_engine(folder, backend, 16, num_pages=24, graphs=True)
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": t[:11 + 6 * i], "want": [10 + 6 * i]} for i, (rid, t) in enumerate(seqs.items())], "end": []}]
    at = {rid: 11 + 6 * i for i, rid in enumerate(seqs)}
    while any(at[rid] < len(seqs[rid]) for rid in seqs):
        entries = [{"id": rid, "tokens": [t[at[rid]]], "want": [0]} for rid, t in seqs.items() if at[rid] < len(t)]
        for e in entries:
            at[e["id"]] += 1
        steps.append({"step": len(steps), "entries": entries, "end": []})
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    if backend[0] == "cuda":
        assert eng.stepper.launched_graphs > 80
    compare_rows(got, plain, backend)


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_scheduler(models, backend):
    """generate(): the engine's own entry point, scheduler and sampler. Every generated token must be (within the
    tolerance) the best one of the plain model given the tokens before it."""
    from serve_b200.run import Request, generate

    cfg = CONFIGS["p"]
    w, reqs, _, folder = models["p"][backend[1]]
    eng = make_engine(folder, backend, 8, num_pages=40, max_slots=3, budget=32)
    prompts = [reqs["r1"], reqs["r2"], reqs["r3"][:30], reqs["r0"]]
    out = generate(eng, [Request(torch.tensor(p), len(p), 12) for p in prompts], temperature=0.0, eos_token_id=None)
    for p, r in zip(prompts, out):
        new = r.generated_tokens.tolist()
        assert len(new) == 12
        logits = plain_logits(w, cfg, p + new)
        # (bfloat16: single logits of these strongly weighted test models are off by up to a tenth of the scale; the sharp
        # check of the choice is the float32 run)
        tol = float(logits.abs().max()) * (2e-4 if backend[1] == "float32" else 2.0 ** -3)
        for i, tok in enumerate(new):
            row = logits[len(p) - 1 + i]
            assert float(row[tok]) >= float(row.max()) - 2 * tol, f"token {i} of a request is not the plain model's choice"
    assert eng.cache.live == 0


# ---- each mechanism alone ---------------------------------------------------------------------------------------
def _ctx(rt, dev, q_lens, starts, slots, mgr=None, rids=None):
    t = sum(q_lens)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    pos = [s + j for q, s in zip(q_lens, starts) for j in range(q)]
    row = [i for i, q in enumerate(q_lens) for _ in range(q)]
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    kv = [s + q for q, s in zip(q_lens, starts)]
    tables = [torch.from_numpy(mgr.table_rows(g, rids)).to(dev) for g in range(len(mgr.groups))] if mgr is not None else []
    return StepContext(rt=rt, shape=BatchShape(len(q_lens), t, max(q_lens), min(q_lens), max(kv), all(q == 1 for q in q_lens)),
                       tokens=i32([0] * t), positions=i32(pos), token_row=i32(row), cu_q=i32(cu), kv_len=i32(kv), slots=i32(slots),
                       logit_rows=i32([]), block_tables=tables, rids=rids or [])


def _run_part(backend, family, spec, weights, x, cuts, page=8):
    """One part alone over one sequence cut as ``cuts`` says, with a cache manager made for its need; a second request
    runs first in the same slot and is closed, so the slot's state and pages have been used before."""
    rt, dev = runtime_for(backend)
    part = build_part(family, spec, rt)
    names = {d.name for d in part.tensor_decls()}
    part.load({n: weights[n].to(dev).to(rt.act_dtype) for n in names})
    need = part.cache_need() if hasattr(part, "cache_need") else None
    mgr = CacheManager([need], [None], page, 128, 1, 1024, device=dev, kv_dtype=rt.act_dtype)
    view = mgr.views()[0]

    def call(h, ctx):
        if family == "mixer":
            return part.forward(h, ctx, view)
        if family == "filter":
            return part.forward(h, ctx, view)
        return part.forward(h, ctx)

    xs = x.to(dev).to(rt.act_dtype)
    with torch.inference_mode():
        mgr.open("warm")
        mgr.reserve([("warm", 5)])
        call(torch.randn_like(xs[:5]), _ctx(rt, dev, [5], [0], [mgr.slot("warm")], mgr, ["warm"]))
        mgr.close("warm")
        mgr.open("r")
        outs, at = [], 0
        for n in cuts:
            mgr.reserve([("r", at + n)])
            outs.append(call(xs[at: at + n], _ctx(rt, dev, [n], [at], [mgr.slot("r")], mgr, ["r"])).float().cpu())
            mgr.commit("r", at + n)
            at += n
    assert at == x.shape[0]
    rt.kernels.check_errors()
    return torch.cat(outs)


def _tol(backend, want):
    return float(want.abs().max()) * (1e-4 if backend[1] == "float32" else 2.0 ** -6)


def _layer(name, index):
    cfg = CONFIGS[name]
    return cfg, cfg["layers"][index], f"l{index}."


CUTS = [[57], [30, 1, 1, 2, 5, 17, 1], [1] * 57]


def _mixer_case(backend, name, index, cuts, seed=5, x=None, tweak=None):
    from serve_b200.models.rogisun import _mixer_spec

    cfg, layer, p = _layer(name, index)
    w = make_weights(cfg, seed)
    if tweak is not None:
        tweak(w, p + "mix.")
    g = torch.Generator().manual_seed(seed + 1)
    if x is None:
        x = torch.randn(sum(cuts), cfg["width"], generator=g)
    x = x.bfloat16().float()
    spec = _mixer_spec(layer["type"], layer["mixer"], cfg["width"], cfg["norm"]["eps"], p + "mix.")
    got = _run_part(backend, "mixer", spec, w, x, cuts)
    want = P.MIXERS[layer["type"]](x.double(), {k: v.double() for k, v in w.items()}, p + "mix.", layer["mixer"], cfg["norm"]["eps"]).float()
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("where", [("p", 0), ("q", 2)], ids=["p", "q"])
def test_lightning_mixer_alone(backend, cuts, where):
    _mixer_case(backend, where[0], where[1], cuts)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("where", [("p", 2), ("q", 1)], ids=["p", "q"])
def test_mamba2_mixer_alone(backend, cuts, where):
    _mixer_case(backend, where[0], where[1], cuts)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("where", [("p", 1), ("q", 0)], ids=["p", "q"])
def test_parallel_mixer_alone(backend, cuts, where):
    _mixer_case(backend, where[0], where[1], cuts)


@pytest.mark.parametrize("backend", BACKENDS[1:])
@pytest.mark.parametrize("index", [0, 1, 2], ids=["lightning", "mamba2", "parallel"])
@pytest.mark.parametrize("cuts", [[420], [130, 1, 1, 270, 18]], ids=["whole", "portions"])
def test_mixers_at_the_sizes_of_a_real_layer(backend, index, cuts):
    """Each mixer alone at heads of 128 and states of 128 rows, over 420 tokens (the block of 256 positions is crossed, the
    recurrences' staging ring turns many times), whole and cut with single tokens in the middle."""
    _mixer_case(backend, "wide", index, cuts, seed=31)


@pytest.mark.parametrize("backend", BACKENDS[1:])
def test_experts_at_the_sizes_of_a_real_layer(backend):
    from serve_b200.models.rogisun import rogisun_spec

    cfg, layer, p = _layer("wide", 0)
    w = make_weights(cfg, 33)
    spec = rogisun_spec(config_from_dict(cfg)).layers[0].parts["feed_forward"]
    x = torch.randn(700, cfg["width"], generator=torch.Generator().manual_seed(3)).bfloat16().float()
    want = P.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, p + "mlp.", layer["mlp"]).float()
    z = x.double() @ w[p + "mlp.router"].double().T
    keep = (torch.sort(z, descending=True).values[:, 1:3].diff(dim=1).abs() >= 0.08).flatten()      # no close call between 2nd and 3rd
    got = _run_part(backend, "feed_forward", spec, w, x, [700], page=16)
    assert int(keep.sum()) > 550
    torch.testing.assert_close(got[keep], want[keep], atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("side,kind", [("left", "distance_bias_attention"), ("right", "gated_delta")])
@pytest.mark.parametrize("cuts", CUTS[:2], ids=["whole", "portions"])
def test_each_side_of_the_pair_alone(backend, side, kind, cuts):
    from serve_b200.models.rogisun import _mixer_spec

    cfg, layer, p = _layer("q", 0)
    w = make_weights(cfg, 9)
    x = torch.randn(sum(cuts), cfg["width"], generator=torch.Generator().manual_seed(2)).bfloat16().float()
    pair = _mixer_spec("parallel", layer["mixer"], cfg["width"], cfg["norm"]["eps"], p + "mix.")
    spec = pair.params[side]
    assert spec.kind == kind
    got = _run_part(backend, "mixer", spec, w, x, cuts, page=16)
    fn = P.chunked_bias_attention if side == "left" else P.gated_delta_mixer
    want = fn(x.double(), {k: v.double() for k, v in w.items()}, p + f"mix.{side}.", layer["mixer"][side], cfg["norm"]["eps"]).float()
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("far_key,query", [(24, 47), (23, 47), (48, 56), (47, 56), (0, 23), (24, 24)])
@pytest.mark.parametrize("cuts", [[57], [40] + [1] * 17], ids=["prompt", "decoded"])
def test_attention_sees_its_block_of_positions_and_nothing_before(backend, far_key, query, cuts):
    """One key is made to stand out for one query (the query projection is minus the key projection and the query token
    minus three times the key token, so the query points along that key and away from its own): if the key lies in the query's block of 24 positions it takes nearly all the weight, one position
    before the block's start it must have none. Positions 23|24 and 47|48 are block edges; pages are 8 tokens, so 24 and
    48 are page borders as well, and 47 -> 24 is the farthest key a query ever reads."""
    from serve_b200.models.rogisun import _mixer_spec

    cfg, layer, p = _layer("p", 1)
    left = p + "mix.left."

    def tweak(w, prefix):
        d, kvh, heads = layer["mixer"]["left"]["dim"], layer["mixer"]["left"]["kv_heads"], layer["mixer"]["left"]["heads"]
        wk = w[left + "k"].view(kvh, d, -1)
        w[left + "q"] = -wk.repeat_interleave(heads // kvh, 0).reshape(heads * d, -1).clone()
        w[left + "g"] = w[left + "g"] * 0                # every gate at one half

    x = torch.randn(57, cfg["width"], generator=torch.Generator().manual_seed(4)) * 0.3
    x[far_key] = torch.randn(cfg["width"], generator=torch.Generator().manual_seed(5)) * 1.5
    if query != far_key:
        x[query] = -3.0 * x[far_key]
    pair = _mixer_spec("parallel", layer["mixer"], cfg["width"], cfg["norm"]["eps"], p + "mix.")
    w = make_weights(cfg, 11)
    tweak(w, None)
    xb = x.bfloat16().float()
    got = _run_part(backend, "mixer", pair.params["left"], w, xb, cuts)
    w64 = {k: v.double() for k, v in w.items()}
    want = P.chunked_bias_attention(xb.double(), w64, left, layer["mixer"]["left"], cfg["norm"]["eps"]).float()
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)
    # the test's own premise: with the key visible the query's output differs a lot from the output without it
    hidden = dict(layer["mixer"]["left"], mask={"size": 10 ** 6})
    if far_key // 24 != query // 24:
        other = P.chunked_bias_attention(xb.double(), w64, left, hidden, cfg["norm"]["eps"]).float()
        assert float((other[query] - want[query]).abs().max()) > 20 * _tol(backend, want)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name,index", [("p", 0), ("p", 2), ("q", 0), ("q", 2)])
def test_routed_experts_alone(backend, name, index):
    from serve_b200.models.rogisun import rogisun_spec

    cfg, layer, p = _layer(name, index)
    w = make_weights(cfg, 13)
    spec = rogisun_spec(config_from_dict(cfg)).layers[index].parts["feed_forward"]
    for seed in range(50):              # inputs on which no router decision is a close call
        x = torch.randn(70, cfg["width"], generator=torch.Generator().manual_seed(seed)).bfloat16().float()
        margins = []
        want = P.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, p + "mlp.", layer["mlp"], margins).float()
        if not margins or margins[0] > 0.05:
            break
    got = _run_part(backend, "feed_forward", spec, w, x, [70])
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)
    got = _run_part(backend, "feed_forward", spec, w, x, [3, 1, 40, 26])
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("top,ff,width", [(2, 96, 128), (1, 64, 160), (4, 40, 96)])
def test_routed_experts_with_many_tokens_per_expert(backend, top, ff, width):
    """Hundreds of tokens over six experts: an expert's rows fill several tiles and the last one partly; with widths that are
    multiples of 32 the bfloat16 products run on the tensor-core kernels, otherwise on the plain ones."""
    layer = {"kind": "moe", "expert": {"ff": ff, "limit": 1.2}, "router": {"experts": 6, "top": top}}
    g = torch.Generator().manual_seed(top)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).bfloat16().float()
    w = {"m.router": rnd(6, width, s=6.0 / width ** 0.5)}
    for e in range(6):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = rnd(ff, width, s=width ** -0.5), rnd(ff, width, s=width ** -0.5), rnd(width, ff, s=ff ** -0.5)
    w["m.router"][0] += 0.4 * w["m.router"][1]                 # an uneven load: expert 0 gets more than its share
    x = rnd(333, width)
    margins = []
    want = P.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, "m.", layer, margins).float()
    close = (torch.sort(x.double() @ w["m.router"].double().T, descending=True).values[:, top - 1:top + 1].diff(dim=1).abs() < 0.08).flatten()
    spec = PartSpec("routed_experts", {"hidden": width, "experts": 6, "top": top, "ff": ff, "limit": 1.2}, "m.")
    got = _run_part(backend, "feed_forward", spec, w, x, [333])
    keep = ~close                                               # rows whose choice of experts is no close call
    assert int(keep.sum()) > 250
    torch.testing.assert_close(got[keep], want[keep], atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("taps,bias,activation,residual", [(4, False, "none", True), (2, True, "silu", False), (1, False, "none", True),
                                                           (7, True, "none", False)])
@pytest.mark.parametrize("cuts", [[41], [1, 2, 1, 30, 3, 4], [1] * 41], ids=["whole", "portions", "tokens"])
def test_short_convolution_alone(backend, taps, bias, activation, residual, cuts):
    c = 40
    g = torch.Generator().manual_seed(taps)
    w = {"f.w": (torch.randn(c, taps, generator=g) * 0.5).bfloat16().float(), "f.b": torch.randn(c, generator=g).bfloat16().float()}
    x = torch.randn(41, c, generator=g).bfloat16().float()
    spec = PartSpec("short_conv", {"channels": c, "taps": taps, "weight_name": "w", "bias_name": "b" if bias else None,
                                   "activation": activation, "residual": residual}, "f.")
    got = _run_part(backend, "filter", spec, w, x, cuts)
    want = P.causal_conv(x.double(), w["f.w"].double(), w["f.b"].double() if bias else None)
    if residual:
        want = want + x.double()
    if activation == "silu":
        want = torch.nn.functional.silu(want)
    torch.testing.assert_close(got, want.float(), atol=_tol(backend, want.float()), rtol=0)


def test_pages_behind_a_block_of_positions_go_back_to_the_pool():
    """A query never reads before the start of its own block, so the cache manager gives the pages before it back while
    the request still runs, and promises a running request no more pages than a block and a portion can span."""
    from serve_b200.parts import CacheNeed

    need = CacheNeed(kv_heads=1, head_dim=16, chunk=24)
    mgr = CacheManager([need], [None], 8, 32, 2, 512)
    mgr.open("a")
    held = []
    for length in (20, 24, 47, 48, 100, 121):
        mgr.reserve([("a", length)])
        mgr.commit("a", length)
        held.append(mgr.pages_held("a")[0])
        mgr.check()
    assert held == [3, 0, 3, 0, 1, 1]        # at 24 and 48 tokens the next query opens a new block: nothing behind it is read again
    assert mgr.peak_pages(1000, 1) == [(24 + 1 - 2) // 8 + 2]
    mgr.close("a")
    assert mgr.groups[0].pool.in_use == 0


def test_named_states_are_cleared_when_a_slot_is_handed_out_again():
    """A layer's states (a recurrence's matrix, the tails of its convolutions) are rows of [max_slots, ...] tensors; a
    request that gets a slot somebody else held must find zeros, and a part sees its own states under its prefix."""
    from serve_b200.parts import CacheNeed

    need = CacheNeed.merged([("", CacheNeed(states=(("state", (2, 3, 4)),))), ("mixer_filter.", CacheNeed(states=(("tail", (2, 5)),))),
                             ("right.", CacheNeed(state_shape=(7,)))])
    assert dict(need.states) == {"state": (2, 3, 4), "mixer_filter.tail": (2, 5), "right.state": (7,)} and not need.has_pages
    mgr = CacheManager([need], [None], 8, 4, 2, 64, device="cpu", kv_dtype=torch.float32)
    view = mgr.views()[0]
    assert set(view.states) == {"state", "mixer_filter.tail", "right.state"} and view.states["state"].shape == (2, 2, 3, 4)
    assert set(view.sub("mixer_filter.").states) == {"tail"} and view.sub("right.").state is view.states["right.state"]
    slot = mgr.open("a")
    for st in view.states.values():
        st[slot].fill_(3.0)
    mgr.close("a")
    assert mgr.open("b") == slot
    assert all(float(st[slot].abs().max()) == 0.0 for st in view.states.values())


@pytest.mark.gpu
def test_trace_run_and_command_line_programs(models, tmp_path):
    """bin/trace_run and `python -m serve_b200.run` as a user starts them, on a model folder of this design: the class is
    chosen by config.json, four state slots and a pool smaller than the requests' total, so slots and pages come again."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        w, reqs, plain, folder = models["q"][dtype]
        steps = helpers.trace_mixed(reqs, live=4, seed=9)
        need = helpers.tokens_needed(steps, 64)
        out_dir = tmp_path / f"out-{dtype}"
        proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out_dir),
                               "--max-tokens", str(need)], input="\n".join(json.dumps(s) for s in steps) + "\n",
                              capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-3000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
        got, at = {}, {}
        for s in steps:
            n_want = sum(len(e["want"]) for e in s["entries"])
            arr = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n_want, CONFIGS["q"]["vocab"])
            i = 0
            for e in s["entries"]:
                base = at.get(e["id"], 0)
                for wi in e["want"]:
                    got[(e["id"], base + wi)] = torch.from_numpy(arr[i].copy())
                    i += 1
                at[e["id"]] = base + len(e["tokens"])
        compare_rows(got, plain, ("cuda", dtype))
    w, reqs, plain, folder = models["q"]["float32"]
    prompt = reqs["r2"]
    out = subprocess.run([sys.executable, "-m", "serve_b200.run", "--model", folder, "--dtype", "float32", "--page-size", "8", "--num-pages",
                          "16", "--max-context", "64", "--max-slots", "2", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "4"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    new = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])["generated_tokens"]
    logits = plain_logits(w, CONFIGS["q"], prompt + new)
    assert all(int(logits[len(prompt) - 1 + i].argmax()) == t for i, t in enumerate(new))
