"""The Bapavik decoder in the engine against the plain implementation of tests/plain/bapavik_plain.py.

Every test runs on the CPU over the torch stand-ins of the kernels (which checks the parts, the cache manager, the step
function and the scheduler) and, marked gpu, on the real kernels in float32 and bfloat16.
"""
import copy

import pytest
import torch

from serve_b200.cache import CacheManager
from serve_b200.config import ConfigError, PartSpec, build_spec, config_from_dict
from serve_b200.engine.step import BatchShape, StepContext
from serve_b200.parts import build_part
from tests import helpers
from tests.bapavik_cases import (BACKENDS, CONFIGS, compare_rows, make_engine, make_weights, plain_logits, runtime_for, write_model)
from tests.plain import bapavik_plain as P

LENGTHS = {"a": [1, 5, 23, 49, 75, 130], "o": [3, 40, 90, 17], "q": [2, 9, 31, 64, 101]}
PAGE = {"a": 8, "o": 4, "q": 16}


# ---- configuration and description ----------------------------------------------------------------------------
def test_configuration_is_read_from_the_file_and_describes_every_layer():
    from serve_b200.weights.random_init import model_tensor_decls

    for name, raw in CONFIGS.items():
        cfg = config_from_dict(raw)
        assert type(cfg).__name__ == "BapavikConfig" and cfg.width == raw["width"] and cfg.embedding_scale == raw["embedding"]["scale"]
        spec = build_spec(cfg)
        kinds = {"attention": "capped_sink_attention", "latent_attention": "latent_attention"}
        assert [l.parts["mixer"].kind for l in spec.layers] == [kinds[l["type"]] for l in raw["layers"]]
        assert [("feed_forward" in l.parts) for l in spec.layers] == [l["mlp"] is not None for l in raw["layers"]]
        assert [e.layer for e in spec.schedule] == P.layer_order(raw)
        assert all(e.cache_of is None for e in spec.schedule)          # every pass of a repeated layer has a cache of its own
        decls = {n: tuple(d.shape) for n, d in model_tensor_decls(cfg).items()}
        assert decls == P.tensor_shapes(raw)
        assert config_from_dict(cfg.to_dict()) == cfg


def test_layer_order_with_and_without_repeats():
    raw = copy.deepcopy(CONFIGS["a"])
    order = lambda: list(config_from_dict(raw).layer_order())
    assert order() == [0, 1, 0, 1, 2, 3]
    raw["loop"] = {"start": 1, "stop": 4, "times": 3}
    assert order() == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3]
    raw["loop"] = {"start": 2, "stop": 2, "times": 5}          # an empty run repeats nothing
    assert order() == [0, 1, 2, 3]
    raw["loop"] = {"start": 0, "stop": 4, "times": 1}
    assert order() == [0, 1, 2, 3]
    del raw["loop"]
    assert order() == [0, 1, 2, 3]


@pytest.mark.parametrize("breaker", [
    lambda c: c["layers"][0].update(type="other"),
    lambda c: c["layers"][0]["mixer"].pop("heads"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=99),
    lambda c: c["layers"][0]["mlp"].update(kind="other"),
    lambda c: c.update(loop={"start": 3, "stop": 2, "times": 2}),
    lambda c: c.update(loop={"start": 0, "stop": 9, "times": 2}),
    lambda c: c.pop("norm"),
])
def test_configuration_refuses_what_it_cannot_run(breaker):
    raw = copy.deepcopy(CONFIGS["a"])
    breaker(raw)
    with pytest.raises(ConfigError):
        config_from_dict(raw)


def test_random_weights_give_every_token_distinct_experts():
    from serve_b200.config import load_preset
    from serve_b200.weights.random_init import model_tensor_decls, random_tensor

    cfg = load_preset("bapavik-tiny")
    tables = [d for d in model_tensor_decls(cfg).values() if d.role == "table"]
    assert tables
    for d in tables:
        t = random_tensor(d, 5)
        n = int(d.init.split(":")[1])
        assert t.dtype == torch.int32 and int(t.min()) >= 0 and int(t.max()) < n
        assert all(len(set(row)) == len(row) for row in t.tolist())


# ---- whole models under every way of cutting the work ------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{config name: {dtype: (weights, requests, plain logits, model folder)}}."""
    out = {}
    for name in LENGTHS:
        cfg = CONFIGS[name]
        reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=20 + i) for i, n in enumerate(LENGTHS[name])}
        w = make_weights(cfg, 100 + len(name))
        plain = {rid: plain_logits(w, cfg, toks) for rid, toks in reqs.items()}
        out[name] = {dt: (w, reqs, plain, write_model(str(tmp_path_factory.mktemp(f"{name}-{dt}")), cfg, w, getattr(torch, dt)))
                     for dt in ("float32", "bfloat16")}
    return out


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["a", "o", "q"])
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
@pytest.mark.parametrize("name", ["a", "o", "q"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, backend):
    """Unequal requests side by side, portions beside single tokens, fewer slots and pages than the requests need in
    all: every row must equal the request run alone. Pages are poisoned first, so that a page that is read without
    having been written shows; a repeated layer's passes must not share pages either."""
    w, reqs, plain, folder = models[name][backend[1]]
    page = PAGE[name]
    steps = helpers.trace_mixed(reqs, live=3, seed=7)
    need = helpers.tokens_needed(steps, page) // page
    assert need < sum(-(-len(t) // page) for t in reqs.values())
    eng = make_engine(folder, backend, page, num_pages=need, max_slots=3, context=160)
    for view in eng.stepper.views:
        if view.k is not None:
            view.k.fill_(float("nan"))
            view.v.fill_(float("nan"))
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    compare_rows(got, plain, backend)
    eng.cache.check()
    assert eng.cache.live == 0 and eng.cache.free_slots == 3
    assert max(g.pool.high_water for g in eng.cache.groups) <= need


def test_latent_layers_keep_one_tensor_per_pass_and_repeated_layers_one_per_pass(models):
    w, reqs, plain, folder = models["a"]["float32"]
    eng = make_engine(folder, ("emu", "float32"), 8, num_pages=8)
    views = eng.stepper.views
    order = P.layer_order(CONFIGS["a"])
    assert len(views) == len(order) == 6
    for v, li in zip(views, order):
        latent = CONFIGS["a"]["layers"][li]["type"] == "latent_attention"
        assert (v.k is v.v) == latent                                # keys and values of a latent layer are the same rows
        if latent:
            m = CONFIGS["a"]["layers"][li]["mixer"]
            assert v.k.shape[1] == 1 and v.k.shape[3] == 16 * -(-(m["kv_rank"] + m["rot_dim"]) // 16)
    tensors = {id(v.k) for v in views}
    assert len(tensors) == len(views)                                # the two passes of layers 0 and 1 write different tensors


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_side_by_side(models, backend):
    """Two requests decoded one token at a time for 120 steps after short prompts (from CUDA graphs on the GPU): pages are
    crossed many times and the temperature's steps (every 5 positions) are passed one by one."""
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
    """generate(): the engine's own entry point, scheduler and sampler (sampled tokens stay on the device between steps,
    so the experts' table is read with them there). Every generated token must be (within the tolerance) the best one
    of the plain model given the tokens before it."""
    from serve_b200.run import Request, generate

    cfg = CONFIGS["a"]
    w, reqs, _, folder = models["a"][backend[1]]
    eng = make_engine(folder, backend, 8, num_pages=40, max_slots=3, budget=32)
    prompts = [reqs["r1"], reqs["r2"], reqs["r3"][:30], reqs["r0"]]
    out = generate(eng, [Request(torch.tensor(p), len(p), 12) for p in prompts], temperature=0.0, eos_token_id=None)
    for p, r in zip(prompts, out):
        new = r.generated_tokens.tolist()
        assert len(new) == 12
        logits = plain_logits(w, cfg, p + new)
        tol = float(logits.abs().max()) * (2e-4 if backend[1] == "float32" else 2.0 ** -4)
        for i, tok in enumerate(new):
            row = logits[len(p) - 1 + i]
            assert float(row[tok]) >= float(row.max()) - 2 * tol, f"token {i} of a request is not the plain model's choice"
    assert eng.cache.live == 0


# ---- each mechanism alone ---------------------------------------------------------------------------------------
def _ctx(rt, dev, q_lens, starts, slots, mgr=None, rids=None, tokens=None):
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
                       tokens=i32(tokens if tokens is not None else [0] * t), positions=i32(pos), token_row=i32(row), cu_q=i32(cu),
                       kv_len=i32(kv), slots=i32(slots), logit_rows=i32([]), block_tables=tables, rids=rids or [])


def _run_part(backend, family, spec, weights, x, cuts, page=8, tokens=None, pages=128):
    """One part alone over one sequence cut as ``cuts`` says, with a cache manager made for its need; another request
    runs first on the same pages and is closed, so the pages have been used before."""
    rt, dev = runtime_for(backend)
    part = build_part(family, spec, rt)
    names = {d.name for d in part.tensor_decls()}
    part.load({n: (weights[n].to(dev).to(rt.act_dtype) if weights[n].dtype.is_floating_point else weights[n].to(dev)) for n in names})
    need = part.cache_need() if hasattr(part, "cache_need") else None
    mgr = CacheManager([need], [None], page, pages, 1, 4096, device=dev, kv_dtype=rt.act_dtype)
    view = mgr.views()[0]
    call = (lambda h, ctx: part.forward(h, ctx, view)) if family == "mixer" else (lambda h, ctx: part.forward(h, ctx))
    xs = x.to(dev).to(rt.act_dtype)
    toks = tokens if tokens is not None else [0] * x.shape[0]
    with torch.inference_mode():
        mgr.open("warm")
        mgr.reserve([("warm", 5)])
        call(torch.randn_like(xs[:5]), _ctx(rt, dev, [5], [0], [mgr.slot("warm")], mgr, ["warm"], toks[:5]))
        mgr.close("warm")
        mgr.open("r")
        outs, at = [], 0
        for n in cuts:
            mgr.reserve([("r", at + n)])
            outs.append(call(xs[at: at + n], _ctx(rt, dev, [n], [at], [mgr.slot("r")], mgr, ["r"], toks[at: at + n])).float().cpu())
            mgr.commit("r", at + n)
            at += n
    assert at == x.shape[0]
    rt.kernels.check_errors()
    return torch.cat(outs)


def _tol(backend, want):
    return float(want.abs().max()) * (1e-4 if backend[1] == "float32" else 2.0 ** -6)


CUTS = [[57], [30, 1, 1, 2, 5, 17, 1], [1] * 57]


def _mixer_case(backend, name, index, cuts, seed=5, x=None, tweak=None, page=8, loose=1.0):
    from serve_b200.models.bapavik import _mixer_spec

    cfg = CONFIGS[name]
    layer, p = cfg["layers"][index], f"l{index}."
    w = make_weights(cfg, seed)
    if tweak is not None:
        tweak(w, p + "mix.")
    if x is None:
        x = torch.randn(sum(cuts), cfg["width"], generator=torch.Generator().manual_seed(seed + 1))
    x = x.bfloat16().float()
    spec = _mixer_spec(layer["type"], layer["mixer"], cfg["width"], cfg["norm"]["eps"], p + "mix.")
    got = _run_part(backend, "mixer", spec, w, x, cuts, page=page)
    want = P.MIXERS[layer["type"]](x.double(), {k: v.double() for k, v in w.items() if v.dtype.is_floating_point}, p + "mix.",
                                   layer["mixer"], cfg["norm"]["eps"]).float()
    torch.testing.assert_close(got, want, atol=_tol(backend, want) * loose, rtol=0)
    return got, want


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("where", [("a", 0), ("a", 2), ("o", 1), ("o", 2), ("q", 1)], ids=["a0", "a2", "o1", "o2", "q1"])
def test_sink_attention_alone(backend, cuts, where):
    _mixer_case(backend, where[0], where[1], cuts)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cuts", CUTS, ids=["whole", "portions", "tokens"])
@pytest.mark.parametrize("where", [("a", 1), ("a", 3), ("o", 0), ("o", 3), ("q", 0)], ids=["a1", "a3", "o0", "o3", "q0"])
def test_latent_attention_alone(backend, cuts, where):
    _mixer_case(backend, where[0], where[1], cuts)


@pytest.mark.parametrize("backend", BACKENDS[1:])
@pytest.mark.parametrize("index", [0, 1], ids=["attention", "latent"])
@pytest.mark.parametrize("cuts", [[420], [130, 1, 1, 270, 18]], ids=["whole", "portions"])
def test_mixers_at_the_sizes_of_a_real_layer(backend, index, cuts):
    """Each mixer alone at heads of 128 and cached rows of 256, over 420 tokens, whole and cut with single tokens in the middle."""
    _mixer_case(backend, "wide", index, cuts, seed=31, page=64)


def _stand_out(width, n, key, query, seed=4):
    """Inputs of which token ``key`` is large and token ``query`` is minus three times it, all others small."""
    x = torch.randn(n, width, generator=torch.Generator().manual_seed(seed)) * 0.3
    x[key] = torch.randn(width, generator=torch.Generator().manual_seed(seed + 1)) * 1.5
    if query != key:
        x[query] = -3.0 * x[key]
    return x


def _premise(fn, x, w, prefix, mixer, eps, key, query, want, backend):
    """The test's own premise: with that key gone the query's output is another one."""
    x2 = x.bfloat16().float().clone()
    x2[key] = 0.0
    other = fn(x2.double(), {k: v.double() for k, v in w.items() if v.dtype.is_floating_point}, prefix, mixer, eps).float()
    assert float((other[query] - want[query]).abs().max()) > 20 * _tol(backend, want)


FAR_KEYS = [(0, 299), (1, 299), (7, 8), (8, 299), (255, 256), (256, 299), (63, 64), (299, 299)]


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("key,query", FAR_KEYS)
@pytest.mark.parametrize("cuts", [[300], [270] + [1] * 30, [100, 2, 150, 3, 45]], ids=["prompt", "decoded", "portions"])
def test_sink_attention_finds_one_key_among_hundreds(backend, key, query, cuts):
    """The query projection is minus the key projection and the query token minus three times the key token, so the
    query points along that key and away from its own: the key takes nearly all the weight wherever it lies: the first
    tokens of the sequence, the last and the first token of a page of 8, hundreds of positions back. A kernel that
    drops or doubles a key at a page's or a tile's edge, or loses the first tokens, shows."""
    cfg = CONFIGS["a"]
    m = cfg["layers"][0]["mixer"]
    rep = m["heads"] // m["kv_heads"]

    def tweak(w, prefix):
        w[prefix + "q"] = -w[prefix + "k"].view(m["kv_heads"], m["dim"], -1).repeat_interleave(rep, 0).reshape(m["heads"] * m["dim"], -1).clone()
        w[prefix + "q.norm"] = 3.0 * w[prefix + "k.norm"].view(m["kv_heads"], m["dim"]).repeat_interleave(rep, 0).reshape(-1).clone()
        w[prefix + "sink"] = w[prefix + "sink"] * 0 - 2.0

    x = _stand_out(cfg["width"], 300, key, query)
    got, want = _mixer_case(backend, "a", 0, cuts, seed=11, x=x, tweak=tweak)
    if key != query:
        w = make_weights(cfg, 11)
        tweak(w, "l0.mix.")
        _premise(P.sink_attention, x, w, "l0.mix.", m, cfg["norm"]["eps"], key, query, want, backend)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("key,query", FAR_KEYS)
@pytest.mark.parametrize("cuts", [[300], [270] + [1] * 30, [100, 2, 150, 3, 45]], ids=["prompt", "decoded", "portions"])
def test_latent_attention_finds_one_key_among_hundreds(backend, key, query, cuts):
    """The same for latent attention: the plain query part of every head is made minus the read-out of the token's own
    latent vector (W_q = -4 U_n W_dkv on the plain rows), so a query that is minus a multiple of a key's token points
    along that key and away from its own."""
    cfg = CONFIGS["a"]
    m = cfg["layers"][1]["mixer"]

    def tweak(w, prefix):
        down = w[prefix + "dkv"][: m["kv_rank"]]                                    # [rank, width]
        uk = w[prefix + "uk"].view(m["heads"], m["dim"], m["kv_rank"])
        q = w[prefix + "q"].view(m["heads"], m["dim"] + m["rot_dim"], -1).clone()
        q[:, : m["dim"]] = torch.einsum("hdr,rw->hdw", uk, down) * -4.0
        q[:, m["dim"]:] *= 0.1
        w[prefix + "q"] = q.reshape(-1, q.shape[-1]).bfloat16().float()

    x = _stand_out(cfg["width"], 300, key, query)
    got, want = _mixer_case(backend, "a", 1, cuts, seed=12, x=x, tweak=tweak)
    if key != query:
        w = make_weights(cfg, 12)
        tweak(w, "l1.mix.")
        _premise(P.latent_attention, x, w, "l1.mix.", m, cfg["norm"]["eps"], key, query, want, backend)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("sink", [-30.0, 0.0, 6.0, 40.0])
def test_the_sink_takes_its_share_once(backend, sink):
    """A sink far below the scores changes nothing, one far above them takes all the weight (the output goes to zero);
    decoded over many keys (where the kernels split the keys over blocks and merge) it must still count once."""
    cfg = CONFIGS["a"]

    def tweak(w, prefix):
        w[prefix + "sink"] = torch.full_like(w[prefix + "sink"], sink)

    for cuts in ([400], [399, 1], [200] + [1] * 200):
        got, want = _mixer_case(backend, "a", 0, cuts, seed=13, tweak=tweak)
    if sink >= 40.0:
        assert float(want.abs().max()) < 1e-6
    if sink <= -30.0:
        w = make_weights(cfg, 13)
        w["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -1e4)
        x = torch.randn(400, cfg["width"], generator=torch.Generator().manual_seed(14)).bfloat16().float()
        none = P.sink_attention(x.double(), {k: v.double() for k, v in w.items() if v.dtype.is_floating_point}, "l0.mix.",
                                cfg["layers"][0]["mixer"], cfg["norm"]["eps"]).float()
        torch.testing.assert_close(want, none, atol=1e-5 * float(none.abs().max()), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cap", [0.5, 3.0])
def test_a_low_cap_bends_the_scores(backend, cap):
    """With strong queries and a cap far below the raw scores nearly every score sits at plus or minus the cap: the
    output differs a lot from the uncapped one, and the engine must follow."""
    cfg = copy.deepcopy(CONFIGS["a"])
    cfg["layers"][0]["mixer"]["softcap"] = cap
    from serve_b200.models.bapavik import _mixer_spec

    layer = cfg["layers"][0]
    w = make_weights(cfg, 15)
    w["l0.mix.q.norm"] = w["l0.mix.q.norm"] * 6.0
    x = torch.randn(90, cfg["width"], generator=torch.Generator().manual_seed(16)).bfloat16().float()
    spec = _mixer_spec("attention", layer["mixer"], cfg["width"], cfg["norm"]["eps"], "l0.mix.")
    w64 = {k: v.double() for k, v in w.items() if v.dtype.is_floating_point}
    want = P.sink_attention(x.double(), w64, "l0.mix.", layer["mixer"], cfg["norm"]["eps"]).float()
    loose = P.sink_attention(x.double(), w64, "l0.mix.", dict(layer["mixer"], softcap=1e6), cfg["norm"]["eps"]).float()
    assert float((want - loose).abs().max()) > 0.1 * float(want.abs().max())
    for cuts in ([90], [50, 2] + [1] * 38):
        got = _run_part(backend, "mixer", spec, w, x, cuts)
        torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("every", [1, 16, 64])
def test_the_temperature_steps_at_the_right_positions(backend, every):
    """With a large coefficient the step of the temperature at positions every-1, 2 every-1, ... changes the output
    visibly; whole, and decoded token by token across the steps."""
    cfg = copy.deepcopy(CONFIGS["a"])
    cfg["layers"][0]["mixer"]["q_temp"] = {"coef": 2.5, "every": every}
    from serve_b200.models.bapavik import _mixer_spec

    layer = cfg["layers"][0]
    w = make_weights(cfg, 17)
    x = torch.randn(140, cfg["width"], generator=torch.Generator().manual_seed(18)).bfloat16().float()
    spec = _mixer_spec("attention", layer["mixer"], cfg["width"], cfg["norm"]["eps"], "l0.mix.")
    w64 = {k: v.double() for k, v in w.items() if v.dtype.is_floating_point}
    want = P.sink_attention(x.double(), w64, "l0.mix.", layer["mixer"], cfg["norm"]["eps"]).float()
    shifted = P.sink_attention(x.double(), w64, "l0.mix.", dict(layer["mixer"], q_temp={"coef": 2.5, "every": every + 1}), cfg["norm"]["eps"]).float()
    assert float((want - shifted).abs().max()) > 0.02 * float(want.abs().max())
    for cuts in ([140], [10] + [1] * 130):
        got = _run_part(backend, "mixer", spec, w, x, cuts)
        torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_rotation_of_the_shared_key_part_far_from_the_start(backend):
    """A sequence of 1,500 tokens whose rotated parts are given nearly all the weight of the score, so an angle that is
    off at large positions shows; the last hundred tokens come as a portion and then one by one."""
    cfg = CONFIGS["q"]
    m = cfg["layers"][0]["mixer"]

    def tweak(w, prefix):
        q = w[prefix + "q"].view(m["heads"], m["dim"] + m["rot_dim"], -1).clone()
        q[:, : m["dim"]] *= 0.05
        q[:, m["dim"]:] *= 4.0
        w[prefix + "q"] = q.reshape(-1, q.shape[-1]).bfloat16().float()

    x = torch.randn(1500, cfg["width"], generator=torch.Generator().manual_seed(19))
    # (bfloat16: queries this strong make a sharp softmax, where the rounding of a score to 8 bits shows twice as much)
    _mixer_case(backend, "q", 0, [1400, 60] + [1] * 40, seed=20, x=x, tweak=tweak, page=16, loose=1.0 if backend[1] == "float32" else 2.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name,index", [("a", 0), ("o", 0), ("q", 1)])
def test_dense_feed_forward_alone(backend, name, index):
    from serve_b200.models.bapavik import _feed_forward_spec

    cfg = CONFIGS[name]
    f, p = cfg["layers"][index]["mlp"], f"l{index}.mlp."
    w = make_weights(cfg, 21)
    x = (torch.randn(70, cfg["width"], generator=torch.Generator().manual_seed(22)) * 2.0).bfloat16().float()      # many sums beyond the limits
    spec = _feed_forward_spec(f, cfg["width"], cfg["vocab"], p)
    want = P.dense_feed_forward(x.double(), {k: v.double() for k, v in w.items() if v.dtype.is_floating_point}, p, f).float()
    g = x.double() @ w[p + "gate"].double().T
    assert float((g > f["limit"]).double().mean()) > 0.05
    for cuts in ([70], [3, 1, 40, 26]):
        got = _run_part(backend, "feed_forward", spec, w, x, cuts)
        torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name,index", [("a", 1), ("a", 2), ("o", 1), ("o", 3), ("q", 0)])
def test_table_experts_alone(backend, name, index):
    from serve_b200.models.bapavik import _feed_forward_spec

    cfg = CONFIGS[name]
    f, p = cfg["layers"][index]["mlp"], f"l{index}.mlp."
    w = make_weights(cfg, 23)
    toks = helpers.random_tokens(cfg["vocab"], 70, seed=24)
    x = torch.randn(70, cfg["width"], generator=torch.Generator().manual_seed(25)).bfloat16().float()
    spec = _feed_forward_spec(f, cfg["width"], cfg["vocab"], p)
    w64 = {k: (v.double() if v.dtype.is_floating_point else v) for k, v in w.items()}
    want = P.table_experts(x.double(), toks, w64, p, f).float()
    for cuts in ([70], [3, 1, 40, 26], [1] * 70):
        got = _run_part(backend, "feed_forward", spec, w, x, cuts, tokens=toks)
        torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("top,ff,width", [(2, 96, 128), (1, 64, 160), (4, 40, 96)])
def test_table_experts_with_many_tokens_per_expert(backend, top, ff, width):
    """Hundreds of tokens over six experts, most of them of a few token ids: an expert's rows fill several tiles and the last
    one partly; with widths that are multiples of 32 the bfloat16 products run on the tensor-core tiles."""
    vocab, experts = 50, 6
    g = torch.Generator().manual_seed(top)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).bfloat16().float()
    w = {"m.table": torch.rand(vocab, experts, generator=g).argsort(1)[:, :top].to(torch.int32).contiguous()}
    for e in range(experts):
        w[f"m.e{e}.up"], w[f"m.e{e}.down"] = rnd(ff, width, s=width ** -0.5), rnd(width, ff, s=ff ** -0.5)
    toks = [t % 5 if i % 3 else t for i, t in enumerate(helpers.random_tokens(vocab, 333, seed=3))]           # an uneven load
    x = rnd(333, width)
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    want = P.table_experts(x.double(), toks, {k: (v.double() if v.dtype.is_floating_point else v) for k, v in w.items()}, "m.", f).float()
    spec = PartSpec("table_experts", {"hidden": width, "experts": experts, "top": top, "ff": ff, "vocab": vocab}, "m.")
    got = _run_part(backend, "feed_forward", spec, w, x, [333], tokens=toks)
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("width", [48, 100, 512, 1030])
def test_layer_norm_and_scaled_embedding(backend, width):
    rt, dev = runtime_for(backend)
    g = torch.Generator().manual_seed(width)
    wt = (1.0 + 0.3 * torch.randn(width, generator=g)).bfloat16().float()
    norm = build_part("norm", PartSpec("layer_norm", {"size": width, "eps": 1e-5, "weight_name": "n"}, "t."), rt)
    norm.load({"t.n": wt.to(dev)})
    x = (torch.randn(37, width, generator=g) * 3.0 + 5.0)          # a mean far from zero: the deviation matters
    delta = torch.randn(37, width, generator=g).to(rt.act_dtype)
    xs, want_x = x.clone().to(dev), x + delta.float()
    got = norm.forward(xs, delta.to(dev), None).float().cpu()
    want = P.layer_norm(want_x.double(), wt.double(), 1e-5).float()
    torch.testing.assert_close(xs.cpu(), want_x, atol=1e-6, rtol=0)
    torch.testing.assert_close(got, want, atol=_tol(backend, want) * 2, rtol=0)
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=dev)
    got = norm.forward_rows(xs, None, rows, None).float().cpu()
    torch.testing.assert_close(got, want[[5, 0, 36]], atol=_tol(backend, want) * 2, rtol=0)
    table = torch.randn(20, width, generator=g).bfloat16().float()
    emb = build_part("embedding", PartSpec("table", {"vocab": 20, "hidden": width, "name": "e", "scale": 7.25}), rt)
    emb.load({"e": table.to(dev).to(rt.act_dtype)})
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32, device=dev)
    torch.testing.assert_close(emb.forward(ids, None).cpu(), table[[3, 19, 0, 3]] * 7.25, atol=0, rtol=0)


@pytest.mark.gpu
def test_trace_run_and_command_line_programs(models, tmp_path):
    """bin/trace_run and `python -m serve_b200.run` as a user starts them, on a model folder of this design: the class is
    chosen by config.json; four slots and a pool smaller than the requests' total, so slots and pages come again."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        w, reqs, plain, folder = models["a"][dtype]
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
            arr = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n_want, CONFIGS["a"]["vocab"])
            i = 0
            for e in s["entries"]:
                base = at.get(e["id"], 0)
                for wi in e["want"]:
                    got[(e["id"], base + wi)] = torch.from_numpy(arr[i].copy())
                    i += 1
                at[e["id"]] = base + len(e["tokens"])
        compare_rows(got, plain, ("cuda", dtype))
    w, reqs, plain, folder = models["a"]["float32"]
    prompt = reqs["r2"]
    out = subprocess.run([sys.executable, "-m", "serve_b200.run", "--model", folder, "--dtype", "float32", "--page-size", "8", "--num-pages",
                          "16", "--max-context", "64", "--max-slots", "2", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "4"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    new = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])["generated_tokens"]
    logits = plain_logits(w, CONFIGS["a"], prompt + new)
    assert all(int(logits[len(prompt) - 1 + i].argmax()) == t for i, t in enumerate(new))


@pytest.mark.parametrize("backend", BACKENDS[1:])
@pytest.mark.parametrize("rows", [5, 16, 300, 2048])
def test_dense_feed_forward_at_the_sizes_of_a_real_layer(backend, rows):
    """Width 512 and 2,048 inner columns: a handful of rows take the few-rows product, thousands the tensor-memory tiles (both
    with the activation in their epilogue, in bfloat16), the row counts between them the library product and the activation
    kernel; all three must give the same numbers."""
    width, ff, limit = 512, 2048, 1.25
    g = torch.Generator().manual_seed(rows)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).bfloat16().float()
    w = {"f.gate": rnd(ff, width, s=2.0 * width ** -0.5), "f.up": rnd(ff, width, s=2.0 * width ** -0.5), "f.down": rnd(width, ff, s=ff ** -0.5)}
    x = rnd(rows, width)
    f = {"kind": "dense", "ff": ff, "limit": limit}
    want = P.dense_feed_forward(x.double(), {k: v.double() for k, v in w.items()}, "f.", f).float()
    spec = PartSpec("gated_dense", {"hidden": width, "intermediate": ff, "activation": "clamped_swish", "limit": limit, "alpha": 1.702,
                                    "names": {"gate": "gate", "up": "up", "down": "down"}}, "f.")
    got = _run_part(backend, "feed_forward", spec, w, x, [rows], page=64, pages=64)
    torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS[2:])
@pytest.mark.parametrize("heads,group", [(16, 8), (32, 8), (24, 8), (8, 4), (12, 8)])
def test_latent_attention_with_many_heads_in_groups(backend, heads, group):
    """All heads read one cached row per token; the bfloat16 kernels deal them to groups that each count as a key/value
    head of their own (12 heads do not divide into groups of 8 and stay one group). Prompt, portions and decoded tokens
    after 700 cached ones, where the keys are also split over blocks."""
    from serve_b200.models.bapavik import _mixer_spec

    m = {"heads": heads, "dim": 32, "rot_dim": 16, "vdim": 32, "kv_rank": 48, "scale": 0.15, "rot": {"base": 10000.0, "dims": 16}}
    width = 128
    g = torch.Generator().manual_seed(heads)
    rnd = lambda *shape: (torch.randn(*shape, generator=g) * 1.5 / shape[-1] ** 0.5).bfloat16().float()
    w = {"t.q": rnd(heads * 48, width), "t.dkv": rnd(64, width), "t.dkv.norm": (1 + 0.2 * torch.randn(48, generator=g)).bfloat16().float(),
         "t.uk": rnd(heads * 32, 48), "t.uv": rnd(heads * 32, 48), "t.o": rnd(width, heads * 32)}
    x = torch.randn(730, width, generator=g).bfloat16().float()
    want = P.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, "t.", m, 1e-5).float()
    spec = _mixer_spec("latent_attention", m, width, 1e-5, "t.")
    rt, _ = runtime_for(backend)
    before = (rt.kernels.LATENT_GROUP, rt.kernels.LATENT_GROUP_DECODE)
    rt.kernels.LATENT_GROUP = rt.kernels.LATENT_GROUP_DECODE = group
    try:
        for cuts in ([730], [700, 3, 2] + [1] * 25):
            got = _run_part(backend, "mixer", spec, w, x, cuts, page=16)
            torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)
    finally:
        rt.kernels.LATENT_GROUP, rt.kernels.LATENT_GROUP_DECODE = before


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("rank,rot", [(272, 16), (40, 8)])
def test_latent_attention_that_caches_keys_and_values_per_head(backend, rank, rot):
    """A latent row wider than the attention kernels' widest head (272 + 16 > 256) is read out per head when the token
    arrives and cached in ordinary pages; asked for by name the same path runs at any size. Same results."""
    from serve_b200.models.bapavik import _mixer_spec

    m = {"heads": 3, "dim": 24, "rot_dim": rot, "vdim": 40, "kv_rank": rank, "scale": 0.2, "rot": {"base": 5000.0, "dims": rot}}
    width = 96
    g = torch.Generator().manual_seed(rank)
    rnd = lambda *shape: (torch.randn(*shape, generator=g) * 1.5 / shape[-1] ** 0.5).bfloat16().float()
    w = {"t.q": rnd(3 * (24 + rot), width), "t.dkv": rnd(rank + rot, width), "t.dkv.norm": (1 + 0.2 * torch.randn(rank, generator=g)).bfloat16().float(),
         "t.uk": rnd(3 * 24, rank), "t.uv": rnd(3 * 40, rank), "t.o": rnd(width, 3 * 40)}
    x = torch.randn(75, width, generator=g).bfloat16().float()
    want = P.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, "t.", m, 1e-5).float()
    spec = _mixer_spec("latent_attention", m, width, 1e-5, "t.")
    spec.params["per_head"] = True
    rt, _ = runtime_for(backend)
    part = build_part("mixer", spec, rt)
    assert part.per_head and part.cache_need().kv_heads == 3 and not part.cache_need().shared_kv
    if rank + rot > 256:
        auto = build_part("mixer", _mixer_spec("latent_attention", m, width, 1e-5, "t."), rt)
        assert auto.per_head
    for cuts in ([75], [40, 2, 1, 1, 30, 1]):
        got = _run_part(backend, "mixer", spec, w, x, cuts, page=16)
        torch.testing.assert_close(got, want, atol=_tol(backend, want), rtol=0)


@pytest.mark.parametrize("backend", BACKENDS[1:])
@pytest.mark.parametrize("dim,vdim,kv", [(128, 128, 2), (64, 64, 8), (128, 48, 1), (40, 64, 4)])
@pytest.mark.parametrize("cap,sink", [(50.0, 0.5), (2.0, -3.0), (None, 6.0), (6.0, 60.0)])
def test_cap_and_sink_at_head_sizes_of_64_and_128(backend, dim, vdim, kv, cap, sink):
    """Heads of 64 and 128 (also padded to them) send the prompt portions of the bfloat16 path to the tensor-memory kernel and the
    decoded tokens to the split-key kernel: a low cap, no cap, sinks below, among and far above the scores, over 700 tokens."""
    from serve_b200.models.bapavik import _mixer_spec

    m = {"heads": 8, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "softcap": cap, "q_temp": {"coef": 0.4, "every": 100}}
    width = 256
    g = torch.Generator().manual_seed(dim + vdim)
    rnd = lambda *shape: (torch.randn(*shape, generator=g) * 1.5 / shape[-1] ** 0.5).bfloat16().float()
    w = {"t.q": rnd(8 * dim, width), "t.k": rnd(kv * dim, width), "t.v": rnd(kv * vdim, width), "t.o": rnd(width, 8 * vdim),
         "t.q.norm": (2.0 + 0.3 * torch.randn(8 * dim, generator=g)).bfloat16().float(), "t.k.norm": (1.0 + 0.2 * torch.randn(kv * dim, generator=g)).bfloat16().float(),
         "t.sink": torch.full((8,), sink) + torch.arange(8) * 0.25}
    x = torch.randn(700, width, generator=g).bfloat16().float()
    want = P.sink_attention(x.double(), {k: v.double() for k, v in w.items()}, "t.", dict(m, softcap=cap or 1e9), 1e-5).float()
    spec = _mixer_spec("attention", m, width, 1e-5, "t.")
    for cuts in ([700], [300, 390, 2, 3] + [1] * 5):
        got = _run_part(backend, "mixer", spec, w, x, cuts, page=64, pages=32)
        torch.testing.assert_close(got, want, atol=max(_tol(backend, want), 1e-6), rtol=0)
