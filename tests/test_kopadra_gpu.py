"""The Kopadra design in the engine against the plain whole-sequence implementation
(`plain_kopadra`): each mechanism alone, whole prompts, token-by-token decoding, portions down to
two tokens, unequal requests in one batch, pages and slots used again, long decoding, and greedy
generation through the entry point.  Random weights are scaled out of their nearly linear range,
and where a fault would still hide (a far key among hundreds, a correction that changes the choice,
a gate beyond its cap) the weights or inputs are made so that it shows."""

import json
import os

import pytest
import torch

import kopadra_configs as KC
import plain_kopadra as PK
import schedules
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = [70, 5, 131, 33, 2, 97]


def options(dtype, **kw):
    from ninfer_amd_mi50_b200.config import EngineOptions
    base = dict(dtype=dtype, page_size=16, num_sequences=4, max_context=256, cache_tokens=1024, use_graph=False)
    base.update(kw)
    return EngineOptions(**base)


def run_chosen(runner, steps, routing=True):
    """Drive the runner through a schedule -> (float64 logits per request, in the order asked; the experts the
    engine chose per request: a list over the routed layers of [tokens, top]).  `routing` false: nothing is
    recorded (a step replayed from a graph runs no Python to record in)."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.engine import StepEntry
    from ninfer_amd_mi50_b200.parts.feedforward import SparseMoeSwiglu
    got, chosen = {}, {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if not runner.cache.is_open(e["id"]):
                runner.open(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        SparseMoeSwiglu.record_routing = [] if routing else None
        try:
            out = runner.step(entries)
            record = SparseMoeSwiglu.record_routing or []
        finally:
            SparseMoeSwiglu.record_routing = None
        r = row = 0
        for e in st["entries"]:
            n = len(e["want"])
            got.setdefault(e["id"], []).append(out[r:r + n].double().cpu())
            r += n
            per = chosen.setdefault(e["id"], [[] for _ in record])
            for layer, idx in enumerate(record):
                per[layer].append(idx[row:row + len(e["tokens"])].long().cpu())
            row += len(e["tokens"])
        for rid in st["end"]:
            runner.close(rid)
        runner.cache.check()
    kernels.check_status("schedule")
    return {k: torch.cat(v) for k, v in got.items()}, {k: [torch.cat(v) for v in per] for k, per in chosen.items()}


def run(runner, steps):
    return run_chosen(runner, steps, routing=False)[0]


def compare(got, want, dtype, what, bf16_bound=6e-2, touchy=None):
    """float32 is the sharp comparison: 1e-4 of the largest logit for every row.  bfloat16 rounds
    every activation between kernels to 8 bits: every row within 6 %, the median row (of a request
    of 16 rows or more) within 2 %; rows found `touchy` only have to be finite, and of the others
    one in thirty may stray further (the search for touchy rows is a few random tries), up to 25 %; the median
    bound is then 2 %."""
    scale = want.abs().max().item()
    err = (got - want).abs().max(dim=1).values / scale
    if dtype == "float32":
        assert err.max().item() <= 1e-4, f"{what}: row {int(err.argmax())} of {len(err)} differs by {err.max().item():.3e} of the scale"
        return err.max().item()
    assert torch.isfinite(got).all(), what
    if touchy is not None:
        assert len(touchy) < 16 or touchy.float().mean().item() <= 0.35, f"{what}: {int(touchy.sum())} of {len(touchy)} rows are touchy"
        err = err[~touchy]
    if len(err) and touchy is not None:
        assert int((err > bf16_bound).sum()) <= max(1, len(err) // 30) and err.max().item() <= 0.25, \
            f"{what}: {int((err > bf16_bound).sum())} of {len(err)} steady rows differ by more than {bf16_bound}, the worst by {err.max().item():.3e}"
    elif len(err):
        assert err.max().item() <= bf16_bound, f"{what}: row {int(err.argmax())} of {len(err)} steady rows differs by {err.max().item():.3e} of the scale"
    if len(err) >= 16:
        # (five layers of two dozen roundings a row: the plain model disturbed by 2^-9 moves its median row by 1 %)
        assert err.median().item() <= 2e-2, f"{what}: the median row differs by {err.median().item():.3e} of the scale"
    return err.max().item() if len(err) else 0.0


def plain(cfg, w, tokens, chosen=None):
    return PK.forward(cfg, w, list(tokens), chosen=chosen)[0]


def touchy_rows(cfg, w, tokens, chosen, want, tries=3):
    """Rows whose logits move by more than 2 % of the scale when every projection's output is disturbed by
    2^-9 of its size, in any of a few tries.  The recurrence's output is divided by its root mean square head
    by head, and an attention's queries and keys by theirs: where a head's sum nearly cancels (a request's
    first tokens, whose recurrence output is sign(q . k) v), the norm blows a rounding up with it."""
    scale = want.abs().max().item()
    out = torch.zeros(want.shape[0], dtype=torch.bool)
    try:
        for i in range(tries):
            PK.NOISE = (torch.Generator().manual_seed(50 + i), 2.0 ** -9)
            out |= (plain(cfg, w, tokens, chosen) - want).abs().max(dim=1).values / scale > 2e-2
    finally:
        PK.NOISE = None
    return out


def check(got, chosen, cfg, w, tokens, dtype, what, want32=None, rows=None):
    """float32 against the plain model as it is; bfloat16 against the plain model with the experts the engine
    chose (a rounding of the router's input flips near-ties, which is no fault), touchy rows set aside."""
    if dtype == "float32":
        want = want32 if want32 is not None else plain(cfg, w, tokens)
        return compare(got, want if rows is None else want[rows], dtype, what)
    want = plain(cfg, w, tokens, chosen)
    touchy = touchy_rows(cfg, w, tokens, chosen, want)
    if rows is not None:
        want, touchy = want[rows], touchy[rows]
    return compare(got, want, dtype, what, touchy=touchy)


@pytest.fixture(scope="module", params=sorted(KC.CONFIGS))
def folder(request, tmp_path_factory):
    cfg, seed = KC.CONFIGS[request.param]
    d = str(tmp_path_factory.mktemp("kopadra") / request.param)
    KC.write_folder(cfg, seed, d, scale=KC.SCALES.get(request.param))
    cfg, w = KC.read_folder(d)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 900 + i) for i, n in enumerate(LENGTHS)}
    want = {r: plain(cfg, w, t) for r, t in reqs.items()}
    return request.param, d, cfg, w, reqs, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_the_plain_model(folder, dtype, how):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs, want = folder
    make = {"whole": schedules.whole, "tail": lambda r: schedules.tail_decoded(r, tail=40),
            "portions": schedules.portions,
            # a pool of 320 tokens for 338 in all, three slots for six requests: pages and slots come back
            "mixed": lambda r: schedules.mixed(r, max_live=3, page=16, pool_tokens=320, tail=9)}[how]
    pool = 320 if how == "mixed" else 1024
    runner = load_runner(d, options=options(dtype, cache_tokens=pool, num_sequences=3 if how == "mixed" else 4))
    got, chosen = run_chosen(runner, make(reqs))
    assert all(n == pool // 16 for n in runner.cache.pages_free())
    for r in reqs:
        check(got[r], chosen[r], cfg, w, reqs[r], dtype, f"{name} {how} {r}", want32=want[r])


# ---- each mechanism alone ---------------------------------------------------------------------

def model_of(layers, width=96, vocab=113, eps=1e-5, cap=None):
    c = {"architecture": "Kopadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


def run_alone(d, tokens, dtype, cuts=None, with_chosen=False, **opt):
    from ninfer_amd_mi50_b200.engine import load_runner
    runner = load_runner(d, options=options(dtype, **opt))
    steps = schedules.whole({"a": tokens}) if cuts is None else schedules.portions({"a": tokens}, cuts=cuts)
    got, chosen = run_chosen(runner, steps)
    return (got["a"], chosen["a"]) if with_chosen else got["a"]


def check_alone(tmp_path, cfg, dtype, n_tokens=90, cuts=(2, 3, 40, 1, 16), replace=None, scale=None, seed=7, **opt):
    d = KC.write_folder(cfg, seed, str(tmp_path / "m"), replace=replace, scale=scale)
    cfg, w = KC.read_folder(d)
    toks = random_tokens(n_tokens, cfg["vocab"], seed)
    want = plain(cfg, w, toks)
    check(*run_alone(d, toks, dtype, with_chosen=True, **opt), cfg, w, toks, dtype, "whole", want32=want)
    if cuts:
        check(*run_alone(d, toks, dtype, cuts=list(cuts), with_chosen=True, **opt), cfg, w, toks, dtype, "portions", want32=want)
    return d, cfg, w, toks, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mixer", [
    KC.attention(2, 1, 8, 8, 0.3, rot=(100.0, 4)),                                      # one row a token, equal sizes
    KC.attention(4, 2, 16, 16, 0.25),                                                   # head-major pages, nothing turned
    KC.attention(4, 4, 32, 32, 0.2, rot=(10000.0, 32), scaling=(4.0, 48, 8.0, 1.0)),    # the whole head turned, stretched
    KC.attention(6, 3, 16, 40, 0.3, rot=(50.0, 10), scaling=(16.0, 16, 2.0, 0.25)),     # values wider than keys
    KC.attention(3, 1, 24, 8, 0.2, rot=(700.0, 24)),                                    # keys wider than values
    KC.attention(8, 8, 64, 64, 0.15, rot=(1e6, 16), scaling=(1.0, 64, 32.0, 1.0)),      # factor 1: the plain frequencies
])
def test_attention_alone_whole_and_in_portions(tmp_path, dtype, mixer):
    check_alone(tmp_path, model_of([KC.layer(mixer, None)], width=72), dtype, n_tokens=150)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_norms_rotation_and_biases_each_change_the_answer(tmp_path, dtype):
    """The plain model without one of the mechanisms differs from the engine by far more than rounding: none
    of them is skipped."""
    mixer = KC.attention(4, 2, 16, 16, 0.3, rot=(100.0, 8), scaling=(4.0, 32, 4.0, 1.0))
    d, cfg, w, toks, want = check_alone(tmp_path, model_of([KC.layer(mixer, None)]), dtype, cuts=None)
    got = run_alone(d, toks, dtype)
    scale = want.abs().max().item()

    def distance(other):
        return ((got - other).abs().max() / scale).item()

    for name, value in (("l0.mix.g", 0.0), ("l0.mix.q.norm", 1.0), ("l0.mix.k.norm", 1.0), ("l0.mix.v.b", 0.0), ("l0.mix.q.b", 0.0)):
        w2 = dict(w)
        w2[name] = torch.full_like(w[name], value)
        assert distance(plain(cfg, w2, toks)) > 0.1, name
    for change in ({"scaling": None}, {"dims": 0}):
        cfg2 = json.loads(json.dumps(cfg))
        cfg2["layers"][0]["mixer"]["rot"].update(change)
        assert distance(plain(cfg2, w, toks)) > 0.1, change


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(4, 2, 32, 32), (4, 1, 32, 24), (2, 2, 48, 80), (8, 2, 64, 64), (2, 1, 128, 128)])
def test_one_far_key_among_hundreds_is_found(tmp_path, dtype, sizes):
    """Queries and keys share their matrix, biases and norm weights, read only the first half of the width,
    nothing is turned and the scale is large: a query's best keys are those of tokens whose first half is its
    own, wherever they stand.  Two tokens share that half and have opposite second halves (of mean zero, so the
    layer norm treats both alike), hence the same key and different values.  One stands last, the other once
    before it - at a page's first or last place, or hundreds back - and takes half of the last row's weight:
    a key that is lost, or read from the wrong place, changes the answer wholly.  In a prompt, in portions
    and decoded."""
    H, G, D, Dv = sizes
    cfg = model_of([KC.layer(KC.attention(H, G, D, Dv, 16.0 / D), None)], width=64, vocab=401)
    d0 = KC.write_folder(cfg, 3, str(tmp_path / "m0"))
    _, w0 = KC.read_folder(d0)
    wk = w0["l0.mix.k"].clone()
    wk[:, 32:] = 0.0
    g = torch.Generator().manual_seed(9)
    a, b = torch.randn(32, generator=g, dtype=torch.float64) * 0.02, torch.randn(32, generator=g, dtype=torch.float64) * 0.02
    b -= b.mean()
    embed = w0["embed"].clone()
    embed[400], embed[398] = torch.cat([a, b]), torch.cat([a, -b])
    replace = {"embed": embed, "l0.mix.k": wk,
               "l0.mix.q": wk.view(G, D, -1).repeat_interleave(H // G, dim=0).reshape(H * D, -1),
               "l0.mix.q.b": w0["l0.mix.k.b"].view(G, D).repeat_interleave(H // G, dim=0).reshape(-1),
               "l0.mix.q.norm": w0["l0.mix.k.norm"].view(G, D).repeat_interleave(H // G, dim=0).reshape(-1)}
    d = KC.write_folder(cfg, 3, str(tmp_path / "m"), replace=replace)
    cfg, w = KC.read_folder(d)
    from ninfer_amd_mi50_b200.engine import load_runner
    n = 500
    for place in (0, 15, 16, 17, 63, 64, 250, 463):
        toks = [1 + (i % 397) for i in range(n)]        # tokens 1..397
        toks[place], toks[-1] = 398, 400
        want = plain(cfg, w, toks)[-1:]
        without = list(toks)
        without[place] = 397
        assert ((plain(cfg, w, without)[-1:] - want).abs().max() / want.abs().max()).item() > 0.2, "the key does not matter"
        for how in ("prompt", "portions", "decoded"):
            runner = load_runner(d, options=options(dtype, max_context=512))
            if how == "prompt":
                steps = [{"entries": [{"id": "a", "tokens": toks, "want": [n - 1]}], "end": ["a"]}]
            elif how == "portions":
                cut = [0, 14, 16, 19, 64, 67, 300, n]
                steps = [{"entries": [{"id": "a", "tokens": toks[a_:b_], "want": [b_ - a_ - 1] if b_ == n else []}],
                          "end": ["a"] if b_ == n else []} for a_, b_ in zip(cut, cut[1:])]
            else:
                steps = [{"entries": [{"id": "a", "tokens": toks[:n - 3], "want": []}], "end": []}]
                steps += [{"entries": [{"id": "a", "tokens": toks[i:i + 1], "want": [0] if i == n - 1 else []}],
                           "end": ["a"] if i == n - 1 else []} for i in range(n - 3, n)]
            compare(run(runner, steps)["a"], want, dtype, f"place {place} {how}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,cap", [(3, 16, 24, 6.0), (5, 10, 7, None), (2, 64, 40, 2.0), (1, 8, 8, 30.0),
                                                (4, 32, 32, 12.0), (2, 128, 96, 8.0), (1, 200, 20, 4.0)])
def test_the_recurrence_alone_whole_and_in_portions(tmp_path, dtype, heads, dim, vdim, cap):
    """Gates beyond their cap (the projections reach about three times the smaller caps), forget gates from a
    quarter to nearly one, input gates large enough that the small constant of the denominator shows; portions
    of one and two tokens carry (S, n, m) through the slot."""
    cfg = model_of([KC.layer(KC.mlstm(heads, dim, vdim, cap), None), KC.layer(KC.mlstm(heads, dim, vdim, cap), KC.dense(40))], width=88)
    check_alone(tmp_path, cfg, dtype, n_tokens=120, cuts=(1, 2, 1, 30, 3, 17, 2), scale=KC.SWINGING)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_cap_on_the_gates_changes_the_answer(tmp_path, dtype):
    cfg = model_of([KC.layer(KC.mlstm(3, 16, 24, 3.0), None)])
    d, cfg, w, toks, want = check_alone(tmp_path, cfg, dtype, cuts=None, scale=KC.SWINGING)
    got = run_alone(d, toks, dtype)
    for cap in (30.0, 1.0):
        cfg2 = json.loads(json.dumps(cfg))
        cfg2["layers"][0]["mixer"]["gate_cap"] = cap
        assert ((got - plain(cfg2, w, toks)).abs().max() / want.abs().max()).item() > 0.05, cap


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff,rows", [(88, 3), (24, 40), (200, 300)])
def test_dense_feed_forward_with_the_tanh_gelu(tmp_path, dtype, ff, rows):
    """The gate's sums reach several units either way, where the tanh form, the exact GELU and SiLU differ."""
    cfg = model_of([KC.layer(KC.attention(2, 1, 8, 8, 0.3), KC.dense(ff))])
    d, cfg, w, toks, want = check_alone(tmp_path, cfg, dtype, n_tokens=rows, cuts=None, scale=dict(KC.LIVELY, **{".gate": 14.0}),
                                          max_context=512)
    saved = PK.gelu_tanh
    try:
        PK.gelu_tanh = PK.silu
        other = plain(cfg, w, toks)
    finally:
        PK.gelu_tanh = saved
    assert ((other - want).abs().max() / want.abs().max()).item() > 0.02


ROUTERS = [
    dict(experts=4, top=1),                                                  # no rules but the correction
    dict(experts=6, top=2, identity=2, groups=(4, 2), scale=2.5, shared=56),
    dict(experts=5, top=6, identity=1),                                      # every expert chosen
    dict(experts=9, top=3, groups=(3, 1)),                                   # one group kept: exactly its experts
    dict(experts=1, top=2, identity=3, groups=(2, 1), scale=0.5),            # more identity experts than real ones
    dict(experts=12, top=4, identity=4, groups=(8, 3), shared=8),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("router", ROUTERS)
@pytest.mark.parametrize("rows", [3, 40, 300])
def test_routed_experts_choice_and_sum(tmp_path, dtype, router, rows):
    """The engine's chosen experts are the plain rule's, row by row (no row's choice is close: the router's
    scores are far apart), and the sum with identity and shared experts matches.  The corrections are large
    enough to change the choice of about a third of the rows, and the group rule that of others."""
    from ninfer_amd_mi50_b200.engine import load_runner
    cfg = model_of([KC.layer(KC.attention(2, 1, 8, 8, 0.3), KC.moe(24, **router))], width=80)
    d = KC.write_folder(cfg, 11, str(tmp_path / "m"))
    cfg, w = KC.read_folder(d)
    toks = random_tokens(rows, cfg["vocab"], 5)
    want = plain(cfg, w, toks)
    got, chosen_all = run_chosen(load_runner(d, options=options(dtype, max_context=512)), schedules.whole({"a": toks}))
    got, chosen = got["a"], chosen_all["a"][0]
    check(got, chosen_all["a"], cfg, w, toks, dtype, "sum", want32=want)
    # whatever the rounding of the router's input did to near-ties, a row's experts are different ones, allowed ones
    total = router["experts"] + router.get("identity", 0)
    assert int(chosen.min()) >= 0 and int(chosen.max()) < total
    assert all(len(set(row.tolist())) == router["top"] for row in chosen)
    if "groups" in router:
        per = total // router["groups"][0]
        assert all(len({e // per for e in row.tolist()}) <= router["groups"][1] for row in chosen)
    if dtype == "float32":
        # the plain rule on the plain model's own input to the router
        x = w["embed"][torch.tensor(toks)]
        f = cfg["layers"][0]
        h = PK.layer_norm(x, w["l0.norm1"], cfg["norm"]["eps"])
        k, v = PK.attention_keys_values(h, w, "l0.mix.", f["mixer"], cfg["norm"]["eps"], torch.arange(rows))
        x = x + PK.attention_mixer(h, w, "l0.mix.", f["mixer"], cfg["norm"]["eps"], torch.arange(rows), k, v)
        idx, _ = PK.route(PK.layer_norm(x, w["l0.norm2"], cfg["norm"]["eps"]), w, "l0.mlp.", f["mlp"]["router"])
        assert torch.equal(chosen.sort(dim=1).values, idx.sort(dim=1).values)
        plain_choice = PK.route(PK.layer_norm(x, w["l0.norm2"], cfg["norm"]["eps"]), {k_: v_ for k_, v_ in w.items() if not k_.endswith("correction")},
                                "l0.mlp.", f["mlp"]["router"])[0]
        if rows >= 40 and router["top"] < router["experts"] + router.get("identity", 0):
            assert not torch.equal(plain_choice.sort(dim=1).values, idx.sort(dim=1).values), "the correction changes nothing"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cap", [None, 0.7, 25.0])
def test_the_cap_on_the_logits_and_the_shared_table(tmp_path, dtype, cap):
    cfg = model_of([KC.layer(KC.attention(2, 1, 8, 8, 0.3), KC.dense(40))], cap=cap)
    d, cfg, w, toks, want = check_alone(tmp_path, cfg, dtype, cuts=None, scale=dict(KC.LIVELY, **{"embed": 8.0}))
    if cap is not None:
        assert want.abs().max().item() <= cap
    assert "head" not in w


# ---- the engine around the design ---------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs, want = folder
    toks = random_tokens(236, cfg["vocab"], 77)
    runner = load_runner(d, options=options(dtype))
    got, chosen = run_chosen(runner, schedules.tail_decoded({"a": toks}, tail=229))
    check(got["a"], chosen["a"], cfg, w, toks, dtype, f"{name} long decoding")
    assert all(n == 1024 // 16 for n in runner.cache.pages_free())


def test_pages_and_slots_that_are_used_again_hold_nothing_of_their_last_user(folder):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs, want = folder
    runner = load_runner(d, options=options("float32", num_sequences=1, cache_tokens=160))
    a, b = reqs["r0"], reqs["r3"]
    got = run(runner, schedules.whole({"a": a}) + schedules.portions({"b": b}) + schedules.whole({"c": a}))
    compare(got["b"], want["r3"], "float32", f"{name} second user of the pages and the slot")
    assert torch.equal(got["a"], got["c"])


def test_unequal_requests_in_one_batch_equal_each_alone(folder):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs, want = folder
    runner = load_runner(d, options=options("float32"))
    alone = run(runner, schedules.whole(reqs))
    pick = {r: reqs[r] for r in ("r0", "r1", "r3", "r4")}
    step = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in pick.items()], "end": list(pick)}]
    together = run(runner, step)
    for r in pick:
        assert (together[r] - alone[r]).abs().max() <= 1e-5 * alone[r].abs().max(), r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_rows_logits_do_not_depend_on_how_the_prompt_was_cut(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs, want = folder
    toks = reqs["r2"]
    runner = load_runner(d, options=options(dtype))
    a, chosen = run_chosen(runner, schedules.whole({"a": toks}))
    a = a["a"]
    b = run(runner, schedules.portions({"a": toks}, cuts=[2, 3, 50, 1, 16]))["a"]
    c = run(runner, schedules.tail_decoded({"a": toks}, tail=60))["a"]
    if dtype == "float32":
        for other in (b, c):
            assert (a - other).abs().max() <= 1e-5 * a.abs().max()
        return
    # bfloat16: a row is served by another kernel when it arrives alone, which rounds elsewhere; touchy rows aside
    steady = ~touchy_rows(cfg, w, toks, chosen["a"], plain(cfg, w, toks, chosen["a"]))
    for other in (b, c):
        diff = (a - other).abs().max(dim=1).values / a.abs().max()
        assert int((diff[steady] > 8e-2).sum()) <= max(1, len(diff) // 30) and diff.median() <= 1e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_replayed_from_graphs_equal_host_driven_ones(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs, want = folder
    pick = {r: reqs[r][:40] for r in ("r0", "r2", "r5")}
    steps = [{"entries": [{"id": r, "tokens": t[:25], "want": [24]} for r, t in pick.items()], "end": []}]
    for i in range(25, 40):
        steps.append({"entries": [{"id": r, "tokens": t[i:i + 1], "want": [0]} for r, t in pick.items()],
                      "end": list(pick) if i == 39 else []})
    host = run(load_runner(d, options=options(dtype)), steps)
    graphs = run(load_runner(d, options=options(dtype, use_graph=True)), steps)
    for r in pick:
        assert torch.equal(host[r], graphs[r]), r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folder, dtype):
    from ninfer_amd_mi50_b200.api import Ninfer
    name, d, cfg, w, reqs, want = folder
    prompts = [reqs["r1"], reqs["r3"], reqs["r4"], reqs["r0"][:40]]
    eng = Ninfer(d, max_context=128, prefill_chunk=16, num_sequences=3, dtype=dtype, page_size=16)
    got = eng.generate(prompts, max_new_tokens=10, temperature=0.0)
    for p, out in zip(prompts, got):
        assert len(out) == 10
        seq = list(p)
        for t in out:
            full = plain(cfg, w, seq)
            lg = full[-1]
            # the engine's token is the plain model's, or (bfloat16) one whose logit is as good as ties go
            slack = 1e-4 if dtype == "float32" else 3e-2
            if float(lg[t]) < float(lg.max()) - slack * float(lg.abs().max()):
                # (bfloat16) unless the row is one whose logits hang on a rounding anyway
                assert dtype == "bfloat16" and bool(touchy_rows(cfg, w, seq, None, full)[-1]), (name, len(seq), t, int(lg.argmax()))
            seq.append(t)


def test_trace_replay_program_runs_the_design(folder, tmp_path):
    """`bin/trace_run` picks the model class by config.json and gives the in-process logits."""
    import subprocess
    import sys
    import numpy as np
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs, want = folder
    small = {r: reqs[r] for r in ("r1", "r3", "r0")}
    steps = schedules.mixed(small, max_live=2, page=64, pool_tokens=192, tail=4)
    lines = "".join(json.dumps({"step": i, **st}) + "\n" for i, st in enumerate(steps))
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "192"], input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    runner = load_runner(d, options=options("float32", page_size=64, cache_tokens=192, max_context=192))
    got = run(runner, steps)
    rows = {r: 0 for r in small}
    for i, st in enumerate(steps):
        arr = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy()).double()
        at = 0
        for e in st["entries"]:
            n = len(e["want"])
            assert torch.equal(arr[at:at + n], got[e["id"]][rows[e["id"]]:rows[e["id"]] + n]), (i, e["id"])
            at += n
            rows[e["id"]] += n


@pytest.mark.parametrize("how", ["folder", "seed"])
def test_the_command_line_generates_from_the_design(tmp_path, how):
    """`bin/ninfer` on a Kopadra folder, and on a folder with only config.json and a seed."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg0, seed = KC.CONFIGS["sharing"]
    d = str(tmp_path / "m")
    if how == "folder":
        KC.write_folder(cfg0, seed, d)
    else:
        from ninfer_amd_mi50_b200.weights import write_random_model
        write_random_model(cfg0, seed, d)
    cfg, w = KC.read_folder(d)
    if how == "seed":
        os.remove(os.path.join(d, "model.safetensors"))
    prompt = random_tokens(30, cfg["vocab"], 12)
    cmd = [sys.executable, os.path.join(root, "bin", "ninfer"), d, "--prompt-ids", ",".join(map(str, prompt)),
           "--temperature", "0", "--max-new", "6", "--dtype", "fp32", "--prefill-chunk", "16", "--repeat-penalty", "1"]
    if how == "seed":
        cmd += ["--random-weights", str(seed)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    got = [int(x) for x in p.stdout.split()]
    assert len(got) == 6
    seq = list(prompt)
    for t in got:
        lg = plain(cfg, w, seq)[-1]
        assert float(lg[t]) >= float(lg.max()) - 1e-4 * float(lg.abs().max())
        seq.append(t)


def test_sampled_generation_and_a_request_preempted_and_recomputed(folder):
    """Sampling with a temperature through the scheduler, with a pool so small that a request is
    preempted and recomputed: its keys are written again from position 0, its state starts again at
    zero, and the tokens are those of a roomy pool."""
    from ninfer_amd_mi50_b200.api import Ninfer
    name, d, cfg, w, reqs, want = folder
    prompts = [reqs["r0"][:50], reqs["r3"], reqs["r5"][:60]]
    roomy = Ninfer(d, max_context=128, prefill_chunk=32, num_sequences=3, dtype="float32", page_size=16)
    want_tokens = roomy.generate(prompts, max_new_tokens=24, temperature=0.8, top_k=20, seed=5)
    tight = Ninfer(d, max_context=128, prefill_chunk=32, num_sequences=3, dtype="float32", page_size=16, cache_tokens=160)
    got = tight.generate(prompts, max_new_tokens=24, temperature=0.8, top_k=20, seed=5)
    assert got == want_tokens
