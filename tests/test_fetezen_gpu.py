"""The Fetezen design in the engine against the plain whole-sequence implementation
(`plain_fetezen`): each mechanism alone, whole prompts, token-by-token decoding, portions down to
two tokens, unequal requests in one batch, pages and slots used again, long decoding, and greedy
generation through the entry point.  Random weights are scaled out of their nearly linear range,
and where a fault would still hide (a far key, a chunk's edge, the sink) the inputs are made so
that it shows."""

import json
import math
import os

import pytest
import torch

import fetezen_configs as FC
import plain_fetezen as PF
import schedules
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = [70, 5, 131, 33, 2, 97]


def options(dtype, **kw):
    from ninfer_amd_mi50_b200.config import EngineOptions
    base = dict(dtype=dtype, page_size=16, num_sequences=4, max_context=256, cache_tokens=1024, use_graph=False)
    base.update(kw)
    return EngineOptions(**base)


def run(runner, steps):
    """Drive the runner through a schedule -> float64 logits per request, in the order asked."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.engine import StepEntry
    got = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if not runner.cache.is_open(e["id"]):
                runner.open(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        out = runner.step(entries)
        r = 0
        for e in st["entries"]:
            n = len(e["want"])
            got.setdefault(e["id"], []).append(out[r:r + n].double().cpu())
            r += n
        for rid in st["end"]:
            runner.close(rid)
        runner.cache.check()
    kernels.check_status("schedule")
    return {k: torch.cat(v) for k, v in got.items()}


def compare(got, want, dtype, what, bf16_bound=6e-2, bf16_scale=None):
    """float32 is the sharp comparison: 1e-4 of the largest logit for every row.  bfloat16 rounds
    every activation between kernels to 8 bits: every row within 6 %, the median row (of a request
    of 16 rows or more) within 1.5 %; `bf16_scale` is the size those 8 bits are taken of, where it
    is not the answer's own (logits under a cap far below their uncapped size)."""
    scale = want.abs().max().item()
    if dtype != "float32" and bf16_scale is not None:
        scale = bf16_scale
    err = (got - want).abs().max(dim=1).values / scale
    if dtype == "float32":
        assert err.max().item() <= 1e-4, f"{what}: row {int(err.argmax())} of {len(err)} differs by {err.max().item():.3e} of the scale"
        return err.max().item()
    assert torch.isfinite(got).all(), what
    assert err.max().item() <= bf16_bound, f"{what}: row {int(err.argmax())} of {len(err)} differs by {err.max().item():.3e} of the scale"
    if len(err) >= 16:
        assert err.median().item() <= 1.5e-2, f"{what}: the median row differs by {err.median().item():.3e} of the scale"
    return err.max().item()


def plain(cfg, w, tokens):
    return PF.forward(cfg, w, list(tokens))[0]


@pytest.fixture(scope="module", params=sorted(FC.CONFIGS))
def folder(request, tmp_path_factory):
    cfg, seed = FC.CONFIGS[request.param]
    d = str(tmp_path_factory.mktemp("fetezen") / request.param)
    FC.write_folder(cfg, seed, d)
    cfg, w = FC.read_folder(d)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 700 + i) for i, n in enumerate(LENGTHS)}
    return request.param, d, cfg, w, reqs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_the_plain_model(folder, dtype, how):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    make = {"whole": schedules.whole, "tail": lambda r: schedules.tail_decoded(r, tail=40),
            "portions": schedules.portions,
            # a pool of 320 tokens for 338 in all, three slots for six requests: pages and slots come back
            "mixed": lambda r: schedules.mixed(r, max_live=3, page=16, pool_tokens=320, tail=9)}[how]
    pool = 320 if how == "mixed" else 1024
    runner = load_runner(d, options=options(dtype, cache_tokens=pool, num_sequences=3 if how == "mixed" else 4))
    got = run(runner, make(reqs))
    assert all(n == pool // 16 for n in runner.cache.pages_free())
    for r, toks in reqs.items():
        compare(got[r], plain(cfg, w, toks), dtype, f"{name} {how} {r}")


# ---- each mechanism alone ---------------------------------------------------------------------

def model_of(layers, width=96, vocab=113, eps=1e-5, groups=None, streams=None, cap=None):
    c = {"architecture": "Fetezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if groups is not None:
        c["norm"]["groups"] = groups
    if streams is not None:
        c["streams"] = streams
    if cap is not None:
        c["logit_softcap"] = cap
    return c


def run_alone(d, tokens, dtype, cuts=None, **opt):
    from ninfer_amd_mi50_b200.engine import load_runner
    runner = load_runner(d, options=options(dtype, **opt))
    steps = schedules.whole({"a": tokens}) if cuts is None else schedules.portions({"a": tokens}, cuts=cuts)
    return run(runner, steps)["a"]


SMALL = FC.attention(2, 1, 8, 8, 0.3, chunk=16, rot=(100.0, 4))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams,groups,width", [(None, None, 96), (1, 1, 80), (2, 5, 100), (4, 3, 96), (3, 96, 96), (5, 2, 1032)])
def test_streams_and_the_norm_in_groups(tmp_path, dtype, streams, groups, width):
    """Two layers, the second without a feed-forward, so that every hand-over of the pending update
    occurs: sublayer to sublayer, layer to layer, and layer to the model's last norm.  The norm's
    weight varies over the vector and the embedding is loud in one group, so a norm over the whole
    vector (or groups that are not consecutive) gives other numbers."""
    cfg = model_of([FC.layer(SMALL, FC.dense(40)), FC.layer(SMALL, None)], width=width, groups=groups, streams=streams)
    g = torch.Generator().manual_seed(5)
    embed = torch.randn((cfg["vocab"], width), generator=g) * 0.5
    embed[:, : width // (groups or 1)] *= 9.0
    replace = {"embed": embed, "l0.norm1": torch.linspace(0.3, 1.7, width), "l0.norm2": torch.linspace(1.5, 0.4, width),
               "final.norm": torch.linspace(0.5, 1.5, width)}
    d = FC.write_folder(cfg, 61, str(tmp_path / "m"), replace=replace)
    cfg, w = FC.read_folder(d)
    toks = random_tokens(37, cfg["vocab"], 3)
    want = plain(cfg, w, toks)
    for cuts in (None, [1], [2, 5, 1]):
        compare(run_alone(d, toks, dtype, cuts=cuts), want, dtype, f"streams={streams} groups={groups} cuts={cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mixer", [
    FC.attention(6, 2, 16, 24, 0.3, chunk=21, rot=(500.0, 8)),
    FC.attention(1, 1, 64, 8, 0.125, chunk=64, rot=(10000.0, 64)),
    FC.attention(8, 8, 8, 40, 0.35, chunk=16),                          # nothing turned; a chunk of one page
    FC.attention(4, 1, 12, 20, 0.4, rot=(300.0, 6)),                    # every earlier position is seen
    FC.attention(3, 3, 128, 128, 0.09, chunk=1, rot=(50.0, 2)),         # a position sees itself and the sink
    FC.attention(16, 4, 32, 16, 0.2, chunk=47, rot=(1e6, 32)),
])
def test_attention_alone_whole_and_in_portions(tmp_path, dtype, mixer):
    cfg = model_of([FC.layer(mixer, None)], streams=2)
    d = FC.write_folder(cfg, 62, str(tmp_path / "m"))
    cfg, w = FC.read_folder(d)
    toks = random_tokens(90, cfg["vocab"], 6)
    want = plain(cfg, w, toks)
    for cuts in (None, [1], [2, 17, 3, 1], [20, 2]):
        compare(run_alone(d, toks, dtype, cuts=cuts), want, dtype, f"attention {mixer} cuts={cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_and_the_mixing_of_heads_each_change_the_answer(tmp_path, dtype):
    """With the mixing matrix a permutation, head h's softmax runs over another head's scores; with
    the identity and sinks of -40 the layer is ordinary attention.  Both are compared with the plain
    model, and the plain model's two answers are far apart, so neither can be left out unseen."""
    mixer = FC.attention(4, 2, 16, 16, 0.5, chunk=32, rot=(100.0, 16))
    cfg = model_of([FC.layer(mixer, None)])
    perm = torch.eye(4)[[2, 3, 0, 1]]
    toks = random_tokens(60, cfg["vocab"], 8)
    wants = []
    for k, (talk, sink) in enumerate([(perm, torch.tensor([4.0, 2.0, 0.0, -2.0])), (torch.eye(4), torch.full((4,), -40.0))]):
        d = FC.write_folder(cfg, 63, str(tmp_path / f"m{k}"), replace={"l0.mix.talk": talk, "l0.mix.sink": sink})
        c, w = FC.read_folder(d)
        wants.append(plain(c, w, toks))
        for cuts in (None, [1]):
            compare(run_alone(d, toks, dtype, cuts=cuts), wants[-1], dtype, f"talk/sink {k} cuts={cuts}")
    assert (wants[0] - wants[1]).abs().max() > 0.05 * wants[0].abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunks", [(21, 50), (64, 5), (16, None), (None, 16)])
def test_a_layer_reads_another_layers_keys_with_a_mask_of_its_own(tmp_path, dtype, chunks):
    own = FC.attention(4, 2, 16, 24, 0.3, chunk=chunks[0], rot=(500.0, 8))
    reader = FC.attention(4, 2, 16, 24, 0.4, chunk=chunks[1], rot=(500.0, 8), kv_from=0)
    other = FC.attention(2, 2, 8, 8, 0.4, chunk=9)
    cfg = model_of([FC.layer(own, FC.dense(40)), FC.layer(other, None), FC.layer(reader, None),
                    FC.layer(dict(reader, heads=2), FC.dense(24))], streams=2)
    d = FC.write_folder(cfg, 64, str(tmp_path / "m"))
    cfg, w = FC.read_folder(d)
    toks = random_tokens(120, cfg["vocab"], 9)
    want = plain(cfg, w, toks)
    for cuts in (None, [1], [2, 30, 7]):
        compare(run_alone(d, toks, dtype, cuts=cuts), want, dtype, f"kv_from chunks={chunks} cuts={cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff,act", [(88, [0.9, -0.6, 0.4, 0.25]), (24, [0.0, 1.0, 0.0, 0.0]), (200, [0.0, 0.0, 1.0, -0.5]),
                                    (7, [1.0, 0.0, 0.0, 0.0])])
def test_dense_feed_forward_with_the_polynomial_of_norms(tmp_path, dtype, ff, act):
    """Each power alone and all together.  The norm of a power is taken over the powers, not over
    the input: with a lively first product the three differ widely."""
    cfg = model_of([FC.layer(SMALL, FC.dense(ff))])
    d = FC.write_folder(cfg, 65, str(tmp_path / "m"), replace={"l0.mlp.act": torch.tensor(act)},
                        scale={".up": 12.0, ".down": 5.0})
    cfg, w = FC.read_folder(d)
    toks = random_tokens(40, cfg["vocab"], 10)
    z = torch.randn(5, ff, dtype=torch.float64)
    assert not torch.allclose(PF.unit_rms(z * z, 1e-5), PF.unit_rms(z, 1e-5) ** 2)
    compare(run_alone(d, toks, dtype), plain(cfg, w, toks), dtype, f"dense ff={ff} act={act}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,shared,rows", [(4, 1, None, 3), (6, 2, 56, 40), (5, 5, None, 40), (9, 3, 8, 300), (1, 1, 16, 20)])
def test_experts_chosen_by_the_table_over_token_ids(tmp_path, dtype, experts, top, shared, rows):
    """The table's rows differ from id to id and the experts from one another (their weights are
    drawn one by one), so a token that takes another id's row, or weights other than 1 / top, shows.
    The shared expert's gate is made lively: from nearly shut to nearly open over the tokens."""
    cfg = model_of([FC.layer(SMALL, FC.moe(24, experts, top, shared=shared))], streams=2)
    d = FC.write_folder(cfg, 66, str(tmp_path / "m"), scale={".up": 10.0, ".down": 4.0, ".shared.sg": 60.0})
    cfg, w = FC.read_folder(d)
    toks = random_tokens(rows, cfg["vocab"], 11)
    table = w["l0.mlp.table"].long()
    assert tuple(table.shape) == (cfg["vocab"], top) and all(len(set(r.tolist())) == top for r in table)
    want = plain(cfg, w, toks)
    for cuts in (None, [1], [2, 7]) if rows <= 40 else (None,):
        compare(run_alone(d, toks, dtype, cuts=cuts, max_context=512), want, dtype, f"table moe {experts}/{top} cuts={cuts}")
    # the same tokens with every id moved by one take other experts: the table is read by id, not by place
    if experts > top:
        moved = [(t + 1) % cfg["vocab"] for t in toks]
        assert (plain(cfg, w, moved) - want).abs().max() > 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cap", [None, 0.7, 30.0])
def test_the_cap_on_the_logits(tmp_path, dtype, cap):
    cfg = model_of([FC.layer(SMALL, None)], cap=cap)
    d = FC.write_folder(cfg, 67, str(tmp_path / "m"), scale={"head": 30.0})
    cfg, w = FC.read_folder(d)
    toks = random_tokens(20, cfg["vocab"], 12)
    want = plain(cfg, w, toks)
    if cap:
        assert want.abs().max() <= cap and (cap > 5 or want.abs().max() > 0.9 * cap)     # the low cap is met
    # the cap's slope is at most 1: rounding before it weighs as much as in the uncapped logits
    free = plain(dict(cfg, logit_softcap=None), w, toks).abs().max().item()
    compare(run_alone(d, toks, dtype), want, dtype, f"cap={cap}", bf16_scale=max(free, want.abs().max().item()))


# ---- the attention kernel on inputs made so that one key decides ------------------------------

def plain_attention_row(q, keys, vals, pos, scale, talk, sink, chunk):
    """q [H, D] at position `pos`; keys [n, G, D], vals [n, G, Dv] -> [H, Dv] by the design's rule."""
    H, G = q.shape[0], keys.shape[1]
    lo = (pos // chunk) * chunk if chunk else 0
    k = keys[lo:pos + 1].repeat_interleave(H // G, dim=1)            # [n, H, D]: head h reads key head h // (H / G)
    v = vals[lo:pos + 1].repeat_interleave(H // G, dim=1)
    mixed = talk @ (torch.einsum("hd,jhd->hj", q, k) * scale)         # [H, n]
    m = torch.maximum(mixed.max(dim=1).values, sink)
    e = torch.exp(mixed - m[:, None])
    p = e / (e.sum(dim=1) + torch.exp(sink - m))[:, None]
    return torch.einsum("hj,jhd->hd", p, v)


@pytest.mark.parametrize("dtype,H,G,D,Dv", [(torch.float32, 4, 2, 16, 24), (torch.bfloat16, 4, 2, 16, 24), (torch.bfloat16, 4, 1, 64, 48),
                                            (torch.bfloat16, 8, 1, 32, 16), (torch.float32, 3, 3, 12, 20), (torch.bfloat16, 16, 4, 128, 128)])
@pytest.mark.parametrize("chunk", [37, 16, 64, 0, 150, 1])
def test_one_loud_key_is_heard_just_inside_and_not_just_outside_a_chunk(dtype, H, G, D, Dv, chunk):
    """The cache is filled by hand: every key is faint but one, whose score towers.  Placed at the
    chunk's first position, on a page's border, or (without chunks) hundreds of positions back, it
    takes the whole output; one position before the chunk's start it must not show, and the sink
    alone is then left beside faint keys.  Rows are served both as a prompt's portion and as single
    decoded tokens; the pages stand in an order of their own."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.parts.base import StepContext
    dev = torch.device("cuda")
    page, n = 16, 200
    gen = torch.Generator().manual_seed(3)
    talk = (torch.eye(H) * 0.9 + torch.randn((H, H), generator=gen).abs() * 0.05).float()      # positive: loud stays loud
    sink = torch.linspace(1.0, -3.0, H).float()
    pos = n - 1
    lo = (pos // chunk) * chunk if chunk else 0
    places = sorted({lo, lo - 1, lo + 1, 0, pos, pos - 1, 15, 16, 63, 64, pos - 37, pos - 64, pos - 65} - {-1})
    places = [j for j in places if 0 <= j <= pos]
    W = G * (D + Dv)
    for loud in places:
        keys = (torch.randn((n, G, D), generator=gen) * 0.05).to(dtype).double()
        vals = torch.randn((n, G, Dv), generator=gen).to(dtype).double()
        direction = torch.ones(D, dtype=torch.float64) / math.sqrt(D)
        keys[loud] = (direction * 30.0).to(dtype).double()
        q_all = (direction[None, None, :] * 2.0 + torch.randn((n, H, D), generator=gen).double() * 0.05).to(dtype)
        pages = torch.zeros((n // page + 2, page, W), dtype=dtype)
        table = list(range(n // page + 1))[::-1]
        for j in range(n):
            pages[table[j // page], j % page, :G * D] = keys[j].reshape(-1).to(dtype)
            pages[table[j // page], j % page, G * D:] = vals[j].reshape(-1).to(dtype)
        for first_row in (pos, pos - 9, pos - 70):                     # one decoded token; portions of 10 and 71 rows
            rows = list(range(first_row, pos + 1))
            T = len(rows)
            mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            ctx = StepContext(dtype=dtype, device=dev, T=T, S=1, token_ids=mk([0] * T), positions=mk(rows), row_seg=mk([0] * T),
                              seg_row0=mk([0, T]), seg_pos0=mk([first_row]), seg_slot=mk([0]), logit_rows=mk([T - 1]),
                              seg_len_host=[T], seg_pos0_host=[first_row], max_rows_per_seg=T, max_context=n)
            q = q_all[rows].reshape(T, H * D).contiguous().to(dev)
            out = kernels.talking_attention(q, H, G, D, Dv, pages.to(dev), mk([table]), page, ctx, chunk, 0.7,
                                            talk.to(dev), sink.to(dev)).double().cpu().reshape(T, H, Dv)
            check = rows if T <= 10 else rows[::7] + [pos]
            for p in check:
                want = plain_attention_row(q_all[p].double(), keys, vals, p, 0.7, talk.double(), sink.double(), chunk)
                tol = 1e-5 if dtype == torch.float32 else 2e-2
                assert (out[p - first_row] - want).abs().max() <= tol * max(1.0, want.abs().max()), (loud, p, chunk, T)
        share = plain_attention_row(q_all[pos].double(), keys, vals, pos, 0.7, talk.double(), sink.double(), chunk)
        if loud >= lo:
            assert (share[H - 1] - vals[loud, G - 1]).abs().max() < 1e-3      # the loud key takes the whole output
        else:
            assert (share[H - 1] - vals[loud, G - 1]).abs().max() > 0.3       # and none of it when the chunk hides it


# ---- the tensor-core kernel: clusters of every size, cut rows, single rows split over their keys ----

def _step_context(segs, dev, graph=False):
    from ninfer_amd_mi50_b200.parts.base import StepContext
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    rows, row_seg, row0 = [], [], [0]
    for s, (p0, n) in enumerate(segs):
        rows += list(range(p0, p0 + n)); row_seg += [s] * n; row0.append(len(rows))
    T = len(rows)
    return StepContext(dtype=torch.bfloat16, device=dev, T=T, S=len(segs), token_ids=mk([0] * T), positions=mk(rows),
                       row_seg=mk(row_seg), seg_row0=mk(row0), seg_pos0=mk([p for p, _ in segs]),
                       seg_slot=mk(list(range(len(segs)))), logit_rows=mk([T - 1]),
                       seg_len_host=None if graph else [n for _, n in segs],
                       seg_pos0_host=None if graph else [p for p, _ in segs],
                       max_rows_per_seg=max(n for _, n in segs), max_context=max(p + n for p, n in segs)), rows, row_seg


@pytest.mark.parametrize("H,G,D,Dv,chunk", [(4, 4, 64, 48, 48), (8, 8, 128, 128, 96), (8, 2, 128, 64, 0), (16, 4, 64, 128, 100),
                                            (32, 32, 128, 128, 70), (12, 4, 64, 64, 64), (24, 8, 32, 48, 33), (3, 3, 16, 16, 7),
                                            (5, 1, 48, 32, 200), (2, 1, 16, 80, 32), (1, 1, 128, 16, 0)])
@pytest.mark.parametrize("segs,graph", [([(0, 75)], False), ([(37, 90), (199, 1), (0, 17), (130, 2)], False),
                                         ([(199, 1), (64, 1), (63, 1), (0, 1), (31, 1), (32, 1)], False),
                                         ([(199, 1), (96, 1), (95, 1), (0, 1)], True),
                                         ([(480, 100), (1030, 3)], False)])
def test_tensor_core_attention_against_the_plain_rule_and_the_plain_kernel(H, G, D, Dv, chunk, segs, graph):
    """The tensor-core kernel deals the heads out over a cluster of CTAs (1, 2, 4 or 8, by the sizes) that
    read one another's scores; prompt portions that begin inside a chunk and end inside another, rows
    at a chunk's first and last position, and steps of single rows, whose keys are cut into runs and
    merged (also as a captured step sees them, without lengths on the host), and a step of few tiles far
    into a request, whose keys are cut into runs counted from position 0, are compared row by row with the
    rule in float64 and with the plain kernel."""
    from ninfer_amd_mi50_b200 import kernels
    from ninfer_amd_mi50_b200.kernels import ops
    dev = torch.device("cuda")
    assert kernels.lib.load().nf_talking_attention_mma_heads_per_cta(H, G, D, Dv, 0) > 0
    gen = torch.Generator().manual_seed(H * 131 + D)
    page, S = 16, len(segs)
    n = max(p + k for p, k in segs)
    per = (n + page - 1) // page
    keys = (torch.randn((S, n, G, D), generator=gen) * 0.6).to(torch.bfloat16)
    vals = torch.randn((S, n, G, Dv), generator=gen).to(torch.bfloat16)
    order = (torch.randperm(S * per, generator=gen) + 1).reshape(S, per)
    pages = torch.zeros((S * per + 1, page, G * (D + Dv)), dtype=torch.bfloat16)
    for s in range(S):
        for j in range(n):
            pages[order[s, j // page], j % page] = torch.cat([keys[s, j].reshape(-1), vals[s, j].reshape(-1)])
    talk = (torch.eye(H) * 0.8 + torch.randn((H, H), generator=gen) * 0.2).float()
    sink = torch.linspace(1.5, -2.0, H).float()
    ctx, rows, row_seg = _step_context(segs, dev, graph)
    q = (torch.randn((len(rows), H, D), generator=gen) * 0.8).to(torch.bfloat16)
    args = (q.reshape(len(rows), H * D).to(dev), H, G, D, Dv, pages.to(dev), order.to(torch.int32).to(dev), page, ctx,
            chunk, D ** -0.5, talk.to(dev), sink.to(dev))
    old = ops.TUNING["bf16_attention"]
    try:
        ops.TUNING["bf16_attention"] = "auto"
        got = kernels.talking_attention(*args).double().cpu().reshape(len(rows), H, Dv)
        ops.TUNING["bf16_attention"] = "generic"
        slow = kernels.talking_attention(*args).double().cpu().reshape(len(rows), H, Dv)
    finally:
        ops.TUNING["bf16_attention"] = old
    for r, (p, s) in enumerate(zip(rows, row_seg)):
        want = plain_attention_row(q[r].double(), keys[s].double(), vals[s].double(), p, D ** -0.5, talk.double(),
                                   sink.double(), chunk)
        bound = 1.2e-2 * max(1.0, want.abs().max().item())            # the output is rounded to bfloat16
        assert (got[r] - want).abs().max() <= bound, (r, p, s)
        assert (got[r] - slow[r]).abs().max() <= bound, (r, p, s)


# ---- pages, slots, long decoding ----------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_lets_chunks_begin_and_end_among_decoded_tokens(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    toks = random_tokens(236, cfg["vocab"], 77)
    runner = load_runner(d, options=options(dtype))
    got = run(runner, schedules.tail_decoded({"a": toks}, tail=229))
    compare(got["a"], plain(cfg, w, toks), dtype, f"{name} long decoding")
    assert all(n == 1024 // 16 for n in runner.cache.pages_free())


def test_pages_that_are_used_again_hold_nothing_of_their_last_user(folder):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    runner = load_runner(d, options=options("float32", num_sequences=1, cache_tokens=160))
    a, b = reqs["r0"], reqs["r3"]
    got = run(runner, schedules.whole({"a": a}) + schedules.portions({"b": b}) + schedules.whole({"c": a}))
    compare(got["b"], plain(cfg, w, b), "float32", f"{name} second user of the pages")
    assert torch.equal(got["a"], got["c"])


def test_unequal_requests_in_one_batch_equal_each_alone(folder):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    runner = load_runner(d, options=options("float32"))
    alone = run(runner, schedules.whole(reqs))
    pick = {r: reqs[r] for r in ("r0", "r1", "r3", "r4")}
    step = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in pick.items()], "end": list(pick)}]
    together = run(runner, step)
    for r in pick:
        assert (together[r] - alone[r]).abs().max() <= 1e-5 * alone[r].abs().max(), r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_rows_logits_do_not_depend_on_how_the_prompt_was_cut(folder, dtype):
    """Beyond the comparison with the plain model: the same row served in a whole prompt, in
    portions, and decoded alone differs by rounding of the products only."""
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
    toks = reqs["r2"]
    runner = load_runner(d, options=options(dtype))
    a = run(runner, schedules.whole({"a": toks}))["a"]
    b = run(runner, schedules.portions({"a": toks}, cuts=[2, 3, 50, 1, 16]))["a"]
    c = run(runner, schedules.tail_decoded({"a": toks}, tail=60))["a"]
    bound = 1e-5 if dtype == "float32" else 4e-2
    for other in (b, c):
        assert (a - other).abs().max() <= bound * a.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_replayed_from_graphs_equal_host_driven_ones(folder, dtype):
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
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
    name, d, cfg, w, reqs = folder
    prompts = [reqs["r1"], reqs["r3"], reqs["r4"], reqs["r0"][:40]]
    eng = Ninfer(d, max_context=128, prefill_chunk=16, num_sequences=3, dtype=dtype, page_size=16)
    got = eng.generate(prompts, max_new_tokens=10, temperature=0.0)
    for p, out in zip(prompts, got):
        assert len(out) == 10
        seq = list(p)
        for t in out:
            lg = plain(cfg, w, seq)[-1]
            # the engine's token is the plain model's, or (bfloat16) one whose logit is as good as ties go
            slack = 1e-4 if dtype == "float32" else 3e-2
            assert float(lg[t]) >= float(lg.max()) - slack * float(lg.abs().max()), (name, len(seq), t, int(lg.argmax()))
            seq.append(t)


def test_trace_replay_program_runs_the_design(folder, tmp_path):
    """`bin/trace_run` picks the model class by config.json and gives the in-process logits."""
    import subprocess
    import sys
    import numpy as np
    from ninfer_amd_mi50_b200.engine import load_runner
    name, d, cfg, w, reqs = folder
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
    """`bin/ninfer` on a Fetezen folder, and on a folder with only config.json and a seed."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg0, seed = FC.CONFIGS["sharing"]
    d = str(tmp_path / "m")
    if how == "folder":
        FC.write_folder(cfg0, seed, d)
    else:
        from ninfer_amd_mi50_b200.weights import write_random_model
        write_random_model(cfg0, seed, d)
    cfg, w = FC.read_folder(d)
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
    preempted and recomputed: its keys are written again from position 0, and the tokens are those
    of a roomy pool."""
    from ninfer_amd_mi50_b200.api import Ninfer
    name, d, cfg, w, reqs = folder
    prompts = [reqs["r0"][:50], reqs["r3"], reqs["r5"][:60]]
    roomy = Ninfer(d, max_context=128, prefill_chunk=32, num_sequences=3, dtype="float32", page_size=16)
    want = roomy.generate(prompts, max_new_tokens=24, temperature=0.8, top_k=20, seed=5)
    tight = Ninfer(d, max_context=128, prefill_chunk=32, num_sequences=3, dtype="float32", page_size=16, cache_tokens=160)
    got = tight.generate(prompts, max_new_tokens=24, temperature=0.8, top_k=20, seed=5)
    assert got == want
