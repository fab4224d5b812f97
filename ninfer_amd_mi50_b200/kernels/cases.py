"""Representative kernel workloads, one layer's worth, for profilers and quick timing; the layer
sizes come from a named set (`--sizes`, by default those of Qwen1.5-MoE-A2.7B):

    python -m ninfer_amd_mi50_b200.kernels.cases moe_prefill
    ncu --set full --clock-control none -k regex:grouped_gemm_tc -c 2 \
        python -m ninfer_amd_mi50_b200.kernels.cases moe_prefill

(run the plain command first and profile only after it exits 0; without `--clock-control none`
a profiler locks the clocks of a GPU that others share.)

Each case warms its kernels up and then runs them a few times; with `--time` it prints the
median time per call from CUDA events (launch included) with an L2 flush between calls.  A case holds about
1.5 GB on the device, larger than L2, so DRAM figures mean something.
"""

from __future__ import annotations

import argparse
import math
import sys
from types import SimpleNamespace

import torch

# name -> layer sizes (config.json's meanings): the two large configurations that are measured
SIZES = {
    "a2.7b": dict(H=2048, I=1408, IS=5632, E=60, K_TOP=4, V=151936, HQ=16, HKV=16, D=128),
    "57b-a14b": dict(H=3584, I=2560, IS=20480, E=64, K_TOP=8, V=151936, HQ=28, HKV=4, D=128),
}
PAGE = 64
H = I = IS = E = K_TOP = V = HQ = HKV = D = 0     # set from SIZES by `use_sizes`


def use_sizes(name: str) -> None:
    globals().update(SIZES[name])


use_sizes("a2.7b")


def _routing(tokens: int, seed: int, device):
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(E, generator=g)[:K_TOP] for _ in range(tokens)])
    return idx.to(torch.int32).to(device)


def _experts(device):
    from . import pack_weights
    w13 = pack_weights((torch.randn(E, 2 * I, H, device=device) * 0.02).bfloat16(), True)
    w2 = pack_weights((torch.randn(E, H, I, device=device) * 0.02).bfloat16(), False)
    return w13, w2


def case_moe(tokens: int, device):
    """Routed experts: both products for `tokens` tokens with uniform random routing."""
    from . import moe_gemm1, moe_gemm2, moe_plan
    w13, w2 = _experts(device)
    x = torch.randn(tokens, H, device=device).bfloat16()
    plan = moe_plan(_routing(tokens, tokens, device), E)
    act = moe_gemm1(x, w13, plan, K_TOP)
    return [("moe_gemm1", lambda: moe_gemm1(x, w13, plan, K_TOP)),
            ("moe_gemm2", lambda: moe_gemm2(act, w2, plan))]


def case_moe_stream(tokens: int, device, whole_block: bool):
    """The persistent launch of a decode step: both products of the routed experts for `tokens`
    tokens (plan given), or with `whole_block` the routing and the shared expert as well."""
    from . import TUNING, moe_experts, moe_plan, pack_shared_expert, route_and_run_experts
    TUNING.update(moe_stream_min_tokens=1, moe_stream_max_tokens=64, moe_stream_route_max_tokens=64,
                  moe_stream_shared_max_tokens=64)
    w13, w2 = _experts(device)
    x = torch.randn(tokens, H, device=device).bfloat16()
    if not whole_block:
        plan = moe_plan(_routing(tokens, tokens, device), E)
        return [("moe_experts", lambda: moe_experts(x, w13, w2, plan, K_TOP))]
    wr = torch.randn(E + 1, H, device=device) * 0.05
    shared = pack_shared_expert((torch.randn(2 * IS, H, device=device) * 0.02).bfloat16(),
                                (torch.randn(H, IS, device=device) * 0.02).bfloat16(), I)
    return [("route_experts_shared", lambda: route_and_run_experts(x, wr, E, K_TOP, False, w13, w2, shared=shared))]


def case_attention_prefill(tokens: int, device):
    """One fresh prompt of `tokens` tokens: flash prefill attention over the paged cache."""
    from . import paged_attention
    from ..parts.base import StepContext
    n_pages = (tokens + PAGE - 1) // PAGE
    pages = torch.randn(n_pages + 1, 2, HKV, PAGE, D, device=device).bfloat16()
    bt = torch.arange(n_pages, dtype=torch.int32, device=device).view(1, -1)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    ctx = StepContext(dtype=torch.bfloat16, device=torch.device(device), T=tokens, S=1, token_ids=mk([0]),
                      positions=torch.arange(tokens, dtype=torch.int32, device=device),
                      row_seg=torch.zeros(tokens, dtype=torch.int32, device=device), seg_row0=mk([0, tokens]),
                      seg_pos0=mk([0]), seg_slot=mk([0]), logit_rows=mk([]), seg_len_host=[tokens],
                      seg_pos0_host=[0], max_rows_per_seg=tokens, max_context=tokens)
    qkv = torch.randn(tokens, (HQ + 2 * HKV) * D, device=device).bfloat16()
    return [("prefill_attention", lambda: paged_attention(qkv, HQ, HKV, D, pages, bt, PAGE, ctx, 0, 1 / math.sqrt(D)))]


def case_attention_decode(batch: int, context: int, device):
    """`batch` requests of `context` tokens each, one new row per request."""
    from . import paged_attention
    per = context // PAGE + 1
    pages = torch.randn(batch * per + 1, 2, HKV, PAGE, D, device=device).bfloat16()
    bt = torch.arange(batch * per, dtype=torch.int32, device=device).view(batch, per)
    ctx = SimpleNamespace(positions=torch.full((batch,), context, dtype=torch.int32, device=device),
                          row_seg=torch.arange(batch, dtype=torch.int32, device=device), all_single=True,
                          max_context=context + 1)
    qkv = torch.randn(batch, (HQ + 2 * HKV) * D, device=device).bfloat16()
    return [("decode_attention", lambda: paged_attention(qkv, HQ, HKV, D, pages, bt, PAGE, ctx, 0, 1 / math.sqrt(D)))]


def case_dense_decode(batch: int, device):
    """The dense products of a decode step: QKV, O, shared expert, LM head."""
    from . import linear, linear_swiglu
    mk = lambda n, k: (torch.randn(n, k, device=device) * 0.02).bfloat16()
    wqkv, wo, ws13, ws2, head = mk((HQ + 2 * HKV) * D, H), mk(H, HQ * D), mk(2 * IS, H), mk(H, IS), mk(V, H)
    x, xs = torch.randn(batch, H, device=device).bfloat16(), torch.randn(batch, IS, device=device).bfloat16()
    return [("qkv", lambda: linear(x, wqkv)), ("o_proj", lambda: linear(x, wo)),
            ("shared_gate_up", lambda: linear_swiglu(x, ws13)), ("shared_down", lambda: linear(xs, ws2)),
            ("lm_head", lambda: linear(x, head, out_dtype=torch.float32))]


def case_small_decode(batch: int, device):
    """The short kernels between a decode step's products: norm with residual add, router with
    plan, weighted sum of the experts' outputs joined with the next norm."""
    from . import add_rmsnorm, moe_combine_add_rmsnorm, moe_plan, route
    h = torch.randn(batch, H, device=device)
    delta = torch.randn(batch, H, device=device).bfloat16()
    w = torch.ones(H, device=device)
    out = torch.empty(batch, H, device=device, dtype=torch.bfloat16)
    wr = torch.randn(E + 1, H, device=device) * 0.02
    plan = moe_plan(_routing(batch, batch, device), E)
    y = torch.randn(batch * K_TOP, H, device=device).bfloat16()
    wts = torch.rand(batch, K_TOP, device=device)
    gate = torch.randn(batch, 1, device=device)
    return [("add_rmsnorm", lambda: add_rmsnorm(h, delta, w, 1e-6, out)),
            ("route", lambda: route(out, wr, E, K_TOP, False)),
            ("combine_add_rmsnorm", lambda: moe_combine_add_rmsnorm(y, plan, wts, delta, gate, h, None, w, 1e-6, out))]


def _one_request(tokens: int, device, single: bool = False, context: int = 0):
    """Step metadata for one prompt of `tokens` rows, or (`single`) `tokens` requests of one row at `context`."""
    from ..parts.base import StepContext
    if single:
        pos = torch.full((tokens,), context, dtype=torch.int32)
        seg, row0, lens, pos0, S = torch.arange(tokens, dtype=torch.int32), torch.arange(tokens + 1, dtype=torch.int32), [1] * tokens, [context] * tokens, tokens
    else:
        pos = torch.arange(tokens, dtype=torch.int32)
        seg, row0, lens, pos0, S = torch.zeros(tokens, dtype=torch.int32), torch.tensor([0, tokens], dtype=torch.int32), [tokens], [0], 1
    z = torch.zeros(1, dtype=torch.int32, device=device)
    return StepContext(dtype=torch.bfloat16, device=torch.device(device), T=tokens, S=S, token_ids=z, positions=pos.to(device),
                       row_seg=seg.to(device), seg_row0=row0.to(device), seg_pos0=z, seg_slot=torch.arange(S, dtype=torch.int32, device=device),
                       logit_rows=z, seg_len_host=lens, seg_pos0_host=pos0, max_rows_per_seg=max(lens),
                       max_context=(context + 1) if single else tokens)


def case_latent_attention(tokens: int, device, single: bool = False, context: int = 0):
    """Attention over latent rows (width 512 + 64 rotated, HQ heads): a prompt of `tokens` rows, or
    `tokens` decoded rows that each see `context` cached rows."""
    from . import latent_attention
    R, Dr, dim = 512, 64, 128
    ctx = _one_request(tokens, device, single, context)
    held = (context + 1) if single else tokens
    per = (held + PAGE - 1) // PAGE
    pages = (torch.randn(ctx.S * per + 1, PAGE, R + Dr, device=device) * 0.5).bfloat16()
    bt = torch.arange(ctx.S * per, dtype=torch.int32, device=device).view(ctx.S, per)
    q_abs = (torch.randn(HQ, tokens, R, device=device) * 0.1).bfloat16()
    q = (torch.randn(tokens, HQ * (dim + Dr), device=device) * 0.1).bfloat16()
    sink = torch.zeros(HQ, device=device)
    return [("latent_attention", lambda: latent_attention(q_abs, q, dim + Dr, dim, Dr, pages, bt, PAGE, ctx, sink, 0.07))]


def case_state_space(tokens: int, device, single: bool = False):
    """The convolution and the selective scan of a state-space mixer with 2 H inner channels (heads of 64,
    state 128, 8 groups): a prompt of `tokens` rows, or `tokens` requests of one row."""
    from . import causal_conv_silu, ssd_scan
    heads, P, N, G, K = 2 * H // 64, 64, 128, 8, 4
    inner = heads * P
    C = inner + 2 * G * N
    ctx = _one_request(tokens, device, single)
    proj = (torch.randn(tokens, 2 * inner + 2 * G * N + heads, device=device) * 0.5).bfloat16()
    state = torch.zeros(ctx.S + 1, (K - 1) * C + heads * P * N, device=device)
    taps, bias, z = torch.randn(K, C, device=device) * 0.3, torch.zeros(C, device=device), torch.zeros(heads, device=device)
    xbc = causal_conv_silu(proj, inner, C, taps, bias, state, ctx)
    return [("causal_conv_silu", lambda: causal_conv_silu(proj, inner, C, taps, bias, state, ctx)),
            ("ssd_scan", lambda: ssd_scan(xbc, 0, inner, inner + G * N, proj, 2 * inner + 2 * G * N, z, z, z, state,
                                          (K - 1) * C, ctx, heads, P, N, G))]


def case_linear_attention(tokens: int, device, single: bool = False, dim: int = 128, rotary: bool = False):
    """The recurrence of a linear attention with a fixed decay per head (HQ heads of `dim` x 128): a prompt of
    `tokens` rows, or `tokens` requests of one row.  `rotary`: q and k are turned and k scaled (retention);
    otherwise q, k, v pass SiLU (lightning)."""
    from . import decay_linear_attention, group_rmsnorm_gate, GATE_SIGMOID
    V = 128
    ctx = _one_request(tokens, device, single)
    if not single:
        ctx.seg_pos0 = torch.zeros(1, dtype=torch.int32, device=device)
    else:
        ctx.seg_pos0 = torch.full((tokens,), 2048, dtype=torch.int32, device=device)
    proj = (torch.randn(tokens, 2 * HQ * dim + 2 * HQ * V, device=device) * 0.5).bfloat16()
    state = torch.zeros(ctx.S + 1, HQ * V * dim, device=device)
    decay = torch.full((HQ,), 0.97, device=device)
    inv = torch.rand(dim // 2, device=device)
    w = torch.ones(HQ * V, device=device)
    run = lambda: decay_linear_attention(proj, 0, HQ * dim, 2 * HQ * dim, decay, inv if rotary else None,
                                         dim if rotary else 0, dim ** -0.5 if rotary else 1.0, not rotary, state, ctx,
                                         HQ, dim, V)
    o = run()
    return [("decay_linear_attention", run),
            ("group_rmsnorm_gate", lambda: group_rmsnorm_gate(o, proj, 2 * HQ * dim + HQ * V, w, 1e-6, 1, GATE_SIGMOID,
                                                              torch.bfloat16))]


def case_window_attention(tokens: int, device, single: bool = False, context: int = 0, window: int = 1024, keep: int = 4):
    """Softmax attention with a distance slope per head, a window that keeps the first `keep` keys and a head
    gate (HQ query and key heads of 128): a prompt of `tokens` rows, or `tokens` decoded rows at `context`."""
    from . import biased_window_attention
    D = 128
    ctx = _one_request(tokens, device, single, context)
    held = (context + 1) if single else tokens
    per = (held + PAGE - 1) // PAGE
    pages = (torch.randn(ctx.S * per + 1, 2, HQ, PAGE, D, device=device) * 0.5).bfloat16()
    bt = torch.arange(ctx.S * per, dtype=torch.int32, device=device).view(ctx.S, per)
    q = (torch.randn(tokens, HQ * D, device=device) * 0.5).bfloat16()
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / HQ) for h in range(HQ)], device=device)
    gate = torch.randn(tokens, HQ, device=device)
    return [("biased_window_attention", lambda: biased_window_attention(q, HQ, HQ, D, pages, bt, PAGE, ctx, window, keep,
                                                                        D ** -0.5, slopes, gate, 0))]


def case_talking_attention(tokens: int, device, single: bool = False, context: int = 0, chunk: int = 1536):
    """Softmax attention whose heads' scores are mixed before the softmax, over chunks of `chunk` positions and
    with a sink (HQ query and key heads of 128): a prompt of `tokens` rows, or `tokens` decoded rows at `context`."""
    from . import talking_attention
    D = 128
    ctx = _one_request(tokens, device, single, context)
    held = (context + 1) if single else tokens
    per = (held + PAGE - 1) // PAGE
    pages = (torch.randn(ctx.S * per + 1, PAGE, HQ * 2 * D, device=device) * 0.5).bfloat16()
    bt = torch.arange(ctx.S * per, dtype=torch.int32, device=device).view(ctx.S, per)
    q = (torch.randn(tokens, HQ * D, device=device) * 0.5).bfloat16()
    talk = torch.eye(HQ, device=device) * 0.8 + torch.randn(HQ, HQ, device=device) * 0.1
    sink = torch.zeros(HQ, device=device)
    return [("talking_attention", lambda: talking_attention(q, HQ, HQ, D, D, pages, bt, PAGE, ctx, chunk, D ** -0.5,
                                                            talk, sink))]


CASES = {
    "talking_attention_prefill": lambda dev: case_talking_attention(2048, dev),
    "talking_attention_decode8": lambda dev: case_talking_attention(8, dev, True, 2047),
    "linear_attention_prefill": lambda dev: case_linear_attention(2048, dev),
    "linear_attention_decode8": lambda dev: case_linear_attention(8, dev, True),
    "retention_prefill": lambda dev: case_linear_attention(2048, dev, dim=64, rotary=True),
    "window_attention_prefill": lambda dev: case_window_attention(2048, dev),
    "window_attention_decode8": lambda dev: case_window_attention(8, dev, True, 2048),
    "latent_attention_prefill": lambda dev: case_latent_attention(2048, dev),
    "latent_attention_decode8": lambda dev: case_latent_attention(8, dev, True, 2048),
    "state_space_prefill": lambda dev: case_state_space(2048, dev),
    "state_space_decode8": lambda dev: case_state_space(8, dev, True),
    "moe_prefill": lambda dev: case_moe(2048, dev),
    "moe_decode8": lambda dev: case_moe(8, dev),
    "moe_decode64": lambda dev: case_moe(64, dev),
    "moe_stream_decode8": lambda dev: case_moe_stream(8, dev, False),
    "moe_stream_decode16": lambda dev: case_moe_stream(16, dev, False),
    "moe_stream_decode64": lambda dev: case_moe_stream(64, dev, False),
    "moe_block_decode8": lambda dev: case_moe_stream(8, dev, True),
    "attention_prefill": lambda dev: case_attention_prefill(2048, dev),
    "attention_decode8": lambda dev: case_attention_decode(8, 2048, dev),
    "attention_decode64": lambda dev: case_attention_decode(64, 2048, dev),
    "dense_decode8": lambda dev: case_dense_decode(8, dev),
    "dense_decode1": lambda dev: case_dense_decode(1, dev),
    "small_decode8": lambda dev: case_small_decode(8, dev),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--sizes", default="a2.7b", choices=sorted(SIZES))
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--time", action="store_true", help="print the median time per call")
    args = ap.parse_args(argv)
    from . import load, tensor_core_status
    use_sizes(args.sizes)
    load()
    ops = CASES[args.case]("cuda")
    for _, fn in ops:
        for _ in range(2):
            fn()
    torch.cuda.synchronize()
    # L2 is flushed by writing one buffer larger than it and then reading another: the read pushes
    # the written lines out, so that the timed call does not pay for their write-back
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if args.time else None
    clean = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda") if args.time else None
    for name, fn in ops:
        times = []
        for _ in range(args.repeat if not args.time else max(args.repeat, 15)):
            if flush is not None:
                flush.zero_()
                clean.sum()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        if args.time:
            times.sort()
            print(f"{args.case}/{name}: {times[len(times) // 2]:.1f} us")
    status = tensor_core_status()
    if status:
        print(f"a tensor-core kernel gave up on a wait (code {status})")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
