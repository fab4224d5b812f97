"""Two designs side by side at equal layer sizes: whole-model prefill and decode throughput, and
every kernel of one step timed by name against its roofline.

    python bench.py --config vekasun
    python bench.py --config difavik
    python bench.py --config fetezen
    python bench.py --config kopadra

For each named size a Vekasun model (latent attention and state-space mixers alternating, routed
experts scored by a sigmoid and weighted on their input) and a Qwen2-MoE model of the same width,
heads, experts and expert width are built with random weights drawn on the device.  Timed with
CUDA events after warm-up: one prompt of `prompt` tokens in one step, and decode steps of `batch`
requests that each hold `context` tokens (synthetic cache contents).  Then one prompt step and one
decode step are run with an event pair around every call into the kernel library, which gives
each kernel's time inside a real step; the roofline time of a kernel is the larger of its
algorithmic bytes over the copy bandwidth and its FLOPs over the dense bfloat16 peak.
"""

from __future__ import annotations

import contextlib
import json
import time
from typing import Dict, List, Tuple

import torch

from . import lib as klib

# width, heads, experts, top, expert width; latent attention and state-space sizes beside them
SIZES = {
    "w1024": dict(width=1024, heads=8, experts=32, top=4, ff=704, q_rank=768, kv_rank=256, ssm_heads=32, state=64),
    "w2048": dict(width=2048, heads=16, experts=60, top=4, ff=1408, q_rank=1536, kv_rank=512, ssm_heads=64, state=128),
    "w4096": dict(width=4096, heads=32, experts=64, top=6, ff=2048, q_rank=1536, kv_rank=512, ssm_heads=128, state=128),
}
HEAD_DIM, ROT_DIM, SSM_HEAD_DIM, VOCAB, LAYERS = 128, 64, 64, 32000, 4


def vekasun_config(s: dict) -> dict:
    att = {"heads": s["heads"], "dim": HEAD_DIM, "rot_dim": ROT_DIM, "vdim": HEAD_DIM, "kv_rank": s["kv_rank"],
           "q_rank": s["q_rank"], "scale": (HEAD_DIM + ROT_DIM) ** -0.5, "rot": {"base": 10000.0, "dims": ROT_DIM}}
    ssm = {"heads": s["ssm_heads"], "vdim": SSM_HEAD_DIM, "state": s["state"], "groups": 8, "conv": 4, "norm_groups": 8}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    kinds = ["latent_attention", "mamba2", "mamba2", "latent_attention"]
    return {"architecture": "Vekasun", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": [{"type": k, "mixer": att if k == "latent_attention" else ssm, "mlp": mlp} for k in kinds]}


# the Difavik design at the same sizes: a window of 1,024 keys that keeps the first four, retention heads of
# 64 x 128, lightning heads of 128 x 128
WINDOW, KEEP_FIRST, RET_DIM = 1024, 4, 64


def difavik_config(s: dict) -> dict:
    H = s["heads"]
    decay = [1.0 - 2.0 ** (-5.0 - 3.0 * h / max(1, H - 1)) for h in range(H)]
    left = {"heads": H, "kv_heads": H, "dim": HEAD_DIM, "vdim": HEAD_DIM, "scale": HEAD_DIM ** -0.5,
            "mask": {"size": WINDOW, "keep_first": KEEP_FIRST}}
    right = {"heads": H, "dim": RET_DIM, "vdim": HEAD_DIM, "decay": decay, "rot": {"base": 10000.0, "dims": RET_DIM}}
    light = {"heads": H, "dim": HEAD_DIM, "vdim": HEAD_DIM, "decay": decay}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"], "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"]}}
    kinds = ["lightning", "parallel", "parallel", "lightning"]
    return {"architecture": "Difavik", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}},
            "layers": [{"type": k, "mixer": light if k == "lightning" else {"left": left, "right": right}, "mlp": mlp}
                       for k in kinds]}


# the Fetezen design at the same sizes: four residual streams, norms in four groups, as many key heads as query
# heads (as the Qwen2-MoE model beside it), chunks of 1,536 positions (a prompt of 2,048 holds one whole chunk and a
# part of the next; a request at 2,048 decodes a third into its chunk), every second layer reading the keys of the
# layer before it, one dense layer as wide as a token's chosen experts together, one shared expert
STREAMS, NORM_GROUPS, CHUNK = 4, 4, 1536


def fetezen_config(s: dict) -> dict:
    H = s["heads"]
    att = lambda src: dict({"heads": H, "kv_heads": H, "dim": HEAD_DIM, "vdim": HEAD_DIM, "scale": HEAD_DIM ** -0.5,
                            "rot": {"base": 10000.0, "dims": HEAD_DIM}, "mask": {"size": CHUNK}},
                           **({} if src is None else {"kv_from": src}))
    moe = lambda shared: dict({"kind": "moe", "expert": {"ff": s["ff"]}, "router": {"experts": s["experts"], "top": s["top"]}},
                              **({"shared": {"ff": s["ff"]}} if shared else {}))
    mlps = [{"kind": "dense", "ff": s["top"] * s["ff"]}, moe(False), moe(True), moe(False)]
    return {"architecture": "Fetezen", "vocab": VOCAB, "width": s["width"], "streams": STREAMS, "logit_softcap": 30.0,
            "norm": {"eps": 1e-6, "groups": NORM_GROUPS},
            "layers": [{"type": "attention", "mixer": att(src), "mlp": mlp} for src, mlp in zip((None, 0, None, 2), mlps)]}


# the Kopadra design at the same sizes: as many key heads as query heads (as the Qwen2-MoE model beside it), heads of
# 128 with half of them turned by stretched frequencies, the second layer reading the first one's keys, one recurrent
# (mLSTM) layer with heads of 64 x 128, one dense layer as wide as a token's chosen experts together, experts in four
# groups of which two are kept, four of them identity experts, and a shared expert in every routed layer
MLSTM_DIM, IDENTITY, ROUTE_GROUPS = 64, 4, (4, 2)


def kopadra_config(s: dict) -> dict:
    H = s["heads"]
    rot = {"base": 1000000.0, "dims": ROT_DIM, "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}
    att = lambda src: {"type": "attention", "mixer": dict({"heads": H, "kv_heads": H, "dim": HEAD_DIM, "vdim": HEAD_DIM,
                                                           "scale": HEAD_DIM ** -0.5, "rot": rot},
                                                          **({} if src is None else {"kv_from": src}))}
    rec = {"type": "mlstm", "mixer": {"heads": H, "dim": MLSTM_DIM, "vdim": HEAD_DIM, "gate_cap": 10.0}}
    moe = {"kind": "moe", "expert": {"ff": s["ff"]}, "shared": {"ff": s["ff"]},
           "router": {"experts": s["experts"] - IDENTITY, "identity": IDENTITY, "top": s["top"], "scale": 2.5,
                      "groups": {"count": ROUTE_GROUPS[0], "keep": ROUTE_GROUPS[1]}}}
    mlps = [{"kind": "dense", "ff": s["top"] * s["ff"]}, moe, moe, moe]
    return {"architecture": "Kopadra", "vocab": VOCAB, "width": s["width"], "logit_softcap": 25.0, "norm": {"eps": 1e-6},
            "layers": [dict(m, mlp=f) for m, f in zip((att(None), att(0), rec, att(None)), mlps)]}


def qwen2_moe_config(s: dict) -> dict:
    return {"architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "num_hidden_layers": LAYERS,
            "hidden_size": s["width"], "num_attention_heads": s["heads"], "num_key_value_heads": s["heads"],
            "head_dim": HEAD_DIM, "intermediate_size": 4 * s["ff"], "num_experts": s["experts"],
            "num_experts_per_tok": s["top"], "moe_intermediate_size": s["ff"], "shared_expert_intermediate_size": 0,
            "norm_topk_prob": False, "decoder_sparse_step": 1, "mlp_only_layers": [], "vocab_size": VOCAB,
            "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
            "qkv_bias": True}


@contextlib.contextmanager
def timed_calls(record: List[Tuple[str, "torch.cuda.Event", "torch.cuda.Event"]]):
    """Every call into the kernel library gets an event pair on the launching stream."""
    plain = klib.call

    def call(name, *args):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        plain(name, *args)
        e1.record()
        record.append((name, e0, e1))

    klib.call = call
    try:
        yield
    finally:
        klib.call = plain


def _by_kernel(record) -> Dict[str, Tuple[int, float]]:
    torch.cuda.synchronize()
    out: Dict[str, List[float]] = {}
    for name, e0, e1 in record:
        out.setdefault(name, []).append(e0.elapsed_time(e1) * 1e3)
    return {k: (len(v), sum(v)) for k, v in out.items()}


def work_models(s: dict, prompt: int, batch: int, context: int, design: str = "") -> Dict[str, Dict[str, Tuple[float, float]]]:
    """Per phase and kernel: (bytes, FLOPs) of ONE call.  Only kernels whose work is the design's
    own are listed (products over weights are the same kernels in both designs)."""
    W, H, R, Dr = s["width"], s["heads"], s["kv_rank"], ROT_DIM
    Wl = R + Dr
    inner, N, G = s["ssm_heads"] * SSM_HEAD_DIM, s["state"], 8
    C = inner + 2 * G * N
    proj = 2 * inner + 2 * G * N + s["ssm_heads"]
    state = s["ssm_heads"] * SSM_HEAD_DIM * N * 4
    D = HEAD_DIM

    def phase(T, pairs, rows_ctx, nseg, pairs_w=0.0, rows_w=0, pairs_c=0.0, rows_c=0):
        # pairs: sum over rows of the keys each sees; rows_ctx: cache tokens that must be read once;
        # pairs_w, rows_w: the same under the Difavik comparison's window; pairs_c, rows_c: under Fetezen's chunks
        la = lambda Dk, Dv: (T * H * (2 * Dk + Dv) * 2 + T * H * Dv * 4 + 2 * nseg * H * Dk * Dv * 4, 4.0 * T * H * Dk * Dv)
        windowed = (rows_w * 2 * H * D * 2 + 2 * T * H * D * 2, 4.0 * H * D * pairs_w)
        chunked = lambda rows, prs: (rows * H * 2 * D * 2 + 2 * T * H * D * 2, (4.0 * H * D + 2.0 * H * H) * prs)
        own = {}
        if design == "kopadra":
            E, k = s["experts"], s["top"]
            own = {
                # the recurrence has one shape here (64 x 128); q, k, v in, outputs and the three gate numbers a row
                "nf_decay_linear_attention": (la(MLSTM_DIM, D)[0] + T * H * 12, la(MLSTM_DIM, D)[1]),
                # the gates' pass: q and k in, two projections in, three numbers out, (n, m) read and written
                "nf_mlstm_gates": (T * H * (2 * MLSTM_DIM * 2 + 8 + 12) + 2 * nseg * H * (MLSTM_DIM + 1) * 4, 4.0 * T * H * MLSTM_DIM),
                # float32 sums of q, k, v in; q, key and value out (a layer that reads another's keys: a third of it)
                "nf_whole_norm_rope_append": (T * 3 * H * D * (4 + 2), 0.0),
                "nf_sigmoid_gate_rows": (T * H * D * (2 + 4 + 2), 0.0),
                "nf_router_logits": (T * W * 2 + E * W * 4 + T * E * 4, 2.0 * T * W * E),
                "nf_router_select_ruled": (T * (E * 4 + k * 8), 0.0),
                "nf_identity_expert_rows": (T * k * W * 2 * 2 * IDENTITY / E, 0.0),
                "nf_gated_bias_act": (T * k * s["ff"] * 2 * 3, 0.0),
            }
        table = {
            # Fetezen: keys and values of the rows' chunks once, queries in and outputs out; both products and the
            # mixing of the heads' scores
            "nf_talking_attention": chunked(rows_c, pairs_c),
            "nf_talking_attention_mma": chunked(rows_c, pairs_c),
            "nf_talking_attention_split": chunked(rows_c, pairs_c),
            "nf_streams_mix_norm": (T * W * (8 * STREAMS + 2 + 2), 0.0),
            "nf_head_norm_rope_append": (T * 3 * H * D * (4 + 2), 0.0),
            "nf_add_bias_rows": (T * W * (4 + 2), 0.0),
            "nf_poly_norm_act": (T * s["top"] * s["ff"] * (4 + 2), 0.0),
            "nf_embed_copies": (T * W * (2 + 4 * STREAMS), 0.0),
            "nf_prefill_attention_biased": windowed,
            "nf_paged_attention_generic": windowed,
            # two shapes share the kernel (lightning 128 x 128, retention 64 x 128): the mean of the two
            "nf_decay_linear_attention": tuple((a + b) / 2 for a, b in zip(la(D, D), la(RET_DIM, D))),
            "nf_scaled_norm_add": (T * W * (4 + 4 + 3 + 2), 0.0),
            "nf_mean_of_rmsnorms": (T * W * (2 + 2 + 4), 0.0),
            "nf_group_rmsnorm_gate": (T * H * D * (4 + 2 + 2), 0.0),
            "nf_qk_whole_norm_append": (T * 2 * H * D * (4 + 2) + T * H * D * 2, 0.0),
            "nf_pair_hash_embed": (T * W * (2 + 4 + 4), 0.0),
            "nf_latent_attention_generic": (rows_ctx * Wl * 2 + 2 * T * H * R * 2, 2.0 * H * (Wl + R) * pairs),
            "nf_latent_attention_mma": (rows_ctx * Wl * 2 + 2 * T * H * R * 2, 2.0 * H * (Wl + R) * pairs),
            "nf_prefill_attention_tc": (rows_ctx * 2 * H * D * 2 + 2 * T * H * D * 2, 4.0 * H * D * pairs),
            "nf_prefill_attention": (rows_ctx * 2 * H * D * 2 + 2 * T * H * D * 2, 4.0 * H * D * pairs),
            "nf_decode_attention": (rows_ctx * 2 * H * D * 2 + 2 * T * H * D * 2, 4.0 * H * D * pairs),
            "nf_ssd_scan": (T * (C * 2 + 2 + inner * 4) + 2 * nseg * state, 6.0 * T * inner * N),
            "nf_causal_conv_silu": (T * C * 4, 8.0 * T * C),
            "nf_gated_group_rmsnorm": (T * inner * (4 + 2 + 2), 0.0),
            "nf_add_layernorm": (T * W * (4 + 4 + 2 + 2), 0.0),
            "nf_add_rmsnorm": (T * W * (4 + 4 + 2 + 2), 0.0),
            "nf_moe_combine_add_rmsnorm": (T * W * (4 + 4 + 2 + 2 * s["top"]), 0.0),
            "nf_moe_combine": (T * W * 2 * (1 + s["top"]), 0.0),
            "nf_latent_append": (T * Wl * 4, 0.0),
            "nf_rope_append": (T * 3 * H * D * 2 * 2, 0.0),
            "nf_rope_head_slices": (T * H * Dr * 4, 0.0),
            "nf_rms_norm_slice": (T * s["q_rank"] * 4, 0.0),
            "nf_heads_sigmoid_gate": (T * H * D * 6, 0.0),
            "nf_scale_gather_rows": (T * s["top"] * W * 4, 0.0),
            "nf_gather_rows": (T * s["top"] * W * 4, 0.0),
        }
        table.update(own)
        return table

    seen = lambda p: min(p + 1, WINDOW) + max(0, min(KEEP_FIRST, p + 1 - WINDOW))       # keys position p sees
    in_chunk = lambda p: p % CHUNK + 1                                                  # keys position p sees in its chunk
    return {"prefill": phase(prompt, prompt * (prompt + 1) / 2, prompt, 1, float(sum(seen(p) for p in range(prompt))), prompt,
                             float(sum(in_chunk(p) for p in range(prompt))), prompt),
            "decode": phase(batch, batch * (context + 1), batch * (context + 1), batch, float(batch * seen(context)),
                            batch * seen(context), float(batch * in_chunk(context)), batch * in_chunk(context))}


def measure(config: dict, prompt: int, batch: int, context: int, steps: int, warmup: int) -> dict:
    from ..config import EngineOptions
    from ..engine import Engine, StepEntry
    opts = EngineOptions(dtype="bfloat16", max_context=context + 512, prefill_chunk=prompt, num_sequences=batch,
                         page_size=64, cache_tokens=batch * (context + 512), max_batched_tokens=prompt)
    engine = Engine(config=config, random_seed=3, options=opts)
    runner, cache, model = engine.runner, engine.cache, engine.runner.model
    g = torch.Generator().manual_seed(0)
    V = model.vocab_size
    for grp in cache.groups:
        grp.pages.normal_(0, 1)
    ptoks = torch.randint(0, V, (prompt,), generator=g).tolist()

    def prefill_once(record=None):
        cache.open("p")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if record is None:
            runner.step([StepEntry("p", ptoks, [prompt - 1])])
        else:
            with timed_calls(record):
                runner.step([StepEntry("p", ptoks, [prompt - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.close("p")
        return e0.elapsed_time(e1)

    for _ in range(max(3, warmup // 2)):
        prefill_once()
    pms = min(prefill_once() for _ in range(3))
    rec: list = []
    prefill_once(rec)
    prefill_kernels = _by_kernel(rec)

    ids = []
    for i in range(batch):
        rid = ("d", i)
        cache.open(rid)
        cache.reserve(rid, context)
        cache.commit(rid, context)
        ids.append(rid)
    toks = torch.randint(0, V, (warmup + steps + 1, batch), generator=g).tolist()
    for s_ in range(warmup):
        runner.step([StepEntry(r, [toks[s_][i]], [0]) for i, r in enumerate(ids)])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s_ in range(warmup, warmup + steps):
        runner.step([StepEntry(r, [toks[s_][i]], [0]) for i, r in enumerate(ids)])
    e1.record()
    torch.cuda.synchronize()
    dms = e0.elapsed_time(e1) / steps
    # one decode step driven from the host, kernel by kernel
    graphs, runner.graphs = runner.graphs, None
    rec = []
    runner.step([StepEntry(r, [toks[-1][i]], [0]) for i, r in enumerate(ids)])
    with timed_calls(rec):
        runner.step([StepEntry(r, [toks[-1][i]], [0]) for i, r in enumerate(ids)])
    decode_kernels = _by_kernel(rec)
    runner.graphs = graphs
    for r in ids:
        cache.close(r)
    from .ops import check_status
    check_status("comparison")
    out = {"weights_gb": round(model.weight_bytes() / 1e9, 2), "graphs": runner.graphs is not None,
           "prefill": {"tokens": prompt, "ms": round(pms, 3), "tokens_per_s": round(prompt / pms * 1e3, 1)},
           "decode": {"batch": batch, "context": context, "ms_per_step": round(dms, 4),
                      "tokens_per_s": round(batch / dms * 1e3, 1)},
           "kernels": {"prefill": prefill_kernels, "decode": decode_kernels}}
    del engine, runner, cache, model
    torch.cuda.empty_cache()
    return out


DESIGNS = {"vekasun": vekasun_config, "difavik": difavik_config, "fetezen": fetezen_config, "kopadra": kopadra_config}


def run_comparison(sizes, peaks: dict, prompt: int = 2048, batch: int = 8, context: int = 2048, steps: int = 32,
                   warmup: int = 8, design: str = "vekasun") -> dict:
    klib.load()
    result = {}
    for name in sizes:
        s = SIZES[name]
        models = work_models(s, prompt, batch, context, design)
        entry = {}
        for which, cfg in ((design, DESIGNS[design](s)), ("qwen2_moe", qwen2_moe_config(s))):
            t0 = time.time()
            m = measure(cfg, prompt, batch, context, steps, warmup)
            for ph in ("prefill", "decode"):
                table = {}
                for k, (calls, us) in sorted(m["kernels"][ph].items(), key=lambda kv: -kv[1][1]):
                    row = {"calls": calls, "us": round(us, 1)}
                    if k in models[ph]:
                        b, f = models[ph][k]
                        floor_us = max(b / (peaks["hbm_gbs"] * 1e9), f / (peaks["bf16_tflops"] * 1e12)) * 1e6
                        row["roofline_frac"] = round(floor_us * calls / us, 4) if us > 0 else None
                        row["bound"] = "hbm" if b / (peaks["hbm_gbs"] * 1e9) >= f / (peaks["bf16_tflops"] * 1e12) else "bf16"
                    table[k] = row
                m["kernels"][ph] = table
            m["seconds"] = round(time.time() - t0)
            entry[which] = m
        result[name] = entry
    return result


if __name__ == "__main__":
    print(json.dumps(run_comparison(["w1024"], {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, steps=8, warmup=4)))
