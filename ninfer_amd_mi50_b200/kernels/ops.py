"""Python faces of the CUDA kernels.  Every function launches on torch's current stream.

One function per operation of the step (reference: the free functions of
src/ops/ops.h:19-234).  Which kernel serves a call is decided by the dtype and by the
number of rows only, never by what the rows are (prompt or decode), so that a row's
result does not depend on its neighbours.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import lib as _lib

c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_DT = {torch.float32: 0, torch.bfloat16: 1}

# Library products of the bfloat16 path must add up in float32: no split-k partial sums
# rounded to bfloat16, and never TF32 for float32 operands.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False

# Tunables that tests may override to force a particular kernel.
TUNING = {
    "bf16_linear": "auto",        # "simt" | "auto"
    "bf16_attention": "auto",     # "generic" | "auto"
    "bf16_moe": "auto",           # "simt" | "auto"
    "skinny_max_rows": 16,        # dense products with more rows go to the library
    # routed experts: up to this many tokens the streaming kernel serves, beyond it the
    # tensor-core kernel (measured decode steps: 4 % slower at 16 tokens, 7 % faster at 32,
    # 10 % faster at 64)
    "skinny_moe_max_tokens": 16,
    # prompt portions: steps with at least this many rows use the tcgen05 attention kernel (head
    # size 64 or 128), fewer the mma.sync one; a huge number turns the tensor-core kernel off
    "prefill_attention_tc_min_rows": 128,
    "qkv_rope_fused": True,       # few bfloat16 rows: rotation and cache append in the projection's epilogue
    "router_tensor_min_rows": 128,   # router logits of more rows than this use tensor cores
    # up to this many rows, routing is a single launch (whole decode steps at 24 and 32 tokens:
    # 0.5 % faster than logits, selection and plan apart; at 64 tokens 1 % slower)
    "router_fused_max_rows": 32,
    # ... by one cluster of 8 CTAs up to this many rows (measured: 6.6 against 10.5 us at 1 row,
    # 10.1 against 11.5 at 8, 17.2 against 15.5 at 16); 0 turns the cluster kernel off
    "router_cluster_max_rows": 8,
    # decode attention can merge its key blocks in the same launch (the last CTA of a row does
    # it); measured slower than the separate merge kernel at every batch size, so it is off
    "decode_merge_fused_max_rows": 0,
    # the routed experts' weighted sum joins the residual add and the next norm in one kernel, up
    # to this many rows (same bits either way; measured on B200: no difference to a decode step,
    # which only loses a launch, and a prompt of 2,048 tokens 2 % slower fused, because the
    # separate combine reads 16 bytes a lane and spreads a row over more CTAs); 0 turns it off
    "fuse_combine_norm_max_rows": 64,
    # a shared expert runs beside the routed path, on a second stream, in steps of up to
    # `shared_fork_max_rows` rows (larger steps fill the device with either alone); it is started
    # beside the router up to `shared_fork_late_rows` rows and after it beyond.  (With the
    # experts as two launches, starting after the router was 3 % faster at 48 and 64 rows; with
    # their persistent launch, starting beside the router is 2 % faster at 40 to 64 rows too, so
    # the second threshold now equals the first.)
    "shared_fork_max_rows": 64,
    "shared_fork_late_rows": 64,
    # in steps of at least this many rows (and more than `shared_fork_max_rows`) the routing
    # (logits, selection, plan, gather: short kernels of a few CTAs, one waiting for the other)
    # runs on a second stream of higher priority while the shared expert's products fill the
    # device; 0 turns it off.  (A prompt of 2,048 tokens: 3 % faster; decode steps of 72 to 128
    # tokens: 1.3 %.)
    "route_beside_shared_min_rows": 65,
    # steps of `moe_stream_min_tokens` to `moe_stream_max_tokens` tokens run both products of the
    # routed experts in one persistent launch (packed bfloat16 weights); a max of 0: always two
    # launches.  Measured at A2.7B sizes, whole decode steps against the two launches (the
    # streaming product up to 16 tokens, the tensor-core grouped product beyond): the same at 4
    # tokens, 3 % faster at 6, 6 % at 8, 16 % at 16, 10 % at 32, 3.5 % at 64, 2 % slower at 96 and
    # 128 (experts with more than eight rows are served eight at a time and stream their weights
    # again).  `moe_stream_smem_kb`: shared memory that launch takes on every SM - what is left
    # stays free for the shared expert's kernels, which run beside it on a second stream (160
    # instead of 192: the same up to 16 tokens, 2 % slower at 32 and 64)
    "moe_stream_min_tokens": 6,
    "moe_stream_max_tokens": 64,
    # ... and up to this many tokens that launch routes as well (logits, selection and plan by
    # its own CTAs before the products); 0: the router's kernels run before it
    "moe_stream_route_max_tokens": 64,
    # ... and up to `moe_stream_shared_max_tokens` tokens it serves a shared expert as well (a
    # second, packed copy of its matrices is then kept: `pack_shared_expert`; 0: no such copy, the
    # shared expert always runs beside the launch on a second stream).  Measured at A2.7B sizes,
    # whole decode steps against the router's kernels + the launch + the second stream: 3 % faster
    # at 6 tokens, 2 % at 8, the same at 16, 3 % slower at 32, 6 % at 64 (the routing inside the
    # launch takes 15 us, and only the CTAs that hold an item of the shared expert have work
    # until it is done); with fewer than 6 tokens the separate kernels win as well
    "moe_stream_shared": 1,
    "moe_stream_shared_max_tokens": 16,
    "moe_stream_smem_kb": 192,
}

SUPPORTED_HEAD_DIMS = tuple(range(16, 257, 16))
DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)   # head sizes of the split-key decode kernel
DECODE_SPLIT = 128                          # keys per block of that kernel
PREFILL_HEAD_DIMS = tuple(range(16, 129, 16))   # head sizes of the flash prefill kernel
PREFILL_TILE_ROWS = 64                      # query rows per tile of that kernel
PREFILL_KEY_BLOCK = 64                      # keys per block of that kernel
MAX_EXPERTS = 3072


def check_head_dim(head_dim: int) -> None:
    if head_dim not in SUPPORTED_HEAD_DIMS:
        raise ValueError(f"head_dim={head_dim} is not supported by the attention kernels "
                         f"(multiples of 16 from 16 to 256)")


DECODE_MAX_SPLITS = 1024                    # key blocks one row's merge takes


def check_attention_limits(dtype: torch.dtype, head_dim: int, max_context: int, page_size: int) -> None:
    """What the attention kernels cannot serve, said at start-up: the bfloat16 decode kernels
    merge at most `DECODE_MAX_SPLITS` blocks of `DECODE_SPLIT` keys per row."""
    check_head_dim(head_dim)
    if dtype == torch.bfloat16 and head_dim in DECODE_HEAD_DIMS:
        most = DECODE_MAX_SPLITS * DECODE_SPLIT
        if max_context > most:
            raise ValueError(f"max_context={max_context} is beyond the {most} keys a request may hold "
                             f"in bfloat16 mode (decode attention merges at most {DECODE_MAX_SPLITS} "
                             f"blocks of {DECODE_SPLIT} keys)")


def check_router_sizes(num_experts: int, top_k: int) -> None:
    if not 1 <= num_experts <= MAX_EXPERTS:
        raise ValueError(f"num_experts={num_experts} is not supported (1..{MAX_EXPERTS})")
    if not 1 <= top_k <= num_experts:
        raise ValueError(f"top_k={top_k} must lie in [1, {num_experts}]")


# The gated activation of a feed-forward's first product: (kind, limit, alpha).  Kind 1 is
# silu(gate) * up; kind 2 the capped form min(g, limit) * sigmoid(alpha * min(g, limit)) *
# (clamp(up, -limit, limit) + 1).
ACT_SILU = (1, 0.0, 0.0)


def capped_activation(limit: float, alpha: float) -> Tuple[int, float, float]:
    if not limit > 0:
        raise ValueError(f"capped activation: limit={limit} must be positive")
    return (2, float(limit), float(alpha))


ACT_GELU_TANH = (4, 0.0, 0.0)     # gelu_tanh(gate) * up, gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))


def _act(swiglu, act) -> Tuple[int, float, float]:
    """The epilogue a product is launched with: none, or the gated activation `act`."""
    if not swiglu:
        return (0, 0.0, 0.0)
    return ACT_SILU if act is None else act


def _p(t: Optional[torch.Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _chk(t: torch.Tensor, name: str, dtype=None, contiguous=True) -> None:
    if not t.is_cuda:
        raise _lib.KernelError(f"{name} must be a CUDA tensor; there is no CPU implementation")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")


# ---------------------------------------------------------------------------------------
# rows
# ---------------------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = float32(table[ids[t]])."""
    _chk(table, "table"); _chk(ids, "ids", torch.int32); _chk(out, "out", torch.float32)
    _lib.call("nf_embed_rows", _p(table), _p(ids), _p(out), c_int(ids.numel()),
              c_int(table.shape[1]), c_int(table.shape[0]), c_int(_dt(table)), _stream())


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """h += delta (float32, in place); out = h * rsqrt(mean(h^2) + eps) * weight."""
    _chk(h, "h", torch.float32); _chk(weight, "weight", torch.float32); _chk(out, "out")
    if delta is not None:
        _chk(delta, "delta", out.dtype)
    _lib.call("nf_add_rmsnorm", _p(h), _p(delta), None, _p(weight), c_float(eps), _p(out),
              c_int(h.shape[0]), c_int(h.shape[1]), c_int(_dt(out)), _stream())


def add_rmsnorm_rows(h: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                     weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[r] = norm(h[rows[r]] + delta[rows[r]]); h is left as it is."""
    _chk(h, "h", torch.float32); _chk(rows, "rows", torch.int32); _chk(out, "out")
    _chk(weight, "weight", torch.float32)
    if delta is not None:
        _chk(delta, "delta", out.dtype)
    _lib.call("nf_add_rmsnorm", _p(h), _p(delta), _p(rows), _p(weight), c_float(eps), _p(out),
              c_int(rows.numel()), c_int(h.shape[1]), c_int(_dt(out)), _stream())


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[M, 2I] -> [M, I]: silu(first half) * second half."""
    _chk(gate_up, "gate_up")
    M, two_i = gate_up.shape
    out = torch.empty((M, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _lib.call("nf_silu_mul", _p(gate_up), _p(out), c_int(M), c_int(two_i // 2), c_int(_dt(gate_up)),
              _stream())
    return out


# ---------------------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------------------

def _gemm_simt(a, lda, b, b_group_stride, c, M, N, K, groups, max_rows, offsets, a_rows, a_div,
               swiglu, act=None) -> None:
    kind, limit, alpha = _act(swiglu, act)
    _lib.call("nf_gemm_simt", _p(a), c_int(lda), _p(b), c_longlong(b_group_stride), _p(c),
              c_int(c.shape[1]), c_int(M), c_int(N), c_int(K), c_int(groups), c_int(max_rows),
              _p(offsets), _p(a_rows), c_int(a_div), c_int(kind), c_int(_dt(a)),
              c_int(_dt(c)), c_float(limit), c_float(alpha), _stream())


def _skinny(x, ldx, w, w_group_stride, out, M, N, K, groups, max_rows, offsets, x_rows, x_div, swiglu,
            packed=False, group_map=None, early_index=False, act=None) -> None:
    kind, limit, alpha = _act(swiglu, act)
    _lib.call("nf_skinny_gemm", _p(x), c_int(ldx), _p(w), c_longlong(w_group_stride), _p(out),
              c_int(out.shape[1]), c_int(M), c_int(N), c_int(K), c_int(groups), c_int(max_rows),
              _p(offsets), _p(x_rows), c_int(x_div), c_int(kind), c_int(_dt(out)),
              c_int(1 if packed else 0), _p(group_map),
              c_int(group_map.numel() if group_map is not None else 0), c_int(1 if early_index else 0),
              c_float(limit), c_float(alpha), _stream())


class PackedWeights:
    """Grouped bfloat16 weights [G, rows, K] in the tile layout the streaming kernels read.

    Tiles of 128 rows x 64 k (SwiGLU: 128 gate rows followed by the 128 matching up rows),
    stored contiguously as [group][feature tile][k tile][tile rows][64], each tile in the
    128-byte-swizzled image (the 16-byte piece j of tile row r is stored at piece j ^ (r & 7)),
    zero-padded to whole tiles.  A CTA that owns 128 features reads one contiguous slab."""

    def __init__(self, data: torch.Tensor, groups: int, n_features: int, K: int, swiglu: bool):
        self.data, self.groups, self.n_features, self.K, self.swiglu = data, groups, n_features, K, swiglu
        self.dtype, self.device = data.dtype, data.device

    @property
    def group_stride(self) -> int:
        return self.data[0].numel()

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    def group_nbytes(self) -> int:
        return self.group_stride * self.data.element_size()


def can_pack(n_features: int, K: int) -> bool:
    return K % 8 == 0


def pack_weights(w: torch.Tensor, swiglu: bool, chunk: int = 4) -> PackedWeights:
    """[G, rows, K] bfloat16 (rows = 2 * features with gate rows first when `swiglu`) -> packed."""
    _chk(w, "w", torch.bfloat16)
    G, R, K = w.shape
    N = R // 2 if swiglu else R
    NT, KT = (N + 127) // 128, (K + 63) // 64
    rows = 256 if swiglu else 128
    out = torch.empty((G, NT, KT, rows, 64), dtype=w.dtype, device=w.device)
    r = torch.arange(rows, device=w.device)
    src_piece = (torch.arange(8, device=w.device)[None, :] ^ (r[:, None] & 7))       # [rows, 8]
    for g0 in range(0, G, chunk):
        blk = w[g0:g0 + chunk]
        n = blk.shape[0]
        halves = [blk[:, :N], blk[:, N:]] if swiglu else [blk]
        tiles = []
        for h in halves:
            p = torch.zeros((n, NT * 128, KT * 64), dtype=w.dtype, device=w.device)
            p[:, :N, :K] = h
            tiles.append(p.view(n, NT, 128, KT, 64).permute(0, 1, 3, 2, 4))             # [n, NT, KT, 128, 64]
        t = torch.cat(tiles, dim=3) if swiglu else tiles[0]                            # [n, NT, KT, rows, 64]
        t = t.reshape(n, NT, KT, rows, 8, 8)
        idx = src_piece.view(1, 1, 1, rows, 8, 1).expand(n, NT, KT, rows, 8, 8)
        out[g0:g0 + n] = torch.gather(t, 4, idx).reshape(n, NT, KT, rows, 64)
    return PackedWeights(out, G, N, K, swiglu)


def _bf16_path(rows: int, K: int, key: str) -> str:
    """Which bfloat16 product serves `rows` rows: decided by the row count and K only."""
    if TUNING[key] == "simt":
        return "simt"
    limit = TUNING["skinny_max_rows"] if key == "bf16_linear" else TUNING["skinny_moe_max_tokens"]
    if rows <= limit and K % 8 == 0:
        return "skinny"
    if key == "bf16_moe":
        return "simt"          # unpacked expert weights and many tokens: the CUDA-core product
    return "large"


def chain_break() -> None:
    """The next kernel launched (by this thread) waits for everything before it in its stream
    in the ordinary way.  To be called after making a stream wait for another stream's event:
    the kernel that follows must not be chained to the kernel before it in its own stream."""
    _lib.load().nf_chain_break()


def tensor_core_status() -> int:
    """0, or the code of the first bounded wait that a kernel with a shared-memory ring gave up on
    since the last call (synchronises the device): 1-4 from the grouped GEMM, 101-110 from
    attention, 401-413 from the persistent experts' kernel (405-407: a plan that does not fit it)."""
    lib = _lib.load()
    gemm, attn = int(lib.nf_grouped_gemm_tc_status()), int(lib.nf_prefill_attention_tc_status())
    ms = int(lib.nf_moe_stream_status())
    return gemm if gemm else (100 + attn if attn else (400 + ms if ms else 0))


def index_status() -> int:
    """0, or what a kernel that follows device-side indices found outside its operands since the
    last call (it skips such an access): 201-203 the streaming product (group, row range, row
    index), 300 + token + 1 the combine, 100000 + row + 1 a decode-attention row whose position
    lay beyond the key blocks its call allowed for.  Synchronises the device."""
    lib = _lib.load()
    sk, cb = int(lib.nf_skinny_index_status()), int(lib.nf_combine_index_status())
    da = int(lib.nf_decode_attention_status())
    return 200 + sk if sk else (300 + cb if cb else (100000 + da if da else 0))


def check_status(where: str = "") -> None:
    """Raise `KernelError` if a kernel gave up on a bounded wait or skipped an access outside
    its operands since the last check: its output is then not to be used.  Synchronises the
    device, so it is called where the host waits anyway (after a step's logits or tokens have
    been read) and every so many decode steps."""
    tc = tensor_core_status()
    ix = index_status()
    if tc or ix:
        what = []
        if tc:
            what.append(f"a tensor-core kernel gave up on a wait (code {tc})")
        if ix:
            what.append(f"a kernel met an index outside its operands (code {ix})")
        raise _lib.KernelError((where + ": " if where else "") + "; ".join(what)
                               + "; the results of the steps since the last check are invalid")


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M, K] times w [N, K] transposed -> [M, N]; float32 accumulation."""
    _chk(x, "x"); _chk(w, "w", x.dtype)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"linear: x has {K} columns, w has {w.shape[1]}")
    out_dtype = out_dtype or x.dtype
    if M == 0:
        return torch.empty((M, N), dtype=out_dtype, device=x.device)
    path = "simt" if x.dtype == torch.float32 else _bf16_path(M, K, "bf16_linear")
    if path == "large":
        # a plain library product, as the reference uses rocBLAS for M > 1 (src/ops/linear.hip)
        if out_dtype == torch.bfloat16:
            return torch.mm(x, w.t())
        try:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            path = "simt"
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if path == "skinny":
        _skinny(x, K, w, 0, out, M, N, K, 1, M, None, None, 1, False)
    else:
        _gemm_simt(x, K, w, 0, out, M, N, K, 1, M, None, None, 1, False)
    return out


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, act=None) -> torch.Tensor:
    """x [M, K], w [2I, K] (gate rows first) -> silu(x gate^T) * (x up^T)  [M, I]; `act`: another gated
    activation in silu's place (the product kernels' epilogues take it; after a library product it is a
    pass of its own)."""
    _chk(x, "x"); _chk(w_gate_up, "w_gate_up", x.dtype)
    M, K = x.shape
    inner = w_gate_up.shape[0] // 2
    if M == 0:
        return torch.empty((M, inner), dtype=x.dtype, device=x.device)
    path = "simt" if x.dtype == torch.float32 else _bf16_path(M, K, "bf16_linear")
    if path == "large":
        gu = torch.mm(x, w_gate_up.t())
        return silu_mul(gu) if act is None else gated_bias_act(gu, None, act, x.dtype)
    out = torch.empty((M, inner), dtype=x.dtype, device=x.device)
    if path == "skinny":
        _skinny(x, K, w_gate_up, 0, out, M, inner, K, 1, M, None, None, 1, True, act=act)
    else:
        _gemm_simt(x, K, w_gate_up, 0, out, M, inner, K, 1, M, None, None, 1, True, act=act)
    return out


# ---------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------

def rope_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                row_seg: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                Hq: int, Hkv: int, D: int, pages: torch.Tensor, block_table: torch.Tensor,
                page_size: int, append: bool) -> None:
    """In place: qkv += bias; rotate q and k heads; write k, v to the cache pages."""
    _chk(qkv, "qkv"); _chk(pages, "pages", qkv.dtype); _chk(block_table, "block_table", torch.int32)
    _chk(positions, "positions", torch.int32); _chk(row_seg, "row_seg", torch.int32)
    if bias is not None:
        _chk(bias, "bias", torch.float32)
    if inv_freq is not None:
        _chk(inv_freq, "inv_freq", torch.float32)
    if qkv.shape[1] != (Hq + 2 * Hkv) * D:
        raise ValueError("rope_append: qkv width does not match the head counts")
    _lib.call("nf_rope_append", _p(qkv), _p(bias), _p(positions), _p(row_seg), _p(inv_freq),
              c_int(rotary_dim if inv_freq is not None else 0), c_int(qkv.shape[0]), c_int(Hq),
              c_int(Hkv), c_int(D), _p(pages), _p(block_table), c_int(block_table.shape[1]),
              c_int(page_size), c_int(pages.shape[0]), c_int(1 if append else 0), c_int(_dt(qkv)),
              _stream())


def linear_rope_append(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                       positions: torch.Tensor, row_seg: torch.Tensor, inv_freq: torch.Tensor,
                       rotary_dim: int, Hq: int, Hkv: int, D: int, pages: torch.Tensor,
                       block_table: torch.Tensor, page_size: int, append: bool) -> torch.Tensor:
    """qkv = x w_qkv^T, then `rope_append` on it -> [T, (Hq + 2 Hkv) D] whose query columns hold
    the rotated queries (the key and value columns are not meant to be read: they went to the
    cache).  A bfloat16 step of few rows does both in one kernel: the streaming product's
    epilogue adds the bias, rotates and writes keys and values into their cache page."""
    T, K = x.shape
    if (TUNING["qkv_rope_fused"] and x.is_cuda and x.dtype == torch.bfloat16 and 0 < T <= min(16, TUNING["skinny_max_rows"])
            and TUNING["bf16_linear"] == "auto" and K % 8 == 0 and D % 16 == 0 and rotary_dim == D
            and inv_freq is not None):
        _chk(x, "x"); _chk(w_qkv, "w_qkv", x.dtype); _chk(pages, "pages", x.dtype)
        _chk(block_table, "block_table", torch.int32); _chk(positions, "positions", torch.int32)
        _chk(row_seg, "row_seg", torch.int32); _chk(inv_freq, "inv_freq", torch.float32)
        if bias is not None:
            _chk(bias, "bias", torch.float32)
        N = (Hq + 2 * Hkv) * D
        if w_qkv.shape != (N, K):
            raise ValueError("linear_rope_append: the projection does not match the head counts")
        qkv = torch.empty((T, N), dtype=x.dtype, device=x.device)
        _lib.call("nf_skinny_qkv_rope", _p(x), c_int(K), _p(w_qkv), _p(qkv), c_int(N), c_int(T), c_int(K),
                  _p(bias), _p(positions), _p(row_seg), _p(inv_freq), c_int(Hq), c_int(Hkv), c_int(D),
                  _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(page_size),
                  c_int(pages.shape[0]), c_int(1 if append else 0), _stream())
        return qkv
    qkv = linear(x, w_qkv)
    rope_append(qkv, bias, positions, row_seg, inv_freq, rotary_dim, Hq, Hkv, D, pages, block_table,
                page_size, append)
    return qkv


_COUNTERS = {}


def _zeroed_counters(device, n: int) -> torch.Tensor:
    """Ints that kernels find zero and leave zero (completion counters of one-launch
    reductions).  Kept for the life of the process, so that captured graphs may refer to them."""
    key = str(device)
    bufs = _COUNTERS.setdefault(key, [])
    if not bufs or bufs[-1].numel() < n:
        # earlier, smaller buffers stay alive: a captured graph may still point at them
        bufs.append(torch.zeros((max(n, 4096),), dtype=torch.int32, device=device))
    return bufs[-1]


def _tiles(ctx, rows_per_tile, window, keys_per_block, pair, min_rows):
    if min_rows > 1:
        return ctx.paired_query_tiles(rows_per_tile, window, keys_per_block, pair=pair, min_rows=min_rows)
    return ctx.paired_query_tiles(rows_per_tile, window, keys_per_block, pair=pair)


def _decode_attention(qkv, Hq, Hkv, D, pages, block_table, page_size, ctx, window, scale, out,
                      rows: Optional[torch.Tensor], n: int) -> None:
    """The split-key decode kernels on all rows of the step (`rows` None) or on the `n` rows
    listed in `rows` (int32 on the device); writes those rows of `out`."""
    nsplit = max(1, (int(ctx.max_context) + DECODE_SPLIT - 1) // DECODE_SPLIT)
    ws_acc = torch.empty((n, Hq, nsplit, D), dtype=torch.float32, device=qkv.device)
    ws_ml = torch.empty((n, Hq, nsplit, 2), dtype=torch.float32, device=qkv.device)
    if rows is not None:
        _lib.call("nf_decode_attention_rows", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(out),
                  _p(ws_acc), _p(ws_ml), _p(rows), c_int(n), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                  c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(nsplit), _stream())
    elif n > TUNING["decode_merge_fused_max_rows"]:
        _lib.call("nf_decode_attention", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(out),
                  _p(ws_acc), _p(ws_ml), c_int(n), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                  c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(nsplit), _stream())
    else:
        counters = _zeroed_counters(qkv.device, n * Hkv)
        _lib.call("nf_decode_attention_fused", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(out),
                  _p(ws_acc), _p(ws_ml), _p(counters), c_int(n), c_int(Hq), c_int(Hkv), c_int(D),
                  c_int(page_size), c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(nsplit),
                  _stream())


def paged_attention(qkv: torch.Tensor, Hq: int, Hkv: int, D: int, pages: torch.Tensor,
                    block_table: torch.Tensor, page_size: int, ctx, window: int, scale: float
                    ) -> torch.Tensor:
    """Causal attention of the rows' (rotated) queries in `qkv` over the cache -> [T, Hq*D].

    In bfloat16 a row is served according to its own segment: a segment of one row (a decoded
    token) by the split-key decode kernel, a segment of several rows (a prompt portion) by a
    flash kernel - whatever else the step holds.  A mixed step is therefore two launches."""
    _chk(qkv, "qkv"); _chk(pages, "pages", qkv.dtype)
    T = qkv.shape[0]
    out = torch.empty((T, Hq * D), dtype=qkv.dtype, device=qkv.device)
    if T == 0:
        return out
    fast = qkv.dtype == torch.bfloat16 and TUNING["bf16_attention"] != "generic"
    if fast and getattr(ctx, "all_single", False) and D in DECODE_HEAD_DIMS:
        _decode_attention(qkv, Hq, Hkv, D, pages, block_table, page_size, ctx, window, scale, out, None, T)
        return out
    if (fast and D in PREFILL_HEAD_DIMS and getattr(ctx, "seg_len_host", None) is not None
            and getattr(ctx, "seg_pos0_host", None) is not None and qkv.shape[1] % 8 == 0):
        min_rows = 1
        if D in DECODE_HEAD_DIMS and hasattr(ctx, "single_rows"):
            rows, n_single = ctx.single_rows()
            if n_single:
                _decode_attention(qkv, Hq, Hkv, D, pages, block_table, page_size, ctx, window, scale, out,
                                  rows, n_single)
                min_rows = 2
        if (T >= TUNING["prefill_attention_tc_min_rows"] and qkv.is_contiguous() and pages.is_contiguous()
                and _lib.load().nf_prefill_attention_tc_fits(c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                                                            c_longlong(pages.shape[0]))):
            # tcgen05 / TMEM / TMA: tiles of 128 rows, blocks of 128 keys
            tiles, n_tiles = _tiles(ctx, 128, window, 128, False, min_rows)
            _lib.call("nf_prefill_attention_tc", _p(qkv), c_longlong(T), c_int(qkv.shape[1]), _p(pages),
                      _p(block_table), c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.seg_row0),
                      _p(tiles), c_int(n_tiles), _p(out), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                      c_int(pages.shape[0]), c_int(window), c_float(scale), _stream())
            return out
        tiles, n_tiles = _tiles(ctx, PREFILL_TILE_ROWS, window, PREFILL_KEY_BLOCK, True, min_rows)
        _lib.call("nf_prefill_attention", _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(block_table),
                  c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.seg_row0), _p(tiles),
                  c_int(n_tiles), _p(out), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
                  c_int(pages.shape[0]), c_int(window), c_float(scale), _stream())
        return out
    _lib.call("nf_paged_attention_generic", _p(qkv), c_int(qkv.shape[1]), _p(pages),
              _p(block_table), c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg),
              _p(out), c_int(T), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size),
              c_int(pages.shape[0]), c_int(window), c_float(scale), c_int(_dt(qkv)), None, c_int(0), None,
              c_int(0), _stream())
    return out


def qk_whole_norm_append(proj: torch.Tensor, q_col0: int, k_col0: int, bias_q: Optional[torch.Tensor],
                         bias_k: Optional[torch.Tensor], wq: torch.Tensor, wk: torch.Tensor, eps: float,
                         Hq: int, Hkv: int, D: int, ctx, pages: torch.Tensor, block_table: torch.Tensor,
                         page_size: int, append: bool) -> torch.Tensor:
    """For an attention whose values are its keys.  proj float32 [T, ld] holds q (Hq x D) at q_col0
    and k (Hkv x D) at k_col0.  Adds the biases; q and k each over the root mean square of their
    whole row slice, times wq / wk; returns q [T, Hq * D] in the cache's type, and writes the normed
    keys as keys and the biased, un-normed keys as values at (request, position)."""
    _chk(proj, "proj", torch.float32); _chk(wq, "wq", torch.float32); _chk(wk, "wk", torch.float32)
    _chk(block_table, "block_table", torch.int32); _chk(pages, "pages")
    for b, n in ((bias_q, "bias_q"), (bias_k, "bias_k")):
        if b is not None:
            _chk(b, n, torch.float32)
    T = proj.shape[0]
    q = torch.empty((T, Hq * D), dtype=pages.dtype, device=proj.device)
    _lib.call("nf_qk_whole_norm_append", _p(proj), c_int(proj.shape[1]), c_int(q_col0), c_int(k_col0), _p(bias_q),
              _p(bias_k), _p(wq), _p(wk), c_float(eps), _p(ctx.positions), _p(ctx.row_seg), _p(q), c_int(T), c_int(Hq),
              c_int(Hkv), c_int(D), _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(page_size),
              c_int(pages.shape[0]), c_int(1 if append else 0), c_int(_dt(pages)), _stream())
    return q


def whole_norm_rope_append(proj: torch.Tensor, q_col0: int, k_col0: int, v_col0: int, bias_q: Optional[torch.Tensor],
                           bias_k: Optional[torch.Tensor], bias_v: Optional[torch.Tensor], wq: torch.Tensor,
                           wk: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot: int,
                           magnitude: float, Hq: int, Hkv: int, D: int, Dv: int, ctx, pages: Optional[torch.Tensor],
                           block_table: Optional[torch.Tensor], page_size: int, out_dtype: torch.dtype) -> torch.Tensor:
    """proj float32 [T, ld] holds q (Hq x D) at q_col0 and, with Hkv > 0, k (Hkv x D) at k_col0 and v (Hkv x Dv)
    at v_col0.  Adds the biases; q and k each over the root mean square of their whole row slice, times wq / wk
    (of the slice's width); the first `rot` dimensions of every q and k head turned by the row's position (pairs
    (i, i + rot/2), inv_freq float32 [rot / 2]), cosine and sine times `magnitude`.  Returns q [T, Hq * D] in
    `out_dtype` and writes key and value at (request, position): into pages [n, 2, Hkv, page_size, D] (then
    Dv == D) or, when `pages` has three dimensions, into rows [n, page_size, Hkv * (D + Dv)].  Hkv = 0: the
    queries alone."""
    _chk(proj, "proj", torch.float32); _chk(wq, "wq", torch.float32)
    for b, n in ((bias_q, "bias_q"), (bias_k, "bias_k"), (bias_v, "bias_v"), (wk, "wk"), (inv_freq, "inv_freq")):
        if b is not None:
            _chk(b, n, torch.float32)
    T = proj.shape[0]
    q = torch.empty((T, Hq * D), dtype=out_dtype, device=proj.device)
    rows_layout = 0
    if Hkv:
        _chk(pages, "pages", out_dtype); _chk(block_table, "block_table", torch.int32)
        rows_layout = 1 if pages.dim() == 3 else 0
    _lib.call("nf_whole_norm_rope_append", _p(proj), c_int(proj.shape[1]), c_int(q_col0), c_int(k_col0), c_int(v_col0),
              _p(bias_q), _p(bias_k), _p(bias_v), _p(wq), _p(wk), c_float(eps), _p(inv_freq) if rot else None, c_int(rot),
              c_float(magnitude), _p(ctx.positions), _p(ctx.row_seg), _p(q), c_int(T), c_int(Hq), c_int(Hkv), c_int(D),
              c_int(Dv), _p(pages) if Hkv else None, _p(block_table) if Hkv else None,
              c_int(block_table.shape[1] if Hkv else 0), c_int(page_size), c_int(pages.shape[0] if Hkv else 0),
              c_int(rows_layout), c_int(_dt(q)), _stream())
    return q


def sigmoid_gate_rows(o: torch.Tensor, g_src: torch.Tensor, g_col0: int) -> torch.Tensor:
    """o [T, n] times sigmoid(g_src[:, g_col0 : g_col0 + n]) element by element; the gate's logits are float32
    or of o's type."""
    _chk(o, "o"); _chk(g_src, "g_src")
    T, n = o.shape
    out = torch.empty_like(o)
    _lib.call("nf_sigmoid_gate_rows", _p(o), _p(g_src), c_int(_dt(g_src)), c_int(g_src.shape[1]), c_int(g_col0), _p(out),
              c_int(T), c_int(n), c_int(_dt(o)), _stream())
    return out


def biased_window_attention(q: torch.Tensor, Hq: int, Hkv: int, D: int, pages: torch.Tensor, block_table: torch.Tensor,
                            page_size: int, ctx, window: int, keep_first: int, scale: float,
                            slopes: Optional[torch.Tensor], gate: Optional[torch.Tensor] = None,
                            gate_col0: int = 0) -> torch.Tensor:
    """Causal softmax attention of q [T, Hq * D] over the paged keys and values -> [T, Hq * D], with
    slopes[h] * (i - j) taken off head h's score of key j (float32 [Hq] or None), a window (0: none) that
    keeps the request's first `keep_first` keys visible, and head h's output times
    sigmoid(gate[t, gate_col0 + h]) (gate float32 [T, ld] or None)."""
    _chk(q, "q"); _chk(pages, "pages", q.dtype); _chk(block_table, "block_table", torch.int32)
    if slopes is not None:
        _chk(slopes, "slopes", torch.float32)
    if gate is not None:
        _chk(gate, "gate", torch.float32)
    T = q.shape[0]
    out = torch.empty((T, Hq * D), dtype=q.dtype, device=q.device)
    if T == 0:
        return out
    gate_p = c_void_p(gate.data_ptr() + 4 * gate_col0) if gate is not None else None
    gate_ld = gate.shape[1] if gate is not None else 0
    keep = keep_first if window > 0 else 0
    if (q.dtype == torch.bfloat16 and TUNING["bf16_attention"] != "generic" and D in PREFILL_HEAD_DIMS
            and q.shape[1] % 8 == 0 and pages.is_contiguous()):
        # the flash kernel on tensor cores: tiles of 64 rows of a segment, key blocks of 64.  A segment of one row
        # (a decoded token) has its key blocks split over several CTAs, whatever else the step holds.
        if getattr(ctx, "seg_len_host", None) is not None and (ctx.all_single or getattr(ctx, "seg_pos0_host", None) is not None):
            def flash(tiles, n_tiles, shares):
                part_o = part_ml = None
                if shares:
                    part_o = torch.empty((T, Hq, shares, D), dtype=torch.float32, device=q.device)
                    part_ml = torch.empty((T, Hq, shares, 2), dtype=torch.float32, device=q.device)
                _lib.call("nf_prefill_attention_biased", _p(q), c_int(q.shape[1]), _p(pages), _p(block_table),
                          c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.seg_row0), _p(tiles), c_int(n_tiles),
                          _p(out), c_int(Hq), c_int(Hkv), c_int(D), c_int(page_size), c_int(pages.shape[0]), c_int(window),
                          c_float(scale), _p(slopes), c_int(keep), gate_p, c_int(gate_ld), c_int(shares), _p(part_o),
                          _p(part_ml), _stream())
            singles, n_single = ctx.one_row_tiles()
            if n_single:
                flash(singles, n_single, int(_lib.load().nf_prefill_attention_shares(c_int(window), c_int(int(ctx.max_context)))))
            if not ctx.all_single:
                tiles, n_tiles = _tiles(ctx, PREFILL_TILE_ROWS, window, PREFILL_KEY_BLOCK, True, 2 if n_single else 1)
                if n_tiles:
                    flash(tiles, n_tiles, 0)
            return out
    _lib.call("nf_paged_attention_generic", _p(q), c_int(q.shape[1]), _p(pages), _p(block_table),
              c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(out), c_int(T), c_int(Hq),
              c_int(Hkv), c_int(D), c_int(page_size), c_int(pages.shape[0]), c_int(window), c_float(scale),
              c_int(_dt(q)), _p(slopes), c_int(keep), gate_p, c_int(gate_ld), _stream())
    return out


# ---------------------------------------------------------------------------------------
# routed experts
# ---------------------------------------------------------------------------------------

@dataclass
class MoePlan:
    offsets: torch.Tensor   # int32 [E + 1] rows of each expert in sorted order
    order: torch.Tensor     # int32 [T * k] pair (t * k + j) at each sorted position
    inv: torch.Tensor       # int32 [T * k] sorted position of each pair
    num_experts: int
    num_tokens: int
    top_k: int
    active: Optional[torch.Tensor] = None   # int32 [min(E, T * k)] experts that have pairs, -1 padded


def split_router(w_router: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """A float32 routing matrix as bfloat16 `hi` plus bfloat16 `lo` with hi + lo = w to 16 bits
    of mantissa; `lo` is None when the matrix is exactly bfloat16 (the usual checkpoint).
    With them, router logits of many rows are tensor-core products whose every partial
    product is exact and whose sums are float32."""
    hi = w_router.to(torch.bfloat16)
    rest = w_router - hi.to(torch.float32)
    lo = rest.to(torch.bfloat16) if bool((rest != 0).any()) else None
    return hi, lo


def _route_flags(norm_topk: bool, scoring: str) -> int:
    """The selection's flags: bit 0 divides the chosen weights by their sum, bit 1 scores an expert
    by the sigmoid of its own logit instead of the softmax over all."""
    if scoring not in ("softmax", "sigmoid"):
        raise ValueError(f"router scoring {scoring!r}: 'softmax' or 'sigmoid'")
    return (1 if norm_topk else 0) | (2 if scoring == "sigmoid" else 0)


def router_topk(x: torch.Tensor, w_router: torch.Tensor, E: int, k: int, norm_topk: bool,
                split: Optional[Tuple[torch.Tensor, Optional[torch.Tensor]]] = None, scoring: str = "softmax"
                ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Router logits (float32), softmax, top-k.  Rows of `w_router` beyond E give raw
    logits back (`extra`, [T, rows - E]).  Returns (idx int32 [T, k], weights float32 [T, k], extra).

    With many bfloat16 rows and a `split` of the matrix (see `split_router`) the logits come
    from tensor-core products with float32 sums; otherwise from the float32 CUDA-core kernel."""
    _chk(x, "x"); _chk(w_router, "w_router", torch.float32)
    T, H = x.shape
    extra = w_router.shape[0] - E
    idx = torch.empty((T, k), dtype=torch.int32, device=x.device)
    wts = torch.empty((T, k), dtype=torch.float32, device=x.device)
    ext = torch.empty((T, extra), dtype=torch.float32, device=x.device) if extra > 0 else None
    if (split is not None and x.dtype == torch.bfloat16 and T > TUNING["router_tensor_min_rows"]
            and TUNING["bf16_linear"] != "simt" and H % 8 == 0):
        # logits^T [E + extra, T] = W_r x^T with the streaming tensor-core kernel: the routing
        # matrix (at most a few dozen rows) plays the part of the batch, the tokens that of the
        # weights.  Products of bfloat16 values are exact, sums are float32.
        rows = E + extra
        logits_t = torch.empty((rows, T), dtype=torch.float32, device=x.device)
        # The streaming product asks for its weight operand before it waits for the kernel before
        # it - and here that operand is `x`, which that kernel may still be writing.  So these
        # launches are ordinary ones (chained, they read rows of x that were not written yet).
        chain_break()
        _skinny(split[0], H, x, 0, logits_t, rows, T, H, 1, rows, None, None, 1, False)
        if split[1] is not None:
            low = torch.empty_like(logits_t)
            chain_break()
            _skinny(split[1], H, x, 0, low, rows, T, H, 1, rows, None, None, 1, False)
            logits_t += low
        _lib.call("nf_router_select", _p(logits_t), c_longlong(1), c_longlong(T), c_int(T), c_int(E),
                  c_int(extra), c_int(k), c_int(_route_flags(norm_topk, scoring)), _p(idx), _p(wts), _p(ext), _stream())
        return idx, wts, ext
    logits = torch.empty((T, E + extra), dtype=torch.float32, device=x.device)
    _lib.call("nf_router_topk", _p(x), _p(w_router), c_int(T), c_int(H), c_int(E), c_int(extra),
              c_int(k), c_int(_route_flags(norm_topk, scoring)), _p(logits), _p(idx), _p(wts), _p(ext),
              c_int(_dt(x)), _stream())
    return idx, wts, ext


def moe_plan(topk_idx: torch.Tensor, E: int) -> MoePlan:
    _chk(topk_idx, "topk_idx", torch.int32)
    T, k = topk_idx.shape
    dev = topk_idx.device
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    order = torch.empty((T * k,), dtype=torch.int32, device=dev)
    inv = torch.empty((T * k,), dtype=torch.int32, device=dev)
    counts = torch.empty((E,), dtype=torch.int32, device=dev)
    active = torch.empty((min(E, max(T * k, 1)),), dtype=torch.int32, device=dev)
    _lib.call("nf_moe_plan", _p(topk_idx), c_int(T * k), c_int(E), _p(offsets), _p(order), _p(inv),
              _p(counts), _p(active), c_int(active.numel()), _stream())
    return MoePlan(offsets, order, inv, E, T, k, active)


_TICKETS = {}


def route(x: torch.Tensor, w_router: torch.Tensor, E: int, k: int, norm_topk: bool,
          split: Optional[Tuple[torch.Tensor, Optional[torch.Tensor]]] = None, scoring: str = "softmax"):
    """Routing of a step: `router_topk` and `moe_plan` together -> (idx, weights, extra, plan).

    Up to `TUNING["router_fused_max_rows"]` rows this is one launch: blocks compute the
    logits, and the block that finishes last selects for every row and builds the plan."""
    _chk(x, "x"); _chk(w_router, "w_router", torch.float32)
    T, H = x.shape
    if T == 0 or T > TUNING["router_fused_max_rows"]:
        idx, wts, ext = router_topk(x, w_router, E, k, norm_topk, split=split, scoring=scoring)
        return idx, wts, ext, moe_plan(idx, E)
    dev = x.device
    extra = w_router.shape[0] - E
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    ext = torch.empty((T, extra), dtype=torch.float32, device=dev) if extra > 0 else None
    logits = torch.empty((T, E + extra), dtype=torch.float32, device=dev)
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    order = torch.empty((T * k,), dtype=torch.int32, device=dev)
    inv = torch.empty((T * k,), dtype=torch.int32, device=dev)
    active = torch.empty((min(E, T * k),), dtype=torch.int32, device=dev)
    if (T <= TUNING["router_cluster_max_rows"] and x.is_contiguous()
            and _lib.load().nf_router_cluster_fits(T, H, E, extra, k)):
        # one thread-block cluster: logits meet selection and plan in distributed shared memory
        _lib.call("nf_router_cluster", _p(x), _p(w_router), c_int(T), c_int(H), c_int(E), c_int(extra), c_int(k),
                  c_int(_route_flags(norm_topk, scoring)), None, _p(idx), _p(wts), _p(ext), _p(offsets), _p(order),
                  _p(inv), _p(active), c_int(active.numel()), c_int(_dt(x)), _stream())
        return idx, wts, ext, MoePlan(offsets, order, inv, E, T, k, active)
    key = str(dev)
    if key not in _TICKETS:
        _TICKETS[key] = torch.zeros((1,), dtype=torch.int32, device=dev)
    _lib.call("nf_router_fused", _p(x), _p(w_router), c_int(T), c_int(H), c_int(E), c_int(extra), c_int(k),
              c_int(_route_flags(norm_topk, scoring)), _p(logits), _p(idx), _p(wts), _p(ext), _p(offsets), _p(order),
              _p(inv), _p(active), c_int(active.numel()), _p(_TICKETS[key]), c_int(_dt(x)), _stream())
    return idx, wts, ext, MoePlan(offsets, order, inv, E, T, k, active)


def route_ruled(x: torch.Tensor, w_router: torch.Tensor, E: int, k: int, correction: Optional[torch.Tensor],
                groups: int, keep: int, scale: float, real_experts: Optional[int] = None,
                split: Optional[Tuple[torch.Tensor, Optional[torch.Tensor]]] = None):
    """Routing with rules of choice -> (idx int32 [T, k], weights float32 [T, k], plan over all E experts, plan of
    the experts that have matrices).  Scores are the softmax of the float32 logits over all E experts; the choice
    uses score + `correction` (float32 [E] or None) and, with `groups` > 0, only experts of the `keep` groups (of
    `groups` equal groups of neighbours) whose best choice score is largest; the weights are the chosen experts'
    scores (without the correction) over their sum (+ 1e-20), times `scale`.  The experts from `real_experts` up
    (default: none) have no matrices - their output is their input, which `identity_expert_rows` fills in - so the
    second plan shares the first one's arrays and stops at `real_experts`.  With many bfloat16 rows and a `split` of
    the matrix (see `split_router`) the logits come from tensor-core products with float32 sums, as `router_topk`'s do."""
    _chk(x, "x"); _chk(w_router, "w_router", torch.float32)
    if correction is not None:
        _chk(correction, "correction", torch.float32)
    T, H = x.shape
    if w_router.shape != (E, H):
        raise ValueError("route_ruled: the routing matrix does not match the experts")
    dev = x.device
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    if T and (split is not None and x.dtype == torch.bfloat16 and T > TUNING["router_tensor_min_rows"]
              and TUNING["bf16_linear"] != "simt" and H % 8 == 0):
        # logits^T [E, T] = W_r x^T with the streaming tensor-core kernel (the routing matrix plays the part of the
        # batch, the tokens that of the weights); its launches are ordinary ones because it asks for its weight
        # operand - here x - before it waits for the kernel before it
        logits_t = torch.empty((E, T), dtype=torch.float32, device=dev)
        chain_break()
        _skinny(split[0], H, x, 0, logits_t, E, T, H, 1, E, None, None, 1, False)
        if split[1] is not None:
            low = torch.empty_like(logits_t)
            chain_break()
            _skinny(split[1], H, x, 0, low, E, T, H, 1, E, None, None, 1, False)
            logits_t += low
        _lib.call("nf_router_select_ruled", _p(logits_t), c_longlong(1), c_longlong(T), c_int(T), c_int(E), c_int(k),
                  _p(correction), c_int(groups), c_int(keep), c_float(scale), _p(idx), _p(wts), _stream())
    elif T:
        logits = torch.empty((T, E), dtype=torch.float32, device=dev)
        _lib.call("nf_router_logits", _p(x), _p(w_router), c_int(T), c_int(H), c_int(E), _p(logits), c_int(_dt(x)), _stream())
        _lib.call("nf_router_select_ruled", _p(logits), c_longlong(E), c_longlong(1), c_int(T), c_int(E), c_int(k),
                  _p(correction), c_int(groups), c_int(keep), c_float(scale), _p(idx), _p(wts), _stream())
    plan = moe_plan(idx, E)
    real = E if real_experts is None else int(real_experts)
    if real == E:
        return idx, wts, plan, plan
    active = torch.where(plan.active < real, plan.active, torch.full_like(plan.active, -1)) if plan.active is not None else None
    return idx, wts, plan, MoePlan(plan.offsets, plan.order, plan.inv, real, T, k, active)


def identity_expert_rows(x: torch.Tensor, plan: MoePlan, k: int, first: int, y: torch.Tensor) -> None:
    """The experts from `first` up return their input: rows of `y` [T * k, H] (sorted pairs) that belong to them
    become copies of their tokens' rows of `x`."""
    _chk(x, "x"); _chk(y, "y", x.dtype)
    if y.shape[0]:
        _lib.call("nf_identity_expert_rows", _p(x), _p(plan.order), c_int(k), _p(plan.offsets), c_int(first), _p(y),
                  c_int(y.shape[0]), c_int(x.shape[1] * x.element_size()), _stream())


def moe_uses_gathered_rows(x: torch.Tensor, w13) -> bool:
    """Whether `moe_gemm1` would first copy the rows of `x` into sorted order (`moe_gather`)."""
    return isinstance(w13, PackedWeights) and x.shape[0] > TUNING["skinny_moe_max_tokens"]


def moe_gather(x: torch.Tensor, plan: MoePlan, k: int) -> torch.Tensor:
    """Row p of the result is row order[p] // k of `x`: the tokens in the experts' order."""
    _chk(x, "x")
    T, H = x.shape
    xp = torch.empty((T * k, H), dtype=x.dtype, device=x.device)
    if T:
        _lib.call("nf_gather_rows", _p(x), _p(plan.order), c_int(k), _p(xp), c_int(T * k),
                  c_int(H * x.element_size()), _stream())
    return xp


def moe_gemm1(x: torch.Tensor, w13, plan: MoePlan, k: int, gathered: Optional[torch.Tensor] = None,
              sorted_rows: bool = False, act=None) -> torch.Tensor:
    """Sorted pair p (token order[p] // k, expert e) -> silu(x Wgate_e^T) * (x Wup_e^T)  [T*k, I].

    `w13` is [E, 2I, H] (gate rows first), or `PackedWeights` of it for the bfloat16 kernels.
    `gathered`: `moe_gather(x, plan, k)` if the caller has it already.  `sorted_rows`: `x` itself
    is [T*k, H] with row p belonging to sorted pair p (gathered, and possibly scaled, by the caller)."""
    _chk(x, "x")
    if sorted_rows:
        T, H = plan.num_tokens, x.shape[1]
        if x.shape[0] != T * k:
            raise ValueError("moe_gemm1: sorted rows do not match the plan")
        rows, div, gathered = None, 1, x
    else:
        T, H = x.shape
        rows, div = plan.order, k
    packed = isinstance(w13, PackedWeights)
    if packed:
        E, inner = w13.groups, w13.n_features
        if x.dtype != torch.bfloat16 or w13.K != H or not w13.swiglu:
            raise ValueError("moe_gemm1: packed weights do not fit the activations")
    else:
        _chk(w13, "w13", x.dtype)
        E, two_i, _ = w13.shape
        inner = two_i // 2
    out = torch.empty((T * k, inner), dtype=x.dtype, device=x.device)
    if T == 0:
        return out
    if packed:
        if T <= TUNING["skinny_moe_max_tokens"]:
            _skinny(x, H, w13.data, w13.group_stride, out, T * k, inner, H, E, T, plan.offsets, rows,
                    div, True, packed=True, group_map=plan.active, act=act)
        else:
            # rows in sorted order, then one tensor-core launch over all experts
            xp = gathered if gathered is not None else moe_gather(x, plan, k)
            kind, limit, alpha = _act(True, act)
            _lib.call("nf_grouped_gemm_tc", _p(xp), c_longlong(T * k), _p(w13.data), c_int(E),
                      c_int(inner), c_int(H), _p(plan.offsets), _p(out), c_int(inner), c_int(kind),
                      c_float(limit), c_float(alpha), _stream())
        return out
    path = "simt" if x.dtype == torch.float32 else _bf16_path(T, H, "bf16_moe")
    if path == "skinny":
        _skinny(x, H, w13, two_i * H, out, T * k, inner, H, E, T, plan.offsets, rows, div, True,
                group_map=plan.active, act=act)
    else:
        _gemm_simt(x, H, w13, two_i * H, out, T * k, inner, H, E, T, plan.offsets, rows, div, True, act=act)
    return out


def moe_experts_sorted(xs: torch.Tensor, w13, w2, plan: MoePlan, act=None) -> torch.Tensor:
    """Both products of the routed experts over rows that are already in the experts' order
    (row p of `xs` is sorted pair p's input) -> [T*k, H] in the same order."""
    return moe_gemm2(moe_gemm1(xs, w13, plan, plan.top_k, sorted_rows=True, act=act), w2, plan, plan_is_older=True)


def moe_gemm2(act: torch.Tensor, w2, plan: MoePlan, plan_is_older: bool = False, gelu: bool = False) -> torch.Tensor:
    """Sorted pair p of expert e -> act[p] Wdown_e^T  [T*k, H].  `w2` is [E, H, I] or packed.
    `gelu`: the exact GELU of the result (in the tensor-core kernel's epilogue, on the float32 sums;
    a pass of its own after the other kernels).

    `plan_is_older`: the plan was complete before the kernel that produced `act` was launched
    (the usual order: router, first product, this).  The streaming kernel then starts fetching
    weights while that kernel is still finishing."""
    _chk(act, "act")
    n, inner = act.shape
    packed = isinstance(w2, PackedWeights)
    if packed:
        E, H = w2.groups, w2.n_features
        if act.dtype != torch.bfloat16 or w2.K != inner or w2.swiglu:
            raise ValueError("moe_gemm2: packed weights do not fit the activations")
    else:
        _chk(w2, "w2", act.dtype)
        E, H, _ = w2.shape
    y = torch.empty((n, H), dtype=act.dtype, device=act.device)
    if n == 0:
        return y
    if packed:
        if plan.num_tokens <= TUNING["skinny_moe_max_tokens"]:
            _skinny(act, inner, w2.data, w2.group_stride, y, n, H, inner, E, plan.num_tokens, plan.offsets,
                    None, 1, False, packed=True, group_map=plan.active, early_index=plan_is_older)
        else:
            _lib.call("nf_grouped_gemm_tc", _p(act), c_longlong(n), _p(w2.data), c_int(E), c_int(H),
                      c_int(inner), _p(plan.offsets), _p(y), c_int(H), c_int(3 if gelu else 0), c_float(0.0),
                      c_float(0.0), _stream())
            return y
        return gelu_erf_(y) if gelu else y
    path = "simt" if act.dtype == torch.float32 else _bf16_path(plan.num_tokens, inner, "bf16_moe")
    if path == "skinny":
        _skinny(act, inner, w2, H * inner, y, n, H, inner, E, plan.num_tokens, plan.offsets, None, 1, False,
                group_map=plan.active, early_index=plan_is_older)
    else:
        _gemm_simt(act, inner, w2, H * inner, y, n, H, inner, E, plan.num_tokens, plan.offsets, None, 1, False)
    return gelu_erf_(y) if gelu else y


_STREAM_WORK = {}


def _stream_items(x: torch.Tensor, w13, w2, E: int, k: int, routes: bool = False, shared_chunks: int = 0) -> int:
    """Sixteen-feature groups an item of the persistent experts' kernel covers (8, 4 or 2), or 0 if
    the step does not fit the kernel.  The fewer experts a step selects, the finer the items, so
    that every SM has some; a finer item also needs a smaller ring.  `routes`: the launch is to
    route as well."""
    T, H = x.shape
    if not (isinstance(w13, PackedWeights) and isinstance(w2, PackedWeights) and x.is_cuda):
        return 0
    if T < max(TUNING["moe_stream_min_tokens"], 1) or T > TUNING["moe_stream_max_tokens"] or x.dtype != torch.bfloat16 or not x.is_contiguous():
        return 0
    if routes and T > TUNING["moe_stream_route_max_tokens"]:
        return 0
    if w13.K != H or w2.n_features != H or w2.K != w13.n_features or not w13.swiglu or w2.swiglu:
        return 0
    pairs = T * k
    q = 8 if pairs >= 16 else (4 if pairs >= 8 else 2)
    fits = _lib.load().nf_moe_stream_fits
    while q >= 2 and not fits(H, w13.n_features, pairs, min(E, pairs), q, TUNING["moe_stream_smem_kb"] * 1024,
                              E if routes else 0, shared_chunks * T):
        q //= 2
    return q if q >= 2 else 0


def moe_experts_fit_stream(x: torch.Tensor, w13, w2, plan: MoePlan, k: int) -> bool:
    """Whether `moe_experts` serves this step with the one persistent launch."""
    return plan.active is not None and _stream_items(x, w13, w2, plan.num_experts, k) > 0


def _stream_work(device: torch.device) -> torch.Tensor:
    """The persistent launch's counters and tables: one buffer a device, so its launches must not
    overlap one another - they are issued to one stream (the step's), eagerly or inside its
    graphs, and each leaves the counters at zero."""
    key = str(device)
    if key not in _STREAM_WORK:
        _STREAM_WORK[key] = torch.zeros((int(_lib.load().nf_moe_stream_work_ints()),), dtype=torch.int32, device=device)
    return _STREAM_WORK[key]


def moe_experts(x: torch.Tensor, w13, w2, plan: MoePlan, k: int,
                gathered: Optional[torch.Tensor] = None, act=None) -> torch.Tensor:
    """Both products of the routed experts: sorted pair p of expert e ->
    (silu(x Wgate_e^T) * (x Wup_e^T)) Wdown_e^T  [T*k, H].

    A decode step with packed bfloat16 weights is one persistent launch that streams the weights
    of both products through one ring (`moe_stream.cu`); everything else is `moe_gemm1` followed
    by `moe_gemm2`."""
    q = _stream_items(x, w13, w2, plan.num_experts, k) if plan.active is not None else 0
    if not q:
        return moe_gemm2(moe_gemm1(x, w13, plan, k, gathered=gathered, act=act), w2, plan, plan_is_older=True)
    T, H = x.shape
    inner = w13.n_features
    kind, limit, alpha = _act(True, act)
    act = torch.empty((T * k, inner), dtype=x.dtype, device=x.device)
    y = torch.empty((T * k, H), dtype=x.dtype, device=x.device)
    _lib.call("nf_moe_stream", _p(x), c_int(x.stride(0)), _p(w13.data), c_longlong(w13.group_stride), _p(w2.data),
              c_longlong(w2.group_stride), _p(act), _p(y), c_int(T * k), c_int(T), c_int(H), c_int(inner),
              c_int(w13.groups), c_int(k), _p(plan.offsets), _p(plan.order), _p(plan.active),
              c_int(plan.active.numel()), _p(_stream_work(x.device)), c_int(q),
              c_int(TUNING["moe_stream_smem_kb"] * 1024), None, c_int(0), c_int(0), None, None, None, None, None,
              None, c_longlong(0), None, c_longlong(0), c_int(0), None, None, c_int(kind), c_float(limit),
              c_float(alpha), _stream())
    return y


def pack_shared_expert(w_gate_up: torch.Tensor, w_down: torch.Tensor, chunk: int) -> Tuple[PackedWeights, PackedWeights]:
    """A shared expert's matrices ([2 Is, H] gate rows first, and [H, Is]) as ceil(Is / chunk)
    experts of `chunk` intermediate features each, packed like the routed ones (the last chunk
    padded with zero features, which contribute nothing).  Its output is then the sum of the
    chunks' outputs, and the persistent experts' launch can serve it."""
    _chk(w_gate_up, "w_gate_up", torch.bfloat16); _chk(w_down, "w_down", torch.bfloat16)
    two_is, H = w_gate_up.shape
    inner = two_is // 2
    n = (inner + chunk - 1) // chunk
    g = torch.zeros((n, 2 * chunk, H), dtype=w_gate_up.dtype, device=w_gate_up.device)
    d = torch.zeros((n, H, chunk), dtype=w_down.dtype, device=w_down.device)
    for c in range(n):
        lo, hi = c * chunk, min(inner, (c + 1) * chunk)
        g[c, :hi - lo] = w_gate_up[lo:hi]
        g[c, chunk:chunk + hi - lo] = w_gate_up[inner + lo:inner + hi]
        d[c, :, :hi - lo] = w_down[:, lo:hi]
    return pack_weights(g, swiglu=True), pack_weights(d, swiglu=False)


def can_route_and_run_experts(x: torch.Tensor, w_router: torch.Tensor, w13, w2, E: int, k: int,
                              shared: Optional[Tuple[PackedWeights, PackedWeights]] = None) -> bool:
    """Whether `route_and_run_experts` serves this step (else: `route`, then `moe_experts`)."""
    if not (w_router.dtype == torch.float32 and w_router.is_contiguous() and w_router.shape[1] == x.shape[1]):
        return False
    chunks = 0
    if shared is not None:
        s13, s2 = shared
        if not (isinstance(w13, PackedWeights) and s13.n_features == w13.n_features and s13.K == w13.K
                and s2.n_features == x.shape[1] and s2.K == w13.n_features and k + s13.groups <= 32):
            return False
        chunks = s13.groups
        if x.shape[0] > TUNING["moe_stream_shared_max_tokens"]:
            return False
    return _stream_items(x, w13, w2, E, k, routes=True, shared_chunks=chunks) > 0


def route_and_run_experts(x: torch.Tensor, w_router: torch.Tensor, E: int, k: int, norm_topk: bool, w13, w2,
                          shared: Optional[Tuple[PackedWeights, PackedWeights]] = None, act=None):
    """`route` and `moe_experts` in the one persistent launch: its CTAs compute the router logits
    between them, the one that finishes last selects and writes the plan, and all go on to the
    experts' products.  Returns (idx, weights, extra, plan, y) as the two calls would.

    With `shared` (`pack_shared_expert`) the launch serves the shared expert too, as further
    experts that every token has - their weights are on their way while the routing is still
    being computed.  Then y has T * (k + chunks) rows, and two more values are returned: the
    weights [T, k + chunks] (the k experts', then sigmoid of the first further logit for every
    chunk, or 1 without one) and a plan whose `inv` [T * (k + chunks)] names the rows of y to add
    up for every token - what `moe_combine` and the fused norm take."""
    chunks = shared[0].groups if shared is not None else 0
    q = _stream_items(x, w13, w2, E, k, routes=True, shared_chunks=chunks)
    if not q:
        raise ValueError("route_and_run_experts: the step does not fit the launch")
    T, H = x.shape
    dev = x.device
    inner = w13.n_features
    extra = w_router.shape[0] - E
    rows = T * (k + chunks)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    wts = torch.empty((T, k), dtype=torch.float32, device=dev)
    ext = torch.empty((T, extra), dtype=torch.float32, device=dev) if extra > 0 else None
    logits = torch.empty((T, E + extra), dtype=torch.float32, device=dev)
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    order = torch.empty((T * k,), dtype=torch.int32, device=dev)
    inv = torch.empty((T * k,), dtype=torch.int32, device=dev)
    active = torch.empty((min(E, T * k),), dtype=torch.int32, device=dev)
    kind, limit, alpha = _act(True, act)
    act = torch.empty((rows, inner), dtype=x.dtype, device=dev)
    y = torch.empty((rows, H), dtype=x.dtype, device=dev)
    cw = torch.empty((T, k + chunks), dtype=torch.float32, device=dev) if chunks else None
    cinv = torch.empty((rows,), dtype=torch.int32, device=dev) if chunks else None
    s13, s2 = shared if shared is not None else (None, None)
    _lib.call("nf_moe_stream", _p(x), c_int(x.stride(0)), _p(w13.data), c_longlong(w13.group_stride), _p(w2.data),
              c_longlong(w2.group_stride), _p(act), _p(y), c_int(T * k), c_int(T), c_int(H), c_int(inner),
              c_int(E), c_int(k), _p(offsets), _p(order), _p(active), c_int(active.numel()),
              _p(_stream_work(dev)), c_int(q), c_int(TUNING["moe_stream_smem_kb"] * 1024), _p(w_router),
              c_int(extra), c_int(1 if norm_topk else 0), _p(logits), _p(idx), _p(wts), _p(ext), _p(inv),
              _p(s13.data) if chunks else None, c_longlong(s13.group_stride if chunks else 0),
              _p(s2.data) if chunks else None, c_longlong(s2.group_stride if chunks else 0), c_int(chunks),
              _p(cw), _p(cinv), c_int(kind), c_float(limit), c_float(alpha), _stream())
    plan = MoePlan(offsets, order, inv, E, T, k, active)
    if not chunks:
        return idx, wts, ext, plan, y
    return idx, wts, ext, plan, y, cw, MoePlan(offsets, order, cinv, E, T, k + chunks, active)


def moe_combine(y: torch.Tensor, plan: MoePlan, wts: torch.Tensor, shared: Optional[torch.Tensor],
                gate: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """out[t] = sum_j wts[t, j] * y[inv[t, j]] (j ascending) + sigmoid(gate[t]) * shared[t]."""
    _chk(y, "y"); _chk(wts, "wts", torch.float32)
    T, k = wts.shape
    H = y.shape[1]
    out = torch.empty((T, H), dtype=out_dtype, device=y.device)
    _lib.call("nf_moe_combine", _p(y), _p(plan.inv), _p(wts), _p(shared), _p(gate),
              c_int(gate.shape[1] if gate is not None else 0), _p(out), c_int(T), c_int(H), c_int(k),
              c_int(_dt(y)), _stream())
    return out


FUSED_COMBINE_MAX_K = 32


def can_fuse_combine_norm(y: torch.Tensor, hidden: int, rows: int, k: int = 1) -> bool:
    """Whether `moe_combine_add_rmsnorm` serves these operands (bfloat16 on the device, a row that
    the kernel's threads can keep in registers, few enough rows)."""
    return (y.is_cuda and y.dtype == torch.bfloat16 and rows <= TUNING["fuse_combine_norm_max_rows"]
            and k <= FUSED_COMBINE_MAX_K and bool(_lib.load().nf_moe_combine_add_rmsnorm_fits(c_int(hidden))))


def moe_combine_add_rmsnorm(y: torch.Tensor, plan: MoePlan, wts: torch.Tensor, shared: Optional[torch.Tensor],
                            gate: Optional[torch.Tensor], h: torch.Tensor, rows: Optional[torch.Tensor],
                            weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """`moe_combine` and `add_rmsnorm` (`rows` None: h updated in place) or `add_rmsnorm_rows` in
    one launch, bit for bit what the two give one after the other."""
    _chk(y, "y", torch.bfloat16); _chk(wts, "wts", torch.float32); _chk(h, "h", torch.float32)
    _chk(weight, "weight", torch.float32); _chk(out, "out", torch.bfloat16)
    T, k = wts.shape
    R = T if rows is None else rows.numel()
    _lib.call("nf_moe_combine_add_rmsnorm", _p(y), _p(plan.inv), _p(wts), _p(shared), _p(gate),
              c_int(gate.shape[1] if gate is not None else 0), _p(h), _p(rows), _p(weight), c_float(eps),
              _p(out), c_int(T), c_int(R), c_int(h.shape[1]), c_int(k), _stream())


# ---------------------------------------------------------------------------------------
# layer norm, slices, gates
# ---------------------------------------------------------------------------------------

def add_layernorm(h: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor],
                  weight: torch.Tensor, eps: float, out: torch.Tensor, routed=None) -> None:
    """h += delta (float32, in place); out = (h - mean) * rsqrt(var + eps) * weight, var the mean of
    the squared deviations.  With `rows`: out[r] from h[rows[r]] + delta[rows[r]], h left alone.
    `routed` = (y, inv, wts or None, k) instead of `delta`: the routed experts' pending sum
    sum_j wts[t, j] * y[inv[t * k + j]] is added up inside the kernel (same bits as `moe_combine` first)."""
    _chk(h, "h", torch.float32); _chk(weight, "weight", torch.float32); _chk(out, "out")
    if delta is not None:
        _chk(delta, "delta", out.dtype)
    if rows is not None:
        _chk(rows, "rows", torch.int32)
    y = inv = wts = None
    k = 0
    if routed is not None:
        y, inv, wts, k = routed
        _chk(y, "y", out.dtype); _chk(inv, "inv", torch.int32)
        if wts is not None:
            _chk(wts, "wts", torch.float32)
    R = h.shape[0] if rows is None else rows.numel()
    _lib.call("nf_add_layernorm", _p(h), _p(delta), _p(rows), _p(weight), c_float(eps), _p(out), c_int(R),
              c_int(h.shape[1]), c_int(_dt(out)), _p(y), _p(inv), _p(wts), c_int(k), _stream())


def rms_norm_slice(x: torch.Tensor, col0: int, n: int, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """Columns [col0, col0 + n) of x [T, ld] over their root mean square (eps inside the root),
    times `weight` (float32 [n], or None) -> [T, n]."""
    _chk(x, "x")
    if weight is not None:
        _chk(weight, "weight", torch.float32)
    T, ld = x.shape
    out = torch.empty((T, n), dtype=x.dtype, device=x.device)
    _lib.call("nf_rms_norm_slice", _p(x), c_int(ld), c_int(col0), c_int(n), _p(weight), c_float(eps), _p(out),
              c_int(n), c_int(T), c_int(_dt(x)), _stream())
    return out


def gated_group_rmsnorm(y: torch.Tensor, z_src: torch.Tensor, z_col0: int, weight: torch.Tensor, eps: float,
                        parts: int, out_dtype: torch.dtype) -> torch.Tensor:
    """g = y * silu(z), z = z_src[:, z_col0 : z_col0 + inner]; every one of `parts` equal parts of
    a row over its own root mean square; times weight -> [T, inner] in `out_dtype`.  y is float32."""
    _chk(y, "y", torch.float32); _chk(z_src, "z_src", out_dtype); _chk(weight, "weight", torch.float32)
    T, inner = y.shape
    out = torch.empty((T, inner), dtype=out_dtype, device=y.device)
    _lib.call("nf_gated_group_rmsnorm", _p(y), _p(z_src), c_int(z_src.shape[1]), c_int(z_col0), _p(weight),
              c_float(eps), _p(out), c_int(T), c_int(inner), c_int(parts), c_int(_dt(out)), _stream())
    return out


def add_row_vector(h: torch.Tensor, vec: torch.Tensor) -> None:
    """h[t] += vec for every row (float32, in place)."""
    _chk(h, "h", torch.float32); _chk(vec, "vec", torch.float32)
    if vec.numel() != h.shape[1]:
        raise ValueError("add_row_vector: the vector does not have the rows' width")
    _lib.call("nf_add_row_vector", _p(h), _p(vec), c_int(h.shape[0]), c_int(h.shape[1]), _stream())


def heads_sigmoid_gate(v: torch.Tensor, g_src: torch.Tensor, g_col0: int) -> torch.Tensor:
    """v [heads, T, n] (head-major) times sigmoid(g_src[:, g_col0 + head * n + i]) -> [T, heads * n]."""
    _chk(v, "v"); _chk(g_src, "g_src", v.dtype)
    heads, T, n = v.shape
    out = torch.empty((T, heads * n), dtype=v.dtype, device=v.device)
    _lib.call("nf_heads_sigmoid_gate", _p(v), _p(g_src), c_int(g_src.shape[1]), c_int(g_col0), _p(out), c_int(T),
              c_int(heads), c_int(n), c_int(_dt(v)), _stream())
    return out


def scale_gather_rows(x: torch.Tensor, plan: "MoePlan", k: int, wts: torch.Tensor) -> torch.Tensor:
    """Row p of the result is wts[pair] * x[pair // k], pair = plan.order[p]: the tokens in the
    experts' order, each already multiplied by the weight of its (token, choice) pair."""
    _chk(x, "x"); _chk(wts, "wts", torch.float32)
    T, H = x.shape
    out = torch.empty((T * k, H), dtype=x.dtype, device=x.device)
    _lib.call("nf_scale_gather_rows", _p(x), _p(plan.order), c_int(k), _p(wts), _p(out), c_int(T * k), c_int(H),
              c_int(_dt(x)), _stream())
    return out


def heads_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [heads, T, a] times w [heads, a, b] -> [heads, T, b]: one product a head (a library's
    batched product; float32 operands are multiplied in true float32)."""
    _chk(x, "x", contiguous=False); _chk(w, "w", x.dtype, contiguous=False)
    return torch.bmm(x, w)


def scaled_norm_add(h: torch.Tensor, delta: torch.Tensor, bias: Optional[torch.Tensor], weight: torch.Tensor,
                    scale: Optional[torch.Tensor], eps: float, out_dtype: Optional[torch.dtype]) -> Optional[torch.Tensor]:
    """h += scale * ((delta + bias) / rms(delta + bias)) * weight, float32 and in place; delta is float32 or
    bfloat16.  With `out_dtype`, also returns the updated rows in that type (the next sublayer's input)."""
    _chk(h, "h", torch.float32); _chk(delta, "delta"); _chk(weight, "weight", torch.float32)
    for t, n in ((bias, "bias"), (scale, "scale")):
        if t is not None:
            _chk(t, n, torch.float32)
    if delta.shape != h.shape:
        raise ValueError("scaled_norm_add: delta does not have the stream's shape")
    out = torch.empty(h.shape, dtype=out_dtype, device=h.device) if out_dtype is not None else None
    _lib.call("nf_scaled_norm_add", _p(h), _p(delta), c_int(_dt(delta)), _p(bias), _p(weight), _p(scale), c_float(eps),
              _p(out), c_int(_dt(out) if out is not None else 0), c_int(h.shape[0]), c_int(h.shape[1]), _stream())
    return out


def routed_scaled_norm_add(h: torch.Tensor, y: torch.Tensor, inv: torch.Tensor, wts: Optional[torch.Tensor], k: int,
                           weight: torch.Tensor, scale: Optional[torch.Tensor], eps: float,
                           out_dtype: Optional[torch.dtype]) -> Optional[torch.Tensor]:
    """`scaled_norm_add` whose delta is the routed experts' pending sum, sum_j wts[t, j] * y[inv[t * k + j]]
    (rounded to y's type, as `moe_combine` rounds it), added up inside the kernel."""
    _chk(h, "h", torch.float32); _chk(y, "y"); _chk(inv, "inv", torch.int32); _chk(weight, "weight", torch.float32)
    for t, n in ((wts, "wts"), (scale, "scale")):
        if t is not None:
            _chk(t, n, torch.float32)
    out = torch.empty(h.shape, dtype=out_dtype, device=h.device) if out_dtype is not None else None
    _lib.call("nf_routed_scaled_norm_add", _p(h), _p(y), _p(inv), _p(wts), c_int(k), c_int(_dt(y)), _p(weight),
              _p(scale), c_float(eps), _p(out), c_int(_dt(out) if out is not None else 0), c_int(h.shape[0]),
              c_int(h.shape[1]), _stream())
    return out


def mean_of_rmsnorms(xs, ws, eps: float) -> torch.Tensor:
    """float32 [T, W]: the mean over m of (xs[m] / rms(xs[m])) * ws[m]; one to four inputs of equal shape."""
    n = len(xs)
    if not 1 <= n <= 4 or len(ws) != n:
        raise ValueError("mean_of_rmsnorms: one to four inputs, a weight each")
    for x in xs:
        _chk(x, "x", xs[0].dtype)
        if x.shape != xs[0].shape:
            raise ValueError("mean_of_rmsnorms: inputs of different shapes")
    for w in ws:
        _chk(w, "w", torch.float32)
    T, W = xs[0].shape
    out = torch.empty((T, W), dtype=torch.float32, device=xs[0].device)
    xp = (c_void_p * n)(*[x.data_ptr() for x in xs])
    wp = (c_void_p * n)(*[w.data_ptr() for w in ws])
    _lib.call("nf_mean_of_rmsnorms", xp, wp, c_int(n), c_float(eps), _p(out), c_int(T), c_int(W), c_int(_dt(xs[0])),
              _stream())
    return out


GATE_SILU, GATE_SIGMOID = 0, 1


def group_rmsnorm_gate(y: torch.Tensor, z_src: torch.Tensor, z_col0: int, weight: Optional[torch.Tensor], eps: float,
                       parts: int, gate: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Every one of `parts` equal parts of a row of y (float32 [T, inner]) over its own root mean square, times
    `weight` (or nothing), times silu or sigmoid of z = z_src[:, z_col0 : z_col0 + inner] (of `out_dtype`, or
    float32 sums) -> [T, inner]."""
    _chk(y, "y", torch.float32); _chk(z_src, "z_src", None if z_src.dtype == torch.float32 else out_dtype)
    if weight is not None:
        _chk(weight, "weight", torch.float32)
    T, inner = y.shape
    out = torch.empty((T, inner), dtype=out_dtype, device=y.device)
    _lib.call("nf_group_rmsnorm_gate", _p(y), _p(z_src), c_int(z_src.shape[1]), c_int(z_col0), _p(weight), c_float(eps),
              _p(out), c_int(T), c_int(inner), c_int(parts), c_int(gate), c_int(_dt(out)), c_int(_dt(z_src)), _stream())
    return out


def gated_bias_act(gu: torch.Tensor, bias: Optional[torch.Tensor], act, out_dtype: torch.dtype) -> torch.Tensor:
    """[M, 2I] (gate columns first; float32 or `out_dtype`) -> the gated activation `act` of (gate + bias, up + bias)."""
    _chk(gu, "gu")
    if bias is not None:
        _chk(bias, "bias", torch.float32)
    M, two_i = gu.shape
    kind, limit, alpha = _act(True, act)
    out = torch.empty((M, two_i // 2), dtype=out_dtype, device=gu.device)
    _lib.call("nf_gated_bias_act", _p(gu), c_int(_dt(gu)), _p(bias), _p(out), c_int(M), c_int(two_i // 2), c_int(kind),
              c_float(limit), c_float(alpha), c_int(_dt(out)), _stream())
    return out


def cast_rows(h: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 stream rounded to the engine's type."""
    _chk(h, "h", torch.float32)
    out = torch.empty(h.shape, dtype=dtype, device=h.device)
    _lib.call("nf_cast_rows", _p(h), _p(out), c_longlong(h.numel()), c_int(_dt(out)), _stream())
    return out


def pair_hash_embed(table: torch.Tensor, ctx, last: torch.Tensor, h: torch.Tensor, buckets: int, mul_prev: int,
                    mul_cur: int) -> None:
    """h[t] += table[(prev * mul_prev + token * mul_cur) mod buckets], or table[buckets] for a request's first
    token.  `last` int32 [slots, 1]: each request's last token + 1 (0: none), read for a segment's first row and
    updated to the segment's last token."""
    _chk(table, "table"); _chk(h, "h", torch.float32); _chk(last, "last", torch.int32)
    if table.shape[0] != buckets + 1 or table.shape[1] != h.shape[1]:
        raise ValueError("pair_hash_embed: the table must be [buckets + 1, width]")
    _lib.call("nf_pair_hash_embed", _p(table), _p(ctx.token_ids), _p(ctx.row_seg), _p(ctx.seg_row0), _p(ctx.seg_slot),
              _p(last), c_longlong(last.stride(0)), _p(h), c_int(h.shape[0]), c_int(h.shape[1]), c_int(buckets),
              c_longlong(mul_prev), c_longlong(mul_cur), c_int(_dt(table)), _stream())


LINEAR_ATTENTION_MAX_DIM = 256


def decay_linear_attention(src: torch.Tensor, q_col0: int, k_col0: int, v_col0: int, decay: torch.Tensor,
                           inv_freq: Optional[torch.Tensor], rot: int, k_scale: float, silu: bool,
                           state: torch.Tensor, ctx, heads: int, D: int, V: int, q_scale: float = 1.0,
                           gates: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The recurrence S <- decay_h S + k v^T, o = S^T q over a step's rows, request by request, from and into
    each request's state (float32 [slots, heads * V * D], a column's D entries contiguous).  q, k (heads x D) and
    v (heads x V) are columns of `src`; `silu` passes all three through SiLU first; the first `rot` dimensions of
    every q and k head are turned by the row's position (inv_freq float32 [rot / 2]); k is scaled by `k_scale`, q by
    `q_scale`.  With `gates` (float32 [T, heads, 3] of (a, b, c) a row and head; `decay` may then be None) the
    recurrence is S <- a S + b k v^T, o = c S^T q.  Returns o float32 [T, heads * V]."""
    _chk(src, "src"); _chk(state, "state", torch.float32)
    if gates is not None:
        _chk(gates, "gates", torch.float32)
    else:
        _chk(decay, "decay", torch.float32)
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32)
    T = src.shape[0]
    out = torch.empty((T, heads * V), dtype=torch.float32, device=src.device)
    prepared = None
    single = bool(getattr(ctx, "all_single", False))
    if not single and D % 4 == 0 and D > 16:
        # a step with prompt portions: q and k are activated, turned and scaled once for all the CTAs of a head
        # (same arithmetic as inside the recurrence kernel, which does it itself for single rows)
        prepared = torch.empty((T, 2 * heads * D), dtype=torch.float32, device=src.device)
        _lib.call("nf_linear_attention_prepare", _p(src), c_int(src.shape[1]), c_int(q_col0), c_int(k_col0),
                  _p(inv_freq) if rot else None, c_int(rot), c_float(k_scale), c_int(1 if silu else 0), _p(ctx.positions),
                  _p(prepared), c_int(T), c_int(heads), c_int(D), c_int(_dt(src)), c_float(q_scale), _stream())
    _lib.call("nf_decay_linear_attention", _p(src), c_int(src.shape[1]), c_int(q_col0), c_int(k_col0), c_int(v_col0),
              _p(decay), _p(inv_freq) if rot else None, c_int(rot), c_float(k_scale), c_int(1 if silu else 0),
              _p(state), c_longlong(state.stride(0)), _p(ctx.seg_row0), _p(ctx.seg_slot), _p(ctx.seg_pos0), _p(out),
              c_int(ctx.S), c_int(heads), c_int(D), c_int(V), c_int(_dt(src)), _p(prepared), c_int(1 if single else 0),
              c_float(q_scale), _p(gates), _stream())
    return out


def mlstm_gates(src: torch.Tensor, q_col0: int, k_col0: int, q_scale: float, pre: torch.Tensor, i_col0: int, f_col0: int,
                bias_i: Optional[torch.Tensor], bias_f: Optional[torch.Tensor], cap: float, state: torch.Tensor,
                n_off: int, m_off: int, ctx, heads: int, D: int) -> torch.Tensor:
    """The gates of the matrix-memory recurrence with a running maximum, request by request from and into each
    request's state: log input gate i = cap tanh((pre_i + bias_i) / cap), log forget gate
    f = logsigmoid(cap tanh((pre_f + bias_f) / cap)), m <- max(f + m, i), a = exp(f + m_old - m), b = exp(i - m),
    n <- a n + b k, c = 1 / (max(|n . q q_scale|, exp(-m)) + 1e-6).  `pre` float32 [T, ld] holds the heads' gate
    projections at i_col0 and f_col0; q and k (heads x D) are columns of `src`; a slot of `state` (float32
    [slots, n]) keeps n at n_off ([heads][D]) and m at m_off ([heads]).  Returns float32 [T, heads, 3] of (a, b, c)
    for `decay_linear_attention(..., gates=)`."""
    _chk(src, "src"); _chk(pre, "pre", torch.float32); _chk(state, "state", torch.float32)
    for b, n in ((bias_i, "bias_i"), (bias_f, "bias_f")):
        if b is not None:
            _chk(b, n, torch.float32)
    T = src.shape[0]
    gates = torch.empty((T, heads, 3), dtype=torch.float32, device=src.device)
    _lib.call("nf_mlstm_gates", _p(src), c_int(src.shape[1]), c_int(q_col0), c_int(k_col0), c_float(q_scale), _p(pre),
              c_int(pre.shape[1]), c_int(i_col0), c_int(f_col0), _p(bias_i), _p(bias_f), c_float(cap),
              c_void_p(state.data_ptr() + 4 * n_off), c_void_p(state.data_ptr() + 4 * m_off), c_longlong(state.stride(0)),
              _p(ctx.seg_row0), _p(ctx.seg_slot), _p(gates), c_int(ctx.S), c_int(heads), c_int(D), c_int(_dt(src)), _stream())
    return gates


# ---------------------------------------------------------------------------------------
# state-space mixer
# ---------------------------------------------------------------------------------------

CONV_MAX_TAPS = 8
SCAN_MAX_STATE = 256


def causal_conv_silu(src: torch.Tensor, col0: int, C: int, taps: torch.Tensor, bias: Optional[torch.Tensor],
                     state: torch.Tensor, ctx) -> torch.Tensor:
    """silu(bias + causal convolution per channel) of columns [col0, col0 + C) of src [T, ld] -> [T, C].
    taps float32 [K, C], tap-major (last row: the current token's).  `state` float32 [slots, >= (K - 1) * C]:
    each request's last K - 1 inputs, read for the positions before this step and replaced by
    the step's last inputs afterwards."""
    _chk(src, "src"); _chk(taps, "taps", torch.float32); _chk(state, "state", torch.float32)
    T, ld = src.shape
    K = taps.shape[0]
    if taps.shape[1] != C:
        raise ValueError("causal_conv_silu: taps must be [K, C]")
    out = torch.empty((T, C), dtype=src.dtype, device=src.device)
    _lib.call("nf_causal_conv_silu", _p(src), c_int(ld), c_int(col0), c_int(C), _p(taps), _p(bias), c_int(K),
              _p(state), c_longlong(state.stride(0)), _p(ctx.row_seg), _p(ctx.seg_row0), _p(ctx.seg_slot), _p(out),
              c_int(T), c_int(ctx.S), c_int(_dt(src)), _stream())
    return out


def ssd_scan(xbc: torch.Tensor, x_col0: int, b_col0: int, c_col0: int, dt_src: torch.Tensor, dt_col0: int,
             dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor, state: torch.Tensor, state_off: int,
             ctx, heads: int, P: int, N: int, groups: int) -> torch.Tensor:
    """The selective scan of a step's rows, request by request, from and into each request's
    state (float32 [slots, ...], the [heads, P, N] block starting at element `state_off`):
    S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, dt = softplus(raw + dt_bias).
    x, B, C are columns of `xbc`, raw dt a column of `dt_src`.  Returns y float32 [T, heads * P]."""
    _chk(xbc, "xbc"); _chk(dt_src, "dt_src", xbc.dtype); _chk(state, "state", torch.float32)
    for t, n in ((dt_bias, "dt_bias"), (A_log, "A_log"), (D, "D")):
        _chk(t, n, torch.float32)
    T = xbc.shape[0]
    y = torch.empty((T, heads * P), dtype=torch.float32, device=xbc.device)
    _lib.call("nf_ssd_scan", _p(xbc), c_int(xbc.shape[1]), c_int(x_col0), c_int(b_col0), c_int(c_col0), _p(dt_src),
              c_int(dt_src.shape[1]), c_int(dt_col0), _p(dt_bias), _p(A_log), _p(D),
              c_void_p(state.data_ptr() + 4 * state_off), c_longlong(state.stride(0)), _p(ctx.seg_row0),
              _p(ctx.seg_slot), _p(y), c_int(ctx.S), c_int(heads), c_int(P), c_int(N), c_int(groups),
              c_int(_dt(xbc)), _stream())
    return y


# ---------------------------------------------------------------------------------------
# attention over latent rows
# ---------------------------------------------------------------------------------------

LATENT_MAX_RANK = 512
LATENT_TILE_PAIRS = 32      # (token, head) pairs a tile of the tensor-core kernel
LATENT_KEY_BLOCK = 64       # keys a block of that kernel
LATENT_SPLIT_CTAS = 148     # long contexts are split until about this many CTAs run (one a SM)


def latent_append(src: torch.Tensor, col0: int, R: int, Dr: int, weight: torch.Tensor, eps: float,
                  inv_freq: Optional[torch.Tensor], rot_dims: int, ctx, pages: torch.Tensor,
                  block_table: torch.Tensor, page_size: int) -> None:
    """Columns [col0, col0 + R + Dr) of src -> the cache row of each row's (request, position):
    the first R over their root mean square times `weight`, the last Dr with their first
    `rot_dims` turned by the position (half-split pairs)."""
    _chk(src, "src"); _chk(pages, "pages", src.dtype); _chk(weight, "weight", torch.float32)
    _chk(block_table, "block_table", torch.int32)
    _lib.call("nf_latent_append", _p(src), c_int(src.shape[1]), c_int(col0), c_int(R), c_int(Dr), _p(weight),
              c_float(eps), _p(inv_freq), c_int(rot_dims if inv_freq is not None else 0), _p(ctx.positions),
              _p(ctx.row_seg), _p(pages), _p(block_table), c_int(block_table.shape[1]), c_int(page_size),
              c_int(pages.shape[0]), c_int(src.shape[0]), c_int(_dt(src)), _stream())


def rope_head_slices(q: torch.Tensor, heads: int, head_stride: int, off: int, rot_dims: int,
                     inv_freq: torch.Tensor, positions: torch.Tensor) -> None:
    """In place: the slice [off, off + rot_dims) of every head of q [T, heads * head_stride] is turned."""
    _chk(q, "q"); _chk(inv_freq, "inv_freq", torch.float32); _chk(positions, "positions", torch.int32)
    _lib.call("nf_rope_head_slices", _p(q), c_int(q.shape[1]), c_int(heads), c_int(head_stride), c_int(off),
              c_int(rot_dims), _p(inv_freq), _p(positions), c_int(q.shape[0]), c_int(_dt(q)), _stream())


def latent_attention(q_abs: torch.Tensor, q: torch.Tensor, head_stride: int, rot_off: int, Dr: int,
                     pages: torch.Tensor, block_table: torch.Tensor, page_size: int, ctx, sink: Optional[torch.Tensor],
                     scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of every head over the cached latent rows [c | k_rot]:
    score = (q_abs[h] . c + q_rot[h] . k_rot) * scale, softmax whose denominator also holds
    exp(sink[h]), result sum_j p_j c_j.  q_abs [heads, T, R]; q_rot is read from q [T, ld] at
    head * head_stride + rot_off.  Returns [heads, T, R]."""
    _chk(q_abs, "q_abs"); _chk(q, "q", q_abs.dtype); _chk(pages, "pages", q_abs.dtype)
    heads, T, R = q_abs.shape
    if sink is not None:
        _chk(sink, "sink", torch.float32)
    out = torch.empty((heads, T, R), dtype=q_abs.dtype, device=q_abs.device)
    if T == 0:
        return out
    if (q_abs.dtype == torch.bfloat16 and TUNING["bf16_attention"] != "generic" and window == 0
            and _lib.load().nf_latent_attention_mma_fits(c_int(R), c_int(Dr), c_int(head_stride), c_int(rot_off),
                                                        c_int(q.shape[1]))):
        # tensor cores: tiles of 32 (token, head) pairs, keys in blocks of 64, long contexts split
        per_row = (heads + LATENT_TILE_PAIRS - 1) // LATENT_TILE_PAIRS
        if getattr(ctx, "all_single", False) or getattr(ctx, "seg_len_host", None) is None:
            tiles, n_tiles = None, ctx.S * per_row          # one row a segment: the kernel numbers the tiles itself
        else:
            tiles, n_tiles = ctx.pair_tiles(heads, LATENT_TILE_PAIRS)
        n_blocks = max(1, (int(ctx.max_context) + LATENT_KEY_BLOCK - 1) // LATENT_KEY_BLOCK)
        nsplit = min(n_blocks, max(1, (LATENT_SPLIT_CTAS + n_tiles - 1) // n_tiles))
        per_split = (n_blocks + nsplit - 1) // nsplit
        nsplit = (n_blocks + per_split - 1) // per_split
        ws_o = torch.empty((T * heads, nsplit, R), dtype=torch.float32, device=q_abs.device)
        ws_ml = torch.empty((T * heads, nsplit, 2), dtype=torch.float32, device=q_abs.device)
        _lib.call("nf_latent_attention_mma", _p(q_abs), _p(q), c_int(q.shape[1]), c_int(head_stride), c_int(rot_off),
                  _p(pages), _p(block_table), c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.seg_row0),
                  _p(tiles), c_int(n_tiles), _p(sink), _p(out), _p(ws_o), _p(ws_ml), c_int(T), c_int(heads), c_int(R),
                  c_int(Dr), c_int(page_size), c_int(pages.shape[0]), c_float(scale), c_int(nsplit), c_int(per_split),
                  _stream())
        return out
    _lib.call("nf_latent_attention_generic", _p(q_abs), _p(q), c_int(q.shape[1]), c_int(head_stride), c_int(rot_off),
              _p(pages), _p(block_table), c_int(block_table.shape[1]), _p(ctx.positions), _p(ctx.row_seg), _p(sink),
              _p(out), c_int(T), c_int(heads), c_int(R), c_int(Dr), c_int(page_size), c_int(pages.shape[0]),
              c_int(window), c_float(scale), c_int(_dt(q_abs)), _stream())
    return out


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------

# ---------------------------------------------------------------------------------------
# several residual streams a token, the norm in groups
# ---------------------------------------------------------------------------------------

MAX_STREAMS = 8


def embed_copies(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, copies: int) -> None:
    """out[t, c] = float32(table[ids[t]]) for c < copies; out is [T, copies * hidden]."""
    _chk(table, "table"); _chk(ids, "ids", torch.int32); _chk(out, "out", torch.float32)
    _lib.call("nf_embed_copies", _p(table), _p(ids), _p(out), c_int(ids.numel()), c_int(table.shape[1]),
              c_int(table.shape[0]), c_int(copies), c_int(_dt(table)), _stream())


def streams_mix_norm(streams: torch.Tensor, S: int, y: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                     out_w: Optional[torch.Tensor], in_w: Optional[torch.Tensor], weight: Optional[torch.Tensor],
                     eps: float, groups: int, out_dtype: Optional[torch.dtype],
                     rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """What lies between two sublayers of a token with S residual streams (float32 [T, S * hidden]):

        x_t <- sum_s mix[s, t] x_s + out_w[t] * y     (if y is given; written back unless `rows`)
        u = sum_t in_w[t] x_t                         (in_w None: the plain sum)
        returns u / rms-in-groups(u) * weight         in `out_dtype` (None: only the update is applied)

    `mix` None is the identity, `out_w` None ones: with S = 1 that is the ordinary residual sum.  With
    `rows`, row r of the result belongs to token rows[r] and the streams are left as they are."""
    _chk(streams, "streams", torch.float32)
    T, SW = streams.shape
    hidden = SW // S
    for name, v in (("mix", mix), ("out_w", out_w), ("in_w", in_w), ("weight", weight)):
        if v is not None:
            _chk(v, name, torch.float32)
    R = T
    if rows is not None:
        _chk(rows, "rows", torch.int32)
        R = rows.numel()
    normed = None
    if out_dtype is not None:
        normed = torch.empty((R, hidden), dtype=out_dtype, device=streams.device)
    if y is not None:
        _chk(y, "y")
        if out_dtype is not None and y.dtype != out_dtype:
            raise TypeError("streams_mix_norm: y and the normed rows have one type")
    dt = _dt(normed) if normed is not None else (_dt(y) if y is not None else 0)
    _lib.call("nf_streams_mix_norm", _p(streams), _p(y), _p(rows), _p(mix), _p(out_w), _p(in_w), _p(weight),
              c_float(eps), c_int(groups), _p(normed), c_int(R), c_int(S), c_int(hidden),
              c_int(0 if rows is not None else 1), c_int(dt), _stream())
    return normed


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap), in place (float32)."""
    _chk(x, "x", torch.float32)
    _lib.call("nf_softcap", _p(x), c_longlong(x.numel()), c_float(cap), _stream())


# ---------------------------------------------------------------------------------------
# attention whose heads' scores are mixed, over chunks, with a sink
# ---------------------------------------------------------------------------------------

def head_norm_rope_append(proj: torch.Tensor, bias: Optional[torch.Tensor], q_norm: Optional[torch.Tensor],
                          k_norm: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot: int,
                          ctx, H: int, G: int, D: int, Dv: int, pages: Optional[torch.Tensor],
                          block_table: Optional[torch.Tensor], page_size: int, out_dtype: torch.dtype) -> torch.Tensor:
    """proj float32 [T, H*D | G*D | G*Dv] (+ bias): queries and keys normed per head (weights [D] shared
    by the heads) and turned over their first `rot` dimensions; returns the queries [T, H*D] in
    `out_dtype` and writes row [k | v] of every token into its page ([pages, page_size, G*(D+Dv)]).
    G = 0: the queries alone."""
    _chk(proj, "proj", torch.float32)
    T = proj.shape[0]
    q = torch.empty((T, H * D), dtype=out_dtype, device=proj.device)
    if G:
        _chk(pages, "pages", out_dtype)
    _lib.call("nf_head_norm_rope_append", _p(proj), c_int(proj.shape[1]), _p(bias), _p(q_norm), _p(k_norm),
              c_float(eps), _p(inv_freq), c_int(rot), _p(ctx.positions), _p(ctx.row_seg), _p(q),
              _p(pages) if G else None, _p(block_table) if G else None,
              c_int(block_table.shape[1] if G else 0), c_int(T), c_int(H), c_int(G), c_int(D), c_int(Dv),
              c_int(page_size), c_int(pages.shape[0] if G else 0), c_int(_dt(q)), _stream())
    return q


TALKING_KEY_BLOCK = 32      # keys a block of that kernel
TALKING_SPLIT_CTAS = 296    # steps of single rows: their keys are cut into runs until about this many CTAs run
TALKING_SPLIT_BLOCKS = 16   # ... without chunks, into runs of this many blocks; so are the keys of steps with few tiles
TALKING_MAX_RUNS = 16       # ... unless that made more runs than this
# ... and only while the tiles' CTAs are fewer than this (a prompt of 2,048 tokens at head size 128: 265 -> 205 us
# a layer with 128 CTAs, but 321 -> 390 us with 256, where the merge's traffic outweighs the better balance)
TALKING_FEW_CTAS = 148


def talking_attention(q: torch.Tensor, H: int, G: int, D: int, Dv: int, pages: torch.Tensor,
                      block_table: torch.Tensor, page_size: int, ctx, chunk: int, scale: float,
                      talk: Optional[torch.Tensor], sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H*D] against the paged rows [k | v] -> [T, H*Dv].  Scores of all heads of a (row, key)
    pair are mixed by `talk` [H, H] before the softmax; key j is seen from position i iff j <= i and,
    with `chunk` > 0, i // chunk == j // chunk; `sink` [H] adds exp(sink_h) to the denominator."""
    _chk(q, "q"); _chk(pages, "pages", q.dtype)
    T = q.shape[0]
    out = torch.empty((T, H * Dv), dtype=q.dtype, device=q.device)
    if T == 0:
        return out
    per_cta = 0
    single = getattr(ctx, "all_single", False) or getattr(ctx, "seg_len_host", None) is None
    if q.dtype == torch.bfloat16 and TUNING["bf16_attention"] != "generic":
        per_cta = _lib.load().nf_talking_attention_mma_heads_per_cta(c_int(H), c_int(G), c_int(D), c_int(Dv),
                                                                     c_int(1 if single else 0))
    if per_cta > 0:
        # tensor cores: tiles of 32 or 16 rows with all heads, the heads dealt out over a cluster's CTAs
        nsplit, per_split, ws_o, ws_ml = 1, 1, None, None
        if single:
            # one row a segment: the kernel numbers the tiles itself, and a row's keys (from its chunk's
            # start) are cut into runs so that the device is filled.  A run's length depends on the number
            # of rows and on the chunk, not on the step's longest context (which only bounds the number of
            # runs launched): a captured step, which knows a bound only, rounds as a host-driven one does.
            tiles, n_tiles = None, ctx.S
            block = TALKING_KEY_BLOCK
            want = max(1, TALKING_SPLIT_CTAS // (n_tiles * (H // per_cta)))
            if chunk > 0:
                chunk_blocks = (chunk + block - 1) // block + (1 if chunk % block else 0)
                per_split = max(2, (chunk_blocks + want - 1) // want)
            else:
                per_split = TALKING_SPLIT_BLOCKS
            span = max(1, min(chunk, int(ctx.max_context)) if chunk > 0 else int(ctx.max_context))
            n_blocks = (span + block - 1) // block + (1 if chunk % block else 0)
            nsplit = (n_blocks + per_split - 1) // per_split
            # partial sums and the merge also when one run is enough: the same arithmetic at every context
            ws_o = torch.empty((T * H, nsplit, Dv), dtype=torch.float32, device=q.device)
            ws_ml = torch.empty((T * H, nsplit, 2), dtype=torch.float32, device=q.device)
        else:
            tile_rows = _lib.load().nf_talking_attention_mma_tile_rows(c_int(H), c_int(G), c_int(D), c_int(Dv), c_int(0))
            tiles, n_tiles = ctx.chunked_query_tiles(tile_rows, chunk)
            # few tiles (fewer CTAs than SMs) with many key blocks each: the keys are cut
            # into runs of TALKING_SPLIT_BLOCKS blocks counted from position 0, so that the longest tile
            # does not set the time; the runs are merged as those of single rows are
            n_blocks = (int(ctx.max_context) + TALKING_KEY_BLOCK - 1) // TALKING_KEY_BLOCK
            runs = (n_blocks + TALKING_SPLIT_BLOCKS - 1) // TALKING_SPLIT_BLOCKS
            if n_tiles * (H // per_cta) < TALKING_FEW_CTAS and 2 <= runs <= TALKING_MAX_RUNS:
                nsplit, per_split = runs, TALKING_SPLIT_BLOCKS
                ws_o = torch.empty((T * H, nsplit, Dv), dtype=torch.float32, device=q.device)
                ws_ml = torch.empty((T * H, nsplit, 2), dtype=torch.float32, device=q.device)
        _lib.call("nf_talking_attention_mma", _p(q), _p(pages), _p(block_table), c_int(block_table.shape[1]),
                  _p(ctx.positions), _p(ctx.seg_row0), _p(tiles), c_int(n_tiles), _p(talk), _p(sink), _p(out),
                  _p(ws_o), _p(ws_ml), c_int(T), c_int(H), c_int(G), c_int(D), c_int(Dv), c_int(page_size),
                  c_int(pages.shape[0]), c_int(chunk), c_float(scale), c_int(nsplit), c_int(per_split), _stream())
        return out
    _lib.call("nf_talking_attention", _p(q), _p(pages), _p(block_table), c_int(block_table.shape[1]),
              _p(ctx.positions), _p(ctx.row_seg), None, _p(talk), _p(sink), _p(out), c_int(T), c_int(H), c_int(G),
              c_int(D), c_int(Dv), c_int(page_size), c_int(pages.shape[0]), c_int(chunk), c_float(scale),
              c_int(_dt(q)), _stream())
    return out


# ---------------------------------------------------------------------------------------
# feed-forwards without a gate
# ---------------------------------------------------------------------------------------

def poly_norm_act(z: torch.Tensor, coef: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """z float32 [T, n] -> coef[0] N(z) + coef[1] N(z^2) + coef[2] N(z^3) + coef[3], N = the row divided
    by its root mean square."""
    _chk(z, "z", torch.float32); _chk(coef, "coef", torch.float32)
    out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    _lib.call("nf_poly_norm_act", _p(z), _p(coef), c_float(eps), _p(out), c_int(z.shape[0]), c_int(z.shape[1]),
              c_int(_dt(out)), _stream())
    return out


def add_bias_rows(y: torch.Tensor, bias: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y float32 [T, n] + bias [n] -> `out_dtype`: the bias meets the projection's unrounded sums."""
    _chk(y, "y", torch.float32); _chk(bias, "bias", torch.float32)
    out = torch.empty(y.shape, dtype=out_dtype, device=y.device)
    _lib.call("nf_add_bias_rows", _p(y), _p(bias), _p(out), c_int(y.shape[0]), c_int(y.shape[1]), c_int(_dt(out)),
              _stream())
    return out


def gelu_erf_(x: torch.Tensor) -> torch.Tensor:
    """The exact GELU, in place."""
    _chk(x, "x")
    _lib.call("nf_gelu_erf", _p(x), c_longlong(x.numel()), c_int(_dt(x)), _stream())
    return x


def table_route(table: torch.Tensor, ids: torch.Tensor, E: int) -> torch.Tensor:
    """int32 [T, k]: row ids[t] of the experts' table [rows, k]."""
    _chk(table, "table", torch.int32); _chk(ids, "ids", torch.int32)
    T, k = ids.numel(), table.shape[1]
    idx = torch.empty((T, k), dtype=torch.int32, device=ids.device)
    _lib.call("nf_table_route", _p(table), _p(ids), _p(idx), c_int(T), c_int(k), c_int(table.shape[0]), c_int(E),
              _stream())
    return idx


def moe_rows_gemm(x: torch.Tensor, w, plan: "MoePlan", k: int, from_tokens: bool, gelu: bool = False) -> torch.Tensor:
    """One ungated product of the routed experts: sorted pair p of expert e -> x_p W_e^T.  With
    `from_tokens`, x is [T, K] and pair p reads token order[p] // k; otherwise x is [T*k, K] in
    sorted order.  `w` is [E, N, K] or its packed form.  `gelu`: the exact GELU of the result."""
    if not from_tokens:
        return moe_gemm2(x, w, plan, plan_is_older=True, gelu=gelu)
    _chk(x, "x")
    T, K = x.shape
    packed = isinstance(w, PackedWeights)
    if packed and T > TUNING["skinny_moe_max_tokens"]:
        return moe_gemm2(moe_gather(x, plan, k), w, plan, plan_is_older=True, gelu=gelu)
    if packed:
        E, N = w.groups, w.n_features
    else:
        _chk(w, "w", x.dtype)
        E, N, _ = w.shape
    out = torch.empty((T * k, N), dtype=x.dtype, device=x.device)
    if T == 0:
        return out
    if packed:
        _skinny(x, K, w.data, w.group_stride, out, T * k, N, K, E, T, plan.offsets, plan.order, k, False,
                packed=True, group_map=plan.active)
        return gelu_erf_(out) if gelu else out
    path = "simt" if x.dtype == torch.float32 else _bf16_path(T, K, "bf16_moe")
    if path == "skinny":
        _skinny(x, K, w, N * K, out, T * k, N, K, E, T, plan.offsets, plan.order, k, False, group_map=plan.active)
    else:
        _gemm_simt(x, K, w, N * K, out, T * k, N, K, E, T, plan.offsets, plan.order, k, False)
    return gelu_erf_(out) if gelu else out


SAMPLE_MAX_TOP_K = 1024


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """First maximum of each row of float32 logits [R, V] -> int32 [R]."""
    _chk(logits, "logits", torch.float32)
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    chunks = int(_lib.load().nf_argmax_chunks(c_int(R), c_int(V))) if R else 1
    if chunks > 1:
        # a long row is cut into pieces so that the whole device reads it
        sv = torch.empty((R, chunks), dtype=torch.float32, device=logits.device)
        si = torch.empty((R, chunks), dtype=torch.int32, device=logits.device)
        _lib.call("nf_argmax_rows_split", _p(logits), c_int(R), c_int(V), c_int(chunks), _p(sv), _p(si),
                  _p(out), _stream())
        return out
    _lib.call("nf_argmax_rows", _p(logits), c_int(R), c_int(V), _p(out), _stream())
    return out


def repetition_penalty(logits: torch.Tensor, ids: torch.Tensor, counts: torch.Tensor,
                       row_of: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: for pair i, logits[row_of[i], ids[i]] is divided (if positive) or multiplied
    (if not) by penalty[row] `counts[i]` times."""
    _chk(logits, "logits", torch.float32); _chk(ids, "ids", torch.int32)
    _chk(counts, "counts", torch.int32); _chk(row_of, "row_of", torch.int32)
    _chk(penalty, "penalty", torch.float32)
    _lib.call("nf_repetition_penalty", _p(logits), c_int(logits.shape[1]), _p(ids), _p(counts),
              _p(row_of), _p(penalty), c_int(ids.numel()), _stream())


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                top_p: torch.Tensor, draw: torch.Tensor) -> torch.Tensor:
    """One token per row from softmax(logits / temperature) limited by top-k and top-p,
    using the uniform draws `draw` in [0, 1).  The caller has checked the parameters."""
    _chk(logits, "logits", torch.float32); _chk(temperature, "temperature", torch.float32)
    _chk(top_k, "top_k", torch.int32); _chk(top_p, "top_p", torch.float32)
    _chk(draw, "draw", torch.float32)
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _lib.call("nf_sample_rows", _p(logits), c_int(R), c_int(V), _p(temperature), _p(top_k),
              _p(top_p), _p(draw), _p(out), _stream())
    return out
