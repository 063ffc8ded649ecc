"""Python faces of the CUDA kernels in ``hi_b200/csrc``.

Every function takes CUDA tensors, checks shapes and dtypes, and enqueues the kernel on
torch's current stream. There is no CPU path and no torch fallback: a tensor that is not
on a CUDA device, or a library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint64, c_void_p
from typing import Optional, Tuple

import torch

from . import build as _build

P, I, F = c_void_p, c_int, c_float

_SIGNATURES = {
    "hb_feed_tokens": [P, P, P, P, I, P],
    "hb_embed_gather": [P, I, P, P, I, I, I, P],
    "hb_add_rmsnorm": [P, P, I, P, P, P, I, P, I, P, I, P, P, I, I, F, P],
    "hb_swiglu": [P, P, I, I, I, P],
    "hb_moe_combine": [P, P, P, P, I, P, I, I, I, P],
    "hb_qkv_post": [P, I, P, I, I, I, F, I, F, F, P, P, P, I, P, P, P, I, I, I, I, I, I, P],
    "hb_paged_attention": [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P, P],
    "hb_attention_merge": [P, P, P, I, I, I, I, P],
    "hb_attention_decode": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P, P],
    "hb_attention_decode_tma": [P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P, P, P],
    "hb_attention_decode_fused": [P, P, I, I, I, F, I, F, F, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P, P, P, P],
    "hb_attention_prefill": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, I, P],
    "hb_attention_prefill_tc": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, P, P, P, P],
    "hb_router_topk": [P, I, P, I, I, I, I, I, I, P, P, P, P],
    "hb_moe_plan": [P, I, I, P, P, P, P, P],
    "hb_router_plan": [P, I, P, I, I, I, I, I, I, P, P, P, P, P, P, P, P, P],
    "hb_moe_gate_up": [P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, P],
    "hb_moe_down": [P, I, P, P, P, I, P, I, I, I, I, P],
    "hb_gather_rows": [P, P, I, P, I, I, P],
    "hb_moe_gate_up_tc": [P, P, P, P, P, I, P, P, I, I, I, P, P],
    "hb_moe_down_tc": [P, P, P, I, P, I, I, I, P, c_longlong, P, I, P, P],
    "hb_argmax_rows": [P, I, I, I, P, P, P, P, P],
    "hb_ranked_rows": [P, I, I, P, P, P, P, P, P],
    "hb_sample_rows": [P, I, I, P, P, P, P],
    "hb_sample_rows_parts": [P, I, I, I, P, P, P, P, P, P, P, P, P],
    "hb_random_normal": [P, I, c_longlong, c_longlong, c_uint64, F, P],
}

_UNSUPPORTED = 1002
_ERRORS = {1001: "bad argument (size, pointer or dtype)", 1002: "shape not supported by this kernel"}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        handle = _build.library()
        for name, sig in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = sig
            fn.restype = c_int
        handle.hb_moe_down_tc_scratch_floats.argtypes = [I]
        handle.hb_moe_down_tc_scratch_floats.restype = c_longlong
        _lib = handle
    return _lib


LAUNCHES = [0]     # kernels of this library enqueued so far (benchmarks report the difference)
CALLS: dict = {}   # ... and by entry point: which kernel family took the work (tests look here)


def _check(code: int, name: str) -> None:
    LAUNCHES[0] += 1
    CALLS[name] = CALLS.get(name, 0) + 1
    if code != 0:
        what = _ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{name}: {what}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# --------------------------------------------------------------------------- elementwise
def feed_tokens(tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor) -> None:
    """tokens[dst[i]] = sampled[src[i]], all int32 on the device: a step takes tokens that the step
    before it sampled without the host having read them."""
    for t, nm in ((tokens, "tokens"), (dst, "dst"), (src, "src"), (sampled, "sampled")):
        _need(t, nm, torch.int32)
    if dst.numel() != src.numel():
        raise KernelError("dst and src need the same number of entries")
    _check(lib().hb_feed_tokens(_ptr(tokens), _ptr(dst), _ptr(src), _ptr(sampled), dst.numel(), _stream()), "feed_tokens")


def embed_gather(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """Rows of ``table`` [V, H] for int32 ``tokens`` [N] -> float32 residual stream [N, H]."""
    _need(table, "table"); _need(tokens, "tokens", torch.int32)
    n, (vocab, hidden) = tokens.numel(), table.shape
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(lib().hb_embed_gather(_ptr(table), _dt(table), _ptr(tokens), _ptr(out), n, hidden, vocab, _stream()),
           "embed_gather")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                out_dtype: torch.dtype, row_map: Optional[torch.Tensor] = None, also_f32: bool = False,
                routed: Optional[torch.Tensor] = None, slot_of_entry: Optional[torch.Tensor] = None,
                top_k: int = 0, routed_weight: Optional[torch.Tensor] = None):
    """``x += delta`` (float32, in place) then ``rmsnorm(x) * weight`` in ``out_dtype``.

    ``routed`` (float32 [N*k, H], rows in expert-sorted order) with ``slot_of_entry`` adds each
    token's k routed-expert rows into the same sum: the experts' combine, fused into the norm;
    ``routed_weight`` (float32 [N*k], by entry) multiplies each of them first (a router score that
    scales the experts' outputs).

    ``also_f32`` returns ``(y, y_float32)``: the same normalised rows unrounded, for a consumer
    that computes in 32-bit (the router).

    With ``row_map`` (int32 [R]) only those rows are normalised (output [R, H]) and ``x`` is
    left untouched: the rows whose logits are wanted.
    """
    _need(x, "x", torch.float32)
    rows_total, hidden = x.shape
    if delta is not None:
        _need(delta, "delta")
        if delta.shape != x.shape:
            raise KernelError(f"delta shape {tuple(delta.shape)} != residual shape {tuple(x.shape)}")
    if weight is not None:
        _need(weight, "weight")
        if weight.numel() != hidden:
            raise KernelError(f"norm weight has {weight.numel()} elements for hidden size {hidden}")
    rows = rows_total
    if row_map is not None:
        _need(row_map, "row_map", torch.int32)
        rows = row_map.numel()
    y = torch.empty((rows, hidden), dtype=out_dtype, device=x.device)
    y32 = None
    if also_f32 and out_dtype != torch.float32:
        y32 = torch.empty((rows, hidden), dtype=torch.float32, device=x.device)
    if routed is not None:
        _need(routed, "routed", torch.float32); _need(slot_of_entry, "slot_of_entry", torch.int32)
        if routed.shape[1] != hidden or not 1 <= top_k <= 8:
            raise KernelError("routed rows do not match the residual, or top_k is outside 1..8")
        if routed_weight is not None:
            _need(routed_weight, "routed_weight", torch.float32)
            if routed_weight.numel() != slot_of_entry.numel():
                raise KernelError("routed_weight needs one factor per routing entry")
    _check(lib().hb_add_rmsnorm(_ptr(x), _ptr(delta), _dt(delta) if delta is not None else 0, _ptr(routed),
                                _ptr(slot_of_entry), _ptr(routed_weight) if routed is not None else None, int(top_k),
                                _ptr(weight),
                                _dt(weight) if weight is not None else 0, _ptr(y), _dt(y), _ptr(y32), _ptr(row_map),
                                rows, hidden, float(eps), _stream()), "add_rmsnorm")
    if also_f32:
        return y, (y if y32 is None else y32)
    return y


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """[N, 2I] (gate columns first) -> silu(gate) * up, [N, I], same dtype, float32 math."""
    _need(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("swiglu input needs an even number of columns")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().hb_swiglu(_ptr(gate_up), _ptr(out), _dt(gate_up), n, two_i // 2, _stream()), "swiglu")
    return out


def moe_combine(y: torch.Tensor, slot_of_entry: torch.Tensor, shared: Optional[torch.Tensor], n: int,
                top_k: int, routed_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = shared[t] + sum_j w[t*k + j] * y[slot_of_entry[t*k + j]]  -> float32 [n, H] (w = 1 without
    ``routed_weight``)."""
    _need(y, "y", torch.float32); _need(slot_of_entry, "slot_of_entry", torch.int32)
    hidden = y.shape[1]
    if shared is not None:
        _need(shared, "shared")
        if tuple(shared.shape) != (n, hidden):
            raise KernelError("shared expert output has the wrong shape")
    out = torch.empty((n, hidden), dtype=torch.float32, device=y.device)
    if routed_weight is not None:
        _need(routed_weight, "routed_weight", torch.float32)
    _check(lib().hb_moe_combine(_ptr(y), _ptr(slot_of_entry), _ptr(routed_weight), _ptr(shared),
                                _dt(shared) if shared is not None else 0,
                                _ptr(out), n, hidden, top_k, _stream()), "moe_combine")
    return out


def random_normal(out: torch.Tensor, key: int, scale: float, first: int = 0) -> torch.Tensor:
    """Fill ``out`` (float32 or bfloat16, contiguous) with the seeded values of elements
    ``first ..`` of the tensor with ``key``; ``scale`` = std / (sigma * 2**24) as float32
    (``hi_b200/weights/random_values.py`` computes the same bits on the host)."""
    _need(out, "out")
    _check(lib().hb_random_normal(_ptr(out), _dt(out), out.numel(), int(first), int(key), float(scale), _stream()),
           "random_normal")
    return out


# --------------------------------------------------------------------------- attention
def qkv_post(qkv: torch.Tensor, nh: int, nkv: int, hd: int, positions: torch.Tensor,
             inv_freq: Optional[torch.Tensor], interleaved: bool, qk_norm: bool, qk_eps: float,
             temperature: Optional[Tuple[float, float]], seq_of_token: Optional[torch.Tensor],
             block_table: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
             v_pages: Optional[torch.Tensor], page_size: int, write_kv: bool) -> torch.Tensor:
    """Rotary or temperature, optional L2 norm, and the cache append; returns q [N, nh, hd].

    ``qkv`` is [N, (nh + 2*nkv) * hd]; ``k_pages``/``v_pages`` are [pages, nkv, page_size, hd];
    ``block_table`` [S, width] int32 maps (sequence row, position // page_size) to a page.
    """
    _need(qkv, "qkv"); _need(positions, "positions", torch.int32)
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(nh + 2 * nkv) * hd}")
    if hd % 16 != 0 or hd > 256:
        raise KernelError(f"head_dim {hd} is not supported (multiples of 16 up to 256)")
    rot_pairs = _rot_pairs(inv_freq, hd)
    stride = 0
    if write_kv:
        for t, nm in ((seq_of_token, "seq_of_token"), (block_table, "block_table")):
            _need(t, nm, torch.int32)
        _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
        if tuple(k_pages.shape[1:]) != (nkv, page_size, hd) or k_pages.shape != v_pages.shape:
            raise KernelError(f"cache pages have shape {tuple(k_pages.shape)}, expected [*, {nkv}, {page_size}, {hd}]")
        stride = block_table.shape[1]
    q = torch.empty((n, nh, hd), dtype=qkv.dtype, device=qkv.device)
    fs, asc = temperature if temperature is not None else (1.0, 0.0)
    _check(lib().hb_qkv_post(_ptr(qkv), _dt(qkv), _ptr(inv_freq), rot_pairs, int(interleaved), int(qk_norm),
                             float(qk_eps), int(temperature is not None), float(fs), float(asc), _ptr(positions),
                             _ptr(seq_of_token), _ptr(block_table), stride, _ptr(q), _ptr(k_pages), _ptr(v_pages),
                             page_size, int(write_kv), n, nh, nkv, hd, _stream()), "qkv_post")
    return q


def _rot_pairs(inv_freq: Optional[torch.Tensor], hd: int) -> int:
    """How many pairs of a head rotate: the table's length; whole lanes of 8 pairs, at most head_dim / 2."""
    if inv_freq is None:
        return 0
    _need(inv_freq, "inv_freq", torch.float32)
    pairs = inv_freq.numel()
    if pairs % 8 or not 0 < 2 * pairs <= hd:
        raise KernelError(f"inv_freq has {pairs} entries: the rotated dims must be a multiple of 16, at most head_dim ({hd})")
    return pairs


ATTENTION_SPLIT = 256      # keys per split of the general attention kernel
DECODE_RESIDENT_BLOCKS = 148 * 3   # blocks of the decode kernel resident at a time


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                    seq_of_token: torch.Tensor, positions: torch.Tensor, chunk: int, window: int,
                    scale: float, max_context: int = 0) -> torch.Tensor:
    """softmax(q k^T * scale) v over the keys each token may read; q [N, nh, hd] -> [N, nh, hd].

    ``max_context`` (an upper bound of position + 1 over the tokens) lets long ranges be cut into
    splits of ``ATTENTION_SPLIT`` keys that run in parallel and are merged; a token's splits depend
    on its own range only. 0 = one pass per (token, head)."""
    _need(q, "q"); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if nh % nkv:
        raise KernelError(f"{nh} query heads are not a multiple of {nkv} kv heads")
    if hd % 16 != 0 or hd > 256:
        raise KernelError(f"head_dim {hd} is not supported (multiples of 16 up to 256)")
    out = torch.empty_like(q)
    longest = max_context
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    splits = max(1, -(-longest // ATTENTION_SPLIT))
    part_acc = part_ml = None
    if splits > 1:
        part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, splits, 2), dtype=torch.float32, device=q.device)
    _check(lib().hb_paged_attention(_ptr(q), _dt(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                    block_table.shape[1], _ptr(seq_of_token), _ptr(positions), _ptr(out), n, nh, nkv,
                                    hd, page_size, int(chunk), int(window), float(scale), ATTENTION_SPLIT, splits,
                                    _ptr(part_acc), _ptr(part_ml), _stream()),
           "paged_attention")
    return out


def _decode_splits(longest: int, groups: int) -> Tuple[int, int]:
    """How to cut ``longest`` keys for ``groups`` (token, kv head) pairs: the number of splits
    that minimises waves x (tiles per block + a block's fixed cost) + a cost per split (the
    merge) on 148 SMs x 3 resident blocks, none shorter than ATTENTION_SPLIT keys. Measured at
    8 requests x 8,192 keys: 6 splits (one wave of 384 blocks) 57 us, 13 splits (two waves) 63 us;
    one request x 32,768 keys: 32 splits 33 us, 47 splits 36 us.
    The cut moves results by rounding only."""
    best = (None, 1, longest)
    for s in range(1, max(1, -(-longest // ATTENTION_SPLIT)) + 1):
        size = -(-(-(-longest // s)) // 64) * 64
        real = -(-longest // size)
        waves = -(-(real * groups) // DECODE_RESIDENT_BLOCKS)
        cost = waves * (size // 64 + 1.5) + 0.2 * real + 0.3 * max(0, real - 32)   # past 32 the merge reads in turns
        if best[0] is None or cost < best[0]:
            best = (cost, real, size)
    return best[2], best[1]


def decode_attention_supported(q_dtype: torch.dtype, nh: int, nkv: int, hd: int) -> bool:
    """Shapes the tensor-core decode kernel takes; anything else goes to the general kernel."""
    return q_dtype == torch.bfloat16 and hd in (64, 128) and nh % nkv == 0 and nh // nkv <= 16


def decode_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                     seq_of_token: torch.Tensor, positions: torch.Tensor, chunk: int, window: int, scale: float,
                     max_context: int) -> torch.Tensor:
    """Attention for a batch of single decoded tokens (every row of ``q`` is one request's
    token), bfloat16, split over runs of ``ATTENTION_SPLIT`` keys. Uses scratch memory for the
    partial results of the splits."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if not decode_attention_supported(q.dtype, nh, nkv, hd):
        raise KernelError(f"decode attention does not take nh={nh} nkv={nkv} head_dim={hd}")
    longest = max(int(max_context), 1)
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    split_size, splits = _decode_splits(longest, n * nkv)
    out = torch.empty_like(q)
    part_acc = part_ml = None
    if splits > 1:
        part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, splits, 2), dtype=torch.float32, device=q.device)
    # tile loads by TMA where the range and the pages allow it (the kernel says if not)
    code = lib().hb_attention_decode_tma(_ptr(q), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(block_table),
                                         block_table.shape[1], _ptr(seq_of_token), _ptr(positions), _ptr(out), n, nh, nkv,
                                         hd, page_size, int(chunk), int(window), float(scale), split_size, splits,
                                         _ptr(part_acc), _ptr(part_ml), _ptr(_tc_status(q.device)), _stream())
    if code == _UNSUPPORTED:
        code = lib().hb_attention_decode(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                         _ptr(seq_of_token), _ptr(positions), _ptr(out), n, nh, nkv, hd, page_size,
                                         int(chunk), int(window), float(scale), split_size, splits, _ptr(part_acc),
                                         _ptr(part_ml), _stream())
        _check(code, "attention_decode")
    else:
        TC_USED[0] = True
        _check(code, "attention_decode_tma")
    if splits > 1:
        _check(lib().hb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), _dt(out), n * nh, hd, splits,
                                        _stream()), "attention_merge")
    return out


FUSED_COUNTERS = 1 << 18     # (token, kv head) pairs the fused decode kernel has counters for
# The fused kernel pays for what it saves in launches with work at the head and the tail of every
# block; once the blocks fill the machine several times over that shows. Measured at 8,192 keys, 8 kv
# heads: 2 / 8 / 16 requests 32.8 / 69.6 / 110.6 us against 38.9 / 76.7 / 117.8 us for the three
# kernels; 32 requests equal; 64 requests 364 against 352 us.
FUSED_MAX_GROUPS = 256       # (token, kv head) pairs up to which a decode step takes the fused kernel
_fused_counters: dict = {}   # device -> int32 zeros that the fused kernel leaves at zero


def _fused_counter_buffer(dev) -> torch.Tensor:
    key = (dev.type, dev.index)
    c = _fused_counters.get(key)
    if c is None:
        c = _fused_counters[key] = torch.zeros(FUSED_COUNTERS, dtype=torch.int32, device=dev)
    return c


def decode_attention_fused(qkv: torch.Tensor, nh: int, nkv: int, hd: int, positions: torch.Tensor,
                           inv_freq: Optional[torch.Tensor], interleaved: bool, qk_norm: bool, qk_eps: float,
                           temperature: Optional[Tuple[float, float]], seq_of_token: torch.Tensor,
                           block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, chunk: int,
                           window: int, scale: float, max_context: int, merge_inside: bool = True) -> Optional[torch.Tensor]:
    """:func:`qkv_post`, :func:`decode_attention` and the merge of its splits in ONE launch, for a step
    of single decoded tokens: ``qkv`` [N, (nh + 2 nkv) * hd] bfloat16 is the projection's output; the
    kernel encodes q, k and v, appends the token's key and value to its page, attends over the cache
    and combines the splits (the block that finishes last does it). Returns [N, nh, hd], or None
    where the kernel does not take the shapes (the caller then runs the three kernels)."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n = qkv.shape[0]
    n_pages, nkv2, page_size, hd2 = k_pages.shape
    if qkv.shape[1] != (nh + 2 * nkv) * hd or hd2 != hd or nkv2 != nkv or k_pages.shape != v_pages.shape:
        raise KernelError("qkv or the cache pages do not match the heads and head_dim")
    if not decode_attention_supported(qkv.dtype, nh, nkv, hd) or n * nkv > min(FUSED_COUNTERS, FUSED_MAX_GROUPS):
        return None
    rot_pairs = _rot_pairs(inv_freq, hd)
    longest = max(int(max_context), 1)
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    split_size, splits = _decode_splits(longest, n * nkv)
    out = torch.empty((n, nh, hd), dtype=qkv.dtype, device=qkv.device)
    part_acc = part_ml = None
    if splits > 1:
        part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n, nh, splits, 2), dtype=torch.float32, device=qkv.device)
    fs, asc = temperature if temperature is not None else (1.0, 0.0)
    code = lib().hb_attention_decode_fused(
        _ptr(qkv), _ptr(inv_freq), rot_pairs, int(interleaved), int(qk_norm), float(qk_eps), int(temperature is not None), float(fs),
        float(asc), _ptr(k_pages), _ptr(v_pages), n_pages, _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), _ptr(out), n, nh, nkv, hd, page_size, int(chunk), int(window), float(scale), split_size, splits,
        _ptr(part_acc), _ptr(part_ml), _ptr(_fused_counter_buffer(qkv.device)) if merge_inside else None,
        _ptr(_tc_status(qkv.device)), _stream())
    if code == _UNSUPPORTED:
        return None
    TC_USED[0] = True
    _check(code, "attention_decode_fused")
    if splits > 1 and not merge_inside:
        _check(lib().hb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), _dt(out), n * nh, hd, splits,
                                        _stream()), "attention_merge")
    return out


def prefill_attention_supported(q_dtype: torch.dtype, nh: int, nkv: int, hd: int) -> bool:
    """Shapes the tensor-core prefill kernel takes; anything else goes to the general kernel."""
    return q_dtype == torch.bfloat16 and hd in (64, 128) and nh % nkv == 0


def prefill_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, positions: torch.Tensor, n_seqs: int, max_new: int, chunk: int,
                      window: int, scale: float, skip_single: bool = False,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention for portions of prompts: request ``s`` owns rows ``cu_seqlens[s]..cu_seqlens[s+1]``
    of ``q`` [N, nh, hd], at consecutive positions; bfloat16, flash attention on tensor cores.
    ``skip_single`` leaves the rows of requests that bring one token unwritten (the caller runs
    the decode kernel for them and passes the same ``out``)."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if not prefill_attention_supported(q.dtype, nh, nkv, hd):
        raise KernelError(f"prefill attention does not take nh={nh} nkv={nkv} head_dim={hd}")
    if cu_seqlens.numel() != n_seqs + 1 or block_table.shape[0] < n_seqs:
        raise KernelError("cu_seqlens / block_table do not match the number of requests")
    if out is None:
        out = torch.empty_like(q)
    _check(lib().hb_attention_prefill(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                      _ptr(cu_seqlens), _ptr(positions), _ptr(out), n_seqs, int(max_new), nh, nkv, hd,
                                      page_size, int(chunk), int(window), float(scale), int(skip_single), _stream()),
           "attention_prefill")
    return out


PREFILL_TC_MIN_TOKENS = 128     # a request needs at least a tile of new tokens for the tcgen05 kernel to pay


def prefill_attention_tc_supported(q_dtype: torch.dtype, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    """Shapes the tcgen05 prefill kernel takes: bfloat16, head_dim 64 or 128, pages of 16, 32 or a
    multiple of 64 positions (a 64-key tile is loaded page by page with TMA)."""
    return q_dtype == torch.bfloat16 and hd in (64, 128) and nh % nkv == 0 and page_size % 16 == 0 and \
        (64 % page_size == 0 or page_size % 64 == 0)


def prefill_attention_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, positions: torch.Tensor, n_seqs: int, max_new: int, chunk: int,
                         window: int, scale: float, skip_single: bool = False,
                         out: Optional[torch.Tensor] = None, key_splits: int = 1) -> torch.Tensor:
    """As :func:`prefill_attention`, on tcgen05 (S, P V and O in tensor memory, TMA page loads).
    ``key_splits`` > 1: that many blocks share the key tiles of every (query tile, head) and a
    merge kernel combines their rows (see :func:`prefill_key_splits`)."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    n_pages, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if not prefill_attention_tc_supported(q.dtype, nh, nkv, hd, page_size):
        raise KernelError(f"tcgen05 prefill attention does not take nh={nh} nkv={nkv} head_dim={hd} page={page_size}")
    if cu_seqlens.numel() != n_seqs + 1 or block_table.shape[0] < n_seqs:
        raise KernelError("cu_seqlens / block_table do not match the number of requests")
    if out is None:
        out = torch.empty_like(q)
    key_splits = int(key_splits)
    part_acc = part_ml = None
    if key_splits > 1:
        part_acc = torch.empty((n * nh, key_splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * nh, key_splits, 2), dtype=torch.float32, device=q.device)
    _check(lib().hb_attention_prefill_tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                         block_table.shape[1], _ptr(cu_seqlens), _ptr(positions), _ptr(out), n, n_pages,
                                         n_seqs, int(max_new), nh, nkv, hd, page_size, int(chunk), int(window),
                                         float(scale), int(skip_single), key_splits, _ptr(part_acc) if part_acc is not None else None,
                                         _ptr(part_ml) if part_ml is not None else None, _ptr(_tc_status(q.device)),
                                         _stream()),
           "attention_prefill_tc")
    TC_USED[0] = True
    if key_splits > 1:
        _check(lib().hb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), _dt(out), n * nh, hd, key_splits,
                                        _stream()), "attention_merge")
    return out


_sm_counts: dict = {}


def sm_count(device) -> int:
    key = torch.device(device)
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_counts[key]


PREFILL_RESIDENT_BLOCKS_PER_SM = 2     # of the tcgen05 prefill kernel (tensor memory: 256 of 512 columns each)
PREFILL_SPLIT_MIN_TILES = 512          # key tiles (of 64 keys) a block must have before its keys are shared out
PREFILL_SPLIT_MIN_SHARE = 128          # and the fewest a share may get


def prefill_key_splits(blocks: int, key_tiles: int, sms: int) -> int:
    """How many blocks should share the key tiles of each (query tile, head) of the tcgen05 prefill
    kernel, when the ``blocks`` of a launch all have about ``key_tiles`` key tiles (a short portion
    far into a long context). The kernel runs two blocks per SM; with fewer blocks than that, or a
    few more, most of the GPU waits for the last ones. Measured at 65,000 cached tokens, 40 heads:
    128 new tokens 933 -> 256 us in six shares, 256 tokens 935 -> 448 us in three, 512 tokens
    1,116 -> 795 us in five, 1,024 tokens 2,163 -> 1,521 us in four; nothing gained at 16,000
    cached tokens, and a loss from 2,048 new tokens on (4,096: 5.09 -> 5.88 ms in three: the
    unnormalised rows written out and merged cost more than the fuller last round gains).
    So: only launches of up to 1.25 rounds with at least 512 key tiles; the number of shares (up to
    8, at least 128 tiles each) that fills the rounds best, the fewest among those within 0.05."""
    places = PREFILL_RESIDENT_BLOCKS_PER_SM * max(int(sms), 1)
    if blocks <= 0 or blocks > 1.25 * places or key_tiles < PREFILL_SPLIT_MIN_TILES:
        return 1
    fill = {k: (blocks * k / places) / -(-blocks * k // places) for k in range(1, 9)
            if k == 1 or key_tiles // k >= PREFILL_SPLIT_MIN_SHARE}
    best = max(fill.values())
    choice = min(k for k, f in fill.items() if f >= best - 0.05)
    return choice if fill[choice] > fill[1] else 1


# --------------------------------------------------------------------------- experts
ROUTER_SOFTMAX, ROUTER_RENORMALIZE = 1, 2     # bits of a router's ``mode``


def router_topk(x: torch.Tensor, w: torch.Tensor, top_k: int, want_logits: bool = False, mode: int = 0):
    """Router logits (float32), the top-k expert ids (ties to the lower id) and their scores: the
    sigmoid of the chosen logit, or with ``ROUTER_SOFTMAX`` its softmax over all experts; with
    ``ROUTER_RENORMALIZE`` divided by the sum of the chosen scores."""
    _need(x, "x"); _need(w, "router weight")
    n, hidden = x.shape
    experts = w.shape[0]
    if w.shape[1] != hidden:
        raise KernelError("router weight does not match the hidden size")
    ids = torch.empty((n, top_k), dtype=torch.int32, device=x.device)
    scores = torch.empty((n, top_k), dtype=torch.float32, device=x.device)
    logits = torch.empty((n, experts), dtype=torch.float32, device=x.device)   # the blocks' meeting place
    _check(lib().hb_router_topk(_ptr(x), _dt(x), _ptr(w), _dt(w), n, hidden, experts, top_k, int(mode), _ptr(logits),
                                _ptr(ids), _ptr(scores), _stream()), "router_topk")
    return ids, scores, logits if want_logits else None


class MoePlan:
    """Rows grouped by expert: ``offsets`` [E+1], ``sorted_entry`` [n] (entry of each sorted slot),
    ``slot_of_entry`` [n], ``active`` [E+1] (count, then the ids of the experts that have rows)."""

    __slots__ = ("offsets", "sorted_entry", "slot_of_entry", "active")

    def __init__(self, offsets, sorted_entry, slot_of_entry, active):
        self.offsets, self.sorted_entry, self.slot_of_entry, self.active = offsets, sorted_entry, slot_of_entry, active

    def __iter__(self):       # (offsets, sorted_entry, slot_of_entry) for callers that unpack
        return iter((self.offsets, self.sorted_entry, self.slot_of_entry))


def _empty_plan(n: int, experts: int, dev) -> MoePlan:
    return MoePlan(torch.empty(experts + 1, dtype=torch.int32, device=dev),
                   torch.empty(max(n, 1), dtype=torch.int32, device=dev),
                   torch.empty(max(n, 1), dtype=torch.int32, device=dev),
                   torch.empty(experts + 1, dtype=torch.int32, device=dev))


_block_counters: dict = {}     # device -> one int32 that kernels leave at zero; launches that share it must
                               # follow one another (the engine runs its steps on one stream)


def _block_counter(dev) -> torch.Tensor:
    c = _block_counters.get(dev)
    if c is None:
        c = _block_counters[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    return c


def router_plan(x: torch.Tensor, w: torch.Tensor, top_k: int, mode: int = 0):
    """:func:`router_topk` and :func:`moe_plan` in one call: with few tokens one kernel does both
    (the block that ends last groups the entries). Returns ids, scores and the plan."""
    _need(x, "x"); _need(w, "router weight")
    n, hidden = x.shape
    experts = w.shape[0]
    if w.shape[1] != hidden:
        raise KernelError("router weight does not match the hidden size")
    ids = torch.empty((n, top_k), dtype=torch.int32, device=x.device)
    scores = torch.empty((n, top_k), dtype=torch.float32, device=x.device)
    logits = torch.empty((n, experts), dtype=torch.float32, device=x.device)   # the blocks' meeting place
    plan = _empty_plan(n * top_k, experts, x.device)
    _check(lib().hb_router_plan(_ptr(x), _dt(x), _ptr(w), _dt(w), n, hidden, experts, top_k, int(mode), _ptr(logits),
                                _ptr(ids), _ptr(scores), _ptr(plan.offsets), _ptr(plan.sorted_entry),
                                _ptr(plan.slot_of_entry), _ptr(plan.active), _ptr(_block_counter(x.device)),
                                _stream()), "router_plan")
    return ids, scores, plan


def moe_plan(ids: torch.Tensor, experts: int) -> MoePlan:
    """Group the routing entries by expert, on the device."""
    _need(ids, "ids", torch.int32)
    n = ids.numel()
    plan = _empty_plan(n, experts, ids.device)
    _check(lib().hb_moe_plan(_ptr(ids), n, experts, _ptr(plan.offsets), _ptr(plan.sorted_entry),
                             _ptr(plan.slot_of_entry), _ptr(plan.active), _stream()), "moe_plan")
    return plan


def moe_gate_up(x: torch.Tensor, plan: MoePlan, top_k: int, w_gate: torch.Tensor,
                w_up: torch.Tensor, scores: torch.Tensor, few_rows: bool) -> torch.Tensor:
    """act[slot] = silu(s * x Wg[e]^T) * (s * x Wu[e]^T), [N*k, I] in the engine dtype."""
    _need(x, "x"); _need(w_gate, "w_gate", x.dtype); _need(w_up, "w_up", x.dtype)
    _need(scores, "scores", torch.float32)
    n, hidden = x.shape
    experts, inter, h2 = w_gate.shape
    if h2 != hidden or w_up.shape != w_gate.shape:
        raise KernelError("expert gate/up weights do not match the hidden size")
    n_entries = n * top_k
    act = torch.empty((n_entries, inter), dtype=x.dtype, device=x.device)
    _check(lib().hb_moe_gate_up(_ptr(x), _dt(x), _ptr(plan.sorted_entry), top_k, _ptr(w_gate), _ptr(w_up),
                                _ptr(plan.offsets), _ptr(plan.active), experts, _ptr(scores), _ptr(act), n_entries,
                                inter, hidden, int(few_rows), _stream()), "moe_gate_up")
    return act


def moe_down(act: torch.Tensor, w_down: torch.Tensor, plan: MoePlan, few_rows: bool) -> torch.Tensor:
    """y[slot] = act[slot] Wd[e]^T, float32 [N*k, H]."""
    _need(act, "act"); _need(w_down, "w_down", act.dtype)
    n_entries, inter = act.shape
    experts, hidden, i2 = w_down.shape
    if i2 != inter:
        raise KernelError("expert down weights do not match the intermediate size")
    y = torch.empty((n_entries, hidden), dtype=torch.float32, device=act.device)
    _check(lib().hb_moe_down(_ptr(act), _dt(act), _ptr(w_down), _ptr(plan.offsets), _ptr(plan.active), experts,
                             _ptr(y), n_entries, hidden, inter, int(few_rows), _stream()), "moe_down")
    return y


# --------------------------------------------------------------------------- experts on tcgen05
_TC_STATUS = {}          # device -> int32[1]: nonzero after a tensor-core kernel gave up a bounded wait
TC_USED = [False]


def _tc_status(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


def check_tc_status(device=None) -> None:
    """Raise if a kernel with bounded mbarrier waits (the tcgen05 products and attention, the TMA
    decode attention) timed out on one of its barriers since the last check
    (synchronises; skipped while a stream is being captured)."""
    TC_USED[0] = False
    if torch.cuda.is_current_stream_capturing():
        return
    for key, st in _TC_STATUS.items():
        code = int(st.item())
        if code != 0:
            st.zero_()
            for buffers in (_down_scratch_buffers.get(key),):       # a kernel that gave up may have left a count behind
                if buffers is not None:
                    buffers[1].zero_()
            where = {1: "grouped product: the TMA producer waiting for a free stage",
                     2: "grouped product: the MMA issuer waiting for a loaded stage",
                     3: "grouped product: the epilogue waiting for the accumulator",
                     4: "grouped product: the MMA issuer waiting for a free accumulator",
                     31: "decode attention: the warps waiting for a tile's TMA loads"}.get(
                code, f"prefill attention, wait {code}" if code >= 11 else f"code {code}")
            raise KernelError(f"a kernel gave up a bounded wait ({where}); its output is invalid")


class PendingStatus:
    """The status word copied to pinned memory behind the step's kernels; read it later."""

    def __init__(self, device: torch.device):
        self.host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self.event = torch.cuda.Event()
        self.device = device
        self.pending = False
        self.claimed = False         # someone other than the engine has taken it and will resolve it

    def enqueue(self) -> None:
        self.host.copy_(_tc_status(self.device), non_blocking=True)
        self.event.record()
        self.pending = True

    def resolve(self, wait: bool = True) -> bool:
        """Read the copied word; raises if a kernel reported a failed wait. With ``wait=False`` it
        returns False, without blocking, while the copy has not run yet (the word on the device
        stays set until it is read, so a later look still sees it)."""
        if not self.pending:
            return True
        if not wait and not self.event.query():
            return False
        self.event.synchronize()
        self.pending = False
        if int(self.host[0]) != 0:
            check_tc_status()          # raises with the reason, and clears the word
        return True


def moe_tc_supported(x: torch.Tensor, w_gate: torch.Tensor) -> bool:
    """The tensor-core expert kernels take bfloat16 with hidden and intermediate sizes that are
    multiples of 8 (TMA needs 16-byte row strides)."""
    return x.dtype == torch.bfloat16 and w_gate.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and \
        w_gate.shape[1] % 8 == 0


def moe_gate_up_tc(x: torch.Tensor, plan: MoePlan, top_k: int, w_gate: torch.Tensor, w_up: torch.Tensor,
                   scores: torch.Tensor) -> torch.Tensor:
    """As :func:`moe_gate_up`, on tcgen05: gathers the rows into expert order, then one grouped
    product with the SwiGLU epilogue."""
    _need(x, "x", torch.bfloat16); _need(w_gate, "w_gate", torch.bfloat16); _need(w_up, "w_up", torch.bfloat16)
    _need(scores, "scores", torch.float32)
    n, hidden = x.shape
    experts, inter, h2 = w_gate.shape
    if h2 != hidden or w_up.shape != w_gate.shape:
        raise KernelError("expert gate/up weights do not match the hidden size")
    rows = n * top_k
    xs = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    _check(lib().hb_gather_rows(_ptr(x), _ptr(plan.sorted_entry), top_k, _ptr(xs), rows, hidden, _stream()),
           "gather_rows")
    act = torch.empty((rows, inter), dtype=x.dtype, device=x.device)
    _check(lib().hb_moe_gate_up_tc(_ptr(xs), _ptr(plan.sorted_entry), _ptr(w_gate), _ptr(w_up), _ptr(plan.offsets),
                                   experts, _ptr(scores), _ptr(act), rows, inter, hidden, _ptr(_tc_status(x.device)),
                                   _stream()), "moe_gate_up_tc")
    TC_USED[0] = True
    return act


_down_scratch_buffers: dict = {}   # device -> (partial tiles of a cut last round, their counters, left at zero)


def _down_scratch(dev):
    key = (dev.type, dev.index)
    b = _down_scratch_buffers.get(key)
    if b is None:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        b = _down_scratch_buffers[key] = (
            torch.empty(int(lib().hb_moe_down_tc_scratch_floats(sms)), dtype=torch.float32, device=dev),
            torch.zeros(sms, dtype=torch.int32, device=dev))
    return b


def moe_down_tc(act: torch.Tensor, w_down: torch.Tensor, plan: MoePlan) -> torch.Tensor:
    """As :func:`moe_down`, on tcgen05."""
    _need(act, "act", torch.bfloat16); _need(w_down, "w_down", torch.bfloat16)
    rows, inter = act.shape
    experts, hidden, i2 = w_down.shape
    if i2 != inter:
        raise KernelError("expert down weights do not match the intermediate size")
    y = torch.empty((rows, hidden), dtype=torch.float32, device=act.device)
    scratch, counters = _down_scratch(act.device)
    _check(lib().hb_moe_down_tc(_ptr(act), _ptr(w_down), _ptr(plan.offsets), experts, _ptr(y), rows, hidden, inter,
                                _ptr(scratch), scratch.numel(), _ptr(counters), counters.numel(),
                                _ptr(_tc_status(act.device)), _stream()), "moe_down_tc")
    TC_USED[0] = True
    return y


# --------------------------------------------------------------------------- sampling
ARGMAX_PARTS = 16            # blocks per row of the all-greedy sampler
ARGMAX_MAX_ROWS = 1024
ARGMAX_MIN_VOCAB = 8192
SAMPLE_PARTS = 16            # blocks per row of the sampler with temperatures, for steps of few rows
SAMPLE_PARTS_MAX_BLOCKS = 2048   # beyond 128 rows a block per row keeps the GPU as busy
_argmax_scratch: dict = {}   # device -> (values, ids, counters); shared by launches that follow one another


def _argmax_buffers(dev):
    b = _argmax_scratch.get(dev)
    if b is None:
        b = _argmax_scratch[dev] = (torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.float32, device=dev),
                                    torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.int32, device=dev),
                                    torch.zeros(ARGMAX_MAX_ROWS, dtype=torch.int32, device=dev),
                                    torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.float32, device=dev),
                                    torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.float32, device=dev))
    return b


def sample_rows(logits: torch.Tensor, temperatures: Optional[torch.Tensor],
                uniforms: Optional[torch.Tensor]) -> torch.Tensor:
    """One token per row of float32 logits: argmax where temperature <= 0, else inverse CDF.
    Without temperatures (every row greedy) a few rows of a large vocabulary are cut over
    ``ARGMAX_PARTS`` blocks each."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if temperatures is None and rows <= ARGMAX_MAX_ROWS and vocab >= ARGMAX_MIN_VOCAB:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        vals, ids, counters = _argmax_buffers(logits.device)[:3]
        _check(lib().hb_argmax_rows(_ptr(logits), rows, vocab, ARGMAX_PARTS, _ptr(vals), _ptr(ids), _ptr(counters),
                                    _ptr(out), _stream()), "argmax_rows")
        return out
    for t, nm in ((temperatures, "temperatures"), (uniforms, "uniforms")):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != rows:
                raise KernelError(f"{nm} needs one entry per row")
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if rows * SAMPLE_PARTS <= SAMPLE_PARTS_MAX_BLOCKS and vocab >= ARGMAX_MIN_VOCAB:
        # a few rows of a large vocabulary: every row over SAMPLE_PARTS blocks, the last of them picks
        vals, ids, counters, maxima, sums = _argmax_buffers(logits.device)
        _check(lib().hb_sample_rows_parts(_ptr(logits), rows, vocab, SAMPLE_PARTS, _ptr(temperatures), _ptr(uniforms),
                                          _ptr(vals), _ptr(ids), _ptr(maxima), _ptr(sums), _ptr(counters), _ptr(out),
                                          _stream()), "sample_rows_parts")
        return out
    _check(lib().hb_sample_rows(_ptr(logits), rows, vocab, _ptr(temperatures), _ptr(uniforms), _ptr(out), _stream()),
           "sample_rows")
    return out


def ranked_rows(logits: torch.Tensor, temperatures: torch.Tensor, top_ps: torch.Tensor, top_ks: torch.Tensor,
                uniforms: torch.Tensor, out: torch.Tensor) -> None:
    """Top-k / top-p rows of float32 logits, sampled in place into ``out`` (int32 [R]) by the host
    sampler's rule; rows without a temperature, or with neither a top-k below the vocabulary nor a
    top-p inside (0, 1), are left as they are. ``out[r] == -1`` afterwards: the row has more than
    4,096 candidates or logits that are not finite, and has to be ranked on the host."""
    _need(logits, "logits", torch.float32)
    rows = logits.shape[0]
    for t, nm, dt in ((temperatures, "temperatures", torch.float32), (top_ps, "top_ps", torch.float32),
                      (top_ks, "top_ks", torch.int32), (uniforms, "uniforms", torch.float32), (out, "out", torch.int32)):
        _need(t, nm, dt)
        if t.numel() != rows:
            raise KernelError(f"{nm} needs one entry per row")
    _check(lib().hb_ranked_rows(_ptr(logits), rows, logits.shape[1], _ptr(temperatures), _ptr(top_ps), _ptr(top_ks),
                                _ptr(uniforms), _ptr(out), _stream()), "ranked_rows")
