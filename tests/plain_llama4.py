"""Plain, slow Llama 4 text decoder: whole sequences, no cache, float32 on the CPU.

This file is the oracle of the test-suite. It shares no code with ``hi_b200``: it reads
``config.json`` as a plain dict and takes the weights as a ``{name: tensor}`` dict.

It rests on the reference's FORMULAS, not on its outputs: the reference's Llama 4 model
(``Llama4Like``, crates/hi-mlx/src/models.rs:5893-6230) sits behind
``cfg(all(target_os = "macos", target_arch = "aarch64", feature = "mlx"))``
(models.rs:294-295) and calls Apple MLX/Metal ops, and no Rust toolchain is installed,
so it can neither be imported nor compiled here; ``tests/golden/`` therefore holds
outputs of THIS file (with the script that made them) that pin it against later edits.
Where the reference has no formula (chunked attention, attention temperature, dense
layers, top-k > 1, NoPE interval) the function says so.

Every function takes one sequence; positions are 0..T-1.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F32 = torch.float32


class precision:
    """``with precision(torch.float64):`` runs the functions below in another float type; tests
    use it to measure how much of a difference is the oracle's own rounding."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global F32
        self.saved, F32 = F32, self.dtype

    def __exit__(self, *exc):
        global F32
        F32 = self.saved


# --------------------------------------------------------------------------- config
def layer_uses_rope(cfg: dict, i: int) -> bool:
    """models.rs:5953-5954 fixes NoPE to every 4th layer; the interval is a config key here.
    An explicit ``no_rope_layers`` list (1 = rotary, 0 = NoPE; config.rs:76-77,411) wins."""
    lst = cfg.get("no_rope_layers")
    if isinstance(lst, list) and lst:
        return bool(lst[i])
    interval = cfg.get("nope_layer_interval", 4)
    return not (interval > 0 and (i + 1) % interval == 0)


def layer_is_moe(cfg: dict, i: int) -> bool:
    """models.rs:6105-6110 makes every layer MoE (Scout); ``interleave_moe_layer_step`` /
    ``moe_layers`` are read here for models that interleave dense layers."""
    lst = cfg.get("moe_layers")
    if isinstance(lst, list) and lst:
        return i in lst
    step = cfg.get("interleave_moe_layer_step", 1)
    return step > 0 and (i + 1) % step == 0


def text_config(raw: dict) -> dict:
    """config.rs:311-326: text_config keys are hoisted without clobbering the top level.
    Sizes are taken from text_config when it exists."""
    if isinstance(raw.get("text_config"), dict):
        merged = dict(raw)
        merged.update(raw["text_config"])
        return merged
    return raw


# --------------------------------------------------------------------------- parts
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w  (models.rs:1977-1979; explicit formula in
    crates/hi-cuda/src/kernels.cu:61-77). ``weight=None`` is the weightless form used
    for q and k (models.rs:6017-6021)."""
    x = x.to(F32)
    y = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight.to(F32)


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """Per-pair inverse frequency, float32 (models.rs:5897-5926 with scaling,
    models.rs:6166-6175 without). The reference divides by zero when
    high_freq_factor == low_freq_factor and the wavelength equals the boundary exactly;
    that one point is given the low-frequency value (smooth = 0)."""
    half = head_dim // 2
    out = []
    base = torch.tensor(theta, dtype=F32)
    for j in range(half):
        th = torch.pow(base, torch.tensor((2 * j) / head_dim, dtype=F32))
        inv = (1.0 / th).to(F32)
        if scaling:
            factor = float(scaling.get("factor", 8.0))
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192.0))
            wavelen = 2.0 * math.pi / float(inv)
            if wavelen > orig / low:
                inv = inv / factor
            elif wavelen < orig / high:
                pass
            else:
                smooth = 0.0 if high == low else (orig / wavelen - low) / (high - low)
                inv = (1.0 - smooth) * inv / factor + smooth * inv
        out.append(float(inv))
    return torch.tensor(out, dtype=F32)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """Rotate all head_dim dims of x [T, heads, hd] (models.rs:5997-6016, traditional=false:
    pairs (j, j+hd/2); the explicit formula with both pairings is
    crates/hi-cuda/src/kernels.cu:3757-3785)."""
    x = x.to(F32)
    T, _, hd = x.shape
    ang = positions.to(F32)[:, None] * inv_freq[None, :]          # [T, hd/2], float32 product
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
    else:
        a, b = x[..., : hd // 2], x[..., hd // 2:]
    ra, rb = a * cos - b * sin, b * cos + a * sin
    out = torch.empty_like(x)
    if interleaved:
        out[..., 0::2], out[..., 1::2] = ra, rb
    else:
        out[..., : hd // 2], out[..., hd // 2:] = ra, rb
    return out


def attention_temperature(q: torch.Tensor, positions: torch.Tensor, floor_scale: float, attn_scale: float) -> torch.Tensor:
    """q * (1 + attn_scale * ln(1 + floor((pos + 1) / floor_scale))) on NoPE layers.
    No counterpart in the reference (no reader of these keys under crates/)."""
    f = torch.log(torch.floor((positions.to(F32) + 1.0) / floor_scale) + 1.0) * attn_scale + 1.0
    return q.to(F32) * f[:, None, None]


def visibility(T: int, chunk: Optional[int]) -> torch.Tensor:
    """[T, T] bool: key <= query (models.rs:11165-11184), and on chunked layers the key lies
    in the query's block of ``chunk`` positions (not in the reference)."""
    q = torch.arange(T)[:, None]
    k = torch.arange(T)[None, :]
    vis = k <= q
    if chunk:
        vis = vis & ((k // chunk) == (q // chunk))
    return vis


def attention_core(q, k, v, chunk: Optional[int]) -> torch.Tensor:
    """softmax(q k^T * hd^-0.5 + mask) v with grouped heads: q head h reads kv head
    h // (nh / nkv) (models.rs:5963, 6024-6050; mapping crates/hi-cuda/src/kernels.cu:12413-12414).
    q [T, nh, hd]; k, v [T, nkv, hd] -> [T, nh*hd]."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    vis = visibility(T, chunk)
    out = torch.empty(T, nh, hd, dtype=F32)
    for h in range(nh):
        s = (q[:, h, :].to(F32) @ k[:, h // g, :].to(F32).T) * (hd ** -0.5)
        s = s.masked_fill(~vis, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, h // g, :].to(F32)
    return out.reshape(T, nh * hd)


def linear(w: Dict[str, torch.Tensor], prefix: str, x: torch.Tensor) -> torch.Tensor:
    """x W^T, plus the bias iff a ``.bias`` tensor exists (Linear::load / forward,
    models.rs:1808, 1843-1847)."""
    y = x @ w[f"{prefix}.weight"].to(F32).T
    bias = w.get(f"{prefix}.bias")
    return y if bias is None else y + bias.to(F32)


def attention(cfg: dict, w: Dict[str, torch.Tensor], prefix: str, i: int, x: torch.Tensor, inv_freq,
              first_position: int = 0) -> torch.Tensor:
    """Llama4Attention::forward (models.rs:5978-6052) plus the chunk rule and temperature.
    ``first_position``: the sequence's positions are first_position .. (tests of what a layer does
    and does not take from absolute positions; the sequence must then stay within one chunk)."""
    T = x.shape[0]
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    pos = torch.arange(T) + first_position
    q = linear(w, f"{prefix}.q_proj", x).reshape(T, nh, hd)
    k = linear(w, f"{prefix}.k_proj", x).reshape(T, nkv, hd)
    v = linear(w, f"{prefix}.v_proj", x).reshape(T, nkv, hd)
    use_rope = layer_uses_rope(cfg, i)
    if use_rope:
        inter = bool(cfg.get("rope_interleaved", False))
        q, k = apply_rope(q, pos, inv_freq, inter), apply_rope(k, pos, inv_freq, inter)
        if cfg.get("use_qk_norm", False):
            eps = cfg.get("qk_norm_eps", 1e-6)            # fixed 1e-6 in models.rs:6019-6020
            q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    elif cfg.get("attn_temperature_tuning", False):
        q = attention_temperature(q, pos, float(cfg.get("floor_scale", 8192)), float(cfg.get("attn_scale", 0.1)))
    chunk = cfg.get("attention_chunk_size", 8192) if use_rope else None
    o = attention_core(q, k, v, chunk)
    return linear(w, f"{prefix}.o_proj", o)


def swiglu(x, wg, wu, wd) -> torch.Tensor:
    """(silu(x Wg^T) * x Wu^T) Wd^T  (Mlp::forward, models.rs:2307-2312)."""
    g, u = x @ wg.to(F32).T, x @ wu.to(F32).T
    return (g * torch.sigmoid(g) * u) @ wd.to(F32).T


def router_top_k(logits: torch.Tensor, k: int):
    """The k largest router logits per token; on equal logits the lower expert id wins
    (crates/hi-cuda/src/kernels.cu:578-580). The reference's host loop is top-1
    (models.rs:6088-6089). Score = sigmoid of the chosen logit, no renormalisation
    (models.rs:6090)."""
    T, E = logits.shape
    ids = torch.empty(T, k, dtype=torch.long)
    for t in range(T):
        row = logits[t].tolist()
        order = sorted(range(E), key=lambda e: (-row[e], e))
        ids[t] = torch.tensor(order[:k])
    chosen = torch.gather(logits, 1, ids)
    return ids, 1.0 / (1.0 + torch.exp(-chosen))


def moe_feed_forward(cfg: dict, w, prefix: str, x: torch.Tensor, forced_ids=None, record=None) -> torch.Tensor:
    """Llama4Moe::forward (models.rs:6055-6103): the score scales the expert INPUT; the
    shared expert sees the unscaled input; outputs are summed.

    ``forced_ids`` [T, k] replaces the top-k choice (scores still come from this function's own
    logits): a reduced-precision engine may pick another expert where two logits are nearly
    equal, and its logits are then compared given ITS choice. ``record(prefix, ids, margin)``
    receives this function's own choice and the gap between the k-th and (k+1)-th logit as a
    fraction of the root mean square of the sequence's router logits in this layer (the size of
    the numbers a rounding error of the input is proportional to)."""
    T, H = x.shape
    k = cfg.get("num_experts_per_tok", 1)
    logits = x @ w[f"{prefix}.router.weight"].to(F32).T
    ids, scores = router_top_k(logits, k)
    if record is not None:
        srt = torch.sort(logits, dim=-1, descending=True).values
        margin = srt[:, k - 1] - srt[:, k] if logits.shape[1] > k else torch.full((T,), float("inf"))
        margin = margin / logits.pow(2).mean().sqrt().clamp_min(1e-30)
        record(prefix, ids.clone(), margin)
    if forced_ids is not None:
        ids = forced_ids.to(torch.long)
        scores = 1.0 / (1.0 + torch.exp(-torch.gather(logits, 1, ids)))
    wg, wu, wd = (w[f"{prefix}.experts.{n}_proj.weight"] for n in ("gate", "up", "down"))
    out = torch.zeros(T, H, dtype=F32)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            xs = x[t: t + 1] * scores[t, j]
            out[t] += swiglu(xs, wg[e], wu[e], wd[e])[0]
    shared = swiglu(x, *(w[f"{prefix}.shared_expert.{n}_proj.weight"] for n in ("gate", "up", "down")))
    return out + shared


def dense_feed_forward(w, prefix: str, x: torch.Tensor) -> torch.Tensor:
    """Dense SwiGLU of non-MoE layers; same formula as models.rs:2307-2312."""
    return swiglu(x, *(w[f"{prefix}.{n}_proj.weight"] for n in ("gate", "up", "down")))


def block(cfg: dict, w, i: int, x: torch.Tensor, inv_freq, forced_routing=None, record=None) -> torch.Tensor:
    """h = x + attn(norm(x)); y = h + ffn(norm(h))  (Llama4Block::forward, models.rs:6143-6149)."""
    p = f"model.layers.{i}"
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = x + attention(cfg, w, f"{p}.self_attn", i, rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), inv_freq)
    n = rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)
    if layer_is_moe(cfg, i):
        forced = forced_routing.get(f"{p}.feed_forward") if forced_routing else None
        return h + moe_feed_forward(cfg, w, f"{p}.feed_forward", n, forced, record)
    return h + dense_feed_forward(w, f"{p}.feed_forward", n)


def forward(raw_cfg: dict, weights: Dict[str, torch.Tensor], token_ids: List[int],
            schedule: Optional[List[int]] = None, forced_routing=None, record=None) -> torch.Tensor:
    """Logits [T, V] at every position of one sequence (Llama4Like::forward,
    models.rs:6204-6217; head by tensor presence, models.rs:6186-6193).
    ``schedule`` lists the layers in the order they run (default 0..L-1).
    ``forced_routing`` {"model.layers.i.feed_forward": ids [T, k]} and ``record``: see
    :func:`moe_feed_forward`."""
    cfg = text_config(raw_cfg)
    w = weights
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    inv_freq = rope_inverse_frequencies(hd, float(cfg.get("rope_theta", 1e6)), cfg.get("rope_scaling"))
    x = w["model.embed_tokens.weight"].to(F32)[torch.tensor(token_ids, dtype=torch.long)]
    for i in (schedule if schedule is not None else range(cfg["num_hidden_layers"])):
        x = block(cfg, w, i, x, inv_freq, forced_routing, record)
    x = rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return x @ head.to(F32).T


# --------------------------------------------------------------------------- sampling
class Lcg:
    """The reference's generator (crates/hi-mlx/src/generate.rs:123-146)."""

    def __init__(self, seed: int):
        self.state = (seed ^ 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF

    def next_f32(self) -> float:
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return float(self.state >> 40) / float(1 << 24)


def sample(logits: torch.Tensor, temperature: float, top_p: float, top_k: int, u: float) -> int:
    """One token from one row of logits, given one uniform draw ``u``.

    Greedy when temperature <= 0 (lowest id on ties, crates/hi-cuda/src/kernels.cu:7176,7225-7234).
    Temperature only (no top-k, top_p >= 1): weights exp(l/T - max) walked in VOCABULARY
    order, first index whose running sum exceeds u * total (kernels.cu:7327-7352).
    Ranked (top-k and/or top-p): sort descending, ties by id, cut to top-k
    (crates/hi-cuda/src/qwen_cpu.rs:3692-3704), keep the shortest prefix whose mass
    reaches top_p, and walk it with draw = u * kept mass
    (crates/hi-mlx/src/generate.rs:86-108)."""
    row = logits.to(F32)
    V = row.numel()
    if not (temperature > 0.0):
        return int(torch.argmax(row))
    z = row / temperature
    wts = torch.exp(z - z.max())
    k_eff = top_k if (top_k and 0 < top_k < V) else V
    cutoff = min(max(top_p, 0.0), 1.0)
    if k_eff == V and cutoff >= 1.0:
        target = u * float(wts.sum())
        cum = 0.0
        last = 0
        for i in range(V):
            wi = float(wts[i])
            if wi <= 0.0:
                continue
            last = i
            cum += wi
            if target < cum:
                return i
        return last
    p = wts / wts.sum()
    order = sorted(range(V), key=lambda i: (-float(p[i]), i))[:k_eff]
    if 0.0 < cutoff < 1.0:
        cum, keep = 0.0, 0
        for i in order:
            cum += float(p[i])
            keep += 1
            if cum >= cutoff:
                break
        order = order[:max(keep, 1)]
    draw = u * sum(float(p[i]) for i in order)
    for i in order:
        if draw <= float(p[i]):
            return i
        draw -= float(p[i])
    return int(torch.argmax(row))
