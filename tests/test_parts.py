"""Each part alone, built through the registry from its parameters, against the plain function."""
import math

import pytest
import torch

import plain_llama4 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = [(torch.float32, 3e-5), (torch.bfloat16, 2.5e-2)]


def env(dt, hidden):
    from hi_b200.parts.linear import configure_matmul_precision
    from hi_b200.parts.registry import BuildEnv

    configure_matmul_precision()
    return BuildEnv(dtype=dt, device=torch.device(DEV), hidden_size=hidden)


def fill(part, dt, seed, std=0.1):
    """Random tensors for a part; returns them on the CPU (as stored) by name."""
    from hi_b200.weights.loader import random_tensor

    stored = {s.name: random_tensor(s, seed, std) for s in part.tensor_specs() if s.init != "absent"}
    part.load(lambda name: None if name not in stored else stored[name].to(DEV).to(dt))
    return stored


def ctx_for(lens, starts, page, tables):
    from hi_b200.parts.context import StepContext

    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return StepContext(n_tokens=sum(lens), n_seqs=len(lens), tokens=torch.zeros(sum(lens), dtype=torch.int32, device=DEV),
                       positions=pos.to(DEV), seq_of_token=sot.to(DEV), cu_seqlens=cu.to(DEV),
                       slots=torch.arange(len(lens), dtype=torch.int32, device=DEV), start_pos=list(starts),
                       n_new=list(lens), slot_ids=list(range(len(lens))),
                       block_tables={g: t.to(DEV) for g, t in tables.items()}, page_size=page,
                       max_context=max(s + n for s, n in zip(starts, lens)))


def close(got, want, tol, what=""):
    err = float((got.float().cpu() - want.float()).abs().max() / (want.float().abs().max() + 1e-12))
    assert math.isfinite(err) and err <= tol, f"{what}: rel err {err:.3e} > {tol}"


@pytest.mark.parametrize("dt,tol", DT)
def test_rmsnorm_part(dt, tol):
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec

    part = build("norm", PartSpec("rmsnorm", {"size": 200, "eps": 3e-4}), env(dt, 200), "n")
    w = fill(part, dt, 1)["n.weight"]
    g = torch.Generator().manual_seed(50)
    x = torch.randn(5, 200, generator=g) * 2
    d = torch.randn(5, 200, generator=g).to(dt)
    xg = x.clone().to(DEV)
    close(part.forward(xg, d.to(DEV)), plain.rms_norm(x + d.float(), torch.ones(200), 3e-4), tol)
    close(xg, x + d.float(), 1e-7)
    assert w.dtype == torch.bfloat16 and bool((w == 1).all())


def test_rotary_table_matches_the_plain_one():
    from hi_b200.parts.basic import llama3_inverse_frequencies

    for hd, theta, sc in ((16, 10000.0, None), (32, 500000.0, dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                                  original_max_position_embeddings=64)),
                          (128, 500000.0, dict(factor=16.0, low_freq_factor=1.0, high_freq_factor=1.0,
                                               original_max_position_embeddings=8192)),
                          (48, 500000.0, dict(factor=16.0, low_freq_factor=1.0, high_freq_factor=1.0,
                                              original_max_position_embeddings=32))):
        mine = torch.from_numpy(llama3_inverse_frequencies(hd, theta, sc))
        ref = plain.rope_inverse_frequencies(hd, theta, sc)
        assert torch.isfinite(mine).all()
        assert float(((mine - ref).abs() / ref).max()) < 1e-6, (hd, theta, sc)


@pytest.mark.parametrize("dt,tol", DT)
@pytest.mark.parametrize("kind", ["chunked_rope_norm", "global_temperature", "sliding_interleaved", "partial_rotary",
                                  "partial_rotary_interleaved"])
def test_attention_mixer(kind, dt, tol):
    """The mixer over a paged cache, fed in two steps, against whole-sequence attention."""
    from hi_b200.parts.context import CacheView
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec

    H, nh, nkv, hd, page, T, cut = 72, 6, 2, 16, 4, 53, 31
    if kind.startswith("partial_rotary"):
        hd = 48                     # 32 of 48 dims rotate; the rest pass through and count in the norm
    cfgs = {
        "partial_rotary": dict(window=("chunk", 20), qk_norm=True,
                               position=PartSpec("rope", {"head_dim": 48, "rot_dim": 32, "theta": 1e4, "scaling": None})),
        "partial_rotary_interleaved": dict(window=None, qk_norm=False, temperature=(8.0, 0.3),
                                           position=PartSpec("rope", {"head_dim": 48, "rot_dim": 16, "theta": 1e4, "scaling": None,
                                                                      "interleaved": True})),
        "chunked_rope_norm": dict(window=("chunk", 12), position=PartSpec("rope", {"head_dim": hd, "theta": 1e4, "scaling": None}),
                                  qk_norm=True),
        "global_temperature": dict(window=None, position=PartSpec("none"), temperature=(8.0, 0.3)),
        "sliding_interleaved": dict(window=("sliding", 9), qk_norm=False,
                                    position=PartSpec("rope", {"head_dim": hd, "theta": 5e5, "interleaved": True,
                                                               "scaling": dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                                               original_max_position_embeddings=16)})),
    }
    params = dict(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, **cfgs[kind])
    part = build("mixer", PartSpec("attention", params), env(dt, H), "m")
    w = fill(part, dt, 2, std=0.3)
    blocks = -(-T // page)
    table = {0: torch.arange(blocks, dtype=torch.int32).flip(0).reshape(1, blocks).contiguous()}
    view = CacheView(group=0, k_pages=torch.zeros(blocks, nkv, page, hd, dtype=dt, device=DEV),
                     v_pages=torch.zeros(blocks, nkv, page, hd, dtype=dt, device=DEV))
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(len(kind))).to(dt)   # inputs do not depend on what ran before
    outs = [part.forward(x[a:b].to(DEV).contiguous(), ctx_for([b - a], [a], page, table), view) for a, b in ((0, cut), (cut, T))]
    got = torch.cat(outs)
    # plain, whole sequence, same formulas with this part's options
    xf = x.float()
    q = (xf @ w["m.q_proj.weight"].float().T).view(T, nh, hd)
    k = (xf @ w["m.k_proj.weight"].float().T).view(T, nkv, hd)
    v = (xf @ w["m.v_proj.weight"].float().T).view(T, nkv, hd)
    pos = torch.arange(T)
    pspec = cfgs[kind]["position"]
    if pspec.kind == "rope":
        rot = pspec.params.get("rot_dim", hd)
        inv = plain.rope_inverse_frequencies(rot, pspec.params["theta"], pspec.params.get("scaling"))
        il = pspec.params.get("interleaved", False)
        q = torch.cat([plain.apply_rope(q[..., :rot], pos, inv, il), q[..., rot:].float()], dim=-1)
        k = torch.cat([plain.apply_rope(k[..., :rot], pos, inv, il), k[..., rot:].float()], dim=-1)
    if cfgs[kind].get("qk_norm"):
        q, k = plain.rms_norm(q, None, 1e-6), plain.rms_norm(k, None, 1e-6)
    if cfgs[kind].get("temperature"):
        q = plain.attention_temperature(q, pos, *cfgs[kind]["temperature"])
    win = cfgs[kind]["window"]
    vis = plain.visibility(T, win[1] if win and win[0] == "chunk" else None)
    if win and win[0] == "sliding":
        vis = vis & (pos[None, :] > pos[:, None] - win[1])
    o = torch.empty(T, nh, hd)
    for h in range(nh):
        s = (q[:, h] @ k[:, h // (nh // nkv)].T) * hd ** -0.5
        o[:, h] = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, h // (nh // nkv)]
    want = o.reshape(T, nh * hd) @ w["m.o_proj.weight"].float().T
    close(got, want, tol, kind)


@pytest.mark.parametrize("dt,tol", DT)
def test_feed_forward_parts(dt, tol):
    from hi_b200.parts.context import StepContext
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec

    H = 88
    x = torch.randn(37, H, generator=torch.Generator().manual_seed(37)).to(dt)
    ctx = ctx_for([37], [0], 4, {})
    dense = build("feed_forward", PartSpec("dense_swiglu", {"hidden_size": H, "intermediate_size": 136}), env(dt, H), "f")
    w = fill(dense, dt, 3, std=0.2)
    close(dense.forward(x.to(DEV), ctx), plain.dense_feed_forward(w, "f", x.float()), tol, "dense")

    moe = build("feed_forward", PartSpec("moe_sigmoid", {"hidden_size": H, "num_experts": 6, "top_k": 2,
                                                         "intermediate_size": 56, "shared_expert": True}), env(dt, H), "e")
    w = fill(moe, dt, 4, std=0.2)
    seen = {}
    ctx.tap = lambda name, t: seen.__setitem__(name, t.cpu())
    got = moe.forward(x.to(DEV), ctx, normed_f32=x.float().to(DEV)).materialize(37)
    cfg = {"num_experts_per_tok": 2}
    want = plain.moe_feed_forward(cfg, w, "e", x.float(), forced_ids=seen["e.router_ids"])
    close(got, want, tol, "experts")
    own, _ = plain.router_top_k(x.float() @ w["e.router.weight"].float().T, 2)
    assert float((own.sort(-1).values == seen["e.router_ids"].long().sort(-1).values).float().mean()) > 0.9


@pytest.mark.parametrize("dt,tol", DT)
@pytest.mark.parametrize("score,renorm,scale", [("softmax", True, "output"), ("softmax", False, "input"), ("sigmoid", True, "output"),
                                                ("sigmoid", False, "output")])
def test_routed_experts_with_other_routing_rules(score, renorm, scale, dt, tol):
    """The routed feed-forward with the routing rules Llama 4 does not use (softmax scores over all
    experts, chosen scores renormalised, the score on the expert's output instead of its input),
    through the same router, grouped-product and combine kernels, for a few rows (the weight-streaming
    kernels) and for many (tcgen05 in bfloat16), summed by the next norm's kernel and by the
    standalone combine; against the formulas written out here."""
    from hi_b200.kernels import ops
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec

    H, E, K, I = 96, 7, 3, 64
    part = build("feed_forward", PartSpec("routed_experts", {"hidden_size": H, "num_experts": E, "top_k": K, "intermediate_size": I,
                                                             "shared_expert": False, "score": score, "renormalize": renorm,
                                                             "scale": scale}), env(dt, H), "e")
    w = {k: v.float() for k, v in fill(part, dt, 6, std=0.25).items()}
    for n in (5, 200):
        x = torch.randn(n, H, generator=torch.Generator().manual_seed(n)).to(dt)
        ctx = ctx_for([n], [0], 4, {})
        seen = {}
        ctx.tap = lambda name, t: seen.__setitem__(name, t.cpu())
        pending = part.forward(x.to(DEV), ctx, normed_f32=x.float().to(DEV))
        ids = seen["e.router_ids"].long()
        logits = x.float() @ w["e.router.weight"].T
        chosen = torch.gather(logits, 1, ids)
        s = torch.softmax(logits, dim=1).gather(1, ids) if score == "softmax" else torch.sigmoid(chosen)
        if renorm:
            s = s / s.sum(dim=1, keepdim=True)
        want = torch.zeros(n, H)
        for t in range(n):
            for j in range(K):
                e = int(ids[t, j])
                xin = x[t: t + 1].float() * (s[t, j] if scale == "input" else 1.0)
                y = plain.swiglu(xin, w["e.experts.gate_proj.weight"][e], w["e.experts.up_proj.weight"][e],
                                 w["e.experts.down_proj.weight"][e])[0]
                want[t] += y * (s[t, j] if scale == "output" else 1.0)
        own, _ = plain.router_top_k(logits, K)
        assert float((own.sort(-1).values == ids.sort(-1).values).all(-1).float().mean()) > 0.85
        close(pending.materialize(n), want, tol, f"{n} rows, standalone combine")
        residual = torch.zeros(n, H, device=DEV)
        ops.add_rmsnorm(residual, pending.dense, None, 1e-5, torch.float32, None, False, pending.routed,
                        pending.slot_of_entry, pending.top_k, pending.entry_weights)
        close(residual, want, tol, f"{n} rows, combine inside the norm")


@pytest.mark.parametrize("dt,tol", DT)
def test_embedding_and_head(dt, tol):
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec

    V, H = 331, 56
    emb = build("embedding", PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}), env(dt, H), "emb")
    we = fill(emb, dt, 5)["emb.weight"]
    toks = torch.tensor([0, 330, 17, 17], dtype=torch.int32)
    close(emb.forward(toks.to(DEV)), we.float()[toks.long()], 1e-7)
    z = torch.randn(4, H, generator=torch.Generator().manual_seed(4)).to(dt)
    tied = build("head", PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "tie": True}), env(dt, H), "head")
    assert fill(tied, dt, 6) == {}
    out = tied.forward(z.to(DEV), emb)
    assert out.dtype == torch.float32 and tied.tied
    close(out, z.float() @ we.float().T, 1e-5 if dt == torch.float32 else 2e-3, "tied head")
    own = build("head", PartSpec("linear_head", {"vocab_size": V, "hidden_size": H}), env(dt, H), "head")
    wh = fill(own, dt, 7)["head.weight"]
    close(own.forward(z.to(DEV), emb), z.float() @ wh.float().T, 1e-5 if dt == torch.float32 else 2e-3, "own head")


@pytest.mark.parametrize("dt,tol", DT)
def test_block_arrangement(dt, tol):
    """One pre-norm block built from a LayerSpec (attention + dense SwiGLU + two norms), with a pending
    sum carried in, against h = x + attn(norm(x)); y = h + ffn(norm(h))."""
    from hi_b200.parts.context import CacheView
    from hi_b200.parts.model import Layer
    from hi_b200.parts.spec import LayerSpec, PartSpec

    H, nh, nkv, hd, page, T = 64, 4, 2, 16, 8, 21
    norm = lambda n: PartSpec("rmsnorm", {"name": n, "size": H, "eps": 1e-5})
    spec = LayerSpec(prefix="L", norm_mixer=norm("n1"), norm_feed_forward=norm("n2"),
                     mixer=PartSpec("attention", {"name": "att", "hidden_size": H, "num_heads": nh, "num_kv_heads": nkv,
                                                  "head_dim": hd, "window": None}),
                     feed_forward=PartSpec("dense_swiglu", {"name": "ff", "hidden_size": H, "intermediate_size": 96}))
    layer = Layer(spec, env(dt, H))
    w = {}
    for part in layer.parts():
        w.update(fill(part, dt, 9, std=0.12))
    g = torch.Generator().manual_seed(257)
    x = torch.randn(T, H, generator=g)
    carried = (torch.randn(T, H, generator=g) * 0.5).to(dt)
    blocks = -(-T // page)
    view = CacheView(group=0, k_pages=torch.zeros(blocks, nkv, page, hd, dtype=dt, device=DEV),
                     v_pages=torch.zeros(blocks, nkv, page, hd, dtype=dt, device=DEV))
    ctx = ctx_for([T], [0], page, {0: torch.arange(blocks, dtype=torch.int32).reshape(1, blocks)})
    residual = x.clone().to(DEV)
    residual, pending = layer.arrangement.forward(layer, residual, carried.to(DEV), ctx, view)
    got = residual.cpu() + pending.float().cpu()
    # plain
    x0 = x + carried.float()
    q = (plain.rms_norm(x0, w["L.n1.weight"], 1e-5) @ w["L.att.q_proj.weight"].float().T).view(T, nh, hd)
    n1 = plain.rms_norm(x0, w["L.n1.weight"], 1e-5)
    k = (n1 @ w["L.att.k_proj.weight"].float().T).view(T, nkv, hd)
    v = (n1 @ w["L.att.v_proj.weight"].float().T).view(T, nkv, hd)
    a = plain.attention_core(q, k, v, None) @ w["L.att.o_proj.weight"].float().T
    hmid = x0 + a
    want = hmid + plain.dense_feed_forward(w, "L.ff", plain.rms_norm(hmid, w["L.n2.weight"], 1e-5))
    close(got, want, tol, "pre-norm block")
