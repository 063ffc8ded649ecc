"""Each CUDA kernel alone against a plain float32 reference, at sizes other than the models'."""
import math

import pytest
import torch

import plain_llama4 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)]


def ops():
    from hi_b200.kernels import ops as o
    from hi_b200.parts.linear import configure_matmul_precision

    configure_matmul_precision()
    return o


def close(got, want, tol, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    err = float((got - want).abs().max() / (want.abs().max() + 1e-12))
    assert math.isfinite(err) and err <= tol, f"{what}: rel err {err:.3e} > {tol}"


@pytest.mark.parametrize("dt,tol", DT)
def test_embed_and_norm(dt, tol):
    o = ops()
    g = torch.Generator().manual_seed(0)
    table = torch.randn(331, 120, generator=g).to(dt)
    toks = torch.randint(0, 331, (29,), generator=g, dtype=torch.int32)
    close(o.embed_gather(table.to(DEV), toks.to(DEV)), table.float()[toks.long()], 1e-7, "embed")
    for hidden in (48, 120, 1000, 1001, 5120, 7168, 20000):
        x = torch.randn(11, hidden, generator=g) * 3
        d = torch.randn(11, hidden, generator=g).to(dt)
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dt)
        xg = x.clone().to(DEV)
        y, y32 = o.add_rmsnorm(xg, d.to(DEV), w.to(DEV), 1e-5, dt, None, True)
        want = plain.rms_norm(x + d.float(), w, 1e-5)
        close(y, want, tol, f"rmsnorm hidden {hidden}")
        close(y32, want, 2e-6, "rmsnorm float32 output")
        close(xg, x + d.float(), 1e-7, "residual sum")
        # the routed experts' rows join the same sum (top-2 of 5 sorted rows per token)
        routed = torch.randn(22, hidden, generator=g)
        slots = torch.randperm(22, generator=g).to(torch.int32)
        xr = x.clone().to(DEV)
        yr = o.add_rmsnorm(xr, d.to(DEV), w.to(DEV), 1e-5, dt, None, False, routed.to(DEV), slots.to(DEV), 2)
        summed = x + d.float() + routed[slots.long()].view(11, 2, hidden).sum(1)
        close(yr, plain.rms_norm(summed, w, 1e-5), tol, f"rmsnorm with routed rows, hidden {hidden}")
        close(xr, summed, 1e-6, "residual sum with routed rows")
        rows = torch.tensor([10, 0, 4], dtype=torch.int32)
        before = xg.clone()
        y2 = o.add_rmsnorm(xg, d.to(DEV), w.to(DEV), 1e-5, dt, rows.to(DEV))
        close(y2, plain.rms_norm(before.cpu()[rows.long()] + d.float()[rows.long()], w, 1e-5), tol, "row map")
        assert torch.equal(xg, before), "row-mapped norm must not touch the residual"


@pytest.mark.parametrize("dt,tol", DT)
def test_swiglu(dt, tol):
    o = ops()
    gu = (torch.randn(13, 2 * 72, generator=torch.Generator().manual_seed(13)) * 2).to(dt)
    g, u = gu[:, :72].float(), gu[:, 72:].float()
    close(o.swiglu(gu.to(DEV)), g * torch.sigmoid(g) * u, tol, "swiglu")


def paged_case(o, dt, nh, nkv, hd, page, chunk, window, lens, starts, inv_freq, interleaved, qk_norm, temp, seed,
               split=True, tc=False, key_splits=()):
    """Two phases: fill `starts` tokens of every sequence, then run `lens` new tokens; returns the
    kernel's q and attention output for the second phase and the plain reference's."""
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    total = [s + l for s, l in zip(starts, lens)]
    n_pages = sum(-(-t // page) for t in total) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-t // page) for t in total)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    c = 0
    for s in range(S):
        for b in range(-(-total[s] // page)):
            bt[s, b] = perm[c]; c += 1
    kp = torch.full((n_pages, nkv, page, hd), float("nan")).to(dt).to(DEV)     # unwritten slots poison
    vp = kp.clone()
    qkv_all = [(torch.randn(t, (nh + 2 * nkv) * hd, generator=g) * 1.5).to(dt) for t in total]
    got = None
    for phase, (lo, hi) in enumerate((([0] * S, starts), (starts, total))):
        spans = [(lo[s], hi[s]) for s in range(S)]
        if sum(b - a for a, b in spans) == 0:
            continue
        qkv = torch.cat([qkv_all[s][a:b] for s, (a, b) in enumerate(spans)])
        pos = torch.cat([torch.arange(a, b) for a, b in spans]).to(torch.int32)
        sot = torch.cat([torch.full((b - a,), s) for s, (a, b) in enumerate(spans)]).to(torch.int32)
        q = o.qkv_post(qkv.to(DEV), nh, nkv, hd, pos.to(DEV), None if inv_freq is None else inv_freq.to(DEV),
                       interleaved, qk_norm, 1e-6, temp, sot.to(DEV), bt.to(DEV), kp, vp, page, True)
        out = o.paged_attention(q, kp, vp, bt.to(DEV), sot.to(DEV), pos.to(DEV), chunk, window, hd ** -0.5,
                                max(total) if split else 0)
        got = (q, out)
        if o.prefill_attention_supported(dt, nh, nkv, hd):
            cu = torch.tensor([0] + list(torch.tensor([b - a for a, b in spans]).cumsum(0)), dtype=torch.int32)
            fast = o.prefill_attention(q, kp, vp, bt.to(DEV), cu.to(DEV), pos.to(DEV), S, max(b - a for a, b in spans),
                                       chunk, window, hd ** -0.5)
            got = (q, out, fast)
            if tc:
                # and the same with the key tiles of every block shared among k blocks
                for k in (1,) + tuple(key_splits):
                    got = got + (o.prefill_attention_tc(q, kp, vp, bt.to(DEV), cu.to(DEV), pos.to(DEV), S,
                                                        max(b - a for a, b in spans), chunk, window, hd ** -0.5,
                                                        key_splits=k),)
    # plain: whole sequences
    want_q, want_o = [], []
    for s in range(S):
        x = qkv_all[s].float().view(total[s], nh + 2 * nkv, hd)
        q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]
        pos = torch.arange(total[s])
        if inv_freq is not None:
            q, k = plain.apply_rope(q, pos, inv_freq, interleaved), plain.apply_rope(k, pos, inv_freq, interleaved)
        if qk_norm:
            q, k = plain.rms_norm(q, None, 1e-6), plain.rms_norm(k, None, 1e-6)
        if temp:
            q = plain.attention_temperature(q, pos, *temp)
        # the cache holds k, v in the engine dtype
        k, v, qr = k.to(dt).float(), v.to(dt).float(), q.to(dt).float()
        vis = plain.visibility(total[s], chunk or None)
        if window:
            idx = torch.arange(total[s])
            vis = vis & (idx[None, :] > idx[:, None] - window)
        o_ref = torch.empty(total[s], nh, hd)
        for hh in range(nh):
            sc = (qr[:, hh] @ k[:, hh // (nh // nkv)].T) * hd ** -0.5
            o_ref[:, hh] = torch.softmax(sc.masked_fill(~vis, float("-inf")), -1) @ v[:, hh // (nh // nkv)]
        want_q.append(q[starts[s]:]); want_o.append(o_ref[starts[s]:])
    return got, (torch.cat(want_q), torch.cat(want_o))


CASES = [  # nh, nkv, hd, page, chunk, window, interleaved, qk_norm, temp
    (4, 2, 16, 4, 32, 0, False, True, None),
    (10, 2, 48, 8, 0, 0, True, False, (8.0, 0.25)),
    (6, 3, 32, 16, 16, 0, False, False, None),
    (40, 8, 128, 64, 0, 0, False, True, None),
    (5, 1, 256, 16, 0, 20, True, True, None),
    (8, 8, 64, 32, 24, 0, False, False, None),
    (7, 7, 80, 2, 10, 7, False, True, None),
    (12, 4, 112, 64, 100, 0, False, False, None),
]


@pytest.mark.parametrize("dt,tol", DT)
@pytest.mark.parametrize("case", CASES)
def test_qkv_post_and_paged_attention(case, dt, tol):
    o = ops()
    nh, nkv, hd, page, chunk, window, inter, qkn, temp = case
    inv = None if temp else plain.rope_inverse_frequencies(hd, 10000.0, None)
    for lens, starts, split in (([37, 1, 70, 1], [0, 130, 23, 63], False), ([300, 1, 2, 1], [0, 700, 255, 256], True)):
        got, want = paged_case(o, dt, nh, nkv, hd, page, chunk, window, lens=lens, starts=starts,
                               inv_freq=inv, interleaved=inter, qk_norm=qkn, temp=temp, seed=nh * hd, split=split)
        close(got[0], want[0].reshape(got[0].shape), tol, f"q {case}")
        close(got[1], want[1].reshape(got[1].shape), tol, f"attention {case} split={split}")
        if len(got) > 2:
            close(got[2], want[1].reshape(got[2].shape), tol, f"tensor-core prefill attention {case}")


@pytest.mark.parametrize("shape", [(40, 8, 128, 64, 0, 0), (8, 8, 64, 16, 0, 0), (32, 2, 128, 32, 512, 0), (10, 2, 64, 8, 0, 300),
                                   (3, 1, 128, 64, 100, 0), (16, 4, 128, 128, 0, 0), (12, 4, 64, 64, 192, 0)])
def test_decode_attention_on_tensor_cores(shape):
    """The decode kernels (bfloat16, split over runs of keys) against whole-sequence attention, for
    requests of very different lengths in one batch, and against the general kernel. Pages of 16,
    32, 64 and 128 with no window or a chunk that is a multiple of 64 run the kernel with TMA tile
    loads; pages of 8, a chunk of 100 and the sliding window run the cp.async kernel."""
    o = ops()
    nh, nkv, hd, page, chunk, window = shape
    lens = [1, 1, 1, 1, 1, 1]
    starts = [0, 63, 255, 256, 1030, 2500]
    inv = plain.rope_inverse_frequencies(hd, 10000.0, None)
    g = torch.Generator().manual_seed(nh + hd)
    S = len(lens)
    total = [s + l for s, l in zip(starts, lens)]
    n_pages = sum(-(-t // page) for t in total) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-t // page) for t in total)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    c = 0
    for s in range(S):
        for b in range(-(-total[s] // page)):
            bt[s, b] = perm[c]; c += 1
    dt = torch.bfloat16
    kp = torch.zeros(n_pages, nkv, page, hd, dtype=dt)
    vp = torch.zeros_like(kp)
    ks = [torch.randn(t, nkv, hd, generator=g).to(dt) for t in total]
    vs = [torch.randn(t, nkv, hd, generator=g).to(dt) for t in total]
    for s in range(S):
        for p in range(total[s]):
            kp[bt[s, p // page], :, p % page] = ks[s][p]; vp[bt[s, p // page], :, p % page] = vs[s][p]
    q = (torch.randn(S, nh, hd, generator=g) * 2).to(dt)
    pos = torch.tensor([t - 1 for t in total], dtype=torch.int32)
    sot = torch.arange(S, dtype=torch.int32)
    args = (q.to(DEV), kp.to(DEV), vp.to(DEV), bt.to(DEV), sot.to(DEV), pos.to(DEV), chunk, window, hd ** -0.5, max(total))
    got = o.decode_attention(*args)
    general = o.paged_attention(*args)
    want = torch.empty(S, nh, hd)
    for s in range(S):
        p = total[s] - 1
        lo = (p // chunk) * chunk if chunk else 0
        if window:
            lo = max(lo, p - window + 1)
        for hh in range(nh):
            kv = hh // (nh // nkv)
            sc = (ks[s][lo:p + 1, kv].float() @ q[s, hh].float()) * hd ** -0.5
            want[s, hh] = torch.softmax(sc, 0) @ vs[s][lo:p + 1, kv].float()
    close(got, want, 2e-2, f"decode attention {shape}")
    close(general, want, 2e-2, f"general attention {shape}")
    assert not o.decode_attention_supported(torch.float32, nh, nkv, hd)
    assert not o.decode_attention_supported(torch.bfloat16, 40, 2, 128) and not o.decode_attention_supported(torch.bfloat16, 4, 2, 48)


@pytest.mark.parametrize("shape", [(4, 2, 128, 64, 0, 0), (4, 2, 128, 16, 100, 0), (8, 2, 64, 32, 0, 50),
                                   (2, 1, 128, 128, 0, 0), (2, 2, 64, 256, 300, 0), (5, 1, 128, 64, 256, 0)])
def test_prefill_attention_on_tcgen05(shape):
    """The tcgen05 prefill kernel (TMA page loads, S / P V / O in tensor memory) against whole-sequence
    attention: portions that start inside a sequence, straddle chunks and pages, and end off a tile;
    and the same with the key tiles of every (query tile, head) shared among two, three or five
    blocks whose rows a merge kernel combines (some shares are empty: fewer tiles than blocks)."""
    o = ops()
    nh, nkv, hd, page, chunk, window = shape
    dt = torch.bfloat16
    assert o.prefill_attention_tc_supported(dt, nh, nkv, hd, page)
    inv = plain.rope_inverse_frequencies(hd, 10000.0, None)
    got, want = paged_case(o, dt, nh, nkv, hd, page, chunk, window, lens=[300, 140, 1, 129], starts=[0, 77, 500, 128],
                           inv_freq=inv, interleaved=False, qk_norm=True, temp=None, seed=hd + page, split=True, tc=True,
                           key_splits=(2, 3, 5))
    o.check_tc_status()
    labels = ["one block per query tile and head"] + [f"keys in {k} shares" for k in (2, 3, 5)]
    assert len(got) == 3 + len(labels)
    for label, res in zip(labels, got[3:]):
        close(res, want[1].reshape(res.shape), 2e-2, f"tcgen05 prefill attention {shape}, {label}")
    close(got[1], want[1].reshape(got[1].shape), 2e-2, f"general attention {shape}")


@pytest.mark.parametrize("dt,tol", DT)
def test_one_far_key_among_hundreds(dt, tol):
    """One old key, in the first page, matches the decoded token's query exactly and strongly:
    the output must be that key's value row. Any key dropped at a page's edge shows at once."""
    o = ops()
    nh, nkv, hd, page = 4, 2, 64, 16
    for far in (0, 15, 16, 17, 255, 256, 600):
        n = 601
        g = torch.Generator().manual_seed(far)
        k = torch.randn(n, nkv, hd, generator=g) * 0.05
        v = torch.randn(n, nkv, hd, generator=g)
        q = torch.randn(1, nh, hd, generator=g) * 0.05
        direction = torch.nn.functional.normalize(torch.randn(hd, generator=g), dim=0)
        k[far] = direction * 30.0
        q[0] = direction * 30.0
        blocks = -(-n // page)
        bt = torch.arange(blocks, dtype=torch.int32).flip(0).reshape(1, blocks).contiguous()
        kp = torch.zeros(blocks, nkv, page, hd); vp = torch.zeros_like(kp)
        for p in range(n):
            kp[bt[0, p // page], :, p % page] = k[p]; vp[bt[0, p // page], :, p % page] = v[p]
        out = o.paged_attention(q.to(dt).to(DEV), kp.to(dt).to(DEV), vp.to(dt).to(DEV), bt.to(DEV),
                                torch.zeros(1, dtype=torch.int32, device=DEV),
                                torch.tensor([n - 1], dtype=torch.int32, device=DEV), 0, 0, hd ** -0.5, n)
        want = v[far].to(dt).float().repeat_interleave(nh // nkv, 0)
        close(out[0], want, tol, f"far key at {far}")
        if dt == torch.bfloat16:
            fast = o.decode_attention(q.to(dt).to(DEV), kp.to(dt).to(DEV), vp.to(dt).to(DEV), bt.to(DEV),
                                      torch.zeros(1, dtype=torch.int32, device=DEV),
                                      torch.tensor([n - 1], dtype=torch.int32, device=DEV), 0, 0, hd ** -0.5, n)
            close(fast[0], want, tol, f"far key at {far}, decode kernel")


@pytest.mark.parametrize("dt,tol", DT)
def test_window_edges(dt, tol):
    """The strong key sits just inside or just outside the chunk or the sliding window."""
    o = ops()
    nh, nkv, hd, page = 2, 1, 32, 8
    n = 100
    g = torch.Generator().manual_seed(1)
    direction = torch.nn.functional.normalize(torch.randn(hd, generator=g), dim=0)
    for chunk, window, key, visible in ((32, 0, 96, True), (32, 0, 95, False), (0, 10, 90, True), (0, 10, 89, False),
                                        (40, 0, 80, True), (40, 0, 79, False)):
        k = torch.randn(n, nkv, hd, generator=g) * 0.05
        v = torch.randn(n, nkv, hd, generator=g)
        k[key] = direction * 30.0
        q = (direction * 30.0).repeat(1, nh, 1)
        blocks = -(-n // page)
        bt = torch.arange(blocks, dtype=torch.int32).reshape(1, blocks)
        kp = k.reshape(blocks, page, nkv, hd).permute(0, 2, 1, 3).contiguous() if n % page == 0 else None
        if kp is None:
            pad = blocks * page - n
            kp = torch.cat([k, torch.zeros(pad, nkv, hd)]).reshape(blocks, page, nkv, hd).permute(0, 2, 1, 3).contiguous()
            vp = torch.cat([v, torch.zeros(pad, nkv, hd)]).reshape(blocks, page, nkv, hd).permute(0, 2, 1, 3).contiguous()
        else:
            vp = v.reshape(blocks, page, nkv, hd).permute(0, 2, 1, 3).contiguous()
        out = o.paged_attention(q.to(dt).to(DEV), kp.to(dt).to(DEV), vp.to(dt).to(DEV), bt.to(DEV),
                                torch.zeros(1, dtype=torch.int32, device=DEV),
                                torch.tensor([n - 1], dtype=torch.int32, device=DEV), chunk, window, hd ** -0.5)
        hit = float((out[0, 0].float().cpu() - v[key, 0].to(dt).float()).abs().max()) < 0.05
        assert hit == visible, f"chunk {chunk} window {window}: key {key} should be {'seen' if visible else 'masked'}"


def counts_of(ids, experts):
    return torch.bincount(ids.cpu().view(-1).long(), minlength=experts).tolist()


@pytest.mark.parametrize("dt,tol", DT)
@pytest.mark.parametrize("shape", [(64, 4, 1, 128, 50), (192, 8, 2, 96, 33), (120, 5, 3, 72, 300), (120, 5, 5, 72, 1),
                                   (256, 16, 1, 512, 8), (200, 128, 1, 64, 200), (104, 3, 2, 40, 700), (100, 4, 2, 36, 20)])
def test_router_plan_and_experts(shape, dt, tol):
    o = ops()
    H, E, k, I, n = shape
    g = torch.Generator().manual_seed(H + n)
    x32 = torch.randn(n, H, generator=g)
    x = x32.to(dt)
    wr = torch.randn(E, H, generator=g).to(dt)
    wg, wu = ((torch.randn(E, I, H, generator=g) * 0.1).to(dt) for _ in range(2))
    wd = (torch.randn(E, H, I, generator=g) * 0.1).to(dt)
    ids, scores, logits = o.router_topk(x32.to(DEV), wr.to(DEV), k, True)
    ref_logits = x32 @ wr.float().T
    close(logits, ref_logits, 1e-5, "router logits")
    # the reference choice computed from the kernel's own logits: ties and order must agree exactly
    ref_ids, ref_scores = plain.router_top_k(logits.cpu(), k)
    assert torch.equal(ids.cpu().long(), ref_ids), "top-k choice or its order differs"
    close(scores, ref_scores, 1e-6, "sigmoid scores")
    plan = o.moe_plan(ids, E)
    offsets, sorted_entry, slot_of_entry = plan
    live = [e for e in range(E) if counts_of(ids, E)[e] > 0]
    assert plan.active.cpu().tolist()[: 1 + len(live)] == [len(live)] + live
    flat = ids.cpu().view(-1).long()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=E)
    assert offsets.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
    assert torch.equal(sorted_entry.cpu()[: n * k].long(), order), "plan is not the stable sort by expert"
    assert torch.equal(slot_of_entry.cpu()[: n * k].long()[order], torch.arange(n * k))
    # experts: per sorted slot
    expert_of_slot = flat[order]
    token_of_slot = order // k
    s = scores.cpu().view(-1)[order]
    gate = torch.einsum("rh,rih->ri", x.float()[token_of_slot], wg.float()[expert_of_slot]) * s[:, None]
    up = torch.einsum("rh,rih->ri", x.float()[token_of_slot], wu.float()[expert_of_slot]) * s[:, None]
    act_ref = gate * torch.sigmoid(gate) * up
    for few in (True, False):
        act = o.moe_gate_up(x.to(DEV), plan, k, wg.to(DEV), wu.to(DEV), scores, few)
        close(act, act_ref, tol, f"gate/up few={few}")
        a = act_ref.to(dt)
        y = o.moe_down(a.to(DEV), wd.to(DEV), plan, few)
        y_ref = torch.einsum("ri,rhi->rh", a.float(), wd.float()[expert_of_slot])
        close(y, y_ref, 1e-5 if dt == torch.float32 else 1e-5, f"down few={few}")
    shared = torch.randn(n, H, generator=g).to(dt)
    out = o.moe_combine(y, slot_of_entry, shared.to(DEV), n, k)
    want = shared.float() + y_ref[slot_of_entry.cpu()[: n * k].long()].view(n, k, H).sum(1)
    close(out, want, 1e-5, "combine")


@pytest.mark.parametrize("shape", [(256, 4, 1, 128, 300), (5120, 16, 1, 512, 2048), (192, 8, 2, 96, 700), (136, 3, 2, 72, 50),
                                   (1024, 5, 1, 1032, 1000), (64, 2, 1, 64, 129), (256, 4, 1, 2112, 100),
                                   (128, 2, 2, 2048, 40), (5120, 4, 1, 1024, 100), (2432, 10, 1, 1600, 300),
                                   (2560, 8, 2, 1536, 60), (1280, 16, 1, 1536, 64)])
def test_expert_products_on_tcgen05(shape):
    """The tcgen05 grouped products (TMA + tensor memory) against float32 references: token counts
    per expert above and below a tile and a slot of tensor memory, widths that are no multiple of
    the tile, K tails, and (from the seventh shape on) a long K with tiles that do not fill the last
    round over the SMs, where the down projection cuts those tiles along K into two, three or four
    pieces (with and without full rounds before them) and the piece that arrives last adds them:
    the same bits on every call."""
    o = ops()
    H, E, k, I, n = shape
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(H + n)
    x = torch.randn(n, H, generator=g).to(dt)
    wg, wu = ((torch.randn(E, I, H, generator=g) * 0.1).to(dt) for _ in range(2))
    wd = (torch.randn(E, H, I, generator=g) * 0.1).to(dt)
    logits = torch.randn(n, E, generator=g)
    logits[:, 0] += 1.5                                        # uneven load: expert 0 gets most rows
    ids, ref_scores = plain.router_top_k(logits, k)
    ids_d = ids.to(torch.int32).to(DEV)
    scores = ref_scores.float().to(DEV).contiguous()
    plan = o.moe_plan(ids_d, E)
    assert o.moe_tc_supported(x.to(DEV), wg.to(DEV))
    flat = ids.view(-1)
    order = torch.sort(flat, stable=True).indices
    expert_of_slot, token_of_slot = flat[order], order // k
    s = ref_scores.reshape(-1)[order].float()
    gate = torch.einsum("rh,rih->ri", x.float()[token_of_slot], wg.float()[expert_of_slot]) * s[:, None]
    up = torch.einsum("rh,rih->ri", x.float()[token_of_slot], wu.float()[expert_of_slot]) * s[:, None]
    act_ref = gate * torch.sigmoid(gate) * up
    act = o.moe_gate_up_tc(x.to(DEV), plan, k, wg.to(DEV), wu.to(DEV), scores)
    o.check_tc_status()
    close(act, act_ref, 2e-2, f"tcgen05 gate/up {shape}")
    a = act_ref.to(dt)
    a_d, wd_d = a.to(DEV), wd.to(DEV)
    y = o.moe_down_tc(a_d, wd_d, plan)
    o.check_tc_status()
    y_ref = torch.einsum("ri,rhi->rh", a.float(), wd.float()[expert_of_slot])
    close(y, y_ref, 2e-5, f"tcgen05 down {shape}")
    for _ in range(3):                 # pieces arrive in another order; their counters were left at zero
        again = o.moe_down_tc(a_d, wd_d, plan)
        o.check_tc_status()
        assert torch.equal(again, y), f"tcgen05 down {shape}: two calls differ"
    # and against the general kernels on the same inputs
    close(o.moe_gate_up(x.to(DEV), plan, k, wg.to(DEV), wu.to(DEV), scores, False), act_ref, 2e-2, "general gate/up")
    assert not o.moe_tc_supported(x.float().to(DEV), wg.float().to(DEV))


@pytest.mark.parametrize("shape", [(1288, 16, 200), (5120, 16, 257), (328, 40, 230), (2048, 5, 192)])
def test_router_logits_do_not_depend_on_the_number_of_tokens(shape):
    """The many-token router kernel and the one-token kernel add in the same order: the logits of
    a token are the same bits whether it is routed in a long step or in a short one."""
    o = ops()
    H, E, n = shape
    g = torch.Generator().manual_seed(H + E)
    x = torch.randn(n, H, generator=g).to(DEV)
    for wdt in (torch.bfloat16, torch.float32):
        w = torch.randn(E, H, generator=g).to(wdt).to(DEV)
        ids_all, _, logits_all = o.router_topk(x, w, 2, True)                 # n >= 192: the tiled kernel
        for lo in range(0, n, 37):
            ids, _, logits = o.router_topk(x[lo:lo + 37].contiguous(), w, 2, True)   # few rows: one block per token
            assert torch.equal(logits, logits_all[lo:lo + 37]), f"{shape} {wdt}: logits differ between the kernels"
            assert torch.equal(ids, ids_all[lo:lo + 37])
        close(logits_all, x.float() @ w.float().T, 1e-5, "router logits")


@pytest.mark.parametrize("shape", [(96, 5, 2, 1), (200, 16, 1, 8), (72, 40, 3, 33), (128, 128, 1, 150), (64, 24, 2, 200),
                                   (100, 6, 2, 5000)])     # an odd width keeps a long step on the few-token kernel
def test_router_and_plan_in_one_call_match_the_two_calls(shape):
    """With few tokens the plan is made by the router kernel's last block; launches follow one
    another so the block counter has to come back to zero every time."""
    o = ops()
    H, E, k, n = shape
    g = torch.Generator().manual_seed(H + E + n)
    w = torch.randn(E, H, generator=g).to(torch.bfloat16).to(DEV)
    for turn in range(4):
        x = torch.randn(n, H, generator=g).to(DEV)
        ids, scores, _ = o.router_topk(x, w, k)
        plan = o.moe_plan(ids, E)
        ids2, scores2, plan2 = o.router_plan(x, w, k)
        assert torch.equal(ids, ids2) and torch.equal(scores, scores2)
        m = n * k
        n_active = int(plan.active[0])
        assert torch.equal(plan.offsets, plan2.offsets), f"{shape} turn {turn}"
        assert torch.equal(plan.sorted_entry[:m], plan2.sorted_entry[:m])
        assert torch.equal(plan.slot_of_entry[:m], plan2.slot_of_entry[:m])
        assert torch.equal(plan.active[: 1 + n_active], plan2.active[: 1 + n_active])
    empty = o.router_plan(torch.zeros(0, H, device=DEV), w, k)[2]
    assert empty.offsets.cpu().tolist() == [0] * (E + 1) and int(empty.active[0]) == 0


def test_router_ties_go_to_the_lower_id():
    o = ops()
    x = torch.zeros(3, 16); x[:, 0] = 1.0
    w = torch.zeros(6, 16)
    w[:, 0] = torch.tensor([0.5, 2.0, 2.0, -1.0, 2.0, 0.5])
    ids, scores, _ = o.router_topk(x.to(DEV), w.to(DEV), 4)
    assert ids.cpu().tolist() == [[1, 2, 4, 0]] * 3
    close(scores[0], torch.sigmoid(torch.tensor([2.0, 2.0, 2.0, 0.5])), 1e-6)


def test_greedy_rows_cut_over_many_blocks():
    """Every row greedy and a large vocabulary: each row is read by several blocks and the last
    one picks. Ties across parts go to the lower id; calls follow one another (the counters come
    back to zero); more rows than the scratch holds take the one-block kernel."""
    o = ops()
    g = torch.Generator().manual_seed(9)
    for rows, vocab in ((1, 8192), (8, 202048), (5, 8193), (64, 33333), (1100, 9000)):
        for turn in range(3):
            logits = torch.randn(rows, vocab, generator=g)
            logits[0, vocab - 1] = logits[0, 7] = 50.0                 # first and last part tie
            if rows > 2:
                logits[2] = -float("inf")                              # nothing finite: id 0
                logits[1, vocab // 2 + 1] = float("nan")
            got = o.sample_rows(logits.to(DEV), None, None).cpu()
            want = torch.stack([torch.argmax(torch.nan_to_num(r, nan=-float("inf"))) for r in logits])
            if rows > 2:
                want[2] = 0
            assert got[0] == 7
            assert torch.equal(got.long(), want), f"rows {rows} vocab {vocab} turn {turn}"


def test_ranked_rows_follow_the_host_sampler():
    """top-k / top-p on the GPU against the host's rule, row by row: peaked and flatter rows, ties,
    several vocabularies; rows that are not ranked stay as they were; a row with more candidates
    than the kernel sorts comes back as -1."""
    from hi_b200.sampling import ranked_sample

    o = ops()
    g = torch.Generator().manual_seed(31)
    handed_back = 0
    for vocab, scale in ((17, 2.0), (515, 3.0), (5000, 1.0), (50000, 4.0), (202048, 3.0), (202048, 6.0)):
        rows = 12
        logits = torch.randn(rows, vocab, generator=g) * scale
        logits[1, 3] = logits[1, vocab - 2] = logits[1].max() + 1.0          # the two largest tie
        logits[2, : min(vocab, 40)] = 5.0 * scale                             # a run of equal words
        temps = torch.tensor([0.7, 1.0, 1.3, 0.5, 1.0, 0.0, 0.9, 1.0, 2.0, 1.0, 0.8, 1.0])
        top_ps = torch.tensor([0.9, 0.5, 1.0, 0.1, 0.95, 0.9, 1.0, 0.3, 0.8, 1.0, 0.999, 0.6])
        top_ks = torch.tensor([0, 5, 50, 0, 3, 7, 0, 1, 20, vocab + 5, 0, 64], dtype=torch.int32)
        for turn in range(3):
            us = torch.rand(rows, generator=g)
            before = torch.full((rows,), -7, dtype=torch.int32)
            out = before.to(DEV)
            o.ranked_rows(logits.to(DEV), temps.to(DEV), top_ps.to(DEV), top_ks.to(DEV), us.to(DEV), out)
            got = out.cpu().tolist()
            for r in range(rows):
                k = int(top_ks[r])
                is_ranked = float(temps[r]) > 0 and ((0 < k < vocab) or 0.0 < float(top_ps[r]) < 1.0)
                if not is_ranked:
                    assert got[r] == -7, f"row {r} is not ranked and was touched"
                    continue
                want = ranked_sample(logits[r].numpy(), float(temps[r]), float(top_ps[r]), k or None, float(us[r]))
                if got[r] == -1:
                    handed_back += 1
                    assert not (0 < k <= 64), f"vocab {vocab} row {r}: a small top-k was handed back"
                    continue
                assert got[r] == want, f"vocab {vocab} scale {scale} row {r} turn {turn}: {got[r]} != {want}"
    assert handed_back < 30, "too many rows went back to the host"
    # a flat row with a wide top-p has more candidates than the kernel sorts
    flat = torch.zeros(1, 5000)
    out = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.ranked_rows(flat.to(DEV), torch.ones(1, device=DEV), torch.full((1,), 0.9, device=DEV),
                  torch.zeros(1, dtype=torch.int32, device=DEV), torch.full((1,), 0.5, device=DEV), out)
    assert int(out[0]) == -1


def test_sampling_kernel_matches_the_plain_sampler():
    o = ops()
    g = torch.Generator().manual_seed(5)
    for vocab in (17, 515, 1024, 50000):
        logits = torch.randn(8, vocab, generator=g) * 3
        logits[2, vocab // 2] = logits[2, 3] = 40.0            # a tie: the lower id wins
        got = o.sample_rows(logits.to(DEV), None, None).cpu().tolist()
        assert got == [int(torch.argmax(r)) for r in logits] and got[2] == 3
        temps = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.5, 2.0, 0.9, 1.0])
        us = torch.tensor([0.1, 0.5, 0.9, 0.3, 0.999, 0.0, 0.25, 0.75])
        got = o.sample_rows(logits.to(DEV), temps.to(DEV), us.to(DEV)).cpu().tolist()
        want = [plain.sample(logits[i], float(temps[i]), 1.0, 0, float(us[i])) for i in range(8)]
        assert got == want, f"vocab {vocab}: {got} != {want}"


def test_sampling_with_rows_cut_over_many_blocks():
    """Few rows of a large vocabulary are cut over 16 blocks each and the block that finishes last
    picks. The pick must be the word at which the running sum of the weights, in vocabulary order,
    passes u * total: checked in float64, with 2e-5 of the total for the kernel's float32 sums (the
    choice is a threshold on a sum of 200,000 terms; u = 0 and a row whose whole weight is one word
    are checked exactly). Peaked and flat rows, rows that are greedy beside rows that sample, logits
    that are not finite, parts without any weight, and the same again on later calls (the counters
    were left at zero)."""
    o = ops()
    g = torch.Generator().manual_seed(77)
    for vocab, rows in ((8192, 5), (50000, 16), (202048, 8), (202049, 3)):
        logits = torch.randn(rows, vocab, generator=g) * torch.linspace(0.5, 6.0, rows)[:, None]
        logits[0, vocab - 1] = 200.0                              # all of the weight in the last word
        logits[1, 5] = float("-inf")
        if rows > 3:
            logits[3, : vocab // 2] = float("-inf")               # whole parts without weight
        temps = torch.tensor([0.7, 0.0, 1.0, 1.3, 0.5, 2.0, 0.9, 1.0, 0.0, 0.3, 1.0, 1.0, 5.0, 1.0, 0.8, 1.1][:rows])
        for turn in range(3):
            us = torch.rand(rows, generator=g)
            us[turn % rows] = 0.0
            us[(turn + 1) % rows] = 0.99999994
            got = o.sample_rows(logits.to(DEV), temps.to(DEV), us.to(DEV)).cpu().tolist()
            for r in range(rows):
                what = f"vocab {vocab} turn {turn} row {r}: picked {got[r]}"
                if not float(temps[r]) > 0:
                    assert got[r] == int(torch.argmax(logits[r])), what
                    continue
                z = (logits[r] / float(temps[r])).double()
                w = torch.exp(z - z[torch.isfinite(z)].max())
                w[~torch.isfinite(z)] = 0.0
                total = float(w.sum())
                before = float(w[: got[r]].sum())
                target = float(us[r]) * total
                assert float(w[got[r]]) > 0, what + ", a word without weight"
                if float(us[r]) == 0.0:
                    first = int(torch.nonzero(torch.exp((z - z[torch.isfinite(z)].max()).float()) > 0)[0])
                    assert got[r] == first, what + f", not the first word with a float32 weight ({first})"
                else:
                    assert before <= target + 2e-5 * total and target < before + float(w[got[r]]) + 2e-5 * total, \
                        what + f": sum before {before / total:.7f}, its weight {float(w[got[r]]) / total:.2e}, u {float(us[r]):.7f}"
            assert got[0] == vocab - 1


def test_kernels_refuse_what_they_cannot_do():
    o = ops()
    from hi_b200.kernels.ops import KernelError

    with pytest.raises(KernelError):
        o.embed_gather(torch.zeros(4, 4), torch.zeros(1, dtype=torch.int32))        # not on the GPU
    q = torch.zeros(1, 2, 24, device=DEV)
    pages = torch.zeros(1, 2, 4, 24, device=DEV)
    bt = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError):
        o.paged_attention(q, pages, pages, bt, z, z, 0, 0, 1.0)                     # head_dim 24
    with pytest.raises(KernelError):
        o.router_topk(torch.zeros(2, 8, device=DEV), torch.zeros(3, 8, device=DEV), 4)   # k > experts


def test_random_fill_has_the_hosts_bits():
    """hb_random_normal against the same arithmetic written out in numpy (and the host runtime's
    C++): float32 and bfloat16, sizes that are no multiple of anything, an offset into the tensor,
    indices past 2^32."""
    import numpy as np

    from hi_b200.weights import random_values as rv

    o = ops()
    for n, first, std, seed in ((1, 0, 0.02, 0), (1023, 0, 0.02, 1), (70001, 7, 0.08, 2), (4096, (1 << 33) + 5, 1.0, 3)):
        key = rv.tensor_key(seed, f"t{n}")
        want = rv.normal_values_numpy(key, first, n, std)
        assert (rv.normal_values(key, first, n, std).view(np.uint32) == want.view(np.uint32)).all()
        got32 = o.random_normal(torch.empty(n, dtype=torch.float32, device=DEV), key, float(rv.scale_for(std)), first)
        assert (got32.cpu().numpy().view(np.uint32) == want.view(np.uint32)).all(), f"float32, n {n}"
        got16 = o.random_normal(torch.empty(n, dtype=torch.bfloat16, device=DEV), key, float(rv.scale_for(std)), first)
        assert torch.equal(got16.cpu(), torch.from_numpy(want).to(torch.bfloat16)), f"bfloat16, n {n}"


@pytest.mark.parametrize("shape", [(40, 8, 128, 64, 8192, True, True, False), (40, 8, 128, 64, 0, False, False, True),
                                   (8, 8, 64, 16, 0, True, False, False), (32, 2, 64, 32, 512, True, True, True),
                                   (16, 1, 128, 128, 64, False, True, False), (12, 4, 64, 16, 128, True, True, True)])
def test_fused_decode_attention_equals_its_three_kernels(shape):
    """hb_attention_decode_fused (encoding of q, k and v, cache append, attention, merge of the splits,
    one launch) against qkv_post + the decode kernel + the merge kernel on the same inputs: the keys
    and values it appends are the same bits, the outputs agree to bfloat16 rounding, and its counters
    are zero again. Requests of very different lengths in one batch (one split and many), positions
    on and beside page, tile and chunk edges; twice in a row on the same buffers."""
    o = ops()
    nh, nkv, hd, page, chunk, rope, norm, temp = shape
    starts = [0, 1, 63, 64, 255, 256, 1030, 2500, 8191, 8192, 8200]
    S = len(starts)
    total = [s + 1 for s in starts]
    g = torch.Generator().manual_seed(nh * 7 + hd)
    n_pages = sum(-(-t // page) for t in total) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-t // page) for t in total)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    c = 0
    for s in range(S):
        for b in range(-(-total[s] // page)):
            bt[s, b] = perm[c]; c += 1
    dt = torch.bfloat16
    kp = (torch.randn(n_pages, nkv, page, hd, generator=g)).to(dt)      # whatever earlier steps left, and stale rows
    vp = (torch.randn(n_pages, nkv, page, hd, generator=g)).to(dt)
    qkv = (torch.randn(S, (nh + 2 * nkv) * hd, generator=g) * 1.5).to(dt).to(DEV)
    pos = torch.tensor(starts, dtype=torch.int32).to(DEV)
    sot = torch.arange(S, dtype=torch.int32).to(DEV)
    inv = plain.rope_inverse_frequencies(hd, 10000.0, None).to(DEV) if rope else None
    temperature = (16.0, 0.1) if temp else None
    interleaved = bool(nh % 3 == 0)
    bt = bt.to(DEV)
    for _round in range(2):
        k1, v1, k2, v2 = kp.to(DEV), vp.to(DEV), kp.to(DEV), vp.to(DEV)
        q = o.qkv_post(qkv, nh, nkv, hd, pos, inv, interleaved, norm, 1e-6, temperature, sot, bt, k1, v1, page, True)
        want = o.decode_attention(q, k1, v1, bt, sot, pos, chunk, 0, hd ** -0.5, max(total))
        got = o.decode_attention_fused(qkv, nh, nkv, hd, pos, inv, interleaved, norm, 1e-6, temperature, sot, bt, k2, v2,
                                       chunk, 0, hd ** -0.5, max(total))
        assert got is not None, "the fused kernel refused shapes it is written for"
        torch.cuda.synchronize()
        assert torch.equal(k1, k2) and torch.equal(v1, v2), "the appended keys or values differ"
        close(got, want, 1e-2, f"fused decode attention {shape}")
        assert int(o._fused_counter_buffer(torch.device(DEV)).abs().sum()) == 0, "the counters were not left at zero"
    o.check_tc_status()
    # a sliding window is not taken: the caller falls back
    assert o.decode_attention_fused(qkv, nh, nkv, hd, pos, inv, interleaved, norm, 1e-6, temperature, sot, bt, k2, v2,
                                    0, 100, hd ** -0.5, max(total)) is None


@pytest.mark.parametrize("n,experts", [(1, 4), (255, 16), (256, 16), (2048, 16), (2047, 128), (5000, 5), (9001, 300), (300, 4000)])
def test_plan_is_a_stable_sort_by_expert(n, experts):
    """The device-side plan against a stable argsort on the host: offsets, the entry of every
    sorted slot, the slot of every entry, and the list of experts that have rows; with one warp
    ranking (few entries, or more experts than fit) and with all of them."""
    import numpy as np

    o = ops()
    g = torch.Generator().manual_seed(n + experts)
    ids = torch.randint(0, experts, (n,), generator=g, dtype=torch.int32)
    if n > 100:
        ids[ids == 3] = 2                                   # an expert without rows
    plan = o.moe_plan(ids.to(DEV), experts)
    order = np.argsort(ids.numpy(), kind="stable")
    counts = np.bincount(ids.numpy(), minlength=experts)
    assert plan.offsets.cpu().tolist() == [0] + np.cumsum(counts).tolist()
    assert plan.sorted_entry.cpu().numpy()[:n].tolist() == order.tolist()
    inverse = np.empty(n, dtype=np.int64)
    inverse[order] = np.arange(n)
    assert plan.slot_of_entry.cpu().numpy()[:n].tolist() == inverse.tolist()
    active = plan.active.cpu().tolist()
    assert active[0] == int((counts > 0).sum()) and active[1: 1 + active[0]] == np.nonzero(counts)[0].tolist()
