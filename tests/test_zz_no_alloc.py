"""hb_attention_decode_static, the entry point that allocates nothing, called through its
exported C symbol the way a host program without an allocator to spare would call it: inputs
and output only. Its result must equal the allocating entry point's, on two calls in a row that
share the library's built-in scratch (the second with other sizes, so that what the first left
behind lies under it). This file sorts last on purpose: a run that stops at the first failure
has then already run every other test."""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HB_ERR_SCRATCH_CAPACITY = 1003


def library():
    from hi_b200.kernels import build

    lib = build.library()
    fn = lib.hb_attention_decode_static
    fn.argtypes = [c_void_p] * 3 + [c_void_p, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_int, c_int,
                                                                                                 c_void_p]
    fn.restype = c_int
    lib.hb_attention_decode_static_need.argtypes = [c_int] * 4
    lib.hb_attention_decode_static_need.restype = c_longlong
    lib.hb_attention_decode_static_fits.argtypes = [c_int] * 4
    lib.hb_attention_decode_static_fits.restype = c_int
    return lib


def case(seed, n, nh, nkv, hd, page, lengths):
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-l // page) for l in lengths]
    n_pages = sum(blocks) + 1
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    c = 0
    for s in range(n):
        for b in range(blocks[s]):
            bt[s, b] = perm[c]; c += 1
    kp = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16)
    vp = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16)
    q = (torch.randn(n, nh, hd, generator=g) * 2).to(torch.bfloat16)
    pos = torch.tensor([l - 1 for l in lengths], dtype=torch.int32)
    return [t.to(DEV) for t in (q, kp, vp, bt, torch.arange(n, dtype=torch.int32), pos)]


def call_static(lib, q, kp, vp, bt, sot, pos, chunk, window, scale, split_size, splits):
    n, nh, hd = q.shape
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.hb_attention_decode_static(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), bt.data_ptr(), bt.shape[1],
                                        sot.data_ptr(), pos.data_ptr(), out.data_ptr(), n, nh, kp.shape[1], hd,
                                        kp.shape[2], chunk, window, scale, split_size, splits, stream)
    return rc, out


def test_static_entry_point_matches_the_allocating_one_twice_in_a_row():
    from hi_b200.kernels import ops

    lib = library()
    # first call: 3 requests, 7 splits of 256 keys; second: other sizes and fewer, longer splits
    for seed, (n, nh, nkv, hd, page, lengths, chunk, window, split_size) in enumerate((
            (3, 40, 8, 128, 64, [1700, 300, 1], 0, 0, 256),
            (5, 8, 2, 64, 16, [900, 64, 65, 1, 513], 0, 400, 128))):
        q, kp, vp, bt, sot, pos = case(seed, n, nh, nkv, hd, page, lengths)
        longest = max(lengths) if not window else min(max(lengths), window)
        splits = -(-longest // split_size)
        assert splits > 1
        assert lib.hb_attention_decode_static_need(n, nh, hd, splits) == n * nh * splits * (hd + 2)
        rc, got = call_static(lib, q, kp, vp, bt, sot, pos, chunk, window, hd ** -0.5, split_size, splits)
        assert rc == 0, f"hb_attention_decode_static returned {rc}"
        want = ops.decode_attention(q, kp, vp, bt, sot, pos, chunk, window, hd ** -0.5, max(lengths))
        general = ops.paged_attention(q, kp, vp, bt, sot, pos, chunk, window, hd ** -0.5, max(lengths))
        torch.cuda.synchronize()
        scale = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= 2e-2 * scale, "static and allocating entry points differ"
        assert float((got.float() - general.float()).abs().max()) <= 2e-2 * scale
        assert torch.isfinite(got.float()).all()


def test_static_entry_point_refuses_what_its_scratch_cannot_hold():
    lib = library()
    q, kp, vp, bt, sot, pos = case(9, 2, 40, 8, 128, 64, [200, 100])
    # 2 tokens x 40 heads x 400 splits x 128 dims is more than the built-in array holds
    rc, _ = call_static(lib, q, kp, vp, bt, sot, pos, 0, 0, 128 ** -0.5, 64, 400)
    assert rc == HB_ERR_SCRATCH_CAPACITY
    # each part of the scratch has its own bound: 2 x 40 x 205 rows of 128 floats are 2,048 floats more than
    # the part for partial outputs holds, although both parts together would have room for them
    assert lib.hb_attention_decode_static_fits(2, 40, 128, 204) == 1
    assert lib.hb_attention_decode_static_fits(2, 40, 128, 205) == 0
    assert lib.hb_attention_decode_static_need(2, 40, 128, 205) <= (1 << 21) + (1 << 16)
    rc, _ = call_static(lib, q, kp, vp, bt, sot, pos, 0, 0, 128 ** -0.5, 64, 205)
    assert rc == HB_ERR_SCRATCH_CAPACITY
    # one split needs no scratch at all
    rc, got = call_static(lib, q, kp, vp, bt, sot, pos, 0, 0, 128 ** -0.5, 256, 1)
    assert rc == 0 and torch.isfinite(got.float()).all()
