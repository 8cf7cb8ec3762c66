"""The allocation-free decode attention entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory when they need attention: a serving
loop that owns all GPU memory in its own pools and forbids cudaMalloc (which also stalls every
stream of the device), or a C/C++ program that links the kernels without torch and so has no
caching allocator.  For them `rllm_paged_flash_decode_static` keeps the split-key partials in a
fixed array inside the library.  This test checks that it gives the same output as the regular
entry point (which takes caller-allocated scratch) and as the plain implementation of attention,
on calls in a row that share the array (both decode kernels: tiles of 8 and of 16 rows), that the
device's free memory does not move across its calls (it allocates nothing), and that it refuses a
problem larger than the array with a clear message.

The file is named to be collected last: a run that stops at the first failure has then already
run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOO_LARGE = 20001


def make_case(seed, hd, H, K, bs, lens):
    """Pure decode: one query token per request at the end of a context of `lens` tokens, pages
    scattered over the pool."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    n_pages = sum(-(-L // bs) for L in lens) + 5
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.randn(n_pages, K, bs, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(n_pages, K, bs, hd, generator=g).to(torch.bfloat16)
    width = max(-(-L // bs) for L in lens)
    table = torch.zeros(R, width, dtype=torch.int32)
    for r, L in enumerate(lens):
        for b in range(-(-L // bs)):
            table[r, b] = perm.pop()
    q = torch.randn(R, H * hd, generator=g).to(torch.bfloat16)
    pos = torch.tensor([L - 1 for L in lens], dtype=torch.int32)
    cu = torch.arange(R + 1, dtype=torch.int32)
    tiles = torch.arange(R, dtype=torch.int32)
    return {k: v.to(DEV) for k, v in dict(q=q, kc=kc, vc=vc, table=table, pos=pos, cu=cu, tiles=tiles).items()}


def call_static(lib, c, H, K, hd, bs, n_splits, split_keys=128, out=None):
    out = torch.full_like(c["q"], float("nan")) if out is None else out
    g = H // K
    p = lambda t: c_void_p(t.data_ptr())
    rc = lib.rllm_paged_flash_decode_static(
        p(c["q"]), p(c["kc"]), p(c["vc"]), p(out), p(c["pos"]), p(c["cu"]), p(c["table"]),
        c_int(c["table"].stride(0)), p(c["tiles"]), p(c["tiles"]), c_int(c["q"].shape[0]), c_int(H), c_int(K),
        c_int(hd), c_int(bs), c_float(1.0 / math.sqrt(hd)), c_int(0), c_int(1), c_int(min(g, 16)),
        c_int(-(-g // min(g, 16))), c_int(split_keys), c_int(n_splits),
        c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def call_regular(c, H, K, hd, bs, n_splits):
    from rllm_b200.csrc import ops
    out = torch.full_like(c["q"], float("nan"))
    g = H // K
    ops.paged_flash_attention(c["q"], c["kc"], c["vc"], out, c["pos"], c["cu"], c["table"], c["tiles"],
                              c["tiles"], c["q"].shape[0], H, K, hd, bs, 1.0 / math.sqrt(hd), 0, 1, 1,
                              min(g, 16), -(-g // min(g, 16)), 128, n_splits)
    return out


def plain_decode_attention(c, H, K, hd, bs, lens):
    """The plain implementation (whole sequences, no pages) on the keys and values gathered from
    the pages of each request; the query of the last position is the one the kernels got."""
    import plain_impl
    q, kc, vc, table = (c[k].float().cpu() for k in ("q", "kc", "vc", "table"))
    out = torch.zeros(len(lens), H * hd)
    for r, L in enumerate(lens):
        pages = [int(table[r, p // bs]) for p in range(L)]
        k = torch.stack([kc[pages[p], :, p % bs, :] for p in range(L)])        # [L, K, hd]
        v = torch.stack([vc[pages[p], :, p % bs, :] for p in range(L)])
        qs = torch.zeros(L, H, hd)
        qs[L - 1] = q[r].view(H, hd)
        out[r] = plain_impl.attention(qs, k, v, 1.0 / math.sqrt(hd))[L - 1].reshape(-1)
    return out


def test_static_scratch_entry_point_matches_regular_one():
    from rllm_b200.csrc import build
    lib = ctypes.CDLL(str(build.build("attn")))
    lib.rllm_paged_flash_decode_static.restype = c_int
    lib.rllm_paged_flash_decode_static_error.restype = ctypes.c_char_p

    # two calls in a row on the shared array: a large problem, then a smaller one with other sizes,
    # so that anything read from the first call's leftovers would show
    # (the third has 16 query heads per key/value head: the decode kernel with 16-row tiles)
    cases = [(31, 128, 8, 2, 16, [700, 129, 1, 333, 512]), (32, 64, 6, 2, 8, [90, 260, 17]),
             (34, 128, 16, 1, 32, [301, 64, 150])]
    for seed, hd, H, K, bs, lens in cases:
        c = make_case(seed, hd, H, K, bs, lens)
        n_splits = -(-max(lens) // 128)
        rc, got = call_static(lib, c, H, K, hd, bs, n_splits)
        assert rc == 0, lib.rllm_paged_flash_decode_static_error()
        torch.cuda.synchronize()
        want = call_regular(c, H, K, hd, bs, n_splits)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # same kernels, same order of operations: the tolerance of the attention kernel tests (1.5e-2
        # of the largest value) is far from needed, the outputs are expected to be equal
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= 1.5e-2
        assert torch.equal(got, want)
        # and against the plain implementation, within the tolerance of the attention kernel tests
        plain = plain_decode_attention(c, H, K, hd, bs, lens)
        assert float((got.float().cpu() - plain).abs().max() / plain.abs().max()) <= 1.5e-2
        # it allocates nothing: across further calls (the first one looked the array's address up) into an
        # output that exists already, the device's free memory stays where it was
        again = torch.full_like(c["q"], float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        for _ in range(3):
            rc, _ = call_static(lib, c, H, K, hd, bs, n_splits, out=again)
            assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(again, want)

    # larger than the array: refused with a message, nothing launched
    c = make_case(33, 128, 8, 8, 16, [40] * 64)
    rc, _ = call_static(lib, c, 8, 8, 128, 16, n_splits=512)
    assert rc == TOO_LARGE
    msg = lib.rllm_paged_flash_decode_static_error().decode()
    assert "static scratch holds" in msg and "262144" in msg
    torch.cuda.synchronize()
