"""The decode attention entry point that allocates nothing, called through its exported C symbol.

Some users of the library's C functions cannot allocate device memory when they call: a serving loop
must not hit the device-wide synchronisation of cudaMalloc, and a process that gave all memory to the
page pool has none left to ask for.  ``jk_attention_decode_static`` serves them with a scratch array
built into the library.  This test calls it twice in a row (the array keeps the first call's
contents) and compares both results with the ordinary entry point, which takes its scratch from the
caller, and with the plain implementation.  The file sorts last on purpose: a run that stops at
the first failure has then run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_FLOATS = 1 << 20


def _case(seed, nh, nkvh, dh, page, lens, window=0):
    """Random queries (one decoded token per request), pages and block tables on the device."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    max_blocks = (max(lens) + page - 1) // page + 1
    num_pages = R * max_blocks + 1
    bf = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).to(DEV)
    q = bf(R, nh * dh)
    k_pages, v_pages = bf(num_pages, nkvh, page, dh), bf(num_pages, nkvh, page, dh)
    table = (torch.randperm(R * max_blocks, generator=g) + 1).view(R, max_blocks).to(torch.int32).to(DEV)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    row_req = torch.arange(R, dtype=torch.int32, device=DEV)
    return q, k_pages, v_pages, table, positions, row_req


def _call_static(lib, q, k_pages, v_pages, out, positions, row_req, table, nh, scale, window, splits):
    _, nkvh, page, dh = k_pages.shape
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i = ctypes.c_int
    return lib.jk_attention_decode_static(
        p(q), p(k_pages), p(v_pages), p(out), ctypes.c_void_p(0), i(q.shape[0]), p(positions), p(row_req), p(table),
        i(table.shape[1]), i(page), i(nh), i(nkvh), i(dh), ctypes.c_float(scale), i(window), i(splits),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _plain(q, k_pages, v_pages, table, lens, nh, window):
    """The same attention by the plain implementation: each request's keys gathered from its pages, float64."""
    from plain_minicpm import plain_attention
    _, nkvh, page, dh = k_pages.shape
    rows = []
    for r, n in enumerate(lens):
        idx = torch.arange(n)
        pages = table[r].cpu()[idx // page].long()
        k = k_pages.cpu()[pages, :, idx % page].double()             # [n, nkvh, dh]
        v = v_pages.cpu()[pages, :, idx % page].double()
        qr = torch.zeros(n, nh, dh, dtype=torch.float64)
        qr[n - 1] = q[r].cpu().double().view(nh, dh)                 # the decoded token is the request's last position
        rows.append(plain_attention(qr, k, v, dh ** -0.5, window or None)[n - 1].reshape(nh * dh))
    return torch.stack(rows)


def test_static_scratch_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row():
    from infinicore_infer_b200 import kernels
    from infinicore_infer_b200.kernels import build
    lib = build.load("attention")                     # the shared object; symbols are taken from it directly
    assert hasattr(lib, "jk_attention_decode_static")
    lib.jk_attention_decode_scratch_floats.restype = ctypes.c_longlong
    # Both problems leave partial results in the built-in array (heads of 128 and heads of 32 never merge inside a
    # cluster), and the second one is smaller: its partials land where the first call's still lie, so a merge
    # that read a stale slot would show.
    cases = [dict(seed=1, nh=8, nkvh=2, dh=128, page=16, lens=[300, 17, 129, 64], splits=5, window=0),
             dict(seed=2, nh=6, nkvh=6, dh=32, page=8, lens=[95, 200], splits=3, window=40)]
    needs = []
    for c in cases:
        q, kp, vp, table, positions, row_req = _case(c["seed"], c["nh"], c["nkvh"], c["dh"], c["page"], c["lens"])
        need = lib.jk_attention_decode_scratch_floats(ctypes.c_int(q.shape[0]), ctypes.c_int(c["nh"]), ctypes.c_int(c["dh"]),
                                                      ctypes.c_int(c["splits"]))
        assert 0 < need <= STATIC_FLOATS
        needs.append(need)
        scale = c["dh"] ** -0.5
        want = torch.empty_like(q)
        kernels.attention_decode(q, kp, vp, want, None, q.shape[0], positions, row_req, table, c["nh"], scale,
                                 c["window"], c["splits"])
        got = torch.full_like(q, 7.0)
        rc = _call_static(lib, q, kp, vp, got, positions, row_req, table, c["nh"], scale, c["window"], c["splits"])
        assert rc == 0, lib.jk_attention_last_error()
        torch.cuda.synchronize()
        # the tolerance of the bfloat16 kernel tests: one rounding of the stored result
        torch.testing.assert_close(got.float(), want.float(), rtol=4e-3, atol=8e-3)
        assert torch.isfinite(got.float()).all()
        plain = _plain(q, kp, vp, table, c["lens"], c["nh"], c["window"])
        torch.testing.assert_close(got.double().cpu(), plain, rtol=4e-3, atol=8e-3)
    assert needs[1] < needs[0]


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from infinicore_infer_b200.kernels import build
    lib = build.load("attention")
    lib.jk_attention_last_error.restype = ctypes.c_char_p
    nh, nkvh, dh, page = 64, 8, 128, 16
    rows = 32
    splits = 8
    assert rows * nh * splits * (dh + 2) > STATIC_FLOATS
    q, kp, vp, table, positions, row_req = _case(3, nh, nkvh, dh, page, [40] * rows)
    out = torch.full_like(q, 3.0)
    rc = _call_static(lib, q, kp, vp, out, positions, row_req, table, nh, dh ** -0.5, 0, splits)
    assert rc != 0
    msg = lib.jk_attention_last_error().decode()
    assert "floats of scratch" in msg and str(STATIC_FLOATS) in msg
    torch.cuda.synchronize()
    assert float(out.float().min()) == 3.0            # nothing was launched
    # with one split no scratch is needed at all, whatever the size
    rc = _call_static(lib, q, kp, vp, out, positions, row_req, table, nh, dh ** -0.5, 0, 1)
    assert rc == 0
