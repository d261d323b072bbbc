"""Each CUDA kernel alone against a plain float64 torch reference, at sizes other than the engine's."""
import math

import pytest
import torch

from plain_minicpm import plain_attention, plain_rmsnorm, plain_rope, plain_sample

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    # float32: summation order only.  bfloat16: one rounding of the stored result (2^-9 relative).
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=4e-3, atol=4e-3)


def _close(got, want, dtype, scale=1.0):
    t = _tol(dtype)
    torch.testing.assert_close(got.double().cpu(), want.double().cpu(), rtol=t["rtol"], atol=t["atol"] * scale)


@pytest.fixture(scope="module")
def K():
    from infinicore_infer_b200 import kernels
    return kernels


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,d,T", [(301, 80, 7), (1000, 2304, 3), (17, 6, 1)])
def test_embed(K, dtype, V, d, T):
    g = torch.Generator().manual_seed(V)
    table = torch.randn(V, d, generator=g).to(dtype)
    tok = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    tok[0] = V - 1
    out = torch.empty(T, d, device=DEV)
    K.embed(tok.to(DEV), table.to(DEV), 2.5, out)
    assert torch.equal(out.cpu(), table.float()[tok.long()] * 2.5)


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("delta_dtype", [None, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d,eps", [(5, 80, 1e-5), (3, 2304, 1e-6), (2, 5000, 3e-6), (1, 14336, 1e-5),
                                     (300, 2304, 1e-6), (261, 1000, 1e-5), (257, 3072, 1e-5), (256, 132, 1e-5), (400, 3076, 1e-5)])
def test_add_rmsnorm(K, out_dtype, delta_dtype, T, d, eps):
    g = torch.Generator().manual_seed(d)
    x = torch.randn(T, d, generator=g) * 3
    w = 1 + 0.1 * torch.randn(d, generator=g)
    delta = None if delta_dtype is None else torch.randn(T, d, generator=g).to(delta_dtype)
    xd = x.to(DEV).clone()
    out = torch.empty(T, d, dtype=out_dtype, device=DEV)
    K.add_rmsnorm(xd, None if delta is None else delta.to(DEV), 0.7, w.to(DEV), eps, out, out_scale=4.0)
    v = x.double() + (0 if delta is None else 0.7 * delta.double())
    _close(xd, v, torch.float32)                       # the sum is written back in float32
    _close(out, 4.0 * plain_rmsnorm(v, w.double(), eps), out_dtype, scale=4.0)


def test_add_rmsnorm_gathers_rows_without_touching_the_stream(K):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 96, generator=g)
    delta = torch.randn(9, 96, generator=g)
    w = torch.ones(96)
    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32)
    xd = x.to(DEV).clone()
    out = torch.empty(4, 96, device=DEV)
    K.add_rmsnorm(xd, delta.to(DEV), 2.0, w.to(DEV), 1e-6, out, rows=rows.to(DEV))
    assert torch.equal(xd.cpu(), x)
    _close(out, plain_rmsnorm((x + 2 * delta).double()[rows.long()], w.double(), 1e-6), torch.float32)
    # many gathered rows (a warp a row)
    x = torch.randn(400, 264, generator=g)
    delta = torch.randn(400, 264, generator=g)
    w = 1 + 0.1 * torch.randn(264, generator=g)
    rows = torch.randint(0, 400, (300,), generator=g).to(torch.int32)
    xd = x.to(DEV).clone()
    out = torch.empty(300, 264, device=DEV)
    K.add_rmsnorm(xd, delta.to(DEV), 2.0, w.to(DEV), 1e-6, out, rows=rows.to(DEV))
    assert torch.equal(xd.cpu(), x)
    _close(out, plain_rmsnorm((x + 2 * delta).double()[rows.long()], w.double(), 1e-6), torch.float32)


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                 (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("T,di", [(3, 136), (1, 5760), (17, 33)])
def test_swiglu(K, in_dtype, out_dtype, T, di):
    g = torch.Generator().manual_seed(di)
    gu = (torch.randn(T, 2 * di, generator=g) * 3).to(in_dtype)
    out = torch.empty(T, di, dtype=out_dtype, device=DEV)
    K.swiglu(gu.to(DEV), out)
    a, b = gu.double()[:, :di], gu.double()[:, di:]
    _close(out, a * torch.sigmoid(a) * b, out_dtype, scale=3.0)


@pytest.mark.parametrize("M,N,K_", [(1, 1, 1), (7, 301, 80), (65, 129, 33), (130, 64, 2304), (3, 1000, 17)])
def test_gemm_f32_is_a_true_float32_product(K, M, N, K_):
    g = torch.Generator().manual_seed(M * N)
    a = torch.randn(M, K_, generator=g)
    w = torch.randn(N, K_, generator=g)
    bias = torch.randn(N, generator=g)
    out = torch.empty(M, N, device=DEV)
    K.gemm_f32(a.to(DEV), w.to(DEV), out, bias.to(DEV))
    want = a.double() @ w.double().T + bias.double()
    # TF32 would be wrong by 2^-11 of |a||w| ~ 5e-4 * sqrt(K); float32 stays below 1e-6 * sqrt(K)
    assert (out.cpu().double() - want).abs().max() <= 2e-6 * math.sqrt(K_) * 4
    # a row's result does not depend on the batch it is in
    if M > 1:
        one = torch.empty(1, N, device=DEV)
        K.gemm_f32(a[M - 1:].contiguous().to(DEV), w.to(DEV), one, bias.to(DEV))
        assert torch.equal(one[0], out[M - 1])


def _scatter_pages(k, v, tables, page, num_pages, dtype, junk=7.0):
    """Dense per-request keys/values [len, nkvh, dh] -> pages [num_pages, nkvh, page, dh]."""
    nkvh, dh = k[0].shape[1:]
    kp = torch.full((num_pages, nkvh, page, dh), junk).to(dtype)       # junk where nothing was written
    vp = torch.full((num_pages, nkvh, page, dh), -junk).to(dtype)
    for r, (kr, vr) in enumerate(zip(k, v)):
        for j in range(kr.shape[0]):
            p = tables[r][j // page]
            kp[p, :, j % page] = kr[j].to(dtype)
            vp[p, :, j % page] = vr[j].to(dtype)
    return kp, vp


@pytest.mark.parametrize("nh,nkvh,dh,page,with_rope", [(4, 2, 64, 16, True), (3, 1, 128, 8, True), (5, 5, 64, 32, False),
                                                        (9, 3, 64, 16, True)])
def test_qkv_product_rotates_and_writes_the_cache_in_its_epilogue(K, pairs, nh, nkvh, dh, page, with_rope):
    """The tcgen05 product of the fused [q | k | v] matrix, rotation and cache write included, against
    a plain product, a plain rotation and a plain scatter."""
    assert K.gemm_tcgen05_qkv_supports(dh) and not K.gemm_tcgen05_qkv_supports(48)
    g = torch.Generator().manual_seed(dh + nh)
    lens = [(37, 150), (0, 131), (200, 3)]              # (start position, rows): tiles of 128 rows straddle requests
    T = sum(n for _, n in lens)
    kdim = 200
    width = (nh + 2 * nkvh) * dh
    act = (torch.randn(T, kdim, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(width, kdim, generator=g) * 0.1).to(torch.bfloat16)
    max_pos, theta = 384, 5000.0
    j = torch.arange(dh // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] / theta ** (j / (dh // 2))
    cos, sin = ang.cos().float(), ang.sin().float()
    max_blocks = max_pos // page
    table = (torch.randperm(3 * max_blocks, generator=g) + 1).view(3, max_blocks).to(torch.int32)
    positions = torch.cat([torch.arange(s, s + n) for s, n in lens]).to(torch.int32)
    row_req = torch.cat([torch.full((n,), i) for i, (_, n) in enumerate(lens)]).to(torch.int32)
    num_pages = 3 * max_blocks + 1
    kp = torch.zeros(num_pages, nkvh, page, dh, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.full((T, nh * dh), 9.0, dtype=torch.bfloat16, device=DEV)
    K.gemm_tcgen05_qkv(act.to(DEV), w.to(DEV), q_out, kp, vp, cos.to(DEV) if with_rope else None,
                       sin.to(DEV) if with_rope else None, positions.to(DEV), row_req.to(DEV), table.to(DEV), nh)
    K.check_gemm_status(DEV)
    x = act.double() @ w.double().T
    q = x[:, :nh * dh].view(T, nh, dh)
    k = x[:, nh * dh:(nh + nkvh) * dh].view(T, nkvh, dh)
    v = x[:, (nh + nkvh) * dh:].view(T, nkvh, dh)
    rot = (lambda t: plain_rope(t, positions, theta)) if with_rope else (lambda t: t)
    _close(q_out.view(T, nh, dh), rot(q), torch.bfloat16, scale=2.0)
    want_k = torch.zeros(num_pages, nkvh, page, dh, dtype=torch.float64)
    want_v = torch.zeros_like(want_k)
    rk = rot(k)
    for t in range(T):
        p = int(table[row_req[t], positions[t] // page])
        want_k[p, :, positions[t] % page] = rk[t]
        want_v[p, :, positions[t] % page] = v[t]
    _close(kp, want_k, torch.bfloat16, scale=2.0)
    _close(vp, want_v, torch.bfloat16, scale=2.0)
    assert float(kp[0].abs().max()) == 0.0              # the null page was not written


@pytest.mark.parametrize("nh,nkvh,dh,page,with_rope,rows", [(4, 2, 64, 16, True, 8), (3, 1, 128, 8, True, 1), (5, 5, 48, 32, False, 16),
                                                             (9, 3, 16, 16, True, 11), (2, 2, 80, 4, True, 5)])
def test_small_row_qkv_product_rotates_and_writes_the_cache_in_its_epilogue(K, nh, nkvh, dh, page, with_rope, rows):
    """The same for at most 16 rows (decoded tokens of several requests): the small-row kernel."""
    kdim = 160
    assert K.linear_small_qkv_supports(rows, kdim, dh) and not K.linear_small_qkv_supports(17, kdim, dh)
    assert not K.linear_small_qkv_supports(rows, kdim, 24)
    g = torch.Generator().manual_seed(dh + nh + rows)
    width = (nh + 2 * nkvh) * dh
    act = (torch.randn(rows, kdim, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(width, kdim, generator=g) * 0.1).to(torch.bfloat16)
    max_pos, theta = 96, 5000.0
    j = torch.arange(dh // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] / theta ** (j / (dh // 2))
    cos, sin = ang.cos().float(), ang.sin().float()
    max_blocks = max_pos // page
    table = (torch.randperm(rows * max_blocks, generator=g) + 1).view(rows, max_blocks).to(torch.int32)
    positions = torch.randint(0, max_pos, (rows,), generator=g).to(torch.int32)      # one decoded token per request
    row_req = torch.arange(rows, dtype=torch.int32)
    num_pages = rows * max_blocks + 1
    kp = torch.zeros(num_pages, nkvh, page, dh, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.full((rows, nh * dh), 9.0, dtype=torch.bfloat16, device=DEV)
    K.linear_small_qkv(act.to(DEV), w.to(DEV), q_out, kp, vp, cos.to(DEV) if with_rope else None,
                       sin.to(DEV) if with_rope else None, positions.to(DEV), row_req.to(DEV), table.to(DEV), nh)
    x = act.double() @ w.double().T
    q = x[:, :nh * dh].view(rows, nh, dh)
    k = x[:, nh * dh:(nh + nkvh) * dh].view(rows, nkvh, dh)
    v = x[:, (nh + nkvh) * dh:].view(rows, nkvh, dh)
    rot = (lambda t: plain_rope(t, positions, theta)) if with_rope else (lambda t: t)
    _close(q_out.view(rows, nh, dh), rot(q), torch.bfloat16, scale=2.0)
    want_k = torch.zeros(num_pages, nkvh, page, dh, dtype=torch.float64)
    want_v = torch.zeros_like(want_k)
    rk = rot(k)
    for t in range(rows):
        p = int(table[row_req[t], positions[t] // page])
        want_k[p, :, positions[t] % page] = rk[t]
        want_v[p, :, positions[t] % page] = v[t]
    _close(kp, want_k, torch.bfloat16, scale=2.0)
    _close(vp, want_v, torch.bfloat16, scale=2.0)
    assert float(kp[0].abs().max()) == 0.0              # the null page was not written


@pytest.mark.parametrize("rows,width,kdim", [(8, 96, 160), (1, 40, 64), (16, 333, 2304), (11, 2304, 5760)])
def test_a_chain_of_few_row_products_carries_the_norm_between_them(K, rows, width, kdim):
    """The product before a norm adds itself into the residual stream, leaves bfloat16(x * norm weight) and the
    rows' sums of squares; the product after it scales its rows by 1 / rms: together they are product, residual
    add, RMSNorm and product, without a norm kernel."""
    assert K.linear_small_norm_supports(rows, width, kdim) and not K.linear_small_norm_supports(17, width, kdim)
    g = torch.Generator().manual_seed(rows + width + kdim)
    act = (torch.randn(rows, kdim, generator=g)).to(torch.bfloat16)
    w = (torch.randn(width, kdim, generator=g) / math.sqrt(kdim)).to(torch.bfloat16)
    x0 = torch.randn(rows, width, generator=g) * 3
    gain = 1 + 0.1 * torch.randn(width, generator=g)
    eps, scale = 1e-5, 0.7
    x = x0.to(DEV).clone()
    xb = torch.full((rows, width), 9.0, dtype=torch.bfloat16, device=DEV)
    sumsq = torch.zeros(16, dtype=torch.int64, device=DEV)
    K.linear_small_norm(act.to(DEV), w.to(DEV), x, K.EPI_RESIDUAL, xb=xb, next_w=gain.to(DEV), out_sumsq=sumsq, scale=scale)
    want_x = x0.double() + scale * (act.double() @ w.double().T)
    torch.testing.assert_close(x.double().cpu(), want_x, rtol=1e-5, atol=1e-5)
    _close(xb, want_x * gain.double(), torch.bfloat16, scale=2.0)
    got_ss = sumsq[:rows].cpu().double() / K.SUMSQ_FIXED
    torch.testing.assert_close(got_ss, (want_x ** 2).sum(-1), rtol=1e-5, atol=1e-5)
    assert int(sumsq[rows:].abs().max()) == 0 if rows < 16 else True
    # the same again gives the same counters to the last bit (integer additions, whatever the order of the tiles)
    x2, sumsq2 = x0.to(DEV).clone(), torch.zeros_like(sumsq)
    K.linear_small_norm(act.to(DEV), w.to(DEV), x2, K.EPI_RESIDUAL, xb=torch.empty_like(xb), next_w=gain.to(DEV), out_sumsq=sumsq2, scale=scale)
    assert torch.equal(sumsq, sumsq2) and torch.equal(x, x2)
    # without activations for a next product (the last layer): only the addition
    x3 = x0.to(DEV).clone()
    K.linear_small_norm(act.to(DEV), w.to(DEV), x3, K.EPI_RESIDUAL, scale=scale)
    assert torch.equal(x3, x)
    # the product after the norm: plain output and SwiGLU
    n2 = 72
    w2 = (torch.randn(2 * n2, width, generator=g) * 2 / math.sqrt(width)).to(torch.bfloat16)
    if K.linear_small_norm_supports(rows, n2, width):
        # the activations are what the first product left (rounded to bfloat16 before the 1 / rms)
        inv = 1 / torch.sqrt((want_x ** 2).mean(-1, keepdim=True) + eps)
        out = torch.full((rows, 2 * n2), 9.0, device=DEV)
        K.linear_small_norm(xb, w2.to(DEV), out, K.EPI_F32, in_sumsq=sumsq, in_eps=eps)
        ref = (xb.double().cpu() @ w2.double().T) * inv
        _close(out, ref, torch.bfloat16, scale=2.0)
        act2 = torch.full((rows, n2), 9.0, dtype=torch.bfloat16, device=DEV)
        K.linear_small_norm(xb, w2.to(DEV), act2, K.EPI_SWIGLU, in_sumsq=sumsq, in_eps=eps)
        _close(act2, ref[:, :n2] * torch.sigmoid(ref[:, :n2]) * ref[:, n2:], torch.bfloat16, scale=2.0)


def test_sums_of_squares_beyond_the_counters_are_reported(K):
    """The counters hold sums up to 2^38 a row; a tile whose share is beyond 2^27 says so in the status word that
    the engine checks, instead of wrapping around."""
    rows, width, kdim = 4, 64, 64
    act = torch.zeros(rows, kdim, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(width, kdim, dtype=torch.bfloat16, device=DEV)
    x = torch.full((rows, width), 1.0e4, device=DEV)          # 16 features x 1e8 = 1.6e9 a tile and row
    x[0] = 1.0
    sumsq = torch.zeros(16, dtype=torch.int64, device=DEV)
    K.check_gemm_status(DEV)
    K.linear_small_norm(act, w, x, K.EPI_RESIDUAL, xb=torch.empty(rows, width, dtype=torch.bfloat16, device=DEV),
                        next_w=torch.ones(width, device=DEV), out_sumsq=sumsq)
    with pytest.raises(K.KernelError, match="sum of squares"):
        K.check_gemm_status(DEV)
    K.check_gemm_status(DEV)                                   # the word was cleared
    assert int(sumsq[0]) == int(width * K.SUMSQ_FIXED)         # the row within range was counted as ever


def test_small_row_qkv_product_scales_its_rows_by_the_norm(K):
    nh, nkvh, dh, page, rows, kdim = 4, 2, 64, 16, 7, 192
    g = torch.Generator().manual_seed(3)
    width = (nh + 2 * nkvh) * dh
    x = torch.randn(rows, kdim, generator=g) * 4
    gain = 1 + 0.1 * torch.randn(kdim, generator=g)
    eps = 1e-6
    xb = (x * gain).to(torch.bfloat16)
    sumsq = torch.zeros(16, dtype=torch.int64)
    sumsq[:rows] = ((x.double() ** 2).sum(-1) * K.SUMSQ_FIXED).round().long()
    h = (x.double() * gain.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps)).float().to(torch.bfloat16)
    w = (torch.randn(width, kdim, generator=g) * 0.1).to(torch.bfloat16)
    max_pos, theta = 96, 5000.0
    j = torch.arange(dh // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] / theta ** (j / (dh // 2))
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    max_blocks = max_pos // page
    table = (torch.randperm(rows * max_blocks, generator=g) + 1).view(rows, max_blocks).to(torch.int32).to(DEV)
    positions = torch.randint(0, max_pos, (rows,), generator=g).to(torch.int32).to(DEV)
    row_req = torch.arange(rows, dtype=torch.int32, device=DEV)
    num_pages = rows * max_blocks + 1
    kp = torch.zeros(num_pages, nkvh, page, dh, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.full((rows, nh * dh), 9.0, dtype=torch.bfloat16, device=DEV)
    K.linear_small_qkv_norm(xb.to(DEV), w.to(DEV), q_out, kp, vp, cos, sin, positions, row_req, table, nh, sumsq.to(DEV), eps)
    # what it has to be: the product of the activations as they are (rounded before the 1 / rms), scaled, rotated
    inv = 1 / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps)
    y = (xb.double() @ w.double().T) * inv
    q = y[:, :nh * dh].view(rows, nh, dh)
    k = y[:, nh * dh:(nh + nkvh) * dh].view(rows, nkvh, dh)
    v = y[:, (nh + nkvh) * dh:].view(rows, nkvh, dh)
    pos = positions.cpu()
    _close(q_out.view(rows, nh, dh), plain_rope(q, pos, theta), torch.bfloat16, scale=2.0)
    rk = plain_rope(k, pos, theta)
    for t in range(rows):
        p = int(table[t, pos[t] // page])
        _close(kp[p, :, pos[t] % page], rk[t], torch.bfloat16, scale=2.0)
        _close(vp[p, :, pos[t] % page], v[t], torch.bfloat16, scale=2.0)
    # and it is the plain kernel's result on normalised activations, up to where those were rounded
    kp2, vp2, q2 = torch.zeros_like(kp), torch.zeros_like(vp), torch.empty_like(q_out)
    K.linear_small_qkv(h.to(DEV), w.to(DEV), q2, kp2, vp2, cos, sin, positions, row_req, table, nh)
    assert float((q2.float() - q_out.float()).abs().max()) <= 0.05 * float(q2.float().abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkvh,dh,page,interleaved", [(6, 2, 48, 8, False), (4, 4, 16, 16, True),
                                                          (3, 1, 128, 4, False), (8, 2, 256, 32, False)])
def test_rope_and_cache_write(K, dtype, nh, nkvh, dh, page, interleaved):
    g = torch.Generator().manual_seed(dh + nh)
    lens = [(5, 9), (0, 3), (20, 1)]                    # (start position, rows) of three requests
    T = sum(n for _, n in lens)
    width = (nh + 2 * nkvh) * dh
    qkv = torch.randn(T, width, generator=g)
    bias = torch.randn(width, generator=g) * 0.1
    max_pos, theta = 64, 5000.0
    j = torch.arange(dh // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] / theta ** (j / (dh // 2))
    cos, sin = ang.cos().float(), ang.sin().float()
    max_blocks = max_pos // page
    perm = torch.randperm(3 * max_blocks, generator=g) + 1
    table = perm.view(3, max_blocks).to(torch.int32)
    positions = torch.cat([torch.arange(s, s + n) for s, n in lens]).to(torch.int32)
    row_req = torch.cat([torch.full((n,), i) for i, (_, n) in enumerate(lens)]).to(torch.int32)
    num_pages = 3 * max_blocks + 1
    kp = torch.zeros(num_pages, nkvh, page, dh, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.empty(T, nh * dh, dtype=dtype, device=DEV)
    K.rope_kv(qkv.to(DEV), bias.to(DEV), positions.to(DEV), row_req.to(DEV), table.to(DEV), page,
              cos.to(DEV), sin.to(DEV), interleaved, q_out, kp, vp, T, nh, nkvh, dh)
    x = (qkv + bias).double()
    q = x[:, :nh * dh].view(T, nh, dh)
    k = x[:, nh * dh:(nh + nkvh) * dh].view(T, nkvh, dh)
    v = x[:, (nh + nkvh) * dh:].view(T, nkvh, dh)
    if interleaved:
        def rot(t):
            c, s = ang[positions.long()][:, None, :].cos(), ang[positions.long()][:, None, :].sin()
            o = torch.empty_like(t)
            o[..., 0::2] = t[..., 0::2] * c - t[..., 1::2] * s
            o[..., 1::2] = t[..., 0::2] * s + t[..., 1::2] * c
            return o
    else:
        rot = lambda t: plain_rope(t, positions, theta)
    _close(q_out.view(T, nh, dh), rot(q), dtype, scale=4.0)
    want_k = torch.zeros(num_pages, nkvh, page, dh, dtype=torch.float64)
    want_v = torch.zeros_like(want_k)
    rk = rot(k)
    for t in range(T):
        p = int(table[row_req[t], positions[t] // page])
        want_k[p, :, positions[t] % page] = rk[t]
        want_v[p, :, positions[t] % page] = v[t]
    _close(kp, want_k, dtype, scale=4.0)
    _close(vp, want_v, dtype, scale=4.0)
    assert float(kp[0].abs().max()) == 0.0              # the null page was not written


def _attention_case(K, dtype, nh, nkvh, dh, page, window, lens, queries, plant=None, seed=0, impl="rows", splits=1, junk=7.0):
    """lens: cached length of each request; queries: per request the positions that are rows.
    impl: "rows" (one warp per row and head), "decode" (split keys), "prefill" (tensor cores; the
    positions of a request must be consecutive)."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    k = [torch.randn(n, nkvh, dh, generator=g) for n in lens]
    v = [torch.randn(n, nkvh, dh, generator=g) for n in lens]
    qf = [torch.randn(n, nh, dh, generator=g) for n in lens]
    if plant:
        # one key far back gets a score that stands out: the row's output must be that key's value
        for (r, qpos, kpos, head) in plant:
            kk = k[r][kpos, head // (nh // nkvh)]
            qf[r][qpos, head] = kk * (40.0 / float(kk.norm()) ** 2) * math.sqrt(dh)
    qf = [t.to(dtype).float() for t in qf]; k = [t.to(dtype).float() for t in k]; v = [t.to(dtype).float() for t in v]
    max_blocks = (max(lens) + page - 1) // page + 1
    perm = (torch.randperm(R * max_blocks, generator=g) + 1).view(R, max_blocks)
    tables = perm.tolist()
    num_pages = R * max_blocks + 1
    kp, vp = _scatter_pages(k, v, tables, page, num_pages, dtype, junk)
    positions = torch.tensor([p for r in range(R) for p in queries[r]], dtype=torch.int32)
    row_req = torch.tensor([r for r in range(R) for _ in queries[r]], dtype=torch.int32)
    q = torch.stack([qf[r][p] for r in range(R) for p in queries[r]]).to(dtype)
    T = q.shape[0]
    out = torch.full((T, nh * dh), 55.0, dtype=dtype, device=DEV)
    scale = dh ** -0.5
    bt = perm.to(torch.int32).to(DEV)
    qd, kd, vd = q.view(T, nh * dh).to(DEV), kp.to(DEV), vp.to(DEV)
    if impl == "rows":
        K.attention_rows(qd, kd, vd, out, positions.to(DEV), row_req.to(DEV), bt, T, nh, scale, window or 0)
    elif impl == "decode":
        # work on a shuffled list of all rows, to show that the list is honoured
        rows = torch.randperm(T, generator=g).to(torch.int32).to(DEV)
        K.attention_decode(qd, kd, vd, out, rows, T, positions.to(DEV), row_req.to(DEV), bt, nh, scale,
                           window or 0, splits)
    else:                                                  # "prefill" (mma.sync) or "tcgen05"
        starts = [0]
        for r in range(R):
            assert list(queries[r]) == list(range(queries[r][0], queries[r][0] + len(queries[r]))) if len(queries[r]) else True
            starts.append(starts[-1] + len(queries[r]))
        tiles = [(r, t0) for r in range(R) for t0 in range(starts[r], starts[r + 1], K.TILE_ROWS)]
        req_pos = [queries[r][0] if len(queries[r]) else 0 for r in range(R)]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        if impl == "tcgen05":
            K.attention_tcgen05(qd, kd, vd, out, i32(tiles).flatten(), len(tiles), T, i32(starts), i32(req_pos), bt, nh,
                                scale, window or 0)
            K.check_gemm_status(DEV)
        else:
            K.attention_prefill(qd, kd, vd, out, i32(tiles).flatten(), len(tiles), i32(starts), i32(req_pos), bt, nh,
                                scale, window or 0)
    want = torch.cat([plain_attention(qf[r].double(), k[r].double(), v[r].double(), scale, window)[queries[r]]
                      for r in range(R) if len(queries[r])])
    return out.view(T, nh, dh), want, v


SHAPES = [(4, 4, 16, 16, None), (3, 1, 32, 8, None), (6, 2, 48, 4, None), (8, 2, 128, 16, None),
          (5, 5, 64, 16, 7), (2, 1, 80, 32, 33), (2, 2, 256, 16, None), (16, 1, 64, 16, None), (10, 2, 96, 5, 70)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkvh,dh,page,window", SHAPES[:7])
def test_attention_rows_over_pages(K, dtype, nh, nkvh, dh, page, window):
    lens = [37, 1, 130, 64]
    # a portion at the end, a single first token, decoded tokens, a whole prompt cut at page edges
    queries = [list(range(30, 37)), [0], [129], list(range(0, 64))]
    got, want, _ = _attention_case(K, dtype, nh, nkvh, dh, page, window, lens, queries, seed=dh)
    _close(got, want, dtype, scale=2.0)


# grouped heads of 64 or 128: the decode kernel that puts the group on the tensor cores (16 heads fill a tile;
# 20 need a second one; 2 to 7 leave most of it empty)
GROUPED = [(32, 2, 128, 16, None), (10, 2, 64, 16, 70), (40, 2, 128, 8, None), (6, 1, 64, 32, 33), (7, 1, 128, 5, None),
           (6, 3, 64, 16, None), (24, 8, 64, 16, 100)]


@pytest.mark.parametrize("splits", [1, 2, 5, 32])
@pytest.mark.parametrize("nh,nkvh,dh,page,window", SHAPES + GROUPED)
def test_attention_decode_kernel_with_split_keys(K, nh, nkvh, dh, page, window, splits):
    lens = [37, 1, 300, 64, 2]
    queries = [list(range(30, 37)), [0], [299], [62, 63], [0, 1]]
    got, want, _ = _attention_case(K, torch.bfloat16, nh, nkvh, dh, page, window, lens, queries, seed=dh,
                                   impl="decode", splits=splits)
    _close(got, want, torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("nh,nkvh,dh,page,window", [s for s in SHAPES if s[2] != 256] + [(2, 2, 256, 16, None), (4, 2, 64, 16, 100)])
def test_attention_prefill_kernel_on_tensor_cores(K, nh, nkvh, dh, page, window):
    # a whole prompt of several tiles with a ragged end; a portion that starts mid-page far into the
    # context; a portion of exactly one tile; a short one
    lens = [150, 333, 64, 40]
    queries = [list(range(0, 150)), list(range(203, 333)), list(range(0, 64)), list(range(31, 40))]
    got, want, _ = _attention_case(K, torch.bfloat16, nh, nkvh, dh, page, window, lens, queries, seed=dh, impl="prefill")
    _close(got, want, torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("dh", [64, 128])
@pytest.mark.parametrize("requests,splits", [(3, 4), (40, 2), (18, 8), (20, 8)])
def test_grouped_decode_attention_in_blocks_of_four_and_of_eight_warps(K, dh, requests, splits):
    """A launch of at most one block an SM (3 requests x 2 key/value heads x 4 cuts) runs blocks of eight warps on tiles
    of 128 keys, a larger one blocks of four on tiles of 64, whose cuts merge inside clusters (heads of 64: 40 x 2 x 2 and
    18 x 2 x 8) or through the merge kernel (20 x 2 x 8, and heads of 128); all against the plain attention, with a key
    far back that a row must find."""
    nh, nkvh, page = 32, 2, 16
    g = torch.Generator().manual_seed(requests)
    lens = [int(x) for x in torch.randint(130, 700, (requests,), generator=g)]
    queries = [[n - 1] for n in lens]
    plant = [(0, lens[0] - 1, 3, 17), (requests - 1, lens[-1] - 1, lens[-1] // 2, 5)]
    got, want, v = _attention_case(K, torch.bfloat16, nh, nkvh, dh, page, None, lens, queries, plant=plant, seed=7,
                                   impl="decode", splits=splits)
    _close(got, want, torch.bfloat16, scale=2.0)
    assert torch.allclose(got[0, 17].float().cpu(), v[0][3, 17 // 16], atol=2e-2)        # the row found the far key
    assert torch.allclose(got[requests - 1, 5].float().cpu(), v[-1][lens[-1] // 2, 0], atol=2e-2)


@pytest.mark.parametrize("nh,nkvh,dh,page,window", [(4, 4, 64, 16, None), (3, 1, 64, 8, None), (8, 2, 128, 16, None),
                                                     (6, 2, 64, 32, 100), (2, 1, 128, 64, 33), (4, 2, 64, 128, None),
                                                     (36, 36, 64, 16, None)])
def test_attention_prefill_kernel_on_tcgen05(K, nh, nkvh, dh, page, window):
    assert K.attention_tcgen05_supports(dh, page) and not K.attention_tcgen05_supports(48, 16)
    lens = [150, 460, 128, 40]
    queries = [list(range(0, 150)), list(range(203, 460)), list(range(0, 128)), list(range(31, 40))]
    got, want, _ = _attention_case(K, torch.bfloat16, nh, nkvh, dh, page, window, lens, queries, seed=dh + page, impl="tcgen05")
    _close(got, want, torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("impl,dtype", [("rows", torch.float32), ("rows", torch.bfloat16), ("decode", torch.bfloat16),
                                         ("decode grouped", torch.bfloat16), ("prefill", torch.bfloat16),
                                         ("tcgen05", torch.bfloat16)])
@pytest.mark.parametrize("window", [None, 50])
def test_attention_finds_one_far_key_among_hundreds(K, impl, dtype, window):
    nh, nkvh, dh, page = 4, 2, 64, 16
    if impl == "decode grouped":                 # six query heads per key/value head instead of two
        nh, impl = 12, "decode"
    lens = [700]
    # the query at 699 must find key 3 (or, with a window, the key at the window's far edge); the query
    # at 320 the key at 319, across a page's edge
    far = 3 if window is None else 699 - window + 1
    plant = [(0, 699, far, 1), (0, 320, 319, 2)]
    if impl in ("prefill", "tcgen05"):
        queries, i699, i320 = [list(range(300, 700))], 399, 20
    else:
        queries, i699, i320 = [[320, 512, 699]], 2, 0
    kw = dict(impl=impl, splits=3) if impl != "rows" else {}
    got, want, v = _attention_case(K, dtype, nh, nkvh, dh, page, window, lens, queries, plant, seed=5, **kw)
    _close(got, want, dtype, scale=2.0)
    group = nh // nkvh
    assert torch.allclose(got[i699, 1].float().cpu(), v[0][far, 1 // group], atol=2e-2)
    assert torch.allclose(got[i320, 2].float().cpu(), v[0][319, 2 // group], atol=2e-2)
    if window:
        # one position beyond the window's edge must NOT be seen
        plant = [(0, 699, far - 1, 1)]
        got, want, v = _attention_case(K, dtype, nh, nkvh, dh, page, window, lens, queries, plant, seed=5, **kw)
        _close(got, want, dtype, scale=2.0)
        assert not torch.allclose(got[i699, 1].float().cpu(), v[0][far - 1, 1 // group], atol=0.2)


@pytest.mark.parametrize("junk", [float("nan"), float("inf")])
@pytest.mark.parametrize("impl,dtype,nh,nkvh,dh,page", [
    ("rows", torch.float32, 4, 2, 48, 8), ("rows", torch.bfloat16, 4, 4, 16, 16), ("decode", torch.bfloat16, 3, 3, 32, 8),
    ("decode", torch.bfloat16, 6, 2, 64, 16), ("decode", torch.bfloat16, 8, 2, 128, 16), ("prefill", torch.bfloat16, 4, 2, 64, 16),
    ("prefill", torch.bfloat16, 2, 1, 80, 32), ("tcgen05", torch.bfloat16, 4, 2, 64, 16), ("tcgen05", torch.bfloat16, 4, 2, 128, 64),
    ("tcgen05", torch.bfloat16, 2, 2, 64, 128)])
def test_attention_ignores_what_lies_beyond_a_request_s_length(K, impl, dtype, nh, nkvh, dh, page, junk):
    """The slots of a held page beyond the request's last position, and pages that were never written, may hold
    anything: what another request left there (a request whose activations overflowed leaves NaN or Inf) or what
    the allocator handed out.  No kernel may let it reach a result, not even multiplied by a weight of zero."""
    lens = [150, 333, 70, 41]
    if impl in ("prefill", "tcgen05"):
        queries = [list(range(0, 150)), list(range(203, 333)), list(range(6, 70)), list(range(31, 41))]
    else:
        queries = [[149], [331, 332], [69], list(range(36, 41))]
    kw = dict(impl=impl, splits=3) if impl == "decode" else dict(impl=impl)
    got, want, _ = _attention_case(K, dtype, nh, nkvh, dh, page, None, lens, queries, seed=dh + page, junk=junk, **kw)
    assert torch.isfinite(got.float()).all()
    _close(got, want, dtype, scale=2.0)


@pytest.mark.parametrize("V", [5, 301, 122753])
def test_argmax_takes_the_first_of_equal_maxima(K, V):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(3, V, generator=g)
    logits[1, V - 1] = 50.0
    logits[2, V // 2] = 60.0; logits[2, V // 3] = 60.0
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    K.argmax(logits.to(DEV), out)
    assert out.tolist() == [int(logits[0].argmax()), V - 1, V // 3]
    # rows with a stride (a padded leading dimension)
    wide = torch.zeros(3, V + 3)
    wide[:, :V] = logits
    K.argmax(wide.to(DEV)[:, :V], out)
    assert out.tolist() == [int(logits[0].argmax()), V - 1, V // 3]


@pytest.mark.parametrize("V", [37, 1000, 122753])
def test_sample_matches_the_plain_rule(K, V):
    g = torch.Generator().manual_seed(V)
    cases = []
    for i, (temp, topk, topp) in enumerate([(0.0, 0, 1.0), (1.0, 1, 1.0), (1.0, 0, 1.0), (0.8, 0, 1.0), (2.5, 0, 1.0),
                                             (1.0, 5, 1.0), (0.7, 20, 1.0), (1.0, 0, 0.6), (1.3, 0, 0.9),
                                             (0.9, 8, 0.5), (1.0, V, 1.0), (1.0, 3, 0.999)]):
        for u in (0.0, 0.013, 0.31, 0.5, 0.77, 0.9991):
            cases.append((temp, topk, topp, u))
    n = len(cases)
    # logits on a grid of 1/64 with distinct values near the top: no ties at the cut, float32-exact
    base = (torch.randperm(V, generator=g).float() / 64.0)
    base = base - base.max() + 3.0
    logits = base.repeat(n, 1)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    f = lambda xs, dt: torch.tensor(xs, dtype=dt, device=DEV)
    K.sample(logits.to(DEV), f([c[0] for c in cases], torch.float32), f([c[1] for c in cases], torch.int32),
             f([c[2] for c in cases], torch.float32), f([c[3] for c in cases], torch.float32), out)
    got = out.tolist()
    miss = []
    for i, c in enumerate(cases):
        want = plain_sample(logits[i], *c)
        if got[i] != want:
            # a float32-vs-float64 difference may move the pick only to a neighbour in the running mass
            miss.append((c, got[i], want))
    assert not miss, miss[:5]


def test_sample_is_reproducible_and_follows_the_distribution(K):
    V, n = 50, 4000
    g = torch.Generator().manual_seed(1)
    row = torch.randn(V, generator=g) * 2
    logits = row.repeat(n, 1).to(DEV)
    u = torch.rand(n, generator=g).to(DEV)
    ones = torch.full((n,), 1.0, device=DEV)
    zeros = torch.zeros(n, dtype=torch.int32, device=DEV)
    a = torch.empty(n, dtype=torch.int32, device=DEV)
    b = torch.empty_like(a)
    K.sample(logits, ones, zeros, ones, u, a)
    K.sample(logits, ones, zeros, ones, u, b)
    assert torch.equal(a, b)
    freq = torch.bincount(a.long().cpu(), minlength=V).double() / n
    p = torch.softmax(row.double(), 0)
    assert (freq - p).abs().max() < 4 * math.sqrt(0.25 / n)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K_", [(48, 64), (301, 96), (2304, 2304), (1000, 5760), (6912, 2304), (17, 32)])
def test_linear_small_streams_weights_for_few_rows(K, M, N, K_):
    g = torch.Generator().manual_seed(M * N + K_)
    act = torch.randn(M, K_, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    # (16 rows of 5760 activations leave the ring kernel no room in shared memory; the tile kernel, which keeps a
    # tile of the weights there instead, takes them)
    assert K.linear_small_supports(M, N, K_)
    out = torch.full((M, N), 9.0, device=DEV)
    K.linear_small(act.to(DEV), w.to(DEV), out)
    want = act.double() @ w.double().T
    torch.testing.assert_close(out.double().cpu(), want, rtol=1e-4, atol=1e-4)      # float32 accumulation of bf16 products


def test_linear_small_with_copies_from_every_thread_instead_of_tma_boxes():
    """The tile kernel's other way to bring its tile (what runs where the weights are not 16-byte aligned for TMA or
    a tensor map cannot be had): a process of its own, because the switch is read once."""
    import os, subprocess, sys
    code = """
import math, os, sys, torch
sys.path.insert(0, os.getcwd())
from infinicore_infer_b200 import kernels as K
for M, N, K_ in ((1, 48, 64), (8, 301, 96), (13, 1000, 5760), (16, 2304, 2304)):
    g = torch.Generator().manual_seed(M * N + K_)
    act = torch.randn(M, K_, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    out = torch.full((M, N), 9.0, device="cuda:0")
    K.linear_small(act.cuda(), w.cuda(), out)
    torch.testing.assert_close(out.double().cpu(), act.double() @ w.double().T, rtol=1e-4, atol=1e-4)
print("equal")
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-c", code], cwd=root, env=dict(os.environ, JK_SMALL_NO_TMA="1"),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "equal" in p.stdout, p.stderr[-2000:]


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("N,K_", [(136, 96), (5760, 2304), (50, 64)])
def test_linear_small_with_swiglu_epilogue(K, M, N, K_):
    g = torch.Generator().manual_seed(M + N + K_)
    act = torch.randn(M, K_, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * N, K_, generator=g) * 2 / math.sqrt(K_)).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    K.linear_small(act.to(DEV), w.to(DEV), out, K.EPI_SWIGLU)
    gu = act.double() @ w.double().T
    want = gu[:, :N] * torch.sigmoid(gu[:, :N]) * gu[:, N:]
    _close(out, want, torch.bfloat16, scale=2.0)


def test_linear_small_refuses_what_it_cannot_take(K):
    assert not K.linear_small_supports(17, 64, 64)
    assert not K.linear_small_supports(4, 64, 80)       # K must be a multiple of 32
    assert not K.linear_small_supports(16, 64, 1 << 20)
    with pytest.raises(K.KernelError, match="outside what the kernel takes"):
        K.linear_small(torch.zeros(4, 80, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 80, dtype=torch.bfloat16, device=DEV),
                       torch.zeros(4, 8, device=DEV))


@pytest.fixture(params=["rule", "pairs"])
def pairs(K, request):
    """The tcgen05 products under their own rule for pairs of blocks, and with every product of more than
    128 rows forced onto pairs (the rule sends only products of more than one wave there)."""
    before = K.gemm_tcgen05_pairs(2 if request.param == "pairs" else 1)
    yield request.param
    K.gemm_tcgen05_pairs(1 if before < 0 else before)


TG_SHAPES = [(128, 256, 64), (128, 128, 128), (1, 8, 8), (300, 520, 200), (257, 100, 2304), (512, 6912, 2304), (2048, 2304, 5760),
             # long K and few tiles: the residual epilogue cuts K into units that add themselves (four; two with a ragged end)
             (512, 512, 8192), (300, 520, 4104)]


@pytest.mark.parametrize("M,N,K_", TG_SHAPES)
@pytest.mark.parametrize("epi", ["f32", "bf16", "residual"])
def test_gemm_tcgen05_with_store_and_residual_epilogues(K, pairs, M, N, K_, epi):
    g = torch.Generator().manual_seed(M + N + K_)
    act = torch.randn(M, K_, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    want = act.double() @ w.double().T
    assert K.gemm_tcgen05_supports(M, N, K_)
    if epi == "f32":
        out = torch.full((M, N), 9.0, device=DEV)
        K.gemm_tcgen05(act.to(DEV), w.to(DEV), out, K.TG_F32)
        K.check_gemm_status(DEV)
        torch.testing.assert_close(out.double().cpu(), want, rtol=1e-4, atol=1e-4)
    elif epi == "bf16":
        out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
        K.gemm_tcgen05(act.to(DEV), w.to(DEV), out, K.TG_BF16)
        K.check_gemm_status(DEV)
        _close(out, want, torch.bfloat16, scale=2.0)
    else:
        x = torch.randn(M, N, generator=g)
        out = x.to(DEV).clone()
        K.gemm_tcgen05(act.to(DEV), w.to(DEV), out, K.TG_RESIDUAL, scale=0.7)
        K.check_gemm_status(DEV)
        torch.testing.assert_close(out.double().cpu(), x.double() + 0.7 * want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (300, 136, 96), (2048, 5760, 2304), (77, 520, 200)])
def test_gemm_tcgen05_with_swiglu_epilogue(K, pairs, M, N, K_):
    g = torch.Generator().manual_seed(M * 3 + N)
    act = torch.randn(M, K_, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * N, K_, generator=g) * 2 / math.sqrt(K_)).to(torch.bfloat16)
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    K.gemm_tcgen05(act.to(DEV), w.to(DEV), out, K.TG_SWIGLU)
    K.check_gemm_status(DEV)
    gu = act.double() @ w.double().T
    _close(out, gu[:, :N] * torch.sigmoid(gu[:, :N]) * gu[:, N:], torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("M,N,K_", [(32, 128, 64), (17, 256, 512), (64, 520, 200), (1, 100, 72), (100, 333, 4096), (128, 1200, 2304),
                                    (9, 77, 16384)])
@pytest.mark.parametrize("epi", ["f32", "residual", "swiglu"])
def test_gemm_of_few_rows_with_the_weights_on_the_m_side(K, M, N, K_, epi):
    """jk_gemm_skinny: up to 128 rows, any width (ragged tiles of 128 features, 64 for SwiGLU), K with a tail and
    long enough to be split among blocks whose partial sums meet in the output."""
    g = torch.Generator().manual_seed(M + N + K_)
    act = torch.randn(M, K_, generator=g).to(torch.bfloat16)
    rows = 2 * N if epi == "swiglu" else N
    w = (torch.randn(rows, K_, generator=g) * (2 if epi == "swiglu" else 1) / math.sqrt(K_)).to(torch.bfloat16)
    ref = act.double() @ w.double().T
    assert K.gemm_skinny_supports(M, N, K_) and not K.gemm_skinny_supports(129, N, K_) and not K.gemm_skinny_supports(M, N, 20)
    if epi == "f32":
        out = torch.full((M, N), 9.0, device=DEV)
        K.gemm_skinny(act.to(DEV), w.to(DEV), out, K.TG_F32)
        K.check_gemm_status(DEV)
        torch.testing.assert_close(out.double().cpu(), ref, rtol=1e-4, atol=1e-4)
    elif epi == "residual":
        x = torch.randn(M, N, generator=g)
        out = x.to(DEV).clone()
        K.gemm_skinny(act.to(DEV), w.to(DEV), out, K.TG_RESIDUAL, scale=0.7)
        K.check_gemm_status(DEV)
        torch.testing.assert_close(out.double().cpu(), x.double() + 0.7 * ref, rtol=1e-4, atol=1e-4)
    else:
        out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
        K.gemm_skinny(act.to(DEV), w.to(DEV), out, K.TG_SWIGLU)
        K.check_gemm_status(DEV)
        _close(out, ref[:, :N] * torch.sigmoid(ref[:, :N]) * ref[:, N:], torch.bfloat16, scale=2.0)
    # an output with padded rows
    if epi == "f32":
        wide = torch.full((M, N + 5), 9.0, device=DEV)
        K.gemm_skinny(act.to(DEV), w.to(DEV), wide[:, :N], K.TG_F32)
        torch.testing.assert_close(wide[:, :N].double().cpu(), ref, rtol=1e-4, atol=1e-4)
        assert float(wide[:, N:].min()) == 9.0


def test_gemm_tcgen05_refuses_rows_that_tma_cannot_address(K):
    assert not K.gemm_tcgen05_supports(4, 4, 20)
    with pytest.raises(K.KernelError, match="multiple of 8"):
        K.gemm_tcgen05(torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV), torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV),
                       torch.zeros(4, 4, device=DEV))

