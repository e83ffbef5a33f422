"""Each CUDA kernel alone against its plain statement in ``kernel_refs``, at sizes that the tiny
models do not use (odd widths, partial rotation, windows, shuffled pages)."""
import pytest
import torch

import kernel_refs as R
from helpers import rel_err

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.2e-2}  # bfloat16: one rounding of the stored result is 2^-8


def dev():
    return torch.device("cuda")


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
def test_embedding_gather(dtype, wdtype):
    from inferrs_b200 import kernels as K
    table = rand((1000, 200), wdtype, 0)
    ids = torch.randint(0, 1000, (37,), dtype=torch.int32, device=dev())
    out = torch.empty((37, 200), dtype=torch.float32, device=dev())
    ref = torch.empty_like(out)
    K.embedding_gather(table, ids, out, dtype)
    R.embedding_gather(table, ids, ref)
    assert torch.equal(out, ref)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_gather_scaled(dtype):
    from inferrs_b200 import kernels as K
    table = rand((300, 72), dtype, 0)
    ids = torch.randint(0, 300, (11,), dtype=torch.int32, device=dev())
    out = torch.empty((11, 72), dtype=torch.float32, device=dev())
    K.embedding_gather(table, ids, out, dtype, scale=8.485281)
    assert torch.equal(out, table[ids.long()].float() * torch.tensor(8.485281, dtype=torch.float32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 200, 4100])
def test_rms_norm_rows_and_add_cast(dtype, width):
    """The norm on a sub-layer's output, and the addition into the residual stream where no norm follows."""
    from inferrs_b200 import kernels as K
    n = 13
    x = rand((n, width), dtype, 1, scale=2.0)
    w = (1 + 0.1 * rand((width,), torch.float32, 3)).to(dtype)
    out, ref = torch.empty_like(x), torch.empty_like(x)
    K.rms_norm_rows(x, w, 1e-5, out)
    R.rms_norm_rows(x, w, 1e-5, ref)
    assert rel_err(out, ref) < TOL[dtype]
    res = rand((n, width), torch.float32, 4)
    for delta in (x, None):
        r1, r2 = res.clone(), res.clone()
        K.add_cast(r1, delta, out)
        R.add_cast(r2, delta, ref)
        assert torch.equal(out, ref) and torch.equal(r1, r2)
    rows = torch.tensor([5, 0, 12], dtype=torch.int32, device=dev())
    r1 = res.clone()
    o3, f3 = out[:3].clone(), ref[:3].clone()
    K.add_cast(r1, x, o3, rows)
    R.add_cast(res.clone(), x, f3, rows)
    assert torch.equal(o3, f3) and torch.equal(r1, res)


@pytest.mark.parametrize("cap", [None, 30.0])
def test_logit_scale_softcap(cap):
    from inferrs_b200 import kernels as K
    x = rand((5, 1237), torch.float32, 6, scale=40.0)
    got, ref = x.clone(), x.clone()
    K.logit_scale_softcap(got, 0.25, cap, torch.float32)
    R.logit_scale_softcap(ref, 0.25, cap)
    assert rel_err(got, ref) < 1e-6
    if cap:
        assert float(got.abs().max()) <= cap
    with pytest.raises(K.KernelError):
        K.logit_scale_softcap(got, 1.0, -1.0, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 37, 1000])
def test_resolve_tokens(dtype, n):
    """ids[i] < 0 names place -1 - ids[i] of the tokens that an earlier step sampled; other ids stay; a place
    beyond those tokens becomes an id that is no token (the embedding gives zeros for it)."""
    from inferrs_b200 import kernels as K
    g = torch.Generator().manual_seed(n)
    carry = torch.randint(0, 5000, (11,), generator=g, dtype=torch.int32).to(dev())
    ids = torch.randint(0, 5000, (n,), generator=g, dtype=torch.int32)
    places = torch.randint(0, 11, (n,), generator=g, dtype=torch.int32)
    named = torch.rand(n, generator=g) < 0.4
    given = torch.where(named, -1 - places, ids)
    want = torch.where(named, carry.cpu()[places.long()], ids)
    if n > 2:
        given[2], want[2] = -1 - 11, -1        # a place that does not exist
    got = given.to(dev())
    K.resolve_tokens(got, carry, dtype)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [200, 96, 4096, 5000])
def test_add_rms_norm(dtype, width):
    from inferrs_b200 import kernels as K
    n = 19
    for wdtype in ([torch.float32] if dtype == torch.float32 else DTYPES):
        res = rand((n, width), torch.float32, 1)
        delta = rand((n, width), dtype, 2)
        w = (1 + 0.1 * rand((width,), torch.float32, 3)).to(wdtype)
        for use_delta in (True, False):
            r1, r2 = res.clone(), res.clone()
            out = torch.empty((n, width), dtype=dtype, device=dev())
            ref = torch.empty_like(out)
            K.add_rms_norm(r1, delta if use_delta else None, w, 1e-5, out)
            R.add_rms_norm(r2, delta if use_delta else None, w, 1e-5, ref)
            assert rel_err(out, ref) < TOL[dtype]
            assert rel_err(r1, r2) < 1e-6
        rows = torch.tensor([3, 0, 18, 7], dtype=torch.int32, device=dev())
        r1 = res.clone()
        out = torch.empty((4, width), dtype=dtype, device=dev())
        ref = torch.empty_like(out)
        K.add_rms_norm(r1, delta, w, 1e-6, out, rows)
        R.add_rms_norm(res.clone(), delta, w, 1e-6, ref, rows)
        assert rel_err(out, ref) < TOL[dtype]
        assert torch.equal(r1, res), "the row-gathering form must not write the residual back"


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_gate(dtype):
    from inferrs_b200 import kernels as K
    gu = rand((33, 2 * 150), dtype, 4, scale=3.0)
    out = torch.empty((33, 150), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    K.silu_gate(gu, out)
    R.silu_gate(gu, ref)
    assert rel_err(out, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inner", [(33, 152), (300, 1536), (5, 8)])
def test_silu_gate_wide_rows(dtype, rows, inner):
    """Inner sizes that are multiples of 8 (the form with sixteen bytes per thread in bfloat16), gates so large
    and so small that the exponential overflows or vanishes, and every element on its own against the formula."""
    from inferrs_b200 import kernels as K
    gu = rand((rows, 2 * inner), dtype, 5, scale=3.0)
    gu[0, :8] = torch.tensor([100.0, -100.0, 88.0, -88.0, 30.0, -30.0, 0.0, -0.0], dtype=dtype, device=dev())
    gu[0, inner:inner + 8] = 1.5
    out = torch.full((rows, inner), float("nan"), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    K.silu_gate(gu, out)
    R.silu_gate(gu, ref)
    assert not torch.isnan(out.float()).any()
    assert rel_err(out, ref) < TOL[dtype]
    want = torch.tensor([150.0, 0.0, 132.0, 0.0, 45.0, 0.0, 0.0, 0.0])
    assert torch.allclose(out[0, :8].float().cpu(), want, rtol=1e-2, atol=1e-6)
    g, u = gu[:, :inner].float(), gu[:, inner:].float()
    exact = (g / (1.0 + torch.exp(-g)) * u)
    worst = ((out.float() - exact).abs() / (exact.abs() + 1e-3)).max()
    assert worst < (1e-5 if dtype == torch.float32 else 8e-3), worst     # bfloat16 keeps eight bits


def _paged_setup(dtype, n_kv, d, page_size, lens, new, seed, n_pages=None):
    """Requests with lens[r] cached tokens of which the last new[r] are this step's rows."""
    g = torch.Generator().manual_seed(seed)
    pages_per = [(l + page_size - 1) // page_size for l in lens]
    total = sum(pages_per)
    n_pages = n_pages or total + 3
    perm = torch.randperm(n_pages, generator=g)[:total].tolist()
    table = torch.full((len(lens), max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    positions, row_request = [], []
    for r, (l, t) in enumerate(zip(lens, new)):
        positions += list(range(l - t, l))
        row_request += [r] * t
    k_pages = rand((n_pages, n_kv, page_size, d), dtype, seed + 1)
    v_pages = rand((n_pages, n_kv, page_size, d), dtype, seed + 2)
    return (table.to(dev()), torch.tensor(positions, dtype=torch.int32, device=dev()),
            torch.tensor(row_request, dtype=torch.int32, device=dev()), k_pages, v_pages)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot,ps", [(6, 3, 48, 48, 8), (4, 4, 16, 8, 4), (8, 2, 128, 128, 16), (5, 1, 128, 64, 16)])
def test_qk_norm_rope_store_with_neighbours_turning_together(dtype, nh, nkv, d, rot, ps):
    """The other pairing: element 2i of a head turns with element 2i + 1 (head size 128 too, which has kernels of its
    own for the pairing by halves only)."""
    from inferrs_b200 import kernels as K
    lens, new = [21, 9, 40], [5, 9, 1]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 17)
    n = sum(new)
    qkv = rand((n, (nh + 2 * nkv) * d), dtype, 18)
    wq = (1 + 0.1 * rand((d,), torch.float32, 19)).to(dtype)
    wk = (1 + 0.1 * rand((d,), torch.float32, 20)).to(dtype)
    ang = torch.arange(64, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(rot // 2) * 2.0 / rot))[None]
    cos, sin = torch.cos(ang).to(dev()), torch.sin(ang).to(dev())
    k1, v1, k2, v2 = k_pages.clone(), v_pages.clone(), k_pages.clone(), v_pages.clone()
    q1 = torch.empty((n, nh, d), dtype=dtype, device=dev())
    q2, q3 = torch.empty_like(q1), torch.empty_like(q1)
    K.qk_norm_rope_store(qkv, nh, nkv, d, True, wq, wk, 1e-5, cos, sin, rot, positions, row_request, table, k1, v1, q1,
                         interleaved=True)
    R.qk_norm_rope_store(qkv, nh, nkv, d, True, wq, wk, 1e-5, cos, sin, rot, positions, row_request, table, k2, v2, q2,
                         interleaved=True)
    assert rel_err(q1, q2) < TOL[dtype] and rel_err(k1, k2) < TOL[dtype] and torch.equal(v1, v2)
    R.qk_norm_rope_store(qkv, nh, nkv, d, True, wq, wk, 1e-5, cos, sin, rot, positions, row_request, table, k2, v2, q3)
    assert rel_err(q1, q3) > 10 * TOL[dtype], "the two pairings were meant to differ"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot,ps", [(6, 3, 48, 48, 8), (4, 4, 16, 8, 4), (8, 2, 128, 128, 16), (3, 1, 80, 0, 16)])
def test_qk_norm_rope_store(dtype, nh, nkv, d, rot, ps):
    from inferrs_b200 import kernels as K
    lens, new = [21, 9, 40], [5, 9, 1]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 7)
    n = sum(new)
    qkv = rand((n, (nh + 2 * nkv) * d), dtype, 8)
    wq = (1 + 0.1 * rand((d,), torch.float32, 9)).to(dtype)
    wk = (1 + 0.1 * rand((d,), torch.float32, 10)).to(dtype)
    cos = sin = None
    if rot:
        ang = torch.arange(64, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(rot // 2) * 2.0 / rot))[None]
        cos, sin = torch.cos(ang).to(dev()), torch.sin(ang).to(dev())
    for use_norm in (True, False):
        k1, v1, k2, v2 = k_pages.clone(), v_pages.clone(), k_pages.clone(), v_pages.clone()
        q1 = torch.empty((n, nh, d), dtype=dtype, device=dev())
        q2 = torch.empty_like(q1)
        a = (wq, wk) if use_norm else (None, None)
        K.qk_norm_rope_store(qkv, nh, nkv, d, True, a[0], a[1], 1e-5, cos, sin, rot, positions, row_request, table,
                             k1, v1, q1)
        R.qk_norm_rope_store(qkv, nh, nkv, d, True, a[0], a[1], 1e-5, cos, sin, rot, positions, row_request, table,
                             k2, v2, q2)
        assert rel_err(q1, q2) < TOL[dtype]
        assert rel_err(k1, k2) < TOL[dtype]
        assert torch.equal(v1, v2)
    # queries only: a layer that reads another layer's cache
    q1 = torch.empty((n, nh, d), dtype=dtype, device=dev())
    q2 = torch.empty_like(q1)
    qo = qkv[:, :nh * d].contiguous()
    K.qk_norm_rope_store(qo, nh, nkv, d, False, wq, None, 1e-5, cos, sin, rot, positions, row_request, None, None,
                         None, q1)
    R.qk_norm_rope_store(qo, nh, nkv, d, False, wq, None, 1e-5, cos, sin, rot, positions, row_request, None, None,
                         None, q2)
    assert rel_err(q1, q2) < TOL[dtype]


@pytest.mark.parametrize("nh,nkv", [(8, 2), (5, 1), (3, 3)])
def test_qk_norm_rope_store_many_rows(nh, nkv):
    """Hundreds of rows at head size 128 in bfloat16: the form that takes four heads per warp (head counts
    that are no multiple of four leave a warp with fewer)."""
    from inferrs_b200 import kernels as K
    dtype, d, ps = torch.bfloat16, 128, 16
    lens, new = [310, 75], [290, 75]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 17)
    n = sum(new)
    qkv = rand((n, (nh + 2 * nkv) * d), dtype, 18)
    wq = (1 + 0.1 * rand((d,), torch.float32, 19)).to(dtype)
    wk = (1 + 0.1 * rand((d,), torch.float32, 20)).to(dtype)
    ang = torch.arange(320, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(d // 2) * 2.0 / d))[None]
    cos, sin = torch.cos(ang).to(dev()), torch.sin(ang).to(dev())
    k1, v1, k2, v2 = k_pages.clone(), v_pages.clone(), k_pages.clone(), v_pages.clone()
    q1 = torch.empty((n, nh, d), dtype=dtype, device=dev())
    q2 = torch.empty_like(q1)
    K.qk_norm_rope_store(qkv, nh, nkv, d, True, wq, wk, 1e-6, cos, sin, d, positions, row_request, table, k1, v1, q1)
    R.qk_norm_rope_store(qkv, nh, nkv, d, True, wq, wk, 1e-6, cos, sin, d, positions, row_request, table, k2, v2, q2)
    assert rel_err(q1, q2) < TOL[dtype]
    assert rel_err(k1, k2) < TOL[dtype]
    assert torch.equal(v1, v2)
    assert K.row_fault(dtype) is None


@pytest.mark.parametrize("dtype,d", [(torch.float32, 48), (torch.bfloat16, 128)])
def test_a_position_outside_the_rotation_tables_is_left_out_and_reported(dtype, d):
    """The kernel reads no table row that does not exist: such a row writes nothing and is reported."""
    from inferrs_b200 import kernels as K
    nh, nkv, ps = 4, 2, 16
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, [40], [6], 27)
    qkv = rand((6, (nh + 2 * nkv) * d), dtype, 28)
    ang = torch.arange(37, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(d // 2) * 2.0 / d))[None]
    cos, sin = torch.cos(ang).to(dev()), torch.sin(ang).to(dev())   # positions 34..39 come; the tables end at 36
    k1, v1 = k_pages.clone(), v_pages.clone()
    q1 = torch.full((6, nh, d), 7.0, dtype=dtype, device=dev())
    assert K.row_fault(dtype) is None
    K.qk_norm_rope_store(qkv, nh, nkv, d, True, None, None, 1e-6, cos, sin, d, positions, row_request, table, k1, v1, q1)
    assert K.row_fault(dtype) in (3, 4, 5)
    assert K.row_fault(dtype) is None          # reading it clears it
    assert bool((q1[3:] == 7.0).all()) and not bool((q1[:3] == 7.0).any())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,ps,window", [(6, 3, 48, 8, None), (4, 2, 16, 4, 9), (8, 2, 128, 16, None),
                                                (5, 5, 80, 16, 33), (2, 1, 256, 16, None)])
def test_paged_attention_generic(dtype, nh, nkv, d, ps, window):
    from inferrs_b200 import kernels as K
    lens, new = [300, 17, 64, 1], [40, 17, 1, 1]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 20)
    n = sum(new)
    q = rand((n, nh, d), dtype, 23)
    # one far key of request 0 stands out for its last row: the row's output must be close to that key's value
    far = 5 if window is None else lens[0] - window  # the window's far edge
    page, slot = int(table[0, far // ps]), far % ps
    k_pages[page, :, slot, :] = 0
    k_pages[page, :, slot, 0] = 16.0
    q[new[0] - 1, :, :] = 0
    q[new[0] - 1, :, 0] = 16.0
    out = torch.empty((n, nh * d), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    scale = d ** -0.5 * 4  # the marked score is 256 * scale, the others' spread 16 * scale
    K.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, out)
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    assert rel_err(out, ref) < TOL[dtype]
    got = out[new[0] - 1].view(nh, d).float()
    want = v_pages[page, :, slot, :].float().repeat_interleave(nh // nkv, dim=0)
    assert rel_err(got, want) < 5e-2, "the far key that stands out was not seen"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,m,k", [(70, 130, 100), (1, 517, 96), (64, 64, 16), (129, 65, 33)])
def test_gemm_tn_simt(dtype, n, m, k):
    from inferrs_b200 import kernels as K
    combos = [(torch.float32, torch.float32, torch.float32)]
    if dtype == torch.bfloat16:
        combos = [(torch.bfloat16, torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.bfloat16, torch.float32),
                  (torch.bfloat16, torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32, torch.float32)]
    for xd, wd, od in combos:
        x, w = rand((n, k), xd, 30), rand((m, k), wd, 31)
        out = torch.empty((n, m), dtype=od, device=dev())
        K.gemm_tn_simt(x, w, out, dtype)
        ref = (x.double() @ w.double().t())
        assert rel_err(out, ref) < (1e-5 if od == torch.float32 else 1e-2)


def test_gemm_rows_do_not_depend_on_the_batch():
    from inferrs_b200 import kernels as K
    x, w = rand((100, 300), torch.float32, 40), rand((200, 300), torch.float32, 41)
    full = torch.empty((100, 200), dtype=torch.float32, device=dev())
    K.gemm_tn_simt(x, w, full, torch.float32)
    one = torch.empty((1, 200), dtype=torch.float32, device=dev())
    K.gemm_tn_simt(x[77:78].contiguous(), w, one, torch.float32)
    assert torch.equal(one[0], full[77])


def test_gemm_bf16_library():
    from inferrs_b200 import kernels as K
    x, w = rand((70, 256), torch.bfloat16, 50), rand((136, 256), torch.bfloat16, 51)
    ref = x.double() @ w.double().t()
    for od in (torch.bfloat16, torch.float32):
        out = torch.empty((70, 136), dtype=od, device=dev())
        K.gemm_tn_bf16(x, w, out)
        assert rel_err(out, ref) < (1e-2 if od == torch.bfloat16 else 1e-5)


def test_argmax():
    from inferrs_b200 import kernels as K
    logits = rand((9, 151), torch.float32, 60)
    logits[2, 17] = logits[2, 99] = 50.0   # equal maxima: the lowest index wins
    logits[3, :] = -float("inf")
    logits[3, 150] = -1e30
    big = rand((3, 151936), torch.float32, 61)
    for l in (logits, big):
        out = torch.empty((l.shape[0],), dtype=torch.int32, device=dev())
        K.argmax(l, out)
        assert torch.equal(out.long(), torch.argmax(l, dim=-1)) or l is logits
        if l is logits:
            assert out[2] == 17 and out[3] == 150
            mask = torch.ones(9, dtype=torch.bool)
            mask[2] = False
            assert torch.equal(out.long()[mask], torch.argmax(l, dim=-1)[mask])


def test_kernels_refuse_cpu_tensors():
    from inferrs_b200 import kernels as K
    with pytest.raises(K.KernelError):
        K.silu_gate(torch.zeros(2, 4), torch.zeros(2, 2))


def _tiles(new, tokens_per_tile):
    req, row0, at = [], [], 0
    for r, n in enumerate(new):
        for s in range(0, n, tokens_per_tile):
            req.append(r)
            row0.append(at + s)
        at += n
    return (torch.tensor(req, dtype=torch.int32, device=dev()), torch.tensor(row0, dtype=torch.int32, device=dev()),
            len(req))


@pytest.mark.parametrize("nh,nkv,d,ps,window", [(8, 2, 128, 16, None), (4, 4, 64, 4, None), (6, 2, 128, 16, 70),
                                                (16, 2, 64, 64, None), (5, 1, 256, 8, None), (32, 8, 128, 16, 33)])
def test_paged_attention_mma_prefill_form(nh, nkv, d, ps, window):
    from inferrs_b200 import kernels as K
    dtype = torch.bfloat16
    lens, new = [300, 17, 200, 64, 1], [40, 17, 200, 1, 1]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 20)
    n = sum(new)
    q = rand((n, nh, d), dtype, 23)
    q_start = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev())
    far = 5 if window is None else lens[0] - window
    page, slot = int(table[0, far // ps]), far % ps
    k_pages[page, :, slot, :] = 0
    k_pages[page, :, slot, 0] = 16.0
    q[new[0] - 1, :, :] = 0
    q[new[0] - 1, :, 0] = 16.0
    out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    scale = d ** -0.5 * 4
    tile_req, tile_row0, n_tiles = _tiles(new, 64 // (nh // nkv))
    K.paged_attention_mma(q, k_pages, v_pages, table, tile_req, tile_row0, n_tiles, q_start, positions, scale, window,
                          out, False)
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    assert rel_err(out, ref) < 2e-2
    got = out[new[0] - 1].view(nh, d).float()
    want = v_pages[page, :, slot, :].float().repeat_interleave(nh // nkv, dim=0)
    assert rel_err(got, want) < 5e-2, "the far key that stands out was not seen"


@pytest.mark.parametrize("nh,nkv,d,ps,window,splits", [(8, 2, 128, 16, None, 1), (32, 8, 128, 16, None, 7),
                                                        (4, 4, 64, 4, 50, 3), (16, 1, 256, 32, None, 40),
                                                        (6, 2, 128, 16, 129, 2)])
def test_paged_attention_mma_decode_form(nh, nkv, d, ps, window, splits):
    from inferrs_b200 import kernels as K
    dtype = torch.bfloat16
    lens = [300, 17, 64, 1, 65, 1000]
    new = [1] * len(lens)
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 30)
    n = len(lens)
    q = rand((n, nh, d), dtype, 33)
    q_start = torch.arange(n + 1, dtype=torch.int32, device=dev())
    far = 5 if window is None else lens[5] - window
    page, slot = int(table[5, far // ps]), far % ps
    k_pages[page, :, slot, :] = 0
    k_pages[page, :, slot, 0] = 16.0
    q[5, :, :] = 0
    q[5, :, 0] = 16.0
    out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    scale = d ** -0.5 * 4
    K.paged_attention_mma(q, k_pages, v_pages, table, row_request, q_start, n, q_start, positions, scale, window, out,
                          True, splits)
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    assert rel_err(out, ref) < 2e-2
    got = out[5].view(nh, d).float()
    want = v_pages[page, :, slot, :].float().repeat_interleave(nh // nkv, dim=0)
    assert rel_err(got, want) < 5e-2, "the far key that stands out was not seen"


@pytest.mark.parametrize("nh,nkv,ps,window", [(8, 2, 16, None), (32, 8, 16, None), (6, 2 * 3, 16, 70), (4, 1, 64, None),
                                              (16, 1, 8, 200), (2, 2, 128, None), (10, 2, 16, None), (6, 2, 32, 90)])
def test_paged_attention_tcgen05(nh, nkv, ps, window):
    from inferrs_b200 import kernels as K
    dtype, d = torch.bfloat16, 128
    lens, new = [300, 17, 200, 64, 1, 700], [40, 17, 200, 1, 1, 333]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 20)
    n = sum(new)
    q = rand((n, nh, d), dtype, 23)
    q_start = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev())
    far = 5 if window is None else lens[0] - window
    page, slot = int(table[0, far // ps]), far % ps
    k_pages[page, :, slot, :] = 0
    k_pages[page, :, slot, 0] = 16.0
    q[new[0] - 1, :, :] = 0
    q[new[0] - 1, :, 0] = 16.0
    out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    scale = d ** -0.5 * 4
    tile_req, tile_row0, n_tiles = _tiles(new, 128 // (nh // nkv))
    K.paged_attention_tcgen05(q, k_pages, v_pages, table, tile_req, tile_row0, n_tiles, q_start, positions, scale, window,
                              out)
    assert K.attention_tcgen05_error() == 0
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    assert rel_err(out, ref) < 2e-2
    got = out[new[0] - 1].view(nh, d).float()
    want = v_pages[page, :, slot, :].float().repeat_interleave(nh // nkv, dim=0)
    assert rel_err(got, want) < 5e-2, "the far key that stands out was not seen"


@pytest.mark.parametrize("nh,nkv,ps,window", [(8, 2, 16, None), (32, 8, 16, None), (6, 2 * 3, 16, 70), (4, 1, 64, None),
                                              (16, 1, 8, 200), (2, 2, 32, None), (10, 2, 16, None), (6, 2, 32, 90)])
def test_paged_attention_pair_tcgen05(nh, nkv, ps, window):
    """The kernel with two query tiles per CTA: tiles of 256/G tokens, so that requests with one token, with fewer
    tokens than one query tile holds, with a few more, and with many all occur; one far key and the last query of
    the first request are made so that this key alone decides that row (the reference maximum of the row jumps
    when its tile comes, and the output accumulated so far must be scaled away)."""
    from inferrs_b200 import kernels as K
    dtype, d = torch.bfloat16, 128
    lens, new = [300, 17, 200, 64, 1, 700], [40, 17, 200, 1, 1, 333]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 20)
    n = sum(new)
    q = rand((n, nh, d), dtype, 23)
    q_start = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev())
    far = 150 if window is None else lens[0] - window
    page, slot = int(table[0, far // ps]), far % ps
    k_pages[page, :, slot, :] = 0
    k_pages[page, :, slot, 0] = 16.0
    q[new[0] - 1, :, :] = 0
    q[new[0] - 1, :, 0] = 16.0
    out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    scale = d ** -0.5 * 4
    tile_req, tile_row0, n_tiles = _tiles(new, K.pair_tile_tokens(nh, nkv))
    K.paged_attention_pair_tcgen05(q, k_pages, v_pages, table, tile_req, tile_row0, n_tiles, q_start, positions, scale,
                                   window, out)
    assert K.attention_pair_tcgen05_error() == 0
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    assert not torch.isnan(out.float()).any()
    assert rel_err(out, ref) < 2e-2
    got = out[new[0] - 1].view(nh, d).float()
    want = v_pages[page, :, slot, :].float().repeat_interleave(nh // nkv, dim=0)
    assert rel_err(got, want) < 5e-2, "the far key that stands out was not seen"


@pytest.mark.parametrize("nh,nkv,ps,window,max_splits", [(8, 2, 16, None, 1), (32, 8, 16, None, 9), (4, 4, 8, 50, 3),
                                                          (16, 1, 32, None, 40), (6, 2, 64, 129, 2), (32, 8, 16, None, 64)])
def test_paged_attention_decode(nh, nkv, ps, window, max_splits):
    from inferrs_b200 import kernels as K
    dtype, d = torch.bfloat16, 128
    lens = [300, 17, 64, 1, 65, 1000, 2049, 513]
    new = [1] * len(lens)
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 30)
    n = len(lens)
    q = rand((n, nh, d), dtype, 33)
    far = 5 if window is None else lens[5] - window
    page, slot = int(table[5, far // ps]), far % ps
    k_pages[page, :, slot, :] = 0
    k_pages[page, :, slot, 0] = 16.0
    q[5, :, :] = 0
    q[5, :, 0] = 16.0
    ref = torch.empty((n, nh * d), dtype=dtype, device=dev())
    scale = d ** -0.5 * 4
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    for min_tiles in (4, 4, 9):   # twice the same: the counters must be back at zero after a launch
        out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
        K.paged_attention_decode(q, k_pages, v_pages, table, positions, scale, window, out, max_splits,
                                 min_tiles=min_tiles)
        assert K.attention_decode_error() == 0
        assert rel_err(out, ref) < 2e-2
    got = out[5].view(nh, d).float()
    want = v_pages[page, :, slot, :].float().repeat_interleave(nh // nkv, dim=0)
    assert rel_err(got, want) < 5e-2, "the far key that stands out was not seen"


def test_how_the_decode_kernel_is_cut_follows_the_waves_of_ctas():
    """Host arithmetic only: the slices per request for numbers of (request, head group) pairs around one and two
    waves of resident CTAs."""
    from inferrs_b200 import kernels as K
    room = K.DECODE_RESIDENT_CTAS
    assert K.decode_slices(1, 8, 4096) == (16, 4) and K.decode_slices(8, 8, 4096) == (room // 64, 4)
    assert K.decode_slices(37, 8, 4096) == (1, 4), "one wave: one slice"
    assert K.decode_slices(40, 8, 4096) == (3, 4) and K.decode_slices(52, 8, 4096) == (2, 4)
    assert K.decode_slices(64, 8, 4096) == (1, 4) and K.decode_slices(64, 8, 40960) == (1, 4), "nearly two waves: one slice"
    assert K.decode_slices(256, 8, 40960) == (1, 4)
    assert K.decode_max_splits(48, 8, 16384) == 3


@pytest.mark.parametrize("nh,nkv,ps,window", [(8, 2, 16, None), (32, 8, 16, 300)])
def test_attention_of_a_step_with_portions_and_single_tokens(nh, nkv, ps, window):
    """The way a replayed step with prompt portions uses the two kernels: the portions' tiles in a list of fixed
    length in which -1 marks empty places (prefill kernel), the rows that are single tokens in another such list
    (decode kernel); together they must give every row of the step, and leave the rows of no request alone."""
    from inferrs_b200 import kernels as K
    dtype, d = torch.bfloat16, 128
    lens, new = [300, 650, 200, 64, 1, 700, 90], [40, 1, 200, 1, 1, 1, 33]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 20)
    n_real = sum(new)
    n = n_real + 7                                    # seven rows that fill the step up
    pad = torch.zeros(7, dtype=torch.int32, device=dev())
    positions = torch.cat([positions, pad])
    row_request = torch.cat([row_request, pad + len(lens)])
    table = torch.cat([table, torch.full((2, table.shape[1]), -1, dtype=torch.int32, device=dev())])
    q = rand((n, nh, d), dtype, 23)
    starts = [0] + list(torch.tensor(new).cumsum(0))
    q_start = torch.tensor(starts + [n, n], dtype=torch.int32, device=dev())   # the filling request and an empty one
    tpt = 128 // (nh // nkv)
    req, row0 = [], []
    for r, t in enumerate(new):
        if t > 1:
            for s0 in range(0, t, tpt):
                req.append(r)
                row0.append(int(starts[r]) + s0)
    t_max = len(req) + 5
    tile_req = torch.tensor(req + [-1] * 5, dtype=torch.int32, device=dev())
    tile_row0 = torch.tensor(row0 + [0] * 5, dtype=torch.int32, device=dev())
    singles = [(int(starts[r]), r) for r, t in enumerate(new) if t == 1]
    rows = torch.tensor([s[0] for s in singles] + [-1, -1, -1], dtype=torch.int32, device=dev())
    reqs = torch.tensor([s[1] for s in singles] + [-1, -1, -1], dtype=torch.int32, device=dev())
    scale = d ** -0.5 * 2
    out = torch.full((n, nh * d), 5.0, dtype=dtype, device=dev())
    K.paged_attention_decode(q, k_pages, v_pages, table, positions, scale, window, out, 4, rows, reqs)
    K.paged_attention_tcgen05(q, k_pages, v_pages, table, tile_req, tile_row0, t_max, q_start, positions, scale, window,
                              out)
    assert K.attention_tcgen05_error() == 0 and K.attention_decode_error() == 0
    ref = torch.empty((n_real, nh * d), dtype=dtype, device=dev())
    R.paged_attention_generic(q[:n_real].contiguous(), k_pages, v_pages, table, row_request[:n_real].contiguous(),
                              positions[:n_real].contiguous(), scale, window, ref)
    assert rel_err(out[:n_real], ref) < 2e-2
    assert bool((out[n_real:] == 5.0).all()), "rows of no request must be left alone"


def _attention_kernels(nh, nkv):
    """name -> function(q, k_pages, v_pages, table, new, positions, row_request, scale, window, out) for every
    bfloat16 attention kernel of head size 128 that serves prompt portions, and for single tokens."""
    from inferrs_b200 import kernels as K

    def prefill(kernel, tokens_per_tile):
        def run(q, k_pages, v_pages, table, new, positions, row_request, scale, window, out):
            q_start = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev())
            tile_req, tile_row0, n_tiles = _tiles(new, tokens_per_tile)
            kernel(q, k_pages, v_pages, table, tile_req, tile_row0, n_tiles, q_start, positions, scale, window, out)
        return run

    def mma(q, k_pages, v_pages, table, new, positions, row_request, scale, window, out):
        q_start = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev())
        tile_req, tile_row0, n_tiles = _tiles(new, 64 // (nh // nkv))
        K.paged_attention_mma(q, k_pages, v_pages, table, tile_req, tile_row0, n_tiles, q_start, positions, scale,
                              window, out, False)

    def decode(q, k_pages, v_pages, table, new, positions, row_request, scale, window, out):
        assert all(t == 1 for t in new)
        K.paged_attention_decode(q, k_pages, v_pages, table, positions, scale, window, out, 6)

    return {"tcgen05": prefill(K.paged_attention_tcgen05, 128 // (nh // nkv)),
            "pair": prefill(K.paged_attention_pair_tcgen05, K.pair_tile_tokens(nh, nkv)),
            "mma": mma, "decode": decode, "generic": lambda q, k, v, table, new, positions, row_request, scale, window,
            out: K.paged_attention_generic(q, k, v, table, row_request, positions, scale, window, out)}


def _no_error():
    from inferrs_b200 import kernels as K
    assert K.attention_tcgen05_error() == 0 and K.attention_pair_tcgen05_error() == 0 and K.attention_decode_error() == 0


@pytest.mark.parametrize("name", ["tcgen05", "pair", "mma", "decode", "generic"])
@pytest.mark.parametrize("window", [70, 128, 200])
def test_the_key_just_outside_the_window_is_not_seen(name, window):
    """The key at pos - window + 1 is the last one inside the window, the key at pos - window the first outside.
    The outside key is made to stand out so much that it alone would decide the row if it were admitted."""
    nh, nkv, d, ps, dtype = 8, 2, 128, 16, torch.bfloat16
    lens = [500, 330, 700]
    new = [1, 1, 1] if name == "decode" else [40, 1, 333]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 40)
    n = sum(new)
    q = rand((n, nh, d), dtype, 41)
    scale = d ** -0.5 * 4
    rows_last = [sum(new[:r + 1]) - 1 for r in range(len(new))]        # each request's last row
    marked = []
    for r, row in enumerate(rows_last):
        outside = lens[r] - 1 - window
        page, slot = int(table[r, outside // ps]), outside % ps
        k_pages[page, :, slot, :] = 0
        k_pages[page, :, slot, 0] = 16.0
        v_pages[page, :, slot, :] = 100.0                              # it would show at once
        q[row, :, :] = 0
        q[row, :, 0] = 16.0
        marked.append((row, page, slot))
    out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    _attention_kernels(nh, nkv)[name](q, k_pages, v_pages, table, new, positions, row_request, scale, window, out)
    _no_error()
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    assert rel_err(out, ref) < 2e-2
    for row, _, _ in marked:
        assert float(out[row].float().abs().max()) < 10.0, "the key just outside the window was seen"
    # and one step further in: the same key at the inside edge decides the row
    out2 = torch.empty_like(out)
    _attention_kernels(nh, nkv)[name](q, k_pages, v_pages, table, new, positions, row_request, scale, window + 1, out2)
    for row, _, _ in marked:
        assert float((out2[row].float() - 100.0).abs().max()) < 2.0, "the key at the inside edge was not seen"


@pytest.mark.parametrize("name", ["tcgen05", "pair", "mma", "decode"])
@pytest.mark.parametrize("window", [None, 90])
def test_what_an_earlier_owner_left_in_the_pages_does_not_reach_the_output(name, window):
    """Pages are used again without being cleared.  Everything a request does not own holds NaN here: the pages of
    no request, the places of its last page behind its last token (keys only: the kernel that writes a request's
    last value clears the values behind it, which is done here by hand), and, with a window, the pages that the
    window has passed (their block-table entries are -1).  Every output must be finite and equal the reference."""
    nh, nkv, d, ps, dtype = 8, 2, 128, 16, torch.bfloat16
    lens = [300, 17, 200, 65, 1, 700]
    new = [1] * len(lens) if name == "decode" else [40, 17, 200, 1, 1, 333]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 50)
    owned = torch.zeros(k_pages.shape[0], dtype=torch.bool)
    nan = float("nan")
    table_h = table.cpu()
    for r, n_tok in enumerate(lens):
        n_pg = (n_tok + ps - 1) // ps
        first = 0
        if window is not None:
            first = max(0, n_tok - new[r] - window + 1) // ps          # pages that every query's window has passed
            for p in range(first):
                table_h[r, p] = -1
        for p in range(first, n_pg):
            owned[int(table_h[r, p])] = True
        last, used = int(table_h[r, n_pg - 1]), n_tok - (n_pg - 1) * ps
        k_pages[last, :, used:, :] = nan
        v_pages[last, :, used:, :] = 0.0
    k_pages[~owned.to(dev())] = nan
    v_pages[~owned.to(dev())] = nan
    table = table_h.to(dev())
    n = sum(new)
    q = rand((n, nh, d), dtype, 51)
    scale = d ** -0.5
    out = torch.full((n, nh * d), nan, dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    _attention_kernels(nh, nkv)[name](q, k_pages, v_pages, table, new, positions, row_request, scale, window, out)
    _no_error()
    assert bool(torch.isfinite(out.float()).all()), "something that no request owns reached the output"
    R.paged_attention_generic(q, k_pages, v_pages, table, row_request, positions, scale, window, ref)
    assert rel_err(out, ref) < 2e-2


def test_the_last_value_of_a_request_clears_the_places_behind_it():
    """The kernel that writes keys and values: behind the value of a request's last row its page holds zeros
    afterwards, whatever was there; other pages and the places before it are untouched."""
    from inferrs_b200 import kernels as K
    nh, nkv, d, ps = 4, 2, 128, 16
    for dtype, n_rows in ((torch.bfloat16, [3, 1, 300]), (torch.bfloat16, [3, 1, 20]), (torch.float32, [3, 1, 20])):
        lens = [35, 64, n_rows[2] + 5]
        table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, n_rows, 60)
        k_pages[:], v_pages[:] = float("nan"), float("nan")
        n = sum(n_rows)
        qkv = rand((n, (nh + 2 * nkv) * d), dtype, 61)
        ang = torch.arange(max(lens), dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(d // 2) * 2.0 / d))[None]
        cos, sin = torch.cos(ang).to(dev()), torch.sin(ang).to(dev())
        q = torch.empty((n, nh, d), dtype=dtype, device=dev())
        K.qk_norm_rope_store(qkv, nh, nkv, d, True, None, None, 1e-6, cos, sin, d, positions, row_request, table,
                             k_pages, v_pages, q)
        for r, n_tok in enumerate(lens):
            last_page, used = int(table[r, (n_tok - 1) // ps]), (n_tok - 1) % ps + 1
            assert bool((v_pages[last_page, :, used:, :] == 0).all()), (dtype, r)
            assert bool(torch.isfinite(v_pages[last_page, :, used - 1, :].float()).all())
            if used < ps:
                assert bool(torch.isnan(k_pages[last_page, :, used:, :].float()).all()), "keys are left alone"
        written = torch.zeros(k_pages.shape[0], dtype=torch.bool)
        for r, n_tok in enumerate(lens):
            for p in range((n_tok - n_rows[r]) // ps, (n_tok + ps - 1) // ps):
                written[int(table[r, p])] = True
        assert bool(torch.isnan(v_pages[~written.to(dev())].float()).all()), "a page of no row was written to"


@pytest.mark.parametrize("name", ["tcgen05", "pair", "decode"])
@pytest.mark.parametrize("context", [8192, 16384])
def test_attention_over_long_contexts(name, context):
    """Thousands of cached keys (two key/value heads): one request with a portion at the end of a long context
    beside a short one, or single tokens at the end; a key near the start stands out for the last row."""
    nh, nkv, d, ps, dtype = 8, 2, 128, 16, torch.bfloat16
    lens = [context, 333, context - 4097]
    new = [1, 1, 1] if name == "decode" else [200, 70, 1]
    table, positions, row_request, k_pages, v_pages = _paged_setup(dtype, nkv, d, ps, lens, new, 70)
    n = sum(new)
    q = rand((n, nh, d), dtype, 71)
    far = 3
    page, slot = int(table[0, far // ps]), far % ps
    k_pages[page, :, slot, :] = 0
    k_pages[page, :, slot, 0] = 16.0
    q[new[0] - 1, :, :] = 0
    q[new[0] - 1, :, 0] = 16.0
    scale = d ** -0.5 * 4
    out = torch.full((n, nh * d), float("nan"), dtype=dtype, device=dev())
    _attention_kernels(nh, nkv)[name](q, k_pages, v_pages, table, new, positions, row_request, scale, None, out)
    _no_error()
    # the reference for the rows that are compared: the first, middle and last rows of every request
    starts = [0] + list(torch.tensor(new).cumsum(0).tolist())
    pick = sorted({starts[r] + i for r in range(len(new)) for i in (0, new[r] // 2, new[r] - 1)})
    idx = torch.tensor(pick, device=dev())
    ref = torch.empty((len(pick), nh * d), dtype=dtype, device=dev())
    R.paged_attention_generic(q[idx].contiguous(), k_pages, v_pages, table, row_request[idx].contiguous(),
                              positions[idx].contiguous(), scale, None, ref)
    assert bool(torch.isfinite(out.float()).all())
    assert rel_err(out[idx], ref) < 2e-2
    got = out[new[0] - 1].view(nh, d).float()
    want = v_pages[page, :, slot, :].float().repeat_interleave(nh // nkv, dim=0)
    assert rel_err(got, want) < 5e-2, "the far key that stands out was not seen"


@pytest.mark.parametrize("n,m,k", [(1, 4096, 4096), (8, 4096, 12288), (16, 300, 136), (5, 6144, 1024), (13, 384, 64)])
def test_products_with_folded_norms(n, m, k):
    """The tcgen05 product for a few rows with the addition to the residual stream and the norm that follows folded
    into its read-back (a sink), and the products that read what it hands on (scaled rows): against the same
    arithmetic in plain float32, and against the unfolded kernels (product, then the norm kernel)."""
    from inferrs_b200 import kernels as K
    dtype = torch.bfloat16
    x, w = rand((n, k), dtype, 90), rand((m, k), dtype, 91, scale=0.05)
    res0 = rand((n, m), torch.float32, 92)
    wn = (1 + 0.1 * rand((m,), torch.float32, 93)).to(dtype)
    eps = 1e-5
    assert K.folded_norm_supported(n, dtype, w)
    # the sink
    res, out = res0.clone(), torch.full((n, m), float("nan"), dtype=dtype, device=dev())
    scaled = K.linear(x, w, out, dtype, sink=K.ResidualSink(res, wn, eps))
    assert K.gemm_tcgen05_error() == 0
    assert isinstance(scaled, K.ScaledRows) and scaled.x is out and scaled.width == m
    res_ref, out_ref = res0.clone(), torch.empty_like(out)
    scaled_ref = R.linear(x, w, out_ref, dtype, sink=K.ResidualSink(res_ref, wn, eps))
    assert rel_err(res, res_ref) < 1e-2 and rel_err(out, out_ref) < TOL[dtype]
    ss = scaled.ssq[:scaled.n_parts, :n].sum(dim=0)
    assert rel_err(ss, (res.double() ** 2).sum(dim=1).float()) < 1e-5, "the parts must add up to the rows' sums of squares"
    # ... is what the product and then the norm kernel give
    y = torch.empty((n, m), dtype=dtype, device=dev())
    K.linear(x, w, y, dtype)
    res2, normed = res0.clone(), torch.empty((n, m), dtype=dtype, device=dev())
    K.add_rms_norm(res2, y, wn, eps, normed)
    assert torch.equal(res2, res), "the stream must get the same bits either way"
    assert rel_err(R._unscale(scaled), normed) < TOL[dtype]
    # scaled rows into a product and into the gated pair of products
    if m % 8 == 0:
        w2 = rand((264, m), dtype, 94, scale=0.05)
        got, ref = torch.empty((n, 264), dtype=dtype, device=dev()), torch.empty((n, 264), dtype=dtype, device=dev())
        K.linear(scaled, w2, got, dtype)
        R.linear(scaled, w2, ref, dtype)
        assert rel_err(got, ref) < TOL[dtype]
        K.linear(normed, w2, ref, dtype)            # the unfolded way: the norm kernel's output into the product
        assert rel_err(got, ref) < 2 * TOL[dtype]
        wg = rand((2 * 192, m), dtype, 95, scale=0.05)
        got, ref = torch.empty((n, 192), dtype=dtype, device=dev()), torch.empty((n, 192), dtype=dtype, device=dev())
        K.gated_linear(scaled, wg, got, dtype)
        R.gated_linear(scaled, wg, ref, dtype)
        assert rel_err(got, ref) < 2 * TOL[dtype]
        # a sink fed from scaled rows (both folded forms in one launch)
        res3, out3 = res0[:, :264].contiguous(), torch.empty((n, 264), dtype=dtype, device=dev())
        res3_ref, out3_ref = res3.clone(), torch.empty_like(out3)
        wn3 = wn[:264].contiguous()
        K.linear(scaled, w2, out3, dtype, sink=K.ResidualSink(res3, wn3, eps))
        R.linear(scaled, w2, out3_ref, dtype, sink=K.ResidualSink(res3_ref, wn3, eps))
        assert rel_err(res3, res3_ref) < 1e-2 and rel_err(out3, out3_ref) < 2 * TOL[dtype]
    assert K.gemm_tcgen05_error() == 0
    assert not K.folded_norm_supported(40, dtype, w) and not K.folded_norm_supported(n, torch.float32, w.float())


@pytest.mark.parametrize("n,m,k,split_k", [(5, 20000, 72, 0), (20, 10000, 136, 0), (8, 6100, 1024, 0), (3, 3000, 8192, 0),
                                           (40, 6100, 256, 0), (12, 5000, 512, 4)])
def test_products_with_tiles_lower_than_the_mma(n, m, k, split_k):
    """A product whose CTAs number between one and two per SM gets tiles of fewer rows than the MMA has, so that
    every SM holds two CTAs: the rows that the MMA computes beyond a tile are never stored, the last tile ends in
    the middle of a box, the owners of a cluster share a tile that is no power of two high.  Plain, with a sink and
    from scaled rows, against float32 and, bit for bit, against the same kernels with tiles of the MMA's height."""
    from inferrs_b200 import kernels as K
    dtype, eps = torch.bfloat16, 1e-6
    rows = K.gemm_tcgen05_tile_rows(n, m, k, split_k)
    assert 0 < rows < 128, "these sizes are meant to take lowered tiles"
    x, w = rand((n, k), dtype, 120), rand((m, k), dtype, 121, scale=0.05)

    def run():
        out = torch.full((n, m), float("nan"), dtype=dtype, device=dev())
        K.gemm_tn_tcgen05(x, w, out, split_k)
        if n > 32:
            return out, None, None, None
        res = rand((n, m), torch.float32, 122)
        wn = (1 + 0.1 * rand((m,), torch.float32, 123)).to(dtype)
        handed = torch.full((n, m), float("nan"), dtype=dtype, device=dev())
        scaled = K.gemm_tn_tcgen05(x, w, handed, split_k, sink=K.ResidualSink(res, wn, eps))
        w2 = rand((136, m), dtype, 124, scale=0.05)
        nxt = torch.empty((n, 136), dtype=dtype, device=dev())
        K.gemm_tn_tcgen05(scaled, w2, nxt) if m % 8 == 0 else None
        return out, res, handed, (scaled.ssq[:scaled.n_parts, :n].sum(dim=0), nxt)

    out, res, handed, rest = run()
    assert K.gemm_tcgen05_error() == 0
    ref = x.float() @ w.float().t()
    assert bool(torch.isfinite(out.float()).all()) and rel_err(out, ref) < TOL[dtype]
    if res is not None:
        res_ref = rand((n, m), torch.float32, 122) + ref.to(dtype).float()
        assert rel_err(res, res_ref) < 1e-2
        assert rel_err(rest[0], (res.double() ** 2).sum(dim=1).float()) < 1e-5
    K.gemm_tcgen05_set_even_tiles(False)
    try:
        assert K.gemm_tcgen05_tile_rows(n, m, k, split_k) == 128
        out_full, res_full, handed_full, rest_full = run()
    finally:
        K.gemm_tcgen05_set_even_tiles(True)
    assert torch.equal(out, out_full)
    if res is not None:
        assert torch.equal(res, res_full) and torch.equal(handed, handed_full)
        if m % 8 == 0:
            assert rel_err(rest[1], rest_full[1]) < 1e-2   # the parts of the sums of squares are cut elsewhere


@pytest.mark.parametrize("n,inner,k", [(7, 10000, 136), (24, 12288, 512), (1, 15000, 64)])
def test_gated_products_with_tiles_lower_than_the_mma(n, inner, k):
    """The gate/up form with fewer than 64 rows of each matrix per tile: the gate box of the last tile reaches into
    the up matrix and the up box beyond the matrix, and neither is stored."""
    from inferrs_b200 import kernels as K
    dtype = torch.bfloat16
    assert 0 < K.gemm_tcgen05_tile_rows(n, inner, k, 0, gated=True) < 64, "these sizes are meant to take lowered tiles"
    x, w = rand((n, k), dtype, 130), rand((2 * inner, k), dtype, 131, scale=0.08)
    out = torch.full((n, inner), float("nan"), dtype=dtype, device=dev())
    K.gemm_swiglu_tcgen05(x, w, out)
    assert K.gemm_tcgen05_error() == 0
    g = (x.float() @ w[:inner].float().t()).to(dtype).float()
    u = (x.float() @ w[inner:].float().t()).to(dtype).float()
    ref = torch.nn.functional.silu(g) * u
    assert bool(torch.isfinite(out.float()).all()) and rel_err(out, ref) < 2 * TOL[dtype]
    K.gemm_tcgen05_set_even_tiles(False)
    try:
        full = torch.empty_like(out)
        K.gemm_swiglu_tcgen05(x, w, full)
    finally:
        K.gemm_tcgen05_set_even_tiles(True)
    assert torch.equal(out, full)


@pytest.mark.parametrize("n,width,inner,qkv", [(8, 4096, 12288, 6144), (1, 1024, 3072, 4096), (16, 192, 320, 1280), (3, 5120, 1088, 640)])
def test_a_chain_of_products_is_one_launch_and_gives_what_the_single_products_give(n, width, inner, qkv):
    """The four products between two attention kernels of a decode step (o projection into the stream, gate and up with
    the gate, down into the stream, the next layer's q/k/v) as one persistent kernel, against the same products
    launched one by one; twice in a row (the workspace and the counters must be as they were), with the same bits both
    times; then shorter chains, one of them fed by a plain tensor."""
    from inferrs_b200 import kernels as K
    dtype, eps = torch.bfloat16, 1e-6
    attn = rand((n, width), dtype, 100)
    w_o, w_gu = rand((width, width), dtype, 101, scale=0.03), rand((2 * inner, width), dtype, 102, scale=0.03)
    w_d, w_qkv = rand((width, inner), dtype, 103, scale=0.03), rand((qkv, width), dtype, 104, scale=0.03)
    n1 = (1 + 0.1 * rand((width,), torch.float32, 105)).to(dtype)
    n2 = (1 + 0.1 * rand((width,), torch.float32, 106)).to(dtype)
    res0 = rand((n, width), torch.float32, 107)

    def run(chained, products=4):
        res = res0.clone()
        o = torch.empty((n, width), dtype=dtype, device=dev())
        a = torch.empty((n, inner), dtype=dtype, device=dev())
        d = torch.empty((n, width), dtype=dtype, device=dev())
        q = torch.full((n, qkv), float("nan"), dtype=dtype, device=dev())
        chain = K.ProductChain() if chained else None
        linear = chain.linear if chained else (lambda x, w, out, sink=None: K.linear(x, w, out, dtype, sink=sink))
        gated = chain.gated_linear if chained else (lambda x, w, out: K.gated_linear(x, w, out, dtype))
        before = K.launch_count()
        s1 = linear(attn, w_o, o, sink=K.ResidualSink(res, n1, eps))
        gated(s1, w_gu, a)
        if products > 2:
            s2 = linear(a, w_d, d, sink=K.ResidualSink(res, n2, eps))
            linear(s2, w_qkv, q)
        if chained:
            chain.launch()
        launches = K.launch_count() - before
        torch.cuda.synchronize()
        return res, q, a, launches

    res_c, q_c, a_c, launches = run(True)
    assert launches == 1 and K.gemm_chain_error() == 0
    res_c2, q_c2, a_c2, _ = run(True)
    assert torch.equal(res_c, res_c2) and torch.equal(q_c, q_c2) and torch.equal(a_c, a_c2)
    res_s, q_s, a_s, launches = run(False)
    assert launches == 4
    assert K.gemm_chain_error() == 0 and K.gemm_tcgen05_error() == 0
    assert rel_err(a_c, a_s) < 2e-2 and rel_err(res_c, res_s) < 1e-2
    assert not torch.isnan(q_c.float()).any()
    assert rel_err(q_c, q_s) < 2e-2
    res_c, _, a_c, launches = run(True, products=2)
    res_s, _, a_s, _ = run(False, products=2)
    assert launches == 1 and K.gemm_chain_error() == 0
    assert rel_err(a_c, a_s) < 2e-2 and rel_err(res_c, res_s) < 1e-2
    # one product alone, from a plain tensor, and what a chain refuses
    chain = K.ProductChain()
    y = torch.empty((n, qkv), dtype=dtype, device=dev())
    assert chain.linear(attn, w_qkv, y) is None
    chain.launch()
    y_s = torch.empty_like(y)
    K.linear(attn, w_qkv, y_s, dtype)
    assert K.gemm_chain_error() == 0 and rel_err(y, y_s) < 2e-2
    with pytest.raises(K.KernelError):
        chain.linear(attn[:, :width - 8], w_qkv, y)
    with pytest.raises(K.KernelError):
        K.ProductChain().linear(rand((17, width), dtype, 108), w_qkv, torch.empty((17, qkv), dtype=dtype, device=dev()))
