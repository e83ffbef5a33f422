"""The entry point that allocates nothing, called the way a foreign host calls it: through its exported C
symbol, with raw device pointers.  Its result must be the regular entry point's, on two calls in a row
(the second finds the first call's leftovers in the built-in scratch)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def _symbol():
    from inferrs_b200.csrc.build import build_library
    lib = ctypes.CDLL(build_library("core_bf16"))
    fn = lib.ib_paged_attention_decode_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                   c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p]
    fn.restype = c_int
    msg = lib.ib_paged_attention_decode_noalloc_strerror
    msg.argtypes = [c_int]
    msg.restype = ctypes.c_char_p
    return fn, msg


def _case(seed, lens, nh, nkv, d, ps):
    g = torch.Generator().manual_seed(seed)
    dev = torch.device("cuda")
    pages_per = [(l + ps - 1) // ps for l in lens]
    n_pages = sum(pages_per) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    n = len(lens)
    return dict(q=mk(n, nh, d), k=mk(n_pages, nkv, ps, d), v=mk(n_pages, nkv, ps, d), table=table.to(dev),
                positions=torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev),
                rows=torch.arange(n, dtype=torch.int32, device=dev),
                q_start=torch.arange(n + 1, dtype=torch.int32, device=dev))


def test_no_alloc_entry_point_matches_the_regular_one_twice():
    from inferrs_b200 import kernels as K
    fn, msg = _symbol()
    nh, nkv, d, ps, splits = 32, 8, 128, 16, 5
    stream = torch.cuda.current_stream().cuda_stream
    # a first call sets the entry point up on this device (it looks the scratch's address up, the kernel's image is
    # loaded): what is measured below are calls in the state in which a server makes them
    c = _case(0, [100, 70], nh, nkv, d, ps)
    warm = torch.empty((2, nh * d), dtype=torch.bfloat16, device="cuda")
    rc = fn(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1], ps,
            c["k"].shape[0], c["rows"].data_ptr(), c["q_start"].data_ptr(), c["positions"].data_ptr(), 2, nh, nkv, d,
            d ** -0.5, 0, warm.data_ptr(), splits, stream)
    assert rc == 0, msg(rc).decode()
    torch.cuda.synchronize()
    for seed, lens in ((1, [700, 33, 64, 1, 129]), (2, [90, 500, 17])):   # two calls in a row, different shapes
        c = _case(seed, lens, nh, nkv, d, ps)
        n = len(lens)
        want = torch.empty((n, nh * d), dtype=torch.bfloat16, device="cuda")
        K.paged_attention_mma(c["q"], c["k"], c["v"], c["table"], c["rows"], c["q_start"], n, c["q_start"],
                              c["positions"], d ** -0.5, None, want, True, splits)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]      # the device's own count: sees what torch's allocator does not
        rc = fn(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1],
                ps, c["k"].shape[0], c["rows"].data_ptr(), c["q_start"].data_ptr(), c["positions"].data_ptr(), n, nh,
                nkv, d, d ** -0.5, 0, got.data_ptr(), splits, stream)
        assert rc == 0, msg(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] >= free_before, "the call took device memory"
        # the same kernel with the same number of slices, only the scratch lies elsewhere: the same bits
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got, want)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    fn, msg = _symbol()
    c = _case(3, [40, 40], 32, 8, 128, 16)
    out = torch.empty((2, 32 * 128), dtype=torch.bfloat16, device="cuda")
    args = lambda n_rows, nh, d, splits: (  # noqa: E731
        c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["table"].data_ptr(), c["table"].shape[1], 16,
        c["k"].shape[0], c["rows"].data_ptr(), c["q_start"].data_ptr(), c["positions"].data_ptr(), n_rows, nh, 8, d,
        0.1, 0, out.data_ptr(), splits, torch.cuda.current_stream().cuda_stream)
    rc = fn(*args(4096, 32, 128, 64))          # 4096 * 32 * 64 * 130 floats: far beyond the 16 MiB
    assert rc == -3 and b"exceeds the built-in scratch" in msg(rc)
    assert fn(*args(2, 32, 80, 2)) == -1       # a head size the kernel does not take
    assert fn(*args(2, 30, 128, 2)) == -2      # 30 heads over 8 kv heads
    assert fn(*args(2, 32, 128, 0)) == -2
    torch.cuda.synchronize()
