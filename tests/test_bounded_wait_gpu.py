"""The kernels' bounded waits, made to run out without anything hanging: a probe kernel of this folder waits with
the package's own wait (``csrc/sm100.cuh``) on a barrier that nobody arrives at, with a limit of one millisecond;
it must come back, say so, and leave the device usable.  Then the engine's way of reading such a report."""
import ctypes
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    from inferrs_b200.csrc import build
    out = str(tmp_path_factory.mktemp("probe") / "bounded_wait_probe.so")
    cmd = [build.find_nvcc()] + build.ARCH_FLAGS + ["-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-I", build.HERE,
                                                    os.path.join(HERE, "csrc", "bounded_wait_probe.cu"), "-o", out]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    lib = ctypes.CDLL(out)
    lib.bounded_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_void_p]
    lib.bounded_wait_probe.restype = ctypes.c_int
    return lib


def test_a_wait_that_nobody_answers_runs_out_and_reports(probe):
    status = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    word = torch.zeros((1,), dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # somebody arrives: the wait completes, nothing is reported
    assert probe.bounded_wait_probe(status.data_ptr(), word.data_ptr(), 1_000_000, 1, stream) == 0
    torch.cuda.synchronize()
    assert status[0].item() == 1 and word.item() == 0
    # nobody arrives: after about a millisecond the wait gives up, says so and records its code
    assert probe.bounded_wait_probe(status.data_ptr(), word.data_ptr(), 1_000_000, 0, stream) == 0
    torch.cuda.synchronize()
    assert status[0].item() == 0 and word.item() == 7
    assert 900 <= status[1].item() < 100_000, f"the wait took {status[1].item()} us"
    # the first code stays until it is read and cleared; the device is as usable as before
    word2 = word.clone()
    assert probe.bounded_wait_probe(status.data_ptr(), word2.data_ptr(), 500_000, 0, stream) == 0
    torch.cuda.synchronize()
    assert word2.item() == 7
    x = torch.arange(1000, device="cuda", dtype=torch.float32)
    assert float((x * 2).sum()) == 999000.0


def test_the_engine_reads_the_words_in_stream_order():
    """The words of the real kernel libraries, asked for behind the work in the stream and read from pinned
    memory: all zero after clean work, and the reset path gives the same answer."""
    from inferrs_b200 import kernels
    from inferrs_b200.engine.health import KernelHealth
    for dtype in (torch.bfloat16, torch.float32):
        h = KernelHealth(dtype)
        assert h.poll() is None and not h.pending
        h.queue()
        assert h.pending
        assert h.poll(wait=True) == {}
        assert h.reset() == {}
        assert len(kernels.ERROR_WORDS) == 6
