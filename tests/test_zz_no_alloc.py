"""The sum-of-squares entry point that brings its own scratch (toner_sumsq_static).

Some hosts cannot let a library allocate on the device, or cannot spare a scratch buffer for it: every device
byte is budgeted and owned by their own pool.  For them the library carries a fixed scratch array in its own
image.  This file checks, through the C ABI, that the variant returns exactly what the ordinary entry point
(caller-provided scratch) returns, twice in a row -- the second call reuses the array the first one left full --
that it takes no device memory while doing so, that the whole array and strided inputs work, and that a batch
beyond the built-in limit and a leading dimension below the row length are refused.

The file is named to be collected last.  In that position the library has long been in use by the time these
tests run; the case where toner_sumsq_static is the very first thing a process asks of the library runs in a
child process of its own (test_first_call_of_a_fresh_process)."""

import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from toner_b200 import _lib
    torch.cuda.set_device(0)
    return _lib.load()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _static(lib, x, got):
    batch, rows, cols = x.shape
    return lib.toner_sumsq_static(x.data_ptr(), batch, rows, cols, x.stride(1), x.stride(0), got.data_ptr(), _stream())


def _both(lib, x):
    batch, rows, cols = x.shape
    want = torch.empty(batch, device="cuda")
    got = torch.full((batch,), float("nan"), device="cuda")
    scratch = torch.empty(lib.toner_sumsq_scratch_bytes(batch), dtype=torch.uint8, device="cuda")
    rc = _static(lib, x, got)
    assert rc == 0, lib.toner_last_error().decode()
    rc = lib.toner_sumsq(x.data_ptr(), batch, rows, cols, x.stride(1), x.stride(0), scratch.data_ptr(), want.data_ptr(),
                         _stream())
    assert rc == 0, lib.toner_last_error().decode()
    torch.cuda.synchronize()
    return got.cpu(), want.cpu()


def test_static_scratch_matches_caller_scratch_twice(lib):
    g = torch.Generator(device="cuda").manual_seed(3)
    first = torch.randn(7, 192, 320, device="cuda", generator=g)
    second = torch.randn(3, 64, 1000, device="cuda", generator=g) * 5.0   # fewer, differently shaped matrices
    for x in (first, second):
        got, want = _both(lib, x)
        assert torch.equal(got, want)                       # same reduction tree: same bits
        ref = x.double().pow(2).sum(dim=(1, 2)).cpu()
        assert torch.allclose(got.double(), ref, rtol=1e-5)


def test_the_call_takes_no_device_memory(lib):
    """Free device memory as the driver reports it is the same before and after the calls: nothing was allocated
    (the inputs and the result buffer exist before the first reading is taken)."""
    x = torch.randn(5, 128, 256, device="cuda")
    got = torch.empty(5, device="cuda")
    assert _static(lib, x, got) == 0            # once before measuring: this device's array address is now known
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert _static(lib, x, got) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.allclose(got.double().cpu(), x.double().pow(2).sum(dim=(1, 2)).cpu(), rtol=1e-5)


def test_whole_array_and_strided_rows(lib):
    """As many matrices as the built-in array holds, and rows that are slices of wider rows (ld > cols)."""
    limit = lib.toner_sumsq_static_max_batch()
    g = torch.Generator(device="cuda").manual_seed(4)
    full = torch.randn(limit, 24, 40, device="cuda", generator=g)
    got, want = _both(lib, full)
    assert torch.equal(got, want)
    assert torch.allclose(got.double(), full.double().pow(2).sum(dim=(1, 2)).cpu(), rtol=1e-5)
    wide = torch.randn(6, 50, 96, device="cuda", generator=g)
    view = wide[:, :, 8:72]                      # 64 of every 96 columns: ld = 96, cols = 64
    assert view.stride(1) == 96
    got, want = _both(lib, view)
    assert torch.equal(got, want)
    assert torch.allclose(got.double(), view.double().pow(2).sum(dim=(1, 2)).cpu(), rtol=1e-5)


def test_bad_sizes_are_refused(lib):
    limit = lib.toner_sumsq_static_max_batch()
    x = torch.zeros(limit + 1, 8, 8, device="cuda")
    out = torch.zeros(limit + 1, device="cuda")
    rc = lib.toner_sumsq_static(x.data_ptr(), limit + 1, 8, 8, 8, 64, out.data_ptr(), _stream())
    assert rc != 0
    assert b"exceeds the built-in scratch" in lib.toner_last_error()
    # rows that overlap (fewer elements between rows than a row holds) are a caller's mistake in both entry points
    scratch = torch.empty(lib.toner_sumsq_scratch_bytes(2), dtype=torch.uint8, device="cuda")
    assert lib.toner_sumsq_static(x.data_ptr(), 2, 8, 8, 4, 64, out.data_ptr(), _stream()) != 0
    assert b"ld" in lib.toner_last_error()
    assert lib.toner_sumsq(x.data_ptr(), 2, 8, 8, 4, 64, scratch.data_ptr(), out.data_ptr(), _stream()) != 0
    assert b"ld" in lib.toner_last_error()


_CHILD = r"""
import ctypes as C, sys, torch
sys.path.insert(0, sys.argv[1])
from toner_b200 import _lib
torch.cuda.set_device(0)
x = torch.randn(4, 96, 160, device="cuda")
got = torch.empty(4, device="cuda")
torch.cuda.synchronize()
lib = _lib.load()                              # nothing else of the library has run in this process
s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
def call():
    rc = lib.toner_sumsq_static(x.data_ptr(), 4, 96, 160, x.stride(1), x.stride(0), got.data_ptr(), s)
    assert rc == 0, lib.toner_last_error()
    torch.cuda.synchronize()
free_start, _ = torch.cuda.mem_get_info()
call()                                         # the set-up call: the driver loads the library's image here
first = got.clone().cpu()
free_before, _ = torch.cuda.mem_get_info()
call()
call()
free_after, _ = torch.cuda.mem_get_info()
ok = torch.allclose(got.double().cpu(), x.double().pow(2).sum(dim=(1, 2)).cpu(), rtol=1e-5) and torch.equal(first, got.cpu())
print("RESULT", int(ok), free_before - free_after, free_start - free_before)
"""


def test_first_call_of_a_fresh_process(lib):
    """A process whose first and only request to the library is toner_sumsq_static.  Its first call is the set-up
    call: the array's address is looked up and the driver loads the library's image (kernels and the array itself)
    onto the device, which is the memory the header speaks of.  From then on free device memory does not move, and
    every call, the first included, returns the right sums."""
    out = subprocess.run([sys.executable, "-c", _CHILD, ROOT], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("RESULT")][-1].split()
    assert line[1] == "1"
    assert int(line[2]) == 0, f"free device memory changed by {line[2]} bytes across calls after the set-up call"
    print(f"image loaded by the set-up call: {line[3]} bytes of device memory")
