"""The sum-of-squares entry point that brings its own scratch (toner_sumsq_static).

Some hosts cannot let a library allocate on the device, or cannot spare a scratch buffer for it: every device
byte is budgeted and owned by their own pool.  For them the library carries a fixed scratch array in its own
image.  This file checks, through the C ABI, that the variant returns exactly what the ordinary entry point
(caller-provided scratch) returns, twice in a row -- the second call reuses the array the first one left full --
and that a batch beyond the built-in limit is refused.  It is named to be collected last."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from toner_b200 import _lib
    torch.cuda.set_device(0)
    return _lib.load()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _both(lib, x):
    batch, rows, cols = x.shape
    want = torch.empty(batch, device="cuda")
    got = torch.full((batch,), float("nan"), device="cuda")
    scratch = torch.empty(lib.toner_sumsq_scratch_bytes(batch), dtype=torch.uint8, device="cuda")
    # the variant goes first: in a fresh process it is then the first thing this library does on the device
    rc = lib.toner_sumsq_static(x.data_ptr(), batch, rows, cols, x.stride(1), x.stride(0), got.data_ptr(), _stream())
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


def test_batch_beyond_the_builtin_scratch_is_refused(lib):
    limit = lib.toner_sumsq_static_max_batch()
    x = torch.zeros(limit + 1, 8, 8, device="cuda")
    out = torch.zeros(limit + 1, device="cuda")
    rc = lib.toner_sumsq_static(x.data_ptr(), limit + 1, 8, 8, 8, 64, out.data_ptr(), _stream())
    assert rc != 0
    assert b"exceeds the built-in scratch" in lib.toner_last_error()
