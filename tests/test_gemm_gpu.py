"""The tcgen05 GEMM behind every operator, through the C ABI, against FP64 matmul of the same
16-bit operands.  Products of 16-bit values are exact in FP32, so the only difference from the FP64
result is the FP32 accumulation order: tolerances are a few ulp times sqrt(k)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from toner_b200 import ops as _ops
    return _ops


def rnd(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype).cuda()


def ref_mm(a, b, a_mn, b_mn):
    """a, b as stored; returns FP64 A @ B^T with A (m,k), B (n,k)."""
    A = a.double().transpose(-1, -2) if a_mn else a.double()
    B = b.double().transpose(-1, -2) if b_mn else b.double()
    return A @ B.transpose(-1, -2)


def close(got, want, k, tol=4e-7):
    err = (got.double() - want).abs().max().item()
    scale = want.abs().max().item() + 1e-30
    assert err <= tol * (k ** 0.5) * scale + 1e-30, (err, scale)


@pytest.mark.parametrize("tile_n", [128, 256, 512, 1024])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_k_major_square(ops, tile_n, dtype):
    m = n = k = 256
    a, b = rnd((m, k), dtype, 1), rnd((n, k), dtype, 2)
    d = torch.zeros(1, m, n, device="cuda")
    ops.gemm(ops.operand(a), ops.operand(b), m=m, n=n, k=k, batch=1, fmt=ops._FMT[dtype], d=d, tile_n=tile_n)
    ops.assert_healthy()
    close(d[0], ref_mm(a, b, False, False), k)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("tile_n", [128, 256, 512, 1024])   # 512 / 1024: 256 x 256 / 256 x 512 tiles on CTA pairs
def test_layouts_ragged_batched(ops, a_mn, b_mn, tile_n):
    """Sizes that are not multiples of the tile or of the k-block; three matrices per call."""
    batch, m, n, k = 3, 200, 328, 136
    a = rnd((batch, k, m) if a_mn else (batch, m, k), torch.bfloat16, 3)
    b = rnd((batch, k, n) if b_mn else (batch, n, k), torch.bfloat16, 4)
    d = torch.full((batch, m, n), float("nan"), device="cuda")
    ops.gemm(ops.operand(a, mn_major=a_mn), ops.operand(b, mn_major=b_mn), m=m, n=n, k=k, batch=batch, fmt=1, d=d,
             tile_n=tile_n)
    ops.assert_healthy()
    close(d, ref_mm(a, b, a_mn, b_mn), k)


def test_many_tiles_persistent_loop(ops):
    """More tiles than SMs: every CTA loops, alternating the two accumulator buffers."""
    m, n, k = 4096, 2304, 320
    a, b = rnd((m, k), torch.bfloat16, 5), rnd((n, k), torch.bfloat16, 6)
    d = torch.empty(1, m, n, device="cuda")
    ops.gemm(ops.operand(a), ops.operand(b), m=m, n=n, k=k, batch=1, fmt=1, d=d)
    ops.assert_healthy()
    close(d[0], ref_mm(a, b, False, False), k)
    d2 = torch.empty_like(d)
    ops.gemm(ops.operand(a), ops.operand(b), m=m, n=n, k=k, batch=1, fmt=1, d=d2)
    assert torch.equal(d, d2), "same inputs must give bitwise equal results"


def test_wide_tiles_persistent_loop(ops):
    """256 x 512 tiles on CTA pairs, more tiles than pairs: the single accumulator's two halves are handed back and
    forth several times per CTA.  Each element is accumulated in the same order as with 256 x 256 tiles: same bits."""
    m, n, k = 4096, 6144 + 72, 320
    a, b = rnd((m, k), torch.bfloat16, 15), rnd((n, k), torch.bfloat16, 16)
    d = torch.full((1, m, n), float("nan"), device="cuda")
    ops.gemm(ops.operand(a), ops.operand(b), m=m, n=n, k=k, batch=1, fmt=1, d=d, tile_n=1024)
    ops.assert_healthy()
    close(d[0], ref_mm(a, b, False, False), k)
    d2 = torch.empty_like(d)
    ops.gemm(ops.operand(a), ops.operand(b), m=m, n=n, k=k, batch=1, fmt=1, d=d2, tile_n=512)
    ops.assert_healthy()
    assert torch.equal(d, d2)


def test_epilogue_affine_and_outputs(ops):
    batch, m, n, k = 2, 192, 264, 192
    a, b = rnd((batch, m, k), torch.float16, 7), rnd((batch, n, k), torch.float16, 8)
    c = rnd((batch, m, n), torch.float32, 9)
    va = torch.tensor([0.5, 2.0], device="cuda")
    vb = torch.tensor([3.0, 0.25], device="cuda")
    vbeta = torch.tensor([1.0, -2.0], device="cuda")
    d = torch.empty(batch, m, n, device="cuda")
    dh = torch.empty(batch, m, n, device="cuda", dtype=torch.bfloat16)
    ssq = torch.zeros(batch, device="cuda")
    mab = torch.zeros(batch, device="cuda", dtype=torch.int32)
    maf = torch.zeros(batch, device="cuda", dtype=torch.int32)
    ops.gemm(ops.operand(a), ops.operand(b), m=m, n=n, k=k, batch=batch, fmt=0, d=d, d16=dh, c=c, alpha=0.1, beta=0.7,
             alpha_a=va, alpha_b=vb, beta_v=vbeta, sumsq=ssq, maxabs=mab, maxaff=maf, aff=(1.5, -2.0))
    ops.assert_healthy()
    want = 0.1 * (va * vb).double()[:, None, None] * ref_mm(a, b, False, False) + 0.7 * vbeta.double()[:, None, None] * c.double()
    close(d, want, k, tol=1e-6)
    assert torch.equal(dh, d.to(torch.bfloat16))
    assert torch.allclose(ssq.double(), (d.double() ** 2).sum((1, 2)), rtol=1e-5)
    assert torch.equal(mab.view(torch.float32), d.abs().amax((1, 2)))
    eye = torch.eye(m, n, device="cuda")
    assert torch.allclose(maf.view(torch.float32), (1.5 * eye - 2.0 * d).abs().amax((1, 2)), rtol=1e-6)


@pytest.mark.parametrize("n", [256, 328, 768])
@pytest.mark.parametrize("tile_n", [128, 256, 1024])
def test_symmetric_tiles_mirror_and_packed(ops, n, tile_n):
    batch, k = 2, 200
    x = rnd((batch, k, n), torch.bfloat16, 10)  # X^T X: both operands are the MN-major view of X
    want = ref_mm(x, x, True, True)
    full = torch.full((batch, n, n), float("nan"), device="cuda")
    ops.gemm(ops.operand(x, mn_major=True), ops.operand(x, mn_major=True), m=n, n=n, k=k, batch=batch, fmt=1, d=full,
             tri=True, mirror=True, tile_n=tile_n)
    ops.assert_healthy()
    close(full, want, k)
    assert torch.equal(full, full.transpose(1, 2)), "mirrored result must be exactly symmetric"
    packed = torch.full((batch, n * (n + 1) // 2), float("nan"), device="cuda")
    ops.gemm(ops.operand(x, mn_major=True), ops.operand(x, mn_major=True), m=n, n=n, k=k, batch=batch, fmt=1, d=packed,
             tri=True, packed=True, tile_n=tile_n)
    ops.assert_healthy()
    iu = torch.triu_indices(n, n, device="cuda")
    assert torch.equal(packed, full[:, iu[0], iu[1]])


@pytest.mark.parametrize("promote", [1, 3])
def test_promoted_chains_match_one_chain(ops, promote):
    """Summing short accumulation chains in registers gives the same product (ragged sizes, two segments)."""
    batch, m, n, k = 2, 200, 328, 200
    a, b = rnd((2, batch, m, k), torch.bfloat16, 50), rnd((2, batch, n, k), torch.bfloat16, 51)
    want = ref_mm(a[0], b[0], False, False) + ref_mm(a[1], b[1], False, False)
    d = torch.empty(batch, m, n, device="cuda")
    ops.gemm(ops.operand(a, seg_z=(0, batch, 0)), ops.operand(b, seg_z=(0, batch, 0)), m=m, n=n, k=k, batch=batch,
             fmt=1, segs=2, d=d, promote=promote, promote_all=(promote == 3))
    ops.assert_healthy()
    close(d, want, 2 * k)


def test_listed_operands(ops):
    m, n, k = 136, 264, 72
    a_s = [rnd((m, k), torch.bfloat16, 20 + i) for i in range(3)]
    b_s = [rnd((n, k), torch.bfloat16, 30 + i) for i in range(3)]
    a, keep_a = ops.operand_list(a_s)
    b, keep_b = ops.operand_list(b_s)
    d = torch.empty(3, m, n, device="cuda")
    ops.gemm(a, b, m=m, n=n, k=k, batch=3, fmt=1, d=d)
    ops.assert_healthy()
    for i in range(3):
        close(d[i], ref_mm(a_s[i], b_s[i], False, False), k)


@pytest.mark.parametrize("scale", [1.0, 1e-6, 3e4])
def test_split_product_is_fp32_accurate(ops, scale):
    """FP16 hi/lo planes, three plane products in one accumulator: error near FP32 rounding, far below FP16's."""
    batch, m, n, k = 2, 256, 192, 512
    a = rnd((batch, m, k), torch.float32, 40) * scale
    b = rnd((batch, n, k), torch.float32, 41)
    b[0] *= 1e-3  # matrices of one stack may have very different magnitudes
    ap, ai = ops.split16(a)
    bp, bi = ops.split16(b)
    d = torch.empty(batch, m, n, device="cuda")
    ops.mm_split(ap, ai, bp, bi, d)
    one_chain = torch.empty_like(d)
    ops.mm_split(ap, ai, bp, bi, one_chain, promote=0)
    ops.assert_healthy()
    want = a.double() @ b.double().transpose(1, 2)
    for i in range(batch):
        rel = ((d[i].double() - want[i]).norm() / want[i].norm()).item()
        assert rel < 6e-7, rel  # short accumulation chains summed with round-to-nearest: FP32-level
        rel1 = ((one_chain[i].double() - want[i]).norm() / want[i].norm()).item()
        assert rel1 < 5e-6, rel1  # one chain of 96 truncating accumulator updates; FP16 alone gives 3e-4
    # planes reconstruct the source to ~2^-22 of its largest entry
    rec = (ap[0].double() + ap[1].double()) * ai.double()[:, None, None]
    assert ((rec - a.double()).abs().amax() / a.abs().amax()).item() < 2 ** -21


@pytest.mark.parametrize("promote", [0, 2])
def test_cta_pair_symmetric_split_product_matches_single_cta_tiles(ops, promote):
    """256 x 256 tiles on CTA pairs against 128 x 256 single-CTA tiles: FP16 hi/lo split product with a symmetric,
    mirrored result, all epilogue outputs (FP32, operand planes, statistics), sizes that leave ragged edge tiles."""
    batch, n = 3, 600
    x = rnd((batch, n, n), torch.float32, 9)
    x = x + x.transpose(1, 2)
    planes, inv = ops.split16(x)
    a = ops.operand(planes, seg_z=(0, 0, batch))
    b = ops.operand(planes, seg_z=(0, batch, 0))
    out = {}
    tiles = (256, 512) if promote else (256, 512, 1024)      # the wide tile has no chained accumulation
    for tile in tiles:
        d = torch.full((batch, n, n), float("nan"), device="cuda")
        sp = torch.zeros(2, batch, n, n, device="cuda", dtype=torch.float16)
        mx = torch.zeros(batch, device="cuda", dtype=torch.int32)
        desc_extra = dict(tri=True, mirror=True, promote=promote, maxabs=mx, tile_n=tile)
        ops.gemm(a, b, m=n, n=n, k=n, batch=batch, fmt=0, segs=3, d=d, alpha_a=inv, alpha_b=inv, **desc_extra)
        ops.assert_healthy()
        out[tile] = (d, mx.clone())
    want = x.double() @ x.double()
    for tile in tiles:
        # one chain over the whole depth adds by truncation (about 1.2e-7 per k-block on the all-positive diagonal)
        tol = 2e-6 if promote else 1e-5
        assert (out[tile][0].double() - want).abs().max().item() <= tol * want.abs().max().item()
        assert torch.equal(out[tile][0], out[tile][0].transpose(1, 2))
    for tile in tiles[1:]:
        assert torch.equal(out[256][0], out[tile][0])   # same accumulation order, same bits
        assert torch.equal(out[256][1], out[tile][1])


def test_a_wait_that_runs_out_is_reported_not_fatal(ops):
    """Failure detection on the device: a wait nothing will satisfy gives up after its limit, the kernel returns, the
    host reads the status word (and clears it), and the next product on the same context is correct."""
    import ctypes as C
    from toner_b200 import _lib
    lib = _lib.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.toner_selftest_bounded_wait(C.c_longlong(2_000_000), stream) == 0      # about a millisecond
    assert ops.device_status() == 199
    assert ops.device_status() == 0                                                    # read-and-clear
    a, b = rnd((128, 64), torch.bfloat16, 5), rnd((128, 64), torch.bfloat16, 6)
    d = torch.zeros(1, 128, 128, device="cuda")
    ops.gemm(ops.operand(a), ops.operand(b), m=128, n=128, k=64, batch=1, fmt=1, d=d)
    ops.assert_healthy()
    close(d[0], ref_mm(a, b, False, False), 64)


def test_fewer_ctas_give_the_same_bits(ops):
    """toner_set_gemm_sm_limit: the persistent kernel on 64 CTAs (32 pairs) walks the same tiles in the same order per
    tile, so results are bit-identical to the full grid; 0 restores one CTA per SM."""
    a, b = rnd((1024, 512), torch.bfloat16, 7), rnd((1536, 512), torch.bfloat16, 8)

    def run():
        d = torch.zeros(1, 1024, 1536, device="cuda")
        ops.gemm(ops.operand(a), ops.operand(b), m=1024, n=1536, k=512, batch=1, fmt=1, d=d)
        return d

    full = run()
    try:
        ops.set_gemm_sm_limit(64)
        limited = run()
        ops.set_gemm_sm_limit(3)      # rounded down to one pair
        tiny = run()
    finally:
        ops.set_gemm_sm_limit(0)
    ops.assert_healthy()
    assert torch.equal(full, limited) and torch.equal(full, tiny)
    close(full[0], ref_mm(a, b, False, False), 512)
