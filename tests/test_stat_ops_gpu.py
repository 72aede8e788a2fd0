"""Statistic path through the C ABI against the CPU oracle: upper-triangle SYRK in its three output
modes, the packed-triangle EMA and the FP16 hi/lo split."""

import pytest
import torch

from oracle import toner_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from toner_b200 import ops as _ops
    return _ops


def rows_bf16(k, rows, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(k, rows, n, generator=g).to(torch.bfloat16)


@pytest.mark.parametrize("k,rows,n", [(1, 64, 256), (3, 752, 768), (2, 1000, 328), (1, 6016, 3072), (2, 94, 2048)])
def test_syrk_packed_matches_oracle_gram(ops, k, rows, n):
    x = rows_bf16(k, rows, n, 0)
    out = torch.full((k, n * (n + 1) // 2), float("nan"), device="cuda")
    ops.syrk_upper(x.cuda(), out, ops.PACKED)
    ops.assert_healthy()
    for b in range(k):
        want = orc.pack_upper(orc.gram(x[b]))
        got = out[b].cpu()
        # Products are exact; the tensor core adds each 16-deep partial sum into its FP32 accumulator by
        # truncation, so long all-positive sums (the diagonal) come out low by up to depth/16 * 2^-24, where
        # the kernel keeps the depth of one accumulation chain at 4096 rows or less.
        tol = 2e-6 + (min(rows, 4096) / 16) * 2.0 ** -24
        assert orc.rel_fro(got[None], want[None]) < tol
        assert (got - want).abs().max() <= 2 * tol * want.abs().max()


def test_syrk_list_equals_stack_bitwise_and_accumulates(ops):
    """Separately allocated buffers give the same bits as a stacked tensor (the reference's own
    list-vs-stack expectation), and PACKED_ACC adds to what is there."""
    k, rows, n = 4, 300, 512
    x = rows_bf16(k, rows, n, 1).cuda()
    stacked = torch.empty(k, n * (n + 1) // 2, device="cuda")
    ops.syrk_upper(x, stacked, ops.PACKED)
    listed = torch.empty_like(stacked)
    ops.syrk_upper([x[i].clone() for i in range(k)], listed, ops.PACKED)
    ops.assert_healthy()
    assert torch.equal(stacked, listed)
    acc = stacked.clone()
    ops.syrk_upper(x, acc, ops.PACKED_ACC)
    ops.assert_healthy()
    assert torch.equal(acc, stacked + stacked)


@pytest.mark.parametrize("n", [256, 776])
def test_syrk_fused_ema_and_unpack_ema_agree_with_oracle(ops, n):
    k, rows = 2, 500
    x = rows_bf16(k, rows, n, 2)
    g = torch.Generator().manual_seed(3)
    base = torch.randn(k, n, n, generator=g)
    base = base + base.transpose(1, 2)  # an EMA is symmetric
    beta, gamma = 0.95, 0.05 / rows
    want = torch.stack([orc.unpack_ema(orc.pack_upper(orc.gram(x[b])), base[b], beta, gamma) for b in range(k)])
    fused = base.clone().cuda()
    ops.syrk_upper(x.cuda(), fused, ops.EMA_FULL, beta, gamma)
    packed = torch.empty(k, n * (n + 1) // 2, device="cuda")
    ops.syrk_upper(x.cuda(), packed, ops.PACKED)
    two_step = base.clone().cuda()
    ops.unpack_ema(packed, two_step, beta, gamma)
    ops.assert_healthy()
    for got in (fused, two_step):
        assert orc.rel_fro(got.cpu().reshape(k * n, n), want.reshape(k * n, n)) < 1e-6
        assert torch.equal(got, got.transpose(1, 2)), "the EMA must stay exactly symmetric"


def test_unpack_ema_first_step_from_zero(ops):
    n, k = 136, 3
    g = torch.Generator().manual_seed(4)
    full = torch.randn(k, n, n, generator=g)
    full = full + full.transpose(1, 2)
    packed = torch.stack([orc.pack_upper(full[b]) for b in range(k)]).cuda()
    ema = torch.zeros(k, n, n, device="cuda")
    ops.unpack_ema(packed, ema, 0.9, 0.1)
    assert torch.allclose(ema.cpu(), 0.1 * full, rtol=1e-6, atol=1e-7)


def test_syrk_rejects_bad_arguments(ops):
    x = torch.zeros(1, 16, 12, device="cuda", dtype=torch.bfloat16)  # n not a multiple of 8
    with pytest.raises(Exception):
        ops.syrk_upper(x, torch.zeros(1, 78, device="cuda"), ops.PACKED)
    with pytest.raises(ValueError):
        ops.syrk_upper(torch.zeros(1, 16, 16), torch.zeros(1, 136), ops.PACKED)  # CPU tensors: no CPU path


def test_split16_affine_source(ops):
    n = 200
    g = torch.Generator().manual_seed(5)
    m = torch.randn(2, n, n, generator=g).cuda()
    planes, inv = ops.split16(m, aff=(1.5, -0.25))
    want = 1.5 * torch.eye(n, device="cuda") - 0.25 * m
    rec = (planes[0].double() + planes[1].double()) * inv.double()[:, None, None]
    assert ((rec - want.double()).abs().amax() / want.abs().amax()).item() < 2 ** -21
    assert planes[0].float().abs().amax().item() < 2 ** 14


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gather_rows_matches_index_select(ops, dtype):
    """Sampled-row capture: bit-exact against index_select + BF16 rounding, also from a strided view."""
    from toner_b200.statistics import sample_positions
    g = torch.Generator(device="cuda").manual_seed(2)
    batch, seq, n = 3, 200, 264
    wide = torch.randn(batch, seq, n + 24, device="cuda", generator=g).to(dtype)
    x = wide[:, :, 8:8 + n]                              # rows 16-byte aligned, not contiguous
    pos = sample_positions(seq, 32, 16)
    positions = torch.tensor(pos, device="cuda", dtype=torch.int32)
    dst = torch.full((batch * len(pos), n), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gather_rows(x, positions, dst)
    ops.assert_healthy()
    want = x.index_select(1, positions.long()).to(torch.bfloat16).reshape(batch * len(pos), n)
    assert torch.equal(dst, want)
    assert orc.sample_positions(seq, 32, 16) == pos
