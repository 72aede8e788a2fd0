"""Row-capture oracle against the fixture made by the reference's own model code, and the host checks of the CUDA path."""

import os

import numpy as np
import pytest
import torch

from oracle import capture_oracle as cap

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "capture.npz"))


def bf16(name):
    return torch.from_numpy(GOLD[name].copy()).view(torch.bfloat16)


def test_norm_rows_match_the_references_norm_bit_for_bit():
    idx, eps = torch.from_numpy(GOLD["idx"]), float(GOLD["eps"])
    for src, w, rows in (("x", "w1", "rows_attn"), ("xmid", "w2", "rows_mlp")):
        got = cap.norm_rows(bf16(src), torch.from_numpy(GOLD[w]), idx, eps)
        assert torch.equal(got.view(torch.int16), bf16(rows).view(torch.int16))


def test_gathered_rows_and_destination_map():
    idx = torch.from_numpy(GOLD["idx"])
    rows = int(GOLD["batch"]) * idx.numel()
    at = torch.arange(rows).flip(0) + 5                       # reversed, offset into a larger buffer
    buf = torch.full((rows + 9, int(GOLD["hidden"])), 7.0, dtype=torch.bfloat16)
    cap.capture_rows([bf16("attn")], [buf], at, idx)
    assert torch.equal(buf[at], bf16("rows_o"))
    assert torch.all(buf[:5] == 7.0) and torch.all(buf[rows + 5:] == 7.0)


def test_recomputed_capture_fills_the_four_buffers_of_each_layer():
    idx, eps = torch.from_numpy(GOLD["idx"]), float(GOLD["eps"])
    rows, h = int(GOLD["batch"]) * idx.numel(), int(GOLD["hidden"])
    g = torch.Generator().manual_seed(1)
    gate = torch.randn(int(GOLD["batch"]), int(GOLD["seq"]), 2 * h, generator=g).to(torch.bfloat16)
    up = torch.randn(int(GOLD["batch"]), int(GOLD["seq"]), 2 * h, generator=g).to(torch.bfloat16)
    bufs = [torch.zeros(rows, w, dtype=torch.bfloat16) for w in (h, h, h, 2 * h)]
    cap.capture_recomputed([bf16("x")], [bf16("attn")], [bf16("xmid")], [gate], [up], [torch.from_numpy(GOLD["w1"])],
                           [torch.from_numpy(GOLD["w2"])], bufs, torch.arange(rows), idx, eps)
    assert torch.equal(bufs[0], bf16("rows_attn")) and torch.equal(bufs[1], bf16("rows_o"))
    assert torch.equal(bufs[2], bf16("rows_mlp"))
    want = (torch.nn.functional.silu(gate[:, idx].float()) * up[:, idx].float()).reshape(rows, -1)
    assert (bufs[3].float() - want).abs().max() <= 2.0 ** -8 * want.abs().max()   # one BF16 rounding of the FP32 value


def test_recomputed_rows_against_the_references_triton_kernels():
    """capture_recomputed of the reference (reproduce/marin/ops.py:107-163) run on a B200 by
    tests/golden/make_tpu_golden.py: two layers, hidden 64, gated width 160.  The SiLU-gated and copied rows agree
    bit for bit; the RMSNorm rows within one BF16 unit in the last place on a few elements in ten thousand (the
    kernel's mean square is summed in another order)."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "capture_recomputed.npz"))
    batch, seq, hidden, mlp, layers = (int(v) for v in g["dims"])
    idx, eps = torch.from_numpy(g["idx"]), float(g["eps"])

    def b16(name):
        return torch.from_numpy(g[name].copy()).view(torch.bfloat16)

    for l in range(layers):
        norm1 = cap.norm_rows(b16(f"x{l}"), torch.from_numpy(g[f"w1{l}"]), idx, eps)
        norm2 = cap.norm_rows(b16(f"xmid{l}"), torch.from_numpy(g[f"w2{l}"]), idx, eps)
        for got, want in ((norm1, b16(f"rows_attn{l}")), (norm2, b16(f"rows_mlp{l}"))):
            ulps = cap.bf16_ulps(got.contiguous(), want)
            assert int(ulps.max()) <= 1 and float((ulps > 0).float().mean()) < 2e-3
        assert torch.equal(b16(f"attn{l}")[:, idx].reshape(-1, hidden), b16(f"rows_o{l}"))
        gated = cap.silu_mul_rows(b16(f"g{l}"), b16(f"u{l}"), idx)
        assert torch.equal(gated.view(torch.int16), b16(f"rows_down{l}").view(torch.int16))


def test_ulps_helper():
    a = torch.tensor([1.0, -1.0, 0.0], dtype=torch.bfloat16)
    b = torch.tensor([1.0078125, -1.0078125, 0.0], dtype=torch.bfloat16)
    assert cap.bf16_ulps(a, b).tolist() == [1, 1, 0]


def test_the_cuda_path_refuses_cpu_tensors():
    from toner_b200 import capture
    x = torch.zeros(1, 8, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        capture.capture_rows([x], [torch.zeros(8, 8, dtype=torch.bfloat16)], torch.arange(8), torch.arange(8))
    with pytest.raises(ValueError):
        capture.capture_rows([x], [], torch.arange(8), torch.arange(8))
