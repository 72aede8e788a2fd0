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
