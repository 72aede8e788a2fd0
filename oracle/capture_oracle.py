"""CPU restatement of the reference's row-capture operations.  TEST INFRASTRUCTURE ONLY: nothing in the product
imports this file.

Restates capture_rows / capture_recomputed (reproduce/marin/ops.py:30-54,107-163 and their kernels :10-27,63-100)
in plain torch on CPU:
  * gathered rows         bufs[i][at[b P + p]] = srcs[i][b, idx[p]]                              (ops.py:10-27)
  * RMSNorm rows          bf16(x rsqrt(mean x^2 + eps)) then bf16(w) * that, rounded to BF16      (ops.py:63-79)
                          -- the arithmetic of the model's own norm(), reproduce/marin/model.py:10-15
  * SiLU-gated rows       bf16(g (1 / (1 + exp(-g))) u), FP32 arithmetic and one rounding          (ops.py:82-100)
Pinned against the reference: the gathered and RMSNorm rows against the model's norm() and plain indexing on CPU
(tests/golden/capture.npz, made by tests/golden/make_capture_golden.py), and all four kinds of rows -- the SiLU-gated
ones exist only as a Triton kernel -- against capture_recomputed itself, run on a B200
(tests/golden/capture_recomputed.npz, made by tests/golden/make_tpu_golden.py): SiLU-gated and copied rows bit for bit,
RMSNorm rows within one BF16 unit in the last place.
"""

from __future__ import annotations

from typing import List, Sequence

import torch


def _rows(t: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """(B, T, D) -> (B * P, D): row b P + p is t[b, idx[p]]."""
    return t[:, idx].reshape(-1, t.size(-1))


def norm_rows(x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor, eps: float) -> torch.Tensor:
    xf = _rows(x, idx).float()
    out = (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)).to(torch.bfloat16)
    return (w.to(torch.bfloat16).float() * out.float()).to(torch.bfloat16)


def silu_mul_rows(g: torch.Tensor, u: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    gf, uf = _rows(g, idx).float(), _rows(u, idx).float()
    return (gf * (1.0 / (1.0 + torch.exp(-gf))) * uf).to(torch.bfloat16)


def capture_rows(srcs: Sequence[torch.Tensor], bufs: List[torch.Tensor], at: torch.Tensor, idx: torch.Tensor) -> None:
    for s, b in zip(srcs, bufs):
        b[at] = _rows(s, idx)


def capture_recomputed(xs, attn_out, xmid, gs, us, w1, w2, bufs, at, idx, eps) -> None:
    for l in range(len(xs)):
        b_attn, b_o, b_mlp, b_down = bufs[4 * l: 4 * l + 4]
        b_attn[at] = norm_rows(xs[l], w1[l], idx, eps)
        b_o[at] = _rows(attn_out[l], idx)
        b_mlp[at] = norm_rows(xmid[l], w2[l], idx, eps)
        b_down[at] = silu_mul_rows(gs[l], us[l], idx)


def bf16_ulps(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in BF16 units in the last place between two BF16 tensors (as int32)."""
    def key(t):
        v = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(v < 0, -(v & 0x7FFF), v)
    return (key(a) - key(b)).abs()
