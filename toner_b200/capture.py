"""Sampled-row capture after the forward pass, one launch per micro-batch for the whole model.

Host-side mirror of the two operations the reference's Marin trainer calls once per micro-batch
(``capture_rows`` and ``capture_recomputed``, reproduce/marin/ops.py:30-54,107-163): same names, argument order and
meaning.  The rows are written by ``toner_capture`` (csrc/capture_ops.cu); there is no other path.

A job table is built once per set of tensor addresses and kept on the device: the activations' addresses repeat
across micro-batches (caching allocator), so in steady state nothing is built or copied (the reference caches its
pointer tables the same way, reproduce/marin/ops.py:103-105,142-157).
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence, Tuple

import torch

from . import _lib
from ._lib import check
from .ops import _need_cuda, _stream

COPY, RMSNORM, SILU_MUL, COPY_F32 = 0, 1, 2, 3
_TABLES: Dict[tuple, Tuple[object, torch.Tensor]] = {}
_MAX_TABLES = 64


def _job(kind: int, a: torch.Tensor, b, dst: torch.Tensor) -> Tuple[int, int, int, int, int, int, int]:
    if kind == COPY and a.dtype == torch.float32:
        kind = COPY_F32                                  # rounded to BF16 on the way, as autocast would
    if a.dtype != (torch.float32 if kind == COPY_F32 else torch.bfloat16) or a.ndim != 3 or a.stride(-1) != 1:
        raise ValueError("capture sources are (batch, seq, width) BF16 tensors with contiguous features "
                         "(copied rows may also come from FP32 tensors)")
    width = a.size(-1)
    if dst.dtype != torch.bfloat16 or dst.ndim != 2 or dst.size(1) != width or not dst.is_contiguous():
        raise ValueError("capture destinations are contiguous (capacity, width) BF16 row buffers")
    if kind == RMSNORM and (b.dtype != torch.float32 or b.numel() != width or not b.is_contiguous()):
        raise ValueError("the norm weight is a contiguous FP32 vector of the row width")
    if kind == SILU_MUL and (b.dtype != torch.bfloat16 or b.shape != a.shape or b.stride() != a.stride()):
        raise ValueError("gate and up projections must share dtype, shape and strides")
    return (a.data_ptr(), 0 if b is None else b.data_ptr(), dst.data_ptr(), a.stride(0), a.stride(1), width, kind)


def _signature(t: torch.Tensor) -> tuple:
    return (t.dtype, tuple(t.shape), t.stride())


def _run(key: tuple, build, batch: int, at: torch.Tensor, idx: torch.Tensor, eps: float) -> None:
    """Launch the jobs `build()` describes; `key` (addresses and layouts) names the cached table."""
    entry = _TABLES.get(key)
    if entry is None:
        jobs = build()                               # full validation happens here, once per set of addresses
        if len(_TABLES) >= _MAX_TABLES:              # addresses that keep changing: keep the cache bounded
            _TABLES.clear()
        host = (_lib.CaptureJob * len(jobs))(*[_lib.CaptureJob(*j) for j in jobs])
        raw = torch.frombuffer(bytearray(bytes(host)), dtype=torch.uint8)
        entry = _TABLES[key] = (host, raw.pin_memory().to(at.device, non_blocking=True), len(jobs))
    host, dev, count = entry
    if at.dtype != torch.int64 or idx.dtype != torch.int64 or not (at.is_contiguous() and idx.is_contiguous()):
        raise ValueError("`at` and `idx` are contiguous int64 device tensors")
    positions = idx.numel()
    if at.numel() != batch * positions:
        raise ValueError("`at` must name one destination row per (sequence, sampled position)")
    _need_cuda(at, idx)
    check(_lib.load().toner_capture(dev.data_ptr(), C.addressof(host), count, at.data_ptr(), idx.data_ptr(), batch,
                                    positions, float(eps), _stream()), "toner_capture")


def capture_rows(srcs: Sequence[torch.Tensor], bufs: Sequence[torch.Tensor], at: torch.Tensor, idx: torch.Tensor) -> None:
    """bufs[i][at[b P + p]] = srcs[i][b, idx[p]] for BF16 inputs srcs[i] (B, T, D_i) and row buffers (rows, D_i)
    (capture_rows, reproduce/marin/ops.py:30-54).  FP32 inputs are rounded to BF16 (the fast optimizers' hooks see a
    projection's input before autocast casts it)."""
    if len(srcs) != len(bufs) or not srcs:
        raise ValueError("one row buffer per source")
    batch = srcs[0].size(0)

    def build():
        _need_cuda(*srcs, *bufs)
        if any(s.size(0) != batch for s in srcs):
            raise ValueError("all sources hold the same micro-batch")
        return [_job(COPY, s, None, d) for s, d in zip(srcs, bufs)]

    key = ("rows", tuple(t.data_ptr() for t in srcs), tuple(t.data_ptr() for t in bufs),
           tuple(_signature(t) for t in srcs), tuple(_signature(t) for t in bufs))
    _run(key, build, batch, at, idx, 0.0)


def capture_recomputed(xs, attn_out, xmid, gs, us, w1, w2, bufs, at: torch.Tensor, idx: torch.Tensor, eps: float) -> None:
    """Per layer l (bufs in blocks of four: attn, o, mlp, down): norm(ln1, x) | a | norm(ln2, x_mid) | silu(g) * u at
    the sampled rows into the row buffers; inputs BF16 (B, T, D), norm weights FP32
    (capture_recomputed, reproduce/marin/ops.py:107-163).  As there, the tensors of one list must share dtype, shape
    and strides; that is checked when a new set of addresses is first seen."""
    layers = len(xs)
    if not layers or not all(len(t) == layers for t in (attn_out, xmid, gs, us, w1, w2)) or len(bufs) != 4 * layers:
        raise ValueError("one entry per layer in every list and four row buffers per layer")
    batch = xs[0].size(0)
    cols = (xs, attn_out, xmid, gs, us, w1, w2, bufs)

    def build():
        _need_cuda(*(t for col in cols for t in col))
        x0, g0 = _signature(xs[0]), _signature(gs[0])
        if any(_signature(t) != x0 for t in (*xs, *attn_out, *xmid)) or any(_signature(t) != g0 for t in (*gs, *us)):
            raise ValueError("hidden-width tensors must share one layout, and gate / up projections another")
        if g0[1][0] != batch:
            raise ValueError("all sources hold the same micro-batch")
        jobs = []
        for l in range(layers):
            b_attn, b_o, b_mlp, b_down = bufs[4 * l: 4 * l + 4]
            jobs.append(_job(RMSNORM, xs[l], w1[l], b_attn))
            jobs.append(_job(COPY, attn_out[l], None, b_o))
            jobs.append(_job(RMSNORM, xmid[l], w2[l], b_mlp))
            jobs.append(_job(SILU_MUL, gs[l], us[l], b_down))
        return jobs

    key = ("recomputed", tuple(t.data_ptr() for col in cols for t in col), _signature(xs[0]), _signature(gs[0]),
           _signature(bufs[0]), _signature(bufs[3]), w1[0].dtype)
    _run(key, build, batch, at, idx, eps)
