"""Forward capture of input second moments, with the interface of the reference's collector
(src/toner/statistics.py:11-155) and the Gram products on the sm_100a SYRK kernel.

Each hooked ``nn.Linear`` contributes the rows of its input (all rows of a 2-D input; the sampled
positions of a (..., sequence, features) input).  Their Gram ``X^T X`` is accumulated over
microbatches as a packed upper triangle in FP32, pooled over ranks at ``commit`` (half the bytes of
a full matrix), and handed to the optimizer as the mean ``sum(X^T X) / rows``.
"""

from __future__ import annotations

from collections.abc import Mapping
from contextlib import contextmanager
from typing import Dict, List

import torch
import torch.distributed as dist
from torch import nn

from . import ops


def sample_positions(sequence: int, head: int = 32, stride: int = 16) -> List[int]:
    """The first ``head`` positions, then head+1, head+1+stride, ...; with head == 0 the tail starts at 1
    (src/toner/statistics.py:68-71)."""
    first = list(range(min(head, sequence)))
    return first + list(range(head + 1 if head else 1, sequence, stride))


class ActivationStatistics:
    """Accumulate uncentred input second moments across forward microbatches.

    ``layers`` maps names to the ``nn.Linear`` modules a Toner optimizer updates.  Wrap exactly the
    forward passes that should count in ``capture()``; call ``commit(optimizer)`` once after all
    microbatches and before ``optimizer.step()``.
    """

    def __init__(self, layers: Mapping[str, nn.Linear], *, head: int = 32, stride: int = 16,
                 distributed: bool = True, process_group=None) -> None:
        if not layers:
            raise ValueError("Select at least one nn.Linear layer.")
        if head < 0 or stride < 1:
            raise ValueError("head must be nonnegative and stride positive.")
        self.layers = dict(layers)
        self.head, self.stride = head, stride
        self.distributed, self.process_group = distributed, process_group
        self._active = False
        self._closed = False
        self._sums: Dict[str, torch.Tensor] = {}
        self._counts: Dict[str, int] = {}
        self._positions: Dict[tuple, torch.Tensor] = {}
        seen = set()
        for name, layer in self.layers.items():
            if not isinstance(layer, nn.Linear):
                raise TypeError(f"{name}: expected nn.Linear.")
            if id(layer.weight) in seen:
                raise ValueError("Shared/tied weights require an explicit statistic; do not register them twice.")
            seen.add(id(layer.weight))
            if layer.in_features % 8:
                raise ValueError(f"{name}: toner_b200 needs input widths that are multiples of 8")
        self._handles = [layer.register_forward_pre_hook(self._make_hook(name)) for name, layer in self.layers.items()]

    # ------------------------------------------------------------------ capture
    def _gram_into(self, name: str, rows: torch.Tensor) -> None:
        """Add rows^T rows (FP32 accumulation) to the packed running sum of ``name``."""
        n = rows.shape[1]
        first = name not in self._sums
        if first:
            self._sums[name] = torch.empty(1, n * (n + 1) // 2, device=rows.device, dtype=torch.float32)
            self._counts[name] = 0
        out = self._sums[name]
        if rows.dtype == torch.bfloat16:
            ops.syrk_upper(rows.unsqueeze(0), out, ops.PACKED if first else ops.PACKED_ACC)
        elif rows.dtype == torch.float16:
            x = ops.operand(rows.unsqueeze(0), mn_major=True)
            ops.gemm(x, x, m=n, n=n, k=rows.shape[0], batch=1, fmt=0, d=out, tri=True, packed=True,
                     c=None if first else out, beta=0.0 if first else 1.0)
        else:  # FP32 rows: FP32-accurate Gram from FP16 hi/lo planes
            planes, inv = ops.split16(rows.float().unsqueeze(0))
            a = ops.operand(planes, mn_major=True, seg_z=(0, 0, 1))
            b = ops.operand(planes, mn_major=True, seg_z=(0, 1, 0))
            ops.gemm(a, b, m=n, n=n, k=rows.shape[0], batch=1, fmt=0, segs=3, d=out, tri=True, packed=True,
                     alpha_a=inv, alpha_b=inv, c=None if first else out, beta=0.0 if first else 1.0,
                     promote=ops.PROMOTE_ACCURATE)
        self._counts[name] += rows.shape[0]

    def _make_hook(self, name: str):
        @torch.no_grad()
        def collect(module, inputs):
            if not self._active:
                return
            if not inputs or not torch.is_tensor(inputs[0]):
                raise TypeError(f"{name}: capture expects a positional tensor input.")
            x = inputs[0].detach()
            if x.ndim < 2 or x.shape[-1] != module.in_features:
                raise ValueError(f"{name}: expected rows of {module.in_features} input features.")
            if not x.is_cuda:
                raise ValueError(f"{name}: toner_b200 captures CUDA activations only (there is no CPU path)")
            if x.ndim > 2:
                seq = x.shape[-2]
                key = (seq, x.device)
                if key not in self._positions:
                    positions = sample_positions(seq, self.head, self.stride)
                    if not positions:
                        raise ValueError(f"{name}: sampling selects no input positions.")
                    self._positions[key] = torch.tensor(positions, device=x.device, dtype=torch.long)
                x = x.index_select(-2, self._positions[key])
            # Linear's autocast happens after its pre-hook: use the values its GEMM will actually read.
            if torch.is_autocast_enabled(x.device.type):
                x = x.to(torch.get_autocast_dtype(x.device.type))
            x = x.reshape(-1, x.shape[-1]).contiguous()
            if not x.shape[0]:
                raise ValueError(f"{name}: cannot estimate a statistic from zero rows.")
            self._gram_into(name, x)

        return collect

    @contextmanager
    def capture(self):
        """Capture one forward; an exception discards the whole pending step."""
        if self._closed:
            raise RuntimeError("The statistic collector is closed.")
        if self._active:
            raise RuntimeError("Nested capture contexts would double-count activations.")
        self._active = True
        try:
            yield self
        except BaseException:
            self._active = False
            self.clear()
            raise
        finally:
            self._active = False

    # ------------------------------------------------------------------ commit
    @torch.no_grad()
    def commit(self, optimizer) -> None:
        """Pool the sums over ranks, update the optimizer's statistic EMAs once, clear the captures."""
        if self._active:
            raise RuntimeError("Exit capture() before committing statistics.")
        if self._closed:
            raise RuntimeError("The statistic collector is closed.")
        missing = [name for name in self.layers if name not in self._sums]
        if missing:
            raise RuntimeError(f"No captured inputs for: {', '.join(missing)}")
        pooled = self.distributed and dist.is_available() and dist.is_initialized()
        means = {}
        for name, layer in self.layers.items():
            packed = self._sums[name]
            rows = self._counts[name]
            if pooled:
                count = torch.tensor(rows, device=packed.device, dtype=torch.int64)
                dist.all_reduce(packed, group=self.process_group)
                dist.all_reduce(count, group=self.process_group)
                rows = int(count.item())
            n = layer.in_features
            mean = torch.zeros(1, n, n, device=packed.device, dtype=torch.float32)
            ops.unpack_ema(packed, mean, 0.0, 1.0 / float(rows))
            means[layer.weight] = mean[0]
        optimizer.update_statistics(means)
        self.clear()

    def clear(self) -> None:
        """Discard captured sums, for example after skipping a training step."""
        if self._active:
            raise RuntimeError("Cannot clear statistics during capture.")
        self._sums.clear()
        self._counts.clear()

    def close(self) -> None:
        for handle in self._handles:
            handle.remove()
        self._handles.clear()
        self.clear()
        self._closed = True
