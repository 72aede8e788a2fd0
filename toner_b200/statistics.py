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
        if len(layers) == 0:
            raise ValueError("no layers given: pass a mapping name -> nn.Linear")
        if stride < 1 or head < 0:
            raise ValueError("sampling needs head >= 0 and stride >= 1")
        self.layers = dict(layers)
        self.head = head
        self.stride = stride
        self.distributed = distributed
        self.process_group = process_group
        self._active = self._closed = False
        self._sums: Dict[str, torch.Tensor] = {}     # packed upper triangles, summed over microbatches
        self._counts: Dict[str, int] = {}            # rows behind each sum
        # Layers that read one and the same tensor (q, k, v of an attention block) have one and the same Gram: within a
        # capture() the first of them computes it and the others share the result (the reference computes it three times).
        self._shared: Dict[tuple, tuple] = {}        # input signature -> (layer that holds its sum, the tensor)
        self._alias: Dict[str, str] = {}             # layer -> layer whose sum it shares
        self._positions: Dict[tuple, torch.Tensor] = {}
        weights_seen = set()
        for name, layer in self.layers.items():
            if not isinstance(layer, nn.Linear):
                raise TypeError(f"layer '{name}' is a {type(layer).__name__}, not an nn.Linear")
            if layer.in_features % 8:
                raise ValueError(f"layer '{name}': toner_b200 needs input widths that are multiples of 8")
            if id(layer.weight) in weights_seen:
                raise ValueError(f"layer '{name}' shares its weight with another registered layer; a tied weight "
                                 "needs one explicit statistic")
            weights_seen.add(id(layer.weight))
        self._handles = []
        for name, layer in self.layers.items():
            self._handles.append(layer.register_forward_pre_hook(self._make_hook(name)))

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
            x = inputs[0] if inputs else None
            if not torch.is_tensor(x):
                raise TypeError(f"layer '{name}' was called without a positional tensor input")
            x = x.detach()
            if x.ndim < 2 or x.shape[-1] != module.in_features:
                raise ValueError(f"layer '{name}': input rows must have {module.in_features} features")
            if not x.is_cuda:
                raise ValueError(f"layer '{name}': toner_b200 captures CUDA activations only (there is no CPU path)")
            # Same storage, layout and version as a tensor another layer read in this forward: the same rows.  The first
            # reader's tensor is kept alive until the forward ends, so its address cannot be handed to a different
            # tensor in the meantime.
            signature = (x.data_ptr(), tuple(x.shape), tuple(x.stride()), x.dtype, x._version)
            first = self._shared.get(signature)
            if first is not None and (self._alias.get(name) == first[0] or
                                      (name not in self._alias and name not in self._sums)):
                self._alias[name] = first[0]
                return
            if name in self._alias:
                raise RuntimeError(f"layer '{name}' read the same tensor as '{self._alias[name]}' in an earlier microbatch "
                                   "of this step but not in this one")
            if first is None:
                self._shared[signature] = (name, x)
            if x.ndim > 2:  # (..., sequence, features): keep the sampled positions of every sequence
                key = (x.shape[-2], x.device)
                idx = self._positions.get(key)
                if idx is None:
                    chosen = sample_positions(x.shape[-2], self.head, self.stride)
                    if not chosen:
                        raise ValueError(f"layer '{name}': the sampling rule keeps no position of a length-"
                                         f"{x.shape[-2]} sequence")
                    idx = self._positions[key] = torch.tensor(chosen, device=x.device, dtype=torch.long)
                x = x.index_select(-2, idx)
            # The pre-hook runs before Linear's autocast: round to what its GEMM will actually read.
            if torch.is_autocast_enabled(x.device.type):
                x = x.to(torch.get_autocast_dtype(x.device.type))
            rows = x.reshape(-1, x.shape[-1]).contiguous()
            if rows.shape[0] == 0:
                raise ValueError(f"layer '{name}': no rows to estimate a statistic from")
            self._gram_into(name, rows)

        return collect

    @contextmanager
    def capture(self):
        """Capture one forward; an exception discards the whole pending step."""
        if self._closed:
            raise RuntimeError("capture() after close()")
        if self._active:
            raise RuntimeError("capture() is already active; nesting would count activations twice")
        self._active = True
        self._shared = {}
        failed = True
        try:
            yield self
            failed = False
        finally:
            self._active = False
            self._shared = {}
            if failed:  # a forward that raised may have captured only some layers: drop the pending step
                self.clear()

    # ------------------------------------------------------------------ commit
    @torch.no_grad()
    def commit(self, optimizer) -> None:
        """Pool the sums over ranks, update the optimizer's statistic EMAs once, clear the captures."""
        if self._closed:
            raise RuntimeError("commit() after close()")
        if self._active:
            raise RuntimeError("commit() inside capture(); leave the context first")
        absent = sorted(set(self.layers) - set(self._sums) - set(self._alias))
        if absent:
            raise RuntimeError("nothing was captured for layer(s): " + ", ".join(absent))
        pooled = self.distributed and dist.is_available() and dist.is_initialized()
        means = {}
        done: Dict[str, torch.Tensor] = {}
        for name, layer in self.layers.items():
            source = self._alias.get(name, name)
            if source in done:                       # shares its input with a layer already pooled: the same mean
                means[layer.weight] = done[source]
                continue
            packed = self._sums[source]
            rows = self._counts[source]
            if pooled:
                count = torch.tensor(rows, device=packed.device, dtype=torch.int64)
                dist.all_reduce(packed, group=self.process_group)
                dist.all_reduce(count, group=self.process_group)
                rows = int(count.item())
            n = layer.in_features
            mean = torch.zeros(1, n, n, device=packed.device, dtype=torch.float32)
            ops.unpack_ema(packed, mean, 0.0, 1.0 / float(rows))
            means[layer.weight] = done[source] = mean[0]
        optimizer.update_statistics(means)
        self.clear()

    def clear(self) -> None:
        """Discard captured sums, for example after skipping a training step."""
        if self._active:
            raise RuntimeError("clear() inside capture()")
        self._sums = {}
        self._counts = {}
        self._alias = {}

    def close(self) -> None:
        while self._handles:
            self._handles.pop().remove()
        self.clear()
        self._closed = True
