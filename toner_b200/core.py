"""Step arithmetic shared by the general optimizers and the layer-sharded engine.

Everything numerical happens in the CUDA library (``ops``); this module sequences the launches for
one *factor set* (a stack of equally sized input statistics) and one *matrix group* (a stack of
equally shaped weights whose statistics sit at regular positions in a factor set).

Numerical specification followed (reference files):
  factors   src/toner/linalg.py:54-89      A = sym(C)/mean(diag C) + damping I, R_s = A^-s,
                                           decay = R_out^2 n / ||R_out||_F^2
  MuonT     src/toner/reference.py:186-215 m <- mu m + g, d = g + mu m, P = NS(d R_in),
                                           W <- W - lr wd W decay - lr sqrt(max(1, out/in)) P R_out sqrt(n)/||R_out||_F
  AdamT     src/toner/reference.py:287-313
The two right-multiplications of the MuonT update are fused the way the reference's engine does it
(src/toner/fast/engine.py:42-51):  delta = -((lr wd n/||R||^2) W R + (lr s sqrt(n)/||R||) P) R.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import ops


class Scratch:
    """Named persistent device buffers.  Stable addresses keep the library's TMA tensor maps cached."""

    def __init__(self) -> None:
        self._buffers: Dict[Tuple, torch.Tensor] = {}

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        key = (name, tuple(shape), dtype, str(device))
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty(tuple(shape), dtype=dtype, device=device)
            self._buffers[key] = buf
        return buf

    def bytes_like(self, name: str, nbytes: int, device: torch.device) -> torch.Tensor:
        """A byte workspace that only ever grows."""
        key = (name, "bytes", str(device))
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
            self._buffers[key] = buf
        return buf


def root_orders(strength_a: float, strength_b: float) -> Tuple[int, int]:
    """Map two inverse-power strengths to (p, q): the weaker is A^(-1/p), the stronger A^(-q/p).

    The Newton factor engine computes inverse p-th roots for p a power of two; other strengths are
    rejected (the reference's fast path is narrower still: 1/8, 1/4, 1/2, src/toner/fast/adapter.py:169-171)."""
    nz = [s for s in (strength_a, strength_b) if s != 0]
    for s in nz:
        inv = 1.0 / s
        if s < 0 or abs(inv - round(inv)) > 1e-9 or int(round(inv)) & (int(round(inv)) - 1) or round(inv) > 32:
            raise ValueError("strengths must be 0 or 1/p with p a power of two up to 32 "
                             "(the factor engine is a coupled Newton inverse p-th root)")
    if not nz:
        return 1, 1
    p = int(round(1.0 / min(nz)))
    q = int(round(max(nz) * p))
    return p, q


class FactorSet:
    """EMAs of k input statistics of width n and their inverse-power factors, stacked.

    ``strengths`` = (inner, outer).  After :meth:`compute`, ``planes(which)`` gives the FP16 hi/lo planes
    (2, k, n, n) and inverse scales (k,) of the requested factor, ``fro2_outer`` the squared Frobenius norm
    of the outer factor."""

    def __init__(self, k: int, n: int, device: torch.device, strengths: Tuple[float, float], damping: float,
                 scratch: Optional[Scratch] = None, chunk: Optional[int] = None) -> None:
        if n % 8:
            raise ValueError("statistic width must be a multiple of 8 (TMA row pitch of the 16-bit operands)")
        self.k, self.n, self.device, self.damping = k, n, device, float(damping)
        self.inner_strength, self.outer_strength = float(strengths[0]), float(strengths[1])
        self.p, self.q = root_orders(*strengths)
        self.scratch = scratch or Scratch()
        self.ema = torch.zeros(k, n, n, device=device, dtype=torch.float32)
        self.weight = 0.0
        self.root_lo = torch.empty(k, n, n, device=device, dtype=torch.float32)
        self.root_hi = torch.empty(k, n, n, device=device, dtype=torch.float32) if self.q > 1 else None
        self.fro2_lo = torch.empty(k, device=device, dtype=torch.float32)
        self.fro2_hi = torch.empty(k, device=device, dtype=torch.float32) if self.q > 1 else None
        self.status = torch.zeros(k, device=device, dtype=torch.int32)
        self.status_host = torch.zeros(k, dtype=torch.int32).pin_memory()
        # ||A'||_F of every statistic as the last factorisation saw it: next step's spectrum bound comes from it
        # (the statistics are EMAs and move by a few percent per step)
        self.norms = torch.zeros(k, device=device, dtype=torch.float32)
        self.norms_host = torch.zeros(k, dtype=torch.float32).pin_memory()
        self.lower = 0.0
        # Tracking of each statistic's smallest eigenvalue (toner_inv_roots_tracked): with it the next step's Newton
        # schedule starts from an estimate of the actual spectrum (verified after the chain) instead of the bound
        # damping / norm, which is far too pessimistic for well-conditioned statistics.
        self.tracking = True
        self.track = torch.zeros(k, n, device=device, dtype=torch.float32)
        self.lmin = torch.zeros(k, device=device, dtype=torch.float32)
        self.lmin_host = torch.zeros(k, dtype=torch.float32).pin_memory()
        self.track_restart = True        # the vectors hold nothing yet (or the statistics were replaced)
        # Dominant directions (outlier features): eight vector slots per statistic, found by block power iteration and
        # deflated where they stand out.  The block is two vectors wider than the number of directions that looked like
        # outliers last time (a block wider than the group of outliers is what makes close outliers converge).
        self.deflate = torch.zeros(k, 8, n, device=device, dtype=torch.float32)
        self.deflated = torch.zeros(k, device=device, dtype=torch.int32)
        self.deflated_host = torch.zeros(k, dtype=torch.int32).pin_memory()
        self.deflate_rank = 4
        self.block_deflation = True      # False: the engine's own single-vector deflation (one dominant direction)
        self.ritz_norm = True            # the norm from the block iteration once it has followed the statistic for two steps
        self._warm_calls = 0             # tracked calls in a row whose vectors came from the call before
        self._rank_used = 0              # block width of the last call
        self.lower_is_estimate = False
        self.estimate_backoff = 0        # steps left during which only certified bounds are used (after a bound failed)
        self.bound_failures = 0
        self.status_event: Optional[torch.cuda.Event] = None
        self.health = ops.Health()
        self._root_bounds = None
        self.lo_planes = torch.empty(2, k, n, n, device=device, dtype=torch.float16)
        self.lo_inv = torch.empty(k, device=device, dtype=torch.float32)
        if self.q > 1:
            self.hi_planes = torch.empty(2, k, n, n, device=device, dtype=torch.float16)
            self.hi_inv = torch.empty(k, device=device, dtype=torch.float32)
        else:
            self.hi_planes, self.hi_inv = self.lo_planes, self.lo_inv
        per = ops.inv_roots_workspace_bytes(1, n)
        if k == 0:            # a rank that owns no statistic of this width (weighted ownership): nothing to factor
            self.workspace = None
            self.iterations = self.finish_order = 0
            self.fallbacks = self.repairs = 0
            return
        if chunk is None:
            # One launch over all statistics keeps the persistent kernel's last wave full (24 statistics of width
            # 5632 are 83 waves of pair tiles; five at a time would be 18 waves per launch with a ragged tail each).
            budget = min(32 << 30, torch.cuda.get_device_properties(device).total_memory // 5)
            chunk = max(1, min(k, budget // per))
        self.workspace = self.scratch.bytes_like("inv_roots", ops.inv_roots_workspace_bytes(chunk, n), device)
        self.iterations = ops.inv_roots_iterations(n, self.damping, self.p)
        self.finish_order = ops.inv_roots_finish_order(n, self.damping, self.p)
        self.fallbacks = 0
        self.repairs = 0

    # -- which stored root serves a given strength
    def _is_hi(self, strength: float) -> bool:
        return self.q > 1 and strength == max(self.inner_strength, self.outer_strength)

    def planes(self, which: str) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        s = self.inner_strength if which == "inner" else self.outer_strength
        if s == 0:
            return None, None  # identity factor: the product is skipped
        return (self.hi_planes, self.hi_inv) if self._is_hi(s) else (self.lo_planes, self.lo_inv)

    def root(self, which: str) -> Optional[torch.Tensor]:
        s = self.inner_strength if which == "inner" else self.outer_strength
        if s == 0:
            return None
        return self.root_hi if self._is_hi(s) else self.root_lo

    @property
    def fro2_outer(self) -> torch.Tensor:
        if self.outer_strength == 0:
            raise ValueError("outer strength 0 has no factor norm")
        return self.fro2_hi if self._is_hi(self.outer_strength) else self.fro2_lo

    def compute(self) -> None:
        """Enqueue the Newton factor computation and the operand split of the results."""
        if self.k == 0 or (self.inner_strength == 0 and self.outer_strength == 0):
            return
        blocked = self.tracking and self.block_deflation
        # The largest Ritz value left in the statistic replaces the norm bound's three squarings when the vector it
        # belongs to is at least two calls old (a fresh slot's Rayleigh quotient sits near the MEAN eigenvalue) and the
        # lower bound is an estimate as well, so that both are verified after the chain.
        ritz = (blocked and self.ritz_norm and self.lower_is_estimate and not self.track_restart
                and self._warm_calls >= 2
                and int((self.deflated_host & 255).max()) < min(self._rank_used, self.deflate_rank))
        self._warm_calls = 0 if (self.track_restart or not blocked) else self._warm_calls + 1
        self._rank_used = self.deflate_rank if blocked else 0
        self.ritz_in_flight = bool(ritz)
        ops.inv_roots(self.ema, self.damping, self.p, self.q, root_lo=self.root_lo, root_hi=self.root_hi,
                      fro2_lo=self.fro2_lo, status=self.status, workspace=self.workspace, lower=self.lower,
                      norms=self.norms, lower_is_estimate=self.lower_is_estimate,
                      track=self.track if self.tracking else None, lmin=self.lmin if self.tracking else None,
                      track_sweeps=(12 if self.track_restart else 4) if self.tracking else 0,
                      track_restart=self.track_restart,
                      deflate=self.deflate if self.tracking and self.block_deflation else None,
                      deflate_rank=self.deflate_rank,
                      deflate_restart=self.track_restart, deflated=self.deflated if self.tracking else None,
                      ritz_norm=ritz)
        self.track_restart = False
        self._estimate_in_flight = self.lower_is_estimate
        self.iterations = (ops.inv_roots_iterations_for(self.lower, self.p) if self.lower > 0
                           else ops.inv_roots_iterations(self.n, self.damping, self.p))
        self.finish_order = ops.inv_roots_finish_order(self.n, self.damping, self.p, self.lower)
        self._split()
        self.status_host.copy_(self.status, non_blocking=True)
        self.norms_host.copy_(self.norms, non_blocking=True)
        self.lmin_host.copy_(self.lmin, non_blocking=True)
        self.deflated_host.copy_(self.deflated, non_blocking=True)
        self.health.arm("the factor computation")
        self.status_event = torch.cuda.Event()
        self.status_event.record(torch.cuda.current_stream())

    def statistics_replaced(self) -> None:
        """The EMAs were overwritten from outside (a checkpoint): nothing learnt from earlier factorisations applies."""
        self.lower, self.lower_is_estimate, self.track_restart, self.estimate_backoff = 0.0, False, True, 0
        self._warm_calls = 0

    def _split(self) -> None:
        # Operand planes of the roots, scaled by a bound known without a pass over them: the statistic is factored
        # with damping added, so no entry of A^-s exceeds damping^-s.
        if self._root_bounds is None:
            bits = lambda s: torch.full((self.k,), 1.01 * self.damping ** -s, device=self.device,
                                        dtype=torch.float32).view(torch.int32)
            self._root_bounds = (bits(1.0 / self.p), bits(self.q / self.p))
        ops.split16(self.root_lo, planes=self.lo_planes, inv_scale=self.lo_inv, maxabs=self._root_bounds[0])
        if self.q > 1:
            ops.split16(self.root_hi, planes=self.hi_planes, inv_scale=self.hi_inv, maxabs=self._root_bounds[1])
            if self.outer_strength != 0 and self._is_hi(self.outer_strength):   # (only the outer factor's norm is used)
                ops.sumsq(self.root_hi, out=self.fro2_hi,
                          scratch=self.scratch.bytes_like("sumsq", ops.sumsq_scratch_bytes(self.k), self.device))

    def finish(self) -> int:
        """Wait for the convergence flags only; recompute flagged statistics by eigendecomposition (the
        reference's exact fallback, src/toner/fast/engine.py:714-731).  Returns how many were flagged."""
        if self.status_event is None:
            return 0
        self.status_event.synchronize()
        self.status_event = None
        self.health.check()   # a product of the factor engine that gave up a wait: raise before the factors are used
        codes = self.status_host.tolist()
        bad = [i for i, s in enumerate(codes) if s != 0]
        # Next step's bound.  Certified: damping / norm of the widest statistic, with room for one step of EMA drift.
        # Estimated (tracking): the smallest eigenvalue found in this step's roots over the norm, halved -- the
        # estimate errs high by up to a quarter, the statistic moves by a few percent per step -- and used only where it
        # buys a step.  A flagged statistic (not converged, or below the bound used) sends the next step back to the
        # bound that always holds; an estimate that failed its verification is not tried again for eight steps.
        top = float(self.norms_host.max())
        worst = self.damping / (self.n * (1.0 + self.damping))
        if self.tracking and self.block_deflation:
            candidates = int((self.deflated_host >> 8).max())
            self.deflate_rank = max(2, min(8, candidates + 2))
        self.lower, self.lower_is_estimate = 0.0, False
        if getattr(self, "_estimate_in_flight", False) and any(c in (1, 4) for c in codes):
            self.estimate_backoff = 8     # (a gross overestimate already fails the convergence test, status 1)
            self.bound_failures += 1
        elif self.estimate_backoff:
            self.estimate_backoff -= 1
        if all(c in (0, 4) or (c == 1 and getattr(self, "_estimate_in_flight", False)) for c in codes) \
                and math.isfinite(top) and top > 0:
            # (a norm taken from the block iteration is an estimate and sits up to a third below the certified bound
            # the device will check this hint against)
            hint = 0.6 * self.damping / (top * (1.5 if getattr(self, "ritz_in_flight", False) else 1.0))
            if worst < hint < 1.0:
                self.lower = hint
            if self.tracking and not self.estimate_backoff and not bad:
                ratio = float((self.lmin_host / self.norms_host).min())
                guess = min(0.5 * ratio, 0.8)
                if math.isfinite(guess) and guess > 1.5 * max(self.lower, worst):
                    self.lower, self.lower_is_estimate = guess, True
        if not bad:
            return 0
        # Repair round (the reference's engine repairs flagged roots before it falls back,
        # src/toner/fast/engine.py:646-713): the flagged statistics once more with the bound that always holds.
        self.repairs += len(bad)
        idx = torch.tensor(bad, device=self.device)
        sub = self.ema.index_select(0, idx).contiguous()
        lo, hi, fro2, st = ops.inv_roots(sub, self.damping, self.p, self.q)
        self.root_lo.index_copy_(0, idx, lo)
        if self.q > 1:
            self.root_hi.index_copy_(0, idx, hi)
        still = [b for b, s in zip(bad, st.tolist()) if s != 0]   # host sync: this path is the exception
        bad = still
        self.fallbacks += len(bad)
        for i in bad:
            c = self.ema[i]
            c = 0.5 * (c + c.T)
            lam, vec = torch.linalg.eigh(c.double())
            lam = lam.clamp_min(0)
            unit = lam / lam.mean().clamp_min(1e-30)
            self.root_lo[i] = ((vec * (unit + self.damping).pow(-1.0 / self.p)) @ vec.T).float()
            if self.q > 1:
                self.root_hi[i] = ((vec * (unit + self.damping).pow(-float(self.q) / self.p)) @ vec.T).float()
        ops.sumsq(self.root_lo, out=self.fro2_lo, scratch=self.scratch.bytes_like("sumsq", ops.sumsq_scratch_bytes(self.k), self.device))
        self._split()
        return len(bad) if bad else 0


class MatrixGroup:
    """Equally shaped weights whose input statistics are entries first, first+step, ... of a FactorSet."""

    def __init__(self, weights: Sequence[torch.Tensor], factors: FactorSet, first: int, step: int, kind: str) -> None:
        self.weights = list(weights)
        w0 = self.weights[0]
        self.count = len(self.weights)
        self.out_features, self.in_features = w0.shape
        if self.in_features != factors.n:
            raise ValueError("weight input width does not match its statistic")
        if self.out_features % 8 or self.in_features % 8:
            raise ValueError("matrix dimensions must be multiples of 8 (TMA row pitch of the 16-bit operands)")
        for w in self.weights:
            if w.shape != w0.shape or w.dtype != torch.float32 or not w.is_contiguous() or w.device != w0.device:
                raise ValueError("a matrix group needs equally shaped, contiguous FP32 weights on one device")
        self.factors, self.first, self.step, self.kind = factors, first, step, kind
        self.device = w0.device
        shape = (self.count, self.out_features, self.in_features)
        self.m = torch.zeros(shape, device=self.device, dtype=torch.float32)
        self.v = torch.zeros(shape, device=self.device, dtype=torch.float32) if kind == "adamt" else None
        self.weight_ptrs = ops.pointer_table(self.weights)
        self._grad_key: Optional[Tuple[int, ...]] = None
        self._grad_ptrs: Optional[torch.Tensor] = None

    def grad_ptrs(self, grads: Sequence[torch.Tensor]) -> torch.Tensor:
        for g in grads:
            if g.dtype != torch.float32 or not g.is_contiguous() or g.shape != self.weights[0].shape:
                raise ValueError("gradients must be contiguous FP32 tensors of the weight's shape")
        key = tuple(g.data_ptr() for g in grads)
        if key != self._grad_key:
            self._grad_ptrs = ops.pointer_table(grads)
            self._grad_key = key
        return self._grad_ptrs


def _product(a_planes, a_inv, group: MatrixGroup, which: str, d, coarse: bool = False, **kw) -> None:
    """d[b] = A[b] @ R[first + b*step], R the inner or outer factor (symmetric).  FP32-accurate from the FP16 hi/lo
    planes (three plane products in one accumulator); ``coarse`` multiplies the hi planes only (relative error
    about 5e-4), for terms that enter the result with a small coefficient."""
    f = group.factors
    r_planes, r_inv = f.planes(which)
    count, m, n = group.count, group.out_features, group.in_features
    if coarse:
        a = ops.operand(a_planes, seg_z=(0, 0, 0))
        b = ops.operand(r_planes, seg_z=(group.first, group.first, group.first), z_step=group.step)
        segs = 1
    else:
        a = ops.operand(a_planes, seg_z=(0, 0, count))
        b = ops.operand(r_planes, seg_z=(group.first, f.k + group.first, group.first), z_step=group.step)
        segs = 3
    ops.gemm(a, b, m=m, n=n, k=n, batch=count, fmt=0, segs=segs, d=d, alpha_a=a_inv,
             alpha_b=r_inv[group.first:], alpha_b_step=group.step, promote=0, **kw)


def _muont_buffers(group: MatrixGroup, scratch: Scratch, work: Optional[torch.Tensor] = None):
    """Scratch of one matrix group's update.  `work` (count, out, in) replaces the shared FP32 work stack: several groups
    of one shape can then keep their stacks side by side and go through Newton-Schulz as one batch."""
    dev = group.device
    count, m, n = group.count, group.out_features, group.in_features
    shape = (count, m, n)
    if work is not None and (tuple(work.shape) != shape or work.dtype != torch.float32 or not work.is_contiguous()):
        raise ValueError("the work stack of a matrix group is a contiguous FP32 (count, out, in) tensor")
    return dict(work=work if work is not None else scratch.get("work", shape, torch.float32, dev),
                planes=scratch.get("planes", (2,) + shape, torch.float16, dev),
                inv=scratch.get("inv", (count,), torch.float32, dev),
                maxabs=scratch.get("maxabs", (count,), torch.int32, dev),
                c1=scratch.get("c1", (count,), torch.float32, dev),
                c2=scratch.get("c2", (count,), torch.float32, dev))


def muont_ns_input(group: MatrixGroup, grads: Sequence[torch.Tensor], scratch: Scratch, *, momentum: float,
                   nesterov: bool, work: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Stage 1 of the MuonT update: momentum, Nesterov direction and the inner preconditioning d R_in
    (src/toner/reference.py:197-204).  Returns the (count, out, in) stack the polar iteration starts from."""
    f = group.factors
    buf = _muont_buffers(group, scratch, work)
    work, planes, inv, maxabs = buf["work"], buf["planes"], buf["inv"], buf["maxabs"]
    ops.muont_momentum(group.grad_ptrs(grads), group.m, work, momentum, nesterov, maxabs)
    if f.inner_strength != 0:
        ops.split16(work, planes=planes, inv_scale=inv, maxabs=maxabs)
        _product(planes, inv, group, "inner", work)
    return work


def muont_delta_from_polar(group: MatrixGroup, polar: torch.Tensor, delta: torch.Tensor, scratch: Scratch, *, lr: float,
                           weight_decay: float, polar_maxabs: Optional[torch.Tensor] = None,
                           work: Optional[torch.Tensor] = None) -> None:
    """Stage 3: outer map, shape scale and shaped weight decay (src/toner/reference.py:206-215), fused as the
    reference's engine fuses them (src/toner/fast/engine.py:42-51):
    delta = -((lr wd n / ||R||^2) W R + (lr s sqrt(n) / ||R||) P) R.  `polar` may be the work stack itself."""
    f = group.factors
    count, m, n = group.count, group.out_features, group.in_features
    buf = _muont_buffers(group, scratch, work)
    work, planes, inv, maxabs, c1, c2 = (buf[k] for k in ("work", "planes", "inv", "maxabs", "c1", "c2"))
    if polar.data_ptr() != work.data_ptr():
        work.copy_(polar)
        polar_maxabs = None
    scale = max(1.0, m / n) ** 0.5
    if f.outer_strength == 0:
        raise ValueError("outer_strength 0 is not supported by the CUDA path")
    ops.muont_coeffs(f.fro2_outer, group.first, group.step, count, n, lr, weight_decay, scale, c1, c2)
    if weight_decay != 0:
        ops.split16_list(group.weight_ptrs, count, m, n, planes, inv, maxabs)
        ops.scale_vec(inv, c1)
        maxabs.zero_()
        # V = c1 W R + c2 P.  The decay term is lr wd ||W|| against lr ||P||, about 1 % of V: the hi planes suffice
        _product(planes, inv, group, "outer", work, coarse=True, c=work, beta=1.0, beta_v=c2, maxabs=maxabs)
        ops.split16(work, planes=planes, inv_scale=inv, maxabs=maxabs)
    else:
        if polar_maxabs is None:
            ops.split16(work, planes=planes, inv_scale=inv, scratch=maxabs)
        else:
            ops.split16(work, planes=planes, inv_scale=inv, maxabs=polar_maxabs)
        ops.scale_vec(inv, c2)  # V = c2 P
    _product(planes, inv, group, "outer", delta, alpha=-1.0)


def muont_group_delta(group: MatrixGroup, grads: Sequence[torch.Tensor], delta: torch.Tensor, scratch: Scratch, *,
                      lr: float, weight_decay: float, momentum: float, nesterov: bool, ns_steps: int,
                      ns_eps: float) -> None:
    """Write the MuonT parameter change of every matrix of the group into ``delta`` (count, out, in)."""
    dev = group.device
    count, m, n = group.count, group.out_features, group.in_features
    work = muont_ns_input(group, grads, scratch, momentum=momentum, nesterov=nesterov)
    maxabs = _muont_buffers(group, scratch)["maxabs"]
    ns_ws = scratch.bytes_like("ns", ops.ns_polar_workspace_bytes(count, m, n), dev)
    ops.ns_polar(work, ns_steps, ns_eps, out=work, maxabs=maxabs, workspace=ns_ws)
    muont_delta_from_polar(group, work, delta, scratch, lr=lr, weight_decay=weight_decay, polar_maxabs=maxabs)


def muont_groups_delta(groups: Sequence[MatrixGroup], grads: Sequence[Sequence[torch.Tensor]],
                       deltas: Sequence[torch.Tensor], scratch: Scratch, *, lr: float, weight_decay: float,
                       momentum: float, nesterov: bool, ns_steps: int, ns_eps: float) -> None:
    """muont_group_delta for several groups of ONE matrix shape (for instance the q, k, v and o projections of the owned
    layers): momentum and inner preconditioning per group, then ONE Newton-Schulz call over all their matrices, then the
    outer map per group.  The arithmetic per matrix is unchanged; the polar iteration's thirty products run on a batch
    several times larger, which matters when a rank owns few layers (three layers are 108 symmetric tiles on 74 SM
    pairs: a wave and a half)."""
    first = groups[0]
    count, m, n = first.count, first.out_features, first.in_features
    if any((g.count, g.out_features, g.in_features) != (count, m, n) for g in groups):
        raise ValueError("groups that share a Newton-Schulz batch need one matrix shape and one count")
    dev = first.device
    total = count * len(groups)
    merged = scratch.get("work_merged", (total, m, n), torch.float32, dev)
    maxabs = scratch.get("maxabs_merged", (total,), torch.int32, dev)
    slices = [merged[j * count:(j + 1) * count] for j in range(len(groups))]
    for g, gr, w in zip(groups, grads, slices):
        muont_ns_input(g, gr, scratch, momentum=momentum, nesterov=nesterov, work=w)
    ns_ws = scratch.bytes_like("ns", ops.ns_polar_workspace_bytes(total, m, n), dev)
    ops.ns_polar(merged, ns_steps, ns_eps, out=merged, maxabs=maxabs, workspace=ns_ws)
    for j, (g, w, d) in enumerate(zip(groups, slices, deltas)):
        muont_delta_from_polar(g, w, d, scratch, lr=lr, weight_decay=weight_decay,
                               polar_maxabs=maxabs[j * count:(j + 1) * count], work=w)


def adamt_group_delta(group: MatrixGroup, grads: Sequence[torch.Tensor], delta: torch.Tensor, scratch: Scratch, *,
                      lr: float, weight_decay: float, betas: Tuple[float, float], eps: float, t: int) -> None:
    """Write the AdamT parameter change of every matrix of the group into ``delta``."""
    f, dev = group.factors, group.device
    count, m, n = group.count, group.out_features, group.in_features
    shape = (count, m, n)
    b1, b2 = betas
    bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
    work = scratch.get("work", shape, torch.float32, dev)
    work2 = scratch.get("work2", shape, torch.float32, dev)
    planes = scratch.get("planes", (2,) + shape, torch.float16, dev)
    inv = scratch.get("inv", (count,), torch.float32, dev)
    maxabs = scratch.get("maxabs", (count,), torch.int32, dev)
    c1 = scratch.get("c1", (count,), torch.float32, dev)
    c2 = scratch.get("c2", (count,), torch.float32, dev)
    ss0 = scratch.get("ss0", (count,), torch.float32, dev)
    ss1 = scratch.get("ss1", (count,), torch.float32, dev)
    ssq_ws = scratch.bytes_like("sumsq", ops.sumsq_scratch_bytes(count), dev)
    gp = group.grad_ptrs(grads)
    ops.adamt_first_moment(gp, group.m, b1)
    ops.split16_list(gp, count, m, n, planes, inv, maxabs)
    _product(planes, inv, group, "inner", work)                       # t = g R
    ops.split16(group.m, planes=planes, inv_scale=inv, scratch=maxabs)
    _product(planes, inv, group, "inner", work2, alpha=1.0 / bc1)     # (m / bc1) R
    ops.adamt_ratio(work, group.v, work2, b2, bc2, eps, maxabs)       # U, in work2
    ops.sumsq(work2, out=ss0, scratch=ssq_ws)
    ops.split16(work2, planes=planes, inv_scale=inv, maxabs=maxabs)
    _product(planes, inv, group, "inner", work)                       # U R
    ops.sumsq(work, out=ss1, scratch=ssq_ws)
    ops.adamt_coeffs(f.fro2_outer, group.first, group.step, count, n, lr, weight_decay, ss0, ss1, c1, c2)
    if weight_decay != 0:
        ops.split16_list(group.weight_ptrs, count, m, n, planes, inv, maxabs)
        ops.scale_vec(inv, c1)
        maxabs.zero_()
        _product(planes, inv, group, "outer", work2, coarse=True, maxabs=maxabs)   # c1 W R (small term: hi planes)
        ops.split16(work2, planes=planes, inv_scale=inv, maxabs=maxabs)
        _product(planes, inv, group, "outer", delta, alpha=-1.0, c=work, beta=1.0, beta_v=c2)
    else:
        ops.scale_stack(work, c2, delta)                              # delta = c2 * U R


def apply_group_delta(group: MatrixGroup, delta: torch.Tensor) -> None:
    ops.apply_delta(group.weight_ptrs, delta)
