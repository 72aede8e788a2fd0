"""MuonT and AdamT with the reference's general-path interface, running on the sm_100a library.

Same constructor arguments, defaults, state keys and error behaviour as the reference's readable
optimizers (src/toner/reference.py:29-315), but every parameter with a gradient is updated by the
CUDA kernels: statistic EMA, Newton inverse-root factors instead of an eigendecomposition per
parameter, Newton-Schulz in "tpu" arithmetic, split-precision preconditioning products.  Parameters
of equal shape inside a parameter group are stacked so that each kernel launch covers all of them.

Differences from the reference, all raised as errors rather than silently emulated:
  * parameters must live on a CUDA device (there is no CPU path here);
  * matrix dimensions must be multiples of 8;
  * strengths must be 0 or 1/p with p a power of two (Newton inverse p-th roots);
  * ``ns_mode`` is "tpu" (the other modes are different numerical configurations).
"""

from __future__ import annotations

import math
from collections.abc import Iterable, Mapping
from typing import Callable, Dict, List, Optional, Tuple

import torch
from torch import Tensor
from torch.optim import Optimizer

from . import core, ops


# Hyper-parameter ranges: name -> (smallest allowed value, exclusive upper limit or None).  The limits and the
# exception types are those of the reference's general optimizers (src/toner/reference.py:17-36,153-166,266-273);
# the checks themselves are table-driven here.
_RANGES = {
    "lr": (0.0, None), "weight_decay": (0.0, None), "statistic_momentum": (0.0, 1.0), "damping": (1e-30, None),
    "inner_strength": (0.0, None), "outer_strength": (0.0, None), "strength": (0.0, None), "momentum": (0.0, 1.0),
    "ns_eps": (1e-30, None), "eps": (1e-30, None), "beta": (0.0, 1.0),
}


def _in_range(name: str, value, key: Optional[str] = None) -> None:
    """ValueError unless `value` is a real, finite number inside the range registered under `key` (default: name)."""
    low, high = _RANGES[key or name]
    real = isinstance(value, (int, float)) and not isinstance(value, complex)
    if real and math.isfinite(value) and value >= low and (high is None or value < high):
        return
    span = f"[{low}, {high})" if high is not None else f"[{low}, inf)"
    raise ValueError(f"{name} = {value!r} is outside {span}")


def _check_matrix(p: Tensor) -> None:
    """What the CUDA path needs of a weight: a non-empty FP32 matrix on a CUDA device, dimensions multiples of 8."""
    if p.ndim != 2 or p.numel() == 0:
        raise ValueError("Toner expects nonempty 2-D matrix weights; optimize other parameters separately")
    if p.dtype != torch.float32:
        raise ValueError("Toner keeps FP32 master weights; use FP32 parameters")
    if p.device.type != "cuda":
        raise ValueError("toner_b200 runs on CUDA (sm_100a) only; move the parameters to the GPU")
    if p.shape[0] % 8 or p.shape[1] % 8:
        raise ValueError("toner_b200 needs matrix dimensions that are multiples of 8")


class _Bucket:
    """Equally shaped parameters of one parameter group: one FactorSet entry and one stack row each."""

    def __init__(self, params: List[Tensor], strengths: Tuple[float, float], damping: float, kind: str,
                 scratch: core.Scratch) -> None:
        self.params = params
        n = params[0].shape[1]
        self.factors = core.FactorSet(len(params), n, params[0].device, strengths, damping, scratch)
        self.group = core.MatrixGroup(params, self.factors, 0, 1, kind)
        self.delta = torch.empty_like(self.group.m)
        self.index = {p: i for i, p in enumerate(params)}

    def stacks(self) -> Dict[str, Tensor]:
        """Per-parameter state keys of the reference (src/toner/reference.py:76-81,198-199,297-300) and the stacked
        storage row i of which holds parameter i's value."""
        out = {"input_ema": self.factors.ema}
        if self.group.kind == "muont":
            out["momentum_buffer"] = self.group.m
        else:
            out["exp_avg"], out["exp_avg_sq"] = self.group.m, self.group.v
        return out


class _TonerGeneral(Optimizer):
    """Statistic EMA, validation and bookkeeping common to MuonT and AdamT."""

    _kind = ""
    _group_ranges: Tuple[str, ...] = ("lr", "weight_decay", "statistic_momentum", "damping")

    def __init__(self, params, defaults) -> None:
        super().__init__(params, defaults)
        self._scratch = core.Scratch()
        self._buckets: Optional[Dict[Tuple, _Bucket]] = None
        self._bucket_of: Dict[Tensor, Tuple[_Bucket, int]] = {}
        self._health: Optional[ops.Health] = None   # the update kernels of the last step (created with the buckets)

    # ------------------------------------------------------------------ validation
    def _validate_common(self) -> None:
        for group in self.param_groups:
            for name in self._group_ranges:
                _in_range(name, group[name])
            for p in group["params"]:
                _check_matrix(p)

    def _strengths(self, group) -> Tuple[float, float]:
        raise NotImplementedError

    def add_param_group(self, param_group) -> None:
        super().add_param_group(param_group)
        self._buckets = None  # rebuilt lazily; optimizer state is kept in self.state

    def _build(self) -> None:
        """Stack equally shaped parameters of each group (first use, after add_param_group or load_state_dict)."""
        old = self._bucket_of
        self._buckets, self._bucket_of = {}, {}
        if self._health is None:
            self._health = ops.Health()
        for gi, group in enumerate(self.param_groups):
            by_shape: Dict[Tuple[int, int], List[Tensor]] = {}
            for p in group["params"]:
                if not p.is_contiguous():
                    raise ValueError("toner_b200 needs contiguous weights")
                by_shape.setdefault(tuple(p.shape), []).append(p)
            for shape, ps in by_shape.items():
                core.root_orders(*self._strengths(group))
                bucket = _Bucket(ps, self._strengths(group), group["damping"], self._kind, self._scratch)
                self._buckets[(gi, shape)] = bucket
                for i, p in enumerate(ps):
                    self._bucket_of[p] = (bucket, i)
                    if p in old:  # carry values over when the grouping is rebuilt
                        ob, oi = old[p]
                        for key, stack in bucket.stacks().items():
                            stack[i].copy_(ob.stacks()[key][oi])
                    self._adopt(p, bucket, i)

    def _adopt(self, p: Tensor, bucket: _Bucket, i: int) -> None:
        """Make the reference's per-parameter state keys views of the stacked storage.  A tensor that is already in
        the state but lives elsewhere -- loaded from a checkpoint -- is copied into its row first, so its value is
        the one the kernels read."""
        state = self.state[p]
        for key, stack in bucket.stacks().items():
            if key not in state:
                continue
            held, row = state[key], stack[i]
            if held.data_ptr() != row.data_ptr():
                row.copy_(held.to(device=row.device, dtype=row.dtype))
                if key == "input_ema":
                    bucket.factors.statistics_replaced()
            state[key] = row

    def load_state_dict(self, state_dict) -> None:
        """torch's loader puts fresh tensors into ``self.state``; the stacks the kernels read are rebuilt from them
        at the next use (the factors are recomputed, so the first step after a resume runs the Newton schedule of
        the bound that always holds)."""
        super().load_state_dict(state_dict)
        self._buckets, self._bucket_of = None, {}

    def _ensure_built(self) -> None:
        if self._buckets is None:
            self._validate_common()
            self._build()

    # ------------------------------------------------------------------ statistics
    @torch.no_grad()
    def update_statistics(self, second_moments: Mapping[Tensor, Tensor]) -> None:
        """Update each parameter's input EMA once from this step's mean Gram ``sum(x.T @ x) / rows``.

        The whole mapping is validated before any state changes; calling twice without ``step()`` is an
        error (src/toner/reference.py:51-81)."""
        self._ensure_built()
        owner = {p: g for g in self.param_groups for p in g["params"]}
        finite = {}
        for p, cov in second_moments.items():   # nothing is touched until every entry has passed
            if p not in owner:
                raise ValueError("Received a statistic for a parameter not owned by this optimizer")
            if tuple(cov.shape) != (p.shape[1], p.shape[1]):
                raise ValueError("Statistic shape must match the matrix weight's input dimension")
            if cov.device != p.device:
                raise ValueError("Input statistics and matrix weights must be on the same device")
            if not cov.is_floating_point():
                raise ValueError("Input statistics must be finite floating-point matrices")
            if self.state[p].get("statistics_ready", False):
                raise RuntimeError("Statistics already updated; aggregate microbatches before update_statistics()")
            finite.setdefault(cov.data_ptr(), torch.isfinite(cov).all())     # one flag per distinct statistic
        if finite and not bool(torch.stack(list(finite.values())).all()):    # one wait for all of them
            raise ValueError("Input statistics must be finite floating-point matrices")
        for p, cov in second_moments.items():
            bucket, i = self._bucket_of[p]
            state, beta = self.state[p], owner[p]["statistic_momentum"]
            if "input_ema" not in state:
                bucket.factors.ema[i].zero_()
                state["input_ema"] = bucket.factors.ema[i]
                state["input_weight"] = 0.0
            c = cov.to(torch.float32).contiguous()
            ops.axpby(state["input_ema"], c, state["input_ema"], beta, 1 - beta)
            state["input_weight"] = beta * state["input_weight"] + (1 - beta)
            state["statistics_ready"] = True

    def _check_step(self) -> None:
        self._validate_common()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("Toner does not support sparse gradients")
                if not self.state[p].get("statistics_ready", False):
                    raise RuntimeError("Call update_statistics() with this step's input second moments before step()")

    def _consume_statistics(self) -> None:
        for group in self.param_groups:
            for p in group["params"]:
                self.state[p]["statistics_ready"] = False

    def _active_buckets(self):
        """(group, bucket) pairs with work to do.  A bucket steps only as a whole: parameters of one
        shape inside one group either all have gradients or none (mixed cases are stepped one by one)."""
        for (gi, _), bucket in self._buckets.items():
            group = self.param_groups[gi]
            with_grad = [p for p in bucket.params if p.grad is not None]
            if not with_grad:
                continue
            if len(with_grad) != len(bucket.params):
                raise RuntimeError("toner_b200 stacks equally shaped parameters of a group: give all of them "
                                   "gradients, or put the ones without into a separate parameter group")
            yield group, bucket

    def _factor_all(self, work) -> None:
        """Factors of every active bucket: enqueue all, then wait for their flags (and for the status of the previous
        step's update kernels, which finished before them)."""
        for _, bucket in work:
            bucket.factors.compute()
        for _, bucket in work:
            bucket.factors.finish()
        self._health.check()

    @property
    def fallbacks(self) -> int:
        """Statistics whose Newton factors were flagged and recomputed by eigendecomposition so far."""
        return sum(b.factors.fallbacks for b in (self._buckets or {}).values())


class MuonT(_TonerGeneral):
    """Muon with input preconditioning and shaped weight decay (src/toner/reference.py:102-217).

    ``lr`` is the matrix learning rate; defaults use the half / eighth geometry.  ``statistic_momentum=None``
    inherits each group's ``momentum``."""

    _kind = "muont"

    def __init__(self, params: Iterable[Tensor] | Iterable[dict], *, lr: float, weight_decay: float = 0.0,
                 inner_strength: float = 0.5, outer_strength: float = 0.125,
                 statistic_momentum: Optional[float] = None, damping: float = 1e-3, momentum: float = 0.95,
                 nesterov: bool = True, ns_steps: int = 10, ns_eps: float = 1e-5, ns_mode: str = "tpu") -> None:
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, inner_strength=inner_strength,
                                      outer_strength=outer_strength, statistic_momentum=statistic_momentum,
                                      damping=damping, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      ns_eps=ns_eps, ns_mode=ns_mode))
        self._validate_common()
        self._validate_muon()

    def add_param_group(self, param_group) -> None:
        super().add_param_group(param_group)
        group = self.param_groups[-1]
        if group["statistic_momentum"] is None:
            group["statistic_momentum"] = group["momentum"]

    def _strengths(self, group) -> Tuple[float, float]:
        return float(group["inner_strength"]), float(group["outer_strength"])

    def _validate_muon(self) -> None:
        for group in self.param_groups:
            for name in ("inner_strength", "outer_strength", "momentum", "ns_eps"):
                _in_range(name, group[name])
            core.root_orders(*self._strengths(group))
            if group["outer_strength"] == 0:
                raise ValueError("outer_strength 0 is not supported by the CUDA path")
            if group["ns_mode"] not in {"tpu", "f32", "bf16"}:
                raise ValueError("ns_mode must be 'tpu', 'f32', or 'bf16'")
            if group["ns_mode"] != "tpu":
                raise ValueError("toner_b200 implements ns_mode='tpu' (BF16 operands, FP32 accumulation) only")
            if not isinstance(group["ns_steps"], int) or isinstance(group["ns_steps"], bool) or group["ns_steps"] < 1:
                raise ValueError("ns_steps must be a positive integer")

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._ensure_built()
        self._check_step()
        self._validate_muon()
        work = list(self._active_buckets())
        self._factor_all(work)
        for group, bucket in work:
            grads = [p.grad for p in bucket.params]
            core.muont_group_delta(bucket.group, grads, bucket.delta, self._scratch, lr=group["lr"],
                                   weight_decay=group["weight_decay"], momentum=group["momentum"],
                                   nesterov=group["nesterov"], ns_steps=group["ns_steps"], ns_eps=group["ns_eps"])
            core.apply_group_delta(bucket.group, bucket.delta)
            for i, p in enumerate(bucket.params):
                self.state[p]["momentum_buffer"] = bucket.group.m[i]
        if work:
            self._health.arm("the previous step's update")
        self._consume_statistics()
        return loss


class AdamT(_TonerGeneral):
    """Matched-strength AdamT with an unnormalised second-moment factor (src/toner/reference.py:220-315).

    ``statistic_momentum=None`` inherits each group's ``betas[1]``."""

    _kind = "adamt"

    def __init__(self, params: Iterable[Tensor] | Iterable[dict], *, lr: float, weight_decay: float = 0.0,
                 strength: float = 0.25, statistic_momentum: Optional[float] = None, damping: float = 1e-3,
                 betas: Tuple[float, float] = (0.9, 0.98), eps: float = 1e-20) -> None:
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, strength=strength,
                                      statistic_momentum=statistic_momentum, damping=damping, betas=betas, eps=eps))
        self._validate_common()
        self._validate_adam()

    def add_param_group(self, param_group) -> None:
        super().add_param_group(param_group)
        group = self.param_groups[-1]
        if group["statistic_momentum"] is None:
            if len(group["betas"]) != 2:
                raise ValueError("betas must contain two coefficients")
            group["statistic_momentum"] = group["betas"][1]

    def _strengths(self, group) -> Tuple[float, float]:
        return float(group["strength"]), float(group["strength"])

    def _validate_adam(self) -> None:
        for group in self.param_groups:
            _in_range("strength", group["strength"])
            core.root_orders(*self._strengths(group))
            if group["strength"] == 0:
                raise ValueError("strength 0 is not supported by the CUDA path")
            _in_range("eps", group["eps"])
            if len(group["betas"]) != 2:
                raise ValueError("betas must contain two coefficients")
            for j, beta in enumerate(group["betas"]):
                _in_range(f"betas[{j}]", beta, key="beta")

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._ensure_built()
        self._check_step()
        self._validate_adam()
        work = list(self._active_buckets())
        self._factor_all(work)
        for group, bucket in work:
            steps = {self.state[p].get("step", 0) for p in bucket.params}
            if len(steps) != 1:
                raise RuntimeError("parameters stacked together must have taken the same number of steps")
            t = steps.pop() + 1
            grads = [p.grad for p in bucket.params]
            core.adamt_group_delta(bucket.group, grads, bucket.delta, self._scratch, lr=group["lr"],
                                   weight_decay=group["weight_decay"], betas=tuple(group["betas"]), eps=group["eps"], t=t)
            core.apply_group_delta(bucket.group, bucket.delta)
            for i, p in enumerate(bucket.params):
                st = self.state[p]
                st["step"] = t
                st["exp_avg"], st["exp_avg_sq"] = bucket.group.m[i], bucket.group.v[i]
        if work:
            self._health.arm("the previous step's update")
        self._consume_statistics()
        return loss
