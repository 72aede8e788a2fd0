"""FastMuonT / FastAdamT for uniform Llama-style and modded-nanoGPT blocks on the sm_100a engine.

Constructor arguments, defaults, lifecycle (``capture_microbatch`` -> ``begin`` -> ``step``), error
behaviour, parameter naming and checkpoint format follow the reference's adapter
(src/toner/fast/adapter.py:16-592).  Root-engine knobs that only make sense for the reference's
cached-eigenbasis iteration (``root_refresh``, ``root_inline_steps``, ``root_repair_rounds``,
``root_graphs``, ``host_workers``, ``host_threads``) are accepted and recorded but have no effect:
factors here are recomputed from scratch every step by the Newton engine, whose iteration count is
fixed by (width, damping, power) -- see ``toner_b200.ops.inv_roots_iterations``.
"""

from __future__ import annotations

import math
import weakref
from contextlib import contextmanager
from dataclasses import dataclass
from types import SimpleNamespace

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..statistics import sample_positions


@dataclass(frozen=True)
class ProjectionBlock:
    """The seven bias-free projections of one Llama-style block; q/k/v share an input, as do gate/up."""

    q: nn.Linear
    k: nn.Linear
    v: nn.Linear
    o: nn.Linear
    gate: nn.Linear
    up: nn.Linear
    down: nn.Linear

    @classmethod
    def from_module(cls, block: nn.Module) -> "ProjectionBlock":
        return cls(**{name: getattr(block, name) for name in cls.__dataclass_fields__})


@dataclass(frozen=True)
class NanoGPTBlock:
    """The six projections of a modded-nanoGPT block; q/k/v share an input.  Biases are left to the caller."""

    q: nn.Linear
    k: nn.Linear
    v: nn.Linear
    attn_proj: nn.Linear
    fc: nn.Linear
    mlp_proj: nn.Linear

    @classmethod
    def from_module(cls, block: nn.Module) -> "NanoGPTBlock":
        a, m = block.attn, block.mlp
        return cls(a.q, a.k, a.v, a.proj, m.fc, m.proj)


_LIVE = weakref.WeakSet()
_ROLES = {"llama": ("q", "k", "v", "o", "gate", "up", "down"),
          "nanogpt": ("q", "k", "v", "attn_proj", "fc", "mlp_proj")}
_STAT_OF_ROLE = {"q": "attn", "k": "attn", "v": "attn", "o": "o", "gate": "mlp", "up": "mlp", "down": "down",
                 "attn_proj": "o", "fc": "mlp", "mlp_proj": "down"}
_NANOGPT_PATH = {"q": "attn.q", "k": "attn.k", "v": "attn.v", "attn_proj": "attn.proj", "fc": "mlp.fc",
                 "mlp_proj": "mlp.proj"}


def _as_block(block):
    if isinstance(block, (ProjectionBlock, NanoGPTBlock)):
        return block
    if hasattr(block, "attn") and hasattr(block, "mlp"):
        return NanoGPTBlock.from_module(block)
    return ProjectionBlock.from_module(block)


def _positive_int(name, value):
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{name} must be a positive integer")


def _check_hyperparameters(kind, lr, weight_decay, momentum, betas, eps, ns_eps, statistic_momentum, statistic_head,
                           sequence_length, strengths, counts, nonnegative_counts):
    """Argument checks shared by both optimizers; every violation is a ValueError."""
    for label, value in counts.items():
        _positive_int(label, value)
    for label, value in nonnegative_counts.items():
        if isinstance(value, bool) or not isinstance(value, int) or value < 0:
            raise ValueError(f"{label} must be a nonnegative integer")
    if isinstance(statistic_head, bool) or not isinstance(statistic_head, int) or not 0 <= statistic_head <= sequence_length:
        raise ValueError("statistic_head must lie in [0, sequence_length]")
    for label, value in (("lr", lr), ("weight_decay", weight_decay)):
        if not (math.isfinite(value) and value >= 0):
            raise ValueError(f"{label} must be a finite nonnegative number")
    for label, value in (("eps", eps), ("ns_eps", ns_eps)):
        if not (math.isfinite(value) and value > 0):
            raise ValueError(f"{label} must be a finite positive number")
    for label, value in (("statistic_momentum", statistic_momentum), ("momentum", momentum)):
        if not 0 <= value < 1:
            raise ValueError(f"{label} must lie in [0, 1)")
    if len(betas) != 2 or any(not 0 <= b < 1 for b in betas):
        raise ValueError("betas must be two numbers in [0, 1)")
    if any(s not in (0.125, 0.25, 0.5) for s in strengths):
        raise ValueError("inner_strength and outer_strength must each be 1/8, 1/4 or 1/2")
    if kind == "adamt" and strengths != (0.25, 0.25):
        raise ValueError("FastAdamT uses the matched quarter-power factors (1/4, 1/4)")


def _expected_shapes(layout, hidden, mlp):
    square = (hidden, hidden)
    if layout == "nanogpt":
        return dict(q=square, k=square, v=square, attn_proj=square, fc=(mlp, hidden), mlp_proj=(hidden, mlp))
    return dict(q=square, k=square, v=square, o=square, gate=(mlp, hidden), up=(mlp, hidden), down=(hidden, mlp))


class _FastToner(torch.optim.Optimizer):
    """Shared adapter; use FastMuonT or FastAdamT.  ``state_dict`` / ``load_state_dict`` are collective."""

    def __init__(self, blocks, lr, *, kind, micro_batch_size, sequence_length, accumulation_steps=1,
                 weight_decay=0.0, momentum=0.95, nesterov=True, betas=(0.8, 0.98), eps=1e-15,
                 inner_strength=0.5, outer_strength=0.125, statistic_momentum=0.938, statistic_head=32,
                 statistic_stride=16, ns_steps=10, ns_eps=1e-5, root_refresh=4, root_iterations=2,
                 root_inline_steps=20, root_repair_rounds=3, root_graphs=True, host_workers=2, host_threads=4,
                 statistic_chunks=4, row_pieces=1, owner_weights=None, check_every=0):
        if len(_LIVE):
            raise RuntimeError("another fast Toner optimizer is alive in this process; close() it first")
        strengths = (float(inner_strength), float(outer_strength))
        _check_hyperparameters(
            kind, lr, weight_decay, momentum, betas, eps, ns_eps, statistic_momentum, statistic_head, sequence_length,
            strengths,
            counts=dict(micro_batch_size=micro_batch_size, sequence_length=sequence_length,
                        accumulation_steps=accumulation_steps, statistic_stride=statistic_stride, ns_steps=ns_steps,
                        root_refresh=root_refresh, root_iterations=root_iterations, host_workers=host_workers,
                        host_threads=host_threads, statistic_chunks=statistic_chunks, row_pieces=row_pieces),
            nonnegative_counts=dict(root_inline_steps=root_inline_steps, root_repair_rounds=root_repair_rounds))
        self.blocks = [_as_block(b) for b in blocks]
        if len(self.blocks) == 0:
            raise ValueError("no projection blocks given")
        first = self.blocks[0]
        if any(type(b) is not type(first) for b in self.blocks):
            raise ValueError("all blocks of one fast optimizer must use the same projection layout")
        self._layout = "nanogpt" if isinstance(first, NanoGPTBlock) else "llama"
        self._roles = _ROLES[self._layout]
        self.micro_batch_size = micro_batch_size
        self.sequence_length = sequence_length
        self.accumulation_steps = accumulation_steps
        positions = sample_positions(sequence_length, statistic_head, statistic_stride)
        if len(positions) == 0:
            raise ValueError("statistic_head / statistic_stride keep no token position")
        for role in self._roles:
            if not isinstance(getattr(first, role), nn.Linear):
                raise TypeError(f"block member '{role}' must be an nn.Linear")
        hidden = first.q.in_features
        mlp = (first.fc if self._layout == "nanogpt" else first.gate).out_features
        if hidden % 256 != 0 or mlp % 256 != 0:
            raise ValueError("hidden and MLP widths must be multiples of 256")
        shapes = _expected_shapes(self._layout, hidden, mlp)
        device = first.q.weight.device
        if device.type != "cuda":
            raise ValueError("fast Toner needs CUDA parameters; toner_b200 has no CPU path")
        if torch.cuda.get_device_capability(device)[0] != 10:
            raise ValueError("toner_b200 kernels are built for sm_100a (B200) only")
        named, bindings, modules = {}, {}, []
        taken = set()
        for index, block in enumerate(self.blocks):
            for role in self._roles:
                module = getattr(block, role)
                if not isinstance(module, nn.Linear) or tuple(module.weight.shape) != shapes[role]:
                    raise ValueError(f"block {index}: '{role}' must be an nn.Linear with weight shape {shapes[role]}")
                if module.bias is not None and self._layout == "llama":
                    raise ValueError(f"block {index}: ProjectionBlock projections are bias-free; NanoGPTBlock allows biases")
                weight = module.weight
                usable = (weight.device == device and weight.dtype == torch.float32 and weight.requires_grad
                          and weight.is_contiguous())
                if not usable:
                    raise ValueError(f"block {index}: '{role}' weight must be a contiguous trainable FP32 tensor on {device}")
                if id(weight) in taken:
                    raise ValueError(f"block {index}: '{role}' shares its weight with another projection")
                taken.add(id(weight))
                if self._layout == "nanogpt":
                    name = f"blocks.{index}.{_NANOGPT_PATH[role]}.weight"
                else:
                    name = f"body.blocks.{index}.{role}.weight"
                named[name] = weight
                bindings[name] = (index, role, _STAT_OF_ROLE[role])
                modules.append((index, role, module))
        in_group = dist.is_initialized()
        world = dist.get_world_size() if in_group else 1
        rank = dist.get_rank() if in_group else 0
        if world > 1 and dist.get_backend() != "nccl":
            raise ValueError("more than one rank needs the NCCL backend (and replicated, synchronised gradients)")
        # Optional (the reference's engine has both, its adapter does not pass them: --toner-owner-weights and
        # toner_check_every, src/toner/fast/engine.py:215-219,743-770): layers per rank in proportion to `owner_weights`
        # instead of equal blocks, and a cross-check of the factors against an eigendecomposition every `check_every` steps.
        if owner_weights is not None:
            owner_weights = [float(x) for x in owner_weights]
            if len(owner_weights) != world or min(owner_weights) < 0 or sum(owner_weights) <= 0:
                raise ValueError("owner_weights needs one non-negative weight per rank, not all zero")
        elif len(self.blocks) % world != 0:
            raise ValueError("the number of blocks must be a multiple of the number of ranks (or give owner_weights)")
        if isinstance(check_every, bool) or not isinstance(check_every, int) or check_every < 0:
            raise ValueError("check_every must be a nonnegative integer")
        super().__init__(list(named.values()), {"lr": float(lr), "weight_decay": float(weight_decay)})
        self._closed = self._capturing = False
        self._microbatches = 0
        self._seen = set()
        self._input_signatures = {}
        self._hooks = []
        self._device = device
        self._positions = torch.tensor(positions, device=device, dtype=torch.int32)
        self._positions64 = self._positions.to(torch.int64)
        self._row_targets = {}
        self._pending = []
        self._rows_per_microbatch = micro_batch_size * len(positions)
        local_rows = self._rows_per_microbatch * accumulation_steps
        # Optional (not in the reference's adapter; its engine has it as chunk_stats / chunk_wait): the row buffers hold
        # only accumulation_steps / row_pieces microbatches, and each full piece is folded into the partial Grams.
        if accumulation_steps % row_pieces:
            raise ValueError("row_pieces must divide accumulation_steps")
        self._piece_microbatches = accumulation_steps // row_pieces
        args = SimpleNamespace(
            statistic_momentum=float(statistic_momentum), inner_strength=strengths[0], outer_strength=strengths[1],
            damping=1e-3, weight_decay=float(weight_decay), beta1=float(betas[0]), beta2=float(betas[1]),
            eps=float(eps), momentum=float(momentum), nesterov=bool(nesterov), ns_steps=ns_steps,
            ns_eps=float(ns_eps), stat_chunks=int(statistic_chunks), owner_weights=owner_weights,
            check_every=int(check_every))
        # the checkpoint's "config" block: same keys as the reference writes (src/toner/fast/adapter.py:321-340)
        self._config = dict(
            layout=self._layout, kind=kind, inner_strength=strengths[0], outer_strength=strengths[1],
            statistic_momentum=statistic_momentum, momentum=momentum, nesterov=bool(nesterov), betas=tuple(betas),
            eps=eps, ns_steps=ns_steps, ns_eps=ns_eps, statistic_head=statistic_head,
            statistic_stride=statistic_stride, root_refresh=root_refresh, root_iterations=root_iterations,
            root_inline_steps=root_inline_steps, root_repair_rounds=root_repair_rounds, root_graphs=bool(root_graphs))
        from .engine import KINDS_D, FastTonerCore  # CUDA library is loaded here, not at package import

        self._core = FastTonerCore(named, bindings, kind, layers=len(self.blocks), hid=hidden, mlp=mlp,
                                   local_rows=local_rows, args=args, world=world, rank=rank, device=device,
                                   row_capacity=self._rows_per_microbatch * self._piece_microbatches)
        # per-layer views of the stacked row buffers, under the reference's attribute names
        self._buffers = []
        d, f = self._core.groups["d"], self._core.groups["f"]
        for i in range(len(self.blocks)):
            views = {f"input_rows_{k}": d.rows_buf[len(KINDS_D) * i + j] for j, k in enumerate(KINDS_D)}
            views["input_rows_down"] = f.rows_buf[i]
            self._buffers.append(SimpleNamespace(**views))
        self.param_groups = self._core.param_groups
        self.param_groups[0]["lr"] = float(lr)
        for i, role, module in modules:
            self._hooks.append(module.register_forward_pre_hook(self._make_hook(i, role)))
        _LIVE.add(self)

    # ------------------------------------------------------------------ lifecycle
    def _assert_open(self):
        if self._closed:
            raise RuntimeError("This fast Toner optimizer has been closed")
        if torch.cuda.current_stream(self._device) != self._core.main_stream:
            raise RuntimeError("Use fast Toner on the CUDA stream on which it was constructed")

    def _make_hook(self, layer, role):
        def hook(module, inputs):
            if not self._capturing:
                return
            if (layer, role) in self._seen:
                raise RuntimeError(f"block {layer}: '{role}' ran twice inside one captured microbatch")
            x = inputs[0] if inputs else None
            if not isinstance(x, torch.Tensor):
                raise TypeError(f"block {layer}: '{role}' was called without a tensor input")
            x = x.detach()
            expected = (self.micro_batch_size, self.sequence_length, module.in_features)
            if tuple(x.shape) != expected:
                raise ValueError(f"block {layer}: '{role}' input has shape {tuple(x.shape)}, configured {expected}")
            under_autocast = torch.is_autocast_enabled("cuda")
            if under_autocast:
                if torch.get_autocast_dtype("cuda") != torch.bfloat16:
                    raise ValueError("autocast must use BF16 (FP16 autocast is not supported)")
            elif x.dtype != torch.bfloat16:
                raise ValueError("projection inputs must be BF16 tensors, or the forward must run under BF16 autocast")
            stat = _STAT_OF_ROLE[role]
            signature = (x.data_ptr(), tuple(x.shape), tuple(x.stride()))
            previous = self._input_signatures.get((layer, stat))
            if previous not in (None, signature):
                raise ValueError(f"block {layer}: projections sharing the '{stat}' statistic (q/k/v, gate/up) must "
                                 "read one and the same input tensor")
            self._seen.add((layer, role))
            if previous is None:
                self._input_signatures[(layer, stat)] = signature
                if x.dtype not in (torch.bfloat16, torch.float32):
                    x = x.float()
                if x.stride(2) != 1 or (x.stride(1) * x.element_size()) % 16 or (x.stride(0) * x.element_size()) % 16 \
                        or x.data_ptr() % 16:
                    x = x.contiguous()
                # The sampled rows of every statistic are written by ONE launch when the forward has finished
                # (_flush_capture): until then the input is kept alive here, as autograd keeps it for backward.
                self._pending.append((x, getattr(self._buffers[layer], f"input_rows_{stat}")))

        return hook

    @contextmanager
    def capture_microbatch(self):
        """Capture one forward pass; call exactly ``accumulation_steps`` times between updates."""
        self._assert_open()
        if self._capturing:
            raise RuntimeError("capture_microbatch() is already active")
        if self._core.begun or self._microbatches >= self.accumulation_steps:
            raise RuntimeError("all microbatches of this step are captured; call step() before the next forward")
        self._seen = set()
        self._input_signatures = {}
        self._pending = []
        if self._microbatches and self._microbatches % self._piece_microbatches == 0:
            self._core.chunk_wait()               # the previous piece's Grams must have read the row buffers
        self._capturing = True
        complete = False
        try:
            yield
            ran, wanted = len(self._seen), len(self.blocks) * len(self._roles)
            if ran != wanted:
                raise RuntimeError(f"the captured forward ran {ran} of the {wanted} configured projections")
            self._flush_capture()
            complete = True
        finally:
            self._capturing = False
            self._pending = []
            # a failed or partial forward discards every microbatch captured so far in this step
            self._microbatches = self._microbatches + 1 if complete else 0
            if not complete:
                self._core.discard_pieces()
            elif self._microbatches % self._piece_microbatches == 0 and self._microbatches < self.accumulation_steps:
                self._core.chunk_stats()          # a full piece that is not the step's last

    def _flush_capture(self):
        """The sampled rows of this micro-batch, for every layer and statistic, in one launch (toner_capture):
        row (b, p) of an input goes to row  slot * rows_per_microbatch + b * P + p  of the statistic's buffer."""
        from .. import capture
        slot = self._microbatches % self._piece_microbatches
        at = self._row_targets.get(slot)
        if at is None:
            lo = slot * self._rows_per_microbatch
            at = self._row_targets[slot] = torch.arange(lo, lo + self._rows_per_microbatch, device=self._device,
                                                        dtype=torch.int64)
        capture.capture_rows([x for x, _ in self._pending], [b for _, b in self._pending], at, self._positions64)

    def begin(self):
        """Start statistics and factors asynchronously after the final forward, before backward."""
        self._assert_open()
        if self._core.begun:
            raise RuntimeError("begin() was already called for this step")
        if self._capturing or self._microbatches != self.accumulation_steps:
            raise RuntimeError(f"begin() needs all {self.accumulation_steps} microbatches captured "
                               f"({self._microbatches} so far)")
        self._core.begin()

    @torch.no_grad()
    def step(self, closure=None):
        self._assert_open()
        if closure is not None:
            raise ValueError("step() takes no closure: capture the forward passes explicitly")
        if self._capturing or self._microbatches != self.accumulation_steps:
            raise RuntimeError(f"step() needs all {self.accumulation_steps} microbatches captured "
                               f"({self._microbatches} so far)")
        for p in self.param_groups[0]["params"]:
            if p.grad is None or p.grad.is_sparse:
                raise RuntimeError("every projection weight needs a dense gradient (already synchronised across ranks)")
        try:
            self._core.step()
        finally:
            self._microbatches = 0   # the captured rows were consumed by begin(), whether or not the step went through

    # ------------------------------------------------------------------ checkpoints
    def state_dict(self):
        """Collective on all ranks; the full checkpoint is returned on rank zero only (None elsewhere).

        Format "toner.fast.v3" (src/toner/fast/adapter.py:460-478): {"format", "config", "core": {"ema":
        {"<layer>.<kind>": (n, n)}, "weight", "moments": {name: {"m"[, "v"]}}, "t"}, "lr", "weight_decay"}."""
        self._assert_open()
        mid_step = self._capturing or self._microbatches or self._core.begun
        if mid_step or self._core.t == 0:
            raise RuntimeError("state_dict() is valid only between completed steps (and after the first one)")
        core_state = self._core.full_state()
        if core_state is None:
            return None
        group = self.param_groups[0]
        return {"format": "toner.fast.v3", "config": dict(self._config), "core": core_state, "lr": group["lr"],
                "weight_decay": group["weight_decay"]}

    def _validate_checkpoint(self, ckpt):
        if not isinstance(ckpt, dict) or ckpt.get("format") not in ("toner.fast.v2", "toner.fast.v3"):
            raise ValueError("not a toner.fast.v3 checkpoint (every rank must receive the same one)")
        config = dict(ckpt.get("config", {}))
        if ckpt["format"] == "toner.fast.v2":  # v2 predates the layout field and was Llama-only
            if self._layout != "llama" or config.get("layout", "llama") != "llama":
                raise ValueError("toner.fast.v2 checkpoints exist for the Llama layout only")
            config.setdefault("layout", "llama")
        if config != self._config:
            raise ValueError("checkpoint settings or layout differ from this optimizer's")
        state = ckpt["core"]
        if not isinstance(state.get("t"), int) or state["t"] < 1:
            raise ValueError("checkpoint holds no completed step")
        weight = state.get("weight")
        if not isinstance(weight, (int, float)) or not 0 < weight <= 1:
            raise ValueError("checkpoint statistic weight must lie in (0, 1]")
        for key in ("lr", "weight_decay"):
            value = ckpt.get(key)
            if not isinstance(value, (int, float)) or not math.isfinite(value) or value < 0:
                raise ValueError(f"checkpoint {key} must be a finite nonnegative number")
        ema_shapes = {f"{layer}.{stat}": (g.n, g.n) for g in self._core.groups.values() for layer, stat in g.keys}
        moment_shapes = dict(zip(self._core.names, (tuple(p.shape) for p in self._core.params)))
        if set(state.get("ema", {})) != set(ema_shapes) or set(state.get("moments", {})) != set(moment_shapes):
            raise ValueError("checkpoint statistic / projection names differ from these blocks")
        for key, shape in ema_shapes.items():
            if tuple(state["ema"][key].shape) != shape:
                raise ValueError(f"checkpoint statistic {key} has the wrong shape")
        wanted = {"m", "v"} if self._config["kind"] == "adamt" else {"m"}
        for name, shape in moment_shapes.items():
            entry = state["moments"][name]
            if set(entry) != wanted or any(tuple(x.shape) != shape for x in entry.values()):
                raise ValueError(f"checkpoint moments of {name} do not fit this optimizer")
        return state

    def load_state_dict(self, state_dict):
        """Load the same full checkpoint on every rank into a fresh optimizer (factors are recomputed)."""
        self._assert_open()
        if self._capturing or self._microbatches or self._core.t:
            raise RuntimeError("load_state_dict() needs a fresh optimizer: nothing captured, no step taken")
        state = self._validate_checkpoint(state_dict)
        self._core.load_full_state(state)
        group = self.param_groups[0]
        group["lr"], group["weight_decay"] = state_dict["lr"], state_dict["weight_decay"]

    @property
    def diagnostics(self):
        """Fallback counts and recent timings of the engine."""
        self._assert_open()
        out = {"fallbacks": self._core.fallbacks, "extra_iterations": self._core.extra,
               "timing": dict(self._core.timing), "gpu_ms": dict(self._core.gpu_ms)}
        if self._core.check:
            out["check"] = dict(self._core.check)
        return out

    def close(self):
        """Finish outstanding work, detach hooks and release the engine's NCCL group (call on every rank)."""
        if getattr(self, "_closed", True):
            return
        self._core.side.synchronize()
        for handle in self._hooks:
            handle.remove()
        self._hooks.clear()
        if self._core.pg is not None and dist.is_initialized():
            dist.destroy_process_group(self._core.pg)
        self._closed = True
        _LIVE.discard(self)


class FastMuonT(_FastToner):
    """Fast MuonT: strengths (1/2, 1/8), statistic momentum equal to Muon's momentum, ten Newton-Schulz steps with
    BF16 operands and FP32 accumulation, shaped decay.  ``lr`` is the matrix learning rate."""

    def __init__(self, blocks, lr, *, statistic_momentum=None, **kwargs):
        if statistic_momentum is None:
            statistic_momentum = kwargs.get("momentum", 0.95)
        super().__init__(blocks, lr, kind="muont", statistic_momentum=statistic_momentum, **kwargs)


class FastAdamT(_FastToner):
    """Fast AdamT with matched quarter-power factors; statistic momentum defaults to ``betas[1]``."""

    def __init__(self, blocks, lr, *, statistic_momentum=None, **kwargs):
        kwargs.setdefault("betas", (0.9, 0.98))
        if statistic_momentum is None:
            if len(kwargs["betas"]) != 2:
                raise ValueError("betas must contain two coefficients")
            statistic_momentum = kwargs["betas"][1]
        kwargs.setdefault("inner_strength", 0.25)
        kwargs.setdefault("outer_strength", 0.25)
        super().__init__(blocks, lr, kind="adamt", statistic_momentum=statistic_momentum, **kwargs)
