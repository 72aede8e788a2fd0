"""The plain Muon baseline on the same kernels as MuonT: momentum, batched Newton-Schulz, scaled apply.

Mirror of the reference's baseline optimizer (``Muon``, src/toner/fast/muon.py:53-164): same constructor arguments,
state key (``momentum_buffer``), ``precond`` hook and distributed scheme (rank r orthogonalises matrices r, r + W, ...
of every stack, the results are all-gathered, every rank applies all updates).  Matrices of one shape are always
stacked (``batched`` is accepted; both settings run the batched kernels, which compute the same per-matrix math).
Only ``ns_mode="tpu"`` exists here: BF16 operands with FP32 accumulation on the tensor cores.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .. import ops


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr, momentum=0.95, nesterov=True, ns_steps=10, eps=1e-5, weight_decay=0.0,
                 ns_mode="tpu", batched=True, distributed=True):
        if ns_mode != "tpu":
            raise ValueError("the CUDA Newton-Schulz kernel implements ns_mode='tpu' only")
        if lr < 0 or weight_decay < 0 or not 0 <= momentum < 1 or ns_steps < 1 or eps <= 0:
            raise ValueError("lr and weight_decay must be non-negative, momentum in [0, 1), ns_steps >= 1, eps > 0")
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps, eps=eps,
                                      weight_decay=weight_decay, ns_mode=ns_mode, batched=batched))
        for group in self.param_groups:
            for p in group["params"]:
                if p.ndim != 2 or p.dtype != torch.float32 or not p.is_contiguous():
                    raise ValueError("Muon takes contiguous two-dimensional FP32 matrices")
                if p.shape[0] % 8 or p.shape[1] % 8:
                    raise ValueError("matrix sides must be multiples of 8")
        import torch.distributed as dist
        self.dist = dist if (distributed and dist.is_available() and dist.is_initialized()
                             and dist.get_world_size() > 1) else None
        self.precond = None   # optional (p, grad) -> preconditioned gradient, as in the reference
        self._stacks: Dict[Tuple[int, Tuple[int, int]], dict] = {}

    def _stack(self, gi: int, shape: Tuple[int, int], members: List[torch.nn.Parameter]) -> dict:
        """Momentum buffers of one shape live in one (count, rows, cols) stack; state[p]['momentum_buffer'] are views."""
        key = (gi, shape)
        ids = tuple(id(p) for p in members)
        st = self._stacks.get(key)
        if st is None or st["ids"] != ids:
            dev = members[0].device
            buf = torch.zeros((len(members),) + shape, device=dev)
            for j, p in enumerate(members):
                old = self.state[p].get("momentum_buffer")
                if old is not None:
                    buf[j].copy_(old)
                self.state[p]["momentum_buffer"] = buf[j]
            st = self._stacks[key] = dict(ids=ids, buf=buf, u=torch.empty_like(buf), weights=ops.pointer_table(members),
                                          grad_ptrs=None, grad_key=None)
        return st

    @torch.no_grad()
    def step(self, closure=None):
        if closure is not None:
            raise ValueError("Muon.step() takes no closure")
        for gi, g in enumerate(self.param_groups):
            mu, lr, wd = g["momentum"], g["lr"], g["weight_decay"]
            by_shape: Dict[Tuple[int, int], List[torch.nn.Parameter]] = {}
            for p in g["params"]:
                if p.grad is None:
                    continue
                if not p.is_cuda:
                    raise ValueError("toner_b200 kernels need CUDA tensors (there is no CPU path)")
                if p.grad.is_sparse:
                    raise RuntimeError("Muon does not support sparse gradients")
                by_shape.setdefault(tuple(p.shape), []).append(p)
            for shape, members in by_shape.items():
                st = self._stack(gi, shape, members)
                grads = [p.grad if self.precond is None else self.precond(p, p.grad) for p in members]
                grads = [x if x.is_contiguous() and x.dtype == torch.float32 else x.float().contiguous() for x in grads]
                key = tuple(x.data_ptr() for x in grads)
                if st["grad_key"] != key:
                    st["grad_ptrs"], st["grad_key"] = ops.pointer_table(grads), key
                ops.muont_momentum(st["grad_ptrs"], st["buf"], st["u"], mu, bool(g["nesterov"]), None)
                u = st["u"] if g["nesterov"] else st["buf"]
                if self.dist is None:
                    o = ops.ns_polar(u, g["ns_steps"], g["eps"], out=st["u"])
                else:   # rank r takes matrices r, r + W, ...; padded to equal shares for the all-gather
                    world, rank = self.dist.get_world_size(), self.dist.get_rank()
                    count = len(members)
                    per = -(-count // world)
                    mine = torch.zeros((per,) + shape, device=u.device)
                    own = u[rank::world]
                    mine[: own.shape[0]].copy_(own)
                    ops.ns_polar(mine, g["ns_steps"], g["eps"], out=mine)
                    gathered = torch.empty((world, per) + shape, device=u.device)
                    self.dist.all_gather_into_tensor(gathered, mine)
                    o = gathered.transpose(0, 1).reshape((per * world,) + shape)[:count].contiguous()
                ops.apply_scaled(st["weights"], o, 1.0 - lr * wd, -lr * max(1.0, shape[0] / shape[1]) ** 0.5)
        return None
