"""Layer-sharded asynchronous Toner step for uniform transformer blocks.

Work split on one multi-GPU box (one process per GPU):

* every rank holds the sampled BF16 input rows of *all* layers for its own tokens and computes the
  partial Grams of every statistic with the SYRK kernel (data parallel);
* layers are owned by ranks in contiguous blocks; owners receive the summed Grams (NCCL
  reduce-scatter of packed FP32 triangles, issued chunk by chunk so that it overlaps the SYRK of the
  next chunk), keep the statistic EMAs, compute the inverse-root factors and the parameter changes of
  their layers;
* the changes of the roles sit in two flat buffers per rank; each is moved by one NCCL all-gather, the first
  while the second is still being computed, and every rank adds all of them to its replica of the weights.

``begin()`` runs statistics and factors on a high-priority side stream so that they overlap the
last backward pass; ``step()`` joins it.  The only host synchronisation in ``step()`` is the wait
for the factors' convergence flags.

Interface and ownership rules follow the reference's FastTonerCore (src/toner/fast/engine.py:173-345,
556-644, 774-880); the arithmetic is the one documented in ``toner_b200.core``.
"""

from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import core, ops

KINDS_D = ("attn", "o", "mlp")  # statistics of hidden width, per layer, in this order
ROLE_KIND = {"q": "attn", "k": "attn", "v": "attn", "o": "o", "attn_proj": "o", "gate": "mlp", "up": "mlp",
             "fc": "mlp", "down": "down", "mlp_proj": "down"}


def layer_counts(layers: int, world: int, weights: Optional[Sequence[float]] = None) -> List[int]:
    """Layers owned by each rank, as contiguous blocks: equal split, or proportional to ``weights`` by
    largest remainder (src/toner/fast/engine.py:66-83)."""
    if not weights:
        if layers % world:
            raise ValueError("layers must split evenly over the ranks (or give owner weights)")
        return [layers // world] * world
    w = [max(0.0, float(x)) for x in weights]
    if len(w) != world or sum(w) <= 0:
        raise ValueError("owner weights need one non-negative weight per rank")
    raw = [layers * x / sum(w) for x in w]
    cnt = [int(x) for x in raw]
    by_remainder = sorted(range(world), key=lambda r: raw[r] - cnt[r], reverse=True)
    for r in by_remainder[: layers - sum(cnt)]:
        cnt[r] += 1
    return cnt


def chunk_plan(per_rank: int, chunks: int) -> int:
    """Number of chunks actually used: the largest divisor of `per_rank` not above the request."""
    chunks = max(1, min(int(chunks), per_rank))
    while per_rank % chunks:
        chunks -= 1
    return chunks


def chunk_members(world: int, per_rank: int, chunks: int, c: int) -> List[int]:
    """Statistic indices reduced together in chunk c, in (rank, j) order: statistic r*per + c*cs + j lands
    at row r*cs + j of the chunk's send buffer, so a reduce-scatter hands rank r rows [r*cs, (r+1)*cs), i.e.
    its own statistics c*cs .. (c+1)*cs - 1."""
    cs = per_rank // chunks
    return [r * per_rank + c * cs + j for r in range(world) for j in range(cs)]


def flat_layout(sizes: Sequence[int]) -> List[int]:
    """Offsets of the roles' change stacks inside one rank's flat exchange buffer (roles in registration order)."""
    offsets, total = [], 0
    for size in sizes:
        offsets.append(total)
        total += int(size)
    return offsets


def gathered_block(gathered: torch.Tensor, rank: int, offset: int, size: int, shape) -> torch.Tensor:
    """Rank `rank`'s stack of one role inside the all-gathered (world, total) buffer: layers rank*per .. of that role."""
    return gathered[rank, offset: offset + size].view(tuple(shape))


def owner_block(flat: torch.Tensor, owned: int, unit_offset: int, numel: int, shape) -> torch.Tensor:
    """One role's stack inside the flat exchange buffer of a rank that owns `owned` layers.  The buffer is the roles'
    stacks back to back, each (owned, out, in); `unit_offset` is the sum of the earlier roles' matrix sizes, so the
    stack starts at owned * unit_offset whatever the rank owns (ranks may own different numbers of layers)."""
    return flat[owned * unit_offset: owned * (unit_offset + numel)].view((owned,) + tuple(shape))


class StatGroup:
    """All statistics of one width: row buffers for every layer, EMAs and factors for the owned ones."""

    def __init__(self, name: str, keys: List[Tuple[int, str]], n: int, rows: int, counts: Sequence[int], rank: int,
                 world: int, device: torch.device, strengths: Tuple[float, float], damping: float,
                 scratch: core.Scratch) -> None:
        """`counts[r]` statistics are owned by rank r, in key order (contiguous layer blocks; ranks may own different
        numbers of layers, a rank may own none)."""
        self.name, self.keys, self.n, self.rows = name, keys, n, rows
        self.counts = [int(c) for c in counts]
        per_rank = self.counts[rank]
        self.uneven = len(set(self.counts)) > 1
        self.k_all, self.per, self.rank, self.world = len(keys), per_rank, rank, world
        self.lo = sum(self.counts[:rank])
        self.own = keys[self.lo: self.lo + per_rank]
        self.tri = n * (n + 1) // 2
        # one stacked row buffer: statistic s of this rank's tokens is rows_buf[s]
        self.rows_buf = torch.empty(self.k_all, rows, n, device=device, dtype=torch.bfloat16)
        self.factors = core.FactorSet(per_rank, n, device, strengths, damping, scratch)
        self.partial: Optional[torch.Tensor] = None   # (chunks, world, cs, tri) packed partial Grams (world > 1)
        self.summed: Optional[torch.Tensor] = None    # (per, tri) summed Grams of the owned statistics
        self.chunk_stats = per_rank

    def plan_chunks(self, chunks: int) -> None:
        """Split the owned block into `chunks` pieces; chunk c of every rank is reduced together."""
        dev = self.rows_buf.device
        if self.uneven:
            # Ranks own different numbers of statistics: one piece, the partial Grams in key order (rank blocks are
            # contiguous), summed at the owners by the uneven (list) form of reduce-scatter.
            self.chunks, self.chunk_stats = 1, self.per
            self.partial = torch.empty(1, self.k_all, self.tri, device=dev, dtype=torch.float32)
            self.summed = torch.empty(1, self.per, self.tri, device=dev, dtype=torch.float32)
            self.chunk_lists = [[self.rows_buf[s] for s in range(self.k_all)]]
            return
        chunks = chunk_plan(self.per, chunks)
        self.chunks = chunks
        self.chunk_stats = self.per // chunks
        self.partial = torch.empty(chunks, self.world, self.chunk_stats, self.tri, device=dev, dtype=torch.float32)
        self.summed = (torch.empty(chunks, self.chunk_stats, self.tri, device=dev, dtype=torch.float32)
                       if self.world > 1 else None)
        # row buffers feeding chunk c, in (rank, j) order: statistic r*per + c*cs + j
        self.chunk_lists = [[self.rows_buf[s] for s in chunk_members(self.world, self.per, chunks, c)]
                            for c in range(chunks)]


class FastTonerCore:
    """MuonT or AdamT over the projection matrices of L uniform blocks, sharded by layer."""

    def __init__(self, named: Dict[str, torch.Tensor], bindings: Dict[str, Tuple[int, str, str]], kind: str, *,
                 layers: int, hid: int, mlp: int, local_rows: int, args, world: int, rank: int,
                 device: torch.device, row_capacity: Optional[int] = None) -> None:
        """`row_capacity` (default: `local_rows`) is what the row buffers hold: with a smaller capacity the step's
        rows arrive in local_rows / row_capacity pieces, each folded into the partial Grams by chunk_stats()."""
        if kind not in ("adamt", "muont"):
            raise ValueError("kind must be 'adamt' or 'muont'")
        row_capacity = local_rows if row_capacity is None else int(row_capacity)
        if row_capacity <= 0 or local_rows % row_capacity:
            raise ValueError("the row buffers' capacity must divide this rank's rows per step")
        self.row_pieces = local_rows // row_capacity
        self.pieces_done = 0
        self.ev_chunk: Optional[torch.cuda.Event] = None
        self.kind, self.args, self.world, self.rank, self.device = kind, args, world, rank, device
        self.L = layers
        self.rows_total = local_rows * world
        self.decay = float(args.statistic_momentum)
        # Layers per rank: equal blocks, or in proportion to `owner_weights` (a slower GPU can be given fewer layers to
        # factor and update, a zero weight none; every rank still computes its rows' partial Grams of every statistic),
        # as --toner-owner-weights does in the reference (src/toner/fast/engine.py:66-83,215-239).
        weights = getattr(args, "owner_weights", None)
        self.layer_counts = layer_counts(layers, world, list(weights) if weights else None)
        self.uneven = len(set(self.layer_counts)) > 1
        self.per_layers = self.layer_counts[rank]
        self.lo_layer = sum(self.layer_counts[:rank])
        self.check_every = int(getattr(args, "check_every", 0) or 0)
        self.check: Dict[str, Tuple[float, float, float]] = {}
        self.owner_of_layer = [r for r, c in enumerate(self.layer_counts) for _ in range(c)]
        self.scratch = core.Scratch()
        strengths = (float(args.inner_strength), float(args.outer_strength))
        damping = float(getattr(args, "damping", 1e-3))
        self.groups = {
            "d": StatGroup("d", [(i, k) for i in range(layers) for k in KINDS_D], hid, row_capacity,
                           [len(KINDS_D) * c for c in self.layer_counts], rank, world, device, strengths, damping,
                           self.scratch),
            "f": StatGroup("f", [(i, "down") for i in range(layers)], mlp, row_capacity, list(self.layer_counts), rank,
                           world, device, strengths, damping, self.scratch),
        }
        self.weight = 0.0
        # matrices by role; the owned layers of a role form one MatrixGroup
        self.names = list(named.keys())
        self.params = list(named.values())
        self.param_groups = [{"params": self.params, "lr": 0.0, "weight_decay": float(args.weight_decay)}]
        roles: Dict[str, List[Tuple[int, str, torch.Tensor]]] = {}
        for name, p in named.items():
            layer, role, stat_kind = bindings[name]
            if stat_kind != ROLE_KIND[role]:
                raise ValueError(f"Invalid input-statistic binding for matrix {name}")
            roles.setdefault(role, []).append((layer, name, p))
        self.roles = {}
        lo_layer = self.lo_layer
        plan = []
        for role, items in roles.items():
            items.sort(key=lambda it: it[0])
            if [it[0] for it in items] != list(range(layers)):
                raise ValueError(f"role {role} must have exactly one matrix per layer")
            plan.append((role, items))
        # Exchange layout.  Roles of one matrix shape go through Newton-Schulz together and their changes sit in one flat
        # buffer (a "part"); the parts are worked through largest first, and each is all-gathered (one large NCCL
        # transfer) while the next ones are still being computed.  Only the last part's transfer has nothing to hide
        # behind, and it is the smallest.  One buffer when there is nothing to exchange.
        plan.sort(key=lambda pr: -pr[1][0][2].numel())
        if world > 1 and len(plan) > 1:
            by_shape: Dict[Tuple[int, ...], List[int]] = {}
            for i, (_, items) in enumerate(plan):
                by_shape.setdefault(tuple(items[0][2].shape), []).append(i)
            groups_of = sorted(by_shape.values(), key=lambda idx: -sum(plan[i][1][0][2].numel() for i in idx))
            plan = [plan[i] for idx in groups_of for i in idx]
            bounds, at = [], 0
            for idx in groups_of:
                bounds.append((at, at + len(idx)))
                at += len(idx)
        else:
            bounds = [(0, len(plan))]
        self.parts = []
        for lo_i, hi_i in bounds:
            numels = [items[0][2].numel() for _, items in plan[lo_i:hi_i]]
            unit = sum(numels)                                   # elements one layer contributes to this part
            total = self.per_layers * unit
            if world == 1:
                gathered = None
            elif self.uneven:   # one flat buffer per rank, sized by what that rank owns
                gathered = [torch.empty(c * unit, device=device, dtype=torch.float32) for c in self.layer_counts]
            else:
                gathered = torch.empty(world, total, device=device, dtype=torch.float32)
            part = dict(delta=torch.empty(total, device=device, dtype=torch.float32), gathered=gathered, roles=[])
            for (role, items), numel, unit_offset in zip(plan[lo_i:hi_i], numels, flat_layout(numels)):
                all_w = [it[2] for it in items]
                own_w = all_w[lo_layer: lo_layer + self.per_layers]
                stat_kind = ROLE_KIND[role]
                if stat_kind == "down":
                    g, first, step = self.groups["f"], 0, 1
                else:
                    g, first, step = self.groups["d"], KINDS_D.index(stat_kind), len(KINDS_D)
                group = core.MatrixGroup(own_w, g.factors, first, step, kind) if own_w else None
                matrix = tuple(all_w[0].shape)
                delta = owner_block(part["delta"], self.per_layers, unit_offset, numel, matrix)
                self.roles[role] = dict(group=group, all=all_w, names=[it[1] for it in items], delta=delta,
                                        unit_offset=unit_offset, numel=numel, matrix=matrix,
                                        all_ptrs=ops.pointer_table(all_w))
                part["roles"].append(role)
            self.parts.append(part)
        self.t = 0
        self.steps = 0
        self.timing: Dict[str, float] = {}
        self.gpu_ms: Dict[str, float] = {}
        self.main_stream = torch.cuda.current_stream(device)
        self.side = torch.cuda.Stream(device=device, priority=-1)
        self.pg = dist.new_group(backend="nccl") if world > 1 else None
        # SMs left free for NCCL's kernels while a collective overlaps the persistent GEMMs (see _beside_collective)
        # (off by default: on two ranks reserving 8-32 SMs changed nothing or cost 1-2 %)
        self.sm_reserve = int(getattr(args, "nccl_sm_reserve", 0)) if world > 1 else 0
        if world > 1 or self.row_pieces > 1:   # packed partial Grams: summed over ranks, or over the pieces of a step
            for g in self.groups.values():
                g.plan_chunks(int(getattr(args, "stat_chunks", 4)) if world > 1 else 1)
        self.begun = False
        self.health = ops.Health()   # the update phase's products: armed at the end of step(), read in the next one
        self._ev: Optional[List[torch.cuda.Event]] = None
        self._ev_last: Optional[List[torch.cuda.Event]] = None
        self.ev_done: Optional[torch.cuda.Event] = None

    @classmethod
    def from_blocks(cls, blocks, named: Dict[str, torch.Tensor], kind: str, *, hid: int, mlp: int, rows_total: int, args,
                    world: int, rank: int, device: torch.device) -> "FastTonerCore":
        """Direct construction the way a trainer that owns the model does it (the reference's
        ``FastTonerCore(blocks, named, kind, hid=..., mlp=..., rows_total=..., args=..., world, rank, device)``,
        src/toner/fast/engine.py:176-190, used by reproduce/marin/optimizer.py:67-78).

        ``blocks[i]`` carries the row buffers ``input_rows_{attn,o,mlp,down}`` of capacity (rows, width); ``named``
        maps ``body.blocks.<i>.<q|k|v|o|gate|up|down>.weight`` to the FP32 matrices; ``args`` is the reference's
        argument namespace (``toner_decay``, ``toner_alpha[_in|_out]``, ``toner_split``, ``wd``, ``beta1``, ``beta2``,
        ``eps``, ``muon_*``).  The blocks' row-buffer attributes are rebound to views of this engine's stacked
        buffers, so the model's capture writes where the SYRK reads; a capacity below the rank's rows per step means
        the trainer folds pieces with chunk_stats() / chunk_wait()."""
        from types import SimpleNamespace
        layers = len(blocks)
        matrices, bindings = {}, {}
        for name, p in named.items():
            if not (name.startswith("body.blocks.") and p.ndim == 2):
                continue
            parts = name.split(".")
            if len(parts) != 5 or parts[3] not in ROLE_KIND:
                raise ValueError(f"cannot bind matrix {name} to an input statistic")
            matrices[name] = p
            bindings[name] = (int(parts[2]), parts[3], ROLE_KIND[parts[3]])
        if getattr(args, "muon_ns_mode", "tpu") != "tpu":
            raise ValueError("the CUDA Newton-Schulz kernel implements ns_mode='tpu' only")
        if kind == "muont":
            split = bool(getattr(args, "toner_split", False))
            inner = float(args.toner_alpha_in if split else args.toner_alpha)
            outer = float(args.toner_alpha_out if split else args.toner_alpha)
        else:
            inner = outer = 0.25
        ours = SimpleNamespace(
            statistic_momentum=float(args.toner_decay), inner_strength=inner, outer_strength=outer, damping=1e-3,
            weight_decay=float(args.wd), beta1=float(getattr(args, "beta1", 0.9)), beta2=float(getattr(args, "beta2", 0.98)),
            eps=float(getattr(args, "eps", 1e-15)), momentum=float(getattr(args, "muon_momentum", 0.95)),
            nesterov=bool(getattr(args, "muon_nesterov", True)), ns_steps=int(getattr(args, "muon_ns_steps", 10)),
            ns_eps=float(getattr(args, "muon_eps", 1e-5)), stat_chunks=4,
            owner_weights=([float(x) for x in str(args.toner_owner_weights).split(",")]
                           if getattr(args, "toner_owner_weights", "") else None),
            check_every=int(getattr(args, "toner_check_every", 0) or 0))
        if rows_total % world:
            raise ValueError("rows_total must be a multiple of the number of ranks")
        capacity = int(blocks[0].input_rows_attn.size(0))
        core_ = cls(matrices, bindings, kind, layers=layers, hid=hid, mlp=mlp, local_rows=rows_total // world, args=ours,
                    world=world, rank=rank, device=device, row_capacity=capacity)
        d, f_ = core_.groups["d"], core_.groups["f"]
        for i, block in enumerate(blocks):
            for j, k in enumerate(KINDS_D):
                setattr(block, f"input_rows_{k}", d.rows_buf[len(KINDS_D) * i + j])
            block.input_rows_down = f_.rows_buf[i]
        # stored for the trainer's schedule, as in the reference (src/toner/fast/engine.py:265-272); step() uses "lr"
        core_.param_groups[0]["lr_scale"] = float(getattr(args, "toner_lr_mult", 1.0))
        return core_

    class _NoPool:
        """The reference keeps a thread pool for host eigendecompositions and trainers shut it down at exit; there is
        no host work here."""

        def shutdown(self, wait: bool = True) -> None:
            return None

    pool = _NoPool()

    @property
    def fallbacks(self) -> int:
        return sum(g.factors.fallbacks for g in self.groups.values())

    @property
    def bound_failures(self) -> int:
        """Steps in which an estimated spectrum bound failed its verification (those statistics were repaired)."""
        return sum(g.factors.bound_failures for g in self.groups.values())

    @property
    def extra(self) -> int:
        """Statistics that needed a repair round (factored again with the bound that always holds)."""
        return sum(g.factors.repairs for g in self.groups.values())

    # ------------------------------------------------------------------ statistics (side stream)
    def _beside_collective(self, active: bool) -> None:
        """Products launched from here on run beside a collective (True) or alone (False).  The persistent GEMM
        assigns tiles to its CTAs up front; with all 148 launched while NCCL holds some SMs, the CTAs that find no
        SM start only after others have finished their whole share, which can double the product's duration.
        Leaving `sm_reserve` SMs unclaimed costs that fraction of throughput instead."""
        if self.sm_reserve > 0:
            ops.set_gemm_sm_limit(max(2, ops.sm_count() - self.sm_reserve) if active else 0)

    def _partial_grams(self, g: "StatGroup", c: int) -> None:
        """Packed Grams of statistic chunk c from the rows now in the buffers, added to earlier pieces of the step."""
        mode = ops.PACKED_ACC if self.pieces_done else ops.PACKED
        ops.syrk_upper(g.chunk_lists[c], g.partial[c].view(-1, g.tri), mode)

    def _reduce_to_owners(self, g: "StatGroup", c: int):
        """Sum chunk c's partial Grams over the ranks at the owners (asynchronous; returns the NCCL work)."""
        if g.uneven:
            return dist.reduce_scatter(g.summed[0], list(g.partial[0].split(g.counts)), group=self.pg, async_op=True)
        return dist.reduce_scatter_tensor(g.summed[c], g.partial[c], group=self.pg, async_op=True)

    def chunk_stats(self) -> None:
        """Fold the rows now in the buffers into the step's partial Grams (side stream); the buffers then take the
        next piece of the step.  Call after the forward of a piece's last microbatch, except for the step's last
        piece, which begin() handles (chunk_stats, src/toner/fast/engine.py:348-363)."""
        if self.row_pieces == 1:
            raise RuntimeError("the row buffers hold the whole step; there are no pieces to fold")
        if self.begun or self.pieces_done >= self.row_pieces - 1:
            raise RuntimeError("the last piece of a step belongs to begin()")
        ev = torch.cuda.Event()
        ev.record(self.main_stream)
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            for g in self.groups.values():
                for c in range(g.chunks):
                    self._partial_grams(g, c)
            self.ev_chunk = torch.cuda.Event()
            self.ev_chunk.record(self.side)
        self.pieces_done += 1

    def chunk_wait(self) -> None:
        """The main stream waits until the last piece's Grams have read the row buffers; call before the next piece's
        first forward overwrites them (chunk_wait, src/toner/fast/engine.py:365-369)."""
        if self.ev_chunk is not None:
            self.main_stream.wait_event(self.ev_chunk)

    def discard_pieces(self) -> None:
        """Forget the pieces folded so far (a failed forward discards the step's captured rows)."""
        self.pieces_done = 0

    def _stats(self) -> None:
        """Partial Grams of every statistic from this rank's rows, summed over ranks at the owners, EMA."""
        b = self.decay
        gamma = (1 - b) / self.rows_total
        if self.pieces_done != self.row_pieces - 1:
            raise RuntimeError(f"{self.pieces_done + 1} of the step's {self.row_pieces} row pieces were captured")
        if self.world == 1 and self.row_pieces == 1:
            for g in self.groups.values():
                ops.syrk_upper(g.rows_buf, g.factors.ema, ops.EMA_FULL, b, gamma)   # SYRK with the EMA fused
        elif self.world == 1:
            for g in self.groups.values():
                self._partial_grams(g, 0)
                ops.unpack_ema(g.partial[0, 0], g.factors.ema, b, gamma)
        else:
            pending = []
            for g in self.groups.values():
                for c in range(g.chunks):
                    self._partial_grams(g, c)
                    # NCCL waits for the SYRK just enqueued and runs on its own stream: the next chunk's SYRK overlaps it
                    pending.append((g, c, self._reduce_to_owners(g, c)))
                    self._beside_collective(True)
            self._beside_collective(False)
            for g, c, work in pending:
                work.wait()
                cs = g.chunk_stats
                if cs:
                    ops.unpack_ema(g.summed[c], g.factors.ema[c * cs:(c + 1) * cs], b, gamma)
        self.pieces_done = 0
        self.weight = b * self.weight + (1 - b)

    @torch.no_grad()
    def _stats_as_rows_arrive(self, ready) -> None:
        """Rows still arriving (for example copied from host memory on another stream): `ready` lists (group name,
        first statistic, one past the last, event) in the order the rows land, each group's slices contiguous and in
        order.  On a single rank each slice's SYRK + EMA waits for its own event; with several ranks a group's
        chunked SYRK / reduce-scatter waits for the group's last event.  Either way a group's factors are enqueued
        as soon as its statistics are, so the remaining transfers overlap them."""
        if self.row_pieces != 1:
            raise RuntimeError("streamed rows need row buffers that hold the whole step")
        b = self.decay
        gamma = (1 - b) / self.rows_total
        done = {name: 0 for name in self.groups}
        for name, lo, hi, _ in ready:
            if name not in done or lo != done[name] or not lo < hi <= self.groups[name].k_all:
                raise ValueError(f"slices of group {name} must be contiguous and in order")
            done[name] = hi
        if any(done[name] != g.k_all for name, g in self.groups.items()):
            raise ValueError("the slices must cover every statistic")
        for name, lo, hi, event in ready:
            g = self.groups[name]
            self.side.wait_event(event)
            if self.world == 1:
                ops.syrk_upper(g.rows_buf[lo:hi], g.factors.ema[lo:hi], ops.EMA_FULL, b, gamma)
            if hi != g.k_all:
                continue
            if self.world > 1:   # all of the group's rows are in: partial Grams, sums at the owners, EMA
                pending = []
                for c in range(g.chunks):
                    self._partial_grams(g, c)
                    pending.append((c, self._reduce_to_owners(g, c)))
                    self._beside_collective(True)
                self._beside_collective(False)
                cs = g.chunk_stats
                for c, work in pending:
                    work.wait()
                    if cs:
                        ops.unpack_ema(g.summed[c], g.factors.ema[c * cs:(c + 1) * cs], b, gamma)
            g.factors.compute()
        self.weight = b * self.weight + (1 - b)

    @torch.no_grad()
    def begin(self, ready=None) -> None:
        """Statistics and factors on the side stream; call right after the last microbatch's forward.  With `ready`
        (see _stats_as_rows_arrive) the work follows the rows as they arrive; gpu_ms then reports statistics and
        factors together under "stats"."""
        t0 = time.perf_counter()
        ev_fwd = torch.cuda.Event()
        ev_fwd.record(self.main_stream)
        self._ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev_fwd)
            self._ev[0].record(self.side)
            if ready is None:
                self._stats()
                self._ev[1].record(self.side)
                for g in self.groups.values():
                    g.factors.compute()
            else:
                self._stats_as_rows_arrive(ready)
                self._ev[1].record(self.side)
            self._ev[2].record(self.side)
            self.ev_done = torch.cuda.Event()
            self.ev_done.record(self.side)
        self.begun = True
        self.timing["begin_host"] = time.perf_counter() - t0

    # ------------------------------------------------------------------ updates (main stream)
    @torch.no_grad()
    def step(self) -> None:
        a = self.args
        lr, wd = self.param_groups[0]["lr"], self.param_groups[0]["weight_decay"]
        if self._ev_last is not None and self._ev_last[3].query():
            e = self._ev_last
            self.gpu_ms = {"stats": e[0].elapsed_time(e[1]), "roots": e[1].elapsed_time(e[2]),
                           "update": e[2].elapsed_time(e[3])}
            if self.world > 1:   # the part of "update" spent gathering and applying the other ranks' changes
                self.gpu_ms["exchange"] = e[4].elapsed_time(e[5])   # not hidden behind the last roles' products
        t0 = time.perf_counter()
        if not self.begun:
            self.begin()
        self.begun = False
        flagged = 0
        try:
            with torch.cuda.stream(self.side):
                for g in self.groups.values():
                    flagged += g.factors.finish()       # host waits for the convergence flags only
            # The previous step's update finished long before these flags arrived: its status costs no extra wait.
            self.health.check()
        finally:
            self.main_stream.wait_stream(self.side)
        t1 = time.perf_counter()
        self.t += 1
        works = []
        for part in self.parts:
            # roles of one matrix shape (q, k, v, o; gate, up) go through Newton-Schulz together
            by_shape: Dict[Tuple[int, ...], List[str]] = {}
            for role in part["roles"]:
                by_shape.setdefault(self.roles[role]["matrix"], []).append(role)
            for shape, names in by_shape.items():
                infos = [self.roles[r] for r in names]
                if infos[0]["group"] is not None:
                    grads = [[p.grad for p in info["group"].weights] for info in infos]
                    if self.kind == "muont":
                        core.muont_groups_delta([info["group"] for info in infos], grads, [info["delta"] for info in infos],
                                                self.scratch, lr=lr, weight_decay=wd, momentum=float(a.momentum),
                                                nesterov=bool(a.nesterov), ns_steps=int(a.ns_steps),
                                                ns_eps=float(a.ns_eps))
                    else:
                        for info, gr in zip(infos, grads):
                            core.adamt_group_delta(info["group"], gr, info["delta"], self.scratch, lr=lr, weight_decay=wd,
                                                   betas=(float(a.beta1), float(a.beta2)), eps=float(a.eps), t=self.t)
                if self.world == 1:
                    for info in infos:
                        ops.apply_delta(info["all_ptrs"], info["delta"])
            if self.world > 1:   # this part's changes travel while the next part is computed
                if self.uneven:
                    works.append(dist.all_gather(part["gathered"], part["delta"], group=self.pg, async_op=True))
                else:
                    works.append(dist.all_gather_into_tensor(part["gathered"], part["delta"], group=self.pg, async_op=True))
                self._beside_collective(True)
        self._beside_collective(False)
        self._ev[4].record(self.main_stream)
        for part, work in zip(self.parts, works):
            work.wait()
            for role in part["roles"]:
                info = self.roles[role]
                lo = 0
                for r, owned in enumerate(self.layer_counts):   # rank r's block holds layers lo .. lo + owned - 1
                    if owned:
                        flat = part["gathered"][r]
                        block = owner_block(flat, owned, info["unit_offset"], info["numel"], info["matrix"])
                        ops.apply_delta(info["all_ptrs"][lo: lo + owned], block)
                    lo += owned
        self._ev[5].record(self.main_stream)
        self._ev[3].record(self.main_stream)
        if self.check_every and self.steps % self.check_every == 0:
            self._cross_check()
        self.health.arm("the previous step's update")
        self._ev_last = self._ev
        self.steps += 1
        self.timing.update(roots_host=t1 - t0, update_host=time.perf_counter() - t1)

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            p.grad = None

    # ------------------------------------------------------------------ checkpoint state
    def _gather(self, t: torch.Tensor, counts: Sequence[int]) -> torch.Tensor:
        """Stacks (counts[r], ...) of all ranks, concatenated in rank order (= layer order)."""
        if self.world == 1:
            return t
        if len(set(counts)) == 1:
            full = torch.empty((self.world,) + tuple(t.shape), device=t.device, dtype=t.dtype)
            dist.all_gather_into_tensor(full, t.contiguous(), group=self.pg)
            return full.view((-1,) + tuple(t.shape[1:]))
        outs = [torch.empty((c,) + tuple(t.shape[1:]), device=t.device, dtype=t.dtype) for c in counts]
        dist.all_gather(outs, t.contiguous(), group=self.pg)
        return torch.cat(outs)

    @torch.no_grad()
    def snapshot(self, layers):
        """Collective: the bias-corrected statistics (EMA / weight) of the chosen layers on rank zero, None elsewhere
        (snapshot, src/toner/fast/engine.py:929-941); keys "<layer>.<kind>"."""
        self.main_stream.wait_stream(self.side)
        wanted = set(int(i) for i in layers)
        out = {}
        for g in self.groups.values():
            full = self._gather(g.factors.ema, g.counts)
            if self.rank == 0:
                for (i, k), c in zip(g.keys, full.unbind(0)):
                    if i in wanted:
                        out[f"{i}.{k}"] = (c / self.weight).cpu()
            del full
        return out if self.rank == 0 else None

    @torch.no_grad()
    def _cross_check(self) -> None:
        """Validation only (toner_check_every, src/toner/fast/engine.py:743-770): the factors of this rank's
        statistics against an eigendecomposition of the same EMAs.  For every group and power, check[key] = (largest and
        median relative Frobenius error, largest error weighted by the statistic itself -- the norm the gradient sees)."""
        for name, g in self.groups.items():
            f = g.factors
            if not f.k:
                continue
            c = f.ema.double()
            c = 0.5 * (c + c.transpose(-1, -2))
            lam, vec = torch.linalg.eigh(c)
            lam = lam.clamp_min(0)
            unit = lam / lam.mean(-1, keepdim=True).clamp_min(1e-30) + f.damping
            cn = c / c.diagonal(dim1=-2, dim2=-1).sum(-1)[:, None, None]
            pairs = [(name, f.root("inner"), f.inner_strength)]
            if f.outer_strength != f.inner_strength:
                pairs.append((name + "_out", f.root("outer"), f.outer_strength))
            for key, got, strength in pairs:
                if got is None:
                    continue
                exact = (vec * unit.pow(-strength).unsqueeze(-2)) @ vec.transpose(-1, -2)
                d = got.double() - exact
                rel = d.norm(dim=(-2, -1)) / exact.norm(dim=(-2, -1))
                num = (d @ cn @ d.transpose(-1, -2)).diagonal(dim1=-2, dim2=-1).sum(-1)
                den = (exact @ cn @ exact.transpose(-1, -2)).diagonal(dim1=-2, dim2=-1).sum(-1)
                ec = (num / den).clamp_min(0).sqrt()
                self.check[key] = (rel.max().item(), rel.median().item(), ec.max().item())

    @torch.no_grad()
    def full_state(self):
        """Collective: statistic EMAs and parameter moments gathered on rank zero (None elsewhere)."""
        self.main_stream.wait_stream(self.side)
        ema = {}
        for g in self.groups.values():
            full = self._gather(g.factors.ema, g.counts)
            if self.rank == 0:
                for (i, k), c in zip(g.keys, full.unbind(0)):
                    ema[f"{i}.{k}"] = c.cpu()
            del full
        moments: Dict[str, Dict[str, torch.Tensor]] = {}
        for role, info in self.roles.items():
            group = info["group"]
            for key in (("m",) if self.kind == "muont" else ("m", "v")):
                # a rank that owns no layer still joins the gather, with an empty stack
                stack = getattr(group, key) if group is not None else torch.empty((0,) + info["matrix"], device=self.device)
                full = self._gather(stack, self.layer_counts)
                if self.rank == 0:
                    for name, val in zip(info["names"], full.unbind(0)):
                        moments.setdefault(name, {})[key] = val.cpu()
                del full
        if self.rank != 0:
            return None
        return {"ema": ema, "weight": self.weight, "moments": moments, "t": self.t}

    @torch.no_grad()
    def load_full_state(self, sd) -> None:
        """Every rank picks its owned statistics and moments by name (any world size)."""
        for g in self.groups.values():
            for j, (i, k) in enumerate(g.own):
                g.factors.ema[j].copy_(sd["ema"][f"{i}.{k}"])
            g.factors.statistics_replaced()
        self.weight = sd["weight"]
        self.t = sd["t"]
        lo_layer = self.lo_layer
        for role, info in self.roles.items():
            group = info["group"]
            if group is None:
                continue
            names = info["names"][lo_layer: lo_layer + self.per_layers]
            missing = [nm for nm in names if nm not in sd["moments"]]
            if missing:
                raise ValueError(f"checkpoint has no Toner moments for {missing[:3]}...")
            for j, nm in enumerate(names):
                group.m[j].copy_(sd["moments"][nm]["m"])
                if group.v is not None:
                    group.v[j].copy_(sd["moments"][nm]["v"])
