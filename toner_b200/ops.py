"""Tensor-level wrappers over the C ABI: torch supplies device memory and streams, nothing else.

Every function enqueues work on the current CUDA stream and raises if the CUDA library is missing or
reports an error; there is no CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import GemmDesc, Operand, check

PACKED, PACKED_ACC, EMA_FULL = 0, 1, 2
PROMOTE_ACCURATE = 2  # k-blocks per tensor-core accumulation chain in FP32-accurate products
_FMT = {torch.float16: 0, torch.bfloat16: 1}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("toner_b200 kernels need CUDA tensors (there is no CPU path)")


def sm_count() -> int:
    return _lib.load().toner_sm_count()


def set_gemm_sm_limit(sms: int) -> None:
    """CTAs the persistent GEMM launches from now on (0: one per SM); see toner_set_gemm_sm_limit."""
    check(_lib.load().toner_set_gemm_sm_limit(int(sms)), "toner_set_gemm_sm_limit")


def launch_count() -> int:
    """Kernels launched by the CUDA library so far."""
    return int(_lib.load().toner_launch_count())


def device_status() -> int:
    """Synchronise the current stream and return (and clear) the kernels' status word; 0 is healthy."""
    out = C.c_int(0)
    check(_lib.load().toner_device_status(_stream(), C.byref(out)), "toner_device_status")
    return out.value


def assert_healthy() -> None:
    code = device_status()
    if code:
        raise _lib.TonerError(f"a CUDA kernel gave up a bounded wait (status {code})")


class Health:
    """The kernels' status word, read without a synchronisation of its own.

    ``arm()`` enqueues a copy of the word into pinned host memory on the current stream and records an event;
    ``check()`` waits for that event (the callers place it where they wait for the stream anyway) and raises
    TonerError if a kernel had given up a bounded wait by then: a product that gave up has written only part of
    its result.  The word is cleared when the error is raised, so the optimizer can be used again."""

    def __init__(self) -> None:
        self._host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._event: Optional[torch.cuda.Event] = None
        self._what = ""

    def arm(self, what: str) -> None:
        check(_lib.load().toner_status_snapshot(self._host.data_ptr(), _stream()), "toner_status_snapshot")
        self._event = torch.cuda.Event()
        self._event.record(torch.cuda.current_stream())
        self._what = what

    def check(self) -> None:
        if self._event is None:
            return
        self._event.synchronize()
        self._event = None
        code = int(self._host[0])
        if code:
            self._host.zero_()
            device_status()   # clears the word on the device
            raise _lib.TonerError(f"a CUDA kernel gave up a bounded wait (status {code}) during {self._what}: "
                                  "its results are incomplete and were not applied")


def gemm_phase_cycles(enable: bool):
    """Read and clear the GEMM kernels' phase cycle counters, then switch the counting on or off
    (toner_gemm_phase_cycles).  Returns a dict of per-CTA averages, or None if nothing was counted."""
    out = (C.c_uint64 * 8)()
    check(_lib.load().toner_gemm_phase_cycles(int(enable), _stream(), out), "toner_gemm_phase_cycles")
    ctas = int(out[7])
    if not ctas:
        return None
    names = ("mma_total", "mma_wait_accumulator", "mma_wait_operands", "tma_wait_stage", "epilogue_wait",
             "epilogue_write", "epilogue_sum")
    return {"ctas": ctas, **{n: int(out[i]) // ctas for i, n in enumerate(names)}}


def operand(t: torch.Tensor, *, mn_major: bool = False, seg_z: Sequence[int] = (0, 0, 0),
            nz: Optional[int] = None, z_step: int = 1) -> Operand:
    """Describe a 16-bit matrix stack (..., rows, cols) with contiguous columns as a GEMM operand."""
    if t.dtype not in _FMT:
        raise ValueError("GEMM operands are FP16 or BF16")
    if t.stride(-1) != 1:
        raise ValueError("GEMM operands need contiguous columns")
    op = Operand()
    op.base = t.data_ptr()
    op.list = None
    op.rows, op.cols = t.shape[-2], t.shape[-1]
    op.ld = t.stride(-2)
    lead = t.shape[:-2]
    count = 1
    for s in lead:
        count *= s
    op.z_stride = t.stride(-3) if t.ndim >= 3 else t.shape[-2] * t.stride(-2)
    if t.ndim > 3:  # (planes, batch, rows, cols): planes and batch must be evenly spaced
        if t.stride(-4) != t.shape[-3] * t.stride(-3):
            raise ValueError("leading dimensions of an operand stack must be evenly spaced")
    op.nz = count if nz is None else nz
    op.mn_major = 1 if mn_major else 0
    for i in range(3):
        op.seg_z[i] = int(seg_z[i])
    op.z_step = z_step
    return op


def operand_list(tensors: Sequence[torch.Tensor], *, mn_major: bool = False) -> Tuple[Operand, object]:
    """Operand made of separately allocated, equally shaped 2-D matrices.  Returns (operand, keepalive)."""
    first = tensors[0]
    arr = (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    for t in tensors:
        if t.shape != first.shape or t.stride() != first.stride() or t.dtype != first.dtype:
            raise ValueError("listed operands must share shape, strides and dtype")
    op = Operand()
    op.base = None
    op.list = C.cast(arr, C.POINTER(C.c_void_p))
    op.rows, op.cols = first.shape
    op.ld = first.stride(0)
    op.z_stride = first.shape[0] * first.stride(0)
    op.nz = 1
    op.mn_major = 1 if mn_major else 0
    return op, arr


def gemm(a: Operand, b: Operand, *, m: int, n: int, k: int, batch: int, fmt: int, segs: int = 1,
         d: Optional[torch.Tensor] = None, d16: Optional[torch.Tensor] = None,
         c: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
         alpha_a: Optional[torch.Tensor] = None, alpha_b: Optional[torch.Tensor] = None,
         beta_v: Optional[torch.Tensor] = None, tri: bool = False, mirror: bool = False, packed: bool = False,
         sumsq: Optional[torch.Tensor] = None, maxabs: Optional[torch.Tensor] = None,
         maxaff: Optional[torch.Tensor] = None, aff: Tuple[float, float] = (0.0, 1.0), tile_n: int = 0, promote: int = 0,
         alpha_b_step: int = 1, promote_all: bool = False, raster: int = 0) -> None:
    """Launch the tcgen05 GEMM (toner_gemm).  d / c are FP32 (batch, m, n) stacks (or packed triangles)."""
    desc = GemmDesc()
    desc.a, desc.b = a, b
    desc.m, desc.n, desc.k, desc.batch = m, n, k, batch
    desc.segs, desc.fmt = segs, fmt
    desc.tri, desc.mirror, desc.packed = int(tri), int(mirror), int(packed)
    desc.alpha, desc.beta = alpha, beta
    desc.alpha_a, desc.alpha_b, desc.beta_v = _ptr(alpha_a), _ptr(alpha_b), _ptr(beta_v)

    def strides(t: torch.Tensor) -> Tuple[int, int]:
        if packed:
            return n, n * (n + 1) // 2
        if t.stride(-1) != 1:
            raise ValueError("results need contiguous columns")
        return t.stride(-2), (t.stride(-3) if t.ndim >= 3 else t.shape[-2] * t.stride(-2))

    if c is not None:
        desc.c = c.data_ptr()
        desc.ldc, desc.c_bs = strides(c)
    if d is not None:
        desc.d = d.data_ptr()
        desc.ldd, desc.d_bs = strides(d)
    if d16 is not None:
        desc.d16 = d16.data_ptr()
        desc.ld16, desc.d16_bs = strides(d16)
        desc.d16_fmt = _FMT[d16.dtype]
    desc.sumsq, desc.maxabs, desc.maxaff = _ptr(sumsq), _ptr(maxabs), _ptr(maxaff)
    desc.aff_a, desc.aff_b = aff
    desc.tile_n = tile_n
    desc.promote = promote
    desc.promote_all = int(promote_all)
    desc.raster = raster
    desc.alpha_b_step = alpha_b_step
    check(_lib.load().toner_gemm(C.byref(desc), _stream()), "toner_gemm")


def syrk_upper(x, out: torch.Tensor, mode: int = PACKED, beta: float = 0.0, gamma: float = 1.0) -> None:
    """Upper-triangle X^T X of BF16 row buffers (toner_syrk_upper).

    ``x`` is a (k, rows, n) stack or a list of k separately allocated (rows, n) buffers."""
    lib = _lib.load()
    if isinstance(x, torch.Tensor):
        _need_cuda(x, out)
        if x.dtype != torch.bfloat16 or x.ndim != 3 or x.stride(2) != 1:
            raise ValueError("row buffers are (k, rows, n) BF16 with contiguous columns")
        k, rows, n = x.shape
        check(lib.toner_syrk_upper(None, x.data_ptr(), x.stride(0), k, rows, n, x.stride(1), out.data_ptr(), mode,
                                   beta, gamma, _stream()), "toner_syrk_upper")
        return
    xs = list(x)
    _need_cuda(*xs, out)
    first = xs[0]
    for t in xs:
        if t.dtype != torch.bfloat16 or t.ndim != 2 or t.stride(1) != 1 or t.shape != first.shape or t.stride(0) != first.stride(0):
            raise ValueError("row buffers are equally shaped (rows, n) BF16 matrices with contiguous columns")
    arr = (C.c_void_p * len(xs))(*[t.data_ptr() for t in xs])
    rows, n = first.shape
    check(lib.toner_syrk_upper(C.cast(arr, C.POINTER(C.c_void_p)), None, 0, len(xs), rows, n, first.stride(0),
                               out.data_ptr(), mode, beta, gamma, _stream()), "toner_syrk_upper")


def gather_rows(x: torch.Tensor, positions: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[(b*P + j), :] = bf16(x[b, positions[j], :]) for a (batch, seq, n) BF16 or FP32 tensor (toner_gather_rows).
    ``positions`` is an int32 device tensor; ``dst`` a contiguous (batch*P, n) BF16 buffer (slice)."""
    _need_cuda(x, positions, dst)
    if x.ndim != 3 or x.stride(2) != 1 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("gather_rows takes a (batch, seq, n) BF16 or FP32 tensor with contiguous features")
    if positions.dtype != torch.int32 or dst.dtype != torch.bfloat16 or not dst.is_contiguous():
        raise ValueError("gather_rows needs int32 positions and a contiguous BF16 destination")
    batch, seq, n = x.shape
    count = positions.numel()
    if dst.numel() != batch * count * n:
        raise ValueError("destination does not hold batch * positions rows")
    check(_lib.load().toner_gather_rows(x.data_ptr(), int(x.dtype == torch.float32), batch, seq, n, x.stride(0), x.stride(1),
                                        positions.data_ptr(), count, dst.data_ptr(), _stream()), "toner_gather_rows")


def unpack_ema(packed: torch.Tensor, ema: torch.Tensor, beta: float, gamma: float) -> None:
    """ema <- beta*ema + gamma*S, S given as packed upper triangles (toner_unpack_ema)."""
    _need_cuda(packed, ema)
    k, n = ema.shape[0], ema.shape[-1]
    if not (packed.is_contiguous() and ema.is_contiguous() and packed.dtype == ema.dtype == torch.float32):
        raise ValueError("unpack_ema needs contiguous FP32 tensors")
    if packed.numel() != k * n * (n + 1) // 2:
        raise ValueError("packed triangle size does not match the EMA stack")
    check(_lib.load().toner_unpack_ema(packed.data_ptr(), ema.data_ptr(), k, n, beta, gamma, _stream()),
          "toner_unpack_ema")


def split16(x: torch.Tensor, *, planes: Optional[torch.Tensor] = None, inv_scale: Optional[torch.Tensor] = None,
            aff: Tuple[float, float] = (0.0, 1.0), maxabs: Optional[torch.Tensor] = None,
            scratch: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """FP16 hi/lo planes (2, batch, rows, cols) of a scaled FP32 stack and the inverse scales (toner_split16)."""
    _need_cuda(x)
    if x.ndim == 2:
        x = x.unsqueeze(0)
    if x.dtype != torch.float32 or x.stride(-1) != 1:
        raise ValueError("split16 takes an FP32 stack with contiguous columns")
    batch, rows, cols = x.shape
    if planes is None:
        planes = torch.empty((2, batch, rows, cols), device=x.device, dtype=torch.float16)
    if inv_scale is None:
        inv_scale = torch.empty(batch, device=x.device, dtype=torch.float32)
    if maxabs is None and scratch is None:
        scratch = torch.empty(batch, device=x.device, dtype=torch.int32)
    check(_lib.load().toner_split16(x.data_ptr(), None, batch, rows, cols, x.stride(1), x.stride(0), aff[0], aff[1],
                                    _ptr(maxabs), _ptr(scratch), planes.data_ptr(), inv_scale.data_ptr(), _stream()),
          "toner_split16")
    return planes, inv_scale


def mm_split(a_planes: torch.Tensor, a_inv: torch.Tensor, b_planes: torch.Tensor, b_inv: torch.Tensor,
             d: torch.Tensor, **kw) -> None:
    """FP32-accurate D[b] = A[b] @ B[b]^T from FP16 hi/lo planes: Ah*Bh + Ah*Bl + Al*Bh in one accumulator."""
    batch, m, k = a_planes.shape[1:]
    n = b_planes.shape[2]
    a = operand(a_planes, seg_z=(0, 0, batch))
    b = operand(b_planes, seg_z=(0, batch, 0))
    kw.setdefault("promote", PROMOTE_ACCURATE)
    gemm(a, b, m=m, n=n, k=k, batch=batch, fmt=0, segs=3, d=d, alpha_a=a_inv, alpha_b=b_inv, **kw)


def inv_roots_iterations(n: int, damping: float, p: int) -> int:
    """The stated Newton iteration count for (n, damping, p) (toner_inv_roots_iterations)."""
    return _lib.load().toner_inv_roots_iterations(n, damping, p)


def inv_roots_workspace_bytes(chunk: int, n: int) -> int:
    return _lib.load().toner_inv_roots_workspace_bytes(chunk, n)


def inv_roots_iterations_for(lower: float, p: int) -> int:
    """Newton steps needed when the normalised spectrum is known to lie in [lower, 1]."""
    return _lib.load().toner_inv_roots_iterations_for(lower, p)


def inv_roots_finish_order(n: int, damping: float, p: int, lower: float = 0.0, iters: int = 0) -> int:
    """Degree of the polynomial that finishes the iteration (its degree - 1 products are single passes); `lower` = 0
    means the bound damping / (n (1 + damping)) that always holds."""
    worst = damping / (n * (1.0 + damping))
    return _lib.load().toner_inv_roots_finish_order_for(max(lower, worst), p, iters)


def inv_roots_schedule(lower: float, p: int, iters: int = 0) -> dict:
    """The whole schedule the engine runs for a spectrum lower bound (toner_inv_roots_schedule; needs no device):
    {"iterations", "steps": [(a_k, b_k), ...], "coefficients": [c_0, ...] of the finishing polynomial in powers of
    r = 1 - mu, "distance": e}."""
    ab = (C.c_double * 128)()
    coef = (C.c_double * 16)()
    order, e = C.c_int32(0), C.c_double(0.0)
    count = _lib.load().toner_inv_roots_schedule(lower, p, iters, ab, 128, coef, 16, C.byref(order), C.byref(e))
    if count <= 0:
        raise ValueError("inv_roots_schedule: lower must lie inside (0, 1), p >= 1, iters 0 or >= 2")
    return {"iterations": count, "steps": [(ab[2 * k], ab[2 * k + 1]) for k in range(count - 1)],
            "coefficients": [coef[j] for j in range(order.value + 1)], "distance": e.value}


def inv_roots(ema: torch.Tensor, damping: float, p: int, q: int = 1, *, iters: int = 0,
              root_lo: Optional[torch.Tensor] = None, root_hi: Optional[torch.Tensor] = None,
              fro2_lo: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
              workspace: Optional[torch.Tensor] = None, chunk: Optional[int] = None, lower: float = 0.0,
              norms: Optional[torch.Tensor] = None, lower_is_estimate: bool = False,
              track: Optional[torch.Tensor] = None, lmin: Optional[torch.Tensor] = None,
              resid: Optional[torch.Tensor] = None, track_sweeps: int = 0, track_restart: bool = False,
              deflate: Optional[torch.Tensor] = None, deflate_rank: int = 1, deflate_restart: bool = False,
              deflated: Optional[torch.Tensor] = None, ritz_norm: bool = False):
    """A^(-1/p) and A^(-q/p) of the damped, trace-normalised statistics (toner_inv_roots_tracked).

    ``lower``: a lower bound of the normalised spectrum valid for every statistic (0: the bound that always
    holds); ``norms`` (k,) receives the bound of lambda_max(A'_b) the engine normalised by, from which the next call's
    bound can be derived.  ``track`` (k, n), ``lmin`` (k,), ``track_sweeps``, ``track_restart``, ``lower_is_estimate``,
    ``resid`` (k,): tracking of the smallest eigenvalue between calls and a bound that is an estimate, verified after
    the chain; ``deflate`` (k, 8, n), ``deflate_rank``, ``deflate_restart``, ``deflated`` (k,) int32: several dominant
    directions found by block power iteration and deflated (see the header); ``ritz_norm``: take the norm from that
    iteration's largest remaining Ritz value instead of three squarings (an estimate, verified with ``lower``).
    Returns (root_lo, root_hi or None, fro2_lo, status); nothing is synchronised."""
    _need_cuda(ema)
    if ema.ndim == 2:
        ema = ema.unsqueeze(0)
    if ema.dtype != torch.float32 or not ema.is_contiguous() or ema.shape[-1] != ema.shape[-2]:
        raise ValueError("statistics are a contiguous FP32 (k, n, n) stack")
    k, n, _ = ema.shape
    dev = ema.device
    if root_lo is None:
        root_lo = torch.empty_like(ema)
    if q > 1 and root_hi is None:
        root_hi = torch.empty_like(ema)
    if fro2_lo is None:
        fro2_lo = torch.empty(k, device=dev, dtype=torch.float32)
    if status is None:
        status = torch.zeros(k, device=dev, dtype=torch.int32)
    if workspace is None:
        if chunk is None:  # keep scratch near 4 GiB unless one statistic needs more
            per = inv_roots_workspace_bytes(1, n)
            chunk = max(1, min(k, (4 << 30) // per))
        workspace = torch.empty(inv_roots_workspace_bytes(chunk, n), device=dev, dtype=torch.uint8)
    if track is not None and (track.shape != (k, n) or track.dtype != torch.float32 or not track.is_contiguous()):
        raise ValueError("the tracking vectors are a contiguous FP32 (k, n) tensor")
    sweeps = (int(track_sweeps) & 63) | (256 if track_restart else 0)
    if deflate is not None and (deflate.shape != (k, 8, n) or deflate.dtype != torch.float32 or not deflate.is_contiguous()):
        raise ValueError("the deflation vectors are a contiguous FP32 (k, 8, n) tensor")
    rank = (int(deflate_rank) & 15) | (256 if deflate_restart else 0) | (512 if ritz_norm else 0)
    check(_lib.load().toner_inv_roots_tracked(ema.data_ptr(), k, n, damping, p, q, iters, lower, int(lower_is_estimate),
                                              root_lo.data_ptr(), _ptr(root_hi), fro2_lo.data_ptr(), status.data_ptr(),
                                              _ptr(norms), _ptr(track), _ptr(lmin), _ptr(resid), sweeps,
                                              _ptr(deflate), rank, _ptr(deflated),
                                              workspace.data_ptr(), workspace.numel(), _stream()),
          "toner_inv_roots_tracked")
    return root_lo, root_hi, fro2_lo, status


def ns_polar_workspace_bytes(batch: int, m: int, n: int) -> int:
    return _lib.load().toner_ns_polar_workspace_bytes(batch, m, n)


def ns_polar(u: torch.Tensor, steps: int = 10, eps: float = 1e-5, *, out: Optional[torch.Tensor] = None,
             maxabs: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Newton-Schulz polar iteration with BF16 operands / FP32 accumulation on a (batch, m, n) stack."""
    _need_cuda(u)
    if u.ndim == 2:
        u = u.unsqueeze(0)
    if u.dtype != torch.float32 or not u.is_contiguous():
        raise ValueError("ns_polar takes a contiguous FP32 (batch, m, n) stack")
    batch, m, n = u.shape
    if out is None:
        out = torch.empty_like(u)
    need = ns_polar_workspace_bytes(batch, m, n)
    if workspace is None:
        workspace = torch.empty(need, device=u.device, dtype=torch.uint8)
    check(_lib.load().toner_ns_polar(u.data_ptr(), batch, m, n, steps, eps, out.data_ptr(), _ptr(maxabs),
                                     workspace.data_ptr(), workspace.numel(), _stream()), "toner_ns_polar")
    return out


def sumsq_scratch_bytes(batch: int) -> int:
    return int(_lib.load().toner_sumsq_scratch_bytes(batch))


def sumsq(x: torch.Tensor, out: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reproducible per-matrix sum of squares of a (batch, rows, cols) FP32 stack (toner_sumsq)."""
    _need_cuda(x)
    if x.ndim == 2:
        x = x.unsqueeze(0)
    batch, rows, cols = x.shape
    if out is None:
        out = torch.empty(batch, device=x.device, dtype=torch.float32)
    if scratch is None:
        scratch = torch.empty(sumsq_scratch_bytes(batch), device=x.device, dtype=torch.uint8)
    check(_lib.load().toner_sumsq(x.data_ptr(), batch, rows, cols, x.stride(1), x.stride(0), scratch.data_ptr(),
                                  out.data_ptr(), _stream()), "toner_sumsq")
    return out


def sumsq_static(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Per-matrix sum of squares with the library's built-in scratch (toner_sumsq_static): for hosts that may
    not give the library device memory to work in.  ``out`` is the caller's (batch,) FP32 result buffer; the
    call itself allocates nothing.  At most ``toner_sumsq_static_max_batch()`` matrices; calls that may overlap
    on the GPU share the scratch and race."""
    _need_cuda(x, out)
    if x.ndim == 2:
        x = x.unsqueeze(0)
    batch, rows, cols = x.shape
    check(_lib.load().toner_sumsq_static(x.data_ptr(), batch, rows, cols, x.stride(1), x.stride(0), out.data_ptr(),
                                         _stream()), "toner_sumsq_static")
    return out


def pointer_table(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """Device array of the tensors' addresses (int64), for kernels over separately allocated matrices."""
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64).to(tensors[0].device, non_blocking=False)


def muont_momentum(grad_ptrs: torch.Tensor, m: torch.Tensor, u: torch.Tensor, mu: float, nesterov: bool,
                   maxabs: Optional[torch.Tensor]) -> None:
    count, per = m.shape[0], m[0].numel()
    check(_lib.load().toner_muont_momentum(grad_ptrs.data_ptr(), m.data_ptr(), u.data_ptr(), count, per, mu,
                                           int(nesterov), _ptr(maxabs), _stream()), "toner_muont_momentum")


def muont_coeffs(fro2: torch.Tensor, first: int, step: int, count: int, n: int, lr: float, wd: float, scale: float,
                 c1: torch.Tensor, c2: torch.Tensor) -> None:
    check(_lib.load().toner_muont_coeffs(fro2.data_ptr(), first, step, count, n, lr, wd, scale, c1.data_ptr(),
                                         c2.data_ptr(), _stream()), "toner_muont_coeffs")


def scale_vec(a: torch.Tensor, b: torch.Tensor) -> None:
    check(_lib.load().toner_scale_vec(a.data_ptr(), b.data_ptr(), a.numel(), _stream()), "toner_scale_vec")


def adamt_first_moment(grad_ptrs: torch.Tensor, m: torch.Tensor, beta1: float) -> None:
    check(_lib.load().toner_adamt_first_moment(grad_ptrs.data_ptr(), m.data_ptr(), m.shape[0], m[0].numel(), beta1,
                                               _stream()), "toner_adamt_first_moment")


def adamt_ratio(t: torch.Tensor, v: torch.Tensor, num: torch.Tensor, beta2: float, bc2: float, eps: float,
                maxabs: Optional[torch.Tensor]) -> None:
    check(_lib.load().toner_adamt_ratio(t.data_ptr(), v.data_ptr(), num.data_ptr(), v.shape[0], v[0].numel(), beta2,
                                        bc2, eps, _ptr(maxabs), _stream()), "toner_adamt_ratio")


def adamt_coeffs(fro2: torch.Tensor, first: int, step: int, count: int, n: int, lr: float, wd: float,
                 ss_before: torch.Tensor, ss_after: torch.Tensor, c1: torch.Tensor, c2: torch.Tensor) -> None:
    check(_lib.load().toner_adamt_coeffs(fro2.data_ptr(), first, step, count, n, lr, wd, ss_before.data_ptr(),
                                         ss_after.data_ptr(), c1.data_ptr(), c2.data_ptr(), _stream()),
          "toner_adamt_coeffs")


def apply_delta(weight_ptrs: torch.Tensor, delta: torch.Tensor) -> None:
    check(_lib.load().toner_apply_delta(weight_ptrs.data_ptr(), delta.data_ptr(), delta.shape[0], delta[0].numel(),
                                        _stream()), "toner_apply_delta")


def apply_scaled(weight_ptrs: torch.Tensor, delta: torch.Tensor, weight_scale: float, delta_scale: float) -> None:
    """W_b <- weight_scale * W_b + delta_scale * delta_b over a pointer table of weights (toner_apply_scaled)."""
    check(_lib.load().toner_apply_scaled(weight_ptrs.data_ptr(), delta.data_ptr(), delta.shape[0], delta[0].numel(),
                                         weight_scale, delta_scale, _stream()), "toner_apply_scaled")


def split16_list(ptrs: torch.Tensor, batch: int, rows: int, cols: int, planes: torch.Tensor, inv_scale: torch.Tensor,
                 scratch: torch.Tensor) -> None:
    """split16 of separately allocated contiguous (rows, cols) FP32 matrices given by a device pointer table."""
    check(_lib.load().toner_split16(None, ptrs.data_ptr(), batch, rows, cols, cols, rows * cols, 0.0, 1.0, None,
                                    scratch.data_ptr(), planes.data_ptr(), inv_scale.data_ptr(), _stream()),
          "toner_split16")


def scale_stack(x: torch.Tensor, coeff: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = coeff[b] * x[b] for (count, ...) FP32 stacks (toner_scale_stack)."""
    check(_lib.load().toner_scale_stack(x.data_ptr(), coeff.data_ptr(), out.data_ptr(), x.shape[0], x[0].numel(),
                                        _stream()), "toner_scale_stack")


def axpby(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor, a: float, b: float) -> None:
    """out = a*x + b*y on contiguous FP32 tensors of equal size (toner_axpby)."""
    _need_cuda(x, y, out)
    if not (x.is_contiguous() and y.is_contiguous() and out.is_contiguous()) or x.numel() != y.numel() != out.numel():
        raise ValueError("axpby needs contiguous tensors of equal size")
    check(_lib.load().toner_axpby(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel(), a, b, _stream()), "toner_axpby")
