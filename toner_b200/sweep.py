"""Kernel sweep: times one kernel of the optimizer step in isolation and reports its roofline fraction.

    python -m toner_b200.sweep syrk  --rows 65536 --n 2048 --k 4 [--mode ema|packed]
    python -m toner_b200.sweep roots --n 2048 --k 4 --p 8 --q 4 [--cond 1e4]
    python -m toner_b200.sweep ns    --m 2048 --n 8192 --batch 2
    python -m toner_b200.sweep gemm  --n 8192 [--split] [--tri]
    python -m toner_b200.sweep ema   --n 2048 --k 16
    python -m toner_b200.sweep update --per 4194304 --count 24
    python -m toner_b200.sweep all   (the shapes of the reference's kernel sweep, reduced to fit a few GB)

Shapes follow the reference's own self-benchmarks (src/toner/fast/syrk.py:389-442, src/toner/fast/muon.py:165-199):
BF16 N x d rows for SYRK, SPD d x d matrices Q diag(lambda) Q^T with log-uniform lambda for the roots, FP32
d x 4d Gaussian matrices for Newton-Schulz.  Every input is synthetic and seeded.  Timing: CUDA events on
the launching stream, `--warmup` untimed calls, `--reps` timed calls, inputs larger than L2 or an L2 flush
between calls.  Each run prints one JSON line per kernel with the algorithmic work, the time, the achieved
rate and its fraction of the peak in MEASURED_PEAKS.json (burst BF16 figure: the kernel is timed alone).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from toner_b200 import ops  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops": p["bf16_tflops"], "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


_flush = None


def flush_l2():
    """Write a buffer larger than the 126 MB L2 so that the next call starts cold."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


PHASES = False


def timed(fn, warmup: int, reps: int, flush: bool):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if PHASES:  # one extra, untimed call with the kernels' own cycle counters on
        ops.gemm_phase_cycles(True)
        fn()
        print(json.dumps({"phase_cycles_per_cta": ops.gemm_phase_cycles(False)}), flush=True)
    total = 0.0
    best = float("inf")
    for _ in range(reps):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        total += ms
        best = min(best, ms)
    return total / reps, best


def report(kernel, shape, ms, best, *, flops=None, bytes_=None, extra=None):
    pk = peaks()
    line = {"kernel": kernel, "shape": shape, "ms": round(ms, 4), "ms_best": round(best, 4)}
    if flops is not None:
        t = flops / ms / 1e9
        line.update(bound="tensor", algorithmic_flops=int(flops), achieved=round(t, 1), unit="TFLOP/s", peak=pk["tflops"],
                    frac=round(t / pk["tflops"], 4))
    else:
        g = bytes_ / ms / 1e6
        line.update(bound="hbm", algorithmic_bytes=int(bytes_), achieved=round(g, 1), unit="GB/s", peak=pk["hbm_gbs"],
                    frac=round(g / pk["hbm_gbs"], 4))
    line["peak_source"] = pk["source"]
    if extra:
        line.update(extra)
    ops.assert_healthy()
    print(json.dumps(line), flush=True)
    return line


def rows_like(k, rows, n, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(k, rows, n, device="cuda", generator=g).to(torch.bfloat16)


def spd_stack(k, n, cond, seed=0):
    """Q diag(lambda) Q^T with Haar Q (QR of a Gaussian matrix, sign-fixed) and log-uniform lambda."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = torch.empty(k, n, n, device="cuda")
    for i in range(k):
        q, r = torch.linalg.qr(torch.randn(n, n, device="cuda", dtype=torch.float64, generator=g))
        q = q * torch.sign(torch.diagonal(r)).unsqueeze(0)
        lam = torch.exp(torch.rand(n, device="cuda", dtype=torch.float64, generator=g) * math.log(cond))
        out[i] = ((q * lam) @ q.T).float()
    return out


def bench_syrk(a):
    x = rows_like(a.k, a.rows, a.n)
    small = x.numel() * 2 < (160 << 20)
    if a.mode == "ema":
        out = torch.zeros(a.k, a.n, a.n, device="cuda")
        fn = lambda: ops.syrk_upper(x, out, ops.EMA_FULL, 0.95, 0.05 / a.rows)
    else:
        out = torch.zeros(a.k, a.n * (a.n + 1) // 2, device="cuda")
        fn = lambda: ops.syrk_upper(x, out, ops.PACKED)
    ms, best = timed(fn, a.warmup, a.reps, small)
    flops = a.k * a.rows * a.n * (a.n + 1)
    byts = a.k * (2 * a.rows * a.n + (12 * a.n * a.n if a.mode == "ema" else 2 * a.n * (a.n + 1)))
    return report("syrk_" + a.mode, {"k": a.k, "rows": a.rows, "n": a.n}, ms, best, flops=flops,
                  extra={"full_equivalent_tflops": round(2 * a.k * a.rows * a.n * a.n / ms / 1e9, 1),
                         "algorithmic_bytes": int(byts)})


def bench_roots(a):
    c = spd_stack(a.k, a.n, a.cond)
    iters = ops.inv_roots_iterations(a.n, 1e-3, a.p)
    ws = torch.empty(ops.inv_roots_workspace_bytes(a.k, a.n), device="cuda", dtype=torch.uint8)
    lo = torch.empty_like(c)
    hi = torch.empty_like(c) if a.q > 1 else None
    fn = lambda: ops.inv_roots(c, 1e-3, a.p, a.q, root_lo=lo, root_hi=hi, workspace=ws)
    ms, best = timed(fn, a.warmup, a.reps, False)
    log2p, log2q = int(math.log2(a.p)), int(math.log2(a.q))
    order = ops.inv_roots_finish_order(a.n, 1e-3, a.p)
    split = (iters - 1) * (log2p + 2) + log2q     # X T and T^p M per step (no X product first, no M last), squarings
    single = order - 1                            # Horner steps of the finishing series
    flops = a.k * (split + single) * 2 * a.n ** 3
    return report("inv_roots", {"k": a.k, "n": a.n, "p": a.p, "q": a.q, "cond": a.cond}, ms, best, flops=flops,
                  extra={"iterations": iters, "finish_order": order, "damping": 1e-3, "split_products": split,
                         "single_pass_products": single,
                         "note": "dense count 2 n^3 per product; a split product runs 3 FP16 plane passes, a "
                                 "single-pass one 1, over the tiles meeting the upper triangle"})


def bench_roots_tracked(a):
    """The factor engine as the optimizers drive it: a first call that learns the spectrum (the bound that always
    holds, eight vector slots for dominant directions), then repeated calls scheduled from what it learnt."""
    from . import core
    f = core.FactorSet(a.k, a.n, torch.device("cuda"), (a.q / a.p, 1.0 / a.p) if a.q > 1 else (1.0 / a.p, 1.0 / a.p), 1e-3)
    f.ema.copy_(spd_stack(a.k, a.n, a.cond))
    for _ in range(3):
        f.compute()
        f.finish()

    def fn():
        f.compute()
        f.finish()

    ms, best = timed(fn, 1, a.reps, False)
    log2p, log2q = int(math.log2(a.p)), int(math.log2(a.q))
    split = (f.iterations - 1) * (log2p + 2) + log2q
    single = f.finish_order - 1
    flops = a.k * (split + single) * 2 * a.n ** 3
    return report("inv_roots_tracked", {"k": a.k, "n": a.n, "p": a.p, "q": a.q, "cond": a.cond}, ms, best, flops=flops,
                  extra={"iterations": f.iterations, "finish_order": f.finish_order, "split_products": split,
                         "single_pass_products": single, "deflated": int((f.deflated_host & 255).max()),
                         "estimate": bool(f._estimate_in_flight), "repairs": f.repairs,
                         "note": "includes the host wait for the flags; three single-pass squarings for the norm bound, "
                                 "the block power iteration and the tracking sweeps are not counted as work"})


def bench_ns(a):
    g = torch.Generator(device="cuda").manual_seed(0)
    u = torch.randn(a.batch, a.m, a.n, device="cuda", generator=g)
    out = torch.empty_like(u)
    ws = torch.empty(ops.ns_polar_workspace_bytes(a.batch, a.m, a.n), device="cuda", dtype=torch.uint8)
    fn = lambda: ops.ns_polar(u, a.steps, 1e-5, out=out, workspace=ws)
    ms, best = timed(fn, a.warmup, a.reps, False)
    s, l = min(a.m, a.n), max(a.m, a.n)
    flops = a.batch * a.steps * (4 * s * s * l + 2 * s ** 3)
    return report("ns_polar", {"batch": a.batch, "m": a.m, "n": a.n, "steps": a.steps}, ms, best, flops=flops,
                  extra={"note": "dense count as the reference executes it; the two symmetric products run on the "
                                 "tiles meeting the upper triangle only"})


def bench_gemm(a):
    n, batch = a.n, a.batch
    g = torch.Generator(device="cuda").manual_seed(0)
    d = torch.empty(batch, n, n, device="cuda")
    if a.split:
        x = torch.randn(batch, n, n, device="cuda", generator=g)
        x = x + x.transpose(1, 2)
        pl, inv = ops.split16(x)
        A = ops.operand(pl, seg_z=(0, 0, batch))
        B = ops.operand(pl, seg_z=(0, batch, 0))
        fn = lambda: ops.gemm(A, B, m=n, n=n, k=n, batch=batch, fmt=0, segs=3, d=d, alpha_a=inv, alpha_b=inv,
                              tri=a.tri, mirror=a.tri, promote=a.promote, tile_n=a.tile)
        name = "gemm_split3" + ("_sym" if a.tri else "")
    else:
        x = torch.randn(batch, n, n, device="cuda", generator=g).to(torch.bfloat16)
        y = torch.randn(batch, n, n, device="cuda", generator=g).to(torch.bfloat16)
        A, B = ops.operand(x), ops.operand(y)
        fn = lambda: ops.gemm(A, B, m=n, n=n, k=n, batch=batch, fmt=1, d=d, tri=a.tri, mirror=a.tri, tile_n=a.tile)
        name = "gemm_bf16" + ("_sym" if a.tri else "")
    ms, best = timed(fn, a.warmup, a.reps, n * n * batch * 2 < (80 << 20))
    if a.split:
        name += f"_chain{a.promote}"
    return report(name, {"n": n, "batch": batch}, ms, best, flops=batch * 2 * n ** 3,
                  extra={"note": "single-pass dense count 2 n^3 per product"})


def bench_ema(a):
    tri = a.n * (a.n + 1) // 2
    packed = torch.randn(a.k, tri, device="cuda")
    ema = torch.zeros(a.k, a.n, a.n, device="cuda")
    fn = lambda: ops.unpack_ema(packed, ema, 0.95, 0.05)
    ms, best = timed(fn, a.warmup, a.reps, a.k * a.n * a.n * 4 < (160 << 20))
    byts = a.k * 4 * (tri + tri + a.n * a.n)   # read packed, read the upper triangle of C, write all of C
    return report("unpack_ema", {"k": a.k, "n": a.n}, ms, best, bytes_=byts)


def bench_update(a):
    g = torch.Generator(device="cuda").manual_seed(0)
    grads = [torch.randn(a.per, device="cuda", generator=g) for _ in range(a.count)]
    weights = [torch.randn(a.per, device="cuda", generator=g) for _ in range(a.count)]
    m = torch.zeros(a.count, a.per, device="cuda")
    u = torch.empty_like(m)
    mx = torch.zeros(a.count, device="cuda", dtype=torch.int32)
    gp, wp = ops.pointer_table(grads), ops.pointer_table(weights)
    small = a.count * a.per * 4 < (160 << 20)
    ms, best = timed(lambda: ops.muont_momentum(gp, m, u, 0.95, True, mx), a.warmup, a.reps, small)
    report("muont_momentum", {"count": a.count, "per": a.per}, ms, best, bytes_=16 * a.count * a.per)
    ms, best = timed(lambda: ops.apply_delta(wp, u), a.warmup, a.reps, small)
    report("apply_delta", {"count": a.count, "per": a.per}, ms, best, bytes_=12 * a.count * a.per)
    side = int(math.isqrt(a.per))
    if side * side == a.per and side % 8 == 0:
        x = u.view(a.count, side, side)
        planes = torch.empty(2, a.count, side, side, device="cuda", dtype=torch.float16)
        inv = torch.empty(a.count, device="cuda")
        ms, best = timed(lambda: ops.split16(x, planes=planes, inv_scale=inv, maxabs=mx), a.warmup, a.reps, small)
        report("split16", {"count": a.count, "per": a.per}, ms, best, bytes_=8 * a.count * a.per)
        ms, best = timed(lambda: ops.split16(x, planes=planes, inv_scale=inv, scratch=mx), a.warmup, a.reps, small)
        report("maxabs+split16", {"count": a.count, "per": a.per}, ms, best, bytes_=12 * a.count * a.per)
        out = torch.empty(a.count, device="cuda")
        ws = torch.empty(ops.sumsq_scratch_bytes(a.count), device="cuda", dtype=torch.uint8)
        ms, best = timed(lambda: ops.sumsq(x, out=out, scratch=ws), a.warmup, a.reps, small)
        report("sumsq", {"count": a.count, "per": a.per}, ms, best, bytes_=4 * a.count * a.per)
    return None


def bench_capture(a):
    """Recomputed row capture of one micro-batch for `--count` layers of width --n / MLP width --m (one launch)."""
    from . import capture
    from .statistics import sample_positions
    layers, batch, seq, d, dm = a.count, a.batch, 4096, a.n, a.m
    idx = torch.tensor(sample_positions(seq, 32, 16), device="cuda")
    rows = batch * idx.numel()
    at = torch.arange(rows, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda w: [torch.randn(batch, seq, w, device="cuda", generator=g).to(torch.bfloat16) for _ in range(layers)]
    xs, attn, xmid, gs, us = mk(d), mk(d), mk(d), mk(dm), mk(dm)
    w1 = [torch.ones(d, device="cuda") for _ in range(layers)]
    w2 = [torch.ones(d, device="cuda") for _ in range(layers)]
    bufs = [torch.empty(rows, w, device="cuda", dtype=torch.bfloat16) for _ in range(layers) for w in (d, d, d, dm)]
    fn = lambda: capture.capture_recomputed(xs, attn, xmid, gs, us, w1, w2, bufs, at, idx, 1e-5)
    ms, best = timed(fn, a.warmup, a.reps, True)
    byts = layers * rows * 2 * (3 * 2 * d + 3 * dm)      # 2 B in + 2 B out per element; the gated rows read two inputs
    return report("capture_rows_kernel", {"layers": layers, "batch": batch, "seq": seq, "hidden": d, "mlp": dm, "rows": rows},
                  ms, best, bytes_=byts)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["syrk", "roots", "tracked", "ns", "gemm", "ema", "update", "capture", "all", "large"])
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--k", type=int, default=4)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--p", type=int, default=8)
    ap.add_argument("--q", type=int, default=4)
    ap.add_argument("--cond", type=float, default=1e4)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--per", type=int, default=2048 * 2048)
    ap.add_argument("--count", type=int, default=24)
    ap.add_argument("--mode", default="ema", choices=["ema", "packed"])
    ap.add_argument("--split", action="store_true")
    ap.add_argument("--tri", action="store_true")
    ap.add_argument("--tile", type=int, default=0, help="force a tile: 128, 256, 512 for 256x256 on CTA pairs, 1024 for 256x512 on pairs (0: the library chooses)")
    ap.add_argument("--promote", type=int, default=ops.PROMOTE_ACCURATE, help="k-blocks per accumulation chain of a split product")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--phases", action="store_true", help="also print the GEMM kernels' phase cycle counters")
    a = ap.parse_args()
    global PHASES
    PHASES = a.phases
    if not torch.cuda.is_available():
        raise SystemExit("the kernel sweep needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(0)
    table = {"syrk": bench_syrk, "roots": bench_roots, "tracked": bench_roots_tracked, "ns": bench_ns, "gemm": bench_gemm,
             "ema": bench_ema, "update": bench_update, "capture": bench_capture}
    import copy
    if a.kernel == "large":
        # the upper end of the sweep: a million rows, width 8192, condition 1e2 .. 1e6 (a few GB per case)
        for rows, n, k in ((1048576, 768, 2), (1048576, 2048, 1), (262144, 4096, 1), (262144, 8192, 1)):
            b = copy.copy(a); b.rows, b.n, b.k = rows, n, k
            bench_syrk(b)
            torch.cuda.empty_cache()
        for n, k, cond in ((2048, 4, 1e2), (2048, 4, 1e6), (8192, 1, 1e4)):
            b = copy.copy(a); b.n, b.k, b.cond, b.p, b.q = n, k, cond, 8, 4
            bench_roots(b)
            bench_roots_tracked(b)
            torch.cuda.empty_cache()
        b = copy.copy(a); b.m, b.n, b.batch = 8192, 32768, 1
        bench_ns(b)
        return
    if a.kernel != "all":
        table[a.kernel](a)
        return
    for rows, n, k in ((65536, 768, 8), (65536, 2048, 4), (262144, 2048, 1), (65536, 4096, 2), (65536, 8192, 1)):
        b = copy.copy(a); b.rows, b.n, b.k = rows, n, k
        bench_syrk(b)
    for n, k in ((768, 8), (2048, 4), (4096, 2)):
        for p, q in ((8, 4), (4, 1)):
            b = copy.copy(a); b.n, b.k, b.p, b.q = n, k, p, q
            bench_roots(b)
    for d, batch in ((768, 8), (2048, 2), (4096, 1)):
        b = copy.copy(a); b.m, b.n, b.batch = d, 4 * d, batch
        bench_ns(b)
    b = copy.copy(a); b.n, b.k = 2048, 16
    bench_ema(b)
    bench_update(a)
    b = copy.copy(a); b.n, b.m, b.batch = 2048, 5632, 4
    bench_capture(b)


if __name__ == "__main__":
    main()
