"""Run the reference itself on a CUDA device: fixtures for what it computes only there, and its timings.

    python tests/golden/make_tpu_golden.py [--out DIR] [--skip-timing] [--layers L]

The reference package must be importable: either ``REFERENCE_SRC=/path/to/Toner/src`` or an installed copy under
``baseline/_ref`` (``pip install --no-deps --target baseline/_ref <checkout>``; the folder is not tracked).

Three things are produced, each independent of the others (a failure of one is recorded and the rest still runs):

1. Fixtures for arithmetic the reference refuses to run on a CPU (``ns_mode="tpu"`` = BF16 operands, FP32
   accumulation in cuBLAS): ``newton_schulz_tpu.npz`` (per-matrix ``toner.linalg.newton_schulz`` on small seeded
   matrices at 1, 2, 3, 5 and 10 steps, plus how far the reference's own batched and per-matrix paths drift apart,
   ``toner.fast.muon``), ``muont_tpu_small.npz`` / ``muont_tpu_tall.npz`` (``toner.MuonT(ns_mode="tpu")``, weights after
   every step).
2. ``fast_v3_checkpoint_muont.pt``, ``fast_v3_layout.json``, ``fast_v3_case.npz``: a one-block run of
   ``toner.fast.FastMuonT`` and ``FastAdamT`` (the ``toner.fast.v3`` checkpoint ``state_dict()`` returns after two
   steps -- in full for FastMuonT, keys and shapes for both -- and a sample of the third step's weight changes).
   ``capture_recomputed.npz``: the rows the reference's Triton capture kernels write (RMSNorm rows, SiLU-gated rows).
3. ``reference_gpu_timings.json``: CUDA-event times of the reference's own kernels on this device at the shapes of the
   24-layer d=2048 / mlp=5632 stack (packed SYRK, unpack + EMA, batched Newton-Schulz, split-precision products, and
   ``FastMuonT.begin() + step()`` ``gpu_ms``).

Fixtures go to this directory (or --out); the timing file goes to --out.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for cand in (os.environ.get("REFERENCE_SRC"), os.path.join(ROOT, "baseline", "_ref")):
    if cand and os.path.isdir(os.path.join(cand, "toner")):
        sys.path.insert(0, cand)
        break
else:
    raise SystemExit("the reference package `toner` was not found: set REFERENCE_SRC or install it under baseline/_ref")
sys.path.insert(0, ROOT)

import toner  # noqa: E402
from toner.linalg import newton_schulz  # noqa: E402

DEV = torch.device("cuda", 0)


def save(out_dir: str, name: str, **arrays) -> None:
    np.savez_compressed(os.path.join(out_dir, name), **{k: np.asarray(v.cpu() if torch.is_tensor(v) else v)
                                                        for k, v in arrays.items()})
    print("wrote", name, flush=True)


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-300))


# ------------------------------------------------------------------ 1. tpu-mode fixtures
def tpu_fixtures(out_dir: str) -> dict:
    from toner.fast import muon as fmuon

    torch.backends.cuda.matmul.allow_tf32 = False
    out, notes = {}, {}
    for tag, shape in (("square", (64, 64)), ("wide", (48, 96)), ("tall", (96, 48)), ("mid", (128, 256))):
        m = torch.randn(*shape, generator=torch.Generator().manual_seed(11))
        out[f"{tag}_in"] = m
        for steps in (1, 2, 3, 5, 10):
            out[f"{tag}_out{steps}"] = newton_schulz(m.to(DEV), steps, 1e-5, "tpu")
    # The reference's own spread: batched against per-matrix products of the same inputs (toner.fast.muon's
    # self-check prints this difference), and two modes against each other.
    u = torch.randn(4, 768, 768, generator=torch.Generator().manual_seed(0)).to(DEV)
    for steps in (1, 2, 3, 5, 10):
        batched = fmuon.newton_schulz_batched(u, steps, 1e-5, "tpu")
        single = torch.stack([fmuon.newton_schulz(u[i], steps, 1e-5, "tpu") for i in range(4)])
        f32 = torch.stack([fmuon.newton_schulz(u[i], steps, 1e-5, "f32") for i in range(4)])
        notes[f"batched_vs_single_{steps}"] = rel(batched, single)
        notes[f"tpu_vs_f32_{steps}"] = rel(single, f32)
    sv = torch.linalg.svdvals(fmuon.newton_schulz(u[0], 10, 1e-5, "tpu").double())
    notes["singular_values_10_steps"] = [float(sv.min()), float(sv.max())]
    out["self_noise_steps"] = np.array([1, 2, 3, 5, 10])
    out["self_noise_batched_vs_single"] = np.array([notes[f"batched_vs_single_{s}"] for s in (1, 2, 3, 5, 10)])
    out["self_noise_tpu_vs_f32"] = np.array([notes[f"tpu_vs_f32_{s}"] for s in (1, 2, 3, 5, 10)])
    save(out_dir, "newton_schulz_tpu.npz", **out)

    # MuonT general path in tpu mode, the same cases make_golden.py writes in f32 mode
    for tag, n_out, n_in, rows, steps, ns_steps in (("small", 40, 48, 256, 4, 10), ("tall", 96, 32, 128, 3, 10),
                                                    ("small2", 40, 48, 256, 4, 2)):
        torch.manual_seed(0)
        lin = torch.nn.Linear(n_in, n_out, bias=False)
        with torch.no_grad():
            lin.weight.normal_(0, 0.02)
        w0 = lin.weight.detach().clone()
        lin = lin.to(DEV)
        opt = toner.MuonT([lin.weight], lr=0.02, weight_decay=0.1, momentum=0.95, ns_mode="tpu", ns_steps=ns_steps)
        ws, xs, gs = [], [], []
        for s in range(steps):
            g = torch.Generator().manual_seed(1234 + s)
            x = torch.randn(rows, n_in, generator=g).to(torch.bfloat16).float()
            grad = torch.randn(n_out, n_in, generator=g) * 1e-3
            opt.update_statistics({lin.weight: (x.T @ x / rows).to(DEV)})
            lin.weight.grad = grad.to(DEV)
            opt.step()
            ws.append(lin.weight.detach().cpu().clone())
            xs.append(x)
            gs.append(grad)
        save(out_dir, f"muont_tpu_{tag}.npz", w0=w0, w=torch.stack(ws), x=torch.stack(xs), g=torch.stack(gs),
             ns_steps=np.array(ns_steps))
    return notes


# ------------------------------------------------------------------ 2. a checkpoint written by the reference
def _tiny_stack(hidden: int, mlp: int, layers: int):
    """Weights drawn on the CPU (so that any machine reproduces them from the seed), then moved to the device."""
    from toner_b200.synthetic import make_stack
    stack = make_stack("llama", layers, hidden, mlp, "cpu", seed=0)
    return [b.to(DEV) for b in stack]


def _matrices(stack):
    return [p for b in stack for p in b.parameters() if p.ndim == 2]


def _describe(obj):
    """Keys, shapes and dtypes of a checkpoint, without its values."""
    if torch.is_tensor(obj):
        return {"tensor": list(obj.shape), "dtype": str(obj.dtype).replace("torch.", "")}
    if isinstance(obj, dict):
        return {str(k): _describe(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_describe(v) for v in obj]
    return obj


def checkpoint_case(out_dir: str) -> dict:
    """One Llama-style block (hidden 256, MLP 256) through the reference's fast optimizers: three steps on seeded
    inputs.  Kept: the checkpoint FastMuonT returns after step 2 (in full), the layout (keys, shapes) of both
    optimizers' checkpoints, and a strided sample plus the norm of every matrix's third-step change."""
    from toner.fast import FastAdamT, FastMuonT, ProjectionBlock

    hidden, mlp, layers, seq, mb, acc = 256, 256, 1, 256, 2, 2
    notes, layout = {}, {}
    arrays = {"dims": np.array([hidden, mlp, layers, seq, mb, acc])}
    for kind in ("muont", "adamt"):
        stack = _tiny_stack(hidden, mlp, layers)
        blocks = [ProjectionBlock.from_module(b) for b in stack]
        if kind == "muont":
            opt = FastMuonT(blocks, 0.02, weight_decay=0.1, micro_batch_size=mb, sequence_length=seq,
                            accumulation_steps=acc, statistic_head=8, statistic_stride=4, ns_steps=2)
        else:
            opt = FastAdamT(blocks, 2e-3, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-4, micro_batch_size=mb,
                            sequence_length=seq, accumulation_steps=acc, statistic_head=8, statistic_stride=4)
        try:
            before = None
            for step in range(3):
                for i in range(acc):
                    x = torch.randn(mb, seq, hidden, generator=torch.Generator().manual_seed(500 + 10 * step + i))
                    with opt.capture_microbatch():
                        with torch.autocast("cuda", dtype=torch.bfloat16):
                            h = x.to(DEV)
                            for b in stack:
                                h = b(h)
                opt.begin()
                g = torch.Generator().manual_seed(900 + step)
                for p in _matrices(stack):
                    p.grad = (torch.randn(p.shape, generator=g) * 1e-3).to(DEV)
                opt.step()
                torch.cuda.synchronize()
                now = [p.detach().cpu().clone() for p in _matrices(stack)]
                if step == 1:
                    ckpt = opt.state_dict()
                    layout[kind] = _describe(ckpt)
                    if kind == "muont":
                        torch.save(ckpt, os.path.join(out_dir, "fast_v3_checkpoint_muont.pt"))
                        arrays["muont_w2"] = torch.stack([w.flatten() for w in now])
                if step == 2:
                    change = [b_ - a_ for a_, b_ in zip(before, now)]
                    arrays[f"{kind}_change3_sample"] = torch.stack([c[::4, ::4].flatten() for c in change])
                    arrays[f"{kind}_change3_norm"] = torch.stack([c.double().norm() for c in change])
                    arrays[f"{kind}_w3_norm"] = torch.stack([w.double().norm() for w in now])
                before = now
            notes[kind] = "ok"
        finally:
            opt.close()
    save(out_dir, "fast_v3_case.npz", **arrays)
    with open(os.path.join(out_dir, "fast_v3_layout.json"), "w") as f:
        json.dump(layout, f, indent=1)
    return notes


# ------------------------------------------------------------------ 2b. the reference's recomputed capture rows
def capture_fixture(out_dir: str) -> dict:
    """Rows written by the reference's recompute-and-capture operator (reproduce/marin/ops.py: capture_recomputed), whose
    RMSNorm and SiLU-gated rows exist only as Triton kernels.  The module is looked for as ``marin_ops`` beside the
    installed reference (a copy of that one file) or under REFERENCE_ROOT."""
    import importlib.util
    cands = [os.path.join(ROOT, "baseline", "_ref", "marin_ops.py")]
    if os.environ.get("REFERENCE_ROOT"):
        cands.insert(0, os.path.join(os.environ["REFERENCE_ROOT"], "reproduce", "marin", "ops.py"))
    path = next((c for c in cands if os.path.exists(c)), None)
    if path is None:
        raise FileNotFoundError("reproduce/marin/ops.py of the reference was not found")
    spec = importlib.util.spec_from_file_location("marin_ops", path)
    mops = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mops)

    def bits(t):
        return t.detach().cpu().contiguous().view(torch.int16).numpy()

    g = torch.Generator().manual_seed(5)
    batch, seq, hidden, mlp, head, stride, eps, layers = 3, 96, 64, 160, 8, 8, 1e-5, 2
    idx_list = list(range(head)) + list(range(head + 1, seq, stride))
    idx = torch.tensor(idx_list, dtype=torch.int64)
    P = idx.numel()
    out = {"idx": idx.numpy(), "eps": np.float32(eps), "dims": np.array([batch, seq, hidden, mlp, layers])}
    dev_in = {}
    for l in range(layers):
        for name, width, scale in (("x", hidden, 1.0), ("xmid", hidden, 3.0), ("attn", hidden, 0.5), ("g", mlp, 2.0),
                                   ("u", mlp, 1.0)):
            t = (torch.randn(batch, seq, width, generator=g) * scale).to(torch.bfloat16)
            out[f"{name}{l}"] = bits(t)
            dev_in[f"{name}{l}"] = t.to(DEV)
        for name in ("w1", "w2"):
            w = 1.0 + 0.1 * torch.randn(hidden, generator=g)
            out[f"{name}{l}"] = w.numpy()
            dev_in[f"{name}{l}"] = w.to(DEV)
    rows = batch * P
    bufs = []
    for l in range(layers):
        bufs += [torch.zeros(rows, hidden, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
        bufs.insert(len(bufs), torch.zeros(rows, mlp, device=DEV, dtype=torch.bfloat16))
    at = torch.arange(rows, device=DEV, dtype=torch.int64)
    col = lambda name: [dev_in[f"{name}{l}"] for l in range(layers)]
    mops.capture_recomputed(col("x"), col("attn"), col("xmid"), col("g"), col("u"), col("w1"), col("w2"), bufs, at,
                            idx.to(DEV), float(eps))
    torch.cuda.synchronize()
    for l in range(layers):
        for j, kind in enumerate(("attn", "o", "mlp", "down")):
            out[f"rows_{kind}{l}"] = bits(bufs[4 * l + j])
    save(out_dir, "capture_recomputed.npz", **out)
    return {"layers": layers, "rows": rows}


# ------------------------------------------------------------------ 3. the reference's kernels timed on this device
def timed(fn, warm: int = 3, reps: int = 10) -> dict:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return {"min_ms": round(times[0], 3), "median_ms": round(times[len(times) // 2], 3)}


def kernel_timings(layers: int, deadline: float) -> dict:
    from toner.fast import roots, syrk
    from toner.fast import muon as fmuon

    res = {"device": torch.cuda.get_device_name(0), "torch": torch.__version__}
    try:
        import triton
        res["triton"] = triton.__version__
    except Exception as exc:  # pragma: no cover
        res["triton"] = f"unavailable: {exc}"
    rows = 256 * 286

    def leg(name, fn):
        if time.time() > deadline:
            res[name] = {"skipped": "out of time"}
            return
        try:
            res[name] = fn()
        except Exception as exc:
            res[name] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
            traceback.print_exc()
        print(name, res[name], flush=True)
        torch.cuda.empty_cache()

    def syrk_leg(k, n):
        def run():
            xs_all = torch.randn(k, rows, n, device=DEV, dtype=torch.bfloat16)
            xs = list(xs_all.unbind(0))
            offs = syrk.list_offsets(xs)
            out = torch.empty(k, n * (n + 1) // 2, device=DEV, dtype=torch.float32)
            t = timed(lambda: syrk.syrk_list_packed(xs, offs, out), warm=2, reps=5)
            t["tflops_triangle"] = round(k * rows * n * (n + 1) / t["min_ms"] / 1e9, 1)
            C = torch.zeros(k, n, n, device=DEV)
            t2 = timed(lambda: syrk.unpack_ema_(out, C, 0.95, 0.05 / rows), warm=2, reps=5)
            t["unpack_ema"] = dict(t2, gbs=round(4 * k * (n * (n + 1) / 2 + 2 * n * n) / t2["min_ms"] / 1e6, 1))
            return t
        return run

    leg(f"syrk_list_packed k={3 * layers} n=2048 rows={rows}", syrk_leg(3 * layers, 2048))
    leg(f"syrk_list_packed k={layers} n=5632 rows={rows}", syrk_leg(layers, 5632))

    def ns_leg(b, m, n):
        def run():
            u = torch.randn(b, m, n, device=DEV)
            t = timed(lambda: fmuon.newton_schulz_batched(u, 10, 1e-5, "tpu"), warm=2, reps=5)
            a, bb = min(m, n), max(m, n)
            t["tflops_dense"] = round(b * 10 * (4 * a * a * bb + 2 * a ** 3) / t["min_ms"] / 1e9, 1)
            return t
        return run

    leg(f"newton_schulz_batched {layers}x2048x2048", ns_leg(layers, 2048, 2048))
    leg(f"newton_schulz_batched {layers}x5632x2048", ns_leg(layers, 5632, 2048))
    leg(f"newton_schulz_batched {layers}x2048x5632", ns_leg(layers, 2048, 5632))

    def apply_leg(b, m, n):
        def run():
            a = torch.randn(b, m, n, device=DEV)
            r = torch.randn(b, n, n, device=DEV)
            r = r @ r.transpose(-1, -2) / n
            r2 = roots.rows_lo(r)
            t = timed(lambda: roots.apply16(a, r2), warm=2, reps=5)
            t["tflops_single_pass"] = round(b * 2 * m * n * n / t["min_ms"] / 1e9, 1)
            return t
        return run

    leg(f"apply16 {layers}x2048x2048", apply_leg(layers, 2048, 2048))
    leg(f"apply16 {layers}x2048x5632", apply_leg(layers, 2048, 5632))

    def engine_leg(nl, steps, inline):
        def run():
            from toner.fast import FastMuonT, ProjectionBlock
            from toner_b200.synthetic import fill_rows, make_stack
            stack = make_stack("llama", nl, 2048, 5632, DEV, seed=0)
            blocks = [ProjectionBlock.from_module(b) for b in stack]
            opt = FastMuonT(blocks, 0.02, weight_decay=0.1, momentum=0.95, micro_batch_size=1, sequence_length=4096,
                            accumulation_steps=256, root_inline_steps=inline)
            try:
                core = opt._core
                # the engine seam: rows straight into the row buffers, gradients into .grad, begin() + step()
                for bi, buf in enumerate(opt._buffers):
                    for j, name in enumerate(("input_rows_attn", "input_rows_o", "input_rows_mlp", "input_rows_down")):
                        fill_rows(getattr(buf, name).unsqueeze(0), seed=1 + 4 * bi + j, mean_seed=1000 + (j == 3))
                gen = torch.Generator(device=DEV).manual_seed(99)
                for p in _matrices(stack):
                    p.grad = torch.randn(p.shape, device=DEV, generator=gen) * 1e-3
                hist = []
                for s in range(steps):
                    if time.time() > deadline:
                        break
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    e0.record()
                    core.begin()
                    core.step()
                    e1.record()
                    torch.cuda.synchronize()
                    hist.append({"step": s, "ms": round(e0.elapsed_time(e1), 2),
                                 "gpu_ms": {k: round(float(v), 2) for k, v in dict(getattr(core, "gpu_ms", {}) or {}).items()}})
                    print("reference engine step", hist[-1], flush=True)
                d = opt.diagnostics
                return {"layers": nl, "root_inline_steps": inline, "steps": hist,
                        "fallbacks": d.get("fallbacks"), "extra_iterations": d.get("extra_iterations")}
            finally:
                opt.close()
        return run

    leg(f"FastMuonT begin+step, {layers} layers", engine_leg(layers, 10, 2))
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--timing-out", default=None)
    ap.add_argument("--skip-timing", action="store_true")
    ap.add_argument("--skip-fixtures", action="store_true")
    ap.add_argument("--only", default=None, help="run one fixture function only (tpu_fixtures, checkpoint_case, capture_fixture)")
    ap.add_argument("--layers", type=int, default=6, help="layers of the 2048 / 5632 stack the timing legs cover")
    ap.add_argument("--budget", type=float, default=600.0, help="seconds after which remaining timing legs are skipped")
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    torch.cuda.set_device(0)
    report = {}
    if not args.skip_fixtures:
        for name, fn in (("tpu_fixtures", tpu_fixtures), ("checkpoint_case", checkpoint_case),
                         ("capture_fixture", capture_fixture)):
            if args.only and name != args.only:
                continue
            try:
                report[name] = fn(args.out)
            except Exception as exc:
                traceback.print_exc()
                report[name] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    if not args.skip_timing:
        report["timings"] = kernel_timings(args.layers, time.time() + args.budget)
    path = os.path.join(args.timing_out or args.out, "reference_gpu_timings.json")
    with open(path, "w") as f:
        json.dump(report, f, indent=1)
    print(json.dumps(report)[:4000])


if __name__ == "__main__":
    main()
