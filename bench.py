"""Optimizer-step benchmark: a full MuonT step of the 24-layer d=2048 Llama-style block stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = statistics (SYRK over the sampled BF16 rows of 256 x 4096 tokens, fused EMA) + inverse-root
factors of all 96 statistics + momentum, preconditioning products, Newton-Schulz and the weight update of
all 168 projection matrices.  Inputs are synthetic (seeded activation-like rows, Gaussian gradients,
random-init weights).  The token count is fixed as N grows (strong scaling): every rank holds 1/N of the
rows and owns 1/N of the layers.

Prints one JSON line (rank 0).  `value` is the step time with rows and gradients resident in HBM; `e2e`
repeats the measurement with the step's rows and gradients copied from pinned host memory inside the timed
region and a checksum read back.  `--impl reference` times the CPU restatement of the reference's general
path (oracle/) on the host cores for one of the 24 layers and extrapolates.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

LAYERS, HIDDEN, MLP, SEQUENCES, SEQ_LEN = 24, 2048, 5632, 256, 4096
HEAD, STRIDE = 32, 16
LR, WD, MOMENTUM = 0.02, 0.1, 0.95


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops": p["bf16_tflops_sustained"], "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int) -> None:
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().split(",")
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
                for name, val in zip(names, out[2:]):
                    if val.strip().lower().startswith("active"):
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# DRAM bytes per launch of the dominant kernel from the ncu capture summarised in profiles/gemm_tcgen05_kernel_ncu.md:
# the factor engine's M-update product moved 564 MB (dram__bytes_read + write) for 8 statistics of 2048^2; traffic is
# proportional to the operand size (every operand byte is read from DRAM once), so a launch over k statistics of
# width n moves 564e6 * k n^2 / (8 * 2048^2).
def roots_traffic(k: int, n: int) -> int:
    return int(564e6 * k * n * n / (8 * 2048 * 2048))


def tri_fraction(n: int, bm: int = 128, bn: int = 256) -> float:
    """Share of the bm x bn result tiles that meet the upper triangle of an n x n symmetric product."""
    tm, tn = -(-n // bm), -(-n // bn)
    return sum(max(0, tn - (i * bm) // bn) for i in range(tm)) / (tm * tn)


def workload_config(layers: int, hidden: int, mlp: int, sequences: int) -> dict:
    rows = sequences * len(list(range(HEAD)) + list(range(HEAD + 1, SEQ_LEN, STRIDE)))
    return {"workload": f"MuonT step, {layers}-layer Llama-style stack d={hidden} mlp={mlp}, "
                        f"{sequences}x{SEQ_LEN} tokens per update ({rows} sampled rows)"}


def sampled_positions() -> int:
    return len(list(range(HEAD)) + list(range(HEAD + 1, SEQ_LEN, STRIDE)))


def step_flops(layers: int, hidden: int, mlp: int, rows_total: int, root_gemms_d: int, root_gemms_f: int, ns_steps: int = 10,
               products: int = 3):
    """Algorithmic work of one whole-job step (single-pass dense counts: 2 n^3 per product, rows n (n+1) for the triangle of a Gram)."""
    syrk = rows_total * (3 * layers * hidden * (hidden + 1) + layers * mlp * (mlp + 1))
    shapes = [(hidden, hidden)] * 4 + [(mlp, hidden)] * 2 + [(hidden, mlp)]
    ns = precond = 0
    for m, n in shapes:
        a, b = min(m, n), max(m, n)
        ns += layers * ns_steps * (4 * a * a * b + 2 * a ** 3)
        precond += layers * products * 2 * m * n * n
    roots = 3 * layers * root_gemms_d * 2 * hidden ** 3 + layers * root_gemms_f * 2 * mlp ** 3
    return {"syrk": syrk, "ns": ns, "precond": precond, "roots": roots}


def run_ours(args) -> None:
    import torch.distributed as dist

    from toner_b200 import ops
    from toner_b200.fast import FastAdamT, FastMuonT, ProjectionBlock
    from toner_b200.synthetic import fill_rows, make_stack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    layers, hidden, mlp, sequences = args.layers, args.hidden, args.mlp, args.sequences
    if sequences % world or layers % world:
        raise SystemExit("sequences and layers must be multiples of the number of ranks")
    P = sampled_positions()
    micro = 1
    acc = sequences // world
    stack = make_stack("llama", layers, hidden, mlp, dev, seed=0)
    blocks = [ProjectionBlock.from_module(b) for b in stack]
    if args.optimizer == "adamt":   # AdamT: factors A^-1/4 only, five right-products per matrix, no Newton-Schulz
        opt = FastAdamT(blocks, 2e-3, weight_decay=WD, betas=(0.9, 0.95), micro_batch_size=micro,
                        sequence_length=SEQ_LEN, accumulation_steps=acc)
    else:
        opt = FastMuonT(blocks, LR, weight_decay=WD, momentum=MOMENTUM, micro_batch_size=micro,
                        sequence_length=SEQ_LEN, accumulation_steps=acc)
    core = opt._core
    if args.sm_reserve is not None and world > 1:
        core.sm_reserve = int(args.sm_reserve)
    # Engine-level seam (what the reference's second trainer uses): the sampled rows of this rank's tokens
    # are written straight into the row buffers, gradients into .grad, then begin() and step().
    for gi, g in enumerate(core.groups.values()):
        fill_rows(g.rows_buf, seed=1 + rank * 7 + gi, mean_seed=1000 + gi)   # every rank's tokens share the model's mean activation
    gen = torch.Generator(device=dev).manual_seed(99)   # gradients are replicated (already synchronised)
    for p in core.params:
        p.grad = torch.randn(p.shape, device=dev, generator=gen) * 1e-3
    local_rows = core.groups["d"].rows
    assert local_rows == acc * micro * P

    def one_step():
        core.begin()
        core.step()

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            tms = torch.tensor([ms], device=dev)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ms = float(tms.item())
        return ms

    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()
    launches0 = ops.launch_count()
    phases = []
    with ClockSampler(local) as clocks:
        ms = timed(lambda: (one_step(), phases.append(dict(core.gpu_ms))), args.steps)
    launches = (ops.launch_count() - launches0) // args.steps
    ops.assert_healthy()

    # ---- end to end: this step's rows and gradients come from pinned host memory, a checksum goes back
    d, f = core.groups["d"], core.groups["f"]
    host_rows_d = torch.empty(3, local_rows, hidden, dtype=torch.bfloat16).pin_memory()
    host_rows_f = torch.empty(local_rows, mlp, dtype=torch.bfloat16).pin_memory()
    host_rows_d.copy_(d.rows_buf[:3].cpu())
    host_rows_f.copy_(f.rows_buf[0].cpu())
    roles = list(core.roles.values())
    host_grads = [torch.randn(info["all"][0].shape).mul_(1e-3).pin_memory() for info in roles]
    checksum = torch.zeros(1, dtype=torch.float32).pin_memory()
    # a rank reads the gradients of the layers it owns only (the other layers' changes arrive by all-gather)
    own_lo = sum(core.layer_counts[:rank])
    own_layers = range(own_lo, own_lo + core.per_layers)
    h2d = world * (layers * (host_rows_d.numel() * 2 + host_rows_f.numel() * 2) +
                   len(own_layers) * sum(g.numel() * 4 for g in host_grads))        # all ranks together

    # The copies run on their own stream in the order the step consumes them -- the wide (MLP) statistics first, whose
    # factors are most of the step, then the hidden-width ones, then the gradients -- four layers per event, and
    # begin(ready=...) lets each slice's SYRK and each group's factors start as soon as their rows have landed.
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    per_event = 4

    def e2e_step():
        ready = []
        copy_stream.wait_stream(main_stream)      # the previous step has read the rows and gradients
        with torch.cuda.stream(copy_stream):
            for lo in range(0, layers, per_event):
                hi = min(layers, lo + per_event)
                for i in range(lo, hi):
                    f.rows_buf[i].copy_(host_rows_f, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
                ready.append(("f", lo, hi, ev))
            for lo in range(0, layers, per_event):
                hi = min(layers, lo + per_event)
                for i in range(lo, hi):
                    d.rows_buf[3 * i: 3 * i + 3].copy_(host_rows_d, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
                ready.append(("d", 3 * lo, 3 * hi, ev))
            for i in own_layers:
                for info, hg in zip(roles, host_grads):
                    info["all"][i].grad.copy_(hg, non_blocking=True)
            grads_in = torch.cuda.Event()
            grads_in.record(copy_stream)
        core.begin(ready=ready)
        main_stream.wait_event(grads_in)
        core.step()
        checksum.copy_(roles[0]["all"][0][0, :1], non_blocking=True)

    e2e_ms = None
    if not args.no_e2e:
        e2e_step()
        e2e_ms = timed(e2e_step, max(1, min(args.steps, 3)))
        ops.assert_healthy()

    check = check_results(core, world, dev)
    if rank == 0:
        pk = peaks()
        # products per statistic: X T and T^2 T^4 T^8 T^8 M per Newton step (no X product in the first, no M update
        # in the last), two squarings for A^-1/2 -- each three FP16 plane passes -- plus the single-pass products of
        # the finishing series (its order - 1); the step count follows each group's spectrum bound
        fd, ff = core.groups["d"].factors, core.groups["f"].factors
        it_d, it_f = fd.iterations, ff.iterations
        single_d, single_f = fd.finish_order - 1, ff.finish_order - 1
        if args.optimizer == "adamt":   # p = 4: X T, T^2, T^4, T^4 M per step, no squarings afterwards
            split_d, split_f = (it_d - 1) * 4, (it_f - 1) * 4
            fl = step_flops(layers, hidden, mlp, local_rows * world, split_d + single_d, split_f + single_f, ns_steps=0,
                            products=5)
        else:
            split_d, split_f = (it_d - 1) * 5 + 2, (it_f - 1) * 5 + 2
            fl = step_flops(layers, hidden, mlp, local_rows * world, split_d + single_d, split_f + single_f)
        ph = phases[-1] if phases and phases[-1] else {}
        per_phase = {}
        for name, work in (("stats", fl["syrk"]), ("roots", fl["roots"]), ("update", fl["ns"] + fl["precond"])):
            if name in ph and ph[name] > 0:
                # phases are per rank; the whole-job work is divided over `world` ranks
                per_phase[name] = {"ms": round(ph[name], 3), "tflops_per_gpu": round(work / world / ph[name] / 1e9, 1)}
        if "exchange" in ph:
            per_phase["update"]["exchange_ms"] = round(ph["exchange"], 3)
        top = max(per_phase, key=lambda k: per_phase[k]["ms"]) if per_phase else None
        roof = None
        if top:
            a = per_phase[top]["tflops_per_gpu"]
            roof = {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "phase": top, "achieved": a, "peak": pk["tflops"],
                    "unit": "TFLOP/s", "frac": round(a / pk["tflops"], 4), "traffic": (roots_traffic(layers // world, mlp) if top == "roots" else None),
                    "peak_source": pk["source"] + " (sustained cuBLAS BF16: the kernel runs inside a long step)",
                    "note": "achieved = algorithmic single-pass flops of the phase / its CUDA-event time on the launching "
                            "stream; the phase is >97% this kernel by ncu share"}
            if top == "roots":
                # what the tensor cores execute: three FP16 plane products per accumulator, on the 128x256 tiles
                # that meet the upper triangle (fractions 0.5625 at n=2048, 0.523 at n=5632)
                ex = (3 * layers * (3 * split_d + single_d) * 2 * hidden ** 3 * tri_fraction(hidden, 256) +
                      layers * (3 * split_f + single_f) * 2 * mlp ** 3 * tri_fraction(mlp, 256)) / world / ph[top] / 1e9
                roof["newton_steps"] = {"hidden": it_d, "mlp": it_f}
                roof["finish_order"] = {"hidden": fd.finish_order, "mlp": ff.finish_order}
                roof["executed"] = round(ex, 1)
                roof["frac_executed"] = round(ex / pk["tflops"], 4)
        line = {
            "metric": f"{args.optimizer}_optimizer_step_ms", "value": round(ms, 3), "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 operands / fp16 hi-lo splits, fp32 accumulate",
            "data": "synthetic",
            "config": dict(workload_config(layers, hidden, mlp, sequences), parallelism=f"layer-sharded x{world}",
                           l2="inputs larger than L2",
                           entry="engine seam: rows resident in the row buffers, begin()+step()"),
            "e2e": ({"value": round(e2e_ms, 3), "unit": "ms", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4}
                    if e2e_ms is not None else None),
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": roof,
            "phases": per_phase,
            "algorithmic_flops": fl,
            "fallbacks": core.fallbacks,
            "check": check,
        }
        mhz = line["clocks"]["sm_mhz"]
        if mhz:   # time x clock: comparable between runs whose power-capped clocks differ
            line["mhz_ms"] = round(ms * mhz, 1)
            for ph in per_phase.values():
                ph["mhz_ms"] = round(ph["ms"] * mhz, 1)
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(args, sample_rows=2048)
        print(json.dumps(line), flush=True)
    opt.close()
    if world > 1:
        dist.destroy_process_group()


def check_results(core, world: int, dev) -> dict:
    """Results, not timings: (1) every rank must hold bit-identical weights after the exchange (FP64 sums of every
    matrix and of its square, compared through MIN / MAX all-reduces); (2) on every rank the factors of one owned
    hidden-width statistic -- they went through SYRK, reduce-scatter, EMA and the Newton engine -- against an FP64
    eigendecomposition of that rank's EMA on the host (src/toner/linalg.py:54-89 in double precision), worst rank
    reported.  Runs after the timed regions."""
    import torch.distributed as dist
    sums = torch.stack([torch.stack([p.detach().double().sum(), p.detach().double().square().sum()]) for p in core.params])
    agree = True
    if world > 1:
        lo, hi = sums.clone(), sums.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        agree = bool(torch.equal(lo, hi))
    f = core.groups["d"].factors
    torch.cuda.synchronize()
    c = f.ema[0].double().cpu()
    lam, vec = torch.linalg.eigh(0.5 * (c + c.T))
    lam = lam.clamp_min(0)
    unit = lam / lam.mean().clamp_min(1e-30) + f.damping
    errs = []
    for root, power in ((f.root_lo, 1.0 / f.p), (f.root_hi, float(f.q) / f.p)):
        if root is None:
            continue
        want = (vec * unit.pow(-power)) @ vec.T
        errs.append(float((root[0].double().cpu() - want).norm() / want.norm()))
    err = torch.tensor([max(errs)], device=dev)
    if world > 1:
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
    finite = bool(torch.isfinite(sums).all())
    return {"ranks_agree": agree, "weights_finite": finite, "factor_err": float(f"{float(err.item()):.3e}"),
            "factor_err_bound": 2e-3, "ok": bool(agree and finite and float(err.item()) <= 2e-3)}


def cpu_baseline(args, sample_rows: int = 2048):
    """The CPU restatement of the reference's general path (oracle/) for ONE layer, extrapolated to the stack.

    Gram products are timed on `sample_rows` rows and scaled to the full row count; the optimizer step
    (eigh factors, FP32 Newton-Schulz, update) is timed in full for the layer's seven matrices."""
    from oracle import toner_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    layers, hidden, mlp = args.layers, args.hidden, args.mlp
    rows_total = args.sequences * sampled_positions()
    g = torch.Generator().manual_seed(0)
    t_gram = 0.0
    stats = {}
    for kind, n in (("attn", hidden), ("o", hidden), ("mlp", hidden), ("down", mlp)):
        x = torch.randn(sample_rows, n, generator=g).to(torch.bfloat16)
        t0 = time.perf_counter()
        gram = orc.gram(x)
        t_gram += (time.perf_counter() - t0) * (rows_total / sample_rows)
        stats[kind] = gram / sample_rows
    shapes = dict(q=(hidden, hidden, "attn"), k=(hidden, hidden, "attn"), v=(hidden, hidden, "attn"),
                  o=(hidden, hidden, "o"), gate=(mlp, hidden, "mlp"), up=(mlp, hidden, "mlp"), down=(hidden, mlp, "down"))
    t_step = 0.0
    for role, (m, n, kind) in shapes.items():
        w = torch.randn(m, n, generator=g) * 0.02
        grad = torch.randn(m, n, generator=g) * 1e-3
        adam = getattr(args, "optimizer", "muont") == "adamt"
        st = orc.AdamTState() if adam else orc.MuonTState()
        st.ema, st.weight = orc.ema_update(None, 0.0, stats[kind], MOMENTUM)
        t0 = time.perf_counter()
        if adam:
            orc.adamt_step(w, grad, st, lr=2e-3, weight_decay=WD, betas=(0.9, 0.95), eps=1e-15)
        else:
            orc.muont_step(w, grad, st, lr=LR, weight_decay=WD, momentum=MOMENTUM, ns_mode="f32")
        t_step += time.perf_counter() - t0
    per_layer_ms = (t_gram + t_step) * 1e3
    return {"value": round(per_layer_ms * layers, 1), "unit": "ms", "cores": cores, "kind": "port",
            "sample": f"1 of {layers} layers timed (7 matrices: eigh factors, FP32 Newton-Schulz, update) and "
                      f"Gram products on {sample_rows} of {rows_total} rows, both extrapolated linearly"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    base = None
    for _ in range(max(1, min(args.steps, 2))):
        base = cpu_baseline(args)
        times.append(base["value"])
    ms = min(times)
    base["value"] = ms
    line = {"impl": "reference", "metric": f"{args.optimizer}_optimizer_step_ms", "value": ms, "unit": "ms",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": dict(workload_config(args.layers, args.hidden, args.mlp, args.sequences),
                           entry="reference general path (eigh factors, FP32 Newton-Schulz) restated on CPU, host cores"),
            "cpu_baseline": base,
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--hidden", type=int, default=HIDDEN)
    ap.add_argument("--mlp", type=int, default=MLP)
    ap.add_argument("--sequences", type=int, default=SEQUENCES)
    ap.add_argument("--optimizer", default="muont", choices=["muont", "adamt"], help="FastMuonT (headline) or FastAdamT")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--sm-reserve", type=int, default=None,
                    help="SMs the GEMMs leave to NCCL while a collective overlaps them (several ranks; default: the engine's)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (for profiler runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
