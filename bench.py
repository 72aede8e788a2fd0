"""Optimizer-step benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2|3|4] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

--config 4 (default, the headline): a full FastMuonT step of the 24-layer d=2048 / mlp=5632 Llama-style block stack,
            256 x 4096 tokens per update (73 216 sampled rows per statistic), layer-sharded over N ranks.
--config 3: FastMuonT with the NanoGPTBlock adapter on the 12-layer d=768 / mlp=3072 stack, 4 x 16 x 1024 tokens.
--config 2: AdamT + ActivationStatistics (the general interface) on the same 12-layer stack, 8 x 1024 tokens.

One "step" = statistics (SYRK over the sampled BF16 rows, EMA) + inverse-root factors of every statistic + momentum /
moments, preconditioning products, Newton-Schulz (MuonT) and the weight update of every projection matrix.  Inputs are
synthetic (seeded activation-like rows, Gaussian gradients, random-init weights); `--spectrum` chooses the covariance
spectrum of the rows.  The token count is fixed as N grows (strong scaling): every rank holds 1/N of the rows and owns
1/N of the layers.

Prints one JSON line (rank 0).  `value` is the step time with rows and gradients resident in HBM; `e2e` repeats the
measurement with the step's rows and gradients copied from pinned host memory inside the timed region and a checksum
read back; `value_by_spectrum` repeats `value` on harder spectra; `capture` times the forward hooks that fill the row
buffers; `check` compares results (ranks against each other, factors against an FP64 eigendecomposition).
`--impl reference` times the CPU restatement of the reference's general path (oracle/) on the host cores for one layer
and extrapolates.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from dataclasses import dataclass

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

HEAD, STRIDE = 32, 16
LR, WD, MOMENTUM = 0.02, 0.1, 0.95


@dataclass(frozen=True)
class Workload:
    config: int
    layout: str        # "llama": q k v o gate up down;  "nanogpt": q k v attn_proj fc mlp_proj
    layers: int
    hidden: int
    mlp: int
    sequences: int     # per update, all ranks together
    seq_len: int
    optimizer: str     # muont | adamt
    entry: str

    @property
    def positions(self) -> int:
        return len(list(range(HEAD)) + list(range(HEAD + 1, self.seq_len, STRIDE)))

    @property
    def rows(self) -> int:
        return self.sequences * self.positions

    @property
    def shapes(self):
        h, m = self.hidden, self.mlp
        wide = [(m, h)] * (2 if self.layout == "llama" else 1)
        return [(h, h)] * 4 + wide + [(h, m)]

    def describe(self) -> str:
        names = {"muont": "MuonT", "adamt": "AdamT"}
        stack = "Llama-style" if self.layout == "llama" else "modded-nanoGPT"
        return (f"{names[self.optimizer]} step, {self.layers}-layer {stack} stack d={self.hidden} mlp={self.mlp}, "
                f"{self.sequences}x{self.seq_len} tokens per update ({self.rows} sampled rows)")


def workload_of(args) -> Workload:
    base = {
        4: Workload(4, "llama", 24, 2048, 5632, 256, 4096, "muont", "engine seam: rows resident in the row buffers, begin()+step()"),
        3: Workload(3, "nanogpt", 12, 768, 3072, 64, 1024, "muont", "engine seam: rows resident in the row buffers, begin()+step()"),
        2: Workload(2, "nanogpt", 12, 768, 3072, 8, 1024, "adamt", "ActivationStatistics.capture() forward + commit() + AdamT.step()"),
    }[args.config]
    return Workload(base.config, base.layout, args.layers or base.layers, args.hidden or base.hidden, args.mlp or base.mlp,
                    args.sequences or base.sequences, base.seq_len, args.optimizer or base.optimizer, base.entry)


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


# The update phase's largest launch is the Newton-Schulz x-update of the widest role group (x <- a x + B x: reads B and x
# in BF16 and x in FP32, writes x in FP32 and BF16).  Its capture on 24 matrices of 2048^2 (section 5 of the same
# summary) moved 821 + 553 MB; the traffic is proportional to the number of elements of x.
def update_traffic(count: int, m: int, n: int) -> int:
    return int(1374e6 * count * m * n / (24 * 2048 * 2048))


def tri_fraction(n: int, bm: int = 128, bn: int = 256) -> float:
    """Share of the bm x bn result tiles that meet the upper triangle of an n x n symmetric product."""
    tm, tn = -(-n // bm), -(-n // bn)
    return sum(max(0, tn - (i * bm) // bn) for i in range(tm)) / (tm * tn)


def step_flops(w: Workload, root_gemms_d: int, root_gemms_f: int, ns_steps: int = 10, products: int = 3):
    """Algorithmic work of one whole-job step (single-pass dense counts: 2 n^3 per product, rows n (n+1) for the triangle
    of a Gram)."""
    L, h, m = w.layers, w.hidden, w.mlp
    syrk = w.rows * (3 * L * h * (h + 1) + L * m * (m + 1))
    ns = precond = 0
    for rows_, cols_ in w.shapes:
        a, b = min(rows_, cols_), max(rows_, cols_)
        ns += L * ns_steps * (4 * a * a * b + 2 * a ** 3)
        precond += L * products * 2 * rows_ * cols_ * cols_
    roots = 3 * L * root_gemms_d * 2 * h ** 3 + L * root_gemms_f * 2 * m ** 3
    return {"syrk": syrk, "ns": ns, "precond": precond, "roots": roots}


def product_counts(core, optimizer: str):
    """Products per statistic of the factor engine as it ran last: X T and the log2(p) + 1 products of the M update per
    Newton step (no X product in the first step, no M update in the last), the squarings for the stronger power --
    each three FP16 plane passes -- plus the single-pass products of the finishing series (its order - 1)."""
    out = {}
    for name, g in core.groups.items():
        f = g.factors
        log2p = f.p.bit_length() - 1
        split = (f.iterations - 1) * (log2p + 2) + (f.q.bit_length() - 1)
        out[name] = {"newton_steps": f.iterations, "finish_order": f.finish_order, "split": split,
                     "single": f.finish_order - 1}
    return out


def timed(fn, steps, world, dev):
    import torch.distributed as dist
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


def run_fast(args, w: Workload) -> None:
    """Configs 3 and 4: the layer-sharded engine behind FastMuonT / FastAdamT."""
    import torch.distributed as dist

    from toner_b200 import ops
    from toner_b200.fast import FastAdamT, FastMuonT, NanoGPTBlock, ProjectionBlock
    from toner_b200.synthetic import fill_rows_spectrum, make_stack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if w.sequences % world or w.layers % world:
        raise SystemExit("sequences and layers must be multiples of the number of ranks")
    micro = 1
    acc = w.sequences // world
    stack = make_stack(w.layout, w.layers, w.hidden, w.mlp, dev, seed=0)
    wrap = ProjectionBlock if w.layout == "llama" else NanoGPTBlock
    blocks = [wrap.from_module(b) for b in stack]
    if w.optimizer == "adamt":   # AdamT: factors A^-1/4 only, five right-products per matrix, no Newton-Schulz
        opt = FastAdamT(blocks, 2e-3, weight_decay=WD, betas=(0.9, 0.95), micro_batch_size=micro,
                        sequence_length=w.seq_len, accumulation_steps=acc)
    else:
        opt = FastMuonT(blocks, LR, weight_decay=WD, momentum=MOMENTUM, micro_batch_size=micro,
                        sequence_length=w.seq_len, accumulation_steps=acc)
    core = opt._core
    if args.sm_reserve is not None and world > 1:
        core.sm_reserve = int(args.sm_reserve)
    if args.single_deflation:
        for g in core.groups.values():
            g.factors.block_deflation = False
    gen = torch.Generator(device=dev).manual_seed(99)   # gradients are replicated (already synchronised)
    for p in core.params:
        p.grad = torch.randn(p.shape, device=dev, generator=gen) * 1e-3
    local_rows = core.groups["d"].rows
    assert local_rows == acc * micro * w.positions

    def load_rows(spectrum: str) -> None:
        """Engine-level seam (what the reference's second trainer uses): the sampled rows of this rank's tokens are
        written straight into the row buffers.  Every rank's tokens share the model's population statistics."""
        for gi, g in enumerate(core.groups.values()):
            fill_rows_spectrum(g.rows_buf, seed=1 + rank * 7 + gi, spectrum=spectrum, mean_seed=1000 + gi)
            g.factors.ema.zero_()
            g.factors.statistics_replaced()
        core.weight = 0.0

    def one_step():
        core.begin()
        core.step()

    def measure(spectrum: str, warmup: int, steps: int, sampler=None):
        load_rows(spectrum)
        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        repairs0, failures0, fallbacks0 = core.extra, core.bound_failures, core.fallbacks
        phases = []
        launches0 = ops.launch_count()
        if sampler is not None:
            with sampler:
                ms = timed(lambda: (one_step(), phases.append(dict(core.gpu_ms))), steps, world, dev)
        else:
            ms = timed(lambda: (one_step(), phases.append(dict(core.gpu_ms))), steps, world, dev)
        launches = (ops.launch_count() - launches0) // steps
        ops.assert_healthy()
        counts = product_counts(core, w.optimizer)
        return {"ms": ms, "phases": phases[-1] if phases and phases[-1] else {}, "launches": launches, "counts": counts,
                "repairs": core.extra - repairs0, "bound_failures": core.bound_failures - failures0,
                "fallbacks": core.fallbacks - fallbacks0}

    clocks = ClockSampler(local)
    head = measure(args.spectrum, args.warmup, args.steps, clocks)
    ms, launches = head["ms"], head["launches"]

    # ---- end to end: this step's rows and gradients come from pinned host memory, a checksum goes back
    d, f = core.groups["d"], core.groups["f"]
    layers, hidden, mlp = w.layers, w.hidden, w.mlp
    e2e_ms, h2d = None, 0
    if not args.no_e2e:
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
        # The copies run on their own stream in the order the step consumes them -- the wide (MLP) statistics first,
        # whose factors are most of the step, then the hidden-width ones, then the gradients -- four layers per event,
        # and begin(ready=...) lets each slice's SYRK and each group's factors start as soon as their rows have landed.
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

        e2e_step()
        e2e_ms = timed(e2e_step, max(1, min(args.steps, 3)), world, dev)
        ops.assert_healthy()
        del host_rows_d, host_rows_f

    check = check_results(core, world, dev)

    # ---- the same step on harder spectra (statistics reset, a few steps for the engine's tracking to settle)
    by_spectrum = {}
    extra = [s for s in (args.extra_spectra.split(",") if args.extra_spectra else []) if s and s != args.spectrum]
    for spectrum in extra:
        r = measure(spectrum, max(5, args.warmup), max(1, min(args.steps, 2)))   # the deflation block widens over a few steps
        by_spectrum[spectrum] = {
            "ms": round(r["ms"], 3), "phases_ms": {k: round(v, 2) for k, v in r["phases"].items()},
            "newton_steps": {k: c["newton_steps"] for k, c in r["counts"].items()},
            "finish_order": {k: c["finish_order"] for k, c in r["counts"].items()},
            "repairs": r["repairs"], "bound_failures": r["bound_failures"], "fallbacks": r["fallbacks"]}

    # ---- row capture: one micro-batch of the forward through capture_microbatch() (hooks -> toner_gather_rows)
    capture = None
    if not args.no_capture:
        x = torch.randn(micro, w.seq_len, hidden, device=dev).to(torch.bfloat16)

        def forward():
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                hcur = x
                for b in stack:
                    hcur = b(hcur)

        def captured():
            with opt.capture_microbatch():
                forward()
            opt._microbatches = 0     # the same micro-batch slot again: nothing here is followed by a step

        for fn in (forward, captured):
            for _ in range(2):
                fn()
        plain = timed(forward, 5, 1, dev)
        with_hooks = timed(captured, 5, 1, dev)
        capture = {"forward_ms": round(plain, 3), "forward_with_capture_ms": round(with_hooks, 3),
                   "capture_ms_per_microbatch": round(with_hooks - plain, 3), "microbatches_per_step": acc,
                   "capture_ms_per_step": round((with_hooks - plain) * acc, 2),
                   "note": "stand-in forward (projections only); the difference is the hooks' row capture"}

    if rank == 0:
        pk = peaks()
        cd, cf = head["counts"]["d"], head["counts"]["f"]
        fl = step_flops(w, cd["split"] + cd["single"], cf["split"] + cf["single"],
                        ns_steps=0 if w.optimizer == "adamt" else 10, products=5 if w.optimizer == "adamt" else 3)
        ph = head["phases"]
        per_phase = {}
        for name, work in (("stats", fl["syrk"]), ("roots", fl["roots"]), ("update", fl["ns"] + fl["precond"])):
            if name in ph and ph[name] > 0:
                # phases are per rank; the whole-job work is divided over `world` ranks
                per_phase[name] = {"ms": round(ph[name], 3), "tflops_per_gpu": round(work / world / ph[name] / 1e9, 1)}
        if "exchange" in ph and "update" in per_phase:
            per_phase["update"]["exchange_ms"] = round(ph["exchange"], 3)
        for v in per_phase.values():
            v["frac"] = round(v["tflops_per_gpu"] / pk["tflops"], 4)
        top = max(per_phase, key=lambda k: per_phase[k]["ms"]) if per_phase else None
        roof = None
        if top:
            a = per_phase[top]["tflops_per_gpu"]
            roof = {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "phase": top, "achieved": a, "peak": pk["tflops"],
                    "unit": "TFLOP/s", "frac": round(a / pk["tflops"], 4),
                    "traffic": (roots_traffic(layers // world, mlp) if top == "roots" else
                                update_traffic(2 * layers // world, mlp, hidden) if top == "update" and w.layout == "llama"
                                else None),
                    "peak_source": pk["source"] + " (sustained cuBLAS BF16: the kernel runs inside a long step)",
                    "note": "achieved = algorithmic single-pass flops of the phase / its CUDA-event time on the launching "
                            "stream; this kernel is 100 / 82 / 91 % of the statistics / factor / update phase by ncu share"}
            roof["newton_steps"] = {"hidden": cd["newton_steps"], "mlp": cf["newton_steps"]}
            roof["finish_order"] = {"hidden": cd["finish_order"], "mlp": cf["finish_order"]}
            if top == "roots":
                # what the tensor cores execute: three FP16 plane products per accumulator, on the 128x256 tiles
                # that meet the upper triangle (fractions 0.5625 at n=2048, 0.523 at n=5632)
                ex = (3 * layers * (3 * cd["split"] + cd["single"]) * 2 * hidden ** 3 * tri_fraction(hidden, 256) +
                      layers * (3 * cf["split"] + cf["single"]) * 2 * mlp ** 3 * tri_fraction(mlp, 256)) / world / ph[top] / 1e9
                roof["executed"] = round(ex, 1)
                roof["frac_executed"] = round(ex / pk["tflops"], 4)
        line = {
            "metric": f"{w.optimizer}_optimizer_step_ms", "value": round(ms, 3), "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 operands / fp16 hi-lo splits, fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": w.describe(), "parallelism": f"layer-sharded x{world}", "l2": "inputs larger than L2",
                       "entry": w.entry, "spectrum": args.spectrum, "baseline_config": w.config},
            "e2e": ({"value": round(e2e_ms, 3), "unit": "ms", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4}
                    if e2e_ms is not None else None),
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": roof,
            "phases": per_phase,
            "algorithmic_flops": fl,
            "fallbacks": head["fallbacks"], "repairs": head["repairs"], "bound_failures": head["bound_failures"],
            "value_by_spectrum": by_spectrum,
            "capture": capture,
            "check": check,
        }
        mhz = line["clocks"]["sm_mhz"]
        if mhz:   # time x clock: comparable between runs whose power-capped clocks differ
            line["mhz_ms"] = round(ms * mhz, 1)
            for phase in per_phase.values():
                phase["mhz_ms"] = round(phase["ms"] * mhz, 1)
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(w, sample_rows=2048)
        print(json.dumps(line), flush=True)
    opt.close()
    if world > 1:
        dist.destroy_process_group()


def run_general(args, w: Workload) -> None:
    """Config 2: AdamT + ActivationStatistics, the general interface, on one GPU.  The statistic Grams are computed by the
    forward hooks, so the measured step is  (forward under capture() - plain forward) + commit() + step()."""
    import toner_b200
    from toner_b200 import ops
    from toner_b200.synthetic import make_stack

    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise SystemExit("--config 2 is the single-process general path; run it without torchrun")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    stack = make_stack(w.layout, w.layers, w.hidden, w.mlp, dev, seed=0)
    layers = {}
    for i, b in enumerate(stack):
        for name, mod in (("attn.q", b.attn.q), ("attn.k", b.attn.k), ("attn.v", b.attn.v), ("attn.proj", b.attn.proj),
                          ("mlp.fc", b.mlp.fc), ("mlp.proj", b.mlp.proj)):
            layers[f"blocks.{i}.{name}"] = mod
    params = [m.weight for m in layers.values()]
    opt = toner_b200.AdamT(params, lr=2e-3, weight_decay=WD, betas=(0.9, 0.95), eps=1e-15)
    stats = toner_b200.ActivationStatistics(layers, head=HEAD, stride=STRIDE, distributed=False)
    gen = torch.Generator(device=dev).manual_seed(99)
    grads = [torch.randn(p.shape, device=dev, generator=gen) * 1e-3 for p in params]
    x = torch.randn(w.sequences, w.seq_len, w.hidden, device=dev, generator=gen).to(torch.bfloat16)
    host_x = x.cpu().pin_memory()
    host_grads = [g.cpu().pin_memory() for g in grads]
    checksum = torch.zeros(1).pin_memory()

    def forward():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            h = x
            for b in stack:
                h = torch.nn.functional.layer_norm(b(h).float(), (w.hidden,)).to(torch.bfloat16)

    def step():
        with stats.capture():
            forward()
        for p, g in zip(params, grads):
            p.grad = g
        stats.commit(opt)
        opt.step()

    def e2e_step():
        x.copy_(host_x, non_blocking=True)
        for g, hg in zip(grads, host_grads):
            g.copy_(hg, non_blocking=True)
        step()
        checksum.copy_(params[0][0, :1], non_blocking=True)

    for _ in range(args.warmup):
        step()
    launches0 = ops.launch_count()
    with ClockSampler(0) as clocks:
        total = timed(step, args.steps, 1, dev)
    launches = (ops.launch_count() - launches0) // args.steps
    plain = timed(forward, max(3, args.steps), 1, dev)
    e2e_total = timed(e2e_step, args.steps, 1, dev) if not args.no_e2e else None
    ops.assert_healthy()
    ms = total - plain
    buckets = list(opt._buckets.values())
    fd = next(b.factors for b in buckets if b.factors.n == w.hidden)
    ff = next(b.factors for b in buckets if b.factors.n == w.mlp)
    log2p = fd.p.bit_length() - 1
    # the general interface factors one statistic per parameter (q, k, v each their own): 5 hidden-width, 1 MLP-width
    per_d = (fd.iterations - 1) * (log2p + 2) + fd.finish_order - 1
    per_f = (ff.iterations - 1) * (log2p + 2) + ff.finish_order - 1
    L, h, m = w.layers, w.hidden, w.mlp
    fl = {"syrk": w.rows * L * (5 * h * (h + 1) + m * (m + 1)), "ns": 0,
          "precond": sum(L * 5 * 2 * r * c * c for r, c in w.shapes),
          "roots": L * (5 * per_d * 2 * h ** 3 + per_f * 2 * m ** 3)}
    pk = peaks()
    achieved = sum(fl.values()) / ms / 1e9
    bytes_h2d = host_x.numel() * 2 + sum(g.numel() * 4 for g in host_grads)
    line = {
        "metric": "adamt_optimizer_step_ms", "value": round(ms, 3), "unit": "ms", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 operands / fp16 hi-lo splits, fp32 accumulate", "data": "synthetic",
        "config": {"workload": w.describe(), "parallelism": "single process", "entry": w.entry, "baseline_config": 2,
                   "l2": "L2 flushed by the step itself: 340 MB of gradients and 680 MB of moments stream through",
                   "timing": "value = (capture forward + commit + step) - plain forward"},
        "e2e": ({"value": round(e2e_total - plain, 3), "unit": "ms", "h2d_bytes_per_step": int(bytes_h2d),
                 "d2h_bytes_per_step": 4} if e2e_total is not None else None),
        "gpu_launches": int(launches), "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "phase": "whole step", "achieved": round(achieved, 1),
                     "peak": pk["tflops"], "unit": "TFLOP/s", "frac": round(achieved / pk["tflops"], 4), "traffic": None,
                     "newton_steps": {"hidden": fd.iterations, "mlp": ff.iterations},
                     "note": "launch-bound: 72 matrices of 768 x 768 .. 768 x 3072 and 752 rows per statistic; achieved = "
                             "algorithmic single-pass flops of the step / its time"},
        "phases": {"total_with_forward_ms": round(total, 3), "plain_forward_ms": round(plain, 3)},
        "algorithmic_flops": fl, "fallbacks": opt.fallbacks,
    }
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(w, sample_rows=w.rows)
    print(json.dumps(line), flush=True)
    stats.close()


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


def cpu_baseline(w: Workload, sample_rows: int = 2048):
    """The CPU restatement of the reference's general path (oracle/) for ONE layer, extrapolated to the stack.

    Gram products are timed on `sample_rows` rows and scaled to the full row count; the optimizer step
    (eigh factors, FP32 Newton-Schulz, update) is timed in full for the layer's matrices.  The two measured
    components are reported so that the extrapolation can be redone."""
    from oracle import toner_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    hidden, mlp, rows_total = w.hidden, w.mlp, w.rows
    sample_rows = min(sample_rows, rows_total)
    g = torch.Generator().manual_seed(0)
    t_gram = 0.0
    stats = {}
    for kind, n in (("attn", hidden), ("o", hidden), ("mlp", hidden), ("down", mlp)):
        x = torch.randn(sample_rows, n, generator=g).to(torch.bfloat16)
        t0 = time.perf_counter()
        gram = orc.gram(x)
        t_gram += time.perf_counter() - t0
        stats[kind] = gram / sample_rows
    if w.layout == "llama":
        shapes = dict(q=(hidden, hidden, "attn"), k=(hidden, hidden, "attn"), v=(hidden, hidden, "attn"),
                      o=(hidden, hidden, "o"), gate=(mlp, hidden, "mlp"), up=(mlp, hidden, "mlp"), down=(hidden, mlp, "down"))
    else:
        shapes = dict(q=(hidden, hidden, "attn"), k=(hidden, hidden, "attn"), v=(hidden, hidden, "attn"),
                      attn_proj=(hidden, hidden, "o"), fc=(mlp, hidden, "mlp"), mlp_proj=(hidden, mlp, "down"))
    t_step = 0.0
    adam = w.optimizer == "adamt"
    for role, (m, n, kind) in shapes.items():
        wt = torch.randn(m, n, generator=g) * 0.02
        grad = torch.randn(m, n, generator=g) * 1e-3
        st = orc.AdamTState() if adam else orc.MuonTState()
        st.ema, st.weight = orc.ema_update(None, 0.0, stats[kind], MOMENTUM)
        t0 = time.perf_counter()
        if adam:
            orc.adamt_step(wt, grad, st, lr=2e-3, weight_decay=WD, betas=(0.9, 0.95), eps=1e-15)
        else:
            orc.muont_step(wt, grad, st, lr=LR, weight_decay=WD, momentum=MOMENTUM, ns_mode="f32")
        t_step += time.perf_counter() - t0
    gram_full = t_gram * (rows_total / sample_rows)
    per_layer_ms = (gram_full + t_step) * 1e3
    return {"value": round(per_layer_ms * w.layers, 1), "unit": "ms", "cores": cores, "kind": "port",
            "measured": {"layer_step_ms": round(t_step * 1e3, 1), "gram_ms_on_sample": round(t_gram * 1e3, 2),
                         "sample_rows": sample_rows, "rows": rows_total, "layers": w.layers},
            "sample": f"1 of {w.layers} layers timed ({len(shapes)} matrices: eigh factors, "
                      f"{'AdamT moments' if adam else 'FP32 Newton-Schulz'}, update) and Gram products on {sample_rows} of "
                      f"{rows_total} rows; value = layers x (layer_step_ms + gram_ms_on_sample x rows / sample_rows)"}


def run_reference(args, w: Workload) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    runs = [cpu_baseline(w) for _ in range(max(1, min(args.steps, 2)))]
    base = min(runs, key=lambda r: r["value"])
    ms = base["value"]
    line = {"impl": "reference", "metric": f"{w.optimizer}_optimizer_step_ms", "value": ms, "unit": "ms",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": w.describe(), "baseline_config": w.config,
                       "entry": "reference general path (eigh factors, FP32 Newton-Schulz) restated on CPU, host cores"},
            "cpu_baseline": base,
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=4, choices=[2, 3, 4],
                    help="4: FastMuonT on the 24-layer Llama-style stack (headline); 3: FastMuonT on the 12-layer nanoGPT "
                         "stack; 2: AdamT + ActivationStatistics on the nanoGPT stack")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--hidden", type=int, default=0)
    ap.add_argument("--mlp", type=int, default=0)
    ap.add_argument("--sequences", type=int, default=0)
    ap.add_argument("--optimizer", default=None, choices=["muont", "adamt"], help="override the config's optimizer")
    ap.add_argument("--spectrum", default="iid", help="row covariance of the headline value: iid, loguniform:<cond>, spiked:<k>")
    ap.add_argument("--extra-spectra", default=None,
                    help="comma-separated spectra for value_by_spectrum (default for config 4: loguniform:1e6,spiked:8)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-capture", action="store_true", help="skip the row-capture timing")
    ap.add_argument("--sm-reserve", type=int, default=None,
                    help="SMs the GEMMs leave to NCCL while a collective overlaps them (several ranks; default: the engine's)")
    ap.add_argument("--single-deflation", action="store_true",
                    help="factor engine deflates one dominant direction only (A/B against the block power iteration)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (for profiler runs)")
    args = ap.parse_args()
    w = workload_of(args)
    if args.extra_spectra is None:
        args.extra_spectra = "loguniform:1e6,spiked:8" if w.config == 4 else ""
    if args.impl == "reference":
        run_reference(args, w)
    elif w.config == 2:
        run_general(args, w)
    else:
        run_fast(args, w)


if __name__ == "__main__":
    main()
