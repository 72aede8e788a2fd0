"""Generate the golden fixtures in this directory by running the reference itself.

Usage (only where the reference checkout is available):

    REFERENCE_SRC=/path/to/Toner/src python tests/golden/make_golden.py

The reference is pure Python and runs on CPU, so its outputs on small seeded
inputs are stored as ``*.npz`` next to this script.  The tests compare the CPU
oracle (``oracle/toner_oracle.py``) with these files, and the CUDA path with
the oracle.  ``ns_mode="tpu"`` is not covered: the reference refuses it on CPU.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if "REFERENCE_SRC" not in os.environ:
    raise SystemExit("set REFERENCE_SRC to the src/ directory of a Toner checkout")
sys.path.insert(0, os.environ["REFERENCE_SRC"])

import toner  # noqa: E402
from toner.linalg import input_factors, newton_schulz  # noqa: E402
from toner.fast.engine import layer_counts  # noqa: E402
from toner.statistics import ActivationStatistics  # noqa: E402


def spd(n: int, cond: float, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(n, n, generator=g, dtype=torch.float64))
    lam = torch.exp(torch.rand(n, generator=g, dtype=torch.float64) * np.log(cond))
    return ((q * lam) @ q.T).float()


def step_inputs(seed: int, rows: int, n_in: int, n_out: int):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, n_in, generator=g).to(torch.bfloat16).float()
    grad = torch.randn(n_out, n_in, generator=g) * 1e-3
    return x, grad


def save(name: str, **arrays) -> None:
    np.savez_compressed(os.path.join(HERE, name), **{k: np.asarray(v) for k, v in arrays.items()})
    print("wrote", name, {k: np.asarray(v).shape for k, v in arrays.items()})


def main() -> None:
    torch.set_num_threads(4)

    # 1. sampling positions: read off the hook by feeding position-coded inputs.
    cases = [(1024, 32, 16), (4096, 32, 16), (70, 32, 16), (20, 32, 16), (64, 0, 16), (33, 32, 16), (50, 4, 7)]
    out = {}
    for seq, head, stride in cases:
        # One-hot rows: the mean Gram's diagonal is non-zero exactly at the sampled positions.
        probe = torch.nn.Linear(seq, 1, bias=False)
        stats = ActivationStatistics({"l": probe}, head=head, stride=stride, distributed=False)
        seen = {}

        class Recorder:
            def update_statistics(self, means):
                seen.update(means)

        with stats.capture():
            probe(torch.eye(seq).unsqueeze(0))
        stats.commit(Recorder())
        out[f"pos_{seq}_{head}_{stride}"] = seen[probe.weight].diagonal().nonzero().flatten().numpy()
        stats.close()
    save("positions.npz", **out)

    # 2. input_factors
    out = {}
    for tag, n, cond, s_in, s_out in (("muont", 48, 1e4, 0.5, 0.125), ("adamt", 48, 1e4, 0.25, 0.25),
                                     ("rankdef", 40, 1e2, 0.5, 0.125)):
        c = spd(n, cond, seed=7)
        if tag == "rankdef":  # rank-deficient Gram: 12 rows in 40 dims
            x = torch.randn(12, n, generator=torch.Generator().manual_seed(3))
            c = x.T @ x / 12
        inner, outer, decay = input_factors(c, s_in, s_out, 1e-3)
        out.update({f"{tag}_c": c, f"{tag}_inner": inner, f"{tag}_outer": outer, f"{tag}_decay": decay})
    save("factors.npz", **out)

    # 3. newton_schulz, f32 mode (the only mode the reference runs on CPU)
    out = {}
    for tag, shape in (("wide", (32, 48)), ("tall", (48, 32)), ("square", (40, 40))):
        m = torch.randn(*shape, generator=torch.Generator().manual_seed(11))
        out[f"{tag}_in"] = m
        out[f"{tag}_out"] = newton_schulz(m, 10, 1e-5, "f32")
        out[f"{tag}_out3"] = newton_schulz(m, 3, 1e-5, "f32")
    save("newton_schulz.npz", **out)

    # 4./5. MuonT and AdamT, small and at the 768x768 / 8192-row configuration
    for opt_name in ("muont", "adamt"):
        for tag, n_out, n_in, rows, steps in (("small", 40, 48, 256, 4), ("tall", 96, 32, 128, 3),
                                              ("cfg1", 768, 768, 8192, 10)):
            torch.manual_seed(0)
            lin = torch.nn.Linear(n_in, n_out, bias=False)
            with torch.no_grad():
                lin.weight.normal_(0, 0.02)
            w0 = lin.weight.detach().clone()
            if opt_name == "muont":
                opt = toner.MuonT([lin.weight], lr=0.02, weight_decay=0.1, momentum=0.95, ns_mode="f32")
            else:
                opt = toner.AdamT([lin.weight], lr=2e-3, weight_decay=0.1, betas=(0.9, 0.95))
            ws, xs, gs = [], [], []
            for s in range(steps):
                x, grad = step_inputs(1234 + s, rows, n_in, n_out)
                opt.update_statistics({lin.weight: x.T @ x / rows})
                lin.weight.grad = grad.clone()
                opt.step()
                ws.append(lin.weight.detach().clone())
                xs.append(x)
                gs.append(grad)
            if tag == "cfg1":  # keep the fixture small: strided sample + norms; inputs come from the seeds
                save(f"{opt_name}_{tag}.npz", w0_sample=w0[::16, ::16],
                     w_sample=torch.stack([w[::16, ::16] for w in ws]),
                     w_norm=torch.stack([w.double().norm() for w in ws]),
                     dw_norm=torch.stack([(b.double() - a.double()).norm() for a, b in zip([w0] + ws[:-1], ws)]))
            else:
                save(f"{opt_name}_{tag}.npz", w0=w0, w=torch.stack(ws), x=torch.stack(xs), g=torch.stack(gs))

    # 6. ActivationStatistics end to end on a two-layer model with a 3-D input, two microbatches
    torch.manual_seed(5)
    a, b = torch.nn.Linear(16, 24, bias=False), torch.nn.Linear(24, 8, bias=False)
    stats = ActivationStatistics({"a": a, "b": b}, head=4, stride=3, distributed=False)
    got = {}

    class Recorder2:
        def update_statistics(self, means):
            got.update(means)

    xs = [torch.randn(2, 19, 16, generator=torch.Generator().manual_seed(20 + i)) for i in range(2)]
    for x in xs:
        with stats.capture():
            b(torch.relu(a(x)))
    stats.commit(Recorder2())
    save("activation_statistics.npz", x=torch.stack(xs), wa=a.weight.detach(), wb=b.weight.detach(),
         mean_a=got[a.weight], mean_b=got[b.weight])

    # 7. layer ownership
    save("layer_counts.npz",
         even_24_8=np.array(layer_counts(24, 8)), even_12_1=np.array(layer_counts(12, 1)),
         weighted_24=np.array(layer_counts(24, 4, [1.0, 2.0, 0.0, 1.5])),
         weighted_7=np.array(layer_counts(7, 3, [1.0, 1.0, 1.0])))


if __name__ == "__main__":
    main()
