"""Generate muon.npz by running the reference's plain Muon baseline on CPU.

    REFERENCE_SRC=/path/to/Toner/src python tests/golden/make_muon_golden.py

Three matrices (two of one shape, so that the batched path stacks them; one tall), three steps, Newton-Schulz in
"f32" mode -- the mode the reference runs on CPU (src/toner/fast/muon.py:53-164).
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
from toner.fast.muon import Muon  # noqa: E402

SHAPES = ((40, 48), (40, 48), (96, 32))


def main() -> None:
    g = torch.Generator().manual_seed(17)
    params = [torch.nn.Parameter(torch.randn(*s, generator=g) * 0.02) for s in SHAPES]
    out = {f"w0_{i}": p.detach().clone().numpy() for i, p in enumerate(params)}
    opt = Muon(params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=10, eps=1e-5, weight_decay=0.1, ns_mode="f32",
               batched=True, distributed=False)
    for step in range(3):
        for i, p in enumerate(params):
            p.grad = torch.randn(p.shape, generator=g) * 1e-3
            out[f"g{step}_{i}"] = p.grad.clone().numpy()
        opt.step()
        for i, p in enumerate(params):
            out[f"w{step + 1}_{i}"] = p.detach().clone().numpy()
    np.savez_compressed(os.path.join(HERE, "muon.npz"), **out)
    print("wrote muon.npz")


if __name__ == "__main__":
    main()
