"""Generate capture.npz by running the reference's own model code on CPU.

    REFERENCE_ROOT=/path/to/Toner python tests/golden/make_capture_golden.py

The Marin model's norm() and sample_positions() (reproduce/marin/model.py:10-19) are imported from the checkout and
evaluated on small seeded BF16 activations; the rows at the sampled positions are what the reference's capture
kernels must reproduce (they recompute exactly this, reproduce/marin/ops.py:63-79).  Gathered rows are plain
indexing of the same tensors.  BF16 tensors are stored as their 16-bit patterns.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if "REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set REFERENCE_ROOT to the root of a Toner checkout")
sys.path.insert(0, os.environ["REFERENCE_ROOT"])
from reproduce.marin.model import norm, sample_positions  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def main() -> None:
    g = torch.Generator().manual_seed(5)
    batch, seq, hidden, head, stride, eps = 3, 96, 64, 8, 8, 1e-5
    idx = torch.tensor(sample_positions(seq, head, stride))
    out = {"idx": idx.numpy(), "eps": np.float32(eps), "batch": batch, "seq": seq, "hidden": hidden}
    for name, scale in (("x", 1.0), ("xmid", 3.0), ("attn", 0.5)):
        out[name] = bits((torch.randn(batch, seq, hidden, generator=g) * scale).to(torch.bfloat16))
    for name in ("w1", "w2"):
        out[name] = (1.0 + 0.1 * torch.randn(hidden, generator=g)).numpy()
    for src, w, key in (("x", "w1", "rows_attn"), ("xmid", "w2", "rows_mlp")):
        x = torch.from_numpy(out[src]).view(torch.bfloat16)
        layer = types.SimpleNamespace(weight=torch.from_numpy(out[w]), eps=eps)
        out[key] = bits(norm(layer, x)[:, idx].reshape(-1, hidden))        # the reference's BF16-residual RMSNorm
    out["rows_o"] = bits(torch.from_numpy(out["attn"]).view(torch.bfloat16)[:, idx].reshape(-1, hidden))
    np.savez_compressed(os.path.join(HERE, "capture.npz"), **out)
    print("wrote capture.npz", {k: getattr(v, "shape", v) for k, v in out.items()})


if __name__ == "__main__":
    main()
