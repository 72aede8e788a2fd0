"""Synthetic transformer-block stacks and inputs for tests and benchmarks.

Only the projection modules matter to the optimizers: a "block" here is a bag of ``nn.Linear`` layers
with the attribute names the adapters expect, and a cheap forward that feeds every projection an input
of the right shape (so the capture hooks run) without paying for attention.
"""

from __future__ import annotations

from typing import List

import torch
from torch import nn


class LlamaProjections(nn.Module):
    """q, k, v, o, gate, up, down of one Llama-style block (bias-free)."""

    def __init__(self, hidden: int, mlp: int, device, std: float = 0.02) -> None:
        super().__init__()
        for name, (o, i) in dict(q=(hidden, hidden), k=(hidden, hidden), v=(hidden, hidden), o=(hidden, hidden),
                                 gate=(mlp, hidden), up=(mlp, hidden), down=(hidden, mlp)).items():
            lin = nn.Linear(i, o, bias=False, device=device)
            nn.init.normal_(lin.weight, 0.0, std)
            setattr(self, name, lin)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Shape-correct stand-in for a block: every projection runs once on a plausible input."""
        a = self.q(x) + self.k(x) + self.v(x)
        x = x + self.o(a)
        h = torch.nn.functional.silu(self.gate(x)) * self.up(x)
        return x + self.down(h)


class NanoGPTAttention(nn.Module):
    def __init__(self, hidden: int, device, std: float) -> None:
        super().__init__()
        for name in ("q", "k", "v", "proj"):
            lin = nn.Linear(hidden, hidden, bias=True, device=device)
            nn.init.normal_(lin.weight, 0.0, std)
            setattr(self, name, lin)


class NanoGPTMlp(nn.Module):
    def __init__(self, hidden: int, mlp: int, device, std: float) -> None:
        super().__init__()
        self.fc = nn.Linear(hidden, mlp, bias=True, device=device)
        self.proj = nn.Linear(mlp, hidden, bias=True, device=device)
        nn.init.normal_(self.fc.weight, 0.0, std)
        nn.init.normal_(self.proj.weight, 0.0, std)


class NanoGPTProjections(nn.Module):
    """attn.{q,k,v,proj} and mlp.{fc,proj} of one modded-nanoGPT block (squared-ReLU MLP)."""

    def __init__(self, hidden: int, mlp: int, device, std: float = 0.02) -> None:
        super().__init__()
        self.attn = NanoGPTAttention(hidden, device, std)
        self.mlp = NanoGPTMlp(hidden, mlp, device, std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a = self.attn.q(x) + self.attn.k(x) + self.attn.v(x)
        x = x + self.attn.proj(a)
        return x + self.mlp.proj(torch.relu(self.mlp.fc(x)).square())


def make_stack(layout: str, layers: int, hidden: int, mlp: int, device, seed: int = 0) -> List[nn.Module]:
    torch.manual_seed(seed)
    cls = LlamaProjections if layout == "llama" else NanoGPTProjections
    return [cls(hidden, mlp, device) for _ in range(layers)]


def fill_rows(buf: torch.Tensor, seed: int, mean_seed: int = None) -> None:
    """Activation-like BF16 rows: unit-variance noise plus a shared mean direction (as residual streams have).
    `mean_seed` fixes the mean direction separately from the noise: ranks that hold different tokens of the same
    model see different rows around the same mean."""
    g = torch.Generator(device=buf.device).manual_seed(seed)
    k, rows, n = buf.shape
    gm = g if mean_seed is None else torch.Generator(device=buf.device).manual_seed(mean_seed)
    mean = torch.randn(1, 1, n, device=buf.device, generator=gm) * 0.5
    step = max(1, min(k, (1 << 28) // max(1, rows * n)))
    for s in range(0, k, step):
        e = min(k, s + step)
        buf[s:e].copy_(torch.randn(e - s, rows, n, device=buf.device, generator=g) + mean)


def fill_rows_spectrum(buf: torch.Tensor, seed: int, spectrum: str = "iid", mean_seed: int = None) -> None:
    """Rows whose population covariance has a chosen spectrum, plus the shared mean direction of ``fill_rows``.

    ``iid``            unit-variance noise: the sample covariance is Marchenko-Pastur around 1 (condition 2-3)
    ``loguniform:C``   rows = Z diag(sqrt(lambda)) Q^T with Q Haar and lambda log-uniform on [1, C] (scaled to unit mean):
                       the recipe of the inverse-root kernel sweep, condition C before damping
    ``spiked:K``       unit noise plus K strong directions of standard deviation 3 .. 20 (eigenvalues 10 .. 400 times
                       the bulk), as outlier features of a residual stream give
    Every statistic of the stack shares the population covariance (drawn from ``mean_seed``); the samples differ."""
    kind, _, arg = spectrum.partition(":")
    if kind == "iid":
        fill_rows(buf, seed, mean_seed)
        return
    dev = buf.device
    k, rows, n = buf.shape
    g = torch.Generator(device=dev).manual_seed(seed)
    gp = torch.Generator(device=dev).manual_seed(seed if mean_seed is None else mean_seed)
    mean = torch.randn(1, n, device=dev, generator=gp) * 0.5
    chunk = max(1, min(rows, (1 << 27) // n))
    if kind == "loguniform":
        cond = float(arg)
        q, _ = torch.linalg.qr(torch.randn(n, n, device=dev, generator=gp))
        lam = torch.exp(torch.rand(n, device=dev, generator=gp) * torch.log(torch.tensor(cond)))
        mix = (q * (lam / lam.mean()).sqrt()).T.contiguous()        # diag(sqrt(lambda)) Q^T
        tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True                # input synthesis only
        try:
            for s in range(k):
                for r0 in range(0, rows, chunk):
                    r1 = min(rows, r0 + chunk)
                    z = torch.randn(r1 - r0, n, device=dev, generator=g)
                    buf[s, r0:r1].copy_(z @ mix + mean)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = tf32
    elif kind == "spiked":
        spikes = int(arg)
        d, _ = torch.linalg.qr(torch.randn(n, spikes, device=dev, generator=gp))
        scale = torch.linspace(3.0, 20.0, spikes, device=dev)
        for s in range(k):
            for r0 in range(0, rows, chunk):
                r1 = min(rows, r0 + chunk)
                z = torch.randn(r1 - r0, n, device=dev, generator=g)
                z += (torch.randn(r1 - r0, spikes, device=dev, generator=g) * scale) @ d.T
                buf[s, r0:r1].copy_(z + mean)
    else:
        raise ValueError("spectrum is 'iid', 'loguniform:<condition>' or 'spiked:<directions>'")
