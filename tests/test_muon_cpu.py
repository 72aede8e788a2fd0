"""The oracle's plain Muon step against the fixture made by the reference's Muon (f32 Newton-Schulz, CPU)."""

import os

import numpy as np
import pytest
import torch

from oracle import toner_oracle as orc

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "muon.npz"))


def test_three_steps_match_the_reference():
    for i in range(3):
        w, buf = torch.from_numpy(GOLD[f"w0_{i}"]), None
        for step in range(3):
            w, buf = orc.muon_step(w, torch.from_numpy(GOLD[f"g{step}_{i}"]), buf, lr=0.02, momentum=0.95, nesterov=True,
                                   ns_steps=10, eps=1e-5, weight_decay=0.1, ns_mode="f32")
            # the reference stacks same-shape matrices (bmm), the oracle multiplies them one by one: last-bit noise
            assert orc.rel_fro(w, torch.from_numpy(GOLD[f"w{step + 1}_{i}"])) < 1e-5


def test_constructor_checks_do_not_need_a_gpu():
    from toner_b200.fast import Muon
    p = torch.nn.Parameter(torch.zeros(16, 16))
    with pytest.raises(ValueError):
        Muon([p], lr=0.02, ns_mode="f32")
    with pytest.raises(ValueError):
        Muon([torch.nn.Parameter(torch.zeros(16))], lr=0.02)
    with pytest.raises(ValueError):
        Muon([torch.nn.Parameter(torch.zeros(12, 16))], lr=0.02)
    opt = Muon([p], lr=0.02)
    p.grad = torch.zeros(16, 16)
    with pytest.raises(ValueError):
        opt.step()                                    # CPU tensors: there is no CPU path
