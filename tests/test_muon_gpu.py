"""The plain Muon baseline on the CUDA kernels against the oracle (BF16-operand Newton-Schulz restated on CPU)."""

import pytest
import torch

from oracle import toner_oracle as orc

pytestmark = pytest.mark.gpu
SHAPES = ((256, 384), (256, 384), (512, 128), (256, 384))


@pytest.fixture(scope="module")
def Muon():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from toner_b200.fast import Muon as cls
    return cls


@pytest.mark.parametrize("nesterov", [True, False])
def test_steps_match_the_oracle(Muon, nesterov):
    from toner_b200 import ops
    g = torch.Generator().manual_seed(2)
    w0 = [torch.randn(*s, generator=g) * 0.02 for s in SHAPES]
    params = [torch.nn.Parameter(w.clone().cuda()) for w in w0]
    opt = Muon(params, lr=0.02, momentum=0.95, nesterov=nesterov, ns_steps=2, weight_decay=0.1)
    ref, bufs = [w.clone() for w in w0], [None] * len(w0)
    for step in range(3):
        grads = [torch.randn(*s, generator=g) * 1e-3 for s in SHAPES]
        for i, p in enumerate(params):
            p.grad = None if (step == 1 and i == 3) else grads[i].cuda()     # one matrix sits a step out
        opt.step()
        for i in range(len(ref)):
            if step == 1 and i == 3:
                continue
            before = ref[i]
            ref[i], bufs[i] = orc.muon_step(before, grads[i], bufs[i], lr=0.02, momentum=0.95, nesterov=nesterov,
                                            ns_steps=2, eps=1e-5, weight_decay=0.1, ns_mode="tpu")
            got = params[i].detach().cpu()
            assert orc.rel_fro(got - before, ref[i] - before) < 2e-3, (step, i)
            assert orc.rel_fro(opt.state[params[i]]["momentum_buffer"].cpu(), bufs[i]) < 1e-6
            ref[i] = got.clone()        # continue from the CUDA weights so that steps are compared one at a time
    ops.assert_healthy()


def test_ten_steps_give_the_newton_schulz_envelope(Muon):
    """With the full ten steps the update is lr * sqrt(max(1, rows/cols)) times a matrix whose singular values lie in
    the iteration's fixed band (about 0.68 .. 1.13 for these coefficients)."""
    g = torch.Generator().manual_seed(4)
    w = torch.nn.Parameter(torch.zeros(512, 256, device="cuda"))
    opt = Muon([w], lr=1.0, momentum=0.0, nesterov=False, weight_decay=0.0)
    w.grad = torch.randn(512, 256, generator=g).cuda()
    opt.step()
    s = torch.linalg.svdvals((-w.detach() / 2 ** 0.5).double().cpu())
    assert 0.6 < s.min() and s.max() < 1.25, (s.min().item(), s.max().item())
