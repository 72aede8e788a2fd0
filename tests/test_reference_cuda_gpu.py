"""The CUDA path against what the reference itself computed on a CUDA device.

The reference refuses its "tpu" Newton-Schulz arithmetic (BF16 operands, FP32 accumulation) on a CPU and its fast
optimizers need CUDA and Triton, so those outputs were produced once by running the reference on a B200
(tests/golden/make_tpu_golden.py) and are kept as fixtures:
  newton_schulz_tpu.npz          toner.linalg.newton_schulz(mode="tpu") at 1, 2, 3, 5 and 10 steps
  muont_tpu_small2.npz           toner.MuonT(ns_mode="tpu", ns_steps=2), weights after each of four steps
  fast_v3_checkpoint_muont.pt    the toner.fast.v3 checkpoint toner.fast.FastMuonT returns after two steps
  fast_v3_case.npz               the weights that checkpoint belongs to and a sample of the third step's changes
                                 (FastMuonT and FastAdamT)
Two correct implementations of this Newton-Schulz iteration differ by the summation order of their products, and every
step multiplies that difference by up to 3.44 in directions that have not converged: one step agrees to 1e-6, two to
1e-5, three to 1e-3, ten to a few 1e-2 (the reference's CUDA output against its CPU restatement shows the same
numbers, tests/test_oracle_golden.py).  The bounds below follow that growth."""

import os

import numpy as np
import pytest
import torch

from oracle import toner_oracle as orc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.fixture(scope="module")
def tb():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import toner_b200
    return toner_b200


@pytest.mark.parametrize("tag", ["square", "wide", "tall", "mid"])
def test_newton_schulz_against_the_reference_on_cuda(tb, golden, tag):
    from toner_b200 import ops
    g = golden("newton_schulz_tpu.npz")
    m = t(g[f"{tag}_in"]).cuda()
    worst = {}
    for steps, bound in ((1, 2e-6), (2, 5e-5), (3, 5e-3), (10, 8e-2)):
        got = ops.ns_polar(m.clone(), steps, 1e-5)[0].cpu()
        worst[steps] = orc.rel_fro(got, t(g[f"{tag}_out{steps}"]))
        assert worst[steps] < bound, (tag, steps, worst[steps])
    s = torch.linalg.svdvals(ops.ns_polar(m.clone(), 10, 1e-5)[0].double().cpu())
    ref = torch.linalg.svdvals(t(g[f"{tag}_out10"]).double())
    assert abs(float(s.max()) - float(ref.max())) < 5e-2 and abs(float(s.min()) - float(ref.min())) < 1e-1
    print(f"newton_schulz {tag}: relative difference from the reference's CUDA output by steps {worst}")


def test_muont_against_the_reference_on_cuda(tb, golden):
    """General-path MuonT, two Newton-Schulz steps in tpu arithmetic: the change of every step within 2e-3."""
    g = golden("muont_tpu_small2.npz")
    w = torch.nn.Parameter(t(g["w0"]).clone().cuda())
    opt = tb.MuonT([w], lr=0.02, weight_decay=0.1, momentum=0.95, ns_steps=int(g["ns_steps"]))
    prev_got = prev_want = t(g["w0"])
    for s in range(g["w"].shape[0]):
        x, grad = t(g["x"][s]).cuda(), t(g["g"][s]).cuda()
        opt.update_statistics({w: x.T @ x / x.shape[0]})
        w.grad = grad
        opt.step()
        got, want = w.detach().cpu().clone(), t(g["w"][s])
        err = orc.rel_fro(got - prev_got, want - prev_want)
        assert err < 2e-3, (s, err)
        assert orc.rel_fro(got, want) < 2e-4 * (s + 1)
        prev_got, prev_want = got, want


def _tiny_case(g):
    hidden, mlp, layers, seq, mb, acc = (int(v) for v in g["dims"])
    from toner_b200.synthetic import make_stack
    stack = [b.cuda() for b in make_stack("llama", layers, hidden, mlp, "cpu", seed=0)]   # weights drawn on the CPU
    mats = [p for b in stack for p in b.parameters() if p.ndim == 2]
    return stack, mats, (hidden, mlp, layers, seq, mb, acc)


def _one_step(opt, stack, mats, dims, step):
    hidden, _, _, seq, mb, acc = dims
    for i in range(acc):
        x = torch.randn(mb, seq, hidden, generator=torch.Generator().manual_seed(500 + 10 * step + i))
        with opt.capture_microbatch():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                h = x.cuda()
                for b in stack:
                    h = b(h)
    opt.begin()
    gen = torch.Generator().manual_seed(900 + step)
    for p in mats:
        p.grad = (torch.randn(p.shape, generator=gen) * 1e-3).cuda()
    opt.step()
    torch.cuda.synchronize()


def test_checkpoint_written_by_the_reference_resumes_here(tb, golden):
    """A toner.fast.v3 checkpoint from the reference's FastMuonT (state after two steps) is loaded into FastMuonT here;
    the third step, on the same inputs, must change every matrix as the reference's third step did."""
    import toner_b200.fast as fast
    g = golden("fast_v3_case.npz")
    ckpt = torch.load(os.path.join(GOLDEN, "fast_v3_checkpoint_muont.pt"), weights_only=False)
    assert ckpt["format"] == "toner.fast.v3" and ckpt["core"]["t"] == 2
    stack, mats, dims = _tiny_case(g)
    with torch.no_grad():
        for p, w in zip(mats, t(g["muont_w2"])):
            p.copy_(w.view_as(p))
    opt = fast.FastMuonT([fast.ProjectionBlock.from_module(b) for b in stack], 0.02, weight_decay=0.1,
                         micro_batch_size=dims[4], sequence_length=dims[3], accumulation_steps=dims[5],
                         statistic_head=8, statistic_stride=4, ns_steps=2)
    try:
        opt.load_state_dict(ckpt)
        before = [p.detach().cpu().clone() for p in mats]
        _one_step(opt, stack, mats, dims, 2)
        for j, p in enumerate(mats):
            change = p.detach().cpu() - before[j]
            sample = change[::4, ::4].flatten()
            want = t(g["muont_change3_sample"][j])
            # the sample's norm is the yardstick: both vectors hold the same sixteenth of the entries
            err = float((sample - want).norm() / want.norm())
            assert err < 2e-3, (j, err)
            assert abs(float(change.double().norm()) / float(g["muont_change3_norm"][j]) - 1) < 1e-3
        again = opt.state_dict()
        assert again["format"] == ckpt["format"] and again["config"] == ckpt["config"] and again["core"]["t"] == 3
        assert set(again["core"]["ema"]) == set(ckpt["core"]["ema"])
        assert set(again["core"]["moments"]) == set(ckpt["core"]["moments"])
    finally:
        opt.close()


@pytest.mark.parametrize("kind", ["muont", "adamt"])
def test_three_steps_from_scratch_follow_the_reference_fast_path(tb, golden, kind):
    """The same run from its start: three steps of the fast optimizers here against the reference's own fast path
    (exact eigendecomposition factors in its first steps, split-precision products, its Triton statistics)."""
    import toner_b200.fast as fast
    g = golden("fast_v3_case.npz")
    stack, mats, dims = _tiny_case(g)
    common = dict(weight_decay=0.1, micro_batch_size=dims[4], sequence_length=dims[3], accumulation_steps=dims[5],
                  statistic_head=8, statistic_stride=4)
    if kind == "muont":
        opt = fast.FastMuonT([fast.ProjectionBlock.from_module(b) for b in stack], 0.02, ns_steps=2, **common)
    else:
        opt = fast.FastAdamT([fast.ProjectionBlock.from_module(b) for b in stack], 2e-3, betas=(0.9, 0.95), eps=1e-4,
                             **common)
    try:
        for step in range(3):
            before = [p.detach().cpu().clone() for p in mats]
            _one_step(opt, stack, mats, dims, step)
        for j, p in enumerate(mats):
            change = p.detach().cpu() - before[j]
            want = t(g[f"{kind}_change3_sample"][j])
            err = float((change[::4, ::4].flatten() - want).norm() / want.norm())
            assert err < (2e-3 if kind == "muont" else 5e-3), (kind, j, err)
            assert abs(float(p.detach().double().norm()) / float(g[f"{kind}_w3_norm"][j]) - 1) < 1e-4
    finally:
        opt.close()
