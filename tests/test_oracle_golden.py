"""The CPU oracle against outputs of the reference itself (tests/golden/*.npz,
written by tests/golden/make_golden.py)."""

import numpy as np
import pytest
import torch

from oracle import toner_oracle as orc


def t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("seq,head,stride", [(1024, 32, 16), (4096, 32, 16), (70, 32, 16), (20, 32, 16),
                                             (64, 0, 16), (33, 32, 16), (50, 4, 7)])
def test_sample_positions(golden, seq, head, stride):
    want = golden("positions.npz")[f"pos_{seq}_{head}_{stride}"]
    assert orc.sample_positions(seq, head, stride) == want.tolist()


def test_position_counts_of_the_benchmark_configurations():
    assert len(orc.sample_positions(1024)) == 94
    assert len(orc.sample_positions(4096)) == 286


@pytest.mark.parametrize("tag,s_in,s_out", [("muont", 0.5, 0.125), ("adamt", 0.25, 0.25), ("rankdef", 0.5, 0.125)])
def test_input_factors(golden, tag, s_in, s_out):
    g = golden("factors.npz")
    inner, outer, decay = orc.input_factors(t(g[f"{tag}_c"]), s_in, s_out, 1e-3)
    # same LAPACK, same arithmetic: agreement to rounding of the eigensolver
    assert orc.rel_fro(inner, t(g[f"{tag}_inner"])) < 2e-5
    assert orc.rel_fro(outer, t(g[f"{tag}_outer"])) < 2e-5
    assert orc.rel_fro(decay, t(g[f"{tag}_decay"])) < 2e-5
    assert abs(float(decay.diagonal().mean()) - 1.0) < 1e-5


@pytest.mark.parametrize("tag", ["wide", "tall", "square"])
def test_newton_schulz_f32(golden, tag):
    g = golden("newton_schulz.npz")
    got3 = orc.newton_schulz(t(g[f"{tag}_in"]), 3, 1e-5, "f32")
    assert orc.rel_fro(got3, t(g[f"{tag}_out3"])) < 1e-5
    got = orc.newton_schulz(t(g[f"{tag}_in"]), 10, 1e-5, "f32")
    assert orc.rel_fro(got, t(g[f"{tag}_out"])) < 1e-4


@pytest.mark.parametrize("tag", ["square", "wide", "tall", "mid"])
def test_newton_schulz_tpu_against_the_reference_on_cuda(golden, tag):
    """The restated "tpu" arithmetic (operands rounded to BF16, FP32 products) against the reference's own
    toner.linalg.newton_schulz(mode="tpu") run on a B200 (tests/golden/make_tpu_golden.py).  The two differ by the
    summation order inside each product only; the iteration multiplies that by up to 3.44 per step in directions
    that have not converged (measured here: 7e-7 after one step, 1e-5 after two, 9e-4 after three, 3.6e-2 after ten,
    the same as the reference's tpu mode against its own f32 mode)."""
    g = golden("newton_schulz_tpu.npz")
    m = t(g[f"{tag}_in"])
    for steps, bound in ((1, 1e-6), (2, 2e-5), (3, 2e-3), (5, 3e-2), (10, 6e-2)):
        got = orc.newton_schulz(m, steps, 1e-5, "tpu")
        assert orc.rel_fro(got, t(g[f"{tag}_out{steps}"])) < bound, (tag, steps)
    # the reference's batched and per-matrix products agree bit for bit on that device; its tpu and f32 modes do not
    assert float(g["self_noise_batched_vs_single"].max()) == 0.0
    assert 2e-2 < float(g["self_noise_tpu_vs_f32"][-1]) < 6e-2


@pytest.mark.parametrize("tag,update_bound,weight_bound", [("small2", 2e-3, 1e-4), ("small", 8e-2, 2e-2),
                                                           ("tall", 8e-2, 2e-2)])
def test_muont_tpu_against_the_reference_on_cuda(golden, tag, update_bound, weight_bound):
    """muont_step(ns_mode="tpu") against toner.MuonT(ns_mode="tpu") run on a B200: with two Newton-Schulz steps every
    step's change agrees to 2e-3 (measured 1e-4 .. 3e-4); with ten, the iteration's sensitivity shows (4e-2 .. 5e-2 on
    a change, up to 1e-2 on these small weights, which move by 15 % of their norm per step)."""
    g = golden(f"muont_tpu_{tag}.npz")
    w, state, prev = t(g["w0"]).clone(), orc.MuonTState(), t(g["w0"])
    for s in range(g["w"].shape[0]):
        x, grad = t(g["x"][s]), t(g["g"][s])
        state.ema, state.weight = orc.ema_update(state.ema, state.weight, x.T @ x / x.shape[0], 0.95)
        mine = orc.muont_step(w, grad, state, lr=0.02, weight_decay=0.1, momentum=0.95, ns_mode="tpu",
                              ns_steps=int(g["ns_steps"]))
        want = t(g["w"][s])
        assert orc.rel_fro(mine - w, want - prev) < update_bound, (tag, s)
        assert orc.rel_fro(mine, want) < weight_bound, (tag, s)
        w, prev = mine, want


def test_newton_schulz_tpu_restatement_is_a_polar_approximation():
    m = torch.randn(64, 96, generator=torch.Generator().manual_seed(2))
    x = orc.newton_schulz(m, 10, 1e-5, "tpu")
    s = torch.linalg.svdvals(x.double())
    assert 0.6 < float(s.min()) and float(s.max()) < 1.2
    # one step: BF16 operand rounding only perturbs at the 2^-8 level
    assert orc.rel_fro(orc.newton_schulz(m, 1, 1e-5, "tpu"), orc.newton_schulz(m, 1, 1e-5, "f32")) < 1e-2


def _run(kind, g, steps):
    w = t(g["w0"]).clone()
    state = orc.MuonTState() if kind == "muont" else orc.AdamTState()
    out = []
    for s in range(steps):
        x, grad = t(g["x"][s]), t(g["g"][s])
        beta = 0.95
        state.ema, state.weight = orc.ema_update(state.ema, state.weight, x.T @ x / x.shape[0], beta)
        if kind == "muont":
            w = orc.muont_step(w, grad, state, lr=0.02, weight_decay=0.1, momentum=0.95, ns_mode="f32")
        else:
            w = orc.adamt_step(w, grad, state, lr=2e-3, weight_decay=0.1, betas=(0.9, 0.95))
        out.append(w)
    return out


@pytest.mark.parametrize("kind", ["muont", "adamt"])
@pytest.mark.parametrize("tag", ["small", "tall"])
def test_optimizer_steps(golden, kind, tag):
    g = golden(f"{kind}_{tag}.npz")
    ws = _run(kind, g, g["w"].shape[0])
    prev = t(g["w0"])
    for s, w in enumerate(ws):
        want = t(g["w"][s])
        # compare the per-step change, which is what the optimizer computes
        assert orc.rel_fro(w - prev, want - prev) < 2e-3 * (s + 1), (kind, tag, s)
        assert orc.rel_fro(w, want) < 1e-4
        prev = want


def _cfg1_inputs(step):
    gen = torch.Generator().manual_seed(1234 + step)
    x = torch.randn(8192, 768, generator=gen).to(torch.bfloat16).float()
    grad = torch.randn(768, 768, generator=gen) * 1e-3
    return x, grad


@pytest.mark.parametrize("kind", ["muont", "adamt"])
def test_config1_three_steps(golden, kind):
    """768x768 weight, 8192 BF16-rounded rows per step: first three of the ten golden steps."""
    g = golden(f"{kind}_cfg1.npz")
    torch.manual_seed(0)
    lin = torch.nn.Linear(768, 768, bias=False)
    with torch.no_grad():
        lin.weight.normal_(0, 0.02)
    w = lin.weight.detach().clone()
    assert torch.equal(w[::16, ::16], t(g["w0_sample"]))
    state = orc.MuonTState() if kind == "muont" else orc.AdamTState()
    for s in range(3):
        x, grad = _cfg1_inputs(s)
        state.ema, state.weight = orc.ema_update(state.ema, state.weight, x.T @ x / 8192, 0.95)
        if kind == "muont":
            w = orc.muont_step(w, grad, state, lr=0.02, weight_decay=0.1, momentum=0.95, ns_mode="f32")
        else:
            w = orc.adamt_step(w, grad, state, lr=2e-3, weight_decay=0.1, betas=(0.9, 0.95))
        assert orc.rel_fro(w[::16, ::16], t(g["w_sample"][s])) < 1e-4
        assert abs(orc.fro(w) - float(g["w_norm"][s])) / float(g["w_norm"][s]) < 1e-5


def test_activation_statistics(golden):
    g = golden("activation_statistics.npz")
    xs, wa = t(g["x"]), t(g["wa"])
    rows_a = torch.cat([orc.sampled_rows(x, 4, 3) for x in xs])
    rows_b = torch.cat([orc.sampled_rows(torch.relu(x @ wa.T), 4, 3) for x in xs])
    assert orc.rel_fro(orc.gram(rows_a) / rows_a.shape[0], t(g["mean_a"])) < 1e-6
    assert orc.rel_fro(orc.gram(rows_b) / rows_b.shape[0], t(g["mean_b"])) < 1e-5


def test_layer_counts(golden):
    g = golden("layer_counts.npz")
    assert orc.layer_counts(24, 8) == g["even_24_8"].tolist()
    assert orc.layer_counts(12, 1) == g["even_12_1"].tolist()
    assert orc.layer_counts(24, 4, [1.0, 2.0, 0.0, 1.5]) == g["weighted_24"].tolist()
    assert orc.layer_counts(7, 3, [1.0, 1.0, 1.0]) == g["weighted_7"].tolist()
    with pytest.raises(ValueError):
        orc.layer_counts(7, 2)


def test_packed_triangle_round_trip():
    n = 13
    full = torch.randn(n, n)
    full = full + full.T
    packed = orc.pack_upper(full)
    assert packed.numel() == n * (n + 1) // 2
    for r, c in ((0, 0), (0, 12), (5, 5), (5, 9), (12, 12)):
        assert packed[orc.packed_index(r, c, n)] == full[r, c]
    ema = torch.randn(n, n)
    got = orc.unpack_ema(packed, ema, 0.9, 0.25)
    assert torch.allclose(got, 0.9 * ema + 0.25 * full, atol=1e-6)
