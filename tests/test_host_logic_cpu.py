"""Host-side logic that needs no GPU: sampling, ownership maps, strength handling, argument validation."""

import pytest
import torch

from oracle import toner_oracle as orc


@pytest.mark.parametrize("seq,head,stride", [(1024, 32, 16), (4096, 32, 16), (70, 32, 16), (20, 32, 16), (64, 0, 16),
                                             (33, 32, 16), (50, 4, 7)])
def test_sample_positions_match_reference(golden, seq, head, stride):
    from toner_b200.statistics import sample_positions
    assert sample_positions(seq, head, stride) == golden("positions.npz")[f"pos_{seq}_{head}_{stride}"].tolist()


def test_layer_counts_match_reference(golden):
    from toner_b200.fast.engine import layer_counts
    g = golden("layer_counts.npz")
    assert layer_counts(24, 8) == g["even_24_8"].tolist()
    assert layer_counts(24, 4, [1.0, 2.0, 0.0, 1.5]) == g["weighted_24"].tolist()
    assert layer_counts(7, 3, [1.0, 1.0, 1.0]) == g["weighted_7"].tolist()
    with pytest.raises(ValueError):
        layer_counts(7, 2)


def test_chunk_plan_covers_every_statistic_once():
    from toner_b200.fast.engine import chunk_members, chunk_plan
    for world, per, want in ((8, 9, 4), (2, 36, 4), (4, 6, 4), (8, 3, 4), (1, 5, 2)):
        chunks = chunk_plan(per, want)
        assert per % chunks == 0 and chunks <= max(1, want)
        seen = []
        for c in range(chunks):
            members = chunk_members(world, per, chunks, c)
            cs = per // chunks
            for r in range(world):   # rows [r*cs, (r+1)*cs) of the chunk buffer are rank r's own statistics
                assert members[r * cs:(r + 1) * cs] == [r * per + c * cs + j for j in range(cs)]
            seen += members
        assert sorted(seen) == list(range(world * per))


def test_root_orders():
    from toner_b200.core import root_orders
    assert root_orders(0.5, 0.125) == (8, 4)
    assert root_orders(0.125, 0.5) == (8, 4)
    assert root_orders(0.25, 0.25) == (4, 1)
    assert root_orders(1.0, 0.5) == (2, 2)
    assert root_orders(0.0, 0.25) == (4, 1)
    for bad in (0.3, -0.5, 1 / 64):
        with pytest.raises(ValueError):
            root_orders(bad, 0.5)


def test_general_optimizers_validate_before_touching_the_gpu():
    import toner_b200
    w = torch.nn.Parameter(torch.zeros(8, 8))
    with pytest.raises(ValueError, match="CUDA"):
        toner_b200.MuonT([w], lr=0.1)
    with pytest.raises(ValueError, match="CUDA"):
        toner_b200.AdamT([w], lr=0.1)
    with pytest.raises(ValueError):
        toner_b200.MuonT([torch.nn.Parameter(torch.zeros(8))], lr=0.1)          # not a matrix
    with pytest.raises(ValueError):
        toner_b200.MuonT([torch.nn.Parameter(torch.zeros(8, 8).half())], lr=0.1)  # not FP32
    with pytest.raises(ValueError):
        toner_b200.AdamT([w], lr=-1.0)


def test_fast_adapter_argument_errors():
    from toner_b200.fast import FastAdamT, FastMuonT, ProjectionBlock
    from toner_b200.synthetic import LlamaProjections
    block = LlamaProjections(256, 512, "cpu")
    common = dict(micro_batch_size=2, sequence_length=64)
    with pytest.raises(ValueError, match="CUDA"):
        FastMuonT([ProjectionBlock.from_module(block)], 0.02, **common)       # parameters on the CPU
    with pytest.raises(ValueError):
        FastMuonT([], 0.02, **common)
    with pytest.raises(ValueError):
        FastMuonT([block], 0.02, micro_batch_size=0, sequence_length=64)
    with pytest.raises(ValueError):
        FastMuonT([block], 0.02, inner_strength=0.3, **common)
    with pytest.raises(ValueError):
        FastAdamT([block], 0.02, inner_strength=0.5, **common)
    with pytest.raises(ValueError):
        FastMuonT([block], 0.02, statistic_head=65, **common)
    with pytest.raises(ValueError):
        FastMuonT([LlamaProjections(200, 512, "cpu")], 0.02, **common)        # widths must be multiples of 256


def test_activation_statistics_argument_errors():
    from toner_b200 import ActivationStatistics
    lin = torch.nn.Linear(16, 8)
    with pytest.raises(ValueError):
        ActivationStatistics({})
    with pytest.raises(TypeError):
        ActivationStatistics({"a": torch.nn.ReLU()})
    with pytest.raises(ValueError):
        ActivationStatistics({"a": lin, "b": lin})
    with pytest.raises(ValueError):
        ActivationStatistics({"a": lin}, stride=0)
    s = ActivationStatistics({"a": lin}, distributed=False)
    with pytest.raises(ValueError, match="CUDA"):
        with s.capture():
            lin(torch.randn(4, 16))
    with pytest.raises(RuntimeError):
        s.commit(object())                 # the failed capture discarded everything
    s.close()
    with pytest.raises(RuntimeError):
        with s.capture():
            pass


def test_newton_schedule_is_restated_consistently():
    """The oracle-side probe of the factor method: scaled coupled Newton in FP64 reaches the eigh answer."""
    torch.manual_seed(0)
    n, p, damping = 48, 8, 1e-3
    x = torch.randn(20, n, dtype=torch.float64)
    c = x.T @ x / 20
    truth = orc.inverse_root_truth(c.float(), 1.0 / p, damping).double()
    a = c / c.diagonal().mean() + damping * torch.eye(n, dtype=torch.float64)
    ub = a.norm()
    m, xk = a / ub, torch.eye(n, dtype=torch.float64)
    for _ in range(60):  # plain Newton coefficients: enough iterations always converge
        t = ((p + 1) * torch.eye(n, dtype=torch.float64) - m) / p
        xk = xk @ t
        m = torch.linalg.matrix_power(t, p) @ m
    assert orc.rel_fro(xk * ub ** (-1.0 / p), truth) < 1e-5


def test_flat_exchange_layout_with_uneven_ownership():
    """Ranks that own different numbers of layers: every rank's flat buffer is its roles' stacks back to back, and the
    stack of a role is found from the per-layer offset alone, whatever the rank owns (also nothing)."""
    from toner_b200.fast.engine import flat_layout, layer_counts, owner_block
    layers, world = 6, 3
    counts = layer_counts(layers, world, [1.0, 0.0, 2.0])
    assert counts == [2, 0, 4]
    shapes = {"down": (3, 4), "q": (2, 3)}
    numels = [a * b for a, b in shapes.values()]
    offsets = flat_layout(numels)
    lo = 0
    seen = {}
    for r, owned in enumerate(counts):
        flat = torch.empty(owned * sum(numels))
        for (role, shape), off, numel in zip(shapes.items(), offsets, numels):
            block = owner_block(flat, owned, off, numel, shape)
            assert block.shape == (owned,) + shape
            for j in range(owned):
                block[j] = 100.0 * list(shapes).index(role) + lo + j     # (role, global layer)
        # a reader that knows only counts[r] recovers every (role, layer)
        for (role, shape), off, numel in zip(shapes.items(), offsets, numels):
            got = owner_block(flat, owned, off, numel, shape)
            for j in range(owned):
                seen[(role, lo + j)] = got[j].unique().tolist()
        assert flat.numel() == 0 or torch.isfinite(flat).all()
        lo += owned
    assert len(seen) == layers * len(shapes)
    for (role, layer), vals in seen.items():
        assert vals == [100.0 * list(shapes).index(role) + layer]


@pytest.mark.parametrize("p", [2, 4, 8])
def test_the_stated_schedule_takes_every_eigenvalue_to_its_root(p):
    """toner_inv_roots_schedule states everything the factor engine does to an eigenvalue: the Newton coefficients
    (a_k, b_k) and the finishing polynomial.  Taking scalars through it on the host -- x = 1, mu = lambda; t = a - b mu,
    x *= t, mu *= t^p per step; then x q(1 - mu) -- must give lambda^(-1/p) for every lambda the bound allows; mu must
    never exceed 1 (the iteration would leave the interval its coefficients were levelled for) and must end within the
    stated distance of 1."""
    import numpy as np
    from toner_b200 import ops
    for lower in (2e-7, 1e-5, 1e-3, 0.03, 0.12, 0.3, 0.6):
        s = ops.inv_roots_schedule(lower, p)
        assert s["iterations"] == ops.inv_roots_iterations_for(lower, p) >= 2
        assert len(s["steps"]) == s["iterations"] - 1
        lam = np.exp(np.linspace(np.log(float(np.float32(lower))), 0.0, 4001))   # (the entry point takes a float)
        x, mu = np.ones_like(lam), lam.copy()
        for a, b in s["steps"]:
            t = a - b * mu
            assert (t > 0).all()
            x, mu = x * t, mu * t ** p
            assert mu.max() <= 1.0 + 1e-9, (p, lower, mu.max())
        assert 1.0 - mu.min() <= s["distance"] * (1 + 1e-6) + 1e-9, (p, lower)
        q = np.polyval(np.array(s["coefficients"])[::-1], 1.0 - mu)
        assert np.abs(x * q * lam ** (1.0 / p) - 1.0).max() < 5e-6, (p, lower)


def test_finishing_polynomial_holds_its_tolerance():
    """The Chebyshev fit of (1 - r)^(-1/p) the engine finishes with: relative error below 3e-6 on the interval it is
    stated for, [-0.02, 1.15 e + 1e-3], and coefficients without cancellation."""
    import numpy as np
    from toner_b200 import ops
    for p in (2, 4, 8):
        for lower in (1e-6, 1e-4, 1e-2, 0.05, 0.1, 0.2, 0.4):
            s = ops.inv_roots_schedule(lower, p)
            c, e = np.array(s["coefficients"]), s["distance"]
            assert 0 < e < 0.6 and 2 <= len(c) - 1 <= 12
            hi = 1.15 * e + 1e-3
            r = np.linspace(-0.02, hi, 2001)
            q = np.polyval(c[::-1], r)
            assert np.abs(q * (1 - r) ** (1.0 / p) - 1).max() < 3.2e-6, (p, lower)
            assert (np.abs(c) * hi ** np.arange(len(c))).sum() <= 2.5 + 1e-9
