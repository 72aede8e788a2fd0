"""Factor engine (toner_inv_roots) against the CPU oracle's eigh factors and against FP64 truth.

The FP32 eigh oracle is itself up to ~1e-3 away from the exact factor on ill-conditioned statistics
(its eigenvalue error is ~1e-7 of the largest eigenvalue, against a damping floor of 1e-3), so each
case measures the oracle's own distance from FP64 truth and allows for it."""

import math

import pytest
import torch

from oracle import toner_oracle as orc

pytestmark = pytest.mark.gpu
DAMPING = 1e-3


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from toner_b200 import ops as _ops
    return _ops


def spd(n, cond, seed):
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(n, n, generator=g, dtype=torch.float64))
    lam = torch.exp(torch.rand(n, generator=g, dtype=torch.float64) * math.log(cond))
    return ((q * lam) @ q.T).float()


def check_roots(ops, stats, p, q, tol_truth=5e-4):
    ema = torch.stack(stats).cuda()
    lo, hi, fro2, status = ops.inv_roots(ema, DAMPING, p, q)
    ops.assert_healthy()
    assert status.tolist() == [0] * len(stats)
    for b, c in enumerate(stats):
        s_lo, s_hi = 1.0 / p, q / p
        inner, outer, decay = orc.input_factors(c, s_hi, s_lo, DAMPING)
        for got, strength, oracle in ((lo[b], s_lo, outer), (hi[b] if q > 1 else lo[b], s_hi, inner)):
            truth = orc.inverse_root_truth(c, strength, DAMPING)
            e_truth = orc.rel_fro(got.cpu(), truth)
            o_truth = orc.rel_fro(oracle, truth)
            e_oracle = orc.rel_fro(got.cpu(), oracle)
            # FP16 hi/lo operands carry 22 bits against FP32's 24: allow a few times the oracle's own error
            assert e_truth < max(tol_truth, 3 * o_truth), (b, strength, e_truth, o_truth)
            assert e_oracle < max(2e-3, 3 * o_truth), (b, strength, e_oracle, o_truth)
        assert abs(fro2[b].item() - orc.fro(outer) ** 2) / orc.fro(outer) ** 2 < 1e-3
        assert torch.equal(lo[b], lo[b].T)


@pytest.mark.parametrize("p,q", [(8, 4), (4, 1), (2, 1)])
def test_conditioning_sweep(ops, p, q):
    check_roots(ops, [spd(256, cond, 7) for cond in (1e2, 1e4, 1e6)], p, q)


def test_muont_powers_at_768(ops):
    check_roots(ops, [spd(768, 1e4, 3), spd(768, 1e6, 4)], 8, 4)


def test_rank_deficient_and_spiked_statistics(ops):
    """A Gram of 40 rows in 256 dimensions (216 zero eigenvalues sit on the damping floor), and a
    statistic with one dominant direction, as a mean activation gives."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(40, 256, generator=g)
    low_rank = x.T @ x / 40
    v = torch.randn(256, 1, generator=g)
    spiked = spd(256, 1e3, 5)
    spiked = spiked + (v @ v.T) * spiked.diagonal().mean() * 20
    # The 216 floor eigenvalues are 2.5e-5 of ||A||_F: 22-bit operands resolve them to ~1e-3 relative, which
    # the fourth power (A^-1/2 from A^-1/8) quadruples.  The FP32 eigh oracle is a few times closer here.
    check_roots(ops, [low_rank, spiked], 8, 4, tol_truth=3e-3)


def test_dominant_direction_at_full_width(ops):
    """Activation-like rows (noise plus a shared mean direction): one eigenvalue hundreds of times the rest,
    sitting at the very top of the normalised spectrum.  This is the case that needs the capped schedule."""
    from toner_b200.synthetic import fill_rows
    n, rows = 2048, 4096
    buf = torch.empty(2, rows, n, device="cuda", dtype=torch.bfloat16)
    fill_rows(buf, seed=1)
    ema = torch.zeros(2, n, n, device="cuda")
    ops.syrk_upper(buf, ema, ops.EMA_FULL, 0.95, 0.05 / rows)
    lo, hi, fro2, status = ops.inv_roots(ema, DAMPING, 8, 4)
    ops.assert_healthy()
    assert status.tolist() == [0, 0]
    for b in range(2):
        c = ema[b].cpu()
        assert orc.rel_fro(lo[b].cpu(), orc.inverse_root_truth(c, 0.125, DAMPING)) < 5e-4
        assert orc.rel_fro(hi[b].cpu(), orc.inverse_root_truth(c, 0.5, DAMPING)) < 2e-3


def test_zero_statistic_gives_scaled_identity(ops):
    ema = torch.zeros(1, 128, 128, device="cuda")
    lo, hi, fro2, status = ops.inv_roots(ema, DAMPING, 4, 1)
    ops.assert_healthy()
    want = torch.eye(128) * DAMPING ** -0.25  # (0 / 1e-30 + damping)^(-1/4), as the eigh rule gives
    assert status.item() == 0
    assert orc.rel_fro(lo[0].cpu(), want) < 1e-5


def test_chunked_workspace_gives_identical_roots(ops):
    stats = torch.stack([spd(256, 1e3, s) for s in range(5)]).cuda()
    full = ops.inv_roots(stats, DAMPING, 4, 1)[0]
    small_ws = torch.empty(ops.inv_roots_workspace_bytes(2, 256), device="cuda", dtype=torch.uint8)
    chunked = ops.inv_roots(stats, DAMPING, 4, 1, workspace=small_ws)[0]
    ops.assert_healthy()
    assert torch.equal(full, chunked)


def test_iteration_counts_are_stated(ops):
    assert ops.inv_roots_iterations(5632, 1e-3, 8) == 8
    assert ops.inv_roots_iterations(5632, 1e-3, 4) == 8
    assert ops.inv_roots_iterations(5632, 1e-3, 2) == 10
    assert ops.inv_roots_iterations(768, 1e-3, 8) <= 10


@pytest.mark.parametrize("p,q", [(8, 4), (4, 1), (2, 1)])
def test_finishing_series_at_every_order(ops, p, q):
    """The iteration stops where Newton steps plus finishing polynomial cost the fewest plane passes (the spectrum of M
    is then within 0.6 of 1) and the degree of the polynomial follows from that distance.  Sweeping the caller's bound
    moves the stopping point, so several degrees are exercised; every one must give the same roots as FP64 truth."""
    n = 384
    stats = torch.stack([spd(n, 3e2, 11), spd(n, 1e3, 12)]).cuda()
    norms = torch.zeros(2, device="cuda")
    ops.inv_roots(stats, DAMPING, p, q, norms=norms)
    top = 0.99 * DAMPING / norms.max().item()          # the largest bound both statistics satisfy
    truth = [(orc.inverse_root_truth(c.cpu(), 1.0 / p, DAMPING), orc.inverse_root_truth(c.cpu(), q / p, DAMPING))
             for c in stats]
    orders = set()
    for k in range(14):
        lower = top * 0.6 ** k
        orders.add(ops.inv_roots_finish_order(n, DAMPING, p, lower))
        lo, hi, _, st = ops.inv_roots(stats, DAMPING, p, q, lower=lower)
        ops.assert_healthy()
        assert st.tolist() == [0, 0], (k, st.tolist())
        for b in range(2):
            assert orc.rel_fro(lo[b].cpu(), truth[b][0]) < 5e-5, (k, b)
            if q > 1:
                assert orc.rel_fro(hi[b].cpu(), truth[b][1]) < 2e-4, (k, b)
    assert min(orders) <= 4 and max(orders) >= 7 and len(orders) >= 4, orders


def test_callers_spectrum_bound_saves_steps_and_is_checked(ops):
    """toner_inv_roots_ex: with the bound a caller derives from the reported ||A'||_F the engine takes fewer Newton
    steps and returns the same roots; a bound the statistics do not satisfy is flagged (status 3), not trusted."""
    stats = torch.stack([spd(512, 1e3, s) for s in range(3)]).cuda()
    norms = torch.zeros(3, device="cuda")
    lo0, hi0, _, st0 = ops.inv_roots(stats, DAMPING, 8, 4, norms=norms)
    assert st0.tolist() == [0, 0, 0]
    lower = 0.6 * DAMPING / norms.max().item()
    assert ops.inv_roots_iterations_for(lower, 8) < ops.inv_roots_iterations(512, DAMPING, 8)
    lo1, hi1, _, st1 = ops.inv_roots(stats, DAMPING, 8, 4, lower=lower)
    ops.assert_healthy()
    assert st1.tolist() == [0, 0, 0]
    for b in range(3):
        assert orc.rel_fro(lo1[b].cpu(), lo0[b].cpu()) < 2e-5 and orc.rel_fro(hi1[b].cpu(), hi0[b].cpu()) < 1e-4
    too_high = 5.0 * DAMPING / norms.min().item()
    _, _, _, st2 = ops.inv_roots(stats, DAMPING, 8, 4, lower=too_high)
    assert all(s in (1, 3) for s in st2.tolist()) and 3 in st2.tolist()


def test_dominant_direction_is_deflated(ops):
    """One eigenvalue 400 times the rest: the reported norm is that of the deflated statistic (about
    0.8 sqrt(n), not 0.8 (1 + n/4)), and the roots are as accurate as for a flat spectrum."""
    from toner_b200.synthetic import fill_rows
    n, rows = 2048, 16384
    buf = torch.empty(1, rows, n, device="cuda", dtype=torch.bfloat16)
    fill_rows(buf, seed=5)
    ema = torch.zeros(1, n, n, device="cuda")
    ops.syrk_upper(buf, ema, ops.EMA_FULL, 0.0, 1.0 / rows)
    norms = torch.zeros(1, device="cuda")
    lo, hi, _, status = ops.inv_roots(ema, DAMPING, 8, 4, norms=norms)
    ops.assert_healthy()
    assert status.tolist() == [0]
    assert norms.item() < 3.0 * n ** 0.5
    c = ema[0].cpu()
    assert orc.rel_fro(lo[0].cpu(), orc.inverse_root_truth(c, 0.125, DAMPING)) < 1e-4
    assert orc.rel_fro(hi[0].cpu(), orc.inverse_root_truth(c, 0.5, DAMPING)) < 5e-4
    assert torch.equal(lo[0], lo[0].T)


def test_repair_round_when_the_bound_no_longer_holds(ops):
    """FactorSet: between two steps one statistic is replaced by a far worse conditioned one, so the spectrum estimate
    carried over from the previous step is two orders of magnitude too high for it; the verification after the chain
    flags it, the repair round refactors it with the bound that always holds, and no eigendecomposition fallback is
    needed.  Two strong directions appearing in the other statistic break nothing: they are found and deflated."""
    from toner_b200 import core
    n = 512
    f = core.FactorSet(2, n, torch.device("cuda"), (0.5, 0.125), DAMPING)
    f.ema.copy_(torch.stack([spd(n, 10.0, 1), spd(n, 10.0, 2)]))
    f.compute()
    assert f.finish() == 0 and f.lower > 0 and f.lower_is_estimate
    g = torch.Generator().manual_seed(3)
    u, v = torch.randn(n, 1, generator=g), torch.randn(n, 1, generator=g)
    f.ema[0] += ((u @ u.T) + (v @ v.T)).cuda() * 50.0
    f.ema[1].copy_(spd(n, 3e3, 5))
    f.compute()
    assert f.finish() == 0
    # (the other statistic is repaired too if its two new directions have not converged within this call's sweeps)
    assert f.repairs in (1, 2) and f.fallbacks == 0 and f.bound_failures == 1
    assert not f.lower_is_estimate and f.estimate_backoff == 8     # estimates are suspended for a while
    for b in range(2):
        c = f.ema[b].cpu()
        assert orc.rel_fro(f.root_lo[b].cpu(), orc.inverse_root_truth(c, 0.125, DAMPING)) < 5e-4
        assert orc.rel_fro(f.root_hi[b].cpu(), orc.inverse_root_truth(c, 0.5, DAMPING)) < 2e-3


def test_non_finite_statistic_is_flagged_and_does_not_touch_its_neighbours(ops):
    """Failure detection without a fault: a statistic full of NaN (or with an infinite entry) comes back with status 2,
    nothing hangs or traps, and the healthy statistics of the same call are factored as if they were alone."""
    good = spd(256, 1e3, 21)
    bad_nan = torch.full((256, 256), float("nan"))
    bad_inf = spd(256, 1e3, 22)
    bad_inf[3, 3] = float("inf")
    alone = ops.inv_roots(good.unsqueeze(0).cuda(), DAMPING, 4, 1)[0][0]
    lo, _, _, status = ops.inv_roots(torch.stack([bad_nan, good, bad_inf]).cuda(), DAMPING, 4, 1)
    ops.assert_healthy()                       # no bounded wait ran out: the kernels finished normally
    assert status.tolist() == [2, 0, 2]
    assert torch.equal(lo[1], alone)


def _activation_like(n, rows, seed, k=3):
    """Statistics of well-conditioned rows (unit noise plus a shared mean direction), as the benchmark's."""
    from toner_b200.synthetic import fill_rows
    from toner_b200 import ops as _ops
    buf = torch.empty(k, rows, n, device="cuda", dtype=torch.bfloat16)
    fill_rows(buf, seed=seed)
    ema = torch.zeros(k, n, n, device="cuda")
    _ops.syrk_upper(buf, ema, _ops.EMA_FULL, 0.0, 1.0 / rows)
    return ema


def _extremes(c, damping=DAMPING):
    """Smallest eigenvalue of A = sym(C) / mean diag + damping I, and the largest once the top one is set aside."""
    c = c.double().cpu()
    lam = torch.linalg.eigvalsh(0.5 * (c + c.T)).clamp_min(0)
    lam = lam / lam.mean() + damping
    return float(lam[0]), float(lam[-2])


def test_tracked_spectrum_estimate_saves_steps(ops):
    """toner_inv_roots_tracked on well-conditioned statistics: the first call reports an estimate of lambda_min(A)
    (a little high, as a Rayleigh quotient is) and a certified bound of lambda_max(A'); the second call, scheduled for
    half the ratio of the two, takes fewer than half the plane passes and returns the same roots, verified."""
    n = 512
    ema = _activation_like(n, 8192, seed=3)
    k = ema.shape[0]
    norms, lmin, track = torch.zeros(k, device="cuda"), torch.zeros(k, device="cuda"), torch.zeros(k, n, device="cuda")
    lo0, hi0, _, st0 = ops.inv_roots(ema, DAMPING, 8, 4, norms=norms, track=track, lmin=lmin, track_sweeps=12,
                                     track_restart=True)
    ops.assert_healthy()
    assert st0.tolist() == [0] * k
    for b in range(k):
        true_min, true_max = _extremes(ema[b])
        assert 0.98 * true_min < lmin[b].item() < 1.4 * true_min, (lmin[b].item(), true_min)
        assert true_max < norms[b].item() < 2.5 * true_max, (norms[b].item(), true_max)   # certified, and tight
    assert abs(track.norm(dim=1) - 1).max().item() < 1e-4
    lower = 0.5 * float((lmin / norms).min())
    cold, warm = ops.inv_roots_iterations(n, DAMPING, 8), ops.inv_roots_iterations_for(lower, 8)
    assert warm <= 3 < cold, (warm, cold)
    resid = torch.zeros(k, device="cuda")
    lo1, hi1, _, st1 = ops.inv_roots(ema, DAMPING, 8, 4, lower=lower, lower_is_estimate=True, track=track, lmin=lmin,
                                     resid=resid, track_sweeps=4)
    ops.assert_healthy()
    assert st1.tolist() == [0] * k
    e_assumed = 1.0    # the verified distance of the last M from the identity stays inside what the schedule assumed
    assert 0 <= resid.min().item() and resid.max().item() < e_assumed
    for b in range(k):
        c = ema[b].cpu()
        assert orc.rel_fro(lo1[b].cpu(), orc.inverse_root_truth(c, 0.125, DAMPING)) < 5e-5
        assert orc.rel_fro(hi1[b].cpu(), orc.inverse_root_truth(c, 0.5, DAMPING)) < 2e-4
        assert orc.rel_fro(lo1[b].cpu(), lo0[b].cpu()) < 5e-5


def test_an_estimate_that_is_too_high_is_caught_after_the_chain(ops):
    """A caller's estimate above the true lower end of the spectrum cannot be checked before the chain has run; the
    verification afterwards (power iteration on I - M) must flag it: status 4, and only where it does not hold."""
    n = 512
    benign = _activation_like(n, 8192, seed=4, k=2)
    harder = spd(n, 300.0, 9).cuda().unsqueeze(0)          # smallest eigenvalue 300 times below the largest
    ema = torch.cat([benign, harder])
    k = ema.shape[0]
    norms, lmin, track = torch.zeros(k, device="cuda"), torch.zeros(k, device="cuda"), torch.zeros(k, n, device="cuda")
    ops.inv_roots(ema, DAMPING, 8, 4, norms=norms, track=track, lmin=lmin, track_sweeps=12, track_restart=True)
    ratio = (lmin / norms).tolist()
    assert ratio[2] < 0.1 * min(ratio[:2])
    lower = 0.5 * min(ratio[:2])                            # right for the first two statistics, far too high for the third
    _, _, _, st = ops.inv_roots(ema, DAMPING, 8, 4, lower=lower, lower_is_estimate=True, track=track, lmin=lmin,
                                track_sweeps=4)
    ops.assert_healthy()
    # (4: caught by the verification; 1: so far off that the last M already fails the convergence test)
    assert st.tolist()[:2] == [0, 0] and st.tolist()[2] in (1, 4)
    milder = 3.0 * ratio[2]                                 # three times too high for the third statistic only
    _, _, _, st = ops.inv_roots(ema, DAMPING, 8, 4, lower=milder, lower_is_estimate=True, track=track, lmin=lmin,
                                track_sweeps=4)
    assert st.tolist()[:2] == [0, 0] and st.tolist()[2] in (1, 4)
    with pytest.raises(Exception):                          # an estimate needs the tracked vectors to be verified
        ops.inv_roots(ema, DAMPING, 8, 4, lower=lower, lower_is_estimate=True)


def test_fifty_steps_on_a_drifting_statistic(ops):
    """FactorSet on an EMA (decay 0.95) fed fresh rows every step: after the first step the schedule follows the tracked
    spectrum (fewer Newton steps than the bound that always holds needs), no statistic is ever flagged, and the factors
    stay as close to the exact ones as those of a cold factorisation of the same statistic."""
    from toner_b200 import core
    from toner_b200.synthetic import fill_rows
    n, rows, k = 512, 4096, 2
    dev = torch.device("cuda")
    warm = core.FactorSet(k, n, dev, (0.5, 0.125), DAMPING)
    buf = torch.empty(k, rows, n, device="cuda", dtype=torch.bfloat16)
    counts, worst_ratio = [], 0.0
    for step in range(50):
        fill_rows(buf, seed=100 + step, mean_seed=7)
        ops.syrk_upper(buf, warm.ema, ops.EMA_FULL, 0.95 if step else 0.0, (0.05 if step else 1.0) / rows)
        warm.compute()
        counts.append(warm.iterations)
        assert warm.finish() == 0
        if step % 7 == 0 or step == 49:
            cold_lo, cold_hi, _, st = ops.inv_roots(warm.ema, DAMPING, 8, 4)
            assert st.tolist() == [0] * k
            for b in range(k):
                c = warm.ema[b].cpu()
                for got, ref, s in ((warm.root_lo[b], cold_lo[b], 0.125), (warm.root_hi[b], cold_hi[b], 0.5)):
                    truth = orc.inverse_root_truth(c, s, DAMPING)
                    e_warm, e_cold = orc.rel_fro(got.cpu(), truth), orc.rel_fro(ref.cpu(), truth)
                    worst_ratio = max(worst_ratio, e_warm / max(e_cold, 2e-5))
                    assert e_warm < 2e-4, (step, b, s, e_warm)
    assert warm.repairs == 0 and warm.fallbacks == 0 and warm.bound_failures == 0
    assert counts[0] == ops.inv_roots_iterations(n, DAMPING, 8) and max(counts[2:]) <= 3, counts
    assert worst_ratio < 2.0, worst_ratio
    print(f"Newton steps per factorisation over 50 steps: first {counts[0]}, then {sorted(set(counts[1:]))}; "
          f"warm / cold error ratio at most {worst_ratio:.2f}")


def test_block_deflation_of_outlier_directions(ops):
    """Five strong directions on top of a flat spectrum (outlier features): with vector slots the engine finds them by
    block power iteration, deflates all five, and the norm it reports -- the bound of what is left -- drops from the
    second-largest eigenvalue to the bulk's edge; the roots stay exact, and a second call started from the vectors of
    the first finds the same five with half the sweeps."""
    n, rows, k = 512, 8192, 2
    g = torch.Generator().manual_seed(5)
    stats = []
    for s in range(k):
        x = torch.randn(rows, n, generator=g)
        d, _ = torch.linalg.qr(torch.randn(n, 5, generator=g))
        x = x + (torch.randn(rows, 5, generator=g) * torch.tensor([4.0, 6.0, 9.0, 12.0, 16.0])) @ d.T
        stats.append(x.T @ x / rows)
    ema = torch.stack(stats).cuda()
    single_norms = torch.zeros(k, device="cuda")
    ops.inv_roots(ema, DAMPING, 8, 4, norms=single_norms)                      # one direction deflated (the old way)
    norms, lmin = torch.zeros(k, device="cuda"), torch.zeros(k, device="cuda")
    track, vectors = torch.zeros(k, n, device="cuda"), torch.zeros(k, 8, n, device="cuda")
    count = torch.zeros(k, device="cuda", dtype=torch.int32)
    for restart in (True, False):
        lo, hi, _, st = ops.inv_roots(ema, DAMPING, 8, 4, norms=norms, track=track, lmin=lmin,
                                      track_sweeps=12 if restart else 4, track_restart=restart, deflate=vectors,
                                      deflate_rank=8, deflate_restart=restart, deflated=count)
        ops.assert_healthy()
        assert st.tolist() == [0] * k
        # (from fixed vectors the weakest of the five may need the second call's sweeps to converge)
        assert all(c & 255 == 5 or (restart and c & 255 == 4) for c in count.tolist()), count.tolist()
        assert all(c >> 8 == 5 for c in count.tolist())      # five Ritz values stand out, converged or not
        if not restart:
            assert (norms < 0.1 * single_norms).all(), (norms.tolist(), single_norms.tolist())
        for b in range(k):
            c = ema[b].cpu()
            assert orc.rel_fro(lo[b].cpu(), orc.inverse_root_truth(c, 0.125, DAMPING)) < 1e-4
            assert orc.rel_fro(hi[b].cpu(), orc.inverse_root_truth(c, 0.5, DAMPING)) < 5e-4
            assert torch.equal(lo[b], lo[b].T)
            # the kept vectors are the statistic's top eigenvectors
            if not restart:
                top = torch.linalg.eigh(c.double())[1][:, -5:]
                inside = (vectors[b, :5].double().cpu() @ top).norm(dim=1)
                assert (inside > 1 - 1e-6).all()


def test_norm_from_the_block_iteration(ops):
    """Once the block's vectors have followed a statistic for a few calls, the largest Ritz value that was not deflated
    (times 1.4) replaces the certified norm bound and its three squarings: the norm reported stays above lambda_max of
    what is left and close to it, the schedule is no longer, nothing is flagged and the roots are as exact as before."""
    from toner_b200 import core
    n, k = 512, 3
    f = core.FactorSet(k, n, torch.device("cuda"), (0.5, 0.125), DAMPING)
    f.ema.copy_(_activation_like(n, 8192, seed=21, k=k))
    seen = []
    for call in range(6):
        f.compute()
        assert f.finish() == 0
        seen.append((f.ritz_in_flight, f.iterations, f.finish_order, f.norms_host.clone()))
    assert not seen[0][0] and not seen[1][0] and seen[-1][0], [s[0] for s in seen]
    assert f.repairs == 0 and f.fallbacks == 0 and f.bound_failures == 0
    certified = next(s for s in seen if not s[0] and s[1] <= 3)           # a tracked call before the switch
    assert seen[-1][1] == certified[1] and seen[-1][2] <= certified[2] + 1, (seen[-1][:3], certified[:3])
    for b in range(k):
        _, true_max = _extremes(f.ema[b])
        est = seen[-1][3][b].item()
        assert true_max < est < 1.5 * true_max, (true_max, est)           # above lambda_max(A'), and close to it
        c = f.ema[b].cpu()
        assert orc.rel_fro(f.root_lo[b].cpu(), orc.inverse_root_truth(c, 0.125, DAMPING)) < 5e-5
        assert orc.rel_fro(f.root_hi[b].cpu(), orc.inverse_root_truth(c, 0.5, DAMPING)) < 2e-4


def test_a_norm_estimate_that_is_too_low_is_caught(ops):
    """The Ritz value is only as good as its vector.  Vectors that miss the top of the spectrum (here: exact
    eigenvectors from its middle, which a few sweeps do not leave) give a norm below lambda_max; the statistic's largest
    eigenvalues then start ABOVE 1, lag or diverge, and every statistic must come back flagged, never silently wrong.
    With the vectors a proper call leaves behind the same request succeeds."""
    n, k = 384, 2
    stats = torch.stack([spd(n, 30.0, 31), spd(n, 30.0, 32)]).cuda()      # no outliers: nothing is deflated
    norms, lmin = torch.zeros(k, device="cuda"), torch.zeros(k, device="cuda")
    track, vectors = torch.zeros(k, n, device="cuda"), torch.zeros(k, 8, n, device="cuda")
    count = torch.zeros(k, device="cuda", dtype=torch.int32)
    kw = dict(norms=norms, track=track, lmin=lmin, deflate=vectors, deflate_rank=4, deflated=count)
    ops.inv_roots(stats, DAMPING, 8, 4, track_sweeps=12, track_restart=True, deflate_restart=True, **kw)
    lo_ref, hi_ref, _, st = ops.inv_roots(stats, DAMPING, 8, 4, track_sweeps=4, **kw)
    assert st.tolist() == [0] * k and (count & 255).tolist() == [0] * k
    lower = 0.5 * float((lmin / norms).min())
    good = vectors.clone()
    lo, hi, _, st = ops.inv_roots(stats, DAMPING, 8, 4, lower=lower, lower_is_estimate=True, track_sweeps=4,
                                  ritz_norm=True, **kw)
    ops.assert_healthy()
    assert st.tolist() == [0] * k
    for b in range(k):
        assert orc.rel_fro(lo[b].cpu(), lo_ref[b].cpu()) < 5e-5 and orc.rel_fro(hi[b].cpu(), hi_ref[b].cpu()) < 2e-4
    for b in range(k):
        c = stats[b].double().cpu()
        vec = torch.linalg.eigh(0.5 * (c + c.T))[1]
        vectors[b, :4] = vec[:, n // 2: n // 2 + 4].T.float().cuda()
    _, _, _, st = ops.inv_roots(stats, DAMPING, 8, 4, lower=lower, lower_is_estimate=True, track_sweeps=4,
                                ritz_norm=True, **kw)
    ops.assert_healthy()
    assert all(s in (1, 4) for s in st.tolist()), st.tolist()
    vectors.copy_(good)
    with pytest.raises(Exception):       # the norm estimate is verified together with an estimated lower bound only
        ops.inv_roots(stats, DAMPING, 8, 4, lower=lower, track_sweeps=4, ritz_norm=True, **kw)


def test_abrupt_changes_of_the_statistic_are_never_silently_wrong(ops):
    """FactorSet carries estimates of both ends of the spectrum and a block of vectors from step to step.  When the
    statistic changes abruptly under it -- new outlier directions of every strength, another mean, an ill-conditioned
    bulk, and back -- those are stale.  The a-posteriori checks must then flag, the repair round must run, and the
    roots handed to the optimizer must be right at EVERY step, flagged or not."""
    from toner_b200 import core
    n, k, rows = 384, 3, 3072
    g = torch.Generator().manual_seed(77)

    def stat(kind, seed):
        gg = torch.Generator().manual_seed(seed)
        x = torch.randn(rows, n, generator=gg) + 0.5 * torch.randn(1, n, generator=torch.Generator().manual_seed(5))
        if kind.startswith("spike"):
            strength = float(kind[5:])
            d, _ = torch.linalg.qr(torch.randn(n, 3, generator=gg))
            x = x + (torch.randn(rows, 3, generator=gg) * torch.tensor([1.0, 0.7, 0.5]) * strength) @ d.T
        elif kind == "mean":
            x = x + 2.0 * torch.randn(1, n, generator=gg)
        elif kind == "ill":
            return spd(n, 1e4, seed)
        return x.T @ x / rows

    f = core.FactorSet(k, n, torch.device("cuda"), (0.5, 0.125), DAMPING)
    plan = ["iid"] * 5 + ["spike1.5"] * 3 + ["spike3"] * 3 + ["spike12"] * 4 + ["iid"] * 4 + ["mean"] * 3 + ["ill"] * 4 + ["iid"] * 5
    used_estimate = False
    for step, kind in enumerate(plan):
        f.ema.copy_(torch.stack([stat(kind, 1000 + 10 * plan.index(kind) + b) for b in range(k)]))
        f.compute()
        used_estimate = used_estimate or f.ritz_in_flight
        f.finish()
        for b in range(k):
            c = f.ema[b].cpu()
            e_lo = orc.rel_fro(f.root_lo[b].cpu(), orc.inverse_root_truth(c, 0.125, DAMPING))
            e_hi = orc.rel_fro(f.root_hi[b].cpu(), orc.inverse_root_truth(c, 0.5, DAMPING))
            assert e_lo < 2e-4 and e_hi < 6e-4, (step, kind, b, e_lo, e_hi, f.repairs, f.fallbacks)
    assert used_estimate                      # the norm estimate was in use when the changes came
    print(f"repairs {f.repairs}, eigendecomposition fallbacks {f.fallbacks}, bound failures {f.bound_failures}")


def test_wide_tiles_in_the_factor_engine_give_the_same_bits(ops):
    """Three 5632-wide statistics in one call are enough tiles for the 256 x 512 tile variant of the deep split-precision
    products (X T, the finishing product, the squarings of the root); one statistic per call runs the same products on
    256 x 256 tiles.  Every element is accumulated in the same order either way, so the roots must be bit-identical --
    this pins the wide variant's operand-plane outputs, mirrored halves and affine epilogue inside the engine."""
    n, k = 5632, 3
    stats = _activation_like(n, 8192, seed=41, k=k)
    lo, hi, _, st = ops.inv_roots(stats, DAMPING, 8, 4)
    ops.assert_healthy()
    assert st.tolist() == [0] * k
    for b in range(k):
        lo1, hi1, _, st1 = ops.inv_roots(stats[b:b + 1].contiguous(), DAMPING, 8, 4)
        assert st1.tolist() == [0]
        assert torch.equal(lo[b], lo1[0]) and torch.equal(hi[b], hi1[0]), b
    ops.assert_healthy()
