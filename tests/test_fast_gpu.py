"""FastMuonT / FastAdamT through their public lifecycle (capture_microbatch -> begin -> step) against the
CPU oracle's general path fed with the same sampled rows and gradients."""

import pytest
import torch

from oracle import toner_oracle as orc

pytestmark = pytest.mark.gpu
HID, MLP, SEQ, MB, ACC, LAYERS = 256, 512, 64, 2, 2, 2
# Adam's eps for the parity run.  With the adapter's default (1e-15) the early updates are num / sqrt(v) on entries
# whose v is nearly zero: the first step is sign(g R), later ones have unbounded outliers where g R_old vanishes but
# g R_new does not, and one such entry rescales a whole matrix through ||U|| / ||U R||.  Both sides then amplify
# last-bit differences to 1e-2..1e-1 on the weights.  A comparable eps (gradients here are ~1e-3) keeps the same
# arithmetic on every path and makes the comparison meaningful.
ADAM_EPS = 1e-4


@pytest.fixture()
def fast():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import toner_b200.fast as f
    return f


def make(fast, layout, kind, dims=None, **kw):
    from toner_b200.synthetic import make_stack
    hid, mlp, seq, mb, acc, layers, head, stride = dims or (HID, MLP, SEQ, MB, ACC, LAYERS, 8, 4)
    stack = make_stack(layout, layers, hid, mlp, torch.device("cuda"), seed=0)
    wrap = fast.ProjectionBlock if layout == "llama" else fast.NanoGPTBlock
    cls = fast.FastMuonT if kind == "muont" else fast.FastAdamT
    opt = cls([wrap.from_module(b) for b in stack], 0.02 if kind == "muont" else 2e-3, weight_decay=0.1,
              micro_batch_size=mb, sequence_length=seq, accumulation_steps=acc, statistic_head=head,
              statistic_stride=stride, **kw)
    return stack, opt


def forward(stack, x):
    with torch.autocast("cuda", dtype=torch.bfloat16):
        for b in stack:
            x = b(x)
            if len(stack) > 4:   # deep stacks: keep the residual stream O(1), as the real blocks' norms do
                x = torch.nn.functional.layer_norm(x.float(), (x.shape[-1],))
    return x


def role_modules(block, layout):
    if layout == "llama":
        return {"attn": [block.q, block.k, block.v], "o": [block.o], "mlp": [block.gate, block.up], "down": [block.down]}
    return {"attn": [block.attn.q, block.attn.k, block.attn.v], "o": [block.attn.proj], "mlp": [block.mlp.fc],
            "down": [block.mlp.proj]}


@pytest.mark.parametrize("layout,kind", [("llama", "muont"), ("nanogpt", "muont"), ("llama", "adamt")])
def test_two_steps_match_oracle(fast, layout, kind):
    steps_against_oracle(fast, layout, kind, (HID, MLP, SEQ, MB, ACC, LAYERS, 8, 4), 2)


def test_nanogpt_stack_at_full_size(fast):
    """The 12-layer modded-nanoGPT shape (hidden 768, MLP 3072, six matrices per layer), 4 x 16 sequences of 1024
    tokens per update sampled with head 32 / stride 16: 6016 rows per statistic, 36 statistics of 768^2 and 12 of
    3072^2, 72 matrices -- one FastMuonT step against the oracle's general path on the same rows."""
    steps_against_oracle(fast, "nanogpt", "muont", (768, 3072, 1024, 16, 4, 12, 32, 16), 1)


def test_snapshot_and_cross_check(fast):
    """Engine extras of the reference: snapshot(layers) returns the bias-corrected statistics of the chosen layers
    (src/toner/fast/engine.py:929-941); check_every compares the factors with an eigendecomposition of the same
    statistics and reports (largest, median, statistic-weighted) relative errors per group and power (:743-770)."""
    stack, opt = make(fast, "llama", "muont", ns_steps=2, check_every=1)
    try:
        gen = torch.Generator().manual_seed(2)
        for _ in range(2):
            for _ in range(ACC):
                with opt.capture_microbatch():
                    forward(stack, torch.randn(MB, SEQ, HID, generator=gen).cuda())
            opt.begin()
            for b in stack:
                for p in b.parameters():
                    p.grad = (torch.randn(p.shape, generator=gen) * 1e-3).cuda()
            opt.step()
        core_ = opt._core
        snap = core_.snapshot([1])
        assert set(snap) == {"1.attn", "1.o", "1.mlp", "1.down"}
        d = core_.groups["d"]
        want = d.factors.ema[d.keys.index((1, "o"))] / core_.weight
        assert torch.equal(snap["1.o"], want.cpu())
        assert abs(core_.weight - (1 - 0.95 ** 2)) < 1e-12
        check = opt.diagnostics["check"]
        assert set(check) == {"d", "d_out", "f", "f_out"}
        for key, (worst, median, weighted) in check.items():
            assert 0 <= median <= worst < 2e-3 and weighted < 2e-3, (key, worst, median, weighted)
    finally:
        opt.close()


def test_llama_layer_at_full_width(fast):
    """One layer of the benchmark's Llama shape -- hidden 2048, MLP 5632, sequences of 4096 tokens sampled with head
    32 / stride 16 -- with 5 x 4 sequences per update: 5720 rows per statistic, so the 5632-wide statistic has full
    rank.  One FastMuonT step against the oracle's general path on the rows every projection read."""
    steps_against_oracle(fast, "llama", "muont", (2048, 5632, 4096, 4, 5, 1, 32, 16), 1)


def test_status_word_is_read_at_the_step(fast):
    """The engine reads the kernels' status word where it waits for the factors anyway: a kernel that gave up a wait
    (here the library's self-test kernel, which waits a millisecond for a barrier nothing arrives at) makes step()
    raise before any change is applied; the optimizer works again afterwards."""
    import ctypes as C
    from toner_b200 import _lib, ops
    stack, opt = make(fast, "llama", "muont", ns_steps=2)
    try:
        gen = torch.Generator().manual_seed(3)
        weights = [p for b in stack for p in b.parameters() if p.ndim == 2]

        def one(expect_error):
            for _ in range(ACC):
                with opt.capture_microbatch():
                    forward(stack, torch.randn(MB, SEQ, HID, generator=gen).cuda())
            if expect_error:
                stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                assert _lib.load().toner_selftest_bounded_wait(2_000_000, stream) == 0
            opt.begin()
            for p in weights:
                p.grad = (torch.randn(p.shape, generator=gen) * 1e-3).cuda()
            if expect_error:
                with pytest.raises(_lib.TonerError, match="gave up a bounded wait"):
                    opt.step()
            else:
                opt.step()
            torch.cuda.synchronize()

        one(False)
        before = [p.detach().clone() for p in weights]
        one(True)
        assert all(torch.equal(a, p.detach()) for a, p in zip(before, weights))
        assert ops.device_status() == 0
        one(False)
        assert not torch.equal(before[0], weights[0].detach())
        ops.assert_healthy()
    finally:
        opt.close()


def steps_against_oracle(fast, layout, kind, dims, steps):
    HID, MLP, SEQ, MB, ACC, LAYERS, head, stride = dims
    extra = dict(ns_steps=2) if kind == "muont" else dict(betas=(0.9, 0.95), eps=ADAM_EPS)
    stack, opt = make(fast, layout, kind, dims, **extra)
    try:
        positions = orc.sample_positions(SEQ, head, stride)
        params = [(li, k, m) for li, b in enumerate(stack) for k, ms in role_modules(b, layout).items() for m in ms]
        ref_w = {id(m): m.weight.detach().cpu().clone() for _, _, m in params}
        states = {id(m): (orc.MuonTState() if kind == "muont" else orc.AdamTState()) for _, _, m in params}
        gen = torch.Generator().manual_seed(5)
        for step in range(steps):
            captured = {}
            hooks = []
            for li, k, m in params:  # record what each projection really read (after autocast rounding)
                def rec(mod, inp, key=(li, k)):
                    captured.setdefault(key, []).append(inp[0].detach().to(torch.bfloat16).cpu())
                hooks.append(m.register_forward_pre_hook(rec))
            for mb in range(ACC):
                x = torch.randn(MB, SEQ, HID, generator=gen).cuda()
                with opt.capture_microbatch():
                    forward(stack, x)
            for h in hooks:
                h.remove()
            opt.begin()
            for _, _, m in params:
                m.weight.grad = (torch.randn(m.weight.shape, generator=gen) * 1e-3).cuda()
            opt.step()
            worst = worst_update = 0.0
            for li, k, m in params:
                rows = torch.cat([t[:, positions].reshape(-1, t.shape[-1]) for t in captured[(li, k)][::len(role_modules(stack[li], layout)[k])]])
                st = states[id(m)]
                st.ema, st.weight = orc.ema_update(st.ema, st.weight, orc.gram(rows) / rows.shape[0], 0.95)
                g = m.weight.grad.cpu()
                before = ref_w[id(m)]
                momentum_before = getattr(st, "momentum", None)
                if kind == "muont":
                    after = orc.muont_step(before, g, st, lr=0.02, weight_decay=0.1, momentum=0.95, ns_steps=2, ns_mode="tpu")
                else:
                    after = orc.adamt_step(before, g, st, lr=2e-3, weight_decay=0.1, betas=(0.9, 0.95), eps=ADAM_EPS)
                ref_w[id(m)] = after
                got = m.weight.detach().cpu()
                worst = max(worst, orc.rel_fro(got, after))
                if step == 0:   # later steps start from weights that already differ: compare the first change
                    err = orc.rel_fro(got - before, after - before)
                    if err > 2e-3 and kind == "muont":
                        # The oracle's FP32 eigendecomposition is itself 1e-3 from the exact factor on an
                        # ill-conditioned statistic, and two Newton-Schulz steps multiply that by up to 12: measure
                        # the oracle against its own FP64-factor variant and allow three times that distance.
                        exact = orc.MuonTState()
                        exact.ema, exact.weight, exact.momentum = st.ema, st.weight, momentum_before
                        after64 = orc.muont_step(before, g, exact, lr=0.02, weight_decay=0.1, momentum=0.95, ns_steps=2,
                                                 ns_mode="tpu", exact_factors=True)
                        own = orc.rel_fro(after - before, after64 - before)
                        err64 = orc.rel_fro(got - before, after64 - before)
                        print(f"  layer {li} {k}: change vs FP32-factor oracle {err:.2e}, vs FP64-factor oracle {err64:.2e}, "
                              f"oracle FP32 vs FP64 {own:.2e}")
                        # A statistic with (nearly) as many dimensions as rows has eigenvalues at the damping floor:
                        # condition 1e3 and more after normalisation.  There the Newton factors are within 5e-4 of the
                        # exact ones (tests/test_factors_gpu.py), A^(-1/2) being the fourth power of the computed
                        # A^(-1/8), and the two Newton-Schulz steps multiply that by up to 12.
                        near_singular = rows.shape[0] <= 1.05 * rows.shape[1]
                        allowed = max(2e-3, 3 * own, 6e-3 if near_singular else 0.0)
                        assert min(err, err64) < allowed, (layout, kind, li, k, err, err64, own)
                        err = min(err, 2e-3)
                    worst_update = max(worst_update, err)
            print(f"{layout} {kind} hidden {HID} step {step}: weights {worst:.2e}, first change {worst_update:.2e}")
            assert worst < 2e-3, (layout, kind, step, worst)
            assert worst_update < 4e-3, (layout, kind, step, worst_update)
            if kind == "adamt":  # the moments themselves are smooth functions of the factors
                for li, k, m in params[:3]:
                    role = [r for r, info in opt._core.roles.items() if any(w is m.weight for w in info["all"])][0]
                    info = opt._core.roles[role]
                    j = [i for i, w in enumerate(info["all"]) if w is m.weight][0]
                    assert orc.rel_fro(info["group"].m[j].cpu(), states[id(m)].exp_avg) < 1e-5
                    assert orc.rel_fro(info["group"].v[j].cpu(), states[id(m)].exp_avg_sq) < 5e-3
        d = opt.diagnostics
        assert d["fallbacks"] == 0 and set(d["gpu_ms"]) <= {"stats", "roots", "update"}
        from toner_b200 import ops
        ops.assert_healthy()
    finally:
        opt.close()


def test_lifecycle_errors_and_checkpoint_round_trip(fast):
    stack, opt = make(fast, "llama", "muont", ns_steps=2)
    try:
        with pytest.raises(RuntimeError):
            fast.FastMuonT([fast.ProjectionBlock.from_module(stack[0])], 0.02, micro_batch_size=MB, sequence_length=SEQ)
        with pytest.raises(RuntimeError):
            opt.begin()                                   # nothing captured yet
        with pytest.raises(RuntimeError):
            opt.state_dict()                              # no completed step
        with pytest.raises(ValueError):
            with opt.capture_microbatch():
                forward(stack, torch.randn(MB, SEQ + 1, HID).cuda())   # wrong shape
        with pytest.raises(RuntimeError):
            with opt.capture_microbatch():
                stack[0](torch.randn(MB, SEQ, HID, device="cuda", dtype=torch.bfloat16))   # not every projection ran
        gen = torch.Generator().manual_seed(1)
        for _ in range(ACC):
            with opt.capture_microbatch():
                forward(stack, torch.randn(MB, SEQ, HID, generator=gen).cuda())
        with pytest.raises(RuntimeError):
            with opt.capture_microbatch():
                pass                                      # one microbatch too many
        with pytest.raises(RuntimeError):
            opt.step()                                    # gradients missing
        for p in opt.param_groups[0]["params"]:
            p.grad = torch.randn_like(p) * 1e-3
        with pytest.raises(ValueError):
            opt.step(closure=lambda: None)
        opt.step()                                        # begin() is implied
        ckpt = opt.state_dict()
        assert ckpt["format"] == "toner.fast.v3" and ckpt["core"]["t"] == 1
        assert set(ckpt["core"]["ema"]) == {f"{i}.{k}" for i in range(LAYERS) for k in ("attn", "o", "mlp", "down")}
        assert set(ckpt["core"]["moments"]) == {f"body.blocks.{i}.{r}.weight" for i in range(LAYERS)
                                                for r in ("q", "k", "v", "o", "gate", "up", "down")}
        with pytest.raises(RuntimeError):
            opt.load_state_dict(ckpt)                     # not a fresh optimizer
    finally:
        opt.close()
    stack2, opt2 = make(fast, "llama", "muont", ns_steps=2)
    try:
        bad = dict(ckpt, config=dict(ckpt["config"], ns_steps=3))
        with pytest.raises(ValueError):
            opt2.load_state_dict(bad)
        opt2.load_state_dict(ckpt)
        core = opt2._core
        assert core.t == 1 and abs(core.weight - 0.05) < 1e-9
        assert torch.equal(core.groups["d"].factors.ema[0].cpu(), ckpt["core"]["ema"]["0.attn"])
        assert torch.equal(core.roles["q"]["group"].m[1].cpu(), ckpt["core"]["moments"]["body.blocks.1.q.weight"]["m"])
    finally:
        opt2.close()


@pytest.mark.parametrize("kind", ["muont", "adamt"])
def test_row_buffers_that_hold_half_a_step(fast, kind):
    """row_pieces=2: the row buffers hold two of the four microbatches; the first piece is folded into the partial
    Grams when its last forward has run (chunk_stats), the second by begin().  Same weights as with buffers for the
    whole step, up to the summation order of the statistic; a failed forward discards the folded piece too."""
    from toner_b200 import ops
    LONG = 256      # 70 sampled positions x 2 sequences x 4 microbatches = 560 rows: full-rank statistics
    extra = dict(ns_steps=2) if kind == "muont" else dict(betas=(0.9, 0.95), eps=ADAM_EPS)

    def run(pieces):
        from toner_b200.synthetic import make_stack
        stack = make_stack("llama", LAYERS, HID, MLP, torch.device("cuda"), seed=0)
        cls = fast.FastMuonT if kind == "muont" else fast.FastAdamT
        opt = cls([fast.ProjectionBlock.from_module(b) for b in stack], 0.02 if kind == "muont" else 2e-3, weight_decay=0.1,
                  micro_batch_size=MB, sequence_length=LONG, accumulation_steps=4, statistic_head=8, statistic_stride=4,
                  row_pieces=pieces, **extra)
        try:
            assert opt._core.groups["d"].rows_buf.shape[1] == 4 // pieces * MB * len(orc.sample_positions(LONG, 8, 4))
            gen = torch.Generator().manual_seed(11)
            for step in range(2):
                if step == 1 and pieces > 1:       # three good microbatches, then a forward that fails: all discarded
                    for _ in range(3):
                        with opt.capture_microbatch():
                            forward(stack, torch.zeros(MB, LONG, HID, device="cuda"))
                    with pytest.raises(RuntimeError):
                        with opt.capture_microbatch():
                            pass
                    assert opt._core.pieces_done == 0
                for mb in range(4):
                    x = torch.randn(MB, LONG, HID, generator=gen).cuda()
                    with opt.capture_microbatch():
                        forward(stack, x)
                opt.begin()
                for b in stack:
                    for p in b.parameters():
                        if p.ndim == 2:
                            p.grad = (torch.randn(p.shape, generator=gen) * 1e-3).cuda()
                opt.step()
            ops.assert_healthy()
            assert opt.diagnostics["fallbacks"] == 0
            return [p.detach().cpu().clone() for b in stack for p in b.parameters() if p.ndim == 2]
        finally:
            opt.close()

    # the statistic differs only in its last bits; the factor engine's own accuracy (1e-4) bounds what that can do
    whole, halves = run(1), run(2)
    for a, b in zip(whole, halves):
        assert orc.rel_fro(b, a) < 3e-4


def test_row_pieces_must_divide_the_accumulation(fast):
    with pytest.raises(ValueError):
        make(fast, "llama", "muont", row_pieces=3)


def test_statistics_follow_rows_that_arrive_in_slices(fast):
    """begin(ready=...): each slice of statistics waits for its own event and a group's factors start when its last
    slice is in.  Statistics are independent of one another, so the weights are bit-identical to a plain begin()."""
    def run(streamed):
        stack, opt = make(fast, "llama", "muont", ns_steps=2)
        try:
            gen = torch.Generator().manual_seed(21)
            for step in range(2):
                for mb in range(ACC):
                    with opt.capture_microbatch():
                        forward(stack, torch.randn(MB, SEQ, HID, generator=gen).cuda())
                if streamed:
                    ev = torch.cuda.Event()
                    ev.record()
                    core = opt._core
                    if step == 0:
                        with pytest.raises(ValueError):
                            core.begin(ready=[("d", 1, 3, ev)])           # does not start at the first statistic
                    core.begin(ready=[("f", 0, 1, ev), ("d", 0, 2, ev), ("f", 1, 2, ev), ("d", 2, 5, ev), ("d", 5, 6, ev)])
                else:
                    opt.begin()
                for b in stack:
                    for p in b.parameters():
                        if p.ndim == 2:
                            p.grad = (torch.randn(p.shape, generator=gen) * 1e-3).cuda()
                opt.step()
            torch.cuda.synchronize()
            return [p.detach().cpu().clone() for b in stack for p in b.parameters() if p.ndim == 2]
        finally:
            opt.close()

    plain, streamed = run(False), run(True)
    for a, b in zip(plain, streamed):
        assert torch.equal(a, b)


def test_direct_construction_from_a_model_that_owns_its_row_buffers(fast):
    """FastTonerCore.from_blocks: a trainer-side model with `input_rows_*` buffers and `body.blocks.<i>.<role>.weight`
    names, the reference's argument namespace, rows written by capture_recomputed-style code straight into the
    (rebound) buffers, lr set on param_groups.  Must give the same weights as FastMuonT fed the same rows."""
    from types import SimpleNamespace
    from toner_b200 import ops
    from toner_b200.fast.engine import FastTonerCore
    from toner_b200.synthetic import make_stack
    dev = torch.device("cuda")
    positions = orc.sample_positions(SEQ, 8, 4)
    rows = ACC * MB * len(positions)
    gen = torch.Generator().manual_seed(31)
    xs = [torch.randn(MB, SEQ, HID, generator=gen) for _ in range(2 * ACC)]
    grads_seed = 77

    def grads_for(stack, step):
        g = torch.Generator().manual_seed(grads_seed + step)
        for b in stack:
            for p in b.parameters():
                if p.ndim == 2:
                    p.grad = (torch.randn(p.shape, generator=g) * 1e-3).cuda()

    # reference run through the adapter, recording the rows each statistic saw
    stack, opt = make(fast, "llama", "muont", ns_steps=2)
    seen = []
    try:
        for step in range(2):
            for mb in range(ACC):
                with opt.capture_microbatch():
                    forward(stack, xs[step * ACC + mb].cuda())
            core = opt._core
            seen.append((core.groups["d"].rows_buf.clone(), core.groups["f"].rows_buf.clone()))
            opt.begin()
            grads_for(stack, step)
            opt.step()
        want = [p.detach().cpu().clone() for b in stack for p in b.parameters() if p.ndim == 2]
    finally:
        opt.close()

    # the same through the direct seam
    stack2 = make_stack("llama", LAYERS, HID, MLP, dev, seed=0)
    blocks = []
    for b in stack2:
        holder = torch.nn.Module()
        for k, w in (("attn", HID), ("o", HID), ("mlp", HID), ("down", MLP)):
            holder.register_buffer(f"input_rows_{k}", torch.zeros(rows, w, dtype=torch.bfloat16, device=dev), persistent=False)
        blocks.append(holder)
    named = {f"body.blocks.{i}.{r}.weight": getattr(b, r).weight for i, b in enumerate(stack2)
             for r in ("q", "k", "v", "o", "gate", "up", "down")}
    named["body.emb.weight"] = torch.zeros(8, 8, device=dev)              # not a block matrix: ignored
    args = SimpleNamespace(toner_decay=0.95, toner_split=True, toner_alpha=0.5, toner_alpha_in=0.5, toner_alpha_out=0.125,
                           wd=0.1, beta1=0.9, beta2=0.98, eps=1e-15, muon_momentum=0.95, muon_nesterov=True,
                           muon_ns_steps=2, muon_eps=1e-5, muon_ns_mode="tpu", toner_lr_mult=1.0)
    core = FastTonerCore.from_blocks(blocks, named, "muont", hid=HID, mlp=MLP, rows_total=rows, args=args, world=1, rank=0,
                                     device=dev)
    assert blocks[0].input_rows_attn.data_ptr() == core.groups["d"].rows_buf[0].data_ptr()
    core.param_groups[0]["lr"] = 0.02
    for step in range(2):
        d_rows, f_rows = seen[step]
        for i, holder in enumerate(blocks):
            for j, k in enumerate(("attn", "o", "mlp")):
                getattr(holder, f"input_rows_{k}").copy_(d_rows[3 * i + j])
            holder.input_rows_down.copy_(f_rows[i])
        core.begin()
        grads_for(stack2, step)
        core.step()
    core.side.synchronize()
    core.pool.shutdown(wait=True)
    ops.assert_healthy()
    got = [p.detach().cpu().clone() for b in stack2 for p in b.parameters() if p.ndim == 2]
    for a, b in zip(got, want):
        assert torch.equal(a, b)
