"""Layer-sharded engine on two GPUs (NCCL) against the same step on one GPU.

Each rank captures its own microbatches (its share of the tokens), owns half of the layers, and after the step every
rank must hold the weights a single process gets from all microbatches.  Two things differ between the runs: the order
of FP32 additions in the statistic (packed partial Grams summed by reduce-scatter instead of one SYRK with a fused EMA)
and the Newton schedule of the factor engine, whose spectrum bound is taken over the statistics a rank owns.  Both
stay inside the factor engine's accuracy (1e-4 on a factor), hence the bound on the weights below.
Needs two visible GPUs; skipped otherwise."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu
HID, MLP, SEQ, MB, ACC, LAYERS = 256, 512, 256, 2, 2, 2   # 704 sampled rows: full-rank statistics


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _microbatch(rank, mb_index):
    g = torch.Generator().manual_seed(1000 + 17 * rank + mb_index)
    return torch.randn(MB, SEQ, HID, generator=g)


def _run(kind, world, rank, device, microbatches, steps=2, first_step=0, resume=None, save_to=None, streamed=False,
         layers=LAYERS, owner_weights=None, snapshot_to=None):
    """One process's part of optimizer steps first_step .. steps-1; returns its weights.  `resume` = (weights,
    checkpoint) continues a run saved after `first_step` steps; `save_to` writes rank zero's checkpoint at the end."""
    import toner_b200.fast as fast
    from toner_b200.synthetic import make_stack
    stack = make_stack("llama", layers, HID, MLP, device, seed=0)
    cls = fast.FastMuonT if kind == "muont" else fast.FastAdamT
    extra = dict(ns_steps=2) if kind == "muont" else dict(betas=(0.9, 0.95), eps=1e-4)
    opt = cls([fast.ProjectionBlock.from_module(b) for b in stack], 0.02 if kind == "muont" else 2e-3, weight_decay=0.1,
              micro_batch_size=MB, sequence_length=SEQ, accumulation_steps=len(microbatches), statistic_head=32,
              statistic_stride=4, owner_weights=owner_weights, **extra)
    try:
        if resume is not None:
            weights, ckpt = resume
            with torch.no_grad():
                for p, w in zip([p for b in stack for p in b.parameters() if p.ndim == 2], weights):
                    p.copy_(w)
            opt.load_state_dict(ckpt)
        for step in range(first_step, steps):
            for x in microbatches:
                with opt.capture_microbatch():
                    with torch.autocast("cuda", dtype=torch.bfloat16):
                        h = (x + step).to(device)
                        for b in stack:
                            h = b(h)
            if streamed:    # rows "arrive" group by group: wide statistics first, then the hidden-width ones in two slices
                ev = torch.cuda.Event()
                ev.record()
                opt._core.begin(ready=[("f", 0, layers, ev), ("d", 0, 2, ev), ("d", 2, 3 * layers, ev)])
            else:
                opt.begin()
            g = torch.Generator().manual_seed(77 + step)     # gradients arrive already synchronised
            for b in stack:
                for p in b.parameters():
                    if p.ndim == 2:
                        p.grad = (torch.randn(p.shape, generator=g) * 1e-3).to(device)
            opt.step()
        torch.cuda.synchronize(device)
        from toner_b200 import ops
        ops.assert_healthy()
        if snapshot_to is not None:
            snap = opt._core.snapshot([0, layers - 1])       # collective; the statistics come back on rank zero
            if rank == 0:
                torch.save({"snapshot": snap, "counts": opt._core.layer_counts}, snapshot_to)
        if save_to is not None:
            ckpt = opt.state_dict()                          # collective; the checkpoint comes back on rank zero
            if rank == 0:
                torch.save(ckpt, save_to)
        return [p.detach().cpu().clone() for b in stack for p in b.parameters() if p.ndim == 2]
    finally:
        opt.close()


def _worker(rank, world, port, kind, out_dir, steps=2, save=False, streamed=False):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        weights = _run(kind, world, rank, device, [_microbatch(rank, i) for i in range(ACC)], steps=steps,
                       save_to=os.path.join(out_dir, f"ckpt{steps}.pt") if save else None, streamed=streamed)
        torch.save(weights, os.path.join(out_dir, f"w{rank}_{steps}{'s' if streamed else ''}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["muont", "adamt"])
def test_two_ranks_match_one_process(tmp_path, kind):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), kind, str(tmp_path)), nprocs=world, join=True)
    torch.cuda.set_device(0)
    single = _run(kind, 1, 0, torch.device("cuda", 0), [_microbatch(r, i) for r in range(world) for i in range(ACC)])
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"w{r}_2.pt"))
        assert len(got) == len(single)
        for a, b in zip(got, single):
            rel = (a - b).norm().item() / b.norm().item()
            assert rel < 3e-4, (kind, r, rel)


def test_checkpoint_saved_by_two_ranks_resumes_on_one(tmp_path):
    """A toner.fast.v3 checkpoint gathered from two ranks after two steps is loaded into a single process, which
    takes the third step with all microbatches; the result must match three steps on two ranks."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, kind = 2, "muont"
    mp.spawn(_worker, args=(world, _free_port(), kind, str(tmp_path), 2, True), nprocs=world, join=True)
    mp.spawn(_worker, args=(world, _free_port(), kind, str(tmp_path), 3, False), nprocs=world, join=True)
    ckpt = torch.load(os.path.join(tmp_path, "ckpt2.pt"), weights_only=False)
    assert ckpt["format"] == "toner.fast.v3" and ckpt["core"]["t"] == 2
    after_two = torch.load(os.path.join(tmp_path, "w0_2.pt"))
    torch.cuda.set_device(0)
    resumed = _run(kind, 1, 0, torch.device("cuda", 0), [_microbatch(r, i) for r in range(world) for i in range(ACC)],
                   steps=3, first_step=2, resume=(after_two, ckpt))
    want = torch.load(os.path.join(tmp_path, "w1_3.pt"))
    for a, b in zip(resumed, want):
        rel = (a - b).norm().item() / b.norm().item()
        assert rel < 3e-4, rel


def test_streamed_rows_on_two_ranks_change_nothing(tmp_path):
    """begin(ready=...) with several ranks: each group's SYRK / reduce-scatter / factors start when that group's rows
    are in.  Statistics are independent, so the weights are bit-identical to the plain order."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), "muont", str(tmp_path), 2, False, False), nprocs=world, join=True)
    mp.spawn(_worker, args=(world, _free_port(), "muont", str(tmp_path), 2, False, True), nprocs=world, join=True)
    for r in range(world):
        plain = torch.load(os.path.join(tmp_path, f"w{r}_2.pt"))
        streamed = torch.load(os.path.join(tmp_path, f"w{r}_2s.pt"))
        assert all(torch.equal(a, b) for a, b in zip(plain, streamed))


def _uneven_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        weights = _run("muont", world, rank, device, [_microbatch(rank, i) for i in range(ACC)], layers=4,
                       owner_weights=[1.0, 3.0], save_to=os.path.join(out_dir, "ckpt_uneven.pt"),
                       snapshot_to=os.path.join(out_dir, "snap.pt"))
        torch.save(weights, os.path.join(out_dir, f"u{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_uneven_layer_ownership_matches_one_process(tmp_path):
    """owner_weights (1, 3) on four layers: rank 0 owns one layer, rank 1 three.  The statistics reach their owners
    through the uneven form of reduce-scatter, the changes come back through the uneven all-gather, and every rank
    ends with the weights one process computes from all microbatches; the gathered checkpoint and the statistics
    snapshot name every layer."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_uneven_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    torch.cuda.set_device(0)
    single = _run("muont", 1, 0, torch.device("cuda", 0), [_microbatch(r, i) for r in range(world) for i in range(ACC)],
                  layers=4)
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"u{r}.pt"))
        for a, b in zip(got, single):
            rel = (a - b).norm().item() / b.norm().item()
            assert rel < 3e-4, (r, rel)
    snap = torch.load(os.path.join(tmp_path, "snap.pt"), weights_only=False)
    assert snap["counts"] == [1, 3]
    assert set(snap["snapshot"]) == {f"{i}.{k}" for i in (0, 3) for k in ("attn", "o", "mlp", "down")}
    ckpt = torch.load(os.path.join(tmp_path, "ckpt_uneven.pt"), weights_only=False)
    assert len(ckpt["core"]["ema"]) == 16 and len(ckpt["core"]["moments"]) == 28
    # the snapshot is the bias-corrected statistic: EMA / weight
    for key, value in snap["snapshot"].items():
        assert torch.allclose(value, ckpt["core"]["ema"][key] / ckpt["core"]["weight"], rtol=1e-6, atol=0)
