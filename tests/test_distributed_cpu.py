"""Two gloo ranks on CPU: the index maps the NCCL path relies on (chunked statistic reduction to owners,
all-gather of per-role changes in layer order) give the same result as one process."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import toner_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from toner_b200.fast.engine import chunk_members, chunk_plan, layer_counts
        layers, n, rows = 4, 16, 24
        counts = layer_counts(layers, world)
        per = 3 * counts[rank]                       # three hidden-width statistics per owned layer
        k_all = 3 * layers
        g = torch.Generator().manual_seed(100 + rank)  # every rank has its own rows of every statistic
        x = torch.randn(k_all, rows, n, generator=g).to(torch.bfloat16)
        partial = torch.stack([orc.pack_upper(orc.gram(x[s])) for s in range(k_all)])
        chunks = chunk_plan(per, 2)
        cs = per // chunks
        owned = torch.empty(per, partial.shape[1])
        for c in range(chunks):
            send = partial[chunk_members(world, per, chunks, c)].clone()   # (world*cs, tri) in (rank, j) order
            dist.all_reduce(send)                                           # stand-in for reduce-scatter on gloo
            owned[c * cs:(c + 1) * cs] = send[rank * cs:(rank + 1) * cs]
        # all-gather of per-rank stacks in rank order == layer order
        delta = torch.full((counts[rank], 2, 2), float(rank)) + torch.arange(counts[rank]).view(-1, 1, 1) * 0.1
        gathered = [torch.empty_like(delta) for _ in range(world)]
        dist.all_gather(gathered, delta)
        torch.save({"owned": owned, "gathered": torch.cat(gathered), "lo": rank * per}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reduce_to_owners_and_gather_in_layer_order(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    layers, n, rows = 4, 16, 24
    k_all = 3 * layers
    xs = [torch.randn(k_all, rows, n, generator=torch.Generator().manual_seed(100 + r)).to(torch.bfloat16) for r in range(world)]
    total = torch.stack([sum(orc.pack_upper(orc.gram(x[s])) for x in xs) for s in range(k_all)])
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        per = got["owned"].shape[0]
        assert torch.allclose(got["owned"], total[got["lo"]: got["lo"] + per], rtol=1e-6, atol=1e-5)
        # layer l is owned by rank l // 2 at position l % 2: gathered row l must carry that signature
        want = torch.tensor([0.0, 0.1, 1.0, 1.1]).view(-1, 1, 1).expand(-1, 2, 2)
        assert torch.allclose(got["gathered"], want)


def _flat_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from toner_b200.fast.engine import flat_layout, gathered_block, layer_counts
        layers = 4
        per = layer_counts(layers, world)[rank]
        shapes = {"q": (per, 2, 3), "up": (per, 4, 3), "down": (per, 3, 4)}     # roles of different sizes
        sizes = [int(torch.tensor(s).prod()) for s in shapes.values()]
        offsets = flat_layout(sizes)
        flat = torch.empty(sum(sizes))
        for (role, shape), off, size in zip(shapes.items(), offsets, sizes):
            # value encodes (role, global layer): what every rank must find after the exchange
            stack = torch.stack([torch.full(shape[1:], 100.0 * list(shapes).index(role) + rank * per + j) for j in range(per)])
            flat[off: off + size] = stack.reshape(-1)
        gathered = torch.empty(world, sum(sizes))
        dist.all_gather_into_tensor(gathered.view(-1), flat)   # gloo wants the concatenated form
        found = {}
        for (role, shape), off, size in zip(shapes.items(), offsets, sizes):
            for r in range(world):
                block = gathered_block(gathered, r, off, size, shape)
                for j in range(per):
                    found[(role, r * per + j)] = block[j].unique().tolist()
        torch.save(found, os.path.join(out_dir, f"f{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_flat_exchange_buffer_maps_back_to_role_and_layer(tmp_path):
    world = 2
    mp.spawn(_flat_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        found = torch.load(os.path.join(tmp_path, f"f{r}.pt"))
        for (role, layer), vals in found.items():
            assert vals == [100.0 * ["q", "up", "down"].index(role) + layer]
