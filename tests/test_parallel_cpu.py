"""CPU: sharding planner and result gather over world_size-2 gloo ranks (host logic of the multi-GPU path)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from matris_b200 import workloads
from matris_b200.parallel import gather_results, predicted_cost, shard_by_cost


def test_shard_by_cost_balances_and_covers():
    crystals = workloads.random_crystals(64, seed=3)
    costs = [predicted_cost(c.numbers, c.lattice) for c in crystals]
    for world in (1, 2, 4, 8):
        shards = shard_by_cost(costs, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        load = np.array([sum(costs[i] for i in s) for s in shards])
        assert load.max() <= 1.25 * load.mean()
    assert shard_by_cost(costs, 2) == shard_by_cost(costs, 2)  # deterministic: identical on every rank


def test_predicted_cost_tracks_triplets():
    from oracle import pipeline
    crystals = workloads.random_crystals(12, seed=8)
    trip = np.array([len(pipeline.graph_from_arrays(c.numbers, c.cart, c.lattice)["line_graph"]) for c in crystals])
    cost = np.array([predicted_cost(c.numbers, c.lattice) for c in crystals])
    assert np.corrcoef(trip, cost)[0, 1] > 0.9


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_total, out_path):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sizes = [3 + (i % 4) for i in range(n_total)]
    shards = shard_by_cost([float(s) for s in sizes], world)
    mine = shards[rank]
    # fake per-rank results that encode the global structure id
    local = {"e": torch.tensor([float(i) for i in mine]),
             "f": [torch.full((sizes[i], 3), float(i)) for i in mine],
             "s": [torch.eye(3) * i for i in mine]}
    merged = gather_results(local, mine, n_total)
    if rank == 0:
        ok = all(float(merged["e"][i]) == i and merged["f"][i].shape == (sizes[i], 3)
                 and float(merged["f"][i][0, 0]) == i and float(merged["s"][i][1, 1]) == i for i in range(n_total))
        torch.save({"ok": ok}, out_path)
    else:
        assert merged is None
    dist.barrier()
    dist.destroy_process_group()


def test_gather_results_two_ranks(tmp_path):
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), 11, out), nprocs=2, join=True)
    assert torch.load(out)["ok"]


def test_gather_results_single_process():
    merged = gather_results({"e": torch.tensor([1.0, 2.0]), "m": [torch.zeros(2), torch.ones(3)]}, [1, 0], 2)
    assert float(merged["e"][1]) == 1.0 and float(merged["e"][0]) == 2.0 and merged["m"][0].shape == (3,)
