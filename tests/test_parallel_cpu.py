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


class _FakeModel:
    """Stands in for MatRIS on CPU ranks: results that encode (structure, atom) through the atomic numbers."""
    device = "cpu"
    config = {"pairwise_cutoff": 6.0, "three_body_cutoff": 4.0}

    def predict(self, structures, task):
        out = {"e": torch.tensor([float(np.sum(s.numbers)) for s in structures]),
               "ref_energy": torch.tensor([float(len(s.numbers)) for s in structures])}
        if "f" in task:
            out["f"] = tuple(torch.tensor(s.cart, dtype=torch.float32) * 2 for s in structures)
        if "s" in task:
            out["s"] = [torch.tensor(s.lattice, dtype=torch.float32) for s in structures]
        if "m" in task:
            out["m"] = [torch.tensor(s.numbers, dtype=torch.float32) for s in structures]
        return out


def _check_sharded(res, crystals, task):
    assert torch.equal(res["e"], torch.tensor([float(np.sum(c.numbers)) for c in crystals]))
    assert torch.equal(res["ref_energy"], torch.tensor([float(len(c.numbers)) for c in crystals]))
    assert list(res["atoms_per_graph"]) == [len(c.numbers) for c in crystals]
    for i, c in enumerate(crystals):
        if "f" in task:
            assert torch.equal(res["f"][i], torch.tensor(c.cart, dtype=torch.float32) * 2)
        if "s" in task:
            assert torch.equal(res["s"][i], torch.tensor(c.lattice, dtype=torch.float32))
        if "m" in task:
            assert torch.equal(res["m"][i], torch.tensor(c.numbers, dtype=torch.float32))
    assert ("m" in res) == ("m" in task)


def _eval_worker(rank, world, port, task, out_path):
    from matris_b200.parallel import evaluate
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    crystals = workloads.random_crystals(7, seed=4)
    res = evaluate(_FakeModel(), crystals, task)
    if rank == 0:
        _check_sharded(res, crystals, task)
        covered = sorted(i for s in res["shards"] for i in s)
        torch.save({"ok": covered == list(range(7)), "nonempty": all(len(s) > 0 for s in res["shards"])}, out_path)
    else:
        assert res is None
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("task", ["efsm", "ef"])
def test_sharded_evaluate_two_ranks(tmp_path, task):
    """The sharded form of predict(): cost-balanced shards, one flat gather, results back in the original order."""
    out = str(tmp_path / "r0.pt")
    mp.spawn(_eval_worker, args=(2, _free_port(), task, out), nprocs=2, join=True)
    got = torch.load(out)
    assert got["ok"] and got["nonempty"]


def test_sharded_evaluate_single_process_and_more_ranks_than_structures(tmp_path):
    from matris_b200.parallel import evaluate
    crystals = workloads.random_crystals(3, seed=6)
    _check_sharded(evaluate(_FakeModel(), crystals, "efs"), crystals, "efs")
    out = str(tmp_path / "r0.pt")
    mp.spawn(_few_worker, args=(4, _free_port(), out), nprocs=4, join=True)
    assert torch.load(out)["ok"]


def _few_worker(rank, world, port, out_path):
    from matris_b200.parallel import evaluate
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    crystals = workloads.random_crystals(2, seed=6)  # two structures on four ranks: two ranks stay empty
    res = evaluate(_FakeModel(), crystals, "efsm")
    if rank == 0:
        _check_sharded(res, crystals, "efsm")
        torch.save({"ok": True}, out_path)
    dist.barrier()
    dist.destroy_process_group()
