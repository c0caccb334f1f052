"""Sharding a batch of independent structures over the GPUs of one node.

Structures never interact (every index of the batched graph is offset per
structure and the energy is pooled per structure), so the path shards by
structure with no data-path collective; the only exchange is a gather of the
results.  One process per GPU (``torch.distributed``; NCCL on GPUs, gloo in the
CPU tests).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def predicted_cost(numbers, lattice, cutoff=6.0, line_cutoff=4.0) -> float:
    """Relative cost of one structure: the work is dominated by the triplet rows, which grow as
    n_atoms * (bonds shorter than the line cutoff per atom)^2, plus a term for the directed edges."""
    n = len(numbers)
    rho = n / abs(float(np.linalg.det(np.asarray(lattice, dtype=np.float64))))
    short = 4.0 / 3.0 * np.pi * line_cutoff ** 3 * rho
    edges = 4.0 / 3.0 * np.pi * cutoff ** 3 * rho
    return float(n * (1.1 * short * short + edges))


def shard_by_cost(costs, world_size: int) -> list[list[int]]:
    """Greedy longest-processing-time assignment: returns the structure indices of every rank
    (each list ascending).  Deterministic, identical on every rank."""
    costs = np.asarray(costs, dtype=np.float64)
    order = np.argsort(-costs, kind="stable")
    load = np.zeros(world_size)
    shards: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = int(np.argmin(load))
        shards[r].append(int(i))
        load[r] += costs[i]
    return [sorted(s) for s in shards]


def gather_results(local: dict, indices: list[int], n_total: int, group=None) -> dict | None:
    """Gather per-structure results to rank 0 and put them back in the original order.

    ``local``: ``e`` [b] tensor, optional ``f`` / ``m`` lists of per-structure tensors, ``s`` list of [3,3].
    Returns on rank 0 a dict of lists indexed by global structure id; None elsewhere."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    payload = {"idx": list(indices)}
    for k, v in local.items():
        if k in ("e", "ref_energy") and torch.is_tensor(v):
            payload[k] = v.detach().cpu()
        elif k in ("f", "s", "m"):
            payload[k] = [t.detach().cpu() for t in v]
    if world == 1:
        gathered = [payload]
    else:
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(payload, gathered, dst=0, group=group)
    if rank != 0:
        return None
    out: dict = {}
    for p in gathered:
        for j, gi in enumerate(p["idx"]):
            for k, v in p.items():
                if k == "idx":
                    continue
                out.setdefault(k, [None] * n_total)[gi] = v[j]
    return out
