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


def _layout(atoms_per_structure, indices, keys):
    """Offsets of one rank's results inside its flat float32 buffer: e [b] | ref_energy [b] | s [b,9] | f [n,3] | m [n]
    (only the keys present), b = structures of the rank, n = their atoms."""
    b = len(indices)
    n = int(sum(atoms_per_structure[i] for i in indices))
    sizes = {"e": b, "ref_energy": b, "s": 9 * b, "f": 3 * n, "m": n}
    off, o = {}, 0
    for k in ("e", "ref_energy", "s", "f", "m"):
        if k in keys:
            off[k] = (o, sizes[k])
            o += sizes[k]
    return off, o


def evaluate(model, structures, task: str = "efsm", group=None, dst: int = 0) -> dict | None:
    """Evaluate one list of structures on all ranks of ``group``: the sharded form of ``model.predict``.

    Every rank passes the SAME list (the usual torchrun pattern: each rank runs the same script).  The structures
    are assigned to ranks by predicted cost (``shard_by_cost``), each rank evaluates its share with
    ``model.predict`` on its own GPU, and energies, forces, stresses and magnetic moments are gathered to rank
    ``dst`` with ONE collective on a flat float32 buffer per rank (NCCL on GPUs, gloo on CPU; about 16 bytes per
    atom).  Returns on ``dst`` the dictionary ``model.predict`` would return for the whole list (``e`` and
    ``ref_energy`` [B] tensors, ``f`` / ``m`` lists of per-structure tensors, ``s`` list of [3,3], ``atoms_per_graph``),
    in the original order, on the model's device; ``None`` on the other ranks.  The reference has no counterpart:
    its only distributed line is a rank-0 print guard (matris/model/model.py:180)."""
    from .graph import as_arrays
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    arrays = [as_arrays(s) for s in structures]
    n_total = len(arrays)
    if n_total == 0:
        raise ValueError("no structures")
    atoms = [len(a[0]) for a in arrays]
    cut = float(getattr(model, "config", {}).get("pairwise_cutoff", 6.0))
    lcut = float(getattr(model, "config", {}).get("three_body_cutoff", 4.0))
    shards = shard_by_cost([predicted_cost(a[0], a[2], cut, lcut) for a in arrays], world)
    mine = shards[rank]
    keys = ["e", "ref_energy"] + [k for k in ("s", "f", "m") if k in task]
    device = torch.device(getattr(model, "device", "cpu"))
    layouts = [_layout(atoms, sh, keys) for sh in shards]
    width = max(1, max(total for _, total in layouts))  # ranks pad to the longest buffer: one equal-size gather
    buf = torch.zeros(width, dtype=torch.float32, device=device)
    if mine:
        out = model.predict([structures[i] for i in mine], task)
        off, _ = layouts[rank]
        ref = out["ref_energy"]
        if not torch.is_tensor(ref):
            ref = torch.full((len(mine),), float(ref), device=device)
        flat = {"e": out["e"], "ref_energy": ref}
        if "s" in keys:
            flat["s"] = torch.stack(list(out["s"]))
        if "f" in keys:
            flat["f"] = torch.cat(list(out["f"]))
        if "m" in keys:
            flat["m"] = torch.cat(list(out["m"]))
        for k, (o, n) in off.items():
            buf[o:o + n] = flat[k].reshape(-1).to(device=device, dtype=torch.float32)
    if world > 1:
        parts = [torch.empty_like(buf) for _ in range(world)] if rank == dst else None
        dist.gather(buf, parts, dst=dst, group=group)
    else:
        parts = [buf]
    if rank != dst:
        return None
    res: dict = {k: [None] * n_total for k in keys}
    for r, sh in enumerate(shards):
        off, _ = layouts[r]
        p = parts[r]
        a0 = 0
        for j, gi in enumerate(sh):
            na = atoms[gi]
            res["e"][gi] = p[off["e"][0] + j]
            res["ref_energy"][gi] = p[off["ref_energy"][0] + j]
            if "s" in off:
                res["s"][gi] = p[off["s"][0] + 9 * j:off["s"][0] + 9 * j + 9].view(3, 3)
            if "f" in off:
                res["f"][gi] = p[off["f"][0] + 3 * a0:off["f"][0] + 3 * (a0 + na)].view(na, 3)
            if "m" in off:
                res["m"][gi] = p[off["m"][0] + a0:off["m"][0] + a0 + na]
            a0 += na
    res["e"], res["ref_energy"] = torch.stack(res["e"]), torch.stack(res["ref_energy"])
    if "f" in res:
        res["f"] = tuple(res["f"])
    res["atoms_per_graph"] = torch.tensor(atoms, dtype=torch.int32, device=device)
    res["shards"] = shards
    return res


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
