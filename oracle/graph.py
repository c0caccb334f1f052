"""Restatement of the reference's bond-graph / line-graph construction
(test infrastructure only).

Follows
  * matris/graph/fast_converter_libraries/create_graph.c:100-219 (and its legacy
    twin Graph.add_edge, matris/graph/radiusgraph.py:298-386): sequential scan
    of directed edges, pairing (i,j,n) with an earlier (j,i,-n);
  * Graph.adjacency_list / undirected2directed (radiusgraph.py:388-410, 489-496);
  * Graph.line_graph_adjacency_list (radiusgraph.py:412-487).

Two implementations are given: ``*_sequential`` mirrors the reference's loop
structure literally (pure Python, small inputs); ``build_graph`` /
``line_graph`` are vectorised closed forms of the same result.  Both are
pinned against the reference's own classes in tests/golden.
"""
from __future__ import annotations

import numpy as np


# --------------------------------------------------------------------- sequential
def build_graph_sequential(center, neighbor, image):
    """Literal restatement of create_graph.c's scan.  Returns (d2u, u2d)."""
    groups: dict[tuple[int, int], list[int]] = {}  # unordered node pair -> undirected ids
    first_de: list[int] = []                        # undirected id -> first directed edge
    d2u = np.empty(len(center), dtype=np.int64)
    for k in range(len(center)):
        i, j = int(center[k]), int(neighbor[k])
        key = (i, j) if i <= j else (j, i)
        found = False
        for u in groups.get(key, ()):  # create_graph.c:170-182
            k0 = first_de[u]
            if (center[k0] == j and neighbor[k0] == i
                    and image[k0][0] == -image[k][0] and image[k0][1] == -image[k][1]
                    and image[k0][2] == -image[k][2]):
                d2u[k] = u
                found = True
                break
        if not found:
            u = len(first_de)
            first_de.append(k)
            groups.setdefault(key, []).append(u)
            d2u[k] = u
    return d2u, np.asarray(first_de, dtype=np.int64)


def line_graph_sequential(center, neighbor, distance, d2u, u2d, cutoff):
    """Literal restatement of Graph.line_graph_adjacency_list."""
    n_u = len(u2d)
    second = np.full(n_u, -1, dtype=np.int64)
    for k in range(len(center)):
        if u2d[d2u[k]] != k:
            second[d2u[k]] = k
    # per-node neighbour map in insertion order (create_graph.c:382-408)
    nbrs: dict[int, dict[int, list[int]]] = {}
    for k in range(len(center)):
        nbrs.setdefault(int(center[k]), {}).setdefault(int(neighbor[k]), []).append(k)
    rows = []
    for u in range(n_u):
        k0 = int(u2d[u])
        if distance[k0] > cutoff:           # radiusgraph.py:450 (skip only if '>')
            continue
        if second[u] < 0:
            raise AssertionError("Did not find 2 Directed_edges !!!")
        ends = (int(center[k0]), int(neighbor[k0]))
        for c, de in zip(ends, (k0, int(second[u]))):
            for group in nbrs.get(c, {}).values():
                for b in group:
                    if b == de:
                        continue
                    if distance[b] < cutoff:  # strict (radiusgraph.py:477)
                        rows.append((c, u, de, int(d2u[b]), b))
    return np.asarray(rows, dtype=np.int64).reshape(-1, 5)


# --------------------------------------------------------------------- vectorised
def _edge_keys(center, neighbor, image):
    im = np.asarray(image, dtype=np.int64)
    off = int(np.abs(im).max()) + 1 if im.size else 1
    base = 2 * off + 1
    n_atoms = int(max(center.max(), neighbor.max())) + 1 if len(center) else 1

    def pack(a, b, m):
        return (((a * n_atoms + b) * base + (m[:, 0] + off)) * base + (m[:, 1] + off)) * base + (m[:, 2] + off)

    return pack(center, neighbor, im), pack(neighbor, center, -im)


def reverse_edge_index(center, neighbor, image):
    """rev[k] = index of the directed edge (j,i,-n) for k = (i,j,n); -1 if missing."""
    center = np.asarray(center, dtype=np.int64)
    neighbor = np.asarray(neighbor, dtype=np.int64)
    fwd, bwd = _edge_keys(center, neighbor, image)
    order = np.argsort(fwd, kind="stable")
    pos = np.searchsorted(fwd[order], bwd)
    pos = np.clip(pos, 0, max(len(fwd) - 1, 0))
    rev = order[pos] if len(fwd) else np.zeros(0, dtype=np.int64)
    ok = fwd[rev] == bwd if len(fwd) else np.zeros(0, dtype=bool)
    return np.where(ok, rev, -1)


def build_graph(center, neighbor, image):
    """Closed form of the sequential scan: the undirected edge of k is the pair
    {k, rev[k]}, numbered by order of its first-seen member.  Returns (d2u, u2d, rev)."""
    rev = reverse_edge_index(center, neighbor, image)
    k = np.arange(len(rev), dtype=np.int64)
    first = np.where((rev >= 0) & (rev < k), rev, k)
    is_first = first == k
    u_of_first = np.cumsum(is_first) - 1
    d2u = u_of_first[first]
    u2d = k[is_first]
    return d2u, u2d, rev


def line_graph(center, neighbor, distance, d2u, u2d, rev, cutoff):
    """Vectorised Graph.line_graph_adjacency_list (same rows, same order)."""
    center = np.asarray(center, dtype=np.int64)
    neighbor = np.asarray(neighbor, dtype=np.int64)
    distance = np.asarray(distance, dtype=np.float64)
    n_e = len(center)
    if n_e == 0:
        return np.zeros((0, 5), dtype=np.int64)
    if (rev < 0).any():
        raise AssertionError("Did not find 2 Directed_edges !!!")
    # out-edge order at each centre: groups by neighbour in first-appearance order, then edge index
    k = np.arange(n_e, dtype=np.int64)
    pair = center * (int(neighbor.max()) + 1) + neighbor
    _, inv = np.unique(pair, return_inverse=True)
    first_of_pair = np.full(inv.max() + 1, n_e, dtype=np.int64)
    np.minimum.at(first_of_pair, inv, k)
    grp = first_of_pair[inv]
    order = np.lexsort((k, grp, center))
    sc = center[order]
    n_atoms = int(max(center.max(), neighbor.max())) + 1
    start = np.searchsorted(sc, np.arange(n_atoms))
    stop = np.searchsorted(sc, np.arange(n_atoms), side="right")
    short = distance < cutoff                    # candidate "other" bonds
    # the (u, side) slots in emission order
    us = np.nonzero(distance[u2d] <= cutoff)[0]
    de = np.stack([u2d[us], rev[u2d[us]]], axis=1).reshape(-1)      # DE per slot
    uu = np.repeat(us, 2)
    cc = center[de]
    cnt = stop[cc] - start[cc]
    tot = int(cnt.sum())
    slot = np.repeat(np.arange(len(de)), cnt)
    within = np.arange(tot) - np.repeat(np.cumsum(cnt) - cnt, cnt)
    b = order[start[cc][slot] + within]
    keep = (b != de[slot]) & short[b]
    slot, b = slot[keep], b[keep]
    return np.stack([cc[slot], uu[slot], de[slot], d2u[b], b], axis=1)
