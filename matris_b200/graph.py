"""Structure -> radius graph / bond graph / line graph on the GPU.

Host-side mirror of the reference's graph package: ``GraphConverter`` and
``RadiusGraph`` keep the names, arguments and error behaviour of
matris/graph/converter.py:22-129 and matris/graph/radiusgraph.py:17-113, but
the work (neighbour search, edge pairing, triplet enumeration; reference:
pymatgen's get_neighbor_list + create_graph.c + line_graph_adjacency_list) runs
in CUDA for a whole batch of structures at once through the C ABI.

Structures are accepted duck-typed: pymatgen-like (``.lattice.matrix``,
``.frac_coords``, sites with ``.specie.Z``), ASE-like (``get_cell``,
``get_positions``, ``get_atomic_numbers``) or plain ``(numbers, cart, lattice)``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Any, Sequence

import numpy as np
import torch
from torch import nn

from . import _lib

datatype = torch.float32


# ------------------------------------------------------------------ input handling
def as_arrays(structure) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Return (numbers int64 [N], cart float64 [N,3], lattice float64 [3,3])."""
    if hasattr(structure, "lattice") and hasattr(structure.lattice, "matrix"):  # pymatgen-like
        lattice = np.asarray(structure.lattice.matrix, dtype=np.float64)
        if hasattr(structure, "cart_coords"):
            cart = np.asarray(structure.cart_coords, dtype=np.float64)
        else:
            cart = np.asarray(structure.frac_coords, dtype=np.float64) @ lattice
        numbers = np.asarray([site.specie.Z for site in structure], dtype=np.int64)
    elif hasattr(structure, "get_positions"):  # ASE-like
        lattice = np.asarray(structure.get_cell(), dtype=np.float64).reshape(3, 3)
        cart = np.asarray(structure.get_positions(), dtype=np.float64)
        numbers = np.asarray(structure.get_atomic_numbers(), dtype=np.int64)
    elif hasattr(structure, "numbers") and hasattr(structure, "cart"):
        numbers, cart, lattice = structure.numbers, structure.cart, structure.lattice
    else:
        numbers, cart, lattice = structure
    numbers = np.ascontiguousarray(numbers, dtype=np.int64).reshape(-1)
    cart = np.ascontiguousarray(cart, dtype=np.float64).reshape(-1, 3)
    lattice = np.ascontiguousarray(lattice, dtype=np.float64).reshape(3, 3)
    if len(numbers) != len(cart):
        raise ValueError("numbers and positions differ in length")
    return numbers, cart, lattice


def _formula(numbers: np.ndarray) -> str:
    z, n = np.unique(numbers, return_counts=True)
    return " ".join(f"Z{int(a)}:{int(b)}" for a, b in zip(z, n))


def cell_grid(lattice: np.ndarray, n_atoms: np.ndarray, cutoff: float) -> tuple[np.ndarray, int]:
    """Per-structure cell grid for the neighbour search: cells per axis (each cell at
    least ``cutoff`` wide where the cell allows it), search half-width in cells, and
    the first global cell index.  lattice [B,3,3], n_atoms [B] -> int32 [B,8], n_cells."""
    a, b, c = lattice[:, 0], lattice[:, 1], lattice[:, 2]
    vol = np.abs(np.einsum("bi,bi->b", a, np.cross(b, c)))
    if (vol <= 0).any():
        raise ValueError("singular lattice")
    width = np.stack([vol / np.linalg.norm(np.cross(b, c), axis=1),
                      vol / np.linalg.norm(np.cross(c, a), axis=1),
                      vol / np.linalg.norm(np.cross(a, b), axis=1)], axis=1)
    g = np.maximum(1, np.floor(width / cutoff)).astype(np.int64)
    # never more cells than a few per atom (huge vacuum boxes would waste memory)
    cap = 4 * n_atoms.astype(np.int64) + 8
    for _ in range(64):
        over = g.prod(axis=1) > cap
        if not over.any():
            break
        k = g.argmax(axis=1)
        rows = np.nonzero(over)[0]
        g[rows, k[rows]] = np.maximum(1, g[rows, k[rows]] // 2)
    s = np.maximum(1, np.ceil(cutoff * g / width - 1e-12)).astype(np.int64)
    cells = g.prod(axis=1)
    base = np.concatenate([[0], np.cumsum(cells)[:-1]])
    grid = np.zeros((len(lattice), 8), dtype=np.int32)
    grid[:, 0:3], grid[:, 3:6], grid[:, 6] = g, s, base
    if cells.sum() > 2**31 - 2:
        raise ValueError("cell grid too large")
    return grid, int(cells.sum())


# ------------------------------------------------------------------ batched graph
class BatchedGraph:
    """Device-resident graph of a batch of structures (all indices global)."""

    def __init__(self):
        self.n_atoms = self.n_struct = self.n_edges = self.n_bonds = self.n_triplets = 0

    @property
    def device(self):
        return self.cart32.device

    def structure_slices(self):
        """Host index ranges of every structure: atoms, directed edges, bonds, triplets."""
        if getattr(self, "_slices", None) is None:
            ap = self.atom_ptr_host
            ep = self.edge_ptr.cpu().numpy()[ap]
            first = self.u2d.cpu().numpy()
            bp = np.searchsorted(first, ep)
            tp = self.trip_ptr.cpu().numpy()[bp]
            self._slices = (ap, ep, bp, tp)
        return self._slices


def _i32(n, device):
    return torch.empty(max(int(n), 1), dtype=torch.int32, device=device)


class HostBatch:
    """Host-side (NumPy, pinned where it is copied from) description of a batch of structures."""

    def __init__(self, numbers, carts, lattices, cutoff, pin=True):
        n_per = np.asarray([len(z) for z in numbers], dtype=np.int64)
        if len(n_per) == 0 or (n_per <= 0).any():
            raise ValueError("empty structure")
        self.n_struct, self.n_atoms = len(n_per), int(n_per.sum())
        self.atoms_per_graph = [int(x) for x in n_per]
        self.atom_ptr = np.concatenate([[0], np.cumsum(n_per)]).astype(np.int32)
        self.numbers = np.concatenate(numbers).astype(np.int64)
        self.cart = np.ascontiguousarray(np.concatenate(carts), dtype=np.float64)
        self.lattice = np.ascontiguousarray(np.stack(lattices), dtype=np.float64)
        inv = np.linalg.inv(self.lattice)
        self.atom_struct = np.repeat(np.arange(self.n_struct, dtype=np.int32), n_per)
        grid, self.n_cells = cell_grid(self.lattice, n_per, float(cutoff))
        # float32 model inputs exactly as the reference derives them (converter.py:82-83, processgraph.py:87)
        self.frac32 = np.einsum("ni,nij->nj", self.cart, inv[self.atom_struct]).astype(np.float32)
        lat32 = self.lattice.astype(np.float32)
        cart32 = np.einsum("ni,nij->nj", self.frac32, lat32[self.atom_struct]).astype(np.float32)
        vol32 = np.einsum("bi,bi->b", lat32[:, 0], np.cross(lat32[:, 1], lat32[:, 2])).astype(np.float32)
        # two staging buffers (one float64, one 32-bit) so that a batch is two host->device copies
        f64 = np.concatenate([self.cart.ravel(), self.lattice.ravel(), inv.ravel()])
        i32 = np.concatenate([self.atom_struct, self.atom_ptr, grid.ravel(), self.numbers.astype(np.int32),
                              cart32.ravel().view(np.int32), lat32.ravel().view(np.int32), vol32.view(np.int32)])
        self.f64, self.i32 = torch.from_numpy(f64), torch.from_numpy(i32)
        if pin and torch.cuda.is_available():
            self.f64, self.i32 = self.f64.pin_memory(), self.i32.pin_memory()
        self.h2d_bytes = self.f64.numel() * 8 + self.i32.numel() * 4


def upload(hb: HostBatch, cutoff, line_cutoff, device) -> BatchedGraph:
    """Copy a HostBatch to the device (two copies) and slice it into named tensors."""
    N, Bn = hb.n_atoms, hb.n_struct
    f64, i32 = hb.f64.to(device, non_blocking=True), hb.i32.to(device, non_blocking=True)
    g = BatchedGraph()
    g.n_atoms, g.n_struct, g.n_cells = N, Bn, hb.n_cells
    g.cutoff, g.line_cutoff = float(cutoff), float(line_cutoff)
    g.atoms_per_graph, g.atom_ptr_host, g.numbers_host = hb.atoms_per_graph, hb.atom_ptr, hb.numbers
    g.cart64_host, g.lattice64_host, g.frac32_host = hb.cart, hb.lattice, hb.frac32
    g.cart64, g.lattice64, g.inv_lattice64 = f64[:3 * N].view(N, 3), f64[3 * N:3 * N + 9 * Bn].view(Bn, 3, 3), \
        f64[3 * N + 9 * Bn:].view(Bn, 3, 3)
    o = 0

    def take(n, shape=None, as_float=False):
        nonlocal o
        t = i32[o:o + n]
        o += n
        if as_float:
            t = t.view(torch.float32)
        return t if shape is None else t.view(*shape)

    g.atom_struct, g.atom_ptr, g.grid, g.numbers = take(N), take(Bn + 1), take(8 * Bn, (Bn, 8)), take(N)
    g.cart32, g.lattice32, g.volume = take(3 * N, (N, 3), True), take(9 * Bn, (Bn, 3, 3), True), take(Bn, None, True)
    g._staging = (f64, i32)
    return g


def _capacity_estimate(g: BatchedGraph) -> tuple[int, int]:
    """First guess of the edge / triplet capacities from the number density of every structure (neighbours inside a
    sphere; triplets = ordered pairs of short bonds per atom), with a margin.  A guess that turns out too small costs
    one more launch with the exact sizes."""
    n = np.asarray(g.atoms_per_graph, dtype=np.float64)
    lat = g.lattice64_host
    vol = np.abs(np.einsum("bi,bi->b", lat[:, 0], np.cross(lat[:, 1], lat[:, 2])))
    rho = n / vol
    nbr = 4.0 / 3.0 * np.pi * g.cutoff ** 3 * rho
    short = 4.0 / 3.0 * np.pi * g.line_cutoff ** 3 * rho
    edges = float((n * nbr).sum())
    trips = float((n * short * np.maximum(short - 1.0, 0.0)).sum())
    return int(1.25 * edges) + 1024, int(1.5 * trips) + 4096


class _GraphBuffers:
    """Capacity buffers of one batch: outputs and scratch of mb_graph_build, kept across rebuilds of the same batch
    (an MD or relaxation loop rebuilds the graph of the same atoms every step)."""

    def __init__(self, g: BatchedGraph, cap_e: int, cap_t: int, device):
        lib = _lib.load()
        cap_e += cap_e & 1
        n_atoms, n_cells = g.n_atoms, g.n_cells
        self.cap_e, self.cap_t = cap_e, cap_t
        i64 = lambda n: torch.empty(max(int(n), 1), dtype=torch.int64, device=device)  # noqa: E731
        self.scratch = dict(
            cell_ptr=_i32(n_cells + 1, device), cell_fill=_i32(n_cells, device), cell_atoms=_i32(n_atoms, device),
            atom_cell=_i32(4 * n_atoms, device), atom_wrap=_i32(4 * n_atoms, device),
            scan_tmp=_i32(lib.mb_graph_scan_tmp_len(max(n_atoms, n_cells, cap_e)), device),
            key_unsorted=i64(cap_e), dist_unsorted=torch.empty(cap_e, dtype=torch.float64, device=device),
            key=i64(cap_e), atom_counts=_i32(2 * n_atoms, device), edge_rank=_i32(2 * cap_e + 2, device),
            bond_counts=_i32(cap_e + 4, device), edge_flag=torch.empty(cap_e, dtype=torch.uint8, device=device))
        self.out = dict(
            edge_ptr=_i32(n_atoms + 1, device), center=_i32(cap_e, device), neighbor=_i32(cap_e, device),
            image=_i32(3 * cap_e, device), dist=torch.empty(cap_e, dtype=torch.float64, device=device),
            rev=_i32(cap_e, device), d2u=_i32(cap_e, device), u2d=_i32(cap_e // 2, device),
            trip_ptr=_i32(cap_e // 2 + 1, device), trip_src_ptr=_i32(cap_e // 2 + 1, device),
            line_graph=_i32(5 * cap_t, device), trip_src_perm=_i32(cap_t, device))
        self.counts = torch.zeros(64, dtype=torch.int32, device=device)  # 16 used; the rest is spare
        self.counts_host = torch.zeros(64, dtype=torch.int32).pin_memory()


class _Candidates:
    """Verlet-skin state of one batch: the sorted directed-edge list of a build with the cut-off enlarged by the skin
    (the candidates), the positions it was built at, and the flag word the device-side displacement check sets."""

    def __init__(self, g: BatchedGraph, skin: float, cap: int, device):
        lib = _lib.load()
        self.skin, self.cap = float(skin), int(cap)
        n_atoms = g.n_atoms
        n_per = np.asarray(g.atoms_per_graph, dtype=np.int64)
        grid, self.n_cells = cell_grid(g.lattice64_host, n_per, g.cutoff + self.skin)
        self.grid = torch.from_numpy(grid).to(device)
        i64 = lambda n: torch.empty(max(int(n), 1), dtype=torch.int64, device=device)  # noqa: E731
        f64 = lambda n: torch.empty(max(int(n), 1), dtype=torch.float64, device=device)  # noqa: E731
        self.bufs = dict(
            cell_ptr=_i32(self.n_cells + 1, device), cell_fill=_i32(self.n_cells, device),
            cell_atoms=_i32(n_atoms, device), atom_cell=_i32(4 * n_atoms, device), atom_wrap=_i32(4 * n_atoms, device),
            scan_tmp=_i32(lib.mb_graph_scan_tmp_len(max(n_atoms, self.n_cells, cap)), device),
            key_unsorted=i64(cap), dist_unsorted=f64(cap), key=i64(cap),
            edge_ptr=_i32(n_atoms + 1, device), center=_i32(cap, device), neighbor=_i32(cap, device),
            image=_i32(3 * cap, device), dist=f64(cap))
        self.cart_ref = torch.zeros(n_atoms, 3, dtype=torch.float64, device=device)
        self.flag = torch.tensor([1, 0], dtype=torch.int32, device=device)  # [rebuild wanted, rebuilds so far]

    def invalidate(self):
        """Force a candidate rebuild at the next call (after a change of the lattices)."""
        self.flag[:1].fill_(1)


def _candidate_capacity(g: BatchedGraph, skin: float) -> int:
    n = np.asarray(g.atoms_per_graph, dtype=np.float64)
    lat = g.lattice64_host
    vol = np.abs(np.einsum("bi,bi->b", lat[:, 0], np.cross(lat[:, 1], lat[:, 2])))
    cap = int(1.25 * float((n * 4.0 / 3.0 * np.pi * (g.cutoff + skin) ** 3 * n / vol).sum())) + 1024
    return cap + (cap & 1)


def build_on_device(g: BatchedGraph, tol: float = 1e-8, stream=None, skin: float = 0.0) -> BatchedGraph:
    """Build the graph of the device-resident inputs of ``g`` (positions, lattices, cell grid) and attach the outputs.
    Can be called again after ``g.cart64`` changed on the device: the capacity buffers of the previous build are
    reused.  One asynchronous launch (mb_graph_build) and one copy of the status block to the host, which is
    the only synchronisation: the sizes of the model's tensors depend on the counts in it.

    ``skin`` > 0 (Angstrom) reuses the neighbour search across calls: a candidate list with the cut-off enlarged by
    the skin is kept with the batch and rebuilt (on the device, decided on the device) only when some atom has moved
    by half the skin since; every call then tests the candidates instead of searching the cells.  The graph is the
    one a fresh build gives, bit for bit.  The lattices must stay as they are between calls (fixed-cell MD and
    relaxation); after writing to them call ``g._candidates.invalidate()``."""
    lib = _lib.load()
    device = g.cart64.device
    n_atoms, n_struct, n_cells = g.n_atoms, g.n_struct, g.n_cells
    with torch.cuda.device(device):
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        buf = getattr(g, "_buffers", None)
        if buf is None:
            buf = g._buffers = _GraphBuffers(g, *_capacity_estimate(g), device)
        cand = None
        if skin > 0.0:
            cand = getattr(g, "_candidates", None)
            if cand is None or cand.skin != float(skin):
                cand = g._candidates = _Candidates(g, skin, _candidate_capacity(g, skin), device)

        def base_desc():
            m = _lib.MbGraph()
            m.n_atoms, m.n_struct = n_atoms, n_struct
            m.tol = float(tol)
            m.cart, m.lattice, m.inv_lattice = g.cart64.data_ptr(), g.lattice64.data_ptr(), g.inv_lattice64.data_ptr()
            m.atom_struct = g.atom_struct.data_ptr()
            return m

        for attempt in range(6):
            if cand is not None:
                # displacement check -> candidate rebuild if the flag is set -> record the positions it was built at
                _lib.call("mb_graph_skin_check", n_atoms, g.cart64.data_ptr(), cand.cart_ref.data_ptr(), 0.5 * cand.skin,
                          cand.flag.data_ptr(), st)
                c = base_desc()
                c.n_cells, c.cap_edges, c.cap_triplets, c.flags = cand.n_cells, cand.cap, 0, _lib.MB_GRAPH_EDGES_ONLY
                c.cutoff, c.line_cutoff, c.grid = g.cutoff + cand.skin, 0.0, cand.grid.data_ptr()
                for k, v in cand.bufs.items():
                    setattr(c, k, v.data_ptr())
                c.counts = buf.counts.data_ptr() + 64  # ints 16..31 of the block that is copied to the host
                c.run_if = cand.flag.data_ptr()
                _lib.call("mb_graph_build", C.byref(c), st)
                _lib.call("mb_graph_skin_commit", n_atoms, g.cart64.data_ptr(), cand.cart_ref.data_ptr(),
                          cand.flag.data_ptr(), st)
            m = base_desc()
            m.n_cells, m.cap_edges, m.cap_triplets = n_cells, buf.cap_e, buf.cap_t
            m.cutoff, m.line_cutoff, m.grid = g.cutoff, g.line_cutoff, g.grid.data_ptr()
            for k, v in buf.scratch.items():
                setattr(m, k, v.data_ptr())
            for k, v in buf.out.items():
                setattr(m, k, v.data_ptr())
            m.counts = buf.counts.data_ptr()
            if cand is not None:
                m.cand_ptr, m.cand_nbr, m.cand_img = (cand.bufs[k].data_ptr() for k in ("edge_ptr", "neighbor", "image"))
                m.cand_counts = buf.counts.data_ptr() + 64
            _lib.call("mb_graph_build", C.byref(m), st)
            buf.counts_host.copy_(buf.counts, non_blocking=True)
            torch.cuda.current_stream().synchronize() if stream is None else torch.cuda.synchronize()
            counts = buf.counts_host.numpy()
            if cand is not None and counts[9]:
                # the candidate build did not run to its end: a real error, or its buffers were too small
                cstat = lib.mb_graph_status(counts[16:32].ctypes.data_as(C.POINTER(C.c_int32)))
                if cstat != _lib.MB_ERR_CAPACITY:
                    _lib.check(cstat if cstat != _lib.MB_OK else _lib.MB_ERR_INVALID, "mb_graph_build (candidates)")
                rebuilds = int(cand.flag[1])
                cand = g._candidates = _Candidates(g, skin, int(1.1 * counts[16]) + 64, device)
                cand.flag[1] = rebuilds
                continue
            status = lib.mb_graph_status(counts.ctypes.data_as(C.POINTER(C.c_int32)))
            if status != _lib.MB_ERR_CAPACITY:
                break
            # enlarge to what this build needed (plus a margin for the steps to come) and run it again
            cap_e = max(buf.cap_e, int(1.1 * counts[0]) + 64)
            cap_t = int(1.1 * counts[2]) + 64 if counts[7] else max(buf.cap_t, int(1.5 * buf.cap_t * cap_e / buf.cap_e))
            old = buf
            buf = g._buffers = _GraphBuffers(g, cap_e, cap_t, device)
            buf.counts.copy_(old.counts)  # ints 16..31: the status of the candidate build, which is still valid
        _lib.check(status, "mb_graph_build")
        ne, nb, nt = int(counts[0]), int(counts[1]), int(counts[2])
        g.n_edges, g.n_bonds, g.n_triplets = ne, nb, nt
        o = buf.out
        g.edge_ptr = o["edge_ptr"]
        g.center, g.neighbor, g.image = o["center"][:ne], o["neighbor"][:ne], o["image"][:3 * ne].view(ne, 3)
        g.dist64, g.rev, g.d2u, g.u2d = o["dist"][:ne], o["rev"][:ne], o["d2u"][:ne], o["u2d"][:nb]
        g.trip_ptr, g.trip_src_ptr = o["trip_ptr"][:nb + 1], o["trip_src_ptr"][:nb + 1]
        g.line_graph = o["line_graph"][:5 * nt].view(nt, 5)
        g.trip_src_perm = o["trip_src_perm"][:nt]
        # column-major copy: each of (centre atom, target bond, target DE, source bond, source DE) contiguous
        g.lg_cols = g.line_graph.t().contiguous() if nt else torch.empty(5, 0, dtype=torch.int32, device=device)
    g._row_graphs = g._slices = None
    return g


def set_positions_on_device(g: BatchedGraph, cart64: torch.Tensor) -> None:
    """New Cartesian positions (float64, on the device) for the atoms of ``g``.  The float32 positions the model
    reads are derived exactly as for a fresh batch and as in the reference: fractional coordinates rounded to
    float32, times the float32 lattice (matris/graph/converter.py:82-83, matris/model/processgraph.py:87)."""
    g.cart64.copy_(cart64)
    struct = g.atom_struct.long()
    frac32 = torch.einsum("ni,nij->nj", g.cart64, g.inv_lattice64[struct]).to(torch.float32)
    g.cart32.copy_(torch.einsum("ni,nij->nj", frac32, g.lattice32[struct]))


def build_batched_graph(numbers: Sequence[np.ndarray], carts: Sequence[np.ndarray], lattices: Sequence[np.ndarray],
                        cutoff: float = 6.0, line_cutoff: float = 4.0, device="cuda", tol: float = 1e-8,
                        stream=None) -> BatchedGraph:
    """Build atom graph, bond graph and line graph for a batch of structures on ``device``."""
    device = torch.device(device)
    if device.type != "cuda":
        raise _lib.MbError("matris_b200 builds graphs on a CUDA device only (no CPU path)")
    hb = HostBatch(numbers, carts, lattices, cutoff)
    with torch.cuda.device(device):
        return build_on_device(upload(hb, cutoff, line_cutoff, device), tol, stream)


# ------------------------------------------------------------------ reference-compatible value type
class RadiusGraph:
    """One structure's graph with the reference's field names
    (matris/graph/radiusgraph.py:17-113).  Instances produced by
    ``GraphConverter`` also carry the device-resident batch they were built in
    (``_batch`` / ``_index``), which is what the model consumes."""

    def __init__(self, graph_id=None, mp_id=None, composition=None, atomic_number=None, atom_frac_coord=None,
                 lattice=None, neighbor_image=None, atom_graph=None, atom_graph_cutoff=6.0, line_graph=None,
                 line_graph_cutoff=4.0, directed2undirected=None, undirected2directed=None):
        self.graph_id, self.mp_id, self.composition = graph_id, mp_id, composition
        self.atomic_number, self.atom_frac_coord, self.lattice = atomic_number, atom_frac_coord, lattice
        self.neighbor_image, self.atom_graph, self.line_graph = neighbor_image, atom_graph, line_graph
        self.atom_graph_cutoff, self.line_graph_cutoff = atom_graph_cutoff, line_graph_cutoff
        self.directed2undirected, self.undirected2directed = directed2undirected, undirected2directed
        self._batch, self._index, self._source = None, 0, None
        assert len(directed2undirected) == 2 * len(undirected2directed), (
            f"Number of directed indices ({len(directed2undirected)}) != "
            f"2 * number of undirected indices ({2 * len(undirected2directed)})!")

    _TENSORS = ("atomic_number", "atom_frac_coord", "lattice", "neighbor_image", "atom_graph", "line_graph",
                "directed2undirected", "undirected2directed")

    def to(self, device="cpu") -> "RadiusGraph":
        d = self.to_dict()
        for k in self._TENSORS:
            d[k] = d[k].to(device)
        out = RadiusGraph(**d)
        out._batch, out._index, out._source = self._batch, self._index, self._source
        return out

    def to_dict(self) -> dict[str, Any]:
        return {k: getattr(self, k) for k in ("graph_id", "mp_id", "composition", "atomic_number", "atom_frac_coord",
                                               "lattice", "neighbor_image", "atom_graph", "atom_graph_cutoff",
                                               "line_graph", "line_graph_cutoff", "directed2undirected",
                                               "undirected2directed")}

    def save(self, fname=None, save_dir=".") -> str:
        name = fname or (f"{self.graph_id}.pt" if self.graph_id is not None else f"{self.composition}.pt")
        path = os.path.join(save_dir, name)
        torch.save({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in self.to_dict().items()}, path)
        return path

    @classmethod
    def from_file(cls, file_name: str) -> "RadiusGraph":
        return cls.from_dict(torch.load(file_name))

    @classmethod
    def from_dict(cls, dic: dict[str, Any]) -> "RadiusGraph":
        return RadiusGraph(**dic)

    def source_arrays(self):
        """(numbers, cart, lattice) this graph was built from; falls back to the float32 fields."""
        if self._source is not None:
            return self._source
        lat = self.lattice.detach().cpu().double().numpy()
        return (self.atomic_number.detach().cpu().numpy().astype(np.int64),
                self.atom_frac_coord.detach().cpu().double().numpy() @ lat, lat)

    def __repr__(self) -> str:
        return (f"RadiusGraph(composition={self.composition!r}, atom_graph_cutoff={self.atom_graph_cutoff}, "
                f"line_graph_cutoff={self.line_graph_cutoff}, n_atoms={len(self.atomic_number)}, "
                f"atom_graph_len={len(self.atom_graph)}, line_graph_len={len(self.line_graph)})")


def split_batch(batch: BatchedGraph, sources=None, graph_ids=None) -> list[RadiusGraph]:
    """Per-structure RadiusGraph views (local indices, reference layout) of a batch."""
    ap, ep, bp, tp = batch.structure_slices()
    out = []
    frac = torch.from_numpy(batch.frac32_host).to(batch.device)
    for b in range(batch.n_struct):
        a0, a1, e0, e1, u0, u1, t0, t1 = ap[b], ap[b + 1], ep[b], ep[b + 1], bp[b], bp[b + 1], tp[b], tp[b + 1]
        lg = batch.line_graph[t0:t1].clone()
        if len(lg):
            lg -= torch.tensor([a0, u0, e0, u0, e0], dtype=torch.int32, device=batch.device)
        rg = RadiusGraph(
            graph_id=None if graph_ids is None else graph_ids[b], mp_id=None,
            composition=_formula(batch.numbers_host[a0:a1]),
            atomic_number=batch.numbers[a0:a1], atom_frac_coord=frac[a0:a1], lattice=batch.lattice32[b],
            neighbor_image=batch.image[e0:e1].to(datatype),
            atom_graph=torch.stack([batch.center[e0:e1] - a0, batch.neighbor[e0:e1] - a0], dim=1),
            atom_graph_cutoff=batch.cutoff, line_graph=lg, line_graph_cutoff=batch.line_cutoff,
            directed2undirected=batch.d2u[e0:e1] - u0, undirected2directed=batch.u2d[u0:u1] - e0)
        rg._batch, rg._index = batch, b
        rg._source = (batch.numbers_host[a0:a1], batch.cart64_host[a0:a1], batch.lattice64_host[b])
        out.append(rg)
    return out


class GraphConverter(nn.Module):
    """Convert a structure to a RadiusGraph (matris/graph/converter.py:22-129) on the GPU."""

    def __init__(self, atom_graph_cutoff: float = 6, line_graph_cutoff: float = 4, verbose: bool = False,
                 device: str | None = None) -> None:
        super().__init__()
        self.atom_graph_cutoff = atom_graph_cutoff
        self.line_graph_cutoff = atom_graph_cutoff if line_graph_cutoff is None else line_graph_cutoff
        self.algorithm = "cuda"
        self.device = device
        if verbose:
            print(self)

    def __repr__(self) -> str:
        return (f"GraphConverter(algorithm={self.algorithm!r}, atom_graph_cutoff={self.atom_graph_cutoff}, "
                f"line_graph_cutoff={self.line_graph_cutoff})")

    def _device(self):
        return torch.device(self.device if self.device is not None else "cuda")

    def batch(self, structures) -> BatchedGraph:
        """Graphs of many structures in one pass (the batched entry the model uses)."""
        arrays = [as_arrays(s) for s in structures]
        return build_batched_graph([a[0] for a in arrays], [a[1] for a in arrays], [a[2] for a in arrays],
                                   self.atom_graph_cutoff, self.line_graph_cutoff, self._device())

    def forward(self, structure, graph_id=None, mp_id=None) -> RadiusGraph:
        """Convert one structure; raises ValueError for an isolated atom like the reference."""
        rg = split_batch(self.batch([structure]), graph_ids=[graph_id])[0]
        rg.mp_id = mp_id
        return rg

    def as_dict(self) -> dict[str, float]:
        return {"atom_graph_cutoff": self.atom_graph_cutoff, "line_graph_cutoff": self.line_graph_cutoff,
                "algorithm": self.algorithm}

    @classmethod
    def from_dict(cls, dict) -> "GraphConverter":
        dict = {k: v for k, v in dict.items() if k != "algorithm"}
        return GraphConverter(**dict)
