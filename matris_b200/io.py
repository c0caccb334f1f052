"""Structure and trajectory files without third-party packages.

The reference reads and writes structures through pymatgen / ASE (matris/graph/converter.py:63-70 takes a pymatgen
``Structure``; matris/applications/md.py:223-236 writes an ASE trajectory).  On a box without those packages the
evaluation path still needs a way in and out, so this module reads and writes the three plain-text formats that cover
it: extended XYZ (frames with cell, species, positions and per-atom / per-frame properties), VASP POSCAR, and CIF
files that list every atom of the cell (space group P1: no symmetry expansion is done, and a file with symmetry
operations other than the identity is rejected).  Every reader returns ``SimpleAtoms`` objects, which all entry
points of the package accept.
"""
from __future__ import annotations

import re
import shlex

import numpy as np

SYMBOLS = (
    "X H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr Y Zr Nb "
    "Mo Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W Re Os Ir Pt Au Hg "
    "Tl Pb Bi Po At Rn Fr Ra Ac Th Pa U Np Pu Am Cm Bk Cf Es Fm Md No Lr Rf Db Sg Bh Hs Mt Ds Rg Cn Nh Fl Mc Lv Ts Og"
).split()
NUMBER_OF = {s: z for z, s in enumerate(SYMBOLS)}


def _atoms(numbers, positions, cell, pbc=True, momenta=None):
    from .applications import SimpleAtoms

    return SimpleAtoms(numbers, positions, cell, pbc=pbc, momenta=momenta)


def _number(token: str) -> int:
    token = token.strip()
    if token.isdigit():
        return int(token)
    m = re.match(r"[A-Za-z]+", token)
    sym = m.group(0).capitalize() if m else ""
    if sym not in NUMBER_OF:
        raise ValueError(f"unknown element {token!r}")
    return NUMBER_OF[sym]


# ---------------------------------------------------------------------------------------------------- extended XYZ
def _parse_comment(line: str) -> dict:
    """key=value pairs of an extended-XYZ comment line; values may be quoted."""
    out = {}
    lex = shlex.shlex(line, posix=True)
    lex.whitespace_split = True
    lex.commenters = ""
    for tok in lex:
        if "=" in tok:
            k, v = tok.split("=", 1)
            out[k.strip()] = v.strip()
        else:
            out[tok] = "T"
    return out


def _properties(spec: str):
    """'species:S:1:pos:R:3:forces:R:3' -> [(name, kind, ncols), ...]"""
    p = spec.split(":")
    if len(p) % 3:
        raise ValueError(f"malformed Properties string {spec!r}")
    return [(p[i], p[i + 1].upper(), int(p[i + 2])) for i in range(0, len(p), 3)]


def read_extxyz(path: str, index=slice(None)):
    """Read frames of an (extended) XYZ file.  Returns a list of ``SimpleAtoms`` (one object for an integer
    ``index``).  Per-frame keys other than Lattice / Properties / pbc land in ``atoms.info`` (numbers and arrays
    parsed where possible), per-atom columns other than species / pos / momenta in ``atoms.arrays``."""
    frames = []
    with open(path) as f:
        lines = f.read().splitlines()
    i = 0
    while i < len(lines):
        if not lines[i].strip():
            i += 1
            continue
        n = int(lines[i].split()[0])
        info = _parse_comment(lines[i + 1]) if i + 1 < len(lines) else {}
        body = [ln.split() for ln in lines[i + 2:i + 2 + n]]
        if len(body) != n or any(not b for b in body):
            raise ValueError(f"{path}: frame starting at line {i + 1} is truncated")
        i += 2 + n
        low = {k.lower(): k for k in info}
        props = _properties(info[low["properties"]]) if "properties" in low else [("species", "S", 1), ("pos", "R", 3)]
        cols, o = {}, 0
        for name, kind, nc in props:
            block = [b[o:o + nc] for b in body]
            o += nc
            if kind == "S":
                cols[name] = [b[0] if nc == 1 else b for b in block]
            elif kind == "L":
                cols[name] = np.array([[t.upper().startswith("T") for t in b] for b in block]).reshape(n, nc)
            else:
                cols[name] = np.array(block, dtype=np.int64 if kind == "I" else np.float64).reshape(n, nc)
        species = cols.pop("species", None)
        if species is None:
            species = [str(int(z)) for z in cols.pop("Z").reshape(-1)]
        numbers = np.array([_number(s) for s in species], dtype=np.int64)
        pos = cols.pop("pos")
        cell = np.zeros((3, 3))
        pbc = False
        if "lattice" in low:
            cell = np.array(info[low["lattice"]].split(), dtype=np.float64).reshape(3, 3)
            pbc = True
        if "pbc" in low:
            pbc = [t.upper().startswith("T") for t in info[low["pbc"]].split()]
        momenta = cols.pop("momenta", None)
        a = _atoms(numbers, pos, cell, pbc=pbc, momenta=momenta)
        a.arrays = {k: (v[:, 0] if isinstance(v, np.ndarray) and v.shape[1] == 1 else v) for k, v in cols.items()}
        a.info = {}
        for k, v in info.items():
            if k.lower() in ("lattice", "properties", "pbc"):
                continue
            try:
                arr = np.array(v.split(), dtype=np.float64)
                a.info[k] = float(arr[0]) if arr.size == 1 else arr
            except ValueError:
                a.info[k] = v
        frames.append(a)
    if isinstance(index, int):
        return frames[index]
    return frames[index]


def write_extxyz(path: str, frames, append: bool = False, results=None) -> None:
    """Write ``frames`` (one atoms object or a sequence) as extended XYZ.  ``results`` (optional, one dict per frame
    with the calculator's keys ``energy``, ``forces``, ``stress``, ``magmoms``) is written along; momenta are written
    when they are not all zero."""
    if hasattr(frames, "get_positions"):
        frames = [frames]
    if isinstance(results, dict):
        results = [results]
    with open(path, "a" if append else "w") as f:
        for k, a in enumerate(frames):
            numbers = np.asarray(a.get_atomic_numbers())
            pos = np.asarray(a.get_positions(), dtype=float)
            cell = np.asarray(a.get_cell(), dtype=float).reshape(3, 3)
            pbc = np.asarray(a.get_pbc(), dtype=bool) if hasattr(a, "get_pbc") else np.array([True] * 3)
            res = results[k] if results is not None else {}
            cols, spec = [pos], "species:S:1:pos:R:3"
            mom = np.asarray(a.get_momenta(), dtype=float) if hasattr(a, "get_momenta") else None
            if mom is not None and np.any(mom):
                cols.append(mom)
                spec += ":momenta:R:3"
            if res.get("forces") is not None:
                cols.append(np.asarray(res["forces"], dtype=float))
                spec += ":forces:R:3"
            if res.get("magmoms") is not None:
                cols.append(np.asarray(res["magmoms"], dtype=float).reshape(-1, 1))
                spec += ":magmoms:R:1"
            head = 'Lattice="' + " ".join(f"{x:.12g}" for x in cell.reshape(-1)) + f'" Properties={spec}'
            head += ' pbc="' + " ".join("T" if p else "F" for p in pbc) + '"'
            if res.get("energy") is not None:
                head += f" energy={float(np.asarray(res['energy']).reshape(-1)[0]):.12g}"
            if res.get("stress") is not None:
                head += ' stress="' + " ".join(f"{x:.12g}" for x in np.asarray(res["stress"], dtype=float).reshape(-1)) + '"'
            f.write(f"{len(numbers)}\n{head}\n")
            data = np.concatenate(cols, axis=1)
            for z, row in zip(numbers, data):
                f.write(SYMBOLS[int(z)] + " " + " ".join(f"{x:.12g}" for x in row) + "\n")


# ---------------------------------------------------------------------------------------------------- POSCAR
def read_poscar(path: str):
    """VASP 5 POSCAR / CONTCAR (species line required; selective dynamics flags are skipped)."""
    with open(path) as f:
        ln = [x.rstrip("\n") for x in f]
    scale = float(ln[1].split()[0])
    cell = np.array([ln[i].split()[:3] for i in (2, 3, 4)], dtype=np.float64)
    if scale < 0:  # negative: target volume
        scale = (-scale / abs(np.linalg.det(cell))) ** (1.0 / 3.0)
    cell *= scale
    species = ln[5].split()
    if all(t.isdigit() for t in species):
        raise ValueError(f"{path}: VASP 4 files without a species line are not supported")
    counts = [int(t) for t in ln[6].split()]
    i = 7
    if ln[i].strip()[:1] in "sS":
        i += 1
    direct = ln[i].strip()[:1] not in "cCkK"
    n = sum(counts)
    xyz = np.array([ln[i + 1 + k].split()[:3] for k in range(n)], dtype=np.float64)
    pos = xyz @ cell if direct else xyz * scale
    numbers = np.repeat([_number(s) for s in species], counts)
    return _atoms(numbers, pos, cell)


def write_poscar(path: str, atoms, comment: str = "written by matris_b200") -> None:
    numbers = np.asarray(atoms.get_atomic_numbers())
    cell = np.asarray(atoms.get_cell(), dtype=float).reshape(3, 3)
    frac = np.asarray(atoms.get_positions(), dtype=float) @ np.linalg.inv(cell)
    order = np.argsort(numbers, kind="stable")
    zs, counts = np.unique(numbers[order], return_counts=True)
    with open(path, "w") as f:
        f.write(comment + "\n1.0\n")
        for row in cell:
            f.write(" ".join(f"{x:.16f}" for x in row) + "\n")
        f.write(" ".join(SYMBOLS[int(z)] for z in zs) + "\n" + " ".join(str(int(c)) for c in counts) + "\nDirect\n")
        for row in frac[order]:
            f.write(" ".join(f"{x:.16f}" for x in row) + "\n")


# ---------------------------------------------------------------------------------------------------- CIF (P1)
def _cif_number(tok: str) -> float:
    return float(re.sub(r"\(.*\)", "", tok))


def read_cif(path: str):
    """CIF that lists every atom of the cell (P1).  Reads the six cell parameters and the ``_atom_site`` loop
    (fractional coordinates; ``_atom_site_type_symbol`` or, failing that, the label).  Symmetry is not expanded:
    a file whose symmetry loop holds anything but the identity operation raises ``ValueError``."""
    with open(path) as f:
        raw = [x.strip() for x in f]
    lines = [x for x in raw if x and not x.startswith("#")]
    cellp, i = {}, 0
    loops = []
    while i < len(lines):
        ln = lines[i]
        if ln.lower().startswith("loop_"):
            tags, rows = [], []
            i += 1
            while i < len(lines) and lines[i].startswith("_"):
                tags.append(lines[i].split()[0].lower())
                i += 1
            while i < len(lines) and not lines[i].startswith("_") and not lines[i].lower().startswith(("loop_", "data_")):
                rows.append(shlex.split(lines[i]))
                i += 1
            loops.append((tags, rows))
            continue
        if ln.startswith("_cell_"):
            p = ln.split()
            if len(p) >= 2:
                cellp[p[0].lower()] = _cif_number(p[1])
        i += 1
    for tags, rows in loops:
        for key in ("_symmetry_equiv_pos_as_xyz", "_space_group_symop_operation_xyz"):
            if key in tags:
                c = tags.index(key)
                ops = {re.sub(r"\s+", "", r[c]).lower() for r in rows if len(r) > c}
                if ops - {"x,y,z", "+x,+y,+z"}:
                    raise ValueError(f"{path}: symmetry operations present; only P1 files (all atoms listed) are read")
    try:
        a, b, c = (cellp[f"_cell_length_{k}"] for k in "abc")
        al, be, ga = (np.radians(cellp[f"_cell_angle_{k}"]) for k in ("alpha", "beta", "gamma"))
    except KeyError as e:
        raise ValueError(f"{path}: cell parameter {e} missing") from None
    cx = c * np.cos(be)
    cy = c * (np.cos(al) - np.cos(be) * np.cos(ga)) / np.sin(ga)
    cell = np.array([[a, 0.0, 0.0], [b * np.cos(ga), b * np.sin(ga), 0.0],
                     [cx, cy, np.sqrt(max(c * c - cx * cx - cy * cy, 0.0))]])
    for tags, rows in loops:
        if "_atom_site_fract_x" in tags:
            ix, iy, iz = (tags.index(f"_atom_site_fract_{k}") for k in "xyz")
            isym = tags.index("_atom_site_type_symbol") if "_atom_site_type_symbol" in tags else tags.index("_atom_site_label")
            frac = np.array([[_cif_number(r[ix]), _cif_number(r[iy]), _cif_number(r[iz])] for r in rows])
            numbers = np.array([_number(r[isym]) for r in rows], dtype=np.int64)
            return _atoms(numbers, frac @ cell, cell)
    raise ValueError(f"{path}: no _atom_site loop with fractional coordinates")
