"""CPU: the shared library builds, loads, exports every symbol the header declares,
and the ctypes signatures agree with the header's parameter lists."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from matris_b200 import _lib, build

HEADER = os.path.join(ROOT, "include", "matris_b200.h")


def _declarations():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    decls = {}
    for m in re.finditer(r"\b(int|size_t|const char\*)\s+(mb_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        args = m.group(3).strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        decls[m.group(2)] = (m.group(1), n, args)
    return decls


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    decls = _declarations()
    assert len(decls) >= 30
    for name in decls:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_signatures_match_header(lib):
    decls = _declarations()
    bound = dict(_lib._SIGNATURES)
    bound.update({k: v[1] for k, v in _lib._OTHER.items()})
    assert set(bound) == set(decls), set(bound) ^ set(decls)
    for name, argtypes in bound.items():
        ret, n, args = decls[name]
        assert len(argtypes) == n, f"{name}: header has {n} parameters, binding has {len(argtypes)}"
        # integer / float / pointer kinds agree position by position
        for a, t in zip([x.strip() for x in args.split(",")] if n else [], argtypes):
            is_ptr = "*" in a
            if is_ptr:
                assert t in (ctypes.c_void_p,) or hasattr(t, "contents") or t is ctypes.c_char_p, (name, a, t)
            elif a.startswith("float"):
                assert t is ctypes.c_float, (name, a, t)
            elif a.startswith("int64_t"):
                assert t is ctypes.c_int64, (name, a, t)
            elif a.startswith("int32_t") or a.startswith("int "):
                assert t in (ctypes.c_int32, ctypes.c_int), (name, a, t)


def test_struct_layouts_match_header():
    """Compile a tiny C program against the header and compare sizeof/offsetof."""
    import subprocess
    import tempfile
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "matris_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu\n", sizeof(mb_graph), sizeof(mb_src), sizeof(mb_colblock), sizeof(mb_gemm_desc));
  printf("%zu %zu %zu %zu\n", offsetof(mb_graph, cart), offsetof(mb_graph, edge_ptr), offsetof(mb_graph, trip_src_perm),
         offsetof(mb_graph, tol));
  printf("%zu %zu %zu %zu %zu\n", offsetof(mb_colblock, W), offsetof(mb_colblock, gate), offsetof(mb_colblock, res),
         offsetof(mb_colblock, out), offsetof(mb_colblock, out_scale));
  return 0;
}
'''
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), os.path.join(d, "t.c"), "-o",
                               os.path.join(d, "t")])
        out = subprocess.check_output([os.path.join(d, "t")], text=True).split()
    got = [int(x) for x in out]
    G, S, B, D = _lib.MbGraph, _lib.MbSrc, _lib.MbColBlock, _lib.MbGemmDesc
    want = [ctypes.sizeof(G), ctypes.sizeof(S), ctypes.sizeof(B), ctypes.sizeof(D),
            G.cart.offset, G.edge_ptr.offset, G.trip_src_perm.offset, G.tol.offset,
            B.W.offset, B.gate.offset, B.res.offset, B.out.offset, B.out_scale.offset]
    assert got == want


def test_version_and_status_strings(lib):
    assert lib.mb_version() == 1
    assert lib.mb_status_string(0) == b"ok"
    assert b"isolated" in lib.mb_status_string(5)
    assert lib.mb_graph_scan_tmp_len(10_000_000) >= 2 * (10_000_000 // 8192)  # two partial sums per 8192-element chunk
    assert b"capacity" in lib.mb_status_string(7)


def test_invalid_arguments_are_status_codes_before_any_launch(lib):
    """Argument validation happens on the host before a device is touched: NULL descriptors, impossible sizes and
    missing pointers come back as MB_ERR_INVALID (no exception, no trap, no CUDA call), also on a box without a GPU."""
    import ctypes as C
    assert lib.mb_gemm(None, None) == 1
    d = _lib.MbGemmDesc()
    d.n_rows, d.n_blocks = 10, 0
    assert lib.mb_gemm(C.byref(d), None) == 1                   # no column block
    d.n_blocks = 5
    assert lib.mb_gemm(C.byref(d), None) == 1                   # more than four
    assert lib.mb_gated_mlp_fwd(None, None) == 1
    g = _lib.MbGatedMlp()
    g.n_rows, g.n_src = 10, 7
    assert lib.mb_gated_mlp_fwd(C.byref(g), None) == 1          # K segments out of range
    assert lib.mb_graph_build(None, None) == 1
    m = _lib.MbGraph()
    m.n_atoms, m.n_struct, m.n_cells, m.cap_edges = 4, 1, 1, 64
    assert lib.mb_graph_build(C.byref(m), None) == 1            # no buffers given
    assert lib.mb_graph_status(None) == 1
    counts = (C.c_int32 * 16)()
    assert lib.mb_graph_status(counts) == 0
    counts[3] = 2
    assert lib.mb_graph_status(counts) == 5                     # isolated atoms
    counts[3], counts[6] = 0, 1
    assert lib.mb_graph_status(counts) == 7                     # edge capacity too small
    counts[6], counts[9] = 0, 1
    assert lib.mb_graph_status(counts) == 7                     # candidate list unusable: rebuild it
    assert lib.mb_graph_skin_check(0, None, None, 0.25, None, None) == 1
    assert lib.mb_set_gemm_mode(9) == 1
    assert lib.mb_set_gemm_mode(0) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.MbError):
        _lib.load()


def test_gemm_descriptor_packing_matches_ctypes_mirror(monkeypatch):
    """ops.gemm packs mb_gemm_desc with struct; every field must land where the ctypes mirror (and the header) put it."""
    import torch

    from matris_b200 import _lib, ops

    captured = {}
    monkeypatch.setattr(ops, "call", lambda name, *a: captured.update(name=name, desc=bytes(a[0]._obj)))
    monkeypatch.setattr(ops, "_stream", lambda: 0)

    class FakeSplit:
        def __init__(self, w):
            self.w, self.hi, self.lo, self.shape = w, w.clone(), w.clone(), w.shape
            self.hi16, self.lo16 = w.to(torch.bfloat16), w.to(torch.bfloat16)
            self.ptrs = tuple(t.data_ptr() for t in (self.w, self.hi, self.lo, self.hi16, self.lo16))
            self.ldw = w.stride(0)

    monkeypatch.setattr(ops, "as_split", lambda w: w if isinstance(w, FakeSplit) else FakeSplit(w))
    x, idx, W = torch.randn(300, 256), torch.arange(300, dtype=torch.int32), FakeSplit(torch.randn(256, 384))
    out, g, r, rw, bias = torch.empty(300, 256), torch.randn(300, 256), torch.randn(300, 256), torch.randn(128), torch.randn(256)
    ops.gemm(300, [ops.B([ops.S(x, None, 0, 1), ops.S(x, idx, 128, 0), ops.S(x, idx, 0, 0)], W, w_row=128 * j, bias=bias,
                         bias_off=128 * j, gate=g, gate_col=128 * j, res=r, res_col=128 * j, res_w=rw, out=out,
                         out_idx=idx, out_col=128 * j, mode=ops.OUT_ATOMIC, scale=0.5, out_act=1) for j in (0, 1)])
    assert captured["name"] == "mb_gemm"
    separate = captured["desc"]
    # column blocks that share ONE list of sources pack the same bytes as blocks with equal lists of their own
    shared = [ops.S(x, None, 0, 1), ops.S(x, idx, 128, 0), ops.S(x, idx, 0, 0)]
    ops.gemm(300, [ops.B(shared, W, w_row=128 * j, bias=bias, bias_off=128 * j, gate=g, gate_col=128 * j, res=r,
                         res_col=128 * j, res_w=rw, out=out, out_idx=idx, out_col=128 * j, mode=ops.OUT_ATOMIC, scale=0.5,
                         out_act=1) for j in (0, 1)])
    assert captured["desc"] == separate
    d = _lib.MbGemmDesc.from_buffer_copy(captured["desc"])
    assert (d.n_rows, d.n_blocks) == (300, 2)
    for j in (0, 1):
        cb = d.blk[j]
        assert (cb.n_src, cb.out_act, cb.mode) == (3, 1, ops.OUT_ATOMIC) and abs(cb.out_scale - 0.5) < 1e-9
        assert (cb.src[0].ptr, cb.src[0].idx or 0, cb.src[0].ld, cb.src[0].col, cb.src[0].act) == (x.data_ptr(), 0, 256, 0, 1)
        assert (cb.src[1].idx, cb.src[1].col, cb.src[1].act) == (idx.data_ptr(), 128, 0) and not cb.src[3].ptr
        off = 4 * 384 * 128 * j
        assert (cb.W, cb.W_hi, cb.W_lo, cb.ldw) == (W.w.data_ptr() + off, W.hi.data_ptr() + off, W.lo.data_ptr() + off, 384)
        assert (cb.W_hi16, cb.W_lo16) == (W.hi16.data_ptr() + off // 2, W.lo16.data_ptr() + off // 2)
        assert cb.bias == bias.data_ptr() + 512 * j
        assert (cb.gate, cb.ld_gate, cb.col_gate) == (g.data_ptr(), 256, 128 * j)
        assert (cb.res, cb.res_w, cb.ld_res, cb.col_res) == (r.data_ptr(), rw.data_ptr(), 256, 128 * j)
        assert (cb.out, cb.out_idx, cb.ld_out, cb.col_out) == (out.data_ptr(), idx.data_ptr(), 256, 128 * j)
