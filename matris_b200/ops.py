"""Thin Python wrappers over the C-ABI kernels (device pointers in, nothing computed here).

Tensors are float32 / int32, contiguous, on the current CUDA device.  Every
wrapper launches on torch's current stream.
"""
from __future__ import annotations

import ctypes as C
import struct

import torch

from . import _lib
from ._lib import OUT_ADD, OUT_ATOMIC, OUT_STORE, call, ptr  # noqa: F401

D = 128


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_pinned_stream = None


class pinned_stream:
    """Within the block every entry point launches on the stream that is current at entry (looked up once instead
    of once per launch).  The autograd engine runs backward functions on that same stream, from its own thread,
    so the handle is shared process-wide for the duration of the block; blocks do not nest across devices."""

    def __enter__(self):
        global _pinned_stream
        self.outer, _pinned_stream = _pinned_stream, None
        _pinned_stream = _stream()
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self.outer
        return False


def _stream():
    """Raw handle of torch's current stream on the current device (the stream every entry point launches on)."""
    if _pinned_stream is not None:
        return _pinned_stream
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def new(rows, cols, like, zero=False):
    f = torch.zeros if zero else torch.empty
    return f((int(rows), int(cols)), dtype=torch.float32, device=like.device)


# ------------------------------------------------------------------ GEMM descriptors
class SplitWeight:
    """A weight matrix [n_out, K] with its tensor-core operand splits, all in the layout of ``w``:
    ``hi16`` = bf16(w), ``lo16`` = bf16(w - hi16) for the 3xBF16 core (the default);
    ``hi`` = tf32-rounded values, ``lo`` = w - hi (float32) for the 3xTF32 cores.
    ``w`` itself feeds the exact-fp32 SIMT core."""

    __slots__ = ("w", "hi", "lo", "hi16", "lo16", "shape", "ptrs", "ldw")

    def __init__(self, w: torch.Tensor):
        w = w.detach().contiguous()
        bits = w.view(torch.int32)
        hi = ((bits + 0x1000) & ~0x1FFF).view(torch.float32)  # round to nearest (ties away) at 10 mantissa bits
        self.w, self.hi, self.lo, self.shape = w, hi.contiguous(), (w - hi).contiguous(), w.shape
        self.hi16 = w.to(torch.bfloat16).contiguous()          # round to nearest even
        self.lo16 = (w - self.hi16.float()).to(torch.bfloat16).contiguous()
        # device addresses and row stride, looked up once: the descriptor packing runs for every launch
        self.ptrs = (w.data_ptr(), self.hi.data_ptr(), self.lo.data_ptr(), self.hi16.data_ptr(), self.lo16.data_ptr())
        self.ldw = w.stride(0)
        assert w.dim() == 2 and w.stride(1) == 1

    def t(self) -> "SplitWeight":
        return SplitWeight(self.w.t())


_split_cache: dict = {}


def as_split(W) -> SplitWeight:
    if isinstance(W, SplitWeight):
        return W
    key = (W.data_ptr(), tuple(W.shape), W._version)
    sw = _split_cache.get(key)
    if sw is None:
        if len(_split_cache) > 256:
            _split_cache.clear()
        sw = _split_cache[key] = SplitWeight(W)
    return sw


def S(t, idx=None, col=0, act=0):
    """One 128-wide K segment: rows of ``t`` (optionally gathered by ``idx``), columns col..col+127."""
    return (t, idx, col, act)


def B(srcs, W, w_row=0, bias=None, bias_off=0, gate=None, gate_col=0, out_act=0, res=None, res_col=0, res_w=None,
      out=None, out_idx=None, out_col=0, mode=OUT_STORE, scale=1.0):
    """One 128-column output block (see mb_colblock)."""
    return dict(srcs=srcs, W=W, w_row=w_row, bias=bias, bias_off=bias_off, gate=gate, gate_col=gate_col,
                out_act=out_act, res=res, res_col=res_col, res_w=res_w, out=out, out_idx=out_idx, out_col=out_col,
                mode=mode, scale=scale)


# Byte layout of mb_colblock / mb_gemm_desc (little endian, every member naturally aligned; checked against the
# ctypes mirror at import).  The descriptor is packed with one struct call per column block: filling the ctypes
# mirror field by field costs more host time than a small launch takes on the device.
_BLK_FMT = struct.Struct("<ii" + "QQqii" * 4 + "QQQQQqQ" + "Qqii" + "QQqii" + "QQqif")
_HDR_FMT = struct.Struct("<qii")
_BLK_OFF, _BLK_SIZE, _DESC_SIZE = _lib.MbGemmDesc.blk.offset, C.sizeof(_lib.MbColBlock), C.sizeof(_lib.MbGemmDesc)
assert _BLK_FMT.size == _BLK_SIZE and _HDR_FMT.size == _BLK_OFF and _DESC_SIZE == _BLK_OFF + 4 * _BLK_SIZE
_NO_SRC = (0, 0, 0, 0, 0)


_PAD = ((), _NO_SRC, _NO_SRC * 2, _NO_SRC * 3, _NO_SRC * 4)  # by number of missing sources


def gemm(n_rows: int, blocks: list[dict]) -> None:
    if n_rows == 0:
        return
    buf = bytearray(_DESC_SIZE)
    _HDR_FMT.pack_into(buf, 0, n_rows, len(blocks), 0)
    off = _BLK_OFF
    last_srcs = flat = None
    for b in blocks:
        srcs = b["srcs"]
        n_src = len(srcs)
        if srcs is not last_srcs:  # column blocks that share one list of sources share its packed form
            flat = []
            for t, idx, col, act in srcs:
                assert t.dtype == torch.float32 and t.stride(-1) == 1
                flat += (t.data_ptr(), 0 if idx is None else idx.data_ptr(), t.stride(0), col, act)
            flat += _PAD[4 - n_src]
            last_srcs = srcs
        sw = b["W"]
        if type(sw) is not SplitWeight:
            sw = as_split(sw)
        ldw = sw.ldw
        assert sw.shape[1] >= D * n_src
        w_off = 4 * ldw * b["w_row"]
        w_off16 = w_off // 2
        pw, ph, pl, ph16, pl16 = sw.ptrs
        bias, gate, res, res_w, out, out_idx = b["bias"], b["gate"], b["res"], b["res_w"], b["out"], b["out_idx"]
        _BLK_FMT.pack_into(
            buf, off, n_src, b["out_act"], *flat,
            pw + w_off, ph + w_off, pl + w_off, ph16 + w_off16, pl16 + w_off16, ldw,
            0 if bias is None else bias.data_ptr() + 4 * b["bias_off"],
            0 if gate is None else gate.data_ptr(), 0 if gate is None else gate.stride(0),
            0 if gate is None else b["gate_col"], 0,
            0 if res is None else res.data_ptr(), 0 if res is None or res_w is None else res_w.data_ptr(),
            0 if res is None else res.stride(0), 0 if res is None else b["res_col"], b["mode"],
            out.data_ptr(), 0 if out_idx is None else out_idx.data_ptr(), out.stride(0), b["out_col"],
            b["scale"])
        off += _BLK_SIZE
    if _lib.profile is not None:
        _lib.profile_meta = dict(flops=sum(2.0 * n_rows * D * D * len(b["srcs"]) for b in blocks), rows=int(n_rows),
                                 k=D * len(blocks[0]["srcs"]), n=D * len(blocks),
                                 bytes=4.0 * n_rows * D * (len(blocks[0]["srcs"]) + len(blocks) +
                                                           sum(b.get("gate") is not None for b in blocks) +
                                                           sum(b.get("res") is not None for b in blocks)))
    call("mb_gemm", C.byref(_lib.MbGemmDesc.from_buffer(buf)), _stream())


_GATED_FMT = struct.Struct("<qii" + "QQqii" * 4 + "QQQQQqQ" + "QQQQQqQ" + "QQ" + "Qq" * 3 + "QQq" + "Qq")
assert _GATED_FMT.size == C.sizeof(_lib.MbGatedMlp)


def gated_mlp_fwd(p, n_rows, srcs, want_h=True, res=None, res_w=None, save=True):
    """GatedMLP forward as one fused kernel (mb_gated_mlp_fwd).  ``p`` holds the packed weights (w1 [256,K], b1,
    w2 [256,128], b2, nc, ng).  Returns (z1, z2, h, out2); z1 / z2 only when ``save`` (the backward pass reads
    them), h only when ``want_h``, out2 = h + res_w * res only when ``res`` is given."""
    ref = srcs[0][0]
    n_rows = int(n_rows)
    # the composed path of the non-default GEMM modes uses z1 / z2 as scratch
    save = save or _gemm_mode != 0
    z1 = new(n_rows, 2 * D, ref) if save else None
    z2 = new(n_rows, 2 * D, ref) if save else None
    h = new(n_rows, D, ref) if want_h else None
    out2 = new(n_rows, D, ref) if res is not None else None
    if n_rows == 0:
        return z1, z2, h, out2
    flat = []
    for t, idx, col, act in srcs:
        assert t.dtype == torch.float32 and t.stride(-1) == 1
        flat += (t.data_ptr(), 0 if idx is None else idx.data_ptr(), t.stride(0), int(col), int(act))
    for _ in range(4 - len(srcs)):
        flat += _NO_SRC
    w1, w2 = as_split(p.w1), as_split(p.w2)
    assert w1.shape[0] == 2 * D and w1.shape[1] == D * len(srcs) and tuple(w2.shape) == (2 * D, D)

    def pl(t):
        return (0, 0) if t is None else (t.data_ptr(), t.stride(0))

    buf = _GATED_FMT.pack(
        n_rows, len(srcs), 0, *flat,
        *w1.ptrs, w1.ldw,
        0 if p.b1 is None else p.b1.data_ptr(),
        *w2.ptrs, w2.ldw,
        0 if p.b2 is None else p.b2.data_ptr(),
        p.nc.data_ptr(), p.ng.data_ptr(), *pl(z1), *pl(z2), *pl(h),
        0 if res is None else res.data_ptr(), 0 if res is None or res_w is None else res_w.data_ptr(),
        0 if res is None else res.stride(0), *pl(out2))
    if _lib.profile is not None:
        cols = len(srcs) + (4 if z1 is not None else 0) + (h is not None) + 2 * (out2 is not None)
        _lib.profile_meta = dict(flops=2.0 * n_rows * 2 * D * D * (len(srcs) + 1), rows=n_rows, k=D * len(srcs),
                                 n=2 * D, fused=True, bytes=4.0 * n_rows * D * cols)
    call("mb_gated_mlp_fwd", C.byref(_lib.MbGatedMlp.from_buffer_copy(buf)), _stream())
    return z1, z2, h, out2


def ffn_fwd(p, x, want_y=True, res=None, res_w=None, save=True):
    """Two-layer perceptron  y = W2 SiLU(W1 x + b1) + b2  as one launch of the fused kernel in its plain form
    (mb_gated_mlp_fwd with kind = MB_MLP_PLAIN).  ``p`` holds w1 [128, K], b1, w2 [128, 128], b2.  Returns
    (z1, y, out2): z1 = W1 x + b1 only when ``save`` (the backward pass reads it), y only when ``want_y``,
    out2 = y + res_w * res only when ``res`` is given."""
    n_rows = int(x.shape[0])
    w1, w2 = as_split(p.w1), as_split(p.w2)
    k = w1.shape[1]
    assert w1.shape[0] == D and k % D == 0 and x.shape[1] == k and tuple(w2.shape) == (D, D)
    assert x.dtype == torch.float32 and x.stride(-1) == 1
    save = save or _gemm_mode != 0  # the composed path of the non-default GEMM modes uses z1 as scratch
    z1 = new(n_rows, D, x) if save else None
    y = new(n_rows, D, x) if want_y else None
    out2 = new(n_rows, D, x) if res is not None else None
    if n_rows == 0:
        return z1, y, out2
    n_src = k // D
    flat = []
    for s in range(n_src):
        flat += (x.data_ptr(), 0, x.stride(0), D * s, 0)
    for _ in range(4 - n_src):
        flat += _NO_SRC

    def pl(t):
        return (0, 0) if t is None else (t.data_ptr(), t.stride(0))

    buf = _GATED_FMT.pack(
        n_rows, n_src, 1, *flat,
        *w1.ptrs, w1.ldw, 0 if p.b1 is None else p.b1.data_ptr(),
        *w2.ptrs, w2.ldw, 0 if p.b2 is None else p.b2.data_ptr(),
        0, 0, *pl(z1), 0, 0, *pl(y),
        0 if res is None else res.data_ptr(), 0 if res is None or res_w is None else res_w.data_ptr(),
        0 if res is None else res.stride(0), *pl(out2))
    if _lib.profile is not None:
        cols = n_src + (z1 is not None) + (y is not None) + 2 * (out2 is not None)
        _lib.profile_meta = dict(flops=2.0 * n_rows * D * D * (n_src + 1), rows=n_rows, k=k, n=D, fused=True,
                                 bytes=4.0 * n_rows * D * cols)
    call("mb_gated_mlp_fwd", C.byref(_lib.MbGatedMlp.from_buffer_copy(buf)), _stream())
    return z1, y, out2


def linear(x, W, bias=None, out_act=0, in_act=0, gate=None, res=None, res_w=None, scale=1.0, idx=None, out=None):
    """y[R,128*nb] = epilogue(x[R,128*ns] @ W^T): plain dense layer built on gemm()."""
    n_rows = x.shape[0] if idx is None else idx.shape[0]
    W = as_split(W)
    n_out, k = W.shape
    assert n_out % D == 0 and k % D == 0
    if out is None:
        out = new(n_rows, n_out, x)
    srcs = [S(x, idx, D * s, in_act) for s in range(k // D)]
    gemm(n_rows, [B(srcs, W, w_row=D * j, bias=bias, bias_off=D * j, gate=gate, gate_col=D * j, out_act=out_act,
                    res=res, res_col=D * j, res_w=res_w, out=out, out_col=D * j, scale=scale)
                  for j in range(n_out // D)])
    return out


# ------------------------------------------------------------------ row-wise kernels
def gate_fwd(z, wc, wg, want_h=True, res=None, res_w=None):
    n = z.shape[0]
    h = new(n, D, z) if want_h else None
    out2 = new(n, D, z) if res is not None else None
    call("mb_gate_fwd", n, ptr(z), ptr(wc), ptr(wg), ptr(h), ptr(res), ptr(res_w), ptr(out2), _stream())
    return h, out2


def gate_bwd(z, wc, wg, dh):
    dz = torch.empty_like(z)
    call("mb_gate_bwd", z.shape[0], ptr(z), ptr(wc), ptr(wg), ptr(dh), ptr(dz), _stream())
    return dz


def seg_attn_fwd(n_nodes, tgt_ptr, src_ptr, src_perm, emap, logits, h):
    agg_t, agg_s, stats = new(n_nodes, D, h), new(n_nodes, D, h), new(n_nodes, 4 * D, h)
    call("mb_seg_attn_fwd", n_nodes, ptr(tgt_ptr), ptr(src_ptr), ptr(src_perm), ptr(emap), ptr(logits), ptr(h),
         ptr(agg_t), ptr(agg_s), ptr(stats), _stream())
    return agg_t, agg_s, stats


def seg_attn_bwd(tgt, src, emap, logits, h, agg_t, agg_s, stats, dagg_t, dagg_s, dh_in, dh_map, dh_scale, gate=None):
    """``gate`` = (z2, w_core, w_gate): the row gradient goes straight through the gated MLP's tail adjoint and the
    first result is dz2 [rows,256] instead of dh [rows,128]."""
    n = h.shape[0]
    dlogits = new(n, 2 * D, h)
    if gate is None:
        first, gz, gc, gg = new(n, D, h), None, None, None
    else:
        gz, gc, gg = gate
        first = new(n, 2 * D, h)
    call("mb_seg_attn_bwd", n, ptr(tgt), ptr(src), 1, ptr(emap), ptr(logits), ptr(h), ptr(agg_t), ptr(agg_s),
         ptr(stats), ptr(dagg_t), ptr(dagg_s), ptr(dh_in), ptr(dh_map), float(dh_scale),
         ptr(first) if gate is None else None, ptr(dlogits), ptr(gz), ptr(gc), ptr(gg),
         None if gate is None else ptr(first), _stream())
    return first, dlogits


def seg_smooth_sum_fwd(n_nodes, tgt_ptr, emap, src, env, h):
    agg = new(n_nodes, D, h)
    call("mb_seg_smooth_sum_fwd", n_nodes, ptr(tgt_ptr), ptr(emap), ptr(src), 1, ptr(env), ptr(h), ptr(agg), _stream())
    return agg


def seg_smooth_sum_bwd_rows(tgt, src, emap, env, dagg, dh, accumulate=True, gate=None):
    """``gate`` = (z2, w_core, w_gate): returns dz2 [rows,256], the finished row gradient passed through the gated
    MLP's tail adjoint (dh is then read, if ``accumulate``, but not written); otherwise updates dh in place."""
    gz, gc, gg = gate if gate is not None else (None, None, None)
    dz = new(dh.shape[0], 2 * D, dh) if gate is not None else None
    call("mb_seg_smooth_sum_bwd_rows", dh.shape[0], ptr(tgt), ptr(src), 1, ptr(emap), ptr(env), ptr(dagg), ptr(dh),
         int(accumulate), ptr(gz), ptr(gc), ptr(gg), ptr(dz), _stream())
    return dz


def seg_smooth_sum_bwd_env(n_nodes, tgt_ptr, src_ptr, src_perm, tgt, src, u2d, rev, env, h, dagg, drow=None):
    denv = new(n_nodes, D, h)
    call("mb_seg_smooth_sum_bwd_env", n_nodes, ptr(tgt_ptr), ptr(src_ptr), ptr(src_perm), ptr(tgt), ptr(src), 1,
         ptr(u2d), ptr(rev), ptr(env), ptr(h), ptr(dagg), ptr(drow), ptr(denv), _stream())
    return denv


def mul_rows_gather(x, s, idx=None):
    """y[r] = x[r] * s[idx[r]] channel-wise."""
    y = torch.empty_like(x)
    call("mb_mul_rows_gather", x.shape[0], ptr(x), ptr(s), ptr(idx), ptr(y), _stream())
    return y


def pair_mean_res(n_bonds, u2d, rev, y, res=None, res_w=None):
    out = new(n_bonds, D, y)
    call("mb_pair_mean_res", n_bonds, ptr(u2d), ptr(rev), ptr(y), ptr(res), ptr(res_w), ptr(out), _stream())
    return out


def scale_rows(x, a, y=None, accumulate=False):
    if y is None:
        y = torch.empty_like(x)
    call("mb_scale_rows", x.shape[0], ptr(x), ptr(a), ptr(y), int(accumulate), _stream())
    return y


def small_linear_fwd(x, w):
    y = new(x.shape[0], D, x)
    call("mb_small_linear_fwd", x.shape[0], x.shape[1], ptr(x), ptr(w), ptr(y), _stream())
    return y


def small_linear_bwd(dy, w, dx=None, accumulate=False):
    k = w.shape[1]
    if dx is None:
        dx = new(dy.shape[0], k, dy)
    call("mb_small_linear_bwd", dy.shape[0], k, ptr(dy), ptr(w), ptr(dx), int(accumulate), _stream())
    return dx


def layernorm_fwd(x, w, b):
    y = torch.empty_like(x)
    call("mb_layernorm_fwd", x.shape[0], ptr(x), ptr(w), ptr(b), ptr(y), _stream())
    return y


def layernorm_bwd(x, w, dy):
    dx = torch.empty_like(x)
    call("mb_layernorm_bwd", x.shape[0], ptr(x), ptr(w), ptr(dy), ptr(dx), _stream())
    return dx


def rmsnorm_fwd(x, w):
    y = torch.empty_like(x)
    call("mb_rmsnorm_fwd", x.shape[0], ptr(x), ptr(w), ptr(y), _stream())
    return y


def rmsnorm_bwd(x, w, dy):
    dx = torch.empty_like(x)
    call("mb_rmsnorm_bwd", x.shape[0], ptr(x), ptr(w), ptr(dy), ptr(dx), _stream())
    return dx


def embedding(idx, offset, table):
    y = new(idx.shape[0], D, table)
    call("mb_embedding", idx.shape[0], ptr(idx), int(offset), ptr(table), ptr(y), _stream())
    return y


def head_dot_fwd(z, w, b, take_abs=False):
    out = torch.empty(z.shape[0], dtype=torch.float32, device=z.device)
    call("mb_head_dot_fwd", z.shape[0], z.shape[1], ptr(z), ptr(w), ptr(b), int(take_abs), ptr(out), _stream())
    return out


def head_dot_bwd(z, w, seed=None, seed_map=None):
    dz = torch.empty_like(z)
    call("mb_head_dot_bwd", z.shape[0], z.shape[1], ptr(z), ptr(w), ptr(seed), ptr(seed_map), ptr(dz), _stream())
    return dz


def silu_bwd(dy, z):
    dz = torch.empty_like(z)
    call("mb_silu_bwd", z.shape[0], ptr(dy), ptr(z), ptr(dz), _stream())
    return dz


def segment_sum_scalar(n_seg, seg_ptr, x):
    out = torch.empty(n_seg, dtype=torch.float32, device=x.device)
    call("mb_segment_sum_scalar", n_seg, ptr(seg_ptr), ptr(x), ptr(out), _stream())
    return out


# ------------------------------------------------------------------ geometry and bases
def edge_geometry_fwd(cart, lattice, atom_struct, center, neighbor, image):
    ne = center.shape[0]
    vec, unit = new(ne, 3, cart), new(ne, 3, cart)
    length = torch.empty(ne, dtype=torch.float32, device=cart.device)
    call("mb_edge_geometry_fwd", ne, ptr(cart), ptr(lattice), ptr(atom_struct), ptr(center), ptr(neighbor),
         ptr(image), ptr(vec), ptr(length), ptr(unit), _stream())
    return vec, length, unit


def edge_geometry_bwd(n_atoms, n_struct, edge_ptr, atom_ptr, rev, vec, length, unit, dlen, dunit):
    ne = rev.shape[0]
    g = new(ne, 3, vec)
    dcart, virial_atom, dstrain = new(n_atoms, 3, vec), new(n_atoms, 9, vec), new(n_struct, 9, vec)
    call("mb_edge_geometry_bwd", n_atoms, n_struct, ne, ptr(edge_ptr), ptr(atom_ptr), ptr(rev), ptr(vec), ptr(length),
         ptr(unit), ptr(dlen), ptr(dunit), ptr(g), ptr(dcart), ptr(virial_atom), ptr(dstrain), _stream())
    return dcart, dstrain.view(n_struct, 3, 3), g


def bessel_fwd(u2d, length, fa, ca, fb, cb, p):
    nb = u2d.shape[0]
    ra, rb = new(nb, 7, length), new(nb, 7, length)
    call("mb_bessel_fwd", nb, ptr(u2d), ptr(length), ptr(fa), float(ca), ptr(fb), float(cb), int(p), ptr(ra), ptr(rb),
         _stream())
    return ra, rb


def bessel_bwd(u2d, length, fa, ca, fb, cb, p, dra, drb):
    dlen = torch.zeros_like(length)
    call("mb_bessel_bwd", u2d.shape[0], ptr(u2d), ptr(length), ptr(fa), float(ca), ptr(fb), float(cb), int(p),
         ptr(dra), ptr(drb), ptr(dlen), _stream())
    return dlen


def gaussian_fwd(u2d, length, oa, ca, ob, cb):
    nb = u2d.shape[0]
    ra, rb = new(nb, 7, length), new(nb, 7, length)
    call("mb_gaussian_fwd", nb, ptr(u2d), ptr(length), ptr(oa), float(ca), ptr(ob), float(cb), ptr(ra), ptr(rb), _stream())
    return ra, rb


def gaussian_bwd(u2d, length, oa, ca, ob, cb, dra, drb):
    dlen = torch.zeros_like(length)
    call("mb_gaussian_bwd", u2d.shape[0], ptr(u2d), ptr(length), ptr(oa), float(ca), ptr(ob), float(cb), ptr(dra),
         ptr(drb), ptr(dlen), _stream())
    return dlen


def fourier_basis_fwd(line_graph, unit, freq):
    nt = line_graph.shape[0]
    basis = new(nt, 7, unit)
    call("mb_fourier_basis_fwd", nt, ptr(line_graph), ptr(unit), ptr(freq), ptr(basis), _stream())
    return basis


def fourier_basis_bwd(line_graph, unit, freq, dbasis):
    dunit = torch.zeros_like(unit)
    call("mb_fourier_basis_bwd", line_graph.shape[0], ptr(line_graph), ptr(unit), ptr(freq), ptr(dbasis), ptr(dunit),
         _stream())
    return dunit


def angle_basis_fwd(line_graph, unit, factor, cutoff):
    nt = line_graph.shape[0]
    basis = new(nt, 16, unit)
    call("mb_angle_basis_fwd", nt, ptr(line_graph), ptr(unit), float(factor), float(cutoff), ptr(basis), _stream())
    return basis


def angle_basis_bwd(line_graph, unit, factor, cutoff, dbasis):
    dunit = torch.zeros_like(unit)
    call("mb_angle_basis_bwd", line_graph.shape[0], ptr(line_graph), ptr(unit), float(factor), float(cutoff),
         ptr(dbasis), ptr(dunit), _stream())
    return dunit


# ------------------------------------------------------------------ GEMM core selection / status
_gemm_mode = 0


def set_gemm_mode(mode: str) -> None:
    """'tcgen05' (default): persistent tensor-core kernels (GEMM and fused gated MLP), 3-term BF16 operand split;
    'tcgen05_tf32': the persistent GEMM with a 3-term TF32 split; 'tcgen05_tile': a one-tile-per-CTA tensor-core
    kernel (3-term TF32); 'simt': exact fp32 FMA cross-check.  Outside the default mode a gated MLP is composed from
    two GEMM launches and the gate kernel.  A test knob."""
    global _gemm_mode
    _gemm_mode = {"tcgen05": 0, "simt": 1, "tcgen05_tile": 2, "tcgen05_tf32": 3}[mode]
    _lib.check(_lib.load().mb_set_gemm_mode(_gemm_mode), "mb_set_gemm_mode")


def gemm_status_async(pinned_int32: torch.Tensor) -> None:
    """Enqueue a copy of the tensor-core kernels' status word into a pinned int32 tensor (no synchronisation)."""
    assert pinned_int32.dtype == torch.int32 and pinned_int32.is_pinned()
    call("mb_gemm_status_async", pinned_int32.data_ptr(), _stream())


def gemm_status_clear() -> None:
    """Zero the status word in stream order."""
    call("mb_gemm_status_clear", _stream())


def selftest_wait_expiry() -> None:
    """Launch the one-CTA self-test whose bounded wait runs out (sets bit 0 of the status word)."""
    call("mb_selftest_wait_expiry", _stream())


def mma_rate(kind: str = "tf32", iters: int = 20000):
    """Timed tcgen05.mma issue rate with resident operands: (TFLOP/s, elapsed ms)."""
    ms, sms = C.c_float(0), C.c_int(0)
    k = {"tf32": 0, "bf16": 1}[kind]
    _lib.check(_lib.load().mb_bench_mma_rate(k, int(iters), C.byref(ms), C.byref(sms), _stream()), "mb_bench_mma_rate")
    flops = 2.0 * 128 * 128 * (8 if k == 0 else 16) * 4 * iters * sms.value
    return flops / (ms.value * 1e-3) / 1e12, ms.value


def gemm_status() -> int:
    """Synchronise and return (then clear) the tensor-core kernel's status word; 0 = no wait expired."""
    st = C.c_int(0)
    _lib.check(_lib.load().mb_gemm_status(C.byref(st), _stream()), "mb_gemm_status")
    return st.value
