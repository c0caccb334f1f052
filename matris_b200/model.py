"""MatRIS energy / force / stress / magmom evaluation on B200.

Host-side mirror of the reference's ``MatRIS`` module
(matris/model/model.py:30-317): same constructor arguments, ``config``,
``state_dict`` key names, ``from_dict`` / ``load`` checkpoint interface,
``graph_converter`` attribute and ``forward(graphs, task, is_training)`` result
dictionary.  All arithmetic runs in the CUDA kernels behind the C ABI; the
sub-blocks are ``torch.autograd.Function``s whose backward passes are
hand-written kernel sequences (data gradients only: weights are frozen at
inference), so forces = -dE/dr and stress = (1/V) dE/d(strain) come out of
``torch.autograd.grad`` exactly as in the reference's conservative head
(matris/model/readout.py:202-224).

Memory policy: a sub-block always keeps its inputs for the backward pass.  Its
internals are kept too while they fit in a fraction of the free device memory;
beyond that they are recomputed in the backward pass (the reference switches to
recomputation above 60,000 triplets, matris/model/interaction_block.py:15, 400-403).
"""
from __future__ import annotations

import os
from collections.abc import Sequence
from types import SimpleNamespace

import numpy as np
import torch
from torch import nn
from torch.autograd.function import once_differentiable

from . import ops
from ._lib import MbError
from .graph import BatchedGraph, GraphConverter, RadiusGraph, build_batched_graph, as_arrays
from .ops import B, OUT_ADD, OUT_ATOMIC, OUT_STORE, S, gemm
from .weights import BUFFER_KEYS, check_supported, full_config, random_state_dict, schema

GPA_PER_EV_A3 = 160.21766208  # matris/model/readout.py:215
D = 128


# ------------------------------------------------------------------ packed parameters
def _pack_gated(get, prefix, dev):
    """GatedMLP weights in kernel layout: first layers of core|gate stacked to
    [256,K], second layers stacked to [256,128], plus the transposes the backward
    GEMMs contract with."""
    c, g = prefix + "mlp_core.layers.", prefix + "mlp_gate.layers."
    w1 = torch.cat([get(c + "0.weight"), get(g + "0.weight")], 0).contiguous()
    w2 = torch.cat([get(c + "3.weight"), get(g + "3.weight")], 0).contiguous()
    SW = ops.SplitWeight
    return SimpleNamespace(
        w1=SW(w1), b1=torch.cat([get(c + "0.bias"), get(g + "0.bias")]).contiguous(),
        w2=SW(w2), b2=torch.cat([get(c + "3.bias"), get(g + "3.bias")]).contiguous(),
        w1t=SW(w1.t()),                                                           # [K,256]
        w2t=SW(torch.cat([get(c + "3.weight").t(), get(g + "3.weight").t()], 0)),  # [256,128]
        nc=get(prefix + "core_norm.weight").contiguous(), ng=get(prefix + "gate_norm.weight").contiguous(),
        k=w1.shape[1])


def _pack_mlp(get, prefix, bias):
    """The plain-MLP variant of an update block (graph_conv_mlp = "MLP"): nn.Sequential(MLP, RMSNorm)
    (matris/model/interaction_block.py:39-62, 172-184): weights, transposes for the backward products, norm weight."""
    w1, w2 = get(prefix + "0.layers.0.weight"), get(prefix + "0.layers.3.weight")
    SW = ops.SplitWeight
    return SimpleNamespace(
        kind="mlp", w1=SW(w1), w2=SW(w2), w1t=SW(w1.t()), w2t=SW(w2.t()),
        b1=get(prefix + "0.layers.0.bias").contiguous() if bias else None,
        b2=get(prefix + "0.layers.3.bias").contiguous() if bias else None,
        nw=get(prefix + "1.weight").contiguous(), k=w1.shape[1])


def _pack_ffn(get, prefix, bias):
    """node_FFN / edge_FFN (matris/model/interaction_block.py:197-210): two linear layers, biases only with use_bias."""
    w1, w2 = get(prefix + "layers.0.weight"), get(prefix + "layers.3.weight")
    SW = ops.SplitWeight
    b1 = get(prefix + "layers.0.bias").contiguous() if bias else None
    b2 = get(prefix + "layers.3.bias").contiguous() if bias else None
    return SimpleNamespace(w1=SW(w1), w2=SW(w2), w1t=SW(w1.t()), w2t=SW(w2.t()), b1=b1, b2=b2)


def pack_parameters(sd: dict, cfg: dict, device) -> SimpleNamespace:
    def get(k):
        return sd[k].detach().to(device=device, dtype=torch.float32)

    P = SimpleNamespace()
    P.emb_table = get("atom_embedding.embedding.weight").contiguous()
    SW = ops.SplitWeight
    P.emb_w = SW(get("atom_embedding.atom_swish_layer.linear.weight"))
    e = "edge_embedding."
    P.gaussian = str(cfg["distance_expansion"]).lower() == "gaussian"
    if P.gaussian:
        # GaussianExpansion: the offsets are a buffer, the coefficient is derived from them at construction
        # (matris/model/basis_function.py:203-205: float32 spacing, then Python float arithmetic)
        P.freq2, P.freq3 = get(e + "pairwise_rbf_expansion.offset").contiguous(), get(
            e + "threebody_rbf_expansion.offset").contiguous()
        P.coeff2, P.coeff3 = (-0.5 / (2.0 * (o[1] - o[0])).item() ** 2 for o in (P.freq2.cpu(), P.freq3.cpu()))
    else:
        P.freq2, P.freq3 = get(e + "pairwise_rbf_expansion.frequencies").contiguous(), get(
            e + "threebody_rbf_expansion.frequencies").contiguous()
    P.e_w1 = get(e + "edge_linear1.weight").contiguous()
    P.e_w2 = SW(get(e + "edge_linear2.weight"))
    P.e_w3 = SW(get(e + "swish_layer.linear.weight"))
    P.e_w2t, P.e_w3t = P.e_w2.t(), P.e_w3.t()
    P.e_lnw, P.e_lnb = get(e + "edge_init_norm.weight").contiguous(), get(e + "edge_init_norm.bias").contiguous()
    t = "three_body_embedding."
    P.fourier = str(cfg["three_body_expansion"]).lower() == "fourier"
    if P.fourier:
        P.t_freq = get(t + "expansion.frequencies").contiguous()
    else:
        P.sph_factor = float(sd[t + "expansion.factor"])
    P.t_wa = get(t + "angle_embedding.weight").contiguous()
    P.t_wb = SW(get(t + "swish_layer.linear.weight"))
    P.t_wbt = P.t_wb.t()
    P.layers = []
    if str(cfg["graph_conv_mlp"]).lower() == "mlp":
        pack_update = lambda prefix: _pack_mlp(get, prefix, bool(cfg["use_bias"]))  # noqa: E731
    else:
        pack_update = lambda prefix: _pack_gated(get, prefix, device)  # noqa: E731
    for i in range(int(cfg["num_layers"])):
        L = SimpleNamespace()
        for gname in ("atom", "line"):
            p = f"interaction_block.{i}.attn_block_{gname}_graph."
            A = SimpleNamespace(node=pack_update(p + "node_nonlinear_update."),
                                edge=pack_update(p + "edge_nonlinear_update."),
                                wn=get(p + "node_res_weight").reshape(-1).contiguous(),
                                we=get(p + "edge_res_weight").reshape(-1).contiguous())
            A.wst = SW(torch.cat([get(p + "source_weight_linear.weight"), get(p + "target_weight_linear.weight")],
                                 0))                  # [256,128]
            A.wstt = A.wst.t()                        # [128,256]
            setattr(L, "attn_" + gname, A)
            p = f"interaction_block.{i}.refine_block_{gname}_graph."
            R = SimpleNamespace(edge=pack_update(p + "edge_nonlinear_update."),
                                nffn=_pack_ffn(get, p + "node_FFN.", bool(cfg["use_bias"])),
                                effn=_pack_ffn(get, p + "edge_FFN.", bool(cfg["use_bias"])),
                                smoothed_edge=bool(cfg["use_smoothed_for_delta_edge"]) and gname == "atom",
                                wenv=get(p + "learnable_envelope.weight").contiguous(),
                                wn=get(p + "node_res_weight").reshape(-1).contiguous(),
                                we=get(p + "edge_res_weight").reshape(-1).contiguous())
            setattr(L, "refine_" + gname, R)
        P.layers.append(L)
    P.out_norm = get("readout_norm.weight").contiguous()
    h = "energy_head.energy_head.layers."
    P.h_w0, P.h_b0 = SW(get(h + "0.weight")), get(h + "0.bias").contiguous()
    P.h_w3, P.h_b3 = SW(get(h + "3.weight")), get(h + "3.bias").contiguous()
    P.h_w0t, P.h_w3t = P.h_w0.t(), P.h_w3.t()
    P.h_w6, P.h_b6 = get(h + "6.weight").reshape(-1).contiguous(), get(h + "6.bias").contiguous()
    m = "magmom_head.magmom_head.layers."
    P.m_w0, P.m_b0 = SW(get(m + "0.weight")), get(m + "0.bias").contiguous()
    P.m_w3, P.m_b3 = get(m + "3.weight").reshape(-1).contiguous(), get(m + "3.bias").contiguous()
    return P


# ------------------------------------------------------------------ row graphs
def row_graphs(g: BatchedGraph):
    """The two message-passing graphs in the form the kernels take: rows grouped by
    target node (tgt_ptr), the source-side grouping as a permutation."""
    if getattr(g, "_row_graphs", None) is None:
        atom = SimpleNamespace(is_atom=True, n_rows=g.n_edges, n_nodes=g.n_atoms, n_edge_rows=g.n_bonds,
                               tgt=g.center, src=g.neighbor, ctr=None, tgt_ptr=g.edge_ptr, src_ptr=g.edge_ptr,
                               src_perm=g.rev, emap=g.d2u, u2d=g.u2d, rev=g.rev, keep=False, skip_edge_out=False)
        line = None
        if g.n_triplets:
            c = g.lg_cols
            line = SimpleNamespace(is_atom=False, n_rows=g.n_triplets, n_nodes=g.n_bonds, n_edge_rows=g.n_triplets,
                                   ctr=c[0], tgt=c[1], src=c[3], tgt_ptr=g.trip_ptr, src_ptr=g.trip_src_ptr,
                                   src_perm=g.trip_src_perm, emap=None, u2d=None, rev=None, keep=False,
                                   skip_edge_out=False)
        g._row_graphs = (atom, line)
    return g._row_graphs


# ------------------------------------------------------------------ gated MLP building block
def gated_fwd(p, n_rows, srcs, want_h=True, res=None, res_w=None, save=True):
    """GatedMLP.forward (matris/model/functions.py:300-311) in one kernel: returns (z1, z2, h, out2) with
    z1 = X W1^T + b1 (core|gate pre-activations) and z2 = SiLU(z1) W2^T + b2 (pre-norm) only when ``save``."""
    if getattr(p, "kind", "gated") == "mlp":
        return _mlp_fwd(p, n_rows, srcs, want_h, res, res_w)
    return ops.gated_mlp_fwd(p, n_rows, srcs, want_h=want_h, res=res, res_w=res_w, save=save)


def _mlp_fwd(p, n_rows, srcs, want_h, res, res_w):
    """The plain-MLP variant of an update block: h = RMSNorm(W2 SiLU(W1 x + b1) + b2); same return convention, with
    z1 / z2 the two [rows,128] pre-activation / pre-norm tensors (always produced: they are the intermediates)."""
    like = srcs[0][0]
    z1, z2 = ops.new(n_rows, D, like), ops.new(n_rows, D, like)
    gemm(n_rows, [B(srcs, p.w1, bias=p.b1, out=z1)])
    gemm(n_rows, [B([S(z1, None, 0, 1)], p.w2, bias=p.b2, out=z2)])
    h = ops.rmsnorm_fwd(z2, p.nw)
    out2 = None
    if res is not None:
        out2 = h.clone()
        ops.scale_rows(res, res_w, y=out2, accumulate=True)
    return z1, z2, (h if want_h else None), out2


def _gate_args(p, z2):
    """What the kernels that produce a gated MLP's dh need to apply the tail adjoint themselves (None for the
    plain-MLP variant, whose tail is an RMSNorm handled in ``gated_bwd``)."""
    return None if getattr(p, "kind", "gated") == "mlp" else (z2, p.nc, p.ng)


def gated_bwd(p, n_rows, z1, z2, dh, dests, dz2=None):
    """Backward through the gated MLP: dests[c] = (tensor, idx, mode[, res, res_w]) for K segment c.  With ``res``
    the block stores ``gemm + res_w * res`` (the residual branch's gradient joins in the epilogue instead of in a
    separate scaling pass followed by an accumulate).  ``dz2``: the tail adjoint, where the producer of dh has
    already applied it (then ``dh`` is not read)."""
    if getattr(p, "kind", "gated") == "mlp":
        dy = ops.rmsnorm_bwd(z2, p.nw, dh.contiguous())
        da1 = torch.empty_like(z1)
        gemm(n_rows, [B([S(dy)], p.w2t, gate=z1, out=da1)])
        blocks, srcs = [], [S(da1)]  # one list of sources for all column blocks
        for c, dest in enumerate(dests):
            t, idx, mode = dest[:3]
            if t is None:
                continue
            res, res_w = (dest[3], dest[4]) if len(dest) > 3 else (None, None)
            blocks.append(B(srcs, p.w1t, w_row=D * c, out=t, out_idx=idx, mode=mode, res=res, res_w=res_w))
        gemm(n_rows, blocks)
        return
    if dz2 is None:
        dz2 = ops.gate_bwd(z2, p.nc, p.ng, dh)
    dz1 = torch.empty_like(z1)
    gemm(n_rows, [B([S(dz2, None, D * j)], p.w2t, w_row=D * j, gate=z1, gate_col=D * j, out=dz1, out_col=D * j)
                  for j in (0, 1)])
    del dz2
    blocks, srcs = [], [S(dz1, None, 0), S(dz1, None, D)]  # one list of sources for all column blocks
    for c, dest in enumerate(dests):
        t, idx, mode = dest[:3]
        if t is None:
            continue
        res, res_w = (dest[3], dest[4]) if len(dest) > 3 else (None, None)
        blocks.append(B(srcs, p.w1t, w_row=D * c, out=t, out_idx=idx, mode=mode, res=res, res_w=res_w))
    gemm(n_rows, blocks)


# ------------------------------------------------------------------ attention layer
def _attn_forward(P, rg, node, edge, save=True):
    """``save``: also return the internals the backward pass reads (z1, z2 of both gated MLPs are then written)."""
    R, Nn, Ne = rg.n_rows, rg.n_nodes, rg.n_edge_rows
    srcs = [S(edge, rg.emap), S(node, rg.tgt), S(node, rg.src)]
    if rg.is_atom:
        z1, z2, h, _ = gated_fwd(P.edge, R, srcs, save=save)
        edge_out = ops.pair_mean_res(Ne, rg.u2d, rg.rev, h, edge, P.we)
    else:
        z1, z2, h, edge_out = gated_fwd(P.edge, R, srcs, res=edge, res_w=P.we, save=save)
    logits = ops.linear(edge, P.wst)                      # [Ne,256]: source | target logits
    agg_t, agg_s, stats = ops.seg_attn_fwd(Nn, rg.tgt_ptr, rg.src_ptr, rg.src_perm, rg.emap, logits, h)
    z1n, z2n, _, node_out = gated_fwd(P.node, Nn, [S(node), S(agg_t), S(agg_s)], want_h=False, res=node, res_w=P.wn,
                                      save=save)
    return node_out, edge_out, (z1, z2, h, logits, agg_t, agg_s, stats, z1n, z2n)


class AttentionFn(torch.autograd.Function):
    """Graph_Attention_Layer.forward (matris/model/interaction_block.py:87-143)."""

    @staticmethod
    def forward(ctx, node, edge, P, rg):
        node, edge = node.contiguous(), edge.contiguous()
        keep = bool(rg.keep and any(ctx.needs_input_grad))
        node_out, edge_out, inter = _attn_forward(P, rg, node, edge, save=keep)
        ctx.save_for_backward(node, edge)
        ctx.P, ctx.rg = P, rg
        ctx.inter = inter if keep else None
        return node_out, edge_out

    @staticmethod
    @once_differentiable
    def backward(ctx, d_node_out, d_edge_out):
        node, edge = ctx.saved_tensors
        P, rg = ctx.P, ctx.rg
        R, Nn, Ne = rg.n_rows, rg.n_nodes, rg.n_edge_rows
        d_node_out, d_edge_out = d_node_out.contiguous(), d_edge_out.contiguous()
        inter, ctx.inter = ctx.inter, None
        if inter is None:  # internals were not kept: recompute them from the saved inputs
            _, _, inter = _attn_forward(P, rg, node, edge)
        z1, z2, h, logits, agg_t, agg_s, stats, z1n, z2n = inter
        del inter
        # node update
        d_node = ops.scale_rows(d_node_out, P.wn)
        dagg_t, dagg_s = ops.new(Nn, D, node), ops.new(Nn, D, node)
        gated_bwd(P.node, Nn, z1n, z2n, d_node_out,
                  [(d_node, None, OUT_ADD), (dagg_t, None, OUT_STORE), (dagg_s, None, OUT_STORE)])
        del z1n, z2n
        # softmax-weighted aggregation
        # (the row gradient dh goes straight on through the gated MLP's tail adjoint: dz2 comes back instead)
        gate = _gate_args(P.edge, z2)
        dh, dlogits = ops.seg_attn_bwd(rg.tgt, rg.src, rg.emap, logits, h, agg_t, agg_s, stats, dagg_t, dagg_s,
                                       d_edge_out, rg.emap, 0.5 if rg.is_atom else 1.0, gate=gate)
        dz2, dh = (dh, None) if gate is not None else (None, dh)
        del logits, h, agg_t, agg_s, stats, dagg_t, dagg_s
        # edge update (line graph: rows map one to one, so the residual gradient we * d_edge_out rides in the
        # epilogue of the store; atom graph: two directed rows add into one bond row, so it is laid down first)
        emode = OUT_ATOMIC if rg.is_atom else OUT_ADD
        if rg.is_atom:
            d_edge = ops.scale_rows(d_edge_out, P.we)
            edge_dest = (d_edge, rg.emap, OUT_ATOMIC)
        else:
            d_edge = torch.empty_like(d_edge_out)
            edge_dest = (d_edge, None, OUT_STORE, d_edge_out, P.we)
        gated_bwd(P.edge, R, z1, z2, dh, [edge_dest, (d_node, rg.tgt, OUT_ATOMIC), (d_node, rg.src, OUT_ATOMIC)],
                  dz2=dz2)
        del z1, z2, dh, dz2
        gemm(R, [B([S(dlogits, None, 0), S(dlogits, None, D)], P.wstt, out=d_edge, out_idx=rg.emap, mode=emode)])
        return d_node, d_edge, None, None


# ------------------------------------------------------------------ refinement layer
def _refine_forward(P, rg, node, edge, rbf, atom_feat, save=True, want_edge=True):
    R, Nn, Ne = rg.n_rows, rg.n_nodes, rg.n_edge_rows
    if rg.is_atom:
        srcs = [S(edge, rg.emap), S(node, rg.tgt), S(node, rg.src)]
    else:
        srcs = [S(edge), S(atom_feat, rg.ctr), S(node, rg.tgt), S(node, rg.src)]
    z1, z2, h, _ = gated_fwd(P.edge, R, srcs, save=save)
    env = ops.small_linear_fwd(rbf, P.wenv)               # [bonds,128]
    agg = ops.seg_smooth_sum_fwd(Nn, rg.tgt_ptr, rg.emap, None if rg.is_atom else rg.src, env, h)
    zn, _, node_out = ops.ffn_fwd(P.nffn, agg, want_y=False, res=node, res_w=P.wn, save=save)
    # the edge update reads the unsmoothed rows unless use_smoothed_for_delta_edge (atom graph only,
    # interaction_block.py:262-266): then it reads h * s, s = the envelope row of the edge's bond
    if not want_edge:  # the last layer's edge update feeds nothing
        return node_out, None, (z1, z2, h, env, zn, None)
    ffn_in = ops.mul_rows_gather(h, env, rg.emap) if P.smoothed_edge else h
    if rg.is_atom:
        ze, y, _ = ops.ffn_fwd(P.effn, ffn_in, save=save)
        edge_out = ops.pair_mean_res(Ne, rg.u2d, rg.rev, y, edge, P.we)
    else:
        ze, _, edge_out = ops.ffn_fwd(P.effn, ffn_in, want_y=False, res=edge, res_w=P.we, save=save)
    return node_out, edge_out, (z1, z2, h, env, zn, ze)


class RefineFn(torch.autograd.Function):
    """Refinement.forward (matris/model/interaction_block.py:218-278)."""

    @staticmethod
    def forward(ctx, node, edge, rbf, atom_feat, P, rg):
        node, edge, rbf = node.contiguous(), edge.contiguous(), rbf.contiguous()
        if atom_feat is not None:
            atom_feat = atom_feat.contiguous()
        keep = bool(rg.keep and any(ctx.needs_input_grad))
        want_edge = not rg.skip_edge_out
        node_out, edge_out, inter = _refine_forward(P, rg, node, edge, rbf, atom_feat, save=keep, want_edge=want_edge)
        ctx.save_for_backward(node, edge, rbf, atom_feat)
        ctx.P, ctx.rg, ctx.want_edge = P, rg, want_edge
        ctx.inter = inter if keep else None
        if not want_edge:  # a placeholder nobody reads, so that the signature stays (node, edge)
            edge_out = edge.new_empty(0)
            ctx.mark_non_differentiable(edge_out)
        return node_out, edge_out

    @staticmethod
    @once_differentiable
    def backward(ctx, d_node_out, d_edge_out):
        node, edge, rbf, atom_feat = ctx.saved_tensors
        P, rg = ctx.P, ctx.rg
        R, Nn, Ne = rg.n_rows, rg.n_nodes, rg.n_edge_rows
        want_edge = ctx.want_edge
        d_node_out = d_node_out.contiguous()
        d_edge_out = d_edge_out.contiguous() if want_edge else None
        inter, ctx.inter = ctx.inter, None
        if inter is None:
            _, _, inter = _refine_forward(P, rg, node, edge, rbf, atom_feat, want_edge=want_edge)
        z1, z2, h, env, zn, ze = inter
        del inter
        # node FFN
        d_node = ops.scale_rows(d_node_out, P.wn)
        dzn = ops.linear(d_node_out, P.nffn.w2t, gate=zn)
        dagg = ops.linear(dzn, P.nffn.w1t)
        del zn, dzn
        # edge FFN (atom graph: the mean over the two directions is a gather * 0.5)
        drow = None
        if want_edge:
            if rg.is_atom:
                dze = ops.linear(d_edge_out, P.effn.w2t, gate=ze, scale=0.5, idx=rg.emap)
            else:
                dze = ops.linear(d_edge_out, P.effn.w2t, gate=ze)
            dh = ops.linear(dze, P.effn.w1t)
            del ze, dze
            if P.smoothed_edge:  # dh so far is the gradient of the smoothed rows h * s
                drow, dh = dh, ops.mul_rows_gather(dh, env, rg.emap)
        else:
            dh = ops.new(R, D, dagg)  # no edge update, no gradient from it: the aggregation's term starts the row
        # smoothed aggregation
        src = None if rg.is_atom else rg.src
        dz2 = ops.seg_smooth_sum_bwd_rows(rg.tgt, src, rg.emap, env, dagg, dh, accumulate=want_edge,
                                          gate=_gate_args(P.edge, z2))  # with a gate: dh is finished in registers
        denv = ops.seg_smooth_sum_bwd_env(env.shape[0], rg.tgt_ptr, None if rg.is_atom else rg.src_ptr, rg.src_perm,
                                          rg.tgt, src if src is not None else rg.src, rg.u2d, rg.rev, env, h, dagg,
                                          drow=drow)
        del drow
        d_rbf = ops.small_linear_bwd(denv, P.wenv)
        del env, denv, dagg, h
        # gated MLP
        if rg.is_atom:
            d_atom = None
            d_edge = ops.scale_rows(d_edge_out, P.we) if want_edge else torch.zeros_like(edge)
            dests = [(d_edge, rg.emap, OUT_ATOMIC), (d_node, rg.tgt, OUT_ATOMIC), (d_node, rg.src, OUT_ATOMIC)]
        else:
            d_atom = torch.zeros_like(atom_feat)
            d_edge = torch.empty_like(edge)  # stored once: gemm (+ we * d_edge_out in the epilogue)
            edge_dest = (d_edge, None, OUT_STORE, d_edge_out, P.we) if want_edge else (d_edge, None, OUT_STORE)
            dests = [edge_dest, (d_atom, rg.ctr, OUT_ATOMIC), (d_node, rg.tgt, OUT_ATOMIC), (d_node, rg.src, OUT_ATOMIC)]
        gated_bwd(P.edge, R, z1, z2, dh, dests, dz2=dz2)
        return d_node, d_edge, d_rbf, d_atom, None, None


# ------------------------------------------------------------------ geometry, embeddings, readout
class EdgeGeometryFn(torch.autograd.Function):
    """Edge vectors / lengths / unit vectors and their adjoint: forces and virial
    (matris/model/processgraph.py:169-199, matris/model/readout.py:202-224).  ``strain`` is the
    zero strain leaf; the forward value does not depend on it, its gradient is sym(sum v (x) dE/dv)."""

    @staticmethod
    def forward(ctx, cart, strain, g):
        vec, length, unit = ops.edge_geometry_fwd(cart.contiguous(), g.lattice32, g.atom_struct, g.center, g.neighbor,
                                                  g.image)
        ctx.save_for_backward(vec, length, unit)
        ctx.g, ctx.has_strain = g, strain is not None
        ctx.mark_non_differentiable(vec)
        return length, unit, vec

    @staticmethod
    @once_differentiable
    def backward(ctx, dlen, dunit, _dvec):
        vec, length, unit = ctx.saved_tensors
        g = ctx.g
        dcart, dstrain, _ = ops.edge_geometry_bwd(g.n_atoms, g.n_struct, g.edge_ptr, g.atom_ptr, g.rev, vec, length,
                                                  unit, dlen.contiguous(), dunit.contiguous())
        return dcart, (dstrain if ctx.has_strain else None), None


def _rbf_forward(P, g, length, cfg):
    if P.gaussian:
        return ops.gaussian_fwd(g.u2d, length, P.freq2, P.coeff2, P.freq3, P.coeff3)
    return ops.bessel_fwd(g.u2d, length, P.freq2, cfg["pairwise_cutoff"], P.freq3, cfg["three_body_cutoff"],
                          cfg["envelope_exponent"])


def _angle_basis(P, g, unit, cfg):
    if P.fourier:
        return ops.fourier_basis_fwd(g.line_graph, unit, P.t_freq)
    return ops.angle_basis_fwd(g.line_graph, unit, P.sph_factor, cfg["pairwise_cutoff"])


def _edge_embed_forward(P, g, length, cfg):
    rbf2, rbf3 = _rbf_forward(P, g, length, cfg)
    e1 = ops.small_linear_fwd(rbf2, P.e_w1)
    e2 = ops.linear(e1, P.e_w2)
    # both directed copies of a bond carry the same row, so their mean is the row itself:
    # the expand-to-directed / average-back pair of the reference is the identity here
    e3 = ops.layernorm_fwd(e2, P.e_lnw, P.e_lnb)
    return rbf2, rbf3, e2, e3


class EdgeEmbedFn(torch.autograd.Function):
    """EdgeBasisEmbedding.forward (matris/model/feature_embed.py:114-148)."""

    @staticmethod
    def forward(ctx, length, P, g, cfg):
        length = length.contiguous()
        rbf2, rbf3, _, e3 = _edge_embed_forward(P, g, length, cfg)
        edge = ops.linear(e3, P.e_w3, out_act=1)
        ctx.save_for_backward(length)
        ctx.P, ctx.g, ctx.cfg = P, g, cfg
        return edge, rbf2, rbf3

    @staticmethod
    @once_differentiable
    def backward(ctx, d_edge, d_rbf2, d_rbf3):
        (length,) = ctx.saved_tensors
        P, g, cfg = ctx.P, ctx.g, ctx.cfg
        _, _, e2, e3 = _edge_embed_forward(P, g, length, cfg)
        z = ops.linear(e3, P.e_w3)
        dz = ops.silu_bwd(d_edge.contiguous(), z)
        de3 = ops.linear(dz, P.e_w3t)
        de2 = ops.layernorm_bwd(e2, P.e_lnw, de3)
        de1 = ops.linear(de2, P.e_w2t)
        d2 = d_rbf2.contiguous().clone()
        ops.small_linear_bwd(de1, P.e_w1, d2, accumulate=True)
        if P.gaussian:
            dlen = ops.gaussian_bwd(g.u2d, length, P.freq2, P.coeff2, P.freq3, P.coeff3, d2, d_rbf3.contiguous())
        else:
            dlen = ops.bessel_bwd(g.u2d, length, P.freq2, cfg["pairwise_cutoff"], P.freq3, cfg["three_body_cutoff"],
                                  cfg["envelope_exponent"], d2, d_rbf3.contiguous())
        return dlen, None, None, None


class AngleEmbedFn(torch.autograd.Function):
    """ThreebodyEmbedding.forward (matris/model/feature_embed.py:183-203)."""

    @staticmethod
    def forward(ctx, unit, P, g, cfg):
        unit = unit.contiguous()
        basis = _angle_basis(P, g, unit, cfg)
        t1 = ops.small_linear_fwd(basis, P.t_wa)
        trip = ops.linear(t1, P.t_wb, out_act=1)
        ctx.save_for_backward(unit)
        ctx.P, ctx.g, ctx.cfg = P, g, cfg
        return trip

    @staticmethod
    @once_differentiable
    def backward(ctx, d_trip):
        (unit,) = ctx.saved_tensors
        P, g, cfg = ctx.P, ctx.g, ctx.cfg
        basis = _angle_basis(P, g, unit, cfg)
        t1 = ops.small_linear_fwd(basis, P.t_wa)
        z = ops.linear(t1, P.t_wb)
        del basis, t1
        dz = ops.silu_bwd(d_trip.contiguous(), z)
        dt1 = ops.linear(dz, P.t_wbt)
        del z, dz
        dbasis = ops.small_linear_bwd(dt1, P.t_wa)
        if P.fourier:
            dunit = ops.fourier_basis_bwd(g.line_graph, unit, P.t_freq, dbasis)
        else:
            dunit = ops.angle_basis_bwd(g.line_graph, unit, P.sph_factor, cfg["pairwise_cutoff"], dbasis)
        return dunit, None, None, None


class EnergyFn(torch.autograd.Function):
    """readout_norm + EnergyHead + per-structure sum (matris/model/model.py:216-218,
    matris/model/readout.py:66-75).  Also returns the normalised features for the magmom head."""

    @staticmethod
    def forward(ctx, node, P, g):
        node = node.contiguous()
        nn_ = ops.rmsnorm_fwd(node, P.out_norm)
        z1 = ops.linear(nn_, P.h_w0, bias=P.h_b0)
        z2 = ops.linear(z1, P.h_w3, bias=P.h_b3, in_act=1)
        e_atom = ops.head_dot_fwd(z2, P.h_w6, P.h_b6)
        energy = ops.segment_sum_scalar(g.n_struct, g.atom_ptr, e_atom)
        ctx.save_for_backward(node)
        ctx.P, ctx.g = P, g
        ctx.mark_non_differentiable(nn_)
        return energy, nn_

    @staticmethod
    @once_differentiable
    def backward(ctx, d_energy, _d_nn):
        (node,) = ctx.saved_tensors
        P, g = ctx.P, ctx.g
        nn_ = ops.rmsnorm_fwd(node, P.out_norm)
        z1 = ops.linear(nn_, P.h_w0, bias=P.h_b0)
        z2 = ops.linear(z1, P.h_w3, bias=P.h_b3, in_act=1)
        dz2 = ops.head_dot_bwd(z2, P.h_w6, d_energy.contiguous(), g.atom_struct)
        dz1 = ops.linear(dz2, P.h_w3t, gate=z1)
        dnn = ops.linear(dz1, P.h_w0t)
        return ops.rmsnorm_bwd(node, P.out_norm, dnn), None, None


# ------------------------------------------------------------------ the module
class _Node(nn.Module):
    """Anonymous container so that parameters sit under the reference's dotted key names."""


def kept_layers_for(n_layers: int, n_triplets: int, n_edges: int, avail: float) -> int:
    """The memory policy of ``MatRIS.kept_layers`` as a function of the available bytes."""
    per_layer = 6.7e3 * n_triplets + 6.2e3 * n_edges
    budget = 0.45 * avail
    n_keep = n_layers if per_layer * n_layers < budget else max(0, int(budget // max(per_layer, 1.0)))
    # Second bound, on the peak of the backward pass (saved inputs of all layers + the temporaries of one recomputed
    # layer + gradients).  Measured on three graph shapes (4.1 M - 6.6 M triplets, 1.0 M - 1.7 M directed edges):
    # 17.4 KB per triplet + 13.8 KB per directed edge with nothing kept, growing by 2.5 KB per triplet + 4.3 KB per
    # directed edge per kept layer; that peak must stay below 92 % of the memory.
    base = 18.0e3 * n_triplets + 14.2e3 * n_edges
    step = 2.6e3 * n_triplets + 4.4e3 * n_edges
    # Third bound, on the end of the forward pass (saved inputs of all layers, about 17 KB per triplet, + the kept
    # internals).
    inputs = 17.0e3 * n_triplets + 2.0e3 * n_edges
    while 0 < n_keep < n_layers and max(base + step * n_keep, inputs + per_layer * n_keep) > 0.92 * avail:
        n_keep -= 1
    return n_keep


def split_ranges(triplets, edges, fits) -> list[tuple[int, int]]:
    """Cut a list of structures (per-structure triplet and directed-edge counts) into contiguous ranges with
    ``fits(sum of triplets, sum of edges)`` true for every range, as few as a greedy walk needs and then balanced
    by triplet + edge rows.  A structure that does not fit alone gets a range of its own."""
    triplets, edges = np.asarray(triplets, dtype=np.int64), np.asarray(edges, dtype=np.int64)
    n = len(triplets)
    greedy, a, t, e = [], 0, 0, 0
    for i in range(n):
        if i > a and not fits(t + int(triplets[i]), e + int(edges[i])):
            greedy.append((a, i))
            a, t, e = i, 0, 0
        t, e = t + int(triplets[i]), e + int(edges[i])
    greedy.append((a, n))
    if len(greedy) == 1:
        return greedy
    cum = np.cumsum(triplets + edges, dtype=np.float64)
    for parts in range(len(greedy), min(n, len(greedy) + 2) + 1):
        cuts = [0] + [int(np.searchsorted(cum, cum[-1] * k / parts, side="left")) + 1 for k in range(1, parts)] + [n]
        ranges = [(cuts[k], cuts[k + 1]) for k in range(parts)]
        if all(b > a for a, b in ranges) and all(fits(int(triplets[a:b].sum()), int(edges[a:b].sum())) or b - a == 1
                                                 for a, b in ranges):
            return ranges
    return greedy


class MatRIS(nn.Module):
    """Drop-in for the reference's ``MatRIS`` (matris/model/model.py:30-317)."""

    def __init__(self, num_layers: int = 6, node_feat_dim: int = 128, edge_feat_dim: int = 128,
                 three_body_feat_dim: int = 128, mlp_hidden_dims=(128, 128), dropout: float = 0.0,
                 use_bias: bool = False, distance_expansion: str = "Bessel", three_body_expansion: str = "SH",
                 num_radial: int = 7, num_angular: int = 7, max_l: int = 4, max_n: int = 4,
                 envelope_exponent: int = 8, graph_conv_mlp: str = "GateMLP", activation_type: str = "silu",
                 norm_type: str = "rms", pairwise_cutoff: float = 6, three_body_cutoff: float = 4,
                 use_smoothed_for_delta_edge: bool = False, learnable_basis: bool = True, is_intensive: bool = True,
                 is_conservation: bool = True, reference_energy: str | None = None, seed: int = 0):
        super().__init__()
        self.config = {k: v for k, v in locals().items() if k not in ("self", "__class__", "seed")}
        cfg = full_config(self.config)
        check_supported(cfg)
        self.is_intensive = is_intensive
        self.graph_converter = GraphConverter(atom_graph_cutoff=pairwise_cutoff, line_graph_cutoff=three_body_cutoff)
        for key, value in random_state_dict(cfg, seed=seed).items():
            self._register(key, value, buffer=key in BUFFER_KEYS, trainable=not key.startswith("reference_energy"))
        self._packed = None
        self._ref_table = None
        self._packed_device = None
        self.last_batch = None
        # None: decide per call from free memory; True / False: keep / recompute all; n: keep the last n layers' internals
        self.keep_activations = None
        # plan as if at most this many bytes of device memory were available (None: what the device has left)
        self.memory_limit_bytes = None

    # -- parameter tree -------------------------------------------------------------------
    def _register(self, key, value, buffer, trainable):
        mod = self
        parts = key.split(".")
        for p in parts[:-1]:
            if not hasattr(mod, p):
                mod.add_module(p, _Node())
            mod = getattr(mod, p)
        if buffer:
            mod.register_buffer(parts[-1], value.clone())
        else:
            mod.register_parameter(parts[-1], nn.Parameter(value.clone(), requires_grad=False))

    def get_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def _apply(self, fn, *a, **k):
        self._packed = None
        self._ref_table = None
        out = super()._apply(fn, *a, **k)
        # graphs are built where the weights live: a batch on another GPU would be read through peer pointers
        # (or fault without peer access) by kernels launched on this one
        dev = self.device
        self.graph_converter.device = dev if dev.type == "cuda" else None
        return out

    def load_state_dict(self, state_dict, strict: bool = True, **kw):
        self._packed = None
        self._ref_table = None
        return super().load_state_dict(state_dict, strict=strict, **kw)

    def packed(self, device):
        if self._packed is None or self._packed_device != device:
            self._packed = pack_parameters(self.state_dict(), full_config(self.config), device)
            self._packed_device = device
        return self._packed

    @property
    def device(self):
        return next(self.parameters()).device

    # -- checkpoint interface ---------------------------------------------------------------
    @classmethod
    def from_dict(cls, dct: dict):
        model = MatRIS(**dct["config"])
        model.load_state_dict(dct["state_dict"])
        return model

    @classmethod
    def load(cls, model_name: str = "matris_10m_oam", device: str | None = None, path: str | None = None):
        """Load a checkpoint ``{"config", "state_dict"}``.  ``model_name`` resolves to
        ``~/.cache/matris/MatRIS_10M_{OAM,MP}.pth.tar`` exactly like the reference
        (matris/model/model.py:262-317); ``path`` (an extension) names the file directly."""
        if path is None:
            model_name = model_name.lower()
            supported = ["matris_10m_oam", "matris_10m_mp"]
            if os.path.isfile(model_name):
                path = model_name
            elif model_name not in supported:
                raise ValueError(f"Unsupported model_name: {model_name}. Supported models are: {supported}")
            else:
                files = {"matris_10m_oam": "MatRIS_10M_OAM.pth.tar", "matris_10m_mp": "MatRIS_10M_MP.pth.tar"}
                urls = {"matris_10m_oam": "https://figshare.com/ndownloader/files/59142728",
                        "matris_10m_mp": "https://figshare.com/ndownloader/files/59143058"}
                cache_dir = os.path.expanduser("~/.cache/matris")
                os.makedirs(cache_dir, exist_ok=True)
                path = os.path.join(cache_dir, files[model_name])
                if not os.path.exists(path):
                    print(f"Checkpoint not found, downloading to {path} ...")
                    torch.hub.download_url_to_file(urls[model_name], path)
        if device is None:
            device = "cuda"
        ckpt = torch.load(path, map_location=torch.device("cpu"), weights_only=False)
        model = MatRIS.from_dict(ckpt).to(device)
        print(f"Loading {model_name} successfully, running on {device}.")
        return model

    # -- evaluation -------------------------------------------------------------------------
    def _as_batch(self, graphs) -> BatchedGraph:
        if isinstance(graphs, BatchedGraph):
            if graphs.device != self.device:
                raise ValueError(f"the batch lives on {graphs.device} but the model on {self.device}: build it with "
                                 "model.graph_converter (which follows the model) or pass device= to "
                                 "build_batched_graph")
            return graphs
        if isinstance(graphs, RadiusGraph):
            graphs = [graphs]
        graphs = list(graphs)
        if not graphs:
            raise ValueError("no graphs")
        b0 = getattr(graphs[0], "_batch", None)
        if (b0 is not None and len(graphs) == b0.n_struct and b0.device == self.device
                and all(getattr(g, "_batch", None) is b0 and g._index == i for i, g in enumerate(graphs))):
            return b0
        arrays = [g.source_arrays() if isinstance(g, RadiusGraph) else as_arrays(g) for g in graphs]
        return build_batched_graph([a[0] for a in arrays], [a[1] for a in arrays], [a[2] for a in arrays],
                                   self.config["pairwise_cutoff"], self.config["three_body_cutoff"], self.device)

    def forward(self, graphs: Sequence[RadiusGraph] | BatchedGraph, task: str = "ef", is_training: bool = False):
        """Same result dictionary as the reference's ``MatRIS.forward`` (model.py:183-250): ``e`` [B] energy per
        atom including the reference energy, ``f`` tuple of [n_i,3], ``s`` list of [3,3] in GPa, ``m`` list of
        [n_i], ``atoms_per_graph``, ``ref_energy``.  ``graphs`` may also be a ``BatchedGraph``."""
        if is_training:
            raise NotImplementedError("matris_b200 evaluates frozen models only (no parameter gradients)")
        if self.device.type != "cuda":
            raise RuntimeError("matris_b200 runs on a CUDA device only: move the model with .to('cuda')")
        g = self._as_batch(graphs)
        self.last_batch = g
        with torch.cuda.device(self.device):
            # The GEMM kernels bound every wait and raise a status word instead of hanging.  The word of the previous
            # evaluation was copied to pinned memory in stream order; it is read here, so a failure surfaces at the
            # latest one call later and costs no synchronisation.
            flag = getattr(self, "_gemm_flag", None)
            if flag is None:
                flag = self._gemm_flag = torch.zeros(1, dtype=torch.int32).pin_memory()
            self.check_status()
            with ops.pinned_stream():  # one stream look-up per evaluation instead of one per launch
                out = self._evaluate(g, task)
            ops.gemm_status_async(flag)
            return out

    def check_status(self) -> None:
        """Raise if a bounded wait of a tensor-core kernel expired in an evaluation whose status word has reached
        the host (``forward`` enqueues the copy; it is valid once the stream has been synchronised, e.g. by reading
        a result).  The word is cleared on raising, so that one expiry does not disable the model."""
        flag = getattr(self, "_gemm_flag", None)
        if flag is not None and int(flag[0]) != 0:
            status = int(flag[0])
            flag.zero_()
            with torch.cuda.device(self.device):
                ops.gemm_status_clear()
            raise MbError(f"a tensor-core kernel's bounded wait expired (status {status}): the results of that "
                          "evaluation are invalid")

    # -- memory policy -----------------------------------------------------------------------
    def _available_bytes(self) -> float:
        """Memory the allocator can still hand out = device total - what lives outside this allocator - what it has
        allocated (capped by ``memory_limit_bytes`` when set).  The driver query behind the middle term costs
        milliseconds (during which the GPU idles at the start of an evaluation), so it is refreshed every 64th call
        only; the last term is a counter."""
        st = getattr(self, "_mem_state", None)
        if st is None:
            st = self._mem_state = {"calls": 0, "total": 0, "outside": 0}
        if st["calls"] % 64 == 0:
            free, total = torch.cuda.mem_get_info(self.device)
            st["total"], st["outside"] = total, total - free - torch.cuda.memory_reserved(self.device)
        st["calls"] += 1
        avail = st["total"] - st["outside"] - torch.cuda.memory_allocated(self.device)
        if self.memory_limit_bytes is not None:
            avail = min(avail, float(self.memory_limit_bytes))
        return avail

    def kept_layers(self, n_triplets: int, n_edges: int, avail: float | None = None) -> int:
        """How many (last) layers keep their sub-block internals for the backward pass on a batch with that many
        triplet rows and directed edges; the internals of the earlier layers are recomputed there.  The internals
        take ~6.7 KB per triplet row and ~6.2 KB per directed edge per layer and are consumed and released last
        layer first: all layers are kept when that fits in 45 % of the available memory, otherwise as many as do,
        within two more bounds (see below).  ``keep_activations`` overrides: True / False / a number of layers."""
        n_layers = int(self.config["num_layers"])
        keep = self.keep_activations
        if keep is not None:
            if isinstance(keep, bool):
                return n_layers if keep else 0
            return max(0, min(n_layers, int(keep)))
        return kept_layers_for(n_layers, n_triplets, n_edges, self._available_bytes() if avail is None else avail)

    def split_for_memory(self, g: BatchedGraph, headroom: float = 0.93) -> list[tuple[int, int]]:
        """Contiguous ranges of the structures of batch ``g`` such that every range, evaluated as a batch of its own,
        keeps the internals of all layers (no recomputation in the backward pass): ``[(0, n_struct)]`` when the
        whole batch does.  Structures are independent, so evaluating the ranges one after another gives the same
        results; on a batch that would recompute most layers it is about a fifth faster.  ``headroom`` scales the
        available memory the plan may count on (the ranges' own graphs and results take some)."""
        if g.n_struct <= 1 or self.keep_activations is not None:
            return [(0, g.n_struct)]
        n_layers = int(self.config["num_layers"])
        avail = headroom * self._available_bytes()
        if kept_layers_for(n_layers, g.n_triplets, g.n_edges, avail / headroom) == n_layers:
            return [(0, g.n_struct)]
        _, ep, _, tp = g.structure_slices()
        return split_ranges(np.diff(tp), np.diff(ep), lambda t, e: kept_layers_for(n_layers, t, e, avail) == n_layers)

    def _evaluate(self, g: BatchedGraph, task: str):
        cfg = self.config
        P = self.packed(self.device)
        atom_rg, line_rg = row_graphs(g)
        want_f, want_s = "f" in task, "s" in task
        need_grad = want_f or want_s
        n_layers = len(P.layers)
        n_keep = self.kept_layers(g.n_triplets, g.n_edges)
        self.last_kept_layers = n_keep
        out = {}
        with torch.set_grad_enabled(need_grad):
            cart = g.cart32.detach().clone().requires_grad_(need_grad)
            strain = None
            if want_s:
                strain = torch.zeros(g.n_struct, 3, 3, dtype=torch.float32, device=cart.device, requires_grad=True)
            length, unit, _ = EdgeGeometryFn.apply(cart, strain, g)
            node = ops.linear(ops.embedding(g.numbers, -1, P.emb_table), P.emb_w, out_act=1)
            edge, rbf2, rbf3 = EdgeEmbedFn.apply(length, P, g, cfg)
            trip = AngleEmbedFn.apply(unit, P, g, cfg) if line_rg is not None else None
            for i, L in enumerate(P.layers):
                atom_rg.keep = i >= n_layers - n_keep
                # after the last layer only the atom features are read (matris/model/model.py:215-231; the edge features
                # go to the non-conservative force head only): its two refinements need no edge update
                atom_rg.skip_edge_out = i == n_layers - 1
                if line_rg is not None:
                    line_rg.keep, line_rg.skip_edge_out = atom_rg.keep, atom_rg.skip_edge_out
                e_att, t_att = edge, trip
                if trip is not None:
                    e_att, t_att = AttentionFn.apply(edge, trip, L.attn_line, line_rg)
                n_att, e_att = AttentionFn.apply(node, e_att, L.attn_atom, atom_rg)
                e_upd, t_upd = edge, trip
                if trip is not None:
                    e_upd, t_upd = RefineFn.apply(e_att, t_att, rbf3, n_att, L.refine_line, line_rg)
                node, edge = RefineFn.apply(n_att, e_upd, rbf2, None, L.refine_atom, atom_rg)
                trip = t_upd
            energy, node_n = EnergyFn.apply(node, P, g)
            if need_grad:
                leaves = [cart] + ([strain] if want_s else [])
                grads = torch.autograd.grad(energy.sum(), leaves)
                if want_f:
                    out["f"] = torch.split(-grads[0], g.atoms_per_graph)
                if want_s:
                    scale = (GPA_PER_EV_A3 / g.volume).view(-1, 1, 1)
                    out["s"] = list(torch.unbind(grads[-1] * scale, dim=0))
        energy = energy.detach()
        if "m" in task:
            zm = ops.linear(node_n, P.m_w0, bias=P.m_b0)
            out["m"] = list(torch.split(ops.head_dot_fwd(zm, P.m_w3, P.m_b3, take_abs=True), g.atoms_per_graph))
        apg = g.atom_ptr[1:] - g.atom_ptr[:-1]  # atoms per structure, on the device (no host copy, no synchronisation)
        out["e"] = energy / apg if self.is_intensive else energy
        out["atoms_per_graph"] = apg
        ref = 0
        if cfg["reference_energy"] is not None:
            ref = self._reference_energy(g)
        out["e"] = out["e"] + ref
        out["ref_energy"] = ref
        return out

    def _reference_energy(self, g: BatchedGraph):
        """AtomRef.forward (matris/model/reference_energy.py:34-55): composition-weighted table sum, float32."""
        # evaluated on the device from the batch's own index tensors: a host round trip here would synchronise the
        # stream at the end of every evaluation
        table = getattr(self, "_ref_table", None)
        if table is None or table.device != g.numbers.device:
            table = self._ref_table = (self.state_dict()["reference_energy.fc.weight"].detach().reshape(-1)
                                       .to(device=g.numbers.device, dtype=torch.float32))
        comp = torch.zeros(g.n_struct, table.numel(), dtype=torch.float32, device=table.device)
        comp.index_put_((g.atom_struct.long(), (g.numbers - 1).long()),
                        torch.ones(g.n_atoms, dtype=torch.float32, device=table.device), accumulate=True)
        if self.is_intensive:
            comp = comp / (g.atom_ptr[1:] - g.atom_ptr[:-1]).to(torch.float32)[:, None]
        return comp @ table

    # -- convenience ------------------------------------------------------------------------
    def plan_batches(self, structures) -> list[BatchedGraph]:
        """The device-resident graphs ``predict`` evaluates for a list of structures: one batch when the internals of
        every layer fit in memory beside it, otherwise the contiguous sub-batches of ``split_for_memory``."""
        structures = list(structures)
        g = self.graph_converter.batch(structures)
        ranges = self.split_for_memory(g)
        if len(ranges) == 1:
            return [g]
        del g
        return [self.graph_converter.batch(structures[a:b]) for a, b in ranges]

    def forward_batches(self, graphs: Sequence[BatchedGraph], task: str = "efsm") -> dict:
        """Evaluate sub-batches one after another and join the results in order: the dictionary ``forward`` returns
        for the concatenated list of structures."""
        outs = [self.forward(g, task=task) for g in graphs]
        if len(outs) == 1:
            return outs[0]
        res = {"e": torch.cat([o["e"] for o in outs]), "atoms_per_graph": torch.cat([o["atoms_per_graph"] for o in outs])}
        ref = [o["ref_energy"] for o in outs]
        res["ref_energy"] = torch.cat(ref) if torch.is_tensor(ref[0]) else ref[0]
        if "f" in outs[0]:
            res["f"] = tuple(t for o in outs for t in o["f"])
        for k in ("s", "m"):
            if k in outs[0]:
                res[k] = [t for o in outs for t in o[k]]
        return res

    def predict(self, structures, task: str = "efsm"):
        """Evaluate a list of structures (any accepted structure type): as one batch, or, when the backward pass of
        that batch would have to recompute layers for lack of memory, as the sub-batches of ``plan_batches``."""
        return self.forward_batches(self.plan_batches(structures), task=task)

    def predict_sharded(self, structures, task: str = "efsm", group=None, dst: int = 0):
        """``predict`` over all ranks of a ``torch.distributed`` group (one process per GPU, every rank passes the
        same list): structures are assigned to ranks by predicted cost, evaluated locally, and E / F / S / M are
        gathered to rank ``dst`` (see matris_b200.parallel.evaluate).  Returns the full result there, None elsewhere."""
        from .parallel import evaluate
        return evaluate(self, structures, task, group=group, dst=dst)
