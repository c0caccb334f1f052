"""Functional PyTorch restatement of the reference's E/F/S/M evaluation
(test infrastructure only).

Everything is a plain function of ``(state_dict, config, graphs)``; forces and
stress come from ``torch.autograd.grad`` exactly as in the reference's
conservative head.  Follows, by reference file:line,

  process_graphs          matris/model/processgraph.py:6-245
  atom / edge / angle embeddings   matris/model/feature_embed.py:16-203
  Bessel, envelope, spherical basis matris/model/basis_function.py:8-50, 116-186, 222-338
  GatedMLP / MLP / softmax / aggregate   matris/model/functions.py:97-311
  attention + refinement + block   matris/model/interaction_block.py:87-143, 218-278, 372-446
  heads                    matris/model/readout.py:66-75, 123-133, 202-224
  reference energy         matris/model/reference_energy.py:34-55
  MatRIS.forward           matris/model/model.py:183-250

Only the default architecture family is covered (Bessel + SH bases, GateMLP,
SiLU, RMSNorm, conservative forces); other values raise.  Pinned against the
reference's own ``MatRIS`` in tests/golden.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

GPA_PER_EV_A3 = 160.21766208  # readout.py:215


# ------------------------------------------------------------------ basis functions
_SPH_COEF = None


def _sph_coef():
    """Coefficient table of the spherical-Bessel radial formulas
    (basis_function.py:241-279), rounded to float32 as the reference stores it."""
    global _SPH_COEF
    if _SPH_COEF is None:
        c = torch.zeros(4, 9, 4)
        c[0, 0] = torch.tensor([3.14159274101257, 6.28318548202515, 9.42477798461914, 12.5663709640503])
        z1 = [4.49340963363647, 7.7252516746521, 10.9041213989258, 14.0661935806274]
        c[1, :4] = torch.tensor([
            [-1.02446483277785, -1.00834335996107, -1.00419641763893, -1.00252381898662], z1,
            [0.22799275301076, 0.130525632358311, 0.092093290316619, 0.0712718627992818], z1])
        z2 = [5.76345920562744, 9.09501171112061, 12.322940826416, 15.5146026611328]
        c[2, :6] = torch.tensor([
            [-1.04807944170731, -1.01861796359391, -1.01002272174988, -1.00628955560036], z2,
            [0.545547077361439, 0.335992298618515, 0.245888396928293, 0.194582402961821], z2,
            [0.0946561878721665, 0.0369424811413594, 0.0199537107571916, 0.0125418876146463], z2])
        z3 = [6.9879322052002, 10.4171180725098, 13.6980228424072, 16.9236221313477]
        c[3, :8] = torch.tensor([
            [1.06942831392075, 1.0292173312802, 1.01650804843248, 1.01069656069999], z3,
            [0.918235852195231, 0.592803493701152, 0.445250264272671, 0.358326327374518], z3,
            [0.328507713452024, 0.142266673367543, 0.0812617757677838, 0.0529328657590962], z3,
            [0.0470107184508114, 0.0136570088173405, 0.0059323726279831, 0.00312775039221944], z3])
        _SPH_COEF = c
    return _SPH_COEF


def envelope(dist, cutoff, p):
    x = dist / cutoff
    a = -(p + 1) * (p + 2) / 2
    b = p * (p + 2)
    c = -p * (p + 1) / 2
    val = 1 + a * x ** p + b * x ** (p + 1) + c * x ** (p + 2)
    return torch.where(x < 1, val, torch.zeros_like(x))


def bessel(dist, freqs, cutoff, p):
    d = dist[:, None]
    out = (2.0 / cutoff) ** 0.5 * torch.sin(freqs * (d * (1.0 / cutoff))) / d
    return envelope(d, cutoff, float(p)) * out


def gaussian(dist, offset):
    """GaussianExpansion.forward (matris/model/basis_function.py:189-216)."""
    coeff = -0.5 / (2.0 * (offset[1] - offset[0])).item() ** 2
    return torch.exp(coeff * (dist[:, None] - offset[None, :]) ** 2)


def fourier_basis(theta, freqs):
    """FourierExpansion.forward (matris/model/basis_function.py:106-113): [1/sqrt 2, sin, cos] / sqrt(pi)."""
    ang = torch.outer(theta, freqs)
    first = torch.full_like(theta, float(1 / torch.sqrt(torch.tensor([2.0]))))[:, None]
    return torch.cat([first, torch.sin(ang), torch.cos(ang)], dim=1) / math.sqrt(math.pi)


def spherical_basis(dist, theta, factor, cutoff, max_n=4, max_l=4):
    c = _sph_coef().to(dist.dtype)
    x = dist / cutoff
    r = []
    for j in range(max_l):
        r.append(torch.sin(c[0, 0, j] * x) / x)
    for j in range(max_l):
        r.append((c[1, 0, j] * x * torch.cos(c[1, 1, j] * x) + c[1, 2, j] * torch.sin(c[1, 3, j] * x)) / x ** 2)
    for j in range(max_l):
        r.append((c[2, 0, j] * x ** 2 * torch.sin(c[2, 1, j] * x) - c[2, 2, j] * x * torch.cos(c[2, 3, j] * x)
                  + c[2, 4, j] * torch.sin(c[2, 5, j] * x)) / x ** 3)
    for j in range(max_l):
        r.append((c[3, 0, j] * x ** 3 * torch.cos(c[3, 1, j] * x) - c[3, 2, j] * x ** 2 * torch.sin(c[3, 3, j] * x)
                  - c[3, 4, j] * x * torch.cos(c[3, 5, j] * x) + c[3, 6, j] * torch.sin(c[3, 7, j] * x)) / x ** 4)
    rbf = torch.stack(r, dim=-1) * factor
    ct = torch.cos(theta)
    sh = torch.stack([
        torch.ones_like(ct) * 0.5 * math.sqrt(1.0 / math.pi),
        math.sqrt(3.0 / (4.0 * math.pi)) * ct,
        math.sqrt(5.0 / (16.0 * math.pi)) * (3.0 * ct ** 2 - 1.0),
        math.sqrt(7.0 / (16.0 * math.pi)) * ct * (5.0 * ct ** 2 - 3.0)], dim=-1)
    return rbf * sh.repeat_interleave(max_n, dim=1)


# ------------------------------------------------------------------ generic pieces
def segment_softmax(x, seg):
    n = int(seg.max()) + 1
    idx = seg[:, None].expand(-1, x.shape[1])
    mx = torch.full((n, x.shape[1]), float("-inf"), dtype=x.dtype).scatter_reduce(
        0, idx, x, reduce="amax", include_self=False)
    e = (x - mx[seg]).exp()
    sm = torch.zeros(n, x.shape[1], dtype=x.dtype).scatter_reduce(0, idx, e, reduce="sum", include_self=False)
    return e / sm[seg]


def segment_sum(x, seg, n):
    return x.new_zeros(n, x.shape[1]).index_add_(0, seg, x)


def pair_mean(x, d2u):
    n = int(d2u.max()) + 1
    cnt = torch.bincount(d2u, minlength=n).clamp(min=1)
    return (segment_sum(x, d2u, n).T / cnt).T


class _P:
    """state-dict view under a key prefix."""

    def __init__(self, sd, prefix=""):
        self.sd, self.prefix = sd, prefix

    def __call__(self, name):
        return self.sd[self.prefix + name]

    def sub(self, name):
        return _P(self.sd, self.prefix + name + ".")

    def has(self, name):
        return self.prefix + name in self.sd


def mlp2(p, x, bias):
    h = F.silu(F.linear(x, p("layers.0.weight"), p("layers.0.bias") if bias else None))
    return F.linear(h, p("layers.3.weight"), p("layers.3.bias") if bias else None)


def gated_mlp(p, x):
    """GatedMLP.forward (matris/model/functions.py:245-311), or - where the state dict holds the plain-MLP variant of
    the block (graph_conv_mlp = "MLP": nn.Sequential(MLP, norm), matris/model/interaction_block.py:39-62) - that."""
    if p.has("0.layers.0.weight"):
        y = mlp2(p.sub("0"), x, p.has("0.layers.0.bias"))  # biases only with use_bias
        return F.rms_norm(y, (y.shape[1],), p("1.weight"), None)
    core = F.rms_norm(mlp2(p.sub("mlp_core"), x, True), (p("core_norm.weight").shape[0],),
                      p("core_norm.weight"), None)
    gate = F.rms_norm(mlp2(p.sub("mlp_gate"), x, True), (p("gate_norm.weight").shape[0],),
                      p("gate_norm.weight"), None)
    return F.silu(core) * torch.sigmoid(gate)


# ------------------------------------------------------------------ message passing
def attention_layer(p, node, edge, g, d2u=None):
    src, tgt = g["source_index"], g["target_index"]
    e0 = edge[d2u] if d2u is not None else edge
    h = gated_mlp(p.sub("edge_nonlinear_update"), torch.cat([e0, node[tgt], node[src]], dim=1))
    a_s = segment_softmax(F.linear(e0, p("source_weight_linear.weight")), src)
    a_t = segment_softmax(F.linear(e0, p("target_weight_linear.weight")), tgt)
    agg_s = segment_sum(a_s * h, src, len(node))
    agg_t = segment_sum(a_t * h, tgt, len(node))
    edge_new = pair_mean(h, d2u) if d2u is not None else h
    node_new = gated_mlp(p.sub("node_nonlinear_update"), torch.cat([node, agg_t, agg_s], dim=1))
    return node_new + p("node_res_weight") * node, edge_new + p("edge_res_weight") * edge


def refinement_layer(p, node, edge, smooth, g, d2u=None, atom_feat=None, smoothed_delta_edge=False, ffn_bias=False):
    src, tgt = g["source_index"], g["target_index"]
    atom_graph = d2u is not None
    if atom_graph:
        e0 = edge[d2u]
        s = F.linear(smooth[d2u], p("learnable_envelope.weight"))
        x = torch.cat([e0, node[tgt], node[src]], dim=1)
    else:
        env = F.linear(smooth, p("learnable_envelope.weight"))
        s = env[src] * env[tgt]
        x = torch.cat([edge, atom_feat[g["atom_list"]], node[tgt], node[src]], dim=1)
    h = gated_mlp(p.sub("edge_nonlinear_update"), x)
    hs = h * s
    node_delta = mlp2(p.sub("node_FFN"), segment_sum(hs, tgt, len(node)), ffn_bias)
    edge_delta = mlp2(p.sub("edge_FFN"), hs if (atom_graph and smoothed_delta_edge) else h, ffn_bias)
    if atom_graph:
        edge_delta = pair_mean(edge_delta, d2u)
    return node_delta + p("node_res_weight") * node, edge_delta + p("edge_res_weight") * edge


# ------------------------------------------------------------------ batching
def process_graphs(graphs, compute_stress, dtype=torch.float32):
    """graphs: list of dicts with atomic_number, frac, lattice, image, atom_graph,
    directed2undirected, undirected2directed, line_graph (torch tensors)."""
    z, cart, lat, img, ag, d2u, u2d, lg, seg, egraph = [], [], [], [], [], [], [], [], [], []
    na = ne = nu = 0
    for b, g in enumerate(graphs):
        n = g["atomic_number"].shape[0]
        z.append(g["atomic_number"].long())
        cart.append(g["frac"].to(dtype) @ g["lattice"].to(dtype))
        lat.append(g["lattice"].to(dtype))
        img.append(g["image"].to(dtype))
        ag.append(g["atom_graph"].long() + na)
        d2u.append(g["directed2undirected"].long() + nu)
        u2d.append(g["undirected2directed"].long() + ne)
        if len(g["line_graph"]):
            l = g["line_graph"].long().clone()
            l[:, 0] += na
            l[:, 1] += nu
            l[:, 3] += nu
            l[:, 2] += ne
            l[:, 4] += ne
            lg.append(l)
        seg.append(torch.full((n,), b, dtype=torch.long))
        egraph.append(torch.full((len(g["atom_graph"]),), b, dtype=torch.long))
        na += n
        ne += len(g["atom_graph"])
        nu += len(g["undirected2directed"])
    z, cart, ag = torch.cat(z), torch.cat(cart), torch.cat(ag)
    lat = torch.stack(lat)
    img, d2u, u2d, seg, egraph = torch.cat(img), torch.cat(d2u), torch.cat(u2d), torch.cat(seg), torch.cat(egraph)
    vol = torch.einsum("ni,ni->n", lat[:, 0], torch.linalg.cross(lat[:, 1], lat[:, 2]))
    cart.requires_grad_(True)
    strain = None
    pos, latt = cart, lat
    if compute_stress:
        strain = torch.zeros(len(graphs), 3, 3, dtype=dtype, requires_grad=True)
        sym = 0.5 * (strain + strain.transpose(-1, -2))
        pos = cart + torch.einsum("be,bec->bc", cart, sym[seg])
        latt = lat + torch.matmul(lat, sym)
    tgt, src = ag[:, 0], ag[:, 1]
    shift = torch.einsum("ek,ekc->ec", img, latt[egraph])
    vec = pos[tgt] - (pos[src] + shift)
    length = torch.norm(vec, dim=1)
    batch = dict(atomic_numbers=z, atom_segment=seg, atoms_per_graph=[len(g["atomic_number"]) for g in graphs],
                 directed2undirected=d2u, undirected2directed=u2d, volumes=vol, cart=cart, strain=strain,
                 edge_lengths=length, unit_edge_vectors=vec / length[:, None],
                 atom_graph=dict(source_index=src, target_index=tgt), line_graph=None)
    if lg:
        l = torch.cat(lg)
        batch["line_graph"] = dict(atom_list=l[:, 0], target_index=l[:, 1], target_DE_index=l[:, 2],
                                   source_index=l[:, 3], source_DE_index=l[:, 4])
    return batch


# ------------------------------------------------------------------ whole model
def _check_config(cfg):
    want = dict(activation_type="silu", norm_type="rms")
    for k, v in want.items():
        if str(cfg.get(k, v)).lower() != v:
            raise NotImplementedError(f"oracle covers {k}={v!r} only, got {cfg[k]!r}")
    if str(cfg.get("graph_conv_mlp", "gatemlp")).lower() not in ("gatemlp", "mlp"):
        raise NotImplementedError(f"oracle covers graph_conv_mlp 'GateMLP' and 'MLP', got {cfg['graph_conv_mlp']!r}")
    if str(cfg.get("distance_expansion", "bessel")).lower() not in ("bessel", "gaussian"):
        raise NotImplementedError(f"oracle covers Bessel and Gaussian distance expansions, got {cfg['distance_expansion']!r}")
    if str(cfg.get("three_body_expansion", "sh")).lower() not in ("sh", "fourier"):
        raise NotImplementedError(f"oracle covers SH and Fourier angle expansions, got {cfg['three_body_expansion']!r}")
    if not cfg.get("is_conservation", True):
        raise NotImplementedError("oracle covers the conservative force/stress head only")


def forward(sd, cfg, graphs, task="ef", dtype=torch.float32):
    """Restatement of MatRIS.forward (model.py:183-250). ``sd`` is a reference
    state_dict, ``cfg`` the constructor kwargs.  Returns the same dict layout."""
    _check_config(cfg)
    sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    P = _P(sd)
    rc2, rc3 = float(cfg.get("pairwise_cutoff", 6)), float(cfg.get("three_body_cutoff", 4))
    p_env = cfg.get("envelope_exponent", 8)
    bg = process_graphs(graphs, "s" in task, dtype)
    d2u, u2d = bg["directed2undirected"], bg["undirected2directed"]
    # embeddings
    pe = P.sub("atom_embedding")
    node = F.silu(F.linear(pe("embedding.weight")[bg["atomic_numbers"] - 1], pe("atom_swish_layer.linear.weight")))
    pe = P.sub("edge_embedding")
    du = bg["edge_lengths"][u2d]
    if str(cfg.get("distance_expansion", "bessel")).lower() == "gaussian":
        rbf2 = gaussian(du, pe("pairwise_rbf_expansion.offset"))
        rbf3 = gaussian(du, pe("threebody_rbf_expansion.offset"))
    else:
        rbf2 = bessel(du, pe("pairwise_rbf_expansion.frequencies"), rc2, p_env)
        rbf3 = bessel(du, pe("threebody_rbf_expansion.frequencies"), rc3, p_env)
    e = F.linear(F.linear(rbf2, pe("edge_linear1.weight"))[d2u], pe("edge_linear2.weight"))
    e = F.layer_norm(e, (e.shape[1],), pe("edge_init_norm.weight"), pe("edge_init_norm.bias"))
    edge = F.silu(F.linear(pair_mean(e, d2u), pe("swish_layer.linear.weight")))
    lgd = bg["line_graph"]
    trip = None
    if lgd is not None:
        pe = P.sub("three_body_embedding")
        ua = bg["unit_edge_vectors"][lgd["target_DE_index"]]
        ub = bg["unit_edge_vectors"][lgd["source_DE_index"]]
        theta = torch.acos((ua * ub).sum(dim=1) * (1 - 1e-6))
        if str(cfg.get("three_body_expansion", "sh")).lower() == "fourier":
            basis = fourier_basis(theta, pe("expansion.frequencies"))
        else:
            basis = spherical_basis(torch.norm(ub, dim=1), theta, pe("expansion.factor"), rc2,
                                    cfg.get("max_n", 4), cfg.get("max_l", 4))
        trip = F.silu(F.linear(F.linear(basis, pe("angle_embedding.weight")), pe("swish_layer.linear.weight")))
    # interaction blocks (interaction_block.py:372-446)
    sde = cfg.get("use_smoothed_for_delta_edge", False)
    fb = bool(cfg.get("use_bias", False))  # biases of node_FFN / edge_FFN (interaction_block.py:197-210)
    for i in range(cfg.get("num_layers", 6)):
        pb = P.sub(f"interaction_block.{i}")
        e_att, t_att = edge, trip
        if trip is not None:
            e_att, t_att = attention_layer(pb.sub("attn_block_line_graph"), edge, trip, lgd)
        n_att, e_att = attention_layer(pb.sub("attn_block_atom_graph"), node, e_att, bg["atom_graph"], d2u)
        e_upd, t_upd = edge, trip
        if trip is not None:
            e_upd, t_upd = refinement_layer(pb.sub("refine_block_line_graph"), e_att, t_att, rbf3, lgd,
                                            atom_feat=n_att, ffn_bias=fb)
        node, edge = refinement_layer(pb.sub("refine_block_atom_graph"), n_att, e_upd, rbf2, bg["atom_graph"],
                                      d2u, smoothed_delta_edge=sde, ffn_bias=fb)
        trip = t_upd
    # readout
    node = F.rms_norm(node, (node.shape[1],), P("readout_norm.weight"), None)
    pe = P.sub("energy_head.energy_head")
    h = F.silu(F.linear(node, pe("layers.0.weight"), pe("layers.0.bias")))
    h = F.silu(F.linear(h, pe("layers.3.weight"), pe("layers.3.bias")))
    e_atom = F.linear(h, pe("layers.6.weight"), pe("layers.6.bias"))
    n_graph = len(graphs)
    total = segment_sum(e_atom, bg["atom_segment"], n_graph).view(-1)
    out = {}
    if "f" in task and "s" in task:
        g_r, g_s = torch.autograd.grad(total.sum(), [bg["cart"], bg["strain"]])
        out["f"] = torch.split(-g_r, bg["atoms_per_graph"])
        out["s"] = list(torch.unbind(g_s * (1 / bg["volumes"].view(-1, 1, 1) * GPA_PER_EV_A3), dim=0))
    elif "f" in task:
        (g_r,) = torch.autograd.grad(total.sum(), [bg["cart"]])
        out["f"] = torch.split(-g_r, bg["atoms_per_graph"])
    if "m" in task:
        pe = P.sub("magmom_head.magmom_head")
        m = F.linear(F.silu(F.linear(node, pe("layers.0.weight"), pe("layers.0.bias"))),
                     pe("layers.3.weight"), pe("layers.3.bias"))
        out["m"] = list(torch.split(m.abs().view(-1).detach(), bg["atoms_per_graph"]))
    apg = torch.tensor(bg["atoms_per_graph"], dtype=torch.int32)
    total = total.detach()
    out["e"] = total / apg if cfg.get("is_intensive", True) else total
    out["atoms_per_graph"] = apg
    ref = 0
    if cfg.get("reference_energy") is not None:
        comp = []
        for g in graphs:
            c = torch.bincount(g["atomic_number"].long() - 1, minlength=94)
            comp.append(c / len(g["atomic_number"]) if cfg.get("is_intensive", True) else c)
        ref = F.linear(torch.stack(comp).float(), sd["reference_energy.fc.weight"].float()).view(-1)
    out["e"] = out["e"] + ref
    out["ref_energy"] = ref
    return out
