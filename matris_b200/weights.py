"""Parameter schema of a MatRIS checkpoint and a reproducible random initialiser.

The checkpoint format is the reference's: ``{"config": <constructor kwargs>,
"state_dict": {...}}`` (matris/model/model.py:256-260).  ``schema(config)`` lists
every ``state_dict`` key with its shape in the reference's registration order;
``random_state_dict`` fills them from a counter-based generator keyed on the
parameter NAME, so the values do not depend on module construction order and
any implementation that knows the key names reproduces them exactly.
"""
from __future__ import annotations

import json
import math
import os
import zlib
from collections import OrderedDict

import numpy as np
import torch

DEFAULT_CONFIG = OrderedDict(
    num_layers=6, node_feat_dim=128, edge_feat_dim=128, three_body_feat_dim=128,
    mlp_hidden_dims=(128, 128), dropout=0.0, use_bias=False, distance_expansion="Bessel",
    three_body_expansion="SH", num_radial=7, num_angular=7, max_l=4, max_n=4,
    envelope_exponent=8, graph_conv_mlp="GateMLP", activation_type="silu", norm_type="rms",
    pairwise_cutoff=6, three_body_cutoff=4, use_smoothed_for_delta_edge=False,
    learnable_basis=True, is_intensive=True, is_conservation=True, reference_energy=None,
)  # matris/model/model.py:33-59

MAX_ELEMENTS = 94


def full_config(config: dict | None = None, **overrides) -> OrderedDict:
    cfg = OrderedDict(DEFAULT_CONFIG)
    cfg.update(config or {})
    cfg.update(overrides)
    unknown = set(cfg) - set(DEFAULT_CONFIG)
    if unknown:
        raise TypeError(f"unexpected MatRIS config keys: {sorted(unknown)}")
    return cfg


def check_supported(cfg: dict) -> None:
    """The CUDA path implements the default architecture family only; anything
    else is rejected here rather than silently evaluated differently."""
    want = dict(activation_type="silu", norm_type="rms")
    for k, v in want.items():
        if str(cfg[k]).lower() != v:
            raise NotImplementedError(f"matris_b200 implements {k}={v!r} only (got {cfg[k]!r})")
    if str(cfg["graph_conv_mlp"]).lower() not in ("gatemlp", "mlp"):
        raise NotImplementedError(f"graph_conv_mlp={cfg['graph_conv_mlp']!r}: 'GateMLP' or 'MLP'")
    if str(cfg["distance_expansion"]).lower() not in ("bessel", "gaussian"):
        raise NotImplementedError(f"distance_expansion={cfg['distance_expansion']!r}: 'Bessel' or 'Gaussian'")
    if str(cfg["three_body_expansion"]).lower() not in ("sh", "fourier"):
        raise NotImplementedError(f"three_body_expansion={cfg['three_body_expansion']!r}: 'SH' or 'fourier'")
    if str(cfg["three_body_expansion"]).lower() == "fourier" and int(cfg["num_angular"]) != 7:
        raise NotImplementedError("matris_b200 implements num_angular=7 only")
    for k in ("node_feat_dim", "edge_feat_dim", "three_body_feat_dim"):
        if int(cfg[k]) != 128:
            raise NotImplementedError(f"matris_b200 kernels are specialised for {k}=128 (got {cfg[k]})")
    hd = cfg["mlp_hidden_dims"]
    if list(hd if not isinstance(hd, int) else [hd]) != [128, 128]:
        raise NotImplementedError("matris_b200 implements mlp_hidden_dims=(128, 128) only")
    if int(cfg["num_radial"]) != 7 or int(cfg["max_l"]) != 4 or int(cfg["max_n"]) != 4:
        raise NotImplementedError("matris_b200 implements num_radial=7, max_l=max_n=4 only")
    if not cfg["is_conservation"]:
        raise NotImplementedError("matris_b200 implements the conservative force/stress head only")
    if float(cfg["dropout"]) != 0.0:
        raise NotImplementedError("dropout is a training-only option")


def schema(config: dict | None = None) -> "OrderedDict[str, tuple]":
    """key -> shape, in the reference's state_dict order."""
    cfg = full_config(config)
    D, R = int(cfg["node_feat_dim"]), int(cfg["num_radial"])
    A = int(cfg["max_n"]) * int(cfg["max_l"])
    s: "OrderedDict[str, tuple]" = OrderedDict()
    if cfg["reference_energy"] is not None:
        s["reference_energy.fc.weight"] = (1, MAX_ELEMENTS)
    s["atom_embedding.embedding.weight"] = (MAX_ELEMENTS, D)
    s["atom_embedding.atom_swish_layer.linear.weight"] = (D, D)
    # BesselExpansion holds `frequencies`, GaussianExpansion an `offset` buffer (basis_function.py:116-216)
    rbf_key = "frequencies" if str(cfg["distance_expansion"]).lower() == "bessel" else "offset"
    s["edge_embedding.pairwise_rbf_expansion." + rbf_key] = (R,)
    s["edge_embedding.threebody_rbf_expansion." + rbf_key] = (R,)
    s["edge_embedding.edge_linear1.weight"] = (D, R)
    s["edge_embedding.edge_linear2.weight"] = (D, D)
    s["edge_embedding.swish_layer.linear.weight"] = (D, D)
    s["edge_embedding.edge_init_norm.weight"] = (D,)
    s["edge_embedding.edge_init_norm.bias"] = (D,)
    if str(cfg["three_body_expansion"]).lower() == "fourier":  # FourierExpansion(max_f = (num_angular - 1) // 2)
        F_ = int(cfg["num_angular"])
        s["three_body_embedding.expansion.frequencies"] = ((F_ - 1) // 2,)
        s["three_body_embedding.angle_embedding.weight"] = (D, F_)
    else:
        s["three_body_embedding.expansion.factor"] = ()
        s["three_body_embedding.angle_embedding.weight"] = (D, A)
    s["three_body_embedding.swish_layer.linear.weight"] = (D, D)

    plain_mlp = str(cfg["graph_conv_mlp"]).lower() == "mlp"

    def gated(prefix, k_in):
        if plain_mlp:  # nn.Sequential(MLP(in, D, D, bias=use_bias), RMSNorm) (interaction_block.py:39-62, 172-184)
            for j, k in ((0, k_in), (3, D)):
                s[f"{prefix}0.layers.{j}.weight"] = (D, k)
                if cfg["use_bias"]:
                    s[f"{prefix}0.layers.{j}.bias"] = (D,)
            s[prefix + "1.weight"] = (D,)
            return
        s[prefix + "gate_norm.weight"] = (D,)
        s[prefix + "core_norm.weight"] = (D,)
        for branch in ("mlp_core", "mlp_gate"):
            s[f"{prefix}{branch}.layers.0.weight"] = (D, k_in)
            s[f"{prefix}{branch}.layers.0.bias"] = (D,)
            s[f"{prefix}{branch}.layers.3.weight"] = (D, D)
            s[f"{prefix}{branch}.layers.3.bias"] = (D,)

    for i in range(int(cfg["num_layers"])):
        for g in ("atom", "line"):
            p = f"interaction_block.{i}.attn_block_{g}_graph."
            s[p + "node_res_weight"] = (1, D)
            s[p + "edge_res_weight"] = (1, D)
            s[p + "source_weight_linear.weight"] = (D, D)
            s[p + "target_weight_linear.weight"] = (D, D)
            gated(p + "node_nonlinear_update.", 3 * D)
            gated(p + "edge_nonlinear_update.", 3 * D)
        for g in ("atom", "line"):
            p = f"interaction_block.{i}.refine_block_{g}_graph."
            s[p + "node_res_weight"] = (1, D)
            s[p + "edge_res_weight"] = (1, D)
            gated(p + "edge_nonlinear_update.", 3 * D if g == "atom" else 4 * D)
            for ffn in ("node_FFN", "edge_FFN"):  # biases only with use_bias (interaction_block.py:197-210)
                for j in (0, 3):
                    s[f"{p}{ffn}.layers.{j}.weight"] = (D, D)
                    if cfg["use_bias"]:
                        s[f"{p}{ffn}.layers.{j}.bias"] = (D,)
            s[p + "learnable_envelope.weight"] = (D, R)
    s["readout_norm.weight"] = (D,)
    for j, (o, k) in zip((0, 3, 6), ((D, D), (D, D), (1, D))):
        s[f"energy_head.energy_head.layers.{j}.weight"] = (o, k)
        s[f"energy_head.energy_head.layers.{j}.bias"] = (o,)
    s["magmom_head.magmom_head.layers.0.weight"] = (2 * D, D)
    s["magmom_head.magmom_head.layers.0.bias"] = (2 * D,)
    s["magmom_head.magmom_head.layers.3.weight"] = (1, 2 * D)
    s["magmom_head.magmom_head.layers.3.bias"] = (1,)
    return s


BUFFER_KEYS = ("three_body_embedding.expansion.factor", "edge_embedding.pairwise_rbf_expansion.offset",
               "edge_embedding.threebody_rbf_expansion.offset")


def atomref_table(name: str) -> torch.Tensor:
    """Per-element reference energies (eV/atom), float32 [1, 94]; the same three
    tables the reference hard-codes (matris/model/reference_energy.py:116-207)."""
    key = {"mptrj": "mptrj", "demo": "mptrj", "omat": "omat", "mpa": "mpa"}.get(str(name).lower())
    if key is None:
        raise NotImplementedError(f"dataset={name!r} not supported yet")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "atomref.json")
    with open(path) as f:
        table = json.load(f)[key]
    return torch.tensor([float.fromhex(v) for v in table], dtype=torch.float32).view(1, MAX_ELEMENTS)


def _rng(seed: int, key: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFF, zlib.crc32(key.encode())]))


def random_state_dict(config: dict | None = None, seed: int = 0, jitter: float = 0.0) -> "OrderedDict[str, torch.Tensor]":
    """Seeded random-init weights with PyTorch's default scales: linear weights and
    biases U(+-1/sqrt(fan_in)), embedding N(0,1), norm / residual weights 1,
    Bessel frequencies k*pi.  ``jitter`` > 0 perturbs the parameters that default
    to constants (norm and residual weights, LayerNorm bias, frequencies) so tests
    can see whether they are honoured."""
    cfg = full_config(config)
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    for key, shape in schema(cfg).items():
        g = _rng(seed, key)
        if key == "reference_energy.fc.weight":
            v = atomref_table(cfg["reference_energy"]).numpy()
        elif key.endswith("expansion.factor"):
            v = np.sqrt(np.float32(2.0 / float(cfg["pairwise_cutoff"]) ** 3), dtype=np.float32)
        elif key.endswith("expansion.offset"):  # torch.linspace(0, cutoff, num_gaussians) (basis_function.py:203)
            stop = cfg["pairwise_cutoff"] if "pairwise" in key else cfg["three_body_cutoff"]
            v = torch.linspace(0.0, float(stop), shape[0]).numpy()
        elif key == "three_body_embedding.expansion.frequencies":  # arange(1, max_f + 1) (basis_function.py:97-103)
            v = np.arange(1, shape[0] + 1, dtype=np.float64) * (1 + 0.2 * jitter * g.uniform(-1, 1, shape))
        elif key.endswith("frequencies"):
            v = np.pi * np.arange(1, shape[0] + 1, dtype=np.float64) * (1 + 0.2 * jitter * g.uniform(-1, 1, shape))
        elif key.endswith("embedding.weight") and key.startswith("atom_embedding"):
            v = g.standard_normal(shape)
        elif key.endswith("_norm.weight") or key.endswith("res_weight") or key.endswith("_update.1.weight"):
            v = 1.0 + jitter * g.uniform(-1, 1, shape)
        elif key.endswith("edge_init_norm.bias"):
            v = jitter * g.uniform(-1, 1, shape)
        elif key.endswith(".weight"):
            v = g.uniform(-1, 1, shape) / math.sqrt(shape[-1])
        elif key.endswith(".bias"):
            fan_in = schema(cfg)[key[:-4] + "weight"][-1]
            v = g.uniform(-1, 1, shape) / math.sqrt(fan_in)
        else:
            raise KeyError(key)
        out[key] = torch.tensor(np.asarray(v, dtype=np.float32))
    return out


def random_checkpoint(config: dict | None = None, seed: int = 0, jitter: float = 0.0) -> dict:
    cfg = full_config(config)
    return {"config": dict(cfg), "state_dict": random_state_dict(cfg, seed, jitter)}
