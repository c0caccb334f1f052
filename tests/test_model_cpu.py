"""CPU: the model-loading interface (matris/model/model.py:256-317) and host-side checks of MatRIS."""
import os

import pytest
import torch

from matris_b200 import MatRIS
from matris_b200.graph import BatchedGraph
from matris_b200.weights import random_checkpoint


def _same_state(model, ck):
    sd = model.state_dict()
    assert list(sd.keys()) == list(ck["state_dict"].keys())
    return all(torch.equal(sd[k].cpu(), v) for k, v in ck["state_dict"].items())


def test_load_from_explicit_path(tmp_path, capsys):
    ck = random_checkpoint(dict(num_layers=1, reference_energy="mpa"), seed=7, jitter=0.1)
    path = str(tmp_path / "ckpt.pth.tar")
    torch.save(ck, path)
    model = MatRIS.load(path=path, device="cpu")
    assert _same_state(model, ck) and model.config["num_layers"] == 1 and model.config["reference_energy"] == "mpa"
    assert "successfully" in capsys.readouterr().out
    # a file name given as model_name is taken as a path too
    assert _same_state(MatRIS.load(path, device="cpu"), ck)


@pytest.mark.parametrize("name,fname", [("matris_10m_oam", "MatRIS_10M_OAM.pth.tar"),
                                        ("MatRIS_10M_MP", "MatRIS_10M_MP.pth.tar")])
def test_load_by_name_reads_the_cache_directory(tmp_path, monkeypatch, name, fname):
    """The reference resolves a model name to ~/.cache/matris/<file> and downloads only when the file is missing
    (model.py:278-296); with the file in place no network is touched."""
    ck = random_checkpoint(dict(num_layers=1, reference_energy="mpa"), seed=8)
    cache = tmp_path / ".cache" / "matris"
    cache.mkdir(parents=True)
    torch.save(ck, str(cache / fname))
    monkeypatch.setenv("HOME", str(tmp_path))

    def no_download(*a, **k):
        raise AssertionError("download attempted although the checkpoint is cached")

    monkeypatch.setattr(torch.hub, "download_url_to_file", no_download)
    model = MatRIS.load(name, device="cpu")
    assert _same_state(model, ck)
    assert os.path.isfile(str(cache / fname))


def test_load_rejects_unknown_names():
    with pytest.raises(ValueError, match="Unsupported model_name"):
        MatRIS.load("matris_10m_omat", device="cpu")


def test_batch_on_another_device_is_rejected():
    model = MatRIS(num_layers=1)
    g = BatchedGraph()
    g.cart32 = torch.zeros(2, 3, device="meta")
    with pytest.raises(ValueError, match="the batch lives on"):
        model._as_batch(g)


def test_graph_converter_follows_the_model():
    model = MatRIS(num_layers=1)
    assert model.graph_converter.device is None
    model.to("meta")  # any non-CUDA device: the converter keeps its default
    assert model.graph_converter.device is None


def test_memory_policy_bounds_and_sub_batch_ranges():
    """kept_layers_for: everything is kept while it fits, fewer layers as memory shrinks, never more than the bounds
    allow; split_ranges: contiguous, complete, every range fits, balanced, single structures that do not fit alone
    stay alone."""
    import numpy as np

    from matris_b200.model import kept_layers_for, split_ranges

    T, E = 6_600_000, 1_410_000   # the 512-perovskite batch
    assert kept_layers_for(10, T, E, 190e9) == 1
    assert kept_layers_for(10, T // 8, E // 8, 190e9) == 10
    assert kept_layers_for(10, T, E, 2000e9) == 10
    assert kept_layers_for(10, T, E, 50e9) == 0
    kept = [kept_layers_for(10, T, E, a * 1e9) for a in (100, 190, 300, 500, 900, 1300)]
    assert kept == sorted(kept) and kept[-1] == 10
    for a, k in zip((100, 190, 300, 500, 900), kept):
        if 0 < k < 10:  # the bounds on the backward-pass peak and on the end of the forward pass hold
            assert (18.0e3 + 2.6e3 * k) * T + (14.2e3 + 4.4e3 * k) * E <= 0.92 * a * 1e9
            assert (17.0e3 + 6.7e3 * k) * T + (2.0e3 + 6.2e3 * k) * E <= 0.92 * a * 1e9

    rng = np.random.default_rng(0)
    trip = rng.integers(5_000, 20_000, 512)
    edge = rng.integers(1_000, 4_000, 512)
    fits = lambda t, e: kept_layers_for(10, t, e, 0.93 * 190e9) == 10
    ranges = split_ranges(trip, edge, fits)
    assert ranges[0][0] == 0 and ranges[-1][1] == 512
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    assert all(fits(int(trip[a:b].sum()), int(edge[a:b].sum())) for a, b in ranges)
    rows = [int((trip[a:b] + edge[a:b]).sum()) for a, b in ranges]
    assert max(rows) < 1.15 * min(rows)                       # balanced
    need = (6.7e3 * trip.sum() + 6.2e3 * edge.sum()) * 10 / (0.45 * 0.93 * 190e9)
    assert need <= len(ranges) <= need + 3                    # about as few ranges as the memory allows
    assert split_ranges(trip[:20], edge[:20], fits) == [(0, 20)]
    # one structure too large to keep everything: a range of its own, its neighbours unaffected
    trip2 = trip.copy()
    trip2[100] = 40_000_000
    ranges2 = split_ranges(trip2, edge, fits)
    assert (100, 101) in ranges2 and ranges2[0][0] == 0 and ranges2[-1][1] == 512
    assert all(fits(int(trip2[a:b].sum()), int(edge[a:b].sum())) or (a, b) == (100, 101) for a, b in ranges2)


def test_forward_batches_joins_results_in_order(monkeypatch):
    """forward_batches concatenates the per-sub-batch dictionaries in order (host logic, no device needed)."""
    ck = random_checkpoint(dict(num_layers=1, reference_energy="mpa"), seed=3)
    model = MatRIS.from_dict(ck)
    sizes = {"a": [2, 3], "b": [4], "c": [1, 1, 5]}

    def fake_forward(g, task="efsm", is_training=False):
        n = sizes[g]
        base = float(ord(g))
        return {"e": torch.full((len(n),), base), "ref_energy": torch.full((len(n),), -base),
                "atoms_per_graph": torch.tensor(n, dtype=torch.int32),
                "f": tuple(torch.full((k, 3), base) for k in n), "s": [torch.full((3, 3), base) for _ in n],
                "m": [torch.full((k,), base) for k in n]}

    monkeypatch.setattr(model, "forward", fake_forward)
    out = model.forward_batches(["a", "b", "c"], task="efsm")
    assert out["atoms_per_graph"].tolist() == [2, 3, 4, 1, 1, 5]
    assert out["e"].tolist() == [97.0, 97.0, 98.0, 99.0, 99.0, 99.0] and out["ref_energy"].tolist()[2] == -98.0
    assert isinstance(out["f"], tuple) and [t.shape[0] for t in out["f"]] == [2, 3, 4, 1, 1, 5]
    assert len(out["s"]) == 6 and [t.numel() for t in out["m"]] == [2, 3, 4, 1, 1, 5]
    assert float(out["f"][2][0, 0]) == 98.0 and float(out["m"][5][0]) == 99.0
    # a single sub-batch is returned as it is; a model without reference energies keeps its scalar 0
    one = model.forward_batches(["b"], task="efsm")
    assert one["e"].tolist() == [98.0]

    def fake_no_ref(g, task="e", is_training=False):
        return {"e": torch.zeros(len(sizes[g])), "ref_energy": 0, "atoms_per_graph": torch.tensor(sizes[g])}

    monkeypatch.setattr(model, "forward", fake_no_ref)
    out = model.forward_batches(["a", "c"], task="e")
    assert out["ref_energy"] == 0 and out["e"].numel() == 5 and "f" not in out
