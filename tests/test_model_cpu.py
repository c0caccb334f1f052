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
