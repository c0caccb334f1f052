"""GPU (needs two devices; skipped otherwise): the sharded evaluation over two NCCL ranks equals single-GPU predict."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    import torch.distributed as dist

    from matris_b200 import MatRIS, workloads
    from matris_b200.weights import random_checkpoint
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    crystals = workloads.random_crystals(9, seed=17)
    ck = random_checkpoint(dict(num_layers=2, reference_energy="mpa"), seed=3)
    model = MatRIS.from_dict(ck).to(f"cuda:{rank}")
    res = model.predict_sharded(crystals, "efsm")
    if rank == 0:
        one = model.predict(crystals, "efsm")
        err = dict(
            e=float((res["e"] - one["e"]).abs().max()), ref=float((res["ref_energy"] - one["ref_energy"]).abs().max()),
            f=max(float((a - b).abs().max()) for a, b in zip(res["f"], one["f"])),
            s=max(float((a - b).abs().max()) for a, b in zip(res["s"], one["s"])),
            m=max(float((a - b).abs().max()) for a, b in zip(res["m"], one["m"])))
        torch.save({"err": err, "shards": res["shards"], "apg": res["atoms_per_graph"].cpu()}, out_path)
    else:
        assert res is None
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_predict_sharded_two_gpus_equals_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    # a structure's result does not depend on which other structures share its batch (up to the summation order of
    # the atomics in the backward GEMM epilogues)
    assert got["err"]["e"] <= 2e-6 and got["err"]["ref"] == 0.0, got
    assert got["err"]["f"] <= 5e-6 and got["err"]["s"] <= 2e-4 and got["err"]["m"] <= 2e-6, got
    assert all(len(s) > 0 for s in got["shards"]) and sorted(i for s in got["shards"] for i in s) == list(range(9))
