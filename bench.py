#!/usr/bin/env python
"""Throughput of the E/F/S/M evaluation path: atoms*evals/s.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
                    [--workload perov512|random256|random64|cu32|fe16k|lipscl] [--scaling weak|strong]
                    [--md-steps N] [--no-cpu-baseline] [--keep auto|on|off]

Default workload: the high-throughput screen of random ABX3 perovskite cells (2x2x2 supercells, 40 atoms, seed 4),
task "efsm", 512 cells per GPU, MatRIS with 10 interaction blocks and seeded random-init weights.  One step = graph
build + forward + backward for the whole batch + the gather of energies, forces, stresses and magnetic moments.
A rank evaluates its structures the way `MatRIS.predict` does: as one batch when the internals of every layer fit in
memory beside it, otherwise as contiguous sub-batches that do, one after another (the structures are independent;
the backward pass then recomputes nothing).
N > 1 (one process per GPU under torchrun): the list of 512 N cells is sharded over the ranks by predicted cost
(matris_b200.parallel), every rank evaluates its share, and the results are gathered to rank 0 with one NCCL gather
per step; no other collective is on the path.  `--scaling strong` keeps the total fixed (256 random crystals by
default there) and splits it over the ranks instead.  Single large structures (cu32, fe16k, lipscl) run on one GPU.

`value` is timed with the inputs resident in HBM (positions, lattices); `e2e` goes through the public API
(`MatRIS.predict_sharded` on host structures) with the host->device copies of the inputs and the device->host read
of E / F / S / M inside the timed region.  `--impl reference` times the CPU oracle (the restatement of the
reference's PyTorch path, pinned to it by golden vectors) on a bounded sample of the same workload instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NUM_LAYERS = 10
GEMM_CALLS = ("mb_gemm", "mb_gated_mlp_fwd")  # the tensor-core entry points
PER_GPU = {"perov512": 512, "random256": 256, "random64": 64}


def metric_name(task: str) -> str:
    return f"atoms*evals/s ({task}, fp32-tol)"


def make_workload(name: str, world: int, scaling: str):
    """(structures of the whole job, task, description).  Batched workloads grow with the number of ranks under weak
    scaling (the generators are sequential in their seed, so N ranks evaluate the first N x per-GPU structures)."""
    from matris_b200 import workloads as w
    n = PER_GPU.get(name, 1) * (world if scaling == "weak" else 1)
    if name == "perov512":
        return w.perovskites(n, seed=4), "efsm", f"{n} ABX3 2x2x2 perovskite cells (40 atoms), seed 4"
    if name in ("random256", "random64"):
        return w.random_crystals(n, seed=1), "efs", f"{n} random crystals (8-64 atoms), seed 1"
    if name == "cu32":
        return [w.cu_fcc()], "efsm", "Cu FCC 2x2x2, 32 atoms"
    if name == "fe16k":
        return [w.fe_bcc()], "efsm", "BCC Fe 20x20x20, 16000 atoms"
    if name == "lipscl":
        return [w.lipscl()], "efsm", "amorphous Li6PS5Cl, 4096 atoms"
    raise SystemExit(f"unknown workload {name}")


def cpu_workload(name: str, crystals):
    """What the CPU arm evaluates.  The two single large structures would cost the host cores tens of minutes per
    evaluation, so a down-sized replica from the same generator stands in for them (the rate is per atom, and the
    cost per atom is set by the local density, which the replica keeps)."""
    from matris_b200 import workloads as w
    if name == "lipscl":
        return [w.lipscl(n_atoms=256)], "256-atom replica of the Li6PS5Cl cell (same density and generator)"
    if name == "fe16k":
        return [w.fe_bcc(reps=(4, 4, 4))], "4x4x4 (128-atom) replica of the BCC Fe supercell"
    return crystals, None


def flops_per_eval(atoms, edges, triplets, layers):
    """Algorithmic GEMM FLOPs of one forward + backward evaluation (no recompute counted):
    2 (fwd+bwd) * 2 (MAC) * L * (360448 T + 327680 Ed + 163840 Eu + 163840 N), Eu = Ed / 2."""
    return 4.0 * layers * (360448.0 * triplets + 327680.0 * edges + 163840.0 * edges / 2 + 163840.0 * atoms)


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read-only queries from a thread of
    this process (no child process competing for the driver), every 100 ms; nvidia-smi as a fallback."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.index, self.proc, self.thread, self.stop = index, None, None, threading.Event()
        self.sm, self.mx, self.reasons, self.source = [], [], set(), None

    def _nvml_handle(self):
        import pynvml
        import torch

        pynvml.nvmlInit()
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll_nvml(self, pynvml, handle):
        while not self.stop.is_set():
            try:
                self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                self.mx.append(float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                bits = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                for name, bit in self.REASON_BITS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self.stop.wait(0.1)

    def _poll_smi(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            p = [x.strip() for x in line.split(",")]
            if len(p) < 7:
                continue
            try:
                self.sm.append(float(p[0]))
                self.mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    self.reasons.add(name)

    def __enter__(self):
        try:
            pynvml, handle = self._nvml_handle()
            self.source = "nvml"
            self.thread = threading.Thread(target=self._poll_nvml, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "500"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._poll_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.stop.set()
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": self.source}
        return {"sm_mhz": float(np.median(self.sm)), "sm_max_mhz": float(max(self.mx)), "reasons": sorted(self.reasons),
                "samples": len(self.sm), "source": self.source}


def cpu_oracle_eval(ck, sample, task):
    """One evaluation of the CPU oracle on ``sample`` as one batch, graph construction included: (seconds, graph s)."""
    from oracle import pipeline
    cfg = ck["config"]
    t0 = time.perf_counter()
    graphs = [pipeline.graph_from_arrays(c.numbers, c.cart, c.lattice, float(cfg["pairwise_cutoff"]),
                                         float(cfg["three_body_cutoff"])) for c in sample]
    t1 = time.perf_counter()
    pipeline.evaluate(ck, sample, task, graphs=graphs)
    return time.perf_counter() - t0, t1 - t0


def cpu_sample(crystals, max_structs=32, max_cost=1.8e5):
    """The bounded sample the CPU arm evaluates: the first structures of the workload, up to ``max_structs`` of them
    and up to ``max_cost`` of predicted work (about the number of triplet plus edge rows: 32 random crystals, 8 of
    the much denser perovskite cells), so that one evaluation takes the host cores some ten seconds.  The rate is
    per atom, and the cost per atom of a structure does not depend on the size of the batch it is evaluated in."""
    from matris_b200.parallel import predicted_cost
    sample, atoms, cost = [], 0, 0.0
    for c in crystals[:max_structs]:
        w = predicted_cost(c.numbers, c.lattice)
        if sample and cost + w > max_cost:
            break
        sample.append(c)
        atoms += len(c.numbers)
        cost += w
    return sample, atoms


def cpu_oracle_rate(crystals, task, budget_s=20.0, threads=None, max_structs=32, max_cost=1.8e5, max_reps=8):
    """atoms*evals/s of the CPU oracle on a bounded sample; repeated until about ``budget_s`` seconds are spent."""
    import torch

    from matris_b200.weights import random_checkpoint
    from oracle import pipeline
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    ck = random_checkpoint(dict(num_layers=NUM_LAYERS, reference_energy="mpa"), seed=0)
    sample, atoms = cpu_sample(crystals, max_structs, max_cost)
    pipeline.evaluate(ck, sample[:1], task)  # warm-up
    times, t_graph = [], 0.0
    while sum(times) < budget_s and len(times) < max_reps:
        t, tg = cpu_oracle_eval(ck, sample, task)
        times.append(t)
        t_graph += tg
    return atoms * len(times) / sum(times), dict(structures=len(sample), atoms=atoms, reps=len(times),
                                                 seconds=sum(times), graph_seconds=t_graph, threads=threads,
                                                 rate_min=atoms / max(times), rate_median=atoms / float(np.median(times)),
                                                 rate_max=atoms / min(times))


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the reference's PyTorch path on all host cores; every step
    evaluates the same bounded sample of the workload (one batch, graph construction included)."""
    if rank != 0:
        return
    import torch

    from matris_b200.weights import random_checkpoint
    from oracle import pipeline
    crystals, task, desc = make_workload(args.workload, world, args.scaling)
    crystals, replica = cpu_workload(args.workload, crystals)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    ck = random_checkpoint(dict(num_layers=NUM_LAYERS, reference_energy="mpa"), seed=0)
    sample, atoms = cpu_sample(crystals)
    pipeline.evaluate(ck, sample[:1], task)
    times, t_graph = [], 0.0
    for _ in range(args.warmup + args.steps):
        t, tg = cpu_oracle_eval(ck, sample, task)
        times.append(t)
        t_graph += tg
    timed = times[args.warmup:]
    rate = atoms * len(timed) / sum(timed)
    what = (f"first {len(sample)} structures ({atoms} atoms) of the workload per step as one batch, graph "
            f"construction included ({t_graph:.2f}s of {sum(times):.2f}s)")
    if replica:
        what = f"{replica}, one evaluation per step, graph construction included"
    line = {"impl": "reference", "metric": metric_name(task), "value": rate, "unit": "atoms*evals/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(timed) / len(timed),
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": desc, "task": task, "num_layers": NUM_LAYERS, "weights": "random-init seed 0",
                       "sample": what},
            "per_step_rate": {"min": atoms / max(timed), "median": atoms / float(np.median(timed)),
                              "max": atoms / min(timed)},
            "cpu_baseline": {"value": rate, "unit": "atoms*evals/s", "cores": threads, "kind": "port", "sample": what},
            "e2e": {"value": rate, "unit": "atoms*evals/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--md-steps", type=int, default=None,
                    help="Langevin MD steps to time on the 4,096-atom cell at N = 1 (default 200 with --workload lipscl, "
                         "else 20; 0 skips the MD leg)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--keep", default="auto", choices=["auto", "on", "off"],
                    help="keep sub-block internals for the backward pass (auto: when they fit in memory)")
    args = ap.parse_args()
    if args.workload is None:
        args.workload = "perov512" if args.scaling == "weak" else "random256"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    from matris_b200 import MatRIS, _lib, ops, parallel
    from matris_b200.graph import HostBatch, build_on_device, upload
    from matris_b200.weights import random_checkpoint

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    crystals, task, desc = make_workload(args.workload, world, args.scaling)
    ck = random_checkpoint(dict(num_layers=NUM_LAYERS, reference_energy="mpa"), seed=0)
    model = MatRIS.from_dict(ck).to(device)
    model.keep_activations = {"auto": None, "on": True, "off": False}[args.keep]
    cut, lcut = model.config["pairwise_cutoff"], model.config["three_body_cutoff"]
    # the same assignment predict_sharded makes: every rank computes it from the whole list
    costs = [parallel.predicted_cost(c.numbers, c.lattice, cut, lcut) for c in crystals]
    shards = parallel.shard_by_cost(costs, world)
    mine = [crystals[i] for i in shards[rank]]
    n_atoms = sum(len(c.numbers) for c in mine)
    atoms_job = sum(len(c.numbers) for c in crystals)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    widths = []
    for sh in shards:
        b, n = len(sh), sum(len(crystals[i].numbers) for i in sh)
        widths.append(2 * b + (9 * b if "s" in task else 0) + (3 * n if "f" in task else 0) + (n if "m" in task else 0))
    width = max(widths)

    def gather_results(out):
        """The result gather of the sharded path: one flat float32 buffer per rank, one NCCL gather."""
        parts = [out["e"], out["ref_energy"]]
        if "s" in task:
            parts.append(torch.stack(list(out["s"])).reshape(-1))
        if "f" in task:
            parts.append(torch.cat(list(out["f"])).reshape(-1))
        if "m" in task:
            parts.append(torch.cat(list(out["m"])).reshape(-1))
        flat = torch.cat([p.reshape(-1).float() for p in parts])
        if world > 1:
            buf = torch.zeros(width, dtype=torch.float32, device=device)
            buf[:flat.numel()] = flat
            dest = [torch.empty_like(buf) for _ in range(world)] if rank == 0 else None
            dist.gather(buf, dest, dst=0)
        return flat

    # ---- device-resident arm: positions/lattices already in HBM; a step = graph build + forward + backward + gather
    # The rank's structures are evaluated as the sub-batches MatRIS.predict would form (split_for_memory: one batch
    # when the internals of every layer fit in memory beside it, else contiguous ranges that do, so that the
    # backward pass recomputes nothing); every sub-batch's inputs are resident before the timed region.
    def resident(part):
        hb_ = HostBatch([c.numbers for c in part], [c.cart for c in part], [c.lattice for c in part], cut)
        return hb_, upload(hb_, cut, lcut, device)

    hb, g = resident(mine)
    build_on_device(g)
    ranges = model.split_for_memory(g)
    h2d_step = hb.h2d_bytes
    if len(ranges) > 1:
        del g
        parts = [resident(mine[a:b]) for a, b in ranges]
        h2d_step += sum(p[0].h2d_bytes for p in parts)  # predict uploads the whole list once to plan, then the parts
        graphs = [p[1] for p in parts]
    else:
        graphs = [g]

    def step_resident(gather=True):
        for g_ in graphs:
            build_on_device(g_)
        out = model.forward_batches(graphs, task=task)
        if gather:
            gather_results(out)
        return out

    for _ in range(args.warmup):
        step_resident()
    barrier()
    launches0 = _lib.launch_count
    ev0, ev1, evg = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        for _ in range(args.steps):
            out = step_resident(gather=False)
            evg.record()
            gather_results(out)
        ev1.record()
        barrier()
    t_gather = evg.elapsed_time(ev1)  # the last step's gather (includes waiting for the slowest rank)
    launches = _lib.launch_count - launches0
    my_ms = ev0.elapsed_time(ev1) / args.steps
    t_res = torch.tensor([my_ms * args.steps * 1e-3], device=device)
    if world > 1:
        dist.all_reduce(t_res, op=dist.ReduceOp.MAX)
    t_res = float(t_res)
    model.check_status()

    # ---- end-to-end arm: the public API on host structures, H2D of inputs and D2H of results inside the timing
    def step_e2e():
        o = model.predict_sharded(crystals, task)
        if o is None:
            return None
        res = [o["e"].cpu(), o["ref_energy"].cpu(), torch.cat(list(o["f"])).cpu()]
        if "s" in o:
            res.append(torch.stack(list(o["s"])).cpu())
        if "m" in o:
            res.append(torch.cat(list(o["m"])).cpu())
        return res

    step_e2e()
    barrier()
    with ClockSampler(local_rank) as clocks_e2e:
        ev0.record()
        for _ in range(args.steps):
            res = step_e2e()
        ev1.record()
        barrier()
    t_e2e = torch.tensor([ev0.elapsed_time(ev1) * 1e-3], device=device)
    h2d = torch.tensor([float(h2d_step)], device=device)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
        dist.all_reduce(h2d, op=dist.ReduceOp.SUM)
    t_e2e, h2d = float(t_e2e), int(h2d)
    d2h = sum(r.numel() * r.element_size() for r in res) if res is not None else 0
    model.check_status()

    # ---- per-rank table (what limits the scaling can be read from it)
    n_edges_mine, n_triplets_mine = sum(g_.n_edges for g_ in graphs), sum(g_.n_triplets for g_ in graphs)
    mine_row = torch.tensor([my_ms, float(n_atoms), float(n_edges_mine), float(n_triplets_mine), t_gather,
                             float(len(mine)), float(len(graphs)), float(model.last_kept_layers)], device=device)
    rows = [torch.empty_like(mine_row) for _ in range(world)] if (world > 1 and rank == 0) else None
    if world > 1:
        dist.gather(mine_row, rows, dst=0)
    else:
        rows = [mine_row]
    rank_table = None
    if rank == 0:
        rank_table = [{"rank": r, "ms_per_step": round(float(x[0]), 3), "atoms": int(x[1]), "directed_edges": int(x[2]),
                       "triplets": int(x[3]), "last_gather_ms": round(float(x[4]), 3), "structures": int(x[5]),
                       "sub_batches": int(x[6]), "kept_layers_last_sub_batch": int(x[7])}
                      for r, x in enumerate(rows)]

    # ---- one instrumented step: per-kernel device time (CUDA events on the launching stream)
    roofline, roofline_graph, kernel_table, gemm_shapes = None, None, None, None
    if rank == 0:
        torch.cuda.synchronize()
        with ClockSampler(local_rank) as clocks_peak:
            mma_peak, peak_ms = ops.mma_rate("bf16", 400000)  # >= 50 ms of resident-operand tcgen05.mma issue
        _lib.profile = []
        step_resident(gather=False)  # rank 0 only: no collective in here
        torch.cuda.synchronize()
        prof, _lib.profile = _lib.profile, None
        per, shapes = {}, {}
        gemm_flops, gemm_ms, gemm_bytes = 0.0, 0.0, 0.0
        for name, a, b, meta in prof:
            ms = a.elapsed_time(b)
            d = per.setdefault(name, [0, 0.0])
            d[0] += 1
            d[1] += ms
            if name in GEMM_CALLS:
                gemm_flops += meta["flops"]
                gemm_ms += ms
                gemm_bytes += meta["bytes"]  # A rows read once + output rows written
                tag = "gated " if meta.get("fused") else ""
                s = shapes.setdefault(f"{tag}rows={meta['rows']} K={meta['k']} N={meta['n']}", [0, 0.0, 0.0])
                s[0] += 1
                s[1] += ms
                s[2] += meta["flops"]
        total_ms = sum(v[1] for v in per.values())
        kernel_table = {k: {"launches": v[0], "ms": round(v[1], 3), "share": round(v[1] / total_ms, 4)}
                        for k, v in sorted(per.items(), key=lambda kv: -kv[1][1])}
        gemm_shapes = {k: {"launches": v[0], "ms": round(v[1], 3), "tflops": round(v[2] / (v[1] * 1e-3) / 1e12, 1)}
                       for k, v in sorted(shapes.items(), key=lambda kv: -kv[1][1])[:10]}
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak_tf = float(peaks.get("bf16_tflops_sustained", 1590.0 * 1411.6 / 1677.1))
        peak_gb = float(peaks.get("hbm_gbs", 6650.0))
        src = "measured" if peaks else "fallback"
        ach = gemm_flops / (gemm_ms * 1e-3) / 1e12
        ach_gb = gemm_bytes / (gemm_ms * 1e-3) / 1e9
        n_gemm = sum(per[k][0] for k in GEMM_CALLS if k in per)
        # DRAM traffic per launch: ncu captures of 151,552-row launches measured 0.91 - 0.95 x the algorithmic bytes
        # (A rows read + gate / residual rows read + output rows written); scaled here to the average launch of the
        # step by its algorithmic bytes.
        pk = clocks_peak.summary()
        roofline = {"kernel": "k_gemm_ps + k_gated_fwd (mb_gemm, mb_gated_mlp_fwd)", "bound": "tensor", "achieved": ach,
                    "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf, "traffic": 0.93 * gemm_bytes / n_gemm,
                    "traffic_note": "bytes per average launch, scaled from ncu captures by the algorithmic bytes",
                    "peak_source": src + " bf16 sustained",
                    "launches": n_gemm, "avg_launch_ms": gemm_ms / n_gemm,
                    "flops_per_step": gemm_flops, "mma_kind": "kind::f16, 3xBF16 operand split",
                    "mma_issued_tflops": 3.0 * ach, "mma_peak_timed_tflops": mma_peak, "mma_peak_timed_ms": peak_ms,
                    "mma_peak_timed_sm_mhz": pk["sm_mhz"], "frac_of_mma_peak": 3.0 * ach / mma_peak,
                    "hbm_view": {"algorithmic_bytes_per_step": gemm_bytes, "achieved_gbs": ach_gb, "peak_gbs": peak_gb,
                                 "frac": ach_gb / peak_gb,
                                 "floor_ms_hbm": gemm_bytes / (peak_gb * 1e9) * 1e3,
                                 "floor_ms_tensor": gemm_flops / (peak_tf * 1e12) * 1e3,
                                 "note": "with the activations these launches read and write (fp32 rows, z1 / z2 kept "
                                         "for the backward) their HBM floor is above their tensor floor: the HBM "
                                         "fraction is what the time follows"},
                    "note": "tcgen05 kind::f16 with a 3-term bf16 operand split: 3 tensor FLOPs are issued per "
                            "algorithmic FLOP; mma_peak_timed = CUDA-event-timed tcgen05.mma issue loop on resident "
                            "operands in this run (mb_bench_mma_rate), with the SM clock sampled during it"}
        gms = sum(per[k][1] for k in per if k.startswith("mb_graph"))
        gbytes = 26.0 * n_edges_mine + 20.0 * n_triplets_mine + 16.0 * n_atoms
        roofline_graph = {"kernels": "mb_graph_*", "bound": "hbm", "achieved": gbytes / (gms * 1e-3) / 1e9,
                          "peak": peak_gb, "unit": "GB/s", "frac": gbytes / (gms * 1e-3) / 1e9 / peak_gb,
                          "traffic": None, "algorithmic_bytes": gbytes, "ms": gms, "peak_source": src}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_crystals, replica = cpu_workload(args.workload, crystals)
        rate, info = cpu_oracle_rate(cpu_crystals, task, budget_s=20.0)
        cpu_baseline = {"value": rate, "unit": "atoms*evals/s", "cores": info["threads"], "kind": "port",
                        "sample": (replica + ", " if replica else "") +
                                  f"first {info['structures']} structures ({info['atoms']} atoms) of the workload as "
                                  f"one batch, {info['reps']} repetitions, {info['seconds']:.1f}s of CPU work",
                        "per_repetition": {"min": info["rate_min"], "median": info["rate_median"],
                                           "max": info["rate_max"]}}
        rate1, info1 = cpu_oracle_rate(cpu_crystals, task, budget_s=8.0, threads=1, max_structs=4, max_cost=2.5e4,
                                       max_reps=3)
        cpu_baseline["one_thread"] = {"value": rate1, "cores": 1,
                                      "sample": f"first {info1['structures']} structures ({info1['atoms']} atoms), "
                                                f"{info1['reps']} repetitions, {info1['seconds']:.1f}s of CPU work"}

    # ---- MD leg (the metric's second figure: MD steps/s on the 4,096-atom Li6PS5Cl cell): the public MolecularDynamics
    # driver, Langevin NVT at 600 K, dt = 1 fs, friction 0.01 / fs, Maxwell-Boltzmann start, one efsm evaluation per
    # step (graph rebuilt every step on the device).  Runs at N = 1 after the evaluation arms: 200 steps when the
    # cell is the workload, 20 otherwise (--md-steps overrides; 0 skips).
    md = None
    md_steps = args.md_steps if args.md_steps is not None else (200 if args.workload == "lipscl" else 20)
    if rank == 0 and world == 1 and md_steps > 0:
        from matris_b200.applications import MolecularDynamics

        md_cell = crystals[0] if args.workload == "lipscl" else make_workload("lipscl", 1, "weak")[0][0]
        dyn = MolecularDynamics(md_cell, model=model, ensemble="nvt", thermostat="langevin", temperature=600,
                                starting_temperature=600, timestep=1.0, friction=0.01, task="efsm", device=device,
                                seed=2)
        dyn.run(3)
        torch.cuda.synchronize()
        with ClockSampler(local_rank) as clocks_md:
            t0 = time.perf_counter()
            dyn.run(md_steps)
            torch.cuda.synchronize()
            t_md = time.perf_counter() - t0
        md = {"metric": "md_steps_per_s", "value": md_steps / t_md, "steps": md_steps, "ms_per_step": 1e3 * t_md / md_steps,
              "atoms": len(md_cell.numbers), "workload": "amorphous Li6PS5Cl, 4096 atoms",
              "setup": "Langevin (BAOAB) NVT 600 K, dt 1 fs, friction 0.01/fs, efsm every step, "
                                         "integrator state and graph rebuild on the device (MolecularDynamics device_resident=True)",
              "temperature_K_end": float(dyn.atoms.get_temperature()), "clocks": clocks_md.summary()}

    if rank == 0:
        value = atoms_job * args.steps / t_res
        job_flops = sum(flops_per_eval(r["atoms"], r["directed_edges"], r["triplets"], NUM_LAYERS) for r in rank_table)
        line = {"metric": metric_name(task), "value": value, "unit": "atoms*evals/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_res / args.steps,
                "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": desc, "task": task, "num_layers": NUM_LAYERS, "weights": "random-init seed 0",
                           "atoms": atoms_job, "structures": len(crystals),
                           "l2": "per-step working set (>1 GB of activations) exceeds the 126 MB L2",
                           "parallelism": f"structures sharded by predicted cost over {world} rank(s); one gather of "
                                          "E, F, S, M per step, no other collective",
                           "sub_batches": f"rank 0 evaluates its {len(mine)} structures as {len(graphs)} sub-batch(es) "
                                          "chosen by MatRIS.split_for_memory (all layers' internals kept, no "
                                          "recomputation in the backward pass)"},
                "ranks": rank_table,
                "clocks": clocks.summary(), "clocks_e2e": clocks_e2e.summary(),
                "e2e": {"value": atoms_job * args.steps / t_e2e, "unit": "atoms*evals/s",
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": 1e3 * t_e2e / args.steps,
                        "api": "MatRIS.predict_sharded(structures, task) + .cpu() of E, F, S, M on rank 0"},
                "gpu_launches": launches, "gpu_launches_note": "C-ABI kernel-launching calls of rank 0 in the timed "
                                                               "region (each issues one or more kernels)",
                "achieved_tflops_algorithmic": job_flops * args.steps / t_res / 1e12,
                "roofline": roofline, "roofline_graph_build": roofline_graph, "kernels": kernel_table,
                "gemm_shapes": gemm_shapes, "cpu_baseline": cpu_baseline}
        if md is not None:
            line["md"] = md
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
