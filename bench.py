#!/usr/bin/env python
"""Throughput of the E/F/S evaluation path: atoms*evals/s on a batch of random crystals.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload random256|perov512|cu32|fe16k|lipscl] [--md-steps N]

Workload (default): 256 random periodic crystals, 8-64 atoms each, seed 1 (+ rank), task
"efs", MatRIS with 10 interaction blocks and seeded random-init weights.  One step =
graph build + forward + backward for the whole batch.  N > 1: one process per GPU
(torchrun), every rank evaluates its own batch (weak scaling, no data-path collective),
energies are gathered to rank 0.

`value` is timed with inputs resident in HBM (positions, lattices); `e2e` goes through the
public API (`MatRIS.predict` on host structures) with the host->device copies and the
device->host read of E/F/S inside the timed region.  `--impl reference` times the CPU
oracle (the restatement of the reference's PyTorch path) on a bounded sample instead.
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
METRIC = "atoms*evals/s (efs, fp32-tol)"


def make_workload(name: str, rank: int):
    from matris_b200 import workloads as w
    if name == "random256":
        return w.random_crystals(256, seed=1 + rank), "efs", "256 random crystals (8-64 atoms), seed 1+rank"
    if name == "random64":  # small case for profiler captures (activations still exceed the L2)
        return w.random_crystals(64, seed=1 + rank), "efs", "64 random crystals (8-64 atoms), seed 1+rank"
    if name == "perov512":
        return w.perovskites(512, seed=4 + rank), "efsm", "512 ABX3 2x2x2 perovskite cells (40 atoms)"
    if name == "cu32":
        return [w.cu_fcc()], "efsm", "Cu FCC 2x2x2, 32 atoms"
    if name == "fe16k":
        return [w.fe_bcc()], "efsm", "BCC Fe 20x20x20, 16000 atoms"
    if name == "lipscl":
        return [w.lipscl()], "efsm", "amorphous Li6PS5Cl, 4096 atoms"
    raise SystemExit(f"unknown workload {name}")


def flops_per_eval(g, layers):
    """Algorithmic GEMM FLOPs of one forward + backward evaluation (no recompute counted):
    2 (fwd+bwd) * 2 (MAC) * L * (360448 T + 327680 Ed + 163840 Eu + 163840 N)."""
    return 4.0 * layers * (360448.0 * g.n_triplets + 327680.0 * g.n_edges + 163840.0 * g.n_bonds + 163840.0 * g.n_atoms)


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


def cpu_oracle_rate(crystals, task, budget_s=20.0, max_structs=16, threads=None):
    """atoms*evals/s of the CPU oracle on the first structures of the workload, evaluated as one batch
    (graph construction included); repeated until about ``budget_s`` seconds of CPU work are spent."""
    import torch

    from matris_b200.weights import random_checkpoint
    from oracle import pipeline
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    ck = random_checkpoint(dict(num_layers=NUM_LAYERS, reference_energy="mpa"), seed=0)
    cfg = ck["config"]
    sample = crystals[:max_structs]
    atoms = sum(len(c.numbers) for c in sample)
    pipeline.evaluate(ck, sample[:1], task)  # warm-up
    t_total = t_graph = 0.0
    reps = 0
    while t_total < budget_s and reps < 8:
        t0 = time.perf_counter()
        graphs = [pipeline.graph_from_arrays(c.numbers, c.cart, c.lattice, float(cfg["pairwise_cutoff"]),
                                             float(cfg["three_body_cutoff"])) for c in sample]
        t1 = time.perf_counter()
        pipeline.evaluate(ck, sample, task, graphs=graphs)
        t2 = time.perf_counter()
        t_graph += t1 - t0
        t_total += t2 - t0
        reps += 1
    return atoms * reps / t_total, dict(structures=len(sample), atoms=atoms, reps=reps, seconds=t_total,
                                        graph_seconds=t_graph, threads=threads)


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the reference's PyTorch path on the host cores."""
    if rank != 0:
        return
    crystals, task, desc = make_workload(args.workload, 0)
    rates, info = [], None
    for _ in range(args.warmup + args.steps):
        r, info = cpu_oracle_rate(crystals, task, budget_s=1.0, max_structs=16)  # one batch evaluation per step
        rates.append(r)
    rate = float(np.mean(rates[args.warmup:]))
    sample = (f"first {info['structures']} structures ({info['atoms']} atoms) of the workload per step as one "
              f"batch, graph construction included ({info['graph_seconds']:.2f}s of {info['seconds']:.2f}s)")
    line = {"impl": "reference", "metric": METRIC, "value": rate, "unit": "atoms*evals/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * info["seconds"] / info["reps"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": desc, "task": task, "num_layers": NUM_LAYERS, "weights": "random-init seed 0"},
            "cpu_baseline": {"value": rate, "unit": "atoms*evals/s", "cores": info["threads"], "kind": "port",
                             "sample": sample},
            "e2e": {"value": rate, "unit": "atoms*evals/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="random256")
    ap.add_argument("--md-steps", type=int, default=None,
                    help="with --workload lipscl: Langevin MD steps to time (default 200; 0 skips the MD leg)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--keep", default="auto", choices=["auto", "on", "off"],
                    help="keep sub-block internals for the backward pass (auto: when they fit in memory)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    from matris_b200 import MatRIS, _lib
    from matris_b200.graph import HostBatch, build_on_device, upload
    from matris_b200.weights import random_checkpoint

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    crystals, task, desc = make_workload(args.workload, rank)
    ck = random_checkpoint(dict(num_layers=NUM_LAYERS, reference_energy="mpa"), seed=0)
    model = MatRIS.from_dict(ck).to(device)
    model.keep_activations = {"auto": None, "on": True, "off": False}[args.keep]
    cut, lcut = model.config["pairwise_cutoff"], model.config["three_body_cutoff"]
    n_atoms = sum(len(c.numbers) for c in crystals)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gather_energy(e):
        if world > 1:
            parts = [torch.empty_like(e) for _ in range(world)] if rank == 0 else None
            dist.gather(e, parts, dst=0)

    # ---- device-resident arm: positions/lattices already in HBM; a step = graph build + forward + backward
    hb = HostBatch([c.numbers for c in crystals], [c.cart for c in crystals], [c.lattice for c in crystals], cut)
    g = upload(hb, cut, lcut, device)

    def step_resident(gather=True):
        build_on_device(g)
        out = model(g, task=task)
        if gather:
            gather_energy(out["e"])
        return out

    for _ in range(args.warmup):
        step_resident()
    barrier()
    launches0 = _lib.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        for _ in range(args.steps):
            out = step_resident()
        ev1.record()
        barrier()
    launches = _lib.launch_count - launches0
    t_res = torch.tensor([ev0.elapsed_time(ev1) * 1e-3], device=device)
    atoms_total = torch.tensor([float(n_atoms)], device=device)
    if world > 1:
        dist.all_reduce(t_res, op=dist.ReduceOp.MAX)
        dist.all_reduce(atoms_total, op=dist.ReduceOp.SUM)
    t_res, atoms_total = float(t_res), float(atoms_total)

    # ---- end-to-end arm: the public API on host structures, H2D of inputs and D2H of results inside the timing
    def step_e2e():
        o = model.predict(crystals, task)
        res = [o["e"].cpu(), torch.cat(list(o["f"])).cpu()]
        if "s" in o:
            res.append(torch.stack(o["s"]).cpu())
        if "m" in o:
            res.append(torch.cat(o["m"]).cpu())
        gather_energy(o["e"])
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
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    t_e2e = float(t_e2e)
    d2h = sum(r.numel() * r.element_size() for r in res)

    # ---- one instrumented step: per-kernel device time (CUDA events on the launching stream)
    roofline, roofline_graph, kernel_table, gemm_shapes = None, None, None, None
    if rank == 0:
        torch.cuda.synchronize()
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
        n_gemm = sum(per[k][0] for k in GEMM_CALLS if k in per)
        # DRAM traffic per launch: ncu measured 0.906 x (A read + output write) on a captured K=384 N=256 launch of
        # 151,552 rows (profiles/k_gemm_ps.md); scaled here to the average launch of the step by its rows x (K + N).
        roofline = {"kernel": "k_gemm_ps + k_gated_fwd (mb_gemm, mb_gated_mlp_fwd)", "bound": "tensor", "achieved": ach, "peak": peak_tf,
                    "unit": "TFLOP/s", "frac": ach / peak_tf, "traffic": 0.906 * gemm_bytes / n_gemm,
                    "traffic_note": "bytes per average launch, scaled from one ncu capture by rows x (K + N)",
                    "peak_source": src + " bf16 sustained",
                    "launches": n_gemm, "avg_launch_ms": gemm_ms / n_gemm,
                    "flops_per_step": gemm_flops, "tf32_issued_tflops": 3.0 * ach, "tf32_peak_measured_tflops": 1151.0,
                    "frac_of_tf32_peak": 3.0 * ach / 1151.0,
                    "note": "tcgen05 kind::tf32 with a 3-term operand split: 3 tensor FLOPs are issued per "
                            "algorithmic FLOP; 1151 TFLOP/s = measured raw tcgen05.mma tf32 rate (64 cycles per "
                            "M128 N128 K8 MMA x 148 SMs x 1.9 GHz)"}
        gms = sum(per[k][1] for k in per if k.startswith("mb_graph"))
        gbytes = 26.0 * g.n_edges + 20.0 * g.n_triplets + 16.0 * g.n_atoms
        roofline_graph = {"kernels": "mb_graph_* (3 phases)", "bound": "hbm", "achieved": gbytes / (gms * 1e-3) / 1e9,
                          "peak": peak_gb, "unit": "GB/s", "frac": gbytes / (gms * 1e-3) / 1e9 / peak_gb,
                          "traffic": None, "algorithmic_bytes": gbytes, "ms": gms, "peak_source": src}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, info = cpu_oracle_rate(crystals, task, budget_s=20.0, max_structs=16)
        cpu_baseline = {"value": rate, "unit": "atoms*evals/s", "cores": info["threads"], "kind": "port",
                        "sample": f"first {info['structures']} structures ({info['atoms']} atoms) of the workload as "
                                  f"one batch, {info['reps']} repetitions, {info['seconds']:.1f}s of CPU work"}
        rate1, info1 = cpu_oracle_rate(crystals, task, budget_s=8.0, max_structs=4, threads=1)
        cpu_baseline["one_thread"] = {"value": rate1, "cores": 1,
                                      "sample": f"first {info1['structures']} structures ({info1['atoms']} atoms), "
                                                f"{info1['reps']} repetitions, {info1['seconds']:.1f}s of CPU work"}

    # ---- MD leg (4,096-atom cell only): the public MolecularDynamics driver, Langevin NVT at 600 K, dt = 1 fs,
    # friction 0.01 / fs, Maxwell-Boltzmann start, one efsm evaluation per step (graph rebuilt every step on the device)
    md = None
    md_steps = args.md_steps if args.md_steps is not None else (200 if args.workload == "lipscl" else 0)
    if rank == 0 and world == 1 and args.workload == "lipscl" and md_steps > 0:
        from matris_b200.applications import MolecularDynamics

        dyn = MolecularDynamics(crystals[0], model=model, ensemble="nvt", thermostat="langevin", temperature=600,
                                starting_temperature=600, timestep=1.0, friction=0.01, task="efsm", device="cuda",
                                seed=2)
        dyn.run(3)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dyn.run(md_steps)
        torch.cuda.synchronize()
        t_md = time.perf_counter() - t0
        md = {"metric": "md_steps_per_s", "value": md_steps / t_md, "steps": md_steps, "ms_per_step": 1e3 * t_md / md_steps,
              "atoms": n_atoms, "setup": "Langevin (BAOAB) NVT 600 K, dt 1 fs, friction 0.01/fs, efsm every step, "
                                         "integrator state and graph rebuild on the device (MolecularDynamics device_resident=True)",
              "temperature_K_end": float(dyn.atoms.get_temperature())}

    if rank == 0:
        value = atoms_total * args.steps / t_res
        line = {"metric": METRIC, "value": value, "unit": "atoms*evals/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": 1e3 * t_res / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": desc, "task": task, "num_layers": NUM_LAYERS, "weights": "random-init seed 0",
                           "atoms_per_rank": n_atoms, "directed_edges": g.n_edges, "triplets": g.n_triplets,
                           "l2": "per-step working set (>1 GB of activations) exceeds the 126 MB L2",
                           "parallelism": f"structures sharded, {world} rank(s), result gather only"},
                "clocks": clocks.summary(), "clocks_e2e": clocks_e2e.summary(),
                "e2e": {"value": atoms_total * args.steps / t_e2e, "unit": "atoms*evals/s",
                        "h2d_bytes_per_step": hb.h2d_bytes, "d2h_bytes_per_step": d2h,
                        "ms_per_step": 1e3 * t_e2e / args.steps},
                "gpu_launches": launches, "gpu_launches_note": "C-ABI kernel-launching calls in the timed region "
                                                               "(each issues one or more kernels)",
                "achieved_tflops_algorithmic": flops_per_eval(g, NUM_LAYERS) * world * args.steps / t_res / 1e12,
                "roofline": roofline, "roofline_graph_build": roofline_graph, "kernels": kernel_table,
                "gemm_shapes": gemm_shapes if rank == 0 else None,
                "cpu_baseline": cpu_baseline}
        if md is not None:
            line["md"] = md
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
