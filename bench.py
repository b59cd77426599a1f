#!/usr/bin/env python
"""Benchmark of the per-atom evaluation path: atoms/s for energy + forces + virial.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload mtp16|nep] [--impl reference]

One step = one pass of the hot path over the workload (neighbour-list build from positions when
the CUDA builder is available, then descriptors + force/virial). Prints ONE JSON line on rank 0.
Synthetic seeded inputs (ai2pot_b200/synth.py) stand in for a dataset.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import numpy as np


def load_tables(level):
    z = np.load(os.path.join(ROOT, "tests", "golden", f"mtp_tables_L{level:02d}.npz"))
    return dict(alpha_moments_count=int(z["alpha_moments_count"]), nmus=int(z["nmus"]),
                alpha_index_basic=z["alpha_index_basic"], alpha_index_times=z["alpha_index_times"],
                alpha_moment_mapping=z["alpha_moment_mapping"])


# algorithmic flops per atom of the descriptor + force/virial path (FMA = 2)
def flops_mtp(nn, n_basic, n_times, n_scalar, nmus, cs, kmax):
    R = 9 * cs + 20 + 4 * nmus * cs
    Pw = 4 * kmax + 4
    return nn * (R + Pw + 29 * n_basic) + 9 * n_times + 4 * n_scalar


def flops_nep(nn_r, nn_a, cs, n_r, n_a, neurons, n_desc):
    return (nn_r * (9 * cs + 20 + 4 * n_r * cs + 4 * n_r + 12) + nn_a * (9 * cs + 20 + 4 * n_a * cs + 384 + 22 * 24 * n_a)
            + 6 * 24 * n_a + 4 * neurons * n_desc + 20 * neurons)


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thr = threading.Thread(target=self._read, daemon=True)
            self.thr.start()
            # nvidia-smi takes ~0.1-0.3 s to attach to the driver; wait for its first line so that this
            # start-up does not run (and perturb kernel launches) inside the timed region
            t0 = time.time()
            while not self.rows and time.time() - t0 < 3.0:
                time.sleep(0.01)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 7 for i in range(4) if r[3 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def make_workload(name):
    from ai2pot_b200 import synth
    if name == "mtp16":
        w = synth.g1(load_tables(16))
        w["label"] = "configs[1]: MTP level 16, fp64, 13,824 atoms, rcut 6.0, 3 species"
        w["dtype"] = "f64"
    elif name == "nep":
        w = synth.g2()
        w["label"] = "configs[2]: NEP fp32 (3-body), 13,824 atoms, rc 6.0/4.0"
        w["dtype"] = "f32"
    elif name == "train":
        w = synth.g3(load_tables(16))
        w["kind"] = "train"
        w["label"] = "configs[3]: MTP level 16 training step, fp64, 64 structures of 64-256 atoms, E/F/V + loss + coefficient gradient"
        w["dtype"] = "f64"
        w["types"] = np.concatenate([s["types"] for s in w["structs"]])
    elif name == "md":
        w = synth.g2()
        w["kind"] = "md"
        w["label"] = "configs[2] system handed over as an MD host holds it (13,824 local atoms + periodic ghost images, double positions), NEP fp32: one force call"
        w["dtype"] = "f32"
    elif name == "nep_train":
        w = synth.g3(load_tables(16))
        w["kind"] = "train"
        w["model"] = synth.nep_model(3, np.random.default_rng(1005), np.float32)
        w["label"] = "configs[3] structures with an fp32 NEP model: training step, 64 structures of 64-256 atoms, E/F/V + loss + gradient w.r.t. coeffs, w0, b0, w1, bias"
        w["dtype"] = "f32"
        w["types"] = np.concatenate([s["types"] for s in w["structs"]])
    elif name.startswith("nep1m"):
        ncell = int(name.split(":")[1]) if ":" in name else 64
        w = synth.g4(ncell=ncell)
        w["kind"] = "slab"
        w["label"] = f"configs[4]: NEP fp32 (3-body), {4 * ncell ** 3:,} atoms, x-slabs with 6 A halos, ghost-force reduction"
        w["dtype"] = "f32"
    else:
        raise SystemExit(f"unknown workload {name}")
    return w


def cpu_reference_run(w, kind_pref, budget_s, threads):
    """Times the CPU implementation (reference build if present, else the C restatement) on the
    workload: neighbour list (serial in the reference) + E/F/V with `threads` OpenMP threads."""
    from oracle import refapi
    from ai2pot_b200 import synth
    kind = "ref" if (kind_pref == "ref" and refapi.available("ref")) else "oracle"
    os.environ["OMP_NUM_THREADS"] = str(threads)
    chk = refapi.Checker(kind)
    t0 = time.perf_counter()
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    t_nb = time.perf_counter() - t0
    nb = synth.batch_from_nblist(nn, fn, rc, ty, w["model"]["ntypes"])
    fn_efv = chk.mtp_efv if w["model"]["kind"] == "mtp" else chk.nep_efv
    times = []
    t_start = time.perf_counter()
    while len(times) < 5 and (time.perf_counter() - t_start < budget_s or not times):
        t0 = time.perf_counter()
        fn_efv(w["model"], nb)
        times.append(time.perf_counter() - t0)
    return kind, t_nb, min(times), len(times), float(nn.mean())


def cpu_reference_train(w, budget_s, threads):
    """CPU arm of the training step: forward E/F/V + loss + analytic gradient on the whole batch
    (the reference evaluates E/F/V a second time inside its backward; that repeat is not timed).
    Neighbour lists are built before the timed part, as the reference's dataset does."""
    from oracle import refapi
    from ai2pot_b200 import synth
    kind = "ref" if refapi.available("ref") else "oracle"
    os.environ["OMP_NUM_THREADS"] = str(threads)
    chk = refapi.Checker(kind)
    lists = []
    for s in w["structs"]:
        nn, fn, rc, ty, mx = chk.nblist(s["cell"], s["types"], s["coords"], w["rcut"], w["umax"])
        lists.append((nn, fn, rc, ty))
    nb = synth.pad_batch(lists, w["model"]["ntypes"], w["umax"])
    t = w["targets"]
    npad = nb["bilist"].shape[1]
    is_nep = w["model"]["kind"] == "nep"
    if is_nep:
        nb["brcs"] = nb["brcs"].astype(np.float32)
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 and (time.perf_counter() - t_start < budget_s or not times):
        t0 = time.perf_counter()
        if is_nep:
            e, f, v = chk.nep_efv(w["model"], nb)
            chk.mtp_loss(nb, w["weights"], e, t["E"], f, t["F"][:, :npad], v, t["V"])
            chk.nep_loss_backward(w["model"], nb, w["weights"], e, t["E"], f, t["F"][:, :npad], v, t["V"])
        else:
            e, f, v = chk.mtp_efv(w["model"], nb)
            chk.mtp_loss(nb, w["weights"], e, t["E"], f, t["F"][:, :npad], v, t["V"])
            chk.mtp_loss_backward(w["model"], nb, w["weights"], e, t["E"], f, t["F"][:, :npad], v, t["V"])
        times.append(time.perf_counter() - t0)
    return kind, 0.0, min(times), len(times)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="mtp16")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    ncores = len(os.sched_getaffinity(0))
    w = make_workload(args.workload)
    natoms = len(w["types"])
    metric = "atoms/sec for E+F+virial"
    strong = w.get("kind") in ("train", "slab")           # a fixed batch / system divided over the ranks (md: replicas)
    config = {"workload": w["label"], "atoms_per_gpu": natoms // world if strong else natoms,
              "l2": "256 MiB buffer written between timed steps"}

    if args.impl == "reference":
        if rank != 0:
            return
        if w.get("kind") == "train":
            kind, t_nb, t_efv, nrep = cpu_reference_train(w, 60.0, ncores)
        else:
            kind, t_nb, t_efv, nrep, mean_nn = cpu_reference_run(w, "ref", 60.0, ncores)
        steps = max(1, args.steps)
        t_step = t_nb + t_efv
        val = natoms / t_step
        line = {"impl": "reference", "metric": metric, "value": val, "unit": "atoms/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_step, "higher_is_better": True,
                "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "config": config,
                "cpu_baseline": {"value": val, "unit": "atoms/s", "cores": ncores,
                                 "kind": "reference" if kind == "ref" else "port",
                                 "sample": f"full workload, nblist {t_nb:.3f}s (serial) + E/F/V best of {nrep} = {t_efv:.3f}s"},
                "e2e": {"value": val, "unit": "atoms/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import torch
    from ai2pot_b200 import capi, engine
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    res = engine.run_benchmark(w, args.steps, args.warmup, dist, ClockSampler(local))
    if world > 1:
        t = torch.tensor([res["t_dev"], res["t_e2e"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["t_dev"], res["t_e2e"] = float(t[0]), float(t[1])
    if rank == 0:
        total_atoms = natoms if strong else natoms * world
        value = total_atoms * args.steps / res["t_dev"]
        line = {"metric": metric, "value": value, "unit": "atoms/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": 1e3 * res["t_dev"] / args.steps, "higher_is_better": True,
                "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "config": config,
                "clocks": res["clocks"], "gpu_launches": res["launches"],
                "e2e": {"value": total_atoms * args.steps / res["t_e2e"], "unit": "atoms/s",
                        "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"], "path": res["e2e_path"]},
                "roofline": res["roofline"], "parts_ms": res.get("parts_ms")}
        if "cuda_graph" in res:
            config["cuda_graph"] = bool(res["cuda_graph"])
        if world > 1:
            config["parallelism"] = ("replicas only: %d independent copies, no data-path collective" % world) if not strong else \
                ("structures dealt over %d ranks + one gradient all-reduce" % world if w["kind"] == "train" else "%d x-slabs, halo exchange + ghost-force reduction over NCCL" % world)
        if world == 1 and not args.no_cpu_baseline and w.get("kind") == "train":
            kind, t_nb, t_efv, nrep = cpu_reference_train(w, 20.0, ncores)
            line["cpu_baseline"] = {"value": natoms / t_efv, "unit": "atoms/s", "cores": ncores, "kind": "reference" if kind == "ref" else "port",
                                    "sample": f"whole batch: E/F/V + loss + gradient, best of {nrep} = {t_efv:.3f}s"}
        elif world == 1 and not args.no_cpu_baseline and (w.get("kind") is None or natoms <= 200000):
            kind, t_nb, t_efv, nrep, mean_nn = cpu_reference_run(w, "ref", 20.0, ncores)
            line["cpu_baseline"] = {"value": natoms / (t_nb + t_efv), "unit": "atoms/s", "cores": ncores,
                                    "kind": "reference" if kind == "ref" else "port",
                                    "sample": f"full workload once: nblist {t_nb:.3f}s (serial) + E/F/V best of {nrep} = {t_efv:.3f}s"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
