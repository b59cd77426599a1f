#!/usr/bin/env python
"""Benchmark of the per-atom evaluation path: atoms/s for energy + forces + virial.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload auto|mtp16|nep|nep1m|train|nep_train|md] [--impl reference]

One step = one pass of the hot path over the workload (neighbour-list build from positions, then
descriptors + force/virial). Prints ONE JSON line on rank 0. Synthetic seeded inputs
(ai2pot_b200/synth.py) stand in for a dataset.

Default workload ("auto"):
  * one process on a box with one visible GPU: configs[1] (MTP level 16, fp64, 13,824 atoms) is the headline
    `value`; configs[2] (NEP fp32 on the same structure) is measured in the same invocation and nested under "nep";
  * under torch.distributed.run (WORLD_SIZE set), or with --gpus 1 on a box that shows several GPUs (the one-GPU
    point of a scaling series): configs[4], the 1,048,576-atom NEP system cut into x-slabs, "scaling": "strong".
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np


def make_workload(name):
    from ai2pot_b200 import synth, tables
    if name == "mtp16":
        w = synth.g1(tables.load(16))
        w["label"] = "configs[1]: MTP level 16, fp64, 13,824 atoms, rcut 6.0, 3 species"
        w["dtype"] = "f64"
    elif name == "nep":
        w = synth.g2()
        w["label"] = "configs[2]: NEP fp32 (3-body), 13,824 atoms, rc 6.0/4.0"
        w["dtype"] = "f32"
    elif name == "train":
        w = synth.g3(tables.load(16))
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
        w = synth.g3(tables.load(16))
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


def visible_gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def resolve_workload(name):
    """'auto' -> the slab workload when this run is (or looks like) a point of a multi-GPU scaling series,
    else the two 13,824-atom configurations."""
    if name != "auto":
        return name, False
    if "WORLD_SIZE" in os.environ or visible_gpus() > 1:
        return "nep1m", False
    return "mtp16", True            # True: also measure configs[2] and nest it under "nep"


def cpu_reference_run(w, budget_s, threads):
    """Times the CPU implementation (reference build if present, else the C restatement) on the
    workload: neighbour list (serial in the reference) + E/F/V with `threads` OpenMP threads.
    Returns kind, t_nblist, best E/F/V time, number of E/F/V calls timed."""
    from oracle import refapi
    from ai2pot_b200 import synth
    kind = "ref" if refapi.available("ref") else "oracle"
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
    return kind, t_nb, min(times), len(times)


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


def cpu_baseline(w, budget_s, threads):
    """cpu_baseline object of a workload: the reference's CPU code on the box's host cores. For the slab workload
    the sample is a smaller periodic cell of the same lattice, density and model (the CPU neighbour list of the full
    1,048,576-atom system alone takes ~10 s and ~4 GB); throughput in atoms/s is what is compared."""
    if w.get("kind") == "train":
        kind, t_nb, t_efv, nrep = cpu_reference_train(w, budget_s, threads)
        n = len(w["types"])
        return {"value": n / t_efv, "unit": "atoms/s", "cores": threads, "kind": "reference" if kind == "ref" else "port",
                "sample": f"whole batch ({n} atoms): E/F/V + loss + gradient, best of {nrep} = {t_efv:.3f}s; neighbour lists not timed",
                "calls_timed": nrep, "ms_per_step": 1e3 * t_efv}
    sample_note = "full workload"
    if w.get("kind") == "slab" and len(w["types"]) > 200000:
        from ai2pot_b200 import synth
        w = dict(synth.g4(ncell=32), kind="slab")
        sample_note = "131,072-atom periodic cell (32^3 cells) of the same lattice, density and model"
    kind, t_nb, t_efv, nrep = cpu_reference_run(w, budget_s, threads)
    n = len(w["types"])
    return {"value": n / (t_nb + t_efv), "unit": "atoms/s", "cores": threads, "kind": "reference" if kind == "ref" else "port",
            "sample": f"{sample_note}: nblist once {t_nb:.3f}s (serial in the reference) + E/F/V best of {nrep} = {t_efv:.3f}s",
            "calls_timed": nrep, "ms_per_step": 1e3 * (t_nb + t_efv)}


def config_of(w, world, strong):
    natoms = len(w["types"])
    config = {"workload": w["label"], "atoms_per_gpu": natoms // world if strong else natoms,
              "l2": "256 MiB buffer written between timed steps"}
    if world > 1:
        config["parallelism"] = ("replicas only: %d independent copies, no data-path collective" % world) if not strong else \
            ("structures dealt over %d ranks + one gradient all-reduce" % world if w["kind"] == "train"
             else "%d x-slabs with 6 A halos: halo exchange, ghost-force return, reduction of E and virial" % world)
    return config


def gpu_line(w, args, world, dist, local):
    """Runs one workload on the GPU(s); returns the JSON object (rank 0) or None."""
    import torch
    import bench_lib
    strong = w.get("kind") in ("train", "slab")           # a fixed batch / system divided over the ranks (md: replicas)
    natoms = len(w["types"])
    res = bench_lib.run_benchmark(w, args.steps, args.warmup, dist, bench_lib.ClockSampler(local))
    if world > 1:
        t = torch.tensor([res["t_dev"], res["t_e2e"], res.get("host_ms_per_call") or 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["t_dev"], res["t_e2e"], res["host_ms_per_call"] = float(t[0]), float(t[1]), float(t[2])
    if int(os.environ.get("RANK", "0")) != 0:
        return None
    total_atoms = natoms if strong else natoms * world
    line = {"metric": "atoms/sec for E+F+virial", "value": total_atoms * args.steps / res["t_dev"], "unit": "atoms/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * res["t_dev"] / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": config_of(w, world, strong), "clocks": res["clocks"], "gpu_launches": res["launches"],
            "e2e": {"value": total_atoms * args.steps / res["t_e2e"], "unit": "atoms/s",
                    "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"], "path": res["e2e_path"],
                    "timing": "CUDA events around each step, copies inside, L2 flushed between steps",
                    # the same call on the host clock, one device synchronisation per call, no L2 flush
                    "host_ms_per_call": res.get("host_ms_per_call"), "host_ms_per_call_eager": res.get("host_ms_per_call_eager")},
            "roofline": res["roofline"], "parts_ms": res.get("parts_ms"),
            "cuda_graph": bool(res["cuda_graph"]) if "cuda_graph" in res else None}
    if "schedule" in res:
        line["schedule"] = res["schedule"]
        if world > 1:     # how the exchanges of a step travel (kept out of `config`, which both arms share)
            line["transport"] = ("peer stores over NVLink by this library's kernels (NCCL for set-up only)" if res["schedule"].endswith("/peer")
                                 else "NCCL send/recv + all-reduce")
        if res.get("note"):
            line["note"] = res["note"]
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    ncores = len(os.sched_getaffinity(0))
    name, with_nep = resolve_workload(args.workload)
    w = make_workload(name)
    strong = w.get("kind") in ("train", "slab")

    if args.impl == "reference":
        # the reference's own CPU code on the host cores, same workload, config, metric and unit; rank 0 only
        if rank != 0:
            return
        cb = cpu_baseline(w, 60.0, ncores)
        line = {"impl": "reference", "metric": "atoms/sec for E+F+virial", "value": cb["value"], "unit": "atoms/s", "n_gpus": args.gpus,
                # the CPU arm times a bounded sample: `steps` is the number of E/F/V evaluations actually timed
                "steps": cb["calls_timed"], "steps_requested": args.steps, "warmup": 0, "ms_per_step": cb["ms_per_step"],
                "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": w["dtype"],
                "data": "synthetic", "config": config_of(w, max(world, args.gpus), strong),
                "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": cb["value"], "unit": "atoms/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        if with_nep:
            w2 = make_workload("nep")
            cb2 = cpu_baseline(w2, 30.0, ncores)
            line["nep"] = {"value": cb2["value"], "unit": "atoms/s", "ms_per_step": cb2["ms_per_step"], "dtype": w2["dtype"],
                           "config": config_of(w2, 1, False), "cpu_baseline": {k: cb2[k] for k in ("value", "unit", "cores", "kind", "sample")}}
        print(json.dumps(line))
        return

    # the peer-store exchange maps the neighbours' arrays with plain peer access; NVLink multicast objects are not used
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    line = gpu_line(w, args, world, dist, local)
    nep_line = None
    if with_nep:
        nep_line = gpu_line(make_workload("nep"), args, world, dist, local)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = {k: v for k, v in cpu_baseline(w, 20.0, ncores).items() if k in ("value", "unit", "cores", "kind", "sample")}
        if nep_line is not None:
            keep = ("value", "unit", "ms_per_step", "dtype", "config", "gpu_launches", "e2e", "roofline", "parts_ms", "cuda_graph", "clocks")
            line["nep"] = {k: nep_line[k] for k in keep}
            if world == 1 and not args.no_cpu_baseline:
                line["nep"]["cpu_baseline"] = {k: v for k, v in cpu_baseline(make_workload("nep"), 15.0, ncores).items()
                                               if k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
