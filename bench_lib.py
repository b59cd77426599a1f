"""Measurement harness of bench.py: timing loops, roofline arithmetic, clock sampling and the per-workload
benchmark drivers. Not part of the product package: it only calls the package's public API
(ai2pot_b200.engine.Evaluator, ai2pot_b200.slab, ai2pot_b200.capi) and a bench-only microbenchmark library."""
import ctypes as C
import json
import os
import re
import subprocess
import threading
import time

import numpy as np
import torch

from ai2pot_b200 import capi
from ai2pot_b200.engine import Evaluator

ROOT = os.path.dirname(os.path.abspath(__file__))
MEASURED_PEAKS = os.path.join(ROOT, "MEASURED_PEAKS.json")
FMA_PEAK_LIB = os.path.join(ROOT, "ai2pot_b200", "_lib", "libai2b_fma_peak.so")


# ---- algorithmic work per atom of the descriptor + force/virial path (FMA = 2) -----------------------------------
def flops_mtp(nn, n_basic, n_times, n_scalar, nmus, cs, kmax):
    R = 9 * cs + 20 + 4 * nmus * cs
    Pw = 4 * kmax + 4
    return nn * (R + Pw + 29 * n_basic) + 9 * n_times + 4 * n_scalar


def flops_nep(nn_r, nn_a, cs, n_r, n_a, neurons, n_desc):
    return (nn_r * (9 * cs + 20 + 4 * n_r * cs + 4 * n_r + 12) + nn_a * (9 * cs + 20 + 4 * n_a * cs + 384 + 22 * 24 * n_a)
            + 6 * 24 * n_a + 4 * neurons * n_desc + 20 * neurons)


def nblist_bytes(n, umax, elem):
    """Algorithmic bytes of one neighbour build: read positions + types, write the padded rows."""
    return n * (3 * elem + 4 + umax * (4 + 3 * elem) + 4)


def profiled_traffic(key):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of a kernel group, as recorded in the
    committed ncu summary that covers it: a line `dram_bytes_per_step(<key>) = <number>` in a file under profiles/.
    Returns (bytes or None, file name or None)."""
    pat = re.compile(r"dram_bytes_per_step\(" + re.escape(key) + r"\)\s*=\s*([0-9.eE+]+)")
    pdir = os.path.join(ROOT, "profiles")
    if os.path.isdir(pdir):
        for name in sorted(os.listdir(pdir)):
            if name.endswith((".md", ".txt")):
                m = pat.search(open(os.path.join(pdir, name)).read())
                if m:
                    return float(m.group(1)), "profiles/" + name
    return None, None


def hbm_peak():
    if os.path.exists(MEASURED_PEAKS):
        v = json.load(open(MEASURED_PEAKS)).get("hbm_gbs")
        if v:
            return float(v), "MEASURED_PEAKS.json (of measured)"
    return 6650.0, "6.65 TB/s (of fallback)"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        self.rows = []
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


_fma_lib = None


def fma_peak_tflops(is_f64, sms):
    """Measured FMA-pipe throughput of this GPU (microbenchmark in libai2b_fma_peak.so, best of 6)."""
    global _fma_lib
    if _fma_lib is None:
        _fma_lib = C.CDLL(FMA_PEAK_LIB)
    blocks, iters = sms * 16, 4096
    out = torch.empty(blocks * 256, dtype=torch.float64 if is_f64 else torch.float32, device="cuda")
    best = 0.0
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = _fma_lib.ai2b_bench_fma_chain(C.c_int(1 if is_f64 else 0), C.c_int(blocks), C.c_int(iters),
                                           C.c_void_p(out.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError("FMA microbenchmark failed to launch")
        e1.record()
        torch.cuda.synchronize()
        best = max(best, blocks * 256 * 8 * iters * 2 / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def timed(fn, steps, warmup, flush, barrier=None):
    """Sum of per-step device times (CUDA events on the current stream), L2 flushed between steps."""
    for _ in range(warmup):
        flush.zero_()
        fn()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
        torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    return sum(a.elapsed_time(b) for a, b in evs) * 1e-3


def host_timed(fn, calls, warmup=3):
    """Host wall clock of `calls` synchronous invocations (each ends with a device synchronisation): what a
    blocking caller sees, launch overhead of the Python / ctypes layer included. No L2 flush."""
    for _ in range(warmup):
        fn()
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(calls):
        fn()
        torch.cuda.synchronize()
    return (time.perf_counter() - t0) / calls


def ghost_images(cell, coords, types, rcut):
    """What an MD host holds for a periodic orthorhombic system: local atoms wrapped into the box plus the
    periodic images within rcut of it (ghosts), as double positions. Returns x_local, x_ghost, types_ghost, owner."""
    L = np.diag(np.asarray(cell, np.float64))
    x = np.mod(np.asarray(coords, np.float64), L)
    gx, gt, owner = [], [], []
    for sx in (-1, 0, 1):
        for sy in (-1, 0, 1):
            for sz in (-1, 0, 1):
                if sx == sy == sz == 0:
                    continue
                y = x + np.array([sx, sy, sz]) * L
                keep = np.all((y > -rcut) & (y < L + rcut), axis=1)
                gx.append(y[keep]); gt.append(np.asarray(types)[keep]); owner.append(np.nonzero(keep)[0])
    return x, np.concatenate(gx), np.concatenate(gt), np.concatenate(owner)


def run_md_benchmark(w, steps, warmup, dist, sampler):
    """Device-resident MD input path (ai2b_md_session_compute): host positions + types of local and ghost atoms
    in, host forces / energy / virial out. The call is synchronous and owns its stream, so a step is timed on
    the host clock around the call; there is no separate device-only number."""
    m = w["model"]
    x, gx, gt, owner = ghost_images(w["cell"], w["coords"], w["types"], w["rcut"])
    nlocal, nghost = len(x), len(gx)
    xa = np.ascontiguousarray(np.concatenate([x, gx])); ta = np.ascontiguousarray(np.concatenate([w["types"], gt]).astype(np.int32))
    ses = capi.MdSession(m, w["umax"])
    for _ in range(max(3, warmup)):
        e, f, v6, mx = ses.compute(nlocal, nghost, xa, ta)
    if dist is not None:
        dist.barrier()
    sampler.start()
    t0 = time.perf_counter()
    for _ in range(steps):
        e, f, v6, mx = ses.compute(nlocal, nghost, xa, ta)
    t = time.perf_counter() - t0
    clocks = sampler.stop()
    ses.close()
    props = torch.cuda.get_device_properties(torch.cuda.current_device())
    peak = fma_peak_tflops(False, props.multi_processor_count)
    roofline = {"kernel": "whole ai2b_md_session_compute call (H2D, neighbour build, nep_fast_kernel, D2H, host accumulation)", "bound": "fp32",
                "achieved": None, "peak": peak, "unit": "TFLOP/s", "frac": None, "traffic": None,
                "note": "host-timed synchronous call; the kernels are those of the nep workload", "max_neighbours": int(mx),
                "local_atoms": nlocal, "ghost_atoms": nghost}
    nall = nlocal + nghost
    return dict(t_dev=t, t_e2e=t, clocks=clocks, launches=(9 + 1) * steps, h2d=nall * 28, d2h=nall * 12 + 48, units=nlocal,
                e2e_path="host double positions + types of local and ghost atoms -> ai2b_md_session_compute -> host forces (+=), energy, virial[6]",
                roofline=roofline, parts_ms=None, host_ms_per_call=1e3 * t / steps)


def mtp_flops(m, mean_nn, training=False):
    tb = m["tables"]
    kmax = int(tb["alpha_index_basic"][:, 1:].sum(1).max())
    nb_, nt_, ns_ = len(tb["alpha_index_basic"]), len(tb["alpha_index_times"]), len(tb["alpha_moment_mapping"])
    fl = flops_mtp(mean_nn, nb_, nt_, ns_, tb["nmus"], m["chebyshev_size"], kmax)
    if training:   # F_train = F_MTP + nn (55 n_basic + R) + 18 n_times + 6 n_scalar
        R = 9 * m["chebyshev_size"] + 20 + 4 * tb["nmus"] * m["chebyshev_size"]
        fl += mean_nn * (55 * nb_ + R) + 18 * nt_ + 6 * ns_
    return fl


def training_batch_on_device(w, structs, dtype, dev):
    """Neighbour tensors of a list of structures, padded to the largest structure of the WHOLE batch, built on the
    device with one batched call (ai2b_nblist_build_batch). Returns the nb dict of device tensors."""
    npdt = np.float32 if dtype == torch.float32 else np.float64
    npad = max(len(s_["types"]) for s_ in w["structs"])
    B = len(structs)
    cells = np.stack([s_["cell"].astype(npdt) for s_ in structs]) if B else np.zeros((0, 3, 3), npdt)
    coords = np.zeros((B, npad, 3), npdt)
    types = np.zeros((B, npad), np.int32)
    binum = np.zeros(B, np.int32)
    for b, s_ in enumerate(structs):
        n = len(s_["types"])
        binum[b] = n
        coords[b, :n] = s_["coords"]
        types[b, :n] = s_["types"]
    nbt = capi.nblist_build_batch(cells, torch.from_numpy(binum).to(dev), torch.from_numpy(coords).to(dev), w["rcut"], w["umax"])
    if int(nbt["status"][1]):
        raise RuntimeError("umax too small for the training batch")
    nbt["btypes"] = torch.from_numpy(types).to(dev)
    nbt["ntypes"] = int(w["model"]["ntypes"])
    nbt["nghost"] = 0
    return nbt


def run_training_benchmark(w, steps, warmup, dist, sampler):
    """configs[3]: one step = forward E/F/V + loss + analytic gradient w.r.t. the model coefficients for
    this rank's share of the batch (structures dealt round-robin), then one all-reduce of the summed
    gradient when there is more than one rank. Neighbour tensors are built once (as the reference's
    dataset does at load time) and are resident."""
    rank = dist.get_rank() if dist is not None else 0
    world = dist.get_world_size() if dist is not None else 1
    model = w["model"]
    is_nep = model["kind"] == "nep"
    dtype = torch.float32 if w.get("dtype") == "f32" else torch.float64
    dev = torch.device("cuda", torch.cuda.current_device())
    structs = w["structs"][rank::world]
    prog = None if is_nep else capi.MtpProgram(model["tables"])
    md = capi.to_device({k: v for k, v in model.items() if k != "tables"}, dev, dtype)
    nbt = training_batch_on_device(w, structs, dtype, dev)
    npad = nbt["bilist"].shape[1]
    t = w["targets"]
    sel = slice(rank, None, world)
    E = torch.from_numpy(t["E"][sel]).to(dev, dtype); F = torch.from_numpy(np.ascontiguousarray(t["F"][sel, :npad])).to(dev, dtype)
    V = torch.from_numpy(np.ascontiguousarray(t["V"][sel])).to(dev, dtype)
    natoms = int(nbt["binum"].sum())
    mean_nn = float(nbt["bnumneigh"].sum()) / natoms
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    if is_nep:
        ngrad = sum(md[k].numel() for k in ("coeffs", "w0", "b0", "w1")) + int(model["ntypes"]) + 1
    else:
        ngrad = md["coeffs"].numel() + prog.ns + int(model["ntypes"]) + 1
    grad = torch.zeros(ngrad, dtype=dtype, device=dev)

    def compute():
        if is_nep:
            e, f, v = capi.nep_efv(md, nbt)
            loss, rmse = capi.nep_loss(nbt, w["weights"], e, E, f, F, v, V)
            parts = capi.nep_loss_backward(md, nbt, w["weights"], e, E, f, F, v, V)
        else:
            e, f, v = capi.mtp_efv(prog, md, nbt)
            loss, rmse = capi.mtp_loss(nbt, w["weights"], e, E, f, F, v, V)
            parts = capi.mtp_loss_backward(prog, md, nbt, w["weights"], e, E, f, F, v, V)
        capi.weighted_sum_rows(list(parts) + [loss.reshape(-1, 1)], None, out=grad)   # sums over the structures, one launch

    # the step's launches are the same every time (resident neighbour tensors, fixed shapes): replay them
    # from a CUDA graph; the all-reduce of the summed gradient stays an eager NCCL call
    graph = None
    if os.environ.get("AI2B_NO_GRAPH") != "1":
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    compute()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                compute()
        except Exception:
            graph = None
            torch.cuda.synchronize()

    def step():
        if graph is not None:
            graph.replay()
        else:
            compute()
        if dist is not None:
            dist.all_reduce(grad)
        return grad
    barrier = (lambda: dist.barrier()) if dist is not None else None
    sampler.start()
    t_dev = timed(step, steps, warmup, flush, barrier)
    clocks = sampler.stop()
    hgrad = torch.empty_like(grad, device="cpu").pin_memory()

    def e2e_step():
        step()
        hgrad.copy_(grad, non_blocking=True)
    t_e2e = timed(e2e_step, steps, warmup, flush, barrier)
    t_host = host_timed(e2e_step, max(3, min(steps, 20)))
    props = torch.cuda.get_device_properties(torch.cuda.current_device())
    peak = fma_peak_tflops(dtype == torch.float64, props.multi_processor_count)
    if is_nep:
        rc_all = nbt["brcs"]
        nn_a = float(((torch.linalg.norm(rc_all, dim=-1) <= model["rmax_angular"]) &
                      (torch.arange(rc_all.shape[2], device=dev)[None, None] < nbt["bnumneigh"][..., None])).sum()) / natoms
        # forward + directional-derivative pass + coefficient-gradient pass: three sweeps of the descriptor work
        fl = 3 * flops_nep(mean_nn, nn_a, model["chebyshev_size"], model["n_radial"], model["n_angular"], model["num_neurons"],
                           model["n_radial"] + model["n_angular"] * model["l_max"])
    else:
        fl = mtp_flops(model, mean_nn, training=True)
    achieved = natoms * fl / (t_dev / steps) / 1e12
    roofline = {"kernel": ("nep" if is_nep else "mtp") + " E/F/V + loss-gradient kernels (whole step)", "bound": "fp32" if dtype == torch.float32 else "fp64",
                "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": "FMA-chain microbenchmark in this run (of measured)",
                "flops_per_atom": fl, "mean_neighbours": mean_nn, "traffic": None}
    name = "nep" if is_nep else "mtp"
    return dict(t_dev=t_dev, t_e2e=t_e2e, clocks=clocks, launches=((2 + 2 + 1 + 1) if is_nep else (4 + 2 + 4 + 1)) * steps, h2d=0,
                d2h=hgrad.numel() * hgrad.element_size(), units=natoms,
                e2e_path=f"resident neighbour tensors -> ai2b_{name}_efv -> ai2b_{name}_loss -> ai2b_{name}_loss_backward -> D2H summed gradient",
                roofline=roofline, parts_ms=None, cuda_graph=graph is not None, host_ms_per_call=1e3 * t_host)


def run_slab_benchmark(w, steps, warmup, dist, sampler):
    """configs[4]: x-slab decomposition, halo exchange, ghost-force reduction (ai2pot_b200/slab.py).
    Strong scaling: the system is fixed, each rank owns 1/N of it."""
    from ai2pot_b200 import slab
    rank = dist.get_rank() if dist is not None else 0
    world = dist.get_world_size() if dist is not None else 1
    dtype = torch.float32 if w["dtype"] == "f32" else torch.float64
    dev = torch.device("cuda", torch.cuda.current_device())
    schedule = os.environ.get("AI2B_SLAB_SCHEDULE", "serial")     # the fastest of the three on B200 at 2, 4 and 8 ranks
    # neighbour exchanges by this library's peer-store kernels unless told otherwise; NCCL carries the set-up
    transport = os.environ.get("AI2B_SLAB_TRANSPORT", "peer")
    note = None
    try:
        dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, dev, dist,
                              halo_cutoffs=2 if (schedule == "owner" and world > 1) else 1, transport=transport)
    except (RuntimeError, ImportError, AttributeError) as exc:
        if transport != "peer":
            raise
        note = f"symmetric memory unavailable ({type(exc).__name__}): NCCL transport"
        dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, dev, dist,
                              halo_cutoffs=2 if (schedule == "owner" and world > 1) else 1, transport="nccl")
    def make_step(d):
        return slab.SlabStep(d, w["model"], w["umax"], dtype, schedule=schedule, tail_fraction=float(os.environ.get("AI2B_SLAB_TAIL", "0.25")))

    step_obj = make_step(dom)
    # First step. A peer exchange that gave up on one rank (bounded waits: the kernels return, the status says where) must not
    # leave the other ranks waiting in the next barrier: the ranks agree on the outcome and, if need be, all change to NCCL.
    ok = 1
    if dist is not None:
        dist.barrier()      # the ranks enter their first exchange together (the waits are bounded to a few seconds)
    try:
        e, f, v = step_obj.evaluate()
        torch.cuda.synchronize()
        step_obj.check_status()
    except RuntimeError as exc:
        if dom.transport != "peer" or dist is None:
            raise
        ok = 0
        note = f"peer exchange failed on rank {rank} ({exc}): NCCL transport"
    if dist is not None and dom.transport == "peer":
        agreed = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            note = note or "peer exchange failed on another rank: NCCL transport"
            dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, dev, dist,
                                  halo_cutoffs=2 if (schedule == "owner" and world > 1) else 1, transport="nccl")
            step_obj = make_step(dom)
            e, f, v = step_obj.evaluate()
            torch.cuda.synchronize()
            step_obj.check_status()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    barrier = (lambda: dist.barrier()) if dist is not None else None
    sampler.start()
    t_dev = timed(step_obj.evaluate, steps, warmup, flush, barrier)
    clocks = sampler.stop()
    host_owned = dom.owned.cpu().pin_memory()
    h_f = torch.empty(dom.nlocal, 3, dtype=dtype).pin_memory()
    h_ev = torch.empty(10, dtype=dtype).pin_memory()


    def e2e_step():
        dom.owned.copy_(host_owned, non_blocking=True)
        e_, f_, v_ = step_obj.evaluate()
        h_f.copy_(f_, non_blocking=True)
        h_ev[:1].copy_(e_.reshape(1), non_blocking=True); h_ev[1:].copy_(v_, non_blocking=True)
    t_e2e = timed(e2e_step, steps, warmup, flush, barrier)
    t_host = host_timed(e2e_step, max(3, min(steps, 20)))
    k = max(3, min(steps, 5))
    parts = step_obj.parts_ms(k, flush, timed)
    m = w["model"]
    props = torch.cuda.get_device_properties(torch.cuda.current_device())
    peak = fma_peak_tflops(dtype == torch.float64, props.multi_processor_count)
    mean_nn, nn_a = step_obj.neighbour_stats()
    fl = flops_nep(mean_nn, nn_a, m["chebyshev_size"], m["n_radial"], m["n_angular"], m["num_neurons"], m["n_radial"] + m["n_angular"] * m["l_max"])
    t_comp = parts["nblist+efv"] * 1e-3
    achieved = dom.nlocal * fl / t_comp / 1e12
    elem = 4 if dtype == torch.float32 else 8
    hbm, hbm_src = hbm_peak()
    roofline = {"kernel": "nep_fast_kernel (+ neighbour build) on this rank's slab", "bound": "fp32", "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": "FMA-chain microbenchmark in this run (of measured)",
                "flops_per_atom": fl, "mean_neighbours": mean_nn, "traffic": None, "owned_atoms": dom.nlocal, "ghost_atoms": dom.nghost,
                "halo_bytes_per_step": step_obj.halo_bytes(), "ghost_force_bytes_per_step": step_obj.return_bytes(),
                "allreduce_bytes_per_step": 10 * elem if world > 1 else 0}
    return dict(t_dev=t_dev, t_e2e=t_e2e, clocks=clocks, launches=step_obj.launches_per_step() * steps,
                h2d=host_owned.numel() * host_owned.element_size(),
                d2h=h_f.numel() * h_f.element_size() + 10 * elem, units=len(w["types"]) / world,
                e2e_path="pinned host positions of the slab -> H2D -> halo exchange -> ai2b_nblist_build_range -> ai2b_nep_efv_accumulate "
                         "-> ghost-force return + reduction of E, virial -> D2H forces, E, virial",
                roofline=roofline, parts_ms=parts, host_ms_per_call=1e3 * t_host, schedule=step_obj.schedule + "/" + dom.transport, note=note)


def run_single_benchmark(w, steps, warmup, dist, sampler):
    dtype = torch.float64 if w["dtype"] == "f64" else torch.float32
    ev = Evaluator(w["model"], w["cell"], w["types"], w["rcut"], w["umax"], dtype)
    n = ev.n
    host_coords = torch.from_numpy(np.ascontiguousarray(w["coords"])).to(dtype).pin_memory()
    coords = host_coords.cuda()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    barrier = (lambda: dist.barrier()) if dist is not None else None
    props = torch.cuda.get_device_properties(torch.cuda.current_device())

    # device-resident throughput: positions already in HBM
    nb = ev.build_list(coords)
    ev.evaluate(nb)
    torch.cuda.synchronize()
    st = ev.status.cpu().numpy()
    if st[1]:
        raise RuntimeError(f"umax {ev.umax} too small (max {st[0]})")
    mean_nn = float(nb["bnumneigh"].float().mean())
    # the step is a fixed sequence of launches on fixed buffers: replayed from a CUDA graph when the capture succeeds
    graphed = ev.capture(coords)
    step = ev.replay if graphed else (lambda: ev.compute(coords))
    sampler.start()
    t_dev = timed(step, steps, warmup, flush, barrier)
    clocks = sampler.stop()

    # end to end: host positions in, host E/F/V out, every step
    h_e = torch.empty(1, dtype=dtype).pin_memory()
    h_f = torch.empty(1, n, 3, dtype=dtype).pin_memory()
    h_v = torch.empty(1, 9, dtype=dtype).pin_memory()
    dcoords = torch.empty_like(coords)

    # with a graph: the two copies are nodes of the same graph as the kernels (one launch per call, one D2H copy of the
    # evaluator's output buffer [E | virial | forces])
    h_all = torch.empty(ev.outbuf.numel(), dtype=dtype).pin_memory()
    graphed_io = graphed and ev.capture_io(coords, host_coords, h_all)

    def e2e_step():
        if graphed_io:
            ev.replay_io()
            return
        if graphed:
            coords.copy_(host_coords, non_blocking=True)
            e, f, v = ev.replay()
        else:
            dcoords.copy_(host_coords, non_blocking=True)
            e, f, v = ev.compute(dcoords)
        h_e.copy_(e, non_blocking=True); h_f.copy_(f, non_blocking=True); h_v.copy_(v, non_blocking=True)
    t_e2e = timed(e2e_step, steps, warmup, flush, barrier)
    # the same call as a blocking caller sees it: host clock, a synchronisation per call, no L2 flush
    t_host = host_timed(e2e_step, max(3, min(steps, 50)))

    def eager_call():
        dcoords.copy_(host_coords, non_blocking=True)
        e, f, v = ev.compute(dcoords)
        h_e.copy_(e, non_blocking=True); h_f.copy_(f, non_blocking=True); h_v.copy_(v, non_blocking=True)
    t_host_eager = host_timed(eager_call, max(3, min(steps, 50)))
    h2d = host_coords.numel() * host_coords.element_size()
    d2h = h_all.numel() * h_all.element_size() if graphed_io else sum(t.numel() * t.element_size() for t in (h_e, h_f, h_v))

    # the two parts separately (same timing rules), for the roofline of the dominant kernel
    k = max(3, min(steps, 10))
    t_nb = timed(lambda: ev.build_list(coords), k, 3, flush) / k
    t_ev = timed(lambda: ev.evaluate(nb), k, 3, flush) / k

    m = w["model"]
    if m["kind"] == "mtp":
        fl = mtp_flops(m, mean_nn)
        bound = "fp64"
    else:
        nn_a = float((torch.linalg.norm(nb["brcs"][0], dim=-1) <= m["rmax_angular"]).logical_and(
            torch.arange(ev.umax, device="cuda")[None] < nb["bnumneigh"][0][:, None]).sum(1).float().mean())
        fl = flops_nep(mean_nn, nn_a, m["chebyshev_size"], m["n_radial"], m["n_angular"], m["num_neurons"],
                       m["n_radial"] + m["n_angular"] * m["l_max"])
        bound = "fp32"
    is64 = dtype == torch.float64
    peak_meas = fma_peak_tflops(is64, props.multi_processor_count)
    sm_max = clocks.get("sm_max_mhz") or 1965.0
    peak_nom = props.multi_processor_count * (64 if is64 else 128) * 2 * sm_max * 1e6 / 1e12
    achieved = n * fl / t_ev / 1e12
    nb_bytes = nblist_bytes(n, ev.umax, 8 if is64 else 4)
    hbm, hbm_src = hbm_peak()
    key = ("mtp16" if m["kind"] == "mtp" else "nep") + f"_{n}_efv"
    traffic, traffic_src = profiled_traffic(key)
    roofline = {"kernel": "mtp_fwd_atoms + mtp_contract_seg + mtp_force_atoms (the three E/F/V kernels of a call)" if m["kind"] == "mtp" else "nep_fast_kernel",
                "bound": bound,
                "achieved": achieved, "peak": peak_meas, "unit": "TFLOP/s", "frac": achieved / peak_meas,
                "peak_source": "FMA-chain microbenchmark in this run (of measured)", "peak_nominal": peak_nom,
                "frac_of_nominal": achieved / peak_nom, "flops_per_atom": fl, "mean_neighbours": mean_nn,
                "traffic": traffic, "traffic_source": traffic_src, "kernel_ms": 1e3 * t_ev,
                "nblist": {"bound": "hbm", "achieved": nb_bytes / t_nb / 1e9, "peak": hbm, "unit": "GB/s",
                           "frac": nb_bytes / t_nb / 1e9 / hbm, "peak_source": hbm_src,
                           "bytes_per_atom": nb_bytes / n, "ms": 1e3 * t_nb}}
    return dict(t_dev=t_dev, t_e2e=t_e2e, clocks=clocks, launches=ev.launches_per_step() * steps, h2d=h2d, d2h=d2h,
                e2e_path="pinned host positions -> H2D -> ai2b_nblist_build -> ai2b_*_efv -> D2H E,F,V (C ABI via ctypes" +
                         (", both copies and all launches replayed as one CUDA graph)" if graphed_io else ", replayed from a CUDA graph)" if graphed else ")"),
                cuda_graph=graphed,
                roofline=roofline, parts_ms={"nblist": 1e3 * t_nb, "efv": 1e3 * t_ev},
                host_ms_per_call=1e3 * t_host, host_ms_per_call_eager=1e3 * t_host_eager)


def run_benchmark(w, steps, warmup, dist, sampler):
    if w.get("kind") == "md":
        return run_md_benchmark(w, steps, warmup, dist, sampler)
    if w.get("kind") == "train":
        return run_training_benchmark(w, steps, warmup, dist, sampler)
    if w.get("kind") == "slab":
        return run_slab_benchmark(w, steps, warmup, dist, sampler)
    return run_single_benchmark(w, steps, warmup, dist, sampler)
