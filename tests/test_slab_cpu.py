"""Slab decomposition logic on CPU ranks (gloo): partition, halo exchange with periodic shifts,
ghost-force reduction and the scalar all-reduce, with the CPU checker standing in for the CUDA
kernels. The decomposed result must equal the single-domain result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _system(dtype):
    from ai2pot_b200 import synth
    w = synth.g4(ncell=5, dtype=dtype)       # 500 atoms, L = 30 A: slabs of 15 / 10 A at 2 / 3 ranks
    return w


def _oracle_compute(chk, model, cell, rcut, umax):
    from ai2pot_b200 import synth

    def compute(local, types, nlocal, pbc):
        pos = local.numpy()
        ty = types.numpy()
        nn, fn, rc, _, mx = chk.nblist(cell, ty, pos, rcut, umax, pbc=[int(p) for p in pbc])
        nb = dict(binum=np.array([nlocal], np.int32), bilist=np.arange(nlocal, dtype=np.int32)[None], bnumneigh=nn[None, :nlocal],
                  bfirstneigh=fn[None, :nlocal], brcs=rc[None, :nlocal], btypes=ty[None], ntypes=model["ntypes"], nghost=len(ty) - nlocal)
        e, f, v = chk.nep_efv(model, nb)
        return torch.from_numpy(e), torch.from_numpy(f[0]), torch.from_numpy(v[0])
    return compute


class _OraclePasses:
    """CPU stand-in for slab.CudaPasses: rows of a range of centres from the CPU checker's neighbour list over the
    first `ncand` atoms, NEP E/F/V of those centres added onto the accumulators."""

    def __init__(self, chk, model, cell, rcut, umax):
        self.chk, self.model, self.cell, self.rcut, self.umax = chk, model, cell, rcut, umax
        self.calls = []

    def run_pass(self, name, local, types, c0, c1, ncand, pbc, acc, reuse_bins=False):
        self.calls.append((name, c0, c1, ncand, reuse_bins))
        if c1 <= c0:
            return
        pos = local[:ncand].numpy()
        ty = types.numpy()
        nn, fn, rc, _, mx = self.chk.nblist(self.cell, ty[:ncand], pos, self.rcut, self.umax, pbc=[int(p) for p in pbc])
        nc = c1 - c0
        ntotal = local.shape[0]
        nb = dict(binum=np.array([nc], np.int32), bilist=np.arange(c0, c1, dtype=np.int32)[None], bnumneigh=nn[None, c0:c1],
                  bfirstneigh=fn[None, c0:c1], brcs=rc[None, c0:c1], btypes=ty[None], ntypes=self.model["ntypes"], nghost=ntotal - nc)
        e, f, v = self.chk.nep_efv(self.model, nb)
        acc[0].add_(torch.from_numpy(e)); acc[1].add_(torch.from_numpy(f[0])); acc[2].add_(torch.from_numpy(v[0]))

    def statuses(self):
        return []


def _step_worker(rank, world, port, schedule, ncell, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import refapi
    from ai2pot_b200 import slab, synth
    w = synth.g4(ncell=ncell, dtype=np.float64)
    model = {k: (v.astype(np.float64) if isinstance(v, np.ndarray) else v) for k, v in w["model"].items()}
    chk = refapi.Checker("oracle")
    dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, torch.device("cpu"), dist, skin=0.2,
                          halo_cutoffs=2 if schedule == "owner" else 1)
    passes = _OraclePasses(chk, model, w["cell"], w["rcut"], 64)
    step = slab.SlabStep(dom, schedule=schedule, passes=passes, tail_fraction=0.4)
    e, f, v = step.evaluate()
    e, f, v = [t.clone() for t in step.evaluate()]   # a second step starts from zeroed accumulators (results are views of them)
    step.check_status()
    # atoms move by less than half the skin: the same domain still gives the moved system's answer
    rng = np.random.default_rng(100)
    shift = rng.normal(0, 0.02, w["coords"].shape)
    dom.owned.add_(torch.from_numpy(shift[dom.global_index]))
    e2, f2, v2 = step.evaluate()
    step.check_status()
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), e=e.numpy(), f=f.numpy(), v=v.numpy(), e2=e2.numpy(), f2=f2.numpy(), v2=v2.numpy(),
             idx=dom.global_index, nghost=dom.nghost, n_interior=dom.n_interior, names=np.array([c[0] for c in passes.calls]))
    dom.owned.add_(1.0)                            # far beyond the skin: must be refused
    try:
        step.check_status()
        moved_ok = 0
    except RuntimeError:
        moved_ok = 1
    assert moved_ok
    dist.barrier()
    dist.destroy_process_group()


# cells of 6 A: 5 cells / 2 ranks = 15 A slabs; 7 cells / 3 ranks = 14 A (the wide halo needs >= 2 cutoffs + skin);
# 5 cells / 3 ranks = 10 A slabs have no interior atom at all (every centre can see a ghost)
@pytest.mark.parametrize("world,schedule,ncell", [(2, "overlap", 5), (3, "overlap", 7), (3, "overlap", 5), (2, "serial", 5),
                                                  (2, "owner", 5), (3, "owner", 7)])
def test_step_schedules_match_single_domain(tmp_path, world, schedule, ncell):
    """SlabStep's schedules (split centres, wide halo without force return) against the single-domain result, before
    and after a displacement within the skin."""
    from oracle import refapi
    from ai2pot_b200 import synth
    if not refapi.available("oracle"):
        pytest.skip("oracle library not built")
    mp.spawn(_step_worker, args=(world, _free_port(), schedule, ncell, str(tmp_path)), nprocs=world, join=True)
    w = synth.g4(ncell=ncell, dtype=np.float64)
    model = {k: (v.astype(np.float64) if isinstance(v, np.ndarray) else v) for k, v in w["model"].items()}
    chk = refapi.Checker("oracle")
    rng = np.random.default_rng(100)
    shift = rng.normal(0, 0.02, w["coords"].shape)
    for tag, coords in (("", w["coords"]), ("2", w["coords"] + shift)):
        nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], coords, w["rcut"], 64)
        er, fr, vr = chk.nep_efv(model, synth.batch_from_nblist(nn, fn, rc, ty, 3))
        F = np.zeros_like(fr[0])
        seen = np.zeros(len(F), bool)
        for r in range(world):
            z = np.load(tmp_path / f"r{r}.npz")
            assert z["nghost"] > 0 and z["n_interior"] < len(z["idx"])
            assert (z["n_interior"] > 0) == (not (world == 3 and ncell == 5))
            assert not seen[z["idx"]].any()
            seen[z["idx"]] = True
            F[z["idx"]] = z["f" + tag]
            assert abs(z["e" + tag] - er[0]) <= 1e-11 * abs(er[0])
            assert np.abs(z["v" + tag] - vr[0]).max() <= 1e-11 * np.abs(vr).max()
            names = set(z["names"].tolist())
            assert names == {"overlap": {"head", "boundary", "tail"}, "serial": {"all"}, "owner": {"head", "boundary", "ghost-centres"}}[schedule]
        assert seen.all()
        assert np.abs(F - fr[0]).max() <= 1e-11 * np.abs(fr).max()


def _worker(rank, world, port, dtype_name, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import refapi
    from ai2pot_b200 import slab
    dtype = np.float64 if dtype_name == "f64" else np.float32
    w = _system(dtype)
    model = {k: (v.astype(dtype) if isinstance(v, np.ndarray) else v) for k, v in w["model"].items()}
    chk = refapi.Checker("oracle")
    dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, torch.device("cpu"), dist)
    e, f, v = dom.evaluate(_oracle_compute(chk, model, w["cell"], w["rcut"], 64))
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), e=e.numpy(), f=f.numpy(), v=v.numpy(), idx=dom.global_index, nghost=dom.nghost)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,dtype_name", [(2, "f64"), (3, "f64"), (2, "f32")])
def test_slabs_match_single_domain(tmp_path, world, dtype_name):
    from oracle import refapi
    from ai2pot_b200 import synth
    if not refapi.available("oracle"):
        pytest.skip("oracle library not built")
    mp.spawn(_worker, args=(world, _free_port(), dtype_name, str(tmp_path)), nprocs=world, join=True)
    dtype = np.float64 if dtype_name == "f64" else np.float32
    w = _system(dtype)
    model = {k: (v.astype(dtype) if isinstance(v, np.ndarray) else v) for k, v in w["model"].items()}
    chk = refapi.Checker("oracle")
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], w["rcut"], 64)
    er, fr, vr = chk.nep_efv(model, synth.batch_from_nblist(nn, fn, rc, ty, 3))
    tol = 1e-11 if dtype_name == "f64" else 2e-5
    F = np.zeros_like(fr[0])
    seen = np.zeros(len(F), bool)
    for r in range(world):
        z = np.load(tmp_path / f"r{r}.npz")
        assert z["nghost"] > 0
        assert not seen[z["idx"]].any()
        seen[z["idx"]] = True
        F[z["idx"]] = z["f"]
        assert abs(z["e"] - er[0]) <= tol * abs(er[0])                     # every rank holds the reduced energy
        assert np.abs(z["v"] - vr[0]).max() <= tol * np.abs(vr).max()
    assert seen.all()
    assert np.abs(F - fr[0]).max() <= tol * np.abs(fr).max()


def test_partition_and_single_rank():
    from ai2pot_b200 import slab
    w = _system(np.float64)
    owner, fx, wrap = slab.partition(w["cell"], w["coords"], 4)
    assert owner.min() == 0 and owner.max() == 3 and np.all((fx >= 0) & (fx < 1))
    dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], 0, 1, torch.device("cpu"))
    assert dom.nghost == 0 and dom.nlocal == len(w["types"]) and dom.pbc == (True, True, True)
    with pytest.raises(ValueError):
        slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], 0, 8, torch.device("cpu"))
