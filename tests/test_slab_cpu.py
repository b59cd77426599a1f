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
