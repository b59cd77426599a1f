"""Slab decomposition on real GPUs (NCCL): two ranks must reproduce the single-GPU forces, energy
and virial of the same system. Skipped on a single-GPU box. Ranks are child processes; each leaves
only after a barrier, with nothing in flight."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from ai2pot_b200 import slab, synth
    w = synth.g4(ncell=12)
    dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, torch.device("cuda", rank), dist)
    comp = slab.LocalCompute(w["model"], w["cell"], w["rcut"], w["umax"], torch.float32)
    e, f, v = dom.evaluate(comp)
    e2, f2, v2 = dom.evaluate(comp)          # a second step reuses every buffer
    torch.cuda.synchronize()
    assert torch.allclose(f, f2, rtol=0, atol=1e-5 * float(f.abs().max()))
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), e=e.cpu().numpy(), f=f.cpu().numpy(), v=v.cpu().numpy(), idx=dom.global_index,
             nghost=dom.nghost)
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_slabs_match_one_gpu(tmp_path):
    sys.path.insert(0, ROOT)
    from ai2pot_b200 import slab, synth
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    w = synth.g4(ncell=12)
    torch.cuda.set_device(0)
    dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], 0, 1, torch.device("cuda", 0))
    comp = slab.LocalCompute(w["model"], w["cell"], w["rcut"], w["umax"], torch.float32)
    e1, f1, v1 = [t.cpu().numpy() for t in dom.evaluate(comp)]
    F = np.zeros_like(f1)
    for r in range(2):
        z = np.load(tmp_path / f"r{r}.npz")
        assert z["nghost"] > 0
        F[z["idx"]] = z["f"]
        assert abs(z["e"] - e1) <= 2e-5 * abs(e1)
        assert np.abs(z["v"] - v1).max() <= 2e-5 * np.abs(v1).max()
    F1 = np.zeros_like(f1)
    F1[dom.global_index] = f1
    assert np.abs(F - F1).max() <= 2e-5 * np.abs(F1).max()
