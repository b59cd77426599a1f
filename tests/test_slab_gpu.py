"""Slab decomposition on real GPUs (NCCL): two ranks must reproduce the single-GPU forces, energy
and virial of the same system, for every schedule of a step (serial, overlapped split-centre passes, wide halo
without force return) and through the one-pass interface. Skipped on a single-GPU box. Ranks are child
processes; each leaves only after a barrier, with nothing in flight. NVLS is switched off for these ranks."""
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
NCELL = 12            # 72 A: two slabs of 36 A


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
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from ai2pot_b200 import slab, synth
    w = synth.g4(ncell=NCELL)
    dev = torch.device("cuda", rank)
    out = {}
    dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, dev, dist)
    comp = slab.LocalCompute(w["model"], w["cell"], w["rcut"], w["umax"], torch.float32)
    e, f, v = dom.evaluate(comp)
    e2, f2, v2 = dom.evaluate(comp)          # a second step reuses every buffer
    torch.cuda.synchronize()
    assert torch.allclose(f, f2, rtol=0, atol=1e-5 * float(f.abs().max()))
    out.update(e_onepass=e.cpu().numpy(), f_onepass=f.cpu().numpy(), v_onepass=v.cpu().numpy(), idx_onepass=dom.global_index)
    for schedule in ("serial", "overlap", "owner"):
        d = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, dev, dist, halo_cutoffs=2 if schedule == "owner" else 1)
        step = slab.SlabStep(d, w["model"], w["umax"], torch.float32, schedule=schedule)
        for _ in range(3):                    # first call runs eagerly and records the graphs, the next ones replay them
            e, f, v = step.evaluate()
        torch.cuda.synchronize()
        step.check_status()
        out.update({"e_" + schedule: e.cpu().numpy(), "f_" + schedule: f.cpu().numpy(), "v_" + schedule: v.cpu().numpy(),
                    "idx_" + schedule: d.global_index, "graphs_" + schedule: len(step._graphs)})
        assert d.nghost > 0 and 0 < d.n_interior < d.nlocal
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), **out)
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_slabs_match_one_gpu(tmp_path):
    sys.path.insert(0, ROOT)
    from ai2pot_b200 import slab, synth
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    w = synth.g4(ncell=NCELL)
    torch.cuda.set_device(0)
    dom = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], 0, 1, torch.device("cuda", 0))
    step = slab.SlabStep(dom, w["model"], w["umax"], torch.float32)
    step.evaluate()
    e1, f1, v1 = [t.cpu().numpy() for t in step.evaluate()]
    F1 = np.zeros_like(f1)
    F1[dom.global_index] = f1
    z = [np.load(tmp_path / f"r{r}.npz") for r in range(2)]
    for tag in ("onepass", "serial", "overlap", "owner"):
        F = np.zeros_like(f1)
        for r in range(2):
            F[z[r]["idx_" + tag]] = z[r]["f_" + tag]
            assert abs(z[r]["e_" + tag] - e1) <= 2e-5 * abs(e1), tag
            assert np.abs(z[r]["v_" + tag] - v1).max() <= 2e-5 * np.abs(v1).max(), tag
        assert np.abs(F - F1).max() <= 2e-5 * np.abs(F1).max(), tag
    assert z[0]["graphs_overlap"] == 3 and z[0]["graphs_owner"] == 2 and z[0]["graphs_serial"] == 1
