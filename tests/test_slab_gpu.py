"""Slab decomposition on real GPUs (NCCL): two ranks must reproduce the single-GPU forces, energy
and virial of the same system, for every schedule of a step (serial, overlapped split-centre passes, wide halo
without force return), with NCCL and with this library's own peer-store exchange, and through the one-pass interface. Skipped on a single-GPU box. Ranks are child
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
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
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
    for tag in ("serial", "overlap", "owner", "serial_peer", "overlap_peer", "owner_peer"):
        schedule, transport = (tag[:-5], "peer") if tag.endswith("_peer") else (tag, "nccl")
        d = slab.SlabDomain(w["cell"], w["coords"], w["types"], w["rcut"], rank, world, dev, dist, halo_cutoffs=2 if schedule == "owner" else 1,
                            transport=transport)
        step = slab.SlabStep(d, w["model"], w["umax"], torch.float32, schedule=schedule)
        for _ in range(3):                    # first call runs eagerly and records the graphs, the next ones replay them
            e, f, v = step.evaluate()
        torch.cuda.synchronize()
        step.check_status()
        out.update({"e_" + tag: e.cpu().numpy(), "f_" + tag: f.cpu().numpy(), "v_" + tag: v.cpu().numpy(),
                    "idx_" + tag: d.global_index, "graphs_" + tag: len(step._graphs)})
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
    for tag in ("onepass", "serial", "overlap", "owner", "serial_peer", "overlap_peer", "owner_peer"):
        F = np.zeros_like(f1)
        for r in range(2):
            F[z[r]["idx_" + tag]] = z[r]["f_" + tag]
            assert abs(z[r]["e_" + tag] - e1) <= 2e-5 * abs(e1), tag
            assert np.abs(z[r]["v_" + tag] - v1).max() <= 2e-5 * np.abs(v1).max(), tag
        assert np.abs(F - F1).max() <= 2e-5 * np.abs(F1).max(), tag
    assert z[0]["graphs_overlap"] == 3 and z[0]["graphs_owner"] == 2 and z[0]["graphs_serial"] == 1


def test_peer_wait_gives_up():
    """The bounded device-side wait: a flag that nothing sets makes ai2b_peer_wait run out of polls, record that in
    its status word and return; a flag that is already at the value passes at once. The context stays usable."""
    from ai2pot_b200 import capi
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.peer_wait(flag, 0, status, max_polls=1000)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    capi.peer_wait(flag, 1, status, max_polls=1000)      # nothing ever writes 1: ~0.2 ms of polling, then gives up
    torch.cuda.synchronize()
    assert int(status[0]) == 1
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_peer_push_rows_on_one_device():
    """ai2b_peer_push_rows with a "neighbour" buffer on the same device: gather, shift, scatter and the flag."""
    from ai2pot_b200 import capi
    rng = np.random.default_rng(2)
    for dt in (torch.float32, torch.float64):
        src = torch.from_numpy(rng.normal(size=(500, 3))).to(dt).cuda()
        sidx = torch.from_numpy(rng.permutation(500)[:300].astype(np.int32)).cuda()
        didx = torch.from_numpy((rng.permutation(400)[:300] + 50).astype(np.int32)).cuda()
        dst = torch.zeros(450, 3, dtype=dt, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        shift = np.array([1.5, -2.0, 0.25])
        for epoch in (1, 2):                                  # the counter resets itself between pushes
            capi.peer_push_rows(src, sidx, didx, 300, shift, dst, flag, epoch, counter)
            capi.peer_wait(flag, epoch, status, max_polls=1000000)
        torch.cuda.synchronize()
        assert int(flag[0]) == 2 and int(status[0]) == 0 and int(counter[0]) == 0
        exp = torch.zeros_like(dst)
        exp[didx.long()] = src[sidx.long()] + torch.tensor(shift, dtype=dt, device="cuda")
        assert torch.equal(dst, exp)
        capi.peer_push_rows(src[100:], None, None, 20, None, dst, flag, 3, counter)    # contiguous rows, no shift
        torch.cuda.synchronize()
        assert torch.equal(dst[:20], src[100:120])


def test_peer_exchange_on_one_device():
    """ai2b_peer_exchange with both "neighbours" on the same device: two pushes, both flags raised, and the wait on
    them inside the same launch; a second launch whose incoming flags nobody raises gives up and reports it."""
    from ai2pot_b200 import capi
    rng = np.random.default_rng(4)
    dt = torch.float32
    src = torch.from_numpy(rng.normal(size=(300, 3))).to(dt).cuda()
    il = torch.arange(0, 100, dtype=torch.int32, device="cuda")
    ir = torch.arange(200, 300, dtype=torch.int32, device="cuda")
    dl = torch.arange(10, 110, dtype=torch.int32, device="cuda")
    dst_l = torch.zeros(120, 3, dtype=dt, device="cuda")
    dst_r = torch.zeros(120, 3, dtype=dt, device="cuda")
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    left = dict(src=src, src_idx=il, dst_idx=dl, n=100, shift=np.array([3.0, 0.0, 0.0]), dst=dst_l, flag=flags[0:1])
    right = dict(src=src, src_idx=ir, dst_idx=None, n=100, shift=None, dst=dst_r, flag=flags[1:2])
    capi.peer_exchange(left, right, 1, flags[0:1], flags[1:2], status, counter)
    torch.cuda.synchronize()
    assert flags[:2].tolist() == [1, 1] and int(status[0]) == 0 and int(counter[0]) == 0
    assert torch.equal(dst_l[10:110], src[:100] + torch.tensor([3.0, 0.0, 0.0], device="cuda")) and torch.equal(dst_r[:100], src[200:300])
    capi.peer_exchange(left, right, 2, flags[2:3], flags[3:4], status, counter, max_polls=2000)   # flags 2, 3 stay 0
    torch.cuda.synchronize()
    assert int(status[0]) == 1 and flags[:2].tolist() == [2, 2]


def test_peer_return_reduce_on_one_device():
    """ai2b_peer_return_reduce with this device as its own neighbour and a world of two table rows (the second row is
    filled by hand, as the other rank would): force rows pushed into `back`, added onto the owned atoms by index
    (an atom listed twice receives both rows), partial sums reduced in rank order."""
    from ai2pot_b200 import capi
    rng = np.random.default_rng(6)
    for dt in (torch.float32, torch.float64):
        ntotal, nl, nr = 400, 60, 50
        force = torch.from_numpy(rng.normal(size=(ntotal, 3))).to(dt).cuda()
        f0 = force.clone()
        back = torch.zeros(nl + nr, 3, dtype=dt, device="cuda")
        idx = torch.from_numpy(rng.integers(0, 200, nl + nr).astype(np.int32)).cuda()
        idx[1] = idx[0]                                        # the same atom twice
        flags = torch.zeros(8 + 2, dtype=torch.int32, device="cuda")
        table = torch.zeros(2 * 16, dtype=dt, device="cuda")
        other = torch.from_numpy(rng.normal(size=10)).to(dt).cuda()
        table[16:26] = other
        flags[9] = 5                                           # "rank 1" has published for step 5
        partial = torch.from_numpy(rng.normal(size=10)).to(dt).cuda()
        reduced = torch.zeros(10, dtype=dt, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        ptrs = torch.tensor([table.data_ptr(), table.data_ptr()], dtype=torch.int64, device="cuda")          # both "ranks" map to this table;
        fptrs = torch.tensor([flags[8:].data_ptr(), flags[8:].data_ptr()], dtype=torch.int64, device="cuda")  # rank 0's writes land in row 0 twice
        left = dict(src=force[300:300 + nl], n=nl, dst=back, flag=flags[2:3])
        right = dict(src=force[340:340 + nr], n=nr, dst=back[nl:], flag=flags[3:4])
        capi.peer_return_reduce(left, right, 5, flags[2:3], flags[3:4], back, idx, force, partial, ptrs, fptrs, table, flags[8:], reduced, 0, 2,
                                status, counter)
        torch.cuda.synchronize()
        assert int(status[0]) == 0 and int(counter[0]) == 0 and flags[2:4].tolist() == [5, 5] and int(flags[8]) == 5
        exp = f0.clone()
        src_rows = torch.cat([f0[300:300 + nl], f0[340:340 + nr]])
        exp.index_add_(0, idx.long(), src_rows)
        tol = 1e-6 if dt == torch.float32 else 1e-14
        assert float((force - exp).abs().max()) <= tol * float(exp.abs().max())
        assert float((reduced - (partial + other)).abs().max()) <= tol * 10
        # reduction only (no force rows), with a rank that never publishes: the wait gives up and says so
        capi.peer_return_reduce(None, None, 6, flags[2:3], flags[3:4], None, None, force, partial, ptrs, fptrs, table, flags[8:], reduced, 0, 2,
                                status, counter, max_polls=2000)
        torch.cuda.synchronize()
        assert int(status[0]) == 1
