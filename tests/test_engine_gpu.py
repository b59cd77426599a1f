"""The Evaluator's recorded calls (CUDA graphs whose kernel launches are chained to one another) against its eager
calls and the CPU checker: the same numbers after many back-to-back replays, and a replay sees the positions that
are in the buffers at that time. What a calculator does per call: ai2pot/models/potential_utils.py:217-268."""
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import engine, synth

pytestmark = pytest.mark.gpu


def _workload(kind, n):
    if kind == "mtp":
        return synth.g1(util.tables(16), n=n), torch.float64, 1e-10
    return synth.g2(n=n), torch.float32, 1e-5


def _moved(w, seed):
    rng = np.random.default_rng(seed)
    return (w["coords"] + rng.normal(0, 0.05, w["coords"].shape)).astype(w["coords"].dtype)


def _host(out):
    return tuple(t.detach().cpu().numpy().copy() for t in out)


def _close(a, b, tol):
    for x, y in zip(a, b):
        assert util.relerr(x, y) < tol


@pytest.mark.parametrize("kind", ["mtp", "nep"])
def test_replay_equals_eager_and_checker(kind, checkers):
    w, dt, tol = _workload(kind, 10)          # 1,000 atoms
    ev = engine.Evaluator(w["model"], w["cell"], w["types"], w["rcut"], w["umax"], dt)
    pos = [np.ascontiguousarray(w["coords"]), _moved(w, 5), _moved(w, 6)]
    coords = torch.from_numpy(pos[0]).to(dt).cuda()
    eager = []
    for p in pos:
        coords.copy_(torch.from_numpy(p).to(dt))
        eager.append(_host(ev.compute(coords)))
    assert int(ev.status.cpu()[1]) == 0
    # the CPU code on the first configuration
    chk = checkers.get("ref") or checkers["oracle"]
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], pos[0], w["rcut"], w["umax"])
    nb = synth.batch_from_nblist(nn, fn, rc, ty, 3)
    ref = chk.mtp_efv(w["model"], nb) if kind == "mtp" else chk.nep_efv(w["model"], nb)
    _close(eager[0], ref[:3], tol)

    assert ev.capture(coords)
    for k in (1, 2, 0):
        coords.copy_(torch.from_numpy(pos[k]).to(dt))
        for _ in range(20):                    # back to back, nothing in between: the outputs are rebuilt by every replay
            out = ev.replay()
        _close(_host(out), eager[k], tol)

    # the whole call as one graph: pinned host positions in, one pinned host buffer out
    h_in = torch.empty_like(coords, device="cpu").pin_memory()
    h_out = torch.empty(ev.outbuf.shape, dtype=dt).pin_memory()
    h_in.copy_(torch.from_numpy(pos[0]).to(dt))
    assert ev.capture_io(coords, h_in, h_out)
    n = len(w["types"])
    for k in (2, 0, 1):
        h_in.copy_(torch.from_numpy(pos[k]).to(dt))
        h_out.fill_(float("nan"))
        for _ in range(5):
            ev.replay_io()
        torch.cuda.synchronize()
        got = (h_out[0:1].numpy(), h_out[16:16 + 3 * n].numpy().reshape(1, n, 3), h_out[1:10].numpy().reshape(1, 9))
        _close(got, eager[k], tol)


@pytest.mark.parametrize("kind", ["mtp", "nep"])
def test_ordinary_launches_give_the_same(kind, monkeypatch):
    """AI2B_CHAIN=0 switches the chained launches off: same numbers either way."""
    w, dt, tol = _workload(kind, 8)
    ev = engine.Evaluator(w["model"], w["cell"], w["types"], w["rcut"], w["umax"], dt)
    coords = torch.from_numpy(np.ascontiguousarray(w["coords"])).to(dt).cuda()
    chained = _host(ev.compute(coords))
    monkeypatch.setenv("AI2B_CHAIN", "0")
    plain = _host(ev.compute(coords))
    monkeypatch.delenv("AI2B_CHAIN")
    again = _host(ev.compute(coords))
    _close(plain, chained, tol)
    _close(again, chained, tol)
