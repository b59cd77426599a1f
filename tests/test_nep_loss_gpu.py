"""NEP training path on the GPU: per-structure loss gradients against the reference's CPU code."""
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _batch(chk, dt, seed=5):
    ws = [util.small_nep_case(n=3, dtype=dt, seed=40, a=3.0), util.small_nep_case(n=4, dtype=dt, seed=41, a=2.8),
          util.small_nep_case(n=3, dtype=dt, seed=42, a=3.3)]
    lists = []
    for w in ws:
        nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], 6.0, 200)
        lists.append((nn, fn, rc, ty))
    nb = synth.pad_batch(lists, 3, 200)
    m = ws[0]["model"]
    rng = np.random.default_rng(seed)
    B, npad = nb["bilist"].shape
    tg = (rng.normal(size=B).astype(dt), rng.normal(size=(B, npad, 3)).astype(dt), rng.normal(size=(B, 9)).astype(dt))
    return m, nb, tg


@pytest.mark.parametrize("dt,tol", [(np.float64, 1e-10), (np.float32, 2e-5)])
@pytest.mark.parametrize("virial", [True, False])
def test_nep_loss_backward(checkers, dt, tol, virial):
    chk = _chk(checkers)
    m, nb, (E, F, V) = _batch(chk, dt)
    e, f, v = chk.nep_efv(m, nb)
    wts = (1.0, 2.0, 0.5)
    ref = chk.nep_loss_backward(m, nb, wts, e, E, f, F, v if virial else None, V if virial else None)
    tdt = torch.float64 if dt == np.float64 else torch.float32
    md = capi.to_device(m, "cuda", tdt)
    nbd = capi.to_device(nb)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    got = capi.nep_loss_backward(md, nbd, wts, t(e), t(E), t(f), t(F), t(v) if virial else None, t(V) if virial else None)
    for name, a, b in zip(("coeffs", "w0", "b0", "w1", "bias"), ref, got):
        assert util.relerr(b.cpu().numpy(), a) < tol, name
