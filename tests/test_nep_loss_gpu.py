"""NEP training path on the GPU: per-structure loss gradients against the reference's CPU code.
fp64: rel 1e-10. fp32: the two-sided statement of util.fp32_parity with tol 1e-5 (within 1e-5 of the same
gradients evaluated in fp64, or at least as close to them as the reference's own fp32 CPU code is)."""
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _batch(chk, dt, seed=5, shape=None):
    ws = [util.small_nep_case(n=3, dtype=dt, seed=40, a=3.0), util.small_nep_case(n=4, dtype=dt, seed=41, a=2.8),
          util.small_nep_case(n=3, dtype=dt, seed=42, a=3.3)]
    if shape is not None:   # same structures, another model shape
        rng = np.random.default_rng(seed + 1)
        ws[0]["model"] = synth.nep_model(3, rng, dt, **shape)
        ws[0]["model"]["type_bias"] = rng.normal(0, 0.1, 3).astype(dt)
        ws[0]["model"]["q_scaler"] = rng.uniform(0.5, 1.5, len(ws[0]["model"]["q_scaler"])).astype(dt)
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


def _compare(chk, m, nb, wts, e, E, f, F, v, V, got, dt, case):
    ref = chk.nep_loss_backward(m, nb, wts, e, E, f, F, v, V)
    names = ("coeffs", "w0", "b0", "w1", "bias")
    if dt == np.float64:
        for name, a, b in zip(names, ref, got):
            assert util.relerr(b.cpu().numpy(), a) < 1e-10, name
        return
    # the same gradients in fp64 (model, rows and the fp32 model outputs promoted)
    nb64 = dict(nb, brcs=nb["brcs"].astype(np.float64))
    up = lambda a: None if a is None else np.asarray(a, np.float64)
    r64 = chk.nep_loss_backward(util.to64(m), nb64, wts, up(e), up(E), up(f), up(F), up(v), up(V))
    for name, a32, a64, b in zip(names, ref, r64, got):
        util.fp32_parity(case, "d" + name, b.cpu().numpy(), a32, a64)


@pytest.mark.parametrize("dt", [np.float64, np.float32])
@pytest.mark.parametrize("virial", [True, False])
def test_nep_loss_backward(checkers, dt, virial):
    chk = _chk(checkers)
    m, nb, (E, F, V) = _batch(chk, dt)
    e, f, v = chk.nep_efv(m, nb)
    wts = (1.0, 2.0, 0.5)
    tdt = torch.float64 if dt == np.float64 else torch.float32
    md = capi.to_device(m, "cuda", tdt)
    nbd = capi.to_device(nb)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    got = capi.nep_loss_backward(md, nbd, wts, t(e), t(E), t(f), t(F), t(v) if virial else None, t(V) if virial else None)
    _compare(chk, m, nb, wts, e, E, f, F, v if virial else None, V if virial else None, got, dt, f"nep_loss_backward virial={virial}")


# model shapes around the specialised kernel's plan (at most 4 radial / angular functions, basis size <= 8):
# narrower than the plan, and two that only the general kernel takes
@pytest.mark.parametrize("shape", [dict(n_radial=3, n_angular=2, chebyshev_size=6, l_max=2, num_neurons=10),
                                   dict(n_radial=4, n_angular=3, chebyshev_size=5, l_max=3, num_neurons=40),
                                   dict(n_radial=6, n_angular=4, chebyshev_size=8, l_max=4, num_neurons=30),
                                   dict(n_radial=4, n_angular=4, chebyshev_size=10, l_max=3, num_neurons=20)])
@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_nep_loss_backward_shapes(checkers, shape, dt):
    chk = _chk(checkers)
    m, nb, (E, F, V) = _batch(chk, dt, shape=shape)
    e, f, v = chk.nep_efv(m, nb)
    wts = (1.0, 2.0, 0.5)
    md = capi.to_device(m, "cuda", torch.float64 if dt == np.float64 else torch.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    got = capi.nep_loss_backward(md, capi.to_device(nb), wts, t(e), t(E), t(f), t(F), t(v), t(V))
    _compare(chk, m, nb, wts, e, E, f, F, v, V, got, dt, "nep_loss_backward shape " + "/".join(str(x) for x in shape.values()))


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_nep_loss_backward_many_blocks_per_structure(checkers, dt):
    """Structures large enough that their blocks do not form one cluster: the gradients are then
    summed over the blocks with atomics (216 atoms = 14 blocks of 16 atoms)."""
    chk = _chk(checkers)
    ws = [util.small_nep_case(n=6, dtype=dt, seed=50, a=3.0), util.small_nep_case(n=3, dtype=dt, seed=51, a=3.1)]
    lists = [chk.nblist(w["cell"], w["types"], w["coords"], 6.0, 200)[:4] for w in ws]
    nb = synth.pad_batch(lists, 3, 200)
    m = ws[0]["model"]
    rng = np.random.default_rng(9)
    B, npad = nb["bilist"].shape
    E, F, V = rng.normal(size=B).astype(dt), rng.normal(size=(B, npad, 3)).astype(dt), rng.normal(size=(B, 9)).astype(dt)
    e, f, v = chk.nep_efv(m, nb)
    wts = (1.0, 2.0, 0.5)
    md = capi.to_device(m, "cuda", torch.float64 if dt == np.float64 else torch.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    got = capi.nep_loss_backward(md, capi.to_device(nb), wts, t(e), t(E), t(f), t(F), t(v), t(V))
    _compare(chk, m, nb, wts, e, E, f, F, v, V, got, dt, "nep_loss_backward 216+27 atoms (atomics path)")


@pytest.mark.parametrize("virial", [True, False])
def test_nep_loss_ops_autograd(checkers, virial):
    """nepToLossOp / nepToEFLossOp: loss values, RMSEs and autograd to coeffs, w0, b0, w1, type_bias."""
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    dt = np.float64
    m, nb, (E, F, V) = _batch(chk, dt)
    e, f, v = chk.nep_efv(m, nb)
    wts = (1.0, 2.0, 0.5)
    ref = chk.nep_loss_backward(m, nb, wts, e, E, f, F, v if virial else None, V if virial else None)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    par = [t(m[k].astype(dt)).requires_grad_(True) for k in ("coeffs", "w0", "b0", "w1", "type_bias")]
    z = torch.zeros(36, dtype=torch.float64, device="cuda")
    tail = (m["chebyshev_size"], m["n_radial"], m["n_angular"], m["l_max"], *par, t(nb["binum"]), t(nb["bilist"]), t(nb["bnumneigh"]),
            t(nb["bfirstneigh"]), t(nb["brcs"]), t(nb["btypes"]), torch.arange(3, dtype=torch.int32, device="cuda"), 0,
            m["rmax_radial"], m["rmax_angular"], t(m["q_scaler"].astype(dt)), 0.0, 0.0, z, z)
    if virial:
        out = fromcc.nepToLossOp(wts[0], wts[1], wts[2], t(E), t(F), t(V), *tail)
    else:
        out = fromcc.nepToEFLossOp(wts[0], wts[1], t(E), t(F), *tail)
    assert len(out) == (4 if virial else 3)
    loss = out[0]
    # loss definition (nepLoss.h:139-215) on the checker's E/F/V
    n = nb["binum"].astype(dt)
    exp = wts[0] / n * (e - E) ** 2
    for b in range(len(n)):
        k = int(n[b])
        exp[b] += wts[1] / (3 * k) * ((f[b, :k] - F[b, :k]) ** 2).sum()
        if virial:
            exp[b] += wts[2] / (9 * k) * ((v[b] - V[b]) ** 2).sum()
    assert util.relerr(loss.detach().cpu().numpy(), exp) < 1e-10
    e_rmse = np.sqrt((((e - E) / n) ** 2).mean())
    assert abs(out[1].item() - e_rmse) < 1e-10 * e_rmse
    g = torch.tensor([0.5, 1.0, 2.0], dtype=torch.float64, device="cuda")
    (loss * g).sum().backward()
    gw = g.cpu().numpy()
    for p, r, name in zip(par, ref, ("coeffs", "w0", "b0", "w1", "bias")):
        assert util.relerr(p.grad.cpu().numpy().ravel(), gw @ r) < 1e-10, name
