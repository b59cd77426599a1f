"""ZBL pair correction on the GPU against the reference's CPU pair functions (through the checker),
directly over the C ABI and through the torch ops with zbl_rmax > 0."""
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu

TYPE_MAP = np.array([14, 8, 29], np.int32)
CK = np.array([0.18175, 0.50986, 0.28022, 0.02817])
DK = np.array([3.1998, 0.94229, 0.4029, 0.20162])


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _coeffs(dt, seed=3):
    rng = np.random.default_rng(seed)
    cks = (np.tile(CK, (9, 1)) * rng.uniform(0.9, 1.1, (9, 4))).astype(dt)
    dks = (np.tile(DK, (9, 1)) * rng.uniform(0.9, 1.1, (9, 4))).astype(dt)
    return cks, dks


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _dense_lists(chk, dt, sizes=(4, 3)):
    """Two small dense structures (nearest neighbours ~2.2 A, so the 2.5 A ZBL range is populated)."""
    lists = []
    for k, n in enumerate(sizes):
        w = util.small_nep_case(n=n, dtype=dt, seed=30 + k, a=2.2)
        nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], 4.0, 96)
        lists.append((nn, fn, rc, ty))
    return lists


@pytest.mark.parametrize("dt,tol", [(np.float64, 1e-10), (np.float32, 1e-5)])
def test_zbl_c_abi_ragged_batch(checkers, dt, tol):
    chk = _chk(checkers)
    lists = _dense_lists(chk, dt)
    nb = synth.pad_batch(lists, 3, 96)
    cks, dks = _coeffs(dt)
    nbd = capi.to_device(nb)
    B, npad = nb["bilist"].shape
    rng = np.random.default_rng(1)
    e0 = rng.normal(size=B).astype(dt); f0 = rng.normal(size=(B, npad, 3)).astype(dt); v0 = rng.normal(size=(B, 9)).astype(dt)
    e, f, v = capi.zbl_efv(nbd, _t(TYPE_MAP), 2.5, 1.0, _t(cks.ravel()), _t(dks.ravel()), _t(e0), _t(f0), _t(v0))
    e2, f2, _ = capi.zbl_efv(nbd, _t(TYPE_MAP), 2.5, 1.0, _t(cks.ravel()), _t(dks.ravel()), _t(e0), _t(f0), None)   # no virial
    for b, (nn, fn, rc, ty) in enumerate(lists):
        n = len(nn)
        nb1 = dict(ilist=np.arange(n, dtype=np.int32), numneigh=nn, firstneigh=fn, rcs=rc, types=ty, nghost=0)
        er, fr, vr = chk.zbl(nb1, TYPE_MAP, 2.5, 1.0, cks, dks)
        assert er > 1.0                                           # the range is populated
        assert abs(e.cpu().numpy()[b] - e0[b] - er) < tol * abs(er)
        assert util.relerr(f.cpu().numpy()[b, :n] - f0[b, :n], fr) < tol
        assert util.relerr(v.cpu().numpy()[b] - v0[b], vr) < tol
        assert np.array_equal(f.cpu().numpy()[b, n:], f0[b, n:])  # padding rows untouched
        assert util.relerr(f2.cpu().numpy()[b, :n] - f0[b, :n], fr) < tol


def test_zbl_through_nep_op(checkers):
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    dt = np.float32
    w = util.small_nep_case(n=4, dtype=dt, seed=30, a=2.2)
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], 6.0, 160)
    nb = synth.batch_from_nblist(nn, fn, rc, ty, 3)
    m = w["model"]
    cks, dks = _coeffs(dt)
    tm = _t(TYPE_MAP)
    base = (m["chebyshev_size"], m["n_radial"], m["n_angular"], m["l_max"], _t(m["coeffs"]), _t(m["w0"]), _t(m["b0"]), _t(m["w1"]),
            _t(m["type_bias"]), _t(nb["binum"]), _t(nb["bilist"]), _t(nb["bnumneigh"]), _t(nb["bfirstneigh"]), _t(nb["brcs"]),
            _t(nb["btypes"]), tm, 0, m["rmax_radial"], m["rmax_angular"], _t(m["q_scaler"]))
    e0, f0, v0 = fromcc.nepToEFVOp(*base, 0.0, 0.0, _t(cks.ravel()), _t(dks.ravel()))
    e1, f1, v1 = fromcc.nepToEFVOp(*base, 2.5, 1.0, _t(cks.ravel()), _t(dks.ravel()))
    n = len(nn)
    nb1 = dict(ilist=np.arange(n, dtype=np.int32), numneigh=nn, firstneigh=fn, rcs=rc, types=ty, nghost=0)
    er, fr, vr = chk.zbl(nb1, TYPE_MAP, 2.5, 1.0, cks, dks)
    assert abs((e1 - e0).item() - er) < 1e-5 * abs(er)
    assert util.relerr((f1 - f0).cpu().numpy()[0], fr) < 1e-5
    assert util.relerr((v1 - v0).cpu().numpy()[0], vr) < 1e-5
    e2, f2 = fromcc.nepToEFOp(*base, 2.5, 1.0, _t(cks.ravel()), _t(dks.ravel()))
    assert util.relerr(f2.cpu().numpy(), f1.cpu().numpy()) < 1e-6


def test_zbl_through_mtp_op(checkers):
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    dt = np.float64
    w = util.small_mtp_case(10, 4, dt)
    w["coords"] = (w["coords"] * 0.75).astype(dt); w["cell"] = (w["cell"] * 0.75).astype(dt)      # compress: pairs inside 2.5 A
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], 4.0, 96)
    nb = synth.batch_from_nblist(nn, fn, rc, ty, w["model"]["ntypes"])
    ntypes = nb["ntypes"]
    model = w["model"]
    tb = model["tables"]
    td = torch.float64
    rng = np.random.default_rng(9)
    cks = (np.tile(CK, (ntypes * ntypes, 1)) * rng.uniform(0.9, 1.1, (ntypes * ntypes, 4))).astype(dt)
    dks = np.tile(DK, (ntypes * ntypes, 1)).astype(dt)
    tmap = np.array([14, 8, 29, 6][:ntypes], np.int32)

    def call(zr, zm):
        return fromcc.linearMtpToEFVOp(
            model["chebyshev_size"], model["scaling"], _t(model["coeffs"]).to(td), _t(model["linear_coeffs"]).to(td),
            _t(model["type_bias"]).to(td), tb["alpha_moments_count"], _t(tb["alpha_index_basic"]), _t(tb["alpha_index_times"]),
            _t(tb["alpha_moment_mapping"]), tb["nmus"], _t(nb["binum"]), _t(nb["bilist"]), _t(nb["bnumneigh"]), _t(nb["bfirstneigh"]),
            _t(nb["brcs"]), _t(nb["btypes"]), _t(tmap), 0, 4.0, model["rmin"], _t(model["q_scaler"]).to(td), zr, zm,
            _t(cks.ravel()), _t(dks.ravel()))
    e0, f0, v0 = call(0.0, 0.0)
    e1, f1, v1 = call(2.5, 1.0)
    n = len(nn)
    nb1 = dict(ilist=np.arange(n, dtype=np.int32), numneigh=nn, firstneigh=fn, rcs=rc, types=ty, nghost=0)
    er, fr, vr = chk.zbl(nb1, tmap, 2.5, 1.0, cks, dks)
    assert er > 0.1
    assert abs((e1 - e0).item() - er) < 1e-10 * max(abs(er), abs(e0.item()))
    assert util.relerr((f1 - f0).cpu().numpy()[0], fr) < 1e-10
    assert util.relerr((v1 - v0).cpu().numpy()[0], vr) < 1e-10


def test_zbl_in_mtp_loss_op(checkers):
    """linearMtpToLossOp with zbl_rmax > 0 (source/descriptor/mtpr/src/linearMtpOp.cc:723-740, 814-819, 1293, 1395): the
    correction is added onto E/F/V before the loss, in forward and backward; loss and the three gradients against
    the CPU checkers fed with corrected E/F/V."""
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    dt = np.float64
    rng = np.random.default_rng(12)
    lists, ws = [], []
    for k, n in enumerate((4, 3)):
        w = util.small_mtp_case(10, n, dt, seed=60 + k)
        w["coords"] = (w["coords"] * 0.75).astype(dt); w["cell"] = (w["cell"] * 0.75).astype(dt)
        nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], 4.0, 96)
        lists.append((nn, fn, rc, ty)); ws.append(w)
    nb = synth.pad_batch(lists, 3, 96)
    model = dict(ws[0]["model"], rmax=4.0)
    tb = model["tables"]
    B, npad = nb["bilist"].shape
    cks, dks = _coeffs(dt)
    E, F, V = rng.normal(size=B), rng.normal(size=(B, npad, 3)), rng.normal(size=(B, 9))
    wts = (1.0, 0.6, 0.3)
    # corrected model outputs from the checkers
    e, f, v = chk.mtp_efv(model, nb)
    for b, (nn, fn, rc, ty) in enumerate(lists):
        n = len(nn)
        nb1 = dict(ilist=np.arange(n, dtype=np.int32), numneigh=nn, firstneigh=fn, rcs=rc, types=ty, nghost=0)
        ez, fz, vz = chk.zbl(nb1, TYPE_MAP, 2.5, 1.0, cks, dks)
        e[b] += ez; f[b, :n] += fz; v[b] += vz
    lr = chk.mtp_loss(nb, wts, e, E, f, F, v, V)
    ref = chk.mtp_loss_backward(model, nb, wts, e, E, f, F, v, V)
    td = torch.float64
    par = [_t(model[k]).to(td).requires_grad_(True) for k in ("coeffs", "linear_coeffs", "type_bias")]
    loss, e_rmse, f_rmse, v_rmse = fromcc.linearMtpToLossOp(
        wts[0], wts[1], wts[2], _t(E), _t(F), _t(V.reshape(B, 3, 3)), model["chebyshev_size"], model["scaling"], par[0], par[1], par[2],
        tb["alpha_moments_count"], _t(tb["alpha_index_basic"]), _t(tb["alpha_index_times"]), _t(tb["alpha_moment_mapping"]), tb["nmus"],
        _t(nb["binum"]), _t(nb["bilist"]), _t(nb["bnumneigh"]), _t(nb["bfirstneigh"]), _t(nb["brcs"]), _t(nb["btypes"]), _t(TYPE_MAP), 0,
        4.0, model["rmin"], _t(model["q_scaler"]).to(td), 2.5, 1.0, _t(cks.ravel()), _t(dks.ravel()))
    assert util.relerr(loss.detach().cpu().numpy(), lr) < 1e-10
    g = torch.tensor([0.5, 2.0], dtype=td, device="cuda")
    (loss * g).sum().backward()
    gw = g.cpu().numpy()
    for p, r, name in zip(par, ref, ("coeffs", "linear", "bias")):
        assert util.relerr(p.grad.cpu().numpy().ravel(), gw @ r) < 1e-10, name


def test_zbl_in_nep_loss_op(checkers):
    """nepToLossOp with zbl_rmax > 0: loss and gradients against the CPU checkers fed with corrected E/F/V (fp64)."""
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    dt = np.float64
    rng = np.random.default_rng(13)
    lists = _dense_lists(chk, dt)
    nb = synth.pad_batch(lists, 3, 96)
    m = util.small_nep_case(n=3, dtype=dt, seed=30)["model"]
    m = dict(m, rmax_radial=4.0, rmax_angular=3.0)
    B, npad = nb["bilist"].shape
    cks, dks = _coeffs(dt)
    E, F, V = rng.normal(size=B), rng.normal(size=(B, npad, 3)), rng.normal(size=(B, 9))
    wts = (1.0, 0.6, 0.3)
    e, f, v = chk.nep_efv(m, nb)
    for b, (nn, fn, rc, ty) in enumerate(lists):
        n = len(nn)
        nb1 = dict(ilist=np.arange(n, dtype=np.int32), numneigh=nn, firstneigh=fn, rcs=rc, types=ty, nghost=0)
        ez, fz, vz = chk.zbl(nb1, TYPE_MAP, 2.5, 1.0, cks, dks)
        e[b] += ez; f[b, :n] += fz; v[b] += vz
    ref = chk.nep_loss_backward(m, nb, wts, e, E, f, F, v, V)
    par = [_t(m[k].astype(dt)).requires_grad_(True) for k in ("coeffs", "w0", "b0", "w1", "type_bias")]
    out = fromcc.nepToLossOp(wts[0], wts[1], wts[2], _t(E), _t(F), _t(V), m["chebyshev_size"], m["n_radial"], m["n_angular"], m["l_max"],
                             *par, _t(nb["binum"]), _t(nb["bilist"]), _t(nb["bnumneigh"]), _t(nb["bfirstneigh"]), _t(nb["brcs"]),
                             _t(nb["btypes"]), _t(TYPE_MAP), 0, 4.0, 3.0, _t(m["q_scaler"].astype(dt)), 2.5, 1.0, _t(cks.ravel()),
                             _t(dks.ravel()))
    n = nb["binum"].astype(dt)
    exp = wts[0] / n * (e - E) ** 2
    for b in range(B):
        k = int(n[b])
        exp[b] += wts[1] / (3 * k) * ((f[b, :k] - F[b, :k]) ** 2).sum() + wts[2] / (9 * k) * ((v[b] - V[b]) ** 2).sum()
    assert util.relerr(out[0].detach().cpu().numpy(), exp) < 1e-10
    g = torch.tensor([0.5, 2.0], dtype=torch.float64, device="cuda")
    (out[0] * g).sum().backward()
    gw = g.cpu().numpy()
    for p, r, name in zip(par, ref, ("coeffs", "w0", "b0", "w1", "bias")):
        assert util.relerr(p.grad.cpu().numpy().ravel(), gw @ r) < 1e-10, name
