"""The reference-facing torch ops (same names / argument lists as ai2pot.fromcc) on CUDA tensors."""
import os
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(util.GOLDEN, "golden_small.npz"))


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _mtp_args(model, nb, dt):
    tb = model["tables"]
    ntypes = nb["ntypes"]
    z = torch.zeros(ntypes * ntypes * 4, dtype=dt, device="cuda")
    return (model["chebyshev_size"], model["scaling"], _t(model["coeffs"], dt), _t(model["linear_coeffs"], dt), _t(model["type_bias"], dt),
            tb["alpha_moments_count"], _t(tb["alpha_index_basic"]), _t(tb["alpha_index_times"]), _t(tb["alpha_moment_mapping"]), tb["nmus"],
            _t(nb["binum"]), _t(nb["bilist"]), _t(nb["bnumneigh"]), _t(nb["bfirstneigh"]), _t(nb["brcs"]), _t(nb["btypes"]),
            torch.arange(ntypes, dtype=torch.int32, device="cuda"), 0, model["rmax"], model["rmin"], _t(model["q_scaler"], dt),
            0.0, 0.0, z, z)


def test_mtp_ops_g0(checkers):
    from ai2pot_b200 import fromcc
    w = synth.g0(util.tables(10))
    nb = util.nblist_batch(_chk(checkers), w)
    args = _mtp_args(w["model"], nb, torch.float64)
    e, f, v = fromcc.linearMtpToEFVOp(*args)
    assert e.shape == (1,) and f.shape == (1, 216, 3) and v.shape == (1, 9) and e.dtype == torch.float64
    for a, k in ((e, "g0_e"), (f, "g0_f"), (v, "g0_v")):
        assert util.relerr(a.cpu().numpy(), G[k]) < 1e-10
    e2, f2 = fromcc.linearMtpToEFOp(*args)            # second call reuses the cached program
    assert util.relerr(f2.cpu().numpy(), G["g0_f"]) < 1e-10
    a = args
    d, = fromcc.linearMtpToDescriptorsOp(a[0], a[1], a[2], a[5], a[6], a[7], a[8], a[9], a[10], a[11], a[12], a[13], a[14], a[15], a[16],
                                         a[17], a[18], a[19])
    assert util.relerr(d.cpu().numpy()[0, :8], G["g0_desc_head"]) < 1e-10
    # zbl_rmax > 0 with all-zero screening coefficients adds nothing (the correction itself: test_zbl_gpu.py)
    e3, f3, v3 = fromcc.linearMtpToEFVOp(*args[:21], 2.0, 1.0, args[23], args[24])
    assert util.relerr(e3.cpu().numpy(), G["g0_e"]) < 1e-10 and util.relerr(v3.cpu().numpy(), G["g0_v"]) < 1e-10


def test_nep_ops(checkers):
    from ai2pot_b200 import fromcc
    w = util.small_nep_case(5, np.float32)
    nb = util.nblist_batch(_chk(checkers), w)
    m = w["model"]
    dt = torch.float32
    z = torch.zeros(36, dtype=dt, device="cuda")
    args = (m["chebyshev_size"], m["n_radial"], m["n_angular"], m["l_max"], _t(m["coeffs"]), _t(m["w0"]), _t(m["b0"]), _t(m["w1"]),
            _t(m["type_bias"]), _t(nb["binum"]), _t(nb["bilist"]), _t(nb["bnumneigh"]), _t(nb["bfirstneigh"]), _t(nb["brcs"]),
            _t(nb["btypes"]), torch.arange(3, dtype=torch.int32, device="cuda"), 0, m["rmax_radial"], m["rmax_angular"], _t(m["q_scaler"]),
            0.0, 0.0, z, z)
    e, f, v = fromcc.nepToEFVOp(*args)
    for a, k in ((e, "_e"), (f, "_f"), (v, "_v")):
        assert util.relerr(a.cpu().numpy(), G["nep_float32" + k]) < 1e-5
    e2, f2 = fromcc.nepToEFOp(*args)
    assert util.relerr(f2.cpu().numpy(), G["nep_float32_f"]) < 1e-5
    d, = fromcc.nepToDescriptorsOp(*args[:5], *args[9:19])
    assert util.relerr(d.cpu().numpy()[0, :8], G["nep_float32_desc_head"]) < 1e-5


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_fvt_ops_values_and_gradients(checkers, dt):
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    w = util.small_mtp_case(6, 4, dt)
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], 4.0, 40)
    n = len(nn)
    rng = np.random.default_rng(3)
    de = rng.normal(size=rc.shape).astype(dt)
    tol = 1e-12 if dt == np.float64 else 1e-5
    tde = _t(de[None]).requires_grad_(True)
    trc = _t(rc[None]).requires_grad_(True)
    binum = torch.tensor([n], dtype=torch.int32, device="cuda")
    bil = torch.arange(n, dtype=torch.int32, device="cuda")[None].contiguous()
    F, = fromcc.forceSrOp(binum, bil, _t(nn[None]), _t(fn[None]), 0, 40, tde)
    V, = fromcc.virialSrOp(_t(nn[None]), trc, 40, tde)
    assert F.shape == (1, n, 3) and V.shape == (1, 3, 3)
    assert util.relerr(F.detach().cpu().numpy()[0], chk.fvt_force(np.arange(n), nn, fn, 0, de)) < tol
    assert util.relerr(V.detach().cpu().numpy().reshape(9), chk.fvt_virial(nn, rc, de)) < tol
    # adjoints: the scatter is linear, so <gF, F(de)> differentiates to the gather of gF
    gF = _t(rng.normal(size=(1, n, 3)).astype(dt)); gV = _t(rng.normal(size=(1, 3, 3)).astype(dt))
    ((F * gF).sum() + (V * gV).sum()).backward()
    mask = (np.arange(40)[None] < nn[:, None])
    gf = gF.cpu().numpy()[0]; gv = gV.cpu().numpy()[0]
    exp_de = np.zeros_like(de); exp_rc = np.zeros_like(rc)
    for i in range(n):
        for j in range(nn[i]):
            exp_de[i, j] = gf[i] - gf[fn[i, j]] - gv @ rc[i, j]
            exp_rc[i, j] = -(gv.T @ de[i, j])
    assert util.relerr(tde.grad.cpu().numpy()[0], exp_de) < tol * 10
    assert util.relerr(trc.grad.cpu().numpy()[0], exp_rc) < tol * 10
    assert np.all(tde.grad.cpu().numpy()[0][~mask] == 0)
