"""Pins the CPU restatement (oracle/oracle.c) against (a) the golden outputs the reference's
own CPU code produced (tests/golden, see make_golden.py), (b) the known answers asserted by
the reference's own unit tests, and (c) the reference build itself when it is present."""
import os
import numpy as np
import pytest

import util
from ai2pot_b200 import synth

G = np.load(os.path.join(util.GOLDEN, "golden_small.npz"))
TOL = {np.float64: 1e-11, np.float32: 2e-5}


@pytest.fixture(scope="module")
def orc(checkers):
    if "oracle" not in checkers:
        pytest.skip("oracle library not built (run make -C oracle oracle)")
    return checkers["oracle"]


def test_mos2_known_answers(orc):
    # source/nblist/tests/test_neighborList.cc:215,244: 12 centre atoms, max 12 neighbours at rcut 3.2
    z = np.load(os.path.join(util.GOLDEN, "mos2_fixture.npz"))
    nn, fn, rc, ty, mx = orc.nblist(z["cell"].astype(np.float32), z["z"], z["frac"].astype(np.float32), 3.2, 16,
                                    is_cart=False, pbc=(1, 1, 0))
    assert len(nn) == 12 and mx == 12 and int(G["mos2_max"]) == 12
    util.assert_nblist_equal((nn, fn, rc), (G["mos2_numneigh"], G["mos2_first"], G["mos2_rcs"]))


def test_switch_known_answers(orc):
    # source/descriptor/mtpr/tests/test_basis.cc:101-111: s(rmin)=1, s'(rmin)=0, s(rmax)=0, s'(rmax)=0
    import ctypes as C
    f = orc.lib.orc_mtp_radial_probe_f64
    q = np.zeros(8); dq = np.zeros(8)
    for r, val in ((2.0, 1.0), (5.0, 0.0)):
        f(C.c_double(r), C.c_double(5.0), C.c_double(2.0), C.c_int(8), q.ctypes.data_as(C.c_void_p), dq.ctypes.data_as(C.c_void_p))
        assert q[0] == val and dq[0] == 0.0      # T_0 = 1, so q[0] = s and dq[0] = s'


def test_g0_golden(orc):
    w = synth.g0(util.tables(10))
    nn, fn, rc, ty, mx = orc.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    assert np.array_equal(nn, G["g0_numneigh"])
    fs, rs = util.canonical_nblist(nn, fn, rc)
    assert np.array_equal(fs, G["g0_first_sorted"]) and np.array_equal(rs.view(np.uint64), G["g0_rcs_sorted"].view(np.uint64))
    nb = synth.batch_from_nblist(nn, fn, rc, ty, 3)
    e, f, v = orc.mtp_efv(w["model"], nb)
    assert util.relerr(e, G["g0_e"]) < 1e-11 and util.relerr(f, G["g0_f"]) < 1e-11 and util.relerr(v, G["g0_v"]) < 1e-11
    e2, f2 = orc.mtp_efv(w["model"], nb, virial=False)
    assert util.relerr(e2, G["g0_e"]) < 1e-11 and util.relerr(f2, G["g0_f"]) < 1e-11
    assert util.relerr(orc.mtp_descriptors(w["model"], nb)[0, :8], G["g0_desc_head"]) < 1e-11


@pytest.mark.parametrize("level,dt", [(6, np.float64), (16, np.float64), (10, np.float32)])
def test_mtp_golden(orc, level, dt):
    w = util.small_mtp_case(level, 5, dt)
    nb = util.nblist_batch(orc, w)
    e, f, v = orc.mtp_efv(w["model"], nb)
    tag = f"mtp{level}_{np.dtype(dt).name}"
    for a, k in ((e, "_e"), (f, "_f"), (v, "_v")):
        assert util.relerr(a, G[tag + k]) < TOL[dt], k


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_nep_golden(orc, dt):
    w = util.small_nep_case(5, dt)
    nb = util.nblist_batch(orc, w)
    e, f, v = orc.nep_efv(w["model"], nb)
    tag = f"nep_{np.dtype(dt).name}"
    for a, k in ((e, "_e"), (f, "_f"), (v, "_v")):
        assert util.relerr(a, G[tag + k]) < TOL[dt], k
    e2, f2 = orc.nep_efv(w["model"], nb, virial=False)
    assert util.relerr(f2, G[tag + "_f"]) < TOL[dt]
    assert util.relerr(orc.nep_descriptors(w["model"], nb)[0, :8], G[tag + "_desc_head"]) < TOL[dt]


def test_training_golden(orc):
    g, nb = util.training_batch(orc)
    e, f, v = orc.mtp_efv(g["model"], nb)
    t = g["targets"]; Fd = t["F"][:, :nb["bilist"].shape[1]]
    assert util.relerr(orc.mtp_loss(nb, g["weights"], e, t["E"], f, Fd, v, t["V"]), G["train_loss"]) < 1e-11
    dco, dli, dbi = orc.mtp_loss_backward(g["model"], nb, g["weights"], e, t["E"], f, Fd, v, t["V"])
    assert util.relerr(dco, G["train_dcoeffs"]) < 1e-10
    assert util.relerr(dli, G["train_dlinear"]) < 1e-10
    assert util.relerr(dbi, G["train_dbias"]) < 1e-11


# ---- direct comparison with the reference build (present where the reference is mounted) ----
@pytest.fixture(scope="module")
def ref(checkers):
    if "ref" not in checkers:
        pytest.skip("reference build not present")
    return checkers["ref"]


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_nblist_vs_reference_triclinic(orc, ref, dt):
    rng = np.random.default_rng(5)
    cell = (np.array([[7.0, 0.3, 0.1], [1.5, 6.5, 0.2], [-0.7, 0.9, 8.0]])).astype(dt)
    frac = rng.random((60, 3))
    pos = (frac @ cell.astype(np.float64) + rng.normal(0, 3.0, (60, 3))).astype(dt)   # not wrapped into the cell
    types = rng.integers(0, 2, 60).astype(np.int32)
    for pbc in ((1, 1, 1), (1, 0, 1), (0, 0, 0)):
        a = orc.nblist(cell, types, pos, 5.5, 160, pbc=pbc)
        b = ref.nblist(cell, types, pos, 5.5, 160, pbc=pbc)
        util.assert_nblist_equal(a[:3], b[:3])
        assert a[4] == b[4]
    a = orc.nblist(cell, types, frac.astype(dt), 5.5, 160, is_cart=False, sort=True)
    b = ref.nblist(cell, types, frac.astype(dt), 5.5, 160, is_cart=False, sort=True)
    util.assert_nblist_equal(a[:3], b[:3])


def test_small_cell_multiple_images(orc, ref):
    # cell edge < rcut: the same neighbour index appears with several images, and an atom sees its own images
    rng = np.random.default_rng(9)
    cell = np.eye(3) * 4.0
    pos = rng.random((3, 3)) * 4.0
    a = orc.nblist(cell, [0, 1, 0], pos, 6.0, 256)
    b = ref.nblist(cell, [0, 1, 0], pos, 6.0, 256)
    util.assert_nblist_equal(a[:3], b[:3])


def test_g1_like_vs_reference(orc, ref):
    w = synth.g1(util.tables(16), n=8)
    a = orc.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    b = ref.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    util.assert_nblist_equal(a[:3], b[:3])
    nb = synth.batch_from_nblist(*b[:4], 3)
    for x, y in zip(orc.mtp_efv(w["model"], nb), ref.mtp_efv(w["model"], nb)):
        assert util.relerr(x, y) < 1e-11


def test_fvt_vs_reference(orc, ref):
    w = util.small_mtp_case(6, 4)
    nn, fn, rc, ty, mx = ref.nblist(w["cell"], w["types"], w["coords"], 4.0, 40)
    de = np.random.default_rng(3).normal(size=rc.shape)
    il = np.arange(len(nn), dtype=np.int32)
    assert util.relerr(orc.fvt_force(il, nn, fn, 0, de), ref.fvt_force(il, nn, fn, 0, de)) < 1e-13
    assert util.relerr(orc.fvt_virial(nn, rc, de), ref.fvt_virial(nn, rc, de)) < 1e-13


@pytest.mark.parametrize("dt,tol", [(np.float64, 1e-12), (np.float32, 1e-5)])
def test_zbl_restatement_against_reference_pair_functions(checkers, dt, tol):
    """ZBL: the C restatement against the reference's own PairZBL methods; and what the reference's CPU
    group calls do with them (correct_efv: energy only, zbl.h:545-548; correct_ef: energy and force)."""
    if "ref" not in checkers:
        pytest.skip("reference build not available")
    ref, orc = checkers["ref"], checkers["oracle"]
    w = util.small_nep_case(n=4, dtype=dt, seed=30, a=2.2)
    nn, fn, rc, ty, mx = ref.nblist(w["cell"], w["types"], w["coords"], 4.0, 96)
    n = len(nn)
    nb1 = dict(ilist=np.arange(n, dtype=np.int32), numneigh=nn, firstneigh=fn, rcs=rc, types=ty, nghost=0)
    tm = np.array([14, 8, 29], np.int32)
    rng = np.random.default_rng(3)
    cks = (np.tile([0.18175, 0.50986, 0.28022, 0.02817], (9, 1)) * rng.uniform(0.9, 1.1, (9, 4))).astype(dt)
    dks = np.tile([3.1998, 0.94229, 0.4029, 0.20162], (9, 1)).astype(dt)
    er, fr, vr = ref.zbl(nb1, tm, 2.5, 1.0, cks, dks)
    eo, fo, vo = orc.zbl(nb1, tm, 2.5, 1.0, cks, dks)
    assert er > 1.0
    assert abs(eo - er) <= tol * abs(er) and util.relerr(fo, fr) < tol and util.relerr(vo, vr) < tol
    assert abs(np.trace(vr.reshape(3, 3))) > 0 and np.allclose(vr.reshape(3, 3), vr.reshape(3, 3).T, rtol=1e-4, atol=1e-6 * abs(vr).max())
    ec, fc, vc = ref.zbl(nb1, tm, 2.5, 1.0, cks, dks, variant="cpu_efv")
    assert abs(ec - er) <= 1e-5 * abs(er) and not fc.any() and not vc.any()
    ee, fe, _ = ref.zbl(nb1, tm, 2.5, 1.0, cks, dks, variant="cpu_ef")
    assert util.relerr(fe, fr) < tol


@pytest.mark.parametrize("dt,tol", [(np.float64, 1e-12), (np.float32, 2e-6)])
def test_statistics_restatement(checkers, dt, tol):
    """fitutils statistics: C restatement against the reference templates (descriptorsStatistics.h, targetStatistics.h)."""
    if "ref" not in checkers:
        pytest.skip("reference build not available")
    import test_stats_gpu as tsg
    ref, orc = checkers["ref"], checkers["oracle"]
    binum, desc, bilist, btypes, etot, force = tsg._batch(dt)
    for args in ((binum, desc), (binum, desc, bilist, btypes, 3)):
        a, b = ref.desc_stats(*args), orc.desc_stats(*args)
        assert np.array_equal(a[0], b[0]) and util.relerr(b[1], a[1]) < tol and util.relerr(b[2], a[2]) < tol
    a, b = ref.desc_maxmin(binum, desc), orc.desc_maxmin(binum, desc)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    a, b = ref.target_stats(binum, etot, force), orc.target_stats(binum, etot, force)
    assert a[0] == b[0] and np.all(np.abs(a[1] - b[1]) <= tol * np.abs(a[1]))

