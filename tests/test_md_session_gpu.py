"""Device-resident MD input path (ai2b_md_session_*): a periodic system is handed over the way an MD
host holds it (local atoms + ghost images, double positions, model types), and the folded forces,
the energy and the six virial components must equal the periodic evaluation of the checker."""
import numpy as np
import pytest

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _with_ghosts(cell, coords, types, rcut):
    """Local atoms wrapped into an orthorhombic box + images with any coordinate within rcut of it."""
    L = np.diag(cell).astype(np.float64)
    x = np.mod(coords.astype(np.float64), L)
    gx, gt, owner = [], [], []
    for sx in (-1, 0, 1):
        for sy in (-1, 0, 1):
            for sz in (-1, 0, 1):
                if sx == sy == sz == 0:
                    continue
                y = x + np.array([sx, sy, sz]) * L
                keep = np.all((y > -rcut) & (y < L + rcut), axis=1)
                gx.append(y[keep]); gt.append(types[keep]); owner.append(np.nonzero(keep)[0])
    return x, np.concatenate(gx), np.concatenate(gt), np.concatenate(owner)


def _fold(f, nlocal, owner):
    out = f[:nlocal].copy()
    np.add.at(out, owner, f[nlocal:])
    return out


def test_md_session_nep(checkers):
    chk = _chk(checkers)
    w = util.small_nep_case(6, np.float32, a=3.0)                      # 216 atoms, 18 A box, rcut 6
    m = w["model"]
    x, gx, gt, owner = _with_ghosts(w["cell"], w["coords"], w["types"], 6.0)
    nlocal, nghost = len(x), len(gx)
    # periodic reference on the same (wrapped, float-rounded as the host would see them in double) positions
    nb = util.nblist_batch(chk, dict(w, coords=x.astype(np.float64), cell=w["cell"].astype(np.float64), umax=96))
    nb["brcs"] = nb["brcs"].astype(np.float32)
    e_ref, f_ref, v_ref = chk.nep_efv(m, nb)
    ses = capi.MdSession(m, 96)
    for _ in range(2):                                                  # second step reuses every buffer
        e, f, v6, mx = ses.compute(nlocal, nghost, np.concatenate([x, gx]), np.concatenate([w["types"], gt]))
        assert 20 < mx <= 96
        assert abs(e - e_ref[0]) < 1e-5 * abs(e_ref[0])
        assert util.relerr(_fold(f, nlocal, owner), f_ref[0]) < 1e-5
        assert util.relerr(v6, v_ref[0][[0, 4, 8, 1, 2, 5]]) < 1e-5
    # growing the system re-allocates; a too small umax is reported, not overrun
    tight = capi.MdSession(m, 8)
    with pytest.raises(capi.Ai2bError):
        tight.compute(nlocal, nghost, np.concatenate([x, gx]), np.concatenate([w["types"], gt]))
    tight.close(); ses.close()


def test_md_session_mtp(checkers):
    chk = _chk(checkers)
    w = util.small_mtp_case(10, 5, np.float32, rcut=5.0)                # 125 atoms, 15 A box
    m = w["model"]
    x, gx, gt, owner = _with_ghosts(w["cell"], w["coords"], w["types"], 5.0)
    nlocal, nghost = len(x), len(gx)
    nb = util.nblist_batch(chk, dict(w, coords=x.astype(np.float64), cell=w["cell"].astype(np.float64), umax=64))
    nb["brcs"] = nb["brcs"].astype(np.float32)
    e_ref, f_ref, v_ref = chk.mtp_efv(m, nb)
    prog = capi.MtpProgram(m["tables"])
    ses = capi.MdSession(m, 64, prog)
    e, f, v6, mx = ses.compute(nlocal, nghost, np.concatenate([x, gx]), np.concatenate([w["types"], gt]))
    assert abs(e - e_ref[0]) < 1e-5 * max(abs(e_ref[0]), np.abs(f_ref).max())
    assert util.relerr(_fold(f, nlocal, owner), f_ref[0]) < 1e-5
    assert util.relerr(v6, v_ref[0][[0, 4, 8, 1, 2, 5]]) < 1e-5
    e2, f2, _, _ = ses.compute(nlocal, nghost, np.concatenate([x, gx]), np.concatenate([w["types"], gt]), want_virial=False)
    assert util.relerr(_fold(f2, nlocal, owner), f_ref[0]) < 1e-5
    ses.close()
