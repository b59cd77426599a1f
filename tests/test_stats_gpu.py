"""Dataset-statistics ops (fitutils) on the GPU against the reference's CPU templates."""
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi

pytestmark = pytest.mark.gpu


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _batch(dt, seed=4, B=5, npad=37, nd=20, ntypes=3):
    rng = np.random.default_rng(seed)
    binum = rng.integers(9, npad + 1, B).astype(np.int32)
    binum[0] = npad
    desc = (rng.normal(0.3, 1.0, (B, npad, nd)) * rng.uniform(0.1, 5.0, nd)).astype(dt)
    desc[:, :, 3] = -np.abs(desc[:, :, 3]) - 0.5          # an all-negative component (max keeps its FLT_MIN start)
    bilist = np.tile(np.arange(npad, dtype=np.int32), (B, 1))
    for b in range(B):
        bilist[b, :binum[b]] = rng.permutation(binum[b])
    btypes = rng.integers(0, ntypes, (B, npad)).astype(np.int32)
    btypes[btypes == 2] = 1                                # type 2 has no atoms
    etot = rng.normal(-300.0, 20.0, B).astype(dt)
    force = rng.normal(0, 1.5, (B, npad, 3)).astype(dt)
    return binum, desc, bilist, btypes, etot, force


@pytest.mark.parametrize("dt,tol", [(np.float64, 1e-10), (np.float32, 1e-5)])
def test_statistics_ops(checkers, dt, tol):
    from ai2pot_b200 import fromcc
    chk = _chk(checkers)
    binum, desc, bilist, btypes, etot, force = _batch(dt)
    n, mean, m2 = fromcc.allTypeDescriptorsStatisticsOp(_t(binum), _t(desc))
    rn, rmean, rm2 = chk.desc_stats(binum, desc)
    assert int(n) == int(rn[0]) == int(binum.sum())
    assert util.relerr(mean.cpu().numpy(), rmean) < tol and util.relerr(m2.cpu().numpy(), rm2) < tol
    n3, mean3, m23 = fromcc.eachTypeDescriptorsStatisticsOp(_t(binum), _t(bilist), _t(btypes), 3, _t(desc))
    rn3, rmean3, rm23 = chk.desc_stats(binum, desc, bilist, btypes, 3)
    assert np.array_equal(n3.cpu().numpy(), rn3) and rn3[2] == 0
    assert util.relerr(mean3.cpu().numpy(), rmean3) < tol and util.relerr(m23.cpu().numpy(), rm23) < tol
    assert not mean3.cpu().numpy()[2].any()                # empty type: zeros, as the reference leaves them
    mx, mn = fromcc.allTypeDescriptorsMaxminOp(_t(binum), _t(desc))
    rmx, rmn = chk.desc_maxmin(binum, desc)
    assert np.array_equal(mx.cpu().numpy(), rmx) and np.array_equal(mn.cpu().numpy(), rmn)
    assert 0 < rmx[3] < 1e-30                              # the reference's FLT_MIN start shows through
    nt, em, em2, f2 = fromcc.targetStatisticsOp(_t(binum), _t(etot), _t(force))
    rnt, rout = chk.target_stats(binum, etot, force)
    assert int(nt) == rnt
    got = np.array([em.item(), em2.item(), f2.item()])
    assert np.all(np.abs(got - rout) <= tol * np.abs(rout))


@pytest.mark.parametrize("dt", [torch.float64, torch.float32])
@pytest.mark.parametrize("weighted", [True, False])
def test_weighted_sum_rows(dt, weighted):
    """One launch for `grad_out @ per-structure gradients` of several parameter tensors."""
    g = torch.Generator(device="cuda").manual_seed(3)
    B = 37
    parts = [torch.randn(B, n, dtype=dt, device="cuda", generator=g) for n in (576, 1800, 90, 90, 3, 1)]
    parts[1] = parts[1].reshape(B, 90, 20)          # any trailing shape
    w = torch.randn(B, dtype=dt, device="cuda", generator=g) if weighted else None
    got = capi.weighted_sum_rows(parts, w)
    ww = w if weighted else torch.ones(B, dtype=dt, device="cuda")
    exp = torch.cat([(ww.double() @ p_.reshape(B, -1).double()) for p_ in parts])
    tol = 1e-12 if dt == torch.float64 else 2e-5
    assert got.dtype == dt and got.shape == exp.shape
    assert (got.double() - exp).abs().max().item() <= tol * exp.abs().max().item()
    assert capi.weighted_sum_rows([torch.zeros(0, 5, dtype=dt, device="cuda")]).abs().sum().item() == 0   # empty batch: zeros
