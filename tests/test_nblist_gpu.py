"""Neighbour lists from the CUDA builder: bit-exact with the CPU checkers after canonical sort."""
import os
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth
from ai2pot_b200.fromcc import nblist as nblist_mod

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(util.GOLDEN, "golden_small.npz"))


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _gpu(cell, types, coords, rcut, umax, is_cart=True, pbc=(1, 1, 1), sort=False):
    out = nblist_mod.find_info4mlff(np.ascontiguousarray(cell, dtype=coords.dtype), np.asarray(types), coords, rcut, umax,
                                    is_cart, [bool(p) for p in pbc], sort)
    inum, ilist, nn, fn, rc, ty, ng = out
    assert inum == len(coords) and ng == 0 and np.array_equal(ilist, np.arange(inum)) and ty.dtype == np.int32
    return nn, fn, rc


def test_mos2_fixture():
    z = np.load(os.path.join(util.GOLDEN, "mos2_fixture.npz"))
    nn, fn, rc = _gpu(z["cell"].astype(np.float32), z["z"], z["frac"].astype(np.float32), 3.2, 16, is_cart=False, pbc=(1, 1, 0))
    assert nn.max() == 12
    util.assert_nblist_equal((nn, fn, rc), (G["mos2_numneigh"], G["mos2_first"], G["mos2_rcs"]))


def test_g0_golden():
    w = synth.g0(util.tables(10))
    nn, fn, rc = _gpu(w["cell"], w["types"].astype(np.int64), w["coords"], w["rcut"], w["umax"])
    assert np.array_equal(nn, G["g0_numneigh"])
    fs, rs = util.canonical_nblist(nn, fn, rc)
    assert np.array_equal(fs, G["g0_first_sorted"]) and np.array_equal(rs.view(np.uint64), G["g0_rcs_sorted"].view(np.uint64))
    # padding convention
    pad = np.arange(fn.shape[1])[None] >= nn[:, None]
    assert np.all(fn[pad] == -1) and np.all(rc[pad] == 0)


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_triclinic_unwrapped_open_axes(checkers, dt):
    chk = _chk(checkers)
    rng = np.random.default_rng(5)
    cell = np.array([[7.0, 0.3, 0.1], [1.5, 6.5, 0.2], [-0.7, 0.9, 8.0]]).astype(dt)
    frac = rng.random((60, 3))
    pos = (frac @ cell.astype(np.float64) + rng.normal(0, 3.0, (60, 3))).astype(dt)
    types = rng.integers(0, 2, 60).astype(np.int32)
    for pbc in ((1, 1, 1), (1, 0, 1), (0, 0, 0), (0, 1, 0)):
        a = _gpu(cell, types, pos, 5.5, 160, pbc=pbc)
        b = chk.nblist(cell, types, pos, 5.5, 160, pbc=pbc)
        util.assert_nblist_equal(a, b[:3])
    a = _gpu(cell, types, frac.astype(dt), 5.5, 160, is_cart=False, sort=True)
    b = chk.nblist(cell, types, frac.astype(dt), 5.5, 160, is_cart=False, sort=True)
    util.assert_nblist_equal(a, b[:3])
    # sorted rows: distances ascending
    d = np.sqrt((a[2].astype(np.float64) ** 2).sum(-1))
    for i in range(len(a[0])):
        assert np.all(np.diff(d[i, :a[0][i]]) >= 0)


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_atoms_many_periods_outside_the_cell(checkers, dt):
    """Unwrapped trajectories: some atoms sit hundreds of lattice periods away from the cell. Beyond 127 periods
    the builder leaves its packed-wrap form for full integers; both forms must give the reference algorithm's
    list. Checked against the plain-C restatement: the reference's own CPU build overruns its bins on such input."""
    chk = checkers["oracle"]
    rng = np.random.default_rng(17)
    cell = np.array([[7.0, 0.3, 0.1], [1.5, 6.5, 0.2], [-0.7, 0.9, 8.0]])
    frac = rng.random((80, 3))
    types = rng.integers(0, 2, 80).astype(np.int32)
    for far in (100, 400):   # within / beyond the packed range
        k = rng.integers(-far, far + 1, (80, 3))
        k[::3] = 0           # a third of the atoms stay at home
        pos = ((frac + k) @ cell).astype(dt)
        a = _gpu(cell.astype(dt), types, pos, 5.5, 160)
        b = chk.nblist(cell.astype(dt), types, pos, 5.5, 160)
        util.assert_nblist_equal(a, b[:3])
        assert a[0][::3].min() > 0   # (like the reference, only images within the supercell range count: far atoms get none)


def test_tiny_cell_many_images(checkers):
    chk = _chk(checkers)
    rng = np.random.default_rng(9)
    cell = np.eye(3) * 4.0
    pos = rng.random((3, 3)) * 4.0
    a = _gpu(cell, np.array([0, 1, 0]), pos, 6.0, 256)
    b = chk.nblist(cell, [0, 1, 0], pos, 6.0, 256)
    util.assert_nblist_equal(a, b[:3])
    # one atom alone sees only its own images
    a = _gpu(cell, np.array([0]), pos[:1], 6.0, 64)
    b = chk.nblist(cell, [0], pos[:1], 6.0, 64)
    util.assert_nblist_equal(a, b[:3])


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_g1_full_size_vs_checker(checkers, dt):
    """13,824 atoms, rcut 6 (the benchmark structure), both float types."""
    w = synth.g1(util.tables(16))
    chk = _chk(checkers)
    pos = w["coords"].astype(dt); cell = w["cell"].astype(dt)
    a = _gpu(cell, w["types"], pos, 6.0, 64)
    b = chk.nblist(cell, w["types"], pos, 6.0, 64)
    util.assert_nblist_equal(a, b[:3])


def test_g4_slice_float(checkers):
    w = synth.g4(ncell=8)
    chk = _chk(checkers)
    a = _gpu(w["cell"], w["types"], w["coords"], 6.0, 32)
    b = chk.nblist(w["cell"], w["types"], w["coords"], 6.0, 32)
    util.assert_nblist_equal(a, b[:3])


def test_overflow_and_errors():
    w = synth.g0(util.tables(10))
    with pytest.raises(ValueError):
        _gpu(w["cell"], w["types"], w["coords"], 5.0, 8)
    with pytest.raises(TypeError):
        nblist_mod.find_info4mlff(w["cell"].tolist(), w["types"], w["coords"], 5.0, 64, True, [True] * 3, False)
    with pytest.raises(TypeError):
        nblist_mod.find_info4mlff(w["cell"], w["types"], w["coords"].astype(np.float32), 5.0, 64, True, [True] * 3, False)
    # device-level status of a truncated build
    nb = capi.NeighborBuilder()
    nn, fn, rc, st = nb.build(w["cell"], torch.from_numpy(w["coords"]).cuda(), 5.0, 8)
    st = st.cpu().numpy()
    assert st[1] == 1 and st[0] == G["g0_numneigh"].max() and nn.max().item() == 8


def test_empty_structure():
    nb = capi.NeighborBuilder()
    nn, fn, rc, st = nb.build(np.eye(3) * 5, torch.zeros(0, 3, dtype=torch.float64, device="cuda"), 3.0, 8)
    assert nn.numel() == 0


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_centre_ranges_bin_reuse_and_host_extent(checkers, dt):
    """ai2b_nblist_build_range_*: rows for a range of centres equal the same rows of the full list; a second range
    built from the bins the first call left in the workspace is identical; a host-given extent along an open
    first axis (even a wrong one: atoms outside it share the edge bins) changes nothing."""
    chk = _chk(checkers)
    rng = np.random.default_rng(8)
    cell, pos = synth.cubic_lattice(8, 2.9, 0.12, rng, dt)
    n = len(pos)
    types = np.zeros(n, np.int32)
    tdt = torch.float64 if dt == np.float64 else torch.float32
    dpos = torch.from_numpy(pos).cuda()
    for pbc in ((True, True, True), (False, True, True)):
        ref = chk.nblist(cell, types, pos, 5.0, 64, pbc=[int(p) for p in pbc])
        b = capi.NeighborBuilder()
        c0, c1, c2 = 37, 300, n
        o1 = capi.NeighborBuilder.new_outputs(c1 - c0, 64, tdt, dpos.device)
        o2 = capi.NeighborBuilder.new_outputs(c2 - c1, 64, tdt, dpos.device)
        b.build(cell, dpos, 5.0, 64, pbc=pbc, ncentres=c1, cbegin=c0, out=o1)
        b.build(cell, dpos, 5.0, 64, pbc=pbc, ncentres=c2, cbegin=c1, reuse_bins=True, out=o2)
        for (nn, fn, rc, st), (lo, hi) in ((o1, (c0, c1)), (o2, (c1, c2))):
            assert int(st[1]) == 0
            util.assert_nblist_equal((nn.cpu().numpy(), fn.cpu().numpy(), rc.cpu().numpy()), (ref[0][lo:hi], ref[1][lo:hi], ref[2][lo:hi]))
        if not pbc[0]:
            frac = pos[:, 0].astype(np.float64) / float(cell[0, 0])
            for ext in ((frac.min(), frac.max()), (0.2, 0.7)):
                o3 = capi.NeighborBuilder.new_outputs(n, 64, tdt, dpos.device)
                capi.NeighborBuilder().build(cell, dpos, 5.0, 64, pbc=pbc, out=o3, open_extent=ext)
                util.assert_nblist_equal((o3[0].cpu().numpy(), o3[1].cpu().numpy(), o3[2].cpu().numpy()), ref[:3])


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_batched_build_ragged_triclinic_fractional(checkers, dt):
    """ai2b_nblist_build_batch_*: a ragged batch (one empty structure, one cell thinner than the cutoff, triclinic cells,
    fractional input, an open axis) against the CPU code structure by structure; truncation to umax is flagged."""
    chk = _chk(checkers)
    rng = np.random.default_rng(21)
    tdt = torch.float64 if dt == np.float64 else torch.float32
    cells, fracs, ns = [], [], [40, 0, 9, 75, 130]
    for k, n in enumerate(ns):
        L = (3.4 if k == 2 else 9.0) + k
        cell = (np.eye(3) * L + rng.normal(0, 0.4, (3, 3))).astype(dt)
        cells.append(cell)
        fracs.append((rng.random((n, 3)) * 1.6 - 0.3).astype(dt))          # some atoms outside the cell
    npad = max(ns)
    B = len(ns)
    coords = np.zeros((B, npad, 3), dt)
    for b in range(B):
        coords[b, :ns[b]] = fracs[b]
    for pbc in ((True, True, True), (True, False, True)):
        out = capi.nblist_build_batch(np.stack(cells), torch.tensor(ns, dtype=torch.int32).cuda(), torch.from_numpy(coords).cuda(), 4.5, 200,
                                      is_cart=False, pbc=pbc)
        st = out["status"].cpu().numpy()
        assert st[1] == 0
        mxs = [0]
        for b in range(B):
            n = ns[b]
            if n == 0:
                assert int(out["bnumneigh"][b].abs().sum()) == 0
                continue
            nn, fn, rc, ty, mx = chk.nblist(cells[b], np.zeros(n, np.int32), fracs[b], 4.5, 200, is_cart=False, pbc=[int(p) for p in pbc])
            mxs.append(mx)
            util.assert_nblist_equal((out["bnumneigh"][b, :n].cpu().numpy(), out["bfirstneigh"][b, :n].cpu().numpy(),
                                      out["brcs"][b, :n].cpu().numpy()), (nn, fn, rc))
            assert bool((out["bfirstneigh"][b, n:] == -1).all()) and float(out["brcs"][b, n:].abs().sum()) == 0.0
        assert st[0] == max(mxs)
    small = capi.nblist_build_batch(np.stack(cells), torch.tensor(ns, dtype=torch.int32).cuda(), torch.from_numpy(coords).cuda(), 4.5, 8,
                                    is_cart=False)
    st = small["status"].cpu().numpy()
    assert st[1] & 1 and st[0] > 8 and int(small["bnumneigh"].max()) == 8


@pytest.mark.parametrize("dt", [np.float64, np.float32])
def test_lanes_as_centres_kernel_on_small_cases(checkers, dt, monkeypatch):
    """Large systems (220,000 atoms and more) take the kernel whose lanes are centre atoms (the full-size configs[4]
    test runs it). AI2B_NBL_MIN_ATOMS = 0 sends every build with merged columns through it: triclinic cell with
    atoms outside it, open axes, fractional input, a centre range with bin reuse, truncated rows."""
    monkeypatch.setenv("AI2B_NBL_MIN_ATOMS", "0")
    chk = _chk(checkers)
    rng = np.random.default_rng(15)
    cell = np.array([[17.0, 0.3, 0.1], [1.5, 16.5, 0.2], [-0.7, 0.9, 18.0]]).astype(dt)
    frac = rng.random((400, 3))
    pos = (frac @ cell.astype(np.float64) + rng.normal(0, 6.0, (400, 3))).astype(dt)
    types = rng.integers(0, 2, 400).astype(np.int32)
    for pbc in ((1, 1, 1), (1, 0, 1), (0, 0, 0), (0, 1, 0), (1, 1, 0)):
        a = _gpu(cell, types, pos, 5.5, 160, pbc=pbc)
        b = chk.nblist(cell, types, pos, 5.5, 160, pbc=pbc)
        util.assert_nblist_equal(a, b[:3])
    a = _gpu(cell, types, frac.astype(dt), 5.5, 160, is_cart=False)
    b = chk.nblist(cell, types, frac.astype(dt), 5.5, 160, is_cart=False)
    util.assert_nblist_equal(a, b[:3])
    # the benchmark structure, a centre range and bin reuse
    w = synth.g1(util.tables(16))
    p1 = w["coords"].astype(dt); c1 = w["cell"].astype(dt)
    ref = chk.nblist(c1, w["types"], p1, 6.0, 64)
    util.assert_nblist_equal(_gpu(c1, w["types"], p1, 6.0, 64), ref[:3])
    tdt = torch.float64 if dt == np.float64 else torch.float32
    dpos = torch.from_numpy(p1).cuda()
    nb = capi.NeighborBuilder()
    lo, mid, hi = 1000, 5000, 9000
    o1 = capi.NeighborBuilder.new_outputs(mid - lo, 64, tdt, dpos.device)
    o2 = capi.NeighborBuilder.new_outputs(hi - mid, 64, tdt, dpos.device)
    nb.build(c1, dpos, 6.0, 64, ncentres=mid, cbegin=lo, out=o1)
    nb.build(c1, dpos, 6.0, 64, ncentres=hi, cbegin=mid, reuse_bins=True, out=o2)
    for (nn, fn, rc, st), (x0, x1) in ((o1, (lo, mid)), (o2, (mid, hi))):
        util.assert_nblist_equal((nn.cpu().numpy(), fn.cpu().numpy(), rc.cpu().numpy()), (ref[0][x0:x1], ref[1][x0:x1], ref[2][x0:x1]))
    # truncated rows are flagged, the counts are the true ones
    nn, fn, rc, st = capi.NeighborBuilder().build(c1, dpos, 6.0, 8)
    st = st.cpu().numpy()
    assert st[1] == 1 and st[0] == ref[0].max() and nn.max().item() == 8
