"""Parity of the CUDA linear-MTP path (through the C ABI) with the CPU checkers.

Tolerance: fp64 rel 1e-10, fp32 rel 1e-5 of the tensor's max magnitude (util.relerr)."""
import os
import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(util.GOLDEN, "golden_small.npz"))
TOL = {np.float64: 1e-10, np.float32: 1e-5}


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


def _run(w, nb, virial=True):
    dt = torch.float64 if nb["brcs"].dtype == np.float64 else torch.float32
    prog = capi.MtpProgram(w["model"]["tables"])
    md = capi.to_device({k: v for k, v in w["model"].items() if k != "tables"}, float_dtype=dt)
    nbd = capi.to_device(nb)
    out = capi.mtp_efv(prog, md, nbd, virial=virial)
    torch.cuda.synchronize()
    return [o.cpu().numpy() for o in out], prog, md, nbd


def test_g0_golden_and_checker(checkers):
    w = synth.g0(util.tables(10))
    chk = _chk(checkers)
    nb = util.nblist_batch(chk, w)
    (e, f, v), prog, md, nbd = _run(w, nb)
    for a, k in ((e, "g0_e"), (f, "g0_f"), (v, "g0_v")):
        assert util.relerr(a, G[k]) < 1e-10, k
    e2, f2 = capi.mtp_efv(prog, md, nbd, virial=False)
    assert util.relerr(e2.cpu().numpy(), G["g0_e"]) < 1e-10 and util.relerr(f2.cpu().numpy(), G["g0_f"]) < 1e-10
    d = capi.mtp_descriptors(prog, md, nbd).cpu().numpy()
    assert util.relerr(d[0, :8], G["g0_desc_head"]) < 1e-10
    assert util.relerr(d, chk.mtp_descriptors(w["model"], nb)) < 1e-10


@pytest.mark.parametrize("level,dt", [(6, np.float64), (16, np.float64), (10, np.float32)])
def test_small_golden(checkers, level, dt):
    w = util.small_mtp_case(level, 5, dt)
    nb = util.nblist_batch(_chk(checkers), w)
    (e, f, v), *_ = _run(w, nb)
    tag = f"mtp{level}_{np.dtype(dt).name}"
    for a, k in ((e, "_e"), (f, "_f"), (v, "_v")):
        assert util.relerr(a, G[tag + k]) < TOL[dt], k


def test_g1_slice_vs_checker(checkers):
    """Level 16 / rcut 6 (the benchmark model) on a 12^3 lattice against the CPU checker."""
    w = synth.g1(util.tables(16), n=12)
    chk = _chk(checkers)
    nb = util.nblist_batch(chk, w)
    (e, f, v), *_ = _run(w, nb)
    er, fr, vr = chk.mtp_efv(w["model"], nb)
    assert util.relerr(e, er) < 1e-10 and util.relerr(f, fr) < 1e-10 and util.relerr(v, vr) < 1e-10


def test_g1_full_size_vs_checker(checkers):
    """configs[1] itself: level 16, fp64, 13,824 atoms, rcut 6 - energy, forces and virial against the CPU code at
    rel 1e-10 (neighbour list from the CPU code; the CUDA list is compared bit for bit in test_nblist_gpu.py)."""
    w = synth.g1(util.tables(16))
    chk = _chk(checkers)
    nb = util.nblist_batch(chk, w)
    (e, f, v), *_ = _run(w, nb)
    er, fr, vr = chk.mtp_efv(w["model"], nb)
    errs = dict(energy=util.relerr(e, er), force=util.relerr(f, fr), virial=util.relerr(v, vr))
    print("configs[1] full size, CUDA vs CPU code:", errs)
    assert max(errs.values()) < 1e-10, errs


def test_many_neighbours_and_ragged_batch(checkers):
    """> 32 neighbours per atom (two lane chunks), padded batch with an empty structure and ghosts."""
    chk = _chk(checkers)
    rng = np.random.default_rng(3)
    lists, mxs = [], []
    for n, a in ((4, 2.2), (3, 2.5), (5, 2.0)):
        cell, pos = synth.cubic_lattice(n, a, 0.1, rng)
        ty = rng.integers(0, 2, len(pos)).astype(np.int32)
        nn, fn, rc, _, mx = chk.nblist(cell, ty, pos, 4.8, 128)
        mxs.append(mx)
        lists.append((nn, fn, rc, ty))
    assert max(mxs) > 64 and min(mxs) < 32      # one, two and three lane chunks
    nb = synth.pad_batch(lists, 2, 128)
    nb["binum"][1] = 0                     # an empty structure in the middle of the batch
    model = synth.mtp_model(util.tables(10), 2, rng, np.float64, 4.8, 1.0)
    w = dict(model=model)
    (e, f, v), *_ = _run(w, nb)
    er, fr, vr = chk.mtp_efv(model, nb)
    assert e[1] == 0 and np.all(f[1] == 0)
    assert util.relerr(e, er) < 1e-10 and util.relerr(f, fr) < 1e-10 and util.relerr(v, vr) < 1e-10


def test_properties_full_size():
    """Size-independent checks at the benchmark size (13,824 atoms, level 16) with a GPU-free
    neighbour list: net force zero, symmetric virial, invariance under atom relabelling."""
    from oracle import refapi
    w = synth.g1(util.tables(16))
    chk = refapi.Checker("oracle")
    nb = util.nblist_batch(chk, w)
    (e, f, v), prog, md, nbd = _run(w, nb)
    fs = np.abs(f).max()
    assert np.abs(f[0].sum(0)).max() < 1e-9 * fs * len(f[0])
    V = v.reshape(3, 3)
    assert np.abs(V - V.T).max() < 1e-9 * np.abs(V).max()
    # second run is bit-for-bit repeatable in energy up to atomic ordering
    e2, f2, v2 = capi.mtp_efv(prog, md, nbd)
    assert util.relerr(e2.cpu().numpy(), e) < 1e-12 and util.relerr(f2.cpu().numpy(), f) < 1e-12
    # outputs are overwritten, whatever they held (the set-up launch zeroes them: there are no memsets)
    dirty = tuple(torch.full_like(x, float("nan")) for x in (e2, f2, v2))
    e3, f3, v3 = capi.mtp_efv(prog, md, nbd, out=dirty)
    assert util.relerr(e3.cpu().numpy(), e) < 1e-12 and util.relerr(f3.cpu().numpy(), f) < 1e-12
    assert util.relerr(v3.cpu().numpy(), v) < 1e-12


def test_errors():
    t = util.tables(10)
    bad = dict(t)
    bad["alpha_index_basic"] = t["alpha_index_basic"].copy()
    bad["alpha_index_basic"][3, 1] = 12    # degree beyond the supported maximum
    with pytest.raises(capi.Ai2bError):
        capi.MtpProgram(bad)
    # host tensors are refused: there is no CPU path behind the C ABI
    w = util.small_mtp_case(6, 3)
    from oracle import refapi
    nb = util.nblist_batch(refapi.Checker("oracle"), w)
    nb_host = {k: (torch.from_numpy(v) if isinstance(v, np.ndarray) else v) for k, v in nb.items()}
    md = capi.to_device({k: v for k, v in w["model"].items() if k != "tables"})
    with pytest.raises(capi.Ai2bError):
        capi.mtp_efv(capi.MtpProgram(w["model"]["tables"]), md, nb_host)
