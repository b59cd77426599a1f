"""Parity of the CUDA NEP path (through the C ABI) with the CPU checkers.
Tolerance: fp32 rel 1e-5, fp64 rel 1e-10 of the tensor's max magnitude."""
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


def _run(model, nb, virial=True):
    dt = torch.float64 if nb["brcs"].dtype == np.float64 else torch.float32
    md = capi.to_device(model, float_dtype=dt)
    nbd = capi.to_device(nb)
    out = capi.nep_efv(md, nbd, virial=virial)
    torch.cuda.synchronize()
    return [o.cpu().numpy() for o in out], md, nbd


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_small_golden(checkers, dt):
    w = util.small_nep_case(5, dt)
    nb = util.nblist_batch(_chk(checkers), w)
    (e, f, v), md, nbd = _run(w["model"], nb)
    tag = f"nep_{np.dtype(dt).name}"
    for a, k in ((e, "_e"), (f, "_f"), (v, "_v")):
        assert util.relerr(a, G[tag + k]) < TOL[dt], k
    e2, f2 = capi.nep_efv(md, nbd, virial=False)
    assert util.relerr(f2.cpu().numpy(), G[tag + "_f"]) < TOL[dt]
    d = capi.nep_descriptors(md, nbd).cpu().numpy()
    assert util.relerr(d[0, :8], G[tag + "_desc_head"]) < TOL[dt]
    assert util.relerr(d, _chk(checkers).nep_descriptors(w["model"], nb)) < TOL[dt]


def _g2(dt):
    w = synth.g2()
    w["coords"] = w["coords"].astype(dt); w["cell"] = w["cell"].astype(dt)
    model = {k: (v.astype(dt) if isinstance(v, np.ndarray) else v) for k, v in w["model"].items()}
    return w, model


def test_g2_full_size_fp64(checkers):
    """The benchmark structure (13,824 atoms, rc 6/4) in fp64 against the CPU checker."""
    chk = _chk(checkers)
    w, model = _g2(np.float64)
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    nb = synth.batch_from_nblist(nn, fn, rc, ty, 3)
    (e, f, v), *_ = _run(model, nb)
    er, fr, vr = chk.nep_efv(model, nb)
    assert util.relerr(e, er) < 1e-10 and util.relerr(f, fr) < 1e-10 and util.relerr(v, vr) < 1e-10


def test_g2_full_size_fp32(checkers):
    """The benchmark configuration itself (fp32). Sums over 4e5 pairs in fp32 carry the CPU
    code's own rounding (its energy moves by 4e-7 between two OpenMP runs, its virial by more), so
    the check is the two-sided one of util.fp32_parity (tol 1e-5), with the three distances recorded."""
    chk = _chk(checkers)
    w, model = _g2(np.float32)
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    nb = synth.batch_from_nblist(nn, fn, rc, ty, 3)
    (e, f, v), *_ = _run(model, nb)
    r32 = chk.nep_efv(model, nb)
    r64 = chk.nep_efv(util.to64(model), dict(nb, brcs=nb["brcs"].astype(np.float64)))
    for a, a32, a64, name in zip((e, f, v), r32, r64, ("energy", "force", "virial")):
        util.fp32_parity("configs[2] NEP fp32, 13,824 atoms", name, a, a32, a64)


def _g4_case(chk, ncell):
    """configs[4] lattice with ncell^3 cells: CUDA neighbour list (bit-exact against the CPU code) and NEP E/F/V."""
    from ai2pot_b200 import engine
    w = synth.g4(ncell=ncell)
    n = len(w["types"])
    ev = engine.Evaluator(w["model"], w["cell"], w["types"], w["rcut"], w["umax"], torch.float32)
    coords = torch.from_numpy(np.ascontiguousarray(w["coords"])).cuda()
    nbd = ev.build_list(coords)
    st = ev.status.cpu().numpy()
    assert st[1] == 0
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    assert mx == st[0]
    util.assert_nblist_equal((nbd["bnumneigh"][0].cpu().numpy(), nbd["bfirstneigh"][0].cpu().numpy(), nbd["brcs"][0].cpu().numpy()),
                             (nn, fn, rc))
    e, f, v = [t.cpu().numpy() for t in ev.evaluate(nbd)]
    nb = synth.batch_from_nblist(nn, fn, rc, ty, 3)
    r32 = chk.nep_efv(w["model"], nb)
    r64 = chk.nep_efv(util.to64(w["model"]), dict(nb, brcs=rc[None].astype(np.float64)))
    for a, a32, a64, name in zip((e, f, v), r32, r64, ("energy", "force", "virial")):
        util.fp32_parity(f"configs[4] NEP fp32, {n:,} atoms", name, a, a32, a64)


def test_g4_one_rank_share(checkers):
    """A 32^3-cell system of the configs[4] lattice (131,072 atoms: what one of eight ranks owns): neighbour list
    bit-exact and E/F/V against the CPU code."""
    _g4_case(_chk(checkers), 32)


def test_g4_full_size_vs_checker(checkers):
    """configs[4] itself, 1,048,576 atoms, against the CPU code (neighbour list bit-exact, E/F/V two-sided fp32
    statement). Needs ~8 GB of host memory and about a minute of host time; skipped on smaller hosts."""
    import psutil
    if psutil.virtual_memory().available < 24e9:
        pytest.skip("needs 24 GB of free host memory for the CPU code's neighbour list")
    _g4_case(_chk(checkers), 64)


@pytest.mark.parametrize("cfg", [dict(n_radial=6, n_angular=3, l_max=2, chebyshev_size=5, num_neurons=17),
                                 dict(n_radial=3, n_angular=5, l_max=3, chebyshev_size=12, num_neurons=40),
                                 dict(n_radial=5, n_angular=2, l_max=0, chebyshev_size=8, num_neurons=9),
                                 dict(n_radial=2, n_angular=2, l_max=1, chebyshev_size=3, num_neurons=4)])
def test_other_shapes_fp64(checkers, cfg):
    chk = _chk(checkers)
    rng = np.random.default_rng(17)
    cell, pos = synth.cubic_lattice(4, 2.6, 0.12, rng)
    types = rng.integers(0, 2, len(pos)).astype(np.int32)
    model = synth.nep_model(2, rng, np.float64, rmax_radial=5.0, rmax_angular=3.5, **cfg)
    model["q_scaler"] = rng.uniform(0.5, 2.0, len(model["q_scaler"]))
    model["type_bias"] = rng.normal(0, 0.1, 2)
    nn, fn, rc, ty, mx = chk.nblist(cell, types, pos, 5.0, 96)
    nb = synth.batch_from_nblist(nn, fn, rc, ty, 2)
    (e, f, v), md, nbd = _run(model, nb)
    er, fr, vr = chk.nep_efv(model, nb)
    assert util.relerr(e, er) < 1e-10 and util.relerr(f, fr) < 1e-10 and util.relerr(v, vr) < 1e-10
    assert util.relerr(capi.nep_descriptors(md, nbd).cpu().numpy(), chk.nep_descriptors(model, nb)) < 1e-10


def test_ragged_batch(checkers):
    chk = _chk(checkers)
    rng = np.random.default_rng(4)
    lists = []
    for n, a in ((3, 2.8), (4, 2.4), (2, 3.0)):
        cell, pos = synth.cubic_lattice(n, a, 0.1, rng, np.float32)
        ty = rng.integers(0, 3, len(pos)).astype(np.int32)
        nn, fn, rc, _, mx = chk.nblist(cell, ty, pos, 6.0, 160)
        lists.append((nn, fn, rc, ty))
    nb = synth.pad_batch(lists, 3, 160)
    model = synth.nep_model(3, rng)
    (e, f, v), md, nbd = _run(model, nb)
    er, fr, vr = chk.nep_efv(model, nb)
    assert util.relerr(e, er) < 1e-5 and util.relerr(f, fr) < 1e-5 and util.relerr(v, vr) < 1e-5
    # outputs are overwritten, whatever they held (one zeroing launch ahead of the kernel, no memsets)
    e0, f0, v0 = capi.nep_efv(md, nbd)
    dirty = tuple(torch.full_like(x, float("nan")) for x in (e0, f0, v0))
    e3, f3, v3 = capi.nep_efv(md, nbd, out=dirty)
    assert util.relerr(e3.cpu().numpy(), er) < 1e-5 and util.relerr(f3.cpu().numpy(), fr) < 1e-5 and util.relerr(v3.cpu().numpy(), vr) < 1e-5


def test_g4_full_size_properties():
    """configs[4] at full size (1,048,576 atoms, fp32, umax 32) through size-independent properties: the full
    list holds every pair from both ends (index and displacement sums cancel), no row overflows, net force
    zero, symmetric virial, and the energy does not move under a rigid translation across the periodic faces."""
    from ai2pot_b200 import engine
    w = synth.g4()
    n = len(w["types"])
    dt = torch.float32
    ev = engine.Evaluator(w["model"], w["cell"], w["types"], w["rcut"], w["umax"], dt)
    coords = torch.from_numpy(np.ascontiguousarray(w["coords"])).to(dt).cuda()
    nb = ev.build_list(coords)
    st = ev.status.cpu().numpy()
    assert st[1] == 0 and 16 <= st[0] <= 32
    nn, fn, rc = nb["bnumneigh"][0], nb["bfirstneigh"][0], nb["brcs"][0]
    mask = torch.arange(w["umax"], device="cuda")[None] < nn[:, None]
    assert bool((fn[~mask] == -1).all())
    # every pair is listed from both ends, except pairs whose fp32 distance sits on the cutoff (the reference's
    # single-precision image arithmetic rounds r_j + L - r_i and r_i - L - r_j differently)
    centre = torch.arange(n, device="cuda", dtype=torch.int64)[:, None].expand(-1, w["umax"])
    i_, j_ = centre[mask], fn.to(torch.int64)[mask]
    dist = torch.linalg.norm(rc[mask].double(), dim=-1)
    key = torch.minimum(i_, j_) * n + torch.maximum(i_, j_)
    key, order = torch.sort(key)
    same_next = torch.zeros_like(key, dtype=torch.bool); same_next[:-1] = key[:-1] == key[1:]
    same_prev = torch.zeros_like(key, dtype=torch.bool); same_prev[1:] = same_next[:-1]
    single = ~(same_next | same_prev)
    assert int(single.sum()) < 1e-5 * len(key)
    assert bool((torch.abs(dist[order][single] - w["rcut"]) < 1e-4).all())
    pair_sum = (rc.double() * mask[..., None]).sum((0, 1))
    assert float(pair_sum.abs().max()) < 1e-6 * float(nn.sum())                        # r_ij + r_ji = 0 up to fp32 image rounding
    e, f, v = [t.clone() for t in ev.evaluate(nb)]
    fs = float(f.abs().max())
    assert float(f[0].double().sum(0).abs().max()) < 1e-5 * fs * np.sqrt(n)
    V = v.double().reshape(3, 3)
    assert float((V - V.T).abs().max()) < 1e-5 * float(V.abs().max())
    shift = torch.tensor([1.7, -2.3, 190.0], dtype=dt, device="cuda")                 # wraps about half the atoms in z
    e2, f2, v2 = ev.compute(coords + shift)
    assert abs(float(e2) - float(e)) < 2e-5 * abs(float(e))
    assert float((f2 - f).abs().max()) < 1e-3 * fs                                     # fp32 positions at |x| ~ 400 A move rcs by ~3e-5 A
