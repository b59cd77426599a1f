"""Shared helpers for the parity tests (test infrastructure)."""
import os
import numpy as np

from ai2pot_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def tables(level):
    z = np.load(os.path.join(GOLDEN, f"mtp_tables_L{level:02d}.npz"))
    return dict(alpha_moments_count=int(z["alpha_moments_count"]), nmus=int(z["nmus"]),
                alpha_index_basic=z["alpha_index_basic"], alpha_index_times=z["alpha_index_times"],
                alpha_moment_mapping=z["alpha_moment_mapping"])


def canonical_nblist(numneigh, firstneigh, rcs):
    """Order-independent form: per atom, rows sorted by (neighbour index, rcs bits)."""
    n, umax = firstneigh.shape
    itype = np.uint64 if rcs.dtype == np.float64 else np.uint32
    bits = np.ascontiguousarray(rcs).view(itype).astype(np.uint64)
    idx = firstneigh.astype(np.int64).copy()
    pad = np.arange(umax)[None, :] >= numneigh[:, None]
    idx[pad] = np.iinfo(np.int64).max
    order = np.lexsort((bits[..., 2], bits[..., 1], bits[..., 0], idx), axis=1)
    f = np.take_along_axis(firstneigh, order, 1)
    r = np.take_along_axis(rcs, order[..., None], 1)
    return f, r


def assert_nblist_equal(a, b):
    """a, b = (numneigh, firstneigh, rcs); bit-exact after canonical sort."""
    assert np.array_equal(a[0], b[0]), "numneigh differs"
    fa, ra = canonical_nblist(*a)
    fb, rb = canonical_nblist(*b)
    assert np.array_equal(fa, fb), "neighbour indices differ"
    it = np.uint64 if ra.dtype == np.float64 else np.uint32
    assert np.array_equal(ra.view(it), rb.view(it)), "rcs bits differ"


def relerr(a, ref):
    """max|a - ref| / max|ref| over the tensor (components near zero get the tensor's scale)."""
    a = np.asarray(a, np.float64); ref = np.asarray(ref, np.float64)
    s = np.abs(ref).max()
    return float(np.abs(a - ref).max() / (s if s > 0 else 1.0))


def small_mtp_case(level=10, n=5, dtype=np.float64, seed=7, rcut=5.0, ntypes=3, a=3.0):
    rng = np.random.default_rng(seed)
    cell, pos = synth.cubic_lattice(n, a, 0.1, rng, dtype)
    types = rng.integers(0, ntypes, len(pos)).astype(np.int32)
    model = synth.mtp_model(tables(level), ntypes, rng, dtype, rcut, 0.5)
    model["type_bias"] = rng.normal(0, 0.1, ntypes).astype(dtype)
    model["q_scaler"] = rng.uniform(0.5, 1.5, len(model["q_scaler"])).astype(dtype)
    model["scaling"] = 0.9
    return dict(cell=cell, coords=pos, types=types, rcut=rcut, umax=48, model=model)


def small_nep_case(n=5, dtype=np.float32, seed=11, ntypes=3, a=3.0):
    rng = np.random.default_rng(seed)
    cell, pos = synth.cubic_lattice(n, a, 0.1, rng, dtype)
    types = rng.integers(0, ntypes, len(pos)).astype(np.int32)
    model = synth.nep_model(ntypes, rng, dtype)
    model["type_bias"] = rng.normal(0, 0.1, ntypes).astype(dtype)
    model["q_scaler"] = rng.uniform(0.5, 1.5, len(model["q_scaler"])).astype(dtype)
    return dict(cell=cell, coords=pos, types=types, rcut=6.0, umax=96, model=model)


def nblist_batch(chk, w):
    nn, fn, rc, ty, mx = chk.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
    return synth.batch_from_nblist(nn, fn, rc, ty, w["model"]["ntypes"])


def training_batch(chk, level=10, B=3, seed=21, nmin=20, nmax=40):
    """A small padded batch with random targets, shaped like the training configuration."""
    g = synth.g3(tables(level), seed=seed, batch=B, nmin=nmin, nmax=nmax)
    lists = []
    for s in g["structs"]:
        nn, fn, rc, ty, mx = chk.nblist(s["cell"], s["types"], s["coords"], 5.0, g["umax"] * 2)
        lists.append((nn, fn, rc, ty))
    g["model"]["rmax"] = 5.0
    nb = synth.pad_batch(lists, 3, g["umax"] * 2)
    return g, nb
