"""Shared helpers for the parity tests (test infrastructure)."""
import os
import numpy as np

from ai2pot_b200 import synth, tables as _tables

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# where the reference tree is mounted (absent on the GPU box): tests that read it are skipped without it
REF_ROOT = os.environ.get("REF_ROOT", os.path.join(os.sep, "root", "reference"))


def tables(level):
    return _tables.load(level)


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


_FP32_RECORD = os.path.join(os.path.dirname(GOLDEN), os.pardir, "gpurun_out", "parity_fp32_distances.jsonl")


def fp32_parity(case, name, got, r32, r64, tol=1e-5):
    """Single-precision parity as a measured, two-sided statement. Three distances (relerr):
        d_cuda64 = CUDA fp32 result   <-> the same model evaluated in fp64 by the CPU checker
        d_cpu64  = fp32 CPU checker   <-> that fp64 value (the CPU code's own fp32 rounding)
        d_cuda32 = CUDA fp32 result   <-> fp32 CPU checker
    Required: the CUDA result is within `tol` of the fp64 value, or at least as close to it as the CPU code's own
    fp32 result is; and it is within tol + d_cpu64 of the fp32 CPU result. The distances are printed and appended
    to the record file (_FP32_RECORD, one JSON object per line)."""
    import json
    d_cuda64, d_cpu64, d_cuda32 = relerr(got, r64), relerr(r32, r64), relerr(got, r32)
    rec = dict(case=case, tensor=name, cuda_vs_fp64=d_cuda64, cpu32_vs_fp64=d_cpu64, cuda_vs_cpu32=d_cuda32)
    print("fp32 parity", json.dumps(rec))
    try:
        os.makedirs(os.path.dirname(_FP32_RECORD), exist_ok=True)
        with open(_FP32_RECORD, "a") as fh:
            fh.write(json.dumps(rec) + "\n")
    except OSError:
        pass
    assert d_cuda64 < tol or d_cuda64 <= d_cpu64, rec
    assert d_cuda32 < tol + d_cpu64, rec


def to64(model):
    return {k: (v.astype(np.float64) if isinstance(v, np.ndarray) and v.dtype == np.float32 else v) for k, v in model.items()}


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
