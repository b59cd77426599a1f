"""Regenerates the golden outputs in tests/golden/golden_small.npz and the MoS2 fixture.

Everything here is produced by the REFERENCE's own CPU code (oracle/_ref, compiled from the
reference tree by oracle/Makefile) on the seeded inputs defined in tests/util.py, with one
OpenMP thread so the sums are reproducible. The 12-atom MoS2 cell is read from the text of the
reference's own neighbour-list unit test (source/nblist/tests/test_neighborList.cc:30-93).
Run where the reference is mounted:  REF_ROOT=<reference tree> OMP_NUM_THREADS=1 python tests/golden/make_golden.py
"""
import os, re, sys
os.environ.setdefault("OMP_NUM_THREADS", "1")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))
import numpy as np
from oracle.refapi import Checker
from ai2pot_b200 import synth
import util

root = sys.argv[1] if len(sys.argv) > 1 else os.environ["REF_ROOT"]
ref = Checker("ref")
out = {}

# -- MoS2 fixture of the reference's nblist test ------------------------------------------
txt = open(f"{root}/source/nblist/tests/test_neighborList.cc").read()
def grab(name, shape):
    a = np.zeros(shape)
    for m in re.finditer(name + r"\[(\d+)\]\[(\d+)\]\s*=\s*(-?[\d.]+);", txt):
        a[int(m.group(1)), int(m.group(2))] = float(m.group(3))
    return a
cell = grab("basis_vectors", (3, 3)); frac = grab("frac_coords", (12, 3))
z = np.zeros(12, np.int32)
for m in re.finditer(r"atomic_numbers\[(\d+)\]\s*=\s*(\d+);", txt):
    z[int(m.group(1))] = int(m.group(2))
np.savez(os.path.join(HERE, "mos2_fixture.npz"), cell=cell, frac=frac, z=z)
nn, fn, rc, ty, mx = ref.nblist(cell.astype(np.float32), z, frac.astype(np.float32), 3.2, 16, is_cart=False, pbc=(1, 1, 0))
out["mos2_numneigh"] = nn; out["mos2_first"] = fn; out["mos2_rcs"] = rc; out["mos2_max"] = np.int32(mx)

# -- G0: MTP level 10, 216 atoms (the reference's CPU-runnable configuration) --------------
w = synth.g0(util.tables(10))
nn, fn, rc, ty, mx = ref.nblist(w["cell"], w["types"], w["coords"], w["rcut"], w["umax"])
out["g0_numneigh"] = nn
fs, rs = util.canonical_nblist(nn, fn, rc)
out["g0_first_sorted"] = fs; out["g0_rcs_sorted"] = rs
nb = synth.batch_from_nblist(nn, fn, rc, ty, 3)
e, f, v = ref.mtp_efv(w["model"], nb)
out["g0_e"] = e; out["g0_f"] = f; out["g0_v"] = v
out["g0_desc_head"] = ref.mtp_descriptors(w["model"], nb)[0, :8]

# -- small MTP cases (level 6/10/16, fp64 and fp32) ----------------------------------------
for level, dt in ((6, np.float64), (16, np.float64), (10, np.float32)):
    w = util.small_mtp_case(level, 5, dt)
    nb = util.nblist_batch(ref, w)
    e, f, v = ref.mtp_efv(w["model"], nb)
    tag = f"mtp{level}_{np.dtype(dt).name}"
    out[tag + "_e"] = e; out[tag + "_f"] = f; out[tag + "_v"] = v

# -- small NEP cases ------------------------------------------------------------------------
for dt in (np.float32, np.float64):
    w = util.small_nep_case(5, dt)
    nb = util.nblist_batch(ref, w)
    e, f, v = ref.nep_efv(w["model"], nb)
    tag = f"nep_{np.dtype(dt).name}"
    out[tag + "_e"] = e; out[tag + "_f"] = f; out[tag + "_v"] = v
    out[tag + "_desc_head"] = ref.nep_descriptors(w["model"], nb)[0, :8]

# -- MTP loss + coefficient gradient on a small training batch -----------------------------
g, nb = util.training_batch(ref)
e, f, v = ref.mtp_efv(g["model"], nb)
t = g["targets"]
Fd = t["F"][:, :nb["bilist"].shape[1]]
out["train_loss"] = ref.mtp_loss(nb, g["weights"], e, t["E"], f, Fd, v, t["V"])
dco, dli, dbi = ref.mtp_loss_backward(g["model"], nb, g["weights"], e, t["E"], f, Fd, v, t["V"])
out["train_dcoeffs"] = dco; out["train_dlinear"] = dli; out["train_dbias"] = dbi

np.savez_compressed(os.path.join(HERE, "golden_small.npz"), **out)
print("wrote", len(out), "arrays,", os.path.getsize(os.path.join(HERE, "golden_small.npz")), "bytes")
