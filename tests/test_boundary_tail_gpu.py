"""The reference-facing boundary beyond the eager torch ops:
  * the TorchScript route of the LAMMPS pair style (interface/lammps/AI2POT/pair_ai2pot.cpp:408-432: a scripted model's
    `predict_efv(7 tensors)` that calls torch.ops.nep.nepToEFVOp / torch.ops.mtpr.linearMtpToEFVOp), saved and reloaded
    in a fresh process that has loaded nothing but this build's lib*_bind.so files;
  * the top-level `nblist` module the reference's loader imports from its library directory;
  * one host process driving two devices;
  * the MD session's recovery from a failed buffer growth.
"""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi, synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "ai2pot_b200", "_lib")


def _chk(checkers):
    return checkers.get("ref") or checkers["oracle"]


class ScriptedNep(torch.nn.Module):
    """predict_efv with the argument order of ai2pot/models/nep/nep.py:298-355 (unit conversions left at 1)."""

    def __init__(self, m):
        super().__init__()
        self.chebyshev_size, self.n_radial_basis, self.n_angular_basis, self.l_max = int(m["chebyshev_size"]), int(m["n_radial"]), int(m["n_angular"]), int(m["l_max"])
        self.rmax_radial, self.rmax_angular = float(m["rmax_radial"]), float(m["rmax_angular"])
        for k, name in (("coeffs", "coeffs_tensor"), ("w0", "w0_tensor"), ("b0", "b0_tensor"), ("w1", "w1_tensor"), ("type_bias", "type_bias_tensor"),
                        ("q_scaler", "q_scaler_tensor")):
            self.register_buffer(name, torch.from_numpy(np.ascontiguousarray(m[k])))
        nt = int(m["ntypes"])
        self.register_buffer("type_map_tensor", torch.arange(nt, dtype=torch.int32))
        self.register_buffer("zbl_tensor", torch.zeros(nt * nt * 4, dtype=self.coeffs_tensor.dtype))

    @torch.jit.export
    def predict_efv(self, binum_tensor: torch.Tensor, bilist_tensor: torch.Tensor, bnumneigh_tensor: torch.Tensor,
                    bfirstneigh_tensor: torch.Tensor, brcs_tensor: torch.Tensor, btypes_tensor: torch.Tensor,
                    bnghost_tensor: torch.Tensor):
        out = torch.ops.nep.nepToEFVOp(self.chebyshev_size, self.n_radial_basis, self.n_angular_basis, self.l_max, self.coeffs_tensor,
                                       self.w0_tensor, self.b0_tensor, self.w1_tensor, self.type_bias_tensor, binum_tensor, bilist_tensor,
                                       bnumneigh_tensor, bfirstneigh_tensor, brcs_tensor, btypes_tensor, self.type_map_tensor,
                                       int(bnghost_tensor[0].item()), self.rmax_radial, self.rmax_angular, self.q_scaler_tensor, 0.0, 0.0,
                                       self.zbl_tensor, self.zbl_tensor)
        return out[0], out[1], out[2]

    def forward(self, x: torch.Tensor):
        return x


class ScriptedMtp(torch.nn.Module):
    """predict_efv over torch.ops.mtpr.linearMtpToEFVOp (25 arguments, source/descriptor/mtpr/bind/mtpr_bind.cc:334-393)."""

    def __init__(self, m):
        super().__init__()
        tb = m["tables"]
        self.chebyshev_size, self.scaling, self.nmus, self.alpha_moments_count = int(m["chebyshev_size"]), float(m["scaling"]), int(tb["nmus"]), int(tb["alpha_moments_count"])
        self.rmax, self.rmin = float(m["rmax"]), float(m["rmin"])
        for k, name in (("coeffs", "coeffs_tensor"), ("linear_coeffs", "linear_coeffs_tensor"), ("type_bias", "type_bias_tensor"),
                        ("q_scaler", "q_scaler_tensor")):
            self.register_buffer(name, torch.from_numpy(np.ascontiguousarray(m[k])))
        for k in ("alpha_index_basic", "alpha_index_times", "alpha_moment_mapping"):
            self.register_buffer(k + "_tensor", torch.from_numpy(np.ascontiguousarray(tb[k], np.int32)))
        nt = int(m["ntypes"])
        self.register_buffer("type_map_tensor", torch.arange(nt, dtype=torch.int32))
        self.register_buffer("zbl_tensor", torch.zeros(nt * nt * 4, dtype=self.coeffs_tensor.dtype))

    @torch.jit.export
    def predict_efv(self, binum_tensor: torch.Tensor, bilist_tensor: torch.Tensor, bnumneigh_tensor: torch.Tensor,
                    bfirstneigh_tensor: torch.Tensor, brcs_tensor: torch.Tensor, btypes_tensor: torch.Tensor,
                    bnghost_tensor: torch.Tensor):
        out = torch.ops.mtpr.linearMtpToEFVOp(self.chebyshev_size, self.scaling, self.coeffs_tensor, self.linear_coeffs_tensor,
                                              self.type_bias_tensor, self.alpha_moments_count, self.alpha_index_basic_tensor,
                                              self.alpha_index_times_tensor, self.alpha_moment_mapping_tensor, self.nmus, binum_tensor,
                                              bilist_tensor, bnumneigh_tensor, bfirstneigh_tensor, brcs_tensor, btypes_tensor,
                                              self.type_map_tensor, int(bnghost_tensor[0].item()), self.rmax, self.rmin,
                                              self.q_scaler_tensor, 0.0, 0.0, self.zbl_tensor, self.zbl_tensor)
        return out[0], out[1], out[2]

    def forward(self, x: torch.Tensor):
        return x


# what the LAMMPS process does: load the op libraries it links (-lmtpr_bind -lnep_bind), torch::jit::load, get_method
_CHILD = textwrap.dedent("""
    import sys, numpy as np, torch
    libdir, model_path, inp, out = sys.argv[1:5]
    for name in ("libmtpr_bind.so", "libnep_bind.so"):
        torch.ops.load_library(libdir + "/" + name)
    assert "ai2pot_b200" not in sys.modules
    model = torch.jit.load(model_path, map_location="cuda:0")
    z = np.load(inp)
    args = [torch.from_numpy(z[k]).cuda() for k in ("binum", "bilist", "bnumneigh", "bfirstneigh", "brcs", "btypes", "bnghost")]
    with torch.no_grad():
        e, f, v = model.get_method("predict_efv")(*args) if hasattr(model, "get_method") else model.predict_efv(*args)
    np.savez(out, e=e.cpu().numpy(), f=f.cpu().numpy(), v=v.cpu().numpy())
""")


@pytest.mark.parametrize("kind", ["nep", "mtp"])
def test_torchscript_predict_efv_in_fresh_process(checkers, tmp_path, kind):
    from ai2pot_b200 import fromcc  # noqa: F401  (registers the ops so that the module can be scripted)
    chk = _chk(checkers)
    if kind == "nep":
        w = util.small_nep_case(5, np.float32)
        module, tol = ScriptedNep(w["model"]), 1e-5
    else:
        w = util.small_mtp_case(10, 5, np.float64)
        module, tol = ScriptedMtp(w["model"]), 1e-10
    nb = util.nblist_batch(chk, w)
    scripted = torch.jit.script(module)
    path = str(tmp_path / "model.pt")
    torch.jit.save(scripted, path)
    inp, out = str(tmp_path / "in.npz"), str(tmp_path / "out.npz")
    np.savez(inp, bnghost=np.zeros(1, np.int32), **{k: nb[k] for k in ("binum", "bilist", "bnumneigh", "bfirstneigh", "brcs", "btypes")})
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    r = subprocess.run([sys.executable, "-c", _CHILD, LIBDIR, path, inp, out], cwd=str(tmp_path), env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    z = np.load(out)
    er, fr, vr = chk.nep_efv(w["model"], nb) if kind == "nep" else chk.mtp_efv(w["model"], nb)
    assert util.relerr(z["e"], er) < tol and util.relerr(z["f"], fr) < tol and util.relerr(z["v"], vr) < tol


def test_toplevel_nblist_module(checkers):
    """`sys.path.append(lib_dir); import nblist` (ai2pot/fromcc/__init__.py:52-58) with lib_dir = ai2pot_b200/_lib."""
    code = textwrap.dedent("""
        import sys, numpy as np
        sys.path.append(sys.argv[1])
        import nblist
        z = np.load(sys.argv[2])
        out = nblist.find_info4mlff(z["cell"], z["types"], z["coords"], 5.0, 48, True, [True, True, True], False)
        assert out[0] == len(z["types"]) and out[6] == 0
        np.savez(sys.argv[3], nn=out[2], fn=out[3], rc=out[4])
    """)
    import tempfile
    w = util.small_mtp_case(6, 4, np.float64)
    with tempfile.TemporaryDirectory() as d:
        np.savez(os.path.join(d, "in.npz"), cell=w["cell"], types=w["types"].astype(np.int64), coords=w["coords"])
        env = dict(os.environ)
        env.pop("PYTHONPATH", None)
        r = subprocess.run([sys.executable, "-c", code, LIBDIR, os.path.join(d, "in.npz"), os.path.join(d, "out.npz")], cwd=d, env=env,
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        z = np.load(os.path.join(d, "out.npz"))
        nn, fn, rc, ty, mx = _chk(checkers).nblist(w["cell"], w["types"], w["coords"], 5.0, 48)
        util.assert_nblist_equal((z["nn"], z["fn"], z["rc"]), (nn, fn, rc))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_devices_in_one_process(checkers):
    """Kernels that need more than 48 KB of dynamic shared memory are configured per device: a process that has run
    on cuda:0 must be able to run the same calls on cuda:1 (each on its own device's memory)."""
    chk = _chk(checkers)
    w = util.small_mtp_case(16, 4, np.float64, rcut=6.0)
    nb = util.nblist_batch(chk, w)
    er, fr, vr = chk.mtp_efv(w["model"], nb)
    wn = util.small_nep_case(4, np.float32)
    nbn = util.nblist_batch(chk, wn)
    ern, frn, vrn = chk.nep_efv(wn["model"], nbn)
    for dev in (0, 1):
        with torch.cuda.device(dev):
            d = torch.device("cuda", dev)
            prog = capi.MtpProgram(w["model"]["tables"])
            md = capi.to_device({k: v for k, v in w["model"].items() if k != "tables"}, d)
            e, f, v = capi.mtp_efv(prog, md, capi.to_device(nb, d))
            torch.cuda.synchronize()
            assert util.relerr(e.cpu().numpy(), er) < 1e-10 and util.relerr(f.cpu().numpy(), fr) < 1e-10 and util.relerr(v.cpu().numpy(), vr) < 1e-10
            e, f, v = capi.nep_efv(capi.to_device(wn["model"], d), capi.to_device(nbn, d))
            torch.cuda.synchronize()
            assert util.relerr(f.cpu().numpy(), frn) < 1e-5 and util.relerr(e.cpu().numpy(), ern) < 1e-5


def test_md_session_survives_failed_growth():
    """A growth of the session's buffers that fails must leave the session usable: the next call with sane sizes
    allocates afresh and gives the same answer as before. The failing request asks for neighbour rows of
    7e8 atoms (215 GB of indices alone): the allocation is refused, nothing is read or launched."""
    import ctypes as C
    w = synth.g2(n=6)
    m = w["model"]
    x = np.ascontiguousarray(np.mod(w["coords"].astype(np.float64), 18.0))
    ty = np.ascontiguousarray(w["types"], np.int32)
    big = capi.MdSession(m, 1 << 30)            # a neighbour width no device can hold: the first growth fails
    with pytest.raises(capi.Ai2bError):
        big.compute(len(x), 0, x, ty)
    big.close()
    ses = capi.MdSession(m, 64)
    e1, f1, v1, mx1 = ses.compute(len(x), 0, x, ty)
    f = np.zeros((len(x), 3)); e = C.c_double(0.0); v = np.zeros(6); mx = C.c_int(0)
    rc = capi.lib().ai2b_md_session_compute(ses.h, C.c_int(700_000_000), C.c_int(0), x.ctypes.data_as(C.c_void_p), ty.ctypes.data_as(C.c_void_p),
                                            C.c_int(1), f.ctypes.data_as(C.c_void_p), C.byref(e), v.ctypes.data_as(C.c_void_p), C.byref(mx))
    assert rc != 0 and not f.any()
    e2, f2, v2, mx2 = ses.compute(len(x), 0, x, ty)
    ses.close()
    assert mx1 == mx2 and abs(e1 - e2) <= 1e-6 * abs(e1) and np.abs(f1 - f2).max() <= 1e-5 * np.abs(f1).max()
