"""The C-ABI library and the torch-op libraries load without a GPU and export what the header
declares; the .almtp parser and mtpParamOp agree with the reference's parser. No compute calls."""
import ctypes as C
import glob
import os
import re

import numpy as np
import pytest
import torch

import util
from ai2pot_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TEMPLATES = os.path.join(util.REF_ROOT, "source", "descriptor", "mtpr", "MTP_templates")


def _declared():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        txt = open(h).read()
        txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
        # plain declarations
        names |= set(re.findall(r"\b(ai2b_[a-z0-9_]+)\s*\(", txt))
        # macro-generated pairs: name##SUF with SUF in (f64, f32)
        for base in re.findall(r"\b(ai2b_[a-z0-9_]+_)##SUF", txt):
            names |= {base + "f64", base + "f32"}
    return {n for n in names if not n.endswith("_")}


def test_library_exports_every_declared_symbol():
    lib = capi.lib()
    decl = _declared()
    assert len(decl) >= 25
    missing = [n for n in sorted(decl) if not hasattr(lib, n)]
    assert not missing, missing
    assert lib.ai2b_version() >= 100


def test_error_reporting_without_gpu():
    lib = capi.lib()
    counts = np.zeros(5, np.int32)
    rc = lib.ai2b_mtp_parse_almtp(b"/nonexistent/16.almtp", counts.ctypes.data_as(C.c_void_p), None, None, None)
    assert rc == -1 and b"cannot open" in lib.ai2b_last_error_string()
    assert lib.ai2b_nblist_workspace_bytes(C.c_int(1000), C.c_int(1)) > 1000 * 3 * 8
    assert lib.ai2b_nep_workspace_bytes(C.c_int(4), C.c_int(3), C.c_int(4), C.c_int(4), C.c_int(8), C.c_int(0)) >= 9 * 8 * 8 * 4


def test_argument_checks_return_codes_without_gpu():
    """NULL pointers and bad sizes are refused before any CUDA call, with a message."""
    lib = capi.lib()
    null = C.c_void_p(None)
    one = C.c_int(1)
    rc = lib.ai2b_zbl_efv_f32(null, null, null, one, one, null, null, null, null, null, null, one, null, one, C.c_int(0),
                              C.c_float(2.0), C.c_float(1.0), null, null, null)
    assert rc == -1 and b"NULL" in lib.ai2b_last_error_string()
    rc = lib.ai2b_md_session_compute(null, one, one, null, null, one, null, null, null, null)
    assert rc == -1
    rc = lib.ai2b_desc_maxmin_f64(null, null, one, one, one, null, null, null)
    assert rc == -1
    rc = lib.ai2b_target_stats_f32(null, null, one, one, null, null, null, null)
    assert rc == -1
    rc = lib.ai2b_weighted_sum_rows_f32(C.c_int(9), null, null, one, null, null, null)
    assert rc == -1 and b"parts" in lib.ai2b_last_error_string()
    rc = lib.ai2b_nep_loss_backward_f64(null, null, null, null, null, C.c_double(1), C.c_double(1), C.c_double(1), null, null, null,
                                        null, null, null, one, one, one, one, one, null, null, null, null, one, one, null, null, null,
                                        null, null, null, one, one, C.c_int(0), C.c_double(6), C.c_double(4), null, null)
    assert rc == -1 and b"NULL" in lib.ai2b_last_error_string()
    ses = C.c_void_p()
    rc = lib.ai2b_md_session_create_nep(C.byref(ses), one, one, one, one, one, one, null, null, null, null, null, null, C.c_float(6),
                                        C.c_float(4), one)
    assert rc == -1 and not ses.value


@pytest.mark.skipif(not os.path.isdir(REF_TEMPLATES), reason="reference templates not mounted")
@pytest.mark.parametrize("level", [6, 8, 10, 12, 14, 16, 18, 20, 24, 28])
def test_almtp_parser_matches_reference(checkers, level):
    path = f"{REF_TEMPLATES}/{level:02d}.almtp"
    mine = capi.parse_almtp(path)
    if "ref" in checkers:
        ref = checkers["ref"].mtp_param_file(path)
        for k in ("alpha_index_basic", "alpha_index_times", "alpha_moment_mapping"):
            assert np.array_equal(mine[k], ref[k]), k
        assert mine["alpha_moments_count"] == ref["alpha_moments_count"] and mine["nmus"] == ref["nmus"]
    if level in (6, 10, 16):
        t = util.tables(level)
        assert np.array_equal(mine["alpha_index_times"], t["alpha_index_times"]) and mine["nmus"] == t["nmus"]
    if level == 18:
        assert mine["nmus"] == 5          # source/descriptor/mtpr/tests/test_mtpParam.cc:137-141


def test_torch_ops_registered(monkeypatch):
    if os.path.isdir(REF_TEMPLATES):
        monkeypatch.setenv("AI2POT_PATH", util.REF_ROOT)
    from ai2pot_b200 import fromcc
    for name in ("mtpParamOp", "linearMtpToEFVOp", "linearMtpToEFOp", "linearMtpToDescriptorsOp", "nepToEFVOp", "nepToEFOp",
                 "nepToDescriptorsOp", "forceSrOp", "virialSrOp"):
        assert getattr(fromcc, name) is not None
    assert callable(fromcc.nblist.find_info4mlff)
    # schema check: argument count of the EFV op equals the reference's 25
    schema = torch.ops.mtpr.linearMtpToEFVOp.default._schema
    assert len(schema.arguments) == 25 and len(torch.ops.nep.nepToEFVOp.default._schema.arguments) == 24
    if os.path.isdir(REF_TEMPLATES):
        out = fromcc.mtpParamOp(16)
        assert int(out[0]) == 350 and out[1].shape == (130, 4) and out[2].shape == (969, 4) and int(out[6]) == 4
        assert out[4].shape == (350,) and out[5].shape[0] == 350
        t = util.tables(16)
        assert np.array_equal(out[2].numpy(), t["alpha_index_times"])
    # host tensors are refused, loudly
    z = torch.zeros(1)
    zi = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        fromcc.nepToEFVOp(8, 4, 4, 4, z, z, z, z, z, zi, zi.view(1, 1), zi.view(1, 1), zi.view(1, 1, 1), torch.zeros(1, 1, 1, 3), zi.view(1, 1),
                          zi, 0, 6.0, 4.0, z, 0.0, 0.0, z, z)


def test_toplevel_nblist_module_resolves():
    """`sys.path.append(lib_dir); import nblist`, as the reference's loader does (ai2pot/fromcc/__init__.py:52-58), finds
    the module the build step installs next to the libraries (no compute call here)."""
    import subprocess
    import sys
    code = ("import sys; sys.path.append(sys.argv[1]); import nblist; "
            "assert callable(nblist.find_info4mlff) and nblist.__file__.startswith(sys.argv[1])")
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    r = subprocess.run([sys.executable, "-c", code, os.path.join(ROOT, "ai2pot_b200", "_lib")], cwd="/", env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-1500:]


def test_predict_efv_modules_script_and_save(tmp_path):
    """The modules of the TorchScript route (what pair_style ai2pot loads) script and serialise against this build's
    op schemas; running them needs a GPU (tests/test_boundary_tail_gpu.py)."""
    from ai2pot_b200 import fromcc  # noqa: F401
    import test_boundary_tail_gpu as tail
    for module in (tail.ScriptedNep(util.small_nep_case(3, np.float32)["model"]), tail.ScriptedMtp(util.small_mtp_case(10, 3, np.float64)["model"])):
        path = str(tmp_path / "m.pt")
        torch.jit.save(torch.jit.script(module), path)
        back = torch.jit.load(path)
        assert hasattr(back, "predict_efv")
